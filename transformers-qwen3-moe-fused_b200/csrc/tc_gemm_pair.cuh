// CTA-pair (tcgen05 cta_group::2) grouped GEMMs.  Included by tc_gemm.cu.
//
// A pair of CTAs (cluster of 2 on neighbouring SMs) computes one 256-row accumulator:
// each CTA stages 128 rows of the A operand and half of the B operand, the leader CTA
// issues M=256 MMAs that read both CTAs' shared memory, and each CTA ends up with its own
// 128 accumulator rows in its own TMEM.  Per SM this halves the B-operand bytes that have
// to be written to and read from shared memory for the same tensor work, which is what
// the single-CTA kernels are limited by.
//
// Forward / dX are computed "swapped": the accumulator rows are WEIGHT rows (always a full
// 256-row slice) and the accumulator columns are TOKENS, so the ragged dimension becomes the
// MMA's N extent, which is chosen per tile in steps of 16.  An expert with 520 rows costs
// 256 + 256 + 16 token columns instead of five 128-row tiles.
//
//   pair_fwd_kernel<false>: y[t,n] = sum_k w[e,n,k] x[t,k]   A = w (K-major),  B = x (K-major)
//   pair_fwd_kernel<true> : y[t,n] = sum_k w[e,k,n] x[t,k]   A = w (MN-major), B = x (K-major)
#pragma once

namespace moe {
namespace tc {

constexpr int PAIR_THREADS = 192;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_TOKENS = 256;             // token columns per tile (MMA N), upper bound
constexpr int PAIR_HALF_BYTES = 128 * BK * 2;  // 16 KB: 128 rows x 64 x 16-bit

struct PairControl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum { GM_IN = 0, GM_OUT = 1 };            // per-expert tensor-map slots of the forward / dX kernels
constexpr int PAIR_STAGING_BYTES = 32 * 128;  // 32 tokens x 64 weight rows x 16 bit

enum PairWaitCode { PW_EMPTY = 11, PW_FULL = 12, PW_TMEM_EMPTY = 13, PW_TMEM_FULL = 14, PW_PEER = 15 };

template <typename T>
__device__ __forceinline__ void store_scalar(void* out, int64_t idx, float v) {
  reinterpret_cast<T*>(out)[idx] = from_f32<T>(v);
}

// Epilogue of one accumulator (n_mma token columns of this CTA's 128 weight rows) for 16-bit
// outputs: TMEM is read in the accumulator-fragment shape, packed to 16 bit and transposed by
// stmatrix into a swizzled [token][weight row] staging tile (32 tokens x 2 x 64 weight rows per
// round, double buffered), which leaves through TMA stores; `my` is the expert's output map,
// so rows past the group's end and columns past N are clipped.  Called by the 128 epilogue
// threads (warps 2..5); `staging` holds 4 * PAIR_STAGING_BYTES.
__device__ __forceinline__ void pair_store_tile_staged(uint8_t* staging, uint32_t& chunk_it, uint32_t taddr, int n_mma,
                                                       int quarter, int lane, int epi_tid, bool is_bf16,
                                                       const CUtensorMap* my, int n_cta, int t0, int N, int debug) {
  const int half = quarter >> 1;
  const int chunk = 4 * (quarter & 1) + (lane >> 3);  // 16-byte chunk of the 128-byte staging row
#pragma unroll 1
  for (int c = 0; c < n_mma; c += 32, ++chunk_it) {
    uint8_t* buf = staging + (chunk_it & 1) * (2 * PAIR_STAGING_BYTES);
    if (epi_tid == 0) tma_store_wait_read<1>();  // the stores of two rounds ago have read this buffer
    named_barrier_sync(1, 128);
    uint32_t lo[16], hi[16];
    if (!(debug & 2)) {
      tmem_ld_16x256b_x4(taddr + c, lo);
      tmem_ld_16x256b_x4(taddr + c + (16u << 16), hi);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) { lo[i] = 0; hi[i] = 0; }
    }
    uint8_t* tile_buf = buf + half * PAIR_STAGING_BYTES;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t m0, m1, m2, m3;
      if (is_bf16) {
        m0 = pack2<__nv_bfloat16>(__uint_as_float(lo[4 * g + 0]), __uint_as_float(lo[4 * g + 1]));
        m1 = pack2<__nv_bfloat16>(__uint_as_float(lo[4 * g + 2]), __uint_as_float(lo[4 * g + 3]));
        m2 = pack2<__nv_bfloat16>(__uint_as_float(hi[4 * g + 0]), __uint_as_float(hi[4 * g + 1]));
        m3 = pack2<__nv_bfloat16>(__uint_as_float(hi[4 * g + 2]), __uint_as_float(hi[4 * g + 3]));
      } else {
        m0 = pack2<__half>(__uint_as_float(lo[4 * g + 0]), __uint_as_float(lo[4 * g + 1]));
        m1 = pack2<__half>(__uint_as_float(lo[4 * g + 2]), __uint_as_float(lo[4 * g + 3]));
        m2 = pack2<__half>(__uint_as_float(hi[4 * g + 0]), __uint_as_float(hi[4 * g + 1]));
        m3 = pack2<__half>(__uint_as_float(hi[4 * g + 2]), __uint_as_float(hi[4 * g + 3]));
      }
      const int trow = 8 * g + (lane & 7);
      stmatrix_x4_trans(smem_u32(tile_buf + trow * 128 + ((chunk ^ (trow & 7)) << 4)), m0, m1, m2, m3);
    }
    fence_proxy_async_smem();
    named_barrier_sync(1, 128);
    if (epi_tid == 0 && !(debug & 1)) {
      tma_store_2d(my, buf, n_cta, t0 + c);
      if (n_cta + 64 < N) tma_store_2d(my, buf + PAIR_STAGING_BYTES, n_cta + 64, t0 + c);
      tma_store_commit();
    }
  }
}

// h = T(T(e * sigmoid(e)) * g) for e = T(acc_gate), g = T(acc_up): the rounding points of the
// separate kernels (grouped GEMM output in T, then qwen3_moe_fused/kernels/silu_mul.py:34-39),
// so the fused result is bit-identical to forward + forward + SiLU-mul.
template <typename T>
__device__ __forceinline__ float gate_up_one(float acc_gate, float acc_up) {
  const float e = to_f32(from_f32<T>(acc_gate));
  const float g = to_f32(from_f32<T>(acc_up));
  const float f = to_f32(from_f32<T>(e * __fdividef(1.f, 1.f + __expf(-e))));
  return f * g;  // rounded to T by the caller's pack
}

// Epilogue of the fused gate/up kernel.  A warp's 32 accumulator rows are 16 gate rows (TMEM
// lanes 0..15 of its quarter) and the 16 up rows of the same features (lanes 16..31): the two
// 16x256b loads put gate and up of one (feature, token) into the same register index of the same
// thread.  The warp stores 16 features x 32 tokens per round (two transposed 8x8 matrices per
// 8 tokens); the CTA's four warps fill a [32 tokens][64 features] tile that leaves by TMA.
__device__ __forceinline__ void pair_store_tile_gate_up(uint8_t* staging, uint32_t& chunk_it, uint32_t taddr, int n_mma,
                                                        int quarter, int lane, int epi_tid, bool is_bf16,
                                                        const CUtensorMap* my, int feat_cta, int t0, int n_feat, int debug) {
  const int chunk = 2 * quarter + ((lane >> 3) & 1);  // 16-byte chunk of the 128-byte staging row
#pragma unroll 1
  for (int c = 0; c < n_mma; c += 32, ++chunk_it) {
    uint8_t* buf = staging + (chunk_it & 1) * (2 * PAIR_STAGING_BYTES);
    if (epi_tid == 0) tma_store_wait_read<1>();
    named_barrier_sync(1, 128);
    uint32_t lo[16], hi[16];
    tmem_ld_16x256b_x4(taddr + c, lo);
    tmem_ld_16x256b_x4(taddr + c + (16u << 16), hi);
    tmem_ld_wait();
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = __uint_as_float(lo[4 * g + i]), b = __uint_as_float(hi[4 * g + i]);
        h[i] = is_bf16 ? gate_up_one<__nv_bfloat16>(a, b) : gate_up_one<__half>(a, b);
      }
      const uint32_t m0 = is_bf16 ? pack2<__nv_bfloat16>(h[0], h[1]) : pack2<__half>(h[0], h[1]);
      const uint32_t m1 = is_bf16 ? pack2<__nv_bfloat16>(h[2], h[3]) : pack2<__half>(h[2], h[3]);
      const int trow = 8 * g + (lane & 7);
      stmatrix_x2_trans(smem_u32(buf + trow * 128 + ((chunk ^ (trow & 7)) << 4)), m0, m1);
    }
    fence_proxy_async_smem();
    named_barrier_sync(1, 128);
    if (epi_tid == 0 && !(debug & 1)) {
      if (feat_cta < n_feat) tma_store_2d(my, buf, feat_cta, t0 + c);  // columns past the last feature are clipped
      tma_store_commit();
    }
  }
}

// ---------------------------------------------------------------------------------------
// forward / dX
//
// GATE_UP (forward only): tmap_w / tmap_w2 are the gate and up weights (E, I, K); the pair's 256
// accumulator rows are 128 features x {gate, up}, interleaved in slabs of 16 rows
// [gate f..f+15][up f..f+15]... so that a warp's quarter of TMEM holds gate and up of the same 16
// features; the epilogue writes h = silu(gate) * up (p.N = I columns) and neither projection.
// ---------------------------------------------------------------------------------------
template <bool W_MN, bool GATE_UP = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
pair_fwd_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const GemmParams p, const __grid_constant__ CUtensorMap tmap_w2) {
  static_assert(!(W_MN && GATE_UP), "the fused gate/up form reads K-major weights");
  constexpr int TILE_N = GATE_UP ? 128 : 256;  // output columns (features) per pair
  constexpr int STAGE_BYTES = 2 * PAIR_HALF_BYTES;  // A half-tile + B half-tile per CTA
  constexpr int STAGES = PAIR_STAGES;
  constexpr uint32_t TMEM_COLS = 512;  // two accumulators of up to 256 token columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // [buffer 0/1][weight-row half 0/1][32 tokens x 128 B]
  PairControl* ctl = reinterpret_cast<PairControl*>(staging + 4 * PAIR_STAGING_BYTES);
  int* row_start = reinterpret_cast<int*>(ctl + 1);
  int* tt_start = row_start + (p.E + 1);  // token tiles before each expert
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 8); }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, PAIR_TOKENS, row_start, tt_start);
  tc_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs are initialised before anybody signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + TILE_N - 1) / TILE_N;  // 256 weight rows per pair
  const int k_blocks = (p.K + BK - 1) / BK;
  const int64_t total_tiles = (int64_t)tt_start[p.E] * n_tiles;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // tile -> (expert, first token, token columns rounded up to 16, first weight row)
  auto decode = [&](int64_t tile, int& e, int& t0, int& n_mma, int& n0) {
    const int q = (int)(tile / n_tiles);
    e = find_group(tt_start, p.E, q);
    const int tt_e = tt_start[e + 1] - tt_start[e];
    const int j = (int)(tile - (int64_t)tt_start[e] * n_tiles);
    t0 = row_start[e] + (j % tt_e) * PAIR_TOKENS;
    n0 = (j / tt_e) * TILE_N;
    const int left = row_start[e + 1] - t0;
    n_mma = left >= PAIR_TOKENS ? PAIR_TOKENS : ((left + 15) & ~15);
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      const uint32_t full_leader0 = map_to_cta(smem_u32(&ctl->full[0]), 0);
      uint32_t it = 0;
      bool ok = true;
      int last_e = -1;
      for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
        int e, t0, n_mma, n0;
        decode(tile, e, t0, n_mma, n0);
        const int we = p.weight_index ? __ldg(p.weight_index + e) : e;  // several groups may share a weight slice
        const int w_row = n0 + (int)rank * 128;
        const int tok = t0 + (int)rank * (n_mma >> 1);
        // with per-expert maps the token rows past the group's end are zero-filled, not fetched
        const CUtensorMap* mx = p.group_maps ? p.group_maps + (size_t)GM_IN * p.E + e : &tmap_x;
        if (p.group_maps && e != last_e) { tensormap_acquire(mx); last_e = e; }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + PAIR_HALF_BYTES;
          const uint32_t bar = full_leader0 + s * 8;
          if (leader) mbar_expect_tx(&ctl->full[s], 2 * STAGE_BYTES);  // both CTAs' bytes
          if constexpr (GATE_UP) {
            const int feat = n0 + (int)rank * 64;  // this CTA's 64 features
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              tma_load_3d_pair(sa + (2 * q) * 2048, &tmap_w, bar, kb * BK, feat + 16 * q, we);
              tma_load_3d_pair(sa + (2 * q + 1) * 2048, &tmap_w2, bar, kb * BK, feat + 16 * q, we);
            }
          } else if constexpr (!W_MN) {
            tma_load_3d_pair(sa, &tmap_w, bar, kb * BK, w_row, we);
          } else {
            tma_load_3d_pair(sa, &tmap_w, bar, w_row, kb * BK, we);
            tma_load_3d_pair(sa + BK * 128, &tmap_w, bar, w_row + 64, kb * BK, we);
          }
          tma_load_2d_pair(sb, mx, bar, kb * BK, tok);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (leader && elect_one()) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs, ++acc_it) {
        int e, t0, n_mma, n0;
        decode(tile, e, t0, n_mma, n0);
        const uint32_t idesc = p.idesc | ((uint32_t)(n_mma >> 3) << 17);
        const uint32_t acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait_cluster(&ctl->tmem_empty[acc], acc_ph ^ 1, abort_flag, PW_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * PAIR_TOKENS;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cluster(&ctl->full[s], ph, abort_flag, PW_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + PAIR_HALF_BYTES;
          const uint64_t da = W_MN ? make_smem_desc(sa, BK * 128, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t db = make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t b_adv = (uint64_t)((k * UMMA_K * 2) >> 4);
            const uint64_t a_adv = W_MN ? (uint64_t)((k * UMMA_K * 128) >> 4) : b_adv;
            if (!(p.debug & 4)) umma_f16_pair(d_tmem, da + a_adv, db + b_adv, idesc, (kb | k) != 0);
          }
          umma_commit_pair(&ctl->empty[s], 3);
        }
        if (ok) umma_commit_pair(&ctl->tmem_full[acc], 3);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 64;  // 0..127
    const uint32_t tmem_empty_leader0 = map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0);
    // 16-bit outputs with per-expert output maps leave through shared memory and TMA stores
    const bool staged = p.group_maps != nullptr && p.dtype_out != MOE_F32;
    const bool is_bf16 = p.dtype_out == MOE_BF16;
    uint32_t acc_it = 0, chunk_it = 0;
    int last_e = -1;
    bool ok = true;
    for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs, ++acc_it) {
      int e, t0, n_mma, n0;
      decode(tile, e, t0, n_mma, n0);
      const int n = n0 + (int)rank * 128 + quarter * 32 + lane;  // this thread's weight row = output column
      const bool n_ok = n < p.N;
      const int t_end = row_start[e + 1];
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      const CUtensorMap* my = staged ? p.group_maps + (size_t)GM_OUT * p.E + e : nullptr;
      if (staged && epi_tid == 0 && e != last_e) { tensormap_acquire(my); last_e = e; }
      if (!mbar_wait_cluster(&ctl->tmem_full[acc], acc_ph, abort_flag, PW_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * PAIR_TOKENS + ((uint32_t)(quarter * 32) << 16);
      if constexpr (GATE_UP) {
        // (the host only launches this form with per-expert output maps and a 16-bit output)
        pair_store_tile_gate_up(staging, chunk_it, taddr, n_mma, quarter, lane, epi_tid, is_bf16, my,
                                n0 + (int)rank * 64, t0, p.N, p.debug);
      } else if (staged) {
        pair_store_tile_staged(staging, chunk_it, taddr, n_mma, quarter, lane, epi_tid, is_bf16, my,
                               n0 + (int)rank * 128, t0, p.N, p.debug);
      } else {
#pragma unroll 1
      for (int c = 0; c < n_mma; c += 32) {
        uint32_t v[32];
        if (!(p.debug & 2)) {
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = c + i;
        }
        if (n_ok && !(p.debug & 1)) {
          const int64_t base = (int64_t)(t0 + c) * p.N + n;
          const int valid = min(32, t_end - (t0 + c));  // tokens of this chunk that belong to the expert
          if (p.dtype_out == MOE_BF16) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) store_scalar<__nv_bfloat16>(p.out, base + (int64_t)j * p.N, __uint_as_float(v[j]));
          } else if (p.dtype_out == MOE_F16) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) store_scalar<__half>(p.out, base + (int64_t)j * p.N, __uint_as_float(v[j]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) store_scalar<float>(p.out, base + (int64_t)j * p.N, __uint_as_float(v[j]));
          }
        }
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tmem_empty_leader0 + acc * 8);
    }
    if (staged && epi_tid == 0) tma_store_wait_all();
  }

  tc_fence_before_sync();
  cluster_sync_all();  // nobody frees TMEM or exits while the peer may still touch this CTA
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace tc
}  // namespace moe
