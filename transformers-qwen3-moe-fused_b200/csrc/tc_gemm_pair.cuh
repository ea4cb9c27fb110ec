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
//   pair_dw_kernel        : w[e,n,k] = sum_t y[t,n] x[t,k]   A = y^T, B = x (both MN-major),
//                           output tiles written with TMA stores from a swizzled staging tile
#pragma once

namespace moe {
namespace tc {

constexpr int PAIR_THREADS = 192;
constexpr int PAIR_TOKENS = 256;             // token columns per tile (MMA N), upper bound
constexpr int PAIR_HALF_BYTES = 128 * BK * 2;  // 16 KB: 128 rows x 64 x 16-bit

struct PairControl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t peer_ready[8];   // dW only: peer CTA's stage is loaded (and its tail zeroed)
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

enum PairWaitCode { PW_EMPTY = 11, PW_FULL = 12, PW_TMEM_EMPTY = 13, PW_TMEM_FULL = 14, PW_PEER = 15 };

template <typename T>
__device__ __forceinline__ void store_scalar(void* out, int64_t idx, float v) {
  reinterpret_cast<T*>(out)[idx] = from_f32<T>(v);
}

// ---------------------------------------------------------------------------------------
// forward / dX
// ---------------------------------------------------------------------------------------
template <bool W_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
pair_fwd_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const GemmParams p) {
  constexpr int STAGE_BYTES = 2 * PAIR_HALF_BYTES;  // A half-tile + B half-tile per CTA
  constexpr int STAGES = 6;
  constexpr uint32_t TMEM_COLS = 512;  // two accumulators of up to 256 token columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  PairControl* ctl = reinterpret_cast<PairControl*>(smem + STAGES * STAGE_BYTES);
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

  const int n_tiles = (p.N + 255) / 256;  // 256 weight rows per pair
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
    n0 = (j / tt_e) * 256;
    const int left = row_start[e + 1] - t0;
    n_mma = left >= PAIR_TOKENS ? PAIR_TOKENS : ((left + 15) & ~15);
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      const uint32_t full_leader0 = map_to_cta(smem_u32(&ctl->full[0]), 0);
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
        int e, t0, n_mma, n0;
        decode(tile, e, t0, n_mma, n0);
        const int w_row = n0 + (int)rank * 128;
        const int tok = t0 + (int)rank * (n_mma >> 1);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + PAIR_HALF_BYTES;
          const uint32_t bar = full_leader0 + s * 8;
          if (leader) mbar_expect_tx(&ctl->full[s], 2 * STAGE_BYTES);  // both CTAs' bytes
          if constexpr (!W_MN) {
            tma_load_3d_pair(sa, &tmap_w, bar, kb * BK, w_row, e);
          } else {
            tma_load_3d_pair(sa, &tmap_w, bar, w_row, kb * BK, e);
            tma_load_3d_pair(sa + BK * 128, &tmap_w, bar, w_row + 64, kb * BK, e);
          }
          tma_load_2d_pair(sb, &tmap_x, bar, kb * BK, tok);
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
    const uint32_t tmem_empty_leader0 = map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0);
    uint32_t acc_it = 0;
    bool ok = true;
    for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs, ++acc_it) {
      int e, t0, n_mma, n0;
      decode(tile, e, t0, n_mma, n0);
      const int n = n0 + (int)rank * 128 + quarter * 32 + lane;  // this thread's weight row = output column
      const bool n_ok = n < p.N;
      const int t_end = row_start[e + 1];
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait_cluster(&ctl->tmem_full[acc], acc_ph, abort_flag, PW_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * PAIR_TOKENS + ((uint32_t)(quarter * 32) << 16);
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
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tmem_empty_leader0 + acc * 8);
    }
  }

  tc_fence_before_sync();
  cluster_sync_all();  // nobody frees TMEM or exits while the peer may still touch this CTA
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// dW
// ---------------------------------------------------------------------------------------
// Work item = (expert, 256 weight rows, 256 weight columns); CTA r of the pair owns weight
// rows n0 + 128 r .. +127 (its A half and its accumulator rows) and stages weight columns
// k0 + 128 r .. +127 of the B operand.  Each CTA's loads complete on its own barrier; warp 1
// of the peer zeroes the rows of a tail block that belong to the next expert and then
// tells the leader (peer_ready) that its half of the stage can be consumed.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
pair_dw_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x,
               const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
  constexpr int STAGE_BYTES = 2 * PAIR_HALF_BYTES;  // 32 KB
  constexpr int STAGES = 5;
  constexpr int CHUNK_BYTES = BK * 128;   // 64 reduction rows x 128 B
  constexpr int STAGING_BYTES = 128 * 128;  // 128 output rows x 64 16-bit columns
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // two buffers
  PairControl* ctl = reinterpret_cast<PairControl*>(staging + 2 * STAGING_BYTES);
  int* row_start = reinterpret_cast<int*>(ctl + 1);
  int* scratch = row_start + (p.E + 1);
  int* sorted = scratch + (p.E + 1);  // sorted[r] = expert with the r-th largest group
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
      mbar_init(&ctl->peer_ready[s], 1);
    }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 8); }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_dy);
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, BK, row_start, scratch);
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const int me = row_start[e + 1] - row_start[e];
    int rk = 0;
    for (int o = 0; o < p.E; ++o) {
      const int mo = row_start[o + 1] - row_start[o];
      rk += (mo > me) || (mo == me && o < e);
    }
    sorted[rk] = e;
  }
  __syncthreads();
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + 255) / 256;
  const int k_tiles = (p.K + 255) / 256;
  const int per_expert = n_tiles * k_tiles;
  const int64_t total_items = (int64_t)p.E * per_expert;
  const int G = gridDim.x >> 1;
  const int pair_id = blockIdx.x >> 1;
  const int64_t rounds = (total_items + G - 1) / G;
  auto item_of = [&](int64_t r) -> int64_t { return r * G + ((r & 1) ? (G - 1 - pair_id) : pair_id); };

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t r = 0; r < rounds && ok; ++r) {
        const int64_t item = item_of(r);
        if (item >= total_items) continue;
        const int e = sorted[item / per_expert];
        const int j = (int)(item % per_expert);
        const int n0 = (j % n_tiles) * 256 + (int)rank * 128;
        const int k0 = (j / n_tiles) * 256 + (int)rank * 128;
        const int r0 = row_start[e];
        const int m_blocks = (row_start[e + 1] - r0 + BK - 1) / BK;
        for (int mb = 0; mb < m_blocks; ++mb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + PAIR_HALF_BYTES;
          mbar_expect_tx(&ctl->full[s], STAGE_BYTES);
          tma_load_2d(sa, &tmap_dy, &ctl->full[s], n0, r0 + mb * BK);
          tma_load_2d(sa + CHUNK_BYTES, &tmap_dy, &ctl->full[s], n0 + 64, r0 + mb * BK);
          tma_load_2d(sb, &tmap_x, &ctl->full[s], k0, r0 + mb * BK);
          tma_load_2d(sb + CHUNK_BYTES, &tmap_x, &ctl->full[s], k0 + 64, r0 + mb * BK);
        }
      }
    }
  } else if (warp == 1) {
    // Both CTAs: wait for the own stage, fix the tail, then the peer reports and the leader issues.
    const uint32_t peer_ready_leader0 = map_to_cta(smem_u32(&ctl->peer_ready[0]), 0);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    for (int64_t r = 0; r < rounds && ok; ++r) {
      const int64_t item = item_of(r);
      if (item >= total_items) continue;
      const int e = sorted[item / per_expert];
      const int rows = row_start[e + 1] - row_start[e];
      const int m_blocks = (rows + BK - 1) / BK;
      if (m_blocks == 0) continue;
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (leader) {
        if (!mbar_wait_cluster(&ctl->tmem_empty[acc], acc_ph ^ 1, abort_flag, PW_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
      }
      const uint32_t d_tmem = tmem_base + acc * 256;
      for (int mb = 0; mb < m_blocks; ++mb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&ctl->full[s], ph, abort_flag, PW_FULL)) { ok = false; break; }
        uint8_t* sa_ptr = smem + s * STAGE_BYTES;
        const int valid = rows - mb * BK;
        if (valid < BK) {
          // lane -> (chunk = lane / 8 of the 4 chunks, 16-byte column = lane % 8); rows past `valid`
          uint8_t* col = sa_ptr + (lane >> 3) * CHUNK_BYTES + (lane & 7) * 16;
          for (int row = valid; row < BK; ++row) *reinterpret_cast<uint4*>(col + row * 128) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (!leader) {
          if (lane == 0) mbar_arrive_cluster(peer_ready_leader0 + s * 8);
        } else {
          if (!mbar_wait_cluster(&ctl->peer_ready[s], ph, abort_flag, PW_PEER)) { ok = false; break; }
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t sa = smem_u32(sa_ptr);
            const uint32_t sb = sa + PAIR_HALF_BYTES;
            const uint64_t da = make_smem_desc(sa, CHUNK_BYTES, 1024);
            const uint64_t db = make_smem_desc(sb, CHUNK_BYTES, 1024);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adv = (uint64_t)((k * UMMA_K * 128) >> 4);
              if (!(p.debug & 4)) umma_f16_pair(d_tmem, da + adv, db + adv, p.idesc, (mb | k) != 0);
            }
            umma_commit_pair(&ctl->empty[s], 3);
          }
        }
        __syncwarp();
      }
      if (ok && leader && lane == 0) umma_commit_pair(&ctl->tmem_full[acc], 3);
      __syncwarp();
      ++acc_it;
    }
  } else {
    // epilogue: TMEM -> 16-bit -> swizzled staging tile -> TMA store, 64 columns at a time
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // accumulator row = weight row inside this CTA's 128
    const int epi_tid = threadIdx.x - 64;  // 0..127
    const uint32_t tmem_empty_leader0 = map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0);
    const bool is_bf16 = p.dtype_out == MOE_BF16;
    uint32_t acc_it = 0, chunk_it = 0;
    bool ok = true;
    for (int64_t r = 0; r < rounds && ok; ++r) {
      const int64_t item = item_of(r);
      if (item >= total_items) continue;
      const int e = sorted[item / per_expert];
      const int j = (int)(item % per_expert);
      const int n0 = (j % n_tiles) * 256 + (int)rank * 128;
      const int k0 = (j / n_tiles) * 256;
      const int rows = row_start[e + 1] - row_start[e];
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (rows > 0) {
        if (!mbar_wait_cluster(&ctl->tmem_full[acc], acc_ph, abort_flag, PW_TMEM_FULL)) { ok = false; break; }
        tc_fence_after_sync();
      }
      const uint32_t taddr = tmem_base + acc * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 4; ++c, ++chunk_it) {
        if (k0 + c * 64 >= p.K) break;  // uniform over the CTA
        uint8_t* buf = staging + (chunk_it & 1) * STAGING_BYTES;
        // the store that last read this buffer (two chunks ago) must have finished reading
        if (epi_tid == 0) tma_store_wait_read<1>();
        named_barrier_sync(1, 128);
        uint32_t v[64];
        if (rows > 0 && !(p.debug & 2)) {
          tmem_ld_32x32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
          tmem_ld_32x32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] = 0;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {  // 8 chunks of 16 bytes = 64 columns
          uint4 o;
          if (is_bf16) {
            o.x = pack2<__nv_bfloat16>(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
            o.y = pack2<__nv_bfloat16>(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
            o.z = pack2<__nv_bfloat16>(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
            o.w = pack2<__nv_bfloat16>(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
          } else {
            o.x = pack2<__half>(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
            o.y = pack2<__half>(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
            o.z = pack2<__half>(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
            o.w = pack2<__half>(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
          }
          *reinterpret_cast<uint4*>(buf + row * 128 + ((q ^ (row & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (epi_tid == 0 && !(p.debug & 1)) {
          tma_store_3d(&tmap_out, buf, k0 + c * 64, n0, e);  // rows/columns past N/K are clipped
          tma_store_commit();
        }
      }
      if (rows > 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tmem_empty_leader0 + acc * 8);
        ++acc_it;
      }
    }
    if (epi_tid == 0) tma_store_wait_all();
  }

  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace tc
}  // namespace moe
