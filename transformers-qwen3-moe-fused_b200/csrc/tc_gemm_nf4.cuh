// CTA-pair forward grouped GEMM with the NF4 weight decoded into the A stage.
// Included by tc_gemm.cu.
//
// Same tiling as pair_fwd_kernel<false> (accumulator rows = 256 weight rows of one expert,
// 128 per CTA; accumulator columns = up to 256 tokens; two TMEM accumulators so the epilogue
// overlaps the next tile), but the weight half-tile of a stage is not loaded as 16-bit data:
// TMA brings the 4 KB of packed 4-bit codes (128 rows x 32 bytes) and sixteen decode warps per
// CTA (four groups of four, taking k-blocks in turn) expand them to the swizzled K-major 16-bit tile the MMA reads.  HBM and L2 see
// 0.5 + 4/blocksize bytes per weight instead of 2.
//
// Synchronisation per stage s:
//   qfull[s]  (local)   packed codes of this CTA have landed            TMA tx
//   full[s]   (leader)  token tiles of both CTAs have landed            TMA tx from both CTAs
//   ready[s]  (leader)  decoded weight tiles of both CTAs are written   8 arrivals (4 warps x 2 CTAs)
//   empty[s]  (both)    the MMAs that read the stage have completed     tcgen05.commit, multicast
// The decode warps publish their shared-memory writes to the async proxy
// (fence.proxy.async) before arriving on the leader's barrier.
//
// pair_fwd_nf4_kernel<IS_BF16, true> is the transposed form (dX through an NF4 weight):
//   y[t, n] = sum_k w[e, k, n] x[t, k],  w = the (E, K, N) NF4 tensor, n contiguous in a block
// A stage then holds 64 contraction rows x 128 output features per CTA: the codes arrive as a
// 64 x 64-byte box, a decode thread owns (contraction row, 64-feature half) = one absmax block,
// and the 16-bit tile is written in the MN-major form pair_fwd_kernel<true> loads by TMA
// (two chunks of 64 rows x 128 bytes).
//
// Decode without table reads from shared memory (shared-memory bandwidth is what bounds
// these kernels): a thread owns 32 consecutive weights of one row, which share one absmax.
// It first forms the 16 possible values round16(code[n] * absmax) in registers, splits
// them into a low-byte and a high-byte plane of 16 bytes each, and then looks four 4-bit
// codes up at a time with byte permutes (prmt): one permute per half of a plane, one to
// choose between the halves by the codes' top bit, and two to interleave the planes back
// into 16-bit values.  The result is bit-identical to rounding code[n] * absmax per weight.
#pragma once

namespace moe {
namespace tc {

#ifndef MOE_NF4P_GROUPS
#define MOE_NF4P_GROUPS 4
#endif
constexpr int NF4P_GROUPS = MOE_NF4P_GROUPS;                    // decode groups of four warps, taking k-blocks in turn
constexpr int NF4P_THREADS = 192 + NF4P_GROUPS * 128;           // TMA, MMA, 4 epilogue warps + the decode warps
constexpr int NF4P_STAGES = 5;
constexpr int NF4P_PACKED_BYTES = 128 * (BK / 2);               // 4 KB
constexpr int NF4P_STAGE_BYTES = 2 * PAIR_HALF_BYTES + NF4P_PACKED_BYTES;  // 36 KB

struct Nf4PairControl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t qfull[8];
  uint64_t ready[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// Byte planes of the 16 scaled values: lo[i] holds the low bytes of values 4i..4i+3, hi[i] the high bytes.
struct Nf4Planes { uint32_t lo[4], hi[4]; };

template <bool IS_BF16>
__device__ __forceinline__ Nf4Planes nf4_make_planes(const float (&code)[16], float absmax) {
  Nf4Planes pl;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t p0, p1;  // (v[4i], v[4i+1]) and (v[4i+2], v[4i+3]) as packed 16-bit pairs
    if constexpr (IS_BF16) {
      p0 = pack2<__nv_bfloat16>(code[4 * i] * absmax, code[4 * i + 1] * absmax);
      p1 = pack2<__nv_bfloat16>(code[4 * i + 2] * absmax, code[4 * i + 3] * absmax);
    } else {
      p0 = pack2<__half>(code[4 * i] * absmax, code[4 * i + 1] * absmax);
      p1 = pack2<__half>(code[4 * i + 2] * absmax, code[4 * i + 3] * absmax);
    }
    pl.lo[i] = prmt(p0, p1, 0x6420);
    pl.hi[i] = prmt(p0, p1, 0x7531);
  }
  return pl;
}

// Two packed bytes (four codes; element 2b is the high nibble of byte b) -> two words of
// 16-bit values in element order.
__device__ __forceinline__ void nf4_lookup4(const Nf4Planes& pl, uint32_t two_bytes, uint32_t& out01, uint32_t& out23) {
  // nibbles of `two_bytes` from the least significant: e1, e0, e3, e2
  const uint32_t sel = two_bytes & 0x7777u;                          // index inside a half plane
  const uint32_t pick = 0x3210u | ((two_bytes >> 1) & 0x4444u);      // byte i from the upper half when bit 3 is set
  const uint32_t lo = prmt(prmt(pl.lo[0], pl.lo[1], sel), prmt(pl.lo[2], pl.lo[3], sel), pick);
  const uint32_t hi = prmt(prmt(pl.hi[0], pl.hi[1], sel), prmt(pl.hi[2], pl.hi[3], sel), pick);
  out01 = prmt(lo, hi, 0x4051);  // (e0, e1)
  out23 = prmt(lo, hi, 0x6273);  // (e2, e3)
}

template <bool IS_BF16, bool W_T = false>
__global__ void __launch_bounds__(NF4P_THREADS, 1)
pair_fwd_nf4_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_x,
                    const GemmParams p, const Nf4Params q) {
  constexpr int STAGES = NF4P_STAGES;
  constexpr int STAGE_BYTES = NF4P_STAGE_BYTES;
  constexpr int B_OFF = PAIR_HALF_BYTES;
  constexpr int Q_OFF = 2 * PAIR_HALF_BYTES;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // epilogue staging, 4 * PAIR_STAGING_BYTES
  Nf4PairControl* ctl = reinterpret_cast<Nf4PairControl*>(staging + 4 * PAIR_STAGING_BYTES);
  int* row_start = reinterpret_cast<int*>(ctl + 1);
  int* tt_start = row_start + (p.E + 1);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
      mbar_init(&ctl->qfull[s], 1);
      mbar_init(&ctl->ready[s], 8);
    }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 8); }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, PAIR_TOKENS, row_start, tt_start);
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + 255) / 256;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int64_t total_tiles = (int64_t)tt_start[p.E] * n_tiles;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  auto decode = [&](int64_t tile, int& e, int& t0, int& n_mma, int& n0) {
    const int qd = (int)(tile / n_tiles);
    e = find_group(tt_start, p.E, qd);
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
      int last_e = -1;
      for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
        int e, t0, n_mma, n0;
        decode(tile, e, t0, n_mma, n0);
        const int w_row = n0 + (int)rank * 128;
        const int tok = t0 + (int)rank * (n_mma >> 1);
        const CUtensorMap* mx = p.group_maps ? p.group_maps + (size_t)GM_IN * p.E + e : &tmap_x;
        if (p.group_maps && e != last_e) { tensormap_acquire(mx); last_e = e; }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY)) { ok = false; break; }
          uint8_t* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&ctl->qfull[s], NF4P_PACKED_BYTES);
          if constexpr (!W_T) tma_load_3d(st + Q_OFF, &tmap_q, &ctl->qfull[s], kb * (BK / 2), w_row, e);
          else tma_load_3d(st + Q_OFF, &tmap_q, &ctl->qfull[s], w_row / 2, kb * BK, e);
          if (leader) mbar_expect_tx(&ctl->full[s], 2 * PAIR_HALF_BYTES);
          tma_load_2d_pair(st + B_OFF, mx, full_leader0 + s * 8, kb * BK, tok);
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
          if (!mbar_wait_cluster(&ctl->ready[s], ph, abort_flag, PW_PEER)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = W_T ? make_smem_desc(sa, BK * 128, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t db = make_smem_desc(sa + B_OFF, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
            const uint64_t a_adv = W_T ? (uint64_t)((k * UMMA_K * 128) >> 4) : adv;
            umma_f16_pair(d_tmem, da + a_adv, db + adv, idesc, (kb | k) != 0);
          }
          umma_commit_pair(&ctl->empty[s], 3);
        }
        if (ok) umma_commit_pair(&ctl->tmem_full[acc], 3);
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 64;
    const uint32_t tmem_empty_leader0 = map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0);
    const bool staged = p.group_maps != nullptr && p.dtype_out != MOE_F32;
    uint32_t acc_it = 0, chunk_it = 0;
    int last_e = -1;
    bool ok = true;
    for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs, ++acc_it) {
      int e, t0, n_mma, n0;
      decode(tile, e, t0, n_mma, n0);
      const int n = n0 + (int)rank * 128 + quarter * 32 + lane;
      const bool n_ok = n < p.N;
      const int t_end = row_start[e + 1];
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      const CUtensorMap* my = staged ? p.group_maps + (size_t)GM_OUT * p.E + e : nullptr;
      if (staged && epi_tid == 0 && e != last_e) { tensormap_acquire(my); last_e = e; }
      if (!mbar_wait_cluster(&ctl->tmem_full[acc], acc_ph, abort_flag, PW_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * PAIR_TOKENS + ((uint32_t)(quarter * 32) << 16);
      if (staged) {
        pair_store_tile_staged(staging, chunk_it, taddr, n_mma, quarter, lane, epi_tid, p.dtype_out == MOE_BF16, my,
                               n0 + (int)rank * 128, t0, p.N);
      } else {
#pragma unroll 1
      for (int c = 0; c < n_mma; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        if (n_ok) {
          const int64_t base = (int64_t)(t0 + c) * p.N + n;
          const int valid = min(32, t_end - (t0 + c));
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
  } else {
    // ------------------------------ decode warps (both CTAs) ------------------------------
    // NF4P_GROUPS groups of four warps take the k-blocks in turn, so the decode of one k-block (a
    // few hundred cycles of dependent work per thread) overlaps the decode of the next ones.
    // Measured at 262144 rows: 2 groups 1162 TFLOP/s, 4 groups 1255.  Inside a
    // group, thread -> weight row (t % 128) of this CTA's half-tile; it decodes the row's 64
    // weights of the k-block (32 packed bytes, one absmax).
    const int t = threadIdx.x - 6 * 32;
    const int row = t & 127;
    const int group = t >> 7;
    const uint32_t ready_leader0 = map_to_cta(smem_u32(&ctl->ready[0]), 0);
    float code[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) code[i] = __ldg(q.code + i);
    uint32_t it = 0;
    bool ok = true;
    for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
      int e, t0, n_mma, n0;
      decode(tile, e, t0, n_mma, n0);
      // forward: the thread's weight row n, its k-block kb covers columns kb*64..; flat index of
      // (e, n, kb*64).  transposed: contraction row kb*64 + (row & 63), output features
      // n0 + rank*128 + (row >> 6)*64 ..+63; flat index of (e, that row, that first feature).
      const int n = W_T ? n0 + (int)rank * 128 + (row >> 6) * 64 : n0 + (int)rank * 128 + row;
      const bool n_ok = n < p.N;
      const int64_t row_flat = W_T ? ((int64_t)e * p.K + (row & 63)) * p.N + (n_ok ? n : 0)
                                   : ((int64_t)e * p.N + (n_ok ? n : 0)) * p.K;
      const int64_t kb_stride = W_T ? (int64_t)BK * p.N : (int64_t)BK;  // flat elements from one k-block to the next
      // k-blocks of this tile that belong to this group: kb0, kb0 + NF4P_GROUPS, ... (global k-block it + kb goes to group (it + kb) % NF4P_GROUPS)
      const int kb0 = (int)(((uint32_t)group + NF4P_GROUPS - (it % NF4P_GROUPS)) % NF4P_GROUPS);
      // absmax of the next AM_AHEAD own k-blocks is kept in flight: one L2 round trip per
      // k-block would otherwise sit on the decode path
      constexpr int AM_AHEAD = 3;
      float am_ring[AM_AHEAD];
#pragma unroll
      for (int i = 0; i < AM_AHEAD; ++i) {
        const int kbi = kb0 + NF4P_GROUPS * i;
        am_ring[i] = (n_ok && kbi < k_blocks) ? __ldg(q.absmax + ((row_flat + (int64_t)kbi * kb_stride) >> q.shift)) : 0.f;
      }
      for (int kb = kb0; kb < k_blocks; kb += NF4P_GROUPS) {
        const uint32_t my_it = it + kb;
        const int s = my_it % STAGES;
        const uint32_t ph = (my_it / STAGES) & 1;
        const float am = am_ring[0];
#pragma unroll
        for (int i = 0; i + 1 < AM_AHEAD; ++i) am_ring[i] = am_ring[i + 1];
        {
          const int kbn = kb + NF4P_GROUPS * AM_AHEAD;
          am_ring[AM_AHEAD - 1] = (n_ok && kbn < k_blocks) ? __ldg(q.absmax + ((row_flat + (int64_t)kbn * kb_stride) >> q.shift)) : 0.f;
        }
        if (!mbar_wait(&ctl->qfull[s], ph, abort_flag, PW_FULL)) { ok = false; break; }
        uint8_t* st = smem + s * STAGE_BYTES;
        // forward: 128 rows x 32 bytes; transposed: 64 rows x 64 bytes, this thread's half of its row
        const uint4* src = reinterpret_cast<const uint4*>(st + Q_OFF + (W_T ? (row & 63) * 64 + (row >> 6) * 32 : row * (BK / 2)));
        const uint4 raw0 = src[0], raw1 = src[1];
        const uint32_t words[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
        uint8_t* dst_row = st + row * 128;
        const Nf4Planes pl = nf4_make_planes<IS_BF16>(code, am);
#pragma unroll
        for (int w = 0; w < 8; ++w) {  // 4 bytes -> 8 values -> one 16-byte chunk
          uint32_t outw[4];
          nf4_lookup4(pl, words[w] & 0xffffu, outw[0], outw[1]);
          nf4_lookup4(pl, words[w] >> 16, outw[2], outw[3]);
          *reinterpret_cast<uint4*>(dst_row + ((w ^ (row & 7)) << 4)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(ready_leader0 + s * 8);
      }
      it += k_blocks;
    }
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
