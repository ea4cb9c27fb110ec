// CTA-pair forward / dX with 512-token tiles.  Included by tc_gemm.cu.
//
// Same operand roles as tc_gemm_pair.cuh (accumulator rows = 256 weight rows of one expert,
// accumulator columns = tokens), with two changes that cut the bytes each SM has to pull
// from L2 per unit of tensor work, which is what bounds the 256-token form:
//   * one tile covers up to 512 tokens: the weight (A) stage is loaded once per k-block and
//     used by two MMAs, one per 256-token accumulator (TMEM columns 0..255 and 256..511);
//   * token (B) tiles are loaded through per-expert tensor maps whose row extent ends at the
//     group's last row, so a partial tile's missing rows are zero-filled without being fetched.
// Both TMEM accumulators belong to the same tile, so the epilogue is not overlapped with the
// next tile's MMAs; it is kept short instead: TMEM is read in the 16x256b shape (the mma
// fragment layout), packed to 16 bit, transposed by stmatrix.trans into a swizzled
// [token][weight row] staging tile, and written with TMA stores through a per-expert output
// map that clips at the group's last row.  The loads of the next tile's first stages proceed
// during the epilogue.  fp32 outputs are stored from registers.
#pragma once

namespace moe {
namespace tc {

constexpr int P2_THREADS = 192;
constexpr int P2_STAGES = 4;
constexpr int P2_STAGE_BYTES = 3 * PAIR_HALF_BYTES;  // A half + two B halves = 48 KB
constexpr int P2_STAGING_BYTES = 64 * 128;           // 64 tokens x 64 weight rows x 16 bit
enum { GM_IN = 0, GM_OUT = 1 };                       // per-expert map slots

__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Four 8x8 16-bit matrices, stored transposed: lane l supplies the address of memory row
// (l % 8) of matrix (l / 8).
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t smem_addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};"
               ::"r"(smem_addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}

template <bool W_MN>
__global__ void __launch_bounds__(P2_THREADS, 1)
pair_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
  constexpr int STAGES = P2_STAGES;
  constexpr int STAGE_BYTES = P2_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * STAGE_BYTES;  // [buffer 0/1][weight-row half 0/1][64 tokens x 128 B]
  PairControl* ctl = reinterpret_cast<PairControl*>(staging + 4 * P2_STAGING_BYTES);
  int* row_start = reinterpret_cast<int*>(ctl + 1);
  int* tt_start = row_start + (p.E + 1);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    mbar_init(&ctl->tmem_full[0], 1);
    mbar_init(&ctl->tmem_empty[0], 8);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, 512, row_start, tt_start);
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + 255) / 256;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int64_t total_tiles = (int64_t)tt_start[p.E] * n_tiles;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // tile -> expert, first token, token columns of the two accumulators (multiples of 16; the
  // second may be 0), first weight row
  auto decode = [&](int64_t tile, int& e, int& t0, int& c0, int& c1, int& n0) {
    const int q = (int)(tile / n_tiles);
    e = find_group(tt_start, p.E, q);
    const int tt_e = tt_start[e + 1] - tt_start[e];
    const int j = (int)(tile - (int64_t)tt_start[e] * n_tiles);
    t0 = row_start[e] + (j % tt_e) * 512;
    n0 = (j / tt_e) * 256;
    const int left = min(512, row_start[e + 1] - t0);
    c0 = left >= 256 ? 256 : ((left + 15) & ~15);
    c1 = left > 256 ? ((left - 256 + 15) & ~15) : 0;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      const uint32_t full_leader0 = map_to_cta(smem_u32(&ctl->full[0]), 0);
      uint32_t it = 0;
      bool ok = true;
      int last_e = -1;
      for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs) {
        int e, t0, c0, c1, n0;
        decode(tile, e, t0, c0, c1, n0);
        const CUtensorMap* mx = p.group_maps + (size_t)GM_IN * p.E + e;
        if (e != last_e) { tensormap_acquire(mx); last_e = e; }
        const int w_row = n0 + (int)rank * 128;
        const int tok0 = t0 + (int)rank * (c0 >> 1);
        const int tok1 = t0 + 256 + (int)rank * (c1 >> 1);
        const uint32_t tx = 2 * (uint32_t)(c1 > 0 ? 3 : 2) * PAIR_HALF_BYTES;  // both CTAs
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          const uint32_t bar = full_leader0 + s * 8;
          if (leader) mbar_expect_tx(&ctl->full[s], tx);
          if constexpr (!W_MN) {
            tma_load_3d_pair(sa, &tmap_w, bar, kb * BK, w_row, e);
          } else {
            tma_load_3d_pair(sa, &tmap_w, bar, w_row, kb * BK, e);
            tma_load_3d_pair(sa + BK * 128, &tmap_w, bar, w_row + 64, kb * BK, e);
          }
          tma_load_2d_pair(sa + PAIR_HALF_BYTES, mx, bar, kb * BK, tok0);
          if (c1 > 0) tma_load_2d_pair(sa + 2 * PAIR_HALF_BYTES, mx, bar, kb * BK, tok1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (leader && elect_one()) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs, ++tile_it) {
        int e, t0, c0, c1, n0;
        decode(tile, e, t0, c0, c1, n0);
        const uint32_t idesc0 = p.idesc | ((uint32_t)(c0 >> 3) << 17);
        const uint32_t idesc1 = p.idesc | ((uint32_t)(c1 >> 3) << 17);
        // the epilogue of the previous tile has read both accumulators
        if (!mbar_wait_cluster(&ctl->tmem_empty[0], (tile_it & 1) ^ 1, abort_flag, PW_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cluster(&ctl->full[s], ph, abort_flag, PW_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = W_MN ? make_smem_desc(sa, BK * 128, 1024) : make_smem_desc(sa, 16, 1024);
          const uint64_t db0 = make_smem_desc(sa + PAIR_HALF_BYTES, 16, 1024);
          const uint64_t db1 = make_smem_desc(sa + 2 * PAIR_HALF_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t b_adv = (uint64_t)((k * UMMA_K * 2) >> 4);
            const uint64_t a_adv = W_MN ? (uint64_t)((k * UMMA_K * 128) >> 4) : b_adv;
            if (!(p.debug & 4)) {
              umma_f16_pair(tmem_base, da + a_adv, db0 + b_adv, idesc0, (kb | k) != 0);
              if (c1 > 0) umma_f16_pair(tmem_base + 256, da + a_adv, db1 + b_adv, idesc1, (kb | k) != 0);
            }
          }
          umma_commit_pair(&ctl->empty[s], 3);
        }
        if (ok) umma_commit_pair(&ctl->tmem_full[0], 3);
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int quarter = warp & 3;             // TMEM lanes [32*quarter, +32) = weight rows of this warp
    const int epi_tid = threadIdx.x - 64;     // 0..127
    const int half = quarter >> 1;            // which 64-row staging tile this warp fills
    const uint32_t tmem_empty_leader = map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0);
    const bool staged = p.dtype_out != MOE_F32;
    const bool is_bf16 = p.dtype_out == MOE_BF16;
    uint32_t tile_it = 0, chunk_it = 0;
    bool ok = true;
    int last_e = -1;
    for (int64_t tile = pair_id; tile < total_tiles && ok; tile += num_pairs, ++tile_it) {
      int e, t0, c0, c1, n0;
      decode(tile, e, t0, c0, c1, n0);
      const CUtensorMap* my = p.group_maps + (size_t)GM_OUT * p.E + e;
      if (staged && epi_tid == 0 && e != last_e) { tensormap_acquire(my); last_e = e; }
      const int n_cta = n0 + (int)rank * 128;  // first weight row (= output column) of this CTA
      const int t_end = row_start[e + 1];
      if (!mbar_wait_cluster(&ctl->tmem_full[0], tile_it & 1, abort_flag, PW_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const int cols = c1 > 0 ? 256 + c1 : c0;  // accumulator columns in use (c0 == 256 when c1 > 0)
      if (staged) {
#pragma unroll 1
        for (int c = 0; c < cols; c += 64, ++chunk_it) {
          uint8_t* buf = staging + (chunk_it & 1) * (2 * P2_STAGING_BYTES);
          if (epi_tid == 0) tma_store_wait_read<1>();
          named_barrier_sync(1, 128);
          uint32_t lo[32], hi[32];  // TMEM lanes +0..15 and +16..31 of this warp, 64 token columns
          if (!(p.debug & 2)) {
            tmem_ld_16x256b_x8(tmem_base + c + ((uint32_t)(quarter * 32) << 16), lo);
            tmem_ld_16x256b_x8(tmem_base + c + ((uint32_t)(quarter * 32 + 16) << 16), hi);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) { lo[i] = 0; hi[i] = 0; }
          }
          // this lane addresses staging row (token) 8 g + lane % 8 and 16-byte chunk
          // 4 (quarter % 2) + lane / 8 of the 128-byte row; 128-byte swizzle on the chunk index
          uint8_t* tile_buf = buf + half * P2_STAGING_BYTES;
          const int chunk = 4 * (quarter & 1) + (lane >> 3);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
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
          if (epi_tid == 0 && !(p.debug & 1)) {
            // rows past the group's end and columns past N are clipped by the tensor map
            tma_store_2d(my, buf, n_cta, t0 + c);
            if (n_cta + 64 < p.N) tma_store_2d(my, buf + P2_STAGING_BYTES, n_cta + 64, t0 + c);
            tma_store_commit();
          }
        }
      } else {
        const int n = n_cta + quarter * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < cols; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + c + ((uint32_t)(quarter * 32) << 16), v);
          tmem_ld_wait();
          if (n < p.N && !(p.debug & 1)) {
            const int64_t base = (int64_t)(t0 + c) * p.N + n;
            const int valid = min(32, t_end - (t0 + c));
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) store_scalar<float>(p.out, base + (int64_t)j * p.N, __uint_as_float(v[j]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tmem_empty_leader);
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
