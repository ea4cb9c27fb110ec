// Weight-gradient grouped GEMM, w[e,n,k] = sum_{t in group e} dy[t,n] * x[t,k], and the
// set-up kernel that derives per-expert tensor maps.  Included by tc_gemm.cu.
//
// Per-expert tensor maps.  The reduction runs over an expert's rows in blocks of 64; the
// last block reaches past the group's end into the next expert's rows.  Instead of
// zeroing those rows in shared memory, every expert gets its own copy of the dy / x tensor
// maps whose row extent ends at the group's last row, so TMA zero-fills the overhang (and
// does not even fetch it).  The copies are produced on the device from m_sizes by
// build_group_maps_kernel (tensormap.replace + tensormap.cp_fenceproxy) into caller-provided
// workspace, one launch before the GEMM.
//
// dw_kernel<PAIR, BN>
//   PAIR = false: one CTA per work item (expert, 128 weight rows, BN weight columns)
//   PAIR = true : a CTA pair per work item (expert, 256 weight rows, 256 weight columns),
//                 tcgen05 cta_group::2; both CTAs' loads complete on the leader's barrier
// Work items are ordered by decreasing group size and handed out one by one from a global
// counter (drawn by the otherwise idle warp 1 of the non-leader CTA and passed to the working
// roles through a ring in shared memory): longest items first onto whichever CTA pair is free,
// so one expert with a quarter of the rows does not leave most of the GPU waiting for the few
// pairs that drew its items.  Without a counter the items are dealt round-robin.
// The last reduction block of an expert only issues the MMA k-steps that hold real rows.
// 16-bit outputs leave through a swizzled staging tile and TMA stores (the output has no ragged
// dimension; TMA clips at N and K); fp32 outputs (single-CTA form only) are stored from registers.
#pragma once

namespace moe {
namespace tc {

struct GroupMapTemplates {
  static constexpr int MAX = 3;
  CUtensorMap t[MAX];
  int mask;  // bit t set: slot t is derived for every expert
};

// out[t * E + e] = templates.t[t] with the extent of dimension 1 (rows) set to the last row
// of expert e (exclusive), for every slot t of templates.mask.  One warp per expert.
// Also resets the work-item counter of the GEMM launched after it.
// With `out_ptrs`, slot `ptr_slot` of group e is additionally re-based so that row row_start[e]
// of the map is the address out_ptrs[e]: each group's rows then land in a buffer of their own
// (possibly in a peer GPU's memory) while the kernels keep addressing rows by their position in
// the concatenated input.  `row_bytes` is the pitch of that slot's rows.
__global__ void __launch_bounds__(256)
build_group_maps_kernel(const __grid_constant__ GroupMapTemplates tm, const void* __restrict__ m_sizes, int ms64,
                        int E, int64_t M, CUtensorMap* __restrict__ out, int* __restrict__ counters,
                        const uint64_t* __restrict__ out_ptrs = nullptr, int ptr_slot = -1, int64_t row_bytes = 0) {
  extern __shared__ uint8_t gm_smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gm_smem_raw) + 127) & ~(uintptr_t)127);
  CUtensorMap* slots = reinterpret_cast<CUtensorMap*>(base);  // 8 slots, one per warp
  int* row_start = reinterpret_cast<int*>(base + 8 * 128);
  int* scratch = row_start + (E + 1);
  // the GEMM that follows draws its work items from counters[0]
  if (counters != nullptr && blockIdx.x == 0 && threadIdx.x == 0) counters[0] = 0;
  build_group_tables(m_sizes, ms64, E, M, 64, row_start, scratch);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * 8 + warp;
  if (e >= E) return;
  const uint32_t row_end = (uint32_t)max(row_start[e + 1], 1);
  for (int t = 0; t < GroupMapTemplates::MAX; ++t) {
    if (!(tm.mask & (1 << t))) continue;
    reinterpret_cast<uint32_t*>(&slots[warp])[lane] = reinterpret_cast<const uint32_t*>(&tm.t[t])[lane];
    __syncwarp();
    if (lane == 0) {
      tensormap_replace_dim<1>(&slots[warp], row_end);
      if (out_ptrs != nullptr && t == ptr_slot) {
        uint64_t addr = out_ptrs[e];
        if (addr & 15) {  // a tensor map needs a 16-byte aligned base: record it and keep the store legal
          atomicCAS(&g_tc_error, 0, (16 << 16) | (e & 0xffff));
          addr &= ~(uint64_t)15;
        }
        tensormap_replace_address(&slots[warp], addr - (uint64_t)row_start[e] * (uint64_t)row_bytes);
      }
    }
    __syncwarp();
    tensormap_publish(&out[(size_t)t * E + e], &slots[warp]);
    __syncwarp();
  }
}

enum { GM_DY = 0, GM_X = 1 };  // slots of the dW kernel's per-expert maps

struct DwControl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  SchedRing sched;
  uint32_t tmem_base;
  int abort_flag;
};

template <bool PAIR, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
dw_kernel(const __grid_constant__ CUtensorMap tmap_out, const GemmParams p) {
  constexpr int ROWS = PAIR ? 256 : 128;          // weight rows per work item
  constexpr int B_CHUNKS = PAIR ? 2 : BN / 64;    // 64-wide chunks of the x operand staged per CTA
  constexpr int CHUNK_BYTES = BK * 128;           // 64 reduction rows x 128 B
  constexpr int STAGE_BYTES = (2 + B_CHUNKS) * CHUNK_BYTES;
  constexpr int STAGING_BYTES = 128 * 128;        // 128 output rows x 64 16-bit columns
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t NCTA = PAIR ? 2 : 1;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  DwControl* ctl = reinterpret_cast<DwControl*>(staging + 2 * STAGING_BYTES);
  int* row_start = reinterpret_cast<int*>(ctl + 1);
  int* sorted = row_start + (p.E + 1);  // E + 1 entries: scratch for the table builder, then the order
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0;
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 4 * NCTA); }
    TileFeed<NCTA>::init(&ctl->sched);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    if constexpr (PAIR) { tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(&ctl->tmem_base, TMEM_COLS); tmem_relinquish(); }
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, BK, row_start, sorted);
  {
    // rank by (size descending, expert ascending); ranks are kept in registers until every
    // thread has finished reading the scratch use of `sorted`
    int my_rank[8];
    int cnt = 0;
    for (int e = threadIdx.x; e < p.E; e += blockDim.x, ++cnt) {
      const int me = row_start[e + 1] - row_start[e];
      int rk = 0;
      for (int o = 0; o < p.E; ++o) {
        const int mo = row_start[o + 1] - row_start[o];
        rk += (mo > me) || (mo == me && o < e);
      }
      my_rank[cnt & 7] = rk;
    }
    __syncthreads();
    cnt = 0;
    for (int e = threadIdx.x; e < p.E; e += blockDim.x, ++cnt) sorted[my_rank[cnt & 7]] = e;
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + ROWS - 1) / ROWS;
  const int k_tiles = (p.K + BN - 1) / BN;
  const int per_expert = n_tiles * k_tiles;
  const int total_items = p.E * per_expert;
  const int G = PAIR ? (gridDim.x >> 1) : gridDim.x;
  const int unit = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      TileFeed<NCTA> feed(&ctl->sched, abort_flag);
      const uint32_t full0 = PAIR ? map_to_cta(smem_u32(&ctl->full[0]), 0) : smem_u32(&ctl->full[0]);
      uint32_t it = 0;
      bool ok = true;
      int last_e = -1;
      // single-CTA form: this thread also draws the work items (the value of a draw is first looked
      // at one item later, so that the atomic's round trip overlaps the loads in between)
      uint32_t drawn = 0;
      auto draw = [&]() -> int64_t {
        const int64_t t = p.tile_counter ? (int64_t)atomicAdd(p.tile_counter, 1) : (int64_t)unit + (int64_t)drawn * G;
        ++drawn;
        return t;
      };
      int64_t next = PAIR ? 0 : draw();
      while (ok) {
        int item;
        if constexpr (PAIR) {
          item = feed.take();
        } else {
          item = next < total_items ? (int)next : -1;
          if (!feed.publish(item)) break;
          if (item >= 0) next = draw();
        }
        if (item < 0) break;
        const int e = sorted[item / per_expert];
        const int j = (int)(item % per_expert);
        const int n0 = (j % n_tiles) * ROWS + (int)rank * 128;
        const int k0 = (j / n_tiles) * BN + (PAIR ? (int)rank * 128 : 0);
        const int r0 = row_start[e];
        const int m_blocks = (row_start[e + 1] - r0 + BK - 1) / BK;
        const CUtensorMap* mdy = p.group_maps + (size_t)GM_DY * p.E + e;
        const CUtensorMap* mx = p.group_maps + (size_t)GM_X * p.E + e;
        if (e != last_e && m_blocks > 0) { tensormap_acquire(mdy); tensormap_acquire(mx); last_e = e; }
        for (int mb = 0; mb < m_blocks; ++mb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, W_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + 2 * CHUNK_BYTES;
          const uint32_t bar = full0 + s * 8;
          if (leader) mbar_expect_tx(&ctl->full[s], NCTA * STAGE_BYTES);
          const int row = r0 + mb * BK;
          if constexpr (PAIR) {
            tma_load_2d_pair(sa, mdy, bar, n0, row);
            tma_load_2d_pair(sa + CHUNK_BYTES, mdy, bar, n0 + 64, row);
#pragma unroll
            for (int c = 0; c < B_CHUNKS; ++c) tma_load_2d_pair(sb + c * CHUNK_BYTES, mx, bar, k0 + c * 64, row);
          } else {
            tma_load_2d(sa, mdy, &ctl->full[s], n0, row);
            tma_load_2d(sa + CHUNK_BYTES, mdy, &ctl->full[s], n0 + 64, row);
#pragma unroll
            for (int c = 0; c < B_CHUNKS; ++c) tma_load_2d(sb + c * CHUNK_BYTES, mx, &ctl->full[s], k0 + c * 64, row);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA) ------------------------------
    if (!leader) {
      // (CTA pairs only) this warp has no MMAs to issue in the non-leader CTA: it draws the work items
      if (elect_one()) {
        TileFeed<NCTA> feed(&ctl->sched, abort_flag);
        feed.run(p.tile_counter, total_items, unit, G);
      }
    } else if (elect_one()) {
      TileFeed<NCTA> feed(&ctl->sched, abort_flag);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      while (ok) {
        const int item = feed.take();
        if (item < 0) break;
        const int e = sorted[item / per_expert];
        const int rows = row_start[e + 1] - row_start[e];
        const int m_blocks = (rows + BK - 1) / BK;
        if (m_blocks == 0) continue;  // empty expert: the epilogue writes zeros on its own
        // rows of the last block past the expert's end are zero-filled by TMA: their k-steps are skipped
        const int last_steps = (rows - (m_blocks - 1) * BK + UMMA_K - 1) / UMMA_K;
        const uint32_t acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait_cluster(&ctl->tmem_empty[acc], acc_ph ^ 1, abort_flag, W_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        // One reduction block of 64 rows: `steps` MMAs of 16 rows.  The full blocks use the unrolled,
        // branch-free form (a test between the MMAs of one block slows the issuing thread markedly);
        // only the expert's last block runs the counted loop.
        auto issue_block = [&](int mb, auto full_block, int steps) -> bool {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_cluster(&ctl->full[s], ph, abort_flag, W_FULL)) return false;
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + 2 * CHUNK_BYTES;
          const uint64_t da = make_smem_desc(sa, CHUNK_BYTES, 1024);
          const uint64_t db = make_smem_desc(sb, CHUNK_BYTES, 1024);
          if constexpr (decltype(full_block)::value) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t adv = (uint64_t)((k * UMMA_K * 128) >> 4);
              if constexpr (PAIR) umma_f16_pair(d_tmem, da + adv, db + adv, p.idesc, (mb | k) != 0);
              else umma_f16(d_tmem, da + adv, db + adv, p.idesc, (mb | k) != 0);
            }
          } else {
#pragma unroll 1
            for (int k = 0; k < steps; ++k) {
              const uint64_t adv = (uint64_t)((k * UMMA_K * 128) >> 4);
              if constexpr (PAIR) umma_f16_pair(d_tmem, da + adv, db + adv, p.idesc, (mb | k) != 0);
              else umma_f16(d_tmem, da + adv, db + adv, p.idesc, (mb | k) != 0);
            }
          }
          if constexpr (PAIR) umma_commit_pair(&ctl->empty[s], 3); else umma_commit(&ctl->empty[s]);
          ++it;
          return true;
        };
        for (int mb = 0; mb + 1 < m_blocks && ok; ++mb) ok = issue_block(mb, std::true_type{}, BK / UMMA_K);
        if (ok) ok = issue_block(m_blocks - 1, std::false_type{}, last_steps);
        if (ok) { if constexpr (PAIR) umma_commit_pair(&ctl->tmem_full[acc], 3); else umma_commit(&ctl->tmem_full[acc]); }
        ++acc_it;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;   // accumulator row = weight row inside this CTA's 128
    const int epi_tid = threadIdx.x - 64;  // 0..127
    const uint32_t tmem_empty0 = PAIR ? map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0) : smem_u32(&ctl->tmem_empty[0]);
    const bool staged = p.dtype_out != MOE_F32;
    const bool is_bf16 = p.dtype_out == MOE_BF16;
    const bool vec = ((p.K * (int)dtype_size(p.dtype_out)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    TileFeed<NCTA> feed(&ctl->sched, abort_flag);
    uint32_t acc_it = 0, chunk_it = 0;
    bool ok = true;
    while (ok) {
      const int item = feed.take_warp(lane);
      if (named_barrier_any(2, 128, item < 0)) break;  // the four warps leave together
      const int e = sorted[item / per_expert];
      const int j = (int)(item % per_expert);
      const int n0 = (j % n_tiles) * ROWS + (int)rank * 128;
      const int k0 = (j / n_tiles) * BN;
      const int rows = row_start[e + 1] - row_start[e];
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (rows > 0) {
        if (named_barrier_any(2, 128, !mbar_wait_cluster(&ctl->tmem_full[acc], acc_ph, abort_flag, W_TMEM_FULL))) { ok = false; break; }
        tc_fence_after_sync();
      }
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        if (k0 + c * 64 >= p.K) break;  // uniform over the CTA
        uint32_t v[64];
        if (rows > 0) {
          tmem_ld_32x32(taddr + c * 64, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
          tmem_ld_32x32(taddr + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] = 0;
        }
        if (!staged) {
          // fp32 output: straight from registers
          const int n = n0 + row;
          if (n < p.N) {
            const int64_t o = ((int64_t)e * p.N + n) * p.K + k0 + c * 64;
            store_acc(p.out, p.dtype_out, o, *reinterpret_cast<uint32_t(*)[32]>(&v[0]), min(32, p.K - (k0 + c * 64)), vec);
            if (k0 + c * 64 + 32 < p.K)
              store_acc(p.out, p.dtype_out, o + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]), min(32, p.K - (k0 + c * 64 + 32)), vec);
          }
          continue;
        }
        uint8_t* buf = staging + (chunk_it & 1) * STAGING_BYTES;
        ++chunk_it;
        // the store that last read this buffer (two chunks ago) must have finished reading it
        if (epi_tid == 0) tma_store_wait_read<1>();
        named_barrier_sync(1, 128);
#pragma unroll
        for (int q = 0; q < 8; ++q) {  // 8 x 16 bytes = 64 columns
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
        if (epi_tid == 0) {
          tma_store_3d(&tmap_out, buf, k0 + c * 64, n0, e);  // rows / columns past N / K are clipped
          tma_store_commit();
        }
      }
      if (rows > 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(tmem_empty0 + acc * 8);
          else mbar_arrive(&ctl->tmem_empty[acc]);
        }
        ++acc_it;
      }
    }
    if (epi_tid == 0) tma_store_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace tc
}  // namespace moe
