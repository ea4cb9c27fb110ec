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
// MMA's N extent, which is chosen per tile in steps of 16.
//
//   pair_fwd_kernel<false>: y[t,n] = sum_k w[e,n,k] x[t,k]   A = w (K-major),  B = x (K-major)
//   pair_fwd_kernel<true> : y[t,n] = sum_k w[e,k,n] x[t,k]   A = w (MN-major), B = x (K-major)
//
// Tiles with a tail.  Streaming a 256 x K weight slice through shared memory costs the same
// for 16 tokens as for 256, so an expert with 520 rows must not become 256 + 256 + 8: its
// last tile carries the extra tokens as a second, narrow MMA on the same weight stage
// ("main" up to 256 columns + "tail" up to PAIR_TAIL columns).  TMEM has 512 columns, exactly
// two main accumulators, so the tails live inside the OTHER accumulator's column range:
//
//     columns   0 ........ 256-T | 256-T .. 256 | 256 .. 256+T | 256+T ........ 512
//     region          E0         |      RA      |      RB      |        E1
//     even tile   main ................main      | tail         |
//     odd tile                   | tail         | main ................ main
//
// Each region has its own "drained" barrier.  The epilogue drains the two contested regions
// first, so the next tile's MMAs wait for one or two 32-column rounds of the epilogue, not for
// all of it; tiles without a tail never wait for each other.
//
// Tile order.  Tiles are handed out in index order from a global counter (one atomicAdd per
// tile, by a thread that has nothing else to do: warp 1 of the non-leader CTA), and travel to
// the working roles of both CTAs through a small ring in shared memory, several tiles ahead of
// their use: ragged groups make tile costs uneven, and a static round-robin left a fifth of
// the pairs idle at the end.  Without a counter (no workspace) the same ring carries a static
// round-robin order.
#pragma once

namespace moe {
namespace tc {

#ifndef MOE_PAIR_TAIL
#define MOE_PAIR_TAIL 32
#endif
constexpr int PAIR_THREADS = 192;
constexpr int PAIR_MAX_STAGES = 6;
constexpr int PAIR_TOKENS = 256;               // main token columns per tile (MMA N), upper bound
constexpr int PAIR_TAIL = MOE_PAIR_TAIL;       // extra token columns the last tile of an expert may carry
constexpr int PAIR_HALF_BYTES = 128 * BK * 2;  // 16 KB: 128 rows x 64 x 16-bit
constexpr int PAIR_TAIL_BYTES = (PAIR_TAIL / 2) * BK * 2;           // this CTA's half of the tail tokens
constexpr int PAIR_STAGE_BYTES = 2 * PAIR_HALF_BYTES + PAIR_TAIL_BYTES;
constexpr int PAIR_SMALL_BOX = 16;             // token rows of the small TMA box (tails and narrow tiles)
constexpr int SCHED_DEPTH = 8;                 // tile ids in flight between the producer and the other roles
static_assert(PAIR_TAIL % 32 == 0 && PAIR_TAIL <= 64, "regions are drained in rounds of 32 columns");
static_assert(PAIR_STAGE_BYTES % 1024 == 0, "stages keep the 1024-byte alignment of the swizzle atoms");

// Ring that carries tile ids from the thread that draws them to the other roles.
struct SchedRing {
  uint64_t full[SCHED_DEPTH];
  uint64_t empty[SCHED_DEPTH];  // the leader CTA's copies are the ones used
  int tile[SCHED_DEPTH];
};

struct PairControl {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_free[4];            // regions E0, RA, RB, E1 (leader CTA's copies are the ones used)
  SchedRing sched;
  uint32_t tmem_base;
  int abort_flag;
};

enum { GM_IN = 0, GM_OUT = 1, GM_IN_SMALL = 2 };  // per-expert tensor-map slots of the forward / dX kernels
enum { REG_E0 = 0, REG_RA = 1, REG_RB = 2, REG_E1 = 3 };
constexpr int PAIR_STAGING_BYTES = 32 * 128;  // 32 tokens x 64 weight rows x 16 bit

enum PairWaitCode { PW_EMPTY = 11, PW_FULL = 12, PW_TMEM_EMPTY = 13, PW_TMEM_FULL = 14, PW_PEER = 15,
                    PW_SCHED_FULL = 17, PW_SCHED_EMPTY = 18, PW_SCHED_VALUE = 19 };

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
                                                       const CUtensorMap* my, int n_cta, int t0, int N) {
  const int half = quarter >> 1;
  const int chunk = 4 * (quarter & 1) + (lane >> 3);  // 16-byte chunk of the 128-byte staging row
#pragma unroll 1
  for (int c = 0; c < n_mma; c += 32, ++chunk_it) {
    uint8_t* buf = staging + (chunk_it & 1) * (2 * PAIR_STAGING_BYTES);
    if (epi_tid == 0) tma_store_wait_read<1>();  // the stores of two rounds ago have read this buffer
    named_barrier_sync(1, 128);
    uint32_t lo[16], hi[16];
    tmem_ld_16x256b_x4(taddr + c, lo);
    tmem_ld_16x256b_x4(taddr + c + (16u << 16), hi);
    tmem_ld_wait();
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
    if (epi_tid == 0) {
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
                                                        const CUtensorMap* my, int feat_cta, int t0, int n_feat) {
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
    if (epi_tid == 0) {
      if (feat_cta < n_feat) tma_store_2d(my, buf, feat_cta, t0 + c);  // columns past the last feature are clipped
      tma_store_commit();
    }
  }
}

// Tile ids travel from the thread that draws them to every role that works on the tile.
// Slot q of the ring holds one id; `full[q]` (one per CTA) says it is there, `empty[q]` (the copy
// in the drawing thread's CTA; one arrival per reader) says everybody has read it.
//   NCTA = 2: the drawing thread is a thread of its own (warp 1 of the non-leader CTA, which has no
//             MMAs to issue); readers: both producers, the MMA thread, 8 epilogue warps.  It runs up
//             to SCHED_DEPTH tiles ahead, so the round trip of its atomicAdd is never waited for.
//   NCTA = 1: the producer thread draws for itself; readers: the MMA thread, 4 epilogue warps.
template <int NCTA>
struct TileFeed {
  static constexpr int READERS = NCTA == 2 ? 11 : 5;
  static constexpr uint32_t HOME = NCTA == 2 ? 1 : 0;  // CTA of the drawing thread
  SchedRing* ring;
  uint32_t home_empty0;  // address of the home CTA's empty[0] (shared::cluster window when NCTA = 2)
  uint32_t n = 0;        // sequence number of the next tile of this CTA / pair
  volatile int* abort_flag;

  __device__ __forceinline__ TileFeed(SchedRing* r, volatile int* a)
      : ring(r), home_empty0(NCTA == 2 ? map_to_cta(smem_u32(&r->empty[0]), HOME) : smem_u32(&r->empty[0])), abort_flag(a) {}

  // A slot holds (tile + 1) with the parity of its round (n / SCHED_DEPTH) in bit 31, so that a reader
  // can tell the id of its round from the one the slot held a round earlier.
  static __device__ __forceinline__ uint32_t encode(int tile, uint32_t round_parity) {
    return ((uint32_t)(tile + 1) & 0x7fffffffu) | (round_parity << 31);
  }
  static __device__ __forceinline__ void init(SchedRing* r) {  // one thread per CTA, before the barriers are used
    for (int q = 0; q < SCHED_DEPTH; ++q) {
      mbar_init(&r->full[q], 1);
      mbar_init(&r->empty[q], READERS);
      r->tile[q] = (int)0x80000000u;  // parity 1: not a value of round 0
    }
  }
  // drawing thread: make `tile` (or -1: no more tiles) visible to every reader
  __device__ __forceinline__ bool publish(int tile) {
    const uint32_t q = n % SCHED_DEPTH, ph = (n / SCHED_DEPTH) & 1;
    if (!mbar_wait_cluster(&ring->empty[q], ph ^ 1, abort_flag, PW_SCHED_EMPTY)) return false;
    const uint32_t v = encode(tile, ph);
    *(volatile uint32_t*)&ring->tile[q] = v;
    if constexpr (NCTA == 2) {
      st_shared_cluster_u32(map_to_cta(smem_u32(&ring->tile[q]), HOME ^ 1), v);
      fence_acq_rel_cluster();  // the value is in both CTAs' shared memory before either barrier hears of it
      mbar_arrive_release_cluster(map_to_cta(smem_u32(&ring->full[q]), 0));
      mbar_arrive_release_cluster(map_to_cta(smem_u32(&ring->full[q]), 1));
    } else {
      mbar_arrive(&ring->full[q]);
    }
    ++n;
    return true;
  }
  // Body of the drawing thread when it has nothing else to do (NCTA = 2): ids come from the global
  // counter, or round-robin (first, first + stride, ...) without one.
  __device__ __forceinline__ void run(int* counter, int total, int first, int stride) {
    for (int64_t next = first;; next += stride) {
      const int64_t t = counter ? (int64_t)atomicAdd(counter, 1) : next;
      const int tile = t < total ? (int)t : -1;
      if (!publish(tile) || tile < 0) return;
    }
  }
  // a reader (one thread): next tile id, or -1 when there are no more (or the wait was abandoned)
  __device__ __forceinline__ int take() {
    const uint32_t q = n % SCHED_DEPTH, ph = (n / SCHED_DEPTH) & 1;
    if (!mbar_wait_cluster(&ring->full[q], ph, abort_flag, PW_SCHED_FULL)) return -1;
    // the slot must hold this round's value (checked, not assumed: all roles of the pair have to agree
    // on the tile, or their barrier counts and byte counts stop matching)
    uint32_t v = *(volatile uint32_t*)&ring->tile[q];
    if ((v >> 31) != ph) {
      const unsigned long long t0 = global_ns();
      do {
        v = *(volatile uint32_t*)&ring->tile[q];
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
          atomicCAS(&g_tc_error, 0, (PW_SCHED_VALUE << 16) | (int)(blockIdx.x & 0xffff));
          *abort_flag = 1;
          return -1;
        }
      } while ((v >> 31) != ph);
      atomicAdd(&g_tc_late_values, 1);  // diagnostic: the barrier completed before the value was visible
    }
    // (the parity test above depends on the loaded value, so the load has completed before the slot is
    // handed back below)
    if constexpr (NCTA == 2) mbar_arrive_cluster(home_empty0 + q * 8);
    else mbar_arrive(&ring->empty[q]);
    ++n;
    return (int)(v & 0x7fffffffu) - 1;
  }
  // a whole warp: lane 0 takes the id and signs the slot off for the warp
  __device__ __forceinline__ int take_warp(int lane) {
    int tile = 0;
    if (lane == 0) tile = take();
    return __shfl_sync(0xffffffffu, tile, 0);
  }
};

struct PairTile {
  int e, t0, n0;       // expert, first token row, first weight row (output column) of the pair
  int n_main, n_tail;  // token columns of the two MMAs, multiples of 16 (n_tail may be 0)
  int t_end;           // first row past the expert
};

// Regions (bit r of the result) whose columns a tile of the given parity writes.
__device__ __forceinline__ uint32_t pair_regions(uint32_t parity, int n_main, int n_tail) {
  if (parity == 0)
    return (1u << REG_E0) | (n_main > PAIR_TOKENS - PAIR_TAIL ? 1u << REG_RA : 0u) | (n_tail > 0 ? 1u << REG_RB : 0u);
  return (1u << REG_RB) | (n_main > PAIR_TAIL ? 1u << REG_E1 : 0u) | (n_tail > 0 ? 1u << REG_RA : 0u);
}

// ---------------------------------------------------------------------------------------
// forward / dX
//
// GATE_UP (forward only): tmap_w / tmap_w2 are the gate and up weights (E, I, K); the pair's 256
// accumulator rows are 128 features x {gate, up}, interleaved in slabs of 16 rows
// [gate f..f+15][up f..f+15]... so that a warp's quarter of TMEM holds gate and up of the same 16
// features; the epilogue writes h = silu(gate) * up (p.N = I columns) and neither projection.
// ---------------------------------------------------------------------------------------
template <bool W_MN, bool GATE_UP = false, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
pair_fwd_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const GemmParams p, const __grid_constant__ CUtensorMap tmap_w2) {
  static_assert(!(W_MN && GATE_UP), "the fused gate/up form reads K-major weights");
  static_assert(!(W_MN && GATHER), "rows are gathered in the forward forms only");
  constexpr int TILE_N = GATE_UP ? 128 : 256;  // output columns (features) per pair
  constexpr int STAGE_BYTES = PAIR_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 512;
  const int STAGES = p.stages;

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
  // tails and small boxes need the per-expert small-box maps
  const bool small_maps = p.group_maps != nullptr && p.small_maps;
  const int tail = (small_maps || GATHER) ? PAIR_TAIL : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) mbar_init(&ctl->tmem_full[a], 1);
    for (int r = 0; r < 4; ++r) mbar_init(&ctl->tmem_free[r], 8);
    TileFeed<2>::init(&ctl->sched);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, PAIR_TOKENS, row_start, tt_start, tail);
  tc_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs are initialised before anybody signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + TILE_N - 1) / TILE_N;  // 256 weight rows per pair
  const int k_blocks = (p.K + BK - 1) / BK;
  const int64_t total_tiles = (int64_t)tt_start[p.E] * n_tiles;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // tile index -> tile.  Within an expert the token tile varies fastest, so neighbouring tiles
  // (which run at about the same time) read the same weight slice.
  auto decode = [&](int tile) {
    PairTile t;
    const int q = tile / n_tiles;
    t.e = find_group(tt_start, p.E, q);
    const int tt_e = tt_start[t.e + 1] - tt_start[t.e];
    const int j = tile - tt_start[t.e] * n_tiles;
    const int jt = j % tt_e;
    t.t0 = row_start[t.e] + jt * PAIR_TOKENS;
    t.n0 = (j / tt_e) * TILE_N;
    t.t_end = row_start[t.e + 1];
    const int left = t.t_end - t.t0;
    if (left >= PAIR_TOKENS) {
      t.n_main = PAIR_TOKENS;
      t.n_tail = (jt == tt_e - 1) ? ((left - PAIR_TOKENS + 15) & ~15) : 0;  // at most `tail` by the tile count
    } else {
      t.n_main = (left + 15) & ~15;
      t.n_tail = 0;
    }
    return t;
  };
  // B-operand loads of one stage: rows of this CTA's half of the main tokens, in boxes of 128 or of
  // PAIR_SMALL_BOX rows, and bytes both CTAs' loads of the stage bring in
  auto main_small_boxes = [&](int n_main) {  // 0: one 128-row box
    const int rows = n_main >> 1;
    return (small_maps && rows <= 64) ? (rows + PAIR_SMALL_BOX - 1) / PAIR_SMALL_BOX : 0;
  };
  auto tail_boxes = [&](int n_tail) { return ((n_tail >> 1) + PAIR_SMALL_BOX - 1) / PAIR_SMALL_BOX; };

  if (warp == 0 && GATHER) {
    // ---------------- TMA producer, token rows gathered through an index (both CTAs) ----------------
    // The tile's token rows are x[row_index[r] / index_div] for its sorted rows r: every lane owns four of
    // this CTA's (up to 128) main rows and fetches them per k-block with one tile::gather4 load (four rows
    // of 128 bytes, swizzled like a four-row box); lanes 0.. also own the tail rows.  Rows past the expert's
    // end get the row index x_rows, which lies outside the tensor: TMA fills them with zeros.
    TileFeed<2> feed(&ctl->sched, abort_flag);
    const uint32_t full_leader0 = map_to_cta(smem_u32(&ctl->full[0]), 0);
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    while (ok) {
      const int tile = feed.take_warp(lane);
      if (tile < 0) break;
      const PairTile t = decode(tile);
      const int we = p.weight_index ? __ldg(p.weight_index + t.e) : t.e;
      const int w_row = t.n0 + (int)rank * 128;
      const int rows_main = t.n_main >> 1, rows_tail = t.n_tail >> 1;  // this CTA's rows: multiples of 8
      const int tok = t.t0 + (int)rank * rows_main;
      const int tok_tail = t.t0 + PAIR_TOKENS + (int)rank * rows_tail;
      auto source_row = [&](int r) { return r < t.t_end ? __ldg(p.row_index + r) / p.index_div : (int)p.x_rows; };
      int mr[4], tr[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mr[j] = source_row(tok + 4 * lane + j);
        tr[j] = source_row(tok_tail + 4 * lane + j);
      }
      const bool has_main = 4 * lane < rows_main, has_tail = 4 * lane < rows_tail;
      const uint32_t b_bytes = (uint32_t)(rows_main + rows_tail) * (BK * 2);
      for (int kb = 0; kb < k_blocks; ++kb) {
        uint8_t* sa = smem + s * STAGE_BYTES;
        uint8_t* sb = sa + PAIR_HALF_BYTES;
        const uint32_t bar = full_leader0 + s * 8;
        int go = 1;
        if (lane == 0) {
          go = mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY) ? 1 : 0;
          if (go) {
            if (leader) mbar_expect_tx(&ctl->full[s], 2 * (PAIR_HALF_BYTES + b_bytes));  // both CTAs' bytes
            if constexpr (GATE_UP) {
              const int feat = t.n0 + (int)rank * 64;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                tma_load_3d_pair(sa + (2 * q) * 2048, &tmap_w, bar, kb * BK, feat + 16 * q, we);
                tma_load_3d_pair(sa + (2 * q + 1) * 2048, &tmap_w2, bar, kb * BK, feat + 16 * q, we);
              }
            } else {
              tma_load_3d_pair(sa, &tmap_w, bar, kb * BK, w_row, we);
            }
          }
        }
        go = __shfl_sync(0xffffffffu, go, 0);  // the stage is free (and its byte count announced) for every lane
        if (!go) { ok = false; break; }
        if (has_main) tma_gather4_pair(sb + lane * (4 * BK * 2), &tmap_x, bar, kb * BK, mr[0], mr[1], mr[2], mr[3]);
        if (has_tail) tma_gather4_pair(sb + PAIR_HALF_BYTES + lane * (4 * BK * 2), &tmap_x, bar, kb * BK, tr[0], tr[1], tr[2], tr[3]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (elect_one()) {
      TileFeed<2> feed(&ctl->sched, abort_flag);
      const uint32_t full_leader0 = map_to_cta(smem_u32(&ctl->full[0]), 0);
      uint32_t it = 0;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int last_e = -1;
      while (ok) {
        const int tile = feed.take();
        if (tile < 0) break;
        const PairTile t = decode(tile);
        const int we = p.weight_index ? __ldg(p.weight_index + t.e) : t.e;  // several groups may share a weight slice
        const int w_row = t.n0 + (int)rank * 128;
        const int tok = t.t0 + (int)rank * (t.n_main >> 1);
        const int tok_tail = t.t0 + PAIR_TOKENS + (int)rank * (t.n_tail >> 1);
        // with per-expert maps the token rows past the group's end are zero-filled, not fetched
        const CUtensorMap* mx = p.group_maps ? p.group_maps + (size_t)GM_IN * p.E + t.e : &tmap_x;
        const CUtensorMap* ms = small_maps ? p.group_maps + (size_t)GM_IN_SMALL * p.E + t.e : nullptr;
        if (p.group_maps && t.e != last_e) {
          tensormap_acquire(mx);
          if (ms) tensormap_acquire(ms);
          last_e = t.e;
        }
        const int nsb = main_small_boxes(t.n_main);
        const int ntb = tail_boxes(t.n_tail);
        const uint32_t b_bytes = (nsb ? nsb * PAIR_SMALL_BOX * BK * 2 : PAIR_HALF_BYTES) + ntb * PAIR_SMALL_BOX * BK * 2;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, PW_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + PAIR_HALF_BYTES;
          const uint32_t bar = full_leader0 + s * 8;
          if (leader) mbar_expect_tx(&ctl->full[s], 2 * (PAIR_HALF_BYTES + b_bytes));  // both CTAs' bytes
          if constexpr (GATE_UP) {
            const int feat = t.n0 + (int)rank * 64;  // this CTA's 64 features
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
          if (nsb == 0) {
            tma_load_2d_pair(sb, mx, bar, kb * BK, tok);
          } else {
            for (int b = 0; b < nsb; ++b)
              tma_load_2d_pair(sb + b * (PAIR_SMALL_BOX * BK * 2), ms, bar, kb * BK, tok + b * PAIR_SMALL_BOX);
          }
          for (int b = 0; b < ntb; ++b)
            tma_load_2d_pair(sb + PAIR_HALF_BYTES + b * (PAIR_SMALL_BOX * BK * 2), ms, bar, kb * BK, tok_tail + b * PAIR_SMALL_BOX);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------- MMA issuer (leader CTA); the same warp of the other CTA draws the tiles -------------
    if (!leader) {
      if (elect_one()) {
        TileFeed<2> feed(&ctl->sched, abort_flag);
        feed.run(p.tile_counter, (int)total_tiles, pair_id, num_pairs);
      }
    } else if (elect_one()) {
      TileFeed<2> feed(&ctl->sched, abort_flag);
      uint32_t seq = 0;
      uint32_t uses[4] = {0, 0, 0, 0};  // how often each TMEM region has been written so far
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok) {
        const int tile = feed.take();
        if (tile < 0) break;
        const PairTile t = decode(tile);
        const uint32_t par = seq & 1;
        const uint32_t idesc_main = p.idesc | ((uint32_t)(t.n_main >> 3) << 17);
        const uint32_t idesc_tail = p.idesc | ((uint32_t)(t.n_tail >> 3) << 17);
        // every region this tile writes must have been drained by its previous user
        const uint32_t regs = pair_regions(par, t.n_main, t.n_tail);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (!(regs & (1u << r))) continue;
          if (ok && !mbar_wait_cluster(&ctl->tmem_free[r], (uses[r] & 1) ^ 1, abort_flag, PW_TMEM_EMPTY)) ok = false;
          ++uses[r];
        }
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_main = tmem_base + (par ? PAIR_TOKENS : 0);
        const uint32_t d_tail = tmem_base + (par ? PAIR_TOKENS - PAIR_TAIL : PAIR_TOKENS);
        // Two copies of the k-loop, with and without the tail MMAs: a test of n_tail between the
        // MMAs of one loop costs the issuing thread a quarter of its rate.
        auto k_loop = [&](auto has_tail) {
          for (int kb = 0; kb < k_blocks; ++kb) {
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
              umma_f16_pair(d_main, da + a_adv, db + b_adv, idesc_main, (kb | k) != 0);
            }
            if constexpr (decltype(has_tail)::value) {
              const uint64_t dbt = make_smem_desc(sb + PAIR_HALF_BYTES, 16, 1024);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t b_adv = (uint64_t)((k * UMMA_K * 2) >> 4);
                const uint64_t a_adv = W_MN ? (uint64_t)((k * UMMA_K * 128) >> 4) : b_adv;
                umma_f16_pair(d_tail, da + a_adv, dbt + b_adv, idesc_tail, (kb | k) != 0);
              }
            }
            umma_commit_pair(&ctl->empty[s], 3);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        };
        if (t.n_tail) k_loop(std::true_type{}); else k_loop(std::false_type{});
        if (ok) umma_commit_pair(&ctl->tmem_full[par], 3);
        ++seq;
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    TileFeed<2> feed(&ctl->sched, abort_flag);
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 64;  // 0..127
    const uint32_t tmem_free_leader0 = map_to_cta(smem_u32(&ctl->tmem_free[0]), 0);
    // 16-bit outputs with per-expert output maps leave through shared memory and TMA stores
    const bool staged = p.group_maps != nullptr && p.dtype_out != MOE_F32;
    const bool is_bf16 = p.dtype_out == MOE_BF16;
    uint32_t seq = 0, chunk_it = 0;
    int last_e = -1;
    while (true) {
      const int tile = feed.take_warp(lane);
      if (named_barrier_any(2, 128, tile < 0)) break;  // the four warps leave together
      const PairTile t = decode(tile);
      const uint32_t par = seq & 1;
      const uint32_t full_ph = (seq >> 1) & 1;
      const int n = t.n0 + (int)rank * 128 + quarter * 32 + lane;  // this thread's weight row = output column
      const bool n_ok = n < p.N;
      const CUtensorMap* my = staged ? p.group_maps + (size_t)GM_OUT * p.E + t.e : nullptr;
      if (staged && epi_tid == 0 && t.e != last_e) { tensormap_acquire(my); last_e = t.e; }
      if (named_barrier_any(2, 128, !mbar_wait_cluster(&ctl->tmem_full[par], full_ph, abort_flag, PW_TMEM_FULL))) break;
      tc_fence_after_sync();
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);

      // n_cols accumulator columns from TMEM column `col` on are the tokens tok0, tok0 + 1, ...
      auto drain = [&](int col, int n_cols, int tok0) {
        const uint32_t taddr = lane_base + (uint32_t)col;
        if constexpr (GATE_UP) {
          // (the host only launches this form with per-expert output maps and a 16-bit output)
          pair_store_tile_gate_up(staging, chunk_it, taddr, n_cols, quarter, lane, epi_tid, is_bf16, my,
                                  t.n0 + (int)rank * 64, tok0, p.N);
        } else if (staged) {
          pair_store_tile_staged(staging, chunk_it, taddr, n_cols, quarter, lane, epi_tid, is_bf16, my,
                                 t.n0 + (int)rank * 128, tok0, p.N);
        } else {
#pragma unroll 1
          for (int c = 0; c < n_cols; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c, v);
            tmem_ld_wait();
            if (n_ok) {
              const int64_t base = (int64_t)(tok0 + c) * p.N + n;
              const int valid = min(32, t.t_end - (tok0 + c));  // tokens of this chunk that belong to the expert
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
      };
      // this warp has finished reading region r
      auto release = [&](int r) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tmem_free_leader0 + r * 8);
      };
      // The tile's columns as up to three segments (first TMEM column, columns, first token, region),
      // contested regions first: the next tile's MMAs wait for them.  One loop, so that the drain code
      // exists once (several inlined copies made the kernel miss in the instruction cache).
      constexpr int SPLIT = PAIR_TOKENS - PAIR_TAIL;
      const uint32_t regs = pair_regions(par, t.n_main, t.n_tail);
#pragma unroll 1
      for (int i = 0; i < 3; ++i) {
        int col, n_cols, tok, reg;
        if (par == 0) {
          if (i == 0)      { col = PAIR_TOKENS; n_cols = t.n_tail;                 tok = t.t0 + PAIR_TOKENS; reg = REG_RB; }
          else if (i == 1) { col = SPLIT;       n_cols = max(t.n_main - SPLIT, 0); tok = t.t0 + SPLIT;       reg = REG_RA; }
          else             { col = 0;           n_cols = min(t.n_main, SPLIT);     tok = t.t0;               reg = REG_E0; }
        } else {
          if (i == 0)      { col = SPLIT;                   n_cols = t.n_tail;                     tok = t.t0 + PAIR_TOKENS; reg = REG_RA; }
          else if (i == 1) { col = PAIR_TOKENS;             n_cols = min(t.n_main, PAIR_TAIL);     tok = t.t0;               reg = REG_RB; }
          else             { col = PAIR_TOKENS + PAIR_TAIL; n_cols = max(t.n_main - PAIR_TAIL, 0); tok = t.t0 + PAIR_TAIL;   reg = REG_E1; }
        }
        if (!(regs & (1u << reg))) continue;  // the tile does not write this region
        drain(col, n_cols, tok);
        release(reg);
      }
      ++seq;
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
