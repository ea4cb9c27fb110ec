// Tensor-core grouped GEMMs for sm_100a: tcgen05.mma with fp32 accumulators in TMEM,
// operands staged by TMA into 128-byte-swizzled shared memory, warp-specialised
// persistent CTAs (one per SM) that walk a tile list derived on the device from m_sizes.
//
//   tc_fwd_kernel<BN, false> : y[m,n] = sum_k x[m,k] w[e,n,k]   (B operand K-major)
//   tc_fwd_kernel<BN, true>  : y[m,n] = sum_k x[m,k] w[e,k,n]   (B operand MN-major; dX)
//   dw_kernel (tc_gemm_dw.cuh): w[e,n,k] = sum_m y[m,n] x[m,k]   (both operands MN-major)
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (TMEM -> registers -> global).  The accumulator is double
// buffered in TMEM so the epilogue of tile i overlaps the main loop of tile i+1.
// No tile ever crosses an expert boundary on the store side: an M tile starts at a group's
// first row and rows past the group's end are computed but not stored.
#include <cstdio>
#include <mutex>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "tc_common.cuh"

namespace moe {
namespace tc {

constexpr int BM = 128;          // rows of the accumulator tile (UMMA M)
constexpr int BK = 64;           // 16-bit elements per 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int MAX_E = 1024;      // group tables live in shared memory
constexpr int SMEM_LIMIT = 232448;  // 227 KB opt-in maximum per CTA
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB

struct GemmParams {
  const void* m_sizes;
  const void* a;   // activations (forward / dX) or x (dW), as passed by the caller
  const void* b;   // weights (forward / dX) or dy (dW)
  void* out;
  int64_t M;
  int N, K, E;
  int ms64;
  int dtype_out;  // MOE_F32 / MOE_BF16 / MOE_F16
  uint32_t idesc;
  const CUtensorMap* group_maps;  // per-expert tensor maps in workspace ([slot][expert]), or null
  const int* weight_index = nullptr;  // weight slice of each group (null: group e uses slice e)
  int* tile_counter = nullptr;  // work items are drawn from this counter (zeroed by build_group_maps_kernel); null: round-robin
  int stages = 0;               // CTA-pair forward / dX: depth of the operand ring
  int small_maps = 0;           // CTA-pair forward / dX: per-expert maps with the small token box exist (slot GM_IN_SMALL)
  const int* row_index = nullptr;  // gathered forms: sorted row r reads row row_index[r] / index_div of the token tensor
  int index_div = 1;
  int64_t x_rows = 0;           // gathered forms: rows of the token tensor
};

struct Control {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int total_m_tiles;
  int pad;
};

enum WaitCode { W_EMPTY = 1, W_FULL = 2, W_TMEM_EMPTY = 3, W_TMEM_FULL = 4 };

// Fills row_start[0..E] (first row of each group, saturated at M) and mt_start[0..E]
// (number of tile_rows-row tiles before each group).  With `tail` > 0 the last tile of a group
// may hold up to tile_rows + tail rows.  Called by every thread of the CTA.
__device__ void build_group_tables(const void* m_sizes, int ms64, int E, int64_t M, int tile_rows,
                                   int* row_start, int* mt_start, int tail = 0) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int64_t v = load_index(m_sizes, ms64, e);
    v = v < 0 ? 0 : (v > M ? M : v);
    row_start[e + 1] = (int)v;  // raw size for now
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int64_t carry_rows = 0;
    int carry_tiles = 0;
    if (lane == 0) { row_start[0] = 0; mt_start[0] = 0; }
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int64_t v = e < E ? row_start[e + 1] : 0;
      int64_t incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int64_t o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      int64_t end = carry_rows + incl;
      int64_t begin = end - v;
      end = end > M ? M : end;
      begin = begin > M ? M : begin;
      const int64_t rows = end - begin;
      const int tiles = rows <= 0 ? 0 : (rows <= tail ? 1 : (int)((rows - tail + tile_rows - 1) / tile_rows));
      int tincl = tiles;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, tincl, d);
        if (lane >= d) tincl += o;
      }
      if (e < E) {
        row_start[e + 1] = (int)end;
        mt_start[e + 1] = carry_tiles + tincl;
      }
      carry_rows += __shfl_sync(0xffffffffu, incl, 31);
      carry_tiles += __shfl_sync(0xffffffffu, tincl, 31);
    }
  }
  __syncthreads();
}

// Largest e with table[e] <= q (table is non-decreasing, table[0] = 0, q < table[E]).
__device__ __forceinline__ int find_group(const int* table, int E, int q) {
  int lo = 0, hi = E;  // invariant: table[lo] <= q < table[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (table[mid] <= q) lo = mid; else hi = mid;
  }
  return lo;
}

template <typename T>
__device__ __forceinline__ void store_row_chunk(T* dst, const uint32_t (&acc)[32], int ncols, bool vec);

template <>
__device__ __forceinline__ void store_row_chunk<float>(float* dst, const uint32_t (&acc)[32], int ncols, bool vec) {
  if (vec && ncols == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols) dst[i] = __uint_as_float(acc[i]);
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T>
__device__ __forceinline__ void store_row_chunk16(T* dst, const uint32_t (&acc)[32], int ncols, bool vec) {
  if (vec && ncols == 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 v;
      v.x = pack2<T>(__uint_as_float(acc[8 * i + 0]), __uint_as_float(acc[8 * i + 1]));
      v.y = pack2<T>(__uint_as_float(acc[8 * i + 2]), __uint_as_float(acc[8 * i + 3]));
      v.z = pack2<T>(__uint_as_float(acc[8 * i + 4]), __uint_as_float(acc[8 * i + 5]));
      v.w = pack2<T>(__uint_as_float(acc[8 * i + 6]), __uint_as_float(acc[8 * i + 7]));
      reinterpret_cast<uint4*>(dst)[i] = v;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols) dst[i] = from_f32<T>(__uint_as_float(acc[i]));
  }
}
template <>
__device__ __forceinline__ void store_row_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&acc)[32], int ncols, bool vec) {
  store_row_chunk16(dst, acc, ncols, vec);
}
template <>
__device__ __forceinline__ void store_row_chunk<__half>(__half* dst, const uint32_t (&acc)[32], int ncols, bool vec) {
  store_row_chunk16(dst, acc, ncols, vec);
}

// Writes 32 accumulator columns of one output row.  `dst_elem` is the element offset of the
// first column in the output tensor.
__device__ __forceinline__ void store_acc(void* out, int dtype_out, int64_t dst_elem, const uint32_t (&acc)[32], int ncols, bool vec) {
  if (dtype_out == MOE_BF16) store_row_chunk((__nv_bfloat16*)out + dst_elem, acc, ncols, vec);
  else if (dtype_out == MOE_F16) store_row_chunk((__half*)out + dst_elem, acc, ncols, vec);
  else store_row_chunk((float*)out + dst_elem, acc, ncols, vec);
}

// ---------------------------------------------------------------------------------------
// Forward / dX
// ---------------------------------------------------------------------------------------
template <int BN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_fwd_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
              const GemmParams p) {
  constexpr int B_CHUNKS = (BN + 63) / 64;  // 64-wide chunks of an MN-major B tile
  constexpr int B_STAGE_BYTES = B_MN ? B_CHUNKS * BK * 128 : (BN < 8 ? 8 : BN) * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + ((B_STAGE_BYTES + 1023) & ~1023);
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  constexpr int ACC_STRIDE = BN < 32 ? 32 : BN;  // TMEM columns between the two accumulators
  constexpr uint32_t TMEM_COLS = 2 * ACC_STRIDE;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES);
  int* row_start = reinterpret_cast<int*>(ctl + 1);
  int* mt_start = row_start + (p.E + 1);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 4); }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, BM, row_start, mt_start);  // contains __syncthreads
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int64_t total_tiles = (int64_t)mt_start[p.E] * n_tiles;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int q = (int)(tile / n_tiles);
        const int e = find_group(mt_start, p.E, q);
        const int mt_e = mt_start[e + 1] - mt_start[e];
        const int j = (int)(tile - (int64_t)mt_start[e] * n_tiles);
        const int m0 = row_start[e] + (j % mt_e) * BM;
        const int n0 = (j / mt_e) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, W_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&ctl->full[s], A_STAGE_BYTES + B_STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &ctl->full[s], kb * BK, m0);
          if constexpr (!B_MN) {
            tma_load_3d(sb, &tmap_b, &ctl->full[s], kb * BK, n0, e);
          } else {
#pragma unroll
            for (int c = 0; c < B_CHUNKS; ++c)
              tma_load_3d(sb + c * (BK * 128), &tmap_b, &ctl->full[s], n0 + c * 64, kb * BK, e);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++acc_it) {
        const uint32_t acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&ctl->tmem_empty[acc], acc_ph ^ 1, abort_flag, W_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, W_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint64_t da = make_smem_desc(sa, 16, 1024);
          const uint64_t db = B_MN ? make_smem_desc(sb, BK * 128, 1024) : make_smem_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 elements = 32 bytes inside the swizzle row; MN-major: 16 rows of 128 B.
            const uint64_t a_adv = (uint64_t)((k * UMMA_K * 2) >> 4);
            const uint64_t b_adv = B_MN ? (uint64_t)((k * UMMA_K * 128) >> 4) : a_adv;
            umma_f16(d_tmem, da + a_adv, db + b_adv, p.idesc, (kb | k) != 0);
          }
          umma_commit(&ctl->empty[s]);  // frees the stage when these MMAs have read it
        }
        if (ok) umma_commit(&ctl->tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, +32)
    const int row_in_tile = quarter * 32 + lane;
    const bool vec = ((p.N * (int)dtype_size(p.dtype_out)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    uint32_t acc_it = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++acc_it) {
      const int q = (int)(tile / n_tiles);
      const int e = find_group(mt_start, p.E, q);
      const int mt_e = mt_start[e + 1] - mt_start[e];
      const int j = (int)(tile - (int64_t)mt_start[e] * n_tiles);
      const int m0 = row_start[e] + (j % mt_e) * BM;
      const int n0 = (j / mt_e) * BN;
      const int64_t grow = (int64_t)m0 + row_in_tile;
      const bool row_ok = grow < row_start[e + 1] && grow < p.M;
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag, W_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= p.N) break;  // warp-uniform
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        if (row_ok) {
          const int ncols = min(32, p.N - (n0 + c));
          store_acc(p.out, p.dtype_out, grow * p.N + n0 + c, v, ncols, vec);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->tmem_empty[acc]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// Forward with the NF4 weight decoded into the B stage.
// Per k-block the producer brings the activation tile (TMA, swizzled) and the packed
// weight bytes of the 256 x 64 weight tile (TMA, 8 KB, linear) into shared memory; eight
// decode warps turn the bytes into the swizzled 16-bit K-major B tile (one weight row per
// thread: 32 packed bytes -> 64 values -> eight 16-byte chunks), publish it to the async
// proxy and signal the MMA warp.  HBM sees 0.5 byte + 4/blocksize bytes per weight.
// Extra warps: 6..13 = decode.
// ---------------------------------------------------------------------------------------
constexpr int NF4_THREADS = 448;
constexpr int NF4_BN = 256;
constexpr int NF4_STAGES = 3;
constexpr int NF4_PACKED_BYTES = NF4_BN * (BK / 2);                               // 8 KB
constexpr int NF4_STAGE_BYTES = A_STAGE_BYTES + NF4_BN * BK * 2 + NF4_PACKED_BYTES;  // 56 KB

struct Nf4Params {
  const float* code;
  const float* absmax;
  int shift;  // log2(blocksize), blocksize >= 64
};

struct Nf4Control {
  uint64_t ready[8];  // decoded B tile published (8 warp arrivals)
  float2 lut[256];    // byte -> (code[hi nibble], code[lo nibble])
};

template <bool IS_BF16>
__global__ void __launch_bounds__(NF4_THREADS, 1)
tc_fwd_nf4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_q,
                  const GemmParams p, const Nf4Params q) {
  constexpr int BN = NF4_BN;
  constexpr int STAGES = NF4_STAGES;
  constexpr int STAGE_BYTES = NF4_STAGE_BYTES;
  constexpr int B_OFF = A_STAGE_BYTES;
  constexpr int Q_OFF = A_STAGE_BYTES + BN * BK * 2;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Control* ctl = reinterpret_cast<Control*>(smem + STAGES * STAGE_BYTES);
  Nf4Control* nctl = reinterpret_cast<Nf4Control*>(ctl + 1);
  int* row_start = reinterpret_cast<int*>(nctl + 1);
  int* mt_start = row_start + (p.E + 1);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
      mbar_init(&nctl->ready[s], 8);
    }
    for (int a = 0; a < 2; ++a) { mbar_init(&ctl->tmem_full[a], 1); mbar_init(&ctl->tmem_empty[a], 4); }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_q);
  }
  if (threadIdx.x < 256) nctl->lut[threadIdx.x] = make_float2(q.code[threadIdx.x >> 4], q.code[threadIdx.x & 15]);
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  build_group_tables(p.m_sizes, p.ms64, p.E, p.M, BM, row_start, mt_start);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  const int n_tiles = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int64_t total_tiles = (int64_t)mt_start[p.E] * n_tiles;

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int qd = (int)(tile / n_tiles);
        const int e = find_group(mt_start, p.E, qd);
        const int mt_e = mt_start[e + 1] - mt_start[e];
        const int j = (int)(tile - (int64_t)mt_start[e] * n_tiles);
        const int m0 = row_start[e] + (j % mt_e) * BM;
        const int n0 = (j / mt_e) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, W_EMPTY)) { ok = false; break; }
          uint8_t* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&ctl->full[s], A_STAGE_BYTES + NF4_PACKED_BYTES);
          tma_load_2d(st, &tmap_a, &ctl->full[s], kb * BK, m0);
          tma_load_3d(st + Q_OFF, &tmap_q, &ctl->full[s], kb * (BK / 2), n0, e);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++acc_it) {
        const uint32_t acc = acc_it & 1;
        const uint32_t acc_ph = (acc_it >> 1) & 1;
        if (!mbar_wait(&ctl->tmem_empty[acc], acc_ph ^ 1, abort_flag, W_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, W_FULL)) { ok = false; break; }
          if (!mbar_wait(&nctl->ready[s], ph, abort_flag, W_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa, 16, 1024);
          const uint64_t db = make_smem_desc(sa + B_OFF, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
            umma_f16(d_tmem, da + adv, db + adv, p.idesc, (kb | k) != 0);
          }
          umma_commit(&ctl->empty[s]);
        }
        if (ok) umma_commit(&ctl->tmem_full[acc]);
      }
    }
  } else if (warp < 6) {
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const bool vec = ((p.N * (int)dtype_size(p.dtype_out)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    uint32_t acc_it = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++acc_it) {
      const int qd = (int)(tile / n_tiles);
      const int e = find_group(mt_start, p.E, qd);
      const int mt_e = mt_start[e + 1] - mt_start[e];
      const int j = (int)(tile - (int64_t)mt_start[e] * n_tiles);
      const int m0 = row_start[e] + (j % mt_e) * BM;
      const int n0 = (j / mt_e) * BN;
      const int64_t grow = (int64_t)m0 + row_in_tile;
      const bool row_ok = grow < row_start[e + 1] && grow < p.M;
      const uint32_t acc = acc_it & 1;
      const uint32_t acc_ph = (acc_it >> 1) & 1;
      if (!mbar_wait(&ctl->tmem_full[acc], acc_ph, abort_flag, W_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (n0 + c >= p.N) break;
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        if (row_ok) store_acc(p.out, p.dtype_out, grow * p.N + n0 + c, v, min(32, p.N - (n0 + c)), vec);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->tmem_empty[acc]);
    }
  } else {
    // ------------------------------ decode warps ------------------------------
    const int t = threadIdx.x - 6 * 32;  // weight row inside the tile, 0..255
    uint32_t it = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int qd = (int)(tile / n_tiles);
      const int e = find_group(mt_start, p.E, qd);
      const int mt_e = mt_start[e + 1] - mt_start[e];
      const int j = (int)(tile - (int64_t)mt_start[e] * n_tiles);
      const int n0 = (j / mt_e) * BN;
      const int n = n0 + t;
      const bool n_ok = n < p.N;
      const int64_t row_flat = ((int64_t)e * p.N + (n_ok ? n : 0)) * p.K;
      float am_next = n_ok ? __ldg(q.absmax + (row_flat >> q.shift)) : 0.f;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const float am = am_next;
        if (kb + 1 < k_blocks && n_ok) am_next = __ldg(q.absmax + ((row_flat + (int64_t)(kb + 1) * BK) >> q.shift));
        if (!mbar_wait(&ctl->full[s], ph, abort_flag, W_FULL)) { ok = false; break; }
        uint8_t* st = smem + s * STAGE_BYTES;
        const uint4* src = reinterpret_cast<const uint4*>(st + Q_OFF + t * (BK / 2));
        uint8_t* dst_row = st + B_OFF + t * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 raw = src[h];
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {  // 4 bytes -> 8 values -> one 16-byte chunk
            uint32_t outw[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const float2 c = nctl->lut[(words[w] >> (8 * b)) & 0xffu];
              if constexpr (IS_BF16) outw[b] = pack2<__nv_bfloat16>(c.x * am, c.y * am);
              else outw[b] = pack2<__half>(c.x * am, c.y * am);
            }
            const int chunk = h * 4 + w;
            *reinterpret_cast<uint4*>(dst_row + ((chunk ^ (t & 7)) << 4)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&nctl->ready[s]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace tc
}  // namespace moe

#include "tc_gemm_pair.cuh"
#include "tc_gemm_dw.cuh"
#include "tc_gemm_nf4.cuh"

namespace moe {
namespace tc {

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    if (qres != cudaDriverEntryPointSuccess) return nullptr;
    return (EncodeTiledFn)ptr;
  }();
  return fn;
}

// Tensor map over a dense 16-bit tensor viewed as (d2, d1, d0) with d0 contiguous.
// Box = (b0 = 64 elements, b1 rows, 1).  rank 2 when d2 == 0.
thread_local char g_detail[320] = "";

static int make_map(CUtensorMap* map, int dtype, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                    uint32_t b1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return MOE_ERR_DEVICE;
  const CUtensorMapDataType dt = dtype == MOE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint32_t rank = d2 ? 3 : 2;
  cuuint64_t dims[3] = {d0, d1, d2 ? d2 : 1};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {64, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, dt, rank, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    snprintf(g_detail, sizeof(g_detail), "cuTensorMapEncodeTiled -> %d: base=%p dims=(%llu,%llu,%llu) box=(64,%u,1) rank=%u",
             (int)r, base, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, b1, rank);
  return r == CUDA_SUCCESS ? MOE_OK : MOE_ERR_UNSUPPORTED;
}

template <int BN>
static constexpr int smem_bytes_for(int E, int tables) {
  // upper bound that covers both the K-major and the MN-major B stage of tc_fwd_kernel<BN, *>
  return ((BN == 256) ? 4 : 6) * (A_STAGE_BYTES + (BN < 64 ? 64 : BN) * BK * 2) + (int)sizeof(Control) + tables * (E + 1) * 4 + 1024;
}

// Per-kernel, per-device memo of launch set-up that does not change between calls: a call of a thin
// (LoRA-sized) GEMM would otherwise spend more host time on attribute and occupancy queries than the
// kernel runs.  Entries are keyed by the kernel's address (template instantiations share their
// function-pointer TYPE, so the key cannot be the type).
struct LaunchMemo {
  const void* kernel;
  int device;
  int smem_granted;     // largest dynamic shared-memory limit set so far
  int pairs_smem;       // shared-memory size of the memoised occupancy answer (0: none)
  int pairs;
};
constexpr int MEMO_SLOTS = 96;
static LaunchMemo g_memo[MEMO_SLOTS];
static int g_memo_used = 0;
static std::mutex g_memo_lock;

// Entry of (kernel, current device), created on first use; nullptr when the table is full (callers then
// simply repeat the query).  Call with g_memo_lock held.
static LaunchMemo* memo_entry(const void* kernel) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  for (int i = 0; i < g_memo_used; ++i)
    if (g_memo[i].kernel == kernel && g_memo[i].device == dev) return &g_memo[i];
  if (g_memo_used == MEMO_SLOTS) return nullptr;
  g_memo[g_memo_used] = LaunchMemo{kernel, dev, 0, 0, 0};
  return &g_memo[g_memo_used++];
}

// Raises the kernel's dynamic shared-memory limit to at least `bytes` (once per kernel, device and size).
template <typename K>
static int set_smem(K kernel, int bytes) {
  std::lock_guard<std::mutex> guard(g_memo_lock);
  LaunchMemo* m = memo_entry(reinterpret_cast<const void*>(kernel));
  if (m != nullptr && m->smem_granted >= bytes) return MOE_OK;
  const int st = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (st == MOE_OK && m != nullptr) m->smem_granted = bytes;
  return st;
}

}  // namespace tc

// Shapes the tensor-core kernels accept.  N, K are the output columns / contraction
// length of the call (for dW: rows / columns of one expert's weight).
bool tc_eligible(int which, const void* a, const void* b, const void* out, int64_t M, int N, int K, int E,
                 int dtype_in, int dtype_out) {
  if (dtype_in != MOE_BF16 && dtype_in != MOE_F16) return false;
  if (!is_float_dtype(dtype_out)) return false;
  if (E < 1 || E > tc::MAX_E || M < 1 || M > 0x7fffffffLL - 1024) return false;
  if (N < 8 || K < 8 || (N % 8) || (K % 8)) return false;  // 16-byte row pitches; thin (LoRA) shapes included
  if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)out & 3)) return false;
  (void)which;
  return true;
}

// The driver's tensor-map encoder needs a current context on the calling thread; threads
// that have not yet issued a runtime call of this library (autograd worker threads) get the
// primary context bound here, once per thread and device.
static void bind_context_once() {
  thread_local int bound = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  if (bound != dev) {
    cudaFree(nullptr);
    bound = dev;
  }
}

// Number of CTA pairs that can be resident at once (persistent grid = 2 x this).
template <typename Kern>
static int resident_pairs(Kern kernel, int smem_bytes, int threads = 192) {
  {
    std::lock_guard<std::mutex> guard(tc::g_memo_lock);
    tc::LaunchMemo* m = tc::memo_entry(reinterpret_cast<const void*>(kernel));
    if (m != nullptr && m->pairs_smem == smem_bytes && m->pairs > 0) return m->pairs;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count());
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = sm_count() / 2;
  }
  const int cap = sm_count() / 2;
  n = n < cap ? n : cap;
  {
    std::lock_guard<std::mutex> guard(tc::g_memo_lock);
    tc::LaunchMemo* m = tc::memo_entry(reinterpret_cast<const void*>(kernel));
    if (m != nullptr) { m->pairs_smem = smem_bytes; m->pairs = n; }
  }
  return n;
}

template <typename... KArgs, typename... Args>
static int launch_pair(void (*kernel)(KArgs...), int grid, int smem_bytes, cudaStream_t stream, Args... args);
template <typename... KArgs, typename... Args>
static int launch_pair_threads(void (*kernel)(KArgs...), int grid, int threads, int smem_bytes, cudaStream_t stream, Args... args);

// Workspace of the tensor-core grouped GEMMs: GroupMapTemplates::MAX per-expert tensor maps per expert
// (slot-major, 128 bytes each), then the work-item counter of the launch.
static size_t ws_maps_bytes(int E) { return (size_t)tc::GroupMapTemplates::MAX * (size_t)E * sizeof(CUtensorMap); }
size_t tc_workspace_bytes(int E) { return E > 0 ? ws_maps_bytes(E) + 128 : 0; }
static bool ws_usable(const void* ws, size_t ws_bytes, int E) {
  return ws != nullptr && (((uintptr_t)ws & 127) == 0) && ws_bytes >= tc_workspace_bytes(E);
}
static int* ws_counter(void* ws, int E) { return reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ws) + ws_maps_bytes(E)); }

// Shared-memory footprint of the CTA-pair forward / dX kernels with `stages` ring slots.
static int pair_smem_bytes(int stages, int E) {
  using namespace tc;
  return stages * PAIR_STAGE_BYTES + 4 * PAIR_STAGING_BYTES + (int)sizeof(PairControl) + 2 * (E + 1) * 4 + 1024;
}
// Deepest ring that fits (0: none does).
static int pair_stages(int E) {
  for (int st = tc::PAIR_MAX_STAGES; st >= 3; --st)
    if (pair_smem_bytes(st, E) <= tc::SMEM_LIMIT) return st;
  return 0;
}

// Launches build_group_maps_kernel for the forward / dX / gate-up kernels: per-expert copies of the
// token maps (128-row and small box) and, for 16-bit outputs, of the output map.
static int build_pair_maps(tc::GemmParams& p, const CUtensorMap& mx, const void* a, void* out, int dtype_in, int dtype_out,
                           void* ws, cudaStream_t stream, const uint64_t* out_ptrs, bool gather = false) {
  using namespace tc;
  GroupMapTemplates tm;
  int st;
  tm.mask = 0;
  if (!gather) {  // (gathered token rows are addressed by index: no per-expert token maps)
    tm.mask = (1 << GM_IN) | (1 << GM_IN_SMALL);
    tm.t[GM_IN] = mx;
    if ((st = make_map(&tm.t[GM_IN_SMALL], dtype_in, a, (uint64_t)p.K, (uint64_t)p.M, 0, PAIR_SMALL_BOX)) != MOE_OK) return st;
  }
  if (dtype_out != MOE_F32) {
    tm.mask |= 1 << GM_OUT;
    if ((st = make_map(&tm.t[GM_OUT], dtype_out, out, (uint64_t)p.N, (uint64_t)p.M, 0, 32)) != MOE_OK) return st;
  }
  const int gm_smem = 8 * 128 + 2 * (p.E + 1) * 4 + 128;
  build_group_maps_kernel<<<(p.E + 7) / 8, 256, gm_smem, stream>>>(tm, p.m_sizes, p.ms64, p.E, p.M, reinterpret_cast<CUtensorMap*>(ws),
                                                                   ws_counter(ws, p.E), out_ptrs, GM_OUT, (int64_t)p.N * 2);
  if ((st = launch_status()) != MOE_OK) return st;
  p.group_maps = reinterpret_cast<const CUtensorMap*>(ws);
  p.tile_counter = ws_counter(ws, p.E);
  p.small_maps = gather ? 0 : 1;
  return MOE_OK;
}

// `weight_index` / `n_weights` / `out_ptrs` (all optional) describe the scattered form: group e
// multiplies by weight slice weight_index[e] of n_weights, and its output rows start at the
// address out_ptrs[e] instead of row row_start[e] of `out`.
static int pair_grouped_gemm(int which, const void* a, const void* b, const void* m_sizes, int ms64, void* out,
                             int64_t M, int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes,
                             cudaStream_t stream, const int* weight_index = nullptr, int n_weights = 0,
                             const uint64_t* out_ptrs = nullptr, const int* row_index = nullptr, int index_div = 1,
                             int64_t x_rows = 0) {
  using namespace tc;
  if (which != 0 && which != 1) return MOE_ERR_UNSUPPORTED;
  const bool gather = row_index != nullptr;
  if (gather && (which != 0 || index_div <= 0 || x_rows <= 0 || x_rows > 0x7fffffffLL)) return MOE_ERR_UNSUPPORTED;
  if (n_weights <= 0) n_weights = E;
  GemmParams p;
  p.row_index = row_index; p.index_div = index_div; p.x_rows = x_rows;
  p.weight_index = weight_index;
  p.a = a; p.b = b;
  p.m_sizes = m_sizes; p.out = out; p.M = M; p.N = N; p.K = K; p.E = E; p.ms64 = ms64; p.dtype_out = dtype_out;
  const int fmt = dtype_in == MOE_BF16 ? 1 : 0;
  p.group_maps = nullptr;
  // tile ids are 32-bit
  if (((M + PAIR_TOKENS - 1) / PAIR_TOKENS + E) * (int64_t)((N + 255) / 256) >= (int64_t)1 << 30) return MOE_ERR_UNSUPPORTED;
  CUtensorMap mw, mx;
  int st;
  // A = weight (accumulator rows), B = activations (accumulator columns = tokens)
  if (which == 0) st = make_map(&mw, dtype_in, b, (uint64_t)K, (uint64_t)N, (uint64_t)n_weights, 128);
  else st = make_map(&mw, dtype_in, b, (uint64_t)N, (uint64_t)K, (uint64_t)n_weights, BK);
  if (st != MOE_OK) return st;
  // token map: 128-row boxes over the M sorted rows, or one-row boxes (for gather4) over the x_rows token rows
  if (gather) st = make_map(&mx, dtype_in, a, (uint64_t)K, (uint64_t)x_rows, 0, 1);
  else st = make_map(&mx, dtype_in, a, (uint64_t)K, (uint64_t)M, 0, 128);
  if (st != MOE_OK) return st;
  p.idesc = make_idesc(fmt, which == 1, 0, 256, 0);  // N field is filled per tile
  // Per-expert copies of the token and output maps (row extent = the group's last row): partial
  // tiles then load no rows of the next expert, and 16-bit outputs can leave through TMA stores.
  if (ws_usable(ws, ws_bytes, E) && (((uintptr_t)out & 15) == 0 || dtype_out == MOE_F32)) {
    if ((st = build_pair_maps(p, mx, a, out, dtype_in, dtype_out, ws, stream, out_ptrs, gather)) != MOE_OK) return st;
  }
  if (gather && p.group_maps == nullptr) return MOE_ERR_WORKSPACE;
  // scattered outputs exist only as per-group output maps
  if (out_ptrs != nullptr && (p.group_maps == nullptr || dtype_out == MOE_F32)) return MOE_ERR_UNSUPPORTED;
  p.stages = pair_stages(E);
  if (p.stages == 0) return MOE_ERR_UNSUPPORTED;
  const int bytes = pair_smem_bytes(p.stages, E);
  if (gather) {
    auto kern = pair_fwd_kernel<false, false, true>;
    if ((st = set_smem(kern, bytes)) != MOE_OK) return st;
    const int grid = 2 * resident_pairs(kern, bytes);
    kern<<<grid, PAIR_THREADS, bytes, stream>>>(mw, mx, p, mw);
  } else if (which == 0) {
    if ((st = set_smem(pair_fwd_kernel<false>, bytes)) != MOE_OK) return st;
    const int grid = 2 * resident_pairs(pair_fwd_kernel<false>, bytes);
    pair_fwd_kernel<false><<<grid, PAIR_THREADS, bytes, stream>>>(mw, mx, p, mw);
  } else {
    if ((st = set_smem(pair_fwd_kernel<true>, bytes)) != MOE_OK) return st;
    const int grid = 2 * resident_pairs(pair_fwd_kernel<true>, bytes);
    pair_fwd_kernel<true><<<grid, PAIR_THREADS, bytes, stream>>>(mw, mx, p, mw);
  }
  return launch_status();
}

// Launch with a cluster of 2 CTAs.
template <typename... KArgs, typename... Args>
static int launch_pair(void (*kernel)(KArgs...), int grid, int smem_bytes, cudaStream_t stream, Args... args) {
  return launch_pair_threads(kernel, grid, 192, smem_bytes, stream, args...);
}

template <typename... KArgs, typename... Args>
static int launch_pair_threads(void (*kernel)(KArgs...), int grid, int threads, int smem_bytes, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&cfg, kernel, args...));
}

// dW on tensor cores: per-expert maps are built into `ws`, then one GEMM launch.
static int dw_grouped_gemm(const void* x, const void* dy, const void* m_sizes, int ms64, void* out, int64_t M, int N,
                           int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, cudaStream_t stream,
                           bool single_cta) {
  using namespace tc;
  if (!ws_usable(ws, ws_bytes, E)) return MOE_ERR_WORKSPACE;
  GemmParams p;
  p.m_sizes = m_sizes; p.out = out; p.M = M; p.N = N; p.K = K; p.E = E; p.ms64 = ms64; p.dtype_out = dtype_out;
  p.group_maps = reinterpret_cast<const CUtensorMap*>(ws);
  p.tile_counter = ws_counter(ws, E);
  if ((int64_t)E * ((N + 127) / 128) * (int64_t)((K + 127) / 128) >= (int64_t)1 << 30) return MOE_ERR_UNSUPPORTED;  // 32-bit work-item ids
  const int fmt = dtype_in == MOE_BF16 ? 1 : 0;
  int st;
  GroupMapTemplates tm;
  tm.mask = (1 << GM_DY) | (1 << GM_X);
  if ((st = make_map(&tm.t[GM_DY], dtype_in, dy, (uint64_t)N, (uint64_t)M, 0, BK)) != MOE_OK) return st;
  if ((st = make_map(&tm.t[GM_X], dtype_in, x, (uint64_t)K, (uint64_t)M, 0, BK)) != MOE_OK) return st;
  const int gm_smem = 8 * 128 + 2 * (E + 1) * 4 + 128;
  build_group_maps_kernel<<<(E + 7) / 8, 256, gm_smem, stream>>>(tm, m_sizes, ms64, E, M, reinterpret_cast<CUtensorMap*>(ws),
                                                                 ws_counter(ws, E));
  if ((st = launch_status()) != MOE_OK) return st;

  const bool staged = dtype_out != MOE_F32;
  CUtensorMap mo;
  if (staged) {
    if ((st = make_map(&mo, dtype_out, out, (uint64_t)K, (uint64_t)N, (uint64_t)E, 128)) != MOE_OK) return st;
  } else {
    memset(&mo, 0, sizeof(mo));
  }
  const int tables = 2 * (E + 1) * 4 + (int)sizeof(DwControl) + 1024 + 2 * 128 * 128;
  const bool pair = !single_cta && staged && N >= 192 && K >= 192 && (((uintptr_t)out & 15) == 0);
  if (pair) {
    constexpr int ST = 5;
    const int bytes = ST * 4 * BK * 128 + tables;
    if (bytes > SMEM_LIMIT) return MOE_ERR_UNSUPPORTED;
    p.idesc = make_idesc(fmt, 1, 1, 256, 256);
    auto kern = dw_kernel<true, 256, ST>;
    if ((st = set_smem(kern, bytes)) != MOE_OK) return st;
    return launch_pair(kern, 2 * resident_pairs(kern, bytes), bytes, stream, mo, p);
  }
  if (K > 128) {
    p.idesc = make_idesc(fmt, 1, 1, BM, 256);
    const int bytes4 = 4 * 6 * BK * 128 + tables;
    if (bytes4 <= SMEM_LIMIT) {
      auto kern = dw_kernel<false, 256, 4>;
      if ((st = set_smem(kern, bytes4)) != MOE_OK) return st;
      kern<<<sm_count(), 192, bytes4, stream>>>(mo, p);
    } else {
      const int bytes3 = 3 * 6 * BK * 128 + tables;
      if (bytes3 > SMEM_LIMIT) return MOE_ERR_UNSUPPORTED;
      auto kern = dw_kernel<false, 256, 3>;
      if ((st = set_smem(kern, bytes3)) != MOE_OK) return st;
      kern<<<sm_count(), 192, bytes3, stream>>>(mo, p);
    }
  } else {
    p.idesc = make_idesc(fmt, 1, 1, BM, 128);
    const int bytes = 6 * 4 * BK * 128 + tables;
    if (bytes > SMEM_LIMIT) return MOE_ERR_UNSUPPORTED;
    auto kern = dw_kernel<false, 128, 6>;
    if ((st = set_smem(kern, bytes)) != MOE_OK) return st;
    kern<<<sm_count(), 192, bytes, stream>>>(mo, p);
  }
  return launch_status();
}

// which: 0 forward, 1 dX, 2 dW (a = x, b = dy).  single_cta selects the one-CTA kernels.
int tc_grouped_gemm(int which, const void* a, const void* b, const void* m_sizes, int ms64, void* out,
                    int64_t M, int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes,
                    cudaStream_t stream, bool single_cta) {
  using namespace tc;
  bind_context_once();
  if (which == 2)
    return dw_grouped_gemm(a, b, m_sizes, ms64, out, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, stream, single_cta);
  if (!single_cta) {
    // a pair covers 256 weight rows (and, for dW, 256 weight columns): narrower problems
    // would leave most of the tile empty
    const bool pair_ok = N >= 192;
    if (pair_ok) return pair_grouped_gemm(which, a, b, m_sizes, ms64, out, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, stream);
  }
  GemmParams p;
  p.m_sizes = m_sizes; p.out = out; p.M = M; p.N = N; p.K = K; p.E = E; p.ms64 = ms64; p.dtype_out = dtype_out;
  const int fmt = dtype_in == MOE_BF16 ? 1 : 0;
  const int grid = sm_count();
  CUtensorMap ma, mb;
  int st;
  if (which == 0 || which == 1) {
    // narrowest accumulator that covers N: thin outputs (LoRA down-projections) do not pay for 128 columns
    const int bn = N > 128 ? 256 : N > 64 ? 128 : N > 32 ? 64 : N > 16 ? 32 : 16;
    if ((st = make_map(&ma, dtype_in, a, (uint64_t)K, (uint64_t)M, 0, BM)) != MOE_OK) return st;
    if (which == 0) st = make_map(&mb, dtype_in, b, (uint64_t)K, (uint64_t)N, (uint64_t)E, (uint32_t)bn);
    else st = make_map(&mb, dtype_in, b, (uint64_t)N, (uint64_t)K, (uint64_t)E, BK);
    if (st != MOE_OK) return st;
    p.idesc = make_idesc(fmt, 0, which == 1, BM, bn);
#define MOE_TC_LAUNCH(BN_, BMN_)                                                              \
  do {                                                                                        \
    const int bytes = smem_bytes_for<BN_>(E, 2);                                              \
    if (bytes > SMEM_LIMIT) return MOE_ERR_UNSUPPORTED;                                       \
    if ((st = set_smem(tc_fwd_kernel<BN_, BMN_>, bytes)) != MOE_OK) return st;                \
    tc_fwd_kernel<BN_, BMN_><<<grid, NUM_THREADS, bytes, stream>>>(ma, mb, p);                \
  } while (0)
    if (which == 0) {
      switch (bn) {
        case 256: MOE_TC_LAUNCH(256, false); break;
        case 128: MOE_TC_LAUNCH(128, false); break;
        case 64: MOE_TC_LAUNCH(64, false); break;
        case 32: MOE_TC_LAUNCH(32, false); break;
        default: MOE_TC_LAUNCH(16, false); break;
      }
    } else {
      switch (bn) {
        case 256: MOE_TC_LAUNCH(256, true); break;
        case 128: MOE_TC_LAUNCH(128, true); break;
        case 64: MOE_TC_LAUNCH(64, true); break;
        case 32: MOE_TC_LAUNCH(32, true); break;
        default: MOE_TC_LAUNCH(16, true); break;
      }
    }
#undef MOE_TC_LAUNCH
    return launch_status();
  }
  return MOE_ERR_UNSUPPORTED;
}

// h = silu(x w_gate^T) * (x w_up^T) per expert in one launch (pair_fwd_kernel<false, true>).
int tc_gate_up_silu(const void* x, const void* w_gate, const void* w_up, const void* m_sizes, int ms64, void* h,
                    int64_t M, int I, int K, int E, int dtype, void* ws, size_t ws_bytes, cudaStream_t stream,
                    const int* row_index, int index_div, int64_t x_rows) {
  using namespace tc;
  bind_context_once();
  if (!ws_usable(ws, ws_bytes, E)) return MOE_ERR_WORKSPACE;
  GemmParams p;
  p.a = x; p.b = w_gate;
  p.m_sizes = m_sizes; p.out = h; p.M = M; p.N = I; p.K = K; p.E = E; p.ms64 = ms64; p.dtype_out = dtype;
  p.idesc = make_idesc(dtype == MOE_BF16 ? 1 : 0, 0, 0, 256, 0);
  if (((M + PAIR_TOKENS - 1) / PAIR_TOKENS + E) * (int64_t)((I + 127) / 128) >= (int64_t)1 << 30) return MOE_ERR_UNSUPPORTED;
  CUtensorMap mg, mu, mx;
  int st;
  if ((st = make_map(&mg, dtype, w_gate, (uint64_t)K, (uint64_t)I, (uint64_t)E, 16)) != MOE_OK) return st;
  if ((st = make_map(&mu, dtype, w_up, (uint64_t)K, (uint64_t)I, (uint64_t)E, 16)) != MOE_OK) return st;
  const bool gather = row_index != nullptr;
  if (gather && (index_div <= 0 || x_rows <= 0 || x_rows > 0x7fffffffLL)) return MOE_ERR_SHAPE;
  p.row_index = row_index; p.index_div = index_div; p.x_rows = x_rows;
  if (gather) st = make_map(&mx, dtype, x, (uint64_t)K, (uint64_t)x_rows, 0, 1);
  else st = make_map(&mx, dtype, x, (uint64_t)K, (uint64_t)M, 0, 128);
  if (st != MOE_OK) return st;
  if ((st = build_pair_maps(p, mx, x, h, dtype, dtype, ws, stream, nullptr, gather)) != MOE_OK) return st;
  p.stages = pair_stages(E);
  if (p.stages == 0) return MOE_ERR_UNSUPPORTED;
  const int bytes = pair_smem_bytes(p.stages, E);
  if (gather) {
    auto kern = pair_fwd_kernel<false, true, true>;
    if ((st = set_smem(kern, bytes)) != MOE_OK) return st;
    kern<<<2 * resident_pairs(kern, bytes), PAIR_THREADS, bytes, stream>>>(mg, mx, p, mu);
    return launch_status();
  }
  auto kern = pair_fwd_kernel<false, true>;
  if ((st = set_smem(kern, bytes)) != MOE_OK) return st;
  const int grid = 2 * resident_pairs(kern, bytes);
  kern<<<grid, PAIR_THREADS, bytes, stream>>>(mg, mx, p, mu);
  return launch_status();
}

// Forward whose sorted row r is row row_index[r] / index_div of x (x_rows rows): CTA-pair kernel only.
int tc_grouped_gemm_gather(const void* x, int64_t x_rows, const int* row_index, int index_div, const void* w,
                           const void* m_sizes, int ms64, void* y, int64_t M, int N, int K, int E, int dtype_in,
                           int dtype_out, void* ws, size_t ws_bytes, cudaStream_t stream) {
  bind_context_once();
  if (N < 192) return MOE_ERR_UNSUPPORTED;
  return pair_grouped_gemm(0, x, w, m_sizes, ms64, y, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, stream, nullptr, 0,
                           nullptr, row_index, index_div, x_rows);
}

// Scattered forward (which = 0) / dX (which = 1) on the CTA-pair kernels: see pair_grouped_gemm.
int tc_grouped_gemm_scattered(int which, const void* a, const void* b, const void* group_sizes, int ms64,
                              const int* weight_index, int n_weights, const uint64_t* out_ptrs, void* out_template,
                              int64_t M, int N, int K, int G, int dtype_in, int dtype_out, void* ws, size_t ws_bytes,
                              cudaStream_t stream) {
  bind_context_once();
  if (which != 0 && which != 1) return MOE_ERR_UNSUPPORTED;
  return pair_grouped_gemm(which, a, b, group_sizes, ms64, out_template, M, N, K, G, dtype_in, dtype_out, ws, ws_bytes,
                           stream, weight_index, n_weights, out_ptrs);
}

bool tc_nf4_eligible(const void* x, const void* packed, const void* absmax, const void* out, int64_t M, int N, int K,
                     int E, int blocksize, int dtype_in, int dtype_out) {
  if (!tc_eligible(0, x, packed, out, M, N, K, E, dtype_in, dtype_out)) return false;
  if (blocksize < 64 || (K % 64) != 0 || N < 64) return false;  // one absmax per (row, 64-wide k-block); packed pitch % 16 B
  if ((uintptr_t)absmax & 3) return false;
  return true;
}

int tc_grouped_gemm_nf4(const void* x, const uint8_t* packed, const float* code, const float* absmax, int blocksize,
                        const void* m_sizes, int ms64, void* out, int64_t M, int N, int K, int E,
                        int dtype_in, int dtype_out, void* ws, size_t ws_bytes, cudaStream_t stream, bool transposed) {
  // transposed: y[m,n] = sum_k w[e,k,n] x[m,k] with the NF4 tensor of logical shape (E, K, N)
  using namespace tc;
  bind_context_once();
  GemmParams p;
  p.m_sizes = m_sizes; p.out = out; p.M = M; p.N = N; p.K = K; p.E = E; p.ms64 = ms64; p.dtype_out = dtype_out; p.group_maps = nullptr;
  p.idesc = make_idesc(dtype_in == MOE_BF16 ? 1 : 0, 0, 0, BM, NF4_BN);
  if (transposed && N < 192) return MOE_ERR_UNSUPPORTED;  // only the CTA-pair kernel has the transposed decode
  Nf4Params q;
  q.code = code; q.absmax = absmax; q.shift = 0;
  while ((1 << q.shift) < blocksize) ++q.shift;
  CUtensorMap ma, mq;
  int st;
  if (N >= 192) {
    // CTA-pair form: 128 weight rows of packed codes per CTA and stage (transposed: 64
    // contraction rows x 128 output features)
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MOE_ERR_DEVICE;
    cuuint64_t dims[3] = {(cuuint64_t)K / 2, (cuuint64_t)N, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)K / 2, (cuuint64_t)K / 2 * (cuuint64_t)N};
    cuuint32_t box[3] = {BK / 2, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (transposed) {
      dims[0] = (cuuint64_t)N / 2; dims[1] = (cuuint64_t)K;
      strides[0] = (cuuint64_t)N / 2; strides[1] = (cuuint64_t)N / 2 * (cuuint64_t)K;
      box[0] = 64; box[1] = BK;
    }
    if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(packed), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return MOE_ERR_UNSUPPORTED;
    if ((st = make_map(&ma, dtype_in, x, (uint64_t)K, (uint64_t)M, 0, 128)) != MOE_OK) return st;
    p.idesc = make_idesc(dtype_in == MOE_BF16 ? 1 : 0, transposed ? 1 : 0, 0, 256, 0);
    const int pbytes = NF4P_STAGES * NF4P_STAGE_BYTES + 4 * PAIR_STAGING_BYTES + (int)sizeof(Nf4PairControl) + 2 * (E + 1) * 4 + 1024;
    if (pbytes <= SMEM_LIMIT) {
      if (ws_usable(ws, ws_bytes, E) && (((uintptr_t)out & 15) == 0 || dtype_out == MOE_F32)) {
        GroupMapTemplates tm;
        tm.mask = 1 << GM_IN;
        tm.t[GM_IN] = ma;
        if (dtype_out != MOE_F32) {
          tm.mask |= 1 << GM_OUT;
          if ((st = make_map(&tm.t[GM_OUT], dtype_out, out, (uint64_t)N, (uint64_t)M, 0, 32)) != MOE_OK) return st;
        }
        const int gm_smem = 8 * 128 + 2 * (E + 1) * 4 + 128;
        build_group_maps_kernel<<<(E + 7) / 8, 256, gm_smem, stream>>>(tm, m_sizes, ms64, E, M, reinterpret_cast<CUtensorMap*>(ws), nullptr);
        if ((st = launch_status()) != MOE_OK) return st;
        p.group_maps = reinterpret_cast<const CUtensorMap*>(ws);
      }
#define MOE_NF4P_LAUNCH(BF, WT)                                                                          \
  do {                                                                                                   \
    auto kern = pair_fwd_nf4_kernel<BF, WT>;                                                             \
    if ((st = set_smem(kern, pbytes)) != MOE_OK) return st;                                              \
    return launch_pair_threads(kern, 2 * resident_pairs(kern, pbytes, NF4P_THREADS), NF4P_THREADS, pbytes, \
                               stream, mq, ma, p, q);                                                    \
  } while (0)
      if (dtype_in == MOE_BF16) {
        if (transposed) MOE_NF4P_LAUNCH(true, true);
        MOE_NF4P_LAUNCH(true, false);
      }
      if (transposed) MOE_NF4P_LAUNCH(false, true);
      MOE_NF4P_LAUNCH(false, false);
#undef MOE_NF4P_LAUNCH
    }
  }
  if (transposed) return MOE_ERR_UNSUPPORTED;
  if ((st = make_map(&ma, dtype_in, x, (uint64_t)K, (uint64_t)M, 0, BM)) != MOE_OK) return st;
  {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MOE_ERR_DEVICE;
    cuuint64_t dims[3] = {(cuuint64_t)K / 2, (cuuint64_t)N, (cuuint64_t)E};
    cuuint64_t strides[2] = {(cuuint64_t)K / 2, (cuuint64_t)K / 2 * (cuuint64_t)N};
    cuuint32_t box[3] = {BK / 2, NF4_BN, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(packed), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return MOE_ERR_UNSUPPORTED;
  }
  const int bytes = NF4_STAGES * NF4_STAGE_BYTES + (int)sizeof(Control) + (int)sizeof(Nf4Control) + 2 * (E + 1) * 4 + 1024;
  if (bytes > SMEM_LIMIT) return MOE_ERR_UNSUPPORTED;
  const int grid = sm_count();
  if (dtype_in == MOE_BF16) {
    if ((st = set_smem(tc_fwd_nf4_kernel<true>, bytes)) != MOE_OK) return st;
    tc_fwd_nf4_kernel<true><<<grid, NF4_THREADS, bytes, stream>>>(ma, mq, p, q);
  } else {
    if ((st = set_smem(tc_fwd_nf4_kernel<false>, bytes)) != MOE_OK) return st;
    tc_fwd_nf4_kernel<false><<<grid, NF4_THREADS, bytes, stream>>>(ma, mq, p, q);
  }
  return launch_status();
}

// Text describing the most recent host-side failure on the calling thread ("" if none).
const char* tc_last_detail() { return tc::g_detail; }

// Reads and clears the device-side error word written by an abandoned wait.
int tc_read_error(int* flag_out, bool clear) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, tc::g_tc_error, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e);
  if (clear && v != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(tc::g_tc_error, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e);
  }
  *flag_out = v;
  return MOE_OK;
}

// Diagnostic counter of the tile ring: how often a reader found the ring's barrier complete before the
// value of its round was visible (it then waited for the value).
int tc_read_late_values(int* out) {
  return cuda_status(cudaMemcpyFromSymbol(out, tc::g_tc_late_values, sizeof(int)));
}

}  // namespace moe
