// Stable sort of rows by expert id: histogram -> scan -> stable scatter, as one cooperative launch
// (sort_fused_kernel) when all chunks fit on the GPU at once, otherwise as the three kernels below.
//
// Work is split into chunks of SORT_CHUNK consecutive rows, one CTA per chunk.
//   sort_hist    : per-chunk histogram                       -> ws.hist[chunk][e]
//   sort_scan    : per-expert exclusive scan over chunks     -> ws.hist[chunk][e] (in place)
//                  expert totals -> counts[e], exclusive scan over experts -> ws.offset[e]
//   sort_scatter : position of row b = offset[e] + hist[chunk][e] + (#earlier rows of the
//                  same expert inside the chunk); the in-chunk rank is computed warp by
//                  warp with __match_any_sync so equal ids keep their original order.
// Essential traffic is M*(sizeof(id) + 8) bytes; the E*M compare matrix of the reference
// formulation (qwen3_moe_fused/kernels/indexing.py:52-56) is never materialised.
#include <cooperative_groups.h>

#include "common.cuh"

namespace moe {

constexpr int SORT_THREADS = 256;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_ROWS_PER_WARP = 256;
constexpr int SORT_CHUNK = SORT_WARPS * SORT_ROWS_PER_WARP;  // 2048 rows per CTA
constexpr int SORT_MAX_E = 4096;                             // smem: 8 warps * E * 4 B

__global__ void __launch_bounds__(SORT_THREADS)
sort_hist_kernel(const void* __restrict__ s, int is64, int64_t M, int E, int32_t* __restrict__ hist) {
  extern __shared__ int32_t sh[];  // E
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) sh[e] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * SORT_CHUNK;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < SORT_CHUNK; i += SORT_THREADS) {
    const int64_t b = base + i;
    const int64_t e = (b < M) ? load_index(s, is64, b) : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned key = ok ? (unsigned)e : (unsigned)(E + lane);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (ok && lane == (__ffs(peers) - 1)) atomicAdd(&sh[e], __popc(peers));
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) hist[(int64_t)blockIdx.x * E + e] = sh[e];
}

// One CTA of 1024 threads.  Thread e walks the chunks of expert e (turning the per-chunk
// counts into per-chunk exclusive prefixes), then the CTA scans the expert totals.
__global__ void __launch_bounds__(1024)
sort_scan_kernel(int32_t* __restrict__ hist, int nchunks, int E, int32_t* __restrict__ counts,
                 int32_t* __restrict__ offsets /* may be null */) {
  __shared__ int32_t warp_excl[32];
  __shared__ int32_t pass_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t carry = 0;  // same value in every thread
  for (int e0 = 0; e0 < E; e0 += 1024) {
    const int e = e0 + (int)threadIdx.x;
    int32_t total = 0;
    if (e < E) {
      // eight chunks per step: the loads of a step are independent of each other and of the
      // stores of the step before, so a step costs one memory latency instead of eight
      constexpr int STEP = 8;
      int c = 0;
      for (; c + STEP <= nchunks; c += STEP) {
        int32_t t[STEP];
#pragma unroll
        for (int i = 0; i < STEP; ++i) t[i] = hist[(int64_t)(c + i) * E + e];
#pragma unroll
        for (int i = 0; i < STEP; ++i) {
          hist[(int64_t)(c + i) * E + e] = total;
          total += t[i];
        }
      }
      for (; c < nchunks; ++c) {
        const int32_t t = hist[(int64_t)c * E + e];
        hist[(int64_t)c * E + e] = total;
        total += t;
      }
      counts[e] = total;
    }
    int32_t incl = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    if (lane == 31) warp_excl[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int32_t w = warp_excl[lane];
      int32_t wi = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t v = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += v;
      }
      warp_excl[lane] = wi - w;
      if (lane == 31) pass_total = wi;
    }
    __syncthreads();
    if (e < E && offsets != nullptr) offsets[e] = carry + warp_excl[warp] + (incl - total);
    carry += pass_total;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(SORT_THREADS)
sort_scatter_kernel(const void* __restrict__ s, int is64, int64_t M, int E,
                    const int32_t* __restrict__ hist, const int32_t* __restrict__ offsets,
                    int32_t* __restrict__ inv_idx, int32_t* __restrict__ idx) {
  extern __shared__ int32_t sh[];  // [SORT_WARPS][E] running positions
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* mine = sh + (size_t)warp * E;
  for (int i = threadIdx.x; i < SORT_WARPS * E; i += SORT_THREADS) sh[i] = 0;
  __syncthreads();
  const int64_t wbase = (int64_t)blockIdx.x * SORT_CHUNK + (int64_t)warp * SORT_ROWS_PER_WARP;

  // Pass A: rows of each expert inside this warp's slice.
  for (int it = 0; it < SORT_ROWS_PER_WARP / 32; ++it) {
    const int64_t b = wbase + it * 32 + lane;
    const int64_t e = (b < M) ? load_index(s, is64, b) : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned key = ok ? (unsigned)e : (unsigned)(E + lane);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (ok && lane == (__ffs(peers) - 1)) mine[e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  // Exclusive scan over the warps of the CTA, seeded with the global position of this
  // chunk's first row of expert e.
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int32_t run = offsets[e] + hist[(int64_t)blockIdx.x * E + e];
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) {
      const int32_t t = sh[(size_t)w * E + e];
      sh[(size_t)w * E + e] = run;
      run += t;
    }
  }
  __syncthreads();
  // Pass B: assign positions in original order.
  for (int it = 0; it < SORT_ROWS_PER_WARP / 32; ++it) {
    const int64_t b = wbase + it * 32 + lane;
    const int64_t e = (b < M) ? load_index(s, is64, b) : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned key = ok ? (unsigned)e : (unsigned)(E + lane);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    int32_t pos = 0;
    if (ok) pos = mine[e] + __popc(peers & ((1u << lane) - 1u));
    __syncwarp();
    if (ok && lane == (__ffs(peers) - 1)) mine[e] += __popc(peers);
    __syncwarp();
    if (ok) {
      idx[b] = pos;
      inv_idx[pos] = (int32_t)b;
    }
  }
}

// The whole sort in ONE cooperative launch (all chunks' CTAs resident at once, one grid-wide barrier):
//   A  per-warp histograms of the chunk in shared memory; the chunk's totals go to hist[chunk][e]
//   -- grid barrier --
//   B  every CTA sums the totals of all chunks per expert (E * chunks words from L2), scans the experts,
//      adds the rows of earlier chunks, and turns its per-warp histograms into running positions
//   C  stable scatter, as in sort_scatter_kernel
// The ids are read twice from L2 (A and C); nothing else is shared between launches, so the three-kernel
// path's two launch gaps disappear.  Used when every chunk's CTA fits on the GPU at once.
__global__ void __launch_bounds__(SORT_THREADS)
sort_fused_kernel(const void* __restrict__ s, int is64, int64_t M, int E, int nchunks, int32_t* __restrict__ hist,
                  int32_t* __restrict__ counts, int32_t* __restrict__ inv_idx, int32_t* __restrict__ idx) {
  extern __shared__ int32_t sh[];            // [SORT_WARPS][E] histograms, then running positions
  int32_t* base_of = sh + (size_t)SORT_WARPS * E;  // [E] first position of this chunk's rows of expert e
  __shared__ int32_t warp_excl[SORT_WARPS];
  __shared__ int32_t pass_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* mine = sh + (size_t)warp * E;
  for (int i = threadIdx.x; i < SORT_WARPS * E; i += SORT_THREADS) sh[i] = 0;
  __syncthreads();
  const int64_t wbase = (int64_t)blockIdx.x * SORT_CHUNK + (int64_t)warp * SORT_ROWS_PER_WARP;
  for (int it = 0; it < SORT_ROWS_PER_WARP / 32; ++it) {
    const int64_t b = wbase + it * 32 + lane;
    const int64_t e = (b < M) ? load_index(s, is64, b) : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned key = ok ? (unsigned)e : (unsigned)(E + lane);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (ok && lane == (__ffs(peers) - 1)) mine[e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int32_t t = 0;
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) t += sh[(size_t)w * E + e];
    hist[(int64_t)blockIdx.x * E + e] = t;
  }
  __threadfence();
  cooperative_groups::this_grid().sync();

  // B: expert totals, exclusive scan over the experts, rows of earlier chunks
  int32_t carry = 0;  // same value in every thread
  for (int e0 = 0; e0 < E; e0 += SORT_THREADS) {
    const int e = e0 + (int)threadIdx.x;
    int32_t total = 0, before = 0;
    if (e < E) {
      for (int c = 0; c < nchunks; ++c) {
        const int32_t t = __ldcg(hist + (int64_t)c * E + e);
        if (c < (int)blockIdx.x) before += t;
        total += t;
      }
      if (blockIdx.x == 0) counts[e] = total;
    }
    int32_t incl = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    if (lane == 31) warp_excl[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int32_t w = lane < SORT_WARPS ? warp_excl[lane] : 0;
      int32_t wi = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t v = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += v;
      }
      if (lane < SORT_WARPS) warp_excl[lane] = wi - w;
      if (lane == 31) pass_total = wi;
    }
    __syncthreads();
    if (e < E) base_of[e] = carry + warp_excl[warp] + (incl - total) + before;
    carry += pass_total;
    __syncthreads();
  }
  if (idx == nullptr) return;
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) {
    int32_t run = base_of[e];
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) {
      const int32_t t = sh[(size_t)w * E + e];
      sh[(size_t)w * E + e] = run;
      run += t;
    }
  }
  __syncthreads();
  // C: positions in original order
  for (int it = 0; it < SORT_ROWS_PER_WARP / 32; ++it) {
    const int64_t b = wbase + it * 32 + lane;
    const int64_t e = (b < M) ? load_index(s, is64, b) : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned key = ok ? (unsigned)e : (unsigned)(E + lane);
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    int32_t pos = 0;
    if (ok) pos = mine[e] + __popc(peers & ((1u << lane) - 1u));
    __syncwarp();
    if (ok && lane == (__ffs(peers) - 1)) mine[e] += __popc(peers);
    __syncwarp();
    if (ok) {
      idx[b] = pos;
      inv_idx[pos] = (int32_t)b;
    }
  }
}

// Single CTA: counts of ids below / at-or-below each expert (any input order).
__global__ void __launch_bounds__(1024)
begins_ends_kernel(const void* __restrict__ s, int is64, int64_t M, int E, int32_t* __restrict__ out) {
  extern __shared__ int32_t sh[];  // E
  __shared__ int32_t warp_excl[32];
  __shared__ int32_t pass_total;
  for (int e = threadIdx.x; e < E; e += 1024) sh[e] = 0;
  __syncthreads();
  for (int64_t b = threadIdx.x; b < M; b += 1024) {
    const int64_t e = load_index(s, is64, b);
    if (e >= 0 && e < E) atomicAdd(&sh[e], 1);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t carry = 0;
  for (int e0 = 0; e0 < E; e0 += 1024) {
    const int e = e0 + (int)threadIdx.x;
    const int32_t total = e < E ? sh[e] : 0;
    int32_t incl = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    if (lane == 31) warp_excl[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int32_t w = warp_excl[lane];
      int32_t wi = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t v = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += v;
      }
      warp_excl[lane] = wi - w;
      if (lane == 31) pass_total = wi;
    }
    __syncthreads();
    if (e < E) {
      const int32_t begin = carry + warp_excl[warp] + (incl - total);
      out[2 * e] = begin;
      out[2 * e + 1] = begin + total;
    }
    carry += pass_total;
    __syncthreads();
  }
}

static inline int64_t sort_chunks(int64_t M) { return M <= 0 ? 0 : (M + SORT_CHUNK - 1) / SORT_CHUNK; }

}  // namespace moe

using namespace moe;

MOE_API size_t moe_sort_workspace_bytes(int64_t M, int E) {
  if (M < 0 || E <= 0) return 0;
  // hist[chunks][E] + offsets[E]; never zero so callers can always allocate it.
  return (size_t)(sort_chunks(M) + 1) * (size_t)E * sizeof(int32_t);
}

// Argument checks shared by the two sort entry points.
static int sort_check(const void* s, int s_dtype, int64_t M, int E, const int32_t* counts, const int32_t* inv_idx,
                      const int32_t* idx) {
  if (!is_int_dtype(s_dtype)) return MOE_ERR_DTYPE;
  if (M < 0 || E <= 0 || E > SORT_MAX_E || M > 0x7fffffffLL) return MOE_ERR_SHAPE;
  if (counts == nullptr || (M > 0 && s == nullptr)) return MOE_ERR_NULL;
  if ((inv_idx == nullptr) != (idx == nullptr)) return MOE_ERR_NULL;
  return MOE_OK;
}

// The three launches of the sort, with `scratch` holding moe_sort_workspace_bytes(M, E) bytes.
// Every word of the scratch that the scan and scatter kernels read is written first by the
// histogram and scan kernels of the same call, so its previous contents do not matter.
// Chunks whose CTAs of sort_fused_kernel can all be resident at once on the current device (0: the
// device cannot launch cooperatively); the answer depends on E through the shared-memory size.
static int sort_fused_capacity(int E, size_t smem) {
  static int coop[64] = {0};  // 0 unknown, 1 yes, 2 no
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (coop[dev] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev);
    coop[dev] = v ? 1 : 2;
  }
  if (coop[dev] != 1) return 0;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sort_fused_kernel, SORT_THREADS, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  (void)E;
  return per_sm * sm_count();
}

static int sort_launch(const void* s, int is64, int64_t M, int E, int32_t* counts, int32_t* inv_idx, int32_t* idx,
                       void* scratch, cudaStream_t stream) {
  const int nchunks = (int)sort_chunks(M);
  int32_t* hist = (int32_t*)scratch;
  // one cooperative launch when every chunk's CTA fits on the GPU at once (up to a few million rows)
  const size_t fused_smem = (size_t)(SORT_WARPS + 1) * E * sizeof(int32_t);
  if (nchunks > 0 && fused_smem <= 48 * 1024 && nchunks <= sort_fused_capacity(E, fused_smem)) {
    int nch = nchunks;
    void* args[] = {(void*)&s, (void*)&is64, (void*)&M, (void*)&E, (void*)&nch, (void*)&hist, (void*)&counts, (void*)&inv_idx, (void*)&idx};
    const cudaError_t e = cudaLaunchCooperativeKernel((const void*)sort_fused_kernel, dim3(nchunks), dim3(SORT_THREADS), args,
                                                      fused_smem, stream);
    if (e == cudaSuccess) return MOE_OK;
    (void)cudaGetLastError();  // (e.g. the device is shared with another resident kernel's reservation): three launches
  }
  int32_t* offsets = hist + (size_t)nchunks * E;
  if (nchunks > 0) {
    sort_hist_kernel<<<nchunks, SORT_THREADS, E * sizeof(int32_t), stream>>>(s, is64, M, E, hist);
  }
  sort_scan_kernel<<<1, 1024, 0, stream>>>(hist, nchunks, E, counts, idx ? offsets : nullptr);
  if (idx != nullptr && nchunks > 0) {
    const size_t smem = (size_t)SORT_WARPS * E * sizeof(int32_t);
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cuda_status(e);
    }
    sort_scatter_kernel<<<nchunks, SORT_THREADS, smem, stream>>>(s, is64, M, E, hist, offsets, inv_idx, idx);
  }
  return launch_status();
}

MOE_API int moe_sort_by_expert(const void* s, int s_dtype, int64_t M, int E, int32_t* counts,
                               int32_t* inv_idx, int32_t* idx, void* ws, size_t ws_bytes,
                               void* stream_) {
  const int st = sort_check(s, s_dtype, M, E, counts, inv_idx, idx);
  if (st != MOE_OK) return st;
  if (ws == nullptr || ws_bytes < moe_sort_workspace_bytes(M, E)) return MOE_ERR_WORKSPACE;
  return sort_launch(s, s_dtype == MOE_I64, M, E, counts, inv_idx, idx, ws, (cudaStream_t)stream_);
}

MOE_API int moe_batch_begins_ends(const void* s_sorted, int s_dtype, int64_t M, int E,
                                  int32_t* begins_ends, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!is_int_dtype(s_dtype)) return MOE_ERR_DTYPE;
  if (M < 0 || E <= 0 || E > SORT_MAX_E) return MOE_ERR_SHAPE;
  if (begins_ends == nullptr || (M > 0 && s_sorted == nullptr)) return MOE_ERR_NULL;
  begins_ends_kernel<<<1, 1024, E * sizeof(int32_t), stream>>>(s_sorted, s_dtype == MOE_I64, M, E, begins_ends);
  return launch_status();
}

// ---------------------------------------------------------------------------------------
// Sort without caller-provided workspace.
//
// Some hosts of this library cannot hand it scratch memory: a caller that must not call
// cudaMalloc at that point (inside a region where allocation is forbidden or would
// synchronise, such as a latency-critical serving loop or a plugin interface that only
// passes inputs and outputs), or one that has no allocator of its own at all.  For them the
// per-chunk histograms and expert offsets live in the fixed device array below, which every
// GPU that loads the library holds until the process exits.
// ---------------------------------------------------------------------------------------
namespace moe {

constexpr size_t SORT_STATIC_BYTES = 256 * 1024;  // e.g. 262144 rows with 128 experts need 66 KB
static __device__ __align__(256) unsigned char g_sort_scratch[SORT_STATIC_BYTES];

// Device address of g_sort_scratch on the current device.  In host code the array's name
// is only a handle for the runtime, not a device pointer, so the address is looked up once
// per device (with that device current) and cached.
static int sort_static_scratch(void** out) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (dev < 0 || dev >= 64) return MOE_ERR_DEVICE;
  void* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(&p, g_sort_scratch);
    if (e != cudaSuccess) return cuda_status(e);
    if (p == nullptr) return MOE_ERR_DEVICE;
    __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return MOE_OK;
}

}  // namespace moe

MOE_API size_t moe_sort_static_capacity_bytes(void) { return moe::SORT_STATIC_BYTES; }

MOE_API int moe_sort_by_expert_static(const void* s, int s_dtype, int64_t M, int E, int32_t* counts,
                                      int32_t* inv_idx, int32_t* idx, void* stream_) {
  const int chk = sort_check(s, s_dtype, M, E, counts, inv_idx, idx);
  if (chk != MOE_OK) return chk;
  // the fixed array bounds the problem size: refuse anything that would not fit
  if (moe_sort_workspace_bytes(M, E) > SORT_STATIC_BYTES) return MOE_ERR_WORKSPACE;
  void* scratch = nullptr;
  const int st = sort_static_scratch(&scratch);
  if (st != MOE_OK) return st;
  // the array still holds the previous call's contents; sort_launch does not depend on them
  return sort_launch(s, s_dtype == MOE_I64, M, E, counts, inv_idx, idx, scratch, (cudaStream_t)stream_);
}
