// Expert-parallel row movement over peer memory (NVLink): rows that are sorted by expert are
// copied, segment by segment, to one destination address per expert.  The destination may be
// local memory or a peer GPU's memory mapped into this process; the stores are plain 16-byte
// global stores, posted over NVLink when the address is remote.  The kernel waits on nothing
// and signals nothing: ordering against the consumer is the caller's (stream order plus a
// collective or event on both sides).
#include "common.cuh"

namespace moe {

constexpr int PUSH_THREADS = 256;
constexpr int PUSH_MAX_E = 1024;
constexpr int PLAN_MAX_WORLD_TOK = 16;  // ranks of one expert-parallel group (= PLAN_MAX_WORLD)

// begins[e] = rows before expert e; computed by warp 0, E / 32 consecutive entries per lane.
__device__ __forceinline__ void push_build_begins(const void* m_sizes, int ms64, int E, int* begins) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const int per = (E + 31) / 32;
    const int lo = min(lane * per, E), hi = min(lo + per, E);
    int sum = 0;
    for (int e = lo; e < hi; ++e)
      sum += ms64 ? (int)reinterpret_cast<const int64_t*>(m_sizes)[e] : reinterpret_cast<const int32_t*>(m_sizes)[e];
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    int run = incl - sum;
    for (int e = lo; e < hi; ++e) {
      begins[e] = run;
      run += ms64 ? (int)reinterpret_cast<const int64_t*>(m_sizes)[e] : reinterpret_cast<const int32_t*>(m_sizes)[e];
    }
    if (lane == 31) begins[E] = incl;
  }
  __syncthreads();
}

// One warp per row; each lane keeps up to UNROLL 16-byte vectors in flight.
template <int UNROLL>
__global__ void __launch_bounds__(PUSH_THREADS)
ep_push_rows_kernel(const uint4* __restrict__ rows, int64_t M, int row_vecs, const void* __restrict__ m_sizes, int ms64,
                    int E, const uint64_t* __restrict__ dst_ptrs, const int32_t* __restrict__ dst_limit, int first_expert,
                    const int32_t* __restrict__ src_index, int src_div, int32_t* __restrict__ dropped) {
  __shared__ int begins[PUSH_MAX_E + 1];
  push_build_begins(m_sizes, ms64, E, begins);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = PUSH_THREADS / 32;
  const int64_t total = min(M, (int64_t)begins[E]);
  // rows are visited starting at `first_expert` (wrapping around): ranks that start at different
  // experts write to different destinations at any one time instead of all to the same one
  const int64_t start = min((int64_t)begins[first_expert], total);
  for (int64_t i = (int64_t)blockIdx.x * warps + warp; i < total; i += (int64_t)gridDim.x * warps) {
    const int64_t r = i + start < total ? i + start : i + start - total;
    // expert of row r: last e with begins[e] <= r
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (begins[mid] <= (int)r) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int local = (int)r - begins[e];
    if (dst_limit != nullptr) {
      const int limit = dst_limit[e];
      if (limit < 0) continue;  // this expert's rows are not part of this push
      if (local >= limit) {     // would overrun the receiver's buffer: not written, but counted
        if (dropped != nullptr && lane == 0) atomicAdd(dropped, 1);
        continue;
      }
    }
    // with a source index, sorted row r is row src_index[r] / src_div of `rows` (token rows expanded on the fly)
    const uint4* src = rows + (src_index ? (int64_t)(src_index[r] / src_div) : r) * row_vecs;
    uint4* dst = reinterpret_cast<uint4*>(dst_ptrs[e]) + (int64_t)local * row_vecs;
    for (int c0 = 0; c0 < row_vecs; c0 += 32 * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < row_vecs) v[u] = src_index ? __ldg(src + c) : __ldcs(src + c);  // plain rows are read once: streaming
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < row_vecs) __stcs(dst + c, v[u]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Token-deduplicated dispatch.  A token whose k experts live on r distinct ranks travels r
// times, not k times: every token row is stored once per destination rank, at the slot
// slot[t][d] of that rank's token buffer (-1: the token has no expert there), and every
// expanded row (sorted by expert) sends just a 4-byte index, the slot of its token on the
// rank that owns its expert, to the row's expert-major position there.  The owner expands
// the rows locally (or gathers them in its GEMM's token load).
// ---------------------------------------------------------------------------------------

// Bookkeeping of the token-deduplicated dispatch, one CTA: for token t and rank d, pos[t * world + d] =
// number of earlier tokens (of this rank) that also have an expert on rank d, or -1 when t has none there;
// n_tokens[d] = tokens with an expert on d.  selected: T * k expert ids, token-major.
constexpr int TOKPOS_THREADS = 1024;

__global__ void __launch_bounds__(TOKPOS_THREADS)
ep_token_positions_kernel(const void* __restrict__ selected, int sel64, int64_t T, int k, int e_all, int world,
                          int32_t* __restrict__ pos, int32_t* __restrict__ n_tokens) {
  // Rounds of 1024 consecutive tokens, one per thread (a warp reads its 32 tokens' ids as one contiguous
  // run).  Per destination: ballot -> position inside the warp, warp totals scanned by warp d.
  __shared__ int32_t warp_cnt[PLAN_MAX_WORLD_TOK][TOKPOS_THREADS / 32];
  __shared__ int32_t round_total[PLAN_MAX_WORLD_TOK];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lower = (1u << lane) - 1u;
  int32_t running[PLAN_MAX_WORLD_TOK];
#pragma unroll
  for (int d = 0; d < PLAN_MAX_WORLD_TOK; ++d) running[d] = 0;
  auto dest_mask = [&](int64_t t) {
    uint32_t m = 0;
    if (t < T) {
      for (int j = 0; j < k; ++j) {
        const int64_t e = sel64 ? __ldg(reinterpret_cast<const int64_t*>(selected) + t * k + j)
                                : (int64_t)__ldg(reinterpret_cast<const int32_t*>(selected) + t * k + j);
        const int64_t d = e / e_all;
        if (d >= 0 && d < world) m |= 1u << d;
      }
    }
    return m;
  };
  uint32_t m_next = dest_mask(tid);
  for (int64_t base = 0; base < T; base += TOKPOS_THREADS) {
    const int64_t t = base + tid;
    const uint32_t m = m_next;
    m_next = dest_mask(t + TOKPOS_THREADS);  // the next round's ids are in flight during this round's scan
    int32_t in_warp[PLAN_MAX_WORLD_TOK];
#pragma unroll
    for (int d = 0; d < PLAN_MAX_WORLD_TOK; ++d) {
      if (d < world) {
        const uint32_t b = __ballot_sync(0xffffffffu, (m >> d) & 1u);
        in_warp[d] = __popc(b & lower);
        if (lane == 0) warp_cnt[d][warp] = __popc(b);
      }
    }
    __syncthreads();
    if (warp < world) {  // warp d scans the 32 warp totals of destination d
      const int32_t w = warp_cnt[warp][lane];
      int32_t incl = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      warp_cnt[warp][lane] = incl - w;
      if (lane == 31) round_total[warp] = incl;
    }
    __syncthreads();
#pragma unroll
    for (int d = 0; d < PLAN_MAX_WORLD_TOK; ++d) {
      if (d < world) {
        if (t < T) pos[t * world + d] = ((m >> d) & 1u) ? running[d] + warp_cnt[d][warp] + in_warp[d] : -1;
        running[d] += round_total[d];
      }
    }
    __syncthreads();  // warp_cnt / round_total are rewritten by the next round
  }
#pragma unroll
  for (int d = 0; d < PLAN_MAX_WORLD_TOK; ++d)
    if (d < world && tid == d) n_tokens[d] = running[d];
}

// One warp per token: the row is read once and stored to up to `world` destinations.
template <int UNROLL>
__global__ void __launch_bounds__(PUSH_THREADS)
ep_push_tokens_kernel(const uint4* __restrict__ tokens, int64_t T, int row_vecs, const int32_t* __restrict__ pos,
                      const int32_t* __restrict__ slot_base, int world, int first_rank, const uint64_t* __restrict__ dst_ptrs,
                      int slot_limit, int32_t* __restrict__ dropped) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = PUSH_THREADS / 32;
  for (int64_t t = (int64_t)blockIdx.x * warps + warp; t < T; t += (int64_t)gridDim.x * warps) {
    const uint4* src = tokens + t * row_vecs;
    for (int c0 = 0; c0 < row_vecs; c0 += 32 * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < row_vecs) v[u] = __ldg(src + c);
      }
      // destinations are visited starting at `first_rank`, so that the ranks' stores fan out
      for (int j = 0; j < world; ++j) {
        const int d = (first_rank + j) % world;
        const int ps = pos[t * world + d];
        if (ps < 0) continue;
        const int sl = ps + (slot_base ? slot_base[d] : 0);
        if (sl >= slot_limit) {  // would overrun the receiver's token buffer: not written, but counted
          if (dropped != nullptr && lane == 0 && c0 == 0) atomicAdd(dropped, 1);
          continue;
        }
        uint4* dst = reinterpret_cast<uint4*>(dst_ptrs[d]) + (int64_t)sl * row_vecs;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int c = c0 + u * 32 + lane;
          if (c < row_vecs) __stcs(dst + c, v[u]);
        }
      }
    }
  }
}

// One thread per expanded row r (sorted by expert): the slot of its token on the owner of its expert
// goes to position i of expert e's index run on that owner (dst_ptrs[e] + 4 i); rows with
// i >= dst_limit[e] are not written (the row push counts them).
__global__ void __launch_bounds__(PUSH_THREADS)
ep_push_index_kernel(const int32_t* __restrict__ pos, const int32_t* __restrict__ slot_base, int world, int e_all,
                     const int32_t* __restrict__ sort_idx, int k, int64_t M, const void* __restrict__ m_sizes, int ms64, int E,
                     const uint64_t* __restrict__ dst_ptrs, const int32_t* __restrict__ dst_limit, int32_t* __restrict__ dropped) {
  __shared__ int begins[PUSH_MAX_E + 1];
  push_build_begins(m_sizes, ms64, E, begins);
  const int64_t total = min(M, (int64_t)begins[E]);
  for (int64_t r = (int64_t)blockIdx.x * PUSH_THREADS + threadIdx.x; r < total; r += (int64_t)gridDim.x * PUSH_THREADS) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (begins[mid] <= (int)r) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int local = (int)r - begins[e];
    if (dst_limit != nullptr) {
      const int limit = dst_limit[e];
      if (limit < 0) continue;
      if (local >= limit) {
        if (dropped != nullptr) atomicAdd(dropped, 1);
        continue;
      }
    }
    const int64_t t = sort_idx[r] / k;
    const int d = e / e_all;
    reinterpret_cast<int32_t*>(dst_ptrs[e])[local] = pos[t * world + d] + (slot_base ? slot_base[d] : 0);
  }
}

// The owner's side of the token-deduplicated dispatch: out[r] = tokens[index[r]] for the rows it
// received, r < min(*n_rows, max_rows) with the count read on the device.  An index outside the
// token buffer (possible only where a sender dropped rows) reads row 0 instead of faulting.
template <int UNROLL>
__global__ void __launch_bounds__(PUSH_THREADS)
ep_expand_kernel(const uint4* __restrict__ tokens, int64_t token_rows, int row_vecs, const int32_t* __restrict__ index,
                 const int64_t* __restrict__ n_rows, int64_t max_rows, uint4* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = PUSH_THREADS / 32;
  const int64_t total = min(*n_rows, max_rows);
  for (int64_t r = (int64_t)blockIdx.x * warps + warp; r < total; r += (int64_t)gridDim.x * warps) {
    int64_t t = index[r];
    if (t < 0 || t >= token_rows) t = 0;
    const uint4* src = tokens + t * row_vecs;
    uint4* dst = out + r * row_vecs;
    for (int c0 = 0; c0 < row_vecs; c0 += 32 * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < row_vecs) v[u] = __ldg(src + c);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < row_vecs) __stcs(dst + c, v[u]);
      }
    }
  }
}

// Row bookkeeping of one routing decision for the peer-memory exchange, in one launch.
// counts[s][e]: rows of source rank s for global expert e.  Expert e = d * e_all + el lives on
// rank d.  The plan covers local experts lo..hi-1 of every rank.  On owner d the groups are laid
// out (local expert, slot j) with slot j holding the rows of source (d + 1 + j) % world.
constexpr int PLAN_MAX_WORLD = 16;
constexpr int PLAN_MAX_E = 1024;

__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ counts, int world, int rank, int E, int lo, int hi,
               int64_t* __restrict__ send_row, int32_t* __restrict__ send_ok, int32_t* __restrict__ group_sizes,
               int32_t* __restrict__ weight_index, int64_t* __restrict__ group_src, int64_t* __restrict__ return_row,
               int32_t* __restrict__ local_m_sizes, int64_t* __restrict__ recv_rows) {
  extern __shared__ int32_t plan_smem[];
  int32_t* cnt = plan_smem;                // [world][E]
  int32_t* begins = cnt + world * E;       // [world][E]: first row of expert e in source s's sorted order
  int32_t* first = begins + world * E;     // [world][n_local * world]: first row of each group on its owner
  const int e_all = E / world;
  const int n_local = hi - lo;
  const int G = n_local * world;
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) cnt[i] = counts[i];
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const int s = threadIdx.x;
    int run = 0;
    for (int e = 0; e < E; ++e) { begins[s * E + e] = run; run += cnt[s * E + e]; }
  } else if ((int)threadIdx.x >= 32 && (int)threadIdx.x < 32 + world) {
    const int d = threadIdx.x - 32;
    int run = 0;
    for (int g = 0; g < G; ++g) {
      const int el = g / world, j = g % world;
      first[d * G + g] = run;
      run += cnt[((d + 1 + j) % world) * E + d * e_all + lo + el];
    }
    if (d == rank) *recv_rows = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / e_all, el = e % e_all;
    const bool in = el >= lo && el < hi;
    const int slot = ((rank - d - 1) % world + world) % world;
    send_row[e] = in ? first[d * G + (el - lo) * world + slot] : 0;
    send_ok[e] = in ? 1 : 0;
  }
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    const int el = g / world, j = g % world;
    const int src = (rank + 1 + j) % world;
    const int e = rank * e_all + lo + el;
    group_sizes[g] = cnt[src * E + e];
    weight_index[g] = el;
    group_src[g] = src;
    return_row[g] = begins[src * E + e];
  }
  for (int el = threadIdx.x; el < n_local; el += blockDim.x) {
    int sum = 0;
    for (int s = 0; s < world; ++s) sum += cnt[s * E + rank * e_all + lo + el];
    local_m_sizes[el] = sum;
  }
}

}  // namespace moe

using namespace moe;

MOE_API int moe_ep_plan(const int32_t* counts, int world, int rank, int E, int lo, int hi, int64_t* send_row,
                        int32_t* send_ok, int32_t* group_sizes, int32_t* weight_index, int64_t* group_src,
                        int64_t* return_row, int32_t* local_m_sizes, int64_t* recv_rows, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (world <= 0 || world > PLAN_MAX_WORLD || E <= 0 || E > PLAN_MAX_E || (E % world) != 0) return MOE_ERR_SHAPE;
  if (rank < 0 || rank >= world || lo < 0 || hi <= lo || hi > E / world) return MOE_ERR_SHAPE;
  if (!counts || !send_row || !send_ok || !group_sizes || !weight_index || !group_src || !return_row ||
      !local_m_sizes || !recv_rows)
    return MOE_ERR_NULL;
  const size_t smem = (size_t)(2 * world * E + world * (hi - lo) * world) * sizeof(int32_t);
  if (smem > 227 * 1024) return MOE_ERR_SHAPE;
  if (smem > 48 * 1024) {  // above the default limit the kernel has to opt in
    const cudaError_t e = cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_status(e);
  }
  ep_plan_kernel<<<1, 256, smem, stream>>>(counts, world, rank, E, lo, hi, send_row, send_ok, group_sizes, weight_index,
                                           group_src, return_row, local_m_sizes, recv_rows);
  return launch_status();
}

MOE_API int moe_ep_push_rows(const void* rows, int64_t M, int64_t row_bytes, const void* m_sizes, int m_sizes_dtype,
                             int E, const uint64_t* dst_ptrs, const int32_t* dst_limit, int first_expert,
                             const int32_t* src_index, int src_div, int max_ctas, int32_t* dropped, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!is_int_dtype(m_sizes_dtype)) return MOE_ERR_DTYPE;
  if (M < 0 || row_bytes < 0 || E <= 0 || E > PUSH_MAX_E || M > 0x7fffffffLL) return MOE_ERR_SHAPE;
  if (first_expert < 0 || first_expert >= E || (src_index != nullptr && src_div <= 0)) return MOE_ERR_SHAPE;
  if (M == 0 || row_bytes == 0) return MOE_OK;
  if (!rows || !m_sizes || !dst_ptrs) return MOE_ERR_NULL;
  if ((row_bytes & 15) || ((uintptr_t)rows & 15)) return MOE_ERR_ALIGN;
  const int warps = PUSH_THREADS / 32;
  int64_t grid = (M + warps - 1) / warps;
  const int64_t cap = max_ctas > 0 ? max_ctas : (int64_t)sm_count() * 4;
  if (grid > cap) grid = cap;
  ep_push_rows_kernel<8><<<(int)grid, PUSH_THREADS, 0, stream>>>(
      reinterpret_cast<const uint4*>(rows), M, (int)(row_bytes / 16), m_sizes, m_sizes_dtype == MOE_I64, E, dst_ptrs, dst_limit, first_expert,
      src_index, src_div, dropped);
  return launch_status();
}

MOE_API int moe_ep_token_positions(const void* selected, int sel_dtype, int64_t T, int k, int E, int world, int32_t* pos,
                                   int32_t* n_tokens, void* stream_) {
  if (!is_int_dtype(sel_dtype)) return MOE_ERR_DTYPE;
  if (T < 0 || T > 0x7fffffffLL || k <= 0 || world <= 0 || world > PLAN_MAX_WORLD_TOK || E <= 0 || (E % world) != 0) return MOE_ERR_SHAPE;
  if (!n_tokens || (T > 0 && (!selected || !pos))) return MOE_ERR_NULL;
  ep_token_positions_kernel<<<1, TOKPOS_THREADS, 0, (cudaStream_t)stream_>>>(selected, sel_dtype == MOE_I64, T, k, E / world, world, pos,
                                                                              n_tokens);
  return launch_status();
}

MOE_API int moe_ep_push_tokens(const void* tokens, int64_t T, int64_t row_bytes, const int32_t* slot, const int32_t* slot_base,
                               int world, int first_rank, const uint64_t* dst_ptrs, int slot_limit, int max_ctas,
                               int32_t* dropped, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (T < 0 || row_bytes < 0 || world <= 0 || world > PLAN_MAX_WORLD || T > 0x7fffffffLL || slot_limit < 0) return MOE_ERR_SHAPE;
  if (first_rank < 0 || first_rank >= world) return MOE_ERR_SHAPE;
  if (T == 0 || row_bytes == 0) return MOE_OK;
  if (!tokens || !slot || !dst_ptrs) return MOE_ERR_NULL;
  if ((row_bytes & 15) || ((uintptr_t)tokens & 15)) return MOE_ERR_ALIGN;
  const int warps = PUSH_THREADS / 32;
  int64_t grid = (T + warps - 1) / warps;
  const int64_t cap = max_ctas > 0 ? max_ctas : (int64_t)sm_count() * 4;
  if (grid > cap) grid = cap;
  ep_push_tokens_kernel<8><<<(int)grid, PUSH_THREADS, 0, stream>>>(reinterpret_cast<const uint4*>(tokens), T, (int)(row_bytes / 16),
                                                                  slot, slot_base, world, first_rank, dst_ptrs, slot_limit, dropped);
  return launch_status();
}

MOE_API int moe_ep_push_index(const int32_t* slot, const int32_t* slot_base, int world, const int32_t* sort_idx, int k, int64_t M,
                              const void* m_sizes, int m_sizes_dtype, int E, const uint64_t* dst_ptrs, const int32_t* dst_limit,
                              int32_t* dropped, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!is_int_dtype(m_sizes_dtype)) return MOE_ERR_DTYPE;
  if (M < 0 || M > 0x7fffffffLL || world <= 0 || world > PLAN_MAX_WORLD || E <= 0 || E > PUSH_MAX_E || (E % world) != 0 || k <= 0)
    return MOE_ERR_SHAPE;
  if (M == 0) return MOE_OK;
  if (!slot || !sort_idx || !m_sizes || !dst_ptrs) return MOE_ERR_NULL;
  int64_t grid = (M + PUSH_THREADS - 1) / PUSH_THREADS;
  const int64_t cap = (int64_t)sm_count() * 4;
  if (grid > cap) grid = cap;
  ep_push_index_kernel<<<(int)grid, PUSH_THREADS, 0, stream>>>(slot, slot_base, world, E / world, sort_idx, k, M, m_sizes,
                                                             m_sizes_dtype == MOE_I64, E, dst_ptrs, dst_limit, dropped);
  return launch_status();
}

MOE_API int moe_ep_expand_rows(const void* tokens, int64_t token_rows, int64_t row_bytes, const int32_t* index,
                               const int64_t* n_rows, int64_t max_rows, void* out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (token_rows < 0 || row_bytes < 0 || max_rows < 0) return MOE_ERR_SHAPE;
  if (max_rows == 0 || row_bytes == 0) return MOE_OK;
  if (!tokens || !index || !n_rows || !out || token_rows == 0) return MOE_ERR_NULL;
  if ((row_bytes & 15) || ((uintptr_t)tokens & 15) || ((uintptr_t)out & 15)) return MOE_ERR_ALIGN;
  const int warps = PUSH_THREADS / 32;
  int64_t grid = (max_rows + warps - 1) / warps;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (grid > cap) grid = cap;
  ep_expand_kernel<8><<<(int)grid, PUSH_THREADS, 0, stream>>>(reinterpret_cast<const uint4*>(tokens), token_rows, (int)(row_bytes / 16),
                                                             index, n_rows, max_rows, reinterpret_cast<uint4*>(out));
  return launch_status();
}
