// HBM-bound kernels around the grouped GEMMs: SiLU-mul (forward, backward, in-place
// backward), NF4 decode, expand+gather of token rows, un-permute+weighted combine.
// All of them move 16 bytes per thread per access when pointers and extents allow it
// and fall back to scalar accesses otherwise; grids are a multiple of the SM count and
// loop with a grid stride.
#include "common.cuh"

namespace moe {

constexpr int EW_THREADS = 256;

static inline int ew_grid(int64_t work_items) {
  const int64_t want = (work_items + EW_THREADS - 1) / EW_THREADS;
  const int64_t cap = (int64_t)sm_count() * 16;
  int64_t g = want < cap ? want : cap;
  return (int)(g < 1 ? 1 : g);
}

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); T v[N]; };

template <typename T>
__device__ __forceinline__ Vec<T> load_vec(const T* p) {
  Vec<T> r;
  *reinterpret_cast<uint4*>(r.v) = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const Vec<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(r.v);
}

// Sigmoid in fp32.  fp32 tensors take the IEEE division; 16-bit tensors take the hardware
// reciprocal (1 ulp in fp32, far below the storage rounding), which keeps the 16-bit kernels
// bound by memory rather than by instruction issue.
template <typename T>
__device__ __forceinline__ float sigmoid_for(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
template <>
__device__ __forceinline__ float sigmoid_for<float>(float x) { return 1.f / (1.f + __expf(-x)); }

// Rounding points follow qwen3_moe_fused/kernels/silu_mul.py:34-39 (forward) and
// :66-73 / :101-111 (backward): f = T(e*sigmoid(e)) with e in fp32; h = f*g, df = dh*g,
// dg = f*dh in T; de = T(f32(df) * sigmoid * (1 + e - e*sigmoid)).
template <typename T>
__device__ __forceinline__ T mul_t(T a, T b) { return from_f32<T>(to_f32(a) * to_f32(b)); }

template <typename T>
__device__ __forceinline__ T silu_fwd_one(T e, T g) {
  const float e32 = to_f32(e);
  const T f = from_f32<T>(e32 * sigmoid_for<T>(e32));
  return mul_t(f, g);
}

template <typename T>
__device__ __forceinline__ void silu_bwd_one(T dh, T e, T g, T& h, T& de, T& dg) {
  const float e32 = to_f32(e);
  const float se = sigmoid_for<T>(e32);
  const float ese = e32 * se;
  const T f = from_f32<T>(ese);
  h = mul_t(f, g);
  const T df = mul_t(dh, g);
  dg = mul_t(f, dh);
  de = from_f32<T>(to_f32(df) * se * (1.f + e32 - ese));
}

// Packed forms for the 16-bit types: two elements per conversion and per multiply.  A packed
// 16-bit multiply rounds the exact product once, which is what mul_t computes.
template <typename T> struct Packed;
template <> struct Packed<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ float2 unpack(type v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ type pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Packed<__half> {
  using type = __half2;
  static __device__ __forceinline__ float2 unpack(type v) { return __half22float2(v); }
  static __device__ __forceinline__ type pack(float a, float b) { return __floats2half2_rn(a, b); }
};

template <typename T>
__device__ __forceinline__ Vec<T> silu_fwd_vec(const Vec<T>& ve, const Vec<T>& vg) {
  Vec<T> vh;
  if constexpr (sizeof(T) == 2) {
    using P = Packed<T>;
    using P2 = typename P::type;
    const P2* e2 = reinterpret_cast<const P2*>(ve.v);
    const P2* g2 = reinterpret_cast<const P2*>(vg.v);
    P2* h2 = reinterpret_cast<P2*>(vh.v);
#pragma unroll
    for (int j = 0; j < Vec<T>::N / 2; ++j) {
      const float2 e = P::unpack(e2[j]);
      const P2 f = P::pack(e.x * sigmoid_for<T>(e.x), e.y * sigmoid_for<T>(e.y));
      h2[j] = __hmul2(f, g2[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < Vec<T>::N; ++j) vh.v[j] = silu_fwd_one(ve.v[j], vg.v[j]);
  }
  return vh;
}

template <typename T>
__device__ __forceinline__ void silu_bwd_vec(const Vec<T>& vdh, const Vec<T>& ve, const Vec<T>& vg,
                                             Vec<T>& vh, Vec<T>& vde, Vec<T>& vdg) {
  if constexpr (sizeof(T) == 2) {
    using P = Packed<T>;
    using P2 = typename P::type;
    const P2* dh2 = reinterpret_cast<const P2*>(vdh.v);
    const P2* e2 = reinterpret_cast<const P2*>(ve.v);
    const P2* g2 = reinterpret_cast<const P2*>(vg.v);
    P2* h2 = reinterpret_cast<P2*>(vh.v);
    P2* de2 = reinterpret_cast<P2*>(vde.v);
    P2* dg2 = reinterpret_cast<P2*>(vdg.v);
#pragma unroll
    for (int j = 0; j < Vec<T>::N / 2; ++j) {
      const float2 e = P::unpack(e2[j]);
      const float s0 = sigmoid_for<T>(e.x), s1 = sigmoid_for<T>(e.y);
      const float es0 = e.x * s0, es1 = e.y * s1;
      const P2 f = P::pack(es0, es1);
      h2[j] = __hmul2(f, g2[j]);
      const float2 df = P::unpack(__hmul2(dh2[j], g2[j]));
      dg2[j] = __hmul2(f, dh2[j]);
      de2[j] = P::pack(df.x * s0 * (1.f + e.x - es0), df.y * s1 * (1.f + e.y - es1));
    }
  } else {
#pragma unroll
    for (int j = 0; j < Vec<T>::N; ++j) silu_bwd_one(vdh.v[j], ve.v[j], vg.v[j], vh.v[j], vde.v[j], vdg.v[j]);
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(EW_THREADS)
silu_fwd_kernel(const T* __restrict__ e, const T* __restrict__ g, T* __restrict__ h, int64_t n) {
  constexpr int V = VEC ? Vec<T>::N : 1;
  const int64_t nv = n / V;
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
  if constexpr (VEC) {
    // two vectors per stream per iteration: four 16-byte loads in flight per thread
    for (; i + stride < nv; i += 2 * stride) {
      const int64_t i2 = i + stride;
      const Vec<T> ve = load_vec(e + i * V), vg = load_vec(g + i * V);
      const Vec<T> ve2 = load_vec(e + i2 * V), vg2 = load_vec(g + i2 * V);
      store_vec(h + i * V, silu_fwd_vec(ve, vg));
      store_vec(h + i2 * V, silu_fwd_vec(ve2, vg2));
    }
  }
  for (; i < nv; i += stride) {
    if constexpr (VEC) {
      store_vec(h + i * V, silu_fwd_vec(load_vec(e + i * V), load_vec(g + i * V)));
    } else {
      h[i] = silu_fwd_one(e[i], g[i]);
    }
  }
  if constexpr (VEC) {  // tail
    const int64_t t = nv * V + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    if (t < n) h[t] = silu_fwd_one(e[t], g[t]);
  }
}

// dh/e/g may alias h/de/dg (in-place form), so no __restrict__ here.
template <typename T, bool VEC, bool WRITE_H>
__global__ void __launch_bounds__(EW_THREADS)
silu_bwd_kernel(const T* dh, const T* e, const T* g, T* h, T* de, T* dg, int64_t n) {
  constexpr int V = VEC ? Vec<T>::N : 1;
  const int64_t nv = n / V;
  for (int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < nv; i += (int64_t)gridDim.x * EW_THREADS) {
    if constexpr (VEC) {
      const Vec<T> vdh = load_vec(dh + i * V), ve = load_vec(e + i * V), vg = load_vec(g + i * V);
      Vec<T> vh, vde, vdg;
      silu_bwd_vec(vdh, ve, vg, vh, vde, vdg);
      if constexpr (WRITE_H) store_vec(h + i * V, vh);
      store_vec(de + i * V, vde);
      store_vec(dg + i * V, vdg);
    } else {
      T oh, ode, odg;
      silu_bwd_one(dh[i], e[i], g[i], oh, ode, odg);
      if constexpr (WRITE_H) h[i] = oh;
      de[i] = ode;
      dg[i] = odg;
    }
  }
  if constexpr (VEC) {
    const int64_t t = nv * V + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    if (t < n) {
      T oh, ode, odg;
      silu_bwd_one(dh[t], e[t], g[t], oh, ode, odg);
      if constexpr (WRITE_H) h[t] = oh;
      de[t] = ode;
      dg[t] = odg;
    }
  }
}

// Double-quantised ("nested") absmax -> fp32 absmax: out[i] = code2[q[i]] * absmax2[i / blocksize2]
// + offset, the product and the sum each rounded to fp32 (what dequantize_blockwise followed by
// `+= offset` computes at qwen3_moe_fused/grouped_gemm/forward_4bit.py:149-153).
__global__ void __launch_bounds__(EW_THREADS)
absmax_unnest_kernel(const uint8_t* __restrict__ q, const float* __restrict__ code2, const float* __restrict__ absmax2,
                     int bs_shift, const float* __restrict__ offset, float* __restrict__ out, int64_t n) {
  __shared__ float tbl[256];
  for (int i = threadIdx.x; i < 256; i += EW_THREADS) tbl[i] = code2[i];
  __syncthreads();
  const float off = offset ? __ldg(offset) : 0.f;
  const bool vec = ((reinterpret_cast<uintptr_t>(q) & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  const int64_t groups = vec ? n / 4 : 0;
  for (int64_t g = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; g < groups; g += stride) {
    const uint32_t raw = __ldg(reinterpret_cast<const uint32_t*>(q) + g);
    float4 v;
    float* pv = reinterpret_cast<float*>(&v);
#pragma unroll
    for (int b = 0; b < 4; ++b)
      pv[b] = __fadd_rn(__fmul_rn(tbl[(raw >> (8 * b)) & 0xffu], __ldg(absmax2 + ((g * 4 + b) >> bs_shift))), off);
    reinterpret_cast<float4*>(out)[g] = v;
  }
  for (int64_t i = groups * 4 + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n; i += stride)
    out[i] = __fadd_rn(__fmul_rn(tbl[q[i]], __ldg(absmax2 + (i >> bs_shift))), off);
}

// NF4 decode, 8 weights (4 packed bytes) per thread iteration: a warp reads 128 contiguous
// bytes and, for 16-bit outputs, writes 512 contiguous bytes per store instruction.
// Element 2j is the high nibble of byte j, element 2j+1 the low nibble
// (qwen3_moe_fused/grouped_gemm/forward_4bit.py:99-104).
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
nf4_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ code,
                   const float* __restrict__ absmax, int bs_shift, T* __restrict__ out,
                   int64_t n_elems, bool vec_ok) {
  __shared__ float tbl[16];
  if (threadIdx.x < 16) tbl[threadIdx.x] = code[threadIdx.x];
  __syncthreads();
  const int64_t ngroups = vec_ok ? n_elems / 8 : 0;
  const bool one_scale = bs_shift >= 3;  // the 8 elements of a group share one absmax block
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  auto decode_store = [&](int64_t gi, uint32_t raw, float a_all) {
    const int64_t base = gi * 8;
    T vals[8];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (raw >> (b * 8)) & 0xffu;
      const float a0 = one_scale ? a_all : absmax[(base + 2 * b) >> bs_shift];
      const float a1 = one_scale ? a_all : absmax[(base + 2 * b + 1) >> bs_shift];
      vals[2 * b] = from_f32<T>(tbl[byte >> 4] * a0);
      vals[2 * b + 1] = from_f32<T>(tbl[byte & 15] * a1);
    }
    constexpr int NV = 8 * sizeof(T) / 16;
#pragma unroll
    for (int v = 0; v < NV; ++v)
      __stcs(reinterpret_cast<uint4*>(out + base) + v, reinterpret_cast<const uint4*>(vals)[v]);
  };
  int64_t gi = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
  // four groups per step: their loads are issued together
  for (; gi + 3 * stride < ngroups; gi += 4 * stride) {
    uint32_t raw[4];
    float am[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      raw[u] = __ldcs(reinterpret_cast<const uint32_t*>(packed) + gi + u * stride);
      am[u] = __ldg(absmax + (((gi + u * stride) * 8) >> bs_shift));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) decode_store(gi + u * stride, raw[u], am[u]);
  }
  for (; gi < ngroups; gi += stride)
    decode_store(gi, __ldcs(reinterpret_cast<const uint32_t*>(packed) + gi), __ldg(absmax + ((gi * 8) >> bs_shift)));
  // scalar remainder (or everything when the buffers are not 16-byte aligned)
  const int64_t start = ngroups * 8;
  for (int64_t i = start + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x; i < n_elems; i += (int64_t)gridDim.x * EW_THREADS) {
    const uint8_t byte = packed[i >> 1];
    const int nib = (i & 1) ? (byte & 15) : (byte >> 4);
    out[i] = from_f32<T>(tbl[nib] * absmax[i >> bs_shift]);
  }
}

// 16-byte load that asks L2 to keep the line (token rows are read k times each, while the
// output streams through the cache).
__device__ __forceinline__ uint64_t l2_keep_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ld_keep(const uint4* ptr, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr), "l"(policy));
  return v;
}

// out[j,:] = hidden[sort_idx[j] / k, :].  Vector form: one warp per output row, up to eight
// 16-byte loads in flight per lane, and the index of the warp's next row is fetched before the
// current row is copied (the index -> row -> store chain is what bounds this kernel otherwise).
template <typename T, bool VEC>
__global__ void __launch_bounds__(EW_THREADS)
gather_rows_kernel(const T* __restrict__ hidden, const int32_t* __restrict__ sort_idx, int k,
                   T* __restrict__ out, int64_t rows, int H) {
  if constexpr (VEC) {
    constexpr int UNROLL = 8;
    const int row_vecs = H / Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (EW_THREADS / 32);
    int64_t j = (int64_t)blockIdx.x * (EW_THREADS / 32) + (threadIdx.x >> 5);
    const uint64_t keep = l2_keep_policy();
    int idx = j < rows ? sort_idx[j] : 0;
    for (; j < rows; j += warps) {
      const int64_t jn = j + warps;
      const int idx_next = jn < rows ? sort_idx[jn] : 0;
      const uint4* src = reinterpret_cast<const uint4*>(hidden + (int64_t)(idx / k) * H);
      uint4* dst = reinterpret_cast<uint4*>(out + j * H);
      for (int c0 = 0; c0 < row_vecs; c0 += 32 * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int c = c0 + u * 32 + lane;
          if (c < row_vecs) v[u] = ld_keep(src + c, keep);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int c = c0 + u * 32 + lane;
          if (c < row_vecs) __stcs(dst + c, v[u]);  // streaming: keep the re-read token rows in L2, not the output
        }
      }
      idx = idx_next;
    }
  } else {
    for (int64_t j = blockIdx.x; j < rows; j += gridDim.x) {
      const T* src = hidden + (int64_t)(sort_idx[j] / k) * H;
      T* dst = out + j * H;
      for (int c = threadIdx.x; c < H; c += EW_THREADS) dst[c] = src[c];
    }
  }
}

// out[inv_sort_idx[t*k + j], :] = hidden[t, :]: the same result as gather_rows, produced token by
// token, so every token row is read from memory exactly once (the gather form re-reads each row
// k times, and the output stream pushes the rows out of L2 in between).  One warp per token.
template <typename T, bool VEC>
__global__ void __launch_bounds__(EW_THREADS)
expand_rows_kernel(const T* __restrict__ hidden, const int32_t* __restrict__ inv_sort_idx, int k,
                   T* __restrict__ out, int64_t tokens, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (EW_THREADS / 32);
  for (int64_t t = (int64_t)blockIdx.x * (EW_THREADS / 32) + (threadIdx.x >> 5); t < tokens; t += warps) {
    if constexpr (VEC) {
      constexpr int UNROLL = 8;
      const int row_vecs = H / Vec<T>::N;
      const uint4* src = reinterpret_cast<const uint4*>(hidden + t * H);
      for (int c0 = 0; c0 < row_vecs; c0 += 32 * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int c = c0 + u * 32 + lane;
          if (c < row_vecs) v[u] = __ldcs(src + c);
        }
        for (int j0 = 0; j0 < k; j0 += 32) {
          const int mine = j0 + lane < k ? inv_sort_idx[t * k + j0 + lane] : 0;
          const int nj = min(32, k - j0);
          for (int j = 0; j < nj; ++j) {
            uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)__shfl_sync(0xffffffffu, mine, j) * H);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
              const int c = c0 + u * 32 + lane;
              if (c < row_vecs) __stcs(dst + c, v[u]);
            }
          }
        }
      }
    } else {
      for (int j = 0; j < k; ++j) {
        T* dst = out + (int64_t)inv_sort_idx[t * k + j] * H;
        for (int c = lane; c < H; c += 32) dst[c] = hidden[t * H + c];
      }
    }
  }
}

// out[t,:] = T( sum_j f32(weights[t,j]) * f32(y[inv_sort_idx[t*k+j],:]) )
// KFIX > 0 fixes k at compile time so that the k row loads of a thread are all in flight.
template <typename T, bool VEC, int KFIX>
__global__ void __launch_bounds__(EW_THREADS)
combine_kernel(const T* __restrict__ y, const int32_t* __restrict__ inv_sort_idx,
               const T* __restrict__ weights, T* __restrict__ out, int64_t tokens, int k_rt, int H) {
  constexpr int V = VEC ? Vec<T>::N : 1;
  const int k = KFIX > 0 ? KFIX : k_rt;
  const int hv = H / V;
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    if constexpr (KFIX > 0 && VEC) {
      int64_t src[KFIX];
      float wj[KFIX];
#pragma unroll
      for (int j = 0; j < KFIX; ++j) {
        src[j] = inv_sort_idx[t * KFIX + j];
        wj[j] = to_f32(weights[t * KFIX + j]);
      }
      for (int c = threadIdx.x; c < hv; c += EW_THREADS) {
        Vec<T> v[KFIX];
#pragma unroll
        for (int j = 0; j < KFIX; ++j) v[j] = load_vec(y + src[j] * H + c * V);
        Vec<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < KFIX; ++j) acc = fmaf(wj[j], to_f32(v[j].v[i]), acc);  // same order as the generic loop
          o.v[i] = from_f32<T>(acc);
        }
        store_vec(out + t * H + c * V, o);
      }
      continue;
    }
    for (int c = threadIdx.x; c < hv; c += EW_THREADS) {
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int64_t src = inv_sort_idx[t * k + j];
        const float wj = to_f32(weights[t * k + j]);
        if constexpr (VEC) {
          const Vec<T> v = load_vec(y + src * H + c * V);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = fmaf(wj, to_f32(v.v[i]), acc[i]);
        } else {
          acc[0] = fmaf(wj, to_f32(y[src * H + c]), acc[0]);
        }
      }
      if constexpr (VEC) {
        Vec<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) o.v[i] = from_f32<T>(acc[i]);
        store_vec(out + t * H + c * V, o);
      } else {
        out[t * H + c] = from_f32<T>(acc[0]);
      }
    }
  }
}

static inline int ilog2_exact(int v) {
  if (v <= 0 || (v & (v - 1)) != 0) return -1;
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

}  // namespace moe

using namespace moe;

MOE_API int moe_silu_mul_fwd(const void* e, const void* g, void* h, int64_t n, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (n < 0) return MOE_ERR_SHAPE;
  if (n == 0) return MOE_OK;
  if (!e || !g || !h) return MOE_ERR_NULL;
  const bool vec = aligned16(e) && aligned16(g) && aligned16(h);
  MOE_DISPATCH_FLOAT(dtype, T, {
    const int64_t items = vec ? (n + Vec<T>::N - 1) / Vec<T>::N : n;
    if (vec) silu_fwd_kernel<T, true><<<ew_grid(items), EW_THREADS, 0, stream>>>((const T*)e, (const T*)g, (T*)h, n);
    else silu_fwd_kernel<T, false><<<ew_grid(items), EW_THREADS, 0, stream>>>((const T*)e, (const T*)g, (T*)h, n);
  });
  return launch_status();
}

static int silu_bwd_impl(const void* dh, const void* e, const void* g, void* h, void* de, void* dg,
                         int64_t n, int dtype, bool write_h, cudaStream_t stream) {
  if (n < 0) return MOE_ERR_SHAPE;
  if (n == 0) return MOE_OK;
  if (!dh || !e || !g || !de || !dg || (write_h && !h)) return MOE_ERR_NULL;
  const bool vec = aligned16(dh) && aligned16(e) && aligned16(g) && aligned16(de) && aligned16(dg) && (!write_h || aligned16(h));
  MOE_DISPATCH_FLOAT(dtype, T, {
    const int64_t items = vec ? (n + Vec<T>::N - 1) / Vec<T>::N : n;
    const int grid = ew_grid(items);
    // The tail of the vector form is handled by the first CTAs; it needs at least
    // Vec::N-1 threads in total, which one CTA always has.
    if (vec && write_h) silu_bwd_kernel<T, true, true><<<grid, EW_THREADS, 0, stream>>>((const T*)dh, (const T*)e, (const T*)g, (T*)h, (T*)de, (T*)dg, n);
    else if (vec) silu_bwd_kernel<T, true, false><<<grid, EW_THREADS, 0, stream>>>((const T*)dh, (const T*)e, (const T*)g, (T*)h, (T*)de, (T*)dg, n);
    else if (write_h) silu_bwd_kernel<T, false, true><<<grid, EW_THREADS, 0, stream>>>((const T*)dh, (const T*)e, (const T*)g, (T*)h, (T*)de, (T*)dg, n);
    else silu_bwd_kernel<T, false, false><<<grid, EW_THREADS, 0, stream>>>((const T*)dh, (const T*)e, (const T*)g, (T*)h, (T*)de, (T*)dg, n);
  });
  return launch_status();
}

MOE_API int moe_silu_mul_bwd(const void* dh, const void* e, const void* g, void* de, void* dg,
                             int64_t n, int dtype, void* stream) {
  return silu_bwd_impl(dh, e, g, nullptr, de, dg, n, dtype, false, (cudaStream_t)stream);
}

MOE_API int moe_silu_mul_bwd_inplace(void* dh, void* e, void* g, int64_t n, int dtype, void* stream) {
  // (dh, e, g) <- (h, de, dg): every element is read before it is overwritten by the
  // same thread, so aliasing inputs and outputs is safe.
  return silu_bwd_impl(dh, e, g, dh, e, g, n, dtype, true, (cudaStream_t)stream);
}

MOE_API int moe_absmax_unnest(const uint8_t* q, const float* code2, const float* absmax2, int blocksize2,
                              const float* offset, float* out, int64_t n, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const int shift = ilog2_exact(blocksize2);
  if (shift < 0 || n < 0) return MOE_ERR_SHAPE;
  if (n == 0) return MOE_OK;
  if (!q || !code2 || !absmax2 || !out) return MOE_ERR_NULL;
  absmax_unnest_kernel<<<ew_grid((n + 3) / 4), EW_THREADS, 0, stream>>>(q, code2, absmax2, shift, offset, out, n);
  return launch_status();
}

MOE_API int moe_nf4_dequant(const uint8_t* packed, const float* code, const float* absmax, int blocksize,
                            void* out, int64_t n_elems, int dtype_out, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const int shift = ilog2_exact(blocksize);
  if (shift < 0 || n_elems < 0 || (n_elems & 1)) return MOE_ERR_SHAPE;
  if (n_elems == 0) return MOE_OK;
  if (!packed || !code || !absmax || !out) return MOE_ERR_NULL;
  const bool vec_ok = (((uintptr_t)packed & 3) == 0) && aligned16(out);
  MOE_DISPATCH_FLOAT(dtype_out, T, {
    nf4_dequant_kernel<T><<<ew_grid((n_elems + 7) / 8), EW_THREADS, 0, stream>>>(
        packed, code, absmax, shift, (T*)out, n_elems, vec_ok);
  });
  return launch_status();
}

MOE_API int moe_gather_rows(const void* hidden, const int32_t* sort_idx, int k, void* out,
                            int64_t rows, int H, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (rows < 0 || H < 0 || k <= 0) return MOE_ERR_SHAPE;
  if (rows == 0 || H == 0) return MOE_OK;
  if (!hidden || !sort_idx || !out) return MOE_ERR_NULL;
  MOE_DISPATCH_FLOAT(dtype, T, {
    const bool vec = aligned16(hidden) && aligned16(out) && (H % Vec<T>::N == 0);
    // vector form: a warp per row (8 rows per CTA per pass); scalar form: a CTA per row
    const int64_t want = vec ? (rows + EW_THREADS / 32 - 1) / (EW_THREADS / 32) : rows;
    const int64_t cap = (int64_t)sm_count() * (vec ? 8 : 16);
    const int grid = (int)(want < cap ? want : cap);
    if (vec) gather_rows_kernel<T, true><<<grid, EW_THREADS, 0, stream>>>((const T*)hidden, sort_idx, k, (T*)out, rows, H);
    else gather_rows_kernel<T, false><<<grid, EW_THREADS, 0, stream>>>((const T*)hidden, sort_idx, k, (T*)out, rows, H);
  });
  return launch_status();
}

MOE_API int moe_expand_rows(const void* hidden, const int32_t* inv_sort_idx, int k, void* out,
                            int64_t tokens, int H, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (tokens < 0 || H < 0 || k <= 0) return MOE_ERR_SHAPE;
  if (tokens == 0 || H == 0) return MOE_OK;
  if (!hidden || !inv_sort_idx || !out) return MOE_ERR_NULL;
  const int64_t want = (tokens + EW_THREADS / 32 - 1) / (EW_THREADS / 32);
  const int64_t cap = (int64_t)sm_count() * 8;
  const int grid = (int)(want < cap ? want : cap);
  MOE_DISPATCH_FLOAT(dtype, T, {
    const bool vec = aligned16(hidden) && aligned16(out) && (H % Vec<T>::N == 0);
    if (vec) expand_rows_kernel<T, true><<<grid, EW_THREADS, 0, stream>>>((const T*)hidden, inv_sort_idx, k, (T*)out, tokens, H);
    else expand_rows_kernel<T, false><<<grid, EW_THREADS, 0, stream>>>((const T*)hidden, inv_sort_idx, k, (T*)out, tokens, H);
  });
  return launch_status();
}

MOE_API int moe_combine(const void* y, const int32_t* inv_sort_idx, const void* weights, void* out,
                        int64_t T_, int k, int H, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (T_ < 0 || H < 0 || k <= 0) return MOE_ERR_SHAPE;
  if (T_ == 0 || H == 0) return MOE_OK;
  if (!y || !inv_sort_idx || !weights || !out) return MOE_ERR_NULL;
  const int64_t g64 = T_ < (int64_t)sm_count() * 16 ? T_ : (int64_t)sm_count() * 16;
  const int grid = (int)g64;
  MOE_DISPATCH_FLOAT(dtype, T, {
    const bool vec = aligned16(y) && aligned16(out) && (H % Vec<T>::N == 0);
    if (vec && k == 8) combine_kernel<T, true, 8><<<grid, EW_THREADS, 0, stream>>>((const T*)y, inv_sort_idx, (const T*)weights, (T*)out, T_, k, H);
    else if (vec) combine_kernel<T, true, 0><<<grid, EW_THREADS, 0, stream>>>((const T*)y, inv_sort_idx, (const T*)weights, (T*)out, T_, k, H);
    else combine_kernel<T, false, 0><<<grid, EW_THREADS, 0, stream>>>((const T*)y, inv_sort_idx, (const T*)weights, (T*)out, T_, k, H);
  });
  return launch_status();
}
