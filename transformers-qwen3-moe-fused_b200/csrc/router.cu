// Router: fp32 softmax over the E logits of a token, top-k by (probability descending,
// expert id ascending), optional renormalisation over the k winners, cast to the
// activation dtype.  One warp per token; every lane keeps E/32 probabilities in
// registers (expert id = lane + 32*i, so logits are read with coalesced accesses) and
// the k arg-max rounds are warp-shuffle reductions.
// Stands in for the softmax / topk / divide / cast sequence at
// qwen3_moe_fused/modular_qwen3_moe_fused.py:87-93.
#include <math_constants.h>

#include "common.cuh"

namespace moe {

constexpr int RT_WARPS = 8;

template <typename TL, typename TW, int NPL>
__global__ void __launch_bounds__(RT_WARPS * 32)
router_kernel(const TL* __restrict__ logits, int64_t T, int E, int k, int norm,
              TW* __restrict__ weights, int64_t* __restrict__ experts) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * RT_WARPS + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * RT_WARPS;
  for (int64_t t = warp_global; t < T; t += warp_stride) {
    const TL* row = logits + t * E;
    float p[NPL];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      p[i] = e < E ? to_f32(row[e]) : -CUDART_INF_F;
      mx = fmaxf(mx, p[i]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      p[i] = e < E ? expf(p[i] - mx) : 0.f;
      sum += p[i];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      p[i] = e < E ? p[i] * inv : -1.f;  // -1 never wins against a probability
    }
    // k rounds of arg-max.
    float top_sum = 0.f;
    float my_w = 0.f;
    int my_e = 0;
    for (int r = 0; r < k; ++r) {
      float bv = -2.f;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int e = lane + 32 * i;
        if (p[i] > bv) { bv = p[i]; be = e; }  // ascending e inside a lane: first hit wins
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, d);
        const int oe = __shfl_xor_sync(0xffffffffu, be, d);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      // remove the winner
#pragma unroll
      for (int i = 0; i < NPL; ++i)
        if (lane + 32 * i == be) p[i] = -1.f;
      top_sum += bv;
      if (r == lane) { my_w = bv; my_e = be; }  // lane r keeps the r-th winner (k <= 32)
    }
    if (lane < k) {
      experts[t * k + lane] = (int64_t)my_e;
      // Same operation as the reference: each probability divided by the winners' sum.
      weights[t * k + lane] = from_f32<TW>(norm ? my_w / top_sum : my_w);
    }
  }
}

// k is limited to 32 (one winner per lane); Qwen3-MoE uses 8.

// Faster form for k <= 8: eight lanes per token (four tokens per warp), E/8 logits per lane.
// The winners are chosen on the logits (the same order as on the probabilities, without the
// rounding of exp in between); only the softmax denominator needs every exponential.
//
// Logits are mapped to unsigned keys that sort like the floats, so that a lane's maximum is a
// tree of integer max instructions (no serial compare-select chain) and the maximum over the
// token's eight lanes is three shuffle steps; the winner's expert id (lowest id among equal
// keys) is a second three-step minimum.  (redux.sync with one mask per group of eight lanes
// was measured slower than the shuffles.)
// VLOAD: every lane reads four consecutive logits per access (needs E % 32 == 0 and 16-byte
// aligned rows); expert ids are ascending in v inside a lane under both mappings.
__device__ __forceinline__ uint32_t router_key(float x) {
  const uint32_t u = __float_as_uint(x + 0.0f);  // -0 and +0 share a key, as they compare equal
  return u ^ ((uint32_t)((int32_t)u >> 31) | 0x80000000u);
}
__device__ __forceinline__ float router_unkey(uint32_t key) {
  return __uint_as_float(key ^ ((uint32_t)((int32_t)~key >> 31) | 0x80000000u));
}

template <typename TL, int NV, bool VLOAD>
__device__ __forceinline__ void router_load(const TL* __restrict__ row, int sub, int E, bool live, float (&x)[NV]) {
  if constexpr (VLOAD) {
#pragma unroll
    for (int q = 0; q < NV / 4; ++q) {
      const TL* p = row + 32 * q + 4 * sub;
      if constexpr (sizeof(TL) == 4) {
        const float4 v = live ? *reinterpret_cast<const float4*>(p) : make_float4(0.f, 0.f, 0.f, 0.f);
        x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
      } else {
        TL t[4];
        *reinterpret_cast<uint2*>(t) = live ? *reinterpret_cast<const uint2*>(p) : make_uint2(0u, 0u);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[4 * q + j] = to_f32(t[j]);
      }
    }
  } else {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int e = sub + 8 * v;
      x[v] = (live && e < E) ? to_f32(row[e]) : 0.f;
    }
  }
}

template <typename TL, typename TW, int NV, bool VLOAD>
__global__ void __launch_bounds__(RT_WARPS * 32)
router8_kernel(const TL* __restrict__ logits, int64_t T, int E, int k, int norm,
               TW* __restrict__ weights, int64_t* __restrict__ experts) {
  const int lane = threadIdx.x & 31;
  const int sub = lane & 7;                 // lane inside the token's group of 8
  const int64_t group_global = ((int64_t)blockIdx.x * (RT_WARPS * 32) + threadIdx.x) >> 3;
  const int64_t group_stride = ((int64_t)gridDim.x * (RT_WARPS * 32)) >> 3;
  auto expert_of = [&](int v) { return VLOAD ? 32 * (v >> 2) + 4 * sub + (v & 3) : sub + 8 * v; };
  for (int64_t t0 = group_global - (lane >> 3); t0 < T; t0 += group_stride) {
    // t0 is the first token of this warp's four; all lanes of the warp loop together
    const int64_t t = t0 + (lane >> 3);
    const bool live = t < T;
    float x[NV];
    router_load<TL, NV, VLOAD>(logits + (live ? t : 0) * E, sub, E, live, x);
    uint32_t key[NV];  // 0 = absent (padding past E, or already taken); every real logit has a key > 0
#pragma unroll
    for (int v = 0; v < NV; ++v) key[v] = expert_of(v) < E ? router_key(x[v]) : 0u;
    auto lane_max = [&]() {
      uint32_t m[NV];
#pragma unroll
      for (int v = 0; v < NV; ++v) m[v] = key[v];
#pragma unroll
      for (int w = NV / 2; w > 0; w >>= 1)
#pragma unroll
        for (int v = 0; v < w; ++v) m[v] = max(m[v], m[v + w]);
      return m[0];
    };
    auto group_max = [&](uint32_t v) {
#pragma unroll
      for (int d = 4; d > 0; d >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, d));
      return v;
    };
    auto group_min = [&](uint32_t v) {
#pragma unroll
      for (int d = 4; d > 0; d >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, d));
      return v;
    };
    const float mx = router_unkey(group_max(lane_max()));
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) sum += key[v] != 0u ? __expf(x[v] - mx) : 0.f;
#pragma unroll
    for (int d = 4; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    float top_sum = 0.f, my_p = 0.f;
    int my_e = 0;
    for (int r = 0; r < k; ++r) {
      const uint32_t best = group_max(lane_max());
      // lowest expert id among the keys equal to the best one: scan down so the lowest v stays
      uint32_t cand = 0x7fffffffu;
#pragma unroll
      for (int v = NV - 1; v >= 0; --v) cand = key[v] == best ? (uint32_t)expert_of(v) : cand;
      const int be = (int)group_min(cand);
#pragma unroll
      for (int v = 0; v < NV; ++v) key[v] = expert_of(v) == be ? 0u : key[v];
      const float pr = __expf(router_unkey(best) - mx) / sum;  // softmax probability of the winner
      top_sum += pr;
      if (r == sub) { my_p = pr; my_e = be; }
    }
    if (live && sub < k) {
      experts[t * k + sub] = (int64_t)my_e;
      weights[t * k + sub] = from_f32<TW>(norm ? my_p / top_sum : my_p);
    }
  }
}

// One warp per token, E / 32 logits per lane (at most 8).  Every lane sorts its few keys once
// (descending, equal keys by ascending expert id); a round then takes the best of the 32 list
// heads with one full-warp redux.sync (max of the keys), resolves equal keys with a second one
// (min of the expert ids among the lanes whose head is the best key), and only the winning lane
// advances its list.
// VLOAD: lane l reads logits 4l..4l+3 of every block of 128 (needs E % 128 == 0, aligned rows).
template <typename TL, typename TW, int NPL, bool VLOAD>
__global__ void __launch_bounds__(RT_WARPS * 32)
router_warp_kernel(const TL* __restrict__ logits, int64_t T, int E, int k, int norm,
                   TW* __restrict__ weights, int64_t* __restrict__ experts) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * RT_WARPS + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * RT_WARPS;
  auto expert_of = [&](int v) { return VLOAD ? 128 * (v >> 2) + 4 * lane + (v & 3) : lane + 32 * v; };
  for (int64_t t = warp_global; t < T; t += warp_stride) {
    const TL* row = logits + t * E;
    float x[NPL];
    if constexpr (VLOAD) {
#pragma unroll
      for (int q = 0; q < NPL / 4; ++q) {
        const TL* p = row + 128 * q + 4 * lane;
        if constexpr (sizeof(TL) == 4) {
          const float4 v = *reinterpret_cast<const float4*>(p);
          x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
        } else {
          TL tmp[4];
          *reinterpret_cast<uint2*>(tmp) = *reinterpret_cast<const uint2*>(p);
#pragma unroll
          for (int j = 0; j < 4; ++j) x[4 * q + j] = to_f32(tmp[j]);
        }
      }
    } else {
#pragma unroll
      for (int v = 0; v < NPL; ++v) x[v] = expert_of(v) < E ? to_f32(row[expert_of(v)]) : 0.f;
    }
    uint32_t key[NPL];
    int eid[NPL];
#pragma unroll
    for (int v = 0; v < NPL; ++v) {
      eid[v] = expert_of(v);
      key[v] = eid[v] < E ? router_key(x[v]) : 0u;  // 0 = absent; every real logit has a key > 0
    }
    // bubble sort (adjacent exchanges on strictly greater keys only: equal keys keep ascending ids)
#pragma unroll
    for (int pass = 0; pass < NPL - 1; ++pass)
#pragma unroll
      for (int v = 0; v < NPL - 1 - pass; ++v) {
        const bool sw = key[v + 1] > key[v];
        const uint32_t ka = key[v], kb = key[v + 1];
        const int ea = eid[v], eb = eid[v + 1];
        key[v] = sw ? kb : ka; key[v + 1] = sw ? ka : kb;
        eid[v] = sw ? eb : ea; eid[v + 1] = sw ? ea : eb;
      }
    const float mx = router_unkey(__reduce_max_sync(0xffffffffu, key[0]));
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < NPL; ++v) sum += key[v] != 0u ? __expf(router_unkey(key[v]) - mx) : 0.f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    uint32_t my_key = 0u;
    int my_e = 0;
    for (int r = 0; r < k; ++r) {
      const uint32_t best = __reduce_max_sync(0xffffffffu, key[0]);
      const uint32_t cand = key[0] == best ? (uint32_t)eid[0] : 0x7fffffffu;
      const uint32_t be = __reduce_min_sync(0xffffffffu, cand);
      const bool won = cand == be;
#pragma unroll
      for (int v = 0; v < NPL - 1; ++v) {
        key[v] = won ? key[v + 1] : key[v];
        eid[v] = won ? eid[v + 1] : eid[v];
      }
      key[NPL - 1] = won ? 0u : key[NPL - 1];
      if (lane == r) { my_key = best; my_e = (int)be; }  // lane r keeps the r-th winner (k <= 32)
    }
    const float pr = lane < k ? __expf(router_unkey(my_key) - mx) / sum : 0.f;
    float top_sum = pr;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) top_sum += __shfl_xor_sync(0xffffffffu, top_sum, d);
    if (lane < k) {
      experts[t * k + lane] = (int64_t)my_e;
      weights[t * k + lane] = from_f32<TW>(norm ? pr / top_sum : pr);
    }
  }
}

template <typename TL, typename TW>
static int launch_router(const void* logits, int64_t T, int E, int k, int norm, void* weights,
                         int64_t* experts, cudaStream_t stream) {
  const int64_t want = (T + RT_WARPS - 1) / RT_WARPS;
  const int64_t cap = (int64_t)sm_count() * 8;
  const int grid = (int)(want < cap ? want : cap);
  // Measured on B200 at E = 128, k = 8: the warp-per-token form is faster while the launch is
  // latency-bound (10 / 14 us against 11 / 15 us at 8192 / 16384 tokens), the eight-lane form when
  // it is issue-bound (0.46 against 0.50 ms at 1 M tokens).
  const bool small = T <= 131072 || k > 8;
  if (small && E <= 8 * 32 && E >= k && E >= 32) {
    // a warp per token, at most eight logits per lane
    const int npl = (E + 31) / 32;
    const bool vload = (E % 128) == 0 && (((uintptr_t)logits) & 15) == 0;
#define MOE_RTW_CASE(NPL)                                                                                         \
  do {                                                                                                            \
    if (vload && (NPL) % 4 == 0 && (NPL) * 32 == E)                                                               \
      router_warp_kernel<TL, TW, NPL, true><<<grid, RT_WARPS * 32, 0, stream>>>((const TL*)logits, T, E, k, norm, \
                                                                                (TW*)weights, experts);           \
    else                                                                                                          \
      router_warp_kernel<TL, TW, NPL, false><<<grid, RT_WARPS * 32, 0, stream>>>((const TL*)logits, T, E, k, norm, \
                                                                                 (TW*)weights, experts);          \
  } while (0)
    if (npl <= 1) MOE_RTW_CASE(1);
    else if (npl <= 2) MOE_RTW_CASE(2);
    else if (npl <= 4) MOE_RTW_CASE(4);
    else MOE_RTW_CASE(8);
#undef MOE_RTW_CASE
    return launch_status();
  }
  if (k <= 8 && E <= 8 * 64 && E >= k) {
    const int64_t want8 = (T + 31) / 32;  // 32 tokens per CTA
    const int grid8 = (int)(want8 < cap ? want8 : cap);
    const int nv = (E + 7) / 8;
    const bool vload = (E % 32) == 0 && (((uintptr_t)logits) & 15) == 0;
#define MOE_RT8_CASE(NV)                                                                                         \
  do {                                                                                                           \
    if (vload && (NV) % 4 == 0 && (NV) * 8 == E)                                                                 \
      router8_kernel<TL, TW, NV, true><<<grid8, RT_WARPS * 32, 0, stream>>>((const TL*)logits, T, E, k, norm,    \
                                                                            (TW*)weights, experts);              \
    else                                                                                                         \
      router8_kernel<TL, TW, NV, false><<<grid8, RT_WARPS * 32, 0, stream>>>((const TL*)logits, T, E, k, norm,   \
                                                                             (TW*)weights, experts);             \
  } while (0)
    if (nv <= 2) MOE_RT8_CASE(2);
    else if (nv <= 4) MOE_RT8_CASE(4);
    else if (nv <= 8) MOE_RT8_CASE(8);
    else if (nv <= 16) MOE_RT8_CASE(16);
    else if (nv <= 32) MOE_RT8_CASE(32);
    else MOE_RT8_CASE(64);
#undef MOE_RT8_CASE
    return launch_status();
  }
  const int npl = (E + 31) / 32;
#define MOE_RT_CASE(NPL)                                                                           \
  router_kernel<TL, TW, NPL><<<grid, RT_WARPS * 32, 0, stream>>>((const TL*)logits, T, E, k, norm, \
                                                                 (TW*)weights, experts)
  if (npl <= 1) MOE_RT_CASE(1);
  else if (npl <= 2) MOE_RT_CASE(2);
  else if (npl <= 4) MOE_RT_CASE(4);
  else if (npl <= 8) MOE_RT_CASE(8);
  else if (npl <= 16) MOE_RT_CASE(16);
  else MOE_RT_CASE(32);
#undef MOE_RT_CASE
  return launch_status();
}

}  // namespace moe

using namespace moe;

MOE_API int moe_router_softmax_topk(const void* logits, int dtype_logits, int64_t T, int E, int k,
                                    int norm_topk, void* weights, int dtype_w, int64_t* experts,
                                    void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (T < 0 || E <= 0 || E > 1024 || k <= 0 || k > E || k > 32) return MOE_ERR_SHAPE;
  if (T == 0) return MOE_OK;
  if (!logits || !weights || !experts) return MOE_ERR_NULL;
  MOE_DISPATCH_FLOAT(dtype_logits, TL, {
    MOE_DISPATCH_FLOAT(dtype_w, TW, { return launch_router<TL, TW>(logits, T, E, k, norm_topk, weights, experts, stream); });
  });
  return MOE_ERR_DTYPE;
}
