// CUDA-core grouped GEMMs: correct for every shape, dtype and alignment.
//
// They serve (1) fp32 inputs, which are multiplied in full fp32 (no TF32 rounding),
// (2) shapes the tensor-core kernels cannot take (row pitch not a multiple of 16 bytes,
// very thin N or K), and (3) as the on-device anchor the tcgen05 kernels are checked
// against.  64x64 output tile, 16-deep shared-memory slices, 4x4 micro-tile per thread.
#include "common.cuh"

namespace moe {

constexpr int ST_BM = 64, ST_BN = 64, ST_BK = 16, ST_THREADS = 256;

// Weight element readers.  `k_fastest` tells the kernel which index is contiguous in
// memory so that the tile loads are coalesced.
template <typename TIn>
struct DenseWeight {  // w[e*se + n*sn + k*sk]; forward: sn = K, sk = 1; dX ((E,K,N) storage): sn = 1, sk = N
  const TIn* w; int64_t se, sn, sk;
  __device__ __forceinline__ bool k_fastest() const { return sk == 1; }
  __device__ __forceinline__ float load(int e, int n, int k) const { return to_f32(w[e * se + n * sn + k * sk]); }
};
template <typename TIn>
struct Nf4Weight {  // (E,N,K) NF4: high nibble = even element, absmax per `1 << shift` flat elements
  const uint8_t* packed; const float* code; const float* absmax; int shift; int64_t N, K;
  __device__ __forceinline__ bool k_fastest() const { return true; }
  __device__ __forceinline__ float load(int e, int n, int k) const {
    const int64_t flat = ((int64_t)e * N + n) * K + k;
    const uint8_t byte = packed[flat >> 1];
    const int nib = (flat & 1) ? (byte & 15) : (byte >> 4);
    // decoded weight is rounded to the activation dtype before the product
    // (qwen3_moe_fused/grouped_gemm/forward_4bit.py:104)
    return to_f32(from_f32<TIn>(code[nib] * absmax[flat >> shift]));
  }
};

// y[m,n] = sum_k x[m,k] * W(e(m), n, k)
template <typename TIn, typename TOut, typename WLoad>
__global__ void __launch_bounds__(ST_THREADS)
simt_grouped_gemm_kernel(const TIn* __restrict__ x, const WLoad wl,
                         const void* __restrict__ m_sizes, int ms64, TOut* __restrict__ y,
                         int64_t M, int N, int K, int E) {
  __shared__ float As[ST_BK][ST_BM + 1];
  __shared__ float Bs[ST_BK][ST_BN + 1];
  __shared__ int64_t sh_row0, sh_rows;
  __shared__ int sh_expert;

  // Map blockIdx.x (an m-tile slot) to (expert, first row, rows in tile).
  if (threadIdx.x == 0) {
    int64_t slot = blockIdx.x, row = 0;
    int found = -1;
    int64_t r0 = 0, nr = 0;
    for (int e = 0; e < E; ++e) {
      int64_t me = load_index(m_sizes, ms64, e);
      if (me < 0) me = 0;
      if (row + me > M) me = M - row;  // never run past the buffers
      const int64_t tiles = (me + ST_BM - 1) / ST_BM;
      if (slot < tiles) {
        found = e;
        r0 = row + slot * ST_BM;
        nr = me - slot * ST_BM;
        if (nr > ST_BM) nr = ST_BM;
        break;
      }
      slot -= tiles;
      row += me;
    }
    sh_expert = found; sh_row0 = r0; sh_rows = nr;
  }
  __syncthreads();
  const int expert = sh_expert;
  if (expert < 0) return;
  const int64_t row0 = sh_row0;
  const int rows = (int)sh_rows;
  const int n0 = blockIdx.y * ST_BN;

  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += ST_BK) {
    // A slice: ST_BM rows x ST_BK k  (k fastest over threads: coalesced along K)
    for (int i = threadIdx.x; i < ST_BM * ST_BK; i += ST_THREADS) {
      const int kk = i % ST_BK, mm = i / ST_BK;
      float v = 0.f;
      if (mm < rows && k0 + kk < K) v = to_f32(x[(row0 + mm) * K + k0 + kk]);
      As[kk][mm] = v;
    }
    if (wl.k_fastest()) {
      for (int i = threadIdx.x; i < ST_BN * ST_BK; i += ST_THREADS) {
        const int kk = i % ST_BK, nn = i / ST_BK;
        float v = 0.f;
        if (n0 + nn < N && k0 + kk < K) v = wl.load(expert, n0 + nn, k0 + kk);
        Bs[kk][nn] = v;
      }
    } else {
      for (int i = threadIdx.x; i < ST_BN * ST_BK; i += ST_THREADS) {
        const int nn = i % ST_BN, kk = i / ST_BN;
        float v = 0.f;
        if (n0 + nn < N && k0 + kk < K) v = wl.load(expert, n0 + nn, k0 + kk);
        Bs[kk][nn] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < ST_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int mm = ty * 4 + i;
    if (mm >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nn = n0 + tx * 4 + j;
      if (nn < N) y[(row0 + mm) * N + nn] = from_f32<TOut>(acc[i][j]);
    }
  }
}

// dw[e,n,k] = sum_{m in group e} dy[m,n] * x[m,k].  grid = (n tiles, k tiles, E).
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(ST_THREADS)
simt_grouped_dw_kernel(const TIn* __restrict__ x, const TIn* __restrict__ dy,
                       const void* __restrict__ m_sizes, int ms64, TOut* __restrict__ dw,
                       int64_t M, int N, int K, int E) {
  __shared__ float As[ST_BK][ST_BM + 1];  // dy slice: [m][n]
  __shared__ float Bs[ST_BK][ST_BN + 1];  // x slice:  [m][k]
  __shared__ int64_t sh_row0, sh_rows;
  const int expert = blockIdx.z;
  if (threadIdx.x == 0) {
    int64_t row = 0, me = 0;
    for (int e = 0; e <= expert; ++e) {
      row += me;
      me = load_index(m_sizes, ms64, e);
      if (me < 0) me = 0;
      if (row + me > M) me = M - row;
    }
    sh_row0 = row; sh_rows = me;
  }
  __syncthreads();
  const int64_t row0 = sh_row0, rows = sh_rows;
  const int n0 = blockIdx.x * ST_BN, k0 = blockIdx.y * ST_BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int64_t m0 = 0; m0 < rows; m0 += ST_BK) {
    for (int i = threadIdx.x; i < ST_BM * ST_BK; i += ST_THREADS) {
      const int nn = i % ST_BM, mm = i / ST_BM;
      float v = 0.f;
      if (m0 + mm < rows && n0 + nn < N) v = to_f32(dy[(row0 + m0 + mm) * N + n0 + nn]);
      As[mm][nn] = v;
    }
    for (int i = threadIdx.x; i < ST_BN * ST_BK; i += ST_THREADS) {
      const int kk = i % ST_BN, mm = i / ST_BN;
      float v = 0.f;
      if (m0 + mm < rows && k0 + kk < K) v = to_f32(x[(row0 + m0 + mm) * K + k0 + kk]);
      Bs[mm][kk] = v;
    }
    __syncthreads();
#pragma unroll
    for (int mm = 0; mm < ST_BK; ++mm) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[mm][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[mm][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  TOut* out = dw + (int64_t)expert * N * K;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int nn = n0 + ty * 4 + i;
    if (nn >= N) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = k0 + tx * 4 + j;
      if (kk < K) out[(int64_t)nn * K + kk] = from_f32<TOut>(acc[i][j]);
    }
  }
}

template <typename TIn, typename TOut, typename WLoad>
static int launch_fwd_like(const void* x, const WLoad& wl, const void* m_sizes, int ms64, void* y,
                           int64_t M, int N, int K, int E, cudaStream_t stream) {
  if (M == 0 || N == 0) return MOE_OK;
  const int64_t slots = (M + ST_BM - 1) / ST_BM + E;
  const int64_t ntiles = (N + ST_BN - 1) / ST_BN;
  if (slots > 0x7fffffffLL || ntiles > 65535) return MOE_ERR_SHAPE;
  dim3 grid((unsigned)slots, (unsigned)ntiles);
  simt_grouped_gemm_kernel<TIn, TOut, WLoad><<<grid, ST_THREADS, 0, stream>>>(
      (const TIn*)x, wl, m_sizes, ms64, (TOut*)y, M, N, K, E);
  return launch_status();
}

template <typename TIn, typename TOut>
static int launch_dw(const void* x, const void* dy, const void* m_sizes, int ms64, void* dw,
                     int64_t M, int N, int K, int E, cudaStream_t stream) {
  if (N == 0 || K == 0 || E == 0) return MOE_OK;
  const int64_t nt = (N + ST_BN - 1) / ST_BN, kt = (K + ST_BN - 1) / ST_BN;
  if (kt > 65535 || E > 65535) return MOE_ERR_SHAPE;
  dim3 grid((unsigned)nt, (unsigned)kt, (unsigned)E);
  simt_grouped_dw_kernel<TIn, TOut><<<grid, ST_THREADS, 0, stream>>>(
      (const TIn*)x, (const TIn*)dy, m_sizes, ms64, (TOut*)dw, M, N, K, E);
  return launch_status();
}

// which: 0 forward, 1 dX, 2 dW.  Called by the dispatcher in gemm_api.cu.
int simt_grouped_gemm(int which, const void* a, const void* b, const void* m_sizes, int ms64,
                      void* out, int64_t M, int N, int K, int E, int dtype_in, int dtype_out,
                      cudaStream_t stream) {
  MOE_DISPATCH_FLOAT(dtype_in, TIn, {
    MOE_DISPATCH_FLOAT(dtype_out, TOut, {
      if (which == 0) return launch_fwd_like<TIn, TOut>(a, DenseWeight<TIn>{(const TIn*)b, (int64_t)N * K, K, 1}, m_sizes, ms64, out, M, N, K, E, stream);
      if (which == 1) return launch_fwd_like<TIn, TOut>(a, DenseWeight<TIn>{(const TIn*)b, (int64_t)N * K, 1, N}, m_sizes, ms64, out, M, N, K, E, stream);
      return launch_dw<TIn, TOut>(a, b, m_sizes, ms64, out, M, N, K, E, stream);
    });
  });
  return MOE_ERR_DTYPE;
}

// Forward with the weight decoded from NF4 on the fly.
int simt_grouped_gemm_nf4(const void* x, const uint8_t* packed, const float* code, const float* absmax, int shift,
                          const void* m_sizes, int ms64, void* out, int64_t M, int N, int K, int E,
                          int dtype_in, int dtype_out, cudaStream_t stream) {
  MOE_DISPATCH_FLOAT(dtype_in, TIn, {
    MOE_DISPATCH_FLOAT(dtype_out, TOut, {
      return launch_fwd_like<TIn, TOut>(x, Nf4Weight<TIn>{packed, code, absmax, shift, N, K}, m_sizes, ms64, out, M, N, K, E, stream);
    });
  });
  return MOE_ERR_DTYPE;
}

}  // namespace moe
