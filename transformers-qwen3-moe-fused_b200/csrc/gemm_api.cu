// C ABI of the grouped GEMMs: argument checking and the choice between the tcgen05
// kernels and the CUDA-core kernels.  Nothing here touches device memory.
#include <atomic>

#include "common.cuh"

namespace moe {
int simt_grouped_gemm(int which, const void* a, const void* b, const void* m_sizes, int ms64, void* out,
                      int64_t M, int N, int K, int E, int dtype_in, int dtype_out, cudaStream_t stream);
int simt_grouped_gemm_nf4(const void* x, const uint8_t* packed, const float* code, const float* absmax, int shift,
                          const void* m_sizes, int ms64, void* out, int64_t M, int N, int K, int E,
                          int dtype_in, int dtype_out, cudaStream_t stream);
bool tc_eligible(int which, const void* a, const void* b, const void* out, int64_t M, int N, int K, int E,
                 int dtype_in, int dtype_out);
int tc_grouped_gemm(int which, const void* a, const void* b, const void* m_sizes, int ms64, void* out,
                    int64_t M, int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes,
                    cudaStream_t stream, bool single_cta);
bool tc_nf4_eligible(const void* x, const void* packed, const void* absmax, const void* out, int64_t M, int N, int K,
                     int E, int blocksize, int dtype_in, int dtype_out);
int tc_grouped_gemm_nf4(const void* x, const uint8_t* packed, const float* code, const float* absmax, int blocksize,
                        const void* m_sizes, int ms64, void* out, int64_t M, int N, int K, int E,
                        int dtype_in, int dtype_out, void* ws, size_t ws_bytes, cudaStream_t stream, bool transposed);
int tc_grouped_gemm_scattered(int which, const void* a, const void* b, const void* group_sizes, int ms64,
                              const int* weight_index, int n_weights, const uint64_t* out_ptrs, void* out_template,
                              int64_t M, int N, int K, int G, int dtype_in, int dtype_out, void* ws, size_t ws_bytes,
                              cudaStream_t stream);
int tc_gate_up_silu(const void* x, const void* w_gate, const void* w_up, const void* m_sizes, int ms64, void* h,
                    int64_t M, int I, int K, int E, int dtype, void* ws, size_t ws_bytes, cudaStream_t stream,
                    const int* row_index, int index_div, int64_t x_rows);
int tc_grouped_gemm_gather(const void* x, int64_t x_rows, const int* row_index, int index_div, const void* w,
                           const void* m_sizes, int ms64, void* y, int64_t M, int N, int K, int E, int dtype_in,
                           int dtype_out, void* ws, size_t ws_bytes, cudaStream_t stream);
int tc_read_error(int* flag_out, bool clear);
size_t tc_workspace_bytes(int E);
int tc_read_late_values(int* out);
const char* tc_last_detail();

static std::atomic<int> g_path{MOE_PATH_AUTO};

static bool device_is_sm100() {
  static int cached[64] = {0};  // 0 unknown, 1 yes, 2 no
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (cached[dev] == 0) {
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cached[dev] = major == 10 ? 1 : 2;
  }
  return cached[dev] == 1;
}

static int check_common(const void* a, const void* b, const void* m_sizes, int msd, const void* out,
                        int64_t M, int N, int K, int E, int dtype_in, int dtype_out) {
  if (!is_float_dtype(dtype_in) || !is_float_dtype(dtype_out) || !is_int_dtype(msd)) return MOE_ERR_DTYPE;
  if (M < 0 || N < 0 || K < 0 || E <= 0 || M > 0x7fffffffLL) return MOE_ERR_SHAPE;
  if (!m_sizes) return MOE_ERR_NULL;
  if ((M > 0 && (N > 0 || K > 0)) && (!a || !b)) return MOE_ERR_NULL;
  if (!out && M > 0 && N > 0) return MOE_ERR_NULL;
  return MOE_OK;
}

static int run(int which, const void* a, const void* b, const void* m_sizes, int msd, void* out, int64_t M,
               int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  const int ms64 = msd == MOE_I64;
  const int path = g_path.load(std::memory_order_relaxed);
  const bool can_tc = tc_eligible(which, a, b, out, M, N, K, E, dtype_in, dtype_out);
  if ((path == MOE_PATH_TC || path == MOE_PATH_TC_SINGLE) && !can_tc) return MOE_ERR_UNSUPPORTED;
  if (can_tc && path != MOE_PATH_SIMT)
    return tc_grouped_gemm(which, a, b, m_sizes, ms64, out, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, stream, path == MOE_PATH_TC_SINGLE);
  return simt_grouped_gemm(which, a, b, m_sizes, ms64, out, M, N, K, E, dtype_in, dtype_out, stream);
}

}  // namespace moe

using namespace moe;

MOE_API int moe_b200_version(void) { return 1; }

MOE_API const char* moe_status_string(int status) {
  switch (status) {
    case MOE_OK: return "ok";
    case MOE_ERR_DTYPE: return "unsupported dtype";
    case MOE_ERR_SHAPE: return "invalid or unsupported shape";
    case MOE_ERR_NULL: return "null pointer";
    case MOE_ERR_WORKSPACE: return "workspace missing or too small";
    case MOE_ERR_UNSUPPORTED: return "request not supported by the selected kernel family";
    case MOE_ERR_ALIGN: return "pointer or pitch misaligned";
    case MOE_ERR_DEVICE: return "device is not sm_100 or a driver entry point is missing";
  }
  if (status > 0) return cudaGetErrorString((cudaError_t)status);
  return "unknown status";
}

MOE_API int moe_set_gemm_path(int path) {
  if (path < MOE_PATH_AUTO || path > MOE_PATH_TC_SINGLE) return g_path.load();
  return g_path.exchange(path);
}
MOE_API int moe_get_gemm_path(void) { return g_path.load(); }

MOE_API size_t moe_grouped_gemm_workspace_bytes(int, int64_t, int, int, int E) {
  // per-expert tensor maps derived from m_sizes on the device, and the launch's work-item counter
  return tc_workspace_bytes(E);
}

MOE_API int moe_grouped_gemm_fwd(const void* x, const void* w, const void* m_sizes, int msd, void* y, int64_t M,
                                 int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  int st = check_common(x, w, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out);
  if (st != MOE_OK) return st;
  if (M == 0 || N == 0) return MOE_OK;
  if (K == 0) return cuda_status(cudaMemsetAsync(y, 0, (size_t)M * N * dtype_size(dtype_out), (cudaStream_t)stream));
  return run(0, x, w, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, (cudaStream_t)stream);
}

MOE_API int moe_grouped_gemm_dx(const void* x, const void* w, const void* m_sizes, int msd, void* y, int64_t M,
                                int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  int st = check_common(x, w, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out);
  if (st != MOE_OK) return st;
  if (M == 0 || N == 0) return MOE_OK;
  if (K == 0) return cuda_status(cudaMemsetAsync(y, 0, (size_t)M * N * dtype_size(dtype_out), (cudaStream_t)stream));
  return run(1, x, w, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, (cudaStream_t)stream);
}

MOE_API int moe_grouped_gemm_dw(const void* x, const void* y, const void* m_sizes, int msd, void* w, int64_t M,
                                int N, int K, int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  if (!is_float_dtype(dtype_in) || !is_float_dtype(dtype_out) || !is_int_dtype(msd)) return MOE_ERR_DTYPE;
  if (M < 0 || N < 0 || K < 0 || E <= 0 || M > 0x7fffffffLL) return MOE_ERR_SHAPE;
  if (!m_sizes) return MOE_ERR_NULL;
  if (N == 0 || K == 0) return MOE_OK;
  if (!w || (M > 0 && (!x || !y))) return MOE_ERR_NULL;
  if (M == 0) return cuda_status(cudaMemsetAsync(w, 0, (size_t)E * N * K * dtype_size(dtype_out), (cudaStream_t)stream));
  return run(2, x, y, m_sizes, msd, w, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, (cudaStream_t)stream);
}

MOE_API int moe_grouped_gemm_fwd_nf4(const void* x, const uint8_t* packed, const float* code, const float* absmax,
                                     int blocksize, const void* m_sizes, int msd, void* y, int64_t M, int N, int K,
                                     int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  int st = check_common(x, packed, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out);
  if (st != MOE_OK) return st;
  if (!code || !absmax) return MOE_ERR_NULL;
  int shift = -1;
  for (int s = 0; s < 31; ++s) if ((1 << s) == blocksize) shift = s;
  if (shift < 0 || (K & 1) || (((int64_t)E * N * K) % blocksize) != 0) return MOE_ERR_SHAPE;
  if (M == 0 || N == 0) return MOE_OK;
  if (K == 0) return cuda_status(cudaMemsetAsync(y, 0, (size_t)M * N * dtype_size(dtype_out), (cudaStream_t)stream));
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  const int path = g_path.load(std::memory_order_relaxed);
  const bool can_tc = tc_nf4_eligible(x, packed, absmax, y, M, N, K, E, blocksize, dtype_in, dtype_out);
  if ((path == MOE_PATH_TC || path == MOE_PATH_TC_SINGLE) && !can_tc) return MOE_ERR_UNSUPPORTED;
  if (can_tc && path != MOE_PATH_SIMT)
    return tc_grouped_gemm_nf4(x, packed, code, absmax, blocksize, m_sizes, msd == MOE_I64, y, M, N, K, E, dtype_in, dtype_out, ws, ws_bytes, (cudaStream_t)stream, false);
  return simt_grouped_gemm_nf4(x, packed, code, absmax, shift, m_sizes, msd == MOE_I64, y, M, N, K, E, dtype_in, dtype_out, (cudaStream_t)stream);
}

MOE_API int moe_grouped_gemm_dx_nf4(const void* x, const uint8_t* packed, const float* code, const float* absmax,
                                    int blocksize, const void* m_sizes, int msd, void* y, int64_t M, int N, int K,
                                    int E, int dtype_in, int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  int st = check_common(x, packed, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out);
  if (st != MOE_OK) return st;
  if (!code || !absmax) return MOE_ERR_NULL;
  int shift = -1;
  for (int s = 0; s < 31; ++s) if ((1 << s) == blocksize) shift = s;
  if (shift < 0 || (N & 1) || (((int64_t)E * N * K) % blocksize) != 0) return MOE_ERR_SHAPE;
  if (M == 0 || N == 0) return MOE_OK;
  if (K == 0) return cuda_status(cudaMemsetAsync(y, 0, (size_t)M * N * dtype_size(dtype_out), (cudaStream_t)stream));
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  // Tensor-core CTA-pair kernel only: 16-bit activations, an absmax block = 64 (or a multiple)
  // consecutive output features of one contraction row, whole 64-row contraction blocks.
  if (!tc_eligible(1, x, packed, y, M, N, K, E, dtype_in, dtype_out) || blocksize < 64 || (N % 64) != 0 ||
      (K % 64) != 0 || N < 192 || ((uintptr_t)absmax & 3))
    return MOE_ERR_UNSUPPORTED;
  return tc_grouped_gemm_nf4(x, packed, code, absmax, blocksize, m_sizes, msd == MOE_I64, y, M, N, K, E, dtype_in,
                             dtype_out, ws, ws_bytes, (cudaStream_t)stream, true);
}

MOE_API int moe_gate_up_silu_fwd(const void* x, const void* w_gate, const void* w_up, const void* m_sizes, int msd,
                                 void* h, int64_t M, int I, int K, int E, int dtype, void* ws, size_t ws_bytes,
                                 void* stream) {
  int st = check_common(x, w_gate, m_sizes, msd, h, M, I, K, E, dtype, dtype);
  if (st != MOE_OK) return st;
  if (M > 0 && I > 0 && K > 0 && !w_up) return MOE_ERR_NULL;
  if (M == 0 || I == 0) return MOE_OK;
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  // CTA-pair tensor-core kernel only: 16-bit data, 16-byte aligned rows and bases
  if (K == 0 || dtype == MOE_F32 || !tc_eligible(0, x, w_gate, h, M, I, K, E, dtype, dtype) ||
      ((uintptr_t)w_up & 15) || ((uintptr_t)h & 15))
    return MOE_ERR_UNSUPPORTED;
  return tc_gate_up_silu(x, w_gate, w_up, m_sizes, msd == MOE_I64, h, M, I, K, E, dtype, ws, ws_bytes, (cudaStream_t)stream,
                         nullptr, 1, 0);
}

MOE_API int moe_gate_up_silu_fwd_gather(const void* x, int64_t x_rows, const int32_t* row_index, int index_div,
                                        const void* w_gate, const void* w_up, const void* m_sizes, int msd, void* h,
                                        int64_t M, int I, int K, int E, int dtype, void* ws, size_t ws_bytes, void* stream) {
  int st = check_common(x, w_gate, m_sizes, msd, h, M, I, K, E, dtype, dtype);
  if (st != MOE_OK) return st;
  if (x_rows < 0 || index_div <= 0) return MOE_ERR_SHAPE;
  if (M > 0 && I > 0 && K > 0 && (!w_up || !row_index)) return MOE_ERR_NULL;
  if (M == 0 || I == 0) return MOE_OK;
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  if (K == 0 || x_rows == 0 || dtype == MOE_F32 || !tc_eligible(0, x, w_gate, h, M, I, K, E, dtype, dtype) ||
      ((uintptr_t)w_up & 15) || ((uintptr_t)h & 15))
    return MOE_ERR_UNSUPPORTED;
  return tc_gate_up_silu(x, w_gate, w_up, m_sizes, msd == MOE_I64, h, M, I, K, E, dtype, ws, ws_bytes, (cudaStream_t)stream,
                         row_index, index_div, x_rows);
}

MOE_API int moe_grouped_gemm_fwd_gather(const void* x, int64_t x_rows, const int32_t* row_index, int index_div, const void* w,
                                        const void* m_sizes, int msd, void* y, int64_t M, int N, int K, int E, int dtype_in,
                                        int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  int st = check_common(x, w, m_sizes, msd, y, M, N, K, E, dtype_in, dtype_out);
  if (st != MOE_OK) return st;
  if (x_rows < 0 || index_div <= 0) return MOE_ERR_SHAPE;
  if (M > 0 && N > 0 && K > 0 && !row_index) return MOE_ERR_NULL;
  if (M == 0 || N == 0) return MOE_OK;
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  if (K == 0 || x_rows == 0 || !tc_eligible(0, x, w, y, M, N, K, E, dtype_in, dtype_out)) return MOE_ERR_UNSUPPORTED;
  return tc_grouped_gemm_gather(x, x_rows, row_index, index_div, w, m_sizes, msd == MOE_I64, y, M, N, K, E, dtype_in,
                                dtype_out, ws, ws_bytes, (cudaStream_t)stream);
}

static int run_scattered(int which, const void* x, const void* w, const void* group_sizes, int msd,
                         const int32_t* weight_index, int n_weights, const uint64_t* out_ptrs, void* out_template,
                         int64_t M, int N, int K, int G, int dtype_in, int dtype_out, void* ws, size_t ws_bytes,
                         void* stream) {
  int st = check_common(x, w, group_sizes, msd, out_template, M, N, K, G, dtype_in, dtype_out);
  if (st != MOE_OK) return st;
  if (n_weights <= 0 || !out_ptrs) return n_weights <= 0 ? MOE_ERR_SHAPE : MOE_ERR_NULL;
  if (M == 0 || N == 0) return MOE_OK;
  if (!device_is_sm100()) return MOE_ERR_DEVICE;
  // only the CTA-pair tensor-core kernels have per-group output maps
  if (K == 0 || N < 192 || dtype_out == MOE_F32 || !tc_eligible(which, x, w, out_template, M, N, K, G, dtype_in, dtype_out))
    return MOE_ERR_UNSUPPORTED;
  if (!ws || ws_bytes < moe_grouped_gemm_workspace_bytes(which, M, N, K, G)) return MOE_ERR_WORKSPACE;
  return tc_grouped_gemm_scattered(which, x, w, group_sizes, msd == MOE_I64, weight_index, n_weights, out_ptrs,
                                   out_template, M, N, K, G, dtype_in, dtype_out, ws, ws_bytes, (cudaStream_t)stream);
}

MOE_API int moe_grouped_gemm_fwd_scattered(const void* x, const void* w, const void* group_sizes, int msd,
                                           const int32_t* weight_index, int n_weights, const uint64_t* out_ptrs,
                                           void* out_template, int64_t M, int N, int K, int G, int dtype_in,
                                           int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  return run_scattered(0, x, w, group_sizes, msd, weight_index, n_weights, out_ptrs, out_template, M, N, K, G, dtype_in,
                       dtype_out, ws, ws_bytes, stream);
}

MOE_API int moe_grouped_gemm_dx_scattered(const void* x, const void* w, const void* group_sizes, int msd,
                                          const int32_t* weight_index, int n_weights, const uint64_t* out_ptrs,
                                          void* out_template, int64_t M, int N, int K, int G, int dtype_in,
                                          int dtype_out, void* ws, size_t ws_bytes, void* stream) {
  return run_scattered(1, x, w, group_sizes, msd, weight_index, n_weights, out_ptrs, out_template, M, N, K, G, dtype_in,
                       dtype_out, ws, ws_bytes, stream);
}

MOE_API int moe_debug_read_error(int* flag_out, int clear) {
  if (!flag_out) return MOE_ERR_NULL;
  return tc_read_error(flag_out, clear != 0);
}

MOE_API int moe_debug_read_late_values(int* out) {
  if (!out) return MOE_ERR_NULL;
  return tc_read_late_values(out);
}

MOE_API const char* moe_debug_last_detail(void) { return tc_last_detail(); }
