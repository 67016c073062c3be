// Entry points that choose between kernels, and the library's bookkeeping calls.
#include <cstdlib>

#include "common.cuh"

namespace mq {

static thread_local cudaError_t g_last_error = cudaSuccess;
void set_last_cuda_error(cudaError_t e) { g_last_error = e; }

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("MQMOE_PDL");
    return v != nullptr && v[0] == '1';
  }();
  return on;
}

int grouped_gemm_generic_dispatch(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E,
                                  int64_t period, int64_t N, int64_t Kd, int dtype, bool swiglu, void* out,
                                  cudaStream_t st);

// tcgen05 kernel (bf16). Returns MQ_ERR_UNSUPPORTED_SHAPE when the shape is outside its cover.
int grouped_gemm_tc5(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E, int64_t period,
                     int64_t N, int64_t Kd, bool swiglu, void* out, int32_t* d_status, cudaStream_t st,
                     const int32_t* perm, int64_t top_k, const int32_t* row_dst, const uint64_t* dst_bases);
bool tc5_covers(int64_t S, int64_t E, int64_t N, int64_t Kd, bool swiglu);

}  // namespace mq

extern "C" int mq_version(void) { return 1; }

extern "C" const char* mq_status_string(int status) {
  switch (status) {
    case MQ_OK: return "ok";
    case MQ_ERR_INVALID_ARGUMENT: return "invalid argument (null or misaligned pointer, negative size)";
    case MQ_ERR_UNSUPPORTED_SHAPE: return "size outside what the kernels cover";
    case MQ_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case MQ_ERR_LAUNCH_FAILED: return "kernel launch failed";
    case MQ_ERR_DRIVER_ENTRY: return "cuTensorMapEncodeTiled unavailable or failed";
    case MQ_ERR_STATIC_SCRATCH_EXCEEDED:
      return "request needs more scratch than the 10 MiB array built into the library (use the entry point "
             "that takes a caller workspace)";
    default: return "unknown status";
  }
}

extern "C" const char* mq_last_cuda_error(void) { return cudaGetErrorString(mq::g_last_error); }

static int grouped_common(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E,
                          int64_t period, int64_t N, int64_t Kd, int dtype, bool swiglu, void* out,
                          int32_t* d_status, void* stream) {
  using namespace mq;
  if (S < 0 || E <= 0 || N <= 0 || Kd <= 0 || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (period <= 0 || period > E) return MQ_ERR_INVALID_ARGUMENT;
  if (S >= (int64_t)1 << 31) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!a || !w || !offsets || !out) return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MQ_BF16 && tc5_covers(S, period, N, Kd, swiglu) && aligned16(a) && aligned16(w) && aligned16(out))
    return grouped_gemm_tc5(a, w, offsets, S, E, period, N, Kd, swiglu, out, d_status, st, nullptr, 1, nullptr, nullptr);
  return grouped_gemm_generic_dispatch(a, w, offsets, S, E, period, N, Kd, dtype, swiglu, out, st);
}

extern "C" int mq_grouped_gemm(const void* a, const void* w, const int32_t* offsets,
                               int64_t S, int64_t E, int64_t weight_period, int64_t N, int64_t Kd, int dtype,
                               void* out, int32_t* d_status, void* stream) {
  return grouped_common(a, w, offsets, S, E, weight_period, N, Kd, dtype, false, out, d_status, stream);
}

extern "C" int mq_grouped_swiglu(const void* a, const void* w_gate_up, const int32_t* offsets,
                                 int64_t S, int64_t E, int64_t weight_period, int64_t I, int64_t H, int dtype,
                                 void* h, int32_t* d_status, void* stream) {
  return grouped_common(a, w_gate_up, offsets, S, E, weight_period, I, H, dtype, true, h, d_status, stream);
}

extern "C" int mq_grouped_swiglu_gather(const void* x, const int32_t* perm, const void* w_gate_up,
                                        const int32_t* offsets, int64_t T, int64_t top_k, int64_t E,
                                        int64_t weight_period, int64_t I, int64_t H, int dtype,
                                        void* h, int32_t* d_status, void* stream) {
  using namespace mq;
  if (T < 0 || top_k <= 0 || E <= 0 || I <= 0 || H <= 0 || weight_period <= 0 || weight_period > E)
    return MQ_ERR_INVALID_ARGUMENT;
  const int64_t S = T * top_k;
  // the kernel addresses x with 32-bit element offsets
  if (dtype != MQ_BF16 || !tc5_covers(S, weight_period, I, H, true) || T * H >= ((int64_t)1 << 32))
    return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!x || !perm || !w_gate_up || !offsets || !h) return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(x) || !aligned16(w_gate_up) || !aligned16(h)) return MQ_ERR_INVALID_ARGUMENT;
  return grouped_gemm_tc5(x, w_gate_up, offsets, S, E, weight_period, I, H, true, h, d_status,
                          reinterpret_cast<cudaStream_t>(stream), perm, top_k, nullptr, nullptr);
}

extern "C" int mq_grouped_gemm_scatter(const void* a, const void* w, const int32_t* offsets,
                                       const int32_t* row_dst, const uint64_t* dst_bases, int64_t S, int64_t E,
                                       int64_t weight_period, int64_t N, int64_t Kd, int dtype, int32_t* d_status,
                                       void* stream) {
  using namespace mq;
  if (S < 0 || E <= 0 || N <= 0 || Kd <= 0 || weight_period <= 0 || weight_period > E || !valid_dtype(dtype))
    return MQ_ERR_INVALID_ARGUMENT;
  if (dtype != MQ_BF16 || !tc5_covers(S, weight_period, N, Kd, false)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!a || !w || !offsets || !row_dst || !dst_bases || !aligned16(a) || !aligned16(w)) return MQ_ERR_INVALID_ARGUMENT;
  return grouped_gemm_tc5(a, w, offsets, S, E, weight_period, N, Kd, false, nullptr, d_status,
                          reinterpret_cast<cudaStream_t>(stream), nullptr, 1, row_dst, dst_bases);
}
