// Shared helpers for the libmqmoe kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mqmoe.h"

namespace mq {

// Records the last CUDA launch error of this host thread for mq_last_cuda_error().
void set_last_cuda_error(cudaError_t e);

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return MQ_ERR_LAUNCH_FAILED;
  }
  return MQ_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t dtype_size(int dt) { return dt == MQ_F32 ? 4 : 2; }
inline bool valid_dtype(int dt) { return dt == MQ_F32 || dt == MQ_BF16 || dt == MQ_F16; }

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Element of a row-major array of runtime element type, widened to fp32.
__device__ __forceinline__ float load_as_float(const void* p, int dt, size_t i) {
  if (dt == MQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  if (dt == MQ_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

// round-to-`T` of x, returned as fp32 (the rounding points of a torch op chain in dtype T)
template <typename T> __device__ __forceinline__ float round_to(float x) { return to_float<T>(from_float<T>(x)); }

// SwiGLU with the rounding points of  silu(gate(x)) * up(x)  evaluated op by op in dtype T:
// g and u are the fp32 accumulators of the two projections.
template <typename T> __device__ __forceinline__ float swiglu_rounded(float g, float u) {
  float gb = round_to<T>(g);
  float sb = round_to<T>(gb / (1.0f + expf(-gb)));
  float ub = round_to<T>(u);
  return sb * ub;  // caller rounds on store
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Programmatic dependent launch.  A kernel launched with launch_after_predecessor() may start while the kernel
// before it in the stream is still running; it must call pdl_wait() before it touches anything that kernel (or
// any earlier one) wrote or reads, which blocks until the predecessor has completed and its writes are visible.
// pdl_release() lets the NEXT kernel of the stream be scheduled from here on (it still waits in its own
// pdl_wait()).  A kernel that calls neither behaves as in an ordinary launch, so the two kinds mix freely.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The launch attribute is OFF unless MQMOE_PDL=1 is in the environment (every launch then serialises as usual and
// the two instructions are no-ops): measured on the decode chain it changes a single-GPU layer call by less than
// two percent either way and makes the expert-parallel 48-layer pass 12 % slower.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_after_predecessor(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace mq
