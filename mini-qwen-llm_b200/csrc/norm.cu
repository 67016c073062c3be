// RMSNorm in front of the MoE block, in the reference's rounding order
// (mini_qwen/model/layers/rms_norm.py:11-18): r = 1/sqrt(mean(float(x)^2) + eps) in fp32,
// y = cast(float(x) * r) to the model type, out = weight * y as a product of two model-type values.
// HBM-bound: one read and one write of the rows; a warp keeps its whole row in registers between the
// sum of squares and the scaling, so the rows are read once.
#include "common.cuh"

namespace mq {
namespace {

template <typename T>
__device__ __forceinline__ float inv_rms(float sum_sq, int64_t H, float eps) {
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)H), eps)));
}

template <typename T>
__device__ __forceinline__ T norm_value(T x, T w, float r) {
  const T y = from_float<T>(__fmul_rn(to_float<T>(x), r));
  return from_float<T>(__fmul_rn(to_float<T>(w), to_float<T>(y)));
}

// One warp per row, NV 16-byte vectors per lane: the row stays in registers.
template <typename T, int NV>
__global__ void __launch_bounds__(256)
rms_norm_rows(const T* __restrict__ x, const T* __restrict__ weight, float eps, int64_t rows, int64_t H,
              T* __restrict__ out) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  pdl_wait();                     // x comes from the kernel before this one
  pdl_release();
  if (row >= rows) return;
  const int nvec = (int)(H / V);                       // vectors in a row; H is a multiple of V
  const uint4* src = reinterpret_cast<const uint4*>(x + row * H);
  uint4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int q = i * 32 + lane;
    v[i] = q < nvec ? src[q] : make_uint4(0u, 0u, 0u, 0u);
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const T* e = reinterpret_cast<const T*>(&v[i]);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float f = to_float<T>(e[j]);
      ss = fmaf(f, f, ss);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = inv_rms<T>(ss, H, eps);
  const uint4* wsrc = reinterpret_cast<const uint4*>(weight);
  uint4* dst = reinterpret_cast<uint4*>(out + row * H);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int q = i * 32 + lane;
    if (q < nvec) {
      const uint4 wv = wsrc[q];
      const T* e = reinterpret_cast<const T*>(&v[i]);
      const T* w = reinterpret_cast<const T*>(&wv);
      T o[V];
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = norm_value<T>(e[j], w[j], r);
      dst[q] = *reinterpret_cast<const uint4*>(o);
    }
  }
}

// Any row length: one CTA per row, the row is read a second time (from L2) for the scaling.
template <typename T>
__global__ void __launch_bounds__(256)
rms_norm_long_rows(const T* __restrict__ x, const T* __restrict__ weight, float eps, int64_t H, T* __restrict__ out) {
  __shared__ float s_part[8];
  const T* src = x + (int64_t)blockIdx.x * H;
  float ss = 0.0f;
  for (int64_t h = threadIdx.x; h < H; h += 256) {
    const float f = to_float<T>(src[h]);
    ss = fmaf(f, f, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += s_part[i];
  const float r = inv_rms<T>(total, H, eps);
  T* dst = out + (int64_t)blockIdx.x * H;
  for (int64_t h = threadIdx.x; h < H; h += 256) dst[h] = norm_value<T>(src[h], weight[h], r);
}

template <typename T>
int launch_rms_norm(const void* x, const void* weight, float eps, int64_t rows, int64_t H, void* out,
                    cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  const T* xs = reinterpret_cast<const T*>(x);
  const T* ws = reinterpret_cast<const T*>(weight);
  T* os = reinterpret_cast<T*>(out);
  const bool vectors = H % V == 0 && aligned16(x) && aligned16(weight) && aligned16(out);
  const int64_t nvec = H / V;
  if (vectors && nvec <= 32 * 16) {
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    if (nvec <= 32 * 2) launch_after_predecessor(rms_norm_rows<T, 2>, dim3(blocks), dim3(256), 0, st, xs, ws, eps, rows, H, os);
    else if (nvec <= 32 * 4) launch_after_predecessor(rms_norm_rows<T, 4>, dim3(blocks), dim3(256), 0, st, xs, ws, eps, rows, H, os);
    else if (nvec <= 32 * 8) launch_after_predecessor(rms_norm_rows<T, 8>, dim3(blocks), dim3(256), 0, st, xs, ws, eps, rows, H, os);
    else launch_after_predecessor(rms_norm_rows<T, 16>, dim3(blocks), dim3(256), 0, st, xs, ws, eps, rows, H, os);
  } else {
    rms_norm_long_rows<T><<<(unsigned)rows, 256, 0, st>>>(xs, ws, eps, H, os);
  }
  return check_launch();
}

}  // namespace
}  // namespace mq

extern "C" int mq_rms_norm(const void* x, int dtype, const void* weight, float eps, int64_t T, int64_t H,
                           void* out, void* stream) {
  using namespace mq;
  if (T < 0 || H <= 0 || !valid_dtype(dtype) || !(eps >= 0.0f)) return MQ_ERR_INVALID_ARGUMENT;
  if (T > 0x7fffffff) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!x || !weight || !out) return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MQ_F32) return launch_rms_norm<float>(x, weight, eps, T, H, out, st);
  if (dtype == MQ_BF16) return launch_rms_norm<__nv_bfloat16>(x, weight, eps, T, H, out, st);
  return launch_rms_norm<__half>(x, weight, eps, T, H, out, st);
}
