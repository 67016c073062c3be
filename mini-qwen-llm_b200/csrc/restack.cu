// Load-time stacking of per-expert tensors (no counterpart in the reference, whose loaders leave one
// nn.Linear / LinearW4A16 per expert and projection: mini_qwen/model/loader.py:63-75 for dense
// checkpoints, :245-250 for GPTQ ones; the block's restack in Python is torch.stack).  A host without a
// tensor library builds the expert-major stacks the grouped kernels index with this call:
// n equally sized tensors, given by a device array of their addresses, are concatenated into `out`.
#include "common.cuh"

namespace mq {
namespace {

__global__ void __launch_bounds__(256)
stack_vec_kernel(const uint64_t* __restrict__ src_ptrs, int64_t vec_each, uint4* __restrict__ out) {
  const uint4* src = reinterpret_cast<const uint4*>(src_ptrs[blockIdx.y]);
  uint4* dst = out + (int64_t)blockIdx.y * vec_each;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < vec_each; i += (int64_t)gridDim.x * 256) dst[i] = __ldg(src + i);
}

__global__ void __launch_bounds__(256)
stack_bytes_kernel(const uint64_t* __restrict__ src_ptrs, int64_t bytes_each, uint8_t* __restrict__ out) {
  const uint8_t* src = reinterpret_cast<const uint8_t*>(src_ptrs[blockIdx.y]);
  uint8_t* dst = out + (int64_t)blockIdx.y * bytes_each;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < bytes_each; i += (int64_t)gridDim.x * 256) dst[i] = src[i];
}

}  // namespace
}  // namespace mq

extern "C" int mq_stack_tensors(const uint64_t* d_src_ptrs, int64_t n, int64_t bytes_each, int sources_aligned16,
                                void* out, void* stream) {
  using namespace mq;
  if (n < 0 || bytes_each < 0) return MQ_ERR_INVALID_ARGUMENT;
  if (n == 0 || bytes_each == 0) return MQ_OK;
  if (!d_src_ptrs || !out) return MQ_ERR_INVALID_ARGUMENT;
  if (n > 65535) return MQ_ERR_UNSUPPORTED_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // a few CTAs per tensor: the copy is a one-off at load time, but a 9 MB expert still deserves more than one
  if (sources_aligned16 && bytes_each % 16 == 0 && aligned16(out)) {
    const int64_t vec = bytes_each / 16;
    const int64_t want = (vec + 4095) / 4096;
    stack_vec_kernel<<<dim3((unsigned)(want < 32 ? want : 32), (unsigned)n), 256, 0, st>>>(
        d_src_ptrs, vec, reinterpret_cast<uint4*>(out));
  } else {
    const int64_t want = (bytes_each + 4095) / 4096;
    stack_bytes_kernel<<<dim3((unsigned)(want < 32 ? want : 32), (unsigned)n), 256, 0, st>>>(
        d_src_ptrs, bytes_each, reinterpret_cast<uint8_t*>(out));
  }
  return check_launch();
}
