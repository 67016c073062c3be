// Expert parallelism for DECODE batches, by replication instead of dispatch.
//
// With a few tokens per GPU the dispatch / return exchange of ep.cu is bound by its four rank barriers per
// layer call, not by bytes.  Here every rank instead holds ALL tokens of the step (an all-gather of a few
// rows), routes them itself (the same kernel on the same bytes gives the same ids, weights and plan on every
// rank), runs only ITS experts on the slots they own, and forms for every token the partial weighted sum over
// those slots in fp32.  The partial sums of a token go to the rank that owns the token, which adds the G of
// them up in rank order.  Two rank barriers per layer call, each at the tail of a kernel that is needed
// anyway; every rank streams only the weights of its own experts.
//
//   mq_ep_gather_tokens   x [T,H] of this rank -> rows [rank*T, rank*T + T) of every peer's token buffer,
//                         then the rank barrier (one CTA; the rows are a few KB).
//   mq_ep_send_partials   for every token t of the step: sum over the slots k whose expert this rank owns of
//                         weights[t,k] * float(rows[inv[t*K+k]]), fp32, k ascending, stored into row
//                         (rank*T + t % T) of the partial-sum buffer of rank t / T; then the rank barrier, done
//                         by the CTA that finishes last.
//   mq_ep_sum_partials    out[t] = cast(sum over ranks r, ascending, of partial[r*T + t]) (+ residual, added
//                         as the layer's add of two model-type tensors).
//
// The sums are taken in another order than on one GPU (per rank first), so outputs equal the single-GPU ones
// to rounding, not to the bit; ids, weights and the plan are identical.  The barrier is ep.cu's: an epoch
// written into every peer's signal array, a bounded poll of the own one, MQ_DEV_WAIT_EXPIRED on expiry.
// All ranks must call with the same T.
#include "common.cuh"

namespace mq {
namespace {

constexpr uint32_t EPD_SPIN_LIMIT = 1u << 22;

// One warp: bump the epoch, publish it to every peer, wait (bounded) until every peer's has arrived.
__device__ void epd_rank_barrier(const uint64_t* __restrict__ peer_sig, int32_t* __restrict__ epoch_ctr, int G,
                                 int rank, uint32_t max_polls, int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  int epoch = 0;
  if (lane == 0) {
    epoch = *epoch_ctr + 1;
    *epoch_ctr = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  __threadfence_system();                        // the peer stores before this point are complete; the flag goes behind them
  for (int r = lane; r < G; r += 32) {
    int32_t* remote = reinterpret_cast<int32_t*>(peer_sig[r]) + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  const int32_t* mine = reinterpret_cast<const int32_t*>(peer_sig[rank]);
  for (int r = lane; r < G; r += 32) {
    uint32_t spin = 0;
    int v;
    do {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + r) : "memory");
    } while (v < epoch && ++spin < max_polls);
    if (v < epoch) atomicOr(status, (int)MQ_DEV_WAIT_EXPIRED);
  }
}

__global__ void __launch_bounds__(1024)
ep_gather_tokens_kernel(const uint4* __restrict__ x, int row_vecs, int T, int G, int rank,
                        const uint64_t* __restrict__ peer_tokens, const uint64_t* __restrict__ peer_sig,
                        int32_t* __restrict__ epoch_ctr, uint32_t max_polls, int32_t* __restrict__ status) {
  const int n = T * row_vecs;
  for (int d = 0; d < G; ++d) {
    uint4* dst = reinterpret_cast<uint4*>(peer_tokens[d]) + (size_t)rank * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = x[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) epd_rank_barrier(peer_sig, epoch_ctr, G, rank, max_polls, status);
}

template <typename Tv>
__global__ void __launch_bounds__(256)
ep_send_partials_kernel(const Tv* __restrict__ rows, const float* __restrict__ weights, const int32_t* __restrict__ ids,
                        const int32_t* __restrict__ inv, int K, int H, int T, int G, int rank, int experts_per_rank,
                        const uint64_t* __restrict__ peer_partials, int* __restrict__ done_ctr,
                        const uint64_t* __restrict__ peer_sig, int32_t* __restrict__ epoch_ctr, uint32_t max_polls,
                        int32_t* __restrict__ status) {
  __shared__ int s_row[32];
  __shared__ float s_w[32];
  __shared__ int s_n, s_last;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    // this rank's slots of the token, k ascending; a slot whose position is outside the sorted order is left out
    // and recorded (the plan comes from this library's own routing kernel, so this is a guard, not a case)
    int n = 0;
    for (int k = 0; k < K; ++k) {
      const int e = ids[t * K + k];
      if (e >= 0 && e / experts_per_rank == rank) {
        const int row = inv[t * K + k];
        if (row < 0 || row >= (int)gridDim.x * K) {
          atomicOr(status, (int)MQ_DEV_BAD_LAUNCH);
          continue;
        }
        s_row[n] = row;
        s_w[n] = weights[t * K + k];
        ++n;
      }
    }
    s_n = n;
  }
  __syncthreads();
  const int n = s_n;
  float* dst = reinterpret_cast<float*>(peer_partials[t / T]) + ((size_t)rank * T + (t % T)) * H;
  constexpr int V = 16 / sizeof(Tv);
  for (int h0 = threadIdx.x * V; h0 < H; h0 += 256 * V) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.0f;
    for (int i = 0; i < n; ++i) {
      const float wk = s_w[i];
      const uint4 raw = *reinterpret_cast<const uint4*>(rows + (size_t)s_row[i] * H + h0);
      const Tv* v = reinterpret_cast<const Tv*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(wk, to_float<Tv>(v[j])));
    }
#pragma unroll
    for (int j = 0; j < V; j += 4)
      *reinterpret_cast<float4*>(dst + h0 + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
  }
  // the CTA that finishes last holds the rank barrier
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(done_ctr, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) *done_ctr = 0;                             // ready for the next call
  if (threadIdx.x < 32) epd_rank_barrier(peer_sig, epoch_ctr, G, rank, max_polls, status);
}

template <typename Tv>
__global__ void __launch_bounds__(256)
ep_sum_partials_kernel(const float* __restrict__ partials, const Tv* __restrict__ residual, int H, int T, int G,
                       Tv* __restrict__ out) {
  const int t = blockIdx.x;
  for (int h = threadIdx.x * 4; h < H; h += 256 * 4) {
    float4 acc = *reinterpret_cast<const float4*>(partials + (size_t)t * H + h);
    for (int r = 1; r < G; ++r) {
      const float4 p = *reinterpret_cast<const float4*>(partials + ((size_t)r * T + t) * H + h);
      acc.x = __fadd_rn(acc.x, p.x); acc.y = __fadd_rn(acc.y, p.y);
      acc.z = __fadd_rn(acc.z, p.z); acc.w = __fadd_rn(acc.w, p.w);
    }
    const float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      Tv o = from_float<Tv>(a[j]);
      if (residual != nullptr)
        o = from_float<Tv>(__fadd_rn(to_float<Tv>(residual[(size_t)t * H + h + j]), to_float<Tv>(o)));
      out[(size_t)t * H + h + j] = o;
    }
  }
}

}  // namespace
}  // namespace mq

extern "C" int mq_ep_gather_tokens(const void* x, int dtype, int64_t T, int64_t H, int64_t G, int64_t rank,
                                   const uint64_t* peer_token_ptrs, const uint64_t* peer_signal_ptrs,
                                   int32_t* epoch_counter, int64_t max_polls, int32_t* d_status, void* stream) {
  using namespace mq;
  if (T <= 0 || H <= 0 || G <= 0 || rank < 0 || rank >= G || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (max_polls < 0 || max_polls > (int64_t)EPD_SPIN_LIMIT) return MQ_ERR_INVALID_ARGUMENT;
  const int64_t row_bytes = H * (int64_t)dtype_size(dtype);
  if (row_bytes % 16 != 0 || T * G > 4096 || T * row_bytes > ((int64_t)1 << 24)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (!x || !peer_token_ptrs || !peer_signal_ptrs || !epoch_counter || !d_status || !aligned16(x))
    return MQ_ERR_INVALID_ARGUMENT;
  ep_gather_tokens_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), (int)(row_bytes / 16), (int)T, (int)G, (int)rank, peer_token_ptrs,
      peer_signal_ptrs, epoch_counter, max_polls ? (uint32_t)max_polls : EPD_SPIN_LIMIT, d_status);
  return check_launch();
}

extern "C" int mq_ep_send_partials(const void* rows, int dtype, const float* weights, const int32_t* topk_ids,
                                   const int32_t* inv, int64_t tokens, int64_t K, int64_t H, int64_t T, int64_t G,
                                   int64_t rank, int64_t experts_per_rank, const uint64_t* peer_partial_ptrs,
                                   int32_t* done_counter, const uint64_t* peer_signal_ptrs, int32_t* epoch_counter,
                                   int64_t max_polls, int32_t* d_status, void* stream) {
  using namespace mq;
  if (tokens <= 0 || K <= 0 || H <= 0 || T <= 0 || G <= 0 || rank < 0 || rank >= G || experts_per_rank <= 0 ||
      !valid_dtype(dtype))
    return MQ_ERR_INVALID_ARGUMENT;
  if (tokens != T * G) return MQ_ERR_INVALID_ARGUMENT;
  if (max_polls < 0 || max_polls > (int64_t)EPD_SPIN_LIMIT) return MQ_ERR_INVALID_ARGUMENT;
  if (K > 32 || H % 8 != 0) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (!rows || !weights || !topk_ids || !inv || !peer_partial_ptrs || !done_counter || !peer_signal_ptrs ||
      !epoch_counter || !d_status || !aligned16(rows))
    return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint32_t polls = max_polls ? (uint32_t)max_polls : EPD_SPIN_LIMIT;
#define MQ_EPD_SEND(TV)                                                                                              \
  ep_send_partials_kernel<TV><<<(unsigned)tokens, 256, 0, st>>>(                                                     \
      reinterpret_cast<const TV*>(rows), weights, topk_ids, inv, (int)K, (int)H, (int)T, (int)G, (int)rank,          \
      (int)experts_per_rank, peer_partial_ptrs, done_counter, peer_signal_ptrs, epoch_counter, polls, d_status)
  if (dtype == MQ_F32) MQ_EPD_SEND(float);
  else if (dtype == MQ_BF16) MQ_EPD_SEND(__nv_bfloat16);
  else MQ_EPD_SEND(__half);
#undef MQ_EPD_SEND
  return check_launch();
}

extern "C" int mq_ep_sum_partials(const float* partials, int dtype, const void* residual, int64_t T, int64_t H,
                                  int64_t G, void* out, void* stream) {
  using namespace mq;
  if (T <= 0 || H <= 0 || G <= 0 || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (H % 4 != 0) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (!partials || !out || !aligned16(partials)) return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MQ_F32)
    ep_sum_partials_kernel<float><<<(unsigned)T, 256, 0, st>>>(partials, reinterpret_cast<const float*>(residual),
                                                              (int)H, (int)T, (int)G, reinterpret_cast<float*>(out));
  else if (dtype == MQ_BF16)
    ep_sum_partials_kernel<__nv_bfloat16><<<(unsigned)T, 256, 0, st>>>(
        partials, reinterpret_cast<const __nv_bfloat16*>(residual), (int)H, (int)T, (int)G,
        reinterpret_cast<__nv_bfloat16*>(out));
  else
    ep_sum_partials_kernel<__half><<<(unsigned)T, 256, 0, st>>>(partials, reinterpret_cast<const __half*>(residual),
                                                               (int)H, (int)T, (int)G, reinterpret_cast<__half*>(out));
  return check_launch();
}
