// Expert-sorted permute plan (stable counting sort of the T*K slots by expert id), row gather,
// and the weighted unpermute-combine.
// Follows mini_qwen/kernels/moe_permute.py:22-33 and mini_qwen/kernels/moe_unpermute.py:20-31.
//
// The reference sorts T*K int64 keys with a general stable argsort (three times per layer call);
// here the keys have at most 1024 distinct values, so a histogram + prefix scan + ranked placement
// gives the same permutation: within an expert, slots keep ascending flat index t*K+k.
#include "common.cuh"
#include "route_helpers.cuh"

namespace mq {
namespace {

constexpr int P_THREADS = 256;            // 8 warps
constexpr int P_CHUNK = P_THREADS;        // slots ranked per step
constexpr int P_SEG = P_CHUNK;            // slots per CTA in the multi-CTA plan
constexpr int P_SMALL = 8 * P_CHUNK;      // up to this many slots the whole plan runs in one CTA
constexpr int P_MAX_E = 1024;


template <bool IDS64>
__global__ void __launch_bounds__(P_THREADS)
permute_hist(const void* __restrict__ ids, int64_t S, int E, int32_t* __restrict__ seg_hist) {
  __shared__ int hist[P_MAX_E];
  for (int e = threadIdx.x; e < E; e += P_THREADS) hist[e] = 0;
  __syncthreads();
  const int64_t lo = (int64_t)blockIdx.x * P_SEG;
  const int64_t hi = min(lo + (int64_t)P_SEG, S);
  for (int64_t i = lo + threadIdx.x; i < hi; i += P_THREADS) {
    int e = load_id<IDS64>(ids, i);
    if ((unsigned)e < (unsigned)E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  // stored expert-major [E][nseg] so that the scan over segments reads contiguous memory
  for (int e = threadIdx.x; e < E; e += P_THREADS) seg_hist[(size_t)e * gridDim.x + blockIdx.x] = hist[e];
}

// seg_hist[e][seg] -> exclusive prefix over segments (in place) and totals[e]; one warp per expert,
// 32 segments at a time (coalesced loads, shuffle scan, carry).
__global__ void __launch_bounds__(P_THREADS)
permute_scan(int32_t* __restrict__ seg_hist, int nseg, int E, int32_t* __restrict__ totals) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.x * (P_THREADS / 32) + warp;
  if (e >= E) return;
  int32_t* row = seg_hist + (size_t)e * nseg;
  int carry = 0;
  for (int s0 = 0; s0 < nseg; s0 += 32) {
    const int sidx = s0 + lane;
    const int c = sidx < nseg ? row[sidx] : 0;
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (sidx < nseg) row[sidx] = carry + incl - c;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) totals[e] = carry;
}

// Every CTA turns the per-expert totals into offsets itself (E loads and a block scan); CTA 0 also
// publishes them.  Then the segment is ranked and placed.
template <bool IDS64>
__global__ void __launch_bounds__(P_THREADS)
permute_place(const void* __restrict__ ids, int64_t S, int E, int nseg, const int32_t* __restrict__ seg_base,
              const int32_t* __restrict__ totals, int64_t* __restrict__ off64, int32_t* __restrict__ off32,
              int32_t* __restrict__ perm, int32_t* __restrict__ inv) {
  __shared__ int run[P_MAX_E];
  __shared__ int warp_tot[P_THREADS / 32];
  for (int e = threadIdx.x; e < E; e += P_THREADS) run[e] = totals[e];
  __syncthreads();
  const int total = block_exclusive_scan<P_THREADS>(run, E, warp_tot);
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < E; e += P_THREADS) {
      if (off64) off64[e] = run[e];
      if (off32) off32[e] = run[e];
    }
    if (threadIdx.x == 0) {
      if (off64) off64[E] = total;
      if (off32) off32[E] = total;
    }
  }
  for (int e = threadIdx.x; e < E; e += P_THREADS) run[e] += seg_base[(size_t)e * nseg + blockIdx.x];
  __syncthreads();
  const int64_t lo = (int64_t)blockIdx.x * P_SEG;
  place_segment<IDS64, P_THREADS>(ids, lo, min(lo + (int64_t)P_SEG, S), E, run, perm, inv);
}

// Whole plan in one CTA when all slots fit one segment (decode batches).
template <bool IDS64>
__global__ void __launch_bounds__(P_THREADS)
permute_plan_small(const void* __restrict__ ids, int64_t S, int E, int32_t* __restrict__ perm,
                   int32_t* __restrict__ inv, int64_t* __restrict__ off64, int32_t* __restrict__ off32) {
  __shared__ int run[P_MAX_E];
  __shared__ int warp_tot[P_THREADS / 32];
  for (int e = threadIdx.x; e < E; e += P_THREADS) run[e] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < S; i += P_THREADS) {
    int e = load_id<IDS64>(ids, i);
    if ((unsigned)e < (unsigned)E) atomicAdd(&run[e], 1);
  }
  __syncthreads();
  int total = block_exclusive_scan<P_THREADS>(run, E, warp_tot);
  for (int e = threadIdx.x; e < E; e += P_THREADS) {
    if (off64) off64[e] = run[e];
    if (off32) off32[e] = run[e];
  }
  if (threadIdx.x == 0) {
    if (off64) off64[E] = total;
    if (off32) off32[E] = total;
  }
  __syncthreads();
  place_segment<IDS64, P_THREADS>(ids, 0, S, E, run, perm, inv);
}

// ---------------------------------------------------------------------------------------------
// out[p,:] = x[perm[p] / K, :], one warp per row, 16-byte copies (row_bytes % 16 == 0).
__global__ void __launch_bounds__(256)
gather_rows_vec(const uint4* __restrict__ x, const int32_t* __restrict__ perm, int64_t S, int K,
                int vec_per_row, uint4* __restrict__ out) {
  const int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p >= S) return;
  const int lane = threadIdx.x & 31;
  const int64_t src = perm[p] / K;
  const uint4* s = x + src * vec_per_row;
  uint4* d = out + p * vec_per_row;
  for (int v = lane; v < vec_per_row; v += 32) d[v] = __ldg(s + v);
}

__global__ void __launch_bounds__(256)
gather_rows_bytes(const uint8_t* __restrict__ x, const int32_t* __restrict__ perm, int64_t S, int K,
                  int64_t row_bytes, uint8_t* __restrict__ out) {
  const int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p >= S) return;
  const int lane = threadIdx.x & 31;
  const int64_t src = perm[p] / K;
  for (int64_t b = lane; b < row_bytes; b += 32) out[p * row_bytes + b] = x[src * row_bytes + b];
}

// ---------------------------------------------------------------------------------------------
// out[t,h] = cast( sum_k w[t,k] * float(rows[inv[t*K+k], h]) ): the product is rounded to fp32
// before the add (no FMA contraction), k ascending, as a tensor multiply followed by sum(dim=1).
// With `residual` the decoder layer's add follows (mini_qwen/model/qwen3_moe.py:66): the block output is
// first rounded to the model type, then out = cast(float(residual) + float(block output)).
template <typename T>
__device__ __forceinline__ T finish_combine(float acc, const T* residual, int64_t at) {
  const T o = from_float<T>(acc);
  return residual ? from_float<T>(__fadd_rn(to_float<T>(residual[at]), to_float<T>(o))) : o;
}

template <typename T>
__global__ void __launch_bounds__(128)
unpermute_combine(const T* __restrict__ rows, const float* __restrict__ weights,
                  const int32_t* __restrict__ inv, const T* __restrict__ residual, int K, int64_t H,
                  T* __restrict__ out) {
  __shared__ int s_row[32];
  __shared__ float s_w[32];
  const int64_t t = blockIdx.x;
  pdl_wait();                     // the rows come from the kernel before this one
  pdl_release();
  if (threadIdx.x < K) {
    s_row[threadIdx.x] = inv[t * K + threadIdx.x];
    s_w[threadIdx.x] = weights[t * K + threadIdx.x];
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);
  const int64_t h0 = ((int64_t)blockIdx.y * 128 + threadIdx.x) * V;
  if (h0 >= H) return;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.0f;
  if (h0 + V <= H && (H % V) == 0) {
    for (int k = 0; k < K; ++k) {
      const float wk = s_w[k];
      uint4 raw = *reinterpret_cast<const uint4*>(rows + (int64_t)s_row[k] * H + h0);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(wk, to_float<T>(v[j])));
    }
    T o[V];
    if (residual) {
      const uint4 rraw = *reinterpret_cast<const uint4*>(residual + t * H + h0);
      const T* rv = reinterpret_cast<const T*>(&rraw);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = finish_combine<T>(acc[j], rv, j);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = from_float<T>(acc[j]);
    }
    *reinterpret_cast<uint4*>(out + t * H + h0) = *reinterpret_cast<const uint4*>(o);
  } else {
    for (int j = 0; j < V && h0 + j < H; ++j) {
      float a = 0.0f;
      for (int k = 0; k < K; ++k)
        a = __fadd_rn(a, __fmul_rn(s_w[k], to_float<T>(rows[(int64_t)s_row[k] * H + h0 + j])));
      out[t * H + h0 + j] = finish_combine<T>(a, residual, t * H + h0 + j);
    }
  }
}

template <typename T>
int launch_combine(const void* rows, const float* weights, const int32_t* inv, const void* residual, int64_t T_,
                   int K, int64_t H, void* out, cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  dim3 grid((unsigned)T_, (unsigned)((H + 128 * V - 1) / (128 * V)));
  launch_after_predecessor(unpermute_combine<T>, grid, dim3(128), 0, st, reinterpret_cast<const T*>(rows), weights, inv,
                           reinterpret_cast<const T*>(residual), K, H, reinterpret_cast<T*>(out));
  return check_launch();
}

}  // namespace
}  // namespace mq

extern "C" size_t mq_permute_workspace_bytes(int64_t S, int64_t E) {
  if (S <= 0 || E <= 0) return 16;
  int64_t nseg = (S + mq::P_SEG - 1) / mq::P_SEG;
  return (size_t)(nseg * E) * sizeof(int32_t) + (size_t)(E + 1) * sizeof(int32_t) + 16;
}

extern "C" int mq_permute_plan(const void* ids, int ids_are_64, int64_t T, int64_t K, int64_t E,
                               int32_t* perm, int32_t* inv, int64_t* offsets64, int32_t* offsets32,
                               void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  if (T < 0 || K <= 0 || E <= 0) return MQ_ERR_INVALID_ARGUMENT;
  if (E > P_MAX_E || T * K >= (int64_t)1 << 31) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (!offsets64 && !offsets32) return MQ_ERR_INVALID_ARGUMENT;
  const int64_t S = T * K;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (S > 0 && (!ids || !perm || !inv)) return MQ_ERR_INVALID_ARGUMENT;

  if (S <= P_SMALL) {
    // also covers S == 0: the kernel then only writes zero offsets
    if (ids_are_64) permute_plan_small<true><<<1, P_THREADS, 0, st>>>(ids, S, (int)E, perm, inv, offsets64, offsets32);
    else permute_plan_small<false><<<1, P_THREADS, 0, st>>>(ids, S, (int)E, perm, inv, offsets64, offsets32);
    return check_launch();
  }
  if (!workspace || workspace_bytes < mq_permute_workspace_bytes(S, E)) return MQ_ERR_WORKSPACE_TOO_SMALL;
  const int nseg = (int)((S + P_SEG - 1) / P_SEG);
  int32_t* seg_hist = reinterpret_cast<int32_t*>(workspace);
  int32_t* totals = seg_hist + (size_t)nseg * E;
  if (ids_are_64) permute_hist<true><<<nseg, P_THREADS, 0, st>>>(ids, S, (int)E, seg_hist);
  else permute_hist<false><<<nseg, P_THREADS, 0, st>>>(ids, S, (int)E, seg_hist);
  permute_scan<<<(unsigned)((E + P_THREADS / 32 - 1) / (P_THREADS / 32)), P_THREADS, 0, st>>>(seg_hist, nseg, (int)E, totals);
  if (ids_are_64)
    permute_place<true><<<nseg, P_THREADS, 0, st>>>(ids, S, (int)E, nseg, seg_hist, totals, offsets64, offsets32, perm, inv);
  else
    permute_place<false><<<nseg, P_THREADS, 0, st>>>(ids, S, (int)E, nseg, seg_hist, totals, offsets64, offsets32, perm, inv);
  return check_launch();
}

extern "C" int mq_gather_rows(const void* x, int dtype, const int32_t* perm, int64_t S, int64_t K, int64_t H,
                              void* out, void* stream) {
  using namespace mq;
  if (S < 0 || K <= 0 || H <= 0 || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (S == 0) return MQ_OK;
  if (!x || !perm || !out) return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t row_bytes = H * (int64_t)dtype_size(dtype);
  const unsigned blocks = (unsigned)((S + 7) / 8);
  if (row_bytes % 16 == 0 && aligned16(x) && aligned16(out)) {
    gather_rows_vec<<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(x), perm, S, (int)K,
                                            (int)(row_bytes / 16), reinterpret_cast<uint4*>(out));
  } else {
    gather_rows_bytes<<<blocks, 256, 0, st>>>(reinterpret_cast<const uint8_t*>(x), perm, S, (int)K, row_bytes,
                                              reinterpret_cast<uint8_t*>(out));
  }
  return check_launch();
}

extern "C" int mq_unpermute_combine_residual(const void* rows, int dtype, const float* weights, const int32_t* inv,
                                             const void* residual, int64_t T, int64_t K, int64_t H, void* out,
                                             void* stream) {
  using namespace mq;
  if (T < 0 || K <= 0 || H <= 0 || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (K > 32) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!rows || !weights || !inv || !out) return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(rows) || !aligned16(out) || !aligned16(residual)) return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MQ_F32) return launch_combine<float>(rows, weights, inv, residual, T, (int)K, H, out, st);
  if (dtype == MQ_BF16) return launch_combine<__nv_bfloat16>(rows, weights, inv, residual, T, (int)K, H, out, st);
  return launch_combine<__half>(rows, weights, inv, residual, T, (int)K, H, out, st);
}

extern "C" int mq_unpermute_combine(const void* rows, int dtype, const float* weights, const int32_t* inv,
                                    int64_t T, int64_t K, int64_t H, void* out, void* stream) {
  return mq_unpermute_combine_residual(rows, dtype, weights, inv, nullptr, T, K, H, out, stream);
}
