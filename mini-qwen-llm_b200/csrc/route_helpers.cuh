// Device helpers shared by the routing kernels: the per-token softmax / top-k of the router and the
// block-level pieces of the expert-sorted permute plan (a stable counting sort of the slots by expert id).
#pragma once

#include <climits>

#include "common.cuh"

namespace mq {

// One warp, one token: fp32 softmax over the E logits of the row (the K slices of the logits are summed in
// ascending order first), then K rounds of warp arg-max on (score, -id): descending scores, equal scores to
// the lower expert id.  Follows mini_qwen/kernels/moe_router.py:20-21 and the renormalisation of
// mini_qwen/model/layers/moe.py:55-56.  p: the token's row in the first logits slice; the rows of the
// other slices are slice_stride floats apart.
template <int NS>
__device__ __forceinline__ float sum_slices(const float* p, size_t stride) {
  float part[NS];
#pragma unroll
  for (int sl = 0; sl < NS; ++sl) part[sl] = p[sl * stride];
  float v = part[0];
#pragma unroll
  for (int sl = 1; sl < NS; ++sl) v += part[sl];
  return v;
}

template <int EPL>
__device__ __forceinline__ void softmax_topk_row(const float* __restrict__ p, int slices, size_t slice_stride,
                                                 const float* __restrict__ bias, int E, int K, int renorm, int lane,
                                                 int64_t* __restrict__ ids64_row, int32_t* __restrict__ ids32_row,
                                                 float* __restrict__ weights_row) {
  float s[EPL];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    int e = lane + 32 * j;
    float v = -INFINITY;
    if (e < E) {
      // the K slices are summed in ascending order; the usual counts are unrolled (loads first, then adds)
      const float* q = p + e;
      if (slices == 1) v = sum_slices<1>(q, slice_stride);
      else if (slices == 2) v = sum_slices<2>(q, slice_stride);
      else if (slices == 3) v = sum_slices<3>(q, slice_stride);
      else if (slices == 4) v = sum_slices<4>(q, slice_stride);
      else {
        v = q[0];
        for (int sl = 1; sl < slices; ++sl) v += q[sl * slice_stride];
      }
      if (bias != nullptr) v += bias[e];
    }
    s[j] = v;
    m = fmaxf(m, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    int e = lane + 32 * j;
    float pe = (e < E) ? expf(s[j] - m) : 0.0f;
    s[j] = pe;
    sum += pe;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int j = 0; j < EPL; ++j) s[j] = (lane + 32 * j < E) ? s[j] / sum : -1.0f;  // scores >= 0; -1 = absent

  // Selection on the scores' bit patterns: a non-negative float orders like its bits read as a signed integer,
  // so one warp-wide integer maximum finds the best score and one integer minimum over the lanes that hold it
  // finds the lowest expert id among equals (two reductions per round instead of a shuffle tree on pairs).
  int key[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) key[j] = (lane + 32 * j < E) ? __float_as_int(s[j]) : INT_MIN;
  float my_w = 0.0f;
  int my_id = 0;
  float wsum = 0.0f;
  for (int k = 0; k < K; ++k) {
    int best = INT_MIN, best_j = 0;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      // ascending j = ascending id within the lane, strict > keeps the lower id on ties
      if (key[j] > best) { best = key[j]; best_j = j; }
    }
    const int top = __reduce_max_sync(0xffffffffu, best);
    const int id = __reduce_min_sync(0xffffffffu, best == top ? lane + 32 * best_j : INT_MAX);
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (lane + 32 * j == id) key[j] = INT_MIN;
    const float score = __int_as_float(top);
    if (lane == k) { my_w = score; my_id = id; }
    wsum += score;
  }
  if (lane < K) {
    float wv = renorm ? my_w / wsum : my_w;
    weights_row[lane] = wv;
    if (ids64_row != nullptr) ids64_row[lane] = my_id;
    if (ids32_row != nullptr) ids32_row[lane] = my_id;
  }
}

// The same selection with EIGHT lanes per token, four tokens per warp at a time (for many tokens on few warps).
// Sub-lane sl of a token's group holds experts sl, sl + 8, ...; the reductions are three-level butterflies inside
// the group.  The scores' sum runs in another order than in softmax_topk_row, so weights may differ from it in the
// last place.  All 32 lanes must call it together; a group whose `live` is false computes on its row but stores
// nothing.  K <= 32, E <= 8 * EPS.
template <int EPS>
__device__ __forceinline__ void softmax_topk_sub8(const float* __restrict__ row, const float* __restrict__ bias, int E,
                                                  int K, int renorm, int sl, bool live,
                                                  int64_t* __restrict__ ids64_row, int32_t* __restrict__ ids32_row,
                                                  float* __restrict__ weights_row) {
  float s[EPS];
  float m = -INFINITY;
#pragma unroll
  for (int j = 0; j < EPS; ++j) {
    const int e = sl + 8 * j;
    float v = -INFINITY;
    if (e < E) {
      v = row[e];
      if (bias != nullptr) v += bias[e];
    }
    s[j] = v;
    m = fmaxf(m, v);
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < EPS; ++j) {
    const float pe = (sl + 8 * j < E) ? expf(s[j] - m) : 0.0f;
    s[j] = pe;
    sum += pe;
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  int key[EPS];
#pragma unroll
  for (int j = 0; j < EPS; ++j) key[j] = (sl + 8 * j < E) ? __float_as_int(s[j] / sum) : INT_MIN;
  float my_w[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  int my_id[4] = {0, 0, 0, 0};
  float wsum = 0.0f;
  for (int k = 0; k < K; ++k) {
    int best = INT_MIN, id = INT_MAX;
#pragma unroll
    for (int j = 0; j < EPS; ++j) {
      if (key[j] > best) { best = key[j]; id = sl + 8 * j; }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const int ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (ob > best || (ob == best && oi < id)) { best = ob; id = oi; }
    }
#pragma unroll
    for (int j = 0; j < EPS; ++j)
      if (sl + 8 * j == id) key[j] = INT_MIN;
    const float score = __int_as_float(best);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (k == sl + 8 * q) { my_w[q] = score; my_id[q] = id; }
    wsum += score;
  }
  if (live) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = sl + 8 * q;
      if (k < K) {
        weights_row[k] = renorm ? my_w[q] / wsum : my_w[q];
        if (ids64_row != nullptr) ids64_row[k] = my_id[q];
        if (ids32_row != nullptr) ids32_row[k] = my_id[q];
      }
    }
  }
}

template <bool IDS64>
__device__ __forceinline__ int load_id(const void* ids, int64_t i) {
  if (IDS64) return (int)reinterpret_cast<const int64_t*>(ids)[i];
  return reinterpret_cast<const int32_t*>(ids)[i];
}

// Exclusive scan over v[0..E) in shared memory (E <= 4 * THREADS), all THREADS threads of the CTA; returns the total.
template <int THREADS>
__device__ int block_exclusive_scan(int* v, int E, int* warp_tot /* shared [THREADS / 32] */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int local[4];
  int sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int e = tid * 4 + j;
    local[j] = (e < E) ? v[e] : 0;
    sum += local[j];
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int base = 0, total = 0;
#pragma unroll
  for (int wi = 0; wi < THREADS / 32; ++wi) {
    int wt = warp_tot[wi];
    if (wi < warp) base += wt;
    total += wt;
  }
  int run = base + incl - sum;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int e = tid * 4 + j;
    if (e < E) v[e] = run;
    run += local[j];
  }
  __syncthreads();
  return total;
}

// Ranks the slots [seg_lo, seg_hi) in ascending order; run[e] holds the next free sorted
// position of expert e on entry and is advanced.  One warp at a time touches run[], which keeps
// the placement stable without atomics.
template <bool IDS64, int THREADS>
__device__ void place_segment(const void* ids, int64_t seg_lo, int64_t seg_hi, int E, int* run,
                              int32_t* perm, int32_t* inv) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t c0 = seg_lo; c0 < seg_hi; c0 += THREADS) {
    const int64_t i = c0 + tid;
    int e = -1;
    if (i < seg_hi) {
      e = load_id<IDS64>(ids, i);
      if ((unsigned)e >= (unsigned)E) e = -1;   // an id outside [0,E) is left unplaced
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    for (int wi = 0; wi < THREADS / 32; ++wi) {
      if (warp == wi && e >= 0) {
        const int pos = run[e] + rank;
        __syncwarp(peers);
        if (rank == 0) run[e] += __popc(peers);
        perm[pos] = (int32_t)i;
        inv[i] = pos;
      }
      __syncthreads();
    }
  }
}


}  // namespace mq
