// Expert-parallel exchange fused into the permute and combine kernels, over peer memory.
//
// The reference has no distributed code; the exchange exists because the 128 experts are sharded
// over the GPUs of one NVSwitch box.  Instead of materialising the expert-sorted rows locally and
// then moving them with a collective, the dispatch kernel gathers each token row straight into the
// receive buffer of the GPU that owns its expert (16-byte peer stores over NVLink), and the combine
// kernel reads each expert output row straight from the GPU that produced it (16-byte peer loads)
// while forming the weighted sum.  Ordering between the ranks is a flag barrier on the stream
// (ep_barrier_kernel, and the same code inside ep_exchange_plan_kernel): a rank writes its epoch into
// every peer's signal array and polls its own array until every peer's epoch has arrived.  The poll is
// bounded (EP_SPIN_LIMIT polls by default, one to two seconds); when it runs out the kernel sets
// MQ_DEV_WAIT_EXPIRED, leaves a plan that sends and computes nothing, and returns.  The ranks of a group
// must therefore enter a layer call within that time of one another, and the caller has to read the
// status word before it trusts an output.  The data kernels (dispatch, combine) wait on nobody.
//
// Receive layout on every rank: slots grouped by local expert and, inside an expert, by source rank
// (each source's slots in its own expert-sorted order).  The grouped GEMM kernels see E_local ordinary
// groups, each expert's weights are streamed once, and rows bound for different ranks alternate
// inside every tile, which spreads the NVLink traffic of the way back over the whole kernel.
#include "common.cuh"

namespace mq {
namespace {

constexpr int EP_MAX_G = 8;
constexpr int HOME_BITS = 26;        // home code of a slot: source rank << 26 | position in the source's sorted order

// From the gathered per-expert counts [G, E]:
//   send_base[e]  = slot in the owner's receive order where this rank's slots for expert e start
//   seg_offsets[] = prefix sums of this rank's own E/G receive groups (one per local expert)
__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ all_counts, int G, int rank, int E,
               int32_t* __restrict__ send_base, int32_t* __restrict__ seg_offsets) {
  const int el = E / G;
  // one thread per expert: slots of the owner's earlier experts (all sources), then earlier sources'
  // slots of this expert.  At most E additions each.
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / el, j = e - d * el;
    int base = 0;
    for (int jj = 0; jj < j; ++jj)
      for (int s = 0; s < G; ++s) base += all_counts[s * E + d * el + jj];
    for (int s = 0; s < rank; ++s) base += all_counts[s * E + e];
    send_base[e] = base;
  }
  // own receive groups
  if (threadIdx.x == 0) {
    int run = 0;
    for (int j = 0; j < el; ++j) {
      seg_offsets[j] = run;
      for (int s = 0; s < G; ++s) run += all_counts[s * E + rank * el + j];
    }
    seg_offsets[el] = run;
  }
}

// Per-expert slot counts of this rank (differences of its offsets) into row `rank` of every peer's
// counts table: an all-gather made of E * G 4-byte peer stores.
__global__ void __launch_bounds__(256)
ep_share_counts_kernel(const int32_t* __restrict__ offsets, int E, int G, int rank,
                       const uint64_t* __restrict__ peer_counts) {
  for (int i = threadIdx.x; i < E * G; i += blockDim.x) {
    const int d = i / E, e = i - d * E;
    reinterpret_cast<int32_t*>(peer_counts[d])[rank * E + e] = offsets[e + 1] - offsets[e];
  }
}

// Barrier across the ranks of the group, on the stream: every rank bumps its epoch, writes it into its
// slot of every peer's signal array and waits until all slots of its own array have reached the epoch.
// The wait is bounded; when it runs out the kernel records MQ_DEV_WAIT_EXPIRED and returns, so a
// missing rank costs a second, not a hang.
constexpr uint32_t EP_SPIN_LIMIT = 1u << 22;
constexpr int EP_DROP_BASE = 0x3FFFFFFF;         // send_base of a plan that must not send: beyond every buffer

__global__ void __launch_bounds__(32)
ep_barrier_kernel(const uint64_t* __restrict__ peer_sig, int32_t* __restrict__ epoch_ctr, int G, int rank,
                  uint32_t max_polls, int32_t* __restrict__ status) {
  __shared__ int s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_ctr + 1;
    *epoch_ctr = s_epoch;
  }
  __syncwarp();
  const int epoch = s_epoch;
  __threadfence_system();                        // earlier kernels' peer stores are complete; order the flag behind them
  for (int r = threadIdx.x; r < G; r += 32) {
    int32_t* remote = reinterpret_cast<int32_t*>(peer_sig[r]) + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  const int32_t* mine = reinterpret_cast<const int32_t*>(peer_sig[rank]);
  for (int r = threadIdx.x; r < G; r += 32) {
    uint32_t spin = 0;
    int v;
    do {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + r) : "memory");
    } while (v < epoch && ++spin < max_polls);
    if (v < epoch) atomicOr(status, (int)MQ_DEV_WAIT_EXPIRED);
  }
}

// The three steps that open a layer call in one launch: this rank's counts go into every peer's table,
// the ranks meet (same bounded barrier as above), and the plan is formed from the now complete table.
__global__ void __launch_bounds__(256)
ep_exchange_plan_kernel(const int32_t* __restrict__ offsets, int E, int G, int rank,
                        const uint64_t* __restrict__ peer_counts, const uint64_t* __restrict__ peer_sig,
                        int32_t* __restrict__ epoch_ctr, int32_t* __restrict__ send_base,
                        int32_t* __restrict__ seg_offsets, uint32_t max_polls, int32_t* __restrict__ status) {
  __shared__ int s_epoch;
  __shared__ int s_expired;
  __shared__ int s_tot[1024];                    // slots per expert over all sources
  if (threadIdx.x == 0) s_expired = 0;
  const int el = E / G;
  for (int i = threadIdx.x; i < E * G; i += blockDim.x) {
    const int d = i / E, e = i - d * E;
    reinterpret_cast<int32_t*>(peer_counts[d])[rank * E + e] = offsets[e + 1] - offsets[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    if (threadIdx.x == 0) {
      s_epoch = *epoch_ctr + 1;
      *epoch_ctr = s_epoch;
    }
    __syncwarp();
    const int epoch = s_epoch;
    __threadfence_system();
    for (int r = threadIdx.x; r < G; r += 32) {
      int32_t* remote = reinterpret_cast<int32_t*>(peer_sig[r]) + rank;
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    }
    const int32_t* mine = reinterpret_cast<const int32_t*>(peer_sig[rank]);
    for (int r = threadIdx.x; r < G; r += 32) {
      uint32_t spin = 0;
      int v;
      do {
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + r) : "memory");
      } while (v < epoch && ++spin < max_polls);
      if (v < epoch) {
        atomicOr(status, (int)MQ_DEV_WAIT_EXPIRED);
        s_expired = 1;
      }
    }
  }
  __syncthreads();
  if (s_expired) {
    // A rank did not arrive: its row of the counts table is stale or was never written.  Leave a plan that
    // sends nothing (every slot's row number lies beyond any receive buffer, so the dispatch kernels drop
    // it) and gives the grouped kernels no rows, instead of one built from those counts.
    for (int e = threadIdx.x; e < E; e += blockDim.x) send_base[e] = EP_DROP_BASE;
    for (int j = threadIdx.x; j <= el; j += blockDim.x) seg_offsets[j] = 0;
    return;
  }
  const int32_t* all_counts = reinterpret_cast<const int32_t*>(peer_counts[rank]);   // [G, E], written by the peers
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0;
    for (int s = 0; s < G; ++s) tot += __ldcg(all_counts + s * E + e);
    s_tot[e] = tot;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / el;
    int base = 0;
    for (int ee = d * el; ee < e; ++ee) base += s_tot[ee];
    for (int s = 0; s < rank; ++s) base += __ldcg(all_counts + s * E + e);
    send_base[e] = base;
  }
  for (int j = threadIdx.x; j <= el; j += blockDim.x) {
    int run = 0;
    for (int jj = 0; jj < j; ++jj) run += s_tot[rank * el + jj];
    seg_offsets[j] = run;
  }
}

// One warp per expert-sorted slot p: copy the token row to the owner's receive buffer.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ perm,
                   const int32_t* __restrict__ offsets, const int32_t* __restrict__ send_base,
                   int64_t S, int K, int vec_per_row, int E, int el, const uint64_t* __restrict__ peer_recv,
                   const uint64_t* __restrict__ peer_home, int rank,
                   int64_t cap_rows, int32_t* __restrict__ slot_dst, int32_t* __restrict__ status) {
  const int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (p >= S) return;
  const int lane = threadIdx.x & 31;
  // expert of sorted position p: last e with offsets[e] <= p
  int lo = 0, hi = E;                       // invariant: offsets[lo] <= p < offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= (int)p) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int d = e / el;
  const int64_t row = (int64_t)send_base[e] + (p - offsets[e]);
  if (row < 0 || row >= cap_rows) {         // outside the receive buffer (too small, or a plan that sends nothing)
    if (lane == 0) { atomicOr(status, 2); slot_dst[p] = -1; }
    return;
  }
  if (lane == 0) {
    slot_dst[p] = (int32_t)(d * cap_rows + row);
    // where the slot's output row goes home to: (this rank, sorted position p)
    if (peer_home != nullptr) reinterpret_cast<int32_t*>(peer_home[d])[row] = (rank << HOME_BITS) | (int32_t)p;
  }
  const uint4* src = x + (int64_t)(perm[p] / K) * vec_per_row;
  uint4* dst = reinterpret_cast<uint4*>(peer_recv[d]) + row * vec_per_row;
  for (int v = lane; v < vec_per_row; v += 32) dst[v] = __ldg(src + v);
}

// ---- dispatch with one copy per (token, destination rank) instead of one per slot.
// A token with several of its K experts on the same GPU needs its row there once.  uniq[d, t] is the
// index of token t among this rank's tokens that have at least one expert on rank d (token order), or
// -1; the row travels to row rank * src_stride + uniq[d, t] of rank d's receive buffer, and every
// slot carries only that row number (4 bytes) to its place in the (source, local expert) order.  The
// gate/up kernel of the owner then gathers its rows through those numbers.


// One CTA of 1024 threads; a pass covers 4096 tokens, four consecutive ones per thread.  The per-rank
// counts of a thread's tokens travel through the scans packed 16 bits per rank in two 64-bit words
// (a pass never counts past 4096), so one warp scan and one scan of the 32 warp totals serve all ranks.
__global__ void __launch_bounds__(1024)
ep_unique_rows_kernel(const int32_t* __restrict__ ids, int T, int K, int el, int G, int32_t* __restrict__ uniq) {
  __shared__ unsigned long long s_warp[32][2];
  __shared__ int s_carry[EP_MAX_G];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned long long magic = 0x100000000ull / (unsigned)el + 1ull;      // id / el = (id * magic) >> 32 for id, el < 2^16
  auto owner = [&](int id) { return (unsigned)(((unsigned long long)(unsigned)id * magic) >> 32); };
  const bool vec = (K & 3) == 0 && ((reinterpret_cast<uintptr_t>(ids) & 15) == 0);
  if (threadIdx.x < EP_MAX_G) s_carry[threadIdx.x] = 0;
  __syncthreads();
  for (int t0 = 0; t0 < T; t0 += 4096) {
    const int tb = t0 + 4 * threadIdx.x;            // this thread's tokens tb .. tb+3
    unsigned mask[4];
    unsigned long long cnt[2] = {0ull, 0ull};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      unsigned m = 0;
      const int t = tb + i;
      if (t < T) {
        const int32_t* row = ids + (int64_t)t * K;
        if (vec) {
          for (int k = 0; k < K; k += 4) {
            const int4 v = *reinterpret_cast<const int4*>(row + k);
            m |= 1u << owner(v.x);
            m |= 1u << owner(v.y);
            m |= 1u << owner(v.z);
            m |= 1u << owner(v.w);
          }
        } else {
          for (int k = 0; k < K; ++k) m |= 1u << owner(row[k]);
        }
      }
      mask[i] = m;
#pragma unroll
      for (int d = 0; d < EP_MAX_G; ++d) cnt[d >> 2] += (unsigned long long)((m >> d) & 1u) << (16 * (d & 3));
    }
    // inclusive warp scan of the packed counts
    unsigned long long inc[2] = {cnt[0], cnt[1]};
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, inc[h], o);
        if (lane >= o) inc[h] += up;
      }
    }
    if (lane == 31) { s_warp[warp][0] = inc[0]; s_warp[warp][1] = inc[1]; }
    __syncthreads();
    if (warp == 0) {                                // exclusive scan of the 32 warp totals
      unsigned long long v[2] = {s_warp[lane][0], s_warp[lane][1]}, w[2] = {v[0], v[1]};
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const unsigned long long up = __shfl_up_sync(0xffffffffu, w[h], o);
          if (lane >= o) w[h] += up;
        }
      }
      s_warp[lane][0] = w[0] - v[0];
      s_warp[lane][1] = w[1] - v[1];
    }
    __syncthreads();
    int base[EP_MAX_G];                             // tokens before this thread's first, per rank
#pragma unroll
    for (int d = 0; d < EP_MAX_G; ++d) {
      const int h = d >> 2, sh = 16 * (d & 3);
      base[d] = s_carry[d] + (int)((s_warp[warp][h] >> sh) & 0xffffu) + (int)(((inc[h] - cnt[h]) >> sh) & 0xffffu);
    }
    // uniq is rank-major [G][T]: a thread's four tokens are 16 contiguous bytes per rank
    const bool vec_out = (T & 3) == 0 && ((reinterpret_cast<uintptr_t>(uniq) & 15) == 0);
#pragma unroll
    for (int d = 0; d < EP_MAX_G; ++d) {
      int v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool hit = (mask[i] >> d) & 1u;
        v[i] = hit ? base[d] : -1;
        base[d] += hit ? 1 : 0;
      }
      if (d < G) {
        int32_t* dst = uniq + (int64_t)d * T + tb;
        if (vec_out && tb + 3 < T) {
          *reinterpret_cast<int4*>(dst) = make_int4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (tb + i < T) dst[i] = v[i];
        }
      }
    }
    __syncthreads();                                // every thread has read s_warp and s_carry
    if (threadIdx.x == 1023) {                      // the last thread's running counts are the pass totals
#pragma unroll
      for (int d = 0; d < EP_MAX_G; ++d) s_carry[d] = base[d];
    }
    __syncthreads();
  }
}

// Blocks [0, row_blocks): one warp per token, the row is read once and stored to every rank that needs it.
// Blocks after: one thread per expert-sorted slot, the slot's row number goes to its owner.
__global__ void __launch_bounds__(256)
ep_dispatch_unique_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ uniq,
                          const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets,
                          const int32_t* __restrict__ send_base, int T, int64_t S, int K, int vec_per_row, int E,
                          int el, int G, int rank, int src_stride, int row_blocks,
                          const uint64_t* __restrict__ peer_recv, const uint64_t* __restrict__ peer_ridx,
                          const uint64_t* __restrict__ peer_home,
                          int64_t cap_rows, int32_t* __restrict__ slot_dst, int32_t* __restrict__ status) {
  if ((int)blockIdx.x < row_blocks) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= T) return;
    const int lane = threadIdx.x & 31;
    const int mine = lane < G ? uniq[(int64_t)lane * T + t] : -1;
    const uint4* src = x + (int64_t)t * vec_per_row;
    // consecutive tokens start with different ranks, so that the stores of the warps in flight spread
    // over all links instead of visiting the ranks in step
    const int rot = t & (EP_MAX_G - 1);
    // four 16-byte pieces per lane are loaded before the first store, so that a row's loads overlap
    for (int v0 = lane; v0 < vec_per_row; v0 += 4 * 32) {
      uint4 val[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (v0 + 32 * i < vec_per_row) val[i] = __ldg(src + v0 + 32 * i);
#pragma unroll
      for (int dd = 0; dd < EP_MAX_G; ++dd) {
        const int d = (dd + rot) & (EP_MAX_G - 1);
        const int u = __shfl_sync(0xffffffffu, mine, d);
        if (u >= 0) {
          uint4* dst = reinterpret_cast<uint4*>(peer_recv[d]) + ((int64_t)rank * src_stride + u) * vec_per_row;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (v0 + 32 * i < vec_per_row) dst[v0 + 32 * i] = val[i];
        }
      }
    }
    return;
  }
  const int64_t p = (int64_t)(blockIdx.x - row_blocks) * 256 + threadIdx.x;
  if (p >= S) return;
  int lo = 0, hi = E;                       // expert of sorted position p: offsets[lo] <= p < offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= (int)p) lo = mid; else hi = mid;
  }
  const int e = lo, d = e / el;
  const int64_t row = (int64_t)send_base[e] + (p - offsets[e]);
  if (row < 0 || row >= cap_rows) {         // outside the owner's slot table (too small, or a plan that sends nothing)
    atomicOr(status, 2);
    slot_dst[p] = -1;
    return;
  }
  slot_dst[p] = (int32_t)(d * cap_rows + row);
  reinterpret_cast<int32_t*>(peer_ridx[d])[row] = rank * src_stride + uniq[(int64_t)d * T + perm[p] / K];
  if (peer_home != nullptr) reinterpret_cast<int32_t*>(peer_home[d])[row] = (rank << HOME_BITS) | (int32_t)p;
}

// out[t,:] = cast(sum_k w[t,k] * float(y_on_owner[slot row, :])), fp32 multiply then add, k ascending.
template <typename T>
__global__ void __launch_bounds__(128)
ep_combine_kernel(const uint64_t* __restrict__ peer_y, const float* __restrict__ weights,
                  const int32_t* __restrict__ inv, const int32_t* __restrict__ slot_dst,
                  const T* __restrict__ residual, int K, int64_t H, int64_t cap_rows, T* __restrict__ out) {
  __shared__ const T* s_row[32];
  __shared__ float s_w[32];
  const int64_t t = blockIdx.x;
  if (threadIdx.x < K) {
    const int v = slot_dst[inv[t * K + threadIdx.x]];
    const T* row = nullptr;
    if (v >= 0) {
      const int d = (int)(v / cap_rows);
      row = reinterpret_cast<const T*>(peer_y[d]) + (int64_t)(v - d * cap_rows) * H;
    }
    s_row[threadIdx.x] = row;
    s_w[threadIdx.x] = weights[t * K + threadIdx.x];
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);
  const int64_t h0 = ((int64_t)blockIdx.y * 128 + threadIdx.x) * V;
  if (h0 >= H) return;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.0f;
  // peer loads go out eight at a time before their first use (NVLink latency is microseconds)
  for (int k0 = 0; k0 < K; k0 += 8) {
    uint4 raw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const T* row = k0 + i < K ? s_row[k0 + i] : nullptr;
      raw[i] = row ? *reinterpret_cast<const uint4*>(row + h0) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (k0 + i < K) {
        const float wk = s_w[k0 + i];
        const T* v = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(wk, to_float<T>(v[j])));
      }
    }
  }
  T o[V];
#pragma unroll
  for (int j = 0; j < V; ++j) o[j] = from_float<T>(acc[j]);
  if (residual) {
    // the decoder layer's add of two model-type tensors: the block output is rounded first
    const uint4 rraw = *reinterpret_cast<const uint4*>(residual + t * H + h0);
    const T* rv = reinterpret_cast<const T*>(&rraw);
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = from_float<T>(__fadd_rn(to_float<T>(rv[j]), to_float<T>(o[j])));
  }
  *reinterpret_cast<uint4*>(out + t * H + h0) = *reinterpret_cast<const uint4*>(o);
}

template <typename T>
int launch_ep_combine(const uint64_t* peer_y, const float* weights, const int32_t* inv, const int32_t* slot_dst,
                      const void* residual, int64_t T_, int K, int64_t H, int64_t cap_rows, void* out,
                      cudaStream_t st) {
  constexpr int V = 16 / sizeof(T);
  dim3 grid((unsigned)T_, (unsigned)((H + 128 * V - 1) / (128 * V)));
  ep_combine_kernel<T><<<grid, 128, 0, st>>>(peer_y, weights, inv, slot_dst, reinterpret_cast<const T*>(residual), K, H,
                                            cap_rows, reinterpret_cast<T*>(out));
  return check_launch();
}

}  // namespace
}  // namespace mq

extern "C" int mq_ep_plan(const int32_t* all_counts, int64_t G, int64_t rank, int64_t E,
                          int32_t* send_base, int32_t* seg_offsets, void* stream) {
  using namespace mq;
  if (G <= 0 || E <= 0 || rank < 0 || rank >= G || E % G != 0) return MQ_ERR_INVALID_ARGUMENT;
  if (E > 1024) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (!all_counts || !send_base || !seg_offsets) return MQ_ERR_INVALID_ARGUMENT;
  ep_plan_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(all_counts, (int)G, (int)rank, (int)E,
                                                                       send_base, seg_offsets);
  return check_launch();
}

extern "C" int mq_ep_share_counts(const int32_t* offsets, int64_t E, int64_t G, int64_t rank,
                                  const uint64_t* peer_counts_ptrs, void* stream) {
  using namespace mq;
  if (E <= 0 || G <= 0 || rank < 0 || rank >= G || !offsets || !peer_counts_ptrs) return MQ_ERR_INVALID_ARGUMENT;
  ep_share_counts_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(offsets, (int)E, (int)G, (int)rank,
                                                                                peer_counts_ptrs);
  return check_launch();
}

extern "C" int mq_ep_barrier(const uint64_t* peer_signal_ptrs, int32_t* epoch_counter, int64_t G, int64_t rank,
                             int64_t max_polls, int32_t* d_status, void* stream) {
  using namespace mq;
  if (G <= 0 || rank < 0 || rank >= G || !peer_signal_ptrs || !epoch_counter || !d_status) return MQ_ERR_INVALID_ARGUMENT;
  if (max_polls < 0 || max_polls > (int64_t)EP_SPIN_LIMIT) return MQ_ERR_INVALID_ARGUMENT;
  ep_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      peer_signal_ptrs, epoch_counter, (int)G, (int)rank, max_polls ? (uint32_t)max_polls : EP_SPIN_LIMIT, d_status);
  return check_launch();
}

extern "C" int mq_ep_dispatch(const void* x, int dtype, const int32_t* perm, const int32_t* offsets,
                              const int32_t* send_base, int64_t S, int64_t K, int64_t H, int64_t E, int64_t G,
                              int64_t rank, const uint64_t* peer_recv_ptrs, const uint64_t* peer_home_ptrs,
                              int64_t cap_rows, int32_t* slot_dst, int32_t* d_status, void* stream) {
  using namespace mq;
  if (S < 0 || K <= 0 || H <= 0 || E <= 0 || G <= 0 || E % G != 0 || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (rank < 0 || rank >= G) return MQ_ERR_INVALID_ARGUMENT;
  if (cap_rows <= 0 || G * cap_rows >= ((int64_t)1 << 31)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (peer_home_ptrs && (S > ((int64_t)1 << HOME_BITS) || G > 32)) return MQ_ERR_UNSUPPORTED_SHAPE;
  const int64_t row_bytes = H * (int64_t)dtype_size(dtype);
  if (row_bytes % 16 != 0) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!x || !perm || !offsets || !send_base || !peer_recv_ptrs || !slot_dst || !d_status) return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(x)) return MQ_ERR_INVALID_ARGUMENT;
  ep_dispatch_kernel<<<(unsigned)((S + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), perm, offsets, send_base, S, (int)K, (int)(row_bytes / 16), (int)E,
      (int)(E / G), peer_recv_ptrs, peer_home_ptrs, (int)rank, cap_rows, slot_dst, d_status);
  return check_launch();
}

extern "C" int mq_ep_combine(const uint64_t* peer_y_ptrs, int dtype, const float* weights, const int32_t* inv,
                             const int32_t* slot_dst, const void* residual, int64_t T, int64_t K, int64_t H,
                             int64_t cap_rows, void* out, void* stream) {
  using namespace mq;
  if (T < 0 || K <= 0 || H <= 0 || cap_rows <= 0 || !valid_dtype(dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (K > 32 || (H * (int64_t)dtype_size(dtype)) % 16 != 0) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!peer_y_ptrs || !weights || !inv || !slot_dst || !out || !aligned16(out) || !aligned16(residual))
    return MQ_ERR_INVALID_ARGUMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == MQ_F32)
    return launch_ep_combine<float>(peer_y_ptrs, weights, inv, slot_dst, residual, T, (int)K, H, cap_rows, out, st);
  if (dtype == MQ_BF16)
    return launch_ep_combine<__nv_bfloat16>(peer_y_ptrs, weights, inv, slot_dst, residual, T, (int)K, H, cap_rows, out, st);
  return launch_ep_combine<__half>(peer_y_ptrs, weights, inv, slot_dst, residual, T, (int)K, H, cap_rows, out, st);
}

extern "C" int mq_ep_unique_rows(const int32_t* topk_ids, int64_t T, int64_t K, int64_t E, int64_t G,
                                 int32_t* uniq, void* stream) {
  using namespace mq;
  if (T < 0 || K <= 0 || E <= 0 || G <= 0 || E % G != 0) return MQ_ERR_INVALID_ARGUMENT;
  if (G > EP_MAX_G || E >= 65536 || T >= ((int64_t)1 << 31) / (K > G ? K : G)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!topk_ids || !uniq) return MQ_ERR_INVALID_ARGUMENT;
  ep_unique_rows_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(topk_ids, (int)T, (int)K,
                                                                                (int)(E / G), (int)G, uniq);
  return check_launch();
}

extern "C" int mq_ep_dispatch_unique(const void* x, int dtype, const int32_t* uniq, const int32_t* perm,
                                     const int32_t* offsets, const int32_t* send_base, int64_t T, int64_t K,
                                     int64_t H, int64_t E, int64_t G, int64_t rank, int64_t src_stride,
                                     const uint64_t* peer_recv_ptrs, const uint64_t* peer_ridx_ptrs,
                                     const uint64_t* peer_home_ptrs, int64_t cap_rows, int32_t* slot_dst,
                                     int32_t* d_status, void* stream) {
  using namespace mq;
  if (T < 0 || K <= 0 || H <= 0 || E <= 0 || G <= 0 || E % G != 0 || rank < 0 || rank >= G || !valid_dtype(dtype))
    return MQ_ERR_INVALID_ARGUMENT;
  if (G > EP_MAX_G || cap_rows <= 0 || G * cap_rows >= ((int64_t)1 << 31) || T * K > ((int64_t)1 << HOME_BITS))
    return MQ_ERR_UNSUPPORTED_SHAPE;
  // every source owns src_stride rows of every receive buffer
  if (T > src_stride || G * src_stride > cap_rows) return MQ_ERR_INVALID_ARGUMENT;
  const int64_t row_bytes = H * (int64_t)dtype_size(dtype);
  if (row_bytes % 16 != 0) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!x || !uniq || !perm || !offsets || !send_base || !peer_recv_ptrs || !peer_ridx_ptrs || !slot_dst || !d_status)
    return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(x)) return MQ_ERR_INVALID_ARGUMENT;
  const int64_t S = T * K;
  const int row_blocks = (int)((T + 7) / 8);
  const int64_t blocks = row_blocks + (S + 255) / 256;
  ep_dispatch_unique_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), uniq, perm, offsets, send_base, (int)T, S, (int)K, (int)(row_bytes / 16),
      (int)E, (int)(E / G), (int)G, (int)rank, (int)src_stride, row_blocks, peer_recv_ptrs, peer_ridx_ptrs,
      peer_home_ptrs, cap_rows, slot_dst, d_status);
  return check_launch();
}

extern "C" int mq_ep_exchange_plan(const int32_t* offsets, int64_t E, int64_t G, int64_t rank,
                                   const uint64_t* peer_counts_ptrs, const uint64_t* peer_signal_ptrs,
                                   int32_t* epoch_counter, int32_t* send_base, int32_t* seg_offsets,
                                   int64_t max_polls, int32_t* d_status, void* stream) {
  using namespace mq;
  if (E <= 0 || G <= 0 || rank < 0 || rank >= G || E % G != 0) return MQ_ERR_INVALID_ARGUMENT;
  if (max_polls < 0 || max_polls > (int64_t)EP_SPIN_LIMIT) return MQ_ERR_INVALID_ARGUMENT;
  if (E > 1024) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (!offsets || !peer_counts_ptrs || !peer_signal_ptrs || !epoch_counter || !send_base || !seg_offsets || !d_status)
    return MQ_ERR_INVALID_ARGUMENT;
  ep_exchange_plan_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      offsets, (int)E, (int)G, (int)rank, peer_counts_ptrs, peer_signal_ptrs, epoch_counter, send_base, seg_offsets,
      max_polls ? (uint32_t)max_polls : EP_SPIN_LIMIT, d_status);
  return check_launch();
}
