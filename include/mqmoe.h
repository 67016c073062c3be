/*
 * mqmoe.h - C ABI of libmqmoe.so: the MoE block of mini-qwen-llm (top-k router, expert-sorted
 * permute, grouped SwiGLU expert GEMM in bf16 and W4A16, weighted unpermute-combine) as
 * hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name starts with "h_";
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = legacy
 *     default stream), allocates nothing and keeps no state between calls (tensor maps are
 *     rebuilt per call on the host);
 *   - matrices are dense row-major; element types are given by mq_dtype;
 *   - the return value is an mq_status; a non-zero value means nothing was launched
 *     (argument checks) or the launch itself failed.  Conditions only the device can see
 *     (a bounded wait that ran out) are written to the optional `d_status` word and never
 *     trap;
 *   - "slot" = one (token, k) pair; S = T * top_k slots; slots are stored expert-sorted.
 *
 * Each entry point names the reference interface it replaces (paths inside the
 * mini-qwen-llm project).
 */
#ifndef MQMOE_H
#define MQMOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { MQ_F32 = 0, MQ_BF16 = 1, MQ_F16 = 2 } mq_dtype;

typedef enum {
  MQ_OK = 0,
  MQ_ERR_INVALID_ARGUMENT = 1,   /* null pointer, negative size, misaligned pointer */
  MQ_ERR_UNSUPPORTED_SHAPE = 2,  /* a size outside what the kernels cover (see each call) */
  MQ_ERR_WORKSPACE_TOO_SMALL = 3,
  MQ_ERR_LAUNCH_FAILED = 4,      /* cudaGetLastError() after the launch was not cudaSuccess */
  MQ_ERR_DRIVER_ENTRY = 5,       /* cuTensorMapEncodeTiled could not be resolved or failed */
  MQ_ERR_STATIC_SCRATCH_EXCEEDED = 6 /* the request needs more scratch than the library's built-in array */
} mq_status;

/* bits of the device status word */
#define MQ_DEV_WAIT_EXPIRED 1u   /* a bounded mbarrier wait gave up; the output is invalid */
#define MQ_DEV_EP_OVERFLOW 2u    /* an expert-parallel receive buffer was too small; rows were dropped */
#define MQ_DEV_BAD_LAUNCH 4u     /* a kernel found less shared memory than its layout needs; it did nothing */

int mq_version(void);
const char* mq_status_string(int status);
/* cudaGetErrorString of the last launch failure seen by this library on this thread. */
const char* mq_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * Router.  Replaces moe_router (mini_qwen/kernels/moe_router.py:7-22): fp32 logits = x . w^T
 * (+ bias), fp32 softmax over the E experts, the K largest scores in descending order; equal
 * scores are ordered by ascending expert id.  renormalize != 0 additionally divides the K
 * weights by their sum (mini_qwen/model/layers/moe.py:55-56).
 *   x [T,H] (x_dtype), w [E,H] (w_dtype), bias fp32 [E] or NULL,
 *   logits_ws: caller-provided workspace of mq_router_workspace_bytes(T, H, E) bytes (overwritten;
 *   holds the fp32 logits, in several K slices when the batch alone would not fill the GPU),
 *   ids64 int64 [T,K] and/or ids32 int32 [T,K] (either may be NULL, not both),
 *   weights fp32 [T,K].
 * Limits: 1 <= K <= E <= 1024, K <= 32.
 */
size_t mq_router_workspace_bytes(int64_t T, int64_t H, int64_t E);
int mq_router_topk(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                   int64_t T, int64_t H, int64_t E, int64_t K, int renormalize,
                   float* logits_ws, size_t logits_ws_bytes, int64_t* ids64, int32_t* ids32,
                   float* weights, void* stream);

/* Router for callers that cannot allocate.  No counterpart in the reference (its router lets
 * torch allocate whatever it needs); same results as mq_router_topk, bit for bit.
 *
 * Meant for callers that cannot give this library a workspace: code that runs where the CUDA
 * allocator must not be called, a foreign-language host (cgo, JNI, a plugin) that owns only its
 * input and output buffers, a process whose pool already holds all device memory.  The logits
 * scratch is a 10 MiB array built into the library image (each GPU that loads the library keeps it
 * until the process exits); the call itself performs no cudaMalloc / cudaFree and calls no
 * allocating routine.  The caller still passes inputs and outputs.
 *   - Limit: mq_router_workspace_bytes(T, H, E) <= 10 MiB; larger requests return
 *     MQ_ERR_STATIC_SCRATCH_EXCEEDED, nothing launched.  The request is slices * T * E * 4 bytes and
 *     the slice count falls as T grows, so it is not monotonic in T: with 128 experts and H = 2048 it
 *     peaks at 9.22 MiB (T = 9440, two slices) and is 8 MiB at T = 16384, so every batch up to 16384
 *     tokens fits (the largest that does is 20480 tokens).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps the last call's contents.  Nothing in
 *     it needs clearing (every element read is written first by the same call), but two calls
 *     whose kernels overlap on the GPU (different streams, no ordering) race on it: order them.
 */
int mq_router_topk_static(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                          int64_t T, int64_t H, int64_t E, int64_t K, int renormalize,
                          int64_t* ids64, int32_t* ids32, float* weights, void* stream);

/* ------------------------------------------------------------------------------------------
 * Router + permute plan (+ activation preparation) for small batches, in one launch.  Replaces, for decode
 * batches, the chain moe_router -> renormalise -> index work of moe_permute (mini_qwen/model/layers/moe.py:
 * 54-57) that the calls above and below make in three launches (plus mq_w4a16_tc_prep): at these sizes the
 * layer call is bound by its chain of launches.  Same ids, perm, inv and offsets as mq_router_topk followed
 * by mq_permute_plan; the weights can differ from that chain's in the last place (the fp32 logit sums run in
 * another order).  Up to 16 tokens: a CTA per expert, the last CTA selects and plans; 17 to 64 tokens with
 * 16-bit x and w: a CTA per (32 experts, token), the last CTA of a token selects, the last token's CTA plans.
 *   workspace: mq_route_small_workspace_bytes(T, E) bytes, 16-byte aligned, ZERO-FILLED ONCE by the caller
 *     after allocating it (it holds counters the kernel leaves at zero again, in its first 512 bytes, and the
 *     logits behind them); calls that share a workspace may differ in T and must not overlap on the GPU;
 *   ids32 int32 [T,K] (required), ids64 int64 [T,K] (optional), weights fp32 [T,K], perm/inv int32 [T*K],
 *     offsets64 / offsets32 [E+1] (one may be NULL);
 *   xp [T,H] (16-bit) and xs fp32 [T,32], both or neither: every token row in the k order 0,4,1,5,2,6,3,7
 *     inside every 8 and its sums over every 128 k, the per-token form of what mq_w4a16_tc_prep writes with
 *     shuffle = xp_format (1: bf16 as it is; 2: fp16 scaled by the row's power of two, H <= 3968); bf16 x
 *     only, H % 128 == 0, H <= 4096.
 * Limits: T <= 64, E <= 256, K <= 32, T*K <= 2048 (MQ_ERR_UNSUPPORTED_SHAPE otherwise).
 */
size_t mq_route_small_workspace_bytes(int64_t T, int64_t E);
int mq_route_small(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                   int64_t T, int64_t H, int64_t E, int64_t K, int renormalize,
                   void* workspace, size_t workspace_bytes, int64_t* ids64, int32_t* ids32,
                   float* weights, int32_t* perm, int32_t* inv, int64_t* offsets64, int32_t* offsets32,
                   void* xp, float* xs, int xp_format, void* stream);

/* ------------------------------------------------------------------------------------------
 * Permute plan.  Replaces the index work of moe_permute / moe_unpermute
 * (mini_qwen/kernels/moe_permute.py:22-27, moe_unpermute.py:23-25): a stable counting sort of
 * the S = T*K flat slots by expert id.
 *   ids: [T,K] int64 (ids_are_64 != 0) or int32, every id in [0, E);
 *   perm  int32 [S]: perm[p] = flat slot t*K+k stored at sorted position p;
 *   inv   int32 [S]: inv[t*K+k] = p;
 *   offsets64 int64 [E+1] and/or offsets32 int32 [E+1] (either may be NULL): exclusive
 *   prefix sum of per-expert slot counts;
 *   workspace: mq_permute_workspace_bytes(S, E) bytes.
 * Limits: E <= 1024, S < 2^31.
 */
size_t mq_permute_workspace_bytes(int64_t S, int64_t E);
int mq_permute_plan(const void* ids, int ids_are_64, int64_t T, int64_t K, int64_t E,
                    int32_t* perm, int32_t* inv, int64_t* offsets64, int32_t* offsets32,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Row gather of moe_permute (moe_permute.py:30-31): out[p,:] = x[perm[p] / K, :].
 * H * sizeof(dtype) must be a multiple of 16 and the pointers 16-byte aligned. */
int mq_gather_rows(const void* x, int dtype, const int32_t* perm, int64_t S, int64_t K, int64_t H,
                   void* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Unpermute + weighted combine.  Replaces moe_unpermute (mini_qwen/kernels/moe_unpermute.py:
 * 20-31): out[t,:] = cast(sum_k weights[t,k] * float(rows[inv[t*K+k],:])), products and the
 * sum in fp32, k ascending.  rows [S,H] and out [T,H] have type `dtype`.
 */
int mq_unpermute_combine(const void* rows, int dtype, const float* weights, const int32_t* inv,
                         int64_t T, int64_t K, int64_t H, void* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * The decoder layer's glue either side of the block (mini_qwen/model/qwen3_moe.py:63-66:
 * h + mlp(post_attention_layernorm(h))).
 * mq_rms_norm replaces RMSNorm.forward (mini_qwen/model/layers/rms_norm.py:11-18) on [T,H] rows:
 *   out = weight * cast(float(x) * 1/sqrt(mean(float(x)^2) + eps)), the mean, the root and the
 *   reciprocal correctly rounded in fp32, the cast to `dtype` before the product with weight [H].
 *   Row sums run in a different order from the reference's CPU sum, so values can differ from it by
 *   one unit in the last place of `dtype`.
 * mq_unpermute_combine_residual is mq_unpermute_combine followed by the layer's residual add in the
 *   same kernel: out[t,:] = cast(float(residual[t,:]) + float(cast(sum_k ...))), the block output
 *   rounded to `dtype` before the add as the reference's two separate tensors are.  residual [T,H]
 *   of `dtype`, 16-byte aligned; NULL gives mq_unpermute_combine.  out may alias residual.
 */
int mq_rms_norm(const void* x, int dtype, const void* weight, float eps, int64_t T, int64_t H,
                void* out, void* stream);
int mq_unpermute_combine_residual(const void* rows, int dtype, const float* weights, const int32_t* inv,
                                  const void* residual, int64_t T, int64_t K, int64_t H, void* out,
                                  void* stream);

/* ------------------------------------------------------------------------------------------
 * Grouped GEMM, one projection.  Replaces moe_grouped_gemm / _moe_grouped_gemm_oracle
 * (mini_qwen/kernels/moe_grouped_gemm.py:17-37,115-156): for every expert e,
 * out[off[e]:off[e+1], :] = a[off[e]:off[e+1], :] . w[e]^T with fp32 accumulation.
 *   a [S,Kd], w [E,N,Kd], out [S,N], all of type `dtype`; offsets int32 [E+1].
 * Rows of `out` that belong to no expert are not written.
 * weight_period: group e uses weight matrix e % weight_period (w then holds weight_period matrices).
 * Plain use passes weight_period = E.  Expert parallelism passes the local expert count: the rows a
 * rank receives are grouped by (source rank, local expert), i.e. G * E_local groups over E_local
 * weight matrices.  The same argument has the same meaning in the calls below.
 * bf16 with Kd % 64 == 0 and N % 128 == 0 runs on the tcgen05/TMEM kernel, everything else on
 * a generic tiled kernel (Kd % 8 == 0 for 16-bit types, % 4 for fp32).
 */
int mq_grouped_gemm(const void* a, const void* w, const int32_t* offsets,
                    int64_t S, int64_t E, int64_t weight_period, int64_t N, int64_t Kd, int dtype,
                    void* out, int32_t* d_status, void* stream);

/* mq_grouped_gemm with one destination per output ROW instead of one [S,N] tensor: row r is written
 * to row (row_dst[r] & 0x3FFFFFF) of the [*, N] buffer at dst_bases[row_dst[r] >> 26].  The buffers
 * may lie in another GPU's memory (peer-mapped): expert parallelism uses this to send every expert
 * output row back to the rank and position it came from out of the GEMM's own epilogue, so the
 * transfer overlaps the remaining tiles.  No counterpart in the reference (it is single-GPU).
 * row_dst int32 [S] (read for rows inside the groups only); dst_bases: device array of buffer
 * addresses, each 16-byte aligned.  bf16, Kd % 64 == 0, N % 128 == 0 only
 * (MQ_ERR_UNSUPPORTED_SHAPE otherwise). */
int mq_grouped_gemm_scatter(const void* a, const void* w, const int32_t* offsets,
                            const int32_t* row_dst, const uint64_t* dst_bases, int64_t S, int64_t E,
                            int64_t weight_period, int64_t N, int64_t Kd, int dtype, int32_t* d_status,
                            void* stream);

/* Fused gate/up projection with SwiGLU. Replaces _ExpertMLP's first half
 * (mini_qwen/model/layers/moe.py:24-25) for all experts at once:
 *   h[s,:] = round(round(silu(round(a[s,:] . wg[e]^T))) * round(a[s,:] . wu[e]^T)),
 * every round() to `dtype`, as the per-expert nn.Linear path rounds.
 *   a [S,H], w_gate_up [E, 2*I, H] (gate rows first, then up rows), h [S,I].
 */
int mq_grouped_swiglu(const void* a, const void* w_gate_up, const int32_t* offsets,
                      int64_t S, int64_t E, int64_t weight_period, int64_t I, int64_t H, int dtype,
                      void* h, int32_t* d_status, void* stream);

/* The same with the permute gather fused in (moe_permute.py:30-31 + layers/moe.py:24-25): `x` is
 * the UNPERMUTED [T,H] activations and row p of the expert-sorted order is x[perm[p] / top_k]; the
 * rows are gathered inside the kernel, so the [T*top_k, H] copy is never written.  The slot count is
 * offsets[E] and need not be T*top_k: with top_k = 1, perm is a table of row numbers into x (the
 * expert-parallel receive buffer and its slot table).  Every perm[p]/top_k read must be < T.
 * bf16 only, H % 64 == 0, I % 128 == 0 (returns MQ_ERR_UNSUPPORTED_SHAPE otherwise: gather with
 * mq_gather_rows and call mq_grouped_swiglu). */
int mq_grouped_swiglu_gather(const void* x, const int32_t* perm, const void* w_gate_up,
                             const int32_t* offsets, int64_t T, int64_t top_k, int64_t E,
                             int64_t weight_period, int64_t I, int64_t H, int dtype,
                             void* h, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Load-time stacking of per-expert tensors.  The reference's loaders leave one module per expert and
 * projection (mini_qwen/model/loader.py:63-75 for dense checkpoints, :245-250 for GPTQ ones: 18 624
 * tensors), and its block walks them in a Python loop; the grouped kernels index expert-major stacks.
 * mq_stack_tensors builds one on the device for a host that has no tensor library:
 *   out = concatenation of the n tensors of bytes_each bytes whose device addresses are in the DEVICE
 *   array d_src_ptrs.  Dense experts: one call for the down weights [H,I] (n = E) and one for the gate
 *   and up weights with the addresses in the order gate[0], up[0], gate[1], up[1], ... (n = 2E), which
 *   gives w_gate_up [E, 2I, H]; W4A16 experts: one call per projection and buffer (qweight, scales,
 *   qzeros).  sources_aligned16 != 0 promises that every source address is 16-byte aligned (16-byte
 *   copies are then used when bytes_each % 16 == 0); n <= 65535.
 */
int mq_stack_tensors(const uint64_t* d_src_ptrs, int64_t n, int64_t bytes_each, int sources_aligned16,
                     void* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * W4A16 linear.  Replaces w4a16_gemm (mini_qwen/kernels/w4a16_gemm.py:8-15,194-247) and,
 * with E > 1, the per-expert calls LinearW4A16.forward makes from the expert loop
 * (mini_qwen/model/layers/linear_w4a16.py:31-36):
 *   out[r, n] = bf16( sum_k x[r,k] * (q[e][k,n] - z[e][k/g, n]) * s[e][k/g, n] )
 * for rows r in [off[e], off[e+1]).
 *   x bf16 [S,Kd]; qweight int32 [E, Kd/8, N] (nibble i of word [j,n] = q[8j+i, n]);
 *   scales bf16 [E, Kd/g, N]; qzeros int32 [E, Kd/g, N/8] (nibble i of word [G,m] = z[G, 8m+i]);
 *   offsets int32 [E+1] (for a single linear: E = 1, offsets = {0, M}); out bf16 [S,N].
 * Limits: g % 32 == 0, Kd % g == 0, N % 8 == 0.
 */
int mq_w4a16_grouped_gemm(const void* x, const int32_t* qweight, const void* scales,
                          const int32_t* qzeros, const int32_t* offsets,
                          int64_t S, int64_t E, int64_t weight_period, int64_t N, int64_t Kd, int64_t group_size,
                          void* out, void* stream);

/* Fused W4A16 gate/up projection with SwiGLU (bf16 rounding after gate, silu, up and the
 * product, as LinearW4A16 returns bf16).  Both projections share shapes: Kd = H, N = I. */
int mq_w4a16_grouped_swiglu(const void* x,
                            const int32_t* qweight_gate, const void* scales_gate, const int32_t* qzeros_gate,
                            const int32_t* qweight_up, const void* scales_up, const int32_t* qzeros_up,
                            const int32_t* offsets,
                            int64_t S, int64_t E, int64_t weight_period, int64_t I, int64_t H, int64_t group_size,
                            void* h, void* stream);

/* The same two operations with PREPARED activations, the form the block's decode path uses (same results as
 * the two calls above up to the order of the fp32 sums):
 *   xp [S,Kd] (16-bit): the expert-sorted rows.  x_format 0: bf16, natural k order.  1: bf16 with the k order
 *     0,4,1,5,2,6,3,7 inside every 8 (what mq_w4a16_tc_prep writes with shuffle = 1, and what
 *     mq_w4a16_stream_swiglu writes with shuffle_out != 0), which saves the kernel four byte permutes per
 *     32 k.  2: that order in fp16, every row scaled by a power of two whose inverse sits in xs[row][31]
 *     (mq_w4a16_tc_prep with shuffle = 2; needs xs, Kd <= 3968): fp16 nibbles unpack with five instead of
 *     seven integer instructions per weight word, and the scaling is exact, so the results equal format 1's
 *     except where an element more than 2^28 times smaller than its row's largest loses low bits;
 *   xs fp32 [S,32] or NULL: the rows' sums over every quantisation group (mq_w4a16_tc_prep); given, the
 *     kernel skips the extra MMA pair per 32 k that otherwise forms them; requires x_format != 0;
 *   shuffle_out != 0: h is written with its columns in the shuffled order, ready to be the xp of the down
 *     projection (pass x_format = 1 there);
 *   perm (mq_w4a16_stream_swiglu, optional): xp and xs then hold one row per TOKEN and row p of the expert-sorted
 *     order is row perm[p] / top_k of them, gathered inside the kernel (what mq_route_small prepares).
 * group_size == 128, N % 32 == 0, at most 384 row groups (MQ_ERR_UNSUPPORTED_SHAPE otherwise).  d_status
 * (optional) receives MQ_DEV_WAIT_EXPIRED if a bounded wait on a bulk copy ran out. */
int mq_w4a16_stream_swiglu(const void* xp, const float* xs, int x_format, const int32_t* perm, int64_t top_k,
                           const int32_t* qweight_gate, const void* scales_gate, const int32_t* qzeros_gate,
                           const int32_t* qweight_up, const void* scales_up, const int32_t* qzeros_up,
                           const int32_t* offsets, int64_t S, int64_t E, int64_t weight_period, int64_t I,
                           int64_t H, int64_t group_size, int shuffle_out, void* h, int32_t* d_status,
                           void* stream);
int mq_w4a16_stream_gemm(const void* xp, const float* xs, int x_format, const int32_t* qweight,
                         const void* scales, const int32_t* qzeros, const int32_t* offsets, int64_t S,
                         int64_t E, int64_t weight_period, int64_t N, int64_t Kd, int64_t group_size,
                         void* out, int32_t* d_status, void* stream);

/* The same two W4A16 operations on the tcgen05 tensor cores, for decode-size groups (any group size
 * is correct; it is tuned for groups of at most 32 rows).  The packed weights stream in by TMA in
 * the checkpoint layout, are turned into bf16 in registers and written to tensor memory, from where
 * the MMA reads them; the activations must be PREPARED first:
 * mq_w4a16_tc_prep: x bf16 [T,Kd] -> xp [S,Kd] (16-bit), row r = x[perm[r]/top_k] (perm NULL: x[r],
 *   S = T) with the k order 0,4,1,5,2,6,3,7 inside every 8 when `shuffle` != 0, and
 *   xs fp32 [S,32]: xs[r][g] = sum of the row over quantisation group g (Kd <= 4096).  xp may be
 *   NULL (sums only: the output of mq_w4a16_tc_swiglu is already in the shuffled order).
 *   shuffle = 2 (the stream kernels' fp16 format, Kd <= 3968): the shuffled row is multiplied by the power
 *   of two 2^e that puts its largest magnitude into [2^14, 2^15) and stored as fp16; xs holds the sums of
 *   the stored values and xs[r][31] = 2^-e.
 * mq_w4a16_tc_swiglu: h_shuffled[r,:] = the fused gate/up + SwiGLU row of mq_w4a16_grouped_swiglu with
 *   its columns in the shuffled k order, ready to be the xp of the down projection.
 * mq_w4a16_tc_gemm: out[r,:] as mq_w4a16_grouped_gemm, natural column order.
 * group_size == 128, Kd % 128 == 0, N % 128 == 0 (MQ_ERR_UNSUPPORTED_SHAPE otherwise). */
int mq_w4a16_tc_prep(const void* x, const int32_t* perm, int64_t top_k, int64_t S, int64_t Kd,
                     int shuffle, void* xp, float* xs, void* stream);
int mq_w4a16_tc_gemm(const void* xp, const float* xs, const int32_t* qweight, const void* scales,
                     const int32_t* qzeros, const int32_t* offsets, int64_t S, int64_t E,
                     int64_t weight_period, int64_t N, int64_t Kd, int64_t group_size, void* out,
                     int32_t* d_status, void* stream);
int mq_w4a16_tc_swiglu(const void* xp, const float* xs,
                       const int32_t* qweight_gate, const void* scales_gate, const int32_t* qzeros_gate,
                       const int32_t* qweight_up, const void* scales_up, const int32_t* qzeros_up,
                       const int32_t* offsets, int64_t S, int64_t E, int64_t weight_period, int64_t I,
                       int64_t H, int64_t group_size, void* h_shuffled, int32_t* d_status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Expert parallelism over peer memory (no counterpart in the reference, which is single-GPU).
 * G ranks, rank r owns experts [r*E/G, (r+1)*E/G).  Every rank provides a receive buffer and an
 * expert-output buffer of cap_rows rows that its peers can address (peer_*_ptrs: device array of
 * G base addresses, entry r being the local buffer).  The slots a rank receives are ordered by
 * local expert and, inside an expert, by source rank (each source's slots in its own sorted order):
 * E/G ordinary groups for the grouped kernels.  The data kernels wait on nobody; the caller orders the
 * ranks between them with mq_ep_barrier (or any stream-ordered collective).  mq_ep_barrier and
 * mq_ep_exchange_plan DO wait on the other ranks, on the device, with a bounded poll: the ranks of a
 * group must enter a layer call within the poll budget of one another (max_polls polls; 0 = the
 * default of 2^22, one to two seconds), and a caller must read d_status before trusting an output.
 *
 * mq_ep_share_counts: writes this rank's per-expert counts (from its offsets [E+1]) into row `rank`
 *   of every peer's counts table int32 [G,E] (peer_counts_ptrs: G base addresses).
 * mq_ep_barrier: stream-ordered barrier across the G ranks through a signal array int32 [G] on every
 *   rank (peer_signal_ptrs) and a local epoch counter.  The wait is bounded (max_polls polls of every
 *   peer's slot, 0 = default, at most 2^22); on expiry MQ_DEV_WAIT_EXPIRED is set in d_status and the
 *   kernel returns; the stream and the context stay usable.
 * mq_ep_plan: all_counts int32 [G,E] (per-expert slot counts of every rank) ->
 *   send_base int32 [E]: slot in the owner's receive order where this rank's slots of expert e start;
 *   seg_offsets int32 [E/G+1]: prefix sums of this rank's receive groups (one per local expert).
 * mq_ep_dispatch: fused permute + dispatch, one row per slot.  Row p of the expert-sorted order
 *   (token perm[p]/K of x) is written into the owner's receive buffer at its slot;
 *   slot_dst[p] = owner * cap_rows + slot (or -1 and status bit 2 when it would not fit in cap_rows).
 *   peer_home_ptrs (optional): the owners' home tables int32 [cap_rows]; entry [slot] becomes
 *   rank << 26 | p, the row_dst code that makes mq_grouped_gemm_scatter (dst_bases = the ranks'
 *   output buffers) deliver the slot's output row to row p of this rank's buffer, after which the
 *   source finishes with a local mq_unpermute_combine instead of mq_ep_combine.
 * mq_ep_combine: fused combine + unpermute.  out[t,:] = cast(sum_k weights[t,k] *
 *   float(y_owner[slot_dst[inv[t*K+k]]])), fp32 multiply then add, k ascending.  residual
 *   (optional, [T,H] of `dtype`): the layer's residual add in the same kernel, as in
 *   mq_unpermute_combine_residual.
 */
int mq_ep_share_counts(const int32_t* offsets, int64_t E, int64_t G, int64_t rank,
                       const uint64_t* peer_counts_ptrs, void* stream);
int mq_ep_barrier(const uint64_t* peer_signal_ptrs, int32_t* epoch_counter, int64_t G, int64_t rank,
                  int64_t max_polls, int32_t* d_status, void* stream);
int mq_ep_plan(const int32_t* all_counts, int64_t G, int64_t rank, int64_t E,
               int32_t* send_base, int32_t* seg_offsets, void* stream);
/* mq_ep_share_counts, mq_ep_barrier and mq_ep_plan in one launch (the plan is formed from this rank's
 * own counts table, peer_counts_ptrs[rank], once every rank has written its row).  When the wait runs
 * out, the plan written is one that moves nothing: send_base[e] = 0x3FFFFFFF for every expert (the
 * dispatch kernels drop rows outside [0, cap_rows) and set MQ_DEV_EP_OVERFLOW) and seg_offsets all 0
 * (the grouped kernels get no rows), so nothing is computed from an incomplete counts table. */
int mq_ep_exchange_plan(const int32_t* offsets, int64_t E, int64_t G, int64_t rank,
                        const uint64_t* peer_counts_ptrs, const uint64_t* peer_signal_ptrs,
                        int32_t* epoch_counter, int32_t* send_base, int32_t* seg_offsets,
                        int64_t max_polls, int32_t* d_status, void* stream);
int mq_ep_dispatch(const void* x, int dtype, const int32_t* perm, const int32_t* offsets,
                   const int32_t* send_base, int64_t S, int64_t K, int64_t H, int64_t E, int64_t G,
                   int64_t rank, const uint64_t* peer_recv_ptrs, const uint64_t* peer_home_ptrs,
                   int64_t cap_rows, int32_t* slot_dst, int32_t* d_status, void* stream);
/* Dispatch that sends a token row once per destination RANK instead of once per slot (a token with
 * several experts on one GPU crosses NVLink once).  G <= 8.
 * mq_ep_unique_rows: topk_ids int32 [T,K] -> uniq int32 [G,T] (rank-major): uniq[d,t] = index of token t
 *   among this rank's tokens that have an expert on rank d, in token order, or -1 when it has none there.
 * mq_ep_dispatch_unique: row t goes to row rank*src_stride + uniq[d,t] of every rank d that needs it
 *   (T <= src_stride, G*src_stride <= cap_rows), and every slot's row number goes to its slot in the
 *   owner's slot table peer_ridx_ptrs[d] (int32 [cap_rows]).  The owner runs
 *   mq_grouped_swiglu_gather with x = its receive buffer, perm = its slot table, top_k = 1.
 *   slot_dst and peer_home_ptrs as in mq_ep_dispatch. */
int mq_ep_unique_rows(const int32_t* topk_ids, int64_t T, int64_t K, int64_t E, int64_t G,
                      int32_t* uniq, void* stream);
int mq_ep_dispatch_unique(const void* x, int dtype, const int32_t* uniq, const int32_t* perm,
                          const int32_t* offsets, const int32_t* send_base, int64_t T, int64_t K,
                          int64_t H, int64_t E, int64_t G, int64_t rank, int64_t src_stride,
                          const uint64_t* peer_recv_ptrs, const uint64_t* peer_ridx_ptrs,
                          const uint64_t* peer_home_ptrs, int64_t cap_rows, int32_t* slot_dst,
                          int32_t* d_status, void* stream);
int mq_ep_combine(const uint64_t* peer_y_ptrs, int dtype, const float* weights, const int32_t* inv,
                  const int32_t* slot_dst, const void* residual, int64_t T, int64_t K, int64_t H,
                  int64_t cap_rows, void* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * Expert parallelism for decode batches by replication (no counterpart in the reference).  With a few
 * tokens per GPU the dispatch / return exchange above is bound by its rank barriers; here every rank
 * gathers ALL tokens of the step, routes them itself (identical ids, weights and plan on every rank), runs
 * only its own experts on the slots they own (the grouped calls take an offsets pointer that starts at the
 * rank's first expert) and sends every token's partial weighted sum to the rank that owns the token.  Two
 * rank barriers per layer call, inside these kernels.  All ranks must call with the same T.
 * mq_ep_gather_tokens: x [T,H] of this rank -> rows [rank*T, rank*T+T) of every peer's token buffer
 *   (peer_token_ptrs: G device addresses of [G*T,H] buffers of `dtype`), then the rank barrier.
 * mq_ep_send_partials: tokens = G*T; for every token t: the fp32 sum over the slots k with
 *   topk_ids[t,k] / experts_per_rank == rank of weights[t,k] * float(rows[inv[t*K+k]]), k ascending, stored
 *   into row (rank*T + t % T) of the fp32 [G*T,H] buffer of rank t / T (peer_partial_ptrs); then the rank
 *   barrier.  done_counter: one int32, zero before the first call (the kernel leaves it at zero).
 * mq_ep_sum_partials: out[t,:] = cast(sum over r ascending of partials[r*T + t,:]) for this rank's T tokens;
 *   residual (optional) as in mq_unpermute_combine_residual.
 * The barrier is mq_ep_barrier's (same signal arrays and epoch counter, same max_polls, same status bit).
 * Outputs equal the single-GPU ones up to the order of the fp32 sums.
 */
int mq_ep_gather_tokens(const void* x, int dtype, int64_t T, int64_t H, int64_t G, int64_t rank,
                        const uint64_t* peer_token_ptrs, const uint64_t* peer_signal_ptrs,
                        int32_t* epoch_counter, int64_t max_polls, int32_t* d_status, void* stream);
int mq_ep_send_partials(const void* rows, int dtype, const float* weights, const int32_t* topk_ids,
                        const int32_t* inv, int64_t tokens, int64_t K, int64_t H, int64_t T, int64_t G,
                        int64_t rank, int64_t experts_per_rank, const uint64_t* peer_partial_ptrs,
                        int32_t* done_counter, const uint64_t* peer_signal_ptrs, int32_t* epoch_counter,
                        int64_t max_polls, int32_t* d_status, void* stream);
int mq_ep_sum_partials(const float* partials, int dtype, const void* residual, int64_t T, int64_t H,
                       int64_t G, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MQMOE_H */
