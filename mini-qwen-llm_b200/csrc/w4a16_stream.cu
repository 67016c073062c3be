// W4A16 linear for decode-size groups as a persistent, TMA-staged stream over the packed weights.
// Format and arithmetic follow mini_qwen/kernels/w4a16_gemm.py:8-15 and tests/test_w4a16_gemm.py:19-44 of
// the reference: W[k,n] = (q[k,n] - z[k/g,n]) * s[k/g,n], group g = 128, out = bf16(x . W) with fp32 sums.
//
// The work is a stream: every packed weight byte is read from HBM once and the arithmetic per byte is
// small.  Two things bound it on this GPU: the memory system wants about 100 KB per SM on its way from HBM
// at all times to run at its streaming rate, and the integer pipe (half rate: 16 lanes per scheduler)
// saturates at about 80 logic/shift instructions per KB of weights, which is where turning nibbles into
// bf16 costs 56.  The kernel is organised around both.
//
//   * One CTA per SM, persistent, sixteen warps that all do arithmetic (four per scheduler, which leaves
//     each thread 128 registers).  There is no producer warp: the warp that is last to finish with a ring
//     stage (a shared counter tells it) issues the copy that refills it.
//   * The weights are fetched with tensor-map bulk copies straight from the checkpoint layout
//     qweight [E, K/8, N]: a 4-D view (32 columns, K/8 word rows, N/32 column panels, expert) lets ONE copy
//     bring a box of (32 columns x RS word rows x P panels) into shared memory as P dense panels of 128-byte
//     rows, the layout the warps read without bank conflicts.  Stages of 64-96 KB rotate through a 192 KB
//     ring; word rows and panels outside the tensor read as zero.
//   * An item = (expert, block of 8 rows, P column panels).  The warps form a KW x CW grid: warp (kw, cw)
//     owns panel cw and, in every stage, gpw consecutive quantisation groups of the stage's K range.  KW, CW
//     and gpw are chosen per launch so that there are several items per SM whatever the number of experts
//     hit (batch 1: 16 x 1, one stage holds all of K; batch 64: 4 x 4).  The items of a CTA are located
//     once, by 32 threads in parallel, into a window of descriptors in shared memory.
//   * A lane reads one 128-bit vector = 4 adjacent columns x 8 consecutive k.  Nibbles become bf16 with one
//     logic op per pair: (w >> 4p) & 0x000F000F | 0x43004300 is the bf16 pair {128+q[p], 128+q[p+4]}; one
//     packed fma on the otherwise idle FMA pipe re-centres it to {q[p]-8, q[p+4]-8}.  The zero point is not
//     subtracted per weight: with xs = sum_k x[k] over the group,
//     sum_k x[k]*(q[k]-z) = sum_k x[k]*(q[k]-8) - (z-8)*xs, evaluated once per group and column in fp32
//     and scaled by s in fp32, so the dequantised weight is never rounded to bf16.
//   * The biased integers are the A operand (16 columns x 16 k) of mma.sync.m16n8k16 with the 8 rows of
//     activations as the B operand; the k order inside a word is permuted identically on both operands.
//     SwiGLU: a warp streams the gate and the up panel of the same 32 columns against the same activations.
//   * Activations come from global memory (L2) into registers half a group ahead, also across items.  They
//     may be PREPARED (mq_w4a16_tc_prep): rows already in the permuted k order (no byte permutes in the
//     loop) and their group sums given (otherwise one more MMA pair per 32 k against a tile of ones forms
//     them).  With a permutation table the rows of an expert are gathered from the unpermuted activations.
//   * The K split meets in shared memory: every warp leaves its partial sums there and signals an mbarrier;
//     the sums are added up (fixed order) and stored one stage LATER, in the middle of the next item, when
//     the other warps' partials are certain to be there: no warp ever stands at a barrier for them.
//
// Every mbarrier wait is bounded; on expiry MQ_DEV_WAIT_EXPIRED is set and all warps leave their loops.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace mq {
namespace {

constexpr int WS_CONSUMERS = 16;
constexpr int WS_THREADS = WS_CONSUMERS * 32;
constexpr int WS_RING_BYTES = 192 * 1024;
constexpr int WS_MAX_STAGES = 3;
constexpr int WS_RED_BYTES = WS_CONSUMERS * 16 * 32 * 4;            // partial sums of the K split: 32 KB
constexpr int WS_MAX_GROUPS = 384;                                  // row groups (experts) the item table can index
constexpr int WS_TABLE_BYTES = (WS_MAX_GROUPS + 1) * 4;
constexpr int WS_LIST = 16;                                         // window of item descriptors (48 bytes each)
constexpr int WS_SMALL_BYTES = 256 /*barriers*/ + WS_LIST * 48 + WS_TABLE_BYTES;
constexpr uint32_t WS_SPIN_LIMIT = 1u << 24;
constexpr uint32_t BF16_ONES2 = 0x3F803F80u;

__device__ __forceinline__ uint32_t ws_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ws_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ws_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ws_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Has the phase of that parity completed?  Never suspends the thread (try_wait may, for a while).
__device__ __forceinline__ bool ws_mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ws_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the wait ran out or another role already gave up.
__device__ __forceinline__ bool ws_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* d_status) {
  for (uint32_t spin = 0; spin < WS_SPIN_LIMIT; ++spin) {
    if (ws_mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (d_status != nullptr) atomicOr(d_status, (int)MQ_DEV_WAIT_EXPIRED);
  return false;
}
__device__ __forceinline__ void ws_tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                               int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// Barrier among the KW warps that share column panel cw (ids 1..CW; id 0 is __syncthreads).
__device__ __forceinline__ void ws_panel_sync(int cw, int KW) {
  asm volatile("bar.sync %0, %1;" ::"r"(cw + 1), "r"(KW * 32) : "memory");
}
__device__ __forceinline__ void ws_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint32_t ws_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// pair p of word w -> bf16x2 {q[p] - 8, q[p+4] - 8}.  The logic op makes {128 + q[p], 128 + q[p+4]} (the
// nibble in the low mantissa bits of 128.0); the packed fused multiply-add that takes the 136 off again
// runs on the FMA pipe, which this kernel leaves idle, and keeps the sums the tensor core accumulates as
// small as the result itself: with the bias left in, a group's sum carries 128 * sum(x) that has to cancel
// later, which costs four bits of the fp32 accumulator and flips ten times more bf16 roundings downstream.
__device__ __forceinline__ uint32_t ws_centered_pair(uint32_t w, int p) {
  uint32_t v, c;
  const uint32_t sh = w >> (4 * p);
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(sh), "r"(0x000F000Fu), "r"(0x43004300u));
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(c) : "r"(v), "r"(0x3F803F80u), "r"(0xC308C308u));
  return c;
}
// The four pairs of a word at once, pair p = {q[p] - 8, q[p+4] - 8}.  bf16: one shift and one logic op per pair
// (seven integer instructions a word).  fp16 has ten mantissa bits, so a nibble can also be picked up where it
// sits four bits higher: (w & 0x00F000F0) | 0x6400 is the pair {1024 + 16 q[1], 1024 + 16 q[5]}, and one packed
// FMA (x 1/16, - 72) re-centres it exactly; a word then costs one shift and four logic ops.
template <bool F16>
__device__ __forceinline__ void ws_dequant_word(uint32_t w, uint32_t (&d)[4]) {
  if (!F16) {
#pragma unroll
    for (int p = 0; p < 4; ++p) d[p] = ws_centered_pair(w, p);
  } else {
    const uint32_t w8 = w >> 8;
    uint32_t t0, t1, t2, t3;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t0) : "r"(w), "r"(0x000F000Fu), "r"(0x64006400u));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t1) : "r"(w), "r"(0x00F000F0u), "r"(0x64006400u));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t2) : "r"(w8), "r"(0x000F000Fu), "r"(0x64006400u));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t3) : "r"(w8), "r"(0x00F000F0u), "r"(0x64006400u));
    // (1024 + q) - 1032 and (1024 + 16 q) / 16 - 72, both exact in fp16
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d[0]) : "r"(t0), "r"(0x3C003C00u), "r"(0xE408E408u));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d[1]) : "r"(t1), "r"(0x2C002C00u), "r"(0xD480D480u));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d[2]) : "r"(t2), "r"(0x3C003C00u), "r"(0xE408E408u));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d[3]) : "r"(t3), "r"(0x2C002C00u), "r"(0xD480D480u));
  }
}
template <bool F16>
__device__ __forceinline__ void ws_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  // not volatile: the accumulator operands carry every dependence, and the scheduler may then interleave
  // the independent accumulator chains of a step
  if (F16) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
// Activation pieces: read-only path, allocating in L1 (the warps that share a K slice read the same pieces within a
// few hundred cycles of one another; with L1::no_allocate every one of them went to L2: 69.6 against 67.7 us on
// the batch-64 gate/up launch).
__device__ __forceinline__ uint4 ws_ldg128(const void* p) {
  uint4 v;
  asm("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

struct WsProj {
  const __nv_bfloat16* sc;   // [period, G, N]
  const int32_t* qz;         // [period, G, N/8]
};

struct WsParams {
  const __nv_bfloat16* x;    // activations [*, Kd]
  const float* xs;           // XSUM: xs[row * 32 + g] = sum of the row over quantisation group g
  const int32_t* perm;       // optional: row p of the sorted order is x[perm[p] / top_k]
  int top_k;
  int shuffle_out;           // write the output columns in the order 0,4,1,5,2,6,3,7 inside every 8
  const int32_t* offsets;    // [E + 1]
  int E, period;
  int N, Kd, G;              // output features, input features, quantisation groups (Kd / 128)
  int KW, CW, gpw;           // consumer grid and groups per warp and stage
  int RS;                    // word rows per stage = 16 * KW * gpw
  int spi;                   // stages per item
  int ipe;                   // column items per expert
  int nst;                   // ring depth
  uint32_t stage_bytes;
  WsProj p0, p1;
  __nv_bfloat16* out;        // [*, N]
  int32_t* d_status;
};

// One weight stream of a lane: 4 columns x (rows 2kq, 2kq+1) in two MMA fragments.
struct WsStream {
  float master[2][4];
  float grp[2][4];
};

// scale / zero-point words of one group for a lane's 4 columns
struct WsMeta {
  uint2 s;
  uint32_t z;
};
__device__ __forceinline__ WsMeta ws_meta_fetch(const WsProj& p, size_t group_row, int N, int col) {
  WsMeta m;
  m.s = __ldg(reinterpret_cast<const uint2*>(p.sc + group_row * N + col));
  m.z = (uint32_t)__ldg(p.qz + group_row * (N >> 3) + (col >> 3)) >> ((col & 7) * 4);
  return m;
}

// End of a group: master += s * (sum_k x*(q-8) - (z-8) * sum_k x), then restart the group sums.
// xs[0], xs[1]: the group sums of rows 2kq and 2kq+1.
__device__ __forceinline__ void ws_flush(WsStream& a, const WsMeta& m, float xs0, float xs1) {
  const float sc[4] = {__uint_as_float(m.s.x << 16), __uint_as_float(m.s.x & 0xffff0000u),
                       __uint_as_float(m.s.y << 16), __uint_as_float(m.s.y & 0xffff0000u)};
  // 8 - z as fp32 without a conversion: the nibble lands in the top mantissa bits of 0x43000000 = 128.0f
  // (one shift and one logic op per column), and 136 - (128 + z) is exact
  float nz[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v;
    const uint32_t sh = m.z << (16 - 4 * c);
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(sh), "r"(0x000F0000u), "r"(0x43000000u));
    nz[c] = 136.0f - __uint_as_float(v);
  }
#pragma unroll
  for (int mm = 0; mm < 2; ++mm)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = 2 * mm + (i >> 1);
      const float t = fmaf(nz[col], (i & 1) ? xs1 : xs0, a.grp[mm][i]);
      a.master[mm][i] = fmaf(sc[col], t, a.master[mm][i]);
      a.grp[mm][i] = 0.0f;
    }
}

// SwiGLU with the rounding points of the op-by-op bf16 path (g, silu(g), u and the product are each rounded to
// bf16); exp and the reciprocal use the SFU approximations, whose error (2^-21) is far below the bf16
// rounding that follows.
__device__ __forceinline__ float ws_swiglu(float g, float u) {
  const float gb = __bfloat162float(__float2bfloat16_rn(g));
  const float sb = __bfloat162float(__float2bfloat16_rn(__fdividef(gb, 1.0f + __expf(-gb))));
  const float ub = __bfloat162float(__float2bfloat16_rn(u));
  return sb * ub;
}

template <bool F16>
__device__ __forceinline__ void ws_step(WsStream& a, const uint4& wv, const uint32_t (&b)[4]) {
  const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
  uint32_t d[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) ws_dequant_word<F16>(w[c], d[c]);
  // the two accumulators alternate, so that an MMA never follows the one it depends on
#pragma unroll
  for (int m = 0; m < 2; ++m)
    ws_mma<F16>(a.grp[m], d[2 * m][0], d[2 * m + 1][0], d[2 * m][1], d[2 * m + 1][1], b[0], b[1]);
#pragma unroll
  for (int m = 0; m < 2; ++m)
    ws_mma<F16>(a.grp[m], d[2 * m][2], d[2 * m + 1][2], d[2 * m][3], d[2 * m + 1][3], b[2], b[3]);
}

// An item of work.
struct WsItem {
  int expert;     // group of rows (weights: expert % period)
  int row0;       // first row of the 8-row block
  int rows;       // 1..8
  int ci;         // column item: panels [ci*CW, (ci+1)*CW)
};
// An item in the CTA's window: the descriptor and the rows of x its eight block rows come from (a row past the
// expert's last repeats the first: computed, not stored), looked up once per item instead of once per warp.
struct WsListed {
  WsItem it;
  int src[8];
};

// Items are numbered in (expert, row block, column item) order.  first_item[e] is the number of the first
// item of expert e (a table in shared memory, built once per CTA), so an item is found by a binary search.
struct WsItems {
  const int32_t* off;
  const int* first_item;   // [E + 1]
  int E, ipe;
  __device__ bool locate(int t, WsItem& it) const {
    if (t >= first_item[E]) return false;
    int lo = 0, hi = E;                       // invariant: first_item[lo] <= t < first_item[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (first_item[mid] <= t) lo = mid; else hi = mid;
    }
    const int row_lo = off[lo], n = off[lo + 1] - row_lo;
    const int local = t - first_item[lo];
    const int rb = local / ipe;
    it.expert = lo;
    it.row0 = row_lo + 8 * rb;
    it.rows = min(8, n - 8 * rb);
    it.ci = local - rb * ipe;
    return true;
  }
};

// first_item[0..E] = exclusive prefix sums of ceil(rows_e / 8) * ipe; all threads of the CTA take part.
__device__ void ws_build_item_table(const int32_t* __restrict__ offsets, int E, int ipe, int* first_item) {
  __shared__ int s_warp_tot[WS_CONSUMERS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (E + WS_THREADS - 1) / WS_THREADS;            // experts per thread (1 or 2)
  const int e_lo = min(tid * per, E), e_hi = min(e_lo + per, E);
  int sum = 0;
  for (int e = e_lo; e < e_hi; ++e) sum += ((offsets[e + 1] - offsets[e] + 7) >> 3) * ipe;
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) s_warp_tot[warp] = incl;
  __syncthreads();
  int base = incl - sum;
  for (int w = 0; w < warp; ++w) base += s_warp_tot[w];
  for (int e = e_lo; e < e_hi; ++e) {
    first_item[e] = base;
    base += ((offsets[e + 1] - offsets[e] + 7) >> 3) * ipe;
  }
  if (tid == WS_THREADS - 1) first_item[E] = base;
  __syncthreads();
}

// XSHUF: the activations already have the k order 0,4,1,5,2,6,3,7 inside every 8 (mq_w4a16_tc_prep, or the
//        shuffled output of the SwiGLU variant); otherwise the order is made with four byte permutes per step.
// XSUM:  the group sums come from P.xs; otherwise from one more MMA pair per step against a tile of ones.
// F16:   the prepared rows are fp16, each scaled by its own power of two whose inverse sits in slot 31 of the row's
//        sums (w4_prep.cuh); needs XSHUF and XSUM.
template <bool SWIGLU, bool XSHUF, bool XSUM, bool F16>
__global__ void __launch_bounds__(WS_THREADS, 1)
w4a16_stream_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                    const WsParams P) {
  constexpr int NS = SWIGLU ? 2 : 1;                   // weight streams per warp
  extern __shared__ __align__(16) uint8_t ws_smem_raw[];
  // Layout: barriers, item list and item table first; they fill most of the gap up to the next 1024-byte
  // boundary, where the ring starts (the copies land with the 128-byte swizzle, whose pattern repeats every
  // 1024 bytes); the partial sums follow the ring.
  const uint32_t raw = ws_smem_u32(ws_smem_raw);
  uint8_t* bar_mem = ws_smem_raw;
  const uint32_t bars = raw;
  const uint32_t ring = (raw + WS_SMALL_BYTES + 1023u) & ~1023u;
  uint8_t* ring_ptr = ws_smem_raw + (ring - raw);
  float* red = reinterpret_cast<float*>(ring_ptr + WS_RING_BYTES);
  // bar_mem: full[3] | abort flag | stage_done[3] ... +128: ready[8] | taken[8] ... +256: item list ... then the table
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto ready_bar = [&](int c) { return bars + 128u + 8u * c; };     // the KW partial sums of panel c are written
  auto taken_bar = [&](int c) { return bars + 192u + 8u * c; };     // ... and have been read again
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * WS_MAX_STAGES);
  int* stage_done = reinterpret_cast<int*>(bar_mem + 8 * WS_MAX_STAGES + 8);   // warps finished with a stage
  WsListed* list = reinterpret_cast<WsListed*>(bar_mem + 256);      // this CTA's items, a window of WS_LIST of them
  int* first_item = reinterpret_cast<int*>(bar_mem + 256 + WS_LIST * sizeof(WsListed));
  {
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if (ring - raw + WS_RING_BYTES + WS_RED_BYTES > dyn_bytes) {     // the launch did not leave room for the alignment
      if (threadIdx.x == 0 && P.d_status != nullptr) atomicOr(P.d_status, MQ_DEV_BAD_LAUNCH);
      return;
    }
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KW = P.KW, CW = P.CW, gpw = P.gpw, RS = P.RS, N = P.N, Kd = P.Kd, G = P.G;
  if (threadIdx.x == 0) {
    for (int s = 0; s < WS_MAX_STAGES; ++s) {
      ws_mbar_init(full_bar(s), 1);
      stage_done[s] = 0;
    }
    for (int c = 0; c < 8; ++c) {
      ws_mbar_init(ready_bar(c), KW);
      ws_mbar_init(taken_bar(c), KW);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();                   // everything above is this kernel's own; from here on it reads the predecessor's outputs
  pdl_release();
  ws_build_item_table(P.offsets, P.E, P.ipe, first_item);      // ends with a __syncthreads
  const WsItems items{P.offsets, first_item, P.E, P.ipe};
  // items of this CTA: numbers blockIdx.x + q * gridDim.x, q = 0 .. n_mine-1
  const int total_items = first_item[P.E];
  const int n_mine = total_items > (int)blockIdx.x ? (total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  // The descriptors of the CTA's items q in [8*floor(q/8), +16) sit in list[q % 16]: one shared-memory read per
  // item instead of a search plus dependent global loads by every warp.  A half is refilled when the walk
  // enters the other one.
  auto fill_list = [&](int q0) {                                 // descriptors q0 .. q0+7, eight threads each
    if (threadIdx.x < (WS_LIST / 2) * 8) {
      const int q = q0 + (threadIdx.x >> 3), r = threadIdx.x & 7;
      WsItem d;
      d.expert = 0; d.row0 = 0; d.rows = 0; d.ci = 0;
      if (q < n_mine) items.locate(blockIdx.x + q * gridDim.x, d);
      const int row = d.row0 + (r < d.rows ? r : 0);
      int src = row;
      if (P.perm != nullptr && d.rows > 0) src = P.perm[row] / P.top_k;
      WsListed& e = list[q % WS_LIST];
      if (r == 0) e.it = d;
      e.src[r] = src;
    }
  };
  fill_list(0);
  fill_list(WS_LIST / 2);
  __syncthreads();

  const uint32_t proj_bytes = (uint32_t)RS * (uint32_t)CW * 128u;       // one projection's box

  // Stage number n of this CTA (counted over its items) is stage n % spi of its item number n / spi and
  // lives in ring slot n % nst.  load_stage issues the copies of stage n, if the CTA has that many.
  auto load_stage = [&](int n) {
    const int q = n / P.spi, sj = n - q * P.spi;
    if (q >= n_mine) return;
    const WsItem fi = list[q % WS_LIST].it;
    const int slot = n % P.nst;
    const uint32_t dst = ring + (uint32_t)slot * P.stage_bytes;
    const int we = fi.expert % P.period;
    ws_mbar_expect_tx(full_bar(slot), P.stage_bytes);
    ws_tma_load_4d(dst, &map0, full_bar(slot), 0, sj * RS, fi.ci * CW, we);
    if (SWIGLU) ws_tma_load_4d(dst + proj_bytes, &map1, full_bar(slot), 0, sj * RS, fi.ci * CW, we);
  };
  if (threadIdx.x == 0)
    for (int n = 0; n < P.nst; ++n) load_stage(n);

  const int kw = warp / CW, cw = warp - kw * CW;
  const int g = lane >> 2, kq = lane & 3;
  const WsProj proj[2] = {P.p0, SWIGLU ? P.p1 : P.p0};
  int stage = 0, nstage = 0;                                  // ring slot and number of the stage being read
  uint32_t phase = 0;
  bool ok = true;
  const int g_first = kw * gpw;                               // this warp's first group of every item
  // row of x this lane multiplies in an item
  auto x_row_of = [&](const WsListed& w) { return P.x + (size_t)w.src[g] * Kd + 16 * kq; };

  // ---- finishing an item: the KW partial sums of every output meet in shared memory
  // (red[cw][stream][element][kw][lane]); each warp of the panel adds up a share of the outputs in a fixed
  // order and stores them.  The finish of item q is DEFERRED into the first stage of item q+1: by then the
  // other warps of the panel have long written their partial sums, so nobody stands at a barrier.
  // element idx = 4*m + i of a stream: column 2m + (i >> 1) of the lane's four, row 2kq + (i & 1)
  struct Pending { int row0, rows, col, q; };
  auto store_out = [&](const Pending& f, int idx, float v0, float v1) {
    const int r = 2 * kq + (idx & 1);
    int c = f.col + 2 * (idx >> 2) + ((idx & 3) >> 1);
    if (r < f.rows && c < N) {
      const float o = SWIGLU ? ws_swiglu(v0, v1) : v0;
      // shuffled order: element j of an 8-block goes to position 2*(j & 3) + (j >> 2)
      if (P.shuffle_out) c = (c & ~7) | (2 * (c & 3) + ((c >> 2) & 1));
      P.out[(size_t)(f.row0 + r) * N + c] = __float2bfloat16_rn(o);
    }
  };
  auto finish = [&](const Pending& f) {
    if (ok) ok = ws_mbar_wait(ready_bar(cw), (uint32_t)(f.q & 1), abort_flag, P.d_status);   // returns at once if complete
    if (ok) {
      for (int idx = kw; idx < 8; idx += KW) {
        const float* src = red + ((size_t)(cw * NS * 8 + idx) * KW) * 32 + lane;
        float v[NS];
#pragma unroll
        for (int q = 0; q < NS; ++q) {
          const float* sq = src + q * 8 * KW * 32;
          float sum = sq[0];
          for (int k = 1; k < KW; ++k) sum += sq[k * 32];
          v[q] = sum;
        }
        store_out(f, idx, v[0], v[NS - 1]);
      }
    }
    __syncwarp();
    if (lane == 0) ws_mbar_arrive(taken_bar(cw));
  };
  Pending pend;
  bool have_pend = false;

  // Activations travel half a group ahead of their use: xa holds steps 0-1 of the group being multiplied
  // (loaded during the previous group's second half, also across items), xb steps 2-3 (loaded during its
  // own first half).
  uint4 xa[2], xb[2];
  WsItem it;
  const __nv_bfloat16* xrow = nullptr;
  if (n_mine > 0) {
    it = list[0].it;
    xrow = x_row_of(list[0]);
    if (g_first < G) {
      xa[0] = ws_ldg128(xrow + g_first * 128);
      xa[1] = ws_ldg128(xrow + g_first * 128 + 8);
    }
  }
  for (int q = 0; q < n_mine; ++q) {
    if (q > 0 && (q & (WS_LIST / 2 - 1)) == 0) {                 // entering the other half of the window: refill this one's predecessor
      __syncthreads();
      fill_list(q + WS_LIST / 2);
      __syncthreads();
    }
    const bool have_next_item = q + 1 < n_mine;
    WsItem it_next = it;
    const __nv_bfloat16* xrow_next = xrow;
    if (have_next_item) {
      const WsListed& ln = list[(q + 1) % WS_LIST];
      it_next = ln.it;
      xrow_next = x_row_of(ln);
    }
    const int we = it.expert % P.period;
    const int panel = it.ci * CW + cw;
    const int col = panel * 32 + 4 * g;                       // first of this lane's 4 columns
    const int colc = col < N ? col : 0;                        // lanes past the last column read column 0's scales
    const size_t meta_row0 = (size_t)we * G;
    // group sums of rows 2kq and 2kq+1 of the block (a row past the expert's last reads the block's first row;
    // its results are not stored)
    const float* xsrow = nullptr;
    int xs_delta = 0;
    float unscale[2] = {1.0f, 1.0f};                          // F16: 2^-e of rows 2kq and 2kq+1, used when the item ends
    if (XSUM) {
      const WsListed& lc = list[q % WS_LIST];
      const int s0 = lc.src[2 * kq], s1 = lc.src[2 * kq + 1];
      xsrow = P.xs + (size_t)s0 * 32;
      xs_delta = (s1 - s0) * 32;
      if (F16) {
        unscale[0] = xsrow[31];
        unscale[1] = xsrow[xs_delta + 31];
      }
    }

    WsStream st[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j)
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i) { st[j].master[m][i] = 0.0f; st[j].grp[m][i] = 0.0f; }
    for (int sj = 0; sj < P.spi; ++sj) {
      if (ok) ok = ws_mbar_wait(full_bar(stage), phase, abort_flag, P.d_status);
      const uint8_t* sbase = ring_ptr + (size_t)stage * P.stage_bytes + (size_t)cw * RS * 128;
      if (ok) {
        for (int j = 0; j < gpw; ++j) {
          const int gi = (sj * KW + kw) * gpw + j;
          if (gi >= G) break;
          // scale / zero words of this group: needed when the group ends
          WsMeta mc[NS];
#pragma unroll
          for (int q2 = 0; q2 < NS; ++q2) mc[q2] = ws_meta_fetch(proj[q2], meta_row0 + gi, N, colc);
          xb[0] = ws_ldg128(xrow + gi * 128 + 64);
          xb[1] = ws_ldg128(xrow + gi * 128 + 72);
          // the group after this one: next j in this stage, or this warp's first group of the next stage
          int gn = gi + 1;
          if (j + 1 == gpw) gn = ((sj + 1) * KW + kw) * gpw;
          const __nv_bfloat16* xnext = xrow;
          bool have_next = gn < G && (j + 1 < gpw || sj + 1 < P.spi);
          if (!have_next && have_next_item && g_first < G) {    // last group of the item: on to the next item
            have_next = true;
            gn = g_first;
            xnext = xrow_next;
          }
          float xs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
          if (XSUM) {                                           // needed when the group ends
            xs[0] = xsrow[gi];
            xs[1] = xsrow[xs_delta + gi];
          }
          // Step s of a group takes word row 8*(s >> 1) + 2*kq + (s & 1) of the group's sixteen (k = 8 x word row):
          // with the swizzle the eight lanes of a quarter warp then read eight different 16-byte positions.
          const uint8_t* rows = sbase + (size_t)((kw * gpw + j) * 16 + 2 * kq) * 128;
          const uint32_t piece[2] = {(uint32_t)((g ^ (2 * kq)) << 4), (uint32_t)((g ^ (2 * kq + 1)) << 4)};
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const uint4 xv = s < 2 ? xa[s] : xb[s - 2];
            if (s == 2 && have_next) {                          // xa is free: fetch the next group's first half
              xa[0] = ws_ldg128(xnext + gn * 128);
              xa[1] = ws_ldg128(xnext + gn * 128 + 8);
            }
            uint32_t b[4] = {xv.x, xv.y, xv.z, xv.w};
            if (!XSHUF) {
              b[0] = ws_prmt(xv.x, xv.z, 0x5410);
              b[1] = ws_prmt(xv.x, xv.z, 0x7632);
              b[2] = ws_prmt(xv.y, xv.w, 0x5410);
              b[3] = ws_prmt(xv.y, xv.w, 0x7632);
            }
            if (!XSUM) {
              ws_mma<false>(xs, BF16_ONES2, BF16_ONES2, BF16_ONES2, BF16_ONES2, b[0], b[1]);
              ws_mma<false>(xs, BF16_ONES2, BF16_ONES2, BF16_ONES2, BF16_ONES2, b[2], b[3]);
            }
            {
              const uint4 wv = *reinterpret_cast<const uint4*>(rows + (s >> 1) * 1024 + (s & 1) * 128 + piece[s & 1]);
              ws_step<F16>(st[0], wv, b);
            }
            if (SWIGLU) {
              const uint4 wv =
                  *reinterpret_cast<const uint4*>(rows + (s >> 1) * 1024 + (s & 1) * 128 + piece[s & 1] + proj_bytes);
              ws_step<F16>(st[NS - 1], wv, b);
            }
          }
#pragma unroll
          for (int q2 = 0; q2 < NS; ++q2) ws_flush(st[q2], mc[q2], xs[0], xs[1]);
        }
      }
      // the previous item's outputs: as soon as the other warps' partial sums are there (a test, not a wait),
      // at the latest in this item's last stage
      if (have_pend && (sj + 1 == P.spi || ws_mbar_test(ready_bar(cw), (uint32_t)(pend.q & 1)))) {
        finish(pend);
        have_pend = false;
      }
      // Done with the stage.  The last warp to get here refills the slot with the stage nst further on.
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        if (atomicAdd(&stage_done[stage], 1) == WS_CONSUMERS - 1) {
          stage_done[stage] = 0;
          ws_fence_proxy_async();                               // the warps' reads precede the copy's writes
          if (!*abort_flag) load_stage(nstage + P.nst);
        }
      }
      ++nstage;
      if (++stage == P.nst) { stage = 0; phase ^= 1u; }
    }
    if (F16) {                                                 // back to the rows' own scale (a power of two: exact)
#pragma unroll
      for (int q2 = 0; q2 < NS; ++q2)
#pragma unroll
        for (int idx = 0; idx < 8; ++idx) st[q2].master[idx >> 2][idx & 3] *= unscale[idx & 1];
    }
    Pending cur_f;
    cur_f.row0 = it.row0; cur_f.rows = it.rows; cur_f.col = col; cur_f.q = q;
    if (KW == 1) {
#pragma unroll
      for (int idx = 0; idx < 8; ++idx)
        store_out(cur_f, idx, st[0].master[idx >> 2][idx & 3], st[NS - 1].master[idx >> 2][idx & 3]);
    } else {
      // the previous item's partial sums have been read by every warp of the panel (they were, a stage ago)
      if (q > 0 && ok) ok = ws_mbar_wait(taken_bar(cw), (uint32_t)((q - 1) & 1), abort_flag, P.d_status);
      float* mine = red + ((size_t)(cw * NS * 8) * KW + kw) * 32 + lane;
#pragma unroll
      for (int q2 = 0; q2 < NS; ++q2)
#pragma unroll
        for (int idx = 0; idx < 8; ++idx) mine[(q2 * 8 + idx) * KW * 32] = st[q2].master[idx >> 2][idx & 3];
      __syncwarp();
      if (lane == 0) ws_mbar_arrive(ready_bar(cw));
      pend = cur_f;
      have_pend = true;
    }
    it = it_next;
    xrow = xrow_next;
  }
  if (have_pend) finish(pend);
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*WsEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

WsEncodeTiledFn ws_encode_fn() {
  static WsEncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<WsEncodeTiledFn>(p);
  });
  return fn;
}

// qweight [period, Kd/8, N] int32 seen as (32 columns, Kd/8 word rows, N/32 panels, period); a box is
// (32, box_rows, box_panels, 1) and lands as box_panels dense panels of box_rows 128-byte rows, the 16-byte
// pieces of a row exchanged by the 128-byte swizzle (piece c of row r sits at position c ^ (r & 7)).  Word rows
// and panels outside the tensor read as zero.
bool ws_make_map(CUtensorMap* map, const void* qweight, int64_t period, int64_t Kd, int64_t N, int box_rows,
                 int box_panels) {
  WsEncodeTiledFn fn = ws_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {32, (cuuint64_t)(Kd / 8), (cuuint64_t)(N / 32), (cuuint64_t)period};
  cuuint64_t strides[3] = {(cuuint64_t)N * 4, 128, (cuuint64_t)(Kd / 8) * (cuuint64_t)N * 4};
  cuuint32_t box[4] = {32, (cuuint32_t)box_rows, (cuuint32_t)box_panels, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, const_cast<void*>(qweight), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Dynamic shared memory of a launch: the small structures, the gap up to the ring's 1024-byte boundary and the
// ring with the partial sums.  The dynamic area starts after the driver's reserved bytes and the kernel's static
// variables; the kernel re-checks the room it finds.  Sets the kernel's limit; 0 if the device cannot give it.
int ws_dynamic_smem_bytes(const void* kernel) {
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) return 0;
  int dev = 0, reserved = 0, optin = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev);
  cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const int start = reserved + (((int)fa.sharedSizeBytes + 15) & ~15);          // where the dynamic area begins
  const int ring = (start + WS_SMALL_BYTES + 1023) & ~1023;
  int need = ring - start + WS_RING_BYTES + WS_RED_BYTES;
  const int room = optin - (int)fa.sharedSizeBytes;
  if (need > room) return 0;
  // whatever is left goes in as well: it costs nothing (one CTA per SM) and covers a start the estimate missed
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, room) != cudaSuccess) return 0;
  return room;
}

int ws_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

bool w4a16_stream_covers(int64_t S, int64_t E, int64_t period, int64_t N, int64_t Kd, int64_t group) {
  if (group != 128 || Kd % 128 != 0 || N % 32 != 0 || E > WS_MAX_GROUPS) return false;
  if (Kd / 128 > 4096 || N / 32 > (1 << 20) || period > (1 << 20)) return false;
  // 32-bit item indices: (experts + row blocks) * column items
  if ((E + S / 8 + 1) * (N / 32) >= ((int64_t)1 << 30)) return false;
  return true;
}

// x: activations; perm != nullptr gathers row p of the sorted order from x[perm[p] / top_k].
// x_format: 0 = bf16 rows in natural k order; 1 = bf16 rows with the k order 0,4,1,5,2,6,3,7 inside every 8;
// 2 = that order in fp16, every row scaled by its power of two (needs xs); xs (optional): group sums of the rows
// of x, [rows, 32] fp32 (both are what mq_w4a16_tc_prep writes).  shuffle_out: write the output columns in
// that same order (it is then the prepared input of the next projection).
// qw/sc/qz of the projection(s) in the checkpoint layout, `period` weight sets.
int w4a16_stream(const void* x, const float* xs, int x_format, const int32_t* perm, int64_t top_k,
                 const int32_t* qw0, const void* sc0, const int32_t* qz0, const int32_t* qw1, const void* sc1,
                 const int32_t* qz1, bool swiglu, bool shuffle_out, const int32_t* offsets, int64_t S, int64_t E,
                 int64_t period, int64_t N, int64_t Kd, void* out, int32_t* d_status, cudaStream_t st) {
  const int G = (int)(Kd / 128);
  const int nproj = swiglu ? 2 : 1;
  if (xs != nullptr && G > 32) return MQ_ERR_UNSUPPORTED_SHAPE;       // the sums table has 32 groups per row
  // Column panels per item: as many as still leave about four items per SM.  The number of experts hit is
  // at most min(E, S), and every one of them has at least one block of rows.
  const int64_t active = S < E ? S : E;
  const int64_t panels = N / 32;
  int CW = 1;
  for (int c : {16, 8, 4, 2}) {
    if (swiglu && c >= 8) continue;                 // a gate + up stage of 8 panels would not fit the ring
    const int64_t items = active * ((panels + c - 1) / c);
    // 16 panels = no K split at all (no partial sums to add up): worth fewer items per SM
    if (items >= (c == 16 ? 3 : 4) * ws_sm_count()) { CW = c; break; }
  }
  const int KW = WS_CONSUMERS / CW;
  // groups per warp and stage: as many as keep a stage within 64 KB (SwiGLU: two projections) / 96 KB
  const int per_group_bytes = nproj * 128 * 16 * KW * CW;          // stage bytes for gpw = 1
  const int limit = swiglu ? 64 * 1024 : 96 * 1024;
  int gpw = limit / per_group_bytes;
  const int need = (G + KW - 1) / KW;                                // groups per warp to cover K in one stage
  if (gpw > need) gpw = need;
  if (gpw < 1) gpw = 1;
  const int RS = 16 * KW * gpw;
  if (RS > 256) return MQ_ERR_UNSUPPORTED_SHAPE;                     // box dimension limit (not reached: KW*gpw <= 16)

  WsParams P;
  P.x = reinterpret_cast<const __nv_bfloat16*>(x);
  P.xs = xs;
  P.perm = perm;
  P.top_k = (int)top_k;
  P.shuffle_out = shuffle_out ? 1 : 0;
  P.offsets = offsets;
  P.E = (int)E;
  P.period = (int)period;
  P.N = (int)N;
  P.Kd = (int)Kd;
  P.G = G;
  P.KW = KW;
  P.CW = CW;
  P.gpw = gpw;
  P.RS = RS;
  P.spi = (G + KW * gpw - 1) / (KW * gpw);
  P.ipe = (int)((panels + CW - 1) / CW);
  P.stage_bytes = (uint32_t)(nproj * RS * CW * 128);
  P.nst = WS_RING_BYTES / (int)P.stage_bytes;
  if (P.nst > WS_MAX_STAGES) P.nst = WS_MAX_STAGES;
  if (P.nst < 2) return MQ_ERR_UNSUPPORTED_SHAPE;
  P.p0 = WsProj{reinterpret_cast<const __nv_bfloat16*>(sc0), qz0};
  P.p1 = WsProj{reinterpret_cast<const __nv_bfloat16*>(swiglu ? sc1 : sc0), swiglu ? qz1 : qz0};
  P.out = reinterpret_cast<__nv_bfloat16*>(out);
  P.d_status = d_status;

  CUtensorMap map0, map1;
  if (!ws_make_map(&map0, qw0, period, Kd, N, RS, CW) || !ws_make_map(&map1, swiglu ? qw1 : qw0, period, Kd, N, RS, CW))
    return MQ_ERR_DRIVER_ENTRY;
  const int grid = ws_sm_count();
  const bool xsum = xs != nullptr;
#define MQ_WS_LAUNCH(SW, XSH, XSU, F16)                                                                            \
  do {                                                                                                             \
    static const int smem =                                                                                        \
        ws_dynamic_smem_bytes(reinterpret_cast<const void*>(w4a16_stream_kernel<SW, XSH, XSU, F16>));              \
    if (smem <= 0) return MQ_ERR_LAUNCH_FAILED;                                                                    \
    launch_after_predecessor(w4a16_stream_kernel<SW, XSH, XSU, F16>, dim3(grid), dim3(WS_THREADS), (size_t)smem,   \
                             st, map0, map1, P);                                                                   \
  } while (0)
  const bool x_shuffled = x_format != 0;
  if (x_format == 2 && (!xsum || G > 31)) return MQ_ERR_INVALID_ARGUMENT;       // fp16 rows come with their sums table
  if (swiglu) {
    if (x_format == 2) MQ_WS_LAUNCH(true, true, true, true);
    else if (x_shuffled && xsum) MQ_WS_LAUNCH(true, true, true, false);
    else if (x_shuffled) MQ_WS_LAUNCH(true, true, false, false);
    else if (!xsum) MQ_WS_LAUNCH(true, false, false, false);
    else return MQ_ERR_INVALID_ARGUMENT;             // sums without the shuffled rows: not a combination any caller makes
  } else {
    if (x_format == 2) MQ_WS_LAUNCH(false, true, true, true);
    else if (x_shuffled && xsum) MQ_WS_LAUNCH(false, true, true, false);
    else if (x_shuffled) MQ_WS_LAUNCH(false, true, false, false);
    else if (!xsum) MQ_WS_LAUNCH(false, false, false, false);
    else return MQ_ERR_INVALID_ARGUMENT;
  }
#undef MQ_WS_LAUNCH
  return check_launch();
}

}  // namespace mq

