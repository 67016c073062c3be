// W4A16 linear for few rows per expert (decode): out = x . dequant(q, z, s), bf16 in/out.
// Format and arithmetic follow mini_qwen/kernels/w4a16_gemm.py:8-15 and
// tests/test_w4a16_gemm.py:19-44 of the reference: W[k,n] = (q[k,n] - z[k/g,n]) * s[k/g,n].
//
// The work is a stream over the packed weights.  At 6.5 TB/s a B200 delivers 46 int4 weights per SM
// and clock, which leaves under three lane-instructions per weight: the kernel is organised to
// spend as few instructions per weight as possible, not around an output tile.
//   * A lane reads one 128-bit vector = 4 adjacent columns x 8 consecutive k of packed int4,
//     straight in the checkpoint layout [K/8, N] (8 lanes cover a full 128-byte line).
//   * Nibbles become bf16 with ONE logic op per pair: (w >> 4p) & 0x000F000F | 0x43004300 is the
//     bf16 pair {128+q[p], 128+q[p+4]}, re-centred to {q[p]-8, q[p+4]-8} by one packed fma on the FMA
//     pipe.  The zero point is not subtracted per weight: with
//     xs = sum_k x[k] over the group (obtained from one extra MMA against a tile of ones),
//        sum_k x[k] * (q[k] - z) = sum_k x[k] * (q[k] - 8)  -  (z - 8) * xs ,
//     and the right-hand side is evaluated once per group and column in fp32.
//   * The biased integers are the A operand (16 columns x 16 k) of mma.sync.m16n8k16 with the
//     activations as the 8-wide B operand ("swap-AB": rows of x are the narrow dimension); the k
//     order inside a word is permuted identically on both operands.
//   * A group's sum is scaled once by s (fp32) when the group ends, so the dequantised weight is
//     never rounded to bf16.
//   * Each warp streams TWO weight tiles against the same activations (gate and up of the same
//     32 columns for SwiGLU, two adjacent 32-column tiles otherwise); the 4 warps of a CTA split K
//     and their partial sums meet in shared memory in a fixed order.
//   * Every lane moves its own 16-byte pieces (weights and activations) through an 8-deep ring of
//     cp.async copies in shared memory: a lane only reads what it copied itself, so the ring needs
//     no barrier and has no bank conflicts, and 12 KB per warp are in flight while it computes.
#include <cstdlib>

#include "common.cuh"

namespace mq {
namespace {

constexpr int W4_WARPS = 4;
constexpr int W4_DEPTH = 4;       // k-steps (32 k each) in flight per warp (power of two)
constexpr int W4_NS = 2;          // weight streams per warp
constexpr uint32_t BF16_ONES = 0x3F803F80u;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc)
               : "memory");
}
// the same through L1: for the activation pieces, which the four warps of a CTA (four column tiles, the same rows and
// k) all fetch within a few hundred cycles of one another (down projection at batch 64: 38.5 -> 36.6 us)
__device__ __forceinline__ void cp_async16_l1(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// pair p of word w -> bf16x2 {q[p] - 8, q[p+4] - 8}: the logic op makes {128 + q[p], 128 + q[p+4]}, a packed
// fma on the (idle) FMA pipe takes the 136 off again, so that a group's sum stays as small as the result
// instead of carrying 128 * sum(x) that has to cancel in fp32 later.
__device__ __forceinline__ uint32_t biased_pair(uint32_t w, int p) {
  uint32_t v, c;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(w >> (4 * p)), "r"(0x000F000Fu), "r"(0x43004300u));
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(c) : "r"(v), "r"(0x3F803F80u), "r"(0xC308C308u));
  return c;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct W4Proj {
  const int32_t* qw;        // [E, Kd/8, N]
  const __nv_bfloat16* sc;  // [E, Kd/g, N]
  const int32_t* qz;        // [E, Kd/g, N/8]
};

// One weight stream of a lane: 4 columns x (rows 2kq, 2kq+1) in two MMA fragments.
struct W4Stream {
  float master[2][4];
  float grp[2][4];
  float scale[4];
  float zoff[4];            // zero point of the current group, minus 8
};

__device__ __forceinline__ void stream_init(W4Stream& a) {
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) { a.master[m][i] = 0.0f; a.grp[m][i] = 0.0f; }
#pragma unroll
  for (int c = 0; c < 4; ++c) { a.scale[c] = 0.0f; a.zoff[c] = 0.0f; }
}

// End of a group: master += s * (sum_k x*(q-8) - (z-8) * sum_k x), then restart the group sums.
__device__ __forceinline__ void stream_flush(W4Stream& a, const float (&xs)[4]) {
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = 2 * m + (i >> 1);
      const float t = fmaf(-a.zoff[col], xs[i & 1], a.grp[m][i]);
      a.master[m][i] = fmaf(a.scale[col], t, a.master[m][i]);
      a.grp[m][i] = 0.0f;
    }
}

__device__ __forceinline__ void stream_step(W4Stream& a, const uint4& wv, const uint32_t (&b)[4]) {
  const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
  uint32_t d[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int p = 0; p < 4; ++p) d[c][p] = biased_pair(w[c], p);
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    mma_bf16_16816(a.grp[m], d[2 * m][0], d[2 * m + 1][0], d[2 * m][1], d[2 * m + 1][1], b[0], b[1]);
    mma_bf16_16816(a.grp[m], d[2 * m][2], d[2 * m + 1][2], d[2 * m][3], d[2 * m + 1][3], b[2], b[3]);
  }
}

// Raw scale / zero-point words of one group for a lane's 4 columns (fetched one group ahead).
struct W4Meta {
  uint2 s;
  uint32_t z;
};

__device__ __forceinline__ W4Meta meta_fetch(const __nv_bfloat16* sc, const int32_t* qz, int col) {
  W4Meta m;
  m.s = __ldg(reinterpret_cast<const uint2*>(sc + col));
  m.z = (uint32_t)__ldg(qz + (col >> 3)) >> ((col & 7) * 4);
  return m;
}

__device__ __forceinline__ void stream_set_group(W4Stream& a, const W4Meta& m) {
  a.scale[0] = __uint_as_float(m.s.x << 16);
  a.scale[1] = __uint_as_float(m.s.x & 0xffff0000u);
  a.scale[2] = __uint_as_float(m.s.y << 16);
  a.scale[3] = __uint_as_float(m.s.y & 0xffff0000u);
#pragma unroll
  for (int c = 0; c < 4; ++c) a.zoff[c] = (float)((int)((m.z >> (4 * c)) & 0xFu) - 8);
}

// The y-th non-empty group of rows (y = blockIdx.y), found with ballots over the offsets; -1 if
// there are fewer.  Lets a decode launch size its grid by the slot count instead of the expert count.
__device__ int nth_nonempty(const int32_t* offsets, int E, int y, int* s_e) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int found = -1, seen = 0;
    for (int e0 = 0; e0 < E && found < 0; e0 += 32) {
      const int e = e0 + lane;
      const bool ne = e < E && offsets[e + 1] > offsets[e];
      const unsigned m = __ballot_sync(0xffffffffu, ne);
      const int c = __popc(m);
      if (y < seen + c) {
        unsigned mm = m;
        for (int i = 0; i < y - seen; ++i) mm &= mm - 1;     // drop the lowest set bits
        found = e0 + __ffs(mm) - 1;
      }
      seen += c;
    }
    if (lane == 0) *s_e = found;
  }
  __syncthreads();
  return *s_e;
}

// KSPLIT = 4: the CTA's warps split K over one column tile (few rows in total: more CTAs per byte).
// KSPLIT = 1: every warp owns its own column tile and runs the whole K (long streams, no exchange).
template <bool SWIGLU, int KSPLIT>
__global__ void __launch_bounds__(W4_WARPS * 32, 4)
w4a16_grouped_kernel(const __nv_bfloat16* __restrict__ x, W4Proj p0, W4Proj p1,
                     const int32_t* __restrict__ offsets, int E, int period, int N, int Kd, int group,
                     int compact, __nv_bfloat16* __restrict__ out) {
  // SWIGLU: the two streams of a warp are the gate and up projections of the same 32 columns.
  // Plain: the two streams are adjacent 32-column tiles (64 columns per warp).
  constexpr int SLOT = W4_NS + 1;                    // 16-byte pieces per lane and k-step: 2 weights + x
  __shared__ uint4 ring[W4_WARPS][W4_DEPTH][SLOT][32];

  pdl_wait();                     // offsets and x come from the kernels before this one
  pdl_release();
  int e = (int)blockIdx.y;
  if (compact) {
    // the first word of the (still unused) ring carries the expert index from warp 0 to the others
    e = nth_nonempty(offsets, E, blockIdx.y, reinterpret_cast<int*>(&ring[0][0][0][0]));
    __syncthreads();                     // everyone has read it before any copy lands in the ring
  }
  if (e < 0) return;
  const int row_lo = offsets[e];
  const int rows = offsets[e + 1] - row_lo;
  if (rows <= 0) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, kq = lane & 3;
  const int cols_per_tile = SWIGLU ? 32 : 64;
  const int tile = KSPLIT == 1 ? (int)blockIdx.x * W4_WARPS + warp : (int)blockIdx.x;
  const int col[W4_NS] = {tile * cols_per_tile + 4 * g, tile * cols_per_tile + (SWIGLU ? 0 : 32) + 4 * g};
  const bool col_ok[W4_NS] = {col[0] < N, col[1] < N};
  // lanes past the last column (or row) stream a valid neighbour instead and simply do not store:
  // the inner loop then carries no per-lane selects
  const int colc[W4_NS] = {col_ok[0] ? col[0] : N - 4, col_ok[1] ? col[1] : N - 4};

  const int steps_total = Kd / 32;
  const int spw = KSPLIT == 1 ? steps_total : (steps_total + W4_WARPS - 1) / W4_WARPS;
  const int s_lo = KSPLIT == 1 ? 0 : warp * spw;
  const int s_hi = min(s_lo + spw, steps_total);
  const int spg = group / 32;           // k-steps per quantisation group
  const int G = Kd / group;

  const int we = e % period;            // weight set of this group of rows
  const W4Proj proj[W4_NS] = {p0, SWIGLU ? p1 : p0};
  const int32_t* qw[W4_NS];
  const __nv_bfloat16* sc[W4_NS];
  const int32_t* qz[W4_NS];
#pragma unroll
  for (int j = 0; j < W4_NS; ++j) {
    qw[j] = proj[j].qw + (size_t)we * (Kd / 8) * N + (size_t)kq * N + colc[j];
    sc[j] = proj[j].sc + (size_t)we * G * N;
    qz[j] = proj[j].qz + (size_t)we * G * (N / 8);
  }
  uint4* const ring_lane = &ring[warp][0][0][lane];
  constexpr int SLOT_STRIDE = SLOT * 32;             // uint4 elements between two ring slots

  for (int r0 = 0; r0 < rows; r0 += 8) {
    W4Stream st[W4_NS];
#pragma unroll
    for (int j = 0; j < W4_NS; ++j) stream_init(st[j]);
    float xs[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    const int rowc = r0 + g < rows ? r0 + g : 0;
    const __nv_bfloat16* xrow = x + (size_t)(row_lo + rowc) * Kd + 8 * kq;

    // Prologue: DEPTH steps in flight.  One commit group per k-step, empty when there is nothing
    // left to fetch, so "all but the newest DEPTH-1 groups are complete" means "this step has landed".
    uint32_t w_off = (uint32_t)(4 * s_lo) * (uint32_t)N;     // element offset of the next step to fetch
    uint32_t x_off = 32u * (uint32_t)s_lo;
    int fetch = s_lo;
#pragma unroll
    for (int i = 0; i < W4_DEPTH; ++i) {
      if (fetch < s_hi) {
        uint4* sl = ring_lane + i * SLOT_STRIDE;
        cp_async16(sl, qw[0] + w_off);
        cp_async16(sl + 32, qw[1] + w_off);
        cp_async16_l1(sl + 64, xrow + x_off);
      }
      cp_async_commit();
      w_off += 4u * (uint32_t)N;
      x_off += 32u;
      ++fetch;
    }

    // scales and zero points travel one group ahead of their use
    int gi = s_lo / spg;
    int left = spg - (s_lo - gi * spg);                // steps until the current group ends
    W4Meta next[W4_NS];
#pragma unroll
    for (int j = 0; j < W4_NS; ++j) {
      const W4Meta cur = meta_fetch(sc[j] + (size_t)gi * N, qz[j] + (size_t)gi * (N / 8), colc[j]);
      stream_set_group(st[j], cur);
      next[j] = cur;
      if (gi + 1 < G) next[j] = meta_fetch(sc[j] + (size_t)(gi + 1) * N, qz[j] + (size_t)(gi + 1) * (N / 8), colc[j]);
    }

    int slot_idx = 0;
    for (int s = s_lo; s < s_hi; ++s) {
      cp_async_wait<W4_DEPTH - 1>();
      uint4* sl = ring_lane + slot_idx * SLOT_STRIDE;
      const uint4 wv0 = sl[0];
      const uint4 wv1 = sl[32];
      const uint4 xv = sl[64];
      if (fetch < s_hi) {                              // refill the slot just read
        cp_async16(sl, qw[0] + w_off);
        cp_async16(sl + 32, qw[1] + w_off);
        cp_async16_l1(sl + 64, xrow + x_off);
      }
      cp_async_commit();
      w_off += 4u * (uint32_t)N;
      x_off += 32u;
      ++fetch;
      slot_idx = (slot_idx + 1) & (W4_DEPTH - 1);
      // activations: 8 consecutive k of row g, permuted to the nibble-pair order
      const uint32_t b[4] = {prmt(xv.x, xv.z, 0x5410),   // {x0, x4}
                             prmt(xv.x, xv.z, 0x7632),   // {x1, x5}
                             prmt(xv.y, xv.w, 0x5410),   // {x2, x6}
                             prmt(xv.y, xv.w, 0x7632)};  // {x3, x7}
      mma_bf16_16816(xs, BF16_ONES, BF16_ONES, BF16_ONES, BF16_ONES, b[0], b[1]);
      mma_bf16_16816(xs, BF16_ONES, BF16_ONES, BF16_ONES, BF16_ONES, b[2], b[3]);
      stream_step(st[0], wv0, b);
      stream_step(st[1], wv1, b);
      if (--left == 0) {                               // group boundary
        ++gi;
#pragma unroll
        for (int j = 0; j < W4_NS; ++j) {
          stream_flush(st[j], xs);
          stream_set_group(st[j], next[j]);
          if (gi + 1 < G) next[j] = meta_fetch(sc[j] + (size_t)(gi + 1) * N, qz[j] + (size_t)(gi + 1) * (N / 8), colc[j]);
        }
        xs[0] = xs[1] = xs[2] = xs[3] = 0.0f;
        left = spg;
      }
    }
    cp_async_wait<0>();
    if (left != spg) {                                 // the K range ended inside a group
#pragma unroll
      for (int j = 0; j < W4_NS; ++j) stream_flush(st[j], xs);
    }

    if (KSPLIT > 1) {
      // fixed-order reduction over the K split (the ring is idle now and doubles as the exchange buffer)
      float(*red)[W4_NS][8][32] = reinterpret_cast<float(*)[W4_NS][8][32]>(&ring[0][0][0][0]);
      __syncthreads();
#pragma unroll
      for (int j = 0; j < W4_NS; ++j)
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) red[warp][j][m * 4 + i][lane] = st[j].master[m][i];
      __syncthreads();
      if (warp == 0) {
#pragma unroll
        for (int j = 0; j < W4_NS; ++j)
#pragma unroll
          for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float sum = red[0][j][m * 4 + i][lane];
#pragma unroll
              for (int w = 1; w < W4_WARPS; ++w) sum += red[w][j][m * 4 + i][lane];
              st[j].master[m][i] = sum;
            }
      }
    }
    if (KSPLIT == 1 || warp == 0) {
      // fragment element i of mma m: column 2m + (i >> 1), row 2kq + (i & 1)
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = r0 + 2 * kq + half;
          if (r < rows) {
            __nv_bfloat16* orow = out + (size_t)(row_lo + r) * N + 2 * m;
            if (SWIGLU) {
              if (col_ok[0]) {
                const float o0 = swiglu_rounded<__nv_bfloat16>(st[0].master[m][half], st[1].master[m][half]);
                const float o1 = swiglu_rounded<__nv_bfloat16>(st[0].master[m][2 + half], st[1].master[m][2 + half]);
                *reinterpret_cast<__nv_bfloat162*>(orow + col[0]) = __floats2bfloat162_rn(o0, o1);
              }
            } else {
#pragma unroll
              for (int j = 0; j < W4_NS; ++j)
                if (col_ok[j])
                  *reinterpret_cast<__nv_bfloat162*>(orow + col[j]) =
                      __floats2bfloat162_rn(st[j].master[m][half], st[j].master[m][2 + half]);
            }
          }
        }
    }
    if (KSPLIT > 1) __syncthreads();
  }
}

template <bool SWIGLU, int KSPLIT>
void launch_w4_variant(const void* x, W4Proj p0, W4Proj p1, const int32_t* offsets, int64_t S, int64_t E,
                       int64_t period, int64_t N, int64_t Kd, int64_t group, void* out, cudaStream_t st) {
  const int cols_per_tile = SWIGLU ? 32 : 64;
  const int cols_per_cta = KSPLIT == 1 ? cols_per_tile * W4_WARPS : cols_per_tile;
  // with fewer slots than experts most experts are empty: index the grid by non-empty experts instead
  const int compact = S < E;
  dim3 grid((unsigned)((N + cols_per_cta - 1) / cols_per_cta), (unsigned)(compact ? S : E));
  launch_after_predecessor(w4a16_grouped_kernel<SWIGLU, KSPLIT>, grid, dim3(W4_WARPS * 32), 0, st,
                           reinterpret_cast<const __nv_bfloat16*>(x), p0, p1, offsets, (int)E, (int)period, (int)N,
                           (int)Kd, (int)group, compact, reinterpret_cast<__nv_bfloat16*>(out));
}

}  // namespace

// TMA-staged persistent stream kernel (w4a16_stream.cu): group size 128, N a multiple of 32.
bool w4a16_stream_covers(int64_t S, int64_t E, int64_t period, int64_t N, int64_t Kd, int64_t group);
int w4a16_stream(const void* x, const float* xs, int x_format, const int32_t* perm, int64_t top_k,
                 const int32_t* qw0, const void* sc0, const int32_t* qz0, const int32_t* qw1, const void* sc1,
                 const int32_t* qz1, bool swiglu, bool shuffle_out, const int32_t* offsets, int64_t S, int64_t E,
                 int64_t period, int64_t N, int64_t Kd, void* out, int32_t* d_status, cudaStream_t st);

namespace {

int launch_w4(const void* x, W4Proj p0, W4Proj p1, bool swiglu, const int32_t* offsets, int64_t S, int64_t E,
              int64_t period, int64_t N, int64_t Kd, int64_t group, void* out, cudaStream_t st,
              const int32_t* perm = nullptr, int64_t top_k = 1, int32_t* d_status = nullptr,
              const float* xs = nullptr, int x_format = 0, bool shuffle_out = false, bool want_stream = false) {
  if (S < 0 || E <= 0 || N <= 0 || Kd <= 0 || group <= 0) return MQ_ERR_INVALID_ARGUMENT;
  if (period <= 0 || period > E) return MQ_ERR_INVALID_ARGUMENT;
  if (group % 32 != 0 || Kd % group != 0 || N % 8 != 0 || E > 65535) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!x || !p0.qw || !p0.sc || !p0.qz || !offsets || !out) return MQ_ERR_INVALID_ARGUMENT;
  if (swiglu && (!p1.qw || !p1.sc || !p1.qz)) return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(x) || !aligned16(p0.qw) || !aligned16(p0.sc) || !aligned16(out)) return MQ_ERR_INVALID_ARGUMENT;
  if (swiglu && (!aligned16(p1.qw) || !aligned16(p1.sc))) return MQ_ERR_INVALID_ARGUMENT;
  // Which kernel: the TMA-staged stream kernel is the faster one for the fused gate/up projection from a few
  // dozen slots on (batch 64: 66 against 81 us; below 32 slots both are bound by launch latency), the per-lane
  // cp.async kernel below for the single projection (40 against 43 us at batch 64: its K is short and it needs
  // no K split).  The prepared-activation entry points ask for the stream kernel explicitly.
  const bool stream = want_stream || (swiglu && S >= 32);
  if (stream && w4a16_stream_covers(S, E, period, N, Kd, group))
    return w4a16_stream(x, xs, x_format, perm, top_k, p0.qw, p0.sc, p0.qz, p1.qw, p1.sc, p1.qz, swiglu, shuffle_out,
                        offsets, S, E, period, N, Kd, out, d_status, st);
  // the fallback kernel wants expert-sorted rows in natural order
  if (perm != nullptr || x_format != 0 || shuffle_out) return MQ_ERR_UNSUPPORTED_SHAPE;
  // few rows in total (a handful of experts hit): split K across the warps of a CTA to get enough CTAs;
  // otherwise every warp streams the whole K of its own column tile
  bool split = S <= 32;
  if (swiglu) {
    if (split) launch_w4_variant<true, 4>(x, p0, p1, offsets, S, E, period, N, Kd, group, out, st);
    else launch_w4_variant<true, 1>(x, p0, p1, offsets, S, E, period, N, Kd, group, out, st);
  } else {
    if (split) launch_w4_variant<false, 4>(x, p0, p0, offsets, S, E, period, N, Kd, group, out, st);
    else launch_w4_variant<false, 1>(x, p0, p0, offsets, S, E, period, N, Kd, group, out, st);
  }
  return check_launch();
}

}  // namespace
}  // namespace mq

extern "C" int mq_w4a16_grouped_gemm(const void* x, const int32_t* qweight, const void* scales,
                                     const int32_t* qzeros, const int32_t* offsets,
                                     int64_t S, int64_t E, int64_t weight_period, int64_t N, int64_t Kd,
                                     int64_t group_size, void* out, void* stream) {
  mq::W4Proj p{qweight, reinterpret_cast<const __nv_bfloat16*>(scales), qzeros};
  return mq::launch_w4(x, p, p, false, offsets, S, E, weight_period, N, Kd, group_size, out,
                       reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int mq_w4a16_grouped_swiglu(const void* x,
                                       const int32_t* qweight_gate, const void* scales_gate, const int32_t* qzeros_gate,
                                       const int32_t* qweight_up, const void* scales_up, const int32_t* qzeros_up,
                                       const int32_t* offsets,
                                       int64_t S, int64_t E, int64_t weight_period, int64_t I, int64_t H,
                                       int64_t group_size, void* h, void* stream) {
  mq::W4Proj pg{qweight_gate, reinterpret_cast<const __nv_bfloat16*>(scales_gate), qzeros_gate};
  mq::W4Proj pu{qweight_up, reinterpret_cast<const __nv_bfloat16*>(scales_up), qzeros_up};
  return mq::launch_w4(x, pg, pu, true, offsets, S, E, weight_period, I, H, group_size, h,
                       reinterpret_cast<cudaStream_t>(stream));
}

/* Prepared-activation forms: see include/mqmoe.h. */
extern "C" int mq_w4a16_stream_swiglu(const void* xp, const float* xs, int x_format, const int32_t* perm,
                                      int64_t top_k, const int32_t* qweight_gate, const void* scales_gate, const int32_t* qzeros_gate,
                                      const int32_t* qweight_up, const void* scales_up, const int32_t* qzeros_up,
                                      const int32_t* offsets, int64_t S, int64_t E, int64_t weight_period, int64_t I,
                                      int64_t H, int64_t group_size, int shuffle_out, void* h, int32_t* d_status,
                                      void* stream) {
  mq::W4Proj pg{qweight_gate, reinterpret_cast<const __nv_bfloat16*>(scales_gate), qzeros_gate};
  mq::W4Proj pu{qweight_up, reinterpret_cast<const __nv_bfloat16*>(scales_up), qzeros_up};
  if (!mq::w4a16_stream_covers(S, E, weight_period, I, H, group_size)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if ((perm != nullptr && top_k <= 0) || x_format < 0 || x_format > 2) return MQ_ERR_INVALID_ARGUMENT;
  return mq::launch_w4(xp, pg, pu, true, offsets, S, E, weight_period, I, H, group_size, h,
                       reinterpret_cast<cudaStream_t>(stream), perm, perm != nullptr ? top_k : 1, d_status, xs,
                       x_format, shuffle_out != 0, true);
}

extern "C" int mq_w4a16_stream_gemm(const void* xp, const float* xs, int x_format, const int32_t* qweight,
                                    const void* scales, const int32_t* qzeros, const int32_t* offsets, int64_t S,
                                    int64_t E, int64_t weight_period, int64_t N, int64_t Kd, int64_t group_size,
                                    void* out, int32_t* d_status, void* stream) {
  mq::W4Proj p{qweight, reinterpret_cast<const __nv_bfloat16*>(scales), qzeros};
  if (!mq::w4a16_stream_covers(S, E, weight_period, N, Kd, group_size)) return MQ_ERR_UNSUPPORTED_SHAPE;
  return mq::launch_w4(xp, p, p, false, offsets, S, E, weight_period, N, Kd, group_size, out,
                       reinterpret_cast<cudaStream_t>(stream), nullptr, 1, d_status, xs, x_format, false, true);
}
