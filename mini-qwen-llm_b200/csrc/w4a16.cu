// W4A16 linear for few rows per expert (decode): out = x . dequant(q, z, s), bf16 in/out.
// Format and arithmetic follow mini_qwen/kernels/w4a16_gemm.py:8-15 and
// tests/test_w4a16_gemm.py:19-44 of the reference: W[k,n] = (q[k,n] - z[k/g,n]) * s[k/g,n].
//
// The work is a stream over the packed weights (HBM-bound), so the kernel is organised around
// the weight words, not around the output tile:
//   * a lane reads one 128-bit vector = 4 adjacent columns x 8 consecutive k of packed int4,
//     straight in the checkpoint layout [K/8, N] (8 lanes cover a full 128-byte line);
//   * nibbles become bf16 in registers: (w >> 4p) & 0x000F000F | 0x43004300 is the bf16 pair
//     {128+q[p], 128+q[p+4]}, and one packed subtract of {128+z, 128+z} leaves the exact
//     integers q-z;
//   * those integers are the A operand (16 columns x 16 k) of mma.sync.m16n8k16 with the
//     activations as the 8-wide B operand ("swap-AB": rows of x are the narrow dimension), the
//     k order inside a word being permuted identically on both operands;
//   * a group's partial sum is scaled once by s (fp32) when the group ends, so the dequantised
//     weight is never rounded to bf16: sum_k x*(q-z) is exact-integer weights in the tensor core,
//     times s in fp32, which is the reference's all-fp32 formula up to summation order;
//   * the 4 warps of a CTA split K; their partial sums meet in shared memory in a fixed order;
//   * every lane streams its own 16-byte pieces (weights and activations) through an 8-deep ring of
//     cp.async copies in shared memory: a lane only ever reads what it copied itself, so the ring
//     needs no barrier and no bank-conflict care, and 12 KB per warp are in flight while it computes.
#include "common.cuh"

namespace mq {
namespace {

constexpr int W4_WARPS = 4;
constexpr int W4_NB = 1;          // row blocks of 8 handled per pass over the weights
constexpr int W4_DEPTH = 8;       // k-steps (32 k each) in flight per warp

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc)
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

// pair p of word w -> bf16x2 {q[p] - z, q[p+4] - z}
__device__ __forceinline__ uint32_t dequant_pair(uint32_t w, int p, uint32_t zb) {
  uint32_t v;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(w >> (4 * p)), "r"(0x000F000Fu), "r"(0x43004300u));
  __nv_bfloat162 d = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), *reinterpret_cast<__nv_bfloat162*>(&zb));
  return *reinterpret_cast<uint32_t*>(&d);
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

// Accumulators of one projection for one lane: 4 columns x 2 rows per row block.
struct W4Acc {
  float master[W4_NB][2][4];
  float grp[W4_NB][2][4];
  float scale[4];
  uint32_t zb[4];
};

__device__ __forceinline__ void acc_init(W4Acc& a) {
#pragma unroll
  for (int tb = 0; tb < W4_NB; ++tb)
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) { a.master[tb][m][i] = 0.0f; a.grp[tb][m][i] = 0.0f; }
#pragma unroll
  for (int c = 0; c < 4; ++c) { a.scale[c] = 0.0f; a.zb[c] = 0x43004300u; }
}

__device__ __forceinline__ void acc_flush(W4Acc& a) {
#pragma unroll
  for (int tb = 0; tb < W4_NB; ++tb)
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a.master[tb][m][i] = fmaf(a.scale[2 * m + (i >> 1)], a.grp[tb][m][i], a.master[tb][m][i]);
        a.grp[tb][m][i] = 0.0f;
      }
}

__device__ __forceinline__ void load_group(W4Acc& a, const W4Proj& p, size_t sc_row, size_t qz_row, int col0) {
  uint2 s = __ldg(reinterpret_cast<const uint2*>(p.sc + sc_row + col0));
  a.scale[0] = __uint_as_float(s.x << 16);
  a.scale[1] = __uint_as_float(s.x & 0xffff0000u);
  a.scale[2] = __uint_as_float(s.y << 16);
  a.scale[3] = __uint_as_float(s.y & 0xffff0000u);
  uint32_t zw = (uint32_t)__ldg(p.qz + qz_row + (col0 >> 3));
  zw >>= (col0 & 7) * 4;
#pragma unroll
  for (int c = 0; c < 4; ++c) a.zb[c] = (0x4300u | ((zw >> (4 * c)) & 0xFu)) * 0x00010001u;
}

__device__ __forceinline__ void step_mma(W4Acc& a, const uint4& wv, const uint32_t (&bfrag)[W4_NB][4]) {
  const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
  uint32_t d[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int p = 0; p < 4; ++p) d[c][p] = dequant_pair(w[c], p, a.zb[c]);
#pragma unroll
  for (int tb = 0; tb < W4_NB; ++tb) {
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      mma_bf16_16816(a.grp[tb][m], d[2 * m][0], d[2 * m + 1][0], d[2 * m][1], d[2 * m + 1][1],
                     bfrag[tb][0], bfrag[tb][1]);
      mma_bf16_16816(a.grp[tb][m], d[2 * m][2], d[2 * m + 1][2], d[2 * m][3], d[2 * m + 1][3],
                     bfrag[tb][2], bfrag[tb][3]);
    }
  }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(W4_WARPS * 32)
w4a16_grouped_kernel(const __nv_bfloat16* __restrict__ x, W4Proj p0, W4Proj p1,
                     const int32_t* __restrict__ offsets, int period, int N, int Kd, int group,
                     __nv_bfloat16* __restrict__ out) {
  constexpr int NP = SWIGLU ? 2 : 1;
  constexpr int SLOT = NP + W4_NB;                  // 16-byte pieces per lane and k-step
  extern __shared__ uint4 ring_raw[];               // [W4_WARPS][W4_DEPTH][SLOT][32] 16-byte pieces
  uint4(*ring)[W4_DEPTH][SLOT][32] = reinterpret_cast<uint4(*)[W4_DEPTH][SLOT][32]>(ring_raw);
  __shared__ float red[W4_WARPS][NP][W4_NB * 8][32];

  const int e = blockIdx.y;
  const int row_lo = offsets[e];
  const int rows = offsets[e + 1] - row_lo;
  if (rows <= 0) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, kq = lane & 3;
  const int col0 = blockIdx.x * 32 + 4 * g;
  const bool col_ok = col0 < N;

  const int steps_total = Kd / 32;
  const int spw = (steps_total + W4_WARPS - 1) / W4_WARPS;
  const int s_lo = warp * spw;
  const int s_hi = min(s_lo + spw, steps_total);
  const int steps_per_group = group / 32;
  const int G = Kd / group;

  const int we = e % period;            // weight set of this group
  const size_t qw_e = (size_t)we * (Kd / 8) * N;
  const size_t sc_e = (size_t)we * G * N;
  const size_t qz_e = (size_t)we * G * (N / 8);
  const W4Proj proj[2] = {p0, p1};

  for (int r0 = 0; r0 < rows; r0 += 8 * W4_NB) {
    W4Acc acc[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) acc_init(acc[p]);

    const __nv_bfloat16* xrow[W4_NB];
    bool row_ok[W4_NB];
#pragma unroll
    for (int tb = 0; tb < W4_NB; ++tb) {
      int r = r0 + 8 * tb + g;
      row_ok[tb] = r < rows;
      xrow[tb] = x + (size_t)(row_lo + (row_ok[tb] ? r : 0)) * Kd;
    }

    // one commit group per k-step, empty when there is nothing left to fetch, so that
    // "all but the newest DEPTH-1 groups are complete" always means "this step has landed"
    auto issue = [&](int s) {
      if (s < s_hi) {
        uint4(*slot)[32] = ring[warp][(s - s_lo) % W4_DEPTH];
        if (col_ok) {
#pragma unroll
          for (int p = 0; p < NP; ++p)
            cp_async16(&slot[p][lane], proj[p].qw + qw_e + (size_t)(4 * s + kq) * N + col0);
        }
#pragma unroll
        for (int tb = 0; tb < W4_NB; ++tb)
          if (row_ok[tb]) cp_async16(&slot[NP + tb][lane], xrow[tb] + 32 * s + 8 * kq);
      }
      cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < W4_DEPTH; ++i) issue(s_lo + i);

    int cur_group = -1;
    for (int s = s_lo; s < s_hi; ++s) {
      cp_async_wait<W4_DEPTH - 1>();
      uint4(*slot)[32] = ring[warp][(s - s_lo) % W4_DEPTH];
      uint4 wcur[NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) wcur[p] = col_ok ? slot[p][lane] : make_uint4(0, 0, 0, 0);
      // activations: 8 consecutive k of row g (per row block), permuted to the nibble-pair order
      uint32_t bfrag[W4_NB][4];
#pragma unroll
      for (int tb = 0; tb < W4_NB; ++tb) {
        const uint4 xv = row_ok[tb] ? slot[NP + tb][lane] : make_uint4(0, 0, 0, 0);
        bfrag[tb][0] = prmt(xv.x, xv.z, 0x5410);  // {x0, x4}
        bfrag[tb][1] = prmt(xv.x, xv.z, 0x7632);  // {x1, x5}
        bfrag[tb][2] = prmt(xv.y, xv.w, 0x5410);  // {x2, x6}
        bfrag[tb][3] = prmt(xv.y, xv.w, 0x7632);  // {x3, x7}
      }
      issue(s + W4_DEPTH);               // refill the slot just read
      const int gi = s / steps_per_group;
      if (gi != cur_group) {
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          acc_flush(acc[p]);
          if (col_ok) load_group(acc[p], proj[p], sc_e + (size_t)gi * N, qz_e + (size_t)gi * (N / 8), col0);
        }
        cur_group = gi;
      }
#pragma unroll
      for (int p = 0; p < NP; ++p) step_mma(acc[p], wcur[p], bfrag);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int p = 0; p < NP; ++p) acc_flush(acc[p]);

    // fixed-order reduction over the K split
#pragma unroll
    for (int p = 0; p < NP; ++p)
#pragma unroll
      for (int tb = 0; tb < W4_NB; ++tb)
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int i = 0; i < 4; ++i) red[warp][p][tb * 8 + m * 4 + i][lane] = acc[p].master[tb][m][i];
    __syncthreads();
    if (warp == 0 && col_ok) {
#pragma unroll
      for (int tb = 0; tb < W4_NB; ++tb)
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int half = 0; half < 2; ++half) {   // half selects the row 2kq + half
            float v[NP][2];
#pragma unroll
            for (int p = 0; p < NP; ++p)
#pragma unroll
              for (int cc = 0; cc < 2; ++cc) {     // the two columns of this mma
                const int idx = tb * 8 + m * 4 + cc * 2 + half;
                float sum = red[0][p][idx][lane];
#pragma unroll
                for (int w = 1; w < W4_WARPS; ++w) sum += red[w][p][idx][lane];
                v[p][cc] = sum;
              }
            const int r = r0 + 8 * tb + 2 * kq + half;
            if (r < rows) {
              float o0, o1;
              if (SWIGLU) {
                o0 = swiglu_rounded<__nv_bfloat16>(v[0][0], v[NP - 1][0]);
                o1 = swiglu_rounded<__nv_bfloat16>(v[0][1], v[NP - 1][1]);
              } else {
                o0 = v[0][0]; o1 = v[0][1];
              }
              __nv_bfloat162 o = __floats2bfloat162_rn(o0, o1);
              *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(row_lo + r) * N + col0 + 2 * m) = o;
            }
          }
    }
    __syncthreads();
  }
}

int launch_w4(const void* x, W4Proj p0, W4Proj p1, bool swiglu, const int32_t* offsets, int64_t S, int64_t E,
              int64_t period, int64_t N, int64_t Kd, int64_t group, void* out, cudaStream_t st) {
  if (S < 0 || E <= 0 || N <= 0 || Kd <= 0 || group <= 0) return MQ_ERR_INVALID_ARGUMENT;
  if (period <= 0 || period > E) return MQ_ERR_INVALID_ARGUMENT;
  if (group % 32 != 0 || Kd % group != 0 || N % 8 != 0 || E > 65535) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!x || !p0.qw || !p0.sc || !p0.qz || !offsets || !out) return MQ_ERR_INVALID_ARGUMENT;
  if (swiglu && (!p1.qw || !p1.sc || !p1.qz)) return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(x) || !aligned16(p0.qw) || !aligned16(p0.sc) || !aligned16(out)) return MQ_ERR_INVALID_ARGUMENT;
  if (swiglu && (!aligned16(p1.qw) || !aligned16(p1.sc))) return MQ_ERR_INVALID_ARGUMENT;
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)E);
  const int ring_bytes = W4_WARPS * W4_DEPTH * ((swiglu ? 2 : 1) + W4_NB) * 32 * 16;
  if (swiglu) {
    cudaFuncSetAttribute(w4a16_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes);
    w4a16_grouped_kernel<true><<<grid, W4_WARPS * 32, ring_bytes, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), p0, p1,
        offsets, (int)period, (int)N, (int)Kd, (int)group, reinterpret_cast<__nv_bfloat16*>(out));
  } else {
    cudaFuncSetAttribute(w4a16_grouped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ring_bytes);
    w4a16_grouped_kernel<false><<<grid, W4_WARPS * 32, ring_bytes, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), p0, p0,
        offsets, (int)period, (int)N, (int)Kd, (int)group, reinterpret_cast<__nv_bfloat16*>(out));
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
