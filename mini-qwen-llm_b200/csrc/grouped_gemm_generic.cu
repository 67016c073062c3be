// Generic grouped GEMM (any dtype, any shape): out[s:t] = a[s:t] . w[e]^T with fp32 FMA
// accumulation, optionally two projections fused with SwiGLU.
// Follows mini_qwen/kernels/moe_grouped_gemm.py:17-37 and mini_qwen/model/layers/moe.py:24-25.
//
// This is the shape-agnostic kernel: fp32 layers, 16-bit layers whose sizes the tcgen05 kernel
// does not cover.  Tiles of 64x64 outputs; the (expert, row-tile) of a CTA is found on the device
// from the offsets, so no host synchronisation is needed.
#include "common.cuh"

namespace mq {
namespace {

constexpr int G_TM = 64, G_TN = 64, G_KC = 16, G_THREADS = 256, G_PITCH = 68;

template <typename T>
__device__ __forceinline__ void load4(const T* p, size_t base, int64_t k, int64_t Kd, bool vec_ok, float (&v)[4]) {
  if (vec_ok && k + 4 <= Kd) {
    if (sizeof(T) == 4) {
      float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + base + k);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p) + base + k);
      const T* h = reinterpret_cast<const T*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = to_float<T>(h[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (k + j < Kd) ? to_float<T>(p[base + k + j]) : 0.0f;
  }
}

// Finds the expert and row-tile of linear tile index `tile`; false when past the last tile.
__device__ bool locate_tile(const int32_t* offsets, int E, int tile, int tm, int* s_out /* shared [3] */) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int base = 0;
    int found_e = -1, found_mt = 0;
    for (int e0 = 0; e0 < E && found_e < 0; e0 += 32) {
      int e = e0 + lane;
      int n = (e < E) ? offsets[e + 1] - offsets[e] : 0;
      int tiles = (n + tm - 1) / tm;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int lo = base + incl - tiles, hi = base + incl;
      unsigned hit = __ballot_sync(0xffffffffu, tile >= lo && tile < hi);
      if (hit) {
        int src = __ffs(hit) - 1;
        found_e = __shfl_sync(0xffffffffu, e, src);
        found_mt = tile - __shfl_sync(0xffffffffu, lo, src);
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) { s_out[0] = found_e; s_out[1] = found_mt; }
  }
  __syncthreads();
  return s_out[0] >= 0;
}

template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(G_THREADS)
grouped_gemm_generic(const T* __restrict__ a, const T* __restrict__ w, const int32_t* __restrict__ offsets,
                     int E, int period, int64_t N, int64_t Kd, int vec_ok, T* __restrict__ out) {
  // w is [E, N, Kd]; with SWIGLU it is [E, 2N, Kd] (gate rows, then up rows) and out is [S, N].
  __shared__ __align__(16) float As[G_KC][G_PITCH];
  __shared__ __align__(16) float Bs[SWIGLU ? 2 : 1][G_KC][G_PITCH];
  __shared__ int loc[3];
  if (!locate_tile(offsets, E, blockIdx.x, G_TM, loc)) return;
  const int e = loc[0];
  const int64_t row_lo = offsets[e] + (int64_t)loc[1] * G_TM;
  const int64_t row_hi = offsets[e + 1];
  const int64_t n0 = (int64_t)blockIdx.y * G_TN;

  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) * 4;   // loader: row/col lr of the tile, 4 k values

  const bool a_in = row_lo + lr < row_hi;
  const bool b_in = n0 + lr < N;
  const size_t a_base = (size_t)(row_lo + lr) * Kd;
  const int64_t w_rows = SWIGLU ? 2 * N : N;
  const size_t b_base = ((size_t)(e % period) * w_rows + n0 + lr) * Kd;
  const size_t b2_base = b_base + (size_t)N * Kd;

  float acc[SWIGLU ? 2 : 1][4][4];
#pragma unroll
  for (int p = 0; p < (SWIGLU ? 2 : 1); ++p)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[p][i][j] = 0.0f;

  for (int64_t k0 = 0; k0 < Kd; k0 += G_KC) {
    float va[4] = {0, 0, 0, 0}, vb[4] = {0, 0, 0, 0}, vb2[4] = {0, 0, 0, 0};
    if (a_in) load4<T>(a, a_base, k0 + lk, Kd, vec_ok, va);
    if (b_in) {
      load4<T>(w, b_base, k0 + lk, Kd, vec_ok, vb);
      if (SWIGLU) load4<T>(w, b2_base, k0 + lk, Kd, vec_ok, vb2);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      As[lk + j][lr] = va[j];
      Bs[0][lk + j][lr] = vb[j];
      if (SWIGLU) Bs[1][lk + j][lr] = vb2[j];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < G_KC; ++k) {
      float4 av = *reinterpret_cast<const float4*>(&As[k][4 * ty]);
      const float aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int p = 0; p < (SWIGLU ? 2 : 1); ++p) {
        float4 bv = *reinterpret_cast<const float4*>(&Bs[p][k][4 * tx]);
        const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[p][i][j] = fmaf(aa[i], bb[j], acc[p][i][j]);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row_lo + 4 * ty + i;
    if (r >= row_hi) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + 4 * tx + j;
      if (n >= N) continue;
      float v = SWIGLU ? swiglu_rounded<T>(acc[0][i][j], acc[SWIGLU ? 1 : 0][i][j]) : acc[0][i][j];
      out[r * N + n] = from_float<T>(v);
    }
  }
}

template <typename T>
int launch_generic(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E, int64_t period,
                   int64_t N, int64_t Kd, bool swiglu, void* out, cudaStream_t st) {
  const int64_t tiles = (S + G_TM - 1) / G_TM + E;
  dim3 grid((unsigned)tiles, (unsigned)((N + G_TN - 1) / G_TN));
  const int vec_ok = (Kd % 4 == 0) && aligned16(a) && aligned16(w);
  if (swiglu)
    grouped_gemm_generic<T, true><<<grid, G_THREADS, 0, st>>>(reinterpret_cast<const T*>(a),
        reinterpret_cast<const T*>(w), offsets, (int)E, (int)period, N, Kd, vec_ok, reinterpret_cast<T*>(out));
  else
    grouped_gemm_generic<T, false><<<grid, G_THREADS, 0, st>>>(reinterpret_cast<const T*>(a),
        reinterpret_cast<const T*>(w), offsets, (int)E, (int)period, N, Kd, vec_ok, reinterpret_cast<T*>(out));
  return check_launch();
}

}  // namespace

int grouped_gemm_generic_dispatch(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E,
                                  int64_t period, int64_t N, int64_t Kd, int dtype, bool swiglu, void* out,
                                  cudaStream_t st) {
  if (dtype == MQ_F32) return launch_generic<float>(a, w, offsets, S, E, period, N, Kd, swiglu, out, st);
  if (dtype == MQ_BF16) return launch_generic<__nv_bfloat16>(a, w, offsets, S, E, period, N, Kd, swiglu, out, st);
  return launch_generic<__half>(a, w, offsets, S, E, period, N, Kd, swiglu, out, st);
}

}  // namespace mq
