// Top-k router: fp32 logits -> fp32 softmax -> K largest scores (ties: lower expert id).
// Follows mini_qwen/kernels/moe_router.py:19-22 and the renormalisation of
// mini_qwen/model/layers/moe.py:55-56.
//
// Two launches: a logits kernel (x . w^T in fp32 FMA; products of 16-bit inputs are exact in
// fp32, so the only rounding is the running sum) into a [T,E] fp32 workspace, then one warp per
// token for softmax + selection.  Tensor cores are deliberately not used for the logits: expert
// ids must equal those of an fp32 reference, and the adjacent-score gaps are a few fp32 ulp.
#include <mutex>

#include "common.cuh"
#include "w4_prep.cuh"
#include "route_helpers.cuh"

namespace mq {
namespace {

// ---------------------------------------------------------------------------------------------
// 8 consecutive elements starting at element index i (i % 8 == 0, base 16-byte aligned), as fp32.
__device__ __forceinline__ void load8(const void* p, int dt, size_t i, float (&v)[8]) {
  if (dt == MQ_F32) {
    const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    float4 a = __ldg(q), b = __ldg(q + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 r = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p) + i));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (dt == MQ_BF16) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
      } else {
        __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
        float2 f = __half22float2(h);
        v[2 * j] = f.x; v[2 * j + 1] = f.y;
      }
    }
  }
}

// 8 packed 16-bit values -> fp32.
__device__ __forceinline__ void unpack8_16bit(const uint4& r, bool bf16, float (&v)[8]) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (bf16) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      v[2 * j] = f.x; v[2 * j + 1] = f.y;
    }
  }
}

// 8 elements with bounds and alignment handled element by element (any H).
__device__ __forceinline__ void load8_safe(const void* p, int dt, size_t row_base, int64_t k, int64_t H,
                                           bool vec_ok, float (&v)[8]) {
  if (vec_ok && k + 8 <= H) {
    load8(p, dt, row_base + k, v);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (k + j < H) ? load_as_float(p, dt, row_base + k + j) : 0.0f;
  }
}

// ---------------------------------------------------------------------------------------------
// Tiled logits: CTA = 32 tokens x 128 experts x one K slice, 128 threads, each thread 4 tokens x 8
// experts.  The K dimension is split over blockIdx.z so that small batches still fill the GPU; the
// slices are summed in a fixed order by the selection kernel, so results do not depend on timing.
constexpr int R_TM = 32, R_TE = 128, R_KC = 32, R_THREADS = 128;

__global__ void __launch_bounds__(R_THREADS)
router_logits_tiled(const void* __restrict__ x, int xdt, const void* __restrict__ w, int wdt,
                    int64_t T, int64_t H, int64_t E, int64_t k_per_slice, int vec_ok,
                    float* __restrict__ logits /* [slices, T, E] */) {
  __shared__ __align__(16) float xs[R_KC][R_TM];
  __shared__ __align__(16) float ws[R_KC][R_TE];

  const int tid = threadIdx.x;
  const int64_t t0 = (int64_t)blockIdx.x * R_TM;
  const int64_t e0 = (int64_t)blockIdx.y * R_TE;
  const int64_t k_lo = (int64_t)blockIdx.z * k_per_slice;
  const int64_t k_hi = min(k_lo + k_per_slice, H);
  const int tg = tid >> 4, eg = tid & 15;

  // loader roles: x tile: token tid%32, k part tid/32 (8 wide); w tile: expert tid, all 32 k
  const int lx_tok = tid & 31, lx_k = (tid >> 5) * 8;
  const bool x_in = t0 + lx_tok < T;
  const bool w_in = e0 + tid < E;
  const size_t x_row = (size_t)(t0 + lx_tok) * H;
  const size_t w_row = (size_t)(e0 + tid) * H;

  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  float px[8], pw[4][8];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int j = 0; j < 8; ++j) px[j] = 0.0f;
    if (x_in && k0 + lx_k < k_hi) load8_safe(x, xdt, x_row, k0 + lx_k, k_hi, vec_ok, px);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int j = 0; j < 8; ++j) pw[q][j] = 0.0f;
      if (w_in && k0 + 8 * q < k_hi) load8_safe(w, wdt, w_row, k0 + 8 * q, k_hi, vec_ok, pw[q]);
    }
  };

  fetch(k_lo);
  for (int64_t k0 = k_lo; k0 < k_hi; k0 += R_KC) {
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[lx_k + j][lx_tok] = px[j];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int j = 0; j < 8; ++j) ws[8 * q + j][tid] = pw[q][j];
    __syncthreads();
    if (k0 + R_KC < k_hi) fetch(k0 + R_KC);
#pragma unroll
    for (int k = 0; k < R_KC; ++k) {
      const float4 xv = *reinterpret_cast<const float4*>(&xs[k][4 * tg]);
      const float4 wa = *reinterpret_cast<const float4*>(&ws[k][4 * eg]);
      const float4 wb = *reinterpret_cast<const float4*>(&ws[k][64 + 4 * eg]);
      const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
      const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(xa[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }

  float* dst = logits + (size_t)blockIdx.z * T * E;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t t = t0 + 4 * tg + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t e = e0 + (j < 4 ? 4 * eg + j : 64 + 4 * eg + (j - 4));
      if (e < E) dst[t * E + e] = acc[i][j];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core logits for 16-bit inputs of one type (bf16 x bf16 or fp16 x fp16), T > 64.
// CTA = 32 tokens x 128 experts x one K slice; 8 warps, each 16 tokens x 32 experts of
// mma.sync.m16n8k16 with fp32 accumulators.  Products of 16-bit inputs are exact in the tensor core;
// to keep the accumulation as accurate as an fp32 FMA chain, a tensor-core accumulator only ever
// sums 128 k (8 MMAs) and is then added to a master accumulator with an ordinary fp32 add.
// Fragments are fetched with 16-byte loads: the order of k inside a 32-wide block is free as long
// as both operands use the same one, so lane (g, kq) takes k = 8*kq .. 8*kq+7 of its row and feeds
// {0,1 | 2,3} to the first MMA and {4,5 | 6,7} to the second.
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, bool bf16) {
  if (bf16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int RM_TM = 32, RM_TE = 128, RM_THREADS = 256;
constexpr int RM_BK = 64;                       // k per pipeline stage: 128-byte rows in shared memory
constexpr int RM_STAGES = 3;                    // 60 KB per CTA: three CTAs per SM
constexpr int RM_ROWS = RM_TM + RM_TE;          // token rows, then expert rows
constexpr int RM_STAGE_BYTES = RM_ROWS * RM_BK * 2;   // 20 KB
constexpr int RM_SMEM_BYTES = RM_STAGES * RM_STAGE_BYTES;

__device__ __forceinline__ void rm_cp_async16(uint32_t dst, const void* src, bool ok) {
  const int n = ok ? 16 : 0;                    // 0 bytes read: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// The operands travel global -> shared memory in 64-k stages by cp.async (3 stages per CTA, three CTAs per SM),
// 16-byte pieces XOR-swizzled by row so that the fragment loads are conflict-free.  The arithmetic is
// the one described above, in the same order for every token, whatever the staging.
__global__ void __launch_bounds__(RM_THREADS)
router_logits_mma(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, int is_bf16,
                  int64_t T, int64_t H, int64_t E, int64_t k_per_slice, float* __restrict__ logits) {
  extern __shared__ __align__(128) uint8_t rm_smem[];
  const uint32_t smem0 = (uint32_t)__cvta_generic_to_shared(rm_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, kq = lane & 3;
  const int wm = warp & 1, wn = warp >> 1;
  const int64_t tb = (int64_t)blockIdx.x * RM_TM;           // first token of the CTA
  const int64_t eb = (int64_t)blockIdx.y * RM_TE;           // first expert of the CTA
  const int64_t k_lo = (int64_t)blockIdx.z * k_per_slice;
  const int64_t k_hi = min(k_lo + k_per_slice, H);
  const bool bf = is_bf16 != 0;
  const int nstage = k_lo < k_hi ? (int)((k_hi - k_lo + RM_BK - 1) / RM_BK) : 0;

  // loader: 160 rows x 8 pieces of 16 bytes per stage = 1280 pieces, 5 per thread
  auto load_stage = [&](int st) {
    const int64_t k0 = k_lo + (int64_t)st * RM_BK;
    const uint32_t base = smem0 + (uint32_t)(st % RM_STAGES) * RM_STAGE_BYTES;
#pragma unroll
    for (int i = 0; i < (RM_ROWS * 8) / RM_THREADS; ++i) {
      const int piece = threadIdx.x + i * RM_THREADS;
      const int row = piece >> 3, c = piece & 7;
      const int64_t k = k0 + 8 * c;
      const bool is_tok = row < RM_TM;
      const int64_t r = is_tok ? tb + row : eb + (row - RM_TM);
      const bool ok = (is_tok ? r < T : r < E) && k < k_hi;   // H % 32 == 0 and slices are multiples of 128
      const uint16_t* src = (is_tok ? x : w) + (size_t)(ok ? r : 0) * H + (ok ? k : 0);
      rm_cp_async16(base + (uint32_t)row * 128u + (uint32_t)((c ^ (row & 7)) << 4), src, ok);
    }
  };

  float master[4][4], part[4][4];
#pragma unroll
  for (int n = 0; n < 4; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) { master[n][i] = 0.0f; part[n][i] = 0.0f; }

#pragma unroll
  for (int st = 0; st < RM_STAGES - 1; ++st) {
    if (st < nstage) load_stage(st);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  const int row_a = 16 * wm + g, row_b = row_a + 8;         // token rows of this lane's fragments
  int in_chunk = 0;
  for (int st = 0; st < nstage; ++st) {
    asm volatile("cp.async.wait_group %0;" ::"n"(RM_STAGES - 2) : "memory");
    __syncthreads();                                        // stage st has landed; stage st-1 is free
    if (st + RM_STAGES - 1 < nstage) load_stage(st + RM_STAGES - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint8_t* base = rm_smem + (st % RM_STAGES) * RM_STAGE_BYTES;
    const int64_t k0 = k_lo + (int64_t)st * RM_BK;
#pragma unroll
    for (int h = 0; h < 2; ++h) {                           // two 32-k blocks per stage
      if (k0 + 32 * h < k_hi) {
        const int c = 4 * h + kq;
        const uint4 va = *reinterpret_cast<const uint4*>(base + row_a * 128 + ((c ^ (row_a & 7)) << 4));
        const uint4 vb = *reinterpret_cast<const uint4*>(base + row_b * 128 + ((c ^ (row_b & 7)) << 4));
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int row_w = RM_TM + 32 * wn + 8 * n + g;
          const uint4 vw = *reinterpret_cast<const uint4*>(base + row_w * 128 + ((c ^ (row_w & 7)) << 4));
          mma16816(part[n], va.x, vb.x, va.y, vb.y, vw.x, vw.y, bf);
          mma16816(part[n], va.z, vb.z, va.w, vb.w, vw.z, vw.w, bf);
        }
        if (++in_chunk == 4) {          // 128 k summed in the tensor core: fold into the fp32 master
          in_chunk = 0;
#pragma unroll
          for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) { master[n][i] += part[n][i]; part[n][i] = 0.0f; }
        }
      }
    }
  }
#pragma unroll
  for (int n = 0; n < 4; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) master[n][i] += part[n][i];

  const int64_t ra = tb + row_a, rb = tb + row_b;
  const bool ra_ok = ra < T, rb_ok = rb < T;
  const int64_t e0 = eb + 32 * wn;
  float* dst = logits + (size_t)blockIdx.z * T * E;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int64_t e = e0 + 8 * n + 2 * kq;
    if (ra_ok) {
      if (e < E) dst[ra * E + e] = master[n][0];
      if (e + 1 < E) dst[ra * E + e + 1] = master[n][1];
    }
    if (rb_ok) {
      if (e < E) dst[rb * E + e] = master[n][2];
      if (e + 1 < E) dst[rb * E + e + 1] = master[n][3];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Skinny logits (few tokens): one CTA per expert, each warp takes blocks of 8 tokens; the lanes
// split H, partial sums meet in a shuffle tree.
__global__ void __launch_bounds__(128)
router_logits_skinny(const void* __restrict__ x, int xdt, const void* __restrict__ w, int wdt,
                     int64_t T, int64_t H, int64_t E, int vec_ok, float* __restrict__ logits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t e = blockIdx.x;
  const size_t w_row = (size_t)e * H;
  const bool fast = vec_ok && xdt != MQ_F32 && wdt != MQ_F32;     // 16-bit operands, 16-byte pieces
  for (int64_t tb = (int64_t)warp * 8; tb < T; tb += 4 * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    if (fast) {
      const uint16_t* wp = reinterpret_cast<const uint16_t*>(w) + w_row;
      const uint16_t* xp = reinterpret_cast<const uint16_t*>(x);
      for (int64_t k = (int64_t)lane * 8; k < H; k += 32 * 8) {
        // all nine loads of the iteration are issued before the first use
        const uint4 wr = __ldg(reinterpret_cast<const uint4*>(wp + k));
        uint4 xr[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          xr[i] = tb + i < T ? __ldg(reinterpret_cast<const uint4*>(xp + (size_t)(tb + i) * H + k)) : make_uint4(0, 0, 0, 0);
        float wv[8];
        unpack8_16bit(wr, wdt == MQ_BF16, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float xv[8];
          unpack8_16bit(xr[i], xdt == MQ_BF16, xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
        }
      }
    } else {
      for (int64_t k = (int64_t)lane * 8; k < H; k += 32 * 8) {
        float wv[8];
        load8_safe(w, wdt, w_row, k, H, vec_ok, wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (tb + i < T) {
            float xv[8];
            load8_safe(x, xdt, (size_t)(tb + i) * H, k, H, vec_ok, xv);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = acc[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && tb + i < T) logits[(tb + i) * E + e] = v;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// One warp per token: softmax over E logits, then K rounds of warp arg-max on (score, -id).
template <int EPL>
__global__ void __launch_bounds__(128)
router_softmax_topk(const float* __restrict__ logits, int slices, const float* __restrict__ bias,
                    int64_t T, int E, int K, int renorm,
                    int64_t* __restrict__ ids64, int32_t* __restrict__ ids32, float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= T) return;
  softmax_topk_row<EPL>(logits + (size_t)t * E, slices, (size_t)T * E, bias, E, K, renorm, lane,
                        ids64 ? ids64 + t * K : nullptr, ids32 ? ids32 + t * K : nullptr, weights + t * K);
}

// ---------------------------------------------------------------------------------------------
// Small batches (decode): logits, softmax + top-k, the permute plan and the preparation of the activations
// for the W4A16 kernels in ONE launch.  At these sizes each of the four kernels runs for a few microseconds
// and the layer call is bound by the chain of launches, not by any of them.
//   phase A, every CTA: CTA e forms the logits of expert e for all tokens (fp32 FMA chains over 8-element
//     pieces, one piece per thread and pass, shuffle tree, then the warps' sums in warp order), and CTA
//     t < T also writes token t's row in the k order the W4A16 kernels want, with its group sums;
//   phase B, the CTA that finishes last (a counter in the workspace tells it; nobody waits): softmax and
//     top-k of every token (one warp per token, softmax_topk_row), then the stable counting sort of the
//     T*K slots by expert.  It leaves the counter at zero for the next call.
constexpr int RSM_THREADS = 512;
constexpr int RSM_MAX_T = 64, RSM_MAX_E = 256, RSM_MAX_S = 2048;

// The plan of a small batch (a stable counting sort of the T*K slots by expert), by all threads of one CTA.  A
// token's K experts are distinct and the slots are token-major, so the rank of slot (t, k) inside its expert is
// the number of earlier TOKENS that chose the expert: with T <= 64 one 64-bit mask per expert holds everything,
// and no step is serial.  s_ids [T*K] holds the ids; s_mask [E] must be zero on entry; s_run [E] is scratch.
__device__ void route_plan_small(const int* s_ids, unsigned long long* s_mask, int* s_run, int T, int E, int K,
                                 int32_t* __restrict__ ids32, int32_t* __restrict__ perm, int32_t* __restrict__ inv,
                                 int32_t* __restrict__ off32, int64_t* __restrict__ off64) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const int S = T * K;
  for (int i = tid; i < S; i += nthreads) {
    const int ee = s_ids[i];
    if (ids32 != nullptr) ids32[i] = ee;
    atomicOr(&s_mask[ee], 1ull << (i / K));
  }
  __syncthreads();
  if (warp == 0) {
    // exclusive scan of the E counts: each lane takes E/32 (at most 8) consecutive experts
    const int per = (E + 31) / 32;
    int cnt[RSM_MAX_E / 32];
    int sum = 0;
#pragma unroll
    for (int j = 0; j < RSM_MAX_E / 32; ++j) {
      const int ee = lane * per + j;
      cnt[j] = (j < per && ee < E) ? __popcll(s_mask[ee]) : 0;
      sum += cnt[j];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    int run = incl - sum;
#pragma unroll
    for (int j = 0; j < RSM_MAX_E / 32; ++j) {
      const int ee = lane * per + j;
      if (j < per && ee < E) {
        s_run[ee] = run;
        if (off64) off64[ee] = run;
        if (off32) off32[ee] = run;
      }
      run += cnt[j];
    }
    if (lane == 31) {
      if (off64) off64[E] = incl;
      if (off32) off32[E] = incl;
    }
  }
  __syncthreads();
  for (int i = tid; i < S; i += nthreads) {
    const int ee = s_ids[i];
    const int t = i / K;
    const int pos = s_run[ee] + __popcll(s_mask[ee] & ((1ull << t) - 1ull));
    perm[pos] = i;
    inv[i] = pos;
  }
}

// The activation preparation of one token row (w4_prep.cuh) by all threads of a CTA; s_red: a float per warp.
__device__ void route_prepare_row(const __nv_bfloat16* __restrict__ x_row, int H, int prep_mode,
                                  __nv_bfloat16* __restrict__ xp_row, float* __restrict__ xs_row, float* s_red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const uint4* in = reinterpret_cast<const uint4*>(x_row);
  uint4* o = reinterpret_cast<uint4*>(xp_row);
  const bool f16 = prep_mode == 2;
  float scale = 1.0f;
  if (f16) {
    float amax = 0.0f;
    for (int c = tid; c < H / 8; c += nthreads) amax = fmaxf(amax, w4_piece_amax(in[c]));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    __syncthreads();
    if (lane == 0) s_red[warp] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int wi = 0; wi < nthreads / 32; ++wi) amax = fmaxf(amax, s_red[wi]);
    const int ex = w4_row_exponent(amax);
    scale = w4_pow2(ex);
    if (tid == 0) xs_row[W4_XS_UNSCALE] = w4_pow2(-ex);
  }
  for (int c0 = warp * 32; c0 < H / 8; c0 += nthreads) {
    const int c = c0 + lane;
    float sum = 0.0f;
    if (c < H / 8) o[c] = w4_prepare_piece(in[c], true, f16, scale, sum);
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if ((lane & 15) == 0 && c < H / 8) xs_row[c >> 4] = sum;
  }
}

// ---- the same for batches of more than 16 tokens, laid out by TOKEN: CTA (eg, t) forms the logits of experts
// [32 eg, 32 eg + 32) for token t (a warp takes four experts; a lane keeps its pieces of the token's row in
// registers; all loads of a lane are independent: one round trip), the CTA that arrives last on token t's counter
// does that token's softmax and top-k (one warp), and the CTA that finishes the last token makes the plan.  The
// selection of the tokens thus runs on as many SMs as there are tokens instead of on one.  16-bit x and w only.
constexpr int RTK_THREADS = 256;
constexpr int RTK_HEADER_INTS = 128;                  // workspace header: counter of the narrow kernel, all-tokens
                                                      // counter, one counter per token (64)
template <int EPL>
__global__ void __launch_bounds__(RTK_THREADS)
route_tokens_kernel(const uint16_t* __restrict__ x, int x_bf16, const uint16_t* __restrict__ w, int w_bf16,
                    const float* __restrict__ bias, int T, int H, int E, int K, int renorm,
                    float* __restrict__ logits, int* __restrict__ header,
                    int32_t* __restrict__ ids32, int64_t* __restrict__ ids64, float* __restrict__ weights,
                    int32_t* __restrict__ perm, int32_t* __restrict__ inv, int32_t* __restrict__ off32,
                    int64_t* __restrict__ off64, __nv_bfloat16* __restrict__ xp, float* __restrict__ xs,
                    int prep_mode) {
  extern __shared__ __align__(16) uint8_t rtk_smem[];
  __shared__ int s_last;
  __shared__ float s_red[RTK_THREADS / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int eg = blockIdx.x, t = blockIdx.y, groups = gridDim.x;
  int* all_ctr = header + 1;
  int* tok_ctr = header + 2;
  pdl_wait();
  pdl_release();

  // ---- logits: warp `warp` takes experts e0 .. e0+3; a lane's pieces of the row: k = 8 (lane + 32 i)
  {
    constexpr int MAXP = 8;                            // pieces per lane kept in registers (H <= 2048); more: re-read
    const int pieces = H / 8;
    const uint16_t* xr = x + (size_t)t * H;
    const int e0 = eg * 32 + warp * 4;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int p0 = 0; p0 < pieces; p0 += 32 * MAXP) {
      uint4 xv[MAXP];
#pragma unroll
      for (int i = 0; i < MAXP; ++i) {
        const int pc = p0 + lane + 32 * i;
        xv[i] = pc < pieces ? __ldg(reinterpret_cast<const uint4*>(xr) + pc) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = e0 + j;
        if (e < E) {
          const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)e * H);
          uint4 wv[MAXP];
#pragma unroll
          for (int i = 0; i < MAXP; ++i) {
            const int pc = p0 + lane + 32 * i;
            wv[i] = pc < pieces ? __ldg(wr + pc) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int i = 0; i < MAXP; ++i) {
            float a[8], b[8];
            unpack8_16bit(xv[i], x_bf16 != 0, a);
            unpack8_16bit(wv[i], w_bf16 != 0, b);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[j] = fmaf(a[q], b[q], acc[j]);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v = acc[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && e0 + j < E) logits[(size_t)t * E + e0 + j] = v;
    }
  }
  if (xp != nullptr && eg == 0)
    route_prepare_row(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)t * H, H, prep_mode, xp + (size_t)t * H,
                      xs + (size_t)t * W4_XS_STRIDE, s_red);

  // ---- last on this token?
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&tok_ctr[t], 1) == groups - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(rtk_smem);   // [E]
  float* s_logits = reinterpret_cast<float*>(s_mask + E);                        // [E]
  int* s_ids = reinterpret_cast<int*>(s_logits + E);                             // [T * K]
  int* s_run = s_ids + T * K;                                                    // [E]
  for (int i = tid; i < E; i += RTK_THREADS) s_logits[i] = __ldcg(logits + (size_t)t * E + i);
  __syncthreads();
  if (warp == 0)
    softmax_topk_row<EPL>(s_logits, 1, 0, bias, E, K, renorm, lane, ids64 ? ids64 + (size_t)t * K : nullptr,
                          ids32 + (size_t)t * K, weights + (size_t)t * K);
  // ---- last of the tokens?
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(all_ctr, 1) == T - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int ee = tid; ee < E; ee += RTK_THREADS) s_mask[ee] = 0ull;
  for (int i = tid; i < T * K; i += RTK_THREADS) s_ids[i] = __ldcg(ids32 + i);
  __syncthreads();
  route_plan_small(s_ids, s_mask, s_run, T, E, K, nullptr, perm, inv, off32, off64);
  for (int i = tid; i < T + 1; i += RTK_THREADS) header[1 + i] = 0;              // ready for the next call
}

template <int EPL>
__global__ void __launch_bounds__(RSM_THREADS)
route_small_kernel(const void* __restrict__ x, int xdt, const void* __restrict__ w, int wdt,
                   const float* __restrict__ bias, int T, int H, int E, int K, int renorm, int vec_ok,
                   float* __restrict__ logits, int* __restrict__ counter,
                   int32_t* __restrict__ ids32, int64_t* __restrict__ ids64, float* __restrict__ weights,
                   int32_t* __restrict__ perm, int32_t* __restrict__ inv, int32_t* __restrict__ off32,
                   int64_t* __restrict__ off64, __nv_bfloat16* __restrict__ xp, float* __restrict__ xs,
                   int prep_mode) {
  extern __shared__ __align__(16) uint8_t rsm_smem[];
  __shared__ int s_last;
  __shared__ float s_part[8][RSM_MAX_T];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = blockIdx.x;
  pdl_wait();                       // x may come from the kernel before this one
  pdl_release();

  // ---- phase A: logits of expert e.  The K dimension is spread over 256 threads (one 8-element piece each per
  // pass, so the loads of a thread are independent of one another: one round trip to L2), the tokens over the two
  // halves of the CTA in chunks of 8.  A warp reduces its partial sums with shuffles; the eight warps of a half
  // meet in shared memory and are added in warp order.
  {
    const size_t w_row = (size_t)e * H;
    const bool fast = vec_ok && xdt != MQ_F32 && wdt != MQ_F32;     // 16-bit operands, 16-byte pieces
    const int kt = tid & 255, half = tid >> 8, kwarp = kt >> 5;
    for (int tb = half * 8; tb < T; tb += 16) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      if (fast) {
        const uint16_t* wp = reinterpret_cast<const uint16_t*>(w) + w_row;
        const uint16_t* xq = reinterpret_cast<const uint16_t*>(x);
        for (int k = kt * 8; k < H; k += 256 * 8) {
          const uint4 wr = __ldg(reinterpret_cast<const uint4*>(wp + k));
          uint4 xr[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            xr[i] = tb + i < T ? __ldg(reinterpret_cast<const uint4*>(xq + (size_t)(tb + i) * H + k)) : make_uint4(0, 0, 0, 0);
          float wv[8];
          unpack8_16bit(wr, wdt == MQ_BF16, wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float xv[8];
            unpack8_16bit(xr[i], xdt == MQ_BF16, xv);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
          }
        }
      } else {
        for (int64_t k = (int64_t)kt * 8; k < H; k += 256 * 8) {
          float wv[8];
          load8_safe(w, wdt, w_row, k, H, vec_ok, wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (tb + i < T) {
              float xv[8];
              load8_safe(x, xdt, (size_t)(tb + i) * H, k, H, vec_ok, xv);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[i] = fmaf(xv[j], wv[j], acc[i]);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = acc[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && tb + i < T) s_part[kwarp][tb + i] = v;
      }
    }
    __syncthreads();
    if (tid < T) {
      float v = s_part[0][tid];
#pragma unroll
      for (int wi = 1; wi < 8; ++wi) v += s_part[wi][tid];
      logits[(size_t)tid * E + e] = v;
    }
  }
  // ---- phase A: token row e prepared for the W4A16 kernels (w4_prep.cuh), with its sums over every 128 k
  if (xp != nullptr && e < T) {
    __syncthreads();                             // s_part is free again: the logits were formed above
    route_prepare_row(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)e * H, H, prep_mode, xp + (size_t)e * H,
                      xs + (size_t)e * W4_XS_STRIDE, &s_part[0][0]);
  }

  // ---- who is last?
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(counter, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // ---- phase B: the logits of all experts come from L2 into shared memory, then one warp per token
  unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(rsm_smem);   // [E] tokens that chose expert e
  float* s_logits = reinterpret_cast<float*>(s_mask + E);                        // [T, E]
  int* s_ids = reinterpret_cast<int*>(s_logits + (size_t)T * E);                  // [T * K]
  int* s_run = s_ids + T * K;                                                    // [E] first sorted slot of expert e
  for (int i = tid; i < T * E; i += RSM_THREADS) s_logits[i] = __ldcg(logits + i);
  for (int ee = tid; ee < E; ee += RSM_THREADS) s_mask[ee] = 0ull;
  __syncthreads();
  if (T <= RSM_THREADS / 32) {
    for (int t = warp; t < T; t += RSM_THREADS / 32)
      softmax_topk_row<EPL>(s_logits + (size_t)t * E, 1, 0, bias, E, K, renorm, lane,
                            ids64 ? ids64 + (size_t)t * K : nullptr, s_ids + t * K, weights + (size_t)t * K);
  } else {
    // more tokens than warps: eight lanes per token, so that the 64 tokens of the largest batch are one pass
    for (int t0 = warp * 4; t0 < T; t0 += RSM_THREADS / 8) {
      const int t = t0 + (lane >> 3);
      const bool live = t < T;
      const int tr = live ? t : T - 1;
      softmax_topk_sub8<EPL * 4>(s_logits + (size_t)tr * E, bias, E, K, renorm, lane & 7, live,
                                 ids64 ? ids64 + (size_t)tr * K : nullptr, s_ids + tr * K, weights + (size_t)tr * K);
    }
  }
  __syncthreads();
  route_plan_small(s_ids, s_mask, s_run, T, E, K, ids32, perm, inv, off32, off64);
  if (tid == 0) *counter = 0;                       // ready for the next call
}

template <int EPL>
void launch_topk(const float* logits, int slices, const float* bias, int64_t T, int E, int K, int renorm,
                 int64_t* ids64, int32_t* ids32, float* weights, cudaStream_t st) {
  unsigned blocks = (unsigned)((T + 3) / 4);
  router_softmax_topk<EPL><<<blocks, 128, 0, st>>>(logits, slices, bias, T, E, K, renorm, ids64, ids32, weights);
}

}  // namespace
}  // namespace mq

namespace mq {
// Tensor-memory logits kernel (router_tc5.cu).
bool router_tc5_covers(int x_dtype, int w_dtype, int64_t T, int64_t H, int64_t E);
int router_logits_tc5(const void* x, const void* w, bool bf16, int64_t T, int64_t H, int64_t E, int slices,
                      int64_t k_per_slice, float* logits, cudaStream_t st);
namespace {
// Batches up to this size use the one-warp-per-(expert, 8 tokens) kernel.
constexpr int64_t R_SKINNY_MAX_T = 15;

// True when the tensor-core logits kernel applies: both operands 16-bit of the same type, 16-byte rows.
bool router_mma_ok(int x_dtype, int w_dtype, int64_t H) { return x_dtype == w_dtype && x_dtype != MQ_F32 && H % 32 == 0; }

// K slices for the tiled logits kernels: enough CTAs for two per SM.  The tensor-core kernel takes
// slices of at least 128 k (one accumulation chunk), the SIMT kernel of at least 256 k.
int router_slices(int64_t T, int64_t H, int64_t E, bool mma) {
  if (T <= R_SKINNY_MAX_T && !mma) return 1;
  const int64_t ctas = ((T + R_TM - 1) / R_TM) * ((E + R_TE - 1) / R_TE);
  int64_t s = (2 * 148 + ctas - 1) / ctas;
  const int64_t max_s = mma ? (H + 127) / 128 : (H + 255) / 256;
  const int64_t cap = mma ? 16 : 8;
  if (s > max_s) s = max_s;
  if (s > cap) s = cap;
  if (s < 1) s = 1;
  return (int)s;
}
}  // namespace
}  // namespace mq

extern "C" size_t mq_router_workspace_bytes(int64_t T, int64_t H, int64_t E) {
  if (T <= 0 || E <= 0 || H <= 0) return 16;
  // the dtype is not known here: size for the larger of the two slice counts
  return (size_t)mq::router_slices(T, H, E, H % 32 == 0) * (size_t)T * (size_t)E * sizeof(float);
}

extern "C" int mq_router_topk(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                              int64_t T, int64_t H, int64_t E, int64_t K, int renormalize,
                              float* logits_ws, size_t logits_ws_bytes, int64_t* ids64, int32_t* ids32,
                              float* weights, void* stream) {
  using namespace mq;
  if (T < 0 || H <= 0 || E <= 0 || K <= 0) return MQ_ERR_INVALID_ARGUMENT;
  if (!valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (K > E || E > 1024 || K > 32) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!x || !w || !logits_ws || !weights || (!ids64 && !ids32)) return MQ_ERR_INVALID_ARGUMENT;
  if (logits_ws_bytes < mq_router_workspace_bytes(T, H, E)) return MQ_ERR_WORKSPACE_TOO_SMALL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  // vector loads need 16-byte rows: H a multiple of 8 elements and aligned bases
  int vec_ok = (H % 8 == 0) && aligned16(x) && aligned16(w);

  int slices = 1;
  const bool mma = vec_ok && router_mma_ok(x_dtype, w_dtype, H);
  if (T <= R_SKINNY_MAX_T && !mma) {
    router_logits_skinny<<<(unsigned)E, 128, 0, st>>>(x, x_dtype, w, w_dtype, T, H, E, vec_ok, logits_ws);
  } else {
    slices = router_slices(T, H, E, mma);
    int64_t k_per_slice = (H + slices - 1) / slices;
    k_per_slice = mma ? (k_per_slice + 127) / 128 * 128 : (k_per_slice + R_KC - 1) / R_KC * R_KC;
    dim3 grid((unsigned)((T + R_TM - 1) / R_TM), (unsigned)((E + R_TE - 1) / R_TE), (unsigned)slices);
    int tc_rc = MQ_ERR_DRIVER_ENTRY;
    if (mma && router_tc5_covers(x_dtype, w_dtype, T, H, E) && aligned16(logits_ws))
      tc_rc = router_logits_tc5(x, w, x_dtype == MQ_BF16, T, H, E, slices, k_per_slice, logits_ws, st);
    if (tc_rc == MQ_OK) {
      // logits written by the tensor-memory kernel (same slices, same 128-k chunking)
    } else if (mma) {
      // same tile shape as the SIMT kernel (32 tokens x 128 experts), so the grid carries over
      cudaFuncSetAttribute(router_logits_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, RM_SMEM_BYTES);
      router_logits_mma<<<grid, RM_THREADS, RM_SMEM_BYTES, st>>>(reinterpret_cast<const uint16_t*>(x),
          reinterpret_cast<const uint16_t*>(w), x_dtype == MQ_BF16, T, H, E, k_per_slice, logits_ws);
    } else {
      router_logits_tiled<<<grid, R_THREADS, 0, st>>>(x, x_dtype, w, w_dtype, T, H, E, k_per_slice, vec_ok, logits_ws);
    }
  }
  int rc = check_launch();
  if (rc != MQ_OK) return rc;

  int e = (int)E, k = (int)K;
  if (E <= 32) launch_topk<1>(logits_ws, slices, bias, T, e, k, renormalize, ids64, ids32, weights, st);
  else if (E <= 64) launch_topk<2>(logits_ws, slices, bias, T, e, k, renormalize, ids64, ids32, weights, st);
  else if (E <= 128) launch_topk<4>(logits_ws, slices, bias, T, e, k, renormalize, ids64, ids32, weights, st);
  else if (E <= 256) launch_topk<8>(logits_ws, slices, bias, T, e, k, renormalize, ids64, ids32, weights, st);
  else if (E <= 512) launch_topk<16>(logits_ws, slices, bias, T, e, k, renormalize, ids64, ids32, weights, st);
  else launch_topk<32>(logits_ws, slices, bias, T, e, k, renormalize, ids64, ids32, weights, st);
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// Router without a caller-provided workspace.
//
// Some callers cannot hand this library scratch memory because they cannot allocate at the moment
// of the call: a serving loop that runs inside a region where the CUDA allocator must not be
// touched, a host runtime (cgo, JNI, a plugin sandbox) that was given a fixed set of device buffers
// for inputs and outputs and nothing else, or a process whose memory pool already owns the whole
// device.  For them the logits scratch lives in the library image itself: a file-scope device
// array that every GPU loading the library holds until the process exits.
//
// Host code must not pass the array's name to a kernel: on the host that name is only a stand-in
// for the symbol, not a device address.  The address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels get.
// 10 MiB.  The logits take slices * T * E * 4 bytes and the slice count falls as the batch grows; at 128
// experts and 16-bit inputs the largest request up to 16384 tokens is 2 slices x 9440 tokens = 9.22 MiB
// (one slice from 9441 tokens on: 8 MiB at 16384), so every batch up to 16384 tokens fits.
constexpr size_t R_STATIC_SCRATCH_BYTES = (size_t)10 << 20;
static __device__ __align__(256) float g_router_static_scratch[R_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace mq {
namespace {
constexpr int kMaxDevices = 64;

// Device address of the scratch array on the current device (set-up on the first call per device).
float* static_scratch_for_current_device(int* status) {
  static std::mutex mu;
  static float* addr[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    if (e != cudaSuccess) set_last_cuda_error(e);
    *status = MQ_ERR_LAUNCH_FAILED;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_router_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_cuda_error(e);
      *status = MQ_ERR_LAUNCH_FAILED;
      return nullptr;
    }
    addr[dev] = static_cast<float*>(p);
  }
  return addr[dev];
}
}  // namespace
}  // namespace mq

extern "C" int mq_router_topk_static(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                                     int64_t T, int64_t H, int64_t E, int64_t K, int renormalize,
                                     int64_t* ids64, int32_t* ids32, float* weights, void* stream) {
  if (T > 0 && H > 0 && E > 0 && mq_router_workspace_bytes(T, H, E) > R_STATIC_SCRATCH_BYTES)
    return MQ_ERR_STATIC_SCRATCH_EXCEEDED;
  int status = MQ_OK;
  float* scratch = mq::static_scratch_for_current_device(&status);
  if (scratch == nullptr) return status;
  // The logits kernel writes every element of the slices it uses before the selection kernel reads
  // them, so nothing in the array has to start at zero and the previous call's contents are harmless.
  return mq_router_topk(x, x_dtype, w, w_dtype, bias, T, H, E, K, renormalize, scratch, R_STATIC_SCRATCH_BYTES,
                        ids64, ids32, weights, stream);
}

// ---------------------------------------------------------------------------------------------
extern "C" size_t mq_route_small_workspace_bytes(int64_t T, int64_t E) {
  if (T <= 0 || E <= 0) return 16;
  return (size_t)T * (size_t)E * sizeof(float) + 512;       // a header of counters, then the logits
}

extern "C" int mq_route_small(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                              int64_t T, int64_t H, int64_t E, int64_t K, int renormalize,
                              void* workspace, size_t workspace_bytes, int64_t* ids64, int32_t* ids32,
                              float* weights, int32_t* perm, int32_t* inv, int64_t* offsets64, int32_t* offsets32,
                              void* xp, float* xs, int xp_format, void* stream) {
  using namespace mq;
  if (T < 0 || H <= 0 || E <= 0 || K <= 0) return MQ_ERR_INVALID_ARGUMENT;
  if (!valid_dtype(x_dtype) || !valid_dtype(w_dtype)) return MQ_ERR_INVALID_ARGUMENT;
  if (K > E || K > 32 || T > RSM_MAX_T || E > RSM_MAX_E || T * K > RSM_MAX_S) return MQ_ERR_UNSUPPORTED_SHAPE;
  if ((xp != nullptr) != (xs != nullptr)) return MQ_ERR_INVALID_ARGUMENT;
  // the prepared rows are a bf16 format with 128-k groups, 32 of them at most
  if (xp != nullptr && (x_dtype != MQ_BF16 || H % 128 != 0 || H / 128 > 32)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (xp != nullptr && T > E) return MQ_ERR_UNSUPPORTED_SHAPE;     // CTA t prepares token t; there are E CTAs
  if (xp != nullptr && xp_format != 1 && xp_format != 2) return MQ_ERR_INVALID_ARGUMENT;
  if (xp != nullptr && xp_format == 2 && H / 128 > W4_XS_UNSCALE) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (T == 0) return MQ_OK;
  if (!x || !w || !workspace || !weights || !ids32 || !perm || !inv || (!offsets64 && !offsets32))
    return MQ_ERR_INVALID_ARGUMENT;
  if (workspace_bytes < mq_route_small_workspace_bytes(T, E) || !aligned16(workspace)) return MQ_ERR_WORKSPACE_TOO_SMALL;
  if (xp != nullptr && (!aligned16(x) || !aligned16(xp))) return MQ_ERR_INVALID_ARGUMENT;
  const int vec_ok = (H % 8 == 0) && aligned16(x) && aligned16(w);
  // The counters sit at the START of the workspace (a header of 128 ints), the logits behind them: their place
  // must not depend on T, or a call with fewer tokens than an earlier one on the same workspace would find the
  // earlier call's logits where it expects zero counters (no CTA would then be "last" and the plan would never
  // be written).
  int* counter = reinterpret_cast<int*>(workspace);
  float* logits = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + RTK_HEADER_INTS * sizeof(int));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (T > 16 && vec_ok && x_dtype != MQ_F32 && w_dtype != MQ_F32) {
    // more tokens than one CTA has warps: the token-major kernel (selection on as many SMs as there are tokens)
    const size_t smem_t = (size_t)E * 8 + (size_t)E * 4 + (size_t)T * K * 4 + (size_t)E * 4;
    const dim3 grid((unsigned)((E + 31) / 32), (unsigned)T);
#define MQ_RTK_LAUNCH(EPL)                                                                                       \
    launch_after_predecessor(route_tokens_kernel<EPL>, grid, dim3(RTK_THREADS), smem_t, st,                       \
        reinterpret_cast<const uint16_t*>(x), (int)(x_dtype == MQ_BF16), reinterpret_cast<const uint16_t*>(w),    \
        (int)(w_dtype == MQ_BF16), bias, (int)T, (int)H, (int)E, (int)K, renormalize, logits, counter, ids32,     \
        ids64, weights, perm, inv, offsets32, offsets64, reinterpret_cast<__nv_bfloat16*>(xp), xs,                \
        xp_format == 2 ? 2 : 1)
    if (E <= 32) MQ_RTK_LAUNCH(1);
    else if (E <= 64) MQ_RTK_LAUNCH(2);
    else if (E <= 128) MQ_RTK_LAUNCH(4);
    else MQ_RTK_LAUNCH(8);
#undef MQ_RTK_LAUNCH
    return check_launch();
  }
  const size_t smem = (size_t)E * 8 + (size_t)T * E * 4 + (size_t)T * K * 4 + (size_t)E * 4;
#define MQ_RSM_LAUNCH(EPL)                                                                                       \
  do {                                                                                                           \
    cudaFuncSetAttribute(route_small_kernel<EPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    launch_after_predecessor(route_small_kernel<EPL>, dim3((unsigned)E), dim3(RSM_THREADS), smem, st,             \
        x, x_dtype, w, w_dtype, bias, (int)T, (int)H, (int)E, (int)K, renormalize, vec_ok, logits, counter, ids32, \
        ids64, weights, perm, inv, offsets32, offsets64, reinterpret_cast<__nv_bfloat16*>(xp), xs,                \
        xp_format == 2 ? 2 : 1);                                                                                  \
  } while (0)
  if (E <= 32) MQ_RSM_LAUNCH(1);
  else if (E <= 64) MQ_RSM_LAUNCH(2);
  else if (E <= 128) MQ_RSM_LAUNCH(4);
  else MQ_RSM_LAUNCH(8);
#undef MQ_RSM_LAUNCH
  return check_launch();
}
