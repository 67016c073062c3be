// W4A16 grouped GEMM for decode-size batches on the 5th-generation tensor cores:
//   out[r, n] = bf16( sum_k x[r,k] * (q[e][k,n] - z[e][k/128, n]) * s[e][k/128, n] ),  rows r of group e.
// Follows mini_qwen/kernels/w4a16_gemm.py:8-15,194-247 and the expert loop of
// mini_qwen/model/layers/moe.py:24-25,59-65 with LinearW4A16 projections (linear_w4a16.py:31-36).
//
// The packed weights are the only large stream (0.5 byte per weight), so the kernel is built around
// touching each int4 word once with as few instructions as possible:
//   * output columns are the 128 TMEM lanes (M), the group's tokens are N (16 or 32), K = 16 per MMA;
//   * the int32 words [16 k-rows x 128 columns] of one quantisation group (128 k) arrive by TMA in the
//     checkpoint layout, together with the group's slice of the token rows: one ring stage per group;
//   * eight dequantisation warps read one word per lane and column (conflict-free), turn it into four
//     bf16 pairs with one shift and one logic op each ((w >> 4p) & 0x000F000F | 0x43004300 = {128+q_p,
//     128+q_{p+4}}), and write them straight into TENSOR MEMORY (tcgen05.st), from where tcgen05.mma
//     takes its A operand: the dequantised tile never passes through shared memory;
//   * the pairs come out in k order 0,4,1,5,2,6,3,7 inside every 8; the activations are stored in the
//     same order by the preparation kernel (and by the gate/up epilogue for the down projection), so
//     both operands agree and no permute instruction is spent;
//   * zero points and scales never touch the weights: the pairs are re-centred to q-8 (one packed fma),
//     the tensor core sums x*(q-8) over one quantisation group (128 k) into a TMEM accumulator, four
//     fold warps read it and add s * (D - (z-8) * xs) in fp32, xs = sum of x over the group (computed
//     by the preparation kernel).
//     The dequantised weight is never rounded.
// Every wait is a bounded mbarrier wait; on expiry the kernel sets MQ_DEV_WAIT_EXPIRED and leaves.
//
// Measured on B200 (decode layer H=2048, I=768, 128 experts, batch 64: about 4 tokens per expert):
// gate/up 120 us and down 95 us against 87 us and 42 us of the mma.sync stream kernel (w4a16.cu), so the
// block does not use this kernel unless asked to (Qwen3MoEBlock.w4_kernel = "tc").  A timeline taken
// with clock64 shows why: the thread that issues the MMAs needs about 65 cycles per tcgen05.mma whatever
// its size, and an MMA of 16 tokens covers only 128 columns x 16 k = 2048 weights, so issue alone costs
// 1000 cycles per quantisation group and tile (the dequantisation warps need the same 1000, the fold
// warps 450, and they overlap); rotating the k steps over independent accumulators changes nothing.
// The shape pays off only with more tokens per expert than a decode batch has.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "w4_prep.cuh"

namespace mq {
namespace {

constexpr int W_TM = 128;                       // output columns per sub-tile = TMEM lanes
constexpr int W_GK = 128;                       // k per ring stage = one quantisation group
constexpr int W_TN = 32;                        // most tokens per tile (MMA N is 16 or 32)
constexpr int W_STAGES = 6;
constexpr int W_WORDS_BYTES = (W_GK / 8) * W_TM * 4;   // 8 KB: 16 word rows x 128 columns
constexpr int W_XATOM_BYTES = W_TN * 64 * 2;    // 4 KB: 32 token rows of 64 k (128 bytes), 128-byte swizzle
constexpr int W_X_BYTES = 2 * W_XATOM_BYTES;    // 8 KB: the two 64-k halves of the group
constexpr int W_STAGE_BYTES = 2 * W_WORDS_BYTES + W_X_BYTES;   // 24 KB (the second word block: up projection)
constexpr int W_XS_STRIDE = 32;                 // floats per row of the group-sum table (>= Kd / 128)
constexpr int W_XS_BYTES = W_TN * W_XS_STRIDE * 4;             // 4 KB per tile
constexpr int W_FOLD_WARPS = 4, W_DQ_WARPS = 8;
constexpr int W_THREADS = (2 + W_FOLD_WARPS + W_DQ_WARPS) * 32;   // 448
constexpr int W_SMEM_BYTES = W_STAGES * W_STAGE_BYTES + 2 * W_XS_BYTES + 1024 /*alignment*/ + 512 /*barriers*/;
constexpr int W_TMEM_COLS = 512;                // A: columns 0..255 (2 buffers x 2 sub-tiles x 64), D: 256..383
constexpr int W_A_COL = 0, W_D_COL = 256;
constexpr uint32_t W_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t w_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void w_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void w_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void w_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool w_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the wait ran out or another role already gave up.
__device__ __forceinline__ bool w_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* d_status) {
  for (uint32_t spin = 0; spin < W_SPIN_LIMIT; ++spin) {
    if (w_mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (d_status != nullptr) atomicOr(d_status, (int)MQ_DEV_WAIT_EXPIRED);
  return false;
}
__device__ __forceinline__ void w_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void w_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void w_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void w_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory descriptor of the token tile: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t w_umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t w_umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(W_TM >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (row m in lane m, two bf16
// per 32-bit column).
__device__ __forceinline__ void w_umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void w_umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void w_tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void w_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void w_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void w_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One tile: (group, token tile, 128-column weight tile).
struct WTile {
  int expert, wt, tok0, tok_end, n_mma;
};
struct WCursor {
  const int32_t* off;
  int E, NWT;
  int e, base;
  __device__ WCursor(const int32_t* o, int E_, int NWT_) : off(o), E(E_), NWT(NWT_), e(0), base(0) {}
  __device__ bool locate(int t, WTile& tile) {
    while (e < E) {
      const int lo = off[e], hi = off[e + 1];
      const int n = hi - lo;
      const int ntt = (n + W_TN - 1) / W_TN;
      const int span = ntt * NWT;
      if (t < base + span) {
        const int local = t - base;
        const int tt = local / NWT;
        tile.expert = e;
        tile.wt = local - tt * NWT;
        tile.tok0 = lo + tt * W_TN;
        tile.tok_end = min(tile.tok0 + W_TN, hi);
        tile.n_mma = (tile.tok_end - tile.tok0) > 16 ? 32 : 16;
        return true;
      }
      base += span;
      ++e;
    }
    return false;
  }
};

// Position of column c inside its block of 8 in the order the dequantised pairs come out (0,4,1,5,2,6,3,7).
__device__ __forceinline__ int kperm_pos(int c) { return (c & ~7) | (((c & 3) << 1) | ((c >> 2) & 1)); }

struct W4TcProj {
  const __nv_bfloat16* sc;   // [Ew, G, N]
  const int32_t* qz;         // [Ew, G, N/8]
};

template <bool SWIGLU>
__global__ void __launch_bounds__(W_THREADS, 1)
w4a16_tc5_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w0,
                 const __grid_constant__ CUtensorMap map_w1, W4TcProj p0, W4TcProj p1,
                 const float* __restrict__ xs, const int32_t* __restrict__ offsets, int E, int period, int S,
                 int N, int Kd, __nv_bfloat16* __restrict__ out, int32_t* d_status) {
  // map_w0 / p0: the projection (gate with SWIGLU); map_w1 / p1: the up projection (SWIGLU only).
  // out: [S, N]; with SWIGLU its columns are stored in the k order of the next projection's A operand.
  constexpr int NSUB = SWIGLU ? 2 : 1;
  extern __shared__ uint8_t w_smem_raw[];
  const uint32_t raw = w_smem_u32(w_smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t* ring_ptr = w_smem_raw + (ring - raw);
  const uint32_t xs_smem = ring + W_STAGES * W_STAGE_BYTES;
  const float* xs_ptr = reinterpret_cast<const float*>(ring_ptr + W_STAGES * W_STAGE_BYTES);
  const uint32_t bars = xs_smem + 2 * W_XS_BYTES;
  uint8_t* bar_mem = ring_ptr + W_STAGES * W_STAGE_BYTES + 2 * W_XS_BYTES;
  // One tcgen05.commit per quantisation group: `done` tells the fold warps that the group's sums are in
  // TMEM, the dequantisation warps that the A buffer may be rewritten, and (through a fold warp's arrive
  // on raw_empty) the producer that the MMAs have read the stage's token rows.
  auto raw_full = [&](int s) { return bars + 8u * s; };
  auto raw_empty = [&](int s) { return bars + 8u * (W_STAGES + s); };
  auto a_full = [&](int b) { return bars + 8u * (2 * W_STAGES + b); };
  auto done = [&](int b) { return bars + 8u * (2 * W_STAGES + 2 + b); };
  auto d_empty = [&](int b) { return bars + 8u * (2 * W_STAGES + 4 + b); };
  auto xs_full = [&](int b) { return bars + 8u * (2 * W_STAGES + 6 + b); };
  auto xs_empty = [&](int b) { return bars + 8u * (2 * W_STAGES + 8 + b); };
  constexpr int MISC = 8 * (2 * W_STAGES + 10);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(bar_mem + MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + MISC + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NWT = N / W_TM;
  const int G = Kd / W_GK;                       // quantisation groups = ring stages per tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < W_STAGES; ++s) {
      w_mbar_init(raw_full(s), 1);
      w_mbar_init(raw_empty(s), W_DQ_WARPS + 1);       // the dequantisation warps + one fold warp on behalf of the MMAs
    }
    for (int b = 0; b < 2; ++b) {
      w_mbar_init(a_full(b), W_DQ_WARPS);
      w_mbar_init(done(b), 1);
      w_mbar_init(d_empty(b), W_FOLD_WARPS * 32);
      w_mbar_init(xs_full(b), 1);
      w_mbar_init(xs_empty(b), W_FOLD_WARPS * 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(w_smem_u32((const void*)tmem_ptr_smem)), "r"((uint32_t)W_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  w_fence_before();
  __syncthreads();
  w_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: words, tokens, group sums
    if (lane == 0) {
      WCursor cur(offsets, E, NWT);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WTile tl;
      int it = 0;
      for (int t = blockIdx.x; ok; t += gridDim.x, ++it) {
        if (!cur.locate(t, tl)) break;
        // group sums of the tile's tokens: rows of W_XS_STRIDE floats, one bulk copy
        const int xb = it & 1;
        ok = w_mbar_wait(xs_empty(xb), (uint32_t)((it >> 1) & 1) ^ 1u, abort_flag, d_status);
        if (!ok) break;
        const uint32_t xs_bytes = (uint32_t)(tl.tok_end - tl.tok0) * W_XS_STRIDE * 4;
        w_mbar_expect_tx(xs_full(xb), xs_bytes);
        w_bulk_load(xs_smem + xb * W_XS_BYTES, xs + (size_t)tl.tok0 * W_XS_STRIDE, xs_bytes, xs_full(xb));
        const int n0 = tl.wt * W_TM;
        const int wrow = (tl.expert % period) * (Kd / 8);
        for (int g = 0; g < G && ok; ++g) {
          ok = w_mbar_wait(raw_empty(stage), phase ^ 1u, abort_flag, d_status);
          if (!ok) break;
          const uint32_t st = ring + stage * W_STAGE_BYTES;
          w_mbar_expect_tx(raw_full(stage), (uint32_t)(NSUB * W_WORDS_BYTES + W_X_BYTES));
          w_tma_load_2d(st, &map_w0, raw_full(stage), n0, wrow + g * (W_GK / 8));
          if (SWIGLU) w_tma_load_2d(st + W_WORDS_BYTES, &map_w1, raw_full(stage), n0, wrow + g * (W_GK / 8));
          w_tma_load_2d(st + 2 * W_WORDS_BYTES, &map_x, raw_full(stage), g * W_GK, tl.tok0);
          w_tma_load_2d(st + 2 * W_WORDS_BYTES + W_XATOM_BYTES, &map_x, raw_full(stage), g * W_GK + 64, tl.tok0);
          if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      // drain: no bulk copy may still be writing shared memory when the CTA exits
      for (int s = 0; s < W_STAGES && ok; ++s) {
        ok = w_mbar_wait(raw_empty(stage), phase ^ 1u, abort_flag, d_status);
        if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      WCursor cur(offsets, E, NWT);
      int stage = 0;
      uint32_t phase = 0;
      int gc = 0;                                 // groups issued so far
      bool ok = true;
      WTile tl;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        if (!cur.locate(t, tl)) break;
        const uint32_t idesc = w_umma_idesc(tl.n_mma);
        for (int g = 0; g < G && ok; ++g, ++gc) {
          const int b = gc & 1;
          const uint32_t par = (uint32_t)((gc >> 1) & 1);
          ok = w_mbar_wait(d_empty(b), par ^ 1u, abort_flag, d_status) &&      // the fold warps have read D[b]
               w_mbar_wait(a_full(b), par, abort_flag, d_status) &&            // A[b] is written
               w_mbar_wait(raw_full(stage), phase, abort_flag, d_status);      // the token rows have landed
          if (!ok) break;
          w_fence_after();
          const uint32_t xaddr = ring + stage * W_STAGE_BYTES + 2 * W_WORDS_BYTES;
          const uint32_t dcol = tmem_base + W_D_COL + b * 64;
          const uint32_t acol = tmem_base + W_A_COL + b * 128;
#pragma unroll
          for (int k = 0; k < W_GK / 16; ++k) {
            const uint64_t bd = w_umma_desc(xaddr + (k >> 2) * W_XATOM_BYTES) + 2u * (k & 3);
            const uint32_t accum = k != 0 ? 1u : 0u;
            w_umma_ts(dcol, acol + 8 * k, bd, idesc, accum);
            if (SWIGLU) w_umma_ts(dcol + 32, acol + 64 + 8 * k, bd, idesc, accum);
          }
          w_umma_commit(done(b));
          if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 2 + W_FOLD_WARPS) {
    // ------------------------------------------------------------------ dequantisation (warps 6..13)
    // A warp owns one TMEM lane quadrant (32 output columns) and one 64-k half of every group.
    const int quad = warp & 3;                     // TMEM lane quadrant this warp may write
    const int khalf = (warp - (2 + W_FOLD_WARPS)) >> 2;
    const int col = quad * 32 + lane;              // output column inside the tile
    WCursor cur(offsets, E, NWT);
    int stage = 0;
    uint32_t phase = 0;
    int gc = 0;
    bool ok = true;
    WTile tl;
    for (int t = blockIdx.x; ok; t += gridDim.x) {
      if (!cur.locate(t, tl)) break;
      for (int g = 0; g < G && ok; ++g, ++gc) {
        const int b = gc & 1;
        ok = __all_sync(0xffffffffu, w_mbar_wait(raw_full(stage), phase, abort_flag, d_status) &&
                                         w_mbar_wait(done(b), (uint32_t)((gc >> 1) & 1) ^ 1u, abort_flag, d_status));
        if (!ok) break;
        w_fence_after();
        const uint8_t* st = ring_ptr + stage * W_STAGE_BYTES;
#pragma unroll
        for (int sub = 0; sub < NSUB; ++sub) {
          const uint32_t* words = reinterpret_cast<const uint32_t*>(st + sub * W_WORDS_BYTES) + (8 * khalf) * W_TM + col;
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = words[j * W_TM];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                // {128+q_p, 128+q_(p+4)}, re-centred to {q_p - 8, q_(p+4) - 8} by a packed fma (FMA pipe), so
                // that the group's sum in tensor memory stays as small as the result
                const uint32_t biased = ((w[4 * hh + j] >> (4 * p)) & 0x000F000Fu) | 0x43004300u;
                asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r[4 * j + p]) : "r"(biased), "r"(0x3F803F80u), "r"(0xC308C308u));
              }
            w_tmem_st16(tmem_base + ((uint32_t)(quad * 32) << 16) + W_A_COL + b * 128 + sub * 64 + khalf * 32 + hh * 16, r);
          }
        }
        w_tmem_st_wait();
        w_fence_before();
        __syncwarp();
        if (lane == 0) {
          w_mbar_arrive(a_full(b));
          w_mbar_arrive(raw_empty(stage));         // this warp has read its words of the stage
        }
        if (++stage == W_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ fold + epilogue (warps 2..5)
    const int quad = warp & 3;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    WCursor cur(offsets, E, NWT);
    int gc = 0, it = 0, stage = 0;
    bool ok = true;
    WTile tl;
    for (int t = blockIdx.x; ok; t += gridDim.x, ++it) {
      if (!cur.locate(t, tl)) break;
      const int n = tl.wt * W_TM + quad * 32 + lane;          // this lane's output column
      const int ew = tl.expert % period;
      const __nv_bfloat16* sc0 = p0.sc + (size_t)ew * G * N + n;
      const int32_t* qz0 = p0.qz + (size_t)ew * G * (N / 8) + (n >> 3);
      const __nv_bfloat16* sc1 = SWIGLU ? p1.sc + (size_t)ew * G * N + n : nullptr;
      const int32_t* qz1 = SWIGLU ? p1.qz + (size_t)ew * G * (N / 8) + (n >> 3) : nullptr;
      const int zshift = 4 * (n & 7);
      const int xb = it & 1;
      ok = __all_sync(0xffffffffu, w_mbar_wait(xs_full(xb), (uint32_t)((it >> 1) & 1), abort_flag, d_status));
      if (!ok) break;
      const float* xt = xs_ptr + xb * (W_XS_BYTES / 4);       // [token][group]
      float acc[NSUB][W_TN];
#pragma unroll
      for (int s = 0; s < NSUB; ++s)
#pragma unroll
        for (int i = 0; i < W_TN; ++i) acc[s][i] = 0.0f;
      for (int g = 0; g < G && ok; ++g, ++gc) {
        // this group's scale and (zero point - 8) for the lane's column, fetched before the wait
        float sc[NSUB], zb[NSUB];
        sc[0] = __bfloat162float(sc0[(size_t)g * N]);
        zb[0] = (float)((int)((qz0[(size_t)g * (N / 8)] >> zshift) & 15) - 8);
        if (SWIGLU) {
          sc[NSUB - 1] = __bfloat162float(sc1[(size_t)g * N]);
          zb[NSUB - 1] = (float)((int)((qz1[(size_t)g * (N / 8)] >> zshift) & 15) - 8);
        }
        const int b = gc & 1;
        ok = __all_sync(0xffffffffu, w_mbar_wait(done(b), (uint32_t)((gc >> 1) & 1), abort_flag, d_status));
        if (!ok) break;
        if (warp == 2 && lane == 0) w_mbar_arrive(raw_empty(stage));   // the MMAs have read the stage's token rows
        if (++stage == W_STAGES) stage = 0;
        w_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (16 * half < tl.n_mma) {
            uint32_t d[NSUB][16];
#pragma unroll
            for (int s = 0; s < NSUB; ++s) w_tmem_ld16(lane_base + W_D_COL + b * 64 + s * 32 + 16 * half, d[s]);
            w_tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float xsum = xt[(16 * half + i) * W_XS_STRIDE + g];
#pragma unroll
              for (int s = 0; s < NSUB; ++s)
                acc[s][16 * half + i] += sc[s] * (__uint_as_float(d[s][i]) - zb[s] * xsum);
            }
          }
        }
        w_fence_before();
        w_mbar_arrive(d_empty(b));
      }
      if (!ok) break;
      w_mbar_arrive(xs_empty(xb));
      // store: one column per lane, the tile's token rows
      const int ntok = tl.tok_end - tl.tok0;
      const int ocol = SWIGLU ? kperm_pos(n) : n;
#pragma unroll
      for (int i = 0; i < W_TN; ++i) {
        if (i < ntok) {
          const float v = SWIGLU ? swiglu_rounded<__nv_bfloat16>(acc[0][i], acc[NSUB - 1][i]) : acc[0][i];
          out[(size_t)(tl.tok0 + i) * N + ocol] = __float2bfloat16_rn(v);
        }
      }
    }
  }

  w_fence_before();
  __syncthreads();
  if (warp == 1) {
    w_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)W_TMEM_COLS) : "memory");
  }
}

// Preparation of the activations: row r of the output is x[src(r)] with the k order 0,4,1,5,2,6,3,7
// inside every 8 (when `shuffle`), and xs[r][g] = sum of the row over quantisation group g.
// src(r) = perm[r] / top_k when perm is given (the expert-sorted order), else r.  One warp per row.
__global__ void __launch_bounds__(256)
w4_prep_rows(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ perm, int top_k, int S, int Kd,
             int mode, __nv_bfloat16* __restrict__ xp, float* __restrict__ xs) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= S) return;
  const int lane = threadIdx.x & 31;
  const size_t src = perm != nullptr ? (size_t)(perm[r] / top_k) : (size_t)r;
  const uint4* in = reinterpret_cast<const uint4*>(x + src * Kd);
  uint4* o = xp != nullptr ? reinterpret_cast<uint4*>(xp + (size_t)r * Kd) : nullptr;
  const bool f16 = mode == 2;
  float scale = 1.0f;
  if (f16) {                                       // the row's largest magnitude decides its power of two
    float amax = 0.0f;
    for (int c = lane; c < Kd / 8; c += 32) amax = fmaxf(amax, w4_piece_amax(in[c]));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const int e = w4_row_exponent(amax);
    scale = w4_pow2(e);
    if (lane == 0) xs[(size_t)r * W_XS_STRIDE + W4_XS_UNSCALE] = w4_pow2(-e);
  }
  for (int c0 = 0; c0 < Kd / 8; c0 += 32) {      // 16-byte pieces; a group of 128 k is 16 pieces = half a warp
    const int c = c0 + lane;
    float sum = 0.0f;
    if (c < Kd / 8) {
      const uint4 w = w4_prepare_piece(in[c], mode != 0, f16, scale, sum);
      if (o != nullptr) o[c] = w;
    }
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if ((lane & 15) == 0 && c < Kd / 8) xs[(size_t)r * W_XS_STRIDE + (c >> 4)] = sum;
  }
}

typedef CUresult (*W4EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

W4EncodeFn w4_encode_fn() {
  static W4EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<W4EncodeFn>(p);
  });
  return fn;
}

bool w4_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows,
               uint64_t cols, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
  W4EncodeFn fn = w4_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int w4_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

bool w4_tc_covers(int64_t S, int64_t Ew, int64_t N, int64_t Kd, int64_t group_size) {
  return group_size == 128 && Kd % 128 == 0 && Kd / 128 <= W_XS_STRIDE && N % W_TM == 0 &&
         S < ((int64_t)1 << 30) && Ew * (Kd / 8) < ((int64_t)1 << 31) && Ew * N * (Kd / 128) < ((int64_t)1 << 40);
}

}  // namespace
}  // namespace mq

extern "C" int mq_w4a16_tc_prep(const void* x, const int32_t* perm, int64_t top_k, int64_t S, int64_t Kd,
                                int shuffle, void* xp, float* xs, void* stream) {
  using namespace mq;
  if (S < 0 || Kd <= 0 || (perm != nullptr && top_k <= 0)) return MQ_ERR_INVALID_ARGUMENT;
  if (shuffle < 0 || shuffle > 2) return MQ_ERR_INVALID_ARGUMENT;
  if (Kd % 128 != 0 || Kd / 128 > W_XS_STRIDE || S >= ((int64_t)1 << 30)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (shuffle == 2 && Kd / 128 > W4_XS_UNSCALE) return MQ_ERR_UNSUPPORTED_SHAPE;   // the last slot carries 2^-e
  if (S == 0) return MQ_OK;
  if (!x || !xs || !aligned16(x) || (xp && !aligned16(xp))) return MQ_ERR_INVALID_ARGUMENT;
  w4_prep_rows<<<(unsigned)((S + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), perm, (int)(perm ? top_k : 1), (int)S, (int)Kd, shuffle,
      reinterpret_cast<__nv_bfloat16*>(xp), xs);
  return check_launch();
}

static int w4_tc_launch(bool swiglu, const void* xp, const float* xs, const int32_t* qw0, const void* sc0,
                        const int32_t* qz0, const int32_t* qw1, const void* sc1, const int32_t* qz1,
                        const int32_t* offsets, int64_t S, int64_t E, int64_t period, int64_t N, int64_t Kd,
                        int64_t group_size, void* out, int32_t* d_status, void* stream) {
  using namespace mq;
  if (S < 0 || E <= 0 || N <= 0 || Kd <= 0 || period <= 0 || period > E) return MQ_ERR_INVALID_ARGUMENT;
  if (!w4_tc_covers(S, period, N, Kd, group_size)) return MQ_ERR_UNSUPPORTED_SHAPE;
  if (S == 0) return MQ_OK;
  if (!xp || !xs || !qw0 || !sc0 || !qz0 || !offsets || !out || (swiglu && (!qw1 || !sc1 || !qz1)))
    return MQ_ERR_INVALID_ARGUMENT;
  if (!aligned16(xp) || !aligned16(xs) || !aligned16(qw0) || (swiglu && !aligned16(qw1))) return MQ_ERR_INVALID_ARGUMENT;
  CUtensorMap map_x, map_w0, map_w1;
  const uint64_t wrows = (uint64_t)period * (uint64_t)(Kd / 8);
  if (!w4_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xp, (uint64_t)S, (uint64_t)Kd, 64, W_TN,
                 CU_TENSOR_MAP_SWIZZLE_128B) ||
      !w4_map_2d(&map_w0, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, qw0, wrows, (uint64_t)N, W_TM, W_GK / 8, CU_TENSOR_MAP_SWIZZLE_NONE) ||
      !w4_map_2d(&map_w1, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, swiglu ? qw1 : qw0, wrows, (uint64_t)N, W_TM, W_GK / 8,
                 CU_TENSOR_MAP_SWIZZLE_NONE))
    return MQ_ERR_DRIVER_ENTRY;
  const int64_t nwt = N / W_TM;
  const int64_t tiles_max = ((S + W_TN - 1) / W_TN + E) * nwt;
  const int grid = (int)(tiles_max < w4_sm_count() ? tiles_max : w4_sm_count());
  W4TcProj p0{reinterpret_cast<const __nv_bfloat16*>(sc0), qz0};
  W4TcProj p1{reinterpret_cast<const __nv_bfloat16*>(swiglu ? sc1 : sc0), swiglu ? qz1 : qz0};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (swiglu) {
    cudaFuncSetAttribute(w4a16_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES);
    w4a16_tc5_kernel<true><<<grid, W_THREADS, W_SMEM_BYTES, st>>>(map_x, map_w0, map_w1, p0, p1, xs, offsets, (int)E,
        (int)period, (int)S, (int)N, (int)Kd, reinterpret_cast<__nv_bfloat16*>(out), d_status);
  } else {
    cudaFuncSetAttribute(w4a16_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES);
    w4a16_tc5_kernel<false><<<grid, W_THREADS, W_SMEM_BYTES, st>>>(map_x, map_w0, map_w1, p0, p1, xs, offsets, (int)E,
        (int)period, (int)S, (int)N, (int)Kd, reinterpret_cast<__nv_bfloat16*>(out), d_status);
  }
  return check_launch();
}

extern "C" int mq_w4a16_tc_gemm(const void* xp, const float* xs, const int32_t* qweight, const void* scales,
                                const int32_t* qzeros, const int32_t* offsets, int64_t S, int64_t E,
                                int64_t weight_period, int64_t N, int64_t Kd, int64_t group_size, void* out,
                                int32_t* d_status, void* stream) {
  return w4_tc_launch(false, xp, xs, qweight, scales, qzeros, nullptr, nullptr, nullptr, offsets, S, E, weight_period,
                      N, Kd, group_size, out, d_status, stream);
}

extern "C" int mq_w4a16_tc_swiglu(const void* xp, const float* xs,
                                  const int32_t* qweight_gate, const void* scales_gate, const int32_t* qzeros_gate,
                                  const int32_t* qweight_up, const void* scales_up, const int32_t* qzeros_up,
                                  const int32_t* offsets, int64_t S, int64_t E, int64_t weight_period, int64_t I,
                                  int64_t H, int64_t group_size, void* h_shuffled, int32_t* d_status, void* stream) {
  return w4_tc_launch(true, xp, xs, qweight_gate, scales_gate, qzeros_gate, qweight_up, scales_up, qzeros_up, offsets,
                      S, E, weight_period, I, H, group_size, h_shuffled, d_status, stream);
}
