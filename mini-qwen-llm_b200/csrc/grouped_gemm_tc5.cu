// bf16 grouped expert GEMM on the Blackwell tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA), optionally with the gate/up SwiGLU fused into the epilogue.
// Arithmetic follows mini_qwen/kernels/moe_grouped_gemm.py:17-37 (fp32 accumulation, bf16 result)
// and mini_qwen/model/layers/moe.py:24-25 (bf16 rounding after gate, silu, up, product).
//
// Orientation: the WEIGHT rows are the 128-lane M dimension of the MMA and the TOKENS are its N
// dimension (16..256 in steps of 16).  An expert's row count is ragged; making it the N dimension
// means a tile is exactly as wide as the expert needs (no 128-row padding), and a decode batch with
// a handful of rows per expert still streams every weight byte exactly once.
//
// A tile = two weight sub-tiles of 128 rows that share one token tile:
//   SwiGLU: 128 gate rows + the matching 128 up rows  -> 128 output columns of h
//   plain : rows [f0, f0+128) and [f0+128, f0+256)    -> 256 output columns
// so each token tile fetched through L2 feeds two MMAs (64 KB of operands per 1024 MMA cycles at
// 256 tokens, against 48 KB per 512 cycles for a single 128x256 tile: the kernel is bound by the
// per-SM L2 bandwidth, not by the tensor pipe).  The two fp32 accumulators take all 512 TMEM
// columns, so a tile's epilogue does not overlap the next tile's MMAs; the TMA ring keeps loading
// meanwhile and eight epilogue warps keep the drain short.
//
// Persistent kernel, one CTA per SM, 10 warps:
//   warp 0     TMA producer (3-stage ring, 128-byte swizzle, K-major operands);
//   warp 1     MMA issuer: one thread, tcgen05.mma.cta_group::1.kind::f16, M=128, N=tokens, K=16;
//   warps 2-9  epilogue: tcgen05.ld (lane = output column, TMEM column = token), SwiGLU / rounding,
//              stores of 32 adjacent columns per warp and token.
// Tiles are walked in (expert, token tile, weight tile) order: CTAs running at the same time share
// the token rows of an expert through L2 and every weight tile is read from HBM once.
//
// Every mbarrier wait is bounded: when it runs out the kernel sets MQ_DEV_WAIT_EXPIRED in the status
// word, all roles leave their loops, and TMEM is freed before the CTA exits.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace mq {
namespace {

constexpr int TM = 128;                 // weight rows per sub-tile = TMEM lanes
constexpr int BK = 64;                  // k per stage = one 128-byte swizzle span of bf16
constexpr int TN_MAX = 256;             // tokens per tile (MMA N)
constexpr int STAGES = 3;
constexpr int A_BYTES = TM * BK * 2;            // 16 KB per weight sub-tile
constexpr int B_BYTES = TN_MAX * BK * 2;        // 32 KB token tile
constexpr int BOX_TOK = 64;                     // token rows per TMA box
constexpr int BOX_TOK_BYTES = BOX_TOK * BK * 2; // 8 KB
constexpr int STAGE_BYTES = 2 * A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int GATHER_WARPS = 4;                 // producer warps that gather token rows (fused-permute variant)
constexpr int STG_ROWS = 32;                    // token rows per epilogue chunk
constexpr int STG_PITCH_MAX = 2 * TM * 2;       // bytes per staged token row: up to 256 bf16 output columns
constexpr int STG_BYTES = STG_ROWS * STG_PITCH_MAX;   // per group of four epilogue warps
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + (EPI_WARPS / 4) * STG_BYTES;
constexpr int TC5_THREADS = (2 + EPI_WARPS) * 32;
constexpr int TC5_GATHER_THREADS = (2 + EPI_WARPS + GATHER_WARPS) * 32;
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr int ROW_BITS = 26;                    // scattered output: destination code = buffer << 26 | row
constexpr int ROW_MASK = (1 << ROW_BITS) - 1;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// Bounded wait. Returns false when the wait ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* d_status) {
  for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (d_status != nullptr) atomicOr(d_status, (int)MQ_DEV_WAIT_EXPIRED);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// Untiled bulk store of `bytes` contiguous bytes from shared memory (both addresses 16-byte aligned); the
// destination may be another GPU's memory (a plain store, nothing is read from the peer).
__device__ __forceinline__ void bulk_store_1d(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the stores issued by this thread have finished READING their shared-memory source
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Makes this thread's completed shared-memory writes visible to the async proxy (the tensor core reads).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row
// groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}

// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 16 TMEM lanes x 32 columns in the fragment layout of an m16n8 accumulator, four 8-column blocks:
// thread T holds, for block i, r[4i], r[4i+1] = lane T/4, columns 8i + 2(T%4), +1 and r[4i+2], r[4i+3] =
// lane T/4 + 8, same columns.  With output columns in the lanes and tokens in the columns, a pair of
// registers is two consecutive tokens of one output column: packed to bf16 it is the fragment
// stmatrix.trans turns into token-major rows.
__device__ __forceinline__ void tmem_ld_frag(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// Four 8x8 bf16 matrices, stored transposed: lane L gives the address of row L%8 of matrix L/8.
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t saddr, uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};"
               ::"r"(saddr), "r"(m0), "r"(m1), "r"(m2), "r"(m3) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(uint32_t lo_bits, uint32_t hi_bits) {
  const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(lo_bits), __uint_as_float(hi_bits));
  return *reinterpret_cast<const uint32_t*>(&p);
}

// SwiGLU of two accumulator pairs with the rounding points of the op-by-op bf16 path (g, silu(g), u
// and the product are each rounded to bf16); exp and the reciprocal use the SFU approximations,
// whose error (2^-21) is far below the bf16 rounding that follows.  Returns the packed bf16 pair.
__device__ __forceinline__ uint32_t swiglu_pair(float g0, float g1, float u0, float u1) {
  const __nv_bfloat162 gb = __floats2bfloat162_rn(g0, g1);
  const __nv_bfloat162 ub = __floats2bfloat162_rn(u0, u1);
  const float2 gf = __bfloat1622float2(gb);
  const float2 uf = __bfloat1622float2(ub);
  const float s0 = __fdividef(gf.x, 1.0f + __expf(-gf.x));
  const float s1 = __fdividef(gf.y, 1.0f + __expf(-gf.y));
  const float2 sf = __bfloat1622float2(__floats2bfloat162_rn(s0, s1));
  const __nv_bfloat162 o = __floats2bfloat162_rn(sf.x * uf.x, sf.y * uf.y);
  return *reinterpret_cast<const uint32_t*>(&o);
}

// Barrier among the four epilogue warps that drain the same 32-token chunks (ids 1 and 2; 0 is __syncthreads).
__device__ __forceinline__ void epi_group_sync(int group) {
  asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
}

// One tile of work.
struct Tile {
  int expert;     // group index (weights: expert % period)
  int wt;         // weight tile index
  int lo;         // first row of the group
  int tok0;       // first row of the token tile
  int tok_end;    // one past the last valid row (end of the tile or of the expert)
  int n_mma;      // MMA N: rows of the token tile rounded up to 16
};

// Walks the tile list in (expert, token tile, weight tile) order. Every role keeps its own cursor.
struct TileCursor {
  const int32_t* off;
  int E, NWT;
  int e, base;      // first tile index of expert e
  __device__ TileCursor(const int32_t* o, int E_, int NWT_) : off(o), E(E_), NWT(NWT_), e(0), base(0) {}
  // Locates tile t (t must not decrease between calls). Returns false past the last tile.
  __device__ bool locate(int t, Tile& tile) {
    while (e < E) {
      const int lo = off[e], hi = off[e + 1];
      const int n = hi - lo;
      const int ntt = (n + TN_MAX - 1) / TN_MAX;
      const int span = ntt * NWT;
      if (t < base + span) {
        const int local = t - base;
        const int tt = local / NWT;
        const int width = (((n + ntt - 1) / ntt) + 15) & ~15;     // balanced token tiles, multiple of 16
        tile.expert = e;
        tile.lo = lo;
        tile.wt = local - tt * NWT;
        tile.tok0 = lo + tt * width;
        tile.tok_end = min(tile.tok0 + width, hi);
        tile.n_mma = (tile.tok_end - tile.tok0 + 15) & ~15;
        return true;
      }
      base += span;
      ++e;
    }
    return false;
  }
};

// GATHER: the token operand is not read from expert-sorted rows but gathered from the unpermuted
// activations x [T, Kd]: sorted row p is x[perm[p] / top_k].  Four extra producer warps copy the rows
// with 16-byte cp.async into the 128-byte-swizzled layout the MMA expects (chunk c of row r lands at
// chunk c ^ (r & 7)), one commit group per k-block; when a group has landed the thread fences towards
// the async proxy and arrives on the stage's barrier.  Weights still come by TMA.
// DOUBLE (plain projection only): a tile is ONE 128-row weight sub-tile, so an accumulator takes 256 of
// the 512 TMEM columns and tiles alternate between two of them: the epilogue of a tile (and its stores,
// which may be NVLink stores to another GPU) runs under the next tile's MMAs.  The ring then has four
// stages of 48 KB.
template <bool SWIGLU, bool GATHER, bool DOUBLE>
__global__ void __launch_bounds__(GATHER ? TC5_GATHER_THREADS : TC5_THREADS, 1)
grouped_gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                        const int32_t* __restrict__ offsets, int E, int period, int N, int Kd,
                        const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ perm, int top_k,
                        __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ row_dst,
                        const uint64_t* __restrict__ dst_bases, int32_t* d_status) {
  // row_dst == nullptr: row r of the input produces row r of `out`.  Otherwise row r is written to row
  // (row_dst[r] & ROW_MASK) of the buffer at dst_bases[row_dst[r] >> ROW_BITS], which may be another
  // GPU's memory: the epilogue's stores then travel over NVLink while later tiles compute.
  // N: output columns.  SWIGLU: the weights hold 2N rows per expert (gate rows, then up rows).
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;                 // 1024-byte aligned for the swizzle
  static_assert(!(SWIGLU && DOUBLE), "the SwiGLU tile needs both accumulators");
  constexpr int NST = DOUBLE ? 4 : STAGES;                                  // ring stages
  constexpr int SBYTES = DOUBLE ? A_BYTES + B_BYTES : STAGE_BYTES;          // bytes per stage
  constexpr int B_OFF = DOUBLE ? A_BYTES : 2 * A_BYTES;                     // token tile inside a stage
  static_assert(NST * SBYTES == STAGES * STAGE_BYTES, "both ring shapes fill the same shared memory");
  uint8_t* bar_mem = smem_raw + (tiles_base - raw) + NST * SBYTES;
  const uint32_t bars = tiles_base + NST * SBYTES;
  // barriers (8 bytes each): full[NST], empty[NST], tmem_full[2], tmem_empty[2]; then tmem pointer, abort
  // flag, the epilogue groups' go flags
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (NST + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * NST + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * NST + 2 + b); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * (2 * NST + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * (2 * NST + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cols_per_tile = (SWIGLU || DOUBLE) ? TM : 2 * TM;      // output columns per tile
  const int NWT = (N + cols_per_tile - 1) / cols_per_tile;
  const int KB = Kd / BK;
  const int w_rows_per_expert = SWIGLU ? 2 * N : N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(full_bar(s), GATHER ? 1 + GATHER_WARPS * 32 : 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), EPI_WARPS * 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32((const void*)tmem_ptr_smem)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      TileCursor cur(offsets, E, NWT);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tl;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        if (!cur.locate(t, tl)) break;
        const int f0 = tl.wt * cols_per_tile;
        const int wbase = (tl.expert % period) * w_rows_per_expert;
        const int wrow0 = wbase + f0;
        const int wrow1 = SWIGLU ? wbase + N + f0 : wbase + f0 + TM;
        const bool two = !DOUBLE && (SWIGLU || (f0 + TM < N));
        const int nbox = (tl.n_mma + BOX_TOK - 1) / BOX_TOK;
        const uint32_t tx = (uint32_t)((two ? 2 : 1) * A_BYTES + (GATHER ? 0 : nbox * BOX_TOK_BYTES));
        for (int kb = 0; kb < KB && ok; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, d_status);
          if (!ok) break;
          const uint32_t sa0 = tiles_base + stage * SBYTES;
          const uint32_t sa1 = sa0 + A_BYTES;
          const uint32_t sb = sa0 + B_OFF;
          mbar_expect_tx(full_bar(stage), tx);
          tma_load_2d(sa0, &map_w, full_bar(stage), kb * BK, wrow0);
          if (two) tma_load_2d(sa1, &map_w, full_bar(stage), kb * BK, wrow1);
          if (!GATHER) {
            for (int b = 0; b < nbox; ++b)
              tma_load_2d(sb + b * BOX_TOK_BYTES, &map_x, full_bar(stage), kb * BK, tl.tok0 + b * BOX_TOK);
          }
          if (++stage == NST) { stage = 0; phase ^= 1u; }
        }
      }
      // drain: wait until the MMA warp has consumed everything that was loaded, so that no bulk copy is
      // still writing shared memory when the CTA exits
      for (int s = 0; s < NST && ok; ++s) {
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, d_status);
        if (++stage == NST) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      TileCursor cur(offsets, E, NWT);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      Tile tl;
      int it = 0;                                  // tiles this CTA has started
      for (int t = blockIdx.x; ok; t += gridDim.x, ++it) {
        if (!cur.locate(t, tl)) break;
        const bool two = !DOUBLE && (SWIGLU || (tl.wt * cols_per_tile + TM < N));
        const uint32_t idesc = umma_idesc(tl.n_mma);
        const int buf = DOUBLE ? (it & 1) : 0;     // accumulator of this tile
        const uint32_t acc_phase = (uint32_t)((DOUBLE ? (it >> 1) : it) & 1);
        const uint32_t acc = tmem_base + buf * TN_MAX;
        ok = mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, d_status);   // epilogue has drained it
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, d_status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa0 = tiles_base + stage * SBYTES;
          const uint64_t a0 = umma_desc(sa0);
          const uint64_t a1 = umma_desc(sa0 + A_BYTES);
          const uint64_t bd = umma_desc(sa0 + B_OFF);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 k = 32 bytes along the swizzled row: +2 in the (address >> 4) field
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            umma_f16(acc, a0 + 2u * k, bd + 2u * k, idesc, accum);
            if (two) umma_f16(acc + TN_MAX, a1 + 2u * k, bd + 2u * k, idesc, accum);
          }
          umma_commit(empty_bar(stage));          // frees the ring slot once these MMAs have read it
          if (++stage == NST) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(buf));              // accumulators complete
      }
    }
  } else if (GATHER && warp >= 2 + EPI_WARPS) {
    // ------------------------------------------------------------------ gather producers (warps 10..13)
    const int gt = threadIdx.x - (2 + EPI_WARPS) * 32;       // 0 .. 127
    const int chunk = gt & 7;                                // 16-byte piece of a 128-byte row
    const int rbase = gt >> 3;                               // rows rbase, rbase+16, ... of the tile
    TileCursor cur(offsets, E, NWT);
    int stage = 0, prev_stage = -1;
    uint32_t phase = 0;
    bool ok = true;
    // The sorted positions of the NEXT tile are fetched while the current tile is copied, so that the
    // dependent perm loads never sit between two k-blocks of the ring.
    Tile tl, nx;
    int slot[TN_MAX / 16], slot_nx[TN_MAX / 16];
    auto fetch_slots = [&](const Tile& tile, int (&dst)[TN_MAX / 16]) {
#pragma unroll
      for (int i = 0; i < TN_MAX / 16; ++i)   // rows past the end of the expert repeat its last row: computed, never stored
        dst[i] = perm[min(tile.tok0 + rbase + 16 * i, tile.tok_end - 1)];
    };
    int t = blockIdx.x;
    bool have = cur.locate(t, tl);
    if (have) fetch_slots(tl, slot);
    while (have && ok) {
      t += gridDim.x;
      const bool have_nx = cur.locate(t, nx);
      if (have_nx) fetch_slots(nx, slot_nx);
      uint32_t src_off[TN_MAX / 16];           // element offset of this thread's piece of each row in x
#pragma unroll
      for (int i = 0; i < TN_MAX / 16; ++i) src_off[i] = (uint32_t)(slot[i] / top_k) * (uint32_t)Kd + chunk * 8;
      const int nrow = tl.n_mma;                             // rows the MMA reads (multiple of 16)
      for (int kb = 0; kb < KB && ok; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, d_status));
        if (!ok) break;
        const uint32_t sb = tiles_base + stage * SBYTES + B_OFF;
#pragma unroll
        for (int i = 0; i < TN_MAX / 16; ++i) {
          const int r = rbase + 16 * i;
          if (r < nrow)
            cp_async16(sb + (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4), x + src_off[i] + kb * BK);
        }
        cp_async_commit();
        if (prev_stage >= 0) {                               // the previous k-block's rows have landed
          cp_async_wait<1>();
          fence_proxy_async();
          mbar_arrive(full_bar(prev_stage));
        }
        prev_stage = stage;
        if (++stage == NST) { stage = 0; phase ^= 1u; }
      }
      have = have_nx;
      tl = nx;
#pragma unroll
      for (int i = 0; i < TN_MAX / 16; ++i) slot[i] = slot_nx[i];
    }
    cp_async_wait<0>();
    if (prev_stage >= 0 && ok) {
      fence_proxy_async();
      mbar_arrive(full_bar(prev_stage));
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    // Warps 2..5 drain the even 32-token chunks of a tile, warps 6..9 the odd ones.  The four warps of
    // a group hold one TMEM lane quadrant (32 output columns) each; they put their blocks side by side
    // into the group's staging rows, then every warp writes whole rows: 256 (SwiGLU) or 512 bytes of
    // one token row per store instruction, which is what a remote destination over NVLink wants.
    TileCursor cur(offsets, E, NWT);
    const int quad = warp & 3;                     // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;              // which 32-token chunks (even / odd) this group drains
    const int wig = (warp - 2) & 3;                // warp within the group: stores rows 8*wig .. 8*wig+7
    uint8_t* stg = bar_mem + 256 + half * STG_BYTES;
    volatile int* group_go = reinterpret_cast<volatile int*>(bar_mem + 8 * (2 * NST + 4) + 16) + half;
    // Rows that are scattered (expert parallelism: each goes to the GPU and row its code names) leave by bulk
    // stores, one 256-byte row per elected lane: the copy engine moves them while the warps go on, and a peer
    // receives whole rows instead of 16-byte pieces.  A bulk store reads its row as it lies in shared memory, so
    // the staging rows are then unswizzled and padded by 16 bytes instead (272-byte pitch: conflict-free too).
    const bool bulk_rows = DOUBLE && row_dst != nullptr;
    const int pitch = bulk_rows ? cols_per_tile * 2 + 16 : cols_per_tile * 2;
    Tile tl;
    int it = 0;
    for (int t = blockIdx.x;; t += gridDim.x, ++it) {
      if (!cur.locate(t, tl)) break;
      const int buf = DOUBLE ? (it & 1) : 0;
      const uint32_t acc_phase = (uint32_t)((DOUBLE ? (it >> 1) : it) & 1);
      mbar_wait(tfull_bar(buf), acc_phase, abort_flag, d_status);
      // the four warps must take the same decision, or the group barriers below would never fill
      epi_group_sync(half);
      if (wig == 0 && lane == 0) *group_go = (*abort_flag == 0);
      epi_group_sync(half);
      if (*group_go == 0) break;
      tc_fence_after();
      const int f0 = tl.wt * cols_per_tile;
      const bool two = !DOUBLE && (SWIGLU || (f0 + TM < N));
      const int ntok = tl.tok_end - tl.tok0;
      for (int c = half * 32; c < tl.n_mma; c += 64) {
        // The accumulators leave TMEM in fragment layout (16 output columns x 32 tokens per load) and go
        // into the staging rows through stmatrix.trans: token-major rows of 16-byte pieces (8 output
        // columns), piece index XORed with the token's low bits so that stores and loads are conflict-free.
        const uint32_t stg_s = smem_u32(stg);
        const int mi = lane >> 3, ri = lane & 7;       // stmatrix: this lane addresses row ri of matrix mi
#pragma unroll
        for (int hl = 0; hl < 2; ++hl) {               // the two 16-lane halves of the warp's TMEM quadrant
          const uint32_t ta = tmem_base + buf * TN_MAX + ((uint32_t)(quad * 32 + 16 * hl) << 16) + c;
          uint32_t f0r[16], f1r[16];
          tmem_ld_frag(ta, f0r);
          if (two) tmem_ld_frag(ta + TN_MAX, f1r);
          tmem_ld_wait();
#pragma unroll
          for (int sub2 = 0; sub2 < ((SWIGLU || !two) ? 1 : 2); ++sub2) {
            uint32_t m[4][2];                           // [token octet][output-column octet]
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int a = 0; a < 2; ++a) {
                if (SWIGLU)
                  m[i][a] = swiglu_pair(__uint_as_float(f0r[4 * i + 2 * a]), __uint_as_float(f0r[4 * i + 2 * a + 1]),
                                        __uint_as_float(f1r[4 * i + 2 * a]), __uint_as_float(f1r[4 * i + 2 * a + 1]));
                else
                  m[i][a] = sub2 == 0 ? pack_bf16x2(f0r[4 * i + 2 * a], f0r[4 * i + 2 * a + 1])
                                      : pack_bf16x2(f1r[4 * i + 2 * a], f1r[4 * i + 2 * a + 1]);
              }
            // two stores of four matrices: token octets (0,1) and (2,3), each with both column octets
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
              const int tok = 8 * (2 * j2 + (mi >> 1)) + ri;                       // token row of the chunk
              const int piece = (sub2 * TM + quad * 32 + 16 * hl + 8 * (mi & 1)) >> 3;   // 16-byte piece of the row
              const uint32_t addr = stg_s + tok * pitch + ((bulk_rows ? piece : (piece ^ (tok & 7))) << 4);
              stmatrix_x4_trans(addr, m[2 * j2][0], m[2 * j2][1], m[2 * j2 + 1][0], m[2 * j2 + 1][1]);
            }
          }
        }
        const int valid = ntok - c;                    // token rows of this chunk that exist
        // where this warp's rows go: fetched before the barrier so that the lookups overlap the wait
        constexpr int RPI = (SWIGLU || DOUBLE) ? 2 : 1;       // rows per store instruction
        const int sub = RPI == 2 ? (lane >> 4) : 0;
        __nv_bfloat16* orow[8 / RPI];
#pragma unroll
        for (int i = 0; i < 8 / RPI; ++i) {
          const int row = 8 * wig + RPI * i + sub;
          const int64_t r = (int64_t)tl.tok0 + c + row;
          if (row_dst == nullptr) {
            orow[i] = out + (size_t)r * N + f0;
          } else {
            const int code = row < valid ? row_dst[r] : 0;
            orow[i] = reinterpret_cast<__nv_bfloat16*>(dst_bases[code >> ROW_BITS]) + (size_t)(code & ROW_MASK) * N + f0;
          }
        }
        epi_group_sync(half);                          // the chunk's rows are complete
        if (bulk_rows) {
          // lanes 0-7 of each warp send one row each; everyone waits until the copy engine has read them
          if (lane < 8) {
            const int row = 8 * wig + lane;
            if (row < valid) {
              const int code = row_dst[(int64_t)tl.tok0 + c + row];
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(dst_bases[code >> ROW_BITS]) +
                                   (size_t)(code & ROW_MASK) * N + f0;
              fence_proxy_async();                       // the staged rows (generic proxy) before the copy engine reads them
              bulk_store_1d(dst, stg_s + row * pitch, (uint32_t)(cols_per_tile * 2));
            }
            bulk_store_commit();
            bulk_store_wait_read();
          }
        } else if (SWIGLU || DOUBLE) {
          // 16 lanes cover a 256-byte row: two rows per instruction
          const int piece = lane & 15;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = 8 * wig + 2 * i + sub;
            if (row < valid) {
              const uint4 v = *reinterpret_cast<const uint4*>(stg + row * pitch + ((piece ^ (row & 7)) << 4));
              *reinterpret_cast<uint4*>(orow[i] + piece * 8) = v;
            }
          }
        } else {
          const bool col_ok = two || lane < 16;        // the last weight tile may hold one sub-tile only
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = 8 * wig + i;
            if (row < valid && col_ok) {
              const uint4 v = *reinterpret_cast<const uint4*>(stg + row * pitch + ((lane ^ (row & 7)) << 4));
              *reinterpret_cast<uint4*>(orow[i] + lane * 8) = v;
            }
          }
        }
        epi_group_sync(half);                          // the staging rows may be overwritten
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 row-major [rows, cols] tensor, box = 64 columns x box_rows rows, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int sm_count() {
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

bool tc5_covers(int64_t S, int64_t E, int64_t N, int64_t Kd, bool swiglu) {
  if (Kd % BK != 0 || Kd < BK) return false;
  if (N % 128 != 0) return false;
  // coordinates and tile counts are 32-bit
  if (S >= ((int64_t)1 << 30) || E * N * 2 >= ((int64_t)1 << 31)) return false;
  (void)swiglu;
  return true;
}

// perm == nullptr: `a` holds the S expert-sorted rows.  perm != nullptr: `a` holds the unpermuted rows and
// sorted row p is a[perm[p] / top_k], gathered inside the kernel.
int grouped_gemm_tc5(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E, int64_t period,
                     int64_t N, int64_t Kd, bool swiglu, void* out, int32_t* d_status, cudaStream_t st,
                     const int32_t* perm, int64_t top_k, const int32_t* row_dst, const uint64_t* dst_bases) {
  CUtensorMap map_x, map_w;
  const int64_t w_rows = period * (swiglu ? 2 * N : N);
  const bool gather = perm != nullptr;
  // the gathering variant does not use map_x; it still needs a valid descriptor argument
  if (!make_map(&map_x, a, (uint64_t)(gather ? BOX_TOK : S), (uint64_t)Kd, BOX_TOK) ||
      !make_map(&map_w, w, (uint64_t)w_rows, (uint64_t)Kd, TM))
    return MQ_ERR_DRIVER_ENTRY;
  // one weight sub-tile per tile with alternating accumulators when the output rows leave the GPU
  // (measured on this layer: 114 us against 128 us with the two-sub-tile shape when half of the rows go
  // to a peer; for local output the two-sub-tile shape is the faster one, 115 us against 121 us)
  const bool dbl = !swiglu && !gather && row_dst != nullptr;
  const int64_t cols_per_tile = (swiglu || dbl) ? TM : 2 * TM;
  const int64_t nwt = (N + cols_per_tile - 1) / cols_per_tile;
  const int64_t tiles_max = ((S + TN_MAX - 1) / TN_MAX + E) * nwt;
  // gathering: the number of slots is offsets[E], known only on the device (it is not T * top_k when the
  // rows are a receive buffer addressed through a slot table), so the grid is not trimmed
  const int grid = (int)(!gather && tiles_max < sm_count() ? tiles_max : sm_count());
  const __nv_bfloat16* xa = reinterpret_cast<const __nv_bfloat16*>(a);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  // the attribute is per device; setting it is cheap, so it is set on every call
#define MQ_TC5_LAUNCH(SW, GA, DB, THREADS)                                                                          \
  do {                                                                                                              \
    cudaFuncSetAttribute(grouped_gemm_tc5_kernel<SW, GA, DB>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                         SMEM_BYTES);                                                                               \
    grouped_gemm_tc5_kernel<SW, GA, DB><<<grid, THREADS, SMEM_BYTES, st>>>(map_x, map_w, offsets, (int)E,           \
        (int)period, (int)N, (int)Kd, xa, perm, (int)top_k, o, row_dst, dst_bases, d_status);                                \
  } while (0)
  if (swiglu && gather) MQ_TC5_LAUNCH(true, true, false, TC5_GATHER_THREADS);
  else if (swiglu) MQ_TC5_LAUNCH(true, false, false, TC5_THREADS);
  else if (gather) MQ_TC5_LAUNCH(false, true, false, TC5_GATHER_THREADS);
  else if (dbl) MQ_TC5_LAUNCH(false, false, true, TC5_THREADS);
  else MQ_TC5_LAUNCH(false, false, false, TC5_THREADS);
#undef MQ_TC5_LAUNCH
  return check_launch();
}

}  // namespace mq
