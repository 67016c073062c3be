// bf16 grouped expert GEMM on the Blackwell tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA), optionally with the gate/up SwiGLU fused into the epilogue.
// Arithmetic follows mini_qwen/kernels/moe_grouped_gemm.py:17-37 (fp32 accumulation, bf16 result)
// and mini_qwen/model/layers/moe.py:24-25 (bf16 rounding after gate, silu, up, product).
//
// Persistent kernel, one CTA per SM, 6 warps:
//   warp 0   TMA producer: A tile = 128 expert-sorted rows x 64 k, B tile = 256 weight rows x 64 k
//            (for SwiGLU: 128 gate rows followed by 128 up rows), 128-byte swizzle, 4-stage ring;
//   warp 1   MMA issuer: one thread issues tcgen05.mma 128x256x16 (cta_group::1, kind::f16) into one
//            of two 256-column TMEM accumulators, tcgen05.commit releases the ring slot / publishes
//            the accumulator;
//   warps 2-5 epilogue: tcgen05.ld (thread = row), SwiGLU or plain rounding, row-predicated
//            16-byte stores; overlaps the next tile's main loop through the second accumulator.
// Tiles are walked in (expert, n-tile, m-tile) order so that the CTAs working at the same time
// share a weight tile (read once from HBM, then from L2).  The tile list is derived on the device
// from the offsets; no host synchronisation.  A row tile that straddles the end of its expert
// computes the extra rows and masks their stores; rows past the end of the matrix are TMA zero fill.
//
// Every mbarrier wait is bounded: when it runs out the kernel sets MQ_DEV_WAIT_EXPIRED in the status
// word, all roles leave their loops, and TMEM is freed before the CTA exits.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace mq {
namespace {

constexpr int BM = 128;                 // rows (slots) per tile = TMEM lanes
constexpr int BK = 64;                  // k per stage = one 128-byte swizzle span of bf16
constexpr int BN_MAX = 256;             // accumulator columns per tile
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int B_BYTES = BN_MAX * BK * 2;    // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr int TC5_THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

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
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
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

// Walks the tile list in (expert, n-tile, m-tile) order. Every role keeps its own cursor.
struct TileCursor {
  const int32_t* off;
  int E, NT;
  int e, base;      // first tile index of expert e
  __device__ TileCursor(const int32_t* o, int E_, int NT_) : off(o), E(E_), NT(NT_), e(0), base(0) {}
  // Locates tile t (t must not decrease between calls). Returns false past the last tile.
  __device__ bool locate(int t, int& expert, int& nt, int& row0, int& row_end) {
    while (e < E) {
      const int lo = off[e], hi = off[e + 1];
      const int mt = (hi - lo + BM - 1) / BM;
      const int span = mt * NT;
      if (t < base + span) {
        const int local = t - base;
        expert = e;
        nt = local / mt;
        row0 = lo + (local - nt * mt) * BM;
        row_end = hi;
        return true;
      }
      base += span;
      ++e;
    }
    return false;
  }
};

template <bool SWIGLU>
__global__ void __launch_bounds__(TC5_THREADS, 1)
grouped_gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const int32_t* __restrict__ offsets, int E, int period, int N, int Kd, int bn,
                        __nv_bfloat16* __restrict__ out, int32_t* d_status) {
  // N: output columns. SWIGLU: weights have 2N rows per expert, a tile = 128 gate + 128 up rows (bn = 256)
  // and produces 128 output columns.  Plain: a tile = bn (128 or 256) weight rows = bn output columns.
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;                 // 1024-byte aligned for the swizzle
  uint8_t* bar_mem = smem_raw + (tiles_base - raw) + STAGES * STAGE_BYTES;
  const uint32_t bars = tiles_base + STAGES * STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem ptr, abort
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int out_cols = SWIGLU ? 128 : bn;          // output columns per tile
  const int NT = N / out_cols;
  const int KB = Kd / BK;
  const int w_rows_per_expert = SWIGLU ? 2 * N : N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128); }
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
      TileCursor cur(offsets, E, NT);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        int e, nt, row0, row_end;
        if (!cur.locate(t, e, nt, row0, row_end)) break;
        const int wrow = (e % period) * w_rows_per_expert + nt * out_cols;
        for (int kb = 0; kb < KB && ok; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, d_status);
          if (!ok) break;
          const uint32_t sa = tiles_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), (uint32_t)(A_BYTES + bn * BK * 2));
          tma_load_2d(sa, &map_a, full_bar(stage), kb * BK, row0);
          if (SWIGLU) {
            tma_load_2d(sb, &map_w, full_bar(stage), kb * BK, wrow);                     // 128 gate rows
            tma_load_2d(sb + 128 * BK * 2, &map_w, full_bar(stage), kb * BK, wrow + N);  // 128 up rows
          } else {
            tma_load_2d(sb, &map_w, full_bar(stage), kb * BK, wrow);
            if (bn == 256) tma_load_2d(sb + 128 * BK * 2, &map_w, full_bar(stage), kb * BK, wrow + 128);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      // drain: wait until the MMA warp has consumed everything that was loaded, so that no bulk copy is
      // still writing shared memory when the CTA exits
      for (int s = 0; s < STAGES && ok; ++s) {
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, d_status);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      TileCursor cur(offsets, E, NT);
      const uint32_t idesc = umma_idesc(bn);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        int e, nt, row0, row_end;
        if (!cur.locate(t, e, nt, row0, row_end)) break;
        ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, d_status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN_MAX);
        for (int kb = 0; kb < KB; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, d_status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * STAGE_BYTES;
          const uint64_t adesc = umma_desc(sa);
          const uint64_t bdesc = umma_desc(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 k = 32 bytes along the swizzled row: +2 in the (address >> 4) field
            umma_f16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));          // frees the ring slot once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));              // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    TileCursor cur(offsets, E, NT);
    const int quad = warp & 3;                     // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok; t += gridDim.x) {
      int e, nt, row0, row_end;
      if (!cur.locate(t, e, nt, row0, row_end)) break;
      ok = __all_sync(0xffffffffu, mbar_wait(tfull_bar(acc), acc_phase, abort_flag, d_status));
      if (!ok) break;
      tc_fence_after();
      const int row = row0 + row_in_tile;
      const bool row_ok = row < row_end;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN_MAX);
      __nv_bfloat16* orow = out + (size_t)row * N + (size_t)nt * out_cols;
      for (int c = 0; c < out_cols; c += 32) {
        uint32_t g[32];
        uint32_t packed[16];
        tmem_ld32(taddr + c, g);
        if (SWIGLU) {
          uint32_t u[32];
          tmem_ld32(taddr + 128 + c, u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float o0 = swiglu_rounded<__nv_bfloat16>(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j]));
            float o1 = swiglu_rounded<__nv_bfloat16>(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1]));
            __nv_bfloat162 p = __floats2bfloat162_rn(o0, o1);
            packed[j] = *reinterpret_cast<uint32_t*>(&p);
          }
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1]));
            packed[j] = *reinterpret_cast<uint32_t*>(&p);
          }
        }
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c);
#pragma unroll
          for (int v = 0; v < 4; ++v)
            dst[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
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

// 2-D bf16 row-major [rows, cols] tensor, box = 64 columns x 128 rows, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, 128u};
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

int grouped_gemm_tc5(const void* a, const void* w, const int32_t* offsets, int64_t S, int64_t E, int64_t period,
                     int64_t N, int64_t Kd, bool swiglu, void* out, int32_t* d_status, cudaStream_t st) {
  CUtensorMap map_a, map_w;
  const int64_t w_rows = period * (swiglu ? 2 * N : N);
  if (!make_map(&map_a, a, (uint64_t)S, (uint64_t)Kd) || !make_map(&map_w, w, (uint64_t)w_rows, (uint64_t)Kd))
    return MQ_ERR_DRIVER_ENTRY;
  const int bn = swiglu ? 256 : (N % 256 == 0 ? 256 : 128);
  const int out_cols = swiglu ? 128 : bn;
  const int64_t tiles_max = ((S + BM - 1) / BM + E) * (N / out_cols);
  const int grid = (int)(tiles_max < sm_count() ? tiles_max : sm_count());
  // the attribute is per device; setting it is cheap, so it is set on every call
  if (swiglu) {
    cudaFuncSetAttribute(grouped_gemm_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    grouped_gemm_tc5_kernel<true><<<grid, TC5_THREADS, SMEM_BYTES, st>>>(map_a, map_w, offsets, (int)E, (int)period, (int)N,
        (int)Kd, bn, reinterpret_cast<__nv_bfloat16*>(out), d_status);
  } else {
    cudaFuncSetAttribute(grouped_gemm_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    grouped_gemm_tc5_kernel<false><<<grid, TC5_THREADS, SMEM_BYTES, st>>>(map_a, map_w, offsets, (int)E, (int)period, (int)N,
        (int)Kd, bn, reinterpret_cast<__nv_bfloat16*>(out), d_status);
  }
  return check_launch();
}

}  // namespace mq
