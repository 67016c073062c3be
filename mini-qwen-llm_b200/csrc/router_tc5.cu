// Router logits on the 5th-generation tensor cores: logits[slice][t][e] = sum over the slice's k of
// x[t,k] * w[e,k], fp32 (mini_qwen/kernels/moe_router.py:7-22 computes F.linear in fp32).
//
// CTA = 128 tokens (the TMEM lanes) x up to 128 experts (MMA N) x one K slice.  Both operands arrive by
// TMA (128-byte swizzle, 64 k per stage).  Products of 16-bit inputs are exact in the tensor core; to
// keep the accumulation as accurate as an fp32 FMA chain, a TMEM accumulator only ever sums 128 k
// (8 MMAs) and is then added to master accumulators in registers with ordinary fp32 adds: the same
// chunking, in the same order, as the mma.sync kernel in router.cu, which this kernel replaces for
// batches of 256 tokens and more.  Two TMEM accumulators alternate, so the fold of one chunk runs
// under the MMAs of the next.  All waits are bounded.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace mq {
namespace {

constexpr int RT_TM = 128;                      // tokens per CTA = TMEM lanes
constexpr int RT_BK = 64;                       // k per stage
constexpr int RT_STAGES = 4;
constexpr int RT_X_BYTES = RT_TM * RT_BK * 2;   // 16 KB
constexpr int RT_W_BYTES = 128 * RT_BK * 2;     // 16 KB (up to 128 experts)
constexpr int RT_STAGE_BYTES = RT_X_BYTES + RT_W_BYTES;
constexpr int RT_FOLD_WARPS = 8;
constexpr int RT_THREADS = (2 + RT_FOLD_WARPS) * 32;   // 320
constexpr int RT_SMEM_BYTES = RT_STAGES * RT_STAGE_BYTES + 1024 + 256;
constexpr int RT_TMEM_COLS = 256;               // two accumulators of 128 columns
constexpr uint32_t RT_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t rt_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rt_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void rt_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void rt_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool rt_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; false when it ran out or another role already gave up (the CTA then writes NaN logits).
__device__ __forceinline__ bool rt_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t spin = 0; spin < RT_SPIN_LIMIT; ++spin) {
    if (rt_mbar_try_wait(bar, parity)) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void rt_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void rt_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void rt_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ uint64_t rt_umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D fp32; A and B both bf16 (fmt 1) or both fp16 (fmt 0), K-major; M = 128, N = n.
__device__ __forceinline__ uint32_t rt_umma_idesc(int n, uint32_t fmt) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(RT_TM >> 4) << 24);
}
__device__ __forceinline__ void rt_umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void rt_umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void rt_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void rt_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(RT_THREADS, 1)
router_logits_tc5_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         int is_bf16, int T, int H, int E, int n_mma, int k_per_slice, float* __restrict__ logits) {
  extern __shared__ uint8_t rt_smem_raw[];
  const uint32_t raw = rt_smem_u32(rt_smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  uint8_t* bar_mem = rt_smem_raw + (ring - raw) + RT_STAGES * RT_STAGE_BYTES;
  const uint32_t bars = ring + RT_STAGES * RT_STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (RT_STAGES + s); };
  auto chunk_full = [&](int b) { return bars + 8u * (2 * RT_STAGES + b); };
  auto chunk_empty = [&](int b) { return bars + 8u * (2 * RT_STAGES + 2 + b); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(bar_mem + 8 * (2 * RT_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * (2 * RT_STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * RT_TM;
  const int k_lo = blockIdx.y * k_per_slice;
  const int k_hi = min(k_lo + k_per_slice, H);
  const int nkb = k_lo < k_hi ? (k_hi - k_lo) / RT_BK : 0;      // slices are multiples of 128 k, H of 64
  const int nchunk = (nkb + 1) / 2;                              // 128-k chunks (the last may be 64 k)

  if (threadIdx.x == 0) {
    for (int s = 0; s < RT_STAGES; ++s) {
      rt_mbar_init(full_bar(s), 1);
      rt_mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      rt_mbar_init(chunk_full(b), 1);
      rt_mbar_init(chunk_empty(b), RT_FOLD_WARPS * 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(rt_smem_u32((const void*)tmem_ptr_smem)), "r"((uint32_t)RT_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  rt_fence_before();
  __syncthreads();
  rt_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- producer
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % RT_STAGES;
        ok = rt_mbar_wait(empty_bar(s), (uint32_t)((kb / RT_STAGES) & 1) ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t st = ring + s * RT_STAGE_BYTES;
        rt_mbar_expect_tx(full_bar(s), (uint32_t)(RT_X_BYTES + n_mma * RT_BK * 2));
        rt_tma_load_2d(st, &map_x, full_bar(s), k_lo + kb * RT_BK, t0);
        rt_tma_load_2d(st + RT_X_BYTES, &map_w, full_bar(s), k_lo + kb * RT_BK, 0);
      }
      // drain: every stage that was filled has been consumed before the CTA exits
      for (int kb = max(0, nkb - RT_STAGES); kb < nkb && ok; ++kb)
        ok = rt_mbar_wait(empty_bar(kb % RT_STAGES), (uint32_t)((kb / RT_STAGES) & 1), abort_flag);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      const uint32_t idesc = rt_umma_idesc(n_mma, is_bf16 ? 1u : 0u);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % RT_STAGES;
        const int ch = kb >> 1, b = ch & 1;
        if ((kb & 1) == 0) {                        // a new 128-k chunk: its accumulator must have been read
          ok = rt_mbar_wait(chunk_empty(b), (uint32_t)((ch >> 1) & 1) ^ 1u, abort_flag);
          if (!ok) break;
        }
        ok = rt_mbar_wait(full_bar(s), (uint32_t)((kb / RT_STAGES) & 1), abort_flag);
        if (!ok) break;
        rt_fence_after();
        const uint32_t st = ring + s * RT_STAGE_BYTES;
        const uint64_t ad = rt_umma_desc(st), bd = rt_umma_desc(st + RT_X_BYTES);
#pragma unroll
        for (int k = 0; k < RT_BK / 16; ++k)
          rt_umma(tmem_base + b * 128, ad + 2u * k, bd + 2u * k, idesc, ((kb & 1) | k) != 0 ? 1u : 0u);
        rt_umma_commit(empty_bar(s));
        if ((kb & 1) == 1 || kb == nkb - 1) rt_umma_commit(chunk_full(b));
      }
    }
  } else {
    // ------------------------------------------------------------------ fold warps (2..9)
    const int quad = warp & 3;                      // TMEM lane quadrant: tokens t0 + 32*quad + lane
    const int chalf = (warp - 2) >> 2;              // experts 64*chalf .. 64*chalf + 63
    const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + 64 * chalf;
    float master[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) master[i] = 0.0f;
    const bool cols_used = 64 * chalf < n_mma;      // fewer than 65 experts: the second half has nothing to read
    bool ok = true;
    for (int ch = 0; ch < nchunk && ok; ++ch) {
      const int b = ch & 1;
      ok = __all_sync(0xffffffffu, rt_mbar_wait(chunk_full(b), (uint32_t)((ch >> 1) & 1), abort_flag));
      if (!ok) break;
      rt_fence_after();
      if (cols_used) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          if (64 * chalf + 32 * h2 < n_mma) {
            uint32_t d[32];
            rt_tmem_ld32(tbase + b * 128 + 32 * h2, d);
            rt_tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) master[32 * h2 + i] += __uint_as_float(d[i]);
          }
        }
      }
      rt_fence_before();
      rt_mbar_arrive(chunk_empty(b));
    }
    // a wait that gave up leaves NaN logits, which the selection kernel turns into NaN weights
    const int t = t0 + quad * 32 + lane;
    if (t < T) {
      float* dst = logits + ((size_t)blockIdx.y * T + t) * E + 64 * chalf;
      if (!ok) {
#pragma unroll
        for (int i = 0; i < 64; ++i) master[i] = __int_as_float(0x7fc00000);
      }
      if ((E & 3) == 0) {                           // rows of whole 16-byte pieces (the workspace is 16-byte aligned)
#pragma unroll
        for (int i = 0; i < 64; i += 4)
          if (64 * chalf + i < E)
            *reinterpret_cast<float4*>(dst + i) = make_float4(master[i], master[i + 1], master[i + 2], master[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (64 * chalf + i < E) dst[i] = master[i];
      }
    }
  }

  rt_fence_before();
  __syncthreads();
  if (warp == 1) {
    rt_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)RT_TMEM_COLS) : "memory");
  }
}

typedef CUresult (*RtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
RtEncodeFn rt_encode_fn() {
  static RtEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<RtEncodeFn>(p);
  });
  return fn;
}
bool rt_map(CUtensorMap* map, bool bf16, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  RtEncodeFn fn = rt_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)RT_BK, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
            dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// The tensor-memory logits kernel covers: both operands bf16 or both fp16, H a multiple of 64, at most
// 128 experts, at least 256 tokens.
bool router_tc5_covers(int x_dtype, int w_dtype, int64_t T, int64_t H, int64_t E) {
  return x_dtype == w_dtype && x_dtype != MQ_F32 && H % 64 == 0 && E <= 128 && T >= 256 && T < ((int64_t)1 << 30);
}

// Slices [slice][T][E] like the other logits kernels; k_per_slice is a multiple of 128.
// Returns MQ_ERR_DRIVER_ENTRY when the tensor maps cannot be built (the caller then uses the mma.sync kernel).
int router_logits_tc5(const void* x, const void* w, bool bf16, int64_t T, int64_t H, int64_t E, int slices,
                      int64_t k_per_slice, float* logits, cudaStream_t st) {
  CUtensorMap map_x, map_w;
  const int n_mma = (int)((E + 15) / 16 * 16);
  if (!rt_map(&map_x, bf16, x, (uint64_t)T, (uint64_t)H, RT_TM) || !rt_map(&map_w, bf16, w, (uint64_t)E, (uint64_t)H, (uint32_t)n_mma))
    return MQ_ERR_DRIVER_ENTRY;
  cudaFuncSetAttribute(router_logits_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM_BYTES);
  dim3 grid((unsigned)((T + RT_TM - 1) / RT_TM), (unsigned)slices);
  router_logits_tc5_kernel<<<grid, RT_THREADS, RT_SMEM_BYTES, st>>>(map_x, map_w, bf16 ? 1 : 0, (int)T, (int)H, (int)E,
                                                                    n_mma, (int)k_per_slice, logits);
  return check_launch();
}

}  // namespace mq
