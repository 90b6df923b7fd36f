// Self-test of the tensor-core building blocks: one CTA computes D[128,N] = A * B for every operand
// arrangement the attention kernels rely on, so that a descriptor or layout mistake shows up as a wrong
// number in a 128 x N product instead of somewhere inside a flash-attention pipeline.
//
// mode  elt   K    N    A source                         B source
//  0    bf16  128  128  smem, K-major   a[128][K]         smem, K-major   b[N][K]      D = a b^T
//  1    bf16  128  128  TMEM (packed)   a[128][K]         smem, MN-major  b[K][N]      D = a b
//  2    bf16  128   64  smem, MN-major  a[K][128]         smem, MN-major  b[K][N]      D = a^T b
//  3    bf16  128   64  smem, K-major   a[128][K]         smem, K-major   b[N][K]      D = a b^T
//  4    bf16   64  128  TMEM (packed)   a[128][K]         smem, MN-major  b[K][N]      D = a b
//  5    fp32   64  128  smem, K-major   a[128][K]         smem, K-major   b[N][K]      D = a b^T   (tf32)
//  6    fp32   32  128  TMEM            a[128][K]         smem, MN-major  b[K][N]      D = a b     (tf32)
//  7    fp32   32   64  smem, MN-major  a[K][128]         smem, MN-major  b[K][N]      D = a^T b   (tf32)
#include "lvx_internal.h"
#include "sm100_prims.cuh"
#include <cuda_bf16.h>

namespace lvx {

struct SelfTestCfg {
  int elt;      // bytes per element
  int K, N;
  int a_src;    // 0 smem K-major, 1 smem MN-major, 2 TMEM
  int b_major;  // 0 K-major, 1 MN-major
};

__host__ __device__ inline SelfTestCfg selftest_cfg(int mode) {
  switch (mode) {
    case 0: return {2, 128, 128, 0, 0};
    case 1: return {2, 128, 128, 2, 1};
    case 2: return {2, 128, 64, 1, 1};
    case 3: return {2, 128, 64, 0, 0};
    case 4: return {2, 64, 128, 2, 1};
    case 5: return {4, 64, 128, 0, 0};
    case 6: return {4, 32, 128, 2, 1};
    case 7: return {4, 32, 64, 1, 1};
    default: return {0, 0, 0, 0, 0};
  }
}

// Shared memory: A region 32 KiB, B region 32 KiB (both 1024-byte aligned), then barriers.
constexpr int ST_SMEM = 65536 + 1024 + 256;

__global__ void __launch_bounds__(128, 1)
selftest_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const void* __restrict__ a_gmem, float* __restrict__ d_out, int mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + 32768;
  uint64_t* bar_load = reinterpret_cast<uint64_t*>(smem + 65536);
  uint64_t* bar_mma = bar_load + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_load + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const SelfTestCfg c = selftest_cfg(mode);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int epr = 128 / c.elt;  // elements per 128-byte row

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_d = tmem_base;        // columns [0, N)
  const uint32_t tmem_a = tmem_base + 128;  // columns [128, ...)

  // ---- operand staging --------------------------------------------------------------------
  if (tid == 0) {
    uint32_t bytes = 0;
    // B: K-major -> rows = N, cols = K ; MN-major -> rows = K, cols = N
    const int b_rows = c.b_major == 0 ? c.N : c.K;
    const int b_cols = c.b_major == 0 ? c.K : c.N;
    const int b_boxes = b_cols / epr;
    bytes += b_boxes * b_rows * 128;
    int a_rows = 0, a_boxes = 0;
    if (c.a_src != 2) {
      a_rows = c.a_src == 0 ? 128 : c.K;
      const int a_cols = c.a_src == 0 ? c.K : 128;
      a_boxes = a_cols / epr;
      bytes += a_boxes * a_rows * 128;
    }
    mbar_arrive_expect_tx(bar_load, bytes);
    for (int b = 0; b < b_boxes; ++b) tma_load_3d(sB + b * b_rows * 128, &tmB, bar_load, b * epr, 0, 0);
    for (int b = 0; b < a_boxes; ++b) tma_load_3d(sA + b * a_rows * 128, &tmA, bar_load, b * epr, 0, 0);
  }
  if (c.a_src == 2) {
    // thread = row; pack the row of A into TMEM columns (two 16-bit values per column, or one fp32).
    const uint32_t lane_addr = tmem_a + (static_cast<uint32_t>(warp * 32) << 16);
    if (c.elt == 2) {
      const __nv_bfloat16* arow = reinterpret_cast<const __nv_bfloat16*>(a_gmem) + size_t(tid) * c.K;
      for (int c0 = 0; c0 < c.K / 2; c0 += 32) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = pack_bf16x2(__bfloat162float(arow[2 * (c0 + i)]), __bfloat162float(arow[2 * (c0 + i) + 1]));
        tmem_st32(lane_addr + c0, r);
      }
    } else {
      const float* arow = reinterpret_cast<const float*>(a_gmem) + size_t(tid) * c.K;
      for (int c0 = 0; c0 < c.K; c0 += 32) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(arow[c0 + i]);
        tmem_st32(lane_addr + c0, r);
      }
    }
    tc_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- MMA issue ----------------------------------------------------------------------------
  if (tid == 0) {
    if (mbar_wait(bar_load, 0, abort_flag, status, LVX_DEV_TIMEOUT_BASE | 0xF01)) {
      tc_fence_after();
      const uint32_t fmt = c.elt == 2 ? UMMA_BF16 : UMMA_TF32;
      const uint32_t idesc = umma_idesc(fmt, c.a_src == 1 ? UMMA_MN_MAJOR : UMMA_K_MAJOR,
                                        c.b_major ? UMMA_MN_MAJOR : UMMA_K_MAJOR, 128, c.N);
      const int kstep = 32 / c.elt;  // elements of K per MMA
      const int nk = c.K / kstep;
      const uint32_t a_base = smem_u32(sA), b_base = smem_u32(sB);
      const int b_rows = c.b_major == 0 ? c.N : c.K;
      const int a_rows = c.a_src == 0 ? 128 : c.K;
      for (int kk = 0; kk < nk; ++kk) {
        // K-major: step 32 bytes inside the 128-byte row, next swizzle atom after 4 steps.
        // MN-major: step kstep rows of 128 bytes.
        uint64_t bdesc, adesc = 0;
        // 32-bit MN-major operands use the 32-byte-unit swizzle: K rows in groups of 4 (512 bytes)
        const uint32_t mn_sbo = c.elt == 4 ? 512 : 1024, mn_type = c.elt == 4 ? 1 : 2;
        if (c.b_major == 0)
          bdesc = umma_smem_desc(b_base + (kk >> 2) * b_rows * 128 + (kk & 3) * 32, 16, 1024);
        else
          bdesc = umma_smem_desc(b_base + kk * kstep * 128, b_rows * 128, mn_sbo, mn_type);
        if (c.a_src == 0)
          adesc = umma_smem_desc(a_base + (kk >> 2) * a_rows * 128 + (kk & 3) * 32, 16, 1024);
        else if (c.a_src == 1)
          adesc = umma_smem_desc(a_base + kk * kstep * 128, a_rows * 128, mn_sbo, mn_type);
        const uint32_t acc = kk > 0;
        if (c.elt == 2) {
          if (c.a_src == 2) umma_ts_f16(tmem_d, tmem_a + kk * 8, bdesc, idesc, acc);
          else umma_ss_f16(tmem_d, adesc, bdesc, idesc, acc);
        } else {
          if (c.a_src == 2) umma_ts_tf32(tmem_d, tmem_a + kk * 8, bdesc, idesc, acc);
          else umma_ss_tf32(tmem_d, adesc, bdesc, idesc, acc);
        }
      }
    }
    tc_commit(bar_mma);
  }
  __syncwarp();

  // ---- read back ------------------------------------------------------------------------------
  const bool ok = mbar_wait(bar_mma, 0, abort_flag, status, LVX_DEV_TIMEOUT_BASE | 0xF02);
  tc_fence_after();
  if (ok) {
    const uint32_t lane_addr = tmem_d + (static_cast<uint32_t>(warp * 32) << 16);
    for (int c0 = 0; c0 < c.N; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(lane_addr + c0, r);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) d_out[size_t(tid) * c.N + c0 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
}

int launch_selftest(int mode, const void* a, const void* b, float* d_out, int* status, cudaStream_t st) {
  const SelfTestCfg c = selftest_cfg(mode);
  if (c.elt == 0) return fail(LVX_ERR_SHAPE, "lvx_selftest_mma: unknown mode %d", mode);
  const int dtype = c.elt == 2 ? LVX_BF16 : LVX_FP32;
  const int epr = 128 / c.elt;
  CUtensorMap tmA, tmB;
  int rc;
  const int b_rows = c.b_major == 0 ? c.N : c.K, b_cols = c.b_major == 0 ? c.K : c.N;
  rc = make_tmap_3d(&tmB, dtype, b, b_cols, b_rows, 1, uint64_t(b_cols) * c.elt, uint64_t(b_cols) * b_rows * c.elt,
                    epr, b_rows, c.elt == 4 && c.b_major == 1);
  if (rc) return rc;
  if (c.a_src != 2) {
    const int a_rows = c.a_src == 0 ? 128 : c.K, a_cols = c.a_src == 0 ? c.K : 128;
    rc = make_tmap_3d(&tmA, dtype, a, a_cols, a_rows, 1, uint64_t(a_cols) * c.elt,
                      uint64_t(a_cols) * a_rows * c.elt, epr, a_rows, c.elt == 4 && c.a_src == 1);
    if (rc) return rc;
  } else {
    tmA = tmB;
  }
  cudaError_t e = cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(selftest)");
  selftest_kernel<<<1, 128, ST_SMEM, st>>>(tmA, tmB, a, d_out, mode, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "selftest launch");
  return LVX_OK;
}

}  // namespace lvx
