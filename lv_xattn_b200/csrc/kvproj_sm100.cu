// K/V projection of the visual states with the per-head RMSNorm of K fused into the epilogue (sm_100a).
//
//   Kpre = X Wk^T,  V = X Wv^T        X [B*S, Kd] (visual states), Wk, Wv [Hkv*128, Kd] (nn.Linear layout)
//   K    = Kpre * rsqrt(mean_d(Kpre^2) + eps) * w     per key and head, over the 128 head dims
// written straight into the layout the attention kernels read, K, V [B, Hkv, S, 128], plus rstd [B, Hkv, S] fp32
// for the backward of the norm. In the reference this is k_proj / v_proj, view + transpose, repeat_kv and k_norm
// of the patched layer (test_llama3.py:394-419), run in forward and again in the backward recompute (:197, :235).
//
// One GEMM [B*S, Kd] x [Kd, 2*Hkv*128] on the tensor cores: a CTA owns a 256 x 256 output tile (256 keys x two
// heads), as two 128 x 256 x 16 tcgen05.mma per k-step that share the B operand, so that 64 KB of operands feed
// 8.4 MFLOP (64 B/clk/SM at peak). Accumulators fill the 512 TMEM columns: rows 0-127 in columns [0,256), rows
// 128-255 in [256,512). Operands arrive by TMA (128-byte swizzle, no multicast) through a 3-stage ring.
//
// CTA anatomy (320 threads, persistent over tiles; tile index = m_tile * n_tiles + n_tile, so that concurrently
// running CTAs share their X rows and the weights through L2)
//   warp  0     TMA producer (runs ahead into the next tile while the epilogue drains TMEM)
//   warp  1     tcgen05.mma issuer; owns the TMEM allocation
//   warps 2-9   epilogue: thread = output row (TMEM lane), two heads of 128 columns each. For a K tile: pass 1 sums
//               the squares out of TMEM, pass 2 normalises, scales by w, converts and stores 256 bytes per row and
//               head; for a V tile one pass converts and stores.
#include "lvx_internal.h"
#include "sm100_prims.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace lvx {

constexpr int KP_BM = 256, KP_BN = 256, KP_BK = 64;
constexpr int KP_STAGES = 3;
constexpr int KP_HALF = 128 * KP_BK * 2;                 // one 128-row x 64-column 16-bit box: 16 KB
constexpr int KP_STAGE = 4 * KP_HALF;                    // A rows 0-127 | A rows 128-255 | B rows 0-127 | B rows 128-255
constexpr int KP_OFF_W = KP_STAGES * KP_STAGE;           // norm weight, fp32 [128]
constexpr int KP_OFF_BAR = KP_OFF_W + 512;
constexpr int KP_SMEM = KP_OFF_BAR + 256 + 1024;         // + barriers + alignment slack
constexpr int KP_THREADS = 320;
constexpr int KP_EPI_WARPS = 8;
static_assert(KP_SMEM <= 232448, "shared memory budget");

enum { KB_FULL = 0, KB_EMPTY = KP_STAGES, KB_ACC_FULL = 2 * KP_STAGES, KB_ACC_EMPTY, KB_DRAIN, KB_COUNT };

struct KvProjParams {
  int m_total;        // B*S rows of X
  int s_per_batch;    // S
  int kd;             // contraction length (multiple of 64)
  int hkv;            // KV heads (even)
  int m_tiles, n_tiles;   // n_tiles = hkv (hkv/2 K tiles, then hkv/2 V tiles)
  void* k_out;        // [B, Hkv, S, 128]
  void* v_out;
  float* rstd;        // [B, Hkv, S]  (nullable)
  const void* norm_w; // [128] in the input dtype (nullable: no norm, K = Kpre)
  float eps;
  int* status;
};

#define KP_CODE(role, bar) (LVX_DEV_TIMEOUT_BASE | 0x400 | ((role) << 5) | (bar))

template <bool IS_BF16>
__device__ __forceinline__ uint32_t kp_pack(float a, float b) {
  return IS_BF16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

template <bool IS_BF16>
__global__ void __launch_bounds__(KP_THREADS, 1)
kvproj_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmWk,
              const __grid_constant__ CUtensorMap tmWv, const KvProjParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + KP_OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + KB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_w = reinterpret_cast<float*>(smem + KP_OFF_W);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total_tiles = p.m_tiles * p.n_tiles;
  const int kblocks = p.kd / KP_BK;
  const bool poisoned = (*reinterpret_cast<volatile int*>(p.status) != 0);

  if (tid == 0) {
    for (int s = 0; s < KP_STAGES; ++s) {
      mbar_init(&bars[KB_FULL + s], 1);
      mbar_init(&bars[KB_EMPTY + s], 1);
    }
    mbar_init(&bars[KB_ACC_FULL], 1);
    mbar_init(&bars[KB_ACC_EMPTY], KP_EPI_WARPS);
    mbar_init(&bars[KB_DRAIN], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (tid < 128) {
    float w = 1.f;
    if (p.norm_w) {
      if (IS_BF16) w = __bfloat162float(static_cast<const __nv_bfloat16*>(p.norm_w)[tid]);
      else w = __half2float(static_cast<const __half*>(p.norm_w)[tid]);
    }
    s_w[tid] = w;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (!poisoned) {
    if (warp == 0) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmWk);
        tma_prefetch_desc(&tmWv);
        long it = 0, issued = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
          const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
          const bool is_k = nt < p.hkv / 2;
          const CUtensorMap* tmW = is_k ? &tmWk : &tmWv;
          const int m0 = mt * KP_BM, n0 = (is_k ? nt : nt - p.hkv / 2) * KP_BN;
          for (int kb = 0; kb < kblocks; ++kb, ++it) {
            const int s = int(it % KP_STAGES);
            const uint32_t ph = uint32_t(it / KP_STAGES) & 1u;
            if (!mbar_wait(&bars[KB_EMPTY + s], ph ^ 1u, abort_flag, p.status, KP_CODE(0, KB_EMPTY))) {
              ok = false;
              break;
            }
            uint8_t* st = smem + s * KP_STAGE;
            mbar_arrive_expect_tx(&bars[KB_FULL + s], KP_STAGE);
            tma_load_3d(st, &tmX, &bars[KB_FULL + s], kb * KP_BK, m0, 0);
            tma_load_3d(st + KP_HALF, &tmX, &bars[KB_FULL + s], kb * KP_BK, m0 + 128, 0);
            tma_load_3d(st + 2 * KP_HALF, tmW, &bars[KB_FULL + s], kb * KP_BK, n0, 0);
            tma_load_3d(st + 3 * KP_HALF, tmW, &bars[KB_FULL + s], kb * KP_BK, n0 + 128, 0);
            issued = it + 1;
          }
        }
        // a CTA that is giving up must not leave while a copy into its shared memory is in flight
        if (*abort_flag) {
          for (long j = issued > KP_STAGES ? issued - KP_STAGES : 0; j < issued; ++j) {
            const long long t0 = clock64();
            while (!mbar_try_wait(&bars[KB_FULL + j % KP_STAGES], uint32_t(j / KP_STAGES) & 1u) &&
                   clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
          }
        }
      }
    } else if (warp == 1) {
      // =========================== MMA issuer ===========================
      if (lane == 0) {
        constexpr uint32_t FMT = IS_BF16 ? UMMA_BF16 : UMMA_F16;
        constexpr uint32_t IDESC = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, KP_BN);
        constexpr uint32_t HI = umma_desc_hi(1024);
        long it = 0;
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
          // the epilogue of the previous tile must have emptied both accumulators
          ok = mbar_wait(&bars[KB_ACC_EMPTY], (uint32_t(local) & 1u) ^ 1u, abort_flag, p.status, KP_CODE(1, KB_ACC_EMPTY));
          if (!ok) break;
          tc_fence_after();
          for (int kb = 0; kb < kblocks; ++kb, ++it) {
            const int s = int(it % KP_STAGES);
            const uint32_t ph = uint32_t(it / KP_STAGES) & 1u;
            ok = mbar_wait(&bars[KB_FULL + s], ph, abort_flag, p.status, KP_CODE(1, KB_FULL));
            if (!ok) break;
            tc_fence_after();
            const uint32_t sA = smem_u32(smem + s * KP_STAGE);
            const uint32_t a0_lo = umma_desc_lo(sA, 16), a1_lo = umma_desc_lo(sA + KP_HALF, 16);
            const uint32_t b_lo = umma_desc_lo(sA + 2 * KP_HALF, 16);
#pragma unroll
            for (int kk = 0; kk < KP_BK / 16; ++kk) {
              const uint32_t off = (kk * 32) >> 4;
              const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
              const uint64_t bd = umma_desc_join(b_lo + off, HI);
              umma_ss_f16(tmem_base, umma_desc_join(a0_lo + off, HI), bd, IDESC, acc);
              umma_ss_f16(tmem_base + KP_BN, umma_desc_join(a1_lo + off, HI), bd, IDESC, acc);
            }
            tc_commit(&bars[KB_EMPTY + s]);
          }
          if (ok) tc_commit(&bars[KB_ACC_FULL]);
        }
        if (!ok) {
          tc_commit(&bars[KB_DRAIN]);
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars[KB_DRAIN], 0) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
        }
      }
    } else {
      // =========================== epilogue warps ===========================
      const int ew = warp - 2;
      const int half = ew >> 2;                             // which 128 rows of the tile / which accumulator
      const int quarter = warp & 3;                         // TMEM lane quarter this warp may touch
      const int row_in_tile = half * 128 + quarter * 32 + lane;
      const uint32_t tacc = tmem_base + half * KP_BN + (static_cast<uint32_t>(quarter * 32) << 16);
      int local = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
        if (!mbar_wait(&bars[KB_ACC_FULL], uint32_t(local) & 1u, abort_flag, p.status, KP_CODE(2, KB_ACC_FULL))) break;
        tc_fence_after();
        const int mt = tile / p.n_tiles, nt = tile % p.n_tiles;
        const bool is_k = nt < p.hkv / 2;
        const int m = mt * KP_BM + row_in_tile;
        const bool row_ok = m < p.m_total;
        const int b = row_ok ? m / p.s_per_batch : 0, srow = row_ok ? m % p.s_per_batch : 0;
        const bool norm = is_k && p.norm_w != nullptr;
#pragma unroll 1
        for (int head = 0; head < 2; ++head) {
          const int hk = (is_k ? nt : nt - p.hkv / 2) * 2 + head;
          const uint32_t tcol = tacc + head * 128;
          float scale = 1.f;
          if (is_k) {
            float ss = 0.f;
            if (norm) {
#pragma unroll 1
              for (int c = 0; c < 4; ++c) {
                uint32_t x[32];
                tmem_ld32(tcol + c * 32, x);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) ss = fmaf(__uint_as_float(x[i]), __uint_as_float(x[i]), ss);
              }
              scale = rsqrtf(ss * (1.f / 128.f) + p.eps);
            }
            if (row_ok && p.rstd) p.rstd[(size_t(b) * p.hkv + hk) * p.s_per_batch + srow] = scale;
          }
          uint8_t* out = static_cast<uint8_t*>(is_k ? p.k_out : p.v_out) +
                         ((size_t(b) * p.hkv + hk) * p.s_per_batch + srow) * 256;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t x[32];
            tmem_ld32(tcol + c * 32, x);
            tc_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int i4 = 0; i4 < 4; ++i4) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int i = i4 * 8 + 2 * e;
                  float lo = __uint_as_float(x[i]) * scale, hi = __uint_as_float(x[i + 1]) * scale;
                  if (norm) {
                    lo *= s_w[c * 32 + i];
                    hi *= s_w[c * 32 + i + 1];
                  }
                  w[e] = kp_pack<IS_BF16>(lo, hi);
                }
                *reinterpret_cast<uint4*>(out + c * 64 + i4 * 16) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[KB_ACC_EMPTY]);    // both accumulators of this warp's rows are read
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

int launch_kv_project(int dtype, const void* x, const void* wk, const void* wv, const void* norm_w, float eps,
                      int batch, int s, int kd, int hkv, void* k_out, void* v_out, float* rstd, int* status,
                      cudaStream_t st) {
  const long m_total = long(batch) * s;
  CUtensorMap tmX, tmWk, tmWv;
  const uint64_t row_bytes = uint64_t(kd) * 2;
  int rc;
  if ((rc = make_tmap_3d(&tmX, dtype, x, kd, m_total, 1, row_bytes, row_bytes * m_total, 64, 128))) return rc;
  const uint64_t n_rows = uint64_t(hkv) * 128;
  if ((rc = make_tmap_3d(&tmWk, dtype, wk, kd, n_rows, 1, row_bytes, row_bytes * n_rows, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmWv, dtype, wv, kd, n_rows, 1, row_bytes, row_bytes * n_rows, 64, 128))) return rc;
  KvProjParams p;
  p.m_total = int(m_total);
  p.s_per_batch = s;
  p.kd = kd;
  p.hkv = hkv;
  p.m_tiles = int((m_total + KP_BM - 1) / KP_BM);
  p.n_tiles = hkv;
  p.k_out = k_out;
  p.v_out = v_out;
  p.rstd = rstd;
  p.norm_w = norm_w;
  p.eps = eps;
  p.status = status;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const long total = long(p.m_tiles) * p.n_tiles;
  const int grid = int(total < sms ? total : sms);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, KP_SMEM);
    if (e == cudaSuccess) kern<<<grid, KP_THREADS, KP_SMEM, st>>>(tmX, tmWk, tmWv, p);
  };
  if (dtype == LVX_BF16) go(kvproj_kernel<true>);
  else go(kvproj_kernel<false>);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(kvproj)");
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "kvproj_kernel launch");
  return LVX_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward of the fused norm: from dK (gradient of the normalised keys), K (normalised), rstd and w
//   dKpre = rstd * (w * dK - (K / w) * mean_d(K * dK))          dw[d] += sum_rows dK * K / w
// One warp per (key, head) row of 128; dw is reduced per block and added with one atomic per column and block.
template <bool IS_BF16>
__global__ void __launch_bounds__(256)
knorm_bwd_kernel(const void* __restrict__ k, const void* __restrict__ dk, const float* __restrict__ rstd,
                 const void* __restrict__ norm_w, void* __restrict__ dkpre, float* __restrict__ dw, long rows,
                 const int* status) {
  if (status && *reinterpret_cast<const volatile int*>(status) != 0) return;
  __shared__ float s_dw[8][128];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const long row = long(blockIdx.x) * 8 + wib;
  float dwl[4] = {0.f, 0.f, 0.f, 0.f};
  if (row < rows) {
    const uint2 kk = reinterpret_cast<const uint2*>(k)[row * 32 + lane];
    const uint2 gg = reinterpret_cast<const uint2*>(dk)[row * 32 + lane];
    const uint2 ww = reinterpret_cast<const uint2*>(norm_w)[lane];
    float kf[4], gf[4], wf[4];
    auto unpack = [](uint32_t v, float& a, float& b) {
      if (IS_BF16) {
        a = __uint_as_float(v << 16);
        b = __uint_as_float(v & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
        a = f.x;
        b = f.y;
      }
    };
    unpack(kk.x, kf[0], kf[1]);
    unpack(kk.y, kf[2], kf[3]);
    unpack(gg.x, gf[0], gf[1]);
    unpack(gg.y, gf[2], gf[3]);
    unpack(ww.x, wf[0], wf[1]);
    unpack(ww.y, wf[2], wf[3]);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) dot = fmaf(kf[i], gf[i], dot);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float mean = dot * (1.f / 128.f), r = rstd[row];
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float xhat = kf[i] / wf[i];                // Kpre * rstd
      o[i] = r * (wf[i] * gf[i] - xhat * mean);
      dwl[i] = gf[i] * xhat;
    }
    reinterpret_cast<uint2*>(dkpre)[row * 32 + lane] = make_uint2(kp_pack<IS_BF16>(o[0], o[1]), kp_pack<IS_BF16>(o[2], o[3]));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) s_dw[wib][lane * 4 + i] = dwl[i];
  __syncthreads();
  if (threadIdx.x < 128) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += s_dw[w][threadIdx.x];
    atomicAdd(dw + threadIdx.x, a);
  }
}

int launch_knorm_bwd(int dtype, const void* k, const void* dk, const float* rstd, const void* norm_w, void* dkpre,
                     float* dw, long rows, cudaStream_t st) {
  const long blocks = (rows + 7) / 8;
  if (blocks == 0) return LVX_OK;
  const int* sp = device_status_ptr();
  if (dtype == LVX_BF16) knorm_bwd_kernel<true><<<blocks, 256, 0, st>>>(k, dk, rstd, norm_w, dkpre, dw, rows, sp);
  else knorm_bwd_kernel<false><<<blocks, 256, 0, st>>>(k, dk, rstd, norm_w, dkpre, dw, rows, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "knorm_bwd launch");
  return LVX_OK;
}

}  // namespace lvx
