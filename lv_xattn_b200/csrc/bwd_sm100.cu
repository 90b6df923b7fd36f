// Backward flash-attention block for sm_100a.
//
// A CTA owns one 128-row K/V tile of one (batch, kv head) and walks over the packed query rows of the
// group (g*Sq rows, 64 at a time). Everything is computed in the transposed frame, so that the softmax
// statistics are per column and no row reduction is needed:
//     S^T  = K Q^T            (smem x smem)       P^T  = exp2(S^T*c - lse[col])
//     dP^T = V dO^T           (smem x smem)       dS^T = P^T o (dP^T - delta[col])
//     dV  += P^T  dO          (TMEM x smem, dO consumed MN-major)
//     dK  += dS^T Q           (TMEM x smem, Q  consumed MN-major)
//     dQ^T = K^T dS^T         (smem x smem, both MN-major; dS^T staged through shared memory)
// dK/dV stay in TMEM for the whole walk (summing over the query heads of the group on the way) and are
// written once; dQ^T tiles are reduce-added (red.global.add.f32) into the fp32 dQ accumulator. The
// softmax scale is applied once on the way out (dK, dQ).
//
// CTA anatomy (448 threads)
//   warps 0-7   P^T/dS^T producers: thread = K/V row (TMEM lane = 32*(warp%4)+lane); warps 0-3 take query
//               columns 0-31 of the tile, warps 4-7 columns 32-63 (two warps per scheduler hide each other's
//               latencies); epilogue: warps 0-3 write dK, warps 4-7 write dV
//   warps 8-11  dQ reducers: thread = head-dim index (TMEM lane of dQ^T)
//   warp  12    TMA producer: K,V once; Q,dO tiles through a 3-stage ring
//   warp  13    tcgen05.mma issuer; owns the TMEM allocation
//   TMEM columns: dK [0,128) dV [128,256) S^T x2 [256,384) dP^T [384,448) dQ^T [448,512);
//   P^T and dS^T (16-bit, 32 columns each) overwrite the S^T buffer they came from.
#include "lvx_internal.h"
#include "sm100_prims.cuh"
#include <math.h>
#include <stdlib.h>
#include <stdio.h>

namespace lvx {

constexpr int BWD_NSQ = 3;                      // Q/dO pipeline stages
constexpr int BWD_KV_BYTES = 128 * 128 * 2;     // K or V tile
constexpr int BWD_KV_HALF = BWD_KV_BYTES / 2;
constexpr int BWD_Q_BYTES = 64 * 128 * 2;       // Q or dO tile (64 rows)
constexpr int BWD_Q_HALF = BWD_Q_BYTES / 2;
constexpr int BWD_DS_BYTES = 128 * 64 * 2;      // dS^T tile [128 kv][64 q]
constexpr int BWD_OFF_K = 0;
constexpr int BWD_OFF_V = BWD_KV_BYTES;
constexpr int BWD_OFF_Q = 2 * BWD_KV_BYTES;                         // stage s: Q at +s*2*Q_BYTES, dO right after
constexpr int BWD_OFF_DS = BWD_OFF_Q + BWD_NSQ * 2 * BWD_Q_BYTES;
constexpr int BWD_OFF_STAT = BWD_OFF_DS + 2 * BWD_DS_BYTES;         // lse2[3][64], delta[3][64]
constexpr int BWD_OFF_BAR = BWD_OFF_STAT + 6 * 64 * 4;
constexpr int BWD_SMEM = BWD_OFF_BAR + 256 + 1024;
constexpr int BWD_THREADS = 448;

constexpr uint32_t TM_DK = 0, TM_DV = 128, TM_S = 256, TM_DP = 384, TM_DQ = 448;

enum {
  BB_KV_FULL = 0,
  BB_Q_FULL = 1,
  BB_Q_EMPTY = BB_Q_FULL + BWD_NSQ,
  BB_S_FULL = BB_Q_EMPTY + BWD_NSQ,   // x2
  BB_DP_FULL = BB_S_FULL + 2,
  BB_DP_FREE = BB_DP_FULL + 1,
  BB_PDS_FULL = BB_DP_FREE + 1,       // x2
  BB_DS_FREE = BB_PDS_FULL + 2,       // x2
  BB_DQ_FULL = BB_DS_FREE + 2,
  BB_DQ_FREE = BB_DQ_FULL + 1,
  BB_ACC_DONE = BB_DQ_FREE + 1,
  BB_DRAIN = BB_ACC_DONE + 1,
  BB_STAT_FULL = BB_DRAIN + 1,        // x3
  BB_COUNT = BB_STAT_FULL + 3
};

struct BwdParams {
  int rows;            // g * Sq
  int skv;
  int hkv;
  const int32_t* kv_valid_len;
  const float* lse;    // [B*Hq*Sq]  == [slab][rows]
  const float* delta;
  float scale;         // sm_scale
  float scale_log2;    // sm_scale * log2(e)
  float* dq_acc;       // [slab][rows][128]
  float* dk_acc;       // [slab][skv][128]
  float* dv_acc;
  int accumulate;
  int debug;           // development switches (LVX_BWD_DEBUG); 0 in normal use
  int* status;
};

// Development aid (LVX_BWD_DEBUG bit 128): cycle stamps of CTA (0,0), tiles 8..15, 16 slots per tile and role.
__device__ long long g_bwd_ts[3 * 8 * 16];
#define BWD_TS(role, slot)                                                                         \
  do {                                                                                             \
    if ((p.debug & 128) && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && j >= 8 && j < 16)    \
      g_bwd_ts[((role) * 8 + (j - 8)) * 16 + (slot)] = clock64();                                  \
  } while (0)

#define BWD_CODE(role, bar) (LVX_DEV_TIMEOUT_BASE | 0x200 | ((role) << 5) | (bar))

// Writes / accumulates one 128-float row of a TMEM accumulator to global memory.
__device__ __forceinline__ void store_acc_row(uint32_t taddr, float* dst, bool row_ok, bool accumulate, float mul) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t r[32];
    tmem_ld32(taddr + q * 32, r);
    tc_wait_ld();
    if (row_ok) {
      float4* d4 = reinterpret_cast<float4*>(dst) + q * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 v = make_float4(__uint_as_float(r[4 * i]) * mul, __uint_as_float(r[4 * i + 1]) * mul,
                               __uint_as_float(r[4 * i + 2]) * mul, __uint_as_float(r[4 * i + 3]) * mul);
        if (accumulate) {
          const float4 o = d4[i];
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        d4[i] = v;
      }
    }
  }
}

template <bool IS_BF16>
__global__ void __launch_bounds__(BWD_THREADS, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
           const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BWD_OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_lse = reinterpret_cast<float*>(smem + BWD_OFF_STAT);   // [3][64], already times log2(e)
  float* s_delta = s_lse + 192;                                   // [3][64]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kv_tile = blockIdx.x, slab = blockIdx.y;
  const int batch = slab / p.hkv;
  const int kv0 = kv_tile * 128;

  int valid = p.skv;
  if (p.kv_valid_len) valid = min(valid, max(0, p.kv_valid_len[batch]));
  const bool tile_live = kv0 < valid;          // at least one valid K/V row in this tile
  const int nq = (p.rows + 63) >> 6;
  const bool poisoned = (*reinterpret_cast<volatile int*>(p.status) != 0);

  if (tid == 0) {
    mbar_init(&bars[BB_KV_FULL], 1);
    for (int s = 0; s < BWD_NSQ; ++s) {
      mbar_init(&bars[BB_Q_FULL + s], 1);
      mbar_init(&bars[BB_Q_EMPTY + s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars[BB_S_FULL + b], 1);
      mbar_init(&bars[BB_PDS_FULL + b], 8);    // one arrival per producer warp
      mbar_init(&bars[BB_DS_FREE + b], 1);
    }
    mbar_init(&bars[BB_DP_FULL], 1);
    mbar_init(&bars[BB_DP_FREE], 8);
    mbar_init(&bars[BB_DQ_FULL], 1);
    mbar_init(&bars[BB_DQ_FREE], 4);
    mbar_init(&bars[BB_ACC_DONE], 1);
    mbar_init(&bars[BB_DRAIN], 1);
    for (int b = 0; b < 3; ++b) mbar_init(&bars[BB_STAT_FULL + b], 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 13) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (!poisoned && tile_live) {
    if (warp < 8) {
      // =========================== P^T / dS^T producers ===========================
      const int half = warp >> 2;                           // which 32 query columns of the tile
      const int r = (warp & 3) * 32 + lane;                 // K/V row inside the tile
      const bool row_valid = (kv0 + r) < valid;
      const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const float c = p.scale_log2;
      const size_t stat_base = size_t(slab) * p.rows;
      // statistics of the next query tile, fetched one tile ahead by threads 0-63 (lse) and 64-127 (delta)
      auto fetch_stat = [&](int j) -> float {
        const int col = tid & 63;
        const int qrow = j * 64 + col;
        if (tid < 64) {
          float v = INFINITY;   // +inf => P = 0 for query rows that do not exist
          if (qrow < p.rows) {
            v = p.lse[stat_base + qrow] * 1.4426950408889634f;
            if (v == -INFINITY) v = INFINITY;   // a row with no valid key anywhere has P = 0
          }
          return v;
        }
        return (tid < 128 && qrow < p.rows) ? p.delta[stat_base + qrow] : 0.f;
      };
      // Three buffers: a thread may run one tile ahead of the slowest thread of the group (the
      // dP^T hand-over keeps them within one tile of each other), and it writes tile j+1 while in tile j.
      auto put_stat = [&](int j, float v) {
        if (tid >= 128) return;
        const int b = j % 3;
        if (tid < 64) s_lse[b * 64 + tid] = v;
        else s_delta[b * 64 + (tid - 64)] = v;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[BB_STAT_FULL + b]);
      };
      put_stat(0, fetch_stat(0));
      // The statistics are fetched two tiles ahead (global-memory latency is longer than one tile's work)
      // and published one tile ahead.
      float stat_next = nq > 1 ? fetch_stat(1) : 0.f;
      bool alive = true;
      for (int j = 0; j < nq; ++j) {
        const int b = j & 1;
        if (warp == 0) BWD_TS(0, 0);
        const uint32_t tS = tmem_base + TM_S + b * 64 + lane_sel;
        const uint32_t tDP = tmem_base + TM_DP + lane_sel;
        float stat_after = 0.f;
        if (j + 2 < nq) stat_after = fetch_stat(j + 2);
        if (!mbar_wait(&bars[BB_S_FULL + b], (j >> 1) & 1, abort_flag, p.status, BWD_CODE(0, BB_S_FULL)) ||
            !mbar_wait(&bars[BB_DP_FULL], j & 1, abort_flag, p.status, BWD_CODE(0, BB_DP_FULL))) {
          alive = false;
          break;
        }
        tc_fence_after();
        if (warp == 0) BWD_TS(0, 1);
        uint32_t s[32], dp[32];
        tmem_ld32(tS + half * 32, s);
        tmem_ld32(tDP + half * 32, dp);
        tc_wait_ld();
        if (warp == 0) BWD_TS(0, 2);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[BB_DP_FREE]);
        if (!mbar_wait(&bars[BB_STAT_FULL + j % 3], (j / 3) & 1, abort_flag, p.status, BWD_CODE(0, BB_STAT_FULL))) {
          alive = false;
          break;
        }
        if (warp == 0) BWD_TS(0, 3);
        const float4* sl = reinterpret_cast<const float4*>(s_lse + (j % 3) * 64 + half * 32);
        const float4* sd = reinterpret_cast<const float4*>(s_delta + (j % 3) * 64 + half * 32);
        uint32_t pk[16], dsk[16];
        if (p.debug & 2) {
#pragma unroll
          for (int i = 0; i < 16; ++i) { pk[i] = s[i]; dsk[i] = dp[i]; }
        } else
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 l2 = sl[i];
          const float4 dl = sd[i];
          float p0 = ex2f(fmaf(__uint_as_float(s[4 * i]), c, -l2.x));
          float p1 = ex2f(fmaf(__uint_as_float(s[4 * i + 1]), c, -l2.y));
          float p2 = ex2f(fmaf(__uint_as_float(s[4 * i + 2]), c, -l2.z));
          float p3 = ex2f(fmaf(__uint_as_float(s[4 * i + 3]), c, -l2.w));
          if (!row_valid) { p0 = 0.f; p1 = 0.f; p2 = 0.f; p3 = 0.f; }
          const float d0 = p0 * (__uint_as_float(dp[4 * i]) - dl.x);
          const float d1 = p1 * (__uint_as_float(dp[4 * i + 1]) - dl.y);
          const float d2 = p2 * (__uint_as_float(dp[4 * i + 2]) - dl.z);
          const float d3 = p3 * (__uint_as_float(dp[4 * i + 3]) - dl.w);
          pk[2 * i] = IS_BF16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
          pk[2 * i + 1] = IS_BF16 ? pack_bf16x2(p2, p3) : pack_f16x2(p2, p3);
          dsk[2 * i] = IS_BF16 ? pack_bf16x2(d0, d1) : pack_f16x2(d0, d1);
          dsk[2 * i + 1] = IS_BF16 ? pack_bf16x2(d2, d3) : pack_f16x2(d2, d3);
        }
        if (warp == 0) BWD_TS(0, 4);
        tmem_st16(tS + half * 16, pk);
        tmem_st16(tS + 32 + half * 16, dsk);
        if (warp == 0) BWD_TS(0, 5);
        // dS^T row -> shared memory, 128-byte swizzled (16-byte chunk index xor row mod 8)
        if (j >= 2 &&
            !mbar_wait(&bars[BB_DS_FREE + b], ((j >> 1) - 1) & 1, abort_flag, p.status, BWD_CODE(0, BB_DS_FREE))) {
          alive = false;
          tc_wait_st();
          break;
        }
        if (!(p.debug & 32)) {
          uint8_t* rowp = smem + BWD_OFF_DS + b * BWD_DS_BYTES + r * 128;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 v = make_uint4(dsk[4 * ch], dsk[4 * ch + 1], dsk[4 * ch + 2], dsk[4 * ch + 3]);
            *reinterpret_cast<uint4*>(rowp + (((half * 4 + ch) ^ (r & 7)) << 4)) = v;
          }
        }
        if (warp == 0) BWD_TS(0, 6);
        if (j + 1 < nq) put_stat(j + 1, stat_next);
        stat_next = stat_after;
        if (warp == 0) BWD_TS(0, 7);
        tc_wait_st();
        if (warp == 0) BWD_TS(0, 8);
        tc_fence_before();
        if (!(p.debug & 32)) fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[BB_PDS_FULL + b]);
        if (warp == 0) BWD_TS(0, 9);
      }
      // ------------------------------- dK / dV epilogue -------------------------------
      if (alive) alive = mbar_wait(&bars[BB_ACC_DONE], 0, abort_flag, p.status, BWD_CODE(0, BB_ACC_DONE));
      tc_fence_after();
      if (alive) {
        const bool ok_row = (kv0 + r) < p.skv;
        const size_t off = (size_t(slab) * p.skv + kv0 + r) * 128;
        if (half == 0)
          store_acc_row(tmem_base + TM_DK + lane_sel, p.dk_acc + off, ok_row, p.accumulate != 0, p.scale);
        else
          store_acc_row(tmem_base + TM_DV + lane_sel, p.dv_acc + off, ok_row, p.accumulate != 0, 1.f);
      }
    } else if (warp < 12) {
      // =========================== dQ reducers ===========================
      const int d = (warp - 8) * 32 + lane;                  // head-dim index = TMEM lane of dQ^T
      const uint32_t lane_sel = static_cast<uint32_t>((warp - 8) * 32) << 16;
      const uint32_t tDQ = tmem_base + TM_DQ + lane_sel;
      float* dq_base = p.dq_acc + size_t(slab) * p.rows * 128 + d;
      bool alive = true;
      for (int j = 0; j < nq; ++j) {
        if (!mbar_wait(&bars[BB_DQ_FULL], j & 1, abort_flag, p.status, BWD_CODE(1, BB_DQ_FULL))) {
          alive = false;
          break;
        }
        if (warp == 8) BWD_TS(1, 0);
        tc_fence_after();
        uint32_t v[2][32];
        tmem_ld32(tDQ, v[0]);
        tmem_ld32(tDQ + 32, v[1]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[BB_DQ_FREE]);
        if (warp == 8) BWD_TS(1, 1);
        const int q0 = j * 64;
        const int ncols = min(64, p.rows - q0);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (h * 32 + i < ncols && !(p.debug & 1))
              atomicAdd(dq_base + size_t(q0 + h * 32 + i) * 128, __uint_as_float(v[h][i]) * p.scale);
      }
      (void)alive;
    } else if (warp == 12) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_arrive_expect_tx(&bars[BB_KV_FULL], 2 * BWD_KV_BYTES);
        for (int h = 0; h < 2; ++h) {
          tma_load_3d(smem + BWD_OFF_K + h * BWD_KV_HALF, &tmK, &bars[BB_KV_FULL], h * 64, kv0, slab);
          tma_load_3d(smem + BWD_OFF_V + h * BWD_KV_HALF, &tmV, &bars[BB_KV_FULL], h * 64, kv0, slab);
        }
        int issued = 0;
        for (int j = 0; j < nq; ++j) {
          const int s = j % BWD_NSQ;
          const uint32_t ph = (j / BWD_NSQ) & 1;
          if (!mbar_wait(&bars[BB_Q_EMPTY + s], ph ^ 1, abort_flag, p.status, BWD_CODE(2, BB_Q_EMPTY))) break;
          uint8_t* dstq = smem + BWD_OFF_Q + s * 2 * BWD_Q_BYTES;
          if (p.debug & 64) {
            mbar_arrive(&bars[BB_Q_FULL + s]);
          } else {
            mbar_arrive_expect_tx(&bars[BB_Q_FULL + s], 2 * BWD_Q_BYTES);
            for (int h = 0; h < 2; ++h) {
              tma_load_3d(dstq + h * BWD_Q_HALF, &tmQ, &bars[BB_Q_FULL + s], h * 64, j * 64, slab);
              tma_load_3d(dstq + BWD_Q_BYTES + h * BWD_Q_HALF, &tmDO, &bars[BB_Q_FULL + s], h * 64, j * 64, slab);
            }
          }
          issued = j + 1;
        }
        if (*abort_flag) {
          auto drain = [&](uint64_t* bar, uint32_t ph) {
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, ph) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
          };
          drain(&bars[BB_KV_FULL], 0);
          for (int j = max(0, issued - BWD_NSQ); j < issued; ++j) drain(&bars[BB_Q_FULL + j % BWD_NSQ], (j / BWD_NSQ) & 1);
        }
      }
    } else {
      // =========================== MMA issuer ===========================
      if (lane == 0) {
        constexpr uint32_t FMT = IS_BF16 ? UMMA_BF16 : UMMA_F16;
        constexpr uint32_t IDESC_S = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 64);
        constexpr uint32_t IDESC_ACC = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_MN_MAJOR, 128, 128);
        constexpr uint32_t IDESC_DQ = umma_idesc(FMT, UMMA_MN_MAJOR, UMMA_MN_MAJOR, 128, 64);
        const uint32_t sK = smem_u32(smem + BWD_OFF_K), sV = smem_u32(smem + BWD_OFF_V);
        const uint32_t sQ0 = smem_u32(smem + BWD_OFF_Q), sDS0 = smem_u32(smem + BWD_OFF_DS);

        constexpr uint32_t HI = umma_desc_hi(1024);
        // D[128 kv, 64 q] = A[128 kv, 128 d] * B[64 q, 128 d]^T, both K-major
        auto issue_st = [&](uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem) {
          const uint32_t a_lo = umma_desc_lo(a_smem, 16), b_lo = umma_desc_lo(b_smem, 16);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss_f16(d_tmem, umma_desc_join(a_lo + (((kk >> 2) * BWD_KV_HALF + (kk & 3) * 32) >> 4), HI),
                        umma_desc_join(b_lo + (((kk >> 2) * BWD_Q_HALF + (kk & 3) * 32) >> 4), HI), IDESC_S, kk > 0);
        };
        // D[128 kv, 128 d] += A_tmem[128 kv, 64 q] * B[64 q, 128 d]  (B MN-major: rows are q)
        auto issue_acc = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem, bool first) {
          const uint32_t b_lo = umma_desc_lo(b_smem, BWD_Q_HALF);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts_f16(d_tmem, a_tmem + kk * 8, umma_desc_join(b_lo + ((kk * 2048) >> 4), HI), IDESC_ACC,
                        (!first) || kk > 0);
        };
        // D[128 d, 64 q] = K^T[128 d, 128 kv] * dS^T[128 kv, 64 q]  (both MN-major: rows are kv)
        const uint32_t kT_lo = umma_desc_lo(sK, BWD_KV_HALF);
        auto issue_dq = [&](uint32_t ds_smem) {
          const uint32_t b_lo = umma_desc_lo(ds_smem, BWD_DS_BYTES);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss_f16(tmem_base + TM_DQ, umma_desc_join(kT_lo + ((kk * 2048) >> 4), HI),
                        umma_desc_join(b_lo + ((kk * 2048) >> 4), HI), IDESC_DQ, kk > 0);
        };

        bool ok = mbar_wait(&bars[BB_KV_FULL], 0, abort_flag, p.status, BWD_CODE(3, BB_KV_FULL));
        ok = ok && mbar_wait(&bars[BB_Q_FULL + 0], 0, abort_flag, p.status, BWD_CODE(3, BB_Q_FULL));
        if (ok) {
          tc_fence_after();
          issue_st(tmem_base + TM_S, sK, sQ0);
          tc_commit(&bars[BB_S_FULL + 0]);
          issue_st(tmem_base + TM_DP, sV, sQ0 + BWD_Q_BYTES);
          tc_commit(&bars[BB_DP_FULL]);
        }
        for (int j = 0; ok && j < nq; ++j) {
          const int b = j & 1, s = j % BWD_NSQ;
          BWD_TS(2, 0);
          const uint32_t sQ = sQ0 + s * 2 * BWD_Q_BYTES, sDO = sQ + BWD_Q_BYTES;
          if (j + 1 < nq) {
            const int s1 = (j + 1) % BWD_NSQ, b1 = (j + 1) & 1;
            const uint32_t sQ1 = sQ0 + s1 * 2 * BWD_Q_BYTES;
            ok = mbar_wait(&bars[BB_Q_FULL + s1], ((j + 1) / BWD_NSQ) & 1, abort_flag, p.status, BWD_CODE(3, BB_Q_FULL));
            if (!ok) break;
            tc_fence_after();
            BWD_TS(2, 1);
            if (!(p.debug & 8)) issue_st(tmem_base + TM_S + b1 * 64, sK, sQ1);
            tc_commit(&bars[BB_S_FULL + b1]);
            BWD_TS(2, 2);
            ok = mbar_wait(&bars[BB_DP_FREE], j & 1, abort_flag, p.status, BWD_CODE(3, BB_DP_FREE));
            if (!ok) break;
            tc_fence_after();
            BWD_TS(2, 3);
            if (!(p.debug & 8)) issue_st(tmem_base + TM_DP, sV, sQ1 + BWD_Q_BYTES);
            tc_commit(&bars[BB_DP_FULL]);
            BWD_TS(2, 4);
          }
          ok = mbar_wait(&bars[BB_PDS_FULL + b], (j >> 1) & 1, abort_flag, p.status, BWD_CODE(3, BB_PDS_FULL));
          if (!ok) break;
          tc_fence_after();
          BWD_TS(2, 5);
          if (!(p.debug & 16)) {
            issue_acc(tmem_base + TM_DV, tmem_base + TM_S + b * 64, sDO, j == 0);
            issue_acc(tmem_base + TM_DK, tmem_base + TM_S + b * 64 + 32, sQ, j == 0);
          }
          tc_commit(&bars[BB_Q_EMPTY + s]);
          BWD_TS(2, 6);
          if (j > 0) {
            ok = mbar_wait(&bars[BB_DQ_FREE], (j - 1) & 1, abort_flag, p.status, BWD_CODE(3, BB_DQ_FREE));
            if (!ok) break;
            tc_fence_after();
          }
          BWD_TS(2, 7);
          if (!(p.debug & 4)) issue_dq(sDS0 + b * BWD_DS_BYTES);
          tc_commit(&bars[BB_DQ_FULL]);
          tc_commit(&bars[BB_DS_FREE + b]);
          BWD_TS(2, 8);
        }
        if (ok) {
          tc_commit(&bars[BB_ACC_DONE]);
        } else {
          tc_commit(&bars[BB_DRAIN]);
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars[BB_DRAIN], 0) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (!poisoned && !p.accumulate && warp < 8) {
    // No valid K/V row in this tile: its gradients are zero.
    const int r = tid & 127;
    if (kv0 + r < p.skv) {
      float* dst = (warp < 4 ? p.dk_acc : p.dv_acc) + (size_t(slab) * p.skv + kv0 + r) * 128;
#pragma unroll
      for (int i = 0; i < 32; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 13) tmem_dealloc(tmem_base, 512);
}

int launch_bwd_block(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                     const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                     float* dk_acc, float* dv_acc, int accumulate_dkdv, int* status, cudaStream_t st) {
  if (s.dtype == LVX_FP32) return fail(LVX_ERR_DTYPE, "lvx_bwd_block: fp32 inputs are not built yet");
  if (!(sm_scale > 0.f)) return fail(LVX_ERR_SHAPE, "lvx_bwd_block: sm_scale must be positive");
  const int g = s.Hq / s.Hkv;
  const int rows = g * s.Sq;
  const int es = elt_size(s.dtype);
  const uint64_t row_bytes = uint64_t(128) * es;
  const uint64_t slabs = uint64_t(s.B) * s.Hkv;
  CUtensorMap tmQ, tmDO, tmK, tmV;
  int rc;
  if ((rc = make_tmap_3d(&tmQ, s.dtype, q, 128, rows, slabs, row_bytes, row_bytes * rows, 64, 64))) return rc;
  if ((rc = make_tmap_3d(&tmDO, s.dtype, d_o, 128, rows, slabs, row_bytes, row_bytes * rows, 64, 64))) return rc;
  if ((rc = make_tmap_3d(&tmK, s.dtype, k, 128, s.Skv, slabs, row_bytes, row_bytes * s.Skv, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV, s.dtype, v, 128, s.Skv, slabs, row_bytes, row_bytes * s.Skv, 64, 128))) return rc;

  BwdParams p;
  p.rows = rows;
  p.skv = s.Skv;
  p.hkv = s.Hkv;
  p.kv_valid_len = kv_valid_len;
  p.lse = lse;
  p.delta = delta;
  p.scale = sm_scale;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.dq_acc = dq_acc;
  p.dk_acc = dk_acc;
  p.dv_acc = dv_acc;
  p.accumulate = accumulate_dkdv;
  p.status = status;
  {
    const char* dbg = getenv("LVX_BWD_DEBUG");
    p.debug = dbg ? atoi(dbg) : 0;
  }

  dim3 grid((s.Skv + 127) / 128, s.B * s.Hkv, 1);
  cudaError_t e;
  if (s.dtype == LVX_BF16) {
    e = cudaFuncSetAttribute(bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(bwd)");
    bwd_kernel<true><<<grid, BWD_THREADS, BWD_SMEM, st>>>(tmQ, tmDO, tmK, tmV, p);
  } else {
    e = cudaFuncSetAttribute(bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(bwd)");
    bwd_kernel<false><<<grid, BWD_THREADS, BWD_SMEM, st>>>(tmQ, tmDO, tmK, tmV, p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "bwd_kernel launch");
  if (p.debug & 128) {
    static long long ts[3 * 8 * 16];
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(ts, g_bwd_ts, sizeof(ts));
    const char* names[3] = {"softmax", "reducer", "mma"};
    for (int r = 0; r < 3; ++r)
      for (int j = 0; j < 8; ++j) {
        fprintf(stderr, "%s tile %d:", names[r], j + 8);
        for (int k = 0; k < 10; ++k) fprintf(stderr, " %lld", ts[(r * 8 + j) * 16 + k] ? ts[(r * 8 + j) * 16 + k] - ts[0] : -1);
        fprintf(stderr, "\n");
      }
  }
  return LVX_OK;
}

}  // namespace lvx
