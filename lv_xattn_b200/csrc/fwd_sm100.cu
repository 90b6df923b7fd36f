// Forward flash-attention block for sm_100a: one Q block against the K/V shard resident on this GPU.
//
// Work decomposition
//   The g = Hq/Hkv query heads that share a KV head are stacked along M: for one (batch, kv head) the
//   queries form a dense [g*Sq, 128] matrix (they are contiguous in a [B,Hq,Sq,D] tensor), so K/V are
//   read once per group and never expanded. A CTA owns 256 packed rows (two 128-row tiles) and a
//   contiguous range of 128-row K/V tiles (split-KV); it writes the unnormalised partial O plus the
//   running (max, sum) of its range, and the combine kernel merges the splits.
//
// CTA anatomy (320 threads)
//   warps 0-3   softmax for Q tile 0   (thread = row; TMEM lane = row)
//   warps 4-7   softmax for Q tile 1
//   warp  8     TMA producer: Q once, then K/V tiles through a 2-stage ring
//   warp  9     tcgen05.mma issuer (one elected thread); owns the TMEM allocation
//   TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P (16-bit) overwrites S in place.
//   Per K/V tile j and Q tile i:   S_i = Q_i K_j^T (smem x smem) -> softmax -> P_i -> O_i += P_i V_j
//   (TMEM x smem, V consumed MN-major straight from its [kv, d] tile). The issuer interleaves the two
//   Q tiles so that the tensor core works on one tile while the other is in its softmax.
#include "lvx_internal.h"
#include "sm100_prims.cuh"
#include "block_wait.cuh"
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

namespace lvx {

constexpr int FWD_NS = 2;                         // K/V pipeline stages
constexpr int FWD_TILE_BYTES = 128 * 128 * 2;     // one 128x128 16-bit tile
constexpr int FWD_HALF_BYTES = FWD_TILE_BYTES / 2;
constexpr int FWD_OFF_Q = 0;
constexpr int FWD_OFF_K = 2 * FWD_TILE_BYTES;
constexpr int FWD_OFF_V = FWD_OFF_K + FWD_NS * FWD_TILE_BYTES;
constexpr int FWD_OFF_BAR = FWD_OFF_V + FWD_NS * FWD_TILE_BYTES;
constexpr int FWD_SMEM = FWD_OFF_BAR + 256 + 1024;   // + barriers + alignment slack
constexpr int FWD_THREADS = 320;

enum {
  FB_Q_FULL = 0,
  FB_K_FULL = 1,
  FB_K_EMPTY = FB_K_FULL + FWD_NS,
  FB_V_FULL = FB_K_EMPTY + FWD_NS,
  FB_V_EMPTY = FB_V_FULL + FWD_NS,
  FB_S_FULL = FB_V_EMPTY + FWD_NS,
  FB_P_FULL = FB_S_FULL + 2,
  FB_O_DONE = FB_P_FULL + 2,
  FB_DRAIN = FB_O_DONE + 2,
  FB_COUNT = FB_DRAIN + 1
};

struct FwdParams {
  int rows;             // g * Sq
  int skv;              // K/V rows in the shard
  int hkv;              // KV heads (to find the batch index of a CTA)
  int kv_slabs;         // B*Hkv: query slab z reads K/V slab z % kv_slabs (several query blocks per K/V)
  int nsplit;
  int tiles_per_split;
  const int32_t* kv_valid_len;
  float scale_log2;     // sm_scale * log2(e)
  float* o_part;        // [B*Hkv][nsplit][rows][128]
  float* ml_part;       // [B*Hkv][nsplit][rows][2]
  BlockWait bw;         // query blocks that may still be arriving from other ranks
  int* status;
};

// Development aid, compiled only with -DLVX_DEV_STAMPS (never in the shipped library): cycle stamps of CTA
// (0,0,0), K/V tiles 4..11, 8 slots per tile and role, printed by the launcher.
#ifdef LVX_DEV_STAMPS
__device__ long long g_fwd_ts[3 * 8 * 8];
#define FWD_TS(role, slot)                                                                              \
  do {                                                                                                  \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && j >= 4 && j < 12)         \
      g_fwd_ts[((role) * 8 + (j - 4)) * 8 + (slot)] = clock64();                                        \
  } while (0)
#else
#define FWD_TS(role, slot) do {} while (0)
#endif

#define FWD_CODE(role, bar) (LVX_DEV_TIMEOUT_BASE | 0x100 | ((role) << 5) | (bar))

template <bool IS_BF16>
__global__ void __launch_bounds__(FWD_THREADS, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FWD_OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + FB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mb = blockIdx.x, split = blockIdx.z;
  const int kvs = blockIdx.y % p.kv_slabs;      // K/V slab of this query slab
  // query blocks are scheduled starting with this rank's own (which is in place at launch)
  const int nblk = gridDim.y / p.kv_slabs;
  const int blk = (p.bw.first_blk + int(blockIdx.y) / p.kv_slabs) % nblk;
  const int bh = blk * p.kv_slabs + kvs;        // query slab
  const int batch = kvs / p.hkv;

  // K/V tile range of this CTA, clipped to the valid prefix of the shard.
  int valid = p.skv;
  if (p.kv_valid_len) valid = min(valid, max(0, p.kv_valid_len[batch]));
  const int valid_tiles = (valid + 127) >> 7;
  const int tile0 = split * p.tiles_per_split;
  const int n = max(0, min(tile0 + p.tiles_per_split, valid_tiles) - tile0);
  // columns of the last tile of this CTA that are valid (128 unless it is the ragged end of the shard)
  const int last_cols = (n > 0 && tile0 + n == valid_tiles && (valid & 127)) ? (valid & 127) : 128;

  const bool poisoned = (*reinterpret_cast<volatile int*>(p.status) != 0);

  if (tid == 0) {
    mbar_init(&bars[FB_Q_FULL], 1);
    for (int s = 0; s < FWD_NS; ++s) {
      mbar_init(&bars[FB_K_FULL + s], 1);
      mbar_init(&bars[FB_K_EMPTY + s], 1);
      mbar_init(&bars[FB_V_FULL + s], 1);
      mbar_init(&bars[FB_V_EMPTY + s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[FB_S_FULL + i], 1);
      mbar_init(&bars[FB_P_FULL + i], 4);      // one arrival per softmax warp
      mbar_init(&bars[FB_O_DONE + i], 1);
    }
    mbar_init(&bars[FB_DRAIN], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (!poisoned && n > 0) {
    if (warp < 8) {
      // =========================== softmax warpgroups ===========================
      const int wg = warp >> 2;
      const int row_in_tile = (warp & 3) * 32 + lane;
      const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t tS = tmem_base + wg * 128 + lane_sel;
      const uint32_t tO = tmem_base + 256 + wg * 128 + lane_sel;
      const float c = p.scale_log2;
      float m = -INFINITY, l = 0.f;
      bool alive = true;
      for (int j = 0; j < n; ++j) {
        if (!mbar_wait(&bars[FB_S_FULL + wg], j & 1, abort_flag, p.status, FWD_CODE(wg, FB_S_FULL), p.bw.pipe_limit)) {
          alive = false;
          break;
        }
        tc_fence_after();
        if ((warp & 3) == 0) FWD_TS(wg, 0);
        // Fast path (every tile but the first and a ragged last one): the exponentials are taken against the
        // running max as it stands and P is held in registers. The running max is only a reference point:
        // (m, l, O) stay consistent whatever it is, as long as nothing overflows. So if the row sums of the
        // tile stay small (the usual case once the max has settled) P is stored and the tile is done, without a
        // row-max pass at all. Otherwise S is still intact in TMEM and the exact path below runs.
        // A lone warp per scheduler pays the issue time of every instruction in full (measured: 8 cycles per
        // ex2, 4 per cvt.bf16x2, 2 per packed fma/add), so the loop body is kept to the bare minimum.
        bool done = false;
        if (j > 0 && !(j == n - 1 && last_cols < 128)) {
          uint32_t pk[2][32];
          uint64_t sum_a = f32x2(0.f, 0.f), sum_b = f32x2(0.f, 0.f);
          const uint64_t c2 = f32x2(c, c), nm2 = f32x2(-m, -m);
          auto chunk = [&](const uint32_t (&b)[32], uint32_t* out) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float s0 = __uint_as_float(b[4 * i]), s1 = __uint_as_float(b[4 * i + 1]);
              const float s2 = __uint_as_float(b[4 * i + 2]), s3 = __uint_as_float(b[4 * i + 3]);
              float x0, x1, x2, x3;
              f32x2_get(fma2(f32x2(s0, s1), c2, nm2), x0, x1);
              f32x2_get(fma2(f32x2(s2, s3), c2, nm2), x2, x3);
              const float e0 = ex2f(x0), e1 = ex2f(x1), e2 = ex2f(x2), e3 = ex2f(x3);
              sum_a = add2(sum_a, f32x2(e0, e1));
              sum_b = add2(sum_b, f32x2(e2, e3));
              out[2 * i] = IS_BF16 ? pack_bf16x2(e0, e1) : pack_f16x2(e0, e1);
              out[2 * i + 1] = IS_BF16 ? pack_bf16x2(e2, e3) : pack_f16x2(e2, e3);
            }
          };
          // One TMEM round trip costs about 400 cycles whatever its width and tcgen05.wait::ld waits for
          // every load in flight, so the four loads go out together and are waited for once.
          {
            uint32_t sv[4][32];
            tmem_ld32(tS + 0, sv[0]);
            tmem_ld32(tS + 32, sv[1]);
            tmem_ld32(tS + 64, sv[2]);
            tmem_ld32(tS + 96, sv[3]);
            tc_wait_ld();
#pragma unroll
            for (int q = 0; q < 4; ++q) chunk(sv[q], &pk[0][0] + q * 16);
          }
          // Guard: every term is positive, so a row sum of at most 2^14 bounds each P below 2^14 (no overflow
          // in either 16-bit format); an infinity or a NaN fails the comparison as well.
          float t0, t1, t2, t3;
          f32x2_get(sum_a, t0, t1);
          f32x2_get(sum_b, t2, t3);
          const float tile_sum = (t0 + t1) + (t2 + t3);
          if (__all_sync(0xffffffffu, tile_sum <= 16384.f)) {
            if ((warp & 3) == 0) FWD_TS(wg, 2);
            tmem_st32(tS + 0, pk[0]);
            tmem_st32(tS + 32, pk[1]);
            l += tile_sum;
            done = true;
          }
        }
        if (!done) {
          uint32_t s[4][32];
          tmem_ld32(tS + 0, s[0]);
          tmem_ld32(tS + 32, s[1]);
          tmem_ld32(tS + 64, s[2]);
          tmem_ld32(tS + 96, s[3]);
          tc_wait_ld();
          if ((warp & 3) == 0) FWD_TS(wg, 1);
          if (j == n - 1 && last_cols < 128) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (q * 32 + i >= last_cols) s[q][i] = 0xff800000u;  // -inf
          }
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            mx0 = fmaxf(mx0, __uint_as_float(s[0][i]));
            mx1 = fmaxf(mx1, __uint_as_float(s[1][i]));
            mx2 = fmaxf(mx2, __uint_as_float(s[2][i]));
            mx3 = fmaxf(mx3, __uint_as_float(s[3][i]));
          }
          const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * c);
          // The running max is only raised when it would grow by more than 2^8; P then stays below 256
          // and the accumulator rarely needs rescaling. (m, l, O) remain mutually consistent.
          const bool grow = m_new > m + 8.f;
          float alpha = 1.f;
          if (grow) {
            alpha = ex2f(m - m_new);
            m = m_new;
            l *= alpha;
          }
          if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t o[32];
              tmem_ld32(tO + q * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + q * 32, o);
            }
          }
          if ((warp & 3) == 0) FWD_TS(wg, 2);
          const float moff = (m == -INFINITY) ? 0.f : m;
          float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float a0 = ex2f(fmaf(__uint_as_float(s[2 * h][2 * i]), c, -moff));
              const float a1 = ex2f(fmaf(__uint_as_float(s[2 * h][2 * i + 1]), c, -moff));
              const float b0 = ex2f(fmaf(__uint_as_float(s[2 * h + 1][2 * i]), c, -moff));
              const float b1 = ex2f(fmaf(__uint_as_float(s[2 * h + 1][2 * i + 1]), c, -moff));
              sum0 += a0 + a1;
              sum1 += b0 + b1;
              pk[i] = IS_BF16 ? pack_bf16x2(a0, a1) : pack_f16x2(a0, a1);
              pk[16 + i] = IS_BF16 ? pack_bf16x2(b0, b1) : pack_f16x2(b0, b1);
            }
            tmem_st32(tS + h * 32, pk);
          }
          l += sum0 + sum1;
        }
        if ((warp & 3) == 0) FWD_TS(wg, 3);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[FB_P_FULL + wg]);
        if ((warp & 3) == 0) FWD_TS(wg, 4);
      }
      // ------------------------------- epilogue -------------------------------
      const int row = mb * 256 + wg * 128 + row_in_tile;
      if (alive) alive = mbar_wait(&bars[FB_O_DONE + wg], 0, abort_flag, p.status, FWD_CODE(wg, FB_O_DONE), p.bw.pipe_limit);
      tc_fence_after();
      if (alive) {
        const size_t prow = (size_t(bh) * p.nsplit + split) * p.rows + row;
        float4* dst = reinterpret_cast<float4*>(p.o_part + prow * 128);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t o[32];
          tmem_ld32(tO + q * 32, o);
          tc_wait_ld();
          if (row < p.rows) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[q * 8 + i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                           __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
          }
        }
        if (row < p.rows) *reinterpret_cast<float2*>(p.ml_part + prow * 2) = make_float2(m, l);
      }
    } else if (warp == 8) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        const bool q_here = wait_block(p.bw, blk, abort_flag, p.status);
        if (q_here) {
          fence_async_global();
          mbar_arrive_expect_tx(&bars[FB_Q_FULL], 2 * FWD_TILE_BYTES);
          for (int t = 0; t < 2; ++t)
            for (int h = 0; h < 2; ++h)
              tma_load_3d(smem + FWD_OFF_Q + t * FWD_TILE_BYTES + h * FWD_HALF_BYTES, &tmQ, &bars[FB_Q_FULL], h * 64,
                          mb * 256 + t * 128, bh);
        }
        int k_issued = 0, v_issued = 0;
        for (int j = 0; q_here && j < n; ++j) {
          const int s = j % FWD_NS;
          const uint32_t ph = (j / FWD_NS) & 1;
          const int y = (tile0 + j) * 128;
          if (!mbar_wait(&bars[FB_K_EMPTY + s], ph ^ 1, abort_flag, p.status, FWD_CODE(2, FB_K_EMPTY), p.bw.pipe_limit)) break;
          mbar_arrive_expect_tx(&bars[FB_K_FULL + s], FWD_TILE_BYTES);
          tma_load_3d(smem + FWD_OFF_K + s * FWD_TILE_BYTES, &tmK, &bars[FB_K_FULL + s], 0, y, kvs);
          tma_load_3d(smem + FWD_OFF_K + s * FWD_TILE_BYTES + FWD_HALF_BYTES, &tmK, &bars[FB_K_FULL + s], 64, y, kvs);
          k_issued = j + 1;
          if (!mbar_wait(&bars[FB_V_EMPTY + s], ph ^ 1, abort_flag, p.status, FWD_CODE(2, FB_V_EMPTY), p.bw.pipe_limit)) break;
          mbar_arrive_expect_tx(&bars[FB_V_FULL + s], FWD_TILE_BYTES);
          tma_load_3d(smem + FWD_OFF_V + s * FWD_TILE_BYTES, &tmV, &bars[FB_V_FULL + s], 0, y, kvs);
          tma_load_3d(smem + FWD_OFF_V + s * FWD_TILE_BYTES + FWD_HALF_BYTES, &tmV, &bars[FB_V_FULL + s], 64, y, kvs);
          v_issued = j + 1;
        }
        // A CTA that is giving up must not leave while a copy into its shared memory is in flight.
        if (*abort_flag) {
          auto drain = [&](uint64_t* bar, uint32_t ph) {
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, ph) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
          };
          if (q_here) drain(&bars[FB_Q_FULL], 0);
          for (int j = max(0, k_issued - FWD_NS); j < k_issued; ++j) drain(&bars[FB_K_FULL + j % FWD_NS], (j / FWD_NS) & 1);
          for (int j = max(0, v_issued - FWD_NS); j < v_issued; ++j) drain(&bars[FB_V_FULL + j % FWD_NS], (j / FWD_NS) & 1);
        }
      }
    } else {
      // =========================== MMA issuer ===========================
      // The whole warp walks the loop and one elected lane issues: with warp-uniform control flow the
      // descriptor arithmetic stays on the uniform datapath, and the issuing warp needs few issue slots
      // per MMA (it shares its scheduler with two softmax warps, and the tensor pipe queues little: every
      // cycle the issuer is late is a cycle the pipe idles).
      {
        constexpr uint32_t FMT = IS_BF16 ? UMMA_BF16 : UMMA_F16;
        constexpr uint32_t IDESC_QK = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
        constexpr uint32_t IDESC_PV = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_MN_MAJOR, 128, 128);
        const uint32_t sQ = smem_u32(smem + FWD_OFF_Q);
        const uint32_t sK = smem_u32(smem + FWD_OFF_K);
        const uint32_t sV = smem_u32(smem + FWD_OFF_V);

        constexpr uint32_t HI = umma_desc_hi(1024);
        auto issue_qk = [&](int i, int stage) {
          const uint32_t a_lo = umma_desc_lo(sQ + i * FWD_TILE_BYTES, 16);
          const uint32_t b_lo = umma_desc_lo(sK + stage * FWD_TILE_BYTES, 16);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint32_t off = ((kk >> 2) * FWD_HALF_BYTES + (kk & 3) * 32) >> 4;
              umma_ss_f16(tmem_base + i * 128, umma_desc_join(a_lo + off, HI), umma_desc_join(b_lo + off, HI),
                          IDESC_QK, kk > 0);
            }
          }
          __syncwarp();
        };
        auto issue_pv = [&](int i, int stage, bool first) {
          const uint32_t b_lo = umma_desc_lo(sV + stage * FWD_TILE_BYTES, FWD_HALF_BYTES);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ts_f16(tmem_base + 256 + i * 128, tmem_base + i * 128 + kk * 8,
                          umma_desc_join(b_lo + ((kk * 2048) >> 4), HI), IDESC_PV, (!first) || kk > 0);
          }
          __syncwarp();
        };
        auto commit = [&](uint64_t* bar) {
          if (elect_one()) tc_commit(bar);
          __syncwarp();
        };

        bool ok = mbar_wait(&bars[FB_Q_FULL], 0, abort_flag, p.status, FWD_CODE(3, FB_Q_FULL), p.bw.pipe_limit);
        ok = ok && mbar_wait(&bars[FB_K_FULL + 0], 0, abort_flag, p.status, FWD_CODE(3, FB_K_FULL), p.bw.pipe_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          tc_fence_after();
          issue_qk(0, 0);
          commit(&bars[FB_S_FULL + 0]);
          issue_qk(1, 0);
          commit(&bars[FB_S_FULL + 1]);
          commit(&bars[FB_K_EMPTY + 0]);
        }
        for (int j = 0; ok && j < n; ++j) {
          const int s = j % FWD_NS;
          const uint32_t ph = (j / FWD_NS) & 1;
          const int s1 = (j + 1) % FWD_NS;
          const uint32_t ph1 = ((j + 1) / FWD_NS) & 1;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            if (!ok) break;
            FWD_TS(2, i * 4 + 0);
            ok = mbar_wait(&bars[FB_P_FULL + i], j & 1, abort_flag, p.status, FWD_CODE(3, FB_P_FULL), p.bw.pipe_limit);
            FWD_TS(2, i * 4 + 1);
            if (ok && i == 0) ok = mbar_wait(&bars[FB_V_FULL + s], ph, abort_flag, p.status, FWD_CODE(3, FB_V_FULL), p.bw.pipe_limit);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            issue_pv(i, s, j == 0);
            FWD_TS(2, i * 4 + 2);
            if (i == 1) commit(&bars[FB_V_EMPTY + s]);
            if (j + 1 < n) {
              if (i == 0) {
                ok = mbar_wait(&bars[FB_K_FULL + s1], ph1, abort_flag, p.status, FWD_CODE(3, FB_K_FULL), p.bw.pipe_limit);
                ok = __all_sync(0xffffffffu, ok);
              }
              if (!ok) break;
              tc_fence_after();
              issue_qk(i, s1);
              FWD_TS(2, i * 4 + 3);
              commit(&bars[FB_S_FULL + i]);
              if (i == 1) commit(&bars[FB_K_EMPTY + s1]);
            } else {
              commit(&bars[FB_O_DONE + i]);
            }
          }
        }
        if (!ok) {
          // wind down: let every MMA already issued finish before TMEM is released
          commit(&bars[FB_DRAIN]);
          long long t0 = clock64();
          while (!mbar_try_wait(&bars[FB_DRAIN], 0) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (!poisoned && warp < 8) {
    // Nothing valid in this CTA's K/V range: the empty partial (O = 0, max = -inf, sum = 0).
    const int row = mb * 256 + tid;
    if (row < p.rows) {
      const size_t prow = (size_t(bh) * p.nsplit + split) * p.rows + row;
      float4* dst = reinterpret_cast<float4*>(p.o_part + prow * 128);
#pragma unroll
      for (int i = 0; i < 32; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float2*>(p.ml_part + prow * 2) = make_float2(-INFINITY, 0.f);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------
static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_num_sms = n;
    else
      g_num_sms = 148;
  }
  return g_num_sms;
}

FwdPlan plan_fwd(const lvx_shape& s) {
  FwdPlan p;
  const int g = s.Hq / s.Hkv;
  p.rows = g * s.Sq;
  p.m_blocks = (p.rows + 255) / 256;
  p.kv_tiles = (s.Skv + 127) / 128;
  const int qb = q_blocks_of(s);
  const long base = long(p.m_blocks) * s.B * s.Hkv * qb;
  const int sms = 148;  // plan for the full part; a fixed figure keeps the workspace size device-independent
  int best = 1;
  double best_cost = 1e300;
  const int max_split = p.kv_tiles < 64 ? (p.kv_tiles > 0 ? p.kv_tiles : 1) : 64;
  for (int ns = 1; ns <= max_split; ++ns) {
    const long ctas = base * ns;
    const long waves = (ctas + sms - 1) / sms;
    const int tps = (p.kv_tiles + ns - 1) / ns;
    // 3 tiles' worth of fixed cost per CTA (prologue, pipeline fill, epilogue + partial write-out)
    const double cost = double(waves) * (tps + 3);
    if (cost < best_cost * 0.995) {
      best_cost = cost;
      best = ns;
    }
  }
  p.nsplit = best;
  p.tiles_per_split = p.kv_tiles > 0 ? (p.kv_tiles + best - 1) / best : 0;
  p.o_part_bytes = size_t(qb) * s.B * s.Hkv * p.nsplit * p.rows * 128 * sizeof(float);
  p.ml_part_bytes = size_t(qb) * s.B * s.Hkv * p.nsplit * p.rows * 2 * sizeof(float);
  p.ml_part_bytes = (p.ml_part_bytes + 255) & ~size_t(255);
  p.o_part_bytes = (p.o_part_bytes + 255) & ~size_t(255);
  return p;
}

int launch_fwd_block(const lvx_shape& s, const FwdPlan& pl, const void* q, const void* k, const void* v,
                     const int32_t* kv_valid_len, float sm_scale, float* o_part, float* ml_part, int* status,
                     cudaStream_t st, const lvx_block_wait* bw) {
  if (!(sm_scale > 0.f)) return fail(LVX_ERR_SHAPE, "lvx_fwd_block: sm_scale must be positive");
  if (s.dtype == LVX_FP32) return launch_fwd_block_fp32(s, pl, q, k, v, kv_valid_len, sm_scale, o_part, ml_part, st);
  (void)num_sms;
  CUtensorMap tmQ, tmK, tmV;
  const int es = elt_size(s.dtype);
  const uint64_t row_bytes = uint64_t(128) * es;
  const int qb = q_blocks_of(s);
  int rc = make_tmap_3d(&tmQ, s.dtype, q, 128, pl.rows, uint64_t(qb) * s.B * s.Hkv, row_bytes, row_bytes * pl.rows, 64,
                        128);
  if (rc) return rc;
  // A shard with no K/V rows still launches (every CTA writes the empty partial); the maps then
  // describe one dummy row of Q so that encoding succeeds and nothing is ever loaded through them.
  const void* kb = s.Skv > 0 ? k : q;
  const void* vb = s.Skv > 0 ? v : q;
  const uint64_t kvrows = s.Skv > 0 ? s.Skv : 1;
  rc = make_tmap_3d(&tmK, s.dtype, kb, 128, kvrows, uint64_t(s.B) * s.Hkv, row_bytes, row_bytes * kvrows, 64, 128);
  if (rc) return rc;
  rc = make_tmap_3d(&tmV, s.dtype, vb, 128, kvrows, uint64_t(s.B) * s.Hkv, row_bytes, row_bytes * kvrows, 64, 128);
  if (rc) return rc;

  FwdParams p;
  p.rows = pl.rows;
  p.skv = s.Skv;
  p.hkv = s.Hkv;
  p.kv_slabs = s.B * s.Hkv;
  p.nsplit = pl.nsplit;
  p.tiles_per_split = pl.tiles_per_split;
  p.kv_valid_len = kv_valid_len;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.o_part = o_part;
  p.ml_part = ml_part;
  p.status = status;
  p.bw = make_block_wait(bw, qb);

  dim3 grid(pl.m_blocks, qb * s.B * s.Hkv, pl.nsplit);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
    if (e == cudaSuccess) kern<<<grid, FWD_THREADS, FWD_SMEM, st>>>(tmQ, tmK, tmV, p);
  };
  if (s.dtype == LVX_BF16) go(fwd_kernel<true>);
  else go(fwd_kernel<false>);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(fwd)");
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "fwd_kernel launch");
#ifdef LVX_DEV_STAMPS
  {
    static long long ts[3 * 8 * 8];
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(ts, g_fwd_ts, sizeof(ts));
    const char* names[3] = {"softmax0", "softmax1", "mma"};
    for (int r = 0; r < 3; ++r)
      for (int j = 0; j < 8; ++j) {
        fprintf(stderr, "%s tile %d:", names[r], j + 4);
        for (int k2 = 0; k2 < 8; ++k2) fprintf(stderr, " %lld", ts[(r * 8 + j) * 8 + k2] ? ts[(r * 8 + j) * 8 + k2] - ts[0] : -1);
        fprintf(stderr, "\n");
      }
  }
#endif
  return LVX_OK;
}

}  // namespace lvx
