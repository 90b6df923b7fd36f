// Backward flash-attention block for sm_100a.
//
// A work item is one 128-row K/V tile of one (batch, kv head); a CTA walks over the packed query rows of the
// group for it (g*Sq rows of every query block, 128 at a time). The grid is persistent -- one CTA per SM, items
// handed out round-robin -- so that the fixed costs of an item (launch, barrier and TMEM set-up, the K/V load, the
// dK/dV write-out and the last dQ^T drain, about 8 us against 3.3 us per query tile) overlap with the next item's
// start instead of standing between two CTAs: all barrier phases simply keep counting tiles and items across the
// items of a CTA. Everything is computed in the transposed frame, so
// that the softmax statistics are per column and no row reduction is needed:
//     S^T  = K Q^T            (smem x smem)       P^T  = exp2(S^T*c - lse[col])
//     dP^T = V dO^T           (smem x smem)       dS^T = P^T o (dP^T - delta[col])
//     dV  += P^T  dO          (TMEM x smem, dO consumed MN-major)
//     dK  += dS^T Q           (smem x smem: dS^T read K-major, Q consumed MN-major)
//     dQ^T = K^T dS^T         (smem x smem, both MN-major)
// dK/dV stay in TMEM for the whole walk (summing over the query heads of the group and over the query blocks on
// the way) and are written once; dQ^T tiles are reduce-added (red.global.add.f32) into the fp32 dQ accumulator.
// The softmax scale is applied once on the way out (dK, dQ).
//
// Every tcgen05.mma is 128 x 128 x 16 (64 cycles of tensor pipe; an N = 64 instruction takes 48, so 64-wide query
// tiles, which would leave TMEM room for double buffering, run the pipe at two thirds). With 128-wide tiles the
// 512 TMEM columns are exactly
//     dK [0,128)  dV [128,256)  X [256,384)  Y [384,512)
//     X: S^T (fp32)  ->  P^T (16-bit, 64 columns)                  Y: dP^T (fp32)  ->  dQ^T (fp32)
// dS^T lives in shared memory only: it is the B operand of dQ^T (read MN-major) and the A operand of dK (the
// same bytes read K-major), which frees X as soon as dV has consumed P^T. The issue order per tile is
// dV(j), S^T(j+1), dQ^T(j), dK(j), dP^T(j+1). What keeps the tensor pipe fed is that little else sits on the
// critical path:
//   * the P^T half of the elementwise work (the exp) starts as soon as S^T of the tile is complete, i.e. while
//     dP^T is still in the pipe; only the dS^T half waits for dP^T;
//   * the dQ^T tile is taken out of TMEM and reduce-added by eight dedicated drain warps. The reduce traffic
//     (64 KB per tile) is what bounds the kernel: with all SMs adding into L2 it moves at ~14 B/clk/SM, about
//     4,800 cycles per tile against 2,560 cycles of MMA work, so it must not be issued by the warps that
//     produce P^T/dS^T.
//
// CTA anatomy (832 threads, 72 registers each)
//   warps 0-15  compute: warp w works on K/V rows 32*(w%4).. (its TMEM lane quarter) and query columns
//               32*(w/4)..; they also write dK/dV at the end
//   warps 16-23 dQ drain: warp w takes lane quarter w%4 of dQ^T (rows = head dim) and 64 of its query columns,
//               all loaded at once so that Y is free again right away (a warp sustains about one reduce-add
//               per 60-75 cycles, so eight warps are needed)
//   warp  24    TMA producer: K,V once; Q,dO tiles through a 2-stage ring
//   warp  25    tcgen05.mma issuer; owns the TMEM allocation
#include "lvx_internal.h"
#include "sm100_prims.cuh"
#include "block_wait.cuh"
#include <cuda_fp16.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <algorithm>

namespace lvx {

constexpr int BWD_NSQ = 2;                      // Q/dO pipeline stages
constexpr int BWD_TILE = 128 * 128 * 2;         // one 128x128 16-bit tile (K, V, Q, dO, dS^T)
constexpr int BWD_HALF = BWD_TILE / 2;          // one 64-column half (a 128-byte-wide box of 128 rows)
constexpr int BWD_OFF_K = 0;
constexpr int BWD_OFF_V = BWD_TILE;
constexpr int BWD_OFF_Q = 2 * BWD_TILE;                          // stage s: Q at +s*2*TILE, dO right after
constexpr int BWD_OFF_DS = BWD_OFF_Q + BWD_NSQ * 2 * BWD_TILE;
constexpr int BWD_OFF_STAT = BWD_OFF_DS + BWD_TILE;              // [2][lse2 128 | delta 128]
constexpr int BWD_OFF_BAR = BWD_OFF_STAT + 2 * 256 * 4;
constexpr int BWD_SMEM = BWD_OFF_BAR + 256;
constexpr int BWD_COMPUTE_WARPS = 16;
constexpr int BWD_DRAIN_WARPS = 8;
constexpr int BWD_WARP_TMA = BWD_COMPUTE_WARPS + BWD_DRAIN_WARPS;
constexpr int BWD_WARP_MMA = BWD_WARP_TMA + 1;
constexpr int BWD_THREADS = (BWD_WARP_MMA + 1) * 32;
static_assert(BWD_SMEM <= 232448, "shared memory budget");

constexpr uint32_t TM_DK = 0, TM_DV = 128, TM_X = 256, TM_Y = 384;

enum {
  BB_KV_FULL = 0,
  BB_Q_FULL = 1,                       // x2
  BB_Q_EMPTY = BB_Q_FULL + BWD_NSQ,    // x2
  BB_S_FULL = BB_Q_EMPTY + BWD_NSQ,
  BB_DP_FULL,
  BB_X_LOADED,
  BB_P_FULL,
  BB_DS_FREE,                          // dQ^T and dK of a tile have both finished reading dS^T
  BB_PDS_FULL,
  BB_DQ_FULL,
  BB_DQ_FREE,
  BB_ACC_DONE,
  BB_DRAIN,
  BB_STAT_FULL,                        // x2
  BB_COUNT = BB_STAT_FULL + 2
};

struct BwdParams {
  int rows;            // g * Sq
  int skv;
  int hkv;
  int nblk;            // query blocks per K/V batch entry (query slab = kv slab + block * kv_slabs)
  int kv_slabs;        // B*Hkv
  int kv_tiles;        // 128-row K/V tiles per slab
  int nitems;          // kv_tiles * kv_slabs work items, item w = (tile w % kv_tiles, slab w / kv_tiles)
  const int32_t* kv_valid_len;
  const float* lse;    // [nblk*B*Hq*Sq]  == [query slab][rows]
  const float* delta;
  float scale;         // sm_scale
  float scale_log2;    // sm_scale * log2(e)
  float* dq_acc;       // [slab][rows][128]
  float* dk_acc;       // [slab][skv][128]  (fp32; 16-bit when accumulate == 2)
  float* dv_acc;
  int accumulate;      // 0 overwrite fp32, 1 add to fp32, 2 write the finished gradient in the input dtype
  BlockWait bw;        // query blocks that may still be arriving from other ranks
  int* status;
};

// Development aid, compiled only with -DLVX_DEV_STAMPS (never in the shipped library): cycle stamps of CTA
// (0,0), tiles 4..11, 16 slots per tile and role, printed by the launcher.
#ifdef LVX_DEV_STAMPS
__device__ long long g_bwd_ts[2 * 8 * 16];
#define BWD_TS(role, slot)                                                                         \
  do {                                                                                             \
    if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && j >= 4 && j < 12)                       \
      g_bwd_ts[((role) * 8 + (j - 4)) * 16 + (slot)] = clock64();                                  \
  } while (0)
#else
#define BWD_TS(role, slot) do {} while (0)
#endif

#define BWD_CODE(role, bar) (LVX_DEV_TIMEOUT_BASE | 0x200 | ((role) << 5) | (bar))

template <bool IS_BF16>
__device__ __forceinline__ float2 unpack16x2(uint32_t v) {
  if (IS_BF16) return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

template <bool IS_BF16>
__global__ void __launch_bounds__(BWD_THREADS, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
           const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BWD_OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_stat = reinterpret_cast<float*>(smem + BWD_OFF_STAT);   // [2][256]: lse*log2(e) then delta

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  struct Item {
    int slab, kv0, valid;
    bool live, partial;      // at least one valid K/V row in the tile; some rows of the tile are padding
  };
  auto item_of = [&](int w) {
    Item it;
    it.slab = w / p.kv_tiles;
    it.kv0 = (w % p.kv_tiles) * 128;
    it.valid = p.skv;
    if (p.kv_valid_len) it.valid = min(it.valid, max(0, p.kv_valid_len[it.slab / p.hkv]));
    it.live = it.kv0 < it.valid;
    it.partial = it.valid < it.kv0 + 128;
    return it;
  };
  const int nq = (p.rows + 127) >> 7;         // 128-row tiles per query block
  const int ntot = nq * p.nblk;               // tiles walked per item: all blocks, one after the other
  // The operand descriptors assume 1024-byte aligned tiles; refuse to run otherwise.
  const bool misaligned = (smem_u32(smem) & 1023u) != 0;
  if (misaligned && tid == 0) atomicCAS(p.status, 0, BWD_CODE(7, 0));
  const bool poisoned = misaligned || (*reinterpret_cast<volatile int*>(p.status) != 0);

  if (tid == 0) {
    mbar_init(&bars[BB_KV_FULL], 1);
    for (int s = 0; s < BWD_NSQ; ++s) {
      mbar_init(&bars[BB_Q_FULL + s], 1);
      mbar_init(&bars[BB_Q_EMPTY + s], 1);
    }
    mbar_init(&bars[BB_S_FULL], 1);
    mbar_init(&bars[BB_DP_FULL], 1);
    mbar_init(&bars[BB_X_LOADED], BWD_COMPUTE_WARPS);
    mbar_init(&bars[BB_P_FULL], BWD_COMPUTE_WARPS);
    mbar_init(&bars[BB_DS_FREE], 1);
    mbar_init(&bars[BB_PDS_FULL], BWD_COMPUTE_WARPS);
    mbar_init(&bars[BB_DQ_FULL], 1);
    mbar_init(&bars[BB_DQ_FREE], BWD_DRAIN_WARPS);
    mbar_init(&bars[BB_ACC_DONE], 1);
    mbar_init(&bars[BB_DRAIN], 1);
    for (int b = 0; b < 2; ++b) mbar_init(&bars[BB_STAT_FULL + b], 8);   // warps 0-7 publish
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == BWD_WARP_MMA) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Every role walks the same items in the same order and keeps the same two counters: `it` = live items done,
  // `jj0` = query tiles done before the current item. Barriers that complete once per tile take their phase from
  // jj = jj0 + j, those that complete once per item (KV_FULL, ACC_DONE) from `it`.
  if (!poisoned) {
    if (warp < BWD_COMPUTE_WARPS) {
      // =========================== compute warps ===========================
      const int quarter = warp & 3;                         // TMEM lane quarter
      const int cg = warp >> 2;                             // 32-column group of the query tile
      const int r = quarter * 32 + lane;                    // K/V row inside the tile (head-dim index in the drain)
      const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
      const uint32_t tX = tmem_base + TM_X + lane_sel, tY = tmem_base + TM_Y + lane_sel;
      const float c = p.scale_log2;
      bool alive = true;
      int it = 0, jj0 = 0;
      for (int w = blockIdx.x; alive && w < p.nitems; w += gridDim.x) {
        const Item I = item_of(w);
        if (!I.live) {
          // No valid K/V row in this tile: its gradients are zero.
          if (p.accumulate != 1 && warp < 8 && I.kv0 + (tid & 127) < p.skv) {
            const size_t off = (size_t(I.slab) * p.skv + I.kv0 + (tid & 127)) * 128;
            float* base = warp < 4 ? p.dk_acc : p.dv_acc;
            if (p.accumulate == 2) {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(base) + off);
#pragma unroll
              for (int i = 0; i < 16; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) reinterpret_cast<float4*>(base + off)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
          continue;
        }
        const bool row_valid = (I.kv0 + r) < I.valid;
        // tile j -> (query slab, first row inside the block); blocks are walked starting with this rank's own
        auto tile_slab = [&](int j) { return I.slab + ((p.bw.first_blk + j / nq) % p.nblk) * p.kv_slabs; };
        auto tile_row0 = [&](int j) { return (j % nq) * 128; };
        // Per-column statistics of a query tile: threads 0-127 fetch lse, 128-255 delta (warps 0-7).
        auto fetch_stat = [&](int j) -> float {
          // the first tile of a block that another rank sends: its statistics must have landed
          if (tid < 256 && (j % nq) == 0 && !wait_block(p.bw, (p.bw.first_blk + j / nq) % p.nblk, abort_flag, p.status))
            return 0.f;
          const int qrow = tile_row0(j) + (tid & 127);
          const size_t stat_base = size_t(tile_slab(j)) * p.rows;
          if (tid < 128) {
            float v = INFINITY;   // +inf => P = 0 for query rows that do not exist
            if (qrow < p.rows) {
              v = p.lse[stat_base + qrow] * 1.4426950408889634f;
              if (v == -INFINITY) v = INFINITY;   // a row with no valid key anywhere has P = 0
            }
            return v;
          }
          return (tid < 256 && qrow < p.rows) ? p.delta[stat_base + qrow] : 0.f;
        };
        // Two buffers are enough: a warp publishes tile jj+1 only after the X_LOADED rendezvous of tile jj,
        // which every warp reaches after it has finished reading the statistics of tile jj-1 (also across items).
        auto put_stat = [&](int jj, float v) {
          if (tid >= 256) return;
          s_stat[(jj & 1) * 256 + tid] = v;
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[BB_STAT_FULL + (jj & 1)]);
        };
        put_stat(jj0, fetch_stat(0));
        float stat_next = ntot > 1 ? fetch_stat(1) : 0.f;   // fetched two tiles ahead, published one ahead
        for (int j = 0; j < ntot; ++j) {
          const int jj = jj0 + j;
          float stat_after = 0.f;
          if (j + 2 < ntot) stat_after = fetch_stat(j + 2);
          if (warp == 0) BWD_TS(0, 0);
          // ---------------- P^T half: needs S^T only ----------------
          if (!mbar_wait(&bars[BB_S_FULL], jj & 1, abort_flag, p.status, BWD_CODE(0, BB_S_FULL), p.bw.pipe_limit)) {
            alive = false;
            break;
          }
          tc_fence_after();
          if (warp == 0) BWD_TS(0, 1);
          uint32_t s[32];
          tmem_ld32(tX + cg * 32, s);
          tc_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[BB_X_LOADED]);
          if (!mbar_wait(&bars[BB_STAT_FULL + (jj & 1)], (jj >> 1) & 1, abort_flag, p.status, BWD_CODE(0, BB_STAT_FULL), p.bw.pipe_limit)) {
            alive = false;
            break;
          }
          const float4* sl = reinterpret_cast<const float4*>(s_stat + (jj & 1) * 256 + cg * 32);
          const float4* sd = reinterpret_cast<const float4*>(s_stat + (jj & 1) * 256 + 128 + cg * 32);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 l2 = sl[i];
            float p0 = ex2f(fmaf(__uint_as_float(s[4 * i]), c, -l2.x));
            float p1 = ex2f(fmaf(__uint_as_float(s[4 * i + 1]), c, -l2.y));
            float p2 = ex2f(fmaf(__uint_as_float(s[4 * i + 2]), c, -l2.z));
            float p3 = ex2f(fmaf(__uint_as_float(s[4 * i + 3]), c, -l2.w));
            if (I.partial && !row_valid) { p0 = 0.f; p1 = 0.f; p2 = 0.f; p3 = 0.f; }
            pk[2 * i] = IS_BF16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
            pk[2 * i + 1] = IS_BF16 ? pack_bf16x2(p2, p3) : pack_f16x2(p2, p3);
          }
          if (warp == 0) BWD_TS(0, 2);
          // P^T overwrites S^T in X: wait until every warp has taken its S^T columns out.
          if (!mbar_wait(&bars[BB_X_LOADED], jj & 1, abort_flag, p.status, BWD_CODE(0, BB_X_LOADED), p.bw.pipe_limit)) {
            alive = false;
            break;
          }
          tmem_st16(tX + cg * 16, pk);
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[BB_P_FULL]);      // dV of this tile may start
          // ---------------- dS^T half: needs dP^T ----------------
          if (!mbar_wait(&bars[BB_DP_FULL], jj & 1, abort_flag, p.status, BWD_CODE(0, BB_DP_FULL), p.bw.pipe_limit)) {
            alive = false;
            break;
          }
          tc_fence_after();
          if (warp == 0) BWD_TS(0, 3);
          uint32_t dsk[16];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t dp[16];
            tmem_ld16(tY + cg * 32 + h * 16, dp);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              // P is taken back from its packed 16-bit form (the value the dV product uses), which keeps only
              // 16 registers alive across the wait for dP^T
              const float4 dl = sd[h * 4 + i];
              const float2 pa = unpack16x2<IS_BF16>(pk[h * 8 + 2 * i]), pb = unpack16x2<IS_BF16>(pk[h * 8 + 2 * i + 1]);
              const float d0 = pa.x * (__uint_as_float(dp[4 * i]) - dl.x);
              const float d1 = pa.y * (__uint_as_float(dp[4 * i + 1]) - dl.y);
              const float d2 = pb.x * (__uint_as_float(dp[4 * i + 2]) - dl.z);
              const float d3 = pb.y * (__uint_as_float(dp[4 * i + 3]) - dl.w);
              dsk[h * 8 + 2 * i] = IS_BF16 ? pack_bf16x2(d0, d1) : pack_f16x2(d0, d1);
              dsk[h * 8 + 2 * i + 1] = IS_BF16 ? pack_bf16x2(d2, d3) : pack_f16x2(d2, d3);
            }
          }
          tc_fence_before();
          // dS^T row -> shared memory: two 64-column halves, each 128-byte swizzled (chunk ^ row%8). The
          // previous tile's dQ^T and dK products (of this item or the one before) must have finished reading it.
          if (jj > 0 && !mbar_wait(&bars[BB_DS_FREE], (jj - 1) & 1, abort_flag, p.status, BWD_CODE(0, BB_DS_FREE), p.bw.pipe_limit)) {
            alive = false;
            break;
          }
          {
            uint8_t* rowp = smem + BWD_OFF_DS + (cg >> 1) * BWD_HALF + r * 128;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
              uint4 v = make_uint4(dsk[4 * ch], dsk[4 * ch + 1], dsk[4 * ch + 2], dsk[4 * ch + 3]);
              *reinterpret_cast<uint4*>(rowp + ((((cg & 1) * 4 + ch) ^ (r & 7)) << 4)) = v;
            }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[BB_PDS_FULL]);
          if (warp == 0) BWD_TS(0, 4);
          if (j + 1 < ntot) put_stat(jj + 1, stat_next);
          stat_next = stat_after;
        }
        // ------------------------------- dK / dV of the item -------------------------------
        // The issuer is already on the next item's S^T / dP^T (X and Y); it overwrites dK / dV only after every
        // compute warp has published the next item's first P^T, i.e. after these loads.
        if (alive) alive = mbar_wait(&bars[BB_ACC_DONE], it & 1, abort_flag, p.status, BWD_CODE(0, BB_ACC_DONE), p.bw.pipe_limit);
        tc_fence_after();
        if (alive) {
          const bool ok_row = (I.kv0 + r) < p.skv;
          const size_t off = (size_t(I.slab) * p.skv + I.kv0 + r) * 128 + cg * 32;
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            uint32_t a[32];
            tmem_ld32(tmem_base + (which ? TM_DV : TM_DK) + lane_sel + cg * 32, a);
            tc_wait_ld();
            const float mul = which ? 1.f : p.scale;
            if (ok_row && p.accumulate == 2) {
              uint4* d16 = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(which ? p.dv_acc : p.dk_acc) + off);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint32_t wd[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float lo = __uint_as_float(a[8 * i + 2 * e]) * mul, hi = __uint_as_float(a[8 * i + 2 * e + 1]) * mul;
                  wd[e] = IS_BF16 ? pack_bf16x2(lo, hi) : pack_f16x2(lo, hi);
                }
                d16[i] = make_uint4(wd[0], wd[1], wd[2], wd[3]);
              }
            } else if (ok_row) {
              float4* d4 = reinterpret_cast<float4*>((which ? p.dv_acc : p.dk_acc) + off);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 v = make_float4(__uint_as_float(a[4 * i]) * mul, __uint_as_float(a[4 * i + 1]) * mul,
                                       __uint_as_float(a[4 * i + 2]) * mul, __uint_as_float(a[4 * i + 3]) * mul);
                if (p.accumulate == 1) {
                  const float4 o = d4[i];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                d4[i] = v;
              }
            }
          }
          tc_fence_before();
        }
        ++it;
        jj0 += ntot;
      }
    } else if (warp < BWD_WARP_TMA) {
      // =========================== dQ drain warps ===========================
      const int quarter = warp & 3;
      const int ch = (warp - BWD_COMPUTE_WARPS) >> 2;      // which 64 query columns
      const int d = quarter * 32 + lane;                    // head-dim index = TMEM lane of dQ^T
      const uint32_t tY = tmem_base + TM_Y + (static_cast<uint32_t>(quarter * 32) << 16) + ch * 64;
      bool alive = true;
      int jj0 = 0;
      for (int w = blockIdx.x; alive && w < p.nitems; w += gridDim.x) {
        const Item I = item_of(w);
        if (!I.live) continue;
        for (int j = 0; j < ntot; ++j) {
          const int jj = jj0 + j;
          if (!mbar_wait(&bars[BB_DQ_FULL], jj & 1, abort_flag, p.status, BWD_CODE(1, BB_DQ_FULL), p.bw.pipe_limit)) {
            alive = false;
            break;
          }
          tc_fence_after();
          if (warp == BWD_COMPUTE_WARPS) BWD_TS(0, 5);
          uint32_t v[2][32];
          tmem_ld32(tY, v[0]);
          tmem_ld32(tY + 32, v[1]);
          tc_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars[BB_DQ_FREE]);     // Y is free for the next tile's dP^T
          if (warp == BWD_COMPUTE_WARPS) BWD_TS(0, 6);
          {
            const int row0 = (j % nq) * 128 + ch * 64;
            const int ncols = min(64, p.rows - row0);
            float* dst = p.dq_acc + (size_t(I.slab + ((p.bw.first_blk + j / nq) % p.nblk) * p.kv_slabs) * p.rows + row0) * 128 + d;
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (i < ncols) atomicAdd(dst + size_t(i) * 128, __uint_as_float(v[i >> 5][i & 31]) * p.scale);
          }
          if (warp == BWD_COMPUTE_WARPS) BWD_TS(0, 7);
        }
        jj0 += ntot;
      }
    } else if (warp == BWD_WARP_TMA) {
      // =========================== TMA producer ===========================
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        int issued = 0, kv_loads = 0;        // Q/dO tiles and K/V tiles requested so far
        bool alive = true;
        int it = 0, jj0 = 0;
        for (int w = blockIdx.x; alive && w < p.nitems; w += gridDim.x) {
          const Item I = item_of(w);
          if (!I.live) continue;
          for (int j = 0; j < ntot; ++j) {
            const int jj = jj0 + j;
            const int s = jj % BWD_NSQ;
            const uint32_t ph = (jj / BWD_NSQ) & 1;
            const int blk = (p.bw.first_blk + j / nq) % p.nblk;
            const int qslab = I.slab + blk * p.kv_slabs, y = (j % nq) * 128;
            if (y == 0) {      // first tile of a block: it may still be on its way from another rank
              if (!wait_block(p.bw, blk, abort_flag, p.status)) { alive = false; break; }
              fence_async_global();
            }
            if (!mbar_wait(&bars[BB_Q_EMPTY + s], ph ^ 1, abort_flag, p.status, BWD_CODE(2, BB_Q_EMPTY), p.bw.pipe_limit)) {
              alive = false;
              break;
            }
            uint8_t* dstq = smem + BWD_OFF_Q + s * 2 * BWD_TILE;
            mbar_arrive_expect_tx(&bars[BB_Q_FULL + s], 2 * BWD_TILE);
            for (int h = 0; h < 2; ++h) {
              tma_load_3d(dstq + h * BWD_HALF, &tmQ, &bars[BB_Q_FULL + s], h * 64, y, qslab);
              tma_load_3d(dstq + BWD_TILE + h * BWD_HALF, &tmDO, &bars[BB_Q_FULL + s], h * 64, y, qslab);
            }
            issued = jj + 1;
            if (j == 0) {
              // The item's K/V go in after its first Q/dO tile (whose stage frees early): the tile buffers are
              // the previous item's until all of its products have completed.
              if (it > 0 && !mbar_wait(&bars[BB_ACC_DONE], (it - 1) & 1, abort_flag, p.status, BWD_CODE(2, BB_ACC_DONE), p.bw.pipe_limit)) {
                alive = false;
                break;
              }
              mbar_arrive_expect_tx(&bars[BB_KV_FULL], 2 * BWD_TILE);
              for (int h = 0; h < 2; ++h) {
                tma_load_3d(smem + BWD_OFF_K + h * BWD_HALF, &tmK, &bars[BB_KV_FULL], h * 64, I.kv0, I.slab);
                tma_load_3d(smem + BWD_OFF_V + h * BWD_HALF, &tmV, &bars[BB_KV_FULL], h * 64, I.kv0, I.slab);
              }
              ++kv_loads;
            }
          }
          ++it;
          jj0 += ntot;
        }
        if (*abort_flag) {      // let the copies in flight land before the CTA's shared memory goes away
          auto drain = [&](uint64_t* bar, uint32_t ph) {
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, ph) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
          };
          if (kv_loads > 0) drain(&bars[BB_KV_FULL], (kv_loads - 1) & 1);
          for (int jj = max(0, issued - BWD_NSQ); jj < issued; ++jj) drain(&bars[BB_Q_FULL + jj % BWD_NSQ], (jj / BWD_NSQ) & 1);
        }
      }
    } else {
      // =========================== MMA issuer ===========================
      if (lane == 0) {
        constexpr uint32_t FMT = IS_BF16 ? UMMA_BF16 : UMMA_F16;
        constexpr uint32_t IDESC_ST = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_K_MAJOR, 128, 128);
        constexpr uint32_t IDESC_ACC = umma_idesc(FMT, UMMA_K_MAJOR, UMMA_MN_MAJOR, 128, 128);
        constexpr uint32_t IDESC_DQ = umma_idesc(FMT, UMMA_MN_MAJOR, UMMA_MN_MAJOR, 128, 128);
        constexpr uint32_t HI = umma_desc_hi(1024);
        const uint32_t sK = smem_u32(smem + BWD_OFF_K), sV = smem_u32(smem + BWD_OFF_V);
        const uint32_t sQ0 = smem_u32(smem + BWD_OFF_Q), sDS = smem_u32(smem + BWD_OFF_DS);

        // D[128 kv, 128 q] = A[128 kv, 128 d] * B[128 q, 128 d]^T, both K-major
        auto issue_st = [&](uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem) {
          const uint32_t a_lo = umma_desc_lo(a_smem, 16), b_lo = umma_desc_lo(b_smem, 16);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = ((kk >> 2) * BWD_HALF + (kk & 3) * 32) >> 4;
            umma_ss_f16(d_tmem, umma_desc_join(a_lo + off, HI), umma_desc_join(b_lo + off, HI), IDESC_ST, kk > 0);
          }
        };
        // D[128 kv, 128 d] += A_tmem[128 kv, 128 q] * B[128 q, 128 d]  (B MN-major: rows are q)
        auto issue_acc = [&](uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem, bool first) {
          const uint32_t b_lo = umma_desc_lo(b_smem, BWD_HALF);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts_f16(d_tmem, a_tmem + kk * 8, umma_desc_join(b_lo + ((kk * 2048) >> 4), HI), IDESC_ACC,
                        (!first) || kk > 0);
        };
        // dK[128 kv, 128 d] += dS^T[128 kv, 128 q] * Q[128 q, 128 d]: A is the dS^T tile in shared memory read
        // K-major (rows kv, 64-column halves), B is Q read MN-major (rows are q)
        auto issue_dk = [&](uint32_t b_smem, bool first) {
          const uint32_t a_lo = umma_desc_lo(sDS, 16), b_lo = umma_desc_lo(b_smem, BWD_HALF);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss_f16(tmem_base + TM_DK, umma_desc_join(a_lo + (((kk >> 2) * BWD_HALF + (kk & 3) * 32) >> 4), HI),
                        umma_desc_join(b_lo + ((kk * 2048) >> 4), HI), IDESC_ACC, (!first) || kk > 0);
        };
        // D[128 d, 128 q] = K^T[128 d, 128 kv] * dS^T[128 kv, 128 q]  (both MN-major: rows are kv)
        const uint32_t kT_lo = umma_desc_lo(sK, BWD_HALF), ds_lo = umma_desc_lo(sDS, BWD_HALF);
        auto issue_dq = [&]() {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss_f16(tmem_base + TM_Y, umma_desc_join(kT_lo + ((kk * 2048) >> 4), HI),
                        umma_desc_join(ds_lo + ((kk * 2048) >> 4), HI), IDESC_DQ, kk > 0);
        };

        bool ok = true;
        int it = 0, jj0 = 0;
        for (int w = blockIdx.x; ok && w < p.nitems; w += gridDim.x) {
          const Item I = item_of(w);
          if (!I.live) continue;
          // The item's first S^T and dP^T. X is free (the tensor pipe runs in order behind the last dV); Y still
          // holds the previous item's last dQ^T until the drain warps have taken it.
          ok = mbar_wait(&bars[BB_KV_FULL], it & 1, abort_flag, p.status, BWD_CODE(3, BB_KV_FULL), p.bw.pipe_limit);
          ok = ok && mbar_wait(&bars[BB_Q_FULL + jj0 % BWD_NSQ], (jj0 / BWD_NSQ) & 1, abort_flag, p.status, BWD_CODE(3, BB_Q_FULL), p.bw.pipe_limit);
          if (ok && jj0 > 0)
            ok = mbar_wait(&bars[BB_DQ_FREE], (jj0 - 1) & 1, abort_flag, p.status, BWD_CODE(3, BB_DQ_FREE), p.bw.pipe_limit);
          if (!ok) break;
          tc_fence_after();
          {
            const uint32_t sQf = sQ0 + (jj0 % BWD_NSQ) * 2 * BWD_TILE;
            issue_st(tmem_base + TM_X, sK, sQf);
            tc_commit(&bars[BB_S_FULL]);
            issue_st(tmem_base + TM_Y, sV, sQf + BWD_TILE);
            tc_commit(&bars[BB_DP_FULL]);
          }
          for (int j = 0; ok && j < ntot; ++j) {
            const int jj = jj0 + j;
            const int s = jj % BWD_NSQ;
            const uint32_t sQ = sQ0 + s * 2 * BWD_TILE, sDO = sQ + BWD_TILE;
            BWD_TS(1, 0);
            // dV needs P^T only, which is published before the dS^T half of the elementwise work; once dV has
            // read X, S^T of the next tile can go there, i.e. while the warps are still producing dS^T
            ok = mbar_wait(&bars[BB_P_FULL], jj & 1, abort_flag, p.status, BWD_CODE(3, BB_P_FULL), p.bw.pipe_limit);
            if (!ok) break;
            tc_fence_after();
            issue_acc(tmem_base + TM_DV, tmem_base + TM_X, sDO, j == 0);
            BWD_TS(1, 1);
            const int s1 = (jj + 1) % BWD_NSQ;
            const uint32_t sQ1 = sQ0 + s1 * 2 * BWD_TILE;
            if (j + 1 < ntot) {
              ok = mbar_wait(&bars[BB_Q_FULL + s1], ((jj + 1) / BWD_NSQ) & 1, abort_flag, p.status, BWD_CODE(3, BB_Q_FULL), p.bw.pipe_limit);
              if (!ok) break;
              tc_fence_after();
              issue_st(tmem_base + TM_X, sK, sQ1);
              tc_commit(&bars[BB_S_FULL]);
              BWD_TS(1, 2);
            }
            ok = mbar_wait(&bars[BB_PDS_FULL], jj & 1, abort_flag, p.status, BWD_CODE(3, BB_PDS_FULL), p.bw.pipe_limit);
            if (!ok) break;
            tc_fence_after();
            BWD_TS(1, 3);
            issue_dq();                                   // Y: every warp took dP^T out before publishing dS^T
            tc_commit(&bars[BB_DQ_FULL]);
            issue_dk(sQ, j == 0);
            tc_commit(&bars[BB_Q_EMPTY + s]);
            tc_commit(&bars[BB_DS_FREE]);
            BWD_TS(1, 4);
            if (j + 1 < ntot) {
              ok = mbar_wait(&bars[BB_DQ_FREE], jj & 1, abort_flag, p.status, BWD_CODE(3, BB_DQ_FREE), p.bw.pipe_limit);
              if (!ok) break;
              tc_fence_after();
              BWD_TS(1, 5);
              issue_st(tmem_base + TM_Y, sV, sQ1 + BWD_TILE);
              tc_commit(&bars[BB_DP_FULL]);
              BWD_TS(1, 6);
            }
          }
          if (ok) tc_commit(&bars[BB_ACC_DONE]);
          ++it;
          jj0 += ntot;
        }
        if (!ok) {
          tc_commit(&bars[BB_DRAIN]);
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars[BB_DRAIN], 0) && clock64() - t0 < LVX_SPIN_LIMIT_CYCLES) {}
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == BWD_WARP_MMA) tmem_dealloc(tmem_base, 512);
}

// SMs of the current device (one process drives one GPU; looked up once).
static int bwd_num_sms() {
  static int n_sms = 0;
  if (!n_sms) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      n_sms = n;
    else
      n_sms = 148;
  }
  return n_sms;
}

int launch_bwd_block(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                     const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                     float* dk_acc, float* dv_acc, int accumulate_dkdv, int* status, cudaStream_t st,
                     const lvx_block_wait* bw) {
  if (!(sm_scale > 0.f)) return fail(LVX_ERR_SHAPE, "lvx_bwd_block: sm_scale must be positive");
  if (accumulate_dkdv < 0 || accumulate_dkdv > 2)
    return fail(LVX_ERR_SHAPE, "lvx_bwd_block: accumulate_dkdv must be 0, 1 or 2 (got %d)", accumulate_dkdv);
  if (s.dtype == LVX_FP32)
    return launch_bwd_block_fp32(s, q, d_o, lse, delta, k, v, kv_valid_len, sm_scale, dq_acc, dk_acc, dv_acc,
                                 accumulate_dkdv, st);
  const int g = s.Hq / s.Hkv;
  const int rows = g * s.Sq;
  const int es = elt_size(s.dtype);
  const uint64_t row_bytes = uint64_t(128) * es;
  const uint64_t slabs = uint64_t(s.B) * s.Hkv;
  const int qb = q_blocks_of(s);
  CUtensorMap tmQ, tmDO, tmK, tmV;
  int rc;
  if ((rc = make_tmap_3d(&tmQ, s.dtype, q, 128, rows, slabs * qb, row_bytes, row_bytes * rows, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmDO, s.dtype, d_o, 128, rows, slabs * qb, row_bytes, row_bytes * rows, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmK, s.dtype, k, 128, s.Skv, slabs, row_bytes, row_bytes * s.Skv, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV, s.dtype, v, 128, s.Skv, slabs, row_bytes, row_bytes * s.Skv, 64, 128))) return rc;

  BwdParams p;
  p.rows = rows;
  p.skv = s.Skv;
  p.hkv = s.Hkv;
  p.nblk = qb;
  p.kv_slabs = int(slabs);
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
  p.bw = make_block_wait(bw, qb);

  p.kv_tiles = (s.Skv + 127) / 128;
  p.nitems = p.kv_tiles * p.kv_slabs;
  dim3 grid(std::min(p.nitems, bwd_num_sms()), 1, 1);      // persistent: one CTA per SM
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
    if (e == cudaSuccess) kern<<<grid, BWD_THREADS, BWD_SMEM, st>>>(tmQ, tmDO, tmK, tmV, p);
  };
  if (s.dtype == LVX_BF16) go(bwd_kernel<true>);
  else go(bwd_kernel<false>);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(bwd)");
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "bwd_kernel launch");
#ifdef LVX_DEV_STAMPS
  {
    static long long ts[2 * 8 * 16];
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(ts, g_bwd_ts, sizeof(ts));
    const char* names[2] = {"compute", "mma"};
    for (int r = 0; r < 2; ++r)
      for (int j = 0; j < 8; ++j) {
        fprintf(stderr, "%s tile %d:", names[r], j + 4);
        for (int k2 = 0; k2 < 8; ++k2)
          fprintf(stderr, " %lld", ts[(r * 8 + j) * 16 + k2] ? ts[(r * 8 + j) * 16 + k2] - ts[0] : -1);
        fprintf(stderr, "\n");
      }
  }
#endif
  return LVX_OK;
}

}  // namespace lvx
