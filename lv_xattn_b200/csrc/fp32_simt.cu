// The general path: forward and backward flash-attention blocks on the FP32 FMA pipe, exact fp32 arithmetic.
// It serves (1) fp32 inputs and (2) any input dtype when a dense additive bias is given (the reference's
// bias_func protocol, lv_xattn/attn.py:386-389: S = scale * q.k + bias, bias [B, 1 or H, Sq, Skv] fp32).
//
// Why not tf32 on the tensor cores: for 32-bit operands tcgen05 wants K-major tiles in the 16-byte-unit
// 128B swizzle and MN-major tiles in the 32-byte-unit swizzle. In the backward block every streamed tile
// (Q, dO, and the resident K) is consumed both ways, so each would have to sit in shared memory twice, which
// does not fit; and tf32 rounding (2^-11 per operand) leaves little margin under the 1e-4 bar the fp32 case
// is held to. fp32 is the correctness configuration, not the throughput one, so it gets straightforward
// tiled kernels with the same interface, workspace layout and masking rules as the 16-bit tensor-core path.
//
// Both kernels use 64 x 64 score tiles and 256 threads laid out 16 x 16. Shared memory is the resource that
// bounds a register-tiled FP32 product (one 128-byte wavefront per clock and SM against four FMA instructions per
// clock), so every operand is fetched with 16-byte loads that are free of bank conflicts:
//   scores (64 x 64, contraction over d):  thread (ty, tx) owns rows 4*ty+i and columns tx+16*j (i, j = 0..3) and
//     reads four consecutive d of a row at a time; rows are 132 floats apart, and 132/4 = 33 is odd, so the pieces
//     that eight neighbouring tx read from eight neighbouring rows fall into eight different bank groups;
//   64 x 128 products (contraction over a tile edge):  thread (ty, tx) owns rows 4*ty+i and the eight columns
//     4*tx+64*h+e (h = 0..1, e = 0..3): the 16 tx of a row read 256 contiguous bytes, the left operand is a broadcast.
// P and dS tiles ([q][kv], row stride 68) are written with the score layout (conflict-free) and read back 16 bytes
// at a time along either axis. Measured on the part: a 16-byte load costs one wavefront per quarter-warp (two when
// a half-warp reads one address), i.e. 24 wavefronts per 64 FMA instructions in the score products and 40 per 128 in
// the others -- the shared-memory pipe, not the FMA pipe, still sets the pace (FMA pipe 40-43 % busy); only a larger
// register tile per thread would change that ratio.
#include "lvx_internal.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace lvx {

constexpr int SM_T = 64;            // tile edge
constexpr int SM_LD = 132;          // row stride of a [64][128] tile (floats): 16-byte aligned rows, 33 bank groups
constexpr int SM_LDP = 68;          // row stride of a [64][64] tile
constexpr int SM_TILE = SM_T * SM_LD;
constexpr int SM_PTILE = SM_T * SM_LDP;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float comp(const float4& v, int e) { return e == 0 ? v.x : e == 1 ? v.y : e == 2 ? v.z : v.w; }
// acc[0..3] += s * v
__device__ __forceinline__ void axpy4(float* acc, float s, const float4& v) {
  acc[0] = fmaf(s, v.x, acc[0]);
  acc[1] = fmaf(s, v.y, acc[1]);
  acc[2] = fmaf(s, v.z, acc[2]);
  acc[3] = fmaf(s, v.w, acc[3]);
}
// acc += a . b
__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
  return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, fmaf(a.x, b.x, acc))));
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ void from_f32(float* p, float x) { *p = x; }
__device__ __forceinline__ void from_f32(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
__device__ __forceinline__ void from_f32(__half* p, float x) { *p = __float2half_rn(x); }

// Loads rows [row0, row0+64) of a dense [nrows, 128] matrix into a padded fp32 tile; rows past nrows are zero.
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int row0, int nrows, int tid) {
  for (int idx = tid; idx < SM_T * 128; idx += 256) {
    const int r = idx >> 7, c = idx & 127;
    const int gr = row0 + r;
    dst[r * SM_LD + c] = gr < nrows ? to_f32(src[size_t(gr) * 128 + c]) : 0.f;
  }
}

// Dense additive bias on the scores: value for (query block, batch, query head, query row, key) at
// base[blk*s_blk + b*s_b + h*s_h + i*s_q + j*s_kv] (strides in floats; 0 broadcasts). nullptr = no bias.
struct BiasView {
  const float* base;
  long long s_blk, s_b, s_h, s_q, s_kv;
  int sq, g;          // query rows per head, query heads per KV head (to unpack a packed row)
};
// pointer to the bias row of packed row `r` of query slab `slab` (kv slab `kvs`), or nullptr
__device__ __forceinline__ const float* bias_row(const BiasView& b, int slab, int kvs, int kv_slabs, int hkv, int r) {
  if (b.base == nullptr) return nullptr;
  const int blk = slab / kv_slabs, batch = kvs / hkv, hk = kvs % hkv;
  const int h = hk * b.g + r / b.sq, i = r % b.sq;
  return b.base + blk * b.s_blk + batch * b.s_b + h * b.s_h + i * b.s_q;
}

struct Fp32FwdParams {
  const void *q, *k, *v;
  BiasView bias;
  const int32_t* kv_valid_len;
  int rows, skv, hkv, kv_slabs, nsplit, tiles_per_split;   // tiles_per_split counts 128-row tiles, as in the 16-bit plan
  float scale_log2;
  float *o_part, *ml_part;
  const int* status;   // device status word: non-zero => return at once
};

template <typename T>
__global__ void __launch_bounds__(256, 2)
fp32_fwd_kernel(const Fp32FwdParams p) {
  if (p.status && *reinterpret_cast<const volatile int*>(p.status) != 0) return;
  extern __shared__ __align__(16) float sm[];
  float* sQ = sm;
  float* sK = sQ + SM_TILE;
  float* sV = sK + SM_TILE;
  float* sP = sK;                              // P takes K's place once the scores of a tile are in registers
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int mb = blockIdx.x, slab = blockIdx.y, split = blockIdx.z;
  const int kvs = slab % p.kv_slabs;          // several query blocks may share one K/V batch entry
  const int batch = kvs / p.hkv;
  int valid = p.skv;
  if (p.kv_valid_len) valid = min(valid, max(0, p.kv_valid_len[batch]));
  const int kv_begin = min(valid, split * p.tiles_per_split * 128);
  const int kv_end = min(valid, (split + 1) * p.tiles_per_split * 128);
  const T* qs = static_cast<const T*>(p.q) + size_t(slab) * p.rows * 128;
  const T* ks = static_cast<const T*>(p.k) + size_t(kvs) * p.skv * 128;
  const T* vs = static_cast<const T*>(p.v) + size_t(kvs) * p.skv * 128;
  const float* brow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = mb * SM_T + ty * 4 + i;
    brow[i] = row < p.rows ? bias_row(p.bias, slab, kvs, p.kv_slabs, p.hkv, row) : nullptr;
  }

  load_tile(sQ, qs, mb * SM_T, p.rows, tid);
  float m[4], l[4], o[4][8];                  // o[i][4*h+e]: row 4*ty+i, column 4*tx+64*h+e
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) o[i][c] = 0.f;
  }
  for (int kv0 = kv_begin; kv0 < kv_end; kv0 += SM_T) {
    __syncthreads();                           // the previous tile's P and V have been consumed
    load_tile(sK, ks, kv0, p.skv, tid);
    load_tile(sV, vs, kv0, p.skv, tid);
    __syncthreads();
    float s[4][4];                             // s[i][j]: row 4*ty+i, key tx+16*j
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll 2
    for (int d = 0; d < 128; d += 4) {
      float4 a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = ld4(sQ + (ty * 4 + i) * SM_LD + d);
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ld4(sK + (tx + 16 * j) * SM_LD + d);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = dot4(a[i], b[j], s[i][j]);
    }
    __syncthreads();                           // every thread is done with K before P overwrites it
    // online softmax in base 2; a row is spread over the 16 threads that share ty
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = kv0 + tx + 16 * j;
        float sc = -INFINITY;
        if (col < kv_end) {
          sc = s[i][j] * p.scale_log2;
          if (brow[i]) sc = fmaf(brow[i][col * p.bias.s_kv], 1.4426950408889634f, sc);   // scale*q.k + bias, base 2
        }
        s[i][j] = sc;
        mx = fmaxf(mx, sc);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m[i], mx);
      const float moff = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m[i] - moff);       // m = -inf -> 0
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float pv = exp2f(s[i][j] - moff);
        sum += pv;
        sP[(ty * 4 + i) * SM_LDP + tx + 16 * j] = pv;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      l[i] = l[i] * alpha + sum;
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < 8; ++c) o[i][c] *= alpha;
    }
    __syncthreads();
#pragma unroll 2
    for (int j = 0; j < SM_T; j += 4) {
      float4 pr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pr[i] = ld4(sP + (ty * 4 + i) * SM_LDP + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float4 v0 = ld4(sV + (j + jj) * SM_LD + 4 * tx);
        const float4 v1 = ld4(sV + (j + jj) * SM_LD + 64 + 4 * tx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          axpy4(&o[i][0], comp(pr[i], jj), v0);
          axpy4(&o[i][4], comp(pr[i], jj), v1);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = mb * SM_T + ty * 4 + i;
    if (row >= p.rows) continue;
    const size_t prow = (size_t(slab) * p.nsplit + split) * p.rows + row;
#pragma unroll
    for (int h = 0; h < 2; ++h)
      *reinterpret_cast<float4*>(p.o_part + prow * 128 + 64 * h + 4 * tx) =
          make_float4(o[i][4 * h], o[i][4 * h + 1], o[i][4 * h + 2], o[i][4 * h + 3]);
    if (tx == 0) {
      p.ml_part[prow * 2] = m[i];
      p.ml_part[prow * 2 + 1] = l[i];
    }
  }
}

struct Fp32BwdParams {
  const void *q, *d_o, *k, *v;
  const float *lse, *delta;
  BiasView bias;
  const int32_t* kv_valid_len;
  int rows, skv, hkv, nblk, kv_slabs;
  float scale, scale_log2;
  float *dq_acc;
  void *dk_acc, *dv_acc;   // fp32 for accumulate 0/1; the input dtype for accumulate 2
  int accumulate;
  const int* status;   // device status word: non-zero => return at once
};

template <typename T>
__global__ void __launch_bounds__(256, 1)
fp32_bwd_kernel(const Fp32BwdParams p) {
  if (p.status && *reinterpret_cast<const volatile int*>(p.status) != 0) return;
  extern __shared__ __align__(16) float sm[];
  float* sK = sm;
  float* sV = sK + SM_TILE;
  float* sQ = sV + SM_TILE;
  float* sDO = sQ + SM_TILE;
  float* sP = sDO + SM_TILE;     // [q][kv]
  float* sDS = sP + SM_PTILE;    // [q][kv]
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int kv0 = blockIdx.x * SM_T, slab = blockIdx.y;
  const int batch = slab / p.hkv;
  int valid = p.skv;
  if (p.kv_valid_len) valid = min(valid, max(0, p.kv_valid_len[batch]));

  load_tile(sK, static_cast<const T*>(p.k) + size_t(slab) * p.skv * 128, kv0, p.skv, tid);
  load_tile(sV, static_cast<const T*>(p.v) + size_t(slab) * p.skv * 128, kv0, p.skv, tid);
  float dk[4][8], dv[4][8];      // [i][4*h+e]: key row 4*ty+i, column 4*tx+64*h+e
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 8; ++c) dk[i][c] = dv[i][c] = 0.f;

  const bool live = kv0 < valid;
  const int tiles_per_block = (p.rows + SM_T - 1) / SM_T;
  for (int it = 0; live && it < tiles_per_block * p.nblk; ++it) {
    const int qslab = slab + (it / tiles_per_block) * p.kv_slabs;
    const int q0 = (it % tiles_per_block) * SM_T;
    const T* qs = static_cast<const T*>(p.q) + size_t(qslab) * p.rows * 128;
    const T* dos = static_cast<const T*>(p.d_o) + size_t(qslab) * p.rows * 128;
    const float* lses = p.lse + size_t(qslab) * p.rows;
    const float* deltas = p.delta + size_t(qslab) * p.rows;
    float* dqs = p.dq_acc + size_t(qslab) * p.rows * 128;
    __syncthreads();
    load_tile(sQ, qs, q0, p.rows, tid);
    load_tile(sDO, dos, q0, p.rows, tid);
    __syncthreads();
    {
      // S[q][kv] = Q K^T and dP[q][kv] = dO V^T    (this thread: q rows 4*ty+i, keys tx+16*j)
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
#pragma unroll 2
      for (int d = 0; d < 128; d += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = ld4(sQ + (ty * 4 + i) * SM_LD + d);
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = ld4(sK + (tx + 16 * j) * SM_LD + d);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) s[i][j] = dot4(a[i], b[j], s[i][j]);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = ld4(sDO + (ty * 4 + i) * SM_LD + d);
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = ld4(sV + (tx + 16 * j) * SM_LD + d);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) dp[i][j] = dot4(a[i], b[j], dp[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int qrow = q0 + ty * 4 + i;
        float l2 = INFINITY, dl = 0.f;      // +inf: rows that do not exist, or that have no valid key anywhere
        if (qrow < p.rows) {
          l2 = lses[qrow] * 1.4426950408889634f;
          if (l2 == -INFINITY) l2 = INFINITY;
          dl = deltas[qrow];
        }
        const float* br = qrow < p.rows ? bias_row(p.bias, qslab, slab, p.kv_slabs, p.hkv, qrow) : nullptr;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = kv0 + tx + 16 * j;
          const bool ok = col < valid;
          float sc = s[i][j] * p.scale_log2;
          if (ok && br) sc = fmaf(br[col * p.bias.s_kv], 1.4426950408889634f, sc);
          const float pv = ok ? exp2f(sc - l2) : 0.f;
          sP[(ty * 4 + i) * SM_LDP + tx + 16 * j] = pv;
          sDS[(ty * 4 + i) * SM_LDP + tx + 16 * j] = pv * (dp[i][j] - dl);
        }
      }
    }
    __syncthreads();
    // dV[kv][d] += sum_q P[q][kv] dO[q][d];  dK[kv][d] += sum_q dS[q][kv] Q[q][d]
    // (this thread: key rows 4*ty+i -- one 16-byte piece of a P / dS row -- and columns 4*tx+64*h+e)
#pragma unroll 4
    for (int qi = 0; qi < SM_T; ++qi) {
      const float4 pr = ld4(sP + qi * SM_LDP + 4 * ty);
      const float4 dsr = ld4(sDS + qi * SM_LDP + 4 * ty);
      const float4 g0 = ld4(sDO + qi * SM_LD + 4 * tx), g1 = ld4(sDO + qi * SM_LD + 64 + 4 * tx);
      const float4 a0 = ld4(sQ + qi * SM_LD + 4 * tx), a1 = ld4(sQ + qi * SM_LD + 64 + 4 * tx);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        axpy4(&dv[i][0], comp(pr, i), g0);
        axpy4(&dv[i][4], comp(pr, i), g1);
        axpy4(&dk[i][0], comp(dsr, i), a0);
        axpy4(&dk[i][4], comp(dsr, i), a1);
      }
    }
    // dQ[q][d] = sum_kv dS[q][kv] K[kv][d]    (this thread: q rows 4*ty+i, columns 4*tx+64*h+e)
    float dq[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 8; ++c) dq[i][c] = 0.f;
#pragma unroll 2
    for (int j = 0; j < SM_T; j += 4) {
      float4 dsr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dsr[i] = ld4(sDS + (ty * 4 + i) * SM_LDP + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float4 b0 = ld4(sK + (j + jj) * SM_LD + 4 * tx), b1 = ld4(sK + (j + jj) * SM_LD + 64 + 4 * tx);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          axpy4(&dq[i][0], comp(dsr[i], jj), b0);
          axpy4(&dq[i][4], comp(dsr[i], jj), b1);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qrow = q0 + ty * 4 + i;
      if (qrow < p.rows)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          atomicAdd(dqs + size_t(qrow) * 128 + 64 * (c >> 2) + 4 * tx + (c & 3), dq[i][c] * p.scale);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = kv0 + ty * 4 + i;
    if (row >= p.skv) continue;
    if (!live && p.accumulate == 1) continue;
    const size_t off = (size_t(slab) * p.skv + row) * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int d = 64 * (c >> 2) + 4 * tx + (c & 3);
      const float a = dk[i][c] * p.scale, b = dv[i][c];
      if (p.accumulate == 2) {                          // finished gradients in the input dtype
        from_f32(static_cast<T*>(p.dk_acc) + off + d, a);
        from_f32(static_cast<T*>(p.dv_acc) + off + d, b);
      } else {
        float* dkp = static_cast<float*>(p.dk_acc) + off;
        float* dvp = static_cast<float*>(p.dv_acc) + off;
        dkp[d] = p.accumulate == 1 ? dkp[d] + a : a;
        dvp[d] = p.accumulate == 1 ? dvp[d] + b : b;
      }
    }
  }
}

static BiasView make_bias(const lvx_shape& s, const lvx_bias* b) {
  BiasView v;
  v.base = b ? b->bias : nullptr;
  v.s_blk = b ? b->stride_block : 0;
  v.s_b = b ? b->stride_b : 0;
  v.s_h = b ? b->stride_h : 0;
  v.s_q = b ? b->stride_q : 0;
  v.s_kv = b ? b->stride_kv : 0;
  v.sq = s.Sq;
  v.g = s.Hq / s.Hkv;
  return v;
}

int launch_fwd_block_simt(const lvx_shape& s, const FwdPlan& pl, const void* q, const void* k, const void* v,
                          const int32_t* kv_valid_len, const lvx_bias* bias, float sm_scale, float* o_part,
                          float* ml_part, cudaStream_t st) {
  Fp32FwdParams p;
  p.q = q;
  p.k = k;
  p.v = v;
  p.bias = make_bias(s, bias);
  p.kv_valid_len = kv_valid_len;
  p.rows = pl.rows;
  p.skv = s.Skv;
  p.hkv = s.Hkv;
  p.kv_slabs = s.B * s.Hkv;
  p.nsplit = pl.nsplit;
  p.tiles_per_split = pl.tiles_per_split;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.o_part = o_part;
  p.ml_part = ml_part;
  p.status = device_status_ptr();
  const int smem = 3 * SM_TILE * sizeof(float);   // P shares K's tile
  dim3 grid((pl.rows + SM_T - 1) / SM_T, q_blocks_of(s) * s.B * s.Hkv, pl.nsplit);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) kern<<<grid, 256, smem, st>>>(p);
  };
  if (s.dtype == LVX_FP32) go(fp32_fwd_kernel<float>);
  else if (s.dtype == LVX_BF16) go(fp32_fwd_kernel<__nv_bfloat16>);
  else go(fp32_fwd_kernel<__half>);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(simt fwd)");
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "simt fwd kernel launch");
  return LVX_OK;
}

int launch_bwd_block_simt(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                          const void* k, const void* v, const int32_t* kv_valid_len, const lvx_bias* bias,
                          float sm_scale, float* dq_acc, void* dk_acc, void* dv_acc, int accumulate_dkdv,
                          cudaStream_t st) {
  Fp32BwdParams p;
  p.q = q;
  p.d_o = d_o;
  p.lse = lse;
  p.delta = delta;
  p.k = k;
  p.v = v;
  p.bias = make_bias(s, bias);
  p.kv_valid_len = kv_valid_len;
  p.rows = (s.Hq / s.Hkv) * s.Sq;
  p.skv = s.Skv;
  p.hkv = s.Hkv;
  p.nblk = q_blocks_of(s);
  p.kv_slabs = s.B * s.Hkv;
  p.scale = sm_scale;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.dq_acc = dq_acc;
  p.dk_acc = dk_acc;
  p.dv_acc = dv_acc;
  p.accumulate = accumulate_dkdv;
  p.status = device_status_ptr();
  const int smem = (4 * SM_TILE + 2 * SM_PTILE) * sizeof(float);
  dim3 grid((s.Skv + SM_T - 1) / SM_T, s.B * s.Hkv, 1);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) kern<<<grid, 256, smem, st>>>(p);
  };
  if (s.dtype == LVX_FP32) go(fp32_bwd_kernel<float>);
  else if (s.dtype == LVX_BF16) go(fp32_bwd_kernel<__nv_bfloat16>);
  else go(fp32_bwd_kernel<__half>);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(simt bwd)");
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "simt bwd kernel launch");
  return LVX_OK;
}

int launch_fwd_block_fp32(const lvx_shape& s, const FwdPlan& pl, const void* q, const void* k, const void* v,
                          const int32_t* kv_valid_len, float sm_scale, float* o_part, float* ml_part, cudaStream_t st) {
  return launch_fwd_block_simt(s, pl, q, k, v, kv_valid_len, nullptr, sm_scale, o_part, ml_part, st);
}

int launch_bwd_block_fp32(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                          const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                          float* dk_acc, float* dv_acc, int accumulate_dkdv, cudaStream_t st) {
  return launch_bwd_block_simt(s, q, d_o, lse, delta, k, v, kv_valid_len, nullptr, sm_scale, dq_acc, dk_acc, dv_acc,
                               accumulate_dkdv, st);
}

}  // namespace lvx
