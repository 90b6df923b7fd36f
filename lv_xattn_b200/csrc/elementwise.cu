// HBM-bound helper kernels around the two tensor-core blocks:
//   fwd_combine_kernel  split-KV partials (+) travelling (O, lse)  ->  (O, lse)
//   bwd_prep_kernel     delta = rowsum(O * dO)
//   add_cast_kernel     out = cast(a + b)
// One warp handles one 128-wide row with float4 / 8-byte accesses, so every access is a full 512-byte
// (fp32) or 256-byte (16-bit) coalesced row.
#include "lvx_internal.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace lvx {

constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLog2e = 1.4426950408889634f;

// While the device status word is set (a bounded wait ran out somewhere) every kernel returns at once, so that
// nothing is computed from buffers an aborted kernel left unwritten.
__device__ __forceinline__ bool poisoned(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0;
}

template <int OUT>  // 0 bf16, 1 fp16, 2 fp32
__device__ __forceinline__ void store4(void* base, size_t idx4, float4 v) {
  if (OUT == 2) {
    reinterpret_cast<float4*>(base)[idx4] = v;
  } else if (OUT == 0) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(base)[idx4] = u;
  } else {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(base)[idx4] = u;
  }
}

template <int IN>
__device__ __forceinline__ float4 load4(const void* base, size_t idx4) {
  if (IN == 2) return reinterpret_cast<const float4*>(base)[idx4];
  uint2 u = reinterpret_cast<const uint2*>(base)[idx4];
  if (IN == 0) {
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&u.x));
  float2 b = __half22float2(*reinterpret_cast<__half2*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// Partials live in the packed-row order of the forward block: slab (b*Hkv + hk), split, row r = hg*Sq + i
// where the query head is h = hk*g + hg. A [B,Hq,Sq,D] tensor has exactly the same row order
// (row index (b*Hq + h)*Sq + i = slab*rows + r), so "global row" below indexes both.
template <int OUT>
__global__ void __launch_bounds__(256)
fwd_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part, const float* __restrict__ o_in,
                   const float* __restrict__ lse_in, void* __restrict__ o_out, float* __restrict__ lse_out,
                   int rows_per_slab, int nsplit, long total_rows, const int* status) {
  if (poisoned(status)) return;
  const int lane = threadIdx.x & 31;
  const long grow = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (grow >= total_rows) return;
  const long slab = grow / rows_per_slab;
  const int r = int(grow - slab * rows_per_slab);

  // pass 1: the largest running max among the splits (base-2 domain, already scaled)
  float mmax = -INFINITY;
  for (int s = 0; s < nsplit; ++s) {
    const size_t prow = (size_t(slab) * nsplit + s) * rows_per_slab + r;
    mmax = fmaxf(mmax, ml_part[prow * 2]);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  if (mmax != -INFINITY) {
    // four splits per round: the statistics and the partial rows of all four are requested before any is used
    for (int s0 = 0; s0 < nsplit; s0 += 4) {
      float2 ml[4];
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int s = min(s0 + u, nsplit - 1);
        const size_t prow = (size_t(slab) * nsplit + s) * rows_per_slab + r;
        ml[u] = *reinterpret_cast<const float2*>(ml_part + prow * 2);
        v[u] = reinterpret_cast<const float4*>(o_part + prow * 128)[lane];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u >= nsplit || ml[u].x == -INFINITY) continue;
        const float w = exp2f(ml[u].x - mmax);
        lsum += ml[u].y * w;
        acc.x += v[u].x * w;
        acc.y += v[u].y * w;
        acc.z += v[u].z * w;
        acc.w += v[u].w * w;
      }
    }
  }
  // (O_loc, lse_loc) of this shard
  float lse_loc = -INFINITY;
  if (lsum > 0.f) {
    const float inv = 1.f / lsum;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    lse_loc = (mmax + log2f(lsum)) * kLn2;
  } else {
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // merge with the travelling accumulator
  float lse_new = lse_loc;
  if (o_in != nullptr) {
    const float lse_old = lse_in[grow];
    const float mx = fmaxf(lse_old, lse_loc);
    if (mx == -INFINITY) {
      lse_new = -INFINITY;
      acc = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      const float wo = expf(lse_old - mx), wl = expf(lse_loc - mx);
      const float tot = wo + wl;
      lse_new = mx + logf(tot);
      const float co = wo / tot, cl = wl / tot;
      const float4 vo = reinterpret_cast<const float4*>(o_in)[size_t(grow) * 32 + lane];
      acc.x = vo.x * co + acc.x * cl;
      acc.y = vo.y * co + acc.y * cl;
      acc.z = vo.z * co + acc.z * cl;
      acc.w = vo.w * co + acc.w * cl;
    }
  }
  store4<OUT>(o_out, size_t(grow) * 32 + lane, acc);
  if (lane == 0) lse_out[grow] = lse_new;
}

int launch_fwd_combine(const lvx_shape& s, const FwdPlan& p, const float* o_part, const float* ml_part,
                       const float* o_in, const float* lse_in, void* o_out, float* lse_out, int out_is_final,
                       cudaStream_t st) {
  const long total_rows = long(q_blocks_of(s)) * s.B * s.Hq * s.Sq;
  const int threads = 256;
  const int* sp = device_status_ptr();
  const long blocks = (total_rows * 32 + threads - 1) / threads;
  const int out = out_is_final ? s.dtype : LVX_FP32;
  if (out == LVX_BF16)
    fwd_combine_kernel<0><<<blocks, threads, 0, st>>>(o_part, ml_part, o_in, lse_in, o_out, lse_out, p.rows, p.nsplit, total_rows, sp);
  else if (out == LVX_FP16)
    fwd_combine_kernel<1><<<blocks, threads, 0, st>>>(o_part, ml_part, o_in, lse_in, o_out, lse_out, p.rows, p.nsplit, total_rows, sp);
  else
    fwd_combine_kernel<2><<<blocks, threads, 0, st>>>(o_part, ml_part, o_in, lse_in, o_out, lse_out, p.rows, p.nsplit, total_rows, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "fwd_combine launch");
  return LVX_OK;
}

// ---------------------------------------------------------------------------------------------
// Merge of `count` normalised partial results (O fp32, lse) of the same rows; one warp per row.
template <int OUT>
__global__ void __launch_bounds__(256)
fwd_merge_parts_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts, int count,
                       size_t stride_o, size_t stride_lse, void* __restrict__ o_out, float* __restrict__ lse_out,
                       long total_rows, const int* status) {
  if (poisoned(status)) return;
  const int lane = threadIdx.x & 31;
  const long row = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= total_rows) return;
  float mx = -INFINITY;
  for (int c = 0; c < count; ++c) mx = fmaxf(mx, lse_parts[c * stride_lse + row]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float tot = 0.f;
  if (mx != -INFINITY) {
    for (int c = 0; c < count; ++c) {
      const float l = lse_parts[c * stride_lse + row];
      if (l == -INFINITY) continue;
      const float w = expf(l - mx);
      tot += w;
      const float4 v = reinterpret_cast<const float4*>(o_parts + c * stride_o)[size_t(row) * 32 + lane];
      acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
    }
    const float inv = 1.f / tot;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  }
  store4<OUT>(o_out, size_t(row) * 32 + lane, acc);
  if (lane == 0) lse_out[row] = mx == -INFINITY ? -INFINITY : mx + logf(tot);
}

int launch_fwd_merge_parts(const lvx_shape& s, const float* o_parts, const float* lse_parts, int count,
                           size_t stride_o, size_t stride_lse, void* o_out, float* lse_out, cudaStream_t st) {
  const long total_rows = long(q_blocks_of(s)) * s.B * s.Hq * s.Sq;
  const int threads = 256;
  const int* sp = device_status_ptr();
  const long blocks = (total_rows * 32 + threads - 1) / threads;
  if (s.dtype == LVX_BF16)
    fwd_merge_parts_kernel<0><<<blocks, threads, 0, st>>>(o_parts, lse_parts, count, stride_o, stride_lse, o_out, lse_out, total_rows, sp);
  else if (s.dtype == LVX_FP16)
    fwd_merge_parts_kernel<1><<<blocks, threads, 0, st>>>(o_parts, lse_parts, count, stride_o, stride_lse, o_out, lse_out, total_rows, sp);
  else
    fwd_merge_parts_kernel<2><<<blocks, threads, 0, st>>>(o_parts, lse_parts, count, stride_o, stride_lse, o_out, lse_out, total_rows, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "fwd_merge_parts launch");
  return LVX_OK;
}

// ---------------------------------------------------------------------------------------------
template <int IN>
__global__ void __launch_bounds__(256)
bwd_prep_kernel(const void* __restrict__ o, const void* __restrict__ d_o, float* __restrict__ delta, long total_rows,
                const int* status) {
  if (poisoned(status)) return;
  const int lane = threadIdx.x & 31;
  const long row = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= total_rows) return;
  const float4 a = load4<IN>(o, size_t(row) * 32 + lane);
  const float4 b = load4<IN>(d_o, size_t(row) * 32 + lane);
  float v = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if (lane == 0) delta[row] = v;
}

int launch_bwd_prep(const lvx_shape& s, const void* o, const void* d_o, float* delta, cudaStream_t st) {
  const long total_rows = long(q_blocks_of(s)) * s.B * s.Hq * s.Sq;
  const int threads = 256;
  const int* sp = device_status_ptr();
  const long blocks = (total_rows * 32 + threads - 1) / threads;
  if (s.dtype == LVX_BF16) bwd_prep_kernel<0><<<blocks, threads, 0, st>>>(o, d_o, delta, total_rows, sp);
  else if (s.dtype == LVX_FP16) bwd_prep_kernel<1><<<blocks, threads, 0, st>>>(o, d_o, delta, total_rows, sp);
  else bwd_prep_kernel<2><<<blocks, threads, 0, st>>>(o, d_o, delta, total_rows, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "bwd_prep launch");
  return LVX_OK;
}

// ---------------------------------------------------------------------------------------------
template <int OUT>
__global__ void __launch_bounds__(256)
add_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, void* __restrict__ out, size_t n4, size_t n,
                const int* status) {
  if (poisoned(status)) return;
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 v = reinterpret_cast<const float4*>(a)[i];
    if (b) {
      const float4 w = reinterpret_cast<const float4*>(b)[i];
      v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    store4<OUT>(out, i, v);
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const size_t i = n4 * 4 + threadIdx.x;
    const float v = a[i] + (b ? b[i] : 0.f);
    if (OUT == 2) reinterpret_cast<float*>(out)[i] = v;
    else if (OUT == 0) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
  }
}

int launch_add_cast(const float* a, const float* b, void* out, int out_dtype, size_t n, cudaStream_t st) {
  const size_t n4 = n / 4;
  const int threads = 256;
  const int* sp = device_status_ptr();
  size_t blocks = (n4 + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks == 0) blocks = 1;
  if (out_dtype == LVX_BF16) add_cast_kernel<0><<<blocks, threads, 0, st>>>(a, b, out, n4, n, sp);
  else if (out_dtype == LVX_FP16) add_cast_kernel<1><<<blocks, threads, 0, st>>>(a, b, out, n4, n, sp);
  else add_cast_kernel<2><<<blocks, threads, 0, st>>>(a, b, out, n4, n, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "add_cast launch");
  return LVX_OK;
}

// ---------------------------------------------------------------------------------------------
template <int OUT>
__global__ void __launch_bounds__(256)
sum_cast_kernel(const float* __restrict__ parts, int count, size_t stride, void* __restrict__ out, size_t n4,
                const int* status) {
  if (poisoned(status)) return;
  const size_t gstride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += gstride) {
    float4 v = reinterpret_cast<const float4*>(parts)[i];
    for (int c = 1; c < count; ++c) {
      const float4 w = reinterpret_cast<const float4*>(parts + c * stride)[i];
      v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    store4<OUT>(out, i, v);
  }
}

int launch_sum_cast(const float* parts, int count, size_t stride, void* out, int out_dtype, size_t n, cudaStream_t st) {
  const size_t n4 = n / 4;
  const int threads = 256;
  const int* sp = device_status_ptr();
  size_t blocks = (n4 + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks == 0) blocks = 1;
  if (out_dtype == LVX_BF16) sum_cast_kernel<0><<<blocks, threads, 0, st>>>(parts, count, stride, out, n4, sp);
  else if (out_dtype == LVX_FP16) sum_cast_kernel<1><<<blocks, threads, 0, st>>>(parts, count, stride, out, n4, sp);
  else sum_cast_kernel<2><<<blocks, threads, 0, st>>>(parts, count, stride, out, n4, sp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "sum_cast launch");
  return LVX_OK;
}

}  // namespace lvx
