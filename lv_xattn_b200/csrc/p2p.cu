// Exchange steps of the sequence-parallel schedules done by this library's own kernels over peer-mapped memory
// (NVLink / NVSwitch) instead of a collective library: every rank keeps its outgoing blocks in a buffer that all
// ranks of the group have mapped (same layout on every rank), and the consumer pulls what it needs with plain
// loads -- the all-gather of the query-side blocks is a copy kernel, and the two all-to-all + reduce steps
// (forward partial (O, lse) -> merge, backward partial dQ -> sum) read the partials straight out of the peers'
// memory inside the reducing kernel, so the data crosses the link once and is never staged.
//
// Ordering between ranks is a flag protocol in the same mapped memory. After the kernels that produce a buffer, the
// owner runs p2p_signal_kernel: one system-scope release store of the epoch number into word [slot][owner] of every
// peer's flag array. A pulling kernel first waits until its own flag words [slot][0..W) have reached the epoch
// (system-scope acquire loads of local memory), bounded to a few seconds: if a peer never signals, the
// block records LVX_DEV_TIMEOUT_BASE | 0x300 | peer in the status word and returns without touching peer memory.
// A buffer may be rewritten two epochs later: by then every peer has signalled the epoch in between, which it
// does only after its pull of the earlier epoch has finished (stream order). Callers therefore alternate two
// buffers per slot. Only plain loads and stores touch peer memory (no TMA, no multicast).
//
// The push form (p2p_push_kernel + p2p_wait_kernel) turns the direction round: the producer stores its blocks into
// the consumers' buffers and publishes the epoch from the same kernel, after a system-scope fence by every thread
// and a last-block-done count; the consumer runs a one-block wait and then works on local memory with the ordinary
// kernels. Same flag words, same two-buffer rule (the consumer has read a buffer before it signals the epoch
// after, and the producer has waited for that signal before it stores into the buffer again).
#include "lvx_internal.h"
#include "sm100_prims.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

namespace lvx {

// A peer may legitimately be late by far more than a kernel's worth of time (a checkpoint write, a data-loader
// stall, an evaluation on one rank), so the wait for its flag has its own limit, set at run time in seconds
// (lvx_p2p_set_timeout; 120 s unless changed) and converted to SM cycles with the device's peak clock.
static double g_wait_seconds = 120.0;
static long long wait_limit_cycles();
long long p2p_wait_limit_cycles() { return wait_limit_cycles(); }
static long long wait_limit_cycles() {
  static int khz[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 120ll * 2000000000ll;
  if (!khz[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) != cudaSuccess || v <= 0) v = 2000000;
    khz[dev] = v;
  }
  const double cycles = g_wait_seconds * 1e3 * double(khz[dev]);
  return cycles < 1e3 ? 1000ll : (cycles > 9e18 ? (long long)9e18 : (long long)cycles);
}

struct PeerPtrs {
  const uint8_t* p[LVX_MAX_PEERS];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 16 bytes from (possibly peer) memory, not kept in L1.
__device__ __forceinline__ float4 ld_cg_f4(const void* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// Every block waits for all peers (thread 0 polls, the rest wait at the barrier). Returns false on time-out.
__device__ __forceinline__ bool p2p_wait_all(const uint32_t* my_flags, int world, int slot, uint32_t epoch, int* status,
                                             long long limit_cycles) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = (*reinterpret_cast<volatile int*>(status) == 0) ? 1 : 0;
    const long long t0 = clock64();
    for (int s = 0; s < world && ok; ++s) {
      const uint32_t* f = my_flags + slot * LVX_MAX_PEERS + s;
      while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
        if (clock64() - t0 > limit_cycles) {
          atomicCAS(status, 0, LVX_DEV_TIMEOUT_BASE | 0x300 | s);
          ok = 0;
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void p2p_signal_kernel(PeerPtrs flags, int world, int rank, int slot, uint32_t epoch) {
  const int s = threadIdx.x;
  if (s < world) {
    __threadfence_system();
    uint32_t* f = reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(flags.p[s])) + slot * LVX_MAX_PEERS + rank;
    st_release_sys(f, epoch);
  }
}

// dst + s*dst_stride <- peer s's [src_offset, src_offset + bytes) for every s; bytes is a multiple of 16.
__global__ void __launch_bounds__(256)
p2p_gather_kernel(PeerPtrs src, size_t src_offset, size_t bytes, uint8_t* __restrict__ dst, size_t dst_stride, int world,
                  const uint32_t* my_flags, int slot, uint32_t epoch, int* status, long long limit) {
  if (!p2p_wait_all(my_flags, world, slot, epoch, status, limit)) return;
  const size_t n16 = bytes >> 4;
  const size_t gstride = size_t(gridDim.x) * blockDim.x;
  const size_t gtid = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  // source by source (no index division in the copy loop); loads over NVLink are round trips: four in flight per thread
  for (int s = 0; s < world; ++s) {
    const uint8_t* from = src.p[s] + src_offset;
    uint8_t* to = dst + size_t(s) * dst_stride;
    for (size_t i0 = gtid; i0 < n16; i0 += 4 * gstride) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t i = i0 + size_t(u) * gstride;
        if (i < n16) v[u] = ld_cg_f4(from + (i << 4));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t i = i0 + size_t(u) * gstride;
        if (i < n16) reinterpret_cast<float4*>(to)[i] = v[u];
      }
    }
  }
}

template <int OUT>
__device__ __forceinline__ void p2p_store4(void* base, size_t idx4, float4 v) {
  if (OUT == 2) {
    reinterpret_cast<float4*>(base)[idx4] = v;
  } else if (OUT == 0) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    reinterpret_cast<uint2*>(base)[idx4] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  } else {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    reinterpret_cast<uint2*>(base)[idx4] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  }
}

// Merge of the `world` normalised partials (O fp32, lse) of this rank's rows, one per peer; one warp per row.
template <int OUT>
__global__ void __launch_bounds__(256)
p2p_fwd_merge_kernel(PeerPtrs parts, size_t o_offset, size_t lse_offset, int world, void* __restrict__ o_out,
                     float* __restrict__ lse_out, long total_rows, const uint32_t* my_flags, int slot, uint32_t epoch,
                     int* status, long long limit) {
  if (!p2p_wait_all(my_flags, world, slot, epoch, status, limit)) return;
  const int lane = threadIdx.x & 31;
  const long row = (long(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= total_rows) return;
  float ls[LVX_MAX_PEERS];
  float mx = -INFINITY;
#pragma unroll
  for (int c = 0; c < LVX_MAX_PEERS; ++c) {
    ls[c] = -INFINITY;
    if (c < world) {
      float v;
      asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(reinterpret_cast<const float*>(parts.p[c] + lse_offset) + row));
      ls[c] = v;
      mx = fmaxf(mx, v);
    }
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float tot = 0.f;
  if (mx != -INFINITY) {
#pragma unroll
    for (int c = 0; c < LVX_MAX_PEERS; ++c) {
      if (c < world && ls[c] != -INFINITY) {
        const float w = expf(ls[c] - mx);
        tot += w;
        const float4 v = ld_cg_f4(reinterpret_cast<const float4*>(parts.p[c] + o_offset) + size_t(row) * 32 + lane);
        acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
      }
    }
    const float inv = 1.f / tot;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
  }
  p2p_store4<OUT>(o_out, size_t(row) * 32 + lane, acc);
  if (lane == 0) lse_out[row] = mx == -INFINITY ? -INFINITY : mx + logf(tot);
}

// out[i] = (dtype) sum over peers of their fp32 block at `offset`.
template <int OUT>
__global__ void __launch_bounds__(256)
p2p_sum_cast_kernel(PeerPtrs parts, size_t offset, int world, void* __restrict__ out, size_t n4, const uint32_t* my_flags,
                    int slot, uint32_t epoch, int* status, long long limit) {
  if (!p2p_wait_all(my_flags, world, slot, epoch, status, limit)) return;
  const size_t gstride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += gstride) {
    float4 v[LVX_MAX_PEERS];
#pragma unroll
    for (int c = 0; c < LVX_MAX_PEERS; ++c)
      if (c < world) v[c] = ld_cg_f4(reinterpret_cast<const float4*>(parts.p[c] + offset) + i);
    float4 a = v[0];
#pragma unroll
    for (int c = 1; c < LVX_MAX_PEERS; ++c)
      if (c < world) { a.x += v[c].x; a.y += v[c].y; a.z += v[c].z; a.w += v[c].w; }
    p2p_store4<OUT>(out, i, a);
  }
}

// ---- push form: the producer stores into the consumers' memory, the consumer only waits -----------------
// Stores over NVLink are posted, loads are round trips: pushing moves the same bytes in less time than pulling.
struct PushSeg {
  const uint8_t* src;       // local source
  size_t src_stride;        // 0: the same bytes go to every rank (all-gather); else block s goes to rank s (all-to-all)
  size_t dst_offset;        // byte offset inside the peers' buffer
  size_t dst_rank_stride;   // this rank's data lands at dst_offset + rank * dst_rank_stride
  size_t bytes;             // per destination, multiple of 16
};
struct PushArgs {
  PushSeg seg[LVX_P2P_MAX_SEGMENTS];
  int nseg;
  int skip_self;     // 1: this rank's own copy of the buffer is filled by the caller, only the peers are written
};

__device__ unsigned int g_push_done[LVX_P2P_SLOTS];

// Every block copies its share of every (segment, destination) pair; each thread fences its stores at system
// scope; the block that finishes last publishes the epoch to every rank, so the flag can never overtake the data.
__global__ void __launch_bounds__(256)
p2p_push_kernel(PeerPtrs dst, PeerPtrs flags, PushArgs a, int world, int rank, int slot, uint32_t epoch) {
  const size_t gstride = size_t(gridDim.x) * blockDim.x;
  const size_t gtid = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int g = 0; g < a.nseg; ++g) {
    const PushSeg sg = a.seg[g];
    const size_t n16 = sg.bytes >> 4;
    // destination by destination (no index division in the copy loop); four 16-byte chunks per thread and round,
    // all loads issued before the first (posted) store, so that the copy is bound by the link and not by one
    // load-store round trip at a time
    for (int r = 0; r < world; ++r) {
      if (a.skip_self && r == rank) continue;
      const uint8_t* src = sg.src + size_t(r) * sg.src_stride;
      uint8_t* d = const_cast<uint8_t*>(dst.p[r]) + sg.dst_offset + size_t(rank) * sg.dst_rank_stride;
      for (size_t i0 = gtid; i0 < n16; i0 += 4 * gstride) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const size_t i = i0 + size_t(u) * gstride;
          if (i < n16) v[u] = reinterpret_cast<const float4*>(src)[i];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const size_t i = i0 + size_t(u) * gstride;
          if (i < n16) reinterpret_cast<float4*>(d)[i] = v[u];
        }
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(&g_push_done[slot], 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) g_push_done[slot] = 0;     // launches on one slot are stream-ordered
    if (threadIdx.x < world) {
      __threadfence_system();
      uint32_t* f = reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(flags.p[threadIdx.x])) + slot * LVX_MAX_PEERS + rank;
      st_release_sys(f, epoch);
    }
  }
}

__global__ void p2p_wait_kernel(const uint32_t* my_flags, int world, int slot, uint32_t epoch, int* status,
                                long long limit) {
  p2p_wait_all(my_flags, world, slot, epoch, status, limit);
}

static int peers_ok(const lvx_peers* p, const char* who) {
  if (!p) return fail(LVX_ERR_NULL, "%s: null peer table", who);
  if (p->world < 1 || p->world > LVX_MAX_PEERS || p->rank < 0 || p->rank >= p->world)
    return fail(LVX_ERR_SHAPE, "%s: world %d / rank %d out of range (at most %d peers)", who, p->world, p->rank, LVX_MAX_PEERS);
  for (int i = 0; i < p->world; ++i) {
    if (!p->ptr[i]) return fail(LVX_ERR_NULL, "%s: peer %d has no address", who, i);
    if (reinterpret_cast<uintptr_t>(p->ptr[i]) & 15u) return fail(LVX_ERR_ALIGN, "%s: peer %d address is not 16-byte aligned", who, i);
  }
  return LVX_OK;
}
// [offset, offset + bytes) must lie inside every peer's mapping (host-side bounds check: a wrong offset would
// otherwise become a load or store into another GPU's memory).
static int range_ok(const lvx_peers* p, size_t offset, size_t bytes, const char* who, const char* what) {
  if (p->nbytes == 0) return fail(LVX_ERR_SHAPE, "%s: the peer table carries no buffer size (nbytes = 0)", who);
  if (offset > p->nbytes || bytes > p->nbytes - offset)
    return fail(LVX_ERR_LIMIT, "%s: %s [%zu, +%zu) runs past the %zu-byte peer buffer", who, what, offset, bytes,
                size_t(p->nbytes));
  return LVX_OK;
}
static PeerPtrs to_dev(const lvx_peers* p) {
  PeerPtrs d;
  for (int i = 0; i < LVX_MAX_PEERS; ++i) d.p[i] = i < p->world ? static_cast<const uint8_t*>(p->ptr[i]) : nullptr;
  return d;
}
static int grid_for(size_t work_items) {
  size_t b = (work_items + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  return b ? int(b) : 1;
}

}  // namespace lvx

using namespace lvx;

extern "C" {

int lvx_p2p_signal(const lvx_peers* flags, int slot, uint32_t epoch, void* stream) {
  const char* who = "lvx_p2p_signal";
  int rc = peers_ok(flags, who);
  if (rc) return rc;
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  if ((rc = range_ok(flags, 0, sizeof(uint32_t) * LVX_P2P_SLOTS * LVX_MAX_PEERS, who, "the flag array"))) return rc;
  p2p_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(to_dev(flags), flags->world, flags->rank, slot, epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LVX_OK : cuda_fail(e, who);
}

int lvx_p2p_gather(const lvx_peers* src, size_t src_offset, size_t bytes, void* dst, size_t dst_stride,
                   const uint32_t* my_flags, int slot, uint32_t epoch, void* stream) {
  const char* who = "lvx_p2p_gather";
  int rc = peers_ok(src, who);
  if (rc) return rc;
  if (!dst || !my_flags) return fail(LVX_ERR_NULL, "%s: null pointer", who);
  if ((bytes & 15u) || (src_offset & 15u) || (dst_stride & 15u) || (reinterpret_cast<uintptr_t>(dst) & 15u))
    return fail(LVX_ERR_ALIGN, "%s: sizes, offsets and dst must be multiples of 16 bytes", who);
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  if ((rc = range_ok(src, src_offset, bytes, who, "the source range"))) return rc;
  int* status = device_status_ptr();
  if (!status) return fail(LVX_ERR_DRIVER, "%s: no device status word", who);
  if (bytes == 0) return LVX_OK;
  p2p_gather_kernel<<<grid_for(((bytes >> 4) + 3) / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_dev(src), src_offset, bytes, static_cast<uint8_t*>(dst), dst_stride, src->world, my_flags, slot, epoch, status,
      wait_limit_cycles());
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LVX_OK : cuda_fail(e, who);
}

int lvx_p2p_fwd_merge(const lvx_shape* s, const lvx_peers* parts, size_t o_offset, size_t lse_offset, void* o_out,
                      float* lse_out, const uint32_t* my_flags, int slot, uint32_t epoch, void* stream) {
  const char* who = "lvx_p2p_fwd_merge";
  int rc = validate_shape(s, who);
  if (rc) return rc;
  if ((rc = peers_ok(parts, who))) return rc;
  if (!o_out || !lse_out || !my_flags) return fail(LVX_ERR_NULL, "%s: null pointer", who);
  if ((o_offset & 15u) || (lse_offset & 3u)) return fail(LVX_ERR_ALIGN, "%s: offsets must be aligned (16 / 4 bytes)", who);
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  int* status = device_status_ptr();
  if (!status) return fail(LVX_ERR_DRIVER, "%s: no device status word", who);
  const long total_rows = long(s->B) * s->Hq * s->Sq;
  if ((rc = range_ok(parts, o_offset, size_t(total_rows) * 128 * sizeof(float), who, "the O partial"))) return rc;
  if ((rc = range_ok(parts, lse_offset, size_t(total_rows) * sizeof(float), who, "the lse partial"))) return rc;
  const long blocks = (total_rows * 32 + 255) / 256;
  if (blocks == 0) return LVX_OK;
  const PeerPtrs d = to_dev(parts);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long lim = wait_limit_cycles();
  if (s->dtype == LVX_BF16)
    p2p_fwd_merge_kernel<0><<<blocks, 256, 0, st>>>(d, o_offset, lse_offset, parts->world, o_out, lse_out, total_rows, my_flags, slot, epoch, status, lim);
  else if (s->dtype == LVX_FP16)
    p2p_fwd_merge_kernel<1><<<blocks, 256, 0, st>>>(d, o_offset, lse_offset, parts->world, o_out, lse_out, total_rows, my_flags, slot, epoch, status, lim);
  else
    p2p_fwd_merge_kernel<2><<<blocks, 256, 0, st>>>(d, o_offset, lse_offset, parts->world, o_out, lse_out, total_rows, my_flags, slot, epoch, status, lim);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LVX_OK : cuda_fail(e, who);
}

int lvx_p2p_sum_cast(const lvx_peers* parts, size_t offset, void* out, int out_dtype, size_t n, const uint32_t* my_flags,
                     int slot, uint32_t epoch, void* stream) {
  const char* who = "lvx_p2p_sum_cast";
  int rc = peers_ok(parts, who);
  if (rc) return rc;
  if (!out || !my_flags) return fail(LVX_ERR_NULL, "%s: null pointer", who);
  if ((offset & 15u) || (n & 3u)) return fail(LVX_ERR_ALIGN, "%s: offset must be a multiple of 16 bytes and n of 4 floats", who);
  if (out_dtype != LVX_BF16 && out_dtype != LVX_FP16 && out_dtype != LVX_FP32) return fail(LVX_ERR_DTYPE, "%s: dtype %d unsupported", who, out_dtype);
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  if ((rc = range_ok(parts, offset, n * sizeof(float), who, "the partial"))) return rc;
  int* status = device_status_ptr();
  if (!status) return fail(LVX_ERR_DRIVER, "%s: no device status word", who);
  if (n == 0) return LVX_OK;
  const size_t n4 = n / 4;
  const PeerPtrs d = to_dev(parts);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int g = grid_for(n4);
  const long long lim = wait_limit_cycles();
  if (out_dtype == LVX_BF16) p2p_sum_cast_kernel<0><<<g, 256, 0, st>>>(d, offset, parts->world, out, n4, my_flags, slot, epoch, status, lim);
  else if (out_dtype == LVX_FP16) p2p_sum_cast_kernel<1><<<g, 256, 0, st>>>(d, offset, parts->world, out, n4, my_flags, slot, epoch, status, lim);
  else p2p_sum_cast_kernel<2><<<g, 256, 0, st>>>(d, offset, parts->world, out, n4, my_flags, slot, epoch, status, lim);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LVX_OK : cuda_fail(e, who);
}

int lvx_p2p_push(const lvx_peers* dst, const lvx_peers* flags, const lvx_push_segment* segments, int nseg, int slot,
                 uint32_t epoch, int skip_self, void* stream) {
  const char* who = "lvx_p2p_push";
  int rc = peers_ok(dst, who);
  if (rc) return rc;
  if ((rc = peers_ok(flags, who))) return rc;
  if (flags->world != dst->world || flags->rank != dst->rank) return fail(LVX_ERR_SHAPE, "%s: the two peer tables disagree", who);
  if (!segments || nseg < 1 || nseg > LVX_P2P_MAX_SEGMENTS) return fail(LVX_ERR_SHAPE, "%s: 1..%d segments", who, LVX_P2P_MAX_SEGMENTS);
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  if ((rc = range_ok(flags, 0, sizeof(uint32_t) * LVX_P2P_SLOTS * LVX_MAX_PEERS, who, "the flag array"))) return rc;
  PushArgs a;
  a.nseg = nseg;
  a.skip_self = skip_self ? 1 : 0;
  size_t most = 0;
  for (int g = 0; g < nseg; ++g) {
    const lvx_push_segment& u = segments[g];
    if (!u.src) return fail(LVX_ERR_NULL, "%s: segment %d has no source", who, g);
    if ((reinterpret_cast<uintptr_t>(u.src) & 15u) || (u.src_stride & 15u) || (u.dst_offset & 15u) || (u.dst_rank_stride & 15u) ||
        (u.bytes & 15u))
      return fail(LVX_ERR_ALIGN, "%s: segment %d: addresses, strides and sizes must be multiples of 16 bytes", who, g);
    // every rank writes at dst_offset + rank*dst_rank_stride: the last rank's block must still fit
    if ((rc = range_ok(dst, u.dst_offset + size_t(dst->world - 1) * u.dst_rank_stride, u.bytes, who, "a segment's destination")))
      return rc;
    if (u.src_bytes && (u.src_stride ? size_t(dst->world - 1) * u.src_stride + u.bytes : u.bytes) > u.src_bytes)
      return fail(LVX_ERR_LIMIT, "%s: segment %d reads past its %zu-byte source", who, g, size_t(u.src_bytes));
    a.seg[g].src = static_cast<const uint8_t*>(u.src);
    a.seg[g].src_stride = u.src_stride;
    a.seg[g].dst_offset = u.dst_offset;
    a.seg[g].dst_rank_stride = u.dst_rank_stride;
    a.seg[g].bytes = u.bytes;
    if (u.bytes > most) most = u.bytes;
  }
  p2p_push_kernel<<<grid_for(((most >> 4) + 3) / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_dev(dst), to_dev(flags), a, dst->world, dst->rank, slot, epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LVX_OK : cuda_fail(e, who);
}

int lvx_p2p_push_dma(const lvx_peers* dst, const lvx_peers* flags, const lvx_push_segment* segments, int nseg, int slot,
                     uint32_t epoch, int skip_self, void* stream) {
  const char* who = "lvx_p2p_push_dma";
  int rc = peers_ok(dst, who);
  if (rc) return rc;
  if ((rc = peers_ok(flags, who))) return rc;
  if (flags->world != dst->world || flags->rank != dst->rank) return fail(LVX_ERR_SHAPE, "%s: the two peer tables disagree", who);
  if (!segments || nseg < 1 || nseg > LVX_P2P_MAX_SEGMENTS) return fail(LVX_ERR_SHAPE, "%s: 1..%d segments", who, LVX_P2P_MAX_SEGMENTS);
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  if ((rc = range_ok(flags, 0, sizeof(uint32_t) * LVX_P2P_SLOTS * LVX_MAX_PEERS, who, "the flag array"))) return rc;
  const int world = dst->world, rank = dst->rank;
  for (int g = 0; g < nseg; ++g) {
    const lvx_push_segment& u = segments[g];
    if (!u.src) return fail(LVX_ERR_NULL, "%s: segment %d has no source", who, g);
    if ((rc = range_ok(dst, u.dst_offset + size_t(world - 1) * u.dst_rank_stride, u.bytes, who, "a segment's destination")))
      return rc;
    if (u.src_bytes && (u.src_stride ? size_t(world - 1) * u.src_stride + u.bytes : u.bytes) > u.src_bytes)
      return fail(LVX_ERR_LIMIT, "%s: segment %d reads past its %zu-byte source", who, g, size_t(u.src_bytes));
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Peer by peer, starting after this rank (so that at any moment the ranks write to different peers): the data
  // copies, then the 4-byte epoch. Copies of one stream run in order, so the epoch lands after the data.
  for (int step = 0; step < world; ++step) {
    const int s = (rank + 1 + step) % world;
    if (!(skip_self && s == rank)) {
      for (int g = 0; g < nseg; ++g) {
        const lvx_push_segment& u = segments[g];
        if (u.bytes == 0) continue;
        uint8_t* d = const_cast<uint8_t*>(static_cast<const uint8_t*>(dst->ptr[s])) + u.dst_offset + size_t(rank) * u.dst_rank_stride;
        const uint8_t* src = static_cast<const uint8_t*>(u.src) + size_t(s) * u.src_stride;
        cudaError_t e = cudaMemcpyAsync(d, src, u.bytes, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "lvx_p2p_push_dma: data copy");
      }
    }
    uint32_t* f = reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(static_cast<const uint8_t*>(flags->ptr[s]))) + slot * LVX_MAX_PEERS + rank;
    // the source is a host variable: the runtime stages it before the call returns
    cudaError_t e = cudaMemcpyAsync(f, &epoch, sizeof(uint32_t), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_fail(e, "lvx_p2p_push_dma: epoch copy");
  }
  return LVX_OK;
}

int lvx_p2p_wait(const uint32_t* my_flags, int world, int slot, uint32_t epoch, void* stream) {
  const char* who = "lvx_p2p_wait";
  if (!my_flags) return fail(LVX_ERR_NULL, "%s: null flag array", who);
  if (world < 1 || world > LVX_MAX_PEERS) return fail(LVX_ERR_SHAPE, "%s: world %d out of range", who, world);
  if (slot < 0 || slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, slot);
  int* status = device_status_ptr();
  if (!status) return fail(LVX_ERR_DRIVER, "%s: no device status word", who);
  p2p_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(my_flags, world, slot, epoch, status,
                                                                   wait_limit_cycles());
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LVX_OK : cuda_fail(e, who);
}

int lvx_p2p_set_timeout(double seconds) {
  if (!(seconds > 0.0) || seconds > 86400.0)
    return fail(LVX_ERR_SHAPE, "lvx_p2p_set_timeout: %g s is outside (0, 86400]", seconds);
  g_wait_seconds = seconds;
  return LVX_OK;
}

}  // extern "C"
