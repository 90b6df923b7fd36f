// lvx_fwd_block_static: the forward block and its combine step run out of a scratch area that is part
// of the library image, so that a call allocates nothing -- no cudaMalloc, no cudaFree, no torch
// allocator. It is meant for callers that must not touch the device allocator at call time: code
// running inside a region where allocation is forbidden or would synchronise the device (a serving
// loop with a frozen memory budget, a callback on a latency-critical path, a host that has handed all
// free memory to another pool). Inputs and outputs are still the caller's buffers.
#include "lvx_internal.h"

namespace lvx {

// Scratch for the split-KV partials. Every GPU that loads the library keeps these 32 MiB until the
// process exits. All calls share it and it keeps whatever the previous call left behind.
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address
// a kernel can use has to be asked for, per device, with that device current.
static int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(LVX_ERR_LIMIT, "lvx_fwd_block_static: device index %d out of range", dev);
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (!p) return fail(LVX_ERR_DRIVER, "lvx_fwd_block_static: static scratch has no device address");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return LVX_OK;
}

// The regular split-KV plan, with the number of splits lowered until the partials fit the fixed area.
static bool plan_within(const lvx_shape& s, size_t cap, FwdPlan* out) {
  FwdPlan p = plan_fwd(s);
  for (;;) {
    p.tiles_per_split = p.kv_tiles > 0 ? (p.kv_tiles + p.nsplit - 1) / p.nsplit : 0;
    const size_t slabs = size_t(q_blocks_of(s)) * s.B * s.Hkv;
    p.o_part_bytes = (slabs * p.nsplit * p.rows * 128 * sizeof(float) + 255) & ~size_t(255);
    p.ml_part_bytes = (slabs * p.nsplit * p.rows * 2 * sizeof(float) + 255) & ~size_t(255);
    if (p.o_part_bytes + p.ml_part_bytes <= cap) {
      *out = p;
      return true;
    }
    if (p.nsplit == 1) return false;
    p.nsplit -= 1;
  }
}

}  // namespace lvx

using namespace lvx;

extern "C" int lvx_fwd_block_static(const lvx_shape* s, const void* q, const void* k, const void* v,
                                    const int32_t* kv_valid_len, float sm_scale, void* o_out, float* lse_out,
                                    void* stream) {
  const char* who = "lvx_fwd_block_static";
  int rc = validate_shape(s, who);
  if (rc) return rc;
  if ((rc = validate_arch())) return rc;
  const void* need[] = {q, o_out, lse_out};
  for (const void* p : need) {
    if (!p) return fail(LVX_ERR_NULL, "%s: q, o_out and lse_out are required", who);
    if (reinterpret_cast<uintptr_t>(p) & 15u) return fail(LVX_ERR_ALIGN, "%s: a pointer is not 16-byte aligned", who);
  }
  if (s->Skv > 0 && (!k || !v)) return fail(LVX_ERR_NULL, "%s: k and v are required", who);
  FwdPlan plan;
  if (!plan_within(*s, kStaticScratchBytes, &plan))
    return fail(LVX_ERR_LIMIT,
                "%s: the partials of this shape need more than the built-in %zu-byte scratch even unsplit "
                "(B*Hq*Sq = %lld rows; the limit is about %zu rows) -- use lvx_fwd_block with a workspace",
                who, kStaticScratchBytes, (long long)s->B * s->Hq * s->Sq, kStaticScratchBytes / (130 * sizeof(float)));
  void* scratch = nullptr;
  if ((rc = static_scratch_ptr(&scratch))) return rc;
  int* status = device_status_ptr();
  if (!status) return fail(LVX_ERR_DRIVER, "%s: status word unavailable", who);
  float* o_part = static_cast<float*>(scratch);
  float* ml_part = reinterpret_cast<float*>(static_cast<char*>(scratch) + plan.o_part_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = launch_fwd_block(*s, plan, q, k, v, kv_valid_len, sm_scale, o_part, ml_part, status, st);
  if (rc) return rc;
  // Every (slab, split, row) of the partials is written by the block kernel, so nothing in the
  // scratch has to be cleared between calls.
  return launch_fwd_combine(*s, plan, o_part, ml_part, nullptr, nullptr, o_out, lse_out, /*out_is_final=*/1, st);
}
