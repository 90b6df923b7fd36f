// extern "C" surface of liblvx.so (see include/lvx.h): argument validation, error text,
// tensor-map encoding through the driver entry point, and the device status word.
#include "lvx_internal.h"
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace lvx {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return static_cast<int>(e) > 0 ? static_cast<int>(e) : 1;
}

// Device status word: one per device that loads the library, written by bounded waits that ran out.
__device__ int g_status_word[4];

static int* status_ptr() {
  static int* ptrs[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int make_tmap_3d(CUtensorMap* out, int dtype, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, bool swizzle_atom_32b) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(LVX_ERR_DRIVER, "cuTensorMapEncodeTiled could not be resolved");
  CUtensorMapDataType dt = dtype == LVX_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == LVX_FP16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(LVX_ERR_ALIGN, "tensor base %p is not 16-byte aligned", base);
  if (box0 * elt_size(dtype) != 128) return fail(LVX_ERR_SHAPE, "tensor-map box must be 128 bytes wide");
  cuuint64_t dims[3] = {dim0, dim1, dim2 ? dim2 : 1};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_atom_32b ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(LVX_ERR_SHAPE, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu,%llu,%llu box %u,%u)",
                int(r), (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)dim2, box0, box1);
  return LVX_OK;
}

static int check_arch() {
  static int cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev >= 0 && dev < 64 && cached[dev] == 1) return LVX_OK;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
  if (major != 10) return fail(LVX_ERR_ARCH, "device %d has compute capability %d.x; this library is sm_100a only", dev, major);
  if (dev >= 0 && dev < 64) cached[dev] = 1;
  return LVX_OK;
}

static int check_shape(const lvx_shape* s, const char* who) {
  if (!s) return fail(LVX_ERR_NULL, "%s: shape is NULL", who);
  if (s->D != 128) return fail(LVX_ERR_SHAPE, "%s: head dimension %d unsupported (128 only)", who, s->D);
  if (s->B <= 0 || s->Hq <= 0 || s->Hkv <= 0 || s->Sq <= 0 || s->Skv < 0)
    return fail(LVX_ERR_SHAPE, "%s: non-positive dimension (B=%d Hq=%d Hkv=%d Sq=%d Skv=%d)", who, s->B, s->Hq, s->Hkv,
                s->Sq, s->Skv);
  if (s->Hq % s->Hkv) return fail(LVX_ERR_SHAPE, "%s: Hq=%d is not a multiple of Hkv=%d", who, s->Hq, s->Hkv);
  if (s->dtype != LVX_BF16 && s->dtype != LVX_FP16 && s->dtype != LVX_FP32)
    return fail(LVX_ERR_DTYPE, "%s: dtype %d unsupported", who, s->dtype);
  if (s->q_blocks < 0 || s->q_blocks > 4096) return fail(LVX_ERR_SHAPE, "%s: q_blocks %d out of range", who, s->q_blocks);
  if (int64_t(s->Hq / s->Hkv) * s->Sq > (int64_t(1) << 30) ||
      int64_t(s->q_blocks > 1 ? s->q_blocks : 1) * s->B * s->Hkv > 65535)
    return fail(LVX_ERR_SHAPE, "%s: dimension too large", who);
  return LVX_OK;
}

// Non-static doors for the other translation units of the library.
int* device_status_ptr() { return status_ptr(); }
int validate_shape(const lvx_shape* s, const char* who) { return check_shape(s, who); }
int validate_arch() { return check_arch(); }

#define LVX_REQUIRE_PTR(p, who)                                           \
  do {                                                                    \
    if (!(p)) return lvx::fail(LVX_ERR_NULL, "%s: %s is NULL", who, #p);  \
    if (reinterpret_cast<uintptr_t>(p) & 15u)                             \
      return lvx::fail(LVX_ERR_ALIGN, "%s: %s is not 16-byte aligned", who, #p); \
  } while (0)

}  // namespace lvx

using namespace lvx;

extern "C" {

int lvx_version(void) { return LVX_ABI_VERSION; }

const char* lvx_last_error(void) { return g_err; }

int lvx_device_status(void* stream, int* status_out) {
  if (!status_out) return fail(LVX_ERR_NULL, "lvx_device_status: status_out is NULL");
  int* sp = status_ptr();
  if (!sp) return fail(LVX_ERR_DRIVER, "lvx_device_status: status word unavailable");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status_out, sp, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status)");
  e = cudaMemsetAsync(sp, 0, sizeof(int), st);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize(status)");
  return LVX_OK;
}

int lvx_device_status_peek(void* stream, int* host_out) {
  if (!host_out) return fail(LVX_ERR_NULL, "lvx_device_status_peek: host_out is NULL");
  int* sp = status_ptr();
  if (!sp) return fail(LVX_ERR_DRIVER, "lvx_device_status_peek: status word unavailable");
  cudaError_t e = cudaMemcpyAsync(host_out, sp, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status peek)");
  return LVX_OK;
}

int lvx_query_workspace(const lvx_shape* s, size_t* fwd_bytes, size_t* bwd_bytes) {
  int rc = check_shape(s, "lvx_query_workspace");
  if (rc) return rc;
  FwdPlan p = plan_fwd(*s);
  if (fwd_bytes) *fwd_bytes = p.o_part_bytes + p.ml_part_bytes;
  if (bwd_bytes) *bwd_bytes = 0;
  return LVX_OK;
}

static int check_block_wait(const lvx_shape* s, const lvx_block_wait* w, const char* who) {
  if (!w) return LVX_OK;
  if (s->dtype == LVX_FP32) return fail(LVX_ERR_DTYPE, "%s: the fp32 kernels do not take a block wait", who);
  const int qb = s->q_blocks > 1 ? s->q_blocks : 1;
  if (w->first_block < 0 || w->first_block >= qb) return fail(LVX_ERR_SHAPE, "%s: first_block %d outside [0, %d)", who, w->first_block, qb);
  if (w->my_flags) {
    if (w->slot < 0 || w->slot >= LVX_P2P_SLOTS) return fail(LVX_ERR_SHAPE, "%s: slot %d out of range", who, w->slot);
    if (qb > LVX_MAX_PEERS) return fail(LVX_ERR_SHAPE, "%s: %d blocks but only %d flag words per slot", who, qb, LVX_MAX_PEERS);
    if (reinterpret_cast<uintptr_t>(w->my_flags) & 3u) return fail(LVX_ERR_ALIGN, "%s: my_flags is misaligned", who);
  }
  return LVX_OK;
}

int lvx_fwd_block(const lvx_shape* s, const void* q, const void* k, const void* v, const int32_t* kv_valid_len,
                  float sm_scale, void* workspace, size_t workspace_bytes, void* stream) {
  return lvx_fwd_block_gathered(s, q, k, v, kv_valid_len, sm_scale, workspace, workspace_bytes, nullptr, stream);
}

int lvx_fwd_block_gathered(const lvx_shape* s, const void* q, const void* k, const void* v, const int32_t* kv_valid_len,
                           float sm_scale, void* workspace, size_t workspace_bytes, const lvx_block_wait* wait,
                           void* stream) {
  const char* who = wait ? "lvx_fwd_block_gathered" : "lvx_fwd_block";
  int rc = check_shape(s, who);
  if (!rc) rc = check_block_wait(s, wait, who);
  if (rc) return rc;
  if ((rc = check_arch())) return rc;
  LVX_REQUIRE_PTR(q, who);
  LVX_REQUIRE_PTR(workspace, who);
  if (s->Skv > 0) {
    LVX_REQUIRE_PTR(k, who);
    LVX_REQUIRE_PTR(v, who);
  }
  FwdPlan p = plan_fwd(*s);
  if (workspace_bytes < p.o_part_bytes + p.ml_part_bytes)
    return fail(LVX_ERR_WORKSPACE, "%s: workspace has %zu bytes, %zu needed", who, workspace_bytes,
                p.o_part_bytes + p.ml_part_bytes);
  int* sp = status_ptr();
  if (!sp) return fail(LVX_ERR_DRIVER, "%s: status word unavailable", who);
  float* o_part = static_cast<float*>(workspace);
  float* ml_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + p.o_part_bytes);
  return launch_fwd_block(*s, p, q, k, v, kv_valid_len, sm_scale, o_part, ml_part, sp,
                          static_cast<cudaStream_t>(stream), wait);
}

int lvx_fwd_combine_merge(const lvx_shape* s, const void* workspace, const float* o_in, const float* lse_in,
                          void* o_out, float* lse_out, int out_is_final, void* stream) {
  const char* who = "lvx_fwd_combine_merge";
  int rc = check_shape(s, who);
  if (rc) return rc;
  LVX_REQUIRE_PTR(workspace, who);
  LVX_REQUIRE_PTR(o_out, who);
  LVX_REQUIRE_PTR(lse_out, who);
  if ((o_in == nullptr) != (lse_in == nullptr))
    return fail(LVX_ERR_NULL, "%s: o_in and lse_in must both be given or both be NULL", who);
  FwdPlan p = plan_fwd(*s);
  const float* o_part = static_cast<const float*>(workspace);
  const float* ml_part = reinterpret_cast<const float*>(static_cast<const char*>(workspace) + p.o_part_bytes);
  return launch_fwd_combine(*s, p, o_part, ml_part, o_in, lse_in, o_out, lse_out, out_is_final,
                            static_cast<cudaStream_t>(stream));
}

int lvx_bwd_prep(const lvx_shape* s, const void* o, const void* d_o, float* delta, void* stream) {
  const char* who = "lvx_bwd_prep";
  int rc = check_shape(s, who);
  if (rc) return rc;
  LVX_REQUIRE_PTR(o, who);
  LVX_REQUIRE_PTR(d_o, who);
  LVX_REQUIRE_PTR(delta, who);
  return launch_bwd_prep(*s, o, d_o, delta, static_cast<cudaStream_t>(stream));
}

int lvx_bwd_block(const lvx_shape* s, const void* q, const void* d_o, const float* lse, const float* delta,
                  const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                  float* dk_acc, float* dv_acc, int accumulate_dkdv, void* workspace, size_t workspace_bytes,
                  void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  return lvx_bwd_block_gathered(s, q, d_o, lse, delta, k, v, kv_valid_len, sm_scale, dq_acc, dk_acc, dv_acc,
                                accumulate_dkdv, nullptr, stream);
}

int lvx_bwd_block_gathered(const lvx_shape* s, const void* q, const void* d_o, const float* lse, const float* delta,
                           const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                           float* dk_acc, float* dv_acc, int accumulate_dkdv, const lvx_block_wait* wait, void* stream) {
  const char* who = wait ? "lvx_bwd_block_gathered" : "lvx_bwd_block";
  int rc = check_shape(s, who);
  if (!rc) rc = check_block_wait(s, wait, who);
  if (rc) return rc;
  if ((rc = check_arch())) return rc;
  LVX_REQUIRE_PTR(q, who);
  LVX_REQUIRE_PTR(d_o, who);
  LVX_REQUIRE_PTR(lse, who);
  LVX_REQUIRE_PTR(delta, who);
  LVX_REQUIRE_PTR(dq_acc, who);
  if (s->Skv == 0) return LVX_OK;
  LVX_REQUIRE_PTR(k, who);
  LVX_REQUIRE_PTR(v, who);
  LVX_REQUIRE_PTR(dk_acc, who);
  LVX_REQUIRE_PTR(dv_acc, who);
  int* sp = status_ptr();
  if (!sp) return fail(LVX_ERR_DRIVER, "%s: status word unavailable", who);
  return launch_bwd_block(*s, q, d_o, lse, delta, k, v, kv_valid_len, sm_scale, dq_acc, dk_acc, dv_acc,
                          accumulate_dkdv, sp, static_cast<cudaStream_t>(stream), wait);
}

int lvx_fwd_block_bias(const lvx_shape* s, const void* q, const void* k, const void* v, const int32_t* kv_valid_len,
                       const lvx_bias* bias, float sm_scale, void* workspace, size_t workspace_bytes, void* stream) {
  const char* who = "lvx_fwd_block_bias";
  int rc = check_shape(s, who);
  if (rc) return rc;
  if ((rc = check_arch())) return rc;
  LVX_REQUIRE_PTR(q, who);
  LVX_REQUIRE_PTR(workspace, who);
  if (!bias || !bias->bias) return fail(LVX_ERR_NULL, "%s: bias is NULL (use lvx_fwd_block)", who);
  if (reinterpret_cast<uintptr_t>(bias->bias) & 3u) return fail(LVX_ERR_ALIGN, "%s: bias is not 4-byte aligned", who);
  if (!(sm_scale > 0.f)) return fail(LVX_ERR_SHAPE, "%s: sm_scale must be positive", who);
  if (s->Skv > 0) {
    LVX_REQUIRE_PTR(k, who);
    LVX_REQUIRE_PTR(v, who);
  }
  FwdPlan p = plan_fwd(*s);
  if (workspace_bytes < p.o_part_bytes + p.ml_part_bytes)
    return fail(LVX_ERR_WORKSPACE, "%s: workspace has %zu bytes, %zu needed", who, workspace_bytes,
                p.o_part_bytes + p.ml_part_bytes);
  float* o_part = static_cast<float*>(workspace);
  float* ml_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + p.o_part_bytes);
  return launch_fwd_block_simt(*s, p, q, k, v, kv_valid_len, bias, sm_scale, o_part, ml_part,
                               static_cast<cudaStream_t>(stream));
}

int lvx_bwd_block_bias(const lvx_shape* s, const void* q, const void* d_o, const float* lse, const float* delta,
                       const void* k, const void* v, const int32_t* kv_valid_len, const lvx_bias* bias, float sm_scale,
                       float* dq_acc, void* dk_acc, void* dv_acc, int accumulate_dkdv, void* stream) {
  const char* who = "lvx_bwd_block_bias";
  int rc = check_shape(s, who);
  if (rc) return rc;
  if ((rc = check_arch())) return rc;
  LVX_REQUIRE_PTR(q, who);
  LVX_REQUIRE_PTR(d_o, who);
  LVX_REQUIRE_PTR(lse, who);
  LVX_REQUIRE_PTR(delta, who);
  LVX_REQUIRE_PTR(dq_acc, who);
  if (!bias || !bias->bias) return fail(LVX_ERR_NULL, "%s: bias is NULL (use lvx_bwd_block)", who);
  if (!(sm_scale > 0.f)) return fail(LVX_ERR_SHAPE, "%s: sm_scale must be positive", who);
  if (accumulate_dkdv < 0 || accumulate_dkdv > 2)
    return fail(LVX_ERR_SHAPE, "%s: accumulate_dkdv must be 0, 1 or 2 (got %d)", who, accumulate_dkdv);
  if (s->Skv == 0) return LVX_OK;
  LVX_REQUIRE_PTR(k, who);
  LVX_REQUIRE_PTR(v, who);
  LVX_REQUIRE_PTR(dk_acc, who);
  LVX_REQUIRE_PTR(dv_acc, who);
  return launch_bwd_block_simt(*s, q, d_o, lse, delta, k, v, kv_valid_len, bias, sm_scale, dq_acc, dk_acc, dv_acc,
                               accumulate_dkdv, static_cast<cudaStream_t>(stream));
}

int lvx_kv_project(int dtype, const void* x, const void* wk, const void* wv, const void* norm_w, float eps, int batch,
                   int S, int Kd, int Hkv, void* k_out, void* v_out, float* rstd, void* stream) {
  const char* who = "lvx_kv_project";
  int rc = check_arch();
  if (rc) return rc;
  if (dtype != LVX_BF16 && dtype != LVX_FP16) return fail(LVX_ERR_DTYPE, "%s: dtype %d unsupported (bf16 or fp16)", who, dtype);
  if (batch <= 0 || S <= 0 || Kd <= 0 || Hkv <= 0) return fail(LVX_ERR_SHAPE, "%s: non-positive dimension", who);
  if (Kd % 64) return fail(LVX_ERR_SHAPE, "%s: Kd=%d is not a multiple of 64", who, Kd);
  if (Hkv % 2) return fail(LVX_ERR_SHAPE, "%s: Hkv=%d is odd (tiles hold two heads)", who, Hkv);
  if (int64_t(batch) * S > (int64_t(1) << 31) - 512) return fail(LVX_ERR_SHAPE, "%s: batch*S too large", who);
  if (!(eps >= 0.f)) return fail(LVX_ERR_SHAPE, "%s: eps must be non-negative", who);
  LVX_REQUIRE_PTR(x, who);
  LVX_REQUIRE_PTR(wk, who);
  LVX_REQUIRE_PTR(wv, who);
  LVX_REQUIRE_PTR(k_out, who);
  LVX_REQUIRE_PTR(v_out, who);
  if (norm_w && (reinterpret_cast<uintptr_t>(norm_w) & 1u)) return fail(LVX_ERR_ALIGN, "%s: norm_w is misaligned", who);
  int* sp = status_ptr();
  if (!sp) return fail(LVX_ERR_DRIVER, "%s: status word unavailable", who);
  return launch_kv_project(dtype, x, wk, wv, norm_w, eps, batch, S, Kd, Hkv, k_out, v_out, rstd, sp,
                           static_cast<cudaStream_t>(stream));
}

int lvx_knorm_bwd(int dtype, const void* k, const void* dk, const float* rstd, const void* norm_w, void* dkpre,
                  float* dw, size_t rows, void* stream) {
  const char* who = "lvx_knorm_bwd";
  if (dtype != LVX_BF16 && dtype != LVX_FP16) return fail(LVX_ERR_DTYPE, "%s: dtype %d unsupported (bf16 or fp16)", who, dtype);
  if (rows == 0) return LVX_OK;
  LVX_REQUIRE_PTR(k, who);
  LVX_REQUIRE_PTR(dk, who);
  LVX_REQUIRE_PTR(rstd, who);
  LVX_REQUIRE_PTR(dkpre, who);
  LVX_REQUIRE_PTR(dw, who);
  if (!norm_w || (reinterpret_cast<uintptr_t>(norm_w) & 7u)) return fail(LVX_ERR_ALIGN, "%s: norm_w must be given, 8-byte aligned", who);
  return launch_knorm_bwd(dtype, k, dk, rstd, norm_w, dkpre, dw, long(rows), static_cast<cudaStream_t>(stream));
}

int lvx_fwd_merge_parts(const lvx_shape* s, const float* o_parts, const float* lse_parts, int count,
                        size_t part_stride_o, size_t part_stride_lse, void* o_out, float* lse_out, void* stream) {
  const char* who = "lvx_fwd_merge_parts";
  int rc = check_shape(s, who);
  if (rc) return rc;
  LVX_REQUIRE_PTR(o_parts, who);
  LVX_REQUIRE_PTR(lse_parts, who);
  LVX_REQUIRE_PTR(o_out, who);
  LVX_REQUIRE_PTR(lse_out, who);
  if (count < 1 || (part_stride_o & 3) != 0) return fail(LVX_ERR_SHAPE, "%s: count must be >= 1 and the O stride a multiple of 4 floats", who);
  return launch_fwd_merge_parts(*s, o_parts, lse_parts, count, part_stride_o, part_stride_lse, o_out, lse_out,
                                static_cast<cudaStream_t>(stream));
}

int lvx_sum_cast(const float* parts, int count, size_t part_stride, void* out, int out_dtype, size_t n, void* stream) {
  const char* who = "lvx_sum_cast";
  if (n == 0) return LVX_OK;
  LVX_REQUIRE_PTR(parts, who);
  LVX_REQUIRE_PTR(out, who);
  if (count < 1 || (part_stride & 3) != 0 || (n & 3) != 0)
    return fail(LVX_ERR_SHAPE, "%s: count >= 1, stride and n multiples of 4 floats are required", who);
  if (out_dtype != LVX_BF16 && out_dtype != LVX_FP16 && out_dtype != LVX_FP32)
    return fail(LVX_ERR_DTYPE, "%s: dtype %d unsupported", who, out_dtype);
  return launch_sum_cast(parts, count, part_stride, out, out_dtype, n, static_cast<cudaStream_t>(stream));
}

int lvx_add_cast(const float* a, const float* b, void* out, int out_dtype, size_t n, void* stream) {
  const char* who = "lvx_add_cast";
  if (n == 0) return LVX_OK;
  LVX_REQUIRE_PTR(a, who);
  LVX_REQUIRE_PTR(out, who);
  if (b && (reinterpret_cast<uintptr_t>(b) & 15u)) return fail(LVX_ERR_ALIGN, "%s: b is not 16-byte aligned", who);
  if (out_dtype != LVX_BF16 && out_dtype != LVX_FP16 && out_dtype != LVX_FP32)
    return fail(LVX_ERR_DTYPE, "%s: dtype %d unsupported", who, out_dtype);
  return launch_add_cast(a, b, out, out_dtype, n, static_cast<cudaStream_t>(stream));
}

int lvx_selftest_mma(int mode, const void* a, const void* b, float* d_out, void* stream) {
  const char* who = "lvx_selftest_mma";
  int rc = check_arch();
  if (rc) return rc;
  LVX_REQUIRE_PTR(a, who);
  LVX_REQUIRE_PTR(b, who);
  LVX_REQUIRE_PTR(d_out, who);
  int* sp = status_ptr();
  if (!sp) return fail(LVX_ERR_DRIVER, "%s: status word unavailable", who);
  return launch_selftest(mode, a, b, d_out, sp, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
