// Host-side declarations shared by the translation units of liblvx.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/lvx.h"

namespace lvx {

// printf-style setter of the thread-local error text returned by lvx_last_error(); returns `code`.
int fail(int code, const char* fmt, ...);
// Maps a cudaError_t to the ABI's positive return code and records its text.
int cuda_fail(cudaError_t e, const char* what);

// Encodes a 3-D tiled tensor map with 128-byte swizzle. dims/strides are given innermost first;
// stride[0] is implied by the element size. box2 is always 1. Returns an ABI status code.
int make_tmap_3d(CUtensorMap* out, int dtype, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1,
                 bool swizzle_atom_32b = false);

// Device status word of the current device (nullptr if it cannot be resolved), and the ABI's argument checks.
int* device_status_ptr();
int validate_shape(const lvx_shape* s, const char* who);
int validate_arch();

inline int q_blocks_of(const lvx_shape& s) { return s.q_blocks > 1 ? s.q_blocks : 1; }
inline int elt_size(int dtype) { return dtype == LVX_FP32 ? 4 : 2; }

// Split-KV plan of the forward block; shared by the kernel launcher, the combine kernel and
// lvx_query_workspace so that all three agree on the workspace layout.
struct FwdPlan {
  int rows;          // g * Sq : packed query rows per (batch, kv head)
  int m_blocks;      // CTAs along the packed rows (256 rows each)
  int kv_tiles;      // ceil(Skv / 128)
  int nsplit;        // CTAs along the K/V range
  int tiles_per_split;
  size_t o_part_bytes;   // fp32 [B*Hkv][nsplit][rows][D]
  size_t ml_part_bytes;  // fp32 [B*Hkv][nsplit][rows][2]
};
FwdPlan plan_fwd(const lvx_shape& s);

// Launchers (one per .cu). `status` is the device status word.
int launch_fwd_block(const lvx_shape& s, const FwdPlan& p, const void* q, const void* k, const void* v,
                     const int32_t* kv_valid_len, float sm_scale, float* o_part, float* ml_part, int* status,
                     cudaStream_t st, const lvx_block_wait* bw = nullptr);
int launch_fwd_combine(const lvx_shape& s, const FwdPlan& p, const float* o_part, const float* ml_part,
                       const float* o_in, const float* lse_in, void* o_out, float* lse_out, int out_is_final,
                       cudaStream_t st);
int launch_bwd_prep(const lvx_shape& s, const void* o, const void* d_o, float* delta, cudaStream_t st);
int launch_bwd_block(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                     const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                     float* dk_acc, float* dv_acc, int accumulate_dkdv, int* status, cudaStream_t st,
                     const lvx_block_wait* bw = nullptr);
// Limit of the in-kernel waits for a peer's flag, in SM cycles (lvx_p2p_set_timeout).
long long p2p_wait_limit_cycles();
// fp32 inputs (exact FP32-FMA kernels, same workspace layout and masking rules as the tensor-core path)
int launch_fwd_block_fp32(const lvx_shape& s, const FwdPlan& p, const void* q, const void* k, const void* v,
                          const int32_t* kv_valid_len, float sm_scale, float* o_part, float* ml_part, cudaStream_t st);
int launch_bwd_block_fp32(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                          const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                          float* dk_acc, float* dv_acc, int accumulate_dkdv, cudaStream_t st);
// The general (FP32-FMA) block kernels: any input dtype, optional dense additive bias.
int launch_fwd_block_simt(const lvx_shape& s, const FwdPlan& p, const void* q, const void* k, const void* v,
                          const int32_t* kv_valid_len, const lvx_bias* bias, float sm_scale, float* o_part,
                          float* ml_part, cudaStream_t st);
int launch_bwd_block_simt(const lvx_shape& s, const void* q, const void* d_o, const float* lse, const float* delta,
                          const void* k, const void* v, const int32_t* kv_valid_len, const lvx_bias* bias,
                          float sm_scale, float* dq_acc, void* dk_acc, void* dv_acc, int accumulate_dkdv,
                          cudaStream_t st);
// K/V projection with fused per-head RMSNorm (kvproj_sm100.cu) and the backward of that norm.
int launch_kv_project(int dtype, const void* x, const void* wk, const void* wv, const void* norm_w, float eps,
                      int batch, int s, int kd, int hkv, void* k_out, void* v_out, float* rstd, int* status,
                      cudaStream_t st);
int launch_knorm_bwd(int dtype, const void* k, const void* dk, const float* rstd, const void* norm_w, void* dkpre,
                     float* dw, long rows, cudaStream_t st);
int launch_fwd_merge_parts(const lvx_shape& s, const float* o_parts, const float* lse_parts, int count,
                           size_t stride_o, size_t stride_lse, void* o_out, float* lse_out, cudaStream_t st);
int launch_sum_cast(const float* parts, int count, size_t stride, void* out, int out_dtype, size_t n, cudaStream_t st);
int launch_add_cast(const float* a, const float* b, void* out, int out_dtype, size_t n, cudaStream_t st);
int launch_selftest(int mode, const void* a, const void* b, float* d_out, int* status, cudaStream_t st);

}  // namespace lvx
