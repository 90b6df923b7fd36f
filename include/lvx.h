/* lvx.h -- C ABI of liblvx.so: the sm_100a kernels behind lv_xattn's distributed cross-attention.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA stream it is given
 * (a cudaStream_t passed as void*), never synchronises the host, and returns an int:
 *    0   success
 *   <0   invalid argument (nothing was launched); lvx_last_error() says which
 *   >0   CUDA runtime / driver error code of the failing call
 * No C++ exception crosses this boundary. The library keeps no device memory of its own except
 * where an entry point says so; workspaces are supplied by the caller (sizes from
 * lvx_query_workspace).
 *
 * Each declaration names the part of the reference (uw-mad-dash/LV-XAttn) it stands in for.
 *
 * Layouts (all tensors dense, row-major in the listed order):
 *   q, dO, o        [B, Hq,  Sq,  D]   element type = shape.dtype
 *   k, v, dk, dv    [B, Hkv, Skv, D]   element type = shape.dtype (dk/dv accumulators: fp32)
 *   lse, delta      [B*Hq, Sq]         fp32, natural-log log-sum-exp / rowsum(O*dO)
 *   Hq must be a multiple of Hkv; query head h reads KV head h / (Hq/Hkv).  D must be 128.
 */
#ifndef LVX_H_
#define LVX_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LVX_ABI_VERSION 1

enum lvx_dtype { LVX_BF16 = 0, LVX_FP16 = 1, LVX_FP32 = 2 /* exact fp32 on the FP32-FMA pipe, no TF32 */ };

enum lvx_error {
  LVX_OK = 0,
  LVX_ERR_NULL = -1,        /* a required pointer is NULL                       */
  LVX_ERR_SHAPE = -2,       /* unsupported or inconsistent shape                */
  LVX_ERR_DTYPE = -3,       /* unsupported dtype                                */
  LVX_ERR_ALIGN = -4,       /* a pointer is not 16-byte aligned                 */
  LVX_ERR_WORKSPACE = -5,   /* workspace too small                              */
  LVX_ERR_ARCH = -6,        /* current device is not compute capability 10.x    */
  LVX_ERR_DRIVER = -7,      /* a driver entry point could not be resolved       */
  LVX_ERR_LIMIT = -8        /* size beyond a documented fixed limit             */
};

typedef struct lvx_shape {
  int32_t B;       /* batch                                  */
  int32_t Hq;      /* query heads                            */
  int32_t Hkv;     /* key/value heads (divides Hq)           */
  int32_t Sq;      /* query rows of the block being processed */
  int32_t Skv;     /* key/value rows resident on this GPU    */
  int32_t D;       /* head dimension (128)                   */
  int32_t dtype;   /* enum lvx_dtype                         */
  int32_t q_blocks; /* number of query blocks that share each K/V batch entry; 0 or 1 = one.
                     * With q_blocks = n the query-side tensors (q, dO, o, lse, delta, dq) carry a leading
                     * block axis: [n, B, Hq, Sq, D] / [n, B*Hq, Sq]; block i of batch b attends K/V batch b.
                     * Used to run the query blocks of all sequence-parallel ranks in one K/V pass. */
} lvx_shape;

/* Library / ABI version (LVX_ABI_VERSION). No reference counterpart (the reference is pure Python). */
int lvx_version(void);

/* Text of the last error on the calling thread. Replaces the reference's Python asserts
 * (lv_xattn/attn.py:305-309, lv_xattn/flash_attn_kernels.py:913-917) as the error channel. */
const char* lvx_last_error(void);

/* Device status word of the last kernels launched by this library on the current device
 * (0 = fine; otherwise the code of the bounded wait that ran out). Reads the word, clears it and
 * synchronises the stream it is given; while the word is non-zero every kernel of the library
 * returns at once without computing. The reference has no equivalent: its waits are unbounded
 * (lv_xattn/async_communication.py:301-305). */
int lvx_device_status(void* stream, int* status_out);

/* Non-blocking look at the same word: enqueues, on `stream`, a copy of the word into *host_out (which should
 * be pinned host memory that stays valid until the stream reaches the copy) and returns at once. The word is
 * not cleared. Lets a host loop notice a bounded wait that ran out (a lost or very late peer) one call later
 * without synchronising; the reference would simply block for ever (lv_xattn/async_communication.py:301-305). */
int lvx_device_status_peek(void* stream, int* host_out);

/* Bytes of scratch the forward / backward block kernels need for this shape.
 * Stands in for the per-step torch allocations in lv_xattn/attn.py:382-385 and
 * lv_xattn/flash_attn_kernels.py:920-921. */
int lvx_query_workspace(const lvx_shape* s, size_t* fwd_bytes, size_t* bwd_bytes);

/* One flash-attention forward block: the Q block [B,Hq,Sq,D] against the resident K/V shard.
 * Writes split-KV partial results (unnormalised O, running max, running sum) into `workspace`;
 * lvx_fwd_combine_merge turns them into (O, lse).
 * kv_valid_len (nullable, int32 [B], device): number of leading K/V rows of this shard that are
 * valid for each batch entry (key padding); rows beyond it contribute nothing.
 * Replaces the Triton _fwd_kernel and its launch, lv_xattn/attn.py:140-268 and :390-400, and the
 * K/V head expansion lv_xattn/attn.py:271-277 (GQA is handled inside the kernel). */
int lvx_fwd_block(const lvx_shape* s, const void* q, const void* k, const void* v,
                  const int32_t* kv_valid_len, float sm_scale, void* workspace, size_t workspace_bytes,
                  void* stream);

/* Reduce the split-KV partials of lvx_fwd_block and merge the result into the travelling
 * accumulator:  (o_in, lse_in) (+) partials -> (o_out, lse_out).
 * o_in / lse_in may be NULL, meaning the empty accumulator (O = 0, lse = -inf).
 * o_in, o_out are fp32 [B,Hq,Sq,D] when out_is_final == 0 (the travelling form); when
 * out_is_final != 0, o_out is written in shape.dtype (the tensor handed back to the caller).
 * The merge is log-sum-exp stable and yields (0, -inf) when both sides are empty.
 * Replaces _rescale_kernel, lv_xattn/attn.py:37-110 and :405-419. */
int lvx_fwd_combine_merge(const lvx_shape* s, const void* workspace, const float* o_in, const float* lse_in,
                          void* o_out, float* lse_out, int out_is_final, void* stream);

/* delta[b*Hq+h, i] = sum_d O[b,h,i,d] * dO[b,h,i,d]  (fp32).
 * Replaces _bwd_preprocess_do_o_dot, lv_xattn/flash_attn_kernels.py:287-329. */
int lvx_bwd_prep(const lvx_shape* s, const void* o, const void* d_o, float* delta, void* stream);

/* One flash-attention backward block: recomputes P from (q, k, lse), then
 *   dq_acc[B,Hq,Sq,D]   (fp32) += dS K            (reduce-add; the caller zeroes it)
 *   dk_acc[B,Hkv,Skv,D] (fp32) (+)= dS^T Q        (summed over the query heads of the KV group)
 *   dv_acc[B,Hkv,Skv,D] (fp32) (+)= P^T dO
 * accumulate_dkdv: 0 overwrites the fp32 dk_acc/dv_acc, 1 adds to them, 2 treats dk_acc/dv_acc as
 * tensors of shape.dtype and writes the finished gradients there (single-pass use).
 * Replaces _flash_attn_backward / _bwd_kernel, lv_xattn/flash_attn_kernels.py:904-1020 and
 * :364-819, and the per-step accumulation lv_xattn/attn.py:523-527. */
int lvx_bwd_block(const lvx_shape* s, const void* q, const void* d_o, const float* lse, const float* delta,
                  const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                  float* dk_acc, float* dv_acc, int accumulate_dkdv, void* workspace,
                  size_t workspace_bytes, void* stream);

/* Dense additive bias on the scores, S = sm_scale * q.k + bias (natural-log domain, not scaled): the reference's
 * bias_func protocol builds such a tensor for every step, lv_xattn/attn.py:386-389, and its kernels add it at
 * lv_xattn/attn.py:238-240 (forward) and lv_xattn/flash_attn_kernels.py:497-516 (backward recompute). `bias` is fp32
 * on the device; the value for (query block n, batch b, query head h, query row i, key j) is
 * bias[n*stride_block + b*stride_b + h*stride_h + i*stride_q + j*stride_kv] (strides in floats, 0 = broadcast,
 * e.g. stride_h = 0 for a [B,1,Sq,Skv] bias). -inf entries mask a key. No gradient is produced for the bias, as in
 * the reference. */
typedef struct lvx_bias {
  const float* bias;
  int64_t stride_block, stride_b, stride_h, stride_q, stride_kv;
} lvx_bias;

/* lvx_fwd_block / lvx_bwd_block with a dense bias (any dtype). These run the library's general FP32-FMA block
 * kernels instead of the tensor-core ones (key padding expressed as kv_valid_len stays on the tensor-core path);
 * same workspace, outputs and accumulate modes. */
int lvx_fwd_block_bias(const lvx_shape* s, const void* q, const void* k, const void* v,
                       const int32_t* kv_valid_len, const lvx_bias* bias, float sm_scale, void* workspace,
                       size_t workspace_bytes, void* stream);
int lvx_bwd_block_bias(const lvx_shape* s, const void* q, const void* d_o, const float* lse, const float* delta,
                       const void* k, const void* v, const int32_t* kv_valid_len, const lvx_bias* bias,
                       float sm_scale, float* dq_acc, void* dk_acc, void* dv_acc, int accumulate_dkdv, void* stream);

/* K/V projection of the visual states with the per-head RMSNorm of K fused in: one tensor-core GEMM
 *   Kpre = X Wk^T, V = X Wv^T,   K = Kpre * rsqrt(mean_d(Kpre^2) + eps) * norm_w   (per key and head, d = 0..127)
 * X [batch, S, Kd], Wk/Wv [Hkv*128, Kd] (row-major, the nn.Linear layout), norm_w [128]; all in `dtype` (LVX_BF16
 * or LVX_FP16). Outputs are written in the layout the attention kernels read: K, V [batch, Hkv, S, 128] in `dtype`,
 * and rstd [batch, Hkv, S] fp32 (nullable) for the backward of the norm. norm_w NULL = no norm. Kd must be a
 * multiple of 64 and Hkv even. Replaces k_proj / v_proj + view/transpose + repeat_kv + k_norm of the reference's
 * patched layer, test_llama3.py:394-419, which run in forward and again in the backward recompute (:197, :235). */
int lvx_kv_project(int dtype, const void* x, const void* wk, const void* wv, const void* norm_w, float eps,
                   int batch, int S, int Kd, int Hkv, void* k_out, void* v_out, float* rstd, void* stream);

/* Backward of that norm: dKpre = rstd * (norm_w * dK - (K / norm_w) * mean_d(K * dK)) and
 * dw[d] += sum over rows of dK * K / norm_w (dw fp32 [128], zeroed by the caller). K, dK, dKpre: `rows` rows of
 * 128 in `dtype` ([batch, Hkv, S, 128] flattened), rstd fp32 [rows]. The reference lets autograd do this through
 * MllamaTextRMSNorm (test_llama3.py:419). */
int lvx_knorm_bwd(int dtype, const void* k, const void* dk, const float* rstd, const void* norm_w, void* dkpre,
                  float* dw, size_t rows, void* stream);

/* Merge of `count` finished partial results of the same query block, each computed against a different
 * K/V shard: o_parts fp32 [count][B*Hq*Sq*D], lse_parts fp32 [count][B*Hq*Sq] -> o_out (shape.dtype) and
 * lse_out, with the same stable log-sum-exp merge as lvx_fwd_combine_merge ((0,-inf) is the neutral
 * element). part_stride_o / part_stride_lse are the distances, in floats, between consecutive partials.
 * This is the reduce step of the all-blocks-per-pass schedule; in the reference the same merge happens
 * one hop at a time in _rescale_kernel (lv_xattn/attn.py:37-110). */
int lvx_fwd_merge_parts(const lvx_shape* s, const float* o_parts, const float* lse_parts, int count,
                        size_t part_stride_o, size_t part_stride_lse, void* o_out, float* lse_out, void* stream);

/* out[i] = (dtype) sum_{c < count} parts[c * part_stride + i] over n fp32 elements: the reduce step for
 * dQ in the all-blocks-per-pass schedule (reference: lv_xattn/attn.py:527, one hop at a time). */
int lvx_sum_cast(const float* parts, int count, size_t part_stride, void* out, int out_dtype, size_t n,
                 void* stream);

/* out[i] = (dtype) (a[i] + b[i]) over n fp32 elements; b may be NULL; out_dtype is an lvx_dtype
 * (LVX_FP32 keeps fp32). Used for: travelling dQ += local dQ, and the final down-cast of
 * dQ/dK/dV. Replaces lv_xattn/attn.py:527 and lv_xattn/flash_attn_kernels.py:1020. */
int lvx_add_cast(const float* a, const float* b, void* out, int out_dtype, size_t n, void* stream);

/* Forward block + combine in one call that allocates nothing: (O, lse) of the Q block against the
 * K/V shard, O written in shape.dtype, lse fp32 [B*Hq, Sq]. This entry point has no counterpart in
 * the reference; it exists for callers that must not touch the device allocator when they call
 * (no cudaMalloc / cudaFree / framework allocator on a path that has a fixed memory budget or must
 * not synchronise the device). The split-KV partials go to a 32 MiB scratch area built into the
 * library image (held by every GPU that loads the library until the process exits) instead of a
 * caller workspace. The number of K/V splits is lowered until the partials fit; a shape whose
 * unsplit partials exceed the area (more than about 64,500 rows B*Hq*Sq) is refused with
 * LVX_ERR_LIMIT. The first call on a device looks up the area's device address; make that first
 * call outside any stream capture, and not from two host threads at once (the per-device address cache is
 * filled without a lock). All calls share the area, which keeps the previous call's
 * contents (the kernel overwrites every entry it later reads, so nothing needs clearing); two calls
 * whose kernels overlap on the GPU -- different streams or devices' streams on one GPU -- race on it. */
int lvx_fwd_block_static(const lvx_shape* s, const void* q, const void* k, const void* v,
                         const int32_t* kv_valid_len, float sm_scale, void* o_out, float* lse_out,
                         void* stream);

/* ---- Exchange over peer-mapped memory (NVLink / NVSwitch) ------------------------------------------------
 * The reference moves blocks between ranks with torch.distributed batch_isend_irecv
 * (send_recv_fwd_q, send_recv_fwd_Lo, send_recv_bwd_comp_reqs, send_recv_bwd_rescale_reqs and
 * launch_async_handles, lv_xattn/async_communication.py:210-299) and reduces after each hop. These entry points do the same
 * exchanges with the library's own kernels reading the peers' memory directly; they need one buffer per
 * rank that every rank of the group has mapped (CUDA IPC / VMM; the Python host side uses torch's symmetric
 * memory). `lvx_peers.ptr[s]` is the address, in THIS process, of rank s's copy of that buffer; all copies
 * have the same layout. Ordering uses a flag array of LVX_P2P_SLOTS x LVX_MAX_PEERS uint32 words per rank in
 * such a buffer, zero at start: the producer calls lvx_p2p_signal(flags, slot, epoch) after the kernels that
 * fill its buffer (same stream), which stores `epoch` into word [slot][rank] of every peer's array; a pulling
 * call names its own array (`my_flags`, a device pointer), the slot and the epoch it needs and waits inside
 * the kernel, at most lvx_p2p_set_timeout() seconds (120 unless changed), for all `world` words -- on time-out
 * it reads nothing, and lvx_device_status() returns 0x1300 | peer. Epochs of a slot must increase by one per use (compared
 * modulo 2^32); a buffer may be rewritten two epochs after it was signalled, so callers alternate two. */
#define LVX_MAX_PEERS 16
#define LVX_P2P_SLOTS 8
typedef struct lvx_peers {
  int32_t world;                      /* ranks in the group (<= LVX_MAX_PEERS) */
  int32_t rank;                       /* this rank */
  const void* ptr[LVX_MAX_PEERS];     /* ptr[s]: rank s's buffer as mapped in this process (16-byte aligned) */
  size_t nbytes;                      /* size of every rank's buffer; offsets and extents are checked against it
                                       * on the host before anything is launched (LVX_ERR_LIMIT) */
} lvx_peers;

/* Limit, in seconds, of the in-kernel wait for a peer's flag (all lvx_p2p_* calls of this process; 120 s at
 * start). The reference's wait_async_handles blocks without limit (lv_xattn/async_communication.py:301-305). */
int lvx_p2p_set_timeout(double seconds);

/* Publishes `epoch` for `slot` to every rank (stream-ordered after the producer kernels). */
int lvx_p2p_signal(const lvx_peers* flags, int slot, uint32_t epoch, void* stream);
/* All-gather by pulling: dst + s*dst_stride <- rank s's bytes [src_offset, src_offset+bytes) for every s
 * (this rank included). Replaces send_recv_fwd_q / send_recv_bwd_comp_reqs of the reference
 * (lv_xattn/async_communication.py:210-227, :247-273) when every rank needs every block. */
int lvx_p2p_gather(const lvx_peers* src, size_t src_offset, size_t bytes, void* dst, size_t dst_stride,
                   const uint32_t* my_flags, int slot, uint32_t epoch, void* stream);
/* lvx_fwd_merge_parts with partial c read from rank c's buffer: O fp32 [B*Hq*Sq*D] at byte o_offset, lse
 * fp32 [B*Hq*Sq] at byte lse_offset (the offsets select this rank's block inside the peers' buffers).
 * shape describes ONE block (q_blocks ignored). */
int lvx_p2p_fwd_merge(const lvx_shape* s, const lvx_peers* parts, size_t o_offset, size_t lse_offset, void* o_out,
                      float* lse_out, const uint32_t* my_flags, int slot, uint32_t epoch, void* stream);
/* lvx_sum_cast with partial c read from rank c's buffer at byte `offset` (n fp32 elements each). */
int lvx_p2p_sum_cast(const lvx_peers* parts, size_t offset, void* out, int out_dtype, size_t n,
                     const uint32_t* my_flags, int slot, uint32_t epoch, void* stream);

/* Push form of the same exchanges (stores over NVLink are posted, loads are round trips): one launch copies up to
 * LVX_P2P_MAX_SEGMENTS local segments into every rank's buffer and then publishes `epoch` for `slot` (after a
 * system-scope fence and a last-block count, inside the same kernel). For destination rank s a segment copies
 * `bytes` from src + s*src_stride (src_stride 0: the same block to everyone = all-gather; else block s to rank s =
 * all-to-all) to dst->ptr[s] + dst_offset + rank*dst_rank_stride. The consumer calls lvx_p2p_wait (a one-block
 * kernel with the bounded wait described above) and then runs the ordinary kernels on its own buffer:
 * lvx_fwd_block / lvx_bwd_block on gathered blocks, lvx_fwd_merge_parts / lvx_sum_cast on received partials.
 * Replaces send_recv_fwd_q, send_recv_fwd_Lo, send_recv_bwd_comp_reqs, send_recv_bwd_rescale_reqs +
 * wait_async_handles (lv_xattn/async_communication.py:210-289, :301-305). */
#define LVX_P2P_MAX_SEGMENTS 4
typedef struct lvx_push_segment {
  const void* src;
  size_t src_stride;
  size_t dst_offset;
  size_t dst_rank_stride;
  size_t bytes;
  size_t src_bytes;   /* size of the source allocation (0 = not checked): an all-to-all segment reads
                       * world*src_stride bytes from it */
} lvx_push_segment;
int lvx_p2p_push(const lvx_peers* dst, const lvx_peers* flags, const lvx_push_segment* segments, int nseg, int slot,
                 uint32_t epoch, int skip_self, void* stream);
/* skip_self != 0: the segments are stored into the peers' buffers only (this rank's own copy is filled by the
 * caller, e.g. with a local copy that need not wait for the link); the epoch is still published to every rank. */

/* lvx_p2p_push done by the copy engines instead of a kernel: one cudaMemcpyAsync per peer and segment followed by
 * a 4-byte copy of the epoch into that peer's flag word, all on `stream` (copies of one stream complete in order, so
 * a flag never overtakes its data). It needs no SM, so it proceeds while a kernel of this library that fills the
 * GPU -- and may itself be waiting for peers inside lvx_*_block_gathered -- is running on another stream. */
int lvx_p2p_push_dma(const lvx_peers* dst, const lvx_peers* flags, const lvx_push_segment* segments, int nseg, int slot,
                     uint32_t epoch, int skip_self, void* stream);

/* Fused exchange + compute: lvx_fwd_block / lvx_bwd_block on a gathered buffer ([q_blocks, B, Hq, Sq, D] etc.)
 * whose blocks are still being stored by the other ranks (lvx_p2p_push on their side) while the kernel runs. The
 * kernel starts with block `first_block` (this rank's own, in place at launch) and walks the others in ring order;
 * before it first touches block b it waits -- bounded by lvx_p2p_set_timeout, 0x1300 | b in the status word on
 * time-out -- until word [slot][b] of this rank's flag array has reached `epoch`. The transfer of the remote blocks
 * thus overlaps the work on the local one instead of preceding the launch. my_flags NULL: no waits, block order only.
 * This is the reference's "post the transfer for the next block, compute on the current one" overlap
 * (lv_xattn/attn.py:369-377, :481-498) moved inside one kernel launch. bf16 / fp16 only. */
typedef struct lvx_block_wait {
  const uint32_t* my_flags;   /* this rank's flag array (device pointer), LVX_P2P_SLOTS x LVX_MAX_PEERS words */
  int32_t slot;
  uint32_t epoch;
  int32_t first_block;        /* 0 .. q_blocks-1 */
} lvx_block_wait;
int lvx_fwd_block_gathered(const lvx_shape* s, const void* q, const void* k, const void* v,
                           const int32_t* kv_valid_len, float sm_scale, void* workspace, size_t workspace_bytes,
                           const lvx_block_wait* wait, void* stream);
int lvx_bwd_block_gathered(const lvx_shape* s, const void* q, const void* d_o, const float* lse, const float* delta,
                           const void* k, const void* v, const int32_t* kv_valid_len, float sm_scale, float* dq_acc,
                           float* dk_acc, float* dv_acc, int accumulate_dkdv, const lvx_block_wait* wait, void* stream);
int lvx_p2p_wait(const uint32_t* my_flags, int world, int slot, uint32_t epoch, void* stream);

/* Self-test of the tensor-core building blocks (TMA tile load, shared-memory and TMEM operand
 * descriptors, TMEM load/store): runs one 128 x N x K product in the operand arrangement `mode`
 * and writes D (fp32 [128,N]) to `d_out`. a/b are device buffers in the arrangement the mode
 * documents (see csrc/selftest.cu). No reference counterpart. */
int lvx_selftest_mma(int mode, const void* a, const void* b, float* d_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LVX_H_ */
