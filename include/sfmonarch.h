/*
 * sfmonarch.h - C ABI of libsfmonarch.so: Monarch-structured self-attention for the
 * causal Wan DiT's chunk-wise KV-cache rollout, hand-written CUDA for sm_100a.
 *
 * Every entry point takes plain pointers, sizes and a cudaStream_t (passed as void*),
 * launches on that stream without synchronising the device, and returns an int:
 *   0   success
 *   <0  argument / shape / alignment / capability error (SFM_ERR_*)
 *   >0  a cudaError_t reported by the runtime
 * Device tensors are bf16 (uint16 storage) unless stated.  "Natural order" is the
 * model's token order [B, N, H, D]; "Monarch order" is the block order produced by
 * the layout map below.  The caller owns every buffer; nothing is allocated here.
 *
 * Each declaration names the reference interface it stands in for (paths inside the
 * reference project).
 */
#ifndef SFMONARCH_H_
#define SFMONARCH_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SFM_OK                    0
#define SFM_ERR_NULL_POINTER     -1
#define SFM_ERR_BAD_SHAPE        -2   /* sizes inconsistent with the blocking            */
#define SFM_ERR_UNSUPPORTED      -3   /* head_dim != 128, b2 > 64, ...                   */
#define SFM_ERR_ALIGNMENT        -4   /* pointers / strides must be 16-byte aligned      */
#define SFM_ERR_WORKSPACE        -5   /* workspace too small                             */
#define SFM_ERR_NO_DEVICE        -6   /* not an sm_100 device                            */
#define SFM_ERR_DEVICE_STATUS    -7   /* a kernel recorded an internal error status      */
#define SFM_ERR_STATIC_SCRATCH   -8   /* too large for the built-in scratch array        */

/* Version of this ABI (major*100 + minor). */
int sfm_version(void);

/* Static text for a return code of this library (never NULL). */
const char* sfm_error_string(int code);

/*
 * Blocking of an h x w token grid, shared by the calls below:
 *   f_tied   frames tied into one Monarch group (1 = framewise, 3 = tied3frame)
 *   h_reduce, w_reduce   split of the rows / columns of a frame into bands
 *   h, w     token rows / columns per latent frame (30 x 52 at 480p)
 * giving b1 = f_tied*h/h_reduce block rows, b2 = w/w_reduce block columns and
 * h_reduce*w_reduce groups per f_tied frames.
 */

/*
 * Token permutation between natural and Monarch order for n_tokens tokens.
 * Host pointers; either output may be NULL.  nat2mon[n] = Monarch position of natural
 * token n; mon2nat is the inverse.
 * Replaces: _get_rearrange_fns (wan/modules/monarch_attn.py:1696-1703).
 */
int sfm_build_maps(int32_t* nat2mon, int32_t* mon2nat, int n_tokens,
                   int f_tied, int h_reduce, int w_reduce, int h, int w);

/*
 * Rotary table on the HOST: out[pos][m] = {cos, sin} (fp32, from fp64 angles) for
 * pos < max_len and pair m < head_dim/2; pairs are split frame/row/column as
 * (c-2*(c/3), c/3, c/3) with c = head_dim/2, axis with p pairs using
 * pos * theta^(-m'/p).  out holds max_len*head_dim floats.
 * Replaces: rope_params (wan/modules/model.py:421-428) as assembled at
 * wan/modules/causal_model.py:1352-1357.
 */
int sfm_rope_table(float* out, int head_dim, int max_len, double theta);

/*
 * Fused 3-axis RoPE + layout + in-place KV-cache write (one pass, 16-byte accesses).
 *   q, k, v      [B, n_new, H, D] natural order, contiguous; q may be NULL
 *   q_out        [B, n_new, H, D] natural order: rotated q (ignored when q is NULL)
 *   k_cache, v_cache   [B, >= start_idx+n_new, H, D], batch stride cache_batch_stride
 *                (elements); tokens [start_idx, start_idx+n_new) are overwritten with
 *                rotated k and v, in Monarch order when monarch_order != 0, else natural
 *   rope         device table from sfm_rope_table (max_len 1024), or NULL: no rotation
 *                (inputs already rotated); frame position = start_frame + frame index,
 *                the chunk being a (n_new/(h*w)) x h x w grid
 * Replaces: causal_rope_apply (wan/modules/causal_model.py:687-715), the einops
 * permutes and slice assignment of monarch_attn_with_kv_cache
 * (wan/modules/monarch_attn.py:1782-1785, 1230-1231) and the natural-order cache write
 * of the dense branch (wan/modules/causal_model.py:961-962).
 */
int sfm_rope_cache_write(const void* q, const void* k, const void* v, void* q_out,
                         void* k_cache, void* v_cache, int64_t cache_batch_stride,
                         const float* rope, int B, int n_new, int H, int D,
                         int start_idx, int f_tied, int h_reduce, int w_reduce, int h, int w,
                         int start_frame, int monarch_order, void* stream);

/*
 * Stand-alone 3-axis RoPE of one tensor x [B, L, H, D] -> out (same shape): the first
 * frames*h*w tokens are rotated as a frames x h x w grid whose frame positions start at
 * start_frame; the rest are copied.  rope = device table from sfm_rope_table.
 * Replaces: causal_rope_apply (wan/modules/causal_model.py:687-715).
 */
int sfm_rope_apply(const void* x, void* out, const float* rope, int B, int L, int H, int D,
                   int frames, int h, int w, int start_frame, void* stream);

/*
 * Scratch bytes sfm_monarch_fwd needs for these sizes.  The row-step results (aL, Y,
 * cL) of one chunk of (batch, head, query-group) live there between the two kernels;
 * bridge_budget_bytes bounds one chunk so that it stays L2 resident (0 = default).
 * Replaces: the aL / y / cL scratch tensors of _attention_with_cache.forward
 * (wan/modules/monarch_attn.py:1246-1259).
 */
size_t sfm_monarch_workspace_bytes(int B, int H, int D, int n_q, int n_kv,
                                   int f_tied, int h_reduce, int w_reduce, int h, int w,
                                   int num_iters, size_t bridge_budget_bytes);

/*
 * Monarch attention forward over a KV cache that already holds the new chunk.
 *   q        [B, n_q, H, D] natural order (rotated), batch stride q_batch_stride
 *   k_cache, v_cache  [B, n_kv, H, D] Monarch order, batch stride cache_batch_stride
 *   out      [B, n_q, H, D] natural order, contiguous
 *   num_iters  1 = single row/column pass; >1 = alternating updates with the
 *              min(1/(cR+1e-6), 1e4) multiplier of the reference's iterative path
 * Every query group attends every cached group (causality = cache extent).
 * Replaces: _attention_with_cache.forward and its two Triton kernels
 * (wan/modules/monarch_attn.py:1227-1323, 109-253, 698-842), monarch_attn_slow
 * (wan/modules/monarch_attn.py:1705-1751) and return_fn (:1702).
 */
int sfm_monarch_fwd(const void* q, int64_t q_batch_stride,
                    const void* k_cache, const void* v_cache, int64_t cache_batch_stride,
                    void* out, void* workspace, size_t workspace_bytes,
                    int B, int H, int D, int n_q, int n_kv,
                    int f_tied, int h_reduce, int w_reduce, int h, int w,
                    float sm_scale, int num_iters, size_t bridge_budget_bytes, void* stream);

/*
 * sfm_monarch_fwd for callers that cannot give the library a workspace because they are not
 * allowed to allocate device memory at the point of the call: code running inside another
 * framework's memory plan, inside a region where the allocator is frozen, or in a process whose
 * device memory is fully handed out in advance.  It has no counterpart in the reference (whose
 * op allocates its scratch with torch.empty on every call).
 *
 * The scratch is an array of sfm_static_scratch_bytes() bytes (32 MiB) compiled into the
 * library; every GPU context that loads the library carries it until the process exits.  The
 * work is cut into chunks whose row-step results fit the array; a problem in which even one
 * (batch*head, query group) slice does not fit is refused with SFM_ERR_STATIC_SCRATCH and
 * nothing is launched.  At 480p every single-pass (num_iters = 1) Wan shape fits.
 *
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside any stream capture.  No call allocates or frees memory.  All
 * calls on a device share the one array and it keeps the previous call's contents (what must
 * start clean is cleared on the stream first), so two calls whose kernels may overlap on the
 * GPU (different streams without ordering between them) race: order them.
 * Arguments and result are those of sfm_monarch_fwd.
 */
int sfm_monarch_fwd_static(const void* q, int64_t q_batch_stride,
                           const void* k_cache, const void* v_cache, int64_t cache_batch_stride,
                           void* out, int B, int H, int D, int n_q, int n_kv,
                           int f_tied, int h_reduce, int w_reduce, int h, int w,
                           float sm_scale, int num_iters, void* stream);

/* Size in bytes of the scratch array behind sfm_monarch_fwd_static. */
size_t sfm_static_scratch_bytes(void);

/*
 * Waits for the work queued on `stream` and reports whether any kernel of the last
 * sfm_monarch_fwd call that used `workspace` gave up on an internal wait (every device-side
 * wait is bounded): SFM_OK or SFM_ERR_DEVICE_STATUS.  Synchronises the stream; meant for
 * tests and debugging.
 * Replaces: nothing in the reference (its Triton kernels have no device-side status).
 */
int sfm_workspace_status(const void* workspace, void* stream);

/*
 * The same report for the two paths that have no caller workspace.  sfm_static_scratch_status: the last
 * sfm_monarch_fwd_static call on the current device (its status word is the first word of the built-in
 * array).  sfm_dense_status: the dense-attention kernels on the current device; their word is shared by
 * all streams and keeps the first failure since the previous sfm_dense_status call, which clears it.
 * Both synchronise `stream`.
 * Replaces: nothing in the reference.
 */
int sfm_static_scratch_status(void* stream);
int sfm_dense_status(void* stream);

/*
 * Block-causal Monarch attention without a cache: q, k, v [B, N, H, D] natural order,
 * contiguous.  Query groups of causal block c attend the key groups of blocks 0..c;
 * causal_groups = groups per causal block (0 = no mask).  k_mon / v_mon are scratch
 * [B, N, H, D] that receive k, v in Monarch order.
 * Replaces: monarch_attn / _attention_no_cache.forward
 * (wan/modules/monarch_attn.py:1753-1776, 1472-1563).
 */
int sfm_monarch_nocache_fwd(const void* q, const void* k, const void* v,
                            void* k_mon, void* v_mon, void* out,
                            void* workspace, size_t workspace_bytes,
                            int B, int H, int D, int N,
                            int f_tied, int h_reduce, int w_reduce, int h, int w,
                            float sm_scale, int causal_groups, int num_iters,
                            size_t bridge_budget_bytes, void* stream);

/*
 * Dense softmax attention, no mask: out = softmax(q k^T * scale) v.
 *   q [B, n_q, H, D] batch stride q_batch_stride; k, v [B, n_kv, H, D] batch stride
 *   kv_batch_stride; out [B, n_q, H, D] contiguous.
 * Replaces: attention / flash_attention (wan/modules/attention.py:34-187) as called
 * for the dense-init chunk and the regular configuration
 * (wan/modules/causal_model.py:963-967).
 */
int sfm_dense_fwd(const void* q, int64_t q_batch_stride,
                  const void* k, const void* v, int64_t kv_batch_stride,
                  void* out, int B, int H, int D, int n_q, int n_kv,
                  float sm_scale, void* stream);

/*
 * sfm_rope_cache_write with the full-width RMS normalisation of q and k in front, in the same
 * pass: per token, x <- bf16(bf16(x * rsqrt(mean(x^2 over all H*D elements) + eps)) * weight),
 * for q with norm_q_weight and for k with norm_k_weight (bf16 [H*D] each), then the rotation,
 * the layout and the cache write as in sfm_rope_cache_write.  v is not normalised.  q is required.
 * Replaces: norm_q / norm_k of qkv_fn (wan/modules/causal_model.py:801-807; WanRMSNorm,
 * wan/modules/model.py:462-478) in front of causal_rope_apply and the cache write.
 */
int sfm_norm_rope_cache_write(const void* q, const void* k, const void* v,
                              const void* norm_q_weight, const void* norm_k_weight, float eps,
                              void* q_out, void* k_cache, void* v_cache,
                              int64_t cache_batch_stride, const float* rope,
                              int B, int n_new, int H, int D, int start_idx,
                              int f_tied, int h_reduce, int w_reduce, int h, int w,
                              int start_frame, int monarch_order, void* stream);

/*
 * sfm_norm_rope_cache_write (the norm weights may both be null: no normalisation) with the sliding
 * window's eviction folded into the same launch: before the new tokens are written at start_idx, the cached
 * tokens of [roll_dst + roll_shift, start_idx + roll_shift) move left by roll_shift positions (in place, no
 * temporary; roll_shift = 0 moves nothing).  Requires roll_dst <= start_idx and roll_shift <= n_new, which
 * hold whenever a full window evicts to make room for a new chunk.  Positions are relative to the cache
 * pointers given; roll_dst may be negative when those point into the middle of the cache buffer.
 * Replaces: the shift of the cache after the sink tokens, done through a cloned slice
 * (wan/modules/causal_model.py:912-926), together with the write that follows it.
 */
int sfm_rope_cache_write_roll(const void* q, const void* k, const void* v,
                              const void* norm_q_weight, const void* norm_k_weight, float eps,
                              void* q_out, void* k_cache, void* v_cache,
                              int64_t cache_batch_stride, const float* rope,
                              int B, int n_new, int H, int D, int start_idx,
                              int roll_dst, int roll_shift,
                              int f_tied, int h_reduce, int w_reduce, int h, int w,
                              int start_frame, int monarch_order, void* stream);

/*
 * Normalisation and rotation of a token SLICE of a chunk, for sequence-parallel callers that hold n_tokens
 * consecutive tokens starting at token0 of the chunk's (frames, h, w) grid: q_out, k_out <- RoPE(RMSNorm(q, k))
 * with each token's true grid position, v_out <- v, all [B, n_tokens, H, D] in natural order (the outputs may be
 * the buffers another GPU's sfm_rope_cache_write_gather reads, which then runs without a rotation table).
 * The norm weights may both be null (rotation only).
 * Replaces: norm_q / norm_k and causal_rope_apply of the cache branch (wan/modules/causal_model.py:801-807,
 * 902-905) on a token slice; the reference has no sequence-parallel form of this path.
 */
int sfm_norm_rope_token_slice(const void* q, const void* k, const void* v,
                              const void* norm_q_weight, const void* norm_k_weight, float eps,
                              void* q_out, void* k_out, void* v_out, const float* rope,
                              int B, int n_tokens, int H, int D, int token0, int h, int w,
                              int start_frame, void* stream);

/*
 * Head-sharded attention across the GPUs of one box (Ulysses style), with the exchange done by
 * the kernels themselves over peer memory instead of two all-to-all collectives.
 *
 * Outside attention every GPU p of `world` (<= 8) holds a token shard: tokens
 * [p*n/world, (p+1)*n/world) of the chunk with ALL heads, [B, n/world, H*world, D].  Inside
 * attention GPU `rank` works on all tokens of heads [rank*H, (rank+1)*H), H heads, with a KV
 * cache of those heads only.  The shard pointers must be valid on the calling GPU (peer access /
 * symmetric memory); the caller orders the calls against the peers' writes and reads with its
 * own barriers (one before the gather: the shards are complete; one after the scatter: every
 * row has landed).
 *
 *   sfm_rope_cache_write_gather   sfm_rope_cache_write whose q, k, v are read from the
 *                                 token shards q_shards[p], k_shards[p], v_shards[p]
 *                                 (NVLink loads); outputs are local as before
 *   sfm_monarch_fwd_scatter       sfm_monarch_fwd (num_iters = 1) whose result rows go
 *                                 straight to out_shards[t / (n_q/world)] at heads
 *                                 [rank*H, (rank+1)*H) (NVLink stores) instead of a local
 *                                 [B, n_q, H, D] tensor; SFM_ERR_UNSUPPORTED for blockings
 *                                 whose block rows exceed 128
 * No counterpart in the reference: its causal model has no sequence / head parallel path
 * (the only precedent is the all-to-all wrapper for the bidirectional model,
 * wan/distributed/xdit_context_parallel.py:131-184).
 */
int sfm_rope_cache_write_gather(const void* const* q_shards, const void* const* k_shards,
                                const void* const* v_shards, int world, int rank,
                                void* q_out, void* k_cache, void* v_cache,
                                int64_t cache_batch_stride, const float* rope,
                                int B, int n_new, int H, int D, int start_idx,
                                int f_tied, int h_reduce, int w_reduce, int h, int w,
                                int start_frame, int monarch_order, void* stream);
int sfm_monarch_fwd_scatter(const void* q, int64_t q_batch_stride,
                            const void* k_cache, const void* v_cache, int64_t cache_batch_stride,
                            void* const* out_shards, int world, int rank,
                            void* workspace, size_t workspace_bytes,
                            int B, int H, int D, int n_q, int n_kv,
                            int f_tied, int h_reduce, int w_reduce, int h, int w,
                            float sm_scale, size_t bridge_budget_bytes, void* stream);

/*
 * Backward of sfm_monarch_fwd (single pass): gradients of the attention output with respect to
 * q and to the cached keys / values.
 *   q        [B, n_q, H, D] bf16, natural token order, as given to sfm_monarch_fwd (batch stride
 *            q_batch_stride elements)
 *   k_cache, v_cache  [B, n_kv, H, D] bf16 in Monarch block order (batch stride kv_batch_stride)
 *   dout     [B, n_q, H, D] bf16, contiguous, natural order: gradient of the output
 *   dq       [B, n_q, H, D] fp32, contiguous, natural order: written (not accumulated)
 *   dk, dv   [B, (kv_group_end - kv_group_begin) * b1 * b2, H, D] bf16, contiguous, Monarch block
 *            order: gradients of the cached groups kv_group_begin .. kv_group_end - 1 (a group =
 *            b1 * b2 tokens); the whole cache for 0 .. n_kv / (b1 * b2); may be null when the range
 *            is empty.  The range is how grad_only_new_kv is expressed: the groups that the call
 *            wrote.
 *   causal_groups  0, or the block-causal mask of sfm_monarch_nocache_fwd (query group a sees the
 *            cached groups below (a / causal_groups + 1) * causal_groups; needs n_q == n_kv):
 *            the backward of the no-cache call, with k_cache / v_cache = its k_mon / v_mon
 *   workspace  sfm_monarch_bwd_workspace_bytes(...) bytes; the call is cut into slices of
 *            (batch, head) pairs whose scratch stays under budget_bytes (0 = 2 GiB)
 * Nothing has to be saved by the forward call: the backward recomputes the row step (and the column
 * step's softmax statistics) itself, then runs the column-step and the row-step backward; dq, dk and dv
 * are accumulated without atomics (results are run-to-run identical).  Block rows and block columns
 * up to 128.  Without a mask, for block rows up to 96 and block columns up to 64, all of it runs on
 * the tensor cores with aL, Y and their gradients in bf16 (as in the reference); other shapes run
 * fp32 kernels.  The first word of the workspace is the call's status word (sfm_workspace_status).
 * Replaces: _attention_with_cache.backward (wan/modules/monarch_attn.py:1325-1470) and its
 * kernels (:403-596, 1034-1222), and _attention_no_cache.backward (:1565-1694).
 */
size_t sfm_monarch_bwd_workspace_bytes(int B, int H, int D, int n_q, int n_kv,
                                       int f_tied, int h_reduce, int w_reduce, int h, int w,
                                       size_t budget_bytes);
int sfm_monarch_bwd(const void* q, int64_t q_batch_stride,
                    const void* k_cache, const void* v_cache, int64_t kv_batch_stride,
                    const void* dout, void* dq, void* dk, void* dv,
                    void* workspace, size_t workspace_bytes,
                    int B, int H, int D, int n_q, int n_kv,
                    int f_tied, int h_reduce, int w_reduce, int h, int w,
                    float sm_scale, int kv_group_begin, int kv_group_end,
                    int causal_groups, size_t budget_bytes, void* stream);

/*
 * Launch accounting and optional per-kernel timing.  Kernel classes: 0 layout / RoPE /
 * cache write, 1 Monarch row step, 2 Monarch column step, 3 Monarch iteration update,
 * 4 dense attention, 5 Monarch backward (SFM_NUM_KERNEL_CLASSES of them).
 *   sfm_launch_count    kernels this library has launched in this process
 *   sfm_profile_enable  when on, each launch is bracketed by CUDA events on its stream
 *   sfm_profile_read    waits for the recorded events, returns per-class total milliseconds
 *                       and launch counts since the previous read, and forgets them
 * Replaces: the CUDA-event profiling of CausalInferencePipeline.inference(profile=True)
 * (pipeline/causal_inference.py:104-115, 247-281), at kernel granularity.
 */
#define SFM_NUM_KERNEL_CLASSES 6
long long sfm_launch_count(void);
int sfm_profile_enable(int on);
int sfm_profile_read(float* ms, long long* launches, int n_classes);

/*
 * Diagnostic (no counterpart in the reference): store bandwidth between the CTAs of a thread-block
 * cluster through distributed shared memory, the traffic pattern of an on-chip hand-off between the row
 * step and the column step.  `cluster` CTAs per cluster (1, 2, 4, 8, 16), one CTA per SM, `iters` passes of
 * 64 KB per CTA; pattern 0 = one 256-byte row per lane written in 32-byte pieces, 1 = coalesced 16-byte
 * stores; remote 0 = own shared memory, 1 = the peers'.  Plain stores to cluster-mapped addresses only.
 * Returns elapsed milliseconds, CTAs launched and bytes stored.
 */
int sfm_probe_dsmem_store(int cluster, int pattern, int remote, int iters, float* ms, int* ctas, double* bytes);

/*
 * Self-test of the failure path (no counterpart in the reference, whose kernels have no device-side waits): one
 * small CTA allocates tensor memory as the attention kernels do and waits, for `polls` polls (1 .. 65536), on an
 * mbarrier nothing arrives at.  The wait runs out, the kernel stores `code` (1 .. 255) in the status word at the
 * start of `workspace` (cleared first), releases its tensor memory and returns; sfm_workspace_status(workspace,
 * stream) then reports SFM_ERR_DEVICE_STATUS and the context stays usable.  Nothing faults or traps.
 */
int sfm_selftest_bounded_wait(void* workspace, int polls, int code, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SFMONARCH_H_ */
