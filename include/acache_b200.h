/*
 * acache_b200 - C ABI of the B200 (sm_100a) affix-KV-reuse kernels.
 *
 * The reference engine has no FFI: its operator boundary is a set of Python
 * callables backed by Triton kernels and eager PyTorch ops.  Each entry point
 * below replaces one of them and cites it (paths are relative to the reference
 * repository).  All pointers are device pointers unless stated otherwise, all
 * tensors are borrowed for the duration of the call, nothing is retained, and no
 * entry point allocates device memory unless its comment says so.  `stream` is a
 * cudaStream_t passed as void* (NULL = default stream); work is enqueued, not
 * synchronised.  Return value: 0 on success, a negative ACACHE_E* code otherwise
 * (acache_status_string gives the text).  No entry point has a CPU fallback.
 */
#ifndef ACACHE_B200_H
#define ACACHE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ACACHE_API __attribute__((visibility("default")))
#else
#define ACACHE_API
#endif

#define ACACHE_OK 0
#define ACACHE_EINVAL (-1)      /* bad argument (shape, dtype, alignment)            */
#define ACACHE_EUNSUPPORTED (-2)/* valid request this build has no kernel for        */
#define ACACHE_ECUDA (-3)       /* a CUDA call failed; see acache_last_cuda_error()  */
#define ACACHE_ELIMIT (-4)      /* size beyond a documented fixed limit              */
#define ACACHE_ETIMEOUT (-5)    /* a bounded device-side wait gave up                */

/* element types of K/V/Q tensors and RoPE tables */
#define ACACHE_F32 0
#define ACACHE_F16 1
#define ACACHE_BF16 2

ACACHE_API const char* acache_status_string(int status);
/* text of the last CUDA error seen by this library on the calling thread */
ACACHE_API const char* acache_last_cuda_error(void);
/* ABI version, bumped on any signature change */
ACACHE_API int acache_abi_version(void);

/* ------------------------------------------------------------------ K/V scatter
 * Replaces store_kvcache (nano-vdllm/model/attention.py:11-41).
 * key/value: [n_tokens, row_elems] rows `key_stride`/`value_stride` elements apart
 * (row_elems = n_kv_heads*head_dim, contiguous inside a row).  Caches are addressed
 * flat: row `slot` starts at slot*row_elems.  slot == -1 skips the token; any other
 * slot outside [0, num_slots) is an error that the kernel reports by skipping the
 * row and raising the flag *err_flag (device int32, may be NULL). */
ACACHE_API int acache_store_kvcache(const void* key, int64_t key_stride, const void* value, int64_t value_stride,
                         void* k_cache, void* v_cache, const int32_t* slot_mapping, int n_tokens,
                         int row_elems, int64_t num_slots, int dtype, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ affix relocation
 * Replaces materialize_relocated_affix (nano-vdllm/model/acache_attention.py:7-128;
 * caller nano-vdllm/model_runner.py:314-341): for every layer l, affix token t, kv head h
 *   K[l, dst(t), h, :] = K[l, t, h, :]*cos[shift] + rotate_half(K[l, t, h, :])*sin[shift]
 *   V[l, dst(t), h, :] = V[l, t, h, :]
 * in ONE launch for all layers and all requests.  k_cache/v_cache: layer l starts at
 * l*layer_stride elements, slot s at s*n_kv_heads*head_dim inside a layer; the source
 * is slots 0..affix_len-1.  Arithmetic is in promote(dtype, rope_dtype) with one
 * rounding per operation (no FMA contraction), result cast to `dtype`.
 * Request r is relocated by shifts[r] (row of the RoPE tables) to
 *   dst(t) = dst_block_tables ? dst_block_tables[r*table_stride + t/block_size]*block_size + t%block_size
 *                             : dst_slots[r] + t.
 * The single-request reference call is n_requests = 1, dst_block_tables = NULL.
 * shifts, dst_slots, dst_block_tables are device int32 arrays.  Source and
 * destination slots must not overlap. */
ACACHE_API int acache_relocate_affix(void* k_cache, void* v_cache, int64_t layer_stride, int n_layers, int64_t num_slots,
                          int n_kv_heads, int head_dim, int dtype, const void* rope_cos, const void* rope_sin,
                          int64_t rope_row_stride, int rope_rows, int rope_dtype, int affix_len, int n_requests,
                          const int32_t* shifts, const int32_t* dst_slots, const int32_t* dst_block_tables,
                          int table_stride, int block_size, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ RoPE + K/V scatter
 * Replaces RotaryEmbedding.forward (nano-vdllm/model/modeling_llada.py:412-453; Dream:
 * nano-vdllm/model/modeling_dream.py:159-170,472-476) followed by store_kvcache
 * (nano-vdllm/model/attention.py:34-41) for the rows of one forward:
 *   q[i], k[i] rotated in place by table row positions[i]; rotated k[i] and v[i]
 *   scattered to slot_mapping[i] (skipped if slot_mapping is NULL or the slot is -1).
 * q: [n, n_heads, head_dim] rows q_stride elements apart; k/v: [n, n_kv_heads, head_dim]
 * rows k_stride/v_stride apart.  Arithmetic as in acache_relocate_affix:
 * rope_dtype == ACACHE_F32 gives the LLaDA flow (fp32 math, one cast), a table of the
 * activation dtype gives the Dream flow (every product and sum rounded to it). */
ACACHE_API int acache_rope_store(void* q, int64_t q_stride, void* k, int64_t k_stride, const void* v, int64_t v_stride,
                      int n_tokens, int n_heads, int n_kv_heads, int head_dim, int dtype,
                      const int64_t* positions, const void* rope_cos, const void* rope_sin,
                      int64_t rope_row_stride, int rope_rows, int rope_dtype, void* k_cache, void* v_cache,
                      const int32_t* slot_mapping, int64_t num_slots, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ fused QKV projection
 * Replaces, for the rows of one forward, the three projections q_proj / k_proj / v_proj
 * (nano-vdllm/model/modeling_llada.py:687-704,738; Dream with bias: modeling_dream.py:351-354,
 * 452-454), the rotary embedding (modeling_llada.py:412-453) and store_kvcache
 * (model/attention.py:34-41) by ONE tcgen05 GEMM with a fused epilogue:
 *   [q | k | v] = x[n_rows, hidden] . w_qkv[(n_heads + 2 n_kv_heads) * head_dim, hidden]^T (+ bias)
 *   q, k rotated by table row positions[i]; q -> out_q[i, :] (rows q_stride apart);
 *   rotated k and v -> caches at slot_mapping[i] (-1 skips the row's k/v).
 * Each head's projection is rounded to `dtype` before the rotation, as an unfused GEMM would
 * leave it.  16-bit dtypes, head_dim 128, hidden a multiple of 64, 16-byte aligned rows; anything
 * else returns ACACHE_EUNSUPPORTED (use the library GEMM + acache_rope_store then). */
ACACHE_API int acache_qkv_rope_scatter(const void* x, int64_t x_stride, int n_rows, int hidden, const void* w_qkv,
                                       const void* bias, int n_heads, int n_kv_heads, int head_dim, int dtype,
                                       const int64_t* positions, const void* rope_cos, const void* rope_sin,
                                       int64_t rope_row_stride, int rope_rows, int rope_dtype, void* out_q,
                                       int64_t q_stride, void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                       int64_t num_slots, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ dense projections (CTA-pair tcgen05 GEMMs)
 * Replace the nn.Linear calls of the served model blocks (LLaDA: attn_out, ff_proj / up_proj, ff_out
 * and the output head, nano-vdllm/model/modeling_llada.py:687-704,738,757-763,978; Dream: o_proj,
 * gate_proj / up_proj, down_proj and lm_head, modeling_dream.py:297-303,351-354,880) together with
 * the elementwise work that follows each of them.  All compute
 *   acc[n_rows, N] = x[n_rows, in_features] . weight[N, in_features]^T   (fp32 accumulation)
 * on pairs of CTAs with tcgen05.mma.cta_group::2; x rows are x_stride elements apart, weight is
 * row-major and dense.  16-bit dtypes only, N a multiple of 16, in_features a multiple of 8,
 * 16-byte aligned pointers and row strides; anything else returns ACACHE_EUNSUPPORTED.
 * tile_mb (0, 1 or 2) and tile_bn (0 or a multiple of 16 in 64..256) override the tile shape
 * the launch would choose (256 * tile_mb rows by tile_bn columns per CTA pair); 0 = choose.
 *
 * acache_linear: out[n_rows, out_features] = acc (+ bias), rounded once to dtype.  */
ACACHE_API int acache_linear(const void* x, int64_t x_stride, int n_rows, int in_features, const void* weight,
                             int out_features, const void* bias, int dtype, void* out, int64_t out_stride,
                             int tile_mb, int tile_bn, int32_t* err_flag, void* stream);

/* The same projection (no bias) for shapes with so few 256-column output tiles that whole tiles
 * would leave most CTA pairs idle (the attention-output and feed-forward-output projections of a
 * block-decode step, modeling_llada.py:738,763; modeling_dream.py:303,354): the in_features range
 * is cut into n_splits slices, every (tile, slice) runs on a pair of its own and leaves its fp32
 * sums in partials[slice][n_rows][out_features] (dense).  acache_add_rmsnorm_partials consumes
 * them.  acache_linear_partials_splits returns the slice count the launch would choose for a shape
 * (1 = slicing does not pay, use acache_linear); n_splits = 0 asks for that count, and a count
 * that would leave a slice without a 64-wide k block returns ACACHE_EINVAL. */
ACACHE_API int acache_linear_partials_splits(int n_rows, int in_features, int out_features);
ACACHE_API int acache_linear_partials(const void* x, int64_t x_stride, int n_rows, int in_features, const void* weight,
                                      int out_features, int dtype, float* partials, int n_splits, int tile_mb,
                                      int tile_bn, int32_t* err_flag, void* stream);

/* acache_linear_swiglu: the gate and up projections and act(gate) * up (modeling_llada.py:757-763,
 * modeling_dream.py:297-303) in one GEMM.  weight_gate_up is [2 * ffn_features, in_features] with the
 * two projections interleaved in groups of 8 rows: rows 16g..16g+7 are gate rows 8g..8g+7, rows
 * 16g+8..16g+15 are up rows 8g..8g+7.  out[n_rows, ffn_features]; act: 0 silu, 1 relu, 2 gelu.
 * Both projections are rounded to dtype, then the activation, then the product, as the separate
 * operators do. */
ACACHE_API int acache_linear_swiglu(const void* x, int64_t x_stride, int n_rows, int in_features,
                                    const void* weight_gate_up, int ffn_features, int act, int dtype, void* out,
                                    int64_t out_stride, int tile_mb, int tile_bn, int32_t* err_flag, void* stream);

/* acache_linear_qkv_rope_scatter: acache_qkv_rope_scatter on CTA pairs.  The rows of w_qkv (and the
 * entries of bias) are interleaved inside every 128-row head in groups of 8: rows 16g..16g+7 of a head
 * are its features 8g..8g+7, rows 16g+8..16g+15 its features 64+8g..64+8g+7, so that both halves of
 * a rotation pair reach the same thread.  Outputs are in the natural feature order. */
ACACHE_API int acache_linear_qkv_rope_scatter(const void* x, int64_t x_stride, int n_rows, int hidden,
                                              const void* w_qkv_interleaved, const void* bias_interleaved, int n_heads,
                                              int n_kv_heads, int head_dim, int dtype, const int64_t* positions,
                                              const void* rope_cos, const void* rope_sin, int64_t rope_row_stride,
                                              int rope_rows, int rope_dtype, void* out_q, int64_t q_stride,
                                              void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                              int64_t num_slots, int tile_mb, int tile_bn, int32_t* err_flag,
                                              void* stream);

/* acache_linear_argmax: the output head followed by the statistics greedy unmasking needs
 * (modeling_llada.py:978 + model_runner.py:2279-2296): per row the arg-max of the logits (rounded
 * to dtype as the projection leaves them; the lowest index among equal maxima) as int64 x0[n_rows]
 * and confidence[n_rows] = exp(max - logsumexp) in fp32.  The logits are never written to global
 * memory.  scratch must hold acache_linear_argmax_scratch_bytes() bytes. */
ACACHE_API int64_t acache_linear_argmax_scratch_bytes(int n_rows, int out_features);
ACACHE_API int acache_linear_argmax(const void* x, int64_t x_stride, int n_rows, int in_features, const void* weight,
                                    int out_features, int dtype, int64_t* x0, float* confidence, void* scratch,
                                    int64_t scratch_bytes, int tile_mb, int tile_bn, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ anchor top-k
 * Replaces torch.topk + sort + add in anchor selection (nano-vdllm/model_runner.py:833-843;
 * llada/generate_ACache.py:225-262).  scores: fp32 [n_rows, row_stride] (first n_cols of
 * a row are used).  Writes, per row, the k selected column indices in ascending order plus
 * offsets[row] (offsets may be NULL) as int64 into out[row*k ...].  largest != 0 selects
 * the k largest scores, else the k smallest; among equal scores the lowest index wins;
 * NaN orders above +inf.  k is clamped to n_cols. */
ACACHE_API int acache_anchor_topk(const float* scores, int n_rows, int n_cols, int64_t row_stride, int k, int largest,
                       const int32_t* offsets, int64_t* out, void* stream);

/* ------------------------------------------------------------------ anchor influence score
 * Replaces the eager code patched into Attention.forward during the anchor-selection
 * probe (nano-vdllm/model_runner.py:730-773; HF: llada/generate_ACache.py:139-183) for one
 * layer and one request:
 *   K' = rotate(affix K rows 0..affix_len-1 of the layer's cache, by table row affix_shift)
 *   W  = softmax_over_affix( q[rows] K'^T * scale )      (GQA: head h reads kv head h/group)
 *   importance[a] += sum_heads sum_rows W[h, row, a]      (fp32, accumulated in place)
 * q: [*, n_heads, head_dim] post-RoPE, rows q_stride apart; q_rows: device int32[n_q_rows]
 * row indices (the mask-token rows).  Deterministic: per-CTA partial sums go to `scratch`
 * and are reduced in a fixed order.  scratch must hold acache_anchor_importance_scratch_bytes()
 * bytes; contents on entry are irrelevant.  err_flag (device int32, may be NULL) receives a
 * non-zero code when a wait inside the tensor-core kernel ran out (5) or its shared memory
 * was misplaced (6); the scores are then not valid. */
ACACHE_API int64_t acache_anchor_importance_scratch_bytes(int n_q_rows, int n_heads, int affix_len);
ACACHE_API int acache_anchor_importance(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q_rows, int n_heads,
                             int n_kv_heads, int head_dim, int dtype, const void* affix_k, int64_t k_slot_stride,
                             int affix_len, int affix_shift, const void* rope_cos, const void* rope_sin,
                             int64_t rope_row_stride, int rope_rows, int rope_dtype, float scale,
                             float* importance, void* scratch, int64_t scratch_bytes, int32_t* err_flag,
                             void* stream);

/* One layer's influence scores of ALL requests of a probe batch in one launch (the reference runs
 * the probe per request, nano-vdllm/model_runner.py:862-907; a batch of newly admitted requests
 * shares one ragged forward here).  Request r owns the mask rows
 * q_rows[q_row_offsets[r] .. q_row_offsets[r + 1]) (device int32[n_requests + 1]; at most
 * max_q_rows of them), the rotation row affix_shifts[r] (device int32[n_requests]; NULL = no
 * rotation) and the scores importance[r * importance_stride ...].  Every request's result has the
 * bits of its own acache_anchor_importance call.  Tensor-core shapes only (16-bit dtype, head_dim
 * 64 or 128, affix_len at most 2048): anything else returns ACACHE_EUNSUPPORTED and the caller
 * loops over the requests.  An affix_shifts entry outside the table raises err_flag code 4 and is
 * treated as 0. */
ACACHE_API int64_t acache_anchor_importance_batched_scratch_bytes(int n_requests, int max_q_rows, int n_heads,
                                                                  int affix_len);
ACACHE_API int acache_anchor_importance_batched(const void* q, int64_t q_stride, const int32_t* q_rows,
                                                const int32_t* q_row_offsets, int n_requests, int max_q_rows,
                                                int n_heads, int n_kv_heads, int head_dim, int dtype,
                                                const void* affix_k, int64_t k_slot_stride, int affix_len,
                                                const int32_t* affix_shifts, const void* rope_cos,
                                                const void* rope_sin, int64_t rope_row_stride, int rope_rows,
                                                int rope_dtype, float scale, float* importance,
                                                int64_t importance_stride, void* scratch, int64_t scratch_bytes,
                                                int32_t* err_flag, void* stream);

/* The same computation for callers that cannot provide scratch memory and must not cause an
 * allocation: hosts that have given the whole device to their own memory arena, plugins that
 * only ever receive their input and output buffers, and latency-critical loops that cannot
 * afford the device-wide synchronisation an allocation implies.  This entry point has no
 * counterpart in the reference.  The partial sums go to a fixed array of
 * acache_anchor_importance_static_scratch_bytes() bytes (8 MiB) that is part of the library
 * image on every GPU that loads it; a request whose
 * acache_anchor_importance_scratch_bytes(n_q_rows, n_heads, affix_len) exceeds that returns
 * ACACHE_ELIMIT and does nothing.  Neither this call nor anything it calls allocates or frees
 * memory.  The first call on a device looks the array's device address up (once per device,
 * for the device current at that time, assuming the device's primary context lives as long as
 * the process); make that first call before any stream capture - a first call on a capturing
 * stream returns ACACHE_EUNSUPPORTED and does nothing.
 * All calls on a device share the one array and it keeps whatever the last call left in it:
 * nothing in it needs clearing between calls (every entry that is read was written by the same
 * call), but two calls whose kernels overlap on the GPU (different streams) race on it -
 * serialise them.  Results are identical to acache_anchor_importance. */
ACACHE_API int64_t acache_anchor_importance_static_scratch_bytes(void);
ACACHE_API int acache_anchor_importance_static(const void* q, int64_t q_stride, const int32_t* q_rows, int n_q_rows,
                                               int n_heads, int n_kv_heads, int head_dim, int dtype,
                                               const void* affix_k, int64_t k_slot_stride, int affix_len,
                                               int affix_shift, const void* rope_cos, const void* rope_sin,
                                               int64_t rope_row_stride, int rope_rows, int rope_dtype, float scale,
                                               float* importance, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ varlen attention, slot map
 * Replaces acache_attention (nano-vdllm/model/acache_attention.py:338-514,643-738):
 * bidirectional attention of ragged queries q[total_q, n_heads, head_dim] (rows q_stride
 * apart) over K/V rows gathered from the flat caches through read_slot_mapping
 * (int32[sum kv_len], request b uses [cu_seqlens_k[b], cu_seqlens_k[b+1])).
 * Relocation modes (all NULL / 0 = none):
 *   key side:   shared_prefix_len > 0, affix_shifts != NULL, shared_kv_lens == NULL:
 *               a key whose slot < shared_prefix_len is rotated by table row
 *               |j - slot| (j = its index in the request), sine negated when j < slot;
 *   query side: additionally shared_kv_lens != NULL: the first shared_kv_lens[b] keys of
 *               request b are scored with q rotated by the inverse of table row
 *               affix_shifts[b]; the remaining keys with q as given.
 * Two extensions over the reference, both neutral for a caller that does not use them:
 *   holes:      an entry of -1 in read_slot_mapping is a key that takes no part (weight 0);
 *               any other entry outside [0, num_slots) is reported through err_flag.  Since
 *               attention does not depend on the order of the keys, a caller may list the
 *               shared span as the consecutive slots it occupies, with -1 where a private
 *               copy (an anchor) replaces the shared row, and append the private slots: all
 *               requests then name the shared span the same way (acache_attention_grouped
 *               builds on that);
 *   run split:  shared_kv_lens != NULL with affix_shifts == NULL only splits the keys of
 *               request b after the first shared_kv_lens[b] entries for tiling (the second
 *               run starts a fresh tile); the result is the same as without it.
 * Output rows have the layout of q (rows o_stride apart).  Requests with kv_len <= 0
 * get zeros.  max_seqlen_q / max_seqlen_k are host-known upper bounds (no device
 * synchronisation is done to find them). */
ACACHE_API int acache_attention(const void* q, int64_t q_stride, void* out, int64_t o_stride, const void* k_cache,
                     const void* v_cache, int64_t num_slots, int n_heads, int n_kv_heads, int head_dim, int dtype,
                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch, int max_seqlen_q,
                     int max_seqlen_k, const int32_t* read_slot_mapping, float softmax_scale,
                     int shared_prefix_len, const int32_t* shared_kv_lens, const int32_t* affix_shifts,
                     const void* rope_cos, const void* rope_sin, int64_t rope_row_stride, int rope_rows,
                     int rope_dtype, int32_t* err_flag, void* stream);

/* Block-decode form of acache_attention in which one CTA serves two consecutive requests of a
 * KV head: the shared span is staged once for both (no counterpart in the reference, which
 * reads the span per request; same result up to the order of the floating-point sums), then the
 * CTA walks each request's remaining keys.
 * Contract on top of acache_attention's: shared_kv_lens != NULL; within each group of four
 * consecutive requests shared_kv_lens[b] is the same and the first shared_kv_lens[b] entries of
 * read_slot_mapping name the same slots, up to holes (-1); every request has at most
 * 32 / (n_heads / n_kv_heads) queries; no key-side relocation.  A violated contract is reported
 * through err_flag (code 7), never by a fault.  ACACHE_EUNSUPPORTED means "use acache_attention".
 * scratch / scratch_bytes are not used (pass NULL / 0; acache_attention_grouped_scratch_bytes
 * returns 0): nothing is kept between the CTAs of a call or between calls.  total_q = number
 * of query rows (cu_seqlens_q[batch]). */
ACACHE_API int64_t acache_attention_grouped_scratch_bytes(int total_q, int n_heads, int head_dim, int batch,
                                                          int n_kv_heads);
ACACHE_API int acache_attention_grouped(const void* q, int64_t q_stride, void* out, int64_t o_stride,
                             const void* k_cache, const void* v_cache, int64_t num_slots, int n_heads,
                             int n_kv_heads, int head_dim, int dtype, const int32_t* cu_seqlens_q,
                             const int32_t* cu_seqlens_k, int batch, int total_q, int max_seqlen_q,
                             const int32_t* read_slot_mapping, float softmax_scale, int shared_prefix_len,
                             const int32_t* shared_kv_lens, const int32_t* affix_shifts, const void* rope_cos,
                             const void* rope_sin, int64_t rope_row_stride, int rope_rows, int rope_dtype,
                             void* scratch, int64_t scratch_bytes, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ varlen attention, block tables
 * Replaces baseline_ragged_attention and baseline_decode_attention
 * (nano-vdllm/model/acache_attention.py:132-334,525-640): key j of request b lives at
 * slot block_tables[b*table_stride + j/block_size]*block_size + j%block_size.
 * The decode form is cu_seqlens_q = {0, T, 2T, ...}. */
ACACHE_API int acache_paged_attention(const void* q, int64_t q_stride, void* out, int64_t o_stride, const void* k_cache,
                           const void* v_cache, int64_t num_slots, int n_heads, int n_kv_heads, int head_dim,
                           int dtype, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                           int max_seqlen_q, int max_seqlen_k, const int32_t* block_tables, int table_stride,
                           int block_size, float softmax_scale, int32_t* err_flag, void* stream);

/* ------------------------------------------------------------------ small fused ops of the block
 * RMSNorm as the served models compute it (nano-vdllm/model/modeling_llada.py:308-323,
 * nano-vdllm/model/modeling_dream.py:76-81): y = weight * cast(x_f32 * rsqrt(mean(x_f32^2) + eps)). */
ACACHE_API int acache_rmsnorm(const void* x, int64_t x_stride, const void* weight, void* y, int64_t y_stride, int n_rows,
                   int n_cols, float eps, int dtype, void* stream);
/* Residual add fused into the normalisation that follows it (the two eager ops `x = x + delta;
 * h = norm(x)` of nano-vdllm/model/modeling_llada.py:740-752): x (in place) = x + delta rounded to
 * `dtype`, y = RMSNorm(x).  Needs 16-byte aligned rows of at most 1024 vectors, else
 * ACACHE_EUNSUPPORTED. */
ACACHE_API int acache_add_rmsnorm(void* x, int64_t x_stride, const void* delta, int64_t d_stride, const void* weight,
                                  void* y, int64_t y_stride, int n_rows, int n_cols, float eps, int dtype,
                                  void* stream);
/* The same with the update given as the fp32 K-range slices that acache_linear_partials leaves:
 * partials[s][row][col], rows p_stride floats apart, slices split_stride floats apart.  The
 * slices are summed in order and rounded to `dtype` (the projection's output as a GEMM in `dtype`
 * leaves it) before the add. */
ACACHE_API int acache_add_rmsnorm_partials(void* x, int64_t x_stride, const float* partials, int n_splits,
                                           int64_t split_stride, int64_t p_stride, const void* weight, void* y,
                                           int64_t y_stride, int n_rows, int n_cols, float eps, int dtype,
                                           void* stream);
/* y = act(gate) * up, act: 0 = SiLU, 1 = ReLU, 2 = GELU(erf)
 * (nano-vdllm/model/modeling_llada.py:757-763, nano-vdllm/model/modeling_dream.py:297-303). */
ACACHE_API int acache_act_mul(const void* gate, const void* up, void* y, int64_t n, int act, int dtype, void* stream);
/* The same for a gate and an up projection computed by ONE GEMM over the concatenated weights:
 * x[n_rows, 2 * ffn] = [gate | up] (rows x_stride apart), y[n_rows, ffn] = act(gate) * up. */
ACACHE_API int acache_act_mul_halves(const void* x, int64_t x_stride, void* y, int64_t y_stride, int n_rows, int ffn,
                                     int act, int dtype, void* stream);

/* ------------------------------------------------------------------ threshold unmasking
 * Replaces get_transfer_index at temperature 0 with 'low_confidence' remasking
 * (nano-vdllm/model_runner.py:2279-2314) and applies the result:
 * logits [n_rows*block_len, vocab] (rows logits_stride apart, `dtype`); blocks int64
 * [n_rows, block_len] updated in place: masked positions whose confidence
 * exp(max_logit - logsumexp) >= threshold receive argmax(logits); a row that has masks
 * but no position over the threshold commits its most confident masked position.
 * Ties in argmax resolve to the lowest vocabulary index, ties in confidence to the lowest
 * position.  x0_out (int64) and conf_out (fp32), each n_rows*block_len long, are required
 * work space and receive the per-position argmax and confidence. */
ACACHE_API int acache_transfer_tokens(const void* logits, int64_t logits_stride, int vocab, int dtype, int64_t* blocks,
                           int n_rows, int block_len, int64_t mask_id, float threshold, int64_t* x0_out,
                           float* conf_out, void* stream);

/* The commit rule of acache_transfer_tokens alone (model_runner.py:2297-2312), for callers that
 * already hold the per-position statistics (acache_linear_argmax): blocks[n_rows, block_len] is
 * edited in place from x0 / confidence of the same shape. */
ACACHE_API int acache_apply_transfer(int64_t* blocks, const int64_t* x0, const float* confidence, int n_rows,
                                     int block_len, int64_t mask_id, float threshold, void* stream);

/* ------------------------------------------------------------------ diagnostics
 * No counterpart in the reference.  Runs, on every SM (cta_group 1) or every pair of SMs (2), one
 * thread that issues `iters` x `k_steps` x `n_accumulators` tcgen05.mma products of 128 (256 for a
 * pair) rows x n columns x 16 on zeroed shared-memory operands, alternating between
 * `n_accumulators` TMEM accumulators, with a tcgen05.commit every `commit_every` iterations (0 =
 * only at the end), and waits for the last one.  result4 (device, 4 x int64): SM cycles, nanoseconds,
 * products issued, 1 if the final wait completed.  Measures the tensor pipe and its issue path
 * without any memory traffic. */
ACACHE_API int acache_diag_mma_rate(int cta_group, int n, int n_accumulators, int commit_every, int k_steps, int iters,
                                    long long* result4, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ACACHE_B200_H */
