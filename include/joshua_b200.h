/* joshua_b200 - C ABI of the B200 (sm_100a) quantized-matmul library.
 *
 * A drop-in for one path of the joshua inference engine: the fused
 * dequantise-and-dot matmuls over raw GGUF blocks (Q8_0, Q2_K, Q4_K, IQ2_XXS,
 * MXFP4) and the routed-expert gather / grouped matmul / scatter of its MoE
 * loaders.  Every entry point names the reference interface it stands in for
 * (file:line in the reference tree).
 *
 * Conventions (those of the reference's one C ABI, src/npu/mod.rs:32-50):
 * int32 status, 0 = success, negative = failure; opaque handles; `*_free`
 * releases; nothing throws or aborts across the boundary.  After a failure,
 * `jq_last_error()` returns a message for the calling thread.  Handles are
 * immutable after creation and may be used from several threads at once; each
 * host-buffer call takes a private stream and workspace from the context.
 *
 * Matmul contract (src/quant_matmul.rs:105-118): weights are n rows of k
 * columns stored row-major as n*k/B raw blocks in GGUF byte order; `lhs` is
 * f32 [m, k] row-major; `dst` is f32 [m, n] row-major and is ASSIGNED,
 * dst[i*n + j] = sum_c lhs[i*k + c] * W[j, c] (src/mxfp4.rs:185-189).
 *
 * There is no CPU fallback: every compute entry fails with JQ_E_CUDA when no
 * device is usable.
 */
#ifndef JOSHUA_B200_H
#define JOSHUA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct jq_ctx jq_ctx;       /* one device, its streams and workspaces */
typedef struct jq_weight jq_weight; /* raw blocks resident in device memory */
typedef struct jq_moe jq_moe;       /* one MoE layer: router + expert banks */

/* status codes */
#define JQ_OK 0
#define JQ_E_INVALID (-1)      /* shape / length / alignment / NULL argument */
#define JQ_E_TYPE (-2)         /* GGUF type id without a kernel here */
#define JQ_E_CUDA (-3)         /* a CUDA runtime call failed (incl. no device) */
#define JQ_E_NOMEM (-4)        /* device or pinned-host allocation failed */
#define JQ_E_EXPERT_RANGE (-5) /* router produced an expert id >= n_expert */
#define JQ_E_TOO_LARGE (-6)    /* request exceeds a fixed capacity */
#define JQ_E_TIMEOUT (-7)      /* a bounded wait inside a kernel gave up */

/* GGUF tensor type ids (src/gguf_ext.rs:483-512, src/iq2xxs.rs:23, src/mxfp4.rs:39) */
#define JQ_TYPE_Q8_0 8u
#define JQ_TYPE_Q2_K 10u
#define JQ_TYPE_Q4_K 12u
#define JQ_TYPE_IQ2_XXS 16u
#define JQ_TYPE_MXFP4 39u

/* Message of the last failure on the calling thread ("" if none). */
const char* jq_last_error(void);

/* Elements and bytes of one block of `type` (src/kquant_dot.rs:95-104,
 * src/iq2xxs.rs:25-27, src/mxfp4.rs:36,59). */
int32_t jq_block_size(uint32_t type, uint64_t* elems, uint64_t* bytes);

/* ── context ─────────────────────────────────────────────────────────────
 * Stands in for the reference's device selection (src/engine.rs:764-834).
 * Binds to CUDA device `device`, uploads the decode tables. */
int32_t jq_init(int32_t device, jq_ctx** out);
void jq_free(jq_ctx* ctx);

/* Every wait inside a kernel (on a copy in flight) is bounded; a kernel whose
 * wait runs out sets a device-visible flag and returns.  Host-buffer entries
 * check the flag themselves; callers of the *_dev entries poll it here after
 * synchronising their stream.  JQ_OK or JQ_E_TIMEOUT; a reported timeout is
 * cleared, so the next call answers for the work after it.  (The reference's
 * counterpart is the deadline handling of its plugin shim, src/npu/shim.rs:1-8.) */
int32_t jq_device_status(const jq_ctx* ctx);

/* ── weights ─────────────────────────────────────────────────────────────
 * jq_weight_upload replaces the zero-copy borrow of a tensor's byte range
 * from the model mapping (`borrowed_range*` / `borrowed_qtensor*`,
 * src/mmap_tensor.rs:520-655): `bytes` are the tensor's raw GGUF bytes,
 * copied to device memory unmodified.  Fails like `blocks_from_bytes`
 * (src/iq2xxs.rs:422-435, src/mxfp4.rs:265-279, src/kquant_dot.rs:217-220)
 * when `nbytes` is not a whole number of blocks. */
int32_t jq_weight_upload(jq_ctx* ctx, uint32_t type, const void* bytes, uint64_t nbytes, jq_weight** out);

/* Adopt blocks that already sit in device memory (not copied, not freed). */
int32_t jq_weight_from_device(jq_ctx* ctx, uint32_t type, const void* device_bytes, uint64_t nbytes,
                              jq_weight** out);

/* A run of whole blocks [block0, block0 + n_blocks) of `parent`, sharing its
 * memory: the per-expert slicing of a [n_expert, out, in] tensor
 * (`split_experts`, src/quantized_qwen3_moe.rs:556-651,
 * src/quantized_deepseek4.rs:2193-2379).  The parent must outlive the slice. */
int32_t jq_weight_slice(const jq_weight* parent, uint64_t block0, uint64_t n_blocks, jq_weight** out);

void jq_weight_free(jq_weight* w);

/* QuantizedType::{dtype, storage_size_in_bytes, block_size, as_ptr}
 * (src/mmap_tensor.rs:127-188). */
uint32_t jq_weight_type(const jq_weight* w);
uint64_t jq_weight_storage_size(const jq_weight* w);
uint64_t jq_weight_block_elems(const jq_weight* w);
const void* jq_weight_device_ptr(const jq_weight* w);

/* ── the operator: QuantizedType::matmul_t ───────────────────────────────
 * Replaces `impl QuantizedType for MmapBlocks<T>` / MmapBlocksIq2Xxs /
 * MmapBlocksMxfp4 :: matmul_t (src/mmap_tensor.rs:132-134,374-376,447-449),
 * i.e. matmul_kquant (src/quant_matmul.rs:110-118), iq2xxs::matmul_t
 * (src/iq2xxs.rs:103-111), mxfp4::matmul_t (src/mxfp4.rs:120-128).
 * HOST buffers; `lhs_len` / `dst_len` are the slice lengths in elements and
 * are validated as the reference validates them (src/quant_matmul.rs:133-165):
 * k not a block multiple, block count != n*k/B, lhs_len != m*k or
 * dst_len != m*n fail with JQ_E_INVALID; m == 0 or n == 0 is a no-op. */
int32_t jq_matmul_t(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs, uint64_t lhs_len,
                    float* dst, uint64_t dst_len);

/* QuantizedType::matmul_t_f16 (src/iq2xxs.rs:396-412, src/mxfp4.rs:242-258):
 * IEEE binary16 in and out (as uint16 bit patterns), widened to f32, the f32
 * product, rounded back to nearest-even. */
int32_t jq_matmul_t_f16(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const uint16_t* lhs,
                        uint64_t lhs_len, uint16_t* dst, uint64_t dst_len);

/* Same product with DEVICE buffers on a caller stream (cudaStream_t passed as
 * void*), no synchronisation: the device-resident insertion point that
 * `Weight::Zc` / ZcWeight::forward occupies in the reference
 * (src/quantized_qwen3_moe.rs:215-227, src/zero_copy_metal.rs:374-408). */
int32_t jq_matmul_t_dev(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs_dev,
                        float* dst_dev, void* stream);

/* The same product for callers that must not allocate.  It has no counterpart
 * in the reference.  Some hosts hand this library a GPU whose memory is
 * already fully carved up (weights, KV cache, their own pools), or call it from
 * a latency-critical loop where a cudaMalloc - which takes the driver lock and
 * may synchronise the device - is not acceptable.  jq_matmul_t_dev may
 * allocate scratch the first time a stream needs it; this entry never does: it
 * calls no cudaMalloc, cudaFree or other allocating routine.  The activation
 * planes it needs between its two kernels live in a 4 MiB array that is part of
 * the library image (every GPU that loads the library holds those 4 MiB until
 * the process exits).
 *   Limits: 1 <= m <= 8, k a multiple of 256, and m * (k/32) * 112 + 256 bytes
 *   must fit the 4 MiB array (about m*k <= 1.19 million activations); beyond
 *   that it fails with JQ_E_TOO_LARGE and touches nothing.
 *   The first call on a device looks up the array's device address and sets
 *   kernel attributes; make that call before capturing a stream.
 *   All calls on a device share the array and it is not cleared between
 *   calls (each call rewrites what it reads).  Calls whose kernels overlap on
 *   the GPU - different streams, or two host threads - race on it: keep them on
 *   one stream or serialise them.  Inputs and outputs are the caller's. */
int32_t jq_matmul_t_dev_noalloc(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs_dev,
                                float* dst_dev, void* stream);

/* QuantizedType::dequantize (src/mmap_tensor.rs:169-174) and
 * decode_raw_to_f32 (src/quant_matmul.rs:36-103): all blocks to f32.
 * `two_step` != 0 gives the separately rounded k-quant form fl(fl(d*sc*)q)-m
 * of a plain `d1 * q - m1` (what `to_float` returns); 0 gives the single fused
 * multiply-subtract the matmul kernels form (src/kquant_dot.rs:256-260).  The
 * two differ by at most one ulp; other types have one form. */
int32_t jq_dequantize(const jq_weight* w, float* out, uint64_t elem_count, int32_t two_step);
int32_t jq_dequantize_dev(const jq_weight* w, float* out_dev, uint64_t elem_count, int32_t two_step, void* stream);

/* QuantizedType::embedding (src/mmap_tensor.rs:140-167): out[i, :] = row
 * ids[i] of a [rows, hidden] tensor, decoded.  Fails with JQ_E_INVALID when
 * hidden is not a block multiple, the block count is not rows*hidden/B, or an
 * id is >= rows. */
int32_t jq_embedding(const jq_weight* w, const uint32_t* ids, uint64_t n_ids, uint64_t rows, uint64_t hidden,
                     float* out);

/* QuantizedType::from_float / from_float_imatrix (src/mmap_tensor.rs:190-203):
 * borrowed tensors are read-only; always fails with JQ_E_INVALID. */
int32_t jq_weight_from_float(jq_weight* w, const float* xs, uint64_t len);

/* ── around the matmuls: the rest of a decode step, on the device ───────
 * The callers on either side of the matmul path.  In the reference they are
 * candle tensor ops inside the loaders; here they are kernels so that a token
 * does not leave the device between two quantized matmuls.  All f32, all on a
 * caller stream without synchronisation. */

/* `Mlp::forward` up to the down projection: dst = silu(gate x) * up x, with the
 * optional clamp of src/quantized_deepseek4.rs:445-462 (clamp <= 0: none)
 * (src/quantized_qwen3_moe.rs:396-402).  One launch for batches of 1..8. */
int32_t jq_matmul_swiglu_dev(const jq_weight* gate, const jq_weight* up, uint64_t m, uint64_t k, uint64_t n,
                             const float* lhs_dev, float* dst_dev, float clamp, void* stream);

/* QuantizedType::embedding with device ids (src/mmap_tensor.rs:140-167); an id
 * >= rows sets *bad_id_dev to 1 and leaves that row untouched. */
int32_t jq_embedding_dev(const jq_weight* w, const uint32_t* ids_dev, uint64_t n_ids, uint64_t rows, uint64_t hidden,
                         float* out_dev, int32_t* bad_id_dev, void* stream);

/* RmsNorm (src/quantized_qwen3_moe.rs:532-553): out = (x [+ residual]) /
 * sqrt(mean(.^2) + eps) * weight.  With `residual`, the sum is also written to
 * sum_out (the new residual stream).  weight may be NULL (ones). */
int32_t jq_rmsnorm_dev(const float* x, const float* residual, const float* weight, float eps, uint64_t rows,
                       uint64_t hidden, float* sum_out, float* out, void* stream);

/* The same with the RMS norm of the block folded in: dst = silu(gate xn) * up xn
 * with xn = rmsnorm(lhs; norm_w, eps) computed inside the matmul kernel. */
int32_t jq_matmul_swiglu_norm_dev(const jq_weight* gate, const jq_weight* up, uint64_t m, uint64_t k, uint64_t n,
                                  const float* lhs_dev, const float* norm_w_dev, float eps, float* dst_dev,
                                  float clamp, void* stream);

/* dst = residual + rmsnorm(lhs; norm_w, eps) . W^T: a quantized linear with the
 * RMS norm in front of it and the residual add behind it in the same launch
 * (the `RmsNorm` -> `QMatMul::forward` -> `xs + residual` pattern of
 * src/quantized_qwen3_moe.rs:793-819).  norm_w_dev and residual_dev are each
 * optional; residual_dev may be dst_dev.  One launch when m <= 8 and the
 * activation planes fit shared memory, otherwise the separate kernels. */
int32_t jq_matmul_norm_dev(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs_dev,
                           const float* norm_w_dev, float eps, const float* residual_dev, float* dst_dev,
                           void* stream);

/* Rotary embedding of q and k (pairing element i with i + head_dim/2) at
 * position pos[b], then k and v appended to the cache: the rope + `Tensor::cat`
 * of src/quantized_qwen3_moe.rs:330-364.  qkv: [batch, (n_q + 2 n_kv) *
 * head_dim]; cache_k, cache_v: [batch, n_kv, max_ctx, head_dim].  The cache
 * holds max_ctx positions (the reference stops generating at n_ctx,
 * src/engine.rs:1246-1249): a sequence whose pos[b] is negative or >= max_ctx
 * stores nothing and sets *bad_pos_dev (device int32, may be NULL) to 1. */
int32_t jq_rope_append_dev(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t n_q, uint32_t n_kv,
                           uint32_t head_dim, uint32_t max_ctx, float theta, float* q_out, float* cache_k,
                           float* cache_v, int32_t* bad_pos_dev, void* stream);

/* Rope, cache append and attention in ONE launch, straight from the fused qkv
 * row: out[b, head, :] as jq_rope_append_dev + jq_attention_decode_dev give it.
 * `scratch`: jq_attention_fused_scratch_bytes(...) bytes of caller device
 * memory, ZEROED once before the first call (it holds arrival counters that
 * the kernel leaves at zero).  head_dim 64, 128 or 256; n_q / n_kv 1, 2, 4 or 8.
 * A sequence whose pos[b] lies outside [0, max_ctx) is skipped entirely - no
 * cache store, its rows of `out` untouched - and *bad_pos_dev (may be NULL) is
 * set to 1. */
uint64_t jq_attention_fused_scratch_bytes(uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim,
                                          uint32_t max_ctx);
int32_t jq_attention_fused_dev(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t n_q, uint32_t n_kv,
                               uint32_t head_dim, uint32_t max_ctx, float theta, float* cache_k, float* cache_v,
                               float* out, void* scratch, int32_t* bad_pos_dev, void* stream);

/* The same with the per-head RMS norm of q and k in front of the rotary embedding (Qwen3's `attn_q_norm` /
 * `attn_k_norm`, [head_dim] each, src/quantized_qwen3_moe.rs:343-353).  Both NULL = jq_attention_fused_dev. */
int32_t jq_attention_fused_qknorm_dev(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t n_q, uint32_t n_kv,
                                      uint32_t head_dim, uint32_t max_ctx, float theta, const float* q_norm_w,
                                      const float* k_norm_w, float qk_eps, float* cache_k, float* cache_v, float* out,
                                      void* scratch, int32_t* bad_pos_dev, void* stream);

/* Prefill: `seq` new tokens of ONE sequence at positions pos0[0] .. pos0[0] + seq - 1 (the reference's
 * `forward(input [1, seq_len], offset)`, src/quantized_qwen3_moe.rs:297-386,793-819).
 * jq_rope_append_prefill_dev: qkv [seq, (n_q + 2 n_kv) * head_dim] -> q_out [seq, n_q * head_dim] rotated (after the
 * optional per-head q / k norm), k and v appended to the cache of sequence 0 ([n_kv, max_ctx, head_dim]).
 * jq_attention_prefill_dev: out[s] = attention of token s over cache positions 0 .. pos0 + s (causal); head_dim 64
 * or 128.  Tokens that would run past max_ctx store nothing / the whole call does nothing, and *bad_pos_dev is set. */
int32_t jq_rope_append_prefill_dev(const float* qkv, const int32_t* pos0, uint32_t seq, uint32_t n_q, uint32_t n_kv,
                                   uint32_t head_dim, uint32_t max_ctx, float theta, const float* q_norm_w,
                                   const float* k_norm_w, float qk_eps, float* q_out, float* cache_k, float* cache_v,
                                   int32_t* bad_pos_dev, void* stream);
int32_t jq_attention_prefill_dev(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos0,
                                 uint32_t seq, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_ctx,
                                 float* out, int32_t* bad_pos_dev, void* stream);

/* RmsNorm over the first `hidden` columns of rows that are x_stride floats apart (the latent part of the
 * compressed kv row, `kv_a_norm`, src/quantized_deepseek2.rs:462-466); out rows are `hidden` wide. */
int32_t jq_rmsnorm_strided_dev(const float* x, uint64_t x_stride, const float* weight, float eps, uint64_t rows,
                               uint64_t hidden, float* out, void* stream);

/* Multi-head latent attention, one new token per sequence (`Attention::forward` of src/quantized_deepseek2.rs:422-504
 * between its projections and its attention): interleaved rotary embedding (pairs 2i, 2i + 1; angle
 * pos * inv_freq[i]; cos and sin times `mscale`, the YaRN table of :243-300) of the last qk_rope columns of every
 * q head (in place) and of the shared key k_pe = comp[kv_lora ..], then the per-head rows
 * K[pos] = [k_nope | k_pe] and V[pos] = v are appended to the caches, which hold the reconstructed per-head form
 * as the reference's does (:389-401).  q [batch, n_head * (qk_nope + qk_rope)]; comp [batch, kv_lora + qk_rope];
 * kv [batch, n_head * (qk_nope + v_dim)]; cache_k [batch, n_head, max_ctx, qk_nope + qk_rope]; cache_v
 * [batch, n_head, max_ctx, v_dim]. */
int32_t jq_mla_assemble_dev(float* q, const float* comp, const float* kv, const int32_t* pos, uint32_t batch,
                            uint32_t n_head, uint32_t qk_nope, uint32_t qk_rope, uint32_t v_dim, uint32_t kv_lora,
                            uint32_t max_ctx, const float* inv_freq_dev, float mscale, float* cache_k, float* cache_v,
                            int32_t* bad_pos_dev, void* stream);

/* jq_attention_decode_dev with key rows of qk_dim and value rows of v_dim floats and an explicit softmax scale
 * (MLA: 192 / 128, scale 1 / sqrt(192) times the YaRN factor).  scratch: jq_attention_scratch_bytes(batch, n_q,
 * v_dim, max_ctx). */
int32_t jq_attention_decode_qkv_dev(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                    uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t qk_dim, uint32_t v_dim,
                                    uint32_t max_ctx, float softmax_scale, float* out, float* scratch,
                                    int32_t* bad_pos_dev, void* stream);

/* out = silu(min(gate, clamp)) * clamp(up) element-wise (`Mlp::forward` between its matmuls for batches the fused
 * gate / up kernel does not take; clamp <= 0: none). */
int32_t jq_swiglu_dev(const float* gate, const float* up, uint64_t n, float clamp, float* out, void* stream);

/* Grouped-query attention of one new token per sequence over positions
 * 0..pos[b] of the cache (src/quantized_qwen3_moe.rs:366-386).  `scratch`:
 * jq_attention_scratch_bytes(...) bytes of caller device memory (per-chunk
 * partial results, merged in position order).  pos[b] outside [0, max_ctx)
 * reads nothing, gives NaN rows and sets *bad_pos_dev (may be NULL). */
uint64_t jq_attention_scratch_bytes(uint32_t batch, uint32_t n_q, uint32_t head_dim, uint32_t max_ctx);
int32_t jq_attention_decode_dev(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_ctx,
                                float* out, float* scratch, int32_t* bad_pos_dev, void* stream);

int32_t jq_add_dev(const float* a, const float* b, uint64_t n, float* y, void* stream);

/* Greedy sampling (src/engine.rs:2371-2378): arg-max of each row, the LAST
 * maximal index winning ties; pos (may be NULL) is advanced by one per row.
 * `scratch`: jq_argmax_scratch_bytes(rows) bytes of caller device memory. */
uint64_t jq_argmax_scratch_bytes(uint64_t rows);
int32_t jq_argmax_dev(const float* logits, uint64_t rows, uint64_t vocab, int32_t* token, int32_t* pos, void* scratch,
                      void* stream);

/* The reference's greedy sampler with its repetition penalty (sample_token,
 * src/engine.rs:2339-2378; default penalty 1.1): for every occurrence of a
 * token id in the recent window its logit is divided by the penalty when
 * positive and multiplied by it otherwise, then the arg-max (last maximal index)
 * is taken, and the sampled id is pushed into the window, which holds the last
 * JQ_SAMPLE_WINDOW ids (src/engine.rs:1222-1232,1265-1269).  `logits` is left
 * as it was.  window: device int32 [rows, JQ_SAMPLE_WINDOW]; window_state:
 * device int32 [rows, 2] = {ids held, slot the next id goes to}; seed both
 * with the tail of the prompt, or zero them.  window and window_state NULL =
 * jq_argmax_dev.  `scratch` as for jq_argmax_dev. */
#define JQ_SAMPLE_WINDOW 64
int32_t jq_sample_greedy_dev(const float* logits, uint64_t rows, uint64_t vocab, float repetition_penalty,
                             int32_t* window, int32_t* window_state, int32_t* token, int32_t* pos, void* scratch,
                             void* stream);

/* ── MoE layer ───────────────────────────────────────────────────────────
 * Replaces `Moe::forward` of the three loaders: routing, per-expert gather,
 * SwiGLU MLP over quantized expert banks, weighted scatter-add, optional
 * shared expert (src/quantized_qwen3_moe.rs:412-520,
 * src/quantized_deepseek2.rs:522-671, src/quantized_deepseek4.rs:1354-1492;
 * Kimi routing rule src/kimi_k3.rs:256-282).  Routing, bucketing and the
 * expert matmuls all run on the device; nothing is read back per layer. */
#define JQ_GATE_SOFTMAX 0       /* qwen3moe, deepseek2 gating_func 1 */
#define JQ_GATE_SIGMOID 1       /* deepseek2 gating_func 2 (V3, Kimi) */
#define JQ_GATE_SQRT_SOFTPLUS 2 /* deepseek4 */

typedef struct {
    int32_t gating;          /* JQ_GATE_* */
    uint32_t n_expert;       /* experts in the banks */
    uint32_t n_used;         /* experts per token (top-k) */
    uint32_t hidden;         /* model width (multiple of 256) */
    uint32_t inter;          /* expert feed-forward width (multiple of 256) */
    uint32_t n_group;        /* expert groups for group-limited selection (0 or 1 = off) */
    uint32_t topk_group;     /* groups kept */
    int32_t norm;            /* renormalise the selected weights (norm_topk_prob / expert_weights_norm) */
    int32_t renorm_plus_eps; /* 0: divide by max(sum, 6.1035156e-5); 1: by sum + 1e-20 (Kimi) */
    int32_t oob_policy;      /* expert id >= n_expert: 0 = fail with JQ_E_EXPERT_RANGE
                                (src/quantized_qwen3_moe.rs:464-477), 1 = skip (src/quantized_deepseek4.rs:1439) */
    float scale;             /* expert_weights_scale, applied when != 0 and != 1 */
    float clamp;             /* SwiGLU clamp (src/quantized_deepseek4.rs:445-462), 0 = off */
} jq_moe_config;

/* `router`: host f32 [n_expert, hidden] (`ffn_gate_inp`); `bias`: host f32
 * [n_expert] selection bias (`exp_probs_b`) or NULL.  gate / up / down: banks
 * of n_expert contiguous experts, [n_expert*inter, hidden] twice and
 * [n_expert*hidden, inter] (the layout `split_experts` slices).  sh_*: one
 * shared expert or all NULL.  The weights must outlive the layer.  gate, up
 * and down may all be NULL: the layer then only routes (jq_moe_route_dev), for
 * expert-parallel callers whose banks live in a second, per-device layer. */
int32_t jq_moe_create(jq_ctx* ctx, const jq_moe_config* cfg, const float* router, const float* bias,
                      const jq_weight* gate, const jq_weight* up, const jq_weight* down, const jq_weight* sh_gate,
                      const jq_weight* sh_up, const jq_weight* sh_down, jq_moe** out);
void jq_moe_free(jq_moe* m);

/* Moe::forward with HOST buffers: x f32 [n_tokens, hidden] -> y f32
 * [n_tokens, hidden].  `forced_ids` ([n_tokens, n_used], or NULL) replaces the
 * top-k selection on hash-routed layers (`tid2eid[token_id]`,
 * src/quantized_deepseek4.rs:1375-1398); weights still come from the gate. */
int32_t jq_moe_forward(jq_moe* m, const float* x, uint64_t n_tokens, const uint32_t* forced_ids, float* y);

/* Sizes the layer's device workspace for up to n_tokens tokens (and n_rows rows
 * for jq_moe_experts_dev).  The *_dev entries never allocate: call this first
 * (and before capturing a stream). */
int32_t jq_moe_reserve(jq_moe* m, uint64_t n_tokens, uint64_t n_rows);

/* The same with DEVICE buffers on a caller stream.  No synchronisation for decode-sized and moderate batches;
 * when n_tokens * n_used >= 64 * n_expert (192 * n_expert for experts under 8 M weights; prefill) the call reads the expert histogram back once, which
 * synchronises the stream, and may allocate: such batches cannot be captured in a CUDA graph. */
int32_t jq_moe_forward_dev(jq_moe* m, const float* x_dev, uint64_t n_tokens, const uint32_t* forced_ids_dev,
                           float* y_dev, void* stream);

/* y = residual + layer(x): the residual add of the surrounding block folded into
 * the combine (residual_dev may be y_dev, or NULL for jq_moe_forward_dev). */
int32_t jq_moe_forward_add_dev(jq_moe* m, const float* x_dev, uint64_t n_tokens, const uint32_t* forced_ids_dev,
                               const float* residual_dev, float* y_dev, void* stream);

/* The same with the RMS norm of the block folded in: y = residual +
 * layer(rmsnorm(x; norm_w, eps)).  For batches of up to 8 tokens the layer is
 * four launches: router + routing + job list, gate/up, down, combine. */
int32_t jq_moe_forward_norm_add_dev(jq_moe* m, const float* x_dev, uint64_t n_tokens, const uint32_t* forced_ids_dev,
                                    const float* norm_w_dev, float eps, const float* residual_dev, float* y_dev,
                                    void* stream);

/* The two halves, for expert-parallel callers that exchange rows between
 * devices in between: routing alone (ids, weights: [n_tokens, n_used]), and the
 * expert MLPs alone over arbitrary rows, out[r] = MLP_{expert_ids[r]}(x[r])
 * (unweighted; rows whose id is out of range come back as zeros). */
int32_t jq_moe_route_dev(jq_moe* m, const float* x_dev, uint64_t n_tokens, const uint32_t* forced_ids_dev,
                         uint32_t* ids_dev, float* wts_dev, void* stream);
int32_t jq_moe_experts_dev(jq_moe* m, const float* x_dev, uint64_t n_rows, const uint32_t* expert_ids_dev,
                           float* out_dev, void* stream);
/* The expert matmuls alone (gate/up with SwiGLU, then down) over the job list that the last decode-sized
 * jq_moe_forward*_dev / jq_moe_experts_dev call on this layer left on the device, reading the rows of x_dev
 * (shaped as in that call).  For measuring the matmul kernels without routing and combine; the layer's output
 * buffer is overwritten, no result is returned. */
int32_t jq_moe_experts_replay_dev(jq_moe* m, const float* x_dev, void* stream);
/* Routing of rmsnorm(x; norm_w, eps): the block's norm folded into the router kernel (up to eight tokens). */
int32_t jq_moe_route_norm_dev(jq_moe* m, const float* x_dev, uint64_t n_tokens, const float* norm_w_dev, float eps,
                              const uint32_t* forced_ids_dev, uint32_t* ids_dev, float* wts_dev, void* stream);

/* After synchronising: JQ_E_EXPERT_RANGE if an id was out of range under
 * oob_policy 0, JQ_E_TIMEOUT as jq_device_status, else JQ_OK. */
int32_t jq_moe_status(jq_moe* m);

/* ids and weights chosen by the last forward (host copies), for inspection. */
int32_t jq_moe_last_routing(jq_moe* m, uint64_t n_tokens, uint32_t* ids, float* wts);

/* ── Expert-parallel exchange: one process per GPU, experts split contiguously over the ranks ──
 * No counterpart in the reference, which runs every expert of a layer in one
 * process (src/quantized_qwen3_moe.rs:385-542, expert tensors laid out
 * [n_expert, out, in], :572-613); this is the one place the path shards.
 * Activation rows travel to the rank that owns the chosen expert and the
 * outputs travel back by direct stores into peer memory over NVLink (CUDA IPC
 * mappings); every rank passes its own tokens and gets its own outputs,
 * y[t] = sum over slots in slot order of w[t,s] * MLP_{id[t,s]}(x[t]), the
 * same values for any number of ranks.
 *
 *   jq_ep_create   on every rank (rank < world <= 8, n_expert % world == 0,
 *                  max_tokens * n_used <= 16384): allocates this rank's window
 *   jq_ep_export   writes the JQ_EP_HANDLE_BYTES-byte handle of the window;
 *                  the host gathers the handles of all ranks, in rank order,
 *                  by whatever means it has (MPI, a store, torch.distributed)
 *   jq_ep_connect  maps the peers' windows (handles: world x 64 bytes); every
 *                  rank must have connected before any rank's first forward
 *   jq_ep_forward_dev  one layer.  `router` is a layer with the global expert
 *                  count (it may be router-only), `experts` a layer whose
 *                  banks hold this rank's n_expert / world experts (oob_policy
 *                  1; reserved for world * max_tokens * n_used rows).  Every
 *                  rank must call it the same number of times in the same
 *                  order, one exchange per call.  residual_dev (optional, may be
 *                  y_dev) is added to the result.  Waits on peers are bounded
 *                  (about a second by default): a rank that never arrives is
 *                  reported by jq_device_status as JQ_E_TIMEOUT instead of a hang.
 *   jq_ep_set_poll_limit  the bound of those waits, in polls of a peer flag
 *                  (a poll costs 0.2 - 1 us; 0 restores the default of 2^22)
 *   jq_ep_connect_loopback  instead of jq_ep_connect: every peer window becomes a
 *                  private allocation on this device that nobody serves.  For
 *                  single-GPU tests of the wait bound and of the addressing; the
 *                  waits on the absent peers run out and are reported.
 *   jq_ep_rows_served  after synchronising the device: how many activation rows
 *                  this rank's experts were sent in the last exchange (the load
 *                  figure behind max / mean over ranks under skewed routing). */
#define JQ_EP_HANDLE_BYTES 64
typedef struct jq_ep jq_ep;
int32_t jq_ep_create(jq_ctx* ctx, uint32_t rank, uint32_t world, uint32_t n_expert, uint32_t n_used, uint32_t hidden,
                     uint32_t max_tokens, jq_ep** out);
void jq_ep_free(jq_ep* e);
int32_t jq_ep_export(jq_ep* e, uint8_t* handle);
int32_t jq_ep_connect(jq_ep* e, const uint8_t* handles);
int32_t jq_ep_connect_loopback(jq_ep* e);
int32_t jq_ep_set_poll_limit(jq_ep* e, uint32_t polls);
int32_t jq_ep_rows_served(jq_ep* e, uint32_t* rows);
int32_t jq_ep_forward_dev(jq_ep* e, jq_moe* router, jq_moe* experts, const float* x_dev, uint64_t n_tokens,
                          const float* residual_dev, float* y_dev, void* stream);
/* The same with the block's RMS norm folded in: y = residual + layer(rmsnorm(x; norm_w, eps)); the router
 * normalises inside its kernel and the rows travel normalised.  forced_ids_dev ([n_tokens, n_used] or NULL)
 * replaces the top-k selection as in jq_moe_forward (hash-routed layers, src/quantized_deepseek4.rs:1375-1398). */
int32_t jq_ep_forward_norm_dev(jq_ep* e, jq_moe* router, jq_moe* experts, const float* x_dev, uint64_t n_tokens,
                               const float* norm_w_dev, float eps, const uint32_t* forced_ids_dev,
                               const float* residual_dev, float* y_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* JOSHUA_B200_H */
