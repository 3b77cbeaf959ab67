// C ABI of the decode-step kernels around the matmuls.  Declarations are in include/joshua_b200.h.
#include "handles.cuh"

extern "C" {

int32_t jq_matmul_swiglu_dev(const jq_weight* gate, const jq_weight* up, uint64_t m, uint64_t k, uint64_t n,
                             const float* lhs_dev, float* dst_dev, float clamp, void* stream) {
    if (!gate || !up) return jq_fail(jq::E_INVALID, "jq_matmul_swiglu_dev: NULL weight handle");
    if (gate->type != up->type || gate->n_blocks != up->n_blocks)
        return jq_fail(jq::E_INVALID, "jq_matmul_swiglu_dev: gate and up differ in type or size");
    if (k % gate->fmt.elems != 0 || gate->n_blocks != n * (k / gate->fmt.elems))
        return jq_fail(jq::E_INVALID, std::string(jq_type_name(gate->type)) + " matmul: rhs holds " +
                                          std::to_string(gate->n_blocks) + " blocks, expected " +
                                          std::to_string(k % gate->fmt.elems ? 0 : n * (k / gate->fmt.elems)));
    if (m == 0 || n == 0) return jq::OK;
    if (!lhs_dev || !dst_dev) return jq_fail(jq::E_INVALID, "jq_matmul_swiglu_dev: NULL buffer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    jq_ctx* ctx = gate->ctx;
    if (!ctx->force_f32 && jq::gemv_mma_supports(gate->type, gate->dev, n, k, m) &&
        jq::gemv_mma_supports(up->type, up->dev, n, k, m) && jq::gemv_mma_scratch_bytes(m, k) == 0) {
        JQ_CUDA(jq::launch_gemv_mma_swiglu(gate->type, gate->dev, up->dev, n, k, lhs_dev, m, dst_dev, clamp,
                                           ctx->status_dev, s));
        return jq::OK;
    }
    // two products into scratch, then the element-wise combine
    void* scratch = nullptr;
    size_t need = 2 * m * n * 4 + 512;
    JQ_CUDA(ctx->scratch_for(reinterpret_cast<cudaStream_t>(reinterpret_cast<uintptr_t>(s) ^ 1), need, &scratch));
    float* g = static_cast<float*>(scratch);
    float* u = g + ((m * n + 63) & ~(uint64_t)63);
    if (int32_t rc = jq_matmul_device(gate, m, k, n, lhs_dev, g, s)) return rc;
    if (int32_t rc = jq_matmul_device(up, m, k, n, lhs_dev, u, s)) return rc;
    JQ_CUDA(jq::launch_swiglu(g, u, m * n, clamp, dst_dev, s));
    return jq::OK;
}

int32_t jq_matmul_swiglu_norm_dev(const jq_weight* gate, const jq_weight* up, uint64_t m, uint64_t k, uint64_t n,
                                  const float* lhs_dev, const float* norm_w_dev, float eps, float* dst_dev,
                                  float clamp, void* stream) {
    if (!norm_w_dev) return jq_matmul_swiglu_dev(gate, up, m, k, n, lhs_dev, dst_dev, clamp, stream);
    if (!gate || !up) return jq_fail(jq::E_INVALID, "jq_matmul_swiglu_norm_dev: NULL weight handle");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    jq_ctx* ctx = gate->ctx;
    const bool shapes_ok = gate->type == up->type && gate->n_blocks == up->n_blocks && k % gate->fmt.elems == 0 &&
                           gate->n_blocks == n * (k / gate->fmt.elems) && m > 0 && n > 0 && lhs_dev && dst_dev;
    if (shapes_ok && !ctx->force_f32 && jq::gemv_mma_supports(gate->type, gate->dev, n, k, m) &&
        jq::gemv_mma_supports(up->type, up->dev, n, k, m) && jq::gemv_mma_fusable(m, k)) {
        JQ_CUDA(jq::launch_gemv_mma_swiglu(gate->type, gate->dev, up->dev, n, k, lhs_dev, m, dst_dev, clamp,
                                           ctx->status_dev, s, norm_w_dev, eps));
        return jq::OK;
    }
    // separate kernels: normalise into scratch, then the plain entry (which validates)
    void* scratch = nullptr;
    JQ_CUDA(ctx->scratch_for(reinterpret_cast<cudaStream_t>(reinterpret_cast<uintptr_t>(s) ^ 2), m * k * 4 + 256, &scratch));
    JQ_CUDA(jq::launch_rmsnorm(lhs_dev, nullptr, norm_w_dev, eps, m, (uint32_t)k, nullptr, static_cast<float*>(scratch), s));
    return jq_matmul_swiglu_dev(gate, up, m, k, n, static_cast<const float*>(scratch), dst_dev, clamp, stream);
}

int32_t jq_matmul_norm_dev(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs_dev,
                           const float* norm_w_dev, float eps, const float* residual_dev, float* dst_dev,
                           void* stream) {
    if (!w) return jq_fail(jq::E_INVALID, "jq_matmul_norm_dev: NULL weight handle");
    if (!norm_w_dev && !residual_dev) return jq_matmul_t_dev(w, m, k, n, lhs_dev, dst_dev, stream);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    jq_ctx* ctx = w->ctx;
    const bool shapes_ok = k % w->fmt.elems == 0 && w->n_blocks == n * (k / w->fmt.elems) && m > 0 && n > 0 &&
                           lhs_dev && dst_dev;
    if (shapes_ok && !ctx->force_f32 && jq::gemv_mma_supports(w->type, w->dev, n, k, m) && jq::gemv_mma_fusable(m, k)) {
        JQ_CUDA(jq::launch_gemv_mma_fused(w->type, w->dev, n, k, lhs_dev, m, dst_dev, norm_w_dev, eps, residual_dev,
                                          ctx->status_dev, s));
        return jq::OK;
    }
    // separate kernels: norm into scratch, product into scratch, then the add
    if (m == 0 || n == 0) return jq_matmul_t_dev(w, m, k, n, lhs_dev, dst_dev, stream);
    void* scratch = nullptr;
    const uint64_t xk = (m * k + 63) & ~(uint64_t)63;
    JQ_CUDA(ctx->scratch_for(reinterpret_cast<cudaStream_t>(reinterpret_cast<uintptr_t>(s) ^ 2), (xk + m * n) * 4 + 256, &scratch));
    float* xn = static_cast<float*>(scratch);
    float* prod = xn + xk;
    const float* in = lhs_dev;
    if (norm_w_dev) {
        if (!lhs_dev) return jq_fail(jq::E_INVALID, "jq_matmul_norm_dev: NULL buffer");
        JQ_CUDA(jq::launch_rmsnorm(lhs_dev, nullptr, norm_w_dev, eps, m, (uint32_t)k, nullptr, xn, s));
        in = xn;
    }
    if (!residual_dev) return jq_matmul_t_dev(w, m, k, n, in, dst_dev, stream);
    if (int32_t rc = jq_matmul_t_dev(w, m, k, n, in, prod, stream)) return rc;
    JQ_CUDA(jq::launch_add(residual_dev, prod, m * n, dst_dev, s));
    return jq::OK;
}

uint64_t jq_attention_fused_scratch_bytes(uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim,
                                          uint32_t max_ctx) {
    return jq::attention_fused_scratch_bytes(batch, n_q, n_kv, head_dim, max_ctx);
}

int32_t jq_attention_fused_dev(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t n_q, uint32_t n_kv,
                               uint32_t head_dim, uint32_t max_ctx, float theta, float* cache_k, float* cache_v,
                               float* out, void* scratch, int32_t* bad_pos_dev, void* stream) {
    return jq_attention_fused_qknorm_dev(qkv, pos, batch, n_q, n_kv, head_dim, max_ctx, theta, nullptr, nullptr, 0.0f,
                                         cache_k, cache_v, out, scratch, bad_pos_dev, stream);
}

int32_t jq_attention_fused_qknorm_dev(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t n_q, uint32_t n_kv,
                                      uint32_t head_dim, uint32_t max_ctx, float theta, const float* q_norm_w,
                                      const float* k_norm_w, float qk_eps, float* cache_k, float* cache_v, float* out,
                                      void* scratch, int32_t* bad_pos_dev, void* stream) {
    if (batch == 0) return jq::OK;
    if ((q_norm_w == nullptr) != (k_norm_w == nullptr))
        return jq_fail(jq::E_INVALID, "jq_attention_fused_qknorm_dev: q and k norm weights go together");
    if (!qkv || !pos || !cache_k || !cache_v || !out || !scratch)
        return jq_fail(jq::E_INVALID, "jq_attention_fused_dev: NULL buffer");
    if (n_kv == 0 || n_q % n_kv || !(head_dim == 64 || head_dim == 128 || head_dim == 256) ||
        !(n_q / n_kv == 1 || n_q / n_kv == 2 || n_q / n_kv == 4 || n_q / n_kv == 8))
        return jq_fail(jq::E_INVALID, "jq_attention_fused_dev: need head_dim 64, 128 or 256 and 1, 2, 4 or 8 query heads per kv head");
    JQ_CUDA(jq::launch_attention_fused(qkv, pos, batch, n_q, n_kv, head_dim, max_ctx, theta, cache_k, cache_v, out,
                                       scratch, bad_pos_dev, static_cast<cudaStream_t>(stream), q_norm_w, k_norm_w,
                                       qk_eps));
    return jq::OK;
}

int32_t jq_embedding_dev(const jq_weight* w, const uint32_t* ids_dev, uint64_t n_ids, uint64_t rows, uint64_t hidden,
                         float* out_dev, int32_t* bad_id_dev, void* stream) {
    if (!w) return jq_fail(jq::E_INVALID, "jq_embedding_dev: NULL weight handle");
    if (hidden % w->fmt.elems != 0)
        return jq_fail(jq::E_INVALID, "quantized embedding hidden size " + std::to_string(hidden) +
                                          " is not divisible by block size " + std::to_string(w->fmt.elems));
    if (w->n_blocks != rows * (hidden / w->fmt.elems))
        return jq_fail(jq::E_INVALID, "quantized tensor has " + std::to_string(w->n_blocks) + " blocks, expected " +
                                          std::to_string(rows * (hidden / w->fmt.elems)));
    if (n_ids == 0) return jq::OK;
    if (!ids_dev || !out_dev || !bad_id_dev) return jq_fail(jq::E_INVALID, "jq_embedding_dev: NULL buffer");
    JQ_CUDA(jq::launch_embedding(w->type, w->dev, rows, hidden, ids_dev, n_ids, out_dev, bad_id_dev,
                                 static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_rmsnorm_dev(const float* x, const float* residual, const float* weight, float eps, uint64_t rows,
                       uint64_t hidden, float* sum_out, float* out, void* stream) {
    if (rows == 0) return jq::OK;
    if (!x || !out || hidden == 0) return jq_fail(jq::E_INVALID, "jq_rmsnorm_dev: NULL buffer");
    if (residual && !sum_out) return jq_fail(jq::E_INVALID, "jq_rmsnorm_dev: a residual needs sum_out");
    JQ_CUDA(jq::launch_rmsnorm(x, residual, weight, eps, rows, (uint32_t)hidden, sum_out, out,
                               static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_rope_append_dev(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t n_q, uint32_t n_kv,
                           uint32_t head_dim, uint32_t max_ctx, float theta, float* q_out, float* cache_k,
                           float* cache_v, int32_t* bad_pos_dev, void* stream) {
    if (batch == 0) return jq::OK;
    if (!qkv || !pos || !q_out || !cache_k || !cache_v || head_dim % 2 || n_kv == 0 || n_q % n_kv)
        return jq_fail(jq::E_INVALID, "jq_rope_append_dev: bad argument");
    JQ_CUDA(jq::launch_rope_append(qkv, pos, batch, n_q, n_kv, head_dim, max_ctx, theta, q_out, cache_k, cache_v,
                                   bad_pos_dev, static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

uint64_t jq_attention_scratch_bytes(uint32_t batch, uint32_t n_q, uint32_t head_dim, uint32_t max_ctx) {
    return jq::attention_scratch_bytes(batch, n_q, head_dim, max_ctx);
}

int32_t jq_attention_decode_dev(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_ctx,
                                float* out, float* scratch, int32_t* bad_pos_dev, void* stream) {
    if (batch == 0) return jq::OK;
    if (!q || !cache_k || !cache_v || !pos || !out || !scratch || n_kv == 0 || n_q % n_kv)
        return jq_fail(jq::E_INVALID, "jq_attention_decode_dev: bad argument");
    JQ_CUDA(jq::launch_attention_decode(q, cache_k, cache_v, pos, batch, n_q, n_kv, head_dim, max_ctx, out, scratch,
                                        bad_pos_dev, static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_add_dev(const float* a, const float* b, uint64_t n, float* y, void* stream) {
    if (n == 0) return jq::OK;
    if (!a || !b || !y) return jq_fail(jq::E_INVALID, "jq_add_dev: NULL buffer");
    JQ_CUDA(jq::launch_add(a, b, n, y, static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

uint64_t jq_argmax_scratch_bytes(uint64_t rows) { return jq::argmax_scratch_bytes((uint32_t)rows); }

int32_t jq_argmax_dev(const float* logits, uint64_t rows, uint64_t vocab, int32_t* token, int32_t* pos, void* scratch,
                      void* stream) {
    if (rows == 0) return jq::OK;
    if (!logits || !token || !scratch || vocab == 0) return jq_fail(jq::E_INVALID, "jq_argmax_dev: bad argument");
    JQ_CUDA(jq::launch_argmax(logits, (uint32_t)rows, (uint32_t)vocab, token, pos, scratch,
                              static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_rope_append_prefill_dev(const float* qkv, const int32_t* pos0, uint32_t seq, uint32_t n_q, uint32_t n_kv,
                                   uint32_t head_dim, uint32_t max_ctx, float theta, const float* q_norm_w,
                                   const float* k_norm_w, float qk_eps, float* q_out, float* cache_k, float* cache_v,
                                   int32_t* bad_pos_dev, void* stream) {
    if (seq == 0) return jq::OK;
    if (!qkv || !pos0 || !q_out || !cache_k || !cache_v || head_dim % 2 || n_kv == 0 || n_q % n_kv ||
        (q_norm_w == nullptr) != (k_norm_w == nullptr))
        return jq_fail(jq::E_INVALID, "jq_rope_append_prefill_dev: bad argument");
    JQ_CUDA(jq::launch_rope_append(qkv, pos0, 1, n_q, n_kv, head_dim, max_ctx, theta, q_out, cache_k, cache_v, bad_pos_dev,
                                   static_cast<cudaStream_t>(stream), seq, q_norm_w, k_norm_w, qk_eps));
    return jq::OK;
}

int32_t jq_attention_prefill_dev(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos0,
                                 uint32_t seq, uint32_t n_q, uint32_t n_kv, uint32_t head_dim, uint32_t max_ctx,
                                 float* out, int32_t* bad_pos_dev, void* stream) {
    if (seq == 0) return jq::OK;
    if (!q || !cache_k || !cache_v || !pos0 || !out || n_kv == 0 || n_q % n_kv)
        return jq_fail(jq::E_INVALID, "jq_attention_prefill_dev: bad argument");
    if (head_dim != 64 && head_dim != 128)
        return jq_fail(jq::E_INVALID, "jq_attention_prefill_dev: head_dim 64 or 128");
    JQ_CUDA(jq::launch_attention_prefill(q, cache_k, cache_v, pos0, seq, n_q, n_kv, head_dim, max_ctx, out, bad_pos_dev,
                                         static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_rmsnorm_strided_dev(const float* x, uint64_t x_stride, const float* weight, float eps, uint64_t rows,
                               uint64_t hidden, float* out, void* stream) {
    if (rows == 0) return jq::OK;
    if (!x || !out || hidden == 0 || x_stride < hidden) return jq_fail(jq::E_INVALID, "jq_rmsnorm_strided_dev: bad argument");
    JQ_CUDA(jq::launch_rmsnorm(x, nullptr, weight, eps, rows, (uint32_t)hidden, nullptr, out,
                               static_cast<cudaStream_t>(stream), (uint32_t)x_stride));
    return jq::OK;
}

int32_t jq_mla_assemble_dev(float* q, const float* comp, const float* kv, const int32_t* pos, uint32_t batch,
                            uint32_t n_head, uint32_t qk_nope, uint32_t qk_rope, uint32_t v_dim, uint32_t kv_lora,
                            uint32_t max_ctx, const float* inv_freq_dev, float mscale, float* cache_k, float* cache_v,
                            int32_t* bad_pos_dev, void* stream) {
    if (batch == 0) return jq::OK;
    if (!q || !comp || !kv || !pos || !inv_freq_dev || !cache_k || !cache_v || n_head == 0 || qk_rope % 2)
        return jq_fail(jq::E_INVALID, "jq_mla_assemble_dev: bad argument");
    JQ_CUDA(jq::launch_mla_assemble(q, comp, kv, pos, batch, n_head, qk_nope, qk_rope, v_dim, kv_lora, max_ctx,
                                    inv_freq_dev, mscale, cache_k, cache_v, bad_pos_dev,
                                    static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_attention_decode_qkv_dev(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                    uint32_t batch, uint32_t n_q, uint32_t n_kv, uint32_t qk_dim, uint32_t v_dim,
                                    uint32_t max_ctx, float softmax_scale, float* out, float* scratch,
                                    int32_t* bad_pos_dev, void* stream) {
    if (batch == 0) return jq::OK;
    if (!q || !cache_k || !cache_v || !pos || !out || !scratch || n_kv == 0 || n_q % n_kv || qk_dim == 0 || v_dim == 0)
        return jq_fail(jq::E_INVALID, "jq_attention_decode_qkv_dev: bad argument");
    JQ_CUDA(jq::launch_attention_decode(q, cache_k, cache_v, pos, batch, n_q, n_kv, qk_dim, max_ctx, out, scratch,
                                        bad_pos_dev, static_cast<cudaStream_t>(stream), v_dim, softmax_scale));
    return jq::OK;
}

int32_t jq_swiglu_dev(const float* gate, const float* up, uint64_t n, float clamp, float* out, void* stream) {
    if (n == 0) return jq::OK;
    if (!gate || !up || !out) return jq_fail(jq::E_INVALID, "jq_swiglu_dev: NULL buffer");
    JQ_CUDA(jq::launch_swiglu(gate, up, n, clamp, out, static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_sample_greedy_dev(const float* logits, uint64_t rows, uint64_t vocab, float repetition_penalty,
                             int32_t* window, int32_t* window_state, int32_t* token, int32_t* pos, void* scratch,
                             void* stream) {
    if (rows == 0) return jq::OK;
    if (!logits || !token || !scratch || vocab == 0) return jq_fail(jq::E_INVALID, "jq_sample_greedy_dev: bad argument");
    if ((window == nullptr) != (window_state == nullptr))
        return jq_fail(jq::E_INVALID, "jq_sample_greedy_dev: window and window_state go together");
    if (!(repetition_penalty > 0.0f)) return jq_fail(jq::E_INVALID, "jq_sample_greedy_dev: the penalty must be positive");
    JQ_CUDA(jq::launch_argmax(logits, (uint32_t)rows, (uint32_t)vocab, token, pos, scratch,
                              static_cast<cudaStream_t>(stream), repetition_penalty, window, window_state));
    return jq::OK;
}

}  // extern "C"
