// C ABI of the persistent decode chain: a fixed sequence of quantized linears and attention steps over
// fixed device buffers, replayed in one launch per call.  Declarations are in include/joshua_b200.h.
#include "chain.cuh"
#include "handles.cuh"

struct jq_chain {
    jq_ctx* ctx;
    uint32_t type, m;
    std::vector<jq::ChainOp> ops;
    uint64_t max_k = 0;
    uint32_t att_floats = 0;
    jq::ChainOp* ops_dev = nullptr;
    unsigned long long* arrivals = nullptr;
    bool sealed = false;
    unsigned long long* trace = nullptr;
};

extern "C" {

int32_t jq_chain_create(jq_ctx* ctx, uint32_t type, uint32_t m, jq_chain** out) {
    if (!ctx || !out) return jq_fail(jq::E_INVALID, "jq_chain_create: NULL argument");
    *out = nullptr;
    if (!jq::gemv_chain_supports(type, m, 256, 0))
        return jq_fail(jq::E_TYPE, std::string("jq_chain_create: no chain kernel for ") + jq_type_name(type) +
                                       " at batch " + std::to_string(m) + " (Q4_K and Q8_0, batch 1..8)");
    JQ_CUDA(cudaSetDevice(ctx->device));
    jq_chain* c = new (std::nothrow) jq_chain();
    if (!c) return jq_fail(jq::E_NOMEM, "jq_chain_create: out of host memory");
    c->ctx = ctx;
    c->type = type;
    c->m = m;
    cudaError_t e = cudaMalloc(&c->arrivals, 256);
    if (e == cudaSuccess) e = cudaMemset(c->arrivals, 0, 256);
    if (e != cudaSuccess) {
        delete c;
        return jq_fail_cuda(e, "jq_chain_create");
    }
    *out = c;
    return jq::OK;
}

void jq_chain_free(jq_chain* c) {
    if (!c) return;
    cudaSetDevice(c->ctx->device);
    cudaDeviceSynchronize();
    cudaFree(c->ops_dev);
    cudaFree(c->arrivals);
    delete c;
}

int32_t jq_chain_add_linear(jq_chain* c, const jq_weight* w, const jq_weight* w_up, uint64_t k, uint64_t n,
                            const float* x_dev, const float* norm_w_dev, float eps, const float* residual_dev,
                            float clamp, float* dst_dev) {
    if (!c || !w) return jq_fail(jq::E_INVALID, "jq_chain_add_linear: NULL handle");
    if (c->sealed) return jq_fail(jq::E_INVALID, "jq_chain_add_linear: the chain has already run");
    if (!x_dev || !dst_dev) return jq_fail(jq::E_INVALID, "jq_chain_add_linear: NULL buffer");
    if (w->type != c->type || (w_up && w_up->type != c->type))
        return jq_fail(jq::E_TYPE, std::string("jq_chain_add_linear: the chain holds ") + jq_type_name(c->type) +
                                       " linears, this one is " + jq_type_name(w->type));
    if (n == 0 || k == 0 || k % w->fmt.elems != 0 || w->n_blocks != n * (k / w->fmt.elems) ||
        (w_up && w_up->n_blocks != w->n_blocks))
        return jq_fail(jq::E_INVALID, std::string(jq_type_name(w->type)) + " matmul: rhs holds " +
                                          std::to_string(w->n_blocks) + " blocks, expected " +
                                          std::to_string(k % w->fmt.elems ? 0 : n * (k / w->fmt.elems)));
    if (!jq::gemv_mma_supports(w->type, w->dev, n, k, c->m) || (w_up && !jq::gemv_mma_supports(w_up->type, w_up->dev, n, k, c->m)) ||
        !jq::gemv_chain_supports(c->type, c->m, std::max(c->max_k, k), c->att_floats))
        return jq_fail(jq::E_INVALID, "jq_chain_add_linear: shape or alignment outside the decode kernel "
                                      "(k a multiple of 256, activation planes of m rows in shared memory)");
    if (w_up && residual_dev) return jq_fail(jq::E_INVALID, "jq_chain_add_linear: a SwiGLU pair takes no residual");
    jq::ChainOp op = {};
    op.kind = 0;
    op.swiglu = w_up ? 1 : 0;
    op.w[0] = w->dev;
    op.w[1] = w_up ? w_up->dev : w->dev;
    op.n = n;
    op.k = k;
    op.x = x_dev;
    op.dst = dst_dev;
    op.norm_w = norm_w_dev;
    op.residual = residual_dev;
    op.norm_eps = eps;
    op.clamp = clamp;
    c->ops.push_back(op);
    c->max_k = std::max(c->max_k, k);
    return jq::OK;
}

int32_t jq_chain_add_attention(jq_chain* c, const float* qkv, const int32_t* pos, uint32_t n_q, uint32_t n_kv,
                               uint32_t head_dim, uint32_t max_ctx, float theta, float* cache_k, float* cache_v,
                               float* out, void* scratch) {
    if (!c) return jq_fail(jq::E_INVALID, "jq_chain_add_attention: NULL handle");
    if (c->sealed) return jq_fail(jq::E_INVALID, "jq_chain_add_attention: the chain has already run");
    if (!qkv || !pos || !cache_k || !cache_v || !out || !scratch)
        return jq_fail(jq::E_INVALID, "jq_chain_add_attention: NULL buffer");
    jq::ChainOp op = {};
    op.kind = 1;
    if (!jq::attention_fused_args(qkv, pos, c->m, n_q, n_kv, head_dim, max_ctx, theta, cache_k, cache_v, out, scratch,
                                  &op.att))
        return jq_fail(jq::E_INVALID, "jq_chain_add_attention: need head_dim 64, 128 or 256, 1, 2, 4 or 8 query heads per kv head "
                                      "and a context that fits the kernel's shared memory");
    if (head_dim != 128 || (n_q / n_kv != 4 && n_q / n_kv != 8))
        return jq_fail(jq::E_INVALID, "jq_chain_add_attention: the chain carries head_dim 128 with 4 or 8 query heads per kv head");
    op.att.gsplit = 1;  // the chain runs one item per kv head
    uint32_t fl = jq::attention_fused_smem_floats(n_q, n_kv, head_dim, op.att.n_chunks);
    if (!jq::gemv_chain_supports(c->type, c->m, std::max<uint64_t>(c->max_k, 256), std::max(c->att_floats, fl)))
        return jq_fail(jq::E_INVALID, "jq_chain_add_attention: the attention step does not fit the chain's shared memory");
    c->att_floats = std::max(c->att_floats, fl);
    c->ops.push_back(op);
    return jq::OK;
}

int32_t jq_chain_set_trace(jq_chain* c, uint64_t* trace_dev) {
    if (!c) return jq_fail(jq::E_INVALID, "jq_chain_set_trace: NULL handle");
    c->trace = reinterpret_cast<unsigned long long*>(trace_dev);
    return jq::OK;
}

int32_t jq_chain_run(jq_chain* c, void* stream) {
    if (!c) return jq_fail(jq::E_INVALID, "jq_chain_run: NULL handle");
    if (c->ops.empty()) return jq::OK;
    if (!c->sealed) {
        // first run: the operation list moves to the device (allocates; do it before capturing a stream)
        JQ_CUDA(cudaSetDevice(c->ctx->device));
        JQ_CUDA(cudaMalloc(&c->ops_dev, c->ops.size() * sizeof(jq::ChainOp)));
        JQ_CUDA(cudaMemcpy(c->ops_dev, c->ops.data(), c->ops.size() * sizeof(jq::ChainOp), cudaMemcpyHostToDevice));
        c->sealed = true;
    }
    JQ_CUDA(jq::launch_gemv_chain(c->type, c->m, c->ops_dev, (uint32_t)c->ops.size(), std::max<uint64_t>(c->max_k, 256),
                                  c->att_floats, c->arrivals, c->ctx->status_dev, static_cast<cudaStream_t>(stream),
                                  c->trace));
    return jq::OK;
}

}  // extern "C"
