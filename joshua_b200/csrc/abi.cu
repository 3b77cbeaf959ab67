// The extern "C" boundary: contexts, weight handles, validation, staging of
// host buffers, kernel dispatch.  Declarations and the reference interfaces
// they replace are in include/joshua_b200.h.
#include <cuda_fp16.h>

#include "handles.cuh"

namespace {
thread_local std::string g_err;
}

int32_t jq_fail(int32_t code, const std::string& msg) {
    g_err = msg;
    return code;
}
int32_t jq_fail_cuda(cudaError_t e, const char* what) {
    return jq_fail(e == cudaErrorMemoryAllocation ? jq::E_NOMEM : jq::E_CUDA,
                   std::string(what) + ": " + cudaGetErrorString(e));
}
const char* jq_type_name(uint32_t t) {
    switch (t) {
        case jq::T_Q8_0: return "q8_0";
        case jq::T_Q2_K: return "q2_k";
        case jq::T_Q4_K: return "q4_k";
        case jq::T_IQ2_XXS: return "iq2_xxs";
        case jq::T_MXFP4: return "mxfp4";
        case jq::T_Q4_0: return "q4_0";
        case jq::T_Q4_1: return "q4_1";
        case jq::T_Q5_0: return "q5_0";
        case jq::T_Q5_1: return "q5_1";
        case jq::T_Q8_1: return "q8_1";
        case jq::T_Q3_K: return "q3_k";
        case jq::T_Q5_K: return "q5_k";
        case jq::T_Q6_K: return "q6_k";
        case jq::T_Q8_K: return "q8_k";
        default: return "?";
    }
}

namespace {

struct WsGuard {
    jq_ctx* ctx;
    Workspace* ws;
    ~WsGuard() {
        if (ws) ctx->release(ws);
    }
};

// Shape rules of src/quant_matmul.rs:133-165 / src/iq2xxs.rs:126-153 / src/mxfp4.rs:142-172.
int32_t validate_matmul(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, uint64_t lhs_len, uint64_t dst_len,
                        bool check_lens) {
    if (!w) return jq_fail(jq::E_INVALID, "matmul: NULL weight handle");
    const char* name = jq_type_name(w->type);
    if (k % w->fmt.elems != 0)
        return jq_fail(jq::E_INVALID, std::string(name) + " matmul: k=" + std::to_string(k) +
                                       " is not a multiple of the block size " + std::to_string(w->fmt.elems));
    uint64_t bpr = k / w->fmt.elems;
    if (w->n_blocks != n * bpr)
        return jq_fail(jq::E_INVALID, std::string(name) + " matmul: rhs holds " + std::to_string(w->n_blocks) +
                                       " blocks, expected " + std::to_string(n * bpr));
    if (check_lens && (lhs_len != m * k || dst_len != m * n))
        return jq_fail(jq::E_INVALID, std::string(name) + " matmul: lhs/dst sized " + std::to_string(lhs_len) + "/" +
                                       std::to_string(dst_len) + " expected " + std::to_string(m * k) + "/" +
                                       std::to_string(m * n));
    return jq::OK;
}

// Picks the kernel for a device-resident product.
}  // namespace

int32_t jq_matmul_device(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs, float* dst,
                         cudaStream_t s) {
    jq_ctx* ctx = w->ctx;
    if (!ctx->force_f32 && jq::gemv_mma_supports(w->type, w->dev, n, k, m)) {
        void* scratch = nullptr;
        JQ_CUDA(ctx->scratch_for(s, jq::gemv_mma_scratch_bytes(m, k), &scratch));
        JQ_CUDA(jq::launch_gemv_mma(w->type, w->dev, n, k, lhs, m, dst, scratch, ctx->status_dev, s));
        return jq::OK;
    }
    // Batches a little above the decode kernel's eight rows: eight rows at a time through the decode kernel
    // (the weights are read once per slice, from L2 when they fit) still beats the tile GEMM, whose K loop
    // costs the same at any batch.
    if (!ctx->force_f32 && m > jq::GEMV_MMA_MAX_M && m <= ctx->sliced_max_m &&
        jq::gemv_mma_supports(w->type, w->dev, n, k, jq::GEMV_MMA_MAX_M)) {
        void* scratch = nullptr;
        JQ_CUDA(ctx->scratch_for(s, jq::gemv_mma_scratch_bytes(jq::GEMV_MMA_MAX_M, k), &scratch));
        for (uint64_t r0 = 0; r0 < m; r0 += jq::GEMV_MMA_MAX_M) {
            const uint64_t rows = std::min<uint64_t>(jq::GEMV_MMA_MAX_M, m - r0);
            JQ_CUDA(jq::launch_gemv_mma(w->type, w->dev, n, k, lhs + r0 * k, rows, dst + r0 * n, scratch,
                                        ctx->status_dev, s));
        }
        return jq::OK;
    }
    if (!ctx->force_f32 && m > jq::GEMV_MMA_MAX_M && jq::gemm_tc_supports(w->type, w->dev, n, k, m)) {
        void* scratch = nullptr;
        JQ_CUDA(ctx->scratch_for(reinterpret_cast<cudaStream_t>(reinterpret_cast<uintptr_t>(s) ^ 3), jq::gemm_tc_scratch_bytes(m, k), &scratch));
        JQ_CUDA(jq::launch_gemm_tc(w->type, w->dev, n, k, lhs, m, dst, scratch, ctx->status_dev, s));
        return jq::OK;
    }
    JQ_CUDA(jq::launch_matmul_f32(w->type, w->dev, n, k, lhs, m, dst, s));
    return jq::OK;
}

#ifdef JQ_PROFILING
extern "C" int32_t jq_debug_gemm_trace(uint64_t* trace_dev) {
    jq::gemm_tc_set_trace(reinterpret_cast<unsigned long long*>(trace_dev));
    return jq::OK;
}
#endif

namespace {

// Reports a kernel wait that gave up, once: the flag is cleared as it is reported, so that one late peer or one
// lost copy does not fail every later call on the context.
int32_t check_device_status(const jq_ctx* ctx) {
    volatile int* flag = static_cast<volatile int*>(ctx->status_host);
    if (flag && *flag != 0) {
        *flag = 0;
        return jq_fail(jq::E_TIMEOUT, "a bounded wait inside a kernel gave up (device status flag was set)");
    }
    return jq::OK;
}

__global__ void f16_to_f32_kernel(const __half* in, float* out, uint64_t n) {
    uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (i < n) out[i] = __half2float(in[i]);
}
__global__ void f32_to_f16_kernel(const float* in, __half* out, uint64_t n) {
    uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(in[i]);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" {

const char* jq_last_error(void) { return g_err.c_str(); }

int32_t jq_block_size(uint32_t type, uint64_t* elems, uint64_t* bytes) {
    jq::Format f;
    if (!jq::format_of(type, &f)) return jq_fail(jq::E_TYPE, "unsupported GGUF type id " + std::to_string(type));
    if (elems) *elems = f.elems;
    if (bytes) *bytes = f.bytes;
    return jq::OK;
}

int32_t jq_init(int32_t device, jq_ctx** out) {
    if (!out) return jq_fail(jq::E_INVALID, "jq_init: NULL out");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return jq_fail(jq::E_CUDA, std::string("jq_init: no CUDA device (") +
                                    (e != cudaSuccess ? cudaGetErrorString(e) : "device count 0") +
                                    "); this library has no CPU path");
    if (device < 0 || device >= count)
        return jq_fail(jq::E_INVALID, "jq_init: device " + std::to_string(device) + " out of " + std::to_string(count));
    JQ_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    JQ_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return jq_fail(jq::E_CUDA, "jq_init: kernels are built for sm_100a only, device is sm_" +
                                    std::to_string(prop.major) + std::to_string(prop.minor));
    JQ_CUDA(jq::tables_dequant());
    JQ_CUDA(jq::tables_gemv_f32());
    JQ_CUDA(jq::tables_gemv_mma());
    JQ_CUDA(jq::tables_gemm_tc());
    jq_ctx* c = new (std::nothrow) jq_ctx();
    if (!c) return jq_fail(jq::E_NOMEM, "jq_init: out of host memory");
    c->device = device;
    const char* f = std::getenv("JQ_FORCE_F32_PATH");
    c->force_f32 = f && f[0] == '1';
    if (const char* sm = std::getenv("JQ_SLICED_MAX_M")) c->sliced_max_m = std::strtoull(sm, nullptr, 10);
    cudaError_t he = cudaHostAlloc(&c->status_host, sizeof(int), cudaHostAllocMapped);
    if (he == cudaSuccess) he = cudaHostGetDevicePointer(&c->status_dev, c->status_host, 0);
    if (he != cudaSuccess) {
        delete c;
        return jq_fail_cuda(he, "jq_init: status flag");
    }
    *c->status_host = 0;
    *out = c;
    return jq::OK;
}

void jq_free(jq_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (auto& kv : ctx->scratch) cudaFree(kv.second.dev);
    for (int i = 0; i < 8; ++i) {
        if (ctx->aux[i]) cudaStreamDestroy(ctx->aux[i]);
        if (ctx->join_ev[i]) cudaEventDestroy(ctx->join_ev[i]);
    }
    if (ctx->fork_ev) cudaEventDestroy(ctx->fork_ev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    for (Workspace* w : ctx->idle) {
        cudaStreamSynchronize(w->stream);
        cudaFree(w->dev);
        cudaFree(w->flag);
        cudaStreamDestroy(w->stream);
        delete w;
    }
    delete ctx;
}

static int32_t make_weight(jq_ctx* ctx, uint32_t type, const uint8_t* dev, uint64_t nbytes, bool owns,
                           jq_weight** out) {
    jq_weight* w = new (std::nothrow) jq_weight();
    if (!w) return jq_fail(jq::E_NOMEM, "out of host memory");
    w->ctx = ctx;
    w->type = type;
    jq::format_of(type, &w->fmt);
    w->dev = dev;
    w->n_blocks = nbytes / w->fmt.bytes;
    w->owns = owns;
    *out = w;
    return jq::OK;
}

static int32_t check_blocks(const char* who, uint32_t type, uint64_t nbytes, jq::Format* f) {
    if (!jq::format_of(type, f))
        return jq_fail(jq::E_TYPE, std::string(who) + ": unsupported GGUF type id " + std::to_string(type));
    if (nbytes % f->bytes != 0)
        return jq_fail(jq::E_INVALID, std::string(jq_type_name(type)) + ": " + std::to_string(nbytes) +
                                       " bytes is not a whole number of " + std::to_string(f->bytes) +
                                       " byte blocks");
    return jq::OK;
}

int32_t jq_weight_upload(jq_ctx* ctx, uint32_t type, const void* bytes, uint64_t nbytes, jq_weight** out) {
    if (!ctx || !out || (!bytes && nbytes)) return jq_fail(jq::E_INVALID, "jq_weight_upload: NULL argument");
    *out = nullptr;
    jq::Format f;
    if (int32_t rc = check_blocks("jq_weight_upload", type, nbytes, &f)) return rc;
    JQ_CUDA(cudaSetDevice(ctx->device));
    uint8_t* dev = nullptr;
    // 16 spare bytes: kernels may read whole 16-byte vectors up to the end of the last block
    JQ_CUDA(cudaMalloc(&dev, nbytes + 16));
    cudaError_t e = cudaMemcpy(dev, bytes, nbytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(dev + nbytes, 0, 16);
    if (e != cudaSuccess) {
        cudaFree(dev);
        return jq_fail_cuda(e, "jq_weight_upload copy");
    }
    int32_t rc = make_weight(ctx, type, dev, nbytes, true, out);
    if (rc) cudaFree(dev);
    return rc;
}

int32_t jq_weight_from_device(jq_ctx* ctx, uint32_t type, const void* device_bytes, uint64_t nbytes,
                              jq_weight** out) {
    if (!ctx || !out || (!device_bytes && nbytes)) return jq_fail(jq::E_INVALID, "jq_weight_from_device: NULL argument");
    *out = nullptr;
    jq::Format f;
    if (int32_t rc = check_blocks("jq_weight_from_device", type, nbytes, &f)) return rc;
    if (reinterpret_cast<uintptr_t>(device_bytes) % 16 != 0)
        return jq_fail(jq::E_INVALID, "jq_weight_from_device: device pointer must be 16-byte aligned");
    return make_weight(ctx, type, static_cast<const uint8_t*>(device_bytes), nbytes, false, out);
}

int32_t jq_weight_slice(const jq_weight* parent, uint64_t block0, uint64_t n_blocks, jq_weight** out) {
    if (!parent || !out) return jq_fail(jq::E_INVALID, "jq_weight_slice: NULL argument");
    *out = nullptr;
    if (block0 > parent->n_blocks || n_blocks > parent->n_blocks - block0)
        return jq_fail(jq::E_INVALID, "jq_weight_slice: blocks [" + std::to_string(block0) + ", +" +
                                       std::to_string(n_blocks) + ") outside the tensor's " +
                                       std::to_string(parent->n_blocks));
    return make_weight(parent->ctx, parent->type, parent->dev + block0 * parent->fmt.bytes,
                       n_blocks * parent->fmt.bytes, false, out);
}

void jq_weight_free(jq_weight* w) {
    if (!w) return;
    if (w->owns) {
        cudaSetDevice(w->ctx->device);
        cudaFree(const_cast<uint8_t*>(w->dev));
    }
    delete w;
}

uint32_t jq_weight_type(const jq_weight* w) { return w ? w->type : 0; }
uint64_t jq_weight_storage_size(const jq_weight* w) { return w ? w->n_blocks * w->fmt.bytes : 0; }
uint64_t jq_weight_block_elems(const jq_weight* w) { return w ? w->fmt.elems : 0; }
const void* jq_weight_device_ptr(const jq_weight* w) { return w ? w->dev : nullptr; }

int32_t jq_matmul_t_dev(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs_dev,
                        float* dst_dev, void* stream) {
    if (int32_t rc = validate_matmul(w, m, k, n, 0, 0, false)) return rc;
    if (m == 0 || n == 0) return jq::OK;
    if (!lhs_dev || !dst_dev) return jq_fail(jq::E_INVALID, "jq_matmul_t_dev: NULL buffer");
    if (reinterpret_cast<uintptr_t>(lhs_dev) % 16 != 0)
        return jq_fail(jq::E_INVALID, "jq_matmul_t_dev: lhs must be 16-byte aligned");
    return jq_matmul_device(w, m, k, n, lhs_dev, dst_dev, static_cast<cudaStream_t>(stream));
}

int32_t jq_matmul_t_dev_noalloc(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs_dev,
                                float* dst_dev, void* stream) {
    if (int32_t rc = validate_matmul(w, m, k, n, 0, 0, false)) return rc;
    if (m == 0 || n == 0) return jq::OK;
    if (!lhs_dev || !dst_dev) return jq_fail(jq::E_INVALID, "jq_matmul_t_dev_noalloc: NULL buffer");
    if (reinterpret_cast<uintptr_t>(lhs_dev) % 16 != 0)
        return jq_fail(jq::E_INVALID, "jq_matmul_t_dev_noalloc: lhs must be 16-byte aligned");
    if (!jq::gemv_mma_supports(w->type, w->dev, n, k, m))
        return jq_fail(jq::E_TOO_LARGE, "jq_matmul_t_dev_noalloc: only batches of 1..8 rows with k a multiple of 256 "
                                        "are served without allocating");
    if (jq::gemv_mma_static_bytes_needed(m, k) > jq::GEMV_STATIC_SCRATCH_BYTES)
        return jq_fail(jq::E_TOO_LARGE, "jq_matmul_t_dev_noalloc: m*k = " + std::to_string(m * k) +
                                            " activations need " +
                                            std::to_string(jq::gemv_mma_static_bytes_needed(m, k)) +
                                            " bytes of scratch, the built-in array holds " +
                                            std::to_string(jq::GEMV_STATIC_SCRATCH_BYTES));
    JQ_CUDA(cudaSetDevice(w->ctx->device));
    JQ_CUDA(jq::launch_gemv_mma_static(w->type, w->dev, n, k, lhs_dev, m, dst_dev, w->ctx->status_dev,
                                       static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_matmul_t(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const float* lhs, uint64_t lhs_len,
                    float* dst, uint64_t dst_len) {
    if (int32_t rc = validate_matmul(w, m, k, n, lhs_len, dst_len, true)) return rc;
    if (m == 0 || n == 0) return jq::OK;
    if (!lhs || !dst) return jq_fail(jq::E_INVALID, "jq_matmul_t: NULL buffer");
    JQ_CUDA(cudaSetDevice(w->ctx->device));
    WsGuard g{w->ctx, w->ctx->acquire()};
    if (!g.ws) return jq_fail(jq::E_NOMEM, "jq_matmul_t: no workspace");
    size_t lhs_bytes = align_up(m * k * 4, 256), dst_bytes = m * n * 4;
    JQ_CUDA(g.ws->reserve(lhs_bytes + dst_bytes));
    float* d_lhs = reinterpret_cast<float*>(g.ws->dev);
    float* d_dst = reinterpret_cast<float*>(g.ws->dev + lhs_bytes);
    cudaStream_t s = g.ws->stream;
    JQ_CUDA(cudaMemcpyAsync(d_lhs, lhs, m * k * 4, cudaMemcpyHostToDevice, s));
    if (int32_t rc = jq_matmul_device(w, m, k, n, d_lhs, d_dst, s)) return rc;
    JQ_CUDA(cudaMemcpyAsync(dst, d_dst, dst_bytes, cudaMemcpyDeviceToHost, s));
    JQ_CUDA(cudaStreamSynchronize(s));
    return check_device_status(w->ctx);
}

int32_t jq_matmul_t_f16(const jq_weight* w, uint64_t m, uint64_t k, uint64_t n, const uint16_t* lhs,
                        uint64_t lhs_len, uint16_t* dst, uint64_t dst_len) {
    if (int32_t rc = validate_matmul(w, m, k, n, lhs_len, dst_len, true)) return rc;
    if (m == 0 || n == 0) return jq::OK;
    if (!lhs || !dst) return jq_fail(jq::E_INVALID, "jq_matmul_t_f16: NULL buffer");
    JQ_CUDA(cudaSetDevice(w->ctx->device));
    WsGuard g{w->ctx, w->ctx->acquire()};
    if (!g.ws) return jq_fail(jq::E_NOMEM, "jq_matmul_t_f16: no workspace");
    size_t a = align_up(m * k * 4, 256), b = align_up(m * n * 4, 256), c = align_up(m * k * 2, 256), d = m * n * 2;
    JQ_CUDA(g.ws->reserve(a + b + c + d));
    float* d_lhs = reinterpret_cast<float*>(g.ws->dev);
    float* d_dst = reinterpret_cast<float*>(g.ws->dev + a);
    __half* h_lhs = reinterpret_cast<__half*>(g.ws->dev + a + b);
    __half* h_dst = reinterpret_cast<__half*>(g.ws->dev + a + b + c);
    cudaStream_t s = g.ws->stream;
    JQ_CUDA(cudaMemcpyAsync(h_lhs, lhs, m * k * 2, cudaMemcpyHostToDevice, s));
    f16_to_f32_kernel<<<(unsigned)((m * k + 255) / 256), 256, 0, s>>>(h_lhs, d_lhs, m * k);
    if (int32_t rc = jq_matmul_device(w, m, k, n, d_lhs, d_dst, s)) return rc;
    f32_to_f16_kernel<<<(unsigned)((m * n + 255) / 256), 256, 0, s>>>(d_dst, h_dst, m * n);
    JQ_CUDA(cudaGetLastError());
    JQ_CUDA(cudaMemcpyAsync(dst, h_dst, d, cudaMemcpyDeviceToHost, s));
    JQ_CUDA(cudaStreamSynchronize(s));
    return check_device_status(w->ctx);
}

int32_t jq_dequantize_dev(const jq_weight* w, float* out_dev, uint64_t elem_count, int32_t two_step, void* stream) {
    if (!w) return jq_fail(jq::E_INVALID, "jq_dequantize: NULL weight handle");
    if (elem_count != w->n_blocks * w->fmt.elems)
        return jq_fail(jq::E_INVALID, std::string(jq_type_name(w->type)) + ": output holds " + std::to_string(elem_count) +
                                       " values, expected " + std::to_string(w->n_blocks * w->fmt.elems));
    if (elem_count == 0) return jq::OK;
    if (!out_dev || reinterpret_cast<uintptr_t>(out_dev) % 16 != 0)
        return jq_fail(jq::E_INVALID, "jq_dequantize_dev: output must be a 16-byte aligned device buffer");
    JQ_CUDA(jq::launch_dequant(w->type, w->dev, w->n_blocks, out_dev, two_step != 0,
                               static_cast<cudaStream_t>(stream)));
    return jq::OK;
}

int32_t jq_dequantize(const jq_weight* w, float* out, uint64_t elem_count, int32_t two_step) {
    if (!w) return jq_fail(jq::E_INVALID, "jq_dequantize: NULL weight handle");
    if (elem_count && !out) return jq_fail(jq::E_INVALID, "jq_dequantize: NULL output");
    JQ_CUDA(cudaSetDevice(w->ctx->device));
    WsGuard g{w->ctx, w->ctx->acquire()};
    if (!g.ws) return jq_fail(jq::E_NOMEM, "jq_dequantize: no workspace");
    JQ_CUDA(g.ws->reserve(elem_count * 4 + 16));
    if (int32_t rc = jq_dequantize_dev(w, reinterpret_cast<float*>(g.ws->dev), elem_count, two_step, g.ws->stream))
        return rc;
    if (elem_count == 0) return jq::OK;
    JQ_CUDA(cudaMemcpyAsync(out, g.ws->dev, elem_count * 4, cudaMemcpyDeviceToHost, g.ws->stream));
    JQ_CUDA(cudaStreamSynchronize(g.ws->stream));
    return jq::OK;
}

int32_t jq_embedding(const jq_weight* w, const uint32_t* ids, uint64_t n_ids, uint64_t rows, uint64_t hidden,
                     float* out) {
    if (!w) return jq_fail(jq::E_INVALID, "jq_embedding: NULL weight handle");
    if (hidden % w->fmt.elems != 0)
        return jq_fail(jq::E_INVALID, "quantized embedding hidden size " + std::to_string(hidden) +
                                       " is not divisible by block size " + std::to_string(w->fmt.elems));
    if (w->n_blocks != rows * (hidden / w->fmt.elems))
        return jq_fail(jq::E_INVALID, "quantized tensor has " + std::to_string(w->n_blocks) + " blocks, expected " +
                                       std::to_string(rows * (hidden / w->fmt.elems)));
    if (n_ids == 0) return jq::OK;
    if (!ids || !out) return jq_fail(jq::E_INVALID, "jq_embedding: NULL buffer");
    for (uint64_t i = 0; i < n_ids; ++i)
        if (ids[i] >= rows)
            return jq_fail(jq::E_INVALID, "embedding id " + std::to_string(ids[i]) + " is out of range for " +
                                           std::to_string(rows) + " rows");
    JQ_CUDA(cudaSetDevice(w->ctx->device));
    WsGuard g{w->ctx, w->ctx->acquire()};
    if (!g.ws) return jq_fail(jq::E_NOMEM, "jq_embedding: no workspace");
    size_t out_bytes = align_up(n_ids * hidden * 4, 256);
    JQ_CUDA(g.ws->reserve(out_bytes + n_ids * 4));
    float* d_out = reinterpret_cast<float*>(g.ws->dev);
    uint32_t* d_ids = reinterpret_cast<uint32_t*>(g.ws->dev + out_bytes);
    cudaStream_t s = g.ws->stream;
    JQ_CUDA(cudaMemcpyAsync(d_ids, ids, n_ids * 4, cudaMemcpyHostToDevice, s));
    JQ_CUDA(jq::launch_embedding(w->type, w->dev, rows, hidden, d_ids, n_ids, d_out, g.ws->flag, s));
    JQ_CUDA(cudaMemcpyAsync(out, d_out, n_ids * hidden * 4, cudaMemcpyDeviceToHost, s));
    JQ_CUDA(cudaStreamSynchronize(s));
    return jq::OK;
}

int32_t jq_device_status(const jq_ctx* ctx) {
    if (!ctx) return jq_fail(jq::E_INVALID, "jq_device_status: NULL context");
    return check_device_status(ctx);
}

int32_t jq_weight_from_float(jq_weight*, const float*, uint64_t) {
    return jq_fail(jq::E_INVALID, "cannot quantize into a read-only device-resident tensor");
}

}  // extern "C"
