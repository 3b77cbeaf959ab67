// Shared declarations of the library's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "formats.cuh"

namespace jq {

// Launch with programmatic stream serialization: the kernel may start while its predecessor in the stream
// is still draining; every access that depends on the predecessor sits behind pdl_wait().
template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, unsigned block, size_t smem, cudaStream_t s,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Kernel attributes and device properties are per device: a process may hold contexts on several GPUs, so
// every one-time setup is keyed by the device that is current when it runs.
constexpr int MAX_DEVICES = 64;
inline int current_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev >= 0 && dev < MAX_DEVICES ? dev : 0;
}
inline int num_sms() {
    static int cached[MAX_DEVICES] = {};
    const int dev = current_device();
    if (cached[dev] == 0) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}
// Raises a kernel's dynamic shared-memory limit once per device; `done` is a per-kernel array of MAX_DEVICES flags.
template <class K>
cudaError_t set_max_smem_once(K kern, int bytes, bool* done) {
    const int dev = current_device();
    if (done[dev]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

// Status codes of the C ABI (0 = success, negative = failure), following the
// int32 status / opaque handle convention of the reference's only C ABI
// (src/npu/mod.rs:32-50).
enum : int32_t {
    OK = 0,
    E_INVALID = -1,      // shape / length / alignment / NULL argument
    E_TYPE = -2,         // GGUF type id without a kernel here
    E_CUDA = -3,         // a CUDA runtime call failed
    E_NOMEM = -4,        // device or pinned host allocation failed
    E_EXPERT_RANGE = -5, // router produced an expert id >= n_expert
    E_TOO_LARGE = -6,    // request exceeds a fixed capacity
    E_TIMEOUT = -7,      // a bounded wait inside a kernel gave up
};

// dequant.cu
cudaError_t tables_dequant();
cudaError_t launch_dequant(uint32_t type, const uint8_t* w, uint64_t n_blocks, float* out, bool two_step,
                           cudaStream_t s);
// rows of `hidden` values gathered by id; ids >= rows set *bad_id (device flag) and write nothing
cudaError_t launch_embedding(uint32_t type, const uint8_t* w, uint64_t rows, uint64_t hidden, const uint32_t* ids,
                             uint64_t n_ids, float* out, int* bad_id, cudaStream_t s);

// gemv_f32.cu: exact-decode float path, any m
cudaError_t tables_gemv_f32();
cudaError_t launch_matmul_f32(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                              float* dst, cudaStream_t s);

// gemm_tc.cu: tcgen05 tile GEMM for m > 8 (prefill, batched decode)
cudaError_t tables_gemm_tc();
bool gemm_tc_supports(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, uint64_t m);
// scratch: gemm_tc_scratch_bytes(m, k) bytes (the activations' two TF32 terms), 256-byte aligned
size_t gemm_tc_scratch_bytes(uint64_t m, uint64_t k);
void gemm_tc_set_trace(unsigned long long* dev_buf);  // profiling aid, see gemm_tc.cu
cudaError_t launch_gemm_tc(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                           float* dst, void* scratch, int* error_flag, cudaStream_t s);

// Grouped form for routed experts at prefill sizes: one launch over a device list of tiles, each up to 128
// consecutive rows of the expert-sorted activation matrix x[rows, k] against that expert's slice of a bank
// ([n_expert][n, k] blocks, `expert_bytes` apart).  With `bank_b` / `dst_b` the same activations go through two
// banks in one launch (gate and up).  dst[row, n] is written for the tiles' rows only.  Two lists on the device:
// `narrow` (tiles of at most 32 rows, run as 32-token tiles) and `wide`, their lengths in counts[0] and counts[1]
// (device memory, read by the kernels: the launches cover max_narrow / max_wide entries and the surplus CTAs
// leave at once), so that no host read stands between the routing and the products.  False from
// gemm_tc_grouped_supports = shapes this form does not take (the caller then runs one product per expert).
struct GemmTile {
    uint32_t expert;
    uint32_t row0;  // first row of the tile in x / dst
    uint32_t cnt;   // rows, 1..128
    uint32_t pad;
};
bool gemm_tc_grouped_supports(uint32_t type, const uint8_t* bank, uint64_t n, uint64_t k);
cudaError_t launch_gemm_tc_grouped(uint32_t type, const uint8_t* bank_a, const uint8_t* bank_b, uint64_t expert_bytes,
                                   uint64_t n, uint64_t k, const float* x, uint64_t rows, float* dst_a, float* dst_b,
                                   const GemmTile* narrow, uint32_t max_narrow, const GemmTile* wide, uint32_t max_wide,
                                   const uint32_t* counts, void* scratch, int* error_flag, cudaStream_t s);

// One unit of grouped (MoE) work: up to 8 consecutive positions of the expert-sorted activation list,
// all routed to `expert`.
struct MoeJob {
    uint32_t expert;
    uint32_t row0;  // first position in the list
    uint32_t cnt;   // positions (1..8)
};

// gemv_mma.cu: integer-code tensor-core path for batches 1..GEMV_MMA_MAX_M
constexpr uint64_t GEMV_MMA_MAX_M = 8;
cudaError_t tables_gemv_mma();
// bytes of scratch (activation planes) a launch with these sizes needs
size_t gemv_mma_scratch_bytes(uint64_t m, uint64_t k);
bool gemv_mma_supports(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, uint64_t m);
// error_flag: device int set to 1 if a bounded wait inside the kernel gave up
cudaError_t launch_gemv_mma(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                            float* dst, void* scratch, int* error_flag, cudaStream_t s);
// Fused gate / up pair with the SwiGLU epilogue; valid when gemv_mma_scratch_bytes(m, k) == 0.  With norm_w
// the rows of lhs are RMS-normalised (weights norm_w, epsilon eps) inside the kernel first.
cudaError_t launch_gemv_mma_swiglu(uint32_t type, const uint8_t* w_gate, const uint8_t* w_up, uint64_t n, uint64_t k,
                                   const float* lhs, uint64_t m, float* dst, float clamp, int* error_flag,
                                   cudaStream_t s, const float* norm_w = nullptr, float eps = 0.0f);
// dst = residual + rmsnorm(lhs; norm_w, eps) . W^T in one launch (norm_w, residual optional; residual may be
// dst).  Valid when gemv_mma_fusable(m, k).
bool gemv_mma_fusable(uint64_t m, uint64_t k);
cudaError_t launch_gemv_mma_fused(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs,
                                  uint64_t m, float* dst, const float* norm_w, float eps, const float* residual,
                                  int* error_flag, cudaStream_t s);
// Allocation-free variant: planes in a fixed array inside the library image (see gemv_mma.cu).
constexpr size_t GEMV_STATIC_SCRATCH_BYTES = 4u << 20;
size_t gemv_mma_static_bytes_needed(uint64_t m, uint64_t k);
cudaError_t launch_gemv_mma_static(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs,
                                   uint64_t m, float* dst, int* error_flag, cudaStream_t s);
// f32 rows -> activation planes in `scratch` (gemv_mma_scratch_bytes(rows, k) bytes, for rows that do not fit
// the kernel's shared memory)
cudaError_t launch_quantize_acts(uint32_t type, const float* x, uint64_t rows, uint64_t k, void* scratch,
                                 cudaStream_t s);
// Grouped form: every job multiplies its list positions' activation rows by its expert's [n, k] matrix and
// writes dst[position, n].  With a second bank the two results are combined as silu(clamp(g)) * clamp(u).
struct GroupedLaunch {
    uint32_t type;
    const uint8_t* w0;        // bank of [n_expert][n][k] blocks
    const uint8_t* w1;        // second bank (SwiGLU pair) or NULL
    uint64_t n, k, expert_bytes;
    const float* x;           // activation rows [x_rows, k]
    uint32_t x_rows;
    void* planes;             // pre-split planes of those rows (launch_quantize_acts), or NULL to split in-kernel
    const uint32_t* act_rows; // activation row of each list position, NULL = identity
    const MoeJob* jobs;       // device
    const uint32_t* n_jobs;   // device
    uint32_t max_jobs;        // host bound on *n_jobs (sizes the grid)
    uint32_t rows_per_job;    // host bound on MoeJob::cnt (1, 2, 4 or 8)
    float* dst;
    float clamp;
    int* error_flag;
    const float* norm_w;      // planes == NULL only: RMS-normalise the activation rows with these weights first
    float norm_eps;
};
cudaError_t launch_gemv_grouped(const GroupedLaunch& g, cudaStream_t s);

// moe.cu: routing on the device
enum : int32_t { MOE_GATE_SOFTMAX = 0, MOE_GATE_SIGMOID = 1, MOE_GATE_SQRT_SOFTPLUS = 2 };
struct MoeRouteParams {
    int32_t gating;           // MOE_GATE_*
    uint32_t n_expert, n_used;
    uint32_t n_group, topk_group;
    int32_t norm;             // renormalise the selected weights
    int32_t renorm_plus_eps;  // 0: / max(sum, 6.1035156e-5); 1: / (sum + 1e-20)
    float scale;              // applied when != 0 and != 1
};
cudaError_t launch_moe_logits(const float* x, const float* router, uint32_t T, uint32_t E, uint32_t h, float* logits,
                              cudaStream_t s);
cudaError_t launch_moe_route(const float* logits, const MoeRouteParams& rp, uint32_t T, const float* bias,
                             const uint32_t* forced_ids, uint32_t* ids, float* wts, cudaStream_t s);
cudaError_t launch_moe_jobs(const uint32_t* ids, uint32_t T, uint32_t K, uint32_t E, uint32_t rows_per_job,
                            uint32_t* list_token, uint32_t* inv, MoeJob* jobs, uint32_t* n_jobs, uint32_t* n_list,
                            int* bad_id, cudaStream_t s);
cudaError_t moe_set_trace(unsigned long long* dev_buf);
// xs[pos, :] = x[list_token[pos], :] for pos < min(P, *n_list)
cudaError_t launch_moe_gather(const float* x, const uint32_t* list_token, const uint32_t* n_list, uint32_t P, uint32_t h,
                              float* xs, cudaStream_t s);
// logits + routing (+ job list) in one launch for decode-sized batches; `counter`: a device word that is zero
// between calls.  With norm_w the tokens are RMS-normalised inside the kernel.
cudaError_t launch_moe_route_fused(const float* x, const float* norm_w, float eps, const float* router, uint32_t T,
                                   uint32_t h, float* logits, const MoeRouteParams& rp, const float* bias,
                                   const uint32_t* forced_ids, uint32_t* ids, float* wts, bool do_jobs,
                                   uint32_t rows_per_job, uint32_t* list_token, uint32_t* inv, MoeJob* jobs,
                                   uint32_t* n_jobs, uint32_t* n_list, int* bad_id, uint32_t* counter, cudaStream_t s);
cudaError_t launch_moe_combine(const float* out, const uint32_t* inv, const float* wts, const float* shared, uint32_t T,
                               uint32_t K, uint32_t h, float* y, cudaStream_t s, const float* residual = nullptr);
cudaError_t launch_swiglu(const float* g, const float* u, uint64_t n, float clamp, float* out, cudaStream_t s);
// the same over the first *n_rows (at most max_rows) rows of [rows, inter]
cudaError_t launch_swiglu_rows(const float* g, const float* u, const uint32_t* n_rows, uint32_t max_rows, uint32_t inter,
                               float clamp, float* out, cudaStream_t s);
// work lists of the prefill form from the job list: experts with >= min_rows rows as tiles of the grouped tile GEMM,
// the other experts' jobs copied for the grouped decode kernel;
// counts = {narrow tiles (<= 32 rows), wide tiles, list rows, small jobs}
cudaError_t launch_moe_tiles(const MoeJob* jobs, const uint32_t* n_jobs, const uint32_t* n_list, uint32_t E, uint32_t min_rows,
                             GemmTile* narrow, GemmTile* wide, MoeJob* small_jobs, uint32_t* counts, cudaStream_t s);

// decoder.cu: the element-wise and attention steps around the matmuls of a decode step
cudaError_t launch_rmsnorm(const float* x, const float* res, const float* w, float eps, uint64_t rows, uint32_t h,
                           float* sum_out, float* out, cudaStream_t s, uint32_t x_stride = 0);
cudaError_t launch_mla_assemble(float* q, const float* comp, const float* kv, const int32_t* pos, uint32_t batch,
                                uint32_t nh, uint32_t nope, uint32_t rope, uint32_t vd, uint32_t kv_lora, uint32_t max_ctx,
                                const float* inv_freq, float mscale, float* cache_k, float* cache_v, int32_t* bad_pos,
                                cudaStream_t s);
cudaError_t launch_rope_append(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t nq, uint32_t nkv,
                               uint32_t hd, uint32_t max_ctx, float theta, float* q_out, float* cache_k, float* cache_v,
                               int32_t* bad_pos, cudaStream_t s, uint32_t seq = 0, const float* q_norm = nullptr,
                               const float* k_norm = nullptr, float qk_eps = 0.0f);
// causal attention of `seq` new tokens of one sequence (positions pos[0] ..) over the cache; hd 64 or 128
cudaError_t launch_attention_prefill(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                     uint32_t seq, uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx, float* out,
                                     int32_t* bad_pos, cudaStream_t s);
// rope + cache append + attention + merge in one launch, from the fused qkv row (decoder.cu)
struct AttnArgs;
bool attention_fused_args(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t nq, uint32_t nkv, uint32_t hd,
                          uint32_t max_ctx, float theta, float* cache_k, float* cache_v, float* out, void* scratch,
                          AttnArgs* a);
size_t attention_fused_scratch_bytes(uint32_t batch, uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx);
cudaError_t launch_attention_fused(const float* qkv, const int32_t* pos, uint32_t batch, uint32_t nq, uint32_t nkv,
                                   uint32_t hd, uint32_t max_ctx, float theta, float* cache_k, float* cache_v,
                                   float* out, void* scratch, int32_t* bad_pos, cudaStream_t s,
                                   const float* q_norm = nullptr, const float* k_norm = nullptr, float qk_eps = 0.0f);
// scratch: attention_scratch_bytes(...) bytes of per-chunk partial results
size_t attention_scratch_bytes(uint32_t batch, uint32_t nq, uint32_t hd, uint32_t max_ctx);
cudaError_t launch_attention_decode(const float* q, const float* cache_k, const float* cache_v, const int32_t* pos,
                                    uint32_t batch, uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t max_ctx, float* out,
                                    float* scratch, int32_t* bad_pos, cudaStream_t s, uint32_t dv = 0, float scale = 0.0f);
cudaError_t launch_add(const float* a, const float* b, uint64_t n, float* y, cudaStream_t s);
size_t argmax_scratch_bytes(uint32_t rows);
// greedy token per row; with a window (ids [rows, 64] + state [rows, 2]) and penalty != 1 the reference's
// repetition penalty is applied first and the sampled id is pushed into the window
cudaError_t launch_argmax(const float* logits, uint32_t rows, uint32_t vocab, int32_t* token, int32_t* pos,
                          void* scratch, cudaStream_t s, float penalty = 1.0f, int32_t* window = nullptr,
                          int32_t* win_state = nullptr);

}  // namespace jq
