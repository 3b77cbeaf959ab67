// C ABI of the MoE layer: routing on the device, grouped expert matmuls, weighted combine.
// Declarations and the reference interfaces they replace are in include/joshua_b200.h.
#include "handles.cuh"
#include <algorithm>


namespace {

size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

uint32_t rows_per_job_for(uint64_t pairs, uint64_t tokens, uint32_t n_expert) {
    if (tokens == 1) return 1;
    if (pairs <= n_expert) return 2;
    if (pairs <= 4ull * n_expert) return 4;
    return 8;
}

int32_t reserve(jq_moe* m, uint64_t T, uint64_t P) {
    if (T <= m->cap_tokens && P <= m->cap_pairs) return jq::OK;
    T = std::max(T, m->cap_tokens);
    P = std::max(P, m->cap_pairs);
    const jq_moe_config& c = m->cfg;
    if (m->ws) cudaFree(m->ws);
    m->ws = nullptr;
    m->cap_tokens = m->cap_pairs = 0;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off += up256(bytes);
        return o;
    };
    size_t o_logits = take(T * c.n_expert * 4), o_ids = take(P * 4), o_wts = take(P * 4), o_list = take(P * 4),
           o_inv = take(P * 4), o_jobs = take((P + c.n_expert) * sizeof(jq::MoeJob)), o_nj = take(8),
           o_hidden = take(P * c.inter * 4), o_out = take(P * c.hidden * 4), o_shh = take(T * c.inter * 4 * 3),
           o_sho = take(T * c.hidden * 4), o_ones = take(P * 4), o_xn = take(T * c.hidden * 4),
           o_px = take(jq::gemv_mma_scratch_bytes(T, c.hidden) + (T * (c.hidden / 32) * 112) + 256),
           o_ph = take(jq::gemv_mma_scratch_bytes(P, c.inter) + (P * (c.inter / 32) * 112) + 256);
    JQ_CUDA(cudaMalloc(&m->ws, off));
    uint8_t* b = m->ws;
    m->logits = (float*)(b + o_logits);
    m->ids = (uint32_t*)(b + o_ids);
    m->wts = (float*)(b + o_wts);
    m->list_token = (uint32_t*)(b + o_list);
    m->inv = (uint32_t*)(b + o_inv);
    m->jobs = (jq::MoeJob*)(b + o_jobs);
    m->n_jobs = (uint32_t*)(b + o_nj);
    m->n_list = m->n_jobs + 1;
    m->hidden = (float*)(b + o_hidden);
    m->out = (float*)(b + o_out);
    m->sh_hidden = (float*)(b + o_shh);
    m->sh_out = (float*)(b + o_sho);
    m->ones = (float*)(b + o_ones);
    m->xn = (float*)(b + o_xn);
    m->planes_x = b + o_px;
    m->planes_h = b + o_ph;
    std::vector<float> ones(P, 1.0f);
    JQ_CUDA(cudaMemcpy(m->ones, ones.data(), P * 4, cudaMemcpyHostToDevice));
    m->cap_tokens = T;
    m->cap_pairs = P;
    return jq::OK;
}

bool fits_smem(uint64_t rows, uint64_t k) { return jq::gemv_mma_scratch_bytes(rows, k) == 0; }

// out_list[pos, :] = MLP_expert(pos)(x[list_token[pos], :]) for the list built by the jobs kernel.
// R activation rows, P list positions at most.
// `jobs` / `n_jobs` (device) default to the layer's whole job list; `phases` bit 0 = gate/up, bit 1 = down.
int32_t run_experts(jq_moe* m, const float* x, uint64_t R, uint64_t P, uint32_t rows_per_job, cudaStream_t s,
                    const float* norm_w = nullptr, float eps = 0.0f, const jq::MoeJob* jobs = nullptr,
                    const uint32_t* n_jobs = nullptr, int phases = 3) {
    const jq_moe_config& c = m->cfg;
    jq::GroupedLaunch g = {};
    g.jobs = jobs ? jobs : m->jobs;
    g.n_jobs = n_jobs ? n_jobs : m->n_jobs;
    // a job holds at most rows_per_job positions of one expert
    g.max_jobs = (uint32_t)std::min<uint64_t>(P, P / rows_per_job + c.n_expert);
    g.rows_per_job = rows_per_job;
    g.clamp = c.clamp;
    g.error_flag = m->ctx->status_dev;
    // gate and up with the SwiGLU epilogue: hidden[pos, inter]
    g.type = m->gate->type;
    g.w0 = m->gate->dev;
    g.w1 = m->up->dev;
    g.n = c.inter;
    g.k = c.hidden;
    g.expert_bytes = m->gate_expert_bytes;
    g.x = x;
    g.x_rows = (uint32_t)R;
    g.act_rows = m->list_token;
    g.dst = m->hidden;
    if (phases & 1) {
        if (fits_smem(R, c.hidden)) {
            g.planes = nullptr;
            g.norm_w = norm_w;
            g.norm_eps = eps;
        } else {
            if (norm_w) return jq_fail(jq::E_INVALID, "moe: internal: norm requested for rows that do not fit shared memory");
            JQ_CUDA(jq::launch_quantize_acts(g.type, x, R, c.hidden, m->planes_x, s));
            g.planes = m->planes_x;
        }
        JQ_CUDA(jq::launch_gemv_grouped(g, s));
    }
    if (!(phases & 2)) return jq::OK;
    // down: out[pos, hidden]; activation row = list position
    g.type = m->down->type;
    g.w0 = m->down->dev;
    g.w1 = nullptr;
    g.n = c.hidden;
    g.k = c.inter;
    g.expert_bytes = m->down_expert_bytes;
    g.x = m->hidden;
    g.x_rows = (uint32_t)P;
    g.act_rows = nullptr;
    g.dst = m->out;
    g.clamp = 0.0f;
    g.norm_w = nullptr;
    if (fits_smem(P, c.inter)) {
        g.planes = nullptr;
    } else {
        JQ_CUDA(jq::launch_quantize_acts(g.type, m->hidden, P, c.inter, m->planes_h, s));
        g.planes = m->planes_h;
    }
    JQ_CUDA(jq::launch_gemv_grouped(g, s));
    return jq::OK;
}

// sh_out[T, hidden] = shared expert MLP over all tokens
// The prefill form of the expert MLPs, as the reference buckets tokens per expert and runs one matmul per
// bucket (src/quantized_qwen3_moe.rs:455-520): when an expert sees dozens of rows, its rows are gathered into
// bucket order and the experts' gate / up / down products run on the tile GEMM (tensor cores), as one grouped
// launch per phase over a list of (expert, row range) tiles built on the device.
constexpr uint64_t BUCKET_ROWS_PER_EXPERT = 12;  // rows from which an expert runs on the tile GEMM
constexpr uint64_t BUCKET_MIN_TOKENS = 128;      // tokens from which the prefill form (tile GEMM + decode kernel) is used

int32_t run_experts_bucketed(jq_moe* m, const float* x, uint64_t T, uint64_t P, uint32_t rows_per_job, cudaStream_t s) {
    const jq_moe_config& c = m->cfg;
    if (P > m->bucket_pairs) {
        if (m->bucket) cudaFree(m->bucket);
        m->bucket = nullptr;
        m->bucket_pairs = 0;
        JQ_CUDA(cudaMalloc(&m->bucket, (P * c.hidden + 2 * P * c.inter) * sizeof(float)));
        m->bucket_pairs = P;
    }
    float* xs = m->bucket;
    float* gbuf = xs + P * c.hidden;
    float* ubuf = gbuf + P * c.inter;
    // Usual form, all on the device (`moe_tiles_kernel`): an expert with at least BUCKET_ROWS_PER_EXPERT rows has
    // them cut into tiles of up to 128 rows and runs on the tile GEMM, one grouped launch per phase and tile class
    // (gate and up together, then down); the other experts' jobs run on the grouped decode kernel in the same pass.
    // No host read: the launches cover the lists' capacity and the kernels read their lengths.
    if (jq::gemm_tc_grouped_supports(m->gate->type, m->gate->dev, c.inter, c.hidden) && m->up->type == m->gate->type &&
        jq::gemm_tc_grouped_supports(m->down->type, m->down->dev, c.hidden, c.inter) && P / 33 + 1 <= 65535) {
        // a narrow tile (<= 32 rows) is an expert's only tile (>= min rows) or the last piece behind full tiles; a wide
        // tile holds more than 32 rows
        // With 24 or more rows per expert on average hardly an expert is small: every expert then takes the tile
        // form (an expert with a few rows is one narrow tile) and the decode kernel's passes are left out.
        const bool all_tiles = P >= 24ull * c.n_expert;
        const uint32_t min_rows = all_tiles ? 1u : (uint32_t)BUCKET_ROWS_PER_EXPERT;
        const uint32_t max_narrow = (uint32_t)std::min<uint64_t>(c.n_expert, P / min_rows + 1);
        const uint32_t max_wide = (uint32_t)(P / 33 + 1);
        const uint32_t max_small = (uint32_t)std::min<uint64_t>(P, P / rows_per_job + c.n_expert);
        const uint64_t need_bytes = ((uint64_t)max_narrow + max_wide) * sizeof(jq::GemmTile) + (uint64_t)max_small * sizeof(jq::MoeJob) + 32;
        if (need_bytes > m->tiles_cap) {
            if (m->tiles) cudaFree(m->tiles);
            m->tiles = nullptr;
            m->tiles_cap = 0;
            JQ_CUDA(cudaMalloc(&m->tiles, need_bytes));
            m->tiles_cap = need_bytes;
        }
        jq::GemmTile* narrow = m->tiles;
        jq::GemmTile* wide = narrow + max_narrow;
        jq::MoeJob* small_jobs = reinterpret_cast<jq::MoeJob*>(wide + max_wide);
        // {narrow tiles, wide tiles, list rows, small jobs}, 16-byte aligned behind the lists
        uint32_t* counts = reinterpret_cast<uint32_t*>(
            (reinterpret_cast<uintptr_t>(small_jobs + max_small) + 15) & ~(uintptr_t)15);
        void* scratch = nullptr;
        const size_t need = std::max(jq::gemm_tc_scratch_bytes(P, c.hidden), jq::gemm_tc_scratch_bytes(P, c.inter));
        JQ_CUDA(m->ctx->scratch_for(reinterpret_cast<cudaStream_t>(reinterpret_cast<uintptr_t>(s) ^ 3), need, &scratch));
        JQ_CUDA(jq::launch_moe_gather(x, m->list_token, m->n_list, (uint32_t)P, c.hidden, xs, s));
        JQ_CUDA(jq::launch_moe_tiles(m->jobs, m->n_jobs, m->n_list, c.n_expert, min_rows, narrow, wide, small_jobs, counts, s));
        JQ_CUDA(jq::launch_gemm_tc_grouped(m->gate->type, m->gate->dev, m->up->dev, m->gate_expert_bytes, c.inter, c.hidden, xs, P,
                                           gbuf, ubuf, narrow, max_narrow, wide, max_wide, counts, scratch, m->ctx->status_dev, s));
        // SwiGLU over every list row (rows of the small experts hold nothing yet; the decode kernel writes them next)
        JQ_CUDA(jq::launch_swiglu_rows(gbuf, ubuf, counts + 2, (uint32_t)P, c.inter, c.clamp, m->hidden, s));
        if (!all_tiles)
            if (int32_t rc = run_experts(m, x, T, P, rows_per_job, s, nullptr, 0.0f, small_jobs, counts + 3, 1)) return rc;
        JQ_CUDA(jq::launch_gemm_tc_grouped(m->down->type, m->down->dev, nullptr, m->down_expert_bytes, c.hidden, c.inter,
                                           m->hidden, P, m->out, nullptr, narrow, max_narrow, wide, max_wide, counts, scratch,
                                           m->ctx->status_dev, s));
        return all_tiles ? jq::OK : run_experts(m, x, T, P, rows_per_job, s, nullptr, 0.0f, small_jobs, counts + 3, 2);
    }
    // Shapes the grouped form does not take: the job list is read back to the host (which synchronises the stream)
    // and every expert's bucket is one batched matmul.
    uint32_t n_jobs = 0;
    JQ_CUDA(cudaMemcpyAsync(&n_jobs, m->n_jobs, sizeof(n_jobs), cudaMemcpyDeviceToHost, s));
    JQ_CUDA(cudaStreamSynchronize(s));
    std::vector<jq::MoeJob> jobs(n_jobs);
    if (n_jobs) JQ_CUDA(cudaMemcpyAsync(jobs.data(), m->jobs, n_jobs * sizeof(jq::MoeJob), cudaMemcpyDeviceToHost, s));
    JQ_CUDA(jq::launch_moe_gather(x, m->list_token, m->n_list, (uint32_t)P, c.hidden, xs, s));
    JQ_CUDA(cudaStreamSynchronize(s));
    // consecutive jobs of one expert form its bucket
    struct Bucket {
        uint32_t expert, row0, cnt;
    };
    std::vector<Bucket> buckets;
    for (const jq::MoeJob& j : jobs) {
        if (!buckets.empty() && buckets.back().expert == j.expert && buckets.back().row0 + buckets.back().cnt == j.row0)
            buckets.back().cnt += j.cnt;
        else
            buckets.push_back({j.expert, j.row0, j.cnt});
    }
    auto slice = [&](const jq_weight* bank, uint64_t expert_bytes, uint32_t e) {
        jq_weight w = *bank;
        w.dev = bank->dev + (uint64_t)e * expert_bytes;
        w.n_blocks = expert_bytes / bank->fmt.bytes;
        w.owns = false;
        return w;
    };
    // One expert's product fills only a fraction of the GPU (n / 128 CTAs), so the buckets are dealt to eight
    // auxiliary streams that fork from and join the caller's stream around each phase.
    constexpr int NAUX = 8;
    jq_ctx* cx = m->ctx;
    std::lock_guard<std::mutex> aux_lock(cx->aux_mu);
    if (!cx->fork_ev) {
        JQ_CUDA(cudaEventCreateWithFlags(&cx->fork_ev, cudaEventDisableTiming));
        for (int i = 0; i < NAUX; ++i) {
            JQ_CUDA(cudaStreamCreateWithFlags(&cx->aux[i], cudaStreamNonBlocking));
            JQ_CUDA(cudaEventCreateWithFlags(&cx->join_ev[i], cudaEventDisableTiming));
        }
    }
    auto fork = [&]() -> cudaError_t {
        cudaError_t e = cudaEventRecord(cx->fork_ev, s);
        for (int i = 0; i < NAUX && e == cudaSuccess; ++i) e = cudaStreamWaitEvent(cx->aux[i], cx->fork_ev, 0);
        return e;
    };
    auto join = [&]() -> cudaError_t {
        cudaError_t e = cudaSuccess;
        for (int i = 0; i < NAUX && e == cudaSuccess; ++i) {
            e = cudaEventRecord(cx->join_ev[i], cx->aux[i]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(s, cx->join_ev[i], 0);
        }
        return e;
    };
    // A failure between fork and join must still join: the caller's stream has to wait for whatever the
    // auxiliary streams were already given before it (or the next layer) reuses the buffers.
    int32_t first_rc = jq::OK;
    JQ_CUDA(fork());
    for (size_t bi = 0; bi < buckets.size() && first_rc == jq::OK; ++bi) {
        const Bucket& b = buckets[bi];
        cudaStream_t as = cx->aux[bi % NAUX];
        const jq_weight wg = slice(m->gate, m->gate_expert_bytes, b.expert), wu = slice(m->up, m->gate_expert_bytes, b.expert);
        first_rc = jq_matmul_device(&wg, b.cnt, c.hidden, c.inter, xs + (uint64_t)b.row0 * c.hidden,
                                    gbuf + (uint64_t)b.row0 * c.inter, as);
        if (first_rc == jq::OK)
            first_rc = jq_matmul_device(&wu, b.cnt, c.hidden, c.inter, xs + (uint64_t)b.row0 * c.hidden,
                                        ubuf + (uint64_t)b.row0 * c.inter, as);
    }
    JQ_CUDA(join());
    if (first_rc != jq::OK) return first_rc;
    uint64_t live = 0;
    for (const Bucket& b : buckets) live = std::max<uint64_t>(live, (uint64_t)b.row0 + b.cnt);
    if (live) JQ_CUDA(jq::launch_swiglu(gbuf, ubuf, live * c.inter, c.clamp, m->hidden, s));
    JQ_CUDA(fork());
    for (size_t bi = 0; bi < buckets.size() && first_rc == jq::OK; ++bi) {
        const Bucket& b = buckets[bi];
        const jq_weight wd = slice(m->down, m->down_expert_bytes, b.expert);
        first_rc = jq_matmul_device(&wd, b.cnt, c.inter, c.hidden, m->hidden + (uint64_t)b.row0 * c.inter,
                                    m->out + (uint64_t)b.row0 * c.hidden, cx->aux[bi % NAUX]);
    }
    JQ_CUDA(join());
    if (first_rc != jq::OK) return first_rc;
    (void)T;
    return jq::OK;
}

bool shared_mma_ok(jq_moe* m, uint64_t T) {
    const jq_moe_config& c = m->cfg;
    return T <= 8 && !m->ctx->force_f32 &&
           jq::gemv_mma_supports(m->sh_gate->type, m->sh_gate->dev, c.inter, c.hidden, T) &&
           jq::gemv_mma_supports(m->sh_down->type, m->sh_down->dev, c.hidden, c.inter, T) &&
           fits_smem(T, c.hidden) && fits_smem(T, c.inter) && m->sh_gate->type == m->sh_up->type;
}

int32_t run_shared(jq_moe* m, const float* x, uint64_t T, cudaStream_t s, const float* norm_w = nullptr, float eps = 0.0f) {
    const jq_moe_config& c = m->cfg;
    const bool mma_ok = T <= 8 && !m->ctx->force_f32 &&
                        jq::gemv_mma_supports(m->sh_gate->type, m->sh_gate->dev, c.inter, c.hidden, T) &&
                        jq::gemv_mma_supports(m->sh_down->type, m->sh_down->dev, c.hidden, c.inter, T) &&
                        fits_smem(T, c.hidden) && fits_smem(T, c.inter) && m->sh_gate->type == m->sh_up->type;
    if (mma_ok) {
        jq::GroupedLaunch g = {};
        g.jobs = m->dense_jobs + (T - 1);
        g.n_jobs = m->one;
        g.max_jobs = 1;
        g.rows_per_job = (uint32_t)T;
        g.clamp = c.clamp;
        g.error_flag = m->ctx->status_dev;
        g.type = m->sh_gate->type;
        g.w0 = m->sh_gate->dev;
        g.w1 = m->sh_up->dev;
        g.n = c.inter;
        g.k = c.hidden;
        g.x = x;
        g.x_rows = (uint32_t)T;
        g.dst = m->sh_hidden;
        g.norm_w = norm_w;
        g.norm_eps = eps;
        JQ_CUDA(jq::launch_gemv_grouped(g, s));
        g.norm_w = nullptr;
        g.type = m->sh_down->type;
        g.w0 = m->sh_down->dev;
        g.w1 = nullptr;
        g.n = c.hidden;
        g.k = c.inter;
        g.x = m->sh_hidden;
        g.dst = m->sh_out;
        g.clamp = 0.0f;
        JQ_CUDA(jq::launch_gemv_grouped(g, s));
        return jq::OK;
    }
    float* gbuf = m->sh_hidden + T * c.inter;
    float* ubuf = gbuf + T * c.inter;
    if (int32_t rc = jq_matmul_device(m->sh_gate, T, c.hidden, c.inter, x, gbuf, s)) return rc;
    if (int32_t rc = jq_matmul_device(m->sh_up, T, c.hidden, c.inter, x, ubuf, s)) return rc;
    JQ_CUDA(jq::launch_swiglu(gbuf, ubuf, T * c.inter, c.clamp, m->sh_hidden, s));
    return jq_matmul_device(m->sh_down, T, c.inter, c.hidden, m->sh_hidden, m->sh_out, s);
}

int32_t check_bank(const char* name, const jq_weight* w, uint64_t experts, uint64_t rows, uint64_t cols,
                   uint64_t* expert_bytes) {
    if (!w) return jq_fail(jq::E_INVALID, std::string("jq_moe_create: NULL ") + name + " bank");
    if (cols % w->fmt.elems != 0)
        return jq_fail(jq::E_INVALID, std::string("jq_moe_create: ") + name + " width " + std::to_string(cols) +
                                          " is not a multiple of the block size " + std::to_string(w->fmt.elems));
    uint64_t per = rows * (cols / w->fmt.elems);
    if (w->n_blocks != experts * per)
        return jq_fail(jq::E_INVALID, std::string("jq_moe_create: ") + name + " bank holds " +
                                          std::to_string(w->n_blocks) + " blocks, expected " +
                                          std::to_string(experts * per));
    if (expert_bytes) *expert_bytes = per * w->fmt.bytes;
    return jq::OK;
}

}  // namespace

// Expert MLPs over rows with one expert id each, left in expert-sorted list order: row r's output is
// m->out[m->inv[r], :] (inv = 0xFFFFFFFF for an id out of range).  Arguments are checked by the callers.
uint32_t jq_moe_rows_per_job(uint64_t live_rows, uint32_t n_expert) {
    // up to 16 rows (one or two sequences per rank of an expert-parallel step) few rows share an expert, and the
    // one-row form of the decode kernel is the faster one (a shared expert then is two jobs)
    return rows_per_job_for(live_rows, live_rows <= 16 ? 1 : 2, n_expert);
}

int32_t jq_moe_experts_list(jq_moe* m, const float* x_dev, uint64_t n_rows, const uint32_t* expert_ids_dev,
                            uint64_t live_rows, cudaStream_t s) {
    const jq_moe_config& c = m->cfg;
    uint32_t rpj = jq_moe_rows_per_job(live_rows, c.n_expert);
    JQ_CUDA(jq::launch_moe_jobs(expert_ids_dev, (uint32_t)n_rows, 1, c.n_expert, rpj, m->list_token, m->inv, m->jobs,
                                m->n_jobs, m->n_list, m->bad_dev, s));
    if (!m->ctx->force_f32 && live_rows >= BUCKET_MIN_TOKENS) return run_experts_bucketed(m, x_dev, n_rows, n_rows, rpj, s);
    m->last_rows = m->last_pairs = n_rows, m->last_rpj = rpj;
    return run_experts(m, x_dev, n_rows, n_rows, rpj, s);
}

extern "C" {

int32_t jq_moe_create(jq_ctx* ctx, const jq_moe_config* cfg, const float* router, const float* bias,
                      const jq_weight* gate, const jq_weight* up, const jq_weight* down, const jq_weight* sh_gate,
                      const jq_weight* sh_up, const jq_weight* sh_down, jq_moe** out) {
    if (!ctx || !cfg || !router || !out) return jq_fail(jq::E_INVALID, "jq_moe_create: NULL argument");
    *out = nullptr;
    const jq_moe_config& c = *cfg;
    if (c.n_expert == 0 || c.n_used == 0 || c.n_used > c.n_expert || c.n_expert > 512)
        return jq_fail(jq::E_INVALID, "jq_moe_create: need 0 < n_used <= n_expert <= 512");
    if (c.gating < 0 || c.gating > 2) return jq_fail(jq::E_INVALID, "jq_moe_create: unknown gating function");
    if (c.hidden % 256 || c.inter % 256)
        return jq_fail(jq::E_INVALID, "jq_moe_create: hidden and inter must be multiples of 256");
    if (c.n_group > 1 && (c.n_expert % c.n_group || c.topk_group == 0 || c.topk_group > c.n_group || c.n_group > 64))
        return jq_fail(jq::E_INVALID, "jq_moe_create: bad expert group settings");
    uint64_t geb = 0, ueb = 0, deb = 0;
    const bool router_only = !gate && !up && !down;  // expert-parallel callers route here and compute elsewhere
    if (router_only) {
        if (sh_gate || sh_up || sh_down)
            return jq_fail(jq::E_INVALID, "jq_moe_create: a router-only layer takes no shared expert");
    } else {
    if (int32_t rc = check_bank("gate", gate, c.n_expert, c.inter, c.hidden, &geb)) return rc;
    if (int32_t rc = check_bank("up", up, c.n_expert, c.inter, c.hidden, &ueb)) return rc;
    if (int32_t rc = check_bank("down", down, c.n_expert, c.hidden, c.inter, &deb)) return rc;
    if (gate->type != up->type) return jq_fail(jq::E_INVALID, "jq_moe_create: gate and up banks differ in type");
    if (!jq::gemv_mma_supports(gate->type, gate->dev, c.inter, c.hidden, 1) ||
        !jq::gemv_mma_supports(up->type, up->dev, c.inter, c.hidden, 1) ||
        !jq::gemv_mma_supports(down->type, down->dev, c.hidden, c.inter, 1))
        return jq_fail(jq::E_INVALID, "jq_moe_create: expert banks are not aligned for the grouped kernel");
    }
    if (sh_gate || sh_up || sh_down) {
        if (int32_t rc = check_bank("shared gate", sh_gate, 1, c.inter, c.hidden, nullptr)) return rc;
        if (int32_t rc = check_bank("shared up", sh_up, 1, c.inter, c.hidden, nullptr)) return rc;
        if (int32_t rc = check_bank("shared down", sh_down, 1, c.hidden, c.inter, nullptr)) return rc;
    }
    JQ_CUDA(cudaSetDevice(ctx->device));
    jq_moe* m = new (std::nothrow) jq_moe();
    if (!m) return jq_fail(jq::E_NOMEM, "jq_moe_create: out of host memory");
    m->ctx = ctx;
    m->cfg = c;
    m->rp = {c.gating, c.n_expert, c.n_used, c.n_group ? c.n_group : 1, c.topk_group ? c.topk_group : 1,
             c.norm, c.renorm_plus_eps, c.scale};
    m->gate = gate, m->up = up, m->down = down, m->sh_gate = sh_gate, m->sh_up = sh_up, m->sh_down = sh_down;
    m->gate_expert_bytes = geb;
    m->down_expert_bytes = deb;
    cudaError_t e = cudaMalloc(&m->router, (size_t)c.n_expert * c.hidden * 4);
    if (e == cudaSuccess) e = cudaMemcpy(m->router, router, (size_t)c.n_expert * c.hidden * 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess && bias) {
        e = cudaMalloc(&m->bias, c.n_expert * 4);
        if (e == cudaSuccess) e = cudaMemcpy(m->bias, bias, c.n_expert * 4, cudaMemcpyHostToDevice);
    }
    jq::MoeJob dj[8];
    for (uint32_t i = 0; i < 8; ++i) dj[i] = {0u, 0u, i + 1};
    uint32_t one = 1;
    if (e == cudaSuccess) e = cudaMalloc(&m->dense_jobs, sizeof(dj));
    if (e == cudaSuccess) e = cudaMemcpy(m->dense_jobs, dj, sizeof(dj), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&m->one, 256);
    if (e == cudaSuccess) e = cudaMemset(m->one, 0, 256);
    if (e == cudaSuccess) e = cudaMemcpy(m->one, &one, 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) m->counter = m->one + 16;
    if (e == cudaSuccess) e = cudaHostAlloc(&m->bad_host, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(&m->bad_dev, m->bad_host, 0);
    if (e != cudaSuccess) {
        jq_moe_free(m);
        return jq_fail_cuda(e, "jq_moe_create");
    }
    *m->bad_host = 0;
    *out = m;
    return jq::OK;
}

void jq_moe_free(jq_moe* m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    cudaDeviceSynchronize();
    cudaFree(m->router);
    cudaFree(m->bias);
    cudaFree(m->ws);
    cudaFree(m->bucket);
    cudaFree(m->tiles);
    cudaFree(m->dense_jobs);
    cudaFree(m->one);
    if (m->bad_host) cudaFreeHost(m->bad_host);
    delete m;
}

int32_t jq_moe_reserve(jq_moe* m, uint64_t n_tokens, uint64_t n_rows) {
    if (!m) return jq_fail(jq::E_INVALID, "jq_moe_reserve: NULL handle");
    std::lock_guard<std::mutex> g(m->mu);
    JQ_CUDA(cudaSetDevice(m->ctx->device));
    return reserve(m, std::max<uint64_t>(n_tokens, n_rows), std::max<uint64_t>(n_tokens * m->cfg.n_used, n_rows));
}

int32_t jq_moe_route_dev(jq_moe* m, const float* x_dev, uint64_t T, const uint32_t* forced_ids_dev,
                         uint32_t* ids_dev, float* wts_dev, void* stream) {
    return jq_moe_route_norm_dev(m, x_dev, T, nullptr, 0.0f, forced_ids_dev, ids_dev, wts_dev, stream);
}

// Routing of rmsnorm(x; norm_w, eps) (norm_w NULL: of x).  Up to eight tokens fold the norm into the router kernel.
int32_t jq_moe_route_norm_dev(jq_moe* m, const float* x_dev, uint64_t T, const float* norm_w_dev, float eps,
                              const uint32_t* forced_ids_dev, uint32_t* ids_dev, float* wts_dev, void* stream) {
    if (!m) return jq_fail(jq::E_INVALID, "jq_moe_route_dev: NULL handle");
    if (T == 0) return jq::OK;
    if (!x_dev || !ids_dev || !wts_dev) return jq_fail(jq::E_INVALID, "jq_moe_route_dev: NULL buffer");
    if (T > m->cap_tokens) return jq_fail(jq::E_TOO_LARGE, "jq_moe_route_dev: call jq_moe_reserve for this many tokens first");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const jq_moe_config& c = m->cfg;
    if (T <= 8 && c.hidden % 4 == 0) {
        JQ_CUDA(jq::launch_moe_route_fused(x_dev, norm_w_dev, eps, m->router, (uint32_t)T, c.hidden, m->logits, m->rp,
                                           m->bias, forced_ids_dev, ids_dev, wts_dev, false, 1, nullptr, nullptr, nullptr,
                                           nullptr, nullptr, nullptr, m->counter, s));
        return jq::OK;
    }
    if (norm_w_dev) {
        if (!m->xn) return jq_fail(jq::E_TOO_LARGE, "jq_moe_route_norm_dev: call jq_moe_reserve first");
        JQ_CUDA(jq::launch_rmsnorm(x_dev, nullptr, norm_w_dev, eps, T, c.hidden, nullptr, m->xn, s));
        x_dev = m->xn;
    }
    JQ_CUDA(jq::launch_moe_logits(x_dev, m->router, (uint32_t)T, c.n_expert, c.hidden, m->logits, s));
    JQ_CUDA(jq::launch_moe_route(m->logits, m->rp, (uint32_t)T, m->bias, forced_ids_dev, ids_dev, wts_dev, s));
    return jq::OK;
}

int32_t jq_moe_experts_dev(jq_moe* m, const float* x_dev, uint64_t n_rows, const uint32_t* expert_ids_dev,
                           float* out_dev, void* stream) {
    if (!m) return jq_fail(jq::E_INVALID, "jq_moe_experts_dev: NULL handle");
    if (n_rows == 0) return jq::OK;
    if (!x_dev || !expert_ids_dev || !out_dev) return jq_fail(jq::E_INVALID, "jq_moe_experts_dev: NULL buffer");
    if (!m->gate) return jq_fail(jq::E_INVALID, "jq_moe_experts_dev: this layer was created without expert banks");
    if (n_rows > m->cap_tokens || n_rows > m->cap_pairs)
        return jq_fail(jq::E_TOO_LARGE, "jq_moe_experts_dev: call jq_moe_reserve for this many rows first");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int32_t rc = jq_moe_experts_list(m, x_dev, n_rows, expert_ids_dev, n_rows, s)) return rc;
    // back to row order: out[r] = out_list[inv[r]] (rows with an id out of range come back as zeros)
    JQ_CUDA(jq::launch_moe_combine(m->out, m->inv, m->ones, nullptr, (uint32_t)n_rows, 1, m->cfg.hidden, out_dev, s));
    return jq::OK;
}

int32_t jq_moe_forward_dev(jq_moe* m, const float* x_dev, uint64_t T, const uint32_t* forced_ids_dev, float* y_dev,
                           void* stream) {
    return jq_moe_forward_add_dev(m, x_dev, T, forced_ids_dev, nullptr, y_dev, stream);
}

int32_t jq_moe_forward_add_dev(jq_moe* m, const float* x_dev, uint64_t T, const uint32_t* forced_ids_dev,
                               const float* residual_dev, float* y_dev, void* stream) {
    return jq_moe_forward_norm_add_dev(m, x_dev, T, forced_ids_dev, nullptr, 0.0f, residual_dev, y_dev, stream);
}

int32_t jq_moe_forward_norm_add_dev(jq_moe* m, const float* x_dev, uint64_t T, const uint32_t* forced_ids_dev,
                                    const float* norm_w_dev, float eps, const float* residual_dev, float* y_dev,
                                    void* stream) {
    if (!m) return jq_fail(jq::E_INVALID, "jq_moe_forward_dev: NULL handle");
    if (T == 0) return jq::OK;
    if (!x_dev || !y_dev) return jq_fail(jq::E_INVALID, "jq_moe_forward_dev: NULL buffer");
    const jq_moe_config& c = m->cfg;
    const uint64_t P = T * c.n_used;
    if (!m->gate) return jq_fail(jq::E_INVALID, "jq_moe_forward_dev: this layer was created without expert banks");
    if (T > m->cap_tokens || P > m->cap_pairs)
        return jq_fail(jq::E_TOO_LARGE, "jq_moe_forward_dev: call jq_moe_reserve for this many tokens first");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint32_t rpj = rows_per_job_for(P, T, c.n_expert);
    // Decode-sized batches: router, routing and job list in one launch, the RMS norm folded into it and into
    // the expert (and shared-expert) matmuls' activation split.
    const bool fused = T <= 8 && fits_smem(T, c.hidden) && (!m->sh_gate || shared_mma_ok(m, T));
    const float* x_in = x_dev;
    const float* nw = norm_w_dev;
    if (!fused && norm_w_dev) {
        JQ_CUDA(jq::launch_rmsnorm(x_dev, nullptr, norm_w_dev, eps, T, c.hidden, nullptr, m->xn, s));
        x_in = m->xn;
        nw = nullptr;
    }
    if (fused) {
        JQ_CUDA(jq::launch_moe_route_fused(x_in, nw, eps, m->router, (uint32_t)T, c.hidden, m->logits, m->rp, m->bias,
                                           forced_ids_dev, m->ids, m->wts, true, rpj, m->list_token, m->inv, m->jobs,
                                           m->n_jobs, m->n_list, m->bad_dev, m->counter, s));
    } else {
        if (int32_t rc = jq_moe_route_dev(m, x_in, T, forced_ids_dev, m->ids, m->wts, stream)) return rc;
        JQ_CUDA(jq::launch_moe_jobs(m->ids, (uint32_t)T, c.n_used, c.n_expert, rpj, m->list_token, m->inv, m->jobs,
                                    m->n_jobs, m->n_list, m->bad_dev, s));
    }
    // From BUCKET_MIN_TOKENS tokens on, the prefill form: experts with at least BUCKET_ROWS_PER_EXPERT rows on the
    // tile GEMM, the others on the grouped decode kernel, decided per expert on the device.  Measured crossovers of
    // the two kernels (uniform routing): 128 Q4_K experts of 2048 x 768 between 8 and 16 rows per expert (tile GEMM /
    // decode kernel 0.91 / 0.68 ms at 8, 0.78 / 1.13 ms at 16), 384 MXFP4 experts of 7168 x 2048 near 11
    // (20.8 / 19.2 ms), 256 IQ2_XXS experts of the same shape above 8 (13.3 / 9.2 ms).
    uint64_t min_tokens = BUCKET_MIN_TOKENS;
#ifdef JQ_PROFILING
    if (const char* thr_env = std::getenv("JQ_MOE_BUCKET_TOKENS")) min_tokens = std::strtoull(thr_env, nullptr, 10);  // measurement switch
#endif
    const bool bucketed = !fused && !m->ctx->force_f32 && T >= min_tokens;
    if (bucketed) {
        if (int32_t rc = run_experts_bucketed(m, x_in, T, P, rpj, s)) return rc;
    } else {
        m->last_rows = T, m->last_pairs = P, m->last_rpj = rpj;
        if (int32_t rc = run_experts(m, x_in, T, P, rpj, s, nw, eps)) return rc;
    }
    const float* shared = nullptr;
    if (m->sh_gate) {
        if (int32_t rc = run_shared(m, x_in, T, s, nw, eps)) return rc;
        shared = m->sh_out;
    }
    JQ_CUDA(jq::launch_moe_combine(m->out, m->inv, m->wts, shared, (uint32_t)T, c.n_used, c.hidden, y_dev, s, residual_dev));
    return jq::OK;
}

int32_t jq_moe_experts_replay_dev(jq_moe* m, const float* x_dev, void* stream) {
    if (!m || !x_dev) return jq_fail(jq::E_INVALID, "jq_moe_experts_replay_dev: NULL argument");
    if (!m->gate || m->last_rpj == 0)
        return jq_fail(jq::E_INVALID, "jq_moe_experts_replay_dev: no decode-sized call has left a job list on this layer");
    return run_experts(m, x_dev, m->last_rows, m->last_pairs, m->last_rpj, static_cast<cudaStream_t>(stream));
}

#ifdef JQ_PROFILING
int32_t jq_debug_moe_trace(uint64_t* trace_dev) {
    JQ_CUDA(jq::moe_set_trace(reinterpret_cast<unsigned long long*>(trace_dev)));
    return jq::OK;
}
#endif

int32_t jq_moe_status(jq_moe* m) {
    if (!m) return jq_fail(jq::E_INVALID, "jq_moe_status: NULL handle");
    if (*static_cast<volatile int*>(m->bad_host) != 0) {
        *m->bad_host = 0;
        if (m->cfg.oob_policy == 0)
            return jq_fail(jq::E_EXPERT_RANGE, "moe: router selected an expert id out of " +
                                                   std::to_string(m->cfg.n_expert));
    }
    return jq_device_status(m->ctx);
}

int32_t jq_moe_forward(jq_moe* m, const float* x, uint64_t T, const uint32_t* forced_ids, float* y) {
    if (!m) return jq_fail(jq::E_INVALID, "jq_moe_forward: NULL handle");
    if (T == 0) return jq::OK;
    if (!x || !y) return jq_fail(jq::E_INVALID, "jq_moe_forward: NULL buffer");
    std::lock_guard<std::mutex> g(m->mu);
    JQ_CUDA(cudaSetDevice(m->ctx->device));
    const jq_moe_config& c = m->cfg;
    if (int32_t rc = reserve(m, T, T * c.n_used)) return rc;
    Workspace* ws = m->ctx->acquire();
    if (!ws) return jq_fail(jq::E_NOMEM, "jq_moe_forward: no workspace");
    struct Rel {
        jq_ctx* c;
        Workspace* w;
        ~Rel() { c->release(w); }
    } rel{m->ctx, ws};
    size_t xb = up256(T * c.hidden * 4), fb = up256(T * c.n_used * 4);
    JQ_CUDA(ws->reserve(2 * xb + fb));
    float* d_x = reinterpret_cast<float*>(ws->dev);
    float* d_y = reinterpret_cast<float*>(ws->dev + xb);
    uint32_t* d_f = reinterpret_cast<uint32_t*>(ws->dev + 2 * xb);
    cudaStream_t s = ws->stream;
    JQ_CUDA(cudaMemcpyAsync(d_x, x, T * c.hidden * 4, cudaMemcpyHostToDevice, s));
    if (forced_ids) JQ_CUDA(cudaMemcpyAsync(d_f, forced_ids, T * c.n_used * 4, cudaMemcpyHostToDevice, s));
    if (int32_t rc = jq_moe_forward_dev(m, d_x, T, forced_ids ? d_f : nullptr, d_y, s)) return rc;
    JQ_CUDA(cudaMemcpyAsync(y, d_y, T * c.hidden * 4, cudaMemcpyDeviceToHost, s));
    JQ_CUDA(cudaStreamSynchronize(s));
    return jq_moe_status(m);
}

int32_t jq_moe_last_routing(jq_moe* m, uint64_t T, uint32_t* ids, float* wts) {
    if (!m || !ids || !wts) return jq_fail(jq::E_INVALID, "jq_moe_last_routing: NULL argument");
    if (T * m->cfg.n_used > m->cap_pairs) return jq_fail(jq::E_INVALID, "jq_moe_last_routing: no such forward");
    JQ_CUDA(cudaSetDevice(m->ctx->device));
    JQ_CUDA(cudaDeviceSynchronize());
    JQ_CUDA(cudaMemcpy(ids, m->ids, T * m->cfg.n_used * 4, cudaMemcpyDeviceToHost));
    JQ_CUDA(cudaMemcpy(wts, m->wts, T * m->cfg.n_used * 4, cudaMemcpyDeviceToHost));
    return jq::OK;
}

}  // extern "C"
