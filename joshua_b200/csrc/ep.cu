// Expert-parallel exchange over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The reference runs every expert in one process (src/quantized_qwen3_moe.rs:385-542); this is where the path
// shards.  Experts are split contiguously over `world` ranks.  Each rank owns a WINDOW of device memory that
// its peers map through CUDA IPC and write into directly:
//
//   rows_in  [world][cap][hidden] f32   block s: activation rows sent by rank s for my experts
//   ids_in   [world][cap]         u32   their local expert ids (n_local = "unused slot")
//   rows_back[world][cap][hidden] f32   block o: expert outputs coming back from owner o, in the slot order I chose
//   flag_in  [world], flag_back[world]  u32   epoch of the last completed write from that rank
//
// with cap = max_tokens * n_used (a rank can send at most that many rows to one peer).  One layer is
//
//   route                                   (replicated router, local)
//   dispatch   every (token, slot) pair's row is stored into its owner's rows_in, then flag_in[me] = epoch;
//              its last thread polls flag_in[*] (bounded) before the kernel ends
//   experts    grouped gate/up + SwiGLU and down products over rows_in (the single-GPU kernels)
//   return     valid rows' outputs are stored into their source's rows_back, then flag_back[me] = epoch
//   combine    polls flag_back[*] (bounded), y[t] = sum over slots in slot order of w * rows_back[...]
//
// No collective library call and no host read: the layer is eight kernel launches in one stream and can be
// replayed from a CUDA graph.  One window serves every layer of a model: a rank can only run one exchange
// ahead of a peer, and the flags order every reuse (a peer's next dispatch needs my return of this layer,
// which follows my last read of rows_in; my next return needs the peer's next dispatch, which follows its
// combine of this layer).
//
// Every poll is bounded; a wait that gives up sets the context's status flag (jq_device_status reports it)
// and the kernel carries on with whatever is in the window, so a missing peer cannot hang the GPU.
#include <algorithm>
#include <cstring>

#include "handles.cuh"

namespace {

constexpr uint32_t EP_MAX_WORLD = 8;
constexpr uint32_t EP_POLLS = 1u << 22;  // default bound of a wait: x ~0.25 us, about a second
constexpr uint32_t EP_SPIN = 64;         // polls without a pause before the wait starts to sleep between polls

struct Window {
    uint8_t* base[EP_MAX_WORLD];
};

struct Layout {
    uint32_t world, cap, hidden, n_local;
    uint64_t o_rows_in, o_ids_in, o_rows_back, o_flag_in, o_flag_back, bytes;
};

__host__ __device__ inline uint64_t up256(uint64_t v) { return (v + 255) & ~(uint64_t)255; }

Layout make_layout(uint32_t world, uint32_t cap, uint32_t hidden, uint32_t n_local) {
    Layout l = {world, cap, hidden, n_local, 0, 0, 0, 0, 0, 0};
    uint64_t off = 0;
    l.o_rows_in = off, off += up256((uint64_t)world * cap * hidden * 4);
    l.o_ids_in = off, off += up256((uint64_t)world * cap * 4);
    l.o_rows_back = off, off += up256((uint64_t)world * cap * hidden * 4);
    l.o_flag_in = off, off += 256;
    l.o_flag_back = off, off += 256;
    l.bytes = off;
    return l;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Polls until *flag has reached `target` (wrap-safe).  Gives up after `polls` polls and raises *status.  The
// first polls come back to back (a peer that is in step arrives within a few microseconds); after that the
// thread sleeps between polls.
__device__ void wait_flag(const uint32_t* flag, uint32_t target, uint32_t polls, int* status) {
    for (uint32_t i = 0; i < polls; ++i) {
        if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return;
        if (i >= EP_SPIN) __nanosleep(200);
    }
    *status = 1;
}

// The last of `n_ctas` CTAs to arrive publishes `epoch` in slot `me` of the given flag array of every peer.
// All data stores of the grid are ordered before the flag stores.  Returns true in thread 0 of that last CTA.
__device__ bool publish(uint32_t* done, const Window& win, uint64_t flag_off, uint32_t world, uint32_t me,
                        uint32_t epoch, uint32_t n_ctas) {
    // The CTA's stores are ordered before thread 0's count by the barrier and a device-scope fence; the one thread
    // that sees the last count issues the single system-scope fence (cumulative over everything the counted CTAs
    // stored) and then the flag stores.  A system-scope fence in every thread of every CTA costs several
    // microseconds a launch and adds nothing to that order.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done, 1u) == n_ctas - 1) {
            *done = 0;
            __threadfence_system();
            for (uint32_t d = 0; d < world; ++d)
                st_release_sys(reinterpret_cast<uint32_t*>(win.base[d] + flag_off) + me, epoch);
            return true;
        }
    }
    return false;
}

// grid = P + world CTAs.  CTA p < P stores pair p's activation row and local expert id into its owner's
// window; CTA P + d marks the unused slots of my block on rank d.  pair_slot[p] = owner * cap + slot.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(Window win, Layout l, uint32_t me, const float* __restrict__ x,
                                                          const float* __restrict__ norm_w, float eps,
                                                          const uint32_t* __restrict__ ids, uint32_t T, uint32_t K,
                                                          uint32_t* __restrict__ pair_slot, uint32_t* __restrict__ epoch,
                                                          uint32_t* __restrict__ done, uint32_t polls, int* status) {
    __shared__ uint32_t s_red[8];
    __shared__ int s_last;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t P = T * K, tid = threadIdx.x;
    const uint32_t next_epoch = *epoch + 1;
    const bool is_pair = blockIdx.x < P;
    const uint32_t p = blockIdx.x;
    const uint32_t d = is_pair ? min(ids[p] / l.n_local, l.world) : blockIdx.x - P;  // world = id out of range
    // pairs before p (all pairs, for a fill CTA) that go to the same rank
    const uint32_t upto = is_pair ? p : P;
    uint32_t cnt = 0;
    for (uint32_t q = tid; q < upto; q += blockDim.x) cnt += (ids[q] / l.n_local == d) ? 1u : 0u;
    for (int off = 16; off; off >>= 1) cnt += __shfl_xor_sync(0xFFFFFFFFu, cnt, off);
    if ((tid & 31) == 0) s_red[tid >> 5] = cnt;
    __syncthreads();
    cnt = 0;
    for (uint32_t w = 0; w < blockDim.x / 32; ++w) cnt += s_red[w];
    if (is_pair) {
        if (d < l.world) {
            const uint32_t slot = cnt;
            const uint64_t r = (uint64_t)me * l.cap + slot;
            float4* dst = reinterpret_cast<float4*>(win.base[d] + l.o_rows_in) + r * (l.hidden / 4);
            const float4* src = reinterpret_cast<const float4*>(x) + (uint64_t)(p / K) * (l.hidden / 4);
            if (norm_w == nullptr) {
                for (uint32_t c = tid; c < l.hidden / 4; c += blockDim.x) dst[c] = src[c];
            } else {
                // the row travels RMS-normalised (the block's norm folded into the exchange): sum of squares per
                // thread in column order, threads in thread order
                float ss = 0.0f;
                for (uint32_t c = tid; c < l.hidden / 4; c += blockDim.x) {
                    const float4 v = src[c];
                    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
                }
                for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
                __syncthreads();  // s_red is free again (every thread has read the slot count)
                if ((tid & 31) == 0) reinterpret_cast<float*>(s_red)[tid >> 5] = ss;
                __syncthreads();
                float tot = 0.0f;
                for (uint32_t w = 0; w < blockDim.x / 32; ++w) tot += reinterpret_cast<float*>(s_red)[w];
                const float rs = rsqrtf(tot / (float)l.hidden + eps);
                const float4* g4 = reinterpret_cast<const float4*>(norm_w);
                for (uint32_t c = tid; c < l.hidden / 4; c += blockDim.x) {
                    const float4 v = src[c], g = g4[c];
                    dst[c] = make_float4(v.x * rs * g.x, v.y * rs * g.y, v.z * rs * g.z, v.w * rs * g.w);
                }
            }
            if (tid == 0) {
                reinterpret_cast<uint32_t*>(win.base[d] + l.o_ids_in)[r] = ids[p] - d * l.n_local;
                pair_slot[p] = d * l.cap + slot;
            }
        } else if (tid == 0) {
            pair_slot[p] = 0xFFFFFFFFu;
        }
    } else {
        uint32_t* idd = reinterpret_cast<uint32_t*>(win.base[d] + l.o_ids_in) + (uint64_t)me * l.cap;
        for (uint32_t sl = cnt + tid; sl < l.cap; sl += blockDim.x) idd[sl] = l.n_local;
    }
    const bool last = publish(done, win, l.o_flag_in, l.world, me, next_epoch, gridDim.x);
    if (tid == 0) s_last = last ? 1 : 0;
    __syncthreads();
    if (s_last) {
        // The last CTA also waits (bounded, one thread per rank) for every rank's dispatch of this epoch and then
        // advances the local epoch counter: the kernels behind this one in the stream read rows_in / ids_in and
        // the new epoch, so the kernel must not end before the rows are there.  Every CTA of this grid read the
        // old epoch before it counted itself in.
        if (tid < l.world)
            wait_flag(reinterpret_cast<const uint32_t*>(win.base[me] + l.o_flag_in) + tid, next_epoch, polls, status);
        __syncthreads();
        if (tid == 0) *epoch = next_epoch;
    }
}

// Return and combine in one launch.  CTAs 0 .. n_rows-1 (n_rows = world * cap): row r of my rows_in (source rank
// r / cap, its slot r % cap); a valid row's output, out_list[inv[r], :], is stored into the source's rows_back block
// `me`, and the last of them publishes the return flag.  The CTAs behind them form
//     y[t, :] = sum over slots (in slot order) of w[t, s] * rows_back[pair_slot[t*K+s], :] (+ residual)
// after every owner's return of this epoch has arrived.  The return CTAs wait for nothing and come first in the
// grid, so the combine CTAs' (bounded) wait never keeps them from running, whatever the grid's size.
__global__ void __launch_bounds__(256) ep_return_combine_kernel(Window win, Layout l, uint32_t me, uint32_t n_rows,
                                                                const float* __restrict__ out_list,
                                                                const uint32_t* __restrict__ inv,
                                                                const uint32_t* __restrict__ pair_slot,
                                                                const float* __restrict__ wts, uint32_t T, uint32_t K,
                                                                const uint32_t* __restrict__ epoch, uint32_t* __restrict__ done,
                                                                const float* residual, float* y, uint32_t polls, int* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (blockIdx.x < n_rows) {
        const uint32_t r = blockIdx.x, src_rank = r / l.cap, slot = r % l.cap;
        const uint32_t id = reinterpret_cast<const uint32_t*>(win.base[me] + l.o_ids_in)[r];
        if (id < l.n_local) {
            const uint32_t pos = inv[r];
            float4* dst = reinterpret_cast<float4*>(win.base[src_rank] + l.o_rows_back) +
                          ((uint64_t)me * l.cap + slot) * (l.hidden / 4);
            const float4* src = reinterpret_cast<const float4*>(out_list) + (uint64_t)pos * (l.hidden / 4);
            for (uint32_t c = threadIdx.x; c < l.hidden / 4; c += blockDim.x) dst[c] = src[c];
        }
        publish(done, win, l.o_flag_back, l.world, me, *epoch, n_rows);
        return;
    }
    const uint8_t* my_window = win.base[me];
    if (threadIdx.x < l.world)
        wait_flag(reinterpret_cast<const uint32_t*>(my_window + l.o_flag_back) + threadIdx.x, *epoch, polls, status);
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const float* back = reinterpret_cast<const float*>(my_window + l.o_rows_back);
    const uint32_t h4 = l.hidden / 4, n_comb = gridDim.x - n_rows;
    const uint64_t total = (uint64_t)T * h4;
    for (uint64_t i = (blockIdx.x - n_rows) * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)n_comb * blockDim.x) {
        const uint32_t t = (uint32_t)(i / h4), c = (uint32_t)(i % h4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        // rows_back is written by peers: read it through L2, never from a stale L1 line
        if (K <= 8) {
            // all slots and weights requested first, then all rows, then the sum in slot order (two round trips
            // instead of 2 K dependent ones)
            uint32_t ps[8];
            float w[8];
            float4 v[8];
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) {
                ps[s] = s < K ? pair_slot[(uint64_t)t * K + s] : 0xFFFFFFFFu;
                w[s] = s < K ? wts[(uint64_t)t * K + s] : 0.0f;
            }
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s)
                v[s] = ps[s] != 0xFFFFFFFFu ? __ldcg(reinterpret_cast<const float4*>(back + (uint64_t)ps[s] * l.hidden) + c)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) {
                if (ps[s] == 0xFFFFFFFFu) continue;
                acc.x += v[s].x * w[s];
                acc.y += v[s].y * w[s];
                acc.z += v[s].z * w[s];
                acc.w += v[s].w * w[s];
            }
        } else {
            for (uint32_t s = 0; s < K; ++s) {
                const uint32_t ps = pair_slot[(uint64_t)t * K + s];
                if (ps == 0xFFFFFFFFu) continue;
                const float w = wts[(uint64_t)t * K + s];
                const float4 v = __ldcg(reinterpret_cast<const float4*>(back + (uint64_t)ps * l.hidden) + c);
                acc.x += v.x * w;
                acc.y += v.y * w;
                acc.z += v.z * w;
                acc.w += v.w * w;
            }
        }
        if (residual) {
            const float4 v = *reinterpret_cast<const float4*>(residual + (uint64_t)t * l.hidden + 4 * c);
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
        }
        *reinterpret_cast<float4*>(y + (uint64_t)t * l.hidden + 4 * c) = acc;
    }
}

}  // namespace

struct jq_ep {
    jq_ctx* ctx;
    uint32_t rank, world, n_expert, n_used, hidden, max_tokens, n_local;
    Layout lay;
    Window win;            // win.base[rank] is my own allocation, the others are IPC mappings
    bool connected = false;
    bool loopback = false;  // peer windows are private local allocations (single-GPU tests)
    uint32_t polls = EP_POLLS;
    uint32_t *ids = nullptr, *pair_slot = nullptr, *epoch = nullptr, *done = nullptr;  // local device state
    float* wts = nullptr;
};

extern "C" {

int32_t jq_ep_create(jq_ctx* ctx, uint32_t rank, uint32_t world, uint32_t n_expert, uint32_t n_used, uint32_t hidden,
                     uint32_t max_tokens, jq_ep** out) {
    if (!ctx || !out) return jq_fail(jq::E_INVALID, "jq_ep_create: NULL argument");
    *out = nullptr;
    if (world == 0 || world > EP_MAX_WORLD || rank >= world)
        return jq_fail(jq::E_INVALID, "jq_ep_create: need rank < world <= 8");
    if (n_expert == 0 || n_expert % world) return jq_fail(jq::E_INVALID, "jq_ep_create: experts do not split evenly over the ranks");
    if (n_used == 0 || n_used > n_expert || hidden == 0 || hidden % 4 || max_tokens == 0)
        return jq_fail(jq::E_INVALID, "jq_ep_create: bad n_used / hidden / max_tokens");
    if ((uint64_t)max_tokens * n_used > 16384)
        return jq_fail(jq::E_TOO_LARGE, "jq_ep_create: max_tokens * n_used above 16384 rows per exchange (send more tokens in slices)");
    JQ_CUDA(cudaSetDevice(ctx->device));
    jq_ep* e = new (std::nothrow) jq_ep();
    if (!e) return jq_fail(jq::E_NOMEM, "jq_ep_create: out of host memory");
    e->ctx = ctx;
    e->rank = rank, e->world = world, e->n_expert = n_expert, e->n_used = n_used, e->hidden = hidden;
    e->max_tokens = max_tokens, e->n_local = n_expert / world;
    const uint32_t cap = max_tokens * n_used;
    e->lay = make_layout(world, cap, hidden, e->n_local);
    for (uint32_t i = 0; i < EP_MAX_WORLD; ++i) e->win.base[i] = nullptr;
    cudaError_t ce = cudaMalloc(&e->win.base[rank], e->lay.bytes);
    if (ce == cudaSuccess) ce = cudaMemset(e->win.base[rank], 0, e->lay.bytes);
    if (ce == cudaSuccess) ce = cudaMalloc(&e->ids, (size_t)cap * 4);
    if (ce == cudaSuccess) ce = cudaMalloc(&e->wts, (size_t)cap * 4);
    if (ce == cudaSuccess) ce = cudaMalloc(&e->pair_slot, (size_t)cap * 4);
    if (ce == cudaSuccess) ce = cudaMalloc(&e->epoch, 256);
    if (ce == cudaSuccess) ce = cudaMemset(e->epoch, 0, 256);
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    e->done = e->epoch ? e->epoch + 16 : nullptr;
    if (ce != cudaSuccess) {
        jq_ep_free(e);
        return jq_fail_cuda(ce, "jq_ep_create");
    }
    if (world == 1) e->connected = true;
    *out = e;
    return jq::OK;
}

void jq_ep_free(jq_ep* e) {
    if (!e) return;
    cudaSetDevice(e->ctx->device);
    cudaDeviceSynchronize();
    for (uint32_t i = 0; i < e->world; ++i) {
        if (!e->win.base[i]) continue;
        if (i == e->rank || e->loopback)
            cudaFree(e->win.base[i]);
        else
            cudaIpcCloseMemHandle(e->win.base[i]);
    }
    cudaFree(e->ids);
    cudaFree(e->wts);
    cudaFree(e->pair_slot);
    cudaFree(e->epoch);
    delete e;
}

int32_t jq_ep_export(jq_ep* e, uint8_t* handle) {
    if (!e || !handle) return jq_fail(jq::E_INVALID, "jq_ep_export: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == JQ_EP_HANDLE_BYTES, "IPC handle size");
    JQ_CUDA(cudaSetDevice(e->ctx->device));
    cudaIpcMemHandle_t h;
    JQ_CUDA(cudaIpcGetMemHandle(&h, e->win.base[e->rank]));
    memcpy(handle, &h, sizeof(h));
    return jq::OK;
}

int32_t jq_ep_connect(jq_ep* e, const uint8_t* handles) {
    if (!e || !handles) return jq_fail(jq::E_INVALID, "jq_ep_connect: NULL argument");
    if (e->connected) return jq_fail(jq::E_INVALID, "jq_ep_connect: already connected");
    JQ_CUDA(cudaSetDevice(e->ctx->device));
    for (uint32_t i = 0; i < e->world; ++i) {
        if (i == e->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)i * JQ_EP_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        JQ_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        e->win.base[i] = static_cast<uint8_t*>(p);
    }
    e->connected = true;
    return jq::OK;
}

int32_t jq_ep_connect_loopback(jq_ep* e) {
    if (!e) return jq_fail(jq::E_INVALID, "jq_ep_connect_loopback: NULL handle");
    if (e->connected) return jq_fail(jq::E_INVALID, "jq_ep_connect_loopback: already connected");
    JQ_CUDA(cudaSetDevice(e->ctx->device));
    e->loopback = true;
    for (uint32_t i = 0; i < e->world; ++i) {
        if (i == e->rank) continue;
        JQ_CUDA(cudaMalloc(&e->win.base[i], e->lay.bytes));
        JQ_CUDA(cudaMemset(e->win.base[i], 0, e->lay.bytes));
    }
    JQ_CUDA(cudaDeviceSynchronize());
    e->connected = true;
    return jq::OK;
}

int32_t jq_ep_set_poll_limit(jq_ep* e, uint32_t polls) {
    if (!e) return jq_fail(jq::E_INVALID, "jq_ep_set_poll_limit: NULL handle");
    e->polls = polls ? polls : EP_POLLS;
    return jq::OK;
}

int32_t jq_ep_rows_served(jq_ep* e, uint32_t* rows) {
    if (!e || !rows) return jq_fail(jq::E_INVALID, "jq_ep_rows_served: NULL argument");
    JQ_CUDA(cudaSetDevice(e->ctx->device));
    JQ_CUDA(cudaDeviceSynchronize());
    const size_t n = (size_t)e->world * e->lay.cap;
    std::vector<uint32_t> ids(n);
    JQ_CUDA(cudaMemcpy(ids.data(), e->win.base[e->rank] + e->lay.o_ids_in, n * 4, cudaMemcpyDeviceToHost));
    uint32_t served = 0;
    for (uint32_t id : ids) served += id < e->n_local ? 1u : 0u;
    *rows = served;
    return jq::OK;
}

int32_t jq_ep_forward_dev(jq_ep* e, jq_moe* router, jq_moe* experts, const float* x_dev, uint64_t T,
                          const float* residual_dev, float* y_dev, void* stream) {
    return jq_ep_forward_norm_dev(e, router, experts, x_dev, T, nullptr, 0.0f, nullptr, residual_dev, y_dev, stream);
}

int32_t jq_ep_forward_norm_dev(jq_ep* e, jq_moe* router, jq_moe* experts, const float* x_dev, uint64_t T,
                               const float* norm_w_dev, float eps, const uint32_t* forced_ids_dev,
                               const float* residual_dev, float* y_dev, void* stream) {
    if (!e || !router || !experts) return jq_fail(jq::E_INVALID, "jq_ep_forward_dev: NULL handle");
    if (!e->connected) return jq_fail(jq::E_INVALID, "jq_ep_forward_dev: call jq_ep_connect first");
    if (!x_dev || !y_dev) return jq_fail(jq::E_INVALID, "jq_ep_forward_dev: NULL buffer");
    if (T == 0 || T > e->max_tokens)
        return jq_fail(jq::E_TOO_LARGE, "jq_ep_forward_dev: every rank must pass between 1 and max_tokens tokens");
    const jq_moe_config &rc = router->cfg, &ec = experts->cfg;
    if (rc.n_expert != e->n_expert || rc.n_used != e->n_used || rc.hidden != e->hidden)
        return jq_fail(jq::E_INVALID, "jq_ep_forward_dev: router layer does not match the exchange");
    if (!experts->gate || ec.n_expert != e->n_local || ec.hidden != e->hidden)
        return jq_fail(jq::E_INVALID, "jq_ep_forward_dev: expert layer does not hold this rank's experts");
    const uint32_t cap = e->lay.cap, rows = e->world * cap;
    if (rows > experts->cap_tokens || rows > experts->cap_pairs)
        return jq_fail(jq::E_TOO_LARGE, "jq_ep_forward_dev: call jq_moe_reserve(expert layer, 0, world * max_tokens * n_used) first");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* mine = e->win.base[e->rank];
    const uint32_t P = (uint32_t)T * e->n_used;
    if (int32_t r = jq_moe_route_norm_dev(router, x_dev, T, norm_w_dev, eps, forced_ids_dev, e->ids, e->wts, stream)) return r;
    JQ_CUDA(jq::launch_pdl(ep_dispatch_kernel, dim3(P + e->world), 256, 0, s, e->win, e->lay, e->rank, x_dev,
                           norm_w_dev, eps, (const uint32_t*)e->ids, (uint32_t)T, e->n_used, e->pair_slot, e->epoch, e->done,
                           e->polls, e->ctx->status_dev));
    // (building the expert layer's job list in the dispatch kernel's last CTA instead of a launch of its own was
    // measured slower: 256 threads behind the wait against 1024 threads that are resident before it ends)
    if (int32_t r = jq_moe_experts_list(experts, reinterpret_cast<const float*>(mine + e->lay.o_rows_in), rows,
                                        reinterpret_cast<const uint32_t*>(mine + e->lay.o_ids_in), P, s))
        return r;
    const unsigned cblocks = (unsigned)std::min<uint64_t>(((uint64_t)T * (e->hidden / 4) + 255) / 256, 148 * 4);
    JQ_CUDA(jq::launch_pdl(ep_return_combine_kernel, dim3(rows + cblocks), 256, 0, s, e->win, e->lay, e->rank, rows,
                           (const float*)experts->out, (const uint32_t*)experts->inv, (const uint32_t*)e->pair_slot,
                           (const float*)e->wts, (uint32_t)T, e->n_used, (const uint32_t*)e->epoch, e->done + 1, residual_dev,
                           y_dev, e->polls, e->ctx->status_dev));
    return jq::OK;
}

}  // extern "C"
