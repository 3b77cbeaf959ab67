// Prefill / batched matmul (m > 8) over raw GGUF blocks on the 5th-generation tensor cores.
//
// dst[m, n] = lhs[m, k] . W[n, k]^T with W left in its GGUF bytes.  A CTA owns a 128-row tile of W and a tile
// of up to 256 activation rows (the wider the tile, the fewer times a weight is decoded).  Per 32-column K step its converter warps decode the 128 x 32 weight block to
// the exact f32 weights the reference forms (formats.cuh), split weights and activations into two TF32 terms
// (hi = top 11 significant bits, lo = the exact remainder), and store both terms K-major in the 128-byte
// swizzled layout the tensor core reads.  One thread issues tcgen05.mma (kind::tf32) for the three
// significant products hi*hi + hi*lo + lo*hi into a 128 x N f32 accumulator in tensor memory; each product is
// exact and the split carries ~2^-22 relative error per term.  The tensor core adds into its f32 accumulator
// with truncation, an error that grows linearly with the number of accumulated instructions, so the
// accumulator only ever holds TC_CHUNK K steps (128 columns): the converter warps read each finished chunk
// back with tcgen05.ld and add it, round-to-nearest, to running sums in registers while the next chunk
// accumulates in the other half of tensor memory.  The result then matches f32 accumulation
// (src/kquant_dot.rs:268-483) to the tolerance the path is held to.
//
// Pipeline: NS shared-memory stages, each guarded by a `full` mbarrier (converters -> issuer, after a
// generic-to-async proxy fence) and an `empty` mbarrier (tcgen05.commit -> converters).  Every wait is
// bounded; a wait that runs out raises the device status flag, and every thread still reaches the common
// exit where tensor memory is released.
//
// Tensor-pipe bound for large m: 3 x 2*m*n*k TF32 flops per launch.  Algorithmic flops: 2*m*n*k.
#include <algorithm>

#include "common.cuh"

namespace jq {

cudaError_t tables_gemm_tc() { return upload_tables(); }

namespace {

constexpr int TC_M = 128;          // weight rows per CTA = MMA M = TMEM lanes
constexpr int TC_K = 32;           // K per stage: 32 tf32 = one 128-byte swizzled row
constexpr int TC_CHUNK = 4;        // K steps accumulated in tensor memory before a read-back
constexpr int TC_CONV_WARPS = 16;  // converter / epilogue warps: 4 per quarter of the accumulator's lanes
constexpr int TC_THREADS = (TC_CONV_WARPS + 1) * 32;
constexpr uint32_t PLANE_A = TC_M * 128;  // bytes of one term of the weight tile

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 24); ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address / 16
    d |= (uint64_t)1 << 16;                      // leading byte offset (unused by swizzled K-major) = 1
    d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                      // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                      // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D f32, A and B tf32, both K-major, M = 128, N = n_tile.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n_tile) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((n_tile >> 3) << 17) | ((uint32_t)(TC_M >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t r[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t r[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Split 4 floats into their TF32 hi parts and exact remainders and store both 16-byte chunks.  `row_base`
// is the byte offset of the row inside a term's tile; `chunk` the 16-byte chunk inside the 128-byte row.
__device__ __forceinline__ void store_split(uint8_t* hi_tile, uint8_t* lo_tile, uint32_t row, uint32_t chunk,
                                            const float v[4]) {
    float4 h, l;
    h.x = __uint_as_float(__float_as_uint(v[0]) & 0xFFFFE000u);
    h.y = __uint_as_float(__float_as_uint(v[1]) & 0xFFFFE000u);
    h.z = __uint_as_float(__float_as_uint(v[2]) & 0xFFFFE000u);
    h.w = __uint_as_float(__float_as_uint(v[3]) & 0xFFFFE000u);
    l = make_float4(v[0] - h.x, v[1] - h.y, v[2] - h.z, v[3] - h.w);
    // 128-byte swizzle: chunk index XOR (row mod 8) inside each 8-row x 128-byte atom
    const uint32_t off = row * 128 + ((chunk ^ (row & 7)) << 4);
    *reinterpret_cast<float4*>(hi_tile + off) = h;
    *reinterpret_cast<float4*>(lo_tile + off) = l;
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_tc_kernel(const uint8_t* __restrict__ w, uint64_t n, uint64_t k, const float* __restrict__ lhs, uint64_t m,
                   float* __restrict__ dst, uint32_t n_stages, int* __restrict__ error_flag) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // stage layout: A hi | A lo | B hi | B lo, every tile 1024-byte aligned
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t PLANE_B = N_TILE * 128;
    constexpr uint32_t STAGE = 2 * PLANE_A + 2 * PLANE_B;
    __shared__ uint64_t full[8], empty[8], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t row0 = (uint64_t)blockIdx.x * TC_M;
    const uint64_t tok0 = (uint64_t)blockIdx.y * N_TILE;
    const uint32_t k_steps = (uint32_t)(k / TC_K);
    const uint32_t n_chunks = (k_steps + TC_CHUNK - 1) / TC_CHUNK;
    const uint64_t row_bytes = k / ELEMS * BYTES;
    constexpr uint32_t UPB = ELEMS / 8;
    constexpr uint32_t TMEM_COLS = 2 * N_TILE < 32 ? 32 : 2 * N_TILE;  // two accumulators; a power of two >= 32

    if (tid == 0) {
        for (uint32_t s = 0; s < n_stages; ++s) {
            mbar_init(&full[s], TC_CONV_WARPS);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TC_CONV_WARPS);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_CONV_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < TC_CONV_WARPS) {
        // ── converters: per K step thread (r, unit) decodes 8 weights of row r, and the 512 threads split the
        // N_TILE x 32 activation block between them (16-byte pieces, 8 consecutive threads per 128-byte row).
        // Between chunks they read the finished accumulator back: warp w reads TMEM lanes 32 (w % 4) .. + 31
        // (its weight rows) and the quarter w / 4 of the columns (tokens). ──
        const uint32_t r = tid & 127, unit = tid >> 7;  // weight row of the tile, 8-value unit of the K step
        const uint64_t wrow = row0 + r < n ? row0 + r : n - 1;
        const uint8_t* wr = w + wrow * row_bytes;
        constexpr int B_PER = (N_TILE * 8 + TC_CONV_WARPS * 32 - 1) / (TC_CONV_WARPS * 32);  // 16-byte pieces per thread
        const uint32_t brow0 = tid >> 3, bchunk = tid & 7;
        const uint32_t q = warp & 3, grp = warp >> 2;
        constexpr int MY_COLS = N_TILE / 4;  // columns this thread accumulates
        float sums[MY_COLS];
#pragma unroll
        for (int c = 0; c < MY_COLS; ++c) sums[c] = 0.0f;
        // read chunk `c`'s accumulator and add it to the running sums
        auto drain = [&](uint32_t c) -> bool {
            const uint32_t buf = c & 1;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[buf], (c >> 1) & 1))) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_d + ((q * 32) << 16) + buf * N_TILE + grp * MY_COLS;
            if constexpr (MY_COLS == 8) {
                uint32_t rr[8];
                tmem_ld8(taddr, rr);
#pragma unroll
                for (int i = 0; i < 8; ++i) sums[i] += __uint_as_float(rr[i]);
            } else if constexpr (MY_COLS == 16) {
                uint32_t rr[16];
                tmem_ld16(taddr, rr);
#pragma unroll
                for (int i = 0; i < 16; ++i) sums[i] += __uint_as_float(rr[i]);
            } else {
#pragma unroll
                for (int part = 0; part < MY_COLS / 32; ++part) {
                    uint32_t rr[32];
                    tmem_ld32(taddr + part * 32, rr);
#pragma unroll
                    for (int i = 0; i < 32; ++i) sums[part * 32 + i] += __uint_as_float(rr[i]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            return true;
        };
        // this thread's activation pieces of K step ks (requested one step ahead of their use)
        float4 xb[B_PER];
        auto load_b = [&](uint32_t ks) {
#pragma unroll
            for (int j = 0; j < B_PER; ++j) {
                const uint32_t br = brow0 + j * (TC_CONV_WARPS * 4);
                const bool real = br < N_TILE && tok0 + br < m;
                xb[j] = real ? __ldg(reinterpret_cast<const float4*>(lhs + (tok0 + br) * k + (uint64_t)ks * TC_K + bchunk * 4))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        bool ok = true;
        uint32_t drained = 0;
        load_b(0);
        for (uint32_t ks = 0; ks < k_steps && ok; ++ks) {
            const uint32_t s = ks % n_stages, round = ks / n_stages;
            // decode before waiting for the stage: the global loads overlap the wait
            float v[8];
            {
                const uint32_t u = ks * 4 + unit;  // 8-value unit of the row
                decode_unit<TYPE>(wr + (uint64_t)(u / UPB) * BYTES, u % UPB, v, false);
            }
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&empty[s], (round & 1) ^ 1));  // warp-uniform
            if (!ok) break;
            uint8_t* st = smem + (size_t)s * STAGE;
            store_split(st, st + PLANE_A, r, unit * 2, v);
            store_split(st, st + PLANE_A, r, unit * 2 + 1, v + 4);
#pragma unroll
            for (int j = 0; j < B_PER; ++j) {
                const uint32_t br = brow0 + j * (TC_CONV_WARPS * 4);
                if (br < N_TILE) {
                    float bv[4] = {xb[j].x, xb[j].y, xb[j].z, xb[j].w};
                    store_split(st + 2 * PLANE_A, st + 2 * PLANE_A + PLANE_B, br, bchunk, bv);
                }
            }
            if (ks + 1 < k_steps) load_b(ks + 1);
            // make the generic-proxy stores visible to the tensor core's async proxy, then hand over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            // at a chunk boundary drain every finished chunk but the newest (which is still accumulating)
            if ((ks + 1) % TC_CHUNK == 0)
                while (ok && drained + 1 < (ks + 1) / TC_CHUNK) ok = drain(drained++);
        }
        while (ok && drained < n_chunks) ok = drain(drained++);
        if (!ok) abort_flag = 1;
        if (ok) {
            const uint64_t out_row = row0 + q * 32 + lane;
#pragma unroll
            for (int c = 0; c < MY_COLS; ++c) {
                const uint64_t tok = tok0 + grp * MY_COLS + c;
                if (tok < m && out_row < n) dst[tok * n + out_row] = sums[c];
            }
        }
    } else {
        // ── issuer: one thread feeds the tensor core ──
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(N_TILE);
            bool ok = true;
            for (uint32_t ks = 0; ks < k_steps && ok; ++ks) {
                const uint32_t s = ks % n_stages, round = ks / n_stages;
                const uint32_t chunk = ks / TC_CHUNK, buf = chunk & 1;
                if (ks % TC_CHUNK == 0 && chunk >= 2) {
                    // the accumulator half must have been read back before it is overwritten
                    ok = mbar_wait(&acc_empty[buf], ((chunk >> 1) - 1) & 1);
                    if (!ok) break;
                }
                ok = mbar_wait(&full[s], round & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_hi = smem_u32(smem + (size_t)s * STAGE), a_lo = a_hi + PLANE_A;
                const uint32_t b_hi = a_hi + 2 * PLANE_A, b_lo = b_hi + PLANE_B;
                const uint32_t d = tmem_d + buf * N_TILE;
#pragma unroll
                for (uint32_t kk = 0; kk < TC_K / 8; ++kk) {
                    // one instruction covers K = 8 tf32 = 32 bytes of the swizzled row
                    const uint32_t adv = kk * 32;
                    umma_tf32(d, umma_desc(a_hi + adv), umma_desc(b_hi + adv), idesc, (ks % TC_CHUNK != 0) || kk != 0);
                    umma_tf32(d, umma_desc(a_hi + adv), umma_desc(b_lo + adv), idesc, 1);
                    umma_tf32(d, umma_desc(a_lo + adv), umma_desc(b_hi + adv), idesc, 1);
                }
                umma_commit(&empty[s]);  // arrives when the instructions above have finished reading the stage
                if ((ks + 1) % TC_CHUNK == 0 || ks + 1 == k_steps) umma_commit(&acc_full[buf]);
            }
            if (!ok) abort_flag = 1;
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_flag && tid == 0) *reinterpret_cast<volatile int*>(error_flag) = 1;
    if (warp == TC_CONV_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
cudaError_t launch_tile(const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m, float* dst,
                        int* error_flag, cudaStream_t s) {
    constexpr uint32_t STAGE = 2 * PLANE_A + 2 * N_TILE * 128;
    uint32_t n_stages = std::min<uint32_t>(8, std::min<uint32_t>((uint32_t)(k / TC_K), (216 * 1024) / STAGE));
    size_t smem = (size_t)n_stages * STAGE + 1024;
    auto kern = gemm_tc_kernel<TYPE, ELEMS, BYTES, N_TILE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    dim3 grid((unsigned)((n + TC_M - 1) / TC_M), (unsigned)((m + N_TILE - 1) / N_TILE));
    kern<<<grid, TC_THREADS, smem, s>>>(w, n, k, lhs, m, dst, n_stages, error_flag);
    return cudaGetLastError();
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
cudaError_t launch_type(const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m, float* dst,
                        int* error_flag, cudaStream_t s) {
    if (m <= 32) return launch_tile<TYPE, ELEMS, BYTES, 32>(w, n, k, lhs, m, dst, error_flag, s);
    if (m <= 64) return launch_tile<TYPE, ELEMS, BYTES, 64>(w, n, k, lhs, m, dst, error_flag, s);
    if (m <= 128) return launch_tile<TYPE, ELEMS, BYTES, 128>(w, n, k, lhs, m, dst, error_flag, s);
    // 256-token tiles decode every weight half as often, but only pay off once they still fill the SMs
    const uint64_t ctas256 = ((n + TC_M - 1) / TC_M) * ((m + 255) / 256);
    if (ctas256 < 148) return launch_tile<TYPE, ELEMS, BYTES, 128>(w, n, k, lhs, m, dst, error_flag, s);
    return launch_tile<TYPE, ELEMS, BYTES, 256>(w, n, k, lhs, m, dst, error_flag, s);
}

}  // namespace

bool gemm_tc_supports(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, uint64_t m) {
    if (m == 0 || n == 0 || k == 0 || k % 32 != 0) return false;
    Format f;
    if (!format_of(type, &f)) return false;
    uint64_t row_bytes = k / f.elems * f.bytes;
    uintptr_t a = reinterpret_cast<uintptr_t>(w);
    // decode_unit's alignment needs hold for every row
    switch (type) {
        case T_Q4_K: return a % 4 == 0;
        case T_Q2_K: return a % 4 == 0;
        case T_Q8_0: return a % 2 == 0 && row_bytes % 2 == 0;
        case T_IQ2_XXS: return a % 2 == 0;
        case T_MXFP4: return true;
        default: return false;
    }
}

cudaError_t launch_gemm_tc(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                           float* dst, int* error_flag, cudaStream_t s) {
    switch (type) {
        case T_Q8_0: return launch_type<T_Q8_0, 32, 34>(w, n, k, lhs, m, dst, error_flag, s);
        case T_Q2_K: return launch_type<T_Q2_K, 256, 84>(w, n, k, lhs, m, dst, error_flag, s);
        case T_Q4_K: return launch_type<T_Q4_K, 256, 144>(w, n, k, lhs, m, dst, error_flag, s);
        case T_IQ2_XXS: return launch_type<T_IQ2_XXS, 256, 66>(w, n, k, lhs, m, dst, error_flag, s);
        case T_MXFP4: return launch_type<T_MXFP4, 32, 17>(w, n, k, lhs, m, dst, error_flag, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jq
