// Prefill / batched matmul (m > 8) over raw GGUF blocks on the 5th-generation tensor cores.
//
// dst[m, n] = lhs[m, k] . W[n, k]^T with W left in its GGUF bytes.  A CTA owns a 128-row tile of W and a tile
// of up to 128 activation rows.  Per 32-column K step its converter warps decode the 128 x 32 weight block to
// the exact f32 weights the reference forms (formats.cuh) and split them into two TF32 terms (hi = top 11
// significant bits, lo = the exact remainder); the activations are split the same way once per launch by a
// small kernel (two f32 arrays) and reach shared memory by TMA (`cp.async.bulk.tensor.2d`, 128-byte swizzle).
// One thread issues tcgen05.mma (kind::tf32) for the three significant products hi*hi + hi*lo + lo*hi into a
// 128 x N f32 accumulator in tensor memory; each product is exact and the split carries ~2^-22 relative error
// per term.  The tensor core adds into its f32 accumulator with truncation, an error that grows linearly with
// the number of accumulated instructions, so the accumulator only ever holds a chunk of 4 K steps (128
// columns): the converter warps read each finished chunk back with tcgen05.ld and add it, round-to-nearest, to
// running sums in registers while the next chunk accumulates in the other half of tensor memory.  The result
// then matches f32 accumulation (src/kquant_dot.rs:268-483) to the tolerance the path is held to.
//
// Two forms.  `gemm_ts_kernel` (the usual one): raw weight bytes are staged in shared memory by asynchronous
// copies, the weight terms go to tensor memory (tcgen05.st) and are the MMA's A operand from there, so shared
// memory carries only the activation tiles.  `gemm_tc_kernel`: weights decoded straight from global memory into
// swizzled shared-memory tiles; it takes the shapes the first does not (rows not word-aligned, k not a whole
// number of staged windows).
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the device status flag, and every thread
// still reaches the common exit where tensor memory is released.
//
// Tensor-pipe bound for large m: 3 x 2*m*n*k TF32 flops per launch.  Algorithmic flops: 2*m*n*k.
#include <algorithm>
#include <cstdlib>

#include <cuda.h>
#include <cudaTypedefs.h>

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
    {  // the phase usually is complete already: the non-blocking test answers faster than a try_wait
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
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
__device__ __forceinline__ unsigned long long tc_now() {
    return (unsigned long long)clock64();  // SM cycles: both traced threads run on the same SM
}
// Profiling aid (jq_debug_gemm_trace, a buffer of 512 values): CTA (0, 0) stores eight SM-cycle stamps per K step
// for its first 64 steps.  Converter thread 0: [0] stage free, [1] stage handed over.  Issuer: [2] top of the
// step, [3] accumulator half free, [4] operands complete, [5] MMAs issued, [6] stage commit issued, [7] end.
unsigned long long* g_gemm_trace = nullptr;

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One box of a 2-D tensor map (x = element offset along k, a multiple of 4 floats; y = row) into shared memory.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// x -> its TF32 part (top 11 significant bits) and the exact remainder, element-wise.
__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ x, uint64_t n4, float* __restrict__ hi,
                                                         float* __restrict__ lo) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n4; i += (uint64_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
        float4 h;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
        reinterpret_cast<float4*>(hi)[i] = h;
        reinterpret_cast<float4*>(lo)[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
    }
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
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
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

// Elements of a row that one staged window of raw bytes covers: a whole number of blocks whose bytes are a
// multiple of four (so the window moves as 32-bit words), a few K steps long.
__host__ __device__ constexpr uint32_t window_elems(uint32_t type) {
    return type == T_IQ2_XXS ? 512u : 256u;  // 132 bytes / 272, 144, 84, 136 bytes
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
__global__ void __launch_bounds__(TC_THREADS, 1)
    gemm_tc_kernel(const uint8_t* __restrict__ w, uint64_t n, uint64_t k, const __grid_constant__ CUtensorMap map_hi,
                   const __grid_constant__ CUtensorMap map_lo, uint64_t m, float* __restrict__ dst, uint32_t n_stages,
                   int* __restrict__ error_flag, unsigned long long* __restrict__ trace, int dbg_skip) {
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
    // Converter mapping: warp w owns weight rows 8w .. 8w+7, lane l the unit l % 4 (8 of the step's 32 columns)
    // of row 8w + l / 4, so a warp's loads touch 8 rows (8 L1 wavefronts per load, not 32) and its 16-byte
    // stores to the swizzled tile fall on distinct banks.  The decode reads global memory directly: this form
    // serves the shapes the tensor-memory form below does not take (rows that are not word-aligned, k not a
    // whole number of its windows).
    constexpr uint32_t ROWS_PER_WARP = TC_M / TC_CONV_WARPS;                // 8

    if (tid == 0) {
        for (uint32_t s = 0; s < n_stages; ++s) {
            mbar_init(&full[s], TC_CONV_WARPS + 1);  // the converter warps and the thread that starts the TMA copies
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
        // ── converters: per K step a thread decodes 8 weights of its row and stores their two TF32 terms;
        // thread 0 also starts the TMA copies of the step's activation tiles.
        // Between chunks they read the finished accumulator back: warp w reads TMEM lanes 32 (w % 4) .. + 31
        // (its weight rows) and the quarter w / 4 of the columns (tokens). ──
        const uint32_t r = warp * ROWS_PER_WARP + (lane >> 2), unit = lane & 3;  // this thread's row and unit
        const uint64_t wrow = row0 + r < n ? row0 + r : n - 1;                  // rows past n repeat the last one
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
        bool ok = true;
        uint32_t drained = 0;
        for (uint32_t ks = 0; ks < k_steps && ok; ++ks) {
            const uint32_t s = ks % n_stages, round = ks / n_stages;
            // decode before waiting for the stage (the loads overlap the wait)
            float v[8];
            if (!(dbg_skip & 1)) {
                const uint32_t u = ks * 4 + unit;  // 8-value unit of the row
                decode_unit<TYPE>(w + wrow * row_bytes + (uint64_t)(u / UPB) * BYTES, u % UPB, v, false);
            }
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&empty[s], (round & 1) ^ 1));  // warp-uniform
            if (!ok) break;
            const bool tr = trace != nullptr && tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && ks < 64;
            if (tr) trace[8 * ks] = tc_now();
            uint8_t* st = smem + (size_t)s * STAGE;
            if (tid == 0) {
                // the stage is free: start the two activation tiles (hi, lo) of this K step on their way
                if (dbg_skip & 2) {
                    mbar_arrive(&full[s]);
                } else {
                    mbar_arrive_expect_tx(&full[s], 2 * PLANE_B);
                    tma_load_2d(st + 2 * PLANE_A, &map_hi, ks * TC_K, (uint32_t)tok0, &full[s]);
                    tma_load_2d(st + 2 * PLANE_A + PLANE_B, &map_lo, ks * TC_K, (uint32_t)tok0, &full[s]);
                }
            }
            if (!(dbg_skip & 1)) {
                store_split(st, st + PLANE_A, r, unit * 2, v);
                store_split(st, st + PLANE_A, r, unit * 2 + 1, v + 4);
            }
            // make the generic-proxy stores visible to the tensor core's async proxy, then hand over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            if (tr) trace[8 * ks + 1] = tc_now();
            // drain every finished chunk but the newest (which is still accumulating)
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
        // ── issuer: the whole warp walks the K steps and waits on the barriers (warp-uniform control flow); one
        // elected lane issues the tensor-core instructions and their commits ──
        const uint32_t idesc = umma_idesc(N_TILE);
        const uint32_t base0 = smem_u32(smem);
        const uint64_t d0_a_hi = umma_desc(base0), d0_a_lo = umma_desc(base0 + PLANE_A);
        const uint64_t d0_b_hi = umma_desc(base0 + 2 * PLANE_A), d0_b_lo = umma_desc(base0 + 2 * PLANE_A + PLANE_B);
        bool ok = true;
        uint32_t s = 0, round = 0;  // stage and its use count, stepped without a division
        for (uint32_t ks = 0; ks < k_steps && ok; ++ks) {
            const uint32_t chunk = ks / TC_CHUNK, buf = chunk & 1;
            const bool tr = trace != nullptr && lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && ks < 64;
            if (tr) trace[8 * ks + 2] = tc_now();
            if (ks % TC_CHUNK == 0 && chunk >= 2) {
                // the accumulator half must have been read back before it is overwritten
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(&acc_empty[buf], ((chunk >> 1) - 1) & 1));
                if (!ok) break;
                // orders the MMAs below after the converters' reads of this half of tensor memory; the
                // shared-memory operands need no tensor-core fence (proxy fence + mbarrier)
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (tr) trace[8 * ks + 3] = tc_now();
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&full[s], round & 1));
            if (!ok) break;
            if (tr) trace[8 * ks + 4] = tc_now();
            if (elect_one()) {
                // descriptors differ from the stage-0 ones only in the start-address field (bytes / 16, no carry
                // out of its 14 bits below 256 KB): one add each instead of rebuilding them
                const uint64_t so = (uint64_t)s * (STAGE >> 4);
                const uint64_t da_hi = d0_a_hi + so, da_lo = d0_a_lo + so, db_hi = d0_b_hi + so, db_lo = d0_b_lo + so;
                const uint32_t d = tmem_d + buf * N_TILE;
#pragma unroll
                for (uint32_t kk = 0; kk < TC_K / 8; ++kk) {
                    // one instruction covers K = 8 tf32 = 32 bytes of the swizzled row
                    const uint64_t adv = kk * 2;
                    umma_tf32(d, da_hi + adv, db_hi + adv, idesc, (ks % TC_CHUNK != 0) || kk != 0);
                    if (dbg_skip & 4) continue;  // measurement only: one product of the three
                    umma_tf32(d, da_hi + adv, db_lo + adv, idesc, 1);
                    umma_tf32(d, da_lo + adv, db_hi + adv, idesc, 1);
                }
                if (tr) trace[8 * ks + 5] = tc_now();
                umma_commit(&empty[s]);  // arrives when the instructions above have finished reading the stage
                if (tr) trace[8 * ks + 6] = tc_now();
                if ((ks + 1) % TC_CHUNK == 0 || ks + 1 == k_steps) umma_commit(&acc_full[buf]);
            }
            __syncwarp();
            if (tr) trace[8 * ks + 7] = tc_now();
            if (++s == n_stages) {
                s = 0;
                ++round;
            }
        }
        if (!ok && lane == 0) abort_flag = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_flag && tid == 0) *reinterpret_cast<volatile int*>(error_flag) = 1;
    if (warp == TC_CONV_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}


// ───────────────────────────── weights through tensor memory ─────────────────────────────
//
// Second form of the tile GEMM, the one launched whenever the staged decode applies.  The weight tile's two
// TF32 terms do not pass through shared memory at all: the converter warps write them with tcgen05.st into
// tensor memory and the tensor core reads its A operand from there, so that shared memory carries only the
// activation tiles (TMA in, MMA out).  At a 128-token tile that halves the shared-memory bytes a K step moves
// (the first form's bound: 96 KB of operand reads + 64 KB of tile writes per step against 128 bytes per clock).
//
// Tensor memory, 512 columns: [0, 2N) two accumulators (a chunk of TS_CHUNK steps each), then four stages of 64
// columns: the step's 32 hi terms and 32 lo terms, weight row r in lane r.  The activation ring in shared memory
// has the same four stages, so a step has one `full` and one `empty` barrier and the issuing thread one wait
// and one commit per step (its own instruction latency is what a step costs once the operands keep up).
//
// Warps: 16 converters, warp (q = w % 4, g = w / 4) owns lanes / weight rows 32q .. 32q+31 (the lanes its
// tcgen05.st and tcgen05.ld may touch) and the K steps ks = g (mod 4): it decodes all 32 columns of the step for
// its rows, so four steps are in flight across the warps of a quarter.  The four warps of a quarter share one
// staged window of raw bytes (copied 8 rows each) and hand it over through a pair of bounded mbarriers.  Warp
// 16 issues the MMAs, warp 17 the TMA copies of the activation tiles.
constexpr int TS_CHUNK = 4;
constexpr int TS_PHASES = 4;
constexpr int TS_THREADS = (TC_CONV_WARPS + 2) * 32;

__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t r[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}


// MXFP4 by the block (the tensor-memory form decodes all 32 values of a step in one thread).  The 17-byte block
// sits at any byte offset of a word-aligned row in shared memory: five aligned words and a funnel shift give the
// 16 code bytes.  The padded row stride leaves at least three readable bytes after a row's last block.
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mxfp4_load_block(uint32_t blk_addr, uint32_t codes[4], float* half_scale) {
    const uint32_t e = (lds32(blk_addr & ~3u) >> ((blk_addr & 3u) * 8)) & 0xFFu;
    const uint32_t qa = blk_addr + 1, al = qa & ~3u, sh = (qa & 3u) * 8;
    uint32_t wds[5];
#pragma unroll
    for (int i = 0; i < 5; ++i) wds[i] = lds32(al + 4 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i) codes[i] = __funnelshift_r(wds[i], wds[i + 1], sh);
    // half of the block scale 2^(e-127) (e = 0 reads as 2^-127, src/mxfp4.rs:83-94), exact also when subnormal;
    // a NaN scale (0xFF) decodes to zeros
    *half_scale = e == 0xFFu ? 0.0f : __uint_as_float(e >= 2 ? (e - 1) << 23 : e == 1 ? 0x00400000u : 0x00200000u);
}
// Values 16h .. 16h+15 of the block: the low (h = 0) or high nibbles of the 16 code bytes.  An E2M1 code is
// sign | magnitude index into {0, .5, 1, 1.5, 2, 3, 4, 6}; twice the magnitude comes from a byte table by
// `prmt`, four codes at a time, and (2 * magnitude) * (scale / 2) is the exact product the reference forms.
__device__ __forceinline__ void mxfp4_half(const uint32_t codes[4], uint32_t h, float half_scale, float v[16]) {
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const uint32_t c = codes[wi] >> (4 * h);
        const uint32_t x = c & 0x07070707u, y = x | (x >> 4);
        const uint32_t sel = (y & 0xFFu) | ((y >> 8) & 0xFF00u);
        const uint32_t m2 = __byte_perm(0x03020100u, 0x0C080604u, sel);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float mag = (float)((m2 >> (8 * b)) & 0xFFu);
            const uint32_t sign = (c << (28 - 8 * b)) & 0x80000000u;
            v[4 * wi + b] = __fmul_rn(__uint_as_float(__float_as_uint(mag) | sign), half_scale);
        }
    }
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
__global__ void __launch_bounds__(TS_THREADS, 1)
    gemm_ts_kernel(const uint8_t* __restrict__ w_a, uint64_t n, uint64_t k, const __grid_constant__ CUtensorMap map_hi,
                   const __grid_constant__ CUtensorMap map_lo, uint64_t m_rows, float* __restrict__ dst_a,
                   int* __restrict__ error_flag, const GemmTile* __restrict__ tiles, const uint32_t* __restrict__ n_tiles,
                   uint64_t expert_bytes, const uint8_t* __restrict__ w_b, float* __restrict__ dst_b) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    if (tiles != nullptr && blockIdx.y >= *n_tiles) return;  // the launch covers the list's capacity, not its length
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t PLANE_B = N_TILE * 128;
    constexpr uint32_t STAGE = 2 * PLANE_B;  // activations hi | lo
    constexpr uint32_t TS_STAGES = TS_PHASES;  // step ks uses stage ks % 4 of both rings: the stage of its warps
    constexpr uint32_t A_COL0 = 2 * N_TILE;
    constexpr uint32_t WIN_STEPS = window_elems(TYPE) / TC_K;
    constexpr uint32_t WIN_WORDS = window_elems(TYPE) / ELEMS * BYTES / 4;
    constexpr uint32_t WIN_STRIDE = WIN_WORDS | 1u;
    constexpr int MY_COLS = N_TILE / 4;
    // MXFP4 weights (an E2M1 value times a power of two) are TF32 numbers already: no remainder term, two products
    constexpr bool EXACT_TF32 = TYPE == T_MXFP4;
    static_assert(2 * N_TILE + 64 * TS_STAGES <= 512 && WIN_STEPS % TS_PHASES == 0 && MY_COLS % 8 == 0, "tile shape");
    // full[s]: the step's four converter warps + the TMA thread (and the tiles' bytes); empty[s]: the MMAs' commit
    __shared__ uint64_t full[TS_STAGES], empty[TS_STAGES], acc_full[2], acc_empty[2], raw_full[4], raw_empty[4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t row0 = (uint64_t)blockIdx.x * TC_M;
    // plain form: token tile blockIdx.y of lhs[m_rows, k].  Grouped form: tile blockIdx.y of the list, its
    // expert's slice of the bank (blockIdx.z picks the bank and its destination); rows of the tile box beyond
    // the tile's count belong to other experts, are multiplied along and never stored.
    uint64_t tok0 = (uint64_t)blockIdx.y * N_TILE, m = m_rows;
    const uint8_t* w = blockIdx.z ? w_b : w_a;
    float* dst = blockIdx.z ? dst_b : dst_a;
    if (tiles != nullptr) {
        const GemmTile t = tiles[blockIdx.y];
        w += (uint64_t)t.expert * expert_bytes;
        tok0 = t.row0;
        m = (uint64_t)t.row0 + t.cnt;
    }
    const uint32_t k_steps = (uint32_t)(k / TC_K);
    const uint32_t n_chunks = (k_steps + TS_CHUNK - 1) / TS_CHUNK;
    const uint32_t n_windows = k_steps / WIN_STEPS;
    const uint64_t row_bytes = k / ELEMS * BYTES;
    uint32_t* raw = reinterpret_cast<uint32_t*>(smem + (size_t)TS_STAGES * STAGE);

    if (tid == 0) {
        for (uint32_t s = 0; s < TS_STAGES; ++s) {
            mbar_init(&full[s], 4 + 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TC_CONV_WARPS);
        }
        for (int q = 0; q < 4; ++q) {
            mbar_init(&raw_full[q], TS_PHASES);
            mbar_init(&raw_empty[q], TS_PHASES);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_CONV_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    if (warp < TC_CONV_WARPS) {
        const uint32_t q = warp & 3, g = warp >> 2;
        const uint32_t lane_base = (q * 32) << 16;  // this warp's quarter of the tensor-memory lanes
        float sums[MY_COLS];
#pragma unroll
        for (int c = 0; c < MY_COLS; ++c) sums[c] = 0.0f;
        auto drain = [&](uint32_t c) -> bool {
            const uint32_t buf = c & 1;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&acc_full[buf], (c >> 1) & 1))) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_d + lane_base + buf * N_TILE + g * MY_COLS;
            if constexpr (MY_COLS == 8) {
                uint32_t rr[8];
                tmem_ld8(taddr, rr);
#pragma unroll
                for (int i = 0; i < 8; ++i) sums[i] += __uint_as_float(rr[i]);
            } else {
#pragma unroll
                for (int part = 0; part < MY_COLS / 16; ++part) {
                    uint32_t rr[16];
                    tmem_ld16(taddr + part * 16, rr);
#pragma unroll
                    for (int i = 0; i < 16; ++i) sums[part * 16 + i] += __uint_as_float(rr[i]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            return true;
        };
        // this warp's 8 of the quarter's 32 rows of window wn, consecutive lanes consecutive words
        uint32_t* q_raw = raw + q * 32 * WIN_STRIDE;
        auto copy_window = [&](uint32_t wn) {
            const uint64_t gr0 = row0 + q * 32 + g * 8;
            const uint32_t dst0 = smem_u32(q_raw + g * 8 * WIN_STRIDE) + lane * 4;
#pragma unroll 1
            for (uint32_t rr = 0; rr < 8; ++rr) {
                const uint64_t gr = gr0 + rr < n ? gr0 + rr : n - 1;
                const uint8_t* src = w + gr * row_bytes + ((uint64_t)wn * WIN_WORDS + lane) * 4;
                const uint32_t dstp = dst0 + rr * (WIN_STRIDE * 4);
#pragma unroll
                for (uint32_t c = 0; c < WIN_WORDS; c += 32) {
                    if (c + lane < WIN_WORDS)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dstp + c * 4), "l"(src + c * 4) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        const uint8_t* my_row = reinterpret_cast<const uint8_t*>(q_raw + lane * WIN_STRIDE);
        bool ok = true;
        uint32_t drained = 0;
        copy_window(0);
        for (uint32_t ks = g; ks < k_steps && ok; ks += TS_PHASES) {
            const uint32_t a = g, a_round = ks / TS_STAGES;
            const uint32_t wn = ks / WIN_STEPS, wj = ks - wn * WIN_STEPS;
            if (wj < TS_PHASES) {
                // first step of mine in this window: my copies have landed; hand them over and wait for the others'
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_full[q]);
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(&raw_full[q], wn & 1));
                if (!ok) break;
            }
            // the stage's columns must have been read by the MMAs that used them last
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&empty[a], (a_round & 1) ^ 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acol = tmem_d + lane_base + A_COL0 + a * 64;
            [[maybe_unused]] uint32_t fp4_codes[4];
            [[maybe_unused]] float fp4_half_scale;
            if constexpr (TYPE == T_MXFP4) mxfp4_load_block(smem_u32(my_row) + wj * 17, fp4_codes, &fp4_half_scale);
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {  // 16 columns at a time: hi terms, then the remainders
                float v[16];
                if constexpr (TYPE == T_MXFP4) {
                    mxfp4_half(fp4_codes, h, fp4_half_scale, v);
                } else {
                    decode_unit<TYPE, LdShared>(my_row, wj * 4 + 2 * h, v, false);
                    decode_unit<TYPE, LdShared>(my_row, wj * 4 + 2 * h + 1, v + 8, false);
                }
                uint32_t t[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(v[i]) & 0xFFFFE000u;
                tmem_st16(acol + 16 * h, t);
                if constexpr (!EXACT_TF32) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(v[i] - __uint_as_float(t[i]));
                    tmem_st16(acol + 32 + 16 * h, t);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[a]);
            if (wj + TS_PHASES >= WIN_STEPS && wn + 1 < n_windows) {
                // my last step in this window: once the quarter's other warps are through with it too, bring in
                // my rows of the next one
                if (lane == 0) mbar_arrive(&raw_empty[q]);
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(&raw_empty[q], wn & 1));
                if (!ok) break;
                copy_window(wn + 1);
            }
            // drain every finished chunk but the newest
            while (ok && drained + 1 < ks / TS_CHUNK + 1) ok = drain(drained++);
        }
        while (ok && drained < n_chunks) ok = drain(drained++);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok) abort_flag = 1;
        if (ok) {
            const uint64_t out_row = row0 + q * 32 + lane;
#pragma unroll
            for (int c = 0; c < MY_COLS; ++c) {
                const uint64_t tok = tok0 + g * MY_COLS + c;
                if (tok < m && out_row < n) dst[tok * n + out_row] = sums[c];
            }
        }
    } else if (warp == TC_CONV_WARPS) {
        // ── issuer ──
        const uint32_t idesc = umma_idesc(N_TILE);
        const uint32_t base0 = smem_u32(smem);
        const uint64_t d0_b_hi = umma_desc(base0), d0_b_lo = umma_desc(base0 + PLANE_B);
        bool ok = true;
        for (uint32_t ks = 0; ks < k_steps && ok; ++ks) {
            const uint32_t chunk = ks / TS_CHUNK, buf = chunk & 1;
            const uint32_t s = ks % TS_STAGES, round = ks / TS_STAGES;
            if (s == 0 && chunk >= 2) {
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(&acc_empty[buf], ((chunk >> 1) - 1) & 1));
                if (!ok) break;
            }
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&full[s], round & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");  // the converters' tcgen05.st / .ld
            if (elect_one()) {
                const uint64_t so = (uint64_t)s * (STAGE >> 4);
                const uint64_t db_hi = d0_b_hi + so, db_lo = d0_b_lo + so;
                const uint32_t d = tmem_d + buf * N_TILE;
                const uint32_t a_hi = tmem_d + A_COL0 + s * 64, a_lo = a_hi + 32;
#pragma unroll
                for (uint32_t kk = 0; kk < TC_K / 8; ++kk) {
                    const uint64_t adv = kk * 2;  // 32 bytes of the swizzled activation row = 8 columns of A
                    if (kk == 0)
                        umma_tf32_ts(d, a_hi, db_hi, idesc, s != 0);  // a chunk's first product overwrites
                    else
                        umma_tf32_ts(d, a_hi + kk * 8, db_hi + adv, idesc, 1);
                    umma_tf32_ts(d, a_hi + kk * 8, db_lo + adv, idesc, 1);
                    if constexpr (!EXACT_TF32) umma_tf32_ts(d, a_lo + kk * 8, db_hi + adv, idesc, 1);
                }
                umma_commit(&empty[s]);  // both the weight columns and the activation tiles of the stage are free
                if (s == TS_STAGES - 1 || ks + 1 == k_steps) umma_commit(&acc_full[buf]);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) abort_flag = 1;
    } else {
        // ── activation tiles: one lane keeps the ring of TMA copies full ──
        if (lane == 0) {
            bool ok = true;
            for (uint32_t ks = 0; ks < k_steps && ok; ++ks) {
                const uint32_t s = ks % TS_STAGES, round = ks / TS_STAGES;
                ok = mbar_wait(&empty[s], (round & 1) ^ 1);
                if (!ok) break;
                uint8_t* st = smem + (size_t)s * STAGE;
                mbar_arrive_expect_tx(&full[s], 2 * PLANE_B);
                tma_load_2d(st, &map_hi, ks * TC_K, (uint32_t)tok0, &full[s]);
                tma_load_2d(st + PLANE_B, &map_lo, ks * TC_K, (uint32_t)tok0, &full[s]);
            }
            if (!ok) abort_flag = 1;
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_flag && tid == 0) *reinterpret_cast<volatile int*>(error_flag) = 1;
    if (warp == TC_CONV_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512u) : "memory");
    }
}

PFN_cuTensorMapEncodeTiled g_encode_tiled = nullptr;

cudaError_t tensor_map_for(const float* base, uint64_t m, uint64_t k, uint32_t n_tile, CUtensorMap* out) {
    if (!g_encode_tiled) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
        g_encode_tiled = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
    }
    const cuuint64_t dims[2] = {k, m};
    const cuuint64_t strides[1] = {k * 4};             // bytes between rows (a multiple of 16: k % 32 == 0)
    const cuuint32_t box[2] = {(cuuint32_t)TC_K, n_tile};  // 32 floats = one 128-byte swizzled row, n_tile rows
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_tiled(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);  // rows beyond m read as zeros
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
cudaError_t launch_tile(const uint8_t* w, uint64_t n, uint64_t k, const float* x_hi, const float* x_lo, uint64_t m,
                        float* dst, int* error_flag, cudaStream_t s) {
    constexpr uint32_t STAGE = 2 * PLANE_A + 2 * N_TILE * 128;
    uint32_t n_stages = std::min<uint32_t>(8, std::min<uint32_t>((uint32_t)(k / TC_K), (216 * 1024) / STAGE));
    size_t smem = (size_t)n_stages * STAGE + 1024;
    auto kern = gemm_tc_kernel<TYPE, ELEMS, BYTES, N_TILE>;
    static bool configured[MAX_DEVICES] = {};
    if (cudaError_t ce = set_max_smem_once(kern, 226 * 1024, configured); ce != cudaSuccess) return ce;
    CUtensorMap map_hi, map_lo;
    cudaError_t e = tensor_map_for(x_hi, m, k, N_TILE, &map_hi);
    if (e == cudaSuccess) e = tensor_map_for(x_lo, m, k, N_TILE, &map_lo);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((n + TC_M - 1) / TC_M), (unsigned)((m + N_TILE - 1) / N_TILE));
    // JQ_DEBUG_TC_SKIP (measurement only, results are wrong): bit 0 = no weight decode / stores, bit 1 = no TMA,
    // bit 2 = one tensor-core product instead of three
#ifdef JQ_PROFILING
    static const int dbg_skip = std::getenv("JQ_DEBUG_TC_SKIP") ? std::atoi(std::getenv("JQ_DEBUG_TC_SKIP")) : 0;
#else
    constexpr int dbg_skip = 0;  // the measurement switch exists in profiling builds only
#endif
    kern<<<grid, TC_THREADS, smem, s>>>(w, n, k, map_hi, map_lo, m, dst, n_stages, error_flag, g_gemm_trace, dbg_skip);
    return cudaGetLastError();
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
cudaError_t launch_ts_tile(const uint8_t* w, uint64_t n, uint64_t k, const float* x_hi, const float* x_lo, uint64_t m,
                           float* dst, int* error_flag, cudaStream_t s) {
    constexpr uint32_t STAGE = 2 * N_TILE * 128;
    constexpr uint32_t RAW = TC_M * ((window_elems(TYPE) / ELEMS * BYTES / 4) | 1u) * 4;
    size_t smem = (size_t)TS_PHASES * STAGE + RAW + 1024;  // at most 4 x 32 KB + 35 KB
    auto kern = gemm_ts_kernel<TYPE, ELEMS, BYTES, N_TILE>;
    static bool configured[MAX_DEVICES] = {};
    if (cudaError_t ce = set_max_smem_once(kern, 226 * 1024, configured); ce != cudaSuccess) return ce;
    CUtensorMap map_hi, map_lo;
    cudaError_t e = tensor_map_for(x_hi, m, k, N_TILE, &map_hi);
    if (e == cudaSuccess) e = tensor_map_for(x_lo, m, k, N_TILE, &map_lo);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((n + TC_M - 1) / TC_M), (unsigned)((m + N_TILE - 1) / N_TILE));
    kern<<<grid, TS_THREADS, smem, s>>>(w, n, k, map_hi, map_lo, m, dst, error_flag, nullptr, nullptr, 0, nullptr, nullptr);
    return cudaGetLastError();
}

// Tile width of the tensor-memory form for m activation rows.  128 tokens is its widest tile: two accumulators
// and four weight stages fill the 512 columns, and the four weight stages are what lets each stage belong to one
// group of warps (with fewer, two groups would share a stage and a parity wait could run a whole use ahead).
template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
cudaError_t launch_ts(const uint8_t* w, uint64_t n, uint64_t k, const float* x_hi, const float* x_lo, uint64_t m,
                      float* dst, int* error_flag, cudaStream_t s) {
    if (m <= 32) return launch_ts_tile<TYPE, ELEMS, BYTES, 32>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
    if (m <= 64) return launch_ts_tile<TYPE, ELEMS, BYTES, 64>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
    if (m <= 128) return launch_ts_tile<TYPE, ELEMS, BYTES, 128>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
    return launch_ts_tile<TYPE, ELEMS, BYTES, 128>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES, int N_TILE>
cudaError_t launch_grouped_tiles(const uint8_t* bank_a, const uint8_t* bank_b, uint64_t expert_bytes, uint64_t n, uint64_t k,
                                 const float* x_hi, const float* x_lo, uint64_t rows, float* dst_a, float* dst_b,
                                 const GemmTile* tiles, uint32_t max_tiles, const uint32_t* n_tiles, int* error_flag,
                                 cudaStream_t s) {
    constexpr uint32_t STAGE = 2 * N_TILE * 128;
    constexpr uint32_t RAW = TC_M * ((window_elems(TYPE) / ELEMS * BYTES / 4) | 1u) * 4;
    size_t smem = (size_t)TS_PHASES * STAGE + RAW + 1024;
    auto kern = gemm_ts_kernel<TYPE, ELEMS, BYTES, N_TILE>;
    static bool configured[MAX_DEVICES] = {};
    if (cudaError_t ce = set_max_smem_once(kern, 226 * 1024, configured); ce != cudaSuccess) return ce;
    CUtensorMap map_hi, map_lo;
    cudaError_t e = tensor_map_for(x_hi, rows, k, N_TILE, &map_hi);
    if (e == cudaSuccess) e = tensor_map_for(x_lo, rows, k, N_TILE, &map_lo);
    if (e != cudaSuccess) return e;
    if (max_tiles > 65535) return cudaErrorInvalidValue;  // the tile list is walked along grid.y
    dim3 grid((unsigned)((n + TC_M - 1) / TC_M), max_tiles, bank_b ? 2 : 1);
    kern<<<grid, TS_THREADS, smem, s>>>(bank_a, n, k, map_hi, map_lo, rows, dst_a, error_flag, tiles, n_tiles, expert_bytes,
                                        bank_b, dst_b);
    return cudaGetLastError();
}

template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
cudaError_t launch_grouped_type(const uint8_t* bank_a, const uint8_t* bank_b, uint64_t expert_bytes, uint64_t n, uint64_t k,
                                const float* x, uint64_t rows, float* dst_a, float* dst_b, const GemmTile* narrow,
                                uint32_t max_narrow, const GemmTile* wide, uint32_t max_wide, const uint32_t* counts,
                                float* scratch, int* error_flag, cudaStream_t s) {
    float* x_hi = scratch;
    float* x_lo = scratch + ((rows * k + 63) & ~(uint64_t)63);
    const uint64_t n4 = rows * k / 4;
    split_tf32_kernel<<<(unsigned)std::min<uint64_t>((n4 + 255) / 256, 148 * 16), 256, 0, s>>>(x, n4, x_hi, x_lo);
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    if (max_narrow) {
        cudaError_t e = launch_grouped_tiles<TYPE, ELEMS, BYTES, 32>(bank_a, bank_b, expert_bytes, n, k, x_hi, x_lo, rows, dst_a,
                                                                      dst_b, narrow, max_narrow, counts, error_flag, s);
        if (e != cudaSuccess) return e;
    }
    if (max_wide)
        return launch_grouped_tiles<TYPE, ELEMS, BYTES, 128>(bank_a, bank_b, expert_bytes, n, k, x_hi, x_lo, rows, dst_a, dst_b,
                                                             wide, max_wide, counts + 1, error_flag, s);
    return cudaSuccess;
}

// Splits the activations once (hi and lo arrays of m * k floats each), then the tensor-memory form where the
// weight rows are word-aligned and k is a whole number of staged windows, else the shared-memory form.
template <uint32_t TYPE, uint32_t ELEMS, uint32_t BYTES>
cudaError_t launch_type(const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m, float* dst,
                        float* scratch, int* error_flag, cudaStream_t s) {
    float* x_hi = scratch;
    float* x_lo = scratch + ((m * k + 63) & ~(uint64_t)63);
    const uint64_t n4 = m * k / 4;
    split_tf32_kernel<<<(unsigned)std::min<uint64_t>((n4 + 255) / 256, 148 * 16), 256, 0, s>>>(lhs, n4, x_hi, x_lo);
    if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    const uint64_t row_bytes = k / ELEMS * BYTES;
    if (reinterpret_cast<uintptr_t>(w) % 4 == 0 && row_bytes % 4 == 0 && k % window_elems(TYPE) == 0)
        return launch_ts<TYPE, ELEMS, BYTES>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
    if (m <= 32) return launch_tile<TYPE, ELEMS, BYTES, 32>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
    if (m <= 64) return launch_tile<TYPE, ELEMS, BYTES, 64>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
    return launch_tile<TYPE, ELEMS, BYTES, 128>(w, n, k, x_hi, x_lo, m, dst, error_flag, s);
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

bool gemm_tc_grouped_supports(uint32_t type, const uint8_t* bank, uint64_t n, uint64_t k) {
    Format f;
    if (n == 0 || k == 0 || !format_of(type, &f) || !gemm_tc_supports(type, bank, n, k, 128)) return false;
    const uint64_t row_bytes = k / f.elems * f.bytes;
    // the tensor-memory form's conditions; every expert's slice starts a whole number of rows into the bank
    return reinterpret_cast<uintptr_t>(bank) % 4 == 0 && row_bytes % 4 == 0 && k % window_elems(type) == 0;
}

cudaError_t launch_gemm_tc_grouped(uint32_t type, const uint8_t* bank_a, const uint8_t* bank_b, uint64_t expert_bytes,
                                   uint64_t n, uint64_t k, const float* x, uint64_t rows, float* dst_a, float* dst_b,
                                   const GemmTile* narrow, uint32_t max_narrow, const GemmTile* wide, uint32_t max_wide,
                                   const uint32_t* counts, void* scratch_v, int* error_flag, cudaStream_t s) {
    float* scratch = static_cast<float*>(scratch_v);
#define JQ_GROUPED(T, E, B)                                                                                              \
    return launch_grouped_type<T, E, B>(bank_a, bank_b, expert_bytes, n, k, x, rows, dst_a, dst_b, narrow, max_narrow, wide, \
                                        max_wide, counts, scratch, error_flag, s)
    switch (type) {
        case T_Q8_0: JQ_GROUPED(T_Q8_0, 32, 34);
        case T_Q2_K: JQ_GROUPED(T_Q2_K, 256, 84);
        case T_Q4_K: JQ_GROUPED(T_Q4_K, 256, 144);
        case T_IQ2_XXS: JQ_GROUPED(T_IQ2_XXS, 256, 66);
        case T_MXFP4: JQ_GROUPED(T_MXFP4, 32, 17);
        default: return cudaErrorInvalidValue;
    }
#undef JQ_GROUPED
}

void gemm_tc_set_trace(unsigned long long* dev_buf) { g_gemm_trace = dev_buf; }

size_t gemm_tc_scratch_bytes(uint64_t m, uint64_t k) { return (size_t)(2 * ((m * k + 63) & ~(uint64_t)63) * 4 + 256); }

cudaError_t launch_gemm_tc(uint32_t type, const uint8_t* w, uint64_t n, uint64_t k, const float* lhs, uint64_t m,
                           float* dst, void* scratch_v, int* error_flag, cudaStream_t s) {
    float* scratch = static_cast<float*>(scratch_v);
    switch (type) {
        case T_Q8_0: return launch_type<T_Q8_0, 32, 34>(w, n, k, lhs, m, dst, scratch, error_flag, s);
        case T_Q2_K: return launch_type<T_Q2_K, 256, 84>(w, n, k, lhs, m, dst, scratch, error_flag, s);
        case T_Q4_K: return launch_type<T_Q4_K, 256, 144>(w, n, k, lhs, m, dst, scratch, error_flag, s);
        case T_IQ2_XXS: return launch_type<T_IQ2_XXS, 256, 66>(w, n, k, lhs, m, dst, scratch, error_flag, s);
        case T_MXFP4: return launch_type<T_MXFP4, 32, 17>(w, n, k, lhs, m, dst, scratch, error_flag, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jq
