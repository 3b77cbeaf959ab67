// CPU oracle for the quantized-matmul path of the joshua inference engine.
//
// TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check
// and the `cpu_baseline` / `--impl reference` legs of the benchmark may load
// this library, and only as the checker or as the timed CPU baseline.  The
// CUDA library never links it and has no CPU fallback.
//
// It restates, in C++17 with AVX2/FMA intrinsics, the arithmetic of the
// reference's own CPU kernels, operation for operation, so that it can stand
// in for the Rust binary (which cannot be built where this runs: no Rust
// toolchain, and the `candle` crates it depends on are not vendored):
//
//   * block layouts and decode            src/kquant_dot.rs:53-118 (Q8_0, Q2_K, Q4_K)
//                                         src/iq2xxs.rs:32-71      (IQ2_XXS)
//                                         src/mxfp4.rs:45-113      (MXFP4)
//   * fused AVX2 dequant+dot row kernels  src/kquant_dot.rs:268-483
//                                         src/iq2xxs.rs:331-391
//   * scalar block-at-a-time row kernels  src/iq2xxs.rs:241-268, src/mxfp4.rs:208-235
//   * shape validation and no-op rules    src/quant_matmul.rs:133-185,
//                                         src/iq2xxs.rs:126-185, src/mxfp4.rs:142-202
//   * row chunking over a thread pool     src/simd.rs:128-145 (chunk = n/(4*threads))
//   * horizontal sum order                src/simd.rs:198-206
//   * MoE routing and dispatch            src/quantized_qwen3_moe.rs:396-528,
//                                         src/quantized_deepseek2.rs:343-355,522-685,
//                                         src/quantized_deepseek4.rs:47-51,440-485,1354-1500,
//                                         src/kimi_k3.rs:256-282
//
// Parity pinning.
//   IQ2_XXS decode: PINNED by the reference's golden vectors (4 blocks, 1024
//     values produced by llama.cpp's own decoder; tests/golden/iq2xxs_*).
//   MXFP4 decode and matmul: PINNED by the known-answer tests restated from
//     src/mxfp4.rs:285-457 (tests/test_oracle_mxfp4.py).
//   Q8_0 / Q2_K / Q4_K: PARITY UNPINNED.  The reference tree holds no golden
//     vector for these types (its tests compare against candle's `to_float`,
//     a third-party crate, semver range 0.11, absent here) and the reference
//     cannot be run here.  The formulas below follow the reference's own
//     source text; hand-computed known answers in tests/test_oracle_kquants.py
//     guard the bit positions.
//   MoE routing: PARITY UNPINNED for `softmax_last_dim`, `arg_sort_last_dim`
//     (tie order) and the dense f32 router matmul, which live in candle.
//
// Floating point: compiled with -ffp-contract=off.  A fused multiply-add
// occurs exactly where the reference calls one (`_mm256_fmadd_ps`,
// `_mm256_fmsub_ps`); everything else is separately rounded binary32, as in
// Rust.

#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../joshua_b200/csrc/iq2xxs_grid_packed.h"

namespace {

// ───────────────────────────── errors ─────────────────────────────────────

thread_local std::string g_err;

int fail(const std::string& msg) {
    g_err = msg;
    return -1;
}

// ───────────────────────────── formats ────────────────────────────────────

enum : int {
    T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q8_1 = 9, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12,
    T_Q5_K = 13, T_Q6_K = 14, T_Q8_K = 15, T_IQ2_XXS = 16, T_MXFP4 = 39
};

struct Fmt {
    size_t elems;
    size_t bytes;
    const char* name;
};

bool fmt_of(int type, Fmt* f) {
    switch (type) {
        case T_Q8_0: *f = {32, 34, "q8_0"}; return true;
        case T_Q2_K: *f = {256, 84, "q2_k"}; return true;
        case T_Q4_K: *f = {256, 144, "q4_k"}; return true;
        case T_IQ2_XXS: *f = {256, 66, "iq2_xxs"}; return true;
        case T_MXFP4: *f = {32, 17, "mxfp4"}; return true;
        // the types of the reference's generic path (src/quant_matmul.rs:86-100; sizes src/gguf_ext.rs:483-512)
        case T_Q4_0: *f = {32, 18, "q4_0"}; return true;
        case T_Q4_1: *f = {32, 20, "q4_1"}; return true;
        case T_Q5_0: *f = {32, 22, "q5_0"}; return true;
        case T_Q5_1: *f = {32, 24, "q5_1"}; return true;
        case T_Q8_1: *f = {32, 36, "q8_1"}; return true;
        case T_Q3_K: *f = {256, 110, "q3_k"}; return true;
        case T_Q5_K: *f = {256, 176, "q5_k"}; return true;
        case T_Q6_K: *f = {256, 210, "q6_k"}; return true;
        case T_Q8_K: *f = {256, 292, "q8_k"}; return true;
        default: return false;
    }
}

// IEEE binary16 -> binary32, exact (what `half::f16::to_f32` returns).
inline float f16_to_f32(const uint8_t* p) {
    uint16_t h = (uint16_t)(p[0] | (p[1] << 8));
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline float f32_from_bits(uint32_t b) {
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}

// Scale/min pair j (0..8) of a Q4_K block (src/kquant_dot.rs:106-118).
inline void q4k_scale_min(const uint8_t* s, int j, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// IQ2_XXS tables (src/iq2xxs.rs:438-710).  The sign table entry i is i with
// bit 7 set to the parity of its low seven bits; the codebook is expanded from
// the packed header.
struct Iq2Tables {
    uint8_t grid[256][8];
    uint8_t signs[128];
    alignas(32) float grid_f32[256][8];
    alignas(32) float signs_f32[128][8];
    Iq2Tables() {
        static const uint8_t level[3] = {8, 25, 43};
        for (int i = 0; i < 256; ++i) {
            unsigned c = JQ_IQ2XXS_GRID_PACKED[i];
            for (int j = 0; j < 8; ++j) {
                grid[i][j] = level[c % 3];
                grid_f32[i][j] = (float)grid[i][j];
                c /= 3;
            }
        }
        for (int i = 0; i < 128; ++i) {
            signs[i] = (uint8_t)(i | ((__builtin_popcount((unsigned)i) & 1) << 7));
            for (int j = 0; j < 8; ++j) signs_f32[i][j] = (signs[i] >> j) & 1 ? -1.0f : 1.0f;
        }
    }
};
const Iq2Tables& iq2() {
    static const Iq2Tables t;
    return t;
}

const float E2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                        -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

// src/mxfp4.rs:67-75
inline bool e8m0_to_f32(uint8_t e, float* out) {
    if (e == 0) {
        *out = f32_from_bits(0x00400000u);
        return true;
    }
    if (e == 0xFF) return false;
    *out = f32_from_bits((uint32_t)e << 23);
    return true;
}

// ───────────────────────── block decode (one block) ───────────────────────
//
// `two_step == false` is the form the matmul kernels execute: one fused
// multiply-subtract per weight, w = fma(q, fl(d*sc), -fl(dmin*m))
// (src/kquant_dot.rs:365-384,440-465).  `two_step == true` is the separately
// rounded form fl(fl(d1*q) - m1) that a plain `d1 * q - m1` expression gives
// (candle's `to_float`, which serves QuantizedType::dequantize/embedding,
// src/mmap_tensor.rs:140-174).  The two differ by at most one ulp.  Q8_0,
// IQ2_XXS and MXFP4 have a single form.

void decode_q8_0(const uint8_t* b, float* out) {
    float d = f16_to_f32(b);
    for (int j = 0; j < 32; ++j) out[j] = (float)(int8_t)b[2 + j] * d;
}

void decode_q2k(const uint8_t* b, float* out, bool two_step) {
    const uint8_t* scales = b;
    const uint8_t* qs = b + 16;
    float d = f16_to_f32(b + 80);
    float dmin = f16_to_f32(b + 82);
    for (int v = 0; v < 256; ++v) {
        int sg = v / 128;
        int r = v % 128;
        int j = r / 16;  // 16-value group inside the super-group
        int byte = sg * 32 + (r % 32);
        int shift = 2 * (r / 32);
        uint8_t sc = scales[sg * 8 + j];
        float d1 = d * (float)(sc & 0xF);
        float m1 = dmin * (float)(sc >> 4);
        float q = (float)((qs[byte] >> shift) & 3);
        out[v] = two_step ? (d1 * q - m1) : std::fmaf(q, d1, -m1);
    }
}

void decode_q4k(const uint8_t* b, float* out, bool two_step) {
    float d = f16_to_f32(b);
    float dmin = f16_to_f32(b + 2);
    const uint8_t* scales = b + 4;
    const uint8_t* qs = b + 16;
    for (int v = 0; v < 256; ++v) {
        int pair = v / 32;
        uint8_t sc, mn;
        q4k_scale_min(scales, pair, &sc, &mn);
        float d1 = d * (float)sc;
        float m1 = dmin * (float)mn;
        uint8_t byte = qs[32 * (v / 64) + (v % 32)];
        float q = (float)((pair % 2 == 0) ? (byte & 0xF) : (byte >> 4));
        out[v] = two_step ? (d1 * q - m1) : std::fmaf(q, d1, -m1);
    }
}

// src/iq2xxs.rs:44-71
void decode_iq2xxs(const uint8_t* b, float* out) {
    const Iq2Tables& t = iq2();
    float d = f16_to_f32(b);
    const uint8_t* qs = b + 2;
    for (int ib32 = 0; ib32 < 8; ++ib32) {
        const uint8_t* p = qs + ib32 * 8;
        uint32_t lo = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
        uint32_t hi = (uint32_t)p[4] | ((uint32_t)p[5] << 8) | ((uint32_t)p[6] << 16) | ((uint32_t)p[7] << 24);
        float db = d * (0.5f + (float)(hi >> 28)) * 0.25f;
        for (int l = 0; l < 4; ++l) {
            const uint8_t* grid = t.grid[(lo >> (8 * l)) & 0xFF];
            uint8_t signs = t.signs[(hi >> (7 * l)) & 127];
            for (int j = 0; j < 8; ++j) {
                float s = (signs & (1u << j)) ? -1.0f : 1.0f;
                out[ib32 * 32 + l * 8 + j] = db * (float)grid[j] * s;
            }
        }
    }
}

// src/mxfp4.rs:83-94
void decode_mxfp4(const uint8_t* b, float* out) {
    float d;
    if (!e8m0_to_f32(b[0], &d)) {
        for (int j = 0; j < 32; ++j) out[j] = 0.0f;
        return;
    }
    for (int j = 0; j < 16; ++j) {
        uint8_t byte = b[1 + j];
        out[j] = d * E2M1[byte & 0x0F];
        out[j + 16] = d * E2M1[byte >> 4];
    }
}

// ── the generic path's types ──
// The reference takes these decoders from candle's `k_quants::*::to_float` (not in its tree), which port ggml's
// `dequantize_row_*`; the loops below restate the published ggml layouts and operation order.  "Parity
// unpinned": the reference holds no vectors for them.
void decode_q4_0(const uint8_t* b, float* out) {
    float d = f16_to_f32(b);
    for (int j = 0; j < 16; ++j) {
        out[j] = (float)((int)(b[2 + j] & 0x0F) - 8) * d;
        out[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d;
    }
}
void decode_q4_1(const uint8_t* b, float* out) {
    float d = f16_to_f32(b), m = f16_to_f32(b + 2);
    for (int j = 0; j < 16; ++j) {
        out[j] = (float)(b[4 + j] & 0x0F) * d + m;
        out[j + 16] = (float)(b[4 + j] >> 4) * d + m;
    }
}
void decode_q5(const uint8_t* qhp, const uint8_t* qs, float d, float m, int bias, float* out) {
    uint32_t qh;
    std::memcpy(&qh, qhp, 4);
    for (int j = 0; j < 16; ++j) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        out[j] = (float)((int)((qs[j] & 0x0F) | xh0) - bias) * d + m;
        out[j + 16] = (float)((int)((qs[j] >> 4) | xh1) - bias) * d + m;
    }
}
void decode_q8_1(const uint8_t* b, float* out) {
    float d = f16_to_f32(b);
    for (int j = 0; j < 32; ++j) out[j] = (float)(int8_t)b[4 + j] * d;
}
void decode_q8k(const uint8_t* b, float* out) {
    float d;
    std::memcpy(&d, b, 4);
    for (int j = 0; j < 256; ++j) out[j] = d * (float)(int8_t)b[4 + j];
}
void decode_q3k(const uint8_t* b, float* out) {
    const uint8_t *hm = b, *q = b + 32;
    float d_all = f16_to_f32(b + 108);
    uint32_t aux[4];
    std::memcpy(aux, b + 96, 12);
    const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
    uint32_t tmp = aux[2];
    aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
    aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
    aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
    aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
    int8_t scales[16];
    std::memcpy(scales, aux, 16);
    int is = 0;
    uint8_t m = 1;
    for (int n = 0; n < 256; n += 128) {
        int shift = 0;
        for (int j = 0; j < 4; ++j) {
            float dl = d_all * (float)(scales[is++] - 32);
            for (int l = 0; l < 16; ++l)
                *out++ = dl * (float)((int)((q[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4));
            dl = d_all * (float)(scales[is++] - 32);
            for (int l = 0; l < 16; ++l)
                *out++ = dl * (float)((int)((q[l + 16] >> shift) & 3) - ((hm[l + 16] & m) ? 0 : 4));
            shift += 2;
            m <<= 1;
        }
        q += 32;
    }
}
void decode_q5k(const uint8_t* b, float* out) {
    float d = f16_to_f32(b), dmin = f16_to_f32(b + 2);
    const uint8_t *qh = b + 16, *ql = b + 48;
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int j = 0; j < 256; j += 64) {
        uint8_t sc, mn;
        q4k_scale_min(b + 4, is + 0, &sc, &mn);
        float d1 = d * (float)sc, m1 = dmin * (float)mn;
        q4k_scale_min(b + 4, is + 1, &sc, &mn);
        float d2 = d * (float)sc, m2 = dmin * (float)mn;
        for (int l = 0; l < 32; ++l) *out++ = d1 * (float)((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
        for (int l = 0; l < 32; ++l) *out++ = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
        ql += 32;
        is += 2;
        u1 <<= 2;
        u2 <<= 2;
    }
}
void decode_q6k(const uint8_t* b, float* out) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
    float d = f16_to_f32(b + 208);
    for (int n = 0; n < 256; n += 128) {
        for (int l = 0; l < 32; ++l) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            out[l] = d * (float)sc[is + 0] * (float)q1;
            out[l + 32] = d * (float)sc[is + 2] * (float)q2;
            out[l + 64] = d * (float)sc[is + 4] * (float)q3;
            out[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
        out += 128;
        ql += 64;
        qh += 32;
        sc += 8;
    }
}

inline bool is_generic_type(int type) {
    switch (type) {
        case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_Q8_1: case T_Q3_K: case T_Q5_K: case T_Q6_K:
        case T_Q8_K: return true;
        default: return false;
    }
}

void decode_block(int type, const uint8_t* b, float* out, bool two_step) {
    switch (type) {
        case T_Q4_0: decode_q4_0(b, out); break;
        case T_Q4_1: decode_q4_1(b, out); break;
        case T_Q5_0: decode_q5(b + 2, b + 6, f16_to_f32(b), 0.0f, 16, out); break;
        case T_Q5_1: decode_q5(b + 4, b + 8, f16_to_f32(b), f16_to_f32(b + 2), 0, out); break;
        case T_Q8_1: decode_q8_1(b, out); break;
        case T_Q3_K: decode_q3k(b, out); break;
        case T_Q5_K: decode_q5k(b, out); break;
        case T_Q6_K: decode_q6k(b, out); break;
        case T_Q8_K: decode_q8k(b, out); break;
        case T_Q8_0: decode_q8_0(b, out); break;
        case T_Q2_K: decode_q2k(b, out, two_step); break;
        case T_Q4_K: decode_q4k(b, out, two_step); break;
        case T_IQ2_XXS: decode_iq2xxs(b, out); break;
        case T_MXFP4: decode_mxfp4(b, out); break;
    }
}

// ───────────────────────────── thread pool ────────────────────────────────
//
// The reference spreads rows over a private rayon pool sized from
// `available_parallelism()` in contiguous chunks of max(1, n / (4*threads))
// rows, serial when threads <= 1 or n < 8 (src/simd.rs:73-83,128-145).  Work
// stealing is replaced by an atomic chunk counter; each row is still computed
// by exactly one task with the same operation sequence, so results do not
// depend on the thread count.

class Pool {
   public:
    explicit Pool(unsigned n) : n_(n) {
        for (unsigned i = 0; i + 1 < n_; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(mu_);
            stop_ = true;
            ++epoch_;
        }
        cv_.notify_all();
        for (auto& w : workers_) w.join();
    }
    unsigned size() const { return n_; }

    // Run job(chunk_index) for chunk_index in [0, n_chunks) on up to `use` threads.
    void run(size_t n_chunks, unsigned use, const std::function<void(size_t)>& job) {
        std::lock_guard<std::mutex> serial(run_mu_);
        job_ = &job;
        n_chunks_ = n_chunks;
        next_.store(0);
        unsigned helpers = std::min<unsigned>(use > 0 ? use - 1 : 0, (unsigned)workers_.size());
        {
            std::lock_guard<std::mutex> g(mu_);
            pending_ = helpers;
            wanted_ = helpers;
            ++epoch_;
        }
        cv_.notify_all();
        drain();
        std::unique_lock<std::mutex> g(mu_);
        done_cv_.wait(g, [this] { return pending_ == 0; });
        job_ = nullptr;
    }

   private:
    void drain() {
        for (;;) {
            size_t c = next_.fetch_add(1);
            if (c >= n_chunks_) break;
            (*job_)(c);
        }
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> g(mu_);
                cv_.wait(g, [&] { return epoch_ != seen; });
                seen = epoch_;
                if (stop_) return;
                if (wanted_ == 0) continue;
                --wanted_;
            }
            drain();
            {
                std::lock_guard<std::mutex> g(mu_);
                --pending_;
            }
            done_cv_.notify_one();
        }
    }
    unsigned n_;
    std::vector<std::thread> workers_;
    std::mutex mu_, run_mu_;
    std::condition_variable cv_, done_cv_;
    uint64_t epoch_ = 0;
    bool stop_ = false;
    unsigned pending_ = 0, wanted_ = 0;
    const std::function<void(size_t)>* job_ = nullptr;
    size_t n_chunks_ = 0;
    std::atomic<size_t> next_{0};
};

Pool& pool() {
    static Pool p(std::max(1u, std::thread::hardware_concurrency()));
    return p;
}

// threads == 0: all cores (the reference's default); 1: serial row loop.
template <class RowFn>
void for_each_row(size_t n, int threads, RowFn row_fn) {
    unsigned t = threads <= 0 ? pool().size() : (unsigned)threads;
    t = std::min(t, pool().size());
    if (t <= 1 || n < 8) {
        for (size_t r = 0; r < n; ++r) row_fn(r);
        return;
    }
    size_t chunk = std::max<size_t>(1, n / ((size_t)t * 4));
    size_t n_chunks = (n + chunk - 1) / chunk;
    std::function<void(size_t)> job = [&](size_t c) {
        size_t lo = c * chunk, hi = std::min(n, lo + chunk);
        for (size_t r = lo; r < hi; ++r) row_fn(r);
    };
    pool().run(n_chunks, t, job);
}

// ───────────────────────── AVX2 fused row kernels ─────────────────────────

constexpr size_t MTILE = 4;

// src/simd.rs:198-206: ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7))
inline float hsum256(__m256 v) {
    __m128 hi = _mm256_extractf128_ps(v, 1);
    __m128 lo = _mm256_castps256_ps128(v);
    __m128 s = _mm_add_ps(lo, hi);
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ps(s, _mm_shuffle_ps(s, s, 1));
    return _mm_cvtss_f32(s);
}

inline __m256 widen_u8(__m128i v) { return _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(v)); }
inline __m256 widen_i8(__m128i v) { return _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(v)); }

// src/kquant_dot.rs:268-319
void row_q8_0(size_t m, size_t k, size_t n, const float* lhs, const uint8_t* row_blocks, size_t bpr, size_t row,
              float* dst) {
    for (size_t m0 = 0; m0 < m; m0 += MTILE) {
        size_t mcnt = std::min(MTILE, m - m0);
        __m256 acc[MTILE];
        for (auto& a : acc) a = _mm256_setzero_ps();
        for (size_t b = 0; b < bpr; ++b) {
            const uint8_t* blk = row_blocks + b * 34;
            __m256 d4 = _mm256_set1_ps(f16_to_f32(blk));
            __m128i lo = _mm_loadu_si128((const __m128i*)(blk + 2));
            __m128i hi = _mm_loadu_si128((const __m128i*)(blk + 18));
            __m256 w0 = _mm256_mul_ps(widen_i8(lo), d4);
            __m256 w1 = _mm256_mul_ps(widen_i8(_mm_srli_si128(lo, 8)), d4);
            __m256 w2 = _mm256_mul_ps(widen_i8(hi), d4);
            __m256 w3 = _mm256_mul_ps(widen_i8(_mm_srli_si128(hi, 8)), d4);
            size_t base = b * 32;
            for (size_t i = 0; i < mcnt; ++i) {
                const float* a = lhs + (m0 + i) * k + base;
                acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(a), w0, acc[i]);
                acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(a + 8), w1, acc[i]);
                acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(a + 16), w2, acc[i]);
                acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(a + 24), w3, acc[i]);
            }
        }
        for (size_t i = 0; i < mcnt; ++i) dst[(m0 + i) * n + row] = hsum256(acc[i]);
    }
}

// src/kquant_dot.rs:326-400
void row_q2k(size_t m, size_t k, size_t n, const float* lhs, const uint8_t* row_blocks, size_t bpr, size_t row,
             float* dst) {
    const __m256i m3 = _mm256_set1_epi8(3);
    for (size_t m0 = 0; m0 < m; m0 += MTILE) {
        size_t mcnt = std::min(MTILE, m - m0);
        __m256 acc[MTILE];
        for (auto& a : acc) a = _mm256_setzero_ps();
        for (size_t b = 0; b < bpr; ++b) {
            const uint8_t* blk = row_blocks + b * 84;
            const uint8_t* scales = blk;
            const uint8_t* qs = blk + 16;
            float d = f16_to_f32(blk + 80);
            float dmin = f16_to_f32(blk + 82);
            size_t base = b * 256;
            for (size_t sg = 0; sg < 2; ++sg) {
                __m256i x = _mm256_loadu_si256((const __m256i*)(qs + sg * 32));
                __m256i xf[4] = {
                    _mm256_and_si256(x, m3),
                    _mm256_and_si256(_mm256_srli_epi16(x, 2), m3),
                    _mm256_and_si256(_mm256_srli_epi16(x, 4), m3),
                    _mm256_and_si256(_mm256_srli_epi16(x, 6), m3),
                };
                for (size_t j = 0; j < 8; ++j) {
                    uint8_t sc = scales[sg * 8 + j];
                    __m256 d1 = _mm256_set1_ps(d * (float)(sc & 0xF));
                    __m256 m1 = _mm256_set1_ps(dmin * (float)(sc >> 4));
                    __m256i xv = xf[j / 2];
                    __m128i bytes = (j % 2 == 0) ? _mm256_castsi256_si128(xv) : _mm256_extracti128_si256(xv, 1);
                    __m256 w0 = _mm256_fmsub_ps(widen_u8(bytes), d1, m1);
                    __m256 w1 = _mm256_fmsub_ps(widen_u8(_mm_srli_si128(bytes, 8)), d1, m1);
                    size_t a = base + sg * 128 + 16 * j;
                    for (size_t i = 0; i < mcnt; ++i) {
                        const float* p = lhs + (m0 + i) * k + a;
                        acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(p), w0, acc[i]);
                        acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(p + 8), w1, acc[i]);
                    }
                }
            }
        }
        for (size_t i = 0; i < mcnt; ++i) dst[(m0 + i) * n + row] = hsum256(acc[i]);
    }
}

// src/kquant_dot.rs:407-483
void row_q4k(size_t m, size_t k, size_t n, const float* lhs, const uint8_t* row_blocks, size_t bpr, size_t row,
             float* dst) {
    const __m256i mf = _mm256_set1_epi8(0x0F);
    for (size_t m0 = 0; m0 < m; m0 += MTILE) {
        size_t mcnt = std::min(MTILE, m - m0);
        __m256 acc[MTILE];
        for (auto& a : acc) a = _mm256_setzero_ps();
        for (size_t b = 0; b < bpr; ++b) {
            const uint8_t* blk = row_blocks + b * 144;
            float d = f16_to_f32(blk);
            float dmin = f16_to_f32(blk + 2);
            const uint8_t* scales = blk + 4;
            const uint8_t* qs = blk + 16;
            size_t base = b * 256;
            for (size_t c = 0; c < 4; ++c) {
                __m256i x = _mm256_loadu_si256((const __m256i*)(qs + c * 32));
                __m256i x_lo = _mm256_and_si256(x, mf);
                __m256i x_hi = _mm256_and_si256(_mm256_srli_epi16(x, 4), mf);
                for (size_t r = 0; r < 2; ++r) {
                    __m256i xv = r == 0 ? x_lo : x_hi;
                    uint8_t sc, mn;
                    q4k_scale_min(scales, (int)(2 * c + r), &sc, &mn);
                    __m256 d1 = _mm256_set1_ps(d * (float)sc);
                    __m256 m1 = _mm256_set1_ps(dmin * (float)mn);
                    __m128i low = _mm256_castsi256_si128(xv);
                    __m128i high = _mm256_extracti128_si256(xv, 1);
                    __m256 w0 = _mm256_fmsub_ps(widen_u8(low), d1, m1);
                    __m256 w1 = _mm256_fmsub_ps(widen_u8(_mm_srli_si128(low, 8)), d1, m1);
                    __m256 w2 = _mm256_fmsub_ps(widen_u8(high), d1, m1);
                    __m256 w3 = _mm256_fmsub_ps(widen_u8(_mm_srli_si128(high, 8)), d1, m1);
                    size_t a = base + 64 * c + 32 * r;
                    for (size_t i = 0; i < mcnt; ++i) {
                        const float* p = lhs + (m0 + i) * k + a;
                        acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(p), w0, acc[i]);
                        acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(p + 8), w1, acc[i]);
                        acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(p + 16), w2, acc[i]);
                        acc[i] = _mm256_fmadd_ps(_mm256_loadu_ps(p + 24), w3, acc[i]);
                    }
                }
            }
        }
        for (size_t i = 0; i < mcnt; ++i) dst[(m0 + i) * n + row] = hsum256(acc[i]);
    }
}

// src/iq2xxs.rs:331-391
void row_iq2xxs_avx2(size_t m, size_t k, size_t n, const float* lhs, const uint8_t* row_blocks, size_t bpr,
                     size_t row, float* dst) {
    const Iq2Tables& t = iq2();
    for (size_t m0 = 0; m0 < m; m0 += MTILE) {
        size_t mcnt = std::min(MTILE, m - m0);
        __m256 acc[MTILE];
        for (auto& a : acc) a = _mm256_setzero_ps();
        for (size_t b = 0; b < bpr; ++b) {
            const uint8_t* blk = row_blocks + b * 66;
            float d = f16_to_f32(blk);
            const uint8_t* qs = blk + 2;
            for (size_t ib32 = 0; ib32 < 8; ++ib32) {
                const uint8_t* p = qs + ib32 * 8;
                uint32_t lo, hi;
                std::memcpy(&lo, p, 4);
                std::memcpy(&hi, p + 4, 4);
                __m256 dbv = _mm256_set1_ps(d * (0.5f + (float)(hi >> 28)) * 0.25f);
                for (size_t l = 0; l < 4; ++l) {
                    size_t code = (lo >> (8 * l)) & 0xFF;
                    size_t si = (hi >> (7 * l)) & 0x7F;
                    __m256 g = _mm256_load_ps(t.grid_f32[code]);
                    __m256 s = _mm256_load_ps(t.signs_f32[si]);
                    __m256 v = _mm256_mul_ps(_mm256_mul_ps(g, s), dbv);
                    size_t c = b * 256 + ib32 * 32 + l * 8;
                    for (size_t i = 0; i < mcnt; ++i) {
                        __m256 a = _mm256_loadu_ps(lhs + (m0 + i) * k + c);
                        acc[i] = _mm256_fmadd_ps(a, v, acc[i]);
                    }
                }
            }
        }
        for (size_t i = 0; i < mcnt; ++i) dst[(m0 + i) * n + row] = hsum256(acc[i]);
    }
}

// The generic path (src/quant_matmul.rs:228-249,292-325): the weight row is decoded to f32 once, then dotted
// with every activation row, one FMA per 8 columns in 8 lanes, `hsum256` at the end.
void row_generic(int type, const Fmt& f, size_t m, size_t k, size_t n, const float* lhs, const uint8_t* row_blocks,
                 size_t bpr, size_t row, float* dst) {
    std::vector<float> wrow(k);
    for (size_t b = 0; b < bpr; ++b) decode_block(type, row_blocks + b * f.bytes, wrow.data() + b * f.elems, true);
    for (size_t i = 0; i < m; ++i) {
        __m256 acc = _mm256_setzero_ps();
        for (size_t c = 0; c + 8 <= k; c += 8)
            acc = _mm256_fmadd_ps(_mm256_loadu_ps(lhs + i * k + c), _mm256_loadu_ps(wrow.data() + c), acc);
        dst[i * n + row] = hsum256(acc);
    }
}

// Scalar block-at-a-time row (src/iq2xxs.rs:241-268, src/mxfp4.rs:208-235):
// per block acc = 0; acc += x*w (separately rounded) over the block in order;
// dst += acc.  dst must have been zero-filled.
void row_scalar_blocks(int type, const Fmt& f, size_t m, size_t k, size_t n, const float* lhs,
                       const uint8_t* row_blocks, size_t bpr, size_t row, float* dst) {
    float decoded[256];
    for (size_t b = 0; b < bpr; ++b) {
        decode_block(type, row_blocks + b * f.bytes, decoded, false);
        size_t base = b * f.elems;
        for (size_t i = 0; i < m; ++i) {
            const float* a = lhs + i * k + base;
            float acc = 0.0f;
            for (size_t j = 0; j < f.elems; ++j) acc += a[j] * decoded[j];
            dst[i * n + row] += acc;
        }
    }
}

// Shape rules shared by every entry (src/quant_matmul.rs:133-165,
// src/iq2xxs.rs:126-153, src/mxfp4.rs:142-172, src/kquant_dot.rs:217-224).
int validate(int type, size_t m, size_t k, size_t n, size_t lhs_len, size_t nbytes, size_t dst_len, Fmt* f,
             size_t* bpr) {
    if (!fmt_of(type, f)) return fail("unsupported ggml type id " + std::to_string(type));
    if (k % f->elems != 0)
        return fail(std::string(f->name) + " matmul: k=" + std::to_string(k) +
                    " is not a multiple of the block size " + std::to_string(f->elems));
    if (nbytes % f->bytes != 0)
        return fail(std::string(f->name) + ": " + std::to_string(nbytes) + " bytes is not a whole number of " +
                    std::to_string(f->bytes) + " byte blocks");
    *bpr = k / f->elems;
    if (nbytes / f->bytes != n * *bpr)
        return fail(std::string(f->name) + " matmul: rhs holds " + std::to_string(nbytes / f->bytes) +
                    " blocks, expected " + std::to_string(n * *bpr));
    if (lhs_len != m * k || dst_len != m * n)
        return fail(std::string(f->name) + " matmul: lhs/dst sized " + std::to_string(lhs_len) + "/" +
                    std::to_string(dst_len) + " expected " + std::to_string(m * k) + "/" + std::to_string(m * n));
    return 0;
}

// path 0: what the reference runs on an AVX2 host (fused AVX2 kernels for
//         Q8_0/Q2_K/Q4_K/IQ2_XXS, the scalar block loop for MXFP4).
// path 1: the scalar block-at-a-time loop for every type (the reference's
//         portable path for IQ2_XXS/MXFP4; for the k-quants it is the plain
//         sequential f32 product over decoded weights that the reference's
//         tests use as their second check, src/kquant_dot.rs:857-879).
int matmul_t(int type, size_t m, size_t k, size_t n, const float* lhs, size_t lhs_len, const uint8_t* w,
             size_t nbytes, float* dst, size_t dst_len, int threads, int path) {
    Fmt f;
    size_t bpr = 0;
    if (int rc = validate(type, m, k, n, lhs_len, nbytes, dst_len, &f, &bpr)) return rc;
    if (m == 0 || n == 0) return 0;
    bool scalar = path == 1 || type == T_MXFP4;
    if (scalar) std::fill(dst, dst + m * n, 0.0f);
    size_t row_bytes = bpr * f.bytes;
    for_each_row(n, threads, [&](size_t row) {
        const uint8_t* rb = w + row * row_bytes;
        if (scalar) {
            row_scalar_blocks(type, f, m, k, n, lhs, rb, bpr, row, dst);
            return;
        }
        if (is_generic_type(type)) {
            row_generic(type, f, m, k, n, lhs, rb, bpr, row, dst);
            return;
        }
        switch (type) {
            case T_Q8_0: row_q8_0(m, k, n, lhs, rb, bpr, row, dst); break;
            case T_Q2_K: row_q2k(m, k, n, lhs, rb, bpr, row, dst); break;
            case T_Q4_K: row_q4k(m, k, n, lhs, rb, bpr, row, dst); break;
            case T_IQ2_XXS: row_iq2xxs_avx2(m, k, n, lhs, rb, bpr, row, dst); break;
        }
    });
    return 0;
}

// ───────────────────────────────── MoE ────────────────────────────────────

enum : int { GATE_SOFTMAX = 0, GATE_SIGMOID = 1, GATE_SQRT_SOFTPLUS = 2 };
enum : int { OOB_ERROR = 0, OOB_SKIP = 1 };
enum : int { RENORM_CLAMP = 0, RENORM_PLUS_EPS = 1 };

struct MoeCfg {
    int32_t gating;
    int32_t n_expert;
    int32_t n_used;
    int32_t hidden;
    int32_t inter;
    int32_t n_group;
    int32_t topk_group;
    int32_t norm;         // renormalise the selected weights
    int32_t renorm_mode;  // RENORM_CLAMP: / clamp(sum, 6.1035156e-5, inf); RENORM_PLUS_EPS: / (sum + 1e-20)
    int32_t oob_policy;
    int32_t decode_path;  // 1: a single token takes the slot-order stack-and-sum path
    float scale;          // applied when != 0 and != 1
    float clamp;          // SwiGLU clamp, 0 = off
};

// Indices of the k largest values, descending; equal values keep the lower
// index first (a stable descending sort, which is how a comparator sort over
// indices behaves; the reference delegates to candle's `arg_sort_last_dim`).
void topk_desc(const float* v, int n, int k, uint32_t* out) {
    std::vector<uint32_t> idx(n);
    for (int i = 0; i < n; ++i) idx[i] = (uint32_t)i;
    std::stable_sort(idx.begin(), idx.end(), [&](uint32_t a, uint32_t b) { return v[a] > v[b]; });
    for (int i = 0; i < k; ++i) out[i] = idx[i];
}

inline float sigmoidf(float x) { return 1.0f / (1.0f + std::exp(-x)); }
inline float siluf(float x) { return x / (1.0f + std::exp(-x)); }
// src/quantized_deepseek4.rs:47-51
inline float softplusf(float x) { return std::max(x, 0.0f) + std::log(std::exp(-std::fabs(x)) + 1.0f); }

// Scores for one token from its router logits.
void scores_of(const MoeCfg& c, const float* logits, float* probs) {
    int E = c.n_expert;
    if (c.gating == GATE_SOFTMAX) {
        float mx = logits[0];
        for (int e = 1; e < E; ++e) mx = std::max(mx, logits[e]);
        float sum = 0.0f;
        for (int e = 0; e < E; ++e) {
            probs[e] = std::exp(logits[e] - mx);
            sum += probs[e];
        }
        for (int e = 0; e < E; ++e) probs[e] /= sum;
    } else if (c.gating == GATE_SIGMOID) {
        for (int e = 0; e < E; ++e) probs[e] = sigmoidf(logits[e]);
    } else {
        for (int e = 0; e < E; ++e) probs[e] = std::sqrt(softplusf(logits[e]));
    }
}

// Group-limited selection (src/quantized_deepseek2.rs:563-597): groups are
// scored by the sum of their two best members (sigmoid) or their best member
// (softmax); members of groups outside the top `topk_group` get -1e30 added.
void group_limit(const MoeCfg& c, float* sel) {
    if (c.n_group <= 1) return;
    int per = c.n_expert / c.n_group;
    std::vector<float> gs(c.n_group);
    for (int g = 0; g < c.n_group; ++g) {
        const float* p = sel + g * per;
        if (c.gating == GATE_SIGMOID) {
            uint32_t top2[2];
            topk_desc(p, per, 2, top2);
            gs[g] = p[top2[0]] + p[top2[1]];
        } else {
            float mx = p[0];
            for (int i = 1; i < per; ++i) mx = std::max(mx, p[i]);
            gs[g] = mx;
        }
    }
    std::vector<uint32_t> keep(c.topk_group);
    topk_desc(gs.data(), c.n_group, c.topk_group, keep.data());
    std::vector<float> mask(c.n_group, 0.0f);
    for (uint32_t g : keep) mask[g] += 1.0f;
    for (int g = 0; g < c.n_group; ++g) {
        float penalty = mask[g] * 1e30f + -1e30f;  // affine(1e30, -1e30)
        for (int i = 0; i < per; ++i) sel[g * per + i] += penalty;
    }
}

int moe_route(const MoeCfg& c, const float* logits, size_t T, const float* bias, const uint32_t* forced_ids,
              uint32_t* ids, float* wts) {
    int E = c.n_expert, K = c.n_used;
    if (K > E) return fail("moe: n_used exceeds n_expert");
    std::vector<float> probs(E), sel(E);
    for (size_t t = 0; t < T; ++t) {
        scores_of(c, logits + t * E, probs.data());
        uint32_t* id = ids + t * K;
        if (forced_ids) {
            // Hash-routed layers (src/quantized_deepseek4.rs:1375-1398): ids come
            // from a token-id table, weights still come from the gate scores.
            for (int s = 0; s < K; ++s) {
                id[s] = forced_ids[t * K + s];
                if (id[s] >= (uint32_t)E) return fail("moe: forced expert id out of range");
            }
        } else {
            for (int e = 0; e < E; ++e) sel[e] = bias ? probs[e] + bias[e] : probs[e];
            group_limit(c, sel.data());
            topk_desc(sel.data(), E, K, id);
        }
        float* w = wts + t * K;
        float sum = 0.0f;
        for (int s = 0; s < K; ++s) {
            w[s] = probs[id[s]];
            sum += w[s];
        }
        if (c.norm) {
            float denom = c.renorm_mode == RENORM_PLUS_EPS ? sum + 1e-20f : std::max(sum, 6.1035156e-5f);
            for (int s = 0; s < K; ++s) w[s] /= denom;
        }
        if (c.scale != 0.0f && c.scale != 1.0f)
            for (int s = 0; s < K; ++s) w[s] *= c.scale;
    }
    return 0;
}

struct Bank {
    int type;
    const uint8_t* base;
    size_t per_expert_bytes;
};

size_t tensor_bytes(int type, size_t rows, size_t cols) {
    Fmt f;
    if (!fmt_of(type, &f)) return 0;
    return rows * (cols / f.elems) * f.bytes;
}

// down(silu(clamp(gate x)) * clamp(up x)) for `cnt` rows
// (src/quantized_qwen3_moe.rs:396-402, src/quantized_deepseek4.rs:440-485).
int mlp_forward(const MoeCfg& c, int tg, const uint8_t* g, int tu, const uint8_t* u, int td, const uint8_t* d,
                const float* x, size_t cnt, float* out, int threads) {
    size_t h = c.hidden, I = c.inter;
    std::vector<float> gate(cnt * I), up(cnt * I);
    if (int rc = matmul_t(tg, cnt, h, I, x, cnt * h, g, tensor_bytes(tg, I, h), gate.data(), cnt * I, threads, 0))
        return rc;
    if (int rc = matmul_t(tu, cnt, h, I, x, cnt * h, u, tensor_bytes(tu, I, h), up.data(), cnt * I, threads, 0))
        return rc;
    for (size_t i = 0; i < cnt * I; ++i) {
        float gv = gate[i], uv = up[i];
        if (c.clamp > 0.0f) {
            gv = std::min(gv, c.clamp);
            uv = std::max(-c.clamp, std::min(uv, c.clamp));
        }
        gate[i] = siluf(gv) * uv;
    }
    return matmul_t(td, cnt, I, h, gate.data(), cnt * I, d, tensor_bytes(td, h, I), out, cnt * h, threads, 0);
}

int moe_dispatch(const MoeCfg& c, const float* x, size_t T, const uint32_t* ids, const float* wts, const Bank* banks,
                 const Bank* shared, float* y, int threads) {
    size_t h = c.hidden, K = c.n_used, E = c.n_expert;
    std::fill(y, y + T * h, 0.0f);
    auto run_expert = [&](size_t e, const float* xin, size_t cnt, float* out) {
        return mlp_forward(c, banks[0].type, banks[0].base + e * banks[0].per_expert_bytes, banks[1].type,
                           banks[1].base + e * banks[1].per_expert_bytes, banks[2].type,
                           banks[2].base + e * banks[2].per_expert_bytes, xin, cnt, out, threads);
    };
    if (T == 1 && c.decode_path) {
        // src/quantized_qwen3_moe.rs:504-520: k MLPs on the one row, scaled and
        // summed in slot order.
        std::vector<float> out(h);
        for (size_t s = 0; s < K; ++s) {
            if (ids[s] >= E) return fail("moe: expert id out of range in decode path");
            if (int rc = run_expert(ids[s], x, 1, out.data())) return rc;
            for (size_t j = 0; j < h; ++j) y[j] += out[j] * wts[s];
        }
    } else {
        // src/quantized_qwen3_moe.rs:459-496: token-major buckets, experts in
        // ascending id order, scaled rows added into y.
        std::vector<std::vector<std::pair<uint32_t, float>>> per(E);
        for (size_t t = 0; t < T; ++t)
            for (size_t s = 0; s < K; ++s) {
                size_t e = ids[t * K + s];
                if (e >= E) {
                    if (c.oob_policy == OOB_SKIP) continue;
                    return fail("moe: router selected expert " + std::to_string(e) + " out of " + std::to_string(E) +
                                " (token " + std::to_string(t) + ", slot " + std::to_string(s) + ")");
                }
                per[e].push_back({(uint32_t)t, wts[t * K + s]});
            }
        std::vector<float> xin, out;
        for (size_t e = 0; e < E; ++e) {
            size_t cnt = per[e].size();
            if (!cnt) continue;
            xin.resize(cnt * h);
            out.resize(cnt * h);
            for (size_t i = 0; i < cnt; ++i) std::memcpy(&xin[i * h], x + per[e][i].first * h, h * 4);
            if (int rc = run_expert(e, xin.data(), cnt, out.data())) return rc;
            for (size_t i = 0; i < cnt; ++i) {
                float w = per[e][i].second;
                float* yr = y + per[e][i].first * h;
                for (size_t j = 0; j < h; ++j) yr[j] += out[i * h + j] * w;
            }
        }
    }
    if (shared) {
        std::vector<float> out(T * h);
        if (int rc = mlp_forward(c, shared[0].type, shared[0].base, shared[1].type, shared[1].base, shared[2].type,
                                 shared[2].base, x, T, out.data(), threads))
            return rc;
        for (size_t i = 0; i < T * h; ++i) y[i] += out[i];
    }
    return 0;
}

}  // namespace

// ───────────────────────────── C entry points ─────────────────────────────

extern "C" {

const char* jo_last_error() { return g_err.c_str(); }

int jo_threads() { return (int)pool().size(); }

int jo_block_size(int type, uint64_t* elems, uint64_t* bytes) {
    Fmt f;
    if (!fmt_of(type, &f)) return fail("unsupported ggml type id " + std::to_string(type));
    *elems = f.elems;
    *bytes = f.bytes;
    return 0;
}

// e -> 2^(e-127); returns 0 and leaves *out untouched for the reserved 0xFF.
int jo_e8m0_to_f32(uint8_t e, float* out) { return e8m0_to_f32(e, out) ? 1 : 0; }

float jo_f16_to_f32(uint16_t h) {
    uint8_t b[2] = {(uint8_t)(h & 0xFF), (uint8_t)(h >> 8)};
    return f16_to_f32(b);
}

// Decode whole blocks to f32.  two_step: see decode_q4k.
int jo_dequantize(int type, const uint8_t* bytes, uint64_t nbytes, float* out, uint64_t n_out, int two_step) {
    Fmt f;
    if (!fmt_of(type, &f)) return fail("unsupported ggml type id " + std::to_string(type));
    if (nbytes % f.bytes != 0)
        return fail(std::string(f.name) + ": " + std::to_string(nbytes) + " bytes is not a whole number of " +
                    std::to_string(f.bytes) + " byte blocks");
    if (n_out != nbytes / f.bytes * f.elems)
        return fail(std::string(f.name) + ": output holds " + std::to_string(n_out) + " values, expected " +
                    std::to_string(nbytes / f.bytes * f.elems));
    size_t nb = nbytes / f.bytes;
    for (size_t b = 0; b < nb; ++b) decode_block(type, bytes + b * f.bytes, out + b * f.elems, two_step != 0);
    return 0;
}

int jo_matmul_t(int type, uint64_t m, uint64_t k, uint64_t n, const float* lhs, uint64_t lhs_len, const uint8_t* w,
                uint64_t nbytes, float* dst, uint64_t dst_len, int threads, int path) {
    return matmul_t(type, m, k, n, lhs, lhs_len, w, nbytes, dst, dst_len, threads, path);
}

// logits [T, n_expert] -> ids [T, n_used], weights [T, n_used].
int jo_moe_route(const MoeCfg* cfg, const float* logits, uint64_t T, const float* bias, const uint32_t* forced_ids,
                 uint32_t* ids, float* wts) {
    return moe_route(*cfg, logits, T, bias, forced_ids, ids, wts);
}

// Router logits the way the reference forms them: x [T,h] times the router
// matrix [n_expert, h] transposed, plain sequential f32 accumulation.
int jo_moe_logits(const float* x, uint64_t T, uint64_t h, const float* router, uint64_t E, float* logits) {
    for (size_t t = 0; t < T; ++t)
        for (size_t e = 0; e < E; ++e) {
            float acc = 0.0f;
            for (size_t j = 0; j < h; ++j) acc += x[t * h + j] * router[e * h + j];
            logits[t * E + e] = acc;
        }
    return 0;
}

// Expert banks: types[3] and bases[3] for gate, up, down, each a contiguous
// [n_expert, out, in] tensor; shared_* likewise for one optional shared expert
// (pass NULL bases to leave it out).
int jo_moe_dispatch(const MoeCfg* cfg, const float* x, uint64_t T, const uint32_t* ids, const float* wts,
                    const int32_t* types, const uint8_t* const* bases, const int32_t* shared_types,
                    const uint8_t* const* shared_bases, float* y, int threads) {
    const MoeCfg& c = *cfg;
    Bank banks[3], sh[3];
    for (int i = 0; i < 3; ++i) {
        size_t rows = i == 2 ? c.hidden : c.inter, cols = i == 2 ? c.inter : c.hidden;
        Fmt f;
        if (!fmt_of(types[i], &f)) return fail("unsupported ggml type id " + std::to_string(types[i]));
        if (cols % f.elems) return fail("moe: expert width is not a multiple of the block size");
        banks[i] = {types[i], bases[i], tensor_bytes(types[i], rows, cols)};
        if (shared_bases) {
            if (!fmt_of(shared_types[i], &f)) return fail("unsupported ggml type id");
            sh[i] = {shared_types[i], shared_bases[i], tensor_bytes(shared_types[i], rows, cols)};
        }
    }
    return moe_dispatch(c, x, T, ids, wts, banks, shared_bases ? sh : nullptr, y, threads);
}

}  // extern "C"
