/*
 * CPU oracle for the dequantize-matmul of llm-rs: Q4_K / Q6_K (the measured path) and the other
 * weight types its dispatcher accepts (F32, F16, BF16, Q8_0, Q4_0).
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the CPU code the
 * reference checks its backends against.  It is linked by tests/, by
 * __graft_entry__.smoke() and by bench.py's cpu_baseline / --impl reference
 * legs, and by nothing else; the CUDA library never calls into it.
 *
 * Pinning: the reference keeps no golden vectors on disk for this path (its
 * test compares a backend with CPU code on generated inputs), and it cannot be
 * executed here (Rust, Metal-only).  "Parity unpinned" by reference-produced
 * vectors; the restatement is pinned instead by (1) hand-derived known-answer
 * blocks, (2) an independent pure-Python/numpy restatement and (3) gguf-py's
 * dequantizers for the same GGUF block formats (fixtures in tests/golden/).
 *
 * What each function follows (paths are inside the reference project):
 *   f16/bf16 conversions ... crate `half` 2.7.1 as called at tests/ops.rs:44-45,70-71,82,124
 *   unpack_q4k_scale ....... tests/ops.rs:29-39  (same logic shaders/ops.metal:11-21)
 *   dequant_q4k_row ........ tests/ops.rs:41-59
 *   q6k_elem ............... shaders/ops.metal:28-42
 *   dequant_q6k_row ........ shaders/ops.metal:322-334 and :953-964 (no CPU code exists upstream)
 *   dense rows (F32/F16/BF16)  shaders/ops.metal:52-159 (weight widened to float, multiplied with the input)
 *   dequant_q8_0_row ....... shaders/ops.metal:192-218 (34-byte blocks: f16 scale, 32 int8)
 *   dequant_q4_0_row ....... shaders/ops.metal:161-190 (18-byte blocks: f16 scale, 16 bytes of nibbles;
 *                            element e of a block is the LOW nibble of byte e/2 for even e and the
 *                            HIGH nibble for odd e, minus 8 -- the reference's own order, which is
 *                            not the order of ggml's Q4_0, where byte j holds elements j and j+16)
 *   matmul_ref_f32 ......... tests/ops.rs:116-136 (dequantise all rows, sequential f32 accumulate)
 *   Xor / random_* ......... tests/ops.rs:14-25, 66-85, 93
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define Q4K_BLOCK_BYTES 144
#define Q6K_BLOCK_BYTES 210
#define QK_K 256

/* ---------------- scalar type conversions ---------------- */

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* IEEE binary16 -> binary32, exact (half::f16::to_f32). */
float llmrs_oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_to_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-08f;
        return bits_to_f32(f32_to_bits(v) | sign);
    }
    if (exp == 31) return bits_to_f32(sign | 0x7F800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16, round to nearest even (half::f16::from_f32). */
uint16_t llmrs_oracle_f32_to_f16(float f) {
    uint32_t x = f32_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) {               /* inf / nan */
        uint32_t man = absx & 0x7FFFFFu;
        return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0));
    }
    if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf */
    if (absx < 0x33000001u) return (uint16_t)sign;              /* rounds to zero (<= 2^-25) */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t base;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); base = 0; }
    else         { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x7FFFFFu; }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));    /* carry into the exponent is the correct result */
}

/* bf16 is the top half of binary32 (half::bf16::to_f32). */
float llmrs_oracle_bf16_to_f32(uint16_t b) { return bits_to_f32((uint32_t)b << 16); }

/* binary32 -> bf16, round to nearest even, NaN kept quiet (half::bf16::from_f32). */
uint16_t llmrs_oracle_f32_to_bf16(float f) {
    uint32_t x = f32_to_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t round_bit = 0x8000u;
    if ((x & round_bit) != 0 && (x & (3u * round_bit - 1u)) != 0) return (uint16_t)((x >> 16) + 1u);
    return (uint16_t)(x >> 16);
}

/* ---------------- Q4_K ---------------- */

/* 6-bit (scale, min) of sub-block sb (0..7) from the 12 packed bytes. tests/ops.rs:29-39 */
void llmrs_oracle_unpack_q4k_scale(const uint8_t *scales, int sb, uint32_t *sc, uint32_t *m) {
    if (sb < 4) {
        *sc = scales[sb] & 63u;
        *m = scales[sb + 4] & 63u;
    } else {
        *sc = (uint32_t)(scales[sb + 4] & 0x0Fu) | ((uint32_t)(scales[sb - 4] >> 6) << 4);
        *m = (uint32_t)(scales[sb + 4] >> 4) | ((uint32_t)(scales[sb] >> 6) << 4);
    }
}

/* One row of n_blocks Q4_K blocks -> n_blocks*256 floats. tests/ops.rs:41-59.
 * The expression is evaluated exactly as written there: ((d*sc)*q) - (dmin*m),
 * every operation in binary32; the build uses -ffp-contract=off so no fma is
 * formed (all three products are exact, so the value would not change, but the
 * oracle should not depend on that). */
void llmrs_oracle_dequant_q4k_row(const uint8_t *row, size_t n_blocks, float *out) {
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = row + b * Q4K_BLOCK_BYTES;
        float d = llmrs_oracle_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = llmrs_oracle_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *scales = blk + 4;
        const uint8_t *qs = blk + 16;
        for (int sb = 0; sb < 8; sb++) {
            uint32_t sci, mi;
            llmrs_oracle_unpack_q4k_scale(scales, sb, &sci, &mi);
            float sc = (float)sci, m = (float)mi;
            int pair = sb / 2, hi = sb % 2;
            for (int j = 0; j < 32; j++) {
                uint8_t packed = qs[pair * 32 + j];
                float q = hi ? (float)(packed >> 4) : (float)(packed & 0x0F);
                out[b * QK_K + sb * 32 + j] = d * sc * q - dmin * m;
            }
        }
    }
}

/* ---------------- Q6_K ---------------- */

/* 6-bit quant of element i (0..255) from ql[128], qh[64]. shaders/ops.metal:28-42 */
uint8_t llmrs_oracle_q6k_elem(const uint8_t *ql, const uint8_t *qh, unsigned i) {
    unsigned half_idx = i / 128, j = i % 128;
    uint8_t q_lo, q_hi;
    if (j < 64) q_lo = ql[half_idx * 64 + j] & 0x0F;
    else        q_lo = ql[half_idx * 64 + j - 64] >> 4;
    q_hi = (uint8_t)((qh[half_idx * 32 + (j % 32)] >> (2 * (j / 32))) & 3);
    return (uint8_t)(q_lo | (q_hi << 4));
}

/* One row of n_blocks Q6_K blocks -> floats: d * scales[i/16] * (q - 32).
 * shaders/ops.metal:322-334 (block layout :23-26: ql @0, qh @128, int8 scales @192, f16 d @208). */
void llmrs_oracle_dequant_q6k_row(const uint8_t *row, size_t n_blocks, float *out) {
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = row + b * Q6K_BLOCK_BYTES;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *scales = (const int8_t *)(blk + 192);
        float d = llmrs_oracle_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
        for (unsigned i = 0; i < 256; i++) {
            float sc = (float)scales[i / 16];
            float q = (float)llmrs_oracle_q6k_elem(ql, qh, i);
            out[b * QK_K + i] = d * sc * (q - 32.0f);
        }
    }
}

/* ---------------- the other weight types ---------------- */

/* Q8_0: blocks of 32 weights, 34 bytes: f16 scale then 32 int8. shaders/ops.metal:192-218 */
void llmrs_oracle_dequant_q8_0_row(const uint8_t *row, size_t n_blocks, float *out) {
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = row + b * 34;
        float scale = llmrs_oracle_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int l = 0; l < 32; l++) out[b * 32 + l] = scale * (float)(int8_t)blk[2 + l];
    }
}

/* Q4_0 as the reference's kernel reads it: blocks of 32 weights, 18 bytes: f16 scale then 16 bytes;
 * element l: byte l/2, low nibble for even l, high nibble for odd l, minus 8. shaders/ops.metal:161-190 */
void llmrs_oracle_dequant_q4_0_row(const uint8_t *row, size_t n_blocks, float *out) {
    for (size_t b = 0; b < n_blocks; b++) {
        const uint8_t *blk = row + b * 18;
        float scale = llmrs_oracle_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int l = 0; l < 32; l++) {
            uint8_t packed = blk[2 + l / 2];
            int q = (l % 2 == 0) ? (int)(packed & 0x0F) - 8 : (int)(packed >> 4) - 8;
            out[b * 32 + l] = scale * (float)q;
        }
    }
}

/* GGUF type ids (src/tensor/mod.rs:3-33): 0 F32, 1 F16, 2 Q4_0, 8 Q8_0, 12 Q4_K, 14 Q6_K, 30 BF16.
 * Elements per block and bytes per block (src/tensor/mod.rs:37-86); 0 for a type this oracle lacks. */
static size_t block_elems(int dtype) {
    switch (dtype) { case 0: case 1: case 30: return 1; case 2: case 8: return 32; case 12: case 14: return QK_K; default: return 0; }
}
static size_t block_bytes(int dtype) {
    switch (dtype) { case 0: return 4; case 1: case 30: return 2; case 2: return 18; case 8: return 34;
                     case 12: return Q4K_BLOCK_BYTES; case 14: return Q6K_BLOCK_BYTES; default: return 0; }
}
size_t llmrs_oracle_row_bytes(int dtype, size_t K) {
    size_t be = block_elems(dtype);
    return be && K % be == 0 ? K / be * block_bytes(dtype) : 0;
}
/* One weight row of K elements -> floats (every widening is exact). */
static void dequant_row(int dtype, const uint8_t *row, size_t K, float *out) {
    switch (dtype) {
    case 0: memcpy(out, row, K * 4); break;
    case 1: for (size_t i = 0; i < K; i++) out[i] = llmrs_oracle_f16_to_f32((uint16_t)(row[2 * i] | (row[2 * i + 1] << 8))); break;
    case 30: for (size_t i = 0; i < K; i++) out[i] = llmrs_oracle_bf16_to_f32((uint16_t)(row[2 * i] | (row[2 * i + 1] << 8))); break;
    case 2: llmrs_oracle_dequant_q4_0_row(row, K / 32, out); break;
    case 8: llmrs_oracle_dequant_q8_0_row(row, K / 32, out); break;
    case 12: llmrs_oracle_dequant_q4k_row(row, K / QK_K, out); break;
    default: llmrs_oracle_dequant_q6k_row(row, K / QK_K, out); break;
    }
}

/* ---------------- dequantise a whole weight ---------------- */

/* dtype: a GGUF id from the list above. Weight = N rows of K elements (K / block size consecutive blocks). */
int llmrs_oracle_dequant(int dtype, const uint8_t *w, size_t K, size_t N, float *out, int threads) {
    size_t rb = llmrs_oracle_row_bytes(dtype, K);
    if (!block_elems(dtype)) return 2;
    if (!rb) return 1;
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (long long r = 0; r < (long long)N; r++) dequant_row(dtype, w + (size_t)r * rb, K, out + (size_t)r * K);
    return 0;
}

/* ---------------- matmul (the op under test) ---------------- */

/* out[s*N + row] = sum_i W[row,i] * x[s*K + i].  tests/ops.rs:116-136.
 * acc_f64 = 0: sequential binary32 accumulate, the reference's own arithmetic.
 * acc_f64 = 1: products and sum in binary64 ("truth" for relative-L2 checks).
 * Rows row_begin..row_end only (a bounded sample for timing); output is still
 * indexed by the absolute row.  Weights are dequantised a row at a time, which
 * gives the same numbers as dequantising everything first. */
int llmrs_oracle_matmul(int dtype, const uint8_t *w, size_t K, size_t N,
                        const float *x, size_t M, float *out,
                        size_t row_begin, size_t row_end, int acc_f64, int threads) {
    size_t rb = llmrs_oracle_row_bytes(dtype, K);
    if (!block_elems(dtype)) return 2;
    if (!rb) return 1;
    if (row_end > N) row_end = N;
    (void)threads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        float *wrow = (float *)malloc(K * sizeof(float));
#pragma omp for schedule(static)
        for (long long r = (long long)row_begin; r < (long long)row_end; r++) {
            dequant_row(dtype, w + (size_t)r * rb, K, wrow);
            for (size_t s = 0; s < M; s++) {
                const float *xs = x + s * K;
                if (acc_f64) {
                    double acc = 0.0;
                    for (size_t i = 0; i < K; i++) acc += (double)wrow[i] * (double)xs[i];
                    out[s * N + (size_t)r] = (float)acc;
                } else {
                    float acc = 0.0f;            /* source order: no -ffast-math, no contraction */
                    for (size_t i = 0; i < K; i++) acc += wrow[i] * xs[i];
                    out[s * N + (size_t)r] = acc;
                }
            }
        }
        free(wrow);
    }
    return 0;
}

/* Same arithmetic as acc_f64 = 0 without the ordering barriers, so the compiler
 * may vectorise the sum: this is the "all host cores, -O3" timing baseline.  The
 * result differs from the sequential sum only by float re-association. */
int llmrs_oracle_matmul_fast(int dtype, const uint8_t *w, size_t K, size_t N,
                             const float *x, size_t M, float *out,
                             size_t row_begin, size_t row_end, int threads) {
    size_t rb = llmrs_oracle_row_bytes(dtype, K);
    if (!block_elems(dtype)) return 2;
    if (!rb) return 1;
    if (row_end > N) row_end = N;
    (void)threads;
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
    {
        float *wrow = (float *)malloc(K * sizeof(float));
#pragma omp for schedule(static)
        for (long long r = (long long)row_begin; r < (long long)row_end; r++) {
            dequant_row(dtype, w + (size_t)r * rb, K, wrow);
            for (size_t s = 0; s < M; s++) {
                const float *xs = x + s * K;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                size_t i = 0;
                for (; i + 8 <= K; i += 8)
                    for (int l = 0; l < 8; l++) acc[l] += wrow[i + l] * xs[i + l];
                for (; i < K; i++) acc[0] += wrow[i] * xs[i];
                out[s * N + (size_t)r] =
                    ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
            }
        }
        free(wrow);
    }
    return 0;
}

/* ---------------- the reference test's input generator ---------------- */

/* xorshift64 with the reference's seeding. tests/ops.rs:14-25 */
typedef struct { uint64_t s; } llmrs_xor;
static inline void xor_new(llmrs_xor *x, uint64_t seed) { x->s = (seed * 0x9E3779B97F4A7C15ull) | 1ull; }
static inline uint64_t xor_next(llmrs_xor *x) {
    uint64_t v = x->s; v ^= v << 13; v ^= v >> 7; v ^= v << 17; x->s = v; return v;
}
static inline uint8_t xor_u8(llmrs_xor *x) { return (uint8_t)xor_next(x); }
static inline float xor_f32m1p1(llmrs_xor *x) {
    return ((float)(xor_next(x) >> 40) / (float)(1u << 24)) * 2.0f - 1.0f;
}

/* Inputs of check_matmul_q4k(in_f, out_f, seq_len): tests/ops.rs:91-96 with the
 * generators at :66-77 (weights) and :79-85 (bf16 activations), drawn from ONE
 * generator in that order.  w: out_f*(in_f/256)*144 bytes; x_bf16: in_f*seq_len. */
int llmrs_oracle_ref_case_q4k(size_t in_f, size_t out_f, size_t seq_len, uint8_t *w, uint16_t *x_bf16) {
    if (in_f % QK_K) return 1;
    llmrs_xor rng;
    xor_new(&rng, 0xC0FFEEull ^ (uint64_t)(in_f * out_f * seq_len));
    size_t n_blocks = in_f * out_f / QK_K;
    for (size_t b = 0; b < n_blocks; b++) {
        uint8_t *blk = w + b * Q4K_BLOCK_BYTES;
        uint16_t d = llmrs_oracle_f32_to_f16(0.02f + ((float)xor_u8(&rng) / 255.0f) * 0.03f);
        uint16_t dmin = llmrs_oracle_f32_to_f16(0.01f + ((float)xor_u8(&rng) / 255.0f) * 0.02f);
        blk[0] = (uint8_t)d; blk[1] = (uint8_t)(d >> 8);
        blk[2] = (uint8_t)dmin; blk[3] = (uint8_t)(dmin >> 8);
        for (int i = 4; i < Q4K_BLOCK_BYTES; i++) blk[i] = xor_u8(&rng);
    }
    for (size_t i = 0; i < in_f * seq_len; i++) x_bf16[i] = llmrs_oracle_f32_to_bf16(xor_f32m1p1(&rng));
    return 0;
}

/* The reference's pass criterion, tests/ops.rs:143-154: |e-g| < max(|e|/64, 0.02*sqrt(in_f)).
 * Returns the number of failing elements; *max_rel gets max |e-g| / max(|e|, 1e-6). */
size_t llmrs_oracle_ref_tolerance_failures(const float *expected, const float *got, size_t n,
                                           size_t in_f, float *max_rel) {
    size_t bad = 0; float mr = 0.0f;
    float floor_tol = 0.02f * sqrtf((float)in_f);
    for (size_t i = 0; i < n; i++) {
        float e = expected[i], g = got[i];
        float tol = fmaxf(fabsf(e) / 64.0f, floor_tol);
        float err = fabsf(e - g);
        float rel = err / fmaxf(fabsf(e), 1e-6f);
        if (rel > mr) mr = rel;
        if (!(err < tol)) bad++;
    }
    if (max_rel) *max_rel = mr;
    return bad;
}

int llmrs_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
