/*
 * CPU oracle for the block-scaled FP8/FP4 GEMM path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links, loads or calls this file; it is the
 * checker the parity tests compare the CUDA path against, and the CPU baseline
 * the benchmark times.
 *
 * Every function restates one function of the reference crate's
 * deepgemm/src/reference.rs (cited per function), or -- where the reference
 * has no CPU definition -- states the rule this build defines (marked
 * "parity unpinned": no reference function or test constrains the value).
 *
 * Pinned against the reference's own known-answer vectors
 * (reference.rs:336-376, tests/unit.rs:72-158) by tests/test_oracle_pins.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define DGO_API __attribute__((visibility("default")))

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ------------------------------------------------------------------------ */
/* e4m3 / bf16 codecs                                                        */
/* ------------------------------------------------------------------------ */

/* reference.rs:35-54 -- S.EEEE.MMM, bias 7; 0x7F/0xFF are NaN; exp 0 is subnormal. */
DGO_API float dgo_e4m3_to_f32(uint8_t code) {
    int sign = code >> 7, e = (code >> 3) & 0xF, m = code & 7;
    float v;
    if (e == 0) v = (float)m / 8.0f * ldexpf(1.0f, -6);
    else if (e == 15 && m == 7) return NAN;
    else v = (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
    return sign ? -v : v;
}

/* reference.rs:5-32 -- exhaustive search of the 127 finite codes for the
 * nearest magnitude; an equal-distance candidate wins only if its code is
 * even; anything above 448 saturates; sign comes from (v < 0), so -0.0
 * encodes as 0x00 and a tiny negative that rounds to zero as 0x80. */
DGO_API uint8_t dgo_f32_to_e4m3(float v) {
    if (isnan(v)) return 0x7F;
    uint8_t sign = v < 0.0f ? 1 : 0;
    float a = fabsf(v);
    uint8_t best = 0;
    float best_err = INFINITY;
    for (unsigned c = 0; c < 0x7F; ++c) {
        float err = fabsf(dgo_e4m3_to_f32((uint8_t)c) - a);
        if (err < best_err || (err == best_err && (c & 1) == 0)) { best_err = err; best = (uint8_t)c; }
    }
    if (best_err > 0.0f && a > 448.0f) return (uint8_t)(sign << 7 | 0x7E);
    return (uint8_t)(best | (sign << 7));
}

/* Arithmetic round-to-nearest-even onto the e4m3 grid; must agree with
 * dgo_f32_to_e4m3 on every input (checked exhaustively over all bf16 bit
 * patterns and on random f32 by the oracle tests).  Used where the search
 * version would make a test take minutes. */
DGO_API uint8_t dgo_f32_to_e4m3_fast(float v) {
    if (isnan(v)) return 0x7F;
    uint8_t sign = v < 0.0f ? 0x80 : 0;
    float a = fabsf(v);
    if (a > 448.0f) return sign | 0x7E;
    /* spacing of the grid at magnitude a: 2^(e-3) for normals (e >= -6), 2^-9 below */
    int e;
    (void)frexpf(a, &e);          /* a = f * 2^e, f in [0.5,1) -> floor(log2 a) = e-1 */
    int ex = e - 1;
    if (a == 0.0f || ex < -6) ex = -6;
    float step = ldexpf(1.0f, ex - 3);
    float q = a / step;            /* exact: power-of-two divide */
    float r = nearbyintf(q);       /* default rounding mode = nearest even */
    float mag = r * step;
    if (mag > 448.0f) mag = 448.0f;
    /* encode magnitude (exactly representable now) */
    uint8_t code;
    if (mag == 0.0f) code = 0;
    else {
        int e2;
        float f = frexpf(mag, &e2);    /* mag = f*2^e2, f in [0.5,1) */
        int be = e2 - 1 + 7;           /* biased exponent */
        if (be <= 0) code = (uint8_t)lrintf(mag / ldexpf(1.0f, -9));
        else code = (uint8_t)((be << 3) | (int)lrintf((f * 2.0f - 1.0f) * 8.0f));
    }
    return sign | code;
}

/* reference.rs:67-76 -- round to nearest even on the low 16 bits, no NaN special case. */
DGO_API uint16_t dgo_f32_to_bf16(float v) {
    uint32_t bits = f2u(v);
    uint16_t b = (uint16_t)(bits >> 16);
    uint32_t lsb = (bits & 0xFFFF) + 0x7FFF + ((bits >> 16) & 1);
    if (lsb > 0xFFFF) b += 1;
    return b;
}

/* reference.rs:78-80 */
DGO_API float dgo_bf16_to_f32(uint16_t v) { return u2f((uint32_t)v << 16); }

/* ------------------------------------------------------------------------ */
/* e2m1 / UE8M0 codecs                                                       */
/* ------------------------------------------------------------------------ */

/* reference.rs:215-217 */
static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

DGO_API float dgo_e2m1_to_f32(uint8_t code) { return kE2M1[code & 0xF]; }

/* reference.rs:229-252 -- nearest of the 8 magnitudes, equal distance goes to
 * the even code, saturates at 6, NaN encodes as 0, -0.0 keeps its sign. */
DGO_API uint8_t dgo_encode_e2m1(float v) {
    float a = v < 0.0f ? -v : v;
    if (isnan(a)) a = 0.0f;
    if (a > 6.0f) a = 6.0f;
    uint8_t best = 0;
    float best_err = INFINITY;
    for (unsigned i = 0; i < 8; ++i) {
        float err = fabsf(a - kE2M1[i]);
        if (err < best_err || (err == best_err && (i & 1) == 0)) { best_err = err; best = (uint8_t)i; }
    }
    uint8_t sign = (v < 0.0f || (v == 0.0f && signbit(v))) ? 1 : 0;
    return (uint8_t)(best | (sign << 3));
}

/* reference.rs:255-257 -- the UE8M0 byte is the f32 biased exponent, floored at 1. */
DGO_API uint8_t dgo_f32_to_ue8m0(float sf) {
    uint32_t e = (f2u(sf) >> 23) & 0xFF;
    return (uint8_t)(e < 1 ? 1 : e);
}
/* reference.rs:260-262 */
DGO_API float dgo_ue8m0_to_f32(uint8_t e) { return u2f((uint32_t)e << 23); }

/* ------------------------------------------------------------------------ */
/* Scale selection                                                           */
/* ------------------------------------------------------------------------ */

/* Biased exponent of amax, plus one when its mantissa exceeds the largest
 * mantissa of the target format (0x600000 for 448 = 1.75*2^8, 0x400000 for
 * 6 = 1.5*2^2).  This is the carry trick of reference.rs:273 and
 * cuda/sm100_cast.rs:55. */
static inline uint32_t rounded_exp_f32(float amax, uint32_t qmant) {
    return (f2u(fabsf(amax)) + 0x7FFFFFu - qmant) >> 23;
}

/* Rule ids shared with the library's dg_cast_* entry points. */
enum { DGO_SF_RULE_REFERENCE_CPU = 0, DGO_SF_RULE_RANGE_FIT = 1 };

/* UE8M0 exponent for an e2m1 block.
 * rule 0: reference.rs:273-274 verbatim -- max(rounded, 128) clamped to [1,255];
 *         the block amax lands in (0.5, 1.5] after scaling.
 * rule 1 (parity unpinned): smallest power of two with amax/sf <= 6, i.e.
 *         max(max(rounded,2) - 2, 1), using the constants of
 *         cuda/sm100_cast.rs:51-53 with the bias subtracted instead of added. */
DGO_API uint32_t dgo_sf_exp_e2m1(float amax, int rule) {
    uint32_t r = rounded_exp_f32(amax, 0x400000u);
    if (rule == DGO_SF_RULE_REFERENCE_CPU) {
        uint32_t e = r < 128u ? 128u : r;
        if (e < 1u) e = 1u;
        if (e > 255u) e = 255u;
        return e;
    }
    uint32_t e = (r < 2u ? 2u : r) - 2u;
    return e < 1u ? 1u : e;
}

/* UE8M0 exponent for an e4m3 block (parity unpinned: the reference has no CPU
 * FP8+UE8M0 quantizer): smallest power of two with amax/sf <= 448, floored at
 * 2^-22 -- max(max(rounded,8) - 8, 105), constants of cuda/sm100_cast.rs:51-53. */
DGO_API uint32_t dgo_sf_exp_e4m3(float amax) {
    uint32_t r = rounded_exp_f32(amax, 0x600000u);
    uint32_t e = (r < 8u ? 8u : r) - 8u;
    return e < 105u ? 105u : e;
}

/* Same selection from a bf16 amax bit pattern (the FP8-requantize epilogue,
 * cuda/sm100_common.rs:791-803 with the same bias correction). */
DGO_API uint32_t dgo_sf_exp_e4m3_bf16(uint16_t amax_bits) {
    uint32_t r = ((uint32_t)(amax_bits & 0x7FFF) + 0x7Fu - 0x60u) >> 7;
    uint32_t e = (r < 8u ? 8u : r) - 8u;
    return e < 105u ? 105u : e;
}

static inline float sf_inv(uint32_t sf_exp) { return u2f((254u - sf_exp) << 23); }

/* ------------------------------------------------------------------------ */
/* Packed scale-factor layout                                                */
/* ------------------------------------------------------------------------ */

static inline size_t align4(size_t x) { return (x + 3) / 4 * 4; }

/* Word index of (group g, local row r, word column c):
 * (g*cols + c)*align4(group_rows) + r   (tests/e2e.rs:413-430, sm100_cast.rs:69-73). */
static inline size_t sf_word_index(size_t g, size_t cols, size_t c, size_t stride, size_t r) {
    return (g * cols + c) * stride + r;
}

DGO_API size_t dgo_sf_words(uint32_t rows, uint32_t k, uint32_t gran, uint32_t groups) {
    if (groups == 0) groups = 1;
    size_t cols = (k + 4 * gran - 1) / (4 * gran);
    return cols * groups * align4(rows / groups);
}

/* ------------------------------------------------------------------------ */
/* Quantizers                                                                */
/* ------------------------------------------------------------------------ */

/* reference.rs:266-285 generalised over rows/groups and the packed layout of
 * tests/unit.rs:125-135 / tests/e2e.rs:413-430.  src is bf16 bits (rows, ld).
 * rule 0 multiplies by 1.0f/sf exactly as reference.rs:276 does. */
DGO_API void dgo_cast_bf16_to_fp4_packed_sf(const uint16_t* src, uint32_t ld, uint32_t rows, uint32_t k,
                                            uint32_t groups, int rule, uint8_t* dst, uint32_t* sf) {
    if (groups == 0) groups = 1;
    size_t group_rows = rows / groups, stride = align4(group_rows), cols = (k + 127) / 128;
    memset(sf, 0, cols * groups * stride * 4);
    #pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        size_t g = (size_t)r / group_rows, lr = (size_t)r - g * group_rows;
        for (uint32_t blk = 0; blk < k / 32; ++blk) {
            const uint16_t* p = src + (size_t)r * ld + blk * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) { float a = fabsf(dgo_bf16_to_f32(p[i])); if (a > amax) amax = a; }
            uint32_t e = dgo_sf_exp_e2m1(amax, rule);
            float inv = rule == DGO_SF_RULE_REFERENCE_CPU ? 1.0f / u2f(e << 23) : sf_inv(e);
            for (int i = 0; i < 32; i += 2) {
                uint8_t lo = dgo_encode_e2m1(dgo_bf16_to_f32(p[i]) * inv);
                uint8_t hi = dgo_encode_e2m1(dgo_bf16_to_f32(p[i + 1]) * inv);
                dst[(size_t)r * (k / 2) + (blk * 32 + i) / 2] = (uint8_t)(lo | (hi << 4));
            }
            sf[sf_word_index(g, cols, blk / 4, stride, lr)] |= e << ((blk % 4) * 8);
        }
    }
}

/* bf16 -> e4m3 + packed UE8M0 per gran (32 or 128) K elements.  Parity
 * unpinned (see dgo_sf_exp_e4m3).  Scaling by 2^(127-e) is exact in f32; a
 * product of exactly -0.0 is encoded as +0 because the reference encoder
 * takes the sign from (v < 0). */
DGO_API void dgo_cast_bf16_to_fp8_sf(const uint16_t* src, uint32_t ld, uint32_t rows, uint32_t k,
                                     uint32_t gran, uint32_t groups, uint8_t* dst, uint32_t* sf) {
    if (groups == 0) groups = 1;
    size_t group_rows = rows / groups, stride = align4(group_rows), cols = (k + 4 * gran - 1) / (4 * gran);
    memset(sf, 0, cols * groups * stride * 4);
    #pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        size_t g = (size_t)r / group_rows, lr = (size_t)r - g * group_rows;
        for (uint32_t blk = 0; blk < k / gran; ++blk) {
            const uint16_t* p = src + (size_t)r * ld + (size_t)blk * gran;
            float amax = 0.0f;
            for (uint32_t i = 0; i < gran; ++i) { float a = fabsf(dgo_bf16_to_f32(p[i])); if (a > amax) amax = a; }
            uint32_t e = dgo_sf_exp_e4m3(amax);
            float inv = sf_inv(e);
            for (uint32_t i = 0; i < gran; ++i)
                dst[(size_t)r * k + (size_t)blk * gran + i] = dgo_f32_to_e4m3_fast(dgo_bf16_to_f32(p[i]) * inv);
            sf[sf_word_index(g, cols, blk / 4, stride, lr)] |= e << ((blk % 4) * 8);
        }
    }
}

/* bf16 -> e4m3 with one UE8M0 exponent per block_rows x 128 block (block_rows = 128 is the
 * weight recipe whose scales reference.rs:105 indexes per 128-row tile).  Same exponent rule
 * as dgo_cast_bf16_to_fp8_sf (parity unpinned).  exps: (ceil(rows/block_rows), k/128) bytes. */
DGO_API void dgo_quantize_fp8_ue8m0_blocks(const uint16_t* src, uint32_t ld, uint32_t rows, uint32_t k,
                                           uint32_t block_rows, uint8_t* dst, uint8_t* exps) {
    uint32_t kb_n = k / 128, rb_n = (rows + block_rows - 1) / block_rows;
    #pragma omp parallel for schedule(static)
    for (long rb = 0; rb < (long)rb_n; ++rb)
        for (uint32_t kb = 0; kb < kb_n; ++kb) {
            uint32_t r0 = (uint32_t)rb * block_rows, r1 = r0 + block_rows < rows ? r0 + block_rows : rows;
            float amax = 0.0f;
            for (uint32_t r = r0; r < r1; ++r)
                for (uint32_t c = kb * 128; c < kb * 128 + 128; ++c) {
                    float a = fabsf(dgo_bf16_to_f32(src[(size_t)r * ld + c]));
                    if (a > amax) amax = a;
                }
            uint32_t e = dgo_sf_exp_e4m3(amax);
            float inv = sf_inv(e);
            exps[(size_t)rb * kb_n + kb] = (uint8_t)e;
            for (uint32_t r = r0; r < r1; ++r)
                for (uint32_t c = kb * 128; c < kb * 128 + 128; ++c)
                    dst[(size_t)r * k + c] = dgo_f32_to_e4m3_fast(dgo_bf16_to_f32(src[(size_t)r * ld + c]) * inv);
        }
}

/* The f32-scale recipe of the CPU-runnable case (parity unpinned): sf =
 * amax/448 (amax == 0 -> 1), q = e4m3(v / sf); blocks of block_rows x 128
 * (1 for activations, 128 for weights), scales laid out
 * sf[(r/block_rows)*ceil(k/128) + kb] as reference.rs:104-105 indexes them. */
DGO_API void dgo_quantize_fp8_f32scale(const float* src, uint32_t rows, uint32_t k, uint32_t block_rows,
                                       uint8_t* dst, float* sf) {
    uint32_t kb_n = (k + 127) / 128, rb_n = (rows + block_rows - 1) / block_rows;
    for (uint32_t rb = 0; rb < rb_n; ++rb)
        for (uint32_t kb = 0; kb < kb_n; ++kb) {
            uint32_t r1 = (rb + 1) * block_rows < rows ? (rb + 1) * block_rows : rows;
            uint32_t k1 = (kb + 1) * 128 < k ? (kb + 1) * 128 : k;
            float amax = 0.0f;
            for (uint32_t r = rb * block_rows; r < r1; ++r)
                for (uint32_t c = kb * 128; c < k1; ++c) { float a = fabsf(src[(size_t)r * k + c]); if (a > amax) amax = a; }
            float s = amax > 0.0f ? amax / 448.0f : 1.0f;
            sf[(size_t)rb * kb_n + kb] = s;
            for (uint32_t r = rb * block_rows; r < r1; ++r)
                for (uint32_t c = kb * 128; c < k1; ++c)
                    dst[(size_t)r * k + c] = dgo_f32_to_e4m3_fast(src[(size_t)r * k + c] / s);
        }
}

/* ------------------------------------------------------------------------ */
/* Scale-factor transforms                                                   */
/* ------------------------------------------------------------------------ */

/* cuda/sm100_cast.rs:198-220 -- f32 (rows, k/gran) -> packed words; takes the
 * exponent byte (mantissa dropped); K-tail bytes read as 127. */
DGO_API void dgo_transform_sf1d_packed(const float* src, uint32_t src_ld, uint32_t rows, uint32_t k,
                                       uint32_t gran, uint32_t groups, uint32_t* dst) {
    if (groups == 0) groups = 1;
    size_t group_rows = rows / groups, stride = align4(group_rows);
    size_t kc_n = (k + gran - 1) / gran, cols = (kc_n + 3) / 4;
    memset(dst, 0, cols * groups * stride * 4);
    for (size_t r = 0; r < rows; ++r) {
        size_t g = r / group_rows, lr = r - g * group_rows;
        for (size_t c = 0; c < cols; ++c) {
            uint32_t w = 0;
            for (size_t j = 0; j < 4; ++j) {
                size_t kc = c * 4 + j;
                uint32_t bits = kc < kc_n ? f2u(src[r * src_ld + kc]) : 0x3F800000u;
                w |= ((bits >> 23) & 0xFF) << (j * 8);
            }
            dst[sf_word_index(g, cols, c, stride, lr)] = w;
        }
    }
}

/* cuda/sm100_cast.rs:230-253 -- f32 (ceil(rows/128), k/128) tile scales ->
 * per-row packed words (row r reads tile r/128). */
DGO_API void dgo_transform_sf2d_packed(const float* src, uint32_t src_ld, uint32_t rows, uint32_t k,
                                       uint32_t groups, uint32_t* dst) {
    if (groups == 0) groups = 1;
    size_t group_rows = rows / groups, stride = align4(group_rows);
    size_t kc_n = (k + 127) / 128, cols = (kc_n + 3) / 4;
    memset(dst, 0, cols * groups * stride * 4);
    for (size_t r = 0; r < rows; ++r) {
        size_t g = r / group_rows, lr = r - g * group_rows, tr = r / 128;
        for (size_t c = 0; c < cols; ++c) {
            uint32_t w = 0;
            for (size_t j = 0; j < 4; ++j) {
                size_t kc = c * 4 + j;
                uint32_t bits = kc < kc_n ? f2u(src[tr * src_ld + kc]) : 0x3F800000u;
                w |= ((bits >> 23) & 0xFF) << (j * 8);
            }
            dst[sf_word_index(g, cols, c, stride, lr)] = w;
        }
    }
}

/* cuda/layout.rs:18-49 (transform_sf): (batches, mn, sf_k) f32 ->
 * (batches*sf_k, align4(mn)) f32, padding columns zero. */
DGO_API void dgo_transform_sf_f32(const float* src, uint32_t mn, uint32_t sf_k, uint32_t batches, float* dst) {
    size_t amn = align4(mn);
    memset(dst, 0, (size_t)batches * sf_k * amn * 4);
    for (size_t b = 0; b < batches; ++b)
        for (size_t r = 0; r < mn; ++r)
            for (size_t c = 0; c < sf_k; ++c)
                dst[(b * sf_k + c) * amn + r] = src[(b * mn + r) * sf_k + c];
}

/* cuda/sm100_cast.rs:265-287 -- the transposed f32 layout above -> packed words. */
DGO_API void dgo_transform_sf_t_packed(const float* src, uint32_t rows, uint32_t k, uint32_t gran,
                                       uint32_t groups, uint32_t* dst) {
    if (groups == 0) groups = 1;
    size_t group_rows = rows / groups, stride = align4(group_rows);
    size_t kc_n = (k + gran - 1) / gran, cols = (kc_n + 3) / 4;
    memset(dst, 0, cols * groups * stride * 4);
    for (size_t r = 0; r < rows; ++r) {
        size_t g = r / group_rows, lr = r - g * group_rows;
        for (size_t c = 0; c < cols; ++c) {
            uint32_t w = 0;
            for (size_t j = 0; j < 4; ++j) {
                size_t kc = c * 4 + j;
                uint32_t bits = kc < kc_n ? f2u(src[(g * kc_n + kc) * stride + lr]) : 0x3F800000u;
                w |= ((bits >> 23) & 0xFF) << (j * 8);
            }
            dst[sf_word_index(g, cols, c, stride, lr)] = w;
        }
    }
}

/* One-past-the-last row of each group.  cuda/sm100_cast.rs:293-301 computes
 * max(i+1 : m_indices[i]==g); an expert with no rows would get 0 there, which
 * the scheduler cannot walk, so empty groups inherit the previous end (a
 * running maximum).  Identical to the reference wherever every group is
 * non-empty. */
DGO_API void dgo_psum_from_m_indices(const int32_t* m_indices, uint32_t m, uint32_t groups, uint32_t* psum) {
    for (uint32_t g = 0; g < groups; ++g) psum[g] = 0;
    for (uint32_t i = 0; i < m; ++i) {
        int32_t g = m_indices[i];
        if (g >= 0 && (uint32_t)g < groups && psum[g] < i + 1) psum[g] = i + 1;
    }
    for (uint32_t g = 1; g < groups; ++g) if (psum[g] < psum[g - 1]) psum[g] = psum[g - 1];
}

/* ------------------------------------------------------------------------ */
/* Reference GEMMs                                                           */
/* ------------------------------------------------------------------------ */

/* reference.rs:85-114 -- f32 block accumulator flushed every 128 k with sa*sb.
 * threads <= 1 runs the loop nest exactly as written (single thread); threads
 * > 1 splits the outer row loop only (each output element is still computed
 * by the identical scalar sequence, so results do not depend on threads). */
DGO_API void dgo_ref_fp8_gemm_nt(const uint8_t* a, const float* sfa, uint32_t m, const uint8_t* b,
                                 const float* sfb, uint32_t n, uint32_t k, float* out, int threads) {
    uint32_t kb_n = (k + 127) / 128;
    #pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
    for (long mi = 0; mi < (long)m; ++mi)
        for (uint32_t ni = 0; ni < n; ++ni) {
            float acc = 0.0f, blk = 0.0f;
            for (uint32_t ki = 0; ki < k; ++ki) {
                blk += dgo_e4m3_to_f32(a[(size_t)mi * k + ki]) * dgo_e4m3_to_f32(b[(size_t)ni * k + ki]);
                if ((ki + 1) % 128 == 0 || ki + 1 == k) {
                    uint32_t kb = ki / 128;
                    acc += blk * sfa[(size_t)mi * kb_n + kb] * sfb[(size_t)(ni / 128) * kb_n + kb];
                    blk = 0.0f;
                }
            }
            out[(size_t)mi * n + ni] = acc;
        }
}

/* reference.rs:133-168 -- rows with m_indices < 0 stay zero; note the weight
 * scale is indexed (ni/128)*k_blocks + kb WITHOUT the group, exactly as the
 * reference does (its tests use one constant scale). sfb_group_stride lets a
 * caller supply per-group scales: 0 reproduces the reference indexing. */
DGO_API void dgo_ref_m_grouped_contiguous(const uint8_t* a, const float* sfa, const int32_t* m_indices, uint32_t m,
                                          const uint8_t* b, const float* sfb, size_t sfb_group_stride,
                                          uint32_t n, uint32_t k, float* out, int threads) {
    uint32_t kb_n = (k + 127) / 128;
    memset(out, 0, (size_t)m * n * 4);
    #pragma omp parallel for schedule(dynamic, 4) num_threads(threads > 1 ? threads : 1)
    for (long mi = 0; mi < (long)m; ++mi) {
        int32_t g = m_indices[mi];
        if (g < 0) continue;
        const float* sfb_g = sfb + (size_t)g * sfb_group_stride;
        for (uint32_t ni = 0; ni < n; ++ni) {
            float acc = 0.0f, blk = 0.0f;
            for (uint32_t ki = 0; ki < k; ++ki) {
                blk += dgo_e4m3_to_f32(a[(size_t)mi * k + ki]) * dgo_e4m3_to_f32(b[((size_t)g * n + ni) * k + ki]);
                if ((ki + 1) % 128 == 0 || ki + 1 == k) {
                    uint32_t kb = ki / 128;
                    acc += blk * sfa[(size_t)mi * kb_n + kb] * sfb_g[(size_t)(ni / 128) * kb_n + kb];
                    blk = 0.0f;
                }
            }
            out[(size_t)mi * n + ni] = acc;
        }
    }
}

/* reference.rs:172-208 -- rows >= masked_m[g] stay zero. */
DGO_API void dgo_ref_m_grouped_masked(const uint8_t* a, const float* sfa, const int32_t* masked_m, uint32_t groups,
                                      uint32_t m_per_group, const uint8_t* b, const float* sfb,
                                      size_t sfb_group_stride, uint32_t n, uint32_t k, float* out, int threads) {
    uint32_t kb_n = (k + 127) / 128;
    memset(out, 0, (size_t)groups * m_per_group * n * 4);
    #pragma omp parallel for schedule(dynamic, 4) num_threads(threads > 1 ? threads : 1)
    for (long row = 0; row < (long)groups * m_per_group; ++row) {
        uint32_t g = (uint32_t)(row / m_per_group), mi = (uint32_t)(row % m_per_group);
        if ((int32_t)mi >= masked_m[g]) continue;
        const float* sfb_g = sfb + (size_t)g * sfb_group_stride;
        for (uint32_t ni = 0; ni < n; ++ni) {
            float acc = 0.0f, blk = 0.0f;
            for (uint32_t ki = 0; ki < k; ++ki) {
                blk += dgo_e4m3_to_f32(a[(size_t)row * k + ki]) * dgo_e4m3_to_f32(b[((size_t)g * n + ni) * k + ki]);
                if ((ki + 1) % 128 == 0 || ki + 1 == k) {
                    uint32_t kb = ki / 128;
                    acc += blk * sfa[(size_t)row * kb_n + kb] * sfb_g[(size_t)(ni / 128) * kb_n + kb];
                    blk = 0.0f;
                }
            }
            out[(size_t)row * n + ni] = acc;
        }
    }
}

/* reference.rs:293-329 -- packed e2m1 operands, packed UE8M0 words (flat
 * layout), f64 accumulation of a*sfa*b*sfb per element. */
DGO_API void dgo_mxfp4_gemm_reference(const uint8_t* a, const uint32_t* a_sf, uint32_t m, const uint8_t* b,
                                      const uint32_t* b_sf, uint32_t n, uint32_t k, float* out, int threads) {
    size_t am = align4(m), an = align4(n);
    #pragma omp parallel for schedule(static) num_threads(threads > 1 ? threads : 1)
    for (long i = 0; i < (long)m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (uint32_t kk = 0; kk < k; ++kk) {
                uint8_t ab = a[(size_t)i * (k / 2) + kk / 2], bb = b[(size_t)j * (k / 2) + kk / 2];
                float av = kE2M1[(kk & 1) ? (ab >> 4) : (ab & 0xF)], bv = kE2M1[(kk & 1) ? (bb >> 4) : (bb & 0xF)];
                uint32_t wa = a_sf[(size_t)(kk / 128) * am + i], wb = b_sf[(size_t)(kk / 128) * an + j];
                float sa = dgo_ue8m0_to_f32((uint8_t)(wa >> (((kk % 128) / 32) * 8)));
                float sb = dgo_ue8m0_to_f32((uint8_t)(wb >> (((kk % 128) / 32) * 8)));
                acc += (double)av * (double)sa * (double)bv * (double)sb;
            }
            out[(size_t)i * n + j] = (float)acc;
        }
}

/* ------------------------------------------------------------------------ */
/* Generic packed-operand checker (what the GPU kernel is compared with)     */
/* ------------------------------------------------------------------------ */

/* Decode one operand row segment to f32 with its packed scales applied.
 * data is (rows_total, k) e4m3 or (rows_total, k/2) packed e2m1; sf is the
 * grouped packed layout with `groups` groups of `group_rows` rows. */
DGO_API void dgo_dequant_rows(const uint8_t* data, const uint32_t* sf, uint32_t bits, uint32_t gran, uint32_t k,
                              uint32_t groups, uint32_t group_rows, const uint32_t* row_ids, uint32_t n_rows,
                              float* out) {
    size_t stride = align4(group_rows), cols = (k + 4 * gran - 1) / (4 * gran);
    #pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)n_rows; ++t) {
        size_t r = row_ids[t], g = r / group_rows, lr = r - g * group_rows;
        (void)groups;
        for (uint32_t kk = 0; kk < k; ++kk) {
            uint32_t blk = kk / gran;
            uint32_t w = sf[sf_word_index(g, cols, blk / 4, stride, lr)];
            float s = dgo_ue8m0_to_f32((uint8_t)(w >> ((blk % 4) * 8)));
            float v;
            if (bits == 8) v = dgo_e4m3_to_f32(data[r * k + kk]);
            else { uint8_t byte = data[r * (k / 2) + kk / 2]; v = kE2M1[(kk & 1) ? (byte >> 4) : (byte & 0xF)]; }
            out[(size_t)t * k + kk] = v * s;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* FP8-requantize epilogue (parity unpinned as arithmetic; layout from       */
/* cuda/sm100_common.rs:873-888, order of operations from :1046-1074)        */
/* ------------------------------------------------------------------------ */

/* d: (rows, n) f32 accumulators of one batch/group `batch`; out: (rows, n)
 * e4m3 written at out + 0 (caller offsets); sfd: whole packed buffer with
 * stride = align4(m_stride_rows). */
DGO_API void dgo_requant_fp8(const float* d, uint32_t rows, uint32_t n, uint32_t batch, uint32_t sfd_stride,
                             uint8_t* out, uint32_t* sfd) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t nb = 0; nb < n; nb += 32) {
            uint32_t n1 = nb + 32 < n ? nb + 32 : n;
            uint16_t amax = 0;
            for (uint32_t c = nb; c < n1; ++c) {
                uint16_t h = dgo_f32_to_bf16(d[(size_t)r * n + c]) & 0x7FFF;
                if (h > amax) amax = h;
            }
            uint32_t e = dgo_sf_exp_e4m3_bf16(amax);
            float inv = sf_inv(e);
            for (uint32_t c = nb; c < n1; ++c)
                out[(size_t)r * n + c] = dgo_f32_to_e4m3_fast(dgo_bf16_to_f32(dgo_f32_to_bf16(d[(size_t)r * n + c])) * inv);
            size_t sf_idx = ((size_t)batch * n + nb) / 32;
            uint8_t* wp = (uint8_t*)(sfd + (sf_idx / 4) * sfd_stride + r);
            wp[sf_idx % 4] = (uint8_t)e;
        }
}

/* MoE combine (gather-reduce form of cuda/layout.rs:192-207 followed by :211 f32->bf16):
 * out[t] = bf16(sum_j w[t,j] * rows[pos[t,j]]), f32 accumulation in order with fmaf; pos < 0 skipped. */
DGO_API void dgo_moe_combine(const uint16_t* rows, size_t pitch, const int32_t* pos, const float* w, uint32_t tokens,
                             uint32_t topk, uint32_t n, uint16_t* out) {
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t c = 0; c < n; ++c) {
            float acc = 0.0f;
            for (uint32_t j = 0; j < topk; ++j) {
                int32_t p = pos[(size_t)t * topk + j];
                if (p < 0) continue;
                acc = fmaf(w[(size_t)t * topk + j], dgo_bf16_to_f32(rows[(size_t)p * pitch + c]), acc);
            }
            out[(size_t)t * n + c] = dgo_f32_to_bf16(acc);
        }
}

/* reference.rs:117-129 (ref_bf16_gemm_nt): out[m,n] = sum_k a[m,k] * b[n,k] over bf16 bit patterns, f64
 * accumulation in k order, rounded to f32 once. */
DGO_API void dgo_ref_bf16_gemm_nt(const uint16_t* a, uint32_t m, const uint16_t* b, uint32_t n, uint32_t k, float* out, int threads) {
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for (int64_t mi = 0; mi < (int64_t)m; ++mi)
        for (uint32_t ni = 0; ni < n; ++ni) {
            double acc = 0.0;
            for (uint32_t ki = 0; ki < k; ++ki)
                acc += (double)dgo_bf16_to_f32(a[(size_t)mi * k + ki]) * (double)dgo_bf16_to_f32(b[(size_t)ni * k + ki]);
            out[(size_t)mi * n + ni] = (float)acc;
        }
}

/* SiLU-and-mul (cuda/layout.rs:218-233 as called from moe.rs:273-296): out[r,c] = bf16(silu(gate) * up) on a
 * (rows, 2n) gate|up matrix of bf16 bits, silu(g) = g / (1 + exp(-g)).  The reference's device code uses the
 * fast-math exponential, which no host function reproduces bit for bit; exp is therefore written out here
 * (and identically in the CUDA kernel) in correctly rounded f32 steps: the gate is clamped to [-87, 30];
 * n = rint(-g log2 e) is read from the low mantissa bits of fma(g, -log2 e, 1.5 * 2^23); r = -g - n ln2 with
 * ln 2 in two parts; exp(r) - 1 is a degree-5 Taylor polynomial on |r| <= ln2/2; 2^n is applied by adding n to
 * the exponent field; 1 / (1 + exp(-g)) by three Newton steps x <- x (2 - d x) from the estimate
 * 0x7EF311C7 - bits(d); silu = g * that; gates below -87 give 0.
 * Parity unpinned: a test bounds the distance to the f64 formula instead. */
static float dgo_silu_mul_one(float g, float u) {
    float gc = fminf(fmaxf(g, -87.0f), 30.0f);
    float t = fmaf(gc, -1.44269504f, 12582912.0f);
    float n = t + -12582912.0f;
    float r = fmaf(n, -0.693145752f, -gc);
    r = fmaf(n, -1.42860677e-6f, r);
    float q = fmaf(1.0f / 120.0f, r, 1.0f / 24.0f);
    q = fmaf(q, r, 1.0f / 6.0f);
    q = fmaf(q, r, 0.5f);
    q = fmaf(q, r * r, r);
    float s = q + 1.0f;
    float e = u2f(f2u(s) + (f2u(t) << 23));
    float d = 1.0f + e;
    float x = u2f(0x7EF311C7u - f2u(d));
    x = x * fmaf(-d, x, 2.0f);
    x = x * fmaf(-d, x, 2.0f);
    x = x * fmaf(-d, x, 2.0f);
    float silu = g < -87.0f ? 0.0f : g * x;   /* |g exp(g)| < 2e-36 below -87 */
    float act = silu * u;
    return dgo_bf16_to_f32(dgo_f32_to_bf16(act));
}
DGO_API void dgo_silu_mul_bf16(const uint16_t* gate_up, uint32_t ld, uint32_t rows, uint32_t n, uint16_t* out) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < n; ++c)
            out[(size_t)r * n + c] = dgo_f32_to_bf16(dgo_silu_mul_one(dgo_bf16_to_f32(gate_up[(size_t)r * ld + c]),
                                                                      dgo_bf16_to_f32(gate_up[(size_t)r * ld + n + c])));
}

/* 1 - 2*sum(xy)/sum(x^2+y^2) in f64 (the tolerance metric; the reference has
 * no such function, the benchmark contract defines it). */
DGO_API double dgo_calc_diff(const float* x, const float* y, size_t n) {
    double xy = 0, xx = 0;
    for (size_t i = 0; i < n; ++i) { xy += (double)x[i] * y[i]; xx += (double)x[i] * x[i] + (double)y[i] * y[i]; }
    return xx == 0.0 ? 0.0 : 1.0 - 2.0 * xy / xx;
}

DGO_API int dgo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
