/*
 * act_oracle.c -- CPU restatement of the activation-compression codec.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against and the timed CPU baseline.  It is never linked into, nor
 * called from, the product library; the product has no CPU path.
 *
 * What it restates (paths are inside the Deep_Optimization project):
 *   - grouping [N,*] -> [N*G, group_size], row-major, one (scale,min) pair per
 *     group: Activation_Compression/modules/tensor_act_reshape_utils.py:17-49
 *   - per-group min/max, scale = range/qmax, scale = 1 when the range is not
 *     positive: Activation_Compression/act_triton_kernel.py:60-65
 *   - codes clamped to [0,qmax], word packing "code j of a 32-bit word sits at
 *     bits [j*b,(j+1)*b)": Activation_Compression/act_triton_kernel.py:110-114,155-171
 *   - dequantise q*scale+min: Activation_Compression/act_triton_kernel.py:206-223
 *   - mask pack / unpack of int8 values: Activation_Compression/act_triton_kernel.py:246-322
 *   - greedy bit allocation: Activation_Compression/cpp_extension/src/calc_precision.cc:10-53
 *   - per-row min/max: Activation_Compression/cpp_extension/src/min_max_kernel.cu:66-141
 *   - tiled GEMM C=A.B with fp32 accumulation:
 *     Activation_Compression/triton_kernel/linear.py:43-95
 *
 * Arithmetic of the default ("baseline") scheme, every operation an IEEE-754
 * binary32 round-to-nearest-even operation, nothing contracted:
 *     mn = min(x), mx = max(x)             (-0 orders below +0, NaN propagates)
 *     r  = mx - mn
 *     s  = r / qmax ; if !(s > 0) s = 1
 *     a  = x - mn ; q = a / s ; t = q + u ; code = clamp(floor(t), 0, qmax)
 * u is the caller's noise tensor.
 *
 * Without one (the "hash" mode, the product's default) the noise is one byte h per
 * element from the counter hash below; with FLAG_ROUND_NEAREST h is the constant 127
 * (the reference's rounding constant 0.5f-1e-6f, act_triton_kernel.py:114, on a grid
 * of 1/256: ties go down).  In both a regular group -- range 0 or in
 * [2^-50, 2^50] -- is quantised in fixed point with 8 fraction bits:
 *     y = 1 / s ; Q = RNE(a * y * 256), rounded once (v = fmaf(a, y, 2^15) and
 *     Q = the low mantissa bits of v) ; code = (Q + h) >> 8        (<= qmax, no clamp)
 * i.e. stochastic rounding of Q/256 with 8 noise bits.  An irregular group
 * (denormal, huge, infinite or NaN range) uses the float formula above with
 * u = h / 256 (hash) or u = 0.5f-1e-6f (round to nearest).
 *
 * The "reference-compatible" scheme (ACT_FLAG_REF_COMPAT) follows the live
 * Triton kernel instead: optional clamp to +-alpha, optional tanh squash,
 * inv = 1/s, t = a*inv + (0.5f-1e-6f) with the multiply and the add rounded
 * separately (what the kernel computes when run by Triton's CPU interpreter),
 * truncation toward zero, bf16-rounded scale and min.
 *
 * PARITY STATUS: the reference holds no golden vectors for this path.  The
 * reference-compatible scheme (word layout, clamp, degenerate-range rule,
 * rounding rule, group minimum, mask pack/unpack) is pinned bit-for-bit by
 * outputs of the reference's own kernels run under Triton's CPU interpreter
 * (tests/golden/reference_triton_codec.npz and the script beside it).  The
 * baseline scheme shares layout and clamp/degenerate rules with it; its true
 * division, fixed-point hash mode and counter hash have no counterpart in any reference test:
 * for those the parity is unpinned by the reference and rests on the two
 * independent restatements (C and numpy) agreeing.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_EXPORT __attribute__((visibility("default")))

enum { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

/* flag bits: keep in sync with include/act_b200.h */
enum {
    FLAG_ROUND_NEAREST = 1,   /* u = 0.5f - 1e-6f, no noise                       */
    FLAG_REF_COMPAT    = 2,   /* live-Triton arithmetic (see header comment)       */
    FLAG_REF_CLAMP     = 4,   /* with REF_COMPAT: clamp x to +-alpha first         */
    FLAG_REF_TANH      = 8,   /* with REF_COMPAT: x = tanh(x/0.5)*0.5 before range */
    FLAG_META_BF16     = 16   /* scale/min rounded to bf16 (stored as fp32 values) */
};

/* ---------------------------------------------------------------- scalars */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* round-to-nearest-even fp32 -> bf16, NaN kept quiet */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t b = f32_bits(f);
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u);
    b += 0x7fffu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}

static inline float f16_to_f32(uint16_t h) {
    _Float16 v; memcpy(&v, &h, 2); return (float)v;
}
static inline uint16_t f32_to_f16(float f) {
    _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h;
}

static inline float load_as_f32(const void *x, int dtype, int64_t i) {
    switch (dtype) {
        case DT_F32:  return ((const float *)x)[i];
        case DT_BF16: return bf16_to_f32(((const uint16_t *)x)[i]);
        default:      return f16_to_f32(((const uint16_t *)x)[i]);
    }
}

/* min/max with the ordering -0 < +0; a NaN operand makes the result NaN, so a
 * group that holds a NaN gets min = NaN, scale = 1 and all codes 0            */
static inline float min_ord(float a, float b) {
    if (a != a || b != b) return NAN;
    if (a == b) return signbit(a) ? a : b;
    return a < b ? a : b;
}
static inline float max_ord(float a, float b) {
    if (a != a || b != b) return NAN;
    if (a == b) return signbit(a) ? b : a;
    return a > b ? a : b;
}

/* ------------------------------------------------------------ noise hash
 * Counter hash used when no noise tensor is given.  Eight consecutive elements
 * (one 16-byte piece of 16-bit inputs) share one 64-bit output; element e takes
 * byte (e & 7) of H(e >> 3), low word first.  H is four rounds of a 2x32
 * multiply-xor network keyed by splitmix64(splitmix64(seed) + offset): seed picks
 * a family of streams, offset one stream of it (callers advance it per call).
 * It has no counterpart in the reference (whose generators are an index hash in
 * cpp_extension/include/quant_common.h:32-43 and Triton's tl.rand).          */
#define HASH_MUL   0xD256D193u
#define HASH_WEYL  0x9E3779B9u
#define HASH_ROUNDS 4

/* splitmix64 finaliser: spreads the caller's seed over the 64-bit key so that
 * neighbouring seeds give unrelated streams                                    */
static inline uint64_t hash_key(uint64_t seed) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline void hash_2x32(uint64_t ctr, uint64_t seed, uint64_t offset, uint32_t *o0, uint32_t *o1) {
    const uint64_t key = hash_key(hash_key(seed) + offset);
    uint32_t L = (uint32_t)ctr;
    uint32_t R = (uint32_t)(ctr >> 32) ^ (uint32_t)(key >> 32);
    uint32_t k = (uint32_t)key;
    for (int r = 0; r < HASH_ROUNDS; ++r) {
        uint64_t p = (uint64_t)HASH_MUL * L;
        uint32_t hi = (uint32_t)(p >> 32), lo = (uint32_t)p;
        L = hi ^ k ^ R;
        R = lo;
        k += HASH_WEYL;
    }
    *o0 = L; *o1 = R;
}

static inline uint32_t hash_byte(uint64_t elem, uint64_t seed, uint64_t offset) {
    uint32_t w0, w1;
    hash_2x32(elem >> 3, seed, offset, &w0, &w1);
    const uint32_t w = (elem & 4) ? w1 : w0;
    return (w >> (8 * (elem & 3))) & 0xffu;
}

/* the noise as a fraction: h / 256 */
ORACLE_EXPORT void oracle_hash_noise(uint64_t seed, uint64_t offset, int64_t first,
                                     int64_t count, float *out) {
    for (int64_t i = 0; i < count; ++i)
        out[i] = (float)hash_byte((uint64_t)(first + i), seed, offset) * (1.0f / 256.0f);
}

/* ------------------------------------------------------------- quant-pack */

static inline int code_from_t(float t, int qmax) {
    if (!(t >= 0.0f)) return 0;                 /* negative or NaN */
    if (t >= (float)(qmax + 1)) return qmax;
    return (int)floorf(t);
}

static int valid_bits(int bits) { return bits == 1 || bits == 2 || bits == 4 || bits == 8; }
static int valid_group(int gs, int bits) {
    return gs >= 32 && gs <= 1024 && (gs & (gs - 1)) == 0 && (gs * bits) % 32 == 0;
}

/* x: [n_groups, group_size] of dtype; packed: n_groups*group_size*bits/32 words;
 * scale,mn: [n_groups].  Returns 0, or 1 on a bad argument.                   */
static int quant_pack_from(const void *x, int dtype, int64_t n_groups, int group_size,
                           int bits, const float *noise, uint64_t seed, uint64_t offset,
                           int flags, float clamp_alpha, uint32_t *packed, float *scale,
                           float *mn_out, int64_t first_group);

ORACLE_EXPORT int oracle_quant_pack(const void *x, int dtype, int64_t n_groups, int group_size,
                                    int bits, const float *noise, uint64_t seed, uint64_t offset,
                                    int flags, float clamp_alpha, uint32_t *packed, float *scale,
                                    float *mn_out) {
    return quant_pack_from(x, dtype, n_groups, group_size, bits, noise, seed, offset, flags, clamp_alpha,
                           packed, scale, mn_out, 0);
}

/* The same for a slice of a larger tensor: x, noise and the outputs start at group
 * `first_group` of that tensor, whose element indices feed the counter hash. */
ORACLE_EXPORT int oracle_quant_pack_slice(const void *x, int dtype, int64_t n_groups, int group_size,
                                          int bits, const float *noise, uint64_t seed, uint64_t offset,
                                          int flags, float clamp_alpha, uint32_t *packed, float *scale,
                                          float *mn_out, int64_t first_group) {
    return quant_pack_from(x, dtype, n_groups, group_size, bits, noise, seed, offset, flags, clamp_alpha,
                           packed, scale, mn_out, first_group);
}

static int quant_pack_from(const void *x, int dtype, int64_t n_groups, int group_size,
                           int bits, const float *noise, uint64_t seed, uint64_t offset,
                           int flags, float clamp_alpha, uint32_t *packed, float *scale,
                           float *mn_out, int64_t first_group) {
    if (!(valid_bits(bits) || bits == 3) || !valid_group(group_size, bits) || dtype < 0 || dtype > 2) return 1;
    if (bits == 3 && (flags & FLAG_REF_COMPAT)) return 1;
    const int qmax = (1 << bits) - 1;
    const int vpw = 32 / bits;                         /* unused for the 3-bit planes */
    const int nwords = group_size * bits / 32;
    const float half_c = 0.5f - 1e-6f;
    const int ref = (flags & FLAG_REF_COMPAT) != 0;

#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        float v[1024];
        const int64_t base = g * group_size;
        for (int i = 0; i < group_size; ++i) {
            float f = load_as_f32(x, dtype, base + i);
            if (ref && (flags & FLAG_REF_CLAMP)) {
                if (f < -clamp_alpha) f = -clamp_alpha;
                if (f > clamp_alpha) f = clamp_alpha;
            }
            if (ref && (flags & FLAG_REF_TANH)) f = tanhf(f / 0.5f) * 0.5f;
            v[i] = f;
        }
        float mn = v[0], mx = v[0];
        for (int i = 1; i < group_size; ++i) { mn = min_ord(mn, v[i]); mx = max_ord(mx, v[i]); }
        const float r = mx - mn;
        float s = r / (float)qmax;
        if (!(s > 0.0f)) s = 1.0f;
        float s_store = s, mn_store = mn;
        if (flags & FLAG_META_BF16) {
            s_store = bf16_to_f32(f32_to_bf16(s));
            mn_store = bf16_to_f32(f32_to_bf16(mn));
        }
        scale[g] = s_store;
        mn_out[g] = mn_store;

        uint32_t *pw = packed + g * (int64_t)nwords;
        const float inv = 1.0f / s;
        const int regular = (r == 0.0f) || (r >= 0x1p-50f && r <= 0x1p50f);
        uint8_t code[1024];
        for (int i = 0; i < group_size; ++i) {
            const float a = v[i] - mn;
            int c;
            if (ref) {
                /* act_triton_kernel.py:71,114,151-153: multiply by the reciprocal,
                 * add the rounding constant, truncate, clamp                       */
                float prod = a * inv;
                float t = prod + half_c;
                if (!(t == t)) c = 0;
                else {
                    if (t > 1.0e9f) t = 1.0e9f;
                    if (t < -1.0e9f) t = -1.0e9f;
                    c = (int)t;                 /* toward zero */
                    if (c < 0) c = 0;
                    if (c > qmax) c = qmax;
                }
            } else if (noise && !(flags & FLAG_ROUND_NEAREST)) {
                const float q = a / s;
                const float t = q + noise[base + i];
                c = code_from_t(t, qmax);
            } else {
                /* the two fixed-point modes: a hash byte, or 127 for round to nearest
                 * (0.5f - 1e-6f on the 1/256 grid: a tie goes down)                   */
                const int nearest = (flags & FLAG_ROUND_NEAREST) != 0;
                const uint32_t h = nearest ? 127u
                    : hash_byte((uint64_t)(first_group * group_size + base + i), seed, offset);
                if (regular) {
                    /* one rounding onto the 2^-8 grid; 2^15 <= v < 2^16 for a regular group */
                    const float vv = fmaf(a, inv, 32768.0f);
                    const uint32_t Q = f32_bits(vv) - f32_bits(32768.0f);
                    c = (int)((Q + h) >> 8);
                } else {
                    const float u = nearest ? half_c : (float)h * (1.0f / 256.0f);
                    const float t = a / s + u;
                    c = code_from_t(t, qmax);
                }
            }
            code[i] = (uint8_t)c;
        }
        if (bits == 3) {
            /* bit planes: 32 elements -> 3 words, bit l of word p = bit p of the code of element l
             * (the cpp_extension kernels store planes too, in their ballot order:
             * cpp_extension/include/quant_pack_1bit_sm90.cuh:140-175)                              */
            for (int ch = 0; ch < group_size / 32; ++ch)
                for (int p = 0; p < 3; ++p) {
                    uint32_t word = 0;
                    for (int l = 0; l < 32; ++l) word |= (uint32_t)((code[ch * 32 + l] >> p) & 1) << l;
                    pw[ch * 3 + p] = word;
                }
        } else {
            for (int w = 0; w < nwords; ++w) {
                uint32_t word = 0;
                for (int j = 0; j < vpw; ++j) word |= (uint32_t)code[w * vpw + j] << (j * bits);
                pw[w] = word;
            }
        }
    }
    return 0;
}

/* ------------------------------------------------- sub-group averaging (AVG_ALAM)
 * act_triton_kernel.py:116-118 (quant_pack_kernel) and :212-215 (dequant_unpack_kernel):
 * the quotients of `avg` consecutive elements are averaged before rounding, so a group
 * stores group_size/avg codes, and decoding repeats each code `avg` times.  Sums run left
 * to right in fp32 (Triton reduces in a tree); the noise of a sub-group is that of its
 * first element; no fixed-point path; the reference's decoder noise is not reproduced.  */
ORACLE_EXPORT int oracle_quant_pack_avg(const void *x, int dtype, int64_t n_groups, int group_size,
                                        int bits, int avg, const float *noise, uint64_t seed,
                                        uint64_t offset, int flags, float clamp_alpha,
                                        uint32_t *packed, float *scale, float *mn_out) {
    if (!valid_bits(bits) || !valid_group(group_size, bits) || dtype < 0 || dtype > 2) return 1;
    if ((avg != 2 && avg != 4 && avg != 8) || (group_size * bits) % (32 * avg)) return 1;
    const int qmax = (1 << bits) - 1;
    const int vpw = 32 / bits;
    const int ncodes = group_size / avg;
    const int nwords = ncodes / vpw;
    const float half_c = 0.5f - 1e-6f;
    const int ref = (flags & FLAG_REF_COMPAT) != 0;
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        float v[1024];
        const int64_t base = g * group_size;
        for (int i = 0; i < group_size; ++i) {
            float f = load_as_f32(x, dtype, base + i);
            if (ref && (flags & FLAG_REF_CLAMP)) {
                if (f < -clamp_alpha) f = -clamp_alpha;
                if (f > clamp_alpha) f = clamp_alpha;
            }
            if (ref && (flags & FLAG_REF_TANH)) f = tanhf(f / 0.5f) * 0.5f;
            v[i] = f;
        }
        float mn = v[0], mx = v[0];
        for (int i = 1; i < group_size; ++i) { mn = min_ord(mn, v[i]); mx = max_ord(mx, v[i]); }
        const float r = mx - mn;
        float s = r / (float)qmax;
        if (!(s > 0.0f)) s = 1.0f;
        scale[g] = (flags & FLAG_META_BF16) ? bf16_to_f32(f32_to_bf16(s)) : s;
        mn_out[g] = (flags & FLAG_META_BF16) ? bf16_to_f32(f32_to_bf16(mn)) : mn;
        const float inv = 1.0f / s;
        uint32_t *pw = packed + g * (int64_t)nwords;
        for (int w = 0; w < nwords; ++w) pw[w] = 0;
        for (int c = 0; c < ncodes; ++c) {
            float sum = 0.0f;
            for (int k = 0; k < avg; ++k) {
                const float a = v[c * avg + k] - mn;
                float q;
                if (ref) { const float prod = a * inv; q = prod + half_c; }
                else q = a / s;
                sum = (k == 0) ? q : sum + q;
            }
            const float m = sum * (1.0f / (float)avg);
            int code;
            if (ref) {
                if (!(m == m)) code = 0;
                else {
                    float t = m;
                    if (t > 1.0e9f) t = 1.0e9f;
                    if (t < -1.0e9f) t = -1.0e9f;
                    code = (int)t;
                    if (code < 0) code = 0;
                    if (code > qmax) code = qmax;
                }
            } else {
                float u;
                if (flags & FLAG_ROUND_NEAREST) u = half_c;
                else if (noise) u = noise[base + c * avg];
                else u = (float)hash_byte((uint64_t)(base + c * avg), seed, offset) * (1.0f / 256.0f);
                const float t = m + u;
                code = code_from_t(t, qmax);
            }
            pw[c / vpw] |= (uint32_t)code << ((c % vpw) * bits);
        }
    }
    return 0;
}

ORACLE_EXPORT int oracle_dequant_unpack_avg(const uint32_t *packed, const float *scale, const float *mn,
                                            int64_t n_groups, int group_size, int bits, int avg,
                                            int out_dtype, void *y) {
    if (!valid_bits(bits) || !valid_group(group_size, bits) || out_dtype < 0 || out_dtype > 2) return 1;
    if ((avg != 2 && avg != 4 && avg != 8) || (group_size * bits) % (32 * avg)) return 1;
    const int vpw = 32 / bits;
    const int nwords = group_size / avg / vpw;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        const float s = scale[g], m = mn[g];
        const uint32_t *pw = packed + g * (int64_t)nwords;
        for (int i = 0; i < group_size; ++i) {
            const int c = i / avg;
            const float code = (float)((pw[c / vpw] >> ((c % vpw) * bits)) & mask);
            const float val = fmaf(code, s, m);
            const int64_t e = g * (int64_t)group_size + i;
            if (out_dtype == DT_F32) ((float *)y)[e] = val;
            else if (out_dtype == DT_BF16) ((uint16_t *)y)[e] = f32_to_bf16(val);
            else ((uint16_t *)y)[e] = f32_to_f16(val);
        }
    }
    return 0;
}

/* ---------------------------------------------------------- dequant-unpack
 * y = fma(code, scale, min) rounded once to fp32, then to the output type
 * (the Triton kernel's q*scale+min is contracted to one FMA when compiled for
 * a GPU: act_triton_kernel.py:221).                                           */
ORACLE_EXPORT int oracle_dequant_unpack(const uint32_t *packed, const float *scale,
                                        const float *mn, int64_t n_groups, int group_size,
                                        int bits, int out_dtype, void *y) {
    if (!(valid_bits(bits) || bits == 3) || !valid_group(group_size, bits) || out_dtype < 0 || out_dtype > 2) return 1;
    const int vpw = (bits == 3) ? 32 : 32 / bits;      /* elements per word, or per 3-word chunk */
    const int nwords = group_size / vpw;               /* words, or chunks */
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        const float s = scale[g], m = mn[g];
        const uint32_t *pw = packed + g * (int64_t)(group_size * bits / 32);
        for (int w = 0; w < nwords; ++w) {
            const uint32_t word = (bits == 3) ? 0u : pw[w];
            for (int j = 0; j < vpw; ++j) {
                uint32_t code;
                if (bits == 3)
                    code = ((pw[w * 3] >> j) & 1u) | (((pw[w * 3 + 1] >> j) & 1u) << 1) | (((pw[w * 3 + 2] >> j) & 1u) << 2);
                else
                    code = (word >> (j * bits)) & mask;
                const float c = (float)code;
                const float val = fmaf(c, s, m);
                const int64_t i = g * (int64_t)group_size + w * vpw + j;
                if (out_dtype == DT_F32) ((float *)y)[i] = val;
                else if (out_dtype == DT_BF16) ((uint16_t *)y)[i] = f32_to_bf16(val);
                else ((uint16_t *)y)[i] = f32_to_f16(val);
            }
        }
    }
    return 0;
}

/* --------------------------------------------------------- mask pack/unpack
 * act_triton_kernel.py:246-281: words = sum(x << j*bits) over int8 inputs.  The
 * inputs are masks or already-quantised codes, so only the low `bits` bits of
 * each value are kept here (the reference does not mask; its callers only pass
 * values that fit).                                                            */
ORACLE_EXPORT int oracle_pack_bits(const int8_t *x, int64_t n_groups, int group_size, int bits,
                                   uint32_t *packed) {
    if (!valid_bits(bits) || !valid_group(group_size, bits)) return 1;
    const int vpw = 32 / bits;
    const int64_t nwords = n_groups * (int64_t)(group_size / vpw);
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < nwords; ++w) {
        uint32_t word = 0;
        for (int j = 0; j < vpw; ++j) word |= ((uint32_t)(uint8_t)x[w * vpw + j] & mask) << (j * bits);
        packed[w] = word;
    }
    return 0;
}

/* act_triton_kernel.py:284-322 */
ORACLE_EXPORT int oracle_unpack_bits(const uint32_t *packed, int64_t n_groups, int group_size,
                                     int bits, int8_t *y) {
    if (!valid_bits(bits) || !valid_group(group_size, bits)) return 1;
    const int vpw = 32 / bits;
    const int64_t nwords = n_groups * (int64_t)(group_size / vpw);
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t w = 0; w < nwords; ++w)
        for (int j = 0; j < vpw; ++j) y[w * vpw + j] = (int8_t)((packed[w] >> (j * bits)) & mask);
    return 0;
}

/* ------------------------------------------------------------------ minmax
 * per-row min and max of a [rows, cols] matrix
 * (cpp_extension/src/min_max_kernel.cu:66-95,114-141)                         */
ORACLE_EXPORT int oracle_minmax(const void *x, int dtype, int64_t rows, int64_t cols, float *mn,
                                float *mx) {
    if (dtype < 0 || dtype > 2 || cols <= 0) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float lo = load_as_f32(x, dtype, r * cols), hi = lo;
        for (int64_t c = 1; c < cols; ++c) {
            const float f = load_as_f32(x, dtype, r * cols + c);
            lo = min_ord(lo, f); hi = max_ord(hi, f);
        }
        mn[r] = lo; mx[r] = hi;
    }
    return 0;
}

/* ---------------------------------------------------------- calc_precision
 * Greedy bit allocation (cpp_extension/src/calc_precision.cc:10-53): start from
 * b[i] bits per layer, repeatedly take one bit from the layer whose quantisation
 * -variance increase is smallest until sum(b[i]*w[i]) <= target.  All three
 * arrays are int32, as the reference reads them.  The queue is a max-heap on
 * (delta, index); ties fall to the larger index (std::pair ordering).          */
typedef struct { float delta; int64_t idx; } heap_item;

static int heap_less(heap_item a, heap_item b) {
    if (a.delta < b.delta) return 1;
    if (a.delta > b.delta) return 0;
    return a.idx < b.idx;
}
static void heap_push(heap_item *h, int64_t *n, heap_item it) {
    int64_t i = (*n)++;
    h[i] = it;
    while (i > 0) {
        int64_t p = (i - 1) / 2;
        if (!heap_less(h[p], h[i])) break;
        heap_item t = h[p]; h[p] = h[i]; h[i] = t; i = p;
    }
}
static heap_item heap_pop(heap_item *h, int64_t *n) {
    heap_item top = h[0];
    h[0] = h[--(*n)];
    int64_t i = 0;
    for (;;) {
        int64_t l = 2 * i + 1, r = l + 1, m = i;
        if (l < *n && heap_less(h[m], h[l])) m = l;
        if (r < *n && heap_less(h[m], h[r])) m = r;
        if (m == i) break;
        heap_item t = h[m]; h[m] = h[i]; h[i] = t; i = m;
    }
    return top;
}
static float prec_delta(float C, int b) {
    /* int arithmetic as in the reference; b == 1 makes the second coefficient 0
     * and the quotient infinite, which the reference also produces             */
    int c1 = ((1 << b) - 1) * ((1 << b) - 1);
    int c2 = ((1 << (b - 1)) - 1) * ((1 << (b - 1)) - 1);
    return (float)(C * (1.0 / c1 - 1.0 / c2));
}

ORACLE_EXPORT int oracle_calc_precision(int32_t *b, const int32_t *C, const int32_t *w, int64_t n,
                                        double target) {
    if (n < 0) return 1;
    heap_item *h = (heap_item *)malloc(sizeof(heap_item) * (size_t)(n > 0 ? n : 1));
    if (!h) return 1;
    int64_t hn = 0;
    double b_sum = 0;
    for (int64_t i = 0; i < n; ++i) {
        if (w[i] == 0) { free(h); return 1; }
        heap_item it = { prec_delta((float)C[i], b[i] / w[i]), i };
        heap_push(h, &hn, it);
        b_sum += (double)b[i] * w[i];
    }
    while (b_sum > target) {
        if (hn == 0) { free(h); return 2; }       /* target unreachable */
        heap_item top = heap_pop(h, &hn);
        int64_t i = top.idx;
        b[i] -= 1;
        b_sum -= w[i];
        if (b[i] > 1) {
            heap_item it = { prec_delta((float)C[i], b[i] / w[i]), i };
            heap_push(h, &hn, it);
        }
    }
    free(h);
    return 0;
}

/* ---------------------------------------------------------------- FP8 GEMM
 * C[m,n] = bf16( (sum_k A8[m,k]*B8[k,n]) * sa[m] * sb[n] ), A8/B8 e4m3 bytes.
 * The accumulation here is done in double so the value is the exactly-rounded
 * reference the tensor-core result is compared against within a tolerance.    */
static inline float e4m3_to_f32(uint8_t v) {
    const int sign = v >> 7, exp = (v >> 3) & 0xf, man = v & 7;
    float f;
    if (exp == 0) f = ldexpf((float)man, -9);                 /* subnormal: man * 2^-9 */
    else if (exp == 15 && man == 7) f = NAN;                  /* e4m3fn has no inf */
    else f = ldexpf(1.0f + (float)man / 8.0f, exp - 7);
    return sign ? -f : f;
}

ORACLE_EXPORT void oracle_e4m3_decode(const uint8_t *in, int64_t n, float *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = e4m3_to_f32(in[i]);
}

/* A: [M,K] row-major with leading dimension lda (bytes = elements);
 * B: [K,N] row-major with leading dimension ldb; C: bf16 [M,N], ldc.          */
ORACLE_EXPORT int oracle_fp8_gemm(const uint8_t *A, const uint8_t *B, const float *sa,
                                  const float *sb, uint16_t *C, float *C_f32, int M, int N, int K,
                                  int lda, int ldb, int ldc) {
    if (M < 0 || N < 0 || K < 0) return 1;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        double *acc = (double *)calloc((size_t)(N > 0 ? N : 1), sizeof(double));
        for (int k = 0; k < K; ++k) {
            const double a = lut[A[(int64_t)m * lda + k]];
            const uint8_t *brow = B + (int64_t)k * ldb;
            for (int n = 0; n < N; ++n) acc[n] += a * (double)lut[brow[n]];
        }
        for (int n = 0; n < N; ++n) {
            /* fp32 accumulator, then the two scales applied in fp32 */
            float v = (float)acc[n];
            v = v * sa[m];
            v = v * sb[n];
            if (C_f32) C_f32[(int64_t)m * ldc + n] = v;
            if (C) C[(int64_t)m * ldc + n] = f32_to_bf16(v);
        }
        free(acc);
    }
    return 0;
}

/* ------------------------------------------------ ballot-plane codec (legacy)
 * The reference's second codec, cpp_extension/src/quantization_cuda_kernels.cu:
 *   scale = (2^b - 1) / (max - min + 2e-6)  in the data's own type (:15-28);
 *   q = rint(max((x - min) * scale + noise - 0.5, 0)) with noise = sgd_noise(key),
 *   key = (linear element index << 32) ^ seed (:76-87);
 *   layout: 32 consecutive elements of a group form one chunk; the chunk's b words
 *   follow one another and bit `lane` of word p is bit p of the code of the
 *   chunk's element `lane` (the __ballot_sync order, :94-104);
 *   decode: code / scale + min (:241-242).
 * sgd_noise is cpp_extension/include/quant_common.h:32-43: one multiply-xorshift
 * step, the top 24 bits as u in [0,1), returned as u - 0.5.  Because the noise is
 * already centred, the reference's extra "- 0.5" biases every code down by half a
 * step; FLAG_BALLOT_REF_BIAS keeps that arithmetic, without it the rounding is
 * the unbiased rint((x-min)*scale + noise) = floor((x-min)*scale + u).
 * Every operation is rounded separately (the reference is built with fast-math,
 * so its own last bits are not reproducible); 16-bit types round the scale
 * arithmetic to their own type after every operation as c10's scalar types do. */
enum { FLAG_BALLOT_REF_BIAS = 32 };

static inline float sgd_noise_ref(uint64_t x) {
    x ^= x >> 32;
    x *= 0xD6E8FEB86659FD93ull;
    x ^= x >> 32;
    const float u = (float)(x >> 40) * (1.0f / 16777216.0f);
    return u - 0.5f;
}

ORACLE_EXPORT void oracle_sgd_noise(const uint64_t *keys, int64_t n, float *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = sgd_noise_ref(keys[i]);
}

static inline float round_to(float v, int dtype) {
    if (dtype == DT_BF16) return bf16_to_f32(f32_to_bf16(v));
    if (dtype == DT_F16) return f16_to_f32(f32_to_f16(v));
    return v;
}
static inline void store_from_f32(void *y, int dtype, int64_t i, float v) {
    if (dtype == DT_F32) ((float *)y)[i] = v;
    else if (dtype == DT_BF16) ((uint16_t *)y)[i] = f32_to_bf16(v);
    else ((uint16_t *)y)[i] = f32_to_f16(v);
}

ORACLE_EXPORT int oracle_pack_ballot(const void *x, int dtype, int64_t n_groups, int group_size, int bits,
                                     const void *mn, const void *mx, uint64_t seed, int flags,
                                     uint32_t *packed, void *scale) {
    if (bits < 1 || bits > 8 || group_size < 32 || (group_size & 31)) return 1;
    const int chunks = group_size / 32;
    const float qmax = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        const float m = load_as_f32(mn, dtype, g);
        volatile float denom = round_to(load_as_f32(mx, dtype, g) - m, dtype);
        denom = round_to(denom + round_to(2e-6f, dtype), dtype);
        const float sc = round_to(qmax / denom, dtype);
        store_from_f32(scale, dtype, g, sc);
        for (int c = 0; c < chunks; ++c) {
            uint32_t words[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int lane = 0; lane < 32; ++lane) {
                const int64_t id = g * group_size + c * 32 + lane;
                const float noise = sgd_noise_ref(((uint64_t)id << 32) ^ seed);
                volatile float t = load_as_f32(x, dtype, id) - m;
                t = t * sc;
                t = t + noise;
                if (flags & FLAG_BALLOT_REF_BIAS) t = t - 0.5f;
                float q = nearbyintf(t > 0.0f ? t : 0.0f);       /* NaN -> 0 like fmaxf */
                if (!(q <= qmax)) q = qmax;
                const uint32_t code = (uint32_t)q;
                for (int p = 0; p < bits; ++p) words[p] |= ((code >> p) & 1u) << lane;
            }
            for (int p = 0; p < bits; ++p) packed[(g * chunks + c) * bits + p] = words[p];
        }
    }
    return 0;
}

ORACLE_EXPORT int oracle_unpack_ballot(const uint32_t *packed, const void *scale, const void *mn, int dtype,
                                       int64_t n_groups, int group_size, int bits, void *y) {
    if (bits < 1 || bits > 8 || group_size < 32 || (group_size & 31)) return 1;
    const int chunks = group_size / 32;
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        const float sc = load_as_f32(scale, dtype, g), m = load_as_f32(mn, dtype, g);
        for (int c = 0; c < chunks; ++c)
            for (int lane = 0; lane < 32; ++lane) {
                uint32_t code = 0;
                for (int p = 0; p < bits; ++p) code |= ((packed[(g * chunks + c) * bits + p] >> lane) & 1u) << p;
                volatile float v = (float)code / sc;
                v = v + m;
                store_from_f32(y, dtype, g * group_size + c * 32 + lane, v);
            }
    }
    return 0;
}

/* ------------------------------------------------- division-sequence check
 * The CUDA kernels divide by a per-group scale with a five-operation FMA
 * sequence around the correctly rounded reciprocal instead of a division
 * instruction.  This routine runs the same sequence with fmaf and counts the
 * inputs for which it differs from a/s, so tests can sweep it.                 */
ORACLE_EXPORT int64_t oracle_check_div_sequence(const float *a, const float *s, int64_t n) {
    int64_t bad = 0;
#pragma omp parallel for reduction(+ : bad) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float y = 1.0f / s[i];
        float q = a[i] * y;
        float r = fmaf(-s[i], q, a[i]);
        q = fmaf(r, y, q);
        r = fmaf(-s[i], q, a[i]);
        q = fmaf(r, y, q);
        const float ref = a[i] / s[i];
        if (f32_bits(q) != f32_bits(ref)) bad++;
    }
    return bad;
}

ORACLE_EXPORT int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_EXPORT void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
