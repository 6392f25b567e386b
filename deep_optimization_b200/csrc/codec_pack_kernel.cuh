// Per-group quantise-and-pack (forward-pass half of the codec), sm_100a: the kernel
// template and its launchers.  codec_pack.cu holds the C entry points; the pack_inst_*.cu
// files instantiate the launchers one element type each, so that they compile in parallel.
//
// Work decomposition.  A warp handles a tile of 1024 consecutive elements per
// iteration.  A group of GS elements (32..1024, power of two) is owned by
// L = GS/32 lanes; a lane holds four "pieces" of 8 consecutive elements of its
// group, pieces k*L + j (k = 0..3, j = lane index inside the group), so that
// every load instruction reads L*16 (16-bit types) or L*32 (fp32) contiguous
// bytes per group and all per-lane state (min, scale, reciprocal) belongs to a
// single group.  Group min/max are reduced with log2(L) xor-shuffles.  The
// packed bytes of a tile are staged through shared memory so that they leave
// as 16-byte coalesced stores.
//
// The kernel is bound by instruction issue before it is bound by HBM (about ten
// instructions per 2-byte element), so the per-element arithmetic runs on f32x2
// pairs, 16-bit inputs are subtracted straight out of their packed registers, the
// default (counter-hash) mode quantises in fixed point, the next tile is loaded while
// the current one is encoded, full tiles run without bounds checks, and a tile takes
// one warp-uniform branch between a branch-free fast path and the general slow path.
//
// HBM traffic per element: s_in bytes read, bits/8 written, 8/GS for scale+min.
//
// Replaces: Activation_Compression/act_triton_kernel.py:23-171 (quant_pack_kernel),
// Activation_Compression/cpp_extension/include/quant_pack_1bit_sm90.cuh:18-250.
#pragma once

#include <type_traits>

#include "act_common.cuh"

namespace act {

enum NoiseMode { kNoiseHash = 0, kNoiseTensor = 1, kNoiseConst = 2, kRefCompat = 3 };

// Launch shape, measured on B200 on the 2-bit workloads: 16-bit inputs run best as two
// blocks of 384 threads per SM at 80 registers (24 warps: 25.1 us on bf16 [256,256,28,28]
// against 27-29 us for 16, 20, 28 or 32 warps); fp32 inputs hold twice the raw registers
// and run best as 256-thread blocks, two per SM.
#ifndef ACT_PACK_THREADS
#define ACT_PACK_THREADS 384
#endif
#ifndef ACT_PACK_MIN_BLOCKS
#define ACT_PACK_MIN_BLOCKS 2
#endif
// The batch-norm producers (PRO 3..8 of enum Producer below) hold more live state than the plain
// codec: at 384 threads x 2 blocks (80 registers) they spill.  256 threads x 2 blocks (128
// registers, 16 warps per SM) runs BN+ReLU on bf16 [256,64,56,56] in 50 us against 57.7; the
// channel-minor producer with the residual add, which has two input streams to keep in flight,
// is fastest at 320 x 2 (68 us against 72 at 256 and 75 at 384).
template <int DT, int PRO = 0> struct PackCfg {
    static constexpr bool bn = (PRO >= 3 && PRO <= 8);
    // GELU, SiLU, exact GELU: the same at 256 threads (bf16 [256,197,3072]: 180 -> 161 us, 170 -> 156 us)
    static constexpr bool act = (PRO == 1 || PRO == 2 || PRO == 9);
    static constexpr int threads = (ElemT<DT>::bytes == 4) ? 256 : (bn ? (PRO == 8 ? 320 : 256) : (act ? 256 : ACT_PACK_THREADS));
    static constexpr int min_blocks = (ElemT<DT>::bytes == 4) ? 2 : ACT_PACK_MIN_BLOCKS;
    static constexpr int warps = threads / 32;
};

template <int BITS> struct PieceStore;   // writes the BITS bytes of one 8-element piece to smem
template <> struct PieceStore<1> { static __device__ __forceinline__ void st(uint8_t* p, uint32_t a, uint32_t) { *p = (uint8_t)a; } };
template <> struct PieceStore<2> { static __device__ __forceinline__ void st(uint8_t* p, uint32_t a, uint32_t) { *reinterpret_cast<uint16_t*>(p) = (uint16_t)a; } };
template <> struct PieceStore<4> { static __device__ __forceinline__ void st(uint8_t* p, uint32_t a, uint32_t) { *reinterpret_cast<uint32_t*>(p) = a; } };
template <> struct PieceStore<8> { static __device__ __forceinline__ void st(uint8_t* p, uint32_t a, uint32_t b) { *reinterpret_cast<uint2*>(p) = make_uint2(a, b); } };

// sum over i<n of (0x4B000000 << (i*BITS)) mod 2^32: what the magic-number
// accumulation adds on top of the packed codes
template <int BITS, int N> __host__ __device__ constexpr uint32_t magic_sum() {
    uint32_t s = 0;
    for (int i = 0; i < N; ++i) s += (uint32_t)(kMagicBits << (i * BITS));
    return s;
}

// acc + (v << sh) written as an integer multiply-add, which the FMA pipe can take
__device__ __forceinline__ uint32_t shl_add(uint32_t v, int sh, uint32_t acc) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(v), "r"(1u << sh), "r"(acc));
    return d;
}

// the raw 16-byte vectors of one lane's four pieces
template <int DT> struct RawTile { uint4 v[ElemT<DT>::bytes == 4 ? 8 : 4]; };

// min and max of the 32 packed 16-bit elements of a lane, NaN-propagating, -0 < +0
template <int DT>
__device__ __forceinline__ void minmax16(const RawTile<DT>& r, float& mn, float& mx) {
    if (DT == ACT_DTYPE_BF16) {
        __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&r.v[0].x), hi = lo;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t w[4] = {r.v[k].x, r.v[k].y, r.v[k].z, r.v[k].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
                lo = __hmin2_nan(lo, t); hi = __hmax2_nan(hi, t);
            }
        }
        mn = fmin_nan(__low2float(lo), __high2float(lo));
        mx = fmax_nan(__low2float(hi), __high2float(hi));
    } else {
        __half2 lo = *reinterpret_cast<const __half2*>(&r.v[0].x), hi = lo;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t w[4] = {r.v[k].x, r.v[k].y, r.v[k].z, r.v[k].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2 t = *reinterpret_cast<const __half2*>(&w[i]);
                lo = __hmin2_nan(lo, t); hi = __hmax2_nan(hi, t);
            }
        }
        mn = fmin_nan(__low2float(lo), __high2float(lo));
        mx = fmax_nan(__low2float(hi), __high2float(hi));
    }
}

template <int DT>
__device__ __forceinline__ void zero_raw(RawTile<DT>& r) {
#pragma unroll
    for (int k = 0; k < (ElemT<DT>::bytes == 4 ? 8 : 4); ++k) r.v[k] = make_uint4(0u, 0u, 0u, 0u);
}

template <int DT>
__device__ __forceinline__ void widen_raw(const RawTile<DT>& r, float (&xf)[32]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (ElemT<DT>::bytes == 4) {
            const uint4 a = r.v[2 * k], b = r.v[2 * k + 1];
            xf[k * 8 + 0] = __uint_as_float(a.x); xf[k * 8 + 1] = __uint_as_float(a.y);
            xf[k * 8 + 2] = __uint_as_float(a.z); xf[k * 8 + 3] = __uint_as_float(a.w);
            xf[k * 8 + 4] = __uint_as_float(b.x); xf[k * 8 + 5] = __uint_as_float(b.y);
            xf[k * 8 + 6] = __uint_as_float(b.z); xf[k * 8 + 7] = __uint_as_float(b.w);
        } else {
            constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
            const uint4 a = r.v[k];
            xf[k * 8 + 0] = widen_lo<D16>(a.x); xf[k * 8 + 1] = widen_hi<D16>(a.x);
            xf[k * 8 + 2] = widen_lo<D16>(a.y); xf[k * 8 + 3] = widen_hi<D16>(a.y);
            xf[k * 8 + 4] = widen_lo<D16>(a.z); xf[k * 8 + 5] = widen_hi<D16>(a.z);
            xf[k * 8 + 6] = widen_lo<D16>(a.w); xf[k * 8 + 7] = widen_hi<D16>(a.w);
        }
    }
}

// eight consecutive fp32 noise values of one piece (zeros for a lane past the end)
__device__ __forceinline__ void load_noise8(float (&u8)[8], const float* noise, int64_t e, bool valid) {
    if (valid) {
        const uint4 a = ldg_nc_v4(noise + e), b = ldg_nc_v4(noise + e + 4);
        u8[0] = __uint_as_float(a.x); u8[1] = __uint_as_float(a.y);
        u8[2] = __uint_as_float(a.z); u8[3] = __uint_as_float(a.w);
        u8[4] = __uint_as_float(b.x); u8[5] = __uint_as_float(b.y);
        u8[6] = __uint_as_float(b.z); u8[7] = __uint_as_float(b.w);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) u8[i] = 0.0f;
    }
}

// ---- fast path of the tensor-noise mode (the float formula): one piece -> BITS bytes
// Preconditions (checked per tile, warp-uniformly): the group's range is 0 or in
// [2^-50, 2^50], so the FMA division is exact.  floor is a round-down add of 2^23; the
// code is then the low mantissa bits and the codes of a piece are summed with shifts,
// the 2^23 patterns being subtracted once at the end.
template <int BITS, int NM>
__device__ __forceinline__ void encode_piece_fast(const float* xf8, const float* u8, f32x2 nmn2, f32x2 ns2,
                                                  f32x2 y2, uint32_t& acc0, uint32_t& acc1)
{
    constexpr int QMAX = (1 << BITS) - 1;
    const f32x2 magic2 = pack2(kMagic, kMagic);
    uint32_t a0 = 0, a1 = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const f32x2 a2 = add2_rn(pack2(xf8[2 * p], xf8[2 * p + 1]), nmn2);
        const f32x2 q2 = div_by_scale2(a2, ns2, y2);
        f32x2 t2;
        {
            // caller-supplied noise may lie outside [0,1) or be NaN: clamp t to [0,QMAX]
            // first (NaN -> 0), after which the round-down add is floor again
            uint32_t l, h; unpack2u(add2_rn(q2, pack2(u8[2 * p], u8[2 * p + 1])), l, h);
            t2 = pack2(fminf(fmaxf(__uint_as_float(l), 0.0f), (float)QMAX),
                       fminf(fmaxf(__uint_as_float(h), 0.0f), (float)QMAX));
        }
        uint32_t tb0, tb1;
        unpack2u(add2_rm(t2, magic2), tb0, tb1);
        if (BITS == 8 && p >= 2) {
            a1 = (p == 2) ? shl_add(tb1, 8, tb0) : shl_add(tb1, 24, shl_add(tb0, 16, a1));
        } else {
            a0 = (p == 0) ? shl_add(tb1, BITS, tb0)
                          : shl_add(tb1, (2 * p + 1) * BITS, shl_add(tb0, 2 * p * BITS, a0));
        }
    }
    if (BITS == 8) { acc0 = a0 - magic_sum<8, 4>(); acc1 = a1 - magic_sum<8, 4>(); }
    else { acc0 = a0 - magic_sum<BITS, 8>(); acc1 = 0; }
}

// ---- fixed-point fast path of the counter-hash mode -----------------------------
// For a regular group (range 0 or in [2^-50, 2^50]) the hash mode (and round-to-nearest,
// whose "noise" is the constant 127) is defined in fixed point: v = fma(a, RN(1/s), 2^15) rounds a/s once onto a grid of 8 fraction bits, so the low
// 16 mantissa bits of v are Q = RNE(a*y*256) <= qmax*256; the element's noise byte h is added
// as an integer and code = (Q + h) >> 8 <= qmax: no clamp, no conversion.  Elements 2p and 2p+1
// of a piece share a register (low and high half) after the FMA; one 64-bit hash output holds
// the eight noise bytes of a piece.
template <int DT> __device__ __forceinline__ float sub_from_half(uint32_t w, int hi, float c);
template <> __device__ __forceinline__ float sub_from_half<ACT_DTYPE_BF16>(uint32_t w, int hi, float c) {
    unsigned short h0, h1; float d;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(h0), "=h"(h1) : "r"(w));
    asm("sub.rn.f32.bf16 %0, %1, %2;" : "=f"(d) : "h"(hi ? h1 : h0), "f"(c));
    return d;
}
template <> __device__ __forceinline__ float sub_from_half<ACT_DTYPE_F16>(uint32_t w, int hi, float c) {
    unsigned short h0, h1; float d;
    asm("mov.b32 {%0, %1}, %2;" : "=h"(h0), "=h"(h1) : "r"(w));
    asm("sub.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(hi ? h1 : h0), "f"(c));
    return d;
}
template <> __device__ __forceinline__ float sub_from_half<ACT_DTYPE_F32>(uint32_t, int, float) { return 0.0f; }

__device__ __forceinline__ uint32_t add3(uint32_t a, uint32_t b, uint32_t c) { return a + b + c; }

// hi 32 bits of a 32x32 product, plus c: moves several masked bit fields at once
__device__ __forceinline__ uint32_t mad_hi(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}

__device__ __forceinline__ uint32_t mul_lo(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.lo.u32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}

template <int DT, int BITS, bool FROM_RAW, int NM>
__device__ __forceinline__ void encode_piece_fx(const uint4 rv, const float* xf8, float mn, f32x2 nmn2,
                                                f32x2 y2, uint32_t ctr_lo, uint32_t ctr_hi, uint32_t key_lo,
                                                uint32_t& acc0, uint32_t& acc1)
{
    constexpr uint32_t MB = (uint32_t)(127 + 23 - 8) << 23;          // bit pattern of 2^15: 8 fraction bits
    const f32x2 magic2 = pack2u(MB, MB);
    uint32_t hw[2] = {0u, 0u};
    if (NM == kNoiseHash) hash_2x32_split(ctr_lo, ctr_hi, key_lo, hw[0], hw[1]);   // eight noise bytes, one per element
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t sum[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        // elements 2p and 2p+1 of the piece share a register from here on
        f32x2 a2;
        if (FROM_RAW) a2 = pack2(sub_from_half<DT>(rw[p], 0, mn), sub_from_half<DT>(rw[p], 1, mn));
        else a2 = add2_rn(pack2(xf8[2 * p], xf8[2 * p + 1]), nmn2);
        uint32_t b0, b1;
        unpack2u(fma2_rn(a2, y2, magic2), b0, b1);
        const uint32_t w = shl_add(b1, 16, b0);                       // (Q1 << 16) + Q0 + MB
        // noise bytes under each half; round-to-nearest adds 127/256 to both (the reference's
        // 0.5 - 1e-6 on this grid: ties go down)
        const uint32_t n = (NM == kNoiseHash) ? __byte_perm(hw[p >> 1], 0u, (p & 1) ? 0x4342 : 0x4140) : 0x007F007Fu;
        sum[p] = add3(w, n, 0u - MB);
    }
    // byte 1 of each half is the code: gather them, elements 0-3 and 4-7
    const uint32_t t0 = __byte_perm(sum[0], sum[1], 0x7531), t1 = __byte_perm(sum[2], sum[3], 0x7531);
    if (BITS == 8) {
        acc0 = t0; acc1 = t1;
    } else if (BITS == 4) {
        // low nibbles of bytes 0,2 go to bits 16,24 and those of bytes 1,3 to bits 20,28 of the product
        constexpr uint32_t KE = (1u << 16) + (1u << 8), KO = (1u << 12) + (1u << 4);
        const uint32_t g0 = mul_lo(t0 & 0x00FF00FFu, KE) + mul_lo(t0 & 0xFF00FF00u, KO);
        const uint32_t g1 = mul_lo(t1 & 0x00FF00FFu, KE) + mul_lo(t1 & 0xFF00FF00u, KO);
        acc0 = __byte_perm(g0, g1, 0x7632); acc1 = 0;
    } else if (BITS == 2) {
        // the 2-bit codes at bits 0,8,16,24 go to bits 24,26,28,30 of the product's low word; the
        // other partial products fall on distinct lower fields or leave the word
        constexpr uint32_t K = (1u << 24) + (1u << 18) + (1u << 12) + (1u << 6);
        acc0 = __byte_perm(mul_lo(t0, K), mul_lo(t1, K), 0x0073); acc1 = 0;
    } else {
        constexpr uint32_t K = (1u << 28) + (1u << 21) + (1u << 14) + (1u << 7);
        acc0 = (mul_lo(t0, K) >> 28) | ((mul_lo(t1, K) >> 24) & 0xF0u); acc1 = 0;
    }
}

// ---- slow path: the contract's arithmetic verbatim, any input ------------------
// Taken by a whole tile when one of its groups is irregular (denormal, huge, infinite or
// NaN range).  In hash mode a regular group keeps its fixed-point definition here, so that a
// group's codes never depend on its neighbours in the tile.
template <int BITS, int NM>
__device__ __forceinline__ void encode_piece_slow(const float* xf8, const float* u8, float mn, float s, float y,
                                                  bool regular, uint32_t ctr_lo, uint32_t ctr_hi, uint32_t key_lo,
                                                  uint32_t& acc0, uint32_t& acc1)
{
    constexpr int QMAX = (1 << BITS) - 1;
    uint32_t hw[2] = {0u, 0u};
    if (NM == kNoiseHash) hash_2x32_split(ctr_lo, ctr_hi, key_lo, hw[0], hw[1]);
    acc0 = 0; acc1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float a = __fsub_rn(xf8[i], mn);
        uint32_t c;
        if (NM == kNoiseHash || NM == kNoiseConst) {
            // byte i of the hash output, or the constant 127 of round-to-nearest
            const uint32_t h = (NM == kNoiseHash) ? ((hw[i >> 2] >> ((i & 3) * 8)) & 0xFFu) : 127u;
            if (regular) {
                const uint32_t q = __float_as_uint(__fmaf_rn(a, y, 32768.0f)) - 0x47000000u;
                c = (q + h) >> 8;
            } else {
                const float uu = (NM == kNoiseHash) ? __fmul_rn((float)h, 0x1p-8f) : 0.5f - 1e-6f;
                c = code_from_t(__fadd_rn(__fdiv_rn(a, s), uu), QMAX);
            }
        } else {
            c = code_from_t(__fadd_rn(__fdiv_rn(a, s), u8[i]), QMAX);
        }
        if (BITS == 8 && i >= 4) acc1 |= c << ((i - 4) * 8);
        else acc0 |= c << (i * BITS);
    }
}

// ---- reference-compatible path (act_triton_kernel.py:71,114,151-153): multiply by
// the reciprocal, add 0.5-1e-6 (rounded separately), truncate, integer clamp ------
template <int BITS>
__device__ __forceinline__ void encode_piece_ref(const float* xf8, float mn, float y,
                                                 uint32_t& acc0, uint32_t& acc1)
{
    constexpr int QMAX = (1 << BITS) - 1;
    acc0 = 0; acc1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float a = __fsub_rn(xf8[i], mn);
        float t = __fadd_rn(__fmul_rn(a, y), 0.5f - 1e-6f);
        int c = 0;
        if (t == t) {
            t = fminf(fmaxf(t, -1.0e9f), 1.0e9f);
            c = min(max((int)t, 0), QMAX);
        }
        if (BITS == 8 && i >= 4) acc1 |= (uint32_t)c << ((i - 4) * 8);
        else acc0 |= (uint32_t)c << (i * BITS);
    }
}

// PRO selects a producer fused in front of the codec: kProNone quantises x itself;
// kProGelu / kProSilu write y = act(x) to y_out and quantise the activation's derivative
// (what backward multiplies dy with), replacing the reference's fused forward kernels
// (Activation_Compression/modules/activations/kernel_implementation.py:184-342, 468-559).
enum Producer { kProNone = 0, kProGelu = 1, kProSilu = 2, kProBN = 3, kProBNRelu = 4, kProBNcl = 5, kProBNReluCl = 6,
                kProBNAddRelu = 7, kProBNAddReluCl = 8, kProGeluErf = 9 };

// Per-channel inputs of the batch-norm producer: x is [N, C, HW] contiguous and
// params[c] = (mean, invstd, weight, bias).  The channel of element e is (e / HW) % C;
// inside a lane's group it is found with two exact multiply-high divisions (magic = 0 stands
// for a divisor of 1: the quotient is the dividend), which the host enables only when
// HW*(HW+1024) < 2^32 and C*(C+260) < 2^32.
// kProBNRelu also applies y = max(y, 0) and writes one mask bit per element (bit i of byte
// e/8 = element e, the layout of relu_fwd_pack) to `mask`.
// kProBNcl / kProBNReluCl are the same producers for the channel-minor layout (HW = 1, x is
// [rows, C] with C a multiple of 8, what a channels-last activation is in memory): the
// channel of element e is e % C, so the eight elements of a piece belong to eight
// consecutive channels and every element reads its own row of the table (the rows of a
// warp's loads are contiguous); the kernel keeps the table in shared memory, so C <= 4096.
// kProBNAddRelu / kProBNAddReluCl: y = max(x_hat * weight + bias + residual, 0) with `residual`
// a tensor of x's type and layout (the skip connection of a residual block: the add and the
// ReLU behind the block's last batch norm cost no pass of their own); the sum is rounded to
// fp32 before the ReLU and the mask is that of the sum.
struct BNArgs {
    const float4* params;
    uint32_t hw, c, magic_hw, magic_c;
    uint8_t* mask;
    const uint8_t* residual;
};

// Tiled source addressing (TILED kernels): x is [planes, H, W] and group g is the T x T tile
// (plane, ty, tx) with g = (plane * tiles_y + ty) * tiles_x + tx, its elements row-major inside
// the tile, T = 8, 16 or 32 -- the grouping the reference makes with a permute and a copy
// (Activation_Compression/modules/tensor_act_reshape_utils.py:82-110).  Codes, scale, min and
// the hash counters are those of the permuted [groups, T*T] tensor.
struct TileArgs {
    uint32_t H, W, tiles_x, tiles_y;
    int log2_t;
};

__device__ __forceinline__ float tanh_fast(float v) {
    float r; asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v)); return r;
}

// y and dy/dx of the activation at x (fp32; the transcendental is the hardware approximation)
template <int PRO>
__device__ __forceinline__ void act_and_derivative(float x, float& y, float& d) {
    if (PRO == kProGelu) {
        // u = k (x + c x^3);  y = x * 0.5 (1 + tanh u);
        // d = 0.5 (1 + tanh u) + x (1 - tanh^2 u) * 0.5 k (1 + 3 c x^2).
        // Written as explicit fused multiply-adds (the file builds without contraction):
        // four multiplies and five fmas per element.
        const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
        const float x2 = x * x;
        const float th = tanh_fast(x * __fmaf_rn(kc, x2, k));
        const float hp = __fmaf_rn(0.5f, th, 0.5f);
        y = x * hp;
        const float sech2 = __fmaf_rn(-th, th, 1.0f);
        d = __fmaf_rn(x * sech2, __fmaf_rn(1.5f * kc, x2, 0.5f * k), hp);
    } else if (PRO == kProGeluErf) {
        // exact GELU: x * Phi(x); derivative Phi(x) + x * phi(x)
        const float cdf = __fmaf_rn(0.5f, erff(x * 0.7071067811865476f), 0.5f);
        y = x * cdf;
        d = __fmaf_rn(x, 0.3989422804014327f * __expf(-0.5f * x * x), cdf);
    } else if (PRO == kProSilu) {
        const float sig = __fdividef(1.0f, 1.0f + __expf(-x));
        y = x * sig;
        d = __fmaf_rn(y, 1.0f - sig, sig);
    } else {
        y = x; d = x;
    }
}

// two elements at once: the tanh GELU's polynomial on packed fp32 pairs (five multiplies and five
// fused multiply-adds per pair instead of per element; the two tanh stay scalar)
template <int PRO>
__device__ __forceinline__ void act_and_derivative_pair(float x0, float x1, float& y0, float& y1, float& d0, float& d1) {
    if (PRO == kProGelu) {
        const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
        const f32x2 x = pack2(x0, x1);
        const f32x2 x2 = mul2_rn(x, x);
        uint32_t u0, u1, a, b;
        unpack2u(mul2_rn(x, fma2_rn(pack2(kc, kc), x2, pack2(k, k))), u0, u1);
        const f32x2 th = pack2(tanh_fast(__uint_as_float(u0)), tanh_fast(__uint_as_float(u1)));
        const f32x2 hp = fma2_rn(pack2(0.5f, 0.5f), th, pack2(0.5f, 0.5f));
        unpack2u(mul2_rn(x, hp), a, b);
        y0 = __uint_as_float(a); y1 = __uint_as_float(b);
        const f32x2 sech2 = fma2_rn(mul2_rn(th, th), pack2(-1.0f, -1.0f), pack2(1.0f, 1.0f));
        unpack2u(fma2_rn(mul2_rn(x, sech2), fma2_rn(pack2(1.5f * kc, 1.5f * kc), x2, pack2(0.5f * k, 0.5f * k)), hp), a, b);
        d0 = __uint_as_float(a); d1 = __uint_as_float(b);
    } else {
        act_and_derivative<PRO>(x0, y0, d0);
        act_and_derivative<PRO>(x1, y1, d1);
    }
}

// L2 >= 0 fixes log2(lanes per group) at compile time (the common group sizes get their own
// instantiation: addresses, strides and the shuffle loop then fold to constants); L2 = -1
// takes it from the argument.
template <int DT, int BITS, int NM, int PRO = kProNone, int L2 = -1, bool TILED = false>
__global__ void __launch_bounds__(PackCfg<DT, PRO>::threads, PackCfg<DT, PRO>::min_blocks)
quant_pack_kernel(const void* __restrict__ x_, const float* __restrict__ noise,
                  uint8_t* __restrict__ packed, float* __restrict__ scale_out,
                  float* __restrict__ min_out, int64_t n_elems, int log2_L_arg,
                  uint32_t key_lo, uint32_t key_hi, int flags, float clamp_alpha,
                  uint8_t* __restrict__ y_out = nullptr, BNArgs bn = BNArgs{nullptr, 1u, 1u, 0u, 0u, nullptr, nullptr},
                  TileArgs ta = TileArgs{0u, 0u, 1u, 1u, 3})
{
    static_assert(!TILED || PRO == kProNone, "tiled addressing is built for the plain codec only");
    constexpr int QMAX = (1 << BITS) - 1;
    constexpr int TILE_OUT = kTileElems * BITS / 8;          // packed bytes per tile
    constexpr int kPackWarps = PackCfg<DT, PRO>::warps;
    __shared__ __align__(16) uint8_t stage[kPackWarps][TILE_OUT];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int log2_L = (L2 >= 0) ? L2 : log2_L_arg;
    const int L = 1 << log2_L;                  // lanes per group
    const int j = lane & (L - 1);               // lane index inside the group
    const int g_local = lane >> log2_L;         // group index inside the tile
    const int lane_e0 = g_local << (log2_L + 5);   // first element of the lane's group inside the tile
    const int64_t warp_stride = (int64_t)gridDim.x * kPackWarps;
    const uint8_t* xb = static_cast<const uint8_t*>(x_);
    uint8_t* my_stage = stage[warp];

    // Full tiles run a check-free body; the one partial tile at the end (if any) runs the
    // same body once more with its bounds checks switched on.
    const int64_t n_full = n_elems / kTileElems;
    const bool has_tail = (n_elems % kTileElems) != 0;
    // per-lane constants of the tile walk
    const int piece_stride = 8 << log2_L;                                    // elements between a lane's pieces
    const uint8_t* xlane = xb + (int64_t)(lane_e0 + j * 8) * ElemT<DT>::bytes;   // piece 0 inside tile 0
    const uint32_t lane_ctr = (uint32_t)(lane_e0 >> 3) + (uint32_t)j;        // its hash counter inside a tile
    uint8_t* sts_lane = my_stage + ((g_local << (log2_L + 2)) + j) * BITS;   // its staging slot

    auto load_tile = [&](RawTile<DT>& r, int64_t t) {
        if (TILED) {
            // the lane's group -> (plane, ty, tx); its piece pg -> row pg / (T/8), eight-element
            // column block pg % (T/8) of the tile
            const uint32_t g = (uint32_t)t * (32u >> log2_L) + (uint32_t)g_local;
            const uint32_t q = g / ta.tiles_x, tx = g - q * ta.tiles_x;
            const uint32_t plane = q / ta.tiles_y, ty = q - plane * ta.tiles_y;
            const int64_t base = ((int64_t)plane * ta.H + ((int64_t)ty << ta.log2_t)) * ta.W + ((int64_t)tx << ta.log2_t);
            const int log2_tp = ta.log2_t - 3;                        // pieces per tile row
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int pg = (k << log2_L) + j;
                const int64_t e = base + (int64_t)(pg >> log2_tp) * ta.W + ((pg & ((1 << log2_tp) - 1)) << 3);
                if (ElemT<DT>::bytes == 4) {
                    r.v[2 * k] = ldg_nc_v4(xb + e * 4);
                    r.v[2 * k + 1] = ldg_nc_v4(xb + e * 4 + 16);
                } else {
                    r.v[k] = ldg_nc_v4(xb + e * 2);
                }
            }
            return;
        }
        const uint8_t* p = xlane + t * (int64_t)(kTileElems * ElemT<DT>::bytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (ElemT<DT>::bytes == 4) {
                r.v[2 * k] = ldg_nc_v4(p + (int64_t)(k * piece_stride) * 4);
                r.v[2 * k + 1] = ldg_nc_v4(p + (int64_t)(k * piece_stride) * 4 + 16);
            } else {
                r.v[k] = ldg_nc_v4(p + (int64_t)(k * piece_stride) * 2);
            }
        }
    };

    int64_t tile = (int64_t)blockIdx.x * kPackWarps + warp;
    RawTile<DT> raw_a, raw_b;
    grid_dependency_wait();
    grid_launch_dependents();
    // Channel-minor batch norm: every element needs its own table row, so the table is copied
    // to shared memory once per block, the eight rows of a channel vector followed by one row
    // of padding (144 bytes per vector): the lanes of a quarter warp read consecutive vectors
    // and then fall on distinct banks.
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    float4* const s_table = reinterpret_cast<float4*>(dyn_smem);
    if (PRO == kProBNcl || PRO == kProBNReluCl || PRO == kProBNAddReluCl) {
        for (uint32_t c = threadIdx.x; c < bn.c; c += PackCfg<DT, PRO>::threads)
            s_table[(c >> 3) * 9u + (c & 7u)] = __ldg(bn.params + c);
        __syncthreads();
    }
    if (tile < n_full) load_tile(raw_a, tile);

    // batch norm: where the lane's group starts, as (offset inside its plane, channel) for the
    // plane layout or as its channel alone for the channel-minor layout.  Found with 64-bit
    // divisions once per thread and then advanced tile by tile with additions: a tile step is
    // the same number of elements every time.
    constexpr bool BN_CL = (PRO == kProBNcl || PRO == kProBNReluCl || PRO == kProBNAddReluCl);
    constexpr bool BN_ADD = (PRO == kProBNAddRelu || PRO == kProBNAddReluCl);
    constexpr bool BN_RELU = (PRO == kProBNRelu || PRO == kProBNReluCl || BN_ADD);
    constexpr bool IS_BN = (PRO == kProBN || PRO == kProBNRelu || BN_CL || BN_ADD);
    uint32_t bn_c0 = 0, bn_r0 = 0, bn_dc = 0, bn_dr = 0;
    if (IS_BN) {
        const uint64_t e0 = (uint64_t)tile * kTileElems + (uint64_t)lane_e0;
        const uint64_t step = (uint64_t)warp_stride * kTileElems;
        if (BN_CL) {
            bn_c0 = (uint32_t)(e0 % bn.c);
            bn_dc = (uint32_t)(step % bn.c);
        } else {
            const uint64_t plane = e0 / bn.hw, step_planes = step / bn.hw;
            bn_r0 = (uint32_t)(e0 - plane * bn.hw);
            bn_c0 = (uint32_t)(plane % bn.c);
            bn_dr = (uint32_t)(step - step_planes * bn.hw);
            bn_dc = (uint32_t)(step_planes % bn.c);
        }
    }
    auto bn_advance = [&]() {
        if (!IS_BN) return;
        bn_c0 += bn_dc;
        if (!BN_CL) {
            bn_r0 += bn_dr;
            if (bn_r0 >= bn.hw) { bn_r0 -= bn.hw; ++bn_c0; }
        }
        if (bn_c0 >= bn.c) bn_c0 -= bn.c;
    };

    // raw_cur holds this tile, raw_next receives the following one while this one is encoded
    auto run_tile = [&](auto tail_tag, const RawTile<DT>& raw_cur, RawTile<DT>& raw_next) {
        constexpr bool TAIL = decltype(tail_tag)::value;
        // element index of the lane's group and validity (groups never straddle n_elems)
        const int64_t group_e0 = tile * kTileElems + lane_e0;
        const bool valid = TAIL ? (group_e0 < n_elems) : true;

        // 16-bit inputs in hash mode are consumed straight from the raw registers by the
        // fixed-point encoder; only the slow path widens them
        constexpr bool FIXED = (NM == kNoiseHash || NM == kNoiseConst);      // the fixed-point modes
        constexpr bool RAW16 = (ElemT<DT>::bytes == 2 && FIXED && PRO == kProNone);
        float xf[32];
        // the batch-norm producers subtract the mean straight from the 16-bit halves (one
        // mixed-precision subtraction, the same single rounding as widening first)
        constexpr bool BN_RAW16 = (ElemT<DT>::bytes == 2) && IS_BN;
        if (!RAW16 && !BN_RAW16) widen_raw<DT>(raw_cur, xf);

        // next tile's loads go out before this tile's arithmetic
        if (!TAIL) {
            const int64_t next_tile = tile + warp_stride;
            if (next_tile < n_full) load_tile(raw_next, next_tile);
        }

        // the residual's pieces, at the addresses of the x pieces they are added to
        RawTile<DT> res;
        if (BN_ADD) {
            if (valid) {
                const uint8_t* p = bn.residual + (group_e0 + j * 8) * ElemT<DT>::bytes;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (ElemT<DT>::bytes == 4) {
                        res.v[2 * k] = ldg_nc_v4(p + (int64_t)(k * piece_stride) * 4);
                        res.v[2 * k + 1] = ldg_nc_v4(p + (int64_t)(k * piece_stride) * 4 + 16);
                    } else {
                        res.v[k] = ldg_nc_v4(p + (int64_t)(k * piece_stride) * 2);
                    }
                }
            } else {
                zero_raw<DT>(res);
            }
        }
        if (PRO != kProNone) {
            // fused producer: emit y, keep what backward needs (derivative or x_hat) for the codec
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float yv[8];
                if (BN_CL) {
                    // channel-minor: element i of the piece is channel cc + i (no wrap inside a piece)
                    uint32_t cc = bn_c0 + (uint32_t)(((k << log2_L) + j) * 8);
                    cc -= (bn.magic_c ? __umulhi(cc, bn.magic_c) : cc) * bn.c;
                    float4 p[8];
                    const float4* row = s_table + (cc >> 3) * 9u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) p[i] = row[i];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const int e = k * 8 + i;
                        const uint32_t rw = BN_RAW16 ? (i < 4 ? (i < 2 ? raw_cur.v[k & 3].x : raw_cur.v[k & 3].y) : (i < 6 ? raw_cur.v[k & 3].z : raw_cur.v[k & 3].w)) : 0u;
                        const f32x2 d2 = BN_RAW16 ? pack2(sub_from_half<DT>(rw, 0, p[i].x), sub_from_half<DT>(rw, 1, p[i + 1].x))
                                                  : add2_rn(pack2(xf[e], xf[e + 1]), pack2(-p[i].x, -p[i + 1].x));
                        const f32x2 xh2 = mul2_rn(d2, pack2(p[i].y, p[i + 1].y));                  // x_hat
                        uint32_t a0, a1, c0, c1;
                        unpack2u(xh2, a0, a1);
                        unpack2u(mul2_rn(xh2, pack2(p[i].z, p[i + 1].z)), c0, c1);
                        xf[e] = __uint_as_float(a0); xf[e + 1] = __uint_as_float(a1);
                        yv[i] = __fadd_rn(__uint_as_float(c0), p[i].w);
                        yv[i + 1] = __fadd_rn(__uint_as_float(c1), p[i + 1].w);
                    }
                } else if (IS_BN) {
                    // four consecutive elements share a channel (HW is a multiple of 4), all eight
                    // when HW is a multiple of 8; the four roundings of x_hat and y run on f32x2 pairs
                    const bool one_channel = (bn.hw & 7u) == 0u;
                    float4 p = make_float4(0.0f, 1.0f, 1.0f, 0.0f);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (h == 0 || !one_channel) {
                            const uint32_t t = bn_r0 + (uint32_t)(((k << log2_L) + j) * 8 + h * 4);
                            const uint32_t q = bn.magic_hw ? __umulhi(t, bn.magic_hw) : t;
                            uint32_t cc = bn_c0 + q;
                            cc -= (bn.magic_c ? __umulhi(cc, bn.magic_c) : cc) * bn.c;
                            p = __ldg(bn.params + cc);
                        }
                        const f32x2 nmean2 = pack2(-p.x, -p.x), inv2 = pack2(p.y, p.y);
                        const f32x2 w2 = pack2(p.z, p.z);
#pragma unroll
                        for (int i = 0; i < 4; i += 2) {
                            const int e = k * 8 + h * 4 + i;
                            const int ii = h * 4 + i;
                            const uint32_t rw = BN_RAW16 ? (ii < 4 ? (ii < 2 ? raw_cur.v[k & 3].x : raw_cur.v[k & 3].y) : (ii < 6 ? raw_cur.v[k & 3].z : raw_cur.v[k & 3].w)) : 0u;
                            const f32x2 d2 = BN_RAW16 ? pack2(sub_from_half<DT>(rw, 0, p.x), sub_from_half<DT>(rw, 1, p.x))
                                                      : add2_rn(pack2(xf[e], xf[e + 1]), nmean2);
                            const f32x2 xh2 = mul2_rn(d2, inv2);   // x_hat
                            // affine: the product on the pair, the add as two scalar adds (a packed
                            // multiply followed by a packed add gets fused into one FMA by ptxas,
                            // which would drop the rounding of the product)
                            uint32_t a0, a1, c0, c1;
                            unpack2u(xh2, a0, a1);
                            unpack2u(mul2_rn(xh2, w2), c0, c1);
                            xf[e] = __uint_as_float(a0); xf[e + 1] = __uint_as_float(a1);
                            yv[h * 4 + i] = __fadd_rn(__uint_as_float(c0), p.w);
                            yv[h * 4 + i + 1] = __fadd_rn(__uint_as_float(c1), p.w);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i += 2)
                        act_and_derivative_pair<PRO>(xf[k * 8 + i], xf[k * 8 + i + 1], yv[i], yv[i + 1],
                                                     xf[k * 8 + i], xf[k * 8 + i + 1]);
                }
                if (BN_ADD) {
                    float rf[8];
                    if (ElemT<DT>::bytes == 4) {
                        const uint4 a = res.v[(2 * k) & 7], b = res.v[(2 * k + 1) & 7];
                        rf[0] = __uint_as_float(a.x); rf[1] = __uint_as_float(a.y); rf[2] = __uint_as_float(a.z); rf[3] = __uint_as_float(a.w);
                        rf[4] = __uint_as_float(b.x); rf[5] = __uint_as_float(b.y); rf[6] = __uint_as_float(b.z); rf[7] = __uint_as_float(b.w);
                    } else {
                        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
                        const uint4 a = res.v[k & 3];
                        rf[0] = widen_lo<D16>(a.x); rf[1] = widen_hi<D16>(a.x); rf[2] = widen_lo<D16>(a.y); rf[3] = widen_hi<D16>(a.y);
                        rf[4] = widen_lo<D16>(a.z); rf[5] = widen_hi<D16>(a.z); rf[6] = widen_lo<D16>(a.w); rf[7] = widen_hi<D16>(a.w);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) yv[i] = __fadd_rn(yv[i], rf[i]);
                }
                if (BN_RELU) {
                    uint32_t bits8 = 0;
#pragma unroll
                    for (int i = 7; i >= 0; --i) {
                        // max(y, +0) is +0 for y <= 0, -0 and NaN; any other result carries into bit 31
                        // of the sum, which the funnel shift moves into the mask (element 0 ends at bit 0)
                        yv[i] = fmaxf(yv[i], 0.0f);
                        bits8 = __funnelshift_l(__float_as_uint(yv[i]) + 0x7FFFFFFFu, bits8, 1);
                    }
                    if (valid) bn.mask[(group_e0 >> 3) + ((k << log2_L) + j)] = (uint8_t)bits8;
                }
                if (valid) {
                    const int64_t e = group_e0 + (int64_t)((k << log2_L) + j) * 8;
                    if (DT == ACT_DTYPE_F32) {
                        stg_stream_v4(y_out + e * 4, make_uint4(__float_as_uint(yv[0]), __float_as_uint(yv[1]), __float_as_uint(yv[2]), __float_as_uint(yv[3])));
                        stg_stream_v4(y_out + e * 4 + 16, make_uint4(__float_as_uint(yv[4]), __float_as_uint(yv[5]), __float_as_uint(yv[6]), __float_as_uint(yv[7])));
                    } else {
                        uint32_t o[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (DT == ACT_DTYPE_BF16) { const __nv_bfloat162 t = __floats2bfloat162_rn(yv[2 * i], yv[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
                            else { const __half2 t = __floats2half2_rn(yv[2 * i], yv[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
                        }
                        stg_stream_v4(y_out + e * 2, make_uint4(o[0], o[1], o[2], o[3]));
                    }
                }
            }
        }

        if (NM == kRefCompat) {
            // pre-transform of the live Triton kernel (act_triton_kernel.py:55-58)
            if (flags & ACT_FLAG_REF_CLAMP) {
#pragma unroll
                for (int i = 0; i < 32; ++i) xf[i] = fminf(fmaxf(xf[i], -clamp_alpha), clamp_alpha);
            }
            if (flags & ACT_FLAG_REF_TANH) {
#pragma unroll
                for (int i = 0; i < 32; ++i) xf[i] = __fmul_rn(tanhf(__fdiv_rn(xf[i], 0.5f)), 0.5f);
            }
        }

        // ---- group min / max (NaN propagates, -0 < +0) -------------------------
        float mn, mx;
        if (ElemT<DT>::bytes == 2 && NM != kRefCompat && PRO == kProNone) {
            // 16-bit inputs: min/max are exact in the input format, two elements per op
            minmax16<DT>(raw_cur, mn, mx);
        } else {
            mn = xf[0]; mx = xf[0];
#pragma unroll
            for (int i = 1; i < 31; i += 2) { mn = fmin3_nan(mn, xf[i], xf[i + 1]); mx = fmax3_nan(mx, xf[i], xf[i + 1]); }
            mn = fmin_nan(mn, xf[31]); mx = fmax_nan(mx, xf[31]);
        }
        for (int off = L >> 1; off > 0; off >>= 1) {
            mn = fmin_nan(mn, __shfl_xor_sync(0xffffffffu, mn, off));
            mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        }

        // ---- scale ----------------------------------------------------------------
        const float range = __fsub_rn(mx, mn);
        // the fast paths need a finite range well inside the normal numbers (then
        // 2^-58 <= s <= 2^50); a denormal, huge, infinite or NaN range sends the whole
        // tile the slow way
        const bool fast = (range == 0.0f) || (range >= 0x1p-50f && range <= 0x1p50f);     // a regular group
        const bool tile_fast = (NM != kRefCompat) && __all_sync(0xffffffffu, fast);
        float s;
        if (BITS == 1) {
            s = range;
        } else if (tile_fast) {
            // range / QMAX by the FMA sequence: equal to the IEEE quotient for every normal
            // range (checked over all 2^23 mantissas for the divisors 3, 15 and 255)
            s = div_by_scale(range, (float)QMAX, 1.0f / (float)QMAX);
        } else {
            s = __fdiv_rn(range, (float)QMAX);
        }
        if (!(s > 0.0f)) s = 1.0f;
        const float y = __frcp_rn(s);

        if (valid && j == 0) {
            const int64_t g = (tile << (5 - log2_L)) + g_local;
            float s_st = s, mn_st = mn;
            if (flags & ACT_FLAG_META_BF16) {
                s_st = __bfloat162float(__float2bfloat16_rn(s));
                mn_st = __bfloat162float(__float2bfloat16_rn(mn));
            }
            scale_out[g] = s_st;
            min_out[g] = mn_st;
        }

        // ---- codes ------------------------------------------------------------------
        // hash counter = piece index: 128 per tile, so the lane and piece offsets (< 128)
        // never carry out of the low seven bits
        const uint32_t ctr_lo0 = ((uint32_t)tile << 7) + lane_ctr;
        const uint32_t ctr_hi = (uint32_t)((uint64_t)tile >> 25) ^ key_hi;

        if (tile_fast) {
            const f32x2 nmn2 = pack2(-mn, -mn), ns2 = pack2(-s, -s), y2 = pack2(y, y);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t acc0, acc1;
                const uint32_t ctr_lo = ctr_lo0 + (uint32_t)(k * (piece_stride >> 3));
                if (FIXED) {
                    encode_piece_fx<DT, BITS, RAW16, NM>(raw_cur.v[RAW16 ? k : 0], xf + k * 8, mn, nmn2, y2,
                                                         ctr_lo, ctr_hi, key_lo, acc0, acc1);
                } else {
                    float u8[8];
                    if (NM == kNoiseTensor)
                        load_noise8(u8, noise, group_e0 + (int64_t)(k * piece_stride + j * 8), valid);
                    encode_piece_fast<BITS, NM>(xf + k * 8, u8, nmn2, ns2, y2, acc0, acc1);
                }
                PieceStore<BITS>::st(sts_lane + k * (piece_stride >> 3) * BITS, acc0, acc1);
            }
        } else {
            if (RAW16) widen_raw<DT>(raw_cur, xf);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t acc0, acc1;
                if (NM == kRefCompat) {
                    encode_piece_ref<BITS>(xf + k * 8, mn, y, acc0, acc1);
                } else {
                    float u8[8];
                    if (NM == kNoiseTensor)
                        load_noise8(u8, noise, group_e0 + (int64_t)(k * piece_stride + j * 8), valid);
                    encode_piece_slow<BITS, NM>(xf + k * 8, u8, mn, s, y, fast,
                                                ctr_lo0 + (uint32_t)(k * (piece_stride >> 3)), ctr_hi, key_lo, acc0, acc1);
                }
                PieceStore<BITS>::st(sts_lane + k * (piece_stride >> 3) * BITS, acc0, acc1);
            }
        }
        __syncwarp();

        // ---- coalesced write-out of the tile's packed bytes ---------------------------
        uint8_t* out = packed + tile * (int64_t)TILE_OUT;
        if (!TAIL) {
            if (TILE_OUT / 16 >= 32) {
#pragma unroll
                for (int v = 0; v < TILE_OUT / 16 / 32; ++v)
                    stg_stream_v4(out + (v * 32 + lane) * 16,
                                  *reinterpret_cast<const uint4*>(my_stage + (v * 32 + lane) * 16));
            } else if (lane < TILE_OUT / 16) {
                stg_stream_v4(out + lane * 16, *reinterpret_cast<const uint4*>(my_stage + lane * 16));
            }
        } else {
            const int words = (int)((n_elems - tile * kTileElems) * BITS / 32);   // group bytes are a multiple of 4
            for (int w = lane; w < words; w += 32)
                reinterpret_cast<uint32_t*>(out)[w] = reinterpret_cast<const uint32_t*>(my_stage)[w];
        }
        __syncwarp();
    };

    // two tiles per trip, the raw buffers swapping roles, so that no register copies are needed
    while (tile < n_full) {
        run_tile(std::false_type{}, raw_a, raw_b);
        tile += warp_stride; bn_advance();
        if (tile >= n_full) break;
        run_tile(std::false_type{}, raw_b, raw_a);
        tile += warp_stride; bn_advance();
    }
    if (has_tail && tile == n_full) {
        if (tile * kTileElems + lane_e0 < n_elems) load_tile(raw_a, tile); else zero_raw<DT>(raw_a);
        run_tile(std::true_type{}, raw_a, raw_b);
    }
}
// ------------------------------------------------------------------ launcher

// blocks of one instantiation that fit on an SM (asked once per instantiation)
template <int DT, int BITS, int NM, int L2>
int pack_blocks_per_sm() {
    static int cached = 0;
    if (cached == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM, kProNone, L2>,
                                                          PackCfg<DT>::threads, 0) != cudaSuccess || n < 1) n = 1;
        cached = n;
    }
    return cached;
}

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves = 1);   // cabi.cu

template <int DT, int BITS, int NM, int L2>
cudaError_t launch_pack_fixed(const void* x, const float* noise, void* packed, float* scale,
                              float* mn, int64_t n_elems, int log2_L, uint64_t seed,
                              uint64_t offset, int flags, float clamp_alpha, cudaStream_t st)
{
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    // persistent grid: exactly the resident blocks of one wave (or fewer for small inputs)
    const int grid = stream_grid_for((n_tiles + PackCfg<DT>::warps - 1) / PackCfg<DT>::warps,
                                     pack_blocks_per_sm<DT, BITS, NM, L2>());
    return launch_overlapped(quant_pack_kernel<DT, BITS, NM, kProNone, L2>, grid, PackCfg<DT>::threads, st,
                             x, noise, static_cast<uint8_t*>(packed), scale, mn, n_elems, log2_L,
                             (uint32_t)key, (uint32_t)(key >> 32), flags, clamp_alpha,
                             static_cast<uint8_t*>(nullptr), BNArgs{nullptr, 1u, 1u, 0u, 0u, nullptr, nullptr}, TileArgs{0u, 0u, 1u, 1u, 3});
}

// tiled source addressing, the two fixed-point modes only
template <int DT, int BITS, int NM>
cudaError_t launch_pack_tiled_one(const void* x, void* packed, float* scale, float* mn, int64_t n_elems,
                                  int log2_L, uint64_t seed, uint64_t offset, TileArgs ta, cudaStream_t st)
{
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM, kProNone, -1, true>,
                                                          PackCfg<DT>::threads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((n_tiles + PackCfg<DT>::warps - 1) / PackCfg<DT>::warps, per_sm);
    return launch_overlapped(quant_pack_kernel<DT, BITS, NM, kProNone, -1, true>, grid, PackCfg<DT>::threads, st,
                             x, static_cast<const float*>(nullptr), static_cast<uint8_t*>(packed), scale, mn,
                             n_elems, log2_L, (uint32_t)key, (uint32_t)(key >> 32), 0, 0.0f,
                             static_cast<uint8_t*>(nullptr), BNArgs{nullptr, 1u, 1u, 0u, 0u, nullptr, nullptr}, ta);
}

template <int DT>
cudaError_t launch_pack_tiled(int bits, bool nearest, const void* x, void* packed, float* scale, float* mn,
                              int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, TileArgs ta,
                              cudaStream_t st)
{
#define ACT_TILED_CASE(B) \
    return nearest ? launch_pack_tiled_one<DT, B, kNoiseConst>(x, packed, scale, mn, n_elems, log2_L, seed, offset, ta, st) \
                   : launch_pack_tiled_one<DT, B, kNoiseHash>(x, packed, scale, mn, n_elems, log2_L, seed, offset, ta, st)
    switch (bits) {
        case 1: ACT_TILED_CASE(1);
        case 2: ACT_TILED_CASE(2);
        case 4: ACT_TILED_CASE(4);
        default: ACT_TILED_CASE(8);
    }
#undef ACT_TILED_CASE
}

template <int DT, int BITS, int NM>
cudaError_t launch_pack_one(const void* x, const float* noise, void* packed, float* scale,
                                   float* mn, int64_t n_elems, int log2_L, uint64_t seed,
                                   uint64_t offset, int flags, float clamp_alpha, cudaStream_t st)
{
    // the two fixed-point modes at group sizes 128 and 256 run kernels with the group size compiled in
    constexpr bool kFixedPoint = (NM == kNoiseHash || NM == kNoiseConst);
    if (kFixedPoint && log2_L == 2)
        return launch_pack_fixed<DT, BITS, NM, (kFixedPoint ? 2 : -1)>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    if (kFixedPoint && log2_L == 3)
        return launch_pack_fixed<DT, BITS, NM, (kFixedPoint ? 3 : -1)>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    return launch_pack_fixed<DT, BITS, NM, -1>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
}

template <int DT, int BITS>
cudaError_t launch_pack_mode(int mode, const void* x, const float* noise, void* packed,
                                    float* scale, float* mn, int64_t n_elems, int log2_L,
                                    uint64_t seed, uint64_t offset, int flags, float clamp_alpha,
                                    cudaStream_t st)
{
    switch (mode) {
        case kNoiseHash:   return launch_pack_one<DT, BITS, kNoiseHash>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
        case kNoiseTensor: return launch_pack_one<DT, BITS, kNoiseTensor>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
        case kNoiseConst:  return launch_pack_one<DT, BITS, kNoiseConst>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
        default:           return launch_pack_one<DT, BITS, kRefCompat>(x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    }
}

template <int DT>
cudaError_t launch_pack_bits(int bits, int mode, const void* x, const float* noise,
                                    void* packed, float* scale, float* mn, int64_t n_elems,
                                    int log2_L, uint64_t seed, uint64_t offset, int flags,
                                    float clamp_alpha, cudaStream_t st)
{
    switch (bits) {
        case 1: return launch_pack_mode<DT, 1>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
        case 2: return launch_pack_mode<DT, 2>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
        case 4: return launch_pack_mode<DT, 4>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
        default: return launch_pack_mode<DT, 8>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    }
}


// ------------------------------------------------ fused activation + derivative codec

template <int DT, int BITS, int NM, int PRO>
cudaError_t launch_fused_one(const void* x, void* y, void* packed, float* scale, float* mn,
                                    int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset,
                                    cudaStream_t st)
{
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM, PRO>,
                                                          PackCfg<DT, PRO>::threads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((n_tiles + PackCfg<DT, PRO>::warps - 1) / PackCfg<DT, PRO>::warps, per_sm);
    return launch_overlapped(quant_pack_kernel<DT, BITS, NM, PRO>, grid, PackCfg<DT, PRO>::threads, st,
                             x, static_cast<const float*>(nullptr), static_cast<uint8_t*>(packed), scale, mn,
                             n_elems, log2_L, (uint32_t)key, (uint32_t)(key >> 32), 0, 0.0f,
                             static_cast<uint8_t*>(y), BNArgs{nullptr, 1u, 1u, 0u, 0u, nullptr, nullptr}, TileArgs{0u, 0u, 1u, 1u, 3});
}

template <int DT, int BITS>
cudaError_t launch_fused_bits(int kind, bool nearest, const void* x, void* y, void* packed,
                                     float* scale, float* mn, int64_t n, int l2, uint64_t seed,
                                     uint64_t offset, cudaStream_t st)
{
    if (kind == ACT_KIND_GELU)
        return nearest ? launch_fused_one<DT, BITS, kNoiseConst, kProGelu>(x, y, packed, scale, mn, n, l2, seed, offset, st)
                       : launch_fused_one<DT, BITS, kNoiseHash, kProGelu>(x, y, packed, scale, mn, n, l2, seed, offset, st);
    if (kind == ACT_KIND_GELU_ERF)
        return nearest ? launch_fused_one<DT, BITS, kNoiseConst, kProGeluErf>(x, y, packed, scale, mn, n, l2, seed, offset, st)
                       : launch_fused_one<DT, BITS, kNoiseHash, kProGeluErf>(x, y, packed, scale, mn, n, l2, seed, offset, st);
    return nearest ? launch_fused_one<DT, BITS, kNoiseConst, kProSilu>(x, y, packed, scale, mn, n, l2, seed, offset, st)
                   : launch_fused_one<DT, BITS, kNoiseHash, kProSilu>(x, y, packed, scale, mn, n, l2, seed, offset, st);
}

template <int DT>
cudaError_t launch_fused(int bits, int kind, bool nearest, const void* x, void* y, void* packed,
                                float* scale, float* mn, int64_t n, int l2, uint64_t seed,
                                uint64_t offset, cudaStream_t st)
{
    switch (bits) {
        case 1: return launch_fused_bits<DT, 1>(kind, nearest, x, y, packed, scale, mn, n, l2, seed, offset, st);
        case 2: return launch_fused_bits<DT, 2>(kind, nearest, x, y, packed, scale, mn, n, l2, seed, offset, st);
        case 4: return launch_fused_bits<DT, 4>(kind, nearest, x, y, packed, scale, mn, n, l2, seed, offset, st);
        default: return launch_fused_bits<DT, 8>(kind, nearest, x, y, packed, scale, mn, n, l2, seed, offset, st);
    }
}


// ------------------------------------------------ fused batch-norm normalise + x_hat codec

// ceil(2^32 / d) for the multiply-high division, 0 when d is 1 (then a plain division is used)
inline uint32_t magic_for(uint32_t d) {
    if (d <= 1) return 0;
    return (uint32_t)(((1ull << 32) + d - 1) / d);
}

template <int DT, int BITS, int NM, int PRO>
cudaError_t launch_bn_one(const void* x, void* y, void* packed, float* scale, float* mn,
                                 int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset,
                                 BNArgs bn, cudaStream_t st)
{
    constexpr bool CL = (PRO == kProBNcl || PRO == kProBNReluCl || PRO == kProBNAddReluCl);
    constexpr size_t kMaxTable = (size_t)(4096 / 8) * 144;          // channel-minor table, C <= 4096
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (CL) cudaFuncSetAttribute(quant_pack_kernel<DT, BITS, NM, PRO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxTable);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM, PRO>,
                                                          PackCfg<DT, PRO>::threads, CL ? kMaxTable : 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((n_tiles + PackCfg<DT, PRO>::warps - 1) / PackCfg<DT, PRO>::warps, per_sm);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)PackCfg<DT, PRO>::threads, 1, 1);
    cfg.dynamicSmemBytes = CL ? (size_t)(bn.c / 8u) * 144 : 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ACT_NO_PDL ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, quant_pack_kernel<DT, BITS, NM, PRO>,
                              x, static_cast<const float*>(nullptr), static_cast<uint8_t*>(packed), scale, mn,
                              n_elems, log2_L, (uint32_t)key, (uint32_t)(key >> 32), 0, 0.0f,
                              static_cast<uint8_t*>(y), bn, TileArgs{0u, 0u, 1u, 1u, 3});
}

template <int DT>
cudaError_t launch_bn(int bits, bool nearest, const void* x, void* y, void* packed, float* scale,
                             float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn,
                             cudaStream_t st)
{
#define ACT_BN_CASE(B) \
    if (bn.mask) \
        return nearest ? launch_bn_one<DT, B, kNoiseConst, kProBNRelu>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                       : launch_bn_one<DT, B, kNoiseHash, kProBNRelu>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st); \
    return nearest ? launch_bn_one<DT, B, kNoiseConst, kProBN>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                   : launch_bn_one<DT, B, kNoiseHash, kProBN>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st)
    switch (bits) {
        case 1: ACT_BN_CASE(1);
        case 2: ACT_BN_CASE(2);
        case 4: ACT_BN_CASE(4);
        default: ACT_BN_CASE(8);
    }
#undef ACT_BN_CASE
}

// the same for the channel-minor layout (HW = 1)
template <int DT>
cudaError_t launch_bn_cl(int bits, bool nearest, const void* x, void* y, void* packed, float* scale,
                         float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn,
                         cudaStream_t st)
{
#define ACT_BN_CASE(B) \
    if (bn.mask) \
        return nearest ? launch_bn_one<DT, B, kNoiseConst, kProBNReluCl>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                       : launch_bn_one<DT, B, kNoiseHash, kProBNReluCl>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st); \
    return nearest ? launch_bn_one<DT, B, kNoiseConst, kProBNcl>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                   : launch_bn_one<DT, B, kNoiseHash, kProBNcl>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st)
    switch (bits) {
        case 1: ACT_BN_CASE(1);
        case 2: ACT_BN_CASE(2);
        case 4: ACT_BN_CASE(4);
        default: ACT_BN_CASE(8);
    }
#undef ACT_BN_CASE
}

// batch norm + residual add + ReLU, both layouts (bn.residual and bn.mask set)
template <int DT>
cudaError_t launch_bn_add(int bits, bool nearest, bool channel_minor, const void* x, void* y, void* packed,
                          float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn,
                          cudaStream_t st)
{
#define ACT_BN_CASE(B) \
    if (channel_minor) \
        return nearest ? launch_bn_one<DT, B, kNoiseConst, kProBNAddReluCl>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                       : launch_bn_one<DT, B, kNoiseHash, kProBNAddReluCl>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st); \
    return nearest ? launch_bn_one<DT, B, kNoiseConst, kProBNAddRelu>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                   : launch_bn_one<DT, B, kNoiseHash, kProBNAddRelu>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st)
    switch (bits) {
        case 1: ACT_BN_CASE(1);
        case 2: ACT_BN_CASE(2);
        case 4: ACT_BN_CASE(4);
        default: ACT_BN_CASE(8);
    }
#undef ACT_BN_CASE
}

}  // namespace act
