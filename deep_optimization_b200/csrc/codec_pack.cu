// Per-group quantise-and-pack (forward-pass half of the codec), sm_100a.
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
// The kernel is bound by instruction issue before it is bound by HBM (about a
// dozen instructions per 2-byte element), so the per-element arithmetic runs on
// f32x2 pairs, the next tile is loaded while the current one is encoded, and a
// tile takes one warp-uniform branch between a branch-free fast path and the
// verbatim IEEE slow path.
//
// HBM traffic per element: s_in bytes read, bits/8 written, 8/GS for scale+min.
//
// Replaces: Activation_Compression/act_triton_kernel.py:23-171 (quant_pack_kernel),
// Activation_Compression/cpp_extension/include/quant_pack_1bit_sm90.cuh:18-250.
#include "act_common.cuh"

namespace act {

enum NoiseMode { kNoiseHash = 0, kNoiseTensor = 1, kNoiseConst = 2, kRefCompat = 3 };

// Launch shape: measured on B200, one block of 512 threads per SM with up to 128 registers
// per thread beats more, smaller blocks (39.9 us against 41.3-44.8 us on the 2-bit bf16
// workload): the kernel is bound by instruction issue, not by latency, so registers for
// instruction-level parallelism matter more than resident warps.
#ifndef ACT_PACK_THREADS
#define ACT_PACK_THREADS 512
#endif
#ifndef ACT_PACK_MIN_BLOCKS
#define ACT_PACK_MIN_BLOCKS 1
#endif
// 16-bit inputs: 512 threads, one block per SM; fp32 inputs hold twice the raw registers
// (32 more for the prefetched tile) and run best as 256-thread blocks, two per SM
// (25.0 us on the fp32 configuration against 27.1 us without prefetch, 28.9 us at 512 threads)
template <int DT> struct PackCfg {
    static constexpr int threads = (ElemT<DT>::bytes == 4) ? 256 : ACT_PACK_THREADS;
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

template <int DT>
__device__ __forceinline__ void load_raw(RawTile<DT>& r, const uint8_t* xb, int64_t group_e0,
                                         int log2_L, int j) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t e = group_e0 + (int64_t)((k << log2_L) + j) * 8;
        if (ElemT<DT>::bytes == 4) {
            r.v[2 * k] = ldg_nc_v4(xb + e * 4);
            r.v[2 * k + 1] = ldg_nc_v4(xb + e * 4 + 16);
        } else {
            r.v[k] = ldg_nc_v4(xb + e * 2);
        }
    }
}

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

// ---- fast path: one piece (8 elements) -> BITS bytes -------------------------
// Preconditions (checked per tile, warp-uniformly): the group's range is 0 or in
// [2^-50, 2^50], so the FMA division is exact, t >= 0 and floor(t) <= QMAX
// (8-bit hash noise needs one fminf for the upper bound).  floor is a round-down
// add of 2^23; the code is then the low mantissa bits and the codes of a piece
// are summed with shifts, the 2^23 patterns being subtracted once at the end.
template <int BITS, int NM>
__device__ __forceinline__ void encode_piece_fast(const float* xf8, const float* u8, f32x2 nmn2, f32x2 ns2,
                                                  f32x2 y2, uint32_t ctr_lo, uint32_t ctr_hi, uint32_t key_lo,
                                                  uint32_t& acc0, uint32_t& acc1)
{
    constexpr int QMAX = (1 << BITS) - 1;
    const f32x2 magic2 = pack2(kMagic, kMagic);
    uint32_t hw[4];
    if (NM == kNoiseHash) {
        // two 64-bit hash outputs = eight 16-bit noise fields; the counter's low
        // bits are free of carries because a group starts on a multiple of 8 counters
        hash_2x32_split(ctr_lo, ctr_hi, key_lo, hw[0], hw[1]);
        hash_2x32_split(ctr_lo + 1u, ctr_hi, key_lo, hw[2], hw[3]);
    }
    uint32_t a0 = 0, a1 = 0;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const f32x2 a2 = add2_rn(pack2(xf8[2 * p], xf8[2 * p + 1]), nmn2);
        const f32x2 q2 = div_by_scale2(a2, ns2, y2);
        f32x2 t2;
        if (NM == kNoiseHash) {
            // 16-bit fields -> floats on the conversion unit (keeps the ALU and FMA pipes free)
            unsigned short h0, h1;
            asm("mov.b32 {%0, %1}, %2;" : "=h"(h0), "=h"(h1) : "r"(hw[p]));
            float u0, u1;
            asm("cvt.rn.f32.u16 %0, %1;" : "=f"(u0) : "h"(h0));
            asm("cvt.rn.f32.u16 %0, %1;" : "=f"(u1) : "h"(h1));
            const f32x2 uf2 = pack2(u0, u1);
            t2 = fma2_rn(uf2, pack2(0x1p-16f, 0x1p-16f), q2);        // exact u, one rounding
        } else if (NM == kNoiseTensor) {
            // caller-supplied noise may lie outside [0,1) or be NaN: clamp t to [0,QMAX]
            // first (NaN -> 0), after which the round-down add is floor again
            uint32_t l, h; unpack2u(add2_rn(q2, pack2(u8[2 * p], u8[2 * p + 1])), l, h);
            t2 = pack2(fminf(fmaxf(__uint_as_float(l), 0.0f), (float)QMAX),
                       fminf(fmaxf(__uint_as_float(h), 0.0f), (float)QMAX));
        } else {
            t2 = add2_rn(q2, pack2(0.5f - 1e-6f, 0.5f - 1e-6f));
        }
        if (NM == kNoiseHash && BITS == 8) {
            uint32_t l, h; unpack2u(t2, l, h);
            t2 = pack2(fminf(__uint_as_float(l), (float)QMAX), fminf(__uint_as_float(h), (float)QMAX));
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

// ---- slow path: the contract's arithmetic verbatim, any input ------------------
template <int BITS, int NM>
__device__ __forceinline__ void encode_piece_slow(const float* xf8, const float* u8, float mn, float s,
                                                  uint32_t ctr_lo, uint32_t ctr_hi, uint32_t key_lo,
                                                  uint32_t& acc0, uint32_t& acc1)
{
    constexpr int QMAX = (1 << BITS) - 1;
    uint32_t hw[4] = {0u, 0u, 0u, 0u};
    if (NM == kNoiseHash) {
        hash_2x32_split(ctr_lo, ctr_hi, key_lo, hw[0], hw[1]);
        hash_2x32_split(ctr_lo + 1u, ctr_hi, key_lo, hw[2], hw[3]);
    }
    acc0 = 0; acc1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float a = __fsub_rn(xf8[i], mn);
        const float q = __fdiv_rn(a, s);
        float uu;
        if (NM == kNoiseHash)
            uu = __fmul_rn((i & 1) ? u16_hi_as_float(hw[i >> 1]) : u16_lo_as_float(hw[i >> 1]), 0x1p-16f);
        else if (NM == kNoiseTensor) uu = u8[i];
        else uu = 0.5f - 1e-6f;
        const uint32_t c = code_from_t(__fadd_rn(q, uu), QMAX);
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
enum Producer { kProNone = 0, kProGelu = 1, kProSilu = 2, kProBN = 3 };

// Per-channel inputs of the batch-norm producer: x is [N, C, HW] contiguous and
// params[c] = (mean, invstd, weight, bias).  The channel of element e is (e / HW) % C;
// inside a lane's group it is found with two exact multiply-high divisions, which the
// host enables only when HW*(HW+1024) < 2^32 and C*(C+260) < 2^32.
struct BNArgs {
    const float4* params;
    uint32_t hw, c, magic_hw, magic_c;
};

__device__ __forceinline__ float tanh_fast(float v) {
    float r; asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v)); return r;
}

// y and dy/dx of the activation at x (fp32; the transcendental is the hardware approximation)
template <int PRO>
__device__ __forceinline__ void act_and_derivative(float x, float& y, float& d) {
    if (PRO == kProGelu) {
        const float k = 0.7978845608028654f, c = 0.044715f;
        const float x2 = x * x;
        const float th = tanh_fast(k * (x + c * x2 * x));
        y = 0.5f * x * (1.0f + th);
        d = 0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * k * (1.0f + 3.0f * c * x2);
    } else if (PRO == kProSilu) {
        const float sig = __fdividef(1.0f, 1.0f + __expf(-x));
        y = x * sig;
        d = sig * (1.0f + x * (1.0f - sig));
    } else {
        y = x; d = x;
    }
}

template <int DT, int BITS, int NM, int PRO = kProNone>
__global__ void __launch_bounds__(PackCfg<DT>::threads, PackCfg<DT>::min_blocks)
quant_pack_kernel(const void* __restrict__ x_, const float* __restrict__ noise,
                  uint8_t* __restrict__ packed, float* __restrict__ scale_out,
                  float* __restrict__ min_out, int64_t n_elems, int log2_L,
                  uint32_t key_lo, uint32_t key_hi, int flags, float clamp_alpha,
                  uint8_t* __restrict__ y_out = nullptr, BNArgs bn = BNArgs{nullptr, 1u, 1u, 0u, 0u})
{
    constexpr int QMAX = (1 << BITS) - 1;
    constexpr int TILE_OUT = kTileElems * BITS / 8;          // packed bytes per tile
    constexpr bool PREFETCH = true;                           // next tile's raw registers: 16 (16-bit) or 32 (fp32)
    constexpr int kPackWarps = PackCfg<DT>::warps;
    __shared__ __align__(16) uint8_t stage[kPackWarps][TILE_OUT];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int L = 1 << log2_L;                  // lanes per group
    const int j = lane & (L - 1);               // lane index inside the group
    const int g_local = lane >> log2_L;         // group index inside the tile
    const int lane_e0 = g_local << (log2_L + 5);   // first element of the lane's group inside the tile
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int64_t warp_stride = (int64_t)gridDim.x * kPackWarps;
    const uint8_t* xb = static_cast<const uint8_t*>(x_);
    uint8_t* my_stage = stage[warp];

    int64_t tile = (int64_t)blockIdx.x * kPackWarps + warp;
    RawTile<DT> raw;
    if (tile < n_tiles) {
        const int64_t e0 = tile * kTileElems + lane_e0;
        if (e0 < n_elems) load_raw<DT>(raw, xb, e0, log2_L, j); else zero_raw<DT>(raw);
    }

    for (; tile < n_tiles; tile += warp_stride) {
        // element index of the lane's group and validity (groups never straddle n_elems)
        const int64_t group_e0 = tile * kTileElems + lane_e0;
        const bool valid = group_e0 < n_elems;

        float xf[32];
        widen_raw<DT>(raw, xf);
        const RawTile<DT> raw_cur = raw;

        // next tile's loads go out before this tile's arithmetic
        const int64_t next_tile = tile + warp_stride;
        if (PREFETCH) {
            if (next_tile < n_tiles) {
                const int64_t e0 = next_tile * kTileElems + lane_e0;
                if (e0 < n_elems) load_raw<DT>(raw, xb, e0, log2_L, j); else zero_raw<DT>(raw);
            }
        }

        // batch norm: plane index and offset inside the plane of the lane's group
        uint32_t bn_c0 = 0, bn_r0 = 0;
        if (PRO == kProBN) {
            const uint64_t plane = (uint64_t)group_e0 / bn.hw;
            bn_r0 = (uint32_t)((uint64_t)group_e0 - plane * bn.hw);
            bn_c0 = (uint32_t)(plane % bn.c);
        }
        if (PRO != kProNone) {
            // fused producer: emit y, keep what backward needs (derivative or x_hat) for the codec
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float yv[8];
                if (PRO == kProBN) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // four consecutive elements share a channel (HW is a multiple of 4)
                        const uint32_t t = bn_r0 + (uint32_t)(((k << log2_L) + j) * 8 + h * 4);
                        const uint32_t q = bn.magic_hw ? __umulhi(t, bn.magic_hw) : t / bn.hw;
                        uint32_t cc = bn_c0 + q;
                        cc -= (bn.magic_c ? __umulhi(cc, bn.magic_c) : cc / bn.c) * bn.c;
                        const float4 p = __ldg(bn.params + cc);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float xh = __fmul_rn(__fsub_rn(xf[k * 8 + h * 4 + i], p.x), p.y);   // x_hat
                            yv[h * 4 + i] = __fadd_rn(__fmul_rn(xh, p.z), p.w);                       // affine
                            xf[k * 8 + h * 4 + i] = xh;
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) act_and_derivative<PRO>(xf[k * 8 + i], yv[i], xf[k * 8 + i]);
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
            for (int i = 1; i < 32; ++i) { mn = fmin_nan(mn, xf[i]); mx = fmax_nan(mx, xf[i]); }
        }
        for (int off = L >> 1; off > 0; off >>= 1) {
            mn = fmin_nan(mn, __shfl_xor_sync(0xffffffffu, mn, off));
            mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        }

        // ---- scale ----------------------------------------------------------------
        const float range = __fsub_rn(mx, mn);
        float s = (BITS == 1) ? range : __fdiv_rn(range, (float)QMAX);
        if (!(s > 0.0f)) s = 1.0f;
        const float y = __frcp_rn(s);
        // the FMA division and the clamp-free packing need a finite range well inside
        // the normal numbers (then 2^-58 <= s <= 2^50); a denormal, huge, infinite or
        // NaN range sends the whole tile the slow way
        const bool fast = (range == 0.0f) || (range >= 0x1p-50f && range <= 0x1p50f);
        const bool tile_fast = (NM != kRefCompat) && __all_sync(0xffffffffu, fast);

        if (valid && j == 0) {
            const int64_t g = group_e0 >> (log2_L + 5);
            float s_st = s, mn_st = mn;
            if (flags & ACT_FLAG_META_BF16) {
                s_st = __bfloat162float(__float2bfloat16_rn(s));
                mn_st = __bfloat162float(__float2bfloat16_rn(mn));
            }
            scale_out[g] = s_st;
            min_out[g] = mn_st;
        }

        // ---- codes ------------------------------------------------------------------
        // hash counter of the group's first element; the pieces add less than 8*L to
        // its low word, which has log2(8*L) zero low bits, so no carry reaches ctr_hi
        const uint64_t ctr0 = (uint64_t)group_e0 >> 2;
        const uint32_t ctr_lo0 = (uint32_t)ctr0, ctr_hi = (uint32_t)(ctr0 >> 32) ^ key_hi;
        const int stage_base = (g_local << (log2_L + 2));

        if (tile_fast) {
            const f32x2 nmn2 = pack2(-mn, -mn), ns2 = pack2(-s, -s), y2 = pack2(y, y);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int piece = (k << log2_L) + j;
                uint32_t acc0, acc1;
                float u8[8];
                if (NM == kNoiseTensor) load_noise8(u8, noise, group_e0 + (int64_t)piece * 8, valid);
                encode_piece_fast<BITS, NM>(xf + k * 8, u8, nmn2, ns2, y2, ctr_lo0 + (uint32_t)(piece * 2),
                                            ctr_hi, key_lo, acc0, acc1);
                PieceStore<BITS>::st(my_stage + (stage_base + piece) * BITS, acc0, acc1);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int piece = (k << log2_L) + j;
                uint32_t acc0, acc1;
                if (NM == kRefCompat) {
                    encode_piece_ref<BITS>(xf + k * 8, mn, y, acc0, acc1);
                } else {
                    float u8[8];
                    if (NM == kNoiseTensor) load_noise8(u8, noise, group_e0 + (int64_t)piece * 8, valid);
                    encode_piece_slow<BITS, NM>(xf + k * 8, u8, mn, s, ctr_lo0 + (uint32_t)(piece * 2),
                                                ctr_hi, key_lo, acc0, acc1);
                }
                PieceStore<BITS>::st(my_stage + (stage_base + piece) * BITS, acc0, acc1);
            }
        }
        __syncwarp();

        // ---- coalesced write-out of the tile's packed bytes ---------------------------
        const int64_t out_base = tile * (int64_t)TILE_OUT;
        const int64_t remain_e = n_elems - tile * kTileElems;
        if (remain_e >= kTileElems) {
#pragma unroll
            for (int v = lane; v < TILE_OUT / 16; v += 32) {
                const uint4 d = *reinterpret_cast<const uint4*>(my_stage + v * 16);
                stg_stream_v4(packed + out_base + (int64_t)v * 16, d);
            }
        } else {
            const int words = (int)(remain_e * BITS / 32);       // group bytes are a multiple of 4
            for (int w = lane; w < words; w += 32)
                reinterpret_cast<uint32_t*>(packed + out_base)[w] =
                    reinterpret_cast<const uint32_t*>(my_stage)[w];
        }
        __syncwarp();

        if (!PREFETCH) {
            if (next_tile < n_tiles) {
                const int64_t e0 = next_tile * kTileElems + lane_e0;
                if (e0 < n_elems) load_raw<DT>(raw, xb, e0, log2_L, j); else zero_raw<DT>(raw);
            }
        }
    }
}
// ------------------------------------------------------------------ launcher

// blocks of one instantiation that fit on an SM (asked once per instantiation)
template <int DT, int BITS, int NM>
static int pack_blocks_per_sm() {
    static int cached = 0;
    if (cached == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM>,
                                                          PackCfg<DT>::threads, 0) != cudaSuccess || n < 1) n = 1;
        cached = n;
    }
    return cached;
}

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm);   // cabi.cu

template <int DT, int BITS, int NM>
static cudaError_t launch_pack_one(const void* x, const float* noise, void* packed, float* scale,
                                   float* mn, int64_t n_elems, int log2_L, uint64_t seed,
                                   uint64_t offset, int flags, float clamp_alpha, cudaStream_t st)
{
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    // persistent grid: exactly the resident blocks of one wave (or fewer for small inputs)
    const int grid = stream_grid_for((n_tiles + PackCfg<DT>::warps - 1) / PackCfg<DT>::warps, pack_blocks_per_sm<DT, BITS, NM>());
    quant_pack_kernel<DT, BITS, NM><<<grid, PackCfg<DT>::threads, 0, st>>>(
        x, noise, static_cast<uint8_t*>(packed), scale, mn, n_elems, log2_L,
        (uint32_t)key, (uint32_t)(key >> 32), flags, clamp_alpha);
    return cudaGetLastError();
}

template <int DT, int BITS>
static cudaError_t launch_pack_mode(int mode, const void* x, const float* noise, void* packed,
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
static cudaError_t launch_pack_bits(int bits, int mode, const void* x, const float* noise,
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

}  // namespace act

extern "C" int act_quant_pack(const void* x, int dtype, int64_t n_groups, int group_size, int bits,
                              const float* noise, uint64_t seed, uint64_t offset, int flags,
                              float clamp_alpha, void* packed, float* scale, float* mn, void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!x || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)packed | (uintptr_t)noise) & 15) return ACT_ERR_ALIGN;
    if (((uintptr_t)scale | (uintptr_t)mn) & 3) return ACT_ERR_ALIGN;

    int mode;
    if (flags & ACT_FLAG_REF_COMPAT) mode = kRefCompat;
    else if (flags & ACT_FLAG_ROUND_NEAREST) mode = kNoiseConst;
    else if (noise) mode = kNoiseTensor;
    else mode = kNoiseHash;

    int log2_L = 0;
    while ((32 << log2_L) < group_size) ++log2_L;
    const int64_t n_elems = n_groups * group_size;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32)
        e = launch_pack_bits<ACT_DTYPE_F32>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    else if (dtype == ACT_DTYPE_BF16)
        e = launch_pack_bits<ACT_DTYPE_BF16>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    else
        e = launch_pack_bits<ACT_DTYPE_F16>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

// ------------------------------------------------ fused activation + derivative codec
namespace act {

template <int DT, int BITS, int NM, int PRO>
static cudaError_t launch_fused_one(const void* x, void* y, void* packed, float* scale, float* mn,
                                    int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset,
                                    cudaStream_t st)
{
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM, PRO>,
                                                          PackCfg<DT>::threads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((n_tiles + PackCfg<DT>::warps - 1) / PackCfg<DT>::warps, per_sm);
    quant_pack_kernel<DT, BITS, NM, PRO><<<grid, PackCfg<DT>::threads, 0, st>>>(
        x, nullptr, static_cast<uint8_t*>(packed), scale, mn, n_elems, log2_L,
        (uint32_t)key, (uint32_t)(key >> 32), 0, 0.0f, static_cast<uint8_t*>(y));
    return cudaGetLastError();
}

template <int DT, int BITS>
static cudaError_t launch_fused_bits(int kind, bool nearest, const void* x, void* y, void* packed,
                                     float* scale, float* mn, int64_t n, int l2, uint64_t seed,
                                     uint64_t offset, cudaStream_t st)
{
    if (kind == ACT_KIND_GELU)
        return nearest ? launch_fused_one<DT, BITS, kNoiseConst, kProGelu>(x, y, packed, scale, mn, n, l2, seed, offset, st)
                       : launch_fused_one<DT, BITS, kNoiseHash, kProGelu>(x, y, packed, scale, mn, n, l2, seed, offset, st);
    return nearest ? launch_fused_one<DT, BITS, kNoiseConst, kProSilu>(x, y, packed, scale, mn, n, l2, seed, offset, st)
                   : launch_fused_one<DT, BITS, kNoiseHash, kProSilu>(x, y, packed, scale, mn, n, l2, seed, offset, st);
}

template <int DT>
static cudaError_t launch_fused(int bits, int kind, bool nearest, const void* x, void* y, void* packed,
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

}  // namespace act

extern "C" int act_activation_fwd_quant_pack(const void* x, int dtype, int kind, int64_t n_groups,
                                             int group_size, int bits, uint64_t seed, uint64_t offset,
                                             int flags, void* y, void* packed, float* scale, float* mn,
                                             void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (kind != ACT_KIND_GELU && kind != ACT_KIND_SILU) return ACT_ERR_UNSUPPORTED;
    if (flags & ~ACT_FLAG_ROUND_NEAREST) return ACT_ERR_UNSUPPORTED;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!x || !y || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)packed) & 15) return ACT_ERR_ALIGN;
    int log2_L = 0;
    while ((32 << log2_L) < group_size) ++log2_L;
    const int64_t n = n_groups * group_size;
    const bool nearest = (flags & ACT_FLAG_ROUND_NEAREST) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_fused<ACT_DTYPE_F32>(bits, kind, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_fused<ACT_DTYPE_BF16>(bits, kind, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, st);
    else e = launch_fused<ACT_DTYPE_F16>(bits, kind, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

// ------------------------------------------------ fused batch-norm normalise + x_hat codec
namespace act {

// ceil(2^32 / d) for the multiply-high division, 0 when d is 1 (then a plain division is used)
static uint32_t magic_for(uint32_t d) {
    if (d <= 1) return 0;
    return (uint32_t)(((1ull << 32) + d - 1) / d);
}

template <int DT, int BITS, int NM>
static cudaError_t launch_bn_one(const void* x, void* y, void* packed, float* scale, float* mn,
                                 int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset,
                                 BNArgs bn, cudaStream_t st)
{
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quant_pack_kernel<DT, BITS, NM, kProBN>,
                                                          PackCfg<DT>::threads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((n_tiles + PackCfg<DT>::warps - 1) / PackCfg<DT>::warps, per_sm);
    quant_pack_kernel<DT, BITS, NM, kProBN><<<grid, PackCfg<DT>::threads, 0, st>>>(
        x, nullptr, static_cast<uint8_t*>(packed), scale, mn, n_elems, log2_L,
        (uint32_t)key, (uint32_t)(key >> 32), 0, 0.0f, static_cast<uint8_t*>(y), bn);
    return cudaGetLastError();
}

template <int DT>
static cudaError_t launch_bn(int bits, bool nearest, const void* x, void* y, void* packed, float* scale,
                             float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn,
                             cudaStream_t st)
{
#define ACT_BN_CASE(B) \
    return nearest ? launch_bn_one<DT, B, kNoiseConst>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st) \
                   : launch_bn_one<DT, B, kNoiseHash>(x, y, packed, scale, mn, n, l2, seed, offset, bn, st)
    switch (bits) {
        case 1: ACT_BN_CASE(1);
        case 2: ACT_BN_CASE(2);
        case 4: ACT_BN_CASE(4);
        default: ACT_BN_CASE(8);
    }
#undef ACT_BN_CASE
}

}  // namespace act

extern "C" int act_bn_fwd_norm_quant_pack(const void* x, int dtype, int64_t n_batch, int channels, int64_t hw,
                                          const float* params, int group_size, int bits, uint64_t seed,
                                          uint64_t offset, int flags, void* y, void* packed, float* scale,
                                          float* mn, void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (flags & ~ACT_FLAG_ROUND_NEAREST) return ACT_ERR_UNSUPPORTED;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_batch < 0 || channels <= 0 || hw <= 0) return ACT_ERR_SIZE;
    // exactness of the multiply-high channel lookup, and channel-uniform groups of four
    if ((hw & 3) || (uint64_t)hw * (uint64_t)(hw + 1024) >= (1ull << 32) ||
        (uint64_t)channels * (uint64_t)(channels + 260) >= (1ull << 32)) return ACT_ERR_UNSUPPORTED;
    const int64_t n = n_batch * channels * hw;
    if (n > (INT64_MAX >> 4) || n % group_size) return ACT_ERR_SIZE;
    if (n == 0) return ACT_OK;
    if (!x || !y || !packed || !scale || !mn || !params) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)packed | (uintptr_t)params) & 15) return ACT_ERR_ALIGN;
    int log2_L = 0;
    while ((32 << log2_L) < group_size) ++log2_L;
    BNArgs bn{reinterpret_cast<const float4*>(params), (uint32_t)hw, (uint32_t)channels,
              magic_for((uint32_t)hw), magic_for((uint32_t)channels)};
    const bool nearest = (flags & ACT_FLAG_ROUND_NEAREST) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_bn<ACT_DTYPE_F32>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_bn<ACT_DTYPE_BF16>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    else e = launch_bn<ACT_DTYPE_F16>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
