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
// HBM traffic per element: s_in bytes read, bits/8 written, 8/GS for scale+min.
//
// Replaces: Activation_Compression/act_triton_kernel.py:23-171 (quant_pack_kernel),
// Activation_Compression/cpp_extension/include/quant_pack_1bit_sm90.cuh:18-250.
#include "act_common.cuh"

namespace act {

enum NoiseMode { kNoiseHash = 0, kNoiseTensor = 1, kNoiseConst = 2, kRefCompat = 3 };

constexpr int kPackThreads = 256;
constexpr int kPackWarps = kPackThreads / 32;

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

template <int DT, int BITS, int NM>
__global__ void __launch_bounds__(kPackThreads)
quant_pack_kernel(const void* __restrict__ x_, const float* __restrict__ noise,
                  uint8_t* __restrict__ packed, float* __restrict__ scale_out,
                  float* __restrict__ min_out, int64_t n_elems, int log2_L,
                  uint32_t key_lo, uint32_t key_hi, uint64_t offset, int flags, float clamp_alpha)
{
    constexpr int QMAX = (1 << BITS) - 1;
    constexpr int EB = ElemT<DT>::bytes;
    constexpr int TILE_OUT = kTileElems * BITS / 8;          // packed bytes per tile
    __shared__ __align__(16) uint8_t stage[kPackWarps][TILE_OUT];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int L = 1 << log2_L;                  // lanes per group
    const int j = lane & (L - 1);               // lane index inside the group
    const int g_local = lane >> log2_L;         // group index inside the tile
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int64_t warp_stride = (int64_t)gridDim.x * kPackWarps;
    const uint8_t* xb = static_cast<const uint8_t*>(x_);
    uint8_t* my_stage = stage[warp];

    for (int64_t tile = (int64_t)blockIdx.x * kPackWarps + warp; tile < n_tiles; tile += warp_stride) {
        // element index of the lane's group and validity (groups never straddle n_elems)
        const int64_t group_e0 = tile * kTileElems + ((int64_t)g_local << (log2_L + 5));
        const bool valid = group_e0 < n_elems;

        // ---- load 4 pieces of 8 elements, widened to fp32 ------------------
        float xf[32];
        if (valid) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int64_t e = group_e0 + (int64_t)((k << log2_L) + j) * 8;
                if (EB == 4) {
                    const uint4 a = ldg_nc_v4(xb + e * 4);
                    const uint4 b = ldg_nc_v4(xb + e * 4 + 16);
                    xf[k * 8 + 0] = __uint_as_float(a.x); xf[k * 8 + 1] = __uint_as_float(a.y);
                    xf[k * 8 + 2] = __uint_as_float(a.z); xf[k * 8 + 3] = __uint_as_float(a.w);
                    xf[k * 8 + 4] = __uint_as_float(b.x); xf[k * 8 + 5] = __uint_as_float(b.y);
                    xf[k * 8 + 6] = __uint_as_float(b.z); xf[k * 8 + 7] = __uint_as_float(b.w);
                } else {
                    const uint4 a = ldg_nc_v4(xb + e * 2);
                    constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
                    xf[k * 8 + 0] = widen_lo<D16>(a.x); xf[k * 8 + 1] = widen_hi<D16>(a.x);
                    xf[k * 8 + 2] = widen_lo<D16>(a.y); xf[k * 8 + 3] = widen_hi<D16>(a.y);
                    xf[k * 8 + 4] = widen_lo<D16>(a.z); xf[k * 8 + 5] = widen_hi<D16>(a.z);
                    xf[k * 8 + 6] = widen_lo<D16>(a.w); xf[k * 8 + 7] = widen_hi<D16>(a.w);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) xf[i] = 0.0f;
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

        // ---- group min / max ------------------------------------------------
        float mn = xf[0], mx = xf[0];
#pragma unroll
        for (int i = 1; i < 32; ++i) { mn = fmin_nan(mn, xf[i]); mx = fmax_nan(mx, xf[i]); }
        for (int off = L >> 1; off > 0; off >>= 1) {
            mn = fmin_nan(mn, __shfl_xor_sync(0xffffffffu, mn, off));
            mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        }

        // ---- scale ------------------------------------------------------------
        const float range = __fsub_rn(mx, mn);
        float s = (BITS == 1) ? range : __fdiv_rn(range, (float)QMAX);
        if (!(s > 0.0f)) s = 1.0f;
        // the FMA division and the clamp-free packing need a finite range well inside
        // the normal numbers (then 2^-58 <= s <= 2^50); a denormal, huge, infinite or
        // NaN range goes the slow way, which is the contract's arithmetic verbatim
        const bool fast = (range == 0.0f) || (range >= 0x1p-50f && range <= 0x1p50f);
        const float y = __frcp_rn(s);

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

        // ---- codes ------------------------------------------------------------
        const int64_t hash_ctr0 = (int64_t)((uint64_t)(group_e0 >> 2) + offset);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int piece = (k << log2_L) + j;               // piece index inside the group
            uint32_t acc0 = 0, acc1 = 0;

            if (NM == kRefCompat) {
                // act_triton_kernel.py:71,114,151-153 with the multiply and the add
                // rounded separately, truncation toward zero, integer clamp
                const float half_c = 0.5f - 1e-6f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a = __fsub_rn(xf[k * 8 + i], mn);
                    float t = __fadd_rn(__fmul_rn(a, y), half_c);
                    int c = 0;
                    if (t == t) {
                        t = fminf(fmaxf(t, -1.0e9f), 1.0e9f);
                        c = min(max((int)t, 0), QMAX);
                    }
                    if (BITS == 8 && i >= 4) acc1 |= (uint32_t)c << ((i - 4) * 8);
                    else acc0 |= (uint32_t)c << (i * BITS);
                }
            } else {
                float u[8];
                if (NM == kNoiseHash) {
                    uint32_t w0, w1, w2, w3;
                    const uint64_t c0 = (uint64_t)hash_ctr0 + (uint64_t)(piece * 2);
                    hash_2x32(c0, key_lo, key_hi, w0, w1);
                    hash_2x32(c0 + 1, key_lo, key_hi, w2, w3);
                    u[0] = u16_lo_as_float(w0); u[1] = u16_hi_as_float(w0);
                    u[2] = u16_lo_as_float(w1); u[3] = u16_hi_as_float(w1);
                    u[4] = u16_lo_as_float(w2); u[5] = u16_hi_as_float(w2);
                    u[6] = u16_lo_as_float(w3); u[7] = u16_hi_as_float(w3);
                } else if (NM == kNoiseTensor) {
                    if (valid) {
                        const int64_t e = group_e0 + (int64_t)piece * 8;
                        const uint4 a = ldg_nc_v4(noise + e);
                        const uint4 b = ldg_nc_v4(noise + e + 4);
                        u[0] = __uint_as_float(a.x); u[1] = __uint_as_float(a.y);
                        u[2] = __uint_as_float(a.z); u[3] = __uint_as_float(a.w);
                        u[4] = __uint_as_float(b.x); u[5] = __uint_as_float(b.y);
                        u[6] = __uint_as_float(b.z); u[7] = __uint_as_float(b.w);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) u[i] = 0.0f;
                    }
                }

                if (NM != kNoiseTensor && fast) {
                    // t >= 0 and floor(t) <= QMAX are guaranteed here (for 8-bit hash
                    // noise one fminf restores the upper bound), so floor is a
                    // round-down add of 2^23 and the code is the low mantissa bits
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a = __fsub_rn(xf[k * 8 + i], mn);
                        const float q = div_by_scale(a, s, y);
                        float t;
                        if (NM == kNoiseHash) t = __fmaf_rn(u[i], 0x1p-16f, q);   // exact u*2^-16, one rounding
                        else t = __fadd_rn(q, 0.5f - 1e-6f);
                        if (NM == kNoiseHash && BITS == 8) t = fminf(t, (float)QMAX);
                        const uint32_t tb = __float_as_uint(__fadd_rd(t, kMagic));
                        if (BITS == 8 && i >= 4) acc1 += tb << ((i - 4) * 8);
                        else acc0 += tb << (i * BITS);
                    }
                    if (BITS == 8) { acc0 -= magic_sum<8, 4>(); acc1 -= magic_sum<8, 4>(); }
                    else acc0 -= magic_sum<BITS, 8>();
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a = __fsub_rn(xf[k * 8 + i], mn);
                        const float q = fast ? div_by_scale(a, s, y) : __fdiv_rn(a, s);
                        float uu;
                        if (NM == kNoiseHash) uu = __fmul_rn(u[i], 0x1p-16f);
                        else if (NM == kNoiseTensor) uu = u[i];
                        else uu = 0.5f - 1e-6f;
                        const uint32_t c = code_from_t(__fadd_rn(q, uu), QMAX);
                        if (BITS == 8 && i >= 4) acc1 |= c << ((i - 4) * 8);
                        else acc0 |= c << (i * BITS);
                    }
                }
            }
            // stage the piece's BITS bytes at its place inside the tile
            const int tile_piece = (g_local << (log2_L + 2)) + piece;
            PieceStore<BITS>::st(my_stage + tile_piece * BITS, acc0, acc1);
        }
        __syncwarp();

        // ---- coalesced write-out of the tile's packed bytes -------------------
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
    }
}

// ------------------------------------------------------------------ launcher

template <int DT, int BITS>
static cudaError_t launch_pack_mode(int mode, const void* x, const float* noise, void* packed,
                                    float* scale, float* mn, int64_t n_elems, int log2_L,
                                    uint64_t seed, uint64_t offset, int flags, float clamp_alpha,
                                    cudaStream_t st, int grid)
{
    const uint64_t key = hash_key(seed);
    const uint32_t klo = (uint32_t)key, khi = (uint32_t)(key >> 32);
    uint8_t* p = static_cast<uint8_t*>(packed);
    switch (mode) {
        case kNoiseHash:
            quant_pack_kernel<DT, BITS, kNoiseHash><<<grid, kPackThreads, 0, st>>>(
                x, noise, p, scale, mn, n_elems, log2_L, klo, khi, offset, flags, clamp_alpha);
            break;
        case kNoiseTensor:
            quant_pack_kernel<DT, BITS, kNoiseTensor><<<grid, kPackThreads, 0, st>>>(
                x, noise, p, scale, mn, n_elems, log2_L, klo, khi, offset, flags, clamp_alpha);
            break;
        case kNoiseConst:
            quant_pack_kernel<DT, BITS, kNoiseConst><<<grid, kPackThreads, 0, st>>>(
                x, noise, p, scale, mn, n_elems, log2_L, klo, khi, offset, flags, clamp_alpha);
            break;
        default:
            quant_pack_kernel<DT, BITS, kRefCompat><<<grid, kPackThreads, 0, st>>>(
                x, noise, p, scale, mn, n_elems, log2_L, klo, khi, offset, flags, clamp_alpha);
            break;
    }
    return cudaGetLastError();
}

template <int DT>
static cudaError_t launch_pack_bits(int bits, int mode, const void* x, const float* noise,
                                    void* packed, float* scale, float* mn, int64_t n_elems,
                                    int log2_L, uint64_t seed, uint64_t offset, int flags,
                                    float clamp_alpha, cudaStream_t st, int grid)
{
    switch (bits) {
        case 1: return launch_pack_mode<DT, 1>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
        case 2: return launch_pack_mode<DT, 2>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
        case 4: return launch_pack_mode<DT, 4>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
        default: return launch_pack_mode<DT, 8>(mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
    }
}

int pack_grid_for(int64_t n_tiles);   // defined in cabi.cu

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
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = pack_grid_for(n_tiles);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32)
        e = launch_pack_bits<ACT_DTYPE_F32>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
    else if (dtype == ACT_DTYPE_BF16)
        e = launch_pack_bits<ACT_DTYPE_BF16>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
    else
        e = launch_pack_bits<ACT_DTYPE_F16>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st, grid);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
