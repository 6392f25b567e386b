// Unpack-and-dequantise (backward-pass half of the codec), plain bit pack/unpack
// of int8 masks, and the per-row min/max helper.  sm_100a.
//
// Unpack decomposition: a warp handles a tile of 1024 elements as four chunks of
// 256; in a chunk every lane owns 8 consecutive elements, i.e. BITS bytes of
// codes in and one (16-bit types) or two (fp32) 16-byte vectors out, so every
// load and store instruction of the warp is contiguous.  scale and min are read
// per chunk through the read-only path (all lanes of a group hit the same word).
//
// HBM traffic per element: bits/8 read, s_out written, 8/GS for scale+min.
//
// Replaces: Activation_Compression/act_triton_kernel.py:174-241 (dequant_unpack_kernel),
// :246-322 (pack_kernel / unpack_kernel),
// Activation_Compression/cpp_extension/include/dequant_unpack_1bit_sm90.cuh:5-281,
// Activation_Compression/cpp_extension/src/min_max_kernel.cu:66-141.
#include "act_common.cuh"

namespace act {

constexpr int kUnpackThreads = 256;
constexpr int kUnpackWarps = kUnpackThreads / 32;

template <int BITS> struct CodeLoad;   // the BITS bytes holding 8 consecutive codes
template <> struct CodeLoad<1> { static __device__ __forceinline__ uint2 ld(const uint8_t* p) { return make_uint2(__ldg(p), 0u); } };
template <> struct CodeLoad<2> { static __device__ __forceinline__ uint2 ld(const uint8_t* p) { return make_uint2(__ldg(reinterpret_cast<const uint16_t*>(p)), 0u); } };
template <> struct CodeLoad<4> { static __device__ __forceinline__ uint2 ld(const uint8_t* p) { return make_uint2(__ldg(reinterpret_cast<const uint32_t*>(p)), 0u); } };
template <> struct CodeLoad<8> { static __device__ __forceinline__ uint2 ld(const uint8_t* p) { return __ldg(reinterpret_cast<const uint2*>(p)); } };

// bit pattern of the float 2^23 + code i of the piece (exact integer -> float)
template <int BITS> __device__ __forceinline__ uint32_t code_bits_at(uint2 w, int i) {
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    if (BITS == 8) return __byte_perm(i < 4 ? w.x : w.y, kMagicBits, 0x7440 + (i & 3));   // byte -> low byte
    if (i == 0) return (w.x & MASK) | kMagicBits;
    return ((w.x >> (i * BITS)) & MASK) | kMagicBits;
}

// Tiled destination addressing (TILED kernels): y is [planes, H, W] and group g is the T x T
// tile (plane, ty, tx), g = (plane * tiles_y + ty) * tiles_x + tx, elements row-major inside the
// tile: the inverse of the grouping the reference makes with a permute and a copy
// (Activation_Compression/modules/tensor_act_reshape_utils.py:113-154).
struct UnpackTiles {
    uint32_t H, W, tiles_x, tiles_y;
    int log2_t;
};
// element offset in y of group-ordered element `ge` (a multiple of 4 or 8, so a run of 4 or 8
// stays inside one tile row)
__device__ __forceinline__ int64_t tiled_offset(int64_t ge, int log2_gs, const UnpackTiles& ta) {
    const uint32_t g = (uint32_t)(ge >> log2_gs);
    const uint32_t pe = (uint32_t)ge & ((1u << log2_gs) - 1u);
    const uint32_t q = g / ta.tiles_x, tx = g - q * ta.tiles_x;
    const uint32_t plane = q / ta.tiles_y, ty = q - plane * ta.tiles_y;
    const uint32_t r = pe >> ta.log2_t, col = pe & ((1u << ta.log2_t) - 1u);
    return ((int64_t)plane * ta.H + ((int64_t)ty << ta.log2_t) + r) * ta.W + ((int64_t)tx << ta.log2_t) + col;
}

template <int DT, int BITS, bool TILED = false>
__global__ void __launch_bounds__(kUnpackThreads)
dequant_unpack_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                      const float* __restrict__ mn, uint8_t* __restrict__ y, int64_t n_elems,
                      int log2_gs, UnpackTiles ta = UnpackTiles{0u, 0u, 1u, 1u, 3})
{
    constexpr int EB = ElemT<DT>::bytes;
    const int lane = threadIdx.x & 31;
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int64_t warp_stride = (int64_t)gridDim.x * kUnpackWarps;
    const f32x2 magic2 = pack2(kMagic, kMagic);
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t tile = (int64_t)blockIdx.x * kUnpackWarps + (threadIdx.x >> 5); tile < n_tiles;
         tile += warp_stride) {
        // per-tile 64-bit bases; everything inside the tile is 32-bit arithmetic
        const int64_t tile_e0 = tile * kTileElems;
        const int remain = (int)((n_elems - tile_e0) < kTileElems ? (n_elems - tile_e0) : kTileElems);
        const uint8_t* p_tile = packed + tile * (kTileElems / 8 * BITS);
        const float* s_tile = scale + (tile_e0 >> log2_gs);
        const float* m_tile = mn + (tile_e0 >> log2_gs);
        uint8_t* y_tile = y + tile_e0 * EB;

        uint2 w[4];
        float s[4], m[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int e = k * 256 + lane * 8;               // element inside the tile
            if (e < remain) {
                w[k] = CodeLoad<BITS>::ld(p_tile + (k * 32 + lane) * BITS);
                s[k] = __ldg(s_tile + (e >> log2_gs));
                m[k] = __ldg(m_tile + (e >> log2_gs));
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int e = k * 256 + lane * 8;
            if (e >= remain) continue;
            const f32x2 s2 = pack2(s[k], s[k]), m2 = pack2(m[k], m[k]);
            if (ElemT<DT>::bytes == 2 && BITS <= 2) {
                // 1- and 2-bit codes to 16-bit outputs: a group has only 2^BITS distinct outputs,
                // so they are computed once per chunk (same fma, same rounding) and every element
                // picks its two bytes out of that table with a byte permute.  A code c becomes
                // the selector nibbles (2c, 2c+1); four codes are spread to four bytes with two
                // integer multiplies whose partial products never overlap.
                uint32_t t_lo, t_hi = 0u;
                {
                    uint32_t f0, f1, f2, f3;
                    unpack2u(fma2_rn(pack2(0.0f, 1.0f), s2, m2), f0, f1);
                    if (DT == ACT_DTYPE_BF16) { const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(f0), __uint_as_float(f1)); t_lo = *reinterpret_cast<const uint32_t*>(&t); }
                    else { const __half2 t = __floats2half2_rn(__uint_as_float(f0), __uint_as_float(f1)); t_lo = *reinterpret_cast<const uint32_t*>(&t); }
                    if (BITS == 2) {
                        unpack2u(fma2_rn(pack2(2.0f, 3.0f), s2, m2), f2, f3);
                        if (DT == ACT_DTYPE_BF16) { const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(f2), __uint_as_float(f3)); t_hi = *reinterpret_cast<const uint32_t*>(&t); }
                        else { const __half2 t = __floats2half2_rn(__uint_as_float(f2), __uint_as_float(f3)); t_hi = *reinterpret_cast<const uint32_t*>(&t); }
                    }
                }
                uint4 a;
                uint32_t* ap = &a.x;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t z;
                    if (BITS == 2) {
                        const uint32_t x = (w[k].x >> (8 * h)) & 0xFFu;           // four codes
                        const uint32_t y = (x * 4097u) & 0x000F000Fu;             // two per half
                        z = (y * 65u) & 0x03030303u;                              // one per byte
                    } else {
                        const uint32_t x = (w[k].x >> (4 * h)) & 0xFu;            // four one-bit codes
                        z = (x * 0x00204081u) & 0x01010101u;                      // one per byte
                    }
                    const uint32_t sel = z * 0x22u + 0x10101010u;
                    ap[2 * h] = __byte_perm(t_lo, t_hi, sel);
                    ap[2 * h + 1] = __byte_perm(t_lo, t_hi, sel >> 16);
                }
                stg_stream_v4(TILED ? y + tiled_offset(tile_e0 + e, log2_gs, ta) * 2 : y_tile + e * 2, a);
                continue;
            }
            uint32_t o[8];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                // codes -> floats through the 2^23 bit pattern, then one fused multiply-add
                const f32x2 c2 = sub2_rn(pack2u(code_bits_at<BITS>(w[k], 2 * p),
                                                code_bits_at<BITS>(w[k], 2 * p + 1)), magic2);
                unpack2u(fma2_rn(c2, s2, m2), o[2 * p], o[2 * p + 1]);
            }
            uint8_t* dst = TILED ? y + tiled_offset(tile_e0 + e, log2_gs, ta) * EB : y_tile + e * EB;
            if (DT == ACT_DTYPE_F32) {
                stg_stream_v4(dst, make_uint4(o[0], o[1], o[2], o[3]));
                stg_stream_v4(dst + 16, make_uint4(o[4], o[5], o[6], o[7]));
            } else {
                uint4 a;
                uint32_t* ap = &a.x;
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float lo = __uint_as_float(o[2 * p]), hi = __uint_as_float(o[2 * p + 1]);
                    if (DT == ACT_DTYPE_BF16) {
                        const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
                        ap[p] = *reinterpret_cast<const uint32_t*>(&t);
                    } else {
                        const __half2 t = __floats2half2_rn(lo, hi);
                        ap[p] = *reinterpret_cast<const uint32_t*>(&t);
                    }
                }
                stg_stream_v4(dst, a);
            }
        }
    }
}

// fp32 output: a lane owns 4 consecutive elements per store (one 16-byte vector), eight
// stores per 1024-element tile, so each store instruction of the warp writes 512 contiguous
// bytes.  The 4*BITS code bits of a lane never straddle a 32-bit word.
template <int BITS>
__global__ void __launch_bounds__(kUnpackThreads)
dequant_unpack_f32_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scale,
                          const float* __restrict__ mn, float* __restrict__ y, int64_t n_elems,
                          int log2_gs)
{
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int lane = threadIdx.x & 31;
    const int64_t n_tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int64_t warp_stride = (int64_t)gridDim.x * kUnpackWarps;
    const f32x2 magic2 = pack2(kMagic, kMagic);
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t tile = (int64_t)blockIdx.x * kUnpackWarps + (threadIdx.x >> 5); tile < n_tiles;
         tile += warp_stride) {
        const int64_t tile_e0 = tile * kTileElems;
        const int remain = (int)((n_elems - tile_e0) < kTileElems ? (n_elems - tile_e0) : kTileElems);
        const uint32_t* p_tile = packed + tile * (kTileElems * BITS / 32);
        const float* s_tile = scale + (tile_e0 >> log2_gs);
        const float* m_tile = mn + (tile_e0 >> log2_gs);
        float* y_tile = y + tile_e0;
        uint32_t w[8];
        float s[8], m[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int e = k * 128 + lane * 4;
            if (e < remain) {
                w[k] = __ldg(p_tile + ((e * BITS) >> 5)) >> ((e * BITS) & 31);
                s[k] = __ldg(s_tile + (e >> log2_gs));
                m[k] = __ldg(m_tile + (e >> log2_gs));
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int e = k * 128 + lane * 4;
            if (e >= remain) continue;
            const f32x2 s2 = pack2(s[k], s[k]), m2 = pack2(m[k], m[k]);
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const f32x2 c2 = sub2_rn(pack2u(((w[k] >> (2 * p * BITS)) & MASK) | kMagicBits,
                                                ((w[k] >> ((2 * p + 1) * BITS)) & MASK) | kMagicBits), magic2);
                unpack2u(fma2_rn(c2, s2, m2), o[2 * p], o[2 * p + 1]);
            }
            stg_stream_v4(y_tile + e, make_uint4(o[0], o[1], o[2], o[3]));
        }
    }
}

// ---- int8 <-> bits -----------------------------------------------------------
// A lane owns 16 consecutive int8 values (one 16-byte vector) = 2*BITS bytes of
// packed output; 32-element word boundaries are respected because 16 | 32/BITS*BITS.

template <int BITS>
__global__ void __launch_bounds__(256)
pack_bits_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ packed, int64_t n_elems)
{
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int64_t n_vec = n_elems >> 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += stride) {
        const uint4 d = ldg_nc_v4(x + v * 16);
        const uint32_t r[4] = {d.x, d.y, d.z, d.w};
        uint32_t lo = 0, hi = 0;       // 16*BITS bits: lo only for BITS<=2, lo+hi for 4, 4 words for 8
        if (BITS == 8) {
            *reinterpret_cast<uint4*>(packed + v * 16) = d;      // identity layout
            continue;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t c = (r[i >> 2] >> ((i & 3) * 8)) & MASK;
            const int bit = i * BITS;
            if (bit < 32) lo |= c << bit; else hi |= c << (bit - 32);
        }
        if (BITS == 1) *reinterpret_cast<uint16_t*>(packed + v * 2) = (uint16_t)lo;
        else if (BITS == 2) *reinterpret_cast<uint32_t*>(packed + v * 4) = lo;
        else *reinterpret_cast<uint2*>(packed + v * 8) = make_uint2(lo, hi);
    }
}

template <int BITS>
__global__ void __launch_bounds__(256)
unpack_bits_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ y, int64_t n_elems)
{
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int64_t n_vec = n_elems >> 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += stride) {
        uint32_t lo = 0, hi = 0;
        if (BITS == 8) {
            *reinterpret_cast<uint4*>(y + v * 16) = ldg_nc_v4(packed + v * 16);
            continue;
        }
        if (BITS == 1) lo = __ldg(reinterpret_cast<const uint16_t*>(packed + v * 2));
        else if (BITS == 2) lo = __ldg(reinterpret_cast<const uint32_t*>(packed + v * 4));
        else { const uint2 t = __ldg(reinterpret_cast<const uint2*>(packed + v * 8)); lo = t.x; hi = t.y; }
        uint32_t r[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int bit = i * BITS;
            const uint32_t c = ((bit < 32 ? lo >> bit : hi >> (bit - 32))) & MASK;
            r[i >> 2] |= c << ((i & 3) * 8);
        }
        *reinterpret_cast<uint4*>(y + v * 16) = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

// ---- per-row min / max ---------------------------------------------------------
// One warp per row, lanes stride over the columns; NaN propagates, -0 < +0.
template <int DT>
__global__ void __launch_bounds__(256)
minmax_kernel(const void* __restrict__ x_, float* __restrict__ mn_out, float* __restrict__ mx_out,
              int64_t rows, int64_t cols)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp_stride = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warp_stride) {
        float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);
        for (int64_t c = lane; c < cols; c += 32) {
            float f;
            if (DT == ACT_DTYPE_F32) f = static_cast<const float*>(x_)[r * cols + c];
            else if (DT == ACT_DTYPE_BF16) f = __bfloat162float(static_cast<const __nv_bfloat16*>(x_)[r * cols + c]);
            else f = __half2float(static_cast<const __half*>(x_)[r * cols + c]);
            lo = fmin_nan(lo, f); hi = fmax_nan(hi, f);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            lo = fmin_nan(lo, __shfl_xor_sync(0xffffffffu, lo, off));
            hi = fmax_nan(hi, __shfl_xor_sync(0xffffffffu, hi, off));
        }
        if (lane == 0) { mn_out[r] = lo; mx_out[r] = hi; }
    }
}

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves = 1);   // cabi.cu

static bool bits_ok(int bits) { return bits == 1 || bits == 2 || bits == 4 || bits == 8; }
static bool group_ok(int gs) { return gs >= 32 && gs <= 1024 && !(gs & (gs - 1)); }

template <int DT, int BITS>
static void launch_unpack_one(const uint8_t* p, const float* s, const float* m, uint8_t* y,
                              int64_t n_elems, int log2_gs, cudaStream_t st)
{
    static int per_sm = 0;          // resident blocks of this instantiation, asked once
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, dequant_unpack_kernel<DT, BITS>,
                                                          kUnpackThreads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const int64_t tiles = (n_elems + kTileElems - 1) / kTileElems;
    if (DT == ACT_DTYPE_F32) {
        // fully coalesced fp32 stores (needs the packed words 4-byte aligned, checked by the caller)
        static int per_sm_f32 = 0;
        if (per_sm_f32 == 0) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, dequant_unpack_f32_kernel<BITS>,
                                                              kUnpackThreads, 0) != cudaSuccess || n < 1) n = 1;
            per_sm_f32 = n;
        }
        const int grid = stream_grid_for((tiles + kUnpackWarps - 1) / kUnpackWarps, per_sm_f32, kDecoderWaves);
        launch_overlapped(dequant_unpack_f32_kernel<BITS>, grid, kUnpackThreads, st,
                          reinterpret_cast<const uint32_t*>(p), s, m, reinterpret_cast<float*>(y), n_elems, log2_gs);
        return;
    }
    const int grid = stream_grid_for((tiles + kUnpackWarps - 1) / kUnpackWarps, per_sm, kDecoderWaves);
    launch_overlapped(dequant_unpack_kernel<DT, BITS, false>, grid, kUnpackThreads, st, p, s, m, y, n_elems, log2_gs,
                      UnpackTiles{0u, 0u, 1u, 1u, 3});
}

template <int DT>
static void launch_unpack(int bits, const uint8_t* p, const float* s, const float* m, uint8_t* y,
                          int64_t n_elems, int log2_gs, cudaStream_t st)
{
    switch (bits) {
        case 1: launch_unpack_one<DT, 1>(p, s, m, y, n_elems, log2_gs, st); break;
        case 2: launch_unpack_one<DT, 2>(p, s, m, y, n_elems, log2_gs, st); break;
        case 4: launch_unpack_one<DT, 4>(p, s, m, y, n_elems, log2_gs, st); break;
        default: launch_unpack_one<DT, 8>(p, s, m, y, n_elems, log2_gs, st); break;
    }
}

template <int DT, int BITS>
static void launch_unpack_tiled_one(const uint8_t* p, const float* s, const float* m, uint8_t* y,
                                    int64_t n_elems, int log2_gs, UnpackTiles ta, cudaStream_t st)
{
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, dequant_unpack_kernel<DT, BITS, true>,
                                                          kUnpackThreads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const int64_t tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((tiles + kUnpackWarps - 1) / kUnpackWarps, per_sm, kDecoderWaves);
    launch_overlapped(dequant_unpack_kernel<DT, BITS, true>, grid, kUnpackThreads, st, p, s, m, y, n_elems, log2_gs, ta);
}

template <int DT>
static void launch_unpack_tiled(int bits, const uint8_t* p, const float* s, const float* m, uint8_t* y,
                                int64_t n_elems, int log2_gs, UnpackTiles ta, cudaStream_t st)
{
    switch (bits) {
        case 1: launch_unpack_tiled_one<DT, 1>(p, s, m, y, n_elems, log2_gs, ta, st); break;
        case 2: launch_unpack_tiled_one<DT, 2>(p, s, m, y, n_elems, log2_gs, ta, st); break;
        case 4: launch_unpack_tiled_one<DT, 4>(p, s, m, y, n_elems, log2_gs, ta, st); break;
        default: launch_unpack_tiled_one<DT, 8>(p, s, m, y, n_elems, log2_gs, ta, st); break;
    }
}

}  // namespace act

extern "C" int act_dequant_unpack_tiles(const void* packed, const float* scale, const float* mn,
                                        int64_t n_planes, int height, int width, int tile, int bits,
                                        int out_dtype, void* y, void* stream)
{
    using namespace act;
    if (out_dtype != ACT_DTYPE_F32 && out_dtype != ACT_DTYPE_BF16 && out_dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (!bits_ok(bits)) return ACT_ERR_BITS;
    if (tile != 8 && tile != 16 && tile != 32) return ACT_ERR_GROUP;
    if (n_planes < 0 || height <= 0 || width <= 0 || height % tile || width % tile) return ACT_ERR_SIZE;
    const int64_t groups = n_planes * (height / tile) * (width / tile);
    if (n_planes > (1ll << 31) || groups >= (1ll << 32)) return ACT_ERR_SIZE;
    if (groups == 0) return ACT_OK;
    if (!packed || !scale || !mn || !y) return ACT_ERR_NULL;
    if (((uintptr_t)y & 15) || ((uintptr_t)packed & 7) || (((uintptr_t)scale | (uintptr_t)mn) & 3)) return ACT_ERR_ALIGN;
    int log2_t = 3;
    while ((1 << log2_t) < tile) ++log2_t;
    const int log2_gs = 2 * log2_t;
    const int64_t n_elems = groups << log2_gs;
    const UnpackTiles ta{(uint32_t)height, (uint32_t)width, (uint32_t)(width / tile), (uint32_t)(height / tile), log2_t};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    uint8_t* out = static_cast<uint8_t*>(y);
    if (out_dtype == ACT_DTYPE_F32) launch_unpack_tiled<ACT_DTYPE_F32>(bits, p, scale, mn, out, n_elems, log2_gs, ta, st);
    else if (out_dtype == ACT_DTYPE_BF16) launch_unpack_tiled<ACT_DTYPE_BF16>(bits, p, scale, mn, out, n_elems, log2_gs, ta, st);
    else launch_unpack_tiled<ACT_DTYPE_F16>(bits, p, scale, mn, out, n_elems, log2_gs, ta, st);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

namespace act {
// codec_bits3.cu
cudaError_t dequant_unpack3(const void* packed, const float* scale, const float* mn, int out_dtype, void* y,
                            int64_t n_elems, int log2_gs, cudaStream_t st);
}  // namespace act

extern "C" int act_dequant_unpack(const void* packed, const float* scale, const float* mn,
                                  int64_t n_groups, int group_size, int bits, int out_dtype,
                                  void* y, void* stream)
{
    using namespace act;
    if (out_dtype != ACT_DTYPE_F32 && out_dtype != ACT_DTYPE_BF16 && out_dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (!bits_ok(bits) && bits != 3) return ACT_ERR_BITS;
    if (!group_ok(group_size)) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!packed || !scale || !mn || !y) return ACT_ERR_NULL;
    if (((uintptr_t)y & 15) || ((uintptr_t)packed & 7) || (((uintptr_t)scale | (uintptr_t)mn) & 3)) return ACT_ERR_ALIGN;
    int log2_gs = 5;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    const int64_t n_elems = n_groups * group_size;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (bits == 3)          // bit-plane layout (codec_bits3.cu)
        return dequant_unpack3(packed, scale, mn, out_dtype, y, n_elems, log2_gs, st) == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    uint8_t* out = static_cast<uint8_t*>(y);
    if (out_dtype == ACT_DTYPE_F32) launch_unpack<ACT_DTYPE_F32>(bits, p, scale, mn, out, n_elems, log2_gs, st);
    else if (out_dtype == ACT_DTYPE_BF16) launch_unpack<ACT_DTYPE_BF16>(bits, p, scale, mn, out, n_elems, log2_gs, st);
    else launch_unpack<ACT_DTYPE_F16>(bits, p, scale, mn, out, n_elems, log2_gs, st);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_pack_bits(const int8_t* x, int64_t n_groups, int group_size, int bits,
                             void* packed, void* stream)
{
    using namespace act;
    if (!bits_ok(bits)) return ACT_ERR_BITS;
    if (!group_ok(group_size)) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!x || !packed) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)packed) & 15) return ACT_ERR_ALIGN;
    const int64_t n_elems = n_groups * group_size;
    const int grid = stream_grid_for(((n_elems >> 4) + 255) / 256, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* xi = reinterpret_cast<const uint8_t*>(x);
    uint8_t* p = static_cast<uint8_t*>(packed);
    switch (bits) {
        case 1: pack_bits_kernel<1><<<grid, 256, 0, st>>>(xi, p, n_elems); break;
        case 2: pack_bits_kernel<2><<<grid, 256, 0, st>>>(xi, p, n_elems); break;
        case 4: pack_bits_kernel<4><<<grid, 256, 0, st>>>(xi, p, n_elems); break;
        default: pack_bits_kernel<8><<<grid, 256, 0, st>>>(xi, p, n_elems); break;
    }
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_unpack_bits(const void* packed, int64_t n_groups, int group_size, int bits,
                               int8_t* y, void* stream)
{
    using namespace act;
    if (!bits_ok(bits)) return ACT_ERR_BITS;
    if (!group_ok(group_size)) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!y || !packed) return ACT_ERR_NULL;
    if (((uintptr_t)y | (uintptr_t)packed) & 15) return ACT_ERR_ALIGN;
    const int64_t n_elems = n_groups * group_size;
    const int grid = stream_grid_for(((n_elems >> 4) + 255) / 256, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    uint8_t* out = reinterpret_cast<uint8_t*>(y);
    switch (bits) {
        case 1: unpack_bits_kernel<1><<<grid, 256, 0, st>>>(p, out, n_elems); break;
        case 2: unpack_bits_kernel<2><<<grid, 256, 0, st>>>(p, out, n_elems); break;
        case 4: unpack_bits_kernel<4><<<grid, 256, 0, st>>>(p, out, n_elems); break;
        default: unpack_bits_kernel<8><<<grid, 256, 0, st>>>(p, out, n_elems); break;
    }
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_minmax(const void* x, int dtype, int64_t rows, int64_t cols, float* mn,
                          float* mx, void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (rows < 0 || cols <= 0 || (rows > 0 && cols > INT64_MAX / rows)) return ACT_ERR_SIZE;
    if (rows == 0) return ACT_OK;
    if (!x || !mn || !mx) return ACT_ERR_NULL;
    const int grid = stream_grid_for((rows + 7) / 8, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == ACT_DTYPE_F32) minmax_kernel<ACT_DTYPE_F32><<<grid, 256, 0, st>>>(x, mn, mx, rows, cols);
    else if (dtype == ACT_DTYPE_BF16) minmax_kernel<ACT_DTYPE_BF16><<<grid, 256, 0, st>>>(x, mn, mx, rows, cols);
    else minmax_kernel<ACT_DTYPE_F16><<<grid, 256, 0, st>>>(x, mn, mx, rows, cols);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
