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

template <int BITS> __device__ __forceinline__ uint32_t code_at(uint2 w, int i) {
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    if (BITS == 8) return ((i < 4 ? w.x : w.y) >> ((i & 3) * 8)) & MASK;
    return (w.x >> (i * BITS)) & MASK;
}

template <int DT, int BITS>
__global__ void __launch_bounds__(kUnpackThreads)
dequant_unpack_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                      const float* __restrict__ mn, uint8_t* __restrict__ y, int64_t n_elems,
                      int log2_gs)
{
    const int lane = threadIdx.x & 31;
    const int64_t n_chunks = (n_elems + 255) >> 8;
    const int64_t warp_stride = (int64_t)gridDim.x * kUnpackWarps;
    for (int64_t c4 = ((int64_t)blockIdx.x * kUnpackWarps + (threadIdx.x >> 5)) * 4; c4 < n_chunks;
         c4 += warp_stride * 4) {
        uint2 w[4];
        float s[4], m[4];
        bool ok[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t e = ((c4 + k) << 8) + lane * 8;
            ok[k] = e < n_elems;
            if (ok[k]) {
                w[k] = CodeLoad<BITS>::ld(packed + (e >> 3) * BITS);
                const int64_t g = e >> log2_gs;
                s[k] = __ldg(scale + g);
                m[k] = __ldg(mn + g);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (!ok[k]) continue;
            const int64_t e = ((c4 + k) << 8) + lane * 8;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                // integer code -> float through the 2^23 bit pattern (exact)
                const float cf = __uint_as_float(kMagicBits | code_at<BITS>(w[k], i)) - kMagic;
                v[i] = __fmaf_rn(cf, s[k], m[k]);
            }
            if (DT == ACT_DTYPE_F32) {
                uint4 a, b;
                a.x = __float_as_uint(v[0]); a.y = __float_as_uint(v[1]);
                a.z = __float_as_uint(v[2]); a.w = __float_as_uint(v[3]);
                b.x = __float_as_uint(v[4]); b.y = __float_as_uint(v[5]);
                b.z = __float_as_uint(v[6]); b.w = __float_as_uint(v[7]);
                stg_stream_v4(y + e * 4, a);
                stg_stream_v4(y + e * 4 + 16, b);
            } else if (DT == ACT_DTYPE_BF16) {
                uint4 a;
                __nv_bfloat162 t;
                t = __floats2bfloat162_rn(v[0], v[1]); a.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(v[2], v[3]); a.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(v[4], v[5]); a.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(v[6], v[7]); a.w = *reinterpret_cast<uint32_t*>(&t);
                stg_stream_v4(y + e * 2, a);
            } else {
                uint4 a;
                __half2 t;
                t = __floats2half2_rn(v[0], v[1]); a.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2half2_rn(v[2], v[3]); a.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2half2_rn(v[4], v[5]); a.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2half2_rn(v[6], v[7]); a.w = *reinterpret_cast<uint32_t*>(&t);
                stg_stream_v4(y + e * 2, a);
            }
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

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm);   // cabi.cu

static bool bits_ok(int bits) { return bits == 1 || bits == 2 || bits == 4 || bits == 8; }
static bool group_ok(int gs) { return gs >= 32 && gs <= 1024 && !(gs & (gs - 1)); }

template <int DT>
static void launch_unpack(int bits, const uint8_t* p, const float* s, const float* m, uint8_t* y,
                          int64_t n_elems, int log2_gs, int grid, cudaStream_t st)
{
    switch (bits) {
        case 1: dequant_unpack_kernel<DT, 1><<<grid, kUnpackThreads, 0, st>>>(p, s, m, y, n_elems, log2_gs); break;
        case 2: dequant_unpack_kernel<DT, 2><<<grid, kUnpackThreads, 0, st>>>(p, s, m, y, n_elems, log2_gs); break;
        case 4: dequant_unpack_kernel<DT, 4><<<grid, kUnpackThreads, 0, st>>>(p, s, m, y, n_elems, log2_gs); break;
        default: dequant_unpack_kernel<DT, 8><<<grid, kUnpackThreads, 0, st>>>(p, s, m, y, n_elems, log2_gs); break;
    }
}

}  // namespace act

extern "C" int act_dequant_unpack(const void* packed, const float* scale, const float* mn,
                                  int64_t n_groups, int group_size, int bits, int out_dtype,
                                  void* y, void* stream)
{
    using namespace act;
    if (out_dtype != ACT_DTYPE_F32 && out_dtype != ACT_DTYPE_BF16 && out_dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (!bits_ok(bits)) return ACT_ERR_BITS;
    if (!group_ok(group_size)) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!packed || !scale || !mn || !y) return ACT_ERR_NULL;
    if (((uintptr_t)y & 15) || ((uintptr_t)packed & 7) || (((uintptr_t)scale | (uintptr_t)mn) & 3)) return ACT_ERR_ALIGN;
    int log2_gs = 5;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    const int64_t n_elems = n_groups * group_size;
    const int64_t tiles = (n_elems + kTileElems - 1) / kTileElems;
    const int grid = stream_grid_for((tiles + kUnpackWarps - 1) / kUnpackWarps, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    uint8_t* out = static_cast<uint8_t*>(y);
    if (out_dtype == ACT_DTYPE_F32) launch_unpack<ACT_DTYPE_F32>(bits, p, scale, mn, out, n_elems, log2_gs, grid, st);
    else if (out_dtype == ACT_DTYPE_BF16) launch_unpack<ACT_DTYPE_BF16>(bits, p, scale, mn, out, n_elems, log2_gs, grid, st);
    else launch_unpack<ACT_DTYPE_F16>(bits, p, scale, mn, out, n_elems, log2_gs, grid, st);
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
