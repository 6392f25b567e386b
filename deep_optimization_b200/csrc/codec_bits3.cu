// 3-bit codes: quantise-and-pack and unpack-and-dequantise, sm_100a.
//
// Eight levels do not fill a 32-bit word evenly, so 3-bit codes are stored as bit planes:
// every 32 consecutive elements take three consecutive words, bit l of word p being bit p of
// the code of element l of the chunk (group_size * 3 / 32 words per group).  Everything else
// is the contract of the 1/2/4/8-bit kernels: per-group fp32 min and scale = (max - min) / 7,
// the noise-tensor formula, the fixed-point counter-hash and round-to-nearest modes, and
// y = fma(code, scale, min).
//
// A warp takes max(group_size, 256) consecutive elements per step; a lane holds U pieces of
// eight consecutive elements (U = group_size / 256, at least 1), piece u at offset
// u * 256 + lane * 8, so loads and stores are 16 bytes per lane and contiguous per warp.  The
// planes of a piece are eight bits per word; the four lanes of a 32-element chunk merge theirs
// with two xor-shuffles and lane 0 of the four writes the three words (12 contiguous bytes).
//
// Replaces: cpp_extension.pack3 / unpack3 (Activation_Compression/cpp_extension/bind.cpp:12,18;
// kernels cpp_extension/include/quant_pack_1bit_sm90.cuh:117-249 with bits = 3, whose planes
// come from warp ballots over four values per thread).
#include "act_common.cuh"

namespace act {

constexpr int kB3Threads = 256;

template <int DT> __device__ __forceinline__ void load_piece(const uint8_t* x, int64_t e, float (&f)[8]) {
    if (ElemT<DT>::bytes == 4) {
        const uint4 a = ldg_stream_v4(x + e * 4), b = ldg_stream_v4(x + e * 4 + 16);
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    } else {
        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
        const uint4 a = ldg_stream_v4(x + e * 2);
        f[0] = widen_lo<D16>(a.x); f[1] = widen_hi<D16>(a.x); f[2] = widen_lo<D16>(a.y); f[3] = widen_hi<D16>(a.y);
        f[4] = widen_lo<D16>(a.z); f[5] = widen_hi<D16>(a.z); f[6] = widen_lo<D16>(a.w); f[7] = widen_hi<D16>(a.w);
    }
}

// MODE 0: counter hash, 1: noise tensor, 2: round to nearest.  U pieces per lane.
template <int DT, int MODE, int U>
__global__ void __launch_bounds__(kB3Threads)
quant_pack3_kernel(const uint8_t* __restrict__ x, const float* __restrict__ noise, uint32_t* __restrict__ packed,
                   float* __restrict__ scale_out, float* __restrict__ min_out, int64_t n_elems, int log2_gs,
                   uint32_t key_lo, uint32_t key_hi)
{
    constexpr int STEP = 256 * U;                               // elements per warp step
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * kB3Threads + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * kB3Threads) >> 5;
    const int lanes_per_group = (U > 1) ? 32 : (1 << (log2_gs - 3));
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t base = warp * STEP; base < n_elems; base += n_warps * STEP) {
        float f[U][8];
        bool ok[U];
        float mn = 0.0f, mx = 0.0f;
        bool first = true;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t e = base + u * 256 + lane * 8;
            ok[u] = e < n_elems;                                 // groups never straddle n_elems
            if (ok[u]) {
                load_piece<DT>(x, e, f[u]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    mn = first ? f[u][i] : fmin_nan(mn, f[u][i]);
                    mx = first ? f[u][i] : fmax_nan(mx, f[u][i]);
                    first = false;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[u][i] = 0.0f;
            }
        }
        // the element count is a multiple of the group size, so a lane past the end shares its
        // group only with other lanes past the end: it takes part in the shuffles and writes nothing
        for (int off = lanes_per_group >> 1; off > 0; off >>= 1) {
            const float omn = __shfl_xor_sync(0xffffffffu, mn, off), omx = __shfl_xor_sync(0xffffffffu, mx, off);
            mn = fmin_nan(mn, omn); mx = fmax_nan(mx, omx);
        }
        const float r = __fsub_rn(mx, mn);
        float s = __fdiv_rn(r, 7.0f);
        if (!(s > 0.0f)) s = 1.0f;
        const float inv = __fdiv_rn(1.0f, s);
        const bool regular = (r == 0.0f) || (r >= 0x1p-50f && r <= 0x1p50f);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t e = base + u * 256 + lane * 8;
            uint32_t h0 = 0u, h1 = 0u;
            if (MODE == 0) {
                const uint64_t ctr = (uint64_t)e >> 3;
                hash_2x32_split((uint32_t)ctr, (uint32_t)(ctr >> 32) ^ key_hi, key_lo, h0, h1);
            }
            float un[8];
            if (MODE == 1) {
                if (ok[u]) {
                    const uint4 a = ldg_stream_v4(noise + e), b = ldg_stream_v4(noise + e + 4);
                    un[0] = __uint_as_float(a.x); un[1] = __uint_as_float(a.y); un[2] = __uint_as_float(a.z); un[3] = __uint_as_float(a.w);
                    un[4] = __uint_as_float(b.x); un[5] = __uint_as_float(b.y); un[6] = __uint_as_float(b.z); un[7] = __uint_as_float(b.w);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) un[i] = 0.0f;
                }
            }
            uint32_t p0 = 0u, p1 = 0u, p2 = 0u;                  // the piece's eight bits of each plane
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a = __fsub_rn(f[u][i], mn);
                uint32_t c;
                if (MODE == 1) {
                    c = code_from_t(__fadd_rn(__fdiv_rn(a, s), un[i]), 7);
                } else {
                    const uint32_t h = (MODE == 2) ? 127u : (((i < 4 ? h0 : h1) >> ((i & 3) * 8)) & 0xFFu);
                    if (regular) {
                        const uint32_t q = __float_as_uint(__fmaf_rn(a, inv, 32768.0f)) - 0x47000000u;
                        c = (q + h) >> 8;
                    } else {
                        const float uu = (MODE == 2) ? 0.5f - 1e-6f : __fmul_rn((float)h, 0x1p-8f);
                        c = code_from_t(__fadd_rn(__fdiv_rn(a, s), uu), 7);
                    }
                }
                p0 |= (c & 1u) << i; p1 |= ((c >> 1) & 1u) << i; p2 |= ((c >> 2) & 1u) << i;
            }
            // the four lanes of a chunk: lane q of them holds bits [8q, 8q+8) of each word
            const int q = lane & 3;
            p0 <<= 8 * q; p1 <<= 8 * q; p2 <<= 8 * q;
#pragma unroll
            for (int off = 1; off < 4; off <<= 1) {
                p0 |= __shfl_xor_sync(0xffffffffu, p0, off);
                p1 |= __shfl_xor_sync(0xffffffffu, p1, off);
                p2 |= __shfl_xor_sync(0xffffffffu, p2, off);
            }
            if (ok[u] && q == 0) {
                uint32_t* w = packed + (e >> 5) * 3;
                w[0] = p0; w[1] = p1; w[2] = p2;
            }
        }
        // one lane per group writes scale and min
        const int64_t e0 = base + lane * 8;
        if (e0 < n_elems && (lane & (lanes_per_group - 1)) == 0) {
            const int64_t g = e0 >> log2_gs;
            scale_out[g] = s;
            min_out[g] = mn;
        }
    }
}

template <int DT>
__global__ void __launch_bounds__(kB3Threads)
dequant_unpack3_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scale,
                       const float* __restrict__ mn, uint8_t* __restrict__ y, int64_t n_elems, int log2_gs)
{
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kB3Threads;
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t p = (int64_t)blockIdx.x * kB3Threads + threadIdx.x; p < n_pieces; p += stride) {
        const int64_t e = p * 8;
        const uint32_t* w = packed + (e >> 5) * 3;
        const int sh = (int)(p & 3) * 8;
        const uint32_t p0 = __ldg(w) >> sh, p1 = __ldg(w + 1) >> sh, p2 = __ldg(w + 2) >> sh;
        const int64_t g = e >> log2_gs;
        const float s = __ldg(scale + g), m = __ldg(mn + g);
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t c = ((p0 >> i) & 1u) | (((p1 >> i) & 1u) << 1) | (((p2 >> i) & 1u) << 2);
            f[i] = __fmaf_rn(__uint_as_float(kMagicBits | c) - kMagic, s, m);
        }
        if (DT == ACT_DTYPE_F32) {
            stg_stream_v4(y + e * 4, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
            stg_stream_v4(y + e * 4 + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
        } else {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (DT == ACT_DTYPE_BF16) { const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
                else { const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
            }
            stg_stream_v4(y + e * 2, make_uint4(o[0], o[1], o[2], o[3]));
        }
    }
}

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves = 1);   // cabi.cu

template <int DT, int MODE>
static cudaError_t launch_pack3_u(const uint8_t* x, const float* noise, uint32_t* packed, float* scale, float* mn,
                                  int64_t n_elems, int log2_gs, uint32_t key_lo, uint32_t key_hi, cudaStream_t st)
{
    const int u = log2_gs <= 8 ? 1 : (1 << (log2_gs - 8));
    const int64_t warps = (n_elems + 256 * u - 1) / (256 * u);
    const int grid = stream_grid_for((warps + kB3Threads / 32 - 1) / (kB3Threads / 32), 4);
    if (u == 1) return launch_overlapped(quant_pack3_kernel<DT, MODE, 1>, grid, kB3Threads, st, x, noise, packed, scale, mn, n_elems, log2_gs, key_lo, key_hi);
    if (u == 2) return launch_overlapped(quant_pack3_kernel<DT, MODE, 2>, grid, kB3Threads, st, x, noise, packed, scale, mn, n_elems, log2_gs, key_lo, key_hi);
    return launch_overlapped(quant_pack3_kernel<DT, MODE, 4>, grid, kB3Threads, st, x, noise, packed, scale, mn, n_elems, log2_gs, key_lo, key_hi);
}

template <int DT>
static cudaError_t launch_pack3(int mode, const uint8_t* x, const float* noise, uint32_t* packed, float* scale, float* mn,
                                int64_t n_elems, int log2_gs, uint32_t key_lo, uint32_t key_hi, cudaStream_t st)
{
    if (mode == 1) return launch_pack3_u<DT, 1>(x, noise, packed, scale, mn, n_elems, log2_gs, key_lo, key_hi, st);
    if (mode == 2) return launch_pack3_u<DT, 2>(x, noise, packed, scale, mn, n_elems, log2_gs, key_lo, key_hi, st);
    return launch_pack3_u<DT, 0>(x, noise, packed, scale, mn, n_elems, log2_gs, key_lo, key_hi, st);
}

// called by act_quant_pack / act_dequant_unpack after their argument checks, bits == 3
cudaError_t quant_pack3(const void* x, int dtype, const float* noise, int mode, uint64_t seed, uint64_t offset,
                        void* packed, float* scale, float* mn, int64_t n_elems, int log2_gs, cudaStream_t st)
{
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    uint32_t* p = static_cast<uint32_t*>(packed);
    const uint32_t klo = (uint32_t)key, khi = (uint32_t)(key >> 32);
    if (dtype == ACT_DTYPE_F32) return launch_pack3<ACT_DTYPE_F32>(mode, xb, noise, p, scale, mn, n_elems, log2_gs, klo, khi, st);
    if (dtype == ACT_DTYPE_BF16) return launch_pack3<ACT_DTYPE_BF16>(mode, xb, noise, p, scale, mn, n_elems, log2_gs, klo, khi, st);
    return launch_pack3<ACT_DTYPE_F16>(mode, xb, noise, p, scale, mn, n_elems, log2_gs, klo, khi, st);
}

cudaError_t dequant_unpack3(const void* packed, const float* scale, const float* mn, int out_dtype, void* y,
                            int64_t n_elems, int log2_gs, cudaStream_t st)
{
    const int grid = stream_grid_for(((n_elems >> 3) + kB3Threads - 1) / kB3Threads, 6);
    const uint32_t* p = static_cast<const uint32_t*>(packed);
    uint8_t* out = static_cast<uint8_t*>(y);
    if (out_dtype == ACT_DTYPE_F32) return launch_overlapped(dequant_unpack3_kernel<ACT_DTYPE_F32>, grid, kB3Threads, st, p, scale, mn, out, n_elems, log2_gs);
    if (out_dtype == ACT_DTYPE_BF16) return launch_overlapped(dequant_unpack3_kernel<ACT_DTYPE_BF16>, grid, kB3Threads, st, p, scale, mn, out, n_elems, log2_gs);
    return launch_overlapped(dequant_unpack3_kernel<ACT_DTYPE_F16>, grid, kB3Threads, st, p, scale, mn, out, n_elems, log2_gs);
}

}  // namespace act
