// Sub-group averaging ("AVG_ALAM"): A consecutive elements of a group share one code, sm_100a.
//
// The reference's live kernel has this as a switch (Activation_Compression/act_triton_kernel.py:
// 116-118 in quant_pack_kernel, 212-215 in dequant_unpack_kernel): the per-element quotients of
// A = ALAM_BITS neighbours are averaged before rounding, so a group of gs elements stores gs/A
// codes (gs*bits/(32*A) words), and decoding repeats every code A times.
//
// Contract (per group; min, max and scale exactly as act_quant_pack computes them):
//   reference-compatible mode:  qf_i = RN(RN(a_i * RN(1/s)) + (0.5f - 1e-6f)),
//       m = (qf_0 + ... + qf_{A-1}) / A summed left to right in fp32, code = clamp(trunc(m));
//   otherwise:  q_i = RN(a_i / s), m = (q_0 + ... + q_{A-1}) / A summed left to right,
//       code = clamp(floor(RN(m + u)), 0, qmax) with u the noise of the sub-group's FIRST element:
//       the noise tensor's value there, its hash byte / 256, or 0.5f - 1e-6f (round to nearest).
// A is 2, 4 or 8.  Triton sums the A values in a tree, so bytes can differ from the reference's
// in the last place of m; the reference's decoder also adds Gaussian noise to the code, which
// is not reproduced (decoding here is deterministic).
//
// A lane holds pieces of eight consecutive elements (as in the 3-bit kernel), i.e. 8/A codes,
// a field of 8*bits/A bits; 32 / that many lanes merge their fields into a word with
// xor-shuffles.
#include "act_common.cuh"

namespace act {

constexpr int kAvgThreads = 256;

template <int DT> __device__ __forceinline__ void avg_load_piece(const uint8_t* x, int64_t e, float (&f)[8]) {
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

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// MODE 0: counter hash, 1: noise tensor, 2: round to nearest, 3: reference-compatible.
// U pieces per lane (group_size / 256, at least 1).
template <int DT, int MODE, int U>
__global__ void __launch_bounds__(kAvgThreads)
quant_pack_avg_kernel(const uint8_t* __restrict__ x, const float* __restrict__ noise, uint32_t* __restrict__ packed,
                      float* __restrict__ scale_out, float* __restrict__ min_out, int64_t n_elems, int log2_gs,
                      int bits, int log2_a, uint32_t key_lo, uint32_t key_hi, int flags, float clamp_alpha)
{
    constexpr int STEP = 256 * U;
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * kAvgThreads + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * kAvgThreads) >> 5;
    const int lanes_per_group = (U > 1) ? 32 : (1 << (log2_gs - 3));
    const int qmax = (1 << bits) - 1;
    const int A = 1 << log2_a;
    const int codes_per_piece = 8 >> log2_a;
    const int wbits = codes_per_piece * bits;                    // field of one piece
    const int lanes_per_word = 32 / wbits;
    const float inv_a = 1.0f / (float)A;
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
            ok[u] = e < n_elems;
            if (ok[u]) {
                avg_load_piece<DT>(x, e, f[u]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (MODE == 3) {
                        if (flags & ACT_FLAG_REF_CLAMP) f[u][i] = fminf(fmaxf(f[u][i], -clamp_alpha), clamp_alpha);
                        if (flags & ACT_FLAG_REF_TANH) f[u][i] = __fmul_rn(tanhf(__fdiv_rn(f[u][i], 0.5f)), 0.5f);
                    }
                    mn = first ? f[u][i] : fmin_nan(mn, f[u][i]);
                    mx = first ? f[u][i] : fmax_nan(mx, f[u][i]);
                    first = false;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[u][i] = 0.0f;
            }
        }
        // the element count is a multiple of the group size: a lane past the end shares its group
        // only with other lanes past the end
        for (int off = lanes_per_group >> 1; off > 0; off >>= 1) {
            const float omn = __shfl_xor_sync(0xffffffffu, mn, off), omx = __shfl_xor_sync(0xffffffffu, mx, off);
            mn = fmin_nan(mn, omn); mx = fmax_nan(mx, omx);
        }
        const float r = __fsub_rn(mx, mn);
        float s = __fdiv_rn(r, (float)qmax);
        if (!(s > 0.0f)) s = 1.0f;
        const float inv = __fdiv_rn(1.0f, s);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t e = base + u * 256 + lane * 8;
            uint32_t h0 = 0u, h1 = 0u;
            if (MODE == 0) {
                const uint64_t ctr = (uint64_t)e >> 3;
                hash_2x32_split((uint32_t)ctr, (uint32_t)(ctr >> 32) ^ key_hi, key_lo, h0, h1);
            }
            uint32_t field = 0u;
            for (int c = 0; c < codes_per_piece; ++c) {
                const int i0 = c << log2_a;                              // first element of the sub-group
                float sum = 0.0f;
                for (int k = 0; k < A; ++k) {
                    const float a = __fsub_rn(f[u][i0 + k], mn);
                    const float q = (MODE == 3) ? __fadd_rn(__fmul_rn(a, inv), 0.5f - 1e-6f) : __fdiv_rn(a, s);
                    sum = (k == 0) ? q : __fadd_rn(sum, q);
                }
                const float m = __fmul_rn(sum, inv_a);                   // exact scaling by a power of two
                uint32_t code;
                if (MODE == 3) {
                    int ci = 0;
                    if (m == m) ci = min(max((int)fminf(fmaxf(m, -1.0e9f), 1.0e9f), 0), qmax);
                    code = (uint32_t)ci;
                } else {
                    float uu;
                    if (MODE == 1) uu = ok[u] ? __ldg(noise + e + i0) : 0.0f;
                    else if (MODE == 2) uu = 0.5f - 1e-6f;
                    else uu = __fmul_rn((float)(((i0 < 4 ? h0 : h1) >> ((i0 & 3) * 8)) & 0xFFu), 0x1p-8f);
                    code = code_from_t(__fadd_rn(m, uu), qmax);
                }
                field |= code << (c * bits);
            }
            // lanes_per_word lanes merge their fields: lane j of them holds bits [j*wbits, (j+1)*wbits)
            const int j = lane & (lanes_per_word - 1);
            uint32_t word = (wbits == 32) ? field : (field << (j * wbits));
            for (int off = 1; off < lanes_per_word; off <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, off);
            if (ok[u] && j == 0) packed[(e >> 3) / lanes_per_word] = word;
        }
        const int64_t e0 = base + lane * 8;
        if (e0 < n_elems && (lane & (lanes_per_group - 1)) == 0) {
            const int64_t g = e0 >> log2_gs;
            const bool bf = (flags & ACT_FLAG_META_BF16) != 0;
            scale_out[g] = bf ? round_bf16(s) : s;
            min_out[g] = bf ? round_bf16(mn) : mn;
        }
    }
}

template <int DT>
__global__ void __launch_bounds__(kAvgThreads)
dequant_unpack_avg_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scale,
                          const float* __restrict__ mn, uint8_t* __restrict__ y, int64_t n_elems, int log2_gs,
                          int bits, int log2_a)
{
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kAvgThreads;
    const int codes_per_piece = 8 >> log2_a;
    const int wbits = codes_per_piece * bits;
    const int lanes_per_word = 32 / wbits;
    const uint32_t mask = (1u << bits) - 1u;
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t p = (int64_t)blockIdx.x * kAvgThreads + threadIdx.x; p < n_pieces; p += stride) {
        const int64_t e = p * 8;
        const uint32_t word = __ldg(packed + p / lanes_per_word);
        const uint32_t field = (wbits == 32) ? word : (word >> ((int)(p % lanes_per_word) * wbits));
        const int64_t g = e >> log2_gs;
        const float s = __ldg(scale + g), m = __ldg(mn + g);
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t c = (field >> ((i >> log2_a) * bits)) & mask;
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
static cudaError_t launch_pack_avg_u(const uint8_t* x, const float* noise, uint32_t* packed, float* scale, float* mn,
                                     int64_t n_elems, int log2_gs, int bits, int log2_a, uint32_t klo, uint32_t khi,
                                     int flags, float alpha, cudaStream_t st)
{
    const int u = log2_gs <= 8 ? 1 : (1 << (log2_gs - 8));
    const int64_t warps = (n_elems + 256 * u - 1) / (256 * u);
    const int grid = stream_grid_for((warps + kAvgThreads / 32 - 1) / (kAvgThreads / 32), 4);
    if (u == 1) return launch_overlapped(quant_pack_avg_kernel<DT, MODE, 1>, grid, kAvgThreads, st, x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha);
    if (u == 2) return launch_overlapped(quant_pack_avg_kernel<DT, MODE, 2>, grid, kAvgThreads, st, x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha);
    return launch_overlapped(quant_pack_avg_kernel<DT, MODE, 4>, grid, kAvgThreads, st, x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha);
}

template <int DT>
static cudaError_t launch_pack_avg(int mode, const uint8_t* x, const float* noise, uint32_t* packed, float* scale, float* mn,
                                   int64_t n_elems, int log2_gs, int bits, int log2_a, uint32_t klo, uint32_t khi,
                                   int flags, float alpha, cudaStream_t st)
{
    switch (mode) {
        case 1: return launch_pack_avg_u<DT, 1>(x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha, st);
        case 2: return launch_pack_avg_u<DT, 2>(x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha, st);
        case 3: return launch_pack_avg_u<DT, 3>(x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha, st);
        default: return launch_pack_avg_u<DT, 0>(x, noise, packed, scale, mn, n_elems, log2_gs, bits, log2_a, klo, khi, flags, alpha, st);
    }
}

static bool avg_shape_ok(int group_size, int bits, int avg) {
    if (avg != 2 && avg != 4 && avg != 8) return false;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return false;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return false;
    return (group_size * bits) % (32 * avg) == 0;              // whole words per group
}

}  // namespace act

extern "C" int act_quant_pack_avg(const void* x, int dtype, int64_t n_groups, int group_size, int bits, int avg,
                                  const float* noise, uint64_t seed, uint64_t offset, int flags,
                                  float clamp_alpha, void* packed, float* scale, float* mn, void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (!avg_shape_ok(group_size, bits, avg)) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!x || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)noise) & 15) return ACT_ERR_ALIGN;
    if (((uintptr_t)packed | (uintptr_t)scale | (uintptr_t)mn) & 3) return ACT_ERR_ALIGN;
    int mode;
    if (flags & ACT_FLAG_REF_COMPAT) mode = 3;
    else if (flags & ACT_FLAG_ROUND_NEAREST) mode = 2;
    else if (noise) mode = 1;
    else mode = 0;
    int log2_gs = 5, log2_a = 1;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    while ((1 << log2_a) < avg) ++log2_a;
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const uint32_t klo = (uint32_t)key, khi = (uint32_t)(key >> 32);
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    uint32_t* p = static_cast<uint32_t*>(packed);
    const int64_t n = n_groups * group_size;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_pack_avg<ACT_DTYPE_F32>(mode, xb, noise, p, scale, mn, n, log2_gs, bits, log2_a, klo, khi, flags, clamp_alpha, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_pack_avg<ACT_DTYPE_BF16>(mode, xb, noise, p, scale, mn, n, log2_gs, bits, log2_a, klo, khi, flags, clamp_alpha, st);
    else e = launch_pack_avg<ACT_DTYPE_F16>(mode, xb, noise, p, scale, mn, n, log2_gs, bits, log2_a, klo, khi, flags, clamp_alpha, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_dequant_unpack_avg(const void* packed, const float* scale, const float* mn, int64_t n_groups,
                                      int group_size, int bits, int avg, int out_dtype, void* y, void* stream)
{
    using namespace act;
    if (out_dtype != ACT_DTYPE_F32 && out_dtype != ACT_DTYPE_BF16 && out_dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (!avg_shape_ok(group_size, bits, avg)) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!packed || !scale || !mn || !y) return ACT_ERR_NULL;
    if (((uintptr_t)y & 15) || (((uintptr_t)packed | (uintptr_t)scale | (uintptr_t)mn) & 3)) return ACT_ERR_ALIGN;
    int log2_gs = 5, log2_a = 1;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    while ((1 << log2_a) < avg) ++log2_a;
    const int64_t n = n_groups * group_size;
    const int grid = stream_grid_for(((n >> 3) + kAvgThreads - 1) / kAvgThreads, 6);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t* p = static_cast<const uint32_t*>(packed);
    uint8_t* out = static_cast<uint8_t*>(y);
    cudaError_t e;
    if (out_dtype == ACT_DTYPE_F32) e = launch_overlapped(dequant_unpack_avg_kernel<ACT_DTYPE_F32>, grid, kAvgThreads, st, p, scale, mn, out, n, log2_gs, bits, log2_a);
    else if (out_dtype == ACT_DTYPE_BF16) e = launch_overlapped(dequant_unpack_avg_kernel<ACT_DTYPE_BF16>, grid, kAvgThreads, st, p, scale, mn, out, n, log2_gs, bits, log2_a);
    else e = launch_overlapped(dequant_unpack_avg_kernel<ACT_DTYPE_F16>, grid, kAvgThreads, st, p, scale, mn, out, n, log2_gs, bits, log2_a);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
