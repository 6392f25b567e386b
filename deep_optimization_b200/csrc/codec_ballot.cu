// The legacy codec of the reference's C++ extension, kept for callers of its
// pack_mixed_precision_cuda / unpack_mixed_precision_cuda
// (Activation_Compression/cpp_extension/src/quantization_cuda_kernels.cu:15-298) and of its
// debug copy (cpp_extension/src/copy.cu:50-102):
//   * caller-supplied per-group min and max, scale = (2^b - 1) / (max - min + 2e-6) computed in
//     the data's own type;
//   * stochastic rounding with the reference's index hash sgd_noise
//     (cpp_extension/include/quant_common.h:32-43), key = (element index << 32) ^ seed;
//   * bit-plane layout in warp-ballot order: 32 consecutive elements are one chunk, its b words
//     follow one another, bit `lane` of word p = bit p of the code of element `lane`;
//   * decode = code / scale + min.
// The reference launches one CTA per group with one thread per element and lets lane 0 store
// every word.  Here a warp walks chunks with a grid stride: one coalesced load of 32 elements,
// b ballots, and lanes 0..b-1 store the chunk's b words as one contiguous piece.
// Every floating-point operation is rounded on its own (the build disables contraction), which
// the CPU oracle restates; 16-bit types round the scale arithmetic to their own type after each
// operation, as the reference's scalar types do.  Correctness-tested, not tuned.
#include "act_common.cuh"

namespace act {
namespace ballot {

__device__ __forceinline__ float sgd_noise(uint64_t x) {
    x ^= x >> 32;
    x *= 0xD6E8FEB86659FD93ull;
    x ^= x >> 32;
    const float u = __fmul_rn((float)(x >> 40), 1.0f / 16777216.0f);
    return __fsub_rn(u, 0.5f);
}

template <int DT> struct Io;
template <> struct Io<ACT_DTYPE_F32> {
    typedef float T;
    static __device__ __forceinline__ float load(const T* p, int64_t i) { return __ldg(p + i); }
    static __device__ __forceinline__ void store(T* p, int64_t i, float v) { p[i] = v; }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct Io<ACT_DTYPE_BF16> {
    typedef __nv_bfloat16 T;
    static __device__ __forceinline__ float load(const T* p, int64_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void store(T* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct Io<ACT_DTYPE_F16> {
    typedef __half T;
    static __device__ __forceinline__ float load(const T* p, int64_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ void store(T* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};

template <int DT>
__global__ void __launch_bounds__(256)
pack_ballot_kernel(const typename Io<DT>::T* __restrict__ x, const typename Io<DT>::T* __restrict__ mn,
                   const typename Io<DT>::T* __restrict__ mx, uint32_t* __restrict__ packed,
                   typename Io<DT>::T* __restrict__ scale, int64_t n_chunks, int chunks_per_group, int bits,
                   uint64_t seed, int ref_bias)
{
    typedef Io<DT> IO;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const float qmax = (float)((1 << bits) - 1);
    for (int64_t c = warp0; c < n_chunks; c += n_warps) {
        const int64_t g = c / chunks_per_group;
        const float m = IO::load(mn, g);
        float denom = IO::round(__fsub_rn(IO::load(mx, g), m));
        denom = IO::round(__fadd_rn(denom, IO::round(2e-6f)));
        const float sc = IO::round(__fdiv_rn(qmax, denom));
        if (lane == 0 && c == g * chunks_per_group) IO::store(scale, g, sc);
        const int64_t id = c * 32 + lane;
        const float noise = sgd_noise(((uint64_t)id << 32) ^ seed);
        float t = __fadd_rn(__fmul_rn(__fsub_rn(IO::load(x, id), m), sc), noise);
        if (ref_bias) t = __fsub_rn(t, 0.5f);
        float q = rintf(t > 0.0f ? t : 0.0f);                 // NaN compares false: code 0
        if (!(q <= qmax)) q = qmax;
        const uint32_t code = (uint32_t)q;
        uint32_t mine = 0;
        for (int p = 0; p < bits; ++p) {
            const uint32_t w = __ballot_sync(0xffffffffu, (code >> p) & 1u);
            if (lane == p) mine = w;
        }
        if (lane < bits) packed[c * bits + lane] = mine;
    }
}

template <int DT>
__global__ void __launch_bounds__(256)
unpack_ballot_kernel(const uint32_t* __restrict__ packed, const typename Io<DT>::T* __restrict__ scale,
                     const typename Io<DT>::T* __restrict__ mn, typename Io<DT>::T* __restrict__ y,
                     int64_t n_chunks, int chunks_per_group, int bits)
{
    typedef Io<DT> IO;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t c = warp0; c < n_chunks; c += n_warps) {
        const int64_t g = c / chunks_per_group;
        const float sc = IO::load(scale, g), m = IO::load(mn, g);
        const uint32_t w = lane < bits ? __ldg(packed + c * bits + lane) : 0u;
        uint32_t code = 0;
        for (int p = 0; p < bits; ++p) code |= ((__shfl_sync(0xffffffffu, w, p) >> lane) & 1u) << p;
        IO::store(y, c * 32 + lane, __fadd_rn(__fdiv_rn((float)code, sc), m));
    }
}

// bounds-checked identity copy: 16-byte pieces, then the byte tail
__global__ void __launch_bounds__(256)
copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, size_t nbytes)
{
    const size_t n16 = nbytes >> 4;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < n16; i += nth)
        reinterpret_cast<uint4*>(dst)[i] = ldg_stream_v4(reinterpret_cast<const uint4*>(src) + i);
    for (size_t i = (n16 << 4) + tid; i < nbytes; i += nth) dst[i] = src[i];
}

inline int grid_for(int64_t warps_needed) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t blocks = (warps_needed + 7) / 8;
    const int64_t cap = (int64_t)sms * 8;                     // one wave of 256-thread blocks
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace ballot
}  // namespace act

static int ballot_args_ok(int dtype, int64_t n_groups, int group_size, int bits) {
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (bits < 1 || bits > 8) return ACT_ERR_BITS;
    if (group_size < 32 || (group_size & 31) || group_size > 65536) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 17)) return ACT_ERR_SIZE;
    return ACT_OK;
}

extern "C" int act_pack_ballot(const void* x, int dtype, int64_t n_groups, int group_size, int bits,
                               const void* mn, const void* mx, uint64_t seed, int flags,
                               void* packed, void* scale, void* stream)
{
    using namespace act::ballot;
    const int rc = ballot_args_ok(dtype, n_groups, group_size, bits);
    if (rc != ACT_OK) return rc;
    if (flags & ~ACT_FLAG_BALLOT_REF_BIAS) return ACT_ERR_UNSUPPORTED;
    if (n_groups == 0) return ACT_OK;
    if (!x || !mn || !mx || !packed || !scale) return ACT_ERR_NULL;
    if ((uintptr_t)packed & 3) return ACT_ERR_ALIGN;
    const int cpg = group_size / 32;
    const int64_t n_chunks = n_groups * cpg;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = grid_for(n_chunks);
    const int bias = (flags & ACT_FLAG_BALLOT_REF_BIAS) ? 1 : 0;
    uint32_t* out = static_cast<uint32_t*>(packed);
    if (dtype == ACT_DTYPE_F32)
        pack_ballot_kernel<ACT_DTYPE_F32><<<grid, 256, 0, st>>>((const float*)x, (const float*)mn, (const float*)mx, out,
                                                                (float*)scale, n_chunks, cpg, bits, seed, bias);
    else if (dtype == ACT_DTYPE_BF16)
        pack_ballot_kernel<ACT_DTYPE_BF16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)mn,
                                                                 (const __nv_bfloat16*)mx, out, (__nv_bfloat16*)scale,
                                                                 n_chunks, cpg, bits, seed, bias);
    else
        pack_ballot_kernel<ACT_DTYPE_F16><<<grid, 256, 0, st>>>((const __half*)x, (const __half*)mn, (const __half*)mx, out,
                                                                (__half*)scale, n_chunks, cpg, bits, seed, bias);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_unpack_ballot(const void* packed, const void* scale, const void* mn, int dtype,
                                 int64_t n_groups, int group_size, int bits, void* y, void* stream)
{
    using namespace act::ballot;
    const int rc = ballot_args_ok(dtype, n_groups, group_size, bits);
    if (rc != ACT_OK) return rc;
    if (n_groups == 0) return ACT_OK;
    if (!packed || !scale || !mn || !y) return ACT_ERR_NULL;
    if ((uintptr_t)packed & 3) return ACT_ERR_ALIGN;
    const int cpg = group_size / 32;
    const int64_t n_chunks = n_groups * cpg;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = grid_for(n_chunks);
    const uint32_t* in = static_cast<const uint32_t*>(packed);
    if (dtype == ACT_DTYPE_F32)
        unpack_ballot_kernel<ACT_DTYPE_F32><<<grid, 256, 0, st>>>(in, (const float*)scale, (const float*)mn, (float*)y,
                                                                  n_chunks, cpg, bits);
    else if (dtype == ACT_DTYPE_BF16)
        unpack_ballot_kernel<ACT_DTYPE_BF16><<<grid, 256, 0, st>>>(in, (const __nv_bfloat16*)scale, (const __nv_bfloat16*)mn,
                                                                   (__nv_bfloat16*)y, n_chunks, cpg, bits);
    else
        unpack_ballot_kernel<ACT_DTYPE_F16><<<grid, 256, 0, st>>>(in, (const __half*)scale, (const __half*)mn, (__half*)y,
                                                                  n_chunks, cpg, bits);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_copy(const void* src, void* dst, size_t nbytes, size_t src_capacity, size_t dst_capacity, void* stream)
{
    using namespace act::ballot;
    if (nbytes == 0) return ACT_OK;
    if (!src || !dst) return ACT_ERR_NULL;
    if (nbytes > src_capacity || nbytes > dst_capacity) return ACT_ERR_SIZE;     // the bounds check the reference's copy lacks
    if (((uintptr_t)src | (uintptr_t)dst) & 15) return ACT_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    copy_kernel<<<grid_for((int64_t)((nbytes >> 4) / 32 + 1)), 256, 0, st>>>(static_cast<const uint8_t*>(src),
                                                                             static_cast<uint8_t*>(dst), nbytes);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
