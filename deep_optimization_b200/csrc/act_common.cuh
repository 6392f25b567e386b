// Shared device helpers of the activation-compression kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/act_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "this library is written for sm_100a only"
#endif

namespace act {

constexpr int kWarp = 32;
#ifndef ACT_DECODER_WAVES
#define ACT_DECODER_WAVES 4
#endif
// Waves of resident blocks the decoding kernels are launched with (see stream_grid_for in cabi.cu).
constexpr int kDecoderWaves = ACT_DECODER_WAVES;
constexpr int kTileElems = 1024;          // elements one warp handles per iteration
constexpr uint32_t kMagicBits = 0x4B000000u;   // bit pattern of 2^23
constexpr float kMagic = 8388608.0f;           // 2^23
constexpr uint32_t kHashMul = 0xD256D193u;
constexpr uint32_t kHashWeyl = 0x9E3779B9u;
constexpr int kHashRounds = 4;

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// streaming variant: the line is not kept in L1 once consumed
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void stg_stream_v4(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Programmatic dependent launch.  A kernel started with launch_overlapped() may become
// resident while the kernel before it in the stream is still draining; it must call
// grid_dependency_wait() before its first global access (the wait returns once the earlier
// grid has completed and its writes are visible; without the launch attribute it is a no-op),
// and it lets its own successor in with grid_launch_dependents().
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifndef ACT_NO_PDL
#define ACT_NO_PDL 0
#endif
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), int grid, int block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ACT_NO_PDL ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// NaN-propagating fp32 min/max; -0 orders below +0
__device__ __forceinline__ float fmin_nan(float a, float b) {
    float d; asm("min.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d;
}
__device__ __forceinline__ float fmax_nan(float a, float b) {
    float d; asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b)); return d;
}
// three inputs in one instruction (sm_100)
__device__ __forceinline__ float fmin3_nan(float a, float b, float c) {
    float d; asm("min.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d;
}
__device__ __forceinline__ float fmax3_nan(float a, float b, float c) {
    float d; asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d;
}

// Host side: splitmix64 finaliser; the hash key is hash_key(hash_key(seed) + offset).
__host__ __device__ inline uint64_t hash_key(uint64_t seed) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Four rounds of a 2x32 multiply-xor network: 64 output bits per 64-bit counter,
// the counter already split and key_hi folded into ctr_hi
__device__ __forceinline__ void hash_2x32_split(uint32_t ctr_lo, uint32_t ctr_hi_x_key, uint32_t key_lo,
                                                uint32_t& o0, uint32_t& o1) {
    uint32_t L = ctr_lo, R = ctr_hi_x_key, k = key_lo;
#pragma unroll
    for (int r = 0; r < kHashRounds; ++r) {
        const uint64_t p = (uint64_t)kHashMul * (uint64_t)L;
        L = (uint32_t)(p >> 32) ^ k ^ R;
        R = (uint32_t)p;
        k += kHashWeyl;
    }
    o0 = L; o1 = R;
}

// ---- packed fp32 pairs (sm_100 f32x2 instructions: one issue slot, two lanes) ----
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r;
}
__device__ __forceinline__ f32x2 pack2u(uint32_t a, uint32_t b) {
    f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b)); return r;
}
__device__ __forceinline__ void unpack2u(f32x2 v, uint32_t& a, uint32_t& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 add2_rn(f32x2 a, f32x2 b) {
    f32x2 d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d;
}
__device__ __forceinline__ f32x2 add2_rm(f32x2 a, f32x2 b) {
    f32x2 d; asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d;
}
__device__ __forceinline__ f32x2 sub2_rn(f32x2 a, f32x2 b) {
    f32x2 d; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d;
}
__device__ __forceinline__ f32x2 mul2_rn(f32x2 a, f32x2 b) {
    f32x2 d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d;
}
__device__ __forceinline__ f32x2 fma2_rn(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d;
}
// the same division sequence as div_by_scale on two lanes; ns = (-s,-s), y = (1/s,1/s)
__device__ __forceinline__ f32x2 div_by_scale2(f32x2 a, f32x2 ns, f32x2 y) {
    f32x2 q = mul2_rn(a, y);
    f32x2 r = fma2_rn(ns, q, a);
    q = fma2_rn(r, y, q);
    r = fma2_rn(ns, q, a);
    q = fma2_rn(r, y, q);
    return q;
}

// a / s, correctly rounded, from y = RN(1/s): two Newton corrections on the
// quotient with exact FMA residuals.  Valid while nothing under- or overflows;
// callers keep s inside [2^-60, 2^60].
__device__ __forceinline__ float div_by_scale(float a, float s, float y) {
    float q = __fmul_rn(a, y);
    float r = __fmaf_rn(-s, q, a);
    q = __fmaf_rn(r, y, q);
    r = __fmaf_rn(-s, q, a);
    q = __fmaf_rn(r, y, q);
    return q;
}

// clamp(floor(t), 0, qmax) with NaN -> 0, the general (slow) form
__device__ __forceinline__ uint32_t code_from_t(float t, int qmax) {
    if (!(t >= 0.0f)) return 0u;
    if (t >= (float)(qmax + 1)) return (uint32_t)qmax;
    return (uint32_t)floorf(t);
}

template <int DT> struct ElemT;
template <> struct ElemT<ACT_DTYPE_F32>  { static constexpr int bytes = 4; };
template <> struct ElemT<ACT_DTYPE_BF16> { static constexpr int bytes = 2; };
template <> struct ElemT<ACT_DTYPE_F16>  { static constexpr int bytes = 2; };

// widen the two 16-bit halves of a packed register to fp32 (exact)
template <int DT> __device__ __forceinline__ float widen_lo(uint32_t v);
template <int DT> __device__ __forceinline__ float widen_hi(uint32_t v);
template <> __device__ __forceinline__ float widen_lo<ACT_DTYPE_BF16>(uint32_t v) { return __uint_as_float(v << 16); }
template <> __device__ __forceinline__ float widen_hi<ACT_DTYPE_BF16>(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
template <> __device__ __forceinline__ float widen_lo<ACT_DTYPE_F16>(uint32_t v) {
    return __half2float(__ushort_as_half((unsigned short)(v & 0xFFFFu)));
}
template <> __device__ __forceinline__ float widen_hi<ACT_DTYPE_F16>(uint32_t v) {
    return __half2float(__ushort_as_half((unsigned short)(v >> 16)));
}

}  // namespace act
