// Producer/consumer-fused codec kernels for activations, sm_100a.
//
//   relu_fwd_pack:    y = x > 0 ? x : 0 (or the ReLU6 window) and the 1-bit mask, one pass
//   relu_bwd_unpack:  dx = mask ? dy : 0, one pass
//   act_bwd_dequant:  dx = dy * (code * scale + min), the backward of GELU / SiLU whose
//                     quantised derivative was saved in forward
//
// They remove the extra passes a stand-alone codec costs: the int8 mask the reference's
// unfused path writes and reads back, and the dequantised derivative tensor.
// All three are streaming kernels: a warp takes 1024 elements as four chunks, a lane owns
// 8 consecutive elements per chunk, every load and store instruction is contiguous.
//
// Replaces: Activation_Compression/modules/activations/kernel_implementation.py:34-143
// (relu_variance_fwd_fused_pack_kernel, relu_bwd_fused_unpack_kernel) and :345-424, :562-618
// (silu/gelu_bwd_fused_dequan_unpack_triton).
#include "act_common.cuh"

namespace act {

constexpr int kFusedThreads = 256;

template <int DT> struct Vec8 {          // 8 consecutive elements of a lane
    uint4 a, b;                          // b only for fp32
};
template <int DT> __device__ __forceinline__ Vec8<DT> load8(const uint8_t* p, int64_t e) {
    Vec8<DT> v;
    if (ElemT<DT>::bytes == 4) { v.a = ldg_nc_v4(p + e * 4); v.b = ldg_nc_v4(p + e * 4 + 16); }
    else { v.a = ldg_nc_v4(p + e * 2); v.b = make_uint4(0, 0, 0, 0); }
    return v;
}
template <int DT> __device__ __forceinline__ void to_float8(const Vec8<DT>& v, float (&f)[8]) {
    if (ElemT<DT>::bytes == 4) {
        f[0] = __uint_as_float(v.a.x); f[1] = __uint_as_float(v.a.y); f[2] = __uint_as_float(v.a.z); f[3] = __uint_as_float(v.a.w);
        f[4] = __uint_as_float(v.b.x); f[5] = __uint_as_float(v.b.y); f[6] = __uint_as_float(v.b.z); f[7] = __uint_as_float(v.b.w);
    } else {
        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
        f[0] = widen_lo<D16>(v.a.x); f[1] = widen_hi<D16>(v.a.x); f[2] = widen_lo<D16>(v.a.y); f[3] = widen_hi<D16>(v.a.y);
        f[4] = widen_lo<D16>(v.a.z); f[5] = widen_hi<D16>(v.a.z); f[6] = widen_lo<D16>(v.a.w); f[7] = widen_hi<D16>(v.a.w);
    }
}
template <int DT> __device__ __forceinline__ void store8(uint8_t* p, int64_t e, const float (&f)[8]) {
    if (DT == ACT_DTYPE_F32) {
        stg_stream_v4(p + e * 4, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
        stg_stream_v4(p + e * 4 + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
    } else {
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (DT == ACT_DTYPE_BF16) { const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
            else { const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
        }
        stg_stream_v4(p + e * 2, make_uint4(o[0], o[1], o[2], o[3]));
    }
}

// ---- ReLU forward: y and one mask bit per element (bit i of byte e/8 = element e) -----
template <int DT>
__global__ void __launch_bounds__(kFusedThreads)
relu_fwd_pack_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, uint8_t* __restrict__ bits,
                     int64_t n_elems, int relu6)
{
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kFusedThreads;
    for (int64_t p0 = (int64_t)blockIdx.x * kFusedThreads + threadIdx.x; p0 < n_pieces; p0 += stride * 4) {
        Vec8<DT> v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) if (p0 + k * stride < n_pieces) v[k] = load8<DT>(x, (p0 + k * stride) * 8);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t p = p0 + k * stride;
            if (p >= n_pieces) break;
            float f[8];
            to_float8<DT>(v[k], f);
            uint32_t m = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool keep = relu6 ? (f[i] > 0.0f && f[i] < 6.0f) : (f[i] > 0.0f);
                m |= (uint32_t)keep << i;
                f[i] = keep ? f[i] : 0.0f;
            }
            store8<DT>(y, p * 8, f);
            bits[p] = (uint8_t)m;
        }
    }
}

// ---- ReLU backward: dx = mask ? dy : 0 ----------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kFusedThreads)
relu_bwd_unpack_kernel(const uint8_t* __restrict__ bits, const uint8_t* __restrict__ dy,
                       const uint8_t* __restrict__ dy2, uint8_t* __restrict__ dx, int64_t n_elems)
{
    // dy2 (optional): a second gradient of the same tensor, added in fp32 before the mask: where
    // the tensor has two consumers this pass takes the place of autograd's accumulation as well
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kFusedThreads;
    for (int64_t p0 = (int64_t)blockIdx.x * kFusedThreads + threadIdx.x; p0 < n_pieces; p0 += stride * 4) {
        Vec8<DT> v[4], v2[4];
        uint32_t m[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) if (p0 + k * stride < n_pieces) {
            v[k] = load8<DT>(dy, (p0 + k * stride) * 8);
            if (dy2) v2[k] = load8<DT>(dy2, (p0 + k * stride) * 8);
            m[k] = __ldg(bits + p0 + k * stride);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t p = p0 + k * stride;
            if (p >= n_pieces) break;
            float f[8];
            to_float8<DT>(v[k], f);
            if (dy2) {
                float f2[8];
                to_float8<DT>(v2[k], f2);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __fadd_rn(f[i], f2[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = ((m[k] >> i) & 1u) ? f[i] : 0.0f;
            store8<DT>(dx, p * 8, f);
        }
    }
}

// ---- backward of an activation whose quantised derivative was saved: dx = dy * deq ------
template <int DT, int BITS>
__global__ void __launch_bounds__(kFusedThreads)
act_bwd_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                       const float* __restrict__ mn, const uint8_t* __restrict__ dy,
                       uint8_t* __restrict__ dx, int64_t n_elems, int log2_gs)
{
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kFusedThreads;
    for (int64_t p0 = (int64_t)blockIdx.x * kFusedThreads + threadIdx.x; p0 < n_pieces; p0 += stride * 2) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int64_t p = p0 + k * stride;
            if (p >= n_pieces) break;
            const Vec8<DT> v = load8<DT>(dy, p * 8);
            uint32_t w0, w1 = 0;
            if (BITS == 8) { const uint2 t = __ldg(reinterpret_cast<const uint2*>(packed + p * 8)); w0 = t.x; w1 = t.y; }
            else if (BITS == 4) w0 = __ldg(reinterpret_cast<const uint32_t*>(packed + p * 4));
            else if (BITS == 2) w0 = __ldg(reinterpret_cast<const uint16_t*>(packed + p * 2));
            else w0 = __ldg(packed + p);
            const int64_t g = (p * 8) >> log2_gs;
            const float s = __ldg(scale + g), m = __ldg(mn + g);
            float f[8];
            to_float8<DT>(v, f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t c = (BITS == 8) ? (((i < 4 ? w0 : w1) >> ((i & 3) * 8)) & MASK) : ((w0 >> (i * BITS)) & MASK);
                const float cf = __uint_as_float(kMagicBits | c) - kMagic;
                f[i] = __fmul_rn(f[i], __fmaf_rn(cf, s, m));          // dy * (code*scale + min)
            }
            store8<DT>(dx, p * 8, f);
        }
    }
}

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves = 1);   // cabi.cu

static bool dtype_ok(int d) { return d == ACT_DTYPE_F32 || d == ACT_DTYPE_BF16 || d == ACT_DTYPE_F16; }

}  // namespace act

extern "C" int act_relu_fwd_pack(const void* x, int dtype, int64_t n_elems, int relu6, void* y,
                                 void* mask_bits, void* stream)
{
    using namespace act;
    if (!dtype_ok(dtype)) return ACT_ERR_DTYPE;
    if (n_elems < 0 || (n_elems & 31)) return ACT_ERR_SIZE;
    if (n_elems == 0) return ACT_OK;
    if (!x || !y || !mask_bits) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y) & 15 || ((uintptr_t)mask_bits & 3)) return ACT_ERR_ALIGN;
    const int grid = stream_grid_for(((n_elems >> 3) + kFusedThreads * 4 - 1) / (kFusedThreads * 4), 6, kDecoderWaves);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* xi = static_cast<const uint8_t*>(x);
    uint8_t* yo = static_cast<uint8_t*>(y);
    uint8_t* bo = static_cast<uint8_t*>(mask_bits);
    if (dtype == ACT_DTYPE_F32) relu_fwd_pack_kernel<ACT_DTYPE_F32><<<grid, kFusedThreads, 0, st>>>(xi, yo, bo, n_elems, relu6);
    else if (dtype == ACT_DTYPE_BF16) relu_fwd_pack_kernel<ACT_DTYPE_BF16><<<grid, kFusedThreads, 0, st>>>(xi, yo, bo, n_elems, relu6);
    else relu_fwd_pack_kernel<ACT_DTYPE_F16><<<grid, kFusedThreads, 0, st>>>(xi, yo, bo, n_elems, relu6);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_relu_bwd_unpack_sum(const void* mask_bits, const void* dy, const void* dy2, int dtype,
                                       int64_t n_elems, void* dx, void* stream)
{
    using namespace act;
    if (!dtype_ok(dtype)) return ACT_ERR_DTYPE;
    if (n_elems < 0 || (n_elems & 31)) return ACT_ERR_SIZE;
    if (n_elems == 0) return ACT_OK;
    if (!dy || !dx || !mask_bits) return ACT_ERR_NULL;
    if (((uintptr_t)dy | (uintptr_t)dy2 | (uintptr_t)dx) & 15) return ACT_ERR_ALIGN;
    const int grid = stream_grid_for(((n_elems >> 3) + kFusedThreads * 4 - 1) / (kFusedThreads * 4), 6, kDecoderWaves);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* b = static_cast<const uint8_t*>(mask_bits);
    const uint8_t* g = static_cast<const uint8_t*>(dy);
    const uint8_t* g2 = static_cast<const uint8_t*>(dy2);
    uint8_t* o = static_cast<uint8_t*>(dx);
    if (dtype == ACT_DTYPE_F32) relu_bwd_unpack_kernel<ACT_DTYPE_F32><<<grid, kFusedThreads, 0, st>>>(b, g, g2, o, n_elems);
    else if (dtype == ACT_DTYPE_BF16) relu_bwd_unpack_kernel<ACT_DTYPE_BF16><<<grid, kFusedThreads, 0, st>>>(b, g, g2, o, n_elems);
    else relu_bwd_unpack_kernel<ACT_DTYPE_F16><<<grid, kFusedThreads, 0, st>>>(b, g, g2, o, n_elems);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_relu_bwd_unpack(const void* mask_bits, const void* dy, int dtype, int64_t n_elems,
                                   void* dx, void* stream)
{
    return act_relu_bwd_unpack_sum(mask_bits, dy, nullptr, dtype, n_elems, dx, stream);
}

namespace act {
template <int DT>
static void launch_act_bwd(int bits, const uint8_t* p, const float* s, const float* m, const uint8_t* dy,
                           uint8_t* dx, int64_t n, int log2_gs, int grid, cudaStream_t st)
{
    switch (bits) {
        case 1: act_bwd_dequant_kernel<DT, 1><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, dx, n, log2_gs); break;
        case 2: act_bwd_dequant_kernel<DT, 2><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, dx, n, log2_gs); break;
        case 4: act_bwd_dequant_kernel<DT, 4><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, dx, n, log2_gs); break;
        default: act_bwd_dequant_kernel<DT, 8><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, dx, n, log2_gs); break;
    }
}
}  // namespace act

extern "C" int act_mul_dequant_unpack(const void* packed, const float* scale, const float* mn,
                                      const void* dy, int dtype, int64_t n_groups, int group_size,
                                      int bits, void* dx, void* stream)
{
    using namespace act;
    if (!dtype_ok(dtype)) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!packed || !scale || !mn || !dy || !dx) return ACT_ERR_NULL;
    if (((uintptr_t)dy | (uintptr_t)dx) & 15 || ((uintptr_t)packed & 7)) return ACT_ERR_ALIGN;
    int log2_gs = 5;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    const int64_t n = n_groups * group_size;
    const int grid = stream_grid_for(((n >> 3) + kFusedThreads * 2 - 1) / (kFusedThreads * 2), 6, kDecoderWaves);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    const uint8_t* g = static_cast<const uint8_t*>(dy);
    uint8_t* o = static_cast<uint8_t*>(dx);
    if (dtype == ACT_DTYPE_F32) launch_act_bwd<ACT_DTYPE_F32>(bits, p, scale, mn, g, o, n, log2_gs, grid, st);
    else if (dtype == ACT_DTYPE_BF16) launch_act_bwd<ACT_DTYPE_BF16>(bits, p, scale, mn, g, o, n, log2_gs, grid, st);
    else launch_act_bwd<ACT_DTYPE_F16>(bits, p, scale, mn, g, o, n, log2_gs, grid, st);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

// =========================================================================================
// Batch-norm backward from the packed x_hat (flat sample-major groups of [N, C, HW]):
//   act_bn_bwd_reduce:  sums[c] += sum dy * x_hat,  sums[C + c] += sum dy
//   act_bn_bwd_dx:      dx = k1[c] * dy - k2[c] - k3[c] * x_hat     (coef[c] = (k1, k2, k3, -))
// Replace bn_bwd_reduce_dequant_unpack_fused / bn_bwd_dx_dequant_unpack_fused
// (Activation_Compression/modules/normalization/kernel_implementation.py:328-481): the
// decoded x_hat never goes to memory.  A thread walks pieces of 8 elements with a fixed
// stride and tracks (channel, offset in the HW plane) incrementally, so the only division
// is the one that places its first piece.  HW is a multiple of 4, hence four consecutive
// elements share a channel.
// =========================================================================================
namespace act {

struct PlaneWalk {           // position of a piece inside [N, C, HW] and the step to the next
    uint32_t c, r;           // channel, offset inside the plane
    uint32_t dc, dr;         // channel and offset advance per step (dr < hw, dc < C)
    uint32_t hw, C;
    __device__ __forceinline__ void init(int64_t e, int64_t step_e, uint32_t hw_, uint32_t C_) {
        hw = hw_; C = C_;
        const uint64_t plane = (uint64_t)e / hw;
        r = (uint32_t)((uint64_t)e - plane * hw);
        c = (uint32_t)(plane % C);
        const uint64_t dplane = (uint64_t)step_e / hw;
        dr = (uint32_t)((uint64_t)step_e - dplane * hw);
        dc = (uint32_t)(dplane % C);
    }
    __device__ __forceinline__ void advance() {
        r += dr; c += dc;
        if (r >= hw) { r -= hw; c += 1; }
        if (c >= C) c -= C;
        if (c >= C) c -= C;
    }
    // channel of the element `off` (< 8, multiple of 4) after the piece's first
    __device__ __forceinline__ uint32_t channel_at(uint32_t off) const {
        uint32_t cc = c;
        if (r + off >= hw) { cc += 1; if (cc >= C) cc -= C; }
        return cc;
    }
};

template <int BITS> __device__ __forceinline__ uint2 load_codes8(const uint8_t* packed, int64_t p) {
    if (BITS == 8) return __ldg(reinterpret_cast<const uint2*>(packed + p * 8));
    if (BITS == 4) return make_uint2(__ldg(reinterpret_cast<const uint32_t*>(packed + p * 4)), 0u);
    if (BITS == 2) return make_uint2(__ldg(reinterpret_cast<const uint16_t*>(packed + p * 2)), 0u);
    return make_uint2(__ldg(packed + p), 0u);
}
template <int BITS> __device__ __forceinline__ float decode_at(uint2 w, int i, float s, float m) {
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const uint32_t c = (BITS == 8) ? (((i < 4 ? w.x : w.y) >> ((i & 3) * 8)) & MASK) : ((w.x >> (i * BITS)) & MASK);
    return __fmaf_rn(__uint_as_float(kMagicBits | c) - kMagic, s, m);
}

template <int DT, int BITS>
__global__ void __launch_bounds__(kFusedThreads)
bn_bwd_dx_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                 const float* __restrict__ mn, const uint8_t* __restrict__ dy, const uint8_t* __restrict__ mask,
                 const float4* __restrict__ coef, uint8_t* __restrict__ dx, int64_t n_elems, int log2_gs, uint32_t hw, uint32_t C)
{
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kFusedThreads;
    int64_t p = (int64_t)blockIdx.x * kFusedThreads + threadIdx.x;
    if (p >= n_pieces) return;
    // two pieces per trip (p and p + stride), the loads of both issued before either is used:
    // with one piece per trip the kernel waited on its loads (13 stall cycles per issue on the
    // long scoreboard); each piece has its own walker, stepping two strides at a time
    PlaneWalk walk0, walk1;
    walk0.init(p * 8, stride * 16, hw, C);
    walk1.init((p + stride) * 8, stride * 16, hw, C);
    auto finish = [&](int64_t q, const Vec8<DT>& v, uint2 w, float s, float m, uint32_t keep, float4 k0, float4 k1) {
        float f[8];
        to_float8<DT>(v, f);
        if (mask) {                                   // fused ReLU: dy counts only where y was positive
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = ((keep >> i) & 1u) ? f[i] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 k = i < 4 ? k0 : k1;
            f[i] = __fmaf_rn(-k.z, decode_at<BITS>(w, i, s, m), __fmaf_rn(k.x, f[i], -k.y));
        }
        store8<DT>(dx, q * 8, f);
    };
    for (; p < n_pieces; p += 2 * stride, walk0.advance(), walk1.advance()) {
        const int64_t p1 = p + stride;
        const bool two = p1 < n_pieces;
        const int64_t q1 = two ? p1 : p;
        const Vec8<DT> v0 = load8<DT>(dy, p * 8), v1 = load8<DT>(dy, q1 * 8);
        const uint2 w0 = load_codes8<BITS>(packed, p), w1 = load_codes8<BITS>(packed, q1);
        const int64_t g0 = (p * 8) >> log2_gs, g1 = (q1 * 8) >> log2_gs;
        const float s0 = __ldg(scale + g0), m0 = __ldg(mn + g0), s1 = __ldg(scale + g1), m1 = __ldg(mn + g1);
        const float4 a0 = __ldg(coef + walk0.c), a1 = __ldg(coef + walk0.channel_at(4));
        const float4 b0 = __ldg(coef + (two ? walk1.c : walk0.c)), b1 = __ldg(coef + (two ? walk1.channel_at(4) : walk0.c));
        const uint32_t keep0 = mask ? __ldg(mask + p) : 0xFFu, keep1 = mask ? __ldg(mask + q1) : 0xFFu;
        finish(p, v0, w0, s0, m0, keep0, a0, a1);
        if (two) finish(p1, v1, w1, s1, m1, keep1, b0, b1);
    }
}

// The same for the channel-minor layout (HW = 1: dy is [rows, C], C a multiple of 8): the
// eight elements of a piece belong to channels c..c+7 with c = (8 p) % C.  When the grid
// stride is a multiple of C (every power-of-two C up to 2048 pieces' worth) a thread meets
// the same eight channels in every step and keeps their constants in registers.
template <int DT, int BITS>
__global__ void __launch_bounds__(kFusedThreads)
bn_bwd_dx_cl_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                    const float* __restrict__ mn, const uint8_t* __restrict__ dy, const uint8_t* __restrict__ mask,
                    const float4* __restrict__ coef, uint8_t* __restrict__ dx, int64_t n_elems, int log2_gs, uint32_t C)
{
    const int64_t n_pieces = n_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * kFusedThreads;
    int64_t p = (int64_t)blockIdx.x * kFusedThreads + threadIdx.x;
    if (p >= n_pieces) return;
    uint32_t c = (uint32_t)((uint64_t)(p * 8) % C);
    const uint32_t dc = (uint32_t)((uint64_t)(stride * 8) % C);
    float4 k[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) k[i] = __ldg(coef + c + i);
    auto finish = [&](int64_t q, const Vec8<DT>& v, uint2 w, float s, float m, uint32_t keep) {
        float f[8];
        to_float8<DT>(v, f);
        if (mask) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = ((keep >> i) & 1u) ? f[i] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
            f[i] = __fmaf_rn(-k[i].z, decode_at<BITS>(w, i, s, m), __fmaf_rn(k[i].x, f[i], -k[i].y));
        store8<DT>(dx, q * 8, f);
    };
    if (dc == 0) {
        // two pieces per trip, both sets of loads issued before either is used
        for (; p < n_pieces; p += 2 * stride) {
            const int64_t p1 = p + stride;
            const bool two = p1 < n_pieces;
            const int64_t q1 = two ? p1 : p;
            const Vec8<DT> v0 = load8<DT>(dy, p * 8), v1 = load8<DT>(dy, q1 * 8);
            const uint2 w0 = load_codes8<BITS>(packed, p), w1 = load_codes8<BITS>(packed, q1);
            const int64_t g0 = (p * 8) >> log2_gs, g1 = (q1 * 8) >> log2_gs;
            const float s0 = __ldg(scale + g0), m0 = __ldg(mn + g0), s1 = __ldg(scale + g1), m1 = __ldg(mn + g1);
            const uint32_t keep0 = mask ? __ldg(mask + p) : 0xFFu, keep1 = mask ? __ldg(mask + q1) : 0xFFu;
            finish(p, v0, w0, s0, m0, keep0);
            if (two) finish(p1, v1, w1, s1, m1, keep1);
        }
        return;
    }
    for (; p < n_pieces; p += stride) {
        const Vec8<DT> v = load8<DT>(dy, p * 8);
        const uint2 w = load_codes8<BITS>(packed, p);
        const int64_t g = (p * 8) >> log2_gs;
        const float s = __ldg(scale + g), m = __ldg(mn + g);
        finish(p, v, w, s, m, mask ? __ldg(mask + p) : 0xFFu);
        c += dc;
        if (c >= C) c -= C;
#pragma unroll
        for (int i = 0; i < 8; ++i) k[i] = __ldg(coef + c + i);
    }
}

template <int DT>
static cudaError_t launch_bn_bwd_dx(int bits, const uint8_t* p, const float* s, const float* m,
                                    const uint8_t* dy, const uint8_t* mask, const float4* coef, uint8_t* dx, int64_t n,
                                    int log2_gs, uint32_t hw, uint32_t C, cudaStream_t st)
{
    const int grid = stream_grid_for(((n >> 3) + kFusedThreads - 1) / kFusedThreads, 6);
    if (hw == 1) {
        // the constants held in registers cost occupancy: the grid is what is resident at once
        static int per_sm = 0;
        if (per_sm == 0) {
            int nb = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, bn_bwd_dx_cl_kernel<DT, 2>, kFusedThreads, 0) != cudaSuccess || nb < 1) nb = 4;
            per_sm = nb;
        }
        const int grid = stream_grid_for(((n >> 3) + kFusedThreads - 1) / kFusedThreads, per_sm);
        switch (bits) {
            case 1: bn_bwd_dx_cl_kernel<DT, 1><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, C); break;
            case 2: bn_bwd_dx_cl_kernel<DT, 2><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, C); break;
            case 4: bn_bwd_dx_cl_kernel<DT, 4><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, C); break;
            default: bn_bwd_dx_cl_kernel<DT, 8><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, C); break;
        }
        return cudaGetLastError();
    }
    switch (bits) {
        case 1: bn_bwd_dx_kernel<DT, 1><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, hw, C); break;
        case 2: bn_bwd_dx_kernel<DT, 2><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, hw, C); break;
        case 4: bn_bwd_dx_kernel<DT, 4><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, hw, C); break;
        default: bn_bwd_dx_kernel<DT, 8><<<grid, kFusedThreads, 0, st>>>(p, s, m, dy, mask, coef, dx, n, log2_gs, hw, C); break;
    }
    return cudaGetLastError();
}

}  // namespace act

static int bn_bwd_dx_common(const void* packed, const float* scale, const float* mn, const void* dy,
                            const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                            int group_size, int bits, const float* coef, void* dx, void* stream)
{
    using namespace act;
    if (!dtype_ok(dtype)) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_batch < 0 || channels <= 0 || hw <= 0) return ACT_ERR_SIZE;
    // hw == 1: channel-minor layout, pieces of eight consecutive channels
    if (hw == 1 ? (channels & 7) != 0 : ((hw & 3) || hw >= (1ll << 31))) return ACT_ERR_UNSUPPORTED;
    const int64_t n = n_batch * channels * hw;
    if (n > (INT64_MAX >> 4) || n % group_size) return ACT_ERR_SIZE;
    if (n == 0) return ACT_OK;
    if (!packed || !scale || !mn || !dy || !coef || !dx) return ACT_ERR_NULL;
    if (((uintptr_t)dy | (uintptr_t)dx | (uintptr_t)coef) & 15 || ((uintptr_t)packed & 7)) return ACT_ERR_ALIGN;
    int log2_gs = 5;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    const uint8_t* g = static_cast<const uint8_t*>(dy);
    const float4* k = reinterpret_cast<const float4*>(coef);
    uint8_t* o = static_cast<uint8_t*>(dx);
    const uint8_t* mk = static_cast<const uint8_t*>(mask_bits);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_bn_bwd_dx<ACT_DTYPE_F32>(bits, p, scale, mn, g, mk, k, o, n, log2_gs, (uint32_t)hw, (uint32_t)channels, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_bn_bwd_dx<ACT_DTYPE_BF16>(bits, p, scale, mn, g, mk, k, o, n, log2_gs, (uint32_t)hw, (uint32_t)channels, st);
    else e = launch_bn_bwd_dx<ACT_DTYPE_F16>(bits, p, scale, mn, g, mk, k, o, n, log2_gs, (uint32_t)hw, (uint32_t)channels, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_bn_bwd_dx(const void* packed, const float* scale, const float* mn, const void* dy,
                             int dtype, int64_t n_batch, int channels, int64_t hw, int group_size, int bits,
                             const float* coef, void* dx, void* stream)
{
    return bn_bwd_dx_common(packed, scale, mn, dy, nullptr, dtype, n_batch, channels, hw, group_size, bits,
                            coef, dx, stream);
}

extern "C" int act_bn_relu_bwd_dx(const void* packed, const float* scale, const float* mn, const void* dy,
                                  const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                                  int group_size, int bits, const float* coef, void* dx, void* stream)
{
    if (!mask_bits) return n_batch * channels * hw == 0 ? ACT_OK : ACT_ERR_NULL;
    return bn_bwd_dx_common(packed, scale, mn, dy, mask_bits, dtype, n_batch, channels, hw, group_size, bits,
                            coef, dx, stream);
}
