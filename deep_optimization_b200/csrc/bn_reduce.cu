// Per-channel reductions of batch norm over x [N, C, HW], sm_100a.
//
//   act_bn_stats:       batch mean and inverse deviation of x (forward), written together with
//                       the affine parameters as the [C][4] table the fused normalise+codec
//                       kernel reads; running statistics updated in place
//   act_bn_bwd_reduce:  sum(dy * x_hat) and sum(dy) per channel, x_hat decoded from the codec
//
// Both give block (c, s) channel c and a slice of the batch; the block walks the planes (n, c)
// of its slice as one list of 4- or 8-element vectors, thread t taking vectors t, t + 256, ...,
// and every lane accumulates in registers until the slice is done, so there is one warp
// reduction per block instead of one per load.  Loads are contiguous inside a plane.  The
// grid is one resident wave: the number of slices per channel follows from the occupancy.
// HBM traffic: s_in bytes per element (plus bits/8 in backward); nothing is written but
// 2 floats per block.
//
// A channels-last activation ([rows, C] in memory, "channel-minor", passed as HW = 1) is walked
// by rows instead: bn_rows_reduce_kernel below, a thread owning eight channels.
//
// Replaces: Activation_Compression/modules/normalization/kernel_implementation.py:13-92
// (bn_fwd_reduce) and :328-420 (bn_bwd_reduce_dequant_unpack_fused), whose programs
// accumulate with one atomic per tile.
#include "act_common.cuh"

namespace act {

constexpr int kRedThreads = 256;
constexpr int kRedWarps = kRedThreads / 32;

template <int DT> __device__ __forceinline__ float load1(const uint8_t* p, int64_t e) {
    if (ElemT<DT>::bytes == 4) return __ldg(reinterpret_cast<const float*>(p) + e);
    constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
    return widen_lo<D16>((uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p) + e));
}

// the eight BITS-bit codes of elements e..e+7 (e a multiple of 8), low word first
template <int BITS> __device__ __forceinline__ uint2 load_codes8v(const uint8_t* packed, int64_t e) {
    if (BITS == 8) return __ldg(reinterpret_cast<const uint2*>(packed + e));
    if (BITS == 4) return make_uint2(__ldg(reinterpret_cast<const uint32_t*>(packed + (e >> 1))), 0u);
    if (BITS == 2) return make_uint2(__ldg(reinterpret_cast<const unsigned short*>(packed + (e >> 2))), 0u);
    return make_uint2(__ldg(packed + (e >> 3)), 0u);
}

// the four BITS-bit codes of elements e..e+3 (e a multiple of 4)
template <int BITS> __device__ __forceinline__ uint32_t load_codes4(const uint8_t* packed, int64_t e) {
    if (BITS == 8) return __ldg(reinterpret_cast<const uint32_t*>(packed + e));
    if (BITS == 4) return __ldg(reinterpret_cast<const unsigned short*>(packed + (e >> 1)));
    if (BITS == 2) return __ldg(packed + (e >> 2));
    return ((uint32_t)__ldg(packed + (e >> 3)) >> (uint32_t)(e & 4)) & 0xFu;
}

// MODE 0: a = sum(x - pivot), b = sum((x - pivot)^2), pivot = x[0, c, 0], written as the
//         block's partial pair out[(c * S + s) * 2 + {0, 1}] (no atomics, no zeroing);
// MODE 1: a = sum(dy * x_hat), b = sum(dy), added to out[c] and out[C + c]; with `mask`
//         (one bit per element, the fused ReLU's) dy counts only where its bit is set.
// VEC = elements per lane and step: 8 when HW is a multiple of 8 (16-byte loads), else 4.
template <int DT, int MODE, int BITS, int VEC>
__global__ void __launch_bounds__(kRedThreads)
bn_plane_reduce_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ packed,
                       const float* __restrict__ scale, const float* __restrict__ mn,
                       const uint8_t* __restrict__ mask, float* __restrict__ out, int64_t n_batch,
                       uint32_t C, uint32_t hw, int log2_gs)
{
    __shared__ float s_part[kRedWarps][2];
    const uint32_t c = blockIdx.x, s = blockIdx.y, S = gridDim.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t n0 = n_batch * s / S, n1 = n_batch * (s + 1) / S;
    const uint32_t planes = (uint32_t)(n1 - n0);            // the host keeps a slice below 2^31 planes
    const uint32_t vpp = hw / VEC;                          // VEC-element vectors per plane
    // The slice is walked as one list of (plane, vector) items, thread t taking items
    // t, t + 256, ...: every lane is busy whatever the plane size, and consecutive lanes read
    // consecutive vectors.  The position advances without a division.
    const uint32_t step_n = kRedThreads / vpp, step_v = kRedThreads % vpp;
    uint32_t n = threadIdx.x / vpp, v = threadIdx.x % vpp;
    grid_dependency_wait();
    grid_launch_dependents();
    const float pivot = (MODE == 0) ? load1<DT>(x, (int64_t)c * hw) : 0.0f;
    float a = 0.0f, b = 0.0f;
    // element index of the thread's item, advanced with the position (no multiplies in the loop)
    const int64_t plane_stride = (int64_t)C * hw;
    const int64_t step_e = (int64_t)step_n * plane_stride + (int64_t)step_v * VEC;
    int64_t e_next = ((n0 + n) * C + c) * hw + VEC * (int64_t)v;
    // U items per trip: all their loads go out before the first one is consumed (a thread has
    // only a few dozen items, so the loop is bound by load latency, not by instructions)
#ifndef ACT_BN_U8
#define ACT_BN_U8 4
#endif
#ifndef ACT_BN_U4
#define ACT_BN_U4 2
#endif
    constexpr int U = (MODE == 0) ? 4 : (VEC == 8 ? ACT_BN_U8 : ACT_BN_U4);
    constexpr int RAW = (ElemT<DT>::bytes == 4) ? VEC / 4 : (VEC == 8 ? 1 : 0);   // uint4 per item (0: one uint2)
    while (n < planes) {
        int64_t e[U];
        bool ok[U];
        uint4 raw[U][RAW > 0 ? RAW : 1];
        uint2 w[U];
        uint32_t keep[U];
        float sc[U], m[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            ok[u] = n < planes;
            e[u] = e_next;
            v += step_v; n += step_n; e_next += step_e;
            if (v >= vpp) { v -= vpp; ++n; e_next += plane_stride - hw; }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int r = 0; r < (RAW > 0 ? RAW : 1); ++r) raw[u][r] = make_uint4(0u, 0u, 0u, 0u);
            w[u] = make_uint2(0u, 0u); keep[u] = 0xFFu; sc[u] = 0.0f; m[u] = 0.0f;
            if (!ok[u]) continue;
            const uint8_t* px = x + e[u] * ElemT<DT>::bytes;
            if (RAW == 0) {
                uint2 t;
                asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(t.x), "=r"(t.y) : "l"(px));
                raw[u][0] = make_uint4(t.x, t.y, 0u, 0u);
            } else {
#pragma unroll
                for (int r = 0; r < RAW; ++r) raw[u][r] = ldg_stream_v4(px + 16 * r);
            }
            if (MODE == 1) {
                if (VEC == 8) w[u] = load_codes8v<BITS>(packed, e[u]);
                else w[u] = make_uint2(load_codes4<BITS>(packed, e[u]), 0u);
                const int64_t g = e[u] >> log2_gs;
                sc[u] = __ldg(scale + g); m[u] = __ldg(mn + g);
                if (mask) keep[u] = (VEC == 8) ? (uint32_t)__ldg(mask + (e[u] >> 3)) : load_codes4<1>(mask, e[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float f[VEC];
            if (ElemT<DT>::bytes == 4) {
#pragma unroll
                for (int r = 0; r < VEC / 4; ++r) {
                    f[4 * r] = __uint_as_float(raw[u][r].x); f[4 * r + 1] = __uint_as_float(raw[u][r].y);
                    f[4 * r + 2] = __uint_as_float(raw[u][r].z); f[4 * r + 3] = __uint_as_float(raw[u][r].w);
                }
            } else {
                constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
                const uint32_t h[4] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w};
#pragma unroll
                for (int r = 0; r < VEC / 2; ++r) { f[2 * r] = widen_lo<D16>(h[r]); f[2 * r + 1] = widen_hi<D16>(h[r]); }
            }
            if (MODE == 0) {
                if (ok[u]) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        const float d = __fsub_rn(f[i], pivot);
                        a = __fadd_rn(a, d);
                        b = __fmaf_rn(d, d, b);
                    }
                }
            } else {
                // an item past the end holds zeros and adds nothing
                constexpr uint32_t MASK = (1u << BITS) - 1u;
                if (mask) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) f[i] = ((keep[u] >> i) & 1u) ? f[i] : 0.0f;
                }
                // the item lies inside one group: sum(dy * x_hat) = scale * sum(dy * code) + min * sum(dy),
                // the two inner sums on f32x2 pairs
                const f32x2 magic2 = pack2(kMagic, kMagic);
                f32x2 dc2 = pack2(0.0f, 0.0f), d2 = pack2(0.0f, 0.0f);
#pragma unroll
                for (int p = 0; p < VEC / 2; ++p) {
                    const uint32_t word = (BITS == 8 && p >= 2) ? w[u].y : w[u].x;
                    const int sh0 = (BITS == 8) ? ((2 * p) & 3) * 8 : 2 * p * BITS;
                    const f32x2 code2 = sub2_rn(pack2u(kMagicBits | ((word >> sh0) & MASK),
                                                       kMagicBits | ((word >> (sh0 + BITS)) & MASK)), magic2);
                    const f32x2 dy2 = pack2(f[2 * p], f[2 * p + 1]);
                    dc2 = fma2_rn(dy2, code2, dc2);
                    d2 = add2_rn(d2, dy2);
                }
                uint32_t u0, u1, v0, v1;
                unpack2u(dc2, u0, u1);
                unpack2u(d2, v0, v1);
                const float dc = __fadd_rn(__uint_as_float(u0), __uint_as_float(u1));
                const float dsum = __fadd_rn(__uint_as_float(v0), __uint_as_float(v1));
                a = __fmaf_rn(sc[u], dc, __fmaf_rn(m[u], dsum, a));
                b = __fadd_rn(b, dsum);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    if (lane == 0) { s_part[warp][0] = a; s_part[warp][1] = b; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float ta = 0.0f, tb = 0.0f;
#pragma unroll
        for (int w = 0; w < kRedWarps; ++w) { ta += s_part[w][0]; tb += s_part[w][1]; }
        if (MODE == 0) {
            out[((int64_t)c * S + s) * 2] = ta;
            out[((int64_t)c * S + s) * 2 + 1] = tb;
        } else {
            atomicAdd(out + c, ta);
            atomicAdd(out + C + c, tb);
        }
    }
}

// Channel-minor layout (HW = 1: x is [rows, C], C a multiple of 8, a channels-last
// activation).  A thread owns eight consecutive channels (one 16-byte vector of 16-bit
// elements per row) and walks the rows of the block's slice; tpr = min(C/8, 256) threads
// cover one row (or 2048 channels of it, blockIdx.x choosing which) and the block's other
// threads take the following rows, so a warp reads contiguous memory.  Sixteen accumulators per
// thread; at the end the threads of a channel vector are summed through shared memory and
// every channel leaves once per block with coalesced stores (MODE 0: partial pairs
// out[(s * C + c) * 2 + {0, 1}], slice-major) or coalesced atomics (MODE 1).
template <int DT, int MODE, int BITS>
__global__ void __launch_bounds__(kRedThreads)
bn_rows_reduce_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ packed,
                      const float* __restrict__ scale, const float* __restrict__ mn,
                      const uint8_t* __restrict__ mask, float* __restrict__ out, int64_t n_rows,
                      uint32_t C, uint32_t tpr, int log2_gs)
{
    __shared__ float s_acc[16][kRedThreads + 1];
    const uint32_t s = blockIdx.y, S = gridDim.y;
    const uint32_t rpi = kRedThreads / tpr;                  // rows per block step
    const uint32_t q = threadIdx.x % tpr, rl = threadIdx.x / tpr;
    const uint32_t chunk = blockIdx.x * tpr + q;             // which vector of eight channels
    const bool active = rl < rpi && chunk * 8u < C;
    const int64_t r0 = n_rows * s / S, r1 = n_rows * (s + 1) / S;
    grid_dependency_wait();
    grid_launch_dependents();
    float a[8], b[8], pivot[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = 0.0f; b[i] = 0.0f; pivot[i] = 0.0f; }
    if (active) {
        if (MODE == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) pivot[i] = load1<DT>(x, (int64_t)chunk * 8 + i);
        }
        constexpr int U = 4;
        constexpr int RAW = (ElemT<DT>::bytes == 4) ? 2 : 1;
        for (int64_t r = r0 + rl; r < r1; r += (int64_t)U * rpi) {
            uint4 raw[U][RAW];
            uint2 w[U];
            uint32_t keep[U];
            float sc[U], m[U];
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t row = r + (int64_t)u * rpi;
                ok[u] = row < r1;
#pragma unroll
                for (int k = 0; k < RAW; ++k) raw[u][k] = make_uint4(0u, 0u, 0u, 0u);
                w[u] = make_uint2(0u, 0u); keep[u] = 0xFFu; sc[u] = 0.0f; m[u] = 0.0f;
                if (!ok[u]) continue;
                const int64_t e = row * C + (int64_t)chunk * 8;
                const uint8_t* px = x + e * ElemT<DT>::bytes;
#pragma unroll
                for (int k = 0; k < RAW; ++k) raw[u][k] = ldg_stream_v4(px + 16 * k);
                if (MODE == 1) {
                    w[u] = load_codes8v<BITS>(packed, e);
                    const int64_t g = e >> log2_gs;
                    sc[u] = __ldg(scale + g); m[u] = __ldg(mn + g);
                    if (mask) keep[u] = (uint32_t)__ldg(mask + (e >> 3));
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float f[8];
                if (ElemT<DT>::bytes == 4) {
#pragma unroll
                    for (int k = 0; k < RAW; ++k) {
                        f[4 * k] = __uint_as_float(raw[u][k].x); f[4 * k + 1] = __uint_as_float(raw[u][k].y);
                        f[4 * k + 2] = __uint_as_float(raw[u][k].z); f[4 * k + 3] = __uint_as_float(raw[u][k].w);
                    }
                } else {
                    constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
                    const uint32_t h[4] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) { f[2 * k] = widen_lo<D16>(h[k]); f[2 * k + 1] = widen_hi<D16>(h[k]); }
                }
                if (MODE == 0) {
                    if (ok[u]) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float d = __fsub_rn(f[i], pivot[i]);
                            a[i] = __fadd_rn(a[i], d);
                            b[i] = __fmaf_rn(d, d, b[i]);
                        }
                    }
                } else {
                    // a row past the end holds zeros and adds nothing
                    constexpr uint32_t MASK = (1u << BITS) - 1u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t word = (BITS == 8 && i >= 4) ? w[u].y : w[u].x;
                        const int sh = (BITS == 8) ? (i & 3) * 8 : i * BITS;
                        const float code = __fsub_rn(__uint_as_float(kMagicBits | ((word >> sh) & MASK)), kMagic);
                        const float xh = __fmaf_rn(code, sc[u], m[u]);
                        const float d = ((keep[u] >> i) & 1u) ? f[i] : 0.0f;
                        a[i] = __fmaf_rn(d, xh, a[i]);
                        b[i] = __fadd_rn(b[i], d);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { s_acc[i][threadIdx.x] = a[i]; s_acc[8 + i][threadIdx.x] = b[i]; }
    __syncthreads();
    // channel cl of the block's tile: vector cl / 8, element cl % 8, summed over the row lanes
    const uint32_t tile_c = tpr * 8u, c_base = blockIdx.x * tile_c;
    for (uint32_t cl = threadIdx.x; cl < tile_c && c_base + cl < C; cl += kRedThreads) {
        const uint32_t v = cl >> 3, i = cl & 7u;
        float ta = 0.0f, tb = 0.0f;
        for (uint32_t l = 0; l < rpi; ++l) { ta += s_acc[i][l * tpr + v]; tb += s_acc[8 + i][l * tpr + v]; }
        const uint32_t c = c_base + cl;
        if (MODE == 0) {
            *reinterpret_cast<float2*>(out + ((int64_t)s * C + c) * 2) = make_float2(ta, tb);
        } else {
            atomicAdd(out + c, ta);
            atomicAdd(out + C + c, tb);
        }
    }
}

// LPC lanes per channel (1 after the plane walk; 32 after the row walk, which leaves hundreds of
// partials per channel): the block partials summed in a fixed order in double, then
// mean = pivot + a/M, var = b/M - (a/M)^2 (biased), invstd = 1/sqrt(var + eps).
template <int DT, int LPC>
__global__ void bn_stats_finalize_kernel(const uint8_t* __restrict__ x, const float* __restrict__ part,
                                         const float* __restrict__ weight, const float* __restrict__ bias,
                                         float* __restrict__ running_mean, float* __restrict__ running_var,
                                         float4* __restrict__ params, int64_t n_batch, uint32_t C, uint32_t hw,
                                         uint32_t S, double eps, double momentum, uint32_t stride_c, uint32_t stride_s)
{
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t c = (blockIdx.x * blockDim.x + threadIdx.x) / LPC, sub = threadIdx.x % LPC;
    double a = 0.0, b = 0.0;
    // partial pair (c, s) sits at pair index c * stride_c + s * stride_s (channel-major from the
    // plane walk, slice-major from the row walk)
    if (c < C) {
        // four loads in flight per lane; the order of the additions is fixed
        for (uint32_t s = sub; s < S; s += 4 * LPC) {
            float2 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t su = s + u * LPC;
                t[u] = su < S ? *reinterpret_cast<const float2*>(part + ((int64_t)c * stride_c + (int64_t)su * stride_s) * 2)
                              : make_float2(0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) { a += (double)t[u].x; b += (double)t[u].y; }
        }
    }
#pragma unroll
    for (int off = LPC / 2; off > 0; off >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    if (c >= C || sub != 0) return;
    const double M = (double)n_batch * (double)hw;
    const double dm = a / M;
    const double mean = (double)load1<DT>(x, (int64_t)c * hw) + dm;
    double var = b / M - dm * dm;
    if (!(var > 0.0)) var = 0.0;
    const double invstd = 1.0 / sqrt(var + eps);
    params[c] = make_float4((float)mean, (float)invstd, weight ? weight[c] : 1.0f, bias ? bias[c] : 0.0f);
    if (running_mean) running_mean[c] = (float)((1.0 - momentum) * (double)running_mean[c] + momentum * mean);
    if (running_var) {
        const double unbiased = var * (M / (M > 1.0 ? M - 1.0 : 1.0));
        running_var[c] = (float)((1.0 - momentum) * (double)running_var[c] + momentum * unbiased);
    }
}

// coef[c] = (k1, k1 * sum(dy) / M, k1 * sum(dy * x_hat) / M, 0) with k1 = weight * invstd: the
// per-channel constants of dx = k1 * dy - k2 - k3 * x_hat
__global__ void bn_bwd_coef_kernel(const float* __restrict__ sums, const float4* __restrict__ params,
                                   float4* __restrict__ coef, uint32_t C, float inv_count)
{
    grid_dependency_wait();
    grid_launch_dependents();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float4 p = params[c];
    const float k1 = __fmul_rn(p.z, p.y);
    coef[c] = make_float4(k1, __fmul_rn(__fmul_rn(k1, sums[C + c]), inv_count),
                          __fmul_rn(__fmul_rn(k1, sums[c]), inv_count), 0.0f);
}

// Batch slices per channel: as many as keep the whole grid resident at once (`capacity`
// blocks), at least one plane per slice, and few enough planes per slice for 32-bit counters.
static int bn_splits(int64_t n_batch, int channels, int capacity) {
    int64_t want = capacity / channels;
    if (want < 1) want = 1;
    if (want > n_batch) want = n_batch;
    const int64_t least = (n_batch + (1ll << 30) - 1) >> 30;
    if (want < least) want = least;
    if (want > 65535) want = 65535;
    return (int)want;
}

// resident blocks of a reduce kernel on the current device (SM count x occupancy), asked once
// per instantiation; the statistics workspace is sized for the largest answer possible
constexpr int kMaxCapacity = 148 * 8 * 2;
template <typename K> static int reduce_capacity(K kernel) {
    static int cached = 0;
    if (cached == 0) {
        int per_sm = 0, dev = 0, sms = 148;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRedThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int cap = per_sm * sms;
        if (cap > kMaxCapacity) cap = kMaxCapacity;
        cached = cap;
    }
    return cached;
}

// Row walk (channel-minor layout): threads per row, column tiles of 2048 channels and row
// slices; the grid is col_tiles x slices, at most one resident wave and kMaxRowSlices slices.
constexpr int kMaxRowSlices = 592;
struct RowGeom { uint32_t tpr, col_tiles; int S; };
static RowGeom row_geom(int64_t n_rows, int channels, int capacity) {
    RowGeom g;
    const uint32_t cols8 = (uint32_t)channels / 8u;
    g.tpr = cols8 < (uint32_t)kRedThreads ? cols8 : (uint32_t)kRedThreads;
    g.col_tiles = (cols8 + g.tpr - 1) / g.tpr;
    int64_t want = capacity / (int64_t)g.col_tiles;
    const int64_t rpi = kRedThreads / g.tpr;
    const int64_t steps = (n_rows + rpi - 1) / rpi;          // a slice gets at least one block step of rows
    if (want > steps) want = steps;
    if (want > kMaxRowSlices) want = kMaxRowSlices;
    if (want < 1) want = 1;
    g.S = (int)want;
    return g;
}

static bool dtype_ok(int d) { return d == ACT_DTYPE_F32 || d == ACT_DTYPE_BF16 || d == ACT_DTYPE_F16; }

template <int DT>
static cudaError_t launch_stats(const uint8_t* x, int64_t n_batch, int C, int64_t hw, double eps,
                                const float* weight, const float* bias, float* rm, float* rv, double momentum,
                                float* params, float* ws, cudaStream_t st)
{
    if (hw == 1) {
        // channel-minor: row walk, slice-major partials
        const RowGeom g = row_geom(n_batch, C, reduce_capacity(bn_rows_reduce_kernel<DT, 0, 2>));
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.gridDim = dim3(g.col_tiles, (unsigned)g.S, 1);
        cfg.blockDim = dim3(kRedThreads, 1, 1);
        cfg.stream = st;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, bn_rows_reduce_kernel<DT, 0, 2>, x, static_cast<const uint8_t*>(nullptr),
                                           static_cast<const float*>(nullptr), static_cast<const float*>(nullptr),
                                           static_cast<const uint8_t*>(nullptr), ws, n_batch, (uint32_t)C, g.tpr, 5);
        if (e != cudaSuccess) return e;
        return launch_overlapped(bn_stats_finalize_kernel<DT, 32>, (C * 32 + 127) / 128, 128, st, x, static_cast<const float*>(ws),
                                 weight, bias, rm, rv, reinterpret_cast<float4*>(params), n_batch, (uint32_t)C,
                                 1u, (uint32_t)g.S, eps, momentum, 1u, (uint32_t)C);
    }
    auto kernel = (hw & 7) ? bn_plane_reduce_kernel<DT, 0, 2, 4> : bn_plane_reduce_kernel<DT, 0, 2, 8>;
    const int S = bn_splits(n_batch, C, (hw & 7) ? reduce_capacity(bn_plane_reduce_kernel<DT, 0, 2, 4>)
                                                 : reduce_capacity(bn_plane_reduce_kernel<DT, 0, 2, 8>));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)C, (unsigned)S, 1);
    cfg.blockDim = dim3(kRedThreads, 1, 1);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, x, static_cast<const uint8_t*>(nullptr),
                                       static_cast<const float*>(nullptr), static_cast<const float*>(nullptr),
                                       static_cast<const uint8_t*>(nullptr), ws, n_batch, (uint32_t)C, (uint32_t)hw, 5);
    if (e != cudaSuccess) return e;
    return launch_overlapped(bn_stats_finalize_kernel<DT, 1>, (C + 127) / 128, 128, st, x, static_cast<const float*>(ws),
                             weight, bias, rm, rv, reinterpret_cast<float4*>(params), n_batch, (uint32_t)C,
                             (uint32_t)hw, (uint32_t)S, eps, momentum, (uint32_t)S, 1u);
}

template <int DT, int BITS>
static cudaError_t launch_bwd_reduce_one(const uint8_t* dy, const uint8_t* packed, const float* scale, const float* mn,
                                         const uint8_t* mask, float* sums, int64_t n_batch, int C, int64_t hw, int log2_gs, cudaStream_t st)
{
    if (hw == 1) {
        const RowGeom g = row_geom(n_batch, C, reduce_capacity(bn_rows_reduce_kernel<DT, 1, BITS>));
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.gridDim = dim3(g.col_tiles, (unsigned)g.S, 1);
        cfg.blockDim = dim3(kRedThreads, 1, 1);
        cfg.stream = st;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, bn_rows_reduce_kernel<DT, 1, BITS>, dy, packed, scale, mn, mask, sums, n_batch,
                                  (uint32_t)C, g.tpr, log2_gs);
    }
    auto kernel = (hw & 7) ? bn_plane_reduce_kernel<DT, 1, BITS, 4> : bn_plane_reduce_kernel<DT, 1, BITS, 8>;
    const int S = bn_splits(n_batch, C, (hw & 7) ? reduce_capacity(bn_plane_reduce_kernel<DT, 1, BITS, 4>)
                                                 : reduce_capacity(bn_plane_reduce_kernel<DT, 1, BITS, 8>));
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)C, (unsigned)S, 1);
    cfg.blockDim = dim3(kRedThreads, 1, 1);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, dy, packed, scale, mn, mask, sums, n_batch,
                              (uint32_t)C, (uint32_t)hw, log2_gs);
}

template <int DT>
static cudaError_t launch_bwd_reduce(int bits, const uint8_t* dy, const uint8_t* packed, const float* scale,
                                     const float* mn, const uint8_t* mask, float* sums, int64_t n_batch, int C, int64_t hw, int log2_gs,
                                     cudaStream_t st)
{
    switch (bits) {
        case 1: return launch_bwd_reduce_one<DT, 1>(dy, packed, scale, mn, mask, sums, n_batch, C, hw, log2_gs, st);
        case 2: return launch_bwd_reduce_one<DT, 2>(dy, packed, scale, mn, mask, sums, n_batch, C, hw, log2_gs, st);
        case 4: return launch_bwd_reduce_one<DT, 4>(dy, packed, scale, mn, mask, sums, n_batch, C, hw, log2_gs, st);
        default: return launch_bwd_reduce_one<DT, 8>(dy, packed, scale, mn, mask, sums, n_batch, C, hw, log2_gs, st);
    }
}

}  // namespace act

extern "C" size_t act_bn_stats_workspace(int64_t n_batch, int channels)
{
    if (n_batch <= 0 || channels <= 0) return 0;
    // enough for the plane walk's slices and for the row walk's (channel-minor layout, where
    // n_batch counts rows)
    size_t slices = (size_t)act::bn_splits(n_batch, channels, act::kMaxCapacity);
    const size_t row_slices = (size_t)(n_batch < act::kMaxRowSlices ? n_batch : act::kMaxRowSlices);
    if (row_slices > slices) slices = row_slices;
    return (size_t)channels * slices * 2 * sizeof(float);
}

extern "C" int act_bn_stats(const void* x, int dtype, int64_t n_batch, int channels, int64_t hw, double eps,
                            const float* weight, const float* bias, float* running_mean, float* running_var,
                            double momentum, float* params, void* workspace, size_t ws_bytes, void* stream)
{
    using namespace act;
    if (!dtype_ok(dtype)) return ACT_ERR_DTYPE;
    if (n_batch <= 0 || channels <= 0 || hw <= 0) return ACT_ERR_SIZE;
    // hw == 1: channel-minor layout ([rows, C]), vectors of eight channels
    if (hw == 1 ? (channels & 7) != 0 : ((hw & 3) || hw >= (1ll << 31) || channels > 65535)) return ACT_ERR_UNSUPPORTED;
    if (n_batch * channels > (INT64_MAX >> 4) / hw) return ACT_ERR_SIZE;
    if (!x || !params || !workspace) return ACT_ERR_NULL;
    // a plane starts on a multiple of 4 elements: 8 bytes for 16-bit types, 16 for fp32
    if (((uintptr_t)x | (uintptr_t)params) & 15 || ((uintptr_t)workspace & 3)) return ACT_ERR_ALIGN;
    if (ws_bytes < act_bn_stats_workspace(n_batch, channels)) return ACT_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    float* ws = static_cast<float*>(workspace);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_stats<ACT_DTYPE_F32>(xb, n_batch, channels, hw, eps, weight, bias, running_mean, running_var, momentum, params, ws, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_stats<ACT_DTYPE_BF16>(xb, n_batch, channels, hw, eps, weight, bias, running_mean, running_var, momentum, params, ws, st);
    else e = launch_stats<ACT_DTYPE_F16>(xb, n_batch, channels, hw, eps, weight, bias, running_mean, running_var, momentum, params, ws, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

static int bn_bwd_reduce_common(const void* packed, const float* scale, const float* mn, const void* dy,
                                const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                                int group_size, int bits, float* sums, void* stream)
{
    using namespace act;
    if (!dtype_ok(dtype)) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_batch < 0 || channels <= 0 || hw <= 0) return ACT_ERR_SIZE;
    if (hw == 1 ? (channels & 7) != 0 : ((hw & 3) || hw >= (1ll << 31) || channels > 65535)) return ACT_ERR_UNSUPPORTED;
    const int64_t n = n_batch * channels * hw;
    if (n > (INT64_MAX >> 4) || n % group_size) return ACT_ERR_SIZE;
    if (n == 0) return ACT_OK;
    if (!packed || !scale || !mn || !dy || !sums) return ACT_ERR_NULL;
    if (((uintptr_t)dy & 15) || ((uintptr_t)packed & 7)) return ACT_ERR_ALIGN;
    int log2_gs = 5;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    const uint8_t* g = static_cast<const uint8_t*>(dy);
    const uint8_t* mask = static_cast<const uint8_t*>(mask_bits);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_bwd_reduce<ACT_DTYPE_F32>(bits, g, p, scale, mn, mask, sums, n_batch, channels, hw, log2_gs, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_bwd_reduce<ACT_DTYPE_BF16>(bits, g, p, scale, mn, mask, sums, n_batch, channels, hw, log2_gs, st);
    else e = launch_bwd_reduce<ACT_DTYPE_F16>(bits, g, p, scale, mn, mask, sums, n_batch, channels, hw, log2_gs, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_bn_bwd_reduce(const void* packed, const float* scale, const float* mn, const void* dy,
                                 int dtype, int64_t n_batch, int channels, int64_t hw, int group_size,
                                 int bits, float* sums, void* stream)
{
    return bn_bwd_reduce_common(packed, scale, mn, dy, nullptr, dtype, n_batch, channels, hw, group_size, bits,
                                sums, stream);
}

extern "C" int act_bn_relu_bwd_reduce(const void* packed, const float* scale, const float* mn, const void* dy,
                                      const void* mask_bits, int dtype, int64_t n_batch, int channels,
                                      int64_t hw, int group_size, int bits, float* sums, void* stream)
{
    if (!mask_bits) return n_batch * channels * hw == 0 ? ACT_OK : ACT_ERR_NULL;
    return bn_bwd_reduce_common(packed, scale, mn, dy, mask_bits, dtype, n_batch, channels, hw, group_size, bits,
                                sums, stream);
}

// BN + residual + ReLU: dy under the mask goes to dy_masked (the residual's gradient, written
// by act_relu_bwd_unpack) and the plain reduction reads it.  (Writing dy_masked from inside the
// reduction kernel was tried and gained nothing: that kernel is bound by its ALU work, and the
// extra conversions and stores cost what the separate pass did, 28.8 against 28.6 ms per
// ResNet-50 step.)
extern "C" int act_bn_add_relu_bwd_reduce_sum(const void* packed, const float* scale, const float* mn, const void* dy,
                                              const void* dy2, const void* mask_bits, int dtype, int64_t n_batch,
                                              int channels, int64_t hw, int group_size, int bits, float* sums,
                                              void* dy_masked, void* stream)
{
    if (!mask_bits || !dy_masked) return n_batch * channels * hw == 0 ? ACT_OK : ACT_ERR_NULL;
    const int rc = act_relu_bwd_unpack_sum(mask_bits, dy, dy2, dtype, n_batch * channels * hw, dy_masked, stream);
    if (rc != ACT_OK) return rc;
    return bn_bwd_reduce_common(packed, scale, mn, dy_masked, nullptr, dtype, n_batch, channels, hw, group_size, bits,
                                sums, stream);
}

extern "C" int act_bn_add_relu_bwd_reduce(const void* packed, const float* scale, const float* mn, const void* dy,
                                          const void* mask_bits, int dtype, int64_t n_batch, int channels,
                                          int64_t hw, int group_size, int bits, float* sums, void* dy_masked,
                                          void* stream)
{
    return act_bn_add_relu_bwd_reduce_sum(packed, scale, mn, dy, nullptr, mask_bits, dtype, n_batch, channels, hw,
                                          group_size, bits, sums, dy_masked, stream);
}

extern "C" int act_bn_bwd_coef(const float* sums, const float* params, int channels, double count,
                               float* coef, void* stream)
{
    using namespace act;
    if (channels <= 0 || !(count > 0.0)) return ACT_ERR_SIZE;
    if (!sums || !params || !coef) return ACT_ERR_NULL;
    if (((uintptr_t)params | (uintptr_t)coef) & 15 || ((uintptr_t)sums & 3)) return ACT_ERR_ALIGN;
    cudaError_t e = launch_overlapped(bn_bwd_coef_kernel, (channels + 127) / 128, 128, static_cast<cudaStream_t>(stream),
                                      sums, reinterpret_cast<const float4*>(params), reinterpret_cast<float4*>(coef),
                                      (uint32_t)channels, (float)(1.0 / count));
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
