// LayerNorm over the last dimension fused with the codec of its INPUT, sm_100a.
//
//   act_ln_fwd_quant_pack:  y = (x - mean) * rstd * weight + bias, mean and rstd per row (fp32), and
//                           the packed x (codes, scale, min) exactly as act_quant_pack would write
//                           them for the same seed and offset: x is read once instead of twice, and
//                           ATen's forward kernel (120 us on bf16 [50432, 768]) is not needed.
//   act_ln_bwd_from_packed: dx, dgamma, dbeta from dy, the packed x, mean, rstd and weight: x is
//                           decoded in registers (the arithmetic of act_dequant_unpack with a bf16
//                           result, i.e. the tensor the unfused path hands to ATen), so the [rows, C]
//                           dequantised copy, ATen's dx kernel and the parameter-gradient pass
//                           collapse into one read of dy and the codes and one write of dx.
//
// One warp per row, rows dealt out round-robin to a persistent grid.  Lane l holds the 8-element
// vectors l, l + 32, ... of its row (at most kMaxVecs: C <= 1024), so a warp's loads are 512
// contiguous bytes; a group of G <= 256 elements is G/8 neighbouring lanes of one such step, its
// minimum and maximum come from xor shuffles.  The hash counter of a piece is its index in the flat
// tensor, as in quant_pack_kernel; regular groups use the fixed-point encoder, a warp with an
// irregular group (denormal, huge or non-finite range) the general one, which gives the same codes
// for the regular groups.
//
// The reference has no such operator (it leaves LayerNorm to PyTorch,
// Activation_Compression/controller.py:87); the evaluation configuration for ViT-B/16 counts
// LayerNorm inputs among the compressed activations.
#include <type_traits>

#include "codec_pack_kernel.cuh"

namespace act {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;
constexpr int kMaxVecs = 4;                // 8-element vectors per lane: C <= 32 * 8 * 4 = 1024

// the 8 elements of one vector as loaded (one 16-byte word, two for fp32) and their fp32 values
template <int DT> struct RawVec { uint4 q[ElemT<DT>::bytes == 4 ? 2 : 1]; };
template <int DT> __device__ __forceinline__ void ln_load_raw(const uint8_t* p, RawVec<DT>& r) {
    r.q[0] = ldg_stream_v4(p);
    if (ElemT<DT>::bytes == 4) r.q[ElemT<DT>::bytes == 4 ? 1 : 0] = ldg_stream_v4(p + 16);
}
template <int DT> __device__ __forceinline__ void ln_widen(const RawVec<DT>& r, float (&f)[8]) {
    if (ElemT<DT>::bytes == 4) {
        const uint4 a = r.q[0], b = r.q[ElemT<DT>::bytes == 4 ? 1 : 0];
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    } else {
        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
        const uint32_t h[4] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { f[2 * k] = widen_lo<D16>(h[k]); f[2 * k + 1] = widen_hi<D16>(h[k]); }
    }
}
template <int DT> __device__ __forceinline__ void ln_zero_raw(RawVec<DT>& r) {
    r.q[0] = make_uint4(0u, 0u, 0u, 0u);
    if (ElemT<DT>::bytes == 4) r.q[ElemT<DT>::bytes == 4 ? 1 : 0] = make_uint4(0u, 0u, 0u, 0u);
}
// eight fp32 parameters of a vector of columns (cached loads: every row reads the same ones)
__device__ __forceinline__ void ln_load_param8(const float* p, float fill, float (&f)[8]) {
    if (p) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = fill;
    }
}

template <int DT> __device__ __forceinline__ void ln_store8(uint8_t* p, const float (&f)[8]) {
    if (DT == ACT_DTYPE_F32) {
        stg_stream_v4(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
        stg_stream_v4(p + 16, make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
    } else {
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (DT == ACT_DTYPE_BF16) { const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
            else { const __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]); o[i] = *reinterpret_cast<const uint32_t*>(&t); }
        }
        stg_stream_v4(p, make_uint4(o[0], o[1], o[2], o[3]));
    }
}

// two fp32 values rounded to the 16-bit element type, as one packed word
template <int DT> __device__ __forceinline__ uint32_t round_pair(float lo, float hi) {
    if (DT == ACT_DTYPE_F16) { const __half2 t = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&t); }
    const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&t);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

template <int BITS> __device__ __forceinline__ void store_codes(uint8_t* p, uint32_t a0, uint32_t a1) {
    if (BITS == 1) *p = (uint8_t)a0;
    else if (BITS == 2) *reinterpret_cast<uint16_t*>(p) = (uint16_t)a0;
    else if (BITS == 4) *reinterpret_cast<uint32_t*>(p) = a0;
    else *reinterpret_cast<uint2*>(p) = make_uint2(a0, a1);
}

// ------------------------------------------------------------------------------ forward
// VECS = vectors per lane (the host passes exactly ceil(C / 256)); FULL: C is a multiple of 256, so
// every lane holds a vector in every step and the per-lane tests (and their branches) fall away.
// ADD (16-bit types): the normalised tensor is x + res, rounded to the element type and written to
// sum_out first (what a separate addition would have produced); statistics, y and the codec then
// work on that rounded sum.
template <int DT, int BITS, int NM, int VECS, bool FULL, bool ADD>
__global__ void __launch_bounds__(kLnThreads)
ln_fwd_pack_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ res, uint8_t* __restrict__ sum_out,
                   const float* __restrict__ weight, const float* __restrict__ bias,
                   uint8_t* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                   uint8_t* __restrict__ packed, float* __restrict__ scale_out, float* __restrict__ min_out,
                   int64_t rows, int C, float eps, int log2_L, uint32_t key_lo, uint32_t key_hi)
{
    constexpr int QMAX = (1 << BITS) - 1;
    constexpr int EB = ElemT<DT>::bytes;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvec = C >> 3;
    const int L = 1 << log2_L;                               // lanes per group
    const float inv_c = 1.0f / (float)C;
    const int64_t warp_stride = (int64_t)gridDim.x * kLnWarps;
    // The next row's vectors are requested before this row is worked on (a warp has one row's
    // arithmetic between its loads otherwise, and 16 warps per SM do not cover HBM's latency).
    RawVec<DT> nxt[VECS], nxr[ADD ? VECS : 1];
    auto request = [&](int64_t r) {
        const uint8_t* xr = x + r * C * EB;
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            if (FULL || v < nvec) {
                ln_load_raw<DT>(xr + (int64_t)v * 8 * EB, nxt[k]);
                if (ADD) ln_load_raw<DT>(res + (r * C + (int64_t)v * 8) * EB, nxr[ADD ? k : 0]);
            } else {
                ln_zero_raw<DT>(nxt[k]);
                if (ADD) ln_zero_raw<DT>(nxr[ADD ? k : 0]);
            }
        }
    };
    int64_t row = (int64_t)blockIdx.x * kLnWarps + warp;
    if (row < rows) request(row);
    for (; row < rows; row += warp_stride) {
        float xf[VECS][8];
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            if (ADD) {
                float fa[8], fb[8];
                ln_widen<DT>(nxt[k], fa);
                ln_widen<DT>(nxr[ADD ? k : 0], fb);
                RawVec<DT> sv;
                sv.q[0] = make_uint4(round_pair<DT>(fa[0] + fb[0], fa[1] + fb[1]), round_pair<DT>(fa[2] + fb[2], fa[3] + fb[3]),
                                     round_pair<DT>(fa[4] + fb[4], fa[5] + fb[5]), round_pair<DT>(fa[6] + fb[6], fa[7] + fb[7]));
                const int v = k * 32 + lane;
                if (FULL || v < nvec) stg_stream_v4(sum_out + (row * C + (int64_t)v * 8) * EB, sv.q[0]);
                ln_widen<DT>(sv, xf[k]);
            } else {
                ln_widen<DT>(nxt[k], xf[k]);                 // vectors past the row hold zeros
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += xf[k][i];
        }
        if (row + warp_stride < rows) request(row + warp_stride);
        const float mean = warp_sum(sum) * inv_c;
        float sq = 0.0f;
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            if (FULL || v < nvec) {
#pragma unroll
                for (int i = 0; i < 8; ++i) { const float d = xf[k][i] - mean; sq = fmaf(d, d, sq); }
            }
        }
        const float rstd = 1.0f / sqrtf(warp_sum(sq) * inv_c + eps);
        if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }

        uint8_t* yr = y + row * C * EB;
        const int64_t piece0 = row * nvec;                   // index of the row's first 8-element piece
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            const bool on = FULL || v < nvec;
            if (on) {
                float yv[8], w8[8], b8[8];
                ln_load_param8(weight ? weight + v * 8 : nullptr, 1.0f, w8);
                ln_load_param8(bias ? bias + v * 8 : nullptr, 0.0f, b8);
#pragma unroll
                for (int i = 0; i < 8; ++i) yv[i] = fmaf((xf[k][i] - mean) * rstd, w8[i], b8[i]);
                ln_store8<DT>(yr + (int64_t)v * 8 * EB, yv);
            }
            // ---- the codec of x: one group = L neighbouring lanes of this step
            float mn = xf[k][0], mx = xf[k][0];
#pragma unroll
            for (int i = 1; i < 7; i += 2) { mn = fmin3_nan(mn, xf[k][i], xf[k][i + 1]); mx = fmax3_nan(mx, xf[k][i], xf[k][i + 1]); }
            mn = fmin_nan(mn, xf[k][7]); mx = fmax_nan(mx, xf[k][7]);
            for (int off = L >> 1; off > 0; off >>= 1) {
                mn = fmin_nan(mn, __shfl_xor_sync(0xffffffffu, mn, off));
                mx = fmax_nan(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            }
            const float range = __fsub_rn(mx, mn);
            const bool fast = !on || (range == 0.0f) || (range >= 0x1p-50f && range <= 0x1p50f);
            const bool all_fast = __all_sync(0xffffffffu, fast);
            float s;
            if (BITS == 1) s = range;
            else if (all_fast) s = div_by_scale(range, (float)QMAX, 1.0f / (float)QMAX);
            else s = __fdiv_rn(range, (float)QMAX);
            if (!(s > 0.0f)) s = 1.0f;
            const float rs = __frcp_rn(s);
            const int64_t piece = piece0 + v;
            if (on && (lane & (L - 1)) == 0) {
                const int64_t g = piece >> log2_L;
                scale_out[g] = s;
                min_out[g] = mn;
            }
            const uint32_t ctr_lo = (uint32_t)piece, ctr_hi = (uint32_t)((uint64_t)piece >> 32) ^ key_hi;
            uint32_t a0, a1;
            if (all_fast) {
                encode_piece_fx<DT, BITS, false, NM>(make_uint4(0u, 0u, 0u, 0u), xf[k], mn, pack2(-mn, -mn), pack2(rs, rs),
                                                     ctr_lo, ctr_hi, key_lo, a0, a1);
            } else {
                float u8[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                encode_piece_slow<BITS, NM>(xf[k], u8, mn, s, rs, fast, ctr_lo, ctr_hi, key_lo, a0, a1);
            }
            if (on) store_codes<BITS>(packed + piece * BITS, a0, a1);
        }
    }
}

// ------------------------------------------------------------------------------ backward
// eight codes -> eight values of the input as act_dequant_unpack writes them with a bf16 result:
// fp32 fma(code, scale, min), rounded to bf16
template <int BITS> __device__ __forceinline__ uint64_t ln_load_codes(const uint8_t* p) {
    if (BITS == 1) return __ldg(p);
    if (BITS == 2) return __ldg(reinterpret_cast<const uint16_t*>(p));
    if (BITS == 4) return __ldg(reinterpret_cast<const uint32_t*>(p));
    return __ldg(reinterpret_cast<const unsigned long long*>(p));
}
template <int BITS>
__device__ __forceinline__ void ln_decode8(uint64_t wbits, float s, float m, float (&xv)[8]) {
    constexpr uint64_t MASK = (1ull << BITS) - 1ull;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float c = (float)(uint32_t)((wbits >> (i * BITS)) & MASK);
        xv[i] = __bfloat162float(__float2bfloat16_rn(__fmaf_rn(c, s, m)));
    }
}

template <int DT, int BITS, int VECS, bool FULL>
__global__ void __launch_bounds__(kLnThreads, VECS <= 3 ? 2 : 1)
ln_bwd_packed_kernel(const uint8_t* __restrict__ dy, const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                     const float* __restrict__ mn, const float* __restrict__ mean, const float* __restrict__ rstd,
                     const float* __restrict__ weight, const uint8_t* __restrict__ dres, uint8_t* __restrict__ dx,
                     float* __restrict__ dgamma, float* __restrict__ dbeta, int64_t rows, int C, int log2_L)
{
    constexpr int EB = ElemT<DT>::bytes;
    __shared__ float s_acc[kLnWarps][2][32 * 8 + 8];         // one step's partial sums per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvec = C >> 3;
    const float inv_c = 1.0f / (float)C;
    float ag[VECS][8], ab[VECS][8];
#pragma unroll
    for (int k = 0; k < VECS; ++k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { ag[k][i] = 0.0f; ab[k][i] = 0.0f; }
    }
    const int64_t warp_stride = (int64_t)gridDim.x * kLnWarps;
    // what the next row needs is requested before this row is worked on: its dy vectors, code
    // words, group constants and statistics (the kernel holds 64 accumulators per thread, so only
    // eight warps fit on an SM and each has to keep two rows in flight)
    typedef typename std::conditional<BITS == 8, uint64_t, uint32_t>::type code_t;
    RawVec<DT> ndy[VECS];
    code_t ncw[VECS];
    float nsc[VECS], nmn[VECS], nmu = 0.0f, nrs = 0.0f;
    auto request = [&](int64_t r) {
        const uint8_t* dyr = dy + r * C * EB;
        const int64_t piece0 = r * nvec;
        nmu = __ldg(mean + r); nrs = __ldg(rstd + r);
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            if (FULL || v < nvec) {
                const int64_t piece = piece0 + v;
                const int64_t gi = piece >> log2_L;
                ln_load_raw<DT>(dyr + (int64_t)v * 8 * EB, ndy[k]);
                ncw[k] = (code_t)ln_load_codes<BITS>(packed + piece * BITS);
                nsc[k] = __ldg(scale + gi); nmn[k] = __ldg(mn + gi);
            } else {
                ln_zero_raw<DT>(ndy[k]);
                ncw[k] = 0; nsc[k] = 0.0f; nmn[k] = 0.0f;
            }
        }
    };
    int64_t row = (int64_t)blockIdx.x * kLnWarps + warp;
    if (row < rows) request(row);
    for (; row < rows; row += warp_stride) {
        const float mu = nmu, rs = nrs;
        // the second gradient of this row is requested now and used at the end of the first pass:
        // asked for where it is added, each row waited for it (87 us against 57 on bf16 [50432, 768])
        RawVec<DT> rv[VECS];
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            if (dres && (FULL || v < nvec)) ln_load_raw<DT>(dres + (row * C + (int64_t)v * 8) * EB, rv[k]);
            else ln_zero_raw<DT>(rv[k]);
        }
        float xh[VECS][8], h[VECS][8];                       // h = rstd * dy * weight + second gradient
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            if (FULL || v < nvec) {
                float xv[8], dv[8], w8[8], rf[8];
                ln_decode8<BITS>((uint64_t)ncw[k], nsc[k], nmn[k], xv);
                ln_widen<DT>(ndy[k], dv);
                ln_load_param8(weight ? weight + v * 8 : nullptr, 1.0f, w8);
                ln_widen<DT>(rv[k], rf);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xh[k][i] = (xv[i] - mu) * rs;
                    const float g = dv[i] * w8[i];
                    s1 = fmaf(g, xh[k][i], s1);
                    s2 += g;
                    h[k][i] = __fmaf_rn(g, rs, rf[i]);
                    ag[k][i] = fmaf(dv[i], xh[k][i], ag[k][i]);
                    ab[k][i] += dv[i];
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) { xh[k][i] = 0.0f; h[k][i] = 0.0f; }
            }
        }
        if (row + warp_stride < rows) request(row + warp_stride);
        // dx = rstd * (g - c2 - xhat * c1) + second gradient = h - rstd * c2 - xhat * rstd * c1
        const float nc1 = -(rs * (warp_sum(s1) * inv_c)), nc2 = -(rs * (warp_sum(s2) * inv_c));
        uint8_t* dxr = dx + row * C * EB;
#pragma unroll
        for (int k = 0; k < VECS; ++k) {
            const int v = k * 32 + lane;
            if (FULL || v < nvec) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __fmaf_rn(xh[k][i], nc1, h[k][i] + nc2);
                ln_store8<DT>(dxr + (int64_t)v * 8 * EB, o);
            }
        }
    }
    // the block's warps own the same columns: combine them step by step in shared memory, then
    // one atomic per block and column
#pragma unroll
    for (int k = 0; k < VECS; ++k) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { s_acc[warp][0][lane * 8 + i] = ag[k][i]; s_acc[warp][1][lane * 8 + i] = ab[k][i]; }
        __syncthreads();
        for (int c = threadIdx.x; c < 256; c += kLnThreads) {
            const int col = k * 256 + c;
            if (col < C) {
                float tg = 0.0f, tb = 0.0f;
#pragma unroll
                for (int ww = 0; ww < kLnWarps; ++ww) { tg += s_acc[ww][0][c]; tb += s_acc[ww][1][c]; }
                atomicAdd(dgamma + col, tg);
                atomicAdd(dbeta + col, tb);
            }
        }
        __syncthreads();
    }
}

template <typename K>
static int ln_grid(K kernel, int64_t rows) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kLnThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    return stream_grid_for((rows + kLnWarps - 1) / kLnWarps, per_sm);
}

static int ln_check(int dtype, int64_t rows, int C, int group_size, int bits) {
    if (rows < 0 || C < 0) return ACT_ERR_SIZE;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 256 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (C == 0 || (C % group_size) || C > 32 * 8 * kMaxVecs) return ACT_ERR_SIZE;   // whole groups per row, C <= 1024
    return ACT_OK;
}

template <int DT, int BITS>
int ln_fwd_launch(bool nearest, const void* x, const void* res, void* sum_out, const float* weight, const float* bias, void* y, float* mean, float* rstd,
                  void* packed, float* scale, float* mn, int64_t rows, int C, float eps, int log2_L, uint64_t seed,
                  uint64_t offset, cudaStream_t st)
{
    const uint64_t key = hash_key(hash_key(seed) + offset);
    const int vecs = (C / 8 + 31) / 32;                      // 8-element vectors per lane: 1..kMaxVecs
    const bool full = (C % 256) == 0;
#define ACT_LN_FWD_F(NM, V, F, A) \
    ln_fwd_pack_kernel<DT, BITS, NM, V, F, A><<<ln_grid(ln_fwd_pack_kernel<DT, BITS, NM, V, F, A>, rows), kLnThreads, 0, st>>>( \
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(res), static_cast<uint8_t*>(sum_out), weight, bias, \
        static_cast<uint8_t*>(y), mean, rstd, static_cast<uint8_t*>(packed), \
        scale, mn, rows, C, eps, log2_L, (uint32_t)key, (uint32_t)(key >> 32))
    // the forward kernel keeps its per-lane tests even for full rows: without them it needs 109
    // registers instead of 78 (two blocks per SM instead of three) and is no faster (62.5 us against
    // 60.0 on bf16 [50432, 768]; the backward kernel gains, 62.8 -> 52.5-55.6 us)
    (void)full;
#define ACT_LN_FWD(NM, V) ACT_LN_FWD_F(NM, V, false, false)
#define ACT_LN_FWD_V(NM) \
    switch (vecs) { case 1: ACT_LN_FWD(NM, 1); break; case 2: ACT_LN_FWD(NM, 2); break; \
                    case 3: ACT_LN_FWD(NM, 3); break; default: ACT_LN_FWD(NM, 4); break; }
#define ACT_LN_ADD(NM, V) ACT_LN_FWD_F(NM, V, false, true)
#define ACT_LN_ADD_V(NM) \
    switch (vecs) { case 1: ACT_LN_ADD(NM, 1); break; case 2: ACT_LN_ADD(NM, 2); break; \
                    case 3: ACT_LN_ADD(NM, 3); break; default: ACT_LN_ADD(NM, 4); break; }
    if (res) {
        // the sum is formed on the packed 16-bit pairs: fp32 callers add first
        if constexpr (DT == ACT_DTYPE_F32) return ACT_ERR_UNSUPPORTED;
        else if (nearest) { ACT_LN_ADD_V(kNoiseConst) } else { ACT_LN_ADD_V(kNoiseHash) }
    } else if (nearest) { ACT_LN_FWD_V(kNoiseConst) } else { ACT_LN_FWD_V(kNoiseHash) }
#undef ACT_LN_ADD_V
#undef ACT_LN_ADD
#undef ACT_LN_FWD_V
#undef ACT_LN_FWD
#undef ACT_LN_FWD_F
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

template <int DT>
int ln_fwd_bits(int bits, bool nearest, const void* x, const void* res, void* sum_out, const float* weight, const float* bias, void* y, float* mean,
                float* rstd, void* packed, float* scale, float* mn, int64_t rows, int C, float eps, int log2_L,
                uint64_t seed, uint64_t offset, cudaStream_t st)
{
    switch (bits) {
        case 1: return ln_fwd_launch<DT, 1>(nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, mn, rows, C, eps, log2_L, seed, offset, st);
        case 2: return ln_fwd_launch<DT, 2>(nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, mn, rows, C, eps, log2_L, seed, offset, st);
        case 4: return ln_fwd_launch<DT, 4>(nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, mn, rows, C, eps, log2_L, seed, offset, st);
        default: return ln_fwd_launch<DT, 8>(nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, mn, rows, C, eps, log2_L, seed, offset, st);
    }
}

template <int DT, int BITS>
int ln_bwd_launch(const void* dy, const void* dres, const void* packed, const float* scale, const float* mn, const float* mean,
                  const float* rstd, const float* weight, void* dx, float* dgamma, float* dbeta, int64_t rows, int C,
                  int log2_L, cudaStream_t st)
{
    const int vecs = (C / 8 + 31) / 32;
    const bool full = (C % 256) == 0;
#define ACT_LN_BWD_F(V, F) \
    ln_bwd_packed_kernel<DT, BITS, V, F><<<ln_grid(ln_bwd_packed_kernel<DT, BITS, V, F>, rows), kLnThreads, 0, st>>>( \
        static_cast<const uint8_t*>(dy), static_cast<const uint8_t*>(packed), scale, mn, mean, rstd, weight, \
        static_cast<const uint8_t*>(dres), static_cast<uint8_t*>(dx), dgamma, dbeta, rows, C, log2_L)
#define ACT_LN_BWD(V) do { if (full) ACT_LN_BWD_F(V, true); else ACT_LN_BWD_F(V, false); } while (0)
    switch (vecs) { case 1: ACT_LN_BWD(1); break; case 2: ACT_LN_BWD(2); break; case 3: ACT_LN_BWD(3); break; default: ACT_LN_BWD(4); break; }
#undef ACT_LN_BWD
#undef ACT_LN_BWD_F
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

template <int DT>
int ln_bwd_bits(int bits, const void* dy, const void* dres, const void* packed, const float* scale, const float* mn, const float* mean,
                const float* rstd, const float* weight, void* dx, float* dgamma, float* dbeta, int64_t rows, int C,
                int log2_L, cudaStream_t st)
{
    switch (bits) {
        case 1: return ln_bwd_launch<DT, 1>(dy, dres, packed, scale, mn, mean, rstd, weight, dx, dgamma, dbeta, rows, C, log2_L, st);
        case 2: return ln_bwd_launch<DT, 2>(dy, dres, packed, scale, mn, mean, rstd, weight, dx, dgamma, dbeta, rows, C, log2_L, st);
        case 4: return ln_bwd_launch<DT, 4>(dy, dres, packed, scale, mn, mean, rstd, weight, dx, dgamma, dbeta, rows, C, log2_L, st);
        default: return ln_bwd_launch<DT, 8>(dy, dres, packed, scale, mn, mean, rstd, weight, dx, dgamma, dbeta, rows, C, log2_L, st);
    }
}

}  // namespace act

static int ln_fwd_entry(const void* x, const void* res, void* sum_out, int dtype, int64_t rows, int cols,
                        const float* weight, const float* bias, double eps, int group_size, int bits, uint64_t seed,
                        uint64_t offset, int flags, void* y, float* mean, float* rstd, void* packed, float* scale,
                        float* min, void* stream)
{
    using namespace act;
    const int rc = ln_check(dtype, rows, cols, group_size, bits);
    if (rc != ACT_OK) return rc;
    if (flags & ~ACT_FLAG_ROUND_NEAREST) return ACT_ERR_UNSUPPORTED;
    if (res && dtype == ACT_DTYPE_F32) return ACT_ERR_UNSUPPORTED;
    if (rows == 0) return ACT_OK;
    if (!x || !y || !mean || !rstd || !packed || !scale || !min) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)packed | (uintptr_t)res | (uintptr_t)sum_out) & 15) return ACT_ERR_ALIGN;
    int log2_L = 0;
    while ((8 << log2_L) < group_size) ++log2_L;
    const bool nearest = (flags & ACT_FLAG_ROUND_NEAREST) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case ACT_DTYPE_F32: return ln_fwd_bits<ACT_DTYPE_F32>(bits, nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, min, rows, cols, (float)eps, log2_L, seed, offset, st);
        case ACT_DTYPE_BF16: return ln_fwd_bits<ACT_DTYPE_BF16>(bits, nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, min, rows, cols, (float)eps, log2_L, seed, offset, st);
        default: return ln_fwd_bits<ACT_DTYPE_F16>(bits, nearest, x, res, sum_out, weight, bias, y, mean, rstd, packed, scale, min, rows, cols, (float)eps, log2_L, seed, offset, st);
    }
}

extern "C" int act_ln_fwd_quant_pack(const void* x, int dtype, int64_t rows, int cols, const float* weight,
                                     const float* bias, double eps, int group_size, int bits, uint64_t seed,
                                     uint64_t offset, int flags, void* y, float* mean, float* rstd, void* packed,
                                     float* scale, float* min, void* stream)
{
    return ln_fwd_entry(x, nullptr, nullptr, dtype, rows, cols, weight, bias, eps, group_size, bits, seed, offset, flags,
                        y, mean, rstd, packed, scale, min, stream);
}

extern "C" int act_ln_add_fwd_quant_pack(const void* x, const void* res, int dtype, int64_t rows, int cols,
                                         const float* weight, const float* bias, double eps, int group_size, int bits,
                                         uint64_t seed, uint64_t offset, int flags, void* sum, void* y, float* mean,
                                         float* rstd, void* packed, float* scale, float* min, void* stream)
{
    if (rows > 0 && cols > 0 && (!res || !sum)) return ACT_ERR_NULL;
    return ln_fwd_entry(x, res, sum, dtype, rows, cols, weight, bias, eps, group_size, bits, seed, offset, flags,
                        y, mean, rstd, packed, scale, min, stream);
}

static int ln_bwd_entry(const void* dy, const void* dres, int dtype, int64_t rows, int cols, const void* packed,
                        const float* scale, const float* min, int group_size, int bits,
                        const float* mean, const float* rstd, const float* weight, void* dx,
                        float* dgamma, float* dbeta, void* stream)
{
    using namespace act;
    const int rc = ln_check(dtype, rows, cols, group_size, bits);
    if (rc != ACT_OK) return rc;
    if (!dgamma || !dbeta) return ACT_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dbeta == dgamma + cols) {                            // one buffer [2, cols]: one clearing pass
        if (cudaMemsetAsync(dgamma, 0, (size_t)cols * 2 * sizeof(float), st) != cudaSuccess) return ACT_ERR_LAUNCH;
    } else if (cudaMemsetAsync(dgamma, 0, (size_t)cols * sizeof(float), st) != cudaSuccess ||
               cudaMemsetAsync(dbeta, 0, (size_t)cols * sizeof(float), st) != cudaSuccess) {
        return ACT_ERR_LAUNCH;
    }
    if (rows == 0) return ACT_OK;
    if (!dy || !packed || !scale || !min || !mean || !rstd || !dx) return ACT_ERR_NULL;
    if (((uintptr_t)dy | (uintptr_t)dx | (uintptr_t)dres) & 15) return ACT_ERR_ALIGN;
    if ((uintptr_t)packed & 7) return ACT_ERR_ALIGN;
    int log2_L = 0;
    while ((8 << log2_L) < group_size) ++log2_L;
    switch (dtype) {
        case ACT_DTYPE_F32: return ln_bwd_bits<ACT_DTYPE_F32>(bits, dy, dres, packed, scale, min, mean, rstd, weight, dx, dgamma, dbeta, rows, cols, log2_L, st);
        case ACT_DTYPE_BF16: return ln_bwd_bits<ACT_DTYPE_BF16>(bits, dy, dres, packed, scale, min, mean, rstd, weight, dx, dgamma, dbeta, rows, cols, log2_L, st);
        default: return ln_bwd_bits<ACT_DTYPE_F16>(bits, dy, dres, packed, scale, min, mean, rstd, weight, dx, dgamma, dbeta, rows, cols, log2_L, st);
    }
}

extern "C" int act_ln_bwd_from_packed(const void* dy, int dtype, int64_t rows, int cols, const void* packed,
                                      const float* scale, const float* min, int group_size, int bits,
                                      const float* mean, const float* rstd, const float* weight, void* dx,
                                      float* dgamma, float* dbeta, void* stream)
{
    return ln_bwd_entry(dy, nullptr, dtype, rows, cols, packed, scale, min, group_size, bits, mean, rstd, weight, dx,
                        dgamma, dbeta, stream);
}

extern "C" int act_ln_bwd_from_packed_sum(const void* dy, const void* dy2, int dtype, int64_t rows, int cols,
                                          const void* packed, const float* scale, const float* min, int group_size,
                                          int bits, const float* mean, const float* rstd, const float* weight,
                                          void* dx, float* dgamma, float* dbeta, void* stream)
{
    return ln_bwd_entry(dy, dy2, dtype, rows, cols, packed, scale, min, group_size, bits, mean, rstd, weight, dx,
                        dgamma, dbeta, stream);
}
