// Max pooling on channels-last activations that keeps a 4-bit argmax per output, sm_100a.
//
// PyTorch's max-pool saves one int64 index per output element for backward (8 bytes where the
// output itself takes 2) and its channels-last backward kernel runs far from the memory
// roofline.  Here the position of the maximum inside its k x k window (k*k <= 16) is stored in
// four bits, eight channels per 32-bit word, and backward gathers: every input position looks
// at the few windows that cover it and adds dy where the stored position is its own.  The
// reference has no pooling operator; this is the same save-less-for-backward idea applied to
// the one remaining layer of its ResNet payload (Model/CNN/ResNetV1.py:63,99).
//
//   x  [N, H, W, C] (channel-minor, C a multiple of 8), y [N, OH, OW, C],
//   idx uint32 [N*OH*OW*C/8]: nibble j of word q = window position kh*k + kw of channel 8q'+j
//   OH = (H + 2*pad - k) / stride + 1 (floor), likewise OW; no dilation.
// Ties go to the first position in scan order and a NaN wins, as in PyTorch.
#include "act_common.cuh"

namespace act {

constexpr int kPoolThreads = 256;

template <int DT> __device__ __forceinline__ void pool_load8(const uint8_t* p, int64_t e, float (&f)[8]) {
    if (ElemT<DT>::bytes == 4) {
        const uint4 a = ldg_nc_v4(p + e * 4), b = ldg_nc_v4(p + e * 4 + 16);
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    } else {
        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
        const uint4 a = ldg_nc_v4(p + e * 2);
        f[0] = widen_lo<D16>(a.x); f[1] = widen_hi<D16>(a.x); f[2] = widen_lo<D16>(a.y); f[3] = widen_hi<D16>(a.y);
        f[4] = widen_lo<D16>(a.z); f[5] = widen_hi<D16>(a.z); f[6] = widen_lo<D16>(a.w); f[7] = widen_hi<D16>(a.w);
    }
}

template <int DT> __device__ __forceinline__ void pool_store8(uint8_t* p, int64_t e, const float (&f)[8]) {
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

struct PoolGeom { int H, W, C8, OH, OW, k, s, pad; };

// one thread per output position and vector of eight channels.  K > 0: the window size is known at
// compile time and the scan is unrolled (K = 0: taken from g.k)
template <int DT, int K = 0>
__global__ void __launch_bounds__(kPoolThreads)
maxpool_fwd_cl_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ y, uint32_t* __restrict__ idx,
                      int64_t n_out_pieces, PoolGeom g)
{
    const int64_t stride = (int64_t)gridDim.x * kPoolThreads;
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t p = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; p < n_out_pieces; p += stride) {
        const int c8 = (int)(p % g.C8);
        int64_t t = p / g.C8;
        const int ow = (int)(t % g.OW); t /= g.OW;
        const int oh = (int)(t % g.OH);
        const int64_t n = t / g.OH;
        const int h0 = oh * g.s - g.pad, w0 = ow * g.s - g.pad;
        const int k = K > 0 ? K : g.k;
        if (ElemT<DT>::bytes == 2) {
            // 16-bit inputs: the maximum and its position are tracked on the packed pairs as they
            // were loaded (a comparison of two bf16 or fp16 values is the comparison of their fp32
            // images): per pair one "greater" mask, one "is NaN" mask and two bit selects, instead
            // of widening and four compares and selects per element.  The position sits in the low
            // bits of each 16-bit half of `where`.
            uint32_t best[4], where[4];
            bool first = true;
            const uint32_t ninf2 = (DT == ACT_DTYPE_F16) ? 0xFC00FC00u : 0xFF80FF80u;      // (-inf, -inf)
#pragma unroll
            for (int kh = 0; kh < k; ++kh) {
                const int ih = h0 + kh;
                if (ih < 0 || ih >= g.H) continue;
#pragma unroll
                for (int kw = 0; kw < k; ++kw) {
                    const int iw = w0 + kw;
                    if (iw < 0 || iw >= g.W) continue;
                    const uint4 raw = ldg_nc_v4(x + (((n * g.H + ih) * g.W + iw) * g.C8 + c8) * 16);
                    const uint32_t v[4] = {raw.x, raw.y, raw.z, raw.w};
                    const uint32_t pos2 = (uint32_t)(kh * k + kw) * 0x00010001u;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (first) { best[i] = ninf2; where[i] = pos2; }
                        uint32_t m;
                        if (DT == ACT_DTYPE_F16) {
                            const __half2 a = *reinterpret_cast<const __half2*>(&v[i]), b = *reinterpret_cast<const __half2*>(&best[i]);
                            m = __hgt2_mask(a, b) | __hneu2_mask(a, a);
                        } else {
                            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v[i]), b = *reinterpret_cast<const __nv_bfloat162*>(&best[i]);
                            m = __hgt2_mask(a, b) | __hneu2_mask(a, a);
                        }
                        best[i] = (v[i] & m) | (best[i] & ~m);
                        where[i] = (pos2 & m) | (where[i] & ~m);
                    }
                    first = false;
                }
            }
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) word |= ((where[i] & 0xFu) << (8 * i)) | (((where[i] >> 16) & 0xFu) << (8 * i + 4));
            stg_stream_v4(y + p * 16, make_uint4(best[0], best[1], best[2], best[3]));
            idx[p] = word;
            continue;
        }
        float best[8];
        uint32_t where[8];
        bool first = true;
#pragma unroll
        for (int kh = 0; kh < k; ++kh) {
            const int ih = h0 + kh;
            if (ih < 0 || ih >= g.H) continue;
#pragma unroll
            for (int kw = 0; kw < k; ++kw) {
                const int iw = w0 + kw;
                if (iw < 0 || iw >= g.W) continue;
                float f[8];
                pool_load8<DT>(x, (((n * g.H + ih) * g.W + iw) * g.C8 + c8) * 8, f);
                const uint32_t pos = (uint32_t)(kh * k + kw);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // the first position in range seeds the index; later ones replace it when
                    // larger, or when NaN (which then stays)
                    if (first) { best[i] = -INFINITY; where[i] = pos; }
                    if (f[i] > best[i] || f[i] != f[i]) { best[i] = f[i]; where[i] = pos; }
                }
                first = false;
            }
        }
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) word |= where[i] << (4 * i);
        pool_store8<DT>(y, p * 8, best);
        idx[p] = word;
    }
}

// one thread per input position and vector of eight channels: gather from the covering windows
template <int DT>
__global__ void __launch_bounds__(kPoolThreads)
maxpool_bwd_cl_kernel(const uint32_t* __restrict__ idx, const uint8_t* __restrict__ dy, uint8_t* __restrict__ dx,
                      int64_t n_in_pieces, PoolGeom g)
{
    const int64_t stride = (int64_t)gridDim.x * kPoolThreads;
    grid_dependency_wait();
    grid_launch_dependents();
    for (int64_t p = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; p < n_in_pieces; p += stride) {
        const int c8 = (int)(p % g.C8);
        int64_t t = p / g.C8;
        const int iw = (int)(t % g.W); t /= g.W;
        const int ih = (int)(t % g.H);
        const int64_t n = t / g.H;
        // windows oh with oh*s - pad <= ih <= oh*s - pad + k - 1
        int oh_lo = ih + g.pad - g.k + 1;
        oh_lo = oh_lo <= 0 ? 0 : (oh_lo + g.s - 1) / g.s;
        int oh_hi = (ih + g.pad) / g.s;
        if (oh_hi > g.OH - 1) oh_hi = g.OH - 1;
        int ow_lo = iw + g.pad - g.k + 1;
        ow_lo = ow_lo <= 0 ? 0 : (ow_lo + g.s - 1) / g.s;
        int ow_hi = (iw + g.pad) / g.s;
        if (ow_hi > g.OW - 1) ow_hi = g.OW - 1;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int oh = oh_lo; oh <= oh_hi; ++oh) {
            const uint32_t kh = (uint32_t)(ih - (oh * g.s - g.pad));
            for (int ow = ow_lo; ow <= ow_hi; ++ow) {
                const uint32_t pos = kh * (uint32_t)g.k + (uint32_t)(iw - (ow * g.s - g.pad));
                const int64_t q = ((n * g.OH + oh) * g.OW + ow) * g.C8 + c8;
                const uint32_t word = __ldg(idx + q);
                // skip the gradient load when none of the eight channels points here
                uint32_t hit = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) hit |= (((word >> (4 * i)) & 0xFu) == pos) ? (1u << i) : 0u;
                if (!hit) continue;
                float f[8];
                pool_load8<DT>(dy, q * 8, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) if ((hit >> i) & 1u) acc[i] = __fadd_rn(acc[i], f[i]);
            }
        }
        pool_store8<DT>(dx, p * 8, acc);
    }
}

// ---- backward with the operands of a block staged in shared memory -----------------------------
// A block takes one image, a tile of 8 x 32 input positions and up to 64 channels.  It first copies
// the gradients and index words of the windows that cover its tile into shared memory, every piece
// requested once and all requests independent (the kernel above chases an index word and then a
// gradient, window after window), then every thread gathers from there with the same logic.
// 534 -> 458 us on ResNet-50's pooling layer at batch 256.  The forward kernel gained nothing from
// the same treatment (388 against 381 us) and stays as it is: neither is bound by its loads.
template <int DT> struct PoolVec8 { uint4 q[ElemT<DT>::bytes == 4 ? 2 : 1]; };
template <int DT> __device__ __forceinline__ PoolVec8<DT> pool_load_raw(const uint8_t* p, int64_t e) {
    PoolVec8<DT> v;
    v.q[0] = ldg_nc_v4(p + e * ElemT<DT>::bytes);
    if (ElemT<DT>::bytes == 4) v.q[ElemT<DT>::bytes == 4 ? 1 : 0] = ldg_nc_v4(p + e * 4 + 16);
    return v;
}
template <int DT> __device__ __forceinline__ void pool_widen(const PoolVec8<DT>& v, float (&f)[8]) {
    if (ElemT<DT>::bytes == 4) {
        const uint4 a = v.q[0], b = v.q[ElemT<DT>::bytes == 4 ? 1 : 0];
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    } else {
        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
        const uint4 a = v.q[0];
        f[0] = widen_lo<D16>(a.x); f[1] = widen_hi<D16>(a.x); f[2] = widen_lo<D16>(a.y); f[3] = widen_hi<D16>(a.y);
        f[4] = widen_lo<D16>(a.z); f[5] = widen_hi<D16>(a.z); f[6] = widen_lo<D16>(a.w); f[7] = widen_hi<D16>(a.w);
    }
}

struct PoolTile { int th, tw, tiles_h, tiles_w, chunks, pc; };   // tile size (positions), tiles per image, channel chunks, pieces per chunk

template <int DT>
__global__ void __launch_bounds__(kPoolThreads)
maxpool_bwd_tile_kernel(const uint32_t* __restrict__ idx, const uint8_t* __restrict__ dy, uint8_t* __restrict__ dx,
                        PoolGeom g, PoolTile t, int max_oh, int max_ow)
{
    extern __shared__ __align__(16) uint8_t pool_smem[];
    PoolVec8<DT>* gtile = reinterpret_cast<PoolVec8<DT>*>(pool_smem);
    uint32_t* wtile = reinterpret_cast<uint32_t*>(pool_smem + (size_t)max_oh * max_ow * t.pc * sizeof(PoolVec8<DT>));
    int b = blockIdx.x;
    const int chunk = b % t.chunks; b /= t.chunks;
    const int tw = b % t.tiles_w; b /= t.tiles_w;
    const int th = b % t.tiles_h;
    const int64_t n = b / t.tiles_h;
    const int pc = (g.C8 - chunk * t.pc) < t.pc ? (g.C8 - chunk * t.pc) : t.pc;
    const int ih0 = th * t.th, iw0 = tw * t.tw;
    // output windows that cover some input position of the tile
    auto lo = [&](int i) { const int v = i + g.pad - g.k + 1; return v <= 0 ? 0 : (v + g.s - 1) / g.s; };
    auto hi = [&](int i, int last) { const int v = (i + g.pad) / g.s; return v > last ? last : v; };
    const int ih1 = (ih0 + t.th < g.H ? ih0 + t.th : g.H) - 1, iw1 = (iw0 + t.tw < g.W ? iw0 + t.tw : g.W) - 1;
    const int oh_a = lo(ih0), oh_b = hi(ih1, g.OH - 1), ow_a = lo(iw0), ow_b = hi(iw1, g.OW - 1);
    const int noh = oh_b - oh_a + 1, now = ow_b - ow_a + 1;
    grid_dependency_wait();
    grid_launch_dependents();
    for (int p = threadIdx.x; p < noh * now * pc; p += kPoolThreads) {
        const int piece = p % pc, pix = p / pc;
        const int r = pix / now, c = pix - r * now;
        const int64_t q = ((n * g.OH + oh_a + r) * g.OW + ow_a + c) * g.C8 + chunk * t.pc + piece;
        gtile[p] = pool_load_raw<DT>(dy, q * 8);
        wtile[p] = __ldg(idx + q);
    }
    __syncthreads();
    for (int o = threadIdx.x; o < t.th * t.tw * pc; o += kPoolThreads) {
        const int piece = o % pc, ipix = o / pc;
        const int irow = ipix / t.tw, icol = ipix - irow * t.tw;
        const int ih = ih0 + irow, iw = iw0 + icol;
        if (ih >= g.H || iw >= g.W) continue;
        const int oh_lo = lo(ih), oh_hi = hi(ih, g.OH - 1), ow_lo = lo(iw), ow_hi = hi(iw, g.OW - 1);
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int oh = oh_lo; oh <= oh_hi; ++oh) {
            const uint32_t kh = (uint32_t)(ih - (oh * g.s - g.pad));
            for (int ow = ow_lo; ow <= ow_hi; ++ow) {
                const uint32_t pos = kh * (uint32_t)g.k + (uint32_t)(iw - (ow * g.s - g.pad));
                const int sp = ((oh - oh_a) * now + (ow - ow_a)) * pc + piece;
                const uint32_t word = wtile[sp];
                uint32_t hit = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) hit |= (((word >> (4 * i)) & 0xFu) == pos) ? (1u << i) : 0u;
                if (!hit) continue;
                float f[8];
                pool_widen<DT>(gtile[sp], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) if ((hit >> i) & 1u) acc[i] = __fadd_rn(acc[i], f[i]);
            }
        }
        pool_store8<DT>(dx, (((n * g.H + ih) * g.W + iw) * g.C8 + chunk * t.pc + piece) * 8, acc);
    }
}

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves = 1);   // cabi.cu

static int pool_check(int dtype, int64_t n, int h, int w, int c, int k, int s, int pad, PoolGeom* g) {
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (n < 0 || h <= 0 || w <= 0 || c <= 0) return ACT_ERR_SIZE;
    if ((c & 7) || k < 1 || k > 4 || s < 1 || pad < 0 || 2 * pad > k) return ACT_ERR_UNSUPPORTED;
    if (h + 2 * pad < k || w + 2 * pad < k) return ACT_ERR_SIZE;
    g->H = h; g->W = w; g->C8 = c / 8; g->k = k; g->s = s; g->pad = pad;
    g->OH = (h + 2 * pad - k) / s + 1;
    g->OW = (w + 2 * pad - k) / s + 1;
    if (n > (INT64_MAX >> 8) / ((int64_t)h * w * c)) return ACT_ERR_SIZE;
    return ACT_OK;
}

}  // namespace act

extern "C" int act_maxpool_fwd_cl(const void* x, int dtype, int64_t n, int h, int w, int c, int k, int s, int pad,
                                  void* y, void* idx, void* stream)
{
    using namespace act;
    PoolGeom g;
    const int rc = pool_check(dtype, n, h, w, c, k, s, pad, &g);
    if (rc != ACT_OK) return rc;
    if (n == 0) return ACT_OK;
    if (!x || !y || !idx) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y) & 15 || ((uintptr_t)idx & 3)) return ACT_ERR_ALIGN;
    const int64_t pieces = n * g.OH * g.OW * g.C8;
    const int grid = stream_grid_for((pieces + kPoolThreads - 1) / kPoolThreads, 6);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t* xb = static_cast<const uint8_t*>(x);
    uint8_t* yb = static_cast<uint8_t*>(y);
    uint32_t* ib = static_cast<uint32_t*>(idx);
    cudaError_t e;
    if (k == 3) {
        if (dtype == ACT_DTYPE_F32) e = launch_overlapped(maxpool_fwd_cl_kernel<ACT_DTYPE_F32, 3>, grid, kPoolThreads, st, xb, yb, ib, pieces, g);
        else if (dtype == ACT_DTYPE_BF16) e = launch_overlapped(maxpool_fwd_cl_kernel<ACT_DTYPE_BF16, 3>, grid, kPoolThreads, st, xb, yb, ib, pieces, g);
        else e = launch_overlapped(maxpool_fwd_cl_kernel<ACT_DTYPE_F16, 3>, grid, kPoolThreads, st, xb, yb, ib, pieces, g);
    } else if (dtype == ACT_DTYPE_F32) e = launch_overlapped(maxpool_fwd_cl_kernel<ACT_DTYPE_F32, 0>, grid, kPoolThreads, st, xb, yb, ib, pieces, g);
    else if (dtype == ACT_DTYPE_BF16) e = launch_overlapped(maxpool_fwd_cl_kernel<ACT_DTYPE_BF16, 0>, grid, kPoolThreads, st, xb, yb, ib, pieces, g);
    else e = launch_overlapped(maxpool_fwd_cl_kernel<ACT_DTYPE_F16, 0>, grid, kPoolThreads, st, xb, yb, ib, pieces, g);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_maxpool_bwd_cl(const void* idx, const void* dy, int dtype, int64_t n, int h, int w, int c, int k,
                                  int s, int pad, void* dx, void* stream)
{
    using namespace act;
    PoolGeom g;
    const int rc = pool_check(dtype, n, h, w, c, k, s, pad, &g);
    if (rc != ACT_OK) return rc;
    if (n == 0) return ACT_OK;
    if (!idx || !dy || !dx) return ACT_ERR_NULL;
    if (((uintptr_t)dy | (uintptr_t)dx) & 15 || ((uintptr_t)idx & 3)) return ACT_ERR_ALIGN;
    const int64_t pieces = n * g.H * g.W * g.C8;
    const int grid = stream_grid_for((pieces + kPoolThreads - 1) / kPoolThreads, 6);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t* ib = static_cast<const uint32_t*>(idx);
    const uint8_t* gb = static_cast<const uint8_t*>(dy);
    uint8_t* ob = static_cast<uint8_t*>(dx);
    // tiles of 8 x 32 input positions (8 x 16 for fp32) and up to 64 channels; the gradients and
    // index words of the windows that cover a tile go to shared memory
    PoolTile t;
    t.th = 8; t.tw = dtype == ACT_DTYPE_F32 ? 16 : 32;
    t.pc = g.C8 < 8 ? g.C8 : 8;
    t.chunks = (g.C8 + t.pc - 1) / t.pc;
    t.tiles_h = (g.H + t.th - 1) / t.th; t.tiles_w = (g.W + t.tw - 1) / t.tw;
    const int max_oh = (t.th + g.k - 2) / g.s + 2, max_ow = (t.tw + g.k - 2) / g.s + 2;
    const size_t vec = dtype == ACT_DTYPE_F32 ? 32 : 16;
    const size_t smem = (size_t)max_oh * max_ow * t.pc * (vec + 4);
    const int64_t blocks = n * t.tiles_h * t.tiles_w * t.chunks;
    if (smem <= 48 * 1024 && blocks <= INT32_MAX) {
        if (dtype == ACT_DTYPE_F32) maxpool_bwd_tile_kernel<ACT_DTYPE_F32><<<(unsigned)blocks, kPoolThreads, smem, st>>>(ib, gb, ob, g, t, max_oh, max_ow);
        else if (dtype == ACT_DTYPE_BF16) maxpool_bwd_tile_kernel<ACT_DTYPE_BF16><<<(unsigned)blocks, kPoolThreads, smem, st>>>(ib, gb, ob, g, t, max_oh, max_ow);
        else maxpool_bwd_tile_kernel<ACT_DTYPE_F16><<<(unsigned)blocks, kPoolThreads, smem, st>>>(ib, gb, ob, g, t, max_oh, max_ow);
        return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
    }
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_overlapped(maxpool_bwd_cl_kernel<ACT_DTYPE_F32>, grid, kPoolThreads, st, ib, gb, ob, pieces, g);
    else if (dtype == ACT_DTYPE_BF16) e = launch_overlapped(maxpool_bwd_cl_kernel<ACT_DTYPE_BF16>, grid, kPoolThreads, st, ib, gb, ob, pieces, g);
    else e = launch_overlapped(maxpool_bwd_cl_kernel<ACT_DTYPE_F16>, grid, kPoolThreads, st, ib, gb, ob, pieces, g);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
