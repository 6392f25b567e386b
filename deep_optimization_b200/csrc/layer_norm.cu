// Column reductions over a row-major [rows, C] tensor, sm_100a:
//
//   act_col_sum:        out[c] = sum_r a[r, c]                                   (the bias gradient of a
//                       linear layer: dy summed over its rows)
//   act_ln_bwd_params:  dgamma[c] = sum_r dy[r, c] * (x[r, c] - mean[r]) * rstd[r]
//                       dbeta[c]  = sum_r dy[r, c]                               (the weight and bias
//                       gradients of a LayerNorm over the last dimension)
//
// A thread owns eight consecutive columns (one 16-byte vector of 16-bit elements per row) and walks
// the rows of its block's slice, four rows' loads in flight; tpr = min(C/8, 256) threads cover one
// row (or 2048 columns of it, blockIdx.x choosing which) and the block's other threads take the
// following rows, so a warp reads contiguous memory.  Sixteen fp32 accumulators per thread; at the
// end the threads of a column vector are summed through shared memory and every column leaves once
// per block with coalesced atomics into the zeroed outputs.  HBM traffic: every input byte once.
// The layer-norm form reads mean and rstd of a row once per thread and row (a broadcast load).
//
// These are what ATen's GammaBetaBackward and sum kernels compute for
// Activation_Compression/modules/ops.py:496-526 (db) and for a LayerNorm whose input was saved
// compressed; on bf16 [50432, 768] ATen needs 430 us for the first and 62 us for the second.
#include "act_common.cuh"

namespace act {

constexpr int kColThreads = 256;

int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves = 1);   // cabi.cu

// eight consecutive elements starting at p, widened to fp32
template <int DT> __device__ __forceinline__ void load8(const uint8_t* p, float (&f)[8]) {
    if (ElemT<DT>::bytes == 4) {
        const uint4 a = ldg_stream_v4(p), b = ldg_stream_v4(p + 16);
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    } else {
        constexpr int D16 = (DT == ACT_DTYPE_F32) ? ACT_DTYPE_BF16 : DT;
        const uint4 a = ldg_stream_v4(p);
        const uint32_t h[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { f[2 * k] = widen_lo<D16>(h[k]); f[2 * k + 1] = widen_hi<D16>(h[k]); }
    }
}

// LN = false: out0[c] += sum_r a[r, c].
// LN = true:  out0[c] += sum_r a[r, c] * (b[r, c] - mean[r]) * rstd[r],  out1[c] += sum_r a[r, c].
template <int DT, bool LN>
__global__ void __launch_bounds__(kColThreads)
col_reduce_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, const float* __restrict__ mean,
                  const float* __restrict__ rstd, float* __restrict__ out0, float* __restrict__ out1,
                  int64_t n_rows, uint32_t C, uint32_t tpr)
{
    __shared__ float s_acc[16][kColThreads + 1];
    const uint32_t s = blockIdx.y, S = gridDim.y;
    const uint32_t rpi = kColThreads / tpr;                  // rows per block step
    const uint32_t q = threadIdx.x % tpr, rl = threadIdx.x / tpr;
    const uint32_t chunk = blockIdx.x * tpr + q;             // which vector of eight columns
    const bool active = rl < rpi && chunk * 8u < C;
    const int64_t r0 = n_rows * s / S, r1 = n_rows * (s + 1) / S;
    float acc0[8], acc1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc0[i] = 0.0f; acc1[i] = 0.0f; }
    if (active) {
        constexpr int U = 4;
        constexpr int EB = ElemT<DT>::bytes;
        for (int64_t r = r0 + rl; r < r1; r += (int64_t)U * rpi) {
            float fa[U][8], fb[U][8], mu[U], rs[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t row = r + (int64_t)u * rpi;
                if (row < r1) {
                    const int64_t e = row * C + (int64_t)chunk * 8;
                    load8<DT>(a + e * EB, fa[u]);
                    if (LN) { load8<DT>(b + e * EB, fb[u]); mu[u] = __ldg(mean + row); rs[u] = __ldg(rstd + row); }
                } else {
                    // a row past the end holds zeros and adds nothing
#pragma unroll
                    for (int i = 0; i < 8; ++i) { fa[u][i] = 0.0f; fb[u][i] = 0.0f; }
                    mu[u] = 0.0f; rs[u] = 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (LN) {
                        const float xh = __fmul_rn(__fsub_rn(fb[u][i], mu[u]), rs[u]);
                        acc0[i] = __fmaf_rn(fa[u][i], xh, acc0[i]);
                        acc1[i] = __fadd_rn(acc1[i], fa[u][i]);
                    } else {
                        acc0[i] = __fadd_rn(acc0[i], fa[u][i]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { s_acc[i][threadIdx.x] = acc0[i]; s_acc[8 + i][threadIdx.x] = acc1[i]; }
    __syncthreads();
    // column cl of the block's tile: vector cl / 8, element cl % 8, summed over the row lanes
    const uint32_t tile_c = tpr * 8u, c_base = blockIdx.x * tile_c;
    for (uint32_t cl = threadIdx.x; cl < tile_c && c_base + cl < C; cl += kColThreads) {
        const uint32_t v = cl >> 3, i = cl & 7u;
        float t0 = 0.0f, t1 = 0.0f;
        for (uint32_t l = 0; l < rpi; ++l) { t0 += s_acc[i][l * tpr + v]; if (LN) t1 += s_acc[8 + i][l * tpr + v]; }
        atomicAdd(out0 + c_base + cl, t0);
        if (LN) atomicAdd(out1 + c_base + cl, t1);
    }
}

template <int DT, bool LN>
int launch_col_reduce(const void* a, const void* b, const float* mean, const float* rstd, float* out0, float* out1,
                      int64_t rows, int C, cudaStream_t st)
{
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, col_reduce_kernel<DT, LN>, kColThreads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    const uint32_t vecs = (uint32_t)C / 8u;
    // threads per row: the width that leaves the fewest threads idle (row lanes that do not fit a
    // block, vectors past the last column), the widest such one.  With min(vecs, 256): 288 vectors
    // ran two blocks of which the second used 32 of its 256 threads.
    uint32_t tpr = 1;
    {
        const uint32_t T = (uint32_t)kColThreads, hi = vecs < T ? vecs : T;
        uint64_t best_num = 0, best_den = 1;
        for (uint32_t t = 1; t <= hi; ++t) {
            const uint64_t num = (uint64_t)t * (T / t) * vecs, den = (uint64_t)T * ((vecs + t - 1) / t) * t;
            if (num * best_den >= best_num * den) { best_num = num; best_den = den; tpr = t; }
        }
    }
    const uint32_t gx = (vecs + tpr - 1) / tpr;
    const uint32_t rpi = kColThreads / tpr;
    // slices of the rows: one resident wave of blocks, never a slice shorter than one block step
    int64_t slices = stream_grid_for((int64_t)1 << 30, per_sm) / gx;
    const int64_t max_slices = (rows + rpi - 1) / rpi;
    if (slices > max_slices) slices = max_slices;
    if (slices < 1) slices = 1;
    if (slices > 65535) slices = 65535;
    if (cudaMemsetAsync(out0, 0, (size_t)C * sizeof(float), st) != cudaSuccess) return ACT_ERR_LAUNCH;
    if (LN && cudaMemsetAsync(out1, 0, (size_t)C * sizeof(float), st) != cudaSuccess) return ACT_ERR_LAUNCH;
    col_reduce_kernel<DT, LN><<<dim3(gx, (unsigned)slices), kColThreads, 0, st>>>(
        static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), mean, rstd, out0, out1, rows, (uint32_t)C, tpr);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

static int check_cols(const void* p, int dtype, int64_t rows, int C) {
    if (rows < 0 || C < 0) return ACT_ERR_SIZE;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (C & 7) return ACT_ERR_SIZE;                          // whole vectors of eight columns
    if ((uintptr_t)p & 15) return ACT_ERR_ALIGN;
    return ACT_OK;
}

}  // namespace act

extern "C" int act_col_sum(const void* a, int dtype, int64_t rows, int cols, float* out, void* stream) {
    using namespace act;
    const int rc = check_cols(a, dtype, rows, cols);
    if (rc != ACT_OK) return rc;
    if (cols == 0) return ACT_OK;
    if (!out || (rows > 0 && !a)) return ACT_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) return cudaMemsetAsync(out, 0, (size_t)cols * sizeof(float), st) == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
    switch (dtype) {
        case ACT_DTYPE_F32: return launch_col_reduce<ACT_DTYPE_F32, false>(a, nullptr, nullptr, nullptr, out, nullptr, rows, cols, st);
        case ACT_DTYPE_BF16: return launch_col_reduce<ACT_DTYPE_BF16, false>(a, nullptr, nullptr, nullptr, out, nullptr, rows, cols, st);
        default: return launch_col_reduce<ACT_DTYPE_F16, false>(a, nullptr, nullptr, nullptr, out, nullptr, rows, cols, st);
    }
}

extern "C" int act_ln_bwd_params(const void* dy, const void* x, const float* mean, const float* rstd, int dtype,
                                 int64_t rows, int cols, float* dgamma, float* dbeta, void* stream)
{
    using namespace act;
    int rc = check_cols(dy, dtype, rows, cols);
    if (rc != ACT_OK) return rc;
    if ((uintptr_t)x & 15) return ACT_ERR_ALIGN;
    if (cols == 0) return ACT_OK;
    if (!dgamma || !dbeta || (rows > 0 && (!dy || !x || !mean || !rstd))) return ACT_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        if (cudaMemsetAsync(dgamma, 0, (size_t)cols * sizeof(float), st) != cudaSuccess ||
            cudaMemsetAsync(dbeta, 0, (size_t)cols * sizeof(float), st) != cudaSuccess) return ACT_ERR_LAUNCH;
        return ACT_OK;
    }
    switch (dtype) {
        case ACT_DTYPE_F32: return launch_col_reduce<ACT_DTYPE_F32, true>(dy, x, mean, rstd, dgamma, dbeta, rows, cols, st);
        case ACT_DTYPE_BF16: return launch_col_reduce<ACT_DTYPE_BF16, true>(dy, x, mean, rstd, dgamma, dbeta, rows, cols, st);
        default: return launch_col_reduce<ACT_DTYPE_F16, true>(dy, x, mean, rstd, dgamma, dbeta, rows, cols, st);
    }
}

// ------------------------------------------------------------------ gradient of the q/k/v split
// act_merge_heads: dst[b, t, s, h, :] = src_s[b, h, t, :] for s = 0..parts-1, dst contiguous
// [B, T, parts, H, Dh], the sources given by their element strides for b, h and t (last dimension
// contiguous).  This is the backward of
//     q, k, v = qkv.view(B, T, 3, H, Dh).permute(2, 0, 3, 1, 4).unbind(0)
// (Model/ViT/ViT.py:39-42 of the reference): the three gradients an attention kernel returns
// become the gradient of the qkv projection's output in one pass (232 MB each way for ViT-B/16 at
// batch 256), where autograd runs a stack of the three and a strided copy of the result (557 +
// 292 us).  A block takes whole rows (b, t); a thread keeps its (s, h, 16-byte piece) and walks
// the block's rows, so eight lanes read one 128-byte run of a source and a warp writes 512
// contiguous bytes.
namespace act {

struct MergeSrc {
    const uint8_t* p[4];
    int64_t sb[4], sh[4], st[4];          // byte strides
};

__global__ void __launch_bounds__(1024)
merge_heads_kernel(MergeSrc src, uint8_t* __restrict__ dst, int B, int T, int H, int parts, int pieces_per_head,
                   int rows_per_block)
{
    const int per_row = parts * H * pieces_per_head;         // 16-byte pieces of one (b, t) row of dst
    const int64_t rows = (int64_t)B * T;
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_block;
    for (int piece = threadIdx.x; piece < per_row; piece += blockDim.x) {
        const int s = piece / (H * pieces_per_head);
        const int rem = piece - s * (H * pieces_per_head);
        const int h = rem / pieces_per_head, pp = rem - h * pieces_per_head;
        const uint8_t* base = src.p[s] + (int64_t)h * src.sh[s] + (int64_t)pp * 16;
        for (int r = 0; r < rows_per_block; ++r) {
            const int64_t row = row0 + r;
            if (row >= rows) break;
            const int64_t b = row / T, t = row - b * T;
            const uint4 v = ldg_stream_v4(base + b * src.sb[s] + t * src.st[s]);
            stg_stream_v4(dst + (row * per_row + piece) * 16, v);
        }
    }
}

}  // namespace act

extern "C" int act_merge_heads(const void* const* srcs, const int64_t* strides, int parts, int B, int H, int T,
                               int Dh, int elem_bytes, void* dst, void* stream)
{
    using namespace act;
    if (parts < 1 || parts > 4 || B < 0 || H < 0 || T < 0 || Dh < 0) return ACT_ERR_SIZE;
    if (elem_bytes != 2 && elem_bytes != 4) return ACT_ERR_DTYPE;
    if (B == 0 || H == 0 || T == 0 || Dh == 0) return ACT_OK;
    if (!srcs || !strides || !dst) return ACT_ERR_NULL;
    if (((int64_t)Dh * elem_bytes) & 15) return ACT_ERR_SIZE;              // whole 16-byte pieces per head
    if ((uintptr_t)dst & 15) return ACT_ERR_ALIGN;
    MergeSrc ms;
    for (int s = 0; s < 4; ++s) { ms.p[s] = nullptr; ms.sb[s] = ms.sh[s] = ms.st[s] = 0; }
    for (int s = 0; s < parts; ++s) {
        if (!srcs[s]) return ACT_ERR_NULL;
        ms.p[s] = static_cast<const uint8_t*>(srcs[s]);
        ms.sb[s] = strides[3 * s] * elem_bytes; ms.sh[s] = strides[3 * s + 1] * elem_bytes; ms.st[s] = strides[3 * s + 2] * elem_bytes;
        if (((uintptr_t)ms.p[s] | (uint64_t)ms.sb[s] | (uint64_t)ms.sh[s] | (uint64_t)ms.st[s]) & 15) return ACT_ERR_ALIGN;
    }
    const int64_t rows = (int64_t)B * T;
    const int pieces_per_head = Dh * elem_bytes / 16;
    // about eight resident waves of blocks: a block's rows are contiguous in dst
    int64_t blocks = stream_grid_for(rows, 8, 8);
    const int rows_per_block = (int)((rows + blocks - 1) / blocks);
    blocks = (rows + rows_per_block - 1) / rows_per_block;
    // one thread per 16-byte piece of a row where a block can hold that many
    const int per_row = parts * H * pieces_per_head;
    const int threads = per_row <= 1024 ? ((per_row + 31) & ~31) : 256;
    merge_heads_kernel<<<(unsigned)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        ms, static_cast<uint8_t*>(dst), B, T, H, parts, pieces_per_head, rows_per_block);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
