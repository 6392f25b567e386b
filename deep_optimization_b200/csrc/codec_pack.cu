// C entry points of the quantise-and-pack kernels: argument checks and dispatch on the
// element type.  The kernels live in codec_pack_kernel.cuh and are instantiated by the
// pack_inst_*.cu files.
#include "codec_pack_kernel.cuh"

namespace act {
extern template cudaError_t launch_pack_bits<ACT_DTYPE_F32>(int bits, int mode, const void* x, const float* noise, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, int flags, float clamp_alpha, cudaStream_t st);
extern template cudaError_t launch_fused<ACT_DTYPE_F32>(int bits, int kind, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, cudaStream_t st);
extern template cudaError_t launch_bn<ACT_DTYPE_F32>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_bn_cl<ACT_DTYPE_F32>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_bn_add<ACT_DTYPE_F32>(int bits, bool nearest, bool channel_minor, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_pack_bits<ACT_DTYPE_BF16>(int bits, int mode, const void* x, const float* noise, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, int flags, float clamp_alpha, cudaStream_t st);
extern template cudaError_t launch_fused<ACT_DTYPE_BF16>(int bits, int kind, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, cudaStream_t st);
extern template cudaError_t launch_bn<ACT_DTYPE_BF16>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_bn_cl<ACT_DTYPE_BF16>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_bn_add<ACT_DTYPE_BF16>(int bits, bool nearest, bool channel_minor, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_pack_bits<ACT_DTYPE_F16>(int bits, int mode, const void* x, const float* noise, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, int flags, float clamp_alpha, cudaStream_t st);
extern template cudaError_t launch_fused<ACT_DTYPE_F16>(int bits, int kind, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, cudaStream_t st);
extern template cudaError_t launch_bn<ACT_DTYPE_F16>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_bn_cl<ACT_DTYPE_F16>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_bn_add<ACT_DTYPE_F16>(int bits, bool nearest, bool channel_minor, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
extern template cudaError_t launch_pack_tiled<ACT_DTYPE_F32>(int bits, bool nearest, const void* x, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, TileArgs ta, cudaStream_t st);
extern template cudaError_t launch_pack_tiled<ACT_DTYPE_BF16>(int bits, bool nearest, const void* x, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, TileArgs ta, cudaStream_t st);
extern template cudaError_t launch_pack_tiled<ACT_DTYPE_F16>(int bits, bool nearest, const void* x, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, TileArgs ta, cudaStream_t st);
// codec_bits3.cu
cudaError_t quant_pack3(const void* x, int dtype, const float* noise, int mode, uint64_t seed, uint64_t offset,
                        void* packed, float* scale, float* mn, int64_t n_elems, int log2_gs, cudaStream_t st);
}  // namespace act

extern "C" int act_quant_pack(const void* x, int dtype, int64_t n_groups, int group_size, int bits,
                              const float* noise, uint64_t seed, uint64_t offset, int flags,
                              float clamp_alpha, void* packed, float* scale, float* mn, void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (bits != 1 && bits != 2 && bits != 3 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (bits == 3 && (flags & ACT_FLAG_REF_COMPAT)) return ACT_ERR_UNSUPPORTED;
    if (n_groups == 0) return ACT_OK;
    if (!x || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)packed | (uintptr_t)noise) & 15) return ACT_ERR_ALIGN;
    if (((uintptr_t)scale | (uintptr_t)mn) & 3) return ACT_ERR_ALIGN;
    if (bits == 3) {
        // bit-plane layout, kernels of their own (codec_bits3.cu)
        int log2_gs = 5;
        while ((1 << log2_gs) < group_size) ++log2_gs;
        const int m3 = (flags & ACT_FLAG_ROUND_NEAREST) ? 2 : (noise ? 1 : 0);
        return quant_pack3(x, dtype, noise, m3, seed, offset, packed, scale, mn, n_groups * group_size, log2_gs,
                           static_cast<cudaStream_t>(stream)) == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
    }

    int mode;
    if (flags & ACT_FLAG_REF_COMPAT) mode = kRefCompat;
    else if (flags & ACT_FLAG_ROUND_NEAREST) mode = kNoiseConst;
    else if (noise) mode = kNoiseTensor;
    else mode = kNoiseHash;

    int log2_L = 0;
    while ((32 << log2_L) < group_size) ++log2_L;
    const int64_t n_elems = n_groups * group_size;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32)
        e = launch_pack_bits<ACT_DTYPE_F32>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    else if (dtype == ACT_DTYPE_BF16)
        e = launch_pack_bits<ACT_DTYPE_BF16>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    else
        e = launch_pack_bits<ACT_DTYPE_F16>(bits, mode, x, noise, packed, scale, mn, n_elems, log2_L, seed, offset, flags, clamp_alpha, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_activation_fwd_quant_pack(const void* x, int dtype, int kind, int64_t n_groups,
                                             int group_size, int bits, uint64_t seed, uint64_t offset,
                                             int flags, void* y, void* packed, float* scale, float* mn,
                                             void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (kind != ACT_KIND_GELU && kind != ACT_KIND_SILU && kind != ACT_KIND_GELU_ERF) return ACT_ERR_UNSUPPORTED;
    if (flags & ~ACT_FLAG_ROUND_NEAREST) return ACT_ERR_UNSUPPORTED;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_groups < 0 || n_groups > (INT64_MAX >> 12)) return ACT_ERR_SIZE;
    if (n_groups == 0) return ACT_OK;
    if (!x || !y || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)packed) & 15) return ACT_ERR_ALIGN;
    int log2_L = 0;
    while ((32 << log2_L) < group_size) ++log2_L;
    const int64_t n = n_groups * group_size;
    const bool nearest = (flags & ACT_FLAG_ROUND_NEAREST) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_fused<ACT_DTYPE_F32>(bits, kind, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_fused<ACT_DTYPE_BF16>(bits, kind, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, st);
    else e = launch_fused<ACT_DTYPE_F16>(bits, kind, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

static int bn_fwd_common(const void* x, int dtype, int64_t n_batch, int channels, int64_t hw,
                         const float* params, int group_size, int bits, uint64_t seed, uint64_t offset,
                         int flags, void* y, void* packed, float* scale, float* mn, void* mask_bits,
                         void* stream, const void* residual = nullptr)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (flags & ~ACT_FLAG_ROUND_NEAREST) return ACT_ERR_UNSUPPORTED;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (n_batch < 0 || channels <= 0 || hw <= 0) return ACT_ERR_SIZE;
    // hw == 1 is the channel-minor layout ([rows, C], a channels-last activation): pieces of
    // eight consecutive channels
    const bool channel_minor = (hw == 1);
    if (channel_minor) {
        if ((channels & 7) || channels > 4096) return ACT_ERR_UNSUPPORTED;     // the table sits in shared memory
    }
    // exactness of the multiply-high channel lookup, and channel-uniform groups of four
    else if ((hw & 3) || (uint64_t)hw * (uint64_t)(hw + 1024) >= (1ull << 32) ||
        (uint64_t)channels * (uint64_t)(channels + 260) >= (1ull << 32)) return ACT_ERR_UNSUPPORTED;
    const int64_t n = n_batch * channels * hw;
    if (n > (INT64_MAX >> 4) || n % group_size) return ACT_ERR_SIZE;
    if (n == 0) return ACT_OK;
    if (!x || !y || !packed || !scale || !mn || !params) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)packed | (uintptr_t)params | (uintptr_t)residual) & 15) return ACT_ERR_ALIGN;
    int log2_L = 0;
    while ((32 << log2_L) < group_size) ++log2_L;
    BNArgs bn{reinterpret_cast<const float4*>(params), (uint32_t)hw, (uint32_t)channels,
              magic_for((uint32_t)hw), magic_for((uint32_t)channels), static_cast<uint8_t*>(mask_bits),
              static_cast<const uint8_t*>(residual)};
    const bool nearest = (flags & ACT_FLAG_ROUND_NEAREST) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (residual) {
        if (dtype == ACT_DTYPE_F32) e = launch_bn_add<ACT_DTYPE_F32>(bits, nearest, channel_minor, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
        else if (dtype == ACT_DTYPE_BF16) e = launch_bn_add<ACT_DTYPE_BF16>(bits, nearest, channel_minor, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
        else e = launch_bn_add<ACT_DTYPE_F16>(bits, nearest, channel_minor, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    }
    else if (channel_minor) {
        if (dtype == ACT_DTYPE_F32) e = launch_bn_cl<ACT_DTYPE_F32>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
        else if (dtype == ACT_DTYPE_BF16) e = launch_bn_cl<ACT_DTYPE_BF16>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
        else e = launch_bn_cl<ACT_DTYPE_F16>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    }
    else if (dtype == ACT_DTYPE_F32) e = launch_bn<ACT_DTYPE_F32>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_bn<ACT_DTYPE_BF16>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    else e = launch_bn<ACT_DTYPE_F16>(bits, nearest, x, y, packed, scale, mn, n, log2_L, seed, offset, bn, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

extern "C" int act_bn_fwd_norm_quant_pack(const void* x, int dtype, int64_t n_batch, int channels, int64_t hw,
                                          const float* params, int group_size, int bits, uint64_t seed,
                                          uint64_t offset, int flags, void* y, void* packed, float* scale,
                                          float* mn, void* stream)
{
    return bn_fwd_common(x, dtype, n_batch, channels, hw, params, group_size, bits, seed, offset, flags, y,
                         packed, scale, mn, nullptr, stream);
}

extern "C" int act_bn_relu_fwd_norm_quant_pack(const void* x, int dtype, int64_t n_batch, int channels,
                                               int64_t hw, const float* params, int group_size, int bits,
                                               uint64_t seed, uint64_t offset, int flags, void* y, void* packed,
                                               float* scale, float* mn, void* mask_bits, void* stream)
{
    if (!mask_bits) return n_batch * channels * hw == 0 ? ACT_OK : ACT_ERR_NULL;
    return bn_fwd_common(x, dtype, n_batch, channels, hw, params, group_size, bits, seed, offset, flags, y,
                         packed, scale, mn, mask_bits, stream);
}

extern "C" int act_bn_add_relu_fwd_norm_quant_pack(const void* x, const void* residual, int dtype, int64_t n_batch,
                                                   int channels, int64_t hw, const float* params, int group_size,
                                                   int bits, uint64_t seed, uint64_t offset, int flags, void* y,
                                                   void* packed, float* scale, float* mn, void* mask_bits,
                                                   void* stream)
{
    if (!mask_bits || !residual) return n_batch * channels * hw == 0 ? ACT_OK : ACT_ERR_NULL;
    return bn_fwd_common(x, dtype, n_batch, channels, hw, params, group_size, bits, seed, offset, flags, y,
                         packed, scale, mn, mask_bits, stream, residual);
}

extern "C" int act_quant_pack_tiles(const void* x, int dtype, int64_t n_planes, int height, int width, int tile,
                                    int bits, uint64_t seed, uint64_t offset, int flags, void* packed,
                                    float* scale, float* mn, void* stream)
{
    using namespace act;
    if (dtype != ACT_DTYPE_F32 && dtype != ACT_DTYPE_BF16 && dtype != ACT_DTYPE_F16) return ACT_ERR_DTYPE;
    if (flags & ~ACT_FLAG_ROUND_NEAREST) return ACT_ERR_UNSUPPORTED;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (tile != 8 && tile != 16 && tile != 32) return ACT_ERR_GROUP;
    if (n_planes < 0 || height <= 0 || width <= 0 || height % tile || width % tile) return ACT_ERR_SIZE;
    const int64_t groups = n_planes * (height / tile) * (width / tile);
    if (n_planes > (1ll << 31) || groups >= (1ll << 32)) return ACT_ERR_SIZE;
    if (groups == 0) return ACT_OK;
    if (!x || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)x | (uintptr_t)packed) & 15) return ACT_ERR_ALIGN;
    if (((uintptr_t)scale | (uintptr_t)mn) & 3) return ACT_ERR_ALIGN;
    int log2_t = 3;
    while ((1 << log2_t) < tile) ++log2_t;
    const int log2_L = 2 * log2_t - 5;                       // lanes per group = tile * tile / 32
    const int64_t n_elems = groups << (2 * log2_t);
    const TileArgs ta{(uint32_t)height, (uint32_t)width, (uint32_t)(width / tile), (uint32_t)(height / tile), log2_t};
    const bool nearest = (flags & ACT_FLAG_ROUND_NEAREST) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == ACT_DTYPE_F32) e = launch_pack_tiled<ACT_DTYPE_F32>(bits, nearest, x, packed, scale, mn, n_elems, log2_L, seed, offset, ta, st);
    else if (dtype == ACT_DTYPE_BF16) e = launch_pack_tiled<ACT_DTYPE_BF16>(bits, nearest, x, packed, scale, mn, n_elems, log2_L, seed, offset, ta, st);
    else e = launch_pack_tiled<ACT_DTYPE_F16>(bits, nearest, x, packed, scale, mn, n_elems, log2_L, seed, offset, ta, st);
    return e == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
