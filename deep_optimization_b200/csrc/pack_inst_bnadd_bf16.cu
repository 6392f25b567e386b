// quant_pack_kernel instantiations for ACT_DTYPE_BF16 inputs (batch norm + residual add + ReLU producer)
#include "codec_pack_kernel.cuh"
namespace act {
template cudaError_t launch_bn_add<ACT_DTYPE_BF16>(int bits, bool nearest, bool channel_minor, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
}  // namespace act
