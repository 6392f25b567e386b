// quant_pack_kernel instantiations for ACT_DTYPE_F16 inputs (fused batch-norm producer, channel-minor layout)
#include "codec_pack_kernel.cuh"
namespace act {
template cudaError_t launch_bn_cl<ACT_DTYPE_F16>(int bits, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, BNArgs bn, cudaStream_t st);
}  // namespace act
