// quant_pack_kernel instantiations for ACT_DTYPE_F16 inputs (fused GELU / SiLU producers)
#include "codec_pack_kernel.cuh"
namespace act {
template cudaError_t launch_fused<ACT_DTYPE_F16>(int bits, int kind, bool nearest, const void* x, void* y, void* packed, float* scale, float* mn, int64_t n, int l2, uint64_t seed, uint64_t offset, cudaStream_t st);
}  // namespace act
