// quant_pack_kernel instantiations for ACT_DTYPE_F16 inputs (plain codec)
#include "codec_pack_kernel.cuh"
namespace act {
template cudaError_t launch_pack_bits<ACT_DTYPE_F16>(int bits, int mode, const void* x, const float* noise, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, int flags, float clamp_alpha, cudaStream_t st);
}  // namespace act
