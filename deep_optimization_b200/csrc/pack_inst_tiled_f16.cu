// quant_pack_kernel instantiations for ACT_DTYPE_F16 inputs (tiled source addressing)
#include "codec_pack_kernel.cuh"
namespace act {
template cudaError_t launch_pack_tiled<ACT_DTYPE_F16>(int bits, bool nearest, const void* x, void* packed, float* scale, float* mn, int64_t n_elems, int log2_L, uint64_t seed, uint64_t offset, TileArgs ta, cudaStream_t st);
}  // namespace act
