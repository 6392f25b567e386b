// Host-side pieces of the C ABI that are not a kernel launcher: grid sizing,
// error text, and the host-only greedy bit allocator.
#include <queue>
#include <utility>
#include <vector>

#include "act_common.cuh"

namespace act {

// SM count of the current device, looked up once per device.
static int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev];
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return n;
}

// Grid of a kernel that walks its tiles with a grid stride: `waves` resident waves of
// blocks_per_sm blocks per SM (fewer for small inputs).  The encoders run fastest as exactly one
// wave (20.7 us per launch on the bench workload against 23.3 at four); the decoders, which
// mostly write, as about four (dequant_unpack 23.9 -> 21.7 us, GELU backward 157 -> 123 us,
// ReLU forward and backward 39.5 -> 35.5 us): their blocks then finish at different times and the
// last writes of the launch no longer arrive together.
int stream_grid_for(int64_t n_blocks_wanted, int blocks_per_sm, int waves) {
    const int64_t wave = (int64_t)sm_count() * blocks_per_sm * (waves < 1 ? 1 : waves);
    int64_t g = n_blocks_wanted < wave ? n_blocks_wanted : wave;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace act

extern "C" const char* act_strerror(int code) {
    switch (code) {
        case ACT_OK: return "ok";
        case ACT_ERR_DTYPE: return "unknown element type (expected ACT_DTYPE_F32/BF16/F16)";
        case ACT_ERR_BITS: return "bits must be one of (1,2,4,8)";
        case ACT_ERR_GROUP: return "group size must be a power of two in [32,1024]";
        case ACT_ERR_ALIGN: return "pointer not aligned (activations, noise and packed buffers need 16 bytes)";
        case ACT_ERR_SIZE: return "negative or overflowing size, or bad leading dimension";
        case ACT_ERR_NULL: return "a required pointer is NULL";
        case ACT_ERR_LAUNCH: return "CUDA refused the kernel launch";
        case ACT_ERR_WORKSPACE: return "workspace too small";
        case ACT_ERR_DEVICE: return "device is not sm_100 or a driver entry point is missing";
        case ACT_ERR_TARGET: return "calc_precision: target cannot be reached";
        case ACT_ERR_UNSUPPORTED: return "flag combination not supported";
        case ACT_ERR_STATIC_LIMIT: return "problem too large for the built-in scratch of act_fp8_gemm_static (N*K over 4 MiB)";
        default: return "unknown error code";
    }
}

// 2: hash and round-to-nearest modes are fixed-point (8 fraction bits, noise bytes); entry
// points added for batch-norm statistics, BN+ReLU, backward constants and tiled addressing
extern "C" int act_abi_version(void) { return 2; }

// Greedy bit allocation.  Every layer i starts at b[i] bits and weighs w[i]; the
// layer whose variance term C*(1/(2^b-1)^2 - 1/(2^(b-1)-1)^2) grows least loses
// one bit, until sum(b*w) <= target.  Integer reads, b/w integer division and
// the (delta, index) max-heap tie-break follow
// Activation_Compression/cpp_extension/src/calc_precision.cc:10-53.
extern "C" int act_calc_precision(int32_t* b, const int32_t* C, const int32_t* w, int64_t n,
                                  double target)
{
    if (n < 0) return ACT_ERR_SIZE;
    if (n == 0) return ACT_OK;
    if (!b || !C || !w) return ACT_ERR_NULL;
    auto delta = [](float c, int bits) -> float {
        const int c1 = ((1 << bits) - 1) * ((1 << bits) - 1);
        const int c2 = ((1 << (bits - 1)) - 1) * ((1 << (bits - 1)) - 1);
        return (float)(c * (1.0 / c1 - 1.0 / c2));
    };
    std::priority_queue<std::pair<float, int64_t>> heap;
    double total = 0;
    for (int64_t i = 0; i < n; ++i) {
        if (w[i] == 0) return ACT_ERR_SIZE;
        heap.push(std::make_pair(delta((float)C[i], b[i] / w[i]), i));
        total += (double)b[i] * w[i];
    }
    while (total > target) {
        if (heap.empty()) return ACT_ERR_TARGET;
        const int64_t i = heap.top().second;
        heap.pop();
        b[i] -= 1;
        total -= w[i];
        if (b[i] > 1) heap.push(std::make_pair(delta((float)C[i], b[i] / w[i]), i));
    }
    return ACT_OK;
}

// Clears nbytes at p on the caller's stream (the runtime's own memset).  For hosts that bind this
// library but not the CUDA runtime; bench.py also times it as the pace of a pure write stream,
// the yardstick for the kernels here that mostly write.
extern "C" int act_fill_zero(void* p, size_t nbytes, void* stream) {
    if (nbytes == 0) return ACT_OK;
    if (!p) return ACT_ERR_NULL;
    return cudaMemsetAsync(p, 0, nbytes, static_cast<cudaStream_t>(stream)) == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}
