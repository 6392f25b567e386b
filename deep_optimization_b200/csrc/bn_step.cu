// Whole forward and backward of one fused batch-norm layer behind one call each: the host
// composition of the entry points in bn_reduce.cu, codec_pack.cu and fused_act.cu.  A training
// step of ResNet-50 makes 53 of each; issuing the three to five launches of a layer from one
// C call (instead of one Python-to-C round trip, argument marshalling and temporary allocation
// per launch) takes about 2 ms of host time out of a 27 ms step.
#include "act_common.cuh"

// Forward: statistics (+ running statistics), then normalise + affine (+ residual) (+ ReLU) +
// x_hat codec.  mask_bits may be NULL (no ReLU); residual needs mask_bits.
extern "C" int act_bn_forward(const void* x, const void* residual, int dtype, int64_t n_batch, int channels,
                              int64_t hw, double eps, const float* weight, const float* bias,
                              float* running_mean, float* running_var, double momentum, float* params,
                              void* workspace, size_t ws_bytes, int group_size, int bits, uint64_t seed,
                              uint64_t offset, int flags, void* y, void* packed, float* scale, float* mn,
                              void* mask_bits, void* stream)
{
    int rc = act_bn_stats(x, dtype, n_batch, channels, hw, eps, weight, bias, running_mean, running_var,
                          momentum, params, workspace, ws_bytes, stream);
    if (rc != ACT_OK) return rc;
    if (residual)
        return act_bn_add_relu_fwd_norm_quant_pack(x, residual, dtype, n_batch, channels, hw, params, group_size,
                                                   bits, seed, offset, flags, y, packed, scale, mn, mask_bits, stream);
    if (mask_bits)
        return act_bn_relu_fwd_norm_quant_pack(x, dtype, n_batch, channels, hw, params, group_size, bits, seed,
                                               offset, flags, y, packed, scale, mn, mask_bits, stream);
    return act_bn_fwd_norm_quant_pack(x, dtype, n_batch, channels, hw, params, group_size, bits, seed, offset,
                                      flags, y, packed, scale, mn, stream);
}

// Backward: sums = (sum dy*x_hat, sum dy) per channel [2C] (zeroed here), coef [C][4], dx.
// mask_bits NULL: plain batch norm.  mask_bits with dy_masked NULL: BN + ReLU, the two kernels
// read dy through the mask.  mask_bits with dy_masked: BN + residual + ReLU; dy under the mask
// is written to dy_masked first (act_bn_add_relu_bwd_reduce; the residual's gradient) and is
// what the dx kernel reads.
extern "C" int act_bn_backward_sum(const void* packed, const float* scale, const float* mn, const void* dy,
                                   const void* dy2, const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                               int group_size, int bits, const float* params, double count, float* sums,
                               float* coef, void* dy_masked, void* dx, void* stream)
{
    if (channels <= 0 || !sums) return ACT_ERR_NULL;
    if (dy2 && !(mask_bits && dy_masked)) return ACT_ERR_UNSUPPORTED;     // the second gradient rides in the mask pass
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(sums, 0, (size_t)channels * 2 * sizeof(float), st) != cudaSuccess) return ACT_ERR_LAUNCH;
    int rc;
    if (mask_bits && dy_masked) {
        rc = act_bn_add_relu_bwd_reduce_sum(packed, scale, mn, dy, dy2, mask_bits, dtype, n_batch, channels, hw,
                                            group_size, bits, sums, dy_masked, stream);
        if (rc != ACT_OK) return rc;
        rc = act_bn_bwd_coef(sums, params, channels, count, coef, stream);
        if (rc != ACT_OK) return rc;
        return act_bn_bwd_dx(packed, scale, mn, dy_masked, dtype, n_batch, channels, hw, group_size, bits, coef, dx, stream);
    }
    if (mask_bits) rc = act_bn_relu_bwd_reduce(packed, scale, mn, dy, mask_bits, dtype, n_batch, channels, hw, group_size, bits, sums, stream);
    else rc = act_bn_bwd_reduce(packed, scale, mn, dy, dtype, n_batch, channels, hw, group_size, bits, sums, stream);
    if (rc != ACT_OK) return rc;
    rc = act_bn_bwd_coef(sums, params, channels, count, coef, stream);
    if (rc != ACT_OK) return rc;
    if (mask_bits) return act_bn_relu_bwd_dx(packed, scale, mn, dy, mask_bits, dtype, n_batch, channels, hw, group_size, bits, coef, dx, stream);
    return act_bn_bwd_dx(packed, scale, mn, dy, dtype, n_batch, channels, hw, group_size, bits, coef, dx, stream);
}

extern "C" int act_bn_backward(const void* packed, const float* scale, const float* mn, const void* dy,
                               const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                               int group_size, int bits, const float* params, double count, float* sums,
                               float* coef, void* dy_masked, void* dx, void* stream)
{
    return act_bn_backward_sum(packed, scale, mn, dy, nullptr, mask_bits, dtype, n_batch, channels, hw, group_size, bits,
                               params, count, sums, coef, dy_masked, dx, stream);
}
