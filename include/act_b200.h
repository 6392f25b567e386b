/*
 * act_b200.h -- C ABI of the B200 (sm_100a) activation-compression library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (cudaStream_t passed as void*; NULL is the legacy default stream) and returns
 * 0 or one of the ACT_ERR_* codes.  Unless an entry point says otherwise the
 * library allocates nothing, keeps no pointer past the return, never
 * synchronises the host and launches on the stream it is given, so calls can be
 * captured into CUDA graphs.  All buffers belong to the caller.  The device is
 * the caller's current device.
 *
 * Each declaration names the interface of the Deep_Optimization project it
 * replaces (paths are inside that project; "AC/" = Activation_Compression/).
 */
#ifndef ACT_B200_H
#define ACT_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define ACT_API __attribute__((visibility("default")))
#else
#define ACT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations */
#define ACT_DTYPE_F32  0
#define ACT_DTYPE_BF16 1
#define ACT_DTYPE_F16  2

/* flags of act_quant_pack */
#define ACT_FLAG_ROUND_NEAREST 1   /* no noise: round to nearest (constant of AC/act_triton_kernel.py:114) */
#define ACT_FLAG_REF_COMPAT    2   /* live-Triton arithmetic: a*(1/s)+c, truncate                    */
#define ACT_FLAG_REF_CLAMP     4   /* with REF_COMPAT: clamp x to +-clamp_alpha first                */
#define ACT_FLAG_REF_TANH      8   /* with REF_COMPAT: x = tanh(x/0.5)*0.5 before the range          */
#define ACT_FLAG_META_BF16     16  /* round scale and min to bf16 precision (still stored as fp32)   */
#define ACT_FLAG_BALLOT_REF_BIAS 32 /* act_pack_ballot: keep the reference's extra -0.5 in the rounding */

/* activation kinds of act_activation_fwd_quant_pack */
#define ACT_KIND_GELU 1            /* tanh-approximated GELU */
#define ACT_KIND_SILU 2
#define ACT_KIND_GELU_ERF 3        /* exact GELU, x * Phi(x) */

/* flags of act_fp8_gemm */
#define ACT_GEMM_B_IS_NK 1         /* B is stored [N,K] (K contiguous, like nn.Linear weights)        */
#define ACT_GEMM_SINGLE_CTA 2      /* one CTA per 128x256 tile instead of CTA pairs on 256x256 tiles  */

/* return codes */
#define ACT_OK             0
#define ACT_ERR_DTYPE      1   /* unknown element type                                   */
#define ACT_ERR_BITS       2   /* bits not in {1,2,4,8}                                  */
#define ACT_ERR_GROUP      3   /* group size not a power of two in [32,1024]             */
#define ACT_ERR_ALIGN      4   /* a pointer is not aligned as documented                 */
#define ACT_ERR_SIZE       5   /* negative or overflowing size, bad leading dimension    */
#define ACT_ERR_NULL       6   /* a required pointer is NULL                             */
#define ACT_ERR_LAUNCH     7   /* the CUDA runtime refused the launch (see cudaGetLastError) */
#define ACT_ERR_WORKSPACE  8   /* workspace too small                                    */
#define ACT_ERR_DEVICE     9   /* not an sm_100 device, or a driver entry point missing  */
#define ACT_ERR_TARGET    10   /* act_calc_precision: target cannot be reached           */
#define ACT_ERR_UNSUPPORTED 11 /* flag combination not built                             */
#define ACT_ERR_STATIC_LIMIT 12 /* act_fp8_gemm_static: N*K exceeds the built-in scratch */

/*
 * Per-group quantise-and-pack of a saved activation.
 * Replaces torch.ops.act_lib.quant_pack_triton (AC/act_triton_kernel.py:336-368,
 * kernel :23-171) and cpp_extension.pack{1,2,3,4,8} (AC/cpp_extension/bind.cpp:10-14).
 *
 *   x       [n_groups, group_size] of `dtype`, contiguous, 16-byte aligned
 *   noise   NULL, or fp32 [n_groups, group_size] of u in [0,1), 16-byte aligned
 *   seed, offset   used when noise == NULL and ACT_FLAG_ROUND_NEAREST is clear: element e
 *           takes the noise byte h = byte (e & 7) of hash(e >> 3; key(seed, offset)); seed picks
 *           a family of streams, offset one stream (advance it per call)
 *   packed  n_groups*group_size*bits/8 bytes, 16-byte aligned; 32-bit little-endian
 *           words, code j of a word at bits [j*bits,(j+1)*bits)
 *   scale, min   fp32 [n_groups]
 *
 * Per group: min and max (-0 < +0, a NaN makes min NaN, scale 1, codes 0),
 * s = (max-min)/(2^bits-1) in IEEE binary32, s = 1 if that is not positive.  Codes:
 *   noise given:  code = clamp(floor((x-min)/s + u), 0, 2^bits-1), every operation IEEE
 *                 binary32 round-to-nearest, nothing fused;
 *   noise NULL:   fixed point with 8 fraction bits for a group whose range is 0 or in
 *                 [2^-50, 2^50]: Q = RNE((x-min) * RN(1/s) * 256) rounded once (the low mantissa
 *                 bits of fmaf(x-min, RN(1/s), 2^15)), code = (Q + h) >> 8, which cannot exceed
 *                 2^bits-1; h is the noise byte, or the constant 127 with
 *                 ACT_FLAG_ROUND_NEAREST (0.5f-1e-6f on the 1/256 grid, a tie going down).
 *                 Any other group uses the formula of the first case with u = h/256
 *                 (u = 0.5f-1e-6f for round to nearest).
 * bits = 3 (cpp_extension.pack3 / unpack3, AC/cpp_extension/bind.cpp:12,18) is taken too, with
 * the same arithmetic (eight levels) and a bit-plane layout, since 3-bit codes do not fill a
 * word: every 32 consecutive elements take three consecutive words, bit l of word p = bit p of
 * the code of element l (the reference's kernel stores planes too, in its ballot order).  Not
 * with ACT_FLAG_REF_COMPAT.  act_dequant_unpack reads the same layout.
 */
ACT_API int act_quant_pack(const void* x, int dtype, int64_t n_groups, int group_size, int bits,
                   const float* noise, uint64_t seed, uint64_t offset, int flags,
                   float clamp_alpha, void* packed, float* scale, float* min, void* stream);

/*
 * Unpack-and-dequantise: y = fma(code, scale, min) rounded to `out_dtype`.
 * Replaces torch.ops.act_lib.dequant_unpack_triton (AC/act_triton_kernel.py:372-395,
 * kernel :174-241) and cpp_extension.unpack{1,2,3,4,8} (AC/cpp_extension/bind.cpp:16-20).
 *   y  [n_groups, group_size] of out_dtype, 16-byte aligned.
 */
ACT_API int act_dequant_unpack(const void* packed, const float* scale, const float* min,
                       int64_t n_groups, int group_size, int bits, int out_dtype, void* y,
                       void* stream);

/*
 * Sub-group averaging, the AVG_ALAM switch of the reference's live kernels
 * (AC/act_triton_kernel.py:116-118 and :212-215): `avg` (2, 4 or 8) consecutive elements of a
 * group share one code, so packed holds group_size*bits/(32*avg) words per group (a whole
 * number, else ACT_ERR_GROUP) and decoding repeats every code avg times.  min, max and scale as
 * in act_quant_pack.  With ACT_FLAG_REF_COMPAT: qf_i = RN(RN((x_i-min) * RN(1/s)) + (0.5f-1e-6f)),
 * m = (qf_0 + ... + qf_{avg-1}) / avg summed left to right in fp32, code = clamp(trunc(m))
 * (clamp, tanh and bf16-meta flags as in act_quant_pack).  Otherwise q_i = RN((x_i-min) / s),
 * m likewise, code = clamp(floor(RN(m + u))) with u the noise of the sub-group's first
 * element: its noise-tensor value, its hash byte / 256, or 0.5f-1e-6f for round to nearest.
 * The reference sums in a tree and its decoder adds Gaussian noise to the codes; neither is
 * reproduced.
 */
ACT_API int act_quant_pack_avg(const void* x, int dtype, int64_t n_groups, int group_size, int bits, int avg,
                       const float* noise, uint64_t seed, uint64_t offset, int flags,
                       float clamp_alpha, void* packed, float* scale, float* min, void* stream);
ACT_API int act_dequant_unpack_avg(const void* packed, const float* scale, const float* min, int64_t n_groups,
                           int group_size, int bits, int avg, int out_dtype, void* y, void* stream);

/*
 * The same two kernels on spatial tiles, without the permute-and-copy the reference makes first
 * (AC/modules/tensor_act_reshape_utils.py:82-154): x and y are [n_planes, height, width]
 * (n_planes = N*C), a group is one tile x tile block of one plane (tile = 8, 16 or 32, i.e.
 * group sizes 64, 256, 1024; height and width multiples of tile), group index
 * (plane * height/tile + ty) * width/tile + tx, elements row-major inside the tile.  packed,
 * scale and min are exactly those of act_quant_pack applied to the permuted
 * [groups, tile*tile] tensor (same codes, same hash counters); noise-tensor and
 * reference-compatible modes are not built here (flags: 0 or ACT_FLAG_ROUND_NEAREST).
 */
ACT_API int act_quant_pack_tiles(const void* x, int dtype, int64_t n_planes, int height, int width, int tile,
                         int bits, uint64_t seed, uint64_t offset, int flags, void* packed,
                         float* scale, float* min, void* stream);
ACT_API int act_dequant_unpack_tiles(const void* packed, const float* scale, const float* min,
                             int64_t n_planes, int height, int width, int tile, int bits,
                             int out_dtype, void* y, void* stream);

/*
 * Bit-pack int8 values (masks or ready-made codes), low `bits` bits of each.
 * Replaces torch.ops.act_lib.pack_triton / unpack_triton
 * (AC/act_triton_kernel.py:398-433, kernels :246-322).  x, y: int8 [n_groups, group_size].
 */
ACT_API int act_pack_bits(const int8_t* x, int64_t n_groups, int group_size, int bits, void* packed,
                  void* stream);
ACT_API int act_unpack_bits(const void* packed, int64_t n_groups, int group_size, int bits, int8_t* y,
                    void* stream);

/*
 * Fused activation kernels (one pass instead of activation + mask/derivative + codec).
 * Replace torch.ops.act_lib.relu_fwd_fused_pack / relu_bwd_fused_unpack
 * (AC/modules/activations/kernel_registration.py:43-94, kernels kernel_implementation.py:34-143)
 * and the backward halves silu/gelu_bwd_fused_dequan_unpack (kernel_registration.py:190-237,
 * 285-319).  n_elems is a multiple of 32; mask_bits holds one bit per element in the word
 * layout of act_pack_bits with bits = 1.
 *   act_relu_fwd_pack:  y = x > 0 ? x : 0 (relu6: 0 < x < 6), mask bit = that condition
 *   act_relu_bwd_unpack: dx = mask ? dy : 0
 *   act_mul_dequant_unpack: dx = dy * fma(code, scale, min), fp32 product rounded to dtype
 */
 /*
 * act_activation_fwd_quant_pack: y = act(x) and the quantise-and-pack of act'(x) in one
 * pass (replaces gelu_fwd_fused_quan_pack / silu_fwd_quan_pack, kernel_registration.py:
 * 148-188, 262-283).  Codes follow the default scheme of act_quant_pack applied to the fp32
 * derivative; tanh and exp are the hardware approximations.  flags: 0 or ROUND_NEAREST.
 */
ACT_API int act_activation_fwd_quant_pack(const void* x, int dtype, int kind, int64_t n_groups,
                                  int group_size, int bits, uint64_t seed, uint64_t offset,
                                  int flags, void* y, void* packed, float* scale, float* min,
                                  void* stream);
ACT_API int act_relu_fwd_pack(const void* x, int dtype, int64_t n_elems, int relu6, void* y,
                      void* mask_bits, void* stream);
ACT_API int act_relu_bwd_unpack(const void* mask_bits, const void* dy, int dtype, int64_t n_elems,
                        void* dx, void* stream);
ACT_API int act_mul_dequant_unpack(const void* packed, const float* scale, const float* min,
                           const void* dy, int dtype, int64_t n_groups, int group_size, int bits,
                           void* dx, void* stream);

/*
 * Fused batch-norm kernels on x [N, C, HW] with flat sample-major groups (replace
 * bn_fwd_norm_quant_pack_fused, bn_bwd_reduce_dequant_unpack_fused and
 * bn_bwd_dx_dequant_unpack_fused, AC/modules/normalization/kernel_registration.py:86-299).
 * HW must be a multiple of 4 and N*C*HW a multiple of group_size.
 *   act_bn_fwd_norm_quant_pack: params = fp32 [C][4] (mean, invstd, weight, bias);
 *       x_hat = (x - mean) * invstd, y = x_hat * weight + bias (each step rounded to fp32),
 *       y written in `dtype`, x_hat quantised with the default scheme of act_quant_pack.
 *       Needs HW*(HW+1024) < 2^32 and C*(C+260) < 2^32, else ACT_ERR_UNSUPPORTED.
 *   act_bn_stats: the batch statistics pass in front of it (replaces bn_fwd_reduce,
 *       AC/modules/normalization/kernel_implementation.py:13-92).  Writes params[c] = (mean,
 *       1/sqrt(var + eps), weight[c] or 1, bias[c] or 0) with the biased variance, and, when the
 *       pointers are given, running_mean/var = (1-momentum)*old + momentum*(mean, unbiased
 *       var).  Sums are shifted by x[0,c,0], accumulated in fp32 per block and combined in
 *       double in a fixed order: the result does not vary from run to run.  workspace:
 *       act_bn_stats_workspace(n_batch, channels) bytes, caller-owned.  C <= 65535.
 *   act_bn_bwd_reduce: sums fp32 [2*C], zeroed by the caller; adds sum(dy*x_hat) to sums[c]
 *       and sum(dy) to sums[C+c] (one atomic pair per block: the order of the at most
 *       148*8/C partial sums is not fixed). C <= 65535.
 *   act_bn_bwd_dx: coef = fp32 [C][4] (k1, k2, k3, unused); dx = k1*dy - k2 - k3*x_hat.
 *   act_bn_bwd_coef: that table from the sums of act_bn_bwd_reduce and the params of
 *       act_bn_stats: k1 = weight*invstd, k2 = k1*sum(dy)/count, k3 = k1*sum(dy*x_hat)/count
 *       (count = N*HW); one small launch instead of a chain of elementwise operators.
 * Channel-minor layout: hw = 1 means x is [n_batch, C] with the channel running fastest, which
 * is what a channels-last [N, C, H, W] activation is in memory (pass n_batch = N*H*W).  All of
 * the entry points above and the three BN+ReLU ones below take it, with C a multiple of 8 (and
 * C <= 4096 in the forward kernel, which keeps the parameter table in shared memory); groups,
 * mask bits and hash counters then follow that memory order, and the arithmetic per element is
 * unchanged.  (The reference's kernels address NCHW only; cuDNN's bf16 convolutions work in
 * NHWC, so this layout removes their layout conversions around every batch norm.)
 */
ACT_API int act_bn_fwd_norm_quant_pack(const void* x, int dtype, int64_t n_batch, int channels, int64_t hw,
                               const float* params, int group_size, int bits, uint64_t seed,
                               uint64_t offset, int flags, void* y, void* packed, float* scale,
                               float* min, void* stream);
ACT_API size_t act_bn_stats_workspace(int64_t n_batch, int channels);
ACT_API int act_bn_stats(const void* x, int dtype, int64_t n_batch, int channels, int64_t hw, double eps,
                 const float* weight, const float* bias, float* running_mean, float* running_var,
                 double momentum, float* params, void* workspace, size_t ws_bytes, void* stream);
ACT_API int act_bn_bwd_reduce(const void* packed, const float* scale, const float* min, const void* dy,
                      int dtype, int64_t n_batch, int channels, int64_t hw, int group_size, int bits,
                      float* sums, void* stream);
ACT_API int act_bn_bwd_coef(const float* sums, const float* params, int channels, double count,
                    float* coef, void* stream);
ACT_API int act_bn_bwd_dx(const void* packed, const float* scale, const float* min, const void* dy,
                  int dtype, int64_t n_batch, int channels, int64_t hw, int group_size, int bits,
                  const float* coef, void* dx, void* stream);

/*
 * Batch norm followed by ReLU in the same three kernels (replaces the norm+activation fusion
 * of AC/triton_kernel/norm_act_fusion/bn_act_fusion.py:7-278).  Forward also applies
 * y = max(y, 0) and writes the ReLU mask, one bit per element (bit i of byte e/8 = element e,
 * N*C*HW/8 bytes, the layout of act_relu_fwd_pack); the two backward kernels read dy only
 * where the mask bit is set, so the ReLU backward pass disappears.  Everything else is as in
 * the three entry points above.
 */
ACT_API int act_bn_relu_fwd_norm_quant_pack(const void* x, int dtype, int64_t n_batch, int channels,
                                    int64_t hw, const float* params, int group_size, int bits,
                                    uint64_t seed, uint64_t offset, int flags, void* y, void* packed,
                                    float* scale, float* min, void* mask_bits, void* stream);
/*
 * The same with the skip connection of a residual block between the batch norm and the ReLU
 * (the reference's bottleneck ends `x += identity; return relu3(x)`, Model/CNN/ResNetV1.py:48-49,
 * as an add and a ReLU pass of their own): y = max(x_hat * weight + bias + residual, 0), the
 * sum rounded to fp32 before the ReLU, `residual` of x's type, shape and layout; the mask is
 * that of the sum.  Backward: dy * mask is the gradient of the residual and the dy of the
 * batch norm; act_bn_add_relu_bwd_reduce writes it to dy_masked (act_relu_bwd_unpack) and
 * computes the sums of act_bn_bwd_reduce on it; act_bn_bwd_dx then reads dy_masked.
 */
ACT_API int act_bn_add_relu_fwd_norm_quant_pack(const void* x, const void* residual, int dtype, int64_t n_batch,
                                        int channels, int64_t hw, const float* params, int group_size,
                                        int bits, uint64_t seed, uint64_t offset, int flags, void* y,
                                        void* packed, float* scale, float* min, void* mask_bits,
                                        void* stream);
ACT_API int act_bn_add_relu_bwd_reduce(const void* packed, const float* scale, const float* min, const void* dy,
                               const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                               int group_size, int bits, float* sums, void* dy_masked, void* stream);
ACT_API int act_bn_relu_bwd_reduce(const void* packed, const float* scale, const float* min, const void* dy,
                           const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                           int group_size, int bits, float* sums, void* stream);
ACT_API int act_bn_relu_bwd_dx(const void* packed, const float* scale, const float* min, const void* dy,
                       const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                       int group_size, int bits, const float* coef, void* dx, void* stream);

/*
 * One call per layer and direction: the launches of the entry points above in sequence, for
 * hosts where the round trip per launch matters (53 layers per ResNet-50 step).
 *   act_bn_forward: act_bn_stats, then the forward kernel that the arguments select
 *       (residual != NULL: + residual + ReLU; else mask_bits != NULL: + ReLU; else plain).
 *   act_bn_backward: zeroes sums [2C], then act_bn_bwd_reduce, act_bn_bwd_coef (writes coef
 *       [C][4]) and act_bn_bwd_dx.  mask_bits NULL: plain; mask_bits and dy_masked NULL: the
 *       ReLU variants; mask_bits and dy_masked given: dy under the mask goes to dy_masked
 *       first (act_relu_bwd_unpack; the residual's gradient) and the plain kernels read that.
 */
ACT_API int act_bn_forward(const void* x, const void* residual, int dtype, int64_t n_batch, int channels,
                   int64_t hw, double eps, const float* weight, const float* bias, float* running_mean,
                   float* running_var, double momentum, float* params, void* workspace, size_t ws_bytes,
                   int group_size, int bits, uint64_t seed, uint64_t offset, int flags, void* y,
                   void* packed, float* scale, float* min, void* mask_bits, void* stream);
ACT_API int act_bn_backward(const void* packed, const float* scale, const float* min, const void* dy,
                    const void* mask_bits, int dtype, int64_t n_batch, int channels, int64_t hw,
                    int group_size, int bits, const float* params, double count, float* sums, float* coef,
                    void* dy_masked, void* dx, void* stream);

/*
 * The same with a second gradient of the same tensor (dy2, dy's type and layout, or NULL): the
 * mask pass of the residual form computes mask ? dy + dy2 : 0 (the sum in fp32, rounded once),
 * so that a block output with two consumers needs no accumulation pass of its own
 * (autograd otherwise adds the two gradients with a kernel of its own before the backward of the
 * batch norm runs: 16 such additions per ResNet-50 step).  dy2 is accepted only together with
 * mask_bits and dy_masked.  act_relu_bwd_unpack_sum and act_bn_add_relu_bwd_reduce_sum are the
 * two steps on their own.
 */
ACT_API int act_relu_bwd_unpack_sum(const void* mask_bits, const void* dy, const void* dy2, int dtype,
                                    int64_t n_elems, void* dx, void* stream);
ACT_API int act_bn_add_relu_bwd_reduce_sum(const void* packed, const float* scale, const float* min, const void* dy,
                                           const void* dy2, const void* mask_bits, int dtype, int64_t n_batch,
                                           int channels, int64_t hw, int group_size, int bits, float* sums,
                                           void* dy_masked, void* stream);
ACT_API int act_bn_backward_sum(const void* packed, const float* scale, const float* min, const void* dy,
                                const void* dy2, const void* mask_bits, int dtype, int64_t n_batch, int channels,
                                int64_t hw, int group_size, int bits, const float* params, double count,
                                float* sums, float* coef, void* dy_masked, void* dx, void* stream);

/*
 * Max pooling on a channels-last activation with a 4-bit argmax saved for backward instead of
 * PyTorch's int64 index per output (no counterpart in the reference, which leaves the pooling
 * layer of its ResNet payload, Model/CNN/ResNetV1.py:63,99, to PyTorch): x [N, H, W, C] with C a
 * multiple of 8, square window k <= 4, stride s, zero padding pad <= k/2, no dilation, floor
 * output size OH = (H + 2*pad - k)/s + 1.  idx: uint32 [N*OH*OW*C/8], nibble j of a word = window
 * position kh*k + kw of the maximum for channel 8q+j (ties: first position; a NaN wins).
 * Backward gathers: dx[n,ih,iw,c] = sum of dy over the windows whose saved position is (ih,iw),
 * accumulated in fp32 and rounded once.
 */
ACT_API int act_maxpool_fwd_cl(const void* x, int dtype, int64_t n, int h, int w, int c, int k, int s, int pad,
                       void* y, void* idx, void* stream);
ACT_API int act_maxpool_bwd_cl(const void* idx, const void* dy, int dtype, int64_t n, int h, int w, int c, int k,
                       int s, int pad, void* dx, void* stream);

/*
 * Per-row min and max of a contiguous [rows, cols] matrix.
 * Replaces cpp_extension.min_max_kernel (AC/cpp_extension/src/min_max_kernel.cu:66-141).
 */
ACT_API int act_minmax(const void* x, int dtype, int64_t rows, int64_t cols, float* mn, float* mx,
               void* stream);

/*
 * The reference's second codec: caller-supplied per-group min and max (in x's own type),
 * scale = (2^bits - 1) / (max - min + 2e-6), stochastic rounding with its index hash
 * sgd_noise keyed by (element index << 32) ^ seed, codes stored as bit planes in warp-ballot
 * order (32 consecutive elements = one chunk of `bits` consecutive words; bit i of word p =
 * bit p of the code of the chunk's element i).  group_size: a multiple of 32; bits: 1..8.
 *   packed: uint32 [n_groups * group_size/32 * bits]; scale: [n_groups] in x's type (output).
 *   flags: 0 rounds without bias, rint((x-min)*scale + noise) with noise in [-0.5, 0.5);
 *          ACT_FLAG_BALLOT_REF_BIAS subtracts the further 0.5 the reference subtracts.
 * act_unpack_ballot: y = code / scale + min, in the type of scale and min.
 * Replaces cpp_extension.pack_mixed_precision_cuda / unpack_mixed_precision_cuda
 * (AC/cpp_extension/src/quantization_cuda_kernels.cu:15-195, 200-298; hash:
 * AC/cpp_extension/include/quant_common.h:32-43).
 */
ACT_API int act_pack_ballot(const void* x, int dtype, int64_t n_groups, int group_size, int bits,
                    const void* mn, const void* mx, uint64_t seed, int flags,
                    void* packed, void* scale, void* stream);
ACT_API int act_unpack_ballot(const void* packed, const void* scale, const void* mn, int dtype,
                      int64_t n_groups, int group_size, int bits, void* y, void* stream);

/*
 * Identity copy of nbytes from src to dst (both 16-byte aligned), refused with ACT_ERR_SIZE
 * when nbytes exceeds either buffer's stated capacity.
 * Replaces cpp_extension.copy_launch (AC/cpp_extension/src/copy.cu:50-102), a debugging
 * aid of the reference that copies [N*G, 256] elements without any bounds check.
 */
ACT_API int act_copy(const void* src, void* dst, size_t nbytes, size_t src_capacity, size_t dst_capacity,
             void* stream);

/*
 * Clears nbytes at p on the given stream (cudaMemsetAsync).  No counterpart in the reference:
 * a convenience for hosts that bind this library but not the CUDA runtime.
 */
ACT_API int act_fill_zero(void* p, size_t nbytes, void* stream);

/*
 * Column reductions over a row-major [rows, cols] tensor (cols a multiple of 8, 16-byte aligned
 * base; dtype ACT_DTYPE_*), results fp32 [cols], overwritten (zeroed, then summed with one atomic
 * per block and column: the order of the partial sums is not fixed).
 *   act_col_sum: out[c] = sum_r a[r, c].  Replaces `dy.sum(0)` for the bias gradient in
 *       _DOLinear.backward (AC/modules/ops.py:496-526).
 *   act_ln_bwd_params: dgamma[c] = sum_r dy[r, c] * (x[r, c] - mean[r]) * rstd[r] and
 *       dbeta[c] = sum_r dy[r, c], with mean and rstd fp32 [rows] as the forward pass returned
 *       them: the parameter gradients of a LayerNorm over the last dimension (the reference leaves
 *       LayerNorm to PyTorch, AC/controller.py:87; ATen's kernel for these two sums takes 430 us
 *       on bf16 [50432, 768], a fifth of the ViT-B/16 step).
 */
ACT_API int act_col_sum(const void* a, int dtype, int64_t rows, int cols, float* out, void* stream);
ACT_API int act_ln_bwd_params(const void* dy, const void* x, const float* mean, const float* rstd, int dtype,
                              int64_t rows, int cols, float* dgamma, float* dbeta, void* stream);

/*
 * LayerNorm over the last dimension of a row-major [rows, cols] tensor, fused with the codec of
 * its input (cols a multiple of group_size, group_size in 32..256, cols <= 1024; weight and bias
 * fp32 [cols] or NULL; flags 0 or ACT_FLAG_ROUND_NEAREST).
 *   act_ln_fwd_quant_pack: y = (x - mean) * rstd * weight + bias in x's type, mean and rstd fp32
 *       [rows] (biased variance, 1/sqrt(var + eps)), and packed / scale / min of x bit for bit what
 *       act_quant_pack writes for the same (seed, offset, flags): x is read once.
 *   act_ln_bwd_from_packed: dx (dy's type), dgamma and dbeta (fp32 [cols], overwritten; atomics, so
 *       their summation order is not fixed) from dy, the packed x, mean, rstd and weight; x is
 *       decoded as act_dequant_unpack decodes it to bf16.
 * The reference leaves LayerNorm to PyTorch (AC/controller.py:87); these stand where
 * `unified_quantize` + ATen's native_layer_norm (forward) and `unified_dequantize` +
 * native_layer_norm_backward (backward) stand in a LayerNorm that saves its input compressed.
 */
ACT_API int act_ln_fwd_quant_pack(const void* x, int dtype, int64_t rows, int cols, const float* weight,
                                  const float* bias, double eps, int group_size, int bits, uint64_t seed,
                                  uint64_t offset, int flags, void* y, float* mean, float* rstd, void* packed,
                                  float* scale, float* min, void* stream);
ACT_API int act_ln_bwd_from_packed(const void* dy, int dtype, int64_t rows, int cols, const void* packed,
                                   const float* scale, const float* min, int group_size, int bits,
                                   const float* mean, const float* rstd, const float* weight, void* dx,
                                   float* dgamma, float* dbeta, void* stream);

/*
 * The same pair for a LayerNorm that follows a residual addition, s = x + res (the pre-norm
 * transformer block: s feeds the LayerNorm and the next addition).  16-bit types only.
 *   act_ln_add_fwd_quant_pack: sum = x + res rounded to the element type (what a separate
 *       addition writes), then y, mean, rstd and the packed sum exactly as act_ln_fwd_quant_pack
 *       gives them for x = sum: the addition's kernel and the LayerNorm's read of its result fall away.
 *   act_ln_bwd_from_packed_sum: dx = LayerNorm's input gradient + dy2, where dy2 (dy's type, same
 *       shape, or NULL) is the gradient that reached the sum along its other consumer; added in
 *       fp32 before the one rounding.  The caller hands dx to both x and res.
 */
ACT_API int act_ln_add_fwd_quant_pack(const void* x, const void* res, int dtype, int64_t rows, int cols,
                                      const float* weight, const float* bias, double eps, int group_size, int bits,
                                      uint64_t seed, uint64_t offset, int flags, void* sum, void* y, float* mean,
                                      float* rstd, void* packed, float* scale, float* min, void* stream);
ACT_API int act_ln_bwd_from_packed_sum(const void* dy, const void* dy2, int dtype, int64_t rows, int cols,
                                       const void* packed, const float* scale, const float* min, int group_size,
                                       int bits, const float* mean, const float* rstd, const float* weight,
                                       void* dx, float* dgamma, float* dbeta, void* stream);

/*
 * act_merge_heads: dst[b, t, s, h, :] = srcs[s][b, h, t, :] for s < parts (1..4); dst is contiguous
 * [B, T, parts, H, Dh]; strides = parts x (element stride of b, of h, of t) of the sources, whose
 * last dimension is contiguous.  Dh * elem_bytes, the sources' byte strides and all bases are
 * multiples of 16.  The backward of the q/k/v split of a fused qkv projection
 * (Model/ViT/ViT.py:39-42 of the reference: view, permute, index): the three gradients of the
 * attention become the gradient of the projection's output in one pass.
 */
ACT_API int act_merge_heads(const void* const* srcs, const int64_t* strides, int parts, int B, int H, int T,
                            int Dh, int elem_bytes, void* dst, void* stream);

/*
 * Greedy bit allocation on the host (no GPU work).
 * Replaces cpp_extension.calc_precision (AC/cpp_extension/src/calc_precision.cc:10-53):
 * b, C, w are int32 arrays of length n; b is updated in place until sum(b*w) <= target.
 */
ACT_API int act_calc_precision(int32_t* b, const int32_t* C, const int32_t* w, int64_t n, double target);

/*
 * FP8 GEMM: C[m,n] = bf16( (sum_k A[m,k]*B[k,n]) * sa[m] * sb[n] ), A and B e4m3 bytes,
 * fp32 accumulation in tensor memory (tcgen05), operands fed by TMA.
 * Replaces Triton_Linear (AC/triton_kernel/linear.py:5-95), the reference's FP8-tuned
 * tiled GEMM, and adds the per-row / per-column dequantisation scales.
 *   A   [M,K] row-major, lda bytes per row (multiple of 16), 16-byte aligned
 *   B   [K,N] row-major with ldb (default, the reference's layout), or [N,K] with
 *       ACT_GEMM_B_IS_NK (ldb multiple of 16).  A [K,N] operand is read in place when M > 128,
 *       ldb is a multiple of 16 and B is 16-byte aligned; otherwise it is first transposed into
 *       the workspace (act_fp8_gemm_workspace says how much that takes for ldb = N)
 *   sa  fp32 [M], sb fp32 [N] (16-byte aligned), C bf16 [M,N] with ldc elements per row
 *   K and lda multiples of 16; N and ldc multiples of 8.
 *   workspace: act_fp8_gemm_workspace(M,N,K,flags) bytes, 16-byte aligned (may be NULL if 0).
 */
ACT_API size_t act_fp8_gemm_workspace(int M, int N, int K, int flags);
ACT_API int act_fp8_gemm(const void* A, const void* B, const float* sa, const float* sb, void* C,
                 int M, int N, int K, int lda, int ldb, int ldc, int flags,
                 void* workspace, size_t ws_bytes, void* stream);
/*
 * The same GEMM for callers that must not allocate device memory (no counterpart in the
 * reference; B is always [K,N]).  Its transpose scratch is a 4 MiB array built into the
 * library, so it needs no workspace and calls no allocator, but N * K (K rounded up to 16)
 * must not exceed act_fp8_gemm_static_limit() bytes; larger problems return
 * ACT_ERR_STATIC_LIMIT.  The first call on each device looks the array's address up:
 * make that call before starting any stream capture.  All calls on a device share the one
 * array, so two calls whose GPU work can overlap (different streams) race on it; keep them
 * on one stream or order them with events.  The array holds the previous call's bytes
 * between calls; every call overwrites the part it reads.
 */
ACT_API size_t act_fp8_gemm_static_limit(void);
ACT_API int act_fp8_gemm_static(const void* A, const void* B, const float* sa, const float* sb, void* C,
                        int M, int N, int K, int lda, int ldb, int ldc, void* stream);

/*
 * Weight gradient of a linear layer computed from its compressed input, with the codes decoded
 * inside the GEMM's operand pipeline instead of through a dequantised copy in memory:
 *     dW[n, k] = sum_m dY[m, n] * bf16(code[m, k] * scale[g] + min[g])        (fp32 output)
 *   dy: bf16 [M, N], row pitch ld_dy elements (multiple of 8), 16-byte aligned;
 *   packed / scale / min: what act_quant_pack wrote for the row-major [M, K] input with flat groups
 *       of group_size (a power of two in 32..1024 that divides K); bits in {1,2,4,8};
 *   dw: fp32 [N, K], row pitch ld_dw elements (multiple of 4), 16-byte aligned; overwritten.
 * N and K must be multiples of 8.  No workspace: slices of M owned by different CTAs are summed
 * into dw with vector reductions after the entry has zeroed it on the same stream.
 * Replaces the sequence dequant_unpack_triton + dy.T.mm(x) of _DOLinear.backward
 * (AC/modules/ops.py:496-526); the reference's own attempt at this fusion is
 * AC/test2.ipynb:14-19, 478-491.
 */
ACT_API int act_dw_from_packed(const void* dy, const void* packed, const float* scale, const float* min,
                       int bits, int group_size, int M, int N, int K, int ld_dy,
                       float* dw, int ld_dw, void* stream);
/* Abort reason of the last act_dw_from_packed on the current device (0 = none); synchronises. */
ACT_API int act_dw_from_packed_status(unsigned int* out, int clear);

/* Abort reason of the last GEMM on the current device (0 = none); synchronises. */
ACT_API int act_fp8_gemm_status(unsigned int* out, int clear);

/* Text for a return code; never NULL. */
ACT_API const char* act_strerror(int code);

/* Version of this ABI (bumped when a signature changes). */
ACT_API int act_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ACT_B200_H */
