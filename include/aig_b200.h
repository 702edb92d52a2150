/* aig_b200.h -- C ABI of the B200 (sm_100a) implementation of AI-gamer's frame->action forward path.
 *
 * Everything here is `extern "C"`, takes plain pointers and sizes, and returns an int status
 * (0 = AIG_OK, negative = error; `aig_last_error` gives the text).  Device pointers are raw CUDA
 * device addresses; fp16 tensors are `uint16_t`-sized IEEE binary16 values (`__half` on the caller's
 * side).  Nothing throws across this boundary and there is no CPU fallback: every entry point
 * launches CUDA kernels on the context's stream or fails.
 *
 * Each declaration cites the reference interface it replaces (paths relative to the reference
 * project's "AI gamer/" directory).
 */
#ifndef AIG_B200_H
#define AIG_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint16_t aig_half; /* IEEE binary16 bit pattern (device `__half`) */

enum {
  AIG_OK = 0,
  AIG_ERR_INVALID = -1,     /* bad argument / unsupported shape */
  AIG_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
  AIG_ERR_TIMEOUT = -3,     /* a bounded device-side wait expired (kernel returned early) */
  AIG_ERR_UNSUPPORTED = -4, /* shape outside what the sm_100a kernels cover */
  AIG_ERR_IO = -5           /* checkpoint file problem */
};

/* activation codes used by the fused epilogues */
enum { AIG_ACT_NONE = 0, AIG_ACT_RELU = 1, AIG_ACT_SWISH = 2, AIG_ACT_LEAKY = 3 };

/* ---------------------------------------------------------------------------------------------
 * Context.  Replaces InitCUDA() (CudaStuff.cu:21-51: device 0, global launch shape GS/BS) and the
 * cudnnCreate/cublasCreate handles the reference threads through every layer constructor
 * (Infer.cpp:76-79, NN.h:17-18).  One context = one device + one stream; calls on one context are
 * issued in order on its stream; different contexts are independent. */
typedef struct aig_ctx aig_ctx;
int aig_ctx_create(aig_ctx** out, int device);
int aig_ctx_destroy(aig_ctx* ctx);
/* Use an existing cudaStream_t (passed as void*) instead of the context's own stream. */
int aig_ctx_set_stream(aig_ctx* ctx, void* cuda_stream);
void* aig_ctx_stream(aig_ctx* ctx);
/* Synchronise the stream and report any deferred kernel error (including AIG_ERR_TIMEOUT raised by a
 * bounded device-side wait).  The device error word is cleared. */
int aig_ctx_sync(aig_ctx* ctx);
const char* aig_last_error(aig_ctx* ctx);
/* Self-test of the time-out path every kernel of this library shares (no counterpart in the reference, whose
 * kernels never wait on one another).  Launches one small kernel whose only work is a bounded wait on a
 * barrier that nobody arrives at; after `limit_cycles` SM clocks (at most 2e8, about 0.1 s) the wait gives up,
 * records an error code for the context and the kernel returns normally.  The next aig_ctx_sync then returns
 * AIG_ERR_TIMEOUT once, and the context stays usable. */
int aig_selftest_expiring_wait(aig_ctx* ctx, long long limit_cycles);
int aig_device_sm_count(aig_ctx* ctx);
/* Asynchronous copy on the context's stream (any direction; the checkCUDA(cudaMemcpy(...)) calls of
 * the reference's LoadParameters/SaveParameters and Infer.cpp:112). */
int aig_memcpy(aig_ctx* ctx, void* dst, const void* src, size_t bytes);

/* CUDA-graph capture of everything issued on the context's stream between begin and end; the
 * frame loop (Infer.cpp:96-114) is replayed with aig_graph_launch. */
typedef struct aig_graph aig_graph;
int aig_graph_begin(aig_ctx* ctx);
int aig_graph_end(aig_ctx* ctx, aig_graph** out);
int aig_graph_launch(aig_ctx* ctx, aig_graph* g);
int aig_graph_destroy(aig_graph* g);

/* ---------------------------------------------------------------------------------------------
 * Preprocessing and conversions. */
/* ARGBtoRGBplanar (CudaStuff.cu:63-74, NvDisplayCap.h:68-69): BGRA bytes -> R,G,B planes. */
int aig_bgra_to_planar(aig_ctx* ctx, const uint8_t* src, uint8_t* dst, int n);
/* ConvertAndNormalize (CudaStuff.cu:150-157): out = half(float(u8)/255.0f). */
int aig_convert_normalize(aig_ctx* ctx, aig_half* out, const uint8_t* in, size_t n);
/* Both of the above in one pass: BGRA frames [B][H*W][4] -> fp16 NCHW [B][3][H*W]
 * (GrabFrameInt8 + ConvertAndNormalize, Infer.cpp:103,109). */
int aig_preprocess_bgra(aig_ctx* ctx, const uint8_t* bgra, aig_half* out_nchw, int frames, int hw);
/* UnConvertAndUnNormalize (CudaStuff.cu:158-165). */
int aig_unconvert_unnormalize(aig_ctx* ctx, uint8_t* out, const aig_half* in, size_t n);
/* ConvScale::ScaleInPlace / ScaleToHalf (ConvScale.cpp:41-52) and GrabFrameScaleInt8 / GrabFrameScaleFP16
 * (NvDisplayCap.h:91-119): k x k box-filter down-scaling of uint8 frames -- ConvertAndNormalize, a stride-k
 * convolution with an all-half(1/k^2) filter, fp16 result, UnConvertAndUnNormalize -- as one kernel.  src: planar
 * [frames][channels][h][w] bytes, or with src_is_bgra BGRA pixels [frames][h][w][4] (the colour split of
 * ARGBtoRGBplanar, CudaStuff.cu:63-74, is then fused in; channels = 3).  out_u8 and/or out_half: planar
 * [frames][channels][h/k][w/k].  The reference leaves the accumulation order to cuDNN; here it is fixed (fp32,
 * channel-major then row-major, one fused multiply-add per tap), identical in the CPU oracle, so results are
 * bit-exact.  cross_channel_sum = 1 reproduces the reference's filter, which adds the box means of all three
 * channels into every output channel (ConvScale.cpp:10,17-18); 0 keeps channels apart. */
int aig_resize_box(aig_ctx* ctx, const uint8_t* src, int src_is_bgra, uint8_t* out_u8, aig_half* out_half, int frames,
                   int channels, int h, int w, int k, int cross_channel_sum);

/* ---------------------------------------------------------------------------------------------
 * Training step, the part outside the layers' own Backward (Train.cpp:60-109): losses, loss gradient, NaN check,
 * activation backward passes, bias gradient and parameter updates (CudaStuff.cu:76-153, 194-252, 298-307, 372-459,
 * 571-586).  Per element every kernel performs the arithmetic of the reference's kernel in the same types and
 * order, so gradients, parameters and moments are bit-identical with it; the losses are reduced in a fixed order
 * (the reference adds block sums with float atomics).  Of the layers' own Backward passes the fully connected one is
 * provided (aig_fc_backward, declared with the FC plans below); convolution, normalisation and LSTM backward passes are not.
 *   aig_mse_loss2        MseLoss2: mean squared error over the buttons (control index % n_ctrls < n_buttons) and over
 *                        the mouse axes of a batch; host results; synchronises the context's stream
 *   aig_loss_gradient    Gradient: prediction - target in half arithmetic
 *   aig_any_nan_half     IsnanHalf: *found = 1 if any element is NaN; synchronises
 *   aig_swish_backward   SwishBackward: from the layer's OUTPUT s, d = s + s/(1+s) * (1 - s)   (the reference's form)
 *   aig_leaky_relu_backward, aig_sigmoid_backward: in place on the gradient, as the reference's kernels
 *   aig_bias_gradient    per-channel sum of grad_in [batch][channels] over the batch in fp32 (the reference's kernel,
 *                        CudaStuff.cu:372-394, reduces ACROSS channels after summing: a defect not reproduced)
 *   aig_sgd_step_*       SGDHalf / SGDFloat: decoupled weight decay, gradient clipped to +-128
 *   aig_adamw_step_*     AdamWFloat / AdamWHalf: beta1 0.9, beta2 0.999, eps 1e-7, clip 128, step count t from 1 */
int aig_mse_loss2(aig_ctx* ctx, const aig_half* pred, const float* targets, int n_buttons, int n_ctrls, int batch, float* button_loss, float* axes_loss);
int aig_loss_gradient(aig_ctx* ctx, aig_half* grad, const aig_half* pred, const aig_half* targets, long long n);
int aig_any_nan_half(aig_ctx* ctx, const aig_half* data, long long n, int* found);
int aig_swish_backward(aig_ctx* ctx, aig_half* grad, const aig_half* output, long long n);
int aig_leaky_relu_backward(aig_ctx* ctx, aig_half* grad, const aig_half* input, long long n, float slope);
int aig_sigmoid_backward(aig_ctx* ctx, aig_half* grad, const aig_half* output, int n_ctrls, int n_buttons, long long n);
int aig_bias_gradient(aig_ctx* ctx, const aig_half* grad_in, aig_half* grad_bias, int channels, int batch);
int aig_sgd_step_f16(aig_ctx* ctx, aig_half* params, const aig_half* grads, long long n, float lr, float weight_decay);
int aig_sgd_step_f32(aig_ctx* ctx, float* params, const float* grads, long long n, float lr, float weight_decay);
int aig_adamw_step_f32(aig_ctx* ctx, float* params, const float* grads, float* m, float* v, long long n, float lr, int t, float weight_decay);
int aig_adamw_step_f16(aig_ctx* ctx, aig_half* params, const aig_half* grads, aig_half* m, aig_half* v, long long n, float lr, int t, float weight_decay);
/* ConvertHalfToFloat / ConvertFloatToHalf (CudaStuff.cu:166-181). */
int aig_half_to_float(aig_ctx* ctx, const aig_half* src, float* dst, size_t n);
int aig_float_to_half(aig_ctx* ctx, const float* src, aig_half* dst, size_t n);
/* Layout changes between the operator API's NCHW and the kernels' channels-last layout.
 * `hw` is the product of the spatial extents (D*H*W for 5-D tensors). */
int aig_nchw_to_nhwc(aig_ctx* ctx, const aig_half* src, aig_half* dst, int batch, int c, int hw);
int aig_nhwc_to_nchw(aig_ctx* ctx, const aig_half* src, aig_half* dst, int batch, int c, int hw);

/* ---------------------------------------------------------------------------------------------
 * Element-wise operators, all in place like the reference. */
/* LeakyReluForward (CudaStuff.cu:400-405). */
int aig_leaky_relu_forward(aig_ctx* ctx, aig_half* data, int size, float negative_slope);
/* SwishForward (CudaStuff.cu:416-424). */
int aig_swish_forward(aig_ctx* ctx, aig_half* data, int size);
/* Activate::Forward (Activate.cpp:17-21; cudnnActivationForward RELU). */
int aig_relu_forward(aig_ctx* ctx, aig_half* data, int size);
/* SigmoidForward (CudaStuff.cu:437-446): sigmoid where idx % num_ctrls < num_buts. */
int aig_sigmoid_forward(aig_ctx* ctx, aig_half* data, int num_ctrls, int num_buts, int size);
/* Not in the reference: tanh where idx % num_ctrls >= num_buts (mouse-axis outputs). */
int aig_tanh_tail_forward(aig_ctx* ctx, aig_half* data, int num_ctrls, int num_buts, int size);
/* cudnnAddTensor(alpha=1, beta=1) as used by ResConvLayer::Forward (ResConvLayer.cpp:35): m += r. */
int aig_add_forward(aig_ctx* ctx, aig_half* m, const aig_half* r, int size);
/* BatchNorm::Forward, inference branch (BatchNorm.cpp:55-63).  x,y [B][C][HW] (NCHW); parameters
 * fp32; per_activation != 0 indexes parameters by c*HW+i (CUDNN_BATCHNORM_PER_ACTIVATION). */
int aig_batchnorm_forward(aig_ctx* ctx, const aig_half* x, aig_half* y, const float* gamma,
                          const float* beta, const float* mean, const float* var, int batch, int c,
                          int hw, float eps, int per_activation);

/* ---------------------------------------------------------------------------------------------
 * Normalisation / spatial attention / pooling. */
/* LayerNormForward (CudaStuff.cu:457-515): statistics per channel over N*HW, written to mean/
 * variance; eps is an argument (the reference hard-codes 1e-7).  Every channel gets statistics
 * (the reference's launch covers only the first ceil(C/BS) channels). */
int aig_layernorm_forward(aig_ctx* ctx, aig_half* out, const aig_half* in, const float* gamma,
                          const float* beta, float* mean, float* variance, int n, int c, int hw,
                          float eps);
/* Not in the reference: row-wise LayerNorm over the last dimension (rows x c). */
int aig_layernorm_rows_forward(aig_ctx* ctx, aig_half* out, const aig_half* in, const float* gamma,
                               const float* beta, int rows, int c, float eps);
/* SpatialAttentionForward (CudaStuff.cu:747-760 -> kernel :673-746, scalar branch).  `group` is the
 * softmax-sum group size, i.e. the reference's launch block size BS (64 on its build target);
 * batch*in_h*in_w must be a multiple of it. */
int aig_spatial_attention_forward(aig_ctx* ctx, const aig_half* in, const aig_half* key_w,
                                  const aig_half* query_w, const aig_half* value_w,
                                  aig_half* key_map, aig_half* query_map, aig_half* value_map,
                                  aig_half* attention_scores, aig_half* out, int batch, int in_c,
                                  int att_c, int in_h, int in_w, int group);
/* Not in the reference: "1x1 conv -> sigmoid mask" attention on a channels-last tensor
 * x,y [batch][hw][c]: m = sigmoid(x . w1 + b1), y = half(x*m). */
int aig_spatial_mask_forward(aig_ctx* ctx, const aig_half* x_nhwc, const aig_half* w1, float b1,
                             aig_half* y_nhwc, int batch, int hw, int c);
/* Not in the reference: mean over hw of a channels-last tensor -> [batch][c]. */
int aig_global_avgpool_nhwc(aig_ctx* ctx, const aig_half* x_nhwc, aig_half* y, int batch, int hw, int c);
/* Not in the reference: the whole output head of the frame encoder in one launch -- mask attention,
 * global average pool, FC (W [c][n_out], two roundings like FCLayer.cpp:50-51), sigmoid on the first
 * n_sigmoid outputs and tanh on the rest (Sigmoid.cpp:8-12).  feat [batch][c]; out_half/out_f32
 * [batch][n_out].  Same arithmetic as the separate calls. */
int aig_cnn_head_forward(aig_ctx* ctx, const aig_half* x_nhwc, const aig_half* mask_w, float mask_b,
                         const aig_half* fc_w, const aig_half* fc_b, aig_half* feat, aig_half* out_half,
                         float* out_f32, int batch, int hw, int c, int n_out, int n_sigmoid);
/* FCLayer::Forward (FCLayer.cpp:48-53, both roundings), Sigmoid::Forward on the first n_sigmoid outputs
 * (Sigmoid.cpp:8-12), tanh on the rest and ConvertHalfToFloat (CudaStuff.cu:174-181) as ONE launch, for heads with
 * few rows (one block per row): x [rows][in_c], W [in_c][n_out], bias [n_out] or null; out_half / out_f32
 * [rows][n_out] (out_f32 may be null). */
int aig_fc_head_forward(aig_ctx* ctx, const aig_half* x, const aig_half* w_in_out, const aig_half* bias, aig_half* out_half,
                        float* out_f32, int rows, int in_c, int n_out, int n_sigmoid);
/* Not in the reference: adaptive average pool of channels-last [batch][d][h][w][c] over d and
 * ph x pw spatial cells -> [batch][c*ph*pw] in (c, ph, pw) order. */
int aig_adaptive_avgpool3d_ndhwc(aig_ctx* ctx, const aig_half* x, aig_half* y, int batch, int d, int h,
                                 int w, int c, int ph, int pw);

/* ---------------------------------------------------------------------------------------------
 * Convolution / fully-connected plans: tcgen05 implicit GEMM, operands staged by TMA,
 * accumulators in TMEM.  A plan freezes the shapes like the reference's layer constructors do
 * (ConvLayer.cpp:4-50 builds descriptors and picks an algorithm once).  Activations are
 * channels-last (NDHWC) fp16; weights are given in the reference file layouts and repacked on the
 * device by the set_weights calls.
 *
 * Epilogue: v = acc; if two_step: v = half(v), v = half(v + bias)   [ConvLayer.cpp:76-77]
 *           else v = acc*scale[k] + shift[k]  (bias and inference BatchNorm folded)
 *           if residual: v = half(v) + residual                      [ResConvLayer.cpp:35]
 *           y = half(act(v)). */
typedef struct aig_conv_desc {
  int batch, in_c, in_d, in_h, in_w; /* in_d = 1 for 2-D */
  int out_c;
  int kd, kh, kw;   /* kd = 1 for 2-D */
  int sd, sh, sw;   /* strides */
  int pd, ph, pw;   /* symmetric zero padding */
  int act;          /* AIG_ACT_* */
  float slope;      /* LeakyReLU slope */
  int two_step;     /* 1: reproduce the reference's conv->half, +bias->half roundings, no BN fold */
} aig_conv_desc;
typedef struct aig_conv_plan aig_conv_plan;
/* ConvLayer::ConvLayer / ConvLayer3D::ConvLayer3D (ConvLayer.cpp:4-50, ConvLayer3D.cpp:3-82). */
int aig_conv_plan_create(aig_ctx* ctx, const aig_conv_desc* desc, aig_conv_plan** out);
int aig_conv_plan_destroy(aig_conv_plan* plan);
/* Output extents (ConvLayer.cpp:48-49 writes them back through its int* arguments). */
int aig_conv_plan_out_dims(const aig_conv_plan* plan, int* out_d, int* out_h, int* out_w);
/* ConvLayer::LoadParameters (ConvLayer.cpp:96-107): w fp16 [K][C][kd][kh][kw], bias fp16 [K]
 * (device pointers).  bn_* (fp32 [K], device, may be null = no BatchNorm) are the inference
 * BatchNorm parameters that follow the conv (BatchNorm.cpp:55-63); they are folded into the
 * epilogue's scale/shift. */
int aig_conv_plan_set_weights(aig_conv_plan* plan, const aig_half* w, const aig_half* bias,
                              const float* bn_gamma, const float* bn_beta, const float* bn_mean,
                              const float* bn_var, float bn_eps);
/* ConvLayer::Forward (+ fused BatchNorm/activation/residual).  x NDHWC, y NDHWC,
 * residual NDHWC of the output shape or null. */
int aig_conv_forward(aig_conv_plan* plan, const aig_half* x, const aig_half* residual, aig_half* y);

/* FCLayer (FCLayer.cpp:4-53): y[b][o] = sum_k x[b][k] * W[k*out_c + o] + bias[o].  Same kernel and
 * epilogue as the convolution; `rows` = batch (or batch*time for per-step heads). */
int aig_fc_plan_create(aig_ctx* ctx, int rows, int in_c, int out_c, int act, float slope, int two_step,
                       aig_conv_plan** out);
/* FCLayer::LoadParameters (FCLayer.cpp:70-81): W fp16 [in_c][out_c], bias fp16 [out_c] or null;
 * bn_* = per-activation BatchNorm after the FC (NN.cpp:46), or null. */
int aig_fc_plan_set_weights(aig_conv_plan* plan, const aig_half* w_in_out, const aig_half* bias,
                            const float* bn_gamma, const float* bn_beta, const float* bn_mean,
                            const float* bn_var, float bn_eps);
/* Same, with the matrix given as [out_c][in_c] (the LSTM blob's orientation). */
int aig_fc_plan_set_weights_out_in(aig_conv_plan* plan, const aig_half* w_out_in, const aig_half* bias);

/* Store the result as fp32 (`y` of aig_conv_forward is then a float*): used for the LSTM's input
 * projection, whose pre-activations must not be rounded before the recurrent sum. */
int aig_fc_plan_set_output_f32(aig_conv_plan* plan, int enable);
/* Add a second bias vector (cuDNN's LSTM keeps separate input and recurrent biases,
 * LSTMLayer.cpp:9-40 default bias mode); call after the set_weights function. */
int aig_fc_plan_add_bias(aig_conv_plan* plan, const aig_half* bias2);

/* FCLayer::Backward (FCLayer.cpp:54-59): from the layer's input x [batch][in_c], the incoming gradient grad
 * [batch][out_c] and the weights w_in_out [in_c][out_c] (the reference's layout),
 *   grad_w [in_c][out_c] = x^T . grad,   grad_b [out_c] = aig_bias_gradient(grad),   grad_x [batch][in_c] = grad . W^T,
 * each product accumulated in fp32 on the tensor cores and rounded to fp16 once, like the reference's two
 * cublasGemmEx calls (CUDA_R_32F compute).  Any of the three outputs may be null (then x or w_in_out may be too).
 * The plan holds two GEMM plans and the transposed / zero-padded operand copies; nothing is allocated per call. */
typedef struct aig_fc_backward_plan aig_fc_backward_plan;
int aig_fc_backward_plan_create(aig_ctx* ctx, int batch, int in_c, int out_c, aig_fc_backward_plan** out);
int aig_fc_backward(aig_fc_backward_plan* plan, const aig_half* x, const aig_half* grad, const aig_half* w_in_out, aig_half* grad_w,
                    aig_half* grad_b, aig_half* grad_x);
int aig_fc_backward_plan_destroy(aig_fc_backward_plan* plan);
/* Device storage for [in_c][out_c] weights inside the plan (the input-gradient GEMM's own operand), or null when
 * out_c is not a multiple of 16: a caller that keeps its master weights there and passes this pointer as w_in_out
 * saves aig_fc_backward its copy of the weights.  Owned by the plan. */
aig_half* aig_fc_backward_weight_storage(aig_fc_backward_plan* plan);
/* FCLayer::UpdateParameters, AdamW branch (FCLayer.cpp:60-65): AdamWHalf on weights [in_c][out_c] and bias [out_c]
 * (element for element the arithmetic of aig_adamw_step_f16) in two launches that also refresh what `forward_plan`
 * (an aig_fc_plan_create plan of the same layer whose weights were set once) reads -- its K-major weight operand
 * and its fp32 bias -- so no aig_fc_plan_set_weights call is needed after the step.  t counts steps from 1. */
int aig_fc_adamw_update(aig_ctx* ctx, aig_conv_plan* forward_plan, int in_c, int out_c, aig_half* weights, const aig_half* grad_w,
                        aig_half* m_w, aig_half* v_w, aig_half* bias, const aig_half* grad_b, aig_half* m_b, aig_half* v_b, float lr, int t,
                        float weight_decay);

/* First-layer convolutions (3 input channels), CUDA-core/tensor kernels with the input conversion
 * fused into the load.
 * 2-D: BGRA uint8 frames [B][H][W][4] -> y NHWC fp16 [B][Ho][Wo][K]; the BGRA->RGB split and
 * /255 normalisation (CudaStuff.cu:63-74,150-157) happen in the load, then conv k x k, stride s,
 * pad p over (R,G,B) planes, scale/shift (bias + BatchNorm folded) and activation. */
typedef struct aig_conv0_plan aig_conv0_plan;
int aig_conv0_plan_create(aig_ctx* ctx, int batch, int in_h, int in_w, int out_c, int k, int stride,
                          int pad, int act, float slope, aig_conv0_plan** out);
/* First layer of the 3-D temporal encoder (ConvLayer3D.cpp:3-82 with 3 input channels): input
 * planar fp16 [B][3][D][H][W], output channels-last [B][Do][Ho][Wo][K]. */
int aig_conv0_plan_create_3d(aig_ctx* ctx, int batch, int in_d, int in_h, int in_w, int out_c, int kd,
                             int khw, int sd, int shw, int pd, int phw, int act, float slope,
                             aig_conv0_plan** out);
int aig_conv0_plan_destroy(aig_conv0_plan* plan);
int aig_conv0_plan_out_dims(const aig_conv0_plan* plan, int* out_d, int* out_h, int* out_w);
int aig_conv0_plan_set_weights(aig_conv0_plan* plan, const aig_half* w_kcrs, const aig_half* bias,
                               const float* bn_gamma, const float* bn_beta, const float* bn_mean,
                               const float* bn_var, float bn_eps);
int aig_conv0_forward_bgra(aig_conv0_plan* plan, const uint8_t* bgra, aig_half* y_nhwc);
/* Same convolution from planar uint8 frames [B][3][H][W] (planes R, G, B): what GrabFrameInt8(planar = true)
 * delivers (NvDisplayCap.h:70-87) and what the reference's recordings store per frame
 * (input_recorder.cpp:122-133); the /255 normalisation (CudaStuff.cu:150-157) happens in the load. */
int aig_conv0_forward_rgb_planar(aig_conv0_plan* plan, const uint8_t* rgb_planar, aig_half* y_nhwc);
/* Same convolution from an already normalised planar fp16 NCHW input (the operator-API path). */
int aig_conv0_forward_nchw(aig_conv0_plan* plan, const aig_half* x_nchw, aig_half* y_nhwc);

/* ---------------------------------------------------------------------------------------------
 * Fused down-sampling pair of a residual block.  ResConvLayer (ResConvLayer.cpp:13-21) opens with two
 * stride-2 convolutions of the same input: the main ConvLayer(k4, s2, p1) + BatchNorm + activation and
 * the shortcut ConvLayer(k2, s2, p0) (Forward: ResConvLayer.cpp:28-31).  Over the 2x2 space-to-depth
 * view of the input both are one stride-1 GEMM; this plan runs them as ONE launch that reads the input
 * once and writes both results (channels-last, [batch][Ho][Wo][out_c] each).
 *
 * Space-to-depth layout of an [h][w][c] image: [hb][wb][4][c] with hb = (h-2)/2+2, wb = (w-2)/2+2;
 * pixel (y, x) lives in block ((y+1)>>1, (x+1)>>1) at sub-position ((y+1)&1)*2 + ((x+1)&1).  Buffers in
 * this layout must be zero-filled once before first use (border sub-positions are never written and
 * stand for the padding).  Producers write it directly: aig_conv0_plan_set_output_s2d and
 * aig_conv_plan_set_output_s2d switch a plan's output to this layout. */
size_t aig_s2d_elems(int batch, int h, int w, int c);
int aig_nhwc_to_s2d(aig_ctx* ctx, const aig_half* x, aig_half* s2d, int batch, int h, int w, int c);
int aig_s2d_to_nhwc(aig_ctx* ctx, const aig_half* s2d, aig_half* y, int batch, int h, int w, int c);
int aig_conv_plan_set_output_s2d(aig_conv_plan* plan, int enable);
int aig_conv0_plan_set_output_s2d(aig_conv0_plan* plan, int enable);
/* in_c % 16 == 0; out_c 64, 128 or a multiple of 128 whose double is a multiple of 256. */
int aig_resdown_plan_create(aig_ctx* ctx, int batch, int in_c, int in_h, int in_w, int out_c, int act, float slope,
                            aig_conv_plan** out);
/* w_main fp16 [out_c][in_c][4][4], w_short fp16 [out_c][in_c][2][2] (ConvLayer::LoadParameters layout,
 * ConvLayer.cpp:96-107), biases fp16 [out_c]; bn_* = the BatchNorm after the main convolution or null. */
int aig_resdown_plan_set_weights(aig_conv_plan* plan, const aig_half* w_main, const aig_half* b_main,
                                 const float* bn_gamma, const float* bn_beta, const float* bn_mean,
                                 const float* bn_var, float bn_eps, const aig_half* w_short, const aig_half* b_short);
int aig_resdown_forward(aig_conv_plan* plan, const aig_half* x_s2d, aig_half* y_main, aig_half* y_short);

/* Padded position layout between a fused down-sampling launch and the stride-1 convolution that follows it
 * (ResConvLayer.cpp:28-36: conv0 -> conv1, with the shortcut as conv1's residual).  A [batch][h][w][c] tensor is
 * stored as [batch][h + pad][w + pad][c]: row q = (n * (h + pad) + y) * (w + pad) + x, the extra row and column of
 * every image written as zeros.  One zero column is the right padding of its row and the left padding of the next,
 * one zero row the bottom padding of its image and the top padding of the next, so a convolution with that
 * padding finds every input position of a tile, padding included, in ONE contiguous run of rows (rows before the
 * tensor read as zeros).  aig_conv_padded_rows gives the rows to allocate (rounded up to whole tiles).
 *   aig_resdown_plan_set_output_padded: y_main and y_short of aig_resdown_forward are written in this layout
 *     (pad = 1: the geometry of the 3x3 convolution that follows);
 *   aig_conv_plan_set_input_padded: x AND residual of aig_conv_forward are read in this layout (pad = the plan's
 *     padding); the output layout is unchanged.  Patch-resident plans only (AIG_ERR_UNSUPPORTED otherwise). */
long long aig_conv_padded_rows(int batch, int h, int w, int pad);
int aig_resdown_plan_set_output_padded(aig_conv_plan* plan, int enable);
int aig_conv_plan_set_input_padded(aig_conv_plan* plan, int enable);

/* ---------------------------------------------------------------------------------------------
 * LSTM.  Replaces LSTMLayer (LSTMLayer.cpp:4-40 constructor, :75-104 Forward: cudnnRNNForwardInference,
 * seq-major x [T][B][in] -> y [T][B][hidden], cell clip +-5, two bias vectors) and the cuDNN-8 variant
 * (LSTMLayerv8.cpp:8-39,78-82: batch-major [B][T][.], single bias, no clip).
 * The reference treats the weights as one opaque library blob of weightCount_ halves
 * (LSTMLayer.cpp:29-35,139-146).  This library defines the blob as: for each layer
 * W_i,W_f,W_g,W_o ([hidden][in_l] row-major) then R_i,R_f,R_g,R_o ([hidden][hidden]); then for each
 * layer bW_i..bW_o and, with double_bias, bR_i..bR_o.  h and c are rounded to fp16 every step.
 * Not in the reference: carried state (h_state/c_state, [layers][B][hidden]) for streaming. */
typedef struct aig_lstm_plan aig_lstm_plan;
size_t aig_lstm_weight_count(int in_c, int hidden, int layers, int double_bias);
int aig_lstm_plan_create(aig_ctx* ctx, int seq_len, int layers, int hidden, int batch, int in_c,
                         float clip, int double_bias, int batch_major, aig_lstm_plan** out);
int aig_lstm_plan_destroy(aig_lstm_plan* plan);
/* LSTMLayer::LoadParameters (LSTMLayer.cpp:139-146): the blob stays where it is (device memory,
 * 16-byte aligned) and must outlive the plan's forwards. */
int aig_lstm_plan_set_weights(aig_lstm_plan* plan, const aig_half* blob);
/* LSTMLayer::Forward.  y holds the top layer's h for every step (the reference returns the pointer
 * to the last step's rows, LSTMLayer.cpp:103).  h_state/c_state may be null; they are read as the
 * initial state when use_state != 0 and always receive the final state when non-null. */
int aig_lstm_forward(aig_lstm_plan* plan, const aig_half* x, aig_half* y, aig_half* h_state,
                     aig_half* c_state, int use_state);

/* No counterpart in the reference.  Single-layer LSTM forward (seq-major x [T][B][in] -> y [T][B][hidden],
 * zero initial state, one layer's blob as above) that allocates nothing: its scratch (input
 * projection, zero state, step-barrier counter) is a fixed 2.1 MB array inside the library's device
 * image, held by every GPU that loads the library until the process exits.  Meant for callers that
 * may not call cudaMalloc while running -- a frame loop sharing the GPU with the game it plays
 * (cudaMalloc/cudaFree synchronise the whole device and the game may own almost all memory) or a host
 * that reserves its device budget up front.  Limits: batch <= 128, hidden a multiple of 64 and <= 512,
 * in_c a multiple of 8, seq_len*batch*4*hidden <= 524288 (2 MiB of fp32); larger shapes return
 * AIG_ERR_UNSUPPORTED.  All calls on a device share the array: calls that overlap on the GPU race, so
 * serialise them; each call clears what must start at zero.  The first call on a device looks up the
 * array's device address and should come before any stream capture.  That first call may also be the one
 * that makes the CUDA runtime load this library's device image (module loading is lazy by default), which is
 * when the driver sets the array's memory aside: make one warm-up call per device at start-up, and only after it
 * does "allocates nothing" hold.  Calls must come from one host thread at a time (the per-device address cache
 * and the kernel's attribute set-up are not synchronised).  The input projection of this variant is a plain
 * CUDA-core tile kernel, not the tensor-core GEMM of the plan-based path: sized for what the scratch admits. */
int aig_lstm_forward_noalloc(aig_ctx* ctx, const aig_half* x, const aig_half* blob, aig_half* y,
                             int seq_len, int batch, int in_c, int hidden, float clip, int double_bias);

/* ---------------------------------------------------------------------------------------------
 * Multi-head self-attention.  Replaces MultiHeadAttentionLayer (MHALayer.cpp:4-91 constructor,
 * :128-146 Forward: cudnnMultiHeadAttnForward with q = k = v = input, four E x E projection
 * matrices wq,wk,wv,wo (:42-45), `heads` heads of E/heads, scale 1/sqrt(E/heads), causal window
 * [0, i+1), no biases, no residual).  Matrices are [in][out] like FCLayer; head h uses output
 * columns h*d .. h*d+d-1.
 * Not in the reference: rotary position embedding (rope_base > 0; half-split pairs (j, j+d/2),
 * angle = position * rope_base^(-2j/d)) and a ring key/value cache of `window` slots for
 * step-by-step use (aig_mha_step). */
typedef struct aig_mha_plan aig_mha_plan;
int aig_mha_plan_create(aig_ctx* ctx, int batch, int seq_len, int embed, int heads, float rope_base,
                        int window, aig_mha_plan** out);
int aig_mha_plan_destroy(aig_mha_plan* plan);
/* MultiHeadAttentionLayer::LoadParameters (MHALayer.cpp:191-210): wq, wk, wv, wo, each fp16 [E][E]. */
int aig_mha_plan_set_weights(aig_mha_plan* plan, const aig_half* wq, const aig_half* wk,
                             const aig_half* wv, const aig_half* wo);
/* Full-sequence forward: x, y [B][T][E]; positions pos0 .. pos0+T-1; step t attends to
 * max(0, t-window+1) .. t (window <= 0: all earlier steps). */
int aig_mha_forward(aig_mha_plan* plan, const aig_half* x, aig_half* y, int pos0);
/* Streaming: one new step per sequence, x,y [B][E], appended to the ring cache at `position`
 * (absolute frame index; the cache holds the last `window` steps).  aig_mha_reset empties it. */
int aig_mha_step(aig_mha_plan* plan, const aig_half* x, aig_half* y, int position);
int aig_mha_reset(aig_mha_plan* plan);

/* Output decisions of Infer::ProcessOutput (Infer.cpp:8-57) as a pure function on host values:
 * actions[i] = p[i] > 0.5 for i < n_buttons, (int)(p[i]*256.0f) otherwise. */
int aig_actions_from_outputs(const float* p, int* actions, int frames, int n_ctrls, int n_buttons);

/* Infer::ProcessOutput (Infer.cpp:8-57) as a portable event list instead of Win32 SendInput: the same events in the
 * same order -- a key event for each of the 11 keyboard outputs (scan code key_map[i], down iff p[i] > 0.5), a
 * button event for outputs 11, 12, 13 (left, right, middle; down iff > 0.5) and, when either is non-zero, one
 * relative mouse move by ((int)(p[14]*256.0f), (int)(p[15]*256.0f)).  `predictions` are the 16 values of one frame. */
enum { AIG_EVENT_KEY = 0, AIG_EVENT_MOUSE_BUTTON = 1, AIG_EVENT_MOUSE_MOVE = 2 };
typedef struct aig_input_event {
  int type;   /* AIG_EVENT_* */
  int code;   /* scan code (key) or 0/1/2 = left/right/middle (button) */
  int down;   /* 1 = press, 0 = release */
  int dx, dy; /* mouse move */
} aig_input_event;
/* Writes at most `capacity` events (15 suffice) and returns how many the frame produces. */
int aig_process_output(const float* predictions, const unsigned char* key_map, aig_input_event* events, int capacity);
/* The same, handing every event to `sink` (a uinput writer, a network sender, a test recorder ...). */
typedef void (*aig_event_sink)(const aig_input_event* event, void* user);
int aig_process_output_to(const float* predictions, const unsigned char* key_map, aig_event_sink sink, void* user);

#ifdef __cplusplus
}
#endif
#endif /* AIG_B200_H */
