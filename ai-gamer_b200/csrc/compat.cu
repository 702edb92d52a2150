// compat.cu -- the reference's forward-path launchers under their own names (include/aig_compat.h),
// as wrappers over the context API on a process-wide context bound to the legacy default stream.
#include <mutex>

#include "aig_common.cuh"
#include "aig_compat.h"

namespace {

aig_ctx* g_ctx = nullptr;
int g_status = AIG_OK;
int g_group = 64;
std::mutex g_mu;

aig_ctx* ctx() {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_ctx) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (aig_ctx_create(&g_ctx, dev) == AIG_OK) aig_ctx_set_stream(g_ctx, nullptr);  // legacy default stream, like the reference
    else g_ctx = nullptr;
  }
  return g_ctx;
}

inline void note(int rc) { g_status = rc; }

// CudaStuff.cu:52-58: copy B,G,R of every 4-byte pixel to a packed 3-byte pixel
__global__ void bgra_to_bgr_kernel(const uchar4* __restrict__ src, unsigned char* __restrict__ dst, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += blockDim.x * gridDim.x) {
    const uchar4 p = src[i];
    dst[3 * i + 0] = p.x;
    dst[3 * i + 1] = p.y;
    dst[3 * i + 2] = p.z;
  }
}

// Normal(0, 2/fanIn) weights from a counter-based generator (the reference draws from cuRAND's default
// generator with seed 1234, CudaStuff.cu:49-50,186-193; the sequence here is a different one with the
// same distribution, fixed by `seed` and the element index)
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
__global__ void he_init_kernel(__half* w, int n, float scale, uint32_t seed) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += blockDim.x * gridDim.x) {
    const uint32_t a = mix32(seed ^ (2u * (uint32_t)i + 1u)), b = mix32((seed * 0x9e3779b9U) ^ (2u * (uint32_t)i + 2u));
    const float u1 = ((float)(a >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
    const float u2 = (float)(b >> 8) * (1.0f / 16777216.0f);
    w[i] = __float2half(sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2) * scale);
  }
}
uint32_t g_he_calls = 0;

}  // namespace

extern "C" {

aig_ctx* aig_compat_context(void) { return ctx(); }
int aig_compat_last_status(void) { return g_status; }
void aig_compat_set_attention_group(int group) { g_group = group > 0 ? group : 64; }

void InitCUDA(void) { note(ctx() ? AIG_OK : AIG_ERR_CUDA); }

void ConvertAndNormalize(__half* output, const unsigned char* input, size_t size) {
  note(aig_convert_normalize(ctx(), (aig_half*)output, input, size));
}
void UnConvertAndUnNormalize(unsigned char* output, const __half* input, size_t size) {
  note(aig_unconvert_unnormalize(ctx(), output, (const aig_half*)input, size));
}
void ConvertFloatToHalf(float* src, __half* dst, size_t n) { note(aig_float_to_half(ctx(), src, (aig_half*)dst, n)); }
void ConvertHalfToFloat(__half* src, float* dst, size_t n) { note(aig_half_to_float(ctx(), (const aig_half*)src, dst, n)); }

void HeInit(__half* weightHalf, int numWeights, float fanIn) {
  aig_ctx* c = ctx();
  if (!c || !weightHalf || numWeights <= 0 || fanIn <= 0.f) return note(AIG_ERR_INVALID);
  DeviceGuard g(c->device);
  int blocks = ceil_div(numWeights, 256);
  if (blocks > c->sm_count * 8) blocks = c->sm_count * 8;
  he_init_kernel<<<blocks, 256, 0, c->stream>>>(weightHalf, numWeights, sqrtf(2.0f / fanIn), 1234u + 7919u * g_he_calls++);
  note(cudaGetLastError() == cudaSuccess ? AIG_OK : AIG_ERR_CUDA);
}

void LeakyReluForward(__half* data, int size, float negativeSlope) { note(aig_leaky_relu_forward(ctx(), (aig_half*)data, size, negativeSlope)); }
void SwishForward(__half* data, int size) { note(aig_swish_forward(ctx(), (aig_half*)data, size)); }
float MseLoss(const __half* dPredictions, const float* dTargets, int size) {
  float loss = 0.f;
  note(aig_mse_loss2(ctx(), (const aig_half*)dPredictions, dTargets, 1, 1, size, &loss, nullptr));
  return loss;
}
void MseLoss2(const __half* dPredictions, const float* dTargets, int numButs, int numCtrls, int batchSize, float* butLoss, float* axesLoss) {
  note(aig_mse_loss2(ctx(), (const aig_half*)dPredictions, dTargets, numButs, numCtrls, batchSize, butLoss, axesLoss));
}
void Gradient(__half* dGradient, const __half* dPredictions, const __half* dTargets, int size) {
  note(aig_loss_gradient(ctx(), (aig_half*)dGradient, (const aig_half*)dPredictions, (const aig_half*)dTargets, size));
}
bool IsnanHalf(const __half* data, int size) {
  int found = 0;
  note(aig_any_nan_half(ctx(), (const aig_half*)data, size, &found));
  return found != 0;
}
void LeakyReluBackward(__half* grad, const __half* data, int size, float negativeSlope) {
  note(aig_leaky_relu_backward(ctx(), (aig_half*)grad, (const aig_half*)data, size, negativeSlope));
}
void SwishBackward(__half* grad, const __half* data, int size) { note(aig_swish_backward(ctx(), (aig_half*)grad, (const aig_half*)data, size)); }
void SigmoidBackward(__half* grad, const __half* data, int numCtrls, int numButs, int size) {
  note(aig_sigmoid_backward(ctx(), (aig_half*)grad, (const aig_half*)data, numCtrls, numButs, size));
}
void BiasGradient(const __half* gradInput, __half* gradBias, int c, int batchSize) {
  note(aig_bias_gradient(ctx(), (const aig_half*)gradInput, (aig_half*)gradBias, c, batchSize));
}
void SGDHalf(__half* params, const __half* grads, int size, float learningRate, float weightDecay) {
  note(aig_sgd_step_f16(ctx(), (aig_half*)params, (const aig_half*)grads, size, learningRate, weightDecay));
}
void SGDFloat(float* params, const float* grads, int size, float learningRate, float weightDecay) {
  note(aig_sgd_step_f32(ctx(), params, grads, size, learningRate, weightDecay));
}
void AdamWFloat(float* params, const float* grads, float* m, float* v, float learningRate, int t, float weightDecay, int size) {
  note(aig_adamw_step_f32(ctx(), params, grads, m, v, size, learningRate, t, weightDecay));
}
void AdamWHalf(__half* params, const __half* grads, __half* m, __half* v, float lr, int t, float weightDecay, int size) {
  note(aig_adamw_step_f16(ctx(), (aig_half*)params, (const aig_half*)grads, (aig_half*)m, (aig_half*)v, size, lr, t, weightDecay));
}
void SigmoidForward(__half* data, int numCtrls, int numButs, int size) {
  note(aig_sigmoid_forward(ctx(), (aig_half*)data, numCtrls, numButs, size));
}
void LayerNormForward(__half* output, const __half* data, const float* gamma, const float* beta, float* mean, float* variance,
                      int N, int C, int HW) {
  // epsilon 1e-7 as in the reference kernels; every channel is normalised (the reference launcher covers
  // only the first ceil(C / block size) channels, CudaStuff.cu:509 vs :460)
  note(aig_layernorm_forward(ctx(), (aig_half*)output, (const aig_half*)data, gamma, beta, mean, variance, N, C, HW, 1e-7f));
}
void SpatialAttentionForward(const __half* inData, const __half* keyWeights, const __half* queryWeights, const __half* valueWeights,
                             __half* keyMap, __half* queryMap, __half* valueMap, __half* attentionScores, __half* outData,
                             int batchSize, int inC, int attC, int inH, int inW) {
  note(aig_spatial_attention_forward(ctx(), (const aig_half*)inData, (const aig_half*)keyWeights, (const aig_half*)queryWeights,
                                     (const aig_half*)valueWeights, (aig_half*)keyMap, (aig_half*)queryMap, (aig_half*)valueMap,
                                     (aig_half*)attentionScores, (aig_half*)outData, batchSize, inC, attC, inH, inW, g_group));
}

cudaError_t ARGBtoRGB(unsigned char* src, unsigned char* dst, int n) {
  aig_ctx* c = ctx();
  if (!c) return cudaErrorInitializationError;
  DeviceGuard g(c->device);
  int blocks = ceil_div(n > 0 ? n : 1, 256);
  if (blocks > c->sm_count * 16) blocks = c->sm_count * 16;
  bgra_to_bgr_kernel<<<blocks, 256, 0, c->stream>>>(reinterpret_cast<const uchar4*>(src), dst, n);
  return cudaGetLastError();
}
cudaError_t ARGBtoRGBplanar(unsigned char* src, unsigned char* dst, int n) {
  const int rc = aig_bgra_to_planar(ctx(), src, dst, n);
  note(rc);
  return rc == AIG_OK ? cudaSuccess : cudaErrorLaunchFailure;
}

}  // extern "C"
