// Layers.cpp -- implementation of the reference-compatible layer classes (Layers.h) on the kernel ABI.
// Errors are C++ exceptions (std::runtime_error), like the reference's checkCUDA/checkCUDNN macros
// (common.h:15-34); the C hooks at the end of the file catch them.
#include "Layers.h"

#include "aig_compat.h"

#include <string.h>

#include <iostream>

namespace {

aig_ctx* g_default_ctx = nullptr;

void check(aig_ctx* ctx, int rc, const char* what) {
  if (rc != AIG_OK) throw std::runtime_error(std::string(what) + ": " + aig_last_error(ctx));
}
void checkCuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
// common.h:82-86 (CUDAMallocZero)
// The reference issues every memset and copy on the legacy default stream, where they are ordered with its
// kernels.  A context of this library may run on another (non-blocking) stream, which the legacy stream does
// not order against, so each of these helpers finishes its work before it returns.
void finishLegacyStream() { checkCuda(cudaStreamSynchronize(cudaStreamLegacy), "cudaStreamSynchronize"); }
template <class T>
void mallocZero(T** p, size_t count) {
  checkCuda(cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)), "cudaMalloc");
  checkCuda(cudaMemset(*p, 0, count * sizeof(T)), "cudaMemset");
  finishLegacyStream();
}
void fillOnes(float* dst, size_t count) {
  std::vector<float> ones(count, 1.0f);
  checkCuda(cudaMemcpy(dst, ones.data(), count * sizeof(float), cudaMemcpyHostToDevice), "fill ones");
  finishLegacyStream();
}
// file -> staging buffer -> device, the pattern of every LoadParameters in the reference (e.g. ConvLayer.cpp:96-107)
void loadArray(std::ifstream& file, unsigned char* buffer, void* dst, size_t bytes) {
  file.read(reinterpret_cast<char*>(buffer), (std::streamsize)bytes);
  if ((size_t)file.gcount() != bytes) throw std::runtime_error("checkpoint truncated");
  checkCuda(cudaMemcpy(dst, buffer, bytes, cudaMemcpyHostToDevice), "cudaMemcpy H2D");
  finishLegacyStream();
}
// device -> staging buffer -> file (e.g. ConvLayer.cpp:84-95).  `ctx` is synchronised first so that kernels
// still writing the array on the context's stream have finished.
void saveArray(aig_ctx* ctx, std::ofstream& file, unsigned char* buffer, const void* src, size_t bytes) {
  if (ctx) check(ctx, aig_ctx_sync(ctx), "SaveParameters");
  checkCuda(cudaMemcpy(buffer, src, bytes, cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
  file.write(reinterpret_cast<const char*>(buffer), (std::streamsize)bytes);
}
aig_half* H(__half* p) { return reinterpret_cast<aig_half*>(p); }
const aig_half* H(const __half* p) { return reinterpret_cast<const aig_half*>(p); }

}  // namespace

aig_ctx* aigDefaultContext() {
  if (!g_default_ctx) throw std::runtime_error("no context yet: construct a layer that takes a handle first or call aigSetDefaultContext");
  return g_default_ctx;
}
void aigSetDefaultContext(aig_ctx* ctx) { g_default_ctx = ctx; }

// ------------------------------------------------------------------------------------------ ConvLayer
ConvLayer::ConvLayer(cudnnHandle_t cudnnHandle, int batchSize, int inChannels, int outChannels, int filterSize, int stride,
                     int padding, int* height, int* width, const char* layerName, bool train, float)
    : batchSize_(batchSize), inC_(inChannels), outC_(outChannels), k_(filterSize), stride_(stride), pad_(padding), inH_(*height),
      inW_(*width), ctx_(cudnnHandle) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  if (inC_ == 3) {
    check(ctx_, aig_conv0_plan_create(ctx_, batchSize_, inH_, inW_, outC_, k_, stride_, pad_, AIG_ACT_NONE, 0.f, &plan0_), layerName);
    aig_conv0_plan_out_dims(plan0_, nullptr, &outH_, &outW_);
  } else {
    aig_conv_desc d{};
    d.batch = batchSize_; d.in_c = inC_; d.in_d = 1; d.in_h = inH_; d.in_w = inW_; d.out_c = outC_;
    d.kd = 1; d.kh = d.kw = k_; d.sd = 1; d.sh = d.sw = stride_; d.pd = 0; d.ph = d.pw = pad_;
    d.act = AIG_ACT_NONE; d.two_step = 1;  // conv -> half, + bias -> half (ConvLayer.cpp:76-77)
    check(ctx_, aig_conv_plan_create(ctx_, &d, &plan_), layerName);
    aig_conv_plan_out_dims(plan_, nullptr, &outH_, &outW_);
    mallocZero(&nhwcIn_, (size_t)batchSize_ * inC_ * inH_ * inW_);
  }
  *height = outH_;  // ConvLayer.cpp:48-49
  *width = outW_;
  outNCHW_ = batchSize_ * outC_ * outH_ * outW_;
  outDesc_ = {batchSize_, outC_, outH_, outW_};
  weightCount_ = (size_t)outC_ * inC_ * k_ * k_;
  mallocZero(&weights_, weightCount_);
  mallocZero(&bias_, (size_t)outC_);
  mallocZero(&outData_, (size_t)outNCHW_);
  mallocZero(&nhwcOut_, (size_t)outNCHW_);
  SyncWeights();
}
ConvLayer::~ConvLayer() {
  aig_conv_plan_destroy(plan_);
  aig_conv0_plan_destroy(plan0_);
  cudaFree(weights_); cudaFree(bias_); cudaFree(outData_); cudaFree(nhwcIn_); cudaFree(nhwcOut_);
}
void ConvLayer::SyncWeights() {
  if (plan0_) check(ctx_, aig_conv0_plan_set_weights(plan0_, H(weights_), H(bias_), nullptr, nullptr, nullptr, nullptr, 0.f), layerName_);
  else check(ctx_, aig_conv_plan_set_weights(plan_, H(weights_), H(bias_), nullptr, nullptr, nullptr, nullptr, 0.f), layerName_);
}
__half* ConvLayer::Forward(__half* data) {
  if (plan0_) {
    check(ctx_, aig_conv0_forward_nchw(plan0_, H(data), H(nhwcOut_)), layerName_);
  } else {
    check(ctx_, aig_nchw_to_nhwc(ctx_, H(data), H(nhwcIn_), batchSize_, inC_, inH_ * inW_), layerName_);
    check(ctx_, aig_conv_forward(plan_, H(nhwcIn_), nullptr, H(nhwcOut_)), layerName_);
  }
  check(ctx_, aig_nhwc_to_nchw(ctx_, H(nhwcOut_), H(outData_), batchSize_, outC_, outH_ * outW_), layerName_);
  return outData_;
}
void ConvLayer::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  loadArray(file, buffer, weights_, weightCount_ * sizeof(__half));
  loadArray(file, buffer, bias_, outC_ * sizeof(__half));
  SyncWeights();
}
void ConvLayer::SaveParameters(std::ofstream& file, unsigned char* buffer) {
  saveArray(ctx_, file, buffer, weights_, weightCount_ * sizeof(__half));
  saveArray(ctx_, file, buffer, bias_, outC_ * sizeof(__half));
}

// ------------------------------------------------------------------------------------------ ConvLayer3D
ConvLayer3D::ConvLayer3D(cudnnHandle_t cudnnHandle, int batchSize, int inChannels, int outChannels, int filterSizeD, int filterSizeHW,
                         int strideD, int strideHW, int paddingD, int paddingHW, int* width, int* height, int* depth,
                         const char* layerName, bool train, float)
    : batchSize_(batchSize), inC_(inChannels), outC_(outChannels), inD_(*depth), inH_(*height), inW_(*width), ctx_(cudnnHandle) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  if (inC_ == 3) {
    check(ctx_, aig_conv0_plan_create_3d(ctx_, batchSize_, inD_, inH_, inW_, outC_, filterSizeD, filterSizeHW, strideD, strideHW, paddingD,
                                         paddingHW, AIG_ACT_NONE, 0.f, &plan0_), layerName);
    aig_conv0_plan_out_dims(plan0_, &outD_, &outH_, &outW_);
  } else {
    aig_conv_desc d{};
    d.batch = batchSize_; d.in_c = inC_; d.in_d = inD_; d.in_h = inH_; d.in_w = inW_; d.out_c = outC_;
    d.kd = filterSizeD; d.kh = d.kw = filterSizeHW; d.sd = strideD; d.sh = d.sw = strideHW; d.pd = paddingD; d.ph = d.pw = paddingHW;
    d.act = AIG_ACT_NONE; d.two_step = 1;
    check(ctx_, aig_conv_plan_create(ctx_, &d, &plan_), layerName);
    aig_conv_plan_out_dims(plan_, &outD_, &outH_, &outW_);
    mallocZero(&nhwcIn_, (size_t)batchSize_ * inC_ * inD_ * inH_ * inW_);
  }
  *depth = outD_; *height = outH_; *width = outW_;
  outNCHW_ = batchSize_ * outC_ * outD_ * outH_ * outW_;
  outDesc_ = {batchSize_, outC_, outD_ * outH_, outW_};
  weightCount_ = (size_t)outC_ * inC_ * filterSizeD * filterSizeHW * filterSizeHW;
  mallocZero(&weights_, weightCount_);
  mallocZero(&bias_, (size_t)outC_);
  mallocZero(&outData_, (size_t)outNCHW_);
  mallocZero(&nhwcOut_, (size_t)outNCHW_);
  SyncWeights();
}
ConvLayer3D::~ConvLayer3D() {
  aig_conv_plan_destroy(plan_);
  aig_conv0_plan_destroy(plan0_);
  cudaFree(weights_); cudaFree(bias_); cudaFree(outData_); cudaFree(nhwcIn_); cudaFree(nhwcOut_);
}
void ConvLayer3D::SyncWeights() {
  if (plan0_) check(ctx_, aig_conv0_plan_set_weights(plan0_, H(weights_), H(bias_), nullptr, nullptr, nullptr, nullptr, 0.f), layerName_);
  else check(ctx_, aig_conv_plan_set_weights(plan_, H(weights_), H(bias_), nullptr, nullptr, nullptr, nullptr, 0.f), layerName_);
}
__half* ConvLayer3D::Forward(__half* data) {
  const int ohw = outD_ * outH_ * outW_;
  if (plan0_) {
    check(ctx_, aig_conv0_forward_nchw(plan0_, H(data), H(nhwcOut_)), layerName_);
  } else {
    check(ctx_, aig_nchw_to_nhwc(ctx_, H(data), H(nhwcIn_), batchSize_, inC_, inD_ * inH_ * inW_), layerName_);
    check(ctx_, aig_conv_forward(plan_, H(nhwcIn_), nullptr, H(nhwcOut_)), layerName_);
  }
  check(ctx_, aig_nhwc_to_nchw(ctx_, H(nhwcOut_), H(outData_), batchSize_, outC_, ohw), layerName_);
  return outData_;
}
void ConvLayer3D::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  loadArray(file, buffer, weights_, weightCount_ * sizeof(__half));
  loadArray(file, buffer, bias_, outC_ * sizeof(__half));
  SyncWeights();
}
void ConvLayer3D::SaveParameters(std::ofstream& file, unsigned char* buffer) {  // ConvLayer3D.cpp:128-133
  saveArray(ctx_, file, buffer, weights_, weightCount_ * sizeof(__half));
  saveArray(ctx_, file, buffer, bias_, outC_ * sizeof(__half));
}

// ------------------------------------------------------------------------------------------ BatchNorm
BatchNorm::BatchNorm(cudnnHandle_t cudnnHandle, cudnnBatchNormMode_t bnMode, int batchSize, int channels, int height, int width,
                     const char* layerName, bool train, float)
    : ctx_(cudnnHandle), mode_(bnMode), batch_(batchSize), c_(channels), hw_(height * width) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  outNCHW_ = batch_ * c_ * hw_;
  outDesc_ = {batch_, c_, height, width};
  paramCount_ = mode_ == CUDNN_BATCHNORM_SPATIAL ? (size_t)c_ : (size_t)c_ * hw_;
  float** arrays[6] = {&bnScale_, &bnBias_, &bnRunningMean_, &bnRunningVar_, &bnSavedMean_, &bnSavedInvVariance_};
  for (float** a : arrays) mallocZero(a, paramCount_);
  fillOnes(bnScale_, paramCount_);  // scale = 1 as in BatchNorm.cpp:15-22
  mallocZero(&outData_, (size_t)outNCHW_);
}
BatchNorm::~BatchNorm() {
  float* arrays[6] = {bnScale_, bnBias_, bnRunningMean_, bnRunningVar_, bnSavedMean_, bnSavedInvVariance_};
  for (float* a : arrays) cudaFree(a);
  cudaFree(outData_);
}
__half* BatchNorm::Forward(__half* data) {
  check(ctx_, aig_batchnorm_forward(ctx_, H(data), H(outData_), bnScale_, bnBias_, bnRunningMean_, bnRunningVar_, batch_, c_, hw_, 1e-6f,
                                    mode_ == CUDNN_BATCHNORM_PER_ACTIVATION ? 1 : 0), layerName_);
  return outData_;
}
void BatchNorm::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  float* arrays[6] = {bnScale_, bnBias_, bnRunningMean_, bnRunningVar_, bnSavedMean_, bnSavedInvVariance_};
  for (float* a : arrays) loadArray(file, buffer, a, paramCount_ * sizeof(float));
}
void BatchNorm::SaveParameters(std::ofstream& file, unsigned char* buffer) {
  float* arrays[6] = {bnScale_, bnBias_, bnRunningMean_, bnRunningVar_, bnSavedMean_, bnSavedInvVariance_};
  for (float* a : arrays) saveArray(ctx_, file, buffer, a, paramCount_ * sizeof(float));
}

// ------------------------------------------------------------------------------------------ activations
Activate::Activate(cudnnHandle_t cudnnHandle, cudnnActivationMode_t mode, double, int batchSize, int channels, int height, int width,
                   const char* layerName)
    : ctx_(cudnnHandle) {
  if (mode != CUDNN_ACTIVATION_RELU) throw std::runtime_error("Activate: only CUDNN_ACTIVATION_RELU is used by the reference");
  g_default_ctx = ctx_;
  layerName_ = layerName;
  outNCHW_ = batchSize * channels * height * width;
  outDesc_ = {batchSize, channels, height, width};
}
__half* Activate::Forward(__half* data) {
  check(ctx_, aig_relu_forward(ctx_, H(data), outNCHW_), layerName_);
  return data;
}
Swish::Swish(int size, const char* layerName) {
  layerName_ = layerName;
  outNCHW_ = size;
}
__half* Swish::Forward(__half* data) {
  check(aigDefaultContext(), aig_swish_forward(aigDefaultContext(), H(data), outNCHW_), layerName_);
  return data;
}
LeakyReLU::LeakyReLU(int size, const char* layerName) {
  layerName_ = layerName;
  outNCHW_ = size;
}
__half* LeakyReLU::Forward(__half* data) {
  check(aigDefaultContext(), aig_leaky_relu_forward(aigDefaultContext(), H(data), outNCHW_, slope_), layerName_);
  return data;
}
Sigmoid::Sigmoid(int numSigmoidOutputs, int batchSize, int outC, const char* layerName) : numSigmoid_(numSigmoidOutputs), outC_(outC) {
  layerName_ = layerName;
  outNCHW_ = batchSize * outC;
}
__half* Sigmoid::Forward(__half* data) {
  check(aigDefaultContext(), aig_sigmoid_forward(aigDefaultContext(), H(data), outC_, numSigmoid_, outNCHW_), layerName_);
  return data;
}

// ------------------------------------------------------------------------------------------ FCLayer
FCLayer::FCLayer(cudnnHandle_t cudnnHandle, cublasHandle_t, int batchSize, int inputSize, int outputSize, const char* layerName,
                 bool train, float weightDecay)
    : weightDecay_(weightDecay), batchSize_(batchSize), inC_(inputSize), outC_(outputSize), ctx_(cudnnHandle) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  outNCHW_ = batchSize_ * outC_;
  outDesc_ = {batchSize_, outC_, 1, 1};
  weightCount_ = (size_t)inC_ * outC_;
  check(ctx_, aig_fc_plan_create(ctx_, batchSize_, inC_, outC_, AIG_ACT_NONE, 0.f, /*two_step*/ 1, &plan_), layerName);
  if (train_) {
    check(ctx_, aig_fc_backward_plan_create(ctx_, batchSize_, inC_, outC_, &backward_), layerName);
    // the master weights live in the input-gradient GEMM's operand where its layout is the reference's (no copy per step)
    weights_ = reinterpret_cast<__half*>(aig_fc_backward_weight_storage(backward_));
    weightsInPlan_ = weights_ != nullptr;
  }
  if (!weightsInPlan_) mallocZero(&weights_, weightCount_);
  mallocZero(&bias_, (size_t)outC_);
  mallocZero(&outData_, (size_t)outNCHW_);
  if (train_) {
    mallocZero(&gradWeights_, weightCount_);
    mallocZero(&gradBias_, (size_t)outC_);
    mallocZero(&gradOut_, (size_t)batchSize_ * inC_);
    mallocZero(&m_Weights_, weightCount_);
    mallocZero(&v_Weights_, weightCount_);
    mallocZero(&m_Bias_, (size_t)outC_);
    mallocZero(&v_Bias_, (size_t)outC_);
  }
  SyncWeights();
}
FCLayer::~FCLayer() {
  aig_conv_plan_destroy(plan_);
  if (!weightsInPlan_) cudaFree(weights_);
  aig_fc_backward_plan_destroy(backward_);
  cudaFree(bias_); cudaFree(outData_);
  cudaFree(gradWeights_); cudaFree(gradBias_); cudaFree(gradOut_);
  cudaFree(m_Weights_); cudaFree(v_Weights_); cudaFree(m_Bias_); cudaFree(v_Bias_);
}
void FCLayer::SyncWeights() {
  check(ctx_, aig_fc_plan_set_weights(plan_, H(weights_), H(bias_), nullptr, nullptr, nullptr, nullptr, 0.f), layerName_);
}
__half* FCLayer::Forward(__half* data) {
  inData_ = data;
  check(ctx_, aig_conv_forward(plan_, H(data), nullptr, H(outData_)), layerName_);
  return outData_;
}
__half* FCLayer::Backward(__half* grad) {
  if (!backward_ || !inData_) throw std::runtime_error(std::string(layerName_) + ": Backward needs train = true and a Forward before it");
  check(ctx_, aig_fc_backward(backward_, H(inData_), H(grad), H(weights_), H(gradWeights_), H(gradBias_), H(gradOut_)), layerName_);
  return gradOut_;
}
void FCLayer::UpdateParameters(float learningRate) {
  if (!backward_) throw std::runtime_error(std::string(layerName_) + ": UpdateParameters needs train = true");
  check(ctx_, aig_fc_adamw_update(ctx_, plan_, inC_, outC_, H(weights_), H(gradWeights_), H(m_Weights_), H(v_Weights_), H(bias_), H(gradBias_),
                                  H(m_Bias_), H(v_Bias_), learningRate, t_, weightDecay_), layerName_);
  ++t_;
}
void FCLayer::SaveOptimizerState(std::ofstream& file, unsigned char* buffer) {
  if (!backward_) return;
  saveArray(ctx_, file, buffer, m_Weights_, weightCount_ * sizeof(__half));
  saveArray(ctx_, file, buffer, v_Weights_, weightCount_ * sizeof(__half));
  saveArray(ctx_, file, buffer, m_Bias_, outC_ * sizeof(__half));
  saveArray(ctx_, file, buffer, v_Bias_, outC_ * sizeof(__half));
}
void FCLayer::LoadOptimizerState(std::ifstream& file, unsigned char* buffer) {
  if (!backward_) return;
  loadArray(file, buffer, m_Weights_, weightCount_ * sizeof(__half));
  loadArray(file, buffer, v_Weights_, weightCount_ * sizeof(__half));
  loadArray(file, buffer, m_Bias_, outC_ * sizeof(__half));
  loadArray(file, buffer, v_Bias_, outC_ * sizeof(__half));
}
void FCLayer::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  loadArray(file, buffer, weights_, weightCount_ * sizeof(__half));
  loadArray(file, buffer, bias_, outC_ * sizeof(__half));
  SyncWeights();
}
void FCLayer::SaveParameters(std::ofstream& file, unsigned char* buffer) {
  saveArray(ctx_, file, buffer, weights_, weightCount_ * sizeof(__half));
  saveArray(ctx_, file, buffer, bias_, outC_ * sizeof(__half));
}

// ------------------------------------------------------------------------------------------ ResConvLayer
ResConvLayer::ResConvLayer(cudnnHandle_t cudnnHandle, int batchSize, int inChannels, int outChannels, int* inHeight, int* inWidth,
                           const char* layerName, bool train)
    : ctx_(cudnnHandle), batchSize_(batchSize) {
  layerName_ = layerName;
  train_ = train;
  constexpr float wd = 0.000001f;
  int resH = *inHeight, resW = *inWidth;
  // ResConvLayer.cpp:13-21
  layers_.push_back(new ConvLayer(ctx_, batchSize_, inChannels, outChannels, 4, 2, 1, inHeight, inWidth, "Conv0", train, wd));
  layers_.push_back(new BatchNorm(ctx_, CUDNN_BATCHNORM_SPATIAL, batchSize_, outChannels, *inHeight, *inWidth, "Conv0 BatchNorm", train, wd));
  layers_.push_back(new Activate(ctx_, CUDNN_ACTIVATION_RELU, 1.0, batchSize_, outChannels, *inHeight, *inWidth, "Conv0 ReLU"));
  layers_.push_back(new ConvLayer(ctx_, batchSize_, outChannels, outChannels, 3, 1, 1, inHeight, inWidth, "Conv1", train, wd));
  layers_.push_back(new BatchNorm(ctx_, CUDNN_BATCHNORM_SPATIAL, batchSize_, outChannels, *inHeight, *inWidth, "Conv1 BatchNorm", train, wd));
  residue_ = new ConvLayer(ctx_, batchSize_, inChannels, outChannels, 2, 2, 0, &resH, &resW, "Residue", train, wd);
  if (resH != *inHeight || resW != *inWidth) throw std::runtime_error("ResConvLayer: main and shortcut output sizes differ");
  resAct_ = new Activate(ctx_, CUDNN_ACTIVATION_RELU, 1.0, batchSize_, outChannels, *inHeight, *inWidth, "Residue ReLU");
  outNCHW_ = batchSize_ * outChannels * *inHeight * *inWidth;
  outDesc_ = {batchSize_, outChannels, *inHeight, *inWidth};
}
ResConvLayer::~ResConvLayer() {
  for (Layer* l : layers_) delete l;
  delete residue_;
  delete resAct_;
}
__half* ResConvLayer::Forward(__half* data) {
  // ResConvLayer.cpp:28-37
  __half* residue = residue_->Forward(data);
  for (Layer* l : layers_) data = l->Forward(data);
  check(ctx_, aig_add_forward(ctx_, H(data), H(residue), outNCHW_), layerName_);
  return resAct_->Forward(data);
}
void ResConvLayer::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  for (Layer* l : layers_) l->LoadParameters(file, buffer);
  residue_->LoadParameters(file, buffer);
}
void ResConvLayer::SaveParameters(std::ofstream& file, unsigned char* buffer) {
  for (Layer* l : layers_) l->SaveParameters(file, buffer);
  residue_->SaveParameters(file, buffer);
}
size_t ResConvLayer::GetParameterSize() {
  size_t m = residue_->GetParameterSize();
  for (Layer* l : layers_) m = std::max(m, l->GetParameterSize());
  return m;
}

// ------------------------------------------------------------------------------------------ LayerNorm
LayerNorm::LayerNorm(int batchSize, int channels, int height, int width, const char* layerName, float)
    : n_(batchSize), c_(channels), hw_(height * width) {
  layerName_ = layerName;
  outNCHW_ = n_ * c_ * hw_;
  outDesc_ = {n_, c_, height, width};
  mallocZero(&gamma_, (size_t)c_);
  mallocZero(&beta_, (size_t)c_);
  mallocZero(&mean_, (size_t)c_);
  mallocZero(&variance_, (size_t)c_);
  mallocZero(&outData_, (size_t)outNCHW_);
  fillOnes(gamma_, (size_t)c_);
}
LayerNorm::~LayerNorm() { cudaFree(gamma_); cudaFree(beta_); cudaFree(mean_); cudaFree(variance_); cudaFree(outData_); }
__half* LayerNorm::Forward(__half* data) {
  check(aigDefaultContext(), aig_layernorm_forward(aigDefaultContext(), H(outData_), H(data), gamma_, beta_, mean_, variance_, n_, c_, hw_, 1e-7f),
        layerName_);
  return outData_;
}
void LayerNorm::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  loadArray(file, buffer, gamma_, c_ * sizeof(float));
  loadArray(file, buffer, beta_, c_ * sizeof(float));
}
void LayerNorm::SaveParameters(std::ofstream& file, unsigned char* buffer) {  // LayerNorm.cpp:50-55
  saveArray(nullptr, file, buffer, gamma_, c_ * sizeof(float));
  saveArray(nullptr, file, buffer, beta_, c_ * sizeof(float));
}

// ------------------------------------------------------------------------------------------ SpatialAttentionLayer
SpatialAttentionLayer::SpatialAttentionLayer(cudnnHandle_t cudnnHandle, int attentionChannels, int batchSize, int channels, int height,
                                             int width, const char* layerName, bool train, float)
    : ctx_(cudnnHandle), attC_(attentionChannels), batchSize_(batchSize), inC_(channels), inH_(height), inW_(width) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  outNCHW_ = batchSize_ * inC_ * inH_ * inW_;
  outDesc_ = {batchSize_, inC_, inH_, inW_};
  const size_t kq = std::max((size_t)inC_ * 9, (size_t)attC_ * inC_);
  const size_t maps = std::max((size_t)outNCHW_, (size_t)batchSize_ * inH_ * inW_ * attC_);
  mallocZero(&keyWeights_, kq);
  mallocZero(&queryWeights_, kq);
  mallocZero(&valueWeights_, (size_t)inC_ * attC_);
  mallocZero(&keyMap_, maps);
  mallocZero(&queryMap_, maps);
  mallocZero(&valueMap_, maps);
  mallocZero(&attentionScores_, (size_t)batchSize_ * attC_ * inH_ * inW_);
  mallocZero(&outData_, maps);
}
SpatialAttentionLayer::~SpatialAttentionLayer() {
  __half* bufs[] = {keyWeights_, queryWeights_, valueWeights_, keyMap_, queryMap_, valueMap_, attentionScores_, outData_};
  for (__half* b : bufs) cudaFree(b);
}
__half* SpatialAttentionLayer::Forward(__half* data) {
  check(ctx_, aig_spatial_attention_forward(ctx_, H(data), H(keyWeights_), H(queryWeights_), H(valueWeights_), H(keyMap_), H(queryMap_),
                                            H(valueMap_), H(attentionScores_), H(outData_), batchSize_, inC_, attC_, inH_, inW_, group_),
        layerName_);
  return outData_;
}
void SpatialAttentionLayer::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  loadArray(file, buffer, keyWeights_, (size_t)inC_ * 9 * sizeof(__half));
  loadArray(file, buffer, queryWeights_, (size_t)inC_ * 9 * sizeof(__half));
  loadArray(file, buffer, valueWeights_, (size_t)inC_ * attC_ * sizeof(__half));
}
void SpatialAttentionLayer::SaveParameters(std::ofstream& file, unsigned char* buffer) {  // SpatialAttentionLayer.cpp:143-150
  saveArray(ctx_, file, buffer, keyWeights_, (size_t)inC_ * 9 * sizeof(__half));
  saveArray(ctx_, file, buffer, queryWeights_, (size_t)inC_ * 9 * sizeof(__half));
  saveArray(ctx_, file, buffer, valueWeights_, (size_t)inC_ * attC_ * sizeof(__half));
}

// ------------------------------------------------------------------------------------------ LSTMLayer
void LSTMLayer::init(const char* layerName, bool train, float clip, int doubleBias, int batchMajor) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  check(ctx_, aig_lstm_plan_create(ctx_, seq_, layers_, hidden_, batch_, inC_, clip, doubleBias, batchMajor, &plan_), layerName);
  weightCount_ = aig_lstm_weight_count(inC_, hidden_, layers_, doubleBias);
  mallocZero(&weights_, weightCount_);
  mallocZero(&outData_, (size_t)seq_ * batch_ * hidden_);
  mallocZero(&hy_, (size_t)layers_ * batch_ * hidden_);
  mallocZero(&cy_, (size_t)layers_ * batch_ * hidden_);
  outNCHW_ = batch_ * hidden_;
  outDesc_ = {batch_, hidden_, 1, 1};
  check(ctx_, aig_lstm_plan_set_weights(plan_, H(weights_)), layerName);
}
// LSTMLayer.cpp:4-40: cell clip +-5 (:15), two bias vectors per gate (the library default), seq-major tensors
LSTMLayer::LSTMLayer(cudnnHandle_t cudnnHandle, int seqLength, int numLayers, int hiddenSize, int batchSize, int inC, const char* layerName,
                     bool train)
    : ctx_(cudnnHandle), seq_(seqLength), layers_(numLayers), hidden_(hiddenSize), batch_(batchSize), inC_(inC), v8_(false) {
  init(layerName, train, 5.0f, 1, 0);
}
// LSTMLayerv8.cpp:4-9: CUDNN_RNN_SINGLE_INP_BIAS, no cell clip, CUDNN_RNN_DATA_LAYOUT_BATCH_MAJOR_UNPACKED
LSTMLayer::LSTMLayer(cudnnHandle_t cudnnHandle, cublasHandle_t, int batchSize, int seqLength, int inCHW, int outC, int numLayers,
                     const char* layerName, bool train)
    : ctx_(cudnnHandle), seq_(seqLength), layers_(numLayers), hidden_(outC), batch_(batchSize), inC_(inCHW), v8_(true) {
  init(layerName, train, 0.0f, 0, 1);
}
LSTMLayer::~LSTMLayer() {
  aig_lstm_plan_destroy(plan_);
  cudaFree(weights_); cudaFree(outData_); cudaFree(hy_); cudaFree(cy_);
}
__half* LSTMLayer::Forward(__half* data) {
  check(ctx_, aig_lstm_forward(plan_, H(data), H(outData_), H(hy_), H(cy_), 0), layerName_);
  if (v8_) return hy_;  // LSTMLayerv8.cpp:81: the final hidden state of every layer, [layers][batch][hidden]
  return outData_ + (size_t)(seq_ - 1) * batch_ * hidden_;  // LSTMLayer.cpp:103: the last step's rows
}
void LSTMLayer::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  loadArray(file, buffer, weights_, weightCount_ * sizeof(__half));
  // the input projection keeps its own packed copy of W and the folded biases: refresh it
  check(ctx_, aig_lstm_plan_set_weights(plan_, H(weights_)), layerName_);
}
void LSTMLayer::SaveParameters(std::ofstream& file, unsigned char* buffer) {  // LSTMLayer.cpp:139-142
  saveArray(ctx_, file, buffer, weights_, weightCount_ * sizeof(__half));
}

// ------------------------------------------------------------------------------------------ MultiHeadAttentionLayer
MultiHeadAttentionLayer::MultiHeadAttentionLayer(cudnnHandle_t cudnnHandle, cublasHandle_t, int batchSize, int seqLength, int embedSize,
                                                 int numHeads, const char* layerName, bool train, float)
    : ctx_(cudnnHandle), batch_(batchSize), seq_(seqLength), embed_(embedSize), heads_(numHeads) {
  g_default_ctx = ctx_;
  layerName_ = layerName;
  train_ = train;
  check(ctx_, aig_mha_plan_create(ctx_, batch_, seq_, embed_, heads_, 0.f, 0, &plan_), layerName);
  const size_t ee = (size_t)embed_ * embed_;
  mallocZero(&wq_, ee); mallocZero(&wk_, ee); mallocZero(&wv_, ee); mallocZero(&wo_, ee);
  mallocZero(&outData_, (size_t)batch_ * seq_ * embed_);
  weightCount_ = 4 * ee;
  outNCHW_ = batch_ * seq_ * embed_;
  outDesc_ = {batch_, seq_, embed_, 1};
  check(ctx_, aig_mha_plan_set_weights(plan_, H(wq_), H(wk_), H(wv_), H(wo_)), layerName);
}
MultiHeadAttentionLayer::~MultiHeadAttentionLayer() {
  aig_mha_plan_destroy(plan_);
  cudaFree(wq_); cudaFree(wk_); cudaFree(wv_); cudaFree(wo_); cudaFree(outData_);
}
__half* MultiHeadAttentionLayer::Forward(__half* data) {
  check(ctx_, aig_mha_forward(plan_, H(data), H(outData_), 0), layerName_);
  return outData_;
}
void MultiHeadAttentionLayer::LoadParameters(std::ifstream& file, unsigned char* buffer) {
  const size_t bytes = (size_t)embed_ * embed_ * sizeof(__half);
  loadArray(file, buffer, wq_, bytes);
  loadArray(file, buffer, wk_, bytes);
  loadArray(file, buffer, wv_, bytes);
  loadArray(file, buffer, wo_, bytes);
  check(ctx_, aig_mha_plan_set_weights(plan_, H(wq_), H(wk_), H(wv_), H(wo_)), layerName_);
}
void MultiHeadAttentionLayer::SaveParameters(std::ofstream& file, unsigned char* buffer) {  // MHALayer.cpp:191-200
  const size_t bytes = (size_t)embed_ * embed_ * sizeof(__half);
  saveArray(ctx_, file, buffer, wq_, bytes);
  saveArray(ctx_, file, buffer, wk_, bytes);
  saveArray(ctx_, file, buffer, wv_, bytes);
  saveArray(ctx_, file, buffer, wo_, bytes);
}

// ------------------------------------------------------------------------------------------ NN
NN::NN(cudnnHandle_t cudnnHandle, cublasHandle_t cublasHandle, int w, int h, bool train, const std::string& ckptFileName)
    : cudnn_(cudnnHandle), cublas_(cublasHandle), batchSize_(40), seqLength_(1), inWidth_(0), inHeight_(0), maxBufferSize_(0) {
  if (!train) batchSize_ = 1;  // NN.cpp:12
  std::ifstream ckptFile(ckptFileName, std::ios::binary);
  const bool fileOpen = ckptFile.is_open();
  int netWidth = w, netHeight = h;
  if (fileOpen) {  // NN.cpp:17-20
    ckptFile.read(reinterpret_cast<char*>(&netWidth), sizeof(int));
    ckptFile.read(reinterpret_cast<char*>(&netHeight), sizeof(int));
  }
  inWidth_ = netWidth;
  inHeight_ = netHeight;
  constexpr float wd = 0.000001f;
  int outC = 32;  // NN.cpp:33-61
  layers_.push_back(new ConvLayer(cudnn_, batchSize_, 3, outC, 2, 2, 0, &netHeight, &netWidth, "Conv0", train, wd));
  layers_.push_back(new BatchNorm(cudnn_, CUDNN_BATCHNORM_SPATIAL, batchSize_, outC, netHeight, netWidth, "Conv0 BatchNorm", train, wd));
  layers_.push_back(new Activate(cudnn_, CUDNN_ACTIVATION_RELU, 1.0, batchSize_, outC, netHeight, netWidth, "Conv0 ReLU"));
  layers_.push_back(new ResConvLayer(cudnn_, batchSize_, 32, 64, &netHeight, &netWidth, "ResConv0", train));
  layers_.push_back(new ResConvLayer(cudnn_, batchSize_, 64, 128, &netHeight, &netWidth, "ResConv1", train));
  layers_.push_back(new ResConvLayer(cudnn_, batchSize_, 128, 256, &netHeight, &netWidth, "ResConv2", train));
  outC = 1024;
  layers_.push_back(new FCLayer(cudnn_, cublas_, batchSize_, 256 * netHeight * netWidth, outC, "FC0", train, wd));
  layers_.push_back(new BatchNorm(cudnn_, CUDNN_BATCHNORM_PER_ACTIVATION, batchSize_, outC, 1, 1, "FC0 BatchNorm", train, wd));
  layers_.push_back(new Activate(cudnn_, CUDNN_ACTIVATION_RELU, 1.0, batchSize_, outC, 1, 1, "FC0 ReLU"));
  outC = 512;
  layers_.push_back(new FCLayer(cudnn_, cublas_, batchSize_, 1024, outC, "FC1", train, wd));
  layers_.push_back(new BatchNorm(cudnn_, CUDNN_BATCHNORM_PER_ACTIVATION, batchSize_, outC, 1, 1, "FC1 BatchNorm", train, wd));
  layers_.push_back(new Activate(cudnn_, CUDNN_ACTIVATION_RELU, 1.0, batchSize_, outC, 1, 1, "FC1 ReLU"));
  outC = 256;
  layers_.push_back(new FCLayer(cudnn_, cublas_, batchSize_, 512, outC, "FC2", train, wd));
  layers_.push_back(new BatchNorm(cudnn_, CUDNN_BATCHNORM_PER_ACTIVATION, batchSize_, outC, 1, 1, "FC2 BatchNorm", train, wd));
  layers_.push_back(new Activate(cudnn_, CUDNN_ACTIVATION_RELU, 1.0, batchSize_, outC, 1, 1, "FC2 ReLU"));
  outC = numCtrls_;
  layers_.push_back(new FCLayer(cudnn_, cublas_, batchSize_, 256, outC, "FC Out", train, wd));
  layers_.push_back(new Sigmoid(numButs_, batchSize_, outC, "Sigmoid"));
  for (Layer* layer : layers_) maxBufferSize_ = std::max(maxBufferSize_, layer->GetParameterSize());
  if (fileOpen) {  // NN.cpp:64-75
    unsigned char* buffer = nullptr;
    checkCuda(cudaMallocHost(reinterpret_cast<void**>(&buffer), maxBufferSize_), "cudaMallocHost");
    try {
      for (Layer* layer : layers_) layer->LoadParameters(ckptFile, buffer);
    } catch (...) {
      cudaFreeHost(buffer);
      throw;
    }
    cudaFreeHost(buffer);
  }
}
NN::~NN() {
  for (Layer* l : layers_) delete l;
}
__half* NN::Forward(__half* data) {  // NN.cpp:93-100
  for (Layer* layer : layers_) data = layer->Forward(data);
  return data;
}

// ------------------------------------------------------------------------------------------ C hooks (tests, other languages)
extern "C" {

static thread_local std::string g_layers_error;
const char* aig_layers_last_error() { return g_layers_error.c_str(); }

// new NN(handle, handle, w, h, /*train*/false, ckpt_path): the reference's own network through the layer classes
int aig_refnn_create(aig_ctx* ctx, int w, int h, const char* ckpt_path, void** out) {
  if (!ctx || !ckpt_path || !out) return AIG_ERR_INVALID;
  try {
    *out = new NN(ctx, ctx, w, h, false, ckpt_path);
    return AIG_OK;
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_INVALID;
  }
}
// NN::Forward on one planar fp16 frame [3][h][w]; *out_dev = the network's output buffer (numCtrls_ halves)
int aig_refnn_forward(void* nn, aig_half* x_nchw_dev, const aig_half** out_dev) {
  if (!nn || !x_nchw_dev || !out_dev) return AIG_ERR_INVALID;
  try {
    *out_dev = reinterpret_cast<const aig_half*>(static_cast<NN*>(nn)->Forward(reinterpret_cast<__half*>(x_nchw_dev)));
    return AIG_OK;
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_CUDA;
  }
}
// cudnnCreate as the reference calls it (Infer.cpp:76-79): a handle on the legacy default stream
int aig_compat_handle_create(aig_ctx** out) { return out ? cudnnCreate(out) : AIG_ERR_INVALID; }

// The loop body of Infer::Inference (Infer.cpp:103-112) written with the reference's own names and nothing
// added: ARGBtoRGBplanar (inside GrabFrameInt8, NvDisplayCap.h:70-87), ConvertAndNormalize, NN::Forward,
// ConvertHalfToFloat, cudaMemcpy device-to-host.  No stream or event call appears, as in the reference: the
// order comes from the legacy default stream, so `nn` must have been built on a handle from
// aig_compat_handle_create (or cudnnCreate of cudnn_shim.h).  planar_dev: 3*w*h bytes, frame_half_dev: 3*w*h
// halves, out_f32_dev / out_host: numCtrls_ floats.
int aig_refnn_infer_frame(void* nn, unsigned char* bgra_dev, unsigned char* planar_dev, aig_half* frame_half_dev, float* out_f32_dev,
                          float* out_host) {
  if (!nn || !bgra_dev || !planar_dev || !frame_half_dev || !out_f32_dev || !out_host) return AIG_ERR_INVALID;
  NN* net = static_cast<NN*>(nn);
  const int n = net->inWidth_ * net->inHeight_;
  try {
    if (ARGBtoRGBplanar(bgra_dev, planar_dev, n) != cudaSuccess) throw std::runtime_error("ARGBtoRGBplanar failed");
    ConvertAndNormalize(reinterpret_cast<__half*>(frame_half_dev), planar_dev, (size_t)3 * n);
    __half* out = net->Forward(reinterpret_cast<__half*>(frame_half_dev));
    ConvertHalfToFloat(out, out_f32_dev, numCtrls_);
    checkCuda(cudaMemcpy(out_host, out_f32_dev, numCtrls_ * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
    return aig_compat_last_status();
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_CUDA;
  }
}
int aig_refnn_input_size(void* nn, int* w, int* h) {
  if (!nn) return AIG_ERR_INVALID;
  if (w) *w = static_cast<NN*>(nn)->inWidth_;
  if (h) *h = static_cast<NN*>(nn)->inHeight_;
  return AIG_OK;
}
int aig_refnn_destroy(void* nn) {
  delete static_cast<NN*>(nn);
  return AIG_OK;
}

// One hook per use of a layer object, for every class of Layers.h: `kind` is the class name ("LSTMLayerV8" picks the
// LSTMLayerv8.h:10 constructor) and iargs are the constructor's integer arguments in declaration order (the
// int* size arguments are passed by value).  Handle-less classes run on `ctx` too.
int aig_layer_create(aig_ctx* ctx, const char* kind, const int* a, int n, void** out) {
  if (!ctx || !kind || !a || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  const std::string k(kind);
  auto need = [&](int want) {
    if (n != want) throw std::runtime_error(k + ": expected " + std::to_string(want) + " integer arguments");
  };
  try {
    aigSetDefaultContext(ctx);
    constexpr float wd = 0.000001f;
    Layer* L = nullptr;
    if (k == "ConvLayer") { need(8); int h = a[6], w = a[7]; L = new ConvLayer(ctx, a[0], a[1], a[2], a[3], a[4], a[5], &h, &w, "ConvLayer", false, wd); }
    else if (k == "ConvLayer3D") { need(12); int w = a[9], h = a[10], d = a[11]; L = new ConvLayer3D(ctx, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], &w, &h, &d, "ConvLayer3D", false, wd); }
    else if (k == "BatchNorm") { need(5); L = new BatchNorm(ctx, a[0] ? CUDNN_BATCHNORM_SPATIAL : CUDNN_BATCHNORM_PER_ACTIVATION, a[1], a[2], a[3], a[4], "BatchNorm", false, wd); }
    else if (k == "Activate") { need(4); L = new Activate(ctx, CUDNN_ACTIVATION_RELU, 1.0, a[0], a[1], a[2], a[3], "Activate"); }
    else if (k == "Swish") { need(1); L = new Swish(a[0], "Swish"); }
    else if (k == "LeakyReLU") { need(1); L = new LeakyReLU(a[0], "LeakyReLU"); }
    else if (k == "Sigmoid") { need(3); L = new Sigmoid(a[0], a[1], a[2], "Sigmoid"); }
    else if (k == "FCLayer") { need(3); L = new FCLayer(ctx, ctx, a[0], a[1], a[2], "FCLayer", false, wd); }
    else if (k == "FCLayerTrain") { need(3); L = new FCLayer(ctx, ctx, a[0], a[1], a[2], "FCLayer", true, wd); }
    else if (k == "ResConvLayer") { need(5); int h = a[3], w = a[4]; L = new ResConvLayer(ctx, a[0], a[1], a[2], &h, &w, "ResConvLayer", false); }
    else if (k == "LayerNorm") { need(4); L = new LayerNorm(a[0], a[1], a[2], a[3], "LayerNorm", wd); }
    else if (k == "SpatialAttentionLayer") { need(5); L = new SpatialAttentionLayer(ctx, a[0], a[1], a[2], a[3], a[4], "SpatialAttention", false, wd); }
    else if (k == "LSTMLayer") { need(5); L = new LSTMLayer(ctx, a[0], a[1], a[2], a[3], a[4], "LSTM", false); }
    else if (k == "LSTMLayerV8") { need(5); L = new LSTMLayer(ctx, ctx, a[0], a[1], a[2], a[3], a[4], "LSTM", false); }
    else if (k == "MultiHeadAttentionLayer") { need(4); L = new MultiHeadAttentionLayer(ctx, ctx, a[0], a[1], a[2], a[3], "MHA", false, wd); }
    else if (k == "Dropout") { need(4); L = new Dropout(ctx, 0.5f, a[0], a[1], a[2], a[3], "Dropout", false); }
    else throw std::runtime_error("unknown layer class " + k);
    *out = L;
    return AIG_OK;
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_INVALID;
  }
}
// Layer::Forward: x and *out_dev are device pointers in the layer's own (reference) layout
int aig_layer_forward(void* layer, aig_half* x, const aig_half** out_dev) {
  if (!layer || !x || !out_dev) return AIG_ERR_INVALID;
  try {
    *out_dev = reinterpret_cast<const aig_half*>(static_cast<Layer*>(layer)->Forward(reinterpret_cast<__half*>(x)));
    return AIG_OK;
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_CUDA;
  }
}
// Layer::Backward / Layer::UpdateParameters (Layer.h:8-9); of the classes here FCLayer created as "FCLayerTrain"
// implements them, the others return a null gradient as the base class does
int aig_layer_backward(void* layer, aig_half* grad, const aig_half** grad_in_dev) {
  if (!layer || !grad || !grad_in_dev) return AIG_ERR_INVALID;
  try {
    *grad_in_dev = reinterpret_cast<const aig_half*>(static_cast<Layer*>(layer)->Backward(reinterpret_cast<__half*>(grad)));
    return AIG_OK;
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_CUDA;
  }
}
int aig_layer_update(void* layer, float learning_rate) {
  if (!layer) return AIG_ERR_INVALID;
  try {
    static_cast<Layer*>(layer)->UpdateParameters(learning_rate);
    return AIG_OK;
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    return AIG_ERR_CUDA;
  }
}
size_t aig_layer_param_bytes(void* layer) { return layer ? static_cast<Layer*>(layer)->GetParameterSize() : 0; }
int aig_layer_out_count(void* layer) { return layer ? static_cast<Layer*>(layer)->outNCHW_ : 0; }
// Layer::LoadParameters / SaveParameters on a file that holds exactly this layer's payload, through a pinned
// staging buffer of GetParameterSize() bytes like NN.cpp:62-75 and :113-128 provide.
static int layer_file_io(void* layer, const char* path, bool save) {
  if (!layer || !path) return AIG_ERR_INVALID;
  Layer* L = static_cast<Layer*>(layer);
  unsigned char* buffer = nullptr;
  const size_t n = L->GetParameterSize();
  if (cudaMallocHost(reinterpret_cast<void**>(&buffer), n ? n : 1) != cudaSuccess) return AIG_ERR_CUDA;
  int rc = AIG_OK;
  try {
    if (save) {
      std::ofstream f(path, std::ios::binary);
      if (!f.is_open()) throw std::runtime_error(std::string("cannot write ") + path);
      L->SaveParameters(f, buffer);
    } else {
      std::ifstream f(path, std::ios::binary);
      if (!f.is_open()) throw std::runtime_error(std::string("cannot read ") + path);
      L->LoadParameters(f, buffer);
    }
  } catch (const std::exception& e) {
    g_layers_error = e.what();
    rc = AIG_ERR_IO;
  }
  cudaFreeHost(buffer);
  return rc;
}
int aig_layer_load_file(void* layer, const char* path) { return layer_file_io(layer, path, false); }
int aig_layer_save_file(void* layer, const char* path) { return layer_file_io(layer, path, true); }
int aig_layer_destroy(void* layer) {
  delete static_cast<Layer*>(layer);
  return AIG_OK;
}

}  // extern "C"
