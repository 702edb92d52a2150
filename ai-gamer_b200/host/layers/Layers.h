// Layers.h -- the reference's operator API (Layer.h:5-22 and one class per layer file) implemented on
// the B200 kernel ABI.  Class names, constructor argument lists, the virtual interface and the
// public data members match the reference so that caller code written against it (NN.cpp:33-61,
// ResConvLayer.cpp:13-21) compiles unchanged; `cudnnHandle_t` / `cublasHandle_t` are this library's
// context (cudnn_shim.h).  Contract kept from the reference: every Forward takes and returns NCHW
// fp16 device pointers, the returned buffer is owned by the layer, activations work in place and
// return their argument, LoadParameters reads the layer's payload from the stream through the
// caller's staging buffer.  Backward/UpdateParameters/optimizer state are training-only and are
// not provided (they return nullptr / do nothing, like the reference's base class defaults).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <fstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "aig_b200.h"
#include "cudnn_shim.h"

// common.h:92-94
constexpr int numButs_ = 14;
constexpr int numAxes_ = 2;
constexpr int numCtrls_ = numButs_ + numAxes_;

// Layer.h:5-22
class Layer {
 public:
  virtual ~Layer() = default;
  virtual __half* Forward(__half* data) { return nullptr; }
  virtual __half* Backward(__half* grad) { return nullptr; }
  virtual void UpdateParameters(float learningRate) {}
  virtual void SaveParameters(std::ofstream& file, unsigned char* buffer) {}
  virtual void LoadParameters(std::ifstream& file, unsigned char* buffer) {}
  virtual void SaveOptimizerState(std::ofstream& file, unsigned char* buffer) {}
  virtual void LoadOptimizerState(std::ifstream& file, unsigned char* buffer) {}
  virtual size_t GetParameterSize() { return 0; }
  virtual size_t GetOptimizerStateSize() { return 0; }
  cudnnTensorDescriptor_t outDesc_{};
  int outNCHW_ = 0;
  const char* layerName_ = "";
  bool train_ = false;
  size_t weightCount_ = 0;
};

// ConvLayer.h:8 / ConvLayer.cpp:4-50,74-79
class ConvLayer final : public Layer {
 public:
  ConvLayer(cudnnHandle_t cudnnHandle, int batchSize, int inChannels, int outChannels, int filterSize, int stride, int padding,
            int* height, int* width, const char* layerName, bool train, float weightDecay);
  ~ConvLayer() override;
  __half* Forward(__half* data) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return (weightCount_ + outC_) * sizeof(__half); }
  void SyncWeights();  // push weights_/bias_ (device) into the kernel plan
  __half *weights_ = nullptr, *bias_ = nullptr, *outData_ = nullptr;
  int batchSize_, inC_, outC_, k_, stride_, pad_, inH_, inW_, outH_, outW_;

 private:
  aig_ctx* ctx_;
  aig_conv_plan* plan_ = nullptr;
  aig_conv0_plan* plan0_ = nullptr;
  __half *nhwcIn_ = nullptr, *nhwcOut_ = nullptr;
};

// ConvLayer3D.h:8 / ConvLayer3D.cpp:3-82,106-111
class ConvLayer3D final : public Layer {
 public:
  ConvLayer3D(cudnnHandle_t cudnnHandle, int batchSize, int inChannels, int outChannels, int filterSizeD, int filterSizeHW,
              int strideD, int strideHW, int paddingD, int paddingHW, int* width, int* height, int* depth, const char* layerName,
              bool train, float weightDecay);
  ~ConvLayer3D() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return (weightCount_ + outC_) * sizeof(__half); }
  void SyncWeights();
  __half *weights_ = nullptr, *bias_ = nullptr, *outData_ = nullptr;
  int batchSize_, inC_, outC_, inD_, inH_, inW_, outD_, outH_, outW_;

 private:
  aig_ctx* ctx_;
  aig_conv_plan* plan_ = nullptr;
  aig_conv0_plan* plan0_ = nullptr;
  __half *nhwcIn_ = nullptr, *nhwcOut_ = nullptr;
};

// BatchNorm.h:7 / BatchNorm.cpp:55-63 (inference branch), parameters per BatchNorm.cpp:90-117
class BatchNorm final : public Layer {
 public:
  BatchNorm(cudnnHandle_t cudnnHandle, cudnnBatchNormMode_t bnMode, int batchSize, int channels, int height, int width,
            const char* layerName, bool train, float weightDecay);
  ~BatchNorm() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return 6 * paramCount_ * sizeof(float); }
  float *bnScale_ = nullptr, *bnBias_ = nullptr, *bnRunningMean_ = nullptr, *bnRunningVar_ = nullptr, *bnSavedMean_ = nullptr,
        *bnSavedInvVariance_ = nullptr;
  __half* outData_ = nullptr;
  size_t paramCount_ = 0;

 private:
  aig_ctx* ctx_;
  cudnnBatchNormMode_t mode_;
  int batch_, c_, hw_;
};

// Activate.h:7 / Activate.cpp:17-21 (ReLU in place)
class Activate final : public Layer {
 public:
  Activate(cudnnHandle_t cudnnHandle, cudnnActivationMode_t mode, double coef, int batchSize, int channels, int height, int width,
           const char* layerName);
  __half* Forward(__half* data) override;

 private:
  aig_ctx* ctx_;
};

// Swish.h:6, LeakyReLU.h:7 (slope 1/128, LeakyReLU.cpp:3), Sigmoid.h:5 -- the reference builds these without a handle;
// they use the library's default context (aigDefaultContext()).
class Swish final : public Layer {
 public:
  Swish(int size, const char* layerName);
  __half* Forward(__half* data) override;
};
class LeakyReLU final : public Layer {
 public:
  LeakyReLU(int size, const char* layerName);
  __half* Forward(__half* data) override;
  float slope_ = 1.0f / 128.0f;
};
class Sigmoid final : public Layer {
 public:
  Sigmoid(int numSigmoidOutputs, int batchSize, int outC, const char* layerName);
  __half* Forward(__half* data) override;

 private:
  int numSigmoid_, outC_;
};

// FCLayer.h:8 / FCLayer.cpp:48-53
class FCLayer final : public Layer {
 public:
  FCLayer(cudnnHandle_t cudnnHandle, cublasHandle_t cublasHandle, int batchSize, int inputSize, int outputSize,
          const char* layerName, bool train, float weightDecay);
  ~FCLayer() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return (weightCount_ + outC_) * sizeof(__half); }
  // training mode (train = true in the constructor), FCLayer.cpp:54-70 and :83-104: Backward returns the gradient
  // with respect to the last Forward's input; UpdateParameters is the AdamW step on weights and bias
  __half* Backward(__half* grad) override;
  void UpdateParameters(float learningRate) override;
  void SaveOptimizerState(std::ofstream& file, unsigned char* buffer) override;
  void LoadOptimizerState(std::ifstream& file, unsigned char* buffer) override;
  size_t GetOptimizerStateSize() override { return weightCount_ * sizeof(__half); }
  void SyncWeights();
  __half *weights_ = nullptr, *bias_ = nullptr, *outData_ = nullptr;
  __half *gradOut_ = nullptr, *gradWeights_ = nullptr, *gradBias_ = nullptr;
  __half *m_Weights_ = nullptr, *v_Weights_ = nullptr, *m_Bias_ = nullptr, *v_Bias_ = nullptr;
  const __half* inData_ = nullptr;
  int t_ = 1;
  float weightDecay_;
  int batchSize_, inC_, outC_;

 private:
  aig_ctx* ctx_;
  aig_conv_plan* plan_ = nullptr;
  aig_fc_backward_plan* backward_ = nullptr;
  bool weightsInPlan_ = false;
};

// ResConvLayer.h:12 / ResConvLayer.cpp:8-37
class ResConvLayer final : public Layer {
 public:
  ResConvLayer(cudnnHandle_t cudnnHandle, int batchSize, int inChannels, int outChannels, int* inHeight, int* inWidth,
               const char* layerName, bool train);
  ~ResConvLayer() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override;
  std::vector<Layer*> layers_;
  ConvLayer* residue_ = nullptr;
  Layer* resAct_ = nullptr;

 private:
  aig_ctx* ctx_;
  int batchSize_;
};

// LayerNorm.h:6 / LayerNorm.cpp:36-40 (statistics per channel over N*H*W, eps 1e-7)
class LayerNorm final : public Layer {
 public:
  LayerNorm(int batchSize, int channels, int height, int width, const char* layerName, float weightDecay);
  ~LayerNorm() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return 2 * (size_t)c_ * sizeof(float); }
  float *gamma_ = nullptr, *beta_ = nullptr, *mean_ = nullptr, *variance_ = nullptr;
  __half* outData_ = nullptr;

 private:
  int n_, c_, hw_;
};

// SpatialAttentionLayer.h:7 / SpatialAttentionLayer.cpp:94-110.  Weight buffers hold attC*inC entries
// each (the reference allocates inC*9 for key/query but its kernel indexes attC*inC, CudaStuff.cu:713-714);
// the file payload keeps the reference's sizes (SpatialAttentionLayer.cpp:143-158).
class SpatialAttentionLayer final : public Layer {
 public:
  SpatialAttentionLayer(cudnnHandle_t cudnnHandle, int attentionChannels, int batchSize, int channels, int height, int width,
                        const char* layerName, bool train, float weightDecay);
  ~SpatialAttentionLayer() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return ((size_t)2 * inC_ * 9 + (size_t)inC_ * attC_) * sizeof(__half); }
  __half *keyWeights_ = nullptr, *queryWeights_ = nullptr, *valueWeights_ = nullptr, *keyMap_ = nullptr, *queryMap_ = nullptr,
         *valueMap_ = nullptr, *attentionScores_ = nullptr, *outData_ = nullptr;
  int group_ = 64;  // softmax group = the reference's launch block size on its build target

 private:
  aig_ctx* ctx_;
  int attC_, batchSize_, inC_, inH_, inW_;
};

// The reference has two files that both define `LSTMLayer` (they cannot be linked together); here both
// constructor forms live on one class.
//   LSTMLayer.h:8 / LSTMLayer.cpp:75-104 (cuDNN 7 API): seq-major x [T][B][inC], two bias vectors, cell clip 5,
//     Forward returns the last step's rows [B][hidden] inside outData_ [T][B][hidden].
//   LSTMLayerv8.h:10 / LSTMLayerv8.cpp:78-82 (cuDNN 8 API): batch-major x [B][T][inCHW], one bias vector, no
//     clip, Forward returns hy_ = the final hidden state of every layer [layers][B][outC]; outData_ holds the
//     whole output sequence [B][T][outC] (the reference's own outData_ is sized for one step only).
class LSTMLayer final : public Layer {
 public:
  LSTMLayer(cudnnHandle_t cudnnHandle, int seqLength, int numLayers, int hiddenSize, int batchSize, int inC, const char* layerName,
            bool train);
  LSTMLayer(cudnnHandle_t cudnnHandle, cublasHandle_t cublasHandle, int batchSize, int seqLength, int inCHW, int outC, int numLayers,
            const char* layerName, bool train);
  ~LSTMLayer() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return weightCount_ * sizeof(__half); }
  __half *weights_ = nullptr, *outData_ = nullptr, *hy_ = nullptr, *cy_ = nullptr;

 private:
  void init(const char* layerName, bool train, float clip, int doubleBias, int batchMajor);
  aig_ctx* ctx_;
  aig_lstm_plan* plan_ = nullptr;
  int seq_, layers_, hidden_, batch_, inC_;
  bool v8_;
};

// MHALayer.h:9 / MHALayer.cpp:128-146
class MultiHeadAttentionLayer final : public Layer {
 public:
  MultiHeadAttentionLayer(cudnnHandle_t cudnnHandle, cublasHandle_t cublasHandle, int batchSize, int seqLength, int embedSize,
                          int numHeads, const char* layerName, bool train, float weightDecay);
  ~MultiHeadAttentionLayer() override;
  __half* Forward(__half* data) override;
  void LoadParameters(std::ifstream& file, unsigned char* buffer) override;
  void SaveParameters(std::ofstream& file, unsigned char* buffer) override;
  size_t GetParameterSize() override { return 4 * (size_t)embed_ * embed_ * sizeof(__half); }
  __half *wq_ = nullptr, *wk_ = nullptr, *wv_ = nullptr, *wo_ = nullptr, *outData_ = nullptr;

 private:
  aig_ctx* ctx_;
  aig_mha_plan* plan_ = nullptr;
  int batch_, seq_, embed_, heads_;
};

// Dropout.h:8 / Dropout.cpp:20-25: identity at inference
class Dropout final : public Layer {
 public:
  Dropout(cudnnHandle_t, float, int, int, int, int, const char* layerName, bool train) {
    layerName_ = layerName;
    train_ = train;
  }
  __half* Forward(__half* data) override { return data; }
};

// NN.h / NN.cpp:11-100: the network the reference builds (Conv k2 s2 + BN + ReLU, three ResConv blocks, three
// FC+BN+ReLU, FC(16), Sigmoid(14)).  The checkpoint path is an argument instead of a fixed drive letter.
class NN {
 public:
  NN(cudnnHandle_t cudnnHandle, cublasHandle_t cublasHandle, int w, int h, bool train, const std::string& ckptFile);
  ~NN();
  __half* Forward(__half* data);
  cudnnHandle_t cudnn_;
  cublasHandle_t cublas_;
  std::vector<Layer*> layers_;
  int batchSize_, seqLength_, inWidth_, inHeight_;
  size_t maxBufferSize_;
};

// The context used by layers whose reference constructors take no handle (Swish, LeakyReLU, Sigmoid, LayerNorm):
// the context of the most recently constructed handle-taking layer, or of aigSetDefaultContext.
aig_ctx* aigDefaultContext();
void aigSetDefaultContext(aig_ctx* ctx);
