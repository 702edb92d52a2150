// ref_layers_hooks.cpp -- C hooks around the REFERENCE'S OWN layer classes (ConvLayer, BatchNorm, Activate,
// FCLayer (forward, and Backward / UpdateParameters in training mode), ResConvLayer, ConvLayer3D, LSTMLayer of
// LSTMLayerv8.cpp, LayerNorm, SpatialAttentionLayer, Swish, LeakyReLU, Sigmoid, NN), compiled from where they lie into oracle/_ref/libaig_reflayers.so together with the
// reference's CudaStuff.cu.  TEST INFRASTRUCTURE ONLY: GPU parity tests run these classes (which call cuDNN and
// cuBLAS exactly as the reference does) beside this repository's kernels on the same inputs, and the benchmark
// times them as "the reference's call pattern on this GPU".  Nothing here is linked into libaig_b200.so.
//
// Besides the hooks this file supplies the two functions the layer sources expect from common.cpp, which is
// Windows/MSVC-only (inline assembly, common.cpp:86-146) and cannot be compiled here:
//   GetConvolutionAlgorithms (common.cpp:371-396): the first algorithm cudnnGetConvolutionForwardAlgorithm_v7
//   returns, and its workspace size;  cublasGetErrorString (common.cpp:6-20): a status-to-text table.
// And one direct cuDNN call sequence, ref_cudnn_lstm_forward: the descriptor set-up of LSTMLayerv8.cpp:8-39
// (cuDNN-8 API) / LSTMLayer.cpp:9-40 (clip, two bias vectors) with an output buffer of the right size -- the
// class in LSTMLayerv8.cpp sizes its output for one step only (LSTMLayerv8.cpp:30) and never passes an initial
// state, so through the class itself the recurrent matrices can only be observed at sequence length 1.
#include "ref_compat.h"

#include <cstdlib>
#include <cstring>
#include <string>

#include "Activate.h"
#include "BatchNorm.h"
#include "ConvLayer.h"
#include "ConvLayer3D.h"
#include "FCLayer.h"
#include "LSTMLayerv8.h"
#include "LayerNorm.h"
#include "LeakyReLU.h"
#include "NN.h"
#include "ResConvLayer.h"
#include "Sigmoid.h"
#include "SpatialAttentionLayer.h"
#include "Swish.h"

const char* cublasGetErrorString(cublasStatus_t status) {
  switch (status) {
    case CUBLAS_STATUS_SUCCESS: return "CUBLAS_STATUS_SUCCESS";
    case CUBLAS_STATUS_NOT_INITIALIZED: return "CUBLAS_STATUS_NOT_INITIALIZED";
    case CUBLAS_STATUS_ALLOC_FAILED: return "CUBLAS_STATUS_ALLOC_FAILED";
    case CUBLAS_STATUS_INVALID_VALUE: return "CUBLAS_STATUS_INVALID_VALUE";
    case CUBLAS_STATUS_ARCH_MISMATCH: return "CUBLAS_STATUS_ARCH_MISMATCH";
    case CUBLAS_STATUS_EXECUTION_FAILED: return "CUBLAS_STATUS_EXECUTION_FAILED";
    case CUBLAS_STATUS_INTERNAL_ERROR: return "CUBLAS_STATUS_INTERNAL_ERROR";
    case CUBLAS_STATUS_NOT_SUPPORTED: return "CUBLAS_STATUS_NOT_SUPPORTED";
    default: return "cuBLAS status";
  }
}

ConvolutionAlgorithms GetConvolutionAlgorithms(cudnnHandle_t handle, cudnnTensorDescriptor_t x, cudnnFilterDescriptor_t w,
                                               cudnnConvolutionDescriptor_t conv, cudnnTensorDescriptor_t y, bool) {
  ConvolutionAlgorithms a{};
  cudnnConvolutionFwdAlgoPerf_t perf[10];
  int n = 0;
  checkCUDNN(cudnnGetConvolutionForwardAlgorithm_v7(handle, x, w, conv, y, 10, &n, perf));
  a.fwdAlgo = perf[0].algo;
  a.workspaceSize = perf[0].memory;
  a.bwdDataAlgo = CUDNN_CONVOLUTION_BWD_DATA_ALGO_0;
  a.bwdFilterAlgo = CUDNN_CONVOLUTION_BWD_FILTER_ALGO_0;
  return a;
}

namespace {
cudnnHandle_t g_cudnn = nullptr;
cublasHandle_t g_cublas = nullptr;
std::string g_err;
template <class F>
auto guarded(F&& f, decltype(f()) on_error) -> decltype(f()) {
  try {
    return f();
  } catch (const std::exception& e) {
    g_err = e.what();
    return on_error;
  }
}
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// Infer.cpp:75-79: InitCUDA, cudnnCreate, cublasCreate
int ref_init() {
  return guarded([&] {
    if (!g_cudnn) {
      InitCUDA();
      checkCUDNN(cudnnCreate(&g_cudnn));
      checkCUBLAS(cublasCreate(&g_cublas));
    }
    return 0;
  }, -1);
}

// kind = class name, a = the constructor's integer arguments in declaration order (sizes the reference passes
// as int* go by value); the same convention as aig_layer_create of the library under test
void* ref_layer_create(const char* kind, const int* a, int n) {
  return guarded([&]() -> void* {
    if (ref_init() != 0) return nullptr;
    const std::string k(kind);
    constexpr float wd = 0.000001f;
    auto need = [&](int want) {
      if (n != want) throw std::runtime_error(k + ": wrong number of integer arguments");
    };
    Layer* L = nullptr;
    if (k == "ConvLayer") { need(8); int h = a[6], w = a[7]; L = new ConvLayer(g_cudnn, a[0], a[1], a[2], a[3], a[4], a[5], &h, &w, "ConvLayer", false, wd); }
    else if (k == "ConvLayer3D") { need(12); int w = a[9], h = a[10], d = a[11]; L = new ConvLayer3D(g_cudnn, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], &w, &h, &d, "ConvLayer3D", false, wd); }
    else if (k == "BatchNorm") { need(5); L = new BatchNorm(g_cudnn, a[0] ? CUDNN_BATCHNORM_SPATIAL : CUDNN_BATCHNORM_PER_ACTIVATION, a[1], a[2], a[3], a[4], "BatchNorm", false, wd); }
    else if (k == "Activate") { need(4); L = new Activate(g_cudnn, CUDNN_ACTIVATION_RELU, 1.0, a[0], a[1], a[2], a[3], "Activate"); }
    else if (k == "Swish") { need(1); L = new Swish(a[0], "Swish"); }
    else if (k == "LeakyReLU") { need(1); L = new LeakyReLU(a[0], "LeakyReLU"); }
    else if (k == "Sigmoid") { need(3); L = new Sigmoid(a[0], a[1], a[2], "Sigmoid"); }
    else if (k == "FCLayer") { need(3); L = new FCLayer(g_cudnn, g_cublas, a[0], a[1], a[2], "FCLayer", false, wd); }
    else if (k == "FCLayerTrain") { need(3); L = new FCLayer(g_cudnn, g_cublas, a[0], a[1], a[2], "FCLayer", true, wd); }
    else if (k == "ResConvLayer") { need(5); int h = a[3], w = a[4]; L = new ResConvLayer(g_cudnn, a[0], a[1], a[2], &h, &w, "ResConvLayer", false); }
    else if (k == "LayerNorm") { need(4); L = new LayerNorm(a[0], a[1], a[2], a[3], "LayerNorm", wd); }
    else if (k == "SpatialAttentionLayer") { need(5); L = new SpatialAttentionLayer(g_cudnn, a[0], a[1], a[2], a[3], a[4], "SpatialAttention", false, wd); }
    else if (k == "LSTMLayerV8") { need(5); L = new LSTMLayer(g_cudnn, g_cublas, a[0], a[1], a[2], a[3], a[4], "LSTM", false); }
    else throw std::runtime_error("unknown layer class " + k);
    return L;
  }, nullptr);
}
const void* ref_layer_forward(void* layer, void* x) {
  return guarded([&]() -> const void* { return static_cast<Layer*>(layer)->Forward(static_cast<__half*>(x)); }, nullptr);
}
// FCLayer::Backward (FCLayer.cpp:54-59) on a layer created as "FCLayerTrain" after a Forward (which records the
// input): returns the input gradient and hands out the layer's weight / bias gradient buffers (device pointers)
const void* ref_fc_backward(void* layer, void* grad, const void** grad_w, const void** grad_b) {
  return guarded([&]() -> const void* {
    FCLayer* L = static_cast<FCLayer*>(layer);
    const void* gx = L->Backward(static_cast<__half*>(grad));
    if (grad_w) *grad_w = L->gradWeights_;
    if (grad_b) *grad_b = L->gradBias_;
    return gx;
  }, nullptr);
}
// Layer::UpdateParameters (AdamWHalf on weights and bias for FCLayer, FCLayer.cpp:60-70)
int ref_layer_update(void* layer, float lr) {
  return guarded([&] { static_cast<Layer*>(layer)->UpdateParameters(lr); return 0; }, -1);
}
size_t ref_layer_param_bytes(void* layer) { return static_cast<Layer*>(layer)->GetParameterSize(); }
int ref_layer_out_count(void* layer) { return static_cast<Layer*>(layer)->outNCHW_; }
static int file_io(Layer* L, const char* path, bool save) {
  return guarded([&] {
    unsigned char* buffer = nullptr;
    size_t n = std::max(L->GetParameterSize(), (size_t)1);
    checkCUDA(cudaMallocHost(reinterpret_cast<void**>(&buffer), n));
    if (save) {
      std::ofstream f(path, std::ios::binary);
      L->SaveParameters(f, buffer);
    } else {
      std::ifstream f(path, std::ios::binary);
      if (!f.is_open()) throw std::runtime_error("cannot open payload file");
      L->LoadParameters(f, buffer);
    }
    cudaFreeHost(buffer);
    return 0;
  }, -1);
}
int ref_layer_load_file(void* layer, const char* path) { return file_io(static_cast<Layer*>(layer), path, false); }
int ref_layer_save_file(void* layer, const char* path) { return file_io(static_cast<Layer*>(layer), path, true); }
void ref_layer_destroy(void* layer) { guarded([&] { delete static_cast<Layer*>(layer); return 0; }, -1); }

// new NN(cudnn, cublas, w, h, /*train*/false): the reference opens the checkpoint under its fixed name
// (common.h:88) relative to the current directory, so the caller changes into a directory that holds it
void* ref_nn_create(int w, int h) {
  return guarded([&]() -> void* { return ref_init() == 0 ? new NN(g_cudnn, g_cublas, w, h, false) : nullptr; }, nullptr);
}
const void* ref_nn_forward(void* nn, void* x) {
  return guarded([&]() -> const void* { return static_cast<NN*>(nn)->Forward(static_cast<__half*>(x)); }, nullptr);
}
int ref_nn_input_width(void* nn) { return static_cast<NN*>(nn)->inWidth_; }
int ref_nn_input_height(void* nn) { return static_cast<NN*>(nn)->inHeight_; }
const char* ref_checkpoint_name() { return ckptFileName.c_str(); }

// cuDNN's LSTM through the v8 API with the settings of the reference's two LSTM files: LSTM, unidirectional,
// linear input, standard algorithm, fp16 data and math precision, tensor-op math (LSTMLayerv8.cpp:9,
// LSTMLayer.cpp:13-16); clip > 0 sets the cell clip of LSTMLayer.cpp:15, double_bias the library's default two
// bias vectors (LSTMLayer.cpp) instead of the single input bias of LSTMLayerv8.cpp:9.  Weights arrive as the
// blob of the library under test (per layer W_i,W_f,W_g,W_o [hidden][in_l] then R_i..R_o [hidden][hidden]; then
// per layer bW_i..bW_o [and bR_i..bR_o]) on the HOST and are placed into cuDNN's weight space through
// cudnnGetRNNWeightParams (linear layer IDs 0-3 = input i,f,g,o, 4-7 = recurrent).  x,y device fp16:
// [T][B][.] or, batch_major, [B][T][.]; hy, cy [layers][B][hidden] or null.
int ref_cudnn_lstm_forward(const void* x, const void* blob_host, void* y, void* hy, void* cy, int T, int B, int in_c, int hidden,
                           int layers, float clip, int double_bias, int batch_major) {
  return guarded([&] {
    if (ref_init() != 0) return -1;
    cudnnRNNDescriptor_t rnn;
    checkCUDNN(cudnnCreateRNNDescriptor(&rnn));
    checkCUDNN(cudnnSetRNNDescriptor_v8(rnn, CUDNN_RNN_ALGO_STANDARD, CUDNN_LSTM, double_bias ? CUDNN_RNN_DOUBLE_BIAS : CUDNN_RNN_SINGLE_INP_BIAS,
                                        CUDNN_UNIDIRECTIONAL, CUDNN_LINEAR_INPUT, CUDNN_DATA_HALF, CUDNN_DATA_HALF, CUDNN_TENSOR_OP_MATH,
                                        in_c, hidden, hidden, layers, nullptr, batch_major ? CUDNN_RNN_PADDED_IO_ENABLED : 0));
    // (the batch-major unpacked layout needs the padded-IO flag in cuDNN 9; LSTMLayerv8.cpp:9 passes 0 there)
    if (clip > 0) checkCUDNN(cudnnRNNSetClip_v9(rnn, CUDNN_RNN_CLIP_MINMAX, -(double)clip, (double)clip));
    std::vector<int> lens(B, T);
    int* lens_dev = nullptr;
    checkCUDA(cudaMalloc(reinterpret_cast<void**>(&lens_dev), B * sizeof(int)));
    checkCUDA(cudaMemcpy(lens_dev, lens.data(), B * sizeof(int), cudaMemcpyHostToDevice));
    const cudnnRNNDataLayout_t layout = batch_major ? CUDNN_RNN_DATA_LAYOUT_BATCH_MAJOR_UNPACKED : CUDNN_RNN_DATA_LAYOUT_SEQ_MAJOR_UNPACKED;
    cudnnRNNDataDescriptor_t xd, yd;
    checkCUDNN(cudnnCreateRNNDataDescriptor(&xd));
    checkCUDNN(cudnnCreateRNNDataDescriptor(&yd));
    checkCUDNN(cudnnSetRNNDataDescriptor(xd, CUDNN_DATA_HALF, layout, T, B, in_c, lens.data(), nullptr));
    checkCUDNN(cudnnSetRNNDataDescriptor(yd, CUDNN_DATA_HALF, layout, T, B, hidden, lens.data(), nullptr));
    cudnnTensorDescriptor_t hd, cd;
    checkCUDNN(cudnnCreateTensorDescriptor(&hd));
    checkCUDNN(cudnnCreateTensorDescriptor(&cd));
    // hidden/cell state descriptors as the reference sets them: 4-D (layers, batch, hidden, 1), LSTMLayerv8.cpp:20-23
    checkCUDNN(cudnnSetTensor4dDescriptor(hd, CUDNN_TENSOR_NCHW, CUDNN_DATA_HALF, layers, B, hidden, 1));
    checkCUDNN(cudnnSetTensor4dDescriptor(cd, CUDNN_TENSOR_NCHW, CUDNN_DATA_HALF, layers, B, hidden, 1));
    if (getenv("REF_LSTM_ND3")) {
      const int dims[3] = {layers, B, hidden}, strides[3] = {B * hidden, hidden, 1};
      checkCUDNN(cudnnSetTensorNdDescriptor(hd, CUDNN_DATA_HALF, 3, dims, strides));
      checkCUDNN(cudnnSetTensorNdDescriptor(cd, CUDNN_DATA_HALF, 3, dims, strides));
    }
    size_t wbytes = 0, work = 0, reserve = 0;
    checkCUDNN(cudnnGetRNNWeightSpaceSize(g_cudnn, rnn, &wbytes));
    checkCUDNN(cudnnGetRNNTempSpaceSizes(g_cudnn, rnn, CUDNN_FWD_MODE_INFERENCE, xd, &work, &reserve));
    void *wdev = nullptr, *wsp = nullptr;
    checkCUDA(cudaMalloc(&wdev, wbytes));
    checkCUDA(cudaMemset(wdev, 0, wbytes));
    checkCUDA(cudaMalloc(&wsp, work ? work : 1));
    // place the matrices and biases
    std::vector<unsigned char> wspace(wbytes, 0);
    const __half* blob = static_cast<const __half*>(blob_host);
    size_t off = 0;
    std::vector<size_t> w_off(layers), r_off(layers), bw_off(layers), br_off(layers);
    for (int l = 0; l < layers; ++l) {
      w_off[l] = off; off += (size_t)4 * hidden * (l == 0 ? in_c : hidden);
      r_off[l] = off; off += (size_t)4 * hidden * hidden;
    }
    for (int l = 0; l < layers; ++l) {
      bw_off[l] = off; off += (size_t)4 * hidden;
      br_off[l] = off; if (double_bias) off += (size_t)4 * hidden;
    }
    cudnnTensorDescriptor_t md, bd;
    checkCUDNN(cudnnCreateTensorDescriptor(&md));
    checkCUDNN(cudnnCreateTensorDescriptor(&bd));
    for (int l = 0; l < layers; ++l) {
      const int in_l = l == 0 ? in_c : hidden;
      for (int id = 0; id < 8; ++id) {
        void *maddr = nullptr, *baddr = nullptr;
        checkCUDNN(cudnnGetRNNWeightParams(g_cudnn, rnn, l, wbytes, wdev, id, md, &maddr, bd, &baddr));
        const int g = id & 3, cols = id < 4 ? in_l : hidden;
        const __half* src = blob + (id < 4 ? w_off[l] + (size_t)g * hidden * in_l : r_off[l] + (size_t)g * hidden * hidden);
        if (maddr) {
          cudnnDataType_t dt;
          int nd = 0, d[4] = {0, 0, 0, 0}, s[4] = {0, 0, 0, 0};
          checkCUDNN(cudnnGetTensorNdDescriptor(md, 4, &dt, &nd, d, s));
          if (nd != 3 || d[1] != hidden || d[2] != cols) throw std::runtime_error("unexpected cuDNN RNN matrix descriptor");
          __half* dst = reinterpret_cast<__half*>(wspace.data() + (static_cast<unsigned char*>(maddr) - static_cast<unsigned char*>(wdev)));
          for (int r = 0; r < hidden; ++r)
            for (int c = 0; c < cols; ++c) dst[(size_t)r * s[1] + (size_t)c * s[2]] = src[(size_t)r * cols + c];
        }
        if (baddr) {
          const __half* bsrc = blob + (id < 4 ? bw_off[l] : br_off[l]) + (size_t)g * hidden;
          if (id >= 4 && !double_bias) throw std::runtime_error("cuDNN reports a recurrent bias in single-bias mode");
          memcpy(wspace.data() + (static_cast<unsigned char*>(baddr) - static_cast<unsigned char*>(wdev)), bsrc, (size_t)hidden * sizeof(__half));
        }
      }
    }
    checkCUDA(cudaMemcpy(wdev, wspace.data(), wbytes, cudaMemcpyHostToDevice));
    // cuDNN 9 takes the sequence lengths from the data descriptors and rejects a device array here (the
    // reference passes one, LSTMLayerv8.cpp:80, which cuDNN 8 accepted)
    cudnnStatus_t st = cudnnRNNForward(g_cudnn, rnn, CUDNN_FWD_MODE_INFERENCE, lens_dev, xd, x, yd, y, hd, nullptr, hy, cd, nullptr, cy, wbytes,
                                       wdev, work, wsp, 0, nullptr);
    if (st == CUDNN_STATUS_BAD_PARAM)
      st = cudnnRNNForward(g_cudnn, rnn, CUDNN_FWD_MODE_INFERENCE, nullptr, xd, x, yd, y, hd, nullptr, hy, cd, nullptr, cy, wbytes, wdev, work, wsp,
                           0, nullptr);
    checkCUDNN(st);
    checkCUDA(cudaDeviceSynchronize());
    cudaFree(wdev); cudaFree(wsp); cudaFree(lens_dev);
    cudnnDestroyTensorDescriptor(md); cudnnDestroyTensorDescriptor(bd); cudnnDestroyTensorDescriptor(hd); cudnnDestroyTensorDescriptor(cd);
    cudnnDestroyRNNDataDescriptor(xd); cudnnDestroyRNNDataDescriptor(yd); cudnnDestroyRNNDescriptor(rnn);
    return 0;
  }, -1);
}

// Where cuDNN 9 keeps each matrix and bias of an LSTM inside its weight space: out[(l*8 + id)*2 + 0] = element
// offset of the matrix of linear layer `id` of layer l, [..+1] = element offset of its bias (-1: none); returns
// the weight space size in elements (what the reference stores as weightCount_, LSTMLayerv8.cpp:24-25), or -1.
long long ref_cudnn_lstm_weight_offsets(int in_c, int hidden, int layers, int double_bias, long long* out) {
  return guarded([&]() -> long long {
    if (ref_init() != 0) return -1;
    cudnnRNNDescriptor_t rnn;
    checkCUDNN(cudnnCreateRNNDescriptor(&rnn));
    checkCUDNN(cudnnSetRNNDescriptor_v8(rnn, CUDNN_RNN_ALGO_STANDARD, CUDNN_LSTM, double_bias ? CUDNN_RNN_DOUBLE_BIAS : CUDNN_RNN_SINGLE_INP_BIAS,
                                        CUDNN_UNIDIRECTIONAL, CUDNN_LINEAR_INPUT, CUDNN_DATA_HALF, CUDNN_DATA_HALF, CUDNN_TENSOR_OP_MATH,
                                        in_c, hidden, hidden, layers, nullptr, 0));
    size_t wbytes = 0;
    checkCUDNN(cudnnGetRNNWeightSpaceSize(g_cudnn, rnn, &wbytes));
    void* wdev = nullptr;
    checkCUDA(cudaMalloc(&wdev, wbytes));
    cudnnTensorDescriptor_t md, bd;
    checkCUDNN(cudnnCreateTensorDescriptor(&md));
    checkCUDNN(cudnnCreateTensorDescriptor(&bd));
    for (int l = 0; l < layers; ++l)
      for (int id = 0; id < 8; ++id) {
        void *maddr = nullptr, *baddr = nullptr;
        checkCUDNN(cudnnGetRNNWeightParams(g_cudnn, rnn, l, wbytes, wdev, id, md, &maddr, bd, &baddr));
        out[(l * 8 + id) * 2 + 0] = maddr ? (static_cast<unsigned char*>(maddr) - static_cast<unsigned char*>(wdev)) / 2 : -1;
        out[(l * 8 + id) * 2 + 1] = baddr ? (static_cast<unsigned char*>(baddr) - static_cast<unsigned char*>(wdev)) / 2 : -1;
      }
    cudaFree(wdev);
    cudnnDestroyTensorDescriptor(md); cudnnDestroyTensorDescriptor(bd); cudnnDestroyRNNDescriptor(rnn);
    return (long long)(wbytes / 2);
  }, -1);
}

}  // extern "C"
