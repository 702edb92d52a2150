// cudnn_shim.h -- the few cuDNN/cuBLAS names that appear in the reference's layer constructors
// (Layer.h:2,17; BatchNorm.h:7; Activate.h:7; FCLayer.h:8), defined on top of this library so that
// caller code compiles without cuDNN or cuBLAS: both "handles" are the library's context.
#pragma once
#include <cuda_runtime.h>

#include "aig_b200.h"

typedef aig_ctx* cudnnHandle_t;
typedef aig_ctx* cublasHandle_t;

// shape of a layer's output, what ResConvLayer.cpp:35 reads through outDesc_
struct cudnnTensorDescriptor_t {
  int n = 0, c = 0, h = 0, w = 0;
};

enum cudnnBatchNormMode_t { CUDNN_BATCHNORM_PER_ACTIVATION = 0, CUDNN_BATCHNORM_SPATIAL = 1 };
enum cudnnActivationMode_t { CUDNN_ACTIVATION_SIGMOID = 0, CUDNN_ACTIVATION_RELU = 1 };

// Infer.cpp:76-79: cudnnCreate / cublasCreate.  The reference never sets a stream on its handles, so all of
// its library calls, its own launchers (aig_compat.h here) and its cudaMemcpy calls share the legacy default
// stream and run in issue order (Infer.cpp:109-112).  The handle made here is bound to that stream too, so the
// same call sequence keeps that order without explicit synchronisation.
inline int aigCreateLegacyStreamHandle(aig_ctx** h) {
  int dev = 0;
  cudaGetDevice(&dev);
  const int rc = aig_ctx_create(h, dev);
  return rc == AIG_OK ? aig_ctx_set_stream(*h, nullptr) : rc;
}
inline int cudnnCreate(cudnnHandle_t* h) { return aigCreateLegacyStreamHandle(h); }
inline int cublasCreate(cublasHandle_t* h) { return aigCreateLegacyStreamHandle(h); }
inline int cudnnDestroy(cudnnHandle_t h) { return aig_ctx_destroy(h); }
inline int cublasDestroy(cublasHandle_t h) { return aig_ctx_destroy(h); }
