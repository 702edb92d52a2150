// ref_compat.h -- forced include (-include) for compiling the reference's own layer sources, from where they
// lie, with g++ on Linux against cuDNN 9 / cuBLAS 12.  TEST INFRASTRUCTURE ONLY; nothing of the reference is
// copied here.  It supplies what those files got transitively from their Windows build (<mm_malloc.h> for
// _mm_free at common.h:43, <cfloat>, <vector>, <algorithm>) and one overload: ConvLayer3D.cpp:124,
// LSTMLayerv8.cpp:92 and MHALayer.cpp:185 still call SGDHalf with four arguments while common.h:112 declares
// five (the weight decay came later); the overload forwards with a decay of zero, which only the training
// path would ever reach.
#pragma once
#include <mm_malloc.h>

#include <algorithm>
#include <cfloat>
#include <stdexcept>
#include <vector>

#include <cuda_fp16.h>

#include "common.h"

inline void SGDHalf(__half* param, const __half* grads, int size, float learningRate) { SGDHalf(param, grads, size, learningRate, 0.0f); }
