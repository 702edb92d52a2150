// conv_first_tc.h -- internal interface between the first-layer convolution plan (conv_first.cu)
// and its tensor-core kernel (conv_first_tc.cu).
#pragma once
#include <cuda_fp16.h>

struct aig_ctx;

struct ConvFirstGeom {
  int batch, D, H, W;     // input extents (D = 1 for 2-D)
  int Do, Ho, Wo, K;      // output extents, output channels
  int kd, k, sd, s, pd, pad;
  int act;
  float slope;
};

struct ConvFirstTc;

bool conv_first_tc_supported(const ConvFirstGeom& g);
// scale/shift: device arrays of at least ceil(K/16)*16 floats that outlive the object
int conv_first_tc_create(aig_ctx* ctx, const ConvFirstGeom& g, const float* scale, const float* shift, ConvFirstTc** out);
void conv_first_tc_destroy(ConvFirstTc* t);
int conv_first_tc_set_weights(ConvFirstTc* t, const __half* w_kcx);
int conv_first_tc_forward(ConvFirstTc* t, const void* x, bool bgra, __half* y);
// Output layout switch: [n][Hb][Wb][4][K] blocks of 2x2 pixels (block (y+1)>>1, (x+1)>>1; sub-position ((y+1)&1)*2+((x+1)&1)).
int conv_first_tc_set_s2d(ConvFirstTc* t, int enable, int Hb, int Wb);
