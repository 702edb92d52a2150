// conv_first_rows.h -- internal interface between the first-layer convolution plan (conv_first.cu) and the
// row-resident tensor-core kernel for uint8 frames (conv_first_rows.cu): 3 -> 32 channels, 5x5, stride 2, pad 2.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "conv_first_tc.h"

struct ConvFirstRows;

bool conv_first_rows_supported(const ConvFirstGeom& g);
// scale/shift: device arrays of 32 floats that outlive the object (read back by set_weights)
int conv_first_rows_create(aig_ctx* ctx, const ConvFirstGeom& g, const float* scale, const float* shift, ConvFirstRows** out);
void conv_first_rows_destroy(ConvFirstRows* t);
int conv_first_rows_set_weights(ConvFirstRows* t, const __half* w_kcrs);
int conv_first_rows_set_s2d(ConvFirstRows* t, int enable, int Hb, int Wb);
// frames: BGRA pixels [B][H][W][4] or, planar_rgb != 0, uint8 planes [B][3][H][W]; both 16-byte aligned
int conv_first_rows_forward(ConvFirstRows* t, const uint8_t* frames, int planar_rgb, __half* y);
