// conv_first.cu -- first-layer convolutions (3 input channels) with the input conversion fused into
// the load: BGRA uint8 -> (R,G,B)/255 as fp16 values (CudaStuff.cu:63-74,150-157) for the 2-D
// encoder, planar fp16 NC(D)HW for the operator-API path and the 3-D temporal encoder.
// K = 3*kd*kh*kw is far too small for a TMA-fed pipeline (75 or 81), so the input patch of one
// output tile is staged in shared memory and each thread produces one output pixel x 32 channels.
// Output is channels-last fp16 with bias + folded BatchNorm + activation applied.
#include "aig_common.cuh"
#include "conv_first_rows.h"
#include "conv_first_tc.h"

namespace {

constexpr int kTH = 8, kTW = 32;  // output tile per block (256 threads)
constexpr int kKC = 32;           // output channels per pass

struct ConvFirstParams {
  int batch, D, H, W;            // input extents (D = 1 for 2-D)
  int Do, Ho, Wo, K;             // output extents / channels
  int kd, kh, kw, sd, sh, sw, pd, ph, pw;
  int PH, PW;                    // patch extents
  int act;
  float slope;
  const float* w;                // [tap][Kpad] fp32, tap = ((c*kd+fd)*kh+fr)*kw+fs
  const float* scale;
  const float* shift;
  int Kpad;
};

template <bool BGRA>
__global__ void __launch_bounds__(kTH* kTW)
conv_first_kernel(const void* __restrict__ xin, __half* __restrict__ y, const ConvFirstParams p) {
  extern __shared__ float smem[];
  const int taps = 3 * p.kd * p.kh * p.kw;
  float* s_w = smem;                                 // [taps][kKC]
  float* s_patch = smem + taps * kKC;                // [3][kd][PH][PW+1]
  __shared__ float s_lut[256];
  const int PWp = p.PW + 1;
  const int tid = threadIdx.x;
  const int n = blockIdx.z / p.Do, od = blockIdx.z % p.Do;
  const int oh0 = blockIdx.y * kTH, ow0 = blockIdx.x * kTW;
  const int ih0 = oh0 * p.sh - p.ph, iw0 = ow0 * p.sw - p.pw, id0 = od * p.sd - p.pd;

  if (BGRA) {
    // same arithmetic as the reference: IEEE fp32 divide, round to fp16, widen again
    if (tid < 256) s_lut[tid] = __half2float(__float2half_rn(__fdiv_rn((float)tid, 255.0f)));
    __syncthreads();
    const uint32_t* src = reinterpret_cast<const uint32_t*>(xin) + (size_t)n * p.H * p.W;
    for (int i = tid; i < p.PH * p.PW; i += blockDim.x) {
      const int r = i / p.PW, c = i - r * p.PW;
      const int ih = ih0 + r, iw = iw0 + c;
      float R = 0.f, G = 0.f, B = 0.f;
      if (ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) {
        const uint32_t px = src[(size_t)ih * p.W + iw];
        B = s_lut[px & 0xFFu];
        G = s_lut[(px >> 8) & 0xFFu];
        R = s_lut[(px >> 16) & 0xFFu];
      }
      s_patch[(0 * p.PH + r) * PWp + c] = R;  // plane order R,G,B
      s_patch[(1 * p.PH + r) * PWp + c] = G;
      s_patch[(2 * p.PH + r) * PWp + c] = B;
    }
  } else {
    const __half* src = reinterpret_cast<const __half*>(xin);
    const int per_c = p.kd * p.PH * p.PW;
    for (int i = tid; i < 3 * per_c; i += blockDim.x) {
      const int c = i / per_c, r0 = i - c * per_c;
      const int fd = r0 / (p.PH * p.PW), r1 = r0 - fd * (p.PH * p.PW);
      const int r = r1 / p.PW, cc = r1 - r * p.PW;
      const int id = id0 + fd, ih = ih0 + r, iw = iw0 + cc;
      float v = 0.f;
      if (id >= 0 && id < p.D && ih >= 0 && ih < p.H && iw >= 0 && iw < p.W)
        v = __half2float(src[((((size_t)n * 3 + c) * p.D + id) * p.H + ih) * p.W + iw]);
      s_patch[((c * p.kd + fd) * p.PH + r) * PWp + cc] = v;
    }
  }

  const int ty = tid / kTW, tx = tid - ty * kTW;
  const int oh = oh0 + ty, ow = ow0 + tx;
  const bool valid = oh < p.Ho && ow < p.Wo;
  const size_t pix = (((size_t)n * p.Do + od) * p.Ho + oh) * p.Wo + ow;

  for (int k0 = 0; k0 < p.K; k0 += kKC) {
    __syncthreads();
    for (int i = tid; i < taps * kKC; i += blockDim.x) {
      const int t = i / kKC, k = i - t * kKC;
      s_w[i] = p.w[(size_t)t * p.Kpad + k0 + k];
    }
    __syncthreads();
    float acc[kKC];
#pragma unroll
    for (int k = 0; k < kKC; ++k) acc[k] = 0.f;
    int t = 0;
    for (int cf = 0; cf < 3 * p.kd; ++cf) {
      for (int fr = 0; fr < p.kh; ++fr) {
        const float* prow = s_patch + (cf * p.PH + ty * p.sh + fr) * PWp + tx * p.sw;
        for (int fs = 0; fs < p.kw; ++fs, ++t) {
          const float xv = prow[fs];
          const float4* wv = reinterpret_cast<const float4*>(s_w + t * kKC);
#pragma unroll
          for (int k4 = 0; k4 < kKC / 4; ++k4) {
            const float4 w4 = wv[k4];
            acc[4 * k4 + 0] = fmaf(xv, w4.x, acc[4 * k4 + 0]);
            acc[4 * k4 + 1] = fmaf(xv, w4.y, acc[4 * k4 + 1]);
            acc[4 * k4 + 2] = fmaf(xv, w4.z, acc[4 * k4 + 2]);
            acc[4 * k4 + 3] = fmaf(xv, w4.w, acc[4 * k4 + 3]);
          }
        }
      }
    }
    if (valid) {
      __half* yo = y + pix * p.K + k0;
      if ((p.K & 7) == 0) {
#pragma unroll
        for (int v8 = 0; v8 < kKC / 8; ++v8) {
          if (k0 + v8 * 8 >= p.K) break;
          uint4 o;
          __half* oh8 = reinterpret_cast<__half*>(&o);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int k = k0 + v8 * 8 + e;
            oh8[e] = __float2half(act_apply(acc[v8 * 8 + e] * p.scale[k] + p.shift[k], p.act, p.slope));
          }
          *reinterpret_cast<uint4*>(yo + v8 * 8) = o;
        }
      } else {
        for (int k = 0; k < kKC && k0 + k < p.K; ++k)
          yo[k] = __float2half(act_apply(acc[k] * p.scale[k0 + k] + p.shift[k0 + k], p.act, p.slope));
      }
    }
  }
}

// w [K][3][taps3] fp16 -> [tap][Kpad] fp32 with tap = c*taps3 + t3; scale/shift fold bias + BN.
__global__ void conv_first_pack_kernel(const __half* __restrict__ w, const __half* __restrict__ bias,
                                       const float* gamma, const float* beta, const float* mean, const float* var,
                                       float eps, float* __restrict__ wp, float* scale, float* shift, int K, int Kpad,
                                       int taps) {
  const int total = taps * Kpad;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int t = i / Kpad, k = i - t * Kpad;
    wp[i] = k < K ? __half2float(w[(size_t)k * taps + t]) : 0.f;
  }
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < Kpad; k += gridDim.x * blockDim.x) {
    float s = 0.f, sh = 0.f;
    if (k < K) {
      const float b = bias ? __half2float(bias[k]) : 0.f;
      if (gamma) {
        s = gamma[k] / sqrtf(var[k] + eps);
        sh = (b - mean[k]) * s + beta[k];
      } else {
        s = 1.f;
        sh = b;
      }
    }
    scale[k] = s;
    shift[k] = sh;
  }
}

}  // namespace

struct aig_conv0_plan {
  aig_ctx* ctx = nullptr;
  ConvFirstParams p{};
  float* w = nullptr;
  float* scale = nullptr;
  float* shift = nullptr;
  bool weights_set = false;
  size_t smem = 0;
  dim3 grid;
  ConvFirstTc* tc = nullptr;  // tensor-core path when the filter geometry has an instantiation
  ConvFirstRows* rows = nullptr;  // row-resident tensor-core path for uint8 frames (5x5, stride 2, 32 channels)
  __half* planar_scratch = nullptr;  // planar uint8 frames converted to fp16, for geometries without the row kernel
};

static int conv0_create(aig_ctx* ctx, int batch, int D, int H, int W, int K, int kd, int k, int sd, int s, int pd, int pad,
                        int act, float slope, aig_conv0_plan** out) {
  if (!ctx || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, batch > 0 && D > 0 && H > 0 && W > 0 && K > 0 && k > 0 && kd > 0 && s > 0 && sd > 0 && pad >= 0 && pd >= 0,
              "conv0 plan: bad arguments");
  AIG_REQUIRE(ctx, H + 2 * pad >= k && W + 2 * pad >= k && D + 2 * pd >= kd, "conv0 plan: filter larger than padded input");
  aig_conv0_plan* pl = new aig_conv0_plan();
  pl->ctx = ctx;
  ConvFirstParams& p = pl->p;
  p.batch = batch; p.D = D; p.H = H; p.W = W; p.K = K;
  p.kd = kd; p.kh = k; p.kw = k; p.sd = sd; p.sh = s; p.sw = s; p.pd = pd; p.ph = pad; p.pw = pad;
  p.Do = (D + 2 * pd - kd) / sd + 1;
  p.Ho = (H + 2 * pad - k) / s + 1;
  p.Wo = (W + 2 * pad - k) / s + 1;
  p.PH = (kTH - 1) * s + k;
  p.PW = (kTW - 1) * s + k;
  p.act = act; p.slope = slope;
  p.Kpad = ceil_div(K, kKC) * kKC;
  const int taps = 3 * kd * k * k;
  pl->smem = ((size_t)taps * kKC + (size_t)3 * kd * p.PH * (p.PW + 1)) * sizeof(float);
  if (pl->smem > 200 * 1024) {
    delete pl;
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "conv0 plan: filter %dx%dx%d stride %d needs %zu bytes of shared memory", kd, k, k, s, pl->smem);
  }
  pl->grid = dim3(ceil_div(p.Wo, kTW), ceil_div(p.Ho, kTH), batch * p.Do);
  if (pl->grid.y > 65535 || pl->grid.z > 65535) {
    delete pl;
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "conv0 plan: grid too large");
  }
  AIG_CUDA_OK(ctx, cudaMalloc(&pl->w, (size_t)taps * p.Kpad * sizeof(float)));
  AIG_CUDA_OK(ctx, cudaMalloc(&pl->scale, p.Kpad * sizeof(float)));
  AIG_CUDA_OK(ctx, cudaMalloc(&pl->shift, p.Kpad * sizeof(float)));
  p.w = pl->w; p.scale = pl->scale; p.shift = pl->shift;
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(conv_first_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(conv_first_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  ConvFirstGeom geo{batch, D, H, W, p.Do, p.Ho, p.Wo, K, kd, k, sd, s, pd, pad, act, slope};
  if (conv_first_tc_supported(geo)) {
    const int rc = conv_first_tc_create(ctx, geo, pl->scale, pl->shift, &pl->tc);
    if (rc != AIG_OK) {
      aig_conv0_plan_destroy(pl);
      return rc;
    }
  }
  if (conv_first_rows_supported(geo)) {
    const int rc = conv_first_rows_create(ctx, geo, pl->scale, pl->shift, &pl->rows);
    if (rc != AIG_OK) {
      aig_conv0_plan_destroy(pl);
      return rc;
    }
  }
  *out = pl;
  return AIG_OK;
}

extern "C" {

int aig_conv0_plan_create(aig_ctx* ctx, int batch, int in_h, int in_w, int out_c, int k, int stride, int pad, int act,
                          float slope, aig_conv0_plan** out) {
  return conv0_create(ctx, batch, 1, in_h, in_w, out_c, 1, k, 1, stride, 0, pad, act, slope, out);
}

int aig_conv0_plan_create_3d(aig_ctx* ctx, int batch, int in_d, int in_h, int in_w, int out_c, int kd, int khw, int sd,
                             int shw, int pd, int phw, int act, float slope, aig_conv0_plan** out) {
  return conv0_create(ctx, batch, in_d, in_h, in_w, out_c, kd, khw, sd, shw, pd, phw, act, slope, out);
}

int aig_conv0_plan_destroy(aig_conv0_plan* pl) {
  if (!pl) return AIG_OK;
  DeviceGuard g(pl->ctx->device);
  cudaStreamSynchronize(pl->ctx->stream);
  conv_first_tc_destroy(pl->tc);
  conv_first_rows_destroy(pl->rows);
  cudaFree(pl->planar_scratch);
  cudaFree(pl->w);
  cudaFree(pl->scale);
  cudaFree(pl->shift);
  delete pl;
  return AIG_OK;
}

int aig_conv0_plan_out_dims(const aig_conv0_plan* pl, int* od, int* oh, int* ow) {
  if (!pl) return AIG_ERR_INVALID;
  if (od) *od = pl->p.Do;
  if (oh) *oh = pl->p.Ho;
  if (ow) *ow = pl->p.Wo;
  return AIG_OK;
}

int aig_conv0_plan_set_weights(aig_conv0_plan* pl, const aig_half* w, const aig_half* bias, const float* bn_gamma,
                               const float* bn_beta, const float* bn_mean, const float* bn_var, float bn_eps) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, w != nullptr, "conv0 set_weights: null weights");
  AIG_REQUIRE(ctx, !bn_gamma || (bn_beta && bn_mean && bn_var), "conv0 set_weights: BatchNorm needs all four arrays");
  const int taps = 3 * pl->p.kd * pl->p.kh * pl->p.kw;
  conv_first_pack_kernel<<<ceil_div(taps * pl->p.Kpad, 256), 256, 0, ctx->stream>>>(
      (const __half*)w, (const __half*)bias, bn_gamma, bn_beta, bn_mean, bn_var, bn_eps, pl->w, pl->scale, pl->shift,
      pl->p.K, pl->p.Kpad, taps);
  AIG_LAUNCH_OK(ctx);
  if (pl->tc) {
    const int rc = conv_first_tc_set_weights(pl->tc, (const __half*)w);
    if (rc != AIG_OK) return rc;
  }
  if (pl->rows) {
    const int rc = conv_first_rows_set_weights(pl->rows, (const __half*)w);
    if (rc != AIG_OK) return rc;
  }
  pl->weights_set = true;
  return AIG_OK;
}

int aig_conv0_plan_set_output_s2d(aig_conv0_plan* pl, int enable) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  AIG_REQUIRE(ctx, !enable || (pl->tc && pl->p.D == 1 && pl->p.kd == 1), "conv0: space-to-depth output needs the 2-D tensor-core path");
  if (!pl->tc) return AIG_OK;
  // block extents of a following k4 s2 p1 / k2 s2 p0 pair: one more block than its output extent
  const int Hb = (pl->p.Ho - 2) / 2 + 2, Wb = (pl->p.Wo - 2) / 2 + 2;
  if (pl->rows) {
    const int rc = conv_first_rows_set_s2d(pl->rows, enable, Hb, Wb);
    if (rc != AIG_OK) return rc;
  }
  return conv_first_tc_set_s2d(pl->tc, enable, Hb, Wb);
}

int aig_conv0_forward_bgra(aig_conv0_plan* pl, const uint8_t* bgra, aig_half* y) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, bgra && y && pl->weights_set, "conv0 forward: null pointer or weights not set");
  AIG_REQUIRE(ctx, pl->p.D == 1 && pl->p.kd == 1, "conv0 forward_bgra: 2-D plans only");
  AIG_REQUIRE(ctx, ((uintptr_t)bgra & 3) == 0 && ((uintptr_t)y & 15) == 0, "conv0 forward: misaligned tensors");
  if (pl->rows && ((uintptr_t)bgra & 15) == 0) return conv_first_rows_forward(pl->rows, bgra, 0, (__half*)y);
  if (pl->tc) return conv_first_tc_forward(pl->tc, bgra, true, (__half*)y);
  conv_first_kernel<true><<<pl->grid, kTH * kTW, pl->smem, ctx->stream>>>(bgra, (__half*)y, pl->p);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_conv0_forward_rgb_planar(aig_conv0_plan* pl, const uint8_t* rgb, aig_half* y) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, rgb && y && pl->weights_set, "conv0 forward: null pointer or weights not set");
  AIG_REQUIRE(ctx, pl->p.D == 1 && pl->p.kd == 1, "conv0 forward_rgb_planar: 2-D plans only");
  AIG_REQUIRE(ctx, ((uintptr_t)y & 15) == 0, "conv0 forward: misaligned output");
  if (pl->rows && ((uintptr_t)rgb & 15) == 0) return conv_first_rows_forward(pl->rows, rgb, 1, (__half*)y);
  // other geometries: ConvertAndNormalize into a planar fp16 copy (CudaStuff.cu:150-157), then the planar path
  const size_t n = (size_t)pl->p.batch * 3 * pl->p.H * pl->p.W;
  if (!pl->planar_scratch) AIG_CUDA_OK(ctx, cudaMalloc(&pl->planar_scratch, n * sizeof(__half)));
  const int rc = aig_convert_normalize(ctx, (aig_half*)pl->planar_scratch, rgb, n);
  if (rc != AIG_OK) return rc;
  return aig_conv0_forward_nchw(pl, (const aig_half*)pl->planar_scratch, y);
}

int aig_conv0_forward_nchw(aig_conv0_plan* pl, const aig_half* x, aig_half* y) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, x && y && pl->weights_set, "conv0 forward: null pointer or weights not set");
  AIG_REQUIRE(ctx, ((uintptr_t)y & 15) == 0, "conv0 forward: misaligned output");
  if (pl->tc) return conv_first_tc_forward(pl->tc, x, false, (__half*)y);
  conv_first_kernel<false><<<pl->grid, kTH * kTW, pl->smem, ctx->stream>>>(x, (__half*)y, pl->p);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

}  // extern "C"
