// aig_oracle.cpp -- CPU restatement of the AI-gamer frame->action forward operators.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared against and the
// program timed as the CPU baseline.  Nothing in the product (the CUDA library, the C++ layer
// classes) may call, link or load it.
//
// Every function restates one reference operator; the citation is the reference file:line (paths
// relative to the reference project's "AI gamer/" directory).  fp16 tensors are carried as
// uint16_t bit patterns.  h(x) below means "round to nearest even to IEEE binary16".
//
// Parity status: the reference ships no tests, golden vectors or CPU path.  The element-wise,
// preprocessing, LayerNorm and SpatialAttention kernels are pinned on a GPU box against the
// reference's own CudaStuff.cu compiled from source (oracle/ref_shim.cu).  Everything the reference
// delegates to cuDNN/cuBLAS (convolution, BatchNorm, GEMM, LSTM, multi-head attention) is
// "parity unpinned": the closed libraries' accumulation order, the cuDNN LSTM weight-blob layout
// and the attention weight orientation are fixed here by definition (stated per function).
#include <omp.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>

typedef uint16_t f16;

static inline float h2f(f16 v) {
  _Float16 x;
  std::memcpy(&x, &v, 2);
  return (float)x;
}
static inline f16 f2h(float v) {
  _Float16 x = (_Float16)v;
  f16 r;
  std::memcpy(&r, &x, 2);
  return r;
}
static inline f16 d2h(double v) {
  _Float16 x = (_Float16)v;  // single rounding double -> binary16
  f16 r;
  std::memcpy(&r, &x, 2);
  return r;
}
static inline float hround(float v) { return h2f(f2h(v)); }

extern "C" {

int orc_version() { return 1; }

// Threads the OpenMP loops below use; returns the previous maximum.  The environment variable is read
// once when the OpenMP runtime is loaded, which may be before the caller can set it.
int orc_set_threads(int n) {
  int prev = omp_get_max_threads();
  if (n > 0) omp_set_num_threads(n);
  return prev;
}

// ---------------------------------------------------------------------------------------------
// Preprocessing.  CudaStuff.cu:63-74 (cuARGBtoRGBplanar): pixel bytes are (B,G,R,A); plane 0 = R,
// plane 1 = G, plane 2 = B.
void orc_bgra_to_planar(const uint8_t* src, uint8_t* dst, int n) {
  for (int i = 0; i < n; ++i) {
    dst[i] = src[4 * i + 2];
    dst[i + n] = src[4 * i + 1];
    dst[i + 2 * n] = src[4 * i];
  }
}
// CudaStuff.cu:150-153 (convertAndNormalizeKernel): h(float(u8) / 255.0f), IEEE fp32 divide.
void orc_convert_normalize(f16* out, const uint8_t* in, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = f2h((float)in[i] / 255.0f);
}
// CudaStuff.cu:158-161 (UnConvertAndUnNormalizeKernel): (unsigned char)(float(h) * 255.0f).
void orc_unconvert_unnormalize(uint8_t* out, const f16* in, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = (uint8_t)(h2f(in[i]) * 255.0f);
}
// ConvScale::ScaleInPlace / ScaleToHalf (ConvScale.cpp:41-52): ConvertAndNormalize, a k x k stride-k convolution whose
// filter holds half(1/k^2) everywhere (ConvScale.cpp:17-18), fp16 result, and for ScaleInPlace
// UnConvertAndUnNormalize.  cuDNN's accumulation order is not specified, so the order is fixed here: fp32, one fused
// multiply-add per tap, channel-major, then row-major inside the k x k window.  cross_channel = 1 reproduces the
// reference's filter, which sums the box means of all three channels into every output channel (its filter is
// [3][3][k][k], all equal); 0 keeps the channels apart (a plain box filter).
// src: planar [frames][C][H][W] bytes or, bgra = 1, BGRA pixels [frames][H][W][4] read as planes R, G, B (C = 3).
// out_u8 / out_half: planar [frames][C][H/k][W/k]; either may be null.
void orc_resize_box(const uint8_t* src, uint8_t* out_u8, f16* out_half, int frames, int C, int H, int W, int k, int cross_channel, int bgra) {
  const int Ho = H / k, Wo = W / k;
  const float wk = h2f(f2h(1.0f / (float)(k * k)));
  auto px = [&](int n, int c, int y, int x) -> float {
    const uint8_t b = bgra ? src[(((size_t)n * H + y) * W + x) * 4 + (2 - c)] : src[(((size_t)n * C + c) * H + y) * W + x];
    return h2f(f2h((float)b / 255.0f));
  };
  for (int n = 0; n < frames; ++n)
    for (int c = 0; c < C; ++c)
      for (int oy = 0; oy < Ho; ++oy)
        for (int ox = 0; ox < Wo; ++ox) {
          float acc = 0.f;
          for (int ci = cross_channel ? 0 : c; ci < (cross_channel ? C : c + 1); ++ci)
            for (int dy = 0; dy < k; ++dy)
              for (int dx = 0; dx < k; ++dx) acc = fmaf(px(n, ci, oy * k + dy, ox * k + dx), wk, acc);
          const f16 hv = f2h(acc);
          const size_t o = (((size_t)n * C + c) * Ho + oy) * Wo + ox;
          if (out_half) out_half[o] = hv;
          if (out_u8) out_u8[o] = (uint8_t)(h2f(hv) * 255.0f);
        }
}
// CudaStuff.cu:174-177 / 166-169.
void orc_half_to_float(const f16* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = h2f(src[i]);
}
void orc_float_to_half(const float* src, f16* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = f2h(src[i]);
}

// ---------------------------------------------------------------------------------------------
// Activations (all in place).
// CudaStuff.cu:400-405: if x < 0 (fp16 compare) x = h(x * h(slope)) -- one fp16 product.
void orc_leaky_relu(f16* d, int n, float slope) {
  const float s = hround(slope);
  for (int i = 0; i < n; ++i) {
    float x = h2f(d[i]);
    if (x < 0.0f) d[i] = f2h(x * s);  // exact product of two halves fits fp32 -> single rounding
  }
}
// CudaStuff.cu:416-421: h(x / (1 + exp(-x))) in fp32.
void orc_swish(f16* d, int n) {
  for (int i = 0; i < n; ++i) {
    float x = h2f(d[i]);
    d[i] = f2h(x / (1.0f + expf(-x)));
  }
}
// Activate.cpp:10-21: cudnnActivationForward RELU, NOT_PROPAGATE_NAN: max(x,0), NaN -> 0.
void orc_relu(f16* d, int n) {
  for (int i = 0; i < n; ++i) {
    float x = h2f(d[i]);
    d[i] = (x > 0.0f) ? d[i] : (f16)0;
  }
}
// CudaStuff.cu:437-442 + Sigmoid.cpp:8-12: sigmoid on idx % numCtrls < numButs, others untouched.
void orc_sigmoid_head(f16* d, int numCtrls, int numButs, int size) {
  for (int i = 0; i < size; ++i) {
    if (i % numCtrls >= numButs) continue;
    float x = h2f(d[i]);
    d[i] = f2h(1.0f / (1.0f + expf(-x)));
  }
}
// Extension (not in the reference): tanh on the tail idx % numCtrls >= numButs, for the configs
// that ask for "2 mouse tanh" outputs.
void orc_tanh_tail(f16* d, int numCtrls, int numButs, int size) {
  for (int i = 0; i < size; ++i) {
    if (i % numCtrls < numButs) continue;
    d[i] = f2h(tanhf(h2f(d[i])));
  }
}
// ResConvLayer.cpp:35 (cudnnAddTensor alpha=1,beta=1): m = h(m + r).
void orc_add(f16* m, const f16* r, int n) {
  for (int i = 0; i < n; ++i) m[i] = f2h(h2f(m[i]) + h2f(r[i]));
}

// ---------------------------------------------------------------------------------------------
// Convolution 3-D (2-D is D=kd=1).  ConvLayer.cpp:14-21,74-79 / ConvLayer3D.cpp:16-40,106-111:
// cross-correlation, symmetric zero padding, out = floor((in + 2p - k)/s) + 1;
// t = h(sum) then y = h(float(t) + float(bias)) (cudnnAddTensor is a second fp16 store).
// x [B][C][D][H][W], w [K][C][kd][kh][kw], bias [K], y [B][K][Do][Ho][Wo].
// Accumulation is in double (the library's internal order is not observable).
void orc_conv3d(const f16* x, const f16* w, const f16* bias, f16* y, int B, int C, int D, int H,
                int W, int K, int kd, int khw, int sd, int shw, int pd, int phw) {
  const int Do = (D + 2 * pd - kd) / sd + 1;
  const int Ho = (H + 2 * phw - khw) / shw + 1;
  const int Wo = (W + 2 * phw - khw) / shw + 1;
  std::vector<double> xd((size_t)B * C * D * H * W);
  for (size_t i = 0; i < xd.size(); ++i) xd[i] = h2f(x[i]);
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    for (int k = 0; k < K; ++k) {
      std::vector<double> acc((size_t)Do * Ho * Wo, 0.0);
      for (int c = 0; c < C; ++c) {
        for (int fd = 0; fd < kd; ++fd) {
          for (int fr = 0; fr < khw; ++fr) {
            for (int fs = 0; fs < khw; ++fs) {
              const double wv =
                  h2f(w[((((size_t)k * C + c) * kd + fd) * khw + fr) * khw + fs]);
              for (int od = 0; od < Do; ++od) {
                const int id = od * sd - pd + fd;
                if (id < 0 || id >= D) continue;
                for (int oh = 0; oh < Ho; ++oh) {
                  const int ih = oh * shw - phw + fr;
                  if (ih < 0 || ih >= H) continue;
                  const double* xr = &xd[((((size_t)b * C + c) * D + id) * H + ih) * W];
                  double* ar = &acc[((size_t)od * Ho + oh) * Wo];
                  // valid ow range: 0 <= ow*shw - phw + fs < W
                  int lo = 0;
                  while (lo < Wo && lo * shw - phw + fs < 0) ++lo;
                  int hi = Wo;
                  while (hi > lo && (hi - 1) * shw - phw + fs >= W) --hi;
                  const int off = fs - phw;
                  for (int ow = lo; ow < hi; ++ow) ar[ow] += wv * xr[ow * shw + off];
                }
              }
            }
          }
        }
      }
      const float bv = h2f(bias[k]);
      f16* yo = &y[((size_t)b * K + k) * Do * Ho * Wo];
      for (size_t i = 0; i < acc.size(); ++i) {
        const f16 t = d2h(acc[i]);
        yo[i] = f2h(h2f(t) + bv);
      }
    }
  }
}
void orc_conv2d(const f16* x, const f16* w, const f16* bias, f16* y, int B, int C, int H, int W,
                int K, int k, int stride, int pad) {
  orc_conv3d(x, w, bias, y, B, C, 1, H, W, K, 1, k, 1, stride, 0, pad);
}

// BatchNorm inference.  BatchNorm.cpp:5,55-63 (cudnnBatchNormalizationForwardInference, eps 1e-6):
// y = h(gamma * (x - mean) / sqrt(var + eps) + beta); parameters fp32.
// per_activation == 0: parameter index = channel c (spatial mode); 1: index = c*HW + i.
void orc_batchnorm(const f16* x, f16* y, const float* gamma, const float* beta, const float* mean,
                   const float* var, int B, int C, int HW, double eps, int per_activation) {
  for (int b = 0; b < B; ++b)
    for (int c = 0; c < C; ++c)
      for (int i = 0; i < HW; ++i) {
        const size_t idx = ((size_t)b * C + c) * HW + i;
        const size_t p = per_activation ? (size_t)c * HW + i : (size_t)c;
        const double v =
            (double)gamma[p] * ((double)h2f(x[idx]) - (double)mean[p]) / std::sqrt((double)var[p] + eps) +
            (double)beta[p];
        y[idx] = d2h(v);
      }
}

// Fully connected.  FCLayer.cpp:48-53: cublasGemmEx, weights [inC][outC] row-major, fp32 compute:
// t = h(sum_k x[b][k] * W[k*outC + o]); y = h(float(t) + float(bias[o])).  Double accumulation.
void orc_fc(const f16* x, const f16* W, const f16* bias, f16* y, int B, int inC, int outC) {
  std::vector<double> wd((size_t)inC * outC);
  for (size_t i = 0; i < wd.size(); ++i) wd[i] = h2f(W[i]);
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    std::vector<double> acc(outC, 0.0);
    for (int k = 0; k < inC; ++k) {
      const double xv = h2f(x[(size_t)b * inC + k]);
      const double* wr = &wd[(size_t)k * outC];
      for (int o = 0; o < outC; ++o) acc[o] += xv * wr[o];
    }
    for (int o = 0; o < outC; ++o) {
      const f16 t = d2h(acc[o]);
      y[(size_t)b * outC + o] = bias ? f2h(h2f(t) + h2f(bias[o])) : t;
    }
  }
}

// FCLayer::Backward (FCLayer.cpp:54-59): two cublasGemmEx calls with fp32 compute and fp16 results, and the bias
// gradient.  gw[i][o] = h(sum_b x[b][i] * g[b][o]);  gx[b][i] = h(sum_o g[b][o] * W[i][o]);  gb[o] = h(sum_b g[b][o])
// (the per-channel sum the reference's BiasGradient forms in fp32 before its cross-channel reduction, which is a
// defect and not restated).  Double accumulation for the products, fp32 in batch order for the bias sum.
void orc_fc_backward(const f16* x, const f16* g, const f16* W, f16* gw, f16* gb, f16* gx, int B, int inC, int outC) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < inC; ++i) {
    std::vector<double> acc(outC, 0.0);
    for (int b = 0; b < B; ++b) {
      const double xv = h2f(x[(size_t)b * inC + i]);
      for (int o = 0; o < outC; ++o) acc[o] += xv * (double)h2f(g[(size_t)b * outC + o]);
    }
    for (int o = 0; o < outC; ++o) gw[(size_t)i * outC + o] = d2h(acc[o]);
  }
  for (int o = 0; o < outC; ++o) {
    float s = 0.f;
    for (int b = 0; b < B; ++b) s += h2f(g[(size_t)b * outC + o]);
    gb[o] = f2h(s);
  }
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < inC; ++i) {
      double acc = 0.0;
      for (int o = 0; o < outC; ++o) acc += (double)h2f(g[(size_t)b * outC + o]) * (double)h2f(W[(size_t)i * outC + o]);
      gx[(size_t)b * inC + i] = d2h(acc);
    }
}

// "LayerNorm", reference axis.  CudaStuff.cu:457-515 + LayerNorm.cpp:36-40: statistics per channel
// c over all n < N and i < HW (population variance), written to mean[C], variance[C];
// y = h((x - mean_c) / sqrtf(var_c + eps) * gamma_c + beta_c) in fp32 (eps 1e-7 in the reference).
// The reference launches too few blocks for the statistics kernel (CudaStuff.cu:509 vs :460) and
// merges empty partitions as 0/0 when HW < blockDim (:477-481); neither defect is reproduced:
// every channel gets its statistics.
void orc_layernorm_ref(f16* out, const f16* in, const float* gamma, const float* beta, float* mean,
                       float* variance, int N, int C, int HW, float eps) {
  for (int c = 0; c < C; ++c) {
    double s = 0.0, ss = 0.0;
    const double cnt = (double)N * HW;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) s += h2f(in[((size_t)n * C + c) * HW + i]);
    const double mu = s / cnt;
    for (int n = 0; n < N; ++n)
      for (int i = 0; i < HW; ++i) {
        const double d = h2f(in[((size_t)n * C + c) * HW + i]) - mu;
        ss += d * d;
      }
    mean[c] = (float)mu;
    variance[c] = (float)(ss / cnt);
  }
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int i = 0; i < HW; ++i) {
        const size_t idx = ((size_t)n * C + c) * HW + i;
        const float norm = (h2f(in[idx]) - mean[c]) / sqrtf(variance[c] + eps);
        out[idx] = f2h(norm * gamma[c] + beta[c]);
      }
}
// Extension: row-wise LayerNorm (per sample over C), what a transformer-style LayerNorm means.
// mean/rstd optional outputs [rows].
void orc_layernorm_rows(f16* out, const f16* in, const float* gamma, const float* beta, int rows,
                        int C, float eps) {
  for (int r = 0; r < rows; ++r) {
    double s = 0.0, ss = 0.0;
    for (int c = 0; c < C; ++c) s += h2f(in[(size_t)r * C + c]);
    const double mu = s / C;
    for (int c = 0; c < C; ++c) {
      const double d = h2f(in[(size_t)r * C + c]) - mu;
      ss += d * d;
    }
    const double rstd = 1.0 / std::sqrt(ss / C + (double)eps);
    for (int c = 0; c < C; ++c) {
      const double v = (h2f(in[(size_t)r * C + c]) - mu) * rstd * gamma[c] + beta[c];
      out[(size_t)r * C + c] = d2h(v);
    }
  }
}

// Spatial attention, reference mode.  CudaStuff.cu:673-746 scalar branch (the warp-collective wmma
// branch is taken per thread there, which is undefined; callers must keep its predicate false:
// H < 16 or W < 16 or attC % 16 != 0).  The input buffer is read position-major: X[p][c] =
// in[p*inC + c], p < P = B*H*W.  K/Q/V accumulate with fp16 fused multiply-add (every step rounded
// to fp16).  Softmax max is over the 32-position warp, the sum over the G-position thread block
// (G = launch block size, 64 on the author's GPU).  P must be a multiple of G.
// out[p*attC + a] = h(1*x[p][a % inC] + h(h(a_p) * V[p][a])).
static inline f16 hfma16(f16 a, f16 b, f16 c) {
  // a*b is exact in double (11-bit x 11-bit significands); one rounding to fp16.
  return d2h((double)h2f(a) * (double)h2f(b) + (double)h2f(c));
}
void orc_spatial_attention_ref(const f16* in, const f16* kW, const f16* qW, const f16* vW, f16* kMap,
                               f16* qMap, f16* vMap, f16* scores, f16* out, int B, int inC, int attC,
                               int H, int W, int G) {
  const int P = B * H * W;
  const float scale = 1.0f / sqrtf((float)inC);
  std::vector<float> s(P), e(P);
  for (int p = 0; p < P; ++p) {
    for (int a = 0; a < attC; ++a) {
      f16 ks = 0, qs = 0, vs = 0;
      for (int c = 0; c < inC; ++c) {
        const f16 xv = in[(size_t)p * inC + c];
        ks = hfma16(xv, kW[(size_t)a * inC + c], ks);
        qs = hfma16(xv, qW[(size_t)a * inC + c], qs);
        vs = hfma16(xv, vW[(size_t)a * inC + c], vs);
      }
      kMap[(size_t)p * attC + a] = ks;
      qMap[(size_t)p * attC + a] = qs;
      vMap[(size_t)p * attC + a] = vs;
    }
    float sc = 0.0f;
    for (int a = 0; a < attC; ++a)
      sc += h2f(qMap[(size_t)p * attC + a]) * h2f(kMap[(size_t)p * attC + a]);
    s[p] = sc * scale;
  }
  for (int p0 = 0; p0 < P; p0 += 32) {
    const int p1 = std::min(P, p0 + 32);
    float mx = s[p0];
    for (int p = p0; p < p1; ++p) mx = std::max(mx, s[p]);
    for (int p = p0; p < p1; ++p) e[p] = expf(s[p] - mx);
  }
  for (int g0 = 0; g0 < P; g0 += G) {
    const int g1 = std::min(P, g0 + G);
    // same pairwise tree as the reference's shared-memory reduction (CudaStuff.cu:733-736)
    std::vector<float> t(G, 0.0f);
    for (int p = g0; p < g1; ++p) t[p - g0] = e[p];
    for (int stride = G / 2; stride > 0; stride >>= 1)
      for (int i = 0; i < stride; ++i) t[i] += t[i + stride];
    const float sum = t[0];
    for (int p = g0; p < g1; ++p) {
      const float a_p = sum > 0 ? e[p] / sum : 0.0f;
      scores[p] = f2h(a_p);
      for (int a = 0; a < attC; ++a) {
        const f16 wv = f2h(h2f(scores[p]) * h2f(vMap[(size_t)p * attC + a]));
        out[(size_t)p * attC + a] = f2h(h2f(in[(size_t)p * inC + a % inC]) + h2f(wv));
      }
    }
  }
}
// Extension ("1x1 conv -> sigmoid mask"): m[b,h,w] = sigmoid(sum_c x[b,c,h,w]*w1[c] + b1);
// y = h(x * m).  x, y NCHW; mask kept in fp32.
void orc_spatial_attention_cfg(const f16* x, const f16* w1, float b1, f16* y, int B, int C, int HW) {
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < HW; ++i) {
      double s = b1;
      for (int c = 0; c < C; ++c) s += (double)h2f(x[((size_t)b * C + c) * HW + i]) * h2f(w1[c]);
      const float m = (float)(1.0 / (1.0 + std::exp(-s)));
      for (int c = 0; c < C; ++c) {
        const size_t idx = ((size_t)b * C + c) * HW + i;
        y[idx] = f2h(h2f(x[idx]) * m);
      }
    }
}
// Extension: global average pool over HW (fp32/double mean, fp16 store).  x NCHW -> y [B][C].
void orc_global_avgpool(const f16* x, f16* y, int B, int C, int HW) {
  for (int b = 0; b < B; ++b)
    for (int c = 0; c < C; ++c) {
      double s = 0;
      for (int i = 0; i < HW; ++i) s += h2f(x[((size_t)b * C + c) * HW + i]);
      y[(size_t)b * C + c] = d2h(s / HW);
    }
}
// Extension: adaptive average pool of NCDHW to [B][C][1][ph][pw] (flattened [B][C*ph*pw]); window
// for output cell j along an axis of length L with n cells: [floor(j*L/n), ceil((j+1)*L/n)).
void orc_adaptive_avgpool3d(const f16* x, f16* y, int B, int C, int D, int H, int W, int ph, int pw) {
  for (int b = 0; b < B; ++b)
    for (int c = 0; c < C; ++c)
      for (int oh = 0; oh < ph; ++oh)
        for (int ow = 0; ow < pw; ++ow) {
          const int h0 = (oh * H) / ph, h1 = ((oh + 1) * H + ph - 1) / ph;
          const int w0 = (ow * W) / pw, w1 = ((ow + 1) * W + pw - 1) / pw;
          double s = 0;
          for (int d = 0; d < D; ++d)
            for (int ih = h0; ih < h1; ++ih)
              for (int iw = w0; iw < w1; ++iw)
                s += h2f(x[((((size_t)b * C + c) * D + d) * H + ih) * W + iw]);
          y[(((size_t)b * C + c) * ph + oh) * pw + ow] = d2h(s / ((double)D * (h1 - h0) * (w1 - w0)));
        }
}

// ---------------------------------------------------------------------------------------------
// LSTM.  LSTMLayer.cpp:9-40,75-104 (cudnnRNNForwardInference: LSTM, unidirectional, linear input,
// cell clip +-5, zero initial state) and LSTMLayerv8.cpp:8-39,78-82 (single bias, no clip).
// cuDNN's documented equations: i = s(Wi x + Ri h + bWi + bRi), f, g = tanh(..), o;
// c' = f*c + i*g (clipped), h' = o*tanh(c').
// Definitions fixed here (the library blob layout is not observable from the reference):
//  * gate order i, f, g, o;
//  * blob = for each layer: W_i,W_f,W_g,W_o ([hid][in_l] row-major) then R_i..R_o ([hid][hid]);
//    then for each layer: bW_i..bW_o and (double_bias only) bR_i..bR_o ([hid] each);
//  * h and c are stored as fp16 after every step (the library's hy/cy are fp16 tensors).
// x [T][B][in] (seq-major, the v7 layout); y [T][B][hid] = top-layer h for every step.
// h_state/c_state: optional [layers][B][hid] fp16, read as the initial state when use_state != 0
// and always written with the final state when non-null (carried-state extension).
void orc_lstm(const f16* x, const f16* blob, f16* y, int T, int B, int in, int hid, int layers,
              float clip, int double_bias, f16* h_state, f16* c_state, int use_state) {
  size_t woff = 0;
  std::vector<size_t> Woff(layers), Roff(layers), bWoff(layers), bRoff(layers);
  for (int l = 0; l < layers; ++l) {
    const int inl = l == 0 ? in : hid;
    Woff[l] = woff;
    woff += (size_t)4 * hid * inl;
    Roff[l] = woff;
    woff += (size_t)4 * hid * hid;
  }
  for (int l = 0; l < layers; ++l) {
    bWoff[l] = woff;
    woff += (size_t)4 * hid;
    if (double_bias) {
      bRoff[l] = woff;
      woff += (size_t)4 * hid;
    }
  }
  std::vector<f16> cur((size_t)T * B * std::max(in, hid)), nxt((size_t)T * B * hid);
  std::memcpy(cur.data(), x, (size_t)T * B * in * sizeof(f16));
  for (int l = 0; l < layers; ++l) {
    const int inl = l == 0 ? in : hid;
    std::vector<double> Wd((size_t)4 * hid * inl), Rd((size_t)4 * hid * hid), bd((size_t)4 * hid);
    for (size_t i = 0; i < Wd.size(); ++i) Wd[i] = h2f(blob[Woff[l] + i]);
    for (size_t i = 0; i < Rd.size(); ++i) Rd[i] = h2f(blob[Roff[l] + i]);
    for (int i = 0; i < 4 * hid; ++i)
      bd[i] = (double)h2f(blob[bWoff[l] + i]) + (double_bias ? (double)h2f(blob[bRoff[l] + i]) : 0.0);
    std::vector<f16> hs((size_t)B * hid, 0), cs((size_t)B * hid, 0);
    if (use_state && h_state && c_state) {
      std::memcpy(hs.data(), h_state + (size_t)l * B * hid, (size_t)B * hid * 2);
      std::memcpy(cs.data(), c_state + (size_t)l * B * hid, (size_t)B * hid * 2);
    }
    for (int t = 0; t < T; ++t) {
      std::vector<f16> hn((size_t)B * hid);
#pragma omp parallel for schedule(static)
      for (int b = 0; b < B; ++b) {
        const f16* xt = &cur[((size_t)t * B + b) * inl];
        std::vector<double> xd(inl), hd(hid);
        for (int k = 0; k < inl; ++k) xd[k] = h2f(xt[k]);
        for (int k = 0; k < hid; ++k) hd[k] = h2f(hs[(size_t)b * hid + k]);
        for (int j = 0; j < hid; ++j) {
          double g4[4];
          for (int g = 0; g < 4; ++g) {
            double a = bd[(size_t)g * hid + j];
            const double* wr = &Wd[((size_t)g * hid + j) * inl];
            for (int k = 0; k < inl; ++k) a += wr[k] * xd[k];
            const double* rr = &Rd[((size_t)g * hid + j) * hid];
            for (int k = 0; k < hid; ++k) a += rr[k] * hd[k];
            g4[g] = a;
          }
          const double ig = 1.0 / (1.0 + std::exp(-g4[0]));
          const double fg = 1.0 / (1.0 + std::exp(-g4[1]));
          const double gg = std::tanh(g4[2]);
          const double og = 1.0 / (1.0 + std::exp(-g4[3]));
          double c = fg * (double)h2f(cs[(size_t)b * hid + j]) + ig * gg;
          if (clip > 0) c = std::min((double)clip, std::max(-(double)clip, c));
          const f16 ch = d2h(c);
          cs[(size_t)b * hid + j] = ch;
          hn[(size_t)b * hid + j] = d2h(og * std::tanh((double)h2f(ch)));
        }
      }
      hs = hn;
      std::memcpy(&nxt[(size_t)t * B * hid], hs.data(), (size_t)B * hid * 2);
    }
    if (h_state && c_state) {
      std::memcpy(h_state + (size_t)l * B * hid, hs.data(), (size_t)B * hid * 2);
      std::memcpy(c_state + (size_t)l * B * hid, cs.data(), (size_t)B * hid * 2);
    }
    std::memcpy(cur.data(), nxt.data(), (size_t)T * B * hid * 2);
  }
  std::memcpy(y, cur.data(), (size_t)T * B * hid * 2);
}

// ---------------------------------------------------------------------------------------------
// Multi-head self-attention as the layer's fields define it.  MHALayer.cpp:8,19-32,42-45,84-88:
// four E x E fp16 matrices wq,wk,wv,wo, H heads of d = E/H, scale 1/sqrt(d), causal window
// [0, i+1), no biases, no residual.  Definitions fixed here: matrices are [in][out] row-major like
// FCLayer; head h uses output columns h*d .. h*d+d-1; projections and the per-head context are
// stored as fp16; softmax in fp32-or-better.
// Extensions (not in the reference): rotary embedding on Q and K when rope_base > 0, NeoX
// half-split pairs (j, j + d/2), angle = pos * rope_base^(-2j/d), pos = pos0 + t (absolute frame
// index), q' = h(q_j cos - q_{j+d/2} sin), q'_{j+d/2} = h(q_{j+d/2} cos + q_j sin) in fp32;
// sliding causal window: step t attends to steps max(0, t-window+1) .. t (window <= 0: unbounded),
// which is what a ring KV cache of `window` slots holds.
// x [B][T][E] -> y [B][T][E].
static void rope_rotate(std::vector<f16>& v, int T, int E, int Hh, float base, int pos0) {
  const int d = E / Hh;
  for (int t = 0; t < T; ++t)
    for (int hh = 0; hh < Hh; ++hh)
      for (int j = 0; j < d / 2; ++j) {
        const float inv = powf(base, -2.0f * (float)j / (float)d);
        const float ang = (float)(pos0 + t) * inv;
        const float cs = cosf(ang), sn = sinf(ang);
        f16& a = v[(size_t)t * E + hh * d + j];
        f16& b = v[(size_t)t * E + hh * d + j + d / 2];
        const float fa = h2f(a), fb = h2f(b);
        a = f2h(fa * cs - fb * sn);
        b = f2h(fb * cs + fa * sn);
      }
}
void orc_mha(const f16* x, const f16* wq, const f16* wk, const f16* wv, const f16* wo, f16* y, int B,
             int T, int E, int Hh, float rope_base, int pos0, int window) {
  const int d = E / Hh;
  const double scale = 1.0 / std::sqrt((double)d);
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    std::vector<f16> q((size_t)T * E), k((size_t)T * E), v((size_t)T * E), ctx((size_t)T * E);
    orc_fc(x + (size_t)b * T * E, wq, nullptr, q.data(), T, E, E);
    orc_fc(x + (size_t)b * T * E, wk, nullptr, k.data(), T, E, E);
    orc_fc(x + (size_t)b * T * E, wv, nullptr, v.data(), T, E, E);
    if (rope_base > 0) {
      rope_rotate(q, T, E, Hh, rope_base, pos0);
      rope_rotate(k, T, E, Hh, rope_base, pos0);
    }
    std::vector<double> p(T);
    for (int hh = 0; hh < Hh; ++hh)
      for (int t = 0; t < T; ++t) {
        const int j0 = window > 0 ? std::max(0, t - window + 1) : 0;
        double mx = -1e300;
        for (int j = j0; j <= t; ++j) {
          double s = 0;
          for (int c = 0; c < d; ++c)
            s += (double)h2f(q[(size_t)t * E + hh * d + c]) * h2f(k[(size_t)j * E + hh * d + c]);
          p[j] = s * scale;
          mx = std::max(mx, p[j]);
        }
        double sum = 0;
        for (int j = j0; j <= t; ++j) {
          p[j] = std::exp(p[j] - mx);
          sum += p[j];
        }
        for (int c = 0; c < d; ++c) {
          double o = 0;
          for (int j = j0; j <= t; ++j) o += p[j] * h2f(v[(size_t)j * E + hh * d + c]);
          ctx[(size_t)t * E + hh * d + c] = d2h(o / sum);
        }
      }
    orc_fc(ctx.data(), wo, nullptr, y + (size_t)b * T * E, T, E, E);
  }
}

// ---------------------------------------------------------------------------------------------
// Output decisions.  Infer.cpp:8-57: keys 0..10 and mouse buttons 11..13 pressed iff p > 0.5;
// dx = (int)(p[14] * 256.0f), dy = (int)(p[15] * 256.0f) (C truncation toward zero).
// actions[0..13] = 0/1, actions[14] = dx, actions[15] = dy.  n_buttons/n_ctrls generalise 14/16.
void orc_actions(const float* p, int* actions, int frames, int n_ctrls, int n_buttons) {
  for (int f = 0; f < frames; ++f)
    for (int i = 0; i < n_ctrls; ++i) {
      const float v = p[(size_t)f * n_ctrls + i];
      actions[(size_t)f * n_ctrls + i] = i < n_buttons ? (v > 0.5f ? 1 : 0) : (int)(v * 256.0f);
    }
}

}  // extern "C"
