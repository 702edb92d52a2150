// conv3d_encoder.cpp -- host side of the temporal (3-D convolution) clip encoder: a chain of
// ConvLayer3D -> BatchNorm -> LeakyReLU layers (ConvLayer3D.cpp:106-111, BatchNorm.cpp:55-63,
// LeakyReLU.cpp:9-13), an adaptive average pool to 2x2 cells (mean over depth), an FC head and the
// sigmoid/tanh outputs, composed from the kernel C ABI like NN::Forward chains layers (NN.cpp:93-100).
//
// Parameter blob (little endian, no padding), in layer order:
//   per conv layer: half w[K][C][kd][k][k], half b[K]  (ConvLayer3D.cpp:128-139), then BatchNorm's six
//   float[K] arrays (BatchNorm.cpp:90-117);  FC: half W[in][out], half b[out]  (FCLayer.cpp:70-81)
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "aig_b200.h"
#include "aig_host.h"

struct aig_c3d {
  aig_ctx* ctx = nullptr;
  aig_c3d_config cfg{};
  std::string err;
  aig_conv0_plan* first = nullptr;
  std::vector<aig_conv_plan*> convs;
  aig_conv_plan* fc = nullptr;
  std::vector<aig_half*> acts;
  std::vector<int> d, h, w;
  aig_half *feat = nullptr, *logits = nullptr;
  aig_half *fcw = nullptr, *fcb = nullptr;   // FC parameters as loaded ([in][out], [out])
  float* out_f32 = nullptr;
  uint8_t* params = nullptr;
  bool loaded = false;
};

namespace {
int cfail(aig_c3d* m, int code, const std::string& msg) {
  m->err = msg;
  return code;
}
#define C3D_OK(m, expr)                                                                              \
  do {                                                                                               \
    int rc__ = (expr);                                                                               \
    if (rc__ != AIG_OK) return cfail((m), rc__, std::string(#expr ": ") + aig_last_error((m)->ctx)); \
  } while (0)
size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
}  // namespace

extern "C" {

size_t aig_c3d_param_bytes(const aig_c3d_config* c) {
  if (!c) return 0;
  size_t n = 0;
  for (int i = 0; i < c->n_layers; ++i)
    n += ((size_t)c->widths[i + 1] * c->widths[i] * 27 + c->widths[i + 1]) * 2 + (size_t)c->widths[i + 1] * 24;
  const size_t feat = (size_t)c->widths[c->n_layers] * 4;
  return n + (feat * c->n_out + c->n_out) * 2;
}

int aig_c3d_create(aig_ctx* ctx, const aig_c3d_config* cfg, aig_c3d** out) {
  if (!ctx || !cfg || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  if (cfg->batch <= 0 || cfg->n_layers <= 0 || cfg->n_layers > AIG_C3D_MAX_LAYERS || cfg->widths[0] != 3 || cfg->n_out <= 0) return AIG_ERR_INVALID;
  aig_c3d* m = new aig_c3d();
  m->ctx = ctx;
  m->cfg = *cfg;
  const aig_c3d_config& c = m->cfg;
  int D = c.depth, H = c.height, W = c.width;
  int rc = aig_conv0_plan_create_3d(ctx, c.batch, D, H, W, c.widths[1], 3, 3, 1, 2, 1, 1, AIG_ACT_LEAKY, c.slope, &m->first);
  if (rc == AIG_OK) aig_conv0_plan_out_dims(m->first, &D, &H, &W);
  for (int i = 0; i < c.n_layers && rc == AIG_OK; ++i) {
    if (i > 0) {
      aig_conv_desc d{};
      d.batch = c.batch; d.in_c = c.widths[i]; d.in_d = D; d.in_h = H; d.in_w = W; d.out_c = c.widths[i + 1];
      d.kd = d.kh = d.kw = 3; d.sd = 1; d.sh = d.sw = 2; d.pd = d.ph = d.pw = 1;
      d.act = AIG_ACT_LEAKY; d.slope = c.slope; d.two_step = 0;
      aig_conv_plan* p = nullptr;
      rc = aig_conv_plan_create(ctx, &d, &p);
      if (rc != AIG_OK) break;
      m->convs.push_back(p);
      aig_conv_plan_out_dims(p, &D, &H, &W);
    }
    aig_half* buf = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&buf), (size_t)c.batch * D * H * W * c.widths[i + 1] * 2) != cudaSuccess) rc = AIG_ERR_CUDA;
    m->acts.push_back(buf);
    m->d.push_back(D); m->h.push_back(H); m->w.push_back(W);
  }
  const int feat = c.widths[c.n_layers] * 4;
  if (rc == AIG_OK) rc = aig_fc_plan_create(ctx, c.batch, feat, c.n_out, AIG_ACT_NONE, 0.f, 1, &m->fc);
  if (rc == AIG_OK && (cudaMalloc(reinterpret_cast<void**>(&m->feat), (size_t)c.batch * feat * 2) != cudaSuccess ||
                       cudaMalloc(reinterpret_cast<void**>(&m->logits), (size_t)c.batch * c.n_out * 2) != cudaSuccess ||
                       cudaMalloc(reinterpret_cast<void**>(&m->out_f32), (size_t)c.batch * c.n_out * 4) != cudaSuccess ||
                       cudaMalloc(reinterpret_cast<void**>(&m->params), aig_c3d_param_bytes(&c) + 256 * (8 * (size_t)c.n_layers + 4)) != cudaSuccess))
    rc = AIG_ERR_CUDA;
  if (rc != AIG_OK) {
    aig_c3d_destroy(m);
    return rc;
  }
  *out = m;
  return AIG_OK;
}

int aig_c3d_destroy(aig_c3d* m) {
  if (!m) return AIG_OK;
  if (m->ctx) aig_ctx_sync(m->ctx);
  aig_conv0_plan_destroy(m->first);
  for (aig_conv_plan* p : m->convs) aig_conv_plan_destroy(p);
  aig_conv_plan_destroy(m->fc);
  for (aig_half* a : m->acts) cudaFree(a);
  cudaFree(m->feat); cudaFree(m->logits); cudaFree(m->out_f32); cudaFree(m->params);
  delete m;
  return AIG_OK;
}

const char* aig_c3d_last_error(aig_c3d* m) { return m ? m->err.c_str() : "null model"; }

int aig_c3d_load_memory(aig_c3d* m, const void* blob, size_t bytes) {
  if (!m || !blob) return AIG_ERR_INVALID;
  const aig_c3d_config& c = m->cfg;
  if (bytes != aig_c3d_param_bytes(&c)) return cfail(m, AIG_ERR_IO, "parameter blob size does not match the configuration");
  const uint8_t* src = (const uint8_t*)blob;
  size_t so = 0, dof = 0;
  auto take = [&](size_t n) -> void* {
    void* dst = m->params + dof;
    if (aig_memcpy(m->ctx, dst, src + so, n) != AIG_OK) return nullptr;
    so += n;
    dof = up256(dof + n);
    return dst;
  };
  for (int i = 0; i < c.n_layers; ++i) {
    const size_t K = c.widths[i + 1], C = c.widths[i];
    aig_half* w = (aig_half*)take(K * C * 27 * 2);
    aig_half* b = (aig_half*)take(K * 2);
    float* bn[6];
    for (int j = 0; j < 6; ++j) bn[j] = (float*)take(K * 4);
    if (!w || !b || !bn[5]) return cfail(m, AIG_ERR_CUDA, aig_last_error(m->ctx));
    if (i == 0) C3D_OK(m, aig_conv0_plan_set_weights(m->first, w, b, bn[0], bn[1], bn[2], bn[3], 1e-6f));
    else C3D_OK(m, aig_conv_plan_set_weights(m->convs[i - 1], w, b, bn[0], bn[1], bn[2], bn[3], 1e-6f));
  }
  const size_t feat = (size_t)c.widths[c.n_layers] * 4;
  aig_half* fw = (aig_half*)take(feat * c.n_out * 2);
  aig_half* fb = (aig_half*)take((size_t)c.n_out * 2);
  if (!fw || !fb) return cfail(m, AIG_ERR_CUDA, aig_last_error(m->ctx));
  C3D_OK(m, aig_fc_plan_set_weights(m->fc, fw, fb, nullptr, nullptr, nullptr, nullptr, 0.f));
  m->fcw = fw;
  m->fcb = fb;
  C3D_OK(m, aig_ctx_sync(m->ctx));
  m->loaded = true;
  return AIG_OK;
}

// clips: planar fp16 [batch][3][depth][height][width] on the device
int aig_c3d_forward(aig_c3d* m, const aig_half* clips) {
  if (!m || !clips) return AIG_ERR_INVALID;
  if (!m->loaded) return cfail(m, AIG_ERR_INVALID, "parameters not loaded");
  const aig_c3d_config& c = m->cfg;
  C3D_OK(m, aig_conv0_forward_nchw(m->first, clips, m->acts[0]));
  for (size_t i = 0; i < m->convs.size(); ++i) C3D_OK(m, aig_conv_forward(m->convs[i], m->acts[i], nullptr, m->acts[i + 1]));
  const int L = c.n_layers - 1;
  C3D_OK(m, aig_adaptive_avgpool3d_ndhwc(m->ctx, m->acts[L], m->feat, c.batch, m->d[L], m->h[L], m->w[L], c.widths[c.n_layers], 2, 2));
  if (c.batch <= 64) {
    // FC, sigmoid / tanh and the half -> float conversion in one launch (a block per clip)
    C3D_OK(m, aig_fc_head_forward(m->ctx, m->feat, m->fcw, m->fcb, m->logits, m->out_f32, c.batch, c.widths[c.n_layers] * 4, c.n_out, c.n_sigmoid));
    return AIG_OK;
  }
  C3D_OK(m, aig_conv_forward(m->fc, m->feat, nullptr, m->logits));
  C3D_OK(m, aig_sigmoid_forward(m->ctx, m->logits, c.n_out, c.n_sigmoid, c.batch * c.n_out));
  if (c.n_sigmoid < c.n_out) C3D_OK(m, aig_tanh_tail_forward(m->ctx, m->logits, c.n_out, c.n_sigmoid, c.batch * c.n_out));
  C3D_OK(m, aig_half_to_float(m->ctx, m->logits, m->out_f32, (size_t)c.batch * c.n_out));
  return AIG_OK;
}

const float* aig_c3d_outputs_f32(aig_c3d* m) { return m ? m->out_f32 : nullptr; }
const aig_half* aig_c3d_features(aig_c3d* m) { return m ? m->feat : nullptr; }

}  // extern "C"
