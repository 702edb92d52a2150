// cnn_encoder.cpp -- host side of the 2-D frame encoder: the layer chain NN::NN builds
// (NN.cpp:33-61: Conv -> BatchNorm -> activation -> ResConv blocks -> heads) composed from the
// kernel C ABI, with checkpoint loading in the reference's byte layout (NN.cpp:13-20,67-75 and the
// per-layer LoadParameters order), and the Infer::Inference frame step (Infer.cpp:96-114:
// preprocess -> Forward -> half->float -> device-to-host copy) as one CUDA graph.
//
// Network (the 2-D encoder configuration): BGRA frame -> Conv 3->w0 k x k s2 +BN+act ->
// ResConv blocks (ResConvLayer.cpp:13-21 geometry: main k4 s2 p1 +BN+act, k3 s1 p1 +BN; shortcut
// k2 s2 p0; add; act) -> spatial mask attention -> global average pool -> FC -> sigmoid on the
// first n_sigmoid outputs, tanh on the rest.
//
// Checkpoint layout consumed here (little endian, no padding), following the reference's order:
//   int32 width, int32 height
//   Conv0: half w[K][3][k][k], half b[K];  BatchNorm: float scale[K], bias[K], runningMean[K],
//   runningVar[K], savedMean[K], savedInvVar[K]            (BatchNorm.cpp:90-117)
//   per ResConv block: Conv0, BN0, Conv1, BN1, shortcut conv (ResConvLayer.cpp:55-66)
//   mask attention: half w1[C], float b1                    (not a reference layer)
//   FC: half W[in][out], half b[out]                        (FCLayer.cpp:70-81)
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <fstream>
#include <string>
#include <vector>

#include "aig_b200.h"
#include "aig_host.h"

namespace {

struct Arena {
  uint8_t* base = nullptr;
  size_t cap = 0, used = 0;
  void* take(size_t bytes) {
    const size_t off = (used + 255) & ~(size_t)255;
    if (off + bytes > cap) return nullptr;
    used = off + bytes;
    return base + off;
  }
};

struct ConvP {
  aig_half* w = nullptr;
  aig_half* b = nullptr;
  size_t nw = 0, nb = 0;
};
struct BnP {
  float* a[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int c = 0;
};

}  // namespace

struct aig_cnn {
  aig_ctx* ctx = nullptr;
  aig_cnn_config cfg{};
  std::string err;
  int H0 = 0, W0 = 0;                 // conv0 output extents
  std::vector<int> bh, bw;            // per-block output extents
  aig_conv0_plan* conv0 = nullptr;
  struct Block {
    aig_conv_plan *c0 = nullptr, *c1 = nullptr, *sc = nullptr;
    aig_conv_plan* down = nullptr;  // main k4 s2 + shortcut k2 s2 as one launch over the space-to-depth input (replaces c0 and sc)
    aig_half *t = nullptr, *r = nullptr, *y = nullptr;
    bool y_s2d = false;             // y is written in the space-to-depth layout the next block's fused launch reads
  };
  bool act0_s2d = false;
  aig_half* stage_scratch = nullptr;  // channels-last copy of a space-to-depth stage, made on request
  size_t stage_scratch_elems = 0;
  std::vector<Block> blocks;
  aig_conv_plan* fc = nullptr;
  aig_half *act0 = nullptr, *sa = nullptr, *feat = nullptr, *logits = nullptr;
  float* out_f32 = nullptr;
  uint8_t* frames_dev = nullptr;      // staging for the host-buffer entry point
  Arena params;
  aig_half* sa_w = nullptr;
  aig_half *fcw = nullptr, *fcb = nullptr;  // head FC parameters as loaded ([in][out], [out])
  bool fused_head = false;
  float sa_b = 0.f;
  bool loaded = false;
  static constexpr int kGraphs = 8;    // captured forwards, keyed by input pointer
  aig_graph* graphs[kGraphs] = {};
  const uint8_t* graph_ins[kGraphs] = {};
  bool graph_planar[kGraphs] = {};
  int graph_next = 0;
  // pipelined host-buffer steps: private copy stream, two frame slots
  cudaStream_t copy_stream = nullptr;
  uint8_t* frames_slot[2] = {nullptr, nullptr};
  cudaEvent_t ev_h2d[2] = {nullptr, nullptr}, ev_used[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr};
  bool slot_used[2] = {false, false};
  int launches_per_forward = 0;
  // optional per-launch timing (eager forward only): one CUDA event between consecutive launches
  struct Site {
    std::string name;
    double flops;   // algorithmic 2*MAC of the launch (0 for the element-wise sites)
    double bytes;   // algorithmic bytes read + written by the launch
  };
  std::vector<Site> sites;
  std::vector<cudaEvent_t> prof_ev;
  int prof_cap = 0, prof_steps = 0;
  bool prof_on = false;
};

namespace {

int fail(aig_cnn* m, int code, const std::string& msg) {
  m->err = msg;
  return code;
}

#define CNN_OK(m, expr)                                                        \
  do {                                                                         \
    int rc__ = (expr);                                                         \
    if (rc__ != AIG_OK) return fail((m), rc__, std::string(#expr ": ") + aig_last_error((m)->ctx)); \
  } while (0)
#define CNN_CUDA(m, expr)                                                      \
  do {                                                                         \
    cudaError_t e__ = (expr);                                                  \
    if (e__ != cudaSuccess) return fail((m), AIG_ERR_CUDA, std::string(#expr ": ") + cudaGetErrorString(e__)); \
  } while (0)

template <class T>
int dev_alloc(aig_cnn* m, T** p, size_t count) {
  CNN_CUDA(m, cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)));
  CNN_CUDA(m, cudaMemset(*p, 0, count * sizeof(T)));
  return AIG_OK;
}

struct Reader {
  const uint8_t* p;
  size_t left;
  bool take(void* dst_dev, size_t bytes, cudaStream_t s) {
    if (bytes > left) return false;
    if (cudaMemcpyAsync(dst_dev, p, bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) return false;
    p += bytes;
    left -= bytes;
    return true;
  }
  bool take_host(void* dst, size_t bytes) {
    if (bytes > left) return false;
    memcpy(dst, p, bytes);
    p += bytes;
    left -= bytes;
    return true;
  }
};

bool read_conv(aig_cnn* m, Reader& rd, ConvP& c, size_t nw, size_t nb, cudaStream_t s) {
  c.nw = nw;
  c.nb = nb;
  c.w = (aig_half*)m->params.take(nw * 2);
  c.b = (aig_half*)m->params.take(nb * 2);
  return c.w && c.b && rd.take(c.w, nw * 2, s) && rd.take(c.b, nb * 2, s);
}
bool read_bn(aig_cnn* m, Reader& rd, BnP& b, int c, cudaStream_t s) {
  b.c = c;
  for (int i = 0; i < 6; ++i) {
    b.a[i] = (float*)m->params.take((size_t)c * 4);
    if (!b.a[i] || !rd.take(b.a[i], (size_t)c * 4, s)) return false;
  }
  return true;
}

}  // namespace

extern "C" {

size_t aig_cnn_checkpoint_bytes(const aig_cnn_config* c) {
  if (!c) return 0;
  size_t n = 8;
  auto conv = [](int k, int cin, int kk) { return ((size_t)k * cin * kk * kk + k) * 2; };
  auto bn = [](int k) { return (size_t)k * 4 * 6; };
  n += conv(c->widths[0], 3, c->k0) + bn(c->widths[0]);
  for (int i = 0; i < c->n_blocks; ++i) {
    const int ci = c->widths[i], co = c->widths[i + 1];
    n += conv(co, ci, 4) + bn(co) + conv(co, co, 3) + bn(co) + conv(co, ci, 2);
  }
  const int cl = c->widths[c->n_blocks];
  n += (size_t)cl * 2 + 4;
  n += ((size_t)cl * c->n_out + c->n_out) * 2;
  return n;
}

int aig_cnn_create(aig_ctx* ctx, const aig_cnn_config* cfg, aig_cnn** out) {
  if (!ctx || !cfg || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  if (cfg->batch <= 0 || cfg->height <= 0 || cfg->width <= 0 || cfg->n_blocks < 0 || cfg->n_blocks > AIG_CNN_MAX_BLOCKS ||
      cfg->n_out <= 0 || cfg->n_sigmoid < 0 || cfg->n_sigmoid > cfg->n_out || cfg->k0 <= 0)
    return AIG_ERR_INVALID;
  aig_cnn* m = new aig_cnn();
  m->ctx = ctx;
  m->cfg = *cfg;
  const aig_cnn_config& c = m->cfg;
  int rc = AIG_OK;
  auto bail = [&](int code) {
    // keep the object so the caller can read the error text, then destroy
    aig_cnn_destroy(m);
    return code;
  };
  rc = aig_conv0_plan_create(ctx, c.batch, c.height, c.width, c.widths[0], c.k0, 2, c.k0 / 2, c.act, c.slope, &m->conv0);
  if (rc != AIG_OK) return bail(rc);
  aig_conv0_plan_out_dims(m->conv0, nullptr, &m->H0, &m->W0);
  int h = m->H0, w = m->W0;
  m->launches_per_forward = 1;
  {
    const double px = (double)c.batch * m->H0 * m->W0;
    m->sites.push_back({"conv0_bgra", 2.0 * px * c.widths[0] * 3 * c.k0 * c.k0,
                        (double)c.batch * c.height * c.width * 4 + px * c.widths[0] * 2});
  }
  const char* no_fused = getenv("AIG_CNN_NO_FUSED_DOWN");
  const bool allow_fused = !(no_fused && atoi(no_fused));
  for (int i = 0; i < c.n_blocks; ++i) {
    aig_cnn::Block b;
    const int ci = c.widths[i], co = c.widths[i + 1];
    aig_conv_desc d{};
    d.batch = c.batch; d.in_c = ci; d.in_d = 1; d.in_h = h; d.in_w = w; d.out_c = co;
    d.kd = 1; d.kh = d.kw = 4; d.sd = 1; d.sh = d.sw = 2; d.pd = 0; d.ph = d.pw = 1;
    d.act = c.act; d.slope = c.slope; d.two_step = 0;
    int oh = 0, ow = 0;
    // fused down-sampling launch when the plan fits and the producer of this block's input can write
    // the space-to-depth layout it reads; otherwise the two separate stride-2 convolutions
    if (allow_fused && h >= 2 && w >= 2 && aig_resdown_plan_create(ctx, c.batch, ci, h, w, co, c.act, c.slope, &b.down) == AIG_OK) {
      const int prc = i == 0 ? aig_conv0_plan_set_output_s2d(m->conv0, 1) : aig_conv_plan_set_output_s2d(m->blocks[i - 1].c1, 1);
      if (prc != AIG_OK) {
        aig_conv_plan_destroy(b.down);
        b.down = nullptr;
      } else if (i == 0) {
        m->act0_s2d = true;
      } else {
        m->blocks[i - 1].y_s2d = true;
      }
    }
    if (b.down) {
      aig_conv_plan_out_dims(b.down, nullptr, &oh, &ow);
    } else {
      if ((rc = aig_conv_plan_create(ctx, &d, &b.c0)) != AIG_OK) return bail(rc);
      aig_conv_plan_out_dims(b.c0, nullptr, &oh, &ow);
      aig_conv_desc s = d;
      s.kh = s.kw = 2; s.ph = s.pw = 0; s.act = AIG_ACT_NONE;
      if ((rc = aig_conv_plan_create(ctx, &s, &b.sc)) != AIG_OK) return bail(rc);
      int sh_, sw_;
      aig_conv_plan_out_dims(b.sc, nullptr, &sh_, &sw_);
      if (sh_ != oh || sw_ != ow) {
        aig_cnn_destroy(m);
        return AIG_ERR_INVALID;  // main and shortcut paths disagree on odd extents (ResConvLayer.cpp:13-20)
      }
    }
    aig_conv_desc e = d;
    e.in_c = co; e.in_h = oh; e.in_w = ow; e.kh = e.kw = 3; e.sh = e.sw = 1; e.ph = e.pw = 1;
    if ((rc = aig_conv_plan_create(ctx, &e, &b.c1)) != AIG_OK) return bail(rc);
    size_t n = (size_t)c.batch * oh * ow * co;
    // fused down-sampling launch -> 3x3 convolution: the pair passes both tensors (conv1's input and residual) in the
    // padded position layout when both plans take it, so that conv1 loads each patch as one contiguous run of rows
    if (b.down && aig_resdown_plan_set_output_padded(b.down, 1) == AIG_OK) {
      if (aig_conv_plan_set_input_padded(b.c1, 1) == AIG_OK) n = (size_t)aig_conv_padded_rows(c.batch, oh, ow, 1) * co;
      else aig_resdown_plan_set_output_padded(b.down, 0);
    }
    if (dev_alloc(m, &b.t, n) != AIG_OK || dev_alloc(m, &b.r, n) != AIG_OK) return bail(AIG_ERR_CUDA);
    m->blocks.push_back(b);
    m->bh.push_back(oh);
    m->bw.push_back(ow);
    {
      const double px = (double)c.batch * oh * ow;
      const double in_b = (double)c.batch * h * w * ci * 2, out_b = px * co * 2;
      const std::string nm = "res" + std::to_string(i);
      if (b.down) {
        m->sites.push_back({nm + ".down_k4s2+shortcut_k2s2", 2.0 * px * co * ci * 20, in_b + 2 * out_b + (double)co * ci * 20 * 2});
      } else {
        m->sites.push_back({nm + ".shortcut_k2s2", 2.0 * px * co * ci * 4, in_b + out_b + (double)co * ci * 4 * 2});
        m->sites.push_back({nm + ".conv0_k4s2", 2.0 * px * co * ci * 16, in_b + out_b + (double)co * ci * 16 * 2});
      }
      m->sites.push_back({nm + ".conv1_k3s1", 2.0 * px * co * co * 9, 3 * out_b + (double)co * co * 9 * 2});
    }
    h = oh; w = ow;
    m->launches_per_forward += b.down ? 2 : 3;
  }
  // stage outputs: channels-last, or space-to-depth blocks (zero-filled once: border sub-positions are
  // never written and stand for the padding) where the consumer is a fused down-sampling launch
  {
    const size_t n0 = m->act0_s2d ? aig_s2d_elems(c.batch, m->H0, m->W0, c.widths[0]) : (size_t)c.batch * m->H0 * m->W0 * c.widths[0];
    if (dev_alloc(m, &m->act0, n0) != AIG_OK) return bail(AIG_ERR_CUDA);
    for (int i = 0; i < c.n_blocks; ++i) {
      aig_cnn::Block& b = m->blocks[i];
      const int co = c.widths[i + 1];
      const size_t n = b.y_s2d ? aig_s2d_elems(c.batch, m->bh[i], m->bw[i], co) : (size_t)c.batch * m->bh[i] * m->bw[i] * co;
      if (dev_alloc(m, &b.y, n) != AIG_OK) return bail(AIG_ERR_CUDA);
    }
  }
  const int cl = c.widths[c.n_blocks];
  if (dev_alloc(m, &m->sa, (size_t)c.batch * h * w * cl) != AIG_OK || dev_alloc(m, &m->feat, (size_t)c.batch * cl) != AIG_OK ||
      dev_alloc(m, &m->logits, (size_t)c.batch * c.n_out) != AIG_OK || dev_alloc(m, &m->out_f32, (size_t)c.batch * c.n_out) != AIG_OK ||
      dev_alloc(m, &m->frames_dev, (size_t)c.batch * c.height * c.width * 4) != AIG_OK)
    return bail(AIG_ERR_CUDA);
  if ((rc = aig_fc_plan_create(ctx, c.batch, cl, c.n_out, AIG_ACT_NONE, 0.f, 1, &m->fc)) != AIG_OK) return bail(rc);
  // the head runs as one fused launch when a frame's last feature map fits shared memory
  m->fused_head = ((size_t)h * w * cl * 2 + (size_t)(h * w + cl) * 4 <= 200 * 1024) && ((h * w * cl) % 8 == 0);
  if (m->fused_head) {
    m->launches_per_forward += 1;
    const double fb = (double)c.batch * h * w * cl * 2;
    m->sites.push_back({"head_mask_pool_fc", 2.0 * c.batch * cl * c.n_out, fb + (double)c.batch * (cl * 2 + c.n_out * 6)});
  } else {
    m->launches_per_forward += 2 /*mask, pool*/ + 1 /*fc*/ + 2 /*sigmoid, tanh*/ + 1 /*half->float*/;
    const double fb = (double)c.batch * h * w * cl * 2;
    m->sites.push_back({"mask_attention", 0.0, 2 * fb});
    m->sites.push_back({"global_avgpool", 0.0, fb + (double)c.batch * cl * 2});
    m->sites.push_back({"fc_head", 2.0 * c.batch * cl * c.n_out, (double)c.batch * cl * 2 + (double)cl * c.n_out * 2});
    m->sites.push_back({"sigmoid_tanh_tofloat", 0.0, (double)c.batch * c.n_out * 8});
  }
  m->params.cap = aig_cnn_checkpoint_bytes(&c) + 256 * (16 + 32 * (size_t)c.n_blocks);
  if (cudaMalloc(reinterpret_cast<void**>(&m->params.base), m->params.cap) != cudaSuccess) return bail(AIG_ERR_CUDA);
  *out = m;
  return AIG_OK;
}

int aig_cnn_destroy(aig_cnn* m) {
  if (!m) return AIG_OK;
  if (m->ctx) aig_ctx_sync(m->ctx);
  for (aig_graph* g : m->graphs) aig_graph_destroy(g);
  if (m->copy_stream) {
    cudaStreamSynchronize(m->copy_stream);
    cudaStreamDestroy(m->copy_stream);
    for (int i = 0; i < 2; ++i) {
      cudaFree(m->frames_slot[i]);
      if (m->ev_h2d[i]) cudaEventDestroy(m->ev_h2d[i]);
      if (m->ev_used[i]) cudaEventDestroy(m->ev_used[i]);
      if (m->ev_done[i]) cudaEventDestroy(m->ev_done[i]);
    }
  }
  aig_conv0_plan_destroy(m->conv0);
  for (auto& b : m->blocks) {
    aig_conv_plan_destroy(b.c0);
    aig_conv_plan_destroy(b.c1);
    aig_conv_plan_destroy(b.sc);
    aig_conv_plan_destroy(b.down);
    cudaFree(b.t);
    cudaFree(b.r);
    cudaFree(b.y);
  }
  aig_conv_plan_destroy(m->fc);
  cudaFree(m->act0);
  cudaFree(m->stage_scratch);
  cudaFree(m->sa);
  cudaFree(m->feat);
  cudaFree(m->logits);
  cudaFree(m->out_f32);
  cudaFree(m->frames_dev);
  cudaFree(m->params.base);
  for (cudaEvent_t e : m->prof_ev) cudaEventDestroy(e);
  delete m;
  return AIG_OK;
}

const char* aig_cnn_last_error(aig_cnn* m) { return m ? m->err.c_str() : "null model"; }

int aig_cnn_load_memory(aig_cnn* m, const void* blob, size_t bytes) {
  if (!m || !blob) return AIG_ERR_INVALID;
  const aig_cnn_config& c = m->cfg;
  if (bytes != aig_cnn_checkpoint_bytes(&c))
    return fail(m, AIG_ERR_IO, "checkpoint size " + std::to_string(bytes) + " does not match the network (" +
                                   std::to_string(aig_cnn_checkpoint_bytes(&c)) + " bytes expected)");
  cudaStream_t s = (cudaStream_t)aig_ctx_stream(m->ctx);
  Reader rd{(const uint8_t*)blob, bytes};
  int32_t wh[2];
  rd.take_host(wh, 8);
  if (wh[0] != c.width || wh[1] != c.height)
    return fail(m, AIG_ERR_IO, "checkpoint resolution " + std::to_string(wh[0]) + "x" + std::to_string(wh[1]) +
                                   " does not match the network input");
  m->params.used = 0;
  ConvP cv;
  BnP bn;
  const float eps = 1e-6f;  // BatchNorm.cpp:5
  const char* io = "checkpoint truncated or parameter arena exhausted";
  if (!read_conv(m, rd, cv, (size_t)c.widths[0] * 3 * c.k0 * c.k0, c.widths[0], s) || !read_bn(m, rd, bn, c.widths[0], s))
    return fail(m, AIG_ERR_IO, io);
  CNN_OK(m, aig_conv0_plan_set_weights(m->conv0, cv.w, cv.b, bn.a[0], bn.a[1], bn.a[2], bn.a[3], eps));
  for (int i = 0; i < c.n_blocks; ++i) {
    const int ci = c.widths[i], co = c.widths[i + 1];
    ConvP c0, c1, sc;
    BnP b0, b1;
    if (!read_conv(m, rd, c0, (size_t)co * ci * 16, co, s) || !read_bn(m, rd, b0, co, s) ||
        !read_conv(m, rd, c1, (size_t)co * co * 9, co, s) || !read_bn(m, rd, b1, co, s) ||
        !read_conv(m, rd, sc, (size_t)co * ci * 4, co, s))
      return fail(m, AIG_ERR_IO, io);
    if (m->blocks[i].down) {
      CNN_OK(m, aig_resdown_plan_set_weights(m->blocks[i].down, c0.w, c0.b, b0.a[0], b0.a[1], b0.a[2], b0.a[3], eps, sc.w, sc.b));
    } else {
      CNN_OK(m, aig_conv_plan_set_weights(m->blocks[i].c0, c0.w, c0.b, b0.a[0], b0.a[1], b0.a[2], b0.a[3], eps));
      CNN_OK(m, aig_conv_plan_set_weights(m->blocks[i].sc, sc.w, sc.b, nullptr, nullptr, nullptr, nullptr, 0.f));
    }
    CNN_OK(m, aig_conv_plan_set_weights(m->blocks[i].c1, c1.w, c1.b, b1.a[0], b1.a[1], b1.a[2], b1.a[3], eps));
  }
  const int cl = c.widths[c.n_blocks];
  m->sa_w = (aig_half*)m->params.take((size_t)cl * 2);
  if (!m->sa_w || !rd.take(m->sa_w, (size_t)cl * 2, s) || !rd.take_host(&m->sa_b, 4)) return fail(m, AIG_ERR_IO, io);
  ConvP fc;
  if (!read_conv(m, rd, fc, (size_t)cl * c.n_out, c.n_out, s)) return fail(m, AIG_ERR_IO, io);
  CNN_OK(m, aig_fc_plan_set_weights(m->fc, fc.w, fc.b, nullptr, nullptr, nullptr, nullptr, 0.f));
  m->fcw = fc.w;
  m->fcb = fc.b;
  if (rd.left != 0) return fail(m, AIG_ERR_IO, "trailing bytes in checkpoint");
  CNN_OK(m, aig_ctx_sync(m->ctx));  // the host blob may be freed by the caller after this returns
  m->loaded = true;
  return AIG_OK;
}

int aig_cnn_load_file(aig_cnn* m, const char* path) {
  if (!m || !path) return AIG_ERR_INVALID;
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f.is_open()) return fail(m, AIG_ERR_IO, std::string("cannot open ") + path);
  const std::streamsize n = f.tellg();
  f.seekg(0);
  std::vector<char> buf((size_t)n);
  if (!f.read(buf.data(), n)) return fail(m, AIG_ERR_IO, std::string("cannot read ") + path);
  return aig_cnn_load_memory(m, buf.data(), (size_t)n);
}

}  // extern "C"

// NN::Forward (NN.cpp:93-100) over device-resident frames (BGRA pixels, or planar R,G,B uint8 planes); results
// stay on the device.
static int cnn_forward_impl(aig_cnn* m, const uint8_t* bgra_dev, bool planar) {
  if (!m || !bgra_dev) return AIG_ERR_INVALID;
  if (!m->loaded) return fail(m, AIG_ERR_INVALID, "parameters not loaded");
  const aig_cnn_config& c = m->cfg;
  cudaStream_t ps = (cudaStream_t)aig_ctx_stream(m->ctx);
  const bool prof = m->prof_on && m->prof_steps < m->prof_cap;
  const size_t ev0 = (size_t)m->prof_steps * (m->sites.size() + 1);
  size_t si = 0;
  auto tick = [&]() {
    if (prof) cudaEventRecord(m->prof_ev[ev0 + si++], ps);
  };
  tick();
  if (planar) CNN_OK(m, aig_conv0_forward_rgb_planar(m->conv0, bgra_dev, m->act0));
  else CNN_OK(m, aig_conv0_forward_bgra(m->conv0, bgra_dev, m->act0));
  tick();
  const aig_half* x = m->act0;
  for (auto& b : m->blocks) {
    if (b.down) {
      CNN_OK(m, aig_resdown_forward(b.down, x, b.t, b.r));
      tick();
    } else {
      CNN_OK(m, aig_conv_forward(b.sc, x, nullptr, b.r));
      tick();
      CNN_OK(m, aig_conv_forward(b.c0, x, nullptr, b.t));
      tick();
    }
    CNN_OK(m, aig_conv_forward(b.c1, b.t, b.r, b.y));
    tick();
    x = b.y;
  }
  const int cl = c.widths[c.n_blocks];
  const int h = c.n_blocks ? m->bh.back() : m->H0, w = c.n_blocks ? m->bw.back() : m->W0;
  if (m->fused_head) {
    // mask attention + pool + FC + sigmoid/tanh + half->float in one launch
    CNN_OK(m, aig_cnn_head_forward(m->ctx, x, m->sa_w, m->sa_b, m->fcw, m->fcb, m->feat, m->logits, m->out_f32, c.batch, h * w, cl,
                                   c.n_out, c.n_sigmoid));
    tick();
  } else {
    CNN_OK(m, aig_spatial_mask_forward(m->ctx, x, m->sa_w, m->sa_b, m->sa, c.batch, h * w, cl));
    tick();
    CNN_OK(m, aig_global_avgpool_nhwc(m->ctx, m->sa, m->feat, c.batch, h * w, cl));
    tick();
    CNN_OK(m, aig_conv_forward(m->fc, m->feat, nullptr, m->logits));
    tick();
    // Sigmoid is applied in place on the FC output, as in the reference (Sigmoid.cpp:8-12)
    CNN_OK(m, aig_sigmoid_forward(m->ctx, m->logits, c.n_out, c.n_sigmoid, c.batch * c.n_out));
    if (c.n_sigmoid < c.n_out) CNN_OK(m, aig_tanh_tail_forward(m->ctx, m->logits, c.n_out, c.n_sigmoid, c.batch * c.n_out));
    CNN_OK(m, aig_half_to_float(m->ctx, m->logits, m->out_f32, (size_t)c.batch * c.n_out));
    tick();
  }
  if (prof) ++m->prof_steps;
  return AIG_OK;
}

extern "C" {

int aig_cnn_forward(aig_cnn* m, const uint8_t* bgra_dev) { return cnn_forward_impl(m, bgra_dev, false); }
int aig_cnn_forward_rgb(aig_cnn* m, const uint8_t* rgb_planar_dev) { return cnn_forward_impl(m, rgb_planar_dev, true); }

// Per-launch timing of the eager forward: begin allocates events for up to max_steps forwards; end
// synchronises and returns, per launch site, the mean milliseconds over the recorded steps.
int aig_cnn_profile_begin(aig_cnn* m, int max_steps) {
  if (!m || max_steps <= 0) return AIG_ERR_INVALID;
  const size_t need = (size_t)max_steps * (m->sites.size() + 1);
  while (m->prof_ev.size() < need) {
    cudaEvent_t e;
    CNN_CUDA(m, cudaEventCreate(&e));
    m->prof_ev.push_back(e);
  }
  m->prof_cap = max_steps;
  m->prof_steps = 0;
  m->prof_on = true;
  return AIG_OK;
}
int aig_cnn_profile_end(aig_cnn* m, double* mean_ms, int capacity, int* steps) {
  if (!m || !mean_ms) return AIG_ERR_INVALID;
  m->prof_on = false;
  CNN_OK(m, aig_ctx_sync(m->ctx));
  const size_t n = m->sites.size();
  if (capacity < (int)n) return fail(m, AIG_ERR_INVALID, "profile buffer too small");
  for (size_t i = 0; i < n; ++i) mean_ms[i] = 0.0;
  for (int st = 0; st < m->prof_steps; ++st)
    for (size_t i = 0; i < n; ++i) {
      float ms = 0.f;
      CNN_CUDA(m, cudaEventElapsedTime(&ms, m->prof_ev[st * (n + 1) + i], m->prof_ev[st * (n + 1) + i + 1]));
      mean_ms[i] += ms;
    }
  if (m->prof_steps > 0)
    for (size_t i = 0; i < n; ++i) mean_ms[i] /= m->prof_steps;
  if (steps) *steps = m->prof_steps;
  return AIG_OK;
}
int aig_cnn_site_count(aig_cnn* m) { return m ? (int)m->sites.size() : 0; }
const char* aig_cnn_site_name(aig_cnn* m, int i) { return (m && i >= 0 && i < (int)m->sites.size()) ? m->sites[i].name.c_str() : ""; }
double aig_cnn_site_flops(aig_cnn* m, int i) { return (m && i >= 0 && i < (int)m->sites.size()) ? m->sites[i].flops : 0.0; }
double aig_cnn_site_bytes(aig_cnn* m, int i) { return (m && i >= 0 && i < (int)m->sites.size()) ? m->sites[i].bytes : 0.0; }

}  // extern "C"

// Same, replayed as one CUDA graph (captured on first use for this input pointer and frame format).
static int cnn_forward_graph_impl(aig_cnn* m, const uint8_t* bgra_dev, bool planar) {
  if (!m || !bgra_dev) return AIG_ERR_INVALID;
  int slot = -1;
  for (int i = 0; i < aig_cnn::kGraphs; ++i)
    if (m->graphs[i] && m->graph_ins[i] == bgra_dev && m->graph_planar[i] == planar) slot = i;
  if (slot < 0) {
    slot = m->graph_next;
    m->graph_next = (m->graph_next + 1) % aig_cnn::kGraphs;
    if (m->graphs[slot]) {
      aig_graph_destroy(m->graphs[slot]);
      m->graphs[slot] = nullptr;
    }
    // one eager pass first so that every plan has encoded its tensor maps before capture; per-launch timing
    // is suspended for both passes (its event records must not end up inside the graph)
    const bool prof_was_on = m->prof_on;
    m->prof_on = false;
    int rc = cnn_forward_impl(m, bgra_dev, planar);
    if (rc != AIG_OK) {
      m->prof_on = prof_was_on;
      return rc;
    }
    rc = aig_graph_begin(m->ctx);
    if (rc != AIG_OK) {
      m->prof_on = prof_was_on;
      return fail(m, rc, aig_last_error(m->ctx));
    }
    rc = cnn_forward_impl(m, bgra_dev, planar);
    aig_graph* g = nullptr;
    const int rc2 = aig_graph_end(m->ctx, &g);  // always ends the capture, also after a failed forward
    m->prof_on = prof_was_on;
    if (rc != AIG_OK) {
      aig_graph_destroy(g);
      return rc;
    }
    if (rc2 != AIG_OK) return fail(m, rc2, aig_last_error(m->ctx));
    m->graphs[slot] = g;
    m->graph_ins[slot] = bgra_dev;
    m->graph_planar[slot] = planar;
  }
  CNN_OK(m, aig_graph_launch(m->ctx, m->graphs[slot]));
  return AIG_OK;
}

extern "C" {

int aig_cnn_forward_graph(aig_cnn* m, const uint8_t* bgra_dev) { return cnn_forward_graph_impl(m, bgra_dev, false); }
int aig_cnn_forward_graph_rgb(aig_cnn* m, const uint8_t* rgb_planar_dev) { return cnn_forward_graph_impl(m, rgb_planar_dev, true); }

// Pipelined frame steps with host buffers.  submit(slot) queues, without waiting, the host->device
// copy of one batch on a private copy stream, the forward on the context stream once the copy has
// landed, and the device->host copy of the outputs; wait(slot) blocks until that slot's outputs are
// in the caller's buffer.  With the two slots used alternately the copy of step i+1 runs under the
// forward of step i.  Host buffers should be pinned.
}  // extern "C"

static int cnn_submit_host_impl(aig_cnn* m, int slot, const uint8_t* bgra_host, float* out_host, bool planar) {
  if (!m || !bgra_host || !out_host || slot < 0 || slot > 1) return AIG_ERR_INVALID;
  const aig_cnn_config& c = m->cfg;
  const size_t fb = (size_t)c.batch * c.height * c.width * 4;             // slot buffers hold either format
  const size_t copy_bytes = (size_t)c.batch * c.height * c.width * (planar ? 3 : 4);
  cudaStream_t s = (cudaStream_t)aig_ctx_stream(m->ctx);
  if (!m->copy_stream) {
    CNN_CUDA(m, cudaStreamCreateWithFlags(&m->copy_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      CNN_CUDA(m, cudaMalloc(reinterpret_cast<void**>(&m->frames_slot[i]), fb));
      CNN_CUDA(m, cudaEventCreateWithFlags(&m->ev_h2d[i], cudaEventDisableTiming));
      CNN_CUDA(m, cudaEventCreateWithFlags(&m->ev_used[i], cudaEventDisableTiming));
      CNN_CUDA(m, cudaEventCreateWithFlags(&m->ev_done[i], cudaEventDisableTiming));
    }
  }
  // the slot's frame buffer is free once the forward that last read it has run
  if (m->slot_used[slot]) CNN_CUDA(m, cudaStreamWaitEvent(m->copy_stream, m->ev_used[slot], 0));
  CNN_CUDA(m, cudaMemcpyAsync(m->frames_slot[slot], bgra_host, copy_bytes, cudaMemcpyHostToDevice, m->copy_stream));
  CNN_CUDA(m, cudaEventRecord(m->ev_h2d[slot], m->copy_stream));
  CNN_CUDA(m, cudaStreamWaitEvent(s, m->ev_h2d[slot], 0));
  const int rc = cnn_forward_graph_impl(m, m->frames_slot[slot], planar);
  if (rc != AIG_OK) return rc;
  CNN_CUDA(m, cudaEventRecord(m->ev_used[slot], s));
  m->slot_used[slot] = true;
  CNN_CUDA(m, cudaMemcpyAsync(out_host, m->out_f32, (size_t)c.batch * c.n_out * sizeof(float), cudaMemcpyDeviceToHost, s));
  CNN_CUDA(m, cudaEventRecord(m->ev_done[slot], s));
  return AIG_OK;
}

extern "C" {

int aig_cnn_submit_host(aig_cnn* m, int slot, const uint8_t* bgra_host, float* out_host) {
  return cnn_submit_host_impl(m, slot, bgra_host, out_host, false);
}
int aig_cnn_submit_host_rgb(aig_cnn* m, int slot, const uint8_t* rgb_planar_host, float* out_host) {
  return cnn_submit_host_impl(m, slot, rgb_planar_host, out_host, true);
}

int aig_cnn_wait(aig_cnn* m, int slot) {
  if (!m || slot < 0 || slot > 1 || !m->slot_used[slot]) return AIG_ERR_INVALID;
  CNN_CUDA(m, cudaEventSynchronize(m->ev_done[slot]));
  return AIG_OK;
}

// The frame step of Infer::Inference with host buffers: copy frames in, forward, copy the fp32
// outputs back, synchronise (Infer.cpp:103-112).  Host buffers should be pinned for full speed.
int aig_cnn_infer_host(aig_cnn* m, const uint8_t* bgra_host, float* out_host) {
  if (!m || !bgra_host || !out_host) return AIG_ERR_INVALID;
  const aig_cnn_config& c = m->cfg;
  cudaStream_t s = (cudaStream_t)aig_ctx_stream(m->ctx);
  CNN_CUDA(m, cudaMemcpyAsync(m->frames_dev, bgra_host, (size_t)c.batch * c.height * c.width * 4, cudaMemcpyHostToDevice, s));
  const int rc = aig_cnn_forward_graph(m, m->frames_dev);
  if (rc != AIG_OK) return rc;
  CNN_CUDA(m, cudaMemcpyAsync(out_host, m->out_f32, (size_t)c.batch * c.n_out * sizeof(float), cudaMemcpyDeviceToHost, s));
  CNN_CUDA(m, cudaStreamSynchronize(s));
  return AIG_OK;
}

const aig_half* aig_cnn_outputs_half(aig_cnn* m) { return m ? m->logits : nullptr; }
const float* aig_cnn_outputs_f32(aig_cnn* m) { return m ? m->out_f32 : nullptr; }
const aig_half* aig_cnn_features(aig_cnn* m) { return m ? m->feat : nullptr; }
int aig_cnn_kernel_launches(aig_cnn* m) { return m ? m->launches_per_forward : 0; }
const aig_half* aig_cnn_stage_output(aig_cnn* m, int stage, int* h, int* w, int* ch) {
  if (!m || stage < 0 || stage > (int)m->blocks.size()) return nullptr;
  const int sh = stage == 0 ? m->H0 : m->bh[stage - 1], sw = stage == 0 ? m->W0 : m->bw[stage - 1], sc = m->cfg.widths[stage];
  if (h) *h = sh;
  if (w) *w = sw;
  if (ch) *ch = sc;
  const aig_half* buf = stage == 0 ? m->act0 : m->blocks[stage - 1].y;
  const bool s2d = stage == 0 ? m->act0_s2d : m->blocks[stage - 1].y_s2d;
  if (!s2d) return buf;
  // the stage lives in space-to-depth blocks: hand out a channels-last copy
  const size_t n = (size_t)m->cfg.batch * sh * sw * sc;
  if (m->stage_scratch_elems < n) {
    aig_ctx_sync(m->ctx);
    cudaFree(m->stage_scratch);
    m->stage_scratch = nullptr;
    m->stage_scratch_elems = 0;
    if (cudaMalloc(reinterpret_cast<void**>(&m->stage_scratch), n * sizeof(aig_half)) != cudaSuccess) return nullptr;
    m->stage_scratch_elems = n;
  }
  if (aig_s2d_to_nhwc(m->ctx, buf, m->stage_scratch, m->cfg.batch, sh, sw, sc) != AIG_OK) return nullptr;
  return m->stage_scratch;
}

}  // extern "C"
