// agent.cpp -- the full streaming agent: 2-D frame encoder -> FC (features -> embedding) ->
// sequence head step with carried LSTM state and the attention ring cache.  One call per frame,
// the shape of the loop body of Infer::Inference (Infer.cpp:96-114): frame in, fp32 outputs out.
//
// Parameter blob: the encoder checkpoint (layout of aig_cnn_load_memory), then the bridge
// FC: half W[feat][d], half b[d] (FCLayer.cpp:70-81), then the sequence head blob
// (layout of aig_seq_load_memory).
#include <cuda_runtime.h>

#include <string>

#include "aig_b200.h"
#include "aig_host.h"

struct aig_agent {
  aig_ctx* ctx = nullptr;
  aig_cnn* cnn = nullptr;
  aig_seq* seq = nullptr;
  aig_conv_plan* bridge = nullptr;
  aig_cnn_config ccfg{};
  aig_seq_config scfg{};
  int feat = 0;
  aig_half *bw = nullptr, *bb = nullptr, *emb = nullptr;
  uint8_t* frames_dev = nullptr;
  std::string err;
};

namespace {
int afail(aig_agent* a, int code, const std::string& msg) {
  a->err = msg;
  return code;
}
}  // namespace

extern "C" {

size_t aig_agent_param_bytes(const aig_cnn_config* c, const aig_seq_config* s) {
  if (!c || !s) return 0;
  const size_t feat = c->widths[c->n_blocks];
  return aig_cnn_checkpoint_bytes(c) + (feat * s->in_c + s->in_c) * 2 + aig_seq_param_bytes(s);
}

int aig_agent_create(aig_ctx* ctx, const aig_cnn_config* ccfg, const aig_seq_config* scfg, aig_agent** out) {
  if (!ctx || !ccfg || !scfg || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  if (ccfg->batch != scfg->batch) return AIG_ERR_INVALID;
  aig_agent* a = new aig_agent();
  a->ctx = ctx;
  a->ccfg = *ccfg;
  a->scfg = *scfg;
  a->feat = ccfg->widths[ccfg->n_blocks];
  int rc = aig_cnn_create(ctx, ccfg, &a->cnn);
  if (rc == AIG_OK) rc = aig_seq_create(ctx, scfg, &a->seq);
  if (rc == AIG_OK) rc = aig_fc_plan_create(ctx, ccfg->batch, a->feat, scfg->in_c, AIG_ACT_NONE, 0.f, 1, &a->bridge);
  if (rc == AIG_OK && (cudaMalloc(&a->bw, (size_t)a->feat * scfg->in_c * 2) != cudaSuccess ||
                       cudaMalloc(&a->bb, (size_t)scfg->in_c * 2) != cudaSuccess ||
                       cudaMalloc(&a->emb, (size_t)ccfg->batch * scfg->in_c * 2) != cudaSuccess ||
                       cudaMalloc(&a->frames_dev, (size_t)ccfg->batch * ccfg->height * ccfg->width * 4) != cudaSuccess))
    rc = AIG_ERR_CUDA;
  if (rc != AIG_OK) {
    aig_agent_destroy(a);
    return rc;
  }
  *out = a;
  return AIG_OK;
}

int aig_agent_destroy(aig_agent* a) {
  if (!a) return AIG_OK;
  if (a->ctx) aig_ctx_sync(a->ctx);
  aig_cnn_destroy(a->cnn);
  aig_seq_destroy(a->seq);
  aig_conv_plan_destroy(a->bridge);
  cudaFree(a->bw);
  cudaFree(a->bb);
  cudaFree(a->emb);
  cudaFree(a->frames_dev);
  delete a;
  return AIG_OK;
}

const char* aig_agent_last_error(aig_agent* a) { return a ? a->err.c_str() : "null agent"; }

int aig_agent_load_memory(aig_agent* a, const void* blob, size_t bytes) {
  if (!a || !blob) return AIG_ERR_INVALID;
  if (bytes != aig_agent_param_bytes(&a->ccfg, &a->scfg)) return afail(a, AIG_ERR_IO, "agent parameter blob size mismatch");
  const uint8_t* p = (const uint8_t*)blob;
  const size_t n_cnn = aig_cnn_checkpoint_bytes(&a->ccfg), n_w = (size_t)a->feat * a->scfg.in_c * 2, n_b = (size_t)a->scfg.in_c * 2;
  int rc = aig_cnn_load_memory(a->cnn, p, n_cnn);
  if (rc != AIG_OK) return afail(a, rc, aig_cnn_last_error(a->cnn));
  if ((rc = aig_memcpy(a->ctx, a->bw, p + n_cnn, n_w)) != AIG_OK || (rc = aig_memcpy(a->ctx, a->bb, p + n_cnn + n_w, n_b)) != AIG_OK ||
      (rc = aig_ctx_sync(a->ctx)) != AIG_OK)
    return afail(a, rc, aig_last_error(a->ctx));
  if ((rc = aig_fc_plan_set_weights(a->bridge, a->bw, a->bb, nullptr, nullptr, nullptr, nullptr, 0.f)) != AIG_OK)
    return afail(a, rc, aig_last_error(a->ctx));
  rc = aig_seq_load_memory(a->seq, p + n_cnn + n_w + n_b, bytes - n_cnn - n_w - n_b);
  if (rc != AIG_OK) return afail(a, rc, aig_seq_last_error(a->seq));
  return AIG_OK;
}

// One frame per sequence (device BGRA [B][H][W][4]) -> outputs [B][n_out] (aig_agent_outputs_f32).
int aig_agent_step(aig_agent* a, const uint8_t* bgra_dev) {
  if (!a || !bgra_dev) return AIG_ERR_INVALID;
  // the encoder's launches replay from a CUDA graph (captured per input buffer on first use)
  int rc = aig_cnn_forward_graph(a->cnn, bgra_dev);
  if (rc != AIG_OK) return afail(a, rc, aig_cnn_last_error(a->cnn));
  if ((rc = aig_conv_forward(a->bridge, aig_cnn_features(a->cnn), nullptr, a->emb)) != AIG_OK) return afail(a, rc, aig_last_error(a->ctx));
  if ((rc = aig_seq_step(a->seq, a->emb)) != AIG_OK) return afail(a, rc, aig_seq_last_error(a->seq));
  return AIG_OK;
}

// The frame step with host buffers: H2D copy of the frames, step, D2H copy of [B][n_out] floats, sync.
int aig_agent_step_host(aig_agent* a, const uint8_t* bgra_host, float* out_host) {
  if (!a || !bgra_host || !out_host) return AIG_ERR_INVALID;
  cudaStream_t s = (cudaStream_t)aig_ctx_stream(a->ctx);
  const size_t fb = (size_t)a->ccfg.batch * a->ccfg.height * a->ccfg.width * 4;
  if (cudaMemcpyAsync(a->frames_dev, bgra_host, fb, cudaMemcpyHostToDevice, s) != cudaSuccess) return afail(a, AIG_ERR_CUDA, "H2D copy failed");
  const int rc = aig_agent_step(a, a->frames_dev);
  if (rc != AIG_OK) return rc;
  if (cudaMemcpyAsync(out_host, aig_seq_outputs_f32(a->seq), (size_t)a->scfg.batch * a->scfg.n_out * sizeof(float), cudaMemcpyDeviceToHost, s) !=
          cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    return afail(a, AIG_ERR_CUDA, "D2H copy failed");
  return AIG_OK;
}

int aig_agent_reset(aig_agent* a) { return a ? aig_seq_reset(a->seq) : AIG_ERR_INVALID; }
const float* aig_agent_outputs_f32(aig_agent* a) { return a ? aig_seq_outputs_f32(a->seq) : nullptr; }

}  // extern "C"
