// seq_head.cpp -- host side of the sequence head: LSTMLayer -> MultiHeadAttentionLayer -> LayerNorm ->
// FCLayer -> Sigmoid (+tanh tail), composed from the kernel C ABI the way NN::Forward chains layers
// (NN.cpp:93-100).  Two entry points: the full-sequence forward over [B][T][d] embeddings, and the
// streaming step over [B][d] with carried LSTM state and the attention ring cache (neither exists in
// the reference, which restarts the LSTM at zero on every call: LSTMLayer.cpp:94-95).
//
// Parameter blob consumed by aig_seq_load_memory (little endian, no padding), in layer order:
//   LSTM: weightCount halves, layout of aig_lstm_plan_set_weights     (LSTMLayer.cpp:139-146)
//   MHA : half wq[E*E], wk[E*E], wv[E*E], wo[E*E]                      (MHALayer.cpp:191-210)
//   LayerNorm: float gamma[E], float beta[E]                           (LayerNorm.cpp:50-61)
//   FC  : half W[E][n_out], half b[n_out]                              (FCLayer.cpp:70-81)
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "aig_b200.h"
#include "aig_host.h"
#include "seq_step.h"

struct aig_seq {
  aig_ctx* ctx = nullptr;
  aig_seq_config cfg{};
  std::string err;
  aig_lstm_plan *lstm_full = nullptr, *lstm_step = nullptr;
  aig_mha_plan* mha = nullptr;
  aig_conv_plan *fc_full = nullptr, *fc_step = nullptr;
  uint8_t* params = nullptr;  // device copy of the blob, every array 256-byte aligned
  aig_half *lstm_w = nullptr, *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *fcw = nullptr, *fcb = nullptr;
  float *ln_g = nullptr, *ln_b = nullptr;
  aig_half *y = nullptr, *a = nullptr, *n = nullptr, *logits = nullptr;  // [B][T][.] work buffers
  aig_half *h_state = nullptr, *c_state = nullptr;                        // [layers][B][hid]
  float* out_f32 = nullptr;
  bool loaded = false;
  int position = 0;
  SeqStepFused* fused = nullptr;  // one-kernel streaming step for small batches (replaces the launches of aig_seq_step)
};

namespace {

int sfail(aig_seq* m, int code, const std::string& msg) {
  m->err = msg;
  return code;
}
#define SEQ_OK(m, expr)                                                                               \
  do {                                                                                                \
    int rc__ = (expr);                                                                                \
    if (rc__ != AIG_OK) return sfail((m), rc__, std::string(#expr ": ") + aig_last_error((m)->ctx));  \
  } while (0)

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" {

size_t aig_seq_param_bytes(const aig_seq_config* c) {
  if (!c) return 0;
  const size_t E = c->hidden;
  return aig_lstm_weight_count(c->in_c, c->hidden, c->layers, 1) * 2 + 4 * E * E * 2 + 2 * E * 4 + (E * c->n_out + c->n_out) * 2;
}

int aig_seq_create(aig_ctx* ctx, const aig_seq_config* cfg, aig_seq** out) {
  if (!ctx || !cfg || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  if (cfg->batch <= 0 || cfg->seq_len <= 0 || cfg->in_c <= 0 || cfg->hidden <= 0 || cfg->layers <= 0 || cfg->heads <= 0 ||
      cfg->n_out <= 0 || cfg->n_sigmoid < 0 || cfg->n_sigmoid > cfg->n_out)
    return AIG_ERR_INVALID;
  aig_seq* m = new aig_seq();
  m->ctx = ctx;
  m->cfg = *cfg;
  const aig_seq_config& c = m->cfg;
  int rc = aig_lstm_plan_create(ctx, c.seq_len, c.layers, c.hidden, c.batch, c.in_c, 5.0f, 1, /*batch_major*/ 1, &m->lstm_full);
  if (rc == AIG_OK) rc = aig_lstm_plan_create(ctx, 1, c.layers, c.hidden, c.batch, c.in_c, 5.0f, 1, 1, &m->lstm_step);
  if (rc == AIG_OK) rc = aig_mha_plan_create(ctx, c.batch, c.seq_len, c.hidden, c.heads, c.rope_base, c.window, &m->mha);
  if (rc == AIG_OK) rc = aig_fc_plan_create(ctx, c.batch * c.seq_len, c.hidden, c.n_out, AIG_ACT_NONE, 0.f, 1, &m->fc_full);
  if (rc == AIG_OK) rc = aig_fc_plan_create(ctx, c.batch, c.hidden, c.n_out, AIG_ACT_NONE, 0.f, 1, &m->fc_step);
  const size_t rows = (size_t)c.batch * c.seq_len, E = c.hidden;
  const size_t state = (size_t)c.layers * c.batch * E;
  if (rc == AIG_OK &&
      (cudaMalloc(&m->y, rows * E * 2) != cudaSuccess || cudaMalloc(&m->a, rows * E * 2) != cudaSuccess ||
       cudaMalloc(&m->n, rows * E * 2) != cudaSuccess || cudaMalloc(&m->logits, rows * c.n_out * 2) != cudaSuccess ||
       cudaMalloc(&m->out_f32, rows * c.n_out * 4) != cudaSuccess || cudaMalloc(&m->h_state, state * 2) != cudaSuccess ||
       cudaMalloc(&m->c_state, state * 2) != cudaSuccess || cudaMemset(m->h_state, 0, state * 2) != cudaSuccess ||
       cudaMemset(m->c_state, 0, state * 2) != cudaSuccess ||
       cudaMalloc(&m->params, aig_seq_param_bytes(&c) + 16 * 256) != cudaSuccess))
    rc = AIG_ERR_CUDA;
  if (rc == AIG_OK) {
    const int window = c.window > 0 ? c.window : c.seq_len;
    const SeqStepConfig sc{c.batch, c.in_c, c.hidden, c.layers, c.heads, window, c.n_out, c.n_sigmoid, c.rope_base, 5.0f, 1};
    const char* off = getenv("AIG_SEQ_NO_FUSED_STEP");
    if (seq_step_fused_supported(sc) && !(off && atoi(off))) rc = seq_step_fused_create(ctx, sc, &m->fused);
  }
  if (rc != AIG_OK) {
    aig_seq_destroy(m);
    return rc;
  }
  *out = m;
  return AIG_OK;
}

int aig_seq_destroy(aig_seq* m) {
  if (!m) return AIG_OK;
  if (m->ctx) aig_ctx_sync(m->ctx);
  aig_lstm_plan_destroy(m->lstm_full);
  aig_lstm_plan_destroy(m->lstm_step);
  aig_mha_plan_destroy(m->mha);
  seq_step_fused_destroy(m->fused);
  aig_conv_plan_destroy(m->fc_full);
  aig_conv_plan_destroy(m->fc_step);
  void* bufs[] = {m->params, m->y, m->a, m->n, m->logits, m->out_f32, m->h_state, m->c_state};
  for (void* b : bufs) cudaFree(b);
  delete m;
  return AIG_OK;
}

const char* aig_seq_last_error(aig_seq* m) { return m ? m->err.c_str() : "null model"; }

int aig_seq_load_memory(aig_seq* m, const void* blob, size_t bytes) {
  if (!m || !blob) return AIG_ERR_INVALID;
  const aig_seq_config& c = m->cfg;
  if (bytes != aig_seq_param_bytes(&c)) return sfail(m, AIG_ERR_IO, "parameter blob size does not match the configuration");
  const size_t E = c.hidden;
  const size_t sizes[9] = {aig_lstm_weight_count(c.in_c, c.hidden, c.layers, 1) * 2, E * E * 2, E * E * 2, E * E * 2, E * E * 2,
                           E * 4, E * 4, E * c.n_out * 2, (size_t)c.n_out * 2};
  void** dst[9] = {(void**)&m->lstm_w, (void**)&m->wq, (void**)&m->wk, (void**)&m->wv, (void**)&m->wo,
                   (void**)&m->ln_g, (void**)&m->ln_b, (void**)&m->fcw, (void**)&m->fcb};
  size_t src_off = 0, dst_off = 0;
  for (int i = 0; i < 9; ++i) {
    *dst[i] = m->params + dst_off;
    SEQ_OK(m, aig_memcpy(m->ctx, *dst[i], (const uint8_t*)blob + src_off, sizes[i]));
    src_off += sizes[i];
    dst_off = align256(dst_off + sizes[i]);
  }
  SEQ_OK(m, aig_ctx_sync(m->ctx));  // the caller may free the blob now
  SEQ_OK(m, aig_lstm_plan_set_weights(m->lstm_full, m->lstm_w));
  SEQ_OK(m, aig_lstm_plan_set_weights(m->lstm_step, m->lstm_w));
  SEQ_OK(m, aig_mha_plan_set_weights(m->mha, m->wq, m->wk, m->wv, m->wo));
  SEQ_OK(m, aig_fc_plan_set_weights(m->fc_full, m->fcw, m->fcb, nullptr, nullptr, nullptr, nullptr, 0.f));
  SEQ_OK(m, aig_fc_plan_set_weights(m->fc_step, m->fcw, m->fcb, nullptr, nullptr, nullptr, nullptr, 0.f));
  if (m->fused) SEQ_OK(m, seq_step_fused_set_weights(m->fused, m->lstm_w, m->wq, m->wk, m->wv, m->wo, m->ln_g, m->ln_b, m->fcw, m->fcb));
  m->loaded = true;
  return AIG_OK;
}

static int seq_tail(aig_seq* m, aig_conv_plan* fc, int rows) {
  const aig_seq_config& c = m->cfg;
  SEQ_OK(m, aig_layernorm_rows_forward(m->ctx, m->n, m->a, m->ln_g, m->ln_b, rows, c.hidden, 1e-5f));
  SEQ_OK(m, aig_conv_forward(fc, m->n, nullptr, m->logits));
  SEQ_OK(m, aig_sigmoid_forward(m->ctx, m->logits, c.n_out, c.n_sigmoid, rows * c.n_out));
  if (c.n_sigmoid < c.n_out) SEQ_OK(m, aig_tanh_tail_forward(m->ctx, m->logits, c.n_out, c.n_sigmoid, rows * c.n_out));
  SEQ_OK(m, aig_half_to_float(m->ctx, m->logits, m->out_f32, (size_t)rows * c.n_out));
  return AIG_OK;
}

// emb: [B][T][in_c] fp16 on the device.  Results: aig_seq_outputs_* as [B][T][n_out].
int aig_seq_forward(aig_seq* m, const aig_half* emb, int pos0) {
  if (!m || !emb) return AIG_ERR_INVALID;
  if (!m->loaded) return sfail(m, AIG_ERR_INVALID, "parameters not loaded");
  const aig_seq_config& c = m->cfg;
  SEQ_OK(m, aig_lstm_forward(m->lstm_full, emb, m->y, nullptr, nullptr, 0));
  SEQ_OK(m, aig_mha_forward(m->mha, m->y, m->a, pos0));
  return seq_tail(m, m->fc_full, c.batch * c.seq_len);
}

// One new frame per sequence: emb_t [B][in_c]; carried LSTM state and the attention ring cache advance.
int aig_seq_step(aig_seq* m, const aig_half* emb_t) {
  if (!m || !emb_t) return AIG_ERR_INVALID;
  if (!m->loaded) return sfail(m, AIG_ERR_INVALID, "parameters not loaded");
  const aig_seq_config& c = m->cfg;
  if (m->fused) {
    SEQ_OK(m, seq_step_fused_run(m->fused, emb_t, m->h_state, m->c_state, m->y, m->logits, m->out_f32, m->position));
    ++m->position;
    return AIG_OK;
  }
  SEQ_OK(m, aig_lstm_forward(m->lstm_step, emb_t, m->y, m->h_state, m->c_state, 1));
  SEQ_OK(m, aig_mha_step(m->mha, m->y, m->a, m->position));
  ++m->position;
  return seq_tail(m, m->fc_step, c.batch);
}

int aig_seq_reset(aig_seq* m) {
  if (!m) return AIG_ERR_INVALID;
  const size_t state = (size_t)m->cfg.layers * m->cfg.batch * m->cfg.hidden * 2;
  cudaStream_t s = (cudaStream_t)aig_ctx_stream(m->ctx);
  if (cudaMemsetAsync(m->h_state, 0, state, s) != cudaSuccess || cudaMemsetAsync(m->c_state, 0, state, s) != cudaSuccess)
    return sfail(m, AIG_ERR_CUDA, "state reset failed");
  m->position = 0;
  if (m->fused) seq_step_fused_reset(m->fused);
  return aig_mha_reset(m->mha);
}

const aig_half* aig_seq_outputs_half(aig_seq* m) { return m ? m->logits : nullptr; }
const float* aig_seq_outputs_f32(aig_seq* m) { return m ? m->out_f32 : nullptr; }
const aig_half* aig_seq_lstm_output(aig_seq* m) { return m ? m->y : nullptr; }

}  // extern "C"
