// seq_step.h -- internal interface between the sequence-head runner (host/seq_head.cpp) and the fused
// small-batch streaming step (csrc/seq_step.cu).
#pragma once
#include <stddef.h>

#include "aig_b200.h"

struct SeqStepFused;

struct SeqStepConfig {
  int batch, in_c, hidden, layers, heads, window, n_out, n_sigmoid;
  float rope_base, clip;
  int double_bias;
};

// True when the fused step covers this configuration (small batch, head size 64, bounded window).
bool seq_step_fused_supported(const SeqStepConfig& c);
int seq_step_fused_create(aig_ctx* ctx, const SeqStepConfig& c, SeqStepFused** out);
void seq_step_fused_destroy(SeqStepFused* s);
// Device pointers to the parameters as loaded (reference layouts): LSTM blob, MHA matrices [in][out],
// LayerNorm gamma/beta, FC W [in][out] and bias.  Makes the transposed copies the kernel reads.
int seq_step_fused_set_weights(SeqStepFused* s, const aig_half* lstm_blob, const aig_half* wq, const aig_half* wk,
                               const aig_half* wv, const aig_half* wo, const float* ln_g, const float* ln_b,
                               const aig_half* fcw, const aig_half* fcb);
// One streaming step: emb [B][in_c]; h_state/c_state [layers][B][hidden] are read and updated;
// y [B][hidden] = top LSTM output; logits [B][n_out] fp16 and out_f32 [B][n_out] = the head outputs.
int seq_step_fused_run(SeqStepFused* s, const aig_half* emb, aig_half* h_state, aig_half* c_state, aig_half* y,
                       aig_half* logits, float* out_f32, int position);
int seq_step_fused_reset(SeqStepFused* s);
