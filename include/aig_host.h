/* aig_host.h -- C ABI of the host-side model runners built on the kernel ABI (aig_b200.h).
 *
 * These replace the reference's model container and frame loop for the inference path:
 * NN::NN / NN::Forward (NN.cpp:11-100) and the body of Infer::Inference (Infer.cpp:96-114).
 * They own the per-layer plans and activation buffers, load parameters from a checkpoint in the
 * reference's byte layout, and replay the whole forward as one CUDA graph.
 */
#ifndef AIG_HOST_H
#define AIG_HOST_H
#include "aig_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define AIG_CNN_MAX_BLOCKS 7

/* 2-D frame encoder: Conv(3->widths[0], k0 x k0, stride 2, pad k0/2)+BN+act, n_blocks ResConv
 * blocks widths[i]->widths[i+1] (ResConvLayer.cpp:13-21), mask attention, global average pool,
 * FC -> n_out, sigmoid on the first n_sigmoid outputs and tanh on the rest. */
typedef struct aig_cnn_config {
  int batch, height, width;
  int n_blocks;
  int widths[AIG_CNN_MAX_BLOCKS + 1];
  int k0;
  int n_out, n_sigmoid;
  int act;      /* AIG_ACT_* used after every BatchNorm and after the residual add */
  float slope;
} aig_cnn_config;

typedef struct aig_cnn aig_cnn;
/* NN::NN, layer construction part (NN.cpp:33-61). */
int aig_cnn_create(aig_ctx* ctx, const aig_cnn_config* cfg, aig_cnn** out);
int aig_cnn_destroy(aig_cnn* m);
const char* aig_cnn_last_error(aig_cnn* m);
/* Size in bytes of the checkpoint this network reads. */
size_t aig_cnn_checkpoint_bytes(const aig_cnn_config* cfg);
/* NN::NN, checkpoint part (NN.cpp:13-20,67-75): header int32 width,height then every layer's
 * LoadParameters payload in construction order.  `blob` is host memory. */
int aig_cnn_load_memory(aig_cnn* m, const void* blob, size_t bytes);
int aig_cnn_load_file(aig_cnn* m, const char* path);
/* NN::Forward (NN.cpp:93-100) preceded by the frame preprocessing (Infer.cpp:103,109) on BGRA
 * frames [batch][height][width][4] resident in device memory.  Asynchronous on the context stream. */
int aig_cnn_forward(aig_cnn* m, const uint8_t* bgra_dev);
/* The same from planar uint8 frames [batch][3][height][width] (planes R, G, B): the layout
 * GrabFrameInt8(planar = true) produces (NvDisplayCap.h:70-87) and the reference's recordings store
 * (input_recorder.cpp:122-133), 3 bytes per pixel instead of 4. */
int aig_cnn_forward_rgb(aig_cnn* m, const uint8_t* rgb_planar_dev);
/* The same work replayed from a CUDA graph captured on first use. */
int aig_cnn_forward_graph(aig_cnn* m, const uint8_t* bgra_dev);
int aig_cnn_forward_graph_rgb(aig_cnn* m, const uint8_t* rgb_planar_dev);
/* One frame step with host buffers (Infer.cpp:103-112): host->device copy of the frames, forward,
 * half->float, device->host copy of [batch][n_out] floats, stream synchronise. */
int aig_cnn_infer_host(aig_cnn* m, const uint8_t* bgra_host, float* out_host);
/* The same frame step, pipelined: submit(slot) queues host->device copy (private copy stream), forward
 * and device->host copy of [batch][n_out] floats and returns at once; wait(slot) blocks until that
 * slot's outputs have arrived.  Alternating slots 0 and 1 lets the copy of step i+1 run under the
 * forward of step i.  Host buffers should be pinned and must stay valid until wait() returns. */
int aig_cnn_submit_host(aig_cnn* m, int slot, const uint8_t* bgra_host, float* out_host);
/* The same with planar uint8 RGB frames in host memory (a quarter fewer bytes over PCIe). */
int aig_cnn_submit_host_rgb(aig_cnn* m, int slot, const uint8_t* rgb_planar_host, float* out_host);
int aig_cnn_wait(aig_cnn* m, int slot);
/* Device views of the last forward's results. */
const aig_half* aig_cnn_outputs_half(aig_cnn* m);  /* [batch][n_out] after sigmoid/tanh */
const float* aig_cnn_outputs_f32(aig_cnn* m);      /* the same as fp32 (ConvertHalfToFloat) */
const aig_half* aig_cnn_features(aig_cnn* m);      /* [batch][widths[n_blocks]] pooled features */
/* Channels-last output of stage 0 (first conv) .. n_blocks (last ResConv), for layer-wise checks. */
const aig_half* aig_cnn_stage_output(aig_cnn* m, int stage, int* h, int* w, int* c);
/* Kernels launched by one aig_cnn_forward. */
int aig_cnn_kernel_launches(aig_cnn* m);
/* Per-launch device timing of aig_cnn_forward (eager path) with CUDA events on the context stream:
 * begin() arms it for up to max_steps forwards; end() synchronises and writes the mean milliseconds
 * of every launch site (aig_cnn_site_count of them, in launch order).  site_flops/site_bytes are the
 * algorithmic 2*MAC and bytes of one launch, the numerators of the roofline figures. */
int aig_cnn_profile_begin(aig_cnn* m, int max_steps);
int aig_cnn_profile_end(aig_cnn* m, double* mean_ms, int capacity, int* steps);
int aig_cnn_site_count(aig_cnn* m);
const char* aig_cnn_site_name(aig_cnn* m, int i);
double aig_cnn_site_flops(aig_cnn* m, int i);
double aig_cnn_site_bytes(aig_cnn* m, int i);

/* ---------------------------------------------------------------------------------------------
 * Recording files of the reference's input recorder and offline inference over them.  Layout: int32 width,
 * int32 height (input_recorder.cpp:24-27), then per frame uint16 keyStates, int32 mouseDeltaX, int32 mouseDeltaY
 * (10 bytes, packed) and 3*width*height bytes of planar RGB (input_recorder.cpp:122-133).  Records are counted
 * like the reference's index scan (main.cpp:41-92): whole records only. */
typedef struct aig_recording aig_recording;
int aig_recording_open(const char* path, aig_recording** out);
int aig_recording_close(aig_recording* r);
const char* aig_recording_last_error(aig_recording* r);   /* r may be null after a failed open */
int aig_recording_info(const aig_recording* r, int* width, int* height, long long* n_records);
/* `count` consecutive records from `first` (host buffers; any of the three may be null): frames
 * [count][3][height][width] as stored, key_states [count], mouse_dxdy [count][2]. */
int aig_recording_read(aig_recording* r, long long first, int count, uint8_t* frames, uint16_t* key_states, int32_t* mouse_dxdy);
/* The behaviour-cloning targets the reference trains on (Train.cpp:70-76): targets [count][16], button j = bit j
 * of keyStates for j < 14, then mouseDeltaX / 256 and mouseDeltaY / 256. */
int aig_recording_targets(const uint16_t* key_states, const int32_t* mouse_dxdy, int count, float* targets);
/* Frame encoder over records [first, first + count) in batches of `batch` (= the encoder's batch size; the last
 * batch is padded by repeating its final frame), fed as planar RGB through aig_cnn_submit_host_rgb with two
 * batches in flight.  out_host [count][n_out] fp32. */
int aig_cnn_infer_recording(aig_cnn* m, aig_recording* r, long long first, long long count, int batch, int n_out, float* out_host);

/* ---------------------------------------------------------------------------------------------
 * Sequence head: LSTMLayer (layers x hidden, double bias, clip 5) -> MultiHeadAttentionLayer (causal,
 * heads x 64, optional RoPE, optional sliding window) -> row LayerNorm (eps 1e-5) -> FCLayer ->
 * sigmoid on the first n_sigmoid outputs / tanh on the rest, chained like NN::Forward chains layers.
 * seq_len <= 128; hidden a multiple of 64, <= 512, hidden / heads == 64; in_c a multiple of 16. */
typedef struct aig_seq_config {
  int batch, seq_len;
  int in_c, hidden, layers, heads;
  int n_out, n_sigmoid;
  float rope_base; /* 0 = no rotary embedding */
  int window;      /* attention window in steps = ring cache slots; <= 0: whole sequence (cache of seq_len slots) */
} aig_seq_config;
typedef struct aig_seq aig_seq;
int aig_seq_create(aig_ctx* ctx, const aig_seq_config* cfg, aig_seq** out);
int aig_seq_destroy(aig_seq* m);
const char* aig_seq_last_error(aig_seq* m);
size_t aig_seq_param_bytes(const aig_seq_config* cfg);
/* Parameters in layer order: LSTM blob, MHA wq/wk/wv/wo, LayerNorm gamma/beta, FC W/b (host memory). */
int aig_seq_load_memory(aig_seq* m, const void* blob, size_t bytes);
/* Full sequence: emb [batch][seq_len][in_c] fp16 (device); positions pos0 .. pos0+seq_len-1. */
int aig_seq_forward(aig_seq* m, const aig_half* emb, int pos0);
/* Streaming: one new step per sequence, emb_t [batch][in_c]; LSTM state and the ring cache carry over. */
int aig_seq_step(aig_seq* m, const aig_half* emb_t);
int aig_seq_reset(aig_seq* m);
const aig_half* aig_seq_outputs_half(aig_seq* m); /* [batch][seq_len][n_out] (forward) or [batch][n_out] (step) */
const float* aig_seq_outputs_f32(aig_seq* m);
const aig_half* aig_seq_lstm_output(aig_seq* m);  /* top-layer h, [batch][seq_len][hidden] / [batch][hidden] */

/* ---------------------------------------------------------------------------------------------
 * Streaming agent: frame encoder -> FC (features -> in_c) -> sequence head step; one call per frame,
 * the loop body of Infer::Inference (Infer.cpp:96-114).  The two configs must have the same batch. */
typedef struct aig_agent aig_agent;
int aig_agent_create(aig_ctx* ctx, const aig_cnn_config* cnn, const aig_seq_config* seq, aig_agent** out);
int aig_agent_destroy(aig_agent* a);
const char* aig_agent_last_error(aig_agent* a);
size_t aig_agent_param_bytes(const aig_cnn_config* cnn, const aig_seq_config* seq);
/* Blob: encoder checkpoint, bridge FC (half W[feat][in_c], half b[in_c]), sequence head blob. */
int aig_agent_load_memory(aig_agent* a, const void* blob, size_t bytes);
int aig_agent_step(aig_agent* a, const uint8_t* bgra_dev);
int aig_agent_step_host(aig_agent* a, const uint8_t* bgra_host, float* out_host);
int aig_agent_reset(aig_agent* a);
const float* aig_agent_outputs_f32(aig_agent* a);

/* ---------------------------------------------------------------------------------------------
 * Temporal clip encoder: n_layers of ConvLayer3D(k 3x3x3, stride 1x2x2, pad 1) -> BatchNorm -> LeakyReLU
 * (ConvLayer3D.cpp:106-111) with channel widths[0]=3 .. widths[n_layers], adaptive average pool to 2x2
 * cells (mean over depth), FC -> n_out, sigmoid on the first n_sigmoid outputs and tanh on the rest. */
#define AIG_C3D_MAX_LAYERS 6
typedef struct aig_c3d_config {
  int batch, depth, height, width;
  int n_layers;
  int widths[AIG_C3D_MAX_LAYERS + 1];
  int n_out, n_sigmoid;
  float slope;
} aig_c3d_config;
typedef struct aig_c3d aig_c3d;
int aig_c3d_create(aig_ctx* ctx, const aig_c3d_config* cfg, aig_c3d** out);
int aig_c3d_destroy(aig_c3d* m);
const char* aig_c3d_last_error(aig_c3d* m);
size_t aig_c3d_param_bytes(const aig_c3d_config* cfg);
/* Per layer: ConvLayer3D payload (half w[K][C][3][3][3], half b[K]; ConvLayer3D.cpp:128-139) then the
 * BatchNorm payload (six float[K]; BatchNorm.cpp:90-117); then FC half W[in][out], half b[out]. */
int aig_c3d_load_memory(aig_c3d* m, const void* blob, size_t bytes);
/* clips: planar fp16 [batch][3][depth][height][width] (device).  Asynchronous on the context stream. */
int aig_c3d_forward(aig_c3d* m, const aig_half* clips);
const float* aig_c3d_outputs_f32(aig_c3d* m);   /* [batch][n_out] */
const aig_half* aig_c3d_features(aig_c3d* m);   /* [batch][widths[n_layers]*4] pooled features */

/* ---------------------------------------------------------------------------------------------
 * The reference's own network through the C++ layer classes (ai-gamer_b200/host/layers/Layers.h, the
 * reference-compatible `Layer` subclasses and `NN`): new NN(handle, handle, w, h, train=false) with the
 * checkpoint path as an argument (NN.cpp:11-91), NN::Forward on one planar fp16 frame [3][h][w]
 * (NN.cpp:93-100).  C hooks for tests and other languages; C++ callers use the classes directly. */
int aig_refnn_create(aig_ctx* ctx, int w, int h, const char* ckpt_path, void** out);
int aig_refnn_forward(void* nn, aig_half* x_nchw_dev, const aig_half** out_dev);
int aig_refnn_input_size(void* nn, int* w, int* h);
/* cudnnCreate / cublasCreate as Infer.cpp:76-79 calls them: a context bound to the legacy default stream, on
 * which the reference's launchers (aig_compat.h), its layers and its cudaMemcpy calls run in issue order. */
int aig_compat_handle_create(aig_ctx** out);
/* The loop body of Infer::Inference (Infer.cpp:103-112) through the reference's own names, with no
 * synchronisation added: ARGBtoRGBplanar, ConvertAndNormalize, NN::Forward, ConvertHalfToFloat, cudaMemcpy to
 * the host.  `nn` must live on a handle from aig_compat_handle_create.  bgra_dev [h][w][4] bytes; planar_dev
 * 3*w*h bytes and frame_half_dev 3*w*h halves are scratch; out_f32_dev and out_host hold 16 floats. */
int aig_refnn_infer_frame(void* nn, unsigned char* bgra_dev, unsigned char* planar_dev, aig_half* frame_half_dev,
                          float* out_f32_dev, float* out_host);
int aig_refnn_destroy(void* nn);
const char* aig_layers_last_error(void);

/* Any single layer class of Layers.h through C: `kind` is the class name -- ConvLayer (ConvLayer.h:8),
 * ConvLayer3D (ConvLayer3D.h:8), BatchNorm (BatchNorm.h:7; first integer 1 = spatial, 0 = per activation),
 * Activate (Activate.h:7), Swish (Swish.h:6), LeakyReLU (LeakyReLU.h:7), Sigmoid (Sigmoid.h:5), FCLayer
 * (FCLayer.h:8), ResConvLayer (ResConvLayer.h:12), LayerNorm (LayerNorm.h:6), SpatialAttentionLayer
 * (SpatialAttentionLayer.h:7), LSTMLayer (LSTMLayer.h:8), LSTMLayerV8 (the LSTMLayerv8.h:10 constructor form),
 * MultiHeadAttentionLayer (MHALayer.h:9), Dropout (Dropout.h:8) -- and iargs are that constructor's integer
 * arguments in declaration order (sizes that the reference passes as int* go by value).
 * forward = Layer::Forward (Layer.h:7); load/save = Layer::LoadParameters / SaveParameters (Layer.h:10-11) on a
 * file that holds exactly the layer's payload; param_bytes = GetParameterSize() (the staging size, Layer.h:14);
 * out_count = outNCHW_ (Layer.h:18).
 * backward = Layer::Backward (Layer.h:8) and update = Layer::UpdateParameters (Layer.h:9): implemented by the kind
 * "FCLayerTrain" (FCLayer with train = true: FCLayer.cpp:54-70, gradients of the last forward's input, then the AdamW
 * step on weights and bias); the other kinds hand back a null gradient like the base class. */
int aig_layer_create(aig_ctx* ctx, const char* kind, const int* iargs, int n_iargs, void** out);
int aig_layer_forward(void* layer, aig_half* x_dev, const aig_half** out_dev);
int aig_layer_backward(void* layer, aig_half* grad_dev, const aig_half** grad_in_dev);
int aig_layer_update(void* layer, float learning_rate);
int aig_layer_load_file(void* layer, const char* path);
int aig_layer_save_file(void* layer, const char* path);
size_t aig_layer_param_bytes(void* layer);
int aig_layer_out_count(void* layer);
int aig_layer_destroy(void* layer);

#ifdef __cplusplus
}
#endif
#endif /* AIG_HOST_H */
