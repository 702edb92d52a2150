// seq_step.cu -- the streaming step of the sequence head (LSTM layers -> attention over the ring cache
// -> LayerNorm -> FC -> sigmoid/tanh) as ONE cooperative kernel for small batches.
//
// At batch 1 every matrix of the head is a matrix-vector product: 10.5 MB of fp16 weights against a
// handful of 512-element vectors, no tensor-core shape, and as separate launches (projection GEMM +
// recurrent kernel per LSTM layer, three projections, attention, output projection, LayerNorm, FC,
// activations) the step is ~18 launches of ~10 us each.  Here all SMs stream the weights with 16-byte
// loads, one warp per output row (row-dot with a shuffle reduction), and the dependent stages are
// separated by grid-wide barriers on a global counter (bounded spin, cooperative launch):
//   LSTM layer 0 | LSTM layer 1 | ... | q,k,v | attention per (sequence, head) | output projection | tail
// Arithmetic follows the multi-launch path: fp32 accumulation, fp16 where that path stores fp16
// (h, c, q, k, v, context, attention output, LayerNorm output, FC output before and after the bias).
#include <math.h>

#include "aig_common.cuh"
#include "seq_step.h"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxLayers = 4;
constexpr int kMaxWindow = 128;
constexpr int kHeadDim = 64;

struct StepParams {
  int B, in_c, H, layers, heads, window, n_out, n_sig;
  int position, n_valid, double_bias;
  float rope_base, scale, clip;
  const __half* emb;
  const __half* lstm;
  unsigned long long w_off[kMaxLayers], r_off[kMaxLayers], bw_off[kMaxLayers], br_off[kMaxLayers];
  const __half *wq_t, *wk_t, *wv_t, *wo_t, *fcw_t, *fcb;  // [out][in]
  const float *ln_g, *ln_b;
  __half *h_state, *c_state, *h_new;
  __half *q, *k, *v, *ctx, *a, *n;
  __half *kcache, *vcache;
  __half *y, *logits;
  float* out_f32;
  unsigned int* counter;       // this launch's barrier counter: zero when the launch starts
  unsigned int* counter_next;  // the next launch's counter, zeroed by this launch
  int* gerr;
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Grid-wide barrier number `idx` of this launch.  Every CTA arrives once; the wait is bounded.
__device__ bool grid_barrier(const StepParams& p, int idx, int* s_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    red_release_gpu_add(p.counter, 1u);
    const unsigned int target = (unsigned int)(idx + 1) * gridDim.x;
    const long long t0 = clock64();
    int ok = 1;
    while ((int)(ld_acquire_gpu(p.counter) - target) < 0) {
      if (clock64() - t0 > AIG_WAIT_CYCLES) {
        atomicCAS(p.gerr, 0, 701 + idx);
        ok = 0;
        break;
      }
    }
    *s_flag = ok;
  }
  __syncthreads();
  return *s_flag != 0;
}

// sum_k w[k] * x[k] over n halfs (n % 8 == 0), lanes stride the 16-byte chunks; every lane gets the sum
__device__ __forceinline__ float row_dot(const __half* __restrict__ w, const __half* __restrict__ x, int n, int lane) {
  float acc = 0.f;
  const uint4* w4 = reinterpret_cast<const uint4*>(w);
  const uint4* x4 = reinterpret_cast<const uint4*>(x);
  for (int c = lane; c < n / 8; c += 32) {
    const uint4 a = __ldg(w4 + c), b = x4[c];
    const __half2* ah = reinterpret_cast<const __half2*>(&a);
    const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fa = __half22float2(ah[e]), fb = __half22float2(bh[e]);
      acc = fmaf(fa.x, fb.x, acc);
      acc = fmaf(fa.y, fb.y, acc);
    }
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  return acc;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__global__ void __launch_bounds__(kThreads, 1) seq_step_kernel(const StepParams p) {
  __shared__ int s_flag;
  __shared__ float s_attn[kWarps * (kHeadDim + kMaxWindow)];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * kWarps + warp, tw = gridDim.x * kWarps;
  const int H = p.H, B = p.B;
  int bar = 0;
  // Two counters alternate between launches.  Each launch clears the one its successor will use (its last
  // user, the launch before this one, has finished), so a launch always starts from zero even when an
  // earlier launch gave up on a barrier and left its own counter short.
  if (blockIdx.x == 0 && threadIdx.x == 0) *p.counter_next = 0u;

  // ---- LSTM layers: one warp per (sequence, hidden unit): the four gate rows of W and of R
  for (int l = 0; l < p.layers; ++l) {
    const int in_l = l == 0 ? p.in_c : H;
    const __half* W = p.lstm + p.w_off[l];
    const __half* R = p.lstm + p.r_off[l];
    const __half* bW = p.lstm + p.bw_off[l];
    const __half* bR = p.double_bias ? p.lstm + p.br_off[l] : nullptr;
    for (int i = gw; i < B * H; i += tw) {
      const int b = i / H, u = i - b * H;
      const __half* x = l == 0 ? p.emb + (size_t)b * p.in_c : p.h_new + ((size_t)(l - 1) * B + b) * H;
      const __half* hp = p.h_state + ((size_t)l * B + b) * H;
      float pre[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const size_t row = (size_t)g * H + u;
        const float gx = row_dot(W + row * in_l, x, in_l, lane) + __half2float(bW[row]) + (bR ? __half2float(bR[row]) : 0.f);
        pre[g] = row_dot(R + row * H, hp, H, lane) + gx;
      }
      if (lane == 0) {
        const size_t si = ((size_t)l * B + b) * H + u;
        const float ig = sigmoidf_(pre[0]), fg = sigmoidf_(pre[1]), gg = tanhf(pre[2]), og = sigmoidf_(pre[3]);
        float cn = fg * __half2float(p.c_state[si]) + ig * gg;
        if (p.clip > 0.f) cn = fminf(p.clip, fmaxf(-p.clip, cn));
        const __half ch = __float2half(cn);
        p.c_state[si] = ch;
        const __half hn = __float2half(og * tanhf(__half2float(ch)));
        p.h_new[si] = hn;
        if (l == p.layers - 1) p.y[(size_t)b * H + u] = hn;
      }
    }
    if (!grid_barrier(p, bar++, &s_flag)) return;
  }
  const __half* top = p.h_new + (size_t)(p.layers - 1) * B * H;

  // ---- q, k, v projections: one warp per output row
  for (int i = gw; i < 3 * H; i += tw) {
    const int m = i / H, j = i - m * H;
    const __half* Wt = (m == 0 ? p.wq_t : (m == 1 ? p.wk_t : p.wv_t)) + (size_t)j * H;
    __half* dst = m == 0 ? p.q : (m == 1 ? p.k : p.v);
    for (int b = 0; b < B; ++b) {
      const float acc = row_dot(Wt, top + (size_t)b * H, H, lane);
      if (lane == 0) dst[(size_t)b * H + j] = __float2half(acc);
    }
  }
  // the carried hidden state is no longer read by anyone: publish the new one
  for (int i = blockIdx.x * kThreads + threadIdx.x; i < p.layers * B * H; i += gridDim.x * kThreads) p.h_state[i] = p.h_new[i];
  if (!grid_barrier(p, bar++, &s_flag)) return;

  // ---- attention: one warp per (sequence, head); rotate q and k at `position`, append k, v to the ring
  for (int item = gw; item < B * p.heads; item += tw) {
    const int b = item / p.heads, h = item - b * p.heads;
    const int d = kHeadDim, half_d = d / 2, E = H, window = p.window, position = p.position;
    float* sq = s_attn + warp * (kHeadDim + kMaxWindow);
    float* sp = sq + d;
    const size_t row = (size_t)b * E + (size_t)h * d;
    const int slot = position % window;
    __half* kslot = p.kcache + ((size_t)b * window + slot) * E + (size_t)h * d;
    __half* vslot = p.vcache + ((size_t)b * window + slot) * E + (size_t)h * d;
    for (int j = lane; j < half_d; j += 32) {
      float cs = 1.f, sn = 0.f;
      if (p.rope_base > 0.f) {
        const float inv = powf(p.rope_base, -2.0f * (float)j / (float)d);
        const float ang = (float)position * inv;
        cs = cosf(ang);
        sn = sinf(ang);
      }
      const float qa = __half2float(p.q[row + j]), qb = __half2float(p.q[row + j + half_d]);
      const float ka = __half2float(p.k[row + j]), kb = __half2float(p.k[row + j + half_d]);
      sq[j] = __half2float(__float2half(qa * cs - qb * sn));
      sq[j + half_d] = __half2float(__float2half(qb * cs + qa * sn));
      kslot[j] = __float2half(ka * cs - kb * sn);
      kslot[j + half_d] = __float2half(kb * cs + ka * sn);
      vslot[j] = p.v[row + j];
      vslot[j + half_d] = p.v[row + j + half_d];
    }
    __syncwarp();
    float mx = -INFINITY;
    for (int i = lane; i < p.n_valid; i += 32) {
      const int pos = position - i;
      const __half* kr = p.kcache + ((size_t)b * window + (pos % window)) * E + (size_t)h * d;
      float acc = 0.f;
      for (int c = 0; c < d; c += 8) {
        const uint4 kv = *reinterpret_cast<const uint4*>(kr + c);
        const __half* kh = reinterpret_cast<const __half*>(&kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc = fmaf(sq[c + e], __half2float(kh[e]), acc);
      }
      sp[i] = acc * p.scale;
      mx = fmaxf(mx, sp[i]);
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int i = lane; i < p.n_valid; i += 32) {
      const float e = expf(sp[i] - mx);
      sp[i] = e;
      sum += e;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncwarp();
    const float inv = 1.0f / sum;
    for (int c = lane; c < d; c += 32) {
      float acc = 0.f;
      for (int i = 0; i < p.n_valid; ++i) {
        const int pos = position - i;
        acc = fmaf(sp[i], __half2float(p.vcache[((size_t)b * window + (pos % window)) * E + (size_t)h * d + c]), acc);
      }
      p.ctx[row + c] = __float2half(acc * inv);
    }
    __syncwarp();
  }
  if (!grid_barrier(p, bar++, &s_flag)) return;

  // ---- output projection
  for (int j = gw; j < H; j += tw) {
    for (int b = 0; b < B; ++b) {
      const float acc = row_dot(p.wo_t + (size_t)j * H, p.ctx + (size_t)b * H, H, lane);
      if (lane == 0) p.a[(size_t)b * H + j] = __float2half(acc);
    }
  }
  if (!grid_barrier(p, bar++, &s_flag)) return;

  // ---- tail on CTA 0: row LayerNorm (eps 1e-5), FC with the two-step rounding, sigmoid / tanh, fp32 copy
  if (blockIdx.x != 0) return;
  for (int b = warp; b < B; b += kWarps) {
    const __half* src = p.a + (size_t)b * H;
    float s = 0.f;
    for (int c = lane; c < H; c += 32) s += __half2float(src[c]);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mu = s / (float)H;
    float ss = 0.f;
    for (int c = lane; c < H; c += 32) {
      const float dlt = __half2float(src[c]) - mu;
      ss += dlt * dlt;
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)H + 1e-5f);
    for (int c = lane; c < H; c += 32)
      p.n[(size_t)b * H + c] = __float2half((__half2float(src[c]) - mu) * rstd * p.ln_g[c] + p.ln_b[c]);
  }
  __syncthreads();
  for (int i = warp; i < B * p.n_out; i += kWarps) {
    const int b = i / p.n_out, o = i - b * p.n_out;
    const float acc = row_dot(p.fcw_t + (size_t)o * H, p.n + (size_t)b * H, H, lane);
    if (lane == 0) {
      const float t = __half2float(__float2half(acc));                           // FCLayer: GEMM result stored as half,
      float v = __half2float(__float2half(t + __half2float(p.fcb[o])));          // then bias added and stored again
      v = o < p.n_sig ? 1.0f / (1.0f + expf(-v)) : tanhf(v);
      const __half hv = __float2half(v);
      p.logits[i] = hv;
      p.out_f32[i] = __half2float(hv);
    }
  }
}

__global__ void transpose_kernel(const __half* __restrict__ in_out, __half* __restrict__ out_in, int in_c, int out_c) {
  const long long total = (long long)in_c * out_c;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % in_c), o = (int)(i / in_c);
    out_in[i] = in_out[(size_t)k * out_c + o];
  }
}

}  // namespace

struct SeqStepFused {
  aig_ctx* ctx = nullptr;
  SeqStepConfig cfg{};
  StepParams prm{};
  __half* buf = nullptr;        // transposed weights + scratch
  unsigned int* counter = nullptr;  // two counters, used by alternate launches
  unsigned int launches = 0;
  int grid = 1;
  int stream_start = -1;
  bool weights_set = false;
};

bool seq_step_fused_supported(const SeqStepConfig& c) {
  return c.batch >= 1 && c.batch <= 4 && c.layers >= 1 && c.layers <= kMaxLayers && c.hidden % 8 == 0 && c.in_c % 8 == 0 &&
         c.heads * kHeadDim == c.hidden && c.window >= 1 && c.window <= kMaxWindow && c.n_out >= 1 && c.n_out <= 64;
}

int seq_step_fused_create(aig_ctx* ctx, const SeqStepConfig& c, SeqStepFused** out) {
  *out = nullptr;
  if (!seq_step_fused_supported(c)) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "fused sequence step: configuration not covered");
  DeviceGuard g(ctx->device);
  SeqStepFused* s = new SeqStepFused();
  s->ctx = ctx;
  s->cfg = c;
  const size_t E = c.hidden, BE = (size_t)c.batch * E;
  // layout of buf (halfs): wq_t wk_t wv_t wo_t fcw_t | h_new q k v ctx a n | kcache vcache
  const size_t n_w = 4 * E * E + (size_t)c.n_out * E;
  const size_t n_s = (size_t)c.layers * BE + 6 * BE;
  const size_t n_c = 2 * (size_t)c.batch * c.window * E;
  if (cudaMalloc(&s->buf, (n_w + n_s + n_c) * sizeof(__half)) != cudaSuccess || cudaMalloc(&s->counter, 2 * sizeof(unsigned int)) != cudaSuccess) {
    seq_step_fused_destroy(s);
    return aig_fail(ctx, AIG_ERR_CUDA, "fused sequence step: allocation failed");
  }
  cudaMemsetAsync(s->buf, 0, (n_w + n_s + n_c) * sizeof(__half), ctx->stream);
  cudaMemsetAsync(s->counter, 0, 2 * sizeof(unsigned int), ctx->stream);
  StepParams& p = s->prm;
  p.B = c.batch; p.in_c = c.in_c; p.H = c.hidden; p.layers = c.layers; p.heads = c.heads; p.window = c.window;
  p.n_out = c.n_out; p.n_sig = c.n_sigmoid; p.double_bias = c.double_bias; p.rope_base = c.rope_base;
  p.scale = 1.0f / sqrtf((float)kHeadDim); p.clip = c.clip;
  __half* w = s->buf;
  p.wq_t = w; p.wk_t = w + E * E; p.wv_t = w + 2 * E * E; p.wo_t = w + 3 * E * E; p.fcw_t = w + 4 * E * E;
  __half* sc = s->buf + n_w;
  p.h_new = sc; sc += (size_t)c.layers * BE;
  p.q = sc; p.k = sc + BE; p.v = sc + 2 * BE; p.ctx = sc + 3 * BE; p.a = sc + 4 * BE; p.n = sc + 5 * BE;
  p.kcache = s->buf + n_w + n_s;
  p.vcache = p.kcache + (size_t)c.batch * c.window * E;
  p.gerr = ctx->d_err;
  // blob offsets (halfs): per layer W then R, then per layer bW [and bR]
  size_t off = 0;
  for (int l = 0; l < c.layers; ++l) {
    const size_t in_l = l == 0 ? c.in_c : c.hidden;
    p.w_off[l] = off; off += 4 * E * in_l;
    p.r_off[l] = off; off += 4 * E * E;
  }
  for (int l = 0; l < c.layers; ++l) {
    p.bw_off[l] = off; off += 4 * E;
    if (c.double_bias) { p.br_off[l] = off; off += 4 * E; }
  }
  // one CTA per SM at most, and no more CTAs than there are rows to give every warp one
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, seq_step_kernel, kThreads, 0);
  int grid = (int)((BE + kWarps - 1) / kWarps);
  if (grid > ctx->sm_count) grid = ctx->sm_count;
  if (per_sm < 1) {
    seq_step_fused_destroy(s);
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "fused sequence step: kernel cannot be resident");
  }
  s->grid = grid < 1 ? 1 : grid;
  *out = s;
  return AIG_OK;
}

void seq_step_fused_destroy(SeqStepFused* s) {
  if (!s) return;
  cudaFree(s->buf);
  cudaFree(s->counter);
  delete s;
}

int seq_step_fused_set_weights(SeqStepFused* s, const aig_half* lstm_blob, const aig_half* wq, const aig_half* wk, const aig_half* wv,
                               const aig_half* wo, const float* ln_g, const float* ln_b, const aig_half* fcw, const aig_half* fcb) {
  aig_ctx* ctx = s->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, lstm_blob && wq && wk && wv && wo && ln_g && ln_b && fcw && fcb, "fused sequence step: null parameter");
  StepParams& p = s->prm;
  const int E = s->cfg.hidden;
  const aig_half* src[4] = {wq, wk, wv, wo};
  __half* dst[4] = {(__half*)p.wq_t, (__half*)p.wk_t, (__half*)p.wv_t, (__half*)p.wo_t};
  for (int i = 0; i < 4; ++i) {
    transpose_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>((const __half*)src[i], dst[i], E, E);
    AIG_LAUNCH_OK(ctx);
  }
  transpose_kernel<<<ctx->sm_count, 256, 0, ctx->stream>>>((const __half*)fcw, (__half*)p.fcw_t, E, s->cfg.n_out);
  AIG_LAUNCH_OK(ctx);
  p.lstm = (const __half*)lstm_blob;
  p.ln_g = ln_g;
  p.ln_b = ln_b;
  p.fcb = (const __half*)fcb;
  s->weights_set = true;
  return AIG_OK;
}

int seq_step_fused_reset(SeqStepFused* s) {
  s->stream_start = -1;
  cudaMemsetAsync(s->counter, 0, 2 * sizeof(unsigned int), s->ctx->stream);
  return AIG_OK;
}

int seq_step_fused_run(SeqStepFused* s, const aig_half* emb, aig_half* h_state, aig_half* c_state, aig_half* y, aig_half* logits,
                       float* out_f32, int position) {
  aig_ctx* ctx = s->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, s->weights_set && emb && h_state && c_state && y && logits && out_f32 && position >= 0, "fused sequence step: bad arguments");
  if (s->stream_start < 0) s->stream_start = position;
  AIG_REQUIRE(ctx, position >= s->stream_start, "fused sequence step: positions must not go backwards without a reset");
  StepParams& p = s->prm;
  p.emb = (const __half*)emb;
  p.h_state = (__half*)h_state;
  p.c_state = (__half*)c_state;
  p.y = (__half*)y;
  p.logits = (__half*)logits;
  p.out_f32 = out_f32;
  p.position = position;
  int n_valid = position - s->stream_start + 1;
  p.n_valid = n_valid > s->cfg.window ? s->cfg.window : n_valid;
  p.counter = s->counter + (s->launches & 1u);
  p.counter_next = s->counter + ((s->launches + 1u) & 1u);
  ++s->launches;
  void* args[] = {(void*)&p};
  AIG_CUDA_OK(ctx, cudaLaunchCooperativeKernel((const void*)seq_step_kernel, dim3(s->grid), dim3(kThreads), args, 0, ctx->stream));
  return AIG_OK;
}
