// train_step.cu -- the element-wise and reduction kernels of the reference's training step that lie outside the
// layers' own Backward (Train.cpp:60-109): the behaviour-cloning losses (CudaStuff.cu:76-153), the loss gradient
// (CudaStuff.cu:298-307), the NaN check (CudaStuff.cu:571-586), the activation backward passes
// (CudaStuff.cu:406-459), the bias gradient (CudaStuff.cu:372-399) and the SGD / AdamW parameter updates
// (CudaStuff.cu:194-252).  Every kernel performs, per element, the arithmetic of the reference's kernel in the
// same types and order (half products where the reference multiplies halfs, the double-precision bias
// correction of its AdamW), so parameters, moments and gradients come out bit-identical; the losses are reduced
// in a fixed order (the reference adds block sums with float atomics, i.e. in no fixed order).
// Of the layers' own Backward passes the fully connected one is here (end of the file); the convolution,
// normalisation and LSTM backward passes (cuDNN calls in the reference) are not.
#include <cmath>

#include "aig_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr float kBeta1 = 0.9f, kBeta2 = 0.999f, kAdamEps = 1e-7f, kGradClip = 128.0f;  // CudaStuff.cu:194-198

inline int blocks_for(const aig_ctx* ctx, long long n, int waves = 8) {
  long long b = (n + kThreads - 1) / kThreads, cap = (long long)ctx->sm_count * waves;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

// ---- losses: sum of squared differences, buttons and mouse axes apart (control index % n_ctrls < n_buttons)
__global__ void sq_err_partials_kernel(const __half* __restrict__ pred, const float* __restrict__ target, long long n, int n_buttons, int n_ctrls,
                                       double* __restrict__ partial /* [gridDim.x][2] */) {
  __shared__ double s_b[kThreads], s_a[kThreads];
  double b = 0.0, a = 0.0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float d = __half2float(pred[i]) - target[i];
    d *= d;
    if ((int)(i % n_ctrls) < n_buttons) b += d;
    else a += d;
  }
  s_b[threadIdx.x] = b;
  s_a[threadIdx.x] = a;
  __syncthreads();
  for (int s = kThreads / 2; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) {
      s_b[threadIdx.x] += s_b[threadIdx.x + s];
      s_a[threadIdx.x] += s_a[threadIdx.x + s];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partial[2 * blockIdx.x] = s_b[0];
    partial[2 * blockIdx.x + 1] = s_a[0];
  }
}
__global__ void sq_err_final_kernel(const double* __restrict__ partial, int blocks, float* __restrict__ out /* [2] */) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double b = 0.0, a = 0.0;
    for (int i = 0; i < blocks; ++i) {  // fixed order: the same inputs give the same sums on every run
      b += partial[2 * i];
      a += partial[2 * i + 1];
    }
    out[0] = (float)b;
    out[1] = (float)a;
  }
}

// ---- loss gradient of the squared error as the reference takes it: prediction - target, in half arithmetic
__global__ void loss_gradient_kernel(__half* __restrict__ g, const __half* __restrict__ pred, const __half* __restrict__ target, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) g[i] = __hsub(pred[i], target[i]);
}

__global__ void any_nan_kernel(const __half* __restrict__ x, long long n, int* __restrict__ flag) {
  bool found = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) found |= __hisnan(x[i]);
  if (found) atomicExch(flag, 1);
}

// ---- activation backward passes (in place on the gradient)
// Swish, from the layer's OUTPUT s = x * sigmoid(x): the reference approximates sigmoid(x) by s / (1 + s)
__global__ void swish_backward_kernel(__half* __restrict__ g, const __half* __restrict__ out, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float s = __half2float(out[i]);
    const float sig = s / (1.0f + s);
    g[i] = __float2half(__half2float(g[i]) * (s + sig * (1.0f - s)));
  }
}
__global__ void leaky_relu_backward_kernel(__half* __restrict__ g, const __half* __restrict__ x, long long n, __half slope) {
  const __half zero = __float2half(0.0f), one = __float2half(1.0f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    g[i] = __hmul(g[i], __hlt(x[i], zero) ? slope : one);
}
// sigmoid on the first n_buttons of every n_ctrls controls, from the layer's output y: g *= y * (1 - y)
__global__ void sigmoid_backward_kernel(__half* __restrict__ g, const __half* __restrict__ y, int n_ctrls, int n_buttons, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if ((int)(i % n_ctrls) >= n_buttons) continue;
    const float v = __half2float(y[i]);
    g[i] = __float2half(__half2float(g[i]) * v * (1.0f - v));
  }
}
// bias gradient: per channel, the sum of the incoming gradient over the batch rows, added in row order in fp32
__global__ void bias_gradient_kernel(const __half* __restrict__ g /* [batch][c] */, __half* __restrict__ gb /* [c] */, int c, int batch) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  float sum = 0.0f;
  for (int i = 0; i < batch; ++i) sum += __half2float(g[(size_t)i * c + ch]);
  gb[ch] = __float2half(sum);
}

// ---- parameter updates
__global__ void sgd_f16_kernel(__half* __restrict__ p, const __half* __restrict__ g, long long n, float lr, float wd) {
  const __half decay = __float2half(1.0f - wd);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const __half w = __hmul(p[i], decay);  // decoupled weight decay as a half product, then the step in fp32
    const float gc = fmaxf(fminf(__half2float(g[i]), kGradClip), -kGradClip);
    p[i] = __float2half(__half2float(w) - lr * gc);
  }
}
__global__ void sgd_f32_kernel(float* __restrict__ p, const float* __restrict__ g, long long n, float lr, float wd) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    // (the decayed parameter is a value of its own in the reference -- it is stored before the step is taken -- so
    //  the product is rounded by itself here and cannot be fused with the subtraction that follows)
    float w = __fmul_rn(p[i], 1.0f - wd);
    const float gc = fmaxf(fminf(g[i], kGradClip), -kGradClip);
    w -= lr * gc;
    p[i] = w;
  }
}
// AdamW with the reference's constants and its bias correction evaluated in double precision per element
__global__ void adamw_f32_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, long long n, float lr,
                                 int t, float wd) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gc = fmaxf(fminf(g[i], kGradClip), -kGradClip);
    const float mi = kBeta1 * m[i] + (1.0f - kBeta1) * gc;
    const float vi = kBeta2 * v[i] + (1.0f - kBeta2) * gc * gc;
    m[i] = mi;
    v[i] = vi;
    float w = __fmul_rn(p[i], 1.0f - wd);  // (rounded by itself: see sgd_f32_kernel)
    w -= lr * static_cast<float>(mi / (1.0 - pow(kBeta1, t)) / (sqrt(vi / (1.0 - pow(kBeta2, t))) + kAdamEps));
    p[i] = w;
  }
}
// AdamWHalf of one element (CudaStuff.cu:237-252): fp32 moments from fp16 storage, double-precision bias correction.
// The two correction terms 1 - beta^t are the same for every element; a block evaluates them once (the reference
// evaluates the same expressions in every thread, with the same result) and hands them in as c1, c2.
struct AdamHalf {
  __half p, m, v;
};
__device__ __forceinline__ void adamw_block_corrections(int t, double* s_c) {
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    s_c[0] = 1.0 - pow(kBeta1, t);
    s_c[1] = 1.0 - pow(kBeta2, t);
  }
  __syncthreads();
}
__device__ __forceinline__ AdamHalf adamw_f16_element(__half p, __half g, __half m, __half v, float lr, double c1, double c2, float wd) {
  const float gc = fmaxf(fminf(__half2float(g), kGradClip), -kGradClip);
  const float mi = kBeta1 * __half2float(m) + (1.0f - kBeta1) * gc;
  const float vi = kBeta2 * __half2float(v) + (1.0f - kBeta2) * gc * gc;
  const float w = __half2float(p) * (1.0f - wd);
  AdamHalf r;
  r.p = __float2half(w - lr * static_cast<float>(mi / c1 / (sqrt(vi / c2) + kAdamEps)));
  r.m = __float2half(mi);
  r.v = __float2half(vi);
  return r;
}
__global__ void adamw_f16_kernel(__half* __restrict__ p, const __half* __restrict__ g, __half* __restrict__ m, __half* __restrict__ v, long long n,
                                 float lr, int t, float wd) {
  __shared__ double s_c[2];
  adamw_block_corrections(t, s_c);
  const double c1 = s_c[0], c2 = s_c[1];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const AdamHalf r = adamw_f16_element(p[i], g[i], m[i], v[i], lr, c1, c2, wd);
    p[i] = r.p;
    m[i] = r.m;
    v[i] = r.v;
  }
}
// The same update on an FC layer's weights [rows = in_c][cols = out_c], which also writes the new weights transposed
// ([out_c][in_c], the K-major operand of the forward GEMM) through a shared-memory tile: one launch instead of the
// update and a repacking pass.  Block (32, 8), tile 32 x 32.
__global__ void adamw_f16_fc_weights_kernel(__half* __restrict__ p, const __half* __restrict__ g, __half* __restrict__ m, __half* __restrict__ v,
                                            __half* __restrict__ p_t, int rows, int cols, float lr, int t, float wd) {
  __shared__ __half tile[32][34];
  __shared__ double s_c[2];
  adamw_block_corrections(t, s_c);
  const double c1 = s_c[0], c2 = s_c[1];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) {
      const size_t at = (size_t)r * cols + c;
      const AdamHalf u = adamw_f16_element(p[at], g[at], m[at], v[at], lr, c1, c2, wd);
      p[at] = u.p;
      m[at] = u.m;
      v[at] = u.v;
      tile[i][threadIdx.x] = u.p;
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (c < cols && r < rows) p_t[(size_t)c * rows + r] = tile[threadIdx.x][i];
  }
}
// The same update on the bias, which also refreshes the forward plan's fp32 shift
__global__ void adamw_f16_fc_bias_kernel(__half* __restrict__ p, const __half* __restrict__ g, __half* __restrict__ m, __half* __restrict__ v,
                                         float* __restrict__ shift, int n, float lr, int t, float wd) {
  __shared__ double s_c[2];
  adamw_block_corrections(t, s_c);
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const AdamHalf u = adamw_f16_element(p[i], g[i], m[i], v[i], lr, s_c[0], s_c[1], wd);
    p[i] = u.p;
    m[i] = u.m;
    v[i] = u.v;
    shift[i] = __half2float(u.p);
  }
}

#define AIG_ENTER(ctx)                \
  if (!(ctx)) return AIG_ERR_INVALID; \
  DeviceGuard guard__((ctx)->device)

}  // namespace

extern "C" {

int aig_mse_loss2(aig_ctx* ctx, const aig_half* pred, const float* targets, int n_buttons, int n_ctrls, int batch, float* button_loss, float* axes_loss) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, pred && targets && n_ctrls > 0 && n_buttons >= 0 && n_buttons <= n_ctrls && batch > 0 && (button_loss || axes_loss), "aig_mse_loss2: bad arguments");
  const long long n = (long long)n_ctrls * batch;
  const int blocks = blocks_for(ctx, n, 2);
  double* partial = nullptr;
  float* out = nullptr;
  AIG_CUDA_OK(ctx, cudaMallocAsync(reinterpret_cast<void**>(&partial), (size_t)blocks * 2 * sizeof(double) + 2 * sizeof(float), ctx->stream));
  out = reinterpret_cast<float*>(partial + (size_t)blocks * 2);
  sq_err_partials_kernel<<<blocks, kThreads, 0, ctx->stream>>>((const __half*)pred, targets, n, n_buttons, n_ctrls, partial);
  sq_err_final_kernel<<<1, 32, 0, ctx->stream>>>(partial, blocks, out);
  float h[2] = {0.f, 0.f};
  cudaError_t e = cudaMemcpyAsync(h, out, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFreeAsync(partial, ctx->stream);
  AIG_CUDA_OK(ctx, e);
  // means over the buttons and over the axes of the batch (MseLoss2, CudaStuff.cu:149-150)
  if (button_loss) *button_loss = n_buttons ? h[0] / (float)(n_buttons * batch) : 0.f;
  if (axes_loss) *axes_loss = n_ctrls > n_buttons ? h[1] / (float)((n_ctrls - n_buttons) * batch) : 0.f;
  return AIG_OK;
}

int aig_loss_gradient(aig_ctx* ctx, aig_half* grad, const aig_half* pred, const aig_half* targets, long long n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, grad && pred && targets && n >= 0, "aig_loss_gradient: bad arguments");
  if (n == 0) return AIG_OK;
  loss_gradient_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((__half*)grad, (const __half*)pred, (const __half*)targets, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_any_nan_half(aig_ctx* ctx, const aig_half* data, long long n, int* found) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, data && found && n >= 0, "aig_any_nan_half: bad arguments");
  *found = 0;
  if (n == 0) return AIG_OK;
  int* flag = nullptr;
  AIG_CUDA_OK(ctx, cudaMallocAsync(reinterpret_cast<void**>(&flag), sizeof(int), ctx->stream));
  cudaMemsetAsync(flag, 0, sizeof(int), ctx->stream);
  any_nan_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((const __half*)data, n, flag);
  cudaError_t e = cudaMemcpyAsync(found, flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFreeAsync(flag, ctx->stream);
  AIG_CUDA_OK(ctx, e);
  return AIG_OK;
}

int aig_swish_backward(aig_ctx* ctx, aig_half* grad, const aig_half* output, long long n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, grad && output && n >= 0, "aig_swish_backward: bad arguments");
  if (n == 0) return AIG_OK;
  swish_backward_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((__half*)grad, (const __half*)output, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_leaky_relu_backward(aig_ctx* ctx, aig_half* grad, const aig_half* input, long long n, float slope) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, grad && input && n >= 0, "aig_leaky_relu_backward: bad arguments");
  if (n == 0) return AIG_OK;
  leaky_relu_backward_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((__half*)grad, (const __half*)input, n, __float2half(slope));
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_sigmoid_backward(aig_ctx* ctx, aig_half* grad, const aig_half* output, int n_ctrls, int n_buttons, long long n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, grad && output && n_ctrls > 0 && n_buttons >= 0 && n >= 0, "aig_sigmoid_backward: bad arguments");
  if (n == 0) return AIG_OK;
  sigmoid_backward_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((__half*)grad, (const __half*)output, n_ctrls, n_buttons, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_bias_gradient(aig_ctx* ctx, const aig_half* grad_in, aig_half* grad_bias, int channels, int batch) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, grad_in && grad_bias && channels > 0 && batch > 0, "aig_bias_gradient: bad arguments");
  bias_gradient_kernel<<<(channels + kThreads - 1) / kThreads, kThreads, 0, ctx->stream>>>((const __half*)grad_in, (__half*)grad_bias, channels, batch);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_sgd_step_f16(aig_ctx* ctx, aig_half* params, const aig_half* grads, long long n, float lr, float weight_decay) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, params && grads && n >= 0, "aig_sgd_step_f16: bad arguments");
  if (n == 0) return AIG_OK;
  sgd_f16_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((__half*)params, (const __half*)grads, n, lr, weight_decay);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_sgd_step_f32(aig_ctx* ctx, float* params, const float* grads, long long n, float lr, float weight_decay) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, params && grads && n >= 0, "aig_sgd_step_f32: bad arguments");
  if (n == 0) return AIG_OK;
  sgd_f32_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>(params, grads, n, lr, weight_decay);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_adamw_step_f32(aig_ctx* ctx, float* params, const float* grads, float* m, float* v, long long n, float lr, int t, float weight_decay) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, params && grads && m && v && n >= 0 && t >= 1, "aig_adamw_step_f32: bad arguments (t counts steps from 1)");
  if (n == 0) return AIG_OK;
  adamw_f32_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>(params, grads, m, v, n, lr, t, weight_decay);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_adamw_step_f16(aig_ctx* ctx, aig_half* params, const aig_half* grads, aig_half* m, aig_half* v, long long n, float lr, int t, float weight_decay) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, params && grads && m && v && n >= 0 && t >= 1, "aig_adamw_step_f16: bad arguments (t counts steps from 1)");
  if (n == 0) return AIG_OK;
  adamw_f16_kernel<<<blocks_for(ctx, n), kThreads, 0, ctx->stream>>>((__half*)params, (const __half*)grads, (__half*)m, (__half*)v, n, lr, t, weight_decay);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

}  // extern "C"

// ---- FCLayer::Backward (FCLayer.cpp:54-59) ------------------------------------------------------------------
// Three results from the layer's input x [batch][in_c], the incoming gradient g [batch][out_c] and the weights
// W [in_c][out_c] (fp16, fp32 accumulation, one rounding to fp16 each, as the reference's cublasGemmEx calls):
//   grad_w [in_c][out_c] = x^T . g        grad_b [out_c] = sum over the batch of g        grad_x [batch][in_c] = g . W^T
// Both products run on the tcgen05 GEMM of the forward path (an FC plan computes rows . weights^T with both
// operands K-major).  grad_x has that form as it stands (rows = g, weights = W, K = out_c); grad_w needs the batch
// as the K dimension, so x and g are transposed first (one launch, which also forms grad_b).  K extents that are not a multiple of 16
// (an 18-wide head, odd batches) are padded with zeros, which adds exact zeros to the fp32 sums.
namespace {

constexpr int kTrTile = 32;

// Operands of the weight-gradient GEMM in one launch.  blockIdx.y = 0: x [rows][cols_x] -> x_t [cols_x][rows_pad];
// blockIdx.y = 1: g [rows][cols_g] -> g_t [cols_g][rows_pad] and, when grad_b is given, grad_b[c] = the sum of g[.][c]
// in fp32 in batch order (the order of bias_gradient_kernel).  A block owns 32 columns and walks the rows in tiles of
// 32; destination columns rows..rows_pad-1 are written as zeros.  Block (32, 8).
__global__ void fc_backward_operands_kernel(const __half* __restrict__ x, __half* __restrict__ x_t, int cols_x, const __half* __restrict__ g,
                                            __half* __restrict__ g_t, int cols_g, __half* __restrict__ grad_b, int rows, int rows_pad) {
  __shared__ __half tile[kTrTile][kTrTile + 2];
  const bool is_g = blockIdx.y == 1;
  const __half* __restrict__ src = is_g ? g : x;
  __half* __restrict__ dst = is_g ? g_t : x_t;
  const int cols = is_g ? cols_g : cols_x;
  const int c0 = blockIdx.x * kTrTile;
  if (c0 >= cols) return;
  const bool sums = is_g && grad_b != nullptr && threadIdx.y == 0;
  float sum = 0.f;
  for (int r0 = 0; r0 < rows_pad; r0 += kTrTile) {
    for (int i = threadIdx.y; i < kTrTile; i += blockDim.y) {
      const int r = r0 + i, c = c0 + threadIdx.x;
      tile[i][threadIdx.x] = (r < rows && c < cols) ? src[(size_t)r * cols + c] : __float2half(0.f);
    }
    __syncthreads();
    for (int i = threadIdx.y; i < kTrTile; i += blockDim.y) {
      const int c = c0 + i, r = r0 + threadIdx.x;
      if (c < cols && r < rows_pad) dst[(size_t)c * rows_pad + r] = tile[threadIdx.x][i];
    }
    if (sums) {
      const int n = rows - r0 < kTrTile ? rows - r0 : kTrTile;
      for (int i = 0; i < n; ++i) sum += __half2float(tile[i][threadIdx.x]);
    }
    __syncthreads();
  }
  if (sums && c0 + threadIdx.x < cols) grad_b[c0 + threadIdx.x] = __float2half(sum);
}

// dst [rows][cols_pad] = src [rows][cols], zero beyond cols
__global__ void pad_cols_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int rows, int cols, int cols_pad) {
  const long long total = (long long)rows * cols_pad;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols_pad), c = (int)(i % cols_pad);
    dst[i] = c < cols ? src[(size_t)r * cols + c] : __float2half(0.f);
  }
}

inline int round_up16(int v) { return (v + 15) / 16 * 16; }

}  // namespace

struct aig_fc_backward_plan {
  aig_ctx* ctx = nullptr;
  int batch = 0, in_c = 0, out_c = 0;
  int kd = 0, kw = 0;               // padded K extents of the two products: out_c and batch
  aig_conv_plan* dgrad = nullptr;   // rows = batch, K = kd, out = in_c
  aig_conv_plan* wgrad = nullptr;   // rows = in_c,  K = kw, out = out_c
  __half* x_t = nullptr;            // [in_c][kw]; g^T [out_c][kw] is written into wgrad's weight operand in place
  __half* g_pad = nullptr;          // [batch][kd], only when kd != out_c; W [in_c][kd] goes into dgrad's operand
};

extern "C" {

int aig_fc_backward_plan_destroy(aig_fc_backward_plan* pl) {
  if (!pl) return AIG_OK;
  DeviceGuard g(pl->ctx->device);
  if (pl->dgrad) aig_conv_plan_destroy(pl->dgrad);
  if (pl->wgrad) aig_conv_plan_destroy(pl->wgrad);
  cudaFree(pl->x_t);
  cudaFree(pl->g_pad);
  delete pl;
  return AIG_OK;
}

int aig_fc_backward_plan_create(aig_ctx* ctx, int batch, int in_c, int out_c, aig_fc_backward_plan** out) {
  if (!ctx || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, batch > 0 && in_c > 0 && out_c > 0, "fc backward plan: bad extents");
  aig_fc_backward_plan* pl = new aig_fc_backward_plan();
  pl->ctx = ctx;
  pl->batch = batch; pl->in_c = in_c; pl->out_c = out_c;
  pl->kd = round_up16(out_c);
  pl->kw = round_up16(batch);
  int rc = aig_fc_plan_create(ctx, batch, pl->kd, in_c, AIG_ACT_NONE, 0.f, /*two_step*/ 0, &pl->dgrad);
  if (rc == AIG_OK) rc = aig_fc_plan_create(ctx, in_c, pl->kw, out_c, AIG_ACT_NONE, 0.f, 0, &pl->wgrad);
  auto alloc = [&](__half** p, size_t elems) {
    if (rc != AIG_OK) return;
    if (cudaMalloc(reinterpret_cast<void**>(p), elems * sizeof(__half)) != cudaSuccess) {
      cudaGetLastError();
      rc = aig_fail(ctx, AIG_ERR_CUDA, "fc backward plan: out of device memory");
    }
  };
  if (rc == AIG_OK) rc = fc_plan_identity_affine(pl->dgrad);
  if (rc == AIG_OK) rc = fc_plan_identity_affine(pl->wgrad);
  alloc(&pl->x_t, (size_t)in_c * pl->kw);
  if (pl->kd != out_c) alloc(&pl->g_pad, (size_t)batch * pl->kd);
  if (rc != AIG_OK) {
    aig_fc_backward_plan_destroy(pl);
    return rc;
  }
  *out = pl;
  return AIG_OK;
}

// FCLayer::UpdateParameters (FCLayer.cpp:60-70, the AdamW branch) for a layer whose forward runs on `forward_plan`
// (aig_fc_plan_create): AdamWHalf on the weights [in_c][out_c] and on the bias, each launch also refreshing what
// the forward plan reads (its K-major weight operand and its fp32 shift), so that no aig_fc_plan_set_weights call
// is needed after the step.  The plan's weights must have been set once before.
int aig_fc_adamw_update(aig_ctx* ctx, aig_conv_plan* forward_plan, int in_c, int out_c, aig_half* weights, const aig_half* grad_w,
                        aig_half* m_w, aig_half* v_w, aig_half* bias, const aig_half* grad_b, aig_half* m_b, aig_half* v_b, float lr, int t,
                        float weight_decay) {
  AIG_ENTER(ctx);
  __half* w_t = fc_plan_weight_buffer(forward_plan);
  float* shift = fc_plan_shift_buffer(forward_plan);
  AIG_REQUIRE(ctx, w_t && shift && in_c > 0 && out_c > 0 && weights && grad_w && m_w && v_w && bias && grad_b && m_b && v_b && t >= 1,
              "aig_fc_adamw_update: needs an FC plan with its weights set, all parameter arrays and t >= 1");
  adamw_f16_fc_weights_kernel<<<dim3((out_c + 31) / 32, (in_c + 31) / 32), dim3(32, 8), 0, ctx->stream>>>(
      (__half*)weights, (const __half*)grad_w, (__half*)m_w, (__half*)v_w, w_t, in_c, out_c, lr, t, weight_decay);
  AIG_LAUNCH_OK(ctx);
  adamw_f16_fc_bias_kernel<<<(out_c + kThreads - 1) / kThreads, kThreads, 0, ctx->stream>>>((__half*)bias, (const __half*)grad_b, (__half*)m_b,
                                                                                            (__half*)v_b, shift, out_c, lr, t, weight_decay);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

aig_half* aig_fc_backward_weight_storage(aig_fc_backward_plan* pl) {
  return pl && pl->kd == pl->out_c ? (aig_half*)fc_plan_weight_buffer(pl->dgrad) : nullptr;
}

int aig_fc_backward(aig_fc_backward_plan* pl, const aig_half* x, const aig_half* grad, const aig_half* w_in_out, aig_half* grad_w,
                    aig_half* grad_b, aig_half* grad_x) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, grad != nullptr && (grad_w == nullptr || x != nullptr) && (grad_x == nullptr || w_in_out != nullptr),
              "aig_fc_backward: the weight gradient needs x, the input gradient needs the weights");
  const dim3 tb(kTrTile, 8);
  int rc = AIG_OK;
  if (grad_w) {
    const int widest = pl->in_c > pl->out_c ? pl->in_c : pl->out_c;
    fc_backward_operands_kernel<<<dim3((widest + kTrTile - 1) / kTrTile, 2), tb, 0, ctx->stream>>>(
        (const __half*)x, pl->x_t, pl->in_c, (const __half*)grad, fc_plan_weight_buffer(pl->wgrad), pl->out_c, (__half*)grad_b, pl->batch, pl->kw);
    AIG_LAUNCH_OK(ctx);
    if ((rc = aig_conv_forward(pl->wgrad, (const aig_half*)pl->x_t, nullptr, grad_w)) != AIG_OK) return rc;
  }
  if (grad_b && !grad_w && (rc = aig_bias_gradient(ctx, grad, grad_b, pl->out_c, pl->batch)) != AIG_OK) return rc;
  if (grad_x) {
    const aig_half* g_rows = grad;
    __half* w_rows = fc_plan_weight_buffer(pl->dgrad);   // [in_c][kd]: the reference's weight layout, K padded
    if (pl->kd != pl->out_c) {
      pad_cols_kernel<<<blocks_for(ctx, (long long)pl->batch * pl->kd), kThreads, 0, ctx->stream>>>((const __half*)grad, pl->g_pad, pl->batch,
                                                                                                  pl->out_c, pl->kd);
      AIG_LAUNCH_OK(ctx);
      pad_cols_kernel<<<blocks_for(ctx, (long long)pl->in_c * pl->kd), kThreads, 0, ctx->stream>>>((const __half*)w_in_out, w_rows, pl->in_c,
                                                                                                 pl->out_c, pl->kd);
      AIG_LAUNCH_OK(ctx);
      g_rows = (const aig_half*)pl->g_pad;
    } else if ((const void*)w_in_out != (const void*)w_rows) {   // (a caller may keep its weights in the operand itself)
      AIG_CUDA_OK(ctx, cudaMemcpyAsync(w_rows, w_in_out, (size_t)pl->in_c * pl->kd * sizeof(__half), cudaMemcpyDeviceToDevice, ctx->stream));
    }
    if ((rc = aig_conv_forward(pl->dgrad, g_rows, nullptr, grad_x)) != AIG_OK) return rc;
  }
  return AIG_OK;
}

}  // extern "C"
