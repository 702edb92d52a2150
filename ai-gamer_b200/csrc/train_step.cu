// train_step.cu -- the element-wise and reduction kernels of the reference's training step that lie outside the
// layers' own Backward (Train.cpp:60-109): the behaviour-cloning losses (CudaStuff.cu:76-153), the loss gradient
// (CudaStuff.cu:298-307), the NaN check (CudaStuff.cu:571-586), the activation backward passes
// (CudaStuff.cu:406-459), the bias gradient (CudaStuff.cu:372-399) and the SGD / AdamW parameter updates
// (CudaStuff.cu:194-252).  Every kernel performs, per element, the arithmetic of the reference's kernel in the
// same types and order (half products where the reference multiplies halfs, the double-precision bias
// correction of its AdamW), so parameters, moments and gradients come out bit-identical; the losses are reduced
// in a fixed order (the reference adds block sums with float atomics, i.e. in no fixed order).
// The convolution / GEMM / LSTM backward passes (cuDNN / cuBLAS calls in the reference) are not part of this file.
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
__global__ void adamw_f16_kernel(__half* __restrict__ p, const __half* __restrict__ g, __half* __restrict__ m, __half* __restrict__ v, long long n,
                                 float lr, int t, float wd) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gc = fmaxf(fminf(__half2float(g[i]), kGradClip), -kGradClip);
    const float mi = kBeta1 * __half2float(m[i]) + (1.0f - kBeta1) * gc;
    const float vi = kBeta2 * __half2float(v[i]) + (1.0f - kBeta2) * gc * gc;
    const float w = __half2float(p[i]) * (1.0f - wd);
    p[i] = __float2half(w - lr * static_cast<float>(mi / (1.0 - pow(kBeta1, t)) / (sqrt(vi / (1.0 - pow(kBeta2, t))) + kAdamEps)));
    m[i] = __float2half(mi);
    v[i] = __float2half(vi);
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
