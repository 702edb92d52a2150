// ctx.cu -- context, error reporting, CUDA-graph capture, host-side output decisions.
#include <stdarg.h>

#include "aig_common.cuh"

int aig_fail(aig_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->last_error = buf;
  return code;
}

static thread_local std::string g_noctx_error;

namespace {
// One bounded wait on an mbarrier that nobody arrives at: the wait runs out after `limit_cycles`, records
// `code` in the device error word and the kernel returns normally.
__global__ void expiring_wait_kernel(int* gerr, long long limit_cycles, int code) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, gerr, code, limit_cycles);
  __syncthreads();
}
}  // namespace

extern "C" {

int aig_ctx_create(aig_ctx** out, int device) {
  if (!out) return AIG_ERR_INVALID;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || device < 0 || device >= count) {
    g_noctx_error = std::string("no CUDA device ") + std::to_string(device) + ": " + cudaGetErrorString(e);
    return AIG_ERR_CUDA;
  }
  aig_ctx* ctx = new aig_ctx();
  ctx->device = device;
  DeviceGuard g(device);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    delete ctx;
    return AIG_ERR_CUDA;
  }
  if (prop.major != 10) {
    g_noctx_error = "device is not compute capability 10.x; this library only ships sm_100a kernels";
    delete ctx;
    return AIG_ERR_UNSUPPORTED;
  }
  ctx->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&ctx->d_err, sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&ctx->h_err, sizeof(int)) != cudaSuccess ||
      cudaMemset(ctx->d_err, 0, sizeof(int)) != cudaSuccess) {
    g_noctx_error = "context allocation failed";
    delete ctx;
    return AIG_ERR_CUDA;
  }
  ctx->own_stream = true;
  *out = ctx;
  return AIG_OK;
}

int aig_ctx_destroy(aig_ctx* ctx) {
  if (!ctx) return AIG_OK;
  DeviceGuard g(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  cudaFree(ctx->d_err);
  cudaFreeHost(ctx->h_err);
  delete ctx;
  return AIG_OK;
}

int aig_ctx_set_stream(aig_ctx* ctx, void* cuda_stream) {
  if (!ctx) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  if (ctx->own_stream) {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
    ctx->own_stream = false;
  }
  ctx->stream = static_cast<cudaStream_t>(cuda_stream);
  return AIG_OK;
}

void* aig_ctx_stream(aig_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int aig_ctx_sync(aig_ctx* ctx) {
  if (!ctx) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  AIG_CUDA_OK(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  AIG_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  const int code = *ctx->h_err;
  if (code != 0) {
    cudaMemsetAsync(ctx->d_err, 0, sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return aig_fail(ctx, AIG_ERR_TIMEOUT, "a bounded device-side wait expired (kernel site code %d)", code);
  }
  return AIG_OK;
}

int aig_selftest_expiring_wait(aig_ctx* ctx, long long limit_cycles) {
  if (!ctx) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, limit_cycles > 0 && limit_cycles <= 200ll * 1000 * 1000, "selftest: limit must be 1 .. 2e8 cycles");
  expiring_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_err, limit_cycles, 901);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

const char* aig_last_error(aig_ctx* ctx) { return ctx ? ctx->last_error.c_str() : g_noctx_error.c_str(); }

int aig_device_sm_count(aig_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

int aig_memcpy(aig_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx || (!dst && bytes) || (!src && bytes)) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  if (bytes == 0) return AIG_OK;
  AIG_CUDA_OK(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, ctx->stream));
  return AIG_OK;
}

int aig_graph_begin(aig_ctx* ctx) {
  if (!ctx) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  AIG_CUDA_OK(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  return AIG_OK;
}

int aig_graph_end(aig_ctx* ctx, aig_graph** out) {
  if (!ctx || !out) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  aig_graph* gr = new aig_graph();
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &gr->graph);
  if (e != cudaSuccess || !gr->graph) {
    delete gr;
    return aig_fail(ctx, AIG_ERR_CUDA, "cudaStreamEndCapture failed: %s", cudaGetErrorString(e));
  }
  e = cudaGraphInstantiate(&gr->exec, gr->graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(gr->graph);
    delete gr;
    return aig_fail(ctx, AIG_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  }
  *out = gr;
  return AIG_OK;
}

int aig_graph_launch(aig_ctx* ctx, aig_graph* g) {
  if (!ctx || !g) return AIG_ERR_INVALID;
  DeviceGuard dg(ctx->device);
  AIG_CUDA_OK(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  return AIG_OK;
}

int aig_graph_destroy(aig_graph* g) {
  if (!g) return AIG_OK;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return AIG_OK;
}

// Infer.cpp:8-57: thresholds at 0.5 for the button outputs, (int)(p*256.0f) for the axes.
int aig_actions_from_outputs(const float* p, int* actions, int frames, int n_ctrls, int n_buttons) {
  if (!p || !actions || frames < 0 || n_ctrls <= 0 || n_buttons < 0 || n_buttons > n_ctrls) return AIG_ERR_INVALID;
  for (int f = 0; f < frames; ++f)
    for (int i = 0; i < n_ctrls; ++i) {
      const float v = p[(size_t)f * n_ctrls + i];
      actions[(size_t)f * n_ctrls + i] = i < n_buttons ? (v > 0.5f ? 1 : 0) : static_cast<int>(v * 256.0f);
    }
  return AIG_OK;
}

// Infer.cpp:8-57 without the Win32 call: the INPUT array the reference hands to SendInput, as portable events
int aig_process_output(const float* p, const unsigned char* key_map, aig_input_event* events, int capacity) {
  if (!p || !key_map || (!events && capacity > 0) || capacity < 0) return AIG_ERR_INVALID;
  int n = 0;
  auto put = [&](int type, int code, int down, int dx, int dy) {
    if (n < capacity) events[n] = aig_input_event{type, code, down, dx, dy};
    ++n;
  };
  for (int i = 0; i < 11; ++i) put(AIG_EVENT_KEY, key_map[i], p[i] > 0.5f ? 1 : 0, 0, 0);
  for (int b = 0; b < 3; ++b) put(AIG_EVENT_MOUSE_BUTTON, b, p[11 + b] > 0.5f ? 1 : 0, 0, 0);
  const int mx = static_cast<int>(p[14] * 256.0f), my = static_cast<int>(p[15] * 256.0f);
  if (mx != 0 || my != 0) put(AIG_EVENT_MOUSE_MOVE, 0, 0, mx, my);
  return n;
}

int aig_process_output_to(const float* p, const unsigned char* key_map, aig_event_sink sink, void* user) {
  if (!sink) return AIG_ERR_INVALID;
  aig_input_event ev[16];
  const int n = aig_process_output(p, key_map, ev, 16);
  for (int i = 0; i < n; ++i) sink(&ev[i], user);
  return n;
}

}  // extern "C"
