// elementwise.cu -- HBM-bound operators of the forward path: preprocessing, conversions, layout
// changes, activations, residual add, BatchNorm (stand-alone), LayerNorm (both axes), spatial
// attention (reference mode and mask mode), pooling.  All are 128-bit vectorised where the
// pointer/extent alignment allows and sized as grid-stride loops over a multiple of the SM count.
#include "aig_common.cuh"

namespace {

constexpr int kThreads = 256;

inline int grid_for(const aig_ctx* ctx, long long work_items, int per_block = kThreads, int waves = 8) {
  long long blocks = (work_items + per_block - 1) / per_block;
  long long cap = (long long)ctx->sm_count * waves;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------------------------------
// Preprocessing
__global__ void bgra_to_planar_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int n) {
  // 4 pixels per thread when everything is 4-aligned; scalar tail otherwise.
  const int n4 = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3u) == 0 && (n & 3) == 0) ? n / 4 : 0;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
  for (int i = tid; i < n4; i += nthreads) {
    const uint4 v = reinterpret_cast<const uint4*>(src)[i];
    const uint32_t px[4] = {v.x, v.y, v.z, v.w};
    uint32_t r = 0, g = 0, b = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      b |= (px[k] & 0xFFu) << (8 * k);
      g |= ((px[k] >> 8) & 0xFFu) << (8 * k);
      r |= ((px[k] >> 16) & 0xFFu) << (8 * k);
    }
    reinterpret_cast<uint32_t*>(dst)[i] = r;
    reinterpret_cast<uint32_t*>(dst + n)[i] = g;
    reinterpret_cast<uint32_t*>(dst + 2 * (size_t)n)[i] = b;
  }
  for (int i = n4 * 4 + tid; i < n; i += nthreads) {
    dst[i] = src[4 * (size_t)i + 2];
    dst[i + (size_t)n] = src[4 * (size_t)i + 1];
    dst[i + 2 * (size_t)n] = src[4 * (size_t)i];
  }
}

__device__ __forceinline__ __half norm_u8(uint32_t v) { return __float2half_rn(__fdiv_rn((float)v, 255.0f)); }

__global__ void convert_normalize_kernel(__half* __restrict__ out, const uint8_t* __restrict__ in, size_t n) {
  __shared__ __half lut[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = norm_u8(i);
  __syncthreads();
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  const size_t n16 = (aligned16(in) && aligned16(out)) ? n / 16 : 0;
  for (size_t i = tid; i < n16; i += nthreads) {
    const uint4 v = reinterpret_cast<const uint4*>(in)[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    __align__(16) __half h[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) h[k] = lut[(w[k >> 2] >> (8 * (k & 3))) & 0xFFu];
    reinterpret_cast<uint4*>(out)[2 * i] = reinterpret_cast<const uint4*>(h)[0];
    reinterpret_cast<uint4*>(out)[2 * i + 1] = reinterpret_cast<const uint4*>(h)[1];
  }
  for (size_t i = n16 * 16 + tid; i < n; i += nthreads) out[i] = lut[in[i]];
}

// BGRA [frames][hw][4] -> fp16 [frames][3][hw]; 4 pixels per thread (hw % 4 == 0 path).
__global__ void preprocess_bgra_kernel(const uint8_t* __restrict__ bgra, __half* __restrict__ out, int frames, int hw) {
  __shared__ __half lut[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = norm_u8(i);
  __syncthreads();
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  if ((hw & 3) == 0 && aligned16(bgra) && (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
    const int q = hw / 4;
    const size_t total = (size_t)frames * q;
    for (size_t i = tid; i < total; i += nthreads) {
      const int f = (int)(i / q), j = (int)(i % q);
      const uint4 v = reinterpret_cast<const uint4*>(bgra)[i];
      const uint32_t px[4] = {v.x, v.y, v.z, v.w};
      __align__(8) __half r[4], g[4], b[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        b[k] = lut[px[k] & 0xFFu];
        g[k] = lut[(px[k] >> 8) & 0xFFu];
        r[k] = lut[(px[k] >> 16) & 0xFFu];
      }
      __half* o = out + (size_t)f * 3 * hw + (size_t)j * 4;
      *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(r);
      *reinterpret_cast<uint2*>(o + hw) = *reinterpret_cast<const uint2*>(g);
      *reinterpret_cast<uint2*>(o + 2 * (size_t)hw) = *reinterpret_cast<const uint2*>(b);
    }
  } else {
    const size_t total = (size_t)frames * hw;
    for (size_t i = tid; i < total; i += nthreads) {
      const size_t f = i / hw, j = i % hw;
      __half* o = out + f * 3 * hw + j;
      o[0] = lut[bgra[4 * i + 2]];
      o[hw] = lut[bgra[4 * i + 1]];
      o[2 * (size_t)hw] = lut[bgra[4 * i]];
    }
  }
}

__global__ void unconvert_kernel(uint8_t* __restrict__ out, const __half* __restrict__ in, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = static_cast<unsigned char>(__half2float(in[i]) * 255.0f);
}
// Box-filter down-scaling of uint8 frames (ConvScale.cpp:41-52 = ConvertAndNormalize + k x k stride-k convolution with
// an all-half(1/k^2) filter + UnConvertAndUnNormalize), with the colour split of ARGBtoRGBplanar fused in when the
// source is BGRA.  One thread per output pixel (x fastest).  fp32 accumulation in a fixed order (channel, row,
// column), one fused multiply-add per tap: the same order as the oracle, hence bit-exact.
template <bool BGRA>
__global__ void resize_box_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ out_u8, __half* __restrict__ out_half, int frames, int C,
                                  int H, int W, int k, int cross) {
  const int Ho = H / k, Wo = W / k;
  const long long total = (long long)frames * C * Ho * Wo;
  const float wk = __half2float(__float2half(1.0f / (float)(k * k)));
  const float inv255 = __uint_as_float(0x3B808081u);  // half(b * fl(1/255)) == half(b / 255.0f) for every byte b
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ox = (int)(i % Wo);
    long long t = i / Wo;
    const int oy = (int)(t % Ho);
    t /= Ho;
    const int c = (int)(t % C), n = (int)(t / C);
    float acc = 0.f;
    for (int ci = cross ? 0 : c; ci < (cross ? C : c + 1); ++ci)
      for (int dy = 0; dy < k; ++dy) {
        const int y = oy * k + dy;
        for (int dx = 0; dx < k; ++dx) {
          const int x = ox * k + dx;
          const uint8_t b = BGRA ? src[(((size_t)n * H + y) * W + x) * 4 + (2 - ci)] : src[(((size_t)n * C + ci) * H + y) * W + x];
          acc = fmaf(__half2float(__float2half(__fmul_rn((float)b, inv255))), wk, acc);
        }
      }
    const __half hv = __float2half(acc);
    if (out_half) out_half[i] = hv;
    if (out_u8) out_u8[i] = static_cast<unsigned char>(__half2float(hv) * 255.0f);
  }
}

__global__ void half_to_float_kernel(const __half* __restrict__ src, float* __restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __half2float(src[i]);
}
__global__ void float_to_half_kernel(const float* __restrict__ src, __half* __restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __float2half(src[i]);
}

// [batch][rows][cols] -> [batch][cols][rows], 32x32 tiles through shared memory.
__global__ void transpose_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int rows, int cols) {
  __shared__ __half tile[32][33];
  const size_t boff = (size_t)blockIdx.z * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[boff + (size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[boff + (size_t)c * rows + r] = tile[threadIdx.x][j];
  }
}

// ------------------------------------------------------------------------------------------
// In-place unary operators, 8 halves per thread.
struct OpSwish {
  __device__ __forceinline__ __half operator()(__half v) const {
    const float x = __half2float(v);
    return __float2half(x / (1.0f + expf(-x)));
  }
};
struct OpRelu {
  __device__ __forceinline__ __half operator()(__half v) const {
    return __half2float(v) > 0.0f ? v : __ushort_as_half((unsigned short)0);  // NaN -> 0
  }
};
struct OpLeaky {
  __half slope;
  __device__ __forceinline__ __half operator()(__half v) const {
    return v < __float2half(0.0f) ? __hmul(v, slope) : v;
  }
};

template <class Op>
__global__ void unary_inplace_kernel(__half* __restrict__ data, size_t n, Op op) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  const size_t n8 = aligned16(data) ? n / 8 : 0;
  for (size_t i = tid; i < n8; i += nthreads) {
    uint4 v = reinterpret_cast<uint4*>(data)[i];
    __half* h = reinterpret_cast<__half*>(&v);
#pragma unroll
    for (int k = 0; k < 8; ++k) h[k] = op(h[k]);
    reinterpret_cast<uint4*>(data)[i] = v;
  }
  for (size_t i = n8 * 8 + tid; i < n; i += nthreads) data[i] = op(data[i]);
}

__global__ void sigmoid_head_kernel(__half* data, int num_ctrls, int num_buts, int size, int tanh_tail) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < size; i += gridDim.x * blockDim.x) {
    const bool button = (i % num_ctrls) < num_buts;
    if (!tanh_tail && button) {
      const float v = __half2float(data[i]);
      data[i] = __float2half(1.0f / (1.0f + expf(-v)));
    } else if (tanh_tail && !button) {
      data[i] = __float2half(tanhf(__half2float(data[i])));
    }
  }
}

__global__ void add_kernel(__half* __restrict__ m, const __half* __restrict__ r, size_t n) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
  const size_t n8 = (aligned16(m) && aligned16(r)) ? n / 8 : 0;
  for (size_t i = tid; i < n8; i += nthreads) {
    uint4 a = reinterpret_cast<uint4*>(m)[i];
    const uint4 b = reinterpret_cast<const uint4*>(r)[i];
    __half* ha = reinterpret_cast<__half*>(&a);
    const __half* hb = reinterpret_cast<const __half*>(&b);
#pragma unroll
    for (int k = 0; k < 8; ++k) ha[k] = __float2half(__half2float(ha[k]) + __half2float(hb[k]));
    reinterpret_cast<uint4*>(m)[i] = a;
  }
  for (size_t i = n8 * 8 + tid; i < n; i += nthreads) m[i] = __float2half(__half2float(m[i]) + __half2float(r[i]));
}

// BatchNorm inference on NCHW; parameter index = channel (spatial) or c*HW+i (per activation).
__global__ void batchnorm_kernel(const __half* __restrict__ x, __half* __restrict__ y, const float* __restrict__ gamma,
                                 const float* __restrict__ beta, const float* __restrict__ mean,
                                 const float* __restrict__ var, size_t total, int c, int hw, float eps, int per_act) {
  const size_t chw = (size_t)c * hw;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t p = per_act ? (i % chw) : ((i / hw) % c);
    const float inv = 1.0f / sqrtf(var[p] + eps);
    y[i] = __float2half(gamma[p] * (__half2float(x[i]) - mean[p]) * inv + beta[p]);
  }
}

// ------------------------------------------------------------------------------------------
// LayerNorm, reference axis: one block per channel; Welford per thread, Chan merge across the block,
// then the same block normalises its channel (second read served from L2).
struct Wf {
  float mean, m2, n;
};
__device__ __forceinline__ Wf wf_merge(Wf a, Wf b) {
  if (b.n == 0.f) return a;
  if (a.n == 0.f) return b;
  const float n = a.n + b.n, d = b.mean - a.mean;
  Wf r;
  r.mean = a.mean + d * (b.n / n);
  r.m2 = a.m2 + b.m2 + d * d * (a.n * b.n / n);
  r.n = n;
  return r;
}
__global__ void layernorm_channel_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                                         const float* __restrict__ gamma, const float* __restrict__ beta,
                                         float* __restrict__ mean, float* __restrict__ variance, int N, int C, int HW,
                                         float eps) {
  __shared__ Wf red[32];
  __shared__ float s_mean, s_var;
  for (int c = blockIdx.x; c < C; c += gridDim.x) {
    Wf w = {0.f, 0.f, 0.f};
    for (int n = 0; n < N; ++n) {
      const __half* row = in + ((size_t)n * C + c) * HW;
      for (int i = threadIdx.x; i < HW; i += blockDim.x) {
        const float v = __half2float(row[i]);
        w.n += 1.f;
        const float d = v - w.mean;
        w.mean += d / w.n;
        w.m2 += d * (v - w.mean);
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      Wf other;
      other.mean = __shfl_down_sync(0xffffffffu, w.mean, o);
      other.m2 = __shfl_down_sync(0xffffffffu, w.m2, o);
      other.n = __shfl_down_sync(0xffffffffu, w.n, o);
      w = wf_merge(w, other);
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = w;
    __syncthreads();
    if (threadIdx.x < 32) {
      Wf v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : Wf{0.f, 0.f, 0.f};
      for (int o = 16; o > 0; o >>= 1) {
        Wf other;
        other.mean = __shfl_down_sync(0xffffffffu, v.mean, o);
        other.m2 = __shfl_down_sync(0xffffffffu, v.m2, o);
        other.n = __shfl_down_sync(0xffffffffu, v.n, o);
        v = wf_merge(v, other);
      }
      if (threadIdx.x == 0) {
        s_mean = v.mean;
        s_var = v.m2 / v.n;
        mean[c] = s_mean;
        variance[c] = s_var;
      }
    }
    __syncthreads();
    const float mu = s_mean, rs = sqrtf(s_var + eps), g = gamma[c], b = beta[c];
    for (int n = 0; n < N; ++n) {
      const __half* row = in + ((size_t)n * C + c) * HW;
      __half* orow = out + ((size_t)n * C + c) * HW;
      for (int i = threadIdx.x; i < HW; i += blockDim.x) {
        const float norm = (__half2float(row[i]) - mu) / rs;
        orow[i] = __float2half(norm * g + b);
      }
    }
    __syncthreads();
  }
}

// Row-wise LayerNorm: one warp per row, the row lives in registers (single pass over HBM).
template <int VPL>  // uint4 vectors (8 halves) per lane; C == 32*8*VPL exactly or smaller (masked)
__global__ void layernorm_rows_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                                      const float* __restrict__ gamma, const float* __restrict__ beta, int rows, int C,
                                      float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int nvec = C / 8;
  for (int r = warp; r < rows; r += nwarps) {
    const uint4* src = reinterpret_cast<const uint4*>(in + (size_t)r * C);
    uint4 v[VPL];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int idx = lane + 32 * k;
      if (idx < nvec) {
        v[k] = src[idx];
        const __half* h = reinterpret_cast<const __half*>(&v[k]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += __half2float(h[e]);
      }
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mu = s / (float)C;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int idx = lane + 32 * k;
      if (idx < nvec) {
        const __half* h = reinterpret_cast<const __half*>(&v[k]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = __half2float(h[e]) - mu;
          ss += d * d;
        }
      }
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)C + eps);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * C);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int idx = lane + 32 * k;
      if (idx < nvec) {
        uint4 o4;
        __half* ho = reinterpret_cast<__half*>(&o4);
        const __half* h = reinterpret_cast<const __half*>(&v[k]);
        const float4 g0 = reinterpret_cast<const float4*>(gamma)[2 * idx], g1 = reinterpret_cast<const float4*>(gamma)[2 * idx + 1];
        const float4 b0 = reinterpret_cast<const float4*>(beta)[2 * idx], b1 = reinterpret_cast<const float4*>(beta)[2 * idx + 1];
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) ho[e] = __float2half((__half2float(h[e]) - mu) * rstd * gg[e] + bb[e]);
        dst[idx] = o4;
      }
    }
  }
}
// Generic fallback (any C, any alignment): one block per row, two reads.
__global__ void layernorm_rows_generic_kernel(__half* __restrict__ out, const __half* __restrict__ in,
                                              const float* __restrict__ gamma, const float* __restrict__ beta, int rows,
                                              int C, float eps) {
  __shared__ float red[32];
  __shared__ float s_bc;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __half* x = in + (size_t)r * C;
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) s += __half2float(x[i]);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
      s_bc = t / (float)C;
    }
    __syncthreads();
    const float mu = s_bc;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
      const float d = __half2float(x[i]) - mu;
      ss += d * d;
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
      s_bc = rsqrtf(t / (float)C + eps);
    }
    __syncthreads();
    const float rstd = s_bc;
    for (int i = threadIdx.x; i < C; i += blockDim.x)
      out[(size_t)r * C + i] = __float2half((__half2float(x[i]) - mu) * rstd * gamma[i] + beta[i]);
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------
// Spatial attention, reference mode.  Kernel 1: one thread per (position, attention channel) runs
// the three sequential fp16-fma chains.  Kernel 2: one block of `group` threads per softmax group,
// one thread per position: score, per-warp max, per-block tree sum, output.
__global__ void sa_project_kernel(const __half* __restrict__ in, const __half* __restrict__ kW,
                                  const __half* __restrict__ qW, const __half* __restrict__ vW, __half* __restrict__ kMap,
                                  __half* __restrict__ qMap, __half* __restrict__ vMap, int P, int inC, int attC) {
  const long long total = (long long)P * attC;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(t / attC), a = (int)(t % attC);
    const __half* x = in + (size_t)p * inC;
    const __half* wk = kW + (size_t)a * inC;
    const __half* wq = qW + (size_t)a * inC;
    const __half* wv = vW + (size_t)a * inC;
    __half ks = __float2half(0.0f), qs = ks, vs = ks;
    for (int c = 0; c < inC; ++c) {
      const __half xv = x[c];
      ks = __hfma(xv, wk[c], ks);
      qs = __hfma(xv, wq[c], qs);
      vs = __hfma(xv, wv[c], vs);
    }
    kMap[t] = ks;
    qMap[t] = qs;
    vMap[t] = vs;
  }
}
__global__ void sa_softmax_apply_kernel(const __half* __restrict__ in, const __half* __restrict__ kMap,
                                        const __half* __restrict__ qMap, const __half* __restrict__ vMap,
                                        __half* __restrict__ scores, __half* __restrict__ out, int P, int inC, int attC,
                                        float scale) {
  extern __shared__ float sh[];
  const int p = blockIdx.x * blockDim.x + threadIdx.x;  // P is a multiple of blockDim.x
  float score = 0.0f;
  for (int a = 0; a < attC; ++a) score += __half2float(qMap[(size_t)p * attC + a]) * __half2float(kMap[(size_t)p * attC + a]);
  score *= scale;
  float mx = score;
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float e = expf(score - mx);
  sh[threadIdx.x] = e;
  __syncthreads();
  for (int stride = blockDim.x / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) sh[threadIdx.x] += sh[threadIdx.x + stride];
    __syncthreads();
  }
  const float sum = sh[0];
  const __half ah = __float2half(sum > 0 ? e / sum : 0.0f);
  scores[p] = ah;
  const __half one = __float2half(1.0f);
  for (int a = 0; a < attC; ++a) {
    const __half wv = __hmul(ah, vMap[(size_t)p * attC + a]);
    out[(size_t)p * attC + a] = __hfma(one, in[(size_t)p * inC + a % inC], wv);
  }
}

// Mask mode on channels-last data: one warp per pixel.
__global__ void spatial_mask_kernel(const __half* __restrict__ x, const __half* __restrict__ w1, float b1,
                                    __half* __restrict__ y, long long pixels, int C) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long p = warp; p < pixels; p += nwarps) {
    const __half* px = x + p * C;
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += __half2float(px[c]) * __half2float(w1[c]);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float m = 1.0f / (1.0f + expf(-(s + b1)));
    for (int c = lane; c < C; c += 32) y[p * C + c] = __float2half(__half2float(px[c]) * m);
  }
}

__global__ void global_avgpool_nhwc_kernel(const __half* __restrict__ x, __half* __restrict__ y, int batch, int hw, int C) {
  const long long total = (long long)batch * C;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(t / C), c = (int)(t % C);
    const __half* p = x + (size_t)b * hw * C + c;
    float s = 0.f;
    for (int i = 0; i < hw; ++i) s += __half2float(p[(size_t)i * C]);
    y[t] = __float2half(s / (float)hw);
  }
}

// block per (b, cell): 512 threads = (C/8 channel vectors, 16 bytes each) x position groups; every thread sums a
// strided subset of the cell's D x h x w positions, then a fixed-order tree over the groups (deterministic)
__global__ void __launch_bounds__(512) adaptive_avgpool3d_vec_kernel(const __half* __restrict__ x, __half* __restrict__ y, int batch, int D, int H, int W, int C,
                                                                     int ph, int pw) {
  __shared__ float s_part[512 * 8];
  const int cell = blockIdx.x % (ph * pw), b = blockIdx.x / (ph * pw);
  const int oh = cell / pw, ow = cell % pw;
  const int h0 = (oh * H) / ph, h1 = ((oh + 1) * H + ph - 1) / ph;
  const int w0 = (ow * W) / pw, w1 = ((ow + 1) * W + pw - 1) / pw;
  const int cw = w1 - w0, chh = h1 - h0, npos = D * chh * cw;
  const int cv = C / 8, groups = 512 / cv;            // C/8 divides 512
  const int v = threadIdx.x % cv, g = threadIdx.x / cv;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (g < groups) {
    for (int pos = g; pos < npos; pos += groups) {
      const int iw = w0 + pos % cw, t = pos / cw, ih = h0 + t % chh, d = t / chh;
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(x + ((((size_t)b * D + d) * H + ih) * W + iw) * C) + v);
      const __half2* hq = reinterpret_cast<const __half2*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(hq[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_part[threadIdx.x * 8 + e] = acc[e];
  __syncthreads();
  for (int half = groups / 2; half >= 1; half /= 2) {
    if (g < half) {
#pragma unroll
      for (int e = 0; e < 8; ++e) s_part[threadIdx.x * 8 + e] += s_part[(threadIdx.x + half * cv) * 8 + e];
    }
    __syncthreads();
  }
  if (g == 0) {
    const float inv = 1.0f / (float)npos;
#pragma unroll
    for (int e = 0; e < 8; ++e) y[((size_t)b * C + v * 8 + e) * ph * pw + cell] = __float2half(s_part[threadIdx.x * 8 + e] * inv);
  }
}

__global__ void adaptive_avgpool3d_kernel(const __half* __restrict__ x, __half* __restrict__ y, int batch, int D, int H,
                                          int W, int C, int ph, int pw) {
  // block per (b, cell); threads over channels; output order [b][c][ph][pw]
  const int cell = blockIdx.x % (ph * pw), b = blockIdx.x / (ph * pw);
  const int oh = cell / pw, ow = cell % pw;
  const int h0 = (oh * H) / ph, h1 = ((oh + 1) * H + ph - 1) / ph;
  const int w0 = (ow * W) / pw, w1 = ((ow + 1) * W + pw - 1) / pw;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float s = 0.f;
    for (int d = 0; d < D; ++d)
      for (int ih = h0; ih < h1; ++ih) {
        float rs = 0.f;
        for (int iw = w0; iw < w1; ++iw) rs += __half2float(x[((((size_t)b * D + d) * H + ih) * W + iw) * C + c]);
        s += rs;
      }
    y[((size_t)b * C + c) * ph * pw + cell] = __float2half(s / (float)(D * (h1 - h0) * (w1 - w0)));
  }
}

// FC head for a handful of rows in one launch: y = half(half(x . W) + b) (the two roundings of FCLayer.cpp:50-51),
// sigmoid on the first n_sig outputs and tanh on the rest (Sigmoid.cpp:8-12 and the tanh tail), fp16 and fp32
// results (ConvertHalfToFloat).  One block per row, one warp per output, fp32 accumulation in a fixed order.
__global__ void fc_head_kernel(const __half* __restrict__ x, const __half* __restrict__ w_in_out, const __half* __restrict__ bias,
                               __half* __restrict__ out_h, float* __restrict__ out_f, int in_c, int n_out, int n_sig) {
  extern __shared__ float fch_x[];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < in_c; i += blockDim.x) fch_x[i] = __half2float(x[(size_t)row * in_c + i]);
  __syncthreads();
  for (int o = warp; o < n_out; o += nwarps) {
    float acc = 0.f;
    for (int k = lane; k < in_c; k += 32) acc = fmaf(fch_x[k], __half2float(w_in_out[(size_t)k * n_out + o]), acc);
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) {
      float v = __half2float(__float2half(acc));
      v = __half2float(__float2half(v + (bias ? __half2float(bias[o]) : 0.f)));
      const float a = o < n_sig ? 1.0f / (1.0f + expf(-v)) : tanhf(v);
      const __half h = __float2half(a);
      out_h[(size_t)row * n_out + o] = h;
      if (out_f) out_f[(size_t)row * n_out + o] = __half2float(h);
    }
  }
}

// Fused output head of the frame encoder, one CTA per frame: mask attention (x . w1 + b1 -> sigmoid ->
// x*m), global average pool, FC with the reference's two roundings (FCLayer.cpp:50-51), sigmoid on the
// first n_sig outputs / tanh on the rest (Sigmoid.cpp:8-12), fp16 and fp32 results.  Same arithmetic
// and rounding points as the stand-alone kernels above; x is read once from HBM.
__global__ void cnn_head_kernel(const __half* __restrict__ x, const __half* __restrict__ w1, float b1,
                                const __half* __restrict__ fcw, const __half* __restrict__ fcb, __half* __restrict__ feat,
                                __half* __restrict__ out_h, float* __restrict__ out_f, int HW, int C, int n_out, int n_sig) {
  extern __shared__ uint8_t head_smem[];
  __half* sx = reinterpret_cast<__half*>(head_smem);                 // [HW][C]
  float* s_mask = reinterpret_cast<float*>(sx + (size_t)HW * C);     // [HW]
  float* s_pool = s_mask + HW;                                       // [C]
  const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const __half* xb = x + (size_t)b * HW * C;
  const int nvec = HW * C / 8;
  for (int i = tid; i < nvec; i += blockDim.x) reinterpret_cast<uint4*>(sx)[i] = reinterpret_cast<const uint4*>(xb)[i];
  __syncthreads();
  for (int p = warp; p < HW; p += nwarps) {
    float s = 0.f;
    for (int c = lane; c < C; c += 32) s += __half2float(sx[p * C + c]) * __half2float(w1[c]);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) s_mask[p] = 1.0f / (1.0f + expf(-(s + b1)));
  }
  __syncthreads();
  for (int c = tid; c < C; c += blockDim.x) {
    float s = 0.f;
    for (int p = 0; p < HW; ++p) s += __half2float(__float2half(__half2float(sx[p * C + c]) * s_mask[p]));
    const __half h = __float2half(s / (float)HW);
    feat[(size_t)b * C + c] = h;
    s_pool[c] = __half2float(h);
  }
  __syncthreads();
  for (int o = warp; o < n_out; o += nwarps) {
    float acc = 0.f;
    for (int c = lane; c < C; c += 32) acc = fmaf(s_pool[c], __half2float(fcw[(size_t)c * n_out + o]), acc);
    for (int k = 16; k > 0; k >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, k);
    if (lane == 0) {
      const float t = __half2float(__float2half(acc));
      const float y = __half2float(__float2half(t + (fcb ? __half2float(fcb[o]) : 0.f)));
      const __half v = o < n_sig ? __float2half(1.0f / (1.0f + expf(-y))) : __float2half(tanhf(y));
      out_h[(size_t)b * n_out + o] = v;
      out_f[(size_t)b * n_out + o] = __half2float(v);
    }
  }
}

}  // namespace

// ============================================================================================
extern "C" {

#define AIG_ENTER(ctx)                         \
  if (!(ctx)) return AIG_ERR_INVALID;          \
  DeviceGuard guard__((ctx)->device)

int aig_bgra_to_planar(aig_ctx* ctx, const uint8_t* src, uint8_t* dst, int n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, src && dst && n >= 0, "aig_bgra_to_planar: bad arguments");
  if (n == 0) return AIG_OK;
  bgra_to_planar_kernel<<<grid_for(ctx, n / 4 + 1), kThreads, 0, ctx->stream>>>(src, dst, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_convert_normalize(aig_ctx* ctx, aig_half* out, const uint8_t* in, size_t n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, out && in, "aig_convert_normalize: null pointer");
  if (n == 0) return AIG_OK;
  convert_normalize_kernel<<<grid_for(ctx, (long long)(n / 16 + 1)), kThreads, 0, ctx->stream>>>((__half*)out, in, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_preprocess_bgra(aig_ctx* ctx, const uint8_t* bgra, aig_half* out_nchw, int frames, int hw) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, bgra && out_nchw && frames >= 0 && hw >= 0, "aig_preprocess_bgra: bad arguments");
  if (frames == 0 || hw == 0) return AIG_OK;
  preprocess_bgra_kernel<<<grid_for(ctx, (long long)frames * hw / 4 + 1), kThreads, 0, ctx->stream>>>(
      bgra, (__half*)out_nchw, frames, hw);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_unconvert_unnormalize(aig_ctx* ctx, uint8_t* out, const aig_half* in, size_t n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, out && in, "aig_unconvert_unnormalize: null pointer");
  if (n == 0) return AIG_OK;
  unconvert_kernel<<<grid_for(ctx, (long long)n), kThreads, 0, ctx->stream>>>(out, (const __half*)in, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_resize_box(aig_ctx* ctx, const uint8_t* src, int src_is_bgra, uint8_t* out_u8, aig_half* out_half, int frames, int channels, int h,
                   int w, int k, int cross_channel_sum) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, src && (out_u8 || out_half) && frames >= 0 && channels > 0 && h > 0 && w > 0 && k > 0 && k <= h && k <= w,
              "aig_resize_box: bad arguments");
  AIG_REQUIRE(ctx, !src_is_bgra || channels == 3, "aig_resize_box: BGRA frames have three colour channels");
  const long long total = (long long)frames * channels * (h / k) * (w / k);
  if (total == 0) return AIG_OK;
  if (src_is_bgra)
    resize_box_kernel<true><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(src, out_u8, (__half*)out_half, frames, channels, h, w, k, cross_channel_sum);
  else
    resize_box_kernel<false><<<grid_for(ctx, total), kThreads, 0, ctx->stream>>>(src, out_u8, (__half*)out_half, frames, channels, h, w, k, cross_channel_sum);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_half_to_float(aig_ctx* ctx, const aig_half* src, float* dst, size_t n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, src && dst, "aig_half_to_float: null pointer");
  if (n == 0) return AIG_OK;
  half_to_float_kernel<<<grid_for(ctx, (long long)n), kThreads, 0, ctx->stream>>>((const __half*)src, dst, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_float_to_half(aig_ctx* ctx, const float* src, aig_half* dst, size_t n) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, src && dst, "aig_float_to_half: null pointer");
  if (n == 0) return AIG_OK;
  float_to_half_kernel<<<grid_for(ctx, (long long)n), kThreads, 0, ctx->stream>>>(src, (__half*)dst, n);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

static int launch_transpose(aig_ctx* ctx, const aig_half* src, aig_half* dst, int batch, int rows, int cols) {
  if (batch == 0 || rows == 0 || cols == 0) return AIG_OK;
  AIG_REQUIRE(ctx, batch <= 65535 && ceil_div(rows, 32) <= 65535, "transpose: extent too large");
  dim3 grid(ceil_div(cols, 32), ceil_div(rows, 32), batch), block(32, 8);
  transpose_kernel<<<grid, block, 0, ctx->stream>>>((const __half*)src, (__half*)dst, rows, cols);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_nchw_to_nhwc(aig_ctx* ctx, const aig_half* src, aig_half* dst, int batch, int c, int hw) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, src && dst && batch >= 0 && c >= 0 && hw >= 0, "aig_nchw_to_nhwc: bad arguments");
  return launch_transpose(ctx, src, dst, batch, c, hw);
}
int aig_nhwc_to_nchw(aig_ctx* ctx, const aig_half* src, aig_half* dst, int batch, int c, int hw) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, src && dst && batch >= 0 && c >= 0 && hw >= 0, "aig_nhwc_to_nchw: bad arguments");
  return launch_transpose(ctx, src, dst, batch, hw, c);
}

int aig_leaky_relu_forward(aig_ctx* ctx, aig_half* data, int size, float negative_slope) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, data && size >= 0, "aig_leaky_relu_forward: bad arguments");
  if (size == 0) return AIG_OK;
  OpLeaky op{__float2half(negative_slope)};
  unary_inplace_kernel<<<grid_for(ctx, size / 8 + 1), kThreads, 0, ctx->stream>>>((__half*)data, (size_t)size, op);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_swish_forward(aig_ctx* ctx, aig_half* data, int size) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, data && size >= 0, "aig_swish_forward: bad arguments");
  if (size == 0) return AIG_OK;
  unary_inplace_kernel<<<grid_for(ctx, size / 8 + 1), kThreads, 0, ctx->stream>>>((__half*)data, (size_t)size, OpSwish());
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_relu_forward(aig_ctx* ctx, aig_half* data, int size) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, data && size >= 0, "aig_relu_forward: bad arguments");
  if (size == 0) return AIG_OK;
  unary_inplace_kernel<<<grid_for(ctx, size / 8 + 1), kThreads, 0, ctx->stream>>>((__half*)data, (size_t)size, OpRelu());
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_sigmoid_forward(aig_ctx* ctx, aig_half* data, int num_ctrls, int num_buts, int size) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, data && size >= 0 && num_ctrls > 0, "aig_sigmoid_forward: bad arguments");
  if (size == 0) return AIG_OK;
  sigmoid_head_kernel<<<grid_for(ctx, size), kThreads, 0, ctx->stream>>>((__half*)data, num_ctrls, num_buts, size, 0);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_tanh_tail_forward(aig_ctx* ctx, aig_half* data, int num_ctrls, int num_buts, int size) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, data && size >= 0 && num_ctrls > 0, "aig_tanh_tail_forward: bad arguments");
  if (size == 0) return AIG_OK;
  sigmoid_head_kernel<<<grid_for(ctx, size), kThreads, 0, ctx->stream>>>((__half*)data, num_ctrls, num_buts, size, 1);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_add_forward(aig_ctx* ctx, aig_half* m, const aig_half* r, int size) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, m && r && size >= 0, "aig_add_forward: bad arguments");
  if (size == 0) return AIG_OK;
  add_kernel<<<grid_for(ctx, size / 8 + 1), kThreads, 0, ctx->stream>>>((__half*)m, (const __half*)r, (size_t)size);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}
int aig_batchnorm_forward(aig_ctx* ctx, const aig_half* x, aig_half* y, const float* gamma, const float* beta,
                          const float* mean, const float* var, int batch, int c, int hw, float eps, int per_activation) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, x && y && gamma && beta && mean && var && batch >= 0 && c > 0 && hw > 0, "aig_batchnorm_forward: bad arguments");
  const size_t total = (size_t)batch * c * hw;
  if (total == 0) return AIG_OK;
  batchnorm_kernel<<<grid_for(ctx, (long long)total), kThreads, 0, ctx->stream>>>(
      (const __half*)x, (__half*)y, gamma, beta, mean, var, total, c, hw, eps, per_activation);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_layernorm_forward(aig_ctx* ctx, aig_half* out, const aig_half* in, const float* gamma, const float* beta,
                          float* mean, float* variance, int n, int c, int hw, float eps) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, out && in && gamma && beta && mean && variance && n > 0 && c > 0 && hw > 0, "aig_layernorm_forward: bad arguments");
  const int threads = hw >= 256 ? 256 : (hw >= 64 ? 64 : 32);
  const int blocks = c < ctx->sm_count * 8 ? c : ctx->sm_count * 8;
  layernorm_channel_kernel<<<blocks, threads, 0, ctx->stream>>>((__half*)out, (const __half*)in, gamma, beta, mean,
                                                                variance, n, c, hw, eps);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_layernorm_rows_forward(aig_ctx* ctx, aig_half* out, const aig_half* in, const float* gamma, const float* beta,
                               int rows, int c, float eps) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, out && in && gamma && beta && rows >= 0 && c > 0, "aig_layernorm_rows_forward: bad arguments");
  if (rows == 0) return AIG_OK;
  const bool vec_ok = (c % 8 == 0) && c <= 32 * 8 * 8 && ((uintptr_t)in % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                      ((uintptr_t)gamma % 16 == 0) && ((uintptr_t)beta % 16 == 0);
  if (vec_ok) {
    const int vpl = ceil_div(c / 8, 32);
    const int blocks = grid_for(ctx, (long long)rows * 32, kThreads, 16);
    __half* o = (__half*)out;
    const __half* i = (const __half*)in;
    if (vpl <= 1) layernorm_rows_kernel<1><<<blocks, kThreads, 0, ctx->stream>>>(o, i, gamma, beta, rows, c, eps);
    else if (vpl <= 2) layernorm_rows_kernel<2><<<blocks, kThreads, 0, ctx->stream>>>(o, i, gamma, beta, rows, c, eps);
    else if (vpl <= 4) layernorm_rows_kernel<4><<<blocks, kThreads, 0, ctx->stream>>>(o, i, gamma, beta, rows, c, eps);
    else layernorm_rows_kernel<8><<<blocks, kThreads, 0, ctx->stream>>>(o, i, gamma, beta, rows, c, eps);
  } else {
    const int blocks = rows < ctx->sm_count * 8 ? rows : ctx->sm_count * 8;
    layernorm_rows_generic_kernel<<<blocks, kThreads, 0, ctx->stream>>>((__half*)out, (const __half*)in, gamma, beta, rows, c, eps);
  }
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_spatial_attention_forward(aig_ctx* ctx, const aig_half* in, const aig_half* key_w, const aig_half* query_w,
                                  const aig_half* value_w, aig_half* key_map, aig_half* query_map, aig_half* value_map,
                                  aig_half* attention_scores, aig_half* out, int batch, int in_c, int att_c, int in_h,
                                  int in_w, int group) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, in && key_w && query_w && value_w && key_map && query_map && value_map && attention_scores && out,
              "aig_spatial_attention_forward: null pointer");
  AIG_REQUIRE(ctx, batch > 0 && in_c > 0 && att_c > 0 && in_h > 0 && in_w > 0, "aig_spatial_attention_forward: bad extents");
  AIG_REQUIRE(ctx, group >= 32 && group <= 1024 && (group & (group - 1)) == 0,
              "aig_spatial_attention_forward: group must be a power of two in [32,1024]");
  const int P = batch * in_h * in_w;
  AIG_REQUIRE(ctx, P % group == 0, "aig_spatial_attention_forward: batch*h*w (%d) must be a multiple of group (%d)", P, group);
  sa_project_kernel<<<grid_for(ctx, (long long)P * att_c), kThreads, 0, ctx->stream>>>(
      (const __half*)in, (const __half*)key_w, (const __half*)query_w, (const __half*)value_w, (__half*)key_map,
      (__half*)query_map, (__half*)value_map, P, in_c, att_c);
  AIG_LAUNCH_OK(ctx);
  sa_softmax_apply_kernel<<<P / group, group, group * sizeof(float), ctx->stream>>>(
      (const __half*)in, (const __half*)key_map, (const __half*)query_map, (const __half*)value_map,
      (__half*)attention_scores, (__half*)out, P, in_c, att_c, 1.0f / sqrtf((float)in_c));
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_spatial_mask_forward(aig_ctx* ctx, const aig_half* x_nhwc, const aig_half* w1, float b1, aig_half* y_nhwc,
                             int batch, int hw, int c) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, x_nhwc && w1 && y_nhwc && batch >= 0 && hw >= 0 && c > 0, "aig_spatial_mask_forward: bad arguments");
  const long long pixels = (long long)batch * hw;
  if (pixels == 0) return AIG_OK;
  spatial_mask_kernel<<<grid_for(ctx, pixels * 32, kThreads, 16), kThreads, 0, ctx->stream>>>(
      (const __half*)x_nhwc, (const __half*)w1, b1, (__half*)y_nhwc, pixels, c);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_global_avgpool_nhwc(aig_ctx* ctx, const aig_half* x_nhwc, aig_half* y, int batch, int hw, int c) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, x_nhwc && y && batch >= 0 && hw > 0 && c > 0, "aig_global_avgpool_nhwc: bad arguments");
  if (batch == 0) return AIG_OK;
  global_avgpool_nhwc_kernel<<<grid_for(ctx, (long long)batch * c), kThreads, 0, ctx->stream>>>(
      (const __half*)x_nhwc, (__half*)y, batch, hw, c);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_cnn_head_forward(aig_ctx* ctx, const aig_half* x_nhwc, const aig_half* mask_w, float mask_b, const aig_half* fc_w,
                         const aig_half* fc_b, aig_half* feat, aig_half* out_half, float* out_f32, int batch, int hw, int c,
                         int n_out, int n_sigmoid) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, x_nhwc && mask_w && fc_w && feat && out_half && out_f32, "aig_cnn_head_forward: null pointer");
  AIG_REQUIRE(ctx, batch >= 0 && hw > 0 && c > 0 && n_out > 0 && n_sigmoid >= 0 && n_sigmoid <= n_out && (hw * c) % 8 == 0,
              "aig_cnn_head_forward: bad extents");
  const size_t smem = (size_t)hw * c * 2 + (size_t)(hw + c) * 4;
  if (smem > 200 * 1024) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "aig_cnn_head_forward: %d x %d feature map does not fit shared memory", hw, c);
  if (batch == 0) return AIG_OK;
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(cnn_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  cnn_head_kernel<<<batch, 256, smem, ctx->stream>>>((const __half*)x_nhwc, (const __half*)mask_w, mask_b, (const __half*)fc_w,
                                                     (const __half*)fc_b, (__half*)feat, (__half*)out_half, out_f32, hw, c, n_out,
                                                     n_sigmoid);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_adaptive_avgpool3d_ndhwc(aig_ctx* ctx, const aig_half* x, aig_half* y, int batch, int d, int h, int w, int c,
                                 int ph, int pw) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, x && y && batch >= 0 && d > 0 && h > 0 && w > 0 && c > 0 && ph > 0 && pw > 0 && ph <= h && pw <= w,
              "aig_adaptive_avgpool3d_ndhwc: bad arguments");
  if (batch == 0) return AIG_OK;
  if (c % 8 == 0 && 512 % (c / 8) == 0 && ((uintptr_t)x & 15) == 0)
    adaptive_avgpool3d_vec_kernel<<<batch * ph * pw, 512, 0, ctx->stream>>>((const __half*)x, (__half*)y, batch, d, h, w, c, ph, pw);
  else
    adaptive_avgpool3d_kernel<<<batch * ph * pw, 128, 0, ctx->stream>>>((const __half*)x, (__half*)y, batch, d, h, w, c, ph, pw);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int aig_fc_head_forward(aig_ctx* ctx, const aig_half* x, const aig_half* w_in_out, const aig_half* bias, aig_half* out_half, float* out_f32,
                        int rows, int in_c, int n_out, int n_sigmoid) {
  AIG_ENTER(ctx);
  AIG_REQUIRE(ctx, x && w_in_out && out_half && rows >= 0 && in_c > 0 && n_out > 0 && n_sigmoid >= 0 && n_sigmoid <= n_out && in_c <= 12288,
              "aig_fc_head_forward: bad arguments");
  if (rows == 0) return AIG_OK;
  fc_head_kernel<<<rows, 256, in_c * sizeof(float), ctx->stream>>>((const __half*)x, (const __half*)w_in_out, (const __half*)bias, (__half*)out_half,
                                                                    out_f32, in_c, n_out, n_sigmoid);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

}  // extern "C"
