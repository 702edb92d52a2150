// conv_first_tc.cu -- first-layer (3 input channels) convolution on the tensor cores.
//
// K = 3*kd*k*k (75 for the 5x5 frame encoder, 81 for the 3x3x3 clip encoder) is too ragged for TMA
// boxes, so the im2col rows are gathered by 128 producer threads: each builds one output pixel's row
// (all taps x 3 channels, converted from BGRA bytes with the reference's /255 arithmetic or read from
// planar fp16) in registers and writes it as 16-byte chunks in the 128-byte-swizzled K-major layout
// tcgen05.mma expects.  K is padded to 128 (two 64-element blocks); the padding stays zero.
// The whole weight matrix (out_c x 128) sits in shared memory for the life of the CTA.
// Warps: 0..3 producers, 4..7 epilogue (TMEM lane quarters 0..3), 8 = MMA issuer + TMEM owner.
// A tiles and TMEM accumulators are double buffered; every wait is bounded.
#include "aig_common.cuh"
#include "conv_first_tc.h"

namespace {

constexpr int kThreads = 288;
constexpr int kRows = 128;
constexpr int kABytes = 2 * kRows * 128;  // two K blocks of 128 rows x 128 B

struct TcParams {
  ConvFirstGeom g;
  long long total_px;
  int tiles;
  int NT;
  const float* scale;
  const float* shift;
  int* gerr;
  int pair;         // planar fp16 input, k3 s2 p1, even width: the gather loads column pairs (see the producers)
  int s2d, Hb, Wb;  // s2d: store into the 2x2 space-to-depth layout [n][Hb][Wb][4][K] read by a fused down-sampling block
};

__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

template <int KD, int KHW, bool BGRA>
__global__ void __launch_bounds__(kThreads, 2)
conv_first_tc_kernel(const void* __restrict__ xin, __half* __restrict__ y, const uint4* __restrict__ wimg, const TcParams p) {
  constexpr int TAPS = KD * KHW * KHW;
  constexpr int KTOT = 3 * TAPS;
  constexpr int NCH = (KTOT + 7) / 8;     // 16-byte chunks per row that carry data
  constexpr int KSTEPS = (KTOT + 15) / 16;
  static_assert(KTOT <= 128, "filter too large for the single-tile K");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  uint8_t* sA = sm;                                   // 2 stages x kABytes
  uint8_t* sB = sA + 2 * kABytes;                     // 2 K blocks x NT rows x 128 B
  float* s_scale = reinterpret_cast<float*>(sB + 2 * p.NT * 128);
  float* s_shift = s_scale + 256;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_shift + 256);
  const uint32_t bar_afull = smem_u32(bars), bar_aempty = bar_afull + 16, bar_tfull = bar_afull + 32, bar_tempty = bar_afull + 48;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // (uniform for the compiler)
  const ConvFirstGeom& g = p.g;

  // one-time staging: zero both A stages (the K padding is never written again), weights, scale/shift
  for (int i = threadIdx.x; i < 2 * kABytes / 16; i += kThreads) reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < 2 * p.NT * 128 / 16; i += kThreads) reinterpret_cast<uint4*>(sB)[i] = wimg[i];
  for (int i = threadIdx.x; i < p.NT; i += kThreads) {
    s_scale[i] = p.scale[i];
    s_shift[i] = p.shift[i];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_afull + 8 * s, kRows);
      mbar_init(bar_aempty + 8 * s, 1);
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 4);
    }
    *s_abort = 0;
    fence_mbar_init();
  }
  const uint32_t tmem_cols = 2 * p.NT <= 32 ? 32 : (2 * p.NT <= 64 ? 64 : (2 * p.NT <= 128 ? 128 : (2 * p.NT <= 256 ? 256 : 512)));
  if (warp == 8) {
    tmem_alloc(smem_u32(s_tmem), tmem_cols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp < 4) {
    // ------------------------------------------------------------------ producers: one im2col row each
    const int r = threadIdx.x;
    int it = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
      const int st = it & 1;
      const uint32_t ph = (uint32_t)(it >> 1) & 1u;
      const long long px = (long long)tile * kRows + r;
      const bool valid = px < p.total_px;
      int ow = 0, oh = 0, od = 0, n = 0;
      if (valid) {
        if (p.total_px < (1ll << 31)) {  // 32-bit index arithmetic where it suffices
          const uint32_t t = (uint32_t)px;
          const uint32_t t1 = t / (uint32_t)g.Wo;
          ow = (int)(t - t1 * (uint32_t)g.Wo);
          const uint32_t t2 = t1 / (uint32_t)g.Ho;
          oh = (int)(t1 - t2 * (uint32_t)g.Ho);
          const uint32_t t3 = t2 / (uint32_t)g.Do;
          od = (int)(t2 - t3 * (uint32_t)g.Do);
          n = (int)t3;
        } else {
          long long t = px;
          ow = (int)(t % g.Wo); t /= g.Wo;
          oh = (int)(t % g.Ho); t /= g.Ho;
          od = (int)(t % g.Do); n = (int)(t / g.Do);
        }
      }
      const int iw0 = ow * g.s - g.pad, ih0 = oh * g.s - g.pad, id0 = od * g.sd - g.pd;
      __align__(16) __half hv[NCH * 8];
#pragma unroll
      for (int i = KTOT; i < NCH * 8; ++i) hv[i] = __ushort_as_half((unsigned short)0);
      if (!BGRA && KHW == 3 && p.pair) {
        // k3 s2 p1 over an even width: the taps at columns 2*ow and 2*ow + 1 are one aligned 4-byte load, and the tap
        // at 2*ow - 1 is the neighbouring output pixel's second half (one lane down), fetched by a shuffle; lane 0
        // and the first pixel of a row load it themselves.  27 loads in flight per pixel instead of 81: the gather
        // is bound by the latency of its loads and by the registers that hold them.
        const __half* src = reinterpret_cast<const __half*>(xin);
        const size_t plane = (size_t)g.D * g.H * g.W;
        const bool own_left = lane == 0 || ow == 0;
#pragma unroll
        for (int fd = 0; fd < KD; ++fd) {
          const int id = id0 + fd;
#pragma unroll
          for (int fr = 0; fr < 3; ++fr) {
            const int ih = ih0 + fr;
            const bool rok = valid && id >= 0 && id < g.D && ih >= 0 && ih < g.H;
            const size_t off = (((size_t)n * 3) * g.D + id) * g.H * g.W + (size_t)ih * g.W + 2 * ow;
            const int t0 = (fd * 3 + fr) * 3;
#pragma unroll
            for (int c = 0; c < 3; ++c) {
              const uint32_t two = rok ? *reinterpret_cast<const uint32_t*>(src + off + c * plane) : 0u;
              const unsigned short mine = (own_left && rok && ow > 0) ? __half_as_ushort(src[off + c * plane - 1]) : (unsigned short)0;
              const uint32_t below = __shfl_up_sync(0xffffffffu, two, 1);
              hv[t0 * 3 + c] = __ushort_as_half(own_left ? mine : (unsigned short)(below >> 16));
              hv[(t0 + 1) * 3 + c] = __ushort_as_half((unsigned short)(two & 0xFFFFu));
              hv[(t0 + 2) * 3 + c] = __ushort_as_half((unsigned short)(two >> 16));
            }
          }
        }
      } else {
#pragma unroll
      for (int fd = 0; fd < KD; ++fd) {
        const int id = id0 + fd;
#pragma unroll
        for (int fr = 0; fr < KHW; ++fr) {
          const int ih = ih0 + fr;
          const bool rok = valid && id >= 0 && id < g.D && ih >= 0 && ih < g.H;
#pragma unroll
          for (int fs = 0; fs < KHW; ++fs) {
            const int iw = iw0 + fs;
            const bool ok = rok && iw >= 0 && iw < g.W;
            const int t = (fd * KHW + fr) * KHW + fs;
            if (BGRA) {
              // bytes B,G,R,A; channels of the network are R,G,B; half(float(u8)/255) == half(float(u8)*(1/255))
              // for all 256 byte values
              uint32_t pxl = 0;
              if (ok) pxl = reinterpret_cast<const uint32_t*>(xin)[((size_t)n * g.H + ih) * g.W + iw];
              const float k255 = 1.0f / 255.0f;
              hv[t * 3 + 0] = __float2half_rn((float)((pxl >> 16) & 0xFFu) * k255);
              hv[t * 3 + 1] = __float2half_rn((float)((pxl >> 8) & 0xFFu) * k255);
              hv[t * 3 + 2] = __float2half_rn((float)(pxl & 0xFFu) * k255);
            } else {
              const __half* src = reinterpret_cast<const __half*>(xin);
              const size_t plane = (size_t)g.D * g.H * g.W;
              const size_t off = (((size_t)n * 3) * g.D + id) * g.H * g.W + (size_t)ih * g.W + iw;
#pragma unroll
              for (int c = 0; c < 3; ++c) hv[t * 3 + c] = ok ? src[off + c * plane] : __ushort_as_half((unsigned short)0);
            }
          }
        }
      }
      }
      if (!mbar_wait_bounded(bar_aempty + 8 * st, ph ^ 1u, s_abort, p.gerr, 601)) break;
      uint8_t* a = sA + st * kABytes;
#pragma unroll
      for (int j = 0; j < NCH; ++j)
        *reinterpret_cast<uint4*>(a + (j >> 3) * (kRows * 128) + swz(r, j & 7)) = reinterpret_cast<const uint4*>(hv)[j];
      fence_proxy_async_smem();
      mbar_arrive(bar_afull + 8 * st);
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    // (all lanes run the loop with identical values, one elected lane issues: see elect_one)
    {
      const uint32_t idesc = umma_idesc_f16(kRows, p.NT);
      const bool leader = elect_one();
      int it = 0;
      for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
        const int st = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait_bounded(bar_tempty + 8 * st, ph ^ 1u, s_abort, p.gerr, 602)) break;
        if (!mbar_wait_bounded(bar_afull + 8 * st, ph, s_abort, p.gerr, 603)) break;
        tc_fence_after();
        const uint32_t a0 = smem_u32(sA) + st * kABytes, b0 = smem_u32(sB);
#pragma unroll
        for (int i = 0; i < KSTEPS; ++i) {
          const int kb = i >> 2, k = i & 3;
          if (leader) umma_f16_ss(tmem_base + (uint32_t)(st * p.NT), umma_smem_desc(a0 + kb * (kRows * 128) + k * 32, 128),
                      umma_smem_desc(b0 + kb * (p.NT * 128) + k * 32, 128), idesc, i != 0 ? 1u : 0u);
        }
        if (leader) {
          umma_commit(bar_aempty + 8 * st);
          umma_commit(bar_tfull + 8 * st);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 4..7)
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const bool vec_ok = (g.K & 7) == 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
      const int st = it & 1;
      const uint32_t ph = (uint32_t)(it >> 1) & 1u;
      const long long px = (long long)tile * kRows + r;
      const bool valid = px < p.total_px;
      __half* yrow = y + (size_t)px * g.K;
      if (p.s2d && valid) {
        const int ow = (int)(px % g.Wo);
        const long long t = px / g.Wo;
        const int oh = (int)(t % g.Ho), n = (int)(t / g.Ho);
        const int by = (oh + 1) >> 1, bx = (ow + 1) >> 1, sp = ((oh + 1) & 1) * 2 + ((ow + 1) & 1);
        yrow = y + ((((size_t)n * p.Hb + by) * p.Wb + bx) * 4 + sp) * g.K;
      }
      if (!mbar_wait_bounded(bar_tfull + 8 * st, ph, s_abort, p.gerr, 604)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t)(st * p.NT) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < p.NT; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x16(t_addr + c0, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int v8 = 0; v8 < 2; ++v8) {
            const int n0 = c0 + v8 * 8;
            if (n0 >= g.K) break;
            if (vec_ok) {
              uint4 o;
              __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
              for (int e = 0; e < 8; ++e)
                oh[e] = __float2half(act_apply_fast(__uint_as_float(v[v8 * 8 + e]) * s_scale[n0 + e] + s_shift[n0 + e], g.act, g.slope));
              *reinterpret_cast<uint4*>(yrow + n0) = o;
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (n0 + e < g.K)
                  yrow[n0 + e] = __float2half(act_apply_fast(__uint_as_float(v[v8 * 8 + e]) * s_scale[n0 + e] + s_shift[n0 + e], g.act, g.slope));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * st);
    }
  }

  if (*s_abort) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// w [K][3][taps] fp16 -> shared-memory image: 2 K blocks x NT rows x 128 B, 128-byte swizzle, K index = tap*3 + c
__global__ void pack_wimg_kernel(const __half* __restrict__ w, __half* __restrict__ img, int K, int NT, int taps) {
  const int total = 2 * NT * 64;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int kk = i % 128, n = i / 128;  // kk = K index 0..127, n = output channel row
    const int kb = kk >> 6, kl = kk & 63;
    __half v = __ushort_as_half((unsigned short)0);
    if (n < K && kk < 3 * taps) {
      const int tap = kk / 3, c = kk - tap * 3;
      v = w[((size_t)n * 3 + c) * taps + tap];
    }
    const size_t off = (size_t)kb * NT * 128 + (size_t)n * 128 + (((kl >> 3) ^ (n & 7)) << 4) + (kl & 7) * 2;
    *reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(img) + off) = v;
  }
}


// ------------------------------------------------------------------------------------------
// 2-D BGRA frames: the same GEMM with the gather done through a shared-memory patch.  A tile is a
// block of 8 x 16 output pixels; its input patch ((8-1)*s + k rows, (16-1)*s + k columns) is read
// once with coalesced 4-byte loads, each pixel converted once to four halfs (R, G, B, 0), and every
// producer thread then assembles its im2col row from 8-byte shared-memory reads -- no per-tap
// conversion, bounds check or address arithmetic on global memory.  K index = tap*4 + channel (the
// fourth channel's weights are zero), 100 for 5x5, still two 64-element K blocks.
constexpr int kBH = 8, kBW = 16;
constexpr int kPatchMax = 19 * 36;  // pixels: 5x5 taps at stride 2, rows padded to an even length

template <int KHW>
__global__ void __launch_bounds__(kThreads, 2)
conv_first_patch_kernel(const uint32_t* __restrict__ xin, __half* __restrict__ y, const uint4* __restrict__ wimg, const TcParams p) {
  // K order: filter row, then pairs of adjacent taps (two pixels = one 16-byte chunk; an odd last tap is
  // padded with zeros), then channel: k = ((fr*CPR + fs/2)*2 + (fs&1))*4 + c
  constexpr int CPR = (KHW + 1) / 2;      // 16-byte chunks per filter row
  constexpr int NCH = KHW * CPR;
  constexpr int KTOT = NCH * 8;
  constexpr int KSTEPS = (KTOT + 15) / 16;
  static_assert(KTOT <= 128, "filter too large for the single-tile K");
  static_assert((kPatchMax & 1) == 0, "the staging tiles behind the patch must stay 16-byte aligned");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  uint8_t* sA = sm;
  uint8_t* sB = sA + 2 * kABytes;
  float* s_scale = reinterpret_cast<float*>(sB + 2 * p.NT * 128);
  float* s_shift = s_scale + 256;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_shift + 256);
  const uint32_t bar_afull = smem_u32(bars), bar_aempty = bar_afull + 16, bar_tfull = bar_afull + 32, bar_tempty = bar_afull + 48;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  griddep_launch_dependents();  // the first residual-block launch may set itself up under this kernel
  uint2* s_patch = reinterpret_cast<uint2*>(bars + 16);
  uint8_t* s_stage = reinterpret_cast<uint8_t*>(s_patch + kPatchMax);  // 4 x 2 KB, one tile per epilogue warp (16-byte aligned)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // (uniform for the compiler)
  const ConvFirstGeom& g = p.g;
  const int blocks_x = (g.Wo + kBW - 1) / kBW, blocks_y = (g.Ho + kBH - 1) / kBH;
  const int tiles = g.batch * blocks_y * blocks_x;
  // patch rows are an even number of pixels long so that every row starts on a 16-byte boundary
  const int PH = (kBH - 1) * g.s + KHW, PW = ((kBW - 1) * g.s + KHW + 1) & ~1;

  for (int i = threadIdx.x; i < 2 * kABytes / 16; i += kThreads) reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < 2 * p.NT * 128 / 16; i += kThreads) reinterpret_cast<uint4*>(sB)[i] = wimg[i];
  for (int i = threadIdx.x; i < p.NT; i += kThreads) {
    s_scale[i] = p.scale[i];
    s_shift[i] = p.shift[i];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_afull + 8 * s, kRows);
      mbar_init(bar_aempty + 8 * s, 1);
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 4);
    }
    *s_abort = 0;
    fence_mbar_init();
  }
  const uint32_t tmem_cols = 2 * p.NT <= 32 ? 32 : (2 * p.NT <= 64 ? 64 : (2 * p.NT <= 128 ? 128 : (2 * p.NT <= 256 ? 256 : 512)));
  if (warp == 8) {
    tmem_alloc(smem_u32(s_tmem), tmem_cols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp < 4) {
    // ------------------------------------------------------------------ producers
    const int r = threadIdx.x;
    const int oy = r / kBW, ox = r - oy * kBW;
    const int pbase = oy * g.s * PW + ox * g.s;
    int it = 0;
    bool ok = true;
    constexpr int kPix = (kPatchMax + kRows - 1) / kRows;  // patch pixels per producer thread
    uint32_t nxt[kPix];
    // the pixels of a tile's patch this thread converts, loaded one tile ahead so that their latency
    // hides behind the row assembly of the current tile
    // this thread's patch pixels never change place inside the patch: (row, column) once, not per tile
    int ppy[kPix], ppx[kPix];
#pragma unroll
    for (int k = 0; k < kPix; ++k) {
      const int i = r + k * kRows;
      ppy[k] = i < PH * PW ? i / PW : -(1 << 20);  // past the end of the patch: always out of the image
      ppx[k] = i - (i / PW) * PW;
    }
    auto load_patch = [&](int tile) {
      const int bx = tile % blocks_x, t2 = tile / blocks_x;
      const int by = t2 % blocks_y, n = t2 / blocks_y;
      const int ih0 = by * kBH * g.s - g.pad, iw0 = bx * kBW * g.s - g.pad;
      const uint32_t* img = xin + (size_t)n * g.H * g.W;
#pragma unroll
      for (int k = 0; k < kPix; ++k) {
        const int ih = ih0 + ppy[k], iw = iw0 + ppx[k];
        nxt[k] = (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) ? __ldg(img + (size_t)ih * g.W + iw) : 0u;
      }
    };
    if ((int)blockIdx.x < tiles) load_patch(blockIdx.x);
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const int st = it & 1;
      const uint32_t ph = (uint32_t)(it >> 1) & 1u;
      // every producer is done reading the previous tile's patch
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int k = 0; k < kPix; ++k) {
        const int i = r + k * kRows;
        if (i < PH * PW) {
          // bytes B,G,R,A; channels of the network are R,G,B; half(float(u8)/255) == half(float(u8)*(1/255)) for all bytes
          const float k255 = 1.0f / 255.0f;
          const uint32_t pxl = nxt[k];
          const __half2 rg = __floats2half2_rn((float)((pxl >> 16) & 0xFFu) * k255, (float)((pxl >> 8) & 0xFFu) * k255);
          const __half2 b0 = __floats2half2_rn((float)(pxl & 0xFFu) * k255, 0.f);
          s_patch[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&rg), *reinterpret_cast<const uint32_t*>(&b0));
        }
      }
      if (tile + (int)gridDim.x < tiles) load_patch(tile + gridDim.x);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!ok) continue;  // keep arriving at the producers' barrier; the other roles have drained
      if (!mbar_wait_bounded(bar_aempty + 8 * st, ph ^ 1u, s_abort, p.gerr, 611)) { ok = false; continue; }
      uint8_t* a = sA + st * kABytes;
      const bool pair_ok = (g.s & 1) == 0;  // even stride: every tap pair of this pixel starts on a 16-byte boundary
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int fr = j / CPR, f0 = 2 * (j % CPR);
        const uint2* src = s_patch + pbase + fr * PW + f0;
        uint4 ch;
        if (f0 + 1 < KHW) {
          if (pair_ok) {
            ch = *reinterpret_cast<const uint4*>(src);
          } else {
            const uint2 lo = src[0], hi = src[1];
            ch = make_uint4(lo.x, lo.y, hi.x, hi.y);
          }
        } else {
          const uint2 lo = src[0];
          ch = make_uint4(lo.x, lo.y, 0u, 0u);
        }
        *reinterpret_cast<uint4*>(a + (j >> 3) * (kRows * 128) + swz(r, j & 7)) = ch;
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_afull + 8 * st);
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    // (all lanes run the loop with identical values, one elected lane issues: see elect_one)
    {
      const uint32_t idesc = umma_idesc_f16(kRows, p.NT);
      const bool leader = elect_one();
      int it = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
        const int st = it & 1;
        const uint32_t ph = (uint32_t)(it >> 1) & 1u;
        if (!mbar_wait_bounded(bar_tempty + 8 * st, ph ^ 1u, s_abort, p.gerr, 612)) break;
        if (!mbar_wait_bounded(bar_afull + 8 * st, ph, s_abort, p.gerr, 613)) break;
        tc_fence_after();
        const uint32_t a0 = smem_u32(sA) + st * kABytes, b0 = smem_u32(sB);
#pragma unroll
        for (int i = 0; i < KSTEPS; ++i) {
          const int kb = i >> 2, k = i & 3;
          if (leader) umma_f16_ss(tmem_base + (uint32_t)(st * p.NT), umma_smem_desc(a0 + kb * (kRows * 128) + k * 32, 128),
                      umma_smem_desc(b0 + kb * (p.NT * 128) + k * 32, 128), idesc, i != 0 ? 1u : 0u);
        }
        if (leader) {
          umma_commit(bar_aempty + 8 * st);
          umma_commit(bar_tfull + 8 * st);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 4..7)
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int oy = r / kBW, ox = r - oy * kBW;
    const bool vec_ok = (g.K & 7) == 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const int st = it & 1;
      const uint32_t ph = (uint32_t)(it >> 1) & 1u;
      const int bx = tile % blocks_x, t2 = tile / blocks_x;
      const int by = t2 % blocks_y, n = t2 / blocks_y;
      const int oh = by * kBH + oy, ow = bx * kBW + ox;
      const bool valid = oh < g.Ho && ow < g.Wo;
      size_t pix = ((size_t)n * g.Ho + oh) * g.Wo + ow;
      if (p.s2d) {
        const int sby = (oh + 1) >> 1, sbx = (ow + 1) >> 1, sp = ((oh + 1) & 1) * 2 + ((ow + 1) & 1);
        pix = (((size_t)n * p.Hb + sby) * p.Wb + sbx) * 4 + sp;
      }
      __half* yrow = y + pix * g.K;
      if (!mbar_wait_bounded(bar_tfull + 8 * st, ph, s_abort, p.gerr, 614)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t)(st * p.NT) + ((uint32_t)(q * 32) << 16);
      if (g.K == 32) {
        // 32 channels = 64 bytes per pixel: the warp's 32 rows pass through a 2 KB staging tile (16-byte
        // chunks XOR-swizzled, conflict free both ways) and leave as 8 pixels x 64 contiguous bytes per
        // store instruction instead of 32 scattered 16-byte pieces
        uint8_t* stg = s_stage + q * 2048;
        const int gr = lane >> 2, gc = lane & 3, own = lane * 64, swzl = (lane >> 1) & 3;
        uint32_t v[32];
        tmem_ld_32x32(t_addr, v);
        __half* yp[4];
        bool vj[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          yp[j] = reinterpret_cast<__half*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(yrow), 8 * j + gr));
          vj[j] = __shfl_sync(0xffffffffu, valid ? 1 : 0, 8 * j + gr) != 0;
        }
        tmem_ld_wait();
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
          const int n0 = v8 * 8;
          const float4 s0 = reinterpret_cast<const float4*>(s_scale + n0)[0], s1 = reinterpret_cast<const float4*>(s_scale + n0)[1];
          const float4 h0 = reinterpret_cast<const float4*>(s_shift + n0)[0], h1 = reinterpret_cast<const float4*>(s_shift + n0)[1];
          const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
          float a[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) a[e] = fmaf(__uint_as_float(v[v8 * 8 + e]), sv[e], hv[e]);
          if (g.act == AIG_ACT_SWISH) {
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = act_apply_fast(a[e], AIG_ACT_SWISH, 0.f);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = act_apply_fast(a[e], g.act, g.slope);
          }
          uint4 o;
          __half2* oh2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) oh2[e2] = __floats2half2_rn(a[2 * e2], a[2 * e2 + 1]);
          *reinterpret_cast<uint4*>(stg + own + ((v8 ^ swzl) << 4)) = o;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = 8 * j + gr;
          const uint4 o = *reinterpret_cast<const uint4*>(stg + row * 64 + ((gc ^ ((row >> 1) & 3)) << 4));
          if (vj[j]) *reinterpret_cast<uint4*>(yp[j] + gc * 8) = o;
        }
        __syncwarp();
      } else
#pragma unroll 1
      for (int c0 = 0; c0 < p.NT; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x16(t_addr + c0, v);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int v8 = 0; v8 < 2; ++v8) {
            const int n0 = c0 + v8 * 8;
            if (n0 >= g.K) break;
            if (vec_ok) {
              const float4 s0 = reinterpret_cast<const float4*>(s_scale + n0)[0], s1 = reinterpret_cast<const float4*>(s_scale + n0)[1];
              const float4 h0 = reinterpret_cast<const float4*>(s_shift + n0)[0], h1 = reinterpret_cast<const float4*>(s_shift + n0)[1];
              const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
              const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
              float a[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) a[e] = fmaf(__uint_as_float(v[v8 * 8 + e]), sv[e], hv[e]);
              if (g.act == AIG_ACT_SWISH) {  // the activation of the frame encoder: no per-element dispatch
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = act_apply_fast(a[e], AIG_ACT_SWISH, 0.f);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = act_apply_fast(a[e], g.act, g.slope);
              }
              uint4 o;
              __half2* oh2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
              for (int e2 = 0; e2 < 4; ++e2) oh2[e2] = __floats2half2_rn(a[2 * e2], a[2 * e2 + 1]);
              *reinterpret_cast<uint4*>(yrow + n0) = o;
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (n0 + e < g.K)
                  yrow[n0 + e] = __float2half(act_apply_fast(__uint_as_float(v[v8 * 8 + e]) * s_scale[n0 + e] + s_shift[n0 + e], g.act, g.slope));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * st);
    }
  }

  if (*s_abort) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// w [K][3][k*k] fp16 -> the same shared-memory image in the patch kernel's K order:
// kk = ((fr*CPR + fs/2)*2 + (fs&1))*4 + c with CPR = (k+1)/2; c = 3 and the pad tap of an odd k stay zero
__global__ void pack_wimg4_kernel(const __half* __restrict__ w, __half* __restrict__ img, int K, int NT, int k) {
  const int total = 2 * NT * 64;
  const int cpr = (k + 1) / 2;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int kk = i % 128, n = i / 128;
    const int kb = kk >> 6, kl = kk & 63;
    __half v = __ushort_as_half((unsigned short)0);
    const int c = kk & 3, half_tap = (kk >> 2) & 1, chunk = kk >> 3;
    const int fr = chunk / cpr, fs = 2 * (chunk % cpr) + half_tap;
    if (n < K && fr < k && fs < k && c < 3) v = w[((size_t)n * 3 + c) * k * k + fr * k + fs];
    const size_t off = (size_t)kb * NT * 128 + (size_t)n * 128 + (((kl >> 3) ^ (n & 7)) << 4) + (kl & 7) * 2;
    *reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(img) + off) = v;
  }
}

template <int KD, int KHW>
int launch_tc(ConvFirstTc* t, const void* x, bool bgra, __half* y);

}  // namespace

struct ConvFirstTc {
  aig_ctx* ctx = nullptr;
  TcParams prm{};
  __half* wimg = nullptr;
  __half* wimg4 = nullptr;   // weight image in the tap*4 + channel K layout of the patch kernel
  bool patch_ok = false;     // 2-D, stride <= 2, k in {2, 3, 5}: BGRA frames go through the patch kernel
  size_t smem = 0, smem_patch = 0;
  int grid = 1, grid_patch = 1;
};

namespace {

template <int KHW>
int launch_patch(ConvFirstTc* t, const void* x, __half* y) {
  aig_ctx* ctx = t->ctx;
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(conv_first_patch_kernel<KHW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t->smem_patch));
  conv_first_patch_kernel<KHW><<<t->grid_patch, kThreads, t->smem_patch, ctx->stream>>>(reinterpret_cast<const uint32_t*>(x), y,
                                                                                        reinterpret_cast<const uint4*>(t->wimg4), t->prm);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

}  // namespace

namespace {

template <int KD, int KHW>
int launch_tc(ConvFirstTc* t, const void* x, bool bgra, __half* y) {
  aig_ctx* ctx = t->ctx;
  if (bgra) {
    AIG_CUDA_OK(ctx, cudaFuncSetAttribute(conv_first_tc_kernel<KD, KHW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t->smem));
    conv_first_tc_kernel<KD, KHW, true><<<t->grid, kThreads, t->smem, ctx->stream>>>(x, y, reinterpret_cast<const uint4*>(t->wimg), t->prm);
  } else {
    AIG_CUDA_OK(ctx, cudaFuncSetAttribute(conv_first_tc_kernel<KD, KHW, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t->smem));
    conv_first_tc_kernel<KD, KHW, false><<<t->grid, kThreads, t->smem, ctx->stream>>>(x, y, reinterpret_cast<const uint4*>(t->wimg), t->prm);
  }
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

}  // namespace

bool conv_first_tc_supported(const ConvFirstGeom& g) {
  const bool geom = (g.kd == 1 && (g.k == 2 || g.k == 3 || g.k == 5)) || (g.kd == 3 && g.k == 3);
  return geom && g.K <= 256;
}

int conv_first_tc_create(aig_ctx* ctx, const ConvFirstGeom& g, const float* scale, const float* shift, ConvFirstTc** out) {
  *out = nullptr;
  ConvFirstTc* t = new ConvFirstTc();
  t->ctx = ctx;
  TcParams& p = t->prm;
  p.g = g;
  p.total_px = (long long)g.batch * g.Do * g.Ho * g.Wo;
  p.pair = g.k == 3 && g.s == 2 && g.pad == 1 && g.W % 2 == 0 && g.Wo == g.W / 2;
  p.tiles = (int)ceil_div_ll(p.total_px, kRows);
  p.NT = ceil_div(g.K, 16) * 16;
  p.scale = scale;
  p.shift = shift;
  p.gerr = ctx->d_err;
  t->smem = (size_t)2 * kABytes + (size_t)2 * p.NT * 128 + 2048 + 256 + 1024;
  // two CTAs per SM: the gather of one hides behind the conversion / epilogue work of the other
  t->grid = p.tiles < 2 * ctx->sm_count ? p.tiles : 2 * ctx->sm_count;
  if (cudaMalloc(&t->wimg, (size_t)2 * p.NT * 128) != cudaSuccess || cudaMalloc(&t->wimg4, (size_t)2 * p.NT * 128) != cudaSuccess) {
    cudaFree(t->wimg);
    delete t;
    return aig_fail(ctx, AIG_ERR_CUDA, "conv0: weight image allocation failed");
  }
  t->patch_ok = g.kd == 1 && g.D == 1 && g.s <= 2 && (g.k == 2 || g.k == 3 || g.k == 5);
  if (t->patch_ok) {
    const long long tiles = (long long)g.batch * ceil_div(g.Ho, kBH) * ceil_div(g.Wo, kBW);
    t->grid_patch = (int)(tiles < 2 * ctx->sm_count ? tiles : 2 * ctx->sm_count);
    t->smem_patch = t->smem + (size_t)kPatchMax * 8 + 4 * 2048;
  }
  *out = t;
  return AIG_OK;
}

void conv_first_tc_destroy(ConvFirstTc* t) {
  if (!t) return;
  cudaFree(t->wimg);
  cudaFree(t->wimg4);
  delete t;
}

int conv_first_tc_set_weights(ConvFirstTc* t, const __half* w) {
  aig_ctx* ctx = t->ctx;
  const int taps = t->prm.g.kd * t->prm.g.k * t->prm.g.k;
  pack_wimg_kernel<<<ceil_div(2 * t->prm.NT * 64, 256), 256, 0, ctx->stream>>>(w, t->wimg, t->prm.g.K, t->prm.NT, taps);
  AIG_LAUNCH_OK(ctx);
  if (t->patch_ok) {
    pack_wimg4_kernel<<<ceil_div(2 * t->prm.NT * 64, 256), 256, 0, ctx->stream>>>(w, t->wimg4, t->prm.g.K, t->prm.NT, t->prm.g.k);
    AIG_LAUNCH_OK(ctx);
  }
  return AIG_OK;
}

int conv_first_tc_set_s2d(ConvFirstTc* t, int enable, int Hb, int Wb) {
  if (enable && t->prm.g.Do != 1) return aig_fail(t->ctx, AIG_ERR_UNSUPPORTED, "conv0: space-to-depth output is for 2-D layers");
  t->prm.s2d = enable ? 1 : 0;
  t->prm.Hb = Hb;
  t->prm.Wb = Wb;
  return AIG_OK;
}

int conv_first_tc_forward(ConvFirstTc* t, const void* x, bool bgra, __half* y) {
  const ConvFirstGeom& g = t->prm.g;
  if (bgra && t->patch_ok) {
    if (g.k == 5) return launch_patch<5>(t, x, y);
    if (g.k == 3) return launch_patch<3>(t, x, y);
    return launch_patch<2>(t, x, y);
  }
  if (g.kd == 1 && g.k == 5) return launch_tc<1, 5>(t, x, bgra, y);
  if (g.kd == 1 && g.k == 3) return launch_tc<1, 3>(t, x, bgra, y);
  if (g.kd == 1 && g.k == 2) return launch_tc<1, 2>(t, x, bgra, y);
  if (g.kd == 3 && g.k == 3) return launch_tc<3, 3>(t, x, bgra, y);
  return aig_fail(t->ctx, AIG_ERR_UNSUPPORTED, "conv0: no tensor-core instantiation for this filter");
}
