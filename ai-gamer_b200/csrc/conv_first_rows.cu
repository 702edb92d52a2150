// conv_first_rows.cu -- first convolution of the frame encoder (3 -> 32 channels, 5x5, stride 2, pad 2) straight
// from uint8 frames, for sm_100a.  Replaces GrabFrameInt8's ARGBtoRGBplanar + ConvertAndNormalize + the first
// ConvLayer (+ BatchNorm + activation) of the reference's frame step (NvDisplayCap.h:70-87, CudaStuff.cu:63-74,
// 150-157, ConvLayer.cpp:74-79) by one launch that reads every frame byte once and writes the activation once.
//
// No im2col is assembled.  Input rows live in shared memory as fp16 pixels (R,G,B,0) = 8 bytes, two pixels per
// 16-byte unit, with one zero unit on either side (the padding).  For a stride-2 filter, output pixel x of an
// output row reads input pixels 2x-2 .. 2x+2 = units x, x+1, x+2 of each of five input rows: consecutive output
// pixels read consecutive units, which is exactly the no-swizzle K-major operand layout of tcgen05.mma (rows 16
// bytes apart, eight-row groups 128 bytes apart).  So the A operand of an MMA is the row buffer itself, addressed
// by the shared-memory descriptor: start = row + 32*h, leading-dimension offset 16 bytes (the next unit), and the
// K = 16 of one instruction covers two units (4 pixels x 4 channels).  One tile = one output row (<= 128 pixels):
// 5 input rows x 2 instructions, K = 160 of which 75 carry weights (the rest multiply zeros).
//
// Warp roles (9 warps, two CTAs per SM): warp 0 issues the MMAs; warps 1-4 are the epilogue (TMEM -> scale/shift
// -> activation -> fp16 -> shared memory -> one TMA store per output row, straight into the space-to-depth block
// layout the next layer reads, or plain channels-last); warps 5-8 load and convert frame bytes into a ring of 16
// row buffers, running up to four tiles ahead.  A CTA walks a contiguous range of (frame, output row) tiles, so
// every input row is read and converted once per CTA (twice at range borders).
// Conversion: half(float(u8) / 255.0f) as the reference computes it; float(u8) * fl(1/255) rounds to the same
// half for all 256 byte values, so the division is a multiplication here.
#include "conv_first_rows.h"

#include "aig_common.cuh"

namespace {

constexpr int kThreads = 9 * 32;
constexpr int kRing = 16;             // input row buffers
constexpr int kLead = 4;              // tiles the loaders may run ahead of completed MMAs
constexpr int kPitch = 130 * 16;      // bytes per row buffer: (256 / 2 + 2) units; also what 128 MMA rows x 3 units span
constexpr int kN = 32;                // output channels
constexpr int kMmas = 10;             // 5 filter rows x 2
constexpr int kOutSlots = 130;
constexpr int kOutBytes = 9216;       // one output staging buffer (130 slots x 64 B, 1024-aligned)
constexpr int kSmemRing = kRing * kPitch;
constexpr int kSmemZero = kPitch + 64;                    // the all-zero row (+ what the last instruction over-reads)
constexpr int kSmemB = kMmas * 2 * kN * 16;               // weights: [mma][chunk][n][8 halves]
constexpr int kOffOut = 0;
constexpr int kOffRing = 2 * kOutBytes;
constexpr int kOffZero = kOffRing + kSmemRing;
constexpr int kOffB = kOffZero + ((kSmemZero + 127) & ~127);
constexpr int kOffBars = kOffB + kSmemB;
constexpr int kSmemBytes = kOffBars + 256 + 1024;

struct RowsParams {
  int batch, H, W, Ho, Wo;
  int tiles;               // batch * Ho
  int s2d, Hb;             // output in space-to-depth blocks; block rows per image
  int planar;              // 1: frames are three uint8 planes R, G, B; 0: BGRA pixels
  float slope;
  float scale[kN], shift[kN];
  const uint8_t* frames;
  const uint4* wimg;       // kSmemB bytes, the shared-memory image of the weights
  int* gerr;
};

__device__ __forceinline__ uint64_t desc_noswizzle(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // start address [0,14), leading-dimension byte offset [16,30), stride-dimension byte offset [32,46) (all >> 4),
  // descriptor version 1 at [46,48), layout type 0 = no swizzle at [61,64)
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void tma_store_5d(const void* desc, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(reinterpret_cast<uint64_t>(desc)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* desc, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(reinterpret_cast<uint64_t>(desc)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// byte `sel` (0..3) of w as half(float(byte) / 255): exact integer -> float through the 2^23 trick, one multiply
__device__ __forceinline__ float byte_norm(uint32_t w, uint32_t selector) {
  const float f = __uint_as_float(__byte_perm(w, 0x4B000000u, selector)) - 8388608.0f;
  return __fmul_rn(f, __uint_as_float(0x3B808081u));  // fl(1/255)
}
// one BGRA pixel -> (R, G, B, 0) halves
__device__ __forceinline__ uint2 pixel_bgra(uint32_t w) {
  const __half2 rg = __floats2half2_rn(byte_norm(w, 0x7542u), byte_norm(w, 0x7541u));
  const __half2 b0 = __floats2half2_rn(byte_norm(w, 0x7540u), 0.f);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&rg), *reinterpret_cast<const uint32_t*>(&b0));
}
__device__ __forceinline__ uint2 pixel_rgb(uint32_t r, uint32_t g, uint32_t b, uint32_t selector) {
  const __half2 rg = __floats2half2_rn(byte_norm(r, selector), byte_norm(g, selector));
  const __half2 b0 = __floats2half2_rn(byte_norm(b, selector), 0.f);
  return make_uint2(*reinterpret_cast<const uint32_t*>(&rg), *reinterpret_cast<const uint32_t*>(&b0));
}

template <int ACT>
__device__ __forceinline__ float act_rows(float v, float slope) {
  if (ACT == AIG_ACT_RELU) return fmaxf(v, 0.f);
  if (ACT == AIG_ACT_SWISH) return swish_sfu(v);
  if (ACT == AIG_ACT_LEAKY) return v < 0.f ? v * slope : v;
  return v;
}

template <int ACT>
__global__ void __launch_bounds__(kThreads, 3)
conv_first_rows_kernel(const __grid_constant__ CUtensorMap tmapY, const __grid_constant__ RowsParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const uint32_t sOut = base + kOffOut, sRing = base + kOffRing, sZero = base + kOffZero, sB = base + kOffB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBars);
  const uint32_t bar_ready = smem_u32(bars);         // [8] input rows of tile i landed (128 loader threads)
  const uint32_t bar_done = bar_ready + 64;          // [8] MMAs of tile i completed (ring slots reusable)
  const uint32_t bar_tfull = bar_ready + 128;        // [4] accumulator ready
  const uint32_t bar_tempty = bar_ready + 160;       // [4] accumulator drained (4 epilogue warps)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // (uniform for the compiler)
  griddep_launch_dependents();  // the next layer's launch may set itself up under this one

  // zero everything the MMAs may read (ring, zero row) and the output staging buffers (their border slots stay zero)
  for (int i = threadIdx.x; i < (kOffB - kOffOut) / 16; i += kThreads) reinterpret_cast<uint4*>(sm + kOffOut)[i] = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < kSmemB / 16; i += kThreads) reinterpret_cast<uint4*>(sm + kOffB)[i] = __ldg(p.wimg + i);
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) {
      mbar_init(bar_ready + 8 * i, 128);
      mbar_init(bar_done + 8 * i, 1);
    }
    for (int a = 0; a < 4; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 4);
    }
    *s_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmapY);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(s_tmem), 128);
    tmem_relinquish();
  }
  fence_proxy_async_smem();  // the zero fill and the weights were written with ordinary stores; the MMAs read through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  // contiguous range of (frame, output row) tiles of this CTA
  const int t_begin = (int)((long long)p.tiles * blockIdx.x / gridDim.x), t_end = (int)((long long)p.tiles * (blockIdx.x + 1) / gridDim.x);

  if (warp == 0) {
    // ------------------------------------------------------------------ MMA issuer
    // (all lanes run the loop with identical values, one elected lane issues: see elect_one)
    {
      constexpr uint32_t idesc = umma_idesc_f16(128, kN);
      const bool leader = elect_one();
      bool ok = true;
      int y = t_begin % p.Ho;
      for (int i = 0; i < t_end - t_begin && ok; ++i) {
        const int acc = i & 3;
        if (!mbar_wait_bounded_sleepy(bar_tempty + 8 * acc, (((uint32_t)i >> 2) & 1u) ^ 1u, s_abort, p.gerr, 811)) { ok = false; break; }
        if (!mbar_wait_bounded_sleepy(bar_ready + 8 * (i & 7), ((uint32_t)i >> 3) & 1u, s_abort, p.gerr, 812)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kN);
#pragma unroll
        for (int r = 0; r < 5; ++r) {
          const int row = 2 * y - 2 + r;
          const uint32_t a_row = (row < 0 || row >= p.H) ? sZero : sRing + (uint32_t)(row & (kRing - 1)) * kPitch;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t adesc = desc_noswizzle(a_row + 32u * h, 16u, 128u);
            const uint64_t bdesc = desc_noswizzle(sB + (uint32_t)((r * 2 + h) * 2 * kN * 16), (uint32_t)(kN * 16), 128u);
            if (leader) umma_f16_ss(d_tmem, adesc, bdesc, idesc, (r | h) != 0 ? 1u : 0u);
          }
        }
        if (leader) {
          umma_commit(bar_tfull + 8 * acc);
          umma_commit(bar_done + 8 * (i & 7));
        }
        if (++y == p.Ho) y = 0;
      }
    }
  } else if (warp <= 4) {
    // ------------------------------------------------------------------ epilogue (warps 1..4)
    const int q = warp & 3;                       // TMEM lane quarter of this warp
    const int x = q * 32 + lane;                  // output pixel = accumulator row
    const int tid_e = threadIdx.x - 32;
    const int slot = x + (p.s2d ? 1 : 0);
    const uint32_t swz = (uint32_t)((slot >> 1) & 3);
    int n = t_begin / p.Ho, y = t_begin - n * p.Ho;
    griddep_wait();                               // the output buffer may still be read by an earlier launch
    for (int i = 0; i < t_end - t_begin; ++i) {
      const int acc = i & 3, buf = i & 1;
      if (tid_e == 0) bulk_wait_read_1();         // the store that last read this staging buffer (two tiles ago) is done with it
      named_bar_sync(1, 128);
      const bool ok = mbar_wait_bounded_sleepy(bar_tfull + 8 * acc, ((uint32_t)i >> 2) & 1u, s_abort, p.gerr, 821);
      if (ok) {
        tc_fence_after();
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t)(acc * kN) + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        if (x < p.Wo) {
          const uint32_t dst = sOut + (uint32_t)buf * kOutBytes + (uint32_t)slot * 64u;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int k = c * 8 + e * 2;
              const float a0 = act_rows<ACT>(fmaf(__uint_as_float(r[k]), p.scale[k], p.shift[k]), p.slope);
              const float a1 = act_rows<ACT>(fmaf(__uint_as_float(r[k + 1]), p.scale[k + 1], p.shift[k + 1]), p.slope);
              oh[e] = __floats2half2_rn(a0, a1);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (((uint32_t)c ^ swz) << 4)), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
          }
        }
        fence_proxy_async_smem();                 // the staged row is read by the TMA store (async proxy)
      }
      named_bar_sync(1, 128);
      if (*s_abort) break;                        // uniform: every thread reads the flag after the same barrier
      if (tid_e == 0) {
        const uint32_t src = sOut + (uint32_t)buf * kOutBytes;
        if (p.s2d) tma_store_5d(&tmapY, src, 0, 0, 0, (y + 1) & 1, n * p.Hb + ((y + 1) >> 1));
        else tma_store_4d(&tmapY, src, 0, 0, y, n);
        bulk_commit();
      }
      if (++y == p.Ho) {
        y = 0;
        ++n;
      }
    }
    if (tid_e == 0) bulk_wait_all();
  } else {
    // ------------------------------------------------------------------ loaders (warps 5..8)
    // Every tile needs the input rows not yet in the ring (two in steady state, three at the top of a frame, five
    // at the start of the CTA's range), cut into 16-byte items; thread t takes items t, t+128, ...
    const int tid_l = threadIdx.x - 5 * 32;
    const size_t frame_bytes = (size_t)p.H * p.W * (p.planar ? 3 : 4);
    const size_t plane = (size_t)p.H * p.W;
    const int segs = p.planar ? p.W / 16 : p.W / 4;   // 16-byte loads per input row (per plane when planar)
    const int rr0 = tid_l / segs, seg0 = tid_l - rr0 * segs;  // this thread's first item of any tile
    auto convert_item = [&](const uint8_t* frame, int row, int seg) {
      uint8_t* dst_row = sm + kOffRing + (size_t)(row & (kRing - 1)) * kPitch;
      if (!p.planar) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(frame + ((size_t)row * p.W + 4 * seg) * 4));
        const uint2 p0 = pixel_bgra(v.x), p1 = pixel_bgra(v.y), p2 = pixel_bgra(v.z), p3 = pixel_bgra(v.w);
        uint4* d = reinterpret_cast<uint4*>(dst_row + (2 * seg + 1) * 16);  // pixels 4seg .. 4seg+3 = units 2seg+1, 2seg+2
        d[0] = make_uint4(p0.x, p0.y, p1.x, p1.y);
        d[1] = make_uint4(p2.x, p2.y, p3.x, p3.y);
      } else {
        const size_t off = (size_t)row * p.W + 16 * seg;
        const uint4 vr = __ldg(reinterpret_cast<const uint4*>(frame + off));
        const uint4 vg = __ldg(reinterpret_cast<const uint4*>(frame + plane + off));
        const uint4 vb = __ldg(reinterpret_cast<const uint4*>(frame + 2 * plane + off));
        const uint32_t wr[4] = {vr.x, vr.y, vr.z, vr.w}, wg[4] = {vg.x, vg.y, vg.z, vg.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint4* d = reinterpret_cast<uint4*>(dst_row + (8 * seg + 1) * 16);  // pixels 16seg .. 16seg+15 = units 8seg+1 .. 8seg+8
#pragma unroll
        for (int w4 = 0; w4 < 4; ++w4) {
          const uint2 p0 = pixel_rgb(wr[w4], wg[w4], wb[w4], 0x7540u), p1 = pixel_rgb(wr[w4], wg[w4], wb[w4], 0x7541u);
          const uint2 p2 = pixel_rgb(wr[w4], wg[w4], wb[w4], 0x7542u), p3 = pixel_rgb(wr[w4], wg[w4], wb[w4], 0x7543u);
          d[2 * w4] = make_uint4(p0.x, p0.y, p1.x, p1.y);
          d[2 * w4 + 1] = make_uint4(p2.x, p2.y, p3.x, p3.y);
        }
      }
    };
    int n = t_begin / p.Ho, y = t_begin - n * p.Ho;       // advanced by one output row per tile: no division in the loop
    int loaded_hi = max(2 * y - 2, 0) - 1;                // highest input row of frame n already in the ring
    const uint8_t* frame = p.frames + (size_t)n * frame_bytes;
    bool ok = true;
    griddep_wait();
    for (int i = 0; i < t_end - t_begin && ok; ++i) {
      const int hi = min(2 * y + 2, p.H - 1);
      const int first = loaded_hi + 1, nrows = hi - loaded_hi;
      if (i >= kLead && !mbar_wait_bounded_sleepy(bar_done + 8 * ((i - kLead) & 7), ((uint32_t)(i - kLead) >> 3) & 1u, s_abort, p.gerr, 831)) { ok = false; break; }
      if (rr0 < nrows) convert_item(frame, first + rr0, seg0);
      for (int idx = tid_l + 128; idx < nrows * segs; idx += 128) {
        const int rr = idx / segs;
        convert_item(frame, first + rr, idx - rr * segs);
      }
      fence_proxy_async_smem();                   // rows were written with ordinary stores; the MMAs read through the async proxy
      mbar_arrive(bar_ready + 8 * (i & 7));
      loaded_hi = hi;
      if (++y == p.Ho) {                          // next frame: nothing of it is loaded yet
        y = 0;
        ++n;
        frame += frame_bytes;
        loaded_hi = -1;
      }
    }
  }

  if (*s_abort) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

// w [K=32][3][5][5] fp16 -> the shared-memory image of the B operand: for MMA m = r*2 + h and K chunk c (0,1), row n:
// eight halves e = 4*s + ch covering tap column t = 4h + 2c + s of filter row r, channel ch (zero for t >= 5 or ch == 3)
__global__ void pack_rows_weights_kernel(const __half* __restrict__ w, __half* __restrict__ img) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= kMmas * 2 * kN * 8) return;
  const int e = i & 7, n = (i >> 3) % kN, j = i / (8 * kN);  // j = m*2 + c
  const int m = j >> 1, c = j & 1, r = m >> 1, h = m & 1;
  const int s = e >> 2, ch = e & 3, t = 4 * h + 2 * c + s;
  __half v = __ushort_as_half((unsigned short)0);
  if (t < 5 && ch < 3) v = w[((n * 3 + ch) * 5 + r) * 5 + t];
  img[i] = v;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn rows_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

struct ConvFirstRows {
  aig_ctx* ctx = nullptr;
  ConvFirstGeom g{};
  RowsParams prm{};
  const float *scale_dev = nullptr, *shift_dev = nullptr;
  __half* wimg = nullptr;
  CUtensorMap tmapY{};
  const void* tmap_ptr = nullptr;
  int tmap_s2d = -1;
  int Hb = 0, Wb = 0;
  int grid = 1;
};

bool conv_first_rows_supported(const ConvFirstGeom& g) {
  return g.D == 1 && g.kd == 1 && g.k == 5 && g.s == 2 && g.pad == 2 && g.K == kN && g.W % 16 == 0 && g.W >= 16 && g.W <= 256 && g.H >= 2 &&
         g.Wo <= 128 && g.Wo >= 2 && g.Ho >= 2;
}

int conv_first_rows_create(aig_ctx* ctx, const ConvFirstGeom& g, const float* scale, const float* shift, ConvFirstRows** out) {
  *out = nullptr;
  if (!conv_first_rows_supported(g)) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "first-layer row kernel: unsupported geometry");
  ConvFirstRows* t = new ConvFirstRows();
  t->ctx = ctx;
  t->g = g;
  t->scale_dev = scale;
  t->shift_dev = shift;
  RowsParams& p = t->prm;
  p.batch = g.batch; p.H = g.H; p.W = g.W; p.Ho = g.Ho; p.Wo = g.Wo;
  p.tiles = g.batch * g.Ho;
  p.slope = g.slope;
  p.gerr = ctx->d_err;
  if (cudaMalloc(&t->wimg, kSmemB) != cudaSuccess) {
    delete t;
    return aig_fail(ctx, AIG_ERR_CUDA, "first-layer row kernel: allocation failed");
  }
  p.wimg = reinterpret_cast<const uint4*>(t->wimg);
  t->grid = 3 * ctx->sm_count < p.tiles ? 3 * ctx->sm_count : p.tiles;
  *out = t;
  return AIG_OK;
}

void conv_first_rows_destroy(ConvFirstRows* t) {
  if (!t) return;
  cudaFree(t->wimg);
  delete t;
}

// Call after the plan's scale/shift kernel has been queued on the context's stream: the folded scale and shift
// travel to the kernel as launch parameters (constant bank), so they are read back here once.
int conv_first_rows_set_weights(ConvFirstRows* t, const __half* w) {
  aig_ctx* ctx = t->ctx;
  pack_rows_weights_kernel<<<ceil_div(kMmas * 2 * kN * 8, 256), 256, 0, ctx->stream>>>(w, t->wimg);
  AIG_LAUNCH_OK(ctx);
  AIG_CUDA_OK(ctx, cudaMemcpyAsync(t->prm.scale, t->scale_dev, kN * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  AIG_CUDA_OK(ctx, cudaMemcpyAsync(t->prm.shift, t->shift_dev, kN * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  AIG_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  return AIG_OK;
}

int conv_first_rows_set_s2d(ConvFirstRows* t, int enable, int Hb, int Wb) {
  if (enable && 2 * Wb > kOutSlots) return aig_fail(t->ctx, AIG_ERR_UNSUPPORTED, "first-layer row kernel: block row too wide");
  t->prm.s2d = enable ? 1 : 0;
  t->prm.Hb = Hb;
  t->Hb = Hb;
  t->Wb = Wb;
  return AIG_OK;
}

static int rows_encode_output(ConvFirstRows* t, __half* y) {
  EncodeTiledFn enc = rows_encode_fn();
  if (!enc) return aig_fail(t->ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  const ConvFirstGeom& g = t->g;
  CUresult r;
  if (t->prm.s2d) {
    // blocks [n][hb][wb][sy][sx][c] seen as (c, sx, wb, sy, n*hb): one output row = sub-row sy of block row hb,
    // pixels in (wb, sx) order = x + 1
    cuuint64_t dims[5] = {(cuuint64_t)kN, 2, (cuuint64_t)t->Wb, 2, (cuuint64_t)g.batch * t->Hb};
    cuuint64_t strides[4] = {(cuuint64_t)kN * 2, (cuuint64_t)4 * kN * 2, (cuuint64_t)2 * kN * 2, (cuuint64_t)t->Wb * 4 * kN * 2};
    cuuint32_t box[5] = {(cuuint32_t)kN, 2, (cuuint32_t)t->Wb, 1, 1};
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    r = enc(&t->tmapY, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, y, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[4] = {(cuuint64_t)kN, (cuuint64_t)g.Wo, (cuuint64_t)g.Ho, (cuuint64_t)g.batch};
    cuuint64_t strides[3] = {(cuuint64_t)kN * 2, (cuuint64_t)g.Wo * kN * 2, (cuuint64_t)g.Ho * g.Wo * kN * 2};
    cuuint32_t box[4] = {(cuuint32_t)kN, (cuuint32_t)g.Wo, 1, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    r = enc(&t->tmapY, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, y, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return aig_fail(t->ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled(first-layer output) failed: %d", (int)r);
  t->tmap_ptr = y;
  t->tmap_s2d = t->prm.s2d;
  return AIG_OK;
}

template <int ACT>
static int rows_launch(ConvFirstRows* t) {
  static bool attr_set[64] = {};
  aig_ctx* ctx = t->ctx;
  if (!attr_set[ctx->device & 63]) {
    AIG_CUDA_OK(ctx, cudaFuncSetAttribute(conv_first_rows_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set[ctx->device & 63] = true;
  }
  conv_first_rows_kernel<ACT><<<t->grid, kThreads, kSmemBytes, ctx->stream>>>(t->tmapY, t->prm);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

int conv_first_rows_forward(ConvFirstRows* t, const uint8_t* frames, int planar_rgb, __half* y) {
  aig_ctx* ctx = t->ctx;
  if (((uintptr_t)frames & 15) != 0 || ((uintptr_t)y & 15) != 0) return aig_fail(ctx, AIG_ERR_INVALID, "first-layer row kernel: frames and output must be 16-byte aligned");
  if (t->tmap_ptr != y || t->tmap_s2d != t->prm.s2d) {
    const int rc = rows_encode_output(t, y);
    if (rc != AIG_OK) return rc;
  }
  t->prm.frames = frames;
  t->prm.planar = planar_rgb ? 1 : 0;
  switch (t->g.act) {
    case AIG_ACT_RELU: return rows_launch<AIG_ACT_RELU>(t);
    case AIG_ACT_SWISH: return rows_launch<AIG_ACT_SWISH>(t);
    case AIG_ACT_LEAKY: return rows_launch<AIG_ACT_LEAKY>(t);
    default: return rows_launch<AIG_ACT_NONE>(t);
  }
}
