// lstm.cu -- LSTM forward (LSTMLayer.cpp:75-104 / LSTMLayerv8.cpp:78-82) for sm_100a.
//
// Per layer:  (1) the input projection W.x + bW + bR for all time steps is hoisted into one
// tcgen05 GEMM (rows = T*B, fp32 output);  (2) the recurrence runs as ONE persistent cooperative
// kernel: the recurrent matrix R is split over NC CTAs (each keeps the 4 gate rows of U hidden units,
// 4U x H fp16, resident in shared memory for all steps), every step each CTA
//    - TMA-loads h_{t-1} (128 batch rows x H, the previous step's output rows) into shared memory,
//    - issues tcgen05.mma  [128 x H] x [H x 4U]  into TMEM,
//    - its 128 epilogue threads (one per batch row) add the hoisted projection, apply the gates, keep
//      the cell state in registers (rounded to fp16 every step, like the library's cy tensor), write
//      h_t as fp16 into the output sequence, and
//    - all CTAs of the batch group meet at a device-wide step barrier (monotonic counter in global
//      memory, bounded spin).
// Gate order i,f,g,o; blob layout: per layer W then R, then per layer bW [and bR]  (the library's
// blob is opaque in the reference: LSTMLayer.cpp:29-35,139-146; this layout is this library's
// definition, stated in the header).
#include <vector>

#include "aig_common.cuh"

namespace {

constexpr int kRows = 128;        // batch rows per group (UMMA M)
constexpr int kThreads = 192;
constexpr int kKB = 64;           // K block (128-byte swizzle span of fp16)

struct LstmParams {
  int T, B, H, U, NC, groups;
  float clip;
  const float* gx;                // hoisted projection, element (t,b,j) at t*gx_sT + b*gx_sB + j, j < 4H
  long long gx_sT, gx_sB;
  __half* y;                      // output sequence, element (t,b,j) at t*y_sT + b*y_sB + j
  long long y_sT, y_sB;
  const __half* c0;               // [B][H] initial cell state
  __half* hT;                     // [B][H] final states (may be null)
  __half* cT;
  unsigned int* counter;          // [groups] step barrier counters, zero at launch
  int* gerr;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Gate non-linearities through the special-function unit (ex2 and rcp approximations, relative error ~2^-22, far
// below the fp16 rounding of h and c): an exact expf, IEEE division and tanhf per gate made the 128-thread
// epilogue the longest part of a step.
__device__ __forceinline__ float sigmoid_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}
__device__ __forceinline__ float tanh_fast(float x) {  // 2*sigmoid(2x) - 1
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -2.8853900817779268f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return fmaf(2.0f, r, -1.0f);
}

// U = hidden units per CTA (4U gate columns): 8, 16 or 32.
template <int U>
__global__ void __launch_bounds__(kThreads, 1)
lstm_recurrent_kernel(const __grid_constant__ CUtensorMap tmapR, const __grid_constant__ CUtensorMap tmapY,
                      const __grid_constant__ CUtensorMap tmapH0, const LstmParams p) {
  constexpr int NCOL = 4 * U;
  constexpr int kTmemCols = NCOL < 32 ? 32 : NCOL;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  const int nkb = p.H / kKB;
  const uint32_t sA = base;                                  // nkb slabs of 128 rows x 128 B
  const uint32_t sR = base + nkb * kRows * 128;              // nkb slabs of NCOL rows x 128 B
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + nkb * (kRows + NCOL) * 128);
  const uint32_t bar_a = smem_u32(bars);                     // [nkb] h slab landed
  const uint32_t bar_r = bar_a + 8 * 16;                     // R resident
  const uint32_t bar_tfull = bar_r + 8;                      // accumulator ready
  const uint32_t bar_tempty = bar_tfull + 8;                 // accumulator drained
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // (uniform for the compiler)
  const int group = blockIdx.x / p.NC, cta = blockIdx.x % p.NC;
  const int row0 = group * kRows;
  const int unit0 = cta * U;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nkb; ++i) mbar_init(bar_a + 8 * i, 1);
    mbar_init(bar_r, 1);
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 4);
    *s_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmapR);
    tma_prefetch_desc(&tmapY);
    tma_prefetch_desc(&tmapH0);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer + step barrier
    if (lane == 0) {
      // R slice, once: for every K block, the U rows of each of the four gates
      mbar_expect_tx(bar_r, (uint32_t)(nkb * NCOL * 128));
      for (int kb = 0; kb < nkb; ++kb)
        for (int g = 0; g < 4; ++g)
          tma_load_2d(sR + (kb * NCOL + g * U) * 128, &tmapR, bar_r, kb * kKB, g * p.H + unit0);
      bool ok = true;
      for (int t = 0; t < p.T && ok; ++t) {
        if (t > 0) {
          // wait until every CTA of this batch group has published h_{t-1}
          const unsigned int target = (unsigned int)t * (unsigned int)(p.NC * 4);
          const long long t0 = clock64();
          while (ld_acquire_gpu(p.counter + group) < target) {
            if (*s_abort) { ok = false; break; }
            if (clock64() - t0 > AIG_WAIT_CYCLES) {
              *s_abort = 1;
              atomicCAS(p.gerr, 0, 401);
              ok = false;
              break;
            }
          }
          if (!ok) break;
          fence_proxy_async_global();  // h_{t-1} was written with ordinary stores; TMA reads it through the async proxy
        }
        for (int kb = 0; kb < nkb; ++kb) {
          mbar_expect_tx(bar_a + 8 * kb, kRows * 128);
          if (t == 0) tma_load_3d(sA + kb * kRows * 128, &tmapH0, bar_a + 8 * kb, kb * kKB, row0, 0);
          else tma_load_3d(sA + kb * kRows * 128, &tmapY, bar_a + 8 * kb, kb * kKB, row0, t - 1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // (all lanes run the loop with identical values, one elected lane issues: see elect_one)
    {
      constexpr uint32_t idesc = umma_idesc_f16(kRows, NCOL);
      const bool leader = elect_one();
      bool ok = mbar_wait_bounded(bar_r, 0, s_abort, p.gerr, 402);
      for (int t = 0; t < p.T && ok; ++t) {
        const uint32_t ph = (uint32_t)t & 1u;
        if (!mbar_wait_bounded(bar_tempty, ph ^ 1u, s_abort, p.gerr, 403)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait_bounded(bar_a + 8 * kb, ph, s_abort, p.gerr, 404)) { ok = false; break; }
#pragma unroll
          for (int k = 0; k < kKB / 16; ++k) {
            const uint64_t adesc = umma_smem_desc(sA + kb * kRows * 128 + k * 32, 128);
            const uint64_t bdesc = umma_smem_desc(sR + kb * NCOL * 128 + k * 32, 128);
            if (leader) umma_f16_ss(tmem_base, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
        }
        if (ok && leader) umma_commit(bar_tfull);
      }
    }
  } else {
    // ------------------------------------------------------------------ gates: one thread per batch row
    const int q = warp & 3;
    const int b = row0 + q * 32 + lane;
    const bool valid = b < p.B;
    const int bb = valid ? b : 0;
    float c[U];
#pragma unroll
    for (int u = 0; u < U; ++u) c[u] = (valid && p.c0) ? __half2float(p.c0[(size_t)bb * p.H + unit0 + u]) : 0.f;
    bool ok = true;
    for (int t = 0; t < p.T && ok; ++t) {
      // hoisted projection for this row/step: 4 gates x U units (issued before the accumulator wait)
      float gx[4 * U];
      const float* gsrc = p.gx + (size_t)t * p.gx_sT + (size_t)bb * p.gx_sB + unit0;
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int u4 = 0; u4 < U / 4; ++u4) {
          const float4 v = valid ? *reinterpret_cast<const float4*>(gsrc + (size_t)g * p.H + 4 * u4) : make_float4(0.f, 0.f, 0.f, 0.f);
          gx[g * U + 4 * u4 + 0] = v.x;
          gx[g * U + 4 * u4 + 1] = v.y;
          gx[g * U + 4 * u4 + 2] = v.z;
          gx[g * U + 4 * u4 + 3] = v.w;
        }
      if (!mbar_wait_bounded(bar_tfull, (uint32_t)t & 1u, s_abort, p.gerr, 405)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16);
      __align__(16) __half hout[U];
#pragma unroll
      for (int u0 = 0; u0 < U; u0 += 8) {
        // columns: gate g, unit u -> g*U + u; read 8 units of every gate
        uint32_t ri[8], rf[8], rg[8], ro[8];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(ri[0]), "=r"(ri[1]), "=r"(ri[2]), "=r"(ri[3]), "=r"(ri[4]), "=r"(ri[5]), "=r"(ri[6]), "=r"(ri[7])
                     : "r"(t_addr + 0 * U + u0) : "memory");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(rf[0]), "=r"(rf[1]), "=r"(rf[2]), "=r"(rf[3]), "=r"(rf[4]), "=r"(rf[5]), "=r"(rf[6]), "=r"(rf[7])
                     : "r"(t_addr + 1 * U + u0) : "memory");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(rg[0]), "=r"(rg[1]), "=r"(rg[2]), "=r"(rg[3]), "=r"(rg[4]), "=r"(rg[5]), "=r"(rg[6]), "=r"(rg[7])
                     : "r"(t_addr + 2 * U + u0) : "memory");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(ro[0]), "=r"(ro[1]), "=r"(ro[2]), "=r"(ro[3]), "=r"(ro[4]), "=r"(ro[5]), "=r"(ro[6]), "=r"(ro[7])
                     : "r"(t_addr + 3 * U + u0) : "memory");
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int u = u0 + e;
          const float ig = sigmoid_fast(__uint_as_float(ri[e]) + gx[0 * U + u]);
          const float fg = sigmoid_fast(__uint_as_float(rf[e]) + gx[1 * U + u]);
          const float gg = tanh_fast(__uint_as_float(rg[e]) + gx[2 * U + u]);
          const float og = sigmoid_fast(__uint_as_float(ro[e]) + gx[3 * U + u]);
          float cn = fg * c[u] + ig * gg;
          if (p.clip > 0.f) cn = fminf(p.clip, fmaxf(-p.clip, cn));
          const __half ch = __float2half(cn);
          c[u] = __half2float(ch);
          hout[u] = __float2half(og * tanh_fast(c[u]));
        }
      }
      // accumulator drained: the MMA issuer may start the next step as soon as h_t is published
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty);
      if (valid) {
        __half* dst = p.y + (size_t)t * p.y_sT + (size_t)b * p.y_sB + unit0;
#pragma unroll
        for (int v = 0; v < U / 8; ++v) reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(hout)[v];
        if (t == p.T - 1) {
          if (p.hT) {
            __half* hd = p.hT + (size_t)b * p.H + unit0;
#pragma unroll
            for (int v = 0; v < U / 8; ++v) reinterpret_cast<uint4*>(hd)[v] = reinterpret_cast<const uint4*>(hout)[v];
          }
          if (p.cT) {
            __half* cd = p.cT + (size_t)b * p.H + unit0;
#pragma unroll
            for (int u = 0; u < U; ++u) cd[u] = __float2half(c[u]);
          }
        }
      }
      // publish h_t: make the stores visible device-wide (and to the async proxy), then count this warp in
      fence_proxy_async_global();
      __threadfence();
      __syncwarp();
      if (lane == 0) red_release_gpu_add(p.counter + group, 1u);
    }
  }

  if (*s_abort) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

struct aig_lstm_plan {
  aig_ctx* ctx = nullptr;
  int T = 0, L = 0, H = 0, B = 0, in_c = 0;
  float clip = 0.f;
  bool double_bias = true, batch_major = false;
  int U = 16, NC = 0, groups = 1;
  size_t smem = 0;
  const __half* blob = nullptr;
  std::vector<size_t> w_off, r_off, bw_off, br_off;
  std::vector<aig_conv_plan*> proj;     // hoisted input projection per layer
  float* gx = nullptr;                  // [T*B][4H] fp32 scratch
  __half* mid = nullptr;                // intermediate layer outputs (same layout as y)
  __half* zero_state = nullptr;         // [B][H] zeros for the default initial state
  __half* h_stage = nullptr;            // [B][H] final hidden state of the layer just run
  unsigned int* counters = nullptr;     // [L][groups]
  std::vector<CUtensorMap> mapR;
  size_t weight_count = 0;
};

namespace {

int encode_2d(aig_ctx* ctx, CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t stride1_bytes, uint32_t b0, uint32_t b1) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return aig_fail(ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {stride1_bytes};
  cuuint32_t box[2] = {b0, b1};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return aig_fail(ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled(2d) failed: %d", (int)r);
  return AIG_OK;
}
int encode_3d(aig_ctx* ctx, CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes,
              uint32_t b0, uint32_t b1) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return aig_fail(ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return aig_fail(ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled(3d) failed: %d", (int)r);
  return AIG_OK;
}

template <int U>
int launch_recurrent(aig_lstm_plan* pl, const CUtensorMap& mR, const CUtensorMap& mY, const CUtensorMap& mH0, LstmParams prm) {
  aig_ctx* ctx = pl->ctx;
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(lstm_recurrent_kernel<U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->smem));
  int per_sm = 0;
  AIG_CUDA_OK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_recurrent_kernel<U>, kThreads, pl->smem));
  const int grid = pl->NC * pl->groups;
  if (per_sm * ctx->sm_count < grid)
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm: %d CTAs cannot be co-resident (%d per SM x %d SMs)", grid, per_sm, ctx->sm_count);
  void* args[] = {(void*)&mR, (void*)&mY, (void*)&mH0, (void*)&prm};
  AIG_CUDA_OK(ctx, cudaLaunchCooperativeKernel((const void*)lstm_recurrent_kernel<U>, dim3(grid), dim3(kThreads), args, pl->smem, ctx->stream));
  return AIG_OK;
}

}  // namespace

extern "C" {

size_t aig_lstm_weight_count(int in_c, int hidden, int layers, int double_bias) {
  size_t n = 0;
  for (int l = 0; l < layers; ++l) n += (size_t)4 * hidden * (l == 0 ? in_c : hidden) + (size_t)4 * hidden * hidden;
  n += (size_t)layers * 4 * hidden * (double_bias ? 2 : 1);
  return n;
}

int aig_lstm_plan_create(aig_ctx* ctx, int seq_len, int layers, int hidden, int batch, int in_c, float clip, int double_bias,
                         int batch_major, aig_lstm_plan** out) {
  if (!ctx || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, seq_len > 0 && layers > 0 && hidden > 0 && batch > 0 && in_c > 0, "lstm plan: bad extents");
  if (hidden % 64 != 0 || hidden > 512)
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm plan: hidden must be a multiple of 64 and at most 512 (got %d)", hidden);
  if (in_c % 16 != 0) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm plan: in_c must be a multiple of 16 (got %d)", in_c);
  aig_lstm_plan* pl = new aig_lstm_plan();
  pl->ctx = ctx;
  pl->T = seq_len; pl->L = layers; pl->H = hidden; pl->B = batch; pl->in_c = in_c;
  pl->clip = clip; pl->double_bias = double_bias != 0; pl->batch_major = batch_major != 0;
  pl->groups = ceil_div(batch, kRows);
  // units per CTA: the fewest (most CTAs side by side, shortest epilogue per step) that still fit the device
  pl->U = 8;
  while (pl->U < 32 && (hidden / pl->U) * pl->groups > ctx->sm_count) pl->U *= 2;
  pl->NC = hidden / pl->U;
  if (pl->NC * pl->groups > ctx->sm_count) {
    delete pl;
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm plan: batch %d needs %d co-resident CTAs; split the batch", batch, pl->NC * pl->groups);
  }
  const int nkb = hidden / kKB;
  pl->smem = (size_t)nkb * (kRows + 4 * pl->U) * 128 + 1024 + 256;
  pl->weight_count = aig_lstm_weight_count(in_c, hidden, layers, double_bias);
  size_t off = 0;
  for (int l = 0; l < layers; ++l) {
    pl->w_off.push_back(off);
    off += (size_t)4 * hidden * (l == 0 ? in_c : hidden);
    pl->r_off.push_back(off);
    off += (size_t)4 * hidden * hidden;
  }
  for (int l = 0; l < layers; ++l) {
    pl->bw_off.push_back(off);
    off += (size_t)4 * hidden;
    pl->br_off.push_back(off);
    if (pl->double_bias) off += (size_t)4 * hidden;
  }
  int rc = AIG_OK;
  for (int l = 0; l < layers && rc == AIG_OK; ++l) {
    aig_conv_plan* fp = nullptr;
    rc = aig_fc_plan_create(ctx, seq_len * batch, l == 0 ? in_c : hidden, 4 * hidden, AIG_ACT_NONE, 0.f, 0, &fp);
    if (rc == AIG_OK) {
      aig_fc_plan_set_output_f32(fp, 1);
      pl->proj.push_back(fp);
    }
  }
  const size_t seq = (size_t)seq_len * batch;
  if (rc == AIG_OK && (cudaMalloc(&pl->gx, seq * 4 * hidden * sizeof(float)) != cudaSuccess ||
                       cudaMalloc(&pl->mid, seq * hidden * sizeof(__half)) != cudaSuccess ||
                       cudaMalloc(&pl->zero_state, (size_t)batch * hidden * sizeof(__half)) != cudaSuccess ||
                       cudaMalloc(&pl->h_stage, (size_t)batch * hidden * sizeof(__half)) != cudaSuccess ||
                       cudaMalloc(&pl->counters, (size_t)layers * pl->groups * sizeof(unsigned int)) != cudaSuccess ||
                       cudaMemset(pl->zero_state, 0, (size_t)batch * hidden * sizeof(__half)) != cudaSuccess))
    rc = aig_fail(ctx, AIG_ERR_CUDA, "lstm plan: device allocation failed");
  if (rc != AIG_OK) {
    aig_lstm_plan_destroy(pl);
    return rc;
  }
  pl->mapR.resize(layers);
  *out = pl;
  return AIG_OK;
}

int aig_lstm_plan_destroy(aig_lstm_plan* pl) {
  if (!pl) return AIG_OK;
  DeviceGuard g(pl->ctx->device);
  cudaStreamSynchronize(pl->ctx->stream);
  for (aig_conv_plan* fp : pl->proj) aig_conv_plan_destroy(fp);
  cudaFree(pl->gx);
  cudaFree(pl->mid);
  cudaFree(pl->zero_state);
  cudaFree(pl->h_stage);
  cudaFree(pl->counters);
  delete pl;
  return AIG_OK;
}

int aig_lstm_plan_set_weights(aig_lstm_plan* pl, const aig_half* blob) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, blob != nullptr && ((uintptr_t)blob & 15) == 0, "lstm set_weights: blob must be non-null and 16-byte aligned");
  pl->blob = (const __half*)blob;
  for (int l = 0; l < pl->L; ++l) {
    int rc = aig_fc_plan_set_weights_out_in(pl->proj[l], blob + pl->w_off[l], blob + pl->bw_off[l]);
    if (rc != AIG_OK) return rc;
    if (pl->double_bias && (rc = aig_fc_plan_add_bias(pl->proj[l], blob + pl->br_off[l])) != AIG_OK) return rc;
    // recurrent matrix [4H][H], box = 64 K-elements x U rows
    rc = encode_2d(ctx, &pl->mapR[l], blob + pl->r_off[l], pl->H, (uint64_t)4 * pl->H, (uint64_t)pl->H * 2, kKB, pl->U);
    if (rc != AIG_OK) return rc;
  }
  return AIG_OK;
}

// x: [T][B][in] (or [B][T][in] when the plan is batch-major); y: [T][B][H] (or [B][T][H]).
// h_state/c_state: [layers][B][H] fp16 or null; read when use_state != 0, always written when non-null.
int aig_lstm_forward(aig_lstm_plan* pl, const aig_half* x, aig_half* y, aig_half* h_state, aig_half* c_state, int use_state) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, x && y && pl->blob, "lstm forward: null pointer or weights not set");
  AIG_REQUIRE(ctx, ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0, "lstm forward: tensors must be 16-byte aligned");
  AIG_REQUIRE(ctx, (h_state == nullptr) == (c_state == nullptr), "lstm forward: give both state tensors or neither");
  AIG_REQUIRE(ctx, !use_state || h_state, "lstm forward: use_state needs the state tensors");
  const int T = pl->T, B = pl->B, H = pl->H;
  const long long sT = pl->batch_major ? H : (long long)B * H, sB = pl->batch_major ? (long long)T * H : H;
  AIG_CUDA_OK(ctx, cudaMemsetAsync(pl->counters, 0, (size_t)pl->L * pl->groups * sizeof(unsigned int), ctx->stream));
  const __half* in = (const __half*)x;
  for (int l = 0; l < pl->L; ++l) {
    // a middle layer may read and write `mid`: its input is fully consumed by the hoisted projection
    // before the recurrence starts overwriting it
    __half* out = (l == pl->L - 1) ? (__half*)y : pl->mid;
    int rc = aig_conv_forward(pl->proj[l], (const aig_half*)in, nullptr, (aig_half*)pl->gx);
    if (rc != AIG_OK) return rc;
    CUtensorMap mY, mH0;
    rc = encode_3d(ctx, &mY, out, H, B, T, (uint64_t)sB * 2, (uint64_t)sT * 2, kKB, kRows);
    if (rc != AIG_OK) return rc;
    const __half* h0 = use_state ? (const __half*)h_state + (size_t)l * B * H : pl->zero_state;
    rc = encode_3d(ctx, &mH0, h0, H, B, 1, (uint64_t)H * 2, (uint64_t)B * H * 2, kKB, kRows);
    if (rc != AIG_OK) return rc;
    LstmParams prm{};
    prm.T = T; prm.B = B; prm.H = H; prm.U = pl->U; prm.NC = pl->NC; prm.groups = pl->groups;
    prm.clip = pl->clip;
    prm.gx = pl->gx;
    // the projection's rows follow x's memory order
    prm.gx_sT = pl->batch_major ? (long long)4 * H : (long long)B * 4 * H;
    prm.gx_sB = pl->batch_major ? (long long)T * 4 * H : (long long)4 * H;
    prm.y = out; prm.y_sT = sT; prm.y_sB = sB;
    prm.c0 = use_state ? (const __half*)c_state + (size_t)l * B * H : nullptr;
    // the final h goes to a staging buffer first: with T == 1 other CTAs may still be reading the
    // initial h from the caller's state tensor while this one finishes
    prm.hT = h_state ? pl->h_stage : nullptr;
    prm.cT = c_state ? (__half*)c_state + (size_t)l * B * H : nullptr;
    prm.counter = pl->counters + (size_t)l * pl->groups;
    prm.gerr = ctx->d_err;
    switch (pl->U) {
      case 8: rc = launch_recurrent<8>(pl, pl->mapR[l], mY, mH0, prm); break;
      case 16: rc = launch_recurrent<16>(pl, pl->mapR[l], mY, mH0, prm); break;
      case 32: rc = launch_recurrent<32>(pl, pl->mapR[l], mY, mH0, prm); break;
      default: rc = aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm: unsupported units per CTA %d", pl->U);
    }
    if (rc != AIG_OK) return rc;
    if (h_state)
      AIG_CUDA_OK(ctx, cudaMemcpyAsync((__half*)h_state + (size_t)l * B * H, pl->h_stage, (size_t)B * H * sizeof(__half),
                                       cudaMemcpyDeviceToDevice, ctx->stream));
    in = out;
  }
  return AIG_OK;
}

}  // extern "C"

// =============================================================================================
// Allocation-free single-layer LSTM forward.
//
// For callers that must not allocate device memory once they are running: a frame loop that shares
// the GPU with the game it plays (cudaMalloc/cudaFree synchronise the whole device and stall every
// other stream, and the game may already own nearly all of the memory), or a host application that
// reserves its whole device budget at start-up and forbids later allocations.  Everything the plan
// based entry points keep in cudaMalloc'ed buffers -- the hoisted input projection, the zero initial
// state and the step-barrier counter -- lives here in one fixed array in the library's device image.
//
// The array is part of the module: every GPU that loads the library holds kNoAllocBytes until the
// process exits.  All calls on a device share it, so two calls that overlap on the GPU (different
// streams) race; serialise them.  It keeps the previous call's contents, so each call clears the parts
// that must start at zero (the barrier counter and the zero state) on its stream before use.
namespace {

constexpr size_t kNoAllocProjFloats = (size_t)1 << 19;                       // 2 MiB of fp32 projections
constexpr int kNoAllocMaxBatch = kRows;                                      // one batch group
constexpr int kNoAllocMaxHidden = 512;
constexpr size_t kNoAllocProjBytes = kNoAllocProjFloats * sizeof(float);
constexpr size_t kNoAllocStateBytes = (size_t)kNoAllocMaxBatch * kNoAllocMaxHidden * sizeof(__half);
constexpr size_t kNoAllocCounterOff = kNoAllocProjBytes + kNoAllocStateBytes;
constexpr size_t kNoAllocBytes = kNoAllocCounterOff + 256;

// In host code this name is only a handle for the runtime's symbol table, not a device address: the
// device address is fetched once per device with cudaGetSymbolAddress below and that is what kernels get.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

unsigned char* g_noalloc_ptr[64] = {};  // per device, filled by the first call on that device

// gx[row][j] = sum_k x[row][k] * W[j][k] + bW[j] (+ bR[j]); 32x32 output tile per block, fp32 accumulate.
__global__ void noalloc_projection_kernel(const __half* __restrict__ x, const __half* __restrict__ W,
                                          const __half* __restrict__ bW, const __half* __restrict__ bR,
                                          float* __restrict__ gx, int rows, int in_c, int out_c) {
  __shared__ float sx[32][33], sw[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
  const int row0 = blockIdx.y * 32, col0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < in_c; k0 += 32) {
    for (int i = ty; i < 32; i += 8) {
      const int r = row0 + i, c = col0 + i, k = k0 + tx;
      sx[i][tx] = (r < rows && k < in_c) ? __half2float(x[(size_t)r * in_c + k]) : 0.f;
      sw[i][tx] = (c < out_c && k < in_c) ? __half2float(W[(size_t)c * in_c + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
      const float wv = sw[tx][kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(sx[ty + 8 * i][kk], wv, acc[i]);
    }
    __syncthreads();
  }
  const int c = col0 + tx;
  if (c < out_c) {
    const float b = __half2float(bW[c]) + (bR ? __half2float(bR[c]) : 0.f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = row0 + ty + 8 * i;
      if (r < rows) gx[(size_t)r * out_c + c] = acc[i] + b;
    }
  }
}

}  // namespace

extern "C" {

// Single-layer, seq-major LSTM forward with zero initial state: x [T][B][in] -> y [T][B][hidden], the blob
// laid out as aig_lstm_plan_set_weights expects for one layer.  Asynchronous on the context's stream; no
// device or pinned memory is allocated or freed.  The first call on a device resolves the scratch array's
// device address (cudaGetSymbolAddress); make that first call before any stream capture begins.
int aig_lstm_forward_noalloc(aig_ctx* ctx, const aig_half* x, const aig_half* blob, aig_half* y, int seq_len, int batch,
                             int in_c, int hidden, float clip, int double_bias) {
  if (!ctx) return AIG_ERR_INVALID;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, x && blob && y && seq_len > 0 && batch > 0 && in_c > 0 && hidden > 0, "lstm noalloc: bad arguments");
  AIG_REQUIRE(ctx, ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)blob & 15) == 0,
              "lstm noalloc: tensors must be 16-byte aligned");
  if (hidden % 64 != 0 || hidden > kNoAllocMaxHidden)
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm noalloc: hidden must be a multiple of 64 and at most %d (got %d)", kNoAllocMaxHidden, hidden);
  if (batch > kNoAllocMaxBatch)
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm noalloc: batch %d exceeds the maximum of %d", batch, kNoAllocMaxBatch);
  if (in_c % 8 != 0) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm noalloc: in_c must be a multiple of 8 (got %d)", in_c);
  const size_t proj = (size_t)seq_len * batch * 4 * hidden;
  if (proj > kNoAllocProjFloats)
    return aig_fail(ctx, AIG_ERR_UNSUPPORTED,
                    "lstm noalloc: seq_len*batch*4*hidden = %zu exceeds the fixed scratch of %zu floats (%zu bytes)", proj,
                    kNoAllocProjFloats, kNoAllocProjBytes);
  constexpr int U = 16;
  const int NC = hidden / U, nkb = hidden / kKB;
  const size_t smem = (size_t)nkb * (kRows + 4 * U) * 128 + 1024 + 256;
  // ---- once per device: resolve the symbol, set the kernel's shared-memory limit
  unsigned char*& base = g_noalloc_ptr[ctx->device & 63];
  if (!base) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return aig_fail(ctx, AIG_ERR_CUDA, "lstm noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    base = static_cast<unsigned char*>(p);
  }
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(lstm_recurrent_kernel<U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  float* gx = reinterpret_cast<float*>(base);
  __half* zero_state = reinterpret_cast<__half*>(base + kNoAllocProjBytes);
  unsigned int* counter = reinterpret_cast<unsigned int*>(base + kNoAllocCounterOff);
  int per_sm = 0;
  AIG_CUDA_OK(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_recurrent_kernel<U>, kThreads, smem));
  if (per_sm * ctx->sm_count < NC) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "lstm noalloc: %d CTAs cannot be co-resident", NC);
  // ---- what must start at zero
  AIG_CUDA_OK(ctx, cudaMemsetAsync(counter, 0, 256, ctx->stream));
  AIG_CUDA_OK(ctx, cudaMemsetAsync(zero_state, 0, (size_t)batch * hidden * sizeof(__half), ctx->stream));
  // ---- hoisted input projection into the scratch
  const __half* hb = reinterpret_cast<const __half*>(blob);
  const size_t w_off = 0, r_off = (size_t)4 * hidden * in_c, bw_off = r_off + (size_t)4 * hidden * hidden,
               br_off = bw_off + (size_t)4 * hidden;
  const int rows = seq_len * batch;
  noalloc_projection_kernel<<<dim3(ceil_div(4 * hidden, 32), ceil_div(rows, 32)), 256, 0, ctx->stream>>>(
      (const __half*)x, hb + w_off, hb + bw_off, double_bias ? hb + br_off : nullptr, gx, rows, in_c, 4 * hidden);
  AIG_LAUNCH_OK(ctx);
  // ---- recurrence
  CUtensorMap mR, mY, mH0;
  int rc = encode_2d(ctx, &mR, hb + r_off, hidden, (uint64_t)4 * hidden, (uint64_t)hidden * 2, kKB, U);
  if (rc == AIG_OK) rc = encode_3d(ctx, &mY, y, hidden, batch, seq_len, (uint64_t)hidden * 2, (uint64_t)batch * hidden * 2, kKB, kRows);
  if (rc == AIG_OK) rc = encode_3d(ctx, &mH0, zero_state, hidden, batch, 1, (uint64_t)hidden * 2, (uint64_t)batch * hidden * 2, kKB, kRows);
  if (rc != AIG_OK) return rc;
  LstmParams prm{};
  prm.T = seq_len; prm.B = batch; prm.H = hidden; prm.U = U; prm.NC = NC; prm.groups = 1;
  prm.clip = clip;
  prm.gx = gx;
  prm.gx_sT = (long long)batch * 4 * hidden;
  prm.gx_sB = (long long)4 * hidden;
  prm.y = (__half*)y;
  prm.y_sT = (long long)batch * hidden;
  prm.y_sB = hidden;
  prm.c0 = nullptr; prm.hT = nullptr; prm.cT = nullptr;
  prm.counter = counter;
  prm.gerr = ctx->d_err;
  void* args[] = {(void*)&mR, (void*)&mY, (void*)&mH0, (void*)&prm};
  AIG_CUDA_OK(ctx, cudaLaunchCooperativeKernel((const void*)lstm_recurrent_kernel<U>, dim3(NC), dim3(kThreads), args, smem, ctx->stream));
  return AIG_OK;
}

}  // extern "C"
