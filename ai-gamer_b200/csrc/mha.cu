// mha.cu -- multi-head causal self-attention (MHALayer.cpp:128-146 as its fields define it) for
// sm_100a, with rotary embedding applied while the Q/K tiles are staged and a ring key/value cache
// for step-by-step use.
//
// Full sequence:  Q,K,V = x.Wq, x.Wk, x.Wv (three tcgen05 GEMM launches), then one attention kernel:
//   per (sequence, head) work item a CTA
//     - TMA-loads the Q tile (128 query rows, rows >= T zero-filled), K and V tiles (NK key rows),
//     - its 128 row threads rotate Q and K in shared memory (RoPE), transpose V to K-major,
//     - tcgen05.mma  S = Q.K^T  into TMEM, row threads do the masked softmax from TMEM and write
//       P (fp16) back to shared memory as the next A operand,
//     - tcgen05.mma  O = P.V   into TMEM, row threads normalise and store the context rows,
//   then the output projection (.Wo) is one more GEMM launch.
// Streaming step: projections on [B][E], then one CUDA-core kernel per (sequence, head) warp rotates
// q/k, appends k/v to the ring cache and attends over the cached window.
#include <vector>

#include "aig_common.cuh"

namespace {

constexpr int kThreads = 192;
constexpr int kQRows = 128;
constexpr int kD = 64;  // head dimension handled by the tile kernel

struct AttnParams {
  int B, T, E, heads, window;
  float scale;
  const float2* rope;   // [T][kD/2] (cos, sin) for positions pos0..pos0+T-1, or null
  __half* ctx;          // [B][T][E]
  int* gerr;
};

__device__ __forceinline__ void tma_load_3d_(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// byte offset of logical 16-byte chunk `c` of row `r` in a 128-byte-swizzled tile with 128-byte rows
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// in-place rotation of one 64-wide row held in a swizzled tile: pairs (j, j + 32)
__device__ __forceinline__ void rope_row(uint8_t* tile, int r, const float2* cs) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 lo = *reinterpret_cast<uint4*>(tile + swz(r, c));
    uint4 hi = *reinterpret_cast<uint4*>(tile + swz(r, c + 4));
    __half* a = reinterpret_cast<__half*>(&lo);
    __half* b = reinterpret_cast<__half*>(&hi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float2 t = cs[c * 8 + e];
      const float fa = __half2float(a[e]), fb = __half2float(b[e]);
      a[e] = __float2half(fa * t.x - fb * t.y);
      b[e] = __float2half(fb * t.x + fa * t.y);
    }
    *reinterpret_cast<uint4*>(tile + swz(r, c)) = lo;
    *reinterpret_cast<uint4*>(tile + swz(r, c + 4)) = hi;
  }
}

// NK = key slots per tile (64 or 128); T <= NK, T <= 128.
template <int NK>
__global__ void __launch_bounds__(kThreads, 1)
attention_tile_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                      const __grid_constant__ CUtensorMap mapV, const AttnParams p) {
  constexpr int kKB = NK / 64;                 // 64-key blocks
  constexpr int kTmemCols = 256;               // S: NK columns at 0, O: 64 columns at NK
  constexpr uint32_t kLoadBytes = kQRows * 128 + 2 * NK * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - raw);
  uint8_t* qT = sm;                                   // [128][64] fp16
  uint8_t* kT = qT + kQRows * 128;                    // [NK][64]
  uint8_t* vT = kT + NK * 128;                        // [NK][64] as loaded (key-major)
  uint8_t* vtT = vT + NK * 128;                       // kKB x [64 d rows][64 keys]: V transposed, K-major
  uint8_t* pT = vtT + kKB * 64 * 128;                 // kKB x [128 rows][64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(pT + kKB * kQRows * 128);
  const uint32_t bar_load = smem_u32(bars), bar_qk = bar_load + 8, bar_s = bar_load + 16, bar_p = bar_load + 24,
                 bar_o = bar_load + 32, bar_free = bar_load + 40;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // (uniform for the compiler)

  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_qk, 128);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_o, 1);
    mbar_init(bar_free, 128);
    *s_abort = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(s_tmem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const int items = p.B * p.heads;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
        const int b = item / p.heads, h = item - b * p.heads;
        // the tiles are free again once the previous item's second MMA has completed and its rows are stored
        if (it > 0 && !mbar_wait_bounded(bar_free, (uint32_t)(it - 1) & 1u, s_abort, p.gerr, 501)) break;
        mbar_expect_tx(bar_load, kLoadBytes);
        tma_load_3d_(smem_u32(qT), &mapQ, bar_load, h * kD, 0, b);
        tma_load_3d_(smem_u32(kT), &mapK, bar_load, h * kD, 0, b);
        tma_load_3d_(smem_u32(vT), &mapV, bar_load, h * kD, 0, b);
      }
    }
  } else if (warp == 1) {
    // (all lanes run the loop with identical values, one elected lane issues: see elect_one)
    {
      constexpr uint32_t idesc_s = umma_idesc_f16(kQRows, NK);
      constexpr uint32_t idesc_o = umma_idesc_f16(kQRows, kD);
      const bool leader = elect_one();
      int it = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
        const uint32_t ph = (uint32_t)it & 1u;
        if (!mbar_wait_bounded(bar_qk, ph, s_abort, p.gerr, 502)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (leader) umma_f16_ss(tmem_base, umma_smem_desc(smem_u32(qT) + k * 32, 128), umma_smem_desc(smem_u32(kT) + k * 32, 128), idesc_s,
                      k != 0 ? 1u : 0u);
        if (leader) umma_commit(bar_s);
        if (!mbar_wait_bounded(bar_p, ph, s_abort, p.gerr, 503)) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < kKB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (leader) umma_f16_ss(tmem_base + NK, umma_smem_desc(smem_u32(pT) + kb * kQRows * 128 + k * 32, 128),
                        umma_smem_desc(smem_u32(vtT) + kb * 64 * 128 + k * 32, 128), idesc_o, (kb | k) != 0 ? 1u : 0u);
        if (leader) umma_commit(bar_o);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // query row / key row handled by this thread
    const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
    int it = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++it) {
      const int b = item / p.heads, h = item - b * p.heads;
      const uint32_t ph = (uint32_t)it & 1u;
      if (!mbar_wait_bounded(bar_load, ph, s_abort, p.gerr, 504)) break;
      // ---- stage: RoPE on Q and K rows, V transposed to K-major
      if (p.rope && r < p.T) {
        rope_row(qT, r, p.rope + (size_t)r * (kD / 2));
        if (r < NK) rope_row(kT, r, p.rope + (size_t)r * (kD / 2));
      }
      if (r < NK) {
        const int kb = r >> 6, key = r & 63;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v = *reinterpret_cast<const uint4*>(vT + swz(r, c));
          const __half* hv = reinterpret_cast<const __half*>(&v);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int d = c * 8 + e;
            *reinterpret_cast<__half*>(vtT + kb * 64 * 128 + swz(d, key >> 3) + (key & 7) * 2) = hv[e];
          }
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_qk);
      // ---- softmax over S row r
      if (!mbar_wait_bounded(bar_s, ph, s_abort, p.gerr, 505)) break;
      tc_fence_after();
      const int lo = (p.window > 0 && r - p.window + 1 > 0) ? r - p.window + 1 : 0;
      const int hi = r;  // causal: keys lo..hi
      float mx = -INFINITY;
      float s[NK];
#pragma unroll
      for (int c0 = 0; c0 < NK; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int j = c0 + e;
          const bool ok = r < p.T && j >= lo && j <= hi;
          s[j] = ok ? __uint_as_float(v[e]) * p.scale : -INFINITY;
          mx = fmaxf(mx, s[j]);
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int kb = 0; kb < kKB; ++kb)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 o;
          __half* ho = reinterpret_cast<__half*>(&o);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int j = kb * 64 + c * 8 + e;
            const float pv = (r < p.T && s[j] > -INFINITY) ? expf(s[j] - mx) : 0.f;
            ho[e] = __float2half(pv);
            sum += __half2float(ho[e]);  // normalise by what the second MMA actually multiplies with
          }
          *reinterpret_cast<uint4*>(pT + kb * kQRows * 128 + swz(r, c)) = o;
        }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(bar_p);
      // ---- context row
      if (!mbar_wait_bounded(bar_o, ph, s_abort, p.gerr, 506)) break;
      tc_fence_after();
      const float inv = sum > 0.f ? 1.0f / sum : 0.f;
      __half* dst = p.ctx + ((size_t)b * p.T + r) * p.E + h * kD;
#pragma unroll
      for (int c0 = 0; c0 < kD; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + NK + c0, v);
        tmem_ld_wait();
        if (r < p.T) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 o;
            __half* ho = reinterpret_cast<__half*>(&o);
#pragma unroll
            for (int e = 0; e < 8; ++e) ho[e] = __float2half(__uint_as_float(v[c * 8 + e]) * inv);
            *reinterpret_cast<uint4*>(dst + c0 + c * 8) = o;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_free);
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

__global__ void rope_table_kernel(float2* table, int T, int half_d, int d, float base, int pos0) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half_d) return;
  const int t = i / half_d, j = i - t * half_d;
  const float inv = powf(base, -2.0f * (float)j / (float)d);
  const float ang = (float)(pos0 + t) * inv;
  table[i] = make_float2(cosf(ang), sinf(ang));
}

// Streaming step.  One warp per (sequence, head): rotate q and k at `position`, append k,v to ring slot
// position % window, attend over the `n_valid` most recent slots.  qkv: three [B][E] tensors.
__global__ void attention_step_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                                      __half* __restrict__ kcache, __half* __restrict__ vcache, __half* __restrict__ ctx,
                                      int B, int E, int heads, int d, int window, int position, int n_valid, float base,
                                      float scale) {
  extern __shared__ float sh[];  // per warp: q[d] + probs[window]
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + wib;
  if (item >= B * heads) return;
  const int b = item / heads, h = item - b * heads;
  float* sq = sh + (size_t)wib * (d + window);
  float* sp = sq + d;
  const int half_d = d / 2;
  const size_t row = (size_t)b * E + (size_t)h * d;
  const int slot = position % window;
  __half* kslot = kcache + ((size_t)b * window + slot) * E + (size_t)h * d;
  __half* vslot = vcache + ((size_t)b * window + slot) * E + (size_t)h * d;
  for (int j = lane; j < half_d; j += 32) {
    float cs = 1.f, sn = 0.f;
    if (base > 0.f) {
      const float inv = powf(base, -2.0f * (float)j / (float)d);
      const float ang = (float)position * inv;
      cs = cosf(ang);
      sn = sinf(ang);
    }
    const float qa = __half2float(q[row + j]), qb = __half2float(q[row + j + half_d]);
    const float ka = __half2float(k[row + j]), kb = __half2float(k[row + j + half_d]);
    sq[j] = __half2float(__float2half(qa * cs - qb * sn));
    sq[j + half_d] = __half2float(__float2half(qb * cs + qa * sn));
    kslot[j] = __float2half(ka * cs - kb * sn);
    kslot[j + half_d] = __float2half(kb * cs + ka * sn);
    vslot[j] = v[row + j];
    vslot[j + half_d] = v[row + j + half_d];
  }
  __syncwarp();
  // scores: lane-per-key over the valid window (positions position-n_valid+1 .. position)
  float mx = -INFINITY;
  for (int i = lane; i < n_valid; i += 32) {
    const int pos = position - i;
    const __half* kr = kcache + ((size_t)b * window + (pos % window)) * E + (size_t)h * d;
    float acc = 0.f;
    for (int c = 0; c < d; c += 8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(kr + c);
      const __half* kh = reinterpret_cast<const __half*>(&kv);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc = fmaf(sq[c + e], __half2float(kh[e]), acc);
    }
    sp[i] = acc * scale;
    mx = fmaxf(mx, sp[i]);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int i = lane; i < n_valid; i += 32) {
    const float e = expf(sp[i] - mx);
    sp[i] = e;
    sum += e;
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  const float inv = 1.0f / sum;
  // context: lane-per-dimension
  for (int c = lane; c < d; c += 32) {
    float acc = 0.f;
    for (int i = 0; i < n_valid; ++i) {
      const int pos = position - i;
      acc = fmaf(sp[i], __half2float(vcache[((size_t)b * window + (pos % window)) * E + (size_t)h * d + c]), acc);
    }
    ctx[row + c] = __float2half(acc * inv);
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

struct aig_mha_plan {
  aig_ctx* ctx = nullptr;
  int B = 0, T = 0, E = 0, heads = 0, d = 0, window = 0;
  float rope_base = 0.f;
  aig_conv_plan *pq = nullptr, *pk = nullptr, *pv = nullptr, *po = nullptr;       // full sequence (rows B*T)
  aig_conv_plan *sq = nullptr, *sk = nullptr, *sv = nullptr, *so = nullptr;       // streaming (rows B)
  __half *q = nullptr, *k = nullptr, *v = nullptr, *ctxbuf = nullptr;              // [B][T][E]
  __half *kcache = nullptr, *vcache = nullptr;                                     // [B][window][E]
  float2* rope = nullptr;
  CUtensorMap mq{}, mk{}, mv{};
  bool weights_set = false;
  int stream_start = -1;  // first position appended since the last reset
  int ring = 0;           // slots in the ring cache
};

namespace {

int encode_qkv(aig_mha_plan* pl, CUtensorMap* m, const void* ptr, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return aig_fail(pl->ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[3] = {(cuuint64_t)pl->E, (cuuint64_t)pl->T, (cuuint64_t)pl->B};
  cuuint64_t strides[2] = {(cuuint64_t)pl->E * 2, (cuuint64_t)pl->T * pl->E * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return aig_fail(pl->ctx, AIG_ERR_CUDA, "cuTensorMapEncodeTiled(qkv) failed: %d", (int)r);
  return AIG_OK;
}

template <int NK>
int launch_attention(aig_mha_plan* pl, const AttnParams& prm) {
  aig_ctx* ctx = pl->ctx;
  constexpr int kKB = NK / 64;
  const size_t smem = (size_t)kQRows * 128 + 2 * NK * 128 + kKB * 64 * 128 + kKB * kQRows * 128 + 1024 + 128;
  AIG_CUDA_OK(ctx, cudaFuncSetAttribute(attention_tile_kernel<NK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int items = pl->B * pl->heads;
  const int grid = items < ctx->sm_count ? items : ctx->sm_count;
  attention_tile_kernel<NK><<<grid, kThreads, smem, ctx->stream>>>(pl->mq, pl->mk, pl->mv, prm);
  AIG_LAUNCH_OK(ctx);
  return AIG_OK;
}

}  // namespace

extern "C" {

int aig_mha_plan_create(aig_ctx* ctx, int batch, int seq_len, int embed, int heads, float rope_base, int window, aig_mha_plan** out) {
  if (!ctx || !out) return AIG_ERR_INVALID;
  *out = nullptr;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, batch > 0 && seq_len > 0 && embed > 0 && heads > 0 && embed % heads == 0, "mha plan: bad extents");
  if (embed / heads != kD) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "mha plan: head dimension must be 64 (got %d)", embed / heads);
  if (seq_len > 128) return aig_fail(ctx, AIG_ERR_UNSUPPORTED, "mha plan: full-sequence length above 128 is not supported (got %d)", seq_len);
  aig_mha_plan* pl = new aig_mha_plan();
  pl->ctx = ctx;
  pl->B = batch; pl->T = seq_len; pl->E = embed; pl->heads = heads; pl->d = kD; pl->window = window; pl->rope_base = rope_base;
  pl->ring = window > 0 ? window : seq_len;
  int rc = AIG_OK;
  aig_conv_plan** full[4] = {&pl->pq, &pl->pk, &pl->pv, &pl->po};
  aig_conv_plan** step[4] = {&pl->sq, &pl->sk, &pl->sv, &pl->so};
  for (int i = 0; i < 4 && rc == AIG_OK; ++i) rc = aig_fc_plan_create(ctx, batch * seq_len, embed, embed, AIG_ACT_NONE, 0.f, 1, full[i]);
  for (int i = 0; i < 4 && rc == AIG_OK; ++i) rc = aig_fc_plan_create(ctx, batch, embed, embed, AIG_ACT_NONE, 0.f, 1, step[i]);
  const size_t n = (size_t)batch * seq_len * embed;
  if (rc == AIG_OK && (cudaMalloc(&pl->q, n * 2) != cudaSuccess || cudaMalloc(&pl->k, n * 2) != cudaSuccess ||
                       cudaMalloc(&pl->v, n * 2) != cudaSuccess || cudaMalloc(&pl->ctxbuf, n * 2) != cudaSuccess ||
                       cudaMalloc(&pl->kcache, (size_t)batch * pl->ring * embed * 2) != cudaSuccess ||
                       cudaMalloc(&pl->vcache, (size_t)batch * pl->ring * embed * 2) != cudaSuccess ||
                       cudaMalloc(&pl->rope, (size_t)seq_len * (kD / 2) * sizeof(float2)) != cudaSuccess))
    rc = aig_fail(ctx, AIG_ERR_CUDA, "mha plan: device allocation failed");
  const int nk = seq_len <= 64 ? 64 : 128;
  if (rc == AIG_OK) rc = encode_qkv(pl, &pl->mq, pl->q, kQRows);
  if (rc == AIG_OK) rc = encode_qkv(pl, &pl->mk, pl->k, nk);
  if (rc == AIG_OK) rc = encode_qkv(pl, &pl->mv, pl->v, nk);
  if (rc != AIG_OK) {
    aig_mha_plan_destroy(pl);
    return rc;
  }
  *out = pl;
  return AIG_OK;
}

int aig_mha_plan_destroy(aig_mha_plan* pl) {
  if (!pl) return AIG_OK;
  DeviceGuard g(pl->ctx->device);
  cudaStreamSynchronize(pl->ctx->stream);
  aig_conv_plan* plans[8] = {pl->pq, pl->pk, pl->pv, pl->po, pl->sq, pl->sk, pl->sv, pl->so};
  for (aig_conv_plan* p : plans) aig_conv_plan_destroy(p);
  cudaFree(pl->q);
  cudaFree(pl->k);
  cudaFree(pl->v);
  cudaFree(pl->ctxbuf);
  cudaFree(pl->kcache);
  cudaFree(pl->vcache);
  cudaFree(pl->rope);
  delete pl;
  return AIG_OK;
}

int aig_mha_plan_set_weights(aig_mha_plan* pl, const aig_half* wq, const aig_half* wk, const aig_half* wv, const aig_half* wo) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  AIG_REQUIRE(ctx, wq && wk && wv && wo, "mha set_weights: null pointer");
  const aig_half* w[4] = {wq, wk, wv, wo};
  aig_conv_plan* full[4] = {pl->pq, pl->pk, pl->pv, pl->po};
  aig_conv_plan* step[4] = {pl->sq, pl->sk, pl->sv, pl->so};
  for (int i = 0; i < 4; ++i) {
    int rc = aig_fc_plan_set_weights(full[i], w[i], nullptr, nullptr, nullptr, nullptr, nullptr, 0.f);
    if (rc == AIG_OK) rc = aig_fc_plan_set_weights(step[i], w[i], nullptr, nullptr, nullptr, nullptr, nullptr, 0.f);
    if (rc != AIG_OK) return rc;
  }
  pl->weights_set = true;
  return AIG_OK;
}

int aig_mha_forward(aig_mha_plan* pl, const aig_half* x, aig_half* y, int pos0) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, x && y && pl->weights_set, "mha forward: null pointer or weights not set");
  int rc;
  if ((rc = aig_conv_forward(pl->pq, x, nullptr, (aig_half*)pl->q)) != AIG_OK) return rc;
  if ((rc = aig_conv_forward(pl->pk, x, nullptr, (aig_half*)pl->k)) != AIG_OK) return rc;
  if ((rc = aig_conv_forward(pl->pv, x, nullptr, (aig_half*)pl->v)) != AIG_OK) return rc;
  AttnParams prm{};
  prm.B = pl->B; prm.T = pl->T; prm.E = pl->E; prm.heads = pl->heads; prm.window = pl->window;
  prm.scale = 1.0f / sqrtf((float)pl->d);
  prm.ctx = pl->ctxbuf;
  prm.gerr = ctx->d_err;
  prm.rope = nullptr;
  if (pl->rope_base > 0.f) {
    const int n = pl->T * (kD / 2);
    rope_table_kernel<<<ceil_div(n, 128), 128, 0, ctx->stream>>>(pl->rope, pl->T, kD / 2, kD, pl->rope_base, pos0);
    AIG_LAUNCH_OK(ctx);
    prm.rope = pl->rope;
  }
  rc = pl->T <= 64 ? launch_attention<64>(pl, prm) : launch_attention<128>(pl, prm);
  if (rc != AIG_OK) return rc;
  return aig_conv_forward(pl->po, (const aig_half*)pl->ctxbuf, nullptr, y);
}

int aig_mha_reset(aig_mha_plan* pl) {
  if (!pl) return AIG_ERR_INVALID;
  pl->stream_start = -1;
  return AIG_OK;
}

int aig_mha_step(aig_mha_plan* pl, const aig_half* x, aig_half* y, int position) {
  if (!pl) return AIG_ERR_INVALID;
  aig_ctx* ctx = pl->ctx;
  DeviceGuard g(ctx->device);
  AIG_REQUIRE(ctx, x && y && pl->weights_set && position >= 0, "mha step: bad arguments or weights not set");
  if (pl->stream_start < 0) pl->stream_start = position;
  AIG_REQUIRE(ctx, position >= pl->stream_start, "mha step: positions must not go backwards without aig_mha_reset");
  int n_valid = position - pl->stream_start + 1;
  if (n_valid > pl->ring) n_valid = pl->ring;
  int rc;
  // the per-step projections reuse the head of the sequence buffers: [B][E]
  if ((rc = aig_conv_forward(pl->sq, x, nullptr, (aig_half*)pl->q)) != AIG_OK) return rc;
  if ((rc = aig_conv_forward(pl->sk, x, nullptr, (aig_half*)pl->k)) != AIG_OK) return rc;
  if ((rc = aig_conv_forward(pl->sv, x, nullptr, (aig_half*)pl->v)) != AIG_OK) return rc;
  const int warps = 4;
  const int items = pl->B * pl->heads;
  const size_t smem = (size_t)warps * (pl->d + pl->ring) * sizeof(float);
  attention_step_kernel<<<ceil_div(items, warps), warps * 32, smem, ctx->stream>>>(
      pl->q, pl->k, pl->v, pl->kcache, pl->vcache, pl->ctxbuf, pl->B, pl->E, pl->heads, pl->d, pl->ring, position, n_valid,
      pl->rope_base, 1.0f / sqrtf((float)pl->d));
  AIG_LAUNCH_OK(ctx);
  return aig_conv_forward(pl->so, (const aig_half*)pl->ctxbuf, nullptr, y);
}

}  // extern "C"
