// aig_common.cuh -- context, status handling and sm_100a PTX wrappers shared by the kernels.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "aig_b200.h"

// ---------------------------------------------------------------------------------------------
// Context
struct aig_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int* d_err = nullptr;   // device error word written by kernels whose bounded waits expire
  int* h_err = nullptr;   // pinned mirror
  std::string last_error;
};

struct aig_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};

int aig_fail(aig_ctx* ctx, int code, const char* fmt, ...);

// FC plans whose weight operand is produced inside the library (igemm_tcgen05.cu): the K-major buffer
// [out_c][in_c] to write in place, the epilogue's fp32 shift [out_c] (the bias), and the identity epilogue folded once.
struct aig_conv_plan;
__half* fc_plan_weight_buffer(aig_conv_plan* plan);
float* fc_plan_shift_buffer(aig_conv_plan* plan);
int fc_plan_identity_affine(aig_conv_plan* plan);

#define AIG_CUDA_OK(ctx, expr)                                                             \
  do {                                                                                     \
    cudaError_t e__ = (expr);                                                              \
    if (e__ != cudaSuccess)                                                                \
      return aig_fail((ctx), AIG_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                      __FILE__, __LINE__);                                                 \
  } while (0)

#define AIG_LAUNCH_OK(ctx)                                                                 \
  do {                                                                                     \
    cudaError_t e__ = cudaGetLastError();                                                  \
    if (e__ != cudaSuccess)                                                                \
      return aig_fail((ctx), AIG_ERR_CUDA, "kernel launch failed: %s (%s:%d)",             \
                      cudaGetErrorString(e__), __FILE__, __LINE__);                        \
  } while (0)

#define AIG_REQUIRE(ctx, cond, ...)                                     \
  do {                                                                  \
    if (!(cond)) return aig_fail((ctx), AIG_ERR_INVALID, __VA_ARGS__);  \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------------------------
// Device helpers
#ifdef __CUDACC__

__device__ __forceinline__ float act_apply(float v, int act, float slope) {
  switch (act) {
    case AIG_ACT_RELU: return v > 0.f ? v : 0.f;
    case AIG_ACT_SWISH: return v / (1.0f + expf(-v));
    case AIG_ACT_LEAKY: return v < 0.f ? v * slope : v;
    default: return v;
  }
}

// Swish for the fused epilogues, whose result is rounded to fp16 anyway: v * sigmoid(v) = h + h * tanh(h) with
// h = v / 2 and the special-function unit's tanh.approx.f32 (relative error 2^-11 on tanh): ONE special-function
// operation per value instead of two (ex2 + rcp).  That unit issues 16 lanes per clock per SM and was the busiest
// pipe of the first-layer kernel (57 %) and a quarter of the narrow residual layers' epilogues.  The result is within
// |v| * 2.4e-4 of the exact value: at most one fp16 unit in the last place for v >= 0, below 1e-3 absolute for the
// negative tail.  (The stand-alone Swish operator, which is bit-exact with the reference's kernel, does not use this.)
__device__ __forceinline__ float swish_sfu(float v) {
  const float h = 0.5f * v;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}
__device__ __forceinline__ float act_apply_fast(float v, int act, float slope) {
  switch (act) {
    case AIG_ACT_RELU: return v > 0.f ? v : 0.f;
    case AIG_ACT_SWISH: return swish_sfu(v);
    case AIG_ACT_LEAKY: return v < 0.f ? v * slope : v;
    default: return v;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- programmatic dependent launch ----
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in
// the stream still runs: everything before griddep_wait() (barrier setup, TMEM allocation, loads of constant
// weights) overlaps the predecessor's tail; griddep_wait() returns once the predecessor has completed and
// its writes are visible.  Without the attribute both are no-ops.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait with a suspend-time hint: the thread may sleep in hardware up to `ns` nanoseconds (it wakes as soon
// as the phase completes), so a long wait costs a handful of instructions instead of a hot polling loop
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after ~AIG_WAIT_CYCLES SM cycles, raises the CTA-wide abort flag and the
// context's device error word, and returns false; every role then drains to the common exit.
#ifndef AIG_WAIT_CYCLES
#define AIG_WAIT_CYCLES (600ll * 1000 * 1000)  // ~0.3 s at 1.9 GHz
#endif
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* gerr, int code,
                                                long long limit_cycles) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1;
        atomicCAS(gerr, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* gerr, int code) {
  return mbar_wait_limit(bar, parity, abort_flag, gerr, code, AIG_WAIT_CYCLES);
}
// The same bound for roles that may sleep while they wait (producers far ahead, epilogue warps between tiles):
// every poll suspends up to ~2 us in hardware, the abort flag and the clock are checked on every wake-up.
__device__ __forceinline__ bool mbar_wait_bounded_sleepy(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* gerr, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > AIG_WAIT_CYCLES) {
      *abort_flag = 1;
      atomicCAS(gerr, 0, code);
      return false;
    }
  }
}

// ---- TMA (tiled mode; every CTA issues its own loads) ----
__device__ __forceinline__ void tma_prefetch_desc(const void* desc) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* desc, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// ---- tcgen05 / TMEM ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulate.  Issued by one thread.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same, with the descriptors given as their low words plus the one high word both share: for 128-byte
// rows the high word (stride, version, swizzle) is a constant and the low word is linear in the
// address, so an issue loop advances descriptors with one 32-bit add each.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ constexpr uint32_t umma_desc_hi(uint32_t row_bytes) {
  return ((row_bytes * 8u) >> 4) | (1u << 14) | ((row_bytes == 128 ? 2u : (row_bytes == 64 ? 4u : 6u)) << 29);
}
__device__ __forceinline__ void umma_f16_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// ---- TMA stores (shared -> global, bulk-group completion) and named barriers ----
__device__ __forceinline__ void named_bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void tma_store_2d(const void* desc, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(reinterpret_cast<uint64_t>(desc)), "r"(src),
               "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One lane of a converged warp (the same lane on every call).  A loop that all 32 lanes run with identical values
// and that issues tcgen05.mma / tcgen05.commit under this predicate keeps its address arithmetic in the warp's
// uniform registers, which is where those instructions take their operands from; a loop run by a single lane
// inside a divergent branch pays a vector-to-uniform register move for every operand of every instruction.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
// mbarrier arrives once all previously issued tcgen05.mma of this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane (base_lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- CTA pairs (clusters of two; tcgen05 cta_group::2) ----
// One tcgen05.mma.cta_group::2 computes a 256 x N tile over both CTAs of a pair: each CTA supplies 128 rows of A
// and N/2 rows of B from the SAME shared-memory offsets and receives its 128 rows of D at the same TMEM address.
// The instruction is issued by one thread of the pair's first CTA; barriers of the other CTA are reached through
// their cluster-window address (mapa).
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// arrive on a barrier given by its cluster-window address (own or the other CTA's)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cl(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait with cluster-scope acquire (the arrival may come from the other CTA of the pair)
__device__ __forceinline__ bool mbar_wait_bounded_cl(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                     int* gerr, int code) {
  if (mbar_try_wait_cl(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait_cl(bar, parity)) return true;
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > AIG_WAIT_CYCLES) {
        *abort_flag = 1;
        atomicCAS(gerr, 0, code);
        return false;
      }
    }
  }
}
// TMA loads of a CTA pair: the data lands in the issuing CTA's shared memory, the bytes are counted on a barrier
// given by its cluster-window address -- the first CTA's, so that the thread issuing the pair's MMAs waits on one
// barrier for both halves.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* desc, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_lo_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                                    uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on ONE barrier (cluster-window address: own CTA's or the other's) once the pair's MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are `row_bytes` wide
// (32, 64 or 128 bytes = one swizzle span) and packed densely: 8-row groups are row_bytes*8 apart.
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4 (unused here: 1)
//   bits [32,46) stride byte offset >> 4     bits [46,48) descriptor version = 1 (sm_100)
//   bits [61,64) swizzle: 2 = 128 B, 4 = 64 B, 6 = 32 B
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t row_bytes) {
  const uint64_t swz = row_bytes == 128 ? 2ull : (row_bytes == 64 ? 4ull : 6ull);
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)((row_bytes * 8u) >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= swz << 61;
  return d;
}
// Instruction descriptor, kind::f16: fp16 A/B (K-major both), fp32 accumulate, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

#endif  // __CUDACC__
