// Device-side primitives shared by every kernel of the library (sm_100a only).
//
//  * warp-level tensor-core tiles: mma.sync m16n8k16 (bf16 in, fp32 accumulate) fed by ldmatrix
//    from shared-memory tiles written by TMA with the 128-byte swizzle;
//  * mbarrier producer/consumer pipeline helpers.  Every wait is bounded: after about two
//    seconds it records an error code in a device flag and reports failure, so a kernel whose
//    pipeline is broken returns instead of hanging the GPU;
//  * TMA (cp.async.bulk.tensor) loads of 2-D/4-D boxes and plain bulk copies.  No load here uses
//    cluster multicast.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

typedef __nv_bfloat16 bf16;

// One flag per translation unit; api.cu gathers them through the *_status() accessors.
static __device__ int g_dev_error = 0;

enum DevError { DEV_OK = 0, DEV_ERR_FULL_WAIT = 1, DEV_ERR_EMPTY_WAIT = 2, DEV_ERR_BOUNDS = 3 };

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------------------------------------
// mma.sync / ldmatrix
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// A shared-memory operand tile is ROWS rows of D bf16, stored as D/64 column panels; a panel is
// [ROWS][64] bf16 (128-byte rows) with the 128-byte TMA swizzle: the 16-byte chunk c of row r sits
// at chunk position c ^ (r & 7).  Panel bases are 1024-byte aligned.  `panel_bytes` = ROWS * 128.
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, uint32_t panel_bytes, int row, int chunk) {
  return base + (chunk >> 3) * panel_bytes + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// acc[16 x NK] += A[16 x D] * Tile[row0 .. row0+NK)[D]^T   (contraction over the D columns).
// A is held as mma A-fragments af[D/16][4]; the tile rows play the n index.
template <int D, int NK>
__device__ __forceinline__ void mma_a_bt(float (&acc)[NK / 8][4], const uint32_t (&af)[D / 16][4], uint32_t base,
                                         uint32_t panel_bytes, int row0, int lane) {
  const int m = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int n2 = 0; n2 < NK / 16; ++n2) {
    const int row = row0 + n2 * 16 + (m >> 1) * 8 + rr;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(tile_addr(base, panel_bytes, row, ks * 2 + (m & 1)), b0, b1, b2, b3);
      mma_bf16(acc[2 * n2], af[ks], b0, b1);
      mma_bf16(acc[2 * n2 + 1], af[ks], b2, b3);
    }
  }
}

// acc[16 x D] += P[16 x NK] * Tile[row0 .. row0+NK)[D]       (contraction over the tile rows).
// P is held as mma A-fragments pf[NK/16][4]; the tile columns play the n index.
template <int D, int NK>
__device__ __forceinline__ void mma_a_b(float (&acc)[D / 8][4], const uint32_t (&pf)[NK / 16][4], uint32_t base,
                                        uint32_t panel_bytes, int row0, int lane) {
  const int m = lane >> 3, rr = lane & 7;
#pragma unroll
  for (int kk = 0; kk < NK / 16; ++kk) {
    const int row = row0 + kk * 16 + (m & 1) * 8 + rr;
#pragma unroll
    for (int n2 = 0; n2 < D / 16; ++n2) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(tile_addr(base, panel_bytes, row, n2 * 2 + (m >> 1)), b0, b1, b2, b3);
      mma_bf16(acc[2 * n2], pf[kk], b0, b1);
      mma_bf16(acc[2 * n2 + 1], pf[kk], b2, b3);
    }
  }
}

// Same as mma_a_bt<D,16> but with the contraction split over two accumulator sets (even / odd k-steps): four
// independent mma chains instead of two, which halves the exposed tensor-pipe latency when a warp has no
// other work to overlap.
template <int D>
__device__ __forceinline__ void mma_a_bt16_split(float (&acc)[2][4], const uint32_t (&af)[D / 16][4], uint32_t base,
                                                 uint32_t panel_bytes, int row0, int lane) {
  const int m = lane >> 3, rr = lane & 7;
  const int row = row0 + (m >> 1) * 8 + rr;
  float odd[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i) odd[i][0] = odd[i][1] = odd[i][2] = odd[i][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ks += 2) {
    uint32_t b0, b1, b2, b3, c0, c1, c2, c3;
    ldsm_x4(tile_addr(base, panel_bytes, row, ks * 2 + (m & 1)), b0, b1, b2, b3);
    ldsm_x4(tile_addr(base, panel_bytes, row, ks * 2 + 2 + (m & 1)), c0, c1, c2, c3);
    mma_bf16(acc[0], af[ks], b0, b1);
    mma_bf16(acc[1], af[ks], b2, b3);
    mma_bf16(odd[0], af[ks + 1], c0, c1);
    mma_bf16(odd[1], af[ks + 1], c2, c3);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] += odd[i][c];
}

// Load the A-fragments of 16 rows [row0, row0+16) x D of a swizzled shared tile.
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t (&af)[D / 16][4], uint32_t base, uint32_t panel_bytes,
                                             int row0, int lane) {
  const int m = lane >> 3, rr = lane & 7;
  const int row = row0 + (m & 1) * 8 + rr;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldsm_x4(tile_addr(base, panel_bytes, row, ks * 2 + (m >> 1)), af[ks][0], af[ks][1], af[ks][2], af[ks][3]);
}

// A-fragments of a [16 x D] row-major bf16 matrix in global memory (row stride D elements).
template <int D>
__device__ __forceinline__ void load_a_frags_global(uint32_t (&af)[D / 16][4], const bf16* __restrict__ p, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const uint32_t* r0 = reinterpret_cast<const uint32_t*>(p + (size_t)g * D);
  const uint32_t* r1 = reinterpret_cast<const uint32_t*>(p + (size_t)(g + 8) * D);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    af[ks][0] = __ldg(r0 + ks * 8 + t);
    af[ks][1] = __ldg(r1 + ks * 8 + t);
    af[ks][2] = __ldg(r0 + ks * 8 + 4 + t);
    af[ks][3] = __ldg(r1 + ks * 8 + 4 + t);
  }
}

// Accumulator tile [16 x 8*N] (mma C layout) -> A-fragments of the same 16 rows (bf16).
template <int NT>
__device__ __forceinline__ void acc_to_a_frags(uint32_t (&pf)[NT / 2][4], const float (&c)[NT][4]) {
#pragma unroll
  for (int k = 0; k < NT / 2; ++k) {
    pf[k][0] = pack_bf16(c[2 * k][0], c[2 * k][1]);
    pf[k][1] = pack_bf16(c[2 * k][2], c[2 * k][3]);
    pf[k][2] = pack_bf16(c[2 * k + 1][0], c[2 * k + 1][1]);
    pf[k][3] = pack_bf16(c[2 * k + 1][2], c[2 * k + 1][3]);
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// ---------------------------------------------------------------------------------------------
// mbarrier + TMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase.  mbarrier.try_wait may suspend the thread for a system-dependent time when the phase is
// not complete; a thread that polls SEVERAL barriers (the MMA issuer's event loop, a producer that serves two rings)
// must not sleep on one of them while another is ready, so such loops use test_wait.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) if the phase did not complete in ~2 s.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (global_timer_ns() - t0 > 2000000000ull) {
      atomicCAS(&g_dev_error, 0, code);   // keep the first failure
      return false;
    }
  }
}
// The same with a CTA-wide abort flag in shared memory: once any wait of the CTA has given up, every later wait
// returns false at once, so roles that must keep meeting at named barriers can run their loops to the end without
// waiting (their results are discarded) instead of leaving a partner stuck at a barrier.
__device__ __forceinline__ bool mbar_wait_abortable(uint32_t bar, uint32_t parity, int code, volatile int* abort_flag) {
  if (*abort_flag) return false;
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > 2000000000ull) {
      atomicCAS(&g_dev_error, 0, code);
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          dst),
      "l"(tm), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(dst),
      "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Bulk copy shared -> global (asynchronous, tracked by the issuing thread's bulk groups); both addresses 16-byte
// aligned, bytes a multiple of 16.  The shared-memory writes it reads must be ordered before it by fence_proxy_async.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
// The same with an L2 evict-first policy: data that is written once and read once much later should not displace
// lines other CTAs are about to re-read.
__device__ __forceinline__ void bulk_store_evict_first(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile(
      "{ .reg .b64 pol; createpolicy.fractional.L2::evict_first.b64 pol, 1.0;\n"
      "cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, pol; }" ::"l"(dst),
      "r"(src), "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All of this thread's bulk stores have read their shared-memory source (it may be overwritten).
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All but the most recent of this thread's bulk-store groups have read their source.
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// All of this thread's bulk stores are complete.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Plain bulk copy global -> shared; src/dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// online softmax over one score slice held in mma C layout (rows g and g+8 of 16)
// ---------------------------------------------------------------------------------------------
struct RowState {
  float m[2];  // running max (log2 domain)
  float l[2];  // running sum
};

}  // namespace nsa
