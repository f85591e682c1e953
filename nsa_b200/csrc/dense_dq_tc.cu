// dQ of the dense branches on tcgen05 (head_dim 128): sliding-window attention (mode 0) and compressed attention
// (mode 1).  Semantics of parallel_nsa_bwd_kernel_dq's window half (nsa/selection_attn.py:358-398) and of
// _attn_bwd_only_dq (nsa/triton_attention.py:321-416); same arguments and results as launch_dense_dq.
//
// A persistent CTA owns 8 consecutive tokens x 16 heads = [128 x 128] tiles of Q and dO (resident for the item).
// [128 keys x 128] K and V tiles stream through a 2-stage ring.  Per tile one thread issues
//     S  = Q . K^T,   dP = dO . V^T        (accumulators in TMEM)
// eight soft-max warps (half a row of 64 key columns per thread; lse, delta, gate and the mask are thread-local)
// form  dS = P (g dP - delta)  with  P = exp(scale S - lse)  and store it as a bf16 tile, and the thread issues
//     dQ += dS . K                          (A = dS from shared memory, B = K as an MN-major operand)
// S/dP of tile i+1 are issued as soon as the soft-max warps hold tile i in registers, before dQ of tile i: a soft-max
// thread fetches all 64 + 64 values of its half row first and hands the accumulators back at once, so those MMAs run
// under the whole soft-max of tile i.  That needs about 220 registers in the soft-max warps: the CTA has three
// warpgroups (warps 0-3: TMA, MMA and two idle warps; warps 4-11 soft-max) and redistributes registers with setmaxnreg.
#include "kernels.h"
#include "tc.cuh"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int D = 128;
constexpr int kTok = 8;
constexpr int kThreads = 384;                 // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-11 soft-max
constexpr int kSoft = 256;
constexpr uint32_t PANEL = 128 * 128;         // [128 rows][64 columns] bf16
constexpr uint32_t TILE = 2 * PANEL;          // 32 KB
constexpr uint32_t STAGE = 2 * TILE;          // K + V
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 512;           // S 0..127, dP 128..255, dQ 256..383
constexpr uint32_t kSmem = 2 * TILE + kStages * STAGE + TILE + 256 + 1024 + 1024;   // + [2][128] floats of the row pre-pass

struct Sched {
  int first, n;
};

template <int MODE>
__device__ __forceinline__ Sched make_sched(const DenseArgs& a, int t0) {
  Sched s;
  const int tmax = min(a.q0 + a.Tq - 1, t0 + kTok - 1);   // t0 is a sequence position
  if (MODE == 0) {
    s.first = max(0, t0 - a.window + 1) / 128;
    s.n = tmax / 128 - s.first + 1;
  } else {
    int nvis = a.Lk;
    if (a.causal) nvis = (tmax < a.cblock) ? 0 : min(a.Lk, (tmax - a.cblock) / a.cstride + 1);
    s.first = 0;
    s.n = (nvis + 127) / 128;
  }
  return s;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    dense_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                       const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const DenseArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_s = sbase, do_s = sbase + TILE, ring = sbase + 2 * TILE, ds_s = ring + kStages * STAGE;
  const uint32_t misc = ds_s + TILE;
  const uint32_t q_full = misc, q_free = misc + 8, full0 = misc + 16, empty0 = misc + 32, sdp_full = misc + 48,
                 sdp_free = misc + 56, ds_full = misc + 64, ds_free = misc + 72, dq_full = misc + 80, dq_free = misc + 88,
                 tmem_slot = misc + 96;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + (misc - sbase) + 104);
  float* xpre = reinterpret_cast<float*>(sgen + (misc - sbase) + 256);   // [2 branches][128 rows] exchange of the row pre-pass
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, kSoft);
    mbar_init(ds_full, kSoft);
    mbar_init(ds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, kSoft);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sgen + (tmem_slot - sbase));

  const int HG = a.Hq / 16;
  const int G16 = (a.Hq / a.Hk) / 16;
  const int ntile = (a.Tq + kTok - 1) / kTok;
  const long long total = (long long)a.B * HG * ntile;

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------------
    uint32_t c = 0, ic = 0;
    bool alive = true;
    for (long long item = blockIdx.x; alive && item < total; item += gridDim.x, ++ic) {
      const int hg = (int)(item % HG);
      const int tile = ntile - 1 - (int)((item / HG) % ntile);
      const int b = (int)(item / ((long long)HG * ntile));
      const int hk = hg / G16;
      const int t0l = tile * kTok;             // first local query row of the item
      const Sched sc = make_sched<MODE>(a, a.q0 + t0l);
      int good = 1;
      if (lane == 0) {
        good = mbar_wait_abortable(q_free, (ic & 1) ^ 1, 201, abort_flag) ? 1 : 0;
        if (good) mbar_expect_tx(q_full, 2 * TILE);
      }
      if (!__shfl_sync(0xffffffffu, good, 0)) break;
      if (lane < 4) {
        const int p = lane & 1;
        const CUtensorMap* tm = (lane & 2) ? &tmDO : &tmQ;
        const uint32_t dst = ((lane & 2) ? do_s : q_s) + p * PANEL;
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(dst), "l"(tm), "r"(q_full), "r"(p * 64), "r"(hg * 16), "r"(b * a.Tq + t0l)
            : "memory");
      }
      for (int i = 0; i < sc.n; ++i, ++c) {
        const int jt = sc.first + i;
        const int stage = c & 1;
        if (lane == 0) {
          good = mbar_wait_abortable(empty0 + 8 * stage, ((c >> 1) & 1) ^ 1, 202, abort_flag) ? 1 : 0;
          if (good) mbar_expect_tx(full0 + 8 * stage, STAGE);
        }
        if (!__shfl_sync(0xffffffffu, good, 0)) {
          alive = false;
          break;
        }
        if (lane < 4) {
          const uint32_t dst = ring + stage * STAGE;
          const int p = lane >> 1;
          if (lane & 1)
            tma_load_4d(dst + TILE + p * PANEL, &tmV, full0 + 8 * stage, p * 64, hk, jt * 128, b);
          else
            tma_load_4d(dst + p * PANEL, &tmK, full0 + 8 * stage, p * 64, hk, jt * 128, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 128, 0, 1);
      uint32_t c = 0, ic = 0;
      bool ok = true;
      // operand descriptors are built once; an MMA then costs one 64-bit add per operand
      const uint64_t dq_desc = umma_smem_desc(q_s, 0, 1024), ddo_desc = umma_smem_desc(do_s, 0, 1024);
      const uint64_t dds_desc = umma_smem_desc(ds_s, 0, 1024);
      const uint64_t dk_desc0 = umma_smem_desc(ring, 0, 1024), dk_desc1 = umma_smem_desc(ring + STAGE, 0, 1024);
      const uint64_t dv_desc0 = umma_smem_desc(ring + TILE, 0, 1024), dv_desc1 = umma_smem_desc(ring + STAGE + TILE, 0, 1024);
      const uint64_t dkmn_desc0 = umma_smem_desc(ring, PANEL, 1024), dkmn_desc1 = umma_smem_desc(ring + STAGE, PANEL, 1024);
      for (long long item = blockIdx.x; ok && item < total; item += gridDim.x, ++ic) {
        const int tile = ntile - 1 - (int)((item / HG) % ntile);
        const Sched sc = make_sched<MODE>(a, a.q0 + tile * kTok);
        ok = mbar_wait_abortable(q_full, ic & 1, 203, abort_flag);
        // dQ of the previous item must have been read, and dq_full must not complete twice unseen
        if (ok && ic > 0) ok = mbar_wait_abortable(dq_free, (ic - 1) & 1, 204, abort_flag);
        auto issue_sdp = [&](uint32_t cc) {
          const uint64_t dk = (cc & 1) ? dk_desc1 : dk_desc0, dv = (cc & 1) ? dv_desc1 : dv_desc0;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * PANEL + (ks & 3) * 32;
            umma_ss(tmem + 0, umma_desc_advance(dq_desc, off), umma_desc_advance(dk, off), idesc_s, ks ? 1u : 0u);
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * PANEL + (ks & 3) * 32;
            umma_ss(tmem + 128, umma_desc_advance(ddo_desc, off), umma_desc_advance(dv, off), idesc_s, ks ? 1u : 0u);
          }
          umma_commit(sdp_full);
        };
        // Event loop: S/dP of tile `ns` as soon as its stage has landed and the soft-max warps hold the previous
        // tile's S/dP in registers; dQ of tile `nd` as soon as its dS tile is written -- whichever is ready first.
        const uint32_t c0 = c;
        int ns = 0, nd = 0;
        uint64_t t_idle = 0;
        while (ok && nd < sc.n) {
          bool progressed = false;
          if (ns < sc.n) {
            const uint32_t cc = c0 + ns;
            if (mbar_test(full0 + 8 * (cc & 1), (cc >> 1) & 1) && (cc == 0 || mbar_test(sdp_free, (cc - 1) & 1))) {
              tc_fence_after();
              issue_sdp(cc);
              if (ns == sc.n - 1) umma_commit(q_free);   // every S/dP of the item issued: Q and dO may be reloaded after them
              ++ns;
              progressed = true;
            }
          }
          if (nd < ns) {
            const uint32_t cc = c0 + nd;
            if (mbar_test(ds_full, cc & 1)) {
              tc_fence_after();
              const uint64_t dkm = (cc & 1) ? dkmn_desc1 : dkmn_desc0;
#pragma unroll
              for (int ks = 0; ks < 8; ++ks)
                umma_ss(tmem + 256, umma_desc_advance(dds_desc, (ks >> 2) * PANEL + (ks & 3) * 32),
                        umma_desc_advance(dkm, ks * 2048), idesc_dq, (nd | ks) ? 1u : 0u);
              umma_commit(empty0 + 8 * (cc & 1));
              umma_commit(ds_free);
              ++nd;
              progressed = true;
            }
          }
          if (progressed) {
            t_idle = 0;
          } else {   // bounded: the abort flag of another role, or ~2 s without progress, ends the loop
            if (*abort_flag) ok = false;
            const uint64_t now = global_timer_ns();
            if (t_idle == 0) t_idle = now;
            else if (now - t_idle > 2000000000ull) {
              atomicCAS(&g_dev_error, 0, 205);
              *abort_flag = 1;
              ok = false;
            }
          }
        }
        c = c0 + sc.n;
        if (sc.n == 0) umma_commit(q_free);
        umma_commit(dq_full);
      }
    }
  }
  } else {
    // ------------------------------- soft-max warps ------------------------------------------------
    // budget: the CTA is launched with 384 x 168 = 64512 registers; 128 x 72 + 256 x 216 = 64512 (an inc that the launch
    // pool cannot satisfy blocks for ever)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;
    const int row = 32 * quad + lane;
    const int tl = row >> 4, head = row & 15;
    const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
    const float sl2 = a.scale * kLog2e;
    uint32_t c = 0, ic = 0;
    bool ok = true;
    for (long long item = blockIdx.x; item < total; item += gridDim.x, ++ic) {
      const int hg = (int)(item % HG);
      const int tile = ntile - 1 - (int)((item / HG) % ntile);
      const int b = (int)(item / ((long long)HG * ntile));
      const int t0l = tile * kTok;
      const int tloc = t0l + tl;               // local query row
      const int t = a.q0 + tloc;               // its sequence position
      const bool live = tloc < a.Tq;
      const Sched sc = make_sched<MODE>(a, a.q0 + t0l);
      int nvis = a.Lk;
      if (MODE == 1 && a.causal) nvis = (t < a.cblock) ? 0 : min(a.Lk, (t - a.cblock) / a.cstride + 1);
      const long long qrow = ((long long)b * a.Tq + (live ? tloc : 0)) * a.Hq + hg * 16 + head;
      const float lse2 = a.lse[qrow] * kLog2e;
      const float gv = a.gate ? __bfloat162float(a.gate[qrow]) : 1.f;
      float del;
      if (a.pre_o[0]) {
        // Row pre-pass folded in (parallel_nsa_bwd_kernel_preprocess, nsa/selection_attn.py:520-530; _attn_bwd_preprocess,
        // nsa/triton_attention.py:184-199; the gate gradients of nsa/nsa.py:133): rowsum(o_x * dO) over this thread's 64
        // channels, the two halves of a row meet in shared memory, the first half finishes and publishes the row's delta.
        float part[2] = {0.f, 0.f};
        const uint4* pd = reinterpret_cast<const uint4*>(a.dout + qrow * D + half * 64);
        uint4 dv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) dv[e] = pd[e];
#pragma unroll
        for (int br = 0; br < 2; ++br) {
          if (!a.pre_o[br]) continue;
          const uint4* po = reinterpret_cast<const uint4*>(a.pre_o[br] + qrow * D + half * 64);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const uint4 ov = po[e];
            const __nv_bfloat162* ho2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
            const __nv_bfloat162* hd2 = reinterpret_cast<const __nv_bfloat162*>(&dv[e]);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float2 x = __bfloat1622float2(ho2[u]), y = __bfloat1622float2(hd2[u]);
              part[br] = fmaf(x.x, y.x, fmaf(x.y, y.y, part[br]));
            }
          }
        }
        if (half == 1) {
          xpre[row] = part[0];
          xpre[128 + row] = part[1];
        }
        named_bar_sync(1, kSoft);
        if (half == 0) {
          float own = 0.f;
#pragma unroll
          for (int br = 0; br < 2; ++br) {
            if (!a.pre_o[br]) continue;
            const float tot = part[br] + xpre[br * 128 + row];
            const float gb = a.pre_gate[br] ? __bfloat162float(a.pre_gate[br][qrow]) : 1.f;
            if (live) {
              a.pre_delta[br][qrow] = gb * tot;
              if (a.pre_dgate[br]) a.pre_dgate[br][qrow] = __float2bfloat16(tot);
            }
            if (br == 0) own = gb * tot;
          }
          xpre[row] = own;
          del = own;
        }
        named_bar_sync(1, kSoft);
        if (half == 1) del = xpre[row];
      } else {
        del = a.delta[qrow];
      }
      const bool dead = !live || !(lse2 > -INFINITY);
      // the row's previous dq (accumulate mode) is fetched now, so its latency hides behind the tile loop instead of
      // stalling the epilogue (measured: ~1000 of ~5000 cycles per tile)
      uint4 outv[8];
      bf16* dst = a.dq + qrow * D + half * 64;
      if (a.accumulate && live) {
#pragma unroll
        for (int e = 0; e < 8; ++e) outv[e] = reinterpret_cast<const uint4*>(dst)[e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) outv[e] = make_uint4(0u, 0u, 0u, 0u);
      }
      for (int i = 0; i < sc.n; ++i, ++c) {
        const int j0 = (sc.first + i) * 128 + half * 64;
        ok = mbar_wait_abortable(sdp_full, c & 1, 208, abort_flag) && ok;
        tc_fence_after();
        int lo = 0, hi = 64;
        if (MODE == 0) {
          lo = max(0, t - a.window + 1 - j0);
          hi = min(64, t + 1 - j0);
        } else {
          hi = min(64, nvis - j0);
        }
        if (dead) hi = 0;
        const bool full = lo <= 0 && hi >= 64;
        uint32_t dw[32];
        const float nl = -lse2;
        float s[64], dp[64];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          tmem_ld16(tmem + lane_addr + half * 64 + q4 * 16, *reinterpret_cast<float(*)[16]>(&s[q4 * 16]));
          tmem_ld16(tmem + lane_addr + 128 + half * 64 + q4 * 16, *reinterpret_cast<float(*)[16]>(&dp[q4 * 16]));
        }
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(sdp_free);   // S and dP of this tile are in registers: the next tile's products may overwrite them
        if (full) {
#pragma unroll
          for (int e = 0; e < 64; e += 2) {
            const float p0 = ex2(fmaf(s[e], sl2, nl)), p1 = ex2(fmaf(s[e + 1], sl2, nl));
            dw[e >> 1] = pack_bf16(p0 * fmaf(gv, dp[e], -del), p1 * fmaf(gv, dp[e + 1], -del));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 64; e += 2) {
            const float p0 = (e >= lo && e < hi) ? ex2(fmaf(s[e], sl2, nl)) : 0.f;
            const float p1 = (e + 1 >= lo && e + 1 < hi) ? ex2(fmaf(s[e + 1], sl2, nl)) : 0.f;
            dw[e >> 1] = pack_bf16(p0 * fmaf(gv, dp[e], -del), p1 * fmaf(gv, dp[e + 1], -del));
          }
        }
        if (c > 0) ok = mbar_wait_abortable(ds_free, (c - 1) & 1, 209, abort_flag) && ok;   // dQ of the previous tile read dS
        uint8_t* drow = sgen + (ds_s - sbase) + half * PANEL + row * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(drow + ((ch ^ (row & 7)) << 4)) =
              make_uint4(dw[4 * ch], dw[4 * ch + 1], dw[4 * ch + 2], dw[4 * ch + 3]);
        fence_proxy_async();
        mbar_arrive(ds_full);
      }
      // ---- epilogue: dq = scale * dQ (+ previous contents) --------------------------------------------
      ok = mbar_wait_abortable(dq_full, ic & 1, 210, abort_flag) && ok;
      tc_fence_after();
      __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(outv);
      if (sc.n > 0) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float o[16];
          tmem_ld16(tmem + lane_addr + 256 + half * 64 + q4 * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 prev = __bfloat1622float2(ho[q4 * 8 + e]);
            ho[q4 * 8 + e] = __floats2bfloat162_rn(fmaf(o[2 * e], a.scale, prev.x), fmaf(o[2 * e + 1], a.scale, prev.y));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(dq_free);
      if (live && ok) {
#pragma unroll
        for (int e = 0; e < 8; ++e) reinterpret_cast<uint4*>(dst)[e] = outv[e];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

template <int MODE>
int launch(const DenseArgs& a, cudaStream_t s) {
  CUtensorMap tmQ, tmDO, tmK, tmV;
  const unsigned long long qd[3] = {(unsigned long long)D, (unsigned long long)a.Hq, (unsigned long long)a.B * a.Tq};
  const unsigned long long qs[2] = {(unsigned long long)D * 2, (unsigned long long)a.Hq * D * 2};
  const unsigned qb[3] = {64, 16, (unsigned)kTok};
  int rc = make_tmap_generic(&tmQ, a.q, 3, qd, qs, qb);
  if (!rc) rc = make_tmap_generic(&tmDO, a.dout, 3, qd, qs, qb);
  if (!rc) rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.Lk, a.B, 128);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.Lk, a.B, 128);
  if (rc) return rc;
  auto kern = dense_dq_tc_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * (a.Hq / 16) * ((a.Tq + kTok - 1) / kTok);
  const int grid = (int)(total < num_sms() ? total : num_sms());
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, kSmem, s>>>(tmQ, tmDO, tmK, tmV, a);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

// head_dim 128 only; the caller falls back to launch_dense_dq otherwise.
int launch_dense_dq_tc(const DenseArgs& a, cudaStream_t s) { return a.mode == 0 ? launch<0>(a, s) : launch<1>(a, s); }
int dense_dq_tc_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
