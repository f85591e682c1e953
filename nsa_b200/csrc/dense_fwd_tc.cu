// Dense query-major attention FORWARD on tcgen05 (head_dim 128): sliding-window attention (mode 0) and compressed
// attention with the fused block selection (mode 1).  Same semantics and results layout as dense_attn.cu
// (nsa/selection_attn.py:484-516; nsa/triton_attention.py:87-181,465-475; scoring of nsa/torch_attention.py:121-125).
//
// A persistent CTA owns 8 consecutive tokens x the 16 heads of a GQA group = one [128 x 128] Q tile (a single 3-D
// TMA box per 64-column panel).  [128 keys x 128] K and V tiles stream through a 2-stage mbarrier ring.  One
// thread issues  S = Q.K^T  (M=N=K=128, accumulator in TMEM, two S buffers) and  O += P.V  (A = P from shared
// memory, B = V as an MN-major operand).  Eight soft-max warps own half a row per thread (64 of the 128 key
// columns of their TMEM lane): masks, running max and sum are thread-local; the two halves of a row exchange only
// their tile maximum through shared memory.  O is rescaled in TMEM only when some row's maximum moved.
// S of tile i+1 is issued before P.V of tile i, so the tensor core overlaps the soft-max.
//
// Selection (mode 1): a first pass over all compressed tiles collects the statistics of the unscaled, unmasked
// soft-max while the causal tiles also feed the attention; a second pass recomputes S, forms p / l, pools the 5-wide
// stride-4 windows inside the thread, sums the 16 heads with warp shuffles and accumulates a per-token score vector
// in shared memory; eight warps then pick the top n of their token (ties to the lower block index).
#include "kernels.h"
#include "tc.cuh"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int D = 128;
constexpr int kTok = 8;
constexpr int kThreads = 320;                 // warp 0 TMA, warp 1 MMA, warps 2-9 soft-max
constexpr int kSoft = 256;
constexpr uint32_t PANEL = 128 * 128;         // [128 rows][64 columns] bf16
constexpr uint32_t TILE = 2 * PANEL;          // 32 KB
constexpr uint32_t STAGE = 2 * TILE;          // K + V
constexpr int kStages = 2;
constexpr uint32_t kTmemCols = 512;           // S0 0..127, S1 128..255, O 256..383
constexpr int kMaxPool = 1024;

struct Sched {
  int first, nA, nAttn, nB;
};

template <int MODE>
__device__ __forceinline__ Sched make_sched(const DenseArgs& a, int t0) {
  Sched s;
  const int tmax = min(a.q0 + a.Tq - 1, t0 + kTok - 1);   // t0 is a sequence position
  if (MODE == 0) {
    s.first = max(0, t0 - a.window + 1) / 128;
    s.nA = tmax / 128 - s.first + 1;
    s.nAttn = s.nA;
    s.nB = 0;
  } else {
    const int nt_all = (a.Lk + 127) / 128;
    int nvis = a.Lk;
    if (a.causal) nvis = (tmax < a.cblock) ? 0 : min(a.Lk, (tmax - a.cblock) / a.cstride + 1);
    s.first = 0;
    s.nAttn = (nvis + 127) / 128;
    const bool sel = a.n_sel > 0;
    s.nA = sel ? nt_all : s.nAttn;
    s.nB = sel ? nt_all : 0;
  }
  return s;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    dense_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const DenseArgs a, const int pool_floats,
                        const int smem_bytes) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_s = sbase, ring = sbase + TILE, p_s = ring + kStages * STAGE;
  const uint32_t misc = p_s + TILE;
  // misc: barriers (16 x 8 B), tmem slot, exchange buffers, pooled scores
  const uint32_t q_full = misc, q_free = misc + 8, full0 = misc + 16, empty0 = misc + 32, s_full0 = misc + 48,
                 s_free0 = misc + 64, p_full = misc + 80, p_free = misc + 88, o_full = misc + 96, tmem_slot = misc + 104, o_free = misc + 120;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + (misc - sbase) + 112);
  float* xch = reinterpret_cast<float*>(sgen + (misc - sbase) + 128);  // [2 parity][2 half][128 rows]
  float* xst = xch;                                                     // statistics merge reuses it (see below)
  float* pool = xch + 2 * 2 * 128;                                      // [kTok][pool_floats]
  // the layout must fit behind the 1024-byte round-up of the base (the host leaves less slack for long sequences)
  if ((misc - raw) + 128 + 2 * 2 * 128 * 4 + kTok * pool_floats * 4 > (uint32_t)smem_bytes) {
    if (threadIdx.x == 0) atomicCAS(&g_dev_error, 0, DEV_ERR_BOUNDS);
    return;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, 1);
      mbar_init(s_full0 + 8 * i, 1);
      mbar_init(s_free0 + 8 * i, kSoft);
    }
    mbar_init(p_full, kSoft);
    mbar_init(p_free, 1);
    mbar_init(o_full, 1);
    mbar_init(o_free, kSoft);
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
  const bool do_sel = MODE == 1 && a.n_sel > 0;

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
        good = mbar_wait_abortable(q_free, (ic & 1) ^ 1, 101, abort_flag) ? 1 : 0;
        if (good) mbar_expect_tx(q_full, TILE);
      }
      if (!__shfl_sync(0xffffffffu, good, 0)) break;
      if (lane < 2) {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(q_s + lane * PANEL), "l"(&tmQ), "r"(q_full), "r"(lane * 64), "r"(hg * 16), "r"(b * a.Tq + t0l)
            : "memory");
      }
      for (int i = 0; i < sc.nA + sc.nB; ++i, ++c) {
        const bool withv = i < sc.nAttn;
        const int jt = sc.first + (i < sc.nA ? i : i - sc.nA);
        const int stage = c & 1;
        if (lane == 0) {
          good = mbar_wait_abortable(empty0 + 8 * stage, ((c >> 1) & 1) ^ 1, 102, abort_flag) ? 1 : 0;
          if (good) mbar_expect_tx(full0 + 8 * stage, withv ? STAGE : TILE);
        }
        if (!__shfl_sync(0xffffffffu, good, 0)) {
          alive = false;
          break;
        }
        if (lane < 4) {
          const uint32_t dst = ring + stage * STAGE;
          const int p = lane >> 1;
          if (lane & 1) {
            if (withv) tma_load_4d(dst + TILE + p * PANEL, &tmV, full0 + 8 * stage, p * 64, hk, jt * 128, b);
          } else {
            tma_load_4d(dst + p * PANEL, &tmK, full0 + 8 * stage, p * 64, hk, jt * 128, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      uint32_t c = 0, ic = 0, pc = 0;
      bool ok = true;
      // operand descriptors are built once; an MMA then costs one 64-bit add per operand
      const uint64_t dq_desc = umma_smem_desc(q_s, 0, 1024), dp_desc = umma_smem_desc(p_s, 0, 1024);
      const uint64_t dk_desc0 = umma_smem_desc(ring, 0, 1024), dk_desc1 = umma_smem_desc(ring + STAGE, 0, 1024);
      const uint64_t dv_desc0 = umma_smem_desc(ring + TILE, PANEL, 1024), dv_desc1 = umma_smem_desc(ring + STAGE + TILE, PANEL, 1024);
      for (long long item = blockIdx.x; ok && item < total; item += gridDim.x, ++ic) {
        const int tile = ntile - 1 - (int)((item / (a.Hq / 16)) % ntile);
        const Sched sc = make_sched<MODE>(a, a.q0 + tile * kTok);
        const int nt = sc.nA + sc.nB;
        ok = mbar_wait_abortable(q_full, ic & 1, 103, abort_flag);
        // Event loop over the item's tiles: S of tile `ns` is issued as soon as its K/V stage has landed and its TMEM
        // buffer has been read, P.V of tile `np` as soon as its P tile is written -- whichever is ready first.  A
        // fixed order (S(i), then P.V(i-1)) left the tensor core idle: the stage of tile i+1 is only freed by
        // P.V(i-1), so a thread blocked on that stage could not issue P.V(i) although its P tile was ready.
        const uint32_t c0 = c;
        int ns = 0, np = 0;
        uint64_t t_idle = 0;
        while (ok && np < nt) {
          bool progressed = false;
          if (ns < nt) {
            const uint32_t cc = c0 + ns, st = cc & 1, ph = (cc >> 1) & 1;
            if (mbar_try(full0 + 8 * st, ph) && mbar_try(s_free0 + 8 * st, ph ^ 1)) {
              tc_fence_after();
              const uint32_t k_s = ring + st * STAGE;
#pragma unroll
              for (int ks = 0; ks < 8; ++ks) {
                const uint32_t off = (ks >> 2) * PANEL + (ks & 3) * 32;
                umma_ss(tmem + st * 128, umma_desc_advance(dq_desc, off), umma_desc_advance(st ? dk_desc1 : dk_desc0, off),
                        idesc_s, ks ? 1u : 0u);
              }
              umma_commit(s_full0 + 8 * st);
              if (ns == nt - 1) umma_commit(q_free);
              ++ns;
              progressed = true;
            }
          }
          if (np < ns) {
            const uint32_t cc = c0 + np, st = cc & 1;
            if (np < sc.nAttn) {
              if (mbar_try(p_full, pc & 1)) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                  umma_ss(tmem + 256, umma_desc_advance(dp_desc, (ks >> 2) * PANEL + (ks & 3) * 32),
                          umma_desc_advance(st ? dv_desc1 : dv_desc0, ks * 2048), idesc_pv, (np | ks) ? 1u : 0u);
                umma_commit(empty0 + 8 * st);
                umma_commit(p_free);
                ++pc;
                ++np;
                progressed = true;
              }
            } else {
              umma_commit(empty0 + 8 * st);
              ++np;
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
              atomicCAS(&g_dev_error, 0, 105);
              *abort_flag = 1;
              ok = false;
            }
          }
        }
        c = c0 + nt;
        if (nt == 0) umma_commit(q_free);
        // o_full must not complete twice before the soft-max warps have seen it once: items without P.V tiles do
        // not throttle this thread, so wait until the previous item's epilogue has been done
        if (ok && ic > 0) ok = mbar_wait_abortable(o_free, (ic - 1) & 1, 110, abort_flag);
        umma_commit(o_full);
      }
    }
  } else {
    // ------------------------------- soft-max warps ------------------------------------------------
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;             // key columns 64*half .. +63 of each 128-key tile
    const int row = 32 * quad + lane;             // TMEM lane == Q tile row = (token, head)
    const int tl = row >> 4, head = row & 15;
    const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
    const float sl2 = a.scale * kLog2e;
    const int sthread = threadIdx.x - 64;         // 0..255 among the soft-max threads
    uint32_t c = 0, ic = 0, pc = 0, xp = 0;
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
      const int nt = sc.nA + sc.nB;
      int nvis = a.Lk;
      if (MODE == 1 && a.causal) nvis = (t < a.cblock) ? 0 : min(a.Lk, (t - a.cblock) / a.cstride + 1);
      float m_run = -INFINITY, l_run = 0.f;     // attention soft-max (log2 domain), this thread's columns
      float m2 = -INFINITY, l2 = 0.f;           // selection soft-max over raw scores, this thread's columns
      float sel_m = 0.f, sel_inv = 0.f;         // merged statistics used by the second pass
      if (do_sel) {
        for (int i = sthread; i < kTok * pool_floats; i += kSoft) pool[i] = 0.f;
      }
      int pv_local = 0;
      for (int i = 0; i < nt; ++i, ++c) {
        const bool passB = i >= sc.nA;
        const int jt = sc.first + (passB ? i - sc.nA : i);
        const int j0 = jt * 128 + half * 64;     // first key column of this thread
        const uint32_t st = c & 1;
        if (do_sel && i == sc.nA) {
          // merge the two halves' raw-score statistics before the second pass (the exchange buffer is shared with
          // the per-tile maxima: wait until nobody reads those any more)
          named_bar_sync(1, kSoft);
          xst[(0 * 2 + half) * 128 + row] = m2;
          xst[(1 * 2 + half) * 128 + row] = l2;
          named_bar_sync(1, kSoft);
          const float mo = xst[(0 * 2 + (half ^ 1)) * 128 + row], lo = xst[(1 * 2 + (half ^ 1)) * 128 + row];
          const float M = fmaxf(m2, mo);
          const float L = (m2 > -INFINITY ? l2 * ex2((m2 - M) * kLog2e) : 0.f) + (mo > -INFINITY ? lo * ex2((mo - M) * kLog2e) : 0.f);
          sel_m = M;
          sel_inv = L > 0.f ? 1.f / L : 0.f;
          named_bar_sync(1, kSoft);
        }
        ok = mbar_wait_abortable(s_full0 + 8 * st, (c >> 1) & 1, 107, abort_flag) && ok;
        tc_fence_after();
        float s[64];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          tmem_ld16(tmem + lane_addr + st * 128 + half * 64 + q4 * 16, *reinterpret_cast<float(*)[16]>(&s[q4 * 16]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(s_free0 + 8 * st);

        if (do_sel && !passB) {
          // statistics of the raw-score soft-max; only the last tile can hold columns past Lk
          const int nval = min(64, a.Lk - j0);
          float mx = -INFINITY;
          if (nval >= 64) {
#pragma unroll
            for (int e = 0; e < 64; ++e) mx = fmaxf(mx, s[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 64; ++e)
              if (e < nval) mx = fmaxf(mx, s[e]);
          }
          const float mnew = fmaxf(m2, mx);
          if (mnew > -INFINITY) {
            const float nm = -mnew * kLog2e;
            float rs0 = 0.f, rs1 = 0.f;
            if (nval >= 64) {
#pragma unroll
              for (int e = 0; e < 64; e += 2) {
                rs0 += ex2(fmaf(s[e], kLog2e, nm));
                rs1 += ex2(fmaf(s[e + 1], kLog2e, nm));
              }
            } else {
#pragma unroll
              for (int e = 0; e < 64; ++e)
                if (e < nval) rs0 += ex2(fmaf(s[e], kLog2e, nm));
            }
            l2 = l2 * ex2((m2 - mnew) * kLog2e) + (rs0 + rs1);
            m2 = mnew;
          }
        }
        if (do_sel && passB) {
          // p = softmax(raw) of this row; pool inside the thread (block k: columns 4k..4k+4; its fifth column is the
          // first column of block k+1), then sum the 16 heads of the token with a halving butterfly: after four
          // exchange steps every lane of the 16 holds two of the 32 head sums.
          const int nval = live ? min(64, a.Lk - j0) : 0;
          const float nm = -sel_m * kLog2e;
          float v[32];   // v[k] = columns 4k..4k+3, v[16+k] = column 4k
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            float pe[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int e = 4 * k + u;
              pe[u] = (e < nval) ? ex2(fmaf(s[e], kLog2e, nm)) * sel_inv : 0.f;
            }
            v[k] = (pe[0] + pe[1]) + (pe[2] + pe[3]);
            v[16 + k] = pe[0];
          }
          {
            const bool up8 = (lane & 8) != 0;
#pragma unroll
            for (int x = 0; x < 16; ++x) {
              const float send = up8 ? v[x] : v[x + 16], keep = up8 ? v[x + 16] : v[x];
              v[x] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
            const bool up4 = (lane & 4) != 0;
#pragma unroll
            for (int x = 0; x < 8; ++x) {
              const float send = up4 ? v[x] : v[x + 8], keep = up4 ? v[x + 8] : v[x];
              v[x] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
            }
            const bool up2 = (lane & 2) != 0;
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const float send = up2 ? v[x] : v[x + 4], keep = up2 ? v[x + 4] : v[x];
              v[x] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
            }
            const bool up1 = (lane & 1) != 0;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
              const float send = up1 ? v[x] : v[x + 2], keep = up1 ? v[x + 2] : v[x];
              v[x] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
            }
          }
          // lane's two values are the head sums of original slots  x + 16*b8 + 8*b4 + 4*b2 + 2*b1,  x = 0, 1
          if (live) {
            const int slot0 = ((lane & 8) ? 16 : 0) + ((lane & 4) ? 8 : 0) + ((lane & 2) ? 4 : 0) + ((lane & 1) ? 2 : 0);
            float* pt = pool + tl * pool_floats;
            const int b0 = j0 >> 2;   // global pooled block of k = 0
#pragma unroll
            for (int x = 0; x < 2; ++x) {
              const int slot = slot0 + x;
              const int blk = slot < 16 ? b0 + slot : b0 + (slot - 16) - 1;   // v[16+k] feeds block k-1
              if (blk >= 0 && blk < a.n_pool) atomicAdd(pt + blk, v[x]);
            }
          }
        }
        if (i < sc.nAttn) {
          // ---- attention soft-max of this tile --------------------------------------------------------
          // valid columns of this thread form one interval [lo, hi) of its 64; most tiles are fully valid
          int lo = 0, hi = 64;
          if (MODE == 0) {
            lo = max(0, t - a.window + 1 - j0);
            hi = min(64, t + 1 - j0);
          } else {
            hi = min(64, nvis - j0);
          }
          if (!live) hi = 0;
          const bool full = (lo <= 0) && (hi >= 64);
          float mx = -INFINITY;
          if (full) {
#pragma unroll
            for (int e = 0; e < 64; ++e) mx = fmaxf(mx, s[e]);
          } else {
#pragma unroll
            for (int e = 0; e < 64; ++e) {
              if (e < lo || e >= hi) s[e] = -INFINITY;
              mx = fmaxf(mx, s[e]);
            }
          }
          mx *= sl2;   // sl2 > 0: the maximum of the scaled scores
          float* xb = xch + (xp & 1) * 256;
          xb[half * 128 + row] = mx;
          named_bar_sync(1, kSoft);
          mx = fmaxf(mx, xb[(half ^ 1) * 128 + row]);
          ++xp;
          // Lazy rescale: the reference maximum only follows the true maximum when that has grown by more than 2^8
          // (log2 domain), so exponentials stay below 256 and the TMEM round trip that rescales O is rare.  Both
          // threads of a row see the same mx and m_run and take the same decision.
          const float mtrue = fmaxf(m_run, mx);
          const float mnew = (mtrue > m_run + 8.f || m_run == -INFINITY) ? mtrue : m_run;
          const float muse = (mnew == -INFINITY) ? 0.f : mnew;
          const float alpha = ex2(m_run - muse);   // 0 when m_run = -inf
          float rs0 = 0.f, rs1 = 0.f;
          uint32_t pw[32];
#pragma unroll
          for (int e = 0; e < 64; e += 2) {
            const float p0 = ex2(fmaf(s[e], sl2, -muse)), p1 = ex2(fmaf(s[e + 1], sl2, -muse));
            rs0 += p0;
            rs1 += p1;
            pw[e >> 1] = pack_bf16(p0, p1);
          }
          const float rs = rs0 + rs1;
          l_run = l_run * alpha + rs;
          const bool moved = (mnew != m_run) && (m_run > -INFINITY);
          m_run = mnew;
          if (pv_local > 0) {
            ok = mbar_wait_abortable(p_free, (pc - 1) & 1, 108, abort_flag) && ok;   // previous P.V done: P tile and O are ours
            if (__any_sync(0xffffffffu, moved)) {
              tc_fence_after();
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                float o[16];
                tmem_ld16(tmem + lane_addr + 256 + half * 64 + q4 * 16, o);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e) o[e] *= alpha;
                tmem_st16(tmem + lane_addr + 256 + half * 64 + q4 * 16, o);
              }
              tmem_st_wait();
              tc_fence_before();
            }
          }
          uint8_t* prow = sgen + (p_s - sbase) + half * PANEL + row * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) =
                make_uint4(pw[4 * ch], pw[4 * ch + 1], pw[4 * ch + 2], pw[4 * ch + 3]);
          fence_proxy_async();
          mbar_arrive(p_full);
          ++pc;
          ++pv_local;
        }
      }
      // ---- epilogue of the item ----------------------------------------------------------------------
      ok = mbar_wait_abortable(o_full, ic & 1, 109, abort_flag) && ok;
      tc_fence_after();
      {
        float* xb = xch + (xp & 1) * 256;
        xb[half * 128 + row] = l_run;
        named_bar_sync(1, kSoft);
        const float l_tot = l_run + xb[(half ^ 1) * 128 + row];
        ++xp;
        const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
        const long long orow = ((long long)b * a.Tq + tloc) * a.Hq + hg * 16 + head;
        uint4 outv[8];
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(outv);
        if (pv_local > 0) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            float o[16];
            tmem_ld16(tmem + lane_addr + 256 + half * 64 + q4 * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 8; ++e) ho[q4 * 8 + e] = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) outv[e] = make_uint4(0u, 0u, 0u, 0u);
        }
        tc_fence_before();
        mbar_arrive(o_free);
        if (live && ok) {
          uint4* dst = reinterpret_cast<uint4*>(a.o + orow * D + half * 64);
#pragma unroll
          for (int e = 0; e < 8; ++e) dst[e] = outv[e];
          if (half == 0) a.lse[orow] = l_tot > 0.f ? (m_run + log2f(l_tot)) * kLn2 : -INFINITY;
        }
      }
      if (do_sel) {
        named_bar_sync(1, kSoft);   // every head's pooled contribution has landed
        const int tw = warp - 2;    // this warp finishes token t0 + tw
        const int tt = t0l + tw;   // local row of the token this warp finishes
        if (tt < a.Tq && ok) {
          float* pt = pool + tw * pool_floats;
          for (int blk = lane; blk < a.n_pool; blk += 32) {
            const int lo = blk * a.pool_s - a.pool_p;
            const int hi = min(lo + a.pool_k, a.Lk + a.pool_p);
            const float v = pt[blk] / (float)(hi - lo);
            pt[blk] = v;
            if (a.sel_scores) a.sel_scores[(((long long)b * HG + hg) * a.Tq + tt) * a.n_pool + blk] = v;
          }
          __syncwarp();
          int* out = a.sel_idx + (((long long)b * a.Tq + tt) * HG + hg) * a.n_sel;
          for (int r = 0; r < a.n_sel; ++r) {
            float bv = -2.f;
            int bi = 0x7fffffff;
            for (int blk = lane; blk < a.n_pool; blk += 32) {
              const float v = pt[blk];
              if (v > bv) {
                bv = v;
                bi = blk;
              }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
              const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
              const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
              if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
              }
            }
            const bool found = bv > -1.5f;
            if (lane == 0) {
              out[r] = found ? bi : -1;
              if (found) pt[bi] = -2.f;
            }
            __syncwarp();
          }
        }
        named_bar_sync(1, kSoft);   // the pool is free for the next item
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

template <int MODE>
int launch(const DenseArgs& a, cudaStream_t s) {
  CUtensorMap tmQ, tmK, tmV;
  const unsigned long long qd[3] = {(unsigned long long)D, (unsigned long long)a.Hq, (unsigned long long)a.B * a.Tq};
  const unsigned long long qs[2] = {(unsigned long long)D * 2, (unsigned long long)a.Hq * D * 2};
  const unsigned qb[3] = {64, 16, (unsigned)kTok};
  int rc = make_tmap_generic(&tmQ, a.q, 3, qd, qs, qb);
  if (!rc) rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.Lk, a.B, 128);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.Lk, a.B, 128);
  if (rc) return rc;
  const bool sel = MODE == 1 && a.n_sel > 0;
  const int pool_floats = sel ? (a.n_pool + 3) / 4 * 4 : 0;
  const int need = (int)(TILE + kStages * STAGE + TILE) + 128 + 2 * 2 * 128 * 4 + kTok * pool_floats * 4;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  int smem = need + 1024;                      // room for rounding the base up to 1024 bytes
  if (smem > max_smem) smem = max_smem;        // long sequences: less slack (the kernel checks that it still fits)
  if (smem < need + 128) {
    set_error("dense attention: the pooled-score vector (n_pool=%d) does not fit in shared memory", a.n_pool);
    return -31;
  }
  auto kern = dense_fwd_tc_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * (a.Hq / 16) * ((a.Tq + kTok - 1) / kTok);
  const int grid = (int)(total < num_sms() ? total : num_sms());
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, smem, s>>>(tmQ, tmK, tmV, a, pool_floats, smem);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

// True when the tcgen05 forward covers this configuration (otherwise the caller uses launch_dense_fwd).
bool dense_fwd_tc_supported(const DenseArgs& a, int head_dim) {
  if (head_dim != 128) return false;
  if (a.mode == 1 && a.n_sel > 0) {
    if (a.pool_k != 5 || a.pool_s != 4 || a.pool_p != 0) return false;
    if (a.n_pool > kMaxPool) return false;
  }
  return true;
}
int launch_dense_fwd_tc(const DenseArgs& a, cudaStream_t s) { return a.mode == 0 ? launch<0>(a, s) : launch<1>(a, s); }
int dense_tc_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
