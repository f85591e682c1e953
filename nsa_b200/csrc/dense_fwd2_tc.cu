// Dense query-major attention FORWARD on tcgen05, two query tiles per CTA (head_dim 128): sliding-window attention
// (mode 0) and compressed attention with the fused block selection (mode 1).  Semantics and result layouts of
// nsa/selection_attn.py:484-516 (window), nsa/triton_attention.py:87-181,465-475 (compressed attention, scores, top-n,
// with the scoring of nsa/torch_attention.py:121-125) and, optionally, the gate projection nn.Linear(head_dim, 3) of
// nsa/nsa.py:117 computed from the resident query tiles.
//
// A persistent CTA owns 16 consecutive tokens x the 16 heads of a GQA group = two [128 x 128] Q tiles that share one
// stream of [128 keys x 128] K and V tiles (K and V in separate mbarrier rings, so a K slot is recycled as soon as
// both score MMAs have read it, long before the V slot of the same tile).  One thread issues every tcgen05.mma.  Each
// Q tile has its own soft-max warp group of 128 threads, one thread per (token, head) row holding all 128 key columns
// of its TMEM lane: no shuffles, no exchange, no CTA-wide barrier in the tile loop.  Per group the order is strictly
//     S = Q.K^T (TMEM)  ->  soft-max  ->  P written back over S as packed bf16  ->  O += P.V (A operand read from TMEM)
// and the two groups run half a period apart, so the tensor core works for one group while the other exponentiates.
// O is rescaled in TMEM only when a row maximum grew by more than 2^8.
//
// Selection (mode 1): a first pass over all compressed tiles collects the statistics of the unscaled, unmasked
// soft-max while the causal tiles also feed the attention; a second pass recomputes S, forms p / l, pools the 5-wide
// stride-4 windows inside the thread, sums the 16 heads of a token with a halving shuffle butterfly and accumulates
// a per-token score vector in shared memory; each warp then picks the top n of two tokens (ties to the lower index).
// The [B,Hq,T,Tc] score tensor never exists.
#include "kernels.h"
#include "tc.cuh"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int D = 128;
constexpr int kTokT = 8;                      // tokens per Q tile
constexpr int kTok = 16;                      // tokens per item (two Q tiles)
constexpr int kThreads = 320;                 // warp 0 TMA, warp 1 MMA, warps 2-5 soft-max group 0, warps 6-9 group 1
constexpr int kGroup = 128;
constexpr uint32_t PANEL = 128 * 128;         // [128 rows][64 columns] bf16
constexpr uint32_t TILE = 2 * PANEL;          // 32 KB
constexpr uint32_t kTmemCols = 512;           // S0 0..127 (P0 over 0..63), S1 128..255, O0 256..383, O1 384..511
constexpr int kMaxPool = 1024;
constexpr int kMaxRing = 4;
constexpr uint32_t kMisc = 512;               // barriers, tmem slot, abort flag

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
    if (sel && a.score_mode == 1) {   // causal scores: both passes stop at the last visible tile
      s.nA = s.nAttn;
      s.nB = s.nAttn;
    } else {
      s.nA = sel ? nt_all : s.nAttn;
      s.nB = sel ? nt_all : 0;
    }
  }
  return s;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// max over 128 values: four independent chains of three-input maxima (FMNMX runs at half rate; a single chain of 128
// dependent two-input maxima cost ~600 cycles per tile)
__device__ __forceinline__ float max128(const float (&s)[128]) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int e = 0; e < 128; e += 8) {
    m0 = max3(m0, s[e], s[e + 1]);
    m1 = max3(m1, s[e + 2], s[e + 3]);
    m2 = max3(m2, s[e + 4], s[e + 5]);
    m3 = max3(m3, s[e + 6], s[e + 7]);
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}
struct Fused {          // optional gate projection (null pointers switch it off)
  const bf16* gate_w;   // mode 1: [3, D] gate projection weight; rows: selected, window, compressed
  const bf16* gate_b;   // [3] or null
  bf16* g_out[3];       // [B*Tq*Hq] each
};

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    dense_fwd2_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const DenseArgs a, const Fused fu, const int KST,
                         const int VST, const int pool_floats, const int smem_bytes) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_s = sbase, k_ring = sbase + 2 * TILE, v_ring = k_ring + KST * TILE, misc = v_ring + VST * TILE;
  // barriers (8 bytes each)
  const uint32_t q_full = misc, q_free = misc + 8, k_full0 = misc + 16, k_empty0 = misc + 48, v_full0 = misc + 80,
                 v_empty0 = misc + 112, s_full0 = misc + 144, p_full0 = misc + 160, pv_done0 = misc + 176,
                 o_free0 = misc + 192, tmem_slot = misc + 208;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + (misc - sbase) + 216);
  float* gw = reinterpret_cast<float*>(sgen + (misc - sbase) + kMisc);         // [3][D] gate weights (fp32), mode 1
  float* pool = gw + 3 * D;                                                    // [kTok][pool_floats]
  if ((misc - raw) + kMisc + 3 * D * 4 + kTok * pool_floats * 4 > (uint32_t)smem_bytes) {
    if (threadIdx.x == 0) atomicCAS(&g_dev_error, 0, DEV_ERR_BOUNDS);
    return;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    // the Q tiles go back to the producer when the item's last score MMA has completed and, when the gate projection
    // is fused in, every soft-max thread has read its Q row
    mbar_init(q_free, (MODE == 1 && fu.gate_w != nullptr) ? 1 + 2 * kGroup : 1);
    for (int i = 0; i < kMaxRing; ++i) {
      mbar_init(k_full0 + 8 * i, 1);
      mbar_init(k_empty0 + 8 * i, 1);
      mbar_init(v_full0 + 8 * i, 1);
      mbar_init(v_empty0 + 8 * i, 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full0 + 8 * g, 1);
      mbar_init(p_full0 + 8 * g, kGroup);
      mbar_init(pv_done0 + 8 * g, 1);
      mbar_init(o_free0 + 8 * g, kGroup);
    }
    fence_mbar_init();
  }
  const bool do_gate = MODE == 1 && fu.gate_w != nullptr;
  if (do_gate)
    for (int i = threadIdx.x; i < 3 * D; i += kThreads) gw[i] = __bfloat162float(fu.gate_w[i]);
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
  const bool causal_scores = do_sel && a.score_mode == 1;

  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------------
    uint32_t ck = 0, cv = 0, ic = 0;
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
        if (good) mbar_expect_tx(q_full, 2 * TILE);
      }
      if (!__shfl_sync(0xffffffffu, good, 0)) break;
      if (lane < 4) {   // lane = 2 * tile + panel
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
            ::"r"(q_s + (lane >> 1) * TILE + (lane & 1) * PANEL), "l"(&tmQ), "r"(q_full), "r"((lane & 1) * 64), "r"(hg * 16),
              "r"(b * a.Tq + t0l + (lane >> 1) * kTokT)
            : "memory");
      }
      // K and V tiles are issued independently, whichever ring has a free slot first: K slots come back as soon as both
      // score MMAs have read them, V slots only after both P.V products
      const int nt = sc.nA + sc.nB;
      int ik = 0, iv = 0;
      uint64_t t_idle = 0;
      while (ik < nt || iv < sc.nAttn) {
        const uint32_t ks = ck % (uint32_t)KST, kph = (ck / (uint32_t)KST) & 1;
        const uint32_t vs = cv % (uint32_t)VST, vph = (cv / (uint32_t)VST) & 1;
        int act = 0;
        if (lane == 0) {
          if (ik < nt && mbar_test(k_empty0 + 8 * ks, kph ^ 1)) {
            mbar_expect_tx(k_full0 + 8 * ks, TILE);
            act |= 1;
          }
          if (iv < sc.nAttn && mbar_test(v_empty0 + 8 * vs, vph ^ 1)) {
            mbar_expect_tx(v_full0 + 8 * vs, TILE);
            act |= 2;
          }
          if (!act) {
            if (*abort_flag) act = -1;
            const uint64_t now = global_timer_ns();
            if (t_idle == 0) t_idle = now;
            else if (now - t_idle > 2000000000ull) {
              atomicCAS(&g_dev_error, 0, 102);
              *abort_flag = 1;
              act = -1;
            }
          } else {
            t_idle = 0;
          }
        }
        act = __shfl_sync(0xffffffffu, act, 0);
        if (act < 0) {
          alive = false;
          break;
        }
        if (act & 1) {
          const int jt = sc.first + (ik < sc.nA ? ik : ik - sc.nA);
          if (lane < 2) tma_load_4d(k_ring + ks * TILE + lane * PANEL, &tmK, k_full0 + 8 * ks, lane * 64, hk, jt * 128, b);
          ++ck;
          ++ik;
        }
        if (act & 2) {
          const int jt = sc.first + iv;
          if (lane < 2) tma_load_4d(v_ring + vs * TILE + lane * PANEL, &tmV, v_full0 + 8 * vs, lane * 64, hk, jt * 128, b);
          ++cv;
          ++iv;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ----------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      uint32_t ck0 = 0, cv0 = 0, ic = 0;
      uint32_t pph[2] = {0, 0};   // p_full phases consumed per group
      uint32_t npi[2] = {0, 0};   // items with P.V tiles so far, per group (= o_free phases the group will have arrived on)
      bool ok = true;
      const uint64_t dq_desc0 = umma_smem_desc(q_s, 0, 1024), dq_desc1 = umma_smem_desc(q_s + TILE, 0, 1024);
      const uint64_t dk_base = umma_smem_desc(k_ring, 0, 1024);
      const uint64_t dv_base = umma_smem_desc(v_ring, PANEL, 1024);
      for (long long item = blockIdx.x; ok && item < total; item += gridDim.x, ++ic) {
        const int tile = ntile - 1 - (int)((item / HG) % ntile);
        const Sched sc = make_sched<MODE>(a, a.q0 + tile * kTok);
        const int nt = sc.nA + sc.nB;
        ok = mbar_wait_abortable(q_full, ic & 1, 103, abort_flag);
        int is[2] = {0, 0}, ip[2] = {0, 0};
        bool pv_any[2] = {false, false};
        uint32_t s_cnt = 0, v_cnt = 0;   // bit i%8 set: one group has issued S / P.V of tile i, the other has not yet
        uint64_t t_idle = 0;
        while (ok && (ip[0] < nt || ip[1] < nt)) {
          bool progressed = false;
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            // (1) the group's P (or its "S has been read") of tile ip[g]
            if (ip[g] < is[g]) {
              const int i = ip[g];
              bool ready = mbar_test(p_full0 + 8 * g, pph[g] & 1);
              uint32_t vs = 0;
              if (ready && i < sc.nAttn) {
                const uint32_t c = cv0 + i;
                vs = c % (uint32_t)VST;
                ready = mbar_test(v_full0 + 8 * vs, (c / (uint32_t)VST) & 1);
                // the epilogue of the group's previous item with P.V tiles must have read O before this item's first
                // P.V overwrites it (items without P.V tiles neither touch O nor arrive on o_free)
                if (ready && !pv_any[g] && npi[g] > 0) ready = mbar_test(o_free0 + 8 * g, (npi[g] - 1) & 1);
              }
              if (ready) {
                if (i < sc.nAttn) {
                  tc_fence_after();
                  const uint64_t dv = umma_desc_advance(dv_base, vs * TILE);
#pragma unroll
                  for (int ks = 0; ks < 8; ++ks)   // A = P from tensor memory: 16 keys = 8 packed columns per step
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                        ::"r"(tmem + 256 + g * 128), "r"(tmem + g * 128 + ks * 8), "l"(umma_desc_advance(dv, ks * 2048)),
                          "r"(idesc_pv), "r"((uint32_t)((pv_any[g] || ks) ? 1 : 0))
                        : "memory");
                  umma_commit(pv_done0 + 8 * g);
                  if (!pv_any[g]) ++npi[g];
                  pv_any[g] = true;
                  const uint32_t bit = 1u << (i & 7);
                  if (v_cnt & bit) {
                    umma_commit(v_empty0 + 8 * vs);
                    v_cnt &= ~bit;
                  } else {
                    v_cnt |= bit;
                  }
                }
                ++pph[g];
                ++ip[g];
                progressed = true;
              }
            }
            // (2) S of the group's next tile, once the previous tile's P has been consumed
            if (is[g] < nt && ip[g] == is[g]) {
              const int i = is[g];
              const uint32_t c = ck0 + i, ks_ = c % (uint32_t)KST;
              if (mbar_test(k_full0 + 8 * ks_, (c / (uint32_t)KST) & 1)) {
                tc_fence_after();
                const uint64_t dk = umma_desc_advance(dk_base, ks_ * TILE);
                const uint64_t dq = g ? dq_desc1 : dq_desc0;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                  const uint32_t off = (ks >> 2) * PANEL + (ks & 3) * 32;
                  umma_ss(tmem + g * 128, umma_desc_advance(dq, off), umma_desc_advance(dk, off), idesc_s, ks ? 1u : 0u);
                }
                umma_commit(s_full0 + 8 * g);
                const uint32_t bit = 1u << (i & 7);
                if (s_cnt & bit) {
                  umma_commit(k_empty0 + 8 * ks_);
                  if (i == nt - 1) umma_commit(q_free);
                  s_cnt &= ~bit;
                } else {
                  s_cnt |= bit;
                }
                ++is[g];
                progressed = true;
              }
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
        ck0 += nt;
        cv0 += sc.nAttn;
        if (nt == 0) umma_commit(q_free);
      }
    }
  } else {
    // ------------------------------- soft-max groups ------------------------------------------------
    const int quad = warp & 3;
    const int g = (warp - 2) >> 2;                // group = Q tile
    const int row = 32 * quad + lane;             // TMEM lane == Q tile row = (token, head)
    const int tl = row >> 4, head = row & 15;
    const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
    const uint32_t s_col = tmem + lane_addr + g * 128, o_col = tmem + lane_addr + 256 + g * 128;
    const float sl2 = a.scale * kLog2e;
    const int gthread = threadIdx.x - 64 - g * kGroup;   // 0..127 inside the group
    const int gwarp = gthread >> 5;
    const uint32_t s_full = s_full0 + 8 * g, p_full = p_full0 + 8 * g, pv_done = pv_done0 + 8 * g, o_free = o_free0 + 8 * g;
    uint32_t cs = 0, npv = 0, ic = 0;
    bool ok = true;
    for (long long item = blockIdx.x; item < total; item += gridDim.x, ++ic) {
      const int hg = (int)(item % HG);
      const int tile = ntile - 1 - (int)((item / HG) % ntile);
      const int b = (int)(item / ((long long)HG * ntile));
      const int t0l = tile * kTok;
      const int tloc = t0l + g * kTokT + tl;   // local query row
      const int t = a.q0 + tloc;               // its sequence position
      const bool live = tloc < a.Tq;
      const Sched sc = make_sched<MODE>(a, a.q0 + t0l);
      const int nt = sc.nA + sc.nB;
      const long long orow = ((long long)b * a.Tq + tloc) * a.Hq + hg * 16 + head;
      int nvis = a.Lk;
      if (MODE == 1 && a.causal) nvis = (t < a.cblock) ? 0 : min(a.Lk, (t - a.cblock) / a.cstride + 1);
      float m_run = -INFINITY, l_run = 0.f;     // attention soft-max (log2 domain)
      float m2 = -INFINITY, l2 = 0.f;           // selection soft-max over raw scores
      float sel_m = 0.f, sel_inv = 0.f;
      float* gpool = pool + g * kTokT * pool_floats;   // this group's eight tokens
      if (do_sel) {
        for (int i = gthread; i < kTokT * pool_floats; i += kGroup) gpool[i] = 0.f;
      }
      if (do_gate) {
        // gate projection of this row from the resident Q tile (nn.Linear(head_dim, 3), no activation)
        ok = mbar_wait_abortable(q_full, ic & 1, 106, abort_flag) && ok;
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
        const uint8_t* qrow = sgen + (q_s - sbase) + g * TILE + row * 128;
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          const uint4 qq = *reinterpret_cast<const uint4*>(qrow + (ch >> 3) * PANEL + (((ch & 7) ^ (row & 7)) << 4));
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&qq);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            const int d0 = ch * 8 + 2 * e;
            acc0 = fmaf(f.x, gw[d0], fmaf(f.y, gw[d0 + 1], acc0));
            acc1 = fmaf(f.x, gw[D + d0], fmaf(f.y, gw[D + d0 + 1], acc1));
            acc2 = fmaf(f.x, gw[2 * D + d0], fmaf(f.y, gw[2 * D + d0 + 1], acc2));
          }
        }
        mbar_arrive(q_free);
        if (live && ok) {
          const float b0 = fu.gate_b ? __bfloat162float(fu.gate_b[0]) : 0.f, b1 = fu.gate_b ? __bfloat162float(fu.gate_b[1]) : 0.f,
                      b2 = fu.gate_b ? __bfloat162float(fu.gate_b[2]) : 0.f;
          fu.g_out[0][orow] = __float2bfloat16(acc0 + b0);
          fu.g_out[1][orow] = __float2bfloat16(acc1 + b1);
          fu.g_out[2][orow] = __float2bfloat16(acc2 + b2);
        }
      }
      int pv_local = 0;
      for (int i = 0; i < nt; ++i, ++cs) {
        const bool passB = i >= sc.nA;
        const int jt = sc.first + (passB ? i - sc.nA : i);
        const int j0 = jt * 128;                 // first key column of the tile
        if (do_sel && i == sc.nA) {
          if (causal_scores) {   // the attention soft-max's own statistics (log2 domain, scaled scores)
            sel_m = m_run > -INFINITY ? m_run : 0.f;
            sel_inv = l_run > 0.f ? 1.f / l_run : 0.f;
          } else {
            sel_m = m2;
            sel_inv = l2 > 0.f ? 1.f / l2 : 0.f;
          }
          named_bar_sync(1 + g, kGroup);         // the pool of this group has been cleared by all of its threads
        }
        ok = mbar_wait_abortable(s_full, cs & 1, 107, abort_flag) && ok;
        tc_fence_after();
        float s[128];
#pragma unroll
        for (int c = 0; c < 8; ++c) tmem_ld16(s_col + c * 16, *reinterpret_cast<float(*)[16]>(&s[c * 16]));
        tmem_ld_wait();

        const bool attn_tile = i < sc.nAttn;
        if (!attn_tile) {
          // nothing is written back for this tile: the scores are in registers, so S of the group's next tile may be
          // issued now and runs under the arithmetic below
          tc_fence_before();
          mbar_arrive(p_full);
        }
        if (do_sel && !(causal_scores && !passB)) {
          // columns past Lk exist only in the last tile (reference scores); causal scores stop at the row's last
          // visible key; rows past Tq contribute nothing to the scores
          const int nval = min(128, (causal_scores ? nvis : a.Lk) - j0);
          if (nval < 128) {
#pragma unroll
            for (int e = 0; e < 128; ++e)
              if (e >= nval) s[e] = -INFINITY;
          }
        }
        if (do_sel && !passB && !causal_scores) {
          // statistics of the raw-score soft-max over all compressed keys
          const float mnew = fmaxf(m2, max128(s));
          if (mnew > -INFINITY) {
            const float nm = -mnew * kLog2e;
            float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll
            for (int e = 0; e < 128; e += 4) {
              rs0 += ex2(fmaf(s[e], kLog2e, nm));
              rs1 += ex2(fmaf(s[e + 1], kLog2e, nm));
              rs2 += ex2(fmaf(s[e + 2], kLog2e, nm));
              rs3 += ex2(fmaf(s[e + 3], kLog2e, nm));
            }
            l2 = l2 * ex2((m2 - mnew) * kLog2e) + ((rs0 + rs1) + (rs2 + rs3));
            m2 = mnew;
          }
        }
        if (do_sel && passB) {
          // p = softmax(raw) of this row; pool inside the thread (block k: columns 4k..4k+4; its fifth column is the
          // first column of block k+1), then sum the 16 heads of the token with a halving butterfly: after four
          // exchange steps every lane of the 16 holds two of the 32 sums.  Done per half of 64 columns.
          const float cmul = causal_scores ? sl2 : kLog2e;
          const float nm = causal_scores ? -sel_m : -sel_m * kLog2e;
          const float inv_b = live ? sel_inv : 0.f;
          float* pt = gpool + tl * pool_floats;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int jh = j0 + hh * 64;
            float v[32];   // v[k] = columns 4k..4k+3, v[16+k] = column 4k
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              float pe[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) pe[u] = ex2(fmaf(s[hh * 64 + 4 * k + u], cmul, nm)) * inv_b;   // masked columns: 0
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
              const int b0 = jh >> 2;   // global pooled block of k = 0
#pragma unroll
              for (int x = 0; x < 2; ++x) {
                const int slot = slot0 + x;
                const int blk = slot < 16 ? b0 + slot : b0 + (slot - 16) - 1;   // v[16+k] feeds block k-1
                if (blk >= 0 && blk < a.n_pool) atomicAdd(pt + blk, v[x]);
              }
            }
          }
        }
        if (attn_tile) {
          // ---- attention soft-max of this tile: valid columns form one interval [lo, hi) ----------------------
          int lo = 0, hi = 128;
          if (MODE == 0) {
            lo = max(0, t - a.window + 1 - j0);
            hi = min(128, t + 1 - j0);
          } else {
            hi = min(128, nvis - j0);
          }
          if (!live) hi = 0;
          const bool full = (lo <= 0) && (hi >= 128);
          if (!full) {
#pragma unroll
            for (int e = 0; e < 128; ++e)
              if (e < lo || e >= hi) s[e] = -INFINITY;
          }
          float mx = max128(s);
          mx *= sl2;   // sl2 > 0: the maximum of the scaled scores
          // Lazy rescale: the reference maximum follows the true maximum only when that has grown by more than 2^8
          // (log2 domain), so exponentials stay below 256 and the TMEM round trip that rescales O is rare.
          const float mtrue = fmaxf(m_run, mx);
          const float mnew = (mtrue > m_run + 8.f || m_run == -INFINITY) ? mtrue : m_run;
          const float muse = (mnew == -INFINITY) ? 0.f : mnew;
          const float alpha = ex2(m_run - muse);   // 0 when m_run = -inf
          const bool moved = (mnew != m_run) && (m_run > -INFINITY);
          m_run = mnew;
          if (pv_local > 0 && __any_sync(0xffffffffu, moved)) {
            ok = mbar_wait_abortable(pv_done, (npv - 1) & 1, 108, abort_flag) && ok;   // the previous P.V has completed
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float o[16];
              tmem_ld16(o_col + c * 16, o);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 16; ++e) o[e] *= alpha;
              tmem_st16(o_col + c * 16, o);
            }
          }
          float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {   // 32 keys -> 16 packed columns per store
            float pk[16];
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
              const float p0 = ex2(fmaf(s[c * 32 + 2 * e], sl2, -muse)), p1 = ex2(fmaf(s[c * 32 + 2 * e + 1], sl2, -muse));
              const float p2 = ex2(fmaf(s[c * 32 + 2 * e + 2], sl2, -muse)), p3 = ex2(fmaf(s[c * 32 + 2 * e + 3], sl2, -muse));
              rs0 += p0; rs1 += p1; rs2 += p2; rs3 += p3;
              pk[e] = __uint_as_float(pack_bf16(p0, p1));
              pk[e + 1] = __uint_as_float(pack_bf16(p2, p3));
            }
            tmem_st16(s_col + c * 16, pk);
          }
          rs0 = (rs0 + rs1) + (rs2 + rs3);
          rs1 = 0.f;
          l_run = l_run * alpha + (rs0 + rs1);
          tmem_st_wait();
          ++npv;
          ++pv_local;
        }
        if (attn_tile) {
          tc_fence_before();
          mbar_arrive(p_full);   // P is in place
        }
        if (gthread == 0) {
        }
      }
      // ---- epilogue of the item ----------------------------------------------------------------------
      {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint4 outv[16];
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(outv);
        if (pv_local > 0) {
          ok = mbar_wait_abortable(pv_done, (npv - 1) & 1, 109, abort_flag) && ok;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float o[16];
            tmem_ld16(o_col + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 8; ++e) ho[c * 8 + e] = __floats2bfloat162_rn(o[2 * e] * inv, o[2 * e + 1] * inv);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) outv[e] = make_uint4(0u, 0u, 0u, 0u);
        }
        tc_fence_before();
        if (pv_local > 0) mbar_arrive(o_free);   // O has been read: the next item with P.V tiles may overwrite it
        if (live && ok) {
          uint4* dst = reinterpret_cast<uint4*>(a.o + orow * D);
#pragma unroll
          for (int e = 0; e < 16; ++e) dst[e] = outv[e];
          a.lse[orow] = l_run > 0.f ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
        }
      }
      if (do_sel) {
        named_bar_sync(1 + g, kGroup);   // every head's pooled contribution of this group's tokens has landed
#pragma unroll 1
        for (int u = 0; u < 2; ++u) {
          const int tw = gwarp * 2 + u;              // token of the group this warp finishes
          const int tt = t0l + g * kTokT + tw;       // its local row
          if (tt < a.Tq && ok) {
            float* pt = gpool + tw * pool_floats;
            for (int blk = lane; blk < a.n_pool; blk += 32) {
              const int lo = blk * a.pool_s - a.pool_p;
              const int hi = min(lo + a.pool_k, a.Lk + a.pool_p);
              const float v = pt[blk] / (float)(hi - lo);
              pt[blk] = v;
              if (a.sel_scores) a.sel_scores[(((long long)b * HG + hg) * a.Tq + tt) * a.n_pool + blk] = v;
            }
            __syncwarp();
            int* out = a.sel_idx + (((long long)b * a.Tq + tt) * HG + hg) * a.n_sel;
            // Pooled scores are >= 0, so their bit patterns order like the values: one integer warp reduction finds the
            // maximum, a second the lowest block index that holds it (ties go to the lower index).
            for (int r = 0; r < a.n_sel; ++r) {
              unsigned bv = 0u;
              int bi = 0x7fffffff;
              bool any = false;
              for (int blk = lane; blk < a.n_pool; blk += 32) {
                const float v = pt[blk];
                if (v >= 0.f) {
                  const unsigned u = __float_as_uint(v);
                  if (!any || u > bv) {
                    bv = u;
                    bi = blk;
                  }
                  any = true;
                }
              }
              const unsigned key = any ? bv + 1u : 0u;                         // 0 = this lane has no candidate left
              const unsigned best = __reduce_max_sync(0xffffffffu, key);
              const int win = __reduce_min_sync(0xffffffffu, (key == best && any) ? bi : 0x7fffffff);
              if (lane == 0) out[r] = best ? win : -1;
              if (best && (win & 31) == lane) pt[win] = -2.f;                  // the owner lane retires the block
              __syncwarp();
            }
          }
        }
        named_bar_sync(1 + g, kGroup);   // the pool is free for the next item
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

template <int MODE>
int launch(const DenseArgs& a, const Fused& fu, cudaStream_t s) {
  CUtensorMap tmQ, tmK, tmV;
  const unsigned long long qd[3] = {(unsigned long long)D, (unsigned long long)a.Hq, (unsigned long long)a.B * a.Tq};
  const unsigned long long qs[2] = {(unsigned long long)D * 2, (unsigned long long)a.Hq * D * 2};
  const unsigned qb[3] = {64, 16, (unsigned)kTokT};
  int rc = make_tmap_generic(&tmQ, a.q, 3, qd, qs, qb);
  if (!rc) rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.Lk, a.B, 128);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.Lk, a.B, 128);
  if (rc) return rc;
  const bool sel = MODE == 1 && a.n_sel > 0;
  const int pool_floats = sel ? (a.n_pool + 3) / 4 * 4 : 0;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  // Q tiles + rings + barriers + gate weights + pooled scores; the K ring gets two slots, V two if they fit, else one
  const int fixed = (int)(2 * TILE) + (int)kMisc + 3 * D * 4 + kTok * pool_floats * 4 + 1024;
  int KST = 2, VST = 2;
  if (fixed + (KST + VST) * (int)TILE > max_smem) VST = 1;
  if (fixed + (KST + VST) * (int)TILE > max_smem) {
    set_error("dense attention: the pooled-score vector (n_pool=%d) does not fit in shared memory", a.n_pool);
    return -31;
  }
  const int smem = fixed + (KST + VST) * (int)TILE;
  auto kern = dense_fwd2_tc_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * (a.Hq / 16) * ((a.Tq + kTok - 1) / kTok);
  const int grid = (int)(total < num_sms() ? total : num_sms());
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, smem, s>>>(tmQ, tmK, tmV, a, fu, KST, VST, pool_floats, smem);
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
int launch_dense_fwd2_tc(const DenseArgs& a, cudaStream_t s) {
  Fused fu = {};
  fu.gate_w = a.gate_w;
  fu.gate_b = a.gate_b;
  for (int i = 0; i < 3; ++i) fu.g_out[i] = a.g_out[i];
  return a.mode == 0 ? launch<0>(a, fu, s) : launch<1>(a, fu, s);
}
int dense_tc2_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
