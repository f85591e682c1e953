// Selected attention forward, key-major on tcgen05 (head_dim 128, 64-key blocks, 16 query heads per group).
// Same results as the query-major kernel (nsa/selection_attn.py:401-517: every query attends to the keys k <= t of
// its selected blocks), different decomposition: the 16 heads of one query are the only rows that share a gathered
// block, too few for a tensor-core tile, so here a CTA owns one 64-key block and the QUERIES that selected it arrive in
// batches of 8 tokens x 16 heads = 128 rows (the block's ascending token list from the reverse index).  Per batch:
//     S     [128 rows x 64 keys] = Qg . K^T     A = Qg (K-major, gathered by TMA), B = K (K-major)
//     O_part[128 rows x 128 d  ] = P . V        A = P (K-major, written by the soft-max warps), B = V (MN-major)
// with P = exp(scale S - m), m the row's maximum over the block's visible keys.  The visit leaves (m, l = sum P) per
// row and O_part as a [16 heads x D] bf16 tile at the visit's position in the reverse-index list; a second kernel
// merges a token's visits in slot order (fixed order, no atomics):  o = sum_v 2^(m_v - M) O_v / sum_v 2^(m_v - M) l_v.
// K and V of a block are read once per CTA instead of once per visiting query (32 KB per visit in the query-major
// kernel, which is bound by that gather).
// Roles (512 threads): warps 0-2 TMA producers (4-stage ring of 32 KB Q tiles; a stage is free as soon as its score MMAs
// have completed), warp 3 the MMA issuer (event loop), warps 4-7 / 8-11 two soft-max groups (even / odd batches, one
// row per thread), warps 12-15 read O_part out of tensor memory into a staging tile that one bulk store writes.
// Every wait is bounded; on a time-out the role records an error and leaves its loop.
#include "kernels.h"
#include "tc.cuh"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int D = 128;
constexpr int kProd = 3;
constexpr int kMmaWarp = kProd;
constexpr int kSoftWarp = kProd + 1;        // 8 soft-max warps: two groups of four
constexpr int kDrainWarp = kSoftWarp + 8;   // 4 drain warps
constexpr int kThreads = (kDrainWarp + 4) * 32;
constexpr int kTokB = 8;
constexpr uint32_t KV_PANEL = 64 * 128;     // [64 keys][64 ch]
constexpr uint32_t KV_TILE = 2 * KV_PANEL;  // 16 KB
constexpr uint32_t Q_TILE = 128 * 256;       // 32 KB: [16 row groups][2 column panels][8 rows][128 B]
constexpr uint32_t P_TILE = 128 * 128;      // [128 rows][64 keys]
constexpr uint32_t STG_TILE = 128 * 256;    // [128 rows][128 d] bf16
constexpr int kStages = 3;
constexpr uint32_t kSmem = 2 * KV_TILE + kStages * Q_TILE + 2 * P_TILE + 2 * STG_TILE + 256 + 1024;
constexpr uint32_t kTmemCols = 512;         // S: 0..63 | 64..127; O_part: 128..255 | 256..383
constexpr uint32_t kColO = 128;

__global__ void __launch_bounds__(kThreads, 1)
    sel_fwd_kv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const SelKvArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t k_s = sbase, v_s = sbase + KV_TILE;
  const uint32_t ring = sbase + 2 * KV_TILE;
  const uint32_t p_s0 = ring + kStages * Q_TILE;
  const uint32_t stg = p_s0 + 2 * P_TILE;
  const uint32_t bar_base = stg + 2 * STG_TILE;
  // barriers (8 bytes each); the double ones are indexed by batch & 1
  const uint32_t full0 = bar_base, empty0 = bar_base + 32, kv_bar = bar_base + 64, s_full = bar_base + 72,
                 s_free = bar_base + 88, p_full = bar_base + 104, p_free = bar_base + 120, o_full = bar_base + 136,
                 o_free = bar_base + 152, stg_full = bar_base + 168, stg_free = bar_base + 176,   // stg_free: two
                 tmem_slot = bar_base + 192;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full0 + 8 * i, kProd);
      mbar_init(empty0 + 8 * i, 1);
    }
    mbar_init(kv_bar, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full + 8 * i, 1);
      mbar_init(s_free + 8 * i, 128);
      mbar_init(p_full + 8 * i, 128);
      mbar_init(p_free + 8 * i, 1);
      mbar_init(o_full + 8 * i, 1);
      mbar_init(o_free + 8 * i, 128);
    }
    mbar_init(stg_full, 128);
    mbar_init(stg_free, 1);
    mbar_init(stg_free + 8, 1);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sgen + (tmem_slot - sbase));

  // ---- work item: (batch, kv head)-major so the resident CTAs share one head group's Q rows in L2 -------------
  const int G16 = (a.Hq / a.Hk) / 16;
  const int NB = (a.T + 63) / 64;
  const int blk = (int)(blockIdx.x % NB);
  const int bh = (int)(blockIdx.x / NB);
  const int b = bh / a.Hk, hk = bh % a.Hk;
  const int* rp = a.rev_ptr + (long long)bh * (NB + 1);
  const int ta_lo = rp[blk];
  const int nA = rp[blk + 1] - ta_lo;
  const int* list = a.rev_tok + (long long)bh * a.rev_cap + ta_lo;
  const int key0 = blk * 64;
  const int nb_sub = (nA + kTokB - 1) / kTokB;
  const int nb = nb_sub * G16;   // batches of this CTA (0: nothing selected this block)
  auto token = [&](int i) { return list[min(i, nA - 1)]; };

  if (nb > 0 && warp < kProd) {
    // ------------------------------- TMA producers ------------------------------------------------------------
    // a batch is 8 boxes of 4 KB, one per token: the token's [16 heads x 128 d] rows through a 4-D view of q
    // (64 columns, 8 rows, 2 column panels, row groups) land as [row group][panel][8 rows][128 B], so the 8-row swizzle
    // atoms of one panel sit 2 KB apart over the whole tile (SBO = 2048, second panel at +1 KB).  One box per token
    // instead of one per (token, panel): the gather is bound by the number of boxes.  Box x = 3 * lane + warp belongs
    // to this lane
    if (warp == 0 && lane == 0) {
      mbar_expect_tx(kv_bar, 2 * KV_TILE);
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        tma_load_4d(k_s + p * KV_PANEL, &tmK, kv_bar, p * 64, hk, key0, b);
        tma_load_4d(v_s + p * KV_PANEL, &tmV, kv_bar, p * 64, hk, key0, b);
      }
    }
    const int x = kProd * lane + warp;
    const bool has = x < kTokB;
    const int bj = x;
    const int nmine = (kTokB - warp + kProd - 1) / kProd;
    int tk_next = has ? token(bj) : 0;
    for (int n = 0; n < nb; ++n) {
      const int tk = tk_next;
      const int m1 = (n + 1) % nb_sub;
      tk_next = (has && n + 1 < nb) ? token(m1 * kTokB + bj) : 0;
      const int sub = n / nb_sub;
      const int hg = hk * G16 + sub;
      const int stage = n % kStages;
      const uint32_t ph = (n / kStages) & 1;
      const uint32_t fb = full0 + 8 * stage;
      int good = 1;
      if (lane == 0) {
        good = mbar_wait(empty0 + 8 * stage, ph ^ 1, DEV_ERR_EMPTY_WAIT) ? 1 : 0;
        if (good) mbar_expect_tx(fb, nmine * 4096);
      }
      if (!__shfl_sync(0xffffffffu, good, 0)) break;
      if (has) {
        const int qrow = (int)(((long long)b * a.Tq + (tk - a.q0)) * a.Hq + hg * 16);
        tma_load_4d(ring + stage * Q_TILE + bj * 4096, &tmQ, fb, 0, 0, 0, qrow >> 3);
      }
    }
  } else if (nb > 0 && warp == kMmaWarp) {
    // ------------------------------- MMA issuer ---------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, 0, 0);    // both operands K-major
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, 0, 1);   // A = P K-major, B = V MN-major
      bool ok = mbar_wait(kv_bar, 0, DEV_ERR_FULL_WAIT);
      const uint64_t dK = umma_smem_desc(k_s, 0, 1024);
      const uint64_t dVmn = umma_smem_desc(v_s, KV_PANEL, 1024);
      uint64_t dQ[kStages], dP[2];
#pragma unroll
      for (int i = 0; i < kStages; ++i) dQ[i] = umma_smem_desc(ring + i * Q_TILE, 0, 2048);
#pragma unroll
      for (int i = 0; i < 2; ++i) dP[i] = umma_smem_desc(p_s0 + i * P_TILE, 0, 1024);
      auto issue_s = [&](int n) {
        const int st = n % kStages;
        const uint64_t aq = st == 0 ? dQ[0] : st == 1 ? dQ[1] : dQ[2];
        const uint32_t col = (n & 1) * 64;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t aoff = (ks >> 2) * 1024 + (ks & 3) * 32, boff = (ks >> 2) * KV_PANEL + (ks & 3) * 32;
          umma_ss(tmem + col, umma_desc_advance(aq, aoff), umma_desc_advance(dK, boff), idesc_s, ks ? 1u : 0u);
        }
        umma_commit(empty0 + 8 * st);          // the Q tile is only needed for the scores
        umma_commit(s_full + 8 * (n & 1));
      };
      auto issue_o = [&](int n) {
        const uint64_t ap = (n & 1) ? dP[1] : dP[0];
        const uint32_t col = kColO + (n & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)   // contraction over the 64 keys, 16 per step
          umma_ss(tmem + col, umma_desc_advance(ap, ks * 32), umma_desc_advance(dVmn, ks * 2048), idesc_o, ks ? 1u : 0u);
        umma_commit(p_free + 8 * (n & 1));
        umma_commit(o_full + 8 * (n & 1));
      };
      // event loop: whichever of the next score product and the next P.V is ready
      int ns = 0, no = 0;
      uint64_t t_idle = 0;
      while (ok && no < nb) {
        bool progressed = false;
        if (ns < nb && mbar_test(full0 + 8 * (ns % kStages), (ns / kStages) & 1) &&
            (ns < 2 || mbar_test(s_free + 8 * (ns & 1), ((ns >> 1) - 1) & 1))) {
          tc_fence_after();
          issue_s(ns);
          ++ns;
          progressed = true;
        }
        if (no < ns && mbar_test(p_full + 8 * (no & 1), (no >> 1) & 1) &&
            (no < 2 || mbar_test(o_free + 8 * (no & 1), ((no >> 1) - 1) & 1))) {
          tc_fence_after();
          issue_o(no);
          ++no;
          progressed = true;
        }
        if (progressed) {
          t_idle = 0;
        } else {   // bounded: ~2 s without any progress is reported as a pipeline failure
          const uint64_t now = global_timer_ns();
          if (t_idle == 0) t_idle = now;
          else if (now - t_idle > 2000000000ull) {
            atomicCAS(&g_dev_error, 0, (int)DEV_ERR_FULL_WAIT);
            ok = false;
          }
        }
      }
    }
  } else if (nb > 0 && warp >= kDrainWarp) {
    // ------------------------------- drain warps: O_part, one row per thread -----------------------------------
    // accumulator -> bf16 -> staging tile (128 rows x 256 bytes; within a 128-byte half row the 16-byte chunk c sits at
    // position c ^ (row & 7): conflict-free writes, undone by the merge kernel) -> one bulk store: the batch's 8 tiles
    // are consecutive list positions, contiguous in the partial buffer when the KV head has one 16-head group
    const int quad = warp & 3;
    const int row = 32 * quad + lane;
    const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
    bool ok = true;
    for (int n = 0; ok && n < nb; ++n) {
      const int sub = n / nb_sub, mloc = n % nb_sub;
      ok = mbar_wait(o_full + 8 * (n & 1), (n >> 1) & 1, DEV_ERR_FULL_WAIT);
      // the store of batch n-2 has read this staging tile
      if (ok && n >= 2) ok = mbar_wait(stg_free + 8 * (n & 1), ((n >> 1) - 1) & 1, DEV_ERR_EMPTY_WAIT);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sb = stg + (uint32_t)(n & 1) * STG_TILE;
      uint8_t* sp = sgen + (sb - sbase) + row * 256;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {   // 32 columns at a time
        float vals[2][16];
        tmem_ld16(tmem + lane_addr + kColO + (n & 1) * 128 + q4 * 32, vals[0]);
        tmem_ld16(tmem + lane_addr + kColO + (n & 1) * 128 + q4 * 32 + 16, vals[1]);
        tmem_ld_wait();
        if (q4 == 3) {
          tc_fence_before();
          mbar_arrive(o_free + 8 * (n & 1));   // the accumulator is in registers
        }
#pragma unroll
        for (int c2 = 0; c2 < 4; ++c2) {
          const float* f = &vals[c2 >> 1][(c2 & 1) * 8];
          uint4 o;
          __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e) ho[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
          const int cc = q4 * 4 + c2;
          *reinterpret_cast<uint4*>(sp + (cc >> 3) * 128 + (((cc & 7) ^ (row & 7)) * 16)) = o;
        }
      }
      fence_proxy_async();
      mbar_arrive(stg_full);
      if (warp == kDrainWarp) {
        // one 4 KB bulk store per token, issued by eight lanes at once: a single 32 KB store is read out of shared
        // memory at about 20 bytes per cycle, which made this read-out the kernel's bottleneck
        bool good = mbar_wait(stg_full, n & 1, DEV_ERR_FULL_WAIT);
        const int nvalid = min(kTokB, nA - mloc * kTokB);
        if (good && G16 == 1 && lane == 0 && nvalid > 0) {
          bf16* dst = a.part + (((long long)bh * a.rev_cap + ta_lo + mloc * kTokB) * (16 * D));
          bulk_store_evict_first(dst, sb, (uint32_t)nvalid * 16 * D * 2);
        } else if (good && G16 > 1 && lane < nvalid) {
          bf16* dst = a.part + ((((long long)bh * a.rev_cap + ta_lo + mloc * kTokB + lane) * G16 + sub) * (16 * D));
          bulk_store_evict_first(dst, sb + lane * 16 * D * 2, 16 * D * 2);
        }
        bulk_commit();
        bulk_wait_read_but_one();   // batch n-1's stores have read their tile; this batch's stay in flight
        __syncwarp();
        if (lane == 0 && n > 0) mbar_arrive(stg_free + 8 * ((n - 1) & 1));
        ok = good;
      }
    }
    if (warp == kDrainWarp) bulk_wait_all();
  } else if (nb > 0 && warp >= kSoftWarp) {
    // ------------------------------- soft-max warps: one (token, head) row per thread --------------------------
    const int g = (warp - kSoftWarp) >> 2;      // group: batches n = g, g+2, ...
    const int quad = warp & 3;
    const int row = 32 * quad + lane;           // TMEM lane == tile row
    const int j = row >> 4, head = row & 15;
    const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
    const float sl2 = a.scale * kLog2e;
    bool ok = true;
    int t_next = (g < nb) ? token((g % nb_sub) * kTokB + j) : 0;
    for (int n = g; ok && n < nb; n += 2) {
      const int sub = n / nb_sub, mloc = n % nb_sub;
      const int i = mloc * kTokB + j;
      const bool live = i < nA;
      const int t = t_next;
      if (n + 2 < nb) t_next = token(((n + 2) % nb_sub) * kTokB + j);
      const uint32_t use = n >> 1;
      ok = mbar_wait(s_full + 8 * g, use & 1, DEV_ERR_FULL_WAIT);
      if (!ok) break;
      tc_fence_after();
      float sv[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(tmem + lane_addr + g * 64 + c * 16, *reinterpret_cast<float(*)[16]>(&sv[16 * c]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free + 8 * g);   // S is in registers: batch n+2 may overwrite this buffer
      // visible keys: key0 + c <= t (the block's first key always is, or the token would not be in this list)
      const int nvis = live ? min(64, t - key0 + 1) : 0;
      float m2 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        sv[c] = (c < nvis) ? sv[c] * sl2 : -INFINITY;
        m2 = fmaxf(m2, sv[c]);
      }
      float l = 0.f;
      uint32_t pw[32];
      if (nvis > 0) {
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float p0 = ex2(sv[c] - m2), p1 = ex2(sv[c + 1] - m2);
          pw[c / 2] = pack_bf16(p0, p1);
          // l is the sum of the rounded probabilities the tensor core multiplies, as in the query-major kernel
          const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&pw[c / 2]);
          l += __low2float(pr) + __high2float(pr);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) pw[c] = 0u;
      }
      if (use >= 1) {
        ok = mbar_wait(p_free + 8 * g, (use - 1) & 1, DEV_ERR_EMPTY_WAIT);   // P.V of batch n-2 has read this tile
        if (!ok) break;
      }
      uint8_t* prow = sgen + (p_s0 - sbase) + g * P_TILE + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) * 16)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
      fence_proxy_async();
      mbar_arrive(p_full + 8 * g);
      if (live) {
        float2* st = reinterpret_cast<float2*>(a.stats) + (((long long)bh * a.rev_cap + ta_lo + i) * G16 + sub) * 16 + head;
        *st = make_float2(m2, l);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemCols);
}

// Two warps per (batch, token, 16-head group), each half of the 16 heads: the visits' (m, l) and O tiles merged in slot
// order.  Lanes 0-7 hold the statistics of this half's heads; a load instruction of the warp covers 512 contiguous
// bytes of a tile.
__global__ void __launch_bounds__(256) sel_fwd_merge_kernel(const RevArgs a, const bf16* __restrict__ part,
                                                            const float* __restrict__ stats, bf16* __restrict__ o,
                                                            float* __restrict__ lse, const int G16) {
  constexpr int NV = 8 * D / 8 / 32;   // 16-byte vectors per lane: 4
  const long long w2 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long total = (long long)a.B * a.Tq * a.H * G16;
  const long long w = w2 >> 1;
  if (w >= total) return;
  const int hb = (int)(w2 & 1);
  const int lane = threadIdx.x & 31;
  const int sub = (int)(w % G16);
  const long long row = w / G16;   // (b, tl, h) row of idx / counts
  const int h = (int)(row % a.H);
  const long long bt = row / a.H;
  const int tl = (int)(bt % a.Tq), b = (int)(bt / a.Tq);
  const int t = a.q0 + tl;
  const long long bh = (long long)b * a.H + h;
  int mypos = -1;
  if (lane < a.S && rev_block(a, row, lane, t) >= 0) mypos = a.inv[row * a.S + lane];
  const unsigned live = __ballot_sync(0xffffffffu, mypos >= 0);
  auto tile_index = [&](int s) {
    const long long pos = __shfl_sync(0xffffffffu, mypos, s);
    return (bh * a.cap + pos) * G16 + sub;
  };
  // pass 1: M = max_v m_v per head.  Lane s fetches the maxima of slot s for this half's eight heads (all slots at
  // once, instead of one dependent load per slot), a butterfly takes the maximum over the slots, and every lane keeps
  // the value of head lane & 7, the head whose (m, l) it reads in pass 2.
  const int myhead = hb * 8 + (lane & 7);
  float mh[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) mh[e] = -INFINITY;
  if (mypos >= 0) {
    const float4* sp = reinterpret_cast<const float4*>(stats) + (((bh * a.cap + mypos) * G16 + sub) * 16 + hb * 8) / 2;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 v4 = sp[e];   // (m, l) of two heads
      mh[2 * e] = v4.x;
      mh[2 * e + 1] = v4.z;
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e)
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mh[e] = fmaxf(mh[e], __shfl_xor_sync(0xffffffffu, mh[e], off));
  float M = mh[0];
#pragma unroll
  for (int e = 1; e < 8; ++e) M = ((lane & 7) == e) ? mh[e] : M;
  float L = 0.f;
  float acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
  // vector u = 32 i + lane of this half tile belongs to head u / 16 = 2 i + lane / 16 (of this half)
  for (unsigned rem = live; rem;) {
    const int s = __ffs(rem) - 1;
    rem &= rem - 1;
    const long long ti = tile_index(s);
    const float2 ml = reinterpret_cast<const float2*>(stats)[ti * 16 + myhead];
    const float wgt = ex2(ml.x - M);   // lanes 0-7 (and their copies 8-31) hold head lane & 7
    L += wgt * ml.y;
    const uint4* src = reinterpret_cast<const uint4*>(part) + ti * (16 * D / 8) + hb * (8 * D / 8) + lane;
    uint4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) v[i] = __ldcs(src + 32 * i);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const float wi = __shfl_sync(0xffffffffu, wgt, 2 * i + (lane >> 4));
      const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(hv[k]);
        acc[i][2 * k] = fmaf(wi, f.x, acc[i][2 * k]);
        acc[i][2 * k + 1] = fmaf(wi, f.y, acc[i][2 * k + 1]);
      }
    }
  }
  const int Hq = a.H * G16 * 16;
  const long long orow0 = bt * Hq + (long long)(h * G16 + sub) * 16;   // first of the group's 16 (token, head) rows
  const float inv = L > 0.f ? 1.f / L : 0.f;
  if (lane < 8) lse[orow0 + myhead] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
  uint4* dst = reinterpret_cast<uint4*>(o + orow0 * D) + hb * (8 * D / 8);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const float ii = __shfl_sync(0xffffffffu, inv, 2 * i + (lane >> 4));
    const int u = 32 * i + lane;
    const int ud = (u & ~7) | ((u & 7) ^ ((u >> 4) & 7));   // undo the staging layout: position -> chunk
    uint4 ov;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) ho[k] = __floats2bfloat162_rn(acc[i][2 * k] * ii, acc[i][2 * k + 1] * ii);
    dst[ud] = ov;
  }
}

}  // namespace

bool sel_fwd_kv_supported(const SelKvArgs& a, int Dh) {
  return Dh == 128 && a.BS == 64 && a.S <= 32 && a.Hq % (16 * a.Hk) == 0;
}

int launch_sel_fwd_kv(const SelKvArgs& a, const RevArgs& r, cudaStream_t s) {
  CUtensorMap tmQ, tmK, tmV;
  const long long qrows = (long long)a.B * a.Tq * a.Hq;
  if (qrows > 0x7fffffffLL) {
    set_error("B*T*Hq exceeds the 2^31 rows a TMA coordinate can address");
    return -32;
  }
  // q rows as (64 columns, 8 rows, 2 column panels, groups of 8 rows): one box = 16 rows x 128 columns of one token
  const unsigned long long qd[4] = {64, 8, 2, (unsigned long long)(qrows / 8)};
  const unsigned long long qs[3] = {(unsigned long long)D * 2, 128, (unsigned long long)D * 2 * 8};
  const unsigned qb[4] = {64, 8, 2, 2};
  int rc = make_tmap_generic(&tmQ, a.q, 4, qd, qs, qb);
  if (!rc) rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.T, a.B, 64);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.T, a.B, 64);
  if (rc) return rc;
  cudaError_t e = cudaFuncSetAttribute(sel_fwd_kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
  if (e != cudaSuccess) return (int)e;
  const long long grid = (long long)a.B * a.Hk * ((a.T + 63) / 64);
  if (grid <= 0) return 0;
  if (grid > 0x7fffffffLL) {
    set_error("selected forward: grid too large");
    return -33;
  }
  sel_fwd_kv_kernel<<<(unsigned)grid, kThreads, kSmem, s>>>(tmQ, tmK, tmV, a);
  note_launches(1);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const int G16 = a.Hq / a.Hk / 16;
  const long long total = (long long)a.B * a.Tq * a.Hk * G16;
  sel_fwd_merge_kernel<<<(unsigned)((2 * total + 7) / 8), 256, 0, s>>>(r, a.part, a.stats, a.o, a.lse, G16);
  note_launches(1);
  return (int)cudaGetLastError();
}

int sel_fwd_kv_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
