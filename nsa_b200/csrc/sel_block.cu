// Selected-block attention for 64-key blocks, one query item per warp: forward (o_slc, lse_slc) and the dQ half of the
// backward.
//
// Reference behaviour: parallel_nsa_fwd_kernel (nsa/selection_attn.py:401-482) and the selected half of
// parallel_nsa_bwd_kernel_dq (nsa/selection_attn.py:276-356).  A query (b, t, kv head) visits the selected blocks
// whose first key is <= t (negative entries and entries past `counts` are skipped), masks keys > t inside a block,
// and soft-maxes over everything it visited.
//
// B200 design.  The kernel is bound by the L2 -> SM gather of the selected blocks (32 KB of K and V per visited
// block, used by one token's 16 heads only), so it is organised around keeping that gather busy.  One persistent
// CTA per SM holds four independent consumer/producer warp pairs.  A consumer warp owns a whole item (b, t, 16-head
// group): the 16 query heads are the M=16 rows of mma.sync m16n8k16 and the warp multiplies them against a whole
// gathered [64 keys x D] block at a time (eight independent accumulator chains, the running-maximum rescale paid
// once per 64 keys, nothing merged between warps).  Its producer warp TMA-gathers the item's K and V blocks by
// index into a private ring of [64 x D] slots (full/empty mbarriers, K and V alternating) and stages the item's Q
// (and dO) rows; every lane that issues a box waits for its own slot.  Nothing couples the four pairs, so a slow
// item never blocks another pair's gather, and a K slot is released as soon as the scores are computed (forward)
// or a V slot as soon as dP is (backward).  A shared ring with a single producer was measured 1.4x slower: slot
// reuse in ring order made every warp wait for the slowest one.
#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int BS = 64;                        // keys per selected block
constexpr int kMaxSlots = 64;

__device__ __forceinline__ int load_block_index(const void* idx, int idx64, long long pos) {
  long long v = idx64 ? reinterpret_cast<const long long*>(idx)[pos] : (long long)reinterpret_cast<const int*>(idx)[pos];
  if (v < 0 || v > (long long)(0x7fffffff / BS)) return -1;
  return (int)v;
}

// The ldmatrix / mma helpers below are written as volatile asm, so they execute in exactly the order given here: every
// B fragment is fetched one group ahead of the mma instructions that use it.
//
// acc[16 x NK] += A[16 x D] * Tile[row0 .. row0+NK)[D]^T, contraction step outermost: the mma instructions of a step
// write NK/8 different accumulators.
template <int D, int NK>
__device__ __forceinline__ void mma_a_bt_wide(float (&acc)[NK / 8][4], const uint32_t (&af)[D / 16][4], uint32_t base,
                                              uint32_t panel_bytes, int row0, int lane) {
  const int m = lane >> 3, rr = lane & 7;
  constexpr int NG = NK / 16;   // ldmatrix.x4 per contraction step
  uint32_t b[2][NG][4];
  auto fetch = [&](int ks, uint32_t (&dst)[NG][4]) {
#pragma unroll
    for (int n2 = 0; n2 < NG; ++n2) {
      const int row = row0 + n2 * 16 + (m >> 1) * 8 + rr;
      ldsm_x4(tile_addr(base, panel_bytes, row, ks * 2 + (m & 1)), dst[n2][0], dst[n2][1], dst[n2][2], dst[n2][3]);
    }
  };
  fetch(0, b[0]);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    if (ks + 1 < D / 16) fetch(ks + 1, b[(ks + 1) & 1]);
#pragma unroll
    for (int n2 = 0; n2 < NG; ++n2) {
      mma_bf16(acc[2 * n2], af[ks], b[ks & 1][n2][0], b[ks & 1][n2][1]);
      mma_bf16(acc[2 * n2 + 1], af[ks], b[ks & 1][n2][2], b[ks & 1][n2][3]);
    }
  }
}

// acc[16 x D] += P[16 x NK] * Tile[row0 .. row0+NK)[D], B fragments fetched four ldmatrix ahead.
template <int D, int NK>
__device__ __forceinline__ void mma_a_b_pipelined(float (&acc)[D / 8][4], const uint32_t (&pf)[NK / 16][4], uint32_t base,
                                                  uint32_t panel_bytes, int row0, int lane) {
  const int m = lane >> 3, rr = lane & 7;
  constexpr int G = 4;                       // ldmatrix.x4 per group
  constexpr int NGRP = (NK / 16) * (D / 16) / G;
  uint32_t b[2][G][4];
  auto fetch = [&](int grp, uint32_t (&dst)[G][4]) {
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int idx = grp * G + i, kk = idx / (D / 16), n2 = idx % (D / 16);
      const int row = row0 + kk * 16 + (m & 1) * 8 + rr;
      ldsm_x4_t(tile_addr(base, panel_bytes, row, n2 * 2 + (m >> 1)), dst[i][0], dst[i][1], dst[i][2], dst[i][3]);
    }
  };
  fetch(0, b[0]);
#pragma unroll
  for (int grp = 0; grp < NGRP; ++grp) {
    if (grp + 1 < NGRP) fetch(grp + 1, b[(grp + 1) & 1]);
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int idx = grp * G + i, kk = idx / (D / 16), n2 = idx % (D / 16);
      mma_bf16(acc[2 * n2], pf[kk], b[grp & 1][i][0], b[grp & 1][i][1]);
      mma_bf16(acc[2 * n2 + 1], pf[kk], b[grp & 1][i][2], b[grp & 1][i][3]);
    }
  }
}

// Hand a tile back after ldmatrix.  The loaded fragments are folded into `dep`, which is stored (volatile) to a scratch
// word before the arrive: the store cannot be issued before the loads have returned, and neither the compiler nor
// the assembler may drop it or move the arrive in front of it.  A plain arrive after the ldmatrix instructions is
// not enough: nothing orders it behind loads whose results are not used yet.
__device__ __forceinline__ void mbar_arrive_after(uint32_t bar, uint32_t scratch, uint32_t dep) {
  asm volatile("st.volatile.shared::cta.u32 [%1], %2;\n\t{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar),
               "r"(scratch), "r"(dep)
               : "memory");
}
template <int N>
__device__ __forceinline__ uint32_t fold_frags(const uint32_t (&f)[N][4]) {
  uint32_t x = 0;
#pragma unroll
  for (int i = 0; i < N; ++i) x ^= f[i][0] ^ f[i][1] ^ f[i][2] ^ f[i][3];
  return x;
}

struct Item {
  int b, tl, t, hkv;
  long long row;   // (b, tl, hkv) row of the index / counts tensors
  long long qrow;  // first of the 16 (token, head) rows
  bool valid;
};

__device__ __forceinline__ Item decode_item(const SelArgs& a, long long idx, long long total, int HG, int G16) {
  Item it;
  it.valid = idx < total;
  if (!it.valid) idx = 0;
  int hg;
  if (total <= 0x7fffffffLL) {   // 32-bit divisions: the 64-bit ones cost hundreds of cycles per item
    const unsigned i = (unsigned)idx, th = i / (unsigned)HG;
    hg = (int)(i - th * (unsigned)HG);
    it.b = (int)(th / (unsigned)a.Tq);
    it.tl = a.Tq - 1 - (int)(th - (unsigned)it.b * (unsigned)a.Tq);
  } else {
    hg = (int)(idx % HG);
    it.tl = a.Tq - 1 - (int)((idx / HG) % a.Tq);
    it.b = (int)(idx / ((long long)HG * a.Tq));
  }
  it.t = a.q0 + it.tl;
  it.hkv = hg / G16;
  it.row = ((long long)it.b * a.Tq + it.tl) * a.Hkv + it.hkv;
  it.qrow = ((long long)it.b * a.Tq + it.tl) * a.Hq + hg * 16;
  return it;
}

// The selection entry this lane holds for an item (or -1), to be turned into the item's valid mask by a ballot.
__device__ __forceinline__ int fetch_entry(const SelArgs& a, const Item& it, int lane) {
  if (!it.valid) return -1;
  int cnt = a.S;
  if (a.counts) cnt = min(cnt, a.counts[it.row]);
  if (lane >= cnt) return -1;
  const int blk = load_block_index(a.idx, a.idx64, it.row * a.S + lane);
  return (blk >= 0 && (long long)blk * BS <= it.t) ? blk : -1;
}

template <int D, bool BWD, int kWarps>
__global__ void __launch_bounds__(2 * kWarps * 32, 1)
    sel_block_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO, const SelArgs a,
                     const int spw) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int NP = D / 64;                        // 64-column panels per row
  constexpr uint32_t panel_bytes = BS * 128;        // one panel of a K or V block
  constexpr uint32_t slot_bytes = panel_bytes * NP;
  constexpr uint32_t qpanel_bytes = 16 * 128;       // one panel of a 16-row Q / dO tile
  constexpr uint32_t qtile_bytes = qpanel_bytes * NP;
  constexpr int NQ = BWD ? 2 : 1;                   // Q, and dO in the backward
  const int nst = spw * kWarps;                     // slots in all rings
  const uint32_t q_off = nst * slot_bytes;          // [kWarps][NQ] tiles
  const uint32_t bar_base = sbase + q_off + kWarps * NQ * qtile_bytes;
  auto full_bar = [&](int i) { return bar_base + 8u * i; };
  auto empty_bar = [&](int i) { return bar_base + 8u * (nst + i); };
  auto qfull_bar = [&](int w) { return bar_base + 8u * (2 * nst + w); };
  auto qempty_bar = [&](int w) { return bar_base + 8u * (2 * nst + kWarps + w); };
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(sgen + (bar_base - sbase) + 8 * (2 * nst + 2 * kWarps));
  const uint32_t dep_scratch = bar_base + 8u * (2 * nst + 2 * kWarps) + 16 + 4 * (warp % kWarps);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < nst; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), 1);
    }
    for (int w = 0; w < kWarps; ++w) {
      mbar_init(qfull_bar(w), 1);
      mbar_init(qempty_bar(w), 1);
    }
    fence_mbar_init();
  }
  __syncthreads();

  const int HG = a.Hq / 16;
  const int G16 = (a.Hq / a.Hkv) / 16;
  const long long total = (long long)a.B * a.Tq * HG;
  const int cw = warp % kWarps;                                   // the consumer warp this warp is or serves
  const long long first = (long long)blockIdx.x * kWarps + cw;    // its items: first, first + step, ...
  const long long step = (long long)gridDim.x * kWarps;
  const int ring0 = cw * spw;                                     // first slot of its private ring
  int rs = 0;         // ring position of the next block's K slot (V takes the one after) and its phase parity,
  uint32_t rp = 0;    // stepped without divisions
  auto ring_advance2 = [&]() {
    rs += 2;
    if (rs >= spw) {
      rs -= spw;
      rp ^= 1;
    }
  };
  uint32_t qn = 0;    // Q tiles staged so far

  if (warp >= kWarps) {
    // ------------------------------- producer of consumer warp cw ---------------------------------
    // lane -> (K or V, panel) for block boxes, (Q or dO, panel) for row tiles; every issuing lane waits for its own
    // slot, the first lane of a slot also arms the barrier
    const int bkv = lane / NP, bp = lane % NP;
    const int qwhich = lane / NP, qp = lane % NP;
    int ent_next = fetch_entry(a, decode_item(a, first, total, HG, G16), lane);
    for (long long idx = first; idx < total; idx += step) {
      const Item item = decode_item(a, idx, total, HG, G16);
      const int ent = ent_next;
      unsigned mask = __ballot_sync(0xffffffffu, ent >= 0);
      ent_next = fetch_entry(a, decode_item(a, idx + step, total, HG, G16), lane);
      if (mask == 0) continue;
      int good = 1;
      if (lane < NQ * NP) {
        good = mbar_wait_abortable(qempty_bar(cw), (qn & 1) ^ 1, DEV_ERR_EMPTY_WAIT, abort_flag) ? 1 : 0;
        if (good) {
          if (lane == 0) mbar_expect_tx(qfull_bar(cw), NQ * qtile_bytes);
          tma_load_2d(sbase + q_off + (cw * NQ + qwhich) * qtile_bytes + qp * qpanel_bytes, qwhich ? &tmDO : &tmQ,
                      qfull_bar(cw), qp * 64, (int)item.qrow);
        }
      }
      ++qn;
      if (!__all_sync(0xffffffffu, good)) return;
      while (mask) {
        const int bit = __ffs(mask) - 1;
        mask &= mask - 1;
        const int blk = __shfl_sync(0xffffffffu, ent, bit);
        if (lane < 2 * NP) {
          // Forward: K takes the ring position `rs`, V the next one.  Backward: V first, then K -- V is released
          // after dP, well before the block ends, and the slot freed early is the one the SECOND tensor of the next
          // block reuses (three slots per ring), so both tensors of the next block land while this one computes.
          int stage = rs;
          uint32_t par = rp;
          if ((BWD ? !bkv : bkv) && ++stage == spw) {
            stage = 0;
            par ^= 1;
          }
          stage += ring0;
          good = mbar_wait_abortable(empty_bar(stage), par ^ 1, DEV_ERR_EMPTY_WAIT, abort_flag) ? 1 : 0;
          if (good) {
            if (bp == 0) mbar_expect_tx(full_bar(stage), slot_bytes);
            tma_load_4d(sbase + stage * slot_bytes + bp * panel_bytes, bkv ? &tmV : &tmK, full_bar(stage), bp * 64,
                        item.hkv, blk * BS, item.b);
          }
        }
        ring_advance2();
        if (!__all_sync(0xffffffffu, good)) return;
      }
    }
    return;
  }

  // --------------------------------- consumers -------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const float sl2 = a.scale * kLog2e;
  const uint32_t qtile = sbase + q_off + warp * NQ * qtile_bytes;
  int ent_next = fetch_entry(a, decode_item(a, first, total, HG, G16), lane);
  for (long long idx = first; idx < total; idx += step) {
    const Item me = decode_item(a, idx, total, HG, G16);
    const int my_ent = ent_next;
    unsigned my_mask = __ballot_sync(0xffffffffu, my_ent >= 0);
    ent_next = fetch_entry(a, decode_item(a, idx + step, total, HG, G16), lane);

    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (my_mask) {
      // backward-only row operands: issued before the Q wait so their latency overlaps it
      float lse2[2] = {0.f, 0.f}, dl[2] = {0.f, 0.f}, gt[2] = {1.f, 1.f};
      if constexpr (BWD) {
        lse2[0] = a.lse[me.qrow + g] * kLog2e;
        lse2[1] = a.lse[me.qrow + g + 8] * kLog2e;
        dl[0] = a.delta[me.qrow + g];
        dl[1] = a.delta[me.qrow + g + 8];
        if (a.gate) {
          gt[0] = __bfloat162float(a.gate[me.qrow + g]);
          gt[1] = __bfloat162float(a.gate[me.qrow + g + 8]);
        }
      }
      uint32_t qf[D / 16][4];
      uint32_t dof[BWD ? D / 16 : 1][4];
      bool ok = mbar_wait_abortable(qfull_bar(warp), qn & 1, DEV_ERR_FULL_WAIT, abort_flag);
      load_a_frags<D>(qf, qtile, qpanel_bytes, 0, lane);
      if constexpr (BWD) load_a_frags<D>(dof, qtile + qtile_bytes, qpanel_bytes, 0, lane);
      ++qn;
      // The Q tile is handed back once its fragments are in registers (see mbar_arrive_after: a plain arrive here let
      // the next item's TMA overwrite the tile before it had been read, one wrong item in roughly every fourth launch).
      {
        uint32_t dep = fold_frags(qf);
        if constexpr (BWD) dep ^= fold_frags(dof);
        dep = __reduce_or_sync(0xffffffffu, dep);   // every lane's fragments
        if (lane == 0) mbar_arrive_after(qempty_bar(warp), dep_scratch, dep);
      }

      while (my_mask) {
        const int bit = __ffs(my_mask) - 1;
        my_mask &= my_mask - 1;
        const int blk = __shfl_sync(0xffffffffu, my_ent, bit);
        const bool edge = blk * BS + BS - 1 > me.t;    // the block that contains the query's own position
        // ring positions of the block's two tensors: K then V in the forward, V then K in the backward (see the producer)
        const int first_bar = ring0 + rs;
        const uint32_t first_par = rp;
        int ss = rs + 1;
        uint32_t second_par = rp;
        if (ss == spw) {
          ss = 0;
          second_par ^= 1;
        }
        const int second_bar = ring0 + ss;
        const int kbar = BWD ? second_bar : first_bar, vbar = BWD ? first_bar : second_bar;
        const uint32_t kpar = BWD ? second_par : first_par, vpar = BWD ? first_par : second_par;
        ring_advance2();
        const uint32_t kbase = sbase + kbar * slot_bytes, vbase = sbase + vbar * slot_bytes;
        ok = ok && mbar_wait_abortable(full_bar(kbar), kpar, DEV_ERR_FULL_WAIT, abort_flag);
        if constexpr (!BWD) {
          const int key0 = blk * BS + 2 * tq;  // key of sc[0][0]; sc[nt][c]: + 8*nt + (c&1)
          float sc[BS / 8][4];
#pragma unroll
          for (int i = 0; i < BS / 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
          if (ok) mma_a_bt_wide<D, BS>(sc, qf, kbase, panel_bytes, 0, lane);
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(kbar));
          // maxima on the raw scores (the scale is positive: sel_block_supported), scale folded into the exponent's FMA
          float mx[2] = {-INFINITY, -INFINITY};
          if (edge) {
#pragma unroll
            for (int nt = 0; nt < BS / 8; ++nt)
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int key = key0 + 8 * nt + (c & 1);
                if (key > me.t) sc[nt][c] = -INFINITY;
                mx[c >> 1] = fmaxf(mx[c >> 1], sc[nt][c]);
              }
          } else {
#pragma unroll
            for (int nt = 0; nt < BS / 8; ++nt)
#pragma unroll
              for (int c = 0; c < 4; ++c) mx[c >> 1] = fmaxf(mx[c >> 1], sc[nt][c]);
          }
          float alpha[2];
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const float mnew = fmaxf(m_run[rr], quad_max(mx[rr]) * sl2);
            const float muse = (mnew == -INFINITY) ? 0.f : mnew;
            alpha[rr] = ex2(m_run[rr] - muse);
            m_run[rr] = mnew;
            float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < BS / 8; ++nt) {
              const float e0 = ex2(fmaf(sc[nt][2 * rr], sl2, -muse)), e1 = ex2(fmaf(sc[nt][2 * rr + 1], sl2, -muse));
              sc[nt][2 * rr] = e0;
              sc[nt][2 * rr + 1] = e1;
              rs0 += e0;
              rs1 += e1;
            }
            l_run[rr] = l_run[rr] * alpha[rr] + (rs0 + rs1);
          }
          // the accumulator is rescaled only when some row's maximum moved
          if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
              acc[i][0] *= alpha[0];
              acc[i][1] *= alpha[0];
              acc[i][2] *= alpha[1];
              acc[i][3] *= alpha[1];
            }
          }
          uint32_t pf[BS / 16][4];
          acc_to_a_frags<BS / 8>(pf, sc);
          ok = ok && mbar_wait_abortable(full_bar(vbar), vpar, DEV_ERR_FULL_WAIT, abort_flag);
          if (ok) mma_a_b_pipelined<D, BS>(acc, pf, vbase, panel_bytes, 0, lane);
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(vbar));
        } else {
          ok = ok && mbar_wait_abortable(full_bar(vbar), vpar, DEV_ERR_FULL_WAIT, abort_flag);
          constexpr int CK = 32;   // keys per pass: scores and dP of a pass stay in registers
#pragma unroll
          for (int h = 0; h < BS / CK; ++h) {
            const int key0 = blk * BS + h * CK + 2 * tq;
            float sc[CK / 8][4], dp[CK / 8][4];
#pragma unroll
            for (int i = 0; i < CK / 8; ++i) {
              sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
              dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
            }
            if (ok) {
              mma_a_bt_wide<D, CK>(sc, qf, kbase, panel_bytes, h * CK, lane);
              mma_a_bt_wide<D, CK>(dp, dof, vbase, panel_bytes, h * CK, lane);
            }
            if (h == BS / CK - 1) {   // V is not needed any more
              __syncwarp();
              if (lane == 0) mbar_arrive(empty_bar(vbar));
            }
#pragma unroll
            for (int nt = 0; nt < CK / 8; ++nt)
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int rr = c >> 1;
                float p = ex2(sc[nt][c] * sl2 - lse2[rr]);
                if (edge && key0 + 8 * nt + (c & 1) > me.t) p = 0.f;
                sc[nt][c] = p * (gt[rr] * dp[nt][c] - dl[rr]);
              }
            uint32_t dsf[CK / 16][4];
            acc_to_a_frags<CK / 8>(dsf, sc);
            if (ok) mma_a_b_pipelined<D, CK>(acc, dsf, kbase, panel_bytes, h * CK, lane);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(kbar));
        }
      }
    }

    // ---- epilogue: this warp's 16 rows ---------------------------------------------------------
    if (me.valid) {
      float sc0, sc1;
      if constexpr (!BWD) {
        const float l0 = quad_sum(l_run[0]), l1 = quad_sum(l_run[1]);
        sc0 = (l0 > 0.f) ? 1.f / l0 : 0.f;
        sc1 = (l1 > 0.f) ? 1.f / l1 : 0.f;
        if (tq == 0) {
          a.lse[me.qrow + g] = (l0 > 0.f) ? (m_run[0] + log2f(l0)) * kLn2 : -INFINITY;
          a.lse[me.qrow + g + 8] = (l1 > 0.f) ? (m_run[1] + log2f(l1)) * kLn2 : -INFINITY;
        }
      } else {
        sc0 = sc1 = a.scale;
      }
      bf16* d0 = (BWD ? a.dq : a.o) + (me.qrow + g) * D + 2 * tq;
      bf16* d1 = d0 + 8 * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        float x0 = acc[i][0] * sc0, x1 = acc[i][1] * sc0, y0 = acc[i][2] * sc1, y1 = acc[i][3] * sc1;
        if (BWD && a.accumulate) {
          const __nv_bfloat162 o0 = *reinterpret_cast<const __nv_bfloat162*>(d0 + 8 * i);
          const __nv_bfloat162 o1 = *reinterpret_cast<const __nv_bfloat162*>(d1 + 8 * i);
          x0 += __low2float(o0);
          x1 += __high2float(o0);
          y0 += __low2float(o1);
          y1 += __high2float(o1);
        }
        *reinterpret_cast<__nv_bfloat162*>(d0 + 8 * i) = __floats2bfloat162_rn(x0, x1);
        *reinterpret_cast<__nv_bfloat162*>(d1 + 8 * i) = __floats2bfloat162_rn(y0, y1);
      }
    }
  }
}

template <int D, bool BWD, int kWarps>
int launch_nw(const SelArgs& a, cudaStream_t s) {
  constexpr int kThreads = 2 * kWarps * 32;
  CUtensorMap tmK, tmV, tmQ, tmDO;
  int rc = make_tmap_rows4d(&tmK, a.k, D, a.Hkv, a.T, a.B, BS);
  if (rc) return rc;
  rc = make_tmap_rows4d(&tmV, a.v, D, a.Hkv, a.T, a.B, BS);
  if (rc) return rc;
  const long long qrows = (long long)a.B * a.Tq * a.Hq;
  rc = make_tmap_rows2d(&tmQ, a.q, D, qrows, 16);
  if (rc) return rc;
  rc = make_tmap_rows2d(&tmDO, BWD ? a.dout : a.q, D, qrows, 16);
  if (rc) return rc;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const int slot_bytes = BS * D * 2;
  const int fixed = kWarps * (BWD ? 2 : 1) * 16 * D * 2 + (2 * kMaxSlots + 2 * kWarps) * 8 + 64 + 1024;
  int spw = (max_smem - fixed) / slot_bytes / kWarps;   // slots per private ring
  if (spw > kMaxSlots / kWarps) spw = kMaxSlots / kWarps;
  if (spw < 2) {
    set_error("selected attention: not enough shared memory for the block rings");
    return -30;
  }
  const int smem = fixed + spw * kWarps * slot_bytes;
  auto kern = sel_block_kernel<D, BWD, kWarps>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * a.Tq * (a.Hq / 16);
  const long long ctas = (total + kWarps - 1) / kWarps;
  const int grid = (int)(ctas < num_sms() ? ctas : num_sms());
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, smem, s>>>(tmK, tmV, tmQ, tmDO, a, spw);
  note_launches(1);
  return (int)cudaGetLastError();
}

template <int D, bool BWD>
int launch(const SelArgs& a, cudaStream_t s) {
  // four pairs x three slots measured faster than three pairs x four slots (0.81 vs 1.04 ms forward, 0.95 vs 1.17 ms
  // backward per 8192-token sequence)
  return launch_nw<D, BWD, 4>(a, s);
}

}  // namespace

bool sel_block_supported(const SelArgs& a, int D) {
  return a.BS == BS && a.S <= 32 && (D == 128 || D == 64) && a.scale > 0.f;
}

int launch_sel_block(const SelArgs& a, int D, bool bwd, cudaStream_t s) {
  if (D == 128) return bwd ? launch<128, true>(a, s) : launch<128, false>(a, s);
  if (D == 64) return bwd ? launch<64, true>(a, s) : launch<64, false>(a, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}
int sel_block_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
