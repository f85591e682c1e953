// Key/value-major backward on tcgen05 (head_dim 128, 64-key blocks): dK,dV of the selected + sliding-window
// branches and dCK,dCV of the compressed branch.  Same work decomposition and reference semantics as kv_bwd.cu
// (nsa/selection_attn.py:151-253 through a reverse index; nsa/triton_attention.py:219-318), different engine.
//
// One CTA owns 64 keys.  Query tokens that see them arrive in batches of 8: the 8 x 16 (token, head) rows form a
// [128 x D] tile of Q and of dO in shared memory (8 TMA boxes of 16 rows each, 128-byte swizzle).  Per batch, one
// thread issues four groups of tcgen05.mma (accumulators in TMEM):
//     S   [128 rows x 64 keys] = Qg . K^T          A = Qg (K-major),  B = K  (K-major)
//     dP  [128 rows x 64 keys] = dOg . V^T         A = dOg (K-major), B = V  (K-major)
//     dV^T[128 d    x 64 keys] += dOg^T . (g P)    A = dOg (MN-major), B = P  (MN-major, written by the soft-max warps)
//     dK^T[128 d    x 64 keys] += Qg^T . dS        A = Qg (MN-major),  B = dS (MN-major)
// Eight soft-max warps own half a row per thread (lse, delta, gate and the causal/window mask are thread-local, no
// shuffles; warps 2-5 take key columns 0-31, warps 6-9 columns 32-63 of the same TMEM lanes): they read S and dP
// from TMEM, form P and dS = P (g dP - delta), and store both as bf16 tiles.
// The MMA thread issues S/dP of batch n+1 before dV/dK of batch n, so the tensor core works while the soft-max
// warps compute.  dV^T and dK^T stay in TMEM for the CTA's whole token stream and are stored once.
// Optionally (mode 0) the selected branch's dQ comes out of this kernel too: dS of a batch is already in shared memory,
// so one more product  dQ_part[128 rows x 128 d] = dS . K  (A = dS K-major, B = K MN-major, a third accumulator in TMEM)
// gives the batch's contribution to dQ, which the soft-max warps store as bf16 tiles indexed by the batch's positions
// in the reverse-index list; a small kernel later sums every token's tiles in slot order.  That replaces the
// query-major dQ kernel, which gathers every selected block again (32 KB per visit for 16 rows) and recomputes S and dP.
// Every wait is bounded; on a time-out the role records an error and leaves its loop.
#include "kernels.h"
#include "tc.cuh"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int D = 128;
constexpr int kProd = 2;                   // TMA producer warps (a warp's TMA instructions run one after another,
                                           // ~900 cycles each whatever their size, so the boxes of a batch are
                                           // spread over two warps and issued by one instruction per warp)
constexpr int kMmaWarp = 2;                // issues S and dP
constexpr int kMma2Warp = 3;               // issues dV, dK and the dQ partials: tcgen05.mma costs its issuing thread
                                           // ~60 cycles per instruction, so two threads issue the kernel's 32-36 MMAs
                                           // per batch
constexpr int kSoftWarp = 4;               // eight soft-max / epilogue warps
constexpr int kDrainWarp = 12;             // four more warps read the dQ partials out of tensor memory
constexpr int kThreads = 16 * 32;          // 512: four warpgroups, registers redistributed by setmaxnreg
constexpr int kSoftThreads = 256;          // two threads per row: key columns 0-31 and 32-63
constexpr int kDrainThreads = 128;         // one thread per row
constexpr int kTokB = 8;                   // tokens per batch (x16 heads = 128 rows)
constexpr uint32_t KV_PANEL = 64 * 128;    // [64 keys][64 ch]
constexpr uint32_t KV_TILE = 2 * KV_PANEL; // 16 KB
constexpr uint32_t Q_PANEL = 128 * 128;    // [128 rows][64 ch]
constexpr uint32_t Q_TILE = 2 * Q_PANEL;   // 32 KB
constexpr uint32_t STAGE = 2 * Q_TILE;     // Q + dO
constexpr uint32_t P_TILE = 128 * 128;     // [128 rows][64 keys]
constexpr int kStages = 2;
constexpr uint32_t kSmem = 2 * KV_TILE + kStages * STAGE + 4 * P_TILE + 256 + 1024;
constexpr uint32_t kTmemCols = 512;        // two S/dP buffers: S 0..63, dP 64..127 | 128..255; dV^T 256..319, dK^T 320..383
constexpr uint32_t kColDV = 256, kColDK = 320, kColDQ = 384;   // dQ_part: 384..511

struct Stream {  // the token stream of one CTA: branch A (list or range) then branch B (window range)
  int nA, nB, ta_lo, tb_lo;
  const int* list;
};

__device__ __forceinline__ int stream_token(const Stream& st, int br, int i) {
  if (br == 0) {
    if (i >= st.nA) i = st.nA - 1;
    return st.list ? st.list[st.ta_lo + i] : st.ta_lo + i;
  }
  if (i >= st.nB) i = st.nB - 1;
  return st.tb_lo + i;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    kv_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDOa,
                     const __grid_constant__ CUtensorMap tmDOb, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQw,
                     const __grid_constant__ CUtensorMap tmDOw, const KvArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t k_s = sbase, v_s = sbase + KV_TILE;
  const uint32_t ring = sbase + 2 * KV_TILE;
  const uint32_t p_s0 = ring + kStages * STAGE;   // two [P | dS] tile pairs
  const uint32_t bar_base = p_s0 + 4 * P_TILE;
  // barriers
  // sdp_* and pds_* exist twice (index = batch & 1): S/dP of batch n+1 are computed while the soft-max warps still
  // hold batch n, and P/dS of batch n+1 are written while dV/dK of batch n still read theirs
  const uint32_t full0 = bar_base, empty0 = bar_base + 16, kv_bar = bar_base + 32, sdp_full = bar_base + 40,
                 sdp_free = bar_base + 56, pds_full = bar_base + 72, pds_free = bar_base + 88, acc_full = bar_base + 104,
                 tmem_slot = bar_base + 112, dq_full = bar_base + 120, dq_free = bar_base + 128, stg_full = bar_base + 136,
                 stg_free = bar_base + 144;   // stg_free: two barriers, one per P/dS pair
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(full0 + 8 * i, kProd);
      mbar_init(empty0 + 8 * i, 1);
    }
    mbar_init(kv_bar, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(sdp_full + 8 * i, 1);
      mbar_init(sdp_free + 8 * i, kSoftThreads);
      mbar_init(pds_full + 8 * i, kSoftThreads);
      mbar_init(pds_free + 8 * i, 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, kDrainThreads);
    mbar_init(stg_full, kDrainThreads);
    mbar_init(stg_free, 1);
    mbar_init(stg_free + 8, 1);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sgen + (tmem_slot - sbase));

  // ---- decode the work item (same mapping as kv_bwd.cu) -----------------------------------------------
  const int G16 = (a.Hq / a.Hk) / 16;
  int b, hk, blk, seg = 0;
  Stream st = {0, 0, 0, 0, nullptr};
  bool skip = false;
  {
    long long item = blockIdx.x;
    const int BH = a.B * a.Hk;
    if (MODE == 0) {
      // (batch, kv head)-major: the CTAs resident at one time share one 16-head group's Q and dO rows (67 MB at
      // T = 8192), which then stay in L2; block-major order made every gather a DRAM access
      const int NB = (a.T + 63) / 64;
      blk = (int)(item % NB);
      const int bh = (int)(item / NB);
      b = bh / a.Hk;
      hk = bh % a.Hk;
      if (a.rev_ptr) {
        const int* rp = a.rev_ptr + (long long)bh * (NB + 1);
        st.ta_lo = rp[blk];
        st.nA = rp[blk + 1] - rp[blk];
        st.list = a.rev_tok + (long long)bh * a.rev_cap;
      }
      if (a.window > 0) {
        st.tb_lo = max(blk * 64, a.q0);
        st.nB = max(0, min(a.q0 + a.Tq, blk * 64 + 63 + a.window) - st.tb_lo);
      }
    } else {
      seg = (int)(item % a.nseg);
      item /= a.nseg;
      const int NT = (a.Lk + 63) / 64;
      blk = (int)(item % NT);
      const int bh = (int)(item / NT);
      b = bh / a.Hk;
      hk = bh % a.Hk;
      const int first = a.causal ? blk * 64 * a.cstride + a.cblock : 0;
      st.ta_lo = max(first, a.q0 + seg * a.seg_len);
      st.nA = min(a.q0 + a.Tq, a.q0 + (seg + 1) * a.seg_len) - st.ta_lo;
      if (st.nA <= 0) skip = true;  // the reducer skips this segment too
    }
  }
  const int key0 = blk * 64;
  const int nbA = (st.nA + kTokB - 1) / kTokB, nbB = (st.nB + kTokB - 1) / kTokB;
  const int nb_sub = nbA + nbB;             // batches per 16-head sub-group
  const int nb = skip ? 0 : nb_sub * G16;   // batches of this CTA
  const bool emit_dq = MODE == 0 && a.dq_part != nullptr;   // selected-branch batches also leave their dQ partial

  // 512 threads start with 128 registers each; the soft-max warps need 168.  Warps 0-3 (TMA, MMA) and 12-15 (drain)
  // give registers back, warps 4-11 take them (each instruction is executed by a whole warpgroup).
  // Each role's code follows its own setmaxnreg, so the compiler allocates registers for it under that budget.
  // Budget (setmaxnreg moves registers inside the pool the CTA was launched with, 512 x 128 = 65536; an inc that the
  // pool cannot satisfy blocks for ever): 128 x 80 + 256 x 168 + 128 x 88 = 64512.
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
  if (!skip && warp < kProd) {
    // ------------------------------- TMA producers -----------------------------------------------
    // A batch of gathered tokens (a reverse-index list) is 32 boxes of 2 KB: (token j, Q or dO, column panel).  Box
    // x = 3 * lane + warp belongs to this lane; every producer warp issues its 10 or 11 boxes with a single instruction
    // and arms the stage's barrier with their byte count.  Token ids are fetched one batch ahead.
    // A batch of consecutive tokens (the window's range, the compressed branch's range) is 4 boxes of 16 KB instead:
    // [64 columns x 16 heads x 8 tokens] through the 4-D maps, rows past the last token read as zero.
    if (warp == 0 && lane == 0) {
      mbar_expect_tx(kv_bar, 2 * KV_TILE);
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        tma_load_4d(k_s + p * KV_PANEL, &tmK, kv_bar, p * 64, hk, key0, b);
        tma_load_4d(v_s + p * KV_PANEL, &tmV, kv_bar, p * 64, hk, key0, b);
      }
    }
    const int x = kProd * lane + warp;          // this lane's box of every batch (none if >= 32)
    const bool has = x < 4 * kTokB;
    const int bj = x & 7, bwhich = (x >> 3) & 1, bp = x >> 4;
    const int nmine = (4 * kTokB - warp + kProd - 1) / kProd;   // boxes this warp issues per batch
    const bool has_w = x < 4;                                   // this lane's 16 KB box of a consecutive-token batch
    const int nmine_w = (4 - warp + kProd - 1) / kProd;
    auto batch_token = [&](int n) {
      if (n >= nb || !has) return 0;
      const int m = n % nb_sub;
      const int br = m < nbA ? 0 : 1;
      return stream_token(st, br, (br == 0 ? m : m - nbA) * kTokB + bj);
    };
    int tk_next = batch_token(0);
    for (int n = 0; n < nb; ++n) {
      const int tk = tk_next;
      tk_next = batch_token(n + 1);
      const int sub = n / nb_sub, m = n % nb_sub;
      const int br = m < nbA ? 0 : 1;
      const int hg = hk * G16 + sub;
      const CUtensorMap* tmDO = br == 0 ? &tmDOa : &tmDOb;
      const bool contig = br == 1 || st.list == nullptr;
      const int stage = n % kStages;
      const uint32_t ph = (n / kStages) & 1;
      const uint32_t fb = full0 + 8 * stage;
      int good = 1;
      if (lane == 0) {
        good = mbar_wait(empty0 + 8 * stage, ph ^ 1, DEV_ERR_EMPTY_WAIT) ? 1 : 0;
        if (good) mbar_expect_tx(fb, contig ? nmine_w * 16384 : nmine * 2048);
      }
      if (!__shfl_sync(0xffffffffu, good, 0)) break;
      if (contig) {
        if (has_w) {
          const uint32_t q_s = ring + stage * STAGE, do_s = q_s + Q_TILE;
          const int t0 = (br == 0 ? st.ta_lo + m * kTokB : st.tb_lo + (m - nbA) * kTokB) - a.q0;
          const int wh = x >> 1, pp = x & 1;
          tma_load_4d((wh ? do_s : q_s) + pp * Q_PANEL, wh ? &tmDOw : &tmQw, fb, pp * 64, hg * 16, t0, b);
        }
      } else if (has) {
        const uint32_t q_s = ring + stage * STAGE, do_s = q_s + Q_TILE;
        const int qrow = (int)(((long long)b * a.Tq + (tk - a.q0)) * a.Hq + hg * 16);
        tma_load_2d((bwhich ? do_s : q_s) + bp * Q_PANEL + bj * 2048, bwhich ? tmDO : &tmQ, fb, bp * 64, qrow);
      }
    }
  } else if (!skip && warp == kMmaWarp) {
    // ------------------------------- MMA issuer A: S and dP ----------------------------------------
    // S/dP of batch n is issued as soon as its Q/dO stage has landed and its TMEM buffer is free (the soft-max warps
    // hold batch n-2 in registers), i.e. ahead of dV/dK of batch n-1, which the second issuer handles.
    if (lane == 0 && nb > 0) {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 64, 0, 0);   // both operands K-major
      bool ok = mbar_wait(kv_bar, 0, DEV_ERR_FULL_WAIT);
      const uint64_t dK = umma_smem_desc(k_s, 0, 1024), dV = umma_smem_desc(v_s, 0, 1024);
      uint64_t dQk[kStages], dDOk[kStages];
#pragma unroll
      for (int i = 0; i < kStages; ++i) {
        const uint32_t q_s = ring + i * STAGE, do_s = q_s + Q_TILE;
        dQk[i] = umma_smem_desc(q_s, 0, 1024);
        dDOk[i] = umma_smem_desc(do_s, 0, 1024);
      }
      for (int n = 0; ok && n < nb; ++n) {
        ok = mbar_wait(full0 + 8 * (n % kStages), (n / kStages) & 1, DEV_ERR_FULL_WAIT);
        if (ok && n >= 2) ok = mbar_wait(sdp_free + 8 * (n & 1), ((n >> 1) - 1) & 1, DEV_ERR_EMPTY_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint64_t aq = (n % kStages) ? dQk[1] : dQk[0], ado = (n % kStages) ? dDOk[1] : dDOk[0];
        const uint32_t col = (n & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t aoff = (ks >> 2) * Q_PANEL + (ks & 3) * 32, boff = (ks >> 2) * KV_PANEL + (ks & 3) * 32;
          umma_ss(tmem + col, umma_desc_advance(aq, aoff), umma_desc_advance(dK, boff), idesc_kk, ks ? 1u : 0u);
          umma_ss(tmem + col + 64, umma_desc_advance(ado, aoff), umma_desc_advance(dV, boff), idesc_kk, ks ? 1u : 0u);
        }
        umma_commit(sdp_full + 8 * (n & 1));
      }
    }
  } else if (!skip && warp == kMma2Warp) {
    // ------------------------------- MMA issuer B: dV, dK, dQ partials -----------------------------
    if (lane == 0 && nb > 0) {
      constexpr uint32_t idesc_mn = umma_idesc_bf16(128, 64, 1, 1);   // both operands MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, 128, 0, 1);  // A = dS K-major, B = K MN-major
      bool ok = mbar_wait(kv_bar, 0, DEV_ERR_FULL_WAIT);
      uint64_t dQmn[kStages], dDOmn[kStages], dP[2], dDS[2], dDSk[2];
#pragma unroll
      for (int i = 0; i < kStages; ++i) {
        const uint32_t q_s = ring + i * STAGE, do_s = q_s + Q_TILE;
        dQmn[i] = umma_smem_desc(q_s, Q_PANEL, 1024);
        dDOmn[i] = umma_smem_desc(do_s, Q_PANEL, 1024);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        dP[i] = umma_smem_desc(p_s0 + i * 2 * P_TILE, 0, 1024);
        dDS[i] = umma_smem_desc(p_s0 + i * 2 * P_TILE + P_TILE, 0, 1024);
        dDSk[i] = dDS[i];   // the same tile read K-major for the dQ partial
      }
      const uint64_t dKmn = umma_smem_desc(k_s, KV_PANEL, 1024);
      int ndq = 0;          // dQ partials issued so far
      for (int n = 0; ok && n < nb; ++n) {
        ok = mbar_wait(pds_full + 8 * (n & 1), (n >> 1) & 1, DEV_ERR_FULL_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint64_t aq = (n % kStages) ? dQmn[1] : dQmn[0], ado = (n % kStages) ? dDOmn[1] : dDOmn[0];
        const uint64_t bp = (n & 1) ? dP[1] : dP[0], bds = (n & 1) ? dDS[1] : dDS[0];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {  // contraction over the 128 rows, 16 per step; dV and dK alternate
          umma_ss(tmem + kColDV, umma_desc_advance(ado, ks * 2048), umma_desc_advance(bp, ks * 2048), idesc_mn, (n | ks) ? 1u : 0u);
          umma_ss(tmem + kColDK, umma_desc_advance(aq, ks * 2048), umma_desc_advance(bds, ks * 2048), idesc_mn, (n | ks) ? 1u : 0u);
        }
        umma_commit(empty0 + 8 * (n % kStages));
        if (emit_dq && (n % nb_sub) < nbA) {
          // the previous partial must have been read out of its accumulator by the drain warps
          if (ndq > 0) ok = mbar_wait(dq_free, (ndq - 1) & 1, DEV_ERR_EMPTY_WAIT);
          if (!ok) break;
          tc_fence_after();
          const uint64_t ads = (n & 1) ? dDSk[1] : dDSk[0];
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)   // contraction over the 64 keys, 16 per step
            umma_ss(tmem + kColDQ, umma_desc_advance(ads, ks * 32), umma_desc_advance(dKmn, ks * 2048), idesc_dq, ks ? 1u : 0u);
          umma_commit(dq_full);
          ++ndq;
        }
        umma_commit(pds_free + 8 * (n & 1));
      }
      umma_commit(acc_full);
    }
  }
  } else if (warp >= kDrainWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (!skip) {
    // ------------------------------- drain warps: dQ partials, one row per thread ------------------
    // dQ partial of a selected batch: accumulator -> bf16 -> shared memory -> one bulk store.  The staging area is that
    // batch's own P/dS tile pair (32 KB = 128 rows x 256 bytes): dq_full also says that every MMA that read the pair
    // has completed, and the soft-max warps write it again (batch n+2) only after stg_free.  The 8 tokens' [16 x D]
    // tiles sit at consecutive list positions, i.e. contiguous in dq_part when the KV head has one 16-head group.
    // Within a 128-byte half row the 16-byte chunk c is stored at position c ^ (row & 7) (conflict-free writes;
    // row & 7 == head & 7, and the reduction kernel undoes it).  Plain stores from the accumulator's layout (a thread
    // owns a row: 16 bytes per lane at a 256-byte stride) cost a tenth of the kernel in store wavefronts, and reading
    // the partials out in the soft-max warps delayed the next batch's soft-max.
    if (emit_dq) {
      const int quad = warp & 3;
      const int row = 32 * quad + lane;
      const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
      const bool elected = warp == kDrainWarp && lane == 0;
      bool ok = true;
      int k = 0;   // partials drained so far
      for (int n = 0; ok && n < nb; ++n) {
        const int sub = n / nb_sub, mloc = n % nb_sub;
        if (mloc >= nbA) continue;
        ok = mbar_wait(dq_full, k & 1, DEV_ERR_FULL_WAIT);
        if (!ok) break;
        tc_fence_after();
        const uint32_t stg = p_s0 + (uint32_t)(n & 1) * 2 * P_TILE;
        uint8_t* sp = sgen + (stg - sbase) + row * 256;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {   // 32 columns at a time
          float vals[2][16];
          tmem_ld16(tmem + lane_addr + kColDQ + q4 * 32, vals[0]);
          tmem_ld16(tmem + lane_addr + kColDQ + q4 * 32 + 16, vals[1]);
          tmem_ld_wait();
          if (q4 == 3) {
            tc_fence_before();
            mbar_arrive(dq_free);   // the accumulator is in registers: the next partial may be issued
          }
#pragma unroll
          for (int c2 = 0; c2 < 4; ++c2) {   // four 16-byte chunks
            const float* f = &vals[c2 >> 1][(c2 & 1) * 8];
            uint4 o;
            __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) ho[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
            const int cc = q4 * 4 + c2;       // chunk 0..15 of the row: half cc >> 3, position (cc & 7) ^ (row & 7)
            *reinterpret_cast<uint4*>(sp + (cc >> 3) * 128 + (((cc & 7) ^ (row & 7)) * 16)) = o;
          }
        }
        fence_proxy_async();
        mbar_arrive(stg_full);
        if (elected) {
          ok = mbar_wait(stg_full, k & 1, DEV_ERR_FULL_WAIT);
          const int nvalid = min(kTokB, st.nA - mloc * kTokB);
          if (ok && nvalid > 0) {
            const long long bh = (long long)b * a.Hk + hk;
            bf16* dst = a.dq_part + ((bh * a.rev_cap + st.ta_lo + mloc * kTokB) * G16 + sub) * (16 * D);
            if (G16 == 1) {
              bulk_store_evict_first(dst, stg, (uint32_t)nvalid * 16 * D * 2);
            } else {
              for (int i = 0; i < nvalid; ++i)
                bulk_store_evict_first(dst + (long long)i * G16 * 16 * D, stg + i * 16 * D * 2, 16 * D * 2);
            }
          }
          bulk_commit();
          bulk_wait_read();                       // the pair may be written again
          mbar_arrive(stg_free + 8 * (n & 1));
        }
        ++k;
      }
      if (elected) bulk_wait_all();
    }
  }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
  if (!skip) {
    // ------------------------------- soft-max warps: one (token, head) row per thread --------------
    const int quad = warp & 3;
    const int half = (warp - kSoftWarp) >> 2;    // which 32 key columns this thread owns
    const int row = 32 * quad + lane;           // TMEM lane == tile row
    const int j = row >> 4, head = row & 15;
    const uint32_t lane_addr = (uint32_t)(32 * quad) << 16;
    const float sl2 = a.scale * kLog2e;
    bool ok = true;
    // per-row operands are fetched one batch ahead (token ids two ahead) so their latency hides behind the MMAs
    struct RowInfo {
      int t;
      bool live;
      int br;
      float lse2, del, gv;
    };
    auto row_token = [&](int n, int& br, bool& live) {
      br = 0;
      live = false;
      if (n >= nb) return 0;
      const int m = n % nb_sub;
      br = m < nbA ? 0 : 1;
      const int i = (br == 0 ? m : m - nbA) * kTokB + j;
      live = i < (br == 0 ? st.nA : st.nB);
      return stream_token(st, br, i);
    };
    auto row_load = [&](int n, int t, int br, bool live) {
      RowInfo r;
      r.t = t;
      r.live = live;
      r.br = br;
      r.lse2 = 0.f;
      r.del = 0.f;
      r.gv = 1.f;
      if (n < nb) {
        const int sub = n / nb_sub;
        const long long qrow = ((long long)b * a.Tq + (t - a.q0)) * a.Hq + (hk * G16 + sub) * 16 + head;
        r.lse2 = (br == 0 ? a.lse_a : a.lse_b)[qrow] * kLog2e;
        r.del = (br == 0 ? a.delta_a : a.delta_b)[qrow];
        const bf16* gp = br == 0 ? a.gate_a : a.gate_b;
        if (gp) r.gv = __bfloat162float(gp[qrow]);
      }
      return r;
    };
    // With dQ partials: the drain warps stage the partial of a selected batch n in that batch's own P/dS pair; the pair
    // is written again for batch n+2 only after their bulk store has read it (stg_free of that pair).
    int nstg[2] = {0, 0};   // waits done on each pair's stg_free
    int br1, br2;
    bool live1, live2;
    int t1 = row_token(0, br1, live1);
    RowInfo cur = row_load(0, t1, br1, live1);
    t1 = row_token(1, br1, live1);
    for (int n = 0; ok && n < nb; ++n) {
      const RowInfo ri = cur;
      cur = row_load(n + 1, t1, br1, live1);          // operands of batch n+1
      const int t2 = row_token(n + 2, br2, live2);    // token id of batch n+2
      t1 = t2;
      br1 = br2;
      live1 = live2;
      const int t = ri.t, br = ri.br;
      const bool live = ri.live;
      const float lse2 = ri.lse2, del = ri.del, gv = ri.gv;

      const uint32_t buf = n & 1, use = n >> 1;
      const uint32_t tcol = buf * 128;
      ok = mbar_wait(sdp_full + 8 * buf, use & 1, DEV_ERR_FULL_WAIT);
      if (!ok) break;
      tc_fence_after();
      uint32_t pw[16], dw[16];   // 32 bf16 each
      {
        float sv[32], dpv[32];
        tmem_ld16(tmem + lane_addr + tcol + half * 32, *reinterpret_cast<float(*)[16]>(&sv[0]));
        tmem_ld16(tmem + lane_addr + tcol + half * 32 + 16, *reinterpret_cast<float(*)[16]>(&sv[16]));
        tmem_ld16(tmem + lane_addr + tcol + 64 + half * 32, *reinterpret_cast<float(*)[16]>(&dpv[0]));
        tmem_ld16(tmem + lane_addr + tcol + 64 + half * 32 + 16, *reinterpret_cast<float(*)[16]>(&dpv[16]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(sdp_free + 8 * buf);   // S and dP are in registers: batch n+2 may overwrite this TMEM buffer
        const int kfirst = key0 + half * 32, klast = kfirst + 31;
        bool all_valid;
        if (MODE == 0)
          all_valid = (klast <= t) && (br == 0 || kfirst > t - a.window);
        else
          all_valid = klast < a.Lk && (!a.causal || klast * a.cstride + a.cblock <= t);
        if (!live || !(lse2 > -INFINITY)) {
#pragma unroll
          for (int e = 0; e < 16; ++e) pw[e] = dw[e] = 0u;
        } else if (all_valid) {
          const float nl = -lse2;
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = ex2(fmaf(sv[e], sl2, nl)), p1 = ex2(fmaf(sv[e + 1], sl2, nl));
            pw[e / 2] = pack_bf16(p0 * gv, p1 * gv);
            dw[e / 2] = pack_bf16(p0 * fmaf(gv, dpv[e], -del), p1 * fmaf(gv, dpv[e + 1], -del));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float pv[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int kp = kfirst + e + u;
              bool valid;
              if (MODE == 0)
                valid = (kp <= t) && (br == 0 || kp > t - a.window);
              else
                valid = kp < a.Lk && (!a.causal || kp * a.cstride + a.cblock <= t);
              pv[u] = valid ? ex2(sv[e + u] * sl2 - lse2) : 0.f;
            }
            pw[e / 2] = pack_bf16(pv[0] * gv, pv[1] * gv);
            dw[e / 2] = pack_bf16(pv[0] * fmaf(gv, dpv[e], -del), pv[1] * fmaf(gv, dpv[e + 1], -del));
          }
        }
      }
      if (n >= 2) {
        ok = mbar_wait(pds_free + 8 * buf, (use - 1) & 1, DEV_ERR_EMPTY_WAIT);   // dV/dK of batch n-2 have read this pair
        if (!ok) break;
      }
      if (emit_dq && n >= 2 && ((n - 2) % nb_sub) < nbA) {
        ok = mbar_wait(stg_free + 8 * buf, nstg[buf] & 1, DEV_ERR_EMPTY_WAIT);
        ++nstg[buf];
        if (!ok) break;
      }
      // this thread's half of row `row` of the [128 x 64] bf16 tiles: 4 chunks of 16 bytes at swizzled positions
      uint8_t* prow = sgen + (p_s0 - sbase) + buf * 2 * P_TILE + row * 128;
      uint8_t* drow = prow + P_TILE;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int pos = ((4 * half + c) ^ (row & 7)) * 16;
        *reinterpret_cast<uint4*>(prow + pos) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
        *reinterpret_cast<uint4*>(drow + pos) = make_uint4(dw[4 * c], dw[4 * c + 1], dw[4 * c + 2], dw[4 * c + 3]);
      }
      fence_proxy_async();
      mbar_arrive(pds_full + 8 * buf);
    }
    // ---- epilogue: dV^T / dK^T [d lanes x 64 key columns] -> global ---------------------------------------
    if (ok && nb > 0) ok = mbar_wait(acc_full, 0, DEV_ERR_FULL_WAIT);
    tc_fence_after();
    const int dch = row;  // channel owned by this thread
    {
      const int which = half;   // warps 2-5 store dV, warps 6-9 store dK
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float vals[16];
        if (nb > 0) {
          tmem_ld16(tmem + lane_addr + kColDV + which * 64 + c * 16, vals);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) vals[e] = 0.f;
        }
        const float mul = which ? a.scale : 1.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int kp = key0 + c * 16 + e;
          if (!ok || kp >= a.Lk) continue;
          const long long off = (((long long)b * a.Lk + kp) * a.Hk + hk) * D + dch;
          if (MODE == 0) {
            (which ? a.dk : a.dv)[off] = __float2bfloat16(vals[e] * mul);
          } else {
            const long long N = (long long)a.B * a.Lk * a.Hk * D;
            a.part[((long long)(which ? 0 : a.nseg) + seg) * N + off] = vals[e] * mul;
          }
        }
      }
    }
  }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemCols);
}

template <int MODE>
int launch(const KvArgs& a, cudaStream_t s) {
  CUtensorMap tmQ, tmA, tmB, tmK, tmV, tmQw, tmDOw;
  const long long qrows = (long long)a.B * a.Tq * a.Hq;
  if (qrows > 0x7fffffffLL) {
    set_error("B*T*Hq exceeds the 2^31 rows a TMA coordinate can address");
    return -32;
  }
  int rc = make_tmap_rows2d(&tmQ, a.q, D, qrows, 16);
  if (!rc) rc = make_tmap_rows2d(&tmA, a.dout_a ? a.dout_a : a.dout_b, D, qrows, 16);
  if (!rc) rc = make_tmap_rows2d(&tmB, a.dout_b ? a.dout_b : a.dout_a, D, qrows, 16);
  if (!rc) rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.Lk, a.B, 64);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.Lk, a.B, 64);
  {   // consecutive-token batches: [64 columns x 16 heads x 8 tokens] boxes of q and of that stream's dO
    const unsigned long long dims[4] = {(unsigned long long)D, (unsigned long long)a.Hq, (unsigned long long)a.Tq,
                                        (unsigned long long)a.B};
    const unsigned long long strides[3] = {(unsigned long long)D * 2, (unsigned long long)a.Hq * D * 2,
                                           (unsigned long long)a.Tq * a.Hq * D * 2};
    const unsigned box[4] = {64, 16, (unsigned)kTokB, 1};
    const void* dow = MODE == 0 ? (a.dout_b ? a.dout_b : a.dout_a) : a.dout_a;
    if (!rc) rc = make_tmap_generic(&tmQw, a.q, 4, dims, strides, box);
    if (!rc) rc = make_tmap_generic(&tmDOw, dow, 4, dims, strides, box);
  }
  if (rc) return rc;
  auto kern = kv_bwd_tc_kernel<MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
  if (e != cudaSuccess) return (int)e;
  long long grid;
  if (MODE == 0)
    grid = (long long)a.B * a.Hk * ((a.T + 63) / 64);
  else
    grid = (long long)a.B * a.Hk * ((a.Lk + 63) / 64) * a.nseg;
  if (grid <= 0) return 0;
  if (grid > 0x7fffffffLL) {
    set_error("kv backward: grid too large");
    return -33;
  }
  kern<<<(unsigned)grid, kThreads, kSmem, s>>>(tmQ, tmA, tmB, tmK, tmV, tmQw, tmDOw, a);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

// head_dim 128 and 64-key blocks only; the caller falls back to launch_kv_bwd otherwise.
int launch_kv_bwd_tc(const KvArgs& a, cudaStream_t s) { return a.mode == 0 ? launch<0>(a, s) : launch<1>(a, s); }
int kv_tc_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
