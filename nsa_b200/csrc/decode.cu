// Batched decode step: the whole NSA forward (nsa/nsa.py:94-135) for ONE new query token per sequence, every sequence
// of a packed, ragged K/V cache in a single launch.  The reference has no decode entry point (its module assumes
// len(q) == len(k), nsa/nsa.py:97); the arithmetic is that of its forward evaluated for the row t = L-1:
// compressed attention over the compressed cache with the mask t >= 16 j + 32 (nsa/triton_attention.py:87-181), the
// block scores softmax(q.ck) summed over the 16 heads of the group, 5/4 average-pooled and top-n'd
// (nsa/torch_attention.py:51-62,121-125), attention over the selected 64-key blocks and over the last `window` keys
// (nsa/selection_attn.py:401-517), and the gated sum (nsa/nsa.py:133).
//
// The step is HBM-bound: a sequence contributes its compressed cache (1/16 of its K/V), 16 selected blocks and the
// window, each read once.  One CTA works on one (sequence, kv head): the 16 query heads of the group are the M = 16
// rows of mma.sync.m16n8k16.  Two producer warps stream [64 rows x 128] tiles by TMA through a twelve-slot ring (192 KB
// in flight per SM); six consumer warps own two slots each, so every slot is filled and drained by the same pair of
// warps in order.  The tile stream of an item:
//   1. ck tiles:           raw scores -> per-row maxima and sums of the unscaled soft-max over ALL compressed keys and
//                          of the scaled, masked attention soft-max (merged over the warps in shared memory);
//   2. (ck, cv) pairs:     scores again (ck comes from L2 this time) -> attention P.cv with the final statistics, and
//                          p_sel summed over the heads into a per-position vector in shared memory;
//                          then pooling and a warp top-n while the other warps go on;
//   3. window (k, v) pairs and 4. selected (k, v) pairs: online soft-max per warp.
// Every warp leaves its partial (maximum, sum, unnormalised output) of each branch in a caller-provided workspace; a
// second, small kernel merges the six partials of a branch in a fixed order, computes the gates from q and writes the
// outputs (the split-KV scheme of decode attention).  Measured alternatives: merging through shared memory, warp after
// warp, cost seven named barriers and six serialised rounds per branch (0.29 ms per step of the 128-sequence workload
// against 0.21 ms); merging in the same kernel through an L2-resident scratch idled five of six warps and the TMA ring
// during the merge (0.30 ms).  No atomics; every wait is bounded.
#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int D = 128;
constexpr int kCons = 6;                       // consumer warps
constexpr int kProdW = 2;                      // producer warps
constexpr int kThreads = (kCons + kProdW) * 32;
constexpr int kSlots = 2 * kCons;
constexpr uint32_t PANEL = 64 * 128;           // [64 rows][64 columns] bf16
constexpr uint32_t TILE = 2 * PANEL;           // 16 KB
constexpr int kMaxTc = 2048;                   // compressed positions of one sequence held in shared memory
constexpr int kMaxPoolD = 512;
constexpr int kMaxSel = 32;
constexpr int kPartFloats = 16 * D + 32;        // one warp's partial of one branch: O[16][D], m[16], l[16]

struct Plan {   // tile counts of one item; every phase is an even number of tiles
  int L, Tc, nvis, row_k, row_c;
  int n1;      // ck tiles of pass 1 (rounded up to even)
  int n2p;     // (ck, cv) pairs of pass 2: covers all of Tc
  int nw;      // window pairs
  int w0;      // first window key
};

__device__ __forceinline__ Plan make_plan(const DecodeArgs& a, int seq) {
  Plan p;
  p.row_k = a.cu_k[seq];
  p.row_c = a.cu_c[seq];
  p.L = a.cu_k[seq + 1] - p.row_k;
  p.Tc = a.cu_c[seq + 1] - p.row_c;
  if (p.Tc > kMaxTc) p.Tc = kMaxTc;            // rejected on the host; keeps the indexing inside shared memory
  const int t = p.L - 1;
  p.nvis = (t < a.cblock) ? 0 : min(p.Tc, (t - a.cblock) / a.cstride + 1);
  const int nck = (p.Tc + 63) / 64;
  p.n1 = (nck + 1) & ~1;
  p.n2p = nck;
  p.w0 = max(0, p.L - a.window);
  p.nw = a.window > 0 ? (p.L - p.w0 + 63) / 64 : 0;
  return p;
}

// Items are dealt to the CTAs in boustrophedon order (left to right in even rounds, right to left in odd ones): with
// the sequences sorted longest first, every CTA then gets a long and a short item in turn (maximum / mean load 1.09
// for lengths uniform in [4096, 32768], against 1.23 for a plain round robin).
__device__ __forceinline__ int snake_item(int round, int cta, int ncta) {
  return round * ncta + ((round & 1) ? ncta - 1 - cta : cta);
}

// avg_pool1d(kernel k, stride s, no padding, ceil_mode) output length, as nsa_pool_out_len computes it
__device__ __forceinline__ int pool_len(int n, int k, int s) {
  if (n <= 0) return 0;
  const int num = n - k;
  int out = (num >= 0 ? (num + s - 1) / s : -((-num) / s)) + 1;
  if ((out - 1) * s >= n) --out;
  return out < 0 ? 0 : out;
}

// acc (16 x 128) += P (16 x 64, in sc as mma C layout) . V tile
__device__ __forceinline__ void pv_tile(float (&acc)[D / 8][4], const float (&sc)[8][4], uint32_t vbase, int lane) {
  uint32_t pf[4][4];
  acc_to_a_frags<8>(pf, sc);
  mma_a_b<D, 64>(acc, pf, vbase, PANEL, 0, lane);
}

// One (K, V) pair of an online soft-max: keys key0 .. key0+63 of the tile are valid iff kmin <= key < kmax.
__device__ __forceinline__ void online_pair(float (&acc)[D / 8][4], float (&m_run)[2], float (&l_run)[2],
                                            const uint32_t (&qf)[D / 16][4], uint32_t kbase, uint32_t vbase, uint32_t k_empty,
                                            uint32_t v_full, uint32_t v_par, uint32_t v_empty, int key0, int kmin, int kmax,
                                            float sl2, int lane, bool& ok, volatile int* abort_flag) {
  const int tq = lane & 3;
  float sc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
  if (ok) mma_a_bt<D, 64>(sc, qf, kbase, PANEL, 0, lane);
  __syncwarp();
  if (lane == 0) mbar_arrive(k_empty);
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int key = key0 + nt * 8 + 2 * tq + (c & 1);
      if (key < kmin || key >= kmax) sc[nt][c] = -INFINITY;
      mx[c >> 1] = fmaxf(mx[c >> 1], sc[nt][c]);
    }
  float alpha[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const float mnew = fmaxf(m_run[rr], quad_max(mx[rr]) * sl2);
    const float muse = (mnew == -INFINITY) ? 0.f : mnew;
    alpha[rr] = ex2(m_run[rr] - muse);
    m_run[rr] = mnew;
    float rs = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float e0 = ex2(fmaf(sc[nt][2 * rr], sl2, -muse)), e1 = ex2(fmaf(sc[nt][2 * rr + 1], sl2, -muse));
      sc[nt][2 * rr] = e0;
      sc[nt][2 * rr + 1] = e1;
      rs += e0 + e1;
    }
    l_run[rr] = l_run[rr] * alpha[rr] + rs;
  }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    acc[i][0] *= alpha[0];
    acc[i][1] *= alpha[0];
    acc[i][2] *= alpha[1];
    acc[i][3] *= alpha[1];
  }
  ok = ok && mbar_wait_abortable(v_full, v_par, DEV_ERR_FULL_WAIT, abort_flag);
  if (ok) pv_tile(acc, sc, vbase, lane);
  __syncwarp();
  if (lane == 0) mbar_arrive(v_empty);
}

__global__ void __launch_bounds__(kThreads, 1)
    decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const __grid_constant__ CUtensorMap tmCK, const __grid_constant__ CUtensorMap tmCV, const DecodeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = sbase;
  uint8_t* after = sgen + kSlots * TILE;
  float* ps = reinterpret_cast<float*>(after);                    // [kMaxTc + 64] head-summed p_sel per compressed position
  float* pooled = ps + kMaxTc + 64;                               // [kMaxPoolD]
  float* stat = pooled + kMaxPoolD;                               // [kCons][4][16] per-warp statistics
  float* fin = stat + kCons * 64;                                 // [4][16] merged: M_raw, 1/L_raw, M_att (log2), L_att
  int* sel = reinterpret_cast<int*>(fin + 64);                    // [kMaxSel] selected blocks of the item, [kMaxSel] = count
  volatile int* abort_flag = sel + kMaxSel + 2;
  const uint32_t bar_base = sbase + kSlots * TILE + (uint32_t)((uint8_t*)(sel + kMaxSel + 4) - after);
  const uint32_t bar0 = (bar_base + 7u) & ~7u;
  auto full_bar = [&](uint32_t s) { return bar0 + 8u * s; };
  auto empty_bar = [&](uint32_t s) { return bar0 + 8u * (kSlots + s); };
  const uint32_t sel_ready = bar0 + 8u * (2 * kSlots);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), 1);
    }
    mbar_init(sel_ready, 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int nitem = a.nseq * a.Hkv;
  const int pool_k = a.sel_block / a.cstride + 1, pool_s = a.sel_block / a.cstride;

  if (warp >= kCons) {
    // ------------------------------- producers --------------------------------------------------------
    // A warp's TMA instructions run one after another (about 850 + 52 x boxes cycles each, whatever the box size), so
    // a single warp issuing one 16 KB tile per instruction caps the SM at ~16 bytes per clock.  Tiles therefore go out
    // in PAIRS (four boxes per instruction: both tiles of a (K, V) pair, or two consecutive ck tiles of pass 1), and
    // the two producer warps take alternate pairs.
    const int pw = warp - kCons;
    uint32_t np = 0, it = 0;     // tile pairs issued so far by both producers together; items so far
    auto issue2 = [&](const CUtensorMap* tmA, int rowA, const CUtensorMap* tmB, int rowB, int h) -> bool {
      const uint32_t mine = (np & 1) == (uint32_t)pw;
      const uint32_t n = 2 * np;
      ++np;
      if (!mine) return true;
      const uint32_t s0 = n % kSlots, ph = (n / kSlots) & 1;     // the pair's slots s0, s0+1 belong to one consumer warp
      int good = 1;
      if (lane == 0) {
        good = mbar_wait_abortable(empty_bar(s0), ph ^ 1, DEV_ERR_EMPTY_WAIT, abort_flag) &&
               mbar_wait_abortable(empty_bar(s0 + 1), ph ^ 1, DEV_ERR_EMPTY_WAIT, abort_flag) ? 1 : 0;
        if (good) {
          mbar_expect_tx(full_bar(s0), TILE);
          mbar_expect_tx(full_bar(s0 + 1), TILE);
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (good && lane < 4) {
        const int which = lane >> 1, panel = lane & 1;
        tma_load_4d(ring + (s0 + which) * TILE + panel * PANEL, which ? tmB : tmA, full_bar(s0 + which), panel * 64, h,
                    which ? rowB : rowA, 0);
      }
      return good != 0;
    };
    for (int r = 0; r * (int)gridDim.x < nitem; ++r) {
      const int item = snake_item(r, blockIdx.x, gridDim.x);
      if (item >= nitem) continue;
      const int sq = item / a.Hkv, h = item % a.Hkv;
      const int seq = a.order ? a.order[sq] : sq;
      const Plan p = make_plan(a, seq);
      bool ok = true;
      for (int j = 0; ok && j < p.n1; j += 2) ok = issue2(&tmCK, p.row_c + j * 64, &tmCK, p.row_c + (j + 1) * 64, h);
      for (int j = 0; ok && j < p.n2p; ++j) ok = issue2(&tmCK, p.row_c + j * 64, &tmCV, p.row_c + j * 64, h);
      for (int j = 0; ok && j < p.nw; ++j) ok = issue2(&tmK, p.row_k + p.w0 + j * 64, &tmV, p.row_k + p.w0 + j * 64, h);
      // the selected blocks are known once the consumers have pooled the scores
      if (ok && lane == 0) ok = mbar_wait_abortable(sel_ready, it & 1, DEV_ERR_FULL_WAIT, abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const int nsel = *reinterpret_cast<volatile int*>(sel + kMaxSel);
      for (int j = 0; ok && j < nsel; ++j) {
        const int blk = *reinterpret_cast<volatile int*>(sel + j);
        ok = issue2(&tmK, p.row_k + blk * 64, &tmV, p.row_k + blk * 64, h);
      }
      if (!ok) break;
      ++it;
    }
    return;
  }

  // --------------------------------- consumers ----------------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const float sl2 = a.scale * kLog2e;
  const int cthreads = kCons * 32;
  const int ct = threadIdx.x;               // 0 .. cthreads-1
  uint32_t n0 = 0, it = 0;                  // tiles consumed by the CTA before the current phase; items so far
  bool ok = true;
  // tile pair u (two consecutive tiles) of a phase that starts at tile counter base belongs to warp ((base/2 + u) % kCons)
  for (int r = 0; r * (int)gridDim.x < nitem; ++r) {
    const int item = snake_item(r, blockIdx.x, gridDim.x);
    if (item >= nitem) continue;
    const int sq = item / a.Hkv, h = item % a.Hkv;
    const int seq = a.order ? a.order[sq] : sq;
    const Plan p = make_plan(a, seq);
    const int t = p.L - 1;
    const long long qrow = (long long)seq * a.Hq + h * 16;     // first of the 16 (head) rows of this item
    uint32_t qf[D / 16][4];
    load_a_frags_global<D>(qf, a.q + qrow * D, lane);
    for (int i = ct; i < kMaxTc + 64; i += cthreads) ps[i] = 0.f;

    // ---- pass 1: statistics over all compressed keys ---------------------------------------------------
    float mr[2] = {-INFINITY, -INFINITY}, lr[2] = {0.f, 0.f};   // raw scores, all keys (natural-log domain kept in log2)
    float ma[2] = {-INFINITY, -INFINITY}, la[2] = {0.f, 0.f};   // scaled scores, visible keys
    {
      const uint32_t pair0 = n0 / 2;
      for (int u = 0; u < p.n1 / 2; ++u) {
        if ((int)((pair0 + u) % kCons) != warp) continue;
#pragma unroll 1
        for (int e = 0; e < 2; ++e) {
          const uint32_t n = n0 + 2 * u + e, s = n % kSlots;
          const int j0 = (2 * u + e) * 64;
          ok = ok && mbar_wait_abortable(full_bar(s), (n / kSlots) & 1, DEV_ERR_FULL_WAIT, abort_flag);
          float sc[8][4];
#pragma unroll
          for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
          if (ok) mma_a_bt<D, 64>(sc, qf, ring + s * TILE, PANEL, 0, lane);
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(s));
          float mxr[2] = {-INFINITY, -INFINITY}, mxa[2] = {-INFINITY, -INFINITY};
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int j = j0 + nt * 8 + 2 * tq + (c & 1);
              if (j < p.Tc) mxr[c >> 1] = fmaxf(mxr[c >> 1], sc[nt][c]);
              if (j < p.nvis) mxa[c >> 1] = fmaxf(mxa[c >> 1], sc[nt][c]);
            }
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const float nr = fmaxf(mr[rr], quad_max(mxr[rr]) * kLog2e), na = fmaxf(ma[rr], quad_max(mxa[rr]) * sl2);
            const float ur = (nr == -INFINITY) ? 0.f : nr, ua = (na == -INFINITY) ? 0.f : na;
            float sr = 0.f, sa = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
              for (int c2 = 0; c2 < 2; ++c2) {
                const int j = j0 + nt * 8 + 2 * tq + c2;
                const float x = sc[nt][2 * rr + c2];
                if (j < p.Tc) sr += ex2(fmaf(x, kLog2e, -ur));
                if (j < p.nvis) sa += ex2(fmaf(x, sl2, -ua));
              }
            lr[rr] = lr[rr] * ex2(mr[rr] - ur) + sr;
            la[rr] = la[rr] * ex2(ma[rr] - ua) + sa;
            mr[rr] = nr;
            ma[rr] = na;
          }
        }
      }
      n0 += p.n1;
    }
    // merge the per-warp statistics (each value lives in the four lanes of a quad: sum the partial sums)
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const float l_r = quad_sum(lr[rr]), l_a = quad_sum(la[rr]);
      if (tq == 0) {
        float* st = stat + warp * 64;
        st[0 * 16 + g + 8 * rr] = mr[rr];
        st[1 * 16 + g + 8 * rr] = l_r;
        st[2 * 16 + g + 8 * rr] = ma[rr];
        st[3 * 16 + g + 8 * rr] = l_a;
      }
    }
    named_bar_sync(1, cthreads);
    if (ct < 16) {
      float Mr = -INFINITY, Ma = -INFINITY;
      for (int w = 0; w < kCons; ++w) {
        Mr = fmaxf(Mr, stat[w * 64 + ct]);
        Ma = fmaxf(Ma, stat[w * 64 + 32 + ct]);
      }
      float Lr = 0.f, La = 0.f;
      for (int w = 0; w < kCons; ++w) {
        const float m1 = stat[w * 64 + ct], m2 = stat[w * 64 + 32 + ct];
        if (m1 > -INFINITY) Lr += stat[w * 64 + 16 + ct] * ex2(m1 - Mr);
        if (m2 > -INFINITY) La += stat[w * 64 + 48 + ct] * ex2(m2 - Ma);
      }
      fin[ct] = Mr;
      fin[16 + ct] = Lr > 0.f ? 1.f / Lr : 0.f;
      fin[32 + ct] = Ma;
      fin[48 + ct] = La;
    }
    named_bar_sync(1, cthreads);
    float Mr[2], iLr[2], Ma[2], La[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      Mr[rr] = fin[g + 8 * rr];
      iLr[rr] = fin[16 + g + 8 * rr];
      Ma[rr] = fin[32 + g + 8 * rr];
      La[rr] = fin[48 + g + 8 * rr];
      if (Mr[rr] == -INFINITY) Mr[rr] = 0.f;
      if (Ma[rr] == -INFINITY) Ma[rr] = 0.f;
    }

    // ---- pass 2: attention over the visible compressed keys and the block scores -------------------------
    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    {
      const uint32_t pair0 = n0 / 2;
      for (int u = 0; u < p.n2p; ++u) {
        if ((int)((pair0 + u) % kCons) != warp) continue;
        const uint32_t nk = n0 + 2 * u, nv = nk + 1, sk = nk % kSlots, sv = nv % kSlots;
        const int j0 = u * 64;
        ok = ok && mbar_wait_abortable(full_bar(sk), (nk / kSlots) & 1, DEV_ERR_FULL_WAIT, abort_flag);
        float sc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
        if (ok) mma_a_bt<D, 64>(sc, qf, ring + sk * TILE, PANEL, 0, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(sk));
        // p_sel summed over the 16 heads: rows live in the eight quads of the warp
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          float c0 = 0.f, c1 = 0.f;   // columns nt*8 + 2 tq and + 1, rows g and g+8 of this thread
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            c0 += ex2(fmaf(sc[nt][2 * rr], kLog2e, -Mr[rr])) * iLr[rr];
            c1 += ex2(fmaf(sc[nt][2 * rr + 1], kLog2e, -Mr[rr])) * iLr[rr];
          }
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) {
            c0 += __shfl_xor_sync(0xffffffffu, c0, off);
            c1 += __shfl_xor_sync(0xffffffffu, c1, off);
          }
          if (g == 0) {
            const int j = j0 + nt * 8 + 2 * tq;
            if (j < p.Tc) ps[j] = c0;
            if (j + 1 < p.Tc) ps[j + 1] = c1;
          }
        }
        // attention weights with the final maximum (unnormalised; the sum divides at the end)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int j = j0 + nt * 8 + 2 * tq + (c & 1);
            sc[nt][c] = (j < p.nvis) ? ex2(fmaf(sc[nt][c], sl2, -Ma[c >> 1])) : 0.f;
          }
        ok = ok && mbar_wait_abortable(full_bar(sv), (nv / kSlots) & 1, DEV_ERR_FULL_WAIT, abort_flag);
        if (ok && j0 < p.nvis) pv_tile(acc, sc, ring + sv * TILE, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(sv));
      }
      n0 += 2 * p.n2p;
    }
    // ---- pooled scores and the top-n (warp 0), the compressed-branch output (all warps, fixed order) ------------
    named_bar_sync(1, cthreads);            // ps complete
    const int n_pool = min(kMaxPoolD, pool_len(p.Tc, pool_k, pool_s));
    for (int blk = ct; blk < n_pool; blk += cthreads) {
      const int lo = blk * pool_s, hi = min(lo + pool_k, p.Tc);
      float sum = 0.f;
      for (int j = lo; j < hi; ++j) sum += ps[j];
      pooled[blk] = sum / (float)(hi - lo);
    }
    named_bar_sync(1, cthreads);
    if (warp == 0) {
      int cnt = 0;
      int* out = a.idx + ((long long)seq * a.Hkv + h) * a.n_sel;
      for (int r = 0; r < a.n_sel; ++r) {
        float bv = -2.f;
        int bi = 0x7fffffff;
        for (int blk = lane; blk < n_pool; blk += 32) {
          const float v = pooled[blk];
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
          if (found) {
            pooled[bi] = -2.f;
            if ((long long)bi * 64 <= t && cnt < kMaxSel) sel[cnt++] = bi;   // blocks that start after t are skipped
          }
        }
        __syncwarp();
      }
      if (lane == 0) {
        sel[kMaxSel] = cnt;
        __threadfence_block();
        mbar_arrive(sel_ready);
      }
    }
    // this warp's partial of a branch -> workspace: [item][branch][warp]{ O[16][D], m[16], l[16] } fp32
    auto put_partial = [&](int branch, const float (&x)[D / 8][4], const float (&mm)[2], const float (&ll)[2]) {
      float* dst = a.part + (((long long)item * 3 + branch) * kCons + warp) * kPartFloats;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<float2*>(dst + g * D + i * 8 + 2 * tq) = make_float2(x[i][0], x[i][1]);
        *reinterpret_cast<float2*>(dst + (g + 8) * D + i * 8 + 2 * tq) = make_float2(x[i][2], x[i][3]);
      }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const float l = quad_sum(ll[rr]);
        if (tq == 0) {
          dst[16 * D + g + 8 * rr] = mm[rr];
          dst[16 * D + 16 + g + 8 * rr] = l;
        }
      }
    };
    {
      // compressed branch: every warp used the final maximum; the row sum is known to the CTA and rides with warp 0
      float mm[2], ll[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        mm[rr] = fin[32 + g + 8 * rr];
        ll[rr] = (warp == 0 && tq == 0) ? La[rr] : 0.f;
      }
      put_partial(0, acc, mm, ll);
    }

    // ---- window ---------------------------------------------------------------------------------------
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    {
      const uint32_t pair0 = n0 / 2;
      for (int u = 0; u < p.nw; ++u) {
        if ((int)((pair0 + u) % kCons) != warp) continue;
        const uint32_t nk = n0 + 2 * u, nv = nk + 1, sk = nk % kSlots, sv = nv % kSlots;
        ok = ok && mbar_wait_abortable(full_bar(sk), (nk / kSlots) & 1, DEV_ERR_FULL_WAIT, abort_flag);
        online_pair(acc, m_run, l_run, qf, ring + sk * TILE, ring + sv * TILE, empty_bar(sk), full_bar(sv), (nv / kSlots) & 1,
                    empty_bar(sv), p.w0 + u * 64, p.w0, p.L, sl2, lane, ok, abort_flag);
      }
      n0 += 2 * p.nw;
    }
    {
      // l_run holds this lane's share of the row sums (four lanes per row): put_partial adds the quad
      put_partial(2, acc, m_run, l_run);
    }

    // ---- selected blocks ---------------------------------------------------------------------------------
    ok = ok && mbar_wait_abortable(sel_ready, it & 1, DEV_ERR_FULL_WAIT, abort_flag);
    const int nsel = *reinterpret_cast<volatile int*>(sel + kMaxSel);
    m_run[0] = m_run[1] = -INFINITY;
    l_run[0] = l_run[1] = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    {
      const uint32_t pair0 = n0 / 2;
      for (int u = 0; u < nsel; ++u) {
        if ((int)((pair0 + u) % kCons) != warp) continue;
        const int blk = *reinterpret_cast<volatile int*>(sel + u);
        const uint32_t nk = n0 + 2 * u, nv = nk + 1, sk = nk % kSlots, sv = nv % kSlots;
        ok = ok && mbar_wait_abortable(full_bar(sk), (nk / kSlots) & 1, DEV_ERR_FULL_WAIT, abort_flag);
        online_pair(acc, m_run, l_run, qf, ring + sk * TILE, ring + sv * TILE, empty_bar(sk), full_bar(sv), (nv / kSlots) & 1,
                    empty_bar(sv), blk * 64, 0, p.L, sl2, lane, ok, abort_flag);
      }
      n0 += 2 * nsel;
    }
    put_partial(1, acc, m_run, l_run);
    named_bar_sync(1, cthreads);   // ps, pooled, fin and sel are reused by the next item
    ++it;
  }
}

// Merge of the per-warp partials: one CTA of D threads per (sequence, kv head); thread d owns channel d of the 16 rows.
// Branch order in the workspace: 0 compressed, 1 selected, 2 window.  Fixed summation order (warp 0, 1, ...).  The gates
// are computed here from q when the gate projection is given.
// 4 x D threads per item: four groups of four query rows, one thread per output channel; the sums over the six
// consumer warps are short, so the kernel is pure latency and the rows are spread over as many threads as the GPU holds.
constexpr int kMergeGroups = 4;
__global__ void __launch_bounds__(kMergeGroups * D) decode_merge_kernel(const DecodeArgs a) {
  const int item = blockIdx.x;
  const int sq = item / a.Hkv, h = item % a.Hkv;
  const int seq = a.order ? a.order[sq] : sq;
  const long long qrow = (long long)seq * a.Hq + h * 16;
  const int d = threadIdx.x & (D - 1);
  const int rg = threadIdx.x / D;            // rows 4 rg .. 4 rg + 3
  const int tid = threadIdx.x;
  const float* part = a.part + (long long)item * 3 * kCons * kPartFloats;
  __shared__ float w_s[3][kCons][16];   // per (branch, warp, row): 2^(m_w - M) / L
  __shared__ float lse_s[3][16];
  __shared__ float gp_s[D / 32][48];    // gate projection: per-warp partial dot products of (row, gate)
  __shared__ float gate_s[3][16];       // gates of the item's 16 rows; order: compressed, selected, window
  if (a.gate_w) {
    // g_x[row] = q[row,:] . W[x,:] + b[x] (nn.Linear(head_dim, 3), rows of W: selected, window, compressed), rounded to
    // bf16 as the module's gate tensors are
    const float w0 = __bfloat162float(a.gate_w[d]), w1 = __bfloat162float(a.gate_w[D + d]), w2 = __bfloat162float(a.gate_w[2 * D + d]);
    float qa[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) qa[i] = __bfloat162float(a.q[(qrow + rg * 4 + i) * D + d]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = rg * 4 + i;
      float p0 = qa[i] * w0, p1 = qa[i] * w1, p2 = qa[i] * w2;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        p0 += __shfl_xor_sync(0xffffffffu, p0, off);
        p1 += __shfl_xor_sync(0xffffffffu, p1, off);
        p2 += __shfl_xor_sync(0xffffffffu, p2, off);
      }
      if ((d & 31) == 0) {
        gp_s[d >> 5][r * 3 + 0] = p0;
        gp_s[d >> 5][r * 3 + 1] = p1;
        gp_s[d >> 5][r * 3 + 2] = p2;
      }
    }
  }
  // Launched with programmatic stream serialization: everything above (the gate projection reads only q and the
  // weights) may run while the main kernel is still finishing; its partials are read only behind this wait.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (tid < 48) {
    const int br = tid / 16, r = tid % 16;
    const float* base = part + (long long)br * kCons * kPartFloats;
    float mw[kCons], lw[kCons];
#pragma unroll
    for (int w = 0; w < kCons; ++w) {
      mw[w] = base[w * kPartFloats + 16 * D + r];
      lw[w] = base[w * kPartFloats + 16 * D + 16 + r];
    }
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kCons; ++w) M = fmaxf(M, mw[w]);
    float Ltot = 0.f;
#pragma unroll
    for (int w = 0; w < kCons; ++w)
      if (mw[w] > -INFINITY) Ltot += lw[w] * ex2(mw[w] - M);
#pragma unroll
    for (int w = 0; w < kCons; ++w) w_s[br][w][r] = (mw[w] > -INFINITY && Ltot > 0.f) ? ex2(mw[w] - M) / Ltot : 0.f;
    lse_s[br][r] = Ltot > 0.f ? (M + log2f(Ltot)) * kLn2 : -INFINITY;
  }
  __syncthreads();
  if (tid < 48) {
    const int br = tid / 16, r = tid % 16;
    const bf16* gin[3] = {a.g_cmp, a.g_slc, a.g_swa};
    float gv = 1.f;
    if (a.gate_w) {
      const int x = br == 0 ? 2 : br - 1;     // branch (cmp, slc, swa) -> row of the gate weight (slc, swa, cmp)
      float sum = 0.f;
      for (int w = 0; w < D / 32; ++w) sum += gp_s[w][r * 3 + x];
      if (a.gate_b) sum += __bfloat162float(a.gate_b[x]);
      gv = __bfloat162float(__float2bfloat16(sum));
    } else if (gin[br]) {
      gv = __bfloat162float(gin[br][qrow + r]);
    }
    gate_s[br][r] = gv;
  }
  __syncthreads();
  bf16* outs[3] = {a.o_cmp, a.o_slc, a.o_swa};
#pragma unroll
  for (int i = 0; i < 4; ++i) {   // this group's four rows: 72 independent loads in flight per thread
    const int r = rg * 4 + i;
    float tot = 0.f;
#pragma unroll
    for (int br = 0; br < 3; ++br) {
      if (br == 2 && a.window <= 0) continue;
      const float* base = part + (long long)br * kCons * kPartFloats + r * D + d;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kCons; ++w) v += base[w * kPartFloats] * w_s[br][w][r];
      const bf16 vb = __float2bfloat16(v);
      if (outs[br]) outs[br][(qrow + r) * D + d] = vb;
      tot += gate_s[br][r] * __bfloat162float(vb);
    }
    a.o[(qrow + r) * D + d] = __float2bfloat16(tot);
  }
  if (a.lse && tid < 48) {
    const int br = tid / 16, r = tid % 16;
    if (!(br == 2 && a.window <= 0)) a.lse[(long long)br * a.nseq * a.Hq + qrow + r] = lse_s[br][r];
  }
}

}  // namespace

size_t decode_workspace_bytes(int nseq, int Hkv) {
  return (size_t)nseq * Hkv * 3 * kCons * kPartFloats * sizeof(float);
}

int launch_decode(const DecodeArgs& a, cudaStream_t s) {
  if (a.D != D) {
    set_error("decode: head_dim %d not supported (128)", a.D);
    return -2;
  }
  if (a.Hq != 16 * a.Hkv) {
    set_error("decode: needs exactly 16 query heads per KV head (got %d / %d)", a.Hq, a.Hkv);
    return -7;
  }
  if (a.sel_block != 64 || a.cstride != 16 || a.cblock != 32 || a.n_sel < 1 || a.n_sel > kMaxSel || a.window < 0) {
    set_error("decode: needs 64-key selection blocks, compression 32/16 and 1..%d selected blocks", kMaxSel);
    return -9;
  }
  if (a.max_Tc > kMaxTc) {
    set_error("decode: a sequence has %d compressed positions, the kernel holds %d (cache length <= %d)", a.max_Tc, kMaxTc,
              (kMaxTc - 1) * a.cstride + a.cblock + a.cstride - 1);
    return -14;
  }
  CUtensorMap tmK, tmV, tmCK, tmCV;
  int rc = make_tmap_rows4d(&tmK, a.k, D, a.Hkv, a.total_k, 1, 64);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hkv, a.total_k, 1, 64);
  if (!rc) rc = make_tmap_rows4d(&tmCK, a.ck, D, a.Hkv, a.total_c, 1, 64);
  if (!rc) rc = make_tmap_rows4d(&tmCV, a.cv, D, a.Hkv, a.total_c, 1, 64);
  if (rc) return rc;
  const int nitem0 = a.nseq * a.Hkv;
  if (!a.part || a.part_bytes < decode_workspace_bytes(a.nseq, a.Hkv)) {
    set_error("decode: workspace too small (%lld bytes needed)", (long long)decode_workspace_bytes(a.nseq, a.Hkv));
    return -6;
  }
  (void)nitem0;
  const int smem = kSlots * (int)TILE + (kMaxTc + 64 + kMaxPoolD + kCons * 64 + 64) * 4 + (kMaxSel + 4) * 4 +
                   (2 * kSlots + 1) * 8 + 16 + 1024;
  cudaError_t e = cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const int nitem = a.nseq * a.Hkv;
  const int grid = nitem < num_sms() ? nitem : num_sms();
  if (grid <= 0) return 0;
  decode_kernel<<<grid, kThreads, smem, s>>>(tmK, tmV, tmCK, tmCV, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  {
    // the merge kernel may be scheduled before the main kernel has drained (it waits with griddepcontrol.wait)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nitem);
    cfg.blockDim = dim3(kMergeGroups * D);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_merge_kernel, a);
    if (e != cudaSuccess) return (int)e;
  }
  note_launches(2);
  return (int)cudaGetLastError();
}
int decode_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
