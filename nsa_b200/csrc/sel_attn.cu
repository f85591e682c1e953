// Selected-block attention, query-major: forward (o_slc, lse_slc) and the dQ half of the backward.  General form for
// any block size (16/32/64 keys) and any number of selected blocks; 64-key blocks with at most 32 selections per
// query run the faster one-item-per-warp kernel of sel_block.cu instead.
//
// Reference behaviour: parallel_nsa_fwd_kernel (nsa/selection_attn.py:401-482) and the selected half
// of parallel_nsa_bwd_kernel_dq (nsa/selection_attn.py:276-356).  A query (b, t, kv head) visits the
// selected blocks whose first key is <= t (negative entries and entries past `counts` are skipped),
// masks keys > t inside a block, and soft-maxes over everything it visited.
//
// B200 design.  One persistent CTA per SM walks (b, t, 16-head group) items.  A producer warp TMA-
// gathers each selected [BS keys x D] K and V block by index (4-D tensor map, 128-byte swizzle) into a
// ring of shared-memory stages guarded by full/empty mbarriers, running ahead across items.  Four
// consumer warps each own 16 keys of every block: S = Q.K^T and P.V run on the tensor cores with the
// 16 query heads of the GQA group as the M=16 rows of mma.sync m16n8k16, so a gathered byte is used by
// all 16 heads.  The four partial soft-max states are merged in shared memory once per item.
#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;

__device__ __forceinline__ int load_block_index(const void* idx, int idx64, long long pos, int BS) {
  long long v = idx64 ? reinterpret_cast<const long long*>(idx)[pos] : (long long)reinterpret_cast<const int*>(idx)[pos];
  if (v < 0 || v > (long long)(0x7fffffff / BS)) return -1;
  return (int)v;
}

template <int D, bool BWD>
__global__ void __launch_bounds__(kThreads, BWD ? 1 : 2)
    sel_qmajor_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const SelArgs a,
                      const int nst) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BS = a.BS;
  const uint32_t panel_bytes = BS * 128;
  const uint32_t tile_bytes = panel_bytes * (D / 64);
  const uint32_t stage_bytes = 2 * tile_bytes;
  constexpr int PO = D + 8;  // padded row of the merge buffer (floats)
  const uint32_t merge_off = nst * stage_bytes;
  float* part_o = reinterpret_cast<float*>(sgen + merge_off);  // [4][16][PO]
  float* part_ml = part_o + kConsumerWarps * 16 * PO;          // [4][16][2]
  const uint32_t bar_base = sbase + merge_off + (kConsumerWarps * 16 * PO + kConsumerWarps * 16 * 2) * 4;
  auto full_bar = [&](int i) { return bar_base + 8u * i; };
  auto empty_bar = [&](int i) { return bar_base + 8u * (nst + i); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + (bar_base - sbase) + 8 * 32);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < nst; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), kConsumerWarps);
    }
    fence_mbar_init();
  }
  __syncthreads();

  const int HG = a.Hq / 16;
  const int G16 = (a.Hq / a.Hkv) / 16;
  const long long total = (long long)a.B * a.Tq * HG;

  if (warp == kConsumerWarps) {
    // ------------------------------- producer ------------------------------------------------
    // All 32 lanes fetch the item's block indices at once (one round trip instead of one per block); lane 0
    // then waits for a free stage and issues the TMA gathers.
    uint32_t it = 0;
    // the first 32 indices of the next item are fetched while the current item's gathers are issued
    auto item_row = [&](long long item) {
      const int hg = (int)(item % HG);
      const int tl = a.Tq - 1 - (int)((item / HG) % a.Tq);
      const int b = (int)(item / ((long long)HG * a.Tq));
      return ((long long)b * a.Tq + tl) * a.Hkv + hg / G16;
    };
    auto fetch = [&](long long item, int& cnt, int& first) {
      cnt = 0;
      first = -1;
      if (item >= total) return;
      const long long row = item_row(item);
      cnt = a.S;
      if (a.counts) cnt = min(cnt, a.counts[row]);
      if (lane < cnt) first = load_block_index(a.idx, a.idx64, row * a.S + lane, BS);
    };
    int cnt_next, first_next;
    fetch(blockIdx.x, cnt_next, first_next);
    for (long long item = blockIdx.x; item < total; item += gridDim.x) {
      const int hg = (int)(item % HG);
      const int tl = a.Tq - 1 - (int)((item / HG) % a.Tq);
      const int t = a.q0 + tl;   // sequence position of this query
      const int b = (int)(item / ((long long)HG * a.Tq));
      const int hkv = hg / G16;
      const long long row = ((long long)b * a.Tq + tl) * a.Hkv + hkv;
      const int cnt = cnt_next, first = first_next;
      fetch(item + gridDim.x, cnt_next, first_next);
      for (int s0 = 0; s0 < cnt; s0 += 32) {
        const int mine = (s0 == 0) ? first
                                   : ((s0 + lane < cnt) ? load_block_index(a.idx, a.idx64, row * a.S + s0 + lane, BS) : -1);
        const unsigned valid = __ballot_sync(0xffffffffu, mine >= 0 && (long long)mine * BS <= t);
        // lanes take turns handing their block to lane 0 (warp-uniform loop over the set bits)
        unsigned rem = valid;
        while (rem) {
          const int j = __ffs(rem) - 1;
          rem &= rem - 1;
          const int blk = __shfl_sync(0xffffffffu, mine, j);
          int good = 1;
          const int stage = it % nst;
          if (lane == 0) {
            const uint32_t ph = (it / nst) & 1;
            good = mbar_wait_abortable(empty_bar(stage), ph ^ 1, DEV_ERR_EMPTY_WAIT, abort_flag) ? 1 : 0;
            if (good) mbar_expect_tx(full_bar(stage), stage_bytes);
          }
          good = __shfl_sync(0xffffffffu, good, 0);
          // one box per lane (K/V x column panel): a single thread issuing them back to back is several times slower
          if (good && lane < 2 * (D / 64)) {
            const uint32_t dst = sbase + stage * stage_bytes;
            const int p = lane >> 1;
            if (lane & 1)
              tma_load_4d(dst + tile_bytes + p * panel_bytes, &tmV, full_bar(stage), p * 64, hkv, blk * BS, b);
            else
              tma_load_4d(dst + p * panel_bytes, &tmK, full_bar(stage), p * 64, hkv, blk * BS, b);
          }
          if (!good) return;
          ++it;
        }
      }
    }
    return;
  }

  // --------------------------------- consumers -------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const bool active = warp * 16 < BS;
  const float sl2 = a.scale * kLog2e;
  uint32_t it = 0;
  for (long long item = blockIdx.x; item < total; item += gridDim.x) {
    const int hg = (int)(item % HG);
    const int tl = a.Tq - 1 - (int)((item / HG) % a.Tq);
    const int t = a.q0 + tl;   // sequence position of this query
    const int b = (int)(item / ((long long)HG * a.Tq));
    const int hkv = hg / G16;
    const long long row = ((long long)b * a.Tq + tl) * a.Hkv + hkv;
    const long long qrow = ((long long)b * a.Tq + tl) * a.Hq + hg * 16;  // first of the 16 (token, head) rows

    uint32_t qf[D / 16][4];
    load_a_frags_global<D>(qf, a.q + qrow * D, lane);
    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // backward-only operands (kept in registers for the whole item)
    uint32_t dof[BWD ? D / 16 : 1][4];
    float lse2[2] = {0.f, 0.f}, dl[2] = {0.f, 0.f}, gt[2] = {1.f, 1.f};
    if constexpr (BWD) {
      load_a_frags_global<D>(dof, a.dout + qrow * D, lane);
      lse2[0] = a.lse[qrow + g] * kLog2e;
      lse2[1] = a.lse[qrow + g + 8] * kLog2e;
      dl[0] = a.delta[qrow + g];
      dl[1] = a.delta[qrow + g + 8];
      if (a.gate) {
        gt[0] = __bfloat162float(a.gate[qrow + g]);
        gt[1] = __bfloat162float(a.gate[qrow + g + 8]);
      }
    }

    int cnt = a.S;
    if (a.counts) cnt = min(cnt, a.counts[row]);
    for (int s0 = 0; s0 < cnt; s0 += 32) {
      const int mine = (s0 + lane < cnt) ? load_block_index(a.idx, a.idx64, row * a.S + s0 + lane, BS) : -1;
      const int nb = min(32, cnt - s0);
      for (int j = 0; j < nb; ++j) {
        const int blk = __shfl_sync(0xffffffffu, mine, j);
        if (blk < 0 || (long long)blk * BS > t) continue;
        const int stage = it % nst;
        const uint32_t ph = (it / nst) & 1;
        const bool got = mbar_wait_abortable(full_bar(stage), ph, DEV_ERR_FULL_WAIT, abort_flag);
        if (active && got) {
          const uint32_t kbase = sbase + stage * stage_bytes;
          const uint32_t vbase = kbase + tile_bytes;
          float sc[2][4];
#pragma unroll
          for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
          mma_a_bt16_split<D>(sc, qf, kbase, panel_bytes, warp * 16, lane);
          const int key0 = blk * BS + warp * 16 + 2 * tq;  // key of sc[0][0]; sc[nt][c]: + 8*nt + (c&1)
          if constexpr (!BWD) {
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int key = key0 + 8 * nt + (c & 1);
                const float v = (key <= t) ? sc[nt][c] * sl2 : -INFINITY;
                sc[nt][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
              }
            uint32_t pf[1][4];
            float p[2][4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const float mnew = fmaxf(m_run[r], quad_max(mx[r]));
              const float muse = (mnew == -INFINITY) ? 0.f : mnew;
              const float alpha = ex2(m_run[r] - muse);
              m_run[r] = mnew;
              float rs = 0.f;
#pragma unroll
              for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                  const float e = ex2(sc[nt][2 * r + c] - muse);
                  p[nt][2 * r + c] = e;
                  rs += e;
                }
              l_run[r] = l_run[r] * alpha + rs;
#pragma unroll
              for (int i = 0; i < D / 8; ++i) {
                acc[i][2 * r] *= alpha;
                acc[i][2 * r + 1] *= alpha;
              }
            }
            acc_to_a_frags<2>(pf, p);
            mma_a_b<D, 16>(acc, pf, vbase, panel_bytes, warp * 16, lane);
          } else {
            float dp[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
            mma_a_bt16_split<D>(dp, dof, vbase, panel_bytes, warp * 16, lane);
            float ds[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int key = key0 + 8 * nt + (c & 1);
                const int r = c >> 1;
                const float p = (key <= t) ? ex2(sc[nt][c] * sl2 - lse2[r]) : 0.f;
                ds[nt][c] = p * (gt[r] * dp[nt][c] - dl[r]);
              }
            uint32_t dsf[1][4];
            acc_to_a_frags<2>(dsf, ds);
            mma_a_b<D, 16>(acc, dsf, kbase, panel_bytes, warp * 16, lane);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));
        ++it;
      }
    }

    // ---- merge the four key-slices of this item ------------------------------------------------
    float* po = part_o + warp * 16 * PO;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      *reinterpret_cast<float2*>(po + g * PO + i * 8 + 2 * tq) = make_float2(acc[i][0], acc[i][1]);
      *reinterpret_cast<float2*>(po + (g + 8) * PO + i * 8 + 2 * tq) = make_float2(acc[i][2], acc[i][3]);
    }
    if constexpr (!BWD) {
      const float l0 = quad_sum(l_run[0]), l1 = quad_sum(l_run[1]);
      if (tq == 0) {
        part_ml[(warp * 16 + g) * 2 + 0] = m_run[0];
        part_ml[(warp * 16 + g) * 2 + 1] = l0;
        part_ml[(warp * 16 + g + 8) * 2 + 0] = m_run[1];
        part_ml[(warp * 16 + g + 8) * 2 + 1] = l1;
      }
    }
    named_bar_sync(1, kConsumerWarps * 32);
    {
      const int r = threadIdx.x >> 3, seg = threadIdx.x & 7;
      constexpr int CW = D / 8;  // columns per thread
      float w[kConsumerWarps];
      float inv = 1.f;
      if constexpr (!BWD) {
        float ms = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) ms = fmaxf(ms, part_ml[(ww * 16 + r) * 2]);
        float L = 0.f;
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) {
          const float mw = part_ml[(ww * 16 + r) * 2];
          w[ww] = (mw == -INFINITY) ? 0.f : ex2(mw - ms);
          L += w[ww] * part_ml[(ww * 16 + r) * 2 + 1];
        }
        inv = (L > 0.f) ? 1.f / L : 0.f;
        if (seg == 0) a.lse[qrow + r] = (L > 0.f) ? (ms + log2f(L)) * kLn2 : -INFINITY;
      } else {
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) w[ww] = 1.f;
        inv = a.scale;
      }
      // thread (r, seg) owns the column pairs 16*i + 2*seg: the 8 threads of a row read 64 contiguous bytes
      bf16* dst = (BWD ? a.dq : a.o) + (qrow + r) * D + 2 * seg;
#pragma unroll
      for (int i = 0; i < CW / 2; ++i) {
        const int c = 16 * i;
        float x0 = 0.f, x1 = 0.f;
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) {
          const float2 v = *reinterpret_cast<const float2*>(part_o + (ww * 16 + r) * PO + c + 2 * seg);
          x0 += w[ww] * v.x;
          x1 += w[ww] * v.y;
        }
        x0 *= inv;
        x1 *= inv;
        if (BWD && a.accumulate) {
          const __nv_bfloat162 old = *reinterpret_cast<const __nv_bfloat162*>(dst + c);
          x0 += __low2float(old);
          x1 += __high2float(old);
        }
        *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(x0, x1);
      }
    }
    named_bar_sync(1, kConsumerWarps * 32);
  }
}

template <int D, bool BWD>
int launch(const SelArgs& a, cudaStream_t s) {
  CUtensorMap tmK, tmV;
  int rc = make_tmap_rows4d(&tmK, a.k, D, a.Hkv, a.T, a.B, a.BS);
  if (rc) return rc;
  rc = make_tmap_rows4d(&tmV, a.v, D, a.Hkv, a.T, a.B, a.BS);
  if (rc) return rc;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const int stage_bytes = 2 * a.BS * D * 2;
  const int fixed = (kConsumerWarps * 16 * (D + 8) + kConsumerWarps * 16 * 2) * 4 + 2 * 16 * 8 + 64 + 1024;
  // the forward fits two CTAs per SM (168 registers): more resident warps hide the mma / ldmatrix latencies of
  // the 16-row tiles; the dQ variant needs 244 registers and loses more to spills than it gains
  const int per_cta = BWD ? max_smem : (max_smem - 2048) / 2;
  int nst = (per_cta - fixed) / stage_bytes;
  if (nst > 16) nst = 16;
  if (nst < 2) {
    set_error("selected attention: not enough shared memory for two stages");
    return -30;
  }
  const int smem = fixed + nst * stage_bytes;
  auto kern = sel_qmajor_kernel<D, BWD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * a.Tq * (a.Hq / 16);
  const long long slots = (long long)num_sms() * (BWD ? 1 : 2);
  const int grid = (int)(total < slots ? total : slots);
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, smem, s>>>(tmK, tmV, a, nst);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_sel_fwd(const SelArgs& a, int D, cudaStream_t s) {
  if (sel_block_supported(a, D)) return launch_sel_block(a, D, false, s);
  if (D == 128) return launch<128, false>(a, s);
  if (D == 64) return launch<64, false>(a, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}
int launch_sel_dq(const SelArgs& a, int D, cudaStream_t s) {
  if (sel_block_supported(a, D)) return launch_sel_block(a, D, true, s);
  if (D == 128) return launch<128, true>(a, s);
  if (D == 64) return launch<64, true>(a, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}
int sel_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
