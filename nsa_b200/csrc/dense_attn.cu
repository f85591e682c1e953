// Dense query-major attention over a contiguous key range, shared by two branches:
//
//   mode 0  sliding-window attention: query t sees keys max(0, t-W+1) .. t of k,v [B,T,Hkv,D].
//           Reference: the window half of parallel_nsa_fwd_kernel (nsa/selection_attn.py:484-516) and of
//           parallel_nsa_bwd_kernel_dq (:358-398).
//   mode 1  compressed attention over ck,cv [B,Tc,Hk,D]: compressed position j is visible to t iff
//           t >= j*stride + block; rows with no visible position give 0 / lse = -inf.
//           Reference: _attn_fwd (nsa/triton_attention.py:87-181), _attn_bwd_only_dq (:321-416).
//           The forward can also produce the selected block indices: softmax over ALL compressed
//           positions of the unscaled, unmasked q.ck, summed over the 16 heads of the group, average
//           pooled and top-n'd (nsa/torch_attention.py:51-62,121-125; nsa/triton_attention.py:465-475).
//           Scores never leave the SM: a first pass gathers the row max / row sum, a second pass
//           recomputes q.ck, normalises, reduces over heads with warp shuffles, pools into a per-token
//           shared-memory vector and a warp picks the top n (ties to the lower block index).
//
// B200 design.  A persistent CTA owns 8 consecutive tokens of one 16-head GQA group: warp w holds the
// [16 heads x D] query tile of token t0+w as mma A-fragments.  A producer warp streams [64 keys x D]
// K/V tiles by TMA (128-byte swizzle) through an mbarrier ring; every tile is used by all 8 tokens x 16
// heads, so L2->SM traffic is 1/128 of a per-row gather.
#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int kTok = 8;                       // tokens (= consumer warps) per CTA
constexpr int kThreads = (kTok + 1) * 32;
constexpr uint32_t kPanel = 64 * 128;         // one [64 x 64] bf16 panel

struct Sched {
  int first, nA, nAttn, nB;
};

template <int MODE, bool BWD>
__device__ __forceinline__ Sched make_sched(const DenseArgs& a, int t0) {
  Sched s;
  const int tmax = min(a.T - 1, t0 + kTok - 1);
  if (MODE == 0) {
    s.first = max(0, t0 - a.window + 1) / 64;
    s.nA = tmax / 64 - s.first + 1;
    s.nAttn = s.nA;
    s.nB = 0;
  } else {
    const int nt_all = (a.Lk + 63) / 64;
    int nvis = a.Lk;
    if (a.causal) nvis = (tmax < a.cblock) ? 0 : min(a.Lk, (tmax - a.cblock) / a.cstride + 1);
    s.first = 0;
    s.nAttn = (nvis + 63) / 64;
    const bool sel = (!BWD) && a.n_sel > 0;
    s.nA = sel ? nt_all : s.nAttn;
    s.nB = sel ? nt_all : 0;
  }
  return s;
}

template <int D, int MODE, bool BWD>
__global__ void __launch_bounds__(kThreads, 1)
    dense_qmajor_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const DenseArgs a, const int nst, const int pool_stride_f) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t tile_bytes = kPanel * (D / 64);
  constexpr uint32_t stage_bytes = 2 * tile_bytes;
  float* pool_s = reinterpret_cast<float*>(sgen + nst * stage_bytes);  // [kTok][pool_stride_f]
  const uint32_t bar_base = sbase + nst * stage_bytes + kTok * pool_stride_f * 4;
  auto full_bar = [&](int i) { return bar_base + 8u * i; };
  auto empty_bar = [&](int i) { return bar_base + 8u * (nst + i); };
  if (threadIdx.x == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), kTok);
    }
    fence_mbar_init();
  }
  __syncthreads();

  const int HG = a.Hq / 16;
  const int G16 = (a.Hq / a.Hk) / 16;
  const int ntile = (a.T + kTok - 1) / kTok;
  const long long total = (long long)a.B * HG * ntile;

  if (warp == kTok) {
    // ------------------------------- producer ------------------------------------------------
    // lane 0 waits for a free stage and arms its barrier; the boxes are issued one per lane
    uint32_t it = 0;
    for (long long item = blockIdx.x; item < total; item += gridDim.x) {
      const int hg = (int)(item % HG);
      const int tile = ntile - 1 - (int)((item / HG) % ntile);
      const int b = (int)(item / ((long long)HG * ntile));
      const int hk = hg / G16;
      const Sched sc = make_sched<MODE, BWD>(a, tile * kTok);
      for (int i = 0; i < sc.nA + sc.nB; ++i) {
        const bool withv = i < sc.nAttn;
        const int jt = sc.first + (i < sc.nA ? i : i - sc.nA);
        const int stage = it % nst;
        int good = 1;
        if (lane == 0) {
          const uint32_t ph = (it / nst) & 1;
          good = mbar_wait(empty_bar(stage), ph ^ 1, DEV_ERR_EMPTY_WAIT) ? 1 : 0;
          if (good) mbar_expect_tx(full_bar(stage), withv ? stage_bytes : tile_bytes);
        }
        if (!__shfl_sync(0xffffffffu, good, 0)) return;
        if (lane < 2 * (D / 64)) {
          const uint32_t dst = sbase + stage * stage_bytes;
          const int p = lane >> 1;
          if (lane & 1) {
            if (withv) tma_load_4d(dst + tile_bytes + p * kPanel, &tmV, full_bar(stage), p * 64, hk, jt * 64, b);
          } else {
            tma_load_4d(dst + p * kPanel, &tmK, full_bar(stage), p * 64, hk, jt * 64, b);
          }
        }
        ++it;
      }
    }
    return;
  }

  // --------------------------------- consumers -------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const float sl2 = a.scale * kLog2e;
  float* my_pool = pool_s + warp * pool_stride_f;  // [n_pool_pad] pooled sums, then [64] column sums
  float* my_col = my_pool + (pool_stride_f - 64);
  uint32_t it = 0;
  for (long long item = blockIdx.x; item < total; item += gridDim.x) {
    const int hg = (int)(item % HG);
    const int tile = ntile - 1 - (int)((item / HG) % ntile);
    const int b = (int)(item / ((long long)HG * ntile));
    const int t0 = tile * kTok;
    const int t = t0 + warp;
    const bool live = t < a.T;
    const Sched sch = make_sched<MODE, BWD>(a, t0);
    const long long qrow = ((long long)b * a.T + (live ? t : 0)) * a.Hq + hg * 16;

    uint32_t qf[D / 16][4];
    load_a_frags_global<D>(qf, a.q + qrow * D, lane);
    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float m2[2] = {-INFINITY, -INFINITY}, l2[2] = {0.f, 0.f};  // selection soft-max statistics (raw scores)

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
    // number of compressed positions this token sees (mode 1)
    int nvis = a.Lk;
    if (MODE == 1 && a.causal) nvis = (t < a.cblock) ? 0 : min(a.Lk, (t - a.cblock) / a.cstride + 1);

    const bool do_sel = MODE == 1 && !BWD && a.n_sel > 0;
    if (do_sel) {
      for (int i = lane; i < a.n_pool; i += 32) my_pool[i] = 0.f;
      __syncwarp();
    }

    for (int i = 0; i < sch.nA + sch.nB; ++i) {
      const bool passB = i >= sch.nA;
      const int jt = sch.first + (passB ? i - sch.nA : i);
      const int j0 = jt * 64;
      const int stage = it % nst;
      const uint32_t ph = (it / nst) & 1;
      if (!mbar_wait(full_bar(stage), ph, DEV_ERR_FULL_WAIT)) return;
      const uint32_t kbase = sbase + stage * stage_bytes;
      const uint32_t vbase = kbase + tile_bytes;
      if (live) {
        if constexpr (!BWD) {
          bool attend;
          if (MODE == 0)
            attend = !passB && (j0 <= t) && (j0 + 63 > t - a.window);
          else
            attend = !passB && (j0 < nvis);
          if (attend || do_sel) {
            float sc[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
            mma_a_bt<D, 64>(sc, qf, kbase, kPanel, 0, lane);
            const int jb = j0 + 2 * tq;  // column of sc[0][0]; sc[n][c] is column jb + 8n + (c&1)
            if (do_sel && !passB) {
              // statistics of the unscaled, unmasked soft-max over all Lk positions
              float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
              for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                  if (jb + 8 * n + (c & 1) < a.Lk) mx[c >> 1] = fmaxf(mx[c >> 1], sc[n][c]);
#pragma unroll
              for (int r = 0; r < 2; ++r) {
                const float mnew = fmaxf(m2[r], quad_max(mx[r]));
                const float muse = (mnew == -INFINITY) ? 0.f : mnew;
                float rs = 0.f;
#pragma unroll
                for (int n = 0; n < 8; ++n)
#pragma unroll
                  for (int c = 0; c < 2; ++c)
                    if (jb + 8 * n + c < a.Lk) rs += ex2((sc[n][2 * r + c] - muse) * kLog2e);
                l2[r] = l2[r] * ex2((m2[r] - muse) * kLog2e) + rs;
                m2[r] = mnew;
              }
            }
            if (do_sel && passB) {
              // p = softmax(raw) summed over the 16 heads -> 64 column sums -> pooled blocks
              const float inv0 = 1.f / quad_sum(l2[0]);
              const float inv1 = 1.f / quad_sum(l2[1]);
#pragma unroll
              for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                  float v = 0.f;
                  if (jb + 8 * n + c < a.Lk)
                    v = ex2((sc[n][c] - m2[0]) * kLog2e) * inv0 + ex2((sc[n][2 + c] - m2[1]) * kLog2e) * inv1;
                  v += __shfl_xor_sync(0xffffffffu, v, 4);
                  v += __shfl_xor_sync(0xffffffffu, v, 8);
                  v += __shfl_xor_sync(0xffffffffu, v, 16);
                  if (g == 0) my_col[8 * n + 2 * tq + c] = v;
                }
              __syncwarp();
              // blocks whose window meets columns [j0, j0+64)
              int blo = j0 + a.pool_p - a.pool_k + 1;
              blo = blo <= 0 ? 0 : (blo + a.pool_s - 1) / a.pool_s;
              const int bhi = min(a.n_pool - 1, (j0 + 63 + a.pool_p) / a.pool_s);
              for (int blk = blo + lane; blk <= bhi; blk += 32) {
                const int lo = blk * a.pool_s - a.pool_p;
                const int hi = min(lo + a.pool_k, a.Lk + a.pool_p);
                const int ja = max(max(lo, 0), j0), jz = min(min(hi, a.Lk), j0 + 64);
                float sum = 0.f;
                for (int j = ja; j < jz; ++j) sum += my_col[j - j0];
                my_pool[blk] += sum;
              }
              __syncwarp();
            }
            if (attend) {
              float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
              for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const int j = jb + 8 * n + (c & 1);
                  bool ok;
                  if (MODE == 0)
                    ok = (j <= t) && (j > t - a.window);
                  else
                    ok = j < nvis;
                  const float v = ok ? sc[n][c] * sl2 : -INFINITY;
                  sc[n][c] = v;
                  mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
#pragma unroll
              for (int r = 0; r < 2; ++r) {
                const float mnew = fmaxf(m_run[r], quad_max(mx[r]));
                const float muse = (mnew == -INFINITY) ? 0.f : mnew;
                const float alpha = ex2(m_run[r] - muse);
                m_run[r] = mnew;
                float rs = 0.f;
#pragma unroll
                for (int n = 0; n < 8; ++n)
#pragma unroll
                  for (int c = 0; c < 2; ++c) {
                    const float e = ex2(sc[n][2 * r + c] - muse);
                    sc[n][2 * r + c] = e;
                    rs += e;
                  }
                l_run[r] = l_run[r] * alpha + rs;
#pragma unroll
                for (int d8 = 0; d8 < D / 8; ++d8) {
                  acc[d8][2 * r] *= alpha;
                  acc[d8][2 * r + 1] *= alpha;
                }
              }
              uint32_t pf[4][4];
              acc_to_a_frags<8>(pf, sc);
              mma_a_b<D, 64>(acc, pf, vbase, kPanel, 0, lane);
            }
          }
        } else {
          bool attend;
          if (MODE == 0)
            attend = (j0 <= t) && (j0 + 63 > t - a.window);
          else
            attend = j0 < nvis;
          if (attend) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float sc[4][4], dp[4][4];
#pragma unroll
              for (int n = 0; n < 4; ++n) {
                sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
                dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f;
              }
              mma_a_bt<D, 32>(sc, qf, kbase, kPanel, h * 32, lane);
              mma_a_bt<D, 32>(dp, dof, vbase, kPanel, h * 32, lane);
              const int jb = j0 + h * 32 + 2 * tq;
#pragma unroll
              for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const int j = jb + 8 * n + (c & 1);
                  const int r = c >> 1;
                  bool ok;
                  if (MODE == 0)
                    ok = (j <= t) && (j > t - a.window);
                  else
                    ok = j < nvis;
                  const float p = ok ? ex2(sc[n][c] * sl2 - lse2[r]) : 0.f;
                  sc[n][c] = p * (gt[r] * dp[n][c] - dl[r]);
                }
              uint32_t dsf[2][4];
              acc_to_a_frags<4>(dsf, sc);
              mma_a_b<D, 32>(acc, dsf, kbase, kPanel, h * 32, lane);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(stage));
      ++it;
    }

    if (!live) continue;
    // ---- epilogue ------------------------------------------------------------------------------
    if constexpr (!BWD) {
      const float l0 = quad_sum(l_run[0]), l1 = quad_sum(l_run[1]);
      const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
      bf16* o0 = a.o + (qrow + g) * D + 2 * tq;
      bf16* o1 = a.o + (qrow + g + 8) * D + 2 * tq;
#pragma unroll
      for (int d8 = 0; d8 < D / 8; ++d8) {
        *reinterpret_cast<__nv_bfloat162*>(o0 + d8 * 8) = __floats2bfloat162_rn(acc[d8][0] * i0, acc[d8][1] * i0);
        *reinterpret_cast<__nv_bfloat162*>(o1 + d8 * 8) = __floats2bfloat162_rn(acc[d8][2] * i1, acc[d8][3] * i1);
      }
      if (tq == 0) {
        a.lse[qrow + g] = l0 > 0.f ? (m_run[0] + log2f(l0)) * kLn2 : -INFINITY;
        a.lse[qrow + g + 8] = l1 > 0.f ? (m_run[1] + log2f(l1)) * kLn2 : -INFINITY;
      }
      if (do_sel) {
        // divide by the window length, optionally dump, then pick the top n blocks
        for (int blk = lane; blk < a.n_pool; blk += 32) {
          const int lo = blk * a.pool_s - a.pool_p;
          const int hi = min(lo + a.pool_k, a.Lk + a.pool_p);
          const float v = my_pool[blk] / (float)(hi - lo);
          my_pool[blk] = v;
          if (a.sel_scores) a.sel_scores[(((long long)b * HG + hg) * a.T + t) * a.n_pool + blk] = v;
        }
        __syncwarp();
        int* out = a.sel_idx + (((long long)b * a.T + t) * HG + hg) * a.n_sel;
        for (int r = 0; r < a.n_sel; ++r) {
          float bv = -2.f;
          int bi = 0x7fffffff;
          for (int blk = lane; blk < a.n_pool; blk += 32) {
            const float v = my_pool[blk];
            if (v > bv) {  // ascending scan keeps the lowest index among equals
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
            if (found) my_pool[bi] = -2.f;
          }
          __syncwarp();
        }
      }
    } else {
      bf16* o0 = a.dq + (qrow + g) * D + 2 * tq;
      bf16* o1 = a.dq + (qrow + g + 8) * D + 2 * tq;
#pragma unroll
      for (int d8 = 0; d8 < D / 8; ++d8) {
        float x0 = acc[d8][0] * a.scale, x1 = acc[d8][1] * a.scale, x2 = acc[d8][2] * a.scale,
              x3 = acc[d8][3] * a.scale;
        if (a.accumulate) {
          const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(o0 + d8 * 8);
          const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(o1 + d8 * 8);
          x0 += __low2float(p0);
          x1 += __high2float(p0);
          x2 += __low2float(p1);
          x3 += __high2float(p1);
        }
        *reinterpret_cast<__nv_bfloat162*>(o0 + d8 * 8) = __floats2bfloat162_rn(x0, x1);
        *reinterpret_cast<__nv_bfloat162*>(o1 + d8 * 8) = __floats2bfloat162_rn(x2, x3);
      }
    }
  }
}

template <int D, int MODE, bool BWD>
int launch(const DenseArgs& a, cudaStream_t s) {
  CUtensorMap tmK, tmV;
  int rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.Lk, a.B, 64);
  if (rc) return rc;
  rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.Lk, a.B, 64);
  if (rc) return rc;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const int stage_bytes = 2 * 64 * D * 2;
  const bool sel = MODE == 1 && !BWD && a.n_sel > 0;
  const int pool_stride_f = sel ? ((a.n_pool + 3) / 4 * 4 + 64) : 0;
  const int fixed = kTok * pool_stride_f * 4 + 2 * 16 * 8 + 1024;
  int nst = (max_smem - fixed) / stage_bytes;
  if (nst > 6) nst = 6;
  if (nst < 2) {
    set_error("dense attention: sequence too long for the shared-memory score pool (n_pool=%d)", a.n_pool);
    return -31;
  }
  const int smem = fixed + nst * stage_bytes;
  auto kern = dense_qmajor_kernel<D, MODE, BWD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * (a.Hq / 16) * ((a.T + kTok - 1) / kTok);
  const int grid = (int)(total < num_sms() ? total : num_sms());
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, smem, s>>>(tmK, tmV, a, nst, pool_stride_f);
  note_launches(1);
  return (int)cudaGetLastError();
}

template <bool BWD>
int dispatch(const DenseArgs& a, int D, cudaStream_t s) {
  if (D == 128) return a.mode == 0 ? launch<128, 0, BWD>(a, s) : launch<128, 1, BWD>(a, s);
  if (D == 64) return a.mode == 0 ? launch<64, 0, BWD>(a, s) : launch<64, 1, BWD>(a, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}

}  // namespace

int launch_dense_fwd(const DenseArgs& a, int D, cudaStream_t s) { return dispatch<false>(a, D, s); }
int launch_dense_dq(const DenseArgs& a, int D, cudaStream_t s) { return dispatch<true>(a, D, s); }
int dense_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
