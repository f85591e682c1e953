// Key/value-major half of the backward: dK,dV of the selected + sliding-window branches, and dCK,dCV of
// the compressed branch.
//
// Reference behaviour: parallel_nsa_bwd_kernel_dkv (nsa/selection_attn.py:151-253) walks, for every
// 64-key block, ALL later query tokens and tests a dense boolean block mask built by
// parallel_nsa_kernel_mask (:256-273); _attn_bwd_only_dkv (nsa/triton_attention.py:219-318) does the
// compressed branch.  Here the selected branch instead walks a per-block reverse index (CSR lists of the
// tokens that selected the block, ascending; see build_rev in misc.cu), so the work is proportional to
// the number of (token, block) pairs and there is no global atomic: one CTA owns a key block, keeps dK
// and dV of its 64 keys in registers over the whole list (then over the sliding-window tokens that see
// the block) and stores them once.
//
// B200 design.  The key block [rows x D] of K and V is TMA-loaded once.  A producer warp then streams,
// per (token, 16-head group), the [16 x D] Q tile and dO tile (2-D TMA boxes, 128-byte swizzle) plus the
// 16 lse / delta / gate values (bulk copies) through an mbarrier ring.  Four consumer warps own 16 keys
// each; with keys on the mma M axis and the 16 heads on N:
//     S^T = K.Q^T      P^T = exp(S^T*scale - lse)      dV += (g.P^T).dO
//     dP^T = V.dO^T    dS^T = P^T.(g.dP^T - delta)     dK += dS^T.Q   (times scale at the end)
// The compressed branch splits its long token range into segments that write fp32 partials, reduced by a
// second kernel in a fixed order (deterministic).
#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;

template <int D, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    kv_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDOa,
                  const __grid_constant__ CUtensorMap tmDOb, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const KvArgs a, const int nst) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int rows = (MODE == 0) ? a.BS : 64;              // keys per CTA
  const uint32_t kv_panel = rows * 128;
  const uint32_t kv_tile = kv_panel * (D / 64);
  constexpr uint32_t q_panel = 16 * 128;
  constexpr uint32_t q_tile = q_panel * (D / 64);
  constexpr uint32_t stage_bytes = 2 * q_tile + 1024;
  const uint32_t k_s = sbase, v_s = sbase + kv_tile;
  const uint32_t ring = sbase + 2 * kv_tile;              // kv_tile is a multiple of 1024
  const uint32_t bar_base = ring + nst * stage_bytes;
  auto full_bar = [&](int i) { return bar_base + 8u * i; };
  auto empty_bar = [&](int i) { return bar_base + 8u * (nst + i); };
  const uint32_t kv_bar = bar_base + 16u * nst;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), kConsumerWarps);
    }
    mbar_init(kv_bar, 1);
    fence_mbar_init();
  }
  __syncthreads();

  // ---- decode the work item -----------------------------------------------------------------------
  const int G16 = (a.Hq / a.Hk) / 16;
  int b, hk, blk, seg = 0;
  int ta_lo = 0, ta_hi = 0;    // branch A token range (mode 1) or list range (mode 0)
  int tb_lo = 0, tb_hi = 0;    // branch B token range (mode 0, window)
  const int* list = nullptr;
  {
    long long item = blockIdx.x;
    const int BH = a.B * a.Hk;
    if (MODE == 0) {
      blk = (int)(item / BH);
      const int bh = (int)(item % BH);
      b = bh / a.Hk;
      hk = bh % a.Hk;
      const int NB = (a.T + a.BS - 1) / a.BS;
      if (a.rev_ptr) {
        const int* rp = a.rev_ptr + (long long)bh * (NB + 1);
        ta_lo = rp[blk];
        ta_hi = rp[blk + 1];
        list = a.rev_tok + (long long)bh * a.rev_cap;
      }
      if (a.window > 0) {
        tb_lo = blk * a.BS;
        tb_hi = min(a.T, blk * a.BS + a.BS - 1 + a.window);
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
      ta_lo = max(first, seg * a.seg_len);
      ta_hi = min(a.T, (seg + 1) * a.seg_len);
      if (ta_hi <= ta_lo) return;  // this segment sees nothing of the tile; the reducer knows too
    }
  }
  const int key0 = blk * rows;
  const int nA = max(0, ta_hi - ta_lo), nB = max(0, tb_hi - tb_lo);

  if (warp == kConsumerWarps) {
    // ------------------------------- producer ------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(kv_bar, 2 * kv_tile);
#pragma unroll
      for (int p = 0; p < D / 64; ++p) {
        tma_load_4d(k_s + p * kv_panel, &tmK, kv_bar, p * 64, hk, key0, b);
        tma_load_4d(v_s + p * kv_panel, &tmV, kv_bar, p * 64, hk, key0, b);
      }
    }
    uint32_t it = 0;
    for (int sub = 0; sub < G16; ++sub) {
      const int hg = hk * G16 + sub;
      for (int br = 0; br < 2; ++br) {
        const int n = br == 0 ? nA : nB;
        const CUtensorMap* tmDO = br == 0 ? &tmDOa : &tmDOb;
        const float* lse = br == 0 ? a.lse_a : a.lse_b;
        const float* delta = br == 0 ? a.delta_a : a.delta_b;
        const bf16* gate = br == 0 ? a.gate_a : a.gate_b;
        const uint32_t tx = 2 * q_tile + 128 + (gate ? 32 : 0);
        for (int i0 = 0; i0 < n; i0 += 32) {
          int tok;
          if (br == 0)
            tok = (MODE == 0) ? ((i0 + lane < n) ? list[ta_lo + i0 + lane] : 0) : ta_lo + i0 + lane;
          else
            tok = tb_lo + i0 + lane;
          const int nn = min(32, n - i0);
          for (int j = 0; j < nn; ++j) {
            const int t = __shfl_sync(0xffffffffu, tok, j);
            bool okw = true;
            if (lane == 0) {
              const int stage = it % nst;
              const uint32_t ph = (it / nst) & 1;
              okw = mbar_wait(empty_bar(stage), ph ^ 1, DEV_ERR_EMPTY_WAIT);
              if (okw) {
                const long long qrow = ((long long)b * a.T + t) * a.Hq + hg * 16;
                const uint32_t dst = ring + stage * stage_bytes;
                mbar_expect_tx(full_bar(stage), tx);
#pragma unroll
                for (int p = 0; p < D / 64; ++p) {
                  tma_load_2d(dst + p * q_panel, &tmQ, full_bar(stage), p * 64, (int)qrow);
                  tma_load_2d(dst + q_tile + p * q_panel, tmDO, full_bar(stage), p * 64, (int)qrow);
                }
                bulk_load(dst + 2 * q_tile, lse + qrow, 64, full_bar(stage));
                bulk_load(dst + 2 * q_tile + 64, delta + qrow, 64, full_bar(stage));
                if (gate) bulk_load(dst + 2 * q_tile + 128, gate + qrow, 32, full_bar(stage));
              }
            }
            if (!__shfl_sync(0xffffffffu, (int)okw, 0)) return;
            ++it;
          }
        }
      }
    }
    return;
  }

  // --------------------------------- consumers -------------------------------------------------
  const int g = lane >> 2, tq = lane & 3;
  const bool active = warp * 16 < rows;
  const float sl2 = a.scale * kLog2e;
  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  if (!mbar_wait(kv_bar, 0, DEV_ERR_FULL_WAIT)) return;
  const int kp0 = key0 + warp * 16 + g;  // key position of accumulator rows c<2; +8 for c>=2

  uint32_t it = 0;
  for (int sub = 0; sub < G16; ++sub) {
    for (int br = 0; br < 2; ++br) {
      const int n = br == 0 ? nA : nB;
      const bool has_gate = (br == 0 ? a.gate_a : a.gate_b) != nullptr;
      for (int i0 = 0; i0 < n; i0 += 32) {
        int tok;
        if (br == 0)
          tok = (MODE == 0) ? ((i0 + lane < n) ? list[ta_lo + i0 + lane] : 0) : ta_lo + i0 + lane;
        else
          tok = tb_lo + i0 + lane;
        const int nn = min(32, n - i0);
        for (int j = 0; j < nn; ++j) {
          const int t = __shfl_sync(0xffffffffu, tok, j);
          const int stage = it % nst;
          const uint32_t ph = (it / nst) & 1;
          if (!mbar_wait(full_bar(stage), ph, DEV_ERR_FULL_WAIT)) return;
          if (active) {
            const uint32_t qs = ring + stage * stage_bytes;
            const uint32_t dos = qs + q_tile;
            const uint8_t* aux = sgen + (qs - sbase) + 2 * q_tile;
            const float* lse_s = reinterpret_cast<const float*>(aux);
            const float* del_s = reinterpret_cast<const float*>(aux + 64);
            const bf16* gate_s = reinterpret_cast<const bf16*>(aux + 128);
            float st[2][4], dpt[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
              dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f;
            }
            {
              uint32_t af[D / 16][4];
              load_a_frags<D>(af, k_s, kv_panel, warp * 16, lane);
              mma_a_bt<D, 16>(st, af, qs, q_panel, 0, lane);
            }
            {
              uint32_t af[D / 16][4];
              load_a_frags<D>(af, v_s, kv_panel, warp * 16, lane);
              mma_a_bt<D, 16>(dpt, af, dos, q_panel, 0, lane);
            }
            float pg[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int h = 8 * nt + 2 * tq + (c & 1);
                const int kp = kp0 + (c >> 1) * 8;
                bool ok;
                if (MODE == 0)
                  ok = (kp <= t) && (br == 0 || kp > t - a.window);
                else
                  ok = kp < a.Lk && (!a.causal || kp * a.cstride + a.cblock <= t);
                const float l2v = lse_s[h] * kLog2e;
                const float gv = has_gate ? __bfloat162float(gate_s[h]) : 1.f;
                const float p = (ok && l2v > -INFINITY) ? ex2(st[nt][c] * sl2 - l2v) : 0.f;
                pg[nt][c] = p * gv;
                st[nt][c] = p * (gv * dpt[nt][c] - del_s[h]);
              }
            uint32_t f[1][4];
            acc_to_a_frags<2>(f, pg);
            mma_a_b<D, 16>(dv, f, dos, q_panel, 0, lane);
            acc_to_a_frags<2>(f, st);
            mma_a_b<D, 16>(dk, f, qs, q_panel, 0, lane);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(stage));
          ++it;
        }
      }
    }
  }

  // ---- store ----------------------------------------------------------------------------------------
  if (!active) return;
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int kp = kp0 + hrow * 8;
    if (kp >= a.Lk) continue;
    const long long off = (((long long)b * a.Lk + kp) * a.Hk + hk) * D + 2 * tq;
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<__nv_bfloat162*>(a.dk + off + i * 8) =
            __floats2bfloat162_rn(dk[i][2 * hrow] * a.scale, dk[i][2 * hrow + 1] * a.scale);
        *reinterpret_cast<__nv_bfloat162*>(a.dv + off + i * 8) =
            __floats2bfloat162_rn(dv[i][2 * hrow], dv[i][2 * hrow + 1]);
      }
    } else {
      const long long N = (long long)a.B * a.Lk * a.Hk * D;
      float* pk = a.part + (long long)seg * N + off;
      float* pv = a.part + ((long long)a.nseg + seg) * N + off;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        *reinterpret_cast<float2*>(pk + i * 8) = make_float2(dk[i][2 * hrow] * a.scale, dk[i][2 * hrow + 1] * a.scale);
        *reinterpret_cast<float2*>(pv + i * 8) = make_float2(dv[i][2 * hrow], dv[i][2 * hrow + 1]);
      }
    }
  }
}

template <int D, int MODE>
int launch(const KvArgs& a, cudaStream_t s) {
  CUtensorMap tmQ, tmA, tmB, tmK, tmV;
  const long long qrows = (long long)a.B * a.T * a.Hq;
  if (qrows > 0x7fffffffLL) {
    set_error("B*T*Hq exceeds the 2^31 rows a TMA coordinate can address");
    return -32;
  }
  const int rows = MODE == 0 ? a.BS : 64;
  int rc = make_tmap_rows2d(&tmQ, a.q, D, qrows, 16);
  if (!rc) rc = make_tmap_rows2d(&tmA, a.dout_a ? a.dout_a : a.dout_b, D, qrows, 16);
  if (!rc) rc = make_tmap_rows2d(&tmB, a.dout_b ? a.dout_b : a.dout_a, D, qrows, 16);
  if (!rc) rc = make_tmap_rows4d(&tmK, a.k, D, a.Hk, a.Lk, a.B, rows);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hk, a.Lk, a.B, rows);
  if (rc) return rc;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const int stage_bytes = 2 * 16 * D * 2 + 1024;
  const int fixed = 2 * rows * D * 2 + (2 * 16 + 1) * 8 + 1024;
  int nst = (max_smem / 2 - fixed) / stage_bytes;  // leave room for two CTAs per SM
  if (nst > 8) nst = 8;
  if (nst < 2) nst = 2;
  const int smem = fixed + nst * stage_bytes;
  auto kern = kv_bwd_kernel<D, MODE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  long long grid;
  if (MODE == 0)
    grid = (long long)a.B * a.Hk * ((a.T + a.BS - 1) / a.BS);
  else
    grid = (long long)a.B * a.Hk * ((a.Lk + 63) / 64) * a.nseg;
  if (grid <= 0) return 0;
  if (grid > 0x7fffffffLL) {
    set_error("kv backward: grid too large");
    return -33;
  }
  kern<<<(unsigned)grid, kThreads, smem, s>>>(tmQ, tmA, tmB, tmK, tmV, a, nst);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_kv_bwd(const KvArgs& a, int D, cudaStream_t s) {
  if (D == 128) return a.mode == 0 ? launch<128, 0>(a, s) : launch<128, 1>(a, s);
  if (D == 64) return a.mode == 0 ? launch<64, 0>(a, s) : launch<64, 1>(a, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}
int kv_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
