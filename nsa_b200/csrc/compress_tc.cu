// Compression forward for equal-length sequences as one tcgen05 GEMM per (batch, head, 128 output rows):
//     Y[i, :] = bias + sum_{j<l} X[i*d + j, :] . W_j          (nsa/compression_kv.py:21-57 and :298-307)
// The overlapping windows are never materialised.  x [B,T,H,D] is viewed through a 5-D tensor map
// (channel, head, offset-in-stride jj, stride chunk u, batch): window row i at in-block offset j = r*d + jj is the
// row (u = i + r, jj), so a [128 rows x 64 channels] A tile for one (j, channel half) is ONE TMA box whose rows are
// d tokens apart.  W [l*D, D] chunks are the MN-major B operand (rows = contraction index, 128-byte swizzled; in its
// descriptor the leading byte offset is the distance between the two 64-column panels and the stride byte offset
// the 1024 bytes between 8-row groups).
// Warp 0 streams tiles through an mbarrier ring, one thread of warp 1 issues tcgen05.mma into a [128 x D] fp32
// accumulator in TMEM, warps 2-5 read it back with tcgen05.ld, add the bias and store bf16.
#include "kernels.h"
#include "tc.cuh"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int kThreads = 192;

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
    compress_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                           const bf16* __restrict__ bias, bf16* __restrict__ y, const int Tc, const int H, const int l,
                           const int d, const int nst) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - raw);
  constexpr uint32_t A_BYTES = 128 * 128;          // [128 rows][64 ch]
  constexpr uint32_t W_PANEL = 64 * 128;           // [64 k][64 n]
  constexpr uint32_t W_BYTES = W_PANEL * (D / 64);
  constexpr uint32_t STAGE = A_BYTES + W_BYTES;
  const uint32_t bar_base = sbase + nst * STAGE;
  auto full_bar = [&](int i) { return bar_base + 8u * i; };
  auto empty_bar = [&](int i) { return bar_base + 8u * (nst + i); };
  const uint32_t acc_bar = bar_base + 16u * nst;
  const uint32_t tmem_slot = acc_bar + 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y / H, h = blockIdx.y % H;
  const int i0 = blockIdx.x * 128;
  const int nk = l * D / 64;

  if (threadIdx.x == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), 1);
    }
    mbar_init(acc_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, D);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(sgen + (tmem_slot - sbase));

  if (warp == 0) {
    if (lane == 0) {
      for (int kk = 0; kk < nk; ++kk) {
        const int stage = kk % nst;
        const uint32_t ph = (kk / nst) & 1;
        if (!mbar_wait(empty_bar(stage), ph ^ 1, DEV_ERR_EMPTY_WAIT)) break;
        mbar_expect_tx(full_bar(stage), STAGE);
        const uint32_t a_s = sbase + stage * STAGE, w_s = a_s + A_BYTES;
        const int j = (kk * 64) / D, c0 = (kk * 64) % D;
        tma_load_5d(a_s, &tmX, full_bar(stage), c0, h, j % d, i0 + j / d, b);
#pragma unroll
        for (int p = 0; p < D / 64; ++p) tma_load_2d(w_s + p * W_PANEL, &tmW, full_bar(stage), p * 64, kk * 64);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, D, 0, 1);
      for (int kk = 0; kk < nk; ++kk) {
        const int stage = kk % nst;
        const uint32_t ph = (kk / nst) & 1;
        if (!mbar_wait(full_bar(stage), ph, DEV_ERR_FULL_WAIT)) break;
        tc_fence_after();
        const uint32_t a_s = sbase + stage * STAGE, w_s = a_s + A_BYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem, umma_smem_desc(a_s + ks * 32, 0, 1024), umma_smem_desc(w_s + ks * 2048, W_PANEL, 1024), idesc,
                  (kk | ks) ? 1u : 0u);
        umma_commit(empty_bar(stage));
      }
      umma_commit(acc_bar);
    }
  } else {
    const bool ok = mbar_wait(acc_bar, 0, DEV_ERR_FULL_WAIT);
    tc_fence_after();
    const int row = 32 * (warp & 3) + lane;
    const int i = i0 + row;
    bf16* dst = y + (((long long)b * Tc + i) * H + h) * D;
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      float v[16];
      tmem_ld16(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + c * 16, v);
      tmem_ld_wait();
      if (ok && i < Tc) {
        uint4 o[2];
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float x0 = v[2 * e], x1 = v[2 * e + 1];
          if (bias) {
            x0 += __bfloat162float(bias[c * 16 + 2 * e]);
            x1 += __bfloat162float(bias[c * 16 + 2 * e + 1]);
          }
          ho[e] = __floats2bfloat162_rn(x0, x1);
        }
        *reinterpret_cast<uint4*>(dst + c * 16) = o[0];
        *reinterpret_cast<uint4*>(dst + c * 16 + 8) = o[1];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, D);
}

template <int D>
int launch(const bf16* x, const bf16* w, const bf16* bias, bf16* y, int B, int T, int H, int l, int d, cudaStream_t s) {
  const int Tc = (T - l) / d + 1;
  CUtensorMap tmX, tmW;
  const unsigned long long dims[5] = {(unsigned long long)D, (unsigned long long)H, (unsigned long long)d,
                                      (unsigned long long)(T / d), (unsigned long long)B};
  const unsigned long long strides[4] = {(unsigned long long)D * 2, (unsigned long long)H * D * 2,
                                         (unsigned long long)d * H * D * 2, (unsigned long long)T * H * D * 2};
  const unsigned box[5] = {64, 1, 1, 128, 1};
  int rc = make_tmap_generic(&tmX, x, 5, dims, strides, box);
  if (rc) return rc;
  rc = make_tmap_rows2d(&tmW, w, D, (long long)l * D, 64);
  if (rc) return rc;
  const int stage = 128 * 128 + 64 * 128 * (D / 64);
  const int nst = 6;
  const int smem = nst * stage + 1024 + 256;
  auto kern = compress_fwd_tc_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const dim3 grid((Tc + 127) / 128, B * H);
  kern<<<grid, kThreads, smem, s>>>(tmX, tmW, bias, y, Tc, H, l, d, nst);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

// Equal-length fast path: x [B,T,H,D] with T a multiple of d and at least l.
int launch_compress_fwd_uniform(const bf16* x, const bf16* w, const bf16* bias, bf16* y, int B, int T, int H, int D, int l,
                                int d, cudaStream_t s) {
  if (D == 128) return launch<128>(x, w, bias, y, B, T, H, l, d, s);
  if (D == 64) return launch<64>(x, w, bias, y, B, T, H, l, d, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}
int compress_tc_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
