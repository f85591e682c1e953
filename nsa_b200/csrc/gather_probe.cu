// Measurement aid: the L2 -> shared-memory gather of selected 64-key K/V blocks with no arithmetic behind it.
//
// The selected-attention kernels (sel_block.cu) are bound by this gather: every (token, kv head) item brings in 32 KB
// of K and V per visited block for only 16 query rows.  This kernel visits the items and blocks in the same order
// and fetches the same TMA boxes, but nothing consumes them: every warp keeps a private ring of [64 x D] slots in
// flight and re-issues a slot as soon as its previous box has landed.  Its bytes per second are the ceiling the
// benchmark quotes for the gather path of those kernels (same box shapes, same issue pattern, all of shared memory
// in flight).  Reference access pattern: the block loop of parallel_nsa_fwd_kernel (nsa/selection_attn.py:447-482).
#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

constexpr int BS = 64;
constexpr int kWarps = 6;    // a warp's TMA instructions run one after another, so the ring is spread over six warps

template <int D>
__global__ void __launch_bounds__(kWarps * 32, 1)
    gather_probe_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const SelArgs a,
                        const int spw) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int NP = D / 64;
  constexpr uint32_t panel_bytes = BS * 128;
  constexpr uint32_t slot_bytes = panel_bytes * NP;
  const uint32_t bar_base = sbase + (uint32_t)(spw * kWarps) * slot_bytes;
  if (threadIdx.x == 0) {
    for (int i = 0; i < spw * kWarps; ++i) mbar_init(bar_base + 8u * i, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const int HG = a.Hq / 16;
  const int G16 = (a.Hq / a.Hkv) / 16;
  const long long total = (long long)a.B * a.Tq * HG;
  const long long step = (long long)gridDim.x * kWarps;
  int slot = 0;
  uint32_t issued = 0;          // boxes issued so far into this warp's ring
  bool ok = true;
  for (long long idx = (long long)blockIdx.x * kWarps + warp; ok && idx < total; idx += step) {
    const int hg = (int)(idx % HG);
    const int tl = a.Tq - 1 - (int)((idx / HG) % a.Tq);
    const int b = (int)(idx / ((long long)HG * a.Tq));
    const int t = a.q0 + tl, hkv = hg / G16;
    const long long row = ((long long)b * a.Tq + tl) * a.Hkv + hkv;
    int ent = -1;
    if (lane < a.S) {
      const long long v = a.idx64 ? reinterpret_cast<const long long*>(a.idx)[row * a.S + lane]
                                  : (long long)reinterpret_cast<const int*>(a.idx)[row * a.S + lane];
      if (v >= 0 && v * BS <= t) ent = (int)v;
    }
    unsigned mask = __ballot_sync(0xffffffffu, ent >= 0);
    while (ok && mask) {
      const int bit = __ffs(mask) - 1;
      mask &= mask - 1;
      const int blk = __shfl_sync(0xffffffffu, ent, bit);
      for (int kv = 0; kv < 2; ++kv) {
        const int s = warp * spw + slot;
        const uint32_t bar = bar_base + 8u * s, use = issued / (uint32_t)spw;
        int good = 1;
        if (lane == 0) {
          // the box issued into this slot one ring turn ago must have landed before the slot is overwritten
          if (use > 0) good = mbar_wait(bar, (use - 1) & 1, DEV_ERR_FULL_WAIT) ? 1 : 0;
          if (good) mbar_expect_tx(bar, slot_bytes);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
        if (lane < NP)
          tma_load_4d(sbase + s * slot_bytes + lane * panel_bytes, kv ? &tmV : &tmK, bar, lane * 64, hkv, blk * BS, b);
        ++issued;
        if (++slot == spw) slot = 0;
      }
    }
  }
  // drain: every box still in flight must land before the CTA (and its shared memory) goes away
  const uint32_t n_out = issued < (uint32_t)spw ? issued : (uint32_t)spw;
  if (lane == 0) {
    for (uint32_t i = 0; i < n_out; ++i) {
      const uint32_t j = issued - 1 - i;                 // the i-th most recent box
      const int s = warp * spw + (int)(j % (uint32_t)spw);
      mbar_wait(bar_base + 8u * s, (j / (uint32_t)spw) & 1, DEV_ERR_FULL_WAIT);
    }
  }
}

template <int D>
int launch(const SelArgs& a, cudaStream_t s) {
  CUtensorMap tmK, tmV;
  int rc = make_tmap_rows4d(&tmK, a.k, D, a.Hkv, a.T, a.B, BS);
  if (!rc) rc = make_tmap_rows4d(&tmV, a.v, D, a.Hkv, a.T, a.B, BS);
  if (rc) return rc;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const int slot_bytes = BS * D * 2;
  int spw = (max_smem - 2048) / slot_bytes / kWarps;
  if (spw > 2) spw = 2;
  if (spw < 1) {
    set_error("gather probe: not enough shared memory");
    return -30;
  }
  const int smem = spw * kWarps * slot_bytes + spw * kWarps * 8 + 1024 + 64;
  auto kern = gather_probe_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  const long long total = (long long)a.B * a.Tq * (a.Hq / 16);
  const long long ctas = (total + kWarps - 1) / kWarps;
  const int grid = (int)(ctas < num_sms() ? ctas : num_sms());
  if (grid <= 0) return 0;
  kern<<<grid, kWarps * 32, smem, s>>>(tmK, tmV, a, spw);
  note_launches(1);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_gather_probe(const SelArgs& a, int D, cudaStream_t s) {
  if (a.BS != BS || a.S > 32) {
    set_error("gather probe: 64-key blocks and at most 32 selections per query");
    return -9;
  }
  if (D == 128) return launch<128>(a, s);
  if (D == 64) return launch<64>(a, s);
  set_error("head_dim %d not supported (64 or 128)", D);
  return -2;
}
int gather_probe_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
