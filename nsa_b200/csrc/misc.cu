// Small memory-bound helpers: row dot products for the backward (delta and gate gradients), the gated
// combine of the three branches, the reverse index of the block selection, and the fixed-order reduction
// of the compressed branch's dCK/dCV partials.
#include "kernels.h"
#include "tmap.h"

namespace nsa {

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

namespace {

// ---- delta / gate gradient ------------------------------------------------------------------------
// Reference: parallel_nsa_bwd_kernel_preprocess (nsa/selection_attn.py:520-530), _attn_bwd_preprocess
// (nsa/triton_attention.py:184-199) and the autograd of the gate products (nsa/nsa.py:133,
// nsa/selection_attn.py:808-811).  One warp per (token, head) row.
template <int D>
__global__ void rowdot_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, const bf16* __restrict__ gate,
                              float* __restrict__ delta, bf16* __restrict__ dgate, long long rows) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  constexpr int PER = D / 32;  // 2 or 4 elements per lane
  float acc = 0.f;
  const bf16* po = o + row * D + lane * PER;
  const bf16* pd = dout + row * D + lane * PER;
#pragma unroll
  for (int i = 0; i < PER; i += 2) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + i));
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    if (delta) delta[row] = gate ? acc * __bfloat162float(gate[row]) : acc;
    if (dgate) dgate[row] = __float2bfloat16(acc);
  }
}

// ---- gated combine ------------------------------------------------------------------------------------
// o = g0*a0 + g1*a1 + g2*a2  (nsa/selection_attn.py:808-811 and nsa/nsa.py:133, as one pass)
__global__ void combine_kernel(const bf16* __restrict__ a0, const bf16* __restrict__ g0, const bf16* __restrict__ a1,
                               const bf16* __restrict__ g1, const bf16* __restrict__ a2, const bf16* __restrict__ g2,
                               bf16* __restrict__ o, long long n8, int D8) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const long long row = i / D8;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  auto add = [&](const bf16* a, const bf16* gp) {
    if (!a) return;
    const float gv = gp ? __bfloat162float(gp[row]) : 1.f;
    const uint4 v = *reinterpret_cast<const uint4*>(a + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      acc[2 * k] += gv * f.x;
      acc[2 * k + 1] += gv * f.y;
    }
  };
  add(a0, g0);
  add(a1, g1);
  add(a2, g2);
  uint4 out;
  __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int k = 0; k < 4; ++k) ho[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
  *reinterpret_cast<uint4*>(o + i * 8) = out;
}

// ---- reverse index of the selection -----------------------------------------------------------------
// Replaces the dense boolean block mask of parallel_nsa_kernel_mask (nsa/selection_attn.py:256-273).
// A stable counting sort by block id in three launches; the order inside every list is ascending in t and
// independent of scheduling, so the backward is bit-reproducible.
// grid (NB chunks, B*H): histogram of the block ids selected by the BS tokens of one chunk
__global__ void rev_hist_kernel(const RevArgs a) {
  extern __shared__ int sh[];
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  for (int i = threadIdx.x; i < a.NB; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int n = a.BS * a.S;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int tl = chunk * a.BS + e / a.S, s = e % a.S;
    if (tl >= a.Tq) continue;
    const int blk = rev_block(a, ((long long)b * a.Tq + tl) * a.H + h, s, a.q0 + tl);
    if (blk >= 0) atomicAdd(&sh[blk], 1);
  }
  __syncthreads();
  int* out = a.hist + ((long long)bh * gridDim.x + chunk) * a.NB;
  for (int i = threadIdx.x; i < a.NB; i += blockDim.x) out[i] = sh[i];
}

// grid (B*H): per block id, exclusive prefix over chunks (in place) and the CSR row pointers
__global__ void rev_scan_kernel(const RevArgs a, const int nchunk) {
  extern __shared__ int tot[];
  const int bh = blockIdx.x;
  int* hist = a.hist + (long long)bh * nchunk * a.NB;
  for (int blk = threadIdx.x; blk < a.NB; blk += blockDim.x) {
    int run = 0;
    for (int c = 0; c < nchunk; ++c) {
      const int v = hist[(long long)c * a.NB + blk];
      hist[(long long)c * a.NB + blk] = run;
      run += v;
    }
    tot[blk] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int* rp = a.rev_ptr + (long long)bh * (a.NB + 1);
    int run = 0;
    for (int blk = 0; blk < a.NB; ++blk) {
      rp[blk] = run;
      run += tot[blk];
    }
    rp[a.NB] = run;
  }
}

// grid (NB chunks, B*H), one warp: write the tokens of the chunk, in order, behind each block's cursor
__global__ void rev_fill_kernel(const RevArgs a) {
  extern __shared__ int cur[];
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int lane = threadIdx.x;
  const int* rp = a.rev_ptr + (long long)bh * (a.NB + 1);
  const int* pre = a.hist + ((long long)bh * gridDim.x + chunk) * a.NB;
  for (int i = lane; i < a.NB; i += 32) cur[i] = rp[i] + pre[i];
  __syncwarp();
  int* out = a.rev_tok + (long long)bh * a.cap;
  for (int tt = 0; tt < a.BS; ++tt) {
    const int tl = chunk * a.BS + tt;
    if (tl >= a.Tq) break;
    const int t = a.q0 + tl;   // lists hold sequence positions
    const long long row = ((long long)b * a.Tq + tl) * a.H + h;
    for (int s0 = 0; s0 < a.S; s0 += 32) {
      const int s = s0 + lane;
      const int blk = (s < a.S) ? rev_block(a, row, s, t) : -1;
      const int key = blk >= 0 ? blk : -1 - lane;  // invalid lanes never match each other
      const unsigned same = __match_any_sync(0xffffffffu, key);
      if (blk >= 0) {
        const int rank = __popc(same & ((1u << lane) - 1));
        const int pos = cur[blk] + rank;
        if (pos < a.cap) {
          out[pos] = t;
          if (a.inv) a.inv[row * a.S + s] = pos;
        }
      }
      __syncwarp();
      if (blk >= 0 && (lane == 31 || (same >> (lane + 1)) == 0)) cur[blk] += __popc(same);  // highest lane of the group
      __syncwarp();
    }
  }
}

// ---- fixed-order reduction of segment partials ----------------------------------------------------------
__global__ void reduce_segments_kernel(const float* __restrict__ part, bf16* __restrict__ out, int nseg,
                                       long long n_per_seg, int q0, int Tq, int Lk, int HkD, int seg_len, int cblock,
                                       int cstride, int causal) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= n_per_seg) return;
  const int j = (int)((i / HkD) % Lk);
  const int first = causal ? (j / 64) * 64 * cstride + cblock : 0;
  float x = 0.f, y = 0.f;
  for (int seg = 0; seg < nseg; ++seg) {
    const int lo = max(first, q0 + seg * seg_len), hi = min(q0 + Tq, q0 + (seg + 1) * seg_len);
    if (hi <= lo) continue;
    const float2 v = *reinterpret_cast<const float2*>(part + (long long)seg * n_per_seg + i);
    x += v.x;
    y += v.y;
  }
  *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(x, y);
}

}  // namespace

int launch_rowdot(const bf16* o, const bf16* dout, const bf16* gate, float* delta, bf16* dgate, long long rows, int D,
                  cudaStream_t s) {
  if (rows <= 0) return 0;
  const int wpb = 8;
  const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
  if (D == 128)
    rowdot_kernel<128><<<grid, wpb * 32, 0, s>>>(o, dout, gate, delta, dgate, rows);
  else if (D == 64)
    rowdot_kernel<64><<<grid, wpb * 32, 0, s>>>(o, dout, gate, delta, dgate, rows);
  else {
    set_error("head_dim %d not supported (64 or 128)", D);
    return -2;
  }
  note_launches(1);
  return (int)cudaGetLastError();
}

int launch_combine(const bf16* a0, const bf16* g0, const bf16* a1, const bf16* g1, const bf16* a2, const bf16* g2,
                   bf16* o, long long rows, int D, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (D % 8) {
    set_error("head_dim must be a multiple of 8");
    return -2;
  }
  const long long n8 = rows * (D / 8);
  combine_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, s>>>(a0, g0, a1, g1, a2, g2, o, n8, D / 8);
  note_launches(1);
  return (int)cudaGetLastError();
}

// Two warps per (batch, token, 16-head group), each half of the [16 x D] bf16 tile (heads 0-7 / 8-15): the token's
// visits are added in slot order.  A load instruction of the warp covers 512 contiguous bytes; the list positions of
// all slots are fetched first so that the tiles of several slots are in flight at once.
template <int D>
__global__ void __launch_bounds__(256) sel_dq_reduce_kernel(const RevArgs a, const bf16* __restrict__ part, bf16* __restrict__ dq,
                                                            const int G16, const float scale, const int accumulate) {
  const long long w2 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const long long total = (long long)a.B * a.Tq * a.H * G16;
  const long long w = w2 >> 1;
  if (w >= total) return;
  const int hb = (int)(w2 & 1);                        // which half of the tile
  const int lane = threadIdx.x & 31;
  const int sub = (int)(w % G16);
  const long long row = w / G16;                       // (b, tl, h) row of idx / counts
  const int h = (int)(row % a.H);
  const long long bt = row / a.H;
  const int tl = (int)(bt % a.Tq), b = (int)(bt / a.Tq);
  const int t = a.q0 + tl;
  constexpr int NV = 8 * D / 8 / 32;                   // 16-byte vectors per lane: 4 at D = 128
  float acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
  const long long bh = (long long)b * a.H + h;
  // lane s holds the list position of slot s (or -1): the same validity rule that built the lists
  int mypos = -1;
  if (lane < a.S && rev_block(a, row, lane, t) >= 0) mypos = a.inv[row * a.S + lane];
  unsigned live = __ballot_sync(0xffffffffu, mypos >= 0);
  const uint4* base = reinterpret_cast<const uint4*>(part) + hb * (8 * D / 8) + lane;
  auto tile = [&](int s) {
    const long long pos = __shfl_sync(0xffffffffu, mypos, s);
    return base + ((bh * a.cap + pos) * G16 + sub) * (16 * D / 8);
  };
  auto add = [&](const uint4 (&v)[NV]) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(hv[k]);
        acc[i][2 * k] += f.x;
        acc[i][2 * k + 1] += f.y;
      }
    }
  };
  while (live) {
    const int s0 = __ffs(live) - 1;
    live &= live - 1;
    const int s1 = live ? __ffs(live) - 1 : -1;
    if (s1 >= 0) live &= live - 1;
    const uint4* p0 = tile(s0);
    const uint4* p1 = tile(s1 >= 0 ? s1 : s0);
    uint4 v0[NV], v1[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) v0[i] = __ldcs(p0 + 32 * i);
    if (s1 >= 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) v1[i] = __ldcs(p1 + 32 * i);
    }
    add(v0);
    if (s1 >= 0) add(v1);
  }
  const int Hq = a.H * G16 * 16;
  // the partial tiles keep the staging layout of the kernel that wrote them: within a 128-byte half row the 16-byte
  // chunk c sits at position c ^ (head & 7).  All tiles share it, so the sum is formed in place and undone here:
  // vector u = 32 i + lane of this half tile is row u / 16, position u % 8.
  uint4* dst = reinterpret_cast<uint4*>(dq + ((bt * Hq) + (long long)(h * G16 + sub) * 16) * D) + hb * (8 * D / 8);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float prev[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int u = 32 * i + lane;
    const int ud = (u & ~7) | ((u & 7) ^ ((u >> 4) & 7));
    if (accumulate) {
      const uint4 v = dst[ud];
      const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(hv[k]);
        prev[2 * k] = f.x;
        prev[2 * k + 1] = f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      ho[k] = __floats2bfloat162_rn(fmaf(acc[i][2 * k], scale, prev[2 * k]), fmaf(acc[i][2 * k + 1], scale, prev[2 * k + 1]));
    dst[ud] = o;
  }
}

int launch_sel_dq_reduce(const RevArgs& a, const bf16* part, bf16* dq, int Hq, int D, float scale, int accumulate,
                         cudaStream_t s) {
  if (D != 128) {
    set_error("selected dQ reduction: head_dim 128 only");
    return -2;
  }
  const int G16 = Hq / a.H / 16;
  const long long total = (long long)a.B * a.Tq * a.H * G16;
  if (total <= 0) return 0;
  if (a.S > 32) {
    set_error("selected dQ reduction: at most 32 selected blocks per token");
    return -2;
  }
  sel_dq_reduce_kernel<128><<<(unsigned)((2 * total + 7) / 8), 256, 0, s>>>(a, part, dq, G16, scale, accumulate);
  note_launches(1);
  return (int)cudaGetLastError();
}

int launch_build_rev(const RevArgs& a, cudaStream_t s) {
  if (a.B <= 0 || a.T <= 0) return 0;
  if ((size_t)a.NB * 4 > 200 * 1024) {
    set_error("reverse index: too many selection blocks (%d)", a.NB);
    return -34;
  }
  const int nchunk = (a.Tq + a.BS - 1) / a.BS;   // chunks of BS local tokens
  const dim3 grid(nchunk, a.B * a.H);
  const size_t sm = (size_t)a.NB * 4;
  if (sm > 48 * 1024) {
    cudaFuncSetAttribute(rev_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    cudaFuncSetAttribute(rev_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    cudaFuncSetAttribute(rev_fill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  }
  rev_hist_kernel<<<grid, 128, sm, s>>>(a);
  rev_scan_kernel<<<a.B * a.H, 256, sm, s>>>(a, nchunk);
  rev_fill_kernel<<<grid, 32, sm, s>>>(a);
  note_launches(3);
  return (int)cudaGetLastError();
}

int launch_reduce_segments(const float* part, bf16* out, int nseg, long long n_per_seg, int q0, int Tq, int Lk, int Hk,
                           int D, int seg_len, int cblock, int cstride, int causal, cudaStream_t s) {
  if (n_per_seg <= 0) return 0;
  const long long pairs = n_per_seg / 2;
  reduce_segments_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, s>>>(part, out, nseg, n_per_seg, q0, Tq, Lk, Hk * D,
                                                                          seg_len, cblock, cstride, causal);
  note_launches(1);
  return (int)cudaGetLastError();
}

int misc_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
