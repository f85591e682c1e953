// K/V block compression: y[i] = bias + sum_{j<l} x[i*d + j] . W_j  over overlapping windows (block l, stride d),
// forward and backward.
//
// Reference behaviour: _compress_fwd / _compress_bwd_dw / _compress_bwd_dx (nsa/compression_kv.py:21-171) for the
// functional path (weight [l*D, D], no bias, varlen through cu_seq_len) and nn.Conv1d(D, D, l, stride=d) of
// KVCompressor (nsa/compression_kv.py:292-312) for the module path (same contraction plus bias; the caller passes the
// Conv1d weight permuted to [l*D, D]).  The reference's backward uses fp32 atomics into dX and dW; here
//   * dX: a token belongs to exactly l/d windows, so dX[tok] = sum_r dY[tok/d - r] . W_{tok%d + r*d}^T is a plain
//     GEMM with one writer per output element;
//   * dW: split over (sequence, head) into fp32 partials that a second kernel adds in a fixed order.
//
// These three GEMMs are 0.1 TFLOP of the 13 TFLOP step; they run on mma.sync tiles fed by cp.async double buffering.
#include <mutex>

#include "kernels.h"
#include "tmap.h"

namespace nsa {

namespace {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A-fragments of A[m][k] = Tile[k][m] (the tile holds the operand transposed): 16 m-columns starting at chunk
// `mchunk` (units of 8 columns), 16 k-rows starting at k0.
__device__ __forceinline__ void load_a_frag_trans(uint32_t (&af)[4], uint32_t base, uint32_t panel_bytes, int k0,
                                                  int mchunk, int lane) {
  const int mi = lane >> 3, rr = lane & 7;
  ldsm_x4_t(tile_addr(base, panel_bytes, k0 + (mi >> 1) * 8 + rr, mchunk + (mi & 1)), af[0], af[1], af[2], af[3]);
}

// ---------------------------------------------------------------------------------------------------------------
// forward: tile = 64 output rows x D columns; K loop over (j, 64-channel chunk)
// ---------------------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) compress_fwd_kernel(const CompressArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  constexpr uint32_t A_BYTES = 64 * 128;            // [64 rows][64 k]
  constexpr uint32_t W_PANEL = 64 * 128;            // [64 k][64 n] per panel
  constexpr uint32_t W_BYTES = W_PANEL * (D / 64);
  constexpr uint32_t STAGE = A_BYTES + W_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int in0 = a.cu_in[seq], n_ctx = a.cu_in[seq + 1] - in0;
  const int out0 = a.cu_out[seq], n_out = a.cu_out[seq + 1] - out0;
  const int i0 = blockIdx.x * 64;
  if (i0 >= n_out) return;
  const int nk = a.l * D / 64;

  auto load_stage = [&](int kk, int st) {
    const uint32_t ab = sbase + st * STAGE, wb = ab + A_BYTES;
    const int j = (kk * 64) / D, c0 = (kk * 64) % D;
    // A: 64 rows x 8 chunks
    for (int e = threadIdx.x; e < 64 * 8; e += 128) {
      const int r = e >> 3, c = e & 7;
      const int i = i0 + r;
      const bool ok = i < n_out && (i * a.d + j) < n_ctx;
      const bf16* src = a.x + (((long long)in0 + (ok ? i * a.d + j : 0)) * a.H + h) * D + c0 + c * 8;
      cp_async16(tile_addr(ab, A_BYTES, r, c), src, ok);
    }
    // W rows kk*64 .. +64, all D columns
    for (int e = threadIdx.x; e < 64 * (D / 8); e += 128) {
      const int r = e / (D / 8), c = e % (D / 8);
      const bf16* src = a.w + ((long long)kk * 64 + r) * D + c * 8;
      cp_async16(tile_addr(wb, W_PANEL, r, c), src, true);
    }
    cp_async_commit();
  };

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  load_stage(0, 0);
  for (int kk = 0; kk < nk; ++kk) {
    if (kk + 1 < nk) {
      load_stage(kk + 1, (kk + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t ab = sbase + (kk & 1) * STAGE, wb = ab + A_BYTES;
    uint32_t af[4][4];
    load_a_frags<64>(af, ab, A_BYTES, warp * 16, lane);
    mma_a_b<D, 64>(acc, af, wb, W_PANEL, 0, lane);
    __syncthreads();
  }
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int i = i0 + warp * 16 + g + hr * 8;
    if (i >= n_out) continue;
    bf16* dst = a.y + (((long long)out0 + i) * a.H + h) * D + 2 * tq;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      float x0 = acc[n][2 * hr], x1 = acc[n][2 * hr + 1];
      if (a.bias) {
        x0 += __bfloat162float(a.bias[n * 8 + 2 * tq]);
        x1 += __bfloat162float(a.bias[n * 8 + 2 * tq + 1]);
      }
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(x0, x1);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dX: grid (chunk tiles, seq*H, d).  Tile = 64 stride-chunks u x D channels for one in-chunk offset jj.
// dX[u*d + jj, c] = sum_r sum_o dY[u - r, o] * W[(jj + r*d)*D + c, o]
// ---------------------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) compress_dx_kernel(const CompressArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  constexpr uint32_t A_BYTES = 64 * 128;   // dY tile [64 u][64 o]
  constexpr uint32_t W_BYTES = D * 128;    // W tile  [D c][64 o]
  constexpr uint32_t STAGE = A_BYTES + W_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.y / a.H, h = blockIdx.y % a.H;
  const int jj = blockIdx.z;
  const int in0 = a.cu_in[seq], n_ctx = a.cu_in[seq + 1] - in0;
  const int out0 = a.cu_out[seq], n_out = a.cu_out[seq + 1] - out0;
  const int u0 = blockIdx.x * 64;
  if (u0 * a.d >= n_ctx) return;
  const int R = a.l / a.d;
  const int nk = R * (D / 64);

  auto load_stage = [&](int kk, int st) {
    const uint32_t ab = sbase + st * STAGE, wb = ab + A_BYTES;
    const int r = kk / (D / 64), o0 = (kk % (D / 64)) * 64;
    for (int e = threadIdx.x; e < 64 * 8; e += 128) {
      const int row = e >> 3, c = e & 7;
      const int i = u0 + row - r;
      const bool ok = i >= 0 && i < n_out;
      const bf16* src = a.dy + (((long long)out0 + (ok ? i : 0)) * a.H + h) * D + o0 + c * 8;
      cp_async16(tile_addr(ab, A_BYTES, row, c), src, ok);
    }
    for (int e = threadIdx.x; e < D * 8; e += 128) {
      const int row = e >> 3, c = e & 7;   // row = channel c_in
      const bf16* src = a.w + ((long long)(jj + r * a.d) * D + row) * D + o0 + c * 8;
      cp_async16(tile_addr(wb, W_BYTES, row, c), src, true);
    }
    cp_async_commit();
  };

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  load_stage(0, 0);
  for (int kk = 0; kk < nk; ++kk) {
    if (kk + 1 < nk) {
      load_stage(kk + 1, (kk + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t ab = sbase + (kk & 1) * STAGE, wb = ab + A_BYTES;
    uint32_t af[4][4];
    load_a_frags<64>(af, ab, A_BYTES, warp * 16, lane);
    mma_a_bt<64, D>(acc, af, wb, W_BYTES, 0, lane);
    __syncthreads();
  }
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int tok = (u0 + warp * 16 + g + hr * 8) * a.d + jj;
    if (tok >= n_ctx) continue;
    bf16* dst = a.dx + (((long long)in0 + tok) * a.H + h) * D + 2 * tq;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(acc[n][2 * hr], acc[n][2 * hr + 1]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dW partials: grid (l, nsplit).  CTA (j, split) accumulates sum over its (seq, head) pairs of X_j^T . dY.
// ---------------------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(D * 2) compress_dw_kernel(const CompressArgs a, int nsplit) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  constexpr uint32_t PANEL = 64 * 128;
  constexpr uint32_t T_BYTES = PANEL * (D / 64);   // [64 i][D]
  constexpr uint32_t STAGE = 2 * T_BYTES;
  constexpr int NT = D * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;   // warp owns channels [16*warp, +16)
  const int j = blockIdx.x, split = blockIdx.y;

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  for (int bh = split; bh < a.nseq * a.H; bh += nsplit) {
    const int seq = bh / a.H, h = bh % a.H;
    const int in0 = a.cu_in[seq], n_ctx = a.cu_in[seq + 1] - in0;
    const int out0 = a.cu_out[seq], n_out = a.cu_out[seq + 1] - out0;
    const int nk = (n_out + 63) / 64;
    auto load_stage = [&](int kk, int st) {
      const uint32_t xb = sbase + st * STAGE, yb = xb + T_BYTES;
      for (int e = threadIdx.x; e < 64 * (D / 8); e += NT) {
        const int r = e / (D / 8), c = e % (D / 8);
        const int i = kk * 64 + r;
        const bool ok = i < n_out && (i * a.d + j) < n_ctx;
        const bf16* sx = a.x + (((long long)in0 + (ok ? i * a.d + j : 0)) * a.H + h) * D + c * 8;
        const bf16* sy = a.dy + (((long long)out0 + (ok ? i : 0)) * a.H + h) * D + c * 8;
        cp_async16(tile_addr(xb, PANEL, r, c), sx, ok);
        cp_async16(tile_addr(yb, PANEL, r, c), sy, ok);
      }
      cp_async_commit();
    };
    if (nk > 0) load_stage(0, 0);
    for (int kk = 0; kk < nk; ++kk) {
      if (kk + 1 < nk) {
        load_stage(kk + 1, (kk + 1) & 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const uint32_t xb = sbase + (kk & 1) * STAGE, yb = xb + T_BYTES;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t pf[1][4];
        load_a_frag_trans(pf[0], xb, PANEL, ks * 16, warp * 2, lane);
        mma_a_b<D, 16>(acc, pf, yb, PANEL, ks * 16, lane);
      }
      __syncthreads();
    }
  }
  const int g = lane >> 2, tq = lane & 3;
  float* dst = a.ws + ((long long)split * a.l + j) * D * D;
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int c = warp * 16 + g + hr * 8;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<float2*>(dst + (long long)c * D + n * 8 + 2 * tq) = make_float2(acc[n][2 * hr], acc[n][2 * hr + 1]);
  }
}

__global__ void compress_dw_reduce_kernel(const float* __restrict__ ws, float* __restrict__ dw, long long n, int nsplit) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int k = 0; k < nsplit; ++k) s += ws[(long long)k * n + i];
  dw[i] = s;
}

// dbias[o] = sum over all output rows of dY[row, o]; one CTA, fixed order.  A thread owns 8 channels (one 16-byte
// load per row) of every (blockDim / (D/8))-th row and keeps eight loads in flight.
__global__ void compress_dbias_kernel(const bf16* __restrict__ dy, float* __restrict__ dbias, long long rows, int D) {
  extern __shared__ float red[];   // [nr][D]
  const int cpr = D / 8;           // 16-byte chunks per row
  const int cc = threadIdx.x % cpr, rl = threadIdx.x / cpr, nr = blockDim.x / cpr;
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  constexpr int U = 8;
  for (long long r0 = rl; r0 < rows; r0 += (long long)nr * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long r = r0 + (long long)u * nr;
      v[u] = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows) v[u] = *reinterpret_cast<const uint4*>(dy + r * D + cc * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        s[2 * k] += f.x;
        s[2 * k + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl * D + cc * 8 + k] = s[k];
  __syncthreads();
  if (threadIdx.x < D) {
    float t = 0.f;
    for (int k = 0; k < nr; ++k) t += red[k * D + threadIdx.x];
    dbias[threadIdx.x] = t;
  }
}

constexpr int kDwSplit = 32;

template <int D>
int fwd(const CompressArgs& a, cudaStream_t s) {
  const int smem = 2 * (64 * 128 + 64 * 128 * (D / 64)) + 1024;
  auto kern = compress_fwd_kernel<D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  if (a.max_out <= 0) return 0;
  const dim3 grid((a.max_out + 63) / 64, a.nseq * a.H);
  kern<<<grid, 128, smem, s>>>(a);
  note_launches(1);
  return (int)cudaGetLastError();
}

// dX, dW (fp32 partials in a.ws, `nsplit` of them, then a fixed-order reduction) and dbias.  Shared by the entry point
// that takes a caller workspace and the one that uses the library's fixed array.
template <int D>
int bwd_common(const CompressArgs& a, int nsplit, cudaStream_t s) {
  cudaError_t e;
  if (a.dx) {
    const int smem = 2 * (64 * 128 + D * 128) + 1024;
    auto kern = compress_dx_kernel<D>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    const int nchunk = (a.max_in + a.d - 1) / a.d;
    const dim3 grid((nchunk + 63) / 64, a.nseq * a.H, a.d);
    if (a.max_in > 0) {
      kern<<<grid, 128, smem, s>>>(a);
      note_launches(1);
    }
  }
  if (a.dw) {
    const int smem = 2 * 2 * 64 * 128 * (D / 64) + 1024;
    auto kern = compress_dw_kernel<D>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    // every (j, split) CTA overwrites its whole [D x D] partial, so nothing in the workspace needs clearing
    kern<<<dim3(a.l, (unsigned)nsplit), D * 2, smem, s>>>(a, nsplit);
    const long long n = (long long)a.l * D * D;
    compress_dw_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a.ws, a.dw, n, nsplit);
    note_launches(2);
  }
  if (a.dbias) {
    const int nt = 1024, nr = nt / (D / 8);
    cudaFuncSetAttribute(compress_dbias_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, nr * D * (int)sizeof(float));
    compress_dbias_kernel<<<1, nt, nr * D * sizeof(float), s>>>(a.dy, a.dbias, (long long)a.total_out * a.H, D);
    note_launches(1);
  }
  return (int)cudaGetLastError();
}

template <int D>
int bwd(const CompressArgs& a, cudaStream_t s) {
  return bwd_common<D>(a, a.nseq * a.H < kDwSplit ? a.nseq * a.H : kDwSplit, s);
}


// ---------------------------------------------------------------------------------------------------------------
// Allocation-free weight-gradient path.
//
// Some hosts of this library may not allocate device memory at the point where they need the compression
// backward: an inference/training runtime that hands out all of its HBM at start-up and forbids cudaMalloc
// afterwards, or a plugin sandbox whose allocator the library must not touch.  For them the fp32 partials of the
// dW reduction live in this fixed array instead of a caller workspace.  Every GPU that loads the library holds the
// 16 MiB until the process exits.
// ---------------------------------------------------------------------------------------------------------------
constexpr long long kStaticScratchFloats = 4ll * 1024 * 1024;   // 16 MiB
static __device__ __align__(256) float g_dw_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_scratch_ptr[kMaxDevices] = {};
static std::mutex g_scratch_mutex;

// Device address of g_dw_scratch on the current device.  In host code the symbol's name is only a handle, so the
// address is queried once per device (with that device current) and cached.
static int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device ordinal %d outside the supported range", dev);
    return -40;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_dw_scratch);
    if (e != cudaSuccess) {
      set_error("cudaGetSymbolAddress for the static scratch failed: %s", cudaGetErrorString(e));
      return (int)e;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

template <int D>
int bwd_static(const CompressArgs& a0, cudaStream_t s) {
  CompressArgs a = a0;
  long long nsplit = 1;
  if (a.dw) {
    const long long per_split = (long long)a.l * D * D;
    nsplit = kStaticScratchFloats / per_split;          // >= 1, checked by the caller
    if (nsplit > (long long)a.nseq * a.H) nsplit = (long long)a.nseq * a.H;
    if (nsplit > kDwSplit) nsplit = kDwSplit;
    float* scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc) return rc;
    a.ws = scratch;
  }
  return bwd_common<D>(a, (int)nsplit, s);
}

}  // namespace

int launch_compress_fwd(const CompressArgs& a, cudaStream_t s) {
  if (a.D == 128) return fwd<128>(a, s);
  if (a.D == 64) return fwd<64>(a, s);
  set_error("head_dim %d not supported (64 or 128)", a.D);
  return -2;
}
int launch_compress_bwd(const CompressArgs& a, cudaStream_t s) {
  if (a.D == 128) return bwd<128>(a, s);
  if (a.D == 64) return bwd<64>(a, s);
  set_error("head_dim %d not supported (64 or 128)", a.D);
  return -2;
}
long long compress_static_scratch_floats() { return kStaticScratchFloats; }
int launch_compress_bwd_static(const CompressArgs& a, cudaStream_t s) {
  if (a.D == 128) return bwd_static<128>(a, s);
  if (a.D == 64) return bwd_static<64>(a, s);
  set_error("head_dim %d not supported (64 or 128)", a.D);
  return -2;
}
int compress_status(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_dev_error, sizeof(int));
  if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(int));
  return (int)e;
}

}  // namespace nsa
