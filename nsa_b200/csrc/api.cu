// The C ABI of libnsa_b200.so (declared in include/nsa_b200.h): argument checks, workspace carving and kernel
// launches.  No torch types, no allocation, no synchronisation except nsa_device_status().
#include <stdarg.h>
#include <stdio.h>

#include "../../include/nsa_b200.h"
#include "kernels.h"
#include "tmap.h"

namespace nsa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_attn_shape(const char* who, int B, int T, int Hq, int Hk, int D) {
  if (B <= 0 || T <= 0 || Hq <= 0 || Hk <= 0) return fail(-1, "%s: empty or negative shape", who);
  if (D != 64 && D != 128) return fail(-2, "%s: head_dim %d not supported (64 or 128)", who, D);
  if (Hq % Hk != 0 || (Hq / Hk) % 16 != 0)
    return fail(-3, "%s: query heads per KV head must be a multiple of 16 (Hq=%d, Hkv=%d)", who, Hq, Hk);
  return 0;
}

static int cmp_segments(int T, int* seg_len) {
  int nseg = (T + 1023) / 1024;
  if (nseg > 16) nseg = 16;
  if (nseg < 1) nseg = 1;
  int sl = (T + nseg - 1) / nseg;
  sl = (sl + 63) / 64 * 64;
  *seg_len = sl;
  return (T + sl - 1) / sl;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace nsa

using namespace nsa;

extern "C" {

int nsa_abi_version(void) { return 1; }

long long nsa_kernel_launch_count(void) { return launch_count(); }

const char* nsa_last_error(void) { return g_err; }

int nsa_device_status(void) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(1000 + (int)e, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  int worst = 0, v = 0;
  int (*fns[])(int*) = {sel_status, sel_block_status, dense_status, kv_status, compress_status, misc_status, compress_tc_status, kv_tc_status, dense_dq_tc_status, gather_probe_status, dense_tc2_status, decode_status, sel_fwd_kv_status};
  for (auto f : fns) {
    v = 0;
    const int rc = f(&v);
    if (rc) return fail(1000 + rc, "reading the device status failed: %s", cudaGetErrorString((cudaError_t)rc));
    if (v && !worst) worst = v;
  }
  if (worst) fail(worst, "a kernel gave up waiting on its pipeline (code %d)", worst);
  return worst;
}

int nsa_pool_out_len(int n, int k, int s, int p) {
  if (n <= 0 || k <= 0 || s <= 0) return 0;
  const int num = n + 2 * p - k;
  int out = (num >= 0 ? (num + s - 1) / s : -((-num) / s)) + 1;
  if ((out - 1) * s >= n + p) --out;
  return out < 0 ? 0 : out;
}

// ---- compression ------------------------------------------------------------------------------------
int nsa_compress_fwd(const void* x, const void* w, const void* bias, void* y, const int32_t* cu_in,
                     const int32_t* cu_out, int nseq, int H, int D, int block, int stride, int max_out,
                     void* stream) {
  if (!x || !w || !y || !cu_in || !cu_out) return fail(-1, "nsa_compress_fwd: null pointer");
  if (nseq <= 0 || H <= 0) return fail(-1, "nsa_compress_fwd: empty shape");
  if (stride <= 0 || block <= 0 || block % stride) return fail(-4, "nsa_compress_fwd: block must be a multiple of stride");
  if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return fail(-5, "nsa_compress_fwd: pointers must be 16-byte aligned");
  CompressArgs a = {};
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.bias = (const bf16*)bias; a.y = (bf16*)y;
  a.cu_in = cu_in; a.cu_out = cu_out; a.nseq = nseq; a.H = H; a.D = D; a.l = block; a.d = stride; a.max_out = max_out;
  return launch_compress_fwd(a, (cudaStream_t)stream);
}

int nsa_compress_fwd_uniform(const void* x, const void* w, const void* bias, void* y, int B, int T, int H, int D,
                             int block, int stride, void* stream) {
  if (!x || !w || !y) return fail(-1, "nsa_compress_fwd_uniform: null pointer");
  if (B <= 0 || H <= 0) return fail(-1, "nsa_compress_fwd_uniform: empty shape");
  if (stride <= 0 || block <= 0 || block % stride) return fail(-4, "nsa_compress_fwd_uniform: block must be a multiple of stride");
  if (T < block || T % stride) return fail(-10, "nsa_compress_fwd_uniform: T must be a multiple of stride and at least block");
  if (stride > 256) return fail(-10, "nsa_compress_fwd_uniform: stride too large for a TMA box");
  return launch_compress_fwd_uniform((const bf16*)x, (const bf16*)w, (const bf16*)bias, (bf16*)y, B, T, H, D, block, stride,
                                     (cudaStream_t)stream);
}

size_t nsa_compress_bwd_workspace_bytes(int nseq, int H, int D, int block) {
  long long split = (long long)nseq * H;
  if (split > 32) split = 32;
  return (size_t)split * block * D * D * sizeof(float);
}

int nsa_compress_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, float* dbias, void* ws,
                     size_t ws_bytes, const int32_t* cu_in, const int32_t* cu_out, int nseq, int H, int D, int block,
                     int stride, int max_in, int total_out, void* stream) {
  if (!x || !w || !dy || !cu_in || !cu_out) return fail(-1, "nsa_compress_bwd: null pointer");
  if (nseq <= 0 || H <= 0) return fail(-1, "nsa_compress_bwd: empty shape");
  if (D != 64 && D != 128) return fail(-2, "nsa_compress_bwd: head_dim %d not supported (64 or 128)", D);
  if (stride <= 0 || block <= 0 || block % stride) return fail(-4, "nsa_compress_bwd: block must be a multiple of stride");
  if (dw && (!ws || ws_bytes < nsa_compress_bwd_workspace_bytes(nseq, H, D, block)))
    return fail(-6, "nsa_compress_bwd: workspace too small");
  CompressArgs a = {};
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.dy = (const bf16*)dy; a.dx = (bf16*)dx; a.dw = dw; a.dbias = dbias;
  a.ws = (float*)ws; a.cu_in = cu_in; a.cu_out = cu_out; a.nseq = nseq; a.H = H; a.D = D; a.l = block; a.d = stride;
  a.max_in = max_in; a.total_out = total_out;
  return launch_compress_bwd(a, (cudaStream_t)stream);
}

int nsa_compress_bwd_noalloc(const void* x, const void* w, const void* dy, void* dx, float* dw, float* dbias,
                             const int32_t* cu_in, const int32_t* cu_out, int nseq, int H, int D, int block, int stride,
                             int max_in, int total_out, void* stream) {
  if (!x || !w || !dy || !cu_in || !cu_out) return fail(-1, "nsa_compress_bwd_noalloc: null pointer");
  if (nseq <= 0 || H <= 0) return fail(-1, "nsa_compress_bwd_noalloc: empty shape");
  if (D != 64 && D != 128) return fail(-2, "nsa_compress_bwd_noalloc: head_dim %d not supported (64 or 128)", D);
  if (stride <= 0 || block <= 0 || block % stride)
    return fail(-4, "nsa_compress_bwd_noalloc: block must be a multiple of stride");
  if (dw && (long long)block * D * D > compress_static_scratch_floats())
    return fail(-41, "nsa_compress_bwd_noalloc: block*D*D = %lld floats exceeds the built-in scratch of %lld floats; "
                     "use nsa_compress_bwd with a caller workspace", (long long)block * D * D,
                compress_static_scratch_floats());
  CompressArgs a = {};
  a.x = (const bf16*)x; a.w = (const bf16*)w; a.dy = (const bf16*)dy; a.dx = (bf16*)dx; a.dw = dw; a.dbias = dbias;
  a.cu_in = cu_in; a.cu_out = cu_out; a.nseq = nseq; a.H = H; a.D = D; a.l = block; a.d = stride;
  a.max_in = max_in; a.total_out = total_out;
  return launch_compress_bwd_static(a, (cudaStream_t)stream);
}

// ---- compressed attention ---------------------------------------------------------------------------
struct GateArgs {   // optional gate projection fused into the compressed-attention forward
  const void *w, *b;
  void* g[3];
};

static int cmp_attn_fwd_impl(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                     float* sel_scores, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal,
                     float scale, int n_sel, int pool_k, int pool_s, int pool_p, int Tq, int q0, void* stream,
                     const GateArgs* gate = nullptr, int score_mode = 0) {
  const bool sharded = (Tq != T) || (q0 != 0);
  if (Tq <= 0 || q0 < 0 || q0 + Tq > T) return fail(-12, "%s: query shard [%d, %d) is outside the sequence of %d tokens", "nsa_cmp_attn_fwd", q0, q0 + Tq, T);
  (void)sharded;
  if (!q || !ck || !cv || !o || !lse) return fail(-1, "nsa_cmp_attn_fwd: null pointer");
  int rc = check_attn_shape("nsa_cmp_attn_fwd", B, T, Hq, Hk, D);
  if (rc) return rc;
  if (Tc <= 0) return fail(-1, "nsa_cmp_attn_fwd: no compressed positions (sequence shorter than one block)");
  DenseArgs a = {};
  a.mode = 1; a.q = (const bf16*)q; a.k = (const bf16*)ck; a.v = (const bf16*)cv; a.o = (bf16*)o; a.lse = lse;
  a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Lk = Tc; a.Hq = Hq; a.Hk = Hk; a.cblock = block; a.cstride = stride; a.causal = causal;
  a.scale = scale; a.n_sel = n_sel; a.score_mode = score_mode;
  if (score_mode != 0 && score_mode != 1) return fail(-16, "nsa_cmp_attn_fwd: score_mode must be 0 (reference) or 1 (causal)");
  if (score_mode == 1 && !causal) return fail(-16, "nsa_cmp_attn_fwd: causal selection scores need causal = 1");
  if (n_sel > 0) {
    if (!sel_idx) return fail(-1, "nsa_cmp_attn_fwd: sel_idx is null");
    if (Hq / Hk != 16)
      return fail(-7, "nsa_cmp_attn_fwd: block selection needs exactly 16 query heads per KV head (got %d)", Hq / Hk);
    if (pool_k <= 0 || pool_s <= 0 || pool_p < 0) return fail(-8, "nsa_cmp_attn_fwd: bad pooling parameters");
    a.pool_k = pool_k; a.pool_s = pool_s; a.pool_p = pool_p;
    a.n_pool = nsa_pool_out_len(Tc, pool_k, pool_s, pool_p);
    a.sel_idx = sel_idx; a.sel_scores = sel_scores;
  }
  if (dense_fwd_tc_supported(a, D)) {
    if (gate) {
      a.gate_w = (const bf16*)gate->w; a.gate_b = (const bf16*)gate->b;
      for (int i = 0; i < 3; ++i) a.g_out[i] = (bf16*)gate->g[i];
    }
    return launch_dense_fwd2_tc(a, (cudaStream_t)stream);
  }
  if (sharded) return fail(-11, "query shards need head_dim 128 and the default pooling geometry");
  if (score_mode == 1 && n_sel > 0) return fail(-16, "causal selection scores need head_dim 128 and the default pooling geometry");
  rc = launch_dense_fwd(a, D, (cudaStream_t)stream);
  if (rc || !gate) return rc;
  return launch_gate_fwd((const bf16*)q, (const bf16*)gate->w, (const bf16*)gate->b, (bf16*)gate->g[0], (bf16*)gate->g[1],
                         (bf16*)gate->g[2], (long long)B * Tq * Hq, D, (cudaStream_t)stream);
}

int nsa_cmp_attn_fwd(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                     float* sel_scores, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal,
                     float scale, int n_sel, int pool_k, int pool_s, int pool_p, void* stream) {
  return cmp_attn_fwd_impl(q, ck, cv, o, lse, sel_idx, sel_scores, B, T, Tc, Hq, Hk, D, block, stride, causal, scale, n_sel, pool_k, pool_s, pool_p, T, 0, stream);
}

int nsa_cmp_attn_fwd_sharded(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                     float* sel_scores, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal,
                     float scale, int n_sel, int pool_k, int pool_s, int pool_p, int Tq, int q0, void* stream) {
  return cmp_attn_fwd_impl(q, ck, cv, o, lse, sel_idx, sel_scores, B, T, Tc, Hq, Hk, D, block, stride, causal, scale, n_sel, pool_k, pool_s, pool_p, Tq, q0, stream);
}

int nsa_cmp_attn_fwd_gated(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                           float* sel_scores, const void* gate_w, const void* gate_b, void* g_slc, void* g_swa, void* g_cmp,
                           int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal, float scale,
                           int n_sel, int pool_k, int pool_s, int pool_p, int score_mode, int Tq, int q0, void* stream) {
  if (gate_w && (!g_slc || !g_swa || !g_cmp)) return fail(-1, "nsa_cmp_attn_fwd_gated: null gate output");
  const GateArgs g = {gate_w, gate_b, {g_slc, g_swa, g_cmp}};
  return cmp_attn_fwd_impl(q, ck, cv, o, lse, sel_idx, sel_scores, B, T, Tc, Hq, Hk, D, block, stride, causal, scale, n_sel, pool_k, pool_s, pool_p, Tq, q0, stream, gate_w ? &g : nullptr, score_mode);
}

size_t nsa_cmp_attn_bwd_workspace_bytes(int B, int T, int Tc, int Hk, int D) {
  int sl;
  const int nseg = cmp_segments(T, &sl);
  return (size_t)2 * nseg * B * Tc * Hk * D * sizeof(float);
}

struct PreCmp {   // row pre-pass folded into the compressed branch's dQ kernel
  const void* o_cmp;
  void* dg_cmp;
};

static int cmp_attn_bwd_impl(const void* q, const void* ck, const void* cv, const float* lse, const void* dout,
                     const float* delta, const void* gate, void* dq, int accumulate_dq, void* dck, void* dcv, void* ws,
                     size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal,
                     float scale, int Tq, int q0, void* stream, const PreCmp* pre = nullptr) {
  const bool sharded = (Tq != T) || (q0 != 0);
  if (Tq <= 0 || q0 < 0 || q0 + Tq > T) return fail(-12, "%s: query shard [%d, %d) is outside the sequence of %d tokens", "nsa_cmp_attn_bwd", q0, q0 + Tq, T);
  (void)sharded;
  if (!q || !ck || !cv || !lse || !dout || !delta) return fail(-1, "nsa_cmp_attn_bwd: null pointer");
  int rc = check_attn_shape("nsa_cmp_attn_bwd", B, T, Hq, Hk, D);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  bool fold = false;
  if (pre) {
    if (!pre->o_cmp) return fail(-1, "nsa_cmp_attn_bwd_fused: o_cmp is null");
    fold = dq && D == 128;
    if (!fold) {   // no tcgen05 dQ kernel to carry the pre-pass: run it on its own
      rc = launch_rowdot((const bf16*)pre->o_cmp, (const bf16*)dout, (const bf16*)gate, const_cast<float*>(delta),
                         (bf16*)pre->dg_cmp, (long long)B * Tq * Hq, D, s);
      if (rc) return rc;
    }
  }
  if (dq) {
    DenseArgs a = {};
    if (fold) {
      a.pre_o[0] = (const bf16*)pre->o_cmp; a.pre_gate[0] = (const bf16*)gate; a.pre_delta[0] = const_cast<float*>(delta);
      a.pre_dgate[0] = (bf16*)pre->dg_cmp;
    }
    a.mode = 1; a.q = (const bf16*)q; a.k = (const bf16*)ck; a.v = (const bf16*)cv; a.lse = const_cast<float*>(lse);
    a.dout = (const bf16*)dout; a.delta = delta; a.gate = (const bf16*)gate; a.dq = (bf16*)dq;
    a.accumulate = accumulate_dq; a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Lk = Tc; a.Hq = Hq; a.Hk = Hk; a.cblock = block;
    a.cstride = stride; a.causal = causal; a.scale = scale;
    if (D != 128 && sharded) return fail(-11, "query shards need head_dim 128");
      rc = (D == 128) ? launch_dense_dq_tc(a, s) : launch_dense_dq(a, D, s);
    if (rc) return rc;
  }
  if (dck || dcv) {
    if (!dck || !dcv) return fail(-1, "nsa_cmp_attn_bwd: dck and dcv must be given together");
    if (!ws || ws_bytes < nsa_cmp_attn_bwd_workspace_bytes(B, T, Tc, Hk, D))
      return fail(-6, "nsa_cmp_attn_bwd: workspace too small");
    KvArgs a = {};
    a.mode = 1; a.q = (const bf16*)q; a.k = (const bf16*)ck; a.v = (const bf16*)cv;
    a.dout_a = (const bf16*)dout; a.lse_a = lse; a.delta_a = delta; a.gate_a = (const bf16*)gate;
    a.part = (float*)ws; a.nseg = cmp_segments(Tq, &a.seg_len);
    a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Lk = Tc; a.Hq = Hq; a.Hk = Hk; a.BS = 64; a.cblock = block; a.cstride = stride;
    a.causal = causal; a.scale = scale;
    if (D != 128 && sharded) return fail(-11, "query shards need head_dim 128");
    rc = (D == 128) ? launch_kv_bwd_tc(a, s) : launch_kv_bwd(a, D, s);
    if (rc) return rc;
    const long long N = (long long)B * Tc * Hk * D;
    rc = launch_reduce_segments(a.part, (bf16*)dck, a.nseg, N, q0, Tq, Tc, Hk, D, a.seg_len, block, stride, causal, s);
    if (rc) return rc;
    rc = launch_reduce_segments(a.part + (long long)a.nseg * N, (bf16*)dcv, a.nseg, N, q0, Tq, Tc, Hk, D, a.seg_len, block,
                                stride, causal, s);
    if (rc) return rc;
  }
  return 0;
}

int nsa_cmp_attn_bwd(const void* q, const void* ck, const void* cv, const float* lse, const void* dout,
                     const float* delta, const void* gate, void* dq, int accumulate_dq, void* dck, void* dcv, void* ws,
                     size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal,
                     float scale, void* stream) {
  return cmp_attn_bwd_impl(q, ck, cv, lse, dout, delta, gate, dq, accumulate_dq, dck, dcv, ws, ws_bytes, B, T, Tc, Hq, Hk, D, block, stride, causal, scale, T, 0, stream);
}

int nsa_cmp_attn_bwd_sharded(const void* q, const void* ck, const void* cv, const float* lse, const void* dout,
                     const float* delta, const void* gate, void* dq, int accumulate_dq, void* dck, void* dcv, void* ws,
                     size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal,
                     float scale, int Tq, int q0, void* stream) {
  return cmp_attn_bwd_impl(q, ck, cv, lse, dout, delta, gate, dq, accumulate_dq, dck, dcv, ws, ws_bytes, B, T, Tc, Hq, Hk, D, block, stride, causal, scale, Tq, q0, stream);
}

// ---- selected + sliding window ----------------------------------------------------------------------
static int check_bs(const char* who, int BS) {
  if (BS != 16 && BS != 32 && BS != 64) return fail(-9, "%s: selection block size %d not supported (16, 32, 64)", who, BS);
  return 0;
}

// Workspace of the key-major selected forward: the reverse index (as in the backward), its inverse [B,Tq,Hkv,S] int32,
// one [16 x D] bf16 tile and 16 (max, sum) pairs per (list position, 16-head sub-group).
size_t nsa_sel_swa_fwd_workspace_bytes(int B, int T, int Tq, int Hq, int Hkv, int D, int S, int BS) {
  if (BS <= 0 || Hkv <= 0) return 0;
  const size_t ent = (size_t)B * Tq * Hkv * S;
  const size_t g = (size_t)(Hq / Hkv);
  return nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, S, BS) + align_up(ent * 4, 256) + align_up(ent * g * D * 2, 256) +
         align_up(ent * g * 8, 256);
}

static int sel_swa_fwd_impl(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    void* o_slc, float* lse_slc, void* o_swa, float* lse_swa, const void* g_slc, const void* g_swa,
                    const void* o_cmp, const void* g_cmp, void* o, int B, int T, int Hq, int Hkv, int D, int S, int BS,
                    int window, float scale, int Tq, int q0, void* stream, void* ws = nullptr, size_t ws_bytes = 0) {
  const bool sharded = (Tq != T) || (q0 != 0);
  if (Tq <= 0 || q0 < 0 || q0 + Tq > T) return fail(-12, "%s: query shard [%d, %d) is outside the sequence of %d tokens", "nsa_sel_swa_fwd", q0, q0 + Tq, T);
  (void)sharded;
  if (!q || !k || !v) return fail(-1, "nsa_sel_swa_fwd: null pointer");
  int rc = check_attn_shape("nsa_sel_swa_fwd", B, T, Hq, Hkv, D);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (o_slc) {
    if (!idx || !lse_slc) return fail(-1, "nsa_sel_swa_fwd: idx / lse_slc is null");
    rc = check_bs("nsa_sel_swa_fwd", BS);
    if (rc) return rc;
    if (S <= 0) return fail(-1, "nsa_sel_swa_fwd: no selected blocks");
    SelKvArgs ka = {};
    ka.q = (const bf16*)q; ka.k = (const bf16*)k; ka.v = (const bf16*)v; ka.o = (bf16*)o_slc; ka.lse = lse_slc;
    ka.B = B; ka.T = T; ka.Tq = Tq; ka.q0 = q0; ka.Hq = Hq; ka.Hk = Hkv; ka.S = S; ka.BS = BS; ka.scale = scale;
    if (ws && sel_fwd_kv_supported(ka, D) && ws_bytes >= nsa_sel_swa_fwd_workspace_bytes(B, T, Tq, Hq, Hkv, D, S, BS)) {
      // key-major: reverse index, then one CTA per key block over the queries that selected it, then the per-token merge
      const int NB = (T + BS - 1) / BS;
      const size_t bh = (size_t)B * Hkv, ent = (size_t)B * Tq * Hkv * S, g = (size_t)(Hq / Hkv);
      char* p = (char*)ws;
      RevArgs r = {};
      r.idx = idx; r.idx64 = idx64; r.counts = counts; r.B = B; r.T = T; r.Tq = Tq; r.q0 = q0; r.H = Hkv; r.S = S; r.BS = BS; r.NB = NB;
      r.hist = (int*)p;
      p += align_up(bh * NB * NB * 4, 256);
      r.rev_ptr = (int*)p;
      p += align_up(bh * (NB + 1) * 4, 256);
      r.rev_tok = (int*)p;
      p += align_up(bh * (size_t)T * S * 4, 256);
      r.cap = (long long)Tq * S;
      r.inv = (int*)p;
      p += align_up(ent * 4, 256);
      ka.part = (bf16*)p;
      p += align_up(ent * g * D * 2, 256);
      ka.stats = (float*)p;
      rc = launch_build_rev(r, s);
      if (rc) return rc;
      ka.rev_ptr = r.rev_ptr; ka.rev_tok = r.rev_tok; ka.rev_cap = r.cap;
      rc = launch_sel_fwd_kv(ka, r, s);
      if (rc) return rc;
    } else {
      SelArgs a = {};
      a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.idx = idx; a.idx64 = idx64; a.counts = counts;
      a.o = (bf16*)o_slc; a.lse = lse_slc; a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Hq = Hq; a.Hkv = Hkv; a.S = S; a.BS = BS; a.scale = scale;
      rc = launch_sel_fwd(a, D, s);
      if (rc) return rc;
    }
  }
  if (window > 0) {
    if (!o_swa || !lse_swa) return fail(-1, "nsa_sel_swa_fwd: o_swa / lse_swa is null");
    DenseArgs a = {};
    a.mode = 0; a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.o = (bf16*)o_swa; a.lse = lse_swa;
    a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Lk = T; a.Hq = Hq; a.Hk = Hkv; a.window = window; a.scale = scale;
    if (!dense_fwd_tc_supported(a, D) && sharded) return fail(-11, "query shards need head_dim 128");
    rc = dense_fwd_tc_supported(a, D) ? launch_dense_fwd2_tc(a, s) : launch_dense_fwd(a, D, s);
    if (rc) return rc;
  }
  if (o) {
    rc = launch_combine((const bf16*)o_slc, (const bf16*)g_slc, window > 0 ? (const bf16*)o_swa : nullptr,
                        (const bf16*)g_swa, (const bf16*)o_cmp, (const bf16*)g_cmp, (bf16*)o, (long long)B * Tq * Hq, D, s);
    if (rc) return rc;
  }
  return 0;
}

int nsa_sel_swa_fwd(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    void* o_slc, float* lse_slc, void* o_swa, float* lse_swa, const void* g_slc, const void* g_swa,
                    const void* o_cmp, const void* g_cmp, void* o, int B, int T, int Hq, int Hkv, int D, int S, int BS,
                    int window, float scale, void* stream) {
  return sel_swa_fwd_impl(q, k, v, idx, idx64, counts, o_slc, lse_slc, o_swa, lse_swa, g_slc, g_swa, o_cmp, g_cmp, o, B, T, Hq, Hkv, D, S, BS, window, scale, T, 0, stream);
}

int nsa_sel_swa_fwd_sharded(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    void* o_slc, float* lse_slc, void* o_swa, float* lse_swa, const void* g_slc, const void* g_swa,
                    const void* o_cmp, const void* g_cmp, void* o, int B, int T, int Hq, int Hkv, int D, int S, int BS,
                    int window, float scale, int Tq, int q0, void* stream) {
  return sel_swa_fwd_impl(q, k, v, idx, idx64, counts, o_slc, lse_slc, o_swa, lse_swa, g_slc, g_swa, o_cmp, g_cmp, o, B, T, Hq, Hkv, D, S, BS, window, scale, Tq, q0, stream);
}

int nsa_sel_swa_fwd_ws(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    void* o_slc, float* lse_slc, void* o_swa, float* lse_swa, const void* g_slc, const void* g_swa,
                    const void* o_cmp, const void* g_cmp, void* o, void* ws, size_t ws_bytes, int B, int T, int Hq, int Hkv,
                    int D, int S, int BS, int window, float scale, int Tq, int q0, void* stream) {
  return sel_swa_fwd_impl(q, k, v, idx, idx64, counts, o_slc, lse_slc, o_swa, lse_swa, g_slc, g_swa, o_cmp, g_cmp, o, B, T, Hq, Hkv, D, S, BS, window, scale, Tq, q0, stream, ws, ws_bytes);
}

int nsa_cmp_attn_bwd_fused(const void* q, const void* ck, const void* cv, const void* o_cmp, const float* lse, const void* dout,
                           float* delta, const void* gate, void* dgate, void* dq, int accumulate_dq, void* dck, void* dcv,
                           void* ws, size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride,
                           int causal, float scale, int Tq, int q0, void* stream) {
  const PreCmp pre = {o_cmp, dgate};
  return cmp_attn_bwd_impl(q, ck, cv, lse, dout, delta, gate, dq, accumulate_dq, dck, dcv, ws, ws_bytes, B, T, Tc, Hq, Hk, D, block, stride, causal, scale, Tq, q0, stream, &pre);
}

size_t nsa_sel_swa_bwd_workspace_bytes(int B, int T, int Hkv, int S, int BS) {
  if (BS <= 0) return 0;
  const size_t NB = (size_t)(T + BS - 1) / BS;
  const size_t bh = (size_t)B * Hkv;
  return align_up(bh * NB * NB * 4, 256) + align_up(bh * (NB + 1) * 4, 256) + align_up(bh * (size_t)T * S * 4, 256);
}

// Extra workspace behind the reverse index for the selected branch's dQ as per-visit partials of the kv-major backward:
// the inverse index [B,Tq,Hkv,S] int32 and one [16 x D] bf16 tile per (list position, 16-head sub-group).
static size_t sel_dq_extra_bytes(int B, int Tq, int Hq, int Hkv, int D, int S) {
  const size_t ent = (size_t)B * Tq * Hkv * S;
  return align_up(ent * 4, 256) + align_up(ent * (size_t)(Hq / Hkv) * D * 2, 256);
}

struct PreSel {   // row pre-pass of the selected and window branches folded into the window's dQ kernel
  const void *o_slc, *o_swa;
  void *dg_slc, *dg_swa;
};

static int sel_swa_bwd_impl(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    const void* dout_slc, const float* lse_slc, const float* delta_slc, const void* gate_slc,
                    const void* dout_swa, const float* lse_swa, const float* delta_swa, const void* gate_swa, void* dq,
                    int accumulate_dq, void* dk, void* dv, void* ws, size_t ws_bytes, int B, int T, int Hq, int Hkv,
                    int D, int S, int BS, int window, float scale, int Tq, int q0, void* stream,
                    const PreSel* pre = nullptr) {
  const bool sharded = (Tq != T) || (q0 != 0);
  if (Tq <= 0 || q0 < 0 || q0 + Tq > T) return fail(-12, "%s: query shard [%d, %d) is outside the sequence of %d tokens", "nsa_sel_swa_bwd", q0, q0 + Tq, T);
  (void)sharded;
  if (!q || !k || !v) return fail(-1, "nsa_sel_swa_bwd: null pointer");
  int rc = check_attn_shape("nsa_sel_swa_bwd", B, T, Hq, Hkv, D);
  if (rc) return rc;
  rc = check_bs("nsa_sel_swa_bwd", BS);
  if (rc) return rc;
  const bool has_slc = dout_slc != nullptr, has_swa = window > 0 && dout_swa != nullptr;
  if (!has_slc && !has_swa) return fail(-1, "nsa_sel_swa_bwd: neither branch has an upstream gradient");
  if (has_slc && (!idx || !lse_slc || !delta_slc)) return fail(-1, "nsa_sel_swa_bwd: selected branch inputs missing");
  if (has_swa && (!lse_swa || !delta_swa)) return fail(-1, "nsa_sel_swa_bwd: window branch inputs missing");
  cudaStream_t s = (cudaStream_t)stream;
  const long long rows = (long long)B * Tq * Hq;
  // With the larger workspace of nsa_sel_swa_bwd_workspace_bytes_dq the selected branch's dQ is produced by the
  // kv-major backward (per-visit partial tiles + a slot-order reduction) instead of the query-major dQ kernel.
  const bool dq_from_kv = dq && dk && has_slc && D == 128 && BS == 64 && S <= 32 && ws &&
                          ws_bytes >= nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, S, BS) + sel_dq_extra_bytes(B, Tq, Hq, Hkv, D, S);
  int dq_acc_for_reduce = accumulate_dq;
  bool fold = false;
  if (pre) {
    if ((has_slc && !pre->o_slc) || (has_swa && !pre->o_swa)) return fail(-1, "nsa_sel_swa_bwd_fused: a branch output is null");
    if (has_slc && has_swa && dout_slc != dout_swa)
      return fail(-15, "nsa_sel_swa_bwd_fused: both branches must share one upstream gradient (the module's dO)");
    // the window's tcgen05 dQ kernel carries the pre-pass of both branches and therefore runs first
    fold = dq && has_swa && D == 128;
    if (!fold) {
      const bf16* o3[3] = {has_slc ? (const bf16*)pre->o_slc : nullptr, has_swa ? (const bf16*)pre->o_swa : nullptr, nullptr};
      const bf16* g3[3] = {(const bf16*)gate_slc, (const bf16*)gate_swa, nullptr};
      float* d3[3] = {const_cast<float*>(delta_slc), const_cast<float*>(delta_swa), nullptr};
      bf16* dg3[3] = {(bf16*)pre->dg_slc, (bf16*)pre->dg_swa, nullptr};
      rc = launch_rowdot3(o3, (const bf16*)(has_slc ? dout_slc : dout_swa), g3, d3, dg3, rows, D, s);
      if (rc) return rc;
    }
  }
  if (dq) {
    int acc = accumulate_dq;
    auto run_swa = [&]() -> int {
      DenseArgs a = {};
      a.mode = 0; a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.lse = const_cast<float*>(lse_swa);
      a.dout = (const bf16*)dout_swa; a.delta = delta_swa; a.gate = (const bf16*)gate_swa; a.dq = (bf16*)dq;
      a.accumulate = acc; a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Lk = T; a.Hq = Hq; a.Hk = Hkv; a.window = window; a.scale = scale;
      if (fold) {
        a.pre_o[0] = (const bf16*)pre->o_swa; a.pre_gate[0] = (const bf16*)gate_swa;
        a.pre_delta[0] = const_cast<float*>(delta_swa); a.pre_dgate[0] = (bf16*)pre->dg_swa;
        if (has_slc) {
          a.pre_o[1] = (const bf16*)pre->o_slc; a.pre_gate[1] = (const bf16*)gate_slc;
          a.pre_delta[1] = const_cast<float*>(delta_slc); a.pre_dgate[1] = (bf16*)pre->dg_slc;
        }
      }
      if (D != 128 && sharded) return fail(-11, "query shards need head_dim 128");
      return (D == 128) ? launch_dense_dq_tc(a, s) : launch_dense_dq(a, D, s);
    };
    if (fold) {
      rc = run_swa();
      if (rc) return rc;
      acc = 1;
    }
    if (has_slc && dq_from_kv) {
      // nothing here: the reduction behind the kv-major kernel writes (or adds) the selected branch's dQ.  If the window
      // kernel has not run yet it must not overwrite that: it runs now and the reduction accumulates.
      if (has_swa && !fold) {
        rc = run_swa();
        if (rc) return rc;
      }
      dq_acc_for_reduce = (acc || has_swa) ? 1 : 0;
    } else if (has_slc) {
      SelArgs a = {};
      a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.idx = idx; a.idx64 = idx64; a.counts = counts;
      a.lse = const_cast<float*>(lse_slc); a.dout = (const bf16*)dout_slc; a.delta = delta_slc;
      a.gate = (const bf16*)gate_slc; a.dq = (bf16*)dq; a.accumulate = acc;
      a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Hq = Hq; a.Hkv = Hkv; a.S = S; a.BS = BS; a.scale = scale;
      rc = launch_sel_dq(a, D, s);
      if (rc) return rc;
      acc = 1;
    }
    if (has_swa && !fold && !(has_slc && dq_from_kv)) {
      rc = run_swa();
      if (rc) return rc;
    }
  }
  if (dk || dv) {
    if (!dk || !dv) return fail(-1, "nsa_sel_swa_bwd: dk and dv must be given together");
    KvArgs a = {};
    a.mode = 0; a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v;
    a.B = B; a.T = T; a.Tq = Tq; a.q0 = q0; a.Lk = T; a.Hq = Hq; a.Hk = Hkv; a.BS = BS; a.window = has_swa ? window : 0; a.scale = scale;
    a.dk = (bf16*)dk; a.dv = (bf16*)dv;
    RevArgs r = {};
    if (has_slc) {
      if (!ws || ws_bytes < nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, S, BS))
        return fail(-6, "nsa_sel_swa_bwd: workspace too small");
      const int NB = (T + BS - 1) / BS;
      const size_t bh = (size_t)B * Hkv;
      char* p = (char*)ws;
      r.idx = idx; r.idx64 = idx64; r.counts = counts; r.B = B; r.T = T; r.Tq = Tq; r.q0 = q0; r.H = Hkv; r.S = S; r.BS = BS; r.NB = NB;
      r.hist = (int*)p;
      p += align_up(bh * NB * NB * 4, 256);
      r.rev_ptr = (int*)p;
      p += align_up(bh * (NB + 1) * 4, 256);
      r.rev_tok = (int*)p;
      r.cap = (long long)Tq * S;
      if (dq_from_kv) {
        p += align_up(bh * (size_t)T * S * 4, 256);
        r.inv = (int*)p;
        p += align_up((size_t)B * Tq * Hkv * S * 4, 256);
        a.dq_part = (bf16*)p;
      }
      rc = launch_build_rev(r, s);
      if (rc) return rc;
      a.rev_ptr = r.rev_ptr; a.rev_tok = r.rev_tok; a.rev_cap = r.cap;
      a.dout_a = (const bf16*)dout_slc; a.lse_a = lse_slc; a.delta_a = delta_slc; a.gate_a = (const bf16*)gate_slc;
    }
    if (has_swa) {
      a.dout_b = (const bf16*)dout_swa; a.lse_b = lse_swa; a.delta_b = delta_swa; a.gate_b = (const bf16*)gate_swa;
    }
    if (!(D == 128 && BS == 64) && sharded) return fail(-11, "query shards need head_dim 128 and 64-key selection blocks");
    rc = (D == 128 && BS == 64) ? launch_kv_bwd_tc(a, s) : launch_kv_bwd(a, D, s);
    if (rc) return rc;
    if (dq_from_kv) {   // every token's partial tiles, in slot order, onto dq (after the window's dQ if that ran first)
      rc = launch_sel_dq_reduce(r, a.dq_part, (bf16*)dq, Hq, D, scale, dq_acc_for_reduce, s);
      if (rc) return rc;
    }
  }
  return 0;
}

size_t nsa_sel_swa_bwd_workspace_bytes_dq(int B, int T, int Tq, int Hq, int Hkv, int D, int S, int BS) {
  return nsa_sel_swa_bwd_workspace_bytes(B, T, Hkv, S, BS) + sel_dq_extra_bytes(B, Tq, Hq, Hkv, D, S);
}

int nsa_sel_swa_bwd(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    const void* dout_slc, const float* lse_slc, const float* delta_slc, const void* gate_slc,
                    const void* dout_swa, const float* lse_swa, const float* delta_swa, const void* gate_swa, void* dq,
                    int accumulate_dq, void* dk, void* dv, void* ws, size_t ws_bytes, int B, int T, int Hq, int Hkv,
                    int D, int S, int BS, int window, float scale, void* stream) {
  return sel_swa_bwd_impl(q, k, v, idx, idx64, counts, dout_slc, lse_slc, delta_slc, gate_slc, dout_swa, lse_swa, delta_swa, gate_swa, dq, accumulate_dq, dk, dv, ws, ws_bytes, B, T, Hq, Hkv, D, S, BS, window, scale, T, 0, stream);
}

int nsa_sel_swa_bwd_sharded(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    const void* dout_slc, const float* lse_slc, const float* delta_slc, const void* gate_slc,
                    const void* dout_swa, const float* lse_swa, const float* delta_swa, const void* gate_swa, void* dq,
                    int accumulate_dq, void* dk, void* dv, void* ws, size_t ws_bytes, int B, int T, int Hq, int Hkv,
                    int D, int S, int BS, int window, float scale, int Tq, int q0, void* stream) {
  return sel_swa_bwd_impl(q, k, v, idx, idx64, counts, dout_slc, lse_slc, delta_slc, gate_slc, dout_swa, lse_swa, delta_swa, gate_swa, dq, accumulate_dq, dk, dv, ws, ws_bytes, B, T, Hq, Hkv, D, S, BS, window, scale, Tq, q0, stream);
}

int nsa_gather_probe(const void* k, const void* v, const void* idx, int idx64, int B, int T, int Hq, int Hkv, int D, int S,
                     int BS, void* stream) {
  if (!k || !v || !idx) return fail(-1, "nsa_gather_probe: null pointer");
  int rc = check_attn_shape("nsa_gather_probe", B, T, Hq, Hkv, D);
  if (rc) return rc;
  SelArgs a = {};
  a.k = (const bf16*)k; a.v = (const bf16*)v; a.idx = idx; a.idx64 = idx64;
  a.B = B; a.T = T; a.Tq = T; a.q0 = 0; a.Hq = Hq; a.Hkv = Hkv; a.S = S; a.BS = BS;
  return launch_gather_probe(a, D, (cudaStream_t)stream);
}

int nsa_sel_swa_bwd_fused(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                          const void* o_slc, const void* o_swa, const void* dout, const float* lse_slc, float* delta_slc,
                          const void* gate_slc, void* dgate_slc, const float* lse_swa, float* delta_swa, const void* gate_swa,
                          void* dgate_swa, void* dq, int accumulate_dq, void* dk, void* dv, void* ws, size_t ws_bytes, int B,
                          int T, int Hq, int Hkv, int D, int S, int BS, int window, float scale, int Tq, int q0, void* stream) {
  if (!dout || !delta_slc) return fail(-1, "nsa_sel_swa_bwd_fused: null pointer");
  if (window > 0 && !delta_swa) return fail(-1, "nsa_sel_swa_bwd_fused: delta_swa is null");
  const PreSel pre = {o_slc, o_swa, dgate_slc, dgate_swa};
  return sel_swa_bwd_impl(q, k, v, idx, idx64, counts, dout, lse_slc, delta_slc, gate_slc, window > 0 ? dout : nullptr, lse_swa, delta_swa, gate_swa, dq, accumulate_dq, dk, dv, ws, ws_bytes, B, T, Hq, Hkv, D, S, BS, window, scale, Tq, q0, stream, &pre);
}

// ---- decode ---------------------------------------------------------------------------------------------
int nsa_decode_fwd(const void* q, const void* k, const void* v, const void* ck, const void* cv, const int32_t* cu_k,
                   const int32_t* cu_c, const int32_t* order, const void* gate_w, const void* gate_b, const void* g_slc,
                   const void* g_swa, const void* g_cmp, void* o, void* o_cmp, void* o_slc, void* o_swa, float* lse,
                   int32_t* idx, void* ws, size_t ws_bytes, int nseq,
                   long long total_k, long long total_c, int max_Tc, int Hq, int Hkv, int D, int block, int stride,
                   int sel_block, int n_sel, int window, float scale, void* stream) {
  if (!q || !k || !v || !ck || !cv || !cu_k || !cu_c || !o || !idx || !ws) return fail(-1, "nsa_decode_fwd: null pointer");
  if (nseq <= 0) return 0;
  if (total_k <= 0 || total_c <= 0 || Hq <= 0 || Hkv <= 0) return fail(-1, "nsa_decode_fwd: empty shape");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(ck) || !aligned16(cv) || !aligned16(o))
    return fail(-5, "nsa_decode_fwd: pointers must be 16-byte aligned");
  DecodeArgs a = {};
  a.q = (const bf16*)q; a.k = (const bf16*)k; a.v = (const bf16*)v; a.ck = (const bf16*)ck; a.cv = (const bf16*)cv;
  a.cu_k = cu_k; a.cu_c = cu_c; a.order = order; a.gate_w = (const bf16*)gate_w; a.gate_b = (const bf16*)gate_b;
  a.g_slc = (const bf16*)g_slc; a.g_swa = (const bf16*)g_swa; a.g_cmp = (const bf16*)g_cmp;
  a.o = (bf16*)o; a.o_cmp = (bf16*)o_cmp; a.o_slc = (bf16*)o_slc; a.o_swa = (bf16*)o_swa; a.lse = lse; a.idx = idx;
  a.nseq = nseq; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.n_sel = n_sel; a.window = window; a.cblock = block; a.cstride = stride;
  a.sel_block = sel_block; a.total_k = total_k; a.total_c = total_c; a.max_Tc = max_Tc; a.scale = scale;
  a.part = (float*)ws; a.part_bytes = ws_bytes;
  return launch_decode(a, (cudaStream_t)stream);
}

size_t nsa_decode_workspace_bytes(int nseq, int Hkv) { return decode_workspace_bytes(nseq, Hkv); }

// ---- helpers ------------------------------------------------------------------------------------------
int nsa_rowdot(const void* o, const void* dout, const void* gate, float* delta, void* dgate, long long rows, int D,
               void* stream) {
  if (!o || !dout) return fail(-1, "nsa_rowdot: null pointer");
  return launch_rowdot((const bf16*)o, (const bf16*)dout, (const bf16*)gate, delta, (bf16*)dgate, rows, D,
                       (cudaStream_t)stream);
}

int nsa_gate_fwd(const void* q, const void* w, const void* bias, void* g_slc, void* g_swa, void* g_cmp, long long rows,
                 int D, void* stream) {
  if (!q || !w || !g_slc || !g_swa || !g_cmp) return fail(-1, "nsa_gate_fwd: null pointer");
  return launch_gate_fwd((const bf16*)q, (const bf16*)w, (const bf16*)bias, (bf16*)g_slc, (bf16*)g_swa, (bf16*)g_cmp, rows,
                         D, (cudaStream_t)stream);
}

int nsa_rowdot3(const void* o_slc, const void* o_swa, const void* o_cmp, const void* dout, const void* g_slc,
                const void* g_swa, const void* g_cmp, float* delta_slc, float* delta_swa, float* delta_cmp, void* dg_slc,
                void* dg_swa, void* dg_cmp, long long rows, int D, void* stream) {
  if (!dout) return fail(-1, "nsa_rowdot3: null upstream gradient");
  const bf16* o[3] = {(const bf16*)o_slc, (const bf16*)o_swa, (const bf16*)o_cmp};
  const bf16* g[3] = {(const bf16*)g_slc, (const bf16*)g_swa, (const bf16*)g_cmp};
  float* dl[3] = {delta_slc, delta_swa, delta_cmp};
  bf16* dg[3] = {(bf16*)dg_slc, (bf16*)dg_swa, (bf16*)dg_cmp};
  return launch_rowdot3(o, (const bf16*)dout, g, dl, dg, rows, D, (cudaStream_t)stream);
}

long long nsa_gate_bwd_workspace_bytes(long long rows, int D) { return gate_bwd_workspace_bytes(rows, D); }

int nsa_gate_bwd(const void* q, const void* dg_slc, const void* dg_swa, const void* dg_cmp, const void* w, void* dq,
                 void* dw, void* dbias, void* workspace, long long workspace_bytes, long long rows, int D, void* stream) {
  if (!q || !dg_slc || !dg_swa || !dg_cmp || !w || !dq || !dw || !workspace) return fail(-1, "nsa_gate_bwd: null pointer");
  if (workspace_bytes < gate_bwd_workspace_bytes(rows, D)) return fail(-3, "nsa_gate_bwd: workspace too small");
  return launch_gate_bwd((const bf16*)q, (const bf16*)dg_slc, (const bf16*)dg_swa, (const bf16*)dg_cmp, (const bf16*)w,
                         (bf16*)dq, (bf16*)dw, (bf16*)dbias, (float*)workspace, rows, D, (cudaStream_t)stream);
}

int nsa_combine(const void* a0, const void* g0, const void* a1, const void* g1, const void* a2, const void* g2, void* o,
                long long rows, int D, void* stream) {
  if (!o) return fail(-1, "nsa_combine: null output");
  return launch_combine((const bf16*)a0, (const bf16*)g0, (const bf16*)a1, (const bf16*)g1, (const bf16*)a2,
                        (const bf16*)g2, (bf16*)o, rows, D, (cudaStream_t)stream);
}

}  // extern "C"
