/* C ABI of libnsa_b200.so: the B200 (sm_100a) kernels of the Native Sparse Attention path.
 *
 * The reference project has no native boundary of its own: its boundary is the Python API of the `nsa`
 * package, whose autograd functions launch Triton kernels.  Each entry point below names the reference
 * interface (file:line in the reference project) whose kernels it replaces; the Python package
 * `nsa_b200` keeps the reference's module/function signatures and calls these through ctypes.
 *
 * Conventions
 *  - Every pointer is a device pointer owned by the caller (inputs, outputs and workspaces alike).  The
 *    library never allocates or frees device memory and keeps no pointer after a call returns.
 *  - Tensors are contiguous, bf16 unless stated, with the layouts given per function; `void* stream` is a
 *    cudaStream_t.  Work is enqueued on that stream; no entry point synchronises except
 *    nsa_device_status().
 *  - Return value: 0 on success; negative = rejected arguments / unsupported configuration (text in
 *    nsa_last_error(), thread local); positive = cudaError_t from a launch.
 *  - Supported: head_dim D in {64, 128}; query heads per KV head a multiple of 16; selection block size
 *    in {16, 32, 64}.
 *  - Kernels bound every internal wait; if one gives up it records a code that nsa_device_status()
 *    returns (0 = healthy).
 */
#ifndef NSA_B200_H_
#define NSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int nsa_abi_version(void);
const char* nsa_last_error(void);
/* Synchronises the current device, returns and clears the device-side error code (0 = none). */
int nsa_device_status(void);
/* Number of kernels this library has launched in this process so far (for benchmarks' bookkeeping). */
long long nsa_kernel_launch_count(void);

/* ---- compression -------------------------------------------------------------------------------
 * Replaces compress_kv / _compress_kv.forward (nsa/compression_kv.py:178-217, kernel :21-57) and the two
 * nn.Conv1d calls of KVCompressor.forward (nsa/compression_kv.py:301-307).
 * x [tok,H,D]; w [block*D, D] (row j*D+c multiplies channel c of in-block offset j; a Conv1d weight
 * [D,D,block] is passed as weight.permute(2,1,0)); bias [D] or NULL; y [out_tok,H,D];
 * cu_in / cu_out: device int32 [nseq+1] cumulative input / output lengths; max_out = longest output. */
int nsa_compress_fwd(const void* x, const void* w, const void* bias, void* y, const int32_t* cu_in,
                     const int32_t* cu_out, int nseq, int H, int D, int block, int stride, int max_out,
                     void* stream);
/* The same forward for B equal-length sequences (x [B*T,H,D], T a multiple of stride): one tcgen05 GEMM per
 * (batch, head, 128 output rows) whose A tiles are TMA boxes over the overlapping windows; y [B,Tc,H,D] with
 * Tc = (T-block)/stride + 1 (the Conv1d rule of nsa/compression_kv.py:298-307). */
int nsa_compress_fwd_uniform(const void* x, const void* w, const void* bias, void* y, int B, int T, int H, int D,
                             int block, int stride, void* stream);
/* Replaces _compress_kv.backward (nsa/compression_kv.py:219-266, kernels :62-171) and the Conv1d backward.
 * dy [out_tok,H,D] -> dx [tok,H,D] bf16 (NULL to skip), dw [block*D, D] fp32 (NULL to skip),
 * dbias [D] fp32 (NULL to skip).  ws: nsa_compress_bwd_workspace_bytes() bytes, needed when dw != NULL. */
int nsa_compress_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, float* dbias, void* ws,
                     size_t ws_bytes, const int32_t* cu_in, const int32_t* cu_out, int nseq, int H, int D,
                     int block, int stride, int max_in, int total_out, void* stream);
size_t nsa_compress_bwd_workspace_bytes(int nseq, int H, int D, int block);
/* No counterpart in the reference.  The same backward as nsa_compress_bwd for callers that must not allocate
 * device memory when they need it (a runtime that has already handed out all of its HBM, a plugin host that owns
 * the allocator): the fp32 partials of the dW reduction go to a 16 MiB device array built into the library, so
 * there is no workspace argument and the call itself never allocates.  Limit: block*D*D <= 4 Mi floats (for
 * D = 128 that is block <= 256); larger shapes are rejected with a negative code and must use nsa_compress_bwd.
 * The first call on a device looks up the array's device address; make that call before any stream capture.  The
 * array used is the one of the device that is CURRENT when the call is made (cudaGetDevice), not of the device the
 * stream belongs to: set the device before calling, as for every other entry point.
 * All calls share the one array and leave their partials in it (each call overwrites what it uses, nothing has
 * to be cleared), so two calls whose kernels could overlap on the GPU (different streams) race: serialise them. */
int nsa_compress_bwd_noalloc(const void* x, const void* w, const void* dy, void* dx, float* dw, float* dbias,
                             const int32_t* cu_in, const int32_t* cu_out, int nseq, int H, int D, int block,
                             int stride, int max_in, int total_out, void* stream);

/* ---- compressed attention + block selection ------------------------------------------------------
 * Replaces _attention.forward (nsa/triton_attention.py:421-476: _attn_fwd, softmax_kernel, group sum,
 * avg_pool1d, topk) with one kernel; the [B,Hq,T,Tc] score tensor is never materialised.
 * q [B,T,Hq,D]; ck,cv [B,Tc,Hk,D] (Hq/Hk a multiple of 16); o [B,T,Hq,D]; lse [B,T,Hq] fp32 (natural log,
 * -inf for rows that see nothing).  If n_sel > 0: sel_idx [B,T,Hq/16,n_sel] int32 receives the top-n
 * pooled blocks (ties to the lower index, -1 when fewer than n_sel blocks exist) and sel_scores (NULL or
 * [B,Hq/16,T,n_pool] fp32) the pooled scores; n_pool = nsa_pool_out_len(Tc, pool_k, pool_s, pool_p). */
int nsa_cmp_attn_fwd(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                     float* sel_scores, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride,
                     int causal, float scale, int n_sel, int pool_k, int pool_s, int pool_p, void* stream);
int nsa_pool_out_len(int n, int pool_k, int pool_s, int pool_p);
/* nsa_cmp_attn_fwd_sharded with two options.
 * (1) gate_w != NULL: the module's gate projection fused in.  While the query tile is resident the kernel also computes
 * g_x[r] = q[r,:] . gate_w[x,:] + gate_b[x] for x = 0,1,2 = selected, window, compressed (gate_w [3,D] bf16, gate_b [3]
 * bf16 or NULL, no activation) and writes the three gates to g_slc, g_swa, g_cmp [B,Tq,Hq] bf16.  Replaces, in addition,
 * self.gating = nn.Linear(head_dim, 3) applied at nsa/nsa.py:117.
 * (2) score_mode: 0 = the reference's selection scores (soft-max of the UNSCALED, UNMASKED q.ck over ALL compressed keys,
 * nsa/torch_attention.py:121-125, under which blocks in a query's future can be selected and are then skipped);
 * 1 = causal scores: the compressed branch's own attention probabilities (scaled by `scale`, masked by t >= stride*j +
 * block) summed over the group's heads and pooled, as in the NSA paper; needs causal = 1.  No counterpart in the
 * reference.  Tq = T, q0 = 0 for an unsharded call. */
int nsa_cmp_attn_fwd_gated(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                           float* sel_scores, const void* gate_w, const void* gate_b, void* g_slc, void* g_swa, void* g_cmp,
                           int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride, int causal, float scale,
                           int n_sel, int pool_k, int pool_s, int pool_p, int score_mode, int Tq, int q0, void* stream);
/* Replaces _attention.backward (nsa/triton_attention.py:479-546).  dout [B,T,Hq,D]; delta [B,T,Hq] fp32 =
 * rowsum(o*dout) (times gate if gate != NULL); gate [B,T,Hq] or NULL scales dout per row.
 * dq [B,T,Hq,D] (added to when accumulate_dq); dck,dcv [B,Tc,Hk,D]. */
int nsa_cmp_attn_bwd(const void* q, const void* ck, const void* cv, const float* lse, const void* dout,
                     const float* delta, const void* gate, void* dq, int accumulate_dq, void* dck, void* dcv,
                     void* ws, size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride,
                     int causal, float scale, void* stream);
size_t nsa_cmp_attn_bwd_workspace_bytes(int B, int T, int Tc, int Hk, int D);

/* ---- selected-block + sliding-window attention ----------------------------------------------------
 * Replaces ParallelNSAFunction.forward / parallel_nsa_fwd (nsa/selection_attn.py:90-148, kernel :401-517)
 * and the gated sums of parallel_nsa (:808-811) and NSAAttention.forward (nsa/nsa.py:133).
 * q [B,T,Hq,D]; k,v [B,T,Hkv,D]; idx [B,T,Hkv,S] int32 (idx64 = 0) or int64 (idx64 = 1); counts [B,T,Hkv]
 * int32 or NULL.  Outputs o_slc, lse_slc, and when window > 0 o_swa, lse_swa.  If o != NULL also writes
 * o = g_slc*o_slc + g_swa*o_swa + g_cmp*o_cmp (a NULL tensor drops its term; a NULL gate means 1). */
int nsa_sel_swa_fwd(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    void* o_slc, float* lse_slc, void* o_swa, float* lse_swa, const void* g_slc, const void* g_swa,
                    const void* o_cmp, const void* g_cmp, void* o, int B, int T, int Hq, int Hkv, int D, int S, int BS,
                    int window, float scale, void* stream);
/* Replaces ParallelNSAFunction.backward / parallel_nsa_bwd (nsa/selection_attn.py:572-676: preprocess, dq,
 * block mask and dkv kernels).  The dense block mask is replaced by a reverse index built in ws.
 * Per branch: dout, lse, delta (fp32, = rowsum(o*dout) times gate if given), gate (or NULL).  The window
 * branch is skipped when window == 0.  dq [B,T,Hq,D] (added to when accumulate_dq); dk,dv [B,T,Hkv,D]. */
int nsa_sel_swa_bwd(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                    const void* dout_slc, const float* lse_slc, const float* delta_slc, const void* gate_slc,
                    const void* dout_swa, const float* lse_swa, const float* delta_swa, const void* gate_swa, void* dq,
                    int accumulate_dq, void* dk, void* dv, void* ws, size_t ws_bytes, int B, int T, int Hq, int Hkv,
                    int D, int S, int BS, int window, float scale, void* stream);
size_t nsa_sel_swa_bwd_workspace_bytes(int B, int T, int Hkv, int S, int BS);
/* The larger workspace with which nsa_sel_swa_bwd (and its _sharded / _fused forms; Tq = T when not sharded) takes the
 * selected branch's dQ from the key-major dK/dV kernel: while a key block's dS tile is in shared memory that kernel also
 * forms dS K for the visiting tokens and leaves one [16 heads x D] bf16 tile per (token, slot); a second kernel adds
 * every token's S tiles in slot order (fixed order, no atomics).  This replaces the query-major dQ kernel, i.e. one of
 * the two passes that recompute the selected branch's scores.  Extra bytes: B*Tq*Hkv*S*(4 + Hq/Hkv*D*2).  Used when
 * D = 128, BS = 64 and dq, dk, dv are all requested; with the smaller workspace the query-major kernel runs. */
size_t nsa_sel_swa_bwd_workspace_bytes_dq(int B, int T, int Tq, int Hq, int Hkv, int D, int S, int BS);

/* Measurement aid, no counterpart in the reference: the K/V block gather of nsa_sel_swa_fwd's selected branch (same
 * items, same order, same TMA boxes of [BS keys x D]) with no arithmetic behind it, every SM keeping all of its shared
 * memory in flight.  visited blocks x 2 x BS x D x 2 bytes divided by its run time is the L2 -> SM gather ceiling that
 * the benchmark reports beside the selected-attention kernels.  Needs BS = 64 and S <= 32. */
int nsa_gather_probe(const void* k, const void* v, const void* idx, int idx64, int B, int T, int Hq, int Hkv, int D, int S,
                     int BS, void* stream);

/* ---- query shards (context parallelism) -------------------------------------------------------------
 * No counterpart in the reference (it is single-GPU: neither its modules nor its tests hold distributed code).  The four
 * attention entry points again, for a rank that owns only the queries q0 .. q0+Tq-1 of a T-token sequence while
 * holding the whole K/V (and compressed K/V): every q-indexed tensor (q, o, lse, gates, indices, dout, delta, dq,
 * sel_idx, sel_scores) has Tq rows per batch, row i being sequence position q0+i; k, v, ck, cv, dk, dv, dck, dcv
 * keep their full lengths, and dk/dv/dck/dcv receive only this shard's contribution (sum them over ranks).
 * Needs head_dim 128, 64-key selection blocks and the 5/4/0 pooling geometry. */
int nsa_cmp_attn_fwd_sharded(const void* q, const void* ck, const void* cv, void* o, float* lse, int32_t* sel_idx,
                             float* sel_scores, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride,
                             int causal, float scale, int n_sel, int pool_k, int pool_s, int pool_p, int Tq, int q0,
                             void* stream);
int nsa_cmp_attn_bwd_sharded(const void* q, const void* ck, const void* cv, const float* lse, const void* dout,
                             const float* delta, const void* gate, void* dq, int accumulate_dq, void* dck, void* dcv,
                             void* ws, size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block,
                             int stride, int causal, float scale, int Tq, int q0, void* stream);
int nsa_sel_swa_fwd_sharded(const void* q, const void* k, const void* v, const void* idx, int idx64,
                            const int32_t* counts, void* o_slc, float* lse_slc, void* o_swa, float* lse_swa,
                            const void* g_slc, const void* g_swa, const void* o_cmp, const void* g_cmp, void* o, int B,
                            int T, int Hq, int Hkv, int D, int S, int BS, int window, float scale, int Tq, int q0,
                            void* stream);
/* nsa_sel_swa_fwd_sharded with a workspace (nsa_sel_swa_fwd_workspace_bytes; Tq = T, q0 = 0 when not sharded).  With it,
 * head_dim 128, 64-key blocks, at most 32 selections and a multiple of 16 query heads per KV head, the selected branch
 * runs key-major on the tensor cores: a reverse index of the selection is built, one CTA per key block takes the queries
 * that selected it in batches of 8 tokens x 16 heads (tcgen05 S = Q K^T and P V), every visit leaves a [16 x D] bf16 tile
 * and (max, sum) per row, and a second kernel merges a token's visits in slot order (no atomics).  A block's K and V are
 * then read once per CTA instead of once per visiting query.  Results equal the query-major kernel's up to the bf16
 * rounding of the per-visit tiles.  Without the workspace (ws NULL or too small) this is nsa_sel_swa_fwd_sharded. */
int nsa_sel_swa_fwd_ws(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                       void* o_slc, float* lse_slc, void* o_swa, float* lse_swa, const void* g_slc, const void* g_swa,
                       const void* o_cmp, const void* g_cmp, void* o, void* ws, size_t ws_bytes, int B, int T, int Hq,
                       int Hkv, int D, int S, int BS, int window, float scale, int Tq, int q0, void* stream);
size_t nsa_sel_swa_fwd_workspace_bytes(int B, int T, int Tq, int Hq, int Hkv, int D, int S, int BS);
int nsa_sel_swa_bwd_sharded(const void* q, const void* k, const void* v, const void* idx, int idx64,
                            const int32_t* counts, const void* dout_slc, const float* lse_slc, const float* delta_slc,
                            const void* gate_slc, const void* dout_swa, const float* lse_swa, const float* delta_swa,
                            const void* gate_swa, void* dq, int accumulate_dq, void* dk, void* dv, void* ws,
                            size_t ws_bytes, int B, int T, int Hq, int Hkv, int D, int S, int BS, int window,
                            float scale, int Tq, int q0, void* stream);

/* The two backward entry points above with the row pre-pass folded in (what nsa_rowdot / nsa_rowdot3 compute): instead of
 * taking delta, they take the branch outputs saved by the forward and the ONE upstream gradient `dout` of the gated sum
 * o = g_slc*o_slc + g_swa*o_swa + g_cmp*o_cmp (nsa/nsa.py:133), and they WRITE, per branch x, delta_x = g_x * rowsum(o_x *
 * dout) (fp32 [B,Tq,Hq], also used internally) and dgate_x = rowsum(o_x * dout) (bf16 [B,Tq,Hq], the gate gradient; NULL to
 * skip).  With head_dim 128 the sums are formed inside the tcgen05 dQ kernels while the dO tile is resident (the window
 * kernel serves the selected branch too and runs before it), so o_x and dout are not read by a separate pass; other
 * configurations run the pre-pass kernel first.  Replaces, in addition, parallel_nsa_bwd_kernel_preprocess
 * (nsa/selection_attn.py:520-530), _attn_bwd_preprocess (nsa/triton_attention.py:184-199) and the gate-product gradients
 * of nsa/nsa.py:133.  Tq = T, q0 = 0 for an unsharded call. */
int nsa_sel_swa_bwd_fused(const void* q, const void* k, const void* v, const void* idx, int idx64, const int32_t* counts,
                          const void* o_slc, const void* o_swa, const void* dout, const float* lse_slc, float* delta_slc,
                          const void* gate_slc, void* dgate_slc, const float* lse_swa, float* delta_swa, const void* gate_swa,
                          void* dgate_swa, void* dq, int accumulate_dq, void* dk, void* dv, void* ws, size_t ws_bytes, int B,
                          int T, int Hq, int Hkv, int D, int S, int BS, int window, float scale, int Tq, int q0, void* stream);
int nsa_cmp_attn_bwd_fused(const void* q, const void* ck, const void* cv, const void* o_cmp, const float* lse, const void* dout,
                           float* delta, const void* gate, void* dgate, void* dq, int accumulate_dq, void* dck, void* dcv,
                           void* ws, size_t ws_bytes, int B, int T, int Tc, int Hq, int Hk, int D, int block, int stride,
                           int causal, float scale, int Tq, int q0, void* stream);

/* ---- decode ---------------------------------------------------------------------------------------------
 * No entry point of the reference does this (its module assumes len(q) == len(k), nsa/nsa.py:97); it is the
 * module's forward (nsa/nsa.py:94-135) for ONE new query token per sequence, at position L-1 of a packed, ragged
 * K/V cache, all sequences in ONE kernel launch (one CTA per (sequence, kv head), see csrc/decode.cu).
 * q, o [nseq,Hq,D]; k, v [total_k,Hkv,D]; ck, cv [total_c,Hkv,D] = the compressed cache (nsa_compress_fwd with the
 * Conv1d length rule Tc = (L-block)/stride + 1); cu_k, cu_c: DEVICE int32 [nseq+1] cumulative lengths of k/v and of
 * ck/cv; order: DEVICE int32 [nseq] = the order in which sequences are dealt to the CTAs (pass them longest first for
 * an even load) or NULL.  Gates: either gate_w [3,D] (+ gate_b [3] or NULL), the module's nn.Linear(head_dim, 3) whose rows
 * are selected, window, compressed (nsa/nsa.py:59,117) -- the gates are then computed from q inside the call -- or, with
 * gate_w NULL, precomputed g_slc, g_swa, g_cmp [nseq,Hq] (NULL = 1).  Optional outputs (NULL to skip): the branch outputs o_cmp, o_slc,
 * o_swa [nseq,Hq,D] and lse fp32 [3,nseq,Hq] (compressed, selected, window); idx int32 [nseq,Hkv,n_sel] receives the
 * selected blocks.  max_Tc = the largest per-sequence compressed length (host-known; at most 2048, i.e. caches up to
 * 32 K tokens).  ws: nsa_decode_workspace_bytes(nseq, Hkv) bytes of scratch (the per-warp partial results that a second,
 * small kernel merges in a fixed order).  Needs head_dim 128, 16 query heads per KV head, 64-key blocks, stride 16 /
 * block 32.  Two launches, no host synchronisation, no internal streams: everything is enqueued on `stream`. */
int nsa_decode_fwd(const void* q, const void* k, const void* v, const void* ck, const void* cv, const int32_t* cu_k,
                   const int32_t* cu_c, const int32_t* order, const void* gate_w, const void* gate_b, const void* g_slc,
                   const void* g_swa, const void* g_cmp, void* o, void* o_cmp, void* o_slc, void* o_swa, float* lse,
                   int32_t* idx, void* ws, size_t ws_bytes, int nseq,
                   long long total_k, long long total_c, int max_Tc, int Hq, int Hkv, int D, int block, int stride,
                   int sel_block, int n_sel, int window, float scale, void* stream);
size_t nsa_decode_workspace_bytes(int nseq, int Hkv);

/* ---- helpers --------------------------------------------------------------------------------------
 * delta[r] = (gate ? gate[r] : 1) * sum_d o[r,d]*dout[r,d] (fp32, NULL to skip) and
 * dgate[r] = sum_d o[r,d]*dout[r,d] (bf16, NULL to skip); rows = B*T*Hq.
 * Replaces parallel_nsa_bwd_kernel_preprocess (nsa/selection_attn.py:520-530), _attn_bwd_preprocess
 * (nsa/triton_attention.py:184-199) and the gate gradients of the addcmul at nsa/nsa.py:133. */
int nsa_rowdot(const void* o, const void* dout, const void* gate, float* delta, void* dgate, long long rows, int D,
               void* stream);
/* The gate projection of the module: g_x[r] = q[r,:] . w[x,:] + bias[x] for x = 0,1,2 = selected, window, compressed
 * (w [3,D] bf16, bias [3] bf16 or NULL; no activation), each gate written to its own contiguous [rows] bf16 tensor.
 * Replaces self.gating = nn.Linear(head_dim, 3) applied at nsa/nsa.py:117. */
int nsa_gate_fwd(const void* q, const void* w, const void* bias, void* g_slc, void* g_swa, void* g_cmp, long long rows,
                 int D, void* stream);
/* nsa_rowdot for the three branches in one pass over dout (a NULL o_x drops that branch): delta_x = g_x * rowsum(o_x *
 * dout), dg_x = rowsum(o_x * dout).  Same reference lines as nsa_rowdot. */
int nsa_rowdot3(const void* o_slc, const void* o_swa, const void* o_cmp, const void* dout, const void* g_slc,
                const void* g_swa, const void* g_cmp, float* delta_slc, float* delta_swa, float* delta_cmp, void* dg_slc,
                void* dg_swa, void* dg_cmp, long long rows, int D, void* stream);
/* Backward of the gate projection (the autograd of nn.Linear at nsa/nsa.py:117): dq[r,:] += sum_x dg_x[r] * w[x,:] in
 * place, dw[x,:] = sum_r dg_x[r] * q[r,:], dbias[x] = sum_r dg_x[r] (NULL to skip).  Deterministic: fixed-order
 * partial sums in `workspace` (nsa_gate_bwd_workspace_bytes), no atomics. */
long long nsa_gate_bwd_workspace_bytes(long long rows, int D);
int nsa_gate_bwd(const void* q, const void* dg_slc, const void* dg_swa, const void* dg_cmp, const void* w, void* dq,
                 void* dw, void* dbias, void* workspace, long long workspace_bytes, long long rows, int D, void* stream);
/* o = g0*a0 + g1*a1 + g2*a2 (NULL tensor: term dropped; NULL gate: 1).  nsa/nsa.py:133. */
int nsa_combine(const void* a0, const void* g0, const void* a1, const void* g1, const void* a2, const void* g2,
                void* o, long long rows, int D, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_H_ */
