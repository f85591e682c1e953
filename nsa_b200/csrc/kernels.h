// Internal launcher interface between api.cu (argument checking, C-ABI) and the kernel files.
// All pointers are device pointers; all tensors are contiguous with the layouts given below.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace nsa {

// ---- selected-block attention, query-major (forward and dQ) --------------------------------
struct SelArgs {
  const bf16* q;       // [B,T,Hq,D]
  const bf16* k;       // [B,T,Hkv,D]
  const bf16* v;       // [B,T,Hkv,D]
  const void* idx;     // [B,T,Hkv,S] int32 or int64
  int idx64;           // 1 if idx is int64
  const int* counts;   // [B,T,Hkv] int32 or null
  // forward outputs / backward inputs
  bf16* o;             // [B,T,Hq,D]
  float* lse;          // [B,T,Hq] natural log
  // backward
  const bf16* dout;    // [B,T,Hq,D]
  const float* delta;  // [B,T,Hq]
  const bf16* gate;    // [B,T,Hq] or null: upstream gradient is gate * dout
  bf16* dq;            // [B,T,Hq,D]
  int accumulate;      // dq += instead of =
  int B, T, Hq, Hkv, S, BS;
  float scale;
  int Tq, q0;          // queries are the tokens q0 .. q0+Tq-1 of the T-long sequence (q-indexed tensors hold Tq rows)
};
int launch_sel_fwd(const SelArgs& a, int D, cudaStream_t s);
int launch_sel_dq(const SelArgs& a, int D, cudaStream_t s);
int sel_status(int* out);
// one item per warp, whole 64-key blocks (sel_block.cu); used when sel_block_supported()
bool sel_block_supported(const SelArgs& a, int D);
int launch_sel_block(const SelArgs& a, int D, bool bwd, cudaStream_t s);
int sel_block_status(int* out);
// the same gather with nothing behind it (gather_probe.cu): the bandwidth ceiling quoted for these kernels
int launch_gather_probe(const SelArgs& a, int D, cudaStream_t s);
int gather_probe_status(int* out);

// ---- dense query-major attention: sliding window (mode 0) and compressed (mode 1) ---------
struct DenseArgs {
  int mode;            // 0 sliding window over k,v [B,Lk=T,Hkv,D]; 1 compressed over ck,cv [B,Lk=Tc,Hk,D]
  const bf16* q;       // [B,T,Hq,D]
  const bf16* k;
  const bf16* v;
  bf16* o;             // [B,T,Hq,D]
  float* lse;          // [B,T,Hq] natural log; -inf for rows without a visible key
  const bf16* dout;
  const float* delta;
  const bf16* gate;
  bf16* dq;
  int accumulate;
  int B, T, Lk, Hq, Hk;
  int window;          // mode 0
  int cblock, cstride; // mode 1: key j visible to query t iff t >= j*cstride + cblock
  int causal;          // mode 1
  float scale;
  // mode 1 forward only: block selection fused behind the attention
  int score_mode;      // selection scores: 0 = the reference's (soft-max of the UNSCALED, UNMASKED q.ck over all compressed
                       // keys, nsa/torch_attention.py:121-125); 1 = causal: the compressed branch's own attention
                       // probabilities (scaled, masked), so no block that starts in a query's future can be selected
  int n_sel;           // 0 = no selection
  int pool_k, pool_s, pool_p, n_pool;
  int* sel_idx;        // [B,T,Hq/16,n_sel] int32
  float* sel_scores;   // optional [B,Hq/16,T,n_pool] fp32 dump of the pooled scores, or null
  int Tq, q0;          // query shard: q-indexed tensors hold Tq rows per batch, row i is sequence position q0+i
  // optional, two-tile tcgen05 forward: the module's gate projection computed from the resident query tiles (null = off)
  const bf16* gate_w;  // mode 1: [3,D] gate projection weight (rows: selected, window, compressed); writes g_out
  const bf16* gate_b;  // [3] or null
  bf16* g_out[3];      // [B,Tq,Hq] each
  // optional, dQ kernels (tcgen05): the row pre-pass of the backward folded in.  With pre_o[0] set the kernel computes
  // rowsum(o * dO) itself for its own branch ([0]) and, if given, a second branch ([1]) whose dQ kernel runs later:
  // pre_delta[x] = gate_x * rowsum (fp32, also what this kernel uses as delta), pre_dgate[x] = rowsum (bf16, gate gradient)
  const bf16* pre_o[2];
  const bf16* pre_gate[2];
  float* pre_delta[2];
  bf16* pre_dgate[2];
};
int launch_dense_fwd(const DenseArgs& a, int D, cudaStream_t s);
int launch_dense_dq(const DenseArgs& a, int D, cudaStream_t s);
int dense_status(int* out);
// tcgen05 forward for head_dim 128 (and, for selection, the 5/4/0 pooling of the default block sizes)
bool dense_fwd_tc_supported(const DenseArgs& a, int head_dim);
// two query tiles per CTA, P kept in tensor memory (dense_fwd2_tc.cu)
int launch_dense_fwd2_tc(const DenseArgs& a, cudaStream_t s);
int dense_tc2_status(int* out);
int launch_dense_dq_tc(const DenseArgs& a, cudaStream_t s);
int dense_dq_tc_status(int* out);

// ---- key/value-major backward (dK,dV of selected + sliding window; dCK,dCV of compressed) ---
struct KvArgs {
  int mode;               // 0 selected (+ window) over k,v; 1 compressed
  const bf16* q;          // [B,T,Hq,D]
  const bf16* k;          // [B,Lk,Hk,D]
  const bf16* v;
  // branch A: selected (mode 0) or compressed (mode 1); branch B: sliding window (mode 0 only)
  const bf16* dout_a;  const float* lse_a;  const float* delta_a;  const bf16* gate_a;
  const bf16* dout_b;  const float* lse_b;  const float* delta_b;  const bf16* gate_b;
  const int* rev_ptr;     // [B,Hk,NB+1]   mode 0: CSR over selection blocks
  const int* rev_tok;     // [B,Hk,cap]    tokens ascending inside each block's list
  long long rev_cap;
  bf16* dk;               // [B,Lk,Hk,D]
  bf16* dv;
  bf16* dq_part;          // mode 0, optional: the selected branch's dQ as per-visit partial tiles [B,Hk,rev_cap,G16][16][D]
                          // (position = place in the reverse-index list), summed later by launch_sel_dq_reduce
  float* part;            // mode 1 workspace: [2][nseg][B,Lk,Hk,D] fp32
  int nseg, seg_len;
  int B, T, Lk, Hq, Hk, BS, window;
  int cblock, cstride, causal;
  float scale;
  int Tq, q0;             // query shard (rev_tok holds sequence positions)
};
int launch_kv_bwd(const KvArgs& a, int D, cudaStream_t s);
int kv_status(int* out);
// tcgen05 engine for head_dim 128 and 64-key blocks (same arguments and results)
int launch_kv_bwd_tc(const KvArgs& a, cudaStream_t s);
int kv_tc_status(int* out);

// ---- batched decode (one new query token per sequence of a packed cache; decode.cu) ------------------------------
struct DecodeArgs {
  const bf16* q;        // [nseq,Hq,D]
  const bf16* k;        // [total_k,Hkv,D]
  const bf16* v;
  const bf16* ck;       // [total_c,Hkv,D] compressed cache
  const bf16* cv;
  const int* cu_k;      // [nseq+1] device
  const int* cu_c;      // [nseq+1] device
  const int* order;     // [nseq] device: order in which the sequences are dealt to the CTAs (longest first), or null
  const bf16* gate_w;   // [3,D] gate projection (rows: selected, window, compressed): gates computed from q; or null
  const bf16* gate_b;   // [3] or null
  const bf16* g_slc;    // [nseq,Hq] precomputed gates (used when gate_w is null), or null (= 1)
  const bf16* g_swa;
  const bf16* g_cmp;
  bf16* o;              // [nseq,Hq,D] gated sum
  bf16* o_cmp;          // branch outputs, each may be null
  bf16* o_slc;
  bf16* o_swa;
  float* lse;           // [3,nseq,Hq] (compressed, selected, window) or null
  int* idx;             // [nseq,Hkv,n_sel]
  int nseq, Hq, Hkv, D, n_sel, window, cblock, cstride, sel_block;
  long long total_k, total_c;
  int max_Tc;
  float scale;
  float* part;          // workspace of decode_workspace_bytes(): per (item, branch, consumer warp) partial results
  size_t part_bytes;
};
size_t decode_workspace_bytes(int nseq, int Hkv);
int launch_decode(const DecodeArgs& a, cudaStream_t s);
int decode_status(int* out);

// ---- compression ------------------------------------------------------------------------------
struct CompressArgs {
  const bf16* x;        // [tok,H,D]
  const bf16* w;        // [l*D, D]  row j*D+c, column o
  const bf16* bias;     // [D] or null
  bf16* y;              // [out_tok,H,D]
  const int* cu_in;     // [nseq+1] device
  const int* cu_out;    // [nseq+1] device
  int nseq, H, D, l, d, max_out;   // max_out: longest compressed sequence
  // backward
  const bf16* dy;       // [out_tok,H,D]
  bf16* dx;             // [tok,H,D]
  float* dw;            // [l*D, D] fp32
  float* dbias;         // [D] fp32 or null
  float* ws;            // workspace for dw partials: [nseq*H][l*D*D] fp32
  int max_in;           // longest input sequence
  int total_out;
};
int launch_compress_fwd(const CompressArgs& a, cudaStream_t s);
int launch_compress_bwd(const CompressArgs& a, cudaStream_t s);
int compress_status(int* out);
// dW partials in the library's fixed device array instead of a caller workspace
int launch_compress_bwd_static(const CompressArgs& a, cudaStream_t s);
long long compress_static_scratch_floats();

// tcgen05 GEMM for equal-length sequences (x [B,T,H,D], T % d == 0)
int launch_compress_fwd_uniform(const bf16* x, const bf16* w, const bf16* bias, bf16* y, int B, int T, int H, int D, int l,
                                int d, cudaStream_t s);
int compress_tc_status(int* out);

// ---- small helpers ----------------------------------------------------------------------------
// delta[r] = (gate ? gate[r] : 1) * sum_d o[r,d]*dout[r,d];  dgate[r] = sum_d o[r,d]*dout[r,d]
int launch_rowdot(const bf16* o, const bf16* dout, const bf16* gate, float* delta, bf16* dgate, long long rows, int D,
                  cudaStream_t s);
// o = g0*a0 + g1*a1 + g2*a2  (null pairs skipped); gates [rows], tensors [rows,D]
// gate projection, fused row pre-pass of the backward, gate backward (gate.cu)
int launch_gate_fwd(const bf16* q, const bf16* w, const bf16* bias, bf16* g0, bf16* g1, bf16* g2, long long rows, int D,
                    cudaStream_t s);
int launch_rowdot3(const bf16* const o[3], const bf16* dout, const bf16* const gate[3], float* const delta[3],
                   bf16* const dgate[3], long long rows, int D, cudaStream_t s);
long long gate_bwd_workspace_bytes(long long rows, int D);
int launch_gate_bwd(const bf16* q, const bf16* dg0, const bf16* dg1, const bf16* dg2, const bf16* w, bf16* dq, bf16* dw,
                    bf16* db, float* workspace, long long rows, int D, cudaStream_t s);
int launch_combine(const bf16* a0, const bf16* g0, const bf16* a1, const bf16* g1, const bf16* a2, const bf16* g2,
                   bf16* o, long long rows, int D, cudaStream_t s);
// reverse index of the selection: for every (b,h,block) the ascending list of tokens selecting it.
struct RevArgs {
  const void* idx; int idx64; const int* counts;
  int B, T, H, S, BS, NB;
  int* hist;      // workspace [B,H,NB(chunks),NB] int32
  int* rev_ptr;   // [B,H,NB+1]
  int* rev_tok;   // [B,H,cap]
  long long cap;  // Tq*S
  int Tq, q0;     // query shard: idx/counts hold Tq rows per batch; T is the key sequence length
  int* inv;       // optional [B,Tq,H,S]: for every valid (row, slot) its position in the (b,h) list of rev_tok
};
int launch_build_rev(const RevArgs& a, cudaStream_t s);
#ifdef __CUDACC__
// The block that slot s of a row selects, or -1 if the slot does not count (beyond the row's count, out of range, or a
// block that starts after the token).  `row` is the local (batch, token, head) row of idx/counts, `t` the token's
// sequence position.  Every kernel that walks the selection uses this one rule.
__device__ __forceinline__ int rev_block(const RevArgs& a, long long row, int s, int t) {
  int cnt = a.S;
  if (a.counts) cnt = min(cnt, a.counts[row]);
  if (s >= cnt) return -1;
  long long v = a.idx64 ? reinterpret_cast<const long long*>(a.idx)[row * a.S + s]
                        : (long long)reinterpret_cast<const int*>(a.idx)[row * a.S + s];
  if (v < 0 || v >= a.NB || v * a.BS > t) return -1;
  return (int)v;
}
#endif
// Selected attention forward, key-major (sel_fwd_kv_tc.cu): one CTA per 64-key block, the queries that selected it in
// batches of 8 tokens x 16 heads from the reverse index; per visit a [16 x D] bf16 tile of unnormalised output and
// (max, sum) per row, merged per token in slot order by a second kernel.
struct SelKvArgs {
  const bf16* q;        // [B,Tq,Hq,D]
  const bf16* k;        // [B,T,Hk,D]
  const bf16* v;
  bf16* o;              // [B,Tq,Hq,D]
  float* lse;           // [B,Tq,Hq] natural log
  const int* rev_ptr;   // reverse index (launch_build_rev, with inv)
  const int* rev_tok;
  long long rev_cap;
  bf16* part;           // [B,Hk,rev_cap,G16][16][D]
  float* stats;         // [B,Hk,rev_cap,G16][16][2]: row maximum (log2 domain, scaled) and sum of probabilities
  int B, T, Tq, q0, Hq, Hk, S, BS;
  float scale;
};
bool sel_fwd_kv_supported(const SelKvArgs& a, int D);
int launch_sel_fwd_kv(const SelKvArgs& a, const RevArgs& r, cudaStream_t s);
int sel_fwd_kv_status(int* out);
// dq[(b,t), 16-head group] (+)= scale * sum over the valid slots s of part[(b,h) list position inv[row,s]] (fixed slot
// order).  part holds one [16 heads x D] bf16 tile per (list position, 16-head sub-group), written by the kv-major
// backward; dq rows of a (token, group) are the same contiguous tile.
int launch_sel_dq_reduce(const RevArgs& a, const bf16* part, bf16* dq, int Hq, int D, float scale, int accumulate,
                         cudaStream_t s);
// out(bf16)[i] = sum over valid segments of part[seg][i]
int launch_reduce_segments(const float* part, bf16* out, int nseg, long long n_per_seg, int q0, int Tq, int Lk, int Hk,
                           int D, int seg_len, int cblock, int cstride, int causal, cudaStream_t s);
int misc_status(int* out);

int num_sms();

}  // namespace nsa
