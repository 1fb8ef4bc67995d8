/*
 * daisy_b200 -- C ABI of the B200 (sm_100a) attention hot path.
 *
 * Every entry point takes plain pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*).  Unless its comment says otherwise an entry
 * point allocates no device memory and never synchronises: it validates its
 * arguments on the host, enqueues kernels on `stream` and returns.  Return
 * value: DAISY_OK (0) or a negative DAISY_E* code; daisy_b200_strerror() maps it
 * to text.  Device-side problems (a bounded wait that ran out) are reported
 * asynchronously through `status_word`, a caller-owned int in device memory
 * that kernels only ever write a non-zero DAISY_E* code into (the caller zeroes
 * it and reads it after synchronising).  `status_word` may be NULL.
 *
 * All tensors are bf16 unless stated; strides are in ELEMENTS.  head_dim D must
 * be 128.  The citations name the reference (jonathanmiddleton/daisy) code each
 * entry point stands in for.
 */
#ifndef DAISY_B200_H
#define DAISY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DAISY_B200_VERSION 100

/* status codes */
#define DAISY_OK            0
#define DAISY_EINVAL       -1   /* bad argument (null pointer, non-positive size, bad flag)        */
#define DAISY_EUNSUPPORTED -2   /* shape the kernels do not implement (head_dim != 128, ...)       */
#define DAISY_EALIGN       -3   /* pointer or stride not 16-byte aligned                            */
#define DAISY_EWORKSPACE   -4   /* workspace too small                                              */
#define DAISY_ECUDA        -5   /* a CUDA runtime/driver call failed (launch, tensor-map encode)   */
#define DAISY_ETIMEOUT     -6   /* device side: a bounded barrier wait ran out (status_word only)  */
#define DAISY_ENODEV       -7   /* no CUDA device / not an sm_100 device                            */

/* transform flags (what is applied to raw projected q,k,v on load) */
#define DAISY_NORM_Q     1u     /* weightless RMS norm over D, eps given by the caller             */
#define DAISY_NORM_K     2u
#define DAISY_NORM_V     4u
#define DAISY_ROPE       8u     /* rotate halves (x[:D/2], x[D/2:]) of q and k by cos/sin tables    */
#define DAISY_QKV_DEFAULT 15u
#define DAISY_WRITE_RING 16u    /* decode: store the new k,v row into ring slot t % cap            */
#define DAISY_OUT_BTHD   32u    /* qkv_prep: outputs keep the [B,T,H,D] memory order (default [B,H,T,D]) */
#define DAISY_KV_BHTD    64u    /* swa_prefill_fwd: k_out/v_out memory order [B,H,T,D] (default [B,T,H,D]) */
#define DAISY_Q_IN_KERNEL 128u  /* swa_prefill_fwd: normalise / rotate Q inside the attention kernel (on load) */
#define DAISY_BOUNDED_QK  256u  /* swa_attend: the caller guarantees |q_i . k_j| * scale * log2(e) <= 60 for every pair
                                   (true for RMS-normalised q and k with scale * D <= 41); selects the kernel that
                                   needs no running maximum.  swa_prefill_fwd sets it itself when it normalises q and k. */
/* KDA flags */
#define DAISY_CACHE_FP16 1024u  /* decode entries: the ring holds float16 rows (the reference Generator's default cache dtype,
                                   inference/generate.py:62) instead of bf16; q, k, v and the output stay bf16 */
#define DAISY_WINDOW_BLOCKS 512u /* swa_attend / swa_prefill_fwd: `window` counts blocks of 128 tokens: key block >= query block -
                                   window + 1 (with causality and documents token-exact inside), the mask the flex-attention
                                   BlockMasks of DaisyCore.create_blockmasks select (models/daisy/daisy_core.py:182-229)     */
#define DAISY_KDA_L2NORM_QK 1u  /* L2-normalise q and k over K inside the kernel (eps 1e-6)         */
#define DAISY_KDA_OUT_FP32  2u  /* `o` is float32 instead of bf16                                   */
#define DAISY_KDA_GATE_ROUND_BF16 1u  /* kda_gate: round the result to bf16 first (what the reference's cast of the
                                         gate to a bf16 activation dtype does), then store it as float32     */

#define DAISY_KDA_CONV_SILU 1u  /* kda_short_conv: apply SiLU to the convolution result             */
#define DAISY_KDA_NORM_SIGMOID 0        /* kda_out_norm gate modes: y = norm(o) * w * sigmoid(g)                          */
#define DAISY_KDA_NORM_SWISH 1          /*   y = norm(o) * w * g * sigmoid(g)                                            */
#define DAISY_KDA_NORM_SWISH_SIGMOID 2  /*   y = bf16(norm(o) * w * g * sigmoid(g)) * bf16(sigmoid(g)): what the reference's
                                             CompilableFusedRMSNormGated evaluates (models/daisy/attention_kimi.py:52-60:
                                             rms_norm_gated with its default swish gate, then a second sigmoid factor) */

int         daisy_b200_version(void);
const char* daisy_b200_strerror(int code);
/* Number of SMs of the current device (0 if there is none). */
int         daisy_b200_sm_count(void);

/* ---------------------------------------------------------------------------------------------
 * q/k/v preparation: RMS-norm q,k,v over D and RoPE q,k, writing [B,H,T,D]-contiguous copies.
 * Replaces the elementwise tail of CausalSelfAttention._calc_qkv
 * (models/daisy/attention.py:121-125; norm = models/daisy/functional.py:6-7;
 * _apply_rope = models/daisy/attention.py:16-20).
 *   q,k,v      raw projections, logical [B,T,H,D], strides (s_b,s_t,s_h) each, D contiguous
 *   cos,sin    float32 [T, D/2], row t = position of token t
 *   *_out      [B,H,T,D] contiguous, or [B,T,H,D] contiguous with DAISY_OUT_BTHD (a pure streaming
 *              pass); any of the three pairs (in,out) may be NULL together
 *   ve         NULL, or the layer's value embedding, logical [B,T,H,D] bf16 with strides: the value-embedding
 *              gate of _qkv_common (models/daisy/attention.py:129-136) is applied to the normalised v,
 *              v' = g * norm(v) + (1 - g) * ve,  g = sigmoid(*ve_gate_logit)  (a float32 scalar in device memory,
 *              the module's g_ve parameter)
 */
int daisy_b200_qkv_prep(const void* q, const void* k, const void* v,
                        int64_t q_sb, int64_t q_st, int64_t q_sh,
                        int64_t k_sb, int64_t k_st, int64_t k_sh,
                        int64_t v_sb, int64_t v_st, int64_t v_sh,
                        const float* cos, const float* sin,
                        void* q_out, void* k_out, void* v_out,
                        const void* ve, int64_t ve_sb, int64_t ve_st, int64_t ve_sh, const float* ve_gate_logit,
                        int B, int T, int H, int D, float eps, unsigned flags, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The merged QKV projection with its element-wise tail fused: replaces F.linear(x, qkvo_w[:3].flatten(0,1)),
 * the head split and the norm / RoPE of CausalSelfAttention._calc_qkv in one kernel
 * (models/daisy/attention.py:116-127), i.e. the GEMM plus daisy_b200_qkv_prep.
 *   x          [B*T, dim] bf16, row stride ldx (elements)
 *   w_qkv      [3*H*D, dim] bf16, row stride ldw: rows h*D.. of the first H*D rows are head h of q, then k, then v
 *              (the layout of qkvo_w[:3].flatten(end_dim=1))
 *   q_out,k_out,v_out   [B,T,H,D] bf16 contiguous, normalised (flags) and rotated (q, k)
 *   ve, ve_ld, ve_gate_logit   NULL, or the value embedding [B*T, H*D] bf16 (row stride ve_ld) and the gate
 *              parameter (float32 scalar in device memory): v' = g * norm(v) + (1 - g) * ve, g = sigmoid(gate)
 *              (models/daisy/attention.py:129-136)
 * dim must be a multiple of 64, D = 128.  flags: DAISY_NORM_Q | DAISY_NORM_K | DAISY_NORM_V | DAISY_ROPE.
 */
int daisy_b200_qkv_gemm(const void* x, int64_t ldx, const void* w_qkv, int64_t ldw,
                        const float* cos, const float* sin,
                        void* q_out, void* k_out, void* v_out,
                        const void* ve, int64_t ve_ld, const float* ve_gate_logit,
                        int B, int T, int H, int D, int dim, float eps, unsigned flags,
                        int* status_word, void* stream);

/* The same projection for a prompt whose keys and values also enter the ring-buffer KV cache: besides k_out, v_out the
 * epilogue stores rows t >= ring_first of k' and v' straight into slot t % cap of one layer of the ring (logical
 * [B,H,cap,D], element strides r_sb, r_sh, r_sr; bf16 rows, or float16 with DAISY_CACHE_FP16 in flags).  Replaces the
 * stacking of the per-layer k, v in DaisyCore.prefill (models/daisy/daisy_core.py:358-369) followed by
 * KVCache.bulk_write_packed (inference/kv_cache.py:57-68), which keeps the last min(T, cap - 1) rows: pass
 * ring_first = T - min(T, cap - 1).  T - ring_first must not exceed cap.  ring_k = ring_v = NULL: no ring output. */
int daisy_b200_qkv_gemm_ring(const void* x, int64_t ldx, const void* w_qkv, int64_t ldw,
                             const float* cos, const float* sin,
                             void* q_out, void* k_out, void* v_out,
                             const void* ve, int64_t ve_ld, const float* ve_gate_logit,
                             void* ring_k, void* ring_v, int64_t r_sb, int64_t r_sh, int64_t r_sr,
                             int cap, int ring_first,
                             int B, int T, int H, int D, int dim, float eps, unsigned flags,
                             int* status_word, void* stream);

/* C[M,N] = X[M,K] W[N,K]^T, bf16 in and out, fp32 accumulation: F.linear(y, qkvo_w[3]), the output projection
 * (models/daisy/attention.py:149).  K a multiple of 64, N a multiple of 128; ld* are row strides in elements. */
int daisy_b200_gemm_nt(const void* x, int64_t ldx, const void* w, int64_t ldw, void* c, int64_t ldc,
                       int M, int N, int K, int* status_word, void* stream);

/* y[M,N] = x[M,K] W[N,K]^T for M <= 64 rows: the projections of a single decode token, F.linear(x, qkvo_w[:3]
 * flattened) and F.linear(y, qkvo_w[3]) with x [B,1,dim] (models/daisy/attention.py:119,201).  bf16 in and out, fp32
 * accumulation; weight-streaming (HBM-bound), no tensor cores.  K a multiple of 8; ld* are row strides in elements. */
int daisy_b200_gemm_skinny(const void* x, int64_t ldx, const void* w, int64_t ldw, void* y, int64_t ldy,
                           int M, int N, int K, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Sliding-window causal softmax attention, prefill form.
 * Replaces CausalSelfAttention._sdpa_common between the two projections
 * (models/daisy/attention.py:141-148) with the mask of build_attn_mask
 * (models/daisy/daisy_core.py:53-69): key k is visible to query q iff 0 <= q - k < window and
 * both lie in the same document; window <= 0 means plain causal.  Also produces what prefill()
 * returns for the cache (models/daisy/attention.py:173-179).
 *   doc_start  NULL (one document) or int32: doc_start[b * doc_sb + t] = first position of the document
 *              of token t, non-decreasing in t; doc_sb = 0 shares one row over the batch.  For the
 *              reference's numbering (docs = (input_seq == eos).cumsum(0), an EOS token opens the next
 *              document) that is the position of the last EOS at or before t, else 0.
 *   q,k,v      raw projections, logical [B,T,H,D] with strides as above
 *   out        [B,T,H,D] with strides (o_sb,o_st,o_sh)
 *   k_out,v_out  normalised/rotated k and v; memory order [B,T,H,D] (what the reference returns: a
 *              [B,H,T,D]-shaped view of that memory) or, with DAISY_KV_BHTD, [B,H,T,D] contiguous;
 *              may be NULL (then the copies live in the workspace only)
 *   workspace  daisy_b200_swa_prefill_workspace_bytes(B,T,H,D) bytes, 256-byte aligned
 */
size_t daisy_b200_swa_prefill_workspace_bytes(int B, int T, int H, int D);
int daisy_b200_swa_prefill_fwd(const void* q, const void* k, const void* v,
                               int64_t q_sb, int64_t q_st, int64_t q_sh,
                               int64_t k_sb, int64_t k_st, int64_t k_sh,
                               int64_t v_sb, int64_t v_st, int64_t v_sh,
                               const float* cos, const float* sin,
                               void* out, int64_t o_sb, int64_t o_st, int64_t o_sh,
                               void* k_out, void* v_out,
                               int B, int T, int H, int D, int window, float scale, float eps,
                               const int32_t* doc_start, int64_t doc_sb,
                               unsigned flags, void* workspace, size_t workspace_bytes,
                               int* status_word, void* stream);

/* The attention core alone on already-prepared q,k,v, logical [B,T,H,D] with strides
 * (s_b,s_t,s_h), D contiguous -- any memory order (what F.scaled_dot_product_attention(q_,k_,v_,
 * attn_mask=M,scale=...) computes at models/daisy/attention.py:145).  flags: 0 or DAISY_BOUNDED_QK. */
int daisy_b200_swa_attend(const void* q, const void* k, const void* v,
                          int64_t q_sb, int64_t q_st, int64_t q_sh,
                          int64_t k_sb, int64_t k_st, int64_t k_sh,
                          int64_t v_sb, int64_t v_st, int64_t v_sh,
                          void* out, int64_t o_sb, int64_t o_st, int64_t o_sh,
                          int B, int T, int H, int D, int window, float scale,
                          const int32_t* doc_start, int64_t doc_sb,
                          unsigned flags, int* status_word, void* stream);

/* The same attention core, also returning what the backward pass needs: lse2 [B,H,T] float32, the base-2 logarithm of
 * each row's softmax denominator in the kernel's exp2 domain, P[q,k] = 2^(logit[q,k] * log2(e) - lse2[q]). */
int daisy_b200_swa_attend_lse(const void* q, const void* k, const void* v,
                              int64_t q_sb, int64_t q_st, int64_t q_sh,
                              int64_t k_sb, int64_t k_st, int64_t k_sh,
                              int64_t v_sb, int64_t v_st, int64_t v_sh,
                              void* out, int64_t o_sb, int64_t o_st, int64_t o_sh, float* lse2,
                              int B, int T, int H, int D, int window, float scale,
                              const int32_t* doc_start, int64_t doc_sb,
                              unsigned flags, int* status_word, void* stream);

/* Backward pass of the attention core: what autograd computes for F.scaled_dot_product_attention /
 * flex_attention inside CausalSelfAttention.forward during training (models/daisy/attention.py:141-162), for the same
 * masks as the forward (window in tokens, or in 128-token blocks with DAISY_WINDOW_BLOCKS; documents).
 *   q,k,v      the PREPARED tensors the forward consumed, o its output, d_o the incoming gradient: logical [B,T,H,D]
 *              bf16 with strides (s_b, s_t, s_h) each (o: o_s*, d_o: g_s*)
 *   lse2       [B,H,T] float32 from daisy_b200_swa_attend_lse
 *   dq,dk,dv   gradients w.r.t. the prepared q, k, v: [B,T,H,D] bf16 contiguous
 *   workspace  daisy_b200_swa_attend_bwd_workspace_bytes(B,T,H) bytes
 * Three launches (row-wise delta = sum_d dO O; a key-block-stationary kernel for dK, dV; a query-block-stationary
 * kernel for dQ); no atomics: results are bitwise reproducible. */
size_t daisy_b200_swa_attend_bwd_workspace_bytes(int B, int T, int H);
int daisy_b200_swa_attend_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                              int64_t q_sb, int64_t q_st, int64_t q_sh,
                              int64_t k_sb, int64_t k_st, int64_t k_sh,
                              int64_t v_sb, int64_t v_st, int64_t v_sh,
                              int64_t o_sb, int64_t o_st, int64_t o_sh,
                              int64_t g_sb, int64_t g_st, int64_t g_sh,
                              const float* lse2, void* dq, void* dk, void* dv,
                              int B, int T, int H, int D, int window, float scale,
                              const int32_t* doc_start, int64_t doc_sb, unsigned flags,
                              void* workspace, size_t workspace_bytes, int* status_word, void* stream);

/* Backward of daisy_b200_qkv_prep (the norm / RoPE tail of _calc_qkv, models/daisy/attention.py:121-125, under
 * autograd): q,k,v are the RAW projections the forward read (strides as there), d*_p the gradients w.r.t. the prepared
 * tensors ([B,T,H,D] bf16 contiguous), d* receive the gradients w.r.t. the raw projections ([B,T,H,D] bf16 contiguous).
 * Any of the three triples may be NULL together.  flags: DAISY_NORM_Q | DAISY_NORM_K | DAISY_NORM_V | DAISY_ROPE. */
int daisy_b200_qkv_prep_bwd(const void* q, const void* k, const void* v,
                            int64_t q_sb, int64_t q_st, int64_t q_sh,
                            int64_t k_sb, int64_t k_st, int64_t k_sh,
                            int64_t v_sb, int64_t v_st, int64_t v_sh,
                            const float* cos, const float* sin,
                            const void* dq_p, const void* dk_p, const void* dv_p,
                            void* dq, void* dk, void* dv,
                            int B, int T, int H, int D, float eps, unsigned flags, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Sliding-window decode step over a ring-buffer KV cache, split-KV.
 * Replaces CausalSelfAttention.step between the projections (models/daisy/attention.py:183-200)
 * together with KVCache.view / KVCache.write for one layer (inference/kv_cache.py:26-51):
 * the ring is read in place, no chronological copy is made.
 *   q_new,k_new,v_new  raw projections of the new token, logical [B,1,H,D], strides (s_b,s_h)
 *   kcache,vcache      one layer of the ring, logical [B,H,cap,D], strides (c_sb,c_sh,c_sr);
 *                      token p lives in row p % cap (inference/kv_cache.py:47-50)
 *   t                  tokens already in the ring (KVCache.t); the new token has index t
 *   window             attends the last r = min(t, cap, window-1) ring rows plus the new row
 *                      (models/daisy/attention.py:192-195); window <= 0: r = min(t, cap)
 *   cos_row,sin_row    float32 [D/2], the RoPE table row of position `pos` (= t in the Generator)
 *   out                [B,1,H,D] with strides (o_sb,o_sh)
 *   k_new_out,v_new_out  normalised/rotated new row, [B,1,H,D] contiguous, may be NULL
 *   flags              transform flags | DAISY_WRITE_RING
 *   workspace          daisy_b200_swa_decode_workspace_bytes(B,H,D,splits) bytes (float partials)
 *   splits             KV splits per (b,h); daisy_b200_swa_decode_splits() suggests a value
 * A plain chronological context [B,n,H,D] is the special case cap = n, t = n, strides of that
 * view, without DAISY_WRITE_RING.
 */
int    daisy_b200_swa_decode_splits(int B, int H, int ctx_rows, int sm_count);
size_t daisy_b200_swa_decode_workspace_bytes(int B, int H, int D, int splits);
int daisy_b200_swa_decode_step(const void* q_new, const void* k_new, const void* v_new,
                               int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                               int64_t v_sb, int64_t v_sh,
                               void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                               int64_t t, int cap, int window,
                               const float* cos_row, const float* sin_row,
                               void* out, int64_t o_sb, int64_t o_sh,
                               void* k_new_out, void* v_new_out,
                               int B, int H, int D, float scale, float eps, unsigned flags,
                               void* workspace, size_t workspace_bytes, int splits,
                               int* status_word, void* stream);

/* The same step with the position in DEVICE memory, for CUDA-graph replays of Generator._step
 * (inference/generate.py:231-248): *t_dev (int64) is read by the kernels, so one captured launch sequence serves
 * every token; the caller advances *t_dev on the stream after the last layer.  cos_table / sin_table are the
 * table bases ([table_rows, D/2] float32); the row is *t_dev (a position past the table writes DAISY_EINVAL to
 * the status word and uses the last row).  `splits` must be chosen for the longest context,
 * min(cap, window - 1) rows. */
int daisy_b200_swa_decode_step_dev(const void* q_new, const void* k_new, const void* v_new,
                                   int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                   int64_t v_sb, int64_t v_sh,
                                   void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                   const int64_t* t_dev, int cap, int window,
                                   const float* cos_table, const float* sin_table, int table_rows,
                                   void* out, int64_t o_sb, int64_t o_sh,
                                   void* k_new_out, void* v_new_out,
                                   int B, int H, int D, float scale, float eps, unsigned flags,
                                   void* workspace, size_t workspace_bytes, int splits,
                                   int* status_word, void* stream);

/* The decode step as ONE launch: the last split CTA of a (batch, head) to finish merges that pair's partials itself
 * (a ticket per pair in the workspace), so a decode layer is projection -> this -> projection.  Same arguments as
 * daisy_b200_swa_decode_step plus:
 *   t_dev        NULL: `t` is the position and cos / sin are the table ROWS of that position; non-NULL: the position is
 *                read from *t_dev on the device and cos / sin are the table bases with table_rows rows (the form of
 *                daisy_b200_swa_decode_step_dev, for CUDA-graph replays)
 *   ve, ve_sb, ve_sh, ve_gate_logit   NULL, or the layer's value embedding for the new token, logical [B,1,H,D] bf16:
 *                v = g * norm(v) + (1 - g) * ve, g = sigmoid(*ve_gate_logit) (models/daisy/attention.py:132-135); needs
 *                DAISY_NORM_V in flags
 *   workspace    daisy_b200_swa_decode_fused_workspace_bytes(B,H,D,splits) bytes; its last B*H ints (the tickets)
 *                must be ZERO before the first call and are left zero by every call */
size_t daisy_b200_swa_decode_fused_workspace_bytes(int B, int H, int D, int splits);
int daisy_b200_swa_decode_step_fused(const void* q_new, const void* k_new, const void* v_new,
                                     int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                     int64_t v_sb, int64_t v_sh,
                                     void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                     int64_t t, const int64_t* t_dev, int cap, int window,
                                     const float* cos, const float* sin, int table_rows,
                                     void* out, int64_t o_sb, int64_t o_sh,
                                     void* k_new_out, void* v_new_out,
                                     const void* ve, int64_t ve_sb, int64_t ve_sh, const float* ve_gate_logit,
                                     int B, int H, int D, float scale, float eps, unsigned flags,
                                     void* workspace, size_t workspace_bytes, int splits,
                                     int* status_word, void* stream);

/* The same decode step for callers that cannot allocate device memory (no counterpart in the reference;
 * it exists for embedders: code inside a stream capture, plugins under a pool allocator that forbids
 * cudaMalloc after start-up, FFI hosts that only hold the tensors they were given).  The split partials go
 * to a fixed 2.1 MB array inside the library instead of a caller workspace, so B * H * splits must not exceed
 * daisy_b200_swa_decode_static_capacity() (4096) -- beyond that the call returns DAISY_EWORKSPACE.  The first
 * call on each device resolves the array's device address (make it before any stream capture).  The array is
 * shared by all calls on a device: calls that may overlap on the GPU race.  Allocates nothing, ever. */
size_t daisy_b200_swa_decode_static_capacity(void);
int daisy_b200_swa_decode_step_static(const void* q_new, const void* k_new, const void* v_new,
                                      int64_t q_sb, int64_t q_sh, int64_t k_sb, int64_t k_sh,
                                      int64_t v_sb, int64_t v_sh,
                                      void* kcache, void* vcache, int64_t c_sb, int64_t c_sh, int64_t c_sr,
                                      int64_t t, int cap, int window,
                                      const float* cos_row, const float* sin_row,
                                      void* out, int64_t o_sb, int64_t o_sh,
                                      void* k_new_out, void* v_new_out,
                                      int B, int H, int D, float scale, float eps, unsigned flags,
                                      int splits, int* status_word, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Ring-buffer row copies for one layer (KVCache.view when wrapped, inference/kv_cache.py:36-42,
 * and KVCache.bulk_write_packed, inference/kv_cache.py:57-68).
 *   ring  logical [B,H,cap,D] strides (r_sb,r_sh,r_sr);  lin  logical [B,H,n,D] strides
 *   (l_sb,l_sh,l_sr); row i of `lin` <-> ring row (first_pos + i) % cap.
 *   to_ring != 0 copies lin -> ring, else ring -> lin.  elem_bytes is 2 or 4.
 */
int daisy_b200_ring_copy_rows(void* ring, int64_t r_sb, int64_t r_sh, int64_t r_sr,
                              void* lin, int64_t l_sb, int64_t l_sh, int64_t l_sr,
                              int B, int H, int D, int cap, int64_t first_pos, int n,
                              int elem_bytes, int to_ring, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Kimi delta attention, chunked forward.  Replaces the call
 * chunk_kda(q,k,v,g,beta,initial_state,output_final_state,use_qk_l2norm_in_kernel=True)
 * at models/daisy/attention_kimi.py:133-134 (third-party flash-linear-attention kernel).
 *   q,k [B,T,H,K] bf16, v [B,T,H,V] bf16, g [B,T,H,K] float32 log-decay (<= 0),
 *   beta [B,T,H] float32, h0 / hT [B,H,K,V] float32 (nullable), o [B,T,H,V] bf16
 *   (float32 with DAISY_KDA_OUT_FP32); all contiguous.  K = V = 128, chunk = 64.
 *   scale <= 0 selects K^-1/2.
 */
size_t daisy_b200_kda_workspace_bytes(int B, int T, int H, int K, int V);
int daisy_b200_kda_chunk_fwd(const void* q, const void* k, const void* v, const float* g,
                             const float* beta, const float* h0, void* o, float* hT,
                             int B, int T, int H, int K, int V, int chunk, float scale,
                             unsigned flags, void* workspace, size_t workspace_bytes,
                             int* status_word, void* stream);

/* Packed variable-length form of the same call: chunk_kda(..., cu_seqlens=cu_seqlens) at
 * models/daisy/attention_kimi.py:133-134, with cu_seqlens from get_unpad_data (:150-154; helpers :19-33).  The
 * sequences lie end to end in one row: q, k [1, T_total, H, K], v, o [1, T_total, H, V], g fp32, beta [1, T_total, H];
 * h0 / hT [n_seq, H, K, V] float32 or null.  No chunk spans two sequences; the caller lists the chunks:
 *   chunk_tab [n_chunks][2] int32 (device): first token and number of tokens (1..64) of each chunk, sequence after
 *     sequence, each sequence cut into 64-token chunks from its own first token;
 *   seq_ptr [n_seq + 1] int32 (device): sequence i owns chunks seq_ptr[i] .. seq_ptr[i+1]-1 (none for an empty
 *     sequence, whose final state is its initial state).
 * workspace: daisy_b200_kda_varlen_workspace_bytes(n_chunks, H, K, V).  Other arguments and errors as above. */
size_t daisy_b200_kda_varlen_workspace_bytes(int n_chunks, int H, int K, int V);
int daisy_b200_kda_chunk_fwd_varlen(const void* q, const void* k, const void* v, const float* g,
                                    const float* beta, const float* h0, void* o, float* hT,
                                    int T_total, int H, int K, int V, int chunk, float scale, unsigned flags,
                                    const int32_t* chunk_tab, int n_chunks, const int32_t* seq_ptr, int n_seq,
                                    void* workspace, size_t workspace_bytes, int* status_word, void* stream);

/* The same recurrence token by token, for short inputs (decode steps; the reference calls chunk_kda with
 * T = 1 and the cached state, models/daisy/attention_kimi.py:144-149,175-180).  The state of one (batch, head)
 * stays in registers across the T tokens: read from h0 once (null = zero state), written to hT once (null =
 * discarded; hT may alias h0 for an in-place cache update).  No workspace.  Same layouts and flags as
 * daisy_b200_kda_chunk_fwd. */
int daisy_b200_kda_recurrent_fwd(const void* q, const void* k, const void* v, const float* g,
                                 const float* beta, const float* h0, void* o, float* hT,
                                 int B, int T, int H, int K, int V, float scale, unsigned flags,
                                 void* stream);

/* Log-decay gate of the KDA layer.  Replaces fused_kda_gate(g, A_log, head_k_dim, dt_bias, None, beta,
 * threshold) at models/daisy/attention_kimi.py:132 (forward of _gate_impl, models/daisy/fla_custom_ops.py:71-103):
 *   out[r, h, d] = -exp(a_log[h]) * softplus(g[r, h*D + d] + bias[h*D + d]; beta, threshold)      (fp32 math)
 * g [rows, H*D] bf16 (g_is_bf16 != 0) or float32; a_log [H] float32; bias [H*D] float32 or null; out [rows, H*D]
 * float32, the layout daisy_b200_kda_chunk_fwd takes.  D a multiple of 4.  flags: 0 or DAISY_KDA_GATE_ROUND_BF16. */
int daisy_b200_kda_gate(const void* g, int g_is_bf16, const float* a_log, const float* bias, float* out,
                        int64_t rows, int H, int D, float beta, float threshold, unsigned flags, void* stream);

/* Short causal depthwise convolution of the KDA layer's q / k / v projections.  Replaces the ShortConvolution
 * calls at models/daisy/attention_kimi.py:160-162 (modules built at :88-91; third-party fla.modules, a depthwise
 * nn.Conv1d with padding W-1 and SiLU):
 *   y[b, t, c] = act(bias[c] + sum_{j<W} w[c, j] * in[b, t - (W-1) + j, c]),   in[t<0] = the carried state or 0
 * x, y [B, T, C] bf16 with batch / row strides in elements (multiples of 8); w [C, W] bf16 (the Conv1d weight
 * [C, 1, W]); bias [C] bf16 or null; state_in / state_out [B, C, W] bf16 or null: the last W inputs, oldest first
 * (the `cache` / final state of the reference call; state_out[., ., j] = in[T - W + j]).  state_out may alias
 * state_in only when T <= 32 (decode steps: the in-place cache update of the reference).  W <= 4, C % 8 == 0.
 * flags: 0 or DAISY_KDA_CONV_SILU.  fp32 accumulation, one rounding to bf16. */
int daisy_b200_kda_short_conv(const void* x, int64_t x_sb, int64_t x_st, const void* w, const void* bias,
                              const void* state_in, void* state_out, void* y, int64_t y_sb, int64_t y_st,
                              int B, int T, int C, int W, unsigned flags, void* stream);

/* The same convolution over packed sequences (the reference passes cu_seqlens to each ShortConvolution call,
 * models/daisy/attention_kimi.py:160-162): x, y [T_total, C] with row strides; the window never crosses the first
 * token of a sequence.  tok_tab [T_total][2] int32 (device): for each token the index of its sequence's first token
 * and the sequence's number.  state_in / state_out [n_seq, C, W] or null; state_out is written for every sequence
 * that has at least one token (fill it with state_in beforehand if empty sequences may occur) and must not alias
 * state_in. */
int daisy_b200_kda_short_conv_varlen(const void* x, int64_t x_st, const void* w, const void* bias,
                                     const void* state_in, void* state_out, void* y, int64_t y_st,
                                     int T, int C, int W, const int32_t* tok_tab, unsigned flags, void* stream);

/* Gated RMS norm of the KDA output over the head dimension.  Replaces self.o_norm(o, gp) at
 * models/daisy/attention_kimi.py:137 (CompilableFusedRMSNormGated, :41-62; third-party fla rms_norm_gated):
 *   n = o * rsqrt(mean(o^2) + eps) * weight,  y = n combined with the gate as `mode` says (DAISY_KDA_NORM_*).
 * o [rows, D] bf16 (o_is_fp32 == 0) or float32; gate [rows, D] bf16; weight [D] bf16 or null (ones); y [rows, D]
 * bf16.  D = 128.  The reference passes no eps: rms_norm_gated's default 1e-6.  gate_bias [H, D] bf16 or null: the
 * bias of the gate's projection (g_proj[1].bias, :106), added to `gate` here -- row r belongs to head r % H, the sum is
 * rounded to bf16 as the Linear's output would be -- so the projection itself can run bias-free. */
int daisy_b200_kda_out_norm(const void* o, int o_is_fp32, const void* gate, const void* gate_bias, int H,
                            const void* weight, void* y, int64_t rows, int D, float eps, int mode, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Self-test of the tensor-core building blocks (no reference counterpart): C[128,128] float32 =
 * A[128,K] x B, through TMA-staged swizzled shared memory, tcgen05.mma and a TMEM read-back.
 *   mode 0: B given as [128,K] row-major (K-major operand, the Q K^T form)
 *   mode 1: B given as [K,128] row-major (MN-major operand, the P V form), A from shared memory
 *   mode 2: as mode 1 but A is first written to TMEM as packed bf16 (the P-in-TMEM form)
 *   mode 3: mode 0 with a barrier that nothing completes -- exercises the bounded wait: the kernel gives up after
 *           its time limit, writes DAISY_ETIMEOUT to the status word, frees its TMEM and returns; C is not written
 * K must be a multiple of 64 and <= 128.  Used by the GPU tests only.
 */
int daisy_b200_selftest_umma(const void* a, const void* b, float* c, int K, int mode,
                             int* status_word, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DAISY_B200_H */
