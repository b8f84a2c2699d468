/* C ABI of liblact_b200: B200 (sm_100a) kernels for the LaCT large-chunk fast-weight TTT step.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*),
 * enqueues its kernels on that stream without synchronising, and returns an int:
 *     0   success (work enqueued)
 *   < 0   argument / configuration error detected on the host (nothing was enqueued)
 * Device-side status (a bounded wait that ran out) is recorded in the first word of the
 * caller-provided workspace and read with lact_read_status().
 * The library never allocates or frees device memory: all scratch comes from `workspace`,
 * sized by the matching *_workspace_bytes call.
 *
 * The reference (a1600012888/LaCT) has no FFI: its interface for this path is a set of Python
 * functions on tensors.  Each declaration cites the reference function whose arithmetic the
 * entry point replaces; the Python package `lact_b200` re-exports those functions under the
 * reference's names and signatures and binds to this ABI with ctypes.
 *
 * Layouts ("LLM layout"): w0, w2: [B, H, D]; w1: [B, D, H]; q, k, v, o: [B, L, D];
 * lr0/1/2, momentum: [B, L]; B = batch * heads (merged), D = head dim, H = fast-weight hidden dim.
 */
#ifndef LACT_B200_H_
#define LACT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes */
#define LACT_F32 0
#define LACT_BF16 1

/* error codes (negative: host-side argument errors) */
#define LACT_OK 0
#define LACT_ERR_NULL -1        /* a required pointer is NULL */
#define LACT_ERR_SHAPE -2       /* unsupported or inconsistent sizes / strides / alignment */
#define LACT_ERR_DTYPE -3       /* unsupported dtype combination */
#define LACT_ERR_WORKSPACE -4   /* workspace missing or too small */
#define LACT_ERR_CONFIG -5      /* inconsistent configuration flags */
#define LACT_ERR_STEPS -6       /* malformed step list (empty update range, range outside [0, L]) */
#define LACT_ERR_CUDA -7        /* a CUDA runtime / driver call failed */
#define LACT_ERR_DEVICE -8      /* device is not sm_100 */
#define LACT_ERR_STATIC_LIMIT -9 /* lact_swiglu_ffn_fwd_static: scratch need exceeds the static buffer */

/* step kinds of the scan program */
#define LACT_STEP_APPLY 0
#define LACT_STEP_UPDATE 1

/* renormalisation modes */
#define LACT_RENORM_NONE 0
#define LACT_RENORM_EPS_OUTSIDE 1 /* w / (||w|| + 1e-5) * n0   : ttt_operation.py:198-200 */
#define LACT_RENORM_EPS_INSIDE 2  /* w * rsqrt(sum w^2 + 1e-5) * n0 : l2norm_triton_kernels.py:80 */

typedef struct lact_scan_config {
  int64_t B, L, D, H; /* merged batch*heads, tokens, head dim, fast-weight hidden dim */
  int64_t out_len;    /* tokens in o (== L except for operator lists that concatenate applies) */
  int32_t act_dtype;  /* dtype of q, k, v, o (LACT_BF16; LACT_F32 = split-precision fp32 mode) */
  int32_t lr_dtype;   /* dtype of lr0, lr1, lr2 */
  int32_t mom_dtype;  /* dtype of momentum */
  int32_t w_dtype;    /* dtype of w0, w1, w2 (inputs); outputs and state are always fp32 */
  int32_t use_momentum;
  int32_t use_muon;
  int32_t ns_steps;        /* Newton-Schulz iterations */
  int32_t ns_const_coeffs; /* 0: tuned 5-step table (ns_steps must be 5); 1: constant triple */
  int32_t ns_concat;       /* 1: orthogonalise cat([dw0, dw2], dim=1) as one [2H, D] matrix */
  int32_t ns_gram_right;   /* 1: square matrices iterate on the transpose (NVS weight layout) */
  int32_t renorm;          /* LACT_RENORM_* */
  int32_t prenorm;         /* 1: keep an un-normalised master, compute with the normalised copy */
  int32_t prenorm_bf16;    /* 1: the normalised copy is rounded to bf16 (fused pre-norm path) */
  int32_t overwrite_quirk; /* 1: w <- renorm(NS(dw) + dw) (bidirectional_lact_layer.py:139-146) */
  float w_scale;           /* scalar multiplied into the three learning rates */
  /* strides in elements; innermost (feature) stride is 1 */
  int64_t q_bs, q_ts, k_bs, k_ts, v_bs, v_ts, o_bs, o_ts;
} lact_scan_config;

typedef struct lact_scan_io {
  const void *w0, *w1, *w2;          /* initial fast weights */
  const void *q, *k, *v;             /* activations */
  const void *lr0, *lr1, *lr2;       /* per-token learning rates, [B, L] contiguous */
  const void *momentum;              /* per-token momentum, [B, L] contiguous, or NULL */
  const void *m0_in, *m1_in, *m2_in; /* initial momentum state (fp32, weight shapes) or NULL = zeros */
  void *o;                           /* [B, out_len, D], act_dtype */
  void *w0_out, *w1_out, *w2_out;    /* final fast weights, fp32, or NULL */
  void *m0_out, *m1_out, *m2_out;    /* final momentum state, fp32, or NULL */
  /* training: per UPDATE step u (in program order), fp32 [w0w2 | w1 | g0g2 | g1] with w = the weights
   * that step computed with ([B,2H,D], [B,D,H]) and g = its gradient after momentum; or NULL */
  void *state_dump;
  /* training with Muon (ns_steps 1..5): per UPDATE step, the Newton-Schulz iterates of both groups in the layout
   * lact_ns_trace_bwd reads (lact_scan_ns_trace_bytes per step; 256-byte aligned), so that the backward does not
   * recompute them; or NULL */
  void *ns_trace;
} lact_scan_io;

/* Library version (major * 1000 + minor).  No counterpart in the reference. */
int lact_version(void);

/* Human-readable text for a return code.  No counterpart in the reference. */
const char *lact_error_string(int code);

/* Number of kernels this library has launched in the process so far.  No counterpart in the
 * reference. */
int64_t lact_launch_count(void);

/* Per-kernel-class timing (a measurement aid; no counterpart in the reference).  While enabled,
 * every kernel launch is bracketed by two CUDA events on its stream.  lact_profile_read waits
 * for the recorded events, writes the summed milliseconds and launch counts of each class into
 * arrays of lact_profile_num_classes() entries, and clears the records. */
int lact_profile_enable(int enable);
/* While enabled, every kernel launch sits inside an NVTX range named after its kernel class (gemm_swiglu_gate,
 * ns_fused, add_renorm, ...), for timeline tools.  Off by default.  No counterpart in the reference. */
int lact_nvtx_enable(int enable);
int lact_profile_num_classes(void);
const char *lact_profile_class_name(int cls);
int lact_profile_read(double *ms, int64_t *launches);

/* Reads the device status word of a workspace after synchronising `stream`.
 * Returns 0 (ok), a positive device status (101 = a bounded wait timed out) or LACT_ERR_CUDA.
 * This and lact_static_status are the only entry points that wait for a stream;
 * lact_stream_sync_count returns how often the library has done so in this process.
 * No counterpart in the reference. */
int lact_read_status(const void *workspace, void *stream);
int64_t lact_stream_sync_count(void);

/* Every device-side wait of the kernels (mbarrier waits, completion-counter spins) gives up after
 * this many nanoseconds of wall time and records status 101 instead of hanging (default 2 s;
 * 0 restores the default).  Applies to kernels launched afterwards on the current device.
 * lact_debug_wait_timeout launches one thread that waits on a barrier nobody arrives on, so the
 * time-out path can be exercised without any fault: `status_word` (device memory, zero before
 * the call) holds 101 once the kernel has run.  No counterpart in the reference. */
int lact_set_wait_limit_ns(uint64_t limit_ns);
int lact_debug_wait_timeout(int32_t *status_word, void *stream);

/* Scratch bytes needed by lact_scan_fwd for this configuration and step list. */
int lact_scan_workspace_bytes(const lact_scan_config *cfg, int32_t n_steps, const int32_t *kind,
                              const int64_t *start, const int64_t *end, size_t *bytes_out);

/* Bytes of Newton-Schulz trace that lact_scan_fwd keeps per UPDATE step when lact_scan_io.ns_trace is given
 * ([w0;w2] group first, the w1 group at `second_group_offset`); LACT_ERR_CONFIG if this configuration keeps none
 * (Muon off, or more than five iterations).  No counterpart in the reference (autograd keeps its own graph). */
int lact_scan_ns_trace_bytes(const lact_scan_config *cfg, size_t *bytes_per_update, size_t *second_group_offset);

/* The chunk recurrence: executes `n_steps` steps in order; APPLY writes
 * o[:, out_start : out_start + (end - start)] = f_W(q[:, start:end]); UPDATE updates the fast
 * weights from k, v, lr on [start, end) (gradient, momentum, Newton-Schulz, add, renorm).
 * Replaces the loops of: block_causal_lact_swiglu / prenorm_block_causal_lact_swiglu
 * (lact_llm/lact_model/ttt_operation.py:69-214, :217-364), the fused pair
 * (lact_llm/lact_model/ttt_operation_fused_kernel.py:66-186, :189-316),
 * bidirectional_lact_swiglu (minimal_implementations/bidirectional_lact_layer.py:73-160),
 * fast_weight_swish_glu_weight_norm_mini_batch_apply (lact_nvs/lact_ttt.py:70-147) and the four
 * autoregressive-video functions (lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:22-296,
 * ar_lact_swa_repeat_sp.py:27-339). */
int lact_scan_fwd(const lact_scan_config *cfg, const lact_scan_io *io, int32_t n_steps, const int32_t *kind,
                  const int64_t *start, const int64_t *end, const int64_t *out_start, void *workspace,
                  size_t workspace_bytes, void *stream);

/* out[B, N, D] = (silu(x w0^T) * (x w2^T)) w1^T with w0w2 = [B, 2H, D] (w0 rows first), all bf16.
 * Replaces fused_swiglu_ffn_fwd (lact_llm/lact_model/lact_triton_kernels/lact_swiglu_ffn.py:79-96).
 * Workspace: lact_swiglu_ffn_workspace_bytes. */
int lact_swiglu_ffn_workspace_bytes(int64_t B, int64_t N, int64_t D, int64_t H, size_t *bytes_out);
int lact_swiglu_ffn_fwd(const void *w0w2, const void *w1, const void *x, void *out, int64_t B, int64_t N,
                        int64_t D, int64_t H, void *workspace, size_t workspace_bytes, void *stream);

/* The same computation as lact_swiglu_ffn_fwd for callers that must not allocate and cannot hand
 * over a workspace.  No counterpart in the reference.
 *
 * Who needs it: code that runs where device allocation is off limits -- an inference-server
 * execution callback or plugin `enqueue` hook whose contract forbids cudaMalloc, a process whose
 * framework has already reserved the whole device for its own pool, or a latency-critical loop
 * that cannot afford the implicit device synchronisation of an allocator call.  Such a caller
 * still passes the operands and the output buffer; the hidden activations [B, N, H] (bf16) go
 * into a fixed array that is part of the library image.
 *
 * Limit: 256 + B * N * H * 2 bytes must fit in lact_static_scratch_bytes() (16 MiB; for example
 * B = 4, N = 2048, H = 384).  Larger problems return LACT_ERR_STATIC_LIMIT and enqueue nothing.
 * Every GPU that loads the library holds that array until the process exits.
 *
 * The kernels' status word (see lact_read_status) sits at the head of that array, where the
 * caller cannot point: lact_static_status(stream) synchronises `stream` and returns it (0, 101
 * or LACT_ERR_CUDA), also without allocating.  Read it before the next static call on the
 * device, which clears the word.
 *
 * The first call on a device looks up the array's device address (once per device, with that
 * device current); make that first call before starting any stream capture.  The call itself
 * allocates and frees nothing, on the device or through any library.
 *
 * All calls share the one array and it keeps the previous call's contents (the entry point clears
 * the status word it needs at zero, and overwrites the rest before reading it).  Two calls that
 * overlap on the GPU -- different streams, or different threads -- race on it: serialise them. */
size_t lact_static_scratch_bytes(void);
int lact_swiglu_ffn_fwd_static(const void *w0w2, const void *w1, const void *x, void *out, int64_t B, int64_t N,
                               int64_t D, int64_t H, void *stream);
int lact_static_status(void *stream);

/* dw0w2[B, 2H, D], dw1[B, D, H] (bf16) = per-token-lr weighted fast-weight gradient.
 * Replaces fused_lact_swiglu_ffn_fast_weight_grads
 * (lact_llm/lact_model/lact_triton_kernels/lact_fw_grad.py:159-175).  lr: [B, N], lr_dtype. */
int lact_fw_grad_workspace_bytes(int64_t B, int64_t N, int64_t D, int64_t H, size_t *bytes_out);
int lact_fw_grad(const void *w0w2, const void *w1, const void *k, const void *v, const void *lr0, const void *lr1,
                 const void *lr2, int32_t lr_dtype, void *dw0w2, void *dw1, int64_t B, int64_t N, int64_t D,
                 int64_t H, void *workspace, size_t workspace_bytes, void *stream);

/* x[B, R, C] (bf16) = Newton-Schulz orthogonalisation of g[B, R, C] (g_dtype), bf16 arithmetic.
 * const_coeffs = 0: zeropower_via_newtonschulz5(G) (lact_llm/lact_model/ttt_operation.py:30-66),
 * steps must be 5; const_coeffs = 1: zeropower_via_newtonschulz5(G, steps)
 * (lact_nvs/lact_ttt.py:32-67). */
int lact_newton_schulz_workspace_bytes(int64_t B, int64_t R, int64_t C, size_t *bytes_out);
int lact_newton_schulz(const void *g, int32_t g_dtype, void *x, int64_t B, int64_t R, int64_t C, int32_t steps,
                       int32_t const_coeffs, void *workspace, size_t workspace_bytes, void *stream);

/* y = (x + x_add) * rsqrt(sum_row (x + x_add)^2 + eps) * scale[row]; x: [B, T, D].
 * Replaces l2_norm_add_fused (lact_llm/lact_model/lact_triton_kernels/l2norm_triton_kernels.py:419-427). */
int lact_l2_norm_add(const void *x, int32_t x_dtype, const void *x_add, int32_t add_dtype, const void *scale,
                     void *y, int32_t y_dtype, int64_t B, int64_t T, int64_t D, float eps, void *stream);

/* m' = dx + mu[b] * m; x' = x + m'; y = bf16(x' / sqrt(sum_row x'^2 + eps) * scale[row]).
 * Replaces fused_prenorm_update_with_momentum_and_l2_norm
 * (lact_llm/lact_model/lact_triton_kernels/triton_prenorm_update_with_momentum.py:379-401).
 * x, m: fp32 [B, T, D]; dx: bf16; mu: fp32 [B]; scale: fp32 [B, T]. */
int lact_prenorm_momentum_l2norm(const void *x, const void *dx, const void *m, const void *mu, const void *scale,
                                 void *x_out, void *m_out, void *y_out, int64_t B, int64_t T, int64_t D, float eps,
                                 void *stream);

/* Fast-weight inputs of the LLM layer from the projected activations, in one pass (replaces the SiLU, l2_norm and
 * head split / merge passes of lact_llm/lact_model/layer_lact_swiglu.py:399-414, `ttt_nope` branch, and
 * ttt_operation.py:19-26): q, k <- l2_norm(silu(x)) per head, v <- silu(x) (qkv_silu = 0: no SiLU; v_silu = 0:
 * none on v), every intermediate rounded to bf16 as in the reference's eager arithmetic.
 * xq, xk, xv: bf16 [b][s][n_heads * d] with row stride ld_* and batch stride bs_* (elements; views of a fused
 * projection are fine); q, k, v: bf16 [(b n_heads)][s][d] contiguous.  d <= 1024, a multiple of 8. */
int lact_qkv_prologue(const void *xq, const void *xk, const void *xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                      int64_t bs_q, int64_t bs_k, int64_t bs_v, void *q, void *k, void *v, int64_t b, int64_t s,
                      int64_t n_heads, int64_t d, int32_t qkv_silu, int32_t v_silu, void *stream);

/* The same pass followed by the rotary position embedding the layer applies to fast q and k when `ttt_nope` is off
 * (layer_lact_swiglu.py:417-446: heads merged back, re-split into attention heads of rope_head_dim features, rotated by
 * fla.modules.RotaryEmbedding in its non-interleaved layout, split into fast-weight heads again).  cos, sin: bf16
 * [n_positions][rope_head_dim / 2] (the module's cached tables, in the activations' dtype); token t of every sequence
 * uses row seqlen_offset + t.  rope_head_dim: a power of two in [32, 1024] that divides d.  v is not rotated.
 * seq_start: NULL, or for b = 1 an int32 [s] device array with the first token of the packed sequence every token belongs
 * to (the layer's cu_seqlens, :434): token t then uses row seqlen_offset + t - seq_start[t]. */
int lact_qkv_prologue_rope(const void *xq, const void *xk, const void *xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                           int64_t bs_q, int64_t bs_k, int64_t bs_v, void *q, void *k, void *v, int64_t b, int64_t s,
                           int64_t n_heads, int64_t d, int32_t qkv_silu, int32_t v_silu, const void *cos, const void *sin,
                           int64_t rope_head_dim, int64_t n_positions, int64_t seqlen_offset, const int32_t *seq_start,
                           void *stream);

/* Per-token learning rates and momentum of the LLM layer (layer_lact_swiglu.py:463-480, 245-249):
 * lr = softplus(float(lr_proj) + base_lr_inv), lr_proj [b][s][n_heads * 3] (row stride proj_ld) -> lr0, lr1, lr2
 * fp32 [(b n_heads)][s]; momentum = float(sigmoid(logits) rounded to the logits' dtype), logits [b][s][n_heads]
 * (row stride logits_ld) -> fp32 [(b n_heads)][s]; mom_logits and momentum may both be NULL. */
int lact_lr_prologue(const void *lr_proj, int32_t proj_dtype, int64_t proj_ld, float base_lr_inv, const void *mom_logits,
                     int32_t logits_dtype, int64_t logits_ld, void *lr0, void *lr1, void *lr2, void *momentum, int64_t b,
                     int64_t s, int64_t n_heads, void *stream);

/* Causal sliding-window attention forward, the other half of each hybrid layer, on the same q / k / v layout as
 * the layer's projections: o[b, l, h, d] = softmax over keys (i - window, i] of q_i . k_j * softmax_scale, times v.
 * Replaces flash_attn_func(q, k, v, causal=True, window_size=(window - 1, 0)) at
 * lact_llm/lact_model/layer_lact_swiglu.py:386-394 and
 * minimal_implementations/causal_lact_with_sliding_window_attn.py:380-384.  bf16; d = 64 or 128; heads adjacent within
 * a token (head stride d), token / batch strides in elements (views of a fused projection are fine);
 * window = 0 or >= l: plain causal attention.  window < 0: BLOCK attention, not causal: every query of a batch entry sees
 * all lk keys of that entry (q, o: [b, l, h, d]; k, v: [b, lk, h, d]; lk <= 0 stands for l; with window >= 0, lk must
 * equal l) - the full attention over a frame block that the autoregressive-video layer runs through
 * flash_attention(q, k, v, k_lens, window_size=(-1, -1)) at
 * lact_ar_video/minVid/models/blocks/ar_lact_swa_repeat.py:299-463.  seq_start (causal only): NULL, or for b = 1 an int32 [l] device array giving, for every
 * token, the first token of the packed sequence it belongs to (nondecreasing; what cu_seqlens describes in
 * flash_attn_varlen_func, layer_lact_swiglu.py:371-385): earlier keys are invisible.  lse: optional fp32 [b, n_heads, l], receives every row's log-sum-exp
 * in the log2 domain (what lact_swa_bwd needs), or NULL.  status_word: device word, 0 before the call (101 = a bounded
 * wait ran out). */
int lact_swa_fwd(const void *q, const void *k, const void *v, void *o, int64_t b, int64_t l, int64_t lk, int64_t n_heads,
                 int64_t d, int64_t q_ts, int64_t q_bs, int64_t k_ts, int64_t k_bs, int64_t v_ts, int64_t v_bs, int64_t o_ts,
                 int64_t o_bs, int64_t window, float softmax_scale, const int32_t *seq_start, void *lse,
                 int32_t *status_word, void *stream);

/* Backward of lact_swa_fwd: dq (bf16, contiguous [b, l, n_heads, d]) and dk, dv ([b, lk, n_heads, d]), written, from the forward's inputs, its
 * output o, its lse and the output gradient dout (bf16, token / batch strides in elements).  delta: fp32 scratch
 * [b, n_heads, l].  Three launches: row sums of dout * o, the keys' side (dK, dV), the queries' side (dQ); the
 * probabilities are recomputed from lse.  What autograd of flash_attn_func computes for the reference layer. */
int lact_swa_bwd(const void *q, const void *k, const void *v, const void *o, const void *dout, const void *lse, void *dq,
                 void *dk, void *dv, void *delta, int64_t b, int64_t l, int64_t lk, int64_t n_heads, int64_t d, int64_t q_ts,
                 int64_t q_bs, int64_t k_ts, int64_t k_bs, int64_t v_ts, int64_t v_bs, int64_t o_ts, int64_t o_bs,
                 int64_t do_ts, int64_t do_bs, int64_t window, float softmax_scale, const int32_t *seq_start,
                 int32_t *status_word, void *stream);

/* Backward of lact_qkv_prologue / lact_qkv_prologue_rope on the saved projections (same strides): dq, dk, dv are the
 * gradients of the head-major outputs ([(b n_heads), s, d] bf16, NULL = none), dxq, dxk, dxv the gradients of the
 * projections ([b, s, n_heads * d] bf16, contiguous, written).  The forward's bf16 roundings are treated as identities.
 * rope_head_dim = 0: no rotation.  Autograd of layer_lact_swiglu.py:399-446. */
int lact_qkv_prologue_bwd(const void *xq, const void *xk, const void *xv, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                          int64_t bs_q, int64_t bs_k, int64_t bs_v, const void *dq, const void *dk, const void *dv,
                          void *dxq, void *dxk, void *dxv, int64_t b, int64_t s, int64_t n_heads, int64_t d,
                          int32_t qkv_silu, int32_t v_silu, const void *cos, const void *sin, int64_t rope_head_dim,
                          int64_t n_positions, int64_t seqlen_offset, const int32_t *seq_start, void *stream);

/* Backward of lact_out_epilogue: dx [(b n_heads), s, d] and dgate [b, s, n_heads * d] (bf16, written; dgate NULL iff
 * gate_proj NULL), and per-block partial sums of the norm weight's gradient, dw_partial [lact_out_epilogue_bwd_blocks()][d]
 * fp32 (the caller adds the rows; fixed order, deterministic).  The gradient of the residual input is dout itself.
 * Autograd of layer_lact_swiglu.py:556-568. */
int lact_out_epilogue_bwd_blocks(void);
int lact_out_epilogue_bwd(const void *fw_x, const void *weight, const void *gate_proj, int64_t gate_ld, const void *dout,
                          int64_t dout_ld, void *dx, void *dgate, void *dw_partial, int64_t b, int64_t s, int64_t n_heads,
                          int64_t d, float eps, void *stream);

/* Output side of the LLM layer in one pass (layer_lact_swiglu.py:556-568): per-head RMSNorm of the recurrence's
 * output (fp32 arithmetic x * rsqrt(mean(x^2) + eps) * weight, rounded to bf16: the arithmetic of the
 * fla.modules.RMSNorm kernel the reference calls), times bf16(silu(gate_proj)), heads merged back, plus `resid`.
 * fw_x: bf16 [(b n_heads)][s][d] contiguous; weight: fp32 [d]; gate_proj, resid (either may be NULL), out:
 * bf16 [b][s][n_heads * d] with row strides *_ld (elements); out may alias resid.  d <= 1024, a multiple of 8. */
int lact_out_epilogue(const void *fw_x, const void *weight, const void *gate_proj, int64_t gate_ld, const void *resid,
                      int64_t resid_ld, void *out, int64_t out_ld, int64_t b, int64_t s, int64_t n_heads, int64_t d,
                      float eps, void *stream);

/* Building blocks of the training backward (the reference's backward is autograd through
 * lact_swiglu_ffn.py:46-76, lact_fw_grad.py:61-156 and the eager momentum / Newton-Schulz / renorm ops).
 *
 * lact_bmm2_bf16: c[batch, M, N] (+)= a0 b0^T (+ a1 b1^T), bf16 operands (each [batch, rows, K] or, MN-major,
 *   [batch, K, rows]), fp32 accumulation; c_dtype fp32 (optionally accumulating into c) or bf16.
 *   Replaces torch.bmm and fused_two_mm_wT_x / fused_two_mm_wT_xT (triton_fused_matmul_kernels.py:46-291).
 * lact_swiglu_bwd_planes: from y0|y2 [rows, 2H] and dh [rows, H] (bf16) the planes dy0*lr0 | dy2*lr2 and hidden*lr1
 *   (swiglu_backward_three_bmm pointwise part, triton_swiglu_bwd_kernels.py:140-165); lr pointers may be NULL (= 1).
 * lact_fw_grad_bwd_pointwise: second-order pointwise stage (lact_fw_grad.py:178-260 /
 *   triton_pointwise_kernels.py:6-236) with deterministic row sums for the lr gradients.
 * lact_renorm_bwd: backward of the row renormalisation of w = base + upd (ttt_operation.py:193-200 /
 *   l2norm_triton_kernels.py:97-172); dn0[row] += d<y>/dn0. */
int lact_bmm2_bf16(const void *a0, int32_t a0_mn_major, const void *b0, int32_t b0_mn_major, const void *a1,
                   int32_t a1_mn_major, const void *b1, int32_t b1_mn_major, void *c, int32_t c_dtype,
                   int32_t accumulate, int64_t batch, int64_t M, int64_t N, int64_t K, int32_t *status_word,
                   void *stream);
/* One or two independent batched products c (+)= a0 b0^T [+ a1 b1^T] in ONE persistent launch (the training backward
 * pairs products that share a shape class, halving its launches).  Fields as the arguments of
 * lact_bmm2_strided_bf16; both problems single-product or both two-product.  No counterpart in the reference. */
typedef struct lact_bmm_desc {
  const void *a0, *b0, *a1, *b1; /* a1 = b1 = NULL: single product */
  void *c;
  int64_t a0_ld, a0_bs, b0_ld, b0_bs, a1_ld, a1_bs, b1_ld, b1_bs, c_ld, c_bs;
  int64_t batch, M, N, K;
  int32_t a0_mn, b0_mn, a1_mn, b1_mn, c_dtype, accumulate;
} lact_bmm_desc;
int lact_bmm_group_bf16(const lact_bmm_desc *problems, int32_t n, int32_t *status_word, void *stream);

/* The pointwise stage of lact_fw_grad alone: dy02[B, N, 2H] = [dy0 * lr0 | dy2 * lr2], hid[B, N, H] = hidden * lr1
 * (bf16) from k, v [B, N, D] (bf16; token / batch strides in elements) -- lact_fw_grad.py:25-58.  A NULL learning
 * rate stands for 1 (lr: [B, *] with batch stride lr_bs): with (k, v) = (q, dO) this is the backward of apply's
 * pre-activations, lact_swiglu_ffn.py:46-76. */
int lact_fw_grad_pointwise(const void *w0w2, const void *w1, const void *k, int64_t k_ts, int64_t k_bs, const void *v,
                           int64_t v_ts, int64_t v_bs, const void *lr0, const void *lr1, const void *lr2,
                           int32_t lr_dtype, int64_t lr_bs, float w_scale, void *dy02, void *hid, int64_t B, int64_t N,
                           int64_t D, int64_t H, int32_t *status_word, void *stream);

/* The same product on strided operands and result (views of larger tensors, e.g. a token range of [B, L, D]):
 * *_ld = row stride, *_bs = batch stride, in elements (multiples of 8; base pointers 16-byte aligned). */
int lact_bmm2_strided_bf16(const void *a0, int32_t a0_mn_major, int64_t a0_ld, int64_t a0_bs, const void *b0,
                           int32_t b0_mn_major, int64_t b0_ld, int64_t b0_bs, const void *a1, int32_t a1_mn_major,
                           int64_t a1_ld, int64_t a1_bs, const void *b1, int32_t b1_mn_major, int64_t b1_ld,
                           int64_t b1_bs, void *c, int32_t c_dtype, int64_t c_ld, int64_t c_bs, int32_t accumulate,
                           int64_t batch, int64_t M, int64_t N, int64_t K, int32_t *status_word, void *stream);
/* Newton-Schulz with every iterate kept, and its backward (the reference differentiates
 * zeropower_via_newtonschulz5, ttt_operation.py:30-66 / lact_nvs/lact_ttt.py:32-67, by autograd):
 *   lact_ns_trace_fwd: x_out[B, R, C] (bf16) = Newton-Schulz(g), the iterates and Gram polynomials stay in `trace`
 *     (lact_ns_trace_bytes; 256-byte aligned); status_word: device status word as for lact_bmm2_bf16;
 *   lact_ns_trace_bwd: dx0[B, R, C] (fp32) = gradient w.r.t. the NORMALISED first iterate bf16(g) / (||g|| + 1e-7),
 *     from du[B, R, C] (bf16) = gradient w.r.t. x_out, using the trace of the matching forward call. */
int lact_ns_trace_bytes(int64_t B, int64_t R, int64_t C, int32_t steps, size_t *bytes_out);
/* byte offset, inside a trace, of the final iterate x_out (bf16 [B, R, C]) */
int lact_ns_trace_result_offset(int64_t B, int64_t R, int64_t C, int32_t steps, size_t *offset_out);
int lact_ns_trace_fwd(const void *g, int32_t g_dtype, void *x_out, int64_t B, int64_t R, int64_t C, int32_t steps,
                      int32_t const_coeffs, int32_t gram_right, void *trace, size_t trace_bytes, int32_t *status_word,
                      void *stream);
int lact_ns_trace_bwd(const void *du, void *dx0, int64_t B, int64_t R, int64_t C, int32_t steps, int32_t const_coeffs,
                      int32_t gram_right, void *trace, size_t trace_bytes, int32_t *status_word, void *stream);
int lact_swiglu_bwd_planes(const void *y02, const void *dh, const void *lr0, const void *lr1, const void *lr2,
                           int32_t lr_dtype, float w_scale, void *dy02, void *hid, int64_t rows, int64_t H,
                           void *stream);
int lact_fw_grad_bwd_pointwise(const void *y02, const void *dh, const void *g_dy02, const void *g_hid,
                               const void *lr0, const void *lr1, const void *lr2, int32_t lr_dtype, float w_scale,
                               void *g_y02, void *g_dh, void *dy02, void *hid, void *g_lr0, void *g_lr1, void *g_lr2,
                               int64_t rows, int64_t H, void *stream);
int lact_renorm_bwd(const void *base, const void *upd, int32_t upd_dtype, const void *n0, const void *dy, void *dw,
                    void *dw_bf16 /* optional bf16 copy of dw, or NULL */, void *dn0, int64_t rows, int64_t C,
                    int32_t mode, void *stream);
/* Two more stages of the reverse sweep that the reference leaves to autograd through its eager lines:
 *   lact_ns_norm_bwd: backward of the Frobenius normalisation in front of Newton-Schulz (ttt_operation.py:45-52):
 *     dx0 [nmat][n] (fp32, in/out) <- dx0 / den - bf16(g) <dx0, bf16(g)> / (den^2 nrm), nrm = bf16(||bf16(g)||),
 *     den = bf16(nrm + 1e-7), g [nmat][n] fp32;
 *   lact_momentum_bwd: momentum step (ttt_operation.py:170-179) for both gradient arrays (n0, n1 fp32 elements per
 *     batch entry): dg += carry (if add_carry); sum over s of dbeta[b][s] = <dg, mprev> (mprev NULL at the first update);
 *     carry <- dg * beta[b]; dgb = bf16(dg).  carry / beta NULL: no momentum (bf16 copy only). */
/* The same backward for one or two groups of matrices (e.g. the [w0; w2] and the w1 gradients of one update) in ONE
 * cooperative launch, followed by the normalisation backward: dg = d loss / d G (fp32, written).  Needs the trace of
 * lact_ns_trace_fwd / the training scan (steps <= 5).  LACT_ERR_CONFIG when no fused instantiation covers the shapes:
 * call lact_ns_trace_bwd + lact_ns_norm_bwd per group instead. */
typedef struct lact_ns_bwd_group {
  const void *du;    /* bf16 [nmat][rows][cols]: gradient w.r.t. the iteration's result */
  const void *g;     /* fp32 [nmat][rows][cols]: the matrix the iteration started from (before normalisation) */
  void *dg;          /* fp32 [nmat][rows][cols], written */
  void *trace;       /* the group's trace */
  size_t trace_bytes;
  void *partials;    /* fp32 scratch, nmat * 2 * lact_momentum_bwd_slices() */
  int64_t nmat, rows, cols;
} lact_ns_bwd_group;
int lact_ns_trace_bwd_fused(const lact_ns_bwd_group *groups, int32_t ngroups, int32_t steps, int32_t const_coeffs,
                            int32_t gram_right, int32_t *status_word, void *stream);
int lact_ns_norm_bwd(const void *g, void *dx0, void *partials /* fp32 scratch, nmat * 2 * lact_momentum_bwd_slices() */,
                     int64_t nmat, int64_t elems_per_matrix, void *stream);
int lact_momentum_bwd_slices(void); /* slices per batch entry: dbeta of lact_momentum_bwd is [B][slices] partial sums */
int lact_momentum_bwd(void *dg0, void *dg1, void *carry0, void *carry1, const void *mprev0, const void *mprev1,
                      void *dgb0, void *dgb1, const void *beta, void *dbeta, int64_t B, int64_t n0, int64_t n1,
                      int32_t add_carry, void *stream);

/* fp32 mode (fp32 activations; the reference's CPU configuration, e.g. bidirectional_lact_layer.py with fp32 inputs):
 * plain FFMA kernels for accuracy, no tensor cores.  The Python package runs the step program with them.
 *   lact_sgemm_f32: c[batch, M, N] = a b^T (+ beta[batch] * c when accumulate; beta NULL = 1), a stored [M][K] (a_t = 0) or [K][M], b stored [N][K] (b_t = 0) or [K][N]
 *     (replaces torch.bmm on fp32 tensors, e.g. ttt_operation.py:141-168);
 *   lact_swiglu_planes_f32: hidden (*lr1) and, when dh is given, dy0*lr0 | dy2*lr2 from y0|y2 (ttt_operation.py:149-160);
 *   lact_add_renorm: w <- renorm((quirk ? g : w) + (x ? x : g)) on fp32 masters (ttt_operation.py:189-200). */
int lact_sgemm_f32(const void *a, int32_t a_t, const void *b, int32_t b_t, void *c, int32_t accumulate,
                   const void *beta, int64_t batch, int64_t M, int64_t N, int64_t K, void *stream);
int lact_swiglu_planes_f32(const void *y02, const void *dh, const void *lr0, const void *lr1, const void *lr2,
                           int32_t lr_dtype, float w_scale, void *dy02, void *hid, int64_t rows, int64_t H, void *stream);
int lact_add_renorm(void *master, void *compute, void *shadow, const void *n0, const void *g, const void *x, int64_t B,
                    int64_t R, int64_t C, int32_t mode, int32_t prenorm, int32_t prenorm_bf16, int32_t quirk,
                    void *stream);

/* c[batch, M, N] = a * b^T with bf16 operands and fp32 accumulation (c_dtype output).
 * a is [batch, M, K] (a_mn_major = 0) or [batch, K, M] (a_mn_major = 1); b likewise with N.
 * Test hook for the tcgen05 GEMM engine; no counterpart in the reference (it calls torch.bmm). */
int lact_bmm_bf16(const void *a, int32_t a_mn_major, const void *b, int32_t b_mn_major, void *c, int32_t c_dtype,
                  int64_t batch, int64_t M, int64_t N, int64_t K, int32_t *status_word, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LACT_B200_H_ */
