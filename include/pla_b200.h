/*
 * pla_b200 — C ABI of the B200 (sm_100a) linear-attention hot path.
 *
 * Every entry point takes one plain-old-data argument struct (device pointers,
 * element strides, sizes, small enums) and a CUDA stream handle passed as
 * `void*` (a `cudaStream_t`; NULL = legacy default stream), launches its
 * kernels on that stream and returns immediately. No torch type appears here;
 * the library links only against the CUDA runtime.
 *
 * Return value: PLA_B200_OK, or a negative PLA_B200_E_* code for a host-side
 * contract violation (nothing is launched in that case).
 * `pla_b200_last_error()` returns a thread-local message for the last failure.
 *
 * Device-detected metadata problems (negative sequence offsets, an interval
 * longer than t_max, a tree parent that points forward) never trap: the CTA
 * that sees one ORs a PLA_B200_DEV_* bit into `*status` (when `status` is not
 * NULL), writes zeros to its output rows and returns.
 *
 * Reference interfaces are cited by their path inside t-head/pla.
 */
#ifndef PLA_B200_H_
#define PLA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PLA_B200_ABI_VERSION 1

/* ---- return codes ------------------------------------------------------ */
#define PLA_B200_OK 0
#define PLA_B200_E_INVALID (-1)     /* bad shape / stride / enum             */
#define PLA_B200_E_ALIGN (-2)       /* pointer or pitch not 16-byte aligned  */
#define PLA_B200_E_UNSUPPORTED (-3) /* valid in the reference, not built     */
#define PLA_B200_E_CUDA (-4)        /* the CUDA runtime reported an error    */
#define PLA_B200_E_TOO_LARGE (-5)   /* exceeds a fixed capacity              */

/* ---- device status bits (OR-ed into *status) ---------------------------- */
#define PLA_B200_DEV_BAD_INTERVAL 1 /* cu_seqlens interval invalid or > t_max */
#define PLA_B200_DEV_BAD_PARENT 2   /* tree parent index >= its own step      */
#define PLA_B200_DEV_WAIT_TIMEOUT 4 /* a bounded wait on a bulk copy ran out  */
#define PLA_B200_DEV_BAD_SLOT 8     /* slot index outside the pool            */
#define PLA_B200_DEV_DECAY_RANGE 16 /* chunked KDA prefill: a key channel decayed by more than 80 nats inside 16
                                       tokens (unbounded softplus gate); results of that call are not valid */

/* ---- enums ---------------------------------------------------------------- */
enum pla_b200_dtype { PLA_B200_BF16 = 0, PLA_B200_F16 = 1, PLA_B200_F32 = 2 };
/* Decay gate form. SOFTPLUS: g = -exp(A_log) * softplus(x + dt_bias).
 * SAFE: g = lower_bound * sigmoid(exp(A_log) * (x + dt_bias)).
 * (src/pla_device_helpers.cuh:215-246) */
enum pla_b200_gate { PLA_B200_GATE_SOFTPLUS = 0, PLA_B200_GATE_SAFE = 1 };
/* Which slot ids are padding: SGLANG: slot < 0; VLLM: slot <= 0.
 * (src/decode/k-last/fused_sigmoid_gating_k_last_kernel.cuh:166-169, :232-248) */
enum pla_b200_pad { PLA_B200_PAD_SGLANG = 0, PLA_B200_PAD_VLLM = 1 };

const char* pla_b200_last_error(void);
int pla_b200_abi_version(void);
/* When an entry point is called with `status` == NULL, its kernels OR their PLA_B200_DEV_* bits into a status
 * word that the library keeps on each GPU instead, so that a device-detected problem (a wait that ran out, a
 * slot outside the pool, a decay out of range) is never silent. This call copies the current device's word to
 * `*out` (it waits for the device's earlier work, so keep it off the hot path) and, with `clear` != 0, resets
 * it. No counterpart in the reference, whose kernels trap instead. */
int pla_b200_device_status(int32_t* out, int clear);
/* sizeof() of an argument structure of this header by name (e.g. "pla_b200_klast_args") and offsetof() of one of
 * its fields, as compiled into the library; -1 for an unknown name. For bindings that mirror the structures in
 * another language and want to check their layout at load time. No counterpart in the reference (pybind). */
int64_t pla_b200_struct_size(const char* type);
int64_t pla_b200_field_offset(const char* type, const char* field);

/* ======================================================================== *
 * k-last decode / MTP verify
 * Replaces the launcher behind
 *   pla.decode.fused_sigmoid_gating_delta_rule_forward_k_last         and
 *   pla.decode.fused_sigmoid_gating_delta_rule_forward_k_last_packed
 * (src/decode/k-last/fused_sigmoid_gating.cpp:164-203, host entry
 *  src/decode/k-last/fused_sigmoid_gating_cuda_k_last.cpp:239-435, launcher
 *  prototype src/decode/k-last/generated/fused_sigmoid_gating_dispatch_k_last.h:37-56).
 *
 * State pool: [slots, HV, V=128, K=128], K contiguous, slot pitch
 * `state_slot_stride` elements (>= HV*16384). Activations: q,k [tokens,H,128],
 * v [tokens,HV,128], o [tokens,HV,128] (o is dense), `*_tok_stride` in
 * elements. The packed form is the same call with q,k,v pointing into one
 * mixed_qkv row. All strides are in elements of the tensor's dtype.
 * ======================================================================== */
typedef struct pla_b200_klast_args {
  const void* q;
  const void* k;
  const void* v;
  const void* a;       /* gate logits: [tokens,HV] (GDN) or [tokens,HV,128] (KDA) */
  const void* b;       /* beta logits: [tokens,HV] */
  void* o;             /* [tokens,HV,128] dense, activation dtype */
  int64_t q_tok_stride, k_tok_stride, v_tok_stride, a_tok_stride, b_tok_stride;
  const void* A_log;   /* [HV] */
  const void* dt_bias; /* [HV] (GDN) or [HV,128] (KDA) */
  int32_t act_dtype;      /* pla_b200_dtype: BF16 or F16 */
  int32_t A_log_dtype;    /* any pla_b200_dtype */
  int32_t dt_bias_dtype;  /* any pla_b200_dtype */
  int32_t state_dtype;    /* F32 or BF16 */

  void* state;               /* pool base */
  int64_t state_slot_stride; /* elements between slots */
  int64_t num_slots;         /* slots addressable in the pool (bounds check; 0 = unchecked) */
  const int32_t* slot_indices; /* [B] or [B, S] */
  int32_t slot_row_stride;     /* 0: 1-D table; >0: row stride of the vLLM 2-D table */
  int32_t slot_cols;           /* S of the 2-D table (0 for 1-D) */
  const int32_t* num_accepted; /* [B] or NULL (2-D table: start column = max(acc,1)-1) */
  const int32_t* cu_seqlens;   /* [B+1] or NULL (then request n owns tokens [n*t_max,(n+1)*t_max)) */

  /* SGLang per-step snapshot cache [cache_rows, cache_steps, HV,128,128], same dtype as the pool */
  void* cache;
  const int32_t* cache_indices; /* [B] or NULL */
  int32_t cache_steps;          /* allocated step dimension of `cache` */
  /* EAGLE-tree parents; NULL = chain */
  const void* parents;
  int32_t parents_wide;         /* 0: int32, 1: int64 */
  int64_t parents_seq_stride, parents_tok_stride;

  int32_t B, t_max, H, HV;
  float scale;
  float softplus_beta, softplus_threshold, lower_bound;
  int32_t gate;            /* pla_b200_gate */
  int32_t is_kda;          /* per-key-channel gate */
  int32_t use_qk_l2norm;
  int32_t disable_state_update;
  int32_t pad;             /* pla_b200_pad */
  int32_t rows_per_cta;    /* 0 = pick; 16 = streaming decode kernel; else 32, 64 or 128 state rows per CTA */
  int32_t* status;         /* device word or NULL */

  /* ---- extensions used by the token-recurrent prefill (all zero / NULL for decode) ---- */
  void* state_out;                  /* NULL: the final state goes back into `state` at the request's slot */
  int64_t state_out_slot_stride;
  const int32_t* state_out_indices; /* NULL: request index n */
  int32_t state_by_request;         /* 1: slot_indices may be NULL, request n then uses slot n */
  int32_t state_init_zero;          /* start from a zero state; `state` is not read */
  int32_t state_transposed;         /* slots hold [K,V] (V contiguous) instead of [V,K] */
  int32_t gate_activated;           /* a = fp32 log-decay, b = fp32 beta, both already activated */
  int64_t o_total_rows;             /* > 0: rows [cu_seqlens[B], o_total_rows) of o are set to zero */
  float* o_f32;               /* single-token streaming decode only: when set, the unrounded fp32 outputs go
                                 here ([tokens, HV, 128]) instead of o; padding rows still get zeros in o */
  int32_t prescan;            /* prefill only, context parallelism: run every (request, head) twice without
                                 output rows -- from a zero state (offset B) and from the identity with
                                 V = 0 (transition M) -- and store both to state_out
                                 [B, HV, 2, 128, 128] fp32, so that S_out[v, :] = S_in[v, :] M + B[v, :];
                                 the state pool and its slots are not read */
} pla_b200_klast_args;

int pla_b200_decode_klast(const pla_b200_klast_args* args, void* stream);

/* Chunk-free prefill: the same recurrence token by token over packed varlen sequences
 * (needs cu_seqlens; t_max = longest sequence). Serves
 *   pla.prefill.flashqla.chunk_gated_delta_rule_fwd / gdn_prefill_packed_qkv_fwd
 *   (pla/prefill/flashqla/ops.py:225-738) and pla.prefill.flashkdapro.flashkda_fwd
 *   (pla/prefill/flashkdapro/ops.py:66-219)
 * with exact fp32 state arithmetic; q/k/v/gate rows may be only 2-byte aligned. */
int pla_b200_prefill_recurrent(const pla_b200_klast_args* args, void* stream);

/* ======================================================================== *
 * v-last GDN decode (single token per request)
 * Replaces pla::v_last::Args + pla_v_last_{small,big}batch_h*
 * (src/decode/v-last/v_last_args.h:79-106, v_last_dispatch.cuh:43-67, host
 *  src/decode/v-last/fused_sigmoid_gating_v_last.cpp:133-235).
 * State pool [slots,HV,K=128,V=128] fp32, V contiguous, dense. All activation
 * tensors dense. A slot < 0 leaves the request's `o` rows untouched; a request
 * whose interval is not exactly one token is skipped.
 * ======================================================================== */
typedef struct pla_b200_vlast_args {
  const void* q;  /* [B,H,128] */
  const void* k;  /* [B,H,128] */
  const void* v;  /* [B,HV,128] */
  const void* a;  /* [B,HV] */
  const void* b;  /* [B,HV] */
  void* o;        /* [B,HV,128] */
  const void* A_log;
  const void* dt_bias; /* [HV], activation dtype */
  int32_t act_dtype;
  int32_t A_log_dtype;
  float* state;
  int64_t num_slots;
  const int32_t* slot_indices; /* [>=B] */
  const int32_t* cu_seqlens;   /* [B+1] or NULL */
  int32_t B, H, HV;
  float scale, softplus_beta, softplus_threshold;
  int32_t use_qk_l2norm;
  int32_t* status;
} pla_b200_vlast_args;

int pla_b200_decode_vlast(const pla_b200_vlast_args* args, void* stream);

/* ======================================================================== *
 * Chunked GDN prefill (chunk 64, WY/UT transform) on the tcgen05 tensor cores.
 * Replaces the stage chain chunk_local_cumsum_qk_norm_gated -> kkt_solve -> fused_fwd behind
 * pla.prefill.flashqla.chunk_gated_delta_rule_fwd (pla/prefill/flashqla/ops.py:501-642,
 * src/prefill/flashqla/host/torch_extension_cute.cc:253, :546, :1008).
 * Two launches: "prepare" (per chunk and q/k head: normalised K/Q operands, K K^T and Q K^T on the
 * tensor cores, gate cumsum, the unit-lower-triangular inverse) writes operand images into
 * `workspace`; "chain" (per sequence and value head) walks the chunks with the state resident in
 * tensor memory. q/k/v/gate rows may be only 2-byte aligned. State arguments as in
 * pla_b200_klast_args' prefill extensions.
 * ======================================================================== */
typedef struct pla_b200_gdn_chunk_args {
  const void* q;
  const void* k;
  const void* v;
  int64_t q_tok_stride, k_tok_stride, v_tok_stride;
  int32_t act_dtype;       /* BF16 or F16 */
  int32_t gate_activated;  /* 0: gate/beta are raw 16-bit logits; 1: fp32 log-decay and fp32 beta */
  const void* gate;        /* [T, HV] */
  const void* beta;        /* [T, HV] */
  int64_t gate_tok_stride, beta_tok_stride;
  const float* A_log;      /* [HV] (raw gating) */
  const float* dt_bias;    /* [HV] (raw gating) */
  void* o;                 /* [T, HV, 128] dense, activation dtype; rows >= cu_seqlens[N] are zeroed */
  float* g_cum;            /* optional [T, HV]: chunk-local cumulative log decay */
  void* state;             /* initial state pool or NULL with state_init_zero */
  int32_t state_dtype;     /* F32 or BF16 */
  int32_t state_init_zero;
  int32_t state_transposed;   /* slots hold [K,V] instead of [V,K] */
  int32_t state_by_request;   /* slot_indices may be NULL: sequence n uses slot n */
  int64_t state_slot_stride;
  int64_t num_slots;
  const int32_t* slot_indices;
  void* state_out;            /* NULL: final state goes back into `state` (when write_state); with
                                 state_out_indices, a negative index skips that sequence's final state */
  int64_t state_out_slot_stride;
  const int32_t* state_out_indices;
  int32_t write_state;
  int32_t N;                  /* sequences */
  const int32_t* cu_seqlens;  /* [N+1] device */
  int64_t T_total;            /* physical token rows of q/k/v/o */
  int32_t max_chunks;         /* upper bound on sum_n ceil(len_n / 64), e.g. T_total/64 + N */
  int32_t H, HV;
  float scale;
  int32_t normalize_qk;
  int32_t stage;              /* 0: prepare + chain; 1: prepare only; 2: chain only, over a workspace that a
                                 stage-1 call with the same tokens filled */
  int32_t prescan;            /* context parallelism: instead of outputs, store per (sequence, value head) the
                                 segment's offset B (state reached from zero) and transition M (state reached
                                 from the identity with V = 0) into state_out [N, HV, 2, 128, 128] fp32, so that
                                 S_out[v, :] = S_in[v, :] M + B[v, :]; initial states and slots are not read */
  void* workspace;            /* device scratch of pla_b200_gdn_chunk_workspace_bytes() bytes, 128-byte aligned */
  int64_t workspace_bytes;
  int32_t* status;
  /* KDA only (pla_b200_kda_prefill_chunked): gate is the raw per-channel input [T, H*128] in the activation
   * dtype, dt_bias [H*128], H == HV, gate_activated = 0 */
  int32_t is_kda;             /* set by the KDA entry */
  int32_t gate_kind;          /* pla_b200_gate */
  float lower_bound;
} pla_b200_gdn_chunk_args;

int64_t pla_b200_gdn_chunk_workspace_bytes(int32_t max_chunks, int32_t H, int32_t HV);
int pla_b200_gdn_prefill_chunked(const pla_b200_gdn_chunk_args* args, void* stream);

/* Chunked KDA prefill (chunk 64, decay references every 16 tokens) on the tensor cores: replaces the launch
 * chain behind flashkda_fwd (src/prefill/flashkdapro/host/torch_extension_cute.cc:1686; its tc01 backend also
 * works on 64-token chunks with 16-token sub-chunks, src/prefill/flashkdapro/tc01/kernel_bt64_prefill_tc01.cu:82-96).
 * Same args struct, stages and prescan mode as the GDN entry. Safe gate with lower_bound >= -5, or a softplus
 * gate whose decay stays within 80 nats per 16 tokens (else PLA_B200_DEV_DECAY_RANGE is set). */
int64_t pla_b200_kda_chunk_workspace_bytes(int32_t max_chunks, int32_t H);
int pla_b200_kda_prefill_chunked(const pla_b200_gdn_chunk_args* args, void* stream);

/* ======================================================================== *
 * Context parallelism for one long sequence cut into token ranges (one per GPU). The prescan is the
 * `prescan` mode of the three prefill entries above; the fold below turns the gathered pairs into the state
 * entering a rank's range (the composition the reference applies to its intra-card segments,
 * src/prefill/flashqla/kernels/prepare_h_cute.cu:59-67, docs/prefill_flashkdapro_cp_design.md:22-46).
 * ======================================================================== */
typedef struct pla_b200_cp_fold_args {
  const float* pairs;          /* [world, HV, 2, 128, 128]: offset B, then transition M, per rank and head */
  const float* initial_state;  /* [HV, 128(V), 128(K)] state entering rank 0's range; NULL = zero */
  float* state_out;            /* [HV, 128, 128]: fold over ranks 0 .. rank-1 of S <- S M_j + B_j */
  int32_t HV, rank, world;
  int32_t* status;
  int32_t compose;             /* 1: compose pairs 0 .. rank-1 into ONE pair instead (initial_state unused):
                                  state_out = [HV, 2, 128, 128], offset (fold from zero) then transition
                                  (M_0 M_1 ... M_{rank-1}); `rank` may equal `world` */
} pla_b200_cp_fold_args;

int pla_b200_cp_fold_prefix(const pla_b200_cp_fold_args* args, void* stream);

/* The same fold inside one GPU: long sequences cut into consecutive token ranges that run as independent
 * chains (the reference's intra-card split, pla/prefill/flashqla/private/cp_preprocess.py). Range j of
 * sequence s (ranges seg_first[s] .. seg_first[s+1]-1, in token order) starts from
 *   state_in[seg_first[s]] = the sequence's pool state (or zero),  state_in[j+1] = state_in[j] M_j + B_j. */
typedef struct pla_b200_cp_fold_segments_args {
  const float* pairs;          /* [ranges, HV, 2, 128, 128] from a prescan over the ranges (last range of a sequence unused) */
  const int32_t* seg_first;    /* device [sequences + 1] */
  const float* pool;           /* fp32 k-last pool [slots, HV, 128, 128] or NULL (zero initial states) */
  int64_t pool_slot_stride;
  const int32_t* slot_indices; /* device [sequences] or NULL (= sequence index); a negative slot starts from zero */
  float* state_in;             /* out: [ranges, HV, 128, 128] */
  int32_t HV, sequences, slots;
  int32_t* status;
} pla_b200_cp_fold_segments_args;

int pla_b200_cp_fold_segments(const pla_b200_cp_fold_segments_args* args, void* stream);

/* ======================================================================== *
 * KDA ReplaySSM: verify (read-only checkpoint, replay records out) and commit
 * (integer plan, exact fold of the accepted prefix, conv-window scatter).
 * Replaces launch_verify_native / launch_commit_plan / launch_fold_native /
 * launch_conv_native (src/decode/kda_replayssm/kda_mtp_abi.h:127-150,
 * src/decode/kda_replayssm_vllm/commit_plan.h:7-14).
 * ======================================================================== */

/* A 1-D index vector as the caller holds it: int32 or int64, possibly strided
 * (src/decode/kda_replayssm/kda_mtp_abi.h:101-105). */
typedef struct pla_b200_index {
  const void* data;
  int32_t wide;   /* 0: int32 elements, 1: int64 elements */
  int64_t stride; /* elements between consecutive entries */
} pla_b200_index;

/* Strides (elements) of one conv-history tensor addressed [slot, channel, tap]. */
typedef struct pla_b200_conv_strides {
  int64_t slot, channel, tap;
} pla_b200_conv_strides;

/* Strides (elements) of one conv-window record tensor addressed [row, step, channel, tap]. */
typedef struct pla_b200_window_strides {
  int64_t row, step, channel, tap;
} pla_b200_window_strides;

typedef struct pla_b200_kda_verify_args {
  /* pre-conv activations, bf16, one row per token; q|k|v may be thirds of one mixed_qkv row */
  const void* x_q;
  const void* x_k;
  const void* x_v;
  int64_t xq_tok_stride, xk_tok_stride, xv_tok_stride;
  const void* raw_g;    /* [T, H*128] bf16 view */
  const void* raw_beta; /* [T, H] bf16 view */
  int64_t g_tok_stride, beta_tok_stride;
  const float* w_q;     /* [H*128, 4] causal-conv taps, tap 3 multiplies the current token */
  const float* w_k;
  const float* w_v;
  const void* cs_q;     /* persistent conv history (bf16), first three taps are read */
  const void* cs_k;
  const void* cs_v;
  pla_b200_conv_strides cs_q_strides, cs_k_strides, cs_v_strides;
  const float* A_log;   /* [H] */
  const float* dt_bias; /* [H*128] */
  const float* state;   /* checkpoint pool [slots, H, 128(V), 128(K)], read only */
  int64_t state_slot_stride;
  int32_t slots;
  void* out;            /* [T, H*128] bf16, dense */
  /* replay records; record row = request row (row_by_slot = 0) or = state slot (row_by_slot = 1) */
  void* rec_rawv;       /* [R, H, Q, 128] bf16: post-conv, pre-norm v */
  void* rec_rawk;       /* [R, H, Q, 128] bf16: post-conv, pre-norm k */
  float* rec_g;         /* [R, H, Q, 128] log-decay (pre-exp) */
  float* rec_beta;      /* [R, H, Q] */
  void* win_q;          /* conv windows after consuming each token, bf16 */
  void* win_k;
  void* win_v;
  pla_b200_window_strides win_q_strides, win_k_strides, win_v_strides;
  pla_b200_index slot_idx;    /* [N] */
  pla_b200_index cu;          /* [N+1] query_start_loc */
  pla_b200_index scratch_idx; /* [N] window row per request (row_by_slot = 1); data NULL -> request row */
  int32_t H, N, Q, T;         /* heads, requests, record steps, token capacity */
  int32_t null_block_id;      /* slots <= this are padding: their output interval is zeroed */
  int32_t row_by_slot;
  int32_t gate;               /* pla_b200_gate */
  float scale, lower_bound, softplus_beta, softplus_threshold;
  int32_t* status;
  /* optional fused gated output RMSNorm over the 128 value channels of each (token, head)
   * (src/decode/kda_replayssm/kda_mtp_verify.cu:185-212):
   *   out = o * rsqrt(mean(o^2) + eps) * weight * sigmoid(gate),  o the unrounded fp32 output.
   * All of onorm_gate, onorm_weight and out_f32 or none. */
  const void* onorm_gate;     /* bf16 [T, H*128] view */
  int64_t onorm_gate_tok_stride;
  const float* onorm_weight;  /* [128] */
  float onorm_eps;
  float* out_f32;             /* staging [T, H*128] fp32, overwritten */
  int32_t win_steps;          /* step capacity of the conv-window tensors when smaller than Q; 0 = Q */
} pla_b200_kda_verify_args;

int pla_b200_kda_replay_verify(const pla_b200_kda_verify_args* args, void* stream);
/* The same kernels under the SGLang contract (launch_verify, src/decode/kda_replayssm/kda_mtp_abi.h:127-136):
 * requires row_by_slot = 1, i.e. records are rings addressed by state slot [slots, H, Q, 128] and
 * conv windows are addressed by scratch_idx. */
int pla_b200_kda_ring_verify(const pla_b200_kda_verify_args* args, void* stream);

/* Exact fold of each request's accepted ring prefix into the fp32 state of every layer, in place,
 * one launch (launch_fold, src/decode/kda_replayssm/kda_mtp_abi.h:138-145; kernel
 * kda_mtp_fold.cu:254-529). Request b folds accept_lens[b] steps of ring row slot_idx[b] into
 * state[layer, slot_idx[b]]; rows with slot <= null_block_id or accept_lens <= 0 are skipped.
 * With tracking, the state after step track_step[b] (0-based) is also stored to slot track_idx[b]. */
typedef struct pla_b200_kda_fold_args {
  float* state;               /* [layers, slots, HV, 128(V), 128(K)] */
  int64_t state_layer_stride, state_slot_stride;
  const void* rawv;           /* bf16 [layers, slots, HV, L, 128] */
  int64_t rawv_layer_stride, rawv_slot_stride;
  const void* rawk;           /* bf16 [layers, slots, H, L, 128] */
  int64_t rawk_layer_stride, rawk_slot_stride;
  const float* gate;          /* [layers, slots, HV, L, 128] log-decay */
  int64_t gate_layer_stride, gate_slot_stride;
  const float* beta;          /* [layers, slots, HV, L] */
  int64_t beta_layer_stride, beta_slot_stride;
  pla_b200_index slot_idx, accept_lens;   /* [B] */
  pla_b200_index track_idx, track_step;   /* [B]; data NULL = no tracking */
  int32_t layers, B, H, HV, L, slots, null_block_id;
  int32_t* status;
} pla_b200_kda_fold_args;

int pla_b200_kda_fold_layers(const pla_b200_kda_fold_args* args, void* stream);

/* Conv-state rollback: dst[layer, dst_idx[n], :, :] = src[layer, n, step_idx[n], :, :], byte-exact, for
 * every request n with step_idx[n] >= 0 and a destination in range (launch_conv_scatter,
 * src/decode/kda_replayssm/kda_mtp_abi.h:147-150; kernel kda_mtp_fold.cu:595-640). */
typedef struct pla_b200_kda_conv_scatter_args {
  void* dst;                  /* [layers, slots, dim, taps], any positive strides */
  const void* src;            /* [layers, rows, steps, dim, taps] */
  int64_t dst_layer, dst_slot, dst_channel, dst_tap;            /* element strides */
  int64_t src_layer, src_row, src_step, src_channel, src_tap;
  pla_b200_index dst_idx, step_idx;   /* [reqs] */
  int32_t elem_size;          /* 2 (bf16) or 4 (fp32) */
  int32_t layers, reqs, dim, taps, src_rows, src_steps, dst_slots;
} pla_b200_kda_conv_scatter_args;

int pla_b200_kda_conv_scatter(const pla_b200_kda_conv_scatter_args* args, void* stream);

/* Columns of the per-layer descriptor table (int64 [layers, 11], device memory)
 * (src/decode/kda_replayssm/kda_mtp_abi.h:115-118). */
enum pla_b200_replay_column {
  PLA_B200_COL_STATE = 0, PLA_B200_COL_STATE_STRIDE, PLA_B200_COL_CONV, PLA_B200_COL_CONV_SLOT,
  PLA_B200_COL_CONV_CHANNEL, PLA_B200_COL_CONV_TAP, PLA_B200_COL_RAWV, PLA_B200_COL_RAWK,
  PLA_B200_COL_GATE, PLA_B200_COL_BETA, PLA_B200_COL_WINDOWS, PLA_B200_REPLAY_COLUMNS
};

typedef struct pla_b200_kda_commit_args {
  const int64_t* layers;      /* device table [n_layers, PLA_B200_REPLAY_COLUMNS] */
  int32_t n_layers;
  int32_t* candidate;         /* device int32 [4, capacity] scratch owned by the context */
  int32_t* plan;              /* device int32 [4, capacity]: commit_len, final, boundary, boundary_len */
  pla_b200_index sampled;     /* accepted-token counts per sampler row */
  pla_b200_index source;      /* [N] source checkpoint slot per request */
  pla_b200_index cu;          /* [N+1] */
  pla_b200_index mapping;     /* [N] request -> sampler row, data NULL = identity */
  pla_b200_index computed;    /* tokens already in the cache per sampler row (align mode) */
  pla_b200_index blocks;      /* block table base (align mode), addressed with the two strides below */
  int64_t block_row_stride, block_col_stride;
  int64_t block_size;         /* 0 = no alignment */
  int32_t block_rows, block_cols;
  int32_t N, capacity, sampler_rows;
  int32_t H, slots, Q, null_block_id;
  int64_t token_capacity;
  int32_t* status;
} pla_b200_kda_commit_args;

/* Plan only (bit-exact integer semantics of commit_plan.cu:18-115). */
int pla_b200_kda_replay_plan(const pla_b200_kda_commit_args* args, void* stream);
/* Plan, then fold + conv scatter of every layer in one more launch. */
int pla_b200_kda_replay_commit(const pla_b200_kda_commit_args* args, void* stream);

/* The commit plan for a caller that cannot allocate device memory. No counterpart in the
 * reference: there the candidate buffer always comes from the framework's allocator.
 *
 * Same inputs, same `plan` output and same bit-exact semantics as pla_b200_kda_replay_plan, but
 * `args->candidate` is ignored: the two plan phases exchange their candidates through a fixed
 * 64 KiB array that lives inside the library on every GPU that loads it. Meant for runners that
 * set their commit context up after all free device memory has been given to their cache pools,
 * or from a place where their allocator may not be called.
 *   - at most 4096 request rows (`capacity`); more returns PLA_B200_E_TOO_LARGE;
 *   - the array is shared by all calls on a device and keeps the previous call's contents (each
 *     call rewrites every entry it reads, so nothing needs clearing); calls that overlap on the
 *     GPU without a stream / event dependency between them race on it;
 *   - the first call on each device looks up the array's device address, so issue it before any
 *     stream capture starts;
 *   - it never calls cudaMalloc / cudaFree or any allocating routine. */
int pla_b200_kda_replay_plan_static(const pla_b200_kda_commit_args* args, void* stream);

/* ======================================================================== *
 * Fused KDA decode step (Kimi K3): causal conv (width 4) + SiLU over the packed q|k|v projections with
 * the 3-tap conv state shifted in place, L2 norms, per-channel gate, single-token recurrence on the fp32
 * k-last state in place, optional gated output RMSNorm -- one launch, no scratch. Replaces the launchers behind
 * fused_kda_decode_mega_forward (src/decode/k-last/fused_kda_decode_mega.cu; device contract
 * src/decode/k-last/fused_kda_decode_mega_kernel.cuh:36-79). A slot < 0 is padding: zero output row,
 * nothing else read or written; slot 0 is an ordinary slot.
 * ======================================================================== */
typedef struct pla_b200_kda_mega_args {
  const void* x;               /* [B, 3*H*128] activation dtype, channels contiguous */
  int64_t x_row_stride;
  const float* weight;         /* [3, 4, H*128]: segment (q, k, v), tap (3 = current token), channel */
  const float* bias;           /* [3*H*128] or NULL */
  void* conv_state;            /* activation dtype, addressed [slot, channel, tap] with the strides below */
  pla_b200_conv_strides conv_strides;
  const void* raw_g;           /* [B, H*128] activation dtype, contiguous */
  const void* raw_beta;        /* [B, H] activation dtype */
  int64_t beta_row_stride;
  const float* A_log;          /* [H] */
  const float* dt_bias;        /* [H*128] */
  const int32_t* state_indices; /* [B] */
  float* state;                /* [slots, H, 128(V), 128(K)] fp32 */
  int64_t state_slot_stride;
  int32_t slots;
  void* out;                   /* [B, H*128] activation dtype, contiguous */
  const void* output_gate;     /* [B, H*128] activation dtype view or NULL (then no output norm) */
  int64_t gate_row_stride;
  const float* norm_weight;    /* [128], with output_gate */
  float norm_eps;
  void* mixed;                 /* unused (the step runs as one kernel and keeps the conv outputs on the SM); may be NULL */
  float* out_f32;              /* unused; may be NULL */
  int32_t B, H;
  int32_t act_dtype;           /* pla_b200_dtype: BF16 or F16 */
  int32_t gate;                /* pla_b200_gate */
  float lower_bound, scale;
  int32_t* status;
} pla_b200_kda_mega_args;

int pla_b200_kda_decode_mega(const pla_b200_kda_mega_args* args, void* stream);

/* ======================================================================== *
 * Width-4 causal conv (+ SiLU) over packed varlen token rows with a 3-tap history per request: the
 * caller-side step that produces the packed q|k|v rows of the prefill ops (in the serving stacks a
 * separate kernel in front of the reference's prefill; the same arithmetic as the conv inside its fused decode
 * step, src/decode/k-last/fused_kda_decode_mega_kernel.cuh:36-79, and its verify kernels,
 * src/decode/kda_replayssm/kda_mtp_verify.cu:356-402). y_t = act(bias + h0 w0 + h1 w1 + h2 w2 + x_t w3),
 * (h0,h1,h2) <- (h1,h2,x_t). Rows at or past cu_seqlens[N] are written as zeros. Two launches: the conv, then
 * the history update (last three inputs of every non-empty sequence with a writable slot).
 * ======================================================================== */
typedef struct pla_b200_conv_prefill_args {
  const void* x;               /* [tokens, channels] activation dtype, channels contiguous, 16-byte aligned rows */
  int64_t x_row_stride;        /* elements */
  void* y;                     /* [tokens, channels] activation dtype, not x */
  int64_t y_row_stride;
  const float* weight;         /* [channels, 4]; tap 3 multiplies the current token */
  const float* bias;           /* [channels] or NULL */
  void* conv_state;            /* activation dtype, addressed [slot, channel, tap]; NULL = zero history, none kept */
  pla_b200_conv_strides conv_strides;
  int32_t slots;
  const int32_t* cu_seqlens;   /* [N + 1] */
  const int32_t* state_indices;        /* [N] or NULL (sequence n uses slot n) */
  const uint8_t* has_initial_state;    /* [N] or NULL (all): 0 = start from a zero history */
  int32_t N, tokens, channels;
  int32_t act_dtype;           /* pla_b200_dtype: BF16 or F16 */
  int32_t activation;          /* 0 = none, 1 = SiLU */
  int32_t pad;                 /* pla_b200_pad: which slot values mean "no history read or written" */
  int32_t* status;
} pla_b200_conv_prefill_args;

int pla_b200_causal_conv_prefill(const pla_b200_conv_prefill_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PLA_B200_H_ */
