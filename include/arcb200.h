/*
 * arcb200 — C ABI of the B200 (sm_100a) inference path for the mdlARC_scale
 * TinyTransformer: packed-prompt prefill, static-KV-cache greedy decode
 * (one CUDA graph per decode step) and the standalone kernels behind them.
 *
 * The reference project is pure Python and has no FFI of its own; each entry
 * point below therefore cites the reference *Python* function whose device
 * work it replaces (paths are relative to the reference repository root).
 *
 * Conventions
 *   - every pointer named d_* is a DEVICE pointer owned by the caller
 *     (normally a torch tensor); the library borrows it for the call, or for
 *     the life of the session when it is part of arcb_session_desc;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - return value: 0 = ok, <0 = argument/state error (ARCB_E_*), >0 = a
 *     cudaError_t / CUresult value; arcb_last_error() gives a message;
 *   - no exceptions cross the boundary; besides the handles the library keeps only
 *     per-device constants looked up once (SM count, resident cluster pairs, the
 *     address of the built-in scratch of arcb_op_decode_attention_static).
 */
#ifndef ARCB200_H
#define ARCB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ARCB_OK 0
#define ARCB_E_ARG (-1)       /* bad argument / unsupported shape            */
#define ARCB_E_STATE (-2)     /* call order (weights missing, no prefill...)  */
#define ARCB_E_DEVICE (-3)    /* a kernel reported a device-side error word   */
#define ARCB_E_UNSUPPORTED (-4)

#define ARCB_ACT_F16 0  /* 16-bit activations held as IEEE half (default)     */
#define ARCB_ACT_BF16 1 /* 16-bit activations held as bfloat16                */

#define ARCB_GEMM_AUTO 0 /* tcgen05 GEMM wherever the shape allows (K % 64 == 0)   */
#define ARCB_GEMM_SIMT 1 /* CUDA-core GEMM everywhere (debug cross-check)      */
#define ARCB_GEMM_TC 2   /* tcgen05 GEMM everywhere                            */
#define ARCB_GEMM_TC_1CTA 3 /* arcb_op_gemm only: the 1-CTA tcgen05 kernels        */
#define ARCB_GEMM_TC_2CTA 4 /* arcb_op_gemm only: the 2-CTA (cta_group::2) kernel  */

#define ARCB_ATTN_AUTO 0   /* tcgen05 flash prefill when available             */
#define ARCB_ATTN_STREAM 1 /* per-query streaming kernel for prefill as well   */

typedef struct arcb_engine arcb_engine;
typedef struct arcb_session arcb_session;

/* Mirrors TransformerConfig (src/transformer.py:15-34). Only rope_type "3d",
 * norm_type "rmsnorm", ffn_type "swiglu", vocab_size 14 and head_dim 64 are
 * implemented; anything else is rejected by the host wrapper. */
typedef struct arcb_config {
  int32_t d_model;
  int32_t n_heads;
  int32_t n_layers;
  int32_t d_ff;
  int32_t vocab_size;
  int32_t num_examples;
  int32_t max_x, max_y, max_z; /* RoPE table extents (positions clamp to max-1) */
  int32_t use_example_embedding;
  int32_t act_format; /* ARCB_ACT_*  */
  int32_t gemm_path;  /* ARCB_GEMM_* */
  int32_t attn_path;  /* ARCB_ATTN_* */
  float norm_eps;
} arcb_config;

/* Tensor kinds for arcb_engine_load_tensor: names follow the reference
 * state_dict (src/transformer.py:523-542, 245-263, 436-443). All sources are
 * fp32, row-major, in the reference's own shapes. */
enum arcb_tensor_kind {
  ARCB_T_TOKEN_EMBED = 0, /* token_embed.weight           [vocab, d]        */
  ARCB_T_EXAMPLE_EMBED,   /* example_embed.weight         [num_examples, d] */
  ARCB_T_LN1_W,           /* blocks.L.ln1.weight          [d]               */
  ARCB_T_QKV_W,           /* blocks.L.attn.qkv_proj.weight [3d, d]          */
  ARCB_T_OUT_W,           /* blocks.L.attn.out_proj.weight [d, d]           */
  ARCB_T_LN2_W,           /* blocks.L.ln2.weight          [d]               */
  ARCB_T_GATE_W,          /* blocks.L.ffn.fc_gate.weight  [dff, d]          */
  ARCB_T_GATE_B,          /* blocks.L.ffn.fc_gate.bias    [dff]             */
  ARCB_T_UP_W,            /* blocks.L.ffn.fc_up.weight    [dff, d]          */
  ARCB_T_UP_B,            /* blocks.L.ffn.fc_up.bias      [dff]             */
  ARCB_T_DOWN_W,          /* blocks.L.ffn.fc_down.weight  [d, dff]          */
  ARCB_T_DOWN_B,          /* blocks.L.ffn.fc_down.bias    [d]               */
  ARCB_T_LNF_W,           /* ln_f.weight                  [d]               */
  ARCB_T_LM_HEAD,         /* lm_head.weight               [vocab, d]        */
  ARCB_T_ROPE_COS_X,      /* blocks.0.attn.rope.cos_x     [max_x, 10]       */
  ARCB_T_ROPE_SIN_X,
  ARCB_T_ROPE_COS_Y,      /*                              [max_y, 10]       */
  ARCB_T_ROPE_SIN_Y,
  ARCB_T_ROPE_COS_Z,      /*                              [max_z, 12]       */
  ARCB_T_ROPE_SIN_Z,
  ARCB_T_COUNT
};

const char* arcb_last_error(void);
/* 1 when the library was compiled for sm_100a and a device of compute
 * capability 10.x is current, else 0. */
int arcb_device_ok(void);

/* ---- engine: packed weights of one model ------------------------------ */

/* Replaces moving a TinyTransformer to the device (src/eval.py:881-951 ends in
 * model.to(device)); the engine keeps its own bf16 copies in kernel layout. */
int arcb_engine_create(const arcb_config* cfg, arcb_engine** out);
int arcb_engine_destroy(arcb_engine* eng);

/* Round one fp32 tensor to bf16 (the model precision) and store it in kernel layout; GEMM
 * weights are held in the 16-bit container selected by act_format.  `layer` is
 * ignored for the model-level kinds.  The copy/convert runs on `stream`. */
int arcb_engine_load_tensor(arcb_engine* eng, int32_t kind, int32_t layer, const float* d_src,
                            int64_t numel, void* stream);

/* 16-bit saturation warnings.  GEMM operands are IEEE half by default: a value beyond +-65504 on
 * its way into q16 / k16 / v16 / the SwiGLU activations is clamped, and an attention score that
 * overflows half in the flash prefill kernel becomes infinite.  Neither faults; each occurrence
 * adds one to a device counter that this call reads (after synchronising `stream`) and, with
 * reset != 0, clears.  A non-zero count means the model's activations do not fit the half format
 * and ARCB_ACT_BF16 should be used instead.  No counterpart in the reference (which runs bf16). */
int arcb_engine_saturation_count(arcb_engine* eng, int64_t* count, int32_t reset, void* stream);

/* ---- session: one batch of sequences sharing a static KV cache --------- */

/* StaticKVCache + GridStateUpdater + the per-call tensors of generate_output
 * (src/inference.py:51-96, 104-168, 539-558). */
typedef struct arcb_session_desc {
  int32_t n_seqs;             /* B: cache rows                                        */
  int32_t t_max;              /* cache positions per sequence; also the row pitch of  */
                              /* the cache: prefer t_max % 32 == 16 (an odd multiple  */
                              /* of 2 KB between streams; 1536 or 2048 rows put them  */
                              /* on the same memory channels: -3 % decode bandwidth)  */
  int32_t max_new;            /* generated-token budget per sequence                  */
  int32_t max_prefill_tokens; /* largest packed-token count of one arcb_prefill call  */
  int32_t attn_splits;        /* split-K factor of decode attention; 0 = choose       */
  int32_t stop_on_end;        /* 0: END is an ordinary token; 1: a row that emits END is
                                 counted as finished and frozen (emits END afterwards, its
                                 attention is skipped); 2: counted as finished but decoded on,
                                 as the reference does until every row of its batch has
                                 finished (src/inference.py:593-626)                      */
  void* d_kv_cache;           /* bf16 [L][2][B][H][t_max][64]                         */
  int64_t kv_cache_bytes;
  void* d_workspace;          /* >= arcb_session_workspace_bytes(...)                 */
  int64_t workspace_bytes;
  int32_t* d_out_tokens;      /* int32 [B][max_new]: generated tokens                 */
  const int32_t* d_forced;    /* optional int32 [B][max_new]: teacher-forced tokens   */
  float* d_step_logits;       /* optional fp32 [B][max_new][14]: logits of every step */
  /* Soft decoding constraints (_apply_logit_constraints, src/inference.py:285-364), applied to a
   * copy of the logits before the argmax; all optional (NULL / 0 = off):                        */
  const uint8_t* d_palette_mask; /* [B][10], 1 = colour allowed; disallowed colours lose palette_penalty */
  const int32_t* d_target_shape; /* [B][2] (h, w), negative = no shape constraint for that row     */
  float palette_penalty;
  float shape_penalty;
  uint32_t disallow_token_mask;  /* bit t set: token t gets -inf (reference default: START, IO_SEP) */
  /* Sampling (src/inference.py:575-583, 612-620): temperature <= 0 = greedy argmax.  Otherwise the
   * (constrained) logits are divided by max(temperature, 1e-6), optionally cut to the top_k largest
   * (0 = all), soft-maxed and sampled by inverse CDF with the uniform number
   * u = splitmix64(sample_seed, stream id, generated index) >> 40 scaled to [0, 1): a counter-based
   * stream, reproducible for a seed and independent of batch shape (torch.multinomial's stream
   * cannot be reproduced on the device).  The stream id of a row is d_sample_stream[row] when that
   * array is given, else the row index; a caller that spreads one job over several sessions or
   * ranks passes a job-wide id per row (e.g. the variant number) so that no two sequences of the
   * job share a stream and the draw does not depend on how the job was split. */
  float temperature;
  int32_t top_k;
  uint64_t sample_seed;
  const int32_t* d_sample_stream; /* optional int32 [B] */
} arcb_session_desc;

int64_t arcb_session_workspace_bytes(const arcb_engine* eng, int32_t n_seqs,
                                     int32_t max_prefill_tokens, int32_t attn_splits);
int64_t arcb_kv_cache_bytes(const arcb_engine* eng, int32_t n_seqs, int32_t t_max);
/* Creating a session launches nothing: the session's device state (inside d_workspace) is cleared
 * by the session's FIRST arcb_prefill, on that call's stream, so a workspace recycled from an
 * earlier session is ordered after whatever that stream still has queued on it.  Use one stream
 * (or your own ordering) for all calls of a session. */
int arcb_session_create(arcb_engine* eng, const arcb_session_desc* desc, arcb_session** out);
int arcb_session_destroy(arcb_session* s);

/* One packed-prompt forward over the cache: _prefill (src/inference.py:383-424)
 * and, with d_logits_all, TinyTransformer.forward (src/transformer.py:562-599).
 *
 * Rows are query tokens in any order grouped by sequence.  A row with
 * kv_slot >= 0 stores its K/V at that cache position of its sequence; a row
 * with kv_slot < 0 is query-only (a padded position).  kv_count is the number
 * of cached positions [0, kv_count) the row attends to (causal AND key-padding
 * mask expressed as a prefix length over the compacted keys).
 *
 * The n_first rows named by d_first_row produce the first generated token of
 * the sequences d_first_seq (src/inference.py:417-424, 573-590) and arm the
 * decode state of those sequences (prompt length, grid state, example id). */
typedef struct arcb_prefill_args {
  int32_t n_tokens;
  const int32_t* d_token_ids;  /* [n_tokens]                                   */
  const int32_t* d_pos_xyz;    /* [n_tokens][3]                                */
  const int32_t* d_seq;        /* [n_tokens] cache row of each token           */
  const int32_t* d_kv_slot;    /* [n_tokens]                                   */
  const int32_t* d_kv_count;   /* [n_tokens]                                   */
  const int32_t* d_example_ids; /* [B] indexed by cache row (NULL = no example embedding) */
  /* tensor-core prefill attention work list (optional; without it the streaming kernel runs):
   * query blocks of <= 256 consecutive rows of one sequence, and where each row's K/V goes in
   * the call's contiguous 16-bit K/V scratch (a sequence's keys are consecutive rows in slot order) */
  int32_t n_qblocks;
  const int32_t* d_qblock_row0; /* [n_qblocks] first packed row                */
  const int32_t* d_qblock_rows; /* [n_qblocks] rows in block (1..256)          */
  const int32_t* d_qblock_kv0;  /* [n_qblocks] first scratch row of the block's sequence */
  const int32_t* d_kv_row;      /* [n_tokens] scratch row of the token's K/V, < 0: none  */
  int32_t n_kv_rows;            /* scratch rows written by this call (all in [0, n_kv_rows)) */
  int32_t kv_row_identity;      /* 1 = promise that d_kv_row[i] == i for i < n_kv_rows and < 0 after
                                   (packed prompts with query-only rows, if any, at the end): the
                                   scratch rows are then written with bulk tensor stores */
  float* d_logits_all;         /* optional [n_tokens][14]                      */
  int32_t n_first;
  const int32_t* d_first_row;  /* [n_first] packed row whose hidden state is read */
  const int32_t* d_first_seq;  /* [n_first] cache row it belongs to            */
  const int32_t* d_prompt_len; /* [n_first] cached prompt positions of that row   */
  const int32_t* d_grid_x;     /* [n_first] _derive_initial_state_from_prompt  */
  const int32_t* d_grid_y;     /*           (src/inference.py:171-221)         */
  const int32_t* d_grid_in_output;
  float* d_first_logits;       /* optional [n_first][14]                       */
} arcb_prefill_args;

int arcb_prefill(arcb_session* s, const arcb_prefill_args* a, void* stream);

/* n_steps iterations of the greedy loop body (src/inference.py:593-626):
 * GridStateUpdater.update -> _decode_step -> argmax -> finished/END handling,
 * each iteration one replay of a CUDA graph captured on first use. */
int arcb_decode(arcb_session* s, int32_t n_steps, void* stream);

/* Synchronises `stream`, then reports how many rows have emitted END and the
 * device error word (0 = none). Replaces `finished.all()` (src/inference.py:594). */
int arcb_session_poll(arcb_session* s, int32_t* n_finished, int32_t* device_error, void* stream);

/* Device time (ms) of the layer-0 decode-attention launch (split kernel + combine) in the most
 * recent decode step: an event pair recorded as nodes of the step graph.  A measurement aid with no
 * counterpart in the reference; the cached lengths it ran at are prompt length + generated so far. */
int arcb_session_attention_probe(arcb_session* s, float* ms);

/* Number of kernels the library has launched since the counter was last reset
 * (graph replays count the kernels inside the graph). */
int64_t arcb_launch_count(int reset);

/* ---- standalone operators (unit tests, profiling, partial adoption) ---- */

/* RMSNorm.forward (src/transformer.py:45-48): out16 = act(x*rsqrt(mean(x^2)+eps)*w) */
int arcb_op_rmsnorm(const float* d_x, const float* d_w, void* d_out16, int32_t rows, int32_t d,
                    float eps, int32_t act_format, void* stream);

/* y[M,N] (fp32) = A[M,K] * W[N,K]^T, A and W both in the 16-bit format `act_format`
 * (the tensor-core MMA needs one format for both operands): nn.Linear without bias as used
 * at src/inference.py:402,410 / src/transformer.py:260-263.
 * gemm_path selects the tcgen05 or the CUDA-core kernel. */
int arcb_op_gemm(const void* d_a16, const void* d_w16, float* d_y, int32_t M, int32_t N,
                 int32_t K, int32_t act_format, int32_t gemm_path, void* stream);

/* x[M,N] (fp32, in place) += A[M,K] * W[N,K]^T (+ bias[N], may be NULL): a linear layer followed by
 * the residual add, as out_proj at src/inference.py:410-412 / 453-455 and the FFN's down projection
 * at src/transformer.py:446-451 with src/inference.py:413 / 456.  The tensor-core kernels add through
 * a bulk tensor reduce; every element receives one addend, so the result is deterministic. */
int arcb_op_gemm_residual(const void* d_a16, const void* d_w16, const float* d_bias, float* d_x, int32_t M,
                          int32_t N, int32_t K, int32_t act_format, int32_t gemm_path, void* stream);

/* The same operation through the split-K kernel the decode step uses when a launch has too few
 * rows to give every SM a 128 x 128 tile (e.g. 1024 x 1280): pairs of CTAs each accumulate half of K
 * and combine in a fixed order through d_scratch before the one reduce-add per element, so the
 * result stays deterministic.  arcb_gemm_splitk_scratch_bytes returns the scratch size, or 0 when
 * the kernel does not apply to the shape (the call is then rejected).  No counterpart in the
 * reference: it is an implementation of the same nn.Linear + residual add. */
int64_t arcb_gemm_splitk_scratch_bytes(int32_t M, int32_t N, int32_t K);
int arcb_op_gemm_residual_splitk(const void* d_a16, const void* d_w16, const float* d_bias, float* d_x, int32_t M,
                                 int32_t N, int32_t K, int32_t act_format, void* d_scratch, void* stream);

/* Attention of one query vector per item over a cached K/V prefix:
 * F.scaled_dot_product_attention at src/inference.py:452 (is_causal=False, key mask
 * expressed as a length).  q16/out16: [n_items][H][64]; K, V: [B][H][t_max][64] bf16;
 * item i reads cache row d_item_seq[i] (NULL = i), positions [0, d_item_len[i]).
 * With n_splits > 1, d_scratch must hold arcb_attn_scratch_bytes(...) bytes. */
int64_t arcb_attn_scratch_bytes(int32_t n_items, int32_t n_heads, int32_t n_splits);
int arcb_op_decode_attention(const void* d_q16, const void* d_k, const void* d_v, void* d_out16,
                             const int32_t* d_item_seq, const int32_t* d_item_len,
                             const uint8_t* d_item_skip, int32_t n_items, int32_t n_heads,
                             int32_t t_max, int32_t n_splits, void* d_scratch, int32_t act_format,
                             void* stream);

/* Same operation as arcb_op_decode_attention for callers that cannot allocate device memory
 * (a serving loop with a fixed memory pool, a plugin living inside another framework's allocator,
 * code inside a region where cudaMalloc/cudaFree and their implicit synchronisation are
 * forbidden).  It has no counterpart in the reference, which never leaves PyTorch's allocator.
 * The per-split partial results live in an array built into the library instead of a caller
 * buffer, so there is no d_scratch argument and the call makes no allocation of any kind.
 *   - limit: n_items * n_heads * n_splits <= ARCB_STATIC_ATTN_MAX_RECORDS (4.25 MiB of scratch,
 *     held by every GPU that loads the library until the process exits); larger requests return
 *     ARCB_E_ARG with a message;
 *   - the first call on a device resolves the array's address on that device; make that first
 *     call before any CUDA stream capture;
 *   - all calls on a device share the array, which keeps the last call's contents (nothing in
 *     it needs to start at zero); calls that overlap on the GPU race, so keep them on one stream
 *     or otherwise ordered. */
#define ARCB_STATIC_ATTN_MAX_RECORDS 16384
int arcb_op_decode_attention_static(const void* d_q16, const void* d_k, const void* d_v, void* d_out16,
                                    const int32_t* d_item_seq, const int32_t* d_item_len,
                                    const uint8_t* d_item_skip, int32_t n_items, int32_t n_heads,
                                    int32_t t_max, int32_t n_splits, int32_t act_format, void* stream);

/* ln_f -> lm_head -> argmax (src/inference.py:418/424/459 + 574/611): logits fp32
 * [rows][14] and the index of the first maximum. d_row_index (optional) gathers rows of x. */
int arcb_op_head(const float* d_x, const int32_t* d_row_index, const float* d_lnf_w,
                 const float* d_lm_head, float* d_logits, int32_t* d_argmax, int32_t rows,
                 int32_t d, float eps, void* stream);

/* --------------------------------------------------------------------------
 * Augmentation fan-out on the device (integer / byte work, bit-exact).
 *
 * Replaces the per-cell Python loops either side of generation: prompt construction for every
 * (dihedral x colour permutation) variant of a task (src/inference.py:794-827 with
 * src/data.py:40-93, 124-233 and src/inference.py:1006-1008) and the way back from generated
 * tokens to a canonical candidate grid (src/inference.py:906-915, src/data.py:95-117,
 * src/voting.py:19-54, 57-108).
 * -------------------------------------------------------------------------- */

/* Grids of the tasks, uploaded once: row-major uint8 cells, one (offset, h, w) triple per grid.
 * A prompt template lists the grids of one (task, test input) in prompt order: train input 0,
 * train output 0, ..., test input (odd entries are outputs), at most ARCB_MAX_TEMPLATE_GRIDS. */
#define ARCB_MAX_TEMPLATE_GRIDS 64
typedef struct arcb_prompt_build_args {
  int32_t n_variants;
  int32_t n_perms;                 /* rows of d_perm_lut */
  const uint8_t* d_cells;
  const int32_t* d_grid_off;       /* [n_grids] first cell of each grid */
  const int32_t* d_grid_h;         /* [n_grids] */
  const int32_t* d_grid_w;         /* [n_grids] */
  const int32_t* d_tpl_off;        /* [n_templates + 1] range of each template in d_tpl_grid */
  const int32_t* d_tpl_grid;       /* grid ids */
  const uint8_t* d_perm_lut;       /* [n_perms][10] old colour -> new colour */
  /* per variant */
  const int32_t* d_var_template;
  const int32_t* d_var_dihedral;   /* 0..7, the order of src/data.py:224-233 */
  const int32_t* d_var_perm;       /* row of d_perm_lut */
  const int32_t* d_var_tok_off;    /* [n_variants + 1] first packed token of each variant */
  const int32_t* d_var_seq;        /* cache row of each variant */
  /* packed outputs, [d_var_tok_off[n_variants]] each (d_pos_xyz three per token): the arrays
   * arcb_prefill_args takes for unpadded causal prompts (kv_slot = index in the sequence,
   * kv_count = kv_slot + 1, kv_row = packed index). Any may be NULL. */
  int32_t* d_token_ids;
  int32_t* d_pos_xyz;
  int32_t* d_seq;
  int32_t* d_kv_slot;
  int32_t* d_kv_count;
  int32_t* d_kv_row;
  int32_t* d_status;               /* optional: set to a non-zero ARCB_DEV_* code when a variant's
                                      length differs from its d_var_tok_off range or a template is
                                      too long; the variant is then left unwritten */
} arcb_prompt_build_args;

int arcb_build_prompts(const arcb_prompt_build_args* args, void* stream);

/* One fixed-width record per generated sequence: the candidate grid mapped back to the task's own
 * orientation and colours. status: 0 = no grid (nothing between the last IO_SEP and END),
 * 1 = rectangular grid, 2 = malformed (jagged or only separators). input_copy = 1 when the grid as
 * generated (before mapping back) equals the task's test input, which is the comparison
 * src/voting.py:92 makes. */
#define ARCB_CANDIDATE_MAX_CELLS 936
typedef struct arcb_candidate_record {
  uint8_t status;
  uint8_t input_copy;
  uint16_t h;
  uint16_t w;
  uint16_t n_tokens;               /* generated tokens up to and including the first END */
  uint8_t cells[ARCB_CANDIDATE_MAX_CELLS];   /* row-major h x w */
} arcb_candidate_record;           /* 944 bytes */

typedef struct arcb_candidate_args {
  int32_t n_rows;
  int32_t max_new;                 /* tokens per row, <= ARCB_CANDIDATE_MAX_CELLS */
  const int32_t* d_tokens;         /* [n_rows][max_new] generated tokens (the session's d_out_tokens) */
  const int32_t* d_row_dihedral;   /* [n_rows] transform the prompt was built with; < 0 = padding row */
  const int32_t* d_row_perm;       /* [n_rows] row of d_perm_lut */
  const uint8_t* d_perm_lut;       /* [n_perms][10] old -> new (the forward map; inverted here) */
  int32_t n_perms;
  int32_t reserved;
  /* optional test inputs for the input-copy flag */
  const int32_t* d_row_test_grid;  /* [n_rows] grid id, < 0 = none */
  const uint8_t* d_cells;
  const int32_t* d_grid_off;
  const int32_t* d_grid_h;
  const int32_t* d_grid_w;
  arcb_candidate_record* d_records; /* [n_rows] */
} arcb_candidate_args;

int arcb_canonicalize_candidates(const arcb_candidate_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ARCB200_H */
