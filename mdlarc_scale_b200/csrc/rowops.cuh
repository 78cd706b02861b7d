// Argument blocks and launchers of the row-wise kernels; see rowops.cu.
#pragma once
#include "common.cuh"

// Device-resident state of the greedy loop for one session (all arrays indexed by cache row).
struct DecodeState {
  int n_seqs, t_max, max_new, stop_on_end;
  int* cur_len;     // cached positions so far
  int* len0;        // cached prompt positions (cur_len when decoding started)
  int* cur_tok;     // token fed by the next decode step
  int* gx; int* gy; int* gin;  // grid state: next column, row, inside-output flag
  int* pos;         // [B][3] position of the fed token (written by decode_begin)
  int* slot;        // [B] cache position the step writes
  int* kv_len;      // [B] keys the step attends to
  unsigned char* finished;  // [B]
  int* n_finished;
  int* out_tokens;          // [B][max_new]
  const int* forced;        // optional [B][max_new]
  float* step_logits;       // optional [B][max_new][14] (raw logits, before constraints)
  // soft decoding constraints (all optional)
  const unsigned char* palette_mask;  // [B][10], 1 = allowed
  const int* target_shape;            // [B][2] (h, w), negative = none
  float palette_penalty, shape_penalty;
  unsigned int disallow_mask;         // bit t: token t -> -inf
  // sampling: temperature <= 0 = greedy
  float temperature;
  int top_k;
  unsigned long long sample_seed;
  const int* sample_stream;   // optional [B]: random-stream id of each row (default: the row index)
  int* err;
};

struct EmbedArgs {
  int rows, d, vocab, num_examples;
  const int* token_ids;     // [rows] (unused by decode_begin)
  const int* seq;           // [rows] cache row per token, null = row index
  const int* example_ids;   // indexed by cache row; null = no example embedding
  const float* token_embed; // [vocab][d]
  const float* example_embed;
  const float* ln_w;        // first RMSNorm weight
  float* x;                 // [rows][d] residual stream out
  uint16_t* xn16;           // [rows][d] normalised, 16-bit
  float eps;
  int act_f16;
};

enum : int { HEAD_PLAIN = 0, HEAD_FIRST = 1, HEAD_DECODE = 2 };

struct HeadArgs {
  int mode;
  int rows, d;
  float eps;
  const float* x;
  const int* row_index;  // optional gather of rows of x
  const float* lnf_w;
  const float* lm_head;  // [14][d]
  float* logits;         // optional [rows][14]
  int* argmax;           // optional [rows]
  // HEAD_FIRST only
  const int* first_seq; const int* prompt_len;
  const int* grid_x; const int* grid_y; const int* grid_in_output;
};

int arcb_launch_rmsnorm(const float* x, const float* w, void* out16, int rows, int d, float eps,
                        int act_f16, cudaStream_t stream);
int arcb_launch_embed_norm(const EmbedArgs& a, cudaStream_t stream);
int arcb_launch_decode_begin(const DecodeState& st, const EmbedArgs& a, cudaStream_t stream);
int arcb_launch_head(const HeadArgs& a, const DecodeState& st, cudaStream_t stream);
int arcb_launch_pack_rows(const float* src, void* dst, long long rows, long long cols, int blk,
                          int blk_stride, int blk_off, int to_bf16, cudaStream_t stream);
void arcb_count_launch(long long n);
