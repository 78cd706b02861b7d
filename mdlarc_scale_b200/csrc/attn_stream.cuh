// Launcher of the streaming (one query per item) attention kernel; see attn_stream.cu.
#pragma once
#include "common.cuh"

constexpr int ATTN_SCRATCH_STRIDE = 68;  // floats per (item, head, split): 64 acc, m, l, pad

struct AttnStreamArgs {
  const void* q16;            // [n_items][H][64] 16-bit (act format)
  const __nv_bfloat16* k;     // [n_seqs][H][t_max][64]
  const __nv_bfloat16* v;
  void* out16;                // [n_items][H][64]
  const int* item_seq;        // [n_items] cache row, or null = item index
  const int* item_len;        // [n_items] keys [0, len) are attended
  const unsigned char* item_skip;  // optional [n_items]: non-zero = leave the row untouched (zeros)
  int n_items, n_heads, t_max, n_seqs, n_splits;
  float* scratch;             // n_items * H * n_splits * ATTN_SCRATCH_STRIDE floats when n_splits > 1
  int act_f16;
  int* err;
};

int arcb_launch_attn_stream(const AttnStreamArgs& a, cudaStream_t stream);
void arcb_count_launch(long long n);
