// Flash-style causal prefill attention on tcgen05/TMEM; see attn_prefill.cu.
#pragma once
#include "common.cuh"

struct AttnPrefillArgs {
  const void* q16;          // [n_rows][H][64] 16-bit (act format), packed prompt rows
  const __nv_bfloat16* k;   // layer K base [n_seqs][H][t_max][64]
  const __nv_bfloat16* v;
  void* out16;              // [n_rows][H][64]
  const int* seq;           // [n_rows] cache row of each packed row
  const int* kv_count;      // [n_rows] attended prefix length
  const int* qblock_row0;   // [n_qblocks] first packed row of the block
  const int* qblock_rows;   // [n_qblocks] rows in the block (1..128), all of one sequence
  int n_qblocks, n_rows, n_heads, t_max, n_seqs;
  int act_f16;
  int* err;
};

bool arcb_attn_prefill_available();
int arcb_launch_attn_prefill(const AttnPrefillArgs& a, cudaStream_t stream);
void arcb_count_launch(long long n);
