// Flash-style causal prefill attention on tcgen05/TMEM; see attn_prefill.cu.
#pragma once
#include "common.cuh"

struct AttnPrefillArgs {
  const void* q16;          // [n_rows][H][64] 16-bit (act format), packed prompt rows
  const void* k16;          // [n_kv_rows][H][64] keys of this call in the same 16-bit format
  const void* v16;          // [n_kv_rows][H][64]
  void* out16;              // [n_rows][H][64]
  const int* seq;           // [n_rows] cache row of each packed row
  const int* kv_count;      // [n_rows] attended prefix length
  const int* qblock_row0;   // [n_qblocks] first packed row of the block
  const int* qblock_rows;   // [n_qblocks] rows in the block (1..256), all of one sequence
  const int* qblock_kv0;    // [n_qblocks] first K/V scratch row of the block's sequence
  int n_qblocks, n_rows, n_kv_rows, n_heads;
  int act_f16;
  int* err;
};

bool arcb_attn_prefill_available();
int arcb_attn_prefill_init();
int arcb_launch_attn_prefill(const AttnPrefillArgs& a, cudaStream_t stream);
void arcb_count_launch(long long n);
