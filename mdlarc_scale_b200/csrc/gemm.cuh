// Host-side launcher of the GEMM kernels (see gemm.cu).
#pragma once
#include <cuda.h>
#include "epilogue.cuh"

// A: [M][K] and W: [N][K], both half when act_f16, else both bfloat16.
// Requires N % 128 == 0; the tcgen05 path also K % 64 == 0, the CUDA-core path K % 32 == 0.
// Returns 0, a negative argument error, a cudaError_t, or 1000 + CUresult of the tensor-map encode.
// tc_variant: 0 = choose between the 1-CTA and the 2-CTA (cta_group::2) tensor-core kernels by
// tile count, 1 = 1-CTA kernels only, 2 = 2-CTA kernel whenever clusters can be scheduled.
int arcb_launch_gemm(const void* a16, const void* w16, const GemmEpilogue& ep, int K, int act_f16,
                     bool use_tc, cudaStream_t stream, int tc_variant = 0);
int arcb_gemm_max_pairs();
int arcb_gemm_splitk_bn(int M, int N, int K);
int arcb_gemm_init();
bool arcb_gemm_tc_supported(int M, int N, int K);
int arcb_make_tmap_2d_16b(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                          uint32_t box_rows, uint32_t box_cols, int is_f16);
void arcb_count_launch(long long n);
