// Shared device helpers: 16-bit activation packing, error word, launch counter.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define ARCB_HEAD_DIM 64
#define ARCB_VOCAB 14
#define ARCB_ROPE_PX 10  // rotary pairs driven by x   (src/transformer.py:87-90 with head_dim 64)
#define ARCB_ROPE_PY 10  // rotary pairs driven by y
#define ARCB_ROPE_PZ 12  // rotary pairs driven by z

enum : int { TOK_START = 10, TOK_NEWLINE = 11, TOK_IOSEP = 12, TOK_END = 13 };

// Device error codes written (atomicCAS, first writer wins) to the engine's error word.
enum : int {
  ARCB_DEV_OK = 0,
  ARCB_DEV_WAIT_TIMEOUT_TMA = 1,   // a consumer gave up waiting for a TMA stage
  ARCB_DEV_WAIT_TIMEOUT_MMA = 2,   // the producer gave up waiting for a free stage
  ARCB_DEV_WAIT_TIMEOUT_ACC = 3,   // the epilogue gave up waiting for the accumulator
  ARCB_DEV_BAD_INDEX = 4,          // a cache slot / length was out of range and skipped
};

__device__ __forceinline__ void arcb_set_error(int* err, int code) {
  if (err) atomicCAS(err, 0, code);
}

// Word 1 of the error block counts 16-bit saturations: values the half format cannot hold that were
// clamped to +-65504 on their way into a GEMM operand (or a score that overflowed to infinity).
// It is a warning, not an error: the run continues, the host reads and clears the count.
__device__ __forceinline__ void arcb_count_saturation(int* err) {
  if (err) atomicAdd(err + 1, 1);
}

// ---- programmatic dependent launch (see launch.cuh for the protocol) ----
// Both are no-ops for a kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- 16-bit activation formats -------------------------------------------
// act_f16 != 0: IEEE half (values clamped to the finite half range), else bfloat16.

__device__ __forceinline__ uint32_t pack2_act(float a, float b, int act_f16) {
  if (act_f16) {
    a = fminf(fmaxf(a, -65504.f), 65504.f);
    b = fminf(fmaxf(b, -65504.f), 65504.f);
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// pack2_act that also reports a clamp (half format only) in the saturation counter
__device__ __forceinline__ uint32_t pack2_act_chk(float a, float b, int act_f16, int* err) {
  if (act_f16 && fmaxf(fabsf(a), fabsf(b)) > 65504.f) arcb_count_saturation(err);
  return pack2_act(a, b, act_f16);
}

__device__ __forceinline__ float2 unpack2_act(uint32_t v, int act_f16) {
  if (act_f16) {
    __half2 h = *reinterpret_cast<__half2*>(&v);
    return __half22float2(h);
  }
  float2 r;
  r.x = __uint_as_float(v << 16);
  r.y = __uint_as_float(v & 0xffff0000u);
  return r;
}

__device__ __forceinline__ float2 unpack2_bf16(uint32_t v) {
  float2 r;
  r.x = __uint_as_float(v << 16);
  r.y = __uint_as_float(v & 0xffff0000u);
  return r;
}

__device__ __forceinline__ uint32_t pack2_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Streaming 16-byte load that does not allocate in L1 (data is read once).
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
