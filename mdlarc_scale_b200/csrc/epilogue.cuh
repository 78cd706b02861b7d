// GEMM epilogues shared by the tcgen05 and the CUDA-core GEMM kernels.
// Every epilogue consumes the accumulator in "quads": 4 consecutive output
// columns of one row, which is enough to keep RoPE pairs (2p, 2p+1) together.
#pragma once
#include "common.cuh"

enum : int {
  EPI_STORE_F32 = 0,  // y[m][n] = acc                               (tests)
  EPI_QKV_ROPE = 1,   // 3D RoPE on q,k; q -> q16, k/v -> KV cache    (src/inference.py:402-407)
  EPI_RESID = 2,      // x[m][n] += acc (+ bias[n])                   (src/inference.py:410-413)
  EPI_SWIGLU = 3,     // h16[m][j] = silu(g+bg) * (u+bu)              (src/transformer.py:446-449)
};

struct GemmEpilogue {
  int mode;
  int M, N;      // GEMM output extent (N counts packed columns for EPI_SWIGLU)
  int act_f16;   // format of 16-bit outputs (q16 / h16)
  float* y;      // EPI_STORE_F32: [M][N]
  float* x;      // EPI_RESID: residual stream [M][N], updated in place
  const float* bias;  // EPI_RESID: [N] or null; EPI_SWIGLU: [N] packed like the weight rows
  float* splitk_scratch;  // EPI_RESID, optional: >= 128 * ceil(M / 128) * N floats; allows the split-K kernel for few-row launches
  void* out16;   // EPI_QKV_ROPE: q16 [M][d]; EPI_SWIGLU: h16 [M][N/2]
  // EPI_QKV_ROPE
  const int* pos;   // [M][3] raw (x, y, z); clamped here like RotaryEmbedding3D.apply_rotary
  const int* slot;  // [M] cache position of the row's K/V, < 0: do not store
  const int* seq;   // [M] cache row (sequence) of the token; null = row index
  __nv_bfloat16* kcache;  // layer K base [B][H][t_max][64]
  __nv_bfloat16* vcache;  // layer V base
  void* k16;              // optional [n_kv_rows][d]: K of this call in the activation format
  void* v16;              //   (operands of the tensor-core prefill attention)
  const int* kv_row;      // [M] row of k16/v16 for this token, < 0: none
  int kv16_rows;          // rows of k16 / v16
  int kv16_identity;      // kv_row[m] == m for m < kv16_rows and < 0 after: rows can be stored as boxes
  int t_max, n_heads, d_model, n_seqs;
  const float* rope;  // cos_x | sin_x | cos_y | sin_y | cos_z | sin_z
  int max_x, max_y, max_z;
  int* err;           // error word; word 1 counts 16-bit saturations
};

struct RopeRow {
  int x, y, z;
  long long kv_row;  // (seq * H) * t_max + slot, or -1
  int row16;         // row of k16/v16, or -1
};

__device__ __forceinline__ RopeRow rope_row_ctx(const GemmEpilogue& e, int m) {
  RopeRow r;
  r.row16 = (e.k16 && e.kv_row) ? e.kv_row[m] : -1;
  const int px = e.pos[3 * m + 0], py = e.pos[3 * m + 1], pz = e.pos[3 * m + 2];
  r.x = min(max(px, 0), e.max_x - 1);
  r.y = min(max(py, 0), e.max_y - 1);
  r.z = min(max(pz, 0), e.max_z - 1);
  const int s = e.slot[m];
  const int b = e.seq ? e.seq[m] : m;
  if (s < 0) {
    r.kv_row = -1;
  } else if (s >= e.t_max || b < 0 || b >= e.n_seqs) {
    arcb_set_error(e.err, ARCB_DEV_BAD_INDEX);
    r.kv_row = -1;
  } else {
    r.kv_row = ((long long)b * e.n_heads) * e.t_max + s;
  }
  return r;
}

// cos/sin of rotary pair p (0..31) at the row's clamped position.
__device__ __forceinline__ float2 rope_cs(const GemmEpilogue& e, const RopeRow& r, int p) {
  const float* t = e.rope;
  const int nx = e.max_x * ARCB_ROPE_PX, ny = e.max_y * ARCB_ROPE_PY, nz = e.max_z * ARCB_ROPE_PZ;
  int ic;
  if (p < ARCB_ROPE_PX) {
    ic = r.x * ARCB_ROPE_PX + p;
    return make_float2(__ldg(t + ic), __ldg(t + nx + ic));
  } else if (p < ARCB_ROPE_PX + ARCB_ROPE_PY) {
    ic = r.y * ARCB_ROPE_PY + (p - ARCB_ROPE_PX);
    return make_float2(__ldg(t + 2 * nx + ic), __ldg(t + 2 * nx + ny + ic));
  }
  ic = r.z * ARCB_ROPE_PZ + (p - ARCB_ROPE_PX - ARCB_ROPE_PY);
  return make_float2(__ldg(t + 2 * nx + 2 * ny + ic), __ldg(t + 2 * nx + 2 * ny + nz + ic));
}

// out[2p] = v[2p] cos - v[2p+1] sin ; out[2p+1] = v[2p+1] cos + v[2p] sin
// (src/transformer.py:51-58, 184-185)
__device__ __forceinline__ void epi_qkv_quad(const GemmEpilogue& e, const RopeRow& r, int m, int n,
                                             float4 v) {
  const int d = e.d_model;
  const int sec = n / d;           // 0 q, 1 k, 2 v
  const int c = n - sec * d;       // column inside the section
  const int h = c >> 6, dim = c & 63;
  if (sec < 2) {
    const int p = dim >> 1;
    const float2 cs0 = rope_cs(e, r, p), cs1 = rope_cs(e, r, p + 1);
    float4 o;
    o.x = v.x * cs0.x - v.y * cs0.y;
    o.y = v.y * cs0.x + v.x * cs0.y;
    o.z = v.z * cs1.x - v.w * cs1.y;
    o.w = v.w * cs1.x + v.z * cs1.y;
    v = o;
  }
  if (sec == 0) {
    uint2 pk;
    pk.x = pack2_act_chk(v.x, v.y, e.act_f16, e.err);
    pk.y = pack2_act_chk(v.z, v.w, e.act_f16, e.err);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(e.out16) + (size_t)m * d + c) = pk;
  } else {
    if (r.kv_row >= 0) {
      __nv_bfloat16* base = (sec == 1) ? e.kcache : e.vcache;
      const long long row = r.kv_row + (long long)h * e.t_max;
      uint2 pk;
      pk.x = pack2_bf16(v.x, v.y);
      pk.y = pack2_bf16(v.z, v.w);
      *reinterpret_cast<uint2*>(base + row * ARCB_HEAD_DIM + dim) = pk;
    }
    if (r.row16 >= 0) {
      uint16_t* base16 = reinterpret_cast<uint16_t*>((sec == 1) ? e.k16 : e.v16);
      uint2 pk;
      pk.x = pack2_act_chk(v.x, v.y, e.act_f16, e.err);
      pk.y = pack2_act_chk(v.z, v.w, e.act_f16, e.err);
      *reinterpret_cast<uint2*>(base16 + (size_t)r.row16 * d + c) = pk;
    }
  }
}

// Rotate the 16 rotary pairs [P0, P0 + 16) held in v[0..32) (P0 is 0 or 16: first or second half of
// a 64-wide head).  Which table a pair uses (x: pairs 0-9, y: 10-19, z: 20-31) is known at compile
// time, so the loop unrolls into straight table loads.
template <int P0>
__device__ __forceinline__ void rope_rotate32(const GemmEpilogue& e, const RopeRow& r, float (&v)[32]) {
  const int nx = e.max_x * ARCB_ROPE_PX, ny = e.max_y * ARCB_ROPE_PY, nz = e.max_z * ARCB_ROPE_PZ;
  const float* cx = e.rope + r.x * ARCB_ROPE_PX;
  const float* sx = cx + nx;
  const float* cy = e.rope + 2 * nx + r.y * ARCB_ROPE_PY;
  const float* sy = cy + ny;
  const float* cz = e.rope + 2 * nx + 2 * ny + r.z * ARCB_ROPE_PZ;
  const float* sz = cz + nz;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    constexpr int PX = ARCB_ROPE_PX, PXY = ARCB_ROPE_PX + ARCB_ROPE_PY;
    const int p = P0 + i;
    float c, s;
    if (p < PX) { c = __ldg(cx + p); s = __ldg(sx + p); }
    else if (p < PXY) { c = __ldg(cy + (p - PX)); s = __ldg(sy + (p - PX)); }
    else { c = __ldg(cz + (p - PXY)); s = __ldg(sz + (p - PXY)); }
    const float a = v[2 * i], b = v[2 * i + 1];
    v[2 * i] = a * c - b * s;
    v[2 * i + 1] = b * c + a * s;
  }
}

// 32 consecutive QKV output columns [n0, n0 + 32) of row m (n0 % 32 == 0: one half of one head of
// one of the q / k / v sections): RoPE on q and k, then 16-byte stores of q16 or of the bf16 cache
// row (+ the call's 16-bit K/V scratch row).
__device__ __forceinline__ void epi_qkv_chunk32(const GemmEpilogue& e, const RopeRow& r, int m, int n0,
                                                const uint32_t (&acc)[32]) {
  const int d = e.d_model;
  const int sec = n0 / d;
  const int c = n0 - sec * d;
  const int h = c >> 6, dim0 = c & 63;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
  if (sec < 2) {
    if (dim0 == 0) rope_rotate32<0>(e, r, v);
    else rope_rotate32<16>(e, r, v);
  }
  if (sec == 0) {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(e.out16) + (size_t)m * d + c);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      dst[q] = make_uint4(pack2_act_chk(v[8 * q], v[8 * q + 1], e.act_f16, e.err), pack2_act_chk(v[8 * q + 2], v[8 * q + 3], e.act_f16, e.err),
                          pack2_act_chk(v[8 * q + 4], v[8 * q + 5], e.act_f16, e.err), pack2_act_chk(v[8 * q + 6], v[8 * q + 7], e.act_f16, e.err));
    return;
  }
  if (r.kv_row >= 0) {
    __nv_bfloat16* base = (sec == 1) ? e.kcache : e.vcache;
    uint4* dst = reinterpret_cast<uint4*>(base + (r.kv_row + (long long)h * e.t_max) * ARCB_HEAD_DIM + dim0);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      dst[q] = make_uint4(pack2_bf16(v[8 * q], v[8 * q + 1]), pack2_bf16(v[8 * q + 2], v[8 * q + 3]),
                          pack2_bf16(v[8 * q + 4], v[8 * q + 5]), pack2_bf16(v[8 * q + 6], v[8 * q + 7]));
  }
  if (r.row16 >= 0) {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>((sec == 1) ? e.k16 : e.v16) +
                                          (size_t)r.row16 * d + c);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      dst[q] = make_uint4(pack2_act_chk(v[8 * q], v[8 * q + 1], e.act_f16, e.err), pack2_act_chk(v[8 * q + 2], v[8 * q + 3], e.act_f16, e.err),
                          pack2_act_chk(v[8 * q + 4], v[8 * q + 5], e.act_f16, e.err), pack2_act_chk(v[8 * q + 6], v[8 * q + 7], e.act_f16, e.err));
  }
}

__device__ __forceinline__ void epi_resid_quad(const GemmEpilogue& e, int m, int n, float4 v) {
  float4* px = reinterpret_cast<float4*>(e.x + (size_t)m * e.N + n);
  float4 r = *px;
  if (e.bias) {
    const float4 b = __ldg(reinterpret_cast<const float4*>(e.bias + n));
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
  }
  r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w;
  *px = r;
}

__device__ __forceinline__ void epi_store_quad(const GemmEpilogue& e, int m, int n, float4 v) {
  *reinterpret_cast<float4*>(e.y + (size_t)m * e.N + n) = v;
}

__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// Packed column n (n % 128 < 64) holds gate outputs, n + 64 the matching up outputs.
__device__ __forceinline__ void epi_swiglu_quad(const GemmEpilogue& e, int m, int n, float4 g,
                                                float4 u) {
  if (e.bias) {
    const float4 bg = __ldg(reinterpret_cast<const float4*>(e.bias + n));
    const float4 bu = __ldg(reinterpret_cast<const float4*>(e.bias + n + 64));
    g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w;
    u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
  }
  const int j = (n >> 7) * 64 + (n & 127);
  uint2 pk;
  pk.x = pack2_act_chk(silu_f(g.x) * u.x, silu_f(g.y) * u.y, e.act_f16, e.err);
  pk.y = pack2_act_chk(silu_f(g.z) * u.z, silu_f(g.w) * u.w, e.act_f16, e.err);
  *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(e.out16) + (size_t)m * (e.N >> 1) + j) = pk;
}
