// Row-wise kernels (one warp per row, HBM-bound, float4 accesses):
//   embed_norm    : token + example embedding -> residual stream, fused first RMSNorm
//   rmsnorm       : RMSNorm of the residual stream -> 16-bit GEMM operand
//   decode_begin  : grid-state position update + embedding + first RMSNorm of a decode step
//   head          : final RMSNorm -> 14 logits -> argmax (+ greedy-loop bookkeeping)
//   pack_rows     : fp32 -> bf16-rounded weights in kernel layout
#include "rowops.cuh"
#include "launch.cuh"

namespace {

constexpr int ROWS_PER_CTA = 4;

// sum of squares of a row held in global memory, warp-cooperative
__device__ __forceinline__ float row_sumsq(const float* __restrict__ x, int d, int lane) {
  float ss = 0.f;
  for (int i = lane * 4; i < d; i += 128) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  return warp_sum(ss);
}

// out16 = (x * rsqrt(mean(x^2) + eps)) * w    (src/transformer.py:45-48)
// Rows of up to 128 * NV floats are held in registers: every load of the row is in flight at once
// and the row is read from memory once.  The sum of squares is accumulated in the same order as
// row_sumsq, so both forms give the same bits.
template <int NV>
__device__ __forceinline__ void row_norm_store_regs(const float* __restrict__ x, const float* __restrict__ w,
                                                    uint16_t* __restrict__ out, int d, float eps, int act_f16,
                                                    int lane) {
  float4 v[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane * 4 + k * 128;
    v[k] = (i < d) ? *reinterpret_cast<const float4*>(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (lane * 4 + k * 128 < d) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = lane * 4 + k * 128;
    if (i < d) {
      const float4 g = __ldg(reinterpret_cast<const float4*>(w + i));
      uint2 pk;
      pk.x = pack2_act((v[k].x * inv) * g.x, (v[k].y * inv) * g.y, act_f16);
      pk.y = pack2_act((v[k].z * inv) * g.z, (v[k].w * inv) * g.w, act_f16);
      *reinterpret_cast<uint2*>(out + i) = pk;
    }
  }
}

__device__ __forceinline__ void row_norm_store(const float* __restrict__ x, const float* __restrict__ w,
                                               uint16_t* __restrict__ out, int d, float eps, int act_f16,
                                               int lane) {
  if (d <= 128 * 2) return row_norm_store_regs<2>(x, w, out, d, eps, act_f16, lane);
  if (d <= 128 * 6) return row_norm_store_regs<6>(x, w, out, d, eps, act_f16, lane);
  if (d <= 128 * 10) return row_norm_store_regs<10>(x, w, out, d, eps, act_f16, lane);
  if (d <= 128 * 16) return row_norm_store_regs<16>(x, w, out, d, eps, act_f16, lane);
  const float ss = row_sumsq(x, d, lane);
  const float inv = rsqrtf(ss / (float)d + eps);
  for (int i = lane * 4; i < d; i += 128) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    const float4 g = __ldg(reinterpret_cast<const float4*>(w + i));
    uint2 pk;
    pk.x = pack2_act((v.x * inv) * g.x, (v.y * inv) * g.y, act_f16);
    pk.y = pack2_act((v.z * inv) * g.z, (v.w * inv) * g.w, act_f16);
    *reinterpret_cast<uint2*>(out + i) = pk;
  }
}

__device__ __forceinline__ void row_embed(float* __restrict__ x, const float* __restrict__ tok_row,
                                          const float* __restrict__ ex_row, int d, int lane) {
  for (int i = lane * 4; i < d; i += 128) {
    float4 v = __ldg(reinterpret_cast<const float4*>(tok_row + i));
    if (ex_row) {
      const float4 e = __ldg(reinterpret_cast<const float4*>(ex_row + i));
      v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
    }
    *reinterpret_cast<float4*>(x + i) = v;
  }
  __syncwarp();
}

__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, uint16_t* __restrict__ out,
               int rows, int d, float eps, int act_f16) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= rows) return;
  row_norm_store(x + (size_t)row * d, w, out + (size_t)row * d, d, eps, act_f16, threadIdx.x & 31);
}

__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
embed_norm_kernel(EmbedArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int lane = threadIdx.x & 31;
  int tok = a.token_ids[row];
  tok = min(max(tok, 0), a.vocab - 1);
  const float* ex_row = nullptr;
  if (a.example_ids) {
    int ex = a.example_ids[a.seq ? a.seq[row] : row];
    ex = min(max(ex, 0), a.num_examples - 1);
    ex_row = a.example_embed + (size_t)ex * a.d;
  }
  float* x = a.x + (size_t)row * a.d;
  row_embed(x, a.token_embed + (size_t)tok * a.d, ex_row, a.d, lane);
  row_norm_store(x, a.ln_w, a.xn16 + (size_t)row * a.d, a.d, a.eps, a.act_f16, lane);
}

// GridStateUpdater.update (src/inference.py:127-168) for one sequence, then the
// embedding of the fed token and the first RMSNorm of the step.
__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
decode_begin_kernel(DecodeState st, EmbedArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (b >= st.n_seqs) return;
  const int lane = threadIdx.x & 31;
  const int tok = st.cur_tok[b];
  if (lane == 0) {
    int x = st.gx[b], y = st.gy[b], in_out = st.gin[b];
    const bool is_start = tok == TOK_START, is_sep = tok == TOK_IOSEP, is_end = tok == TOK_END,
               is_nl = tok == TOK_NEWLINE, is_color = tok < 10;
    int z = in_out ? 3 : 1;
    if (is_start) z = 0;
    if (is_sep) z = 2;
    if (is_end) z = 4;
    const int xc = min(max(x, 0), 30), yc = min(max(y, 0), 29);
    st.pos[3 * b + 0] = (is_start || is_sep || is_end || is_nl) ? 0 : xc;
    st.pos[3 * b + 1] = (is_start || is_sep || is_end) ? 0 : yc;
    st.pos[3 * b + 2] = z;
    if (is_start || is_sep) { x = 0; y = 0; }
    if (is_start) in_out = 0;
    if (is_sep) in_out = 1;
    if (is_nl) { x = 0; y = min(y + 1, 29); }
    if (is_color) x = min(x + 1, 30);
    st.gx[b] = min(max(x, 0), 30);
    st.gy[b] = min(max(y, 0), 29);
    st.gin[b] = in_out;
    const int len = st.cur_len[b];
    if (len >= st.t_max) {
      // cache row is full: drop the key and attend to what is there
      arcb_set_error(st.err, ARCB_DEV_BAD_INDEX);
      st.slot[b] = -1;
      st.kv_len[b] = st.t_max;
    } else {
      st.slot[b] = len;
      st.kv_len[b] = len + 1;
    }
  }
  const int tk = min(max(tok, 0), a.vocab - 1);
  const float* ex_row = nullptr;
  if (a.example_ids) {
    int ex = a.example_ids[b];
    ex = min(max(ex, 0), a.num_examples - 1);
    ex_row = a.example_embed + (size_t)ex * a.d;
  }
  float* x = a.x + (size_t)b * a.d;
  row_embed(x, a.token_embed + (size_t)tk * a.d, ex_row, a.d, lane);
  row_norm_store(x, a.ln_w, a.xn16 + (size_t)b * a.d, a.d, a.eps, a.act_f16, lane);
}

__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
head_kernel(HeadArgs a, DecodeState st) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (i >= a.rows) return;
  const int lane = threadIdx.x & 31;
  const int row = a.row_index ? a.row_index[i] : i;
  const float* x = a.x + (size_t)row * a.d;
  const float ss = row_sumsq(x, a.d, lane);
  const float inv = rsqrtf(ss / (float)a.d + a.eps);
  float acc[ARCB_VOCAB];
#pragma unroll
  for (int v = 0; v < ARCB_VOCAB; ++v) acc[v] = 0.f;
  for (int c = lane * 4; c < a.d; c += 128) {
    const float4 xv = *reinterpret_cast<const float4*>(x + c);
    const float4 g = __ldg(reinterpret_cast<const float4*>(a.lnf_w + c));
    const float n0 = (xv.x * inv) * g.x, n1 = (xv.y * inv) * g.y, n2 = (xv.z * inv) * g.z,
                n3 = (xv.w * inv) * g.w;
#pragma unroll
    for (int v = 0; v < ARCB_VOCAB; ++v) {
      const float4 w = __ldg(reinterpret_cast<const float4*>(a.lm_head + (size_t)v * a.d + c));
      acc[v] += n0 * w.x + n1 * w.y + n2 * w.z + n3 * w.w;
    }
  }
#pragma unroll
  for (int v = 0; v < ARCB_VOCAB; ++v) acc[v] = warp_sum(acc[v]);
  if (lane != 0) return;

  int best = 0;
  float bv = acc[0];
#pragma unroll
  for (int v = 1; v < ARCB_VOCAB; ++v)
    if (acc[v] > bv) { bv = acc[v]; best = v; }  // strict '>' keeps the first maximum (argmax semantics)
  if (a.logits) {
#pragma unroll
    for (int v = 0; v < ARCB_VOCAB; ++v) a.logits[(size_t)i * ARCB_VOCAB + v] = acc[v];
  }
  if (a.argmax) a.argmax[i] = best;
  if (a.mode == HEAD_PLAIN) return;

  // ---- greedy-loop bookkeeping (src/inference.py:573-590, 609-626) ----
  const int b = (a.mode == HEAD_FIRST) ? a.first_seq[i] : i;
  if (b < 0 || b >= st.n_seqs) { arcb_set_error(st.err, ARCB_DEV_BAD_INDEX); return; }
  int out_idx;
  if (a.mode == HEAD_FIRST) {
    const int plen = a.prompt_len[i];
    st.len0[b] = plen;
    st.cur_len[b] = plen;
    st.gx[b] = a.grid_x[i];
    st.gy[b] = a.grid_y[i];
    st.gin[b] = a.grid_in_output[i];
    if (st.finished[b]) { st.finished[b] = 0; atomicSub(st.n_finished, 1); }
    out_idx = 0;
  } else {
    out_idx = st.cur_len[b] - st.len0[b] + 1;
    st.cur_len[b] = min(st.cur_len[b] + 1, st.t_max);
  }
  // Soft constraints (src/inference.py:285-364) act on a copy of the logits, using the grid state
  // after the last fed token (st.gx / st.gy were advanced by decode_begin, or armed just above).
  if (st.disallow_mask || st.palette_mask || st.target_shape || st.temperature > 0.f) {
    float adj[ARCB_VOCAB];
#pragma unroll
    for (int v = 0; v < ARCB_VOCAB; ++v) adj[v] = ((st.disallow_mask >> v) & 1u) ? -INFINITY : acc[v];
    if (st.palette_mask) {
#pragma unroll
      for (int c = 0; c < 10; ++c)
        if (!st.palette_mask[(size_t)b * 10 + c]) adj[c] -= st.palette_penalty;
    }
    if (st.target_shape) {
      const int th = st.target_shape[2 * b], tw = st.target_shape[2 * b + 1];
      if (th >= 0 && tw >= 0) {
        const int gx = st.gx[b], gy = st.gy[b];
        const bool row_full = gx >= tw, past_end = gy >= th;
        if (row_full) {
#pragma unroll
          for (int c = 0; c < 10; ++c) adj[c] -= st.shape_penalty;
        } else {
          adj[TOK_NEWLINE] -= st.shape_penalty;
        }
        if (past_end) {
#pragma unroll
          for (int c = 0; c < 10; ++c) adj[c] -= st.shape_penalty;
          adj[TOK_NEWLINE] -= st.shape_penalty;
        }
      }
    }
    best = 0;
    float bv2 = adj[0];
#pragma unroll
    for (int v = 1; v < ARCB_VOCAB; ++v)
      if (adj[v] > bv2) { bv2 = adj[v]; best = v; }
    if (st.temperature > 0.f) {
      // temperature / top-k sampling (src/inference.py:575-583): softmax of the kept logits, inverse CDF
      const float inv_t = 1.f / fmaxf(st.temperature, 1e-6f);
      const int kk = (st.top_k > 0 && st.top_k < ARCB_VOCAB) ? st.top_k : ARCB_VOCAB;
      float p[ARCB_VOCAB];
      float total = 0.f;
#pragma unroll
      for (int v = 0; v < ARCB_VOCAB; ++v) {
        int rank = 0;  // logits ahead of v: larger, or equal with a smaller index
#pragma unroll
        for (int w = 0; w < ARCB_VOCAB; ++w) rank += (adj[w] > adj[v] || (adj[w] == adj[v] && w < v)) ? 1 : 0;
        p[v] = (rank < kk) ? __expf((adj[v] - bv2) * inv_t) : 0.f;
        total += p[v];
      }
      // counter-based uniform number: splitmix64 of (seed, stream id, generated index)
      const unsigned long long sid = st.sample_stream ? (unsigned long long)(unsigned int)st.sample_stream[b]
                                                      : (unsigned long long)b;
      unsigned long long z = st.sample_seed + 0x9E3779B97F4A7C15ull * (sid + 1) +
                             0xD1B54A32D192ED03ull * (unsigned long long)(out_idx + 1);
      z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
      z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
      z ^= z >> 31;
      const float u = (float)(z >> 40) * (1.f / 16777216.f) * total;
      float run = 0.f;
      int pick = best;
      bool found = false;
#pragma unroll
      for (int v = 0; v < ARCB_VOCAB; ++v) {
        run += p[v];
        if (!found && p[v] > 0.f && u < run) { pick = v; found = true; }
      }
      best = pick;
    }
  }
  int tok = best;
  const bool in_range = out_idx >= 0 && out_idx < st.max_new;
  if (st.forced && in_range) tok = st.forced[(size_t)b * st.max_new + out_idx];
  else if (st.stop_on_end == 1 && st.finished[b]) tok = TOK_END;  // frozen row keeps emitting END (mode 2: keeps decoding)
  if (in_range) {
    st.out_tokens[(size_t)b * st.max_new + out_idx] = tok;
    if (st.step_logits) {
#pragma unroll
      for (int v = 0; v < ARCB_VOCAB; ++v)
        st.step_logits[((size_t)b * st.max_new + out_idx) * ARCB_VOCAB + v] = acc[v];
    }
  }
  if (st.stop_on_end && tok == TOK_END && !st.finished[b]) {
    st.finished[b] = 1;
    atomicAdd(st.n_finished, 1);
  }
  st.cur_tok[b] = tok;
}

// dst row = (r / blk) * blk_stride + blk_off + r % blk.  Every value is first rounded to bf16 (the
// model's precision); container: 0 = fp32, 1 = bf16, 2 = IEEE half holding the bf16-rounded value
// (exact for |w| >= 2^-14, within 2^-25 absolute below; saturates at +-65504).
__global__ void pack_rows_kernel(const float* __restrict__ src, void* __restrict__ dst, long long rows,
                                 long long cols, int blk, int blk_stride, int blk_off, int to_bf16) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    const long long dr = (r / blk) * blk_stride + blk_off + (r % blk);
    const __nv_bfloat16 h = __float2bfloat16_rn(src[i]);
    if (to_bf16 == 1) {
      reinterpret_cast<__nv_bfloat16*>(dst)[dr * cols + c] = h;
    } else if (to_bf16 == 2) {
      const float f = fminf(fmaxf(__bfloat162float(h), -65504.f), 65504.f);
      reinterpret_cast<__half*>(dst)[dr * cols + c] = __float2half_rn(f);
    } else {
      reinterpret_cast<float*>(dst)[dr * cols + c] = __bfloat162float(h);
    }
  }
}

}  // namespace

int arcb_launch_rmsnorm(const float* x, const float* w, void* out16, int rows, int d, float eps,
                        int act_f16, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 4) return -1;
  const cudaError_t e = arcb_launch(rmsnorm_kernel, dim3((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA), dim3(ROWS_PER_CTA * 32), 0,
                                    stream, x, w, reinterpret_cast<uint16_t*>(out16), rows, d, eps, act_f16);
  arcb_count_launch(1);
  return (int)e;
}

int arcb_launch_embed_norm(const EmbedArgs& a, cudaStream_t stream) {
  if (a.rows <= 0) return 0;
  const cudaError_t e = arcb_launch(embed_norm_kernel, dim3((a.rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA),
                                    dim3(ROWS_PER_CTA * 32), 0, stream, a);
  arcb_count_launch(1);
  return (int)e;
}

int arcb_launch_decode_begin(const DecodeState& st, const EmbedArgs& a, cudaStream_t stream) {
  const cudaError_t e = arcb_launch(decode_begin_kernel, dim3((st.n_seqs + ROWS_PER_CTA - 1) / ROWS_PER_CTA),
                                    dim3(ROWS_PER_CTA * 32), 0, stream, st, a);
  arcb_count_launch(1);
  return (int)e;
}

int arcb_launch_head(const HeadArgs& a, const DecodeState& st, cudaStream_t stream) {
  if (a.rows <= 0) return 0;
  const cudaError_t e = arcb_launch(head_kernel, dim3((a.rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA), dim3(ROWS_PER_CTA * 32),
                                    0, stream, a, st);
  arcb_count_launch(1);
  return (int)e;
}

int arcb_launch_pack_rows(const float* src, void* dst, long long rows, long long cols, int blk,
                          int blk_stride, int blk_off, int to_bf16, cudaStream_t stream) {
  const long long n = rows * cols;
  if (n <= 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  pack_rows_kernel<<<(unsigned)blocks, threads, 0, stream>>>(src, dst, rows, cols, blk, blk_stride, blk_off,
                                                            to_bf16);
  arcb_count_launch(1);
  return (int)cudaGetLastError();
}
