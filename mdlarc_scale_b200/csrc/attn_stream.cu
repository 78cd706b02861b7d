// Streaming attention of one query vector over a cached K/V prefix (split-K).
//
// One warp owns one (item, head, split).  A K (or V) row is 64 bf16 = 128 bytes = 8 x 16 B,
// so a warp-wide 16-byte load covers 4 rows: lane = 8 * row_in_group + segment.  Four such
// loads of K and four of V are in flight per warp iteration (4 KB), every byte of the prefix
// is read exactly once, and the softmax is kept online per 8-lane group (warp shuffles for the
// dot product, one rescale per 16 rows), merged across the 4 groups at the end.
//
// With n_splits > 1 every split writes (m, l, acc[64]) to scratch and a second kernel merges
// the splits; with n_splits == 1 the normalised output is written directly.
#include <cstdlib>

#include "attn_stream.cuh"
#include "launch.cuh"

namespace {

constexpr int WARPS_PER_CTA = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float dot8(const float (&q)[8], const uint4& k) {
  const float2 a = unpack2_bf16(k.x), b = unpack2_bf16(k.y), c = unpack2_bf16(k.z), d = unpack2_bf16(k.w);
  float s = q[0] * a.x;
  s = fmaf(q[1], a.y, s);
  s = fmaf(q[2], b.x, s);
  s = fmaf(q[3], b.y, s);
  s = fmaf(q[4], c.x, s);
  s = fmaf(q[5], c.y, s);
  s = fmaf(q[6], d.x, s);
  s = fmaf(q[7], d.y, s);
  return s;
}

__device__ __forceinline__ void axpy8(float (&acc)[8], float p, const uint4& v) {
  const float2 a = unpack2_bf16(v.x), b = unpack2_bf16(v.y), c = unpack2_bf16(v.z), d = unpack2_bf16(v.w);
  acc[0] = fmaf(p, a.x, acc[0]);
  acc[1] = fmaf(p, a.y, acc[1]);
  acc[2] = fmaf(p, b.x, acc[2]);
  acc[3] = fmaf(p, b.y, acc[3]);
  acc[4] = fmaf(p, c.x, acc[4]);
  acc[5] = fmaf(p, c.y, acc[5]);
  acc[6] = fmaf(p, d.x, acc[6]);
  acc[7] = fmaf(p, d.y, acc[7]);
}

__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
attn_stream_kernel(AttnStreamArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
  const long long n_work = (long long)a.n_items * a.n_heads * a.n_splits;
  if (w >= n_work) return;
  const int split = (int)(w % a.n_splits);
  const long long ih = w / a.n_splits;
  const int h = (int)(ih % a.n_heads);
  const int item = (int)(ih / a.n_heads);

  const int seq = a.item_seq ? a.item_seq[item] : item;
  int len = a.item_len[item];
  const bool skip = a.item_skip && a.item_skip[item];
  if (len > a.t_max || seq < 0 || seq >= a.n_seqs) {
    if (lane == 0) arcb_set_error(a.err, ARCB_DEV_BAD_INDEX);
    len = 0;
  }
  if (skip || len < 0) len = 0;

  // key range of this split: equal chunks rounded up to 16 rows
  int begin = 0, end = len;
  if (a.n_splits > 1) {
    int chunk = (len + a.n_splits - 1) / a.n_splits;
    chunk = (chunk + 15) & ~15;
    begin = min(split * chunk, len);
    end = min(begin + chunk, len);
  }

  const int sub = lane >> 3, seg = lane & 7;
  // q segment, pre-scaled by 1/sqrt(64) * log2(e) so that exp2 can be used
  float q[8];
  {
    const uint16_t* qp = reinterpret_cast<const uint16_t*>(a.q16) +
                         ((size_t)item * a.n_heads + h) * ARCB_HEAD_DIM + seg * 8;
    const uint4 raw = *reinterpret_cast<const uint4*>(qp);
    const float2 f0 = unpack2_act(raw.x, a.act_f16), f1 = unpack2_act(raw.y, a.act_f16),
                 f2 = unpack2_act(raw.z, a.act_f16), f3 = unpack2_act(raw.w, a.act_f16);
    const float sc = 0.125f * LOG2E;
    q[0] = f0.x * sc; q[1] = f0.y * sc; q[2] = f1.x * sc; q[3] = f1.y * sc;
    q[4] = f2.x * sc; q[5] = f2.y * sc; q[6] = f3.x * sc; q[7] = f3.y * sc;
  }

  const size_t head_row0 = ((size_t)seq * a.n_heads + h) * (size_t)a.t_max;
  const uint4* Kp = reinterpret_cast<const uint4*>(a.k + head_row0 * ARCB_HEAD_DIM) + seg;
  const uint4* Vp = reinterpret_cast<const uint4*>(a.v + head_row0 * ARCB_HEAD_DIM) + seg;

  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;

  for (int r0 = begin; r0 < end; r0 += 16) {
    uint4 kk[4], vv[4];
    bool valid[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int row = r0 + u * 4 + sub;
      valid[u] = row < end;
      kk[u] = make_uint4(0u, 0u, 0u, 0u);
      if (valid[u]) kk[u] = ldg_stream16(Kp + (size_t)row * 8);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int row = r0 + u * 4 + sub;
      vv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (valid[u]) vv[u] = ldg_stream16(Vp + (size_t)row * 8);
    }
    float s[4];
    float mx = m;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float d = dot8(q, kk[u]);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      s[u] = valid[u] ? d : -INFINITY;
      mx = fmaxf(mx, s[u]);
    }
    const float m_safe = (mx == -INFINITY) ? 0.f : mx;
    const float alpha = exp2f(m - m_safe);
    l *= alpha;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float p = exp2f(s[u] - m_safe);
      l += p;
      axpy8(acc, p, vv[u]);
    }
    m = mx;
  }

  // merge the 4 row groups (lanes differing in bits 3 and 4 hold the same dims)
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
    const float mx = fmaxf(m, m_o);
    const float m_safe = (mx == -INFINITY) ? 0.f : mx;
    const float sa = exp2f(m - m_safe), sb = exp2f(m_o - m_safe);
    l = l * sa + l_o * sb;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a_o = __shfl_xor_sync(0xffffffffu, acc[j], o);
      acc[j] = acc[j] * sa + a_o * sb;
    }
    m = mx;
  }

  if (sub == 0) {
    if (a.n_splits == 1) {
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      uint4 o;
      o.x = pack2_act(acc[0] * inv, acc[1] * inv, a.act_f16);
      o.y = pack2_act(acc[2] * inv, acc[3] * inv, a.act_f16);
      o.z = pack2_act(acc[4] * inv, acc[5] * inv, a.act_f16);
      o.w = pack2_act(acc[6] * inv, acc[7] * inv, a.act_f16);
      uint16_t* op = reinterpret_cast<uint16_t*>(a.out16) +
                     ((size_t)item * a.n_heads + h) * ARCB_HEAD_DIM + seg * 8;
      *reinterpret_cast<uint4*>(op) = o;
    } else {
      // scratch record per (item, head, split): 64 acc + m + l, padded to 68 floats
      float* rec = a.scratch + ((size_t)ih * a.n_splits + split) * ATTN_SCRATCH_STRIDE;
      *reinterpret_cast<float4*>(rec + seg * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(rec + seg * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (seg == 0) {
        rec[64] = m;
        rec[65] = l;
      }
    }
  }
}

// Cooperative form for launches with enough work items to fill the machine: a CTA of COOP_WARPS warps
// owns one (item, head, split) and its warps take alternate 32-row slices of the prefix: every warp has
// 4 KB of K and 4 KB of V in flight (8 + 8 sixteen-byte loads per lane) and the CTA's loads cover one
// contiguous 16 KB stretch of each.  DRAM serves such stretches measurably faster than the same bytes
// requested as independent 2 KB pieces by unrelated warps (6.85-7.1 TB/s against 6.2-6.7 TB/s at 1024
// sequences x 20 heads, 300-1200 cached positions).  Every warp keeps its own online softmax; the
// partial (m, l, acc) of the warps are merged in a fixed order through shared memory by warp 0, which
// writes the output (or the split record).  Measured alternatives: 8 warps per item lose 18 % at 300
// cached positions (too few CTAs in flight), 16-row slices lose 3 %.
constexpr int COOP_WARPS = 4;
constexpr int COOP_ROWS = 32;

template <int WARPS, int ROWS, int MIN_CTAS>
__global__ void __launch_bounds__(WARPS * 32, MIN_CTAS)
attn_stream_coop_kernel(AttnStreamArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_part[WARPS][ATTN_SCRATCH_STRIDE];
  const int lane = threadIdx.x & 31, wj = threadIdx.x >> 5;
  const long long w = blockIdx.x;                       // grid = n_items * n_heads * n_splits exactly
  const int split = (int)(w % a.n_splits);
  const long long ih = w / a.n_splits;
  const int h = (int)(ih % a.n_heads);
  const int item = (int)(ih / a.n_heads);

  const int seq = a.item_seq ? a.item_seq[item] : item;
  int len = a.item_len[item];
  const bool skip = a.item_skip && a.item_skip[item];
  if (len > a.t_max || seq < 0 || seq >= a.n_seqs) {
    if (threadIdx.x == 0) arcb_set_error(a.err, ARCB_DEV_BAD_INDEX);
    len = 0;
  }
  if (skip || len < 0) len = 0;

  int begin = 0, end = len;
  if (a.n_splits > 1) {
    int chunk = (len + a.n_splits - 1) / a.n_splits;
    chunk = (chunk + 15) & ~15;
    begin = min(split * chunk, len);
    end = min(begin + chunk, len);
  }

  const int sub = lane >> 3, seg = lane & 7;
  float q[8];
  {
    const uint16_t* qp = reinterpret_cast<const uint16_t*>(a.q16) +
                         ((size_t)item * a.n_heads + h) * ARCB_HEAD_DIM + seg * 8;
    const uint4 raw = *reinterpret_cast<const uint4*>(qp);
    const float2 f0 = unpack2_act(raw.x, a.act_f16), f1 = unpack2_act(raw.y, a.act_f16),
                 f2 = unpack2_act(raw.z, a.act_f16), f3 = unpack2_act(raw.w, a.act_f16);
    const float sc = 0.125f * LOG2E;
    q[0] = f0.x * sc; q[1] = f0.y * sc; q[2] = f1.x * sc; q[3] = f1.y * sc;
    q[4] = f2.x * sc; q[5] = f2.y * sc; q[6] = f3.x * sc; q[7] = f3.y * sc;
  }

  const size_t head_row0 = ((size_t)seq * a.n_heads + h) * (size_t)a.t_max;
  const uint4* Kp = reinterpret_cast<const uint4*>(a.k + head_row0 * ARCB_HEAD_DIM) + seg;
  const uint4* Vp = reinterpret_cast<const uint4*>(a.v + head_row0 * ARCB_HEAD_DIM) + seg;

  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;

  constexpr int U = ROWS / 4;
  for (int r0 = begin + wj * ROWS; r0 < end; r0 += ROWS * WARPS) {
    uint4 kk[U], vv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = r0 + u * 4 + sub;
      kk[u] = make_uint4(0u, 0u, 0u, 0u);
      if (row < end) kk[u] = ldg_stream16(Kp + (size_t)row * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = r0 + u * 4 + sub;
      vv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (row < end) vv[u] = ldg_stream16(Vp + (size_t)row * 8);
    }
    float s[U];
    float mx = m;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float d = dot8(q, kk[u]);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      s[u] = (r0 + u * 4 + sub < end) ? d : -INFINITY;
      mx = fmaxf(mx, s[u]);
    }
    const float m_safe = (mx == -INFINITY) ? 0.f : mx;
    const float alpha = exp2f(m - m_safe);
    l *= alpha;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= alpha;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float p = exp2f(s[u] - m_safe);
      l += p;
      axpy8(acc, p, vv[u]);
    }
    m = mx;
  }

  // merge the 4 row groups of the warp (lanes differing in bits 3 and 4 hold the same dims)
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
    const float mx = fmaxf(m, m_o);
    const float m_safe = (mx == -INFINITY) ? 0.f : mx;
    const float sa = exp2f(m - m_safe), sb = exp2f(m_o - m_safe);
    l = l * sa + l_o * sb;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a_o = __shfl_xor_sync(0xffffffffu, acc[j], o);
      acc[j] = acc[j] * sa + a_o * sb;
    }
    m = mx;
  }
  if (sub == 0) {
    float* rec = s_part[wj];
    *reinterpret_cast<float4*>(rec + seg * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(rec + seg * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (seg == 0) {
      rec[64] = m;
      rec[65] = l;
    }
  }
  __syncthreads();
  if (wj != 0) return;
  // warp 0: merge the warps' partials in a fixed order; lane d holds dims 2d, 2d + 1
  float mt = -INFINITY;
#pragma unroll
  for (int j = 0; j < WARPS; ++j) mt = fmaxf(mt, s_part[j][64]);
  const float mt_safe = (mt == -INFINITY) ? 0.f : mt;
  float lt = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
  for (int j = 0; j < WARPS; ++j) {
    const float sc = exp2f(s_part[j][64] - mt_safe);
    lt += s_part[j][65] * sc;
    const float2 v = *reinterpret_cast<const float2*>(&s_part[j][2 * lane]);
    o0 += v.x * sc;
    o1 += v.y * sc;
  }
  if (a.n_splits == 1) {
    const float inv = (lt > 0.f) ? 1.f / lt : 0.f;
    uint32_t* op = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(a.out16) + (size_t)ih * ARCB_HEAD_DIM) + lane;
    *op = pack2_act(o0 * inv, o1 * inv, a.act_f16);
  } else {
    float* rec = a.scratch + ((size_t)ih * a.n_splits + split) * ATTN_SCRATCH_STRIDE;
    *reinterpret_cast<float2*>(rec + 2 * lane) = make_float2(o0, o1);
    if (lane == 0) {
      rec[64] = mt;
      rec[65] = lt;
    }
  }
}

// One warp per (item, head): lane d handles dims 2d, 2d+1.
__global__ void __launch_bounds__(128)
attn_combine_kernel(AttnStreamArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long ih = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (ih >= (long long)a.n_items * a.n_heads) return;
  const float* rec0 = a.scratch + (size_t)ih * a.n_splits * ATTN_SCRATCH_STRIDE;
  float m = -INFINITY;
  for (int s = 0; s < a.n_splits; ++s) m = fmaxf(m, rec0[s * ATTN_SCRATCH_STRIDE + 64]);
  const float m_safe = (m == -INFINITY) ? 0.f : m;
  float l = 0.f, o0 = 0.f, o1 = 0.f;
  for (int s = 0; s < a.n_splits; ++s) {
    const float* rec = rec0 + s * ATTN_SCRATCH_STRIDE;
    const float sc = exp2f(rec[64] - m_safe);
    l += rec[65] * sc;
    const float2 v = *reinterpret_cast<const float2*>(rec + 2 * lane);
    o0 += v.x * sc;
    o1 += v.y * sc;
  }
  const float inv = (l > 0.f) ? 1.f / l : 0.f;
  uint32_t* op = reinterpret_cast<uint32_t*>(reinterpret_cast<uint16_t*>(a.out16) + (size_t)ih * ARCB_HEAD_DIM) + lane;
  *op = pack2_act(o0 * inv, o1 * inv, a.act_f16);
}

}  // namespace

int arcb_launch_attn_stream(const AttnStreamArgs& a, cudaStream_t stream) {
  if (a.n_items <= 0) return 0;
  if (a.n_splits < 1 || (a.n_splits > 1 && !a.scratch)) return -1;
  const long long n_work = (long long)a.n_items * a.n_heads * a.n_splits;
  const long long blocks = (n_work + WARPS_PER_CTA - 1) / WARPS_PER_CTA;
  if (blocks > 0x7fffffffLL) return -1;
  // enough (item, head, split) work items for two CTAs per SM, and a cache whose per-split share can fill
  // one CTA iteration (4 x 32 rows): one CTA per item (see the kernel's comment); launches over a few
  // dozen rows per split keep one warp per item (13.4 against 14.9 ms for 15 decode steps of 16 sequences)
  static const int coop_min = [] { const char* e = getenv("ARCB_ATTN_COOP_MIN"); return e ? atoi(e) : 296; }();  // A/B switch; < 0 disables
  cudaError_t e;
  if (coop_min >= 0 && n_work >= coop_min && n_work <= 0x7fffffffLL &&
      (long long)a.t_max >= (long long)COOP_WARPS * COOP_ROWS * a.n_splits) {
    e = arcb_launch(attn_stream_coop_kernel<COOP_WARPS, COOP_ROWS, 4>, dim3((unsigned)n_work), dim3(COOP_WARPS * 32), 0, stream, a);
  } else
    e = arcb_launch(attn_stream_kernel, dim3((unsigned)blocks), dim3(WARPS_PER_CTA * 32), 0, stream, a);
  arcb_count_launch(1);
  if (e == cudaSuccess && a.n_splits > 1) {
    const long long nb = ((long long)a.n_items * a.n_heads + 3) / 4;
    e = arcb_launch(attn_combine_kernel, dim3((unsigned)nb), dim3(128), 0, stream, a);
    arcb_count_launch(1);
  }
  return (int)e;
}
