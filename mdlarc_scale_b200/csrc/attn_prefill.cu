// Flash-style causal prefill attention on tcgen05 tensor cores with TMEM accumulators.
//
// One CTA = one block of up to 128 consecutive query rows of one sequence x one head.
// Per 128-key tile:
//   TMA (warp 0)      K tile and V tile [128 keys][64 dims], 128-byte swizzle, 2-stage ring
//   MMA (warp 1)      S = Q K^T  (UMMA 128x128x16 x4, fp32 in TMEM columns [0,128))
//   softmax (w. 2-5)  one thread per query row: tcgen05.ld S, mask by the row's visible-key
//                     count, online softmax (exp2), P written 16-bit into shared memory in the
//                     swizzled K-major layout the MMA reads
//   MMA (warp 1)      O_tile = P V  (UMMA 128x64x16 x8, V is the MN-major B operand,
//                     fp32 in TMEM columns [128,192))
//   softmax threads   o = o * alpha + O_tile   (running output row kept in registers)
// Q, K, V and P share one 16-bit format (half or bfloat16): kind::f16 needs equal A/B formats.
// K/V come from a per-call scratch in that format (the bf16 KV cache is written separately by
// the QKV epilogue), rows [kv0, kv0 + count) of the sequence.  Every mbarrier wait is bounded.
#include "attn_prefill.cuh"
#include "gemm.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 64;
constexpr int Q_BYTES = BQ * HD * 2;          // 16 KB
constexpr int KV_TILE_BYTES = BKV * HD * 2;   // 16 KB each for K and V
constexpr int P_BYTES = BQ * BKV * 2;         // 32 KB: two [128][64] swizzled K-major tiles
constexpr int KV_STAGES = 2;
constexpr int SMEM_BYTES = Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES + P_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 256;                // S: [0,128), O_tile: [128,192)
constexpr float LOG2E = 1.4426950408889634f;

// MN-major operand tile [K rows of 128 bytes][64 elements], 128-byte swizzle: 8-row groups are
// 1024 bytes apart along K (stride byte offset); a single 64-element group along MN.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(1024 >> 4) << 16;  // leading byte offset (next 64-element MN group; unused for N = 64)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset (next group of 8 K rows)
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(192, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, AttnPrefillArgs a, uint32_t idesc_qk,
                    uint32_t idesc_pv) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_max_cnt[4];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t kv_smem = base + Q_BYTES;                      // stage s: K at +s*32K, V at +16K
  const uint32_t p_smem = kv_smem + KV_STAGES * 2 * KV_TILE_BYTES;
  uint8_t* p_ptr = base_ptr + Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES;
  const uint32_t bar0 = p_smem + P_BYTES;
  const uint32_t bar_q = bar0, bar_kv_full = bar0 + 8, bar_kv_empty = bar0 + 24, bar_s = bar0 + 40,
                 bar_p = bar0 + 48, bar_o = bar0 + 56;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(p_ptr + P_BYTES + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, h = blockIdx.y;
  const int row0 = a.qblock_row0[blk];
  const int rows = a.qblock_rows[blk];
  const int kv0 = a.qblock_kv0[blk];

  // visible-key count of this thread's query row (softmax warps) and the block maximum
  int my_cnt = 0;
  const int r = (warp >= 2) ? ((warp & 3) * 32 + lane) : 0;
  if (warp >= 2) {
    if (r < rows) my_cnt = a.kv_count[row0 + r];
    int mx = my_cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_max_cnt[warp & 3] = mx;
  }
  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar_kv_full + 8 * s, 1);
      mbar_init(bar_kv_empty + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_o, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int max_cnt = max(max(s_max_cnt[0], s_max_cnt[1]), max(s_max_cnt[2], s_max_cnt[3]));
  const int n_tiles = (max_cnt + BKV - 1) / BKV;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(bar_q, Q_BYTES);
      tma_load_2d(q_smem, &tmap_q, h * HD, row0, bar_q);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait_bounded(bar_kv_empty + 8 * s, ph ^ 1)) {
          arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_MMA);
          break;
        }
        const uint32_t dst = kv_smem + s * 2 * KV_TILE_BYTES;
        mbar_expect_tx(bar_kv_full + 8 * s, 2 * KV_TILE_BYTES);
        tma_load_2d(dst, &tmap_k, h * HD, kv0 + j * BKV, bar_kv_full + 8 * s);
        tma_load_2d(dst + KV_TILE_BYTES, &tmap_v, h * HD, kv0 + j * BKV, bar_kv_full + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      bool ok = mbar_wait_bounded(bar_q, 0);
      if (!ok) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
      const uint64_t dq = umma_desc_k_sw128(q_smem);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait_bounded(bar_kv_full + 8 * s, ph)) {
          arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
          break;
        }
        tc_fence_after();
        const uint32_t k_addr = kv_smem + s * 2 * KV_TILE_BYTES;
        const uint64_t dk = umma_desc_k_sw128(k_addr);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) umma_f16(tmem_base, dq + 2 * ks, dk + 2 * ks, idesc_qk, ks ? 1u : 0u);
        umma_commit(bar_s);
        // P of this tile (written by the softmax threads, which have also consumed O of the previous tile)
        if (!mbar_wait_bounded(bar_p, j & 1)) {
          arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
          break;
        }
        tc_fence_after();
        const uint64_t dv = umma_desc_mn_sw128(k_addr + KV_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          const uint64_t dp = umma_desc_k_sw128(p_smem + (ks >> 2) * (BQ * 128)) + 2 * (ks & 3);
          // 16 keys = 16 rows of 128 bytes = 2048 bytes further into the V tile
          umma_f16(tmem_base + 128, dp, dv + (uint64_t)(ks * (2048 >> 4)), idesc_pv, ks ? 1u : 0u);
        }
        umma_commit(bar_o);
        umma_commit(bar_kv_empty + 8 * s);
      }
    }
  } else {
    // ---- softmax / output threads: one query row each ----
    const int quarter = warp & 3;
    const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float sc = 0.125f * LOG2E;
    float m = -INFINITY, l = 0.f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (ok && !mbar_wait_bounded(bar_s, j & 1)) {
        arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * BKV;
      // pass 1: row maximum of the visible scores
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t sreg[32];
        tmem_ld_32x32(t_row + c * 32, sreg);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float t = __uint_as_float(sreg[i]) * sc;
          if (key0 + c * 32 + i < my_cnt) mx = fmaxf(mx, t);
        }
      }
      const float m_safe = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f(m - m_safe);
      float lsum = 0.f;
      // pass 2: probabilities -> shared memory (swizzled K-major, 16-bit)
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t sreg[32];
        tmem_ld_32x32(t_row + c * 32, sreg);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int kidx = key0 + c * 32 + i;
          float p0 = exp2f(__uint_as_float(sreg[i]) * sc - m_safe);
          float p1 = exp2f(__uint_as_float(sreg[i + 1]) * sc - m_safe);
          if (kidx >= my_cnt) p0 = 0.f;
          if (kidx + 1 >= my_cnt) p1 = 0.f;
          pk[i >> 1] = pack2_act(p0, p1, a.act_f16);
          // the sum uses the rounded probabilities the MMA will see
          const float2 pr = unpack2_act(pk[i >> 1], a.act_f16);
          lsum += pr.x + pr.y;
        }
        // columns [c*32, c*32+32) of row r: tile = c / 2, 16-byte chunks ch0 .. ch0+3
        uint8_t* tile = p_ptr + (c >> 1) * (BQ * 128) + r * 128;
        const int ch0 = (c & 1) * 4;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int ch = (ch0 + q4) ^ (r & 7);
          *reinterpret_cast<uint4*>(tile + ch * 16) =
              make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
      }
      l = l * alpha + lsum;
      m = mx;
      // make the generic-proxy writes of P visible to the tensor-core (async) proxy
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(bar_p);
      if (!mbar_wait_bounded(bar_o, j & 1)) {
        arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t oreg[32];
        tmem_ld_32x32(t_row + 128 + c * 32, oreg);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(oreg[i]);
      }
      tc_fence_before();
    }
    if (r < rows) {
      const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
      uint16_t* dst = reinterpret_cast<uint16_t*>(a.out16) + ((size_t)(row0 + r) * a.n_heads + h) * HD;
#pragma unroll
      for (int i = 0; i < HD; i += 8) {
        uint4 v;
        v.x = pack2_act(o[i] * inv, o[i + 1] * inv, a.act_f16);
        v.y = pack2_act(o[i + 2] * inv, o[i + 3] * inv, a.act_f16);
        v.z = pack2_act(o[i + 4] * inv, o[i + 5] * inv, a.act_f16);
        v.w = pack2_act(o[i + 6] * inv, o[i + 7] * inv, a.act_f16);
        *reinterpret_cast<uint4*>(dst + i) = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

bool arcb_attn_prefill_available() { return true; }

int arcb_attn_prefill_init() {
  return (int)cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
}

int arcb_launch_attn_prefill(const AttnPrefillArgs& a, cudaStream_t stream) {
  if (a.n_qblocks <= 0) return 0;
  if (a.n_kv_rows <= 0 || a.n_rows <= 0) return -1;
  const uint64_t d = (uint64_t)a.n_heads * HD;
  CUtensorMap tq, tk, tv;
  int r = arcb_make_tmap_2d_16b(&tq, a.q16, (uint64_t)a.n_rows, d, BQ, HD, a.act_f16);
  if (r) return 1000 + r;
  r = arcb_make_tmap_2d_16b(&tk, a.k16, (uint64_t)a.n_kv_rows, d, BKV, HD, a.act_f16);
  if (r) return 1000 + r;
  r = arcb_make_tmap_2d_16b(&tv, a.v16, (uint64_t)a.n_kv_rows, d, BKV, HD, a.act_f16);
  if (r) return 1000 + r;
  const int fmt = a.act_f16 ? 0 : 1;
  const uint32_t idesc_qk = umma_idesc_f16(BQ, BKV, fmt, fmt, 0, 0);
  const uint32_t idesc_pv = umma_idesc_f16(BQ, HD, fmt, fmt, 0, 1);  // B = V is MN-major
  dim3 grid(a.n_qblocks, a.n_heads);
  attn_prefill_kernel<<<grid, 192, SMEM_BYTES, stream>>>(tq, tk, tv, a, idesc_qk, idesc_pv);
  arcb_count_launch(1);
  return (int)cudaGetLastError();
}
