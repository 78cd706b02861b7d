// Flash-style causal prefill attention on tcgen05 tensor cores with TMEM accumulators.
//
// One CTA = up to 256 consecutive query rows of one sequence (two 128-row Q tiles, A and B) x one
// head.  Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 softmax
// group of tile A, warps 6-9 softmax group of tile B.  Per 128-key tile j:
//   TMA        K and V tiles [128 keys][64 dims], 128-byte swizzle, 3-stage ring shared by A and B
//   MMA        S_x = Q_x K^T   (UMMA 128x128x16 x4, fp32 in TMEM)            x in {A, B}
//   softmax_x  one thread per query row: row max (tcgen05.ld), then p = exp2(s*c - m) written
//              16-bit into shared memory in the swizzled K-major layout the MMA reads
//   MMA        Otile_x = P_x V (UMMA 128x64x16 x8, V is the MN-major B operand), into one of two
//              TMEM buffers, so the softmax thread folds Otile(j-1) into its register-resident
//              output row while the tensor core is already busy with tile j
// The two groups run out of phase: the tensor core works on one Q tile while the other group's
// threads do exponentials.  Rows carry their own visible-key count (causal AND key padding as a
// prefix length), so no mask tensor exists.  Q, K, V and P share one 16-bit format (kind::f16
// needs equal A/B formats).  Every mbarrier wait is bounded.
#include "attn_prefill.cuh"
#include "gemm.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 64;
constexpr int Q_BYTES = BQ * HD * 2;          // 16 KB per Q tile
constexpr int KV_TILE_BYTES = BKV * HD * 2;   // 16 KB each for K and V
constexpr int P_BYTES = BQ * BKV * 2;         // 32 KB per Q tile: two [128][64] swizzled K-major tiles
constexpr int KV_STAGES = 3;
constexpr int SMEM_BYTES = 2 * Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES + 2 * P_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;  // S_A [0,128) S_B [128,256) O_A0 [256,320) O_A1 [320,384) O_B0 [384,448) O_B1 [448,512)
constexpr float LOG2E = 1.4426950408889634f;
constexpr int N_THREADS = 320;

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

__device__ __forceinline__ uint32_t pack2_prob(float a, float b, int f16) {
  if (f16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// 2^x on the special-function unit, one instruction (flushes denormals; inputs here are <= 0 or
// masked afterwards)
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Bars {
  uint32_t q, kv_full, kv_empty, s[2], p[2], o[2];
};

__global__ void __launch_bounds__(N_THREADS, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, AttnPrefillArgs a, uint32_t idesc_qk,
                    uint32_t idesc_pv) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_max_cnt[8];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t q_smem = base;                                   // tile x at + x * Q_BYTES
  const uint32_t kv_smem = base + 2 * Q_BYTES;                    // stage s: K at + s*32K, V at +16K
  const uint32_t p_smem = kv_smem + KV_STAGES * 2 * KV_TILE_BYTES;  // tile x at + x * P_BYTES
  uint8_t* p_ptr = base_ptr + 2 * Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES;
  const uint32_t bar0 = p_smem + 2 * P_BYTES;
  Bars B;
  B.q = bar0;
  B.kv_full = bar0 + 8;                  // KV_STAGES barriers
  B.kv_empty = bar0 + 8 + 8 * KV_STAGES;
  B.s[0] = bar0 + 8 + 16 * KV_STAGES;
  B.s[1] = B.s[0] + 8;
  B.p[0] = B.s[0] + 16;
  B.p[1] = B.s[0] + 24;
  B.o[0] = B.s[0] + 32;
  B.o[1] = B.s[0] + 40;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(p_ptr + 2 * P_BYTES + 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, h = blockIdx.y;
  const int row0 = a.qblock_row0[blk];
  const int rows = a.qblock_rows[blk];  // 1..256
  const int kv0 = a.qblock_kv0[blk];

  // visible-key count of this thread's query row and the maxima of the two Q tiles
  const int grp = (warp >= 6) ? 1 : 0;                 // softmax group / Q tile of this warp
  const int r = (warp & 3) * 32 + lane;                // row inside the Q tile (softmax warps)
  int my_cnt = 0;
  if (warp >= 2) {
    const int qr = grp * BQ + r;
    if (qr < rows) my_cnt = a.kv_count[row0 + qr];
    int mx = my_cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_max_cnt[warp - 2] = mx;
  }
  if (threadIdx.x == 0) {
    mbar_init(B.q, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(B.kv_full + 8 * s, 1);
      mbar_init(B.kv_empty + 8 * s, 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(B.s[x], 1);
      mbar_init(B.p[x], 128);
      mbar_init(B.o[x], 1);
    }
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
  const int cnt_a = max(max(s_max_cnt[0], s_max_cnt[1]), max(s_max_cnt[2], s_max_cnt[3]));
  const int cnt_b = max(max(s_max_cnt[4], s_max_cnt[5]), max(s_max_cnt[6], s_max_cnt[7]));
  const int n_a = (cnt_a + BKV - 1) / BKV;
  const int n_b = (cnt_b + BKV - 1) / BKV;
  const int n_tiles = max(n_a, n_b);

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      const bool two = rows > BQ;
      mbar_expect_tx(B.q, two ? 2 * Q_BYTES : Q_BYTES);
      tma_load_2d(q_smem, &tmap_q, h * HD, row0, B.q);
      if (two) tma_load_2d(q_smem + Q_BYTES, &tmap_q, h * HD, row0 + BQ, B.q);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait_bounded(B.kv_empty + 8 * s, ph ^ 1)) {
          arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_MMA);
          break;
        }
        const uint32_t dst = kv_smem + s * 2 * KV_TILE_BYTES;
        mbar_expect_tx(B.kv_full + 8 * s, 2 * KV_TILE_BYTES);
        tma_load_2d(dst, &tmap_k, h * HD, kv0 + j * BKV, B.kv_full + 8 * s);
        tma_load_2d(dst + KV_TILE_BYTES, &tmap_v, h * HD, kv0 + j * BKV, B.kv_full + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      bool ok = mbar_wait_bounded(B.q, 0);
      if (!ok) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
      const uint64_t dq[2] = {umma_desc_k_sw128(q_smem), umma_desc_k_sw128(q_smem + Q_BYTES)};
      const int n_x[2] = {n_a, n_b};
      auto wait_kv = [&](int j) -> bool {
        if (mbar_wait_bounded(B.kv_full + 8 * (j % KV_STAGES), (j / KV_STAGES) & 1)) return true;
        arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
        return false;
      };
      auto mma_s = [&](int x, int j) {  // S_x = Q_x K(j)^T
        const uint64_t dk = umma_desc_k_sw128(kv_smem + (j % KV_STAGES) * 2 * KV_TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_f16(tmem_base + x * 128, dq[x] + 2 * ks, dk + 2 * ks, idesc_qk, ks ? 1u : 0u);
        umma_commit(B.s[x]);
      };
      auto mma_o = [&](int x, int j) -> bool {  // Otile_x[j & 1] = P_x V(j)
        if (!mbar_wait_bounded(B.p[x], j & 1)) {
          arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
          return false;
        }
        tc_fence_after();
        const uint64_t dv = umma_desc_mn_sw128(kv_smem + (j % KV_STAGES) * 2 * KV_TILE_BYTES + KV_TILE_BYTES);
        const uint32_t d_o = tmem_base + 256 + x * 128 + (j & 1) * 64;
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          const uint64_t dp = umma_desc_k_sw128(p_smem + x * P_BYTES + (ks >> 2) * (BQ * 128)) + 2 * (ks & 3);
          // 16 keys = 16 rows of 128 bytes = 2048 bytes further into the V tile
          umma_f16(d_o, dp, dv + (uint64_t)(ks * (2048 >> 4)), idesc_pv, ks ? 1u : 0u);
        }
        umma_commit(B.o[x]);
        return true;
      };
      if (ok) ok = wait_kv(0);
      if (ok) {
        tc_fence_after();
        if (n_x[0] > 0) mma_s(0, 0);
      }
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j < n_x[1]) mma_s(1, j);
        if (j < n_x[0]) ok = mma_o(0, j);
        if (ok && j + 1 < n_x[0]) {
          ok = wait_kv(j + 1);
          if (ok) {
            tc_fence_after();
            mma_s(0, j + 1);
          }
        }
        if (ok && j < n_x[1]) ok = mma_o(1, j);
        if (ok) umma_commit(B.kv_empty + 8 * (j % KV_STAGES));
        if (ok && j + 1 < n_tiles) {
          ok = wait_kv(j + 1);
          if (ok) tc_fence_after();
        }
      }
    }
  } else {
    // ---- softmax / output threads: one query row each ----
    const int quarter = warp & 3;
    const int n_mine = grp ? n_b : n_a;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t t_s = t_lane + grp * 128;
    const uint32_t t_o = t_lane + 256 + grp * 128;
    uint8_t* p_row = p_ptr + grp * P_BYTES + r * 128;
    const float sc = 0.125f * LOG2E;
    float m = -INFINITY, l = 0.f, alpha_pending = 1.f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    bool ok = true;
    // o = o * alpha + Otile(j): folded one tile late, so the PV MMA is off the critical path
    auto fold = [&](int j) -> bool {
      bool good = mbar_wait_bounded(B.o[grp], j & 1);
      if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t oreg[32];
        tmem_ld_32x32(t_o + (j & 1) * 64 + c * 32, oreg);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_pending, __uint_as_float(oreg[i]));
      }
      return true;
    };
    for (int j = 0; j < n_mine; ++j) {
      if (ok && !mbar_wait_bounded(B.s[grp], j & 1)) {
        arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int n_valid = min(max(my_cnt - j * BKV, 0), BKV);   // visible keys of this row in the tile
      const bool full = __all_sync(0xffffffffu, n_valid == BKV);
      // Both passes keep the tcgen05.ld of the next 32-column chunk in flight while the current
      // chunk is processed (two register buffers).
      uint32_t sbuf[2][32];
      // pass 1: row maximum of the visible raw scores
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      tmem_ld_32x32(t_s, sbuf[0]);
      tmem_wait_ld_dep(sbuf[0]);
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t (&cur)[32] = sbuf[c & 1];
        // chunk c+1 of this pass, or chunk 0 of pass 2 (the scores are read twice)
        tmem_ld_32x32(t_s + ((c + 1) & 3) * 32, sbuf[(c + 1) & 1]);
        // four independent running maxima keep the dependency chains short
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx4[0] = fmaxf(mx4[0], __uint_as_float(cur[i]));
            mx4[1] = fmaxf(mx4[1], __uint_as_float(cur[i + 1]));
            mx4[2] = fmaxf(mx4[2], __uint_as_float(cur[i + 2]));
            mx4[3] = fmaxf(mx4[3], __uint_as_float(cur[i + 3]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < n_valid) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(cur[i]));
        }
        tmem_wait_ld_dep(sbuf[(c + 1) & 1]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m, mx * sc);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      if (j > 0) {
        ok = fold(j - 1);  // also guarantees the PV MMA of tile j-1 no longer reads the P buffer
        if (!ok) break;
      }
      const float alpha = exp2f(m - m_safe);
      float ls0 = 0.f, ls1 = 0.f;
      // pass 2: probabilities -> shared memory (swizzled K-major, 16-bit); sbuf[0] holds chunk 0
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t (&cur)[32] = sbuf[c & 1];
        if (c + 1 < BKV / 32) tmem_ld_32x32(t_s + (c + 1) * 32, sbuf[(c + 1) & 1]);
        uint32_t pk[16];
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2_fast(fmaf(__uint_as_float(cur[i]), sc, -m_safe));
            const float p1 = ex2_fast(fmaf(__uint_as_float(cur[i + 1]), sc, -m_safe));
            ls0 += p0;
            ls1 += p1;
            pk[i >> 1] = pack2_prob(p0, p1, a.act_f16);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_fast(fmaf(__uint_as_float(cur[i]), sc, -m_safe));
            float p1 = ex2_fast(fmaf(__uint_as_float(cur[i + 1]), sc, -m_safe));
            if (c * 32 + i >= n_valid) p0 = 0.f;
            if (c * 32 + i + 1 >= n_valid) p1 = 0.f;
            ls0 += p0;
            ls1 += p1;
            pk[i >> 1] = pack2_prob(p0, p1, a.act_f16);
          }
        }
        // columns [c*32, c*32+32) of row r: tile = c / 2, 16-byte chunks ch0 .. ch0+3
        uint8_t* tile = p_row + (c >> 1) * (BQ * 128);
        const int ch0 = (c & 1) * 4;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int ch = (ch0 + q4) ^ (r & 7);
          *reinterpret_cast<uint4*>(tile + ch * 16) =
              make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
        if (c + 1 < BKV / 32) tmem_wait_ld_dep(sbuf[(c + 1) & 1]);
      }
      l = l * alpha + (ls0 + ls1);
      m = m_new;
      alpha_pending = alpha;
      // make the generic-proxy writes of P visible to the tensor-core (async) proxy
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(B.p[grp]);
    }
    if (ok && n_mine > 0) {
      // the last tile's contribution: o = o * alpha_last + Otile(n-1)
      ok = fold(n_mine - 1);
    }
    const int qr = grp * BQ + r;
    if (qr < rows) {
      const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
      uint16_t* dst = reinterpret_cast<uint16_t*>(a.out16) + ((size_t)(row0 + qr) * a.n_heads + h) * HD;
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
  attn_prefill_kernel<<<grid, N_THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, a, idesc_qk, idesc_pv);
  arcb_count_launch(1);
  return (int)cudaGetLastError();
}
