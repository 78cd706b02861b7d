// Flash-style causal prefill attention on tcgen05 tensor cores with TMEM accumulators.
//
// One CTA = up to 256 consecutive query rows of one sequence (two 128-row Q tiles, A and B) x one
// head.  Warp roles (352 threads): warp 0 TMA producer, warp 1 MMA issuer of tile A, warp 2 MMA
// issuer of tile B, warps 3-6 softmax group of tile A, warps 7-10 softmax group of tile B (one
// thread per query row; a warp reads the TMEM lane quarter warp % 4).  Each issuer walks its own
// tile's fixed sequence S(0), S(1), PV(0), S(2), PV(1), ... and BLOCKS on the one barrier its next
// step needs, so a product is issued the moment its operands are ready (an earlier single issuer
// polled both tiles' barriers in turn, and a failed mbarrier.try_wait may suspend its thread, which
// left the tensor pipe idle between steps).  Per 128-key tile j:
//   TMA        K and V tiles [128 keys][64 dims], 128-byte swizzle, 3-stage ring shared by A and B
//   MMA        S_x = Q_x K^T   (UMMA 128x128x16 x4, fp32 in TMEM)            x in {A, B}
//   softmax_x  the row's 128 scores are read once from TMEM into registers; row max;
//              p = exp2(s*c - m_ref) written 16-bit back into TMEM (64 columns per Q tile: the
//              A operand of the next product is read from tensor memory, so P never touches
//              shared memory)
//   MMA        O_x += P_x V    (UMMA 128x64x16 x8, A = P from TMEM, V is the MN-major B operand),
//              accumulated in TMEM across all tiles
// The reference maximum m_ref of a row is only raised when the true maximum exceeds it by more
// than 8 (in log2 units), so p <= 256 stays well inside the 16-bit range and the accumulated O
// rarely needs rescaling; when it does, the row's thread rescales O in TMEM before releasing P.
// The final 1/l normalisation makes the result independent of m_ref.
// Scores stay fp32 until the row's reference maximum has been subtracted (t = s * 1/sqrt(64) *
// log2(e) - m_ref <= 8): only that shifted value is rounded to half, so neither the size of q.k nor
// the 16-bit range limits what the softmax can represent.
// In the packed-half path POLY of every 8 exp2 pairs are evaluated on the FMA pipe (Cody-Waite
// split + cubic polynomial + exponent insertion, all on packed halves) instead of the
// special-function unit, which is the busiest pipe of this kernel; the two kinds are interleaved
// so that both pipes work at once.
// The two groups run out of phase: the tensor core works on one Q tile while the other group's
// threads do exponentials.  Rows carry their own visible-key count (causal AND key padding as a
// prefix length), so no mask tensor exists.  Q, K, V and P share one 16-bit format (kind::f16
// needs equal A/B formats).  Every mbarrier wait is bounded.
#include <cstdlib>

#include "attn_prefill.cuh"
#include "launch.cuh"
#include "gemm.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 64;
constexpr int Q_BYTES = BQ * HD * 2;          // 16 KB per Q tile
constexpr int KV_TILE_BYTES = BKV * HD * 2;   // 16 KB each for K and V
constexpr int KV_STAGES = 4;
constexpr int SMEM_BYTES = 2 * Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES + 1024 + 512;
// S_A [0,128) S_B [128,256) O_A [256,320) O_B [320,384) P_A [384,448) P_B [448,512)
constexpr int TMEM_COLS = 512;
constexpr int TMEM_P = 384;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int N_THREADS = 352;
constexpr int SOFTMAX_WARP0 = 3;   // first softmax warp
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units
#ifndef ARCB_FLASH_SPLIT_DEFAULT
#define ARCB_FLASH_SPLIT_DEFAULT 1
#endif
#ifndef ARCB_FLASH_POLY_DEFAULT
#define ARCB_FLASH_POLY_DEFAULT 2   // of every 8 exp2 pairs on the FMA pipe; with two threads per query row 2 beats 3 by 1.9 % (loop and cold call)
#endif

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

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 h2_from_bits(uint32_t b) { return *reinterpret_cast<__half2*>(&b); }

// Re-division of the CTA's registers between warpgroups (all four warps of a warpgroup execute it)
__device__ __forceinline__ void reg_dealloc_24() { asm volatile("setmaxnreg.dec.sync.aligned.u32 24;"); }
__device__ __forceinline__ void reg_alloc_112() { asm volatile("setmaxnreg.inc.sync.aligned.u32 112;"); }

__device__ __forceinline__ float max3_f32(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
// (t0, t1) = (s0 * c + m, s1 * c + m) with one two-wide fp32 fused multiply-add
__device__ __forceinline__ void shift2_f32(uint32_t s0, uint32_t s1, uint64_t c2, uint64_t m2, float& t0, float& t1) {
  uint64_t sp, tp;
  asm("mov.b64 %0, {%1, %2};" : "=l"(sp) : "r"(s0), "r"(s1));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(tp) : "l"(sp), "l"(c2), "l"(m2));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(t0), "=f"(t1) : "l"(tp));
}

// 2^t for two packed halves, t <= 8, WITHOUT the special-function unit (9 FMA/ALU-pipe instructions
// per pair).  t is clamped to -15 (anything below yields exactly 0, so masked -inf scores work),
// n = round(t) comes from adding 1536 (ulp 1 at that magnitude; the sum's bit pattern is
// 0x6600 + n), f = t - n lies in [-0.5, 0.5] exactly, 2^f ~ 1 + f (c1 + f (c2 + f c3)) (max
// relative error 5.4e-4 in half arithmetic, about one half ulp) and 2^n is built in the exponent
// field: bits = (n + 15) << 10 per half.  One 32-bit multiply-add makes both halves' scale at
// once: (r * 1024 + C) leaves (n + 15) << 10 in each 16-bit lane for n in [-15, 16] because the
// low lane's spill into the high lane plus its carry is the constant 0x198.
__device__ __forceinline__ __half2 ex2_poly_half2(__half2 t) {
  t = __hmax2(t, h2_from_bits(0xCB80CB80u));                   // max(t, -15)
  const __half2 magic = h2_from_bits(0x66006600u);             // 1536
  const __half2 r = __hadd2(t, magic);
  const __half2 f = __hsub2(t, __hsub2(r, magic));
  __half2 q = __hfma2(h2_from_bits(0x2B1B2B1Bu), f, h2_from_bits(0x33C233C2u));
  q = __hfma2(q, f, h2_from_bits(0x398C398Cu));
  const __half2 s = h2_from_bits(h2_bits(r) * 1024u + 0x3A683C00u);  // 2^n
  return __hfma2(q, __hmul2(f, s), s);
}
// which of the 8 exp2 pairs of a group go to the polynomial (spread out so the pipes interleave)
template <int POLY>
__device__ __forceinline__ constexpr bool ex2_on_fma(int e) {
  return POLY >= 8 ? true
       : POLY == 4 ? (e & 1) == 1
       : POLY == 3 ? (e == 1 || e == 4 || e == 6)
       : POLY == 2 ? (e == 3 || e == 7)
       : POLY == 1 ? (e == 5)
       : false;
}

struct Bars {
  uint32_t q, kv_full, kv_empty, s[2], p[2], o[2], sfree[2];
};

// ---- TMA producer (one thread): both Q tiles once, then the K and V tile of every key tile ----
__device__ __forceinline__ void flash_tma_producer(const CUtensorMap* tmap_q, const CUtensorMap* tmap_k,
                                                   const CUtensorMap* tmap_v, const Bars& B, uint32_t q_smem,
                                                   uint32_t kv_smem, int h, int row0, int rows, int kv0, int n_tiles,
                                                   int* err) {
  const bool two = rows > BQ;
  mbar_expect_tx(B.q, two ? 2 * Q_BYTES : Q_BYTES);
  tma_load_2d(q_smem, tmap_q, h * HD, row0, B.q);
  if (two) tma_load_2d(q_smem + Q_BYTES, tmap_q, h * HD, row0 + BQ, B.q);
  for (int j = 0; j < n_tiles; ++j) {
    const int s = j % KV_STAGES;
    const uint32_t ph = (j / KV_STAGES) & 1;
    if (!mbar_wait_bounded(B.kv_empty + 8 * s, ph ^ 1)) {
      arcb_set_error(err, ARCB_DEV_WAIT_TIMEOUT_MMA);
      break;
    }
    const uint32_t dst = kv_smem + s * 2 * KV_TILE_BYTES;
    mbar_expect_tx(B.kv_full + 8 * s, 2 * KV_TILE_BYTES);
    tma_load_2d(dst, tmap_k, h * HD, kv0 + j * BKV, B.kv_full + 8 * s);
    tma_load_2d(dst + KV_TILE_BYTES, tmap_v, h * HD, kv0 + j * BKV, B.kv_full + 8 * s);
  }
}

// ---- MMA issuer of Q tile x (one thread): S(0), S(1), PV(0), S(2), PV(1), ... each behind a blocking
// wait on the one barrier it needs ----
__device__ __forceinline__ void flash_mma_issuer(int x, const Bars& B, uint32_t q_smem, uint32_t kv_smem,
                                                 uint32_t tmem_base, int n_a, int n_b, uint32_t idesc_qk,
                                                 uint32_t idesc_pv, int* err) {
  const int n_x = x ? n_b : n_a;
  const int n_tiles = max(n_a, n_b);
  bool ok = true;
  auto wait_or_flag = [&](uint32_t bar, uint32_t parity, int code) {
    if (ok && !mbar_wait_bounded(bar, parity)) {
      arcb_set_error(err, code);
      ok = false;
    }
  };
  if (n_x > 0) wait_or_flag(B.q, 0, ARCB_DEV_WAIT_TIMEOUT_TMA);
  const uint64_t dq = umma_desc_k_sw128(q_smem + x * Q_BYTES);
  auto mma_s = [&](int j) {  // S_x = Q_x K(j)^T
    const uint64_t dk = umma_desc_k_sw128(kv_smem + (j % KV_STAGES) * 2 * KV_TILE_BYTES);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      umma_f16(tmem_base + x * 128, dq + 2 * ks, dk + 2 * ks, idesc_qk, ks ? 1u : 0u);
    umma_commit(B.s[x]);
  };
  auto mma_o = [&](int j) {  // O_x (+)= P_x V(j); then this tile is done with K/V stage j
    const uint64_t dv = umma_desc_mn_sw128(kv_smem + (j % KV_STAGES) * 2 * KV_TILE_BYTES + KV_TILE_BYTES);
    const uint32_t d_o = tmem_base + 256 + x * 64;
#pragma unroll
    for (int ks = 0; ks < BKV / 16; ++ks) {
      // A = P_x from tensor memory: 16 keys = 8 columns of packed 16-bit pairs;
      // 16 keys = 16 rows of 128 bytes = 2048 bytes further into the V tile
      umma_f16_ts(d_o, tmem_base + TMEM_P + x * 64 + ks * 8, dv + (uint64_t)(ks * (2048 >> 4)), idesc_pv,
                  (j | ks) ? 1u : 0u);
    }
    umma_commit(B.o[x]);
    umma_commit(B.kv_empty + 8 * (j % KV_STAGES));
  };
  for (int j = 0; ok && j < n_x; ++j) {
    wait_or_flag(B.kv_full + 8 * (j % KV_STAGES), (j / KV_STAGES) & 1, ARCB_DEV_WAIT_TIMEOUT_TMA);   // K(j) has landed
    if (j > 0) wait_or_flag(B.sfree[x], (j - 1) & 1, ARCB_DEV_WAIT_TIMEOUT_ACC);   // S(j-1) copied out of TMEM
    if (!ok) break;
    tc_fence_after();
    mma_s(j);
    if (j > 0) {
      wait_or_flag(B.p[x], (j - 1) & 1, ARCB_DEV_WAIT_TIMEOUT_ACC);                // P(j-1) published
      if (!ok) break;
      tc_fence_after();
      mma_o(j - 1);
    }
  }
  if (ok && n_x > 0) {
    wait_or_flag(B.p[x], (n_x - 1) & 1, ARCB_DEV_WAIT_TIMEOUT_ACC);
    if (ok) {
      tc_fence_after();
      mma_o(n_x - 1);
    }
  }
  // K/V stages this tile does not use (the other tile sees more keys): give them back as soon as
  // they have landed, in order, so that each arrival counts for the right use of the stage
  for (int j = n_x; ok && j < n_tiles; ++j) {
    wait_or_flag(B.kv_full + 8 * (j % KV_STAGES), (j / KV_STAGES) & 1, ARCB_DEV_WAIT_TIMEOUT_TMA);
    if (ok) mbar_arrive(B.kv_empty + 8 * (j % KV_STAGES));
  }
}

// SOFTMAX selects the arithmetic of the softmax threads:
//   0  fp32 throughout, probabilities packed to the activation format (used for bfloat16)
//   1  scores packed to half2 as they leave TMEM; max, scale-and-shift, exp2 and sums on half2.
// (A third form, fp32 scores with a 3-input max and fp32 exp2, packing only the probabilities,
// issues fewer instructions but needs all 128 scores live in fp32: it spilled and measured
// 66.8 ms against 62.6 ms for form 1 on 61 482 tokens of 10 247-token prompts.)
// 11 warps are allocated as 12 (registers are handed out per group of four warps): 168 registers per
// thread is what fits, which is also what the launch bound makes the compiler assume.
template <int SOFTMAX, int POLY>
__global__ void __launch_bounds__(N_THREADS, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, AttnPrefillArgs a, uint32_t idesc_qk,
                    uint32_t idesc_pv) {
  pdl_launch_dependents();
  pdl_wait();   // the prologue below already reads the work list from global memory
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_max_cnt[8];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t q_smem = base;                                   // tile x at + x * Q_BYTES
  const uint32_t kv_smem = base + 2 * Q_BYTES;                    // stage s: K at + s*32K, V at +16K
  const uint32_t bar0 = kv_smem + KV_STAGES * 2 * KV_TILE_BYTES;
  uint8_t* bar_ptr = base_ptr + 2 * Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES;
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
  B.sfree[0] = B.s[0] + 48;
  B.sfree[1] = B.s[0] + 56;
  // the barriers above end at byte 136 of this region; the TMEM-address slot sits well clear of them
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, h = blockIdx.y;
  const int row0 = a.qblock_row0[blk];
  const int rows = a.qblock_rows[blk];  // 1..256
  const int kv0 = a.qblock_kv0[blk];

  // visible-key count of this thread's query row and the maxima of the two Q tiles
  const int grp = (warp >= SOFTMAX_WARP0 + 4) ? 1 : 0;    // softmax group / Q tile of this warp
  const int r = (warp & 3) * 32 + lane;                // row inside the Q tile (softmax warps)
  int my_cnt = 0;
  if (warp >= SOFTMAX_WARP0) {
    const int qr = grp * BQ + r;
    if (qr < rows) my_cnt = a.kv_count[row0 + qr];
    int mx = my_cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_max_cnt[warp - SOFTMAX_WARP0] = mx;
  }
  if (threadIdx.x == 0) {
    mbar_init(B.q, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(B.kv_full + 8 * s, 1);
      mbar_init(B.kv_empty + 8 * s, 2);   // one arrival per issuer
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(B.s[x], 1);
      mbar_init(B.p[x], 128);
      mbar_init(B.o[x], 1);
      mbar_init(B.sfree[x], 128);
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
    if (lane == 0 && n_tiles > 0) flash_tma_producer(&tmap_q, &tmap_k, &tmap_v, B, q_smem, kv_smem, h, row0, rows, kv0, n_tiles, a.err);
  } else if (warp == 1 || warp == 2) {
    if (lane == 0 && n_tiles > 0)
      flash_mma_issuer(warp - 1, B, q_smem, kv_smem, tmem_base, n_a, n_b, idesc_qk, idesc_pv, a.err);
  } else {
    // ---- softmax / output threads: one query row each ----
    const int quarter = warp & 3;
    const int n_mine = grp ? n_b : n_a;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t t_s = t_lane + grp * 128;
    const uint32_t t_o = t_lane + 256 + grp * 64;
    const uint32_t t_p = t_lane + TMEM_P + grp * 64;
    const float sc = 0.125f * LOG2E;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // O of earlier tiles was accumulated against the old reference maximum: rescale it in TMEM
    auto rescale_o = [&](float alpha) {
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t oreg[32];
        tmem_ld_32x32(t_o + c * 32, oreg);
        tmem_wait_ld_dep(oreg);
#pragma unroll
        for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
        tmem_st_32x32(t_o + c * 32, oreg);
      }
      tmem_wait_st();
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
      if constexpr (SOFTMAX == 1) {
        // ---- packed-half path.  The row maximum and the shift t = s * c - m_ref are computed in fp32
        // (3-input max, packed two-wide fused multiply-add), t is rounded to half once (|t| is small
        // where the probability is large, so the rounding costs little), and exp2 and the row sum run
        // on packed halves ----
        uint32_t sv[4][32];
        // all four loads in flight before the first wait: the TMEM read latency is paid once per tile
        tmem_ld_32x32(t_s, sv[0]);
        tmem_ld_32x32(t_s + 32, sv[1]);
        tmem_ld_32x32(t_s + 64, sv[2]);
        tmem_ld_32x32(t_s + 96, sv[3]);
        tmem_wait_ld_dep(sv[0]);
        tmem_wait_ld_dep(sv[1]);
        tmem_wait_ld_dep(sv[2]);
        tmem_wait_ld_dep(sv[3]);
        // S is in registers: the tensor core may overwrite it with the next tile's scores
        tc_fence_before();
        mbar_arrive(B.sfree[grp]);
        if (!full) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= n_valid) sv[c][i] = 0xff800000u;   // -inf: exp2 gives exactly 0
        }
        float mx4[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          mx4[c] = fmaxf(__uint_as_float(sv[c][0]), __uint_as_float(sv[c][1]));
#pragma unroll
          for (int i = 2; i < 32; i += 2) mx4[c] = max3_f32(mx4[c], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
        }
        const float mx = fmaxf(max3_f32(mx4[0], mx4[1], mx4[2]), mx4[3]) * sc;
        float alpha = 1.f;
        if (mx > m_ref + RESCALE_THRESHOLD) {  // also the first visible tile (m_ref = -inf)
          alpha = (m_ref == -INFINITY) ? 0.f : ex2_fast(m_ref - mx);
          m_ref = mx;
        }
        l *= alpha;
        const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
        const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(-m_safe, -m_safe);
        // Probabilities of 16 keys at a time, kept as eight registers per group so that each group
        // leaves through one 8-column tensor-memory store without register shuffling.  A pair goes
        // either to the special-function unit (fp32 exp2 of each shifted score, then one rounding of
        // the pair to half) or to the FMA pipe (the pair is rounded to half first and the packed
        // polynomial evaluates both at once).
        uint32_t pr[8][8];
        float lsum = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          __half2 p[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int k = g * 8 + e;                    // keys 2k, 2k + 1 = P column k
            float t0, t1;
            shift2_f32(sv[k >> 4][(2 * k) & 31], sv[k >> 4][((2 * k) & 31) + 1], sc2, nm2, t0, t1);
            p[e] = ex2_on_fma<POLY>(e) ? ex2_poly_half2(__floats2half2_rn(t0, t1))
                                       : __floats2half2_rn(ex2_fast(t0), ex2_fast(t1));
          }
          const __half2 t = __hadd2(__hadd2(__hadd2(p[0], p[1]), __hadd2(p[2], p[3])),
                                    __hadd2(__hadd2(p[4], p[5]), __hadd2(p[6], p[7])));
          lsum += __low2float(t) + __high2float(t);
#pragma unroll
          for (int e = 0; e < 8; ++e) pr[g][e] = h2_bits(p[e]);
        }
        l += lsum;
        if (j > 0) {
          // PV(j-1) must have retired before P is overwritten and O rescaled; the exponentials above
          // needed neither, so they overlap that product
          bool good = mbar_wait_bounded(B.o[grp], (j - 1) & 1);
          if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
          ok = __all_sync(0xffffffffu, good);
          if (!ok) break;
          tc_fence_after();
        }
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) rescale_o(alpha);
#pragma unroll
        for (int g = 0; g < 8; ++g) tmem_st_32x8(t_p + g * 8, pr[g]);
      } else {
        // the row's 128 scores, read once
        uint32_t sv[4][32];
        tmem_ld_32x32(t_s, sv[0]);
        tmem_ld_32x32(t_s + 32, sv[1]);
        tmem_ld_32x32(t_s + 64, sv[2]);
        tmem_ld_32x32(t_s + 96, sv[3]);
        tmem_wait_ld_dep(sv[0]);
        tmem_wait_ld_dep(sv[1]);
        tmem_wait_ld_dep(sv[2]);
        tmem_wait_ld_dep(sv[3]);
        // S is in registers: the tensor core may overwrite it with the next tile's scores
        tc_fence_before();
        mbar_arrive(B.sfree[grp]);
        // row maximum of the visible raw scores (four independent chains)
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  #pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (full) {
  #pragma unroll
            for (int i = 0; i < 32; i += 4) {
              mx4[0] = fmaxf(mx4[0], __uint_as_float(sv[c][i]));
              mx4[1] = fmaxf(mx4[1], __uint_as_float(sv[c][i + 1]));
              mx4[2] = fmaxf(mx4[2], __uint_as_float(sv[c][i + 2]));
              mx4[3] = fmaxf(mx4[3], __uint_as_float(sv[c][i + 3]));
            }
          } else {
  #pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < n_valid) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;
        // raise the reference maximum only when it is far below the true one
        float alpha = 1.f;
        if (mx > m_ref + RESCALE_THRESHOLD) {  // also the first visible tile (m_ref = -inf)
          alpha = (m_ref == -INFINITY) ? 0.f : ex2_fast(m_ref - mx);
          m_ref = mx;
        }
        l *= alpha;
        if (j > 0) {
          // PV(j-1) must have retired: it reads the P buffer written below and updates O
          bool good = mbar_wait_bounded(B.o[grp], (j - 1) & 1);
          if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
          ok = __all_sync(0xffffffffu, good);
          if (!ok) break;
          tc_fence_after();
        }
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // O of earlier tiles was accumulated against the old reference: rescale it in TMEM
  #pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t oreg[32];
            tmem_ld_32x32(t_o + c * 32, oreg);
            tmem_wait_ld_dep(oreg);
  #pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, oreg);
          }
          tmem_wait_st();
        }
        const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
        float ls0 = 0.f, ls1 = 0.f;
        // probabilities -> tensor memory (16-bit pairs, 16 columns per 32 keys)
  #pragma unroll
        for (int c = 0; c < BKV / 32; c += 2) {
          uint32_t pk[32];
  #pragma unroll
          for (int cc = 0; cc < 2; ++cc)
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_fast(fmaf(__uint_as_float(sv[c + cc][i]), sc, -m_safe));
            float p1 = ex2_fast(fmaf(__uint_as_float(sv[c + cc][i + 1]), sc, -m_safe));
            if (!full) {
              if ((c + cc) * 32 + i >= n_valid) p0 = 0.f;
              if ((c + cc) * 32 + i + 1 >= n_valid) p1 = 0.f;
            }
            ls0 += p0;
            ls1 += p1;
            pk[cc * 16 + (i >> 1)] = pack2_prob(p0, p1, a.act_f16);
          }
          tmem_st_32x32(t_p + (c >> 1) * 32, pk);
        }
        l += ls0 + ls1;
      }
      // P is complete in tensor memory before the MMA warp is told
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(B.p[grp]);
    }
    // the accumulated output row
    if (ok && n_mine > 0) {
      bool good = mbar_wait_bounded(B.o[grp], (n_mine - 1) & 1);
      if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
      ok = __all_sync(0xffffffffu, good);
    }
    const int qr = grp * BQ + r;
    const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
    uint16_t* dst = reinterpret_cast<uint16_t*>(a.out16) + ((size_t)(row0 + qr) * a.n_heads + h) * HD;
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t oreg[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) oreg[i] = 0u;
      if (ok && n_mine > 0) {
        tc_fence_after();
        tmem_ld_32x32(t_o + c * 32, oreg);
        tmem_wait_ld_dep(oreg);
      }
      if (qr < rows) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack2_act(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv, a.act_f16);
          v.y = pack2_act(__uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv, a.act_f16);
          v.z = pack2_act(__uint_as_float(oreg[i + 4]) * inv, __uint_as_float(oreg[i + 5]) * inv, a.act_f16);
          v.w = pack2_act(__uint_as_float(oreg[i + 6]) * inv, __uint_as_float(oreg[i + 7]) * inv, a.act_f16);
          *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
        }
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

// ---------------------------------------------------------------------------------------------
// Two threads per query row (half format only).  The one-thread-per-row kernel above leaves two
// softmax warps on each of the SM's four schedulers, and its profile is dominated by fixed-latency
// dependency stalls (issue slots about half used, tensor pipe about a third).  Here every row of a Q
// tile is shared by two threads in two warps of the same TMEM lane quarter: thread `half` owns
// keys [64 half, 64 half + 64) of each tile (64 score columns, 32 packed probability columns) and
// output dims [32 half, 32 half + 32).  That puts four softmax warps on each scheduler.  The two
// threads of a row exchange their half-tile maxima through shared memory once per tile (an
// mbarrier per pair of warps, with the same bounded wait as every other barrier) so that both use
// the same reference maximum; row sums stay private until the end.
//
// 640 threads: warps 0-3 helpers (TMA producer, issuer A, issuer B, one idle), warps 4-7 / 8-11
// tile A halves 0 / 1, warps 12-15 / 16-19 tile B halves 0 / 1.  Registers are re-divided after
// start-up (setmaxnreg): the helper warpgroup keeps 24, the four softmax warpgroups get 112 each
// (24 * 128 + 112 * 512 = 60 416 of the 65 536, so the increase can never wait for registers).
// ---------------------------------------------------------------------------------------------
constexpr int SPLIT_THREADS = 640;

template <int POLY>
__global__ void __launch_bounds__(SPLIT_THREADS, 1)
attn_prefill_split_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, AttnPrefillArgs a, uint32_t idesc_qk,
                          uint32_t idesc_pv) {
  pdl_launch_dependents();
  pdl_wait();   // the prologue below already reads the work list from global memory
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_max_cnt[16];
  __shared__ float s_xchg[2][2][2][BQ];   // [tile parity][Q tile][half][row]: half-tile maxima, then row sums
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t kv_smem = base + 2 * Q_BYTES;
  const uint32_t bar0 = kv_smem + KV_STAGES * 2 * KV_TILE_BYTES;
  uint8_t* bar_ptr = base_ptr + 2 * Q_BYTES + KV_STAGES * 2 * KV_TILE_BYTES;
  Bars B;
  B.q = bar0;
  B.kv_full = bar0 + 8;
  B.kv_empty = bar0 + 8 + 8 * KV_STAGES;
  B.s[0] = bar0 + 8 + 16 * KV_STAGES;
  B.s[1] = B.s[0] + 8;
  B.p[0] = B.s[0] + 16;
  B.p[1] = B.s[0] + 24;
  B.o[0] = B.s[0] + 32;
  B.o[1] = B.s[0] + 40;
  B.sfree[0] = B.s[0] + 48;
  B.sfree[1] = B.s[0] + 56;
  const uint32_t xbar0 = B.s[0] + 64;      // 8 barriers: one per (Q tile, lane quarter) pair of warps
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, h = blockIdx.y;
  const int row0 = a.qblock_row0[blk];
  const int rows = a.qblock_rows[blk];  // 1..256
  const int kv0 = a.qblock_kv0[blk];

  const int wg = (warp >> 2) - 1;          // softmax warpgroup 0..3 (helpers: -1)
  const int grp = wg >> 1;                 // Q tile
  const int half = wg & 1;                 // which 64 keys of a tile / which 32 output dims
  const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
  const int r = quarter * 32 + lane;       // row inside the Q tile
  int my_cnt = 0;
  if (warp >= 4) {
    const int qr = grp * BQ + r;
    if (qr < rows) my_cnt = a.kv_count[row0 + qr];
    int mx = my_cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_max_cnt[warp - 4] = mx;
  }
  if (threadIdx.x == 0) {
    mbar_init(B.q, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(B.kv_full + 8 * s, 1);
      mbar_init(B.kv_empty + 8 * s, 2);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(B.s[x], 1);
      mbar_init(B.p[x], 256);
      mbar_init(B.o[x], 1);
      mbar_init(B.sfree[x], 256);
    }
    for (int i = 0; i < 8; ++i) mbar_init(xbar0 + 8 * i, 64);
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
  int cnt_a = 0, cnt_b = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    cnt_a = max(cnt_a, s_max_cnt[i]);
    cnt_b = max(cnt_b, s_max_cnt[8 + i]);
  }
  const int n_a = (cnt_a + BKV - 1) / BKV;
  const int n_b = (cnt_b + BKV - 1) / BKV;
  const int n_tiles = max(n_a, n_b);

  if (warp < 4) {
    reg_dealloc_24();
    if (warp == 0) {
      if (lane == 0 && n_tiles > 0)
        flash_tma_producer(&tmap_q, &tmap_k, &tmap_v, B, q_smem, kv_smem, h, row0, rows, kv0, n_tiles, a.err);
    } else if (warp <= 2) {
      if (lane == 0 && n_tiles > 0)
        flash_mma_issuer(warp - 1, B, q_smem, kv_smem, tmem_base, n_a, n_b, idesc_qk, idesc_pv, a.err);
    }
  } else {
    reg_alloc_112();
    // ---- softmax / output threads: row r of Q tile grp, key half `half` ----
    const int n_mine = grp ? n_b : n_a;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t t_s = t_lane + grp * 128 + half * 64;
    const uint32_t t_o = t_lane + 256 + grp * 64 + half * 32;
    const uint32_t t_p = t_lane + TMEM_P + grp * 64 + half * 32;
    const uint32_t xbar = xbar0 + 8 * (grp * 4 + quarter);
    const float sc = 0.125f * LOG2E;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t xphase = 0;
    // both threads of a row publish a value and read the partner's; false if the partner never came
    auto exchange = [&](int slot, float mine, float& theirs) -> bool {
      s_xchg[slot][grp][half][r] = mine;
      mbar_arrive(xbar);
      const bool good = mbar_wait_bounded(xbar, xphase);
      xphase ^= 1u;
      theirs = s_xchg[slot][grp][half ^ 1][r];
      return good;
    };
    for (int j = 0; j < n_mine; ++j) {
      if (ok && !mbar_wait_bounded(B.s[grp], j & 1)) {
        arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[2][32];
      tmem_ld_32x32(t_s, sv[0]);
      tmem_ld_32x32(t_s + 32, sv[1]);
      tmem_wait_ld_dep(sv[0]);
      tmem_wait_ld_dep(sv[1]);
      // this thread's share of S is in registers
      tc_fence_before();
      mbar_arrive(B.sfree[grp]);
      const int n_valid = min(max(my_cnt - j * BKV, 0), BKV) - half * 64;   // visible keys within this half (may be <= 0)
      if (!__all_sync(0xffffffffu, n_valid >= 64)) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= n_valid) sv[c][i] = 0xff800000u;   // -inf: exp2 gives exactly 0
      }
      float mx2[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        mx2[c] = fmaxf(__uint_as_float(sv[c][0]), __uint_as_float(sv[c][1]));
#pragma unroll
        for (int i = 2; i < 32; i += 2) mx2[c] = max3_f32(mx2[c], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
      }
      float other;
      bool good = exchange(j & 1, fmaxf(mx2[0], mx2[1]), other);
      if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
      ok = __all_sync(0xffffffffu, good);
      if (!ok) break;
      const float mx = fmaxf(fmaxf(mx2[0], mx2[1]), other) * sc;   // the same value in both threads of the row
      float alpha = 1.f;
      if (mx > m_ref + RESCALE_THRESHOLD) {  // also the first visible tile (m_ref = -inf)
        alpha = (m_ref == -INFINITY) ? 0.f : ex2_fast(m_ref - mx);
        m_ref = mx;
      }
      l *= alpha;
      const float m_safe = (m_ref == -INFINITY) ? 0.f : m_ref;
      const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(-m_safe, -m_safe);
      uint32_t pr[4][8];
      // the 64 probabilities of this half-tile are summed as packed halves in a balanced tree (they are
      // at most 2^8 each and almost always at most 1, so the tree stays far inside the half range) and
      // leave half precision once per tile; the running row sum is fp32
      __half2 gsum[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        __half2 p[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int k = g * 8 + e;                    // this half's keys 2k, 2k + 1 = its P column k
          float t0, t1;
          shift2_f32(sv[k >> 4][(2 * k) & 31], sv[k >> 4][((2 * k) & 31) + 1], sc2, nm2, t0, t1);
          p[e] = ex2_on_fma<POLY>(e) ? ex2_poly_half2(__floats2half2_rn(t0, t1))
                                     : __floats2half2_rn(ex2_fast(t0), ex2_fast(t1));
        }
        gsum[g] = __hadd2(__hadd2(__hadd2(p[0], p[1]), __hadd2(p[2], p[3])),
                          __hadd2(__hadd2(p[4], p[5]), __hadd2(p[6], p[7])));
#pragma unroll
        for (int e = 0; e < 8; ++e) pr[g][e] = h2_bits(p[e]);
      }
      const float2 ts = __half22float2(__hadd2(__hadd2(gsum[0], gsum[1]), __hadd2(gsum[2], gsum[3])));
      l += ts.x + ts.y;
      if (j > 0) {
        // PV(j-1) must have retired before P is overwritten and O rescaled
        good = mbar_wait_bounded(B.o[grp], (j - 1) & 1);
        if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
        ok = __all_sync(0xffffffffu, good);
        if (!ok) break;
        tc_fence_after();
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // this thread's 32 output dims of the row were accumulated against the old reference maximum
        uint32_t oreg[32];
        tmem_ld_32x32(t_o, oreg);
        tmem_wait_ld_dep(oreg);
#pragma unroll
        for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
        tmem_st_32x32(t_o, oreg);
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_st_32x8(t_p + g * 8, pr[g]);
      // P (and a rescaled O) are complete in tensor memory before the MMA warp is told
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(B.p[grp]);
    }
    // the row's normaliser is the sum of the two halves' private sums
    float l_other = 0.f;
    if (ok && n_mine > 0) {
      bool good = exchange(n_mine & 1, l, l_other);
      good = mbar_wait_bounded(B.o[grp], (n_mine - 1) & 1) && good;
      if (!good) arcb_set_error(a.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
      ok = __all_sync(0xffffffffu, good);
    }
    const float l_row = half ? l_other + l : l + l_other;   // same order of addition in both threads
    const int qr = grp * BQ + r;
    const float inv = (ok && l_row > 0.f) ? 1.f / l_row : 0.f;
    uint16_t* dst = reinterpret_cast<uint16_t*>(a.out16) + ((size_t)(row0 + qr) * a.n_heads + h) * HD + half * 32;
    uint32_t oreg[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) oreg[i] = 0u;
    if (ok && n_mine > 0) {
      tc_fence_after();
      tmem_ld_32x32(t_o, oreg);
      tmem_wait_ld_dep(oreg);
    }
    if (qr < rows) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 v;
        v.x = pack2_act(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv, 1);
        v.y = pack2_act(__uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv, 1);
        v.z = pack2_act(__uint_as_float(oreg[i + 4]) * inv, __uint_as_float(oreg[i + 5]) * inv, 1);
        v.w = pack2_act(__uint_as_float(oreg[i + 6]) * inv, __uint_as_float(oreg[i + 7]) * inv, 1);
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

namespace {

// exp2 pairs (of every 8) evaluated on the FMA pipe by the packed-half kernel.  The default is the
// measured optimum on B200; ARCB_FLASH_POLY=0..4 overrides it (read once) for A/B timing.
int flash_poly_share() {
  static const int v = [] {
    const char* e = getenv("ARCB_FLASH_POLY");
    if (e && e[0] >= '0' && e[0] <= '4' && e[1] == 0) return e[0] - '0';
    return ARCB_FLASH_POLY_DEFAULT;
  }();
  return v;
}

// 1 = two threads per query row (attn_prefill_split_kernel), 0 = one.  ARCB_FLASH_SPLIT overrides.
int flash_split() {
  static const int v = [] {
    const char* e = getenv("ARCB_FLASH_SPLIT");
    if (e && (e[0] == '0' || e[0] == '1') && e[1] == 0) return e[0] - '0';
    return ARCB_FLASH_SPLIT_DEFAULT;
  }();
  return v;
}

template <int POLY>
cudaError_t set_split_smem_attr() {
  return cudaFuncSetAttribute(attn_prefill_split_kernel<POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
}

template <int SOFTMAX, int POLY>
cudaError_t set_smem_attr() {
  return cudaFuncSetAttribute(attn_prefill_kernel<SOFTMAX, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              SMEM_BYTES);
}

}  // namespace

int arcb_attn_prefill_init() {
  cudaError_t e;
  if ((e = set_smem_attr<0, 0>()) != cudaSuccess) return (int)e;
  if ((e = set_smem_attr<1, 0>()) != cudaSuccess) return (int)e;
  if ((e = set_smem_attr<1, 1>()) != cudaSuccess) return (int)e;
  if ((e = set_smem_attr<1, 2>()) != cudaSuccess) return (int)e;
  if ((e = set_smem_attr<1, 3>()) != cudaSuccess) return (int)e;
  if ((e = set_smem_attr<1, 4>()) != cudaSuccess) return (int)e;
  if ((e = set_split_smem_attr<0>()) != cudaSuccess) return (int)e;
  if ((e = set_split_smem_attr<2>()) != cudaSuccess) return (int)e;
  if ((e = set_split_smem_attr<3>()) != cudaSuccess) return (int)e;
  if ((e = set_split_smem_attr<4>()) != cudaSuccess) return (int)e;
  return 0;
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
  cudaError_t le = cudaSuccess;
#define ARCB_LAUNCH_FLASH(SM, PL) \
  le = arcb_launch(attn_prefill_kernel<SM, PL>, grid, dim3(N_THREADS), SMEM_BYTES, stream, tq, tk, tv, a, idesc_qk, idesc_pv)
#define ARCB_LAUNCH_SPLIT(PL) \
  le = arcb_launch(attn_prefill_split_kernel<PL>, grid, dim3(SPLIT_THREADS), SMEM_BYTES, stream, tq, tk, tv, a, idesc_qk, idesc_pv)
  if (!a.act_f16) {
    ARCB_LAUNCH_FLASH(0, 0);
  } else if (flash_split()) {
    switch (flash_poly_share()) {
      case 0: case 1: ARCB_LAUNCH_SPLIT(0); break;
      case 2: ARCB_LAUNCH_SPLIT(2); break;
      case 3: ARCB_LAUNCH_SPLIT(3); break;
      default: ARCB_LAUNCH_SPLIT(4); break;
    }
  } else {
    switch (flash_poly_share()) {
      case 0: ARCB_LAUNCH_FLASH(1, 0); break;
      case 1: ARCB_LAUNCH_FLASH(1, 1); break;
      case 2: ARCB_LAUNCH_FLASH(1, 2); break;
      case 3: ARCB_LAUNCH_FLASH(1, 3); break;
      default: ARCB_LAUNCH_FLASH(1, 4); break;
    }
  }
#undef ARCB_LAUNCH_FLASH
#undef ARCB_LAUNCH_SPLIT
  arcb_count_launch(1);
  return (int)le;
}
