// y = A[M,K] * W[N,K]^T, both operands in the same 16-bit format (half or bfloat16: tcgen05
// kind::f16 rejects mixed A/B formats with an illegal-instruction fault), fp32 accumulate, with the
// fused epilogues of epilogue.cuh.  Two kernels:
//   gemm_tc_kernel   : persistent; tcgen05.mma (UMMA 128x256x16 or 128x128x16), two fp32
//                      accumulators in TMEM (the epilogue drains one while the next tile fills the
//                      other), operands staged by TMA (128-byte swizzle) through an mbarrier ring;
//                      warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-9 = epilogue.
//   gemm_simt_kernel : CUDA-core tile kernel for skinny M (weight streaming) and as
//                      the cross-check of the tensor-core path.
#include <cstdlib>

#include "gemm.cuh"
#include "launch.cuh"
#include "ptx_sm100.cuh"

using namespace sm100;

// ---------------------------------------------------------------------------
// tcgen05 kernel
// ---------------------------------------------------------------------------
namespace {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;  // 64 x 2 B = one 128-byte swizzle row
constexpr int TC_EPI_WARPS = 8;                  // two warps per TMEM lane quarter, half of the columns each
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;

template <int BN>
struct TcCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators: the epilogue drains one while the MMA fills the other
  // stages + barriers (full, empty per stage; acc_full, acc_empty x2) + tmem slot, + 1024 alignment slack
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

// The residual epilogue stages 128 x 32 fp32 chunks in shared memory (one 16 KB buffer per group of
// four epilogue warps) and adds them to the residual stream with a bulk tensor reduce.
constexpr int EPI_STAGE_GROUP_BYTES = 128 * 32 * 4;
template <int MODE>
__host__ __device__ constexpr int epi_stage_bytes() {
  return (MODE == EPI_RESID || MODE == EPI_SWIGLU || MODE == EPI_QKV_ROPE) ? 2 * EPI_STAGE_GROUP_BYTES : 0;
}
// epilogues that go through the staging buffers and the third tensor map
template <int BN, int MODE>
__host__ __device__ constexpr bool epi_staged() {
  return MODE == EPI_RESID || ((MODE == EPI_SWIGLU || MODE == EPI_QKV_ROPE) && BN == 256);
}

// Residual epilogue: x[m][n] += acc[m][n] (+ bias[n]) for this CTA's 128 rows and this group's
// column half, 32 columns at a time.  Each thread drops its row's 32 values into the staging
// buffer (128-byte rows, 16-byte chunks XOR-swizzled by row like the TMA 128-byte swizzle, so the
// row-per-thread writes are conflict-free), and one thread issues a bulk tensor reduce-add of the
// 128 x 32 box: the addition happens in L2 on whole sectors, rows beyond M are clipped by the
// tensor map, and every element of x receives exactly one addend per GEMM, so the result is the
// same fp32 sum a load-add-store would give.  The group's four warps meet at named barrier
// 1 + col_half; `elected` is the thread that owns the bulk groups.
template <int BN>
__device__ __forceinline__ void epilogue_resid_tma(const GemmEpilogue& ep, const CUtensorMap* tmap_x, uint32_t t_row,
                                                   int m0, int n_tile0, int col_half, int row_in_tile,
                                                   uint32_t stage_smem, uint8_t* stage_ptr, bool elected) {
  uint8_t* my_row = stage_ptr + row_in_tile * 128;
  const int sw = row_in_tile & 7;
#pragma unroll 1
  for (int c = col_half * (BN / 64); c < (col_half + 1) * (BN / 64); ++c) {
    const int n0 = n_tile0 + c * 32;
    if (n0 >= ep.N) break;  // uniform over the group
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_wait_ld();
    if (ep.bias) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 b = __ldg(reinterpret_cast<const float4*>(ep.bias + n0 + 4 * q));
        r[4 * q] = __float_as_uint(__uint_as_float(r[4 * q]) + b.x);
        r[4 * q + 1] = __float_as_uint(__uint_as_float(r[4 * q + 1]) + b.y);
        r[4 * q + 2] = __float_as_uint(__uint_as_float(r[4 * q + 2]) + b.z);
        r[4 * q + 3] = __float_as_uint(__uint_as_float(r[4 * q + 3]) + b.w);
      }
    }
    if (elected) bulk_wait_read_all();        // the previous reduce has read the buffer
    named_bar_sync(1 + col_half, 128);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<uint4*>(my_row + ((q ^ sw) << 4)) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
    fence_proxy_async_smem();
    named_bar_sync(1 + col_half, 128);
    if (elected && m0 < ep.M) {
      tma_reduce_add_2d(tmap_x, stage_smem, n0, m0);
      bulk_commit_group();
    }
  }
}

// SwiGLU epilogue of one 128-column accumulator group (64 gate columns, then the matching 64 up
// columns) of a 256-column tile: h[m][j] = silu(g + bg) * (u + bu) for the group's 64 outputs.  The
// group's four warps stage the 128 x 64 16-bit box (128-byte rows, XOR-swizzled 16-byte chunks) and
// one thread issues a bulk tensor store, instead of 8-byte stores a row pitch apart.
__device__ __forceinline__ void epilogue_swiglu_tma(const GemmEpilogue& ep, const CUtensorMap* tmap_h, uint32_t t_grp,
                                                    int m0, int n_grp0, int grp, int row_in_tile,
                                                    uint32_t stage_smem, uint8_t* stage_ptr, bool elected) {
  if (n_grp0 >= ep.N) return;  // uniform over the group: tile tail beyond N
  uint8_t* my_row = stage_ptr + row_in_tile * 128;
  const int sw = row_in_tile & 7;
  if (elected) bulk_wait_read_all();   // the previous store has read the buffer
  named_bar_sync(1 + grp, 128);
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t rg[32], ru[32];
    tmem_ld_32x32(t_grp + c * 32, rg);
    tmem_ld_32x32(t_grp + 64 + c * 32, ru);
    tmem_wait_ld();
    const int n0 = n_grp0 + c * 32;
#pragma unroll
    for (int k = 0; k < 4; ++k) {   // 8 outputs = one 16-byte chunk
      uint32_t w[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = k * 8 + h * 4;
        float4 g = make_float4(__uint_as_float(rg[i]), __uint_as_float(rg[i + 1]), __uint_as_float(rg[i + 2]),
                               __uint_as_float(rg[i + 3]));
        float4 u = make_float4(__uint_as_float(ru[i]), __uint_as_float(ru[i + 1]), __uint_as_float(ru[i + 2]),
                               __uint_as_float(ru[i + 3]));
        if (ep.bias) {
          const float4 bg = __ldg(reinterpret_cast<const float4*>(ep.bias + n0 + i));
          const float4 bu = __ldg(reinterpret_cast<const float4*>(ep.bias + n0 + i + 64));
          g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w;
          u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
        }
        w[2 * h] = pack2_act_chk(silu_f(g.x) * u.x, silu_f(g.y) * u.y, ep.act_f16, ep.err);
        w[2 * h + 1] = pack2_act_chk(silu_f(g.z) * u.z, silu_f(g.w) * u.w, ep.act_f16, ep.err);
      }
      *reinterpret_cast<uint4*>(my_row + (((c * 4 + k) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  fence_proxy_async_smem();
  named_bar_sync(1 + grp, 128);
  if (elected && m0 < ep.M) {
    tma_store_2d(tmap_h, stage_smem, (n_grp0 >> 7) * 64, m0);
    bulk_commit_group();
  }
}

// QKV epilogue of one 128-column accumulator group (two heads of one of the q / k / v sections; a
// 256-column tile never straddles sections because d_model is a multiple of 256 wherever this
// kernel is chosen).  Per head: 3D RoPE on q and k, the bf16 cache row written directly (its
// address is per token), and the 16-bit copy -- q16, or the call's K / V scratch when its rows are
// the packed rows themselves (kv16_identity) -- staged as a 128 x 64 box and written by one bulk
// tensor store, which also clips the rows beyond the tensor (M, or the scratch's row count).
//
// cbox_ptr != nullptr: this warp's 32 rows are consecutive cache rows of one sequence (a prompt run),
// so the bf16 cache rows of a head are one contiguous 4 KB block: the warp stages them in its own
// 32 x 64 box (cbox_smem / cbox_ptr, same swizzle) and lane 0 writes the box with one bulk tensor
// store at cache row cbox_row0 + h * t_max, instead of 32 rows x 4 sixteen-byte stores a row apart.
__device__ __forceinline__ void epilogue_qkv_tma(const GemmEpilogue& ep, const RopeRow& rr, const CUtensorMap* tmap_q,
                                                 const CUtensorMap* tmap_k, const CUtensorMap* tmap_v, uint32_t t_grp,
                                                 int m0, bool row_ok, int n_grp0, int grp, int row_in_tile,
                                                 uint32_t stage_smem, uint8_t* stage_ptr, bool elected,
                                                 const CUtensorMap* tmap_kc = nullptr, const CUtensorMap* tmap_vc = nullptr,
                                                 uint32_t cbox_smem = 0, uint8_t* cbox_ptr = nullptr,
                                                 long long cbox_row0 = 0) {
  uint8_t* my_row = stage_ptr + row_in_tile * 128;
  const int sw = row_in_tile & 7;
  const int d = ep.d_model;
  const int lane = row_in_tile & 31;
  uint8_t* my_crow = cbox_ptr ? cbox_ptr + lane * 128 : nullptr;
#pragma unroll 1
  for (int hh = 0; hh < 2; ++hh) {
    const int n_head0 = n_grp0 + hh * 64;
    if (n_head0 >= ep.N) break;  // uniform over the group
    const int sec = n_head0 / d;            // 0 q, 1 k, 2 v
    const int c = n_head0 - sec * d;        // column inside the section
    const int h = c >> 6;
    const bool staged = sec == 0 || (ep.k16 != nullptr && ep.kv16_identity);
    if (staged) {
      if (elected) bulk_wait_read_all();    // the previous store has read the buffer
      named_bar_sync(1 + grp, 128);
    }
    const bool cbox = sec > 0 && cbox_ptr != nullptr;   // warp-uniform
    if (cbox) {
      if (lane == 0) bulk_wait_read_all();  // this warp's previous cache box has been read
      __syncwarp();
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t acc[32];
      tmem_ld_32x32(t_grp + hh * 64 + half * 32, acc);
      tmem_wait_ld();
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
      if (sec < 2) {
        if (half == 0) rope_rotate32<0>(ep, rr, v);
        else rope_rotate32<16>(ep, rr, v);
      }
      if (cbox) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(my_crow + (((half * 4 + q) ^ sw) << 4)) =
              make_uint4(pack2_bf16(v[8 * q], v[8 * q + 1]), pack2_bf16(v[8 * q + 2], v[8 * q + 3]),
                         pack2_bf16(v[8 * q + 4], v[8 * q + 5]), pack2_bf16(v[8 * q + 6], v[8 * q + 7]));
      } else if (sec > 0 && row_ok && rr.kv_row >= 0) {
        __nv_bfloat16* base = (sec == 1) ? ep.kcache : ep.vcache;
        uint4* dst = reinterpret_cast<uint4*>(base + (rr.kv_row + (long long)h * ep.t_max) * ARCB_HEAD_DIM + half * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          dst[q] = make_uint4(pack2_bf16(v[8 * q], v[8 * q + 1]), pack2_bf16(v[8 * q + 2], v[8 * q + 3]),
                              pack2_bf16(v[8 * q + 4], v[8 * q + 5]), pack2_bf16(v[8 * q + 6], v[8 * q + 7]));
      }
      if (staged) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(my_row + (((half * 4 + q) ^ sw) << 4)) =
              make_uint4(pack2_act_chk(v[8 * q], v[8 * q + 1], ep.act_f16, ep.err), pack2_act_chk(v[8 * q + 2], v[8 * q + 3], ep.act_f16, ep.err),
                         pack2_act_chk(v[8 * q + 4], v[8 * q + 5], ep.act_f16, ep.err), pack2_act_chk(v[8 * q + 6], v[8 * q + 7], ep.act_f16, ep.err));
      } else if (sec > 0 && row_ok && rr.row16 >= 0) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>((sec == 1) ? ep.k16 : ep.v16) +
                                              (size_t)rr.row16 * d + c + half * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          dst[q] = make_uint4(pack2_act_chk(v[8 * q], v[8 * q + 1], ep.act_f16, ep.err), pack2_act_chk(v[8 * q + 2], v[8 * q + 3], ep.act_f16, ep.err),
                              pack2_act_chk(v[8 * q + 4], v[8 * q + 5], ep.act_f16, ep.err), pack2_act_chk(v[8 * q + 6], v[8 * q + 7], ep.act_f16, ep.err));
      }
    }
    if (cbox) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(sec == 1 ? tmap_kc : tmap_vc, cbox_smem, 0, (int)(cbox_row0 + (long long)h * ep.t_max));
        bulk_commit_group();
      }
    }
    if (staged) {
      fence_proxy_async_smem();
      named_bar_sync(1 + grp, 128);
      const int limit = (sec == 0) ? ep.M : ep.kv16_rows;
      if (elected && m0 < limit) {
        tma_store_2d(sec == 0 ? tmap_q : (sec == 1 ? tmap_k : tmap_v), stage_smem, c, m0);
        bulk_commit_group();
      }
    }
  }
}

// Drains one accumulator tile (this thread's row, the 32-column chunks of its column half) from
// TMEM through the epilogue MODE.  t_row: TMEM address of the row's first accumulator column;
// n_tile0: first output column of the tile.  tcgen05.ld is warp-collective, so every lane runs the
// loads and only the stores are predicated on row_ok.
template <int BN, int MODE>
__device__ __forceinline__ void epilogue_tile(const GemmEpilogue& ep, uint32_t t_row, int m, bool row_ok,
                                              int n_tile0, int col_half) {
  RopeRow rr;
  rr.x = rr.y = rr.z = 0;
  rr.kv_row = -1;
  rr.row16 = -1;
  if (MODE == EPI_QKV_ROPE && row_ok) rr = rope_row_ctx(ep, m);
  if constexpr (MODE == EPI_SWIGLU) {
    // gate columns [0,64) and up columns [64,128) of every 128-column group
    // BN = 256: each column half owns one 128-column group; BN = 128: one 32-column pair each
    const int g_begin = (BN == 256) ? col_half * 128 : 0, g_end = (BN == 256) ? g_begin + 128 : 128;
    const int c_begin = (BN == 256) ? 0 : col_half, c_end = (BN == 256) ? 2 : col_half + 1;
#pragma unroll 1
    for (int g0 = g_begin; g0 < g_end; g0 += 128) {
      if (n_tile0 + g0 >= ep.N) break;  // warp-uniform: tile tail beyond N
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t rg[32], ru[32];
        tmem_ld_32x32(t_row + g0 + c * 32, rg);
        tmem_ld_32x32(t_row + g0 + 64 + c * 32, ru);
        tmem_wait_ld();
        if (row_ok) {
          const int n0 = n_tile0 + g0 + c * 32;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 g = make_float4(__uint_as_float(rg[4 * q]), __uint_as_float(rg[4 * q + 1]),
                                         __uint_as_float(rg[4 * q + 2]), __uint_as_float(rg[4 * q + 3]));
            const float4 u = make_float4(__uint_as_float(ru[4 * q]), __uint_as_float(ru[4 * q + 1]),
                                         __uint_as_float(ru[4 * q + 2]), __uint_as_float(ru[4 * q + 3]));
            epi_swiglu_quad(ep, m, n0 + 4 * q, g, u);
          }
        }
      }
    }
  } else {
#pragma unroll 1
    for (int c = col_half * (BN / 64); c < (col_half + 1) * (BN / 64); ++c) {
      const int n0 = n_tile0 + c * 32;
      if (n0 >= ep.N) break;  // warp-uniform
      uint32_t r[32];
      tmem_ld_32x32(t_row + c * 32, r);
      tmem_wait_ld();
      if (row_ok) {
        if constexpr (MODE == EPI_QKV_ROPE) {
          epi_qkv_chunk32(ep, rr, m, n0, r);
        } else {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                         __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
            const int n = n0 + 4 * q;
            if constexpr (MODE == EPI_RESID) epi_resid_quad(ep, m, n, v);
            else epi_store_quad(ep, m, n, v);
          }
        }
      }
    }
  }
}

// Persistent kernel: CTA c processes output tiles c, c + gridDim.x, ... (n fastest, so the CTAs
// running at the same time share A rows through L2).  The TMA->MMA shared-memory ring runs
// continuously across tiles; accumulators alternate between two TMEM buffers.
template <int BN, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
               const __grid_constant__ CUtensorMap tmap_z, GemmEpilogue ep, int K, uint32_t idesc, int tiles_n,
               int tiles_total) {
  using Cfg = TcCfg<BN>;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  // operand stages | residual staging (EPI_RESID only) | barriers
  constexpr int RING_BYTES = Cfg::STAGES * Cfg::STAGE_BYTES;
  const uint32_t bar_base = base + RING_BYTES + epi_stage_bytes<MODE>();
  // full[s] at +8s, empty[s] at +8(STAGES+s), acc_full[2], acc_empty[2] after them
  const uint32_t bar_acc_full = bar_base + 16 * Cfg::STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      base_ptr + RING_BYTES + epi_stage_bytes<MODE>() + 16 * Cfg::STAGES + 32);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = K / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (Cfg::STAGES + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 32 * TC_EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (epi_staged<BN, MODE>()) tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // everything above touched only shared / tensor memory and the kernel's own parameters

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      uint32_t kbt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tiles_total; tile += gridDim.x) {
        const int m_blk = tile / tiles_n, n_blk = tile - m_blk * tiles_n;
        for (int kb = 0; kb < num_k; ++kb, ++kbt) {
          const int s = kbt % Cfg::STAGES;
          const uint32_t ph = (kbt / Cfg::STAGES) & 1;
          if (!mbar_wait_bounded(bar_base + 8 * (Cfg::STAGES + s), ph ^ 1)) {
            arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_MMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (*abort_flag) { ok = false; break; }
          const uint32_t full = bar_base + 8 * s;
          const uint32_t a_dst = base + s * Cfg::STAGE_BYTES;
          mbar_expect_tx(full, Cfg::STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, kb * TC_BK, m_blk * TC_BM, full);
          tma_load_2d(a_dst + Cfg::A_BYTES, &tmap_b, kb * TC_BK, n_blk * BN, full);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      uint32_t kbt = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tiles_total; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1;
        // wait until the epilogue has drained this accumulator (two tiles ago)
        if (!mbar_wait_bounded(bar_acc_empty + 8 * acc, ((it >> 1) & 1) ^ 1)) {
          arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb, ++kbt) {
          const int s = kbt % Cfg::STAGES;
          const uint32_t ph = (kbt / Cfg::STAGES) & 1;
          if (!mbar_wait_bounded(bar_base + 8 * s, ph)) {
            arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = base + s * Cfg::STAGE_BYTES;
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + Cfg::A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
            // +32 bytes per K step of 16 elements -> +2 in the (addr >> 4) field
            umma_f16(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) ? 1u : 0u);
          }
          umma_commit(bar_base + 8 * (Cfg::STAGES + s));  // frees the stage when the MMAs retire
        }
        if (ok) umma_commit(bar_acc_full + 8 * acc);
      }
    }
  } else {
    // ---- epilogue: warps 2..9, TMEM lane quarter = warp % 4, column half = (warp - 2) / 4 ----
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < tiles_total; tile += gridDim.x, ++it) {
      const int m_blk = tile / tiles_n, n_blk = tile - m_blk * tiles_n;
      const uint32_t acc = it & 1;
      const int m = m_blk * TC_BM + row_in_tile;
      const bool row_ok = m < ep.M;
      bool ok = mbar_wait_bounded(bar_acc_full + 8 * acc, (it >> 1) & 1);
      if (!ok) arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
      // the four warps of a group share named barriers below, so they must leave together
      if constexpr (epi_staged<BN, MODE>()) ok = !named_bar_or(1 + col_half, 128, !ok);
      else ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      if constexpr (MODE == EPI_RESID)
        epilogue_resid_tma<BN>(ep, &tmap_x, t_row, m_blk * TC_BM, n_blk * BN, col_half, row_in_tile,
                               base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES,
                               base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES, quarter == 0 && lane == 0);
      else if constexpr (MODE == EPI_SWIGLU && BN == 256)
        epilogue_swiglu_tma(ep, &tmap_x, t_row + col_half * 128, m_blk * TC_BM, n_blk * BN + col_half * 128, col_half,
                            row_in_tile, base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES,
                            base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES, quarter == 0 && lane == 0);
      else if constexpr (MODE == EPI_QKV_ROPE && BN == 256) {
        RopeRow rr;
        rr.x = rr.y = rr.z = 0; rr.kv_row = -1; rr.row16 = -1;
        if (row_ok) rr = rope_row_ctx(ep, m);
        epilogue_qkv_tma(ep, rr, &tmap_x, &tmap_y, &tmap_z, t_row + col_half * 128, m_blk * TC_BM, row_ok,
                         n_blk * BN + col_half * 128, col_half, row_in_tile,
                         base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES,
                         base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES, quarter == 0 && lane == 0);
      }
      else
        epilogue_tile<BN, MODE>(ep, t_row, m, row_ok, n_blk * BN, col_half);
      // accumulator drained: hand it back to the MMA warp
      tc_fence_before();
      mbar_arrive(bar_acc_empty + 8 * acc);
    }
    if (epi_staged<BN, MODE>() && quarter == 0 && lane == 0) bulk_wait_all();  // bulk writes done before the CTA exits
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// 2-CTA tcgen05 kernel (cta_group::2): a cluster of two CTAs owns one 256 x 256 output tile.
// CTA r of the pair loads its 128 rows of A and its 128 rows of W (each operand slice crosses
// L2 -> shared memory once per pair, no multicast), CTA 0 issues one 256 x 256 x 16 MMA that reads
// both CTAs' shared memory and writes 128 x 256 accumulators into each CTA's TMEM, and every CTA
// runs the epilogue of its own 128 rows.  Per SM this halves the shared-memory traffic per FLOP
// of the 1-CTA 128 x 256 tile, which is what bounds that kernel.
// Barriers: full[s] lives in CTA 0 (both CTAs' TMA loads complete on it); empty[s] and acc_full[b]
// are signalled in both CTAs by a multicast commit; acc_empty[b] of CTA 0 collects one arrival
// per epilogue warp of both CTAs.
// ---------------------------------------------------------------------------
// The QKV instantiation gives one operand stage to eight 32 x 64 bf16 boxes (one per epilogue warp)
// through which runs of consecutive cache rows are written as bulk tensor stores.
template <int MODE>
struct Tc2Cfg {
  static constexpr int BN = 256;
  static constexpr int STAGES = (MODE == EPI_QKV_ROPE) ? 5 : 6;
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;   // this CTA's 128 rows of A
  static constexpr int B_BYTES = 128 * TC_BK * 2;     // this CTA's 128 rows of W
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int CBOX_BYTES = (MODE == EPI_QKV_ROPE) ? TC_EPI_WARPS * 32 * 128 : 0;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CBOX_BYTES + 1024 + 256;
};

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                const __grid_constant__ CUtensorMap tmap_z, const __grid_constant__ CUtensorMap tmap_kc,
                const __grid_constant__ CUtensorMap tmap_vc, GemmEpilogue ep, int K, uint32_t idesc, int tiles_n,
                int tiles_total, int cache_boxes) {
  using Cfg = Tc2Cfg<MODE>;
  constexpr int BN = Cfg::BN;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  // operand stages | residual staging (EPI_RESID only) | barriers; the same offsets in both CTAs
  constexpr int RING_BYTES = Cfg::STAGES * Cfg::STAGE_BYTES;
  constexpr int CBOX_OFF = RING_BYTES + epi_stage_bytes<MODE>();
  const uint32_t bar_base = base + CBOX_OFF + Cfg::CBOX_BYTES;
  const uint32_t bar_acc_full = bar_base + 16 * Cfg::STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      base_ptr + CBOX_OFF + Cfg::CBOX_BYTES + 16 * Cfg::STAGES + 32);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_k = K / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(bar_base + 8 * s, 1);                   // full: one expect_tx arrival (CTA 0's producer)
      mbar_init(bar_base + 8 * (Cfg::STAGES + s), 1);   // empty: one multicast commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 2 * TC_EPI_WARPS);  // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (epi_staged<256, MODE>()) tma_prefetch_desc(&tmap_x);
    if (MODE == EPI_QKV_ROPE && cache_boxes) {
      tma_prefetch_desc(&tmap_kc);
      tma_prefetch_desc(&tmap_vc);
    }
  }
  if (warp == 1) {
    tmem_alloc_2cta(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrive / TMA completion
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // everything above touched only shared / tensor memory and the kernel's own parameters

  if (warp == 0) {
    // ---- TMA producer (both CTAs) ----
    if (lane == 0) {
      uint32_t kbt = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles_total; tile += n_pairs) {
        const int m_blk = tile / tiles_n, n_blk = tile - m_blk * tiles_n;
        for (int kb = 0; kb < num_k; ++kb, ++kbt) {
          const int s = kbt % Cfg::STAGES;
          const uint32_t ph = (kbt / Cfg::STAGES) & 1;
          if (!mbar_wait_bounded(bar_base + 8 * (Cfg::STAGES + s), ph ^ 1)) {
            arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_MMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (*abort_flag) { ok = false; break; }
          const uint32_t full = bar_base + 8 * s;
          const uint32_t a_dst = base + s * Cfg::STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full, 2 * Cfg::STAGE_BYTES);  // both CTAs' bytes land on CTA 0's barrier
          tma_load_2d_2cta(a_dst, &tmap_a, kb * TC_BK, m_blk * 256 + (int)rank * 128, full);
          tma_load_2d_2cta(a_dst + Cfg::A_BYTES, &tmap_b, kb * TC_BK, n_blk * BN + (int)rank * 128, full);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (leader CTA only) ----
    if (lane == 0 && rank == 0) {
      uint32_t kbt = 0, it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < tiles_total; tile += n_pairs, ++it) {
        const uint32_t acc = it & 1;
        if (!mbar_wait_bounded(bar_acc_empty + 8 * acc, ((it >> 1) & 1) ^ 1)) {
          arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb, ++kbt) {
          const int s = kbt % Cfg::STAGES;
          const uint32_t ph = (kbt / Cfg::STAGES) & 1;
          if (!mbar_wait_bounded(bar_base + 8 * s, ph)) {
            arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = base + s * Cfg::STAGE_BYTES;
          const uint64_t da = umma_desc_k_sw128(a_addr);
          const uint64_t db = umma_desc_k_sw128(a_addr + Cfg::A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4)
            umma_f16_2cta(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) ? 1u : 0u);
          umma_commit_2cta(bar_base + 8 * (Cfg::STAGES + s));  // frees the stage in both CTAs
        }
        if (ok) umma_commit_2cta(bar_acc_full + 8 * acc);
      }
    }
  } else {
    // ---- epilogue (both CTAs): warps 2..9, TMEM lane quarter = warp % 4, column half = (warp - 2) / 4 ----
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t it = 0;
    for (int tile = pair; tile < tiles_total; tile += n_pairs, ++it) {
      const int m_blk = tile / tiles_n, n_blk = tile - m_blk * tiles_n;
      const uint32_t acc = it & 1;
      const int m = m_blk * 256 + (int)rank * 128 + row_in_tile;
      const bool row_ok = m < ep.M;
      bool ok = mbar_wait_bounded(bar_acc_full + 8 * acc, (it >> 1) & 1);
      if (!ok) arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
      if constexpr (epi_staged<256, MODE>()) ok = !named_bar_or(1 + col_half, 128, !ok);
      else ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      if constexpr (MODE == EPI_RESID)
        epilogue_resid_tma<BN>(ep, &tmap_x, t_row, m_blk * 256 + (int)rank * 128, n_blk * BN, col_half, row_in_tile,
                               base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES,
                               base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES, quarter == 0 && lane == 0);
      else if constexpr (MODE == EPI_SWIGLU)
        epilogue_swiglu_tma(ep, &tmap_x, t_row + col_half * 128, m_blk * 256 + (int)rank * 128,
                            n_blk * BN + col_half * 128, col_half, row_in_tile,
                            base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES,
                            base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES, quarter == 0 && lane == 0);
      else if constexpr (MODE == EPI_QKV_ROPE) {
        RopeRow rr;
        rr.x = rr.y = rr.z = 0; rr.kv_row = -1; rr.row16 = -1;
        if (row_ok) rr = rope_row_ctx(ep, m);
        // this warp's 32 rows are one run of consecutive cache rows: write them as boxes
        const long long row0 = __shfl_sync(0xffffffffu, rr.kv_row, 0);
        const bool run = cache_boxes && __all_sync(0xffffffffu, row_ok && rr.kv_row >= 0 && rr.kv_row == row0 + lane);
        const int cbox_off = CBOX_OFF + (warp - 2) * (32 * 128);
        epilogue_qkv_tma(ep, rr, &tmap_x, &tmap_y, &tmap_z, t_row + col_half * 128, m_blk * 256 + (int)rank * 128,
                         row_ok, n_blk * BN + col_half * 128, col_half, row_in_tile,
                         base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES,
                         base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES, quarter == 0 && lane == 0,
                         &tmap_kc, &tmap_vc, base + cbox_off, run ? base_ptr + cbox_off : nullptr, row0);
      }
      else
        epilogue_tile<BN, MODE>(ep, t_row, m, row_ok, n_blk * BN, col_half);
      // accumulator drained by this warp: tell the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cta0(bar_acc_empty + 8 * acc);
    }
    if (epi_staged<256, MODE>() && quarter == 0 && lane == 0) bulk_wait_all();
    else if (MODE == EPI_QKV_ROPE && lane == 0) bulk_wait_all();   // this warp's cache boxes
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the pair's MMAs may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Split-K residual GEMM for few-row launches (the decode step's out-proj and down projections:
// M = sequences in flight, N = d_model).  With 128 x 128 tiles such a launch has fewer tiles than
// SMs (80 for 1024 x 1280) and each CTA streams the whole K extent alone, so the launch is bound by
// one CTA's operand-stream latency.  Here a cluster of two CTAs owns one 128 x BN output tile and
// each CTA accumulates HALF of K in its own tensor memory.  CTA 1 then hands its fp32 partial to CTA 0
// through a small global scratch (written and read with lanes = rows, so every access is a
// contiguous 512 bytes per warp), ordered by a cluster barrier; CTA 0 adds it to its own accumulator
// in a FIXED order (own + partner + bias) and issues the same single bulk reduce-add per element as
// the other kernels.  Every element of x still receives exactly one addend, so the result is
// deterministic (it differs from the unsplit kernel only by fp32 re-association of the K sum).
// BN is chosen so that 2 * tiles <= SM count (160 for d_model 1280: 64 tiles, 128 CTAs).
// ---------------------------------------------------------------------------
template <int BN>
struct SkCfg {
  static constexpr int STAGES = 5;
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 256;
  static constexpr int CHUNKS = BN / 32;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * EPI_STAGE_GROUP_BYTES + 1024 + 256;
};

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_x, GemmEpilogue ep, int K, uint32_t idesc, int tiles_n,
                      float* __restrict__ scratch) {
  using Cfg = SkCfg<BN>;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  constexpr int RING_BYTES = Cfg::STAGES * Cfg::STAGE_BYTES;
  const uint32_t bar_base = base + RING_BYTES + 2 * EPI_STAGE_GROUP_BYTES;
  const uint32_t bar_acc_full = bar_base + 16 * Cfg::STAGES;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(
      base_ptr + RING_BYTES + 2 * EPI_STAGE_GROUP_BYTES + 16 * Cfg::STAGES + 32);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int tile = blockIdx.x >> 1;
  const int m_blk = tile / tiles_n, n_blk = tile - m_blk * tiles_n;
  const int num_k = K / TC_BK;
  const int kb_split = (num_k + 1) / 2;
  const int kb0 = rank ? kb_split : 0, kb1 = rank ? num_k : kb_split;   // this CTA's K blocks

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (Cfg::STAGES + s), 1);
    }
    mbar_init(bar_acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = kb0, i = 0; kb < kb1; ++kb, ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (i / Cfg::STAGES) & 1;
        if (!mbar_wait_bounded(bar_base + 8 * (Cfg::STAGES + s), ph ^ 1)) {
          arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_MMA);
          *abort_flag = 1;
          break;
        }
        if (*abort_flag) break;
        const uint32_t full = bar_base + 8 * s;
        const uint32_t a_dst = base + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(full, Cfg::STAGE_BYTES);
        tma_load_2d(a_dst, &tmap_a, kb * TC_BK, m_blk * TC_BM, full);
        tma_load_2d(a_dst + Cfg::A_BYTES, &tmap_b, kb * TC_BK, n_blk * BN, full);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = kb0, i = 0; kb < kb1; ++kb, ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (i / Cfg::STAGES) & 1;
        if (!mbar_wait_bounded(bar_base + 8 * s, ph)) {
          arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_TMA);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = base + s * Cfg::STAGE_BYTES;
        const uint64_t da = umma_desc_k_sw128(a_addr);
        const uint64_t db = umma_desc_k_sw128(a_addr + Cfg::A_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < TC_BK / 16; ++k4) umma_f16(tmem_base, da + 2 * k4, db + 2 * k4, idesc, (i | k4) ? 1u : 0u);
        umma_commit(bar_base + 8 * (Cfg::STAGES + s));
      }
      if (ok) umma_commit(bar_acc_full);
    }
  }
  // ---- epilogue warps 2..9: lane quarter = warp % 4, chunk set by (warp - 2) / 4 ----
  const int quarter = warp & 3;
  const int col_half = (warp - 2) >> 2;
  const int row_in_tile = quarter * 32 + lane;
  constexpr int C_SPLIT = (Cfg::CHUNKS + 1) / 2;   // chunks [0, C_SPLIT) to half 0, the rest to half 1
  const int c_begin = col_half ? C_SPLIT : 0, c_end = col_half ? Cfg::CHUNKS : C_SPLIT;
  // partial tile in the scratch: [tile][chunk][float4 column q][row] -> lanes (rows) are contiguous
  float4* part = reinterpret_cast<float4*>(scratch) + (size_t)tile * (BN / 4) * TC_BM;
  bool ok = true;
  if (warp >= 2) {
    ok = mbar_wait_bounded(bar_acc_full, 0);
    if (!ok) arcb_set_error(ep.err, ARCB_DEV_WAIT_TIMEOUT_ACC);
    tc_fence_after();
    if (rank == 1 && ok) {
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 8; ++q)
          part[(size_t)(c * 8 + q) * TC_BM + row_in_tile] =
              make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                          __uint_as_float(r[4 * q + 3]));
      }
    }
  }
  // CTA 1's partial is in global memory before CTA 0 reads it (release / acquire at cluster scope)
  cluster_sync_all();
  if (warp >= 2 && rank == 0) {
    // the four warps of a group share named barriers below, so they must leave together
    ok = !named_bar_or(1 + col_half, 128, !ok);
    if (ok) {
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
      uint8_t* stage_ptr = base_ptr + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES;
      const uint32_t stage_smem = base + RING_BYTES + col_half * EPI_STAGE_GROUP_BYTES;
      uint8_t* my_row = stage_ptr + row_in_tile * 128;
      const int sw = row_in_tile & 7;
      const bool elected = quarter == 0 && lane == 0;
      const int m0 = m_blk * TC_BM;
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        const int n0 = n_blk * BN + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        float4 pv[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) pv[q] = part[(size_t)(c * 8 + q) * TC_BM + row_in_tile];
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float4 v = make_float4(__uint_as_float(r[4 * q]) + pv[q].x, __uint_as_float(r[4 * q + 1]) + pv[q].y,
                                 __uint_as_float(r[4 * q + 2]) + pv[q].z, __uint_as_float(r[4 * q + 3]) + pv[q].w);
          if (ep.bias) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(ep.bias + n0 + 4 * q));
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
          }
          pv[q] = v;
        }
        if (elected) bulk_wait_read_all();        // the previous reduce has read the buffer
        named_bar_sync(1 + col_half, 128);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(my_row + ((q ^ sw) << 4)) = pv[q];
        fence_proxy_async_smem();
        named_bar_sync(1 + col_half, 128);
        if (elected && m0 < ep.M) {
          tma_reduce_add_2d(&tmap_x, stage_smem, n0, m0);
          bulk_commit_group();
        }
      }
      if (elected) bulk_wait_all();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// CUDA-core kernel: 32 x 128 x 32 tiles, 256 threads, each thread 2 rows x (4 + 4) columns
// (columns c..c+3 and c+64..c+67 so that the SwiGLU partner columns meet in one thread).
// ---------------------------------------------------------------------------
constexpr int SM_BM = 32, SM_BN = 128, SM_BK = 32;

template <int MODE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ W, GemmEpilogue ep,
                 int K, int a_f16) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[SM_BK][SM_BM + 1];
  __shared__ __align__(16) float Ws[SM_BK][SM_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * SM_BM, n0 = blockIdx.x * SM_BN;
  float acc[2][8];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  const int a_row = tid >> 3, a_kq = (tid & 7) * 4;
  const int w_n = tid >> 1, w_kh = (tid & 1) * 16;
  for (int k0 = 0; k0 < K; k0 += SM_BK) {
    {
      uint2 raw = make_uint2(0u, 0u);
      if (m0 + a_row < ep.M)
        raw = *reinterpret_cast<const uint2*>(A + (size_t)(m0 + a_row) * K + k0 + a_kq);
      const float2 f0 = unpack2_act(raw.x, a_f16), f1 = unpack2_act(raw.y, a_f16);
      As[a_kq + 0][a_row] = f0.x;
      As[a_kq + 1][a_row] = f0.y;
      As[a_kq + 2][a_row] = f1.x;
      As[a_kq + 3][a_row] = f1.y;
    }
    {
      const uint4* src = reinterpret_cast<const uint4*>(W + (size_t)(n0 + w_n) * K + k0 + w_kh);
      const uint4 r0 = __ldg(src), r1 = __ldg(src + 1);
      const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = unpack2_act(w[j], a_f16);
        Ws[w_kh + 2 * j][w_n] = f.x;
        Ws[w_kh + 2 * j + 1][w_n] = f.y;
      }
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < SM_BK; ++k) {
      const float a0 = As[k][2 * ty], a1 = As[k][2 * ty + 1];
      const float4 wl = *reinterpret_cast<const float4*>(&Ws[k][4 * tx]);
      const float4 wh = *reinterpret_cast<const float4*>(&Ws[k][64 + 4 * tx]);
      acc[0][0] += a0 * wl.x; acc[0][1] += a0 * wl.y; acc[0][2] += a0 * wl.z; acc[0][3] += a0 * wl.w;
      acc[0][4] += a0 * wh.x; acc[0][5] += a0 * wh.y; acc[0][6] += a0 * wh.z; acc[0][7] += a0 * wh.w;
      acc[1][0] += a1 * wl.x; acc[1][1] += a1 * wl.y; acc[1][2] += a1 * wl.z; acc[1][3] += a1 * wl.w;
      acc[1][4] += a1 * wh.x; acc[1][5] += a1 * wh.y; acc[1][6] += a1 * wh.z; acc[1][7] += a1 * wh.w;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + 2 * ty + i;
    if (m >= ep.M) continue;
    const float4 lo = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    const float4 hi = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    const int n = n0 + 4 * tx;
    if constexpr (MODE == EPI_SWIGLU) {
      epi_swiglu_quad(ep, m, n, lo, hi);
    } else if constexpr (MODE == EPI_QKV_ROPE) {
      const RopeRow rr = rope_row_ctx(ep, m);
      epi_qkv_quad(ep, rr, m, n, lo);
      epi_qkv_quad(ep, rr, m, n + 64, hi);
    } else if constexpr (MODE == EPI_RESID) {
      epi_resid_quad(ep, m, n, lo);
      epi_resid_quad(ep, m, n + 64, hi);
    } else {
      epi_store_quad(ep, m, n, lo);
      epi_store_quad(ep, m, n + 64, hi);
    }
  }
}

// ---- host: tensor maps -------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn lookup_encode_fn() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    return reinterpret_cast<EncodeTiledFn>(p);
  return nullptr;
}

EncodeTiledFn get_encode_fn() {
  static const EncodeTiledFn fn = lookup_encode_fn();   // initialised once, thread-safe
  return fn;
}

}  // namespace

int arcb_make_tmap_2d_16b(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                          uint32_t box_rows, uint32_t box_cols, int is_f16) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -100;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

// fp32 [rows][cols] tensor with 128 x 32 boxes (128-byte rows, 128-byte swizzle): the residual stream
static int make_tmap_resid_f32(CUtensorMap* out, float* ptr, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -100;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * 4};
  cuuint32_t box[2] = {32, 128};
  cuuint32_t estr[2] = {1, 1};
  return (int)fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, gdim, gstride, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

bool arcb_gemm_tc_supported(int M, int N, int K) {
  (void)M;
  return (N % 128 == 0) && (K % 64 == 0) && K >= 64;
}

template <int MODE>
static cudaError_t set_tc_smem_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<128, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       TcCfg<128>::SMEM_BYTES + epi_stage_bytes<MODE>());
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gemm_tc_kernel<256, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              TcCfg<256>::SMEM_BYTES + epi_stage_bytes<MODE>());
}

// Per-device launch limits, filled by arcb_gemm_init() for the device that is current then and
// read for the device that is current at launch (a process may drive several GPUs).
constexpr int MAX_DEVICES = 64;
static int g_num_sms[MAX_DEVICES] = {0};
static int g_max_pairs[MAX_DEVICES] = {0};  // 2-CTA clusters that can be resident at once

static int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
  return dev;
}
static int num_sms() { const int n = g_num_sms[current_device_slot()]; return n > 0 ? n : 148; }
static int max_pairs() { return g_max_pairs[current_device_slot()]; }

template <int MODE>
static cudaError_t set_tc2_smem_attr() {
  return cudaFuncSetAttribute(gemm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              Tc2Cfg<MODE>::SMEM_BYTES + epi_stage_bytes<MODE>());
}

// Opt in to the large dynamic shared memory of every tcgen05 instantiation (call once, outside
// any stream capture).
int arcb_gemm_init() {
  cudaError_t e;
  if ((e = set_tc_smem_attr<EPI_STORE_F32>()) != cudaSuccess) return (int)e;
  if ((e = set_tc_smem_attr<EPI_QKV_ROPE>()) != cudaSuccess) return (int)e;
  if ((e = set_tc_smem_attr<EPI_RESID>()) != cudaSuccess) return (int)e;
  if ((e = set_tc_smem_attr<EPI_SWIGLU>()) != cudaSuccess) return (int)e;
  if ((e = set_tc2_smem_attr<EPI_STORE_F32>()) != cudaSuccess) return (int)e;
  if ((e = set_tc2_smem_attr<EPI_QKV_ROPE>()) != cudaSuccess) return (int)e;
  if ((e = set_tc2_smem_attr<EPI_RESID>()) != cudaSuccess) return (int)e;
  if ((e = set_tc2_smem_attr<EPI_SWIGLU>()) != cudaSuccess) return (int)e;
  if ((e = cudaFuncSetAttribute(gemm_tc_splitk_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                SkCfg<128>::SMEM_BYTES)) != cudaSuccess) return (int)e;
  if ((e = cudaFuncSetAttribute(gemm_tc_splitk_kernel<160>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                SkCfg<160>::SMEM_BYTES)) != cudaSuccess) return (int)e;
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 148);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = Tc2Cfg<EPI_RESID>::SMEM_BYTES + epi_stage_bytes<EPI_RESID>();
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<EPI_RESID>, &cfg) == cudaSuccess)
      g_max_pairs[current_device_slot()] = n;
    else cudaGetLastError();
  }
  int dev = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
  int sms = 0;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
  if (dev >= 0 && dev < MAX_DEVICES) g_num_sms[dev] = sms;
  return get_encode_fn() ? 0 : -100;
}

template <int BN, int MODE>
static cudaError_t launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tx, const CUtensorMap& ty,
                      const CUtensorMap& tz, const GemmEpilogue& ep, int K, int act_f16, cudaStream_t stream) {
  const int tiles_n = (ep.N + BN - 1) / BN, tiles_m = (ep.M + TC_BM - 1) / TC_BM;
  const int tiles = tiles_n * tiles_m;
  const int sms = num_sms();
  const uint32_t idesc = umma_idesc_f16(TC_BM, BN, act_f16 ? 0 : 1, act_f16 ? 0 : 1);
  return arcb_launch(gemm_tc_kernel<BN, MODE>, dim3(tiles < sms ? tiles : sms), dim3(TC_THREADS),
                     TcCfg<BN>::SMEM_BYTES + epi_stage_bytes<MODE>(), stream, ta, tb, tx, ty, tz, ep, K, idesc, tiles_n,
                     tiles);
}

template <int MODE>
static cudaError_t launch_tc2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tx, const CUtensorMap& ty,
                       const CUtensorMap& tz, const CUtensorMap& tkc, const CUtensorMap& tvc, int cache_boxes,
                       const GemmEpilogue& ep, int K, int act_f16, cudaStream_t stream) {
  const int tiles_n = (ep.N + 255) / 256, tiles_m = (ep.M + 255) / 256;
  const int tiles = tiles_n * tiles_m;
  const int mp = max_pairs();
  const int pairs = tiles < mp ? tiles : mp;
  const uint32_t idesc = umma_idesc_f16(256, 256, act_f16 ? 0 : 1, act_f16 ? 0 : 1);
  return arcb_launch(gemm_tc2_kernel<MODE>, dim3(2 * pairs), dim3(TC_THREADS),
                     Tc2Cfg<MODE>::SMEM_BYTES + epi_stage_bytes<MODE>(), stream, ta, tb, tx, ty, tz, tkc, tvc, ep, K, idesc,
                     tiles_n, tiles, cache_boxes);
}

int arcb_gemm_max_pairs() { return max_pairs(); }

// Column tile of the split-K residual kernel for an M x N x K launch, or 0 when it does not apply:
// the launch must leave most SMs without a 128 x 128 tile, K must be long enough to be worth
// halving, and 2 * tiles must fit in one wave of CTA pairs.
int arcb_gemm_splitk_bn(int M, int N, int K) {
  static const bool enabled = [] { const char* e = getenv("ARCB_SPLITK"); return !(e && e[0] == '0'); }();  // A/B switch
  if (!enabled) return 0;
  const int sms = num_sms(), mp = max_pairs();
  if (mp <= 0 || K < 1024 || K % TC_BK != 0) return 0;
  const int tiles_m = (M + TC_BM - 1) / TC_BM;
  if (tiles_m * ((N + 127) / 128) * 10 >= sms * 7) return 0;   // the plain kernel already fills the machine
  int best = 0, best_tiles = 0;
  const int cand[2] = {160, 128};
  for (int bn : cand) {
    if (N % bn) continue;
    const int tiles = tiles_m * (N / bn);
    if (tiles <= mp && 2 * tiles <= sms && tiles > best_tiles) { best = bn; best_tiles = tiles; }
  }
  return best;
}

template <int BN>
static cudaError_t launch_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tx, const GemmEpilogue& ep,
                                 int K, int act_f16, cudaStream_t stream) {
  const int tiles_n = ep.N / BN, tiles_m = (ep.M + TC_BM - 1) / TC_BM;
  const uint32_t idesc = umma_idesc_f16(TC_BM, BN, act_f16 ? 0 : 1, act_f16 ? 0 : 1);
  return arcb_launch(gemm_tc_splitk_kernel<BN>, dim3(2 * tiles_n * tiles_m), dim3(TC_THREADS), SkCfg<BN>::SMEM_BYTES,
                     stream, ta, tb, tx, ep, K, idesc, tiles_n, ep.splitk_scratch);
}

template <int MODE>
static int launch_gemm_mode(const void* a16, const void* w16, const GemmEpilogue& ep, int K,
                            int act_f16, bool use_tc, int tc_variant, cudaStream_t stream) {
  const int M = ep.M, N = ep.N;
  if (use_tc) {
    // 128 x 256 tiles (one CTA per SM, persistent) unless that leaves most SMs without a tile
    const int sms = num_sms();
    const int tiles256 = ((N + 255) / 256) * ((M + TC_BM - 1) / TC_BM);
    // the QKV epilogue of the 256-column kernels needs tiles that stay inside one of the q / k / v sections
    const bool allow256 = !(MODE == EPI_QKV_ROPE && ep.d_model % 256 != 0);
    const bool wide = allow256 && tiles256 * 10 >= sms * 7;
    // 256 x 256 tiles on CTA pairs when there are enough of them to occupy the machine
    const int tiles2 = ((N + 255) / 256) * ((M + 255) / 256);
    const int mp = max_pairs();
    const bool pair = allow256 && mp > 0 && (tc_variant == 2 || (tc_variant == 0 && tiles2 * 10 >= mp * 7));
    CUtensorMap ta, tb;
    int r = arcb_make_tmap_2d_16b(&ta, a16, (uint64_t)M, (uint64_t)K, TC_BM, TC_BK, act_f16);
    if (r) return 1000 + r;
    if (MODE == EPI_RESID && ep.splitk_scratch && tc_variant == 0) {
      const int bn = arcb_gemm_splitk_bn(M, N, K);
      if (bn) {
        r = arcb_make_tmap_2d_16b(&tb, w16, (uint64_t)N, (uint64_t)K, bn, TC_BK, act_f16);
        if (r) return 1000 + r;
        CUtensorMap txr;
        r = make_tmap_resid_f32(&txr, ep.x, (uint64_t)M, (uint64_t)N);
        if (r) return 1000 + r;
        const cudaError_t le = bn == 160 ? launch_splitk<160>(ta, tb, txr, ep, K, act_f16, stream)
                                         : launch_splitk<128>(ta, tb, txr, ep, K, act_f16, stream);
        arcb_count_launch(1);
        return (int)le;
      }
    }
    r = arcb_make_tmap_2d_16b(&tb, w16, (uint64_t)N, (uint64_t)K, (wide && !pair) ? 256 : 128, TC_BK, act_f16);
    if (r) return 1000 + r;
    CUtensorMap tx = ta;  // only the residual epilogue reads it
    if (MODE == EPI_RESID) {
      r = make_tmap_resid_f32(&tx, ep.x, (uint64_t)M, (uint64_t)N);
      if (r) return 1000 + r;
    } else if (MODE == EPI_SWIGLU && (pair || wide)) {
      // h16 [M][N / 2], 128 x 64 boxes (one accumulator group's outputs)
      r = arcb_make_tmap_2d_16b(&tx, ep.out16, (uint64_t)M, (uint64_t)(N / 2), 128, 64, act_f16);
      if (r) return 1000 + r;
    }
    CUtensorMap ty = ta, tz = ta;
    if (MODE == EPI_QKV_ROPE && (pair || wide)) {
      // q16 [M][d] and, when its rows are the packed rows, the K / V scratch [kv16_rows][d]: 128 x 64 boxes
      r = arcb_make_tmap_2d_16b(&tx, ep.out16, (uint64_t)M, (uint64_t)ep.d_model, 128, 64, act_f16);
      if (r) return 1000 + r;
      if (ep.k16 && ep.kv16_identity && ep.kv16_rows > 0) {
        r = arcb_make_tmap_2d_16b(&ty, ep.k16, (uint64_t)ep.kv16_rows, (uint64_t)ep.d_model, 128, 64, act_f16);
        if (r) return 1000 + r;
        r = arcb_make_tmap_2d_16b(&tz, ep.v16, (uint64_t)ep.kv16_rows, (uint64_t)ep.d_model, 128, 64, act_f16);
        if (r) return 1000 + r;
      }
    }
    // K / V cache of this layer as [n_seqs * n_heads * t_max][64] bf16, 32-row boxes: prompt runs are
    // written through them (only when several rows of a launch can share a sequence)
    CUtensorMap tkc = ta, tvc = ta;
    int cache_boxes = 0;
    if (MODE == EPI_QKV_ROPE && pair && ep.seq != nullptr && ep.kcache && ep.vcache) {
      static const bool boxes_on = [] { const char* e = getenv("ARCB_CACHE_BOXES"); return !(e && e[0] == '0'); }();  // A/B switch
      const unsigned long long rows = (unsigned long long)ep.n_seqs * ep.n_heads * ep.t_max;
      if (boxes_on && rows < (1ull << 31)) {
        r = arcb_make_tmap_2d_16b(&tkc, ep.kcache, rows, 64, 32, 64, 0);
        if (r) return 1000 + r;
        r = arcb_make_tmap_2d_16b(&tvc, ep.vcache, rows, 64, 32, 64, 0);
        if (r) return 1000 + r;
        cache_boxes = 1;
      }
    }
    cudaError_t le;
    if (pair) le = launch_tc2<MODE>(ta, tb, tx, ty, tz, tkc, tvc, cache_boxes, ep, K, act_f16, stream);
    else if (wide) le = launch_tc<256, MODE>(ta, tb, tx, ty, tz, ep, K, act_f16, stream);
    else le = launch_tc<128, MODE>(ta, tb, tx, ty, tz, ep, K, act_f16, stream);
    arcb_count_launch(1);
    return (int)le;
  }
  dim3 grid(N / SM_BN, (M + SM_BM - 1) / SM_BM);
  const cudaError_t le = arcb_launch(gemm_simt_kernel<MODE>, grid, dim3(256), 0, stream,
                                     reinterpret_cast<const uint16_t*>(a16), reinterpret_cast<const uint16_t*>(w16), ep,
                                     K, act_f16);
  arcb_count_launch(1);
  return (int)le;
}

int arcb_launch_gemm(const void* a16, const void* w16, const GemmEpilogue& ep, int K, int act_f16,
                     bool use_tc, cudaStream_t stream, int tc_variant) {
  const int M = ep.M, N = ep.N;
  if (M <= 0) return 0;
  if (N % 128 != 0 || K % 32 != 0) return -1;
  if (use_tc && !arcb_gemm_tc_supported(M, N, K)) return -1;
  switch (ep.mode) {
    case EPI_STORE_F32: return launch_gemm_mode<EPI_STORE_F32>(a16, w16, ep, K, act_f16, use_tc, tc_variant, stream);
    case EPI_QKV_ROPE: return launch_gemm_mode<EPI_QKV_ROPE>(a16, w16, ep, K, act_f16, use_tc, tc_variant, stream);
    case EPI_RESID: return launch_gemm_mode<EPI_RESID>(a16, w16, ep, K, act_f16, use_tc, tc_variant, stream);
    case EPI_SWIGLU: return launch_gemm_mode<EPI_SWIGLU>(a16, w16, ep, K, act_f16, use_tc, tc_variant, stream);
  }
  return -1;
}
