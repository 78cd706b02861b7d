// Augmentation fan-out on the device: prompt construction for every (dihedral x colour
// permutation) variant of a task, and the way back from generated tokens to candidate grids in the
// task's own orientation and colours.  Integer / byte work, bit-exact with the host codec.
//
// Both kernels are bound by HBM traffic that is small next to generation (a prompt token is 28
// bytes of plan arrays, a candidate is 3.7 KB of tokens in and 944 bytes out), so they are written
// for coalesced access and enough CTAs to fill the GPU, nothing more.
#include "../../include/arcb200.h"
#include "common.cuh"

void arcb_set_last_error(const char* msg);
void arcb_count_launch(long long n);

namespace {

constexpr int TOK_START = 10, TOK_NEWLINE = 11, TOK_IO_SEP = 12, TOK_END = 13;
constexpr int MAX_X = 30, MAX_Y = 29;

// Source cell of cell (r, c) of DIHEDRAL_TRANSFORMS[d](G) for an h x w grid G (src/data.py:182-233):
// identity, rot90 (clockwise), rot180, rot270, flip_h, flip_v, transpose, anti-diagonal transpose.
__device__ __forceinline__ int dihedral_src(int d, int r, int c, int h, int w) {
  switch (d) {
    case 0: return r * w + c;
    case 1: return (h - 1 - c) * w + r;
    case 2: return (h - 1 - r) * w + (w - 1 - c);
    case 3: return c * w + (w - 1 - r);
    case 4: return r * w + (w - 1 - c);
    case 5: return (h - 1 - r) * w + c;
    case 6: return c * w + r;
    default: return (h - 1 - c) * w + (w - 1 - r);
  }
}
__device__ __forceinline__ bool dihedral_swaps(int d) { return d == 1 || d == 3 || d == 6 || d == 7; }

constexpr int BUILD_THREADS = 256;

// One CTA per variant.  A prompt is, per train pair, START in-grid IO_SEP out-grid END and then
// START test-in IO_SEP (src/data.py:75-93); a grid is its rows, each followed by NEWLINE.
__global__ void __launch_bounds__(BUILD_THREADS) build_prompts_kernel(arcb_prompt_build_args a) {
  __shared__ int s_start[ARCB_MAX_TEMPLATE_GRIDS + 1];   // first token of each grid's segment
  __shared__ int s_off[ARCB_MAX_TEMPLATE_GRIDS], s_h[ARCB_MAX_TEMPLATE_GRIDS], s_w[ARCB_MAX_TEMPLATE_GRIDS];
  __shared__ unsigned char s_lut[10];
  __shared__ int s_bad;
  for (int v = blockIdx.x; v < a.n_variants; v += gridDim.x) {
    const int tpl = a.d_var_template[v];
    const int g0 = a.d_tpl_off[tpl], n_grids = a.d_tpl_off[tpl + 1] - g0;
    const int d = a.d_var_dihedral[v], perm = a.d_var_perm[v];
    const int base = a.d_var_tok_off[v], want = a.d_var_tok_off[v + 1] - base;
    const bool swap = dihedral_swaps(d);
    __syncthreads();   // previous variant's readers are done with the shared arrays
    if (threadIdx.x == 0) {
      int bad = (n_grids < 1 || n_grids > ARCB_MAX_TEMPLATE_GRIDS || d < 0 || d > 7 || perm < 0 || perm >= a.n_perms);
      int t = 0;
      for (int j = 0; j < n_grids && !bad; ++j) {
        const int g = a.d_tpl_grid[g0 + j];
        const int h = a.d_grid_h[g], w = a.d_grid_w[g];
        s_off[j] = a.d_grid_off[g]; s_h[j] = h; s_w[j] = w;
        const int th = swap ? w : h, tw = swap ? h : w;
        s_start[j] = t;
        // input segment: START + grid + IO_SEP; output segment: grid + END
        t += th * (tw + 1) + ((j & 1) ? 1 : 2);
      }
      s_start[bad ? 0 : n_grids] = t;
      if (!bad && t != want) bad = 1;
      s_bad = bad;
      if (bad && a.d_status) atomicExch(a.d_status, ARCB_DEV_BAD_INDEX);
    }
    if (threadIdx.x < 10) s_lut[threadIdx.x] = a.d_perm_lut[(perm < 0 || perm >= a.n_perms ? 0 : perm) * 10 + threadIdx.x];
    __syncthreads();
    if (s_bad) continue;
    const int seq = a.d_var_seq ? a.d_var_seq[v] : v;
    for (int t = threadIdx.x; t < want; t += BUILD_THREADS) {
      int j = 0;
      while (j + 1 < n_grids && s_start[j + 1] <= t) ++j;
      const int h = s_h[j], w = s_w[j];
      const int tw = swap ? h : w;
      const bool is_out = j & 1;
      const int seg_len = s_start[j + 1] - s_start[j];
      int u = t - s_start[j];
      int tok, x = 0, y = 0, z;
      if (!is_out && u == 0) { tok = TOK_START; z = 0; }
      else if (u == seg_len - 1) { tok = is_out ? TOK_END : TOK_IO_SEP; z = is_out ? 4 : 2; }
      else {
        if (!is_out) --u;
        const int r = u / (tw + 1), c = u - r * (tw + 1);
        z = is_out ? 3 : 1;
        y = min(r, MAX_Y);
        if (c == tw) tok = TOK_NEWLINE;
        else {
          const int cell = a.d_cells[s_off[j] + dihedral_src(d, r, c, h, w)];
          tok = cell < 10 ? s_lut[cell] : cell;
          x = min(c, MAX_X);
        }
      }
      const long long o = (long long)base + t;
      if (a.d_token_ids) a.d_token_ids[o] = tok;
      if (a.d_pos_xyz) { a.d_pos_xyz[o * 3] = x; a.d_pos_xyz[o * 3 + 1] = y; a.d_pos_xyz[o * 3 + 2] = z; }
      if (a.d_seq) a.d_seq[o] = seq;
      if (a.d_kv_slot) a.d_kv_slot[o] = t;
      if (a.d_kv_count) a.d_kv_count[o] = t + 1;
      if (a.d_kv_row) a.d_kv_row[o] = (int)o;
    }
  }
}

constexpr int CAND_THREADS = 128;
constexpr int CAND_PER = 8;   // consecutive tokens per thread: 128 x 8 = 1024 >= ARCB_CANDIDATE_MAX_CELLS

// Block-wide exclusive scans over one value per thread (CAND_THREADS threads); `total` receives the
// reduction over all threads.  s_part: 4 ints of shared scratch (one per warp).
__device__ __forceinline__ int block_excl_sum(int v, int* s_part, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();                     // previous use of s_part is over
  if (lane == 31) s_part[warp] = inc;
  __syncthreads();
  int base = 0;
  total = 0;
#pragma unroll
  for (int w = 0; w < CAND_THREADS / 32; ++w) {
    if (w < warp) base += s_part[w];
    total += s_part[w];
  }
  return base + inc - v;
}
__device__ __forceinline__ int block_excl_max(int v, int* s_part, int& total) {   // identity: -1
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc = max(inc, t);
  }
  int excl = __shfl_up_sync(0xffffffffu, inc, 1);
  if (lane == 0) excl = -1;
  __syncthreads();
  if (lane == 31) s_part[warp] = inc;
  __syncthreads();
  int base = -1;
  total = -1;
#pragma unroll
  for (int w = 0; w < CAND_THREADS / 32; ++w) {
    if (w < warp) base = max(base, s_part[w]);
    total = max(total, s_part[w]);
  }
  return max(base, excl);
}
__device__ __forceinline__ int block_min(int v, int* s_part) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  return min(min(s_part[0], s_part[1]), min(s_part[2], s_part[3]));
}
__device__ __forceinline__ int block_max(int v, int* s_part) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
  __syncthreads();
  return max(max(s_part[0], s_part[1]), max(s_part[2], s_part[3]));
}

// One CTA per generated row.  The grid is read after the last IO_SEP and before the first END
// (src/inference.py:906-915, src/data.py:95-117); rows end at NEWLINE, empty rows are dropped,
// START is ignored (src/data.py:54-72).  Those sequential rules are evaluated with block-wide
// scans over the row's tokens (8 consecutive tokens per thread):
//   P[i]     colour cells before token i             (prefix sum)
//   L[i]     P at the last NEWLINE before i, or -1   (prefix maximum; P never decreases)
//   a NEWLINE at i closes a row iff P[i] > max(L[i], 0); a cell's column is P[i] - max(L[i], 0) and
//   its row the number of closing NEWLINEs before it, so cell i lands at raw[P[i]] and the grid is
//   rectangular iff every closed row (and a trailing unclosed one) has the first row's width.
__global__ void __launch_bounds__(CAND_THREADS) canonicalize_kernel(arcb_candidate_args a) {
  __shared__ int s_tok[CAND_THREADS * CAND_PER];
  __shared__ unsigned char s_raw[ARCB_CANDIDATE_MAX_CELLS];
  __shared__ unsigned char s_inv[10];
  __shared__ int s_part[CAND_THREADS / 32];
  __shared__ int s_same;
  const int row = blockIdx.x;
  if (row >= a.n_rows) return;
  arcb_candidate_record* rec = a.d_records + row;
  const int d = a.d_row_dihedral[row];
  if (d < 0 || d > 7) {  // padding row of an uneven shard
    for (int i = threadIdx.x; i < (int)sizeof(arcb_candidate_record) / 4; i += CAND_THREADS)
      reinterpret_cast<int*>(rec)[i] = 0;
    return;
  }
  const int* toks = a.d_tokens + (long long)row * a.max_new;
  for (int i = threadIdx.x; i < CAND_THREADS * CAND_PER; i += CAND_THREADS)
    s_tok[i] = i < a.max_new ? toks[i] : TOK_END;
  if (threadIdx.x < 10) {
    // inverse of the old -> new colour map
    const int perm = a.d_row_perm ? a.d_row_perm[row] : 0;
    const unsigned char* lut = a.d_perm_lut + (perm < 0 || perm >= a.n_perms ? 0 : perm) * 10;
    s_inv[lut[threadIdx.x] % 10] = (unsigned char)threadIdx.x;
  }
  if (threadIdx.x == 0) s_same = 1;
  __syncthreads();
  const int i0 = threadIdx.x * CAND_PER;
  int tk[CAND_PER];
#pragma unroll
  for (int k = 0; k < CAND_PER; ++k) tk[k] = s_tok[i0 + k];
  // n: tokens before the first END; start: one past the last IO_SEP before it (the prompt ends with
  // IO_SEP, so the grid starts at 0 unless the model emits another)
  int v = a.max_new;
#pragma unroll
  for (int k = CAND_PER - 1; k >= 0; --k) if (tk[k] == TOK_END) v = i0 + k;
  const int n = min(block_min(v, s_part), a.max_new);
  v = -1;
#pragma unroll
  for (int k = 0; k < CAND_PER; ++k) if (i0 + k < n && tk[k] == TOK_IO_SEP) v = i0 + k;
  const int start = block_max(v, s_part) + 1;
  // per-token classes inside [start, n)
  bool is_col[CAND_PER], is_nl[CAND_PER];
  int ncol = 0;
#pragma unroll
  for (int k = 0; k < CAND_PER; ++k) {
    const bool in = i0 + k >= start && i0 + k < n;
    is_col[k] = in && tk[k] >= 0 && tk[k] < 10;
    is_nl[k] = in && tk[k] == TOK_NEWLINE;
    ncol += is_col[k];
  }
  int n_cells;
  int P = block_excl_sum(ncol, s_part, n_cells);      // colours before this thread's first token
  int Pk[CAND_PER];
  int vmax = -1;
#pragma unroll
  for (int k = 0; k < CAND_PER; ++k) {
    Pk[k] = P;
    if (is_nl[k]) vmax = P;                            // P never decreases: the last NEWLINE holds the maximum
    P += is_col[k];
  }
  int last_nl_P;                                       // P at the row's last NEWLINE, or -1
  int L = block_excl_max(vmax, s_part, last_nl_P);
  int neff = 0, jag_w_lo = 1 << 30, jag_w_hi = -1;
  bool eff[CAND_PER];
#pragma unroll
  for (int k = 0; k < CAND_PER; ++k) {
    const int row_start = max(L, 0);
    eff[k] = is_nl[k] && Pk[k] > row_start;
    if (eff[k]) {
      const int w = Pk[k] - row_start;                 // width of the row this NEWLINE closes
      jag_w_lo = min(jag_w_lo, w);
      jag_w_hi = max(jag_w_hi, w);
      ++neff;
    }
    if (is_nl[k]) L = Pk[k];
  }
  int n_closed;
  block_excl_sum(neff, s_part, n_closed);
  const int w_lo = block_min(jag_w_lo, s_part), w_hi = block_max(jag_w_hi, s_part);
  const int trailing = n_cells - max(last_nl_P, 0);   // cells after the last NEWLINE
  int status, h = 0, w = 0;
  if (start >= n) status = 0;
  else {
    h = n_closed + (trailing > 0 ? 1 : 0);
    if (n_closed > 0) w = w_lo; else w = trailing;
    const bool jag = (n_closed > 0 && (w_lo != w_hi || (trailing > 0 && trailing != w_lo)));
    status = (h > 0 && !jag) ? 1 : 2;
    if (status != 1) h = w = 0;
  }
  // cells in row-major order
#pragma unroll
  for (int k = 0; k < CAND_PER; ++k)
    if (is_col[k]) s_raw[Pk[k]] = (unsigned char)tk[k];
  __syncthreads();
  // input-copy flag: the grid as generated against the task's test input (src/voting.py:92)
  int tg = (status == 1 && a.d_row_test_grid) ? a.d_row_test_grid[row] : -1;
  if (tg >= 0) {
    if (a.d_grid_h[tg] != h || a.d_grid_w[tg] != w) tg = -1;
    else {
      const unsigned char* tc = a.d_cells + a.d_grid_off[tg];
      int same = 1;
      for (int i = threadIdx.x; i < h * w; i += CAND_THREADS) same &= (tc[i] == s_raw[i]);
      if (!same) s_same = 0;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    rec->status = (uint8_t)status;
    rec->input_copy = (uint8_t)(tg >= 0 && s_same);
    rec->n_tokens = (uint16_t)min(n + 1, a.max_new);
  }
  // back to the task's orientation: apply DIHEDRAL_TRANSFORMS[inverse(d)] (src/voting.py:16-31)
  const int inv_d = (d == 1) ? 3 : (d == 3) ? 1 : d;
  const bool swap = dihedral_swaps(inv_d);
  const int ch = swap ? w : h, cw = swap ? h : w;
  if (threadIdx.x == 0) { rec->h = (uint16_t)ch; rec->w = (uint16_t)cw; }
  const int n_out = h * w;
  for (int i = threadIdx.x; i < ARCB_CANDIDATE_MAX_CELLS; i += CAND_THREADS) {
    unsigned char out = 0;
    if (i < n_out) {
      const int r = i / cw, c = i - r * cw;
      out = s_inv[s_raw[dihedral_src(inv_d, r, c, h, w)]];
    }
    rec->cells[i] = out;
  }
}

int fail_arg(const char* msg) { arcb_set_last_error(msg); return ARCB_E_ARG; }

}  // namespace

extern "C" int arcb_build_prompts(const arcb_prompt_build_args* a, void* stream) {
  if (!a) return fail_arg("null argument");
  if (a->n_variants < 0 || a->n_perms < 1) return fail_arg("bad variant or permutation count");
  if (a->n_variants == 0) return ARCB_OK;
  if (!a->d_cells || !a->d_grid_off || !a->d_grid_h || !a->d_grid_w || !a->d_tpl_off || !a->d_tpl_grid ||
      !a->d_perm_lut || !a->d_var_template || !a->d_var_dihedral || !a->d_var_perm || !a->d_var_tok_off)
    return fail_arg("null table pointer");
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = a->n_variants < sms * 8 ? a->n_variants : sms * 8;
  build_prompts_kernel<<<grid, BUILD_THREADS, 0, (cudaStream_t)stream>>>(*a);
  arcb_count_launch(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { arcb_set_last_error(cudaGetErrorString(e)); return ARCB_E_DEVICE; }
  return ARCB_OK;
}

extern "C" int arcb_canonicalize_candidates(const arcb_candidate_args* a, void* stream) {
  if (!a) return fail_arg("null argument");
  if (a->n_rows < 0 || a->max_new < 1 || a->max_new > ARCB_CANDIDATE_MAX_CELLS || a->n_perms < 1)
    return fail_arg("bad row count, permutation count or max_new above ARCB_CANDIDATE_MAX_CELLS");
  if (a->n_rows == 0) return ARCB_OK;
  if (!a->d_tokens || !a->d_row_dihedral || !a->d_perm_lut || !a->d_records) return fail_arg("null pointer");
  if (a->d_row_test_grid && (!a->d_cells || !a->d_grid_off || !a->d_grid_h || !a->d_grid_w))
    return fail_arg("test-input grids given without the grid table");
  canonicalize_kernel<<<a->n_rows, CAND_THREADS, 0, (cudaStream_t)stream>>>(*a);
  arcb_count_launch(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { arcb_set_last_error(cudaGetErrorString(e)); return ARCB_E_DEVICE; }
  return ARCB_OK;
}
