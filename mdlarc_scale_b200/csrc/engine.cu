// C ABI of the library: engine (packed weights), session (static KV cache + greedy-loop
// state + the decode-step CUDA graph) and the standalone operator entry points.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/arcb200.h"
#include "attn_prefill.cuh"
#include "attn_stream.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "rowops.cuh"

// ---------------------------------------------------------------------------
// shared host state
// ---------------------------------------------------------------------------
static thread_local std::string g_last_error;
static std::atomic<long long> g_launches{0};

void arcb_count_launch(long long n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Programmatic dependent launch: OFF unless ARCB_PDL=1 (read once).  Measured on the decode-bound
// large workload (1024 sequences, 200 decode steps, two alternating runs each): 185.5 k generated
// tokens/s with it, 193.9 k without -- early-launched dependents hold SM resources while they wait
// and the step graph's kernels are long enough that their launch latency was already hidden.
// Switched off for the process if a graph capture with programmatic edges is refused.
static std::atomic<int> g_pdl{-1};
bool arcb_pdl_enabled() {
  int v = g_pdl.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = getenv("ARCB_PDL");
    v = (e && e[0] == '1') ? 1 : 0;
    g_pdl.store(v, std::memory_order_relaxed);
  }
  return v != 0;
}
void arcb_pdl_set(bool on) { g_pdl.store(on ? 1 : 0, std::memory_order_relaxed); }
static thread_local bool g_pdl_suppress = false;
void arcb_pdl_suppress(bool on) { g_pdl_suppress = on; }
bool arcb_pdl_suppressed() { return g_pdl_suppress; }

void arcb_set_last_error(const char* msg) { g_last_error = msg ? msg : ""; }

static int fail(int code, const char* msg) {
  g_last_error = msg;
  return code;
}
static int fail_cuda(cudaError_t e, const char* where) {
  g_last_error = std::string(where) + ": " + cudaGetErrorString(e);
  return (int)e;
}
#define CK(call)                                         \
  do {                                                   \
    cudaError_t e__ = (call);                            \
    if (e__ != cudaSuccess) return fail_cuda(e__, #call); \
  } while (0)
#define CKL(expr, what)                                            \
  do {                                                             \
    int r__ = (expr);                                              \
    if (r__ != 0) {                                                \
      if (r__ > 0 && r__ < 1000) return fail_cuda((cudaError_t)r__, what); \
      return fail(r__ < 0 ? ARCB_E_ARG : r__, what);              \
    }                                                              \
  } while (0)

// GEMM weights hold the bf16-rounded parameter values in the 16-bit container of the activations
// (half or bfloat16), because the tensor-core MMA needs both operands in one format.
struct LayerWeights {
  float* ln1_w = nullptr;
  uint16_t* w_qkv = nullptr;   // [3d][d]
  uint16_t* w_out = nullptr;   // [d][d]
  float* ln2_w = nullptr;
  uint16_t* w_gu = nullptr;    // [2 dff][d], 64 gate rows then the matching 64 up rows, repeated
  float* b_gu = nullptr;       // [2 dff] packed the same way
  uint16_t* w_down = nullptr;  // [d][dff]
  float* b_down = nullptr;          // [d]
};

struct arcb_engine {
  arcb_config cfg;
  int device = 0;
  std::vector<LayerWeights> layers;
  float* token_embed = nullptr;
  float* example_embed = nullptr;
  float* lnf_w = nullptr;
  float* lm_head = nullptr;
  float* rope = nullptr;  // cos_x | sin_x | cos_y | sin_y | cos_z | sin_z
  int* d_err = nullptr;
  std::vector<void*> allocs;
  std::vector<char> loaded;  // [ARCB_T_COUNT * max(L,1)]
  bool act_f16() const { return cfg.act_format == ARCB_ACT_F16; }
};

struct arcb_session {
  arcb_engine* eng = nullptr;
  arcb_session_desc desc;
  int splits = 1;
  // workspace carve-up
  float* x = nullptr;
  uint16_t* xn16 = nullptr;
  uint16_t* q16 = nullptr;
  uint16_t* attn16 = nullptr;
  uint16_t* h16 = nullptr;
  uint16_t* k16 = nullptr;  // K/V of one prefill call in the activation format
  uint16_t* v16 = nullptr;
  float* attn_scratch = nullptr;
  float* gemm_scratch = nullptr;   // split-K partials of the decode step's residual GEMMs
  int* example_ids = nullptr;
  bool use_examples = false;
  DecodeState st{};
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  cudaStream_t capture_stream = nullptr;
  long long graph_kernels = 0;
  bool armed = false;
  // event pair recorded (as graph nodes) around the layer-0 decode-attention launch of every replay
  cudaEvent_t probe_begin = nullptr, probe_end = nullptr;
  bool probe_recorded = false;
  // the integer state block is cleared by the first arcb_prefill, on that call's stream
  int* state_ints = nullptr;
  size_t n_state_ints = 0;
  bool state_cleared = false;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <typename T>
static int dev_alloc(arcb_engine* e, T** out, size_t count) {
  void* p = nullptr;
  cudaError_t r = cudaMalloc(&p, count * sizeof(T));
  if (r != cudaSuccess) return (int)r;
  e->allocs.push_back(p);
  *out = reinterpret_cast<T*>(p);
  return 0;
}

extern "C" const char* arcb_last_error(void) { return g_last_error.c_str(); }

extern "C" int arcb_device_ok(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return 0;
  return p.major == 10 ? 1 : 0;
}

extern "C" int64_t arcb_launch_count(int reset) {
  return reset ? g_launches.exchange(0) : g_launches.load();
}

// ---------------------------------------------------------------------------
// engine
// ---------------------------------------------------------------------------
extern "C" int arcb_engine_create(const arcb_config* cfg, arcb_engine** out) {
  if (!cfg || !out) return fail(ARCB_E_ARG, "null argument");
  if (cfg->vocab_size != ARCB_VOCAB) return fail(ARCB_E_UNSUPPORTED, "vocab_size must be 14");
  if (cfg->n_heads <= 0 || cfg->d_model != cfg->n_heads * ARCB_HEAD_DIM)
    return fail(ARCB_E_UNSUPPORTED, "head_dim must be 64");
  if (cfg->d_model % 128 || cfg->d_ff % 64 || cfg->n_layers <= 0 || cfg->d_ff <= 0)
    return fail(ARCB_E_UNSUPPORTED, "d_model must be a multiple of 128 and d_ff of 64");
  if (cfg->max_x <= 0 || cfg->max_y <= 0 || cfg->max_z <= 0 || cfg->num_examples <= 0)
    return fail(ARCB_E_ARG, "bad table extents");
  if (!arcb_device_ok()) return fail(ARCB_E_UNSUPPORTED, "current device is not compute capability 10.x");
  CKL(arcb_gemm_init(), "gemm init (shared-memory opt-in / cuTensorMapEncodeTiled lookup)");
  CKL(arcb_attn_prefill_init(), "prefill attention init (shared-memory opt-in)");
  arcb_engine* e = new arcb_engine();
  e->cfg = *cfg;
  cudaGetDevice(&e->device);
  const size_t d = cfg->d_model, dff = cfg->d_ff;
  e->layers.resize(cfg->n_layers);
  e->loaded.assign((size_t)ARCB_T_COUNT * cfg->n_layers, 0);
  int r = 0;
  for (auto& L : e->layers) {
    r |= dev_alloc(e, &L.ln1_w, d);
    r |= dev_alloc(e, &L.w_qkv, 3 * d * d);
    r |= dev_alloc(e, &L.w_out, d * d);
    r |= dev_alloc(e, &L.ln2_w, d);
    r |= dev_alloc(e, &L.w_gu, 2 * dff * d);
    r |= dev_alloc(e, &L.b_gu, 2 * dff);
    r |= dev_alloc(e, &L.w_down, d * dff);
    r |= dev_alloc(e, &L.b_down, d);
  }
  r |= dev_alloc(e, &e->token_embed, (size_t)cfg->vocab_size * d);
  r |= dev_alloc(e, &e->example_embed, (size_t)cfg->num_examples * d);
  r |= dev_alloc(e, &e->lnf_w, d);
  r |= dev_alloc(e, &e->lm_head, (size_t)cfg->vocab_size * d);
  const size_t rope_n = 2 * ((size_t)cfg->max_x * ARCB_ROPE_PX + (size_t)cfg->max_y * ARCB_ROPE_PY +
                             (size_t)cfg->max_z * ARCB_ROPE_PZ);
  r |= dev_alloc(e, &e->rope, rope_n);
  r |= dev_alloc(e, &e->d_err, 64);
  if (r) {
    arcb_engine_destroy(e);
    return fail(ARCB_E_STATE, "cudaMalloc of packed weights failed");
  }
  cudaMemset(e->d_err, 0, 64 * sizeof(int));
  *out = e;
  return ARCB_OK;
}

extern "C" int arcb_engine_destroy(arcb_engine* e) {
  if (!e) return ARCB_OK;
  for (void* p : e->allocs) cudaFree(p);
  delete e;
  return ARCB_OK;
}

extern "C" int arcb_engine_load_tensor(arcb_engine* e, int32_t kind, int32_t layer, const float* src,
                                       int64_t numel, void* stream_v) {
  if (!e || !src) return fail(ARCB_E_ARG, "null argument");
  if (kind < 0 || kind >= ARCB_T_COUNT) return fail(ARCB_E_ARG, "unknown tensor kind");
  cudaStream_t stream = (cudaStream_t)stream_v;
  const arcb_config& c = e->cfg;
  const long long d = c.d_model, dff = c.d_ff;
  const bool per_layer = kind >= ARCB_T_LN1_W && kind <= ARCB_T_DOWN_B;
  if (per_layer && (layer < 0 || layer >= c.n_layers)) return fail(ARCB_E_ARG, "layer out of range");
  LayerWeights* L = per_layer ? &e->layers[layer] : nullptr;
  long long rows = 0, cols = 0;
  void* dst = nullptr;
  int blk = 0, blk_stride = 0, blk_off = 0, to_bf16 = 0;
  const long long nx = (long long)c.max_x * ARCB_ROPE_PX, ny = (long long)c.max_y * ARCB_ROPE_PY,
                  nz = (long long)c.max_z * ARCB_ROPE_PZ;
  switch (kind) {
    case ARCB_T_TOKEN_EMBED: rows = c.vocab_size; cols = d; dst = e->token_embed; break;
    case ARCB_T_EXAMPLE_EMBED: rows = c.num_examples; cols = d; dst = e->example_embed; break;
    case ARCB_T_LN1_W: rows = 1; cols = d; dst = L->ln1_w; break;
    case ARCB_T_QKV_W: rows = 3 * d; cols = d; dst = L->w_qkv; to_bf16 = 1; break;
    case ARCB_T_OUT_W: rows = d; cols = d; dst = L->w_out; to_bf16 = 1; break;
    case ARCB_T_LN2_W: rows = 1; cols = d; dst = L->ln2_w; break;
    case ARCB_T_GATE_W: rows = dff; cols = d; dst = L->w_gu; to_bf16 = 1; blk = 64; blk_stride = 128; break;
    case ARCB_T_UP_W: rows = dff; cols = d; dst = L->w_gu; to_bf16 = 1; blk = 64; blk_stride = 128; blk_off = 64; break;
    case ARCB_T_GATE_B: rows = dff; cols = 1; dst = L->b_gu; blk = 64; blk_stride = 128; break;
    case ARCB_T_UP_B: rows = dff; cols = 1; dst = L->b_gu; blk = 64; blk_stride = 128; blk_off = 64; break;
    case ARCB_T_DOWN_W: rows = d; cols = dff; dst = L->w_down; to_bf16 = 1; break;
    case ARCB_T_DOWN_B: rows = 1; cols = d; dst = L->b_down; break;
    case ARCB_T_LNF_W: rows = 1; cols = d; dst = e->lnf_w; break;
    case ARCB_T_LM_HEAD: rows = c.vocab_size; cols = d; dst = e->lm_head; break;
    // RoPE tables are fp32 buffers of the module, not parameters; they are kept exact.
    case ARCB_T_ROPE_COS_X: rows = 1; cols = nx; dst = e->rope; break;
    case ARCB_T_ROPE_SIN_X: rows = 1; cols = nx; dst = e->rope + nx; break;
    case ARCB_T_ROPE_COS_Y: rows = 1; cols = ny; dst = e->rope + 2 * nx; break;
    case ARCB_T_ROPE_SIN_Y: rows = 1; cols = ny; dst = e->rope + 2 * nx + ny; break;
    case ARCB_T_ROPE_COS_Z: rows = 1; cols = nz; dst = e->rope + 2 * nx + 2 * ny; break;
    case ARCB_T_ROPE_SIN_Z: rows = 1; cols = nz; dst = e->rope + 2 * nx + 2 * ny + nz; break;
    default: return fail(ARCB_E_ARG, "unknown tensor kind");
  }
  if (numel != rows * cols) return fail(ARCB_E_ARG, "tensor has the wrong number of elements");
  if (kind >= ARCB_T_ROPE_COS_X) {
    CK(cudaMemcpyAsync(dst, src, (size_t)numel * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  } else {
    if (blk == 0) { blk = (int)rows; blk_stride = (int)rows; }
    if (to_bf16 && e->act_f16()) to_bf16 = 2;
    CKL(arcb_launch_pack_rows(src, dst, rows, cols, blk, blk_stride, blk_off, to_bf16, stream), "pack_rows");
  }
  e->loaded[(size_t)kind * c.n_layers + (per_layer ? layer : 0)] = 1;
  return ARCB_OK;
}

static bool engine_complete(const arcb_engine* e) {
  const int L = e->cfg.n_layers;
  for (int k = 0; k < ARCB_T_COUNT; ++k) {
    const bool per_layer = k >= ARCB_T_LN1_W && k <= ARCB_T_DOWN_B;
    for (int l = 0; l < (per_layer ? L : 1); ++l)
      if (!e->loaded[(size_t)k * L + l]) return false;
  }
  return true;
}

// ---------------------------------------------------------------------------
// session
// ---------------------------------------------------------------------------
// Split count of decode attention.  t_max = 0: the upper bound used to size the scratch (one warp per
// work item); with the session's cache capacity known, fewer splits when the launch qualifies for the
// kernel that puts four warps on every work item (attn_stream.cu), which also spares small batches
// the merge launch.
static int choose_splits(const arcb_engine* e, int n_seqs, int requested, int t_max = 0) {
  if (requested > 0) return requested > 64 ? 64 : requested;
  // aim for ~16 resident warps on each of the 148 SMs
  const long long work = (long long)n_seqs * e->cfg.n_heads;
  long long s = (148LL * 16 + work - 1) / work;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  static const bool coop_splits = [] { const char* v = getenv("ARCB_COOP_SPLITS"); return !(v && v[0] == '0'); }();  // A/B switch
  if (t_max > 0 && coop_splits) {
    long long s4 = (148LL * 4 + work - 1) / work;
    if (s4 < 1) s4 = 1;
    if (s4 < s && work * s4 >= 296 && (long long)t_max >= 128 * s4) return (int)s4;
  }
  return (int)s;
}

struct WsLayout {
  size_t x, xn, q, attn, h, k16, v16, scratch, gemm_scratch, ints, total;
  size_t n_int;
};

static WsLayout ws_layout(const arcb_engine* e, int B, int P, int splits) {
  const size_t d = e->cfg.d_model, dff = e->cfg.d_ff;
  const size_t R = (size_t)(B > P ? B : P);
  WsLayout w;
  size_t off = 0;
  w.x = off; off = align_up(off + R * d * 4, 256);
  w.xn = off; off = align_up(off + R * d * 2, 256);
  w.q = off; off = align_up(off + R * d * 2, 256);
  w.attn = off; off = align_up(off + R * d * 2, 256);
  w.h = off; off = align_up(off + R * dff * 2, 256);
  w.k16 = off; off = align_up(off + (size_t)P * d * 2, 1024);
  w.v16 = off; off = align_up(off + (size_t)P * d * 2, 1024);
  w.scratch = off;
  off = align_up(off + (splits > 1 ? (size_t)B * e->cfg.n_heads * splits * ATTN_SCRATCH_STRIDE * 4 : 0), 256);
  w.gemm_scratch = off;
  off = align_up(off + align_up((size_t)B, 128) * d * 4, 256);
  w.ints = off;
  // cur_len, len0, cur_tok, gx, gy, gin, slot, kv_len, example_ids (9 x B) + pos (3 x B) + finished (B bytes, as B ints) + counters
  w.n_int = (size_t)B * 13 + 64;
  off = align_up(off + w.n_int * 4, 256);
  w.total = off;
  return w;
}

extern "C" int64_t arcb_session_workspace_bytes(const arcb_engine* e, int32_t n_seqs,
                                                int32_t max_prefill_tokens, int32_t attn_splits) {
  if (!e || n_seqs <= 0 || max_prefill_tokens < 0) return -1;
  return (int64_t)ws_layout(e, n_seqs, max_prefill_tokens, choose_splits(e, n_seqs, attn_splits)).total;
}

extern "C" int64_t arcb_kv_cache_bytes(const arcb_engine* e, int32_t n_seqs, int32_t t_max) {
  if (!e || n_seqs <= 0 || t_max <= 0) return -1;
  return (int64_t)e->cfg.n_layers * 2 * n_seqs * e->cfg.d_model * (int64_t)t_max * 2;
}

extern "C" int arcb_session_create(arcb_engine* e, const arcb_session_desc* dsc, arcb_session** out) {
  if (!e || !dsc || !out) return fail(ARCB_E_ARG, "null argument");
  if (!engine_complete(e)) return fail(ARCB_E_STATE, "engine is missing tensors");
  if (dsc->n_seqs <= 0 || dsc->t_max <= 0 || dsc->max_new <= 0 || dsc->max_prefill_tokens <= 0)
    return fail(ARCB_E_ARG, "bad session sizes");
  if (!dsc->d_kv_cache || !dsc->d_workspace || !dsc->d_out_tokens) return fail(ARCB_E_ARG, "null buffer");
  if (dsc->kv_cache_bytes < arcb_kv_cache_bytes(e, dsc->n_seqs, dsc->t_max))
    return fail(ARCB_E_ARG, "kv cache too small");
  if (((uintptr_t)dsc->d_kv_cache & 255) || ((uintptr_t)dsc->d_workspace & 255))
    return fail(ARCB_E_ARG, "buffers must be 256-byte aligned");
  const int splits = choose_splits(e, dsc->n_seqs, dsc->attn_splits, dsc->t_max);
  const WsLayout w = ws_layout(e, dsc->n_seqs, dsc->max_prefill_tokens, choose_splits(e, dsc->n_seqs, dsc->attn_splits));
  if ((size_t)dsc->workspace_bytes < w.total) return fail(ARCB_E_ARG, "workspace too small");
  arcb_session* s = new arcb_session();
  s->eng = e;
  s->desc = *dsc;
  s->splits = splits;
  uint8_t* base = reinterpret_cast<uint8_t*>(dsc->d_workspace);
  s->x = reinterpret_cast<float*>(base + w.x);
  s->xn16 = reinterpret_cast<uint16_t*>(base + w.xn);
  s->q16 = reinterpret_cast<uint16_t*>(base + w.q);
  s->attn16 = reinterpret_cast<uint16_t*>(base + w.attn);
  s->h16 = reinterpret_cast<uint16_t*>(base + w.h);
  s->k16 = reinterpret_cast<uint16_t*>(base + w.k16);
  s->v16 = reinterpret_cast<uint16_t*>(base + w.v16);
  s->attn_scratch = splits > 1 ? reinterpret_cast<float*>(base + w.scratch) : nullptr;
  s->gemm_scratch = reinterpret_cast<float*>(base + w.gemm_scratch);
  int* ints = reinterpret_cast<int*>(base + w.ints);
  const int B = dsc->n_seqs;
  DecodeState& st = s->st;
  st.n_seqs = B; st.t_max = dsc->t_max; st.max_new = dsc->max_new; st.stop_on_end = dsc->stop_on_end;
  st.cur_len = ints + 0 * B; st.len0 = ints + 1 * B; st.cur_tok = ints + 2 * B;
  st.gx = ints + 3 * B; st.gy = ints + 4 * B; st.gin = ints + 5 * B;
  st.slot = ints + 6 * B; st.kv_len = ints + 7 * B;
  s->example_ids = ints + 8 * B;
  st.pos = ints + 9 * B;                                             // 3 B ints
  st.finished = reinterpret_cast<unsigned char*>(ints + 12 * B);     // B bytes inside B ints
  st.n_finished = ints + 13 * B;
  st.out_tokens = dsc->d_out_tokens;
  st.forced = dsc->d_forced;
  st.step_logits = dsc->d_step_logits;
  st.palette_mask = dsc->d_palette_mask;
  st.target_shape = dsc->d_target_shape;
  st.palette_penalty = dsc->palette_penalty;
  st.shape_penalty = dsc->shape_penalty;
  st.disallow_mask = dsc->disallow_token_mask & 0x3fffu;
  st.temperature = dsc->temperature;
  st.top_k = dsc->top_k;
  st.sample_seed = dsc->sample_seed;
  st.sample_stream = dsc->d_sample_stream;
  st.err = e->d_err;
  // No device work here: the state block may be a recycled allocation whose previous user still
  // has kernels queued on the caller's stream, so it is cleared by the first arcb_prefill, in
  // stream order.
  s->state_ints = ints;
  s->n_state_ints = w.n_int;
  cudaError_t r = cudaStreamCreateWithFlags(&s->capture_stream, cudaStreamNonBlocking);
  if (r != cudaSuccess) { delete s; return fail_cuda(r, "cudaStreamCreate"); }
  if (cudaEventCreate(&s->probe_begin) != cudaSuccess || cudaEventCreate(&s->probe_end) != cudaSuccess) {
    cudaGetLastError();
    s->probe_begin = s->probe_end = nullptr;  // the probe is optional
  }
  *out = s;
  return ARCB_OK;
}

extern "C" int arcb_session_destroy(arcb_session* s) {
  if (!s) return ARCB_OK;
  if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
  if (s->graph) cudaGraphDestroy(s->graph);
  if (s->capture_stream) cudaStreamDestroy(s->capture_stream);
  if (s->probe_begin) cudaEventDestroy(s->probe_begin);
  if (s->probe_end) cudaEventDestroy(s->probe_end);
  delete s;
  return ARCB_OK;
}

static bool use_tc_for(const arcb_engine* e, int M, int N, int K) {
  if (e->cfg.gemm_path == ARCB_GEMM_SIMT) return false;
  if (!arcb_gemm_tc_supported(M, N, K)) return false;
  (void)M;   // the tensor-core kernels also win for a handful of rows: a 16-row launch of the CUDA-core
             // kernel measured 90 us against ~15 us (operand streaming through TMA on every tile's CTA)
  return true;
}

// Suppresses the programmatic-launch attribute for this thread's launches while on (and on scope exit
// restores the default, whichever way the function returns).
struct PdlSuppressGuard {
  bool active = false;
  void on() { arcb_pdl_suppress(true); active = true; }
  void off() { if (active) { arcb_pdl_suppress(false); active = false; } }
  ~PdlSuppressGuard() { off(); }
};

// One transformer block over `rows` rows of the residual stream s->x (xn16 already holds
// ln1(x)); on return xn16 holds the next block's ln1(x) (or is stale after the last block).
static int run_layer(arcb_session* s, int l, int rows, const int* pos, const int* slot, const int* seq,
                     const int* kv_count, const unsigned char* skip, bool prefill,
                     const arcb_prefill_args* pa, cudaStream_t stream) {
  arcb_engine* e = s->eng;
  const arcb_config& c = e->cfg;
  const LayerWeights& L = e->layers[l];
  const int d = c.d_model, dff = c.d_ff, B = s->desc.n_seqs, T = s->desc.t_max;
  const int f16 = e->act_f16() ? 1 : 0;
  const size_t layer_elems = (size_t)2 * B * d * T;
  __nv_bfloat16* kbase = reinterpret_cast<__nv_bfloat16*>(s->desc.d_kv_cache) + (size_t)l * layer_elems;
  __nv_bfloat16* vbase = kbase + (size_t)B * d * T;

  GemmEpilogue ep{};
  ep.M = rows; ep.act_f16 = f16; ep.err = e->d_err;
  // QKV projection + 3D RoPE + cache write
  ep.mode = EPI_QKV_ROPE; ep.N = 3 * d; ep.out16 = s->q16;
  ep.pos = pos; ep.slot = slot; ep.seq = seq; ep.kcache = kbase; ep.vcache = vbase;
  ep.t_max = T; ep.n_heads = c.n_heads; ep.d_model = d; ep.n_seqs = B;
  ep.rope = e->rope; ep.max_x = c.max_x; ep.max_y = c.max_y; ep.max_z = c.max_z;
  const bool want_flash = prefill && c.attn_path == ARCB_ATTN_AUTO && pa && pa->n_qblocks > 0 && pa->d_kv_row &&
                          pa->d_qblock_kv0 && pa->n_kv_rows > 0 && arcb_attn_prefill_available();
  if (want_flash) {
    ep.k16 = s->k16; ep.v16 = s->v16; ep.kv_row = pa->d_kv_row;
    ep.kv16_rows = pa->n_kv_rows; ep.kv16_identity = pa->kv_row_identity == 1;
  }
  CKL(arcb_launch_gemm(s->xn16, L.w_qkv, ep, d, f16, use_tc_for(e, rows, 3 * d, d), stream), "qkv gemm");

  // attention
  PdlSuppressGuard plain_edges;
  const bool flash = prefill && c.attn_path == ARCB_ATTN_AUTO && pa && pa->n_qblocks > 0 && pa->d_kv_row &&
                     pa->d_qblock_kv0 && pa->n_kv_rows > 0 && arcb_attn_prefill_available();
  if (flash) {
    AttnPrefillArgs fa{};
    fa.q16 = s->q16; fa.k16 = s->k16; fa.v16 = s->v16; fa.out16 = s->attn16;
    fa.seq = seq; fa.kv_count = kv_count; fa.qblock_row0 = pa->d_qblock_row0; fa.qblock_rows = pa->d_qblock_rows;
    fa.qblock_kv0 = pa->d_qblock_kv0;
    fa.n_qblocks = pa->n_qblocks; fa.n_rows = rows; fa.n_kv_rows = pa->n_kv_rows; fa.n_heads = c.n_heads;
    fa.act_f16 = f16; fa.err = e->d_err;
    CKL(arcb_launch_attn_prefill(fa, stream), "prefill attention");
  } else {
    AttnStreamArgs aa{};
    aa.q16 = s->q16; aa.k = kbase; aa.v = vbase; aa.out16 = s->attn16;
    aa.item_seq = seq; aa.item_len = kv_count; aa.item_skip = skip;
    aa.n_items = rows; aa.n_heads = c.n_heads; aa.t_max = T; aa.n_seqs = B;
    aa.n_splits = prefill ? 1 : s->splits; aa.scratch = s->attn_scratch; aa.act_f16 = f16; aa.err = e->d_err;
    const bool probe = !prefill && l == 0 && s->probe_begin && s->probe_end;
    // cudaEventRecordExternal: under stream capture this becomes an event-record NODE of the graph (a
    // plain record would only mark a capture dependency and leave the event unusable for timing)
    // the kernels next to the two event-record nodes are joined to them by ordinary edges
    if (probe) {
      plain_edges.on();
      CK(cudaEventRecordWithFlags(s->probe_begin, stream, cudaEventRecordExternal));
    }
    CKL(arcb_launch_attn_stream(aa, stream), "attention");
    if (probe) { CK(cudaEventRecordWithFlags(s->probe_end, stream, cudaEventRecordExternal)); s->probe_recorded = true; }
  }

  // out_proj + residual
  GemmEpilogue er{};
  er.mode = EPI_RESID; er.M = rows; er.N = d; er.x = s->x; er.bias = nullptr; er.act_f16 = f16; er.err = e->d_err;
  er.splitk_scratch = prefill ? nullptr : s->gemm_scratch;   // sized for the decode step's rows only
  CKL(arcb_launch_gemm(s->attn16, L.w_out, er, d, f16, use_tc_for(e, rows, d, d), stream), "out_proj gemm");
  plain_edges.off();
  CKL(arcb_launch_rmsnorm(s->x, L.ln2_w, s->xn16, rows, d, c.norm_eps, f16, stream), "ln2");
  // gate | up + SwiGLU
  GemmEpilogue eg{};
  eg.mode = EPI_SWIGLU; eg.M = rows; eg.N = 2 * dff; eg.bias = L.b_gu; eg.out16 = s->h16; eg.act_f16 = f16; eg.err = e->d_err;
  CKL(arcb_launch_gemm(s->xn16, L.w_gu, eg, d, f16, use_tc_for(e, rows, 2 * dff, d), stream), "gate/up gemm");
  // down + bias + residual
  er.bias = L.b_down;
  CKL(arcb_launch_gemm(s->h16, L.w_down, er, dff, f16, use_tc_for(e, rows, d, dff), stream), "down gemm");
  if (l + 1 < c.n_layers)
    CKL(arcb_launch_rmsnorm(s->x, e->layers[l + 1].ln1_w, s->xn16, rows, d, c.norm_eps, f16, stream), "ln1");
  return ARCB_OK;
}

extern "C" int arcb_prefill(arcb_session* s, const arcb_prefill_args* a, void* stream_v) {
  if (!s || !a) return fail(ARCB_E_ARG, "null argument");
  if (a->n_tokens <= 0 || a->n_tokens > s->desc.max_prefill_tokens)
    return fail(ARCB_E_ARG, "n_tokens outside (0, max_prefill_tokens]");
  if (a->n_kv_rows < 0 || a->n_kv_rows > s->desc.max_prefill_tokens)
    return fail(ARCB_E_ARG, "n_kv_rows outside [0, max_prefill_tokens]");
  if (!a->d_token_ids || !a->d_pos_xyz || !a->d_seq || !a->d_kv_slot || !a->d_kv_count)
    return fail(ARCB_E_ARG, "null token arrays");
  if (a->n_first < 0 || (a->n_first > 0 && (!a->d_first_row || !a->d_first_seq || !a->d_prompt_len ||
                                              !a->d_grid_x || !a->d_grid_y || !a->d_grid_in_output)))
    return fail(ARCB_E_ARG, "null first-token arrays");
  cudaStream_t stream = (cudaStream_t)stream_v;
  arcb_engine* e = s->eng;
  const arcb_config& c = e->cfg;
  if (!s->state_cleared) {
    CK(cudaMemsetAsync(s->state_ints, 0, s->n_state_ints * 4, stream));
    s->state_cleared = true;
  }
  const bool use_ex = c.use_example_embedding && a->d_example_ids;
  if (a->n_first > 0) {
    if (s->graph_exec && s->use_examples != use_ex) {  // the recorded step baked the other choice in
      cudaGraphExecDestroy(s->graph_exec); s->graph_exec = nullptr;
      cudaGraphDestroy(s->graph); s->graph = nullptr;
    }
    s->use_examples = use_ex;
    if (use_ex)
      CK(cudaMemcpyAsync(s->example_ids, a->d_example_ids, (size_t)s->desc.n_seqs * 4,
                         cudaMemcpyDeviceToDevice, stream));
  }
  EmbedArgs ea{};
  ea.rows = a->n_tokens; ea.d = c.d_model; ea.vocab = c.vocab_size; ea.num_examples = c.num_examples;
  ea.token_ids = a->d_token_ids; ea.seq = a->d_seq; ea.example_ids = use_ex ? a->d_example_ids : nullptr;
  ea.token_embed = e->token_embed; ea.example_embed = e->example_embed; ea.ln_w = e->layers[0].ln1_w;
  ea.x = s->x; ea.xn16 = s->xn16; ea.eps = c.norm_eps; ea.act_f16 = e->act_f16() ? 1 : 0;
  CKL(arcb_launch_embed_norm(ea, stream), "embed");
  for (int l = 0; l < c.n_layers; ++l) {
    int r = run_layer(s, l, a->n_tokens, a->d_pos_xyz, a->d_kv_slot, a->d_seq, a->d_kv_count, nullptr, true, a, stream);
    if (r) return r;
  }
  HeadArgs ha{};
  ha.d = c.d_model; ha.eps = c.norm_eps; ha.x = s->x; ha.lnf_w = e->lnf_w; ha.lm_head = e->lm_head;
  if (a->d_logits_all) {
    ha.mode = HEAD_PLAIN; ha.rows = a->n_tokens; ha.row_index = nullptr; ha.logits = a->d_logits_all; ha.argmax = nullptr;
    CKL(arcb_launch_head(ha, s->st, stream), "head(all)");
  }
  if (a->n_first > 0) {
    ha.mode = HEAD_FIRST; ha.rows = a->n_first; ha.row_index = a->d_first_row; ha.logits = a->d_first_logits;
    ha.argmax = nullptr; ha.first_seq = a->d_first_seq; ha.prompt_len = a->d_prompt_len;
    ha.grid_x = a->d_grid_x; ha.grid_y = a->d_grid_y; ha.grid_in_output = a->d_grid_in_output;
    CKL(arcb_launch_head(ha, s->st, stream), "head(first)");
    s->armed = true;
  }
  return ARCB_OK;
}

static int record_decode_step(arcb_session* s, cudaStream_t stream) {
  arcb_engine* e = s->eng;
  const arcb_config& c = e->cfg;
  const int B = s->desc.n_seqs;
  EmbedArgs ea{};
  ea.rows = B; ea.d = c.d_model; ea.vocab = c.vocab_size; ea.num_examples = c.num_examples;
  ea.token_ids = nullptr; ea.seq = nullptr; ea.example_ids = s->use_examples ? s->example_ids : nullptr;
  ea.token_embed = e->token_embed; ea.example_embed = e->example_embed; ea.ln_w = e->layers[0].ln1_w;
  ea.x = s->x; ea.xn16 = s->xn16; ea.eps = c.norm_eps; ea.act_f16 = e->act_f16() ? 1 : 0;
  CKL(arcb_launch_decode_begin(s->st, ea, stream), "decode_begin");
  for (int l = 0; l < c.n_layers; ++l) {
    int r = run_layer(s, l, B, s->st.pos, s->st.slot, nullptr, s->st.kv_len,
                      s->desc.stop_on_end == 1 ? s->st.finished : nullptr, false, nullptr, stream);
    if (r) return r;
  }
  HeadArgs ha{};
  ha.mode = HEAD_DECODE; ha.rows = B; ha.d = c.d_model; ha.eps = c.norm_eps; ha.x = s->x;
  ha.lnf_w = e->lnf_w; ha.lm_head = e->lm_head;
  CKL(arcb_launch_head(ha, s->st, stream), "head(decode)");
  return ARCB_OK;
}

extern "C" int arcb_decode(arcb_session* s, int32_t n_steps, void* stream_v) {
  if (!s) return fail(ARCB_E_ARG, "null session");
  if (!s->armed) return fail(ARCB_E_STATE, "arcb_prefill with first-token rows must run before arcb_decode");
  if (n_steps <= 0) return ARCB_OK;
  cudaStream_t stream = (cudaStream_t)stream_v;
  for (int attempt = 0; !s->graph_exec && attempt < 2; ++attempt) {
    const long long before = g_launches.load();
    CK(cudaStreamBeginCapture(s->capture_stream, cudaStreamCaptureModeThreadLocal));
    int r = record_decode_step(s, s->capture_stream);
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(s->capture_stream, &g);
    s->graph_kernels = g_launches.load() - before;
    g_launches.fetch_sub(s->graph_kernels);  // recording is not launching
    cudaGraphExec_t ge = nullptr;
    if (r == 0 && ce == cudaSuccess) ce = cudaGraphInstantiate(&ge, g, 0);
    if (r == 0 && ce == cudaSuccess) {
      s->graph = g;
      s->graph_exec = ge;
      break;
    }
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    if (attempt == 0 && arcb_pdl_enabled()) {
      arcb_pdl_set(false);   // capture with programmatic edges refused: record plain launches instead
      continue;
    }
    if (r) return r;
    return fail_cuda(ce, "capture / instantiate of the decode step");
  }
  for (int i = 0; i < n_steps; ++i) CK(cudaGraphLaunch(s->graph_exec, stream));
  arcb_count_launch(s->graph_kernels * n_steps);
  return ARCB_OK;
}

extern "C" int arcb_session_poll(arcb_session* s, int32_t* n_finished, int32_t* device_error, void* stream_v) {
  if (!s) return fail(ARCB_E_ARG, "null session");
  cudaStream_t stream = (cudaStream_t)stream_v;
  int nf = 0, err = 0;
  CK(cudaMemcpyAsync(&nf, s->st.n_finished, 4, cudaMemcpyDeviceToHost, stream));
  CK(cudaMemcpyAsync(&err, s->eng->d_err, 4, cudaMemcpyDeviceToHost, stream));
  CK(cudaStreamSynchronize(stream));
  if (n_finished) *n_finished = nf;
  if (device_error) *device_error = err;
  if (err) {
    cudaMemsetAsync(s->eng->d_err, 0, 4, stream);
    char buf[96];
    snprintf(buf, sizeof buf, "device error word = %d", err);
    return fail(ARCB_E_DEVICE, buf);
  }
  return ARCB_OK;
}

extern "C" int arcb_engine_saturation_count(arcb_engine* e, int64_t* count, int32_t reset, void* stream_v) {
  if (!e || !count) return fail(ARCB_E_ARG, "null argument");
  cudaStream_t stream = (cudaStream_t)stream_v;
  int n = 0;
  CK(cudaMemcpyAsync(&n, e->d_err + 1, 4, cudaMemcpyDeviceToHost, stream));
  if (reset) CK(cudaMemsetAsync(e->d_err + 1, 0, 4, stream));
  CK(cudaStreamSynchronize(stream));
  *count = n;
  return ARCB_OK;
}

extern "C" int arcb_session_attention_probe(arcb_session* s, float* ms) {
  if (!s || !ms) return fail(ARCB_E_ARG, "null argument");
  if (!s->probe_recorded || !s->graph_exec) return fail(ARCB_E_STATE, "no decode step has run yet");
  cudaError_t r = cudaEventSynchronize(s->probe_end);
  if (r == cudaSuccess) r = cudaEventElapsedTime(ms, s->probe_begin, s->probe_end);
  if (r != cudaSuccess) {
    cudaGetLastError();  // a failed query must not be picked up by the next launch check
    return fail_cuda(r, "attention probe");
  }
  return ARCB_OK;
}

// ---------------------------------------------------------------------------
// standalone operators
// ---------------------------------------------------------------------------
extern "C" int arcb_op_rmsnorm(const float* x, const float* w, void* out16, int32_t rows, int32_t d,
                               float eps, int32_t act_format, void* stream) {
  if (!x || !w || !out16 || d % 4) return fail(ARCB_E_ARG, "bad rmsnorm arguments");
  CKL(arcb_launch_rmsnorm(x, w, out16, rows, d, eps, act_format == ARCB_ACT_F16, (cudaStream_t)stream), "rmsnorm");
  return ARCB_OK;
}

// The shared-memory opt-in of the GEMM kernels is a per-device attribute: do it once for every
// device a standalone operator is called on (engines do it when they are created).
static int ensure_gemm_init() {
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return arcb_gemm_init();
  std::lock_guard<std::mutex> lock(mu);
  if (!done[dev]) {
    const int r = arcb_gemm_init();
    if (r) return r;
    done[dev] = true;
  }
  return 0;
}

extern "C" int arcb_op_gemm(const void* a16, const void* w, float* y, int32_t M, int32_t N, int32_t K,
                            int32_t act_format, int32_t gemm_path, void* stream) {
  if (!a16 || !w || !y || M <= 0) return fail(ARCB_E_ARG, "bad gemm arguments");
  CKL(ensure_gemm_init(), "gemm init");
  if (N % 128 || K % 32) return fail(ARCB_E_ARG, "gemm needs N % 128 == 0 and K % 32 == 0");
  const int variant = gemm_path == ARCB_GEMM_TC_1CTA ? 1 : (gemm_path == ARCB_GEMM_TC_2CTA ? 2 : 0);
  bool tc = gemm_path == ARCB_GEMM_TC || variant != 0 || (gemm_path == ARCB_GEMM_AUTO);
  if (tc && !arcb_gemm_tc_supported(M, N, K)) {
    if (gemm_path != ARCB_GEMM_AUTO) return fail(ARCB_E_ARG, "tcgen05 gemm needs K % 64 == 0");
    tc = false;
  }
  GemmEpilogue ep{};
  ep.mode = EPI_STORE_F32; ep.M = M; ep.N = N; ep.y = y;
  CKL(arcb_launch_gemm(a16, w, ep, K, act_format == ARCB_ACT_F16, tc, (cudaStream_t)stream, variant), "gemm");
  return ARCB_OK;
}

extern "C" int arcb_op_gemm_residual(const void* a16, const void* w, const float* bias, float* x, int32_t M,
                                     int32_t N, int32_t K, int32_t act_format, int32_t gemm_path, void* stream) {
  if (!a16 || !w || !x || M <= 0) return fail(ARCB_E_ARG, "bad gemm arguments");
  CKL(ensure_gemm_init(), "gemm init");
  if (N % 128 || K % 32) return fail(ARCB_E_ARG, "gemm needs N % 128 == 0 and K % 32 == 0");
  const int variant = gemm_path == ARCB_GEMM_TC_1CTA ? 1 : (gemm_path == ARCB_GEMM_TC_2CTA ? 2 : 0);
  bool tc = gemm_path == ARCB_GEMM_TC || variant != 0 || (gemm_path == ARCB_GEMM_AUTO);
  if (tc && !arcb_gemm_tc_supported(M, N, K)) {
    if (gemm_path != ARCB_GEMM_AUTO) return fail(ARCB_E_ARG, "tcgen05 gemm needs K % 64 == 0");
    tc = false;
  }
  GemmEpilogue ep{};
  ep.mode = EPI_RESID; ep.M = M; ep.N = N; ep.x = x; ep.bias = bias;
  CKL(arcb_launch_gemm(a16, w, ep, K, act_format == ARCB_ACT_F16, tc, (cudaStream_t)stream, variant), "gemm");
  return ARCB_OK;
}

extern "C" int64_t arcb_gemm_splitk_scratch_bytes(int32_t M, int32_t N, int32_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || ensure_gemm_init() != 0) return 0;
  if (!arcb_gemm_splitk_bn(M, N, K)) return 0;
  return (int64_t)align_up((size_t)M, 128) * N * 4;
}

extern "C" int arcb_op_gemm_residual_splitk(const void* a16, const void* w, const float* bias, float* x, int32_t M,
                                            int32_t N, int32_t K, int32_t act_format, void* scratch, void* stream) {
  if (!a16 || !w || !x || M <= 0) return fail(ARCB_E_ARG, "bad gemm arguments");
  CKL(ensure_gemm_init(), "gemm init");
  if (N % 128 || !arcb_gemm_tc_supported(M, N, K)) return fail(ARCB_E_ARG, "gemm needs N % 128 == 0 and K % 64 == 0");
  if (!scratch || !arcb_gemm_splitk_bn(M, N, K))
    return fail(ARCB_E_ARG, "the split-K kernel does not apply to this shape (arcb_gemm_splitk_scratch_bytes returned 0) or no scratch was given");
  GemmEpilogue ep{};
  ep.mode = EPI_RESID; ep.M = M; ep.N = N; ep.x = x; ep.bias = bias; ep.splitk_scratch = reinterpret_cast<float*>(scratch);
  CKL(arcb_launch_gemm(a16, w, ep, K, act_format == ARCB_ACT_F16, true, (cudaStream_t)stream, 0), "gemm");
  return ARCB_OK;
}

extern "C" int64_t arcb_attn_scratch_bytes(int32_t n_items, int32_t n_heads, int32_t n_splits) {
  if (n_items <= 0 || n_heads <= 0 || n_splits <= 1) return 0;
  return (int64_t)n_items * n_heads * n_splits * ATTN_SCRATCH_STRIDE * 4;
}

extern "C" int arcb_op_decode_attention(const void* q16, const void* k, const void* v, void* out16,
                                        const int32_t* item_seq, const int32_t* item_len,
                                        const uint8_t* item_skip, int32_t n_items, int32_t n_heads,
                                        int32_t t_max, int32_t n_splits, void* scratch, int32_t act_format,
                                        void* stream) {
  if (!q16 || !k || !v || !out16 || !item_len) return fail(ARCB_E_ARG, "null attention argument");
  if (n_items <= 0 || n_heads <= 0 || t_max <= 0 || n_splits < 1 || n_splits > 64)
    return fail(ARCB_E_ARG, "bad attention sizes");
  if (n_splits > 1 && !scratch) return fail(ARCB_E_ARG, "split attention needs scratch");
  AttnStreamArgs a{};
  a.q16 = q16; a.k = reinterpret_cast<const __nv_bfloat16*>(k); a.v = reinterpret_cast<const __nv_bfloat16*>(v);
  a.out16 = out16; a.item_seq = item_seq; a.item_len = item_len; a.item_skip = item_skip;
  a.n_items = n_items; a.n_heads = n_heads; a.t_max = t_max; a.n_seqs = 0x7fffffff; a.n_splits = n_splits;
  a.scratch = reinterpret_cast<float*>(scratch); a.act_f16 = act_format == ARCB_ACT_F16; a.err = nullptr;
  CKL(arcb_launch_attn_stream(a, (cudaStream_t)stream), "attention");
  return ARCB_OK;
}

extern "C" int arcb_op_head(const float* x, const int32_t* row_index, const float* lnf_w, const float* lm_head,
                            float* logits, int32_t* argmax, int32_t rows, int32_t d, float eps, void* stream) {
  if (!x || !lnf_w || !lm_head || d % 4) return fail(ARCB_E_ARG, "bad head arguments");
  HeadArgs ha{};
  ha.mode = HEAD_PLAIN; ha.rows = rows; ha.d = d; ha.eps = eps; ha.x = x; ha.row_index = row_index;
  ha.lnf_w = lnf_w; ha.lm_head = lm_head; ha.logits = logits; ha.argmax = argmax;
  DecodeState st{};
  CKL(arcb_launch_head(ha, st, (cudaStream_t)stream), "head");
  return ARCB_OK;
}
