// Split-K decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the hot path: a serving loop whose memory
// pool is fixed at start-up, a plugin running inside another framework's allocator, or code that
// runs between the begin and end of a latency-critical region where an allocation (and the
// implicit device synchronisation a cudaFree can bring) is forbidden.  The regular entry point
// arcb_op_decode_attention needs a caller-provided scratch buffer for the per-split partial
// results; this variant keeps that scratch in a fixed array that is part of the library image.
//
// Limits and rules (also stated in include/arcb200.h):
//   * n_items * n_heads * n_splits <= ARCB_STATIC_ATTN_MAX_RECORDS (16384 records of 68 floats,
//     4.25 MiB).  Every GPU that loads the library holds this array until the process exits.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress with
//     that device current).  Make that first call outside any CUDA stream capture.
//   * All calls on one device share the array and it keeps the previous call's contents.  Nothing
//     in it has to start at zero: the split kernel overwrites every record it later combines.
//     Two calls that overlap on the GPU (different streams) race on it; serialise them.
//   * No cudaMalloc / cudaFree / allocating library routine is called.
#include <mutex>

#include "../../include/arcb200.h"
#include "attn_stream.cuh"

void arcb_set_last_error(const char* msg);

namespace {

constexpr long long MAX_RECORDS = ARCB_STATIC_ATTN_MAX_RECORDS;
constexpr int MAX_DEVICES = 64;

// File-scope device array.  In host code this name is only a handle for the runtime's symbol
// table, never a device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_attn_scratch[MAX_RECORDS * ATTN_SCRATCH_STRIDE];

std::mutex g_mu;
float* g_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_attn_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!p) return -1;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int arcb_op_decode_attention_static(const void* q16, const void* k, const void* v, void* out16,
                                               const int32_t* item_seq, const int32_t* item_len,
                                               const uint8_t* item_skip, int32_t n_items, int32_t n_heads,
                                               int32_t t_max, int32_t n_splits, int32_t act_format,
                                               void* stream) {
  if (!q16 || !k || !v || !out16 || !item_len) {
    arcb_set_last_error("null attention argument");
    return ARCB_E_ARG;
  }
  if (n_items <= 0 || n_heads <= 0 || t_max <= 0 || n_splits < 1 || n_splits > 64) {
    arcb_set_last_error("bad attention sizes");
    return ARCB_E_ARG;
  }
  const long long records = (long long)n_items * n_heads * n_splits;
  if (records > MAX_RECORDS) {
    arcb_set_last_error(
        "arcb_op_decode_attention_static: n_items * n_heads * n_splits exceeds the built-in scratch "
        "(ARCB_STATIC_ATTN_MAX_RECORDS = 16384); use arcb_op_decode_attention with your own scratch");
    return ARCB_E_ARG;
  }
  float* scratch = nullptr;
  const int r = static_scratch(&scratch);
  if (r != 0) {
    arcb_set_last_error(r > 0 ? cudaGetErrorString((cudaError_t)r)
                              : "cannot resolve the built-in scratch on this device");
    return r > 0 ? r : ARCB_E_STATE;
  }
  AttnStreamArgs a{};
  a.q16 = q16;
  a.k = reinterpret_cast<const __nv_bfloat16*>(k);
  a.v = reinterpret_cast<const __nv_bfloat16*>(v);
  a.out16 = out16;
  a.item_seq = item_seq;
  a.item_len = item_len;
  a.item_skip = item_skip;
  a.n_items = n_items;
  a.n_heads = n_heads;
  a.t_max = t_max;
  a.n_seqs = 0x7fffffff;
  a.n_splits = n_splits;
  a.scratch = scratch;
  a.act_f16 = act_format == ARCB_ACT_F16;
  a.err = nullptr;
  const int lr = arcb_launch_attn_stream(a, (cudaStream_t)stream);
  if (lr != 0) {
    arcb_set_last_error(lr > 0 ? cudaGetErrorString((cudaError_t)lr) : "attention launch rejected its arguments");
    return lr > 0 ? lr : ARCB_E_ARG;
  }
  return ARCB_OK;
}
