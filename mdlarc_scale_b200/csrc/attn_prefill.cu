// Flash-style causal prefill attention (placeholder until the tcgen05 kernel lands):
// reports itself unavailable so that the engine uses the streaming kernel.
#include "attn_prefill.cuh"

bool arcb_attn_prefill_available() { return false; }
int arcb_launch_attn_prefill(const AttnPrefillArgs&, cudaStream_t) { return -1; }
