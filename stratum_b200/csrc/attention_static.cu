// Decode/prompt attention with the scratch built into the library: see attention_static.h for who
// this is for and what it promises.  The kernels are the ones of attention_mma.cu, unchanged; only the
// place the split partials are kept differs.
#include "attention_static.h"

#include "attention_mma.cu"

// The scratch.  In host code this name is only a handle for the runtime's symbol calls, not a
// device address: a kernel handed `static_scratch` from the host side would fault (or, where the GPU
// can reach host memory, quietly use the wrong bytes).  Host code gets the real address below.
static __device__ __align__(256) float static_scratch[STRATUM_ATTENTION_STATIC_SCRATCH_FLOATS];

#define STATIC_MAX_DEVICES 64
// Per device, filled at that device's first call.  Two host threads making their first calls on one device at
// the same moment may both look the address up; both get the same value, so the unsynchronised store is harmless.
static float* scratch_address[STATIC_MAX_DEVICES];

// Device address of the array on the current device; looked up once per device.
static int scratch_for_current_device(float** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= STATIC_MAX_DEVICES) return STRATUM_ERR_LIMIT;
  if (scratch_address[device] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return STRATUM_ERR_ALIGN;
    scratch_address[device] = p;
  }
  *out = scratch_address[device];
  return 0;
}

STRATUM_EXPORT long long stratum_attention_static_scratch_floats(void) {
  return (long long)STRATUM_ATTENTION_STATIC_SCRATCH_FLOATS;
}

STRATUM_EXPORT int stratum_attention_mma_static(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                                const int* token_pos, const int* token_seq,
                                                const int* block_table, int bt_stride, const int* qb_seq,
                                                const int* qb_tok0, const int* qb_ntok, int n_qblocks,
                                                int tokens_per_block, void* out, int ldo, int n_tokens, int n_q,
                                                int n_kv, int head_dim, int page_tokens, int window, float scale,
                                                int n_splits, int chunk, cudaStream_t stream) {
  if (n_tokens <= 0 || n_qblocks <= 0) return 0;
  if (n_q < 1 || head_dim < 1 || n_splits < 1) return STRATUM_ERR_SHAPE;
  // floats needed when the keys are split: the value sums [tokens*n_q*n_splits][head_dim], then (max,
  // denominator) pairs.  With one split the kernel writes its result directly and touches no scratch, so no
  // limit applies: any size the regular entry point takes is taken here too.
  const long long slots = (long long)n_tokens * n_q * n_splits;
  const long long o_floats = ((slots * head_dim + 63) / 64) * 64;        // keep the second part 256-byte aligned
  if (n_splits > 1 && o_floats + slots * 2 > (long long)STRATUM_ATTENTION_STATIC_SCRATCH_FLOATS)
    return STRATUM_ERR_LIMIT;
  float* base = nullptr;
  const int st = scratch_for_current_device(&base);
  if (st != 0) return st;
  // Every slot the merge reads is written by the attention kernel of this same call, so the array needs
  // no clearing, whatever an earlier call left in it.
  return stratum_attention_mma(q, ldq, k_cache, v_cache, token_pos, token_seq, block_table, bt_stride, qb_seq,
                               qb_tok0, qb_ntok, n_qblocks, tokens_per_block, out, ldo, base,
                               n_splits > 1 ? base + o_floats : base,
                               n_tokens, n_q, n_kv, head_dim, page_tokens, window, scale, n_splits, chunk, stream);
}
