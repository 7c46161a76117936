// Declaration of the one entry point of this library that allocates no memory at all.
//
// It has no counterpart in the reference (shiaho777/stratum), whose engine keeps its scratch in
// file-scope host arrays and never runs on a CUDA device.
//
// Who needs it.  The regular entry point, stratum_attention_mma, takes its scratch (the per-split
// partial results of decode attention) from the caller, who normally gets it from an allocator.
// Some callers cannot allocate device memory at the moment they need attention: code running
// inside a CUDA stream capture, where cudaMalloc is illegal; a real-time or interrupt-like host
// thread that must not take the driver's allocation locks; a host process that was handed a fixed
// memory budget and a closed allocator; a foreign-language binding that can pass pointers but owns
// no allocator.  For them the scratch lives inside the library, in a file-scope
// `static __device__` array of STRATUM_ATTENTION_STATIC_SCRATCH_FLOATS floats (16 MiB), which every
// GPU that loads this library holds until the process exits.
//
// Contract.
//  * Same arguments and same result as stratum_attention_mma, minus the two scratch pointers.
//    Inputs and outputs are still the caller's.
//  * With n_splits > 1 it needs, for s = tokens * n_q * n_splits,
//        round_up(s * head_dim, 64) + 2 * s  <=  STRATUM_ATTENTION_STATIC_SCRATCH_FLOATS;
//    a larger request is refused with STRATUM_ERR_LIMIT (-4) before anything is launched.  With the
//    Llama-3.1-8B shape (32 heads of 128) and 16 splits that is up to 63 sequences per decode step.
//    With n_splits == 1 no scratch is used and no limit applies.
//  * It calls no cudaMalloc, cudaFree or any allocating routine.  The first call on a device looks
//    up the array's device address (cudaGetSymbolAddress, with that device current) and remembers
//    it; that first call should be made before any stream capture begins.
//  * Every call on a device shares the one array, which keeps the last call's contents.  Nothing in it
//    has to start at zero: each call writes every slot it later reads.  Two calls that overlap on the
//    GPU (different streams, no ordering between them) race on the array; order them.
//  * Returns 0, a positive cudaError_t, or a negative STRATUM_ERR_* code.
#pragma once
#include <cuda_runtime.h>

#define STRATUM_ATTENTION_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int stratum_attention_mma_static(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                 const int* token_pos, const int* token_seq, const int* block_table,
                                 int bt_stride, const int* qb_seq, const int* qb_tok0, const int* qb_ntok,
                                 int n_qblocks, int tokens_per_block, void* out, int ldo, int n_tokens, int n_q,
                                 int n_kv, int head_dim, int page_tokens, int window, float scale, int n_splits,
                                 int chunk, cudaStream_t stream);

// The size of the built-in scratch, in floats, for callers that size their batches by it.
long long stratum_attention_static_scratch_floats(void);

#ifdef __cplusplus
}
#endif
