// Causal grouped-query attention over the paged cache, one warp per (token, query head).
//
// The kernel of the true 32-bit path for prompts and for decoding alike, and the bfloat16
// path's fallback for head sizes its tensor-core kernels refuse.  For query head h of a token at
// position p in sequence s:  score_t = (q_h . K_t[kv(h)]) * scale over the keys t in [lo, p],
// lo = 0 or p - window + 1;  probabilities by softmax;  o_h = sum_t prob_t V_t[kv(h)]
// (stratum/native/stratum_arch_llama.inc.c:435-514; kv(h) = h / (Nq/Nk), :444).
//
// Keys are visited in chunks of 32 whose boundaries are multiples of 32 from position 0, and the
// running maximum, denominator and output are updated once per chunk in key order, all in
// float32.  So the result at a position does not depend on how the tokens were cut into steps,
// on the other sequences of the step, or on which pages hold the keys.
//
// q comes from the fused projection buffer [tokens][ldq] (already rotated); the cache is
// [pages][Nk][page_tokens][Hd]; page of position t = block_table[seq][t / page_tokens].
#include <math.h>

#include "common.cuh"

#define AS_WARPS 4
#define AS_MAX_HD 256

template <typename T>
__global__ void __launch_bounds__(AS_WARPS * 32)
attention_simple_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_cache,
                        const T* __restrict__ v_cache, const int* __restrict__ token_pos,
                        const int* __restrict__ token_seq, const int* __restrict__ block_table, int bt_stride,
                        T* __restrict__ out, int ldo, int n_tokens, int n_q, int n_kv, int head_dim,
                        int page_tokens, int window, float scale) {
  __shared__ float qs[AS_WARPS][AS_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * AS_WARPS + warp;
  if (item >= (long long)n_tokens * n_q) return;
  const int t = (int)(item / n_q), h = (int)(item - (long long)t * n_q);
  const int seq = token_seq[t];
  if (seq < 0) return;                       // padding token
  const int pos = token_pos[t];
  const int kvh = h / (n_q / n_kv);
  const T* qp = q + (size_t)t * ldq + (size_t)h * head_dim;
  for (int d = lane; d < head_dim; d += 32) qs[warp][d] = to_float(qp[d]);
  __syncwarp();

  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* bt = block_table + (size_t)seq * bt_stride;
  const size_t head_off = (size_t)kvh * page_tokens * head_dim;
  const size_t page_stride = (size_t)n_kv * page_tokens * head_dim;

  float m = -INFINITY, l = 0.f;
  float acc[AS_MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < AS_MAX_HD / 32; i++) acc[i] = 0.f;

  for (int base = (lo / 32) * 32; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key >= lo && key <= pos;
    const int page = bt[base / page_tokens];          // page_tokens is a multiple of 32: one page per chunk
    const size_t chunk_off = (size_t)page * page_stride + head_off + (size_t)(base % page_tokens) * head_dim;
    float s = -INFINITY;
    if (valid) {
      const T* kr = k_cache + chunk_off + (size_t)lane * head_dim;
      float dot = 0.f;
      for (int d = 0; d < head_dim; d++) dot = fmaf(qs[warp][d], to_float(kr[d]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));        // finite: every chunk visited holds a valid key
    const float corr = expf(m - m_new);               // exp(-inf) = 0 on the first chunk
    const float p = valid ? expf(s - m_new) : 0.f;
    // denominator: add this chunk's 32 probabilities in key order
    float chunk_sum = 0.f;
#pragma unroll
    for (int j = 0; j < 32; j++) chunk_sum += __shfl_sync(0xffffffffu, p, j);
    l = l * corr + chunk_sum;
#pragma unroll
    for (int i = 0; i < AS_MAX_HD / 32; i++) acc[i] *= corr;
    const T* vr = v_cache + chunk_off;
    const int n_here = min(32, pos - base + 1);
    for (int j = 0; j < n_here; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int i = 0; i < AS_MAX_HD / 32; i++) {
        const int d = lane + 32 * i;
        if (d < head_dim) acc[i] = fmaf(pj, to_float(vr[(size_t)j * head_dim + d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* op = out + (size_t)t * ldo + (size_t)h * head_dim;
#pragma unroll
  for (int i = 0; i < AS_MAX_HD / 32; i++) {
    const int d = lane + 32 * i;
    if (d < head_dim) op[d] = from_float<T>(acc[i] * inv);
  }
}

STRATUM_EXPORT int stratum_attention_simple(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                            int dtype, const int* token_pos, const int* token_seq,
                                            const int* block_table, int bt_stride, void* out, int ldo,
                                            int n_tokens, int n_q, int n_kv, int head_dim, int page_tokens,
                                            int window, float scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim < 1 || head_dim > AS_MAX_HD) return STRATUM_ERR_LIMIT;
  if (n_kv < 1 || n_q % n_kv != 0 || page_tokens % 32 != 0) return STRATUM_ERR_SHAPE;
  const long long items = (long long)n_tokens * n_q;
  const long long blocks = (items + AS_WARPS - 1) / AS_WARPS;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_F32)
    attention_simple_kernel<float><<<(unsigned)blocks, AS_WARPS * 32, 0, stream>>>(
        (const float*)q, ldq, (const float*)k_cache, (const float*)v_cache, token_pos, token_seq, block_table,
        bt_stride, (float*)out, ldo, n_tokens, n_q, n_kv, head_dim, page_tokens, window, scale);
  else if (dtype == STRATUM_DT_BF16)
    attention_simple_kernel<bf16><<<(unsigned)blocks, AS_WARPS * 32, 0, stream>>>(
        (const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, token_pos, token_seq, block_table,
        bt_stride, (bf16*)out, ldo, n_tokens, n_q, n_kv, head_dim, page_tokens, window, scale);
  else
    return STRATUM_ERR_DTYPE;
  return launch_status();
}
