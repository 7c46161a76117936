// Embedding gather, RMSNorm, SwiGLU and rotary position encoding fused with the cache write.
//
// The residual stream is float32 on every path; T is the dtype of weights, of the
// normed activations that feed matrix products, and of the cache (float or bfloat16).
// Every reduction's order depends only on the row it belongs to, so a row's result does
// not depend on what else is in the step.
#include "common.cuh"

// ---------------------------------------------------------------- embedding gather
// out[t][:] = table[ids[t]][:]   (stratum/native/stratum_arch_llama.inc.c:564-593: a row copy, no scaling)
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int hidden, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;   // ids are range-checked on the host before a step; never trust twice
  const T* row = table + (size_t)id * hidden;
  float* o = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
}

STRATUM_EXPORT int stratum_embed_gather(const void* table, int dtype, const int* ids, float* out,
                                        int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == STRATUM_DT_F32)
    return launch_pdl(embed_gather_kernel<float>, n_tokens, threads, 0, stream, (const float*)table, ids, out, hidden,
                      vocab);
  if (dtype == STRATUM_DT_BF16)
    return launch_pdl(embed_gather_kernel<bf16>, n_tokens, threads, 0, stream, (const bf16*)table, ids, out, hidden,
                      vocab);
  return STRATUM_ERR_DTYPE;
}

// ---------------------------------------------------------------- RMSNorm
// y = x * (1/sqrt(mean(x^2) + eps)) * gain     (stratum/native/stratum_arch_llama.inc.c:45-76)
// x float32 [*, hidden]; row r of the output reads row rows[r] of x when rows != nullptr
// (the final norm runs only on the rows whose logits are wanted).
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               const int* __restrict__ rows, T* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float* xr = x + (size_t)src * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = ld_fresh(xr + i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(ld_fresh(xr + i) * scale * gain[i]);
}

// The same, four values per thread and iteration held in registers between the sum and the scaling, so a
// row is read once.  hidden % 4 == 0 and hidden <= 4 * VPT * blockDim.x.
template <typename T, int VPT>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                   const int* __restrict__ rows, T* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  const int r = blockIdx.x;
  const int n4 = hidden >> 2;
  float4 gv[VPT];
#pragma unroll
  for (int j = 0; j < VPT; j++) {               // the gain is a weight: it may be read before the wait
    const int i = threadIdx.x + j * blockDim.x;
    gv[j] = i < n4 ? reinterpret_cast<const float4*>(gain)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const int src = rows ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int i = threadIdx.x + j * blockDim.x;
    v[j] = i < n4 ? ld_fresh(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
    ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
#pragma unroll
  for (int j = 0; j < VPT; j++) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i >= n4) continue;
    const float a = v[j].x * scale * gv[j].x, b = v[j].y * scale * gv[j].y;
    const float c = v[j].z * scale * gv[j].z, d = v[j].w * scale * gv[j].w;
    if constexpr (sizeof(T) == 4) {
      reinterpret_cast<float4*>(o)[i] = make_float4(a, b, c, d);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(o)[i] = pk;
    }
  }
}

template <typename T, int VPT>
static int launch_rmsnorm_vec(const float* x, const float* gain, const int* rows, T* out, int n_rows, int hidden,
                              float eps, cudaStream_t stream) {
  const int threads = (((hidden / 4 + VPT - 1) / VPT + 31) / 32) * 32;
  return launch_pdl(rmsnorm_vec_kernel<T, VPT>, n_rows, threads, 0, stream, x, gain, rows, out, hidden, eps);
}

template <typename T>
static int launch_rmsnorm(const float* x, const float* gain, const int* rows, T* out, int n_rows, int hidden,
                          float eps, cudaStream_t stream) {
  const bool vec = hidden % 4 == 0 && ((((uintptr_t)x | (uintptr_t)gain | (uintptr_t)out) & 15) == 0);
  if (vec && hidden <= 4 * 4 * 1024) {
    // few rows (decode steps): as many threads per row as it has float4s, the shortest path through one row;
    // many rows (prompts): blocks of about 128 threads, several of which share an SM and hide each other's waits
    // On the float32 path the block shape follows from the row's length alone: the order of a row's sum is then
    // the same however the tokens are cut into steps, and so are the bits of its result.
    const int n4 = hidden / 4;
    const bool few = n_rows < 256 || sizeof(T) == 4;
    if (few && n4 <= 1024) return launch_rmsnorm_vec<T, 1>(x, gain, rows, out, n_rows, hidden, eps, stream);
    if (few) return launch_rmsnorm_vec<T, 4>(x, gain, rows, out, n_rows, hidden, eps, stream);
    if (n4 <= 256) return launch_rmsnorm_vec<T, 1>(x, gain, rows, out, n_rows, hidden, eps, stream);
    if (n4 <= 512) return launch_rmsnorm_vec<T, 2>(x, gain, rows, out, n_rows, hidden, eps, stream);
    if (n4 <= 1024) return launch_rmsnorm_vec<T, 8>(x, gain, rows, out, n_rows, hidden, eps, stream);
    return launch_rmsnorm_vec<T, 4>(x, gain, rows, out, n_rows, hidden, eps, stream);
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  return launch_pdl(rmsnorm_kernel<T>, n_rows, threads, 0, stream, x, gain, rows, out, hidden, eps);
}

STRATUM_EXPORT int stratum_rmsnorm(const float* x, const float* gain, const int* rows, void* out, int out_dtype,
                                   int n_rows, int hidden, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (out_dtype == STRATUM_DT_F32) return launch_rmsnorm<float>(x, gain, rows, (float*)out, n_rows, hidden, eps, stream);
  if (out_dtype == STRATUM_DT_BF16) return launch_rmsnorm<bf16>(x, gain, rows, (bf16*)out, n_rows, hidden, eps, stream);
  return STRATUM_ERR_DTYPE;
}

// The same per head, in place: row r of x holds n_heads stretches of head_dim values from column first_col on,
// and each becomes stretch * (1/sqrt(mean(stretch^2) + eps)) * gain (the optional per-head norm of queries and
// keys, stratum/native/stratum_arch_llama.inc.c:403-420).  One warp per (row, head); the sum runs over the
// lane's values in order and then across lanes, whatever else is in the step.
template <typename T>
__global__ void rmsnorm_heads_kernel(T* x, int n_rows, int stride, int first_col, int n_heads, int head_dim,
                                     const float* __restrict__ gain, float eps) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= n_rows * n_heads) return;
  T* p = x + (size_t)(item / n_heads) * stride + first_col + (size_t)(item % n_heads) * head_dim;
  float ss = 0.f;
  for (int d = lane; d < head_dim; d += 32) {
    const float v = ld_fresh(p + d);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)head_dim + eps);
  for (int d = lane; d < head_dim; d += 32) p[d] = from_float<T>(ld_fresh(p + d) * scale * gain[d]);
}

STRATUM_EXPORT int stratum_rmsnorm_heads(void* x, int dtype, int n_rows, int stride, int first_col, int n_heads,
                                         int head_dim, const float* gain, float eps, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0) return 0;
  if (head_dim <= 0 || first_col < 0 || first_col + (long long)n_heads * head_dim > stride) return STRATUM_ERR_SHAPE;
  const int warps = 4;
  const int blocks = (int)(((long long)n_rows * n_heads + warps - 1) / warps);
  if (dtype == STRATUM_DT_F32)
    return launch_pdl(rmsnorm_heads_kernel<float>, blocks, warps * 32, 0, stream, (float*)x, n_rows, stride,
                      first_col, n_heads, head_dim, gain, eps);
  if (dtype == STRATUM_DT_BF16)
    return launch_pdl(rmsnorm_heads_kernel<bf16>, blocks, warps * 32, 0, stream, (bf16*)x, n_rows, stride, first_col,
                      n_heads, head_dim, gain, eps);
  return STRATUM_ERR_DTYPE;
}

// ---------------------------------------------------------------- SwiGLU
// a[j] = silu(g[j]) * u[j], silu(z) = z / (1 + exp(-z))   (stratum/native/stratum_engine.h:373-391)
// gu holds gate and up interleaved: gu[r][2j] = g_j, gu[r][2j+1] = u_j.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / inter;
  const int j = (int)(i - r * inter);
  const T* p = gu + r * (size_t)(2 * inter) + 2 * j;
  const float g = to_float(p[0]), u = to_float(p[1]);
  out[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

STRATUM_EXPORT int stratum_swiglu(const void* gu, void* out, int dtype, int n_rows, int inter, cudaStream_t stream) {
  const size_t total = (size_t)n_rows * inter;
  if (total == 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == STRATUM_DT_F32)
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, inter, total);
  else if (dtype == STRATUM_DT_BF16)
    swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, inter, total);
  else
    return STRATUM_ERR_DTYPE;
  return launch_status();
}

// ---------------------------------------------------------------- rotary encoding + cache write
// qkv: [tokens][(Nq + 2 Nk) * Hd], the fused projection's output: q heads, then k heads, then v heads.
// For every token: rotate each q head in place; rotate each k head and store it, and store each v head,
// into the token's row of the paged cache.  angle = (float)pos * inv_freq[k]; pair (x0,x1) <-
// (x0 c - x1 s, x0 s + x1 c), with c and s scaled by `mscale`
// (stratum/native/stratum_arch_llama.inc.c:132-159).  Pairs are (2k, 2k+1) when interleaved, else
// (k, k + n_pairs).  Dims at and beyond 2*n_pairs pass through unrotated.
// Cache layout: [pages][Nk][page_tokens][Hd]; page of a position = block_table[seq][pos / page_tokens].
// A token whose sequence index is negative (padding) is skipped entirely.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ token_pos,
                                  const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                  int bt_stride, const float* __restrict__ inv_freq, int n_pairs,
                                  int interleaved, float mscale, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  int n_q, int n_kv, int head_dim, int page_tokens, int write_cache) {
  // a block covers one token and blockDim.y heads (q heads, then k heads, then v heads); one thread per pair
  // of dimensions.  Decode steps use one head per block (many small blocks, shortest latency), prompts several.
  pdl_trigger();
  const int t = blockIdx.x, h = blockIdx.y * blockDim.y + threadIdx.y;
  if (h >= n_q + 2 * n_kv) return;
  const int seq = token_seq[t];
  if (seq < 0) return;
  const int slot = threadIdx.x;                 // pair slot: < n_pairs rotates, the rest pass through
  if (slot >= head_dim / 2) return;
  const bool is_q = h < n_q, is_k = !is_q && h < n_q + n_kv;
  if (!is_q && !write_cache) return;
  // positions, page tables and frequencies belong to the step's description and the weights: they are read,
  // and the angle evaluated, before waiting for the projection that produced qkv
  const int pos = token_pos[t];
  int i0, i1;
  float c = 1.f, s = 0.f;
  if (slot < n_pairs && (is_q || is_k)) {
    if (interleaved) { i0 = 2 * slot; i1 = i0 + 1; } else { i0 = slot; i1 = slot + n_pairs; }
    const float angle = (float)pos * inv_freq[slot];
    sincosf(angle, &s, &c);
    c *= mscale;
    s *= mscale;
  } else {
    // dimensions beyond the rotated ones, and v: two plain neighbours per thread
    i0 = (is_q || is_k) ? 2 * n_pairs + 2 * (slot - n_pairs) : 2 * slot;
    i1 = i0 + 1;
  }
  T* dst = nullptr;
  if (!is_q) {
    const int page = block_table[(size_t)seq * bt_stride + pos / page_tokens];
    const int kvh = is_k ? h - n_q : h - n_q - n_kv;
    dst = (is_k ? k_cache : v_cache) +
          (((size_t)page * n_kv + kvh) * page_tokens + (pos % page_tokens)) * (size_t)head_dim;
  }
  T* hp = qkv + (size_t)t * ((size_t)(n_q + 2 * n_kv) * head_dim) + (size_t)h * head_dim;
  pdl_wait();
  const float x0 = ld_fresh(hp + i0), x1 = ld_fresh(hp + i1);
  const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;     // c = 1, s = 0 where nothing rotates: exact copy
  if (is_q) {
    hp[i0] = from_float<T>(y0);
    hp[i1] = from_float<T>(y1);
  } else {
    dst[i0] = from_float<T>(y0);
    dst[i1] = from_float<T>(y1);
  }
}

// The same for prompts in bfloat16 when every dimension of a head is rotated: one block per token; the sines and
// cosines of the token's angles are evaluated once (not once per head) into shared memory, then every thread moves
// 16 bytes at a time: 8 pairs (k, k + n_pairs) from two loads, or 4 pairs (2k, 2k+1) from one when interleaved;
// the v heads are copied.  Needs head_dim % 16 == 0 and 2 * n_pairs == head_dim.
template <bool INTERLEAVED>
__global__ void __launch_bounds__(256)
rope_store_prompt_kernel(bf16* __restrict__ qkv, const int* __restrict__ token_pos,
                         const int* __restrict__ token_seq, const int* __restrict__ block_table, int bt_stride,
                         const float* __restrict__ inv_freq, int n_pairs, float mscale, bf16* __restrict__ k_cache,
                         bf16* __restrict__ v_cache, int n_q, int n_kv, int head_dim, int page_tokens,
                         int write_cache) {
  extern __shared__ float2 cs[];                 // [n_pairs] (cos, sin) * mscale
  pdl_trigger();
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  if (seq < 0) {                       // a padding token
    pdl_wait();                        // no block leaves before the kernel before this one is done
    return;
  }
  const int pos = token_pos[t];
  for (int k = threadIdx.x; k < n_pairs; k += blockDim.x) {
    float sn, c;
    sincosf((float)pos * inv_freq[k], &sn, &c);
    cs[k] = make_float2(c * mscale, sn * mscale);
  }
  const int page = write_cache ? block_table[(size_t)seq * bt_stride + pos / page_tokens] : 0;
  const size_t cache_row = ((size_t)page * n_kv * page_tokens + (pos % page_tokens)) * (size_t)head_dim;
  const size_t kv_stride = (size_t)page_tokens * head_dim;
  bf16* row = qkv + (size_t)t * ((size_t)(n_q + 2 * n_kv) * head_dim);
  __syncthreads();
  pdl_wait();
  const int rot_heads = n_q + (write_cache ? n_kv : 0);
  if (INTERLEAVED) {
    const int per_head = head_dim / 8;           // 16-byte pieces of a head: 4 pairs each
    for (int it = threadIdx.x; it < rot_heads * per_head; it += blockDim.x) {
      const int h = it / per_head, c8 = it % per_head;
      bf16* src = row + (size_t)h * head_dim + 8 * c8;
      bf16* dst = h < n_q ? src : k_cache + cache_row + (size_t)(h - n_q) * kv_stride + 8 * c8;
      uint4 w = __ldcg(reinterpret_cast<const uint4*>(src));
      __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 f = cs[4 * c8 + j];
        const float x0 = __bfloat162float(e[j].x), x1 = __bfloat162float(e[j].y);
        e[j] = __floats2bfloat162_rn(x0 * f.x - x1 * f.y, x0 * f.y + x1 * f.x);
      }
      *reinterpret_cast<uint4*>(dst) = w;
    }
  } else {
    const int per_head = n_pairs / 8;            // pieces of 8 pairs: dims 8c..8c+7 and n_pairs + 8c..
    for (int it = threadIdx.x; it < rot_heads * per_head; it += blockDim.x) {
      const int h = it / per_head, c8 = it % per_head;
      bf16* src = row + (size_t)h * head_dim + 8 * c8;
      bf16* dst = h < n_q ? src : k_cache + cache_row + (size_t)(h - n_q) * kv_stride + 8 * c8;
      uint4 lo = __ldcg(reinterpret_cast<const uint4*>(src));
      uint4 hi = __ldcg(reinterpret_cast<const uint4*>(src + n_pairs));
      bf16* a = reinterpret_cast<bf16*>(&lo);
      bf16* b = reinterpret_cast<bf16*>(&hi);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float2 f = cs[8 * c8 + j];
        const float x0 = __bfloat162float(a[j]), x1 = __bfloat162float(b[j]);
        a[j] = __float2bfloat16_rn(x0 * f.x - x1 * f.y);
        b[j] = __float2bfloat16_rn(x0 * f.y + x1 * f.x);
      }
      *reinterpret_cast<uint4*>(dst) = lo;
      *reinterpret_cast<uint4*>(dst + n_pairs) = hi;
    }
  }
  if (write_cache) {
    const int per_head = head_dim / 8;
    for (int it = threadIdx.x; it < n_kv * per_head; it += blockDim.x) {
      const int h = it / per_head, c8 = it % per_head;
      const uint4 w = __ldcg(reinterpret_cast<const uint4*>(row + (size_t)(n_q + n_kv + h) * head_dim + 8 * c8));
      *reinterpret_cast<uint4*>(v_cache + cache_row + (size_t)h * kv_stride + 8 * c8) = w;
    }
  }
}

STRATUM_EXPORT int stratum_rope_store(void* qkv, int dtype, const int* token_pos, const int* token_seq,
                                      const int* block_table, int bt_stride, const float* inv_freq, int n_pairs,
                                      int interleaved, float mscale, void* k_cache, void* v_cache, int n_tokens,
                                      int n_q, int n_kv, int head_dim, int page_tokens, int write_cache,
                                      cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim % 2 != 0 || 2 * n_pairs > head_dim || n_pairs < 0 || head_dim > 2048) return STRATUM_ERR_SHAPE;
  if (n_q + 2 * n_kv > 65535) return STRATUM_ERR_LIMIT;
  if (dtype == STRATUM_DT_BF16 && n_tokens >= 64 && head_dim % 16 == 0 && 2 * n_pairs == head_dim &&
      ((((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0)) {
    const size_t smem = (size_t)n_pairs * sizeof(float2);
    if (interleaved)
      return launch_pdl(rope_store_prompt_kernel<true>, n_tokens, 256, smem, stream, (bf16*)qkv, token_pos, token_seq,
                        block_table, bt_stride, inv_freq, n_pairs, mscale, (bf16*)k_cache, (bf16*)v_cache, n_q, n_kv,
                        head_dim, page_tokens, write_cache);
    return launch_pdl(rope_store_prompt_kernel<false>, n_tokens, 256, smem, stream, (bf16*)qkv, token_pos, token_seq,
                      block_table, bt_stride, inv_freq, n_pairs, mscale, (bf16*)k_cache, (bf16*)v_cache, n_q, n_kv,
                      head_dim, page_tokens, write_cache);
  }
  const int slots = ((head_dim / 2 + 31) / 32) * 32;
  const int heads = n_q + 2 * n_kv;
  int per_block = n_tokens >= 64 ? 256 / slots : 1;
  if (per_block < 1) per_block = 1;
  if (per_block > heads) per_block = heads;
  const dim3 threads(slots, per_block);
  const dim3 grid(n_tokens, (heads + per_block - 1) / per_block);
  if (dtype == STRATUM_DT_F32)
    return launch_pdl(rope_store_kernel<float>, grid, threads, 0, stream, (float*)qkv, token_pos, token_seq,
                      block_table, bt_stride, inv_freq, n_pairs, interleaved, mscale, (float*)k_cache,
                      (float*)v_cache, n_q, n_kv, head_dim, page_tokens, write_cache);
  if (dtype == STRATUM_DT_BF16)
    return launch_pdl(rope_store_kernel<bf16>, grid, threads, 0, stream, (bf16*)qkv, token_pos, token_seq,
                      block_table, bt_stride, inv_freq, n_pairs, interleaved, mscale, (bf16*)k_cache,
                      (bf16*)v_cache, n_q, n_kv, head_dim, page_tokens, write_cache);
  return STRATUM_ERR_DTYPE;
}

// ---------------------------------------------------------------- rotation factors of a step, once
// cs[t][k] = mscale * (cos, sin)((float)pos[t] * inv_freq[k]): the same arithmetic as in rope_store_kernel, evaluated
// once per step for every token, for the matrix-product epilogues that rotate queries and keys (every layer of
// the step reads the same table).
__global__ void rope_table_kernel(const int* __restrict__ token_pos, const float* __restrict__ inv_freq, float mscale,
                                  float2* __restrict__ cs, int n_tokens, int n_pairs) {
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * n_pairs) return;
  const int t = i / n_pairs, k = i - t * n_pairs;
  float s, c;
  sincosf((float)token_pos[t] * inv_freq[k], &s, &c);
  pdl_wait();                                    // an earlier kernel may still read the table of the step before
  cs[i] = make_float2(c * mscale, s * mscale);
}

STRATUM_EXPORT int stratum_rope_table(const int* token_pos, const float* inv_freq, float mscale, float* cs,
                                      int n_tokens, int n_pairs, cudaStream_t stream) {
  if (n_tokens <= 0 || n_pairs <= 0) return 0;
  const long long total = (long long)n_tokens * n_pairs;
  if (total > (1ll << 30)) return STRATUM_ERR_LIMIT;
  return launch_pdl(rope_table_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, token_pos, inv_freq, mscale,
                    (float2*)cs, n_tokens, n_pairs);
}

// ---------------------------------------------------------------- seeded fill (random weights on the device)
// value = std * z, z standard normal from a counter-based hash of (seed, element index): Box-Muller over
// two 24-bit uniforms.  Filling a tensor in pieces or whole gives the same values.
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t n, uint64_t seed, float std_dev) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint64_t r = mix64(seed ^ mix64(i));
    const float u1 = ((float)((r >> 40) & 0xFFFFFF) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
    const float u2 = (float)((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);             // [0, 1)
    const float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    out[i] = from_float<T>(std_dev * z);
  }
}

STRATUM_EXPORT int stratum_fill_normal(void* out, int dtype, size_t n, uint64_t seed, float std_dev,
                                       cudaStream_t stream) {
  if (n == 0) return 0;
  const int threads = 256;
  size_t want = (n + threads - 1) / threads;
  const unsigned blocks = (unsigned)(want > 148 * 16 ? 148 * 16 : want);
  if (dtype == STRATUM_DT_F32)
    fill_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, n, seed, std_dev);
  else if (dtype == STRATUM_DT_BF16)
    fill_normal_kernel<bf16><<<blocks, threads, 0, stream>>>((bf16*)out, n, seed, std_dev);
  else
    return STRATUM_ERR_DTYPE;
  return launch_status();
}
