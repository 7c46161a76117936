// Picking the next token from float32 logits: greedy argmax and temperature sampling with
// optional top-k / top-p filtering, one thread block per row.
//
// Greedy: the largest logit, the lowest index among equals (stratum/native/stratum_engine.h:429-463).
// Sampling (stratum/native/stratum_arch_qwen35.inc.c:14023-14109): probabilities
// exp((l - max) / T) normalised; a draw u in [0,1) picks the first candidate whose cumulative
// probability exceeds u, the last candidate if rounding leaves none.  Without filters the
// candidates are all ids in id order.  With top-k and/or top-p they are the k largest logits
// (at most SAMPLE_CAND_MAX, the reference's own cap of 512 candidates, :14019) by descending
// logit, lower id first among equals, cut after the first prefix whose probability reaches top_p,
// and renormalised.  The uniform u comes from the host (one PCG32 stream per sequence), so a
// sequence's draws do not depend on what else is in the batch.
#include <float.h>
#include <math.h>

#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_CAND_MAX 512

struct MaxIdx { float v; int i; };

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ MaxIdx block_argmax(MaxIdx mine, MaxIdx* scratch /* 33 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other;
    other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
    mine = better(mine, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    MaxIdx t = lane < n_warps ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other;
      other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, other);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ MaxIdx row_argmax(const float* __restrict__ row, int vocab, MaxIdx* scratch) {
  MaxIdx mine{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = ld_fresh(row + (i));
    if (v > mine.v) { mine.v = v; mine.i = i; }      // ascending i per thread: first of equals is kept
  }
  MaxIdx r = block_argmax(mine, scratch);
  if (r.i == 0x7fffffff) { r.i = 0; r.v = ld_fresh(row + (0)); }  // every logit is -inf or NaN: index 0, as a scalar scan would give
  return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ ids,
              float* __restrict__ values) {
  __shared__ MaxIdx scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const MaxIdx best = row_argmax(logits + (size_t)r * ld, vocab, scratch);
  if (threadIdx.x == 0) {
    ids[r] = best.i;
    if (values) values[r] = best.v;
  }
}

// The same over ARGMAX_SPLITS blocks per row: each block finds the best of its stretch of the row; the block
// that finishes last (a counter per row tells) picks among the stretches, lowest index first among equals,
// and resets the counter, so the scratch needs zeroing only once, when it is made.
#define ARGMAX_SPLITS 32
__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ ids,
                    float* __restrict__ values, float* __restrict__ part_v, int* __restrict__ part_i,
                    unsigned* __restrict__ counters) {
  __shared__ MaxIdx scratch[33];
  __shared__ bool last;
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, sp = blockIdx.y;
  const float* row = logits + (size_t)r * ld;
  const int chunk = (vocab + ARGMAX_SPLITS - 1) / ARGMAX_SPLITS;
  const int b = sp * chunk, e = min(vocab, b + chunk);
  MaxIdx mine{-INFINITY, 0x7fffffff};
  for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
    const float v = ld_fresh(row + (i));
    if (v > mine.v) { mine.v = v; mine.i = i; }
  }
  const MaxIdx best = block_argmax(mine, scratch);
  if (threadIdx.x == 0) {
    part_v[r * ARGMAX_SPLITS + sp] = best.v;
    part_i[r * ARGMAX_SPLITS + sp] = best.i;
    __threadfence();
    last = atomicAdd(&counters[r], 1u) == ARGMAX_SPLITS - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (threadIdx.x < 32) {
    MaxIdx t{-INFINITY, 0x7fffffff};
    if (threadIdx.x < ARGMAX_SPLITS) {
      t.v = __ldcg(&part_v[r * ARGMAX_SPLITS + threadIdx.x]);
      t.i = __ldcg(&part_i[r * ARGMAX_SPLITS + threadIdx.x]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other;
      other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, other);
    }
    if (threadIdx.x == 0) {
      if (t.i == 0x7fffffff) { t.i = 0; t.v = ld_fresh(row + (0)); }
      ids[r] = t.i;
      if (values) values[r] = t.v;
      counters[r] = 0;
    }
  }
}

// scratch (optional): part_v float[n_rows*32], part_i int[n_rows*32], counters unsigned[n_rows] zeroed once by
// the caller; with it, large rows are searched by 32 blocks each.
STRATUM_EXPORT int stratum_argmax(const float* logits, int ld, int n_rows, int vocab, int* ids, float* values,
                                  float* part_v, int* part_i, unsigned* counters, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab < 1) return STRATUM_ERR_SHAPE;
  if (part_v && part_i && counters && vocab >= 8192)
    return launch_pdl(argmax_split_kernel, dim3(n_rows, ARGMAX_SPLITS), 256, 0, stream, logits, ld, vocab, ids, values,
                      part_v, part_i, counters);
  return launch_pdl(argmax_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, ids, values);
}

// ---------------------------------------------------------------- temperature sampling
// Per-row parameters (so one launch serves sequences with different settings):
//   temperature[r] <= 0 -> greedy;  top_k[r] <= 0 -> off;  top_p[r] >= 1 -> off;  uniform[r] in [0,1).

// order-preserving map float -> uint32 (larger float, larger key)
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ ids, float* __restrict__ values) {
  __shared__ MaxIdx mi_scratch[33];
  __shared__ float partial[SAMPLE_THREADS];
  __shared__ unsigned hist[256];
  __shared__ float cand_v[SAMPLE_CAND_MAX];
  __shared__ int cand_i[SAMPLE_CAND_MAX];
  __shared__ unsigned sh_prefix, sh_remaining, sh_count, sh_equal_total;

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const MaxIdx best = row_argmax(row, vocab, mi_scratch);
  if (!(temp > 0.f)) {
    if (tid == 0) { ids[r] = best.i; if (values) values[r] = best.v; }
    return;
  }
  const float inv_t = 1.0f / temp;
  const float u = uniform[r];
  int k = top_k[r];
  const float tp = top_p[r];
  const bool filtered = (k > 0) || (tp < 1.0f);

  if (!filtered) {
    // every id in id order: thread i owns the contiguous ids [i*chunk, (i+1)*chunk)
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int b = tid * chunk, e = min(vocab, b + chunk);
    float s = 0.f;
    for (int i = b; i < e; i++) s += expf((ld_fresh(row + (i)) - best.v) * inv_t);
    partial[tid] = s;
    __syncthreads();
    if (tid == 0) {
      // serial over 1024 partial sums: fixed order, exact same total for the same row every time
      float total = 0.f;
      for (int i = 0; i < SAMPLE_THREADS; i++) total += partial[i];
      const float target = u * total;
      float cum = 0.f;
      int owner = -1;
      for (int i = 0; i < SAMPLE_THREADS; i++) {
        if (target < cum + partial[i]) { owner = i; break; }
        cum += partial[i];
      }
      int pick = vocab - 1;
      if (owner >= 0) {
        const int ob = owner * chunk, oe = min(vocab, ob + chunk);
        pick = oe - 1;
        for (int i = ob; i < oe; i++) {
          cum += expf((ld_fresh(row + (i)) - best.v) * inv_t);
          if (target < cum) { pick = i; break; }
        }
      }
      ids[r] = pick;
      if (values) values[r] = ld_fresh(row + (pick));
    }
    return;
  }

  // ---- filtered: the k largest logits, k <= SAMPLE_CAND_MAX
  if (k <= 0 || k > SAMPLE_CAND_MAX) k = SAMPLE_CAND_MAX;
  if (k > vocab) k = vocab;
  // radix select, 8 bits a pass from the top: find the key of the k-th largest
  if (tid == 0) { sh_prefix = 0; sh_remaining = (unsigned)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; pass++) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const unsigned prefix = sh_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < vocab; i += blockDim.x) {
      const uint32_t key = float_key(ld_fresh(row + (i)));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned remaining = sh_remaining;
      int b = 255;
      for (; b > 0; b--) {
        if (hist[b] >= remaining) break;
        remaining -= hist[b];
      }
      sh_prefix = prefix | ((unsigned)b << shift);
      sh_remaining = remaining;       // how many of the k lie in the chosen bucket
      sh_equal_total = hist[b];       // after the last pass: how many logits equal the k-th largest
    }
    __syncthreads();
  }
  const uint32_t kth_key = sh_prefix;       // key of the k-th largest logit
  const unsigned n_equal_wanted = sh_remaining;
  // gather: everything above the k-th key, then the lowest ids among those equal to it.  When all
  // the equal ones are wanted (no tie straddles the cut) they are gathered in the same parallel pass.
  const bool take_all_equal = sh_equal_total == n_equal_wanted;
  if (tid == 0) sh_count = 0;
  __syncthreads();
  for (int i = tid; i < vocab; i += blockDim.x) {
    const uint32_t key = float_key(ld_fresh(row + (i)));
    if (key > kth_key || (take_all_equal && key == kth_key)) {
      const unsigned slot = atomicAdd(&sh_count, 1u);
      cand_v[slot] = ld_fresh(row + (i));
      cand_i[slot] = i;
    }
  }
  __syncthreads();
  if (tid == 0 && !take_all_equal) {
    unsigned slot = sh_count, taken = 0;
    for (int i = 0; i < vocab && taken < n_equal_wanted; i++) {
      if (float_key(ld_fresh(row + (i))) == kth_key) { cand_v[slot] = ld_fresh(row + (i)); cand_i[slot] = i; slot++; taken++; }
    }
    sh_count = slot;
  }
  __syncthreads();
  const int n_cand = (int)sh_count;        // == k
  // pad to a power of two and sort: descending logit, ascending id among equals (bitonic, in shared memory)
  int n_sort = 1;
  while (n_sort < n_cand) n_sort <<= 1;
  for (int i = n_cand + tid; i < n_sort; i += blockDim.x) { cand_v[i] = -INFINITY; cand_i[i] = 0x7fffffff; }
  __syncthreads();
  for (int size = 2; size <= n_sort; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < n_sort; i += blockDim.x) {
        const int j = i ^ stride;
        if (j > i) {
          const bool up = (i & size) == 0;      // this run is sorted "first comes first"
          const bool i_first = cand_v[i] > cand_v[j] || (cand_v[i] == cand_v[j] && cand_i[i] < cand_i[j]);
          if (i_first != up) {
            const float tv = cand_v[i]; cand_v[i] = cand_v[j]; cand_v[j] = tv;
            const int ti = cand_i[i]; cand_i[i] = cand_i[j]; cand_i[j] = ti;
          }
        }
      }
      __syncthreads();
    }
  }
  if (tid == 0) {
    // probabilities over the candidates, top-p cut, renormalised draw: all serial over <= 512 entries
    const float top = cand_v[0];
    double sum = 0.0;
    for (int i = 0; i < n_cand; i++) sum += (double)expf((cand_v[i] - top) * inv_t);
    int keep = n_cand;
    if (tp < 1.0f) {
      double cum = 0.0;
      for (int i = 0; i < n_cand; i++) {
        cum += (double)(float)((double)expf((cand_v[i] - top) * inv_t) / sum);
        if (cum >= (double)tp) { keep = i + 1; break; }
      }
    }
    double kept = 0.0;
    for (int i = 0; i < keep; i++) kept += (double)expf((cand_v[i] - top) * inv_t);
    const double target = (double)u * kept;
    double cum = 0.0;
    int pick = keep - 1;
    for (int i = 0; i < keep; i++) {
      cum += (double)expf((cand_v[i] - top) * inv_t);
      if (target < cum) { pick = i; break; }
    }
    ids[r] = cand_i[pick];
    if (values) values[r] = cand_v[pick];
  }
}

STRATUM_EXPORT int stratum_sample(const float* logits, int ld, int n_rows, int vocab, const float* temperature,
                                  const int* top_k, const float* top_p, const float* uniform, int* ids,
                                  float* values, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab < 1) return STRATUM_ERR_SHAPE;
  return launch_pdl(sample_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, top_k, top_p,
                    uniform, ids, values);
}
