// Picking the next token from float32 logits: greedy argmax and temperature sampling with
// optional top-k / top-p filtering.  Rows of 8,192 logits or more are cut over 32 thread blocks each
// (argmax_split_kernel, sample_split_kernel); shorter rows, and rows the split sampling kernel marks,
// get one block (argmax_kernel, sample_kernel).
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
static_assert(SAMPLE_THREADS == 1024 && SAMPLE_CAND_MAX % 32 == 0, "the sampling kernel counts on 32 warps");

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

// f(i, logit) for every logit of the row, 16 bytes per load where the row allows it.  A thread meets its ids in
// ascending order; which thread meets which id depends on the row's alignment, so only order-free work goes here.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int vocab, F f) {
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int n4 = vocab >> 2;
    // four loads in flight per thread before the first is used (one block reads a whole row: latency bounds it)
    for (int q0 = threadIdx.x; q0 < n4; q0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int q = q0 + j * blockDim.x;
        if (q < n4) v[j] = ld_fresh(reinterpret_cast<const float4*>(row) + q);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int q = q0 + j * blockDim.x;
        if (q < n4) { f(4 * q, v[j].x); f(4 * q + 1, v[j].y); f(4 * q + 2, v[j].z); f(4 * q + 3, v[j].w); }
      }
    }
    for (int i = 4 * n4 + threadIdx.x; i < vocab; i += blockDim.x) f(i, ld_fresh(row + i));
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) f(i, ld_fresh(row + i));
  }
}

__device__ __forceinline__ MaxIdx row_argmax(const float* __restrict__ row, int vocab, MaxIdx* scratch) {
  MaxIdx mine{-INFINITY, 0x7fffffff};
  for_each_logit(row, vocab, [&](int i, float v) {
    if (v > mine.v) { mine.v = v; mine.i = i; }      // ascending i per thread: first of equals is kept
  });
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
// Every sum is taken in an order that depends on the sizes only, so a row's pick is the same in every batch and run.

// order-preserving map float -> uint32 (larger float, larger key)
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Inclusive prefix sum over the lanes of a warp (lane 0 first).
template <typename T>
__device__ __forceinline__ T warp_incl_scan(T v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int warp_min(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Exclusive prefix sum of one value per thread over the block (thread 0 first); *total gets the sum of all.
// scratch: 33 values.  Every thread of the block calls it.
template <typename T>
__device__ __forceinline__ T block_excl_scan(T v, T* scratch, T* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T incl = warp_incl_scan(v);
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const T w = lane < n_warps ? scratch[lane] : T(0);
    const T wi = warp_incl_scan(w);
    scratch[lane] = wi - w;
    if (lane == 31) scratch[32] = wi;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + incl - v;
}

// One warp: lane l holds the SAMPLE_CAND_MAX / 32 consecutive candidates from its first on (sorted: descending
// logit, ascending id among equals; cand_e their weights, zero beyond n_cand); sums in float64: their total, the
// top-p cut over the normalised weights, and the draw among what is kept.
__device__ __forceinline__ void draw_from_candidates(const float* cand_v, const int* cand_i, const float* cand_e,
                                                     int n_cand, float tp, float u, int r, int* ids, float* values) {
  const int lane = threadIdx.x & 31;
  constexpr int PER = SAMPLE_CAND_MAX / 32;
  const int c0 = lane * PER;
  double own = 0.0;
#pragma unroll
  for (int j = 0; j < PER; j++) own += (double)cand_e[c0 + j];
  const double sum = warp_sum(own);
  int keep = n_cand;
  if (tp < 1.0f) {
    double q[PER], own_q = 0.0;
#pragma unroll
    for (int j = 0; j < PER; j++) { q[j] = (double)(float)((double)cand_e[c0 + j] / sum); own_q += q[j]; }
    double cum = warp_incl_scan(own_q) - own_q;
    int first = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; j++) {
      cum += q[j];
      if (first == 0x7fffffff && c0 + j < n_cand && cum >= (double)tp) first = c0 + j;
    }
    first = warp_min(first);
    if (first != 0x7fffffff) keep = first + 1;
  }
  double own_kept = 0.0;
#pragma unroll
  for (int j = 0; j < PER; j++) own_kept += (c0 + j < keep) ? (double)cand_e[c0 + j] : 0.0;
  const double kept = warp_sum(own_kept);
  const double target = (double)u * kept;
  double cum = warp_incl_scan(own_kept) - own_kept;
  int first = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < PER; j++) {
    if (c0 + j < keep) {
      cum += (double)cand_e[c0 + j];
      if (first == 0x7fffffff && target < cum) first = c0 + j;
    }
  }
  first = warp_min(first);
  const int pick = first == 0x7fffffff ? keep - 1 : first;
  if (lane == 0) {
    ids[r] = cand_i[pick];
    if (values) values[r] = cand_v[pick];
  }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ ids, float* __restrict__ values, const int* redo) {
  __shared__ MaxIdx mi_scratch[33];
  __shared__ float f_scratch[33];
  __shared__ unsigned u_scratch[33];
  __shared__ float cand_e[SAMPLE_CAND_MAX];
  __shared__ unsigned hist[256];
  __shared__ float cand_v[SAMPLE_CAND_MAX];
  __shared__ int cand_i[SAMPLE_CAND_MAX];
  __shared__ unsigned sh_prefix, sh_remaining, sh_count, sh_equal_total;
  __shared__ int sh_owner;

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (redo && !__ldcg(redo + r)) return;       // behind the 32-block kernel: only the rows it marked
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
    // Every id in id order.  Warp w owns the contiguous ids [w*seg, (w+1)*seg) and reads them 32 at a time; the
    // warps' sums are added in warp order, which gives the warp that holds the draw; that warp then walks its
    // stretch again, 32 ids at a time, until the running sum passes the draw.
    const int n_warps = SAMPLE_THREADS / 32;
    const int seg = (((vocab + n_warps - 1) / n_warps) + 31) & ~31;
    const int b = min(vocab, warp * seg), e = min(vocab, b + seg);
    float s = 0.f;
    for (int i = b + lane; i < e; i += 32) s += expf((ld_fresh(row + i) - best.v) * inv_t);
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) f_scratch[warp] = s;
    if (tid == 0) sh_owner = -1;
    __syncthreads();
    if (warp == 0) {
      const float w = f_scratch[lane];                 // n_warps == 32
      const float incl = warp_incl_scan(w);
      const float total = __shfl_sync(0xffffffffu, incl, 31);
      const float target = u * total;
      const unsigned hit = __ballot_sync(0xffffffffu, target < incl);
      if (lane == 0) {
        sh_owner = hit ? (__ffs(hit) - 1) : -1;
        f_scratch[32] = target;
      }
      f_scratch[lane] = incl - w;                      // the sum of the warps before
    }
    __syncthreads();
    const int owner = sh_owner;
    if (owner < 0) {                                   // rounding left no warp: the last id
      if (tid == 0) { ids[r] = vocab - 1; if (values) values[r] = ld_fresh(row + (vocab - 1)); }
      return;
    }
    if (warp != owner) return;
    const float target = f_scratch[32];
    float carry = f_scratch[owner];
    int pick = e - 1;                                  // rounding left no id in the stretch: its last
    for (int base = b; base < e; base += 4 * 32) {
      float x[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int i = base + 32 * j + lane;
        x[j] = i < e ? expf((ld_fresh(row + i) - best.v) * inv_t) : 0.f;
      }
      bool found = false;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (!found) {
          const float incl = carry + warp_incl_scan(x[j]);
          const unsigned hit = __ballot_sync(0xffffffffu, target < incl && base + 32 * j + lane < e);
          if (hit) { pick = base + 32 * j + __ffs(hit) - 1; found = true; }
          carry = __shfl_sync(0xffffffffu, incl, 31);
        }
      }
      if (found) break;
    }
    if (lane == 0) { ids[r] = pick; if (values) values[r] = ld_fresh(row + pick); }
    return;
  }

  // ---- filtered: the k largest logits, k <= SAMPLE_CAND_MAX
  if (k <= 0 || k > SAMPLE_CAND_MAX) k = SAMPLE_CAND_MAX;
  if (k > vocab) k = vocab;
  // radix select, 8 bits a pass from the top: find the key of the k-th largest.  Lanes that meet the same bucket
  // add to it once (the first pass sees nearly every logit in two or three buckets).
  if (tid == 0) { sh_prefix = 0; sh_remaining = (unsigned)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; pass++) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const unsigned prefix = sh_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for_each_logit(row, vocab, [&](int, float v) {
      const uint32_t key = float_key(v);
      if ((key & mask) == prefix) {
        const unsigned bucket = (key >> shift) & 255u;
        const unsigned peers = __match_any_sync(__activemask(), bucket);
        if (__ffs(peers) - 1 == lane) atomicAdd(&hist[bucket], (unsigned)__popc(peers));
      }
    });
    __syncthreads();
    {
      // thread t < 256 looks at bucket 255 - t: the bucket that holds the k-th largest is the one whose count, added
      // to the counts of the buckets above it, first reaches what is still wanted (one thread walking the 256
      // buckets cost 4 us a pass)
      const int b = 255 - tid;
      const unsigned cnt = tid < 256 ? hist[b] : 0u;
      const unsigned remaining = sh_remaining;
      unsigned all;
      const unsigned above = block_excl_scan(cnt, u_scratch, &all);
      if (tid < 256 && above < remaining && remaining <= above + cnt) {
        sh_prefix = prefix | ((unsigned)b << shift);
        sh_remaining = remaining - above;   // how many of the k lie in the chosen bucket
        sh_equal_total = cnt;               // after the last pass: how many logits equal the k-th largest
      }
    }
    __syncthreads();
  }
  const uint32_t kth_key = sh_prefix;       // key of the k-th largest logit
  const unsigned n_equal_wanted = sh_remaining;
  // gather: everything above the k-th key, then the lowest ids among those equal to it.  When all
  // the equal ones are wanted (no tie straddles the cut) they are gathered in the same pass.
  const bool take_all_equal = sh_equal_total == n_equal_wanted;
  if (tid == 0) sh_count = 0;
  __syncthreads();
  for_each_logit(row, vocab, [&](int i, float v) {
    const uint32_t key = float_key(v);
    if (key > kth_key || (take_all_equal && key == kth_key)) {
      const unsigned slot = atomicAdd(&sh_count, 1u);
      cand_v[slot] = v;
      cand_i[slot] = i;
    }
  });
  __syncthreads();
  if (!take_all_equal) {
    // a tie straddles the cut: thread t counts the equal ones among its contiguous ids, the counts are summed in
    // thread order, and the first n_equal_wanted of them in id order are taken
    const unsigned above = sh_count;
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int b = min(vocab, tid * chunk), e = min(vocab, b + chunk);
    unsigned mine = 0;
    for (int i = b; i < e; i++) mine += float_key(ld_fresh(row + i)) == kth_key;
    unsigned all;
    unsigned rank = block_excl_scan(mine, u_scratch, &all);
    for (int i = b; i < e && rank < n_equal_wanted; i++) {
      const float v = ld_fresh(row + i);
      if (float_key(v) == kth_key) { cand_v[above + rank] = v; cand_i[above + rank] = i; rank++; }
    }
    __syncthreads();
    if (tid == 0) sh_count = above + n_equal_wanted;
    __syncthreads();
  }
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
  // weights of the candidates, then (one warp, lane l holding the 16 consecutive candidates from 16 l on, sums
  // in float64): their total, the top-p cut over the normalised weights, and the draw among what is kept
  const float top = cand_v[0];
  for (int i = tid; i < SAMPLE_CAND_MAX; i += blockDim.x) cand_e[i] = i < n_cand ? expf((cand_v[i] - top) * inv_t) : 0.f;
  __syncthreads();
  if (warp != 0) return;
  draw_from_candidates(cand_v, cand_i, cand_e, n_cand, tp, u, r, ids, values);
}

// ---------------------------------------------------------------- the same, a row cut over 32 blocks
// One block per row reads the row five or six times and is bound by what one SM draws from L2: 36 us with a
// temperature alone, 100 to 130 us with filters, whatever the batch.  Here a row is cut into SS_SPLITS stretches
// of consecutive ids.  A block takes one stretch into shared memory and leaves: its largest logit (greedy rows,
// and the row's maximum); without filters, the sums of its weights exp((l - its maximum) / T) over eight
// sub-stretches; with filters, its own min(k, SS_KEEP) largest logits in ascending id order, and the key of the
// last of them.  The block that finishes last (a counter per row tells; no block waits) does the rest from those
// leavings: the row's maximum, then either the sub-stretch that holds the draw and a walk through it, or the k
// largest of the 32 lists (in shared memory), sorted, cut by top-p and drawn from, as above.
//
// A stretch leaves at most SS_KEEP candidates, although any number of the row's k largest could lie in one
// stretch.  So the last block checks: a stretch that kept fewer than k has nothing hidden among the row's k largest
// if the key of its last kept candidate is below the key of the k-th largest of all lists.  With 128,256 logits
// and k = 512 the k-th largest is the 99.6th percentile of the row, a stretch's 64th largest the 98.4th of its
// own, so the check holds unless the large logits crowd in one stretch; when it does not hold the row is marked
// and the one-block kernel, launched behind this one for marked rows only, does the row by itself.
// Sums are taken in an order that depends on the sizes only.
#define SS_SPLITS 32
#define SS_THREADS 256
#define SS_WARPS (SS_THREADS / 32)
static_assert(SS_THREADS == 256, "one thread per bucket of the radix passes");
#define SS_CHUNK_MAX 8192
#define SS_KEEP 64
#define SS_LIST_MAX (SS_SPLITS * SS_KEEP)

struct SsScratch {               // in global memory, per row (counters zeroed once; every launch leaves them at zero)
  float* part_v; int* part_i;    // [rows][SS_SPLITS] largest logit of the stretch and its id
  float* part_e;                 // [rows][SS_SPLITS][SS_WARPS] sums of the sub-stretches' weights (stretch's own maximum)
  unsigned* part_key;            // [rows][SS_SPLITS] key of the stretch's last kept candidate
  float* cand_v; int* cand_i;    // [rows][SS_LIST_MAX]: the stretches' lists one after another
  unsigned* counters;            // [rows]
  int* redo;                     // [rows] 1: the one-block kernel does this row
};

// Among n values in ascending id order (val(j), id(j)), the k largest, the lowest ids first among equals at the
// cut, written in ascending id order to out_v / out_i.  Returns how many (min(k, n)); *kth_key gets the key of the
// smallest of them (0 if all n were taken).  Every thread of the block calls it.  hist: 256 words, sh: 2,
// w_scratch: 2 * SS_WARPS.
template <typename Val, typename Id>
__device__ int select_in_order(Val val, Id id, int n, int k, float* out_v, int* out_i, unsigned* hist, unsigned* sh,
                               unsigned* w_scratch, unsigned* w_scratch33, uint32_t* kth_key) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (k >= n) {
    for (int j = tid; j < n; j += SS_THREADS) { out_v[j] = val(j); out_i[j] = id(j); }
    __syncthreads();
    *kth_key = 0u;
    return n;
  }
  if (tid == 0) { sh[0] = 0; sh[1] = (unsigned)k; }
  __syncthreads();
  for (int pass = 0; pass < 4; pass++) {          // radix select, 8 bits a pass from the top
    const int shift = 24 - 8 * pass;
    hist[tid] = 0;                                 // (SS_THREADS == 256 buckets)
    __syncthreads();
    const unsigned prefix = sh[0];
    const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int j = tid; j < n; j += SS_THREADS) {
      const uint32_t key = float_key(val(j));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    {
      // thread t looks at bucket 255 - t: the bucket that holds the k-th largest is the one whose count, added to
      // the counts of the buckets above it, first reaches what is still wanted
      const int b = 255 - tid;
      const unsigned cnt = hist[b];
      const unsigned remaining = sh[1];
      unsigned all;
      const unsigned above = block_excl_scan(cnt, w_scratch33, &all);
      if (above < remaining && remaining <= above + cnt) {
        sh[0] = prefix | ((unsigned)b << shift);
        sh[1] = remaining - above;                 // how many of the k lie in the chosen bucket
      }
    }
    __syncthreads();
  }
  const uint32_t kth = sh[0];
  const unsigned want_eq = sh[1];                  // how many of those equal to the k-th largest are taken
  // in id order, 256 ids a round: an element's rank among the equal ones and its place in the output are counts of
  // the elements before it (votes inside a warp, the warps' counts through shared memory)
  unsigned eq_before = 0, out_before = 0;
  const unsigned lt = (1u << lane) - 1u;
  for (int j0 = 0; j0 < n; j0 += SS_THREADS) {
    const int j = j0 + tid;
    const float v = j < n ? val(j) : 0.f;
    const uint32_t key = j < n ? float_key(v) : 0u;
    const bool eq = j < n && key == kth;
    const unsigned eq_votes = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) w_scratch[warp] = (unsigned)__popc(eq_votes);
    __syncthreads();
    unsigned eq_rank = eq_before + (unsigned)__popc(eq_votes & lt), eq_round = 0;
    for (int w = 0; w < SS_WARPS; w++) { const unsigned c = w_scratch[w]; if (w < warp) eq_rank += c; eq_round += c; }
    const bool take = j < n && (key > kth || (eq && eq_rank < want_eq));
    const unsigned take_votes = __ballot_sync(0xffffffffu, take);
    if (lane == 0) w_scratch[SS_WARPS + warp] = (unsigned)__popc(take_votes);
    __syncthreads();
    unsigned place = out_before + (unsigned)__popc(take_votes & lt), take_round = 0;
    for (int w = 0; w < SS_WARPS; w++) { const unsigned c = w_scratch[SS_WARPS + w]; if (w < warp) place += c; take_round += c; }
    if (take) { out_v[place] = v; out_i[place] = id(j); }
    eq_before += eq_round;
    out_before += take_round;
  }
  __syncthreads();
  *kth_key = kth;
  return k;
}

__global__ void __launch_bounds__(SS_THREADS)
sample_split_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
                    const int* __restrict__ top_k, const float* __restrict__ top_p,
                    const float* __restrict__ uniform, int* __restrict__ ids, float* __restrict__ values,
                    const SsScratch Q) {
  extern __shared__ __align__(16) float lv[];      // the stretch's logits; in the last block, the lists: values, ids
  __shared__ MaxIdx mi_scratch[33];
  __shared__ float f_scratch[SS_THREADS + 2];
  __shared__ unsigned w_scratch[2 * SS_WARPS];
  __shared__ unsigned u_scratch[33];
  __shared__ unsigned hist[256];
  __shared__ unsigned sh[2];
  __shared__ float cand_e[SAMPLE_CAND_MAX];
  __shared__ float cand_v[SAMPLE_CAND_MAX];
  __shared__ int cand_i[SAMPLE_CAND_MAX];
  __shared__ int sh_owner;
  __shared__ bool last;

  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, sp = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const bool sampled = temp > 0.f;
  const float inv_t = sampled ? 1.0f / temp : 0.f;
  int k = top_k[r];
  const float tp = top_p[r];
  const bool filtered = sampled && ((k > 0) || (tp < 1.0f));
  if (k <= 0 || k > SAMPLE_CAND_MAX) k = SAMPLE_CAND_MAX;
  if (k > vocab) k = vocab;
  const int k1 = min(k, SS_KEEP);                  // what a stretch keeps
  const int chunk = (vocab + SS_SPLITS - 1) / SS_SPLITS;
  auto stretch_len = [&](int s2) { return min(vocab, (s2 + 1) * chunk) - min(vocab, s2 * chunk); };
  const int b0 = min(vocab, sp * chunk), n = stretch_len(sp);
  const int part = r * SS_SPLITS + sp;
  // the sub-stretch of warp w: ids [w sub, (w+1) sub) of the stretch
  const int sub = (chunk + SS_WARPS - 1) / SS_WARPS;

  // ---- this block's stretch
  for (int j = tid; j < n; j += SS_THREADS) lv[j] = ld_fresh(row + b0 + j);
  __syncthreads();
  MaxIdx mine{-INFINITY, 0x7fffffff};
  for (int j = tid; j < n; j += SS_THREADS) {
    const float v = lv[j];
    if (v > mine.v) { mine.v = v; mine.i = b0 + j; }              // ascending ids per thread: the first of equals stays
  }
  const MaxIdx local = block_argmax(mine, mi_scratch);
  if (tid == 0) { Q.part_v[part] = local.v; Q.part_i[part] = local.i; }
  if (sampled && !filtered) {
    float e = 0.f;
    if (local.i != 0x7fffffff)
      for (int j = warp * sub + lane; j < min(n, (warp + 1) * sub); j += 32) e += expf((lv[j] - local.v) * inv_t);
    e = warp_sum(e);
    if (lane == 0) Q.part_e[(size_t)part * SS_WARPS + warp] = e;
  } else if (filtered) {
    int off = 0;                                    // what the stretches before this one leave
    for (int s2 = 0; s2 < sp; s2++) off += min(k1, stretch_len(s2));
    uint32_t kth;
    select_in_order([&](int j) { return lv[j]; }, [&](int j) { return b0 + j; }, n, k1,
                    Q.cand_v + (size_t)r * SS_LIST_MAX + off, Q.cand_i + (size_t)r * SS_LIST_MAX + off, hist, sh,
                    w_scratch, u_scratch, &kth);
    if (tid == 0) Q.part_key[part] = kth;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) last = atomicAdd(&Q.counters[r], 1u) == SS_SPLITS - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();

  // ---- the block that finished last: the row's maximum (the lowest id among equals: stretches are in id order)
  if (warp == 0) {
    MaxIdx t{-INFINITY, 0x7fffffff};
    if (lane < SS_SPLITS) { t.v = __ldcg(Q.part_v + r * SS_SPLITS + lane); t.i = __ldcg(Q.part_i + r * SS_SPLITS + lane); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other;
      other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, other);
    }
    if (lane == 0) {
      if (t.i == 0x7fffffff) { t.i = 0; t.v = ld_fresh(row + 0); }   // every logit is -inf or NaN: index 0
      mi_scratch[32] = t;
      Q.counters[r] = 0;
      Q.redo[r] = 0;
    }
  }
  __syncthreads();
  const MaxIdx best = mi_scratch[32];
  if (!sampled) {
    if (tid == 0) { ids[r] = best.i; if (values) values[r] = best.v; }
    return;
  }
  const float u = uniform[r];

  if (!filtered) {
    // thread t: sub-stretch t % 8 of stretch t / 8; their sums brought to the row's maximum, added in id order
    const int s_of = tid / SS_WARPS;
    const bool any = __ldcg(Q.part_i + r * SS_SPLITS + s_of) != 0x7fffffff;
    const float m_s = __ldcg(Q.part_v + r * SS_SPLITS + s_of);
    const float scale = any ? expf((m_s - best.v) * inv_t) : 0.f;
    const float w = any ? __ldcg(Q.part_e + (size_t)r * SS_SPLITS * SS_WARPS + tid) * scale : 0.f;
    float total;
    const float before = block_excl_scan(w, f_scratch, &total);
    const float target = u * total;
    if (tid == 0) sh_owner = 0x7fffffff;
    __syncthreads();
    // the first sub-stretch whose running sum passes the draw
    if (target < before + w) atomicMin(&sh_owner, tid);
    __syncthreads();
    const int owner = sh_owner;
    if (owner == 0x7fffffff) {                         // rounding left none: the last id
      if (tid == 0) { ids[r] = vocab - 1; if (values) values[r] = ld_fresh(row + (vocab - 1)); }
      return;
    }
    if (tid == owner) { f_scratch[SS_THREADS] = before; f_scratch[SS_THREADS + 1] = scale; mi_scratch[0].v = m_s; }
    __syncthreads();
    if (warp != 0) return;
    const float carry0 = f_scratch[SS_THREADS], scale_o = f_scratch[SS_THREADS + 1], m_o = mi_scratch[0].v;
    const int so = owner / SS_WARPS, wo = owner % SS_WARPS;
    const int sb = min(vocab, so * chunk), sn = stretch_len(so);
    const int b = sb + min(sn, wo * sub), e = sb + min(sn, (wo + 1) * sub);
    float carry = carry0;
    int pick = e - 1;                                  // rounding left no id in the sub-stretch: its last
    for (int base = b; base < e; base += 4 * 32) {
      float x[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int i = base + 32 * j + lane;
        x[j] = i < e ? expf((ld_fresh(row + i) - m_o) * inv_t) * scale_o : 0.f;
      }
      bool found = false;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (!found) {
          const float incl = carry + warp_incl_scan(x[j]);
          const unsigned hit = __ballot_sync(0xffffffffu, target < incl && base + 32 * j + lane < e);
          if (hit) { pick = base + 32 * j + __ffs(hit) - 1; found = true; }
          carry = __shfl_sync(0xffffffffu, incl, 31);
        }
      }
      if (found) break;
    }
    if (lane == 0) { ids[r] = pick; if (values) values[r] = ld_fresh(row + pick); }
    return;
  }

  // ---- filtered: the lists, one after another (ascending ids), into shared memory; the k largest of them
  int n_list = 0;
  for (int s2 = 0; s2 < SS_SPLITS; s2++) n_list += min(k1, stretch_len(s2));
  int* li = reinterpret_cast<int*>(lv + SS_LIST_MAX);
  for (int j = tid; j < n_list; j += SS_THREADS) {
    lv[j] = __ldcg(Q.cand_v + (size_t)r * SS_LIST_MAX + j);
    li[j] = __ldcg(Q.cand_i + (size_t)r * SS_LIST_MAX + j);
  }
  __syncthreads();
  uint32_t kth;
  const int n_cand = select_in_order([&](int j) { return lv[j]; }, [&](int j) { return li[j]; }, n_list, k, cand_v,
                                     cand_i, hist, sh, w_scratch, u_scratch, &kth);
  // a stretch that kept fewer than k of its ids: is anything it did not keep among the row's k largest?
  if (tid == 0) sh_owner = 0;
  __syncthreads();
  if (tid < SS_SPLITS && k1 < k && stretch_len(tid) > k1) {
    const uint32_t t_s = __ldcg(Q.part_key + r * SS_SPLITS + tid);
    if (n_cand < k || t_s >= kth) sh_owner = 1;        // (fewer candidates than k in all: the lists do not hold k)
  }
  __syncthreads();
  if (sh_owner) {
    if (tid == 0) Q.redo[r] = 1;
    return;
  }
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
          const bool up = (i & size) == 0;
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
  const float top = cand_v[0];
  for (int i = tid; i < SAMPLE_CAND_MAX; i += blockDim.x) cand_e[i] = i < n_cand ? expf((cand_v[i] - top) * inv_t) : 0.f;
  __syncthreads();
  if (warp != 0) return;
  draw_from_candidates(cand_v, cand_i, cand_e, n_cand, tp, u, r, ids, values);
}

// scratch (optional, all eight or none): see SsScratch; with it, rows of 8,192 to 262,144 logits are cut over 32
// blocks each, and the one-block kernel runs behind for the rows that were marked.
STRATUM_EXPORT int stratum_sample(const float* logits, int ld, int n_rows, int vocab, const float* temperature,
                                  const int* top_k, const float* top_p, const float* uniform, int* ids,
                                  float* values, float* part_v, int* part_i, float* part_e, unsigned* part_key,
                                  float* cand_v, int* cand_i, unsigned* counters, int* redo, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (vocab < 1) return STRATUM_ERR_SHAPE;
  if (part_v && part_i && part_e && part_key && cand_v && cand_i && counters && redo && vocab >= 8192 &&
      vocab <= SS_SPLITS * SS_CHUNK_MAX) {
    const size_t chunk_bytes = (size_t)((vocab + SS_SPLITS - 1) / SS_SPLITS) * sizeof(float);
    const size_t list_bytes = (size_t)SS_LIST_MAX * (sizeof(float) + sizeof(int));
    const size_t smem = chunk_bytes > list_bytes ? chunk_bytes : list_bytes;
    SsScratch Q{part_v, part_i, part_e, part_key, cand_v, cand_i, counters, redo};
    int st = launch_pdl(sample_split_kernel, dim3(n_rows, SS_SPLITS), SS_THREADS, smem, stream, logits, ld, vocab,
                        temperature, top_k, top_p, uniform, ids, values, Q);
    if (st != 0) return st;
    return launch_pdl(sample_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, top_k, top_p,
                      uniform, ids, values, (const int*)redo);
  }
  return launch_pdl(sample_kernel, n_rows, SAMPLE_THREADS, 0, stream, logits, ld, vocab, temperature, top_k, top_p,
                    uniform, ids, values, (const int*)nullptr);
}

// ---------------------------------------------------------------- feeding picked ids back on the device
// ids[i] = prev[feed[i]] where feed[i] >= 0; elsewhere ids[i] stays what the host wrote.  It lets the next decode
// step be launched before the host has read what this one picked (the reference queues its decode steps on the
// GPU the same way, with the token ring on the device: stratum/native/stratum_arch_llama.inc.c:1992-2030).
__global__ void feed_ids_kernel(int* __restrict__ ids, const int* __restrict__ feed, const int* prev, int n) {
  pdl_trigger();
  pdl_wait();                                      // `prev` is the work of the step before
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int f = feed[i];
  if (f >= 0) ids[i] = __ldcg(prev + f);
}

STRATUM_EXPORT int stratum_feed_ids(int* ids, const int* feed, const int* prev, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  return launch_pdl(feed_ids_kernel, (n + 127) / 128, 128, 0, stream, ids, feed, prev, n);
}

