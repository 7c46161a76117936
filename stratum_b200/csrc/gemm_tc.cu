// y = x W^T (+ bias) on the 5th-generation tensor cores: TMA-fed, tcgen05.mma into TMEM, persistent.
//
// W is row-major [N][K] as stored in the file and x is row-major [M][K], so both operands are
// "K-major" and y[m][n] = sum_k x[m][k] W[n][k] (stratum/native/stratum_linear.h:491-507) needs no
// transpose anywhere.  Each CTA owns one SM and walks over output tiles of 128 x BN:
//
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a 128 x 64
//            tile of x and a BN x 64 tile of W per k-block into a ring of shared-memory stages;
//   warp 1   allocates tensor memory; one lane issues four tcgen05.mma (128 x BN x 16, bf16 in,
//            float32 accumulate) per k-block, then tcgen05.commit to hand the stage back, and after
//            the last k-block a commit that tells the epilogue the accumulator is complete;
//   warps 2-5 the epilogue: tcgen05.ld the accumulator (lane = output row, 32 columns at a time),
//            add bias, and store bf16 / add into the float32 residual stream / store float32 /
//            apply SwiGLU to column pairs.  Two accumulators (2 x BN columns of TMEM) let the
//            epilogue of one tile overlap the k-loop of the next.
//
// Tiles that would form a last, partly filled wave are cut along k and shared by all CTAs (see TcSchedule).
// Further down: the same on pairs of CTAs (tcgen05.mma.cta_group::2, 256-row tiles) for prompts; for up to 128
// rows of x the stream-K form with the roles of x and W exchanged; and for up to 16 rows and few tiles the
// form that shares k inside a cluster and adds the partial tiles through distributed shared memory.
// stratum_gemm_tc at the end chooses among them from the shapes.
//
// Every wait on an mbarrier is bounded.  If one runs out, the kernel records where in a status
// word, tells its other warps through shared memory, lets copies in flight land, frees its tensor
// memory and returns; the host turns the status into an error.  No wait can hang the GPU.
#include "tc_common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

static int g_last_launches = 0;       // kernels the last stratum_gemm_tc call launched (for launch counting)
static int g_last_form = 0;           // and the form it took: 1 tiles, 2 tiles on pairs of CTAs, 3 stream-K,
                                      // 4 + 16 * cluster size: k shared inside clusters, 5 pairs that share
                                      // their left-over tiles along k (for tests)

// Work an epilogue may do beyond its basic form.  Every part is off while its pointer is null.
//
// (1) norm_ss: the rows of x were handed over by a norm that did not write them out in full: x holds r * gain
//     (r: the residual row), and the row's factor 1 / sqrt(sum r^2 / size + eps) is applied here, to the product.
//     norm_ss[p * norm_ld + m], p < norm_parts, are partial sums of r^2 of row m; they are added in the order of p.
// (2) emit_x (epilogue 4, which adds into the float32 residual stream as epilogue 1 does): for the norm that
//     follows, also write emit_x[m][n] = bf16(r * emit_gain[n]) for the new residual values r, and
//     emit_ss[part * emit_ld + m] = the sum of r^2 over this tile's columns, part being the tile's number along N
//     (tiles of 128 columns in the forms for few rows; every (part, m) is written exactly once).
// (3) epilogue 5: the columns are the query heads, then the key heads, then the value heads of an attention layer,
//     the two dimensions of a rotated pair being neighbours.  Queries are rotated and stored to `out`; keys are
//     rotated and written, and values written, to the row's place in the paged cache (rows whose token_seq is
//     negative write nothing there).  rope_cs[m][k] = (cos, sin) of row m's angle for pair k; null: no rotation.
struct EpiExtra {
  const float* norm_ss;
  bf16* emit_x; const float* emit_gain; float* emit_ss;
  const float2* rope_cs; const int* token_pos; const int* token_seq; const int* block_table;
  bf16* k_cache; bf16* v_cache;
  int norm_parts, norm_ld; float norm_size, norm_eps;
  int emit_ldx, emit_ld;
  int rope_pairs, bt_stride, n_q, n_kv, head_dim, page_tokens, write_cache;
  int reserved;
};

__device__ __forceinline__ float epi_row_scale(const EpiExtra& X, int m) {
  // sixteen loads in flight at a time (one after the other they would cost a trip to L2 each), added in order
  float t = 0.f;
  for (int p0 = 0; p0 < X.norm_parts; p0 += 16) {
    float a[16];
#pragma unroll
    for (int u = 0; u < 16; u++)
      a[u] = (p0 + u < X.norm_parts) ? __ldcg(X.norm_ss + (size_t)(p0 + u) * X.norm_ld + m) : 0.f;
#pragma unroll
    for (int u = 0; u < 16; u++) t += a[u];
  }
  return 1.0f / sqrtf(t / X.norm_size + X.norm_eps);
}

// Element offset, in the key or value cache, of (the page of row m's position, kv head 0, the position's place in
// the page, dimension 0); -1 if the row writes nothing there.  Cache layout: [pages][kv heads][page_tokens][head_dim].
__device__ __forceinline__ long long epi_cache_row(const EpiExtra& X, int m) {
  const int seq = X.token_seq[m];
  if (seq < 0 || !X.write_cache) return -1;
  const int pos = X.token_pos[m];
  const int page = X.block_table[(size_t)seq * X.bt_stride + pos / X.page_tokens];
  return ((long long)page * X.n_kv * X.page_tokens + (pos % X.page_tokens)) * (long long)X.head_dim;
}

struct TcParams {
  const float* bias;
  void* out;
  int* status;        // 0, or a code of where a wait ran out
  int M, N, K;        // logical sizes of y = x W^T: x [M][K], W [N][K]
  int ldo;
  int split;          // 1: the tiles left over after the full waves are cut along k and shared by all CTAs
  float* scratch;     // [gridDim.x][2][BN][128] float32: up to two partial tiles per CTA (split only)
  EpiExtra X;
};

// What the thread that owns output row m (one token) carries through the columns of a tile.
struct EpiRow {
  float scale;        // factor of a handed-over norm (1 if none)
  float ss;           // epilogue 4: sum of squares of the row's new residual values in this tile
  long long cache;    // epilogue 5: epi_cache_row
};
template <int EPI>
__device__ __forceinline__ EpiRow epi_row_begin(const EpiExtra& X, int m, int M) {
  EpiRow r;
  r.scale = (X.norm_ss && m < M) ? epi_row_scale(X, m) : 1.0f;
  r.ss = 0.f;
  r.cache = (EPI == 5 && m < M) ? epi_cache_row(X, m) : -1;
  return r;
}
template <int EPI>
__device__ __forceinline__ void epi_row_end(const EpiExtra& X, const EpiRow& r, int part, int m, int M) {
  if (EPI == 4 && X.emit_ss && m < M) X.emit_ss[(size_t)part * X.emit_ld + m] = r.ss;
}

template <int BN, int STAGES>
struct TcSmem {
  alignas(1024) bf16 a[STAGES][TC_BM * TC_BK];
  alignas(1024) bf16 b[STAGES][BN * TC_BK];
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Output row m, columns col0 .. col0 + CW - 1 (contiguous in memory): the row's factor, bias, then the epilogue.
// EPI: 0 store bf16, 1 add into float32, 2 store float32, 3 SwiGLU pairs -> bf16, 4 as 1 and hand on to the next
// norm, 5 queries / keys / values of an attention layer (see EpiExtra).
template <int EPI, int CW>
__device__ __forceinline__ void tc_store_chunk(const TcParams& P, int m, int col0, float (&v)[CW], EpiRow& R) {
  if (R.scale != 1.0f) {
#pragma unroll
    for (int j = 0; j < CW; j++) v[j] *= R.scale;
  }
  if (P.bias) {
#pragma unroll
    for (int j = 0; j < CW; j++)
      if (col0 + j < P.N) v[j] += P.bias[col0 + j];
  }
  const bool whole = col0 + CW <= P.N;
  if (EPI == 5) {
    // (the host checked: head_dim % CW == 0, so a chunk lies inside one head; N % CW == 0; 16-byte aligned rows)
    if (!whole) return;
    const EpiExtra& X = P.X;
    const int h = col0 / X.head_dim, d0 = col0 - h * X.head_dim;
    const bool is_q = h < X.n_q, is_k = !is_q && h < X.n_q + X.n_kv;
    if ((is_q || is_k) && X.rope_cs) {
      const float2* cs = X.rope_cs + (size_t)m * X.rope_pairs + (d0 >> 1);
#pragma unroll
      for (int j = 0; j < CW; j += 2) {
        if ((d0 + j) >> 1 < X.rope_pairs) {
          const float2 f = __ldcg(cs + (j >> 1));
          const float x0 = v[j], x1 = v[j + 1];
          v[j] = x0 * f.x - x1 * f.y;
          v[j + 1] = x0 * f.y + x1 * f.x;
        }
      }
    }
    bf16* o;
    if (is_q) {
      o = (bf16*)P.out + (size_t)m * P.ldo + col0;
    } else {
      if (R.cache < 0) return;
      const int kvh = is_k ? h - X.n_q : h - X.n_q - X.n_kv;
      o = (is_k ? X.k_cache : X.v_cache) + R.cache + (long long)kvh * X.page_tokens * X.head_dim + d0;
    }
#pragma unroll
    for (int q = 0; q < CW / 8; q++) {
      uint32_t w4[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        __nv_bfloat162 pr = __floats2bfloat162_rn(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
        w4[e] = *reinterpret_cast<uint32_t*>(&pr);
      }
      reinterpret_cast<uint4*>(o)[q] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
  } else if (EPI == 3) {
    bf16* o = (bf16*)P.out + (size_t)m * P.ldo + (col0 >> 1);
    uint32_t packed[CW / 4];
#pragma unroll
    for (int j = 0; j < CW; j += 4) {
      float a[2];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const float gate = __bfloat162float(__float2bfloat16_rn(v[j + 2 * e]));
        const float up = __bfloat162float(__float2bfloat16_rn(v[j + 2 * e + 1]));
        a[e] = gate / (1.0f + __expf(-gate)) * up;
      }
      __nv_bfloat162 pr = __floats2bfloat162_rn(a[0], a[1]);
      packed[j / 4] = *reinterpret_cast<uint32_t*>(&pr);
    }
    if (whole && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < CW / 16; q++)
        reinterpret_cast<uint4*>(o)[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < CW; j += 2)
        if (col0 + j + 1 < P.N) {
          const __nv_bfloat162 pr = *reinterpret_cast<__nv_bfloat162*>(&packed[j / 4]);
          o[j >> 1] = (j & 2) ? pr.y : pr.x;
        }
    }
  } else if (EPI == 0) {
    bf16* o = (bf16*)P.out + (size_t)m * P.ldo + col0;
    if (whole && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < CW / 8; q++) {
        uint32_t w4[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          __nv_bfloat162 pr = __floats2bfloat162_rn(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
          w4[e] = *reinterpret_cast<uint32_t*>(&pr);
        }
        reinterpret_cast<uint4*>(o)[q] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < CW; j++)
        if (col0 + j < P.N) o[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* o = (float*)P.out + (size_t)m * P.ldo + col0;
    constexpr bool ADD = EPI == 1 || EPI == 4;
    if (whole && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
      for (int q = 0; q < CW / 4; q++) {
        float4 w4 = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        if (ADD) {
          const float4 old = ld_fresh(reinterpret_cast<const float4*>(o) + q);
          w4.x += old.x; w4.y += old.y; w4.z += old.z; w4.w += old.w;
        }
        reinterpret_cast<float4*>(o)[q] = w4;
        if (EPI == 4) { v[4 * q] = w4.x; v[4 * q + 1] = w4.y; v[4 * q + 2] = w4.z; v[4 * q + 3] = w4.w; }
      }
    } else {
#pragma unroll
      for (int j = 0; j < CW; j++) {
        if (col0 + j < P.N) { v[j] = ADD ? ld_fresh(o + j) + v[j] : v[j]; o[j] = v[j]; }
        else v[j] = 0.f;
      }
    }
    if (EPI == 4 && P.X.emit_x) {
      // v now holds the new residual values: their squares for the norm's sum, and r * gain in bf16 for the
      // product behind the norm
      bf16* e = P.X.emit_x + (size_t)m * P.X.emit_ldx + col0;
#pragma unroll
      for (int j = 0; j < CW; j++) R.ss = fmaf(v[j], v[j], R.ss);
      if (whole && ((reinterpret_cast<uintptr_t>(e) & 15) == 0)) {
#pragma unroll
        for (int q = 0; q < CW / 8; q++) {
          uint32_t w4[4];
#pragma unroll
          for (int k = 0; k < 4; k++) {
            const int j = 8 * q + 2 * k;
            __nv_bfloat162 pr = __floats2bfloat162_rn(v[j] * __ldg(P.X.emit_gain + col0 + j),
                                                      v[j + 1] * __ldg(P.X.emit_gain + col0 + j + 1));
            w4[k] = *reinterpret_cast<uint32_t*>(&pr);
          }
          reinterpret_cast<uint4*>(e)[q] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CW; j++)
          if (col0 + j < P.N) e[j] = __float2bfloat16_rn(v[j] * P.X.emit_gain[col0 + j]);
      }
    }
  }
}

// Output row m, columns n .. n+3 (four neighbours of one row): bias, then the epilogue (PT: TcParams or SkParams).
template <int EPI, typename PT>
__device__ __forceinline__ void fixup_store(const PT& P, int m, int n, float4 v) {
  float e[4] = {v.x, v.y, v.z, v.w};
  if (P.bias) {
#pragma unroll
    for (int j = 0; j < 4; j++) if (n + j < P.N) e[j] += P.bias[n + j];
  }
  if (EPI == 3) {                                   // (gate, up) pairs: n even
    bf16* o = (bf16*)P.out + (size_t)m * P.ldo + (n >> 1);
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      if (n + j + 1 < P.N) {
        const float g = __bfloat162float(__float2bfloat16_rn(e[j])), u = __bfloat162float(__float2bfloat16_rn(e[j + 1]));
        o[j >> 1] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
      }
    }
    return;
  }
  const size_t idx = (size_t)m * P.ldo + n;
  const bool wide = (n + 3 < P.N) && ((idx & 3) == 0);
  if (EPI == 0) {
    bf16* o = (bf16*)P.out + idx;
    if (wide && ((reinterpret_cast<uintptr_t>(o) & 7) == 0)) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(e[0], e[1]), hi = __floats2bfloat162_rn(e[2], e[3]);
      uint2 u; u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(o) = u;
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) if (n + j < P.N) o[j] = __float2bfloat16_rn(e[j]);
    }
  } else {
    float* o = (float*)P.out + idx;
    if (wide && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
      float4 r = make_float4(e[0], e[1], e[2], e[3]);
      if (EPI == 1 || EPI == 4) { const float4 old = __ldcg(reinterpret_cast<const float4*>(o)); r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w; }
      *reinterpret_cast<float4*>(o) = r;
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (n + j < P.N) o[j] = (EPI == 1 || EPI == 4) ? ld_fresh(o + j) + e[j] : e[j];
    }
  }
}

// The work of one CTA as a list of items (tile, k-blocks [kb0, kb1)), the same list for its three roles.
//
// Whole tiles first: blockIdx.x, blockIdx.x + G, ...  Consecutive CTAs take consecutive x tiles of the same W
// tile, so that a wave shares W in L2.  With `split`, the R = n_tiles % G tiles that would form a last, partly
// empty wave are not given to R of the CTAs: their R * n_kb k-blocks are shared evenly, CTA c taking the stretch
// [c U / G, (c+1) U / G) of them, which is the end of one tile and/or the beginning of the next (or a whole tile).
// A piece that is not a whole tile is written to scratch as float32 partial sums (slot 0: the tile the stretch
// begins in; slot 1: the next), and a second kernel adds the pieces of each tile in the order of k and runs the
// epilogue.  No CTA waits for another.  The split depends on the shapes and the grid only: results are the same
// from run to run.
struct TcSchedule {
  int n_tiles, n_kb, G, c;
  int R, U, u0, u1, n_seg, n_full, n_whole;
  __device__ __forceinline__ void init(int n_tiles_, int n_kb_, int split, int G_, int c_) {
    n_tiles = n_tiles_; n_kb = n_kb_; G = G_; c = c_;
    R = split ? n_tiles % G : 0;
    n_full = n_tiles - R;
    n_whole = (n_full > c) ? (n_full - c + G - 1) / G : 0;       // whole tiles of this CTA
    U = R * n_kb;
    u0 = (int)((long long)c * U / G);
    u1 = (int)((long long)(c + 1) * U / G);
    n_seg = (u1 > u0) ? ((u1 - 1) / n_kb - u0 / n_kb + 1) : 0;
  }
  __device__ __forceinline__ bool item(int i, int& tile, int& kb0, int& kb1, int& slot) const {
    if (i < n_whole) {
      tile = c + i * G; kb0 = 0; kb1 = n_kb; slot = -1;
      return true;
    }
    const int j = i - n_whole;
    if (j >= n_seg) return false;
    const int r = u0 / n_kb + j;
    kb0 = (j == 0) ? u0 - r * n_kb : 0;
    kb1 = min(n_kb, u1 - r * n_kb);
    tile = n_full + r;
    slot = (kb0 == 0 && kb1 == n_kb) ? -1 : (j == 0 ? 0 : 1);
    return true;
  }
};
__device__ __forceinline__ int tc_begin(int c, int G, int U) { return (int)((long long)c * U / G); }
__device__ __forceinline__ int tc_owner(int u, int G, int U) {
  int o = (int)(((long long)u * G) / U);
  while (o + 1 < G && tc_begin(o + 1, G, U) <= u) o++;
  while (o > 0 && tc_begin(o, G, U) > u) o--;
  return o;
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const TcParams P) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = TcSmem<BN, STAGES>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();          // barriers and tensor memory are set up while the kernel before this one finishes
  constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;      // a power of two >= 32
  constexpr uint32_t STAGE_BYTES = (TC_BM + BN) * TC_BK * sizeof(bf16);

  const int tiles_a = (P.M + TC_BM - 1) / TC_BM, tiles_b = (P.N + BN - 1) / BN;
  TcSchedule sched;
  sched.init(tiles_a * tiles_b, (P.K + TC_BK - 1) / TC_BK, P.split, gridDim.x, blockIdx.x);
  volatile int* abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 4); }
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  pdl_wait();             // from here on x, the residual stream and the output may be touched

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      uint32_t it = 0;
      bool ok = true;
      int tile, kb0, kb1, slot;
      for (int i = 0; ok && sched.item(i, tile, kb0, kb1, slot); i++) {
        const int ta = tile % tiles_a, tb = tile / tiles_a;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&S.empty[s], ph ^ 1, abort_flag)) {
            atomicCAS(P.status, 0, 101); S.abort_flag = 1; ok = false; break;
          }
          mbar_expect_tx(&S.full[s], STAGE_BYTES);
          tma_load_2d(&map_a, S.a[s], &S.full[s], kb * TC_BK, ta * TC_BM);
          tma_load_2d(&map_b, S.b[s], &S.full[s], kb * TC_BK, tb * BN);
        }
      }
      if (!ok) {
        // let copies already issued land before this block's shared memory can be given to another block
        for (int i = 0; i < 2000; i++) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(BN);
      uint32_t it = 0;
      bool ok = true;
      int tile, kb0, kb1, slot;
      for (int i = 0; ok && sched.item(i, tile, kb0, kb1, slot); i++) {
        const int buf = i & 1;
        const uint32_t acc_ph = (i >> 1) & 1;
        if (!mbar_wait(&S.acc_empty[buf], acc_ph ^ 1, abort_flag)) {
          atomicCAS(P.status, 0, 102); S.abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&S.full[s], ph, abort_flag)) {
            atomicCAS(P.status, 0, 103); S.abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(S.a[s]), b_addr = smem_u32(S.b[s]);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++) {
            // 16 k-values = 32 bytes further along each 128-byte swizzled row
            umma_bf16(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                      (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&S.empty[s]);           // arrives once the MMAs above have read this stage
        }
        if (ok) umma_commit(&S.acc_full[buf]);  // arrives once the whole accumulator is written
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read: 32*quarter ..
    const int row = quarter * 32 + lane;
    bool ok = true;
    int tile, kb0, kb1, slot;
    for (int i = 0; ok && sched.item(i, tile, kb0, kb1, slot); i++) {
      const int ta = tile % tiles_a, tb = tile / tiles_a;
      const int buf = i & 1;
      const uint32_t acc_ph = (i >> 1) & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&S.acc_full[buf], acc_ph, abort_flag))) {   // (a warp gives up as one)
        if (lane == 0) { atomicCAS(P.status, 0, 104); S.abort_flag = 1; }
        ok = false;
        break;
      }
      tc_fence_after();
      const int m = ta * TC_BM + row;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      constexpr int CW = (BN >= 32) ? 32 : 16;                  // columns per tcgen05.ld
      EpiRow R = epi_row_begin<EPI>(P.X, m, slot >= 0 ? 0 : P.M);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CW) {
        uint32_t r[CW];
        if constexpr (CW == 32) tmem_ld32(taddr + c0, r); else tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
        if (slot >= 0) {
          // a piece of a shared tile: partial sums, [column][row] so that the lanes of a warp write neighbours
          float* part = P.scratch + (((size_t)sched.c * 2 + slot) * BN + c0) * TC_BM + row;
#pragma unroll
          for (int j = 0; j < CW; j++) part[(size_t)j * TC_BM] = __uint_as_float(r[j]);
          continue;
        }
        if (m < P.M) {
          float v[CW];
#pragma unroll
          for (int j = 0; j < CW; j++) v[j] = __uint_as_float(r[j]);
          tc_store_chunk<EPI, CW>(P, m, tb * BN + c0, v, R);
        }
      }
      if (slot < 0) epi_row_end<EPI>(P.X, R, tb, m, P.M);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.acc_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- many rows of x: pairs of CTAs
// The tile kernel above is bound by what an SM can pull out of L2: a 128 x 256 tile needs 48 KB of operands per
// k-block.  Here two CTAs on neighbouring SMs (a cluster of two) compute a 256 x 256 tile together with MMAs that
// span both SMs (cta_group::2, M = 256): each CTA fetches its own 128 rows of x and only HALF of the W tile (128
// rows), 32 KB per k-block for the same arithmetic, and holds its own 128 rows of the accumulator in its TMEM.
//
//   warp 0   in both CTAs: one lane issues the TMA loads of its CTA's halves; the bytes of both CTAs are counted
//            on the leader's (rank 0) `full` barrier;
//   warp 1   both CTAs allocate tensor memory together; the leader's elected lane issues the MMAs for the pair
//            and commits to `empty` (stage free) and `acc_full` in BOTH CTAs (multicast commit);
//   warps 2-5 in both CTAs: epilogue of their CTA's 128 rows; they arrive on the LEADER's `acc_empty`.
//
// No TMA multicast is used.  Every mbarrier wait is bounded as above; the two cluster-wide barriers (after set-up
// and before the tensor memory is freed) are reached by every thread of both CTAs on every path.
template <int STAGES>
struct Tc2Smem {
  alignas(1024) bf16 a[STAGES][TC_BM * TC_BK];     // this CTA's 128 rows of x
  alignas(1024) bf16 b[STAGES][TC_BM * TC_BK];     // this CTA's half of the W tile (up to 128 rows)
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

#define TC2_STAGES 6

// BN: columns of a tile (a multiple of 16, at most 256; each CTA fetches BN / 2 rows of W).  The host picks the
// width whose number of waves times width is least.
template <int EPI, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const TcParams P) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = Tc2Smem<TC2_STAGES>;
  // (the same offset in both CTAs: the dynamic shared memory starts at the same address in every CTA of a kernel)
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  pdl_trigger();
  constexpr int STAGES = TC2_STAGES;
  constexpr uint32_t STAGE_BYTES_PAIR = 2 * (TC_BM + BN / 2) * TC_BK * sizeof(bf16);      // both operands, both CTAs
  const int tiles_m = (P.M + 2 * TC_BM - 1) / (2 * TC_BM), tiles_n = (P.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (P.K + TC_BK - 1) / TC_BK;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  // the pairs' work is scheduled like the CTAs' of the tile kernel: whole tiles, then (P.split) the k-blocks of the
  // tiles of a partly filled last wave spread evenly over all pairs, their pieces going to scratch
  TcSchedule sched;
  sched.init(n_tiles, n_kb, P.split, n_pairs, pair);
  volatile int* abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 8); }   // 4 warps x 2 CTAs
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_2cta(&S.tmem_base, 512);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised and its tensor memory is allocated
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  pdl_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (each CTA its halves)
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      uint32_t it = 0;
      bool ok = true;
      int tile, kb0, kb1, slot;
      for (int i = 0; ok && sched.item(i, tile, kb0, kb1, slot); i++) {
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&S.empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) {
            atomicCAS(P.status, 0, 111); S.abort_flag = 1; ok = false; break;
          }
          const uint32_t full_leader = cluster_map(&S.full[s], 0);
          if (leader) mbar_expect_tx(&S.full[s], STAGE_BYTES_PAIR);
          tma_load_2d_2cta(&map_a, S.a[s], full_leader, kb * TC_BK, tm * 2 * TC_BM + (int)rank * TC_BM);
          tma_load_2d_2cta(&map_b, S.b[s], full_leader, kb * TC_BK, tn * BN + (int)rank * (BN / 2));
        }
      }
      if (!ok) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);   // let copies already issued land
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (the leader, for the pair)
    if (leader) {
      const uint32_t idesc = instr_desc_bf16_m256(BN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      int tile, kb0, kb1, slot;
      for (; ok && sched.item((int)t, tile, kb0, kb1, slot); t++) {
        const int buf = t & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&S.acc_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag))) {
          if (lane == 0) { atomicCAS(P.status, 0, 112); S.abort_flag = 1; }
          ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          if (!__all_sync(0xffffffffu, mbar_wait(&S.full[s], (it / STAGES) & 1, abort_flag))) {
            if (lane == 0) { atomicCAS(P.status, 0, 113); S.abort_flag = 1; }
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(S.a[s]), b_addr = smem_u32(S.b[s]);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < TC_BK / 16; k++)
              umma_bf16_2cta(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                             (kb > kb0 || k > 0) ? 1u : 0u);
            umma_commit_2cta(&S.empty[s], 3);             // the stage is free again, in both CTAs
          }
          __syncwarp();
        }
        if (ok && elect_one()) umma_commit_2cta(&S.acc_full[buf], 3);   // the accumulators of both CTAs are complete
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t acc_empty_leader[2] = {cluster_map(&S.acc_empty[0], 0), cluster_map(&S.acc_empty[1], 0)};
    uint32_t t = 0;
    bool ok = true;
    int tile, kb0, kb1, slot;
    for (; ok && sched.item((int)t, tile, kb0, kb1, slot); t++) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int buf = t & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&S.acc_full[buf], (t >> 1) & 1, abort_flag))) {
        if (lane == 0) { atomicCAS(P.status, 0, 114); S.abort_flag = 1; }
        ok = false;
        break;
      }
      tc_fence_after();
      const int m = tm * 2 * TC_BM + (int)rank * TC_BM + row;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256;
      if (slot >= 0) {
        // a piece of a shared tile: this CTA's 128 rows of partial sums, [column][row] so that the lanes of a warp
        // write neighbours; the second kernel adds the pieces (only tiles of 256 columns are shared)
        float* part = P.scratch + ((((size_t)pair * 2 + slot) * 2 + rank) * BN) * TC_BM + row;
#pragma unroll 1
        for (int c0 = 0; c0 + 32 <= BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) part[(size_t)(c0 + j) * TC_BM] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader[buf]);
        continue;
      }
      EpiRow R = epi_row_begin<EPI>(P.X, m, P.M);
#pragma unroll 1
      for (int c0 = 0; c0 + 32 <= BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        tmem_ld_wait();
        if (m < P.M) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
          tc_store_chunk<EPI, 32>(P, m, tn * BN + c0, v, R);
        }
      }
      if constexpr (BN % 32 != 0) {               // the last 16 columns
        uint32_t r[16];
        tmem_ld16(taddr + (BN / 32) * 32, r);
        tmem_ld_wait();
        if (m < P.M) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]);
          tc_store_chunk<EPI, 16>(P, m, tn * BN + (BN / 32) * 32, v, R);
        }
      }
      epi_row_end<EPI>(P.X, R, tn, m, P.M);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader[buf]);
    }
  }
  // nobody leaves, and nobody frees tensor memory, before both CTAs are through with it and with each other's
  // barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- few rows of x: stream-K
// Decode steps multiply a handful of rows of x by all of W, so the time is the time to read W once, and
// the work must be spread evenly over every SM whatever N is.  The k-blocks of all tiles (128 weight rows
// x 64 k each) form one sequence of tiles*n_kb blocks; CTA c takes the contiguous stretch
// [c*total/G, (c+1)*total/G).  A stretch covers the end of one tile, some whole tiles and the beginning of
// another.  Whole tiles go straight from tensor memory through the epilogue.  A tile shared between CTAs is
// written as float32 partial sums to scratch, and a second, small kernel adds the partial sums of every such
// tile in the order of k (the order of the CTA numbers) and runs the epilogue.  The split depends
// only on the shapes and the grid, never on the rows of x, so a row's result does not depend on its batch.
// W tiles do not depend on earlier kernels and are requested before the programmatic-launch wait.
struct SkParams {
  const float* bias;
  void* out;
  int* status;
  float* scratch;         // [gridDim.x][2][BN][128] float32 partial tiles (first / last tile of a CTA's stretch)
  int M, N, K, ldo;
  int tiles, n_kb, total_kb;
  EpiExtra X;
};

__device__ __forceinline__ int sk_begin(int c, int G, int total) { return (int)((long long)c * total / G); }
__device__ __forceinline__ int sk_owner(int i, int G, int total) {
  int c = (int)((long long)i * G / total);
  while (c + 1 < G && sk_begin(c + 1, G, total) <= i) c++;
  while (c > 0 && sk_begin(c, G, total) > i) c--;
  return c;
}

// Per row of x (a token of the step), in shared memory, for the epilogues of the forms below, whose threads own
// weight rows and meet every token.
struct SkTables {
  float scale[TC_BM];       // factor of a handed-over norm (1 if none)
  long long cache[TC_BM];   // epilogue 5: epi_cache_row (-1: the row writes nothing into the cache)
  float ss[4][TC_BM];       // epilogue 4: per epilogue warp, the sum of squares over its 32 weight rows
};
// (The kernels of these forms are compiled twice, XT = false for products without rows of a handed-over norm and
// without epilogue 5: those neither fill nor read the tables, and pay neither the barrier nor the multiply.)
template <int EPI, int BN>
__device__ __forceinline__ void sk_tables_init(const SkParams& P, SkTables& T, int t0, int stride) {
  for (int t = t0; t < BN; t += stride) {
    T.scale[t] = (P.X.norm_ss && t < P.M) ? epi_row_scale(P.X, t) : 1.0f;
    T.cache[t] = (EPI == 5 && t < P.M) ? epi_cache_row(P.X, t) : -1;
  }
}

// Final values of weight row n for x rows m0 .. m0+CW-1 (one thread per weight row, lanes are neighbours in n).
// Epilogue 4 leaves the squares of the new residual values in v (zero where nothing was written), for the caller
// to add up over the weight rows.
template <int EPI, int CW, bool XT>
__device__ __forceinline__ void sk_store(const SkParams& P, const SkTables& T, int n, int m0, float (&v)[CW]) {
  const bool col_ok = n < P.N;
  const float b = (P.bias && col_ok) ? P.bias[n] : 0.0f;
  if constexpr (XT) {
#pragma unroll
    for (int j = 0; j < CW; j++) v[j] = v[j] * T.scale[m0 + j] + b;
  } else {
#pragma unroll
    for (int j = 0; j < CW; j++) v[j] += b;
  }
  if constexpr (EPI == 1 || EPI == 4) {
    // all loads of the old values first, so that they are in flight together (the compiler may not move a load
    // above the store of another row: it cannot know that the rows do not overlap)
    float old[CW];
#pragma unroll
    for (int j = 0; j < CW; j++)
      old[j] = (col_ok && m0 + j < P.M) ? ld_fresh((const float*)P.out + (size_t)(m0 + j) * P.ldo + n) : 0.0f;
#pragma unroll
    for (int j = 0; j < CW; j++) {
      const bool ok = col_ok && m0 + j < P.M;
      v[j] = ok ? old[j] + v[j] : 0.0f;
      if (ok) ((float*)P.out)[(size_t)(m0 + j) * P.ldo + n] = v[j];
    }
    if (EPI == 4 && P.X.emit_x) {
      const float gain = col_ok ? __ldg(P.X.emit_gain + n) : 0.0f;
#pragma unroll
      for (int j = 0; j < CW; j++) {
        if (col_ok && m0 + j < P.M) P.X.emit_x[(size_t)(m0 + j) * P.X.emit_ldx + n] = __float2bfloat16_rn(v[j] * gain);
        v[j] *= v[j];
      }
    }
  } else if constexpr (EPI == 5) {
    // weight row n is dimension d of head h; its partner in the rotation is the neighbouring row, one lane away
    const EpiExtra& X = P.X;
    const int h = n / X.head_dim, d = n - h * X.head_dim;
    const bool is_q = h < X.n_q, is_k = !is_q && h < X.n_q + X.n_kv;
    const bool rot = col_ok && (is_q || is_k) && X.rope_cs && (d >> 1) < X.rope_pairs;
    const int kvh = is_k ? h - X.n_q : h - X.n_q - X.n_kv;
    bf16* cache = (is_k ? X.k_cache : X.v_cache) + (long long)kvh * X.page_tokens * X.head_dim + d;
#pragma unroll
    for (int j = 0; j < CW; j++) {
      const int m = m0 + j;
      float val = v[j];
      const float partner = __shfl_xor_sync(0xffffffffu, val, 1);
      if (m >= P.M || !col_ok) continue;
      if (rot) {
        const float2 f = __ldcg(X.rope_cs + (size_t)m * X.rope_pairs + (d >> 1));
        val = (d & 1) ? partner * f.y + val * f.x : val * f.x - partner * f.y;
      }
      if (is_q) ((bf16*)P.out)[(size_t)m * P.ldo + n] = __float2bfloat16_rn(val);
      else if (T.cache[m] >= 0) cache[T.cache[m]] = __float2bfloat16_rn(val);
    }
  } else {
#pragma unroll
  for (int j = 0; j < CW; j++) {
    const int m = m0 + j;
    float val = v[j];
    if (EPI == 3) {
      val = __bfloat162float(__float2bfloat16_rn(val));
      const float other = __shfl_xor_sync(0xffffffffu, val, 1);     // gate (even n) <-> up (odd n)
      if (m < P.M && n + 1 < P.N && (n & 1) == 0)
        ((bf16*)P.out)[(size_t)m * P.ldo + (n >> 1)] = __float2bfloat16_rn(val / (1.0f + __expf(-val)) * other);
    } else if (m < P.M && n < P.N) {
      const size_t idx = (size_t)m * P.ldo + n;
      if (EPI == 0) ((bf16*)P.out)[idx] = __float2bfloat16_rn(val);
      else ((float*)P.out)[idx] = val;
    }
  }
  }
}

// Epilogue 4, after sk_store: v holds squares; add them over the warp's 32 weight rows and leave the sums for
// sk_emit_sums.
template <int CW>
__device__ __forceinline__ void sk_emit_squares(SkTables& T, int quarter, int lane, int m0, float (&v)[CW]) {
#pragma unroll
  for (int j = 0; j < CW; j++) {
    const float t = warp_sum(v[j]);
    if (lane == 0) T.ss[quarter][m0 + j] = t;
  }
}
// Once the four epilogue warps have left their sums of a tile (a barrier among them lies between): the tile's part.
__device__ __forceinline__ void sk_emit_sums(const SkParams& P, const SkTables& T, int tile, int t) {
  if (t < P.M && P.X.emit_ss)
    P.X.emit_ss[(size_t)tile * P.X.emit_ld + t] = ((T.ss[0][t] + T.ss[1][t]) + T.ss[2][t]) + T.ss[3][t];
}

template <int BN, int STAGES>
struct SkSmem {
  alignas(1024) bf16 a[STAGES][TC_BM * TC_BK];
  alignas(1024) bf16 b[STAGES][BN * TC_BK];
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  SkTables tab;
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, int STAGES, int EPI, bool XT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_streamk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       const SkParams P) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = SkSmem<BN, STAGES>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * sizeof(bf16), B_BYTES = BN * TC_BK * sizeof(bf16);
  const int G = gridDim.x, c = blockIdx.x;
  const int kb0 = sk_begin(c, G, P.total_kb), kb1 = sk_begin(c + 1, G, P.total_kb);
  volatile int* abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 4); }
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      const int count = kb1 - kb0;
      const int pre = count < STAGES ? count : STAGES;
      // weights of the first stages: requested while the kernel before this one may still be running
      for (int i = 0; i < pre; i++) {
        const int g = kb0 + i;
        mbar_expect_tx(&S.full[i], A_BYTES + B_BYTES);
        tma_load_2d(&map_w, S.a[i], &S.full[i], (g % P.n_kb) * TC_BK, (g / P.n_kb) * TC_BM);
      }
      pdl_wait();
      for (int i = 0; i < pre; i++) tma_load_2d(&map_x, S.b[i], &S.full[i], ((kb0 + i) % P.n_kb) * TC_BK, 0);
      bool ok = true;
      for (int i = pre; i < count; i++) {
        const int g = kb0 + i, s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&S.empty[s], ph ^ 1, abort_flag)) {
          atomicCAS(P.status, 0, 101); S.abort_flag = 1; ok = false; break;
        }
        mbar_expect_tx(&S.full[s], A_BYTES + B_BYTES);
        tma_load_2d(&map_w, S.a[s], &S.full[s], (g % P.n_kb) * TC_BK, (g / P.n_kb) * TC_BM);
        tma_load_2d(&map_x, S.b[s], &S.full[s], (g % P.n_kb) * TC_BK, 0);
      }
      if (!ok) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);   // let copies already issued land
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(BN);
      uint32_t it = 0, seg = 0;
      bool ok = true;
      int g = kb0;
      while (g < kb1 && ok) {
        const int tile = g / P.n_kb;
        const int seg_end = min(kb1, (tile + 1) * P.n_kb);
        const int buf = seg & 1;
        if (!mbar_wait(&S.acc_empty[buf], ((seg >> 1) & 1) ^ 1, abort_flag)) {
          atomicCAS(P.status, 0, 102); S.abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        bool first = true;
        for (; g < seg_end; g++, it++) {
          const int s = it % STAGES;
          if (!mbar_wait(&S.full[s], (it / STAGES) & 1, abort_flag)) {
            atomicCAS(P.status, 0, 103); S.abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(S.a[s]), b_addr = smem_u32(S.b[s]);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; k++) {
            umma_bf16(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                      (first && k == 0) ? 0u : 1u);
          }
          first = false;
          umma_commit(&S.empty[s]);
        }
        if (ok) umma_commit(&S.acc_full[buf]);
        seg++;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    pdl_wait();                                   // the output, the residual stream and the scratch are shared
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // weight row within the tile held by this thread
    const int first_tile = kb0 / P.n_kb;
    constexpr int CW = (BN >= 32) ? 32 : 16;
    if constexpr (XT) {
      sk_tables_init<EPI, BN>(P, S.tab, threadIdx.x - 64, 128);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    uint32_t seg = 0;
    bool ok = true;
    int g = kb0;
    while (g < kb1 && ok) {
      const int tile = g / P.n_kb;
      const int seg_end = min(kb1, (tile + 1) * P.n_kb);
      const bool whole = (g == tile * P.n_kb) && (seg_end == (tile + 1) * P.n_kb);
      const int buf = seg & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&S.acc_full[buf], (seg >> 1) & 1, abort_flag))) {
        if (lane == 0) { atomicCAS(P.status, 0, 104); S.abort_flag = 1; }
      }
      // the four epilogue warps go on, or give up, together: the barriers below have no limit of their own
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (S.abort_flag) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      const int n = tile * TC_BM + row;
      float* part = P.scratch + ((size_t)(c * 2 + (tile == first_tile ? 0 : 1)) * BN) * TC_BM;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CW) {
        uint32_t r[CW];
        if constexpr (CW == 32) tmem_ld32(taddr + c0, r); else tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
        if (whole) {
          float v[CW];
#pragma unroll
          for (int j = 0; j < CW; j++) v[j] = __uint_as_float(r[j]);
          sk_store<EPI, CW, XT>(P, S.tab, n, c0, v);
          if (EPI == 4) sk_emit_squares<CW>(S.tab, quarter, lane, c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < CW; j++) part[(size_t)(c0 + j) * TC_BM + row] = __uint_as_float(r[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.acc_empty[buf]);
      if (EPI == 4 && whole) {                    // (uniform over the four warps: they walk the same tiles)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        sk_emit_sums(P, S.tab, tile, threadIdx.x - 64);
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      g = seg_end;
      seg++;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- few rows of x, N small: k shared inside a cluster
// Where W has no more tiles of 128 rows than there are SMs, a cluster of CS CTAs takes one tile and cuts k into
// CS stretches, one per CTA.  Each CTA sums its stretch in tensor memory; the rows of x are then dealt out to the
// ranks, every CTA writes its float32 partial sums of a rank's rows into that rank's shared memory (into its ring,
// idle by then), and every rank adds what it got in the order of the ranks, which is the order of k, and runs the
// epilogue for its rows.  One launch, no scratch in global memory; the cut depends only on the shapes.
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

template <int BN, int STAGES, int EPI, bool XT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_clusterk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        const SkParams P) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = SkSmem<BN, STAGES>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * sizeof(bf16), B_BYTES = BN * TC_BK * sizeof(bf16);
  const int CS = (int)cluster_nctarank(), rank = (int)cluster_ctarank();
  const int tile = blockIdx.x / CS;
  const int kb0 = (int)((long long)rank * P.n_kb / CS), kb1 = (int)((long long)(rank + 1) * P.n_kb / CS);
  volatile int* abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    mbar_init(&S.acc_full[0], 1);
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  constexpr int CW = (BN >= 32) ? 32 : 16;
  // Up to 64 rows of x an epilogue thread holds its weight row's sums for all rows of x in registers; with 256
  // rows (prompts of up to 256 tokens) it reads tensor memory chunk by chunk when it deals the chunks out.
  constexpr bool WIDE = BN > 64;
  static_assert(!WIDE || !XT, "the wide cluster forms know the plain epilogues only");
  float v[WIDE ? 1 : BN];                          // epilogue warps: this thread's weight row, all rows of x

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      const int count = kb1 - kb0;
      const int pre = count < STAGES ? count : STAGES;
      for (int i = 0; i < pre; i++) {               // weights first: the kernel before this one may still be running
        mbar_expect_tx(&S.full[i], A_BYTES + B_BYTES);
        tma_load_2d(&map_w, S.a[i], &S.full[i], (kb0 + i) * TC_BK, tile * TC_BM);
      }
      pdl_wait();
      for (int i = 0; i < pre; i++) tma_load_2d(&map_x, S.b[i], &S.full[i], (kb0 + i) * TC_BK, 0);
      bool ok = true;
      for (int i = pre; i < count; i++) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(&S.empty[s], ph ^ 1, abort_flag)) {
          atomicCAS(P.status, 0, 121); S.abort_flag = 1; ok = false; break;
        }
        mbar_expect_tx(&S.full[s], A_BYTES + B_BYTES);
        tma_load_2d(&map_w, S.a[s], &S.full[s], (kb0 + i) * TC_BK, tile * TC_BM);
        tma_load_2d(&map_x, S.b[s], &S.full[s], (kb0 + i) * TC_BK, 0);
      }
      if (!ok) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);   // let copies already issued land
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(BN);
      bool ok = true;
      for (int i = 0; i < kb1 - kb0; i++) {
        const int s = i % STAGES;
        if (!mbar_wait(&S.full[s], (i / STAGES) & 1, abort_flag)) {
          atomicCAS(P.status, 0, 123); S.abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(S.a[s]), b_addr = smem_u32(S.b[s]);
#pragma unroll
        for (int k = 0; k < TC_BK / 16; k++) {
          umma_bf16(tmem_base, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                    (i == 0 && k == 0) ? 0u : 1u);
        }
        umma_commit(&S.empty[s]);
      }
      if (ok) umma_commit(&S.acc_full[0]);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5): this CTA's sums
    pdl_wait();
    if constexpr (XT) sk_tables_init<EPI, BN>(P, S.tab, threadIdx.x - 64, 128);   // (rank 0 uses them, after the cluster's barriers)
    if (kb1 > kb0) {
      if (!__all_sync(0xffffffffu, mbar_wait(&S.acc_full[0], 0, abort_flag))) {
        if (lane == 0) { atomicCAS(P.status, 0, 124); S.abort_flag = 1; }
      }
      tc_fence_after();
      if constexpr (!WIDE) {
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += CW) {
          uint32_t r[CW];
          if constexpr (CW == 32) tmem_ld32(taddr + c0, r); else tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CW; j++) v[c0 + j] = __uint_as_float(r[j]);
        }
        tc_fence_before();
      }
    } else if constexpr (!WIDE) {
#pragma unroll
      for (int j = 0; j < BN; j++) v[j] = 0.0f;
    }
  }
  // Every thread of the cluster meets here twice, whatever happened above (a wait that ran out leaves its mark in
  // the status word and the CTA goes on with what it has).  After the first meeting every CTA's products have been
  // read out of tensor memory and its ring is idle; between the two, the rows of x are dealt out in chunks of CWS
  // to the ranks (chunk c to rank c % CS) and every CTA writes its partial sums of a chunk into the ring of the
  // chunk's rank; after the second, every rank adds what it was given in the order of the ranks, which is the order
  // of k, and runs the epilogue for its rows: the adding and storing is spread over the cluster.
  constexpr int CWS = BN > 64 ? 16 : (BN >= 32 ? 8 : 4);
  constexpr int NCH = BN / CWS;
  // (what a rank is given fits its ring, a and b together: at most NCH + 7 chunks of CWS x 128 float32)
  static_assert((size_t)(NCH + 7) * CWS * TC_BM * sizeof(float) <= (size_t)STAGES * (TC_BM + BN) * TC_BK * sizeof(bf16),
                "the exchange does not fit the ring");
  const int live = (P.M + CWS - 1) / CWS < NCH ? (P.M + CWS - 1) / CWS : NCH;   // chunks that hold rows of x
  const int row = (warp & 3) * 32 + lane;
  __syncwarp();
  cluster_sync_all();
  float* part = reinterpret_cast<float*>(S.a);      // this CTA's ring: [its chunks][source rank][CWS][128] float32
  if (warp >= 2) {
    if constexpr (WIDE) {
      // (every rank's MMAs are complete: each rank's epilogue warps came to the meeting after their wait for them)
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < live; c++) {
        uint32_t r[CWS];
        if (kb1 > kb0) { tmem_ld16(taddr + c * CWS, r); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int j = 0; j < CWS; j++) r[j] = 0u;
        }
        const int owner = c % CS, slot = c / CS;
        float* mine = part + (size_t)(slot * CS + rank) * CWS * TC_BM + row;
        if (owner == rank) {
#pragma unroll
          for (int j = 0; j < CWS; j++) mine[j * TC_BM] = __uint_as_float(r[j]);
        } else {
          const uint32_t dst = cluster_map(mine, (uint32_t)owner);
#pragma unroll
          for (int j = 0; j < CWS; j++) st_cluster_f32(dst + (uint32_t)(j * TC_BM * sizeof(float)), __uint_as_float(r[j]));
        }
      }
      tc_fence_before();
    } else {
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        if (c < live) {
          const int owner = c % CS, slot = c / CS;
          float* mine = part + (size_t)(slot * CS + rank) * CWS * TC_BM + row;
          if (owner == rank) {
#pragma unroll
            for (int j = 0; j < CWS; j++) mine[j * TC_BM] = v[c * CWS + j];
          } else {
            const uint32_t dst = cluster_map(mine, (uint32_t)owner);
#pragma unroll
            for (int j = 0; j < CWS; j++) st_cluster_f32(dst + (uint32_t)(j * TC_BM * sizeof(float)), v[c * CWS + j]);
          }
        }
      }
    }
  }
  cluster_sync_all();
  if (warp >= 2) {
    const int n = tile * TC_BM + row;
    for (int c = rank, slot = 0; c < live; c += CS, slot++) {
      float o[CWS];
#pragma unroll
      for (int j = 0; j < CWS; j++) o[j] = 0.0f;
      for (int r = 0; r < CS; r++) {
        const float* src = part + (size_t)(slot * CS + r) * CWS * TC_BM + row;
#pragma unroll
        for (int j = 0; j < CWS; j++) o[j] += src[j * TC_BM];
      }
      sk_store<EPI, CWS, XT>(P, S.tab, n, c * CWS, o);
      if (EPI == 4) sk_emit_squares<CWS>(S.tab, warp & 3, lane, c * CWS, o);
    }
  }
  __syncthreads();
  if (EPI == 4 && warp >= 2) {                      // each rank the sums of the rows it stored
    const int t = threadIdx.x - 64;
    if (t < P.M && (t / CWS) % CS == rank) sk_emit_sums(P, S.tab, tile, t);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
// A [rows][K] bf16 matrix with row pitch `ld` elements, fetched in boxes of box_rows x 64 with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return STRATUM_ERR_LIMIT;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(bf16)};
  cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : STRATUM_ERR_SHAPE;
}

// Second pass for tiles shared between CTAs (see TcSchedule).  Block (r, g) takes a 32-row by 64-column part of
// the r-th shared tile.  The pieces lie [column][row]: a warp reads 32 rows of one column at a time and adds the
// pieces in the order of k (eight columns per thread, two pieces in flight); the sums go through shared memory so
// that the epilogue writes rows, four neighbouring columns per thread.
// halves = 2: the pieces of the pair kernel, whose tiles are two CTAs' 128 rows each (G pairs; a pair's slot holds
// rank 0's rows, then rank 1's).
template <int BN, int EPI>
__global__ void __launch_bounds__(256)
gemm_tc_pieces_kernel(const TcParams P, int G, int n_tiles, int n_kb, int tiles_a, int halves) {
  __shared__ float tile_s[32][65];
  pdl_trigger();
  const int R = n_tiles % G, U = R * n_kb;
  const int r = blockIdx.x;
  const int first_c = tc_owner(r * n_kb, G, U), last_c = tc_owner((r + 1) * n_kb - 1, G, U);
  if (first_c == last_c) return;                   // one CTA had the whole tile
  const int tile = n_tiles - R + r;
  const int ta = tile % tiles_a, tb = tile / tiles_a;
  const int half = blockIdx.y % halves, part_y = blockIdx.y / halves;
  const int row0 = (part_y % 4) * 32, col0 = (part_y / 4) * 64;
  const int m0 = (ta * halves + half) * TC_BM + row0;
  if (m0 >= P.M || tb * BN + col0 >= P.N) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; j++) acc[j] = 0.f;
  for (int c0 = first_c; c0 <= last_c; c0 += 2) {
    float a[2][8];
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int cc = c0 + e;
      const int slot = (tc_begin(cc < G ? cc : 0, G, U) / n_kb == r) ? 0 : 1;
      const float* src = P.scratch + ((((size_t)cc * 2 + slot) * halves + half) * BN + col0 + warp * 8) * TC_BM + row0 + lane;
#pragma unroll
      for (int j = 0; j < 8; j++) a[e][j] = (cc <= last_c) ? __ldcg(src + (size_t)j * TC_BM) : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 2; e++)
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] += a[e][j];
  }
#pragma unroll
  for (int j = 0; j < 8; j++) tile_s[lane][warp * 8 + j] = acc[j];
  __syncthreads();
#pragma unroll
  for (int pass = 0; pass < 2; pass++) {
    const int rr = pass * 16 + (threadIdx.x >> 4), cc4 = (threadIdx.x & 15) * 4;
    const int m = m0 + rr;
    if (m < P.M)
      fixup_store<EPI>(P, m, tb * BN + col0 + cc4,
                       make_float4(tile_s[rr][cc4], tile_s[rr][cc4 + 1], tile_s[rr][cc4 + 2], tile_s[rr][cc4 + 3]));
  }
}

// Whether sharing the left-over tiles pays: a model of both ways in units of one k-block of one tile (about half
// a microsecond).  Plain: waves * n_kb.  Shared: the k-blocks spread over all SMs, plus writing and reading the
// pieces (a piece of 128 x 256 float32 per SM costs about as much as 16 k-blocks, measured), plus the second
// launch (6).  STRATUM_GEMM_SPLIT=0 turns sharing off, =1 forces it where it is possible (measurements).
static bool split_pays(int n_tiles, int n_kb, int sms, int bn, float margin = 0.9f) {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("STRATUM_GEMM_SPLIT");
    mode = e ? atoi(e) + 1 : 0;                   // 0: model, 1: off, 2: on
  }
  const int left = n_tiles % sms, waves = (n_tiles + sms - 1) / sms;
  if (left == 0 || (long long)left * n_kb < 4LL * sms || mode == 1) return false;
  if (mode == 2) return true;
  const float plain = (float)waves * n_kb;
  const float pieces = (float)(sms + left) / sms;                        // per SM
  const float shared = (float)n_tiles * n_kb / sms + pieces * 16.0f * bn / 256.0f + 6.0f;
  return shared < margin * plain;
}

// The pair kernel: clusters of two CTAs, as many pairs as can be resident (at most one per two SMs).
static int resident_pairs() {
  static int pairs = 0;
  if (pairs == 0) {
    auto kern = gemm_tc2_kernel<0, 256>;
    const size_t smem = sizeof(Tc2Smem<TC2_STAGES>) + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(sm_count() & ~1); q.blockDim = dim3(TC_THREADS); q.dynamicSmemBytes = smem;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n < 1) { cudaGetLastError(); return -1; }
    pairs = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  return pairs;
}

// split: the tiles of a partly filled last wave are shared along k by all pairs, a second kernel adds their pieces
// (tiles of 256 columns and the four basic epilogues only; scratch as for the tile kernel).
template <int BN>
static int launch_tc2(const CUtensorMap& ma, const CUtensorMap& mb, TcParams P, int epilogue, int n_tiles,
                      cudaStream_t stream, bool split = false, float* scratch = nullptr) {
  const size_t smem = sizeof(Tc2Smem<TC2_STAGES>) + 1024;
  const int max_pairs = resident_pairs();
  if (max_pairs < 1) return STRATUM_ERR_LIMIT;
  if (split && (BN != 256 || epilogue >= 4 || !scratch)) return STRATUM_ERR_SHAPE;
  P.split = split ? 1 : 0; P.scratch = split ? scratch : nullptr;
  const int tiles_m = (P.M + 2 * TC_BM - 1) / (2 * TC_BM), n_kb = (P.K + TC_BK - 1) / TC_BK;
#define TC2_LAUNCH(E)                                                                                       \
  {                                                                                                         \
    auto kern = gemm_tc2_kernel<E, BN>;                                                                     \
    static bool configured = false;                                                                         \
    if (!configured) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                  \
      configured = true;                                                                                    \
    }                                                                                                       \
    const int pairs = (split || n_tiles >= max_pairs) ? max_pairs : n_tiles;                                \
    int st = launch_pdl(kern, 2 * pairs, TC_THREADS, smem, stream, ma, mb, P);                              \
    if (st != 0) return st;                                                                                 \
    g_last_launches = split ? 2 : 1; g_last_form = split ? 5 : 2;                                                    \
    if constexpr (BN == 256 && E < 4) {                                                                     \
      if (split) {                                                                                          \
        st = launch_pdl(gemm_tc_pieces_kernel<BN, E>, dim3(n_tiles % pairs, 4 * (BN / 64) * 2), 256, 0,     \
                        stream, P, pairs, n_tiles, n_kb, tiles_m, 2);                                       \
        if (st != 0) return st;                                                                             \
      }                                                                                                     \
    }                                                                                                       \
  }
  switch (epilogue) {
    case 0: TC2_LAUNCH(0) break;
    case 1: TC2_LAUNCH(1) break;
    case 2: TC2_LAUNCH(2) break;
    case 3: TC2_LAUNCH(3) break;
    case 4: TC2_LAUNCH(4) break;
    case 5: TC2_LAUNCH(5) break;
    default: return STRATUM_ERR_SHAPE;
  }
#undef TC2_LAUNCH
  return launch_status();
}

// The tile width of the pair kernel for a shape: the one whose waves x width is least (a narrower tile that saves
// a wave, or fills the same number of waves with less, wins), 256 among equals.
static int pair_tile_width(int M, int N, int pairs) {
  const int tiles_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
  int best = 256;
  long long best_cost = -1;
  const int widths[3] = {256, 240, 224};
  for (int i = 0; i < 3; i++) {
    const int bn = widths[i];
    const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    const long long cost = ((tiles + pairs - 1) / pairs) * bn;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

// Rows of x from which the pair kernel is used (STRATUM_GEMM_2CTA=0 turns it off, =N sets the number of rows; for
// measurements).
static int pair_kernel_min_rows() {
  static int rows = -1;
  if (rows < 0) {
    const char* e = getenv("STRATUM_GEMM_2CTA");
    rows = e ? atoi(e) : 129;
    if (e && rows <= 0) rows = 0x7fffffff;
  }
  return rows;
}

static bool pair_split_enabled() {                 // STRATUM_GEMM_PAIR_SPLIT=0 turns the sharing among pairs off (measurements)
  static int on = -1;
  if (on < 0) { const char* e = getenv("STRATUM_GEMM_PAIR_SPLIT"); on = (e && e[0] == '0') ? 0 : 1; }
  return on == 1;
}

// Pairs of CTAs that can be resident at once (for reports).
STRATUM_EXPORT int stratum_gemm_tc_resident_pairs(void) { return resident_pairs(); }

template <int BN, int STAGES>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, TcParams P, int epilogue, int n_tiles, int n_kb,
                     int tiles_a, float* scratch, cudaStream_t stream) {
  const size_t smem = sizeof(TcSmem<BN, STAGES>) + 1024;
  const int sms = sm_count();
  int grid = n_tiles < sms ? n_tiles : sms;
  const int left = n_tiles % sms;
  P.split = 0; P.scratch = scratch;
  // (the second kernel of the split knows the four basic epilogues only)
  if (scratch && epilogue < 4 && !P.X.norm_ss && split_pays(n_tiles, n_kb, sms, BN)) {
    P.split = 1;
    grid = sms;
  }
#define TC_LAUNCH(E)                                                                                        \
  {                                                                                                         \
    auto kern = gemm_tc_kernel<BN, STAGES, E>;                                                              \
    static bool configured = false; /* once per instantiation; not a stream operation */                   \
    if (!configured) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                  \
      configured = true;                                                                                    \
    }                                                                                                       \
    int st = launch_pdl(kern, grid, TC_THREADS, smem, stream, ma, mb, P);                                   \
    if (st != 0) return st;                                                                                 \
    g_last_launches = P.split ? 2 : 1; g_last_form = 1;                                                     \
    if (P.split) {                                                                                          \
      st = launch_pdl(gemm_tc_pieces_kernel<BN, E>, dim3(left, 4 * (BN / 64)), 256, 0, stream, P, grid,     \
                      n_tiles, n_kb, tiles_a, 1);                                                           \
      if (st != 0) return st;                                                                               \
    }                                                                                                       \
  }
  switch (epilogue) {
    case 0: TC_LAUNCH(0) break;
    case 1: TC_LAUNCH(1) break;
    case 2: TC_LAUNCH(2) break;
    case 3: TC_LAUNCH(3) break;
    case 4: TC_LAUNCH(4) break;
    case 5: TC_LAUNCH(5) break;
    default: return STRATUM_ERR_SHAPE;
  }
#undef TC_LAUNCH
  return launch_status();
}

// Second pass of the stream-K form: every tile that was shared between CTAs is put together from the partial
// sums in scratch, in the order of k (the order of the CTA numbers), and goes through the epilogue.  A shared
// tile is one that holds the beginning of some CTA's stretch; block x looks at the beginning of CTA x+1 and takes
// the tile if it is the first beginning inside it.  A block is 4 rows of x (one per warp) by 128 weight rows
// (four neighbours per lane, so that every load and store is 16 bytes wide); the loads of up to eight partial
// tiles are in flight together.
template <int BN, int EPI, bool XT>
__global__ void __launch_bounds__(128)
gemm_tc_fixup_kernel(const SkParams P, int G) {
  pdl_trigger();
  const int c1 = blockIdx.x + 1;
  const int b1 = sk_begin(c1, G, P.total_kb);
  const int tile = b1 / P.n_kb;
  if (b1 % P.n_kb == 0) return;                                       // CTA c1 begins with a tile of its own
  if (c1 > 1 && sk_begin(c1 - 1, G, P.total_kb) > tile * P.n_kb) return;   // an earlier block has this tile
  const int m = blockIdx.y * 4 + (threadIdx.x >> 5);
  if (m >= P.M) return;
  const int first_c = c1 - 1;
  const int last_c = sk_owner((tile + 1) * P.n_kb - 1, G, P.total_kb);
  const int col = (threadIdx.x & 31) * 4;
  // The tile is the first of every CTA after first_c (slot 0); for first_c it is the first one only if that CTA's
  // stretch begins exactly with it (it cannot begin later: then an earlier block would have taken the tile).
  const int slot_first = (sk_begin(first_c, G, P.total_kb) == tile * P.n_kb) ? 0 : 1;
  const int n = tile * TC_BM + col;
  const size_t idx = (size_t)m * P.ldo + n;
  // adding into float32: the old values are asked for together with the partial sums, not after them
  constexpr bool ADD = EPI == 1 || EPI == 4;
  const bool add_wide = ADD && n + 3 < P.N && ((reinterpret_cast<uintptr_t>((float*)P.out + idx) & 15) == 0);
  // (positions and page tables are the step's description, not an earlier kernel's work: read before the wait)
  const long long cache_row = (EPI == 5) ? epi_cache_row(P.X, m) : -1;
  pdl_wait();
  float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
  if (add_wide) old = __ldcg(reinterpret_cast<const float4*>((const float*)P.out + idx));
  float scale = 1.0f;
  if constexpr (XT) {
    if (P.X.norm_ss) {                             // one lane adds the row's parts, in their order
      if ((threadIdx.x & 31) == 0) scale = epi_row_scale(P.X, m);
      scale = __shfl_sync(0xffffffffu, scale, 0);
    }
  }
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = first_c; c0 <= last_c; c0 += 8) {
    float4 a[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int cc = c0 + j;
      if (cc <= last_c) {
        const int slot = cc == first_c ? slot_first : 0;
        a[j] = __ldcg(reinterpret_cast<const float4*>(P.scratch + ((size_t)(cc * 2 + slot) * BN + m) * TC_BM + col));
      } else {
        a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      if (c0 + j <= last_c) { v.x += a[j].x; v.y += a[j].y; v.z += a[j].z; v.w += a[j].w; }
    }
  }
  if constexpr (XT) { v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale; }
  if (add_wide) {
    if (P.bias) { v.x += P.bias[n]; v.y += P.bias[n + 1]; v.z += P.bias[n + 2]; v.w += P.bias[n + 3]; }
    const float4 r = make_float4(old.x + v.x, old.y + v.y, old.z + v.z, old.w + v.w);
    *reinterpret_cast<float4*>((float*)P.out + idx) = r;
    if (EPI == 4 && P.X.emit_x) {
      const float4 g = __ldg(reinterpret_cast<const float4*>(P.X.emit_gain + n));
      __nv_bfloat162 lo = __floats2bfloat162_rn(r.x * g.x, r.y * g.y), hi = __floats2bfloat162_rn(r.z * g.z, r.w * g.w);
      uint2 u; u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(P.X.emit_x + (size_t)m * P.X.emit_ldx + n) = u;
      const float ss = warp_sum(fmaf(r.x, r.x, fmaf(r.y, r.y, fmaf(r.z, r.z, r.w * r.w))));
      if ((threadIdx.x & 31) == 0 && P.X.emit_ss) P.X.emit_ss[(size_t)tile * P.X.emit_ld + m] = ss;
    }
    return;
  }
  if (EPI == 5) {
    // four neighbouring dimensions of one head: two rotated pairs
    if (n + 3 >= P.N) return;
    const EpiExtra& X = P.X;
    if (P.bias) { v.x += P.bias[n]; v.y += P.bias[n + 1]; v.z += P.bias[n + 2]; v.w += P.bias[n + 3]; }
    const int h = n / X.head_dim, d = n - h * X.head_dim;
    const bool is_q = h < X.n_q, is_k = !is_q && h < X.n_q + X.n_kv;
    if ((is_q || is_k) && X.rope_cs) {
      const float2* cs = X.rope_cs + (size_t)m * X.rope_pairs + (d >> 1);
      if ((d >> 1) < X.rope_pairs) { const float2 f = __ldcg(cs); const float x0 = v.x, x1 = v.y; v.x = x0 * f.x - x1 * f.y; v.y = x0 * f.y + x1 * f.x; }
      if ((d >> 1) + 1 < X.rope_pairs) { const float2 f = __ldcg(cs + 1); const float x0 = v.z, x1 = v.w; v.z = x0 * f.x - x1 * f.y; v.w = x0 * f.y + x1 * f.x; }
    }
    bf16* o;
    if (is_q) {
      o = (bf16*)P.out + (size_t)m * P.ldo + n;
    } else {
      if (cache_row < 0) return;
      const int kvh = is_k ? h - X.n_q : h - X.n_q - X.n_kv;
      o = (is_k ? X.k_cache : X.v_cache) + cache_row + (long long)kvh * X.page_tokens * X.head_dim + d;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u; u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o) = u;
    return;
  }
  fixup_store<EPI>(P, m, n, v);
}

// Clusters of `cs` CTAs of the cluster kernel that can be resident at once (0: none, or the query failed).
template <int BN, int STAGES, int EPI, bool XT>
static int clusterk_resident(int cs) {
  static int cached[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (cs < 1 || cs > 8) return 0;
  if (cached[cs] < 0) {
    auto kern = gemm_tc_clusterk_kernel<BN, STAGES, EPI, XT>;
    const size_t smem = sizeof(SkSmem<BN, STAGES>) + 1024;
    cached[cs] = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) {
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3((sm_count() / cs) * cs); q.blockDim = dim3(TC_THREADS); q.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      q.attrs = attr; q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &q) == cudaSuccess && n > 0) cached[cs] = n;
      else cudaGetLastError();
    }
  }
  return cached[cs];
}

// The cluster size with which `tiles` clusters fill most SMs in one wave, or 0 if there is none: every rank needs a
// k-block, and all clusters must be resident together.  (What the ranks exchange always fits a ring: at most
// BN / CWS + 7 chunks of CWS x 128 float32, 60 KB.)
// A rank's stretch must be CLUSTERK_MIN_KB k-blocks or more, and a "cluster" of one CTA (a whole tile's k per CTA,
// on fewer SMs than stream-K uses) is not taken.  Both rules are measured in whole decode steps, not derived.
// Llama-3.2-1B shape (QKV 24 clusters of 5 with 6 k-blocks a rank; gate|up 128 tiles, one CTA each): QKV in the
// cluster form costs 5 us a layer at 64 rows, gate|up 4 us at 64 rows and 2.4 us at 8 rows (with an ordinary
// launch instead of a cluster launch of one CTA just the same), against stream-K on all 148 SMs with its second
// pass; with neither, the step takes 0.927 instead of 0.965 ms at 8 rows and 1.071 instead of 1.158 at 16.
// Llama-3.1-8B and Llama-2-7B shapes (16 to 56 k-blocks a rank) are ahead with the cluster form up to about 40
// rows (8B: 5.35 against 5.53 ms at 24 rows, 6.10 against 6.24 at 32, level from 48 on; 3.93 against 4.02 at 8).
#ifndef CLUSTERK_MIN_KB
#define CLUSTERK_MIN_KB 16
#define CLUSTERK_MIN_CS 2
#endif
template <int BN, int STAGES, int EPI, bool XT>
static int clusterk_size(int tiles, int n_kb) {
  const int sms = sm_count();
  if (tiles > sms) return 0;
  for (int cs = sms / tiles > 8 ? 8 : sms / tiles; cs >= 1; cs--) {
    if (tiles * cs * 10 < sms * 8) break;                       // too few SMs at work: the even split is better
    if (cs > n_kb) continue;                                    // (every rank needs a k-block)
    if (cs < CLUSTERK_MIN_CS || n_kb / cs < CLUSTERK_MIN_KB) return 0;
    if (clusterk_resident<BN, STAGES, EPI, XT>(cs) >= tiles) return cs;
  }
  return 0;
}

static int clusterk_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("STRATUM_GEMM_CLUSTERK");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on;
}

template <int BN, int STAGES, int EPI, bool XT>
static int launch_clusterk(const CUtensorMap& mw, const CUtensorMap& mx, const SkParams& P, int cs,
                           cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(P.tiles * cs);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = sizeof(SkSmem<BN, STAGES>) + 1024;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cs; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  g_last_launches = 1; g_last_form = 4 + 16 * cs;
  return (int)cudaLaunchKernelEx(&cfg, gemm_tc_clusterk_kernel<BN, STAGES, EPI, XT>, mw, mx, P);
}

// The cluster form up to this many (padded) rows of x (STRATUM_GEMM_CLUSTERK_ROWS overrides, for measurements).
#ifndef CLUSTERK_MAX_BN
#define CLUSTERK_MAX_BN 256
#endif
static int clusterk_max_rows() {
  static int rows = -1;
  if (rows < 0) {
    const char* e = getenv("STRATUM_GEMM_CLUSTERK_ROWS");
    rows = e ? atoi(e) : CLUSTERK_MAX_BN;
  }
  return rows;
}

#ifndef SK_RING_16
#define SK_RING_16 10
#define SK_RING_32 9
#define SK_RING_64 8
#define SK_RING_128 6
#define SK_RING_256 4
#endif

// The cluster form for 129 to 256 rows of x (prompts of up to 256 tokens): x as one block of 256 rows along N of
// the MMA, the plain epilogues only.  0: not taken (launch another form); 1: launched (*st holds the status).
template <int BN, int STAGES>
static int try_clusterk_wide(const CUtensorMap& mw, const CUtensorMap& mx, const SkParams& P, int epilogue,
                             cudaStream_t stream, int* st) {
  if (!clusterk_enabled() || BN > clusterk_max_rows() || epilogue > 3 || P.X.norm_ss) return 0;
#define CKW(E)                                                                       \
  {                                                                                  \
    const int cs = clusterk_size<BN, STAGES, E, false>(P.tiles, P.n_kb);             \
    if (cs <= 0) return 0;                                                           \
    *st = launch_clusterk<BN, STAGES, E, false>(mw, mx, P, cs, stream);              \
    return 1;                                                                        \
  }
  switch (epilogue) {
    case 0: CKW(0)
    case 1: CKW(1)
    case 2: CKW(2)
    case 3: CKW(3)
    default: return 0;
  }
#undef CKW
}

template <int BN, int STAGES>
static int launch_streamk(const CUtensorMap& mw, const CUtensorMap& mx, const SkParams& P, int epilogue,
                          cudaStream_t stream) {
  const size_t smem = sizeof(SkSmem<BN, STAGES>) + 1024;
  const int grid = P.total_kb < sm_count() ? P.total_kb : sm_count();
  // no tile is shared between CTAs when every CTA's stretch is a whole number of tiles
  const bool split_tiles = !(P.tiles % grid == 0);
#define SK_LAUNCH_X(E, XT)                                                                                  \
  {                                                                                                         \
    if constexpr (BN <= 64) {                                                                               \
      if (split_tiles && clusterk_enabled() && BN <= clusterk_max_rows()) {                                   \
        const int cs = clusterk_size<BN, STAGES, E, XT>(P.tiles, P.n_kb);                                   \
        if (cs > 0) return launch_clusterk<BN, STAGES, E, XT>(mw, mx, P, cs, stream);                       \
      }                                                                                                     \
    }                                                                                                       \
    auto kern = gemm_tc_streamk_kernel<BN, STAGES, E, XT>;                                                  \
    static bool configured = false;                                                                         \
    if (!configured) {                                                                                      \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
      if (e != cudaSuccess) return (int)e;                                                                  \
      configured = true;                                                                                    \
    }                                                                                                       \
    int st = launch_pdl(kern, grid, TC_THREADS, smem, stream, mw, mx, P);                                   \
    g_last_launches = split_tiles ? 2 : 1; g_last_form = 3;                                                 \
    if (st != 0 || !split_tiles) return st;                                                                 \
    return launch_pdl(gemm_tc_fixup_kernel<BN, E, XT>, dim3(grid - 1, (P.M + 3) / 4), 128, 0, stream, P, grid); \
  }
  // the four basic epilogues without rows of a handed-over norm take the kernels compiled without the tables
#define SK_LAUNCH(E)                                                                                        \
  if (E < 4 && !P.X.norm_ss) SK_LAUNCH_X(E, (E >= 4))                                                       \
  else SK_LAUNCH_X(E, true)
  switch (epilogue) {
    case 0: SK_LAUNCH(0)
    case 1: SK_LAUNCH(1)
    case 2: SK_LAUNCH(2)
    case 3: SK_LAUNCH(3)
    case 4: SK_LAUNCH(4)
    case 5: SK_LAUNCH(5)
    default: return STRATUM_ERR_SHAPE;
  }
#undef SK_LAUNCH
#undef SK_LAUNCH_X
}

STRATUM_EXPORT int stratum_gemm_tc_last_launches(void) { return g_last_launches; }
STRATUM_EXPORT int stratum_gemm_tc_last_form(void) { return g_last_form; }

// Scratch for partial tiles (two 128 x 256 float32 tiles per SM cover both forms).
STRATUM_EXPORT long long stratum_gemm_tc_scratch_floats(void) { return (long long)sm_count() * 2 * 256 * TC_BM; }

static int g_last_parts = 0;          // epilogue 4: how many parts of sums of squares the last call wrote per row
STRATUM_EXPORT int stratum_gemm_tc_last_parts(void) { return g_last_parts; }

// x: bf16 [M][ldx], w: bf16 [N][K], bias float32 [N] or null, out [M][ldo] (SwiGLU: [M][N/2]).
// scratch: partial tiles of tiles shared between CTAs (see stratum_gemm_tc_scratch_floats).  Without it more than
// 128 rows of x still work (no tile is shared then); up to 128 rows need it.
// status: one int in device memory, 0 before the call; non-zero afterwards means a wait inside the kernel ran out.
// extra: null, or what EpiExtra describes (epilogues 4 and 5 need it).
// Needs K % 8 == 0, ldx % 8 == 0, 16-byte aligned x and w (a TMA copy starts on a 16-byte boundary and its
// row pitch is a multiple of 16 bytes; the k coordinate of every copy here is a multiple of 64).
STRATUM_EXPORT int stratum_gemm_tc_ex(const void* x, const void* w, const float* bias, void* out, int epilogue, int M,
                                      int N, int K, int ldx, int ldo, int* status, float* scratch,
                                      const EpiExtra* extra, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldx < K) return STRATUM_ERR_SHAPE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return STRATUM_ERR_ALIGN;
  if (epilogue == 3 && (N % 2 != 0)) return STRATUM_ERR_SHAPE;
  if (!status) return STRATUM_ERR_SHAPE;
  EpiExtra X = {};
  if (extra) X = *extra;
  if (epilogue == 4) {
    // the sums of squares are kept per tile of columns; vector stores everywhere
    if (!X.emit_x || !X.emit_gain || !X.emit_ss) return STRATUM_ERR_SHAPE;
    if (N % 128 != 0 || ldo % 4 != 0 || X.emit_ldx % 8 != 0 || X.emit_ld < M) return STRATUM_ERR_SHAPE;
    if (((uintptr_t)out | (uintptr_t)X.emit_x | (uintptr_t)X.emit_gain) & 15) return STRATUM_ERR_ALIGN;
  } else {
    X.emit_x = nullptr; X.emit_gain = nullptr; X.emit_ss = nullptr;
  }
  if (epilogue == 5) {
    if (X.head_dim < 32 || X.head_dim % 32 != 0 || X.n_q < 1 || X.n_kv < 1 || N != (X.n_q + 2 * X.n_kv) * X.head_dim)
      return STRATUM_ERR_SHAPE;
    if (X.rope_cs && (X.rope_pairs < 1 || 2 * X.rope_pairs > X.head_dim)) return STRATUM_ERR_SHAPE;
    if (!X.token_pos || !X.token_seq || X.page_tokens < 1 || ldo % 8 != 0) return STRATUM_ERR_SHAPE;
    if (X.write_cache && (!X.k_cache || !X.v_cache || !X.block_table)) return STRATUM_ERR_SHAPE;
    if (((uintptr_t)out | (uintptr_t)X.k_cache | (uintptr_t)X.v_cache) & 15) return STRATUM_ERR_ALIGN;
  }
  if (X.norm_ss && (X.norm_parts < 1 || X.norm_ld < M || !(X.norm_size > 0.f))) return STRATUM_ERR_SHAPE;
  TcParams P;
  P.bias = bias; P.out = out; P.status = status; P.M = M; P.N = N; P.K = K; P.ldo = ldo;
  P.split = 0; P.scratch = nullptr; P.X = X;
  g_last_parts = 0;
  CUtensorMap ma, mb;
  // up to 64 rows always; 65 to 128 rows unless the tile form fills most of the SMs with one wave (measured on the
  // Llama-8B shapes: 16.7 against 22 us for N = K = 4096, 70 against 53 us for N = 28672)
  const long long tiles_plain = (long long)((M + TC_BM - 1) / TC_BM) * ((N + (N >= 2048 ? 255 : 127)) / (N >= 2048 ? 256 : 128));
  const bool swap = M <= 64 || (M <= 128 && scratch && tiles_plain * 10 < (long long)sm_count() * 7);
  int st;
  if (M > 128 && M <= 256) {
    // 129 to 256 rows and few tiles of W (the output and down projections of a short prompt): k cut inside clusters,
    // the sums exchanged through distributed shared memory, instead of sharing tiles along k with a second kernel
    // that adds the pieces.  Measured on the Llama-8B shapes (K = 4096 / 14336, N = 4096): 17.4 / 36.2 us at 192
    // rows and 20.0 / 39.2 at 256 against 22.3 / 40.1 and 22.5 / 40.5 for pairs of CTAs sharing tiles; with 65 to
    // 128 rows (x as one block of 128) it was level with stream-K and its second pass (14.4 / 29.5 against
    // 13.8 / 28.8), so those stay as they were.
    const int bn = 256;
    SkParams Q;
    Q.bias = bias; Q.out = out; Q.status = status; Q.scratch = scratch;
    Q.M = M; Q.N = N; Q.K = K; Q.ldo = ldo; Q.X = X;
    Q.tiles = (N + TC_BM - 1) / TC_BM;
    Q.n_kb = (K + TC_BK - 1) / TC_BK;
    Q.total_kb = Q.tiles * Q.n_kb;
    if (Q.tiles * 2 <= sm_count() && Q.n_kb / 2 >= CLUSTERK_MIN_KB) {     // (a cluster of two at least: cheap pre-check)
      if ((st = make_map(&ma, w, N, K, K, TC_BM)) != 0) return st;
      if ((st = make_map(&mb, x, M, K, ldx, bn)) != 0) return st;
      g_last_parts = Q.tiles;
      if (try_clusterk_wide<256, SK_RING_256>(ma, mb, Q, epilogue, stream, &st)) return st;
    }
  }
  if (!swap) {
    // prompts: 128 rows of x by 256 (or 128) rows of W per tile
    // tiles of 256 columns from N = 2,048 on, unless a narrow matrix (below 4,096 rows of W) has so few of them
    // that most SMs would idle: then 128 columns and twice the tiles.  Measured on the Llama-3.2-1B shape (N 2,048
    // and 3,072): a prompt of 256 tokens 2.00 against 2.29 ms, of 512 tokens 2.41 against 2.56; from 1,024 tokens on
    // the wide tiles are ahead (3.24 against 3.37 ms).
    const int tiles_wide = ((M + TC_BM - 1) / TC_BM) * ((N + 255) / 256);
    const bool wide = N >= 4096 || (N >= 2048 && tiles_wide > 48);
    // 256 x 256 tiles on pairs of CTAs where they give most pairs of SMs a tile (measured on the Llama-8B shapes:
    // ahead from a few hundred rows on, except where N is small and the tile kernel can share its tiles along k)
    const int n_tiles2 = ((M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((N + 255) / 256);
    const int rows1 = ((M + TC_BM - 1) / TC_BM) * TC_BM, rows2 = ((M + 2 * TC_BM - 1) / (2 * TC_BM)) * 2 * TC_BM;
    // Few tiles of 256 x 256 (a few hundred rows, N of a few thousand): their k-blocks are shared by all pairs,
    // as the tile kernel shares its left-over tiles, but with the pairs' smaller draw on L2 per flop.
    if (wide && M >= pair_kernel_min_rows() && rows2 * 100 <= rows1 * 125 && scratch && epilogue < 4 && !X.norm_ss &&
        pair_split_enabled()) {
      const int pairs = resident_pairs();
      // (measured on the Llama-8B shapes: K = 14336 at 256 and 512 rows 40 and 59 us against 53 and 83 with the tile
      // kernel; at 768 rows, where the model says 0.79 of the unshared time, 82 against 79 us: the pairs that stay
      // idle without sharing leave the busy ones a higher clock)
      // (where the tiles are too few for the pairs to run unshared, the other way is the tile kernel sharing its
      // tiles, which the pairs beat more easily: K = 4096 at 512 rows 27.9 against 30.3 us at 0.88 of the model)
      const bool pairs_unshared_possible = n_tiles2 * 10 >= (sm_count() / 2) * 6;
      if (pairs >= 1 && split_pays(n_tiles2, (K + TC_BK - 1) / TC_BK, pairs, 256, pairs_unshared_possible ? 0.75f : 0.9f)) {
        if ((st = make_map(&ma, x, M, K, ldx, TC_BM)) != 0) return st;
        if ((st = make_map(&mb, w, N, K, K, 128)) != 0) return st;
        g_last_parts = (N + 255) / 256;
        return launch_tc2<256>(ma, mb, P, epilogue, n_tiles2, stream, true, scratch);
      }
    }
    if (wide && M >= pair_kernel_min_rows() && n_tiles2 * 10 >= (sm_count() / 2) * 6 &&
        rows2 * 100 <= rows1 * 125) {               // (not where half of a pair would work on rows beyond M: up to a
                                                    // quarter more rows the pairs still win, 10.1 against 11.0 ms for a
                                                    // prompt of 640 tokens on the Llama-8B shape; a third more, they lose)
      const int pairs = resident_pairs();
      if (pairs >= 1) {
        // (epilogue 5 walks whole heads: tiles of 256 columns begin where a head begins)
        const int bn = epilogue == 5 ? 256 : pair_tile_width(M, N, pairs);
        const int tiles = ((M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((N + bn - 1) / bn);
        if ((st = make_map(&ma, x, M, K, ldx, TC_BM)) != 0) return st;
        if ((st = make_map(&mb, w, N, K, K, bn / 2)) != 0) return st;
        g_last_parts = (N + bn - 1) / bn;
        if (bn == 256) return launch_tc2<256>(ma, mb, P, epilogue, tiles, stream);
        if (bn == 240) return launch_tc2<240>(ma, mb, P, epilogue, tiles, stream);
        return launch_tc2<224>(ma, mb, P, epilogue, tiles, stream);
      }                                             // (no pair can be resident here: the tile kernel below)
    }
    if ((st = make_map(&ma, x, M, K, ldx, TC_BM)) != 0) return st;
    if ((st = make_map(&mb, w, N, K, K, wide ? 256 : 128)) != 0) return st;
    const int tiles_m = (M + TC_BM - 1) / TC_BM, n_kb = (K + TC_BK - 1) / TC_BK;
    g_last_parts = wide ? (N + 255) / 256 : (N + 127) / 128;
    if (wide) return launch_tc<256, 4>(ma, mb, P, epilogue, tiles_m * ((N + 255) / 256), n_kb, tiles_m, scratch, stream);
    return launch_tc<128, 6>(ma, mb, P, epilogue, tiles_m * ((N + 127) / 128), n_kb, tiles_m, scratch, stream);
  }
  // few rows of x: tiles of 128 rows of W by all rows of x, k-blocks spread evenly over the SMs
  if (!scratch) return STRATUM_ERR_SHAPE;
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  if ((st = make_map(&ma, w, N, K, K, TC_BM)) != 0) return st;
  if ((st = make_map(&mb, x, M, K, ldx, bn)) != 0) return st;
  SkParams Q;
  Q.bias = bias; Q.out = out; Q.status = status; Q.scratch = scratch;
  Q.M = M; Q.N = N; Q.K = K; Q.ldo = ldo; Q.X = X;
  Q.tiles = (N + TC_BM - 1) / TC_BM;
  Q.n_kb = (K + TC_BK - 1) / TC_BK;
  Q.total_kb = Q.tiles * Q.n_kb;
  g_last_parts = Q.tiles;
  // rings of about 180 KB: what is in flight per SM decides the rate at which weights stream in (rings half
  // as deep, two CTAs per SM, ran a third slower)
  if (bn == 16) return launch_streamk<16, SK_RING_16>(ma, mb, Q, epilogue, stream);
  if (bn == 32) return launch_streamk<32, SK_RING_32>(ma, mb, Q, epilogue, stream);
  if (bn == 64) return launch_streamk<64, SK_RING_64>(ma, mb, Q, epilogue, stream);
  return launch_streamk<128, SK_RING_128>(ma, mb, Q, epilogue, stream);
}

STRATUM_EXPORT int stratum_gemm_tc(const void* x, const void* w, const float* bias, void* out, int epilogue, int M,
                                   int N, int K, int ldx, int ldo, int* status, float* scratch,
                                   cudaStream_t stream) {
  if (epilogue < 0 || epilogue > 3) return STRATUM_ERR_SHAPE;
  return stratum_gemm_tc_ex(x, w, bias, out, epilogue, M, N, K, ldx, ldo, status, scratch, nullptr, stream);
}
