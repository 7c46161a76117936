// Causal grouped-query attention for prompts on the 5th-generation tensor cores (TMA + tcgen05 + TMEM).
//
// For query head h at position p:  score_t = (q_h . K_t[kv(h)]) * scale over keys t in [lo, p];
// p_t = softmax;  o_h = sum_t p_t V_t[kv(h)]  (stratum/native/stratum_arch_llama.inc.c:435-514).
//
// One CTA owns 128 query rows that share a kv head: 128/gs consecutive new tokens of one sequence times the
// gs heads of the group (row = token * gs + head).  It walks over the sequence's keys in tiles of 64, which is
// exactly one page of the cache, so a K or V tile is one contiguous [64][Hd] block fetched by TMA.
//
//   warp 0      producer: Q once (3-D box: dims x heads of the group x tokens), then K and V tiles into a ring
//   warp 1      one lane issues the MMAs:  S = Q K^T  (128 x 64, into one of two TMEM buffers) and, once the
//               softmax warps have written P,  O += P V  (128 x Hd, accumulated in TMEM over all tiles)
//   warps 2-9   softmax, two threads per row (each owns half of the keys of a tile and half of the output
//               dimensions): read S from TMEM, mask, maximum in float32, exponentials, write P as bfloat16 into
//               shared memory in the swizzled layout the MMA reads.
//
// The exponentials of a row are taken against a reference maximum that is only moved when the row's maximum has
// grown by more than 2^8 beyond it: exp2(s - ref) then stays below 2^8, exactly representable scaling that the
// final division by the row's sum (taken against the same reference) removes again.  Moving the reference means
// multiplying the row of O in TMEM (tcgen05.ld, multiply, tcgen05.st); after the first tiles of a row this is
// rare, so per tile a softmax thread touches S and P only, and its few registers let two CTAs share an SM: one
// CTA's MMAs run under the other's softmax.
//
// Two forms.  NH = 1: one CTA owns 128 query rows and two CTAs share an SM.  NH = 2: one CTA owns 256 query rows
// as two halves of 128 (64 / gs consecutive tokens each), each half with its own MMA-issuing warp, eight softmax
// warps, S buffers, P buffer and O accumulator, exactly as in a CTA of the first form; the halves share the
// producer and the K and V rings, so every key and value tile is fetched from L2 once for 256 rows instead of once
// for 128.  That traffic is what bounds the first form on long prompts: with every MMA and every exponential taken
// out, a prompt of 8,192 tokens still took 251 of its 560 us, fetching 4.3 GB of K and V tiles at 17 TB/s.
//
// V is used as stored, [key][dim]: as the B operand of P V its n index (dim) is the contiguous one
// ("MN-major"), which the instruction takes directly; no transpose is made anywhere.
//
// Every mbarrier wait is bounded (see gemm_tc.cu): on expiry a code goes to the status word and the CTA winds
// down, freeing its tensor memory.
#include <math.h>

#include "tc_common.cuh"

#define FA_ROWS 128
#define FA_KEYS 64
#define FA_STAGES 2
#define FA_SOFTMAX_WARPS 8                         // per half
#define FA_THREADS(NH) (32 + (NH) * 32 + (NH) * FA_SOFTMAX_WARPS * 32)

struct FaParams {
  const int* token_pos;
  const int* block_table; int bt_stride;
  const int* qb_seq; const int* qb_tok0; const int* qb_ntok;
  bf16* out; int ldo;
  int* status;
  int n_q, n_kv, gs, tokens_per_tile, window;
  float scale_log2;        // scale * log2(e): exponentials are taken with exp2
};

template <int HD, int NH>
struct FaSmem {
  alignas(1024) bf16 q[NH][FA_ROWS * HD];             // per half: [HD/64 blocks of 64 dims][128 rows][64]
  alignas(1024) bf16 k[FA_STAGES][FA_KEYS * HD];      // [HD/64][64 keys][64 dims]
  alignas(1024) bf16 v[FA_STAGES][FA_KEYS * HD];      // [HD/64][64 keys][64 dims]
  alignas(1024) bf16 p[NH][FA_ROWS * FA_KEYS];        // per half: [128 rows][64 keys]; at the end: the rows' two half sums
  uint64_t q_full, k_full[FA_STAGES], v_full[FA_STAGES];
  uint64_t s_full[NH][2], p_full[NH], pv_full[NH][2];
  uint32_t tmem_base;
  int abort_flag;
};

// max(a, b, c) in one instruction (sm_100 has the three-input form)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define FA_FAIL(code) { atomicCAS(P.status, 0, code); S.abort_flag = 1; }

// What one half (128 query rows) of a CTA works on.
struct FaHalf {
  int ntok, first_pos, last_pos, n_tiles;
};
__device__ __forceinline__ FaHalf fa_half(const FaParams& P, int h, int seq, int first_pos, int ntok, int lo_tile) {
  FaHalf H;
  H.ntok = min(max(ntok - h * P.tokens_per_tile, 0), P.tokens_per_tile);
  H.first_pos = first_pos + h * P.tokens_per_tile;
  H.last_pos = H.first_pos + H.ntok - 1;
  H.n_tiles = (seq < 0 || H.ntok <= 0) ? 0 : H.last_pos / FA_KEYS - lo_tile + 1;
  return H;
}

template <int HD, int NH>
__global__ void __launch_bounds__(FA_THREADS(NH), NH == 1 ? 2 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const FaParams P) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using Smem = FaSmem<HD, NH>;
  Smem& S = *reinterpret_cast<Smem*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int DB = HD / 64;                           // blocks of 64 dims
  constexpr uint32_t TMEM_COLS = 256 * NH;              // per half: S0 | S1 | O (Hd columns); an SM has 512
  constexpr uint32_t COL_PV = 128;
  pdl_trigger();
  // the swizzled tiles need 1024-byte alignment, and there is no room to round the base up when two CTAs are to
  // share an SM
  if (smem_u32(smem_raw) & 1023) {
    if (threadIdx.x == 0) atomicCAS(P.status, 0, 210);
    return;
  }
  // heaviest tiles first, for all kv heads: the last query tiles of a long prompt see the most keys
  const int qb = (int)(gridDim.x / P.n_kv) - 1 - (int)(blockIdx.x / P.n_kv);
  const int kvh = blockIdx.x % P.n_kv;
  const int seq = P.qb_seq[qb];
  const int tok0 = P.qb_tok0[qb], ntok = P.qb_ntok[qb];
  if (seq < 0 || ntok <= 0) {          // an entry beyond the step's blocks (lists of a fixed length: replayed steps)
    pdl_wait();                        // no CTA leaves before the kernel before this one is done
    return;
  }
  volatile int* abort_flag = &S.abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(&S.q_full, 1);
    for (int s = 0; s < FA_STAGES; s++) { mbar_init(&S.k_full[s], 1); mbar_init(&S.v_full[s], 1); }
    for (int h = 0; h < NH; h++) {
      for (int b = 0; b < 2; b++) { mbar_init(&S.s_full[h][b], 1); mbar_init(&S.pv_full[h][b], 1); }
      mbar_init(&S.p_full[h], FA_SOFTMAX_WARPS);
    }
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

  // keys are walked from the first half's first tile (a later half whose window begins further on masks them out)
  const int first_pos = P.token_pos[tok0];
  const int lo_tile = (P.window > 0 && first_pos - P.window + 1 > 0) ? (first_pos - P.window + 1) / FA_KEYS : 0;
  const int nt0 = fa_half(P, 0, seq, first_pos, ntok, lo_tile).n_tiles;
  const int nt1 = NH > 1 ? fa_half(P, 1, seq, first_pos, ntok, lo_tile).n_tiles : 0;      // (never more than nt0 + 1)
  const int n_tiles_max = max(nt0, nt1);

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && n_tiles_max > 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      pdl_wait();                                        // q and the newest keys come from the kernel before
      const int live = (nt0 > 0) + (nt1 > 0);
      mbar_expect_tx(&S.q_full, (uint32_t)live * FA_ROWS * HD * sizeof(bf16));
#pragma unroll
      for (int h = 0; h < NH; h++)
        if ((h == 0 ? nt0 : nt1) > 0)
          for (int db = 0; db < DB; db++)
            tma_load_3d(&map_q, S.q[h] + db * FA_ROWS * 64, &S.q_full, db * 64, kvh * P.gs, tok0 + h * P.tokens_per_tile);
      const int* bt = P.block_table + (size_t)seq * P.bt_stride;
      // K and V have rings of their own: a K tile is free again as soon as its scores are computed (s_full), a
      // whole tile earlier than the V tile beside it (pv_full), so the next K is already on its way while P V still
      // runs.  One thread feeds both rings, polling (never suspended in a wait on one ring while the other has room).
      // The MMA threads pay about a hundred cycles for every instruction they issue, commits and waits included:
      // so no barrier exists only to free a buffer.  (The S buffer of tile j-1 is free for tile j+1 once P of tile
      // j-1 has arrived, which the MMA thread has waited for by then.)  With two halves a stage is free once every
      // half that walks that tile has read it.
      auto k_free = [&](int j) -> bool {                 // tile j - 2 has left the K stage that tile j wants
        bool ok = true;
#pragma unroll
        for (int h = 0; h < NH; h++)
          if (j - 2 < (h == 0 ? nt0 : nt1)) ok = ok && mbar_test_wait(&S.s_full[h][j & 1], ((j - 2) >> 1) & 1);
        return ok;
      };
      auto v_free = [&](int j) -> bool {
        bool ok = true;
#pragma unroll
        for (int h = 0; h < NH; h++)
          if (j - 2 < (h == 0 ? nt0 : nt1)) ok = ok && mbar_test_wait(&S.pv_full[h][j & 1], ((j - 2) >> 1) & 1);
        return ok;
      };
      bool ok = true;
      int jk = 0, jv = 0;
      uint32_t idle = 0;
      while ((jk < n_tiles_max || jv < n_tiles_max) && ok) {
        bool moved = false;
        if (jk < n_tiles_max && (jk < 2 || k_free(jk))) {
          const int s = jk % FA_STAGES;
          const int row = (bt[lo_tile + jk] * P.n_kv + kvh) * FA_KEYS;
          mbar_expect_tx(&S.k_full[s], FA_KEYS * HD * sizeof(bf16));
          for (int db = 0; db < DB; db++) tma_load_2d(&map_k, S.k[s] + db * FA_KEYS * 64, &S.k_full[s], db * 64, row);
          jk++; moved = true;
        }
        if (jv < n_tiles_max && (jv < 2 || v_free(jv))) {
          const int s = jv % FA_STAGES;
          const int row = (bt[lo_tile + jv] * P.n_kv + kvh) * FA_KEYS;
          mbar_expect_tx(&S.v_full[s], FA_KEYS * HD * sizeof(bf16));
          for (int db = 0; db < DB; db++) tma_load_2d(&map_v, S.v[s] + db * FA_KEYS * 64, &S.v_full[s], db * 64, row);
          jv++; moved = true;
        }
        if (moved) { idle = 0; continue; }
        __nanosleep(64);                       // (a hot poll would take issue slots from the softmax warps beside it)
        if (++idle >= 4u * TC_SPIN_LIMIT || ((idle & 1023u) == 0 && *abort_flag)) { FA_FAIL(201); ok = false; }
      }
      if (!ok) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);   // let copies already issued land
      }
    }
  } else if (warp <= NH) {
    // ---------------------------------------------------------------- MMA issuer of half `warp - 1`
    // The whole warp walks through the waits together and one elected lane issues: with warp-uniform control
    // flow the operands of the MMAs (descriptors, addresses) stay warp-uniform values.
    const int h = warp - 1;
    const int n_tiles = h == 0 ? nt0 : nt1;
    if (n_tiles > 0) {
      const uint32_t idesc_s = instr_desc_bf16(FA_KEYS);
      const uint32_t idesc_pv = instr_desc_bf16(HD, true);
      const uint32_t tmem_h = tmem_base + h * 256;
      bool ok = __all_sync(0xffffffffu, mbar_wait(&S.q_full, 0, abort_flag));
      if (!ok && lane == 0) FA_FAIL(202);
      const uint32_t q_addr = smem_u32(S.q[h]), p_addr = smem_u32(S.p[h]);
      auto issue_scores = [&](int j) -> bool {
        const int s = j % FA_STAGES, b = j & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&S.k_full[s], (j / FA_STAGES) & 1, abort_flag))) {
          if (lane == 0) FA_FAIL(203);
          return false;
        }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(S.k[s]);
        if (elect_one()) {
#pragma unroll
          for (int db = 0; db < DB; db++)
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
              umma_bf16(tmem_h + b * FA_KEYS, smem_desc_sw128(q_addr + db * FA_ROWS * 128 + kk * 32),
                        smem_desc_sw128(k_addr + db * FA_KEYS * 128 + kk * 32), idesc_s, (db | kk) ? 1u : 0u);
          umma_commit(&S.s_full[h][b]);         // to the softmax warps, and to the producer: K of this tile is read
        }
        __syncwarp();
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < n_tiles && ok; j++) {
        if (j + 1 < n_tiles) { ok = issue_scores(j + 1); if (!ok) break; }
        const int s = j % FA_STAGES;
        if (!__all_sync(0xffffffffu, mbar_wait(&S.p_full[h], j & 1, abort_flag))) { if (lane == 0) FA_FAIL(205); ok = false; break; }
        if (!__all_sync(0xffffffffu, mbar_wait(&S.v_full[s], (j / FA_STAGES) & 1, abort_flag))) { if (lane == 0) FA_FAIL(206); ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(S.v[s]);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; kk++)        // 16 keys a step: 32 bytes along a row of P, 16 rows of V
            umma_bf16(tmem_h + COL_PV, smem_desc_sw128(p_addr + kk * 32),
                      smem_desc_sw128_mn(v_addr + kk * 16 * 128, FA_KEYS * 128), idesc_pv, (j | kk) ? 1u : 0u);
          umma_commit(&S.pv_full[h][j & 1]);    // to the softmax warps (P is read, O has the tile), and to the
                                                // producer: V of this tile is read
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (eight warps per half)
    const int sw = warp - (1 + NH);
    const int h = sw / FA_SOFTMAX_WARPS;
    const FaHalf H = fa_half(P, h, seq, first_pos, ntok, lo_tile);
    const int n_tiles = H.n_tiles;
    if (n_tiles > 0) {
    const int quarter = warp & 3;                        // TMEM lanes this warp may read
    const int half = (sw % FA_SOFTMAX_WARPS) >> 2;       // 0: keys 0..31 and dims 0..Hd/2-1;  1: the other halves
    const int row = quarter * 32 + lane;
    const int tok = row / P.gs, head = row % P.gs;
    const bool valid = tok < H.ntok;
    const int pos = H.first_pos + (valid ? tok : 0);
    const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + h * 256 + ((uint32_t)(quarter * 32) << 16);
    constexpr int OD = HD / 2;                           // output dims per thread
    const uint32_t o_addr = lane_addr + COL_PV + half * OD;
    float m_ref = -INFINITY, l = 0.f;                    // reference maximum (scaled, log2 domain); sum of this half
    bool ok = true;

    for (int j = 0; j < n_tiles; j++) {
      const int b = j & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(&S.s_full[h][b], (j >> 1) & 1, abort_flag))) {   // (a warp gives up as one)
        if (lane == 0) FA_FAIL(209);
        ok = false;
        break;
      }
      tc_fence_after();
      float s[32], t[32];                                // this thread's half of the keys, and the other half
      tmem_ld32f(lane_addr + b * FA_KEYS + half * 32, s);
      tmem_ld32f(lane_addr + b * FA_KEYS + (half ^ 1) * 32, t);
      tmem_ld_wait();
      // maximum over the whole tile; keys beyond a row's own position (or before its window) are masked, which
      // only tiles on the diagonal (or at the window's edge) need
      const int key0 = (lo_tile + j) * FA_KEYS;
      const bool needs_mask = (key0 + FA_KEYS - 1 > H.first_pos) || (P.window > 0) || (H.ntok < P.tokens_per_tile);
      // (four running maxima, then combined: one chain of 64 dependent comparisons would cost more time than
      // everything else a thread does per tile)
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (needs_mask) {
        const int ks = key0 + half * 32, kt = key0 + (half ^ 1) * 32;
#pragma unroll
        for (int i = 0; i < 32; i++) {
          s[i] = (valid && ks + i <= pos && ks + i >= lo) ? s[i] : -INFINITY;
          t[i] = (valid && kt + i <= pos && kt + i >= lo) ? t[i] : -INFINITY;
          mx[i & 3] = max3(mx[i & 3], s[i], t[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; i++) mx[i & 3] = max3(mx[i & 3], s[i], t[i]);
      }
      float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      tile_max *= P.scale_log2;                          // scale > 0: the maximum of the scaled scores
      // the reference moves only when the row's maximum has outgrown it by more than 8 (a factor 256); both
      // threads of a row see the same numbers and decide alike
      const bool grow = tile_max > m_ref + 8.0f;
      const float corr = grow ? fast_exp2(m_ref - tile_max) : 1.0f;     // exp2(-inf) = 0 at a row's first keys
      if (grow) m_ref = tile_max;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // probabilities exp2(s * scale - ref) of this thread's keys, their sum, and P in the layout the MMA reads
      uint32_t packed[16];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float p0 = fast_exp2(fmaf(s[i], P.scale_log2, -m_use));
        const float p1 = fast_exp2(fmaf(s[i + 1], P.scale_log2, -m_use));
        // to bfloat16 by dropping the low mantissa bits (one byte permute for two values; the conversion
        // instruction shares the exponential's pipe, which is the busiest one here).  The probabilities are
        // positive, so every one comes out low by a factor in (1 - 2^-7, 1]; the sums below run over the same
        // shortened values, so the common part of that factor divides out and what stays is as wide as
        // round-to-nearest's error.
        const uint32_t u = __byte_perm(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
        sum0 += __uint_as_float(u << 16);
        sum1 += __uint_as_float(u & 0xffff0000u);
        packed[i >> 1] = u;
      }
      if (j > 0) {
        // P V of the tile before has read P and has been added into O
        if (!__all_sync(0xffffffffu, mbar_wait(&S.pv_full[h][(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag))) {
          if (lane == 0) FA_FAIL(208);
          ok = false;
          break;
        }
        if (__any_sync(0xffffffffu, grow)) {             // some row of this warp moves its reference: rescale O
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < OD; c += 32) {
            uint32_t r[32];
            tmem_ld32(o_addr + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
            tmem_st32(o_addr + c, r);
          }
          tmem_st_wait();
        }
      }
      l = l * corr + (sum0 + sum1);
      {
        uint8_t* prow = reinterpret_cast<uint8_t*>(S.p[h]) + row * 128;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int chunk = half * 4 + c;                // 16-byte chunk = 8 keys
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
        }
      }
      fence_async_shared();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.p_full[h]);
    }
    if (ok && !__all_sync(0xffffffffu, mbar_wait(&S.pv_full[h][(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort_flag))) {
      if (lane == 0) FA_FAIL(208);
      ok = false;
    }
    tc_fence_after();
    // the two halves of the keys kept separate sums: add them (P is no longer read; named barrier among the
    // softmax warps of this half of the rows, reached by all of them)
    float* l_buf = reinterpret_cast<float*>(S.p[h]);
    l_buf[half * FA_ROWS + row] = l;
    if (h == 0) asm volatile("bar.sync 1, %0;" ::"n"(FA_SOFTMAX_WARPS * 32) : "memory");
    else asm volatile("bar.sync 2, %0;" ::"n"(FA_SOFTMAX_WARPS * 32) : "memory");
    if (ok && !S.abort_flag) {
      const float inv = 1.0f / (l_buf[row] + l_buf[FA_ROWS + row]);
      bf16* op = P.out + (size_t)(tok0 + h * P.tokens_per_tile + (valid ? tok : 0)) * P.ldo +
                 (size_t)(kvh * P.gs + head) * HD + half * OD;
#pragma unroll
      for (int c = 0; c < OD; c += 32) {
        float o[32];
        tmem_ld32f(o_addr + c, o);                       // (all lanes take part in the load; only valid rows store)
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv);
            __nv_bfloat162 a1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv);
            __nv_bfloat162 a3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
            w.x = *reinterpret_cast<uint32_t*>(&a0); w.y = *reinterpret_cast<uint32_t*>(&a1);
            w.z = *reinterpret_cast<uint32_t*>(&a2); w.w = *reinterpret_cast<uint32_t*>(&a3);
            *reinterpret_cast<uint4*>(op + c + i) = w;
          }
        }
      }
    }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
static int make_map_nd(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                       const cuuint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return STRATUM_ERR_LIMIT;
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : STRATUM_ERR_SHAPE;
}

template <int HD, int NH>
static int launch_attention_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FaParams& P,
                               int n_qblocks, cudaStream_t stream) {
  const size_t smem = sizeof(FaSmem<HD, NH>);
  auto kern = attention_tc_kernel<HD, NH>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(kern, dim3((unsigned)n_qblocks * P.n_kv), FA_THREADS(NH), smem, stream, mq, mk, mv, P);
}

// q: bf16 [tokens][ldq], query heads first (n_q * head_dim values per row are used).
// k_cache / v_cache: bf16 [n_pages][n_kv][64][head_dim].  Query tiles (qb_*): runs of at most
// halves * 128 / (n_q / n_kv) consecutive new tokens of one sequence (halves: 1 or 2, see the top of this file).
// head_dim 64 or 128; 128 % (n_q / n_kv) == 0; pages of 64 tokens.
STRATUM_EXPORT int stratum_attention_tc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                        long long n_pages, const int* token_pos, const int* block_table,
                                        int bt_stride, const int* qb_seq, const int* qb_tok0, const int* qb_ntok,
                                        int n_qblocks, void* out, int ldo, int n_tokens, int n_q, int n_kv,
                                        int head_dim, int page_tokens, int window, float scale, int halves,
                                        int* status, cudaStream_t stream) {
  if (n_tokens <= 0 || n_qblocks <= 0) return 0;
  if (halves != 1 && halves != 2) return STRATUM_ERR_SHAPE;
  if (head_dim != 64 && head_dim != 128) return STRATUM_ERR_SHAPE;
  if (n_kv < 1 || n_q % n_kv != 0 || page_tokens != FA_KEYS) return STRATUM_ERR_SHAPE;
  const int gs = n_q / n_kv;
  if (gs > FA_ROWS || FA_ROWS % gs != 0) return STRATUM_ERR_SHAPE;
  if (ldq % 8 != 0 || ldo % 8 != 0 || !status || !qb_seq || !qb_tok0 || !qb_ntok) return STRATUM_ERR_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return STRATUM_ERR_ALIGN;
  if ((long long)n_qblocks * n_kv > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  const int R = FA_ROWS / gs;
  CUtensorMap mq, mk, mv;
  int st;
  {  // q as [tokens][n_q heads][head_dim]; a box is 64 dims x gs heads x R tokens: rows token * gs + head
    cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)n_q, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * sizeof(bf16), (cuuint64_t)ldq * sizeof(bf16)};
    cuuint32_t box[3] = {64, (cuuint32_t)gs, (cuuint32_t)R};
    if ((st = make_map_nd(&mq, q, 3, dims, strides, box)) != 0) return st;
  }
  {  // the cache as [pages * n_kv * 64 rows][head_dim]; a box is 64 dims x 64 keys
    cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)n_pages * n_kv * FA_KEYS};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * sizeof(bf16)};
    cuuint32_t box[2] = {64, FA_KEYS};
    if ((st = make_map_nd(&mk, k_cache, 2, dims, strides, box)) != 0) return st;
    if ((st = make_map_nd(&mv, v_cache, 2, dims, strides, box)) != 0) return st;
  }
  FaParams P;
  P.token_pos = token_pos; P.block_table = block_table; P.bt_stride = bt_stride;
  P.qb_seq = qb_seq; P.qb_tok0 = qb_tok0; P.qb_ntok = qb_ntok;
  P.out = (bf16*)out; P.ldo = ldo; P.status = status;
  P.n_q = n_q; P.n_kv = n_kv; P.gs = gs; P.tokens_per_tile = R; P.window = window;
  P.scale_log2 = scale * 1.4426950408889634f;
  if (halves == 2) {
    if (head_dim == 64) return launch_attention_tc<64, 2>(mq, mk, mv, P, n_qblocks, stream);
    return launch_attention_tc<128, 2>(mq, mk, mv, P, n_qblocks, stream);
  }
  if (head_dim == 64) return launch_attention_tc<64, 1>(mq, mk, mv, P, n_qblocks, stream);
  return launch_attention_tc<128, 1>(mq, mk, mv, P, n_qblocks, stream);
}
