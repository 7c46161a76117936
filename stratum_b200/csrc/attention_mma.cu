// Causal grouped-query attention over the paged bfloat16 cache on tensor cores, for prompts and for
// decode steps, with the keys of long sequences split across warps (scratch partials + a merge).
//
// One warp owns one work item: up to 16 query rows that share a kv head (R consecutive new tokens of
// a sequence x the heads of the group), and one contiguous range of that sequence's keys.  Scores
// and the value sum are mma.sync.m16n8k16 (bf16 in, float32 accumulate); maxima, exponentials,
// denominators and the running rescale are float32 (online softmax); nothing goes through
// shared memory.  For query head h at position p:  score_t = (q_h . K_t[kv(h)]) * scale over keys
// t in [lo, p];  p_t = softmax;  o_h = sum_t p_t V_t[kv(h)]
// (stratum/native/stratum_arch_llama.inc.c:435-514; kv(h) = h / (Nq/Nk), :444).
//
// Fragments straight from global memory.  Lane (g = lane/4, t = lane%4) loads, of every 32-wide
// chunk of the head dimension, the 8 contiguous values 8t..8t+7 of its row: for Q rows g and g+8
// (the A operand), for K rows key0+g and key0+8+g (the B operand of Q K^T; a dot product may
// visit the head dimension in any order as long as Q and K agree).  V has keys along k, which is
// the transposed arrangement; each 32-bit register of the same kind of load is an 8x8 matrix that
// movmatrix transposes into a B fragment whose column n stands for dimension 8(n/2)+2i+(n%2) of
// the chunk.  The accumulator for output tile (chunk c, register i) then holds, in lane (g,t),
// dimensions 32c+8t+2i and +1: the four tiles of a chunk give 8 contiguous output values per row.
//
// Key ranges: the keys of a sequence are cut into `chunk` keys per split (a multiple of 64).  With
// one split the normalised output is written directly.  With more, every split writes its
// unnormalised value sum, its maximum and its denominator to scratch, and a second kernel merges
// them in split order.
#include <math.h>

#include "common.cuh"
#include "mma_common.cuh"

#define AM_WARPS 4

// q and the newest rows of the cache were written by the kernel before this one
__device__ __forceinline__ uint4 ldg16(const void* p) { return ld_fresh((const uint4*)p); }

struct AttnParams {
  const bf16* q; int ldq;              // [tokens][ldq]: query heads first
  const bf16* k_cache; const bf16* v_cache;   // [pages][Nk][page_tokens][Hd]
  const int* token_pos;                // [tokens]
  const int* token_seq;                // [tokens]: index of the token's sequence in the step, -1 = padding
  const int* block_table; int bt_stride;      // [seqs][bt_stride]
  const int* qb_seq; const int* qb_tok0; const int* qb_ntok;   // query blocks; null = one token per sequence
  int n_qblocks;
  bf16* out; int ldo;                  // [tokens][ldo]
  float* part_o; float* part_ml;       // scratch: [(token*Nq + head)*n_splits + split][Hd] and [..][2]
  int n_q, n_kv, head_dim, page_tokens, window;
  int rows_per_token, head_groups, tokens_per_block;
  int n_splits, chunk;
  float scale;
};

// One block of 16 keys for the 16 query rows of a warp: scores, mask, online softmax, value sum.
// ka/kb: K rows key0+g / key0+8+g; va/vb: V rows likewise (8 contiguous dims per chunk, see the top comment).
template <int CH>
__device__ __forceinline__ void attend_block(const AttnParams& P, const uint4 (&qa)[CH], const uint4 (&qc)[CH],
                                             const uint4 (&ka)[CH], const uint4 (&kb)[CH], const uint4 (&va)[CH],
                                             const uint4 (&vb)[CH], float (&o)[4 * CH][4], float (&m_run)[2],
                                             float (&l_run)[2], const bool (&row_ok)[2], const int (&row_pos)[2],
                                             int key0, int k_end, int t) {
  // scores: s[i] is the tile of keys key0 + 8i + {2t, 2t+1}; [0],[1] row g, [2],[3] row g+8
  float s[2][4];
#pragma unroll
  for (int i = 0; i < 2; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
  for (int c = 0; c < CH; c++) {
    mma16816(s[0], qa[c].x, qc[c].x, qa[c].y, qc[c].y, ka[c].x, ka[c].y);
    mma16816(s[0], qa[c].z, qc[c].z, qa[c].w, qc[c].w, ka[c].z, ka[c].w);
    mma16816(s[1], qa[c].x, qc[c].x, qa[c].y, qc[c].y, kb[c].x, kb[c].y);
    mma16816(s[1], qa[c].z, qc[c].z, qa[c].w, qc[c].w, kb[c].z, kb[c].w);
  }
  // mask, scale, running maximum
  float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < 2; i++) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int e = j >> 1;
      const int key = key0 + 8 * i + 2 * t + (j & 1);
      const int lo = (P.window > 0 && row_pos[e] - P.window + 1 > 0) ? row_pos[e] - P.window + 1 : 0;
      const bool ok = row_ok[e] && key <= row_pos[e] && key >= lo && key < k_end;
      s[i][j] = ok ? s[i][j] * P.scale : -INFINITY;
      bm[e] = fmaxf(bm[e], s[i][j]);
    }
  }
  float corr[2], m_use[2];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 1));
    bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 2));
    const float m_new = fmaxf(m_run[e], bm[e]);
    m_use[e] = (m_new == -INFINITY) ? 0.f : m_new;      // a row with no key yet: exponents of -inf give 0
    corr[e] = __expf(m_run[e] - m_use[e]);              // first keys: exp(-inf) = 0
    m_run[e] = m_new;
  }
  float p[2][4];
#pragma unroll
  for (int i = 0; i < 2; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) p[i][j] = __expf(s[i][j] - m_use[j >> 1]);
#pragma unroll
  for (int e = 0; e < 2; e++)
    l_run[e] = l_run[e] * corr[e] + (p[0][2 * e] + p[0][2 * e + 1] + p[1][2 * e] + p[1][2 * e + 1]);
#pragma unroll
  for (int i = 0; i < 4 * CH; i++) {
    o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
  }
  // the value sum uses probabilities rounded to bfloat16, as its tensor-core operand must be
  const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]), pa1 = pack_bf16(p[0][2], p[0][3]);
  const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]), pa3 = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
  for (int c = 0; c < CH; c++) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t b0 = transpose8x8(reg_of(va[c], i));
      const uint32_t b1 = transpose8x8(reg_of(vb[c], i));
      mma16816(o[4 * c + i], pa0, pa1, pa2, pa3, b0, b1);
    }
  }
}

template <int CH>
__global__ void __launch_bounds__(AM_WARPS * 32)
attention_mma_kernel(const AttnParams P) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_trigger();
  // the step's description (positions, page tables, query blocks) is read before waiting for the kernel
  // that wrote q and the newest keys; q and the cache only after it
  long long item = (long long)blockIdx.x * AM_WARPS + warp;
  const long long n_items = (long long)P.n_qblocks * P.n_kv * P.head_groups * P.n_splits;
  if (item >= n_items) return;
  const int split = (int)(item % P.n_splits); item /= P.n_splits;
  const int hg = (int)(item % P.head_groups); item /= P.head_groups;
  const int kvh = (int)(item % P.n_kv); item /= P.n_kv;
  const int qb = (int)item;
  const int seq = P.qb_seq ? P.qb_seq[qb] : P.token_seq[qb];
  const int tok0 = P.qb_tok0 ? P.qb_tok0[qb] : qb;
  const int ntok = P.qb_ntok ? P.qb_ntok[qb] : 1;
  if (seq < 0) return;                                    // padding
  const int gs = P.n_q / P.n_kv;
  const int Hd = P.head_dim;

  // the two rows of this lane: r = g and g + 8;  row -> (token of the block, head of the group)
  int row_tok[2], row_head[2], row_pos[2];
  bool row_ok[2];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = g + 8 * e;
    const int tr = r / P.rows_per_token, hr = r % P.rows_per_token;
    const int hq = hg * 16 + hr;                          // head within the group
    row_ok[e] = tr < ntok && tr < P.tokens_per_block && hq < gs;
    row_tok[e] = tok0 + (row_ok[e] ? tr : 0);
    row_head[e] = kvh * gs + (row_ok[e] ? hq : 0);
    row_pos[e] = P.token_pos[row_tok[e]];
  }
  const int first_pos = P.token_pos[tok0];
  const int last_pos = first_pos + ntok - 1;
  const int lo_block = (P.window > 0 && first_pos - P.window + 1 > 0) ? first_pos - P.window + 1 : 0;
  int k_begin = split * P.chunk, k_end = min((split + 1) * P.chunk, last_pos + 1);
  if (k_begin < (lo_block / 16) * 16) k_begin = (lo_block / 16) * 16;

  const int* bt = P.block_table + (size_t)seq * P.bt_stride;
  const int first_page = (k_begin < k_end) ? bt[k_begin / P.page_tokens] : 0;
  pdl_wait();

  // Q fragments
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  uint4 qa[CH], qc[CH];
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int d = 32 * c + 8 * t;
    const bool d_ok = d < Hd;
    qa[c] = (row_ok[0] && d_ok) ? ldg16(P.q + (size_t)row_tok[0] * P.ldq + (size_t)row_head[0] * Hd + d) : zero4;
    qc[c] = (row_ok[1] && d_ok) ? ldg16(P.q + (size_t)row_tok[1] * P.ldq + (size_t)row_head[1] * Hd + d) : zero4;
  }

  float o[4 * CH][4];
#pragma unroll
  for (int i = 0; i < 4 * CH; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const size_t head_off = (size_t)kvh * P.page_tokens * Hd;
  const size_t page_stride = (size_t)P.n_kv * P.page_tokens * Hd;

  // K of the next block of 16 keys is requested before the current block is worked on; V of the current block
  // is requested first thing, so that it arrives while the scores are computed.
  auto block_base = [&](int key0) -> size_t {
    const int page = (key0 == k_begin) ? first_page : bt[key0 / P.page_tokens];
    return (size_t)page * page_stride + head_off + (size_t)(key0 % P.page_tokens) * Hd;
  };
  uint4 ka[CH], kb[CH];
  size_t base = 0;
  if (k_begin < k_end) {
    base = block_base(k_begin);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      ka[c] = d < Hd ? ldg16(P.k_cache + base + (size_t)g * Hd + d) : zero4;
      kb[c] = d < Hd ? ldg16(P.k_cache + base + (size_t)(g + 8) * Hd + d) : zero4;
    }
  }
  for (int key0 = k_begin; key0 < k_end; key0 += 16) {
    const bf16* vp = P.v_cache + base;
    uint4 va[CH], vb[CH], nka[CH], nkb[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      va[c] = d < Hd ? ldg16(vp + (size_t)g * Hd + d) : zero4;
      vb[c] = d < Hd ? ldg16(vp + (size_t)(g + 8) * Hd + d) : zero4;
    }
    const bool more = key0 + 16 < k_end;
    if (more) base = block_base(key0 + 16);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      nka[c] = (more && d < Hd) ? ldg16(P.k_cache + base + (size_t)g * Hd + d) : zero4;
      nkb[c] = (more && d < Hd) ? ldg16(P.k_cache + base + (size_t)(g + 8) * Hd + d) : zero4;
    }
    attend_block<CH>(P, qa, qc, ka, kb, va, vb, o, m_run, l_run, row_ok, row_pos, key0, k_end, t);
#pragma unroll
    for (int c = 0; c < CH; c++) { ka[c] = nka[c]; kb[c] = nkb[c]; }
  }
  // denominators across the four lanes of a row
#pragma unroll
  for (int e = 0; e < 2; e++) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
#pragma unroll
  for (int e = 0; e < 2; e++) {
    if (!row_ok[e]) continue;
    if (P.n_splits == 1) {
      const float inv = 1.0f / l_run[e];
      bf16* op = P.out + (size_t)row_tok[e] * P.ldo + (size_t)row_head[e] * Hd;
#pragma unroll
      for (int c = 0; c < CH; c++) {
        const int d = 32 * c + 8 * t;
        if (d >= Hd) continue;
        uint4 v;
        v.x = pack_bf16(o[4 * c + 0][2 * e] * inv, o[4 * c + 0][2 * e + 1] * inv);
        v.y = pack_bf16(o[4 * c + 1][2 * e] * inv, o[4 * c + 1][2 * e + 1] * inv);
        v.z = pack_bf16(o[4 * c + 2][2 * e] * inv, o[4 * c + 2][2 * e + 1] * inv);
        v.w = pack_bf16(o[4 * c + 3][2 * e] * inv, o[4 * c + 3][2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(op + d) = v;
      }
    } else {
      const size_t slot = ((size_t)row_tok[e] * P.n_q + row_head[e]) * P.n_splits + split;
      float* po = P.part_o + slot * Hd;
#pragma unroll
      for (int c = 0; c < CH; c++) {
        const int d = 32 * c + 8 * t;
        if (d >= Hd) continue;
        *reinterpret_cast<float4*>(po + d) =
            make_float4(o[4 * c + 0][2 * e], o[4 * c + 0][2 * e + 1], o[4 * c + 1][2 * e], o[4 * c + 1][2 * e + 1]);
        *reinterpret_cast<float4*>(po + d + 4) =
            make_float4(o[4 * c + 2][2 * e], o[4 * c + 2][2 * e + 1], o[4 * c + 3][2 * e], o[4 * c + 3][2 * e + 1]);
      }
      if (t == 0) {
        P.part_ml[slot * 2] = m_run[e];
        P.part_ml[slot * 2 + 1] = l_run[e];
      }
    }
  }
}

// ---------------------------------------------------------------- prompts: key tiles shared through shared memory
// Four warps share one kv head and 4 x 16 query rows (consecutive new tokens of one sequence x the heads of the
// group).  The keys and values they all need are brought in once per tile of 64 keys (one page, 64 x Hd x 2
// bytes each for K and V) with cp.async, two tiles in flight, and every warp reads its fragments from there with
// the same 16-byte pieces as the direct kernel above.  Pieces are stored with bit 2 of their index flipped on odd
// rows, so that the eight lanes of a quarter-warp (two rows, four pieces each) fall on different banks.
#define AT_WARPS 4
#define AT_KEYS 64

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src) : "memory");
}

template <int CH>
__global__ void __launch_bounds__(AT_WARPS * 32)
attention_tile_kernel(const AttnParams P) {
  extern __shared__ uint4 tile_smem[];           // [2 buffers][K | V][64 rows][Hd / 8 pieces]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_trigger();
  const int qb = blockIdx.x;
  const int kvh = blockIdx.y / P.head_groups, hg = blockIdx.y % P.head_groups;
  const int seq = P.qb_seq[qb];
  if (seq < 0) {                       // an entry beyond the step's blocks
    pdl_wait();                        // no CTA leaves before the kernel before this one is done
    return;
  }
  const int tok0 = P.qb_tok0[qb], ntok = P.qb_ntok[qb];
  const int gs = P.n_q / P.n_kv;
  const int Hd = P.head_dim;
  const int pieces = Hd / 8;                      // 16-byte pieces per row
  const bool swizzle = (pieces % 8) == 0;

  // this warp's share of the tile's tokens
  const int wtok0 = tok0 + warp * P.tokens_per_block;
  const int wntok = max(0, min(P.tokens_per_block, ntok - warp * P.tokens_per_block));
  int row_tok[2], row_head[2], row_pos[2];
  bool row_ok[2];
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int r = g + 8 * e;
    const int tr = r / P.rows_per_token, hr = r % P.rows_per_token;
    const int hq = hg * 16 + hr;
    row_ok[e] = tr < wntok && hq < gs;
    row_tok[e] = row_ok[e] ? wtok0 + tr : tok0;
    row_head[e] = kvh * gs + (row_ok[e] ? hq : 0);
    row_pos[e] = P.token_pos[row_tok[e]];
  }
  const int first_pos = P.token_pos[tok0];
  const int last_pos = first_pos + ntok - 1;
  const int warp_last = first_pos + warp * P.tokens_per_block + wntok - 1;     // last position this warp attends from
  const int lo_block = (P.window > 0 && first_pos - P.window + 1 > 0) ? first_pos - P.window + 1 : 0;
  const int tile_begin = lo_block / AT_KEYS, tile_end = last_pos / AT_KEYS;    // inclusive
  const int k_end = last_pos + 1;
  const int* bt = P.block_table + (size_t)seq * P.bt_stride;
  const size_t page_stride = (size_t)P.n_kv * P.page_tokens * Hd;
  const size_t head_off = (size_t)kvh * P.page_tokens * Hd;
  const int tile_pieces = AT_KEYS * pieces;       // per matrix
  pdl_wait();                                      // q and the newest keys come from the kernel before this one

  auto request_tile = [&](int tile, int buf) {
    const size_t base = (size_t)bt[tile] * page_stride + head_off;    // a page holds exactly one tile per head
    const uint4* ksrc = reinterpret_cast<const uint4*>(P.k_cache + base);
    const uint4* vsrc = reinterpret_cast<const uint4*>(P.v_cache + base);
    uint4* kdst = tile_smem + (size_t)buf * 2 * tile_pieces;
    uint4* vdst = kdst + tile_pieces;
    for (int i = threadIdx.x; i < tile_pieces; i += AT_WARPS * 32) {
      const int row = i / pieces, pc = i % pieces;
      const int at = row * pieces + (swizzle ? (pc ^ ((row & 1) << 2)) : pc);
      cp_async16(kdst + at, ksrc + i);
      cp_async16(vdst + at, vsrc + i);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  request_tile(tile_begin, 0);

  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  uint4 qa[CH], qc[CH];
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int d = 32 * c + 8 * t;
    const bool d_ok = d < Hd;
    qa[c] = (row_ok[0] && d_ok) ? ldg16(P.q + (size_t)row_tok[0] * P.ldq + (size_t)row_head[0] * Hd + d) : zero4;
    qc[c] = (row_ok[1] && d_ok) ? ldg16(P.q + (size_t)row_tok[1] * P.ldq + (size_t)row_head[1] * Hd + d) : zero4;
  }
  float o[4 * CH][4];
#pragma unroll
  for (int i = 0; i < 4 * CH; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int tile = tile_begin; tile <= tile_end; tile++) {
    const int buf = (tile - tile_begin) & 1;
    if (tile < tile_end) {
      request_tile(tile + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();                               // every thread's pieces of this tile have landed
    const uint4* ks = tile_smem + (size_t)buf * 2 * tile_pieces;
    const uint4* vs = ks + tile_pieces;
    if (wntok > 0) {
#pragma unroll 1
      for (int sub = 0; sub < AT_KEYS / 16; sub++) {
        const int key0 = tile * AT_KEYS + sub * 16;
        if (key0 > warp_last) break;               // causal: nothing of this warp sees these keys
        if (key0 + 15 < lo_block) continue;
        uint4 ka[CH], kb[CH], va[CH], vb[CH];
        const int r0 = sub * 16 + g, r1 = r0 + 8;
#pragma unroll
        for (int c = 0; c < CH; c++) {
          const int pc = 4 * c + t;
          if (pc < pieces) {
            const int a0 = r0 * pieces + (swizzle ? (pc ^ ((r0 & 1) << 2)) : pc);
            const int a1 = r1 * pieces + (swizzle ? (pc ^ ((r1 & 1) << 2)) : pc);
            ka[c] = ks[a0]; kb[c] = ks[a1]; va[c] = vs[a0]; vb[c] = vs[a1];
          } else {
            ka[c] = kb[c] = va[c] = vb[c] = zero4;
          }
        }
        attend_block<CH>(P, qa, qc, ka, kb, va, vb, o, m_run, l_run, row_ok, row_pos, key0, k_end, t);
      }
    }
    __syncthreads();                               // the buffer is refilled two tiles from now
  }
#pragma unroll
  for (int e = 0; e < 2; e++) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
#pragma unroll
  for (int e = 0; e < 2; e++) {
    if (!row_ok[e]) continue;
    const float inv = 1.0f / l_run[e];
    bf16* op = P.out + (size_t)row_tok[e] * P.ldo + (size_t)row_head[e] * Hd;
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      if (d >= Hd) continue;
      uint4 v;
      v.x = pack_bf16(o[4 * c + 0][2 * e] * inv, o[4 * c + 0][2 * e + 1] * inv);
      v.y = pack_bf16(o[4 * c + 1][2 * e] * inv, o[4 * c + 1][2 * e + 1] * inv);
      v.z = pack_bf16(o[4 * c + 2][2 * e] * inv, o[4 * c + 2][2 * e + 1] * inv);
      v.w = pack_bf16(o[4 * c + 3][2 * e] * inv, o[4 * c + 3][2 * e + 1] * inv);
      *reinterpret_cast<uint4*>(op + d) = v;
    }
  }
}

template <int CH>
static int launch_attention_tile(const AttnParams& P, cudaStream_t stream) {
  const size_t smem = (size_t)2 * 2 * AT_KEYS * P.head_dim * sizeof(bf16);
  auto kern = attention_tile_kernel<CH>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 2 * AT_KEYS * 128 * 2);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const dim3 grid(P.n_qblocks, P.n_kv * P.head_groups);
  return launch_pdl(kern, grid, AT_WARPS * 32, smem, stream, P);
}

// Prompts and continuations: query tiles of 4 x tokens_per_block tokens (qb_* lists are required).
// Needs page_tokens == 64.
STRATUM_EXPORT int stratum_attention_tile(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                          const int* token_pos, const int* token_seq, const int* block_table,
                                          int bt_stride, const int* qb_seq, const int* qb_tok0, const int* qb_ntok,
                                          int n_qblocks, int tokens_per_block, void* out, int ldo, int n_tokens,
                                          int n_q, int n_kv, int head_dim, int page_tokens, int window, float scale,
                                          cudaStream_t stream) {
  if (n_tokens <= 0 || n_qblocks <= 0) return 0;
  if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 128) return STRATUM_ERR_SHAPE;
  if (n_kv < 1 || n_q % n_kv != 0 || page_tokens != AT_KEYS) return STRATUM_ERR_SHAPE;
  if (!qb_seq || !qb_tok0 || !qb_ntok) return STRATUM_ERR_SHAPE;
  if (ldq % 8 != 0 || ldo % 8 != 0) return STRATUM_ERR_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return STRATUM_ERR_ALIGN;
  const int gs = n_q / n_kv;
  AttnParams P;
  P.q = (const bf16*)q; P.ldq = ldq;
  P.k_cache = (const bf16*)k_cache; P.v_cache = (const bf16*)v_cache;
  P.token_pos = token_pos; P.token_seq = token_seq; P.block_table = block_table; P.bt_stride = bt_stride;
  P.qb_seq = qb_seq; P.qb_tok0 = qb_tok0; P.qb_ntok = qb_ntok; P.n_qblocks = n_qblocks;
  P.out = (bf16*)out; P.ldo = ldo; P.part_o = nullptr; P.part_ml = nullptr;
  P.n_q = n_q; P.n_kv = n_kv; P.head_dim = head_dim; P.page_tokens = page_tokens; P.window = window;
  P.rows_per_token = gs < 16 ? gs : 16;
  P.head_groups = (gs + 15) / 16;
  P.tokens_per_block = tokens_per_block;
  if (tokens_per_block < 1 || tokens_per_block * P.rows_per_token > 16) return STRATUM_ERR_SHAPE;
  if ((long long)n_kv * P.head_groups > 65535) return STRATUM_ERR_LIMIT;
  P.n_splits = 1; P.chunk = 0x40000000;
  P.scale = scale;
  switch ((head_dim + 31) / 32) {
    case 1: return launch_attention_tile<1>(P, stream);
    case 2: return launch_attention_tile<2>(P, stream);
    case 3: return launch_attention_tile<3>(P, stream);
    case 4: return launch_attention_tile<4>(P, stream);
    default: return STRATUM_ERR_SHAPE;
  }
}

// ---------------------------------------------------------------- decode steps: keys along M
// One new token per sequence and at most 8 query heads per kv head.  With the query heads along M a 16-row
// MMA would be three quarters empty, and mma.sync is slow enough on this GPU for that to show next to the
// time the keys take to arrive.  So the roles are swapped: S^T = K Q^T has the 16 keys of a block along M and the
// heads along N (8 columns), and O^T = V^T P^T has 16 output dimensions along M; half as many MMAs, half as many
// accumulator registers.  Fragments still come straight from global memory:
//   K as the A operand: lane (g,t) holds rows key0+g and key0+8+g, its 8 contiguous dims per 32-dim chunk;
//   Q^T as the B operand: lane (g,t) holds head g's same 8 dims;
//   P^T: the accumulator of S^T holds (key g | g+8, heads 2t, 2t+1); packed to bfloat16 and transposed by
//        movmatrix it is the B operand (keys 2t, 2t+1 | +8; head g);
//   V^T as the A operand: each 32-bit register of a V load is an 8x8 (key, dim pair) matrix whose movmatrix
//        transpose gives (dim, keys 2t, 2t+1); registers i and i+1 of a chunk form the 16 rows of one MMA, for the
//        dims 32c + 8(g/2) + (g%2) + 2i  and  + 2(i+1).
template <int CH>
__global__ void __launch_bounds__(AM_WARPS * 32)
attention_decode_kernel(const AttnParams P) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_trigger();
  long long item = (long long)blockIdx.x * AM_WARPS + warp;
  const long long n_items = (long long)P.n_qblocks * P.n_kv * P.n_splits;
  if (item >= n_items) return;
  const int split = (int)(item % P.n_splits); item /= P.n_splits;
  const int kvh = (int)(item % P.n_kv); item /= P.n_kv;
  const int tok = (int)item;                            // token = sequence index of the step
  const int seq = P.token_seq[tok];
  if (seq < 0) return;                                    // padding
  const int gs = P.n_q / P.n_kv;
  const int Hd = P.head_dim;
  const int pos = P.token_pos[tok];
  const int lo = (P.window > 0 && pos - P.window + 1 > 0) ? pos - P.window + 1 : 0;
  int k_begin = split * P.chunk;
  const int k_end = min((split + 1) * P.chunk, pos + 1);
  if (k_begin < (lo / 16) * 16) k_begin = (lo / 16) * 16;
  const int* bt = P.block_table + (size_t)seq * P.bt_stride;
  const int first_page = (k_begin < k_end) ? bt[k_begin / P.page_tokens] : 0;
  pdl_wait();

  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  uint4 qv[CH];                                           // head g of the group (zero beyond the group)
#pragma unroll
  for (int c = 0; c < CH; c++) {
    const int d = 32 * c + 8 * t;
    qv[c] = (g < gs && d < Hd) ? ldg16(P.q + (size_t)tok * P.ldq + (size_t)(kvh * gs + g) * Hd + d) : zero4;
  }
  float o[2 * CH][4];                                     // [chunk, register pair][dim row g | g+8 x heads 2t, 2t+1]
#pragma unroll
  for (int i = 0; i < 2 * CH; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // heads 2t, 2t+1 (over this lane's keys only)

  const size_t head_off = (size_t)kvh * P.page_tokens * Hd;
  const size_t page_stride = (size_t)P.n_kv * P.page_tokens * Hd;
  auto block_base = [&](int key0) -> size_t {
    const int page = (key0 == k_begin) ? first_page : bt[key0 / P.page_tokens];
    return (size_t)page * page_stride + head_off + (size_t)(key0 % P.page_tokens) * Hd;
  };
  uint4 ka[CH], kb[CH];
  size_t base = 0;
  if (k_begin < k_end) {
    base = block_base(k_begin);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      ka[c] = d < Hd ? ldg16(P.k_cache + base + (size_t)g * Hd + d) : zero4;
      kb[c] = d < Hd ? ldg16(P.k_cache + base + (size_t)(g + 8) * Hd + d) : zero4;
    }
  }
  for (int key0 = k_begin; key0 < k_end; key0 += 16) {
    const bf16* vp = P.v_cache + base;
    uint4 va[CH], vb[CH], nka[CH], nkb[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      va[c] = d < Hd ? ldg16(vp + (size_t)g * Hd + d) : zero4;
      vb[c] = d < Hd ? ldg16(vp + (size_t)(g + 8) * Hd + d) : zero4;
    }
    const bool more = key0 + 16 < k_end;
    if (more) base = block_base(key0 + 16);
#pragma unroll
    for (int c = 0; c < CH; c++) {
      const int d = 32 * c + 8 * t;
      nka[c] = (more && d < Hd) ? ldg16(P.k_cache + base + (size_t)g * Hd + d) : zero4;
      nkb[c] = (more && d < Hd) ? ldg16(P.k_cache + base + (size_t)(g + 8) * Hd + d) : zero4;
    }
    // S^T: [0],[1] = (key g, heads 2t, 2t+1); [2],[3] = (key g+8, same heads)
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < CH; c++) {
      mma16816(s, ka[c].x, kb[c].x, ka[c].y, kb[c].y, qv[c].x, qv[c].y);
      mma16816(s, ka[c].z, kb[c].z, ka[c].w, kb[c].w, qv[c].z, qv[c].w);
    }
    const bool ok0 = key0 + g <= pos && key0 + g >= lo && key0 + g < k_end;
    const bool ok1 = key0 + g + 8 <= pos && key0 + g + 8 >= lo && key0 + g + 8 < k_end;
    s[0] = ok0 ? s[0] * P.scale : -INFINITY; s[1] = ok0 ? s[1] * P.scale : -INFINITY;
    s[2] = ok1 ? s[2] * P.scale : -INFINITY; s[3] = ok1 ? s[3] * P.scale : -INFINITY;
    // maximum per head over the block's 16 keys: this lane's two keys, then across g (lanes 4, 8, 16 apart)
    float bm[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
    float corr[2], m_use[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
      bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 4));
      bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 8));
      bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 16));
      const float m_new = fmaxf(m_run[e], bm[e]);
      m_use[e] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[e] = __expf(m_run[e] - m_use[e]);
      m_run[e] = m_new;
    }
    const float p0 = __expf(s[0] - m_use[0]), p1 = __expf(s[1] - m_use[1]);
    const float p2 = __expf(s[2] - m_use[0]), p3 = __expf(s[3] - m_use[1]);
    l_run[0] = l_run[0] * corr[0] + p0 + p2;
    l_run[1] = l_run[1] * corr[1] + p1 + p3;
#pragma unroll
    for (int i = 0; i < 2 * CH; i++) {
      o[i][0] *= corr[0]; o[i][1] *= corr[1]; o[i][2] *= corr[0]; o[i][3] *= corr[1];
    }
    // P^T as the B operand: (keys 2t, 2t+1; head g) and (keys 2t+8, 2t+9; head g)
    const uint32_t pb0 = transpose8x8(pack_bf16(p0, p1)), pb1 = transpose8x8(pack_bf16(p2, p3));
#pragma unroll
    for (int c = 0; c < CH; c++) {
#pragma unroll
      for (int ii = 0; ii < 2; ii++) {
        const uint32_t a0 = transpose8x8(reg_of(va[c], 2 * ii)), a1 = transpose8x8(reg_of(va[c], 2 * ii + 1));
        const uint32_t a2 = transpose8x8(reg_of(vb[c], 2 * ii)), a3 = transpose8x8(reg_of(vb[c], 2 * ii + 1));
        mma16816(o[2 * c + ii], a0, a1, a2, a3, pb0, pb1);
      }
    }
#pragma unroll
    for (int c = 0; c < CH; c++) { ka[c] = nka[c]; kb[c] = nkb[c]; }
  }
  // denominators: this lane summed its own two keys of every block; add across g
#pragma unroll
  for (int e = 0; e < 2; e++) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 4);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 8);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 16);
  }
  // o[2c+ii]: [0],[1] = (dim D(2ii), heads 2t, 2t+1); [2],[3] = (dim D(2ii+1), same heads), D(i) = 32c + 8(g/2) + (g%2) + 2i
#pragma unroll
  for (int e = 0; e < 2; e++) {
    const int hq = 2 * t + e;
    if (hq >= gs) continue;
    const int head = kvh * gs + hq;
    const float inv = (P.n_splits == 1) ? 1.0f / l_run[e] : 1.0f;
    const size_t slot = ((size_t)tok * P.n_q + head) * P.n_splits + split;
#pragma unroll
    for (int c = 0; c < CH; c++) {
#pragma unroll
      for (int ii = 0; ii < 2; ii++) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
          const int d = 32 * c + 8 * (g >> 1) + (g & 1) + 2 * (2 * ii + r);
          if (d >= Hd) continue;
          const float v = o[2 * c + ii][2 * r + e] * inv;
          if (P.n_splits == 1) P.out[(size_t)tok * P.ldo + (size_t)head * Hd + d] = __float2bfloat16_rn(v);
          else P.part_o[slot * Hd + d] = v;
        }
      }
    }
    if (P.n_splits > 1 && g == 0) {
      P.part_ml[slot * 2] = m_run[e];
      P.part_ml[slot * 2 + 1] = l_run[e];
    }
  }
}

// Merge the splits of one (token, head): one block each.  The maxima and denominators of all splits are fetched
// at once (one thread per split), turned into weights exp(m_s - M) in shared memory, then every thread adds up
// its output dimension over the splits in split order.
#define MERGE_MAX_SPLITS 256
__global__ void __launch_bounds__(128)
attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                       bf16* __restrict__ out, int ldo, const int* __restrict__ token_seq, int n_tokens, int n_q,
                       int head_dim, int n_splits) {
  __shared__ float wgt[MERGE_MAX_SPLITS];
  __shared__ float red[2];
  pdl_trigger();
  const int item = blockIdx.x;
  const int tok = item / n_q, h = item % n_q;
  if (token_seq && token_seq[tok] < 0) return;
  pdl_wait();
  const float* ml = part_ml + (size_t)item * n_splits * 2;
  const float* po = part_o + (size_t)item * n_splits * head_dim;
  // warp 0: the maximum over splits, then the weights and the denominator
  if (threadIdx.x < 32) {
    float ms[MERGE_MAX_SPLITS / 32], ls[MERGE_MAX_SPLITS / 32];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < MERGE_MAX_SPLITS / 32; j++) {
      const int sidx = threadIdx.x + 32 * j;
      ms[j] = sidx < n_splits ? ld_fresh(ml + 2 * sidx) : -INFINITY;
      ls[j] = sidx < n_splits ? ld_fresh(ml + 2 * sidx + 1) : 0.f;
      m = fmaxf(m, ms[j]);
    }
    m = warp_max(m);
    float l = 0.f;
#pragma unroll
    for (int j = 0; j < MERGE_MAX_SPLITS / 32; j++) {
      const int sidx = threadIdx.x + 32 * j;
      const float w = (ms[j] == -INFINITY) ? 0.f : __expf(ms[j] - m);
      if (sidx < n_splits) wgt[sidx] = w;
      l += ls[j] * w;
    }
    l = warp_sum(l);
    if (threadIdx.x == 0) red[0] = l;
  }
  __syncthreads();
  const int d = threadIdx.x;
  if (d >= head_dim) return;
  float acc = 0.f;
  int sidx = 0;
  for (; sidx + 4 <= n_splits; sidx += 4) {             // four loads in flight at a time, added in split order
    const float a0 = ld_fresh(po + (size_t)(sidx + 0) * head_dim + d), a1 = ld_fresh(po + (size_t)(sidx + 1) * head_dim + d);
    const float a2 = ld_fresh(po + (size_t)(sidx + 2) * head_dim + d), a3 = ld_fresh(po + (size_t)(sidx + 3) * head_dim + d);
    acc = fmaf(a0, wgt[sidx], acc); acc = fmaf(a1, wgt[sidx + 1], acc);
    acc = fmaf(a2, wgt[sidx + 2], acc); acc = fmaf(a3, wgt[sidx + 3], acc);
  }
  for (; sidx < n_splits; sidx++) acc = fmaf(ld_fresh(po + (size_t)sidx * head_dim + d), wgt[sidx], acc);
  out[(size_t)tok * ldo + (size_t)h * head_dim + d] = __float2bfloat16_rn(acc / red[0]);
}

// Scratch needed for n_splits > 1: floats for part_o = tokens*Nq*n_splits*Hd, for part_ml = tokens*Nq*n_splits*2.
STRATUM_EXPORT int stratum_attention_mma(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                         const int* token_pos, const int* token_seq, const int* block_table,
                                         int bt_stride, const int* qb_seq, const int* qb_tok0, const int* qb_ntok,
                                         int n_qblocks, int tokens_per_block, void* out, int ldo, float* part_o,
                                         float* part_ml, int n_tokens, int n_q, int n_kv, int head_dim,
                                         int page_tokens, int window, float scale, int n_splits, int chunk,
                                         cudaStream_t stream) {
  if (n_tokens <= 0 || n_qblocks <= 0) return 0;
  if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 128) return STRATUM_ERR_SHAPE;
  if (n_kv < 1 || n_q % n_kv != 0 || page_tokens % 16 != 0) return STRATUM_ERR_SHAPE;
  if (n_splits < 1 || (n_splits > 1 && (chunk % page_tokens != 0 || !part_o || !part_ml))) return STRATUM_ERR_SHAPE;
  if (n_splits > MERGE_MAX_SPLITS) return STRATUM_ERR_LIMIT;
  if (ldq % 8 != 0 || ldo % 8 != 0) return STRATUM_ERR_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return STRATUM_ERR_ALIGN;
  const int gs = n_q / n_kv;
  AttnParams P;
  P.q = (const bf16*)q; P.ldq = ldq;
  P.k_cache = (const bf16*)k_cache; P.v_cache = (const bf16*)v_cache;
  P.token_pos = token_pos; P.token_seq = token_seq; P.block_table = block_table; P.bt_stride = bt_stride;
  P.qb_seq = qb_seq; P.qb_tok0 = qb_tok0; P.qb_ntok = qb_ntok; P.n_qblocks = n_qblocks;
  P.out = (bf16*)out; P.ldo = ldo; P.part_o = part_o; P.part_ml = part_ml;
  P.n_q = n_q; P.n_kv = n_kv; P.head_dim = head_dim; P.page_tokens = page_tokens; P.window = window;
  P.rows_per_token = gs < 16 ? gs : 16;
  P.head_groups = (gs + 15) / 16;
  P.tokens_per_block = tokens_per_block;
  if (tokens_per_block < 1 || tokens_per_block * P.rows_per_token > 16) return STRATUM_ERR_SHAPE;
  P.n_splits = n_splits; P.chunk = n_splits > 1 ? chunk : 0x40000000;
  P.scale = scale;
  const long long items = (long long)n_qblocks * n_kv * P.head_groups * n_splits;
  const long long blocks = (items + AM_WARPS - 1) / AM_WARPS;
  if (blocks > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  const int ch = (head_dim + 31) / 32;
  int st = 0;
  if (!qb_seq && tokens_per_block == 1 && gs <= 8) {
    // decode steps: the kernel with the keys along M
    const long long d_items = (long long)n_qblocks * n_kv * n_splits;
    const unsigned d_blocks = (unsigned)((d_items + AM_WARPS - 1) / AM_WARPS);
    switch (ch) {
      case 1: st = launch_pdl(attention_decode_kernel<1>, d_blocks, AM_WARPS * 32, 0, stream, P); break;
      case 2: st = launch_pdl(attention_decode_kernel<2>, d_blocks, AM_WARPS * 32, 0, stream, P); break;
      case 3: st = launch_pdl(attention_decode_kernel<3>, d_blocks, AM_WARPS * 32, 0, stream, P); break;
      case 4: st = launch_pdl(attention_decode_kernel<4>, d_blocks, AM_WARPS * 32, 0, stream, P); break;
      default: return STRATUM_ERR_SHAPE;
    }
  } else
  switch (ch) {
    case 1: st = launch_pdl(attention_mma_kernel<1>, (unsigned)blocks, AM_WARPS * 32, 0, stream, P); break;
    case 2: st = launch_pdl(attention_mma_kernel<2>, (unsigned)blocks, AM_WARPS * 32, 0, stream, P); break;
    case 3: st = launch_pdl(attention_mma_kernel<3>, (unsigned)blocks, AM_WARPS * 32, 0, stream, P); break;
    case 4: st = launch_pdl(attention_mma_kernel<4>, (unsigned)blocks, AM_WARPS * 32, 0, stream, P); break;
    default: return STRATUM_ERR_SHAPE;
  }
  if (st != 0 || n_splits == 1) return st;
  const long long m_items = (long long)n_tokens * n_q;
  if (m_items > 0x7fffffffLL) return STRATUM_ERR_LIMIT;
  return launch_pdl(attention_merge_kernel, (unsigned)m_items, 128, 0, stream, (const float*)part_o,
                    (const float*)part_ml, (bf16*)out, ldo, token_seq, n_tokens, n_q, head_dim, n_splits);
}
