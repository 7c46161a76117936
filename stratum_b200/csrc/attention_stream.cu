// Decode-step attention over the paged bfloat16 cache with the pages of all sequences spread evenly over the SMs.
//
// One new token per sequence: for query head h at position p, score_t = (q_h . K_t[kv(h)]) * scale over keys t in
// [lo, p]; p_t = softmax; o_h = sum_t p_t V_t[kv(h)]  (stratum/native/stratum_arch_llama.inc.c:435-514).  The
// time is the time to read every live key and value once, so the work is cut like a stream-K matrix product:
// the pages (64 keys of one kv head) of all sequences form one sequence of units, ordered by (sequence, kv head,
// page), and CTA c takes the contiguous stretch [c T / G, (c+1) T / G).  A stretch is the end of one (sequence,
// kv head), some whole ones and the beginning of another.
//
//   warp 0      one lane feeds a ring of shared-memory stages by TMA: the K page and the V page of a unit (each
//               64 keys x head_dim, boxes of 64 dims with the 128-byte swizzle), up to 160 KB in flight per SM;
//   warps 1-4   each takes 16 of a page's 64 keys.  The keys lie along M of mma.sync.m16n8k16 and the (up to 8)
//               query heads of the group along N, as in attention_decode_kernel: S^T = K Q^T, online softmax
//               in float32 per head, O^T += V^T P^T with V transposed in registers by movmatrix.  Fragments are
//               16-byte reads of shared memory at the swizzled address of (key, 8 dims).
//               (Heads of 64 with many pages: eight warps, each taking every eighth page whole; see the entry
//               point's note.)
//
// When a (sequence, kv head) ends, the four warps' maxima, sums and outputs are merged through shared memory.
// If the CTA saw all of its keys the normalised output is written; otherwise the unnormalised output, maximum
// and sum go to one of the CTA's two scratch slots (0: the unit its stretch begins in belongs to this (sequence,
// kv head); 1: otherwise) and attention_stream_merge_kernel adds the pieces in CTA order.  No CTA waits for
// another; which keys meet in which CTA depends on the step's batch, the sums differ by rounding only.
//
// Every mbarrier wait is bounded (see gemm_tc.cu): on expiry a code goes to the status word and the CTA winds down.
#include <math.h>
#include <stdlib.h>

#include "mma_common.cuh"
#include "tc_common.cuh"

#define SA_KEYS 64
#define SA_MAX_SEQS 1024
#define SA_MAX_GS 8

struct SaParams {
  const bf16* q; int ldq;                       // [seqs][ldq]: query heads first
  const int* token_pos;                         // [seqs]: position of the new token
  const int* token_seq;                         // [seqs]: row of the block table, -1 = padding
  const int* block_table; int bt_stride;
  bf16* out; int ldo;
  float* scratch;                               // [G][2][gs * (Hd + 2)]
  int* status;
  int n_seqs, n_q, n_kv, gs, window;
  float scale;
  int late_trigger;
};

template <int CH, int NW>
struct SaSmem {
  static constexpr int HD = 32 * CH;
  static constexpr int STAGE = SA_KEYS * HD;    // elements of one K (or V) page
  static constexpr int STAGES = (160 * 1024) / (2 * STAGE * 2);
  alignas(1024) bf16 k[STAGES][STAGE];          // [Hd/64 boxes][64 keys][64 dims]
  alignas(1024) bf16 v[STAGES][STAGE];
  float mo[NW][SA_MAX_GS][HD];                  // the consumer warps' outputs, maxima and sums at the end of a run
  float mm[NW][SA_MAX_GS], ml[NW][SA_MAX_GS];
  int pre[SA_MAX_SEQS + 1];                     // pages before sequence b (per kv head)
  uint64_t full[STAGES], empty[STAGES];
  uint32_t seen[STAGES];                        // whole pages per warp: fillings of the stage that a warp has seen complete
  int abort_flag;
};

__device__ __forceinline__ uint32_t ld_acquire_shared(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_shared(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

struct SaSeq {                                  // the keys sequence b attends to, in pages
  int pos, lo, first, n;
};
__device__ __forceinline__ SaSeq sa_seq(const SaParams& P, int b) {
  SaSeq s;
  s.pos = P.token_pos[b];
  s.lo = (P.window > 0 && s.pos - P.window + 1 > 0) ? s.pos - P.window + 1 : 0;
  s.first = s.lo / SA_KEYS;
  s.n = (P.token_seq[b] < 0) ? 0 : s.pos / SA_KEYS - s.first + 1;
  return s;
}
__device__ __forceinline__ long long sa_begin(int c, int G, long long T) { return (long long)c * T / G; }
__device__ __forceinline__ int sa_owner(long long u, int G, long long T) {
  int o = (int)(u * G / T);
  while (o + 1 < G && sa_begin(o + 1, G, T) <= u) o++;
  while (o > 0 && sa_begin(o, G, T) > u) o--;
  return o;
}

// Walks over the units of a stretch in order: (b, kvh, page).
struct SaCursor {
  int b, kvh, page;
  SaSeq s;
  __device__ __forceinline__ void seek(const SaParams& P, const int* pre, long long u) {
    int lo = 0, hi = P.n_seqs - 1;              // last b with pre[b] * n_kv <= u
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((long long)pre[mid] * P.n_kv <= u) lo = mid; else hi = mid - 1;
    }
    b = lo;
    s = sa_seq(P, b);
    const int r = (int)(u - (long long)pre[b] * P.n_kv);
    kvh = r / s.n;
    page = s.first + r % s.n;
  }
  __device__ __forceinline__ void next(const SaParams& P) {
    if (++page < s.first + s.n) return;
    if (++kvh < P.n_kv) { page = s.first; return; }
    kvh = 0;
    do { b++; if (b < P.n_seqs) s = sa_seq(P, b); } while (b < P.n_seqs && s.n == 0);
    page = s.first;
  }
};

template <int CH, bool WP, int NW>
__global__ void __launch_bounds__(32 + 32 * NW, 1)
attention_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const SaParams P) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using Smem = SaSmem<CH, NW>;
  constexpr int HD = Smem::HD, STAGES = Smem::STAGES, DB = HD / 64;
  static_assert(WP || NW == 4, "a quarter of a page per warp needs four consumer warps");
  static_assert(!WP || NW <= STAGES, "whole pages per warp: more consumer warps than ring stages would only wait");
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x, c = blockIdx.x;
  // (no early trigger: kernels that start while this one streams the cache slow it down more than their own
  // head start is worth; measured)
  volatile int* abort_flag = &S.abort_flag;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], WP ? 1 : NW); S.seen[s] = 0; }
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // pages per sequence (positions and the batch are the step's description, not the work of an earlier kernel)
  for (int b = threadIdx.x; b < P.n_seqs; b += 32 + 32 * NW) S.pre[b + 1] = sa_seq(P, b).n;
  if (threadIdx.x == 0) S.pre[0] = 0;
  __syncthreads();
  if (warp == 0) {                               // running sum, 32 sequences at a time
    int carry = 0;
    for (int base = 0; base < P.n_seqs; base += 32) {
      const int i = base + lane;
      int v = i < P.n_seqs ? S.pre[i + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
      }
      if (i < P.n_seqs) S.pre[i + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  const long long T = (long long)S.pre[P.n_seqs] * P.n_kv;
  const long long u0 = T ? sa_begin(c, G, T) : 0, u1 = T ? sa_begin(c + 1, G, T) : 0;
  if (u0 >= u1) {
    pdl_wait();            // no CTA leaves before the kernel before this one is done: what follows relies on it
    return;
  }

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      SaCursor cur;
      cur.seek(P, S.pre, u0);
      // Only a sequence's last page holds what the kernel before this one wrote (the newest key and value): the
      // pages before it are requested at once, up to a ring's worth, and the wait comes with the first last page.
      bool waited = false;
      uint32_t it = 0;
      bool ok = true;
      for (long long u = u0; u < u1 && ok; u++, it++) {
        const int s = it % STAGES;
        if (!waited && (it >= (uint32_t)STAGES || cur.page == cur.s.first + cur.s.n - 1)) { pdl_wait(); waited = true; }
        if (!mbar_wait(&S.empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) {
          atomicCAS(P.status, 0, 301); S.abort_flag = 1; ok = false; break;
        }
        const int pg = P.block_table[(size_t)P.token_seq[cur.b] * P.bt_stride + cur.page];
        const int row = (pg * P.n_kv + cur.kvh) * SA_KEYS;
        mbar_expect_tx(&S.full[s], 2 * SA_KEYS * HD * sizeof(bf16));
        for (int db = 0; db < DB; db++) {
          tma_load_2d(&map_k, S.k[s] + db * SA_KEYS * 64, &S.full[s], db * 64, row);
          tma_load_2d(&map_v, S.v[s] + db * SA_KEYS * 64, &S.full[s], db * 64, row);
        }
        cur.next(P);
      }
      if (!waited) pdl_wait();
      if (P.late_trigger) pdl_trigger();   // this CTA has asked for its last page
      if (!ok) {
        for (int i = 0; i < 2000; i++) __nanosleep(1000);   // let copies already issued land
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers (warps 1..4)
  const int w = warp - 1;
  const int g = lane >> 2, t = lane & 3;
  const int gs = P.gs;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  SaCursor cur;
  cur.seek(P, S.pre, u0);
  pdl_wait();                                    // q comes from the kernel before
  uint32_t it = 0;
  bool ok = true;
  long long u = u0;
  while (u < u1 && ok) {
    // one run: the units of this stretch that belong to (cur.b, cur.kvh)
    const int b = cur.b, kvh = cur.kvh;
    const SaSeq sq = cur.s;
    const bool from_start = cur.page == sq.first;
    const bool holds_u0 = (u == u0);
    uint4 qv[CH];                                // head g of the group (zero beyond the group)
#pragma unroll
    for (int ch = 0; ch < CH; ch++)
      qv[ch] = g < gs ? ld_fresh((const uint4*)(P.q + (size_t)b * P.ldq + (size_t)(kvh * gs + g) * HD + 32 * ch + 8 * t))
                      : zero4;
    float o[2 * CH][4];                          // [chunk, register pair][dim row g | g+8 x heads 2t, 2t+1]
#pragma unroll
    for (int i = 0; i < 2 * CH; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    bool to_end = false;
    while (u < u1 && cur.b == b && cur.kvh == kvh) {
      const int s = it % STAGES;
      if constexpr (WP) {
        // the pages go round the warps, and a warp takes a page whole: the scores of its 64 keys first, one maximum
        // and one rescaling of the sums per page, then the products with V; NW warps work on NW pages at a time
        to_end = cur.page == sq.first + sq.n - 1;
        if ((int)(it % NW) == w) {
          // A wait can tell a barrier's current phase from the one before only, and the filling of this stage
          // before this one was another warp's page: until that warp has seen its filling complete, a wait for
          // this one would take the filling before that for its own.  So that warp says so (S.seen), and this
          // one waits for its word first.  (The word comes before that warp frees the stage, so before this
          // filling can even be asked for: nothing here waits for anything that is not older than itself.)
          const uint32_t fill = it / STAGES;
          bool seen = false;
          for (uint32_t i = 0; i < TC_SPIN_LIMIT && !seen; i++) {
            seen = ld_acquire_shared(&S.seen[s]) >= fill;
            if ((i & 1023u) == 1023u && *abort_flag) break;
          }
          if (!__all_sync(0xffffffffu, seen && mbar_wait(&S.full[s], fill & 1, abort_flag))) {
            if (lane == 0) { atomicCAS(P.status, 0, 302); S.abort_flag = 1; }
            ok = false;
            break;
          }
          __syncwarp();
          if (lane == 0) st_release_shared(&S.seen[s], fill + 1);
          const uint8_t* kb_ = reinterpret_cast<const uint8_t*>(S.k[s]);
          const uint8_t* vb_ = reinterpret_cast<const uint8_t*>(S.v[s]);
          const int pk0 = cur.page * SA_KEYS;
          float sc[4][4];
#pragma unroll
          for (int blk = 0; blk < 4; blk++) {
            const int key0 = pk0 + 16 * blk;
            sc[blk][0] = sc[blk][1] = sc[blk][2] = sc[blk][3] = 0.f;
            if (key0 <= sq.pos && key0 + 15 >= sq.lo) {   // (a page's last blocks may lie beyond the newest key)
              const int r0 = 16 * blk + g;            // rows r0 and r0 + 8; both have (row & 7) == g
#pragma unroll
              for (int ch = 0; ch < CH; ch++) {
                const int off = (ch >> 1) * (SA_KEYS * 128) + (((((ch & 1) << 2) | t) ^ g) << 4);
                const uint4 ka = *reinterpret_cast<const uint4*>(kb_ + off + r0 * 128);
                const uint4 kb = *reinterpret_cast<const uint4*>(kb_ + off + (r0 + 8) * 128);
                mma16816(sc[blk], ka.x, kb.x, ka.y, kb.y, qv[ch].x, qv[ch].y);
                mma16816(sc[blk], ka.z, kb.z, ka.w, kb.w, qv[ch].z, qv[ch].w);
              }
            }
            const bool ok0 = key0 + g <= sq.pos && key0 + g >= sq.lo;
            const bool ok1 = key0 + g + 8 <= sq.pos && key0 + g + 8 >= sq.lo;
            sc[blk][0] = ok0 ? sc[blk][0] * P.scale : -INFINITY; sc[blk][1] = ok0 ? sc[blk][1] * P.scale : -INFINITY;
            sc[blk][2] = ok1 ? sc[blk][2] * P.scale : -INFINITY; sc[blk][3] = ok1 ? sc[blk][3] * P.scale : -INFINITY;
          }
          float bm[2], corr[2], m_use[2];
#pragma unroll
          for (int e = 0; e < 2; e++) {
            bm[e] = fmaxf(fmaxf(fmaxf(sc[0][e], sc[0][2 + e]), fmaxf(sc[1][e], sc[1][2 + e])),
                          fmaxf(fmaxf(sc[2][e], sc[2][2 + e]), fmaxf(sc[3][e], sc[3][2 + e])));
            bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 4));
            bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 8));
            bm[e] = fmaxf(bm[e], __shfl_xor_sync(0xffffffffu, bm[e], 16));
            const float m_new = fmaxf(m_run[e], bm[e]);
            m_use[e] = (m_new == -INFINITY) ? 0.f : m_new;
            corr[e] = __expf(m_run[e] - m_use[e]);
            m_run[e] = m_new;
            l_run[e] *= corr[e];
          }
#pragma unroll
          for (int i = 0; i < 2 * CH; i++) {
            o[i][0] *= corr[0]; o[i][1] *= corr[1]; o[i][2] *= corr[0]; o[i][3] *= corr[1];
          }
#pragma unroll
          for (int blk = 0; blk < 4; blk++) {
            const int key0 = pk0 + 16 * blk;
            if (key0 <= sq.pos && key0 + 15 >= sq.lo) {
              const float p0 = __expf(sc[blk][0] - m_use[0]), p1 = __expf(sc[blk][1] - m_use[1]);
              const float p2 = __expf(sc[blk][2] - m_use[0]), p3 = __expf(sc[blk][3] - m_use[1]);
              l_run[0] += p0 + p2;
              l_run[1] += p1 + p3;
              // P^T as the B operand: (keys 2t, 2t+1; head g) and (keys 2t+8, 2t+9; head g)
              const uint32_t pb0 = transpose8x8(pack_bf16(p0, p1)), pb1 = transpose8x8(pack_bf16(p2, p3));
              const int r0 = 16 * blk + g;
#pragma unroll
              for (int ch = 0; ch < CH; ch++) {
                const int off = (ch >> 1) * (SA_KEYS * 128) + (((((ch & 1) << 2) | t) ^ g) << 4);
                const uint4 va = *reinterpret_cast<const uint4*>(vb_ + off + r0 * 128);
                const uint4 vb = *reinterpret_cast<const uint4*>(vb_ + off + (r0 + 8) * 128);
#pragma unroll
                for (int ii = 0; ii < 2; ii++) {
                  const uint32_t a0 = transpose8x8(reg_of(va, 2 * ii)), a1 = transpose8x8(reg_of(va, 2 * ii + 1));
                  const uint32_t a2 = transpose8x8(reg_of(vb, 2 * ii)), a3 = transpose8x8(reg_of(vb, 2 * ii + 1));
                  mma16816(o[2 * ch + ii], a0, a1, a2, a3, pb0, pb1);
                }
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&S.empty[s]);   // the stage has been read
        }
      } else {
        // (the lanes of a warp go on or give up together)
        if (!__all_sync(0xffffffffu, mbar_wait(&S.full[s], (it / STAGES) & 1, abort_flag))) {
          if (lane == 0) { atomicCAS(P.status, 0, 302); S.abort_flag = 1; }
          ok = false;
          break;
        }
        const int key0 = cur.page * SA_KEYS + 16 * w;
        to_end = cur.page == sq.first + sq.n - 1;
        if (key0 <= sq.pos && key0 + 15 >= sq.lo) {  // (a page's last 16-key blocks may lie beyond the newest key)
          // 16-byte fragments at the swizzled address of (row, 8 dims): box = dims / 64, chunk ^ (row & 7)
          const uint8_t* kb_ = reinterpret_cast<const uint8_t*>(S.k[s]);
          const uint8_t* vb_ = reinterpret_cast<const uint8_t*>(S.v[s]);
          const int r0 = 16 * w + g;               // rows r0 and r0 + 8; both have (row & 7) == g
          uint4 ka[CH], kb[CH], va[CH], vb[CH];
  #pragma unroll
          for (int ch = 0; ch < CH; ch++) {
            const int off = (ch >> 1) * (SA_KEYS * 128) + (((((ch & 1) << 2) | t) ^ g) << 4);
            ka[ch] = *reinterpret_cast<const uint4*>(kb_ + off + r0 * 128);
            kb[ch] = *reinterpret_cast<const uint4*>(kb_ + off + (r0 + 8) * 128);
            va[ch] = *reinterpret_cast<const uint4*>(vb_ + off + r0 * 128);
            vb[ch] = *reinterpret_cast<const uint4*>(vb_ + off + (r0 + 8) * 128);
          }
          // S^T: [0],[1] = (key g, heads 2t, 2t+1); [2],[3] = (key g+8, same heads)
          float sc[4] = {0.f, 0.f, 0.f, 0.f};
  #pragma unroll
          for (int ch = 0; ch < CH; ch++) {
            mma16816(sc, ka[ch].x, kb[ch].x, ka[ch].y, kb[ch].y, qv[ch].x, qv[ch].y);
            mma16816(sc, ka[ch].z, kb[ch].z, ka[ch].w, kb[ch].w, qv[ch].z, qv[ch].w);
          }
          const bool ok0 = key0 + g <= sq.pos && key0 + g >= sq.lo;
          const bool ok1 = key0 + g + 8 <= sq.pos && key0 + g + 8 >= sq.lo;
          sc[0] = ok0 ? sc[0] * P.scale : -INFINITY; sc[1] = ok0 ? sc[1] * P.scale : -INFINITY;
          sc[2] = ok1 ? sc[2] * P.scale : -INFINITY; sc[3] = ok1 ? sc[3] * P.scale : -INFINITY;
          // maximum per head over the block's 16 keys: this lane's two keys, then across g (lanes 4, 8, 16 apart)
          float bm[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
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
          const float p0 = __expf(sc[0] - m_use[0]), p1 = __expf(sc[1] - m_use[1]);
          const float p2 = __expf(sc[2] - m_use[0]), p3 = __expf(sc[3] - m_use[1]);
          l_run[0] = l_run[0] * corr[0] + p0 + p2;
          l_run[1] = l_run[1] * corr[1] + p1 + p3;
  #pragma unroll
          for (int i = 0; i < 2 * CH; i++) {
            o[i][0] *= corr[0]; o[i][1] *= corr[1]; o[i][2] *= corr[0]; o[i][3] *= corr[1];
          }
          // P^T as the B operand: (keys 2t, 2t+1; head g) and (keys 2t+8, 2t+9; head g)
          const uint32_t pb0 = transpose8x8(pack_bf16(p0, p1)), pb1 = transpose8x8(pack_bf16(p2, p3));
  #pragma unroll
          for (int ch = 0; ch < CH; ch++) {
  #pragma unroll
            for (int ii = 0; ii < 2; ii++) {
              const uint32_t a0 = transpose8x8(reg_of(va[ch], 2 * ii)), a1 = transpose8x8(reg_of(va[ch], 2 * ii + 1));
              const uint32_t a2 = transpose8x8(reg_of(vb[ch], 2 * ii)), a3 = transpose8x8(reg_of(vb[ch], 2 * ii + 1));
              mma16816(o[2 * ch + ii], a0, a1, a2, a3, pb0, pb1);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.empty[s]);   // this warp has read the stage
      }
      cur.next(P);
      u++; it++;
    }
    // ---- the run is over: this warp's sums across g, then the four warps through shared memory
    // (after a failed wait every warp still comes to the barrier below, and all leave together behind it)
#pragma unroll
    for (int e = 0; e < 2; e++) {
      l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 4);
      l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 8);
      l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 16);
    }
    // o[2c+ii]: [0],[1] = (dim D(2ii), heads 2t, 2t+1); [2],[3] = (dim D(2ii+1), same heads),
    // D(i) = 32c + 8(g/2) + (g%2) + 2i
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int hq = 2 * t + e;
      if (g == 0) { S.mm[w][hq] = m_run[e]; S.ml[w][hq] = l_run[e]; }
#pragma unroll
      for (int ch = 0; ch < CH; ch++)
#pragma unroll
        for (int ii = 0; ii < 2; ii++)
#pragma unroll
          for (int r = 0; r < 2; r++)
            S.mo[w][hq][32 * ch + 8 * (g >> 1) + (g & 1) + 2 * (2 * ii + r)] = o[2 * ch + ii][2 * r + e];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * NW) : "memory");
    if (S.abort_flag) break;
    {
      const bool whole = from_start && to_end;
      float* slot = P.scratch + ((size_t)c * 2 + (holds_u0 ? 0 : 1)) * (size_t)(gs * (HD + 2));
      const int tid = threadIdx.x - 32;          // 0 .. 32 NW - 1
      for (int idx = tid; idx < gs * HD; idx += 32 * NW) {
        const int h = idx / HD, d = idx % HD;
        float M = S.mm[0][h];
#pragma unroll
        for (int i = 1; i < NW; i++) M = fmaxf(M, S.mm[i][h]);
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int i = 0; i < NW; i++) {
          const float e = __expf(S.mm[i][h] - Mu);
          acc += e * S.mo[i][h][d];
          L += e * S.ml[i][h];
        }
        if (whole) {
          P.out[(size_t)b * P.ldo + (size_t)(kvh * gs + h) * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
          slot[h * HD + d] = acc;
          if (d == 0) { slot[gs * HD + 2 * h] = M; slot[gs * HD + 2 * h + 1] = L; }
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(32 * NW) : "memory");   // the merge area is free for the next run
  }
}

// Adds the pieces of every (sequence, kv head) that more than one CTA worked on, in CTA order.
// One block per (sequence, query head), one thread per output dimension; the pieces' maxima and sums are fetched
// by as many threads as there are pieces, the outputs eight pieces at a time.
#define SA_MAX_PIECES 160
template <int CH>
__global__ void __launch_bounds__(32 * CH)
attention_stream_merge_kernel(const SaParams P, int G) {
  constexpr int HD = 32 * CH;
  __shared__ int red[2][4];
  __shared__ int off_s[SA_MAX_PIECES];           // float offset of the piece's slot, -1 = that CTA had no work
  __shared__ float m_s[SA_MAX_PIECES], l_s[SA_MAX_PIECES];
  pdl_trigger();
  const int gs = P.gs;
  const int b = blockIdx.x / P.n_q, hq = blockIdx.x % P.n_q;
  const int kvh = hq / gs, h = hq % gs;
  const SaSeq sq = sa_seq(P, b);
  // pages before b and in all: every thread sums a share, then across the block
  int before = 0, total = 0;
  for (int i = threadIdx.x; i < P.n_seqs; i += blockDim.x) {
    const int n = sa_seq(P, i).n;
    total += n;
    if (i < b) before += n;
  }
  for (int d = 16; d > 0; d >>= 1) {
    before += __shfl_xor_sync(0xffffffffu, before, d);
    total += __shfl_xor_sync(0xffffffffu, total, d);
  }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = before; red[1][threadIdx.x >> 5] = total; }
  __syncthreads();
  before = 0; total = 0;
  for (int i = 0; i < (int)(blockDim.x >> 5); i++) { before += red[0][i]; total += red[1][i]; }
  const long long T = (long long)total * P.n_kv;
  const long long ub = (long long)before * P.n_kv + (long long)kvh * sq.n, ue = ub + sq.n;
  pdl_wait();              // every block: the kernel after this one must not start on unfinished output
  if (sq.n == 0) return;
  const int first_c = sa_owner(ub, G, T), last_c = sa_owner(ue - 1, G, T);
  if (first_c == last_c) return;                 // one CTA saw all keys and wrote the output itself
  const int n_c = min(last_c - first_c + 1, SA_MAX_PIECES);      // (the launcher keeps G <= SA_MAX_PIECES)
  const size_t slot_floats = (size_t)(gs * (HD + 2));
  for (int i = threadIdx.x; i < n_c; i += blockDim.x) {
    const int cc = first_c + i;
    const long long s0 = sa_begin(cc, G, T);
    int off = -1;
    float m = -INFINITY, l = 0.f;
    if (sa_begin(cc + 1, G, T) != s0) {          // with fewer pages than CTAs some stretches are empty
      off = (int)(((size_t)cc * 2 + ((s0 >= ub && s0 < ue) ? 0 : 1)) * slot_floats);
      m = __ldcg(P.scratch + off + gs * HD + 2 * h);
      l = __ldcg(P.scratch + off + gs * HD + 2 * h + 1);
    }
    off_s[i] = off; m_s[i] = m; l_s[i] = l;
  }
  __syncthreads();
  float M = -INFINITY;
  for (int i = 0; i < n_c; i++) M = fmaxf(M, m_s[i]);
  const int d = threadIdx.x;
  float acc = 0.f, L = 0.f;
  for (int i0 = 0; i0 < n_c; i0 += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = i0 + j;
      v[j] = (i < n_c && off_s[i] >= 0) ? __ldcg(P.scratch + off_s[i] + h * HD + d) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const int i = i0 + j;
      if (i < n_c && off_s[i] >= 0) {
        const float e = __expf(m_s[i] - M);
        acc += e * v[j];
        L += e * l_s[i];
      }
    }
  }
  P.out[(size_t)b * P.ldo + (size_t)hq * HD + d] = __float2bfloat16_rn(acc / L);
}

// ---------------------------------------------------------------- host side
static int make_cache_map(CUtensorMap* map, const void* base, long long rows, int head_dim) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return STRATUM_ERR_LIMIT;
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * sizeof(bf16)};
  cuuint32_t box[2] = {64, SA_KEYS};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : STRATUM_ERR_SHAPE;
}

template <int CH, bool WP, int NW>
static int launch_stream(const CUtensorMap& mk, const CUtensorMap& mv, const SaParams& P, int grid,
                         cudaStream_t stream) {
  const size_t smem = sizeof(SaSmem<CH, NW>) + 1024;
  auto kern = attention_stream_kernel<CH, WP, NW>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int st = launch_pdl(kern, grid, 32 + 32 * NW, smem, stream, mk, mv, P);
  if (st != 0) return st;
  return launch_pdl(attention_stream_merge_kernel<CH>, P.n_seqs * P.n_q, 32 * CH, 0, stream, P, grid);
}

// Floats of scratch the kernel needs for a group size (two slots per SM).
STRATUM_EXPORT long long stratum_attention_stream_scratch_floats(int gs, int head_dim) {
  return (long long)sm_count() * 2 * gs * (head_dim + 2);
}

// q: bf16 [seqs][ldq], query heads first.  k_cache / v_cache: bf16 [n_pages][n_kv][64][head_dim].
// One new token per sequence (row i of q, token_pos[i], block-table row token_seq[i], -1 = padding).
// head_dim 64 or 128; at most 8 query heads per kv head; pages of 64 tokens; at most 1024 sequences.
// whole_pages (head_dim 64 only): eight warps that take whole pages in turn instead of four warps that take a
// quarter of every page.  With a quarter of a 16 KB page per warp little arrives per pass through a warp's chain of
// dependent instructions, and the four warps together read 3.4 to 4.5 TB/s; eight warps with whole pages (one
// maximum and one rescaling per 64 keys, two warps per scheduler to hide each other's latencies) read 5.8 TB/s at
// 64 sequences of 4,096 tokens, but are behind where an SM gets only a few pages (11.2 against 9.9 us for one
// sequence of 4,096 tokens).  At head_dim 128 (5 stages of 32 KB) the quarter form reads 6.5 TB/s.
STRATUM_EXPORT int stratum_attention_stream(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                            long long n_pages, const int* token_pos, const int* token_seq,
                                            const int* block_table, int bt_stride, void* out, int ldo, int n_seqs,
                                            int n_q, int n_kv, int head_dim, int page_tokens, int window, float scale,
                                            int late_trigger, int whole_pages, float* scratch, int* status,
                                            cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (head_dim != 64 && head_dim != 128) return STRATUM_ERR_SHAPE;
  if (n_kv < 1 || n_q % n_kv != 0 || n_q / n_kv > SA_MAX_GS || page_tokens != SA_KEYS) return STRATUM_ERR_SHAPE;
  if (n_seqs > SA_MAX_SEQS) return STRATUM_ERR_LIMIT;
  if (ldq % 8 != 0 || ldo % 8 != 0 || !scratch || !status) return STRATUM_ERR_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return STRATUM_ERR_ALIGN;
  CUtensorMap mk, mv;
  int st;
  if ((st = make_cache_map(&mk, k_cache, n_pages * n_kv * SA_KEYS, head_dim)) != 0) return st;
  if ((st = make_cache_map(&mv, v_cache, n_pages * n_kv * SA_KEYS, head_dim)) != 0) return st;
  SaParams P;
  P.q = (const bf16*)q; P.ldq = ldq; P.token_pos = token_pos; P.token_seq = token_seq;
  P.block_table = block_table; P.bt_stride = bt_stride; P.out = (bf16*)out; P.ldo = ldo;
  P.scratch = scratch; P.status = status;
  P.n_seqs = n_seqs; P.n_q = n_q; P.n_kv = n_kv; P.gs = n_q / n_kv; P.window = window; P.scale = scale;
  P.late_trigger = late_trigger;
  // one CTA per SM; with fewer pages than SMs the surplus CTAs find an empty stretch and leave
  const int grid = sm_count() < SA_MAX_PIECES ? sm_count() : SA_MAX_PIECES;
  if (whole_pages) {
    if (head_dim != 64) return STRATUM_ERR_SHAPE;
    return launch_stream<2, true, 8>(mk, mv, P, grid, stream);
  }
  if (head_dim == 64) return launch_stream<2, false, 4>(mk, mv, P, grid, stream);
  return launch_stream<4, false, 4>(mk, mv, P, grid, stream);
}
