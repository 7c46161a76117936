// y = x W^T (+ bias) for a handful of rows of x (decode steps): a weight-streaming kernel.
//
// With M <= 32 rows the product is bound by reading W once from HBM, so the kernel is built
// around that stream: every lane loads 16 contiguous bytes of a weight row straight from global
// memory into the registers that feed mma.sync.m16n8k16 (bf16 in, float32 accumulate); there is no
// shared-memory staging and nothing to wait on but the loads themselves.  Weights are the "A"
// operand (16 weight rows per MMA), the rows of x the "B" operand (8 rows of x per MMA), so the
// accumulator holds y^T.
//
// How a 16-byte load lands in a fragment.  For m16n8k16 lane (g = lane/4, t = lane%4) holds of A the
// elements (row g | g+8, col 2t,2t+1 | 2t+8,2t+9) and of B (k 2t,2t+1 | 2t+8,2t+9, col g).  A dot
// product does not care in which order k is visited as long as A and B agree, so within a chunk of
// 32 k-values lane t takes the 8 contiguous values k = 8t..8t+7 of its row, for A and for B alike,
// and feeds them to two MMAs (values 0..3, then 4..7).  The products pair up exactly as in the
// row-major definition  y[m][n] = sum_k x[m][k] W[n][k]  (stratum/native/stratum_linear.h:491-507).
//
// Work split: a block of 8 warps covers RT tiles of 16 weight rows; the K range is cut into 8/RT
// contiguous parts, one per warp, whose partial sums are added in part order in shared memory, so
// the result of a row does not depend on the batch it is in (the order of additions is fixed by K
// and the launch shape alone).
//
// Epilogues: 0 store bf16; 1 add into float32 (residual stream) in place; 2 store float32;
//            3 SwiGLU over row pairs (2j = gate, 2j+1 = up): out[m][j] = silu(g) * u, bf16,
//              silu(z) = z / (1 + exp(-z))  (stratum/native/stratum_engine.h:373-391).
#include "common.cuh"

#define SK_WARPS 8
#define SK_UNROLL 4

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
               "{%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: tiles of 8 rows of x (M <= 8*MT).  RT: tiles of 16 weight rows per block.
template <int MT, int RT, int EPI>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ bias,
                   void* __restrict__ out, int M, int N, int K, int ldx, int ldo, int groups_per_block) {
  constexpr int KS = SK_WARPS / RT;                 // K parts
  __shared__ float part[RT][KS][MT * 8][16 + 1];    // [row tile][k part][x row][weight row]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rt = warp / KS, ks = warp % KS;
  pdl_trigger();
  // a block works through `groups_per_block` consecutive groups of RT row tiles, so that the grid can be
  // sized to what the GPU holds at once and every block gets (almost) the same share of W
  const int n_groups = (N + 16 * RT - 1) / (16 * RT);
  const int group_begin = blockIdx.x * groups_per_block;
  const int group_end = min(n_groups, group_begin + groups_per_block);
  bool waited = false;
  for (int group = group_begin; group < group_end; group++) {
  const int n0 = (group * RT + rt) * 16;
  // K range of this warp, in chunks of 32
  const int n_chunks = (K + 31) / 32;
  const int per = (n_chunks + KS - 1) / KS;
  const int c_begin = ks * per, c_end = min(n_chunks, c_begin + per);

  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

  const int r0 = n0 + g, r1 = n0 + g + 8;
  const bool r0_ok = r0 < N, r1_ok = r1 < N;
  const bf16* w0 = w + (size_t)(r0_ok ? r0 : 0) * K;
  const bf16* w1 = w + (size_t)(r1_ok ? r1 : 0) * K;
  const uint4 zero = make_uint4(0, 0, 0, 0);

  // Weights do not depend on the kernels before this one: the first batch of weight loads is issued
  // before waiting for them (programmatic dependent launch); rows of x are read only after the wait.
  // From then on the next batch of weights and rows is requested before the products of the current one.
  uint4 a0[SK_UNROLL], a1[SK_UNROLL], b[SK_UNROLL][MT];
  auto load_weights = [&](int c, uint4 (&d0)[SK_UNROLL], uint4 (&d1)[SK_UNROLL]) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; u++) {
      const int k = (c + u) * 32 + t * 8;
      const bool k_ok = (c + u) < c_end && k < K;       // K is a multiple of 8: a 16-byte piece is all in or all out
      d0[u] = (k_ok && r0_ok) ? ld_stream16(w0 + k) : zero;
      d1[u] = (k_ok && r1_ok) ? ld_stream16(w1 + k) : zero;
    }
  };
  auto load_rows = [&](int c, uint4 (&d)[SK_UNROLL][MT]) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; u++) {
      const int k = (c + u) * 32 + t * 8;
      const bool k_ok = (c + u) < c_end && k < K;
#pragma unroll
      for (int i = 0; i < MT; i++) {
        const int m = i * 8 + g;
        d[u][i] = (k_ok && m < M) ? ld_fresh((const uint4*)(x + (size_t)m * ldx + k)) : zero;
      }
    }
  };
  load_weights(c_begin, a0, a1);
  if (!waited) { pdl_wait(); waited = true; }
  load_rows(c_begin, b);
  for (int c = c_begin; c < c_end; c += SK_UNROLL) {
    // request the next batch of weights and rows before multiplying the current one
    uint4 next0[SK_UNROLL], next1[SK_UNROLL], nextb[SK_UNROLL][MT];
    load_weights(c + SK_UNROLL, next0, next1);
    load_rows(c + SK_UNROLL, nextb);
#pragma unroll
    for (int u = 0; u < SK_UNROLL; u++) {
#pragma unroll
      for (int i = 0; i < MT; i++) {
        mma_bf16_16x8x16(acc[i], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b[u][i].x, b[u][i].y);
        mma_bf16_16x8x16(acc[i], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b[u][i].z, b[u][i].w);
      }
    }
#pragma unroll
    for (int u = 0; u < SK_UNROLL; u++) {
      a0[u] = next0[u]; a1[u] = next1[u];
#pragma unroll
      for (int i = 0; i < MT; i++) b[u][i] = nextb[u][i];
    }
  }
  // accumulator: c0,c1 -> (weight row g, x row 2t, 2t+1); c2,c3 -> (weight row g+8, same x rows)
#pragma unroll
  for (int i = 0; i < MT; i++) {
    part[rt][ks][i * 8 + 2 * t][g] = acc[i][0];
    part[rt][ks][i * 8 + 2 * t + 1][g] = acc[i][1];
    part[rt][ks][i * 8 + 2 * t][g + 8] = acc[i][2];
    part[rt][ks][i * 8 + 2 * t + 1][g + 8] = acc[i][3];
  }
  __syncthreads();
  // reduce the K parts in part order and write out: one thread per (x row, weight row) of the block
  if (EPI != 3) {
    for (int idx = threadIdx.x; idx < RT * MT * 8 * 16; idx += SK_WARPS * 32) {
      const int tile = idx / (MT * 8 * 16), rem = idx % (MT * 8 * 16);
      const int m = rem / 16, r = rem % 16;
      const int n = (group * RT + tile) * 16 + r;
      if (m >= M || n >= N) continue;
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < KS; s++) v += part[tile][s][m][r];
      if (bias) v += bias[n];
      const size_t o = (size_t)m * ldo + n;
      if (EPI == 0) ((bf16*)out)[o] = __float2bfloat16_rn(v);
      else if (EPI == 1) ((float*)out)[o] = ld_fresh((const float*)out + o) + v;
      else ((float*)out)[o] = v;
    }
  } else {
    for (int idx = threadIdx.x; idx < RT * MT * 8 * 8; idx += SK_WARPS * 32) {
      const int tile = idx / (MT * 8 * 8), rem = idx % (MT * 8 * 8);
      const int m = rem / 8, jr = rem % 8;
      const int n = (group * RT + tile) * 16 + 2 * jr;       // gate row; up row is n + 1
      if (m >= M || n + 1 >= N) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int s = 0; s < KS; s++) { gate += part[tile][s][m][2 * jr]; up += part[tile][s][m][2 * jr + 1]; }
      if (bias) { gate += bias[n]; up += bias[n + 1]; }
      // the unfused path rounds gate and up to bfloat16 before the activation; do the same
      gate = __bfloat162float(__float2bfloat16_rn(gate));
      up = __bfloat162float(__float2bfloat16_rn(up));
      ((bf16*)out)[(size_t)m * ldo + (n >> 1)] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
  }
  __syncthreads();          // the partial sums are reused by the next group
  }
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int MT, int RT, int EPI>
static int launch_skinny_epi(const bf16* x, const bf16* w, const float* bias, void* out, int M, int N, int K,
                             int ldx, int ldo, cudaStream_t stream) {
  auto kern = gemm_skinny_kernel<MT, RT, EPI>;
  static int resident = 0;                 // blocks of this kernel the whole GPU holds at once
  if (!resident) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, SK_WARPS * 32, 0) != cudaSuccess || per_sm < 1)
      per_sm = 1;
    resident = per_sm * sm_count();
  }
  const int n_groups = (N + 16 * RT - 1) / (16 * RT);
  const int per_block = (n_groups + resident - 1) / resident;
  const int blocks = (n_groups + per_block - 1) / per_block;
  return launch_pdl(kern, blocks, SK_WARPS * 32, 0, stream, x, w, bias, out, M, N, K, ldx, ldo, per_block);
}

template <int MT, int RT>
static int launch_skinny(const bf16* x, const bf16* w, const float* bias, void* out, int epilogue, int M, int N,
                         int K, int ldx, int ldo, cudaStream_t stream) {
  switch (epilogue) {
    case 0: return launch_skinny_epi<MT, RT, 0>(x, w, bias, out, M, N, K, ldx, ldo, stream);
    case 1: return launch_skinny_epi<MT, RT, 1>(x, w, bias, out, M, N, K, ldx, ldo, stream);
    case 2: return launch_skinny_epi<MT, RT, 2>(x, w, bias, out, M, N, K, ldx, ldo, stream);
    case 3: return launch_skinny_epi<MT, RT, 3>(x, w, bias, out, M, N, K, ldx, ldo, stream);
    default: return STRATUM_ERR_SHAPE;
  }
}

// x: bf16 [M][ldx], w: bf16 [N][K], bias float32 [N] or null, out [M][ldo] (for SwiGLU: [M][N/2]).
// Needs K % 8 == 0, ldx % 8 == 0 and 16-byte aligned x and w (checked); M <= 32.
STRATUM_EXPORT int stratum_gemm_skinny(const void* x, const void* w, const float* bias, void* out, int epilogue,
                                       int M, int N, int K, int ldx, int ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32) return STRATUM_ERR_LIMIT;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0) return STRATUM_ERR_SHAPE;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return STRATUM_ERR_ALIGN;
  if (epilogue == 3 && (N % 2 != 0)) return STRATUM_ERR_SHAPE;
  const bf16* xb = (const bf16*)x;
  const bf16* wb = (const bf16*)w;
  // few weight rows: one 16-row tile per block (more blocks, K cut 8 ways); many: two tiles, K cut 4 ways
  const bool small_n = N < 16 * 2 * 148 * 2;
  if (M <= 8) return small_n ? launch_skinny<1, 1>(xb, wb, bias, out, epilogue, M, N, K, ldx, ldo, stream)
                             : launch_skinny<1, 2>(xb, wb, bias, out, epilogue, M, N, K, ldx, ldo, stream);
  if (M <= 16) return small_n ? launch_skinny<2, 1>(xb, wb, bias, out, epilogue, M, N, K, ldx, ldo, stream)
                              : launch_skinny<2, 2>(xb, wb, bias, out, epilogue, M, N, K, ldx, ldo, stream);
  return small_n ? launch_skinny<4, 1>(xb, wb, bias, out, epilogue, M, N, K, ldx, ldo, stream)
                 : launch_skinny<4, 2>(xb, wb, bias, out, epilogue, M, N, K, ldx, ldo, stream);
}
