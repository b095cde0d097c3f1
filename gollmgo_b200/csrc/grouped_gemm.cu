// Many small products with one launch: out_g = A_g @ W_g^T for groups g = 0 .. G-1, where a
// group is an expert of a mixture (its rows are the tokens routed to it, found through an
// offsets table and a row list made on the device) or a head of an attention layer (every group
// has all rows, and reads and writes its own columns of A and out).
//
//   rows of group g:  [offsets[g], offsets[g+1])   (offsets given)   or   [0, M)   (no offsets)
//   A row of row r:   row_index ? row_index[r] / row_div : r;   group g reads columns
//                     [g * a_group_cols, g * a_group_cols + K) of it
//   W_g:              [N, K] row-major ([2N, K] if gated: gate rows, then up rows) at W + g * rows * K
//   out row r, columns [g * o_group_cols, g * o_group_cols + Np): the N results, then zeros
//   epilogue:         gated: silu(x Wg^T) * (x Wu^T);   gate given: the row is multiplied by
//                     sigmoid(gate[A row, gate_col0 + g])   (an output gate per head)
//
// No host code learns how many rows a group has: the grid is sized for the worst case and a CTA
// whose tile lies past its group's rows returns.  A row's result depends on that row and on W_g
// alone (fixed order over K), so it is the same wherever the row lands in its group's list.
// bfloat16: tensor cores through wmma 16x16x16 with float32 accumulators; float32: FMA.  Tiles
// of 32 rows x 64 columns, K in steps through shared memory, any N and K.  This is the kernel for
// few rows per group (decoded tokens, heads of short steps) and for float32; long prompt steps
// of a mixture of experts in bfloat16 go through the tcgen05 product instead (gemm_tc.cu,
// gg_gemm_tc_grouped).
#include <mma.h>

#include <stdlib.h>

#include <type_traits>

#include "attention_common.cuh"

#define GGM_BM 32
#define GGM_BN 64
#define GGM_LDC (GGM_BN + 8)
#define GGM_THREADS 256

struct GroupedArgs {
  const void* A; long long lda; long long a_group_cols;
  const int* row_index; int row_div;
  const void* W;
  void* out; long long ldo; long long o_group_cols;
  const int* offsets;
  int M, G, N, K, Np, gated;
  const void* gate; long long ldg; int gate_col0;
};

template <typename TA> struct GgmZero;
template <> struct GgmZero<float> { static __device__ __forceinline__ float v() { return 0.f; } };
template <> struct GgmZero<__nv_bfloat16> { static __device__ __forceinline__ __nv_bfloat16 v() { return __float2bfloat16_rn(0.f); } };

// K is walked in steps of BK (128 for bfloat16, 32 for float32).  VEC: every row of A and W
// starts on a 16-byte boundary and K is a multiple of the 16-byte chunk, so tiles are fetched
// in chunks of 16 bytes, and the chunks of the next step are asked for (into registers) before
// the products of this one, which hides most of a trip to memory when a group has only a few
// rows and the kernel streams its weights (decoded tokens).
template <typename TA, bool GATED, int BK, bool VEC>
__global__ void __launch_bounds__(GGM_THREADS, (sizeof(TA) == 2 ? (GATED ? 2 : 4) : 1)) grouped_gemm_kernel(GroupedArgs a) {
  constexpr int LD = BK + 8;
  constexpr int NB = GATED ? 2 : 1;
  constexpr int VPT = 16 / (int)sizeof(TA);                     // values in a 16-byte chunk
  constexpr int CPR = BK / VPT;                                 // chunks in a tile row
  constexpr int A_CH = GGM_BM * CPR / GGM_THREADS, B_CH = GGM_BN * CPR / GGM_THREADS;
  static_assert(GGM_BM * CPR % GGM_THREADS == 0 && GGM_BN * CPR % GGM_THREADS == 0, "tile chunks must divide over the threads");
  constexpr int AB_BYTES = (GGM_BM + NB * GGM_BN) * LD * (int)sizeof(TA);
  constexpr int C_BYTES = NB * GGM_BM * GGM_LDC * (int)sizeof(float);
  __shared__ __align__(32) unsigned char raw[AB_BYTES > C_BYTES ? AB_BYTES : C_BYTES];
  __shared__ int arow_s[GGM_BM];
  TA* As = reinterpret_cast<TA*>(raw);
  TA* Bs = As + GGM_BM * LD;                                    // [NB][GGM_BN * LD]
  float* Cs = reinterpret_cast<float*>(raw);                    // [NB][GGM_BM * GGM_LDC], over the tiles once they are used up
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  int g = -1, r0 = 0, r_end = 0;
  if (a.offsets) {
    int tile = blockIdx.y;
    for (int e = 0; e < a.G; ++e) {
      const int lo = a.offsets[e], hi = a.offsets[e + 1];
      const int nt = (hi - lo + GGM_BM - 1) / GGM_BM;
      if (tile < nt) { g = e; r0 = lo + tile * GGM_BM; r_end = hi; break; }
      tile -= nt;
    }
    if (g < 0) return;
  } else {
    g = blockIdx.z; r0 = blockIdx.y * GGM_BM; r_end = a.M;
    if (r0 >= r_end) return;
  }
  const int n0 = blockIdx.x * GGM_BN;
  const int nrows = min(GGM_BM, r_end - r0);
  if (tid < GGM_BM) arow_s[tid] = tid < nrows ? (a.row_index ? a.row_index[r0 + tid] / a.row_div : r0 + tid) : -1;
  __syncthreads();
  const int N = a.N, K = a.K;
  const TA* A = (const TA*)a.A + (size_t)g * a.a_group_cols;
  const TA* W = (const TA*)a.W + (size_t)g * NB * N * K;
  const TA zero = GgmZero<TA>::v();

  constexpr bool TC = !std::is_same<TA, float>::value;
  const int warp = tid >> 5;
  const int rt = warp >> 2, ct = warp & 3;                 // tensor cores: the warp's 16 x 16 tile
  const int frow = tid >> 3, fcg = tid & 7;                // FMA: row, and columns fcg + 8 j
  nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, 16, float> acc0, acc1;
  float f0[8], f1[8];
  if (TC) {
    nvcuda::wmma::fill_fragment(acc0, 0.f);
    nvcuda::wmma::fill_fragment(acc1, 0.f);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) { f0[j] = 0.f; f1[j] = 0.f; }
  }

  uint4 ra[A_CH], rb[NB][B_CH];
  auto fetch = [&](int k0) {                               // VEC: this step's chunks into registers
#pragma unroll
    for (int u = 0; u < A_CH; ++u) {
      const int e = tid + u * GGM_THREADS, r = e / CPR, k = k0 + (e - r * CPR) * VPT;
      const int row = arow_s[r];
      ra[u] = (row >= 0 && k < K) ? *reinterpret_cast<const uint4*>(A + (size_t)row * a.lda + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < B_CH; ++u) {
      const int e = tid + u * GGM_THREADS, n = e / CPR, k = k0 + (e - n * CPR) * VPT;
      const bool ok = n0 + n < N && k < K;
      rb[0][u] = ok ? *reinterpret_cast<const uint4*>(W + (size_t)(n0 + n) * K + k) : make_uint4(0, 0, 0, 0);
      if (GATED) rb[NB - 1][u] = ok ? *reinterpret_cast<const uint4*>(W + (size_t)(N + n0 + n) * K + k) : make_uint4(0, 0, 0, 0);
    }
  };
  auto stash = [&]() {                                     // VEC: the registers into the shared tiles
#pragma unroll
    for (int u = 0; u < A_CH; ++u) {
      const int e = tid + u * GGM_THREADS, r = e / CPR, c = (e - r * CPR) * VPT;
      *reinterpret_cast<uint4*>(As + r * LD + c) = ra[u];
    }
#pragma unroll
    for (int u = 0; u < B_CH; ++u) {
      const int e = tid + u * GGM_THREADS, n = e / CPR, c = (e - n * CPR) * VPT;
      *reinterpret_cast<uint4*>(Bs + n * LD + c) = rb[0][u];
      if (GATED) *reinterpret_cast<uint4*>(Bs + (NB - 1) * GGM_BN * LD + n * LD + c) = rb[NB - 1][u];
    }
  };
  if (VEC) fetch(0);
  for (int k0 = 0; k0 < K; k0 += BK) {
    if (VEC) {
      stash();
    } else {
      for (int e = tid; e < GGM_BM * BK; e += GGM_THREADS) {
        const int r = e / BK, c = e - r * BK;
        const int row = arow_s[r], k = k0 + c;
        As[r * LD + c] = (row >= 0 && k < K) ? A[(size_t)row * a.lda + k] : zero;
      }
      for (int e = tid; e < GGM_BN * BK; e += GGM_THREADS) {
        const int n = e / BK, c = e - n * BK;
        const int col = n0 + n, k = k0 + c;
        const bool ok = col < N && k < K;
        Bs[n * LD + c] = ok ? W[(size_t)col * K + k] : zero;
        if (GATED) Bs[(NB - 1) * GGM_BN * LD + n * LD + c] = ok ? W[(size_t)(N + col) * K + k] : zero;
      }
    }
    __syncthreads();
    if (VEC && k0 + BK < K) fetch(k0 + BK);
    if constexpr (TC) {
      using namespace nvcuda;
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
      wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
#pragma unroll
      for (int kk = 0; kk < BK; kk += 16) {
        wmma::load_matrix_sync(fa, As + rt * 16 * LD + kk, LD);
        wmma::load_matrix_sync(fb, Bs + ct * 16 * LD + kk, LD);
        wmma::mma_sync(acc0, fa, fb, acc0);
        if (GATED) {
          wmma::load_matrix_sync(fb, Bs + (NB - 1) * GGM_BN * LD + ct * 16 * LD + kk, LD);
          wmma::mma_sync(acc1, fa, fb, acc1);
        }
      }
    } else {
#pragma unroll 8
      for (int k = 0; k < BK; ++k) {
        const float av = As[frow * LD + k];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          f0[j] = fmaf(av, Bs[(fcg + 8 * j) * LD + k], f0[j]);
          if (GATED) f1[j] = fmaf(av, Bs[(NB - 1) * GGM_BN * LD + (fcg + 8 * j) * LD + k], f1[j]);
        }
      }
    }
    __syncthreads();
  }
  float* Cs1 = Cs + (NB - 1) * GGM_BM * GGM_LDC;
  if constexpr (TC) {
    nvcuda::wmma::store_matrix_sync(Cs + rt * 16 * GGM_LDC + ct * 16, acc0, GGM_LDC, nvcuda::wmma::mem_row_major);
    if (GATED) nvcuda::wmma::store_matrix_sync(Cs1 + rt * 16 * GGM_LDC + ct * 16, acc1, GGM_LDC, nvcuda::wmma::mem_row_major);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      Cs[frow * GGM_LDC + fcg + 8 * j] = f0[j];
      if (GATED) Cs1[frow * GGM_LDC + fcg + 8 * j] = f1[j];
    }
  }
  __syncthreads();
  TA* out = (TA*)a.out + (size_t)g * a.o_group_cols;
  for (int e = tid; e < GGM_BM * GGM_BN; e += GGM_THREADS) {
    const int r = e / GGM_BN, c = e - r * GGM_BN;
    const int col = n0 + c;
    if (r >= nrows || col >= a.Np) continue;
    float v = 0.f;
    if (col < N) {
      v = Cs[r * GGM_LDC + c];
      if (GATED) {
        const float u = Cs1[r * GGM_LDC + c];
        v = v / (1.f + expf(-v)) * u;
      }
      if (a.gate) {
        const float z = to_f32(((const TA*)a.gate)[(size_t)arow_s[r] * a.ldg + a.gate_col0 + g]);
        v *= 1.f / (1.f + expf(-z));
      }
    }
    out[(size_t)(r0 + r) * a.ldo + col] = from_f32<TA>(v);
  }
}

// The same product for bfloat16 with long K (the experts' products of decoded tokens, where a CTA
// streams its slab of W and the rows are few): K in steps of 64 through a ring of four shared-memory
// stages filled by cp.async, so that three steps of a CTA are in flight while it multiplies the
// fourth; two CTAs per SM.  Rows past a group's end and columns past N or K arrive as zeros
// (cp.async with a source size of 0).  Needs what VEC needs.
#define GGR_BK 64
#define GGR_LD (GGR_BK + 8)
#define GGR_STAGES 4

template <bool GATED>
__global__ void __launch_bounds__(GGM_THREADS, 2) grouped_gemm_ring_kernel(GroupedArgs a) {
  using TA = __nv_bfloat16;
  constexpr int NB = GATED ? 2 : 1;
  constexpr int CPR = GGR_BK / 8;                                // 16-byte chunks in a tile row
  constexpr int A_ELEMS = GGM_BM * GGR_LD, B_ELEMS = GGM_BN * GGR_LD;
  constexpr int STAGE_ELEMS = A_ELEMS + NB * B_ELEMS;
  extern __shared__ __align__(128) unsigned char ring_raw[];
  __shared__ int arow_s[GGM_BM];
  TA* stages = reinterpret_cast<TA*>(ring_raw);
  float* Cs = reinterpret_cast<float*>(ring_raw);                // over the ring once it has drained
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  int g = -1, r0 = 0, r_end = 0;
  if (a.offsets) {
    int tile = blockIdx.y;
    for (int e = 0; e < a.G; ++e) {
      const int lo = a.offsets[e], hi = a.offsets[e + 1];
      const int nt = (hi - lo + GGM_BM - 1) / GGM_BM;
      if (tile < nt) { g = e; r0 = lo + tile * GGM_BM; r_end = hi; break; }
      tile -= nt;
    }
    if (g < 0) return;
  } else {
    g = blockIdx.z; r0 = blockIdx.y * GGM_BM; r_end = a.M;
    if (r0 >= r_end) return;
  }
  const int n0 = blockIdx.x * GGM_BN;
  const int nrows = min(GGM_BM, r_end - r0);
  if (tid < GGM_BM) arow_s[tid] = tid < nrows ? (a.row_index ? a.row_index[r0 + tid] / a.row_div : r0 + tid) : -1;
  __syncthreads();
  const int N = a.N, K = a.K;
  const TA* A = (const TA*)a.A + (size_t)g * a.a_group_cols;
  const TA* W = (const TA*)a.W + (size_t)g * NB * N * K;

  // what this thread fetches in every step: one chunk of A, two of each W tile
  const int ar = tid / CPR, ac = (tid % CPR) * 8;
  const int arow = arow_s[ar];
  const TA* a_src = A + (size_t)(arow >= 0 ? arow : 0) * a.lda + ac;
  const TA* b_src[2];
  bool b_ok[2];
  int b_off[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int e = tid + u * GGM_THREADS, n = e / CPR, c = (e % CPR) * 8;
    b_ok[u] = n0 + n < N;
    b_src[u] = W + (size_t)(b_ok[u] ? n0 + n : 0) * K + c;
    b_off[u] = n * GGR_LD + c;
  }
  auto issue = [&](int stage, int k0) {
    TA* As = stages + stage * STAGE_ELEMS;
    TA* Bs = As + A_ELEMS;
    const bool kin = k0 + ac < K;
    cp_async16(smem_u32(As + ar * GGR_LD + ac), kin ? a_src + k0 : A, (arow >= 0 && kin) ? 16 : 0);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int c = (tid + u * GGM_THREADS) % CPR * 8;
      const bool ok = b_ok[u] && k0 + c < K;
      cp_async16(smem_u32(Bs + b_off[u]), ok ? b_src[u] + k0 : W, ok ? 16 : 0);
      if (GATED) cp_async16(smem_u32(Bs + B_ELEMS + b_off[u]), ok ? b_src[u] + (size_t)N * K + k0 : W, ok ? 16 : 0);
    }
  };

  const int warp = tid >> 5, rt = warp >> 2, ct = warp & 3;
  nvcuda::wmma::fragment<nvcuda::wmma::accumulator, 16, 16, 16, float> acc0, acc1;
  nvcuda::wmma::fill_fragment(acc0, 0.f);
  nvcuda::wmma::fill_fragment(acc1, 0.f);
  const int nk = (K + GGR_BK - 1) / GGR_BK;
#pragma unroll
  for (int s = 0; s < GGR_STAGES - 1; ++s) {
    if (s < nk) issue(s, s * GGR_BK);
    cp_async_commit();
  }
  for (int it = 0; it < nk; ++it) {
    cp_async_wait<GGR_STAGES - 2>();                             // this step's stage has landed
    __syncthreads();                                             // ... for every thread; and the stage refilled below is used up
    const int nxt = it + GGR_STAGES - 1;
    if (nxt < nk) issue(nxt % GGR_STAGES, nxt * GGR_BK);
    cp_async_commit();
    const TA* As = stages + (it % GGR_STAGES) * STAGE_ELEMS;
    const TA* Bs = As + A_ELEMS;
    using namespace nvcuda;
    wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
#pragma unroll
    for (int kk = 0; kk < GGR_BK; kk += 16) {
      wmma::load_matrix_sync(fa, As + rt * 16 * GGR_LD + kk, GGR_LD);
      wmma::load_matrix_sync(fb, Bs + ct * 16 * GGR_LD + kk, GGR_LD);
      wmma::mma_sync(acc0, fa, fb, acc0);
      if (GATED) {
        wmma::load_matrix_sync(fb, Bs + B_ELEMS + ct * 16 * GGR_LD + kk, GGR_LD);
        wmma::mma_sync(acc1, fa, fb, acc1);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  float* Cs1 = Cs + (NB - 1) * GGM_BM * GGM_LDC;
  nvcuda::wmma::store_matrix_sync(Cs + rt * 16 * GGM_LDC + ct * 16, acc0, GGM_LDC, nvcuda::wmma::mem_row_major);
  if (GATED) nvcuda::wmma::store_matrix_sync(Cs1 + rt * 16 * GGM_LDC + ct * 16, acc1, GGM_LDC, nvcuda::wmma::mem_row_major);
  __syncthreads();
  TA* out = (TA*)a.out + (size_t)g * a.o_group_cols;
  for (int e = tid; e < GGM_BM * GGM_BN; e += GGM_THREADS) {
    const int r = e / GGM_BN, c = e - r * GGM_BN;
    const int col = n0 + c;
    if (r >= nrows || col >= a.Np) continue;
    float v = 0.f;
    if (col < N) {
      v = Cs[r * GGM_LDC + c];
      if (GATED) {
        const float u = Cs1[r * GGM_LDC + c];
        v = v / (1.f + expf(-v)) * u;
      }
      if (a.gate) {
        const float z = to_f32(((const TA*)a.gate)[(size_t)arow_s[r] * a.ldg + a.gate_col0 + g]);
        v *= 1.f / (1.f + expf(-z));
      }
    }
    out[(size_t)(r0 + r) * a.ldo + col] = from_f32<TA>(v);
  }
}

extern "C" int gg_grouped_gemm(const void* A, long long lda, long long a_group_cols, const int* row_index,
                               int row_div, const void* W, void* out, long long ldo, long long o_group_cols,
                               const int* offsets, int M, int G, int N, int K, int Np, int gated,
                               const void* gate, long long ldg, int gate_col0, int act_dtype,
                               cudaStream_t stream) {
  GG_REQUIRE(M >= 0 && G > 0 && N > 0 && K > 0 && Np >= N, "grouped_gemm: bad sizes M=%d G=%d N=%d K=%d Np=%d", M, G, N, K, Np);
  GG_REQUIRE(A && W && out, "grouped_gemm: a pointer is null");
  GG_REQUIRE(!row_index || row_div > 0, "grouped_gemm: a row list needs its divisor");
  if (M == 0) return GG_OK;
  GroupedArgs a;
  a.A = A; a.lda = lda; a.a_group_cols = a_group_cols; a.row_index = row_index; a.row_div = row_div;
  a.W = W; a.out = out; a.ldo = ldo; a.o_group_cols = o_group_cols; a.offsets = offsets;
  a.M = M; a.G = G; a.N = N; a.K = K; a.Np = Np; a.gated = gated;
  a.gate = gate; a.ldg = ldg; a.gate_col0 = gate_col0;
  const int row_tiles = offsets ? (M + GGM_BM - 1) / GGM_BM + G : (M + GGM_BM - 1) / GGM_BM;
  GG_REQUIRE(row_tiles <= 65535 && G <= 65535, "grouped_gemm: %d row tiles or %d groups are too many for one launch", row_tiles, G);
  dim3 grid((Np + GGM_BN - 1) / GGM_BN, row_tiles, offsets ? 1 : G);
  const int esize = act_dtype == GG_F32 ? 4 : 2, vpt = 16 / esize;
  const bool vec = K % vpt == 0 && lda % vpt == 0 && a_group_cols % vpt == 0 && ((size_t)A % 16) == 0 && ((size_t)W % 16) == 0;
#define GGM_LAUNCH(T, BK)                                                                                      \
  do {                                                                                                         \
    if (gated && vec) gg_launch(grouped_gemm_kernel<T, true, BK, true>, grid, dim3(GGM_THREADS), 0, stream, a);        \
    else if (gated) gg_launch(grouped_gemm_kernel<T, true, BK, false>, grid, dim3(GGM_THREADS), 0, stream, a);         \
    else if (vec) gg_launch(grouped_gemm_kernel<T, false, BK, true>, grid, dim3(GGM_THREADS), 0, stream, a);           \
    else gg_launch(grouped_gemm_kernel<T, false, BK, false>, grid, dim3(GGM_THREADS), 0, stream, a);                   \
  } while (0)
  static const bool ring_on = !(getenv("GOLLMGO_B200_GROUPED_RING") && getenv("GOLLMGO_B200_GROUPED_RING")[0] == '0');
  if (act_dtype == GG_BF16 && vec && K >= 4 * GGR_BK && ring_on) {
    const size_t smem = (size_t)GGR_STAGES * (GGM_BM + (gated ? 2 : 1) * GGM_BN) * GGR_LD * sizeof(__nv_bfloat16);
    cudaError_t e = gated ? cudaFuncSetAttribute(grouped_gemm_ring_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                          : cudaFuncSetAttribute(grouped_gemm_ring_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gg_fail(GG_ERR_CUDA, "grouped_gemm: %s", cudaGetErrorString(e));
    if (gated) gg_launch(grouped_gemm_ring_kernel<true>, grid, dim3(GGM_THREADS), smem, stream, a);
    else gg_launch(grouped_gemm_ring_kernel<false>, grid, dim3(GGM_THREADS), smem, stream, a);
    return gg_check_launch("grouped_gemm");
  }
  if (act_dtype == GG_F32) {
    GGM_LAUNCH(float, 32);
  } else if (act_dtype == GG_BF16) {
    GGM_LAUNCH(__nv_bfloat16, 128);
  } else {
    return gg_fail(GG_ERR_INVALID, "grouped_gemm: unknown dtype %d", act_dtype);
  }
  return gg_check_launch("grouped_gemm");
}
