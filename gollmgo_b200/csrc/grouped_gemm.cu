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
// of 32 rows x 64 columns, K in steps of 32 through shared memory, any N and K.
#include <mma.h>

#include <type_traits>

#include "common.cuh"

#define GGM_BM 32
#define GGM_BN 64
#define GGM_BK 32
#define GGM_LD (GGM_BK + 8)
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

template <typename TA, bool GATED>
__global__ void __launch_bounds__(GGM_THREADS) grouped_gemm_kernel(GroupedArgs a) {
  __shared__ __align__(32) TA As[GGM_BM * GGM_LD];
  __shared__ __align__(32) TA Bs[GATED ? 2 : 1][GGM_BN * GGM_LD];
  __shared__ __align__(32) float Cs[GATED ? 2 : 1][GGM_BM * GGM_LDC];
  __shared__ int arow_s[GGM_BM];
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
  const TA* W = (const TA*)a.W + (size_t)g * (GATED ? 2 : 1) * N * K;
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

  for (int k0 = 0; k0 < K; k0 += GGM_BK) {
    for (int e = tid; e < GGM_BM * GGM_BK; e += GGM_THREADS) {
      const int r = e / GGM_BK, c = e - r * GGM_BK;
      const int row = arow_s[r], k = k0 + c;
      As[r * GGM_LD + c] = (row >= 0 && k < K) ? A[(size_t)row * a.lda + k] : zero;
    }
    for (int e = tid; e < GGM_BN * GGM_BK; e += GGM_THREADS) {
      const int n = e / GGM_BK, c = e - n * GGM_BK;
      const int col = n0 + n, k = k0 + c;
      const bool ok = col < N && k < K;
      Bs[0][n * GGM_LD + c] = ok ? W[(size_t)col * K + k] : zero;
      if (GATED) Bs[GATED ? 1 : 0][n * GGM_LD + c] = ok ? W[(size_t)(N + col) * K + k] : zero;
    }
    __syncthreads();
    if constexpr (TC) {
      using namespace nvcuda;
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
      wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
#pragma unroll
      for (int kk = 0; kk < GGM_BK; kk += 16) {
        wmma::load_matrix_sync(fa, As + rt * 16 * GGM_LD + kk, GGM_LD);
        wmma::load_matrix_sync(fb, Bs[0] + ct * 16 * GGM_LD + kk, GGM_LD);
        wmma::mma_sync(acc0, fa, fb, acc0);
        if (GATED) {
          wmma::load_matrix_sync(fb, Bs[GATED ? 1 : 0] + ct * 16 * GGM_LD + kk, GGM_LD);
          wmma::mma_sync(acc1, fa, fb, acc1);
        }
      }
    } else {
#pragma unroll 8
      for (int k = 0; k < GGM_BK; ++k) {
        const float av = As[frow * GGM_LD + k];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          f0[j] = fmaf(av, Bs[0][(fcg + 8 * j) * GGM_LD + k], f0[j]);
          if (GATED) f1[j] = fmaf(av, Bs[GATED ? 1 : 0][(fcg + 8 * j) * GGM_LD + k], f1[j]);
        }
      }
    }
    __syncthreads();
  }
  if constexpr (TC) {
    nvcuda::wmma::store_matrix_sync(Cs[0] + rt * 16 * GGM_LDC + ct * 16, acc0, GGM_LDC, nvcuda::wmma::mem_row_major);
    if (GATED) nvcuda::wmma::store_matrix_sync(Cs[GATED ? 1 : 0] + rt * 16 * GGM_LDC + ct * 16, acc1, GGM_LDC, nvcuda::wmma::mem_row_major);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      Cs[0][frow * GGM_LDC + fcg + 8 * j] = f0[j];
      if (GATED) Cs[GATED ? 1 : 0][frow * GGM_LDC + fcg + 8 * j] = f1[j];
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
      v = Cs[0][r * GGM_LDC + c];
      if (GATED) {
        const float u = Cs[GATED ? 1 : 0][r * GGM_LDC + c];
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
  if (act_dtype == GG_F32) {
    if (gated) gg_launch(grouped_gemm_kernel<float, true>, grid, dim3(GGM_THREADS), 0, stream, a);
    else gg_launch(grouped_gemm_kernel<float, false>, grid, dim3(GGM_THREADS), 0, stream, a);
  } else if (act_dtype == GG_BF16) {
    if (gated) gg_launch(grouped_gemm_kernel<__nv_bfloat16, true>, grid, dim3(GGM_THREADS), 0, stream, a);
    else gg_launch(grouped_gemm_kernel<__nv_bfloat16, false>, grid, dim3(GGM_THREADS), 0, stream, a);
  } else {
    return gg_fail(GG_ERR_INVALID, "grouped_gemm: unknown dtype %d", act_dtype);
  }
  return gg_check_launch("grouped_gemm");
}
