// Routing of a mixture of experts, on the device from start to end (a step never asks the host
// how many tokens an expert got, so a step of decoded tokens can be captured and replayed).
//
// gg_moe_route:   z[t, e] = h[t] . Wr[e] + b[e] in float32; the `top` largest logits of a token
//                 (ties: the lower index) are its experts, weights = softmax over those alone
// gg_moe_align:   the (token, choice) pairs sorted by expert: offsets[e] .. offsets[e+1] are the
//                 places of expert e in `sorted` (values t * top + j), `place` is the inverse
// gg_moe_combine: out[t] = sum_j weight[t, j] * y[place[t * top + j]] (+ shared[t]), float32 sums
//                 in the order of j
// The products between them are gg_grouped_gemm's (grouped_gemm.cu).
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 32

template <typename TA>
__global__ void moe_route_kernel(const TA* __restrict__ h, const TA* __restrict__ wr, const float* __restrict__ bias,
                                 int D, int E, int top, int* __restrict__ idx, float* __restrict__ wgt) {
  __shared__ float z[MOE_MAX_EXPERTS];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const TA* x = h + (size_t)t * D;
  for (int e = warp; e < E; e += nw) {
    const TA* w = wr + (size_t)e * D;
    float s = 0.f;
    for (int c = lane; c < D; c += 32) s = fmaf(to_f32(x[c]), to_f32(w[c]), s);
    s = warp_sum(s);
    if (lane == 0) z[e] = s + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp == 0) {
    float val[MOE_MAX_TOP];
    for (int j = 0; j < top; ++j) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const float v = z[e];
        if (v > best || (v == best && e < bi)) { best = v; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (bi == 0x7fffffff) bi = 0;                  // every logit left is -inf or NaN
      val[j] = best;
      if (lane == 0) { idx[(size_t)t * top + j] = bi; z[bi] = -INFINITY; }
      __syncwarp();
    }
    if (lane == 0) {
      const float m = val[0];                        // the largest comes first
      float sum = 0.f;
      for (int j = 0; j < top; ++j) { val[j] = expf(val[j] - m); sum += val[j]; }
      for (int j = 0; j < top; ++j) wgt[(size_t)t * top + j] = val[j] / sum;
    }
  }
}

// One CTA.  counts and cursors in shared memory; the order of the rows inside an expert's range
// is whatever the atomics give, which no result depends on.
__global__ void moe_align_kernel(const int* __restrict__ idx, int n, int E, int* __restrict__ offsets,
                                 int* __restrict__ sorted, int* __restrict__ place) {
  __shared__ int cnt[MOE_MAX_EXPERTS + 1];
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { const int c = cnt[e]; cnt[e] = run; offsets[e] = run; run += c; }
    offsets[E] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = atomicAdd(&cnt[idx[i]], 1);
    sorted[p] = i;
    place[i] = p;
  }
}

template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wgt,
                                   const TA* __restrict__ shared_out, TA* __restrict__ out, int D, int top) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < top; ++j)
      s = fmaf(wgt[t * top + j], to_f32(y[(size_t)place[t * top + j] * D + c]), s);
    if (shared_out) s += to_f32(shared_out[t * D + c]);
    out[t * D + c] = from_f32<TA>(s);
  }
}

extern "C" int gg_moe_route(const void* h, const void* wr, const float* bias, int T, int D, int E, int top,
                            int* idx, float* wgt, int act_dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && D > 0 && E > 0 && top > 0 && top <= E, "moe_route: bad sizes T=%d D=%d E=%d top=%d", T, D, E, top);
  GG_REQUIRE(E <= MOE_MAX_EXPERTS && top <= MOE_MAX_TOP, "moe_route: at most %d experts and %d choices a token (got %d, %d)",
             MOE_MAX_EXPERTS, MOE_MAX_TOP, E, top);
  GG_REQUIRE(h && wr && idx && wgt, "moe_route: a pointer is null");
  if (T == 0) return GG_OK;
  if (act_dtype == GG_F32)
    gg_launch(moe_route_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)h, (const float*)wr, bias, D, E, top, idx, wgt);
  else if (act_dtype == GG_BF16)
    gg_launch(moe_route_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)wr,
              bias, D, E, top, idx, wgt);
  else
    return gg_fail(GG_ERR_INVALID, "moe_route: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_route");
}

extern "C" int gg_moe_align(const int* idx, int n, int E, int* offsets, int* sorted, int* place, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && E > 0 && E <= MOE_MAX_EXPERTS, "moe_align: bad sizes n=%d E=%d", n, E);
  GG_REQUIRE(idx && offsets && sorted && place, "moe_align: a pointer is null");
  gg_launch(moe_align_kernel, dim3(1), dim3(1024), 0, stream, idx, n, E, offsets, sorted, place);
  return gg_check_launch("moe_align");
}

extern "C" int gg_moe_combine(const void* y, const int* place, const float* wgt, const void* shared_out, void* out,
                              int T, int D, int top, int act_dtype, cudaStream_t stream) {
  GG_REQUIRE(T >= 0 && D > 0 && top > 0, "moe_combine: bad sizes T=%d D=%d top=%d", T, D, top);
  GG_REQUIRE(y && place && wgt && out, "moe_combine: a pointer is null");
  if (T == 0) return GG_OK;
  const int threads = D >= 1024 ? 256 : 128;
  if (act_dtype == GG_F32)
    gg_launch(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)y, place, wgt, (const float*)shared_out,
              (float*)out, D, top);
  else if (act_dtype == GG_BF16)
    gg_launch(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)y, place, wgt,
              (const __nv_bfloat16*)shared_out, (__nv_bfloat16*)out, D, top);
  else
    return gg_fail(GG_ERR_INVALID, "moe_combine: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_combine");
}
