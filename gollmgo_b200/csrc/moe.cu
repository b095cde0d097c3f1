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

// dot of the staged row xs[0..D) with one router row, over the lanes of a warp
__device__ __forceinline__ float route_dot(const float* xs, const float* w, int D, int lane, bool vec) {
  float s = 0.f;
  if (vec) {
    for (int c = lane * 4; c < D; c += 128) {
      const float4 a = *reinterpret_cast<const float4*>(xs + c), b = *reinterpret_cast<const float4*>(w + c);
      s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
    }
  } else {
    for (int c = lane; c < D; c += 32) s = fmaf(xs[c], w[c], s);
  }
  return s;
}
__device__ __forceinline__ float route_dot(const float* xs, const __nv_bfloat16* w, int D, int lane, bool vec) {
  float s = 0.f;
  if (vec) {
    for (int c = lane * 8; c < D; c += 256) {
      const uint4 r = *reinterpret_cast<const uint4*>(w + c);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
      const float4 x0 = *reinterpret_cast<const float4*>(xs + c), x1 = *reinterpret_cast<const float4*>(xs + c + 4);
      const float2 b0 = __bfloat1622float2(p[0]), b1 = __bfloat1622float2(p[1]);
      const float2 b2 = __bfloat1622float2(p[2]), b3 = __bfloat1622float2(p[3]);
      s = fmaf(x0.x, b0.x, s); s = fmaf(x0.y, b0.y, s); s = fmaf(x0.z, b1.x, s); s = fmaf(x0.w, b1.y, s);
      s = fmaf(x1.x, b2.x, s); s = fmaf(x1.y, b2.y, s); s = fmaf(x1.z, b3.x, s); s = fmaf(x1.w, b3.y, s);
    }
  } else {
    for (int c = lane; c < D; c += 32) s = fmaf(xs[c], __bfloat162float(w[c]), s);
  }
  return s;
}

template <typename TA>
__global__ void moe_route_kernel(const TA* __restrict__ h, const TA* __restrict__ wr, const float* __restrict__ bias,
                                 int D, int E, int top, int* __restrict__ idx, float* __restrict__ wgt, int vec) {
  __shared__ float z[MOE_MAX_EXPERTS];
  extern __shared__ __align__(16) float xs[];              // the token's row, D floats
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const TA* x = h + (size_t)t * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) xs[c] = to_f32(x[c]);
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    const float s = warp_sum(route_dot(xs, wr + (size_t)e * D, D, lane, vec != 0));
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
// is whatever the atomics give, which no result depends on.  pad > 1: every expert's range
// starts at a multiple of pad (the places between its last row and the next range hold -1 in
// `sorted`), `slots` is the length of `sorted`, and tile_group[i] is the expert that places
// pad * i .. pad * i + pad - 1 belong to, or -1 past the last range (n_tiles entries).
__global__ void moe_align_kernel(const int* __restrict__ idx, int n, int E, int pad, int slots, int* __restrict__ offsets,
                                 int* __restrict__ sorted, int* __restrict__ place, int* __restrict__ tile_group,
                                 int n_tiles) {
  __shared__ int cnt[MOE_MAX_EXPERTS + 1];
  __shared__ int start[MOE_MAX_EXPERTS + 1];
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  if (pad > 1)
    for (int i = threadIdx.x; i < slots; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      cnt[e] = run; start[e] = run; offsets[e] = run;
      run += (c + pad - 1) / pad * pad;
    }
    start[E] = run; offsets[E] = run;
  }
  __syncthreads();
  if (tile_group)
    for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) {
      const int p = i * pad;
      int g = -1;
      if (p < start[E]) {
        int lo = 0, hi = E;                          // the last expert whose range starts at or before p
        while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (start[mid] <= p) lo = mid; else hi = mid; }
        g = lo;
      }
      tile_group[i] = g;
    }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = atomicAdd(&cnt[idx[i]], 1);
    sorted[p] = i;
    place[i] = p;
  }
}

// xs[p] = x[sorted[p] / top] for the places that hold a pair, zeros for the others: the rows of
// every expert gathered into one block that starts at a multiple of the product's tile height.
template <typename TA>
__global__ void moe_gather_kernel(const TA* __restrict__ x, const int* __restrict__ sorted, int top, int D,
                                  TA* __restrict__ xs, int vec) {
  pdl_trigger();
  pdl_wait();
  const size_t p = blockIdx.x;
  const int src = sorted[p];
  TA* o = xs + p * D;
  if (vec) {
    constexpr int VPT = 16 / (int)sizeof(TA);
    const uint4* in = src >= 0 ? reinterpret_cast<const uint4*>(x + (size_t)(src / top) * D) : nullptr;
    for (int c = threadIdx.x; c < D / VPT; c += blockDim.x)
      reinterpret_cast<uint4*>(o)[c] = in ? in[c] : make_uint4(0, 0, 0, 0);
  } else {
    const TA* in = src >= 0 ? x + (size_t)(src / top) * D : nullptr;
    for (int c = threadIdx.x; c < D; c += blockDim.x) o[c] = in ? in[c] : from_f32<TA>(0.f);
  }
}

template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wgt,
                                   const TA* __restrict__ shared_out, TA* __restrict__ out, int D, int top) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  if (D % 4 == 0) {                              // rows of every buffer are then 8-byte aligned at least
    for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      for (int j = 0; j < top; ++j) {
        const float w = wgt[t * top + j];
        const TA* r = y + (size_t)place[t * top + j] * D + c;
        s0 = fmaf(w, to_f32(r[0]), s0); s1 = fmaf(w, to_f32(r[1]), s1);
        s2 = fmaf(w, to_f32(r[2]), s2); s3 = fmaf(w, to_f32(r[3]), s3);
      }
      if (shared_out) {
        const TA* r = shared_out + t * D + c;
        s0 += to_f32(r[0]); s1 += to_f32(r[1]); s2 += to_f32(r[2]); s3 += to_f32(r[3]);
      }
      TA* o = out + t * D + c;
      o[0] = from_f32<TA>(s0); o[1] = from_f32<TA>(s1); o[2] = from_f32<TA>(s2); o[3] = from_f32<TA>(s3);
    }
    return;
  }
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
  const size_t smem = (size_t)D * sizeof(float);
  GG_REQUIRE(smem <= 160 * 1024, "moe_route: rows of %d values do not fit in shared memory", D);
  const int vec = (act_dtype == GG_F32 ? D % 4 == 0 : D % 8 == 0) && ((size_t)wr % 16) == 0;
  const int threads = E >= 8 ? 256 : 128;
  if (act_dtype == GG_F32) {
    if (smem > 44 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gg_launch(moe_route_kernel<float>, dim3(T), dim3(threads), smem, stream, (const float*)h, (const float*)wr, bias, D, E, top, idx, wgt, vec);
  } else if (act_dtype == GG_BF16) {
    if (smem > 44 * 1024) cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gg_launch(moe_route_kernel<__nv_bfloat16>, dim3(T), dim3(threads), smem, stream, (const __nv_bfloat16*)h, (const __nv_bfloat16*)wr,
              bias, D, E, top, idx, wgt, vec);
  } else
    return gg_fail(GG_ERR_INVALID, "moe_route: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_route");
}

extern "C" int gg_moe_align(const int* idx, int n, int E, int pad, int slots, int* offsets, int* sorted, int* place,
                            int* tile_group, int n_tiles, cudaStream_t stream) {
  GG_REQUIRE(n >= 0 && E > 0 && E <= MOE_MAX_EXPERTS && pad >= 1, "moe_align: bad sizes n=%d E=%d pad=%d", n, E, pad);
  GG_REQUIRE(idx && offsets && sorted && place, "moe_align: a pointer is null");
  GG_REQUIRE(pad == 1 || (long long)slots >= (long long)n + (long long)E * (pad - 1),
             "moe_align: %d places do not hold %d rows of %d experts padded to %d", slots, n, E, pad);
  GG_REQUIRE(!tile_group || (long long)n_tiles * pad >= slots, "moe_align: %d tile entries for %d places", n_tiles, slots);
  gg_launch(moe_align_kernel, dim3(1), dim3(1024), 0, stream, idx, n, E, pad, slots, offsets, sorted, place, tile_group, n_tiles);
  return gg_check_launch("moe_align");
}

extern "C" int gg_moe_gather(const void* x, const int* sorted, int slots, int top, int D, void* xs, int act_dtype,
                             cudaStream_t stream) {
  GG_REQUIRE(slots >= 0 && top > 0 && D > 0 && x && sorted && xs, "moe_gather: bad arguments");
  if (slots == 0) return GG_OK;
  const int vpt = act_dtype == GG_F32 ? 4 : 8;
  const int vec = D % vpt == 0 && ((size_t)x % 16) == 0 && ((size_t)xs % 16) == 0;
  if (act_dtype == GG_F32)
    gg_launch(moe_gather_kernel<float>, dim3(slots), dim3(128), 0, stream, (const float*)x, sorted, top, D, (float*)xs, vec);
  else if (act_dtype == GG_BF16)
    gg_launch(moe_gather_kernel<__nv_bfloat16>, dim3(slots), dim3(128), 0, stream, (const __nv_bfloat16*)x, sorted, top, D,
              (__nv_bfloat16*)xs, vec);
  else
    return gg_fail(GG_ERR_INVALID, "moe_gather: unknown dtype %d", act_dtype);
  return gg_check_launch("moe_gather");
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
