// Mixture of experts: the router and the weighting of the experts' activations.
//
// moe_route, a block per token (or four): logits z = W_router h in float (h in the activation type,
// the router's rows in float), the `top` largest chosen (the lower index wins a tie), their
// weights the softmax over the chosen logits alone.  It leaves a dense row of weights
// `route_w [T, E (+1)]` (zero for an expert not chosen) beside the chosen ids and weights;
// with a shared expert that has a gate of its own, row E of the router matrix is that gate's
// weight vector and column E receives sigmoid(w_sg . h).
//
// The router has a second way of scoring (`mode` 1): the scores are the softmax over all of
// the router's outputs; a correction per output is added for the choice only; with groups the
// outputs form `n_groups` equal groups of neighbours, a group counts by its largest choice
// score and only the outputs of the best `keep` groups can be chosen; the chosen outputs'
// weights are their scores over their sum (+ weight_eps), times route_scale.  The last
// `identity` of the router's outputs stand for experts that return their input: their weights
// are added up in a column of their own behind the experts' (and the shared gate's), and
// bf_moe_identity_add adds input times that column to the mixture's output.
//
// moe_act: for experts whose gate and up projections are stacked into one product
// `gu [T, 2F]` (gate rows of all experts, then up rows; F = E ff + ff_shared), the
// activations of every expert scaled by the token's weight for that expert,
//   act[t, c] = silu(gu[t, c]) * gu[t, F + c] * route_w[t, expert(c)],
// so that one product with the stacked down projections gives the weighted sum.
#include <float.h>

#include "common.cuh"

// One block per MR_TOKENS tokens: their rows go to shared memory as float; every warp takes a
// slice of the width and, row by row of the router, its share of each token's dot product
// (a router row is fetched once for all the block's tokens); the shares are then added in
// the warps' order, and one warp per token chooses.  A token's sums do not depend on which
// other tokens share its block.
#define MR_TOKENS 4
#define MR_WARPS 8

template <typename A>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(
    const A* __restrict__ h, long long stride, const float* __restrict__ w, int T, int width,
    int E, int top, int shared_gate, int tokens_per_block, float* __restrict__ route_w,
    int* __restrict__ top_ids, float* __restrict__ top_w, int mode,
    const float* __restrict__ correction, int n_groups, int keep, int identity,
    float route_scale, float weight_eps) {
  extern __shared__ __align__(16) float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * tokens_per_block;
  const int nt = min(tokens_per_block, T - t0);
  const int R = E + identity;                      // the router's outputs that can be chosen
  const int rows = R + (shared_gate ? 1 : 0);
  const int rw_cols = E + (shared_gate ? 1 : 0) + (identity ? 1 : 0);
  const int wp = (width + 3) & ~3;
  float* x = sh;                                   // [MR_TOKENS][wp]
  float* part = sh + (size_t)MR_TOKENS * wp;       // [MR_WARPS][MR_TOKENS][rows]
  float* zs = part + (size_t)MR_WARPS * MR_TOKENS * rows;   // [MR_TOKENS][rows]
  float* chs = zs + (size_t)MR_TOKENS * rows;      // [MR_TOKENS][rows]: choice scores (mode 1)
  for (int k = 0; k < nt; ++k) {
    const A* src = h + (size_t)(t0 + k) * stride;
#pragma unroll 8
    for (int c = threadIdx.x; c < width; c += blockDim.x) x[(size_t)k * wp + c] = bf_ld(src + c);
  }
  __syncthreads();
  const bool vec = (width & 3) == 0 && (((uintptr_t)w) & 15) == 0;
  // this warp's slice of the width, in units of four columns (or of one without `vec`)
  const int units = vec ? width >> 2 : width;
  const int per = (units + MR_WARPS - 1) / MR_WARPS;
  const int lo = warp * per, hi = min(units, lo + per);
  for (int e = 0; e < rows; ++e) {
    const float* wr = w + (size_t)e * width;
    float a[MR_TOKENS];
#pragma unroll
    for (int k = 0; k < MR_TOKENS; ++k) a[k] = 0.f;
    if (vec) {
      // four pieces of the row a lane at a time, all fetched before any is used: the round
      // trips to L2 overlap (the sums keep the order of a plain walk)
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      for (int c = lo + lane; c < hi; c += 128) {
        float4 p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          p[u] = c + 32 * u < hi ? w4[c + 32 * u] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c + 32 * u < hi) {
#pragma unroll
            for (int k = 0; k < MR_TOKENS; ++k) {
              if (k < nt) {
                const float4 q = reinterpret_cast<const float4*>(x + (size_t)k * wp)[c + 32 * u];
                a[k] += p[u].x * q.x;
                a[k] += p[u].y * q.y;
                a[k] += p[u].z * q.z;
                a[k] += p[u].w * q.w;
              }
            }
          }
        }
      }
    } else {
      for (int c = lo + lane; c < hi; c += 32) {
        const float p = wr[c];
#pragma unroll
        for (int k = 0; k < MR_TOKENS; ++k)
          if (k < nt) a[k] += p * x[(size_t)k * wp + c];
      }
    }
#pragma unroll
    for (int k = 0; k < MR_TOKENS; ++k) {
      const float r = warp_sum(a[k]);
      if (lane == 0) part[((size_t)warp * MR_TOKENS + k) * rows + e] = r;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nt * rows; i += blockDim.x) {
    const int k = i / rows, e = i - k * rows;
    float r = 0.f;
    for (int wv = 0; wv < MR_WARPS; ++wv) r += part[((size_t)wv * MR_TOKENS + k) * rows + e];
    zs[(size_t)k * rows + e] = r;
  }
  __syncthreads();
  if (warp >= nt) return;
  const int t = t0 + warp;
  float* z = zs + (size_t)warp * rows;
  float* rw = route_w + (size_t)t * rw_cols;
  for (int e = lane; e < rw_cols; e += 32) rw[e] = 0.f;
  if (shared_gate && lane == 0) rw[E] = 1.f / (1.f + expf(-z[R]));
  __syncwarp();
  if (mode == 1) {
    float* ch = chs + (size_t)warp * rows;
    // this warp's slice of the partial sums' place, which nobody reads any more
    float* gsc = part + (size_t)warp * MR_TOKENS * rows;   // [n_groups] scores, [n_groups] kept
    float zmax = -FLT_MAX;
    for (int e = lane; e < R; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float den = 0.f;
    for (int e = lane; e < R; e += 32) den += expf(z[e] - zmax);
    den = warp_sum(den);
    for (int e = lane; e < R; e += 32) {
      const float sc = expf(z[e] - zmax) / den;
      z[e] = sc;
      ch[e] = sc + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
    if (n_groups > 1) {
      const int per = R / n_groups;
      for (int g = lane; g < n_groups; g += 32) {
        float best = -FLT_MAX;
        for (int i = 0; i < per; ++i) best = fmaxf(best, ch[g * per + i]);
        gsc[g] = best;
        gsc[n_groups + g] = 0.f;
      }
      __syncwarp();
      for (int k = 0; k < keep; ++k) {
        float best = -FLT_MAX;
        int at = 0x7fffffff;
        for (int g = lane; g < n_groups; g += 32)
          if (gsc[n_groups + g] == 0.f && (gsc[g] > best || at == 0x7fffffff)) {
            best = gsc[g];
            at = g;
          }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, at, o);
          if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) {
            best = ob;
            at = oa;
          }
        }
        if (lane == 0 && at != 0x7fffffff) gsc[n_groups + at] = 1.f;
        __syncwarp();
      }
      for (int e = lane; e < R; e += 32)
        if (gsc[n_groups + e / per] == 0.f) ch[e] = -FLT_MAX;
      __syncwarp();
    }
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      float best = -FLT_MAX;
      int at = 0x7fffffff;
      for (int e = lane; e < R; e += 32)
        if (ch[e] > best) { best = ch[e]; at = e; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
      }
      if (at == 0x7fffffff) at = 0;             // (fewer outputs left than `top`: not reached)
      const float sc = z[at];
      sum += sc;
      if (lane == 0) {
        top_ids[(size_t)t * top + k] = at;
        top_w[(size_t)t * top + k] = sc;
        ch[at] = -FLT_MAX;
      }
      __syncwarp();
    }
    const float f = route_scale / (sum + weight_eps);
    if (lane == 0) {
      for (int k = 0; k < top; ++k) {
        const float pw = top_w[(size_t)t * top + k] * f;
        const int id = top_ids[(size_t)t * top + k];
        top_w[(size_t)t * top + k] = pw;
        if (id < E) rw[id] = pw;
        else rw[rw_cols - 1] += pw;
      }
    }
    return;
  }
  // the `top` largest, one after the other; the first is the softmax's maximum
  float zmax = 0.f, den = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -FLT_MAX;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (z[e] > best) { best = z[e]; at = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (k == 0) zmax = best;
    const float p = expf(best - zmax);
    den += p;
    if (lane == 0) {
      top_ids[(size_t)t * top + k] = at;
      top_w[(size_t)t * top + k] = p;
      z[at] = -FLT_MAX;
    }
    __syncwarp();
  }
  const float inv = 1.f / den;
  if (lane == 0) {
    for (int k = 0; k < top; ++k) {
      const float p = top_w[(size_t)t * top + k] * inv;
      top_w[(size_t)t * top + k] = p;
      rw[top_ids[(size_t)t * top + k]] = p;
    }
  }
}

BF_EXPORT int bf_moe_route(const void* h, long long stride, const float* w, int T, int width,
                           int E, int top, int shared_gate, float* route_w, int* top_ids,
                           float* top_w, int act_dtype, int mode, const float* correction,
                           int n_groups, int keep, int identity, float route_scale,
                           float weight_eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (mode == 0) { identity = 0; n_groups = 1; correction = nullptr; }
  if (n_groups < 1) n_groups = 1;
  if (top < 1 || top > E + identity || identity < 0 || (E + identity) % n_groups ||
      keep < 1 || keep > n_groups || top > keep * ((E + identity) / n_groups))
    return (int)cudaErrorInvalidValue;
  const int rows = E + identity + (shared_gate ? 1 : 0);
  // few tokens: one a block, so that the step's blocks are many; else a router row serves four
  const int tpb = T >= 4 * 148 ? MR_TOKENS : 1;
  const size_t smem = ((size_t)MR_TOKENS * ((width + 3) & ~3) +
                       (size_t)(MR_WARPS + 2) * MR_TOKENS * rows) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const unsigned blocks = (unsigned)((T + tpb - 1) / tpb);
  if (act_dtype == BF_DTYPE_F32) {
    auto k = moe_route_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<blocks, MR_WARPS * 32, smem, stream>>>((const float*)h, stride, w, T, width, E, top,
                                               shared_gate, tpb, route_w, top_ids, top_w, mode,
                                               correction, n_groups, keep, identity, route_scale,
                                               weight_eps);
  } else {
    auto k = moe_route_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<blocks, MR_WARPS * 32, smem, stream>>>((const __nv_bfloat16*)h, stride, w, T, width, E,
                                               top, shared_gate, tpb, route_w, top_ids, top_w,
                                               mode, correction, n_groups, keep, identity,
                                               route_scale, weight_eps);
  }
  return bf_launch_status();
}

template <typename A>
__global__ void moe_act_kernel(const A* __restrict__ gu, const float* __restrict__ route_w,
                               A* __restrict__ act, int T, int F, int E, int ff, int rw_cols,
                               int shared_gate) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * F) return;
  const int t = (int)(i / F), c = (int)(i % F);
  const int e = c < E * ff ? c / ff : E;
  const float wgt = (e < E || shared_gate) ? route_w[(size_t)t * rw_cols + e] : 1.f;
  float r = 0.f;
  if (wgt != 0.f) {
    const float g = bf_ld(gu + (size_t)t * 2 * F + c), u = bf_ld(gu + (size_t)t * 2 * F + F + c);
    r = g / (1.f + expf(-g)) * u * wgt;
  }
  bf_st(act + i, r);
}

// bfloat16 with F, ff and the experts' total a multiple of 8: eight columns a thread (they
// belong to one expert), 16-byte loads and stores.
__global__ void moe_act_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gu,
                                        const float* __restrict__ route_w,
                                        __nv_bfloat16* __restrict__ act, int T, int F, int E,
                                        int ff, int rw_cols, int shared_gate) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int F8 = F >> 3;
  if (i >= (long long)T * F8) return;
  const int t = (int)(i / F8), c = (int)(i % F8) << 3;
  const int e = c < E * ff ? c / ff : E;
  const float wgt = (e < E || shared_gate) ? route_w[(size_t)t * rw_cols + e] : 1.f;
  uint4 out = make_uint4(0u, 0u, 0u, 0u);
  if (wgt != 0.f) {
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * F + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * F + F + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      o2[j] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x * wgt,
                                    g.y / (1.f + expf(-g.y)) * u.y * wgt);
    }
  }
  *reinterpret_cast<uint4*>(act + (size_t)t * F + c) = out;
}

// rw_cols: the columns of a row of route_w; shared_gate: column E holds the shared expert's
// weight (else that expert's weight is one)
BF_EXPORT int bf_moe_act(const void* gu, const float* route_w, void* act, int T, int F, int E,
                         int ff, int rw_cols, int shared_gate, int act_dtype,
                         cudaStream_t stream) {
  if (T <= 0 || F <= 0) return 0;
  const long long n = (long long)T * F;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == BF_DTYPE_BF16 && F % 8 == 0 && ff % 8 == 0 &&
      (((uintptr_t)gu | (uintptr_t)act) & 15) == 0) {
    moe_act_bf16_vec_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, route_w, (__nv_bfloat16*)act, T, F, E, ff, rw_cols,
        shared_gate);
    return bf_launch_status();
  }
  if (act_dtype == BF_DTYPE_F32)
    moe_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, route_w, (float*)act, T,
                                                      F, E, ff, rw_cols, shared_gate);
  else
    moe_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, route_w, (__nv_bfloat16*)act, T, F, E, ff, rw_cols,
        shared_gate);
  return bf_launch_status();
}

// out[t, c] += h[t, c] * route_w[t, col]: the experts that return their input.
template <typename A>
__global__ void moe_identity_add_kernel(A* __restrict__ out, const A* __restrict__ h,
                                        long long stride, const float* __restrict__ route_w,
                                        int rw_cols, int col, int T, int width) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * width) return;
  const int t = (int)(i / width), c = (int)(i % width);
  const float wgt = route_w[(size_t)t * rw_cols + col];
  if (wgt != 0.f) bf_st(out + i, bf_ld(out + i) + wgt * bf_ld(h + (size_t)t * stride + c));
}

// bfloat16, a width that is a multiple of 8 and rows on 16-byte boundaries: eight columns a thread
__global__ void moe_identity_add_bf16_vec_kernel(__nv_bfloat16* __restrict__ out,
                                                 const __nv_bfloat16* __restrict__ h,
                                                 long long stride,
                                                 const float* __restrict__ route_w, int rw_cols,
                                                 int col, int T, int width) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int w8 = width >> 3;
  if (i >= (long long)T * w8) return;
  const int t = (int)(i / w8), c = (int)(i % w8) << 3;
  const float wgt = route_w[(size_t)t * rw_cols + col];
  if (wgt == 0.f) return;
  uint4 o4 = *reinterpret_cast<const uint4*>(out + (size_t)t * width + c);
  const uint4 h4 = *reinterpret_cast<const uint4*>(h + (size_t)t * stride + c);
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&h4);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = __bfloat1622float2(o2[j]), b = __bfloat1622float2(h2[j]);
    o2[j] = __floats2bfloat162_rn(a.x + wgt * b.x, a.y + wgt * b.y);
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * width + c) = o4;
}

BF_EXPORT int bf_moe_identity_add(void* out, const void* h, long long stride,
                                  const float* route_w, int rw_cols, int col, int T, int width,
                                  int act_dtype, cudaStream_t stream) {
  if (T <= 0 || width <= 0) return 0;
  const long long n = (long long)T * width;
  if (act_dtype == BF_DTYPE_BF16 && width % 8 == 0 && stride % 8 == 0 &&
      (((uintptr_t)out | (uintptr_t)h) & 15) == 0) {
    moe_identity_add_bf16_vec_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)h, stride, route_w, rw_cols, col, T, width);
    return bf_launch_status();
  }
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == BF_DTYPE_F32)
    moe_identity_add_kernel<float><<<blocks, 256, 0, stream>>>(
        (float*)out, (const float*)h, stride, route_w, rw_cols, col, T, width);
  else
    moe_identity_add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)h, stride, route_w, rw_cols, col, T, width);
  return bf_launch_status();
}

// ------------------------------------------------------------------ few tokens: chosen experts only
// A step of very few tokens (a request decoding alone) should not read the experts that no
// token chose.  moe_sparse_gate_up computes, per token and choice (the `top` chosen experts in
// the router's order, then the shared expert if there is one), the expert's activations
// times the token's weight for it, from the expert's rows of the stacked gate/up weight;
// moe_sparse_down multiplies them with the expert's columns of the stacked down weight and
// adds the choices up in that order.  One warp per output row, the token's input in shared
// memory as float, 16-byte pieces of the rows where the sizes allow.
//
// A choice at or beyond E is an expert that returns its input: it has no rows, its activations
// are zeros, and moe_sparse_down adds the input times the identity column of route_w
// (`id_col` >= 0) behind the shared expert.
//
// act: [T][top * ff + ff_sh] (choice k at k * ff, the shared expert behind them).
#define MS_WARPS 8
#define MS_ROWS 4           // rows a warp takes in turn

// Pieces of eight neighbouring values of a row as floats.
__device__ __forceinline__ void ms_ld8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ms_ld8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h2[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}

// A row of n values of the activation type into shared memory as floats, by the whole block,
// in pieces of eight where the row allows it.
template <typename A>
__device__ __forceinline__ void ms_stage(const A* __restrict__ src, float* __restrict__ dst,
                                         int n) {
  const int esz = (int)sizeof(A);
  if ((n & 7) == 0 && (((uintptr_t)src) % (8 * esz)) == 0) {
#pragma unroll 4
    for (int c = threadIdx.x * 8; c < n; c += blockDim.x * 8) {
      float v[8];
      ms_ld8(src + c, v);
      reinterpret_cast<float4*>(dst + c)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(dst + c)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) dst[c] = bf_ld(src + c);
  }
}

// NR rows at `w + r * row_stride` against the same x [n]: the rows' pieces of a trip are all
// fetched before any is used, so that NR round trips to memory overlap.  Every row's sum has
// the order of a plain strided walk followed by the warp's tree.
template <typename A, int NR>
__device__ __forceinline__ void ms_dots(const A* __restrict__ w, size_t row_stride, int rows,
                                        const float* __restrict__ x, int n, int lane, bool vec,
                                        float (&out)[NR]) {
  float a[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) a[r] = 0.f;
  if (vec) {
    for (int c = lane * 8; c < n; c += 256) {
      float p[NR][8];
#pragma unroll
      for (int r = 0; r < NR; ++r)
        if (r < rows) ms_ld8(w + (size_t)r * row_stride + c, p[r]);
      float q[8];
      ms_ld8(x + c, q);
#pragma unroll
      for (int r = 0; r < NR; ++r)
        if (r < rows) {
#pragma unroll
          for (int j = 0; j < 8; ++j) a[r] += p[r][j] * q[j];
        }
    }
  } else {
    for (int c = lane; c < n; c += 32)
#pragma unroll
      for (int r = 0; r < NR; ++r)
        if (r < rows) a[r] += bf_ld(w + (size_t)r * row_stride + c) * x[c];
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) out[r] = warp_sum(a[r]);
}

// grid (row tiles, choices, T)
template <typename A>
__global__ void moe_sparse_gate_up_kernel(const A* __restrict__ h, long long stride,
                                          const A* __restrict__ w_gu, int width, int F, int E,
                                          int ff, int ff_sh, int top,
                                          const int* __restrict__ top_ids,
                                          const float* __restrict__ top_w,
                                          const float* __restrict__ route_w, int rw_cols,
                                          int shared_gate, A* __restrict__ act) {
  extern __shared__ __align__(16) float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.z, k = blockIdx.y;
  const bool shared = k == top;
  const int n_rows = shared ? ff_sh : ff;
  const int row0 = (blockIdx.x * MS_WARPS + warp) * MS_ROWS;
  if (blockIdx.x * MS_WARPS * MS_ROWS >= n_rows) return;
  ms_stage<A>(h + (size_t)t * stride, sh, width);
  __syncthreads();
  const int e = shared ? E : top_ids[(size_t)t * top + k];
  const float wgt = shared ? (shared_gate ? route_w[(size_t)t * rw_cols + E] : 1.f)
                           : top_w[(size_t)t * top + k];
  const size_t base = shared ? (size_t)E * ff : (size_t)e * ff;      // the expert's first row
  const bool vec = (width % 8) == 0 && (((uintptr_t)w_gu) & 15) == 0;
  A* dst = act + (size_t)t * ((size_t)top * ff + ff_sh) + (shared ? (size_t)top * ff : (size_t)k * ff);
  const int rows = min(MS_ROWS, n_rows - row0);
  if (rows <= 0) return;
  if (!shared && e >= E) {                       // an expert that returns its input: no rows
    if (lane == 0)
      for (int r = 0; r < rows; ++r) bf_st(dst + row0 + r, 0.f);
    return;
  }
  float g[MS_ROWS], u[MS_ROWS];
  ms_dots<A, MS_ROWS>(w_gu + (base + row0) * width, (size_t)width, rows, sh, width, lane, vec, g);
  ms_dots<A, MS_ROWS>(w_gu + ((size_t)F + base + row0) * width, (size_t)width, rows, sh, width,
                      lane, vec, u);
  if (lane == 0)
    for (int r = 0; r < rows; ++r) bf_st(dst + row0 + r, g[r] / (1.f + expf(-g[r])) * u[r] * wgt);
}

// grid (row tiles, T)
template <typename A>
__global__ void moe_sparse_down_kernel(const A* __restrict__ act, const A* __restrict__ w_down,
                                       int width, int F, int E, int ff, int ff_sh, int top,
                                       const int* __restrict__ top_ids, A* __restrict__ out,
                                       const A* __restrict__ h, long long h_stride,
                                       const float* __restrict__ route_w, int rw_cols,
                                       int id_col) {
  extern __shared__ __align__(16) float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int n_act = top * ff + ff_sh;
  ms_stage<A>(act + (size_t)t * n_act, sh, n_act);
  __syncthreads();
  const int row0 = (blockIdx.x * MS_WARPS + warp) * MS_ROWS;
  const bool vec = (ff % 8) == 0 && (F % 8) == 0 && (((uintptr_t)w_down) & 15) == 0;
  const int rows = min(MS_ROWS, width - row0);
  if (rows <= 0) return;
  const A* wr = w_down + (size_t)row0 * F;
  float a[MS_ROWS], part[MS_ROWS];
#pragma unroll
  for (int r = 0; r < MS_ROWS; ++r) a[r] = 0.f;
  for (int k = 0; k < top; ++k) {
    if (top_ids[(size_t)t * top + k] >= E) continue;
    ms_dots<A, MS_ROWS>(wr + (size_t)top_ids[(size_t)t * top + k] * ff, (size_t)F, rows,
                        sh + (size_t)k * ff, ff, lane, vec, part);
#pragma unroll
    for (int r = 0; r < MS_ROWS; ++r) a[r] += part[r];
  }
  if (ff_sh) {
    ms_dots<A, MS_ROWS>(wr + (size_t)E * ff, (size_t)F, rows, sh + (size_t)top * ff, ff_sh, lane,
                        vec && (ff_sh % 8) == 0, part);
#pragma unroll
    for (int r = 0; r < MS_ROWS; ++r) a[r] += part[r];
  }
  if (lane == 0) {
    const float idw = id_col >= 0 ? route_w[(size_t)t * rw_cols + id_col] : 0.f;
    for (int r = 0; r < rows; ++r) {
      if (idw != 0.f) a[r] += idw * bf_ld(h + (size_t)t * h_stride + row0 + r);
      bf_st(out + (size_t)t * width + row0 + r, a[r]);
    }
  }
}

BF_EXPORT int bf_moe_sparse(const void* h, long long stride, const void* w_gu, const void* w_down,
                            const int* top_ids, const float* top_w, const float* route_w,
                            int rw_cols, void* act, void* out, int T, int width, int E, int ff,
                            int ff_sh, int top, int act_dtype, int shared_gate, int id_col,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  const int F = E * ff + ff_sh;
  const int choices = top + (ff_sh ? 1 : 0);
  const int n_act = top * ff + ff_sh;
  const int rows_max = ff > ff_sh ? ff : ff_sh;
  const int per_block = MS_WARPS * MS_ROWS;
  if ((size_t)width * 4 > 48 * 1024 || (size_t)n_act * 4 > 48 * 1024)
    return (int)cudaErrorInvalidValue;
  dim3 g1((rows_max + per_block - 1) / per_block, choices, T);
  dim3 g2((width + per_block - 1) / per_block, T);
  if (act_dtype == BF_DTYPE_F32) {
    moe_sparse_gate_up_kernel<float><<<g1, MS_WARPS * 32, (size_t)width * 4, stream>>>(
        (const float*)h, stride, (const float*)w_gu, width, F, E, ff, ff_sh, top, top_ids, top_w,
        route_w, rw_cols, shared_gate, (float*)act);
    moe_sparse_down_kernel<float><<<g2, MS_WARPS * 32, (size_t)n_act * 4, stream>>>(
        (const float*)act, (const float*)w_down, width, F, E, ff, ff_sh, top, top_ids,
        (float*)out, (const float*)h, stride, route_w, rw_cols, id_col);
  } else {
    moe_sparse_gate_up_kernel<__nv_bfloat16><<<g1, MS_WARPS * 32, (size_t)width * 4, stream>>>(
        (const __nv_bfloat16*)h, stride, (const __nv_bfloat16*)w_gu, width, F, E, ff, ff_sh, top,
        top_ids, top_w, route_w, rw_cols, shared_gate, (__nv_bfloat16*)act);
    moe_sparse_down_kernel<__nv_bfloat16><<<g2, MS_WARPS * 32, (size_t)n_act * 4, stream>>>(
        (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, width, F, E, ff, ff_sh, top,
        top_ids, (__nv_bfloat16*)out, (const __nv_bfloat16*)h, stride, route_w, rw_cols, id_col);
  }
  return bf_launch_status();
}
