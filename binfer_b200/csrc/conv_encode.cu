// What lies between the q/k/v projection and the attention of a mixer whose projections pass
// a short causal convolution over time: convolution per channel, rotation of q and k, a
// weightless RMS norm of each q and k head after the rotation, q to its buffer, k and v into
// the cache pages.  Every step is optional (taps 0: no convolution, 1: a factor per channel
// and no state; rot_half 0: no rotation; unit_norm 0: no norm).  Between the convolution and
// the rotation q and k may be multiplied by a factor per token (`pre_factor` [T][2]: q, k) and a
// weight per channel (`pre_weight`): an RMS norm over a whole projection, whose factor a kernel
// in front has taken.  The cosines and sines are multiplied by `rot_mag`.  After the norm of the
// heads q and k may be multiplied by a weight per size of a head that the heads share (`head_w`
// [2][dk]: q's, then k's), and each q head by a number of its own (`q_head_scale` [nh]: a factor
// on the head's scores).
//
//   y_t[c] = sum_j w[c, j] * u_{t - taps + 1 + j}[c],   j = 0 .. taps-1
//
// with zeros before the request's first token.  The projected values of a request's last
// taps-1 tokens are its state (float, `state[slot]` = [taps-1, channels], oldest first), so
// a prompt may be cut anywhere: a token whose taps reach behind the step's first row reads
// them there.  bf_conv_state_shift, launched after the encode kernel, moves the step's last
// rows into the state.
//
// One warp per (token, head); heads are counted q heads, then k heads, then v heads.  The
// cosines and sines of a token's angles are taken once for all its heads, by a small kernel
// in front.  All
// arithmetic is float; only the projection's values and the stored results have the
// activation type.
#include "common.cuh"

#define CE_MAX_TAPS 16

// cos and sin of position x frequency for every token of the step, once, for all heads:
// table [T][rot_half] of (cos, sin).
__global__ void rope_table_kernel(const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int T, int rot_half,
                                  float rot_mag, float2* __restrict__ table) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * rot_half) return;
  const int t = i / rot_half, m = i - t * rot_half;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[m], &sn, &cs);
  table[i] = make_float2(cs * rot_mag, sn * rot_mag);
}

// two neighbouring values of the activation type
__device__ __forceinline__ float2 ce_ld2(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
__device__ __forceinline__ float2 ce_ld2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void ce_st2(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
__device__ __forceinline__ void ce_st2(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename A>
__global__ void conv_encode_kernel(
    const A* __restrict__ proj, long long stride, const float* __restrict__ conv_w, int taps,
    const float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
    int n_state_slots, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
    const float2* __restrict__ rope, int rot_half, const int* __restrict__ slots,
    A* __restrict__ q_out, long long q_stride, A* __restrict__ k_cache, A* __restrict__ v_cache,
    int T, int nh, int nkv, int dk, int dv, int page_size, long long num_slots, int unit_norm,
    float eps, int vec2, int hpw, int* __restrict__ err, const float* __restrict__ pre_factor,
    const float* __restrict__ pre_weight, const float* __restrict__ head_w,
    const float* __restrict__ q_head_scale) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = nh + 2 * nkv;
  // a warp takes `hpw` heads of one token in turn: one round of lookups for all of them
  const int groups = (heads_total + hpw - 1) / hpw;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)T * groups) return;
  const int t = (int)(item / groups), hs0 = (int)(item % groups) * hpw;
  const int C = nh * dk + nkv * dk + nkv * dv;
  // per warp: the head after the convolution, and after the rotation
  const int dm = max(dk, dv);
  float* buf = sh + (size_t)warp * 2 * dm;
  float* res = buf + dm;

  const int b = seq_of_token[t];
  const int local = t - q_start[b];            // index of the token inside the step's portion
  int slot = 0;
  if (taps > 1) {
    slot = state_slots[b];
    if (slot < 0 || slot >= n_state_slots) { atomicOr(err, BF_ERR_SLOT); slot = 0; }
  }
  const float* st = state + (size_t)slot * state_stride;
  const long long cache_slot = k_cache ? slots[t] : 0;
  for (int hs = hs0; hs < min(hs0 + hpw, heads_total); ++hs) {
  __syncwarp();                                // the last head's readers of buf and res are done
  int kind, head, d, c0;                       // 0 q, 1 k, 2 v; first channel of the head
  if (hs < nh) { kind = 0; head = hs; d = dk; c0 = head * dk; }
  else if (hs < nh + nkv) { kind = 1; head = hs - nh; d = dk; c0 = nh * dk + head * dk; }
  else { kind = 2; head = hs - nh - nkv; d = dv; c0 = (nh + nkv) * dk + head * dv; }
  if (vec2) {                                  // two neighbouring channels a lane and trip
    for (int i = 2 * lane; i < d; i += 64) {
      const int c = c0 + i;
      float2 y;
      if (conv_w) {
        y = make_float2(0.f, 0.f);
        for (int j = 0; j < taps; ++j) {
          const int src = local - (taps - 1) + j;     // index inside the portion
          const float2 u = src >= 0 ? ce_ld2(proj + (size_t)(t - (taps - 1) + j) * stride + c)
                                    : ce_ld2(st + (size_t)(taps - 1 + src) * C + c);
          y.x += conv_w[(size_t)c * taps + j] * u.x;
          y.y += conv_w[(size_t)(c + 1) * taps + j] * u.y;
        }
      } else {
        y = ce_ld2(proj + (size_t)t * stride + c);
      }
      buf[i] = y.x;
      buf[i + 1] = y.y;
    }
  } else {
    for (int i = lane; i < d; i += 32) {
      const int c = c0 + i;
      float y;
      if (conv_w) {
        y = 0.f;
        for (int j = 0; j < taps; ++j) {
          const int src = local - (taps - 1) + j;     // index inside the portion
          float u;
          if (src >= 0) u = bf_ld(proj + (size_t)(t - (taps - 1) + j) * stride + c);
          else u = st[(size_t)(taps - 1 + src) * C + c];
          y += conv_w[(size_t)c * taps + j] * u;
        }
      } else {
        y = bf_ld(proj + (size_t)t * stride + c);
      }
      buf[i] = y;
    }
  }
  __syncwarp();
  if (pre_factor && kind < 2) {                // the norm over the whole projection
    const float f = pre_factor[(size_t)t * 2 + kind];
    for (int i = lane; i < d; i += 32) buf[i] *= f * pre_weight[c0 + i];
    __syncwarp();
  }
  float ss = 0.f;
  const bool turn = kind < 2 && rot_half > 0;
  const float2* cs_sn = rope + (size_t)t * rot_half;
  for (int i = lane; i < d; i += 32) {
    float y = buf[i];
    if (turn && i < 2 * rot_half) {
      const int m = i < rot_half ? i : i - rot_half;
      const float cs = cs_sn[m].x, sn = cs_sn[m].y;
      const float other = i < rot_half ? buf[i + rot_half] : buf[i - rot_half];
      y = i < rot_half ? y * cs - other * sn : y * cs + other * sn;
    }
    ss += y * y;
    res[i] = y;
  }
  __syncwarp();
  float f = 1.f;
  if (kind < 2 && unit_norm) f = rsqrtf(warp_sum(ss) / (float)d + eps);
  if (kind < 2 && head_w) {                    // the weight behind the heads' norm
    for (int i = lane; i < d; i += 32) res[i] *= head_w[kind * dk + i];
    __syncwarp();
  }
  if (kind == 0 && q_head_scale) f *= q_head_scale[head];
  if (kind == 0) {
    A* o = q_out + (size_t)t * q_stride + (size_t)head * dk;
    if (vec2 && (q_stride & 1) == 0)
      for (int i = 2 * lane; i < d; i += 64) ce_st2(o + i, res[i] * f, res[i + 1] * f);
    else
      for (int i = lane; i < d; i += 32) bf_st(o + i, res[i] * f);
    continue;
  }
  if (!k_cache) continue;
  const long long s = cache_slot;
  if (s < 0 || s >= num_slots) { if (lane == 0) atomicOr(err, BF_ERR_SLOT); continue; }
  const long long page = s / page_size, off = s % page_size;
  A* o = (kind == 1 ? k_cache : v_cache) + ((page * nkv + head) * page_size + off) * d;
  if (vec2)
    for (int i = 2 * lane; i < d; i += 64) ce_st2(o + i, res[i] * f, res[i + 1] * f);
  else
    for (int i = lane; i < d; i += 32) bf_st(o + i, res[i] * f);
  }
}

BF_EXPORT int bf_conv_encode(
    const void* proj, long long stride, const float* conv_w, int taps, const float* state,
    long long state_stride, const int* state_slots, int n_state_slots, const int* seq_of_token,
    const int* q_start, const float* inv_freq, int rot_half, const int* positions,
    const int* slots, void* q_out, long long q_stride, void* k_cache, void* v_cache, int T,
    int nh, int nkv, int dk, int dv, int page_size, long long num_slots, int unit_norm, float eps,
    int act_dtype, float* rope_table, int* err, const float* pre_factor,
    const float* pre_weight, float rot_mag, const float* head_w, const float* q_head_scale,
    cudaStream_t stream) {
  // rope_table: scratch, float [T][rot_half][2] (unused without a rotation)
  if (T <= 0) return 0;
  if (taps > CE_MAX_TAPS || (taps > 1 && !state)) return (int)cudaErrorInvalidValue;
  if (taps < 1) conv_w = nullptr;              // (one tap: a factor per channel, no state)
  if (!pre_factor || !pre_weight) pre_factor = pre_weight = nullptr;
  if (rot_half > 0) {
    if (!rope_table) return (int)cudaErrorInvalidValue;
    const int n = T * rot_half;
    rope_table_kernel<<<(n + 127) / 128, 128, 0, stream>>>(positions, inv_freq, T, rot_half,
                                                          rot_mag, (float2*)rope_table);
    const int e = bf_launch_status();
    if (e) return e;
  }
  // pairs of channels where every row and head starts at an even element and address
  const int esz = act_dtype == BF_DTYPE_F32 ? 4 : 2;
  const int vec2 = (dk % 2 == 0 && dv % 2 == 0 && stride % 2 == 0 && state_stride % 2 == 0 &&
                    ((uintptr_t)proj % (2 * esz)) == 0 && ((uintptr_t)q_out % (2 * esz)) == 0 &&
                    ((uintptr_t)k_cache % (2 * esz)) == 0 && ((uintptr_t)v_cache % (2 * esz)) == 0 &&
                    ((uintptr_t)state % 8) == 0) ? 1 : 0;
  const int warps = 4;
  // many tokens: a warp walks four heads of its token (one round of lookups), else one
  const int hpw = (long long)T * (nh + 2 * nkv) >= 16 * 148 * 16 ? 4 : 1;
  const long long items = (long long)T * ((nh + 2 * nkv + hpw - 1) / hpw);
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  const int dm = dk > dv ? dk : dv;
  const size_t smem = (size_t)2 * warps * dm * sizeof(float);
  if (act_dtype == BF_DTYPE_F32)
    conv_encode_kernel<float><<<blocks, warps * 32, smem, stream>>>(
        (const float*)proj, stride, conv_w, taps, state, state_stride, state_slots, n_state_slots,
        seq_of_token, q_start, (const float2*)rope_table, rot_half, slots, (float*)q_out,
        q_stride, (float*)k_cache, (float*)v_cache, T, nh, nkv, dk, dv, page_size, num_slots,
        unit_norm, eps, vec2, hpw, err, pre_factor, pre_weight, head_w, q_head_scale);
  else
    conv_encode_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, conv_w, taps, state, state_stride, state_slots,
        n_state_slots, seq_of_token, q_start, (const float2*)rope_table, rot_half, slots,
        (__nv_bfloat16*)q_out, q_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T, nh,
        nkv, dk, dv, page_size, num_slots, unit_norm, eps, vec2, hpw, err, pre_factor,
        pre_weight, head_w, q_head_scale);
  return bf_launch_status();
}

// The state after a step: the projected values of the request's last taps-1 tokens, oldest
// first.  A request that brought n < taps-1 tokens keeps its newest taps-1-n old rows.  One
// thread per (request, channel) reads every old row it needs before it writes any.
template <typename A>
__global__ void conv_state_shift_kernel(const A* __restrict__ proj, long long stride,
                                        float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ state_slots, int n_state_slots,
                                        const int* __restrict__ q_start, int B, int C, int taps) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || b >= B) return;
  const int slot = state_slots[b];
  if (slot < 0 || slot >= n_state_slots) return;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  float* st = state + (size_t)slot * state_stride;
  float v[CE_MAX_TAPS];
  for (int s = 0; s < taps - 1; ++s) {
    const int src = n - (taps - 1) + s;
    v[s] = src >= 0 ? bf_ld(proj + (size_t)(t0 + src) * stride + c)
                    : st[(size_t)(taps - 1 + src) * C + c];
  }
  for (int s = 0; s < taps - 1; ++s) st[(size_t)s * C + c] = v[s];
}

BF_EXPORT int bf_conv_state_shift(const void* proj, long long stride, float* state,
                                  long long state_stride, const int* state_slots,
                                  int n_state_slots, const int* q_start, int B, int C, int taps,
                                  int act_dtype, cudaStream_t stream) {
  if (B <= 0 || taps <= 1) return 0;
  if (taps > CE_MAX_TAPS) return (int)cudaErrorInvalidValue;
  dim3 grid((C + 127) / 128, B);
  if (act_dtype == BF_DTYPE_F32)
    conv_state_shift_kernel<float><<<grid, 128, 0, stream>>>(
        (const float*)proj, stride, state, state_stride, state_slots, n_state_slots, q_start, B,
        C, taps);
  else
    conv_state_shift_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        (const __nv_bfloat16*)proj, stride, state, state_stride, state_slots, n_state_slots,
        q_start, B, C, taps);
  return bf_launch_status();
}
