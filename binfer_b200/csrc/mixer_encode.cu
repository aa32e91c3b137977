// Small kernels between a mixer's stacked projection and its attention or recurrence, and
// behind it: everything here is float arithmetic on rows of the activation type.
//
//   section_rms      rsqrt(mean(x^2) + eps) of two column sections of every row: the factor
//                    of an RMS norm over a whole projection (all heads at once)
//   section_norm     an RMS norm with a weight over one column section of every row, into a
//                    buffer of its own (a latent between two products)
//   latent_encode    attention over a cached latent: the latent's norm, the rotation of the
//                    shared key part and of every query head's rotated part, the latent and
//                    the key part into the cache pages
//   delta_encode     the gated delta rule's inputs: convolution per channel, silu, unit
//                    vectors, and the two gates per head
//   gated_norm_out   a recurrence's raw output divided by its root mean square (per head or
//                    over all heads), times a weight, times silu or sigmoid of a gate
//   head_gate_mul    every head's output times the sigmoid of one number per head
//   stream_inject    the residual stream plus its pending sublayer output, the embedding
//                    output again and one row of a table (the start of a pass over layers)
#include "common.cuh"

#define ME_MAX_TAPS 16

// A pair of one rotation: `interleaved` (2m, 2m + 1), else (m, m + rot_half).
__device__ __forceinline__ void me_pair(int m, int rot_half, int interleaved, int* a, int* b) {
  if (interleaved) { *a = 2 * m; *b = 2 * m + 1; }
  else { *a = m; *b = m + rot_half; }
}

// -------------------------------------------------------------------- section_rms
template <typename A>
__global__ void section_rms_kernel(const A* __restrict__ x, long long stride, int off0, int n0,
                                   int off1, int n1, float eps, float* __restrict__ out) {
  __shared__ float scratch[33];
  const int t = blockIdx.x, s = blockIdx.y;
  const int off = s ? off1 : off0, n = s ? n1 : n0;
  const A* row = x + (size_t)t * stride + off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = bf_ld(row + i);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) out[(size_t)t * 2 + s] = n > 0 ? rsqrtf(ss / (float)n + eps) : 1.f;
}

BF_EXPORT int bf_section_rms(const void* x, long long stride, int off0, int n0, int off1, int n1,
                             float eps, float* out, int T, int act_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = (n0 > 2048 || n1 > 2048) ? 256 : 128;
  dim3 grid(T, 2);
  if (act_dtype == BF_DTYPE_F32)
    section_rms_kernel<float><<<grid, threads, 0, stream>>>((const float*)x, stride, off0, n0,
                                                           off1, n1, eps, out);
  else
    section_rms_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, stride, off0, n0, off1, n1, eps, out);
  return bf_launch_status();
}

// ------------------------------------------------------------------- section_norm
// out[t, i] = x[t, off + i] * rsqrt(mean_i x[t, off + i]^2 + eps) * w[i], one block per row.
template <typename A>
__global__ void section_norm_kernel(const A* __restrict__ x, long long stride, long long off,
                                    int n, const float* __restrict__ w, float eps,
                                    A* __restrict__ out, long long out_stride) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const A* row = x + (size_t)t * stride + off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = bf_ld(row + i);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float f = rsqrtf(ss / (float)n + eps);
  A* o = out + (size_t)t * out_stride;
  for (int i = threadIdx.x; i < n; i += blockDim.x) bf_st(o + i, bf_ld(row + i) * f * w[i]);
}

BF_EXPORT int bf_section_norm(const void* x, long long stride, long long off, int n,
                              const float* w, float eps, void* out, long long out_stride, int T,
                              int act_dtype, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  const int threads = n > 2048 ? 256 : 128;
  if (act_dtype == BF_DTYPE_F32)
    section_norm_kernel<float><<<T, threads, 0, stream>>>((const float*)x, stride, off, n, w, eps,
                                                         (float*)out, out_stride);
  else
    section_norm_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
        (const __nv_bfloat16*)x, stride, off, n, w, eps, (__nv_bfloat16*)out, out_stride);
  return bf_launch_status();
}

// ------------------------------------------------------------------ latent_encode
// A row of `q` holds [H heads of (d plain | dr rotated)] (rows `q_stride` apart: a column block
// of `proj` or a buffer of its own) and a row of `proj`, from kv_off,
// [rank numbers that become the latent | dr numbers that become the shared key part].
// The cache row of a token is [latent (normed, weighted) | key part (rotated)], one "head" of
// rank + dr numbers.  q_abs [T, H, rank + dr] gets only every head's rotated part, at
// [rank, rank + dr); the plain part is turned into latent coordinates by a product elsewhere.
// One block per token.
template <typename A>
__global__ void latent_encode_kernel(
    const A* __restrict__ proj, long long stride, const A* __restrict__ q, long long q_stride,
    long long kv_off,
    const float* __restrict__ norm_w, float eps, const float* __restrict__ inv_freq,
    int rot_half, int interleaved, float rot_mag, const int* __restrict__ positions,
    const int* __restrict__ slots, A* __restrict__ q_abs, A* __restrict__ cache, int H, int d,
    int dr, int rank, int page_size, long long num_slots, int* __restrict__ err) {
  extern __shared__ float sh[];
  float* cs = sh;                   // rot_half cosines, rot_half sines
  float* sn = sh + rot_half;
  float* scratch = sh + 2 * rot_half;
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  for (int m = threadIdx.x; m < rot_half; m += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[m], &s, &c);
    cs[m] = c * rot_mag;
    sn[m] = s * rot_mag;
  }
  const A* row = proj + (size_t)t * stride;
  const A* kv = row + kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = bf_ld(kv + i);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);      // (also orders the table's writes before its readers)
  const float f = rsqrtf(ss / (float)rank + eps);
  const int W = rank + dr;
  if (cache) {
    const long long s = slots[t];
    if (s < 0 || s >= num_slots) {
      if (threadIdx.x == 0) atomicOr(err, BF_ERR_SLOT);
    } else {
      A* o = cache + s * W;         // one head per page row: slot = page * page_size + offset
      for (int i = threadIdx.x; i < rank; i += blockDim.x)
        bf_st(o + i, bf_ld(kv + i) * f * norm_w[i]);
      const A* kr = kv + rank;
      for (int m = threadIdx.x; m < rot_half; m += blockDim.x) {
        int a, b;
        me_pair(m, rot_half, interleaved, &a, &b);
        const float u = bf_ld(kr + a), v = bf_ld(kr + b);
        bf_st(o + rank + a, u * cs[m] - v * sn[m]);
        bf_st(o + rank + b, v * cs[m] + u * sn[m]);
      }
      for (int i = 2 * rot_half + threadIdx.x; i < dr; i += blockDim.x)
        bf_st(o + rank + i, bf_ld(kr + i));
    }
  }
  for (int idx = threadIdx.x; idx < H * rot_half; idx += blockDim.x) {
    const int h = idx / rot_half, m = idx - h * rot_half;
    const A* qr = q + (size_t)t * q_stride + (size_t)h * (d + dr) + d;
    A* o = q_abs + ((size_t)t * H + h) * W + rank;
    int a, b;
    me_pair(m, rot_half, interleaved, &a, &b);
    const float u = bf_ld(qr + a), v = bf_ld(qr + b);
    bf_st(o + a, u * cs[m] - v * sn[m]);
    bf_st(o + b, v * cs[m] + u * sn[m]);
  }
  const int rest = dr - 2 * rot_half;
  for (int idx = threadIdx.x; idx < H * rest; idx += blockDim.x) {
    const int h = idx / rest, i = 2 * rot_half + idx % rest;
    bf_st(q_abs + ((size_t)t * H + h) * W + rank + i,
          bf_ld(q + (size_t)t * q_stride + (size_t)h * (d + dr) + d + i));
  }
}

BF_EXPORT int bf_latent_encode(const void* proj, long long stride, const void* q,
                               long long q_stride, long long kv_off, const float* norm_w,
                               float eps,
                               const float* inv_freq, int rot_half, int interleaved,
                               float rot_mag, const int* positions, const int* slots, void* q_abs,
                               void* cache, int T, int H, int d, int dr, int rank, int page_size,
                               long long num_slots, int act_dtype, int* err,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (2 * rot_half > dr || rank <= 0) return (int)cudaErrorInvalidValue;
  const int threads = 128;
  const size_t smem = (size_t)(2 * rot_half + 33) * sizeof(float);
  if (act_dtype == BF_DTYPE_F32)
    latent_encode_kernel<float><<<T, threads, smem, stream>>>(
        (const float*)proj, stride, (const float*)q, q_stride, kv_off, norm_w, eps, inv_freq,
        rot_half, interleaved, rot_mag, positions, slots, (float*)q_abs, (float*)cache, H, d, dr,
        rank, page_size, num_slots, err);
  else
    latent_encode_kernel<__nv_bfloat16><<<T, threads, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, (const __nv_bfloat16*)q, q_stride, kv_off, norm_w,
        eps, inv_freq, rot_half, interleaved, rot_mag, positions, slots, (__nv_bfloat16*)q_abs,
        (__nv_bfloat16*)cache, H, d, dr, rank, page_size, num_slots, err);
  return bf_launch_status();
}

// ------------------------------------------------------------------- delta_encode
// A row of `proj` holds, from column 0, [q: G heads of dk | k: G heads of dk | v: H heads of
// dv] (the channels that pass the convolution, C of them) and, further on, one number per
// value head at b_off (beta's logit) and at a_off (the decay's).  Per channel
//   y_t[c] = silu(sum_j w[c, j] u_{t - taps + 1 + j}[c])
// with the request's state (`state[slot]` = [taps-1, C], oldest first) behind the step's
// first row; each q and k head then becomes y / sqrt(sum y^2 + unit_eps), q times q_scale.
// Results, float: qkv [T, C] and gates [T, 2, H] = (beta = sigmoid(.), g = exp(-exp(A_log)
// softplus(. + dt_bias))).  One warp per (token, head); one more per token for the gates.
__device__ __forceinline__ float me_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename A>
__global__ void delta_encode_kernel(
    const A* __restrict__ proj, long long stride, const float* __restrict__ conv_w, int taps,
    const float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
    int n_state_slots, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
    long long b_off, long long a_off, const float* __restrict__ A_log,
    const float* __restrict__ dt_bias, float* __restrict__ qkv, float* __restrict__ gates, int T,
    int H, int G, int dk, int dv, float unit_eps, float q_scale, int* __restrict__ err) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_token = 2 * G + H + 1;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)T * per_token) return;
  const int t = (int)(item / per_token), hs = (int)(item % per_token);
  const A* row = proj + (size_t)t * stride;
  if (hs == 2 * G + H) {                       // the token's gates
    for (int h = lane; h < H; h += 32) {
      const float zb = bf_ld(row + b_off + h), za = bf_ld(row + a_off + h);
      gates[((size_t)t * 2) * H + h] = 1.f / (1.f + expf(-zb));
      gates[((size_t)t * 2 + 1) * H + h] = expf(-expf(A_log[h]) * me_softplus(za + dt_bias[h]));
    }
    return;
  }
  const int C = 2 * G * dk + H * dv;
  int kind, d, c0;                             // 0 q, 1 k, 2 v; first channel of the head
  if (hs < G) { kind = 0; d = dk; c0 = hs * dk; }
  else if (hs < 2 * G) { kind = 1; d = dk; c0 = G * dk + (hs - G) * dk; }
  else { kind = 2; d = dv; c0 = 2 * G * dk + (hs - 2 * G) * dv; }
  const int b = seq_of_token[t];
  const int local = t - q_start[b];
  int slot = 0;
  if (taps > 1) {
    slot = state_slots[b];
    if (slot < 0 || slot >= n_state_slots) { atomicOr(err, BF_ERR_SLOT); slot = 0; }
  }
  const float* st = state + (size_t)slot * state_stride;
  float* o = qkv + (size_t)t * C + c0;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const int c = c0 + i;
    float y;
    if (taps >= 1) {
      y = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int src = local - (taps - 1) + j;
        const float u = src >= 0 ? bf_ld(proj + (size_t)(t - (taps - 1) + j) * stride + c)
                                 : st[(size_t)(taps - 1 + src) * C + c];
        y += conv_w[(size_t)c * taps + j] * u;
      }
    } else {
      y = bf_ld(row + c);
    }
    y = y / (1.f + expf(-y));
    ss += y * y;
    o[i] = y;
  }
  if (kind == 2) return;
  const float f = rsqrtf(warp_sum(ss) + unit_eps) * (kind == 0 ? q_scale : 1.f);
  __syncwarp();
  for (int i = lane; i < d; i += 32) o[i] *= f;
}

BF_EXPORT int bf_delta_encode(const void* proj, long long stride, const float* conv_w, int taps,
                              const float* state, long long state_stride, const int* state_slots,
                              int n_state_slots, const int* seq_of_token, const int* q_start,
                              long long b_off, long long a_off, const float* A_log,
                              const float* dt_bias, float* qkv, float* gates, int T, int H, int G,
                              int dk, int dv, float unit_eps, float q_scale, int act_dtype,
                              int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps > ME_MAX_TAPS || (taps > 1 && !state) || G <= 0 || H % G)
    return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const long long items = (long long)T * (2 * G + H + 1);
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (act_dtype == BF_DTYPE_F32)
    delta_encode_kernel<float><<<blocks, warps * 32, 0, stream>>>(
        (const float*)proj, stride, conv_w, taps, state, state_stride, state_slots,
        n_state_slots, seq_of_token, q_start, b_off, a_off, A_log, dt_bias, qkv, gates, T, H, G,
        dk, dv, unit_eps, q_scale, err);
  else
    delta_encode_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
        (const __nv_bfloat16*)proj, stride, conv_w, taps, state, state_stride, state_slots,
        n_state_slots, seq_of_token, q_start, b_off, a_off, A_log, dt_bias, qkv, gates, T, H, G,
        dk, dv, unit_eps, q_scale, err);
  return bf_launch_status();
}

// ----------------------------------------------------------------- gated_norm_out
// out[t, h, i] = o[t, h, i] * f * w * act(gate[t, h, i]) * out_scale with
//   f = rsqrt(mean of o^2 over the head + eps), or over all heads of the token (over_all),
//   w = 1 (w_mode 0), weight[i] (1: one weight of dv numbers for every head) or
//       weight[h dv + i] (2),
//   act = silu (gate_act 0) or the sigmoid (1).
// One block per token, a warp per head in turn.
template <typename A>
__global__ void gated_norm_out_kernel(const float* __restrict__ o_raw,
                                      const A* __restrict__ proj, long long stride,
                                      long long g_off, const float* __restrict__ weight,
                                      int w_mode, int over_all, int gate_act,
                                      A* __restrict__ out, long long out_stride, int H, int dv,
                                      float eps, float out_scale) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const float* o = o_raw + (size_t)t * H * dv;
  float f_all = 0.f;
  if (over_all) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < H * dv; i += blockDim.x) ss += o[i] * o[i];
    ss = block_sum(ss, scratch);
    f_all = rsqrtf(ss / (float)(H * dv) + eps);
  }
  const A* g = proj + (size_t)t * stride + g_off;
  A* dst = out + (size_t)t * out_stride;
  for (int h = warp; h < H; h += warps) {
    float f = f_all;
    if (!over_all) {
      float ss = 0.f;
      for (int i = lane; i < dv; i += 32) ss += o[h * dv + i] * o[h * dv + i];
      f = rsqrtf(warp_sum(ss) / (float)dv + eps);
    }
    f *= out_scale;
    for (int i = lane; i < dv; i += 32) {
      const int c = h * dv + i;
      const float z = bf_ld(g + c);
      const float sg = 1.f / (1.f + expf(-z));
      const float w = w_mode == 0 ? 1.f : weight[w_mode == 1 ? i : c];
      bf_st(dst + c, o[c] * f * w * (gate_act ? sg : z * sg));
    }
  }
}

BF_EXPORT int bf_gated_norm_out(const float* o_raw, const void* proj, long long stride,
                                long long g_off, const float* weight, int w_mode, int over_all,
                                int gate_act, void* out, long long out_stride, int T, int H,
                                int dv, float eps, float out_scale, int act_dtype,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (w_mode && !weight) return (int)cudaErrorInvalidValue;
  const int threads = H >= 8 ? 256 : 128;
  if (act_dtype == BF_DTYPE_F32)
    gated_norm_out_kernel<float><<<T, threads, 0, stream>>>(
        o_raw, (const float*)proj, stride, g_off, weight, w_mode, over_all, gate_act,
        (float*)out, out_stride, H, dv, eps, out_scale);
  else
    gated_norm_out_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
        o_raw, (const __nv_bfloat16*)proj, stride, g_off, weight, w_mode, over_all, gate_act,
        (__nv_bfloat16*)out, out_stride, H, dv, eps, out_scale);
  return bf_launch_status();
}

// ------------------------------------------------------------------ head_gate_mul
// x[t, h, :] *= sigmoid(gate[t, h]); gate is a column block of a wider row.
template <typename A>
__global__ void head_gate_mul_kernel(A* __restrict__ x, const A* __restrict__ gate,
                                     long long gate_stride, long long n, int H, int dv) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long th = i / dv;
  const long long t = th / H;
  const int h = (int)(th - t * H);
  const float z = bf_ld(gate + t * gate_stride + h);
  bf_st(x + i, bf_ld(x + i) / (1.f + expf(-z)));
}

BF_EXPORT int bf_head_gate_mul(void* x, const void* gate, long long gate_stride, int T, int H,
                               int dv, int act_dtype, cudaStream_t stream) {
  const long long n = (long long)T * H * dv;
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == BF_DTYPE_F32)
    head_gate_mul_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, (const float*)gate,
                                                           gate_stride, n, H, dv);
  else
    head_gate_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        (__nv_bfloat16*)x, (const __nv_bfloat16*)gate, gate_stride, n, H, dv);
  return bf_launch_status();
}

// ------------------------------------------------------------------ stream_inject
// resid[t] += delta[t] (if any) + table[ids[t]] * scale (if a table is given) + vec (if any):
// what is added to the stream where a pass over a run of layers starts.
template <typename A, typename W>
__global__ void stream_inject_kernel(float* __restrict__ resid, const A* __restrict__ delta,
                                     const W* __restrict__ table, const int* __restrict__ ids,
                                     int vocab, float scale, const float* __restrict__ vec,
                                     int width, int* __restrict__ err) {
  const int t = blockIdx.x;
  float* x = resid + (size_t)t * width;
  const W* e = nullptr;
  if (table) {
    const int id = ids[t];
    if (id < 0 || id >= vocab) {
      if (threadIdx.x == 0) atomicOr(err, BF_ERR_TOKEN_ID);
    } else {
      e = table + (size_t)id * width;
    }
  }
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float v = x[c];
    if (delta) v += bf_ld(delta + (size_t)t * width + c);
    if (e) v += bf_ld(e + c) * scale;
    if (vec) v += vec[c];
    x[c] = v;
  }
}

BF_EXPORT int bf_stream_inject(float* resid, const void* delta, int delta_dtype,
                               const void* table, int table_dtype, const int* ids, int vocab,
                               float scale, const float* vec, int T, int width, int* err,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
#define SI_GO(AT, WT)                                                                         \
  stream_inject_kernel<AT, WT><<<T, threads, 0, stream>>>(resid, (const AT*)delta,            \
                                                          (const WT*)table, ids, vocab, scale, \
                                                          vec, width, err)
  if (delta_dtype == BF_DTYPE_F32) {
    if (table_dtype == BF_DTYPE_F32) SI_GO(float, float); else SI_GO(float, __nv_bfloat16);
  } else {
    if (table_dtype == BF_DTYPE_F32) SI_GO(__nv_bfloat16, float);
    else SI_GO(__nv_bfloat16, __nv_bfloat16);
  }
#undef SI_GO
  return bf_launch_status();
}
