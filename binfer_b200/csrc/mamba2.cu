// A selective state space layer with a scalar decay per head and token (Mamba-2), around its
// recurrence, which the linear scan of retention.cu runs (bf_linear_scan: q = C, k = B,
// v = dt x, a decay per token and head):
//
//   S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T      y_t = S_t^T C_t + D_h x_t
//
//   mamba2_encode   a row of `proj` holds [z: inner | x: inner | B: G N | C: G N | dt: H].  x, B
//                   and C (the channels from `xbc_off`) pass a causal convolution per channel
//                   with a bias and silu; the request's state (`state[slot]` = [taps-1, channels]
//                   of projected values, oldest first) lies behind the step's first row.  dt
//                   becomes softplus(dt + dt_bias_h).  Results, all float: qk [T][2][G][N] (C,
//                   then B), vf [T][H][P] = dt x, skip [T][H][P] = D_h x, decay [T][H].
//                   One warp per (token, head of x or group of B or of C).
//   gate_norm_out   y = (o_raw + skip) * silu(z), then an RMS norm in `parts` equal parts of
//                   the row (each by its own root mean square), times a weight per column.
//                   One block per (token, part).
//
// All arithmetic is float; only the projection's values and the result have the activation
// type.
#include "common.cuh"

#define M2_MAX_TAPS 16

__device__ __forceinline__ float m2_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename A>
__global__ void mamba2_encode_kernel(
    const A* __restrict__ proj, long long stride, long long xbc_off, long long dt_off,
    const float* __restrict__ conv_w, const float* __restrict__ conv_b, int taps,
    const float* __restrict__ state, long long state_stride, const int* __restrict__ state_slots,
    int n_state_slots, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
    const float* __restrict__ A_log, const float* __restrict__ dt_bias,
    const float* __restrict__ D, float* __restrict__ qk, float* __restrict__ vf,
    float* __restrict__ skip, float* __restrict__ decay, int T, int H, int G, int N, int P,
    int* __restrict__ err) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_token = H + 2 * G;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)T * per_token) return;
  const int t = (int)(item / per_token), u = (int)(item % per_token);
  const int C = H * P + 2 * G * N;             // channels that pass the convolution
  int kind, d, c0;                             // 0 x, 1 B, 2 C; first channel of the unit
  if (u < H) { kind = 0; d = P; c0 = u * P; }
  else if (u < H + G) { kind = 1; d = N; c0 = H * P + (u - H) * N; }
  else { kind = 2; d = N; c0 = H * P + G * N + (u - H - G) * N; }
  const int b = seq_of_token[t];
  const int local = t - q_start[b];
  int slot = 0;
  if (taps > 1) {
    slot = state_slots[b];
    if (slot < 0 || slot >= n_state_slots) { atomicOr(err, BF_ERR_SLOT); slot = 0; }
  }
  const float* st = state + (size_t)slot * state_stride;
  const A* row = proj + (size_t)t * stride;
  float dt = 0.f, dskip = 0.f;
  if (kind == 0) {
    dt = m2_softplus(bf_ld(row + dt_off + u) + dt_bias[u]);
    dskip = D[u];
    if (lane == 0) decay[(size_t)t * H + u] = expf(-expf(A_log[u]) * dt);
  }
  for (int i = lane; i < d; i += 32) {
    const int c = c0 + i;
    float y = conv_b ? conv_b[c] : 0.f;
    if (taps >= 1) {
      for (int j = 0; j < taps; ++j) {
        const int src = local - (taps - 1) + j;
        const float v = src >= 0 ? bf_ld(proj + (size_t)(t - (taps - 1) + j) * stride + xbc_off + c)
                                 : st[(size_t)(taps - 1 + src) * C + c];
        y += conv_w[(size_t)c * taps + j] * v;
      }
    } else {
      y += bf_ld(row + xbc_off + c);
    }
    y = y / (1.f + expf(-y));
    if (kind == 0) {
      vf[((size_t)t * H + u) * P + i] = dt * y;
      skip[((size_t)t * H + u) * P + i] = dskip * y;
    } else if (kind == 1) {
      qk[(((size_t)t * 2 + 1) * G + (u - H)) * N + i] = y;          // k = B
    } else {
      qk[(((size_t)t * 2) * G + (u - H - G)) * N + i] = y;          // q = C
    }
  }
}

BF_EXPORT int bf_mamba2_encode(const void* proj, long long stride, long long xbc_off,
                               long long dt_off, const float* conv_w, const float* conv_b,
                               int taps, const float* state, long long state_stride,
                               const int* state_slots, int n_state_slots,
                               const int* seq_of_token, const int* q_start, const float* A_log,
                               const float* dt_bias, const float* D, float* qk, float* vf,
                               float* skip, float* decay, int T, int H, int G, int N, int P,
                               int act_dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (taps > M2_MAX_TAPS || (taps > 1 && !state) || (taps >= 1 && !conv_w) || G <= 0 || H % G)
    return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const long long items = (long long)T * (H + 2 * G);
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (act_dtype == BF_DTYPE_F32)
    mamba2_encode_kernel<float><<<blocks, warps * 32, 0, stream>>>(
        (const float*)proj, stride, xbc_off, dt_off, conv_w, conv_b, taps, state, state_stride,
        state_slots, n_state_slots, seq_of_token, q_start, A_log, dt_bias, D, qk, vf, skip, decay,
        T, H, G, N, P, err);
  else
    mamba2_encode_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
        (const __nv_bfloat16*)proj, stride, xbc_off, dt_off, conv_w, conv_b, taps, state,
        state_stride, state_slots, n_state_slots, seq_of_token, q_start, A_log, dt_bias, D, qk,
        vf, skip, decay, T, H, G, N, P, err);
  return bf_launch_status();
}

// ------------------------------------------------------------------ gate_norm_out
// out[t, c] = y[c] * rsqrt(mean of y^2 over c's part + eps) * weight[c] with
// y[c] = (o_raw[t, c] + skip[t, c]) * silu(z[t, c]); the row has `parts` equal parts.
template <typename A>
__global__ void gate_norm_out_kernel(const float* __restrict__ o_raw,
                                     const float* __restrict__ skip, const A* __restrict__ proj,
                                     long long stride, long long z_off,
                                     const float* __restrict__ weight, A* __restrict__ out,
                                     long long out_stride, int n, int parts, float eps) {
  __shared__ float scratch[33];
  const int t = blockIdx.x, part = blockIdx.y;
  const int per = n / parts, c0 = part * per;
  const float* o = o_raw + (size_t)t * n + c0;
  const float* sk = skip ? skip + (size_t)t * n + c0 : nullptr;
  const A* z = proj + (size_t)t * stride + z_off + c0;
  A* dst = out + (size_t)t * out_stride + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const float g = bf_ld(z + i);
    const float y = (o[i] + (sk ? sk[i] : 0.f)) * (g / (1.f + expf(-g)));
    ss += y * y;
  }
  const float f = rsqrtf(block_sum(ss, scratch) / (float)per + eps);
  for (int i = threadIdx.x; i < per; i += blockDim.x) {
    const float g = bf_ld(z + i);
    const float y = (o[i] + (sk ? sk[i] : 0.f)) * (g / (1.f + expf(-g)));
    bf_st(dst + i, y * f * (weight ? weight[c0 + i] : 1.f));
  }
}

BF_EXPORT int bf_gate_norm_out(const float* o_raw, const float* skip, const void* proj,
                               long long stride, long long z_off, const float* weight, void* out,
                               long long out_stride, int T, int n, int parts, float eps,
                               int act_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (parts <= 0 || n % parts) return (int)cudaErrorInvalidValue;
  const int per = n / parts;
  const int threads = per > 1024 ? 256 : (per > 64 ? 128 : 32);
  dim3 grid(T, parts);
  if (act_dtype == BF_DTYPE_F32)
    gate_norm_out_kernel<float><<<grid, threads, 0, stream>>>(
        o_raw, skip, (const float*)proj, stride, z_off, weight, (float*)out, out_stride, n, parts,
        eps);
  else
    gate_norm_out_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        o_raw, skip, (const __nv_bfloat16*)proj, stride, z_off, weight, (__nv_bfloat16*)out,
        out_stride, n, parts, eps);
  return bf_launch_status();
}
