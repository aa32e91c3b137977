// The gated delta rule: a matrix memory per request and value head, S [dk, dv] in float,
//
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// walked token by token over the step's tokens of every request.  q and k (unit vectors, q
// scaled), v and the two gates come in float from delta_encode (mixer_encode.cu): qkv
// [T][G dk | G dk | H dv], gates [T][2][H].  Value head h reads q/k head h / (H / G).  The
// state lives in the request's state slot, column by column ([H][dv][dk]: the dk numbers that
// one output column needs lie side by side), and is carried from step to step, so a prompt
// can be cut anywhere.
//
// A block owns `cols` output columns of one (request, head); a column is shared by KS
// adjacent lanes that each hold R consecutive state elements of it in registers.  Up to
// `stage` tokens' q, k, v and gates are staged in shared memory at a time.  Per token a lane
// forms its share of S^T k with the state as it was (the decay multiplies the sum, not the
// elements), the KS shares are added by shuffles, and one pass then updates the state,
// S <- g S + k u^T, and forms the lane's share of S^T q.  Every sum has an order that depends
// on the sizes alone, so the result does not depend on how the tokens were cut into steps.
#include "common.cuh"

#define DR_THREADS 128

template <int R>
__global__ void __launch_bounds__(DR_THREADS) delta_scan_kernel(
    const float* __restrict__ qkv, const float* __restrict__ gates, float* __restrict__ state,
    long long state_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
    int n_slots, float* __restrict__ o_raw, int H, int G, int dk, int dv, int KS, int stage,
    int* __restrict__ err) {
  extern __shared__ __align__(16) float sh[];
  const int cols = DR_THREADS / KS;
  const int dkp = KS * R;
  const int b = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * cols;
  const int g = h / (H / G);
  const int tid = threadIdx.x;
  const int cg = tid / KS, part = tid % KS;
  const int col = col0 + cg;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  const int slot = state_slots[b];
  if (slot < 0 || slot >= n_slots) {
    if (tid == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  const int C = 2 * G * dk + H * dv;
  float* sp = state + (size_t)slot * state_stride + ((size_t)h * dv + col) * dk + (size_t)part * R;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = (col < dv && part * R + r < dk) ? sp[r] : 0.f;

  float* qs = sh;                         // [stage][dkp]
  float* ks = qs + (size_t)stage * dkp;   // [stage][dkp]
  float* vs = ks + (size_t)stage * dkp;   // [stage][cols]
  float* gs = vs + (size_t)stage * cols;  // [stage][2]: beta, decay
  for (int s0 = 0; s0 < n; s0 += stage) {
    const int sn = min(stage, n - s0);
    __syncthreads();                      // the stage before is used up
    for (int idx = tid; idx < sn * dkp; idx += DR_THREADS) {
      const int c = idx / dkp, i = idx - c * dkp;
      const float* row = qkv + (size_t)(t0 + s0 + c) * C + (size_t)g * dk;
      qs[idx] = i < dk ? row[i] : 0.f;
      ks[idx] = i < dk ? row[(size_t)G * dk + i] : 0.f;
    }
    for (int idx = tid; idx < sn * cols; idx += DR_THREADS) {
      const int c = idx / cols, j = idx - c * cols;
      vs[idx] = col0 + j < dv
                    ? qkv[(size_t)(t0 + s0 + c) * C + 2 * (size_t)G * dk + (size_t)h * dv + col0 + j]
                    : 0.f;
    }
    for (int idx = tid; idx < sn * 2; idx += DR_THREADS) {
      const int c = idx >> 1, w = idx & 1;
      gs[idx] = gates[((size_t)(t0 + s0 + c) * 2 + w) * H + h];
    }
    __syncthreads();
    for (int c = 0; c < sn; ++c) {
      const float* kr = ks + (size_t)c * dkp + part * R;
      const float* qr = qs + (size_t)c * dkp + part * R;
      const float beta = gs[2 * c], decay = gs[2 * c + 1];
      float kk[R];
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        kk[r] = kr[r];
        kk[r + 1] = kr[r + 1];
        a0 = fmaf(S[r], kk[r], a0);
        a1 = fmaf(S[r + 1], kk[r + 1], a1);
      }
      float sk = a0 + a1;
      for (int o = 1; o < KS; o <<= 1) sk += __shfl_xor_sync(0xffffffffu, sk, o);
      const float u = beta * (vs[c * cols + cg] - decay * sk);
      a0 = a1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        S[r] = fmaf(decay, S[r], kk[r] * u);
        S[r + 1] = fmaf(decay, S[r + 1], kk[r + 1] * u);
        a0 = fmaf(S[r], qr[r], a0);
        a1 = fmaf(S[r + 1], qr[r + 1], a1);
      }
      float so = a0 + a1;
      for (int o = 1; o < KS; o <<= 1) so += __shfl_xor_sync(0xffffffffu, so, o);
      if (part == 0 && col < dv)
        o_raw[(size_t)(t0 + s0 + c) * H * dv + (size_t)h * dv + col] = so;
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r)
    if (col < dv && part * R + r < dk) sp[r] = S[r];
}

BF_EXPORT int bf_delta_scan(const float* qkv, const float* gates, float* state,
                            long long state_stride, const int* q_start, const int* state_slots,
                            int n_slots, float* o_raw, int T, int B, int max_q, int H, int G,
                            int dk, int dv, int* err, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 1024 || G <= 0 || H % G) return (int)cudaErrorInvalidValue;
  const int R = dk <= 128 ? 16 : 32;
  int KS = 1;
  while (KS * R < dk) KS <<= 1;
  const int cols = DR_THREADS / KS;
  int stage = 32;
  while (stage > 1 && stage / 2 >= max_q) stage >>= 1;
  while (stage > 1 && (size_t)stage * (2 * KS * R + cols + 2) * sizeof(float) > 40 * 1024)
    stage >>= 1;
  const size_t smem = (size_t)stage * (2 * KS * R + cols + 2) * sizeof(float);
  dim3 grid((dv + cols - 1) / cols, H, B);
  if (R == 16)
    delta_scan_kernel<16><<<grid, DR_THREADS, smem, stream>>>(
        qkv, gates, state, state_stride, q_start, state_slots, n_slots, o_raw, H, G, dk, dv, KS,
        stage, err);
  else
    delta_scan_kernel<32><<<grid, DR_THREADS, smem, stream>>>(
        qkv, gates, state, state_stride, q_start, state_slots, n_slots, o_raw, H, G, dk, dv, KS,
        stage, err);
  return bf_launch_status();
}
