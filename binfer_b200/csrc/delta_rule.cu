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
// adjacent lanes.  A lane holds R state elements of its column in registers, in pieces of
// four that lie KS pieces apart (piece r4 of lane `part` is piece r4 KS + part of the
// column), so that the lanes of a column read neighbouring 16-byte pieces of a token's k and
// q from shared memory (no bank conflicts) and of the state from the slot (whole lines).
//
// The chain from token to token is kept short.  Both S^T k and S^T q are formed from the
// state as the token before left it, side by side and added over the KS lanes by one round of
// shuffles; with g the decay and u as above, the read-out of the state after the write is
//
//   o_t = g (S_old^T q_t) + (k_t . q_t) u_t,
//
// and the state's update S <- g S + k u^T then waits for u alone.  Up to `stage` tokens are
// staged in shared memory at a time, in two buffers: the next stage's asynchronous copies (k,
// q, v and both gates alike) travel while this one is walked.  When a stage has landed the
// block forms k_t . q_t for all its tokens, a warp a token; the walk then fetches a token's
// k, q, v, gates and k . q from shared memory one token ahead, under the chain of the token
// before.  The lanes of a column (KS, a template parameter: the shuffle rounds unroll) are
// neighbours in a warp.  Every sum has an order that depends on the sizes alone, so the
// result does not depend on how the tokens were cut into steps.
#include "common.cuh"

#define DR_THREADS 128

__device__ __forceinline__ void dr_cp16(float* smem, const float* gmem) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem));
}

__device__ __forceinline__ void dr_cp4(float* smem, const float* gmem) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sa), "l"(gmem));
}

template <int R, int KS>
__global__ void __launch_bounds__(DR_THREADS) delta_scan_kernel(
    const float* __restrict__ qkv, const float* __restrict__ gates, float* __restrict__ state,
    long long state_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
    int n_slots, float* __restrict__ o_raw, int H, int G, int dk, int dv, int stage,
    int* __restrict__ err) {
  extern __shared__ __align__(16) float sh[];
  constexpr int R4 = R / 4;
  constexpr int cols = DR_THREADS / KS;
  constexpr int dkp = KS * R;               // dk rounded up to what the lanes of a column hold
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
  float* sp = state + (size_t)slot * state_stride + ((size_t)h * dv + col) * dk;
  // whole pieces of four floats where the sizes and the slot's address allow it
  const bool st16 = (dk & 3) == 0 && (state_stride & 3) == 0 && (((uintptr_t)state) & 15) == 0;
  float S[R];
#pragma unroll
  for (int r4 = 0; r4 < R4; ++r4) {
    const int i = (r4 * KS + part) * 4;
    if (st16 && col < dv && i < dk) {
      const float4 x = *reinterpret_cast<const float4*>(sp + i);
      S[4 * r4] = x.x; S[4 * r4 + 1] = x.y; S[4 * r4 + 2] = x.z; S[4 * r4 + 3] = x.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) S[4 * r4 + e] = (col < dv && i + e < dk) ? sp[i + e] : 0.f;
    }
  }

  // one buffer: [stage][dkp] q, [stage][dkp] k, [stage][cols] v, [stage][2] beta and decay,
  // [stage] k . q; a buffer is a whole number of 16-byte pieces long, so that the second one
  // starts on such a boundary too
  const int buf_elems = (stage * (2 * dkp + cols + 3) + 3) & ~3;
  const bool rows16 = (dk & 3) == 0 && (C & 3) == 0;
  auto issue = [&](int s0, int buf) {
    const int sn = min(stage, n - s0);
    float* qd = sh + (size_t)buf * buf_elems;
    float* kd = qd + stage * dkp;
    float* vd = kd + stage * dkp;
    float* gd = vd + stage * cols;
    if (rows16) {
      const int d4 = dkp >> 2, have = dk >> 2;
      for (int idx = tid; idx < sn * d4; idx += DR_THREADS) {
        const int c = idx / d4, i = idx - c * d4;
        if (i < have) {
          const float* row = qkv + (size_t)(t0 + s0 + c) * C + (size_t)g * dk + 4 * i;
          dr_cp16(qd + 4 * idx, row);
          dr_cp16(kd + 4 * idx, row + (size_t)G * dk);
        } else {
          *reinterpret_cast<float4*>(qd + 4 * idx) = make_float4(0.f, 0.f, 0.f, 0.f);
          *reinterpret_cast<float4*>(kd + 4 * idx) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    } else {
      for (int idx = tid; idx < sn * dkp; idx += DR_THREADS) {
        const int c = idx / dkp, i = idx - c * dkp;
        const float* row = qkv + (size_t)(t0 + s0 + c) * C + (size_t)g * dk;
        qd[idx] = i < dk ? row[i] : 0.f;
        kd[idx] = i < dk ? row[(size_t)G * dk + i] : 0.f;
      }
    }
    for (int idx = tid; idx < sn * cols; idx += DR_THREADS) {
      const int c = idx / cols, j = idx - c * cols;
      if (col0 + j < dv)
        dr_cp4(vd + idx,
               qkv + (size_t)(t0 + s0 + c) * C + 2 * (size_t)G * dk + (size_t)h * dv + col0 + j);
      else
        vd[idx] = 0.f;
    }
    for (int idx = tid; idx < sn * 2; idx += DR_THREADS) {
      const int c = idx >> 1, w = idx & 1;
      dr_cp4(gd + idx, gates + ((size_t)(t0 + s0 + c) * 2 + w) * H + h);
    }
    asm volatile("cp.async.commit_group;" ::);
  };
  issue(0, 0);
  int buf = 0;
  for (int s0 = 0; s0 < n; s0 += stage, buf ^= 1) {
    const int sn = min(stage, n - s0);
    if (s0 + stage < n) {                   // the next stage travels while this one is used
      issue(s0 + stage, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::);
    } else {
      asm volatile("cp.async.wait_group 0;" ::);
    }
    __syncthreads();
    const float* qs = sh + (size_t)buf * buf_elems;
    const float* ks = qs + stage * dkp;
    const float* vs = ks + stage * dkp;
    const float* gs = vs + stage * cols;
    float* kqs = sh + (size_t)buf * buf_elems + stage * (2 * dkp + cols + 2);
    for (int c = tid >> 5; c < sn; c += DR_THREADS / 32) {   // a warp a token
      float d = 0.f;
      for (int i = tid & 31; i < dkp; i += 32) d = fmaf(ks[c * dkp + i], qs[c * dkp + i], d);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if ((tid & 31) == 0) kqs[c] = d;
    }
    __syncthreads();
    // a token's k, q, v, gates and k . q, held one token ahead in two sets of registers
    float4 kk[2][R4], qq[2][R4];
    float vv[2], be[2], de[2], kq[2];
#define DR_FETCH(c, bi)                                                                  \
  {                                                                                     \
    const float4* kr = reinterpret_cast<const float4*>(ks + (size_t)(c) * dkp) + part;  \
    const float4* qr = reinterpret_cast<const float4*>(qs + (size_t)(c) * dkp) + part;  \
    _Pragma("unroll") for (int r4 = 0; r4 < R4; ++r4) {                                 \
      kk[bi][r4] = kr[r4 * KS];                                                         \
      qq[bi][r4] = qr[r4 * KS];                                                         \
    }                                                                                   \
    kq[bi] = kqs[(c)];                                                                  \
    vv[bi] = vs[(c) * cols + cg];                                                       \
    be[bi] = gs[2 * (c)];                                                               \
    de[bi] = gs[2 * (c) + 1];                                                           \
  }
#define DR_TOKEN(c, bi)                                                                  \
  {                                                                                     \
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f; \
    _Pragma("unroll") for (int r4 = 0; r4 < R4; ++r4) {                                 \
      a0 = fmaf(S[4 * r4], kk[bi][r4].x, a0);                                           \
      a1 = fmaf(S[4 * r4 + 1], kk[bi][r4].y, a1);                                       \
      a2 = fmaf(S[4 * r4 + 2], kk[bi][r4].z, a2);                                       \
      a3 = fmaf(S[4 * r4 + 3], kk[bi][r4].w, a3);                                       \
      b0 = fmaf(S[4 * r4], qq[bi][r4].x, b0);                                           \
      b1 = fmaf(S[4 * r4 + 1], qq[bi][r4].y, b1);                                       \
      b2 = fmaf(S[4 * r4 + 2], qq[bi][r4].z, b2);                                       \
      b3 = fmaf(S[4 * r4 + 3], qq[bi][r4].w, b3);                                       \
    }                                                                                   \
    float sk = (a0 + a1) + (a2 + a3), sq = (b0 + b1) + (b2 + b3);                       \
    const float decay = de[bi];                                                         \
    _Pragma("unroll") for (int r = 0; r < R; ++r) S[r] *= decay;                        \
    _Pragma("unroll") for (int o = 1; o < KS; o <<= 1) {                                \
      sk += __shfl_xor_sync(0xffffffffu, sk, o);                                        \
      sq += __shfl_xor_sync(0xffffffffu, sq, o);                                        \
    }                                                                                   \
    const float u = be[bi] * (vv[bi] - decay * sk);                                     \
    _Pragma("unroll") for (int r4 = 0; r4 < R4; ++r4) {                                 \
      S[4 * r4] = fmaf(kk[bi][r4].x, u, S[4 * r4]);                                     \
      S[4 * r4 + 1] = fmaf(kk[bi][r4].y, u, S[4 * r4 + 1]);                             \
      S[4 * r4 + 2] = fmaf(kk[bi][r4].z, u, S[4 * r4 + 2]);                             \
      S[4 * r4 + 3] = fmaf(kk[bi][r4].w, u, S[4 * r4 + 3]);                             \
    }                                                                                   \
    if (part == 0 && col < dv)                                                          \
      o_raw[(size_t)(t0 + s0 + (c)) * H * dv + (size_t)h * dv + col] =                  \
          fmaf(decay, sq, kq[bi] * u);                                                  \
  }
    DR_FETCH(0, 0)
    int c = 0;
    for (; c + 1 < sn; c += 2) {
      DR_FETCH(c + 1, 1)
      DR_TOKEN(c, 0)
      if (c + 2 < sn) DR_FETCH(c + 2, 0)
      DR_TOKEN(c + 1, 1)
    }
    if (c < sn) DR_TOKEN(c, 0)
#undef DR_FETCH
#undef DR_TOKEN
    __syncthreads();                        // this buffer is filled again in the next round
  }
#pragma unroll
  for (int r4 = 0; r4 < R4; ++r4) {
    const int i = (r4 * KS + part) * 4;
    if (st16 && col < dv && i < dk) {
      *reinterpret_cast<float4*>(sp + i) =
          make_float4(S[4 * r4], S[4 * r4 + 1], S[4 * r4 + 2], S[4 * r4 + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (col < dv && i + e < dk) sp[i + e] = S[4 * r4 + e];
    }
  }
}

BF_EXPORT int bf_delta_scan(const float* qkv, const float* gates, float* state,
                            long long state_stride, const int* q_start, const int* state_slots,
                            int n_slots, float* o_raw, int T, int B, int max_q, int H, int G,
                            int dk, int dv, int* err, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 1024 || G <= 0 || H % G) return (int)cudaErrorInvalidValue;
  const int R = dk <= 128 ? 16 : 32;
  int KS = dk <= 128 ? 1 : 8;
  while (KS * R < dk) KS <<= 1;
  const int cols = DR_THREADS / KS;
  const size_t per_token = (size_t)(2 * KS * R + cols + 3) * sizeof(float);
  int stage = 32;
  while (stage > 2 && stage / 2 >= max_q) stage >>= 1;
  while (stage > 2 && 2 * stage * per_token > 64 * 1024) stage >>= 1;
  // as the kernel lays it out: two buffers, each rounded up to 16 bytes
  const size_t smem = 2 * ((stage * per_token + 15) & ~(size_t)15);
  dim3 grid((dv + cols - 1) / cols, H, B);
#define DR_GO(RR, KK)                                                                          \
  {                                                                                            \
    if (smem > 48 * 1024)                                                                      \
      cudaFuncSetAttribute(delta_scan_kernel<RR, KK>,                                          \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    delta_scan_kernel<RR, KK><<<grid, DR_THREADS, smem, stream>>>(                             \
        qkv, gates, state, state_stride, q_start, state_slots, n_slots, o_raw, H, G, dk, dv,   \
        stage, err);                                                                           \
  }
  if (R == 16) {
    if (KS == 1) DR_GO(16, 1) else if (KS == 2) DR_GO(16, 2) else if (KS == 4) DR_GO(16, 4)
    else DR_GO(16, 8)
  } else {
    if (KS == 8) DR_GO(32, 8) else if (KS == 16) DR_GO(32, 16) else DR_GO(32, 32)
  }
#undef DR_GO
  return bf_launch_status();
}
