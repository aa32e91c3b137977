// Retention: linear attention with a fixed decay per head and no softmax,
//
//   S_t = decay_h S_{t-1} + k_t v_t^T        o_t = S_t^T q_t
//
// with q and k turned by a rotary angle of the token's position (the first 2 rot_half
// sizes of a head; k is then multiplied by k_scale).  The state S [dk, dv] per request and
// head is float and lives in the request's state slot, stored column by column
// ([dv][dk]: the dk numbers that one output column needs lie side by side), and is carried
// from step to step, so a prompt can be cut anywhere.
//
// With `act` 1, q, k and v pass silu first (lightning attention).
//
// The scan also runs recurrences whose decay differs from token to token and whose q and k
// are shared by several heads (a state space layer in its scalar-decay form: q = C, k = B,
// v = dt x): bf_linear_scan takes q, k and v in float as the encode kernel would leave them,
// q and k with `qk_heads` heads (head h reads head h / (H / qk_heads)), and a decay per
// (token, head), which travels through shared memory beside v.
//
// retention_encode: q and k of every (token, head), turned and scaled, as float rows
// `qk [T][2][H][dk]`, and the head's v in float `vf [T][H][dv]` (one warp per (token, head);
// the scan's blocks, several per head, read them from there by asynchronous copies instead
// of each turning and converting them again).
//
// retention_scan: a block owns `cols` output columns of one (request, head); a column is
// shared by KS adjacent lanes that each hold R consecutive state elements of it in registers
// (of four columns at a time where the sizes allow: a tile of the state per lane).  The
// step's tokens are walked in order: up to RET_STAGE tokens' q, k and v at a time are staged
// in shared memory (two buffers: the next stage's asynchronous copies travel while this one
// is used) and walked in chunks of RET_CHUNK.  Inside a chunk a lane updates its state elements token by token
// and keeps its partial dot product of every token in a register; the KS partial sums of a
// column are added by shuffles once per chunk, all tokens at a time, so that the only
// dependent chain from token to token is the state's own multiply-add.  Every sum has an
// order that depends on the sizes alone, so the result does not depend on how the tokens
// were cut into steps.
//
// retention_out: each head's output divided by its root mean square (no weight), times
// silu of the gate projection, times out_scale, into a column block of `out`.
#include "common.cuh"

#define RET_CHUNK 16        // tokens whose partial sums a lane holds at a time
#define RET_STAGE 64        // tokens staged in shared memory at a time (fewer for large heads)
#define RET_THREADS 128

template <typename A>
__global__ void retention_encode_kernel(const A* __restrict__ proj, long long stride,
                                        long long q_off, long long k_off,
                                        const float* __restrict__ inv_freq, int rot_half,
                                        const int* __restrict__ positions,
                                        float* __restrict__ qk, int T, int H, int dk,
                                        float k_scale, int act, long long v_off, int dv,
                                        float* __restrict__ vf) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const A* row = proj + (size_t)t * stride + (size_t)h * dk;
  float* qo = qk + ((size_t)t * 2 * H + h) * dk;
  float* ko = qo + (size_t)H * dk;
  const float pos = (float)positions[t];
  for (int i = lane; i < dk; i += 32) {
    float qv = bf_ld(row + q_off + i), kv = bf_ld(row + k_off + i);
    if (act) {
      qv = qv / (1.f + expf(-qv));
      kv = kv / (1.f + expf(-kv));
    }
    if (i < 2 * rot_half) {
      const int m = i < rot_half ? i : i - rot_half;
      const int o = i < rot_half ? i + rot_half : i - rot_half;
      float sn, cs;
      sincosf(pos * inv_freq[m], &sn, &cs);
      float qo2 = bf_ld(row + q_off + o), ko2 = bf_ld(row + k_off + o);
      if (act) {
        qo2 = qo2 / (1.f + expf(-qo2));
        ko2 = ko2 / (1.f + expf(-ko2));
      }
      qv = i < rot_half ? qv * cs - qo2 * sn : qv * cs + qo2 * sn;
      kv = i < rot_half ? kv * cs - ko2 * sn : kv * cs + ko2 * sn;
    }
    qo[i] = qv;
    ko[i] = kv * k_scale;
  }
  // the head's values in float (activation applied), for the scan's asynchronous copies
  const A* vrow = proj + (size_t)t * stride + v_off + (size_t)h * dv;
  float* vo = vf + ((size_t)t * H + h) * dv;
  for (int i = lane; i < dv; i += 32) {
    float x = bf_ld(vrow + i);
    if (act) x = x / (1.f + expf(-x));
    vo[i] = x;
  }
}

__device__ __forceinline__ void ret_cp16(float* smem, const float* gmem) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem));
}

// R: state elements along dk that a lane holds per column; CV: columns a lane holds (its
// state tile is CV x R: a token's k and q values are then fetched once for CV columns).
__device__ __forceinline__ void ret_cp4(float* smem, const float* gmem) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sa), "l"(gmem));
}

// KST: the lanes per column where they are known when the kernel is compiled (the rounds of
// shuffles then unroll), 0: `ks_rt` of them.
// TD: the decay comes per (token, head) from `tok_decay [T][H]` instead of per head from `decays`.
template <int R, int CV, int KST, bool TD>
__global__ void __launch_bounds__(RET_THREADS) retention_scan_kernel(
    const float* __restrict__ vf, const float* __restrict__ qk, const float* __restrict__ decays,
    float* __restrict__ state, long long state_stride, const int* __restrict__ q_start,
    const int* __restrict__ state_slots, int n_slots, float* __restrict__ o_raw, int H, int dk,
    int dv, int ks_rt, int stage, int* __restrict__ err, const float* __restrict__ tok_decay,
    int QH) {
  extern __shared__ __align__(16) float sh[];
  const int KS = KST ? KST : ks_rt;
  const int cols = RET_THREADS / KS * CV;
  const int dkp = KS * R;                   // dk rounded up to what the lanes of a column hold
  // two buffers of [stage][dkp] q, [stage][dkp] k, [stage][cols] v (TD: and [stage] decays)
  const int b = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * cols;
  const int hq = h / (H / QH);              // the head of q and k that this head reads
  const int tid = threadIdx.x;
  const int cg = tid / KS, part = tid % KS;
  const int col = col0 + cg * CV;           // the lane's first column
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  int slot = state_slots[b];
  if (slot < 0 || slot >= n_slots) {
    if (tid == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  const float decay_h = TD ? 1.f : decays[h];
  float* sp = state + (size_t)slot * state_stride + (size_t)h * dv * dk + (size_t)part * R;
  float S[CV][R];
  // whole rows of four floats where the sizes and the slot's address allow it
  const bool st16 = dkp == dk && (dk & 3) == 0 && (state_stride & 3) == 0 &&
                    (((uintptr_t)state) & 15) == 0;
#pragma unroll
  for (int j = 0; j < CV; ++j) {
    if (st16 && col + j < dv) {
      const float4* s4 = reinterpret_cast<const float4*>(sp + (size_t)(col + j) * dk);
#pragma unroll
      for (int r4 = 0; r4 < R / 4; ++r4) {
        const float4 x = s4[r4];
        S[j][4 * r4] = x.x; S[j][4 * r4 + 1] = x.y; S[j][4 * r4 + 2] = x.z; S[j][4 * r4 + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r)
        S[j][r] = (col + j < dv && part * R + r < dk) ? sp[(size_t)(col + j) * dk + r] : 0.f;
    }
  }

  // A stage on its way into buffer `buf`: q and k rows by asynchronous 16-byte copies where
  // the rows allow it, v (in float since the first kernel) by asynchronous copies of one.
  const int buf_elems = stage * (2 * dkp + cols) + (TD ? stage : 0);
  const bool rows16 = (dk & 3) == 0 && dkp == dk;
  auto issue = [&](int s0, int buf) {
    const int sn = min(stage, n - s0);
    float* qd = sh + (size_t)buf * buf_elems;
    float* kd = qd + stage * dkp;
    float* vd = kd + stage * dkp;
    // In shared memory a token's k (and q) lies piece by piece of four floats in the order
    // [r4][part]: the lanes of a column, which fetch piece r4 of their R elements together,
    // then read neighbouring addresses (no bank conflicts), not addresses R floats apart.
    if (rows16) {
      const int d4 = dk >> 2;
      for (int idx = tid; idx < sn * d4; idx += RET_THREADS) {
        const int c = idx / d4, i = idx - c * d4;
        const int at = c * d4 + (i % (R / 4)) * KS + i / (R / 4);
        const float* row = qk + ((size_t)(t0 + s0 + c) * 2 * QH + hq) * dk + 4 * i;
        ret_cp16(qd + 4 * at, row);
        ret_cp16(kd + 4 * at, row + (size_t)QH * dk);
      }
    } else {
      for (int idx = tid; idx < sn * dkp; idx += RET_THREADS) {
        const int c = idx / dkp, i = idx % dkp;
        const int pt = i / R, r = i % R;
        const int at = c * dkp + ((r >> 2) * KS + pt) * 4 + (r & 3);
        const float* row = qk + ((size_t)(t0 + s0 + c) * 2 * QH + hq) * dk;
        qd[at] = i < dk ? row[i] : 0.f;
        kd[at] = i < dk ? row[(size_t)QH * dk + i] : 0.f;
      }
    }
    for (int idx = tid; idx < sn * cols; idx += RET_THREADS) {
      const int c = idx / cols, j = idx % cols;
      if (col0 + j < dv)
        ret_cp4(vd + idx, vf + ((size_t)(t0 + s0 + c) * H + h) * dv + col0 + j);
      else
        vd[idx] = 0.f;
    }
    if (TD) {
      float* dd = vd + stage * cols;
      for (int c = tid; c < sn; c += RET_THREADS)
        ret_cp4(dd + c, tok_decay + (size_t)(t0 + s0 + c) * H + h);
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
    const float* ks_ = qs + stage * dkp;
    const float* vs = ks_ + stage * dkp;
    const float* ds = vs + stage * cols;
    for (int c0 = 0; c0 < sn; c0 += RET_CHUNK) {
      const int cn = min(RET_CHUNK, sn - c0);
      float acc[RET_CHUNK][CV];
      // one token: the state's multiply-add and this lane's share of the token's dot products
      // A token's k, q and v are fetched one token ahead of their use (two sets of
      // registers in turn), so that the shared-memory round trip runs under the token
      // before; the state's own chain is one multiply-add a token (k v is formed beside it).
      float4 kk[2][R / 4], qq[2][R / 4];
      float vv[2][CV];
      float dec[2] = {decay_h, decay_h};
#define RET_FETCH(c, bi)                                                                        \
  {                                                                                            \
    if (TD) dec[bi] = ds[c0 + (c)];                                                            \
    const float4* qr = reinterpret_cast<const float4*>(qs + (c0 + (c)) * dkp) + part;          \
    const float4* kr = reinterpret_cast<const float4*>(ks_ + (c0 + (c)) * dkp) + part;         \
    _Pragma("unroll") for (int r4 = 0; r4 < R / 4; ++r4) {                                     \
      kk[bi][r4] = kr[r4 * KS];                                                                 \
      qq[bi][r4] = qr[r4 * KS];                                                                 \
    }                                                                                          \
    _Pragma("unroll") for (int j = 0; j < CV; ++j) vv[bi][j] = vs[(c0 + (c)) * cols + cg * CV + j]; \
  }
#define RET_TOKEN(c, bi)                                                                        \
  {                                                                                            \
    float a0[CV], a1[CV];                                                                      \
    const float decay = dec[bi];                                                               \
    _Pragma("unroll") for (int j = 0; j < CV; ++j) a0[j] = a1[j] = 0.f;                        \
    _Pragma("unroll") for (int r4 = 0; r4 < R / 4; ++r4) {                                     \
      _Pragma("unroll") for (int j = 0; j < CV; ++j) {                                         \
        S[j][4 * r4] = fmaf(decay, S[j][4 * r4], kk[bi][r4].x * vv[bi][j]);                      \
        S[j][4 * r4 + 1] = fmaf(decay, S[j][4 * r4 + 1], kk[bi][r4].y * vv[bi][j]);              \
        S[j][4 * r4 + 2] = fmaf(decay, S[j][4 * r4 + 2], kk[bi][r4].z * vv[bi][j]);              \
        S[j][4 * r4 + 3] = fmaf(decay, S[j][4 * r4 + 3], kk[bi][r4].w * vv[bi][j]);              \
        a0[j] += S[j][4 * r4] * qq[bi][r4].x;                                                   \
        a1[j] += S[j][4 * r4 + 1] * qq[bi][r4].y;                                               \
        a0[j] += S[j][4 * r4 + 2] * qq[bi][r4].z;                                               \
        a1[j] += S[j][4 * r4 + 3] * qq[bi][r4].w;                                               \
      }                                                                                        \
    }                                                                                          \
    _Pragma("unroll") for (int j = 0; j < CV; ++j) acc[c][j] = a0[j] + a1[j];                  \
  }
      RET_FETCH(0, 0)
      if (cn == RET_CHUNK) {
#pragma unroll
        for (int c = 0; c < RET_CHUNK; ++c) {
          if (c + 1 < RET_CHUNK) RET_FETCH(c + 1, (c + 1) & 1)
          RET_TOKEN(c, c & 1)
        }
      } else {
#pragma unroll
        for (int c = 0; c < RET_CHUNK; ++c) {
#pragma unroll
          for (int j = 0; j < CV; ++j) acc[c][j] = 0.f;
          if (c < cn) {
            if (c + 1 < cn) RET_FETCH(c + 1, (c + 1) & 1)
            RET_TOKEN(c, c & 1)
          }
        }
      }
#undef RET_FETCH
#undef RET_TOKEN
      // the KS partial sums of a column, all tokens of the chunk at a time
#pragma unroll
      for (int o = 1; o < KS; o <<= 1) {
#pragma unroll
        for (int c = 0; c < RET_CHUNK; ++c)
#pragma unroll
          for (int j = 0; j < CV; ++j) acc[c][j] += __shfl_xor_sync(0xffffffffu, acc[c][j], o);
      }
      if (part == 0) {
#pragma unroll
        for (int c = 0; c < RET_CHUNK; ++c)
#pragma unroll
          for (int j = 0; j < CV; ++j)
            if (c < cn && col + j < dv)
              o_raw[(size_t)(t0 + s0 + c0 + c) * H * dv + (size_t)h * dv + col + j] = acc[c][j];
      }
    }
    __syncthreads();                        // this buffer is filled again in the next round
  }
#pragma unroll
  for (int j = 0; j < CV; ++j) {
    if (st16 && col + j < dv) {
      float4* s4 = reinterpret_cast<float4*>(sp + (size_t)(col + j) * dk);
#pragma unroll
      for (int r4 = 0; r4 < R / 4; ++r4)
        s4[r4] = make_float4(S[j][4 * r4], S[j][4 * r4 + 1], S[j][4 * r4 + 2], S[j][4 * r4 + 3]);
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (col + j < dv && part * R + r < dk) sp[(size_t)(col + j) * dk + r] = S[j][r];
    }
  }
}

static int ret_launch_scan(const float* vf, const float* qk, const float* decays,
                           const float* tok_decay, int QH, float* state, long long state_stride,
                           const int* q_start, const int* state_slots, int n_slots,
                           float* o_raw, int B, int max_q, int H, int dk, int dv, int* err,
                           cudaStream_t stream) {
  const int R = dk <= 256 ? 8 : 32;
  int KS = 1;
  while (KS * R < dk) KS <<= 1;
  // A tile of two columns a lane: half the fetches of k and q per multiply-add, half the
  // warps.  Measured, 2,048 tokens of heads of 128 x 256, one / two / four columns a lane:
  // 8 heads 0.52 / 0.44 / 0.79 ms, 16 heads 1.35 / 0.67 / 0.95 ms; 8 single tokens 30 / 26 /
  // 28 us and 45 / 34 / 35 us.  Every column's sum has the same order either way.
  const int CV = (R == 8 && dv % 2 == 0) ? 2 : 1;
  const int cols = RET_THREADS / KS * CV;
  dim3 grid((dv + cols - 1) / cols, H, B);
  int stage = RET_STAGE;
  while (stage > RET_CHUNK && stage / 2 >= max_q) stage >>= 1;
  // (keys beyond 512 a head: fewer tokens a stage than a chunk holds; the walk takes what is there)
  const int extra = tok_decay ? 1 : 0;      // a decay per staged token
  const size_t per_token = (size_t)2 * (2 * KS * R + cols + extra) * sizeof(float);
  while (stage > 4 && stage * per_token > 72 * 1024) stage >>= 1;
  if (stage * per_token > 200 * 1024) return (int)cudaErrorInvalidValue;
  // More blocks than SMs: of the staging depths from this one down to a chunk, take the one
  // whose resident blocks walk the grid in the fewest waves (a grid a little larger than what
  // is resident at once runs twice as long), the deepest of those.  No sum's order depends on it.
  static int n_sms[BF_MAX_DEVICES];
  const int dev = bf_current_device();
  if (!n_sms[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    n_sms[dev] = n > 0 ? n : 148;
  }
  const long long blocks_total = (long long)grid.x * grid.y * grid.z;
#define RET_GO1(RR, CC, KK, TT)                                                               \
  {                                                                                            \
    auto kern = retention_scan_kernel<RR, CC, KK, TT>;                                         \
    int st = stage;                                                                            \
    if (stage * per_token > 48 * 1024)                                                         \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                           (int)(stage * per_token));                                          \
    if (blocks_total > n_sms[dev]) {                                                           \
      long long best = -1;                                                                     \
      for (int c = stage; c >= RET_CHUNK; c >>= 1) {                                           \
        int nb = 0;                                                                            \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, RET_THREADS,              \
                                                          c * per_token) != cudaSuccess ||    \
            nb < 1)                                                                            \
          continue;                                                                            \
        const long long at_once = (long long)n_sms[dev] * nb;                                  \
        const long long waves = (blocks_total + at_once - 1) / at_once;                        \
        if (best < 0 || waves < best) { best = waves; st = c; }                                \
      }                                                                                        \
    }                                                                                          \
    kern<<<grid, RET_THREADS, st * per_token, stream>>>(                                       \
        vf, qk, decays, state, state_stride, q_start, state_slots, n_slots, o_raw, H, dk, dv,  \
        KS, st, err, tok_decay, QH);                                                           \
  }
#define RET_GO(RR, CC, KK)                                                                    \
  {                                                                                            \
    if (tok_decay) RET_GO1(RR, CC, KK, true) else RET_GO1(RR, CC, KK, false)                   \
  }
  if (R == 32) RET_GO(32, 1, 0)
  else if (CV == 1) RET_GO(8, 1, 0)
  else if (KS == 8) RET_GO(8, 2, 8)
  else if (KS == 16) RET_GO(8, 2, 16)
  else if (KS == 32) RET_GO(8, 2, 32)
  else RET_GO(8, 2, 0)
#undef RET_GO
#undef RET_GO1
  return bf_launch_status();
}

BF_EXPORT int bf_retention_scan(
    const void* proj, long long stride, long long q_off, long long k_off, long long v_off,
    const float* decays, const float* inv_freq, int rot_half, const int* positions, float* state,
    long long state_stride, const int* q_start, const int* state_slots, int n_slots, float* o_raw,
    float* qk, float* vf, int T, int B, int max_q, int H, int dk, int dv, float k_scale,
    int act_dtype, int* err, int act, cudaStream_t stream) {
  // qk: scratch, float [T][2][H][dk]; vf: scratch, float [T][H][dv]; max_q: the most tokens one request brings (a hint that
  // sizes the staging buffers: single tokens leave room for more blocks an SM)
  if (B <= 0 || T <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 1024 || !qk || !vf) return (int)cudaErrorInvalidValue;
  {
    const int threads = 128;
    const long long blocks = ((long long)T * H * 32 + threads - 1) / threads;
    if (act_dtype == BF_DTYPE_F32)
      retention_encode_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
          (const float*)proj, stride, q_off, k_off, inv_freq, rot_half, positions, qk, T, H, dk,
          k_scale, act, v_off, dv, vf);
    else
      retention_encode_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
          (const __nv_bfloat16*)proj, stride, q_off, k_off, inv_freq, rot_half, positions, qk, T,
          H, dk, k_scale, act, v_off, dv, vf);
    const int e = bf_launch_status();
    if (e) return e;
  }
  return ret_launch_scan(vf, qk, decays, nullptr, H, state, state_stride, q_start, state_slots,
                         n_slots, o_raw, B, max_q, H, dk, dv, err, stream);
}

// The scan alone, on q, k and v that are float already: qk [T][2][qk_heads][dk] (q, then k),
// vf [T][H][dv], tok_decay [T][H].  State and output as in bf_retention_scan.
BF_EXPORT int bf_linear_scan(const float* qk, const float* vf, const float* tok_decay,
                             float* state, long long state_stride, const int* q_start,
                             const int* state_slots, int n_slots, float* o_raw, int T, int B,
                             int max_q, int H, int qk_heads, int dk, int dv, int* err,
                             cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 1024 || !qk || !vf || !tok_decay || qk_heads <= 0 ||
      H % qk_heads)
    return (int)cudaErrorInvalidValue;
  return ret_launch_scan(vf, qk, nullptr, tok_decay, qk_heads, state, state_stride, q_start,
                         state_slots, n_slots, o_raw, B, max_q, H, dk, dv, err, stream);
}

// One warp per (token, head).
template <typename A>
__global__ void retention_out_kernel(const float* __restrict__ o_raw, const A* __restrict__ proj,
                                     long long stride, long long g_off, A* __restrict__ out,
                                     long long out_stride, int T, int H, int dv, float eps,
                                     float out_scale) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float* o = o_raw + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += o[i] * o[i];
  const float f = rsqrtf(warp_sum(ss) / (float)dv + eps) * out_scale;
  const A* g = proj + (size_t)t * stride + g_off + (size_t)h * dv;
  A* dst = out + (size_t)t * out_stride + (size_t)h * dv;
  for (int i = lane; i < dv; i += 32) {
    const float z = bf_ld(g + i);
    bf_st(dst + i, o[i] * f * (z / (1.f + expf(-z))));
  }
}

BF_EXPORT int bf_retention_out(const float* o_raw, const void* proj, long long stride,
                               long long g_off, void* out, long long out_stride, int T, int H,
                               int dv, float eps, float out_scale, int act_dtype,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = 128;
  const long long blocks = ((long long)T * H * 32 + threads - 1) / threads;
  if (act_dtype == BF_DTYPE_F32)
    retention_out_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        o_raw, (const float*)proj, stride, g_off, (float*)out, out_stride, T, H, dv, eps,
        out_scale);
  else
    retention_out_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        o_raw, (const __nv_bfloat16*)proj, stride, g_off, (__nv_bfloat16*)out, out_stride, T, H,
        dv, eps, out_scale);
  return bf_launch_status();
}
