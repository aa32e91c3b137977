// Generic causal attention over the paged cache: any number of query tokens per
// request, any head count, group size, page size and head size up to 256.
//
// One warp per (query token, query head).  The query sits at absolute position p
// of its request; its keys are j in (p - window, p] (window 0: j in [0, p]), read
// through the request's block table.  Keys are walked in tiles of 32 whose edges
// are multiples of 32 counted from position 0, so the order of every sum depends
// only on p and the window, never on how the tokens were cut into steps or on
// what else is in the batch.
//
// This kernel is the whole 32-bit path's attention and the fallback for sizes
// that the tuned kernels refuse.  Formulas: scores (q . k) * scale, online
// softmax in float, probabilities kept in float for the product with v
// (cuda/kernels/bf16_kernels.cu:909-973; cuda/kernels/paged_attention.cu:408-487).
// The reference reads prefill keys from the fresh projection, not the cache
// (src/engine/batched_engine.ts:1082-1086); here every key comes from the pages.
//
// It is also where changes to the scores live, for attention that has them (the tuned
// kernels take none): a soft cap s <- c tanh(s / c), a bias per distance s <- s +
// slope_h (j - p), and a sink, a logit per head that joins the softmax's denominator and
// carries no value.  All three are off with softcap 0 and null pointers.  One more bias per
// distance grows with its logarithm: s <- s - b1_h ln(1 + b2_h (p - j)) (`log_slope` b1 and
// `log_rate` b2, one number per query head; off with null pointers).
//
// Two more things that the tuned kernels do not take: values of another size than keys
// (`dv`), and a window that keeps the request's first tokens: with keep_first > 0 the keys
// j < keep_first stay visible behind the window, at their true positions.  They are walked
// first, again in tiles of 32 counted from position 0.  `out_stride` and `out_scale` let the
// result land, scaled, in a column block of a wider buffer.  `v_stride` is the distance, in
// elements, between the value rows of neighbouring tokens of a page: with v_cache = k_cache
// and v_stride = d the values are the first dv numbers of the keys themselves (attention over
// a latent vector per token that serves as key and as value).  Values up to 256 a head keep
// 8 sums a lane, larger ones (up to 512) 16.
#include <float.h>

#include "common.cuh"

#define ATT_MAX_D 1024  // keys: a query head in shared memory per warp

template <typename A, int ATT_MAX_ACC>     // value size <= 32 * ATT_MAX_ACC
__global__ void paged_attention_generic_kernel(
    const A* __restrict__ q, const A* __restrict__ k_cache, const A* __restrict__ v_cache,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ block_tables, int table_stride, A* __restrict__ out, int nh, int nkv,
    int d, int page_size, int num_pages, int window, float scale, float softcap,
    const float* __restrict__ slopes, const float* __restrict__ sinks, int* __restrict__ err,
    int dv, int keep_first, long long q_stride, long long out_stride, float out_scale,
    long long v_stride, const float* __restrict__ log_slope, const float* __restrict__ log_rate) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int h = blockIdx.y * warps + warp;
  if (h >= nh) return;
  const int g = h / (nh / nkv);
  float* qs = sh + (size_t)warp * d;
  const A* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[i] = bf_ld(qrow + i) * scale;
  __syncwarp();

  const int p = positions[t];
  const int* table = block_tables + (size_t)seq_of_token[t] * table_stride;
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;

  float m = -FLT_MAX, l = 0.f;
  float acc[ATT_MAX_ACC];
#pragma unroll
  for (int c = 0; c < ATT_MAX_ACC; ++c) acc[c] = 0.f;

  // the kept first tokens that the window no longer covers, then the window
  const int kept = window > 0 ? min(keep_first, j0) : 0;
  const int kept_tiles = (kept + 31) >> 5;
  const int first_tile = j0 >> 5;
  const int n_tiles = kept_tiles + (p >> 5) - first_tile + 1;
  for (int it = 0; it < n_tiles; ++it) {
    const bool in_kept = it < kept_tiles;
    const int tile = in_kept ? it : first_tile + (it - kept_tiles);
    const int j = (tile << 5) + lane;
    bool valid = in_kept ? j < kept : (j >= j0 && j <= p);
    long long row = 0;     // index of this lane's key/value row (in rows of the cache)
    if (valid) {
      const int lp = j / page_size;
      const int page = table[lp];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, BF_ERR_PAGE);
        valid = false;
      } else {
        row = ((long long)page * nkv + g) * page_size + (j - lp * page_size);
      }
    }
    float s = -FLT_MAX;
    if (valid) {
      const A* kr = k_cache + row * d;
      float a = 0.f;
#pragma unroll 8
      for (int i = 0; i < d; ++i) a += qs[i] * bf_ld(kr + i);
      if (softcap > 0.f) a = softcap * tanhf(a / softcap);
      if (slopes) a += slopes[h] * (float)(j - p);
      if (log_slope) a -= log_slope[h] * log1pf(log_rate[h] * (float)(p - j));
      s = a;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float pj = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int c = 0; c < ATT_MAX_ACC; ++c) acc[c] *= corr;
    const unsigned live = __ballot_sync(0xffffffffu, valid);
    for (int jj = 0; jj < 32; ++jj) {
      if (!((live >> jj) & 1u)) continue;
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      const long long rb = __shfl_sync(0xffffffffu, row, jj);
      const A* vr = v_cache + rb * v_stride;
#pragma unroll
      for (int c = 0; c < ATT_MAX_ACC; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] += pb * bf_ld(vr + i);
      }
    }
  }
  if (sinks) {                                  // the sink: in the denominator only
    const float m_new = fmaxf(m, sinks[h]);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sinks[h] - m_new);
#pragma unroll
    for (int c = 0; c < ATT_MAX_ACC; ++c) acc[c] *= corr;
  }
  const float inv = out_scale / l;
  A* o = out + (size_t)t * out_stride + (size_t)h * dv;
#pragma unroll
  for (int c = 0; c < ATT_MAX_ACC; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) bf_st(o + i, acc[c] * inv);
  }
}

BF_EXPORT int bf_paged_attention_generic(
    const void* q, const void* k_cache, const void* v_cache, const int* seq_of_token,
    const int* positions, const int* block_tables, int table_stride, void* out, int T, int nh,
    int nkv, int d, int page_size, int num_pages, int window, float scale, float softcap,
    const float* slopes, const float* sinks, int act_dtype, int* err, int dv, int keep_first,
    long long q_stride, long long out_stride, float out_scale, long long v_stride,
    const float* log_slope, const float* log_rate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d > ATT_MAX_D || dv > 512 || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
  if (v_stride <= 0) v_stride = dv;
  if (!log_slope || !log_rate) log_slope = log_rate = nullptr;
  const int warps = 4;
  dim3 grid(T, (nh + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
#define ATT_GO(AT, ACC)                                                                        \
  paged_attention_generic_kernel<AT, ACC><<<grid, warps * 32, smem, stream>>>(                 \
      (const AT*)q, (const AT*)k_cache, (const AT*)v_cache, seq_of_token, positions,           \
      block_tables, table_stride, (AT*)out, nh, nkv, d, page_size, num_pages, window, scale,   \
      softcap, slopes, sinks, err, dv, keep_first, q_stride, out_stride, out_scale, v_stride,  \
      log_slope, log_rate)
  if (act_dtype == BF_DTYPE_F32) {
    if (dv <= 256) ATT_GO(float, 8); else ATT_GO(float, 16);
  } else {
    if (dv <= 256) ATT_GO(__nv_bfloat16, 8); else ATT_GO(__nv_bfloat16, 16);
  }
#undef ATT_GO
  return bf_launch_status();
}
