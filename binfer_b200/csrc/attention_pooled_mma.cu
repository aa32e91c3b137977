// Windowed attention with pooled blocks (see attention_pooled.cu for what it computes) on the
// tensor cores, bfloat16, for prompt portions and single tokens alike.
//
// A CTA of four warps takes 64 *rows* of one request and one key/value head: a row is a
// (token, query head of the group) pair, tokens in order and the group's heads side by side,
// so one tile of keys and values serves every head that shares it.  The CTA walks first the
// pooled blocks that its last row sees (64 block means a tile), then the tokens from the
// first row's window start to the last row's position (64 keys a tile, tile edges at
// multiples of 64).  Per tile: K and V rows come through the block table into shared
// memory, S = Q K^T by mma.sync m16n8k16 (Q fragments stay in registers), each row masks by
// its own position (a block is seen if it lies wholly before the row's window; a token if it
// is inside it), online softmax in float in base 2, P in bfloat16 straight from the
// accumulators into the A fragments of O += P V.  The epilogue adds the sink to the
// denominator, turns the head's output back by the row's position (values are cached
// turned by theirs), multiplies by the head's gate and stores.
//
// Two things for attention without pooled blocks: a window that keeps the request's first
// `keep_first` tokens (their tiles are walked between the blocks' and the window's, each
// row masking what its window covers anyway), and a learned sink logit per query head
// (`sinks`) in place of the constant one.  `q_stride`, `out_stride` and `out_scale` let q and
// the result be column blocks of wider buffers, the result scaled.  A soft cap c > 0 turns a
// scaled score z into c tanh(z / c) before the mask and the softmax.
//
// Key and value head sizes: multiples of 16 up to 128; at most 64 query heads per kv head.
#include <float.h>

#include "common.cuh"

#define PWM_ROWS 64
#define PWM_KEYS 64
#define PWM_THREADS 128

__device__ __forceinline__ void pwm_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pwm_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pwm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float pwm_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pwm_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ void pwm_cp16(void* smem, const void* gmem, bool valid) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;              // 0: nothing is read, the 16 bytes are zeroed
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sa), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void pwm_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N>
__device__ __forceinline__ void pwm_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// Which pieces (16 bytes each) of a 64-row tile a thread copies: row and column of each of
// its at most eight pieces, worked out once (row in the low byte, column above; -1: none).
struct PwmPieces {
  int rc[8];
};
__device__ __forceinline__ PwmPieces pwm_pieces(int d) {
  PwmPieces p;
  const int chunks = d >> 3, total = PWM_KEYS * chunks;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = threadIdx.x + PWM_THREADS * k;
    const int r = i / chunks;
    p.rc[k] = i < total ? (r | (((i - r * chunks) << 3) << 8)) : -1;
  }
  return p;
}

// Rows `first .. first + 63` (entries of a paged cache, through `table`) on their way into a
// shared tile of `d` columns and `pitch` elements a row, by asynchronous 16-byte copies; rows
// before `lo` or at or beyond `limit` are zeroed (their pages may be gone).  The pages of a
// thread's pieces are looked up first, all at once, so that the lookups' round trips overlap.
// `ps_shift`: log2 of the page size, or -1 if that is no power of two.
// (Not inlined: the tile loop's code must stay small enough for the instruction cache, which
// a single resident warp per scheduler cannot hide misses of.)
__device__ __noinline__ void pwm_load_tile(__nv_bfloat16* tile, int pitch, const PwmPieces& pc,
                                              const __nv_bfloat16* __restrict__ cache,
                                              const int* __restrict__ table, int first, int lo,
                                              int limit, int d, int nkv, int g, int page_size,
                                              int ps_shift, int num_pages,
                                              int* __restrict__ err) {
  int pages[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int e = first + (pc.rc[k] & 255);
    const bool want = pc.rc[k] >= 0 && e >= lo && e < limit;
    pages[k] = want ? table[ps_shift >= 0 ? e >> ps_shift : e / page_size] : -2;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (pc.rc[k] >= 0) {
      const int r = pc.rc[k] & 255, c = pc.rc[k] >> 8;
      const int e = first + r;
      const int page = pages[k];
      const bool ok = page >= 0 && page < num_pages;
      if (!ok && page != -2) atomicOr(err, BF_ERR_PAGE);
      const int off = ps_shift >= 0 ? e & (page_size - 1) : e % page_size;
      const __nv_bfloat16* src =
          ok ? cache + (((size_t)page * nkv + g) * page_size + off) * d + c : cache;
      pwm_cp16(tile + (size_t)r * pitch + c, src, ok);
    }
  }
}

// SPLIT: at most 16 rows (a single token's heads of a group, while decoding).  All four warps
// then take the same rows and every fourth key tile each, four tiles in flight at a time,
// and their partial results (maximum, sum, unnormalised output) are merged at the end.
template <int DKS, int DVT, bool SPLIT>   // key size <= 16 DKS, value size <= 8 DVT
__global__ void __launch_bounds__(PWM_THREADS) pwm_attention_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, const __nv_bfloat16* __restrict__ ks_cache,
    const __nv_bfloat16* __restrict__ vs_cache, const int* __restrict__ q_start,
    const int* __restrict__ positions, const int* __restrict__ tables, int table_stride,
    const int* __restrict__ s_tables, int s_table_stride, const __nv_bfloat16* __restrict__ gate,
    long long gate_stride, const float* __restrict__ v_inv_freq, int interleaved,
    __nv_bfloat16* __restrict__ out, int nh, int nkv, int dk, int dv, int page_size,
    int num_pages, int s_page_size, int s_num_pages, int window, int pool, float scale_log2,
    int has_sink, float sink_log2, float* __restrict__ part_o, float* __restrict__ part_ml,
    int* __restrict__ err, const float* __restrict__ sinks, int keep_first, long long q_stride,
    long long out_stride, float out_scale, float cap_pre, float cap_post,
    const float* __restrict__ log_slope, const float* __restrict__ log_rate, float inv_scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int pitch_k = dk + 8, pitch_v = dv + 8;
  // two stages of (K tile, V tile); the first K tile's place holds the Q tile to begin with
  const size_t stage_elems = (size_t)PWM_KEYS * (pitch_k + pitch_v);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);

  const int b = blockIdx.z, g = blockIdx.y;
  const int Gh = nh / nkv;
  const int t0 = q_start[b], n_tok = q_start[b + 1] - t0;
  const int rows_total = n_tok * Gh;
  // SPLIT with scratch for partial results: blockIdx.x is a share of the key tiles (four of
  // them), not a tile of rows; pwm_merge_kernel makes the shares one
  const bool shared_out = SPLIT && part_o != nullptr;
  const int row0 = shared_out ? 0 : blockIdx.x * PWM_ROWS;
  if (row0 >= rows_total) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wrow = SPLIT ? 0 : warp * 16;          // the warp's first row inside the tile
  const int* table = tables + (size_t)b * table_stride;
  const int* s_table = s_tables ? s_tables + (size_t)b * s_table_stride : nullptr;

  // the Q tile: row r is (token t0 + r / Gh, head g Gh + r % Gh)
  {
    const int chunks = dk >> 3;
    for (int i = threadIdx.x; i < PWM_ROWS * chunks; i += PWM_THREADS) {
      const int r = i / chunks, c = (i - r * chunks) << 3;
      const int row = row0 + r;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (row < rows_total) {
        const int tok = t0 + row / Gh, head = g * Gh + row % Gh;
        v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (size_t)head * dk + c);
      }
      *reinterpret_cast<uint4*>(Ks + (size_t)r * pitch_k + c) = v;
    }
  }
  __syncthreads();
  uint32_t qf[DKS][4];
#pragma unroll
  for (int ks = 0; ks < DKS; ++ks)
    if (ks * 16 < dk)
      pwm_ldmatrix_x4(qf[ks], Ks + (size_t)(wrow + (lane & 15)) * pitch_k + ks * 16 +
                                  (lane >> 4) * 8);
  __syncthreads();

  // this thread's two rows and their positions (-1: no such row)
  const int p_first = positions[t0];
  int my_p[2], my_j0[2], my_nb[2], my_kept[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wrow + (lane >> 2) + 8 * i;
    const int p = row < rows_total ? p_first + row / Gh : -1;
    my_p[i] = p;
    my_j0[i] = window > 0 ? max(0, p - window + 1) : 0;
    my_nb[i] = (window > 0 && pool > 0 && p - window + 1 > 0) ? (p - window + 1) / pool : 0;
    my_kept[i] = window > 0 ? min(keep_first, my_j0[i]) : 0;   // kept tokens behind the window
  }
  // a bias that grows with the logarithm of the distance, of this thread's two rows' heads:
  // slope over the scale (the scores stay unscaled until the exponent), and rate
  float lb_slope[2] = {0.f, 0.f}, lb_rate[2] = {0.f, 0.f};
  if (log_slope) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = min(row0 + wrow + (lane >> 2) + 8 * i, rows_total - 1);
      lb_slope[i] = log_slope[g * Gh + row % Gh] * inv_scale;
      lb_rate[i] = log_rate[g * Gh + row % Gh];
    }
  }
  const int last_row = min(rows_total, row0 + PWM_ROWS) - 1;
  const int p_lo = p_first + row0 / Gh, p_hi = p_first + last_row / Gh;
  const int nb_hi = (window > 0 && pool > 0 && s_table && p_hi - window + 1 > 0)
                        ? (p_hi - window + 1) / pool : 0;
  const int block_tiles = (nb_hi + PWM_KEYS - 1) / PWM_KEYS;
  const int j_lo = window > 0 ? max(0, p_lo - window + 1) : 0;     // the first key any row sees
  const int first_tile = j_lo / PWM_KEYS;
  const int token_tiles = p_hi / PWM_KEYS - first_tile + 1;
  const int kept_hi = window > 0 ? min(keep_first, max(0, p_hi - window + 1)) : 0;
  const int kept_tiles = (kept_hi + PWM_KEYS - 1) / PWM_KEYS;

  float m[2] = {-1e30f, -1e30f}, l[2] = {0.f, 0.f};
  float o[DVT][4];
#pragma unroll
  for (int n = 0; n < DVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  const int n_tiles = block_tiles + kept_tiles + token_tiles;
  if (shared_out && 4 * (int)blockIdx.x >= n_tiles) return;
  const PwmPieces pk = pwm_pieces(dk), pv = pwm_pieces(dv);
  const int ps_shift = (page_size & (page_size - 1)) ? -1 : 31 - __clz(page_size);
  const int sps_shift = (s_page_size & (s_page_size - 1)) ? -1 : 31 - __clz(s_page_size);
  auto issue = [&](int it, int stage) {           // tile `it` on its way into a stage
    __nv_bfloat16* kt = Ks + (size_t)stage * stage_elems;
    __nv_bfloat16* vt = kt + (size_t)PWM_KEYS * pitch_k;
    const bool bl = it < block_tiles;
    const bool kp = !bl && it < block_tiles + kept_tiles;
    const int base = bl ? it * PWM_KEYS
                        : (kp ? (it - block_tiles) * PWM_KEYS
                              : (first_tile + it - block_tiles - kept_tiles) * PWM_KEYS);
    const int* tb = bl ? s_table : table;
    const int lo = (bl || kp) ? 0 : j_lo, limit = bl ? nb_hi : (kp ? kept_hi : p_hi + 1);
    const int ps = bl ? s_page_size : page_size, sh = bl ? sps_shift : ps_shift;
    const int np = bl ? s_num_pages : num_pages;
    pwm_load_tile(kt, pitch_k, pk, bl ? ks_cache : k_cache, tb, base, lo, limit, dk, nkv, g, ps,
                  sh, np, err);
    pwm_load_tile(vt, pitch_v, pv, bl ? vs_cache : v_cache, tb, base, lo, limit, dv, nkv, g, ps,
                  sh, np, err);
  };
  if (!SPLIT) {
    issue(0, 0);
    pwm_commit();
  }
  const int g_first = shared_out ? 4 * blockIdx.x : 0;
  const int g_end = shared_out ? min(n_tiles, g_first + 4) : n_tiles;
  for (int g0 = g_first; g0 < g_end; g0 += SPLIT ? 4 : 1) {
    int it, stage;
    if (SPLIT) {                                  // four tiles at a time, one a warp
#pragma unroll 1
      for (int x = 0; x < 4; ++x)
        if (g0 + x < n_tiles) issue(g0 + x, x);
      pwm_commit();
      pwm_wait<0>();
      it = g0 + warp;
      stage = warp;
    } else {
      if (g0 + 1 < n_tiles) issue(g0 + 1, (g0 + 1) & 1);   // travels while this one is used
      pwm_commit();
      pwm_wait<1>();
      it = g0;
      stage = g0 & 1;
    }
    __syncthreads();
    if (it < n_tiles) {
    const bool blocks = it < block_tiles;
    const bool keptt = !blocks && it < block_tiles + kept_tiles;
    const int base = blocks ? it * PWM_KEYS
                            : (keptt ? (it - block_tiles) * PWM_KEYS
                                     : (first_tile + it - block_tiles - kept_tiles) * PWM_KEYS);
    const __nv_bfloat16* Kt = Ks + (size_t)stage * stage_elems;
    const __nv_bfloat16* Vs = Kt + (size_t)PWM_KEYS * pitch_k;

    float s[PWM_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < PWM_KEYS / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < DKS; ++ks) {
      if (ks * 16 < dk) {
#pragma unroll
        for (int np = 0; np < PWM_KEYS / 16; ++np) {
          uint32_t kb[4];
          pwm_ldmatrix_x4(kb, Kt + (size_t)(np * 16 + (lane & 7) + ((lane >> 4) << 3)) * pitch_k +
                                  ks * 16 + ((lane >> 3) & 1) * 8);
          pwm_mma(s[2 * np], qf[ks], kb[0], kb[1]);
          pwm_mma(s[2 * np + 1], qf[ks], kb[2], kb[3]);
        }
      }
    }
    if (cap_pre > 0.f) {       // s <- (c / scale) tanh(s scale / c): the scale still rides below
#pragma unroll
      for (int n = 0; n < PWM_KEYS / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // tanh z = 1 - 2 / (exp(2 z) + 1): right at both ends, where the power is 0 or inf
          float t;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(s[n][e] * cap_pre));
          s[n][e] = cap_post - __fdividef(2.f * cap_post, t + 1.f);
        }
    }
    if (log_slope && !blocks) {  // s <- s - (b1 / scale) ln(1 + b2 (p - j)), keys at their places
#pragma unroll
      for (int n = 0; n < PWM_KEYS / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int kj = base + n * 8 + 2 * (lane & 3) + (e & 1);
          const float dist = (float)max(my_p[i] - kj, 0);
          s[n][e] -= lb_slope[i] * __logf(fmaf(lb_rate[i], dist, 1.f));
        }
    }
    // Each row masks by its own position; a tile that every row of this warp sees whole (the
    // common case inside a window) skips the tests.  Scores stay unscaled: the scale rides on
    // the exponent's multiply-add.
    const int w_first = min(row0 + wrow, rows_total - 1), w_last = min(row0 + wrow + 15,
                                                                       rows_total - 1);
    const int wp_lo = p_first + w_first / Gh, wp_hi = p_first + w_last / Gh;
    const bool whole_rows = row0 + wrow + 15 < rows_total;
    const bool whole_tile =
        whole_rows && (blocks ? base + PWM_KEYS <= ((window > 0 && pool > 0 && wp_lo - window + 1 > 0)
                                                        ? (wp_lo - window + 1) / pool : 0)
                    : keptt ? base + PWM_KEYS <= (window > 0 ? min(keep_first, max(0, wp_lo - window + 1)) : 0)
                              : (base >= (window > 0 ? max(0, wp_hi - window + 1) : 0) &&
                                 base + PWM_KEYS - 1 <= wp_lo));
    float mx[2] = {-1e30f, -1e30f};
    unsigned valid[2] = {0xffffu, 0xffffu};       // bit n*2+e: column n*8 + 2*(lane%4) + e
    if (whole_tile) {
#pragma unroll
      for (int n = 0; n < PWM_KEYS / 8; ++n) {
        mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
      }
    } else {
      valid[0] = valid[1] = 0u;
#pragma unroll
      for (int n = 0; n < PWM_KEYS / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int kj = base + n * 8 + 2 * (lane & 3) + (e & 1);
          const bool ok = blocks ? kj < my_nb[i]
                                 : (keptt ? kj < my_kept[i] : (kj >= my_j0[i] && kj <= my_p[i]));
          if (ok) {
            valid[i] |= 1u << (n * 2 + (e & 1));
            mx[i] = fmaxf(mx[i], s[n][e]);
          }
        }
      }
    }
    float corr[2], m_scaled[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      // m holds the running maximum of the scaled scores (the scale is positive)
      const float m_new = fmaxf(m[i], mx[i] > -1e29f ? mx[i] * scale_log2 : -1e30f);
      corr[i] = pwm_ex2(m[i] - m_new);
      m[i] = m_new;
      m_scaled[i] = -m_new;
      l[i] *= corr[i];
    }
#pragma unroll
    for (int n = 0; n < DVT; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
#pragma unroll
    for (int n = 0; n < PWM_KEYS / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        float pv = pwm_ex2(fmaf(s[n][e], scale_log2, m_scaled[i]));
        if (!whole_tile && !((valid[i] >> (n * 2 + (e & 1))) & 1u)) pv = 0.f;
        s[n][e] = pv;
        l[i] += pv;
      }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < PWM_KEYS / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pwm_pack(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pwm_pack(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pwm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pwm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < DVT / 2; ++np) {
        if (np * 16 < dv) {
          uint32_t vb[4];
          pwm_ldmatrix_x4_trans(vb, Vs + (size_t)(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) *
                                             pitch_v + np * 16 + (lane >> 4) * 8);
          pwm_mma(o[2 * np], pa, vb[0], vb[1]);
          pwm_mma(o[2 * np + 1], pa, vb[2], vb[3]);
        }
      }
    }
    }
    __syncthreads();
  }

  pwm_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  if (SPLIT) {
    // the four warps' partial results of the same 16 rows become one: through shared memory
    // (the tiles are done with), every warp then holds the merged rows
    float* Ow = reinterpret_cast<float*>(smem_raw);               // [4][16][dv]
    float* Mw = Ow + 4 * 16 * dv;                                 // [4][16]
    float* Lw = Mw + 4 * 16;                                      // [4][16]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (lane >> 2) + 8 * i;
      if ((lane & 3) == 0) {
        Mw[warp * 16 + r] = m[i];
        Lw[warp * 16 + r] = l[i];
      }
#pragma unroll
      for (int n = 0; n < DVT; ++n)
        if (n * 8 < dv)
          *reinterpret_cast<float2*>(Ow + ((size_t)warp * 16 + r) * dv + n * 8 + 2 * (lane & 3)) =
              make_float2(o[n][2 * i], o[n][2 * i + 1]);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (lane >> 2) + 8 * i;
      float mm = -1e30f;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, Mw[w * 16 + r]);
      float f[4], ll = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        f[w] = pwm_ex2(Mw[w * 16 + r] - mm);
        ll += Lw[w * 16 + r] * f[w];
      }
      m[i] = mm;
      l[i] = ll;
#pragma unroll
      for (int n = 0; n < DVT; ++n) {
        if (n * 8 < dv) {
          float2 acc = make_float2(0.f, 0.f);
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float2 x = *reinterpret_cast<const float2*>(
                Ow + ((size_t)w * 16 + r) * dv + n * 8 + 2 * (lane & 3));
            acc.x += x.x * f[w];
            acc.y += x.y * f[w];
          }
          o[n][2 * i] = acc.x;
          o[n][2 * i + 1] = acc.y;
        }
      }
    }
    __syncthreads();
    if (shared_out) {                             // this share's maximum, sum and raw output
      if (warp == 0) {
        const size_t at = ((size_t)b * nkv + g) * gridDim.x + blockIdx.x;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int r = (lane >> 2) + 8 * i;
          if ((lane & 3) == 0) {
            part_ml[(at * 16 + r) * 2] = m[i];
            part_ml[(at * 16 + r) * 2 + 1] = l[i];
          }
#pragma unroll
          for (int n = 0; n < DVT; ++n)
            if (n * 8 < dv)
              *reinterpret_cast<float2*>(part_o + (at * 16 + r) * dv + n * 8 + 2 * (lane & 3)) =
                  make_float2(o[n][2 * i], o[n][2 * i + 1]);
        }
      }
      return;
    }
  }
  // the denominator (with the sink), the turn back, the gate, the store
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (has_sink) {
      float sk = sink_log2;
      if (sinks) {                                // a learned logit per query head
        const int row = min(row0 + wrow + (lane >> 2) + 8 * i, rows_total - 1);
        sk = sinks[g * Gh + row % Gh] * 1.4426950408889634f;
      }
      const float m_new = fmaxf(m[i], sk);
      const float c = exp2f(m[i] - m_new);
      l[i] = l[i] * c + exp2f(sk - m_new);
#pragma unroll
      for (int n = 0; n < DVT; ++n) {
        o[n][2 * i] *= c;
        o[n][2 * i + 1] *= c;
      }
    }
  }
  // normalised rows to shared memory (the key and value tiles are done with) ...
  float* Os = reinterpret_cast<float*>(smem_raw);                 // [64][dv]
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = wrow + (lane >> 2) + 8 * i;     // (SPLIT: every warp writes the same values)
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
    for (int n = 0; n < DVT; ++n) {
      if (n * 8 < dv)
        *reinterpret_cast<float2*>(Os + (size_t)r * dv + n * 8 + 2 * (lane & 3)) =
            make_float2(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
  }
  __syncthreads();
  // ... then pair by pair: turned back by the row's position, times the head's gate
  const int half = dv >> 1;
  for (int idx = threadIdx.x; idx < PWM_ROWS * half; idx += PWM_THREADS) {
    const int r = idx / half, mi = idx - r * half;
    const int row = row0 + r;
    if (row >= rows_total) break;
    const int tok = t0 + row / Gh, head = g * Gh + row % Gh;
    const int iu = interleaved ? 2 * mi : mi, iv = interleaved ? 2 * mi + 1 : mi + half;
    float u = Os[(size_t)r * dv + iu], v = Os[(size_t)r * dv + iv];
    if (v_inv_freq) {
      float sn, cs;
      sincosf((float)(p_first + row / Gh) * v_inv_freq[mi], &sn, &cs);
      const float a = u * cs + v * sn, c = v * cs - u * sn;
      u = a;
      v = c;
    }
    float gt = 1.f;
    if (gate) gt = 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)tok * gate_stride + head])));
    gt *= out_scale;
    __nv_bfloat16* dst = out + (size_t)tok * out_stride + (size_t)head * dv;
    dst[iu] = __float2bfloat16_rn(u * gt);
    dst[iv] = __float2bfloat16_rn(v * gt);
  }
}

// The shares of a row's keys (pwm_attention_kernel with scratch) made one: the maxima, sums and
// raw outputs of the shares that exist for the request's position are combined in ascending
// order, then the sink, the turn back and the gate as in the kernel's own epilogue.
// grid (kv head, request); shares: how many the scratch has room for.
__global__ void pwm_merge_kernel(
    const float* __restrict__ part_o, const float* __restrict__ part_ml, int shares,
    const int* __restrict__ q_start, const int* __restrict__ positions,
    const __nv_bfloat16* __restrict__ gate, long long gate_stride,
    const float* __restrict__ v_inv_freq, int interleaved, __nv_bfloat16* __restrict__ out,
    int nh, int nkv, int dv, int window, int pool, int has_summary, int has_sink,
    float sink_log2, const float* __restrict__ sinks, int keep_first, long long out_stride,
    float out_scale) {
  __shared__ float wgt[32][16];                   // share x, row r: exp2(m_x - M) / L
  const int g = blockIdx.x, b = blockIdx.y;
  const int Gh = nh / nkv;
  const int t0 = q_start[b], n_tok = q_start[b + 1] - t0;
  const int rows_total = n_tok * Gh;
  const int p_first = positions[t0];
  const int p_hi = p_first + (rows_total - 1) / Gh;
  const int nb_hi = (window > 0 && pool > 0 && has_summary && p_hi - window + 1 > 0)
                        ? (p_hi - window + 1) / pool : 0;
  const int j_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int kept_hi = window > 0 ? min(keep_first, max(0, p_hi - window + 1)) : 0;
  const int n_tiles = (nb_hi + PWM_KEYS - 1) / PWM_KEYS + (kept_hi + PWM_KEYS - 1) / PWM_KEYS +
                      p_hi / PWM_KEYS - j_lo / PWM_KEYS + 1;
  const int n_shares = min(shares, (n_tiles + 3) / 4);
  const size_t at = ((size_t)b * nkv + g) * shares;
  if (threadIdx.x < 16) {
    const int r = threadIdx.x;
    if (sinks) sink_log2 = sinks[g * Gh + min(r, max(rows_total - 1, 0)) % Gh] * 1.4426950408889634f;
    float M = has_sink ? sink_log2 : -1e30f;
    for (int x = 0; x < n_shares; ++x) M = fmaxf(M, part_ml[((at + x) * 16 + r) * 2]);
    float L = has_sink ? pwm_ex2(sink_log2 - M) : 0.f;
    for (int x = 0; x < n_shares; ++x)
      L += part_ml[((at + x) * 16 + r) * 2 + 1] * pwm_ex2(part_ml[((at + x) * 16 + r) * 2] - M);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int x = 0; x < n_shares; ++x)
      wgt[x][r] = pwm_ex2(part_ml[((at + x) * 16 + r) * 2] - M) * inv;
  }
  __syncthreads();
  const int half = dv >> 1;
  for (int idx = threadIdx.x; idx < rows_total * half; idx += blockDim.x) {
    const int r = idx / half, mi = idx - r * half;
    const int tok = t0 + r / Gh, head = g * Gh + r % Gh;
    const int iu = interleaved ? 2 * mi : mi, iv = interleaved ? 2 * mi + 1 : mi + half;
    float u = 0.f, v = 0.f;
    for (int x = 0; x < n_shares; ++x) {
      const float* o = part_o + ((at + x) * 16 + r) * dv;
      u += o[iu] * wgt[x][r];
      v += o[iv] * wgt[x][r];
    }
    if (v_inv_freq) {
      float sn, cs;
      sincosf((float)(p_first + r / Gh) * v_inv_freq[mi], &sn, &cs);
      const float a = u * cs + v * sn, c = v * cs - u * sn;
      u = a;
      v = c;
    }
    float gt = 1.f;
    if (gate) gt = 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)tok * gate_stride + head])));
    gt *= out_scale;
    __nv_bfloat16* dst = out + (size_t)tok * out_stride + (size_t)head * dv;
    dst[iu] = __float2bfloat16_rn(u * gt);
    dst[iv] = __float2bfloat16_rn(v * gt);
  }
}

// max_rows: the most rows (tokens x heads of a group) that one request brings to this step.
BF_EXPORT int bf_pwm_attention(
    const void* q, const void* k_cache, const void* v_cache, const void* ks_cache,
    const void* vs_cache, const int* q_start, const int* positions, const int* tables,
    int table_stride, const int* s_tables, int s_table_stride, const void* gate,
    long long gate_stride, const float* v_inv_freq, int interleaved, void* out, int B,
    int max_tokens, int nh, int nkv, int dk, int dv, int page_size, int num_pages,
    int s_page_size, int s_num_pages, int window, int pool, float scale, int has_sink,
    float sink, float* part_o, float* part_ml, int shares, int* err, const float* sinks,
    int keep_first, long long q_stride, long long out_stride, float out_scale, float softcap,
    const float* log_slope, const float* log_rate, cudaStream_t stream) {
  // log_slope, log_rate [nh] (both or neither): b1_h ln(1 + b2_h (p - j)) is taken off the
  // scaled score of the query at p and the key at j (not with pooled blocks)
  // part_o [B, nkv, shares, 16, dv], part_ml [B, nkv, shares, 16, 2] (float, or null): scratch
  // for steps of single tokens, whose keys are then shared out over `shares` CTAs a row
  if (B <= 0 || max_tokens <= 0) return 0;
  if (dk % 16 || dv % 16 || dk > 128 || dv > 128 || nkv <= 0 || nh % nkv || nh / nkv > 64)
    return (int)cudaErrorInvalidValue;
  if (pool > 0 && window > 0 && !ks_cache) return (int)cudaErrorInvalidValue;
  if (!(scale > 0.f)) return (int)cudaErrorInvalidValue;     // the running maximum relies on it
  if (!log_slope || !log_rate) log_slope = log_rate = nullptr;
  if (log_slope && ks_cache) return (int)cudaErrorInvalidValue;
  const int Gh = nh / nkv;
  dim3 grid((max_tokens * Gh + PWM_ROWS - 1) / PWM_ROWS, nkv, B);
  const bool split = max_tokens * Gh <= 16;       // single tokens: the keys shared out over warps
  const bool multi = split && part_o && part_ml && shares > 1 && shares <= 32;
  if (multi) grid.x = shares;
  else part_o = part_ml = nullptr;
  size_t smem = (split ? 4 : 2) * (size_t)PWM_KEYS * ((dk + 8) + (dv + 8)) * sizeof(__nv_bfloat16);
  if (smem < (size_t)PWM_ROWS * dv * sizeof(float) + 512)
    smem = (size_t)PWM_ROWS * dv * sizeof(float) + 512;
  const float log2e = 1.4426950408889634f;
  auto kern = split ? pwm_attention_kernel<8, 16, true> : pwm_attention_kernel<8, 16, false>;
  static bool configured[BF_MAX_DEVICES][2];
  const int dev = bf_current_device();
  if (!configured[dev][split]) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (split ? 4 : 2) * PWM_KEYS * (136 + 136) * 2);
    if (e != cudaSuccess) return (int)e;
    configured[dev][split] = true;
  }
  kern<<<grid, PWM_THREADS, smem, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
      (const __nv_bfloat16*)ks_cache, (const __nv_bfloat16*)vs_cache, q_start, positions, tables,
      table_stride, s_tables, s_table_stride, (const __nv_bfloat16*)gate, gate_stride, v_inv_freq,
      interleaved, (__nv_bfloat16*)out, nh, nkv, dk, dv, page_size, num_pages, s_page_size,
      s_num_pages, window, pool, scale * log2e, has_sink, sink * log2e, part_o, part_ml, err,
      sinks, keep_first, q_stride, out_stride, out_scale,
      softcap > 0.f ? 2.f * log2e * scale / softcap : 0.f, softcap > 0.f ? softcap / scale : 0.f,
      log_slope, log_rate, 1.f / scale);
  if (multi) {
    const int e = bf_launch_status();
    if (e) return e;
    pwm_merge_kernel<<<dim3(nkv, B), 128, 0, stream>>>(
        part_o, part_ml, shares, q_start, positions, (const __nv_bfloat16*)gate, gate_stride,
        v_inv_freq, interleaved, (__nv_bfloat16*)out, nh, nkv, dv, window, pool,
        ks_cache != nullptr, has_sink, sink * log2e, sinks, keep_first, out_stride, out_scale);
  }
  return bf_launch_status();
}
