// Attention over a cached latent on the tensor cores (bfloat16), for prompt portions and
// single tokens alike.
//
// Every token's cache row is [latent (rank numbers) | shared rotated key part (dr numbers)],
// W = rank + dr numbers, one "head" per token; a query head arrives in the same coordinates
// (its plain part carried into the latent's by a product elsewhere), so all heads of a token
// read the same keys, and a key row's first `rank` numbers are also the value.  A *row* is a
// (token, head) pair, tokens in order and a token's heads side by side: q [T * H, W],
// out [T * H, rank], both contiguous.
//
// A CTA of eight warps takes 32 rows of one request (two tiles of 16) and walks the keys from
// position 0 to its last row's position, 64 keys a tile (tile edges at multiples of 64, two
// buffers: the next tile's asynchronous copies travel while this one is used).  A key tile is
// fetched once and serves as K and as V.  Warp (mt, qt) holds rows 16 mt .. 16 mt + 15:
//   S = Q K^T for the tile's keys 16 qt .. 16 qt + 15 over all W sizes (mma.sync m16n8k16, Q
//   and K fragments by ldmatrix from shared memory),
//   the rows' maxima over the four warps of a row tile through shared memory, the softmax in
//   float in base 2, P in bfloat16 into shared memory,
//   O += P V for every fourth pair of 8-column value tiles (pairs qt, qt + 4, ...).
// Each row masks by its own token's position.  With `splits` > 1 (steps of single tokens) the
// key tiles of a request are shared out over that many CTAs, whose maxima, sums and raw
// outputs a second kernel makes one.
//
// Sizes: rank and dr multiples of 16, rank at most 512, W at most 640.
#include "common.cuh"
#include "mma_utils.cuh"

#define LAT_ROWS 32
#define LAT_KEYS 64
#define LAT_THREADS 256
#define LAT_PP (LAT_KEYS + 8)      // pitch of the P tile

__device__ __forceinline__ float lat_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Keys `first .. first + 63` of a request (through its block table) on their way into a
// shared tile; keys beyond `last` are zeroed.
__device__ __forceinline__ void lat_load_tile(__nv_bfloat16* tile, int pitch,
                                              const __nv_bfloat16* __restrict__ cache,
                                              const int* __restrict__ table, int first, int last,
                                              int W, int page_size, int num_pages,
                                              int* __restrict__ err) {
  // a warp a key row at a time: the page is looked up once per row, the lanes share the
  // row's 16-byte pieces out
  const int chunks = W >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < LAT_KEYS; r += LAT_THREADS / 32) {
    const int e = first + r;
    bool ok = e <= last;
    const __nv_bfloat16* src = cache;
    if (ok) {
      const int lp = e / page_size;
      const int page = table[lp];
      if (page < 0 || page >= num_pages) {
        if (lane == 0) atomicOr(err, BF_ERR_PAGE);
        ok = false;
      } else {
        src = cache + ((size_t)page * page_size + (e - lp * page_size)) * W;
      }
    }
    __nv_bfloat16* dst = tile + (size_t)r * pitch;
    for (int c = lane; c < chunks; c += 32)
      cp_async16(dst + 8 * c, ok ? src + 8 * c : cache, ok ? 16 : 0);
  }
}

template <int NP>      // pairs of 8-column value tiles a warp holds: rank <= 64 NP
__global__ void __launch_bounds__(LAT_THREADS) latent_attention_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
    const int* __restrict__ q_start, const int* __restrict__ positions,
    const int* __restrict__ tables, int table_stride, __nv_bfloat16* __restrict__ out, int H,
    int W, int rank, int page_size, int num_pages, float scale_log2, float* __restrict__ part_o,
    float* __restrict__ part_ml, int splits, int* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char lat_smem[];
  const int pitch = W + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lat_smem);       // [32][pitch]
  __nv_bfloat16* Ks = Qs + (size_t)LAT_ROWS * pitch;                     // [2][64][pitch]
  __nv_bfloat16* Ps = Ks + (size_t)2 * LAT_KEYS * pitch;                 // [32][LAT_PP]
  float* red = reinterpret_cast<float*>(Ps + LAT_ROWS * LAT_PP);         // [2][4][16]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mt = warp >> 2, qt = warp & 3;
  const int b = blockIdx.y, row0 = blockIdx.x * LAT_ROWS;
  const int t0 = q_start[b], n_tok = q_start[b + 1] - t0;
  const int rows_total = n_tok * H;
  if (row0 >= rows_total) return;
  const int* table = tables + (size_t)b * table_stride;
  const int p_hi = positions[t0 + min(row0 + LAT_ROWS - 1, rows_total - 1) / H];
  const int n_tiles = p_hi / LAT_KEYS + 1;
  int tile_a = 0, tile_b = n_tiles;
  if (splits > 1) {
    const int per = (n_tiles + splits - 1) / splits;
    tile_a = min(n_tiles, (int)blockIdx.z * per);
    tile_b = min(n_tiles, tile_a + per);
  }
  // this lane's two rows (of the accumulator layout) and their positions; -1: no such row
  const int rA = row0 + mt * 16 + (lane >> 2), rB = rA + 8;
  const int pA = rA < rows_total ? positions[t0 + rA / H] : -1;
  const int pB = rB < rows_total ? positions[t0 + rB / H] : -1;
  const bool active = row0 + mt * 16 < rows_total;

  {
    const int chunks = W >> 3;
    for (int i = tid; i < LAT_ROWS * chunks; i += LAT_THREADS) {
      const int r = i / chunks, c = (i - r * chunks) << 3;
      const bool ok = row0 + r < rows_total;
      cp_async16(Qs + (size_t)r * pitch + c,
                 ok ? q + ((size_t)t0 * H + row0 + r) * W + c : q, ok ? 16 : 0);
    }
  }
  if (tile_a < tile_b)
    lat_load_tile(Ks, pitch, cache, table, tile_a * LAT_KEYS, p_hi, W, page_size, num_pages, err);
  cp_async_commit();

  float m[2] = {-1e30f, -1e30f}, l[2] = {0.f, 0.f};
  float o[2 * NP][4];
#pragma unroll
  for (int n = 0; n < 2 * NP; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int it = tile_a; it < tile_b; ++it) {
    const int buf = (it - tile_a) & 1;
    cp_async_wait<0>();
    __syncthreads();                      // the tile is here; the other buffer is used up
    if (it + 1 < tile_b)
      lat_load_tile(Ks + (size_t)(buf ^ 1) * LAT_KEYS * pitch, pitch, cache, table,
                    (it + 1) * LAT_KEYS, p_hi, W, page_size, num_pages, err);
    cp_async_commit();
    const __nv_bfloat16* Kt = Ks + (size_t)buf * LAT_KEYS * pitch;
    const int base = it * LAT_KEYS;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (active) {
      const __nv_bfloat16* qa = Qs + (size_t)(mt * 16 + (lane & 15)) * pitch + (lane >> 4) * 8;
      const __nv_bfloat16* kb_ = Kt + (size_t)(qt * 16 + (lane & 7) + ((lane >> 4) << 3)) * pitch +
                                 ((lane >> 3) & 1) * 8;
      // two sets of accumulators take alternate steps of 16 sizes, so that a product does
      // not wait for the one before it; W is a multiple of 16, the odd last step goes to
      // the first set
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      int ks = 0;
#pragma unroll 2
      for (; ks + 32 <= W; ks += 32) {
        unsigned a[4], kb[4], a2[4], kb2[4];
        ldmatrix_x4(a, qa + ks);
        ldmatrix_x4(kb, kb_ + ks);
        ldmatrix_x4(a2, qa + ks + 16);
        ldmatrix_x4(kb2, kb_ + ks + 16);
        mma_bf16_16816(s[0], a, kb[0], kb[1]);
        mma_bf16_16816(s[1], a, kb[2], kb[3]);
        mma_bf16_16816(s2[0], a2, kb2[0], kb2[1]);
        mma_bf16_16816(s2[1], a2, kb2[2], kb2[3]);
      }
      if (ks < W) {
        unsigned a[4], kb[4];
        ldmatrix_x4(a, qa + ks);
        ldmatrix_x4(kb, kb_ + ks);
        mma_bf16_16816(s[0], a, kb[0], kb[1]);
        mma_bf16_16816(s[1], a, kb[2], kb[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] += s2[nt][e];
    }
    // mask by each row's own position; the rows' maxima over this warp's keys
    float mx[2] = {-1e30f, -1e30f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int kj = base + qt * 16 + nt * 8 + 2 * (lane & 3) + (e & 1);
        if (kj <= (i ? pB : pA)) mx[i] = fmaxf(mx[i], s[nt][e]);
        else s[nt][e] = -1e30f;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    if ((lane & 3) == 0) {
      red[(mt * 4 + qt) * 16 + (lane >> 2)] = mx[0];
      red[(mt * 4 + qt) * 16 + (lane >> 2) + 8] = mx[1];
    }
    __syncthreads();
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (lane >> 2) + 8 * i;
      const float all = fmaxf(fmaxf(red[(mt * 4 + 0) * 16 + r], red[(mt * 4 + 1) * 16 + r]),
                              fmaxf(red[(mt * 4 + 2) * 16 + r], red[(mt * 4 + 3) * 16 + r]));
      // m holds the running maximum of the scaled scores (the scale is positive)
      const float m_new = fmaxf(m[i], all > -1e29f ? all * scale_log2 : -1e30f);
      corr[i] = lat_ex2(m[i] - m_new);
      m[i] = m_new;
      l[i] *= corr[i];
    }
#pragma unroll
    for (int n = 0; n < 2 * NP; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        p[e] = s[nt][e] > -1e29f ? lat_ex2(fmaf(s[nt][e], scale_log2, -m[i])) : 0.f;
        l[i] += p[e];
      }
      __nv_bfloat16* pr = Ps + (size_t)(mt * 16 + (lane >> 2)) * LAT_PP + qt * 16 + nt * 8 +
                          2 * (lane & 3);
      *reinterpret_cast<unsigned*>(pr) = pack_bf16(p[0], p[1]);
      *reinterpret_cast<unsigned*>(pr + 8 * LAT_PP) = pack_bf16(p[2], p[3]);
    }
    __syncthreads();
    if (active) {
#pragma unroll
      for (int kk = 0; kk < LAT_KEYS / 16; ++kk) {
        unsigned pa[4];
        ldmatrix_x4(pa, Ps + (size_t)(mt * 16 + (lane & 15)) * LAT_PP + kk * 16 + (lane >> 4) * 8);
        const __nv_bfloat16* vrow =
            Kt + (size_t)(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * pitch + (lane >> 4) * 8;
#pragma unroll
        for (int np = 0; np < NP; ++np) {
          const int pair = qt + 4 * np;
          if (pair * 16 < rank) {
            unsigned vb[4];
            ldmatrix_x4_trans(vb, vrow + pair * 16);
            mma_bf16_16816(o[2 * np], pa, vb[0], vb[1]);
            mma_bf16_16816(o[2 * np + 1], pa, vb[2], vb[3]);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // the rows' sums: over this lane's quad, then over the four warps of the row tile
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  if ((lane & 3) == 0) {
    red[(mt * 4 + qt) * 16 + (lane >> 2)] = l[0];
    red[(mt * 4 + qt) * 16 + (lane >> 2) + 8] = l[1];
  }
  __syncthreads();
  float L[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (lane >> 2) + 8 * i;
    L[i] = ((red[(mt * 4 + 0) * 16 + r] + red[(mt * 4 + 1) * 16 + r]) +
            red[(mt * 4 + 2) * 16 + r]) + red[(mt * 4 + 3) * 16 + r];
  }
  if (splits > 1) {
    // raw sums, maxima and outputs of this share of the keys
    const size_t at = (((size_t)b * gridDim.x + blockIdx.x) * splits + blockIdx.z) * LAT_ROWS;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = mt * 16 + (lane >> 2) + 8 * i;
      if (qt == 0 && (lane & 3) == 0) {
        part_ml[(at + r) * 2] = m[i];
        part_ml[(at + r) * 2 + 1] = L[i];
      }
#pragma unroll
      for (int np = 0; np < NP; ++np) {
        const int pair = qt + 4 * np;
        if (pair * 16 >= rank) continue;
#pragma unroll
        for (int h8 = 0; h8 < 2; ++h8) {
          const int c = pair * 16 + h8 * 8 + 2 * (lane & 3);
          float* dst = part_o + (at + r) * rank + c;
          dst[0] = o[2 * np + h8][2 * i];
          dst[1] = o[2 * np + h8][2 * i + 1];
        }
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row0 + mt * 16 + (lane >> 2) + 8 * i;
    if (r >= rows_total) continue;
    const float inv = L[i] > 0.f ? 1.f / L[i] : 0.f;
    __nv_bfloat16* dst = out + ((size_t)t0 * H + r) * rank;
#pragma unroll
    for (int np = 0; np < NP; ++np) {
      const int pair = qt + 4 * np;
      if (pair * 16 >= rank) continue;
#pragma unroll
      for (int h8 = 0; h8 < 2; ++h8) {
        const int c = pair * 16 + h8 * 8 + 2 * (lane & 3);
        *reinterpret_cast<unsigned*>(dst + c) =
            pack_bf16(o[2 * np + h8][2 * i] * inv, o[2 * np + h8][2 * i + 1] * inv);
      }
    }
  }
}

// The shares of a row's keys made one, in ascending order.  grid (row, row tile, request).
__global__ void latent_merge_kernel(const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, int splits,
                                    const int* __restrict__ q_start,
                                    __nv_bfloat16* __restrict__ out, int H, int rank) {
  const int r = blockIdx.x, tile = blockIdx.y, b = blockIdx.z;
  const int t0 = q_start[b], rows_total = (q_start[b + 1] - t0) * H;
  const int row = tile * LAT_ROWS + r;
  if (row >= rows_total) return;
  const size_t at = ((size_t)b * gridDim.y + tile) * splits * LAT_ROWS;
  float M = -1e30f;
  for (int x = 0; x < splits; ++x) M = fmaxf(M, part_ml[(at + (size_t)x * LAT_ROWS + r) * 2]);
  float Lsum = 0.f;
  for (int x = 0; x < splits; ++x) {
    const float* ml = part_ml + (at + (size_t)x * LAT_ROWS + r) * 2;
    Lsum += ml[1] * lat_ex2(ml[0] - M);
  }
  const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
  __nv_bfloat16* dst = out + ((size_t)t0 * H + row) * rank;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.f;
    for (int x = 0; x < splits; ++x) {
      const size_t px = at + (size_t)x * LAT_ROWS + r;
      acc += part_o[px * rank + c] * lat_ex2(part_ml[px * 2] - M);
    }
    dst[c] = __float2bfloat16_rn(acc * inv);
  }
}

// max_rows: the most rows (tokens x heads) that one request brings to this step.  part_o
// [B, row tiles, splits, 32, rank] and part_ml [B, row tiles, splits, 32, 2]: float scratch
// for `splits` > 1.
BF_EXPORT int bf_latent_attention(const void* q, const void* cache, const int* q_start,
                                  const int* positions, const int* tables, int table_stride,
                                  void* out, int B, int max_rows, int H, int W, int rank,
                                  int page_size, int num_pages, float scale, float* part_o,
                                  float* part_ml, int splits, int* err, cudaStream_t stream) {
  if (B <= 0 || max_rows <= 0) return 0;
  if (W % 16 || rank % 16 || rank <= 0 || rank > 512 || W < rank || W > 640 || !(scale > 0.f))
    return (int)cudaErrorInvalidValue;
  if (splits > 1 && (!part_o || !part_ml)) return (int)cudaErrorInvalidValue;
  if (splits < 1) splits = 1;
  const int pitch = W + 8;
  const size_t smem = ((size_t)LAT_ROWS * pitch + (size_t)2 * LAT_KEYS * pitch +
                       (size_t)LAT_ROWS * LAT_PP) * sizeof(__nv_bfloat16) + 2 * 4 * 16 * sizeof(float);
  const int tiles = (max_rows + LAT_ROWS - 1) / LAT_ROWS;
  dim3 grid(tiles, B, splits);
  const float log2e = 1.4426950408889634f;
  const int NP = rank <= 128 ? 2 : rank <= 256 ? 4 : 8;
  static bool configured[BF_MAX_DEVICES][3];
  const int dev = bf_current_device();
#define LAT_GO(N, IDX)                                                                          \
  {                                                                                             \
    if (!configured[dev][IDX]) {                                                                \
      const cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<N>,                    \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                                 220 * 1024);                                    \
      if (e != cudaSuccess) return (int)e;                                                      \
      configured[dev][IDX] = true;                                                              \
    }                                                                                           \
    latent_attention_kernel<N><<<grid, LAT_THREADS, smem, stream>>>(                            \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, q_start, positions, tables,       \
        table_stride, (__nv_bfloat16*)out, H, W, rank, page_size, num_pages, scale * log2e,     \
        part_o, part_ml, splits, err);                                                          \
  }
  if (NP == 2) LAT_GO(2, 0) else if (NP == 4) LAT_GO(4, 1) else LAT_GO(8, 2)
#undef LAT_GO
  if (splits > 1) {
    const int e = bf_launch_status();
    if (e) return e;
    latent_merge_kernel<<<dim3(LAT_ROWS, tiles, B), 128, 0, stream>>>(
        part_o, part_ml, splits, q_start, (__nv_bfloat16*)out, H, rank);
  }
  return bf_launch_status();
}
