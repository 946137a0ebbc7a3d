// Attention whose keys and values are made from one small latent per token (multi-head latent attention).
//
// A token's cache row is [latent c: kv_rank numbers, RMS-normed | rotated key part: rot_dim numbers, one for all heads].
// With the keys' up-projection moved onto the queries (q_lat = W_uk[h]^T q_plain[h]) and the values' up-projection applied
// after the weighted sum, every head reads the SAME rows: score = (q_lat . c + q_rot . k_rot) * scale, and a head's
// output before its up-projection is sum_j p_j c_j. So the attention proper is multi-query attention with key rows of
// kv_rank + rot_dim numbers whose first kv_rank numbers are the value.
//
//   r2_latent_prepare   per row of the stacked projection [q heads | c | k_rot]: RMS norm of c (statistics in float), rotation
//                       of k_rot and of every head's rotated query part (pairs (2i, 2i + 1), angle position * freq[i], cos and
//                       sin times `magnitude`, all in float), in place; and the row's [c | k_rot] into its cache slot. The heads'
//                       rotated query parts are also copied to where the attention kernel reads whole query rows. A further
//                       segment of the row (a latent that the queries are made from) may be RMS-normed in the same launch;
//                       the row may hold no query heads (they are made later, from that latent), or no latent (a second
//                       call then rotates and copies the query parts).
//   r2_head_linear      one small product per head: out[t][h][:] = a[t][h][:] W[h] for every head h, where the heads' vectors
//                       lie side by side in the rows of a and out (with strides of their own) and W holds the heads' matrices
//                       one after the other. It is what moves the keys' up-projection onto the queries and applies the
//                       values' up-projection to the heads' weighted sums of latents (there it may also multiply the
//                       outputs by the sigmoid of a gate, element by element).
//   r2_latent_attention the attention proper for bfloat16 on the warp-level tensor cores: a CTA's rows are (token, head) pairs
//                       of one entry, so that one tile of cache rows serves all heads of several tokens.
#include <limits.h>
#include <math.h>

#include "common.cuh"
#include "mma_sync.cuh"
#include "sm100_ptx.cuh"

namespace {

// out[t][h][n] = sum_k a[t][h][k] * w[h](k, n), float sums. w[h] is [K][N] (w_is_nk = 0) or [N][K] (1), the heads' matrices
// one after the other. A CTA has HL_ROWS rows x HL_COLS columns of one head; K in pieces of HL_K through shared memory; a
// thread has 2 rows x 4 columns. The order of a sum depends on K alone.
constexpr int HL_ROWS = 32, HL_COLS = 64, HL_K = 32;

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ a, int a_stride, int a_head, const T* __restrict__ w, int w_is_nk, T* __restrict__ out,
                   int out_stride, int out_head, int n_rows, int k_total, int n_total, const T* __restrict__ gate, int gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float as[HL_K][HL_ROWS + 1];
  __shared__ float ws[HL_K][HL_COLS + 1];
  const int h = blockIdx.z, r0 = blockIdx.x * HL_ROWS, c0 = blockIdx.y * HL_COLS;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // columns tx * 4 .., rows ty * 2 ..
  const T* ah = a + size_t(h) * a_head;
  const T* wh = w + size_t(h) * k_total * n_total;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < k_total; k0 += HL_K) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < HL_ROWS * HL_K; idx += 256) {
      const int r = idx / HL_K, k = idx % HL_K;
      as[k][r] = (r0 + r < n_rows && k0 + k < k_total) ? to_float(ah[size_t(r0 + r) * a_stride + k0 + k]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < HL_COLS * HL_K; idx += 256) {
      int k, n;
      if (w_is_nk) { n = idx / HL_K; k = idx % HL_K; } else { k = idx / HL_COLS; n = idx % HL_COLS; }
      float v = 0.f;
      if (c0 + n < n_total && k0 + k < k_total)
        v = to_float(w_is_nk ? wh[size_t(c0 + n) * k_total + k0 + k] : wh[size_t(k0 + k) * n_total + c0 + n]);
      ws[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HL_K; ++k) {
      const float a0 = as[k][ty * 2], a1 = as[k][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = ws[k][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + ty * 2 + i;
    if (r >= n_rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = c0 + tx * 4 + j;
      if (n < n_total) {
        float y = acc[i][j];
        if (gate != nullptr) y *= 1.f / (1.f + expf(-to_float(gate[size_t(r) * gate_stride + size_t(h) * out_head + n])));
        out[size_t(r) * out_stride + size_t(h) * out_head + n] = from_float<T>(y);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ buf, int row_stride, int n_heads, int q_head_dim, int q_rot_off, int rot_dim, int rot_half,
                      int kv_col, int kv_rank, const float* __restrict__ norm_w, float eps, const float* __restrict__ freq,
                      float magnitude, const int32_t* __restrict__ positions, T* __restrict__ k_cache,
                      const int32_t* __restrict__ slot_mapping, int page_size, long long page_stride, int n_pages,
                      T* __restrict__ q_out, int q_out_stride, int q_out_head_dim, int q_out_off, int xn_col, int xn_rank,
                      const float* __restrict__ xn_w) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  T* row = buf + size_t(t) * row_stride;
  const float p = float(positions[t]);
  if (xn_rank > 0) {   // a further normed segment: the latent that the queries are made from
    T* x = row + xn_col;
    float sq = 0.f;
    for (int d = threadIdx.x; d < xn_rank; d += blockDim.x) {
      const float v = to_float(x[d]);
      sq = fmaf(v, v, sq);
    }
    const float inv = 1.f / sqrtf(block_sum(sq, scratch) / float(xn_rank) + eps);
    for (int d = threadIdx.x; d < xn_rank; d += blockDim.x) x[d] = from_float<T>(to_float(x[d]) * inv * xn_w[d]);
  }
  const bool has_kv = kv_col >= 0;
  // the row's cache slot (none for a pad row, whose slot is the null page's)
  T* slot_row = nullptr;
  if (has_kv && k_cache != nullptr) {
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot % page_size;
    if (slot >= 0 && page < n_pages) slot_row = k_cache + size_t(page) * page_stride + size_t(off) * (kv_rank + rot_dim);
  }
  // the latent: x / sqrt(mean(x^2) + eps) * w
  T* c = row + (has_kv ? kv_col : 0);
  if (has_kv) {
    float sq = 0.f;
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
      const float v = to_float(c[d]);
      sq = fmaf(v, v, sq);
    }
    const float inv = 1.f / sqrtf(block_sum(sq, scratch) / float(kv_rank) + eps);
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
      const T y = from_float<T>(to_float(c[d]) * inv * norm_w[d]);
      c[d] = y;
      if (slot_row != nullptr) slot_row[d] = y;
    }
  }
  // rotated parts: unit 0 is the shared key part (where the row has one), units 1 .. n_heads the heads' query parts
  const int per_unit = rot_dim - rot_half;   // rot_half pairs, then the dimensions that pass unchanged
  for (int idx = threadIdx.x + (has_kv ? 0 : per_unit); idx < (n_heads + 1) * per_unit; idx += blockDim.x) {
    const int unit = idx / per_unit, i = idx - unit * per_unit;
    T* x = unit == 0 ? c + kv_rank : row + size_t(unit - 1) * q_head_dim + q_rot_off;
    T* dst = unit == 0 ? (slot_row != nullptr ? slot_row + kv_rank : nullptr)
                       : (q_out != nullptr ? q_out + size_t(t) * q_out_stride + size_t(unit - 1) * q_out_head_dim + q_out_off : nullptr);
    if (i < rot_half) {
      float sn, cs;
      sincosf(p * freq[i], &sn, &cs);
      sn *= magnitude;
      cs *= magnitude;
      const float u = to_float(x[2 * i]), v = to_float(x[2 * i + 1]);
      const T a = from_float<T>(u * cs - v * sn), b = from_float<T>(v * cs + u * sn);
      x[2 * i] = a;
      x[2 * i + 1] = b;
      if (dst != nullptr) { dst[2 * i] = a; dst[2 * i + 1] = b; }
    } else if (dst != nullptr) {
      const int d = rot_half + i;   // i - rot_half + 2 * rot_half
      dst[d] = x[d];
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------------
// The attention proper on the warp-level tensor cores (bfloat16 in, float scores, weights and sums).
//
// Every head reads the same cache rows, so a CTA's 64 rows of the first product are (token, head) pairs of one entry:
// tokens_here consecutive tokens x heads_here heads, 16 pairs to a warp. A portion of a prompt fills the 64 rows with a
// few tokens and all their heads; a single decoded token fills them with its heads alone. Key rows come in tiles of 64
// through two buffers (16-byte asynchronous copies through the block table; element by element where a row's length or
// an address is no multiple of 16 bytes), rows padded with zeros to a multiple of 16 numbers. A key's value is the
// first kv_rank numbers of its row: the second product reads the same tile, transposed by ldmatrix. Scores are scaled and
// masked in float (causal, window, context length), the softmax is online, and its weights enter the second product
// rounded to bfloat16, or with `split_p` as the sum of two bfloat16 numbers. VT: 16-wide column tiles of the output.
constexpr int LA_WARPS = 4, LA_ROWS = 64, LA_KEYS = 64;
// Key tiles in flight: a decode step's CTA is alone on its SM and does little per tile, so it looks further ahead.
constexpr int latent_stages(bool split) { return split ? 4 : 2; }
static_assert(LA_WARPS * 32 == 2 * LA_KEYS, "the copy of a key tile gives two threads to a key");

struct LatentAttnParams {
  const bf16* q; int q_stride;
  bf16* out; int out_stride;
  const bf16* cache; long long page_stride; int page_size, page_shift, n_pages;
  const int32_t* block_tables; int table_width;
  const int32_t* q_start; const int32_t* positions; const int32_t* seq_lens; int n_entries;
  int n_heads, heads_here, tokens_here;
  int row, kv_rank, row_pad;
  float scale; int window; int split_p;
  const float* sinks;   // may be null: exp(sinks[head]) joins head's denominator (a term without key or value)
  int n_slices; float* parts;   // decode steps: a token's key tiles cut over n_slices CTAs (grid z) that leave partial sums in `parts`
  int q_vec, k_vec, out_vec;   // 16-byte loads of queries / of cache rows, 4-byte stores of outputs are possible
};

// eight numbers of a row from column c * 8 on, zeros from `row` on
__device__ __forceinline__ uint4 eight_of(const bf16* src_row, int c, int row, bool vec) {
  if (vec && c * 8 + 8 <= row) return *reinterpret_cast<const uint4*>(src_row + c * 8);
  __align__(16) bf16 tmp[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) tmp[i] = c * 8 + i < row ? src_row[c * 8 + i] : from_float<bf16>(0.f);
  return *reinterpret_cast<const uint4*>(tmp);
}

// The small products per head for bfloat16 on the warp-level tensor cores: a CTA has 64 rows x 64 columns of one head (16 rows
// to a warp), K in pieces of 64 through shared memory. A head's matrix [N][K] is read like keys (ldmatrix as it lies), [K][N]
// like values (ldmatrix transposed). An output's sum depends on K alone: float sums in the order of the 16-wide steps.
constexpr int HM_TILE = 64, HM_PAD = HM_TILE + 8;

struct HeadLinearParams {
  const bf16* a; int a_stride, a_head;
  const bf16* w; int w_is_nk;
  bf16* out; int out_stride, out_head;
  int n_rows, k_total, n_total;
  int a_vec, w_vec, out_vec;   // 16-byte loads of a's / of w's rows, 4-byte stores of outputs are possible
  const bf16* gate; int gate_stride, gate_vec;   // may be null: outputs times sigmoid(gate), laid out like out (4-byte loads possible)
};

__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const HeadLinearParams p) {
  using namespace r2ptx;
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) bf16 a_s[HM_TILE][HM_PAD];
  __shared__ __align__(16) bf16 w_s[HM_TILE][HM_PAD];
  const int h = blockIdx.z, r0 = blockIdx.x * HM_TILE, c0 = blockIdx.y * HM_TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bf16* ah = p.a + size_t(h) * p.a_head;
  const bf16* wh = p.w + size_t(h) * p.k_total * p.n_total;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  float acc[HM_TILE / 8][4];
#pragma unroll
  for (int i = 0; i < HM_TILE / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const bool warp_has_rows = r0 + warp * 16 < p.n_rows;
  for (int k0 = 0; k0 < p.k_total; k0 += HM_TILE) {
    __syncthreads();
    for (int idx = tid; idx < HM_TILE * (HM_TILE / 8); idx += 128) {
      const int r = idx / (HM_TILE / 8), c = idx % (HM_TILE / 8);
      uint4 av = zero4, wv = zero4;
      if (r0 + r < p.n_rows) av = eight_of(ah + size_t(r0 + r) * p.a_stride + k0, c, p.k_total - k0, p.a_vec != 0);
      if (p.w_is_nk) {   // r: a column of the output, its K numbers lie side by side
        if (c0 + r < p.n_total) wv = eight_of(wh + size_t(c0 + r) * p.k_total + k0, c, p.k_total - k0, p.w_vec != 0);
      } else {           // r: one of the K, the output's columns lie side by side
        if (k0 + r < p.k_total) wv = eight_of(wh + size_t(k0 + r) * p.n_total + c0, c, p.n_total - c0, p.w_vec != 0);
      }
      *reinterpret_cast<uint4*>(&a_s[r][c * 8]) = av;
      *reinterpret_cast<uint4*>(&w_s[r][c * 8]) = wv;
    }
    __syncthreads();
    if (!warp_has_rows) continue;
#pragma unroll
    for (int ks = 0; ks < HM_TILE / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(smem_u32(&a_s[warp * 16 + (lane & 15)][ks * 16 + 8 * (lane >> 4)]), a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < HM_TILE / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        if (p.w_is_nk) ldmatrix_x4(smem_u32(&w_s[np * 16 + (lane & 7) + 8 * (lane >> 4)][ks * 16 + 8 * ((lane >> 3) & 1)]), b0, b1, b2, b3);
        else ldmatrix_x4_trans(smem_u32(&w_s[ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][np * 16 + 8 * (lane >> 4)]), b0, b1, b2, b3);
        mma_bf16(acc[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = r0 + warp * 16 + g + 8 * half;
    if (r >= p.n_rows) continue;
    bf16* dst = p.out + size_t(r) * p.out_stride + size_t(h) * p.out_head;
    const bf16* gr = p.gate != nullptr ? p.gate + size_t(r) * p.gate_stride + size_t(h) * p.out_head : nullptr;
#pragma unroll
    for (int nt = 0; nt < HM_TILE / 8; ++nt) {
      const int n = c0 + nt * 8 + 2 * tq;
      float y0 = acc[nt][2 * half], y1 = acc[nt][2 * half + 1];
      if (gr != nullptr) {
        if (p.gate_vec && n + 1 < p.n_total) {
          const float2 z = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gr + n));
          y0 *= 1.f / (1.f + __expf(-z.x));
          y1 *= 1.f / (1.f + __expf(-z.y));
        } else {
          if (n < p.n_total) y0 *= 1.f / (1.f + __expf(-to_float(gr[n])));
          if (n + 1 < p.n_total) y1 *= 1.f / (1.f + __expf(-to_float(gr[n + 1])));
        }
      }
      if (p.out_vec && n + 1 < p.n_total) {
        *reinterpret_cast<__nv_bfloat162*>(dst + n) = __floats2bfloat162_rn(y0, y1);
      } else {
        if (n < p.n_total) dst[n] = from_float<bf16>(y0);
        if (n + 1 < p.n_total) dst[n + 1] = from_float<bf16>(y1);
      }
    }
  }
}

template <int VT, bool SPLIT>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const LatentAttnParams p) {
  using namespace r2ptx;
  constexpr int NP = SPLIT ? 1 : LA_KEYS / 16;   // 16-key pieces of a tile that a warp takes
  constexpr int STAGES = latent_stages(SPLIT);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t la_smem[];
  __shared__ int tile_info[2];
  const int rs = p.row_pad * 2 + 16;   // bytes of a padded row in shared memory
  uint8_t* q_s = la_smem;
  uint8_t* k_s = la_smem + LA_ROWS * rs;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = SPLIT ? 0 : warp * 16;   // the warp's first row of the tile, and its first key of a key tile
  const int key0 = SPLIT ? warp * 16 : 0;
  if (warp == 0) {   // which entry, and which of its tiles, this CTA has: 32 entries at a time, their tiles summed by shuffles
    int found = -1, first = 0;
    if (SPLIT) {     // every entry is one row
      if (int(blockIdx.x) < p.n_entries) { found = blockIdx.x; first = blockIdx.x; }
    } else {
      int base = 0;
      for (int e0 = 0; e0 < p.n_entries && found < 0; e0 += 32) {
        const int cand = e0 + lane;
        int start = 0, tiles = 0;
        if (cand < p.n_entries) {
          start = p.q_start[cand];
          tiles = (p.q_start[cand + 1] - start + p.tokens_here - 1) / p.tokens_here;
        }
        int upto = tiles;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, upto, d);
          if (lane >= d) upto += v;
        }
        const int before = base + upto - tiles;
        const bool mine = int(blockIdx.x) >= before && int(blockIdx.x) < before + tiles;
        const unsigned who = __ballot_sync(0xffffffffu, mine);
        if (who != 0u) {
          const int src = __ffs(who) - 1;
          found = __shfl_sync(0xffffffffu, cand, src);
          first = __shfl_sync(0xffffffffu, start + (int(blockIdx.x) - before) * p.tokens_here, src);
        }
        base += __shfl_sync(0xffffffffu, upto, 31);
      }
    }
    if (lane == 0) {
      tile_info[0] = found;
      tile_info[1] = first;
    }
  }
  __syncthreads();
  const int e = tile_info[0];
  if (e < 0) return;
  const int t0 = tile_info[1];
  const int n_tok = min(p.tokens_here, p.q_start[e + 1] - t0);
  const int h0 = blockIdx.y * p.heads_here;
  const int n_heads_here = min(p.heads_here, p.n_heads - h0);
  const int seq_len = p.seq_lens[e];
  const int p_first = p.positions[t0], p_last = p.positions[t0 + n_tok - 1];
  const int hi = min(p_last, seq_len - 1);                              // newest key that any row sees
  int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;           // oldest
  int n_tiles = hi >= lo ? (hi - lo) / LA_KEYS + 1 : 0;
  if (SPLIT && p.n_slices > 1) {   // this CTA's share of the token's key tiles: an even cut of the tiles that the token has
    const int per = (n_tiles + p.n_slices - 1) / p.n_slices, first = int(blockIdx.z) * per;
    lo += first * LA_KEYS;
    n_tiles = max(0, min(per, n_tiles - first));
  }
  const int32_t* table = p.block_tables + size_t(e) * p.table_width;
  const int chunks = p.row_pad / 8;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

  for (int idx = tid; idx < (SPLIT ? 16 : LA_ROWS) * chunks; idx += LA_WARPS * 32) {
    const int m = idx / chunks, c = idx - m * chunks;
    const int tok = m / p.heads_here, hh = m - tok * p.heads_here;
    uint4 v = zero4;
    if (tok < n_tok && hh < n_heads_here)
      v = eight_of(p.q + size_t(t0 + tok) * p.q_stride + size_t(h0 + hh) * p.row, c, p.row, p.q_vec != 0);
    *reinterpret_cast<uint4*>(q_s + m * rs + c * 16) = v;
  }
  auto load_keys = [&](int it, int buf) {
    // two threads a key: one look into the block table per key, then its pieces one after the other
    const int key = tid >> 1;
    const int j = lo + it * LA_KEYS + key;
    uint8_t* dst = k_s + buf * (LA_KEYS * rs) + key * rs;
    if (it >= n_tiles) {
      // no such tile: an empty group keeps the count of groups in step with the tiles
    } else if (j <= hi) {
      int page = table[page_index(j, p.page_size, p.page_shift)];
      page = (page < 0 || page >= p.n_pages) ? 0 : page;
      const bf16* src = p.cache + size_t(page) * p.page_stride + size_t(page_offset(j, p.page_size, p.page_shift)) * p.row;
      for (int c = tid & 1; c < chunks; c += 2) {
        if (p.k_vec && c * 8 + 8 <= p.row) cp_async16(smem_u32(dst + c * 16), src + c * 8, true);
        else *reinterpret_cast<uint4*>(dst + c * 16) = eight_of(src, c, p.row, false);
      }
    } else {
      for (int c = tid & 1; c < chunks; c += 2) *reinterpret_cast<uint4*>(dst + c * 16) = zero4;   // no row sees it: zeros, whatever the cache holds there
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // this thread's two rows of a 16-row piece: g and g + 8; of every 8 columns it has 2 tq and 2 tq + 1
  const int g = lane >> 2, tq = lane & 3;
  int pos_r[2], tok_r[2], head_r[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int m = row0 + g + 8 * r;
    tok_r[r] = m / p.heads_here;
    head_r[r] = m - tok_r[r] * p.heads_here;
    const bool valid = tok_r[r] < n_tok && head_r[r] < n_heads_here;
    pos_r[r] = valid ? min(p.positions[t0 + tok_r[r]], seq_len - 1) : -1;
    if (!valid) tok_r[r] = -1;
  }
  // the positions that this warp's rows span (none: the warp only helps to copy)
  const int w_tok_first = row0 / p.heads_here, w_tok_last = min((row0 + 15) / p.heads_here, n_tok - 1);
  const bool warp_has_rows = w_tok_first < n_tok;
  const int w_pmin = warp_has_rows ? p.positions[t0 + w_tok_first] : 0, w_pmax = warp_has_rows ? p.positions[t0 + w_tok_last] : -1;

  float o[2 * VT][4];
#pragma unroll
  for (int i = 0; i < 2 * VT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float scale2 = p.scale * 1.4426950408889634f;   // scores in units of log2(e): one exp2 per weight
  const int k_steps = p.row_pad / 16;

  for (int ahead = 0; ahead < STAGES - 1; ++ahead) load_keys(ahead, ahead);
  for (int it = 0; it < n_tiles; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();   // tile `it` (and, the first time, the queries) is there; nobody reads the buffer of tile `it - 1` any more
    load_keys(it + STAGES - 1, (it + STAGES - 1) % STAGES);
    const int j0 = lo + it * LA_KEYS;
    if (!warp_has_rows || j0 + key0 > w_pmax || (p.window > 0 && j0 + key0 + 16 * NP - 1 <= w_pmin - p.window)) continue;
    const uint32_t kt = smem_u32(k_s) + uint32_t((it % STAGES) * (LA_KEYS * rs));
    float s[2 * NP][4];
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll 2
    for (int ks = 0; ks < k_steps; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(smem_u32(q_s) + uint32_t((row0 + (lane & 15)) * rs + (ks * 16 + 8 * (lane >> 4)) * 2), a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < NP; ++np) {   // two 8-key tiles per ldmatrix
        uint32_t b0, b1, b2, b3;
        const int key = key0 + np * 16 + (lane & 7) + 8 * (lane >> 4);
        ldmatrix_x4(kt + uint32_t(key * rs + (ks * 2 + ((lane >> 3) & 1)) * 16), b0, b1, b2, b3);
        mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // scale and mask: key k of the tile is seen by a row if lo_r <= k <= hi_r
    const int hi_a = pos_r[0] - j0, hi_b = pos_r[1] - j0;
    const int lo_a = p.window > 0 ? pos_r[0] - p.window + 1 - j0 : INT_MIN, lo_b = p.window > 0 ? pos_r[1] - p.window + 1 - j0 : INT_MIN;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int k = key0 + nt * 8 + 2 * tq + c;
        const bool va = (k <= hi_a) & (k >= lo_a), vb = (k <= hi_b) & (k >= lo_b);
        s[nt][c] = va ? s[nt][c] * scale2 : -INFINITY;
        s[nt][2 + c] = vb ? s[nt][2 + c] * scale2 : -INFINITY;
        mx_a = fmaxf(mx_a, s[nt][c]);
        mx_b = fmaxf(mx_b, s[nt][2 + c]);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float m_a = fmaxf(m_run[0], mx_a), m_b = fmaxf(m_run[1], mx_b);
    // a row that has seen no key yet keeps exp(-inf - -inf) out of the way
    const float base_a = m_a == -INFINITY ? 0.f : m_a, base_b = m_b == -INFINITY ? 0.f : m_b;
    const float corr_a = fast_exp2(m_run[0] - base_a), corr_b = fast_exp2(m_run[1] - base_b);
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        s[nt][c] = fast_exp2(s[nt][c] - base_a);
        s[nt][2 + c] = fast_exp2(s[nt][2 + c] - base_b);
        sum_a += s[nt][c];
        sum_b += s[nt][2 + c];
      }
    }
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
    sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
    sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
    l_run[0] = l_run[0] * corr_a + sum_a;
    l_run[1] = l_run[1] * corr_b + sum_b;
    m_run[0] = m_a;
    m_run[1] = m_b;
#pragma unroll
    for (int dt = 0; dt < 2 * VT; ++dt) {
      o[dt][0] *= corr_a;
      o[dt][1] *= corr_a;
      o[dt][2] *= corr_b;
      o[dt][3] *= corr_b;
    }
    // o += weights . values, 16 keys at a time; a key's value is the head of its row
#pragma unroll
    for (int kk = 0; kk < NP; ++kk) {
      const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      uint32_t r0 = 0, r1 = 0, r2 = 0, r3 = 0;   // what the rounding left of each weight, as a second operand
      if (p.split_p) {
        r0 = pack_rest(s[2 * kk][0], s[2 * kk][1], a0); r1 = pack_rest(s[2 * kk][2], s[2 * kk][3], a1);
        r2 = pack_rest(s[2 * kk + 1][0], s[2 * kk + 1][1], a2); r3 = pack_rest(s[2 * kk + 1][2], s[2 * kk + 1][3], a3);
      }
      const int key = key0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int dp = 0; dp < VT; ++dp) {   // two 8-wide output tiles per ldmatrix
        if (dp * 16 < p.kv_rank) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(kt + uint32_t(key * rs + (dp * 2 + (lane >> 4)) * 16), b0, b1, b2, b3);
          mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
          if (p.split_p) {
            mma_bf16(o[2 * dp], r0, r1, r2, r3, b0, b1);
            mma_bf16(o[2 * dp + 1], r0, r1, r2, r3, b2, b3);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  if constexpr (SPLIT) {
    // the four warps hold the same 16 rows over different keys: their maxima, sums and outputs meet in shared memory
    constexpr int PW = VT * 16 + 2;
    float* part = reinterpret_cast<float*>(k_s);   // [warp][row][outputs, maximum, sum]
    __syncthreads();   // nobody reads a key tile any more
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float* mine = part + (warp * 16 + g + 8 * r) * PW;
#pragma unroll
      for (int dt = 0; dt < 2 * VT; ++dt) {
        mine[dt * 8 + 2 * tq] = o[dt][2 * r];
        mine[dt * 8 + 2 * tq + 1] = o[dt][2 * r + 1];
      }
      if (tq == 0) { mine[VT * 16] = m_run[r]; mine[VT * 16 + 1] = l_run[r]; }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * p.kv_rank; idx += LA_WARPS * 32) {
      const int m = idx / p.kv_rank, d = idx - m * p.kv_rank;
      const int tok = m / p.heads_here, hh = m - tok * p.heads_here;
      if (tok >= n_tok || hh >= n_heads_here) continue;
      float top = -INFINITY;
#pragma unroll
      for (int w = 0; w < LA_WARPS; ++w) top = fmaxf(top, part[(w * 16 + m) * PW + VT * 16]);
      float sum = 0.f, y = 0.f;
      if (top != -INFINITY) {
#pragma unroll
        for (int w = 0; w < LA_WARPS; ++w) {
          const float* theirs = part + (w * 16 + m) * PW;
          const float f = fast_exp2(theirs[VT * 16] - top);
          sum += theirs[VT * 16 + 1] * f;
          y += theirs[d] * f;
        }
      }
      if (p.n_slices > 1) {   // the slices of a token meet in the merge kernel: sums relative to this slice's maximum
        float* mine = p.parts + ((size_t(e) * p.n_heads + h0 + hh) * p.n_slices + blockIdx.z) * (p.kv_rank + 2);
        mine[d] = y;
        if (d == 0) { mine[p.kv_rank] = top; mine[p.kv_rank + 1] = sum; }
        continue;
      }
      if (top != -INFINITY && p.sinks != nullptr) sum += exp2f(p.sinks[h0 + hh] * 1.4426950408889634f - top);
      p.out[size_t(t0 + tok) * p.out_stride + size_t(h0 + hh) * p.kv_rank + d] = from_float<bf16>(sum > 0.f ? y / sum : 0.f);
    }
  } else {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (tok_r[r] < 0) continue;
      if (p.sinks != nullptr && m_run[r] != -INFINITY) l_run[r] += exp2f(p.sinks[h0 + head_r[r]] * 1.4426950408889634f - m_run[r]);
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      bf16* dst = p.out + size_t(t0 + tok_r[r]) * p.out_stride + size_t(h0 + head_r[r]) * p.kv_rank;
#pragma unroll
      for (int dt = 0; dt < 2 * VT; ++dt) {
        const int d = dt * 8 + 2 * tq;
        const float y0 = o[dt][2 * r] * inv, y1 = o[dt][2 * r + 1] * inv;
        if (p.out_vec && d + 1 < p.kv_rank) {
          *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(y0, y1);
        } else {
          if (d < p.kv_rank) dst[d] = from_float<bf16>(y0);
          if (d + 1 < p.kv_rank) dst[d + 1] = from_float<bf16>(y1);
        }
      }
    }
  }
}

// A decode step's slices of one (token, head) meet: out = sum_s y_s 2^(top_s - top) / (sum_s l_s 2^(top_s - top) + the sink's term).
// One CTA per (token, head); the slices are added in their order.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ parts, int n_slices, int kv_rank, int n_heads, const float* __restrict__ sinks,
                    bf16* __restrict__ out, int out_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x / n_heads, h = blockIdx.x - e * n_heads;
  const float* mine = parts + size_t(blockIdx.x) * n_slices * (kv_rank + 2);
  float top = -INFINITY;
  for (int s = 0; s < n_slices; ++s) top = fmaxf(top, mine[s * (kv_rank + 2) + kv_rank]);
  float sum = 0.f;
  if (top != -INFINITY) {
    for (int s = 0; s < n_slices; ++s) {
      const float t = mine[s * (kv_rank + 2) + kv_rank];
      if (t != -INFINITY) sum += mine[s * (kv_rank + 2) + kv_rank + 1] * exp2f(t - top);
    }
    if (sinks != nullptr) sum += exp2f(sinks[h] * 1.4426950408889634f - top);
  }
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
    float y = 0.f;
    if (top != -INFINITY) {
      for (int s = 0; s < n_slices; ++s) {
        const float t = mine[s * (kv_rank + 2) + kv_rank];
        if (t != -INFINITY) y += mine[s * (kv_rank + 2) + d] * exp2f(t - top);
      }
    }
    out[size_t(e) * out_stride + size_t(h) * kv_rank + d] = from_float<bf16>(y * inv);
  }
}

}  // namespace

// (kv_col < 0: the rows hold query heads only; n_heads 0: no query heads. xn_rank > 0: the xn_rank numbers from column xn_col on are
// RMS-normed in place with the gain xn_w and the same eps.)
// buf [n_rows, >= kv_col + kv_rank + rot_dim] with row stride `row_stride`: n_heads query heads of q_head_dim numbers (of
// which rot_dim from q_rot_off on are the rotated part), then at kv_col the latent (kv_rank) and the shared key part
// (rot_dim). rot_dims (even, <= rot_dim) of the rotated parts' first dimensions turn. k_cache (may be null): rows of
// kv_rank + rot_dim numbers, page_size of them a page. q_out (may be null): rows of n_heads heads of q_out_head_dim numbers;
// head h's rotated part is copied to q_out[t][h][q_out_off ..].
extern "C" int r2_latent_prepare(void* buf, int row_stride, int n_rows, int n_heads, int q_head_dim, int q_rot_off, int rot_dim,
                                 int rot_dims, int kv_col, int kv_rank, const float* norm_w, float eps, const float* freq,
                                 float magnitude, const int32_t* positions, void* k_cache, const int32_t* slot_mapping,
                                 int page_size, long long page_stride, int n_pages, void* q_out, int q_out_stride,
                                 int q_out_head_dim, int q_out_off, int xn_col, int xn_rank, const float* xn_w, int dtype,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_heads < 0 || (kv_col < 0 && n_heads < 1) || (kv_col >= 0 && (kv_rank < 1 || norm_w == nullptr)) || rot_dim < 0 || rot_dims < 0 ||
      rot_dims % 2 != 0 || rot_dims > rot_dim || q_rot_off < 0 || (n_heads > 0 && q_rot_off + rot_dim > q_head_dim)) return R2_BAD_SHAPE;
  if (xn_rank < 0 || (xn_rank > 0 && (xn_w == nullptr || xn_col < 0))) return R2_BAD_SHAPE;
  if (k_cache != nullptr && (slot_mapping == nullptr || page_size < 1)) return R2_BAD_SHAPE;
  if (q_out != nullptr && (q_out_off < 0 || q_out_off + rot_dim > q_out_head_dim)) return R2_BAD_SHAPE;
  if (dtype == R2_F32) {
    r2_launch(latent_prepare_kernel<float>, dim3(n_rows), dim3(128), size_t(0), stream, (float*)buf, row_stride, n_heads, q_head_dim,
              q_rot_off, rot_dim, rot_dims / 2, kv_col, kv_rank, norm_w, eps, freq, magnitude, positions, (float*)k_cache, slot_mapping,
              page_size, page_stride, n_pages, (float*)q_out, q_out_stride, q_out_head_dim, q_out_off, xn_col, xn_rank, xn_w);
  } else if (dtype == R2_BF16) {
    r2_launch(latent_prepare_kernel<bf16>, dim3(n_rows), dim3(128), size_t(0), stream, (bf16*)buf, row_stride, n_heads, q_head_dim,
              q_rot_off, rot_dim, rot_dims / 2, kv_col, kv_rank, norm_w, eps, freq, magnitude, positions, (bf16*)k_cache, slot_mapping,
              page_size, page_stride, n_pages, (bf16*)q_out, q_out_stride, q_out_head_dim, q_out_off, xn_col, xn_rank, xn_w);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// a [n_rows, ...] with row stride a_stride, head h's k numbers at a[t][h * a_head ..]; out likewise with out_stride and out_head;
// w: n_heads matrices of k x n numbers one after the other, each [k][n] (w_is_nk 0) or [n][k] (1).
// gate (may be null; rows of stride gate_stride, laid out like out): out *= sigmoid(gate), element by element.
extern "C" int r2_head_linear(const void* a, int a_stride, int a_head, const void* w, int w_is_nk, void* out, int out_stride,
                              int out_head, int n_rows, int n_heads, int k, int n, const void* gate, int gate_stride, int dtype,
                              cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || n <= 0) return R2_OK;
  if (k < 1 || n_heads > 65535) return R2_BAD_SHAPE;
  dim3 grid((n_rows + HL_ROWS - 1) / HL_ROWS, (n + HL_COLS - 1) / HL_COLS, n_heads);
  if (dtype == R2_F32) {
    r2_launch(head_linear_kernel<float>, grid, dim3(256), size_t(0), stream, (const float*)a, a_stride, a_head, (const float*)w, w_is_nk,
              (float*)out, out_stride, out_head, n_rows, k, n, (const float*)gate, gate_stride);
  } else if (dtype == R2_BF16) {
    HeadLinearParams p;
    p.a = (const bf16*)a; p.a_stride = a_stride; p.a_head = a_head;
    p.w = (const bf16*)w; p.w_is_nk = w_is_nk;
    p.out = (bf16*)out; p.out_stride = out_stride; p.out_head = out_head;
    p.n_rows = n_rows; p.k_total = k; p.n_total = n;
    p.gate = (const bf16*)gate; p.gate_stride = gate_stride;
    p.gate_vec = (gate != nullptr && uintptr_t(gate) % 4 == 0 && gate_stride % 2 == 0 && out_head % 2 == 0) ? 1 : 0;
    p.a_vec = (uintptr_t(a) % 16 == 0 && a_stride % 8 == 0 && a_head % 8 == 0) ? 1 : 0;
    p.w_vec = (uintptr_t(w) % 16 == 0 && (w_is_nk ? k : n) % 8 == 0 && (size_t(k) * n) % 8 == 0) ? 1 : 0;
    p.out_vec = (uintptr_t(out) % 4 == 0 && out_stride % 2 == 0 && out_head % 2 == 0) ? 1 : 0;
    r2_launch(head_linear_mma_kernel, dim3((n_rows + HM_TILE - 1) / HM_TILE, (n + HM_TILE - 1) / HM_TILE, n_heads), dim3(128), size_t(0),
              stream, p);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// How many (token, head) pairs of a CTA's rows are heads: all heads, or an even share of them where there are more than the
// tile has rows: 64, or 16 where every entry is one row and the four warps share the keys instead (`single_rows`).
static inline void latent_tile_shape(int n_heads, int single_rows, int* heads_here, int* tokens_here, int* head_groups) {
  const int rows = single_rows ? 16 : LA_ROWS;
  *head_groups = (n_heads + rows - 1) / rows;
  *heads_here = (n_heads + *head_groups - 1) / *head_groups;
  *tokens_here = single_rows ? 1 : rows / *heads_here;
}

template <int VT, bool SPLIT>
static void launch_latent_attention(const LatentAttnParams& p, dim3 grid, cudaStream_t stream) {
  const size_t rs = p.row_pad * 2 + 16, tiles = latent_stages(SPLIT) * LA_KEYS * rs, parts = size_t(LA_WARPS) * 16 * (VT * 16 + 2) * sizeof(float);
  const size_t smem = LA_ROWS * rs + (SPLIT && parts > tiles ? parts : tiles);
  static bool raised = false;   // the largest rows need more shared memory than a kernel gets unasked
  if (!raised) {
    if (cudaFuncSetAttribute(latent_attention_kernel<VT, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (LA_ROWS + latent_stages(SPLIT) * LA_KEYS) * (256 * 2 + 16)) != cudaSuccess) return;
    raised = true;
  }
  r2_launch(latent_attention_kernel<VT, SPLIT>, grid, dim3(LA_WARPS * 32), smem, stream, p);
}

template <bool SPLIT>
static void launch_latent_attention_of(int kv_rank, const LatentAttnParams& p, dim3 grid, cudaStream_t stream) {
  if (kv_rank <= 64) launch_latent_attention<4, SPLIT>(p, grid, stream);
  else if (kv_rank <= 128) launch_latent_attention<8, SPLIT>(p, grid, stream);
  else if (kv_rank <= 192) launch_latent_attention<12, SPLIT>(p, grid, stream);
  else launch_latent_attention<16, SPLIT>(p, grid, stream);
}

// q [n_rows, n_heads * row] bfloat16 (a head's query against a cache row: kv_rank numbers against the latent, the rest
// against the shared key part), out [n_rows, n_heads * kv_rank], cache rows of `row` numbers, page_size of them a page.
// Entry e has the rows q_start[e] .. q_start[e + 1] - 1 at consecutive positions and its block table's row e. `single_rows`: every
// entry is one row (a decode step); CTAs then have the heads of one token and their warps a quarter of every key tile each.
// sinks (may be null): float [n_heads], a further term exp(sinks[h]) in head h's softmax denominator.
// n_slices > 1 (decode steps only): every token's key tiles are cut over that many CTAs, whose partial sums (in `parts`, room for
// parts_floats floats: n_entries * n_heads * n_slices * (kv_rank + 2) are needed, else one CTA takes all) a second launch merges.
extern "C" int r2_latent_attention(const void* q, int q_stride, void* out, int out_stride, const void* cache, long long page_stride,
                                   int page_size, int n_pages, const int32_t* block_tables, int table_width, const int32_t* q_start,
                                   const int32_t* positions, const int32_t* seq_lens, int n_entries, int n_rows, int n_heads, int row,
                                   int kv_rank, float scale, int window, int split_p, int single_rows, const float* sinks,
                                   int n_slices, float* parts, long long parts_floats, cudaStream_t stream) {
  if (n_rows <= 0 || n_entries <= 0) return R2_OK;
  if (single_rows && n_rows != n_entries) return R2_BAD_SHAPE;
  if (n_heads < 1 || kv_rank < 1 || kv_rank > row || row > 256 || page_size < 1 || window < 0) return R2_BAD_SHAPE;
  LatentAttnParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.cache = (const bf16*)cache; p.page_stride = page_stride; p.page_size = page_size; p.page_shift = page_shift_of(page_size);
  p.n_pages = n_pages; p.block_tables = block_tables; p.table_width = table_width;
  p.q_start = q_start; p.positions = positions; p.seq_lens = seq_lens; p.n_entries = n_entries;
  int head_groups;
  latent_tile_shape(n_heads, single_rows, &p.heads_here, &p.tokens_here, &head_groups);
  p.n_heads = n_heads;
  p.row = row; p.kv_rank = kv_rank; p.row_pad = (row + 15) / 16 * 16;
  p.scale = scale; p.window = window; p.split_p = split_p; p.sinks = sinks;
  // a decode step's tokens may have their key tiles cut over several CTAs, which leave partial sums for a merge kernel
  if (!single_rows || n_slices < 2 || parts == nullptr || (long long)n_entries * n_heads * n_slices * (kv_rank + 2) > parts_floats) n_slices = 1;
  p.n_slices = n_slices; p.parts = parts;
  p.q_vec = (uintptr_t(q) % 16 == 0 && q_stride % 8 == 0 && row % 8 == 0) ? 1 : 0;
  p.k_vec = (uintptr_t(cache) % 16 == 0 && page_stride % 8 == 0 && row % 8 == 0) ? 1 : 0;
  p.out_vec = (uintptr_t(out) % 4 == 0 && out_stride % 2 == 0 && kv_rank % 2 == 0) ? 1 : 0;
  const dim3 grid((n_rows + n_entries * (p.tokens_here - 1)) / p.tokens_here, head_groups, n_slices);
  if (single_rows) launch_latent_attention_of<true>(kv_rank, p, grid, stream);
  else launch_latent_attention_of<false>(kv_rank, p, grid, stream);
  if (n_slices > 1) {
    const int status = launch_status();
    if (status != R2_OK) return status;
    r2_launch(latent_merge_kernel, dim3(n_entries * n_heads), dim3(128), size_t(0), stream, (const float*)parts, n_slices, kv_rank, n_heads, sinks,
              (bf16*)out, out_stride);
  }
  return launch_status();
}
