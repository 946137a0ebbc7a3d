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
//                       rotated query parts are also copied to where the attention kernel reads whole query rows.
//   r2_head_linear      one small product per head: out[t][h][:] = a[t][h][:] W[h] for every head h, where the heads' vectors
//                       lie side by side in the rows of a and out (with strides of their own) and W holds the heads' matrices
//                       one after the other. It is what moves the keys' up-projection onto the queries and applies the
//                       values' up-projection to the heads' weighted sums of latents.
#include <math.h>

#include "common.cuh"

namespace {

// out[t][h][n] = sum_k a[t][h][k] * w[h](k, n), float sums. w[h] is [K][N] (w_is_nk = 0) or [N][K] (1), the heads' matrices
// one after the other. A CTA has HL_ROWS rows x HL_COLS columns of one head; K in pieces of HL_K through shared memory; a
// thread has 2 rows x 4 columns. The order of a sum depends on K alone.
constexpr int HL_ROWS = 32, HL_COLS = 64, HL_K = 32;

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ a, int a_stride, int a_head, const T* __restrict__ w, int w_is_nk, T* __restrict__ out,
                   int out_stride, int out_head, int n_rows, int k_total, int n_total) {
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
      if (n < n_total) out[size_t(r) * out_stride + size_t(h) * out_head + n] = from_float<T>(acc[i][j]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ buf, int row_stride, int n_heads, int q_head_dim, int q_rot_off, int rot_dim, int rot_half,
                      int kv_col, int kv_rank, const float* __restrict__ norm_w, float eps, const float* __restrict__ freq,
                      float magnitude, const int32_t* __restrict__ positions, T* __restrict__ k_cache,
                      const int32_t* __restrict__ slot_mapping, int page_size, long long page_stride, int n_pages,
                      T* __restrict__ q_out, int q_out_stride, int q_out_head_dim, int q_out_off) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  T* row = buf + size_t(t) * row_stride;
  const float p = float(positions[t]);
  // the row's cache slot (none for a pad row, whose slot is the null page's)
  T* slot_row = nullptr;
  if (k_cache != nullptr) {
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot % page_size;
    if (slot >= 0 && page < n_pages) slot_row = k_cache + size_t(page) * page_stride + size_t(off) * (kv_rank + rot_dim);
  }
  // the latent: x / sqrt(mean(x^2) + eps) * w
  T* c = row + kv_col;
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
  // rotated parts: unit 0 is the shared key part, units 1 .. n_heads the heads' query parts
  const int per_unit = rot_dim - rot_half;   // rot_half pairs, then the dimensions that pass unchanged
  for (int idx = threadIdx.x; idx < (n_heads + 1) * per_unit; idx += blockDim.x) {
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

}  // namespace

// buf [n_rows, >= kv_col + kv_rank + rot_dim] with row stride `row_stride`: n_heads query heads of q_head_dim numbers (of
// which rot_dim from q_rot_off on are the rotated part), then at kv_col the latent (kv_rank) and the shared key part
// (rot_dim). rot_dims (even, <= rot_dim) of the rotated parts' first dimensions turn. k_cache (may be null): rows of
// kv_rank + rot_dim numbers, page_size of them a page. q_out (may be null): rows of n_heads heads of q_out_head_dim numbers;
// head h's rotated part is copied to q_out[t][h][q_out_off ..].
extern "C" int r2_latent_prepare(void* buf, int row_stride, int n_rows, int n_heads, int q_head_dim, int q_rot_off, int rot_dim,
                                 int rot_dims, int kv_col, int kv_rank, const float* norm_w, float eps, const float* freq,
                                 float magnitude, const int32_t* positions, void* k_cache, const int32_t* slot_mapping,
                                 int page_size, long long page_stride, int n_pages, void* q_out, int q_out_stride,
                                 int q_out_head_dim, int q_out_off, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_heads < 1 || kv_rank < 1 || rot_dim < 0 || rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > rot_dim ||
      q_rot_off < 0 || q_rot_off + rot_dim > q_head_dim) return R2_BAD_SHAPE;
  if (k_cache != nullptr && (slot_mapping == nullptr || page_size < 1)) return R2_BAD_SHAPE;
  if (q_out != nullptr && (q_out_off < 0 || q_out_off + rot_dim > q_out_head_dim)) return R2_BAD_SHAPE;
  if (dtype == R2_F32) {
    r2_launch(latent_prepare_kernel<float>, dim3(n_rows), dim3(128), size_t(0), stream, (float*)buf, row_stride, n_heads, q_head_dim,
              q_rot_off, rot_dim, rot_dims / 2, kv_col, kv_rank, norm_w, eps, freq, magnitude, positions, (float*)k_cache, slot_mapping,
              page_size, page_stride, n_pages, (float*)q_out, q_out_stride, q_out_head_dim, q_out_off);
  } else if (dtype == R2_BF16) {
    r2_launch(latent_prepare_kernel<bf16>, dim3(n_rows), dim3(128), size_t(0), stream, (bf16*)buf, row_stride, n_heads, q_head_dim,
              q_rot_off, rot_dim, rot_dims / 2, kv_col, kv_rank, norm_w, eps, freq, magnitude, positions, (bf16*)k_cache, slot_mapping,
              page_size, page_stride, n_pages, (bf16*)q_out, q_out_stride, q_out_head_dim, q_out_off);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// a [n_rows, ...] with row stride a_stride, head h's k numbers at a[t][h * a_head ..]; out likewise with out_stride and out_head;
// w: n_heads matrices of k x n numbers one after the other, each [k][n] (w_is_nk 0) or [n][k] (1).
extern "C" int r2_head_linear(const void* a, int a_stride, int a_head, const void* w, int w_is_nk, void* out, int out_stride,
                              int out_head, int n_rows, int n_heads, int k, int n, int dtype, cudaStream_t stream) {
  if (n_rows <= 0 || n_heads <= 0 || n <= 0) return R2_OK;
  if (k < 1 || n_heads > 65535) return R2_BAD_SHAPE;
  dim3 grid((n_rows + HL_ROWS - 1) / HL_ROWS, (n + HL_COLS - 1) / HL_COLS, n_heads);
  if (dtype == R2_F32) {
    r2_launch(head_linear_kernel<float>, grid, dim3(256), size_t(0), stream, (const float*)a, a_stride, a_head, (const float*)w, w_is_nk,
              (float*)out, out_stride, out_head, n_rows, k, n);
  } else if (dtype == R2_BF16) {
    r2_launch(head_linear_kernel<bf16>, grid, dim3(256), size_t(0), stream, (const bf16*)a, a_stride, a_head, (const bf16*)w, w_is_nk,
              (bf16*)out, out_stride, out_head, n_rows, k, n);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
