// Row-wise kernels: token embedding (+ learned positions), LayerNorm, and the write of new
// keys and values into their cache pages. All statistics and sums are in float.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// x[t] = table[ids[t]] * scale (+ pos_table[positions[t]]), written as float (the residual stream).
// Reference: kelpie-models/kelpie_models/models/torch/gpt2.py:90.
template <typename W>
__global__ void embed_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                             const W* __restrict__ table, const W* __restrict__ pos_table,
                             float* __restrict__ out, int width, int n_vocab, int n_positions, float scale) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= n_vocab ? n_vocab - 1 : id);  // ids are validated on the host
  const W* row = table + size_t(id) * width;
  const W* prow = nullptr;
  if (pos_table != nullptr) {
    int p = positions[t];
    p = p < 0 ? 0 : (p >= n_positions ? n_positions - 1 : p);
    prow = pos_table + size_t(p) * width;
  }
  float* o = out + size_t(t) * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = to_float(row[d]) * scale;
    if (prow != nullptr) v += to_float(prow[d]);
    o[d] = v;
  }
}

extern "C" int r2_embed(const int32_t* ids, const int32_t* positions, const void* table, const void* pos_table,
                        float* out, int n_rows, int width, int n_vocab, int n_positions, int wdtype, float scale,
                        cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1 || n_vocab < 1) return R2_BAD_SHAPE;
  int threads = width >= 256 ? 256 : (width >= 128 ? 128 : 64);
  if (wdtype == R2_F32) {
    r2_launch(embed_kernel<float>, dim3(n_rows), dim3(threads), size_t(0), stream, ids, positions, (const float*)table, (const float*)pos_table,
                                                        out, width, n_vocab, n_positions, scale);
  } else if (wdtype == R2_BF16) {
    r2_launch(embed_kernel<bf16>, dim3(n_rows), dim3(threads), size_t(0), stream, ids, positions, (const bf16*)table, (const bf16*)pos_table,
                                                       out, width, n_vocab, n_positions, scale);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// y = (x - mean) / sqrt(var + eps) * gamma + beta, biased variance, statistics in float.
// `rows` (may be null) picks the input rows: output row i reads input row rows[i].
// Reference: kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23.
template <typename O>
__global__ void layer_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                  O* __restrict__ out, int width, float eps) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  extern __shared__ float row_s[];
  __shared__ float scratch[33];
  int r = blockIdx.x;
  int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + size_t(src) * width;
  float sum = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = xr[d];
    row_s[d] = v;
    sum += v;
  }
  float mean = block_sum(sum, scratch) / float(width);
  float sq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float c = row_s[d] - mean;
    sq += c * c;
  }
  float var = block_sum(sq, scratch) / float(width);
  float inv = 1.f / sqrtf(var + eps);
  O* o = out + size_t(r) * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    o[d] = from_float<O>((row_s[d] - mean) * inv * gamma[d] + beta[d]);
  }
}

// The same with one warp per row, the row in registers, no block-wide barrier: rows of up to
// 2,048 elements whose length is a multiple of 4 (wider or unaligned rows take the kernel above).
template <typename O>
__global__ void __launch_bounds__(128)
layer_norm_warp_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ gamma,
                       const float* __restrict__ beta, O* __restrict__ out, int n_rows, int width, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int src = rows != nullptr ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + size_t(src) * width);
  constexpr int CHUNKS = 2048 / 128;
  float4 v[CHUNKS];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    v[i] = k < width ? xr[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
    sum += v[i].x + v[i].y + v[i].z + v[i].w;
  }
  const float mean = warp_sum(sum) / float(width);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    if (k < width) {
      float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
      sq += a * a + b * b + c * c + d * d;
    }
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(width) + eps);
  O* o = out + size_t(r) * width;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    if (k < width) {
      float4 g = *reinterpret_cast<const float4*>(gamma + k);
      float4 b = *reinterpret_cast<const float4*>(beta + k);
      const float y0 = (v[i].x - mean) * inv * g.x + b.x, y1 = (v[i].y - mean) * inv * g.y + b.y;
      const float y2 = (v[i].z - mean) * inv * g.z + b.z, y3 = (v[i].w - mean) * inv * g.w + b.w;
      if constexpr (sizeof(O) == 2) {  // four values, one 8-byte store (rows are multiples of 4 wide and the output 8-byte aligned)
        __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
        *reinterpret_cast<uint2*>(o + k) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(o + k) = make_float4(y0, y1, y2, y3);
      }
    }
  }
}

extern "C" int r2_layer_norm(const float* x, const int32_t* rows, const float* gamma, const float* beta, void* out,
                             int n_rows, int width, float eps, int odtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1 || size_t(width) * 4 > 200 * 1024) return R2_BAD_SHAPE;
  const bool aligned = width % 4 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) && !(reinterpret_cast<uintptr_t>(gamma) & 15) &&
                       !(reinterpret_cast<uintptr_t>(beta) & 15) && !(reinterpret_cast<uintptr_t>(out) & 15);
  if (width <= 2048 && aligned && (odtype == R2_F32 || odtype == R2_BF16)) {
    dim3 grid((n_rows + 3) / 4);
    if (odtype == R2_F32) {
      r2_launch(layer_norm_warp_kernel<float>, grid, dim3(128), size_t(0), stream, x, rows, gamma, beta, (float*)out, n_rows, width, eps);
    } else {
      r2_launch(layer_norm_warp_kernel<bf16>, grid, dim3(128), size_t(0), stream, x, rows, gamma, beta, (bf16*)out, n_rows, width, eps);
    }
    return launch_status();
  }
  int threads = width >= 1024 ? 256 : 128;
  size_t smem = size_t(width) * sizeof(float);
  if (odtype == R2_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    r2_launch(layer_norm_kernel<float>, dim3(n_rows), dim3(threads), size_t(smem), stream, x, rows, gamma, beta, (float*)out, width, eps);
  } else if (odtype == R2_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    r2_launch(layer_norm_kernel<bf16>, dim3(n_rows), dim3(threads), size_t(smem), stream, x, rows, gamma, beta, (bf16*)out, width, eps);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Keys and values of this step's rows go to their cache slots before attention reads them
// (kelpie-models/kelpie_models/kernels/ops/paged_attention.py:44-53). A slot is
// page * page_size + offset; inside a page the layout is [kv_head][offset][head_dim], and a
// page of this layer starts every `page_stride` elements. Values may have a head size of their own.
template <typename A, typename C>
__global__ void kv_write_kernel(const A* __restrict__ k_src, const A* __restrict__ v_src, int src_row_stride, int v_row_stride,
                                C* __restrict__ k_cache, C* __restrict__ v_cache,
                                const int32_t* __restrict__ slot_mapping, int n_kv_heads, int head_dim, int v_head_dim,
                                int page_size, long long page_stride, int n_pages) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  int t = blockIdx.x;
  int slot = slot_mapping[t];
  int page = slot / page_size, off = slot % page_size;
  if (slot < 0 || page >= n_pages) return;  // slots are validated on the host; never write outside the pool
  const A* ks = k_src + size_t(t) * src_row_stride;
  const A* vs = v_src + size_t(t) * v_row_stride;
  for (int i = threadIdx.x; i < n_kv_heads * head_dim; i += blockDim.x) {
    int h = i / head_dim, d = i % head_dim;
    k_cache[size_t(page) * page_stride + (size_t(h) * page_size + off) * head_dim + d] = from_float<C>(to_float(ks[i]));
  }
  for (int i = threadIdx.x; i < n_kv_heads * v_head_dim; i += blockDim.x) {
    int h = i / v_head_dim, d = i % v_head_dim;
    v_cache[size_t(page) * page_stride + (size_t(h) * page_size + off) * v_head_dim + d] = from_float<C>(to_float(vs[i]));
  }
}

extern "C" int r2_kv_write(const void* k_src, const void* v_src, int src_row_stride, int v_row_stride, void* k_cache, void* v_cache,
                           const int32_t* slot_mapping, int n_rows, int n_kv_heads, int head_dim, int v_head_dim, int page_size,
                           long long page_stride, int n_pages_total, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_kv_heads < 1 || head_dim < 1 || v_head_dim < 1 || page_size < 1 || n_pages_total < 1) return R2_BAD_SHAPE;
  int width = n_kv_heads * (head_dim > v_head_dim ? head_dim : v_head_dim);
  int threads = width >= 256 ? 256 : 128;
  if (dtype == R2_F32) {
    r2_launch(kv_write_kernel<float, float>, dim3(n_rows), dim3(threads), size_t(0), stream, (const float*)k_src, (const float*)v_src, src_row_stride, v_row_stride,
                                                                  (float*)k_cache, (float*)v_cache, slot_mapping,
                                                                  n_kv_heads, head_dim, v_head_dim, page_size, page_stride, n_pages_total);
  } else if (dtype == R2_BF16) {
    r2_launch(kv_write_kernel<bf16, bf16>, dim3(n_rows), dim3(threads), size_t(0), stream, (const bf16*)k_src, (const bf16*)v_src, src_row_stride, v_row_stride,
                                                                (bf16*)k_cache, (bf16*)v_cache, slot_mapping,
                                                                n_kv_heads, head_dim, v_head_dim, page_size, page_stride, n_pages_total);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// Two neighbouring elements as one access (4 bytes of bfloat16, 8 of float).
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(bf16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }
template <typename T> __host__ __device__ inline bool pair_aligned(const T* p) { return (reinterpret_cast<uintptr_t>(p) & (2 * sizeof(T) - 1)) == 0; }

// ---------------------------------------------------------------------------------------------
// RMS norm: y = x / sqrt(mean(x^2) + eps) * (offset + w), statistics in float. `offset` is 1 for a
// weight tensor that holds the gain's offset from one and 0 for a plain gain. `rows` (may be null) picks input rows.
// One warp per row, the row read twice (the second pass comes from L1/L2).
template <typename O>
__global__ void __launch_bounds__(128)
rms_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ weight,
                O* __restrict__ out, int n_rows, int width, float eps, float offset) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + size_t(src) * width;
  float sq = 0.f;
  for (int d = lane; d < width; d += 32) {
    float v = xr[d];
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(width) + eps);
  O* o = out + size_t(r) * width;
  for (int d = lane; d < width; d += 32) o[d] = from_float<O>(xr[d] * inv * (offset + weight[d]));
}

// The same with the row in the warp's registers, read once in 16-byte pieces: rows of up to 2,048 elements
// whose length is a multiple of 4.
template <typename O>
__global__ void __launch_bounds__(128)
rms_norm_reg_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ weight,
                    O* __restrict__ out, int n_rows, int width, float eps, float offset) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int src = rows != nullptr ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + size_t(src) * width);
  constexpr int CHUNKS = 2048 / 128;
  float4 v[CHUNKS];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int k = (lane + 32 * i) * 4;
    v[i] = k < width ? xr[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
    sq += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(width) + eps);
  O* o = out + size_t(r) * width;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int k = (lane + 32 * i) * 4;
    if (k < width) {
      const float4 g = *reinterpret_cast<const float4*>(weight + k);
      const float y0 = v[i].x * inv * (offset + g.x), y1 = v[i].y * inv * (offset + g.y);
      const float y2 = v[i].z * inv * (offset + g.z), y3 = v[i].w * inv * (offset + g.w);
      if constexpr (sizeof(O) == 2) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
        *reinterpret_cast<uint2*>(o + k) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(o + k) = make_float4(y0, y1, y2, y3);
      }
    }
  }
}

extern "C" int r2_rms_norm(const float* x, const int32_t* rows, const float* weight, void* out, int n_rows, int width,
                           float eps, float offset, int odtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1) return R2_BAD_SHAPE;
  dim3 grid((n_rows + 3) / 4);
  const bool aligned = width % 4 == 0 && width <= 2048 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
                       !(reinterpret_cast<uintptr_t>(weight) & 15) && !(reinterpret_cast<uintptr_t>(out) & 15);
  if (aligned && odtype == R2_F32) {
    r2_launch(rms_norm_reg_kernel<float>, grid, dim3(128), size_t(0), stream, x, rows, weight, (float*)out, n_rows, width, eps, offset);
    return launch_status();
  }
  if (aligned && odtype == R2_BF16) {
    r2_launch(rms_norm_reg_kernel<bf16>, grid, dim3(128), size_t(0), stream, x, rows, weight, (bf16*)out, n_rows, width, eps, offset);
    return launch_status();
  }
  if (odtype == R2_F32) {
    r2_launch(rms_norm_kernel<float>, grid, dim3(128), size_t(0), stream, x, rows, weight, (float*)out, n_rows, width, eps, offset);
  } else if (odtype == R2_BF16) {
    r2_launch(rms_norm_kernel<bf16>, grid, dim3(128), size_t(0), stream, x, rows, weight, (bf16*)out, n_rows, width, eps, offset);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// RMS norm of every head of the query and key columns of a fused projection, in place: the row's
// first n_q_heads heads take the gain w_q, the n_k_heads heads after them w_k (both of head_dim
// values, shared by all heads of their kind). One warp per (row, head), sums in float.
// With a cache (k_cache not null) the same launch also puts the row's normed key heads and its value
// heads (n_k_heads heads of v_head_dim values from column v_col on) into the row's cache slot, so that
// no second kernel reads the projection again.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kernel(T* __restrict__ buf, int row_stride, int n_rows, int n_q_heads, int n_k_heads, int head_dim,
                 const float* __restrict__ w_q, const float* __restrict__ w_k, float eps, float offset,
                 T* __restrict__ k_cache, T* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping, int v_col,
                 int v_head_dim, int page_size, long long page_stride, int n_pages) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = n_q_heads + n_k_heads + (k_cache != nullptr ? n_k_heads : 0);
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)n_rows * heads) return;
  const int r = int(item / heads), h = int(item % heads);
  size_t page_base = 0;   // where the slot's page begins in this layer's cache
  int off = 0;            // the slot's place within the page
  bool cached = false;
  if (k_cache != nullptr && h >= n_q_heads) {
    const int slot = slot_mapping[r];
    const int page = slot / page_size;
    cached = slot >= 0 && page < n_pages;  // slots are validated on the host; never write outside the pool
    page_base = size_t(page) * page_stride;
    off = slot % page_size;
  }
  if (h >= n_q_heads + n_k_heads) {  // a value head: copied as it is
    const int vh = h - n_q_heads - n_k_heads;
    const T* src = buf + size_t(r) * row_stride + v_col + size_t(vh) * v_head_dim;
    if (cached) {
      T* dst = v_cache + page_base + (size_t(vh) * page_size + off) * v_head_dim;
      for (int d = lane; d < v_head_dim; d += 32) dst[d] = src[d];
    }
    return;
  }
  T* p = buf + size_t(r) * row_stride + size_t(h) * head_dim;
  const float* w = h < n_q_heads ? w_q : w_k;
  float sq = 0.f;
  for (int d = lane; d < head_dim; d += 32) {
    float v = to_float(p[d]);
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(head_dim) + eps);
  T* dst = nullptr;
  if (cached) dst = k_cache + page_base + (size_t(h - n_q_heads) * page_size + off) * head_dim;
  for (int d = lane; d < head_dim; d += 32) {
    const T y = from_float<T>(to_float(p[d]) * inv * (offset + w[d]));
    p[d] = y;
    if (dst != nullptr) dst[d] = y;
  }
}

// The same with a head in the warp's registers, two neighbouring elements per access: even head sizes up to
// 512 in buffers and caches whose strides and starts are even.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_pair_kernel(T* __restrict__ buf, int row_stride, int n_rows, int n_q_heads, int n_k_heads, int head_dim,
                      const float* __restrict__ w_q, const float* __restrict__ w_k, float eps, float offset,
                      T* __restrict__ k_cache, T* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping, int v_col,
                      int v_head_dim, int page_size, long long page_stride, int n_pages) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = n_q_heads + n_k_heads + (k_cache != nullptr ? n_k_heads : 0);
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)n_rows * heads) return;
  const int r = int(item / heads), h = int(item % heads);
  size_t page_base = 0;
  int off = 0;
  bool cached = false;
  if (k_cache != nullptr && h >= n_q_heads) {
    const int slot = slot_mapping[r];
    const int page = slot / page_size;
    cached = slot >= 0 && page < n_pages;
    page_base = size_t(page) * page_stride;
    off = slot % page_size;
  }
  if (h >= n_q_heads + n_k_heads) {
    const int vh = h - n_q_heads - n_k_heads;
    const T* src = buf + size_t(r) * row_stride + v_col + size_t(vh) * v_head_dim;
    if (cached) {
      T* dst = v_cache + page_base + (size_t(vh) * page_size + off) * v_head_dim;
      for (int d = 2 * lane; d < v_head_dim; d += 64) {
        const float2 v = load2(src + d);
        store2(dst + d, v.x, v.y);
      }
    }
    return;
  }
  T* p = buf + size_t(r) * row_stride + size_t(h) * head_dim;
  const float* w = h < n_q_heads ? w_q : w_k;
  float2 v[8];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = 2 * lane + 64 * i;
    v[i] = d < head_dim ? load2(p + d) : make_float2(0.f, 0.f);
    sq += v[i].x * v[i].x + v[i].y * v[i].y;
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(head_dim) + eps);
  T* dst = cached ? k_cache + page_base + (size_t(h - n_q_heads) * page_size + off) * head_dim : nullptr;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int d = 2 * lane + 64 * i;
    if (d < head_dim) {
      const float2 g = *reinterpret_cast<const float2*>(w + d);
      // rounded once: the buffer and the cache hold the same values
      const T y0 = from_float<T>(v[i].x * inv * (offset + g.x)), y1 = from_float<T>(v[i].y * inv * (offset + g.y));
      store2(p + d, to_float(y0), to_float(y1));
      if (dst != nullptr) store2(dst + d, to_float(y0), to_float(y1));
    }
  }
}

// bfloat16 with head sizes that are multiples of 8: a lane holds eight neighbouring elements (one 16-byte
// access), a head lies in head_dim / 8 neighbouring lanes, and a warp takes as many whole heads of one row as
// fit its 32 lanes. A head's sum of squares is gathered from its lanes by shuffles.
__global__ void __launch_bounds__(128)
head_norm_vec8_kernel(bf16* __restrict__ buf, int row_stride, int n_rows, int n_q_heads, int n_k_heads, int head_dim,
                      const float* __restrict__ w_q, const float* __restrict__ w_k, float eps, float offset,
                      bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping, int v_col,
                      int v_head_dim, int page_size, long long page_stride, int n_pages) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int qk_heads = n_q_heads + n_k_heads;
  const int lanes_qk = head_dim / 8, per_warp_qk = 32 / lanes_qk;            // lanes of a head; heads of a warp
  const int slabs_qk = (qk_heads + per_warp_qk - 1) / per_warp_qk;
  const int lanes_v = k_cache != nullptr ? v_head_dim / 8 : 1, per_warp_v = 32 / lanes_v;
  const int slabs_v = k_cache != nullptr ? (n_k_heads + per_warp_v - 1) / per_warp_v : 0;
  const int w = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (w >= n_rows * (slabs_qk + slabs_v)) return;
  const int r = w / (slabs_qk + slabs_v), slab = w % (slabs_qk + slabs_v);
  bf16* row = buf + size_t(r) * row_stride;
  size_t page_base = 0;
  int off = 0;
  bool cached = false;
  if (k_cache != nullptr) {
    const int slot = slot_mapping[r];
    const int page = slot / page_size;
    cached = slot >= 0 && page < n_pages;
    page_base = size_t(page) * page_stride;
    off = slot % page_size;
  }
  if (slab >= slabs_qk) {  // value heads: copied as they are
    const int vh = (slab - slabs_qk) * per_warp_v + lane / lanes_v, e = (lane % lanes_v) * 8;
    if (cached && lane < per_warp_v * lanes_v && vh < n_k_heads) {
      const uint4 x = *reinterpret_cast<const uint4*>(row + v_col + size_t(vh) * v_head_dim + e);
      *reinterpret_cast<uint4*>(v_cache + page_base + (size_t(vh) * page_size + off) * v_head_dim + e) = x;
    }
    return;
  }
  const int h = slab * per_warp_qk + lane / lanes_qk, e = (lane % lanes_qk) * 8;
  const bool mine = lane < per_warp_qk * lanes_qk && h < qk_heads;
  bf16* p = row + size_t(h) * head_dim + e;
  uint4 x = make_uint4(0u, 0u, 0u, 0u);
  if (mine) x = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x);
  float v[8];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(x2[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
    sq += f.x * f.x + f.y * f.y;
  }
  float total = 0.f;
  const int first_lane = (lane / lanes_qk) * lanes_qk;
  for (int j = 0; j < lanes_qk; ++j) total += __shfl_sync(0xffffffffu, sq, (first_lane + j) & 31);
  if (!mine) return;
  const float inv = 1.f / sqrtf(total / float(head_dim) + eps);
  const float* gain = (h < n_q_heads ? w_q : w_k) + e;
  const float4 g0 = *reinterpret_cast<const float4*>(gain), g1 = *reinterpret_cast<const float4*>(gain + 4);
  uint4 y;
  __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&y);
  y2[0] = __floats2bfloat162_rn(v[0] * inv * (offset + g0.x), v[1] * inv * (offset + g0.y));
  y2[1] = __floats2bfloat162_rn(v[2] * inv * (offset + g0.z), v[3] * inv * (offset + g0.w));
  y2[2] = __floats2bfloat162_rn(v[4] * inv * (offset + g1.x), v[5] * inv * (offset + g1.y));
  y2[3] = __floats2bfloat162_rn(v[6] * inv * (offset + g1.z), v[7] * inv * (offset + g1.w));
  *reinterpret_cast<uint4*>(p) = y;
  if (cached && h >= n_q_heads) {
    *reinterpret_cast<uint4*>(k_cache + page_base + (size_t(h - n_q_heads) * page_size + off) * head_dim + e) = y;
  }
}

extern "C" int r2_head_norm(void* buf, int row_stride, int n_rows, int n_q_heads, int n_k_heads, int head_dim,
                            const float* w_q, const float* w_k, float eps, float offset, void* k_cache, void* v_cache,
                            const int32_t* slot_mapping, int v_col, int v_head_dim, int page_size, long long page_stride,
                            int n_pages, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_q_heads < 0 || n_k_heads < 0 || n_q_heads + n_k_heads < 1 || head_dim < 1) return R2_BAD_SHAPE;
  if (k_cache != nullptr && (v_cache == nullptr || slot_mapping == nullptr || v_head_dim < 1 || page_size < 1 || n_pages < 1)) return R2_BAD_SHAPE;
  const long long items = (long long)n_rows * (n_q_heads + n_k_heads + (k_cache != nullptr ? n_k_heads : 0));
  dim3 grid((unsigned)((items + 3) / 4));
  const size_t esize = dtype == R2_F32 ? 4 : 2;
  auto even = [&](const void* p) { return (reinterpret_cast<uintptr_t>(p) & (2 * esize - 1)) == 0; };
  const bool pairs = head_dim % 2 == 0 && head_dim <= 512 && row_stride % 2 == 0 && even(buf) && even(w_q) && even(w_k) &&
                     !(reinterpret_cast<uintptr_t>(w_q) & 7) && !(reinterpret_cast<uintptr_t>(w_k) & 7) &&
                     (k_cache == nullptr || (v_col % 2 == 0 && v_head_dim % 2 == 0 && page_stride % 2 == 0 && even(k_cache) && even(v_cache)));
  auto on16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (dtype == R2_BF16 && head_dim % 8 == 0 && head_dim <= 256 && row_stride % 8 == 0 && on16(buf) && on16(w_q) && on16(w_k) &&
      (k_cache == nullptr || (v_head_dim % 8 == 0 && v_head_dim <= 256 && v_col % 8 == 0 && page_stride % 8 == 0 && on16(k_cache) && on16(v_cache)))) {
    const int per_warp_qk = 32 / (head_dim / 8);
    int slabs = (n_q_heads + n_k_heads + per_warp_qk - 1) / per_warp_qk;
    if (k_cache != nullptr) {
      const int per_warp_v = 32 / (v_head_dim / 8);
      slabs += (n_k_heads + per_warp_v - 1) / per_warp_v;
    }
    const long long warps = (long long)n_rows * slabs;
    r2_launch(head_norm_vec8_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), size_t(0), stream, (bf16*)buf, row_stride, n_rows, n_q_heads, n_k_heads,
              head_dim, w_q, w_k, eps, offset, (bf16*)k_cache, (bf16*)v_cache, slot_mapping, v_col, v_head_dim, page_size, page_stride, n_pages);
    return launch_status();
  }
  if (pairs && dtype == R2_F32) {
    r2_launch(head_norm_pair_kernel<float>, grid, dim3(128), size_t(0), stream, (float*)buf, row_stride, n_rows, n_q_heads, n_k_heads, head_dim, w_q, w_k, eps, offset,
              (float*)k_cache, (float*)v_cache, slot_mapping, v_col, v_head_dim, page_size, page_stride, n_pages);
    return launch_status();
  }
  if (pairs && dtype == R2_BF16) {
    r2_launch(head_norm_pair_kernel<bf16>, grid, dim3(128), size_t(0), stream, (bf16*)buf, row_stride, n_rows, n_q_heads, n_k_heads, head_dim, w_q, w_k, eps, offset,
              (bf16*)k_cache, (bf16*)v_cache, slot_mapping, v_col, v_head_dim, page_size, page_stride, n_pages);
    return launch_status();
  }
  if (dtype == R2_F32) {
    r2_launch(head_norm_kernel<float>, grid, dim3(128), size_t(0), stream, (float*)buf, row_stride, n_rows, n_q_heads, n_k_heads, head_dim, w_q, w_k, eps, offset,
              (float*)k_cache, (float*)v_cache, slot_mapping, v_col, v_head_dim, page_size, page_stride, n_pages);
  } else if (dtype == R2_BF16) {
    r2_launch(head_norm_kernel<bf16>, grid, dim3(128), size_t(0), stream, (bf16*)buf, row_stride, n_rows, n_q_heads, n_k_heads, head_dim, w_q, w_k, eps, offset,
              (bf16*)k_cache, (bf16*)v_cache, slot_mapping, v_col, v_head_dim, page_size, page_stride, n_pages);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// The inner activation of a gated feed-forward whose two projections are clamped:
//   g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(alpha * g) * (u + up_offset).
// `gate_up` holds a row's gate values in columns [0, inner) and its up values in [inner, 2 inner).
template <typename T>
__global__ void __launch_bounds__(256)
gated_act_kernel(const T* __restrict__ gate_up, int in_stride, T* __restrict__ out, int out_stride, int inner,
                 float limit, float alpha, float up_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const T* in = gate_up + size_t(blockIdx.x) * in_stride;
  T* o = out + size_t(blockIdx.x) * out_stride;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < inner; f += gridDim.y * blockDim.x) {
    float g = fminf(to_float(in[f]), limit);
    float u = fminf(fmaxf(to_float(in[inner + f]), -limit), limit);
    o[f] = from_float<T>(g / (1.f + expf(-alpha * g)) * (u + up_offset));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_act_pair_kernel(const T* __restrict__ gate_up, int in_stride, T* __restrict__ out, int out_stride, int inner,
                      float limit, float alpha, float up_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const T* in = gate_up + size_t(blockIdx.x) * in_stride;
  T* o = out + size_t(blockIdx.x) * out_stride;
  for (int f = 2 * (blockIdx.y * blockDim.x + threadIdx.x); f < inner; f += 2 * gridDim.y * blockDim.x) {
    const float2 gv = load2(in + f), uv = load2(in + inner + f);
    const float g0 = fminf(gv.x, limit), g1 = fminf(gv.y, limit);
    const float u0 = fminf(fmaxf(uv.x, -limit), limit), u1 = fminf(fmaxf(uv.y, -limit), limit);
    store2(o + f, g0 / (1.f + expf(-alpha * g0)) * (u0 + up_offset), g1 / (1.f + expf(-alpha * g1)) * (u1 + up_offset));
  }
}

// bfloat16 rows whose halves start on 16-byte boundaries: eight outputs per thread from two 16-byte loads.
__global__ void __launch_bounds__(256)
gated_act_vec8_kernel(const bf16* __restrict__ gate_up, int in_stride, bf16* __restrict__ out, int out_stride, int inner,
                      float limit, float alpha, float up_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const bf16* in = gate_up + size_t(blockIdx.x) * in_stride;
  bf16* o = out + size_t(blockIdx.x) * out_stride;
  for (int f = 8 * (blockIdx.y * blockDim.x + threadIdx.x); f < inner; f += 8 * gridDim.y * blockDim.x) {
    const uint4 gq = *reinterpret_cast<const uint4*>(in + f), uq = *reinterpret_cast<const uint4*>(in + inner + f);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uq);
    uint4 yq;
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&yq);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 gv = __bfloat1622float2(g2[i]), uv = __bfloat1622float2(u2[i]);
      const float g0 = fminf(gv.x, limit), g1 = fminf(gv.y, limit);
      const float u0 = fminf(fmaxf(uv.x, -limit), limit), u1 = fminf(fmaxf(uv.y, -limit), limit);
      y2[i] = __floats2bfloat162_rn(g0 / (1.f + expf(-alpha * g0)) * (u0 + up_offset), g1 / (1.f + expf(-alpha * g1)) * (u1 + up_offset));
    }
    *reinterpret_cast<uint4*>(o + f) = yq;
  }
}

extern "C" int r2_gated_act(const void* gate_up, int in_stride, void* out, int out_stride, int n_rows, int inner, float limit,
                            float alpha, float up_offset, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (inner < 1) return R2_BAD_SHAPE;
  dim3 grid(n_rows, (inner + 1023) / 1024);
  const size_t esize = dtype == R2_F32 ? 4 : 2;
  const bool pairs = inner % 2 == 0 && in_stride % 2 == 0 && out_stride % 2 == 0 &&
                     !(reinterpret_cast<uintptr_t>(gate_up) & (2 * esize - 1)) && !(reinterpret_cast<uintptr_t>(out) & (2 * esize - 1));
  if (dtype == R2_BF16 && inner % 8 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 &&
      !(reinterpret_cast<uintptr_t>(gate_up) & 15) && !(reinterpret_cast<uintptr_t>(out) & 15)) {
    r2_launch(gated_act_vec8_kernel, dim3(n_rows, (inner + 2047) / 2048), dim3(256), size_t(0), stream, (const bf16*)gate_up, in_stride, (bf16*)out, out_stride, inner, limit, alpha, up_offset);
    return launch_status();
  }
  if (pairs && dtype == R2_F32) {
    r2_launch(gated_act_pair_kernel<float>, dim3(n_rows, (inner + 511) / 512), dim3(256), size_t(0), stream, (const float*)gate_up, in_stride, (float*)out, out_stride, inner, limit, alpha, up_offset);
    return launch_status();
  }
  if (pairs && dtype == R2_BF16) {
    r2_launch(gated_act_pair_kernel<bf16>, dim3(n_rows, (inner + 511) / 512), dim3(256), size_t(0), stream, (const bf16*)gate_up, in_stride, (bf16*)out, out_stride, inner, limit, alpha, up_offset);
    return launch_status();
  }
  if (dtype == R2_F32) {
    r2_launch(gated_act_kernel<float>, grid, dim3(256), size_t(0), stream, (const float*)gate_up, in_stride, (float*)out, out_stride, inner, limit, alpha, up_offset);
  } else if (dtype == R2_BF16) {
    r2_launch(gated_act_kernel<bf16>, grid, dim3(256), size_t(0), stream, (const bf16*)gate_up, in_stride, (bf16*)out, out_stride, inner, limit, alpha, up_offset);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---- rotation of query and key heads by position -------------------------------------------------
// In place on the first n_heads heads of every row of `buf` (a stacked projection: query heads, then key heads).
// Of each head the first rot_dims dimensions are rotated, dimension i with dimension i + rot_dims / 2: the pair (u, v)
// at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i]. Positions and angles are float.
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
rotate_half_kernel(T* __restrict__ buf, int row_stride, int n_heads, int head_dim, int half, const float* __restrict__ inv_freq,
                   const int32_t* __restrict__ positions, T* __restrict__ k_cache, T* __restrict__ v_cache,
                   const int32_t* __restrict__ slot_mapping, int k_col, int v_col, int n_kv_heads, int v_head_dim, int page_size,
                   long long page_stride, int n_pages) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float p = float(positions[t]);
  T* row = buf + size_t(t) * row_stride;
  for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < n_heads * half; idx += gridDim.y * blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    float s, c;
    sincosf(p * inv_freq[i], &s, &c);
    T* x = row + size_t(head) * head_dim;
    const float u = to_float(x[i]), v = to_float(x[i + half]);
    x[i] = from_float<T>(u * c - v * s);
    x[i + half] = from_float<T>(v * c + u * s);
  }
  if (k_cache == nullptr) return;
  // the same launch (one CTA a row then) puts the rotated keys and the values into the row's cache slot
  __syncthreads();
  const int slot = slot_mapping[t];
  const int page = slot / page_size, off = slot % page_size;
  if (slot < 0 || page >= n_pages) return;  // never write outside the pool
  const T* ks = row + k_col;
  const T* vs = row + v_col;
  for (int i = threadIdx.x; i < n_kv_heads * head_dim; i += blockDim.x) {
    const int h = i / head_dim, d = i % head_dim;
    k_cache[size_t(page) * page_stride + (size_t(h) * page_size + off) * head_dim + d] = ks[i];
  }
  for (int i = threadIdx.x; i < n_kv_heads * v_head_dim; i += blockDim.x) {
    const int h = i / v_head_dim, d = i % v_head_dim;
    v_cache[size_t(page) * page_stride + (size_t(h) * page_size + off) * v_head_dim + d] = vs[i];
  }
}

// The same after an RMS norm of every head, with cos and sin times `magnitude`: x / sqrt(mean(x^2) + eps) * w, then the rotation,
// all in float and rounded once on the way out. One warp per unit of work and eight units a CTA (grid: rows x ceil(units / 8)),
// so that a decode step's few rows still spread over many SMs: units 0 .. n_heads - 1 are the heads (the first n_q_heads take the
// gain q_w, the others k_w; null: no norm), and a key head's warp also puts the turned key into the row's cache slot; with a
// cache, units n_heads .. n_heads + n_kv_heads - 1 copy the value heads to the slot. The row's cosines and sines are made once
// a CTA, in shared memory, for all its heads. `vec`: neighbouring pairs of elements may go as one access (even sizes and strides).
constexpr int NORM_ROTATE_MAX_DIM = 512, NORM_ROTATE_WARPS = 8;
template <typename T>
__global__ void __launch_bounds__(NORM_ROTATE_WARPS * 32)
norm_rotate_half_kernel(T* __restrict__ buf, int row_stride, int n_heads, int n_q_heads, int head_dim, int half, const float* __restrict__ freq,
                        float magnitude, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                        const int32_t* __restrict__ positions, T* __restrict__ k_cache, T* __restrict__ v_cache,
                        const int32_t* __restrict__ slot_mapping, int k_col, int v_col, int n_kv_heads, int v_head_dim, int page_size,
                        long long page_stride, int n_pages, int vec) {
  pdl_launch_dependents();
  __shared__ float stage[NORM_ROTATE_WARPS][NORM_ROTATE_MAX_DIM];
  __shared__ float cs_s[NORM_ROTATE_MAX_DIM / 2], sn_s[NORM_ROTATE_MAX_DIM / 2];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = n_heads + (k_cache != nullptr ? n_kv_heads : 0);
  // what no earlier kernel writes: the position and its angles, the slot
  const float p = float(positions[t]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(p * freq[i], &sn, &cs);
    sn_s[i] = sn * magnitude;
    cs_s[i] = cs * magnitude;
  }
  size_t page_at = 0;   // where the slot's page begins, and the slot's place in it
  int off = 0;
  bool has_slot = false;
  if (k_cache != nullptr) {
    const int slot = slot_mapping[t];
    const int page = slot / page_size;
    off = slot % page_size;
    has_slot = slot >= 0 && page < n_pages;   // never write outside the pool
    page_at = size_t(page) * page_stride;
  }
  __syncthreads();
  pdl_wait();
  T* row = buf + size_t(t) * row_stride;
  float* mine = stage[warp];
  // the CTAs of a row share its units; with many rows a row has one CTA, whose warps take the units in turn
  for (int unit = blockIdx.y * NORM_ROTATE_WARPS + warp; unit < n_units; unit += gridDim.y * NORM_ROTATE_WARPS) {
  if (unit >= n_heads) {   // a value head: its copy into the cache
    if (!has_slot) continue;
    const int h = unit - n_heads;
    const T* vs = row + v_col + size_t(h) * v_head_dim;
    T* dst = v_cache + page_at + (size_t(h) * page_size + off) * v_head_dim;
    if (vec && v_head_dim % 2 == 0) {
      for (int d = 2 * lane; d < v_head_dim; d += 64) {
        const float2 v = load2(vs + d);
        store2(dst + d, v.x, v.y);
      }
    } else {
      for (int d = lane; d < v_head_dim; d += 32) dst[d] = vs[d];
    }
    continue;
  }
  __syncwarp();   // (the warp's staging row may still be read from its unit before)
  T* x = row + size_t(unit) * head_dim;
  const float* w = unit < n_q_heads ? q_w : k_w;
  // a key head's place in the cache (the key heads are the n_kv_heads heads from column k_col on)
  T* kdst = nullptr;
  if (has_slot) {
    const long long col = (long long)unit * head_dim - k_col;
    if (col >= 0 && col < (long long)n_kv_heads * head_dim) kdst = k_cache + page_at + (size_t(col / head_dim) * page_size + off) * head_dim;
  }
  float sq = 0.f;
  if (vec) {
    for (int d = 2 * lane; d < head_dim; d += 64) {
      const float2 v = load2(x + d);
      mine[d] = v.x;
      mine[d + 1] = v.y;
      sq = fmaf(v.x, v.x, fmaf(v.y, v.y, sq));
    }
  } else {
    for (int d = lane; d < head_dim; d += 32) {
      const float v = to_float(x[d]);
      mine[d] = v;
      sq = fmaf(v, v, sq);
    }
  }
  sq = warp_sum(sq);
  const float inv = w != nullptr ? 1.f / sqrtf(sq / float(head_dim) + eps) : 1.f;
  __syncwarp();
  // the value at dimension d after its norm
  auto normed = [&](int d) { return w != nullptr ? mine[d] * inv * w[d] : mine[d]; };
  if (vec) {   // half and head_dim are even: two neighbouring pairs (or two passing dimensions) a step
    for (int i = 2 * lane; i < head_dim - half; i += 64) {
      if (i < half) {
        const float u0 = normed(i), u1 = normed(i + 1), v0 = normed(i + half), v1 = normed(i + half + 1);
        const float a0 = u0 * cs_s[i] - v0 * sn_s[i], a1 = u1 * cs_s[i + 1] - v1 * sn_s[i + 1];
        const float b0 = v0 * cs_s[i] + u0 * sn_s[i], b1 = v1 * cs_s[i + 1] + u1 * sn_s[i + 1];
        store2(x + i, a0, a1);
        store2(x + i + half, b0, b1);
        if (kdst != nullptr) { store2(kdst + i, a0, a1); store2(kdst + i + half, b0, b1); }
      } else {
        const int d = i + half;   // the dimensions after the rotated ones pass with their norm alone
        const float a0 = normed(d), a1 = normed(d + 1);
        if (w != nullptr) store2(x + d, a0, a1);
        if (kdst != nullptr) store2(kdst + d, a0, a1);
      }
    }
    continue;
  }
  for (int i = lane; i < head_dim - half; i += 32) {
    if (i < half) {
      const float u = normed(i), v = normed(i + half);
      const T a = from_float<T>(u * cs_s[i] - v * sn_s[i]), b = from_float<T>(v * cs_s[i] + u * sn_s[i]);
      x[i] = a;
      x[i + half] = b;
      if (kdst != nullptr) { kdst[i] = a; kdst[i + half] = b; }
    } else {
      const int d = i + half;
      const T a = w != nullptr ? from_float<T>(mine[d] * inv * w[d]) : x[d];
      if (w != nullptr) x[d] = a;
      if (kdst != nullptr) kdst[d] = a;
    }
  }
  }
}

// out = x + weight_sum * (a / rms(a) * wa + b / rms(b) * wb): two branches' outputs, each normalised over the row with a
// gain of its own, join the residual stream. All float.
__global__ void __launch_bounds__(256)
pair_norm_add_kernel(const float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                     const float* __restrict__ wb, float* __restrict__ out, int width, float eps, float share) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t at = size_t(blockIdx.x) * width;
  float sa = 0.f, sb = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float va = a[at + d], vb = b[at + d];
    sa = fmaf(va, va, sa);
    sb = fmaf(vb, vb, sb);
  }
  const float inv_a = 1.f / sqrtf(block_sum(sa, scratch) / float(width) + eps);
  const float inv_b = 1.f / sqrtf(block_sum(sb, scratch) / float(width) + eps);
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    out[at + d] = x[at + d] + share * (a[at + d] * inv_a * wa[d] + b[at + d] * inv_b * wb[d]);
}
}  // namespace

// With k_cache (may be null) the launch also writes the row's keys (columns k_col .., n_kv_heads heads of head_dim, after
// their rotation) and values (columns v_col .., heads of v_head_dim) to the row's slot of the paged cache.
// With q_norm_w / k_norm_w (float [head_dim]; both or neither) every head is RMS-normed before its rotation: the first
// n_q_heads heads with q_norm_w, the others with k_norm_w. `magnitude` multiplies cos and sin.
extern "C" int r2_rotate_half(void* buf, int row_stride, int n_rows, int n_heads, int head_dim, int rot_dims, const float* inv_freq,
                              const int32_t* positions, void* k_cache, void* v_cache, const int32_t* slot_mapping, int k_col, int v_col,
                              int n_kv_heads, int v_head_dim, int page_size, long long page_stride, int n_pages,
                              const float* q_norm_w, const float* k_norm_w, int n_q_heads, float norm_eps, float magnitude, int dtype,
                              cudaStream_t stream) {
  const bool normed = q_norm_w != nullptr || k_norm_w != nullptr;
  if (n_rows <= 0 || (rot_dims == 0 && k_cache == nullptr && !normed)) return R2_OK;
  if (n_heads < 1 || rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > head_dim) return R2_BAD_SHAPE;
  if (k_cache != nullptr && (v_cache == nullptr || slot_mapping == nullptr || n_kv_heads < 1 || v_head_dim < 1 || page_size < 1)) return R2_BAD_SHAPE;
  const int half = rot_dims / 2;
  if (normed || magnitude != 1.f) {
    if (head_dim > NORM_ROTATE_MAX_DIM || n_q_heads < 0 || n_q_heads > n_heads) return R2_BAD_SHAPE;
    if ((n_q_heads > 0 && normed && q_norm_w == nullptr) || (n_q_heads < n_heads && normed && k_norm_w == nullptr)) return R2_BAD_SHAPE;
    // few rows (a decode step): a row's units spread over several CTAs; a prompt step's rows: one CTA a row, its cosines and sines made
    // once (11.8 against 14.4 us at 2,048 rows of 18 units); beyond that the SMs are full either way and the spread form is the faster
    // again (230 against 372 us at 65,536 rows)
    const bool one_cta_a_row = n_rows >= 512 && n_rows < 16384;
    const dim3 grid2(n_rows, one_cta_a_row ? 1 : (n_heads + (k_cache != nullptr ? n_kv_heads : 0) + NORM_ROTATE_WARPS - 1) / NORM_ROTATE_WARPS);
    // neighbouring elements as one access: every size, stride and column that an address is made of is even
    const bool pairs_ok = head_dim % 2 == 0 && half % 2 == 0 && row_stride % 2 == 0 &&
                          (k_cache == nullptr || (k_col % 2 == 0 && v_col % 2 == 0 && v_head_dim % 2 == 0 && page_stride % 2 == 0));
    if (dtype == R2_F32) {
      const bool vec = pairs_ok && pair_aligned((const float*)buf) && (k_cache == nullptr || (pair_aligned((const float*)k_cache) && pair_aligned((const float*)v_cache)));
      r2_launch(norm_rotate_half_kernel<float>, grid2, dim3(NORM_ROTATE_WARPS * 32), size_t(0), stream, (float*)buf, row_stride, n_heads, n_q_heads, head_dim,
                half, inv_freq, magnitude, q_norm_w, k_norm_w, norm_eps, positions, (float*)k_cache, (float*)v_cache, slot_mapping, k_col, v_col,
                n_kv_heads, v_head_dim, page_size, page_stride, n_pages, int(vec));
    } else if (dtype == R2_BF16) {
      const bool vec = pairs_ok && pair_aligned((const bf16*)buf) && (k_cache == nullptr || (pair_aligned((const bf16*)k_cache) && pair_aligned((const bf16*)v_cache)));
      r2_launch(norm_rotate_half_kernel<bf16>, grid2, dim3(NORM_ROTATE_WARPS * 32), size_t(0), stream, (bf16*)buf, row_stride, n_heads, n_q_heads, head_dim,
                half, inv_freq, magnitude, q_norm_w, k_norm_w, norm_eps, positions, (bf16*)k_cache, (bf16*)v_cache, slot_mapping, k_col, v_col,
                n_kv_heads, v_head_dim, page_size, page_stride, n_pages, int(vec));
    } else {
      return R2_BAD_DTYPE;
    }
    return launch_status();
  }
  dim3 grid(n_rows, k_cache != nullptr ? 1 : (n_heads * half + 1023) / 1024);
  if (dtype == R2_F32) {
    r2_launch(rotate_half_kernel<float>, grid, dim3(256), size_t(0), stream, (float*)buf, row_stride, n_heads, head_dim, half, inv_freq, positions,
              (float*)k_cache, (float*)v_cache, slot_mapping, k_col, v_col, n_kv_heads, v_head_dim, page_size, page_stride, n_pages);
  } else if (dtype == R2_BF16) {
    r2_launch(rotate_half_kernel<bf16>, grid, dim3(256), size_t(0), stream, (bf16*)buf, row_stride, n_heads, head_dim, half, inv_freq, positions,
              (bf16*)k_cache, (bf16*)v_cache, slot_mapping, k_col, v_col, n_kv_heads, v_head_dim, page_size, page_stride, n_pages);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

extern "C" int r2_pair_norm_add(const float* x, const float* a, const float* b, const float* wa, const float* wb, float* out,
                                int n_rows, int width, float eps, float share, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1) return R2_BAD_SHAPE;
  r2_launch(pair_norm_add_kernel, dim3(n_rows), dim3(256), size_t(0), stream, x, a, b, wa, wb, out, width, eps, share);
  return launch_status();
}

// ---- a sublayer's output, normalised, joins the stream (and the next sublayer's input leaves with it) --------------
// out = x + y / rms(y) * w, all float; with `next_w` also h = out / rms(out) * next_w in the compute dtype: the norm after a
// sublayer, the residual sum and the norm before the next sublayer in one pass. One CTA per row; the row stays in
// registers between the passes (ROWS_PER_THREAD elements a thread) where it fits, else it is read again.
namespace {
constexpr int NORM_ADD_THREADS = 256, NORM_ADD_KEEP = 8;

template <typename O>
__global__ void __launch_bounds__(NORM_ADD_THREADS)
norm_add_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ out,
                const float* __restrict__ next_w, O* __restrict__ next, int width, float eps, float next_eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t at = size_t(blockIdx.x) * width;
  const bool fits = width <= NORM_ADD_THREADS * NORM_ADD_KEEP;
  float keep[NORM_ADD_KEEP];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_ADD_KEEP; ++i) {
    const int d = threadIdx.x + i * NORM_ADD_THREADS;
    keep[i] = (fits && d < width) ? y[at + d] : 0.f;
    sq = fmaf(keep[i], keep[i], sq);
  }
  if (!fits)
    for (int d = threadIdx.x; d < width; d += NORM_ADD_THREADS) sq = fmaf(y[at + d], y[at + d], sq);
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / float(width) + eps);
  float sq_out = 0.f;
  if (fits) {
#pragma unroll
    for (int i = 0; i < NORM_ADD_KEEP; ++i) {
      const int d = threadIdx.x + i * NORM_ADD_THREADS;
      if (d < width) {
        keep[i] = x[at + d] + keep[i] * inv * w[d];
        out[at + d] = keep[i];
        sq_out = fmaf(keep[i], keep[i], sq_out);
      }
    }
  } else {
    for (int d = threadIdx.x; d < width; d += NORM_ADD_THREADS) {
      const float v = x[at + d] + y[at + d] * inv * w[d];
      out[at + d] = v;
      sq_out = fmaf(v, v, sq_out);
    }
  }
  if (next == nullptr) return;
  const float inv_out = 1.f / sqrtf(block_sum(sq_out, scratch) / float(width) + next_eps);
  if (fits) {
#pragma unroll
    for (int i = 0; i < NORM_ADD_KEEP; ++i) {
      const int d = threadIdx.x + i * NORM_ADD_THREADS;
      if (d < width) next[at + d] = from_float<O>(keep[i] * inv_out * next_w[d]);
    }
  } else {
    for (int d = threadIdx.x; d < width; d += NORM_ADD_THREADS) next[at + d] = from_float<O>(out[at + d] * inv_out * next_w[d]);
  }
}

// xIELU: for z > 0, a_pos z^2 + z / 2; for z <= 0, a_neg (e^z - 1 - z) + z / 2 (a_pos, a_neg are made from the layer's two
// learned numbers on the host). In float, rounded once on the way out.
__device__ __forceinline__ float xielu(float z, float a_pos, float a_neg) {
  return z > 0.f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, expm1f(z) - z, 0.5f * z);
}

template <typename T>
__global__ void __launch_bounds__(256)
xielu_kernel(const T* __restrict__ in, int in_stride, T* __restrict__ out, int out_stride, int width, float a_pos, float a_neg) {
  pdl_launch_dependents();
  pdl_wait();
  const T* r = in + size_t(blockIdx.x) * in_stride;
  T* o = out + size_t(blockIdx.x) * out_stride;
  if (width % 2 == 0 && pair_aligned(r) && pair_aligned(o) && in_stride % 2 == 0 && out_stride % 2 == 0) {
    for (int d = 2 * (blockIdx.y * blockDim.x + threadIdx.x); d < width; d += 2 * gridDim.y * blockDim.x) {
      const float2 z = load2(r + d);
      store2(o + d, xielu(z.x, a_pos, a_neg), xielu(z.y, a_pos, a_neg));
    }
    return;
  }
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < width; d += gridDim.y * blockDim.x)
    o[d] = from_float<T>(xielu(to_float(r[d]), a_pos, a_neg));
}

// bfloat16 rows that start on 16-byte boundaries: eight numbers per thread, one 16-byte load and one store.
__global__ void __launch_bounds__(256)
xielu_vec8_kernel(const bf16* __restrict__ in, int in_stride, bf16* __restrict__ out, int out_stride, int width, float a_pos, float a_neg) {
  pdl_launch_dependents();
  pdl_wait();
  const bf16* r = in + size_t(blockIdx.x) * in_stride;
  bf16* o = out + size_t(blockIdx.x) * out_stride;
  for (int d = 8 * (blockIdx.y * blockDim.x + threadIdx.x); d < width; d += 8 * gridDim.y * blockDim.x) {
    const uint4 zq = *reinterpret_cast<const uint4*>(r + d);
    const __nv_bfloat162* z2 = reinterpret_cast<const __nv_bfloat162*>(&zq);
    uint4 yq;
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&yq);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 z = __bfloat1622float2(z2[i]);
      y2[i] = __floats2bfloat162_rn(xielu(z.x, a_pos, a_neg), xielu(z.y, a_pos, a_neg));
    }
    *reinterpret_cast<uint4*>(o + d) = yq;
  }
}
}  // namespace

// x, y, out float [n_rows, width] (out may be x); w float [width]. With next_w (float [width]) and next ([n_rows, width] in
// `next_dtype`) the norm of the new stream rows is written too.
extern "C" int r2_norm_add(const float* x, const float* y, const float* w, float* out, const float* next_w, void* next,
                           int n_rows, int width, float eps, float next_eps, int next_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1) return R2_BAD_SHAPE;
  if (next != nullptr && next_w == nullptr) return R2_BAD_SHAPE;
  if (next == nullptr || next_dtype == R2_F32) {
    r2_launch(norm_add_kernel<float>, dim3(n_rows), dim3(NORM_ADD_THREADS), size_t(0), stream, x, y, w, out, next_w, (float*)next, width, eps, next_eps);
  } else if (next_dtype == R2_BF16) {
    r2_launch(norm_add_kernel<bf16>, dim3(n_rows), dim3(NORM_ADD_THREADS), size_t(0), stream, x, y, w, out, next_w, (bf16*)next, width, eps, next_eps);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

extern "C" int r2_xielu(const void* in, int in_stride, void* out, int out_stride, int n_rows, int width, float a_pos, float a_neg,
                        int dtype, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return R2_OK;
  dim3 grid(n_rows, (width + 511) / 512);
  if (dtype == R2_BF16 && width % 8 == 0 && in_stride % 8 == 0 && out_stride % 8 == 0 && !(reinterpret_cast<uintptr_t>(in) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    r2_launch(xielu_vec8_kernel, dim3(n_rows, (width + 2047) / 2048), dim3(256), size_t(0), stream, (const bf16*)in, in_stride, (bf16*)out, out_stride,
              width, a_pos, a_neg);
    return launch_status();
  }
  if (dtype == R2_F32) {
    r2_launch(xielu_kernel<float>, grid, dim3(256), size_t(0), stream, (const float*)in, in_stride, (float*)out, out_stride, width, a_pos, a_neg);
  } else if (dtype == R2_BF16) {
    r2_launch(xielu_kernel<bf16>, grid, dim3(256), size_t(0), stream, (const bf16*)in, in_stride, (bf16*)out, out_stride, width, a_pos, a_neg);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---- the norm AFTER a sum: out = (alpha x + y) / rms(alpha x + y) * w ------------------------------------------------
// The stream's rows are scaled, a sublayer's output joins them, and the sum is normalised: all float, one CTA per row, the row
// in registers between the passes where it fits (else the sum is made again, in the same order). `rounded` (may be null) also
// receives the new rows in the compute dtype: what the next sublayer's products read.
namespace {
template <typename O>
__global__ void __launch_bounds__(NORM_ADD_THREADS)
add_norm_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ out,
                O* __restrict__ rounded, int width, float alpha, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const size_t at = size_t(blockIdx.x) * width;
  const bool fits = width <= NORM_ADD_THREADS * NORM_ADD_KEEP;
  float keep[NORM_ADD_KEEP];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_ADD_KEEP; ++i) {
    const int d = threadIdx.x + i * NORM_ADD_THREADS;
    keep[i] = (fits && d < width) ? fmaf(alpha, x[at + d], y[at + d]) : 0.f;
    sq = fmaf(keep[i], keep[i], sq);
  }
  if (!fits)
    for (int d = threadIdx.x; d < width; d += NORM_ADD_THREADS) {
      const float v = fmaf(alpha, x[at + d], y[at + d]);
      sq = fmaf(v, v, sq);
    }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / float(width) + eps);
  if (fits) {
#pragma unroll
    for (int i = 0; i < NORM_ADD_KEEP; ++i) {
      const int d = threadIdx.x + i * NORM_ADD_THREADS;
      if (d < width) {
        const float v = keep[i] * inv * w[d];
        out[at + d] = v;
        if (rounded != nullptr) rounded[at + d] = from_float<O>(v);
      }
    }
  } else {
    for (int d = threadIdx.x; d < width; d += NORM_ADD_THREADS) {
      const float v = fmaf(alpha, x[at + d], y[at + d]) * inv * w[d];   // (out may be x: a thread reads what it alone writes)
      out[at + d] = v;
      if (rounded != nullptr) rounded[at + d] = from_float<O>(v);
    }
  }
}

template <typename O>
__global__ void __launch_bounds__(256)
round_rows_kernel(const float* __restrict__ x, O* __restrict__ out, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) out[i] = from_float<O>(x[i]);
}
}  // namespace

// x, y, out float [n_rows, width] (out may be x); w float [width]; rounded (may be null) [n_rows, width] in `rounded_dtype`.
extern "C" int r2_add_norm(const float* x, const float* y, const float* w, float* out, void* rounded, int n_rows, int width,
                           float alpha, float eps, int rounded_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1) return R2_BAD_SHAPE;
  if (rounded == nullptr || rounded_dtype == R2_F32) {
    r2_launch(add_norm_kernel<float>, dim3(n_rows), dim3(NORM_ADD_THREADS), size_t(0), stream, x, y, w, out, (float*)rounded, width, alpha, eps);
  } else if (rounded_dtype == R2_BF16) {
    r2_launch(add_norm_kernel<bf16>, dim3(n_rows), dim3(NORM_ADD_THREADS), size_t(0), stream, x, y, w, out, (bf16*)rounded, width, alpha, eps);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// The float rows of the stream in the compute dtype (contiguous, n numbers).
extern "C" int r2_round_rows(const float* x, void* out, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return R2_OK;
  const int blocks = int((n + 1023) / 1024 > 4096 ? 4096 : (n + 1023) / 1024);
  if (dtype == R2_BF16) {
    r2_launch(round_rows_kernel<bf16>, dim3(blocks), dim3(256), size_t(0), stream, x, (bf16*)out, size_t(n));
  } else if (dtype == R2_F32) {
    r2_launch(round_rows_kernel<float>, dim3(blocks), dim3(256), size_t(0), stream, x, (float*)out, size_t(n));
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
