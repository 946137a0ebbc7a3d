// Paged causal attention on the CUDA cores, all arithmetic in float: the true 32-bit path, and
// the general path of the bfloat16 engine for head sizes or batches the tensor-core kernels refuse.
//
// One warp computes one (row, head): it walks the row's visible keys in position order in tiles
// of 32 (lane = key), keeps a running maximum and sum (online softmax) and accumulates P.V with
// lanes over the head dimension. The walk depends only on the row's position, its window and
// the head size, never on how the step was cut or batched, so a row's output is the same bits
// whichever batch it came in. It also takes what the fast kernels leave out: a value head size that
// differs from the key's, a window that keeps a sequence's first keys, a sink in the softmax's
// denominator, an output gate, and values that are the first numbers of the key rows themselves (a
// cache of latents: the value pointer is the key pointer and a value row is as long as a key row).
//
// Reference formulas: kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-240
// (scores * scale 179, visibility 186-212, softmax 215-240, PV 182-183, pad rows zero 140).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int WIDE_HEAD_DIM = 1024;   // a second instance takes rows of up to this many numbers (a cache of long latents)

template <typename T, int MAX_HEAD_DIM>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long page_stride,
                      int page_size, const int32_t* __restrict__ block_tables, int table_width,
                      const int32_t* __restrict__ row_entry, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ seq_lens, int n_heads, int n_kv_heads, int head_dim, int v_head_dim,
                      float scale, int window, int keep_first, int sink, const T* __restrict__ gate, int gate_row_stride,
                      int n_pages, float softcap, const float* __restrict__ sinks, const float* __restrict__ head_gate,
                      int head_gate_stride, int v_row_stride) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  __shared__ float q_s[WARPS][MAX_HEAD_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= n_heads) return;
  T* o = out + size_t(t) * out_row_stride + size_t(h) * v_head_dim;
  const int e = row_entry[t];
  if (e < 0) {  // a pad row
    for (int d = lane; d < v_head_dim; d += 32) o[d] = from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int seq_len = seq_lens[e];
  const int kvh = h / (n_heads / n_kv_heads);
  const int32_t* table = block_tables + size_t(e) * table_width;
  const T* qr = q + size_t(t) * q_row_stride + size_t(h) * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_s[warp][d] = to_float(qr[d]);
  __syncwarp();

  const int last = pos < seq_len - 1 ? pos : seq_len - 1;       // newest visible key
  const int first = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  // With a window, the sequence's first `keep_first` keys stay visible: they are walked first, as a
  // range of their own, so that the walk depends on the row's position alone.
  const int kept = window > 0 ? (keep_first < first ? keep_first : first) : 0;
  // a sink: an extra term in the sum and nothing in the output; exp(0), or exp(sinks[h]) where heads have learned ones
  float m = sinks != nullptr ? sinks[h] : (sink ? 0.f : -INFINITY), l = (sink || sinks != nullptr) ? 1.f : 0.f;
  float acc[MAX_HEAD_DIM / 32];
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
  const size_t k_head_off = size_t(kvh) * page_size * head_dim;
  const size_t v_head_off = size_t(kvh) * page_size * v_row_stride;

  for (int range = 0; range < 2; ++range) {
    const int lo = range == 0 ? 0 : first, hi = range == 0 ? kept - 1 : last;
    for (int j0 = lo; j0 <= hi; j0 += 32) {
      int j = j0 + lane;
      bool valid = j <= hi;
      float s = -INFINITY;
      if (valid) {
        int page = table[j / page_size];
        page = (page < 0 || page >= n_pages) ? 0 : page;
        const T* kr = k_cache + size_t(page) * page_stride + k_head_off + size_t(j % page_size) * head_dim;
        float dot = 0.f;
        for (int d = 0; d < head_dim; ++d) dot = fmaf(q_s[warp][d], to_float(kr[d]), dot);
        s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);   // scores are capped before the softmax
      }
      float m_new = fmaxf(m, warp_max(s));
      float corr = expf(m - m_new);  // exp(-inf) = 0 on the first tile
      float p = valid ? expf(s - m_new) : 0.f;
      l = l * corr + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] *= corr;
      int n_valid = hi - j0 + 1 < 32 ? hi - j0 + 1 : 32;
      for (int jj = 0; jj < n_valid; ++jj) {
        float pj = __shfl_sync(0xffffffffu, p, jj);
        int key = j0 + jj;
        int page = table[key / page_size];
        page = (page < 0 || page >= n_pages) ? 0 : page;
        const T* vr = v_cache + size_t(page) * page_stride + v_head_off + size_t(key % page_size) * v_row_stride;
#pragma unroll
        for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
          int d = lane + 32 * i;
          if (d < v_head_dim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
        }
      }
    }
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  const T* gr = gate != nullptr ? gate + size_t(t) * gate_row_stride + size_t(h) * v_head_dim : nullptr;
  // one gate per head: sigmoid of a float logit
  if (head_gate != nullptr) inv *= 1.f / (1.f + expf(-head_gate[size_t(t) * head_gate_stride + h]));
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
    int d = lane + 32 * i;
    if (d < v_head_dim) {
      float y = acc[i] * inv;
      if (gr != nullptr) y *= 1.f / (1.f + expf(-to_float(gr[d])));   // the output gate: sigmoid of the gate's column
      o[d] = from_float<T>(y);
    }
  }
}

}  // namespace

// q [T, n_heads * head_dim] with row stride q_row_stride (it may be a slice of a fused projection),
// out [T, n_heads * v_head_dim]; the cache of this layer as in r2_kv_write. `window` > 0 limits a row
// at position p to the keys (p - window, p] and, with `keep_first`, the sequence's first keep_first keys;
// `sink` adds one to the softmax's denominator; `gate` (may be null; [T, n_heads * v_head_dim] with its
// own row stride) multiplies the output by its sigmoid. `softcap` > 0 caps the scaled scores (cap * tanh(s / cap));
// `sinks` (may be null; float [n_heads]) puts exp(sinks[h]) into head h's denominator; `head_gate` (may be null; float
// [T, n_heads] with its own row stride) multiplies head h's output by the sigmoid of its entry. `v_row_stride` (0: v_head_dim)
// is the length of a value row in the cache: with v_cache = k_cache and v_row_stride = head_dim the values are the first
// v_head_dim numbers of the keys.
extern "C" int r2_attention_simt(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                                 const void* v_cache, long long page_stride, int page_size,
                                 const int32_t* block_tables, int table_width, const int32_t* row_entry,
                                 const int32_t* positions, const int32_t* seq_lens, int n_rows, int n_heads,
                                 int n_kv_heads, int head_dim, int v_head_dim, float scale, int window, int keep_first,
                                 int sink, const void* gate, int gate_row_stride, int n_pages, int dtype,
                                 float softcap, const float* sinks, const float* head_gate, int head_gate_stride,
                                 int v_row_stride, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (head_dim < 1 || head_dim > WIDE_HEAD_DIM || v_head_dim < 1 || v_head_dim > WIDE_HEAD_DIM) return R2_UNSUPPORTED;
  const bool wide = head_dim > 256 || v_head_dim > 256;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0 || keep_first < 0) return R2_BAD_SHAPE;
  if (v_row_stride <= 0) v_row_stride = v_head_dim;   // values in rows of their own
  if (v_row_stride < v_head_dim) return R2_BAD_SHAPE;
  dim3 grid(n_rows, (n_heads + WARPS - 1) / WARPS);
  if (dtype == R2_F32) {
    if (wide) r2_launch(attention_simt_kernel<float, WIDE_HEAD_DIM>, dim3(grid), dim3(WARPS * 32), size_t(0), stream,
        (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_cache, (const float*)v_cache,
        page_stride, page_size, block_tables, table_width, row_entry, positions, seq_lens, n_heads, n_kv_heads,
        head_dim, v_head_dim, scale, window, keep_first, sink, (const float*)gate, gate_row_stride, n_pages, softcap, sinks, head_gate, head_gate_stride, v_row_stride);
    else r2_launch(attention_simt_kernel<float, 256>, dim3(grid), dim3(WARPS * 32), size_t(0), stream,
        (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_cache, (const float*)v_cache,
        page_stride, page_size, block_tables, table_width, row_entry, positions, seq_lens, n_heads, n_kv_heads,
        head_dim, v_head_dim, scale, window, keep_first, sink, (const float*)gate, gate_row_stride, n_pages, softcap, sinks, head_gate, head_gate_stride, v_row_stride);
  } else if (dtype == R2_BF16) {
    if (wide) r2_launch(attention_simt_kernel<bf16, WIDE_HEAD_DIM>, dim3(grid), dim3(WARPS * 32), size_t(0), stream,
        (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_cache, (const bf16*)v_cache,
        page_stride, page_size, block_tables, table_width, row_entry, positions, seq_lens, n_heads, n_kv_heads,
        head_dim, v_head_dim, scale, window, keep_first, sink, (const bf16*)gate, gate_row_stride, n_pages, softcap, sinks, head_gate, head_gate_stride, v_row_stride);
    else r2_launch(attention_simt_kernel<bf16, 256>, dim3(grid), dim3(WARPS * 32), size_t(0), stream,
        (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_cache, (const bf16*)v_cache,
        page_stride, page_size, block_tables, table_width, row_entry, positions, seq_lens, n_heads, n_kv_heads,
        head_dim, v_head_dim, scale, window, keep_first, sink, (const bf16*)gate, gate_row_stride, n_pages, softcap, sinks, head_gate, head_gate_stride, v_row_stride);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
