// Small projections that must stay in 32-bit, the choice of experts, and the experts' activation.
//
//   r2_small_linear   out[t][n] = bias[n] + sum_k h[t][k] * w[n][k] in float, for a handful of outputs per row (gates
//                     of a recurrence, one gate per head, step sizes, router logits): weights and result are float
//                     whatever the activations' type, every output one warp's sum in a fixed order.
//   r2_route_top_k    router logits in float, the `top` largest per row (the lower index wins a tie), softmax over the
//                     chosen logits only -> a dense row of weights [T, experts] (zero for experts not chosen), and the
//                     choices themselves.
//   r2_route_scored   the same with sigmoid scores: an expert is chosen by its score plus a learned correction, only
//                     inside the best groups of neighbouring experts (a group counts by its two best), and weighted by
//                     its plain score over the chosen experts' sum; further rows of the weight matrix give sigmoid gates
//                     of their own (one number per row of the batch, e.g. for an expert that every row uses). Or with
//                     scores that are the softmax over all experts, groups that count by their best expert alone, and
//                     weights that are the chosen scores times a constant (not made to sum to one).
//   r2_expert_act     the inner activation of gated feed-forwards whose [gate | up] projections of several experts
//                     (and of one more expert that every row uses) lie side by side in one row; each expert's
//                     columns are multiplied by the row's weight for that expert, so that ONE down product over the
//                     stacked matrices is the weighted sum of the experts' outputs.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int MAX_EXPERTS = 1024;

template <typename T>
__global__ void __launch_bounds__(256)
small_linear_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ w, const float* __restrict__ bias,
                    float* __restrict__ out, int out_stride, int n_out, int width) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T* hr = h + size_t(t) * h_stride;
  for (int k = threadIdx.x; k < width; k += blockDim.x) row[k] = to_float(hr[k]);
  __syncthreads();
  for (int n = warp; n < n_out; n += n_warps) {
    const float* wr = w + size_t(n) * width;
    float acc = 0.f;
    for (int k = lane; k < width; k += 32) acc = fmaf(row[k], wr[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[size_t(t) * out_stride + n] = acc + (bias != nullptr ? bias[n] : 0.f);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
route_top_k_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ w, const float* __restrict__ bias,
                   float* __restrict__ dense, int32_t* __restrict__ chosen, float* __restrict__ chosen_weight,
                   int n_experts, int top, int width) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  float* row = smem;             // [width]
  float* logit = smem + width;   // [n_experts]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T* hr = h + size_t(t) * h_stride;
  for (int k = threadIdx.x; k < width; k += blockDim.x) row[k] = to_float(hr[k]);
  __syncthreads();
  for (int n = warp; n < n_experts; n += n_warps) {
    const float* wr = w + size_t(n) * width;
    float acc = 0.f;
    for (int k = lane; k < width; k += 32) acc = fmaf(row[k], wr[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) logit[n] = acc + (bias != nullptr ? bias[n] : 0.f);
  }
  for (int n = threadIdx.x; n < n_experts; n += blockDim.x) dense[size_t(t) * n_experts + n] = 0.f;
  __syncthreads();
  if (warp != 0) return;
  // the first warp picks the largest logit `top` times; a picked one is set to -inf. The first pick is the maximum
  // of the chosen, so the softmax over them needs no second pass for it.
  float best0 = 0.f, sum = 0.f;
  for (int c = 0; c < top; ++c) {
    float v = -INFINITY;
    int at = n_experts;
    for (int n = lane; n < n_experts; n += 32)
      if (logit[n] > v) { v = logit[n]; at = n; }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oat = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > v || (ov == v && oat < at)) { v = ov; at = oat; }
    }
    if (at >= n_experts) { at = c; v = best0; }   // logits that are not numbers: no index may leave the row
    if (c == 0) best0 = v;
    const float p = expf(v - best0);
    sum += p;
    if (lane == 0) {
      chosen[size_t(t) * top + c] = at;
      chosen_weight[size_t(t) * top + c] = p;
      logit[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float inv = 1.f / sum;
  for (int c = lane; c < top; c += 32) {
    const float p = chosen_weight[size_t(t) * top + c] * inv;
    chosen_weight[size_t(t) * top + c] = p;
    dense[size_t(t) * n_experts + chosen[size_t(t) * top + c]] = p;
  }
}

// Router with sigmoid scores. w holds n_experts rows of router weights and then n_extra more rows; their logits leave as
// they are in `extra` [T, n_extra] (gates whose sigmoid another kernel takes). s = sigmoid(logit); an expert's choice score is
// s + correction; the experts form n_groups equal groups of neighbours, a group's mark is the sum of its two largest
// choice scores (of its one, where a group is a single expert), and only experts of the `keep` groups with the largest marks
// can be chosen (the lower index wins a tie, among groups and among experts). The `top` largest choice scores are chosen; a
// chosen expert's weight is its s over the sum of the chosen s (+ 1e-20).
// softmax_scores: s = softmax of the logits over all experts instead of their sigmoids. mark_best_only: a group's mark is its
// largest choice score alone. normalise = 0: a chosen expert's weight is s * weight_scale.
template <typename T>
__global__ void __launch_bounds__(256)
route_scored_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ w, const float* __restrict__ correction,
                    float* __restrict__ dense, int32_t* __restrict__ chosen, float* __restrict__ chosen_weight,
                    float* __restrict__ extra, int n_experts, int n_extra, int top, int n_groups, int keep, int width,
                    int softmax_scores, int mark_best_only, int normalise, float weight_scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  float* row = smem;                    // [width]
  float* score = smem + width;          // [n_experts] sigmoid of the logit
  float* choice = score + n_experts;    // [n_experts] score + correction; -inf once picked or outside the kept groups
  float* mark = choice + n_experts;     // [n_groups]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const T* hr = h + size_t(t) * h_stride;
  for (int k = threadIdx.x; k < width; k += blockDim.x) row[k] = to_float(hr[k]);
  __syncthreads();
  for (int n = warp; n < n_experts + n_extra; n += n_warps) {
    const float* wr = w + size_t(n) * width;
    float acc = 0.f;
    for (int k = lane; k < width; k += 32) acc = fmaf(row[k], wr[k], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      if (n < n_experts) {
        const float s = softmax_scores ? acc : 1.f / (1.f + expf(-acc));   // (the softmax follows once all logits are there)
        score[n] = s;
        choice[n] = s + (correction != nullptr ? correction[n] : 0.f);
      } else {
        extra[size_t(t) * n_extra + (n - n_experts)] = acc;
      }
    }
  }
  for (int n = threadIdx.x; n < n_experts; n += blockDim.x) dense[size_t(t) * n_experts + n] = 0.f;
  __syncthreads();
  if (warp != 0) return;
  if (softmax_scores) {
    // s = exp(z - max) / sum over all experts, one warp, sums in a fixed order
    float top_z = -INFINITY;
    for (int n = lane; n < n_experts; n += 32) top_z = fmaxf(top_z, score[n]);
    for (int o = 16; o > 0; o >>= 1) top_z = fmaxf(top_z, __shfl_xor_sync(0xffffffffu, top_z, o));
    float total = 0.f;
    for (int n = lane; n < n_experts; n += 32) {
      const float e = expf(score[n] - top_z);
      score[n] = e;
      total += e;
    }
    total = warp_sum(total);
    const float inv_total = 1.f / total;
    for (int n = lane; n < n_experts; n += 32) {
      const float s = score[n] * inv_total;
      score[n] = s;
      choice[n] = s + (correction != nullptr ? correction[n] : 0.f);
    }
    __syncwarp();
  }
  const int size = n_experts / n_groups;
  if (keep < n_groups) {
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;   // the group's largest and second largest
      for (int n = g * size; n < (g + 1) * size; ++n) {
        const float c = choice[n];
        if (c > a) { b = a; a = c; }
        else if (c > b) b = c;
      }
      mark[g] = (size > 1 && !mark_best_only) ? a + b : a;
    }
    __syncwarp();
    // the kept groups: `keep` times the largest mark; a kept group's mark becomes +inf, and what is not +inf at the end is out
    for (int c = 0; c < keep; ++c) {
      float v = -INFINITY;
      int at = n_groups;
      for (int g = lane; g < n_groups; g += 32)
        if (mark[g] != INFINITY && (mark[g] > v || at == n_groups)) { v = mark[g]; at = g; }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oat = __shfl_xor_sync(0xffffffffu, at, o);
        if (oat < n_groups && (at == n_groups || ov > v || (ov == v && oat < at))) { v = ov; at = oat; }
      }
      if (lane == 0 && at < n_groups) mark[at] = INFINITY;
      __syncwarp();
    }
    for (int n = lane; n < n_experts; n += 32)
      if (mark[n / size] != INFINITY) choice[n] = -INFINITY;
    __syncwarp();
  }
  float sum = 0.f;
  for (int c = 0; c < top; ++c) {
    float v = -INFINITY;
    int at = n_experts;
    for (int n = lane; n < n_experts; n += 32)
      if (choice[n] > v) { v = choice[n]; at = n; }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oat = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > v || (ov == v && oat < at)) { v = ov; at = oat; }
    }
    if (at >= n_experts) at = c;   // scores that are not numbers: no index may leave the row
    const float s = score[at];
    sum += s;
    if (lane == 0) {
      chosen[size_t(t) * top + c] = at;
      chosen_weight[size_t(t) * top + c] = s;
      choice[at] = -INFINITY;
    }
    __syncwarp();
  }
  const float inv = normalise ? 1.f / (sum + 1e-20f) : weight_scale;
  for (int c = lane; c < top; c += 32) {
    const float p = chosen_weight[size_t(t) * top + c] * inv;
    chosen_weight[size_t(t) * top + c] = p;
    dense[size_t(t) * n_experts + chosen[size_t(t) * top + c]] = p;
  }
}

constexpr int KIND_CLAMPED_SWISH = 0, KIND_RELU = 1, KIND_SILU = 2;

__device__ __forceinline__ float gated_unit(float g, float u, int kind, float limit, float alpha, float up_offset) {
  if (kind == KIND_RELU) return fmaxf(g, 0.f) * u;
  if (kind == KIND_SILU) return g / (1.f + expf(-g)) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + up_offset);
}

// A row of `gate_up` holds [gates of all `inner` columns | ups of all `inner` columns]. The first n_experts *
// expert_width columns belong to routed experts (limit `limit`, times the row's weight for the expert); the rest to the
// expert that every row uses (limit `tail_limit`; weight one, or sigmoid(tail_gate[row]) where a gate is given).
// n_experts = 0: one plain gated unit.
template <typename T>
__global__ void __launch_bounds__(256)
expert_act_kernel(const T* __restrict__ gate_up, int in_stride, T* __restrict__ out, int out_stride, int inner, int kind,
                  float limit, float alpha, float up_offset, const float* __restrict__ route, int n_experts, int expert_width,
                  float tail_limit, const float* __restrict__ tail_gate, int tail_gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const T* in = gate_up + size_t(blockIdx.x) * in_stride;
  // the weight of the columns after the routed experts': one, or the sigmoid of the row's gate logit
  const float tail_weight = tail_gate != nullptr ? 1.f / (1.f + expf(-tail_gate[size_t(blockIdx.x) * tail_gate_stride])) : 1.f;
  T* o = out + size_t(blockIdx.x) * out_stride;
  const int routed = n_experts * expert_width;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < inner; f += gridDim.y * blockDim.x) {
    const bool tail = f >= routed;
    const float weight = tail ? tail_weight : route[size_t(blockIdx.x) * n_experts + f / expert_width];
    float y = 0.f;
    if (weight != 0.f) y = weight * gated_unit(to_float(in[f]), to_float(in[inner + f]), kind, tail ? tail_limit : limit, alpha, up_offset);
    o[f] = from_float<T>(y);
  }
}

}  // namespace

extern "C" int r2_small_linear(const void* h, int h_stride, const float* w, const float* bias, float* out, int out_stride,
                               int n_rows, int n_out, int width, int dtype, cudaStream_t stream) {
  if (n_rows <= 0 || n_out <= 0) return R2_OK;
  if (width < 1) return R2_BAD_SHAPE;
  const size_t smem = sizeof(float) * width;
  if (smem > 48 * 1024) return R2_UNSUPPORTED;
  const int threads = n_out >= 8 ? 256 : 32 * n_out;
  if (dtype == R2_F32) {
    r2_launch(small_linear_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, (const float*)h, h_stride, w, bias, out, out_stride, n_out, width);
  } else if (dtype == R2_BF16) {
    r2_launch(small_linear_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, (const bf16*)h, h_stride, w, bias, out, out_stride, n_out, width);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

extern "C" int r2_route_top_k(const void* h, int h_stride, const float* w, const float* bias, float* dense, int32_t* chosen,
                              float* chosen_weight, int n_rows, int n_experts, int top, int width, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1 || n_experts < 1 || n_experts > MAX_EXPERTS || top < 1 || top > n_experts) return R2_BAD_SHAPE;
  const size_t smem = sizeof(float) * (size_t(width) + n_experts);
  if (smem > 48 * 1024) return R2_UNSUPPORTED;
  if (dtype == R2_F32) {
    r2_launch(route_top_k_kernel<float>, dim3(n_rows), dim3(256), smem, stream, (const float*)h, h_stride, w, bias, dense, chosen, chosen_weight, n_experts, top, width);
  } else if (dtype == R2_BF16) {
    r2_launch(route_top_k_kernel<bf16>, dim3(n_rows), dim3(256), smem, stream, (const bf16*)h, h_stride, w, bias, dense, chosen, chosen_weight, n_experts, top, width);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// w float [n_experts + n_extra, width]; correction float [n_experts] (may be null); dense [T, n_experts], chosen / chosen_weight
// [T, top], extra [T, n_extra] (the further rows' logits; null when n_extra is 0). softmax_scores, mark_best_only, normalise and
// weight_scale choose the router's form (see the kernel).
extern "C" int r2_route_scored(const void* h, int h_stride, const float* w, const float* correction, float* dense, int32_t* chosen,
                               float* chosen_weight, float* extra, int n_rows, int n_experts, int n_extra, int top, int n_groups,
                               int keep, int width, int softmax_scores, int mark_best_only, int normalise, float weight_scale,
                               int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1 || n_experts < 1 || n_experts > MAX_EXPERTS || top < 1 || n_groups < 1 || n_experts % n_groups != 0 || keep < 1 ||
      keep > n_groups || top > n_experts / n_groups * keep || n_extra < 0 || (n_extra > 0 && extra == nullptr)) return R2_BAD_SHAPE;
  const size_t smem = sizeof(float) * (size_t(width) + 2 * n_experts + n_groups);
  if (smem > 48 * 1024) return R2_UNSUPPORTED;
  if (dtype == R2_F32) {
    r2_launch(route_scored_kernel<float>, dim3(n_rows), dim3(256), smem, stream, (const float*)h, h_stride, w, correction, dense, chosen,
              chosen_weight, extra, n_experts, n_extra, top, n_groups, keep, width, softmax_scores, mark_best_only, normalise, weight_scale);
  } else if (dtype == R2_BF16) {
    r2_launch(route_scored_kernel<bf16>, dim3(n_rows), dim3(256), smem, stream, (const bf16*)h, h_stride, w, correction, dense, chosen,
              chosen_weight, extra, n_experts, n_extra, top, n_groups, keep, width, softmax_scores, mark_best_only, normalise, weight_scale);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

extern "C" int r2_expert_act(const void* gate_up, int in_stride, void* out, int out_stride, int n_rows, int inner, int kind,
                             float limit, float alpha, float up_offset, const float* route, int n_experts, int expert_width,
                             float tail_limit, const float* tail_gate, int tail_gate_stride, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (inner < 1 || n_experts < 0 || (n_experts > 0 && (expert_width < 1 || route == nullptr || n_experts * expert_width > inner))) return R2_BAD_SHAPE;
  if (n_experts == 0) expert_width = 1;
  dim3 grid(n_rows, (inner + 1023) / 1024);
  if (dtype == R2_F32) {
    r2_launch(expert_act_kernel<float>, grid, dim3(256), size_t(0), stream, (const float*)gate_up, in_stride, (float*)out, out_stride, inner, kind,
              limit, alpha, up_offset, route, n_experts, expert_width, tail_limit, tail_gate, tail_gate_stride);
  } else if (dtype == R2_BF16) {
    r2_launch(expert_act_kernel<bf16>, grid, dim3(256), size_t(0), stream, (const bf16*)gate_up, in_stride, (bf16*)out, out_stride, inner, kind,
              limit, alpha, up_offset, route, n_experts, expert_width, tail_limit, tail_gate, tail_gate_stride);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
