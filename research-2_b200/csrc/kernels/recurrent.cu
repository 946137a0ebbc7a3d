// Mixers that carry a state of fixed size from token to token instead of a cache that grows: a matrix
// memory with exponential gates (mLSTM), a state-space layer (Mamba-2's recurrence) and retention (linear attention
// with one fixed decay per head, keep_t = decay and take_t = 1; its queries and keys are rotated by position on their way
// into shared memory, in float, so what enters the recurrence is never rounded to 16 bits), all of the form
//
//     S_t = keep_t * S_(t-1) + take_t * w_t v_t^T        S: [rows x columns] per head, float
//     y_t = S_t^T r_t  (+ what the layer adds)
//
// with a write vector w (keys; B), a read vector r (queries; C) and values v. One kernel serves both and
// serves prompts, portions and single decoded tokens alike: a CTA owns one (entry, head, slice of the
// value columns), takes the state from the request's slot (or zeros for a sequence's first rows), walks the
// entry's rows in order and puts the state back. A thread keeps RPT rows of one column in registers; the
// rows of a column are spread over G neighbouring lanes, so the sum over rows is a shuffle and the walk
// needs no barrier but the one that stages the next rows' vectors in shared memory. All arithmetic that
// enters the recurrence is float: gates, decays, their logarithms and exponentials, step sizes, the state.
// The order of operations depends on the row's position alone, so a row's result is the same bits however
// its prompt was cut into steps.
//
// Beside it: the short causal convolution in front of the state-space recurrence (its last inputs are
// state too), and the norm over groups of columns with a gate that follows both mixers.
#include <math.h>

#include "common.cuh"

namespace {

// Rows whose vectors are staged at a time: 32 (16 where a thread has 32 rows of a column in registers); 4 for launches in
// which every entry is a single decoded row (less shared memory: more CTAs to an SM).
constexpr int MAX_TILE = 32, SMALL_TILE = 4;
constexpr int NORM_COPIES = 8;  // copies of a matrix memory's normaliser and maximum: one per slice of the columns at most

constexpr int MODE_MLSTM = 0, MODE_SSD = 1, MODE_DECAY = 2;

__device__ __forceinline__ float soft_cap(float x, float cap) { return cap > 0.f ? cap * tanhf(x / cap) : x; }
__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct ScanArgs {
  const void* read; int read_stride;     // r: [T, groups * rows] (queries: a group per head)
  const void* write; int write_stride;   // w: [T, groups * rows]
  const void* value; int value_stride;   // v: [T, heads * cols]
  const float* gates; int gates_stride;  // mLSTM: [T, 2 heads] input gates then forget gates, before the cap
                                         // state space: [T, heads] step sizes before bias and softplus
  const float* step_bias;                // state space, per head
  const float* log_rate;                 // state space, per head: the decay is exp(-exp(log_rate) * step)
  const float* skip;                     // state space, per head: y += skip * v
  float cap;                             // mLSTM: gates are cap * tanh(x / cap); 0 = no cap
  float read_scale;                      // r is multiplied by it
  float write_scale;                     // retention: w is multiplied by it (after the rotation)
  const float* decay;                    // retention, per head: keep
  const float* inv_freq; int rot_half;   // retention: of r and w the first 2 * rot_half dimensions turn, dimension i with
  const int32_t* positions;              // i + rot_half, by the angle positions[row] * inv_freq[i] (rot_half 0: no rotation)
  float* state; long long slot_stride;   // per request slot; per head: S [rows][cols] (+ mLSTM: NORM_COPIES times n [rows], m)
  int head_stride;
  const int32_t* q_start; const int32_t* state_slot; const int32_t* fresh;
  float* out; int out_stride;            // [T, heads * cols] float
  int heads_per_group, rows, cols, G, cv;
  int single_rows;                       // a hint: no entry has more than one row (a decode step)
  // state space: the convolution's last inputs, kept by the CTA of (entry, head 0, slice 0)
  const void* conv_in; int conv_in_stride; int conv_channels, conv_taps; long long conv_state_off;
};

template <typename T, int RPT, int MODE, int TILE>
__global__ void __launch_bounds__(256)
outer_scan_kernel(const ScanArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int e = blockIdx.x, h = blockIdx.y;
  const int row0 = a.q_start[e], row1 = a.q_start[e + 1];
  if (row1 <= row0) return;  // an entry without rows touches no slot
  const int G = a.G, cv = a.cv, rows = a.rows, cols = a.cols;
  const int padded = RPT * G;
  float* rs = smem;                       // [TILE][padded]
  float* ws = rs + TILE * padded;         // [TILE][padded]
  float* vs = ws + TILE * padded;         // [TILE][cv]
  float* g0 = vs + TILE * cv;             // [TILE] log input gate, then take | step
  float* g1 = g0 + TILE;                  // [TILE] log forget gate, then keep | decay
  float* g2 = g1 + TILE;                  // [TILE] running maximum after the row
  // a thread has the rows g * RPT .. g * RPT + RPT - 1 of column j; the G threads of a column are neighbouring lanes
  const int tid = threadIdx.x, g = tid % G, jl = tid / G;
  const int j = blockIdx.z * cv + jl;
  const bool is_fresh = a.fresh[e] != 0;
  float* head_state = a.state + size_t(a.state_slot[e]) * a.slot_stride + size_t(h) * a.head_stride;
  // the normaliser and the running maximum are kept NORM_COPIES times: the CTA of slice z reads copy z and renews the
  // copies z, z + slices, z + 2 slices, ..., so that every copy is current whatever the number of slices of a launch
  float* norm_state = head_state + size_t(rows) * cols;

  if (MODE == MODE_SSD && a.conv_in != nullptr && h == 0 && blockIdx.z == 0) {
    // the inputs of the convolution's last taps - 1 positions: this step's newest rows, and before them what the
    // slot held (each channel is one thread's: it reads a place before it writes over it)
    const T* in = static_cast<const T*>(a.conv_in);
    float* cs = a.state + size_t(a.state_slot[e]) * a.slot_stride + a.conv_state_off;
    const int keep = a.conv_taps - 1, n = row1 - row0;
    for (int c = tid; c < a.conv_channels; c += blockDim.x)
      for (int s = 0; s < keep; ++s) {
        const int l = n - keep + s;
        float val = 0.f;
        if (l >= 0) val = to_float(in[size_t(row0 + l) * a.conv_in_stride + c]);
        else if (!is_fresh) val = cs[size_t(s + n) * a.conv_channels + c];
        cs[size_t(s) * a.conv_channels + c] = val;
      }
  }

  float S[RPT], nrm[RPT], m = 0.f;
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int i = g * RPT + r;
    S[r] = (!is_fresh && i < rows && j < cols) ? head_state[size_t(i) * cols + j] : 0.f;
    nrm[r] = (MODE == MODE_MLSTM && !is_fresh && i < rows) ? norm_state[size_t(blockIdx.z) * (rows + 1) + i] : 0.f;
  }
  if (MODE == MODE_MLSTM && !is_fresh) m = norm_state[size_t(blockIdx.z) * (rows + 1) + rows];

  const T* read = static_cast<const T*>(a.read) + size_t(h / a.heads_per_group) * rows;
  const T* write = static_cast<const T*>(a.write) + size_t(h / a.heads_per_group) * rows;
  const T* value = static_cast<const T*>(a.value) + size_t(h) * cols + size_t(blockIdx.z) * cv;
  const float skip = MODE == MODE_SSD ? a.skip[h] : 0.f;

  for (int t0 = row0; t0 < row1; t0 += TILE) {
    const int nt = row1 - t0 < TILE ? row1 - t0 : TILE;
    __syncthreads();  // the last rows' vectors have been used
    // (loads in batches of eight before their stores: a loop of load-then-store would wait for every load in turn)
    for (int base = 0; base < nt * padded; base += 8 * blockDim.x) {
      float tr[8], tw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * blockDim.x + tid;
        const int tt = idx / padded, i = idx - tt * padded;
        const bool live = idx < nt * padded && i < rows;
        const size_t row = size_t(t0 + tt);
        tr[u] = live ? to_float(read[row * a.read_stride + i]) : 0.f;
        tw[u] = live ? to_float(write[row * a.write_stride + i]) : 0.f;
        if (MODE == MODE_DECAY && live && i < 2 * a.rot_half) {
          // the pair (u, v) = (x[i], x[i + half]) becomes (u cos - v sin, v cos + u sin); position and angle are float
          const bool low = i < a.rot_half;
          const int other = low ? i + a.rot_half : i - a.rot_half;
          float sn, cs;
          sincosf(float(a.positions[row]) * a.inv_freq[low ? i : other], &sn, &cs);
          if (low) sn = -sn;
          tr[u] = fmaf(tr[u], cs, to_float(read[row * a.read_stride + other]) * sn);
          tw[u] = fmaf(tw[u], cs, to_float(write[row * a.write_stride + other]) * sn);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * blockDim.x + tid;
        if (idx < nt * padded) {
          rs[idx] = tr[u] * a.read_scale;
          ws[idx] = MODE == MODE_DECAY ? tw[u] * a.write_scale : tw[u];
        }
      }
    }
    for (int base = 0; base < nt * cv; base += 4 * blockDim.x) {
      float tv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * blockDim.x + tid;
        const int tt = idx / cv, c = idx - tt * cv;
        tv[u] = (idx < nt * cv && blockIdx.z * cv + c < cols) ? to_float(value[size_t(t0 + tt) * a.value_stride + c]) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * blockDim.x + tid;
        if (idx < nt * cv) vs[idx] = tv[u];
      }
    }
    if (MODE == MODE_DECAY) {
      if (tid < nt) {
        g0[tid] = 1.f;
        g1[tid] = a.decay[h];
      }
    } else if (tid < nt) {
      const float* gr = a.gates + size_t(t0 + tid) * a.gates_stride;
      if (MODE == MODE_MLSTM) {
        g0[tid] = soft_cap(gr[h], a.cap);
        g1[tid] = log_sigmoid(soft_cap(gr[gridDim.y + h], a.cap));
      } else {
        const float step = softplus(gr[h] + a.step_bias[h]);
        g0[tid] = step;
        g1[tid] = expf(-expf(a.log_rate[h]) * step);
      }
    }
    __syncthreads();
    if (MODE == MODE_MLSTM) {
      // the running maximum is a chain of an addition and a maximum per row: every one of the first nt threads walks
      // it up to its own row (in the rows' order, so the result does not depend on where a tile begins); the
      // exponentials, which are what costs, are then one per thread
      float keep = 0.f, take = 0.f, top = 0.f;
      if (tid < nt) {
        float li[TILE], lf[TILE];   // (all loads first: the chain is then an addition and a maximum a row)
#pragma unroll
        for (int tt = 0; tt < TILE; ++tt) {
          li[tt] = g0[tt];
          lf[tt] = g1[tt];
        }
        float before = m;
        top = m;
#pragma unroll
        for (int tt = 0; tt < TILE; ++tt) {
          if (tt <= tid) {
            before = top;
            top = fmaxf(lf[tt] + before, li[tt]);
          }
        }
        keep = expf(g1[tid] + before - top);
        take = expf(g0[tid] - top);
      }
      __syncthreads();
      if (tid < nt) {
        g0[tid] = take;
        g1[tid] = keep;
        g2[tid] = top;
      }
      __syncthreads();
      m = g2[nt - 1];
    }
    float num[TILE], nq[TILE];
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt) {
      if (tt >= nt) break;   // (a branch that every thread of the CTA takes alike: rows that are not there cost nothing)
      num[tt] = 0.f;
      nq[tt] = 0.f;
      {
        const float take = g0[tt], keep = g1[tt];
        const float tv = take * vs[tt * cv + jl];
        const float4* wr = reinterpret_cast<const float4*>(ws + tt * padded + g * RPT);
        const float4* rr = reinterpret_cast<const float4*>(rs + tt * padded + g * RPT);
        float acc = 0.f, acc_n = 0.f;
#pragma unroll
        for (int r4 = 0; r4 < RPT / 4; ++r4) {
          const float4 w4 = wr[r4], q4 = rr[r4];
          const float w[4] = {w4.x, w4.y, w4.z, w4.w}, q[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int r = r4 * 4 + u;
            S[r] = fmaf(keep, S[r], w[u] * tv);
            acc = fmaf(S[r], q[u], acc);
            if (MODE == MODE_MLSTM) {
              nrm[r] = fmaf(keep, nrm[r], take * w[u]);
              acc_n = fmaf(nrm[r], q[u], acc_n);
            }
          }
        }
        num[tt] = acc;
        nq[tt] = acc_n;
      }
    }
    // the sums over a column's rows, for all rows of the tile at once (the shuffles of different rows overlap)
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt) {
      if (tt >= nt) break;
      {
        for (int o = G >> 1; o > 0; o >>= 1) {
          num[tt] += __shfl_xor_sync(0xffffffffu, num[tt], o);
          if (MODE == MODE_MLSTM) nq[tt] += __shfl_xor_sync(0xffffffffu, nq[tt], o);
        }
      }
    }
    if (g == 0 && j < cols) {
#pragma unroll
      for (int tt = 0; tt < TILE; ++tt) {
        if (tt >= nt) break;
        {
          float y;
          if (MODE == MODE_MLSTM) y = num[tt] / (fmaxf(fabsf(nq[tt]), expf(-g2[tt])) + 1e-6f);
          else y = fmaf(skip, vs[tt * cv + jl], num[tt]);
          a.out[size_t(t0 + tt) * a.out_stride + size_t(h) * cols + j] = y;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int i = g * RPT + r;
    if (i < rows && j < cols) head_state[size_t(i) * cols + j] = S[r];
  }
  if (MODE == MODE_MLSTM && jl == 0) {
    for (int copy = blockIdx.z; copy < NORM_COPIES; copy += gridDim.z) {
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int i = g * RPT + r;
        if (i < rows) norm_state[size_t(copy) * (rows + 1) + i] = nrm[r];
      }
      if (tid == 0) norm_state[size_t(copy) * (rows + 1) + rows] = m;
    }
  }
}

// How a head's state is spread over threads: RPT rows of a column in a thread's registers, a column's rows over G
// neighbouring lanes (a power of two up to 32), cv columns a CTA and the columns over 1, 2, 4 or 8 CTAs: as few as the
// 256 threads of a CTA allow, and more while the launch has fewer CTAs than the GPU has SMs.
struct ScanShape { int rpt, G, threads, cv, splits; };

ScanShape scan_shape(int rows, int cols, int pairs) {
  ScanShape s;
  s.rpt = 4;
  while (s.rpt < 32 && (rows + s.rpt - 1) / s.rpt > 4) s.rpt *= 2;
  s.G = 1;
  while (s.G * s.rpt < rows) s.G *= 2;
  const int G = s.G > 32 ? 32 : s.G, per_warp = 32 / G;
  s.splits = 1;
  for (;;) {
    s.cv = ((cols + s.splits - 1) / s.splits + per_warp - 1) / per_warp * per_warp;
    s.threads = s.cv * G;
    if (s.splits == NORM_COPIES) break;
    const bool fits = s.threads <= 256, enough = pairs * s.splits >= 120 || s.threads <= 64;
    if (fits && enough) break;
    s.splits *= 2;
  }
  return s;
}

template <typename T, int MODE>
int launch_scan(const ScanArgs& in, int n_entries, int n_heads, cudaStream_t stream) {
  ScanArgs a = in;
  const ScanShape s = scan_shape(a.rows, a.cols, n_entries * n_heads);
  const int rpt = s.rpt, G = s.G, threads = s.threads, splits = s.splits;
  if (G > 32 || threads > 256) return R2_UNSUPPORTED;
  a.G = G;
  a.cv = s.cv;
  const bool single_rows = a.single_rows != 0;
  const int tile = single_rows ? SMALL_TILE : (rpt <= 16 ? MAX_TILE : 16);
  const size_t smem = sizeof(float) * (size_t(tile) * (2 * rpt * G + a.cv) + 3 * tile);
  if (smem > 48 * 1024) return R2_UNSUPPORTED;
  dim3 grid(n_entries, n_heads, splits);
#define R2_SCAN(RPT_, TILE_) r2_launch(outer_scan_kernel<T, RPT_, MODE, TILE_>, grid, dim3(threads), smem, stream, a)
  switch (rpt) {
    case 4: if (single_rows) R2_SCAN(4, SMALL_TILE); else R2_SCAN(4, MAX_TILE); break;
    case 8: if (single_rows) R2_SCAN(8, SMALL_TILE); else R2_SCAN(8, MAX_TILE); break;
    case 16: if (single_rows) R2_SCAN(16, SMALL_TILE); else R2_SCAN(16, MAX_TILE); break;
    default: if (single_rows) R2_SCAN(32, SMALL_TILE); else R2_SCAN(32, 16); break;
  }
#undef R2_SCAN
  return launch_status();
}

// ---- the short causal convolution --------------------------------------------------------------
// out[t][c] = silu(bias[c] + sum_d taps[c][d] * in[t - (n_taps - 1) + d][c]); inputs before this step's first row
// of an entry come from the request's slot (the inputs of its last n_taps - 1 positions), zeros before a sequence's
// start. The slot is only read here; the recurrence's kernel, which runs after this one, renews it.
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ in, int in_stride, T* __restrict__ out, int out_stride, const float* __restrict__ taps,
                   const float* __restrict__ bias, int n_taps, int channels, const float* __restrict__ state, long long slot_stride,
                   long long conv_state_off, const int32_t* __restrict__ row_entry, const int32_t* __restrict__ q_start,
                   const int32_t* __restrict__ state_slot, const int32_t* __restrict__ fresh) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int e = row_entry[t];
  T* o = out + size_t(t) * out_stride;
  if (e < 0) {  // a pad row
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) o[c] = from_float<T>(0.f);
    return;
  }
  const int l = t - q_start[e];
  const bool is_fresh = fresh[e] != 0;
  const float* cs = state + size_t(state_slot[e]) * slot_stride + conv_state_off;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float acc = bias != nullptr ? bias[c] : 0.f;
    for (int d = 0; d < n_taps; ++d) {
      const int src = l - (n_taps - 1) + d;
      float val = 0.f;
      if (src >= 0) val = to_float(in[size_t(t - (n_taps - 1) + d) * in_stride + c]);
      else if (!is_fresh) val = cs[size_t(n_taps - 1 + src) * channels + c];
      acc = fmaf(taps[size_t(c) * n_taps + d], val, acc);
    }
    o[c] = from_float<T>(acc / (1.f + expf(-acc)));
  }
}

// ---- norm over groups of columns, with a gate ---------------------------------------------------
// One warp per (row, group). gate_first 1: y <- y * silu(gate), then the group's RMS norm, times weight.
// 0: the group's RMS norm, times weight, times sigmoid(gate). 2: the group's RMS norm, times weight, times silu(gate).
// weight may be null: a gain of one.
template <typename T>
__global__ void __launch_bounds__(128)
group_norm_gated_kernel(const float* __restrict__ y, int y_stride, const T* __restrict__ gate, int gate_stride,
                        const float* __restrict__ weight, T* __restrict__ out, int out_stride, int n_rows, int n_groups,
                        int group_size, float eps, int gate_first) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= (long long)n_rows * n_groups) return;
  const int t = int(unit / n_groups), grp = int(unit % n_groups);
  const float* yr = y + size_t(t) * y_stride + size_t(grp) * group_size;
  const T* gr = gate + size_t(t) * gate_stride + size_t(grp) * group_size;
  const float* wr = weight + size_t(grp) * group_size;
  T* o = out + size_t(t) * out_stride + size_t(grp) * group_size;
  float sq = 0.f;
  for (int d = lane; d < group_size; d += 32) {
    float v = yr[d];
    if (gate_first == 1) {
      const float z = to_float(gr[d]);
      v *= z / (1.f + expf(-z));
    }
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(group_size) + eps);
  for (int d = lane; d < group_size; d += 32) {
    float v = yr[d];
    const float z = to_float(gr[d]);
    const float gain = weight != nullptr ? wr[d] : 1.f;
    if (gate_first == 1) v = v * (z / (1.f + expf(-z))) * inv * gain;
    else v = v * inv * gain * ((gate_first == 2 ? z : 1.f) / (1.f + expf(-z)));
    o[d] = from_float<T>(v);
  }
}

// The same with a CTA per (row, group), for groups of many columns.
template <typename T>
__global__ void __launch_bounds__(256)
group_norm_gated_block_kernel(const float* __restrict__ y, int y_stride, const T* __restrict__ gate, int gate_stride,
                              const float* __restrict__ weight, T* __restrict__ out, int out_stride, int n_groups,
                              int group_size, float eps, int gate_first) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x / n_groups, grp = blockIdx.x % n_groups;
  const float* yr = y + size_t(t) * y_stride + size_t(grp) * group_size;
  const T* gr = gate + size_t(t) * gate_stride + size_t(grp) * group_size;
  const float* wr = weight + size_t(grp) * group_size;
  T* o = out + size_t(t) * out_stride + size_t(grp) * group_size;
  float sq = 0.f;
  for (int d = threadIdx.x; d < group_size; d += blockDim.x) {
    float v = yr[d];
    if (gate_first == 1) {
      const float z = to_float(gr[d]);
      v *= z / (1.f + expf(-z));
    }
    sq = fmaf(v, v, sq);
  }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / float(group_size) + eps);
  for (int d = threadIdx.x; d < group_size; d += blockDim.x) {
    float v = yr[d];
    const float z = to_float(gr[d]);
    const float gain = weight != nullptr ? wr[d] : 1.f;
    if (gate_first == 1) v = v * (z / (1.f + expf(-z))) * inv * gain;
    else v = v * inv * gain * ((gate_first == 2 ? z : 1.f) / (1.f + expf(-z)));
    o[d] = from_float<T>(v);
  }
}

}  // namespace

// Floats of one head's state in a request slot: the matrix, and NORM_COPIES times the normaliser vector with the
// running maximum.
extern "C" long long r2_mlstm_state_floats(int dim, int vdim) {
  if (dim < 1 || vdim < 1) return 0;
  return (long long)dim * vdim + (long long)NORM_COPIES * (dim + 1);
}

// The matrix memory's recurrence over a batch of entries. q, k [T, heads * dim] and v [T, heads * vdim] (slices of a
// projection, each with its row stride); gates [T, 2 * heads] float (input gates, then forget gates, before the
// cap); state [slots][heads][r2_mlstm_state_floats(dim, vdim)] float; out [T, heads * vdim] float, before the heads' norm.
extern "C" int r2_mlstm_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                             const float* gates, int gates_stride, float cap, float q_scale, float* state,
                             long long slot_stride, const int32_t* q_start, const int32_t* state_slot, const int32_t* fresh,
                             int n_entries, float* out, int out_stride, int n_heads, int dim, int vdim, int single_rows,
                             int dtype, cudaStream_t stream) {
  if (n_entries <= 0) return R2_OK;
  if (n_heads < 1 || dim < 1 || vdim < 1) return R2_BAD_SHAPE;
  ScanArgs a = {};
  a.read = q; a.read_stride = q_stride; a.write = k; a.write_stride = k_stride; a.value = v; a.value_stride = v_stride;
  a.gates = gates; a.gates_stride = gates_stride; a.cap = cap; a.read_scale = q_scale;
  a.state = state; a.slot_stride = slot_stride; a.head_stride = int(r2_mlstm_state_floats(dim, vdim));
  a.q_start = q_start; a.state_slot = state_slot; a.fresh = fresh; a.out = out; a.out_stride = out_stride;
  a.heads_per_group = 1; a.rows = dim; a.cols = vdim; a.single_rows = single_rows;
  if (dtype == R2_F32) return launch_scan<float, MODE_MLSTM>(a, n_entries, n_heads, stream);
  if (dtype == R2_BF16) return launch_scan<bf16, MODE_MLSTM>(a, n_entries, n_heads, stream);
  return R2_BAD_DTYPE;
}

// Retention: S <- decay[h] S + k v^T, o = S^T q per head, with q and k rotated by position (the first rot_dims dimensions
// of a head, dimension i with i + rot_dims / 2, angle positions[t] * inv_freq[i]; rot_dims 0: none) and k multiplied by
// k_scale after the rotation. q, k [T, heads * dim], v [T, heads * vdim] (slices of a projection); decay float [heads];
// state float [slots][heads][dim][vdim]; out [T, heads * vdim] float, before the heads' norm.
extern "C" int r2_retention_scan(const void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride,
                                 const float* decay, float k_scale, const float* inv_freq, int rot_dims, const int32_t* positions,
                                 float* state, long long slot_stride, const int32_t* q_start, const int32_t* state_slot,
                                 const int32_t* fresh, int n_entries, float* out, int out_stride, int n_heads, int dim, int vdim,
                                 int single_rows, int dtype, cudaStream_t stream) {
  if (n_entries <= 0) return R2_OK;
  if (n_heads < 1 || dim < 1 || vdim < 1 || rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > dim) return R2_BAD_SHAPE;
  if (rot_dims > 0 && (inv_freq == nullptr || positions == nullptr)) return R2_BAD_SHAPE;
  ScanArgs a = {};
  a.read = q; a.read_stride = q_stride; a.write = k; a.write_stride = k_stride; a.value = v; a.value_stride = v_stride;
  a.read_scale = 1.f; a.write_scale = k_scale; a.decay = decay; a.inv_freq = inv_freq; a.rot_half = rot_dims / 2; a.positions = positions;
  a.state = state; a.slot_stride = slot_stride; a.head_stride = dim * vdim;
  a.q_start = q_start; a.state_slot = state_slot; a.fresh = fresh; a.out = out; a.out_stride = out_stride;
  a.heads_per_group = 1; a.rows = dim; a.cols = vdim; a.single_rows = single_rows;
  if (dtype == R2_F32) return launch_scan<float, MODE_DECAY>(a, n_entries, n_heads, stream);
  if (dtype == R2_BF16) return launch_scan<bf16, MODE_DECAY>(a, n_entries, n_heads, stream);
  return R2_BAD_DTYPE;
}

// The state-space recurrence. x [T, heads * vdim], B and C [T, groups * n_state] (after convolution and silu), steps
// [T, heads] float before bias and softplus; per head step_bias, log_rate, skip. state per slot: S [heads][n_state][vdim]
// and, at conv_state_off, the convolution's last conv_taps - 1 inputs [conv_taps - 1][conv_channels], which this kernel
// renews from conv_in (the convolution's input rows of this step; null: no convolution state).
extern "C" int r2_ssd_scan(const void* x, int x_stride, const void* b, int b_stride, const void* c, int c_stride,
                           const float* steps, int steps_stride, const float* step_bias, const float* log_rate,
                           const float* skip, float* state, long long slot_stride, const int32_t* q_start,
                           const int32_t* state_slot, const int32_t* fresh, int n_entries, float* out, int out_stride,
                           int n_heads, int n_groups, int n_state, int vdim, const void* conv_in, int conv_in_stride,
                           int conv_channels, int conv_taps, long long conv_state_off, int single_rows, int dtype,
                           cudaStream_t stream) {
  if (n_entries <= 0) return R2_OK;
  if (n_heads < 1 || n_groups < 1 || n_heads % n_groups != 0 || n_state < 1 || vdim < 1) return R2_BAD_SHAPE;
  ScanArgs a = {};
  a.read = c; a.read_stride = c_stride; a.write = b; a.write_stride = b_stride; a.value = x; a.value_stride = x_stride;
  a.gates = steps; a.gates_stride = steps_stride; a.step_bias = step_bias; a.log_rate = log_rate; a.skip = skip;
  a.read_scale = 1.f; a.state = state; a.slot_stride = slot_stride; a.head_stride = n_state * vdim;
  a.q_start = q_start; a.state_slot = state_slot; a.fresh = fresh; a.out = out; a.out_stride = out_stride;
  a.heads_per_group = n_heads / n_groups; a.rows = n_state; a.cols = vdim; a.single_rows = single_rows;
  a.conv_in = conv_taps > 1 ? conv_in : nullptr; a.conv_in_stride = conv_in_stride; a.conv_channels = conv_channels;
  a.conv_taps = conv_taps; a.conv_state_off = conv_state_off;
  if (dtype == R2_F32) return launch_scan<float, MODE_SSD>(a, n_entries, n_heads, stream);
  if (dtype == R2_BF16) return launch_scan<bf16, MODE_SSD>(a, n_entries, n_heads, stream);
  return R2_BAD_DTYPE;
}

extern "C" int r2_causal_conv(const void* in, int in_stride, void* out, int out_stride, const float* taps, const float* bias,
                              int n_taps, int channels, const float* state, long long slot_stride, long long conv_state_off,
                              const int32_t* row_entry, const int32_t* q_start, const int32_t* state_slot, const int32_t* fresh,
                              int n_rows, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_taps < 1 || channels < 1) return R2_BAD_SHAPE;
  dim3 grid(n_rows, (channels + 1023) / 1024);
  if (dtype == R2_F32) {
    r2_launch(causal_conv_kernel<float>, grid, dim3(256), size_t(0), stream, (const float*)in, in_stride, (float*)out, out_stride,
              taps, bias, n_taps, channels, state, slot_stride, conv_state_off, row_entry, q_start, state_slot, fresh);
  } else if (dtype == R2_BF16) {
    r2_launch(causal_conv_kernel<bf16>, grid, dim3(256), size_t(0), stream, (const bf16*)in, in_stride, (bf16*)out, out_stride,
              taps, bias, n_taps, channels, state, slot_stride, conv_state_off, row_entry, q_start, state_slot, fresh);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

extern "C" int r2_group_norm_gated(const float* y, int y_stride, const void* gate, int gate_stride, const float* weight,
                                   void* out, int out_stride, int n_rows, int n_groups, int group_size, float eps,
                                   int gate_first, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_groups < 1 || group_size < 1) return R2_BAD_SHAPE;
  const long long units = (long long)n_rows * n_groups;
  if (group_size > 256) {
    if (dtype == R2_F32) {
      r2_launch(group_norm_gated_block_kernel<float>, dim3((unsigned)units), dim3(256), size_t(0), stream, y, y_stride, (const float*)gate,
                gate_stride, weight, (float*)out, out_stride, n_groups, group_size, eps, gate_first);
    } else if (dtype == R2_BF16) {
      r2_launch(group_norm_gated_block_kernel<bf16>, dim3((unsigned)units), dim3(256), size_t(0), stream, y, y_stride, (const bf16*)gate,
                gate_stride, weight, (bf16*)out, out_stride, n_groups, group_size, eps, gate_first);
    } else {
      return R2_BAD_DTYPE;
    }
    return launch_status();
  }
  dim3 grid((unsigned)((units + 3) / 4));
  if (dtype == R2_F32) {
    r2_launch(group_norm_gated_kernel<float>, grid, dim3(128), size_t(0), stream, y, y_stride, (const float*)gate, gate_stride,
              weight, (float*)out, out_stride, n_rows, n_groups, group_size, eps, gate_first);
  } else if (dtype == R2_BF16) {
    r2_launch(group_norm_gated_kernel<bf16>, grid, dim3(128), size_t(0), stream, y, y_stride, (const bf16*)gate, gate_stride,
              weight, (bf16*)out, out_stride, n_rows, n_groups, group_size, eps, gate_first);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
