// Recurrent mixers: a linear recurrence with a diagonal decay over a matrix state per head,
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T        (S is K x V; a_t a vector over K, or one number)
//   o_t = S_t^T q_t,
// the short causal convolution that some of them put in front of it, and the gated group norm
// that follows it.  Gated linear attention (a decay per key channel) and state-space mixers of
// the Mamba-2 kind (a scalar decay per head, keys and queries shared by the heads of a group,
// values scaled by the step size) are both this recurrence; which one runs is data.
//
// Everything here is 32-bit: the inputs are the 32-bit results of the projections, the state
// lives in 32-bit floats in the request's state slot, decays and step sizes are made here from
// the projected values.  The tokens of a request are visited one after the other and every sum
// has a fixed order, so the result for a token is the same bits however the prompt was cut into
// steps and whatever else is in the batch.
//
// Which rows of a step belong to which request is read on the device: either every row is a
// request of its own (`single`: slot = row_slot[row]), or a table of (first row, end row) per
// request slot made by llm_segment_table from row_slot.  No host data is involved, so steps of
// single tokens can be recorded and replayed.
#include "common.cuh"

namespace {

// seg[s] = (first row, row after the last) of the rows whose request slot is s; (0, 0): none.
// The rows of a request are consecutive in a step.
__global__ void segment_table_kernel(const int* __restrict__ row_slot, int rows, int2* __restrict__ seg,
                                     int n_slots) {
  pdl_trigger();
  pdl_wait();
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) seg[s] = make_int2(0, 0);
  __syncthreads();
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const int s = row_slot[r];
    if (s < 0 || s >= n_slots) continue;
    if (r == 0 || row_slot[r - 1] != s) seg[s].x = r;
    if (r == rows - 1 || row_slot[r + 1] != s) seg[s].y = r + 1;
  }
}

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

enum DecayKind : int {
  DECAY_VECTOR = 0,        // a = d                       d per (row, head, key channel)
  DECAY_SIGMOID_POW = 1,   // a = sigmoid(d)^c            d per (row, head, key channel), c a constant
  DECAY_RATE_STEP = 2,     // step = softplus(d + p1[h]); a = exp(-exp(p0[h]) * step); v is scaled by step
                           //                             d per (row, head)
};

struct ScanArgs {
  const float* q; int q_stride;          // q[row * q_stride + g * K + i], g = h / (H / G)
  const float* k; int k_stride;          // k[row * k_stride + g * K + i]
  const float* v; int v_stride;          // v[row * v_stride + h * V + j]
  const float* d; int d_stride;          // the decay's argument (see DecayKind)
  const float* p0; const float* p1;      // per-head constants of DECAY_RATE_STEP
  float c;                               // the exponent of DECAY_SIGMOID_POW
  float q_scale;                         // q is multiplied by it
  float* state; long long state_stride;  // state[slot * state_stride + ((h * V) + j) * K + i]
  float* out; int out_stride;            // out[row * out_stride + h * V + j]
  const int2* seg; const int* row_slot;
  int single, H, G, K, V, kind;
};

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_COLS = 16;      // value channels of a block: four to a warp, eight lanes to a channel

// A block owns 16 value channels of one head of one request and walks the request's tokens of
// the step in order.  Lane (c, i) of a warp holds, of column c, the state rows 4 (i + 8 n) + e
// (n < KR4, e < 4) in registers; the token's q, k and decay are staged in shared memory for a
// chunk of tokens at a time and read as 16-byte values that the four columns of a warp share.
template <int KR4, bool VEC>
__global__ void __launch_bounds__(SCAN_THREADS) linear_recurrence_kernel(const ScanArgs a) {
  constexpr int KP = 32 * KR4;                 // key channels, padded
  constexpr int TC = KR4 >= 8 ? 8 : 16;        // tokens of a chunk
  __shared__ float4 q_s[TC][KP / 4];
  __shared__ float4 k_s[TC][KP / 4];
  __shared__ float4 a_s[VEC ? TC : 1][KP / 4];
  __shared__ float v_s[TC][SCAN_COLS];
  __shared__ float a1_s[TC];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int slot, first, end;
  if (a.single) {
    first = blockIdx.x, end = first + 1, slot = a.row_slot[first];
  } else {
    slot = blockIdx.x;
    const int2 s = a.seg[slot];
    first = s.x, end = s.y;
  }
  if (end <= first) return;
  const int K = a.K, V = a.V, g = h / (a.H / a.G);
  const int j0 = blockIdx.z * SCAN_COLS;
  const int col = warp * 4 + (lane >> 3), j = j0 + col, ki = lane & 7;
  const bool live = j < V;
  float* srow = a.state + (size_t)slot * a.state_stride + ((size_t)h * V + (live ? j : 0)) * K;
  const bool k4 = (K & 3) == 0 && ((uintptr_t)srow & 15) == 0;

  float s[KR4][4];
#pragma unroll
  for (int n = 0; n < KR4; ++n) {
    const int i0 = 4 * (ki + 8 * n);
    if (live && k4 && i0 + 3 < K) {
      const float4 t = *reinterpret_cast<const float4*>(srow + i0);
      s[n][0] = t.x, s[n][1] = t.y, s[n][2] = t.z, s[n][3] = t.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = (live && i0 + e < K) ? srow[i0 + e] : 0.f;
    }
  }

  const float rate = a.kind == DECAY_RATE_STEP ? expf(a.p0[h]) : 0.f;
  const float bias = a.kind == DECAY_RATE_STEP ? a.p1[h] : 0.f;
  for (int t0 = first; t0 < end; t0 += TC) {
    const int n_tok = min(TC, end - t0);
    __syncthreads();
    // ---- stage the chunk: q (scaled), k, the decay, and this block's columns of v
    for (int idx = tid; idx < n_tok * KP; idx += SCAN_THREADS) {
      const int tt = idx / KP, i = idx - tt * KP;
      const size_t row = (size_t)(t0 + tt);
      const bool in = i < K;
      reinterpret_cast<float*>(&q_s[tt][0])[i] = in ? a.q[row * a.q_stride + g * K + i] * a.q_scale : 0.f;
      reinterpret_cast<float*>(&k_s[tt][0])[i] = in ? a.k[row * a.k_stride + g * K + i] : 0.f;
      if (VEC) {
        float dec = 1.f;
        if (in) {
          const float d = a.d[row * a.d_stride + h * K + i];
          // sigmoid(d)^c = exp(c * log sigmoid(d)), log sigmoid(d) = -softplus(-d)
          dec = a.kind == DECAY_SIGMOID_POW ? expf(-a.c * softplus_f(-d)) : d;
        }
        reinterpret_cast<float*>(&a_s[tt][0])[i] = dec;
      }
    }
    for (int idx = tid; idx < n_tok * SCAN_COLS; idx += SCAN_THREADS) {
      const int tt = idx / SCAN_COLS, cc = idx - tt * SCAN_COLS;
      const size_t row = (size_t)(t0 + tt);
      float val = j0 + cc < V ? a.v[row * a.v_stride + h * V + j0 + cc] : 0.f;
      if (!VEC) {
        const float step = softplus_f(a.d[row * a.d_stride + h] + bias);
        val *= step;
        if (cc == 0) a1_s[tt] = expf(-rate * step);
      }
      v_s[tt][cc] = val;
    }
    __syncthreads();
    // ---- the tokens of the chunk, one after the other
    for (int tt = 0; tt < n_tok; ++tt) {
      const float vv = v_s[tt][col];
      const float a1 = VEC ? 1.f : a1_s[tt];
      float acc = 0.f;
#pragma unroll
      for (int n = 0; n < KR4; ++n) {
        const float4 qq = q_s[tt][ki + 8 * n], kk = k_s[tt][ki + 8 * n];
        float4 aa = make_float4(a1, a1, a1, a1);
        if (VEC) aa = a_s[tt][ki + 8 * n];
        s[n][0] = fmaf(aa.x, s[n][0], kk.x * vv);
        s[n][1] = fmaf(aa.y, s[n][1], kk.y * vv);
        s[n][2] = fmaf(aa.z, s[n][2], kk.z * vv);
        s[n][3] = fmaf(aa.w, s[n][3], kk.w * vv);
        acc = fmaf(s[n][0], qq.x, acc);
        acc = fmaf(s[n][1], qq.y, acc);
        acc = fmaf(s[n][2], qq.z, acc);
        acc = fmaf(s[n][3], qq.w, acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (ki == 0 && live) a.out[(size_t)(t0 + tt) * a.out_stride + h * V + j] = acc;
    }
  }
  if (!live) return;
#pragma unroll
  for (int n = 0; n < KR4; ++n) {
    const int i0 = 4 * (ki + 8 * n);
    if (k4 && i0 + 3 < K) {
      *reinterpret_cast<float4*>(srow + i0) = make_float4(s[n][0], s[n][1], s[n][2], s[n][3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i0 + e < K) srow[i0 + e] = s[n][e];
    }
  }
}

template <int KR4>
int launch_scan(const ScanArgs& a, dim3 grid, cudaStream_t stream) {
  if (a.kind == DECAY_RATE_STEP)
    return launch_pdl(linear_recurrence_kernel<KR4, false>, grid, SCAN_THREADS, 0, stream, a);
  return launch_pdl(linear_recurrence_kernel<KR4, true>, grid, SCAN_THREADS, 0, stream, a);
}

// ---- short causal convolution per channel, bias, silu
// out[r][c] = silu(b[c] + sum_{j < taps} w[c][taps - 1 - j] * in(r, j, c)); in(r, j, c) is the input
// of channel c, j tokens before row r: a row of this step when the request has that many rows in
// it before r, else one of the request's last taps - 1 inputs of earlier steps (hist, oldest
// first; zeros at the start of a sequence).
__global__ void causal_conv_silu_kernel(const float* __restrict__ src, int src_stride,
                                        const float* __restrict__ w, const float* __restrict__ b,
                                        const float* __restrict__ hist, long long hist_stride,
                                        const int* __restrict__ row_slot, const int2* __restrict__ seg,
                                        int single, float* __restrict__ out, int out_stride, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x, r = blockIdx.x;
  if (c >= C) return;
  const int slot = row_slot[r];
  const int before = single ? 0 : r - seg[slot].x;       // rows of the request in this step before r
  const float* hrow = hist + (size_t)slot * hist_stride + (size_t)c * (taps - 1);
  float acc = b ? b[c] : 0.f;
  for (int j = taps - 1; j >= 0; --j) {       // oldest input first
    const float x = j <= before ? src[(size_t)(r - j) * src_stride + c] : hrow[taps - 1 - (j - before)];
    acc = fmaf(w[(size_t)c * taps + taps - 1 - j], x, acc);
  }
  out[(size_t)r * out_stride + c] = silu_f(acc);
}

// hist[slot][c][:] = the last taps - 1 inputs of the request after this step.  A thread owns one
// (request, channel): it reads the old values it still needs before it overwrites them.
__global__ void conv_history_kernel(const float* __restrict__ src, int src_stride, float* __restrict__ hist,
                                    long long hist_stride, const int* __restrict__ row_slot,
                                    const int2* __restrict__ seg, int single, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  int slot, first, end;
  if (single) {
    first = blockIdx.x, end = first + 1, slot = row_slot[first];
  } else {
    slot = blockIdx.x;
    const int2 s = seg[slot];
    first = s.x, end = s.y;
  }
  const int n = end - first;
  if (n <= 0) return;
  float* hrow = hist + (size_t)slot * hist_stride + (size_t)c * (taps - 1);
  for (int i = 0; i < taps - 1; ++i) {      // ascending: hrow[n + i] is read before it is written
    const int at = n + i;                   // index in (old history, then the step's inputs)
    hrow[i] = at < taps - 1 ? hrow[at] : src[(size_t)(first + at - (taps - 1)) * src_stride + c];
  }
}

// ---- gate and group norm behind the recurrence, one warp per (row, group of `group` channels)
//   y = o (+ skip[ch / head] * x)                        the recurrence's output, plus a direct path
//   gate_first:  out = unit(y * silu(g)) * w             (the gate comes before the norm)
//   otherwise:   out = unit(y) * w * silu(g)
// unit(.) divides a group by its root mean square (eps inside the root); w is indexed by the
// channel modulo w_period (a weight per channel, or one per position in a head shared by heads).
template <typename TOut>
__global__ void gated_group_norm_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ x,
                                        int x_stride, const float* __restrict__ skip, int head,
                                        const float* __restrict__ g, int g_stride, const float* __restrict__ w,
                                        int w_period, TOut* __restrict__ out, int out_stride, int rows,
                                        int groups, int group, float eps, int gate_first) {
  pdl_trigger();
  pdl_wait();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * groups) return;
  const int r = (int)(item / groups), gi = (int)(item % groups), lane = threadIdx.x & 31;
  const int c0 = gi * group;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) {
    const int ch = c0 + i;
    float y = o[(size_t)r * o_stride + ch];
    if (skip) y = fmaf(skip[ch / head], x[(size_t)r * x_stride + ch], y);
    if (gate_first) y *= silu_f(g[(size_t)r * g_stride + ch]);
    ss = fmaf(y, y, ss);
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)group + eps);
  for (int i = lane; i < group; i += 32) {
    const int ch = c0 + i;
    float y = o[(size_t)r * o_stride + ch];
    if (skip) y = fmaf(skip[ch / head], x[(size_t)r * x_stride + ch], y);
    const float gate = silu_f(g[(size_t)r * g_stride + ch]);
    if (gate_first) y *= gate;
    y = y * scale * w[ch % w_period];
    if (!gate_first) y *= gate;
    out[(size_t)r * out_stride + ch] = from_f32<TOut>(y);
  }
}
}  // namespace

LLM_EXPORT int llm_segment_table(const int* row_slot, int rows, int* seg, int n_slots, cudaStream_t stream) {
  if (n_slots <= 0) return 0;
  return launch_pdl(segment_table_kernel, 1, 256, 0, stream, row_slot, rows, (int2*)seg, n_slots);
}

// The recurrence over the rows of a step (see the top of this file).  `single`: every row is a
// request of its own; else `seg` is the table of llm_segment_table over `n_slots` request slots.
// The state of a (slot, head) is V x K floats, the key channel fastest.
LLM_EXPORT int llm_linear_recurrence(const float* q, int q_stride, const float* k, int k_stride, const float* v,
                                     int v_stride, const float* d, int d_stride, const float* p0,
                                     const float* p1, float c, float q_scale, float* state,
                                     long long state_stride, float* out, int out_stride, const int* seg,
                                     const int* row_slot, int rows, int n_slots, int single, int H, int G, int K,
                                     int V, int kind, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || K <= 0 || V <= 0 || kind < 0 || kind > 2) return LLM_ERR_ARGUMENT;
  if (kind == DECAY_RATE_STEP && (!p0 || !p1)) return LLM_ERR_ARGUMENT;
  if (!single && !seg) return LLM_ERR_ARGUMENT;
  if (K > 256) return LLM_ERR_UNSUPPORTED;
  ScanArgs a;
  a.q = q, a.q_stride = q_stride, a.k = k, a.k_stride = k_stride, a.v = v, a.v_stride = v_stride;
  a.d = d, a.d_stride = d_stride, a.p0 = p0, a.p1 = p1, a.c = c, a.q_scale = q_scale;
  a.state = state, a.state_stride = state_stride, a.out = out, a.out_stride = out_stride;
  a.seg = (const int2*)seg, a.row_slot = row_slot;
  a.single = single, a.H = H, a.G = G, a.K = K, a.V = V, a.kind = kind;
  const dim3 grid(single ? rows : n_slots, H, (V + SCAN_COLS - 1) / SCAN_COLS);
  if (K <= 32) return launch_scan<1>(a, grid, stream);
  if (K <= 64) return launch_scan<2>(a, grid, stream);
  if (K <= 128) return launch_scan<4>(a, grid, stream);
  return launch_scan<8>(a, grid, stream);
}

// The convolution of `C` channels over the rows of a step, then the request's history of inputs
// brought up to date (two launches: the second overwrites what the first reads).
LLM_EXPORT int llm_causal_conv_silu(const float* src, int src_stride, const float* w, const float* b,
                                    float* hist, long long hist_stride, const int* row_slot, const int* seg,
                                    int rows, int n_slots, int single, float* out, int out_stride, int C,
                                    int taps, cudaStream_t stream) {
  if (rows <= 0 || C <= 0) return 0;
  if (taps < 1 || (!single && !seg)) return LLM_ERR_ARGUMENT;
  int rc = launch_pdl(causal_conv_silu_kernel, dim3(rows, (C + 127) / 128), 128, 0, stream, src, src_stride, w, b,
                      (const float*)hist, hist_stride, row_slot, (const int2*)seg, single, out, out_stride, C, taps);
  if (rc != 0 || taps == 1) return rc;
  return launch_pdl(conv_history_kernel, dim3(single ? rows : n_slots, (C + 127) / 128), 128, 0, stream, src,
                    src_stride, hist, hist_stride, row_slot, (const int2*)seg, single, C, taps);
}

LLM_EXPORT int llm_gated_group_norm(const float* o, int o_stride, const float* x, int x_stride,
                                    const float* skip, int head, const float* g, int g_stride, const float* w,
                                    int w_period, void* out, int out_dtype, int out_stride, int rows,
                                    int groups, int group, float eps, int gate_first, cudaStream_t stream) {
  if (rows <= 0 || groups <= 0) return 0;
  if (group <= 0 || w_period <= 0 || (skip && (!x || head <= 0))) return LLM_ERR_ARGUMENT;
  const long long items = (long long)rows * groups;
  const int blocks = (int)((items + 3) / 4);
  if (out_dtype == LLM_F32)
    return launch_pdl(gated_group_norm_kernel<float>, blocks, 128, 0, stream, o, o_stride, x, x_stride, skip, head,
                      g, g_stride, w, w_period, (float*)out, out_stride, rows, groups, group, eps, gate_first);
  if (out_dtype == LLM_BF16)
    return launch_pdl(gated_group_norm_kernel<bf16>, blocks, 128, 0, stream, o, o_stride, x, x_stride, skip, head,
                      g, g_stride, w, w_period, (bf16*)out, out_stride, rows, groups, group, eps, gate_first);
  return LLM_ERR_UNSUPPORTED;
}
