// Several residual streams with learned mixing ("hyper-connections").  Instead of one residual
// stream x there are S copies x_0 .. x_{S-1}, stored [S][rows][width] in 32-bit.  A sublayer
//   reads   u   = sum_s a[s] x_s                       (then a norm: h = u / rms(u) * w)
//   writes  x_t <- sum_s M[s][t] x_s + b[t] y          for all t at once, from the old streams.
// One kernel does the write of one sublayer and the read of the next for a row: the new streams
// never travel twice.  Either half can be left out (the first read of a step has no write in front
// of it; the last write may be followed by the final norm at a few chosen rows only).  All of
// it is 32-bit; only the normed output is rounded to the activation type.
#include "common.cuh"

namespace {
constexpr int MAX_STREAMS = 8;
constexpr int KEEP = 16;     // values a thread keeps between the sum of squares and the scaling

struct StreamArgs {
  float* xs; long long stream_stride;     // xs[s * stream_stride + row * width + c]
  float* y;                               // the sublayer's output [rows][width], or null: no write
  const float* mix;                       // M[s * S + t]
  const float* b;                         // b[t]
  const float* a;                         // a[s], or null: no read
  const float* w;                         // the norm's gain [width]
  const int* rows_index;                  // the rows this launch works on, or null: row = block
  int S, width, clear_y, store;           // store: write the new streams back
  float eps;
};

template <typename TOut, int S>
__global__ void __launch_bounds__(256) stream_step_kernel(const StreamArgs p, TOut* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float coef[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
  pdl_trigger();
  // the coefficients are weights: nothing of this step wrote them
  if (threadIdx.x < S * S) coef[threadIdx.x] = p.y ? p.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    coef[S * S + threadIdx.x] = p.y ? p.b[threadIdx.x] : 0.f;
    coef[S * S + S + threadIdx.x] = p.a ? p.a[threadIdx.x] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const size_t row = p.rows_index ? (size_t)p.rows_index[r] : (size_t)r;
  float* x0 = p.xs + row * p.width;
  float* yr = p.y ? p.y + row * p.width : nullptr;
  float u_keep[KEEP];
  float ss = 0.f;
  auto column = [&](int c) {
    float v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) v[s] = x0[(size_t)s * p.stream_stride + c];
    if (yr) {
      const float yv = yr[c];
      if (p.clear_y) yr[c] = 0.f;
      float n[S];
#pragma unroll
      for (int t = 0; t < S; ++t) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) acc = fmaf(coef[s * S + t], v[s], acc);
        n[t] = fmaf(coef[S * S + t], yv, acc);
      }
#pragma unroll
      for (int t = 0; t < S; ++t) {
        v[t] = n[t];
        if (p.store) x0[(size_t)t * p.stream_stride + c] = n[t];
      }
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) u = fmaf(coef[S * S + S + s], v[s], u);
    return u;
  };
  // (a column is visited once: the streams are written on that visit, so the second pass over
  // columns beyond what a thread keeps reads the new streams and must not apply the write again)
  int n = 0;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x, ++n) {
    const float u = column(c);
    if (n < KEEP) u_keep[n] = u;
    ss = fmaf(u, u, ss);
  }
  if (!p.a) return;
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)p.width + p.eps);
  n = 0;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x, ++n) {
    float u;
    if (n < KEEP) {
      u = u_keep[n];
    } else {             // read again what this thread wrote (or what nobody changed)
      u = 0.f;     // (a launch that does not store keeps its width within KEEP * threads)
#pragma unroll
      for (int s = 0; s < S; ++s) u = fmaf(coef[S * S + S + s], x0[(size_t)s * p.stream_stride + c], u);
    }
    out[(size_t)r * p.width + c] = from_f32<TOut>(u * scale * p.w[c]);
  }
}

// The same with 16-byte accesses (the width a multiple of four, every base aligned): a thread
// owns four neighbouring columns at a time, so that a row of a few thousand columns is one access
// per thread and stream; a step of few rows is then one round trip to memory, not sixteen.
constexpr int KEEP4 = 4;
template <typename TOut, int S>
__global__ void __launch_bounds__(1024) stream_step_vec_kernel(const StreamArgs p, TOut* __restrict__ out) {
  __shared__ float scratch[33];
  __shared__ float coef[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
  pdl_trigger();
  if (threadIdx.x < S * S) coef[threadIdx.x] = p.y ? p.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    coef[S * S + threadIdx.x] = p.y ? p.b[threadIdx.x] : 0.f;
    coef[S * S + S + threadIdx.x] = p.a ? p.a[threadIdx.x] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x, n4 = p.width >> 2;
  const size_t row = p.rows_index ? (size_t)p.rows_index[r] : (size_t)r;
  float* x0 = p.xs + row * p.width;
  float* yr = p.y ? p.y + row * p.width : nullptr;
  float4 u_keep[KEEP4];
  float ss = 0.f;
  auto column = [&](int c) {            // c: first of four columns
    float v[S][4];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const float4 t = *reinterpret_cast<const float4*>(x0 + (size_t)s * p.stream_stride + c);
      v[s][0] = t.x, v[s][1] = t.y, v[s][2] = t.z, v[s][3] = t.w;
    }
    if (yr) {
      const float4 yv4 = *reinterpret_cast<const float4*>(yr + c);
      const float yv[4] = {yv4.x, yv4.y, yv4.z, yv4.w};
      if (p.clear_y) *reinterpret_cast<float4*>(yr + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      float n[S][4];
#pragma unroll
      for (int t = 0; t < S; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s) acc = fmaf(coef[s * S + t], v[s][e], acc);
          n[t][e] = fmaf(coef[S * S + t], yv[e], acc);
        }
#pragma unroll
      for (int t = 0; t < S; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[t][e] = n[t][e];
        if (p.store)
          *reinterpret_cast<float4*>(x0 + (size_t)t * p.stream_stride + c) = make_float4(n[t][0], n[t][1], n[t][2], n[t][3]);
      }
    }
    float u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
      for (int e = 0; e < 4; ++e) u[e] = fmaf(coef[S * S + S + s], v[s][e], u[e]);
    return make_float4(u[0], u[1], u[2], u[3]);
  };
  auto square = [&](const float4& u) {
    ss = fmaf(u.x, u.x, ss), ss = fmaf(u.y, u.y, ss), ss = fmaf(u.z, u.z, ss), ss = fmaf(u.w, u.w, ss);
  };
#pragma unroll
  for (int n = 0; n < KEEP4; ++n) {
    const int c4 = threadIdx.x + n * blockDim.x;
    if (c4 < n4) {
      u_keep[n] = column(4 * c4);
      square(u_keep[n]);
    }
  }
  for (int c4 = threadIdx.x + KEEP4 * blockDim.x; c4 < n4; c4 += blockDim.x) square(column(4 * c4));
  if (!p.a) return;
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)p.width + p.eps);
  auto write = [&](int c, const float4& u) {
    const float4 w = *reinterpret_cast<const float4*>(p.w + c);
    TOut* dst = out + (size_t)r * p.width + c;
    dst[0] = from_f32<TOut>(u.x * scale * w.x), dst[1] = from_f32<TOut>(u.y * scale * w.y);
    dst[2] = from_f32<TOut>(u.z * scale * w.z), dst[3] = from_f32<TOut>(u.w * scale * w.w);
  };
#pragma unroll
  for (int n = 0; n < KEEP4; ++n) {
    const int c4 = threadIdx.x + n * blockDim.x;
    if (c4 < n4) write(4 * c4, u_keep[n]);
  }
  // beyond what is kept: read again what this thread wrote (a launch that does not store stays
  // within what is kept)
  for (int c4 = threadIdx.x + KEEP4 * blockDim.x; c4 < n4; c4 += blockDim.x) {
    const int c = 4 * c4;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const float4 t = *reinterpret_cast<const float4*>(x0 + (size_t)s * p.stream_stride + c);
      const float cs = coef[S * S + S + s];
      a[0] = fmaf(cs, t.x, a[0]), a[1] = fmaf(cs, t.y, a[1]), a[2] = fmaf(cs, t.z, a[2]), a[3] = fmaf(cs, t.w, a[3]);
    }
    write(c, make_float4(a[0], a[1], a[2], a[3]));
  }
}

// xs[s][r][:] = xs[0][r][:] for s >= 1: every stream starts as the embedding output
__global__ void stream_fill_kernel(float* __restrict__ xs, long long stream_stride, long long total, int S) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = xs[i];
    for (int s = 1; s < S; ++s) xs[(size_t)s * stream_stride + i] = v;
  }
}

template <typename TOut>
int launch_step(const StreamArgs& p, void* out, int rows, cudaStream_t stream) {
  const bool vec = (p.width & 3) == 0 && (p.stream_stride & 3) == 0 &&
                   (((uintptr_t)p.xs | (uintptr_t)p.y | (uintptr_t)p.w) & 15) == 0;
  if (vec) {
    int threads = ((p.width >> 2) + 31) & ~31;
    threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
    if (p.y == nullptr || p.store || p.width <= 4 * KEEP4 * threads) {
#define STEPV(N) \
  case N: return launched_many_blocks(launch_pdl(stream_step_vec_kernel<TOut, N>, rows, threads, 0, stream, p, (TOut*)out), rows)
      switch (p.S) {
        STEPV(1); STEPV(2); STEPV(3); STEPV(4); STEPV(5); STEPV(6); STEPV(7); STEPV(8);
      }
#undef STEPV
    }
  }
  const int threads = p.width >= 1024 ? 256 : 128;
#define STEP(N) \
  case N: return launched_many_blocks(launch_pdl(stream_step_kernel<TOut, N>, rows, threads, 0, stream, p, (TOut*)out), rows)
  switch (p.S) {
    STEP(1); STEP(2); STEP(3); STEP(4); STEP(5); STEP(6); STEP(7); STEP(8);
  }
#undef STEP
  return LLM_ERR_UNSUPPORTED;
}
}  // namespace

// One sublayer boundary of a model with S residual streams, for `rows` rows (all rows of the
// step in order, or those that rows_index names).  y/mix/b null: no write.  a null: no read (w
// and out are unused).  store: the new streams go back to memory (0 only when nothing reads them
// afterwards, as behind the last layer; such a launch takes a width of at most 4,096).
LLM_EXPORT int llm_stream_step(float* xs, long long stream_stride, int S, float* y, const float* mix,
                               const float* b, int clear_y, int store, const float* a, const float* w,
                               float eps, void* out, int out_dtype, const int* rows_index, int rows,
                               int width, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  if (S < 1 || S > MAX_STREAMS) return LLM_ERR_UNSUPPORTED;
  if ((y != nullptr) != (mix != nullptr) || (y != nullptr) != (b != nullptr)) return LLM_ERR_ARGUMENT;
  if (a != nullptr && (w == nullptr || out == nullptr)) return LLM_ERR_ARGUMENT;
  if (y == nullptr && a == nullptr) return 0;
  if (y != nullptr && !store && width > KEEP * (width >= 1024 ? 256 : 128)) return LLM_ERR_UNSUPPORTED;
  StreamArgs p;
  p.xs = xs, p.stream_stride = stream_stride, p.y = y, p.mix = mix, p.b = b, p.a = a, p.w = w;
  p.rows_index = rows_index, p.S = S, p.width = width, p.clear_y = clear_y, p.store = store, p.eps = eps;
  if (out_dtype == LLM_F32 || a == nullptr) return launch_step<float>(p, out, rows, stream);
  if (out_dtype == LLM_BF16) return launch_step<bf16>(p, out, rows, stream);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_stream_fill(float* xs, long long stream_stride, int S, int rows, int width,
                               cudaStream_t stream) {
  const long long total = (long long)rows * width;
  if (total <= 0 || S <= 1) return 0;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  return launch_pdl(stream_fill_kernel, blocks, 256, 0, stream, xs, stream_stride, total, S);
}
