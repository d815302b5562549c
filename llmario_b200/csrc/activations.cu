// Small passes behind a product that the standard feed-forward and head do not have: a gated
// activation with a choice of function and an optional bias on both halves, and a scaled soft cap.
#include "common.cuh"

namespace {
enum ActKind : int { ACT_SILU = 0, ACT_GELU_TANH = 1 };

__device__ __forceinline__ float act_f(float z, int kind) {
  if (kind == ACT_GELU_TANH)     // 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

// out[t][j] = act(gu[t][j] + b[j]) * (gu[t][ff + j] + b[ff + j]), in 32-bit, rounded once.
// clear: what was read of gu is zeroed (it lies in a buffer that a split-K product adds into).
template <typename TOut>
__global__ void gated_act_kernel(float* __restrict__ gate_up, const float* __restrict__ bias,
                                 TOut* __restrict__ out, long long total, int ff, int kind, int clear) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const long long t = idx / ff;
    const int j = (int)(idx - t * ff);
    float g = gate_up[t * 2 * ff + j], u = gate_up[t * 2 * ff + ff + j];
    if (clear) gate_up[t * 2 * ff + j] = 0.f, gate_up[t * 2 * ff + ff + j] = 0.f;
    if (bias) g += bias[j], u += bias[ff + j];
    out[idx] = from_f32<TOut>(act_f(g, kind) * u);
  }
}

// z <- cap * tanh(z * scale / cap)   (cap <= 0: z <- z * scale)
__global__ void scale_soft_cap_kernel(float* __restrict__ z, long long total, float scale, float cap) {
  pdl_trigger();
  pdl_wait();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const float v = z[idx] * scale;
    z[idx] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}
}  // namespace

LLM_EXPORT int llm_gated_act(float* gate_up, const float* bias, void* out, int out_dtype, int rows,
                             int ff, int kind, int clear, cudaStream_t stream) {
  const long long total = (long long)rows * ff;
  if (total <= 0) return 0;
  if (kind != ACT_SILU && kind != ACT_GELU_TANH) return LLM_ERR_ARGUMENT;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  if (out_dtype == LLM_F32)
    return launched_many_blocks(
        launch_pdl(gated_act_kernel<float>, blocks, 256, 0, stream, gate_up, bias, (float*)out, total, ff, kind, clear), blocks);
  if (out_dtype == LLM_BF16)
    return launched_many_blocks(
        launch_pdl(gated_act_kernel<bf16>, blocks, 256, 0, stream, gate_up, bias, (bf16*)out, total, ff, kind, clear), blocks);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_scale_soft_cap(float* z, long long total, float scale, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  return launch_pdl(scale_soft_cap_kernel, blocks, 256, 0, stream, z, total, scale, cap);
}
