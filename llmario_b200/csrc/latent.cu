// Attention through low-rank latents.  A token's keys and values of all heads are functions of
// one latent vector c (kv_rank numbers) and one rotated key part shared by the heads (rot_dim
// numbers); the cache holds just these, as one key row [c | rotated part] of kv_rank + rot_dim
// channels.  The heads' key and value maps are folded to the query's and the output's side:
//   score_h = (U_k,h^T q_h) . c + q_rot,h . k_rot          out_h = U_v,h (sum_j p_j c_j)
// so attention runs as one shared key head whose values are the first kv_rank channels of its keys.
// This file holds what goes before that attention: the norms of the two latents, the rotation
// of adjacent pairs (2i, 2i + 1) and the write into the paged cache.  Everything is computed in 32-bit from the
// 32-bit results of the projections and rounded once.
#include "common.cuh"

namespace {
// One block per row.  proj[row] = [ query latent (q_rank) | key-value latent (kv_rank) | key part
// to rotate (rot_dim) ].  The query latent is normed (gain wq) into cq_out; the key-value latent
// is normed (gain wc) into the row's place in the K plane and, the same values, the V plane;
// the key part is rotated by the row's angles (cos_sin[row][i] = (cos, sin) of angle i, the first
// rot_half pairs; null: no rotation) and written behind the latent in the K plane.  The V plane's
// channels behind the latent are never written and stay zero.  clear_proj: the row of proj that
// was read is zeroed at the end (it lies in a buffer that a split-K product adds into).
template <typename T>
__global__ void __launch_bounds__(128) latent_store_kernel(
    float* __restrict__ proj, int proj_stride, const float* __restrict__ wq, const float* __restrict__ wc,
    const float2* __restrict__ cos_sin, int rot_half, T* __restrict__ cq_out, T* __restrict__ k_plane,
    T* __restrict__ v_plane, long long page_stride, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ row_slot, const int* __restrict__ row_pos, int page_size, int q_rank, int kv_rank,
    int rot_dim, float eps, int write_cache, int clear_proj) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  float* p = proj + (size_t)r * proj_stride;
  float ss = 0.f;
  for (int i = tid; i < q_rank; i += blockDim.x) ss = fmaf(p[i], p[i], ss);
  ss = block_sum(ss, scratch);
  const float sq = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = tid; i < q_rank; i += blockDim.x)
    cq_out[(size_t)r * q_rank + i] = from_f32<T>(p[i] * sq * wq[i]);
  if (!write_cache) {
    if (clear_proj) {
      __syncthreads();
      for (int i = tid; i < q_rank + kv_rank + rot_dim; i += blockDim.x) p[i] = 0.f;
    }
    return;
  }
  const float* c = p + q_rank;
  ss = 0.f;
  for (int i = tid; i < kv_rank; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
  ss = block_sum(ss, scratch);
  const float sc = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  const int pos = row_pos[r];
  const int page = block_table[(size_t)row_slot[r] * table_stride + pos / page_size];
  const int hd = kv_rank + rot_dim;
  const size_t off = (size_t)page * page_stride + (size_t)(pos % page_size) * hd;
  for (int i = tid; i < kv_rank; i += blockDim.x) {
    const T v = from_f32<T>(c[i] * sc * wc[i]);
    k_plane[off + i] = v;
    v_plane[off + i] = v;
  }
  const float* kr = c + kv_rank;
  for (int j = tid; j < rot_dim; j += blockDim.x) {
    float v = kr[j];
    const int i = j >> 1;
    if (cos_sin && i < rot_half) {
      const float2 cs = cos_sin[(size_t)r * rot_half + i];
      const float a = kr[2 * i], b = kr[2 * i + 1];
      v = (j & 1) ? fmaf(b, cs.x, a * cs.y) : fmaf(a, cs.x, -b * cs.y);
    }
    k_plane[off + kv_rank + j] = from_f32<T>(v);
  }
  if (clear_proj) {
    __syncthreads();
    for (int i = tid; i < q_rank + kv_rank + rot_dim; i += blockDim.x) p[i] = 0.f;
  }
}

// q[row][h] = [ plain part (dim) | part to rotate (rot_dim) ] in 32-bit.  The plain part is rounded
// into q_plain[row][h][0:dim] (the operand of the product with U_k,h); the rotated part goes to
// q_full[row][h][kv_rank : kv_rank + rot_dim], behind the place of that product's result.  A pair
// of the rotated part is one thread's work (both values read, both written).  clear: what was
// read of q is zeroed.
template <typename T>
__global__ void latent_query_kernel(float* __restrict__ q, int q_stride, const float2* __restrict__ cos_sin,
                                    int rot_half, T* __restrict__ q_plain, T* __restrict__ q_full, long long total,
                                    int H, int dim, int rot_dim, int kv_rank, int clear) {
  pdl_trigger();
  pdl_wait();
  const int per_head = dim + rot_dim, hd = kv_rank + rot_dim;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long rh = idx / per_head;
    const int e = (int)(idx - rh * per_head);
    const long long r = rh / H;
    const int h = (int)(rh - r * H);
    float* src = q + (size_t)r * q_stride + (size_t)h * per_head;
    if (e < dim) {
      q_plain[(size_t)rh * dim + e] = from_f32<T>(src[e]);
      if (clear) src[e] = 0.f;
    } else {
      const int j = e - dim, i = j >> 1;
      if (j & 1) continue;                       // the pair's even member does both
      const bool two = j + 1 < rot_dim;
      const float a = src[e], b = two ? src[e + 1] : 0.f;
      float va = a, vb = b;
      if (cos_sin && i < rot_half) {
        const float2 cs = cos_sin[(size_t)r * rot_half + i];
        va = fmaf(a, cs.x, -b * cs.y);
        vb = fmaf(b, cs.x, a * cs.y);
      }
      T* dst = q_full + (size_t)rh * hd + kv_rank + j;
      dst[0] = from_f32<T>(va);
      if (two) dst[1] = from_f32<T>(vb);
      if (clear) {
        src[e] = 0.f;
        if (two) src[e + 1] = 0.f;
      }
    }
  }
}
}  // namespace

LLM_EXPORT int llm_latent_store(float* proj, int proj_stride, const float* wq, const float* wc,
                                const float* cos_sin, int rot_half, void* cq_out, void* k_plane, void* v_plane,
                                int dtype, long long page_stride, const int* block_table, int table_stride,
                                const int* row_slot, const int* row_pos, int rows, int page_size, int q_rank,
                                int kv_rank, int rot_dim, float eps, int write_cache, int clear_proj,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (q_rank <= 0 || kv_rank <= 0 || rot_dim < 0 || 2 * rot_half > rot_dim) return LLM_ERR_ARGUMENT;
  if (dtype == LLM_F32)
    return launched_many_blocks(launch_pdl(latent_store_kernel<float>, rows, 128, 0, stream, proj, proj_stride, wq, wc,
                      (const float2*)cos_sin, rot_half, (float*)cq_out, (float*)k_plane, (float*)v_plane,
                      page_stride, block_table, table_stride, row_slot, row_pos, page_size, q_rank, kv_rank,
                      rot_dim, eps, write_cache, clear_proj), rows);
  if (dtype == LLM_BF16)
    return launched_many_blocks(launch_pdl(latent_store_kernel<bf16>, rows, 128, 0, stream, proj, proj_stride, wq, wc,
                      (const float2*)cos_sin, rot_half, (bf16*)cq_out, (bf16*)k_plane, (bf16*)v_plane,
                      page_stride, block_table, table_stride, row_slot, row_pos, page_size, q_rank, kv_rank,
                      rot_dim, eps, write_cache, clear_proj), rows);
  return LLM_ERR_UNSUPPORTED;
}

LLM_EXPORT int llm_latent_query(float* q, int q_stride, const float* cos_sin, int rot_half, void* q_plain,
                                void* q_full, int dtype, int rows, int H, int dim, int rot_dim, int kv_rank,
                                int clear, cudaStream_t stream) {
  const long long total = (long long)rows * H * (dim + rot_dim);
  if (total <= 0) return 0;
  if (2 * rot_half > rot_dim) return LLM_ERR_ARGUMENT;
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  if (dtype == LLM_F32)
    return launched_many_blocks(
        launch_pdl(latent_query_kernel<float>, blocks, 256, 0, stream, q, q_stride, (const float2*)cos_sin, rot_half,
                   (float*)q_plain, (float*)q_full, total, H, dim, rot_dim, kv_rank, clear), blocks);
  if (dtype == LLM_BF16)
    return launched_many_blocks(
        launch_pdl(latent_query_kernel<bf16>, blocks, 256, 0, stream, q, q_stride, (const float2*)cos_sin, rot_half,
                   (bf16*)q_plain, (bf16*)q_full, total, H, dim, rot_dim, kv_rank, clear), blocks);
  return LLM_ERR_UNSUPPORTED;
}
