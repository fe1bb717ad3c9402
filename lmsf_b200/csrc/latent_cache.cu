// The cached side of attention over a low-rank vector per token: c = norm(x W_down^T) * w is all that a token leaves
// in the cache; keys and values are linear in c, so the attention itself can run on c (the key expansion moved into
// the query, the value expansion applied to the attention's output).
//
// latent_norm_cache_write_kernel: RMS norm of the projected rows (float32 inside) fused with the write into the
// pages: [page][1][1][slot][padded rank], the padding (rank rounded up to what the attention kernels take) is zero.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_latent_cache)

namespace lmsf {

template <typename T>
__global__ void __launch_bounds__(128) latent_norm_cache_write_kernel(const T* __restrict__ x, long long x_stride,
                                                                      const float* __restrict__ w, T* __restrict__ cache,
                                                                      long long page_stride, const int* __restrict__ positions,
                                                                      const int* __restrict__ token_seq,
                                                                      const int* __restrict__ block_table, int max_blocks,
                                                                      int block_size, int rank, int padded, float eps,
                                                                      int* __restrict__ error_flag) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(xr[i]); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int blk = pos / block_size;
  const int page = blk < max_blocks ? block_table[(size_t)token_seq[t] * max_blocks + blk] : -1;
  if (page < 0) {   // no page for this position: a fault of the caller, reported and not written
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  T* dst = cache + (size_t)page * page_stride + (size_t)(pos % block_size) * padded;
  for (int i = threadIdx.x; i < padded; i += blockDim.x)
    dst[i] = i < rank ? from_f32<T>((to_f32(xr[i]) * inv) * w[i]) : from_f32<T>(0.f);
}

// The same with a rotated key part behind the normed vector: a row of x holds rank values to norm and `rot_dim` values of
// one key part that all heads share; of those the first `rot_n` are rotated by the token's position (value i pairs with
// value i + rot_n / 2, angle = position * inv_freq[i], float32), the rest pass unchanged.  The page's row is
// [normed vector | key part | zeros]: the attention reads it as one key (and value) of `padded` values.
template <typename T>
__global__ void __launch_bounds__(128) latent_norm_rope_cache_write_kernel(const T* __restrict__ x, long long x_stride,
                                                                           const float* __restrict__ w, T* __restrict__ cache,
                                                                           long long page_stride, const int* __restrict__ positions,
                                                                           const int* __restrict__ token_seq,
                                                                           const int* __restrict__ block_table, int max_blocks,
                                                                           int block_size, int rank, int padded, float eps,
                                                                           int rot_dim, int rot_n, const float* __restrict__ inv_freq,
                                                                           int* __restrict__ error_flag) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f32(xr[i]); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int blk = pos / block_size;
  const int page = blk < max_blocks ? block_table[(size_t)token_seq[t] * max_blocks + blk] : -1;
  if (page < 0) {
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  T* dst = cache + (size_t)page * page_stride + (size_t)(pos % block_size) * padded;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>((to_f32(xr[i]) * inv) * w[i]);
  const int half = rot_n / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float u = to_f32(xr[rank + i]), v = to_f32(xr[rank + half + i]);
    dst[rank + i] = from_f32<T>(rot_first(u, v, cs, sn));
    dst[rank + half + i] = from_f32<T>(rot_second(u, v, cs, sn));
  }
  for (int i = rank + rot_n + threadIdx.x; i < padded; i += blockDim.x)
    dst[i] = i < rank + rot_dim ? xr[i] : from_f32<T>(0.f);
}

// The query's side of the same: every head's rotated part, q[t, h, plain .. plain + rot_dim), is rotated and written behind
// the head's expanded part in the attention's query, qa[t, h, rank .. rank + rot_dim); the padding after it is zeroed.
template <typename T>
__global__ void __launch_bounds__(128) latent_query_rope_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ qa,
                                                                long long qa_stride, const int* __restrict__ positions,
                                                                int heads, int plain, int rot_dim, int rot_n,
                                                                const float* __restrict__ inv_freq, int rank, int padded) {
  extern __shared__ float cs_sn[];                // cos[half], sin[half]
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot_n / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &cs_sn[half + i], &cs_sn[i]);
  __syncthreads();
  const int tail = padded - rank;                 // values behind the expanded part of a head of qa
  const int width = plain + rot_dim;
  for (int j = threadIdx.x; j < heads * tail; j += blockDim.x) {
    const int h = j / tail, i = j % tail;
    const T* src = q + (size_t)t * q_stride + (size_t)h * width + plain;
    float o = 0.f;
    if (i < rot_n) {
      const int p = i < half ? i : i - half;
      const float u = to_f32(src[p]), v = to_f32(src[p + half]);
      o = i < half ? rot_first(u, v, cs_sn[p], cs_sn[half + p]) : rot_second(u, v, cs_sn[p], cs_sn[half + p]);
    } else if (i < rot_dim) {
      o = to_f32(src[i]);
    }
    qa[(size_t)t * qa_stride + (size_t)h * padded + rank + i] = from_f32<T>(o);
  }
}

// x[t, h, :] *= sigmoid(gate[t, h]): a gate per token and head on the attention's output.
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                 int heads, int head_dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * head_dim; i += blockDim.x) {
    const float g = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + i / head_dim])));
    T* p = x + (size_t)t * x_stride + i;
    *p = from_f32<T>(to_f32(*p) * g);
  }
}

// the same on bfloat16 with 16 bytes a thread: head sizes that 8 divides, rows that start on 16-byte boundaries
__global__ void head_gate8_kernel(bf16* __restrict__ x, long long x_stride, const bf16* __restrict__ gate, long long gate_stride,
                                  int heads, int head_dim) {
  const int t = blockIdx.x;
  uint4* row = reinterpret_cast<uint4*>(x + (size_t)t * x_stride);
  const int per_head = head_dim / 8;
  for (int i = threadIdx.x; i < heads * per_head; i += blockDim.x) {
    const float g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + i / per_head])));
    uint4 v = row[i];
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      p[k] = __floats2bfloat162_rn(f.x * g, f.y * g);
    }
    row[i] = v;
  }
}

// x[t, h, d] *= sigmoid(gate[t, h, d]) for the first `value_dim` values of every head of head_dim values: a gate per element
// of the concatenated value heads (the gate has no padding, the attention's output may have).
template <typename T>
__global__ void value_gate_kernel(T* __restrict__ x, long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                  int heads, int head_dim, int value_dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * value_dim; i += blockDim.x) {
    const int h = i / value_dim, d = i - h * value_dim;
    const float g = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + i])));
    T* p = x + (size_t)t * x_stride + (size_t)h * head_dim + d;
    *p = from_f32<T>(to_f32(*p) * g);
  }
}

// the same, four values a thread and access: sizes that 4 divides, aligned rows
template <typename T>
__global__ void value_gate4_kernel(T* __restrict__ x, long long x_stride, const T* __restrict__ gate, long long gate_stride,
                                   int heads, int head_dim, int value_dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 4; i < heads * value_dim; i += blockDim.x * 4) {
    const int h = i / value_dim, d = i - h * value_dim;
    float g[4], v[4];
    ld4(gate + (size_t)t * gate_stride + i, g);
    T* p = x + (size_t)t * x_stride + (size_t)h * head_dim + d;
    ld4(p, v);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] *= 1.0f / (1.0f + expf(-g[k]));
    st4(p, v);
  }
}

}  // namespace lmsf

LMSF_API int lmsf_value_gate(void* x, long long x_stride, const void* gate, long long gate_stride, int n, int heads,
                             int head_dim, int value_dim, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (heads <= 0 || head_dim <= 0 || value_dim <= 0 || value_dim > head_dim)
    LMSF_REFUSE("value_gate: heads=%d head_dim=%d value_dim=%d", heads, head_dim, value_dim);
  cudaStream_t s = (cudaStream_t)stream;
  if (value_dim % 4 == 0 && head_dim % 4 == 0 && (dtype == LMSF_F32 || dtype == LMSF_BF16)) {
    if (dtype == LMSF_F32 && rows_take4<float>(x, 4, x_stride) && rows_take4<float>(gate, 4, gate_stride)) {
      value_gate4_kernel<float><<<n, 256, 0, s>>>((float*)x, x_stride, (const float*)gate, gate_stride, heads, head_dim, value_dim);
      return LMSF_LAUNCH_STATUS();
    }
    if (dtype == LMSF_BF16 && rows_take4<bf16>(x, 4, x_stride) && rows_take4<bf16>(gate, 4, gate_stride)) {
      value_gate4_kernel<bf16><<<n, 256, 0, s>>>((bf16*)x, x_stride, (const bf16*)gate, gate_stride, heads, head_dim, value_dim);
      return LMSF_LAUNCH_STATUS();
    }
  }
  if (dtype == LMSF_F32) value_gate_kernel<float><<<n, 256, 0, s>>>((float*)x, x_stride, (const float*)gate, gate_stride, heads, head_dim, value_dim);
  else if (dtype == LMSF_BF16) value_gate_kernel<bf16><<<n, 256, 0, s>>>((bf16*)x, x_stride, (const bf16*)gate, gate_stride, heads, head_dim, value_dim);
  else LMSF_REFUSE("value_gate: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_head_gate(void* x, long long x_stride, const void* gate, long long gate_stride, int n, int heads,
                            int head_dim, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (heads <= 0 || head_dim <= 0) LMSF_REFUSE("head_gate: heads=%d head_dim=%d", heads, head_dim);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) head_gate_kernel<float><<<n, 256, 0, s>>>((float*)x, x_stride, (const float*)gate, gate_stride, heads, head_dim);
  else if (dtype == LMSF_BF16) {
    if (head_dim % 8 == 0 && x_stride % 8 == 0 && (uintptr_t)x % 16 == 0)
      head_gate8_kernel<<<n, 256, 0, s>>>((bf16*)x, x_stride, (const bf16*)gate, gate_stride, heads, head_dim);
    else
      head_gate_kernel<bf16><<<n, 256, 0, s>>>((bf16*)x, x_stride, (const bf16*)gate, gate_stride, heads, head_dim);
  }
  else LMSF_REFUSE("head_gate: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// x: rows of [n, rank] of `dtype` (row stride x_stride); w: float32 [rank]; cache: [pages, 1, 1, block_size, padded].
LMSF_API int lmsf_latent_norm_cache_write(const void* x, long long x_stride, const float* w, void* cache,
                                          long long page_stride, const int* positions, const int* token_seq,
                                          const int* block_table, int max_blocks, int block_size, int n, int rank, int padded,
                                          float eps, int dtype, int* error_flag, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (rank <= 0 || padded < rank || block_size <= 0 || max_blocks <= 0 || !(eps > 0.f))
    LMSF_REFUSE("latent cache: rank=%d padded=%d block_size=%d max_blocks=%d", rank, padded, block_size, max_blocks);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32)
    latent_norm_cache_write_kernel<float><<<n, 128, 0, s>>>((const float*)x, x_stride, w, (float*)cache, page_stride, positions,
                                                            token_seq, block_table, max_blocks, block_size, rank, padded, eps, error_flag);
  else if (dtype == LMSF_BF16)
    latent_norm_cache_write_kernel<bf16><<<n, 128, 0, s>>>((const bf16*)x, x_stride, w, (bf16*)cache, page_stride, positions,
                                                           token_seq, block_table, max_blocks, block_size, rank, padded, eps, error_flag);
  else LMSF_REFUSE("latent cache: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// x: rows of [n, rank + rot_dim] of `dtype`; inv_freq: float32 [rot_n / 2]; cache: [pages, 1, 1, block_size, padded] with
// padded >= rank + rot_dim.
LMSF_API int lmsf_latent_norm_rope_cache_write(const void* x, long long x_stride, const float* w, void* cache,
                                               long long page_stride, const int* positions, const int* token_seq,
                                               const int* block_table, int max_blocks, int block_size, int n, int rank,
                                               int padded, float eps, int rot_dim, int rot_n, const float* inv_freq, int dtype,
                                               int* error_flag, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (rank <= 0 || rot_dim < 0 || padded < rank + rot_dim || block_size <= 0 || max_blocks <= 0 || !(eps > 0.f))
    LMSF_REFUSE("latent cache: rank=%d rot_dim=%d padded=%d block_size=%d max_blocks=%d", rank, rot_dim, padded, block_size, max_blocks);
  if (rot_n < 0 || rot_n % 2 || rot_n > rot_dim || (rot_n > 0 && !inv_freq))
    LMSF_REFUSE("latent cache: %d rotated values of %d (even, with their frequencies)", rot_n, rot_dim);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32)
    latent_norm_rope_cache_write_kernel<float><<<n, 128, 0, s>>>((const float*)x, x_stride, w, (float*)cache, page_stride, positions,
                                                                 token_seq, block_table, max_blocks, block_size, rank, padded, eps,
                                                                 rot_dim, rot_n, inv_freq, error_flag);
  else if (dtype == LMSF_BF16)
    latent_norm_rope_cache_write_kernel<bf16><<<n, 128, 0, s>>>((const bf16*)x, x_stride, w, (bf16*)cache, page_stride, positions,
                                                                token_seq, block_table, max_blocks, block_size, rank, padded, eps,
                                                                rot_dim, rot_n, inv_freq, error_flag);
  else LMSF_REFUSE("latent cache: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// q: [n, heads * (plain + rot_dim)] of `dtype`; qa: [n, heads * padded] of `dtype`, of which this call writes the columns
// rank .. padded of every head.
LMSF_API int lmsf_latent_query_rope(const void* q, long long q_stride, void* qa, long long qa_stride, const int* positions,
                                    int n, int heads, int plain, int rot_dim, int rot_n, const float* inv_freq, int rank,
                                    int padded, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (heads <= 0 || plain < 0 || rot_dim < 0 || rank <= 0 || padded < rank + rot_dim)
    LMSF_REFUSE("latent query: heads=%d plain=%d rot_dim=%d rank=%d padded=%d", heads, plain, rot_dim, rank, padded);
  if (rot_n < 0 || rot_n % 2 || rot_n > rot_dim || (rot_n > 0 && !inv_freq))
    LMSF_REFUSE("latent query: %d rotated values of %d (even, with their frequencies)", rot_n, rot_dim);
  if (padded == rank) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = (size_t)rot_n * sizeof(float);
  if (dtype == LMSF_F32)
    latent_query_rope_kernel<float><<<n, 128, smem, s>>>((const float*)q, q_stride, (float*)qa, qa_stride, positions, heads, plain,
                                                         rot_dim, rot_n, inv_freq, rank, padded);
  else if (dtype == LMSF_BF16)
    latent_query_rope_kernel<bf16><<<n, 128, smem, s>>>((const bf16*)q, q_stride, (bf16*)qa, qa_stride, positions, heads, plain,
                                                        rot_dim, rot_n, inv_freq, rank, padded);
  else LMSF_REFUSE("latent query: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}
