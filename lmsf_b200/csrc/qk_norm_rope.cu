// For attention layers that norm their queries and keys per head: RMS norm over the first `norm_dim` values of every head
// of q and k (one weight vector for all query heads, one for all key heads), then the rotary encoding of the first
// `rot_dim` values, then the write of k and v into the paged cache, in one kernel.  Everything between the load and the
// store is float32: a value is rounded once, after the rotation.
//
// A head may be wider than `norm_dim` (query/key and value sizes that differ share one cache width): the norm's mean is
// taken over norm_dim values, the rest pass as they are.
//
// Cache layout of one layer: [page][2 (k, v)][kv_head][slot][head_dim], as in rope_cache.cu.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_qk_norm_rope)

namespace lmsf {

struct QkNormRopeArgs {
  void* q; const void* k; const void* v;
  long long q_stride, k_stride, v_stride;
  const int* positions; const int* token_seq; const int* block_table;
  int max_blocks, block_size;
  void* cache; long long page_stride;
  const float* inv_freq; int rot_dim, is_neox;
  int n_q_heads, n_kv_heads, head_dim, norm_dim;
  const float* wq; const float* wk; float eps;
  int* error_flag;
  int weightless;       // 1: q and k are divided by their root mean square although wq and wk are null (a norm without a weight)
  int v_norm_dim;       // > 0: every value head is divided by the root mean square of its first v_norm_dim values before it is stored
};

constexpr int kWarps = 4;

// One block per token; a warp takes a head at a time: query heads (in place), key heads (to the cache), value heads (copied).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) qk_norm_rope_kernel(QkNormRopeArgs a) {
  extern __shared__ float smem[];                 // cos[half], sin[half], then a head per warp
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = a.positions[t];
  const int half = a.inv_freq ? a.rot_dim / 2 : 0;
  float* cs = smem;
  float* buf = smem + 2 * half + warp * a.head_dim;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * a.inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  const int hd = a.head_dim;
  T* kc = nullptr;
  T* vc = nullptr;
  if (a.cache) {
    const int page = a.block_table[(size_t)a.token_seq[t] * a.max_blocks + pos / a.block_size];
    if (page < 0) {
      if (threadIdx.x == 0 && a.error_flag) atomicExch(a.error_flag, 2);
    } else {
      kc = (T*)a.cache + (size_t)page * a.page_stride + (size_t)(pos % a.block_size) * hd;
      vc = kc + (size_t)a.n_kv_heads * a.block_size * hd;
    }
  }
  const size_t head_pitch = (size_t)a.block_size * hd;
  const int n_k = a.cache ? a.n_kv_heads : 0;
  for (int head = warp; head < a.n_q_heads + 2 * n_k; head += kWarps) {
    if (head >= a.n_q_heads + n_k) {              // a value head: a copy
      const int g = head - a.n_q_heads - n_k;
      if (vc) {
        const T* src = (const T*)a.v + (size_t)t * a.v_stride + (size_t)g * hd;
        if (a.v_norm_dim > 0) {
          float ss = 0.f;
          for (int i = lane; i < a.v_norm_dim; i += 32) { const float x = to_f32(src[i]); ss = fmaf(x, x, ss); }
          const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.v_norm_dim + a.eps);
          for (int i = lane; i < hd; i += 32) vc[g * head_pitch + i] = i < a.v_norm_dim ? from_f32<T>(to_f32(src[i]) * inv) : src[i];
        } else {
          for (int i = lane; i < hd; i += 32) vc[g * head_pitch + i] = src[i];
        }
      }
      continue;
    }
    const bool is_q = head < a.n_q_heads;
    const int g = is_q ? head : head - a.n_q_heads;
    if (!is_q && !kc) continue;
    const T* src = is_q ? (const T*)a.q + (size_t)t * a.q_stride + (size_t)g * hd
                        : (const T*)a.k + (size_t)t * a.k_stride + (size_t)g * hd;
    T* dst = is_q ? (T*)a.q + (size_t)t * a.q_stride + (size_t)g * hd : kc + g * head_pitch;
    const float* w = is_q ? a.wq : a.wk;
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      const float x = to_f32(src[i]);
      buf[i] = x;
      if (i < a.norm_dim) ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    __syncwarp();
    if (w || a.weightless) {
      const float inv = 1.0f / sqrtf(ss / (float)a.norm_dim + a.eps);
      for (int i = lane; i < a.norm_dim; i += 32) buf[i] = w ? (buf[i] * inv) * w[i] : buf[i] * inv;
    }
    __syncwarp();
    for (int p = lane; p < half; p += 32) {
      const int ix = a.is_neox ? p : 2 * p, iy = a.is_neox ? p + half : 2 * p + 1;
      const float c = cs[p], s = cs[half + p], x = buf[ix], y = buf[iy];
      dst[ix] = from_f32<T>(rot_first(x, y, c, s));
      dst[iy] = from_f32<T>(rot_second(x, y, c, s));
    }
    for (int i = 2 * half + lane; i < hd; i += 32) dst[i] = from_f32<T>(buf[i]);
    __syncwarp();
  }
}

// Interleaved pairs (or no rotation) and a head of 32 * VW values: a lane holds VW consecutive values of the head in
// registers from the load to the store, so a pair never leaves its lane and nothing passes through shared memory but
// the token's cosines and sines.  Needs rows and heads aligned to VW values.
template <typename T, int VW> struct alignas(sizeof(T) * VW) HeadVec { T v[VW]; };

template <typename T, int VW>
__global__ void __launch_bounds__(kWarps * 32) qk_norm_rope_vec_kernel(QkNormRopeArgs a) {
  extern __shared__ float smem[];                 // cos[half], sin[half]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = a.positions[t];
  const int half = a.inv_freq ? a.rot_dim / 2 : 0;
  float* cs = smem;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * a.inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  const int hd = a.head_dim;
  T* kc = nullptr;
  T* vc = nullptr;
  if (a.cache) {
    const int page = a.block_table[(size_t)a.token_seq[t] * a.max_blocks + pos / a.block_size];
    if (page < 0) {
      if (threadIdx.x == 0 && a.error_flag) atomicExch(a.error_flag, 2);
    } else {
      kc = (T*)a.cache + (size_t)page * a.page_stride + (size_t)(pos % a.block_size) * hd;
      vc = kc + (size_t)a.n_kv_heads * a.block_size * hd;
    }
  }
  const size_t head_pitch = (size_t)a.block_size * hd;
  const int n_k = a.cache ? a.n_kv_heads : 0;
  const int e0 = lane * VW;
  typedef HeadVec<T, VW> Vec;
  for (int head = warp + kWarps * blockIdx.y; head < a.n_q_heads + 2 * n_k; head += kWarps * gridDim.y) {
    if (head >= a.n_q_heads + n_k) {
      const int g = head - a.n_q_heads - n_k;
      if (vc) {
        Vec raw = *reinterpret_cast<const Vec*>((const T*)a.v + (size_t)t * a.v_stride + (size_t)g * hd + e0);
        if (a.v_norm_dim > 0) {
          float x[VW];
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < VW; ++j) {
            x[j] = to_f32(raw.v[j]);
            if (e0 + j < a.v_norm_dim) ss = fmaf(x[j], x[j], ss);
          }
          const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)a.v_norm_dim + a.eps);
#pragma unroll
          for (int j = 0; j < VW; ++j)
            if (e0 + j < a.v_norm_dim) raw.v[j] = from_f32<T>(x[j] * inv);
        }
        *reinterpret_cast<Vec*>(vc + g * head_pitch + e0) = raw;
      }
      continue;
    }
    const bool is_q = head < a.n_q_heads;
    const int g = is_q ? head : head - a.n_q_heads;
    if (!is_q && !kc) continue;
    const T* src = is_q ? (const T*)a.q + (size_t)t * a.q_stride + (size_t)g * hd
                        : (const T*)a.k + (size_t)t * a.k_stride + (size_t)g * hd;
    T* dst = is_q ? (T*)a.q + (size_t)t * a.q_stride + (size_t)g * hd : kc + g * head_pitch;
    const float* w = is_q ? a.wq : a.wk;
    Vec raw = *reinterpret_cast<const Vec*>(src + e0);
    float x[VW];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VW; ++j) {
      x[j] = to_f32(raw.v[j]);
      if (e0 + j < a.norm_dim) ss = fmaf(x[j], x[j], ss);
    }
    ss = warp_sum(ss);
    if (w || a.weightless) {
      const float inv = 1.0f / sqrtf(ss / (float)a.norm_dim + a.eps);
#pragma unroll
      for (int j = 0; j < VW; ++j)
        if (e0 + j < a.norm_dim) x[j] = w ? (x[j] * inv) * w[e0 + j] : x[j] * inv;
    }
#pragma unroll
    for (int j = 0; j < VW; j += 2) {
      if (e0 + j < 2 * half) {
        const int p = (e0 + j) >> 1;
        const float c = cs[p], s = cs[half + p], u = x[j], v = x[j + 1];
        x[j] = rot_first(u, v, c, s);
        x[j + 1] = rot_second(u, v, c, s);
      }
    }
#pragma unroll
    for (int j = 0; j < VW; ++j) raw.v[j] = from_f32<T>(x[j]);
    *reinterpret_cast<Vec*>(dst + e0) = raw;
  }
}

}  // namespace lmsf

// q: [n, n_q_heads * head_dim] (changed in place), k, v: [n, n_kv_heads * head_dim], rows of `dtype` with the given strides;
// wq, wk: float32 [norm_dim] or null (no norm, or with `weightless` a norm without a weight); inv_freq: float32
// [rot_dim / 2] or null (no rotation); cache null: q only.  v_norm_dim > 0: the value heads are normed too (no weight).
LMSF_API int lmsf_qk_norm_rope_cache_write_unit(void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                                long long v_stride, const int* positions, const int* token_seq,
                                                const int* block_table, int max_blocks, int block_size, void* cache,
                                                long long page_stride, const float* inv_freq, int rot_dim, int is_neox,
                                                int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int norm_dim,
                                                const float* wq, const float* wk, float eps, int dtype, int* error_flag,
                                                int weightless, int v_norm_dim, void* stream) {
  using namespace lmsf;
  if (n_tokens <= 0) return 0;
  if (head_dim <= 0 || n_q_heads < 0 || n_kv_heads < 0 || norm_dim <= 0 || norm_dim > head_dim)
    LMSF_REFUSE("qk_norm_rope: head_dim=%d norm_dim=%d", head_dim, norm_dim);
  if (inv_freq && (rot_dim <= 0 || rot_dim % 2 || rot_dim > norm_dim))
    LMSF_REFUSE("qk_norm_rope: rot_dim=%d must be even and at most %d", rot_dim, norm_dim);
  if ((wq || wk || weightless || v_norm_dim > 0) && !(eps > 0.f)) LMSF_REFUSE("qk_norm_rope: eps must be positive");
  if (v_norm_dim < 0 || v_norm_dim > head_dim) LMSF_REFUSE("qk_norm_rope: v_norm_dim=%d of head_dim=%d", v_norm_dim, head_dim);
  if (cache && (!k || !v || !block_table || !token_seq || block_size <= 0 || max_blocks <= 0))
    LMSF_REFUSE("qk_norm_rope: a cache write needs k, v, a block table and the block size");
  QkNormRopeArgs a{q, k, v, q_stride, k_stride, v_stride, positions, token_seq, block_table, max_blocks, block_size, cache,
                   page_stride, inv_freq, rot_dim, is_neox, n_q_heads, n_kv_heads, head_dim, norm_dim, wq, wk, eps, error_flag,
                   weightless ? 1 : 0, v_norm_dim};
  const size_t smem = ((inv_freq ? rot_dim : 0) + (size_t)kWarps * head_dim) * sizeof(float);
  if (smem > 48 * 1024) LMSF_REFUSE("qk_norm_rope: head_dim=%d is too wide", head_dim);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("qk_norm_rope: unknown dtype code %d", dtype);
  const int vw = head_dim / 32;
  const size_t esz = dtype == LMSF_F32 ? 4 : 2;
  if ((!inv_freq || !is_neox) && head_dim % 32 == 0 && (vw == 2 || vw == 4 || vw == 8) && q_stride % vw == 0 &&
      (!cache || (k_stride % vw == 0 && v_stride % vw == 0 && page_stride % vw == 0)) &&
      ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)cache) % (esz * vw) == 0) {
    const int heads = n_q_heads + (cache ? 2 * n_kv_heads : 0);
    // few tokens (a decode step): a token's heads are spread over several blocks
    dim3 grid(n_tokens, n_tokens >= 256 ? 1 : (heads >= 32 ? 4 : (heads >= 8 ? 2 : 1)));
    const size_t cs_bytes = (inv_freq ? rot_dim : 0) * sizeof(float);
#define LMSF_GO(T, VW) qk_norm_rope_vec_kernel<T, VW><<<grid, kWarps * 32, cs_bytes, s>>>(a)
    if (dtype == LMSF_F32) { if (vw == 2) LMSF_GO(float, 2); else if (vw == 4) LMSF_GO(float, 4); else LMSF_GO(float, 8); }
    else { if (vw == 2) LMSF_GO(bf16, 2); else if (vw == 4) LMSF_GO(bf16, 4); else LMSF_GO(bf16, 8); }
#undef LMSF_GO
    return LMSF_LAUNCH_STATUS();
  }
  if (dtype == LMSF_F32) qk_norm_rope_kernel<float><<<n_tokens, kWarps * 32, smem, s>>>(a);
  else if (dtype == LMSF_BF16) qk_norm_rope_kernel<bf16><<<n_tokens, kWarps * 32, smem, s>>>(a);
  else LMSF_REFUSE("qk_norm_rope: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_qk_norm_rope_cache_write(void* q, const void* k, const void* v, long long q_stride, long long k_stride,
                                           long long v_stride, const int* positions, const int* token_seq,
                                           const int* block_table, int max_blocks, int block_size, void* cache,
                                           long long page_stride, const float* inv_freq, int rot_dim, int is_neox,
                                           int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int norm_dim,
                                           const float* wq, const float* wk, float eps, int dtype, int* error_flag,
                                           void* stream) {
  return lmsf_qk_norm_rope_cache_write_unit(q, k, v, q_stride, k_stride, v_stride, positions, token_seq, block_table, max_blocks,
                                            block_size, cache, page_stride, inv_freq, rot_dim, is_neox, n_tokens, n_q_heads,
                                            n_kv_heads, head_dim, norm_dim, wq, wk, eps, dtype, error_flag, 0, 0, stream);
}
