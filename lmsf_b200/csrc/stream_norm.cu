// Norms around a float32 residual stream, for blocks that norm a branch before AND after it
// (x <- x + scale * norm_post(branch(norm_pre(x)))), and the embedding that is normed before it enters the stream.
//
// One kernel does what lies between two branches:
//   res <- res + norm(y) * w_post * layer_scale * m  (the branch just computed, if there is one; m: one factor for the model)
//   res <- res + first + vec                          (what a repeated span of layers adds at its entry, if given)
//   h    = norm(res) * w_next                         (the input of the next branch, if asked for; without w_next: h = res,
//                                                      for blocks whose branches read the stream itself)
// Every sum, root and product is float32; y and h have the activation type.  One block per token; the row is held
// in registers between the passes (up to kMaxPerThread values per thread), so y and res are read once.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_stream_norm)

namespace lmsf {

constexpr int kThreads = 256;
constexpr int kMaxPerThread = 64;   // widths up to 16,384

// V consecutive values of a row as floats (V = 4: one 16-byte or 8-byte access; V = 1: any width and alignment)
template <int V> __device__ __forceinline__ void ld_vec(const float* p, float (&v)[V]) {
  if (V == 4) { const float4 x = *reinterpret_cast<const float4*>(p); v[0] = x.x; v[1 % V] = x.y; v[2 % V] = x.z; v[3 % V] = x.w; }
  else v[0] = *p;
}
template <int V> __device__ __forceinline__ void ld_vec(const bf16* p, float (&v)[V]) {
  if (V == 4) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
    v[0] = a.x; v[1 % V] = a.y; v[2 % V] = b.x; v[3 % V] = b.y;
  } else v[0] = __bfloat162float(*p);
}
template <int V> __device__ __forceinline__ void st_vec(float* p, const float (&v)[V]) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1 % V], v[2 % V], v[3 % V]);
  else *p = v[0];
}
template <int V> __device__ __forceinline__ void st_vec(bf16* p, const float (&v)[V]) {
  if (V == 4) {
    uint2 x;
    *reinterpret_cast<__nv_bfloat162*>(&x.x) = __floats2bfloat162_rn(v[0], v[1 % V]);
    *reinterpret_cast<__nv_bfloat162*>(&x.y) = __floats2bfloat162_rn(v[2 % V], v[3 % V]);
    *reinterpret_cast<uint2*>(p) = x;
  } else *p = __float2bfloat16_rn(v[0]);
}

// PER passes of kThreads threads with V values each cover a row.
template <typename T, int PER, int V>
__global__ void __launch_bounds__(kThreads) stream_norm_kernel(float* __restrict__ res, const T* __restrict__ y,
                                                               const float* __restrict__ w_post, const float* __restrict__ ls,
                                                               const float* __restrict__ first, const float* __restrict__ vec,
                                                               T* __restrict__ h, const float* __restrict__ w_next,
                                                               int hidden, float eps_post, float eps_next, float branch_scale) {
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * hidden;
  float v[PER][V];
  float r[PER][V];
  pdl_launch_dependents();
  pdl_wait();
  float ss = 0.f;
  if (y != nullptr) {
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int i = (it * kThreads + threadIdx.x) * V;
      if (i < hidden) ld_vec<V>(y + base + i, v[it]);
#pragma unroll
      for (int e = 0; e < V; ++e) { if (i >= hidden) v[it][e] = 0.f; ss = fmaf(v[it][e], v[it][e], ss); }
    }
    ss = block_sum(ss, scratch);
  }
  const float inv_post = 1.0f / sqrtf(ss / (float)hidden + eps_post);
  const bool changes = y != nullptr || first != nullptr || vec != nullptr;
  float s2 = 0.f;
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int i = (it * kThreads + threadIdx.x) * V;
#pragma unroll
    for (int e = 0; e < V; ++e) r[it][e] = 0.f;
    if (i < hidden) {
      ld_vec<V>(res + base + i, r[it]);
      if (y != nullptr) {
        float wp[V], l[V];
        ld_vec<V>(w_post + i, wp);
        if (ls != nullptr) ld_vec<V>(ls + i, l);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          float b = (v[it][e] * inv_post) * wp[e];
          if (ls != nullptr) b *= l[e];
          r[it][e] = fmaf(branch_scale, b, r[it][e]);
        }
      }
      if (first != nullptr) {
        float f[V];
        ld_vec<V>(first + base + i, f);
#pragma unroll
        for (int e = 0; e < V; ++e) r[it][e] += f[e];
      }
      if (vec != nullptr) {
        float f[V];
        ld_vec<V>(vec + i, f);
#pragma unroll
        for (int e = 0; e < V; ++e) r[it][e] += f[e];
      }
      if (changes) st_vec<V>(res + base + i, r[it]);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) s2 = fmaf(r[it][e], r[it][e], s2);
  }
  if (h == nullptr) return;
  if (w_next == nullptr) {        // the stream itself, in the activation type
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int i = (it * kThreads + threadIdx.x) * V;
      if (i < hidden) st_vec<V>(h + base + i, r[it]);
    }
    return;
  }
  s2 = block_sum(s2, scratch);
  const float inv = 1.0f / sqrtf(s2 / (float)hidden + eps_next);
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int i = (it * kThreads + threadIdx.x) * V;
    if (i < hidden) {
      float wn[V], o[V];
      ld_vec<V>(w_next + i, wn);
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = (r[it][e] * inv) * wn[e];
      st_vec<V>(h + base + i, o);
    }
  }
}

// res[t] = norm(table[ids[t]]) * w (float32), and a second copy in `keep` when it is not null.
// An id outside the vocabulary writes zeros and raises the error flag.
template <typename T, int PER>
__global__ void __launch_bounds__(kThreads) embed_norm_kernel(float* __restrict__ res, float* __restrict__ keep,
                                                              const T* __restrict__ table, const int* __restrict__ ids,
                                                              const float* __restrict__ w, int hidden, int vocab, float eps,
                                                              float scale, int* __restrict__ error_flag) {
  __shared__ float scratch[33];
  const int id = ids[blockIdx.x];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  const size_t base = (size_t)blockIdx.x * hidden;
  float v[PER];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int i = it * kThreads + threadIdx.x;
    v[it] = (ok && i < hidden) ? to_f32(src[i]) * scale : 0.f;
    ss = fmaf(v[it], v[it], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int i = it * kThreads + threadIdx.x;
    if (i < hidden) {
      const float o = ok ? (v[it] * inv) * w[i] : 0.f;
      res[base + i] = o;
      if (keep != nullptr) keep[base + i] = o;
    }
  }
}

// res = float(x): an embedding's output becomes the float32 residual stream.
template <typename T>
__global__ void stream_begin_kernel(float* __restrict__ res, const T* __restrict__ x, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) res[i] = to_f32(x[i]);
}

template <typename T, int PER, int V>
static int launch_stream(float* res, const void* y, const float* w_post, const float* ls, const float* first,
                         const float* vec, void* h, const float* w_next, int n, int hidden, float eps_post, float eps_next,
                         float branch_scale, cudaStream_t s) {
  return launch_pdl(stream_norm_kernel<T, PER, V>, dim3(n), dim3(kThreads), 0, s, res, (const T*)y, w_post, ls, first, vec,
                    (T*)h, w_next, hidden, eps_post, eps_next, branch_scale);
}

template <typename T>
static int pick_stream(float* res, const void* y, const float* w_post, const float* ls, const float* first,
                       const float* vec, void* h, const float* w_next, int n, int hidden, float eps_post, float eps_next,
                       float branch_scale, cudaStream_t s) {
  // four values per thread and access where the rows allow it (every pointer is then 8- or 16-byte aligned)
  const bool wide = hidden % 4 == 0 && ((uintptr_t)res | (uintptr_t)first | (uintptr_t)w_post | (uintptr_t)ls | (uintptr_t)vec |
                                        (uintptr_t)w_next) % 16 == 0 && ((uintptr_t)y | (uintptr_t)h) % (4 * sizeof(T)) == 0;
  const int per = ceil_div(hidden, kThreads * (wide ? 4 : 1));
#define LMSF_CASE(P)                                                                                                          \
  if (per <= P) return wide ? launch_stream<T, P, 4>(res, y, w_post, ls, first, vec, h, w_next, n, hidden, eps_post, eps_next, branch_scale, s) \
                            : launch_stream<T, P, 1>(res, y, w_post, ls, first, vec, h, w_next, n, hidden, eps_post, eps_next, branch_scale, s)
  LMSF_CASE(1); LMSF_CASE(2); LMSF_CASE(4); LMSF_CASE(8); LMSF_CASE(16);
  if (!wide) { LMSF_CASE(32); LMSF_CASE(64); }
#undef LMSF_CASE
  return LMSF_EBADARG;
}


// Two branches that read the same normed stream, each behind a gate of its own (a layer whose mixer and feed-forward run
// side by side):  res <- res + sigmoid(z[:, 0:D] + b[0:D]) * y1 + sigmoid(z[:, D:2D] + b[D:2D]) * y2, then, if asked,
// h = norm(res) * w_next for whoever reads the stream next.  z: float32 gate logits [n, D or 2 D] (row stride ldz), b:
// float32 [D or 2 D] or null; y2 may be null (a layer without a feed-forward).  Sigmoid, products and sums are float32.
template <typename T, int PER, int V>
__global__ void __launch_bounds__(kThreads) gated_branches_kernel(float* __restrict__ res, const float* __restrict__ z,
                                                                  long long ldz, const float* __restrict__ b,
                                                                  const T* __restrict__ y1, const T* __restrict__ y2,
                                                                  T* __restrict__ h, const float* __restrict__ w_next,
                                                                  int hidden, float eps_next) {
  __shared__ float scratch[33];
  const size_t base = (size_t)blockIdx.x * hidden;
  const float* zr = z + (size_t)blockIdx.x * ldz;
  float r[PER][V];
  pdl_launch_dependents();
  pdl_wait();
  float s2 = 0.f;
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int i = (it * kThreads + threadIdx.x) * V;
#pragma unroll
    for (int e = 0; e < V; ++e) r[it][e] = 0.f;
    if (i < hidden) {
      ld_vec<V>(res + base + i, r[it]);
      float g[V], c[V], y[V];
      ld_vec<V>(zr + i, g);
      if (b != nullptr) { ld_vec<V>(b + i, c);
#pragma unroll
        for (int e = 0; e < V; ++e) g[e] += c[e]; }
      ld_vec<V>(y1 + base + i, y);
#pragma unroll
      for (int e = 0; e < V; ++e) r[it][e] = fmaf(1.0f / (1.0f + expf(-g[e])), y[e], r[it][e]);
      if (y2 != nullptr) {
        ld_vec<V>(zr + hidden + i, g);
        if (b != nullptr) { ld_vec<V>(b + hidden + i, c);
#pragma unroll
          for (int e = 0; e < V; ++e) g[e] += c[e]; }
        ld_vec<V>(y2 + base + i, y);
#pragma unroll
        for (int e = 0; e < V; ++e) r[it][e] = fmaf(1.0f / (1.0f + expf(-g[e])), y[e], r[it][e]);
      }
      st_vec<V>(res + base + i, r[it]);
    }
#pragma unroll
    for (int e = 0; e < V; ++e) s2 = fmaf(r[it][e], r[it][e], s2);
  }
  if (h == nullptr) return;
  s2 = block_sum(s2, scratch);
  const float inv = 1.0f / sqrtf(s2 / (float)hidden + eps_next);
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int i = (it * kThreads + threadIdx.x) * V;
    if (i < hidden) {
      float wn[V], o[V];
      ld_vec<V>(w_next + i, wn);
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = (r[it][e] * inv) * wn[e];
      st_vec<V>(h + base + i, o);
    }
  }
}

// out[t] = [a[t] | b[t]] in the activation type: two float32 streams side by side as the input of one product.
template <typename T>
__global__ void stream_concat_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                     int hidden, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / (2 * hidden);
  const int c = (int)(i % (2 * hidden));
  out[i] = from_f32<T>(c < hidden ? a[t * hidden + c] : b[t * hidden + c - hidden]);
}

// the same, four values a thread (hidden a multiple of 4, all pointers 16-byte aligned): i counts groups of four
template <typename T>
__global__ void stream_concat4_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                      int hidden, long long n4) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const int q = hidden / 4;
  const long long t = i / (2 * q);
  const int c = (int)(i % (2 * q));
  const float4 v = c < q ? reinterpret_cast<const float4*>(a)[t * q + c] : reinterpret_cast<const float4*>(b)[t * q + c - q];
  T* dst = out + i * 4;
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(dst) = v;
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<unsigned*>(&lo);
    packed.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
  }
}

template <typename T, int PER, int V>
static int launch_gated(float* res, const float* z, long long ldz, const float* b, const void* y1, const void* y2, void* h,
                        const float* w_next, int n, int hidden, float eps_next, cudaStream_t s) {
  return launch_pdl(gated_branches_kernel<T, PER, V>, dim3(n), dim3(kThreads), 0, s, res, z, ldz, b, (const T*)y1, (const T*)y2,
                    (T*)h, w_next, hidden, eps_next);
}

template <typename T>
static int pick_gated(float* res, const float* z, long long ldz, const float* b, const void* y1, const void* y2, void* h,
                      const float* w_next, int n, int hidden, float eps_next, cudaStream_t s) {
  const bool wide = hidden % 4 == 0 && ldz % 4 == 0 && ((uintptr_t)res | (uintptr_t)z | (uintptr_t)b | (uintptr_t)w_next) % 16 == 0 &&
                    ((uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)h) % (4 * sizeof(T)) == 0;
  const int per = ceil_div(hidden, kThreads * (wide ? 4 : 1));
#define LMSF_CASE(P)                                                                                              \
  if (per <= P) return wide ? launch_gated<T, P, 4>(res, z, ldz, b, y1, y2, h, w_next, n, hidden, eps_next, s)   \
                            : launch_gated<T, P, 1>(res, z, ldz, b, y1, y2, h, w_next, n, hidden, eps_next, s)
  LMSF_CASE(1); LMSF_CASE(2); LMSF_CASE(4); LMSF_CASE(8); LMSF_CASE(16);
  if (!wide) { LMSF_CASE(32); LMSF_CASE(64); }
#undef LMSF_CASE
  return LMSF_EBADARG;
}

}  // namespace lmsf

// res: float32 [n, hidden].  y ([n, hidden] of `dtype`, with float32 w_post [hidden] and optional float32 ls [hidden]),
// first (float32 [n, hidden]), vec (float32 [hidden]) and h ([n, hidden] of `dtype`; with float32 w_next it is the normed
// stream, without it the stream itself) may each be null.  branch_scale multiplies the normed branch before it is added.
LMSF_API int lmsf_stream_norm(float* res, const void* y, const float* w_post, const float* ls, const float* first,
                              const float* vec, void* h, const float* w_next, int n, int hidden, float eps_post,
                              float eps_next, float branch_scale, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0 || hidden > kThreads * kMaxPerThread) LMSF_REFUSE("stream_norm: width %d is outside 1..%d", hidden, kThreads * kMaxPerThread);
  if (y != nullptr && w_post == nullptr) LMSF_REFUSE("stream_norm: a branch needs the weight of its norm");
  if ((y != nullptr && !(eps_post > 0.f)) || (w_next != nullptr && !(eps_next > 0.f))) LMSF_REFUSE("stream_norm: eps must be positive");
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
  if (dtype == LMSF_F32) rc = pick_stream<float>(res, y, w_post, ls, first, vec, h, w_next, n, hidden, eps_post, eps_next, branch_scale, s);
  else if (dtype == LMSF_BF16) rc = pick_stream<bf16>(res, y, w_post, ls, first, vec, h, w_next, n, hidden, eps_post, eps_next, branch_scale, s);
  else LMSF_REFUSE("stream_norm: unknown dtype code %d", dtype);
  return rc;
}

// res (and keep, if not null): float32 [n, hidden] = norm(table[ids] * scale) * w; table: [vocab, hidden] of `dtype`.
LMSF_API int lmsf_embed_norm(float* res, float* keep, const void* table, const int* ids, const float* w, int n, int hidden,
                             int vocab, float eps, float scale, int dtype, int* error_flag, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0 || hidden > kThreads * kMaxPerThread) LMSF_REFUSE("embed_norm: width %d is outside 1..%d", hidden, kThreads * kMaxPerThread);
  if (!(eps > 0.f)) LMSF_REFUSE("embed_norm: eps must be positive");
  const int per = ceil_div(hidden, kThreads);
  cudaStream_t s = (cudaStream_t)stream;
#define LMSF_CASE(T, P)                                                                                              \
  if (per <= P) {                                                                                                    \
    embed_norm_kernel<T, P><<<n, kThreads, 0, s>>>(res, keep, (const T*)table, ids, w, hidden, vocab, eps, scale, error_flag); \
    return LMSF_LAUNCH_STATUS();                                                                                     \
  }
  if (dtype == LMSF_F32) { LMSF_CASE(float, 1) LMSF_CASE(float, 2) LMSF_CASE(float, 4) LMSF_CASE(float, 8) LMSF_CASE(float, 16) LMSF_CASE(float, 32) LMSF_CASE(float, 64) }
  else if (dtype == LMSF_BF16) { LMSF_CASE(bf16, 1) LMSF_CASE(bf16, 2) LMSF_CASE(bf16, 4) LMSF_CASE(bf16, 8) LMSF_CASE(bf16, 16) LMSF_CASE(bf16, 32) LMSF_CASE(bf16, 64) }
#undef LMSF_CASE
  LMSF_REFUSE("embed_norm: unknown dtype code %d", dtype);
}

// res: float32 [count] = x [count] of `dtype`.
LMSF_API int lmsf_stream_begin(float* res, const void* x, long long count, int dtype, void* stream) {
  using namespace lmsf;
  if (count <= 0) return 0;
  const unsigned blocks = (unsigned)((count + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) stream_begin_kernel<float><<<blocks, 256, 0, s>>>(res, (const float*)x, count);
  else if (dtype == LMSF_BF16) stream_begin_kernel<bf16><<<blocks, 256, 0, s>>>(res, (const bf16*)x, count);
  else LMSF_REFUSE("stream_begin: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// res: float32 [n, hidden]; z: float32 [n, (y2 ? 2 : 1) * hidden] with row stride ldz; b: float32 of z's width or null; y1,
// y2 (may be null), h (may be null; then w_next is not read): [n, hidden] of `dtype`.
LMSF_API int lmsf_gated_branches(float* res, const float* z, long long ldz, const float* b, const void* y1, const void* y2,
                                 void* h, const float* w_next, int n, int hidden, float eps_next, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0 || hidden > kThreads * kMaxPerThread) LMSF_REFUSE("gated_branches: width %d is outside 1..%d", hidden, kThreads * kMaxPerThread);
  if (!z || !y1 || ldz < (y2 ? 2 : 1) * (long long)hidden) LMSF_REFUSE("gated_branches: gate logits of %lld values a row for width %d", ldz, hidden);
  if (h != nullptr && (w_next == nullptr || !(eps_next > 0.f))) LMSF_REFUSE("gated_branches: the next norm needs its weight and a positive eps");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) return pick_gated<float>(res, z, ldz, b, y1, y2, h, w_next, n, hidden, eps_next, s);
  if (dtype == LMSF_BF16) return pick_gated<bf16>(res, z, ldz, b, y1, y2, h, w_next, n, hidden, eps_next, s);
  LMSF_REFUSE("gated_branches: unknown dtype code %d", dtype);
}

// out: [n, 2 * hidden] of `dtype` = [a | b], both float32 [n, hidden].
LMSF_API int lmsf_stream_concat(void* out, const float* a, const float* b, int n, int hidden, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0) LMSF_REFUSE("stream_concat: width %d", hidden);
  const long long count = 2LL * n * hidden;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("stream_concat: unknown dtype code %d", dtype);
  if (hidden % 4 == 0 && ((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) % 16 == 0) {
    const unsigned blocks4 = (unsigned)((count / 4 + 255) / 256);
    if (dtype == LMSF_F32) stream_concat4_kernel<float><<<blocks4, 256, 0, s>>>((float*)out, a, b, hidden, count / 4);
    else stream_concat4_kernel<bf16><<<blocks4, 256, 0, s>>>((bf16*)out, a, b, hidden, count / 4);
    return LMSF_LAUNCH_STATUS();
  }
  const unsigned blocks = (unsigned)((count + 255) / 256);
  if (dtype == LMSF_F32) stream_concat_kernel<float><<<blocks, 256, 0, s>>>((float*)out, a, b, hidden, count);
  else if (dtype == LMSF_BF16) stream_concat_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)out, a, b, hidden, count);
  else LMSF_REFUSE("stream_concat: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// ---- token shift ----------------------------------------------------------------------------------------------
// out[t] = h[t] + (h[t - 1] - h[t]) * mix, element by element, where h[t - 1] is the row of the token before in the same
// request as it was before this replacement: zeros for a request's first token, and for a portion's first token the row
// that the request's state slot holds (the last row of its portion before).  The block of a portion's first token reads
// the slot and then stores the portion's last row there; no other block touches that slot.  float32 inside, one block per
// token; the slot holds h's values exactly (float32 of what h stores), so a cut changes no bit.
namespace lmsf {

// the same, four values a thread and access: widths that 4 divides, aligned rows
template <typename T>
__global__ void token_shift4_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ mix,
                                    float* __restrict__ state, const int* __restrict__ positions,
                                    const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                    const int* __restrict__ state_slot, int hidden) {
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const bool starts = t == cu_q[seq];
  const bool zero = positions[t] == 0;
  const T* cur = h + (size_t)t * hidden;
  T* dst = out + (size_t)t * hidden;
  float* slot = starts ? state + (size_t)state_slot[seq] * hidden : nullptr;
  const T* last = starts ? h + (size_t)(cu_q[seq + 1] - 1) * hidden : nullptr;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float c[4], b[4] = {0.f, 0.f, 0.f, 0.f}, m[4], o[4];
    ld4(cur + i, c);
    ld4(mix + i, m);
    if (starts) {
      if (!zero) ld4(slot + i, b);
      float l[4];
      ld4(last + i, l);
      st4(slot + i, l);
    } else if (!zero) {
      ld4(cur - hidden + i, b);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = fmaf(b[k] - c[k], m[k], c[k]);
    st4(dst + i, o);
  }
}

template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ mix,
                                   float* __restrict__ state, const int* __restrict__ positions,
                                   const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                   const int* __restrict__ state_slot, int hidden) {
  const int t = blockIdx.x;
  const int seq = token_seq[t];
  const int first = cu_q[seq];
  const bool starts = t == first;
  const bool zero = positions[t] == 0;
  const T* cur = h + (size_t)t * hidden;
  T* dst = out + (size_t)t * hidden;
  if (starts) {
    float* slot = state + (size_t)state_slot[seq] * hidden;
    const T* last = h + (size_t)(cu_q[seq + 1] - 1) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float before = zero ? 0.f : slot[i];
      const float c = to_f32(cur[i]);
      slot[i] = to_f32(last[i]);
      dst[i] = from_f32<T>(fmaf(before - c, mix[i], c));
    }
  } else {
    const T* prev = cur - hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float c = to_f32(cur[i]);
      dst[i] = from_f32<T>(fmaf((zero ? 0.f : to_f32(prev[i])) - c, mix[i], c));
    }
  }
}

}  // namespace lmsf

// out, h: [n, hidden] of `dtype` (out is not h); mix: float32 [hidden]; state: float32 [slots, hidden].
LMSF_API int lmsf_token_shift(void* out, const void* h, const float* mix, float* state, const int* positions,
                              const int* token_seq, const int* cu_q, const int* state_slot, int n, int hidden, int dtype,
                              void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (hidden <= 0 || out == h) LMSF_REFUSE("token_shift: hidden=%d, and out must not be h", hidden);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = hidden >= 1024 ? 256 : 128;
  const bool f32 = dtype == LMSF_F32;
  if ((dtype == LMSF_F32 || dtype == LMSF_BF16) && hidden % 4 == 0 && (uintptr_t)mix % 16 == 0 && (uintptr_t)state % 16 == 0 &&
      ((uintptr_t)out | (uintptr_t)h) % (f32 ? 16 : 8) == 0) {
    if (f32) token_shift4_kernel<float><<<n, threads, 0, s>>>((float*)out, (const float*)h, mix, state, positions, token_seq, cu_q, state_slot, hidden);
    else token_shift4_kernel<bf16><<<n, threads, 0, s>>>((bf16*)out, (const bf16*)h, mix, state, positions, token_seq, cu_q, state_slot, hidden);
    return LMSF_LAUNCH_STATUS();
  }
  if (dtype == LMSF_F32)
    token_shift_kernel<float><<<n, threads, 0, s>>>((float*)out, (const float*)h, mix, state, positions, token_seq, cu_q, state_slot, hidden);
  else if (dtype == LMSF_BF16)
    token_shift_kernel<bf16><<<n, threads, 0, s>>>((bf16*)out, (const bf16*)h, mix, state, positions, token_seq, cu_q, state_slot, hidden);
  else LMSF_REFUSE("token_shift: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}
