// Gated activation of the feed-forward: out[t, i] = act(x[t, i]) * x[t, d + i].
// Counterpart in the reference: silu_and_mul_kernel, vllm/kernels/activation_kernels.cu:26-41
// (gelu variants :13-24, :44-51).  Here both factors are taken to float32 and the product is
// rounded once.
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_activation)

namespace lmsf {

enum { kActSilu = 0, kActGeluTanh = 1 };

__device__ __forceinline__ float act_silu(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float act_gelu_tanh(float g) {
  const float k = 0.7978845608028654f;  // sqrt(2 / pi)
  return 0.5f * g * (1.0f + tanhf(k * (g + 0.044715f * g * g * g)));
}

template <typename T, int ACT>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ in, int d, long long in_stride) {
  const T* row = in + (size_t)blockIdx.x * in_stride;
  T* o = out + (size_t)blockIdx.x * d;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    const float g = to_f32(row[i]), u = to_f32(row[d + i]);
    o[i] = from_f32<T>((ACT == kActSilu ? act_silu(g) : act_gelu_tanh(g)) * u);
  }
}

// 8 bfloat16 values per thread and pass (16-byte loads); d % 8 == 0, in_stride % 8 == 0, aligned pointers.
template <int ACT>
__global__ void gated_act_vec_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, int d, long long in_stride) {
  const bf16* row = in + (size_t)blockIdx.x * in_stride;
  bf16* o = out + (size_t)blockIdx.x * d;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < d; i += gridDim.y * blockDim.x * 8) {
    uint4 gr = *reinterpret_cast<const uint4*>(row + i), ur = *reinterpret_cast<const uint4*>(row + d + i), r;
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
    __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      r2[e] = __floats2bfloat162_rn((ACT == kActSilu ? act_silu(g.x) : act_gelu_tanh(g.x)) * u.x,
                                    (ACT == kActSilu ? act_silu(g.y) : act_gelu_tanh(g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(o + i) = r;
  }
}

// Gate and up clamped before the product: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + 1).
template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* __restrict__ in, int d, long long in_stride, float limit, float alpha) {
  const T* row = in + (size_t)blockIdx.x * in_stride;
  T* o = out + (size_t)blockIdx.x * d;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    const float g = fminf(to_f32(row[i]), limit);
    const float u = fminf(fmaxf(to_f32(row[d + i]), -limit), limit);
    o[i] = from_f32<T>((g / (1.0f + expf(-alpha * g))) * (u + 1.0f));
  }
}

// 8 bfloat16 values per thread and pass (16-byte loads); d % 8 == 0, in_stride % 8 == 0, aligned pointers.
__global__ void clamped_glu_vec_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, int d, long long in_stride, float limit,
                                       float alpha) {
  const bf16* row = in + (size_t)blockIdx.x * in_stride;
  bf16* o = out + (size_t)blockIdx.x * d;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < d; i += gridDim.y * blockDim.x * 8) {
    uint4 gr = *reinterpret_cast<const uint4*>(row + i), ur = *reinterpret_cast<const uint4*>(row + d + i), r;
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gr);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&ur);
    __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
      const float gx = fminf(g.x, limit), gy = fminf(g.y, limit);
      const float ux = fminf(fmaxf(u.x, -limit), limit), uy = fminf(fmaxf(u.y, -limit), limit);
      r2[e] = __floats2bfloat162_rn((gx / (1.0f + expf(-alpha * gx))) * (ux + 1.0f), (gy / (1.0f + expf(-alpha * gy))) * (uy + 1.0f));
    }
    *reinterpret_cast<uint4*>(o + i) = r;
  }
}

// out[t, i] = gelu_tanh(a[t, i]) * table[ids[t], offset + i]: a gate that a per-token vector from a table passes.
template <typename T>
__global__ void gelu_mul_gather_kernel(T* __restrict__ out, const T* __restrict__ a, long long a_stride, const T* __restrict__ table,
                                       long long table_stride, int offset, const int* __restrict__ ids, int vocab, int d,
                                       int* __restrict__ error_flag) {
  const int t = blockIdx.x, id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
  const T* e = table + (size_t)(ok ? id : 0) * table_stride + offset;
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    out[(size_t)t * d + i] = from_f32<T>(ok ? act_gelu_tanh(to_f32(a[(size_t)t * a_stride + i])) * to_f32(e[i]) : 0.f);
}

// x <- cap * tanh(x * scale / cap) (cap 0: x * scale), float32 in place: logits scaled and capped smoothly.
__global__ void scale_softcap_kernel(float* __restrict__ x, long long n, float scale, float cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { const float z = x[i] * scale; x[i] = cap > 0.f ? cap * tanhf(z / cap) : z; }
}

// x[t, i] += bias[i], the sum taken in float32 and rounded once to x's type.
template <typename T>
__global__ void bias_add_kernel(T* __restrict__ x, const T* __restrict__ bias, int d, long long stride) {
  T* row = x + (size_t)blockIdx.x * stride;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x)
    row[i] = from_f32<T>(to_f32(row[i]) + to_f32(bias[i]));
}

}  // namespace lmsf

// x: [n, d] with `stride` elements between rows, bias: [d] of x's type; in place.  The projections of a model whose
// config.json asks for biases (attention_bias, mlp_bias) add them with this kernel after the product; the
// reference's linear layer does the same as a separate broadcast add (core/src/model_executor/layers/linear.rs:100-104).
LMSF_API int lmsf_bias_add(void* x, const void* bias, int n, int d, long long stride, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || stride < d) LMSF_REFUSE("bias_add: d=%d, stride=%lld", d, stride);
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("bias_add: unknown dtype code %d", dtype);
  int gy = ceil_div(d, 256 * 4);
  if (gy > 64) gy = 64;
  dim3 grid(n, gy);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) bias_add_kernel<float><<<grid, 256, 0, s>>>((float*)x, (const float*)bias, d, stride);
  else bias_add_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)x, (const bf16*)bias, d, stride);
  return LMSF_LAUNCH_STATUS();
}

// in: [n, 2 * d] with `in_stride` elements between rows (gate first, up second); out: [n, d].
LMSF_API int lmsf_gated_act(void* out, const void* in, int n, int d, long long in_stride, int act, int dtype,
                            void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || in_stride < 2LL * d) LMSF_REFUSE("gated_act: d=%d, in_stride=%lld", d, in_stride);
  if (act != kActSilu && act != kActGeluTanh) LMSF_REFUSE("gated_act: unknown activation code %d", act);
  if (dtype != LMSF_F32 && dtype != LMSF_BF16) LMSF_REFUSE("gated_act: unknown dtype code %d", dtype);
  const int threads = 256;
  int gy = ceil_div(d, threads * 4);
  if (gy > 64) gy = 64;
  dim3 grid(n, gy);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_BF16 && d % 8 == 0 && in_stride % 8 == 0 && ((uintptr_t)out | (uintptr_t)in) % 16 == 0) {
    int vy = ceil_div(d, 256 * 8);
    if (vy > 64) vy = 64;
    dim3 vgrid(n, vy);
    if (act == kActSilu) gated_act_vec_kernel<kActSilu><<<vgrid, 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride);
    else gated_act_vec_kernel<kActGeluTanh><<<vgrid, 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride);
    return LMSF_LAUNCH_STATUS();
  }
#define LMSF_GA(T, A) gated_act_kernel<T, A><<<grid, threads, 0, s>>>((T*)out, (const T*)in, d, in_stride)
  if (dtype == LMSF_F32) { if (act == kActSilu) LMSF_GA(float, kActSilu); else LMSF_GA(float, kActGeluTanh); }
  else { if (act == kActSilu) LMSF_GA(bf16, kActSilu); else LMSF_GA(bf16, kActGeluTanh); }
#undef LMSF_GA
  return LMSF_LAUNCH_STATUS();
}

// in: [n, 2 * d] (gate first, up second); out: [n, d]; see clamped_glu_kernel.
LMSF_API int lmsf_clamped_glu(void* out, const void* in, int n, int d, long long in_stride, float limit, float alpha, int dtype,
                              void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || in_stride < 2LL * d || !(limit > 0.f)) LMSF_REFUSE("clamped_glu: d=%d, in_stride=%lld, limit=%g", d, in_stride, limit);
  int gy = ceil_div(d, 256 * 4);
  if (gy > 64) gy = 64;
  dim3 grid(n, gy);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_BF16 && d % 8 == 0 && in_stride % 8 == 0 && ((uintptr_t)out | (uintptr_t)in) % 16 == 0) {
    int vy = ceil_div(d, 256 * 8);
    if (vy > 64) vy = 64;
    clamped_glu_vec_kernel<<<dim3(n, vy), 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride, limit, alpha);
    return LMSF_LAUNCH_STATUS();
  }
  if (dtype == LMSF_F32) clamped_glu_kernel<float><<<grid, 256, 0, s>>>((float*)out, (const float*)in, d, in_stride, limit, alpha);
  else if (dtype == LMSF_BF16) clamped_glu_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride, limit, alpha);
  else LMSF_REFUSE("clamped_glu: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// out: [n, d] contiguous; a: [n, d] with a_stride; table: [vocab, table_stride] of which columns offset .. offset + d are taken.
LMSF_API int lmsf_gelu_mul_gather(void* out, const void* a, long long a_stride, const void* table, long long table_stride,
                                  int offset, const int* ids, int vocab, int n, int d, int dtype, int* error_flag, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || offset < 0 || offset + d > table_stride) LMSF_REFUSE("gelu_mul_gather: columns %d..%d of %lld", offset, offset + d, table_stride);
  const int threads = d >= 256 ? 256 : (d >= 64 ? 64 : 32);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32)
    gelu_mul_gather_kernel<float><<<n, threads, 0, s>>>((float*)out, (const float*)a, a_stride, (const float*)table, table_stride, offset, ids, vocab, d, error_flag);
  else if (dtype == LMSF_BF16)
    gelu_mul_gather_kernel<bf16><<<n, threads, 0, s>>>((bf16*)out, (const bf16*)a, a_stride, (const bf16*)table, table_stride, offset, ids, vocab, d, error_flag);
  else LMSF_REFUSE("gelu_mul_gather: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_scale_softcap(float* x, long long n, float scale, float cap, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  scale_softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, scale, cap);
  return LMSF_LAUNCH_STATUS();
}

// ---- polynomial activation with a norm per power ------------------------------------------------------------------
// out[t, i] = a N1(z)_i + b N2(z^2)_i + c N3(z^3)_i + e, where the powers are taken element by element and N divides a
// token's row of d values by its root mean square, x / sqrt(mean(x^2) + eps): the three sums (of z^2, z^4, z^6) and the
// factors are float32.  One block per token; the row is read twice (the second time from L1/L2).  coef: float32 [4] =
// (a, b, c, e) on the device.
namespace lmsf {

template <typename T>
__global__ void __launch_bounds__(256) poly_norm_kernel(T* __restrict__ out, const T* __restrict__ in, int d, long long in_stride,
                                                        const float* __restrict__ coef, float eps) {
  __shared__ float scratch[3][33];
  const T* row = in + (size_t)blockIdx.x * in_stride;
  T* o = out + (size_t)blockIdx.x * d;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float z = to_f32(row[i]), z2 = z * z;
    s2 += z2;
    s4 = fmaf(z2, z2, s4);
    s6 = fmaf(z2 * z2, z2, s6);
  }
  s2 = block_sum(s2, scratch[0]);
  s4 = block_sum(s4, scratch[1]);
  s6 = block_sum(s6, scratch[2]);
  const float inv = 1.0f / (float)d;
  const float f1 = coef[0] / sqrtf(fmaf(s2, inv, eps)), f2 = coef[1] / sqrtf(fmaf(s4, inv, eps)),
              f3 = coef[2] / sqrtf(fmaf(s6, inv, eps)), e = coef[3];
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float z = to_f32(row[i]), z2 = z * z;
    o[i] = from_f32<T>(fmaf(f1, z, fmaf(f2, z2, fmaf(f3, z2 * z, e))));
  }
}

// the same, four values a thread and access: d % 4 == 0, aligned rows
template <typename T>
__global__ void __launch_bounds__(512) poly_norm4_kernel(T* __restrict__ out, const T* __restrict__ in, int d, long long in_stride,
                                                         const float* __restrict__ coef, float eps) {
  __shared__ float scratch[3][33];
  const T* row = in + (size_t)blockIdx.x * in_stride;
  T* o = out + (size_t)blockIdx.x * d;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    float z[4];
    ld4(row + i, z);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float z2 = z[k] * z[k];
      s2 += z2;
      s4 = fmaf(z2, z2, s4);
      s6 = fmaf(z2 * z2, z2, s6);
    }
  }
  s2 = block_sum(s2, scratch[0]);
  s4 = block_sum(s4, scratch[1]);
  s6 = block_sum(s6, scratch[2]);
  const float inv = 1.0f / (float)d;
  const float f1 = coef[0] / sqrtf(fmaf(s2, inv, eps)), f2 = coef[1] / sqrtf(fmaf(s4, inv, eps)),
              f3 = coef[2] / sqrtf(fmaf(s6, inv, eps)), e = coef[3];
  for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
    float z[4], r[4];
    ld4(row + i, z);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float z2 = z[k] * z[k];
      r[k] = fmaf(f1, z[k], fmaf(f2, z2, fmaf(f3, z2 * z[k], e)));
    }
    st4(o + i, r);
  }
}

}  // namespace lmsf

// in: [n, d] with in_stride elements between rows; out: [n, d] contiguous; coef: float32 [4] on the device.
LMSF_API int lmsf_poly_norm(void* out, const void* in, int n, int d, long long in_stride, const float* coef, float eps,
                            int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (d <= 0 || in_stride < d || !(eps > 0.f)) LMSF_REFUSE("poly_norm: d=%d, in_stride=%lld, eps=%g", d, in_stride, eps);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = d >= 4096 ? 512 : 256;
  if (dtype == LMSF_F32 && rows_take4<float>(in, d, in_stride) && (uintptr_t)out % 16 == 0) {
    poly_norm4_kernel<float><<<n, threads, 0, s>>>((float*)out, (const float*)in, d, in_stride, coef, eps);
    return LMSF_LAUNCH_STATUS();
  }
  if (dtype == LMSF_BF16 && rows_take4<bf16>(in, d, in_stride) && (uintptr_t)out % 8 == 0) {
    poly_norm4_kernel<bf16><<<n, threads, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride, coef, eps);
    return LMSF_LAUNCH_STATUS();
  }
  if (dtype == LMSF_F32) poly_norm_kernel<float><<<n, 256, 0, s>>>((float*)out, (const float*)in, d, in_stride, coef, eps);
  else if (dtype == LMSF_BF16) poly_norm_kernel<bf16><<<n, 256, 0, s>>>((bf16*)out, (const bf16*)in, d, in_stride, coef, eps);
  else LMSF_REFUSE("poly_norm: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}
