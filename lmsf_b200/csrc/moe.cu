// Routed experts: every token goes to its `top` experts of `experts` small feed-forward layers.
//
//   moe_topk      router logits (float32) + bias -> the top experts of each token and their weights: a softmax over
//                 the chosen logits only (ties go to the lower expert number)
//   moe_align     (token, choice) pairs sorted by expert: per-expert offsets, the row of every pair, and the list of
//                 row tiles that the products walk; made on the device, so a step never waits for the host and its
//                 launches have the same shape whatever the routing is
//   moe_grouped   one launch for all experts: tile (expert e, rows r0..r0+rows) computes rows x W_e^T; rows are
//                 gathered through the pair list on the way in (up projection) or are already in pair order (down
//                 projection); the activation (square of relu) is applied in the epilogue of the up projection.
//                 float32 accumulation, one thread per output element in ascending k: a row's result does not
//                 depend on which rows share its tile
//   moe_combine   out[t] = sum_j weight[t, j] * down[pair(t, j)]  (+ sigmoid(gate[t]) * shared[t])
#include "common.cuh"

LMSF_DEFINE_LAST_ERROR(lmsf_moe)

namespace lmsf {

constexpr int kMaxExperts = 1024;
constexpr int BM = 64, BN = 64, BK = 16;

// One warp per token.  logits: [n, ld] float32 (the first `experts` columns).
__global__ void moe_topk_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias, int n,
                                int experts, int top, int* __restrict__ ids, float* __restrict__ wts) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= n) return;
  float z[kMaxExperts / 32];
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    const int e = i * 32 + lane;
    z[i] = e < experts ? logits[(size_t)t * ld + e] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float m0 = 0.f, denom = 0.f;
  float mine = 0.f;        // lane j keeps the j-th chosen logit
  int mine_id = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      const int e = i * 32 + lane;
      if (z[i] > best) { best = z[i]; arg = e; }     // ascending e per lane: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (j == 0) m0 = best;
    denom += expf(best - m0);
    if (j == lane) { mine = best; mine_id = arg; }
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i)
      if (i * 32 + lane == arg) z[i] = -INFINITY;
  }
  if (lane < top) {
    ids[(size_t)t * top + lane] = mine_id;
    wts[(size_t)t * top + lane] = expf(mine - m0) / denom;
  }
}

// Routing by sigmoid scores inside the best groups of neighbouring experts.  s = sigmoid(logit); the choice is made by
// s + correction; a group's score is the sum of its two largest choice scores (of its one, if it has one expert); only
// experts of the `keep` best groups can be chosen; the weights are the chosen experts' s (times `weight_scale`), not
// renormalised.  Ties go to the lower number.  One warp per token; shared memory: per warp experts + n_groups floats.
__global__ void moe_topk_sigmoid_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction,
                                        int n, int experts, int top, int n_groups, int keep, float weight_scale,
                                        int* __restrict__ ids, float* __restrict__ wts) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n) return;
  float* c = sm + (size_t)warp * (experts + n_groups);
  float* gs = c + experts;
  for (int e = lane; e < experts; e += 32) {
    const float z = logits[(size_t)t * ld + e];
    c[e] = 1.0f / (1.0f + expf(-z)) + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int size = experts / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;             // the largest and the second
      for (int i = 0; i < size; ++i) {
        const float v = c[g * size + i];
        if (v > a) { b = a; a = v; } else if (v > b) b = v;
      }
      gs[g] = size > 1 ? a + b : a;
    }
    __syncwarp();
    for (int j = 0; j < keep; ++j) {                   // the kept groups are marked by +infinity
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32)
        if (gs[g] != INFINITY && gs[g] > best) { best = gs[g]; arg = g; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
      }
      __syncwarp();
      if (lane == 0 && arg != 0x7fffffff) gs[arg] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (gs[e / size] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  int mine_id = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < experts; e += 32)
      if (c[e] > best) { best = c[e]; arg = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) arg = 0;                   // fewer allowed experts than choices: a configuration fault
    if (j == lane) mine_id = arg;
    __syncwarp();
    if (lane == 0) c[arg] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    ids[(size_t)t * top + lane] = mine_id;
    wts[(size_t)t * top + lane] = weight_scale / (1.0f + expf(-logits[(size_t)t * ld + mine_id]));
  }
}

// Routing by a softmax over ALL `outputs` router logits (more outputs than experts: the outputs behind the experts stand for
// experts that return their input).  s = softmax(logits); the choice is made by s + correction; the weights are the chosen
// outputs' s times `weight_scale`, not renormalised.  Ties go to the lower number.  One warp per token; shared memory: per
// warp 2 * outputs floats.
__global__ void moe_topk_softmax_all_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction,
                                            int n, int outputs, int top, float weight_scale, int* __restrict__ ids,
                                            float* __restrict__ wts) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n) return;
  float* sc = sm + (size_t)warp * 2 * outputs;    // the scores
  float* c = sc + outputs;                        // the choice scores
  float m = -INFINITY;
  for (int e = lane; e < outputs; e += 32) m = fmaxf(m, logits[(size_t)t * ld + e]);
  m = warp_max(m);
  float den = 0.f;
  for (int e = lane; e < outputs; e += 32) {
    const float p = expf(logits[(size_t)t * ld + e] - m);
    sc[e] = p;
    den += p;
  }
  den = warp_sum(den);
  for (int e = lane; e < outputs; e += 32) {
    const float v = sc[e] / den;
    sc[e] = v;
    c[e] = v + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  int mine_id = 0;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32)
      if (c[e] > best) { best = c[e]; arg = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg == 0x7fffffff) arg = 0;                   // nothing left to choose (NaN logits): a fault of the input
    if (j == lane) mine_id = arg;
    __syncwarp();
    if (lane == 0) c[arg] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    ids[(size_t)t * top + lane] = mine_id;
    wts[(size_t)t * top + lane] = sc[mine_id] * weight_scale;
  }
}

// One block.  ids: [pairs]; offsets: [experts + 1]; pair_row: [pairs] row of each pair in expert order;
// row_token: [pairs] token of each row; tiles: [max_tiles][4] = (expert, first row, rows, 0); meta[0] = number of tiles.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ ids, int pairs, int top, int experts,
                                                         int tile_rows, int* __restrict__ offsets, int* __restrict__ pair_row,
                                                         int* __restrict__ row_token, int* __restrict__ tiles,
                                                         int max_tiles, int* __restrict__ meta) {
  __shared__ int count[kMaxExperts];
  __shared__ int start[kMaxExperts + 1];
  __shared__ int tile_start[kMaxExperts + 1];
  __shared__ int cursor[kMaxExperts];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0, ts = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = s; tile_start[e] = ts;
      s += count[e];
      ts += (count[e] + tile_rows - 1) / tile_rows;
    }
    start[experts] = s; tile_start[experts] = ts;
    meta[0] = min(ts, max_tiles);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int ti = tile_start[e];
    for (int r = 0; r < count[e] && ti < max_tiles; r += tile_rows, ++ti) {
      tiles[4 * ti + 0] = e; tiles[4 * ti + 1] = start[e] + r; tiles[4 * ti + 2] = min(tile_rows, count[e] - r); tiles[4 * ti + 3] = 0;
    }
  }
  // Rows inside an expert's segment are dealt in arrival order of the atomics; a row's result does not depend on its
  // place (each output element is one thread's sum in ascending k), so the order is free.
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < experts) {
      const int row = start[e] + atomicAdd(&cursor[e], 1);
      pair_row[p] = row;
      row_token[row] = p / top;
    } else {
      pair_row[p] = -1;
    }
  }
}

template <int ACT> __device__ __forceinline__ float epilogue(float v) {
  if (ACT == 1) { const float r = fmaxf(v, 0.f); return r * r; }
  return v;
}

// C[row, :] = act(A[src(row), :] W_e^T) for the rows of one tile.  A: [*, K] (row stride lda); src(row) = gather[row]
// when `gather` is given, else row.  W: [experts][N][K].  C: [pairs, N] (row stride ldc).
template <typename TA, typename TC, int ACT>
__global__ void __launch_bounds__(256) moe_grouped_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TA* __restrict__ W,
                                                          const int* __restrict__ gather, const int* __restrict__ tiles,
                                                          const int* __restrict__ meta, int N, int K, long long lda,
                                                          long long ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int src[BM];
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int e = tiles[4 * tile], row0 = tiles[4 * tile + 1], rows = tiles[4 * tile + 2];
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BN;
  const TA* We = W + (size_t)e * N * K;
  if (tid < BM) src[tid] = tid < rows ? (gather ? gather[row0 + tid] : row0 + tid) : -1;
  __syncthreads();
  const int tx = tid % 16, ty = tid / 16;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int arow = src[lr];
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + lk + q;
      const int n = n0 + lr;
      As[lk + q][lr] = (arow >= 0 && k < K) ? to_f32(A[(size_t)arow * lda + k]) : 0.f;
      Ws[lk + q][lr] = (n < N && k < K) ? to_f32(We[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = ty * 4 + i;
    if (m >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)(row0 + m) * ldc + n] = from_f32<TC>(epilogue<ACT>(acc[i][j]));
    }
  }
}

// out[t, d] = sum_j wts[t, j] * down[pair_row[t, j], d] + sigmoid(gate[t]) * shared[t, d]; the sum runs in the order
// of the choices, float32.  gate: float32, one value per token at gate[t * gate_stride]; shared and gate may be null.
// wts null: every weight is 1 (the weights went into the experts already).
// ids with x (both or neither): a choice whose number is `experts` or more is an expert that returns its input, x[t].
template <typename TD, typename TS, typename TO>
__global__ void moe_combine_kernel(TO* __restrict__ out, const TD* __restrict__ down, const int* __restrict__ pair_row,
                                   const float* __restrict__ wts, int top, const TS* __restrict__ shared,
                                   const float* __restrict__ gate, long long gate_stride, int width,
                                   const int* __restrict__ ids, int experts, const TS* __restrict__ x) {
  const int t = blockIdx.x;
  const float g = (shared && gate) ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride])) : 1.0f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const int row = pair_row[(size_t)t * top + j];
      if (row >= 0) acc = fmaf(wts ? wts[(size_t)t * top + j] : 1.0f, to_f32(down[(size_t)row * width + d]), acc);
      else if (ids && ids[(size_t)t * top + j] >= experts)
        acc = fmaf(wts ? wts[(size_t)t * top + j] : 1.0f, to_f32(x[(size_t)t * width + d]), acc);
    }
    if (shared) acc = fmaf(g, to_f32(shared[(size_t)t * width + d]), acc);
    out[(size_t)t * width + d] = from_f32<TO>(acc);
  }
}

// Gated experts whose routing weight multiplies what the expert READS: expert(w h) = (act(w g) * (w u)) W_down^T with
// g = W_gate h and u = W_up h, because both products are linear in h.  The weight is applied here, in float32, to the
// products of the unweighted token: y[r, 0:F] = g, y[r, F:2F] = u for row r of the pair (token, choice); out[r, i] =
// act(w g_i) * (w u_i).  ACT 0: silu, 1: the tanh form of gelu.  One block per pair; weights null: w = 1.
template <typename T, int ACT>
__global__ void moe_weighted_glu_kernel(T* __restrict__ out, const T* __restrict__ y, const int* __restrict__ pair_row,
                                        const float* __restrict__ wts, int F) {
  const int pair = blockIdx.x;
  const int row = pair_row[pair];
  if (row < 0) return;
  const float w = wts ? wts[pair] : 1.0f;
  const T* yr = y + (size_t)row * 2 * F;
  for (int i = threadIdx.x; i < F; i += blockDim.x) {
    const float g = w * to_f32(yr[i]), u = w * to_f32(yr[F + i]);
    float a;
    if (ACT == 0) a = g / (1.0f + expf(-g));
    else a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    out[(size_t)row * F + i] = from_f32<T>(a * u);
  }
}

// the same on bfloat16 rows of a multiple of 8 values, 16 bytes a load
template <int ACT>
__global__ void moe_weighted_glu8_kernel(bf16* __restrict__ out, const bf16* __restrict__ y, const int* __restrict__ pair_row,
                                         const float* __restrict__ wts, int F) {
  const int pair = blockIdx.x;
  const int row = pair_row[pair];
  if (row < 0) return;
  const float w = wts ? wts[pair] : 1.0f;
  const uint4* yr = reinterpret_cast<const uint4*>(y + (size_t)row * 2 * F);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * F);
  const int n8 = F / 8;
  for (int i = threadIdx.x; i < n8; i += blockDim.x) {
    const uint4 gv = yr[i], uv = yr[n8 + i];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gf = __bfloat1622float2(g2[k]), uf = __bfloat1622float2(u2[k]);
      float r[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float g = w * (e ? gf.y : gf.x), u = w * (e ? uf.y : uf.x);
        float a;
        if (ACT == 0) a = g / (1.0f + expf(-g));
        else a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        r[e] = a * u;
      }
      o2[k] = __floats2bfloat162_rn(r[0], r[1]);
    }
    dst[i] = ov;
  }
}

template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { const float r = fmaxf(to_f32(x[i]), 0.f); x[i] = from_f32<T>(r * r); }
}

}  // namespace lmsf

LMSF_API int lmsf_moe_topk(const float* logits, long long ld, const float* bias, int n, int experts, int top, int* ids,
                           float* wts, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (experts <= 0 || experts > kMaxExperts || top <= 0 || top > experts || top > 32)
    LMSF_REFUSE("moe: %d choices of %d experts (up to %d experts, up to 32 choices)", top, experts, kMaxExperts);
  moe_topk_kernel<<<ceil_div(n, 4), 128, 0, (cudaStream_t)stream>>>(logits, ld, bias, n, experts, top, ids, wts);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_moe_topk_sigmoid(const float* logits, long long ld, const float* correction, int n, int experts, int top,
                                   int n_groups, int keep, float weight_scale, int* ids, float* wts, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (experts <= 0 || experts > kMaxExperts || top <= 0 || top > experts || top > 32)
    LMSF_REFUSE("moe: %d choices of %d experts (up to %d experts, up to 32 choices)", top, experts, kMaxExperts);
  if (n_groups < 1 || experts % n_groups || keep < 1 || keep > n_groups || (long long)keep * (experts / n_groups) < top)
    LMSF_REFUSE("moe: %d experts in %d groups of which %d are kept cannot give %d choices", experts, n_groups, keep, top);
  const size_t smem = (size_t)4 * (experts + n_groups) * sizeof(float);
  moe_topk_sigmoid_kernel<<<ceil_div(n, 4), 128, smem, (cudaStream_t)stream>>>(logits, ld, correction, n, experts, top, n_groups,
                                                                             keep, weight_scale, ids, wts);
  return LMSF_LAUNCH_STATUS();
}

// logits: float32 [n, ld] of which the first `outputs` columns are the router's; correction: float32 [outputs] or null.
LMSF_API int lmsf_moe_topk_softmax_all(const float* logits, long long ld, const float* correction, int n, int outputs, int top,
                                       float weight_scale, int* ids, float* wts, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (outputs <= 0 || outputs > kMaxExperts || top <= 0 || top > outputs || top > 32)
    LMSF_REFUSE("moe: %d choices of %d router outputs (up to %d outputs, up to 32 choices)", top, outputs, kMaxExperts);
  const size_t smem = (size_t)4 * 2 * outputs * sizeof(float);
  moe_topk_softmax_all_kernel<<<ceil_div(n, 4), 128, smem, (cudaStream_t)stream>>>(logits, ld, correction, n, outputs, top,
                                                                                 weight_scale, ids, wts);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_moe_tile_rows() { return lmsf::BM; }

// tile_rows: rows per tile of the product that will walk the list (lmsf_moe_tile_rows() for the kernel of this file).
LMSF_API int lmsf_moe_align(const int* ids, int pairs, int top, int experts, int tile_rows, int* offsets, int* pair_row,
                            int* row_token, int* tiles, int max_tiles, int* meta, void* stream) {
  using namespace lmsf;
  if (pairs <= 0) return 0;
  if (experts <= 0 || experts > kMaxExperts || top <= 0 || tile_rows <= 0) LMSF_REFUSE("moe: experts=%d top=%d", experts, top);
  if (max_tiles < pairs / tile_rows + min(experts, pairs)) LMSF_REFUSE("moe: room for %d tiles is too little", max_tiles);
  moe_align_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, pairs, top, experts, tile_rows, offsets, pair_row, row_token, tiles,
                                                         max_tiles, meta);
  return LMSF_LAUNCH_STATUS();
}

// C: [pairs, N] of out_dtype; A: rows of K values of in_dtype; W: [experts, N, K] of in_dtype; act: 0 none, 1 relu squared.
LMSF_API int lmsf_moe_grouped(void* C, const void* A, const void* W, const int* gather, const int* tiles, const int* meta,
                              int max_tiles, int N, int K, long long lda, long long ldc, int act, int in_dtype, int out_dtype,
                              void* stream) {
  using namespace lmsf;
  if (max_tiles <= 0 || N <= 0) return 0;
  // (the tile list must have been made with tile_rows = lmsf_moe_tile_rows())
  if (K <= 0 || lda < K || ldc < N) LMSF_REFUSE("moe: N=%d K=%d lda=%lld ldc=%lld", N, K, lda, ldc);
  if (max_tiles > 65535) LMSF_REFUSE("moe: more than 65535 row tiles in one launch");
  if (act != 0 && act != 1) LMSF_REFUSE("moe: unknown activation code %d", act);
  dim3 grid(ceil_div(N, BN), max_tiles);
  cudaStream_t s = (cudaStream_t)stream;
#define LMSF_GO(TA, TC, ACT) moe_grouped_kernel<TA, TC, ACT><<<grid, 256, 0, s>>>((TC*)C, (const TA*)A, (const TA*)W, gather, tiles, meta, N, K, lda, ldc)
  if (in_dtype == LMSF_F32 && out_dtype == LMSF_F32) { if (act) LMSF_GO(float, float, 1); else LMSF_GO(float, float, 0); }
  else if (in_dtype == LMSF_BF16 && out_dtype == LMSF_BF16) { if (act) LMSF_GO(bf16, bf16, 1); else LMSF_GO(bf16, bf16, 0); }
  else if (in_dtype == LMSF_BF16 && out_dtype == LMSF_F32) { if (act) LMSF_GO(bf16, float, 1); else LMSF_GO(bf16, float, 0); }
  else LMSF_REFUSE("moe: unsupported dtype pair (in %d, out %d)", in_dtype, out_dtype);
#undef LMSF_GO
  return LMSF_LAUNCH_STATUS();
}

// out: [n, width] of out_dtype; down: [pairs, width] float32; shared: [n, width] of out_dtype or null.
// ids ([n, top]) and x ([n, width] of out_dtype), both or neither: choices numbered `experts` and up return the token's x.
LMSF_API int lmsf_moe_combine_identity(void* out, const float* down, const int* pair_row, const float* wts, int top,
                                       const void* shared, const float* gate, long long gate_stride, int n, int width,
                                       int out_dtype, const int* ids, int experts, const void* x, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  if (width <= 0 || top <= 0) LMSF_REFUSE("moe: width=%d top=%d", width, top);
  if ((ids == nullptr) != (x == nullptr)) LMSF_REFUSE("moe: experts that return their input need the choices and the input");
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == LMSF_F32)
    moe_combine_kernel<float, float, float><<<n, 256, 0, s>>>((float*)out, down, pair_row, wts, top, (const float*)shared, gate, gate_stride, width, ids, experts, (const float*)x);
  else if (out_dtype == LMSF_BF16)
    moe_combine_kernel<float, bf16, bf16><<<n, 256, 0, s>>>((bf16*)out, down, pair_row, wts, top, (const bf16*)shared, gate, gate_stride, width, ids, experts, (const bf16*)x);
  else LMSF_REFUSE("moe: unknown dtype code %d", out_dtype);
  return LMSF_LAUNCH_STATUS();
}

LMSF_API int lmsf_moe_combine(void* out, const float* down, const int* pair_row, const float* wts, int top, const void* shared,
                              const float* gate, long long gate_stride, int n, int width, int out_dtype, void* stream) {
  return lmsf_moe_combine_identity(out, down, pair_row, wts, top, shared, gate, gate_stride, n, width, out_dtype, nullptr, 0,
                                   nullptr, stream);
}

LMSF_API int lmsf_relu2(void* x, long long n, int dtype, void* stream) {
  using namespace lmsf;
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == LMSF_F32) relu2_kernel<float><<<blocks, 256, 0, s>>>((float*)x, n);
  else if (dtype == LMSF_BF16) relu2_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)x, n);
  else LMSF_REFUSE("relu2: unknown dtype code %d", dtype);
  return LMSF_LAUNCH_STATUS();
}

// out: [pairs, F]; y: [pairs, 2 F] (gate | up) of `dtype`, rows in expert order; pair_row: [pairs] row of every (token,
// choice) pair; wts: float32 [pairs] or null.  act: 0 silu, 1 gelu (tanh form).
LMSF_API int lmsf_moe_weighted_glu(void* out, const void* y, const int* pair_row, const float* wts, int pairs, int F, int act,
                                   int dtype, void* stream) {
  using namespace lmsf;
  if (pairs <= 0) return 0;
  if (F <= 0 || (act != 0 && act != 1)) LMSF_REFUSE("moe: F=%d act=%d", F, act);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = F >= 256 ? 256 : 128;
#define LMSF_GO(T, A) moe_weighted_glu_kernel<T, A><<<pairs, threads, 0, s>>>((T*)out, (const T*)y, pair_row, wts, F)
  if (dtype == LMSF_F32) { if (act) LMSF_GO(float, 1); else LMSF_GO(float, 0); }
  else if (dtype == LMSF_BF16) {
    if (F % 8 == 0 && ((uintptr_t)out | (uintptr_t)y) % 16 == 0) {
      const int t8 = F >= 2048 ? 256 : 128;
      if (act) moe_weighted_glu8_kernel<1><<<pairs, t8, 0, s>>>((bf16*)out, (const bf16*)y, pair_row, wts, F);
      else moe_weighted_glu8_kernel<0><<<pairs, t8, 0, s>>>((bf16*)out, (const bf16*)y, pair_row, wts, F);
    } else if (act) LMSF_GO(bf16, 1); else LMSF_GO(bf16, 0);
  }
  else LMSF_REFUSE("moe: unknown dtype code %d", dtype);
#undef LMSF_GO
  return LMSF_LAUNCH_STATUS();
}
