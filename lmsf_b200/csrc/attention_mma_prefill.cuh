// Prefill half of attention_mma.cu (included there: it shares HD, the stages and the fragment helpers).
#pragma once

namespace lmsf {
namespace fa {

struct PrefillArgs {
  const bf16* q; long long q_stride;         // [n_tokens][n_q_heads * HD]
  bf16* out; long long out_stride;
  PagedKV kv;
  const int* block_table; int max_blocks;
  const int* tile_seq;                       // [grid.x] request of each 64-token query tile
  const int* tile_q0;                        // [grid.x] first token of the tile, counted inside the request's portion
  const int* cu_q; const int* ctx_len;
  float scale; int window;
  int n_q_heads, group;
  ScoreExtras x;
};

// One block: 64 query tokens (16 per warp) of one head.  Query i of a portion of n tokens of a request
// that holds ctx keys after this step sits at position ctx - n + i and sees keys lo..position.
__global__ void __launch_bounds__(kThreads) prefill_kernel(PrefillArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  // blocks start in the order (all heads of tile 0, all heads of tile 1, ...); the caller lists the tiles that
  // see the most keys first
  const int seq = a.tile_seq[blockIdx.y], q0 = a.tile_q0[blockIdx.y];
  const int head = blockIdx.x, kvh = head / a.group;
  const int tok0 = a.cu_q[seq], n = a.cu_q[seq + 1] - tok0, ctx = a.ctx_len[seq];
  const int start = ctx - n;                                    // position of the portion's first token
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g4 = lane >> 2, t4 = lane & 3;
  const int rows_valid = min(kTileKeys, n - q0);                // query rows of this tile that exist
  const int hi = start + q0 + rows_valid;                       // keys < hi are visible to the tile's last row
  const int lo = first_seen(start + q0, a.window, a.x.chunk);      // the first row's: no row of the tile sees an older key
  const int* table = a.block_table + (size_t)seq * a.max_blocks;

  // this thread's two rows
  int pos[2], row_lo[2];
  bool row_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g4 + h * 8;
    row_ok[h] = r < rows_valid;
    pos[h] = start + q0 + min(r, rows_valid - 1);
    row_lo[h] = first_seen(pos[h], a.window, a.x.chunk);
  }
  const bool biased = a.x.r1 != nullptr;
  const float r1 = biased ? a.x.r1[head] : 0.f, r2 = biased ? a.x.r2[head] : 0.f;
  const int keep = a.x.keep_first;                               // keys below it are seen behind the window too
  const bool sig = a.x.sigmoid != 0;
  const float hb2 = a.x.head_bias ? a.x.head_bias[head] * kLog2e : 0.f;
  const int warp_last_pos = start + q0 + min(warp * 16 + 15, rows_valid - 1);
  const int warp_first_pos = start + q0 + min(warp * 16, rows_valid - 1);
  const int warp_lo = first_seen(warp_first_pos, a.window, a.x.chunk);

  uint32_t qf[kKSteps][4];
#pragma unroll
  for (int ks = 0; ks < kKSteps; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int h = r & 1, col = ks * 16 + t4 * 2 + (r >> 1) * 8;
      const int row = warp * 16 + g4 + h * 8;
      qf[ks][r] = row_ok[h] ? *reinterpret_cast<const uint32_t*>(
                                  a.q + (size_t)(tok0 + q0 + row) * a.q_stride + (size_t)head * HD + col) : 0u;
    }

  const TileRange tiles = tile_range(lo, hi, keep, kTileKeys);
  const int n_tiles = tiles.n;
  const uint32_t smem_base = smem_u32(smem);
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) load_stage<HD>(smem_base + s * St::kBytes, a.kv, table, kvh, tiles.at(s) * kTileKeys, lo, hi, 0, keep);
    cp_async_commit();
  }

  // sigmoid weights: the running maximum stays 0 and nothing is ever rescaled
  RowState st{{sig ? 0.f : -INFINITY, sig ? 0.f : -INFINITY}, {0.f, 0.f}};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float sl2 = a.scale * kLog2e;

  for (int i = 0; i < n_tiles; ++i) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    {
      const int nxt = i + kStages - 1;
      if (nxt < n_tiles)
        load_stage<HD>(smem_base + (nxt % kStages) * St::kBytes, a.kv, table, kvh, tiles.at(nxt) * kTileKeys, lo, hi, 0, keep);
      cp_async_commit();
    }
    const int key0 = tiles.at(i) * kTileKeys;
    if (key0 > warp_last_pos || (key0 + kTileKeys <= warp_lo && key0 >= keep)) continue;   // all masked for this warp
    const uint32_t kbase = smem_base + (i % kStages) * St::kBytes;
    const uint32_t vbase = kbase + kTileKeys * St::kRowBytes;

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {            // 16 keys per ldmatrix
        uint32_t b[4];
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4(b, kbase + St::off(kb * 16 + (mi >> 1) * 8 + r, ks * 2 + (mi & 1)));
        mma_16816(s[2 * kb], qf[ks], b[0], b[1]);
        mma_16816(s[2 * kb + 1], qf[ks], b[2], b[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
    // the distance of this thread's first key of the tile from each of its rows, converted once (exact below 2^24)
    const float dist0[2] = {(float)(pos[0] - key0 - t4 * 2), (float)(pos[1] - key0 - t4 * 2)};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + t4 * 2 + (e & 1), h = e >> 1;
        const bool ok = key <= pos[h] && (key >= row_lo[h] || key < keep);
        float v = ok ? fmaf(s[j][e], sl2, hb2) : -INFINITY;
        if (biased && ok) v -= log_distance_bias2f(r1, r2, dist0[h] - (float)(j * 8 + (e & 1)));
        s[j][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = sig ? 0.f : fmaxf(st.m[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;      // a row that has seen no key yet
      alpha[h] = exp2f(st.m[h] - m_use[h]);
      st.m[h] = m_new;
      st.l[h] *= alpha[h];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[j][e] = sig ? sigmoid2(s[j][e]) : exp2f(s[j][e] - m_use[e >> 1]);
        st.l[e >> 1] += s[j][e];
      }
#pragma unroll
    for (int nn = 0; nn < HD / 8; ++nn) {
      o[nn][0] *= alpha[0]; o[nn][1] *= alpha[0];
      o[nn][2] *= alpha[1]; o[nn][3] *= alpha[1];
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      uint32_t pf[4];
      pf[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
      pf[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
      pf[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      pf[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < kKSteps; ++n2) {
        uint32_t b[4];
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4_trans(b, vbase + St::off(kb * 16 + (mi & 1) * 8 + r, n2 * 2 + (mi >> 1)));
        mma_16816(o[2 * n2], pf, b[0], b[1]);
        mma_16816(o[2 * n2 + 1], pf, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 1);
    st.l[h] += __shfl_xor_sync(0xffffffffu, st.l[h], 2);
    // every row has seen its own key at least, so m is finite; a sink far above it makes the weights vanish
    if (a.x.sinks) st.l[h] += exp2f(a.x.sinks[head] * kLog2e - st.m[h]);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row_ok[h]) continue;
    const int row = warp * 16 + g4 + h * 8;
    const float inv = sig ? 1.0f : 1.0f / st.l[h];
    bf16* dst = a.out + (size_t)(tok0 + q0 + row) * a.out_stride + (size_t)head * HD + t4 * 2;
#pragma unroll
    for (int nn = 0; nn < HD / 8; ++nn)
      *reinterpret_cast<uint32_t*>(dst + nn * 8) = pack_bf16(o[nn][2 * h] * inv, o[nn][2 * h + 1] * inv);
  }
}

}  // namespace fa
}  // namespace lmsf

// Portions of prompts: tile_seq / tile_q0 list one entry per 64 query tokens (built by the caller).
LMSF_API int lmsf_attention_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                    const int* block_table, int max_blocks, const int* tile_seq, const int* tile_q0,
                                    int n_tiles, const int* cu_q, const int* ctx_len, float scale, int window,
                                    int n_q_heads, int head_dim, int kv_planes, int chunk, const float* r1,
                                    const float* r2, const float* sinks, int keep_first, int sigmoid,
                                    const float* head_bias, void* stream) {
  using namespace lmsf;
  using namespace lmsf::fa;
  if (n_tiles <= 0) return 0;
  if (head_dim != HD) LMSF_REFUSE("attention_prefill: built for head_dim=%d, called with %d", HD, head_dim);
  if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    LMSF_REFUSE("attention_prefill: %d query heads cannot be grouped over %d kv heads", n_q_heads, n_kv_heads);
  if (n_tiles > 65535) LMSF_REFUSE("attention_prefill: more than 65535 query tiles in one launch");
  if (block_size <= 0 || max_blocks <= 0) LMSF_REFUSE("attention_prefill: bad block table geometry");
  PrefillArgs a;
  a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride;
  if (!make_paged_kv(a.kv, cache, page_stride, block_size, n_kv_heads, HD, kv_planes))
    LMSF_REFUSE("attention: block_size=%d must be a power of two", block_size);
  a.block_table = block_table; a.max_blocks = max_blocks; a.tile_seq = tile_seq; a.tile_q0 = tile_q0;
  a.cu_q = cu_q; a.ctx_len = ctx_len; a.scale = scale; a.window = window; a.n_q_heads = n_q_heads;
  a.group = n_q_heads / n_kv_heads;
  if ((r1 == nullptr) != (r2 == nullptr) || chunk < 0) LMSF_REFUSE("attention_prefill: the distance bias takes both constants; chunk >= 0");
  if (sigmoid && sinks) LMSF_REFUSE("attention_prefill: sinks belong to a softmax, not to sigmoid weights");
  a.x = ScoreExtras{chunk, r1, r2, sinks, (window > 0 && keep_first > 0) ? keep_first : 0, sigmoid ? 1 : 0, head_bias};
  const int smem = kStages * St::kBytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  prefill_kernel<<<dim3(n_q_heads, n_tiles), kThreads, smem, (cudaStream_t)stream>>>(a);
  return LMSF_LAUNCH_STATUS();
}
