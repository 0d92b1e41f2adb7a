// Paged causal attention for any mix of rows, the exact kernel: it serves the
// float32 path and is the fallback of the bfloat16 path for sizes the fast
// kernels refuse.
//
// One block of W warps per (token, query head): eight for head sizes up to 64, four above (a constant of the model, so
// that every step shape computes a token the same way).  The keys a token sees,
// [max(0, pos - window + 1), pos], are cut into tiles of 32 keys that start at
// absolute multiples of 32; warp w takes tiles w, w+W, ... in ascending order with
// an online softmax, and the W partial results are merged in warp order.  So the
// arithmetic for a token depends on its position alone: not on how the sequence was
// cut into steps, not on what else is in the batch, not on which pages hold the keys.
// A warp brings its tile of keys into shared memory row by row (every load a whole row,
// consecutive lanes consecutive elements) and each lane then takes the dot product of
// the query with its own key from there; the values are read row by row as they are.
//
// Counterparts in gqf2008/machserve (crates/mach-model/src/kernels.rs):
// attn_decode_batched :1083-1141 (two-pass, one block per row and head),
// attn_paged_tiled_f32_gqa[_runs] :1895-2261 (online softmax over paged tiles).
// Scores, softmax and the weighted sum are float32; keys and values are widened on
// read.  Cache layout: pages[page][kv_head][slot in page][head_dim].
#include "common.cuh"

#define ATT_MAX_WARPS 8
#define ATT_MAX_HD 256

template <typename TA, typename TC, int ATT_WARPS>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_generic_kernel(const TA* __restrict__ q, const TC* __restrict__ k_pages, const TC* __restrict__ v_pages,
                         TA* __restrict__ out, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_pages,
                         int num_pages, int hq, int hkv, int hd, int page_size, int window, float scale) {
  __shared__ float q_s[ATT_MAX_HD];
  __shared__ float acc_s[ATT_WARPS][ATT_MAX_HD];
  __shared__ float m_s[ATT_WARPS], l_s[ATT_WARPS];
  extern __shared__ float key_tiles[];  // [warp][key of the tile][hd + 1]: the odd stride keeps the lanes' rows in different banks

  const int t = blockIdx.x / hq, h = blockIdx.x - t * hq;
  const int seq = seq_of_token[t];
  if (seq < 0) return;  // padding row
  const int pos = positions[t];
  const int kvh = h / (hq / hkv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  for (int d = threadIdx.x; d < hd; d += blockDim.x) q_s[d] = ms_to_float(q[((size_t)t * hq + h) * hd + d]);
  __syncthreads();

  constexpr int NACC = ATT_MAX_HD / 32;
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  const int* table = block_table + (size_t)seq * max_pages;
  const size_t head_off = (size_t)kvh * page_size * hd;
  const size_t page_elems = (size_t)hkv * page_size * hd;

  float* my_keys = key_tiles + (size_t)warp * 32 * (hd + 1);
  for (int tile = first_key / 32 + warp; tile * 32 <= pos; tile += ATT_WARPS) {
    const int key = tile * 32 + lane;
    const bool valid = key >= first_key && key <= pos;
    long long base = -1;  // element offset of this lane's key row inside the pages
    if (valid) {
      const int page = table[key / page_size];
      if (page >= 0 && page < num_pages) base = (long long)((size_t)page * page_elems + head_off + (size_t)(key % page_size) * hd);
    }
    __syncwarp();  // the tile before has been read
    // eight rows at a time, so that eight loads are in flight per lane
    for (int j0 = 0; j0 < 32; j0 += 8) {
      long long b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) b[u] = __shfl_sync(0xffffffffu, base, j0 + u);
      for (int d = lane; d < hd; d += 32) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = b[u] >= 0 ? ms_to_float(k_pages[b[u] + d]) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) my_keys[(j0 + u) * (hd + 1) + d] = v[u];
      }
    }
    __syncwarp();
    float s = -INFINITY;
    if (base >= 0) {
      const float* kr = my_keys + lane * (hd + 1);
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(q_s[d], kr[d], dot);
      s = dot * scale;
    }
    const float tile_max = ms_warp_max(s);
    const float m_new = fmaxf(m, tile_max);
    // every tile of the range holds at least one visible key, so m_new is finite
    const float p = (base >= 0 && m_new > -INFINITY) ? expf(s - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + ms_warp_sum(p);
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    // the values of eight keys at a time (eight loads in flight), added key by key in ascending order
    for (int j0 = 0; j0 < 32; j0 += 8) {
      long long b[8];
      float pj[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        b[u] = __shfl_sync(0xffffffffu, base, j0 + u);
        pj[u] = __shfl_sync(0xffffffffu, p, j0 + u);
      }
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = b[u] >= 0 ? ms_to_float(v_pages[b[u] + d]) : 0.f;
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (b[u] >= 0) acc[i] = fmaf(pj[u], v[u], acc[i]);
        }
      }
    }
    m = m_new;
  }

  if (lane == 0) {
    m_s[warp] = m;
    l_s[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) acc_s[warp][d] = acc[i];
  }
  __syncthreads();
  if (warp == 0) {
    float mm = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, m_s[w]);
    float f[ATT_WARPS], ll = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) {
      f[w] = l_s[w] > 0.f ? expf(m_s[w] - mm) : 0.f;
      ll += l_s[w] * f[w];
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    for (int d = lane; d < hd; d += 32) {
      float o = 0.f;
      for (int w = 0; w < ATT_WARPS; ++w) o += acc_s[w][d] * f[w];
      out[((size_t)t * hq + h) * hd + d] = ms_from_float<TA>(o * inv);
    }
  }
}

// q, out: [tokens, hq*hd].  window <= 0: every earlier key is visible.
MS_API int ms_attention_generic(const void* q, const void* k_pages, const void* v_pages, void* out, int act_dtype,
                                int cache_dtype, const int* positions, const int* seq_of_token,
                                const int* block_table, int max_pages, int num_pages, int tokens, int hq, int hkv,
                                int hd, int page_size, int window, float scale, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention: bad head counts hq=%d hkv=%d", hq, hkv);
  MS_REQUIRE(hd > 0 && hd <= ATT_MAX_HD, "attention: head_dim %d is outside (0, %d]", hd, ATT_MAX_HD);
  MS_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad cache sizes");
  const unsigned blocks = (unsigned)tokens * (unsigned)hq;
#define MS_ATT_LAUNCH(TA, TC, W)                                                                                \
  do {                                                                                                          \
    const size_t smem = (size_t)(W) * 32 * (hd + 1) * sizeof(float);                                           \
    static size_t configured = 0;                                                                               \
    if (smem > configured) {                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<TA, TC, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      MS_REQUIRE(e == cudaSuccess, "attention: cannot get shared memory for the key tiles: %s", cudaGetErrorString(e)); \
      configured = smem;                                                                                        \
    }                                                                                                           \
    attention_generic_kernel<TA, TC, W><<<blocks, (W) * 32, smem, stream>>>(                                   \
        (const TA*)q, (const TC*)k_pages, (const TC*)v_pages, (TA*)out, positions, seq_of_token, block_table,  \
        max_pages, num_pages, hq, hkv, hd, page_size, window, scale);                                          \
  } while (0)
#define MS_ATT_CASE(TA, TC)                \
  do {                                     \
    if (hd <= 64)                          \
      MS_ATT_LAUNCH(TA, TC, ATT_MAX_WARPS); \
    else                                   \
      MS_ATT_LAUNCH(TA, TC, 4);            \
  } while (0)
  if (act_dtype == MS_F32 && cache_dtype == MS_F32)
    MS_ATT_CASE(float, float);
  else if (act_dtype == MS_BF16 && cache_dtype == MS_BF16)
    MS_ATT_CASE(__nv_bfloat16, __nv_bfloat16);
  else if (act_dtype == MS_F32 && cache_dtype == MS_BF16)
    MS_ATT_CASE(float, __nv_bfloat16);
  else
    MS_REQUIRE(false, "attention: unsupported dtypes act=%d cache=%d", act_dtype, cache_dtype);
#undef MS_ATT_CASE
#undef MS_ATT_LAUNCH
  MS_LAUNCH_CHECK("attention_generic");
  return 0;
}
