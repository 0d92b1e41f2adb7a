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

// The same arithmetic for R consecutive rows of a step per block (portions of prompts): rows of one sequence whose
// ranges of keys begin in the same tile share every tile of keys and values that a warp stages, so the cache is read
// once for R rows instead of once for each; row by row, each warp does exactly what it does in the kernel above (its
// tiles, its order of sums, the merge in warp order), so a row's result is the same bit for bit whichever kernel
// computed it and whatever rows stood beside it.  NACC: head_dim / 32 rounded up.
// HEADS: the R "rows" of a block are instead up to R query heads of ONE token that share a key head (decoding with
// grouped queries): they read the same keys and values, which one block then stages once for all of them.
#define ATT_ROWS 8

template <typename TA, typename TC, int ATT_WARPS, int NACC, bool HEADS>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_generic_rows_kernel(const TA* __restrict__ q, const TC* __restrict__ k_pages, const TC* __restrict__ v_pages,
                              TA* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                              const int* __restrict__ block_table, int max_pages, int num_pages, int tokens, int hq, int hkv, int hd,
                              int page_size, int window, float scale) {
  extern __shared__ float rows_smem[];
  // [R][hd] queries; [warp][32][hd + 1] keys; [warp][32][hd] values; [warp][R][hd + 2] partial results for the merge
  float* q_s = rows_smem;
  float* k_all = q_s + ATT_ROWS * hd;
  float* v_all = k_all + (size_t)ATT_WARPS * 32 * (hd + 1);
  float* part = v_all + (size_t)ATT_WARPS * 32 * hd;
  // row r of the block is (token tok0 + r * tok_step, head head0 + r * head_step), if r < live_rows
  const int groups = hq / hkv;
  int tok0, tok_step, head0, head_step, live_rows, kvh;
  if (HEADS) {
    const int per_kv = (groups + ATT_ROWS - 1) / ATT_ROWS;
    const int t = blockIdx.x / (hkv * per_kv), rem = blockIdx.x - t * (hkv * per_kv);
    kvh = rem / per_kv;
    const int g0 = (rem - kvh * per_kv) * ATT_ROWS;
    tok0 = t; tok_step = 0; head0 = kvh * groups + g0; head_step = 1;
    live_rows = min(ATT_ROWS, groups - g0);
  } else {
    const int group = blockIdx.x / hq, h = blockIdx.x - group * hq;
    kvh = h / groups;
    tok0 = group * ATT_ROWS; tok_step = 1; head0 = h; head_step = 0;
    live_rows = min(ATT_ROWS, tokens - tok0);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t head_off = (size_t)kvh * page_size * hd;
  const size_t page_elems = (size_t)hkv * page_size * hd;
  float* my_k = k_all + (size_t)warp * 32 * (hd + 1);
  float* my_v = v_all + (size_t)warp * 32 * hd;

  int seq[ATT_ROWS], pos[ATT_ROWS], first[ATT_ROWS];
#pragma unroll
  for (int r = 0; r < ATT_ROWS; ++r) {
    seq[r] = r < live_rows ? seq_of_token[tok0 + r * tok_step] : -1;
    pos[r] = seq[r] >= 0 ? positions[tok0 + r * tok_step] : -1;
    first[r] = (window > 0 && pos[r] - window + 1 > 0) ? pos[r] - window + 1 : 0;
  }
  for (int e = threadIdx.x; e < ATT_ROWS * hd; e += blockDim.x) {
    const int r = e / hd, d = e - r * hd;
    q_s[e] = r < live_rows ? ms_to_float(q[((size_t)(tok0 + r * tok_step) * hq + head0 + r * head_step) * hd + d]) : 0.f;
  }
  __syncthreads();

  float m[ATT_ROWS], l[ATT_ROWS], acc[ATT_ROWS][NACC];
#pragma unroll
  for (int r = 0; r < ATT_ROWS; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[r][i] = 0.f;
  }

  // runs of rows that share their tiles: the same sequence and the same first tile
  unsigned done = 0;
#pragma unroll 1
  for (int lead = 0; lead < ATT_ROWS; ++lead) {
    if ((done >> lead) & 1u) continue;
    int lead_seq = -1, lead_tile = 0;
#pragma unroll
    for (int r = 0; r < ATT_ROWS; ++r)
      if (r == lead) {
        lead_seq = seq[r];
        lead_tile = first[r] / 32;
      }
    unsigned run = 0;
    int lo_key = 0x7fffffff, hi_pos = -1;
#pragma unroll
    for (int r = 0; r < ATT_ROWS; ++r)
      if (r >= lead && seq[r] == lead_seq && first[r] / 32 == lead_tile && !((done >> r) & 1u)) {
        run |= 1u << r;
        lo_key = min(lo_key, first[r]);
        hi_pos = max(hi_pos, pos[r]);
      }
    done |= run;
    if (lead_seq < 0) continue;  // padding rows
    const int* table = block_table + (size_t)lead_seq * max_pages;
#pragma unroll 1
    for (int tile = lead_tile + warp; tile * 32 <= hi_pos; tile += ATT_WARPS) {
      const int key = tile * 32 + lane;
      long long base = -1;  // element offset of this lane's key row inside the pages (for any row of the run)
      if (key >= lo_key && key <= hi_pos) {
        const int page = table[key / page_size];
        if (page >= 0 && page < num_pages) base = (long long)((size_t)page * page_elems + head_off + (size_t)(key % page_size) * hd);
      }
      __syncwarp();  // the tile before has been read
      for (int j0 = 0; j0 < 32; j0 += 8) {
        long long b[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) b[u] = __shfl_sync(0xffffffffu, base, j0 + u);
        for (int d = lane; d < hd; d += 32) {
          float kv[8], vv[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            kv[u] = b[u] >= 0 ? ms_to_float(k_pages[b[u] + d]) : 0.f;
            vv[u] = b[u] >= 0 ? ms_to_float(v_pages[b[u] + d]) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            my_k[(j0 + u) * (hd + 1) + d] = kv[u];
            my_v[(j0 + u) * hd + d] = vv[u];
          }
        }
      }
      __syncwarp();
      const float* kr = my_k + lane * (hd + 1);
      // the rows' dot products side by side (each row's own chain of sums in the order of the kernel above; eight
      // chains keep the multiply-add units busy where one would wait for itself)
      float dot[ATT_ROWS];
#pragma unroll
      for (int r = 0; r < ATT_ROWS; ++r) dot[r] = 0.f;
      if ((hd & 3) == 0) {
        for (int d = 0; d < hd; d += 4) {
          const float k0 = kr[d], k1 = kr[d + 1], k2 = kr[d + 2], k3 = kr[d + 3];
#pragma unroll
          for (int r = 0; r < ATT_ROWS; ++r) {
            const float4 qv = *reinterpret_cast<const float4*>(q_s + r * hd + d);
            dot[r] = fmaf(qv.x, k0, dot[r]);
            dot[r] = fmaf(qv.y, k1, dot[r]);
            dot[r] = fmaf(qv.z, k2, dot[r]);
            dot[r] = fmaf(qv.w, k3, dot[r]);
          }
        }
      } else {
        for (int d = 0; d < hd; ++d) {
          const float kd = kr[d];
#pragma unroll
          for (int r = 0; r < ATT_ROWS; ++r) dot[r] = fmaf(q_s[r * hd + d], kd, dot[r]);
        }
      }
      float pr[ATT_ROWS];
      unsigned vmask[ATT_ROWS];
#pragma unroll
      for (int r = 0; r < ATT_ROWS; ++r) {
        pr[r] = 0.f;
        vmask[r] = 0u;
        if (!((run >> r) & 1u) || tile * 32 > pos[r]) continue;  // (the same for the whole warp)
        const bool valid = base >= 0 && key >= first[r] && key <= pos[r];
        const float sc = valid ? dot[r] * scale : -INFINITY;
        const float tile_max = ms_warp_max(sc);
        const float m_new = fmaxf(m[r], tile_max);
        pr[r] = (valid && m_new > -INFINITY) ? expf(sc - m_new) : 0.f;
        const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
        l[r] = l[r] * corr + ms_warp_sum(pr[r]);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[r][i] *= corr;
        vmask[r] = __ballot_sync(0xffffffffu, valid);
        m[r] = m_new;
      }
      // the values key by key in ascending order, as the kernel above adds them; a value serves all rows
      for (int j = 0; j < 32; ++j) {
        float vj[NACC];
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int d = lane + 32 * i;
          vj[i] = d < hd ? my_v[j * hd + d] : 0.f;
        }
#pragma unroll
        for (int r = 0; r < ATT_ROWS; ++r) {
          const float pj = __shfl_sync(0xffffffffu, pr[r], j);
          if ((vmask[r] >> j) & 1u) {
#pragma unroll
            for (int i = 0; i < NACC; ++i) acc[r][i] = fmaf(pj, vj[i], acc[r][i]);
          }
        }
      }
    }
  }

  // every row's partial results of all warps, then warp r merges row r (and r + W, ...) in warp order
  __syncthreads();
  const int pw = hd + 2;
#pragma unroll
  for (int r = 0; r < ATT_ROWS; ++r) {
    float* p = part + ((size_t)warp * ATT_ROWS + r) * pw;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) p[d] = acc[r][i];
    }
    if (lane == 0) {
      p[hd] = m[r];
      p[hd + 1] = l[r];
    }
  }
  __syncthreads();
  for (int r = warp; r < ATT_ROWS; r += ATT_WARPS) {
    const int t = tok0 + r * tok_step, h = head0 + r * head_step;
    if (r >= live_rows || seq_of_token[t] < 0) continue;
    float mm = -INFINITY;
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, part[((size_t)w * ATT_ROWS + r) * pw + hd]);
    float f[ATT_WARPS], ll = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float* p = part + ((size_t)w * ATT_ROWS + r) * pw;
      f[w] = p[hd + 1] > 0.f ? expf(p[hd] - mm) : 0.f;
      ll += p[hd + 1] * f[w];
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    for (int d = lane; d < hd; d += 32) {
      float o = 0.f;
      for (int w = 0; w < ATT_WARPS; ++w) o += part[((size_t)w * ATT_ROWS + r) * pw + d] * f[w];
      out[((size_t)t * hq + h) * hd + d] = ms_from_float<TA>(o * inv);
    }
  }
}

// The heads form once more, for float32 rows that are alone in their sequences (decoding), spread over the GPU: the
// W warps of a (token, group of heads) are W blocks of one warp each in a thread-block cluster, so that a batch of 8
// rows with 2 key heads is 128 blocks instead of 16.  Warp w is the block of rank w: it takes the tiles w, w + W, ...
// exactly as above, with the next tile's keys and values on their way (cp.async, two places) while it works on the
// present one; the partial results go to the shared memory of the block that merges the row (row r: rank r mod W),
// which merges them in warp order with the arithmetic of the kernels above.  Same bits.
// Keys are staged with a row stride of hd + 4 floats: 16-byte copies need it, and 16-byte reads of a row per lane do
// not collide there.  head_dim a multiple of 4, at most 128.
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

__device__ __forceinline__ void attg_cp16(float* smem, const float* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // nothing is read for a key that is not there: the place is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}

template <int W, int NACC, int R>
__global__ void __launch_bounds__(32)
attention_generic_cluster_kernel(const float* __restrict__ q, const float* __restrict__ k_pages, const float* __restrict__ v_pages,
                                 float* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ block_table, int max_pages, int num_pages, int hq, int hkv, int hd,
                                 int page_size, int window, float scale) {
  constexpr int MINE = R > W ? R / W : 1;  // rows this block merges (R: up to this many heads of a group a block; a power of two)
  extern __shared__ __align__(16) float cl_smem[];
  const int ks = hd + 4;
  float* q_s = cl_smem;                               // [R][hd]
  float* k_buf = q_s + R * hd;                 // [2][32][hd + 4]
  float* v_buf = k_buf + 2 * 32 * ks;                 // [2][32][hd]
  float* part = v_buf + 2 * 32 * hd;                  // [MINE][W][hd + 2]: what the W warps found for the rows merged here
  cg::cluster_group cluster = cg::this_cluster();
  // (every block says that it runs; the others wait for that, much later, before they write into its shared memory)
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  const int warp = (int)cluster.block_rank(), lane = threadIdx.x;
  const int groups = hq / hkv;
  const int per_kv = (groups + R - 1) / R;
  const int unit = blockIdx.x / W;
  const int t = unit / (hkv * per_kv), rem = unit - t * (hkv * per_kv);
  const int kvh = rem / per_kv, g0 = (rem - kvh * per_kv) * R;
  const int head0 = kvh * groups + g0, live_rows = min(R, groups - g0);
  const int seq = seq_of_token[t];
  const int pos = seq >= 0 ? positions[t] : -1;  // (a padding row has no tiles, and takes part in the barrier)
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const size_t head_off = (size_t)kvh * page_size * hd;
  const size_t page_elems = (size_t)hkv * page_size * hd;
  const int* table = block_table + (size_t)(seq >= 0 ? seq : 0) * max_pages;
  const int chunks = hd / 4;  // 16-byte pieces of a row

  // requests tile `tile` into place `b`; returns the element offset of this lane's key row (-1: no such key)
  auto request = [&](int tile, int b) -> long long {
    const int key = tile * 32 + lane;
    long long base = -1;
    if (key >= first && key <= pos) {
      const int page = table[key / page_size];
      if (page >= 0 && page < num_pages) base = (long long)((size_t)page * page_elems + head_off + (size_t)(key % page_size) * hd);
    }
    float* kb = k_buf + (size_t)b * 32 * ks;
    float* vb = v_buf + (size_t)b * 32 * hd;
    for (int c = lane; c < 32 * chunks; c += 32) {
      const int j = c / chunks, piece = c - j * chunks;
      const long long bj = __shfl_sync(0xffffffffu, base, j);
      const bool ok = bj >= 0;
      attg_cp16(kb + j * ks + piece * 4, ok ? k_pages + bj + piece * 4 : k_pages, ok);
      attg_cp16(vb + j * hd + piece * 4, ok ? v_pages + bj + piece * 4 : v_pages, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    return base;
  };

  int tile = first / 32 + warp;
  long long base = -1, base_next = -1;
  if (tile * 32 <= pos) base = request(tile, 0);
  for (int e = lane; e < R * hd; e += 32) {
    const int r = e / hd, d = e - r * hd;
    q_s[e] = r < live_rows ? q[((size_t)t * hq + head0 + r) * hd + d] : 0.f;
  }
  __syncwarp();

  float m[R], l[R], acc[R][NACC];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[r][i] = 0.f;
  }

#pragma unroll 1
  for (int b = 0; tile * 32 <= pos; tile += W, b ^= 1) {
    const bool more = (tile + W) * 32 <= pos;
    if (more) {
      base_next = request(tile + W, b ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncwarp();
    const int key = tile * 32 + lane;
    const float* kr = k_buf + (size_t)b * 32 * ks + lane * ks;
    const float* my_v = v_buf + (size_t)b * 32 * hd;
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) dot[r] = 0.f;
    for (int d = 0; d < hd; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float4 qv = *reinterpret_cast<const float4*>(q_s + r * hd + d);
        dot[r] = fmaf(qv.x, kv.x, dot[r]);
        dot[r] = fmaf(qv.y, kv.y, dot[r]);
        dot[r] = fmaf(qv.z, kv.z, dot[r]);
        dot[r] = fmaf(qv.w, kv.w, dot[r]);
      }
    }
    const bool valid = base >= 0;  // (inside the row's range of keys and with a page)
    const unsigned vmask = __ballot_sync(0xffffffffu, valid);
    float pr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      pr[r] = 0.f;
      if (r >= live_rows) continue;
      const float sc = valid ? dot[r] * scale : -INFINITY;
      const float tile_max = ms_warp_max(sc);
      const float m_new = fmaxf(m[r], tile_max);
      pr[r] = (valid && m_new > -INFINITY) ? expf(sc - m_new) : 0.f;
      const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
      l[r] = l[r] * corr + ms_warp_sum(pr[r]);
#pragma unroll
      for (int i = 0; i < NACC; ++i) acc[r][i] *= corr;
      m[r] = m_new;
    }
    for (int j = 0; j < 32; ++j) {
      if (!((vmask >> j) & 1u)) continue;
      float vj[NACC];
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        vj[i] = d < hd ? my_v[j * hd + d] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float pj = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[r][i] = fmaf(pj, vj[i], acc[r][i]);
      }
    }
    __syncwarp();  // the place is free for the tile after the next
    base = base_next;
  }

  // this warp's results go to the blocks that merge the rows
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  const int pw = hd + 2;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float* p = cluster.map_shared_rank(part, r % W) + ((size_t)(r / W) * W + warp) * pw;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) p[d] = acc[r][i];
    }
    if (lane == 0) {
      p[hd] = m[r];
      p[hd + 1] = l[r];
    }
  }
  cluster.sync();
#pragma unroll 1
  for (int k = 0; k < MINE; ++k) {
    const int r = k * W + warp;
    if (r >= live_rows || seq < 0) continue;
    const float* mine = part + (size_t)k * W * pw;
    float mm = -INFINITY;
    for (int w = 0; w < W; ++w) mm = fmaxf(mm, mine[(size_t)w * pw + hd]);
    float f[W], ll = 0.f;
    for (int w = 0; w < W; ++w) {
      const float* p = mine + (size_t)w * pw;
      f[w] = p[hd + 1] > 0.f ? expf(p[hd] - mm) : 0.f;
      ll += p[hd + 1] * f[w];
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    for (int d = lane; d < hd; d += 32) {
      float o = 0.f;
      for (int w = 0; w < W; ++w) o += mine[(size_t)w * pw + d] * f[w];
      out[((size_t)t * hq + head0 + r) * hd + d] = o * inv;
    }
  }
}

template <int W, int NACC, int R>
static int launch_attention_generic_cluster(const float* q, const float* k_pages, const float* v_pages, float* out,
                                            const int* positions, const int* seq_of_token, const int* block_table,
                                            int max_pages, int num_pages, int tokens, int hq, int hkv, int hd, int page_size,
                                            int window, float scale, cudaStream_t stream) {
  const int groups = hq / hkv;
  const unsigned units = (unsigned)tokens * (unsigned)hkv * (unsigned)((groups + R - 1) / R);
  const size_t smem = ((size_t)R * hd + 2 * 32 * (size_t)(hd + 4) + 2 * 32 * (size_t)hd + (size_t)(R > W ? R / W : 1) * W * (hd + 2)) * sizeof(float);
  auto kern = attention_generic_cluster_kernel<W, NACC, R>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "attention: cannot get shared memory for the key tiles: %s", cudaGetErrorString(e));
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units * W);
  cfg.blockDim = dim3(32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = W;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, q, k_pages, v_pages, out, positions, seq_of_token, block_table, max_pages,
                                           num_pages, hq, hkv, hd, page_size, window, scale);
  MS_REQUIRE(e == cudaSuccess, "attention_generic: launch failed: %s", cudaGetErrorString(e));
  return 0;
}

// q, out: [tokens, hq*hd].  window <= 0: every earlier key is visible.  share_rows: the step has rows that follow one
// another in a sequence (portions of prompts): eight rows a block share the tiles they read (head sizes up to 128);
// else the query heads of a token that share a key head do.  The results are the same bits either way.
MS_API int ms_attention_generic(const void* q, const void* k_pages, const void* v_pages, void* out, int act_dtype,
                                int cache_dtype, const int* positions, const int* seq_of_token,
                                const int* block_table, int max_pages, int num_pages, int tokens, int hq, int hkv,
                                int hd, int page_size, int window, float scale, int share_rows, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention: bad head counts hq=%d hkv=%d", hq, hkv);
  MS_REQUIRE(hd > 0 && hd <= ATT_MAX_HD, "attention: head_dim %d is outside (0, %d]", hd, ATT_MAX_HD);
  MS_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention: bad cache sizes");
  const int groups = hq / hkv;
  if (share_rows <= 0 && act_dtype == MS_F32 && cache_dtype == MS_F32 && hd % 4 == 0 && hd <= 128 &&
      ((uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)q) % 16 == 0 && (size_t)tokens * hq * 8 < 0x7fffffffu) {
    // decoding in float32: the warps of a row as blocks of a cluster (same bits as below).  Up to R heads of a group
    // share a block's tiles: the fewest that keep the launch at about four blocks of one warp per SM at head sizes up to
    // 64, under three above (measured at 1, 8 and 64 rows of 2,048 keys, 7 and 6 heads a group; share_rows < 0 asks
    // for R = -share_rows, for such measurements)
    const long long most = hd <= 64 ? 592 : 400;
    int r = 1;
    while (r < 8 && (long long)tokens * hkv * ((groups + r - 1) / r) * (hd <= 64 ? 8 : 4) > most) r <<= 1;
    if (share_rows < 0) r = -share_rows;
    MS_REQUIRE(r == 1 || r == 2 || r == 4 || r == 8, "attention: %d heads a block; 1, 2, 4 or 8", r);
#define MS_ATT_CLUSTER(W, NACC, R)                                                                                        \
  return launch_attention_generic_cluster<W, NACC, R>((const float*)q, (const float*)k_pages, (const float*)v_pages, (float*)out, \
                                                      positions, seq_of_token, block_table, max_pages, num_pages, tokens, hq, hkv, \
                                                      hd, page_size, window, scale, stream)
    if (hd <= 64) {
      if (r == 8) MS_ATT_CLUSTER(ATT_MAX_WARPS, 2, 8);
      if (r == 4) MS_ATT_CLUSTER(ATT_MAX_WARPS, 2, 4);
      if (r == 2) MS_ATT_CLUSTER(ATT_MAX_WARPS, 2, 2);
      MS_ATT_CLUSTER(ATT_MAX_WARPS, 2, 1);
    }
    if (r == 8) MS_ATT_CLUSTER(4, 4, 8);
    if (r == 4) MS_ATT_CLUSTER(4, 4, 4);
    if (r == 2) MS_ATT_CLUSTER(4, 4, 2);
    MS_ATT_CLUSTER(4, 4, 1);
#undef MS_ATT_CLUSTER
  }
  share_rows = share_rows > 0;
  const bool rows = share_rows && hd <= 128 && tokens > 1;      // rows of portions share their tiles
  const bool heads = !rows && hd <= 128 && groups > 1;          // the heads of a group share theirs
  const unsigned blocks = rows    ? (unsigned)((tokens + ATT_ROWS - 1) / ATT_ROWS) * (unsigned)hq
                          : heads ? (unsigned)tokens * (unsigned)hkv * (unsigned)((groups + ATT_ROWS - 1) / ATT_ROWS)
                                  : (unsigned)tokens * (unsigned)hq;
#define MS_ATT_SET_SMEM(KERN, BYTES)                                                                            \
  do {                                                                                                          \
    static size_t configured = 0;                                                                               \
    if ((BYTES) > configured) {                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(KERN, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(BYTES));    \
      MS_REQUIRE(e == cudaSuccess, "attention: cannot get shared memory for the key tiles: %s", cudaGetErrorString(e)); \
      configured = (BYTES);                                                                                     \
    }                                                                                                           \
  } while (0)
#define MS_ATT_LAUNCH(TA, TC, W)                                                                                \
  do {                                                                                                          \
    const size_t smem = (size_t)(W) * 32 * (hd + 1) * sizeof(float);                                           \
    auto kern = attention_generic_kernel<TA, TC, W>;                                                            \
    MS_ATT_SET_SMEM(kern, smem);                                                                                \
    kern<<<blocks, (W) * 32, smem, stream>>>((const TA*)q, (const TC*)k_pages, (const TC*)v_pages, (TA*)out, positions, \
                                            seq_of_token, block_table, max_pages, num_pages, hq, hkv, hd, page_size, window, scale); \
  } while (0)
#define MS_ATT_LAUNCH_ROWS(TA, TC, W, NACC, H)                                                                   \
  do {                                                                                                          \
    const size_t smem = ((size_t)ATT_ROWS * hd + (size_t)(W) * 32 * (2 * hd + 1) + (size_t)(W) * ATT_ROWS * (hd + 2)) * sizeof(float); \
    auto kern = attention_generic_rows_kernel<TA, TC, W, NACC, H>;                                              \
    MS_ATT_SET_SMEM(kern, smem);                                                                                \
    kern<<<blocks, (W) * 32, smem, stream>>>((const TA*)q, (const TC*)k_pages, (const TC*)v_pages, (TA*)out, positions, \
                                            seq_of_token, block_table, max_pages, num_pages, tokens, hq, hkv, hd, page_size, window, scale); \
  } while (0)
#define MS_ATT_CASE(TA, TC)                                \
  do {                                                     \
    if (rows && hd <= 64)                                  \
      MS_ATT_LAUNCH_ROWS(TA, TC, ATT_MAX_WARPS, 2, false); \
    else if (rows)                                         \
      MS_ATT_LAUNCH_ROWS(TA, TC, 4, 4, false);             \
    else if (heads && hd <= 64)                            \
      MS_ATT_LAUNCH_ROWS(TA, TC, ATT_MAX_WARPS, 2, true);  \
    else if (heads)                                        \
      MS_ATT_LAUNCH_ROWS(TA, TC, 4, 4, true);              \
    else if (hd <= 64)                                     \
      MS_ATT_LAUNCH(TA, TC, ATT_MAX_WARPS);                \
    else                                                   \
      MS_ATT_LAUNCH(TA, TC, 4);                            \
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
#undef MS_ATT_LAUNCH_ROWS
#undef MS_ATT_SET_SMEM
  MS_LAUNCH_CHECK("attention_generic");
  return 0;
}
