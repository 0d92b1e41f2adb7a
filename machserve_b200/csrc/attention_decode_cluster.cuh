// Paged GQA attention for single rows (decoding) with the splits of a row's keys held by one
// thread-block cluster: the partial results meet in distributed shared memory, so no scratch
// memory, no counters and no second pass over global memory are needed.
//
// One cluster per (row, kv head); its blocks (up to 8) take consecutive runs of 64-key tiles.
// A block first requests the tiles of its run with asynchronous copies, BEFORE it waits for the
// kernel that precedes it in the stream: keys and values of earlier positions do not depend on
// that kernel, so they stream in while it (the projection and the rotary kernel) still runs.
// Only the row of the current position, which the preceding kernel writes, is copied after
// the wait.  In the fused form the preceding kernel is the q|k|v projection itself: the block adds
// the bias, rotates its query heads and the current key (same arithmetic as rope_kv.cu), puts key and
// value of the current position into its tile and into the cache, and no kernel stands between the
// projection and the attention.  Then, as in attention_decode.cu, each of the four warps takes 16 keys of a tile
// with its own online softmax, the warps are merged in warp order, and block 0 of the cluster
// merges the blocks in rank order.  Scores, softmax and sums are float32.
//
// The reference reads every key once for the query heads that share it
// (attn_decode_batched_f16_gqa, crates/mach-model/src/kernels.rs:2911-3036 of gqf2008/machserve)
// with one block per (row, kv head) and no split over the keys.
#pragma once
#include <cooperative_groups.h>

#include "attention_mma.cuh"
#include "launch.cuh"

namespace cg = cooperative_groups;

#define DCL_TILE 64

// What the fused form reads instead of encoded queries: rows of q|k|v as the projection left them.
struct DclRaw {
  const __nv_bfloat16* qkv;  // [tokens, ld]: q heads, then (if store) k heads, then v heads
  int ld;
  const float* bias;      // [q | k | v] or null
  const float2* cos_sin;  // [positions][HD / 2]
  int store;              // the row carries k and v of its position, to be written into the cache
};

// Few rows with long contexts: a (row, kv head) pair's keys go to `parts` clusters instead of one.  Each cluster
// leaves its merged sums in `scratch` (per pair and part: groups * HD sums, then 16 maxima and 16 sums of a row's
// probabilities) and counts itself in `counters` (one per pair: zero before the first launch, left zero by every
// launch); the cluster that counts last merges the parts in their order, so the result does not depend on who
// came last, and no cluster waits for another.
struct DclOuter {
  int parts;  // 1: the cluster writes the output itself
  float* scratch;
  int* counters;
};
#define DCL_MAX_PARTS 16

// Requests `ntiles` tiles of 64 keys and their values, starting at tile `tile0`, into consecutive stages.  One
// copy of this code serves the request before the wait and those of later rounds (the kernel's code is kept
// small on purpose: a decoding step is a chain of short kernels, and each finds the instruction cache cold).
template <int HD, int DCL_THREADS>
__device__ __noinline__ void dcl_load_round(__nv_bfloat16* kv_s, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages,
                                            const int* table, int num_pages, int page_size, size_t page_elems,
                                            size_t head_off, int tile0, int ntiles, int first_key, int last_key,
                                            int skip_key, int tid) {
  constexpr int STRIDE = HD + 8, TILE_ELEMS = DCL_TILE * STRIDE, CHUNKS = HD / 8, STEP = DCL_THREADS / CHUNKS;
  if (page_size % DCL_TILE == 0 && DCL_THREADS % CHUNKS == 0) {
    // A tile lies inside one page: one look-up serves its keys and its values, whose rows are contiguous there,
    // and a thread's chunks are the same 16 bytes of rows r0, r0 + STEP, ...
    const int r0 = tid / CHUNKS, ch = tid - r0 * CHUNKS;
    const int tiles_per_page = page_size / DCL_TILE;
#pragma unroll 1
    for (int s = 0; s < ntiles; ++s) {
      const int tile = tile0 + s, key0 = tile * DCL_TILE;
      const int lp = tiles_per_page == 1 ? tile : tile / tiles_per_page;
      const int page = (key0 <= last_key && key0 + DCL_TILE > first_key) ? table[lp] : -1;
      const bool page_ok = page >= 0 && page < num_pages;
      const size_t off = (page_ok ? (size_t)page * page_elems + head_off + (size_t)(key0 - lp * page_size) * HD : 0) + r0 * HD + ch * 8;
      __nv_bfloat16* dst = kv_s + (size_t)s * 2 * TILE_ELEMS + r0 * STRIDE + ch * 8;
#pragma unroll
      for (int j = 0; j < DCL_TILE / STEP; ++j) {
        const int key = key0 + r0 + j * STEP;
        if (key == skip_key) continue;  // left alone: the caller fills it
        const bool ok = page_ok && key >= first_key && key <= last_key;
        ms_cp_async16(dst + j * STEP * STRIDE, ok ? k_pages + off + (size_t)j * STEP * HD : k_pages, ok);
        ms_cp_async16(dst + TILE_ELEMS + j * STEP * STRIDE, ok ? v_pages + off + (size_t)j * STEP * HD : v_pages, ok);
      }
    }
  } else {
#pragma unroll 1
    for (int i = 0; i < 2 * ntiles; ++i) {
      const int s = i >> 1, which = i & 1;
      ms_load_kv_tile<HD>(kv_s + (size_t)i * TILE_ELEMS, which ? v_pages : k_pages, table, num_pages, page_size, page_elems,
                          head_off, (tile0 + s) * DCL_TILE, DCL_TILE, first_key, last_key, tid, DCL_THREADS, skip_key);
    }
  }
  ms_cp_async_commit();
}

// A warp requests ITS part of a tile (KPW keys, the rows it will attend to itself) into the stage at `tile_s`: a warp
// that copies what it reads needs no barrier of the block around its copies.  `page`: the page the tile lies in
// (-1: none), `key0`: the tile's first key.  One group of copies (also when there is nothing to copy).
template <int HD, int KPW>
__device__ __forceinline__ void dcl_load_part(__nv_bfloat16* tile_s, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, int page,
                                              int num_pages, int page_size, size_t page_elems, size_t head_off, int key0, int krow0,
                                              int first_key, int last_key, bool any, int lane) {
  constexpr int STRIDE = HD + 8, TILE_ELEMS = DCL_TILE * STRIDE, CHUNKS = HD / 8;
  if (any) {
    const bool page_ok = page >= 0 && page < num_pages;
    const size_t off = (page_ok ? (size_t)page * page_elems + head_off + (size_t)(key0 % page_size) * HD : 0);
#pragma unroll
    for (int j = 0; j < KPW * CHUNKS / 32; ++j) {
      const int idx = lane + 32 * j, r = krow0 + idx / CHUNKS, ch = idx % CHUNKS;
      const int key = key0 + r;
      const bool ok = page_ok && key >= first_key && key <= last_key;
      __nv_bfloat16* dst = tile_s + r * STRIDE + ch * 8;
      ms_cp_async16(dst, ok ? k_pages + off + (size_t)r * HD + ch * 8 : k_pages, ok);
      ms_cp_async16(dst + TILE_ELEMS, ok ? v_pages + off + (size_t)r * HD + ch * 8 : v_pages, ok);
    }
  }
  ms_cp_async_commit();
}

// KPW: keys a warp takes at a time: 64, a whole tile, or 32, half a tile.  DCL_WARPS: 4 or 8.  Four warps with a
// tile each serve blocks with long runs of keys; four warps with half a tile each, blocks that can hold only two
// tiles (many blocks on the GPU: more of them share an SM); eight warps with half a tile each, the few blocks of a
// small batch, where a row's chain of dependent steps is what the step waits for.
template <int HD, bool FUSED, int KPW, int DCL_WARPS, bool OUTER>
__global__ void __launch_bounds__(DCL_WARPS * 32)
attention_decode_cluster_kernel(const __nv_bfloat16* __restrict__ q, DclRaw raw, __nv_bfloat16* k_pages,
                                __nv_bfloat16* v_pages, __nv_bfloat16* __restrict__ out,
                                const int* __restrict__ rows, const int* __restrict__ positions,
                                const int* __restrict__ slot_of_token, const int* __restrict__ block_table,
                                int max_pages, int num_pages, int hq, int hkv, int page_size, int window,
                                float scale_log2, int num_splits, int stages, DclOuter outer) {
  constexpr int STRIDE = HD + 8;
  constexpr int TILE_ELEMS = DCL_TILE * STRIDE;
  constexpr int DCL_THREADS = DCL_WARPS * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [16][STRIDE]
  __nv_bfloat16* kv_s = q_s + 16 * STRIDE;                           // [stages][K, V][DCL_TILE][STRIDE]
  // What the blocks of a cluster hand each other at the end: block k puts its part of (head, coordinate) pair e into
  // the shared memory of the block that merges e, at [k][e - that block's first pair], and its heads' maxima and
  // sums into every block's.  Nothing else lives here, so the others may write while this block still attends.
  __shared__ __align__(16) float gath_o[16 * HD + 32];
  __shared__ float2 gath_ml[8][16];  // (maximum, sum)

  MS_TIMELINE_BEGIN(200);
  ms_pdl_trigger();
  // everything up to the wait reads only what no kernel of this step writes: the step's index arrays,
  // the block tables, and keys and values of positions before the current one
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  // blockIdx.z: the clusters of a pair one after the other (OUTER: more than one); `split` is the block's rank in its
  // cluster (a power of two of blocks)
  const int kvh = blockIdx.y;
  const int split = OUTER ? blockIdx.z & (num_splits - 1) : blockIdx.z;
  const int part = OUTER ? blockIdx.z >> (31 - __clz(num_splits)) : 0;
  const int parts = OUTER ? outer.parts : 1;
  const int groups = hq / hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = t >= 0 ? slot_of_token[t] : -1;  // (a list of rows may be padded with -1)
  const bool live = slot >= 0;  // a padding row still takes part in the cluster's barriers
  const int pos = live ? positions[t] : 0;
  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int tile_lo = first_key / DCL_TILE, tile_hi = pos / DCL_TILE;
  const int ntiles = tile_hi - tile_lo + 1;
  const int runs = num_splits * parts;  // the pair's tiles in this many runs, one per block
  const int per_split = (ntiles + runs - 1) / runs;
  const int my_lo = tile_lo + (part * num_splits + split) * per_split;
  const int my_hi = live ? min(my_lo + per_split - 1, tile_hi) : my_lo - 1;
  const int* table = block_table + (size_t)(live ? slot : 0) * max_pages;
  const size_t page_elems = (size_t)hkv * page_size * HD;
  const size_t head_off = (size_t)kvh * page_size * HD;

  const int n_my = my_hi - my_lo + 1;
  // A run of keys that the stages hold at once is requested whole, before the wait.  A longer run goes through the
  // stages as a ring, a tile at a time: while the warps attend to one tile (a part of it each), the copies of the
  // `stages - 1` tiles after it are on their way.  Every warp copies the part of a tile that it attends to itself, so
  // the warps go through the ring each at its own pace, without a barrier of the block.  That needs the warps to share
  // a tile evenly and tiles that lie inside pages; other shapes take the run in rounds of `stages` tiles.
  // (the warps of a block take the keys of G tiles between them: G = 1 with four warps of 16 keys, 2 with eight)
  constexpr int G = KPW * DCL_WARPS / DCL_TILE;
  constexpr bool RINGS = G >= 1 && KPW * DCL_WARPS == G * DCL_TILE;
  const int slots = RINGS ? stages / (G > 0 ? G : 1) : 0;  // places of the ring, of G tiles each
  const bool ring = RINGS && n_my > stages && n_my <= 64 && slots >= 2 && slots * G == stages && page_size % DCL_TILE == 0;
  const int fill = min(stages, max(n_my, 0));  // tiles requested before the wait, without the current position's row
  // ring: lane l knows the pages of the block's tiles l and 32 + l, so that no copy has to wait for a look-up; a warp's
  // part of a place of the ring is the keys krow .. krow + KPW - 1 of the place's tile wt
  int ring_page[2] = {-1, -1};
  const int wt = warp * KPW / DCL_TILE, krow = warp * KPW % DCL_TILE;
  if (ring) {
    const int tiles_per_page = page_size / DCL_TILE;
#pragma unroll
    for (int h = 0; h < 2; ++h)
      if (32 * h + lane < n_my) ring_page[h] = table[(my_lo + 32 * h + lane) / tiles_per_page];
#pragma unroll 1
    for (int s = 0; s < slots; ++s) {  // a group of copies per place
      const int t = s * G + wt;
      dcl_load_part<HD, KPW>(kv_s + (size_t)t * 2 * TILE_ELEMS, k_pages, v_pages, __shfl_sync(0xffffffffu, ring_page[0], t & 31), num_pages,
                             page_size, page_elems, head_off, (my_lo + t) * DCL_TILE, krow, first_key, pos, t < n_my, lane);
    }
  } else {
    dcl_load_round<HD, DCL_THREADS>(kv_s, k_pages, v_pages, table, num_pages, page_size, page_elems, head_off, my_lo, fill, first_key, pos,
                                    pos, tid);
  }

  ms_pdl_wait();
  MS_TIMELINE_WAITED();

  const int ptile = pos / DCL_TILE;
  bool row_done = false;  // the current position's key and value are in place (fused form)
  if constexpr (FUSED) {
    constexpr int HALF = HD / 2, PER_HEAD = HALF / 4;  // a thread takes 4 pairs (j, j + HALF) of one head
    // query rows past the group, and all of a padding row, are zero
    for (int c = tid; c < 16 * (HD / 8); c += DCL_THREADS)
      if (c / (HD / 8) >= groups || !live)
        *reinterpret_cast<uint4*>(q_s + (c / (HD / 8)) * STRIDE + (c % (HD / 8)) * 8) = make_uint4(0, 0, 0, 0);
    if (live) {
      const __nv_bfloat16* row = raw.qkv + (size_t)t * raw.ld;
      const float2* cs = raw.cos_sin + (size_t)pos * HALF;
      // the block whose run holds the current position's tile encodes and stores its key and value
      const bool mine = raw.store && ptile >= my_lo && ptile <= my_hi;
      row_done = mine;
      bool page_ok = false;
      size_t cache_off = 0;
      __nv_bfloat16* tile_row = nullptr;
      if (mine) {
        const int page = table[pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        cache_off = (size_t)(page_ok ? page : 0) * page_elems + head_off + (size_t)(pos % page_size) * HD;
        if (ptile - my_lo < fill)  // else the tile is copied from the cache later, after a barrier
          tile_row = kv_s + (size_t)(ptile - my_lo) * 2 * TILE_ELEMS + (pos - ptile * DCL_TILE) * STRIDE;
      }
      // heads 0 .. groups-1: the group's query heads; then (mine) the key head and the value head
      const int heads = groups + (mine ? 2 : 0);
#pragma unroll 1
      for (int e = tid; e < heads * PER_HEAD; e += DCL_THREADS) {
        const int h = e / PER_HEAD, j = (e - h * PER_HEAD) * 4;
        const int kind = h < groups ? 0 : h - groups + 1;  // 0: query, 1: key, 2: value (not rotated)
        const int col = kind == 0 ? (kvh * groups + h) * HD : (hq + (kind == 2 ? hkv : 0) + kvh) * HD;
        const uint2 ua = *reinterpret_cast<const uint2*>(row + col + j), ub = *reinterpret_cast<const uint2*>(row + col + j + HALF);
        float a[4], b[4];
        {
          const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ua.x));
          const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ua.y));
          const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub.x));
          const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub.y));
          a[0] = a0.x; a[1] = a0.y; a[2] = a1.x; a[3] = a1.y;
          b[0] = b0.x; b[1] = b0.y; b[2] = b1.x; b[3] = b1.y;
        }
        if (raw.bias) {
          const float4 ba = *reinterpret_cast<const float4*>(raw.bias + col + j), bb = *reinterpret_cast<const float4*>(raw.bias + col + j + HALF);
          a[0] += ba.x; a[1] += ba.y; a[2] += ba.z; a[3] += ba.w;
          b[0] += bb.x; b[1] += bb.y; b[2] += bb.z; b[3] += bb.w;
        }
        if (kind != 2) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 cc = cs[j + i];
            const float ra = a[i] * cc.x - b[i] * cc.y, rb = a[i] * cc.y + b[i] * cc.x;
            a[i] = ra;
            b[i] = rb;
          }
        }
        uint2 oa = make_uint2(ms_pack_bf16(a[0], a[1]), ms_pack_bf16(a[2], a[3]));
        uint2 ob = make_uint2(ms_pack_bf16(b[0], b[1]), ms_pack_bf16(b[2], b[3]));
        if (kind == 0) {
          *reinterpret_cast<uint2*>(q_s + h * STRIDE + j) = oa;
          *reinterpret_cast<uint2*>(q_s + h * STRIDE + j + HALF) = ob;
        } else {
          __nv_bfloat16* pages = kind == 1 ? k_pages : v_pages;
          if (page_ok) {
            *reinterpret_cast<uint2*>(pages + cache_off + j) = oa;
            *reinterpret_cast<uint2*>(pages + cache_off + j + HALF) = ob;
          } else {  // a position without a page reads as zeros, as in the unfused form
            oa = ob = make_uint2(0, 0);
          }
          if (tile_row) {
            __nv_bfloat16* tr = tile_row + (kind == 2 ? TILE_ELEMS : 0);
            *reinterpret_cast<uint2*>(tr + j) = oa;
            *reinterpret_cast<uint2*>(tr + j + HALF) = ob;
          }
        }
      }
    }
  } else {
    // the query rows (written by the preceding kernel): row g = query head kvh*groups + g, the rest zero
    for (int c = tid; c < 16 * (HD / 8); c += DCL_THREADS) {
      const int r = c / (HD / 8), ch = c - r * (HD / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (live && r < groups) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * hq + kvh * groups + r) * HD + ch * 8);
      *reinterpret_cast<uint4*>(q_s + r * STRIDE + ch * 8) = v;
    }
  }
  // the current position's own key and value, if its tile is in the first round
  {
    if (!row_done && live && ptile >= my_lo && ptile <= my_hi && ptile - my_lo < fill && tid < 2 * (HD / 8)) {
      const int which = tid / (HD / 8), ch = tid - which * (HD / 8);
      const int page = table[pos / page_size];
      const bool ok = page >= 0 && page < num_pages;
      const __nv_bfloat16* src = (which ? v_pages : k_pages) + (ok ? (size_t)page * page_elems + head_off + (size_t)(pos % page_size) * HD + ch * 8 : 0);
      __nv_bfloat16* dst = kv_s + (size_t)(ptile - my_lo) * 2 * TILE_ELEMS + (which ? TILE_ELEMS : 0) +
                           (pos - ptile * DCL_TILE) * STRIDE + ch * 8;
      ms_cp_async16(dst, src, ok);
    }
    ms_cp_async_commit();
  }

  MS_TIMELINE_MARK(0);
  MsRowState<HD> st;
  st.init();
  unsigned qa[HD / 16][4];
  const int lo[2] = {first_key, first_key}, hi[2] = {pos, pos};
  const int mat = lane >> 3, within = lane & 7;
  if (ring) {
    __syncthreads();  // the query rows are in place, and the current position's key and value are in the cache
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ms_ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], q_s + (within + 8 * (mat & 1)) * STRIDE + ks * 16 + 8 * (mat >> 1));
    // a thread's groups of copies so far: one per place, the current row's (empty here), then one per turn done (the
    // last ones empty): its part of turn i has landed when at most slots - 1 groups are still on their way
    const int turns = (n_my + G - 1) / G;
#pragma unroll 1
    for (int i = 0; i < turns; ++i) {
      ms_cp_async_wait_dynamic(slots - 1);
      __syncwarp();
      const int t = i * G + wt;
      __nv_bfloat16* buf = kv_s + (size_t)((i % slots) * G + wt) * 2 * TILE_ELEMS;
      if (t < n_my)
        ms_attend_keys<HD, KPW / 16, true>(st, qa, buf, buf + TILE_ELEMS, krow, (my_lo + t) * DCL_TILE + krow, lo, hi, first_key, pos,
                                           scale_log2, lane);
      __syncwarp();  // the warp is done with its part of the place
      const int tn = (i + slots) * G + wt;
      const int page = __shfl_sync(0xffffffffu, tn < 32 ? ring_page[0] : ring_page[1], tn & 31);
      dcl_load_part<HD, KPW>(buf, k_pages, v_pages, page, num_pages, page_size, page_elems, head_off, (my_lo + tn) * DCL_TILE, krow,
                             first_key, pos, tn < n_my, lane);
    }
  } else {
    // rounds of up to `stages` tiles; within a round warp w takes the parts w, w + DCL_WARPS, ... of the round's tiles
#pragma unroll 1
    for (int r0 = 0; r0 < n_my; r0 += stages) {
      const int nr = min(stages, n_my - r0);
      if (r0 > 0) {
        __syncthreads();  // every warp is done with the stages
        dcl_load_round<HD, DCL_THREADS>(kv_s, k_pages, v_pages, table, num_pages, page_size, page_elems, head_off, my_lo + r0, nr, first_key,
                                        pos, -1, tid);
      }
      ms_cp_async_wait<0>();
      __syncthreads();
      if (r0 == 0) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          ms_ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], q_s + (within + 8 * (mat & 1)) * STRIDE + ks * 16 + 8 * (mat >> 1));
      }
      constexpr int PARTS = DCL_TILE / KPW;  // parts of a tile
#pragma unroll 1
      for (int sl = warp; sl < nr * PARTS; sl += DCL_WARPS) {
        const int i = sl / PARTS, krow = (sl % PARTS) * KPW;
        const __nv_bfloat16* ks = kv_s + (size_t)i * 2 * TILE_ELEMS;
        ms_attend_keys<HD, KPW / 16, true>(st, qa, ks, ks + TILE_ELEMS, krow, (my_lo + r0 + i) * DCL_TILE + krow, lo, hi, first_key,
                                           pos, scale_log2, lane);
      }
    }
  }
  ms_cp_async_wait<0>();
  __syncthreads();  // the stages are used for the merge next
  MS_TIMELINE_MARK(1);

  // merge the four warps of the block in warp order
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
    st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
  }
  constexpr int RED = HD + 8;  // (rows eight banks apart: a warp's 8-byte stores below collide two ways, not eight)
  float* red_o = reinterpret_cast<float*>(kv_s);       // [DCL_WARPS][16][RED]
  float* red_m = red_o + DCL_WARPS * 16 * RED;         // [DCL_WARPS][16]
  float* red_l = red_m + DCL_WARPS * 16;               // [DCL_WARPS][16]
  const int g0 = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    float* base = red_o + (warp * 16 + g0) * RED + j * 8 + c0;
    *reinterpret_cast<float2*>(base) = make_float2(st.o[j][0], st.o[j][1]);
    *reinterpret_cast<float2*>(base + 8 * RED) = make_float2(st.o[j][2], st.o[j][3]);
  }
  if ((lane & 3) == 0) {
    red_m[warp * 16 + g0] = st.m[0];
    red_m[warp * 16 + g0 + 8] = st.m[1];
    red_l[warp * 16 + g0] = st.l[0];
    red_l[warp * 16 + g0 + 8] = st.l[1];
  }
  __syncthreads();
  cg::cluster_group cluster = cg::this_cluster();
  const int total = groups * HD;
  // pairs a block of the cluster merges: a multiple of four, so that four neighbours go to the same block in one store
  // (a store into another block's shared memory costs a thread hundreds of cycles: few and wide ones)
  const int per_share = (((total + num_splits - 1) / num_splits) + 3) & ~3;
  for (int e = 4 * tid; e < total; e += 4 * DCL_THREADS) {
    const int r = e / HD, d = e - r * HD;  // the pairs e .. e + 3 are coordinates d .. d + 3 of row r
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DCL_WARPS; ++w) m = fmaxf(m, red_m[w * 16 + r]);
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < DCL_WARPS; ++w) {
      const float mw = red_m[w * 16 + r];
      const float f = mw == -INFINITY ? 0.f : ms_exp2(mw - m);
      const float4 ow = *reinterpret_cast<const float4*>(red_o + ((size_t)w * 16 + r) * RED + d);
      o.x += ow.x * f;
      o.y += ow.y * f;
      o.z += ow.z * f;
      o.w += ow.w * f;
      l += red_l[w * 16 + r] * f;
    }
    if (num_splits == 1) {
      if (live) {
        __nv_bfloat16* dst = out + ((size_t)t * hq + kvh * groups + r) * HD + d;
        *reinterpret_cast<uint2*>(dst) = make_uint2(ms_pack_bf16(l > 0.f ? __fdividef(o.x, l) : 0.f, l > 0.f ? __fdividef(o.y, l) : 0.f),
                                                    ms_pack_bf16(l > 0.f ? __fdividef(o.z, l) : 0.f, l > 0.f ? __fdividef(o.w, l) : 0.f));
      }
    } else {
      // to the block that merges these pairs (stores through distributed shared memory: one way, no round trip)
      const int owner = e / per_share;
      *reinterpret_cast<float4*>(cluster.map_shared_rank(gath_o, owner) + split * per_share + (e - owner * per_share)) = o;
      // the row's maximum and sum go to every block: the row's threads share the blocks between them
      for (int k = d / 4; k < num_splits; k += HD / 4) cluster.map_shared_rank(&gath_ml[0][0], k)[split * 16 + r] = make_float2(m, l);
    }
  }
  if (num_splits == 1) return;

  // One cluster barrier makes the stores visible; then every block merges its share of the pairs in rank order from
  // its own shared memory, so the result does not depend on timing, and no block has to outlive another.
  MS_TIMELINE_MARK(2);
  cluster.sync();
  MS_TIMELINE_MARK(3);
  {
    const int e_end = min(total, (split + 1) * per_share);
    for (int e = split * per_share + tid; e < e_end; e += DCL_THREADS) {
      const int r = e / HD, d = e - r * HD;
      float mk[8], lk[8], ok[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const bool in = k < num_splits;
        mk[k] = in ? gath_ml[k][r].x : -INFINITY;
        lk[k] = in ? gath_ml[k][r].y : 0.f;
        ok[k] = in ? gath_o[k * per_share + (e - split * per_share)] : 0.f;
      }
      float m = -INFINITY;
#pragma unroll
      for (int k = 0; k < 8; ++k) m = fmaxf(m, mk[k]);
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float f = mk[k] == -INFINITY ? 0.f : ms_exp2(mk[k] - m);
        l += lk[k] * f;
        o += ok[k] * f;
      }
      if (OUTER) {
        float* mine = outer.scratch + ((size_t)(blockIdx.x * hkv + kvh) * parts + part) * (total + 32);
        __stcg(mine + e, o);
        if (d == 0) {
          __stcg(mine + total + r, m);
          __stcg(mine + total + 16 + r, l);
        }
      } else if (live) {
        out[((size_t)t * hq + kvh * groups + r) * HD + d] = __float2bfloat16_rn(l > 0.f ? __fdividef(o, l) : 0.f);
      }
    }
  }
  MS_TIMELINE_MARK(4);
  if constexpr (!OUTER) return;

  // The cluster's sums are in global memory.  Its first block counts the cluster; the one that counts last merges the
  // parts in their order.
  __shared__ int last_s;
  __threadfence();
  cluster.sync();
  if (split != 0) return;
  int* counter = outer.counters + blockIdx.x * hkv + kvh;
  if (tid == 0) {
    __threadfence();
    last_s = atomicAdd(counter, 1) == parts - 1;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const float* all = outer.scratch + (size_t)(blockIdx.x * hkv + kvh) * parts * (total + 32);
  for (int e = tid; e < total; e += DCL_THREADS) {
    const int r = e / HD;
    float m = -INFINITY;
    for (int k = 0; k < parts; ++k) m = fmaxf(m, __ldcg(all + (size_t)k * (total + 32) + total + r));
    float l = 0.f, o = 0.f;
    for (int k = 0; k < parts; ++k) {
      const float* pk = all + (size_t)k * (total + 32);
      const float mk = __ldcg(pk + total + r);
      const float f = mk == -INFINITY ? 0.f : ms_exp2(mk - m);
      l += __ldcg(pk + total + 16 + r) * f;
      o += __ldcg(pk + e) * f;
    }
    if (live) out[((size_t)t * hq + kvh * groups + r) * HD + (e - r * HD)] = __float2bfloat16_rn(l > 0.f ? __fdividef(o, l) : 0.f);
  }
  if (tid == 0) *counter = 0;
}

static size_t dcl_smem_bytes(int hd, int stages, int DCL_WARPS) {
  const size_t stride = hd + 8;
  const size_t tiles = (16 + (size_t)stages * 2 * DCL_TILE) * stride * sizeof(__nv_bfloat16);
  const size_t red = 16 * stride * sizeof(__nv_bfloat16) + ((size_t)DCL_WARPS * 16 * (hd + 8 + 2) + 16 * hd) * sizeof(float);
  return tiles > red ? tiles : red;
}

template <int HD, bool FUSED, int KPW, int DCL_WARPS, bool OUTER>
static int launch_decode_cluster_k(const void* q, DclRaw raw, const void* k_pages, const void* v_pages, void* out, const int* rows,
                                 const int* positions, const int* slot_of_token, const int* block_table,
                                 int max_pages, int num_pages, int tokens, int hq, int hkv, int page_size, int window,
                                 float scale, int num_splits, int stages, DclOuter outer, cudaStream_t stream) {
  const size_t smem = dcl_smem_bytes(HD, stages, DCL_WARPS);
  auto kern = attention_decode_cluster_kernel<HD, FUSED, KPW, DCL_WARPS, OUTER>;
  static size_t configured = 0;  // per instantiation: the largest size asked for so far
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // the largest shared-memory share of an SM, so that as many blocks as fit are resident at once
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) {
      ms_set_error("attention_decode_cluster: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return 2;
    }
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tokens, hkv, num_splits * outer.parts);
  cfg.blockDim = dim3(DCL_WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (num_splits > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = num_splits;
    ++n;
  }
  if (g_ms_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  MS_LAUNCH_RESULT("attention_decode_cluster",
                   cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)q, raw, (__nv_bfloat16*)k_pages,
                                      (__nv_bfloat16*)v_pages, (__nv_bfloat16*)out, rows, positions, slot_of_token,
                                      block_table, max_pages, num_pages, hq, hkv, page_size, window, scale * MS_LOG2E,
                                      num_splits, stages, outer));
  return 0;
}

// The form of the kernel: blocks that hold at most two tiles give each of four warps half a tile.
template <int HD, bool FUSED>
static int launch_decode_cluster(const void* q, DclRaw raw, const void* k_pages, const void* v_pages, void* out, const int* rows,
                                 const int* positions, const int* slot_of_token, const int* block_table,
                                 int max_pages, int num_pages, int tokens, int hq, int hkv, int page_size, int window,
                                 float scale, int num_splits, int stages, int warps, int kpw, DclOuter outer, cudaStream_t stream) {
  // (several clusters a pair: built for the two common head sizes only)
#define MS_DCL_LAUNCH(KPW, WARPS)                                                                                              \
  do {                                                                                                                         \
    if constexpr (HD == 64 || HD == 128) {                                                                                     \
      if (outer.parts > 1)                                                                                                     \
        return launch_decode_cluster_k<HD, FUSED, KPW, WARPS, true>(q, raw, k_pages, v_pages, out, rows, positions,           \
                                                                    slot_of_token, block_table, max_pages, num_pages, tokens, \
                                                                    hq, hkv, page_size, window, scale, num_splits, stages,    \
                                                                    outer, stream);                                           \
    }                                                                                                                          \
    return launch_decode_cluster_k<HD, FUSED, KPW, WARPS, false>(q, raw, k_pages, v_pages, out, rows, positions,              \
                                                                 slot_of_token, block_table, max_pages, num_pages, tokens,    \
                                                                 hq, hkv, page_size, window, scale, num_splits, stages,       \
                                                                 outer, stream);                                              \
  } while (0)
  // few tiles a round, or wide heads (a long chain of steps per key): smaller parts keep every warp busy
  if (kpw == 0) kpw = warps == 8 ? 32 : HD > 64 ? 16 : stages <= 4 ? 32 : 64;
  if (warps == 8 && kpw == 64) kpw = 32;
  if (warps == 8 && kpw == 16) MS_DCL_LAUNCH(16, 8);
  if (warps == 8) MS_DCL_LAUNCH(32, 8);
  if (kpw == 16) MS_DCL_LAUNCH(16, 4);
  if (kpw == 32) MS_DCL_LAUNCH(32, 4);
  MS_DCL_LAUNCH(64, 4);
#undef MS_DCL_LAUNCH
}

// The most tiles a block can hold at once for a head size (about 100 KB of shared memory, which leaves room on the SM
// for the blocks of the kernels that follow: they request their weights early).
static int dcl_max_stages(int hd) {
  int s = (int)((100 * 1024) / ((size_t)2 * DCL_TILE * (hd + 8) * sizeof(__nv_bfloat16)));
  return s < 1 ? 1 : (s > 8 ? 8 : s);
}

template <bool FUSED>
static int decode_cluster_dispatch(const void* q, const DclRaw* raw, void* k_pages, void* v_pages, void* out,
                                   const int* rows, const int* positions, const int* slot_of_token,
                                   const int* block_table, int max_pages, int num_pages, int tokens, int hq, int hkv,
                                   int hd, int page_size, int window, float scale, int num_splits, int stages,
                                   int warps, int kpw, int parts, float* scratch, long long scratch_words, int* counters,
                                   int num_counters, cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(parts >= 1 && parts <= DCL_MAX_PARTS, "attention_decode_cluster: %d clusters a pair; 1 to %d", parts, DCL_MAX_PARTS);
  if (parts > 1) {
    const long long need = (long long)tokens * hkv * parts * ((hq / (hkv > 0 ? hkv : 1)) * hd + 32);
    MS_REQUIRE(num_splits > 1, "attention_decode_cluster: several clusters a pair need clusters of more than one block");
    MS_REQUIRE(hd == 64 || hd == 128, "attention_decode_cluster: several clusters a pair are built for head sizes 64 and 128, not %d", hd);
    MS_REQUIRE(scratch != nullptr && counters != nullptr && scratch_words >= need && num_counters >= tokens * hkv,
               "attention_decode_cluster: %d clusters a pair need %lld words of scratch and %d counters; %lld and %d were given",
               parts, need, tokens * hkv, scratch ? scratch_words : 0LL, counters ? num_counters : 0);
  }
  const DclOuter outer = {parts, scratch, counters};
  MS_REQUIRE(warps == 4 || warps == 8, "attention_decode_cluster: 4 or 8 warps a block, not %d", warps);
  MS_REQUIRE(kpw == 0 || kpw == 16 || kpw == 32 || kpw == 64, "attention_decode_cluster: a warp takes 16, 32 or 64 keys at a time (0: by rule), not %d", kpw);
  MS_REQUIRE(tokens > 0 && hq > 0 && hkv > 0 && hq % hkv == 0 && hkv <= 65535, "attention_decode_cluster: bad head counts hq=%d hkv=%d", hq, hkv);
  MS_REQUIRE(hd % 16 == 0 && hd >= 16 && hd <= 128 && hq / hkv <= 16,
             "attention_decode_cluster: head_dim %d (multiples of 16 up to 128) or group size %d (up to 16) is not covered", hd, hq / hkv);
  MS_REQUIRE(num_splits == 1 || num_splits == 2 || num_splits == 4 || num_splits == 8,
             "attention_decode_cluster: %d splits; a cluster holds 1, 2, 4 or 8", num_splits);
  MS_REQUIRE(stages >= 1 && stages <= dcl_max_stages(hd), "attention_decode_cluster: %d stages is outside 1..%d for head_dim %d",
             stages, dcl_max_stages(hd), hd);
  MS_REQUIRE(page_size > 0 && max_pages > 0 && num_pages > 0, "attention_decode_cluster: bad cache sizes");
  const DclRaw none = {nullptr, 0, nullptr, nullptr, 0};
#define MS_DCL_CASE(N)                                                                                              \
  case N:                                                                                                           \
    return launch_decode_cluster<N, FUSED>(q, FUSED ? *raw : none, k_pages, v_pages, out, rows, positions, slot_of_token, \
                                           block_table, max_pages, num_pages, tokens, hq, hkv, page_size, window, scale, \
                                           num_splits, stages, warps, kpw, outer, stream)
  switch (hd) {
    MS_DCL_CASE(16);
    MS_DCL_CASE(32);
    MS_DCL_CASE(48);
    MS_DCL_CASE(64);
    MS_DCL_CASE(80);
    MS_DCL_CASE(96);
    MS_DCL_CASE(112);
    MS_DCL_CASE(128);
  }
#undef MS_DCL_CASE
  MS_REQUIRE(false, "attention_decode_cluster: head_dim %d", hd);
  return 1;
}
