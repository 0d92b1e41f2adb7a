// Paged causal attention for portions of prompts on the fifth-generation tensor cores.
//
// One block per (tile of up to 128 consecutive query rows of one sequence, query head).  Per tile
// of 128 keys:
//   S = Q K^T        tcgen05.mma, Q [128 x hd] and K [128 x hd] K-major in shared memory (TMA, 128-byte
//                    swizzle), S [128 x 128] float32 in tensor memory;
//   softmax          128 threads, one per query row: the whole row of S comes into registers with one round
//                    of tcgen05.ld (tensor memory is then free for the next tile's scores, which the tensor
//                    core computes meanwhile); scale, mask, maximum, 2^x and sum in float32 without any
//                    exchange between threads; the probabilities go to shared memory as bfloat16 in the
//                    swizzled K-major layout;
//   O += P V         tcgen05.mma, V [128 keys x hd] as it lies in the cache (MN-major), O [128 x hd] float32
//                    accumulated in tensor memory over all tiles.
// The probabilities of a row are 2^(s - m) with a reference m that is the row's maximum at some earlier tile:
// m moves to the row's new maximum only when that exceeds it by more than 8 (a probability never exceeds
// 2^8), and only then is the row of O in tensor memory multiplied by 2^(m_old - m_new) (tcgen05.ld, multiply,
// tcgen05.st) before the tile's P V is issued.  So the softmax threads never wait for the product they feed,
// except for the shared-memory tile of P to be free again.  The row's sum follows the same reference; the
// output is O / sum at the end.
// Warp 4 (one thread) drives TMA: Q once, then K and V tiles, page by page through the block table.  Warp 5
// (one thread) issues the matrix instructions.  Warps 0-3 are the softmax threads.
// Every mbarrier wait is bounded (error code for the host, see ms_attention_tc_status); no load uses cluster
// multicast.  Head sizes 64 and 128, page sizes that are powers of two from 8; everything else goes to the
// mma.sync kernel (attention_prefill.cu), which computes the same thing.
//
// The reference's counterpart is a SIMT kernel (attn_paged_tiled_f16_gqa_runs,
// crates/mach-model/src/kernels.rs:1650-1890 of gqf2008/machserve).
#include <cuda.h>

#include "common.cuh"

#define ATC_ROWS 128
#define ATC_KEYS 128
#define ATC_THREADS 192       // one head per block: four softmax warps, a copying warp, an issuing warp
#define ATC_PAIR_THREADS 320  // two heads per block: two groups of four softmax warps, a copying warp, an issuing warp
#define ATC_WAIT_LIMIT (1 << 21)
#define ATC_LOG2E 1.4426950408889634f

__device__ int g_atc_error = 0;  // 0, or which bounded wait gave up: 11 producer, 12-14, 16 issuer, 15 softmax threads

__device__ __forceinline__ unsigned atc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void atc_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void atc_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void atc_mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool atc_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete, at most `limit` polls.  Returns false when it gave
// up (then the block's abort flag and the device's error word are set) or when another thread of the block has.
__device__ __forceinline__ bool atc_mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int code,
                                              int limit = ATC_WAIT_LIMIT) {
  for (int it = 0; it < limit; ++it) {
    if (atc_mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (it > 256) __nanosleep(40);
  }
  *abort_flag = 1;
  atomicCAS(&g_atc_error, 0, code);
  return false;
}
__device__ __forceinline__ void atc_tma_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// K-major tile of 128-byte rows, 128-byte swizzle: 1024 bytes between groups of eight rows
__device__ __forceinline__ unsigned long long atc_desc(unsigned addr) {
  return (unsigned long long)((addr & 0x3FFFF) >> 4) | ((unsigned long long)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// float32 accumulator, bfloat16 operands, M x N; b_mn: the second operand is MN-major
__device__ __forceinline__ unsigned atc_idesc(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void atc_mma(unsigned tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                        unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the first operand in tensor memory: 128 lanes (rows) by 8 columns of two packed bfloat16 each
// per 16 steps of k.
__device__ __forceinline__ void atc_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc,
                                           unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void atc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void atc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void atc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
#define ATC_R32(M, r) \
  M(r[0]), M(r[1]), M(r[2]), M(r[3]), M(r[4]), M(r[5]), M(r[6]), M(r[7]), M(r[8]), M(r[9]), M(r[10]), M(r[11]), M(r[12]), \
      M(r[13]), M(r[14]), M(r[15]), M(r[16]), M(r[17]), M(r[18]), M(r[19]), M(r[20]), M(r[21]), M(r[22]), M(r[23]), M(r[24]), \
      M(r[25]), M(r[26]), M(r[27]), M(r[28]), M(r[29]), M(r[30]), M(r[31])
#define ATC_OUT(x) "=r"(x)
#define ATC_IN(x) "r"(x)
#define ATC_REGS32 \
  "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}"
// 32 consecutive columns of this thread's lane of tensor memory; the registers hold them after atc_wait_ld()
__device__ __forceinline__ void atc_ld32_issue(unsigned taddr, unsigned* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 " ATC_REGS32 ", [%32];\n" : ATC_R32(ATC_OUT, r) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void atc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void atc_st32(unsigned taddr, const unsigned* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], " ATC_REGS32 ";\n" ::ATC_R32(ATC_IN, r), "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float atc_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float atc_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two float32 in one 64-bit register pair, for the instructions that work on both at once.  The softmax
// threads are bound by the number of instructions they issue, so the scale-and-subtract and the sum of a
// row's probabilities take two elements per instruction, and the maximum three.
__device__ __forceinline__ unsigned long long atc_pack(float lo, float hi) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void atc_unpack(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long atc_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long atc_add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// The maximum of a row of 128 raw scores.  INSIDE: every key of the tile is visible to the row; else the keys
// rlo..rhi of the tile are (an empty range gives -inf).
template <bool INSIDE>
__device__ __forceinline__ float atc_row_max(const unsigned (&r)[ATC_KEYS], int rlo, int rhi) {
  float a[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  if (INSIDE) {
#pragma unroll
    for (int i = 0; i < ATC_KEYS; i += 2) a[(i >> 1) & 3] = atc_max3(a[(i >> 1) & 3], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
  } else {
#pragma unroll
    for (int i = 0; i < ATC_KEYS; ++i) a[i & 3] = fmaxf(a[i & 3], (i >= rlo && i <= rhi) ? __uint_as_float(r[i]) : -INFINITY);
  }
  return fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
}
// The probabilities 2^(s*scale_log2 - mu) of one half of a row (keys 64*HALF .. 64*HALF+63), rounded to bfloat16
// and packed in pairs back into the registers of scores already used (r[i / 2] for keys i, i + 1), as they go to
// tensor memory; their float32 sums are added to sum2 (two pairs).
template <bool INSIDE, int HALF>
__device__ __forceinline__ void atc_row_probs(unsigned (&r)[ATC_KEYS], int rlo, int rhi, float scale_log2, float mu,
                                              unsigned long long (&sum2)[2]) {
  const unsigned long long scale2 = atc_pack(scale_log2, scale_log2), nmu2 = atc_pack(-mu, -mu);
#pragma unroll
  for (int j = 0; j < 8; ++j) {  // 8 probabilities at a time
    float p[8];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const int i = HALF * 64 + j * 8 + e;
      float x0, x1;
      atc_unpack(atc_fma2(atc_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2, nmu2), x0, x1);
      p[e] = (INSIDE || (i >= rlo && i <= rhi)) ? atc_exp2(x0) : 0.f;
      p[e + 1] = (INSIDE || (i + 1 >= rlo && i + 1 <= rhi)) ? atc_exp2(x1) : 0.f;
      sum2[(e >> 1) & 1] = atc_add2(sum2[(e >> 1) & 1], atc_pack(p[e], p[e + 1]));
    }
    const int w = (HALF * 64 + j * 8) >> 1;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat162 h2 = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
      r[w + e] = *reinterpret_cast<unsigned*>(&h2);
    }
  }
}


#define ATC_MAX_SPLITS 4
// What a split of an item (a tile of rows with one head) leaves in scratch memory: HD columns of O, then the
// reference of the exponents m and the sum l, each as 128 consecutive rows.
#define ATC_SPLIT_WORDS(HD) (((HD) + 2) * ATC_ROWS)

// The end of a block's key tiles for the 128 rows of one head (one thread per row; the four warps of a softmax
// group call it together).  With one split, out = O / l.  When the item's keys are split over several blocks, the
// block leaves (O, m, l) in scratch memory and counts itself; the block that counts last merges all splits in
// split order (so the result does not depend on who came last), writes the output and clears the counter.
// No block waits for another.
template <int HD>
__device__ __forceinline__ void atc_finish(unsigned tmem_o_lane, bool have_o, float m, float l, int row, int nrows,
                                           __nv_bfloat16* dst, int nsplit, int split, float* item_scratch, int* counter,
                                           int bar_id, volatile int* last_flag) {
  if (nsplit <= 1) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int c = 0; c < HD; c += 32) {
      unsigned v[32];
      if (have_o) {
        atc_ld32_issue(tmem_o_lane + c, v);
        atc_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (row < nrows) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 u;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            hh[e] = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 2 * e]) * inv, __uint_as_float(v[j * 8 + 2 * e + 1]) * inv);
          *reinterpret_cast<uint4*>(dst + c + j * 8) = u;
        }
      }
    }
    return;
  }
  float* mine = item_scratch + (size_t)split * ATC_SPLIT_WORDS(HD);
#pragma unroll
  for (int c = 0; c < HD; c += 32) {
    unsigned v[32];
    if (have_o) {
      atc_ld32_issue(tmem_o_lane + c, v);
      atc_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0u;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) __stcg(mine + (size_t)(c + i) * ATC_ROWS + row, __uint_as_float(v[i]));
  }
  __stcg(mine + (size_t)HD * ATC_ROWS + row, m);
  __stcg(mine + (size_t)(HD + 1) * ATC_ROWS + row, l);
  __threadfence();
  asm volatile("bar.sync %0, 128;\n" ::"r"(bar_id) : "memory");
  if (row == 0) *last_flag = atomicAdd(counter, 1) == nsplit - 1;
  asm volatile("bar.sync %0, 128;\n" ::"r"(bar_id) : "memory");
  if (!*last_flag) return;
  __threadfence();
  float ms[ATC_MAX_SPLITS], w[ATC_MAX_SPLITS];
  float top = -INFINITY;
#pragma unroll
  for (int s = 0; s < ATC_MAX_SPLITS; ++s) {
    ms[s] = s < nsplit ? __ldcg(item_scratch + (size_t)s * ATC_SPLIT_WORDS(HD) + (size_t)HD * ATC_ROWS + row) : -INFINITY;
    top = fmaxf(top, ms[s]);
  }
  float sum = 0.f;
#pragma unroll
  for (int s = 0; s < ATC_MAX_SPLITS; ++s) {
    const float ls = s < nsplit ? __ldcg(item_scratch + (size_t)s * ATC_SPLIT_WORDS(HD) + (size_t)(HD + 1) * ATC_ROWS + row) : 0.f;
    w[s] = ls > 0.f ? atc_exp2(ms[s] - top) : 0.f;
    sum += ls * w[s];
  }
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  if (row < nrows) {
    // 32 columns at a time: all splits' values of them are requested together (a round trip to the L2 per chunk)
#pragma unroll 1
    for (int c = 0; c < HD; c += 32) {
      float o[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = 0.f;
#pragma unroll
      for (int s = 0; s < ATC_MAX_SPLITS; ++s)
        if (s < nsplit) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            o[e] += w[s] * __ldcg(item_scratch + (size_t)s * ATC_SPLIT_WORDS(HD) + (size_t)(c + e) * ATC_ROWS + row);
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u;
        __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(o[j * 8 + 2 * e] * inv, o[j * 8 + 2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(dst + c + j * 8) = u;
      }
    }
  }
  if (row == 0) *counter = 0;
}

struct AtcShared {
  unsigned long long q_full, k_full, k_empty, v_full[2], v_empty[2], s_full, s_free, p_full, o_full;
  unsigned tmem_base;
  int abort_flag;
  int last_flag;
  volatile int group_bad;
};

// One head per block, for head size 64.  Shared memory: [AtcShared, 1 KB][Q: a panel of 16 KB][V stage 0, 1][K]; a
// panel is 128 rows of 128 bytes.  Keys have one stage (the next tile's keys are copied while the softmax of this
// one runs), values two.  That is 66 KB and 256 columns of tensor memory (S 128, O 64, P 64 as packed pairs), so two
// blocks share an SM and one's softmax overlaps the other's.  The value tiles are not last: the tensor core's fetch of an MN-major operand was
// seen to reach past the tile it is given.
template <int HD>
__global__ void __launch_bounds__(ATC_THREADS, 2)
attention_prefill_tc_single_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                            const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                            const int* __restrict__ block_table, int max_pages, int num_pages, int hq, int hkv,
                            int page_size, int window, float scale_log2, int num_runs, int run_tiles, float* __restrict__ scratch,
                            int* __restrict__ counters) {
  constexpr int PANELS = HD / 64;          // 64-column panels of Q, K and V
  constexpr int PANEL_BYTES = 128 * 128;   // 128 rows of 128 bytes
  constexpr int KV_BYTES = PANELS * PANEL_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  AtcShared* sh = reinterpret_cast<AtcShared*>(base);
  unsigned char* q_s = base + 1024;
  unsigned char* v_s = q_s + KV_BYTES;       // two stages
  unsigned char* k_s = v_s + 2 * KV_BYTES;   // one stage
  volatile int* abort_flag = &sh->abort_flag;

  // blocks are handed out in the order of blockIdx.x, then .y: the heads of the last tile's first run of keys, the
  // heads of its second run, ..., then the tile before it: the longest rows of key tiles first, their runs together
  const int nruns = num_runs;
  const int tile_id = (int)(gridDim.y / nruns) - 1 - (int)(blockIdx.y / nruns);
  const int row0 = tile_row0[tile_id], nrows = tile_rows[tile_id];
  const int h = blockIdx.x, kvh = h / (hq / hkv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = slot_of_token[row0];
  const int pos0 = positions[row0];
  const int pos_last = pos0 + nrows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int item_lo = first_key / ATC_KEYS, tile_hi = pos_last / ATC_KEYS;
  const int item_tiles = (slot >= 0 && nrows > 0) ? tile_hi - item_lo + 1 : 0;
  // the item's key tiles in runs of equal length for different blocks: `num_runs` of them, or (run_tiles > 0) as many as
  // keep a run at `run_tiles` tiles at most, so that only long items are cut; blocks past the last run have nothing to do
  const int want = run_tiles > 0 ? min(nruns, max(1, (item_tiles + run_tiles - 1) / run_tiles)) : nruns;
  const int chunk = (item_tiles + want - 1) / want;
  const int nsplit = chunk > 0 ? (item_tiles + chunk - 1) / chunk : 1;
  const int split = blockIdx.y % nruns;
  const bool active = split < nsplit;
  const int tile_lo = item_lo + split * chunk;
  const int ntiles = (active && chunk > 0) ? min(chunk, item_tiles - split * chunk) : 0;
  const int* table = block_table + (size_t)(slot >= 0 ? slot : 0) * max_pages;

  // the copying thread sets the barriers up and sends for the query tile at once (nothing else lies there), while the
  // others clear the stages and tensor memory is taken
  if (warp == 4 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
    atc_mbar_init(atc_smem(&sh->q_full), 1);
    atc_mbar_init(atc_smem(&sh->k_full), 1);
    atc_mbar_init(atc_smem(&sh->k_empty), 1);
    for (int s = 0; s < 2; ++s) {
      atc_mbar_init(atc_smem(&sh->v_full[s]), 1);
      atc_mbar_init(atc_smem(&sh->v_empty[s]), 1);
    }
    atc_mbar_init(atc_smem(&sh->s_full), 1);
    atc_mbar_init(atc_smem(&sh->s_free), ATC_ROWS);
    atc_mbar_init(atc_smem(&sh->p_full), ATC_ROWS);
    atc_mbar_init(atc_smem(&sh->o_full), 1);
    sh->abort_flag = 0;
    sh->group_bad = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (ntiles > 0) {
      atc_mbar_expect_tx(atc_smem(&sh->q_full), KV_BYTES);
      for (int p = 0; p < PANELS; ++p) atc_tma_2d(atc_smem(q_s + p * PANEL_BYTES), &map_q, h * HD + p * 64, row0, atc_smem(&sh->q_full));
    }
  }
  // the key and value stages start as zeros: rows that no page holds are never copied, and what multiplies a
  // probability of zero must be finite
  for (int i = tid; i < 3 * KV_BYTES / 16; i += ATC_THREADS) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(atc_smem(&sh->tmem_base)), "r"(256)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  atc_fence_before();
  __syncthreads();
  atc_fence_after();
  const unsigned tmem = sh->tmem_base;
  const unsigned tmem_s = tmem, tmem_o = tmem + 128;  // columns 0..127: S; 128..128+HD-1: O
  const unsigned tmem_p = tmem + 192;                 // 64 columns of packed bfloat16 P

  if (warp == 4 && lane == 0) {
    // ------------------------------------------------------------------ producer (the query tile is on its way)
    // One thread does all of this next to the softmax warps, so every instruction counts: the page size is a
    // power of two (shifts and masks, no division), and the keys go out before anything else is looked at.
    const int box = page_size < ATC_KEYS ? page_size : ATC_KEYS;  // rows one copy brings
    const int page_shift = __ffs(page_size) - 1, page_mask = page_size - 1;
    const unsigned copy_bytes = (unsigned)PANELS * box * 128;
    for (int t = 0; t < ntiles; ++t) {
      const int s = t & 1;
      const int key0 = (tile_lo + t) * ATC_KEYS;
      // which copies will be made: pages the table holds, inside the keys the tile's rows can see
      unsigned bytes = 0;
      for (int r = 0; r < ATC_KEYS; r += box) {
        const int key = key0 + r;
        if (key > pos_last || key + box - 1 < first_key) continue;
        const int page = table[key >> page_shift];
        if (page >= 0 && page < num_pages) bytes += copy_bytes;
      }
      // keys: one stage, free again when the scores of the tile before are done.  They go first and do not
      // wait for the value stage: the scores of tile t are wanted a whole tile before its values are
      if (t >= 1 && !atc_mbar_wait(atc_smem(&sh->k_empty), (t - 1) & 1, abort_flag, 11)) break;
      atc_mbar_expect_tx(atc_smem(&sh->k_full), bytes);
      for (int r = 0; r < ATC_KEYS; r += box) {
        const int key = key0 + r;
        if (key > pos_last || key + box - 1 < first_key) continue;
        const int page = table[key >> page_shift];
        if (page < 0 || page >= num_pages) continue;
        const int grow = (page * hkv + kvh) * page_size + (key & page_mask);  // row of the [pages*kv_heads*page, hd] view
#pragma unroll
        for (int p = 0; p < PANELS; ++p) atc_tma_2d(atc_smem(k_s + p * PANEL_BYTES + r * 128), &map_k, p * 64, grow, atc_smem(&sh->k_full));
      }
      // values: two stages
      if (t >= 2 && !atc_mbar_wait(atc_smem(&sh->v_empty[s]), ((t >> 1) - 1) & 1, abort_flag, 11)) break;
      atc_mbar_expect_tx(atc_smem(&sh->v_full[s]), bytes);
      for (int r = 0; r < ATC_KEYS; r += box) {
        const int key = key0 + r;
        if (key > pos_last || key + box - 1 < first_key) continue;
        const int page = table[key >> page_shift];
        if (page < 0 || page >= num_pages) continue;
        const int grow = (page * hkv + kvh) * page_size + (key & page_mask);
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          atc_tma_2d(atc_smem(v_s + s * KV_BYTES + p * PANEL_BYTES + r * 128), &map_v, p * 64, grow, atc_smem(&sh->v_full[s]));
      }
    }
  } else if (warp == 5 && lane == 0) {
    // -------------------------------------------------------------------- issuer
    bool ok = ntiles == 0 || atc_mbar_wait(atc_smem(&sh->q_full), 0, abort_flag, 12);
    const unsigned idesc_s = atc_idesc(ATC_ROWS, ATC_KEYS, false);
    const unsigned idesc_o = atc_idesc(ATC_ROWS, 64, true);
    // the descriptors once; an offset of b bytes inside a tile adds b / 16 to the address field
    const unsigned long long desc_q = atc_desc(atc_smem(q_s)), desc_k = atc_desc(atc_smem(k_s));
    const unsigned long long desc_v0 = atc_desc(atc_smem(v_s)), desc_v1 = atc_desc(atc_smem(v_s + KV_BYTES));
    // O += P V of tile j over its 128 keys in steps of 16; one instruction per 64 columns of hd
    auto issue_pv = [&](int j) -> bool {
      const int s = j & 1;
      const unsigned long long desc_v = s ? desc_v1 : desc_v0;
      if (!atc_mbar_wait(atc_smem(&sh->p_full), j & 1, abort_flag, 14) ||
          !atc_mbar_wait(atc_smem(&sh->v_full[s]), (j >> 1) & 1, abort_flag, 14))
        return false;
      atc_fence_after();
#pragma unroll
      for (int k = 0; k < ATC_KEYS / 16; ++k) {
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          atc_mma_ts(tmem_o + p * 64, tmem_p + k * 8, desc_v + ((p * PANEL_BYTES + k * 2048) >> 4), idesc_o,
                     (j > 0 || k != 0) ? 1u : 0u);  // 16 keys = 8 columns of packed pairs
      }
      atc_commit(atc_smem(&sh->v_empty[s]));
      atc_commit(atc_smem(&sh->o_full));
      return true;
    };
    for (int t = 0; t < ntiles && ok; ++t) {
      ok = atc_mbar_wait(atc_smem(&sh->k_full), t & 1, abort_flag, 13);
      // the scores of the tile before have left tensor memory for the softmax threads' registers
      if (ok && t >= 1) ok = atc_mbar_wait(atc_smem(&sh->s_free), (t - 1) & 1, abort_flag, 16);
      if (!ok) break;
      atc_fence_after();
      // S = Q K^T over hd in steps of 16 (four steps per 64-column panel)
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        const unsigned off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
        atc_mma(tmem_s, desc_q + (off >> 4), desc_k + (off >> 4), idesc_s, k != 0);
      }
      atc_commit(atc_smem(&sh->k_empty));
      atc_commit(atc_smem(&sh->s_full));
      // the product of the tile before follows the scores of this one: its probabilities are written while
      // these scores are computed
      if (t >= 1) ok = issue_pv(t - 1);
    }
    if (ok && ntiles > 0) issue_pv(ntiles - 1);
  } else if (warp < 4) {
    // ------------------------------------------------------------ softmax threads
    const int row = tid;  // accumulator lane = query row of the tile
    const int pos = pos0 + row;
    const int hi = row < nrows ? pos : -1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const unsigned lane_addr = (unsigned)(warp * 32) << 16;
    float m = -INFINITY, l = 0.f;  // the reference of the row's exponents, the sum of its probabilities
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      ok = atc_mbar_wait(atc_smem(&sh->s_full), t & 1, abort_flag, 15);
      if (!ok) break;
      atc_fence_after();
      unsigned r[ATC_KEYS];
#pragma unroll
      for (int c = 0; c < ATC_KEYS; c += 32) atc_ld32_issue(tmem_s + lane_addr + c, r + c);
      atc_wait_ld();
      atc_fence_before();
      atc_mbar_arrive(atc_smem(&sh->s_free));
      const int key0 = (tile_lo + t) * ATC_KEYS;
      const int rlo = lo - key0, rhi = hi - key0;
      // whether every row of this warp sees the whole tile: the same for the whole warp, which keeps the
      // warp-wide tensor memory instructions below out of divergent code
      const bool inside = __all_sync(0xffffffffu, rlo <= 0 && rhi >= ATC_KEYS - 1);
      const float mx = (inside ? atc_row_max<true>(r, rlo, rhi) : atc_row_max<false>(r, rlo, rhi)) * scale_log2;
      // the reference moves only when the maximum has grown by more than 8; a row that has seen no key yet
      // (m = -inf) has nothing in O to rescale
      const bool grow = mx > m + 8.f;
      const float corr = grow ? atc_exp2(m - mx) : 1.f;
      const bool rescale = __any_sync(0xffffffffu, grow && m != -INFINITY);
      m = grow ? mx : m;
      const float mu = m == -INFINITY ? 0.f : m;
      // P V of the tile before is done: the tile of P is free and O is complete up to that tile
      if (t >= 1) {
        ok = atc_mbar_wait(atc_smem(&sh->o_full), (t - 1) & 1, abort_flag, 15);
        if (!ok) break;
        atc_fence_after();
      }
      unsigned long long sum2[2] = {atc_pack(0.f, 0.f), atc_pack(0.f, 0.f)};
      if (inside) {
        atc_row_probs<true, 0>(r, rlo, rhi, scale_log2, mu, sum2);
        atc_row_probs<true, 1>(r, rlo, rhi, scale_log2, mu, sum2);
      } else {
        atc_row_probs<false, 0>(r, rlo, rhi, scale_log2, mu, sum2);
        atc_row_probs<false, 1>(r, rlo, rhi, scale_log2, mu, sum2);
      }
      float s0, s1, s2, s3;
      atc_unpack(sum2[0], s0, s1);
      atc_unpack(sum2[1], s2, s3);
      l = l * corr + ((s0 + s1) + (s2 + s3));
      if (rescale) {
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          unsigned v[32];
          atc_ld32_issue(tmem_o + lane_addr + c, v);
          atc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          atc_st32(tmem_o + lane_addr + c, v);
        }
        atc_fence_before();
      }
      atc_st32(tmem_p + lane_addr, r);  // the row of P, two bfloat16 to a column
      atc_st32(tmem_p + lane_addr + 32, r + 32);
      atc_fence_before();
      atc_mbar_arrive(atc_smem(&sh->p_full));
    }
    if (ok && ntiles > 0) {
      ok = atc_mbar_wait(atc_smem(&sh->o_full), (ntiles - 1) & 1, abort_flag, 15);
      atc_fence_after();
    }
    // whether the whole group got through: decided behind a barrier that all of its 128 threads reach whatever
    // happened, so that the barriers inside atc_finish are reached by all of them or by none
    if (!ok) sh->group_bad = 1;
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (!sh->group_bad && active) {
      const size_t item = (size_t)tile_id * hq + h;
      atc_finish<HD>(tmem_o + lane_addr, ntiles > 0, m, l, row, nrows, out + ((size_t)(row0 + row) * hq + h) * HD, nsplit, split,
                     scratch + item * nruns * ATC_SPLIT_WORDS(HD), counters + item, 1, &sh->last_flag);
      atc_fence_before();
    }
  }
  atc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(256) : "memory");
}


struct AtcPairShared {
  unsigned long long q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_done;
  unsigned tmem_base;
  int abort_flag;
  int last_flag[2];
  volatile int group_bad[2];
};

// Shared memory: [AtcShared, 1 KB][Q of head A][Q of head B][V stage 0, 1][K stage 0, 1]; a tile is HD/64 panels
// of 128 rows of 128 bytes.  The value tiles are not last: the tensor core's fetch of an MN-major operand was
// seen to reach past the tile it is given.  Tensor memory (all 512 columns, so one block per SM): S of head A
// in columns 0..127, S of head B in 128..255, O of head A from 256, O of head B from 384; the probabilities of a
// head, packed two bfloat16 to a column, take the place of the first 64 columns of its scores.
template <int HD>
__global__ void __launch_bounds__(ATC_PAIR_THREADS, 1)
attention_prefill_tc_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                            const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                            const int* __restrict__ block_table, int max_pages, int num_pages, int hq, int hkv,
                            int page_size, int window, float scale_log2, int num_runs, int run_tiles, int alone, float* __restrict__ scratch,
                            int* __restrict__ counters) {
  constexpr int PANELS = HD / 64;          // 64-column panels of Q, K and V
  constexpr int PANEL_BYTES = 128 * 128;   // 128 rows of 128 bytes
  constexpr int KV_BYTES = PANELS * PANEL_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  AtcPairShared* sh = reinterpret_cast<AtcPairShared*>(base);
  unsigned char* q_s = base + 1024;          // head A, head B
  unsigned char* v_s = q_s + 2 * KV_BYTES;   // two stages
  unsigned char* k_s = v_s + 2 * KV_BYTES;   // two stages
  volatile int* abort_flag = &sh->abort_flag;

  // blocks are handed out in the order of blockIdx.x, then .y: the head pairs of the last tile's first run of keys,
  // those of its second run, ..., then the tile before it: the longest rows of key tiles first, their runs together
  const int nruns = num_runs;
  const int tile_id = (int)(gridDim.y / nruns) - 1 - (int)(blockIdx.y / nruns);
  const int row0 = tile_row0[tile_id], nrows = tile_rows[tile_id];
  // `alone`: every block takes one head (launches of few blocks: twice as many of half the length)
  const int groups = hq / hkv, pairs = alone ? groups : (groups + 1) >> 1;
  const int kvh = blockIdx.x / pairs, pair = blockIdx.x - kvh * pairs;
  const int head_a = kvh * groups + (alone ? pair : 2 * pair);
  const bool has_b = !alone && 2 * pair + 1 < groups;  // a group of an odd number of heads leaves its last head alone
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = slot_of_token[row0];
  const int pos0 = positions[row0];
  const int pos_last = pos0 + nrows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int item_lo = first_key / ATC_KEYS, tile_hi = pos_last / ATC_KEYS;
  const int item_tiles = (slot >= 0 && nrows > 0) ? tile_hi - item_lo + 1 : 0;
  // the item's key tiles in runs of equal length for different blocks: `num_runs` of them, or (run_tiles > 0) as many as
  // keep a run at `run_tiles` tiles at most, so that only long items are cut; blocks past the last run have nothing to do
  const int want = run_tiles > 0 ? min(nruns, max(1, (item_tiles + run_tiles - 1) / run_tiles)) : nruns;
  const int chunk = (item_tiles + want - 1) / want;
  const int nsplit = chunk > 0 ? (item_tiles + chunk - 1) / chunk : 1;
  const int split = blockIdx.y % nruns;
  const bool active = split < nsplit;
  const int tile_lo = item_lo + split * chunk;
  const int ntiles = (active && chunk > 0) ? min(chunk, item_tiles - split * chunk) : 0;
  const int* table = block_table + (size_t)(slot >= 0 ? slot : 0) * max_pages;

  // the copying thread sets the barriers up and sends for the query tiles at once (nothing else lies there), while the
  // others clear the stages and tensor memory is taken
  if (warp == 8 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
    atc_mbar_init(atc_smem(&sh->q_full), 1);
    for (int s = 0; s < 2; ++s) {
      atc_mbar_init(atc_smem(&sh->k_full[s]), 1);
      atc_mbar_init(atc_smem(&sh->k_empty[s]), 1);
      atc_mbar_init(atc_smem(&sh->v_full[s]), 1);
      atc_mbar_init(atc_smem(&sh->v_empty[s]), 1);
      atc_mbar_init(atc_smem(&sh->s_full[s]), 1);
      atc_mbar_init(atc_smem(&sh->p_full[s]), ATC_ROWS);
    }
    atc_mbar_init(atc_smem(&sh->o_done), 1);
    sh->abort_flag = 0;
    sh->group_bad[0] = sh->group_bad[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if (ntiles > 0) {
      atc_mbar_expect_tx(atc_smem(&sh->q_full), (has_b ? 2 : 1) * KV_BYTES);
      for (int x = 0; x < (has_b ? 2 : 1); ++x)
        for (int p = 0; p < PANELS; ++p)
          atc_tma_2d(atc_smem(q_s + x * KV_BYTES + p * PANEL_BYTES), &map_q, (head_a + x) * HD + p * 64, row0, atc_smem(&sh->q_full));
    }
  }
  // the key and value stages start as zeros: rows that no page holds are never copied, and what multiplies a
  // probability of zero must be finite
  for (int i = tid; i < 4 * KV_BYTES / 16; i += ATC_PAIR_THREADS) reinterpret_cast<uint4*>(v_s)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(atc_smem(&sh->tmem_base)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  atc_fence_before();
  __syncthreads();
  atc_fence_after();
  const unsigned tmem = sh->tmem_base;

  if (warp == 8 && lane == 0) {
    // ------------------------------------------------------------------ producer (the query tiles are on their way)
    // One thread does all of this next to the softmax warps, so every instruction counts: the page size is a
    // power of two (shifts and masks, no division), and the keys go out before anything else is looked at.
    const int box = page_size < ATC_KEYS ? page_size : ATC_KEYS;  // rows one copy brings
    const int page_shift = __ffs(page_size) - 1, page_mask = page_size - 1;
    const unsigned copy_bytes = (unsigned)PANELS * box * 128;
    for (int t = 0; t < ntiles; ++t) {
      const int s = t & 1;
      const int key0 = (tile_lo + t) * ATC_KEYS;
      // which copies will be made: pages the table holds, inside the keys the tile's rows can see
      unsigned bytes = 0;
      for (int r = 0; r < ATC_KEYS; r += box) {
        const int key = key0 + r;
        if (key > pos_last || key + box - 1 < first_key) continue;
        const int page = table[key >> page_shift];
        if (page >= 0 && page < num_pages) bytes += copy_bytes;
      }
      // keys first: the scores of tile t are wanted a whole tile before its values are
      if (t >= 2 && !atc_mbar_wait(atc_smem(&sh->k_empty[s]), ((t >> 1) - 1) & 1, abort_flag, 11)) break;
      atc_mbar_expect_tx(atc_smem(&sh->k_full[s]), bytes);
      for (int r = 0; r < ATC_KEYS; r += box) {
        const int key = key0 + r;
        if (key > pos_last || key + box - 1 < first_key) continue;
        const int page = table[key >> page_shift];
        if (page < 0 || page >= num_pages) continue;
        const int grow = (page * hkv + kvh) * page_size + (key & page_mask);  // row of the [pages*kv_heads*page, hd] view
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          atc_tma_2d(atc_smem(k_s + s * KV_BYTES + p * PANEL_BYTES + r * 128), &map_k, p * 64, grow, atc_smem(&sh->k_full[s]));
      }
      if (t >= 2 && !atc_mbar_wait(atc_smem(&sh->v_empty[s]), ((t >> 1) - 1) & 1, abort_flag, 11)) break;
      atc_mbar_expect_tx(atc_smem(&sh->v_full[s]), bytes);
      for (int r = 0; r < ATC_KEYS; r += box) {
        const int key = key0 + r;
        if (key > pos_last || key + box - 1 < first_key) continue;
        const int page = table[key >> page_shift];
        if (page < 0 || page >= num_pages) continue;
        const int grow = (page * hkv + kvh) * page_size + (key & page_mask);
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          atc_tma_2d(atc_smem(v_s + s * KV_BYTES + p * PANEL_BYTES + r * 128), &map_v, p * 64, grow, atc_smem(&sh->v_full[s]));
      }
    }
  } else if (warp == 9 && lane == 0) {
    // -------------------------------------------------------------------- issuer
    // The tensor core works through its instructions in the order they are issued, and a commit arrives when
    // everything issued before it is done.  Per key tile t: P V of head A (when its probabilities are written),
    // then the scores of head A for tile t + 1 (which overwrite those probabilities: P V was issued first, so it
    // has read them), then the same for head B.  While one head's softmax runs, the other head's products do.
    bool ok = ntiles == 0 || atc_mbar_wait(atc_smem(&sh->q_full), 0, abort_flag, 12);
    const unsigned idesc_s = atc_idesc(ATC_ROWS, ATC_KEYS, false);
    const unsigned idesc_o = atc_idesc(ATC_ROWS, 64, true);
    // the descriptors once; an offset of b bytes inside a tile adds b / 16 to the address field
    const unsigned long long desc_q0 = atc_desc(atc_smem(q_s)), desc_q1 = atc_desc(atc_smem(q_s + KV_BYTES));
    const unsigned long long desc_k0 = atc_desc(atc_smem(k_s)), desc_k1 = atc_desc(atc_smem(k_s + KV_BYTES));
    const unsigned long long desc_v0 = atc_desc(atc_smem(v_s)), desc_v1 = atc_desc(atc_smem(v_s + KV_BYTES));
    // S = Q K^T over hd in steps of 16 (four steps per 64-column panel)
    auto issue_qk = [&](int x, int s) {
      const unsigned long long dq = x ? desc_q1 : desc_q0, dk = s ? desc_k1 : desc_k0;
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        const unsigned off = (k >> 2) * PANEL_BYTES + (k & 3) * 32;
        atc_mma(tmem + x * 128, dq + (off >> 4), dk + (off >> 4), idesc_s, k != 0);
      }
      atc_commit(atc_smem(&sh->s_full[x]));
    };
    // O += P V over the tile's 128 keys in steps of 16 (8 columns of packed pairs); one instruction per 64 columns of hd
    auto issue_pv = [&](int x, int s, int t) {
      const unsigned long long dv = s ? desc_v1 : desc_v0;
#pragma unroll
      for (int k = 0; k < ATC_KEYS / 16; ++k)
#pragma unroll
        for (int p = 0; p < PANELS; ++p)
          atc_mma_ts(tmem + 256 + x * 128 + p * 64, tmem + x * 128 + k * 8, dv + ((p * PANEL_BYTES + k * 2048) >> 4), idesc_o,
                     (t > 0 || k != 0) ? 1u : 0u);
    };
    if (ok && ntiles > 0) {
      ok = atc_mbar_wait(atc_smem(&sh->k_full[0]), 0, abort_flag, 13);
      if (ok) {
        atc_fence_after();
        issue_qk(0, 0);
        if (has_b) issue_qk(1, 0);
        atc_commit(atc_smem(&sh->k_empty[0]));
      }
    }
    for (int t = 0; t < ntiles && ok; ++t) {
      const int s = t & 1, s1 = s ^ 1;
      const bool next = t + 1 < ntiles;
      ok = atc_mbar_wait(atc_smem(&sh->p_full[0]), t & 1, abort_flag, 14) &&
           atc_mbar_wait(atc_smem(&sh->v_full[s]), (t >> 1) & 1, abort_flag, 14);
      if (!ok) break;
      atc_fence_after();
      issue_pv(0, s, t);
      if (!has_b) atc_commit(atc_smem(&sh->v_empty[s]));
      if (next) {
        ok = atc_mbar_wait(atc_smem(&sh->k_full[s1]), ((t + 1) >> 1) & 1, abort_flag, 13);
        if (!ok) break;
        atc_fence_after();
        issue_qk(0, s1);
        if (!has_b) atc_commit(atc_smem(&sh->k_empty[s1]));
      }
      if (has_b) {
        ok = atc_mbar_wait(atc_smem(&sh->p_full[1]), t & 1, abort_flag, 16);
        if (!ok) break;
        atc_fence_after();
        issue_pv(1, s, t);
        atc_commit(atc_smem(&sh->v_empty[s]));
        if (next) {
          issue_qk(1, s1);
          atc_commit(atc_smem(&sh->k_empty[s1]));
        }
      }
    }
    if (ok && ntiles > 0) atc_commit(atc_smem(&sh->o_done));
  } else if (warp < 8) {
    // ------------------------------------------------------------ softmax threads
    const int x = warp >> 2;      // which head of the pair
    const int row = tid & 127;    // accumulator lane = query row of the tile
    const int pos = pos0 + row;
    const int hi = row < nrows ? pos : -1;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const unsigned lane_addr = (unsigned)((warp & 3) * 32) << 16;
    const unsigned tmem_s = tmem + x * 128, tmem_o = tmem + 256 + x * 128;
    const int steps = (x == 0 || has_b) ? ntiles : 0;
    float m = -INFINITY, l = 0.f;  // the reference of the row's exponents, the sum of its probabilities
    bool ok = true;
    for (int t = 0; t < steps && ok; ++t) {
      ok = atc_mbar_wait(atc_smem(&sh->s_full[x]), t & 1, abort_flag, 15);
      if (!ok) break;
      atc_fence_after();
      // the scores have arrived, and with them (the tensor core works in order) the product P V of the tile before
      unsigned r[ATC_KEYS];
#pragma unroll
      for (int c = 0; c < ATC_KEYS; c += 32) atc_ld32_issue(tmem_s + lane_addr + c, r + c);
      atc_wait_ld();
      const int key0 = (tile_lo + t) * ATC_KEYS;
      const int rlo = lo - key0, rhi = hi - key0;
      // whether every row of this warp sees the whole tile: the same for the whole warp, which keeps the
      // warp-wide tensor memory instructions below out of divergent code
      const bool inside = __all_sync(0xffffffffu, rlo <= 0 && rhi >= ATC_KEYS - 1);
      const float mx = (inside ? atc_row_max<true>(r, rlo, rhi) : atc_row_max<false>(r, rlo, rhi)) * scale_log2;
      // the reference moves only when the maximum has grown by more than 8; a row that has seen no key yet
      // (m = -inf) has nothing in O to rescale
      const bool grow = mx > m + 8.f;
      const float corr = grow ? atc_exp2(m - mx) : 1.f;
      const bool rescale = __any_sync(0xffffffffu, grow && m != -INFINITY);
      m = grow ? mx : m;
      const float mu = m == -INFINITY ? 0.f : m;
      unsigned long long sum2[2] = {atc_pack(0.f, 0.f), atc_pack(0.f, 0.f)};
      if (inside) {
        atc_row_probs<true, 0>(r, rlo, rhi, scale_log2, mu, sum2);
        atc_row_probs<true, 1>(r, rlo, rhi, scale_log2, mu, sum2);
      } else {
        atc_row_probs<false, 0>(r, rlo, rhi, scale_log2, mu, sum2);
        atc_row_probs<false, 1>(r, rlo, rhi, scale_log2, mu, sum2);
      }
      float s0, s1, s2, s3;
      atc_unpack(sum2[0], s0, s1);
      atc_unpack(sum2[1], s2, s3);
      l = l * corr + ((s0 + s1) + (s2 + s3));
      if (rescale) {  // (now, when the row of scores has shrunk to 64 registers of packed pairs)
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          unsigned v[32];
          atc_ld32_issue(tmem_o + lane_addr + c, v);
          atc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          atc_st32(tmem_o + lane_addr + c, v);
        }
      }
      // the row of P, two bfloat16 to a column, over the first 64 columns of the scores it was made from
      atc_st32(tmem_s + lane_addr, r);
      atc_st32(tmem_s + lane_addr + 32, r + 32);
      atc_fence_before();
      atc_mbar_arrive(atc_smem(&sh->p_full[x]));
    }
    if (ok && steps > 0) {
      ok = atc_mbar_wait(atc_smem(&sh->o_done), 0, abort_flag, 15);
      atc_fence_after();
    }
    // whether the whole group got through: decided behind a barrier that all of its 128 threads reach whatever
    // happened, so that the barriers inside atc_finish are reached by all of them or by none
    if (!ok) sh->group_bad[x] = 1;
    asm volatile("bar.sync %0, 128;\n" ::"r"(1 + x) : "memory");
    if (!sh->group_bad[x] && (x == 0 || has_b) && active) {
      const size_t item = (size_t)tile_id * hq + head_a + x;
      atc_finish<HD>(tmem_o + lane_addr, steps > 0, m, l, row, nrows, out + ((size_t)(row0 + row) * hq + head_a + x) * HD, nsplit,
                     split, scratch + item * nruns * ATC_SPLIT_WORDS(HD), counters + item, 1 + x, &sh->last_flag[x]);
      atc_fence_before();
    }
  }
  atc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
}

// ------------------------------------------------------------------------------------ host

typedef CUresult (*AtcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int atc_make_map(CUtensorMap* map, const void* base, long long rows, int cols, int ld, int box_rows) {
  static AtcEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (AtcEncodeFn)p;
  }
  MS_REQUIRE(fn != nullptr, "attention_prefill_tc: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MS_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

static int atc_launch_single(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int* tile_row0,
                             const int* tile_rows, int num_tiles, const int* positions, const int* slot_of_token,
                             const int* block_table, int max_pages, int num_pages, int hq, int hkv, int page_size, int window,
                             float scale, int splits, int run_tiles, float* scratch, int* counters, cudaStream_t stream) {
  const size_t smem = 1024 + 1024 + (size_t)16384 * 4;
  auto kern = attention_prefill_tc_single_kernel<64>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "attention_prefill_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  MS_REQUIRE((long long)num_tiles * splits <= 65535, "attention_prefill_tc: %d tiles in %d runs are more than one launch takes", num_tiles, splits);
  dim3 grid(hq, num_tiles * splits);
  kern<<<grid, ATC_THREADS, smem, stream>>>(mq, mk, mv, (__nv_bfloat16*)out, tile_row0, tile_rows, positions, slot_of_token,
                                            block_table, max_pages, num_pages, hq, hkv, page_size, window, scale * ATC_LOG2E,
                                            splits, run_tiles, scratch, counters);
  MS_LAUNCH_CHECK("attention_prefill_tc");
  return 0;
}

template <int HD>
static int atc_launch_pair(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int* tile_row0,
                           const int* tile_rows, int num_tiles, const int* positions, const int* slot_of_token,
                           const int* block_table, int max_pages, int num_pages, int hq, int hkv, int page_size, int window,
                           float scale, int splits, int run_tiles, int alone, float* scratch, int* counters, cudaStream_t stream) {
  // two heads' Q, two stages of K and of V (194 KB at head size 128); never less than half an SM's shared memory, so
  // that a block has the SM and all of its tensor memory to itself
  size_t smem = 1024 + 1024 + (size_t)(HD / 64) * 16384 * 6;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kern = attention_prefill_tc_pair_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "attention_prefill_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int groups = hq / hkv;
  MS_REQUIRE((long long)num_tiles * splits <= 65535, "attention_prefill_tc: %d tiles in %d runs are more than one launch takes", num_tiles, splits);
  // a block attends a tile of rows with two heads of one group, or with one head
  dim3 grid(hkv * (alone ? groups : (groups + 1) / 2), num_tiles * splits);
  kern<<<grid, ATC_PAIR_THREADS, smem, stream>>>(mq, mk, mv, (__nv_bfloat16*)out, tile_row0, tile_rows, positions, slot_of_token,
                                                 block_table, max_pages, num_pages, hq, hkv, page_size, window, scale * ATC_LOG2E,
                                                 splits, run_tiles, alone, scratch, counters);
  MS_LAUNCH_CHECK("attention_prefill_tc");
  return 0;
}

// 0 if no block ever gave up a wait; else the code of the first that did.  Synchronizes the device.
MS_API int ms_attention_tc_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_atc_error, sizeof(int));
  if (reset && v) {
    int z = 0;
    cudaMemcpyToSymbol(g_atc_error, &z, sizeof(int));
  }
  return v;
}


// A wait that runs out, in the form that cannot hang: one thread waits `polls` polls on a barrier in its own
// shared memory that nothing arrives on, through the helper that every wait of the kernel above uses; no
// copy and no tensor memory is involved.  Leaves code 19 for ms_attention_tc_status.
__global__ void atc_wait_probe_kernel(int polls) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    atc_mbar_init(atc_smem(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    atc_mbar_wait(atc_smem(&bar), 0, &abort_flag, 19, polls);
  }
}
MS_API int ms_attention_tc_wait_probe(int polls, cudaStream_t stream) {
  MS_REQUIRE(polls >= 1 && polls <= 100000, "attention_tc_wait_probe: 1 to 100000 polls");
  atc_wait_probe_kernel<<<1, 32, 0, stream>>>(polls);
  MS_LAUNCH_CHECK("attention_tc_wait_probe");
  return 0;
}

MS_API int ms_attention_prefill_tc_supports(int hd, int page_size) {
  return (hd == 64 || hd == 128) && page_size >= 8 && (page_size & (page_size - 1)) == 0;
}

// float32 words of scratch memory that `splits` > 1 need for the items' partial results.  Beside them the launch
// needs num_tiles * hq counters (int32), which must be zero before the first launch and are left zero by every launch.
MS_API long long ms_attention_prefill_tc_scratch_words(int num_tiles, int hq, int hd, int splits) {
  if (splits <= 1) return 0;
  return (long long)num_tiles * hq * splits * ATC_SPLIT_WORDS(hd);
}

// How a launch is laid out so that it fills the GPU: few tiles of rows (a short prompt, a portion of a long one) would
// leave most SMs idle behind the blocks with the longest rows of key tiles.  plan[0]: the number of runs the key tiles
// of every item are cut into for different blocks (1 to 4).  plan[1]: 1 if, at head size 128, every block should take
// one head instead of two of a group.  plan[2]: if not 0, the most key tiles of a run (only longer items are cut).
// `max_keys`: the most keys any row of the launch sees; `total_key_tiles`: the
// tiles of 128 keys that the launch's tiles of rows see, in all (0: every tile sees max_keys).
//
// Head size 64 (two blocks per SM): as many runs as fill the places, at least four key tiles a run.
// Head size 128: the cheapest of the eight layouts by a model of the launch's time, fitted to measurements on B200
// (1.5B and 7B head counts, 128 to 2,048 rows, 128 to 4,096 keys; us): a block costs 13 at its start and end and 2.6
// per key tile with two heads, 9.5 and 2.3 with one; a launch takes as long as its longest block or as its work
// spread over the SMs, whichever is more (blocks of equal length: as the waves they come in); runs of key tiles cost
// 4 + their number for the merge.
MS_API void ms_attention_prefill_tc_plan(int num_tiles, int hq, int hkv, int hd, int max_keys, int total_key_tiles,
                                         int sm_count, int* plan) {
  plan[0] = 1;
  plan[1] = 0;
  if (num_tiles <= 0 || hq <= 0 || hkv <= 0 || sm_count <= 0) return;
  const int groups = hq / hkv;
  const int key_tiles = (max_keys + ATC_KEYS - 1) / ATC_KEYS;
  plan[2] = 0;
  if (hd == 64) {
    const long long blocks = (long long)num_tiles * hq;
    int splits = (int)(2LL * sm_count / blocks);
    if (splits > key_tiles / 4) splits = key_tiles / 4;
    if (splits > ATC_MAX_SPLITS) splits = ATC_MAX_SPLITS;
    plan[0] = splits < 1 ? 1 : splits;
    return;
  }
  const float all_tiles = total_key_tiles > 0 ? (float)total_key_tiles : (float)num_tiles * key_tiles;
  const float mean_tiles = all_tiles / (float)num_tiles;
  const bool alike = mean_tiles >= 0.8f * key_tiles;  // a portion deep in its prompt: blocks of equal length come in waves
  float best = 0.f;
  for (int alone = 0; alone < 2; ++alone) {
    const float fixed = alone ? 9.5f : 13.f, step = alone ? 2.3f : 2.6f;
    const float heads = (float)(alone ? hq : hkv * ((groups + 1) / 2));
    for (int s = 1; s <= ATC_MAX_SPLITS && (s == 1 || 2 * s <= key_tiles); ++s) {
      const float blocks = heads * (float)num_tiles * s;
      const float longest = fixed + (float)((key_tiles + s - 1) / s) * step;
      const float spread = (blocks * fixed + heads * all_tiles * step) / (float)sm_count;
      const float waves = (float)(((long long)blocks + sm_count - 1) / sm_count) * (fixed + mean_tiles / s * step);
      const float body = alike ? (longest > waves ? longest : waves) : (longest > spread ? longest : spread);
      const float t = s > 1 ? (body + 4.f + s) * 1.1f : body;  // (runs have to earn a tenth more than they promise)
      if (best == 0.f || t < best - 0.05f) {
        best = t;
        plan[0] = s;
        plan[1] = alone;
        // blocks of very different lengths (a prompt taken whole): only items longer than a run are cut
        plan[2] = (s > 1 && !alike) ? (key_tiles + s - 1) / s : 0;
      }
    }
  }
}

// As ms_attention_prefill, with tiles of up to 128 rows.  q, out: bfloat16 [total_rows, hq*hd].  `splits` (1 to 4): the
// key tiles of every item go to that many blocks, which meet in `scratch` (ms_attention_prefill_tc_scratch_words) and
// count themselves in `counters` (num_tiles * hq of them, all zero).  `alone` (head size 128): a block takes one head, not two.
// `run_tiles` > 0: an item is cut only into as many runs as keep a run at that many key tiles at most (0: always `splits`).
MS_API int ms_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, void* out, int total_rows,
                                   const int* tile_row0, const int* tile_rows, int num_tiles, const int* positions,
                                   const int* slot_of_token, const int* block_table, int max_pages, int num_pages, int hq,
                                   int hkv, int hd, int page_size, int window, float scale, int splits, int alone,
                                   int run_tiles, float* scratch, long long scratch_words, int* counters,
                                   long long num_counters, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  MS_REQUIRE(num_tiles > 0 && total_rows > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, "attention_prefill_tc: bad sizes");
  MS_REQUIRE(ms_attention_prefill_tc_supports(hd, page_size),
             "attention_prefill_tc: head_dim %d (64 or 128) or page size %d (a power of two from 8) is not covered", hd, page_size);
  MS_REQUIRE(((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) % 16 == 0, "attention_prefill_tc: operands must be 16-byte aligned");
  MS_REQUIRE(splits >= 1 && splits <= ATC_MAX_SPLITS && run_tiles >= 0, "attention_prefill_tc: %d splits (1 to %d)", splits, ATC_MAX_SPLITS);
  const long long need = ms_attention_prefill_tc_scratch_words(num_tiles, hq, hd, splits);
  MS_REQUIRE(need == 0 || (scratch != nullptr && scratch_words >= need),
             "attention_prefill_tc: %d splits need %lld words of scratch memory, %lld were given", splits, need, scratch_words);
  MS_REQUIRE(need == 0 || (counters != nullptr && num_counters >= (long long)num_tiles * hq),
             "attention_prefill_tc: %d splits need %lld counters, %lld were given", splits, (long long)num_tiles * hq, num_counters);
  CUtensorMap mq, mk, mv;
  if (int rc = atc_make_map(&mq, q, total_rows, hq * hd, hq * hd, ATC_ROWS)) return rc;
  const int box = page_size < ATC_KEYS ? page_size : ATC_KEYS;
  const long long cache_rows = (long long)num_pages * hkv * page_size;
  if (int rc = atc_make_map(&mk, k_pages, cache_rows, hd, hd, box)) return rc;
  if (int rc = atc_make_map(&mv, v_pages, cache_rows, hd, hd, box)) return rc;
  if (hd == 64)
    return atc_launch_single(mq, mk, mv, out, tile_row0, tile_rows, num_tiles, positions, slot_of_token, block_table, max_pages,
                             num_pages, hq, hkv, page_size, window, scale, splits, run_tiles, scratch, counters, stream);
  return atc_launch_pair<128>(mq, mk, mv, out, tile_row0, tile_rows, num_tiles, positions, slot_of_token, block_table, max_pages,
                              num_pages, hq, hkv, page_size, window, scale, splits, run_tiles, alone ? 1 : 0, scratch, counters, stream);
}
