// Matrix product for few rows (decoding): out[M, N] = x[M, K] . W[N, K]^T, M <= 64, bfloat16
// operands, float32 accumulation, built to stream the weights once at memory speed.
//
// The weights are the A operand of m16n8k16 tensor-core instructions (16 weight rows per
// warp), the activations the B operand (8 batch rows per instruction).  Both are read
// with 16-byte loads straight into fragments: a thread's 8 consecutive k of one row serve
// two instructions, and since a dot product does not care about the order of k, the
// activations are read in the same permuted order.  The k range of a block of weight rows
// is spread over the warps (4 or 8 per block) of a thread-block cluster.  The weights of a warp's first
// chunks are requested with asynchronous copies into shared memory BEFORE the kernel waits for its
// predecessor in the stream (they do not depend on it), each thread into slots only it reads, so no
// registers are held meanwhile and no barrier is needed; with 4 warps a block the whole product of the
// gated feed-forward at decoding sizes is requested at once and its blocks are resident in one wave.
// Partial sums are added in warp order
// inside a block and in rank order across the cluster through distributed shared memory,
// so the result does not depend on timing.  Epilogues: plain (bfloat16 or float32 out); the
// gated feed-forward's silu(gate) * up, for which a block holds 8 gate rows and the 8 up
// rows of the same outputs; or the residual add, which adds the product into the float32
// residual stream in place and leaves, per row and block of 16 columns, the sum of squares
// of the new residual (and, if asked, a bfloat16 copy of the new residual).  Row scaling
// (optional): the activations are that bfloat16 copy and every output row is multiplied by the row's
// 1 / rms, made from those sums of squares, in the epilogue: the RMS norm for a matrix that has the
// norm's weight folded into its columns, (x / rms * g) . W^T = (x . (W g)^T) / rms.  So neither the
// add nor the norm needs a kernel of its own, and the activations come in one round of copies.
//
// The reference has a small-row kernel of the same purpose on CUDA-core FMAs
// (gemv_f16 / gemv_f16_qkv, crates/mach-model/src/kernels.rs:2665-2808 of gqf2008/machserve:
// one warp per (row, output), rows <= 8).
#include <cooperative_groups.h>

#include "launch.cuh"

namespace cg = cooperative_groups;

#define GSM_MAX_CLUSTER 4  // most blocks that share the k range of the same weight rows
#define GSM_HELD 3         // most chunks of weights a warp requests into registers before the wait
#define GSM_PF 4           // chunks of weights a warp keeps in flight in registers (past the staged ones)

enum { GSM_EPI_BF16 = 0, GSM_EPI_F32 = 1, GSM_EPI_SILU_MUL = 2, GSM_EPI_RESADD = 3 };

// What the row scaling and the residual epilogue need beyond the plain product.
struct GsmExtra {
  const float* stats_in; // row scaling: sums of squares [M][stats_in_nb] of the rows the activations were rounded from
  int stats_in_nb;
  float eps;
  float* residual;       // epilogue: float32 [M][ldr], added into in place
  int ldr;
  float* stats_out;      // epilogue: sums of squares [M][number of blocks] of the new residual
  __nv_bfloat16* copy_out;  // epilogue, optional: the new residual rounded to bfloat16, [M][ldc]
  int ldc;
};

__device__ __forceinline__ uint4 gsm_load_stream(const __nv_bfloat16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ unsigned gsm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ void gsm_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                        unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: batch rows in units of 8.  w_lo / w_hi: where rows 0..7 / 8..15 of a block's 16 weight rows come
// from; block b starts `rows_per_block * b` rows into each.  n_lo / n_hi: how many rows each of them has.
// SCALE == 1: every output row is multiplied by 1 / rms of the row the activations were rounded from.
__device__ __forceinline__ void gsm_cp_async16(void* smem, const void* gmem, bool valid) {
  const int n = valid ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(n));
}

// One chunk of 32 k for all MT groups of 8 batch rows: the B fragments are read from global memory and multiplied
// with the chunk's weight fragments wa (rows 0..7) and wb (rows 8..15).
template <int MT>
__device__ __forceinline__ void gsm_chunk(float (&acc)[MT][4], const uint4& wa, const uint4& wb, const __nv_bfloat16* x,
                                          int ldx, int M, int K, int kb, int g, int c) {
  const bool k_ok = kb + 8 * c + 8 <= K;
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    const int m = j * 8 + g;
    uint4 xv = make_uint4(0, 0, 0, 0);
    if (m < M && k_ok) xv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + kb + 8 * c);
    gsm_mma(acc[j], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
    gsm_mma(acc[j], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
  }
}

// How the kernel is laid out (all sizes in the launch's GsmShape):
//   W warps per block (4 or 8) serve RB blocks of 16 weight rows (1 or 2), W / RB warps each, which take the
//   chunks of 32 k of their rows in turn, together with the other blocks of the cluster.
//   staged   chunks per warp whose weights go through shared memory, requested before the wait for the
//            preceding kernel; `held` (up to GSM_HELD) more chunks are requested into registers at the same time.
//   xs_stride  if not 0, the block's share of the activations is brought into shared memory once after the
//            wait, as bfloat16 rows of this many elements, in one round of
//            copies, and every warp reads its B fragments from there.  Else the fragments are read from
//            global memory chunk by chunk.
struct GsmShape {
  int nblocks;       // blocks of 16 weight rows in all
  int cluster_size;  // blocks of the grid that share the k range of the same rows
  int staged, held;
  int xs_stride, xs_chunks;  // row stride in elements; chunks per row (the block's chunks, compact)
};

template <int MT, int EPI, int SCALE, int W, int RB, bool XS>
__global__ void __launch_bounds__(W * 32, W == 8 ? 3 : 6)
gemm_small_m_kernel(const void* __restrict__ x_any, int ldx, const __nv_bfloat16* __restrict__ w_lo,
                    const __nv_bfloat16* __restrict__ w_hi, int rows_per_block, int n_lo, int n_hi,
                    void* __restrict__ out, int ldo, int M, int K, GsmShape sh, GsmExtra ex) {
  constexpr int THREADS = W * 32, WR = W / RB, COLS = MT * 8;
  constexpr int TPR = THREADS / COLS;  // threads that share a row of the activations: 4 .. 32, within one warp
  MS_TIMELINE_BEGIN(100 + EPI * 10 + SCALE);
  extern __shared__ __align__(16) uint4 gsm_dyn[];
  // dynamic: [warp][staged][rows 0..7 | rows 8..15][lane] weights; then (XS) activations [COLS][xs_stride]
  // bfloat16
  __shared__ float red[W][16][COLS + 1];
  __shared__ float part[RB][16][COLS + 1];
  // block 0 of a cluster: the other blocks' sums (with up to 16 batch rows; with more it fetches them)
  __shared__ float gathered[MT <= 2 ? GSM_MAX_CLUSTER - 1 : 1][RB][16][COLS + 1];
  __shared__ float inv_rms[COLS];
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(x_any);
  const int cluster_size = sh.cluster_size, staged = sh.staged;

  const int group = blockIdx.x / cluster_size, rank = blockIdx.x - group * cluster_size;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rb = warp / WR, warp_in = warp - rb * WR;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = (group * RB + rb) * rows_per_block;  // past the last block of rows: nothing is read or written
  const bool lo_ok = n0 + g < n_lo, hi_ok = n0 + g < n_hi;
  const __nv_bfloat16* a_lo = w_lo + (size_t)(n0 + g) * K + 8 * c;
  const __nv_bfloat16* a_hi = w_hi + (size_t)(n0 + g) * K + 8 * c;
  uint4* my_stage = gsm_dyn + (size_t)warp * staged * 64 + lane;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gsm_dyn + (size_t)W * staged * 64);

  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

  // Chunks of 32 k go round the warps that share the rows: warp_in + WR * rank, then every `stride`-th.
  // The block's own chunks, numbered compactly, are lc = u * WR + w for the u-th chunk of its warp w;
  // chunk lc starts at k = ((lc / WR) * stride + rank * WR + lc % WR) * 32.
  const int chunks = (K + 31) / 32;
  const int stride = cluster_size * WR;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const int ch0 = rank * WR + warp_in;
  // before the wait: everything that does not depend on the preceding kernel
#pragma unroll 1
  for (int u = 0; u < staged; ++u) {
    const int kb = (ch0 + u * stride) * 32;
    const bool k_ok = kb + 8 * c + 8 <= K;  // K is a multiple of 8; also false past the last chunk
    gsm_cp_async16(my_stage + u * 64, (lo_ok && k_ok) ? a_lo + kb : w_lo, lo_ok && k_ok);
    gsm_cp_async16(my_stage + u * 64 + 32, (hi_ok && k_ok) ? a_hi + kb : w_lo, hi_ok && k_ok);
  }
  asm volatile("cp.async.commit_group;\n" ::);
  uint4 held_a[GSM_HELD], held_b[GSM_HELD];
#pragma unroll
  for (int h = 0; h < GSM_HELD; ++h) {
    held_a[h] = held_b[h] = zero;
    if (h < sh.held) {
      const int kb = (ch0 + (staged + h) * stride) * 32;
      const bool k_ok = kb + 8 * c + 8 <= K;
      if (lo_ok && k_ok) held_a[h] = gsm_load_stream(a_lo + kb);
      if (hi_ok && k_ok) held_b[h] = gsm_load_stream(a_hi + kb);
    }
  }
  ms_pdl_trigger();
  ms_pdl_wait();
  MS_TIMELINE_WAITED();

  // the residual epilogue's own elements of the old residual, requested now so that they are there when the sum is
  constexpr int OUT_ELEMS = RB * 16 * COLS;
  constexpr int RES_PER_THREAD = (OUT_ELEMS + THREADS - 1) / THREADS;
  float res_old[RES_PER_THREAD];
  if (EPI == GSM_EPI_RESADD && rank == 0) {
#pragma unroll
    for (int i = 0; i < RES_PER_THREAD; ++i) {
      const int e = tid + i * THREADS, r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
      const int nb0 = (group * RB + b) * rows_per_block;
      const bool ok = e < OUT_ELEMS && m < M && (r < 8 ? nb0 + r < n_lo : nb0 + r - 8 < n_hi);
      res_old[i] = ok ? ex.residual[(size_t)m * ex.ldr + nb0 + r] : 0.f;
    }
  }
  // Thread (row, sub) of the TPR threads of a row: sums of squares and, if the activations are staged, the pieces
  // sub, sub + TPR, ... of 8 values of the block's share of that row.
  const int row = tid / TPR, sub = tid - row * TPR;
  if (SCALE == 1) {
    // the rows' copies first (so that they are in flight), then the sums of squares for the epilogue's 1 / rms
    if (XS) {
      const int pieces = sh.xs_chunks * 4;
#pragma unroll 1
      for (int pc = sub; pc < pieces; pc += TPR) {
        const int lc = pc >> 2;
        const int k = ((lc / WR) * stride + rank * WR + lc % WR) * 32 + (pc & 3) * 8;
        const bool ok = row < M && k + 8 <= K;
        gsm_cp_async16(xs + (size_t)row * sh.xs_stride + pc * 8, ok ? x + (size_t)row * ldx + k : x, ok);
      }
      asm volatile("cp.async.commit_group;\n" ::);
    }
    float ss = 0.f;
    if (row < M)
      for (int b = sub; b < ex.stats_in_nb; b += TPR) ss += ex.stats_in[(size_t)row * ex.stats_in_nb + b];
#pragma unroll
    for (int off = TPR / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (sub == 0) inv_rms[row] = rsqrtf(ss / (float)K + ex.eps);
  } else if (XS) {
    // the block's share of the activation rows, copied as they are
    const int pieces = sh.xs_chunks * 4;
#pragma unroll 1
    for (int pc = sub; pc < pieces; pc += TPR) {
      const int lc = pc >> 2;
      const int k = ((lc / WR) * stride + rank * WR + lc % WR) * 32 + (pc & 3) * 8;
      const bool ok = row < M && k + 8 <= K;
      gsm_cp_async16(xs + (size_t)row * sh.xs_stride + pc * 8, ok ? x + (size_t)row * ldx + k : x, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");  // staged weights: a thread reads only what it copied itself
  if (XS || SCALE) __syncthreads();
  MS_TIMELINE_MARK(0);

  if (XS) {
    // the B fragments of the warp's u-th chunk come from shared memory
    const __nv_bfloat16* xsrc = xs + (size_t)g * sh.xs_stride + warp_in * 32 + 8 * c;
#pragma unroll 1
    for (int u = 0; u < staged; ++u) {
      const uint4 wa = my_stage[u * 64], wb = my_stage[u * 64 + 32];
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xsrc + (size_t)(j * 8) * sh.xs_stride + u * (WR * 32));
        gsm_mma(acc[j], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
        gsm_mma(acc[j], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
      }
    }
#pragma unroll
    for (int h = 0; h < GSM_HELD; ++h) {
      if (h < sh.held) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xsrc + (size_t)(j * 8) * sh.xs_stride + (staged + h) * (WR * 32));
          gsm_mma(acc[j], held_a[h].x, held_b[h].x, held_a[h].y, held_b[h].y, xv.x, xv.y);
          gsm_mma(acc[j], held_a[h].z, held_b[h].z, held_a[h].w, held_b[h].w, xv.z, xv.w);
        }
      }
    }
  } else {
#pragma unroll 1
    for (int u = 0; u < staged; ++u)
      gsm_chunk<MT>(acc, my_stage[u * 64], my_stage[u * 64 + 32], x, ldx, M, K, (ch0 + u * stride) * 32, g, c);
#pragma unroll
    for (int h = 0; h < GSM_HELD; ++h)
      if (h < sh.held) gsm_chunk<MT>(acc, held_a[h], held_b[h], x, ldx, M, K, (ch0 + (staged + h) * stride) * 32, g, c);
    // what is left of a long row streams through registers, GSM_PF chunks in flight
#pragma unroll 1
    for (int u1 = staged + sh.held; ch0 + u1 * stride < chunks; u1 += GSM_PF) {
      uint4 wa[GSM_PF], wb[GSM_PF];
#pragma unroll
      for (int u = 0; u < GSM_PF; ++u) {
        const int kb = (ch0 + (u1 + u) * stride) * 32;
        const bool k_ok = kb + 8 * c + 8 <= K;
        wa[u] = (lo_ok && k_ok) ? gsm_load_stream(a_lo + kb) : zero;
        wb[u] = (hi_ok && k_ok) ? gsm_load_stream(a_hi + kb) : zero;
      }
#pragma unroll
      for (int u = 0; u < GSM_PF; ++u)
        gsm_chunk<MT>(acc, wa[u], wb[u], x, ldx, M, K, (ch0 + (u1 + u) * stride) * 32, g, c);
    }
  }
  MS_TIMELINE_MARK(2);

  // add the warps that share rows, in warp order
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    red[warp][g][j * 8 + 2 * c] = acc[j][0];
    red[warp][g][j * 8 + 2 * c + 1] = acc[j][1];
    red[warp][g + 8][j * 8 + 2 * c] = acc[j][2];
    red[warp][g + 8][j * 8 + 2 * c + 1] = acc[j][3];
  }
  __syncthreads();
#pragma unroll 1
  for (int e = tid; e < OUT_ELEMS; e += THREADS) {
    const int r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WR; ++w) s += red[b * WR + w][r][m];
    part[b][r][m] = s;
  }
  // add the blocks of the cluster in rank order, in block 0: the others put their sums into block 0's shared memory
  // (stores through distributed shared memory: one way, no round trip), one cluster barrier makes them visible, and
  // block 0 adds them in rank order, so the result does not depend on timing
  if (cluster_size > 1 && MT <= 2) {
    cg::cluster_group cluster = cg::this_cluster();
    if (rank != 0) {
      float* dst = cluster.map_shared_rank(&gathered[0][0][0][0], 0) + (size_t)(rank - 1) * RB * 16 * (COLS + 1);
#pragma unroll 1
      for (int e = tid; e < OUT_ELEMS; e += THREADS) {
        const int r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
        dst[(b * 16 + r) * (COLS + 1) + m] = part[b][r][m];  // each element is read and written by the same thread
      }
    }
    cluster.sync();
    if (rank != 0) return;
#pragma unroll 1
    for (int e = tid; e < OUT_ELEMS; e += THREADS) {
      const int r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
      float s = part[b][r][m];
#pragma unroll
      for (int k = 1; k < GSM_MAX_CLUSTER; ++k)
        if (k < cluster_size) s += gathered[k - 1][b][r][m];
      part[b][r][m] = s;
    }
  } else if (cluster_size > 1) {
    // more than 16 batch rows: block 0 fetches the others' sums (a gathering buffer for them would not fit);
    // the same additions in the same order
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (rank == 0) {
#pragma unroll 1
      for (int e = tid; e < OUT_ELEMS; e += THREADS) {
        const int r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
        const int at = (b * 16 + r) * (COLS + 1) + m;
        float other[GSM_MAX_CLUSTER - 1];  // requested together (one round trip), added in rank order
#pragma unroll
        for (int k = 1; k < GSM_MAX_CLUSTER; ++k) other[k - 1] = k < cluster_size ? cluster.map_shared_rank(&part[0][0][0], k)[at] : 0.f;
        float s = part[b][r][m];
#pragma unroll
        for (int k = 1; k < GSM_MAX_CLUSTER; ++k)
          if (k < cluster_size) s += other[k - 1];
        part[b][r][m] = s;
      }
    }
    cluster.sync();  // the other blocks' shared memory must live until block 0 has read it
    if (rank != 0) return;
  }
  __syncthreads();
  MS_TIMELINE_MARK(3);

  if (EPI == GSM_EPI_RESADD) {
    // residual[m][n] += product, in place (each element belongs to one thread of one block); then the sum of
    // squares of each block's 16 columns of the new residual, per row, for the norm that follows
#pragma unroll
    for (int i = 0; i < RES_PER_THREAD; ++i) {
      const int e = tid + i * THREADS, r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
      if (e >= OUT_ELEMS) break;
      const int nb0 = (group * RB + b) * rows_per_block;
      const bool ok = r < 8 ? nb0 + r < n_lo : nb0 + r - 8 < n_hi;
      float v = 0.f;
      if (m < M && ok) {
        v = res_old[i] + part[b][r][m];
        ex.residual[(size_t)m * ex.ldr + nb0 + r] = v;
        if (ex.copy_out) ex.copy_out[(size_t)m * ex.ldc + nb0 + r] = __float2bfloat16_rn(v);
      }
      part[b][r][m] = v;
    }
    __syncthreads();
    for (int e = tid; e < RB * COLS; e += THREADS) {
      const int m = e % COLS, b = e / COLS;
      if (m < M && group * RB + b < sh.nblocks) {
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) ss += part[b][r][m] * part[b][r][m];
        ex.stats_out[(size_t)m * sh.nblocks + group * RB + b] = ss;
      }
    }
  } else if (EPI == GSM_EPI_SILU_MUL) {
#pragma unroll 1
    for (int e = tid; e < RB * 8 * COLS; e += THREADS) {
      const int r = e % 8, m = (e / 8) % COLS, b = e / (8 * COLS);
      const int nb0 = (group * RB + b) * rows_per_block;
      if (m < M && nb0 + r < n_lo) {
        const float rs = SCALE == 1 ? inv_rms[m] : 1.f;
        const float gate = part[b][r][m] * rs, up = part[b][r + 8][m] * rs;
        reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + nb0 + r] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      }
    }
  } else {
#pragma unroll 1
    for (int e = tid; e < OUT_ELEMS; e += THREADS) {
      const int r = e % 16, m = (e / 16) % COLS, b = e / (16 * COLS);
      const int nb0 = (group * RB + b) * rows_per_block;
      const bool ok = r < 8 ? nb0 + r < n_lo : nb0 + r - 8 < n_hi;
      if (m < M && ok) {
        const float v = SCALE == 1 ? part[b][r][m] * inv_rms[m] : part[b][r][m];
        if (EPI == GSM_EPI_F32)
          reinterpret_cast<float*>(out)[(size_t)m * ldo + nb0 + r] = v;
        else
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + nb0 + r] = __float2bfloat16_rn(v);
      }
    }
  }
}

// How a product is spread over the GPU.
struct GsmPlan {
  int warps, rb;
  GsmShape sh;
  size_t smem;
};

#define GSM_STAGE_BYTES (48 * 1024)  // most shared memory for staged weights per block: 1 KB per warp and chunk
#define GSM_XS_BYTES (48 * 1024)     // most shared memory for the activations per block (16 rows of a block's share of K = 4,864 in a cluster of four: 41.5 KB)

// 8 warps a block and about three blocks per SM, the k range split over a cluster when there are few blocks of
// rows.  When that would leave a short second wave of blocks (which would start their copies only after the
// wait), a block takes two blocks of rows (the gated product) or has 4 warps (the residual product).
static GsmPlan gsm_plan(int blocks, int M, int K, int epi, int sm_count) {
  const int chunks = (K + 31) / 32;
  GsmPlan p;
  p.warps = 8;
  p.rb = 1;
  int want = (sm_count * 3 + blocks - 1) / blocks;
  int most = chunks / (2 * 8);  // at least two chunks per warp
  int cs = want < most ? want : most;
  if (cs > GSM_MAX_CLUSTER) cs = GSM_MAX_CLUSTER;  // (eight blocks a cluster spread a long row further but merged slower: measured)
  if (cs < 1) cs = 1;
  while (cs & (cs - 1)) cs &= cs - 1;  // a power of two
  const bool second_wave = blocks * cs > 3 * sm_count && blocks * cs <= 7 * sm_count;
  if (second_wave && epi == GSM_EPI_SILU_MUL && M <= 32 && (chunks + 4 * cs - 1) / (4 * cs) <= 8) p.rb = 2;
  if (second_wave && epi == GSM_EPI_RESADD && (chunks + 4 * cs - 1) / (4 * cs) <= 8) p.warps = 4;
  const int wr = p.warps / p.rb;
  const int per_warp = (chunks + wr * cs - 1) / (wr * cs);
  const int room = GSM_STAGE_BYTES / 1024 / p.warps;
  p.sh.nblocks = blocks;
  p.sh.cluster_size = cs;
  p.sh.staged = per_warp < room ? per_warp : room;
  p.sh.held = per_warp - p.sh.staged <= GSM_HELD ? per_warp - p.sh.staged : 0;
  // the activations in shared memory, if the block's share is small: rows of (its chunks * 32) elements, padded
  // so that the 8 rows a warp reads at once fall into different banks (row stride = 16 words mod 32)
  const int cols = M <= 8 ? 8 : M <= 16 ? 16 : M <= 32 ? 32 : 64;
  const int xs_chunks = per_warp * wr;
  int stride = xs_chunks * 32;
  stride += ((16 - (stride / 2) % 32 + 32) % 32) * 2;
  const bool fits = cols <= 16 && (size_t)cols * stride * 2 <= GSM_XS_BYTES;
  p.sh.xs_stride = fits ? stride : 0;
  p.sh.xs_chunks = fits ? xs_chunks : 0;
  // All blocks of the launch should be resident at once (a block of a second wave starts its copies only after
  // the wait): fewer chunks go through shared memory and more through registers if that is what it takes.
  const size_t fixed = (fits ? (size_t)cols * stride * 2 : 0) +
                       (size_t)(p.warps + p.rb + (cols <= 16 ? (GSM_MAX_CLUSTER - 1) * p.rb : p.rb)) * 16 * (cols + 1) * 4 + 2048;
  const int groups = (blocks + p.rb - 1) / p.rb;
  const int per_sm = (groups * cs + sm_count - 1) / sm_count;
  while (p.sh.staged > 1 && per_warp - (p.sh.staged - 1) <= GSM_HELD && per_sm <= 8 &&
         per_sm * (fixed + (size_t)p.warps * p.sh.staged * 1024) > (size_t)227 * 1024) {
    --p.sh.staged;  // (only as far as the registers can hold the rest: with staged activations nothing streams later)
    p.sh.held = per_warp - p.sh.staged;
  }
  // with staged activations every chunk of weights is requested before the wait, into shared memory or registers;
  // a longer row of weights streams through registers after the wait and reads its activations from global memory
  const bool xs = fits && p.sh.staged + p.sh.held == per_warp;
  if (!xs) p.sh.xs_stride = p.sh.xs_chunks = 0;
  p.smem = (size_t)p.warps * p.sh.staged * 1024 + (xs ? (size_t)cols * stride * 2 : 0);
  return p;
}

template <int MT, int EPI, int SCALE, int W, int RB, bool XS>
static int gsm_launch_x(const void* x, int ldx, const void* w_lo, const void* w_hi, int rows_per_block, int n_lo, int n_hi,
                        void* out, int ldo, int M, int K, const GsmExtra& ex, const GsmPlan& p, cudaStream_t stream) {
  auto kern = gemm_small_m_kernel<MT, EPI, SCALE, W, RB, XS>;
  static bool configured = false;  // per instantiation: room for the staged operands beside the static arrays,
  if (!configured) {               // and the largest shared-memory share of an SM, so that most blocks are resident
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GSM_STAGE_BYTES + GSM_XS_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) {
      ms_set_error("gemm_small_m: cannot configure shared memory: %s", cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  const int groups = (p.sh.nblocks + RB - 1) / RB;
  MS_LAUNCH_RESULT("gemm_small_m",
                   ms_launch(kern, dim3(groups * p.sh.cluster_size), dim3(W * 32), p.smem, stream, p.sh.cluster_size, true, x,
                             ldx, (const __nv_bfloat16*)w_lo, (const __nv_bfloat16*)w_hi, rows_per_block, n_lo, n_hi, out,
                             ldo, M, K, p.sh, ex));
  return 0;
}

// The activations go through shared memory only for up to 16 rows (and only when the block's share fits).
template <int MT, int EPI, int SCALE, int W, int RB>
static int gsm_launch_w(const void* x, int ldx, const void* w_lo, const void* w_hi, int rows_per_block, int n_lo, int n_hi,
                        void* out, int ldo, int M, int K, const GsmExtra& ex, const GsmPlan& p, cudaStream_t stream) {
  if constexpr (MT <= 2)
    if (p.sh.xs_stride)
      return gsm_launch_x<MT, EPI, SCALE, W, RB, true>(x, ldx, w_lo, w_hi, rows_per_block, n_lo, n_hi, out, ldo, M, K, ex, p, stream);
  return gsm_launch_x<MT, EPI, SCALE, W, RB, false>(x, ldx, w_lo, w_hi, rows_per_block, n_lo, n_hi, out, ldo, M, K, ex, p, stream);
}

template <int MT, int EPI, int SCALE>
static int gsm_launch(const void* x, int ldx, const void* w_lo, const void* w_hi, int rows_per_block, int n_lo, int n_hi,
                      void* out, int ldo, int M, int K, int blocks, const GsmExtra& ex, int sm_count,
                      cudaStream_t stream) {
  const GsmPlan p = gsm_plan(blocks, M, K, EPI, sm_count);
  if constexpr (EPI == GSM_EPI_SILU_MUL && MT <= 4)
    if (p.rb == 2)
      return gsm_launch_w<MT, EPI, SCALE, 8, 2>(x, ldx, w_lo, w_hi, rows_per_block, n_lo, n_hi, out, ldo, M, K, ex, p, stream);
  if constexpr (EPI == GSM_EPI_RESADD)
    if (p.warps == 4)
      return gsm_launch_w<MT, EPI, SCALE, 4, 1>(x, ldx, w_lo, w_hi, rows_per_block, n_lo, n_hi, out, ldo, M, K, ex, p, stream);
  return gsm_launch_w<MT, EPI, SCALE, 8, 1>(x, ldx, w_lo, w_hi, rows_per_block, n_lo, n_hi, out, ldo, M, K, ex, p, stream);
}

template <int EPI, int SCALE>
static int gsm_dispatch(const void* x, int ldx, const void* w_lo, const void* w_hi, int rows_per_block, int n_lo,
                        int n_hi, void* out, int ldo, int M, int K, int blocks, const GsmExtra& ex, int sm_count,
                        cudaStream_t stream) {
#define GSM_CASE(MT) \
  return gsm_launch<MT, EPI, SCALE>(x, ldx, w_lo, w_hi, rows_per_block, n_lo, n_hi, out, ldo, M, K, blocks, ex, sm_count, stream)
  if (M <= 8) GSM_CASE(1);
  if (M <= 16) GSM_CASE(2);
  if (SCALE || EPI == GSM_EPI_RESADD) {  // the fused forms are built for up to 16 rows
    ms_set_error("gemm_small_m: the fused forms take at most 16 rows, not %d", M);
    return 1;
  }
  if (M <= 32) GSM_CASE(4);
  GSM_CASE(8);
#undef GSM_CASE
}

MS_TIMELINE_SETTER(ms_timeline_set_gemm_small_m)

MS_API int ms_gemm_small_m_supports(int M, int N, int K) { return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0; }

// How a product of M rows with N outputs over K would be spread (host arithmetic only, for tests and notes).
// gated: the gate/up form (N = the intermediate size), else a product with 16 weight rows a block; residual: the
// residual-adding form.  plan: {warps, blocks of rows a thread block, blocks a cluster, chunks a warp stages in
// shared memory, chunks it holds in registers, row stride of the staged activations (0: read from global memory after
// the wait), dynamic shared memory in bytes}.
MS_API int ms_gemm_small_m_plan(int M, int N, int K, int gated, int residual, int sm_count, int* plan) {
  MS_REQUIRE(ms_gemm_small_m_supports(M, N, K) && plan != nullptr, "gemm_small_m_plan: M=%d (1..64), N=%d, K=%d (a multiple of 8) is not covered", M, N, K);
  const int blocks = gated ? (N + 7) / 8 : (N + 15) / 16;
  const GsmPlan p = gsm_plan(blocks, M, K, gated ? GSM_EPI_SILU_MUL : residual ? GSM_EPI_RESADD : GSM_EPI_BF16, sm_count);
  plan[0] = p.warps;
  plan[1] = p.rb;
  plan[2] = p.sh.cluster_size;
  plan[3] = p.sh.staged;
  plan[4] = p.sh.held;
  plan[5] = p.sh.xs_stride;
  plan[6] = (int)p.smem;
  return 0;
}

// out[M, N] = x[M, K] . w[N, K]^T.  x, w bfloat16; out bfloat16 (out_dtype MS_BF16) or float32.
MS_API int ms_gemm_small_m(const void* x, int ldx, const void* w, void* out, int out_dtype, int ldo, int M, int N,
                           int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ms_gemm_small_m_supports(M, N, K), "gemm_small_m: M=%d (1..64), N=%d, K=%d (a multiple of 8) is not covered", M, N, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ldo >= N, "gemm_small_m: row strides ldx=%d (a multiple of 8) ldo=%d", ldx, ldo);
  MS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_small_m: operands must be 16-byte aligned");
  const int blocks = (N + 15) / 16;
    const __nv_bfloat16* wl = (const __nv_bfloat16*)w;
  const __nv_bfloat16* wh = wl + (size_t)8 * K;
  if (out_dtype == MS_F32)
    return gsm_dispatch<GSM_EPI_F32, 0>(x, ldx, wl, wh, 16, N, N - 8, out, ldo, M, K, blocks, GsmExtra{}, sm_count, stream);
  MS_REQUIRE(out_dtype == MS_BF16, "gemm_small_m: unknown out dtype %d", out_dtype);
  return gsm_dispatch<GSM_EPI_BF16, 0>(x, ldx, wl, wh, 16, N, N - 8, out, ldo, M, K, blocks, GsmExtra{}, sm_count, stream);
}

// out[M, I] = silu(x . w_gate^T) * (x . w_up^T); w_gate, w_up: [I, K] bfloat16; out bfloat16.
MS_API int ms_gemm_small_m_silu_mul(const void* x, int ldx, const void* w_gate, const void* w_up, void* out, int ldo,
                                    int M, int I, int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ms_gemm_small_m_supports(M, I, K), "gemm_small_m_silu_mul: M=%d (1..64), I=%d, K=%d (a multiple of 8) is not covered", M, I, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ldo >= I, "gemm_small_m_silu_mul: row strides ldx=%d (a multiple of 8) ldo=%d", ldx, ldo);
  MS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w_gate % 16 == 0) && ((uintptr_t)w_up % 16 == 0),
             "gemm_small_m_silu_mul: operands must be 16-byte aligned");
  const int blocks = (I + 7) / 8;
    return gsm_dispatch<GSM_EPI_SILU_MUL, 0>(x, ldx, w_gate, w_up, 8, I, I, out, ldo, M, K, blocks, GsmExtra{}, sm_count, stream);
}

// The number of blocks of 16 columns the residual epilogue leaves sums of squares for.
MS_API int ms_gemm_small_m_stats_blocks(int N) { return (N + 15) / 16; }

// residual[M, N] += x[M, K] . w[N, K]^T in place (float32), and stats_out[m][b] = the sum of squares of the
// new residual's row m over columns [16 b, 16 b + 16).  M <= 16.
MS_API int ms_gemm_small_m_resadd(const void* x, int ldx, const void* w, float* residual, int ldr, float* stats_out,
                                  void* copy_out, int ldc, int M, int N, int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ms_gemm_small_m_supports(M, N, K) && M <= 16, "gemm_small_m_resadd: M=%d (1..16), N=%d, K=%d (a multiple of 8) is not covered", M, N, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ldr >= N, "gemm_small_m_resadd: row strides ldx=%d (a multiple of 8) ldr=%d", ldx, ldr);
  MS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "gemm_small_m_resadd: operands must be 16-byte aligned");
  const int blocks = (N + 15) / 16;
    const __nv_bfloat16* wl = (const __nv_bfloat16*)w;
  GsmExtra ex = {};
  ex.residual = residual;
  ex.ldr = ldr;
  ex.stats_out = stats_out;
  ex.copy_out = (__nv_bfloat16*)copy_out;  // optional: the new residual in bfloat16, [M][ldc]
  ex.ldc = ldc;
  MS_REQUIRE(copy_out == nullptr || ldc >= N, "gemm_small_m_resadd: the copy's row stride %d is shorter than N = %d", ldc, N);
  return gsm_dispatch<GSM_EPI_RESADD, 0>(x, ldx, wl, wl + (size_t)8 * K, 16, N, N - 8, nullptr, 0, M, K, blocks, ex, sm_count, stream);
}

// out = (x . w^T) / rms(row), where x is the residual rounded to bfloat16 [M, K] (the copy the residual epilogue
// leaves) and stats_in [M][stats_nb] its sums of squares: the RMS norm of a matrix that has the norm's weight
// folded into its columns.  With w_up, out = silu(.) * (.) of the two scaled products.  M <= 16; out bfloat16.
MS_API int ms_gemm_small_m_scaled(const void* x, int ldx, const float* stats_in, int stats_nb, float eps, const void* w,
                                  const void* w_up, void* out, int ldo, int M, int N, int K, int sm_count,
                                  cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ms_gemm_small_m_supports(M, N, K) && M <= 16, "gemm_small_m_scaled: M=%d (1..16), N=%d, K=%d (a multiple of 8) is not covered", M, N, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ldo >= N && stats_nb >= 1, "gemm_small_m_scaled: row strides ldx=%d (a multiple of 8) ldo=%d", ldx, ldo);
  MS_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)w_up % 16 == 0), "gemm_small_m_scaled: operands must be 16-byte aligned");
  GsmExtra ex = {};
  ex.stats_in = stats_in;
  ex.stats_in_nb = stats_nb;
  ex.eps = eps;
  if (w_up) {
    const int blocks = (N + 7) / 8;
    return gsm_dispatch<GSM_EPI_SILU_MUL, 1>(x, ldx, w, w_up, 8, N, N, out, ldo, M, K, blocks, ex, sm_count, stream);
  }
  const int blocks = (N + 15) / 16;
  const __nv_bfloat16* wl = (const __nv_bfloat16*)w;
  return gsm_dispatch<GSM_EPI_BF16, 1>(x, ldx, wl, wl + (size_t)8 * K, 16, N, N - 8, out, ldo, M, K, blocks, ex, sm_count, stream);
}
