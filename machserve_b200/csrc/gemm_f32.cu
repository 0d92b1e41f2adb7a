// float32 matrix product on the CUDA cores: out[M, N] = x[M, K] . W[N, K]^T (+ bias).
//
// The true 32-bit path multiplies with this kernel: plain fused multiply-adds in
// float32, no tensor cores and no reduced-precision mode.  Every output element is
// the sum over k = 0..K-1 in ascending order, whatever M is and wherever the row
// lies in the batch, so a row's result does not depend on what else is computed
// with it.  The reference's float32 mode calls hipBLAS sgemm here
// (crates/mach-model/src/kernels.rs:5772-5798 of gqf2008/machserve).
#include "common.cuh"

#define G32_BM 128
#define G32_BN 128
#define G32_BK 16

// Four bytes from global to shared memory without passing through registers; `valid` false: a zero instead.
__device__ __forceinline__ void g32_cp_async4(float* smem, const float* gmem, bool valid) {
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(n));
}

// Sixteen bytes from global to shared memory without passing through registers; `valid` false: zeros instead.
__device__ __forceinline__ void g32_cp_async16(float* smem, const float* gmem, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(n));
}

// A tile of 128 x 128 outputs per block of 256 threads, 8 x 8 per thread (rows tm, tm + 16, ..., columns tn, tn + 16, ...:
// a quarter warp's 16-byte reads of rows 80 bytes apart fall into different banks), K in steps of 16 through two stages: the copies of the next
// step are on their way while this one is multiplied.  The operands lie in shared memory as they lie in global memory
// ([row][k], rows padded to 20 floats); every thread adds its products for k = 0..K-1 in ascending order.
// VEC: K and the row strides are multiples of 4 and the bases 16-byte aligned (16-byte copies); else element by element.
template <bool VEC>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ out, int ldo, int M, int N, int K) {
  constexpr int LD = G32_BK + 4;
  __shared__ __align__(16) float xs[2][G32_BM][LD];
  __shared__ __align__(16) float ws[2][G32_BN][LD];
  const int m0 = blockIdx.y * G32_BM, n0 = blockIdx.x * G32_BN;
  const int tid = threadIdx.x;
  const int tm = tid / 16, tn = tid % 16;  // this thread's rows tm, tm + 16, ..., tm + 112; its columns tn, tn + 16, ...
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  auto request = [&](int stage, int k0) {
    if (VEC) {
      // 128 rows x 16 k of each operand = 512 pieces of 16 bytes: two per thread
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int e = tid + i * 256, r = e >> 2, kq = (e & 3) * 4;
        const int gk = k0 + kq;
        const bool xo = m0 + r < M && gk < K, wo = n0 + r < N && gk < K;
        g32_cp_async16(&xs[stage][r][kq], xo ? x + (size_t)(m0 + r) * ldx + gk : x, xo);
        g32_cp_async16(&ws[stage][r][kq], wo ? w + (size_t)(n0 + r) * K + gk : w, wo);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = tid + i * 256, r = e >> 4, kk = e & 15;
        const int gk = k0 + kk;
        const bool xo = m0 + r < M && gk < K, wo = n0 + r < N && gk < K;
        g32_cp_async4(&xs[stage][r][kk], xo ? x + (size_t)(m0 + r) * ldx + gk : x, xo);
        g32_cp_async4(&ws[stage][r][kk], wo ? w + (size_t)(n0 + r) * K + gk : w, wo);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  request(0, 0);
  for (int k0 = 0, stage = 0; k0 < K; k0 += G32_BK, stage ^= 1) {
    if (k0 + G32_BK < K) {
      request(stage ^ 1, k0 + G32_BK);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int kq = 0; kq < G32_BK; kq += 4) {
      float4 a[8], b[8];  // four k of each of the thread's eight rows and eight columns
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        a[i] = *reinterpret_cast<const float4*>(&xs[stage][tm + 16 * i][kq]);
        b[i] = *reinterpret_cast<const float4*>(&ws[stage][tn + 16 * i][kq]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
          acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
          acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
          acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
        }
    }
    __syncthreads();  // all are done with this stage before the copies after the next are requested into it
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + tm + 16 * i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + tn + 16 * j;
      if (n < N) out[(size_t)m * ldo + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

// The same sums for up to 16 rows (decoding), laid out for streaming the weights: a block of 128 threads takes COLS
// weight rows for ROWS rows of x (16 x 8, or 8 x 16 when there are at most 8 rows, so that no thread works on a row that
// is not there); thread (n, m) owns out[m][n] and adds its products for k = 0..K-1 in ascending order, exactly as the
// kernel above does, so a row's result is the same bit for bit whichever of the kernels computed it.  With 8 weight
// rows per block a matrix of 896 rows is spread over 112 blocks (the kernel above would use 7).
// A thread's sum is one chain of dependent multiply-adds; what can be hidden is everything else: the copies of the next
// 128 k are on their way while this thread adds up the present ones, and the loop over a full stage is unrolled, so
// that the reads of shared memory for the next steps are issued while the chain waits for itself.
#define G32S_KT 128

template <int ROWS, int COLS, bool VEC>
__global__ void __launch_bounds__(ROWS * COLS)
gemm_f32_small_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                      float* __restrict__ out, int ldo, int M, int N, int K) {
  constexpr int THREADS = ROWS * COLS;
  __shared__ __align__(16) float ws[2][COLS][G32S_KT + 4];
  __shared__ __align__(16) float xs[2][ROWS][G32S_KT + 4];
  const int tid = threadIdx.x, nl = tid / ROWS, m = tid % ROWS;
  const int n0 = blockIdx.x * COLS;
  auto request = [&](int stage, int k0) {
    if (VEC) {  // 16 bytes a copy: K, ldx multiples of 4, both operands 16-byte aligned
#pragma unroll
      for (int e = tid; e < COLS * (G32S_KT / 4); e += THREADS) {
        const int i = e / (G32S_KT / 4), kq = (e % (G32S_KT / 4)) * 4;
        const bool ok = n0 + i < N && k0 + kq < K;
        g32_cp_async16(&ws[stage][i][kq], ok ? w + (size_t)(n0 + i) * K + k0 + kq : w, ok);
      }
#pragma unroll
      for (int e = tid; e < ROWS * (G32S_KT / 4); e += THREADS) {
        const int i = e / (G32S_KT / 4), kq = (e % (G32S_KT / 4)) * 4;
        const bool ok = i < M && k0 + kq < K;
        g32_cp_async16(&xs[stage][i][kq], ok ? x + (size_t)i * ldx + k0 + kq : x, ok);
      }
    } else {
#pragma unroll
      for (int e = tid; e < COLS * G32S_KT; e += THREADS) {
        const int i = e / G32S_KT, kk = e % G32S_KT;
        const bool ok = n0 + i < N && k0 + kk < K;
        g32_cp_async4(&ws[stage][i][kk], ok ? w + (size_t)(n0 + i) * K + k0 + kk : w, ok);
      }
#pragma unroll
      for (int e = tid; e < ROWS * G32S_KT; e += THREADS) {
        const int i = e / G32S_KT, kk = e % G32S_KT;
        const bool ok = i < M && k0 + kk < K;
        g32_cp_async4(&xs[stage][i][kk], ok ? x + (size_t)i * ldx + k0 + kk : x, ok);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  float acc = 0.f;
  request(0, 0);
  for (int k0 = 0, stage = 0; k0 < K; k0 += G32S_KT, stage ^= 1) {
    if (k0 + G32S_KT < K) {
      request(stage ^ 1, k0 + G32S_KT);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    const float* xr = xs[stage][m];
    const float* wr = ws[stage][nl];
    if (K - k0 >= G32S_KT) {  // a full stage: a loop of known length, unrolled
#pragma unroll 8
      for (int c = 0; c < G32S_KT; c += 4) {
        const float4 a = *reinterpret_cast<const float4*>(xr + c);
        const float4 b = *reinterpret_cast<const float4*>(wr + c);
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
        acc = fmaf(a.z, b.z, acc);
        acc = fmaf(a.w, b.w, acc);
      }
    } else {
      const int kn = K - k0;
      int c = 0;
      for (; c + 4 <= kn; c += 4) {
        const float4 a = *reinterpret_cast<const float4*>(xr + c);
        const float4 b = *reinterpret_cast<const float4*>(wr + c);
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
        acc = fmaf(a.z, b.z, acc);
        acc = fmaf(a.w, b.w, acc);
      }
      for (; c < kn; ++c) acc = fmaf(xr[c], wr[c], acc);
    }
    __syncthreads();  // all are done with this stage before the copies after the next are requested into it
  }
  const int n = n0 + nl;
  if (m < M && n < N) out[(size_t)m * ldo + n] = acc + (bias ? bias[n] : 0.f);
}

// x: [M, K] with row stride ldx; w: [N, K] dense; out: [M, N] with row stride ldo.
MS_API int ms_gemm_f32(const float* x, int ldx, const float* w, const float* bias, float* out, int ldo, int M, int N,
                       int K, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(M > 0 && N > 0 && K > 0 && ldx >= K && ldo >= N, "gemm_f32: bad sizes M=%d N=%d K=%d ldx=%d ldo=%d", M, N, K,
             ldx, ldo);
  const bool vec = K % 4 == 0 && ldx % 4 == 0 && ((uintptr_t)x | (uintptr_t)w) % 16 == 0;
  if (M <= 16) {
#define MS_G32_SMALL(ROWS, COLS)                                                                                       \
  do {                                                                                                                 \
    if (vec)                                                                                                           \
      gemm_f32_small_kernel<ROWS, COLS, true><<<(N + COLS - 1) / COLS, ROWS * COLS, 0, stream>>>(x, ldx, w, bias, out, ldo, M, N, K); \
    else                                                                                                               \
      gemm_f32_small_kernel<ROWS, COLS, false><<<(N + COLS - 1) / COLS, ROWS * COLS, 0, stream>>>(x, ldx, w, bias, out, ldo, M, N, K); \
  } while (0)
    if (M <= 8)
      MS_G32_SMALL(8, 16);
    else
      MS_G32_SMALL(16, 8);
#undef MS_G32_SMALL
    MS_LAUNCH_CHECK("gemm_f32");
    return 0;
  }
  dim3 grid((N + G32_BN - 1) / G32_BN, (M + G32_BM - 1) / G32_BM);
  MS_REQUIRE(grid.y <= 65535, "gemm_f32: %d rows are more than one launch takes", M);
  if (vec)
    gemm_f32_kernel<true><<<grid, 256, 0, stream>>>(x, ldx, w, bias, out, ldo, M, N, K);
  else
    gemm_f32_kernel<false><<<grid, 256, 0, stream>>>(x, ldx, w, bias, out, ldo, M, N, K);
  MS_LAUNCH_CHECK("gemm_f32");
  return 0;
}
