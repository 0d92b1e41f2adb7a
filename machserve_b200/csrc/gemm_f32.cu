// float32 matrix product on the CUDA cores: out[M, N] = x[M, K] . W[N, K]^T (+ bias).
//
// The true 32-bit path multiplies with this kernel: plain fused multiply-adds in
// float32, no tensor cores and no reduced-precision mode.  Every output element is
// the sum over k = 0..K-1 in ascending order, whatever M is and wherever the row
// lies in the batch, so a row's result does not depend on what else is computed
// with it.  The reference's float32 mode calls hipBLAS sgemm here
// (crates/mach-model/src/kernels.rs:5772-5798 of gqf2008/machserve).
#include "common.cuh"

#define G32_BM 64
#define G32_BN 64
#define G32_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ out, int ldo, int M, int N, int K) {
  __shared__ float xs[G32_BK][G32_BM + 4];
  __shared__ float ws[G32_BK][G32_BN + 4];
  const int m0 = blockIdx.y * G32_BM, n0 = blockIdx.x * G32_BN;
  const int tid = threadIdx.x;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;  // this thread's 4x4 corner in the tile
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += G32_BK) {
    // 64 rows x 16 k of each operand; four elements per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / G32_BK, kk = e % G32_BK;
      const int gk = k0 + kk;
      xs[kk][r] = (m0 + r < M && gk < K) ? x[(size_t)(m0 + r) * ldx + gk] : 0.f;
      ws[kk][r] = (n0 + r < N && gk < K) ? w[(size_t)(n0 + r) * K + gk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < G32_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n < N) out[(size_t)m * ldo + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

// The same sums for up to 16 rows (decoding), laid out for streaming the weights: a block of 128 threads takes 8
// weight rows, thread (n, m) owns out[m][n] and adds its products for k = 0..K-1 in ascending order, exactly as
// the kernel above does, so a row's result is the same bit for bit whichever of the two computed it.  With 8
// weight rows per block a matrix of 896 rows is spread over 112 blocks (the kernel above would use 14).
#define G32S_ROWS 16
#define G32S_COLS 8
#define G32S_KT 128

// Four bytes from global to shared memory without passing through registers; `valid` false: a zero instead.
__device__ __forceinline__ void g32_cp_async4(float* smem, const float* gmem, bool valid) {
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(n));
}

__global__ void __launch_bounds__(G32S_ROWS * G32S_COLS)
gemm_f32_small_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, const float* __restrict__ bias,
                      float* __restrict__ out, int ldo, int M, int N, int K) {
  // two stages: the copies of the next 128 k are on their way while this thread adds up the present ones
  __shared__ __align__(16) float ws[2][G32S_COLS][G32S_KT + 4];
  __shared__ __align__(16) float xs[2][G32S_ROWS][G32S_KT + 4];
  const int tid = threadIdx.x, nl = tid >> 4, m = tid & 15;
  const int n0 = blockIdx.x * G32S_COLS;
  auto request = [&](int stage, int k0) {
    const int gk = k0 + tid;
#pragma unroll
    for (int i = 0; i < G32S_COLS; ++i) {  // 8 x 128 weights: a row of 128 consecutive k per 128 threads
      const bool ok = n0 + i < N && gk < K;
      g32_cp_async4(&ws[stage][i][tid], ok ? w + (size_t)(n0 + i) * K + gk : w, ok);
    }
#pragma unroll
    for (int i = 0; i < G32S_ROWS; ++i) {
      const bool ok = i < M && gk < K;
      g32_cp_async4(&xs[stage][i][tid], ok ? x + (size_t)i * ldx + gk : x, ok);
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
    const int kn = K - k0 < G32S_KT ? K - k0 : G32S_KT;
    int c = 0;
    for (; c + 4 <= kn; c += 4) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[stage][m][c]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[stage][nl][c]);
      acc = fmaf(a.x, b.x, acc);
      acc = fmaf(a.y, b.y, acc);
      acc = fmaf(a.z, b.z, acc);
      acc = fmaf(a.w, b.w, acc);
    }
    for (; c < kn; ++c) acc = fmaf(xs[stage][m][c], ws[stage][nl][c], acc);
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
  if (M <= G32S_ROWS) {
    gemm_f32_small_kernel<<<(N + G32S_COLS - 1) / G32S_COLS, G32S_ROWS * G32S_COLS, 0, stream>>>(x, ldx, w, bias, out, ldo, M, N, K);
    MS_LAUNCH_CHECK("gemm_f32");
    return 0;
  }
  dim3 grid((N + G32_BN - 1) / G32_BN, (M + G32_BM - 1) / G32_BM);
  MS_REQUIRE(grid.y <= 65535, "gemm_f32: %d rows are more than one launch takes", M);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, ldx, w, bias, out, ldo, M, N, K);
  MS_LAUNCH_CHECK("gemm_f32");
  return 0;
}
