// Embedding gather, residual-add + RMSNorm, SiLU-multiply, row gather.
//
// Counterparts in gqf2008/machserve (HIP source strings in
// crates/mach-model/src/kernels.rs): embed_batched :578-585, rms_norm :63-80,
// add :143-148, silu_mul :131-140.  Here the residual add is fused into the norm
// that follows it, the norm can pick rows (for the rows whose logits are wanted),
// and all reductions and the residual stream are float32.
#include <stdarg.h>

#include "launch.cuh"

static thread_local char g_error[512] = "";

void ms_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

MS_API const char* ms_last_error() { return g_error; }

int g_ms_pdl = 1;

// 0 launches every kernel the ordinary way; 1 (the default) lets kernels that support it start
// while their predecessor in the stream still runs (programmatic dependent launch).
MS_API void ms_set_pdl(int on) { g_ms_pdl = on ? 1 : 0; }

// ---------------------------------------------------------------- embedding

template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int d, int vocab) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  // ids are checked on the host; an id outside the table reads row 0 of nothing: write zeros.
  const bool ok = id >= 0 && id < vocab;
  const TW* src = table + (size_t)(ok ? id : 0) * d;
  float* dst = out + (size_t)row * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = ok ? ms_to_float(src[c]) : 0.f;
}

MS_API int ms_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int rows,
                           int d, int vocab, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && d > 0 && vocab > 0, "embed_gather: bad sizes rows=%d d=%d vocab=%d", rows, d, vocab);
  const int threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
  if (table_dtype == MS_F32)
    MS_LAUNCH_RESULT("embed_gather", ms_launch(embed_gather_kernel<float>, dim3(rows), dim3(threads), 0, stream, 1, true,
                                               (const float*)table, ids, out, d, vocab));
  else if (table_dtype == MS_BF16)
    MS_LAUNCH_RESULT("embed_gather", ms_launch(embed_gather_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, 1,
                                               true, (const __nv_bfloat16*)table, ids, out, d, vocab));
  else
    MS_REQUIRE(false, "embed_gather: unknown table dtype %d", table_dtype);
  return 0;
}

// ids[i] = sampled[from_rows[i]] where from_rows[i] >= 0: a decoding step that is sent to the device before the
// host has read the token its predecessor sampled takes that token from the sampler's output on the device.
__global__ void take_sampled_tokens_kernel(int* __restrict__ ids, const int* __restrict__ from_rows,
                                           const int* __restrict__ sampled, int n, int sampled_len) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = from_rows[i];
  if (r >= 0 && r < sampled_len) ids[i] = sampled[r];
}

MS_API int ms_take_sampled_tokens(int* ids, const int* from_rows, const int* sampled, int n, int sampled_len,
                                  cudaStream_t stream) {
  if (n == 0) return 0;
  MS_REQUIRE(n > 0 && sampled_len > 0, "take_sampled_tokens: bad sizes n=%d sampled=%d", n, sampled_len);
  take_sampled_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, from_rows, sampled, n, sampled_len);
  MS_LAUNCH_CHECK("take_sampled_tokens");
  return 0;
}

// ------------------------------------------------- residual add + RMSNorm

// One block of 256 threads per output row.  y = r * rsqrt(mean(r^2) + eps) * w with
// r = residual (+ delta).  Without `rows`, the sum is written back to `residual`.
// With `rows`, output row i is made from input row rows[i] and nothing is written back.
// The additions of a row happen in an order that depends on d alone.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ rows, int d, float eps) {
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  float* r = residual + (size_t)irow * d;
  const TD* dl = delta ? delta + (size_t)irow * d : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = r[c];
    if (dl) v += ms_to_float(dl[c]);
    if (dl && !rows) r[c] = v;
    ss += v * v;
  }
  ss = ms_block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)d + eps);
  TO* o = out + (size_t)orow * d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float v = r[c];
    if (dl && rows) v += ms_to_float(dl[c]);
    o[c] = ms_from_float<TO>(v * inv * weight[c]);
  }
}

// The same for widths that are a multiple of 8 and at most 8192: eight elements per thread and
// iteration with 16- and 32-byte accesses, the summed row kept in registers between the two passes.
// The additions of a row still happen in an order that depends on d (and the fixed block size) alone.
__device__ __forceinline__ void ms_load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ms_load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void ms_store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void ms_store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

#define NORM_VEC_THREADS 256
#define NORM_VEC_GROUPS 4  // groups of 8 elements a thread keeps: d <= 256 * 4 * 8

template <typename TD, typename TO>
__global__ void __launch_bounds__(NORM_VEC_THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const float* __restrict__ weight,
                       TO* __restrict__ out, const int* __restrict__ rows, int d, float eps) {
  __shared__ float scratch[33];
  ms_pdl_trigger();
  ms_pdl_wait();
  const int orow = blockIdx.x;
  const int irow = rows ? rows[orow] : orow;
  float* r = residual + (size_t)irow * d;
  const TD* dl = delta ? delta + (size_t)irow * d : nullptr;
  const int ngroups = d / 8;
  float v[NORM_VEC_GROUPS][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_VEC_GROUPS; ++i) {
    const int gidx = threadIdx.x + i * blockDim.x;
    if (gidx < ngroups) {
      ms_load8(r + gidx * 8, v[i]);
      if (dl) {
        float dv[8];
        ms_load8(dl + gidx * 8, dv);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] += dv[k];
        if (!rows) ms_store8(r + gidx * 8, v[i]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[i][k] * v[i][k];
    }
  }
  ss = ms_block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)d + eps);
  TO* o = out + (size_t)orow * d;
#pragma unroll
  for (int i = 0; i < NORM_VEC_GROUPS; ++i) {
    const int gidx = threadIdx.x + i * blockDim.x;
    if (gidx < ngroups) {
      float w[8];
      ms_load8(weight + gidx * 8, w);
#pragma unroll
      for (int k = 0; k < 8; ++k) w[k] = v[i][k] * inv * w[k];
      ms_store8(o + gidx * 8, w);
    }
  }
}

template <typename TD>
static int add_rmsnorm_out(float* residual, const void* delta, const float* weight, void* out, int out_dtype,
                           const int* rows, int n_out, int d, float eps, cudaStream_t stream) {
  const bool aligned = ((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) % 16 == 0;
  if (d % 8 == 0 && d <= 8 * NORM_VEC_THREADS * NORM_VEC_GROUPS && aligned) {
    // no more threads than groups of eight (rounded up to warps): narrow rows leave room for more blocks per SM.
    // The block size is a function of d alone, so the order of a row's additions still is.
    int threads = ((d / 8 + 31) / 32) * 32;
    threads = threads > NORM_VEC_THREADS ? NORM_VEC_THREADS : threads;
    if (out_dtype == MS_F32)
      MS_LAUNCH_RESULT("add_rmsnorm", ms_launch(add_rmsnorm_vec_kernel<TD, float>, dim3(n_out), dim3(threads), 0,
                                                stream, 1, true, residual, (const TD*)delta, weight, (float*)out, rows, d, eps));
    else if (out_dtype == MS_BF16)
      MS_LAUNCH_RESULT("add_rmsnorm",
                       ms_launch(add_rmsnorm_vec_kernel<TD, __nv_bfloat16>, dim3(n_out), dim3(threads), 0, stream, 1,
                                 true, residual, (const TD*)delta, weight, (__nv_bfloat16*)out, rows, d, eps));
    else
      MS_REQUIRE(false, "add_rmsnorm: unknown out dtype %d", out_dtype);
    return 0;
  }
  if (out_dtype == MS_F32)
    MS_LAUNCH_RESULT("add_rmsnorm", ms_launch(add_rmsnorm_kernel<TD, float>, dim3(n_out), dim3(256), 0, stream, 1, true,
                                              residual, (const TD*)delta, weight, (float*)out, rows, d, eps));
  else if (out_dtype == MS_BF16)
    MS_LAUNCH_RESULT("add_rmsnorm", ms_launch(add_rmsnorm_kernel<TD, __nv_bfloat16>, dim3(n_out), dim3(256), 0, stream, 1,
                                              true, residual, (const TD*)delta, weight, (__nv_bfloat16*)out, rows, d, eps));
  else
    MS_REQUIRE(false, "add_rmsnorm: unknown out dtype %d", out_dtype);
  return 0;
}

MS_API int ms_add_rmsnorm(float* residual, const void* delta, int delta_dtype, const float* weight, void* out,
                          int out_dtype, const int* rows, int n_out, int d, float eps, cudaStream_t stream) {
  if (n_out == 0) return 0;
  MS_REQUIRE(n_out > 0 && d > 0, "add_rmsnorm: bad sizes n_out=%d d=%d", n_out, d);
  if (delta_dtype == MS_F32 || delta == nullptr)
    return add_rmsnorm_out<float>(residual, delta, weight, out, out_dtype, rows, n_out, d, eps, stream);
  if (delta_dtype == MS_BF16)
    return add_rmsnorm_out<__nv_bfloat16>(residual, delta, weight, out, out_dtype, rows, n_out, d, eps, stream);
  MS_REQUIRE(false, "add_rmsnorm: unknown delta dtype %d", delta_dtype);
  return 0;
}

// out[r, c] += bias[c] in float32, rounded to out's type: the bias of a bfloat16 matrix product, whose kernels
// (this library's and cuBLAS) add none.  out is [rows, n] with row stride ld.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, int n, int ld, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / n;
  const int c = (int)(i - r * n);
  T* p = out + r * ld + c;
  *p = ms_from_float<T>(ms_to_float(*p) + bias[c]);
}

MS_API int ms_add_bias(void* out, int dtype, const float* bias, int rows, int n, int ld, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && n > 0 && ld >= n, "add_bias: bad sizes rows=%d n=%d ld=%d", rows, n, ld);
  const size_t total = (size_t)rows * n;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32)
    add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, bias, n, ld, total);
  else if (dtype == MS_BF16)
    add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, bias, n, ld, total);
  else
    MS_REQUIRE(false, "add_bias: unknown dtype %d", dtype);
  MS_LAUNCH_CHECK("add_bias");
  return 0;
}

// ---------------------------------------------------------------- SiLU * up

// gate_up is [rows, 2*inter]: the gate in columns [0, inter), up in [inter, 2*inter).
// out[r, c] = gate / (1 + exp(-gate)) * up, computed in float32 with the accurate expf.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / inter;
  const int c = (int)(i - r * inter);
  const float g = ms_to_float(gate_up[r * 2 * inter + c]);
  const float u = ms_to_float(gate_up[r * 2 * inter + inter + c]);
  out[i] = ms_from_float<T>(g / (1.f + expf(-g)) * u);
}

// Eight columns per thread with 16-byte accesses, for bfloat16 and widths that are a multiple of 8.
__global__ void silu_mul_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter) {
  const int row = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= inter) return;
  float g[8], u[8];
  ms_load8(gate_up + (size_t)row * 2 * inter + c, g);
  ms_load8(gate_up + (size_t)row * 2 * inter + inter + c, u);
#pragma unroll
  for (int k = 0; k < 8; ++k) g[k] = g[k] / (1.f + expf(-g[k])) * u[k];
  ms_store8(out + (size_t)row * inter + c, g);
}

MS_API int ms_silu_mul(const void* gate_up, void* out, int dtype, int rows, int inter, cudaStream_t stream) {
  if (rows == 0) return 0;
  MS_REQUIRE(rows > 0 && inter > 0, "silu_mul: bad sizes rows=%d inter=%d", rows, inter);
  if (dtype == MS_BF16 && inter % 8 == 0 && rows <= 65535 && ((uintptr_t)gate_up | (uintptr_t)out) % 16 == 0) {
    dim3 grid((inter / 8 + 127) / 128, rows);
    silu_mul_vec_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter);
    MS_LAUNCH_CHECK("silu_mul");
    return 0;
  }
  const size_t total = (size_t)rows * inter;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MS_F32)
    silu_mul_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
  else if (dtype == MS_BF16)
    silu_mul_kernel<__nv_bfloat16>
        <<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
  else
    MS_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
  MS_LAUNCH_CHECK("silu_mul");
  return 0;
}
