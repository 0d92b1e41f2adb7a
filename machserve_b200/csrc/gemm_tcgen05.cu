// Matrix product for many rows (portions of prompts) on the fifth-generation tensor cores:
// out[M, N] = x[M, K] . W[N, K]^T, bfloat16 operands, float32 accumulation in tensor memory.
//
// One block computes a 128 x 128 tile.  Warp 0 (one thread) brings 128 x 64 tiles of x and W
// into a ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle); warp 1
// (one thread) issues tcgen05.mma, four per stage (K = 16 each), accumulating into 128 columns
// of tensor memory, and releases each stage with tcgen05.commit; warps 2-5 read the finished
// accumulator with tcgen05.ld and write the result.  Both operands are K-major, which is how
// activations [M, K] and weights [N, K] lie in memory.  The W tile is loaded as two boxes of 64
// rows; for the gated feed-forward the second box comes from the `up` half of the weights, so
// that an output's gate and up values meet in one accumulator row and the epilogue writes
// silu(gate) * up directly.
//
// Every wait on an mbarrier is bounded: after the limit the block records an error code that
// the host reads (ms_gemm_tc_status), gives its copies in flight time to land, frees its tensor
// memory and returns.  No load uses cluster multicast.
//
// The reference multiplies through its vendor library here (hipBLAS GemmEx,
// crates/mach-model/src/kernels.rs:6416-6455 of gqf2008/machserve).
#include <cuda.h>

#include "common.cuh"

#define TC_BM 128
#define TC_BN 128
#define TC_BK 64
#define TC_STAGES 3  // 96 KB of tiles: two blocks fit on an SM, one's epilogue overlaps the other's main loop
#define TC_THREADS 192
#define TC_STAGE_BYTES ((TC_BM + TC_BN) * TC_BK * 2)
#define TC_WAIT_LIMIT (1 << 21)

enum { TC_EPI_BF16 = 0, TC_EPI_F32 = 1, TC_EPI_SILU_MUL = 2 };

__device__ int g_tc_error = 0;  // 0, or a code that says which wait gave up: 1 producer, 2 issuer, 3 epilogue

__device__ __forceinline__ unsigned tc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity to complete, at most TC_WAIT_LIMIT polls.  Returns false when it
// gave up or when another thread of the block already has.
__device__ __forceinline__ bool tc_mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int code,
                                             int limit = TC_WAIT_LIMIT) {
  for (int it = 0; it < limit; ++it) {
    if (tc_mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (it > 256) __nanosleep(40);
  }
  *abort_flag = 1;
  atomicCAS(&g_tc_error, 0, code);
  return false;
}

__device__ __forceinline__ void tc_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major tile of 128-byte rows with the 128-byte swizzle: start
// address, stride of 1024 bytes between groups of eight rows, descriptor version 1, layout type 2.
__device__ __forceinline__ unsigned long long tc_smem_desc(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);       // bits 0-13: start address / 16
  d |= (unsigned long long)(1024 >> 4) << 32;              // bits 32-45: stride byte offset / 16
  d |= 1ull << 46;                                         // bits 46-47: version
  d |= 2ull << 61;                                         // bits 61-63: 128-byte swizzle
  return d;
}

// Instruction descriptor for kind::f16: float32 accumulator, bfloat16 A and B, both K-major, M x N.
__host__ __device__ constexpr unsigned tc_instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(unsigned tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, "
      "[%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Stores 32 consecutive outputs of one row as bfloat16: 16-byte stores where the row allows it.
__device__ __forceinline__ void tc_store_row_bf16(__nv_bfloat16* dst, const float (&v)[32], int valid) {
  if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 u;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
      *reinterpret_cast<uint4*>(dst + i) = u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

struct TcShared {
  unsigned long long full[TC_STAGES];
  unsigned long long empty[TC_STAGES];
  unsigned long long done;
  unsigned tmem_base;
  int abort_flag;
};

// n1_offset: where the second 64 rows of the W tile start relative to the first (64 for a plain product;
// the number of gate rows for the gated form, whose block covers 64 outputs).
template <int EPI>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    void* __restrict__ out, int ldo, int M, int N, int K, int n1_offset) {
  extern __shared__ unsigned char smem_raw[];
  // the swizzle works on absolute address bits: tiles start at multiples of 1024 bytes
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  TcShared* sh = reinterpret_cast<TcShared*>(tiles + TC_STAGES * TC_STAGE_BYTES);
  volatile int* abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM;
  const int out_cols = EPI == TC_EPI_SILU_MUL ? 64 : TC_BN;  // output columns of a block
  const int n0 = blockIdx.x * out_cols;
  const int kt_count = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      tc_mbar_init(tc_smem(&sh->full[s]), 1);
      tc_mbar_init(tc_smem(&sh->empty[s]), 1);
    }
    tc_mbar_init(tc_smem(&sh->done), 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {  // this warp owns the tensor memory: 128 columns of 128 lanes, float32
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(&sh->tmem_base)),
                 "r"(TC_BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = sh->tmem_base;

  if (warp == 0 && lane == 0) {
    // producer: fill the ring
    for (int kt = 0; kt < kt_count; ++kt) {
      const int s = kt % TC_STAGES;
      if (kt >= TC_STAGES && !tc_mbar_wait(tc_smem(&sh->empty[s]), ((kt / TC_STAGES) - 1) & 1, abort_flag, 1)) break;
      const unsigned a_dst = tc_smem(tiles + s * TC_STAGE_BYTES);
      const unsigned b_dst = a_dst + TC_BM * TC_BK * 2;
      const unsigned bar = tc_smem(&sh->full[s]);
      tc_mbar_expect_tx(bar, TC_STAGE_BYTES);
      tc_tma_load_2d(a_dst, &map_x, kt * TC_BK, m0, bar);
      tc_tma_load_2d(b_dst, &map_w, kt * TC_BK, n0, bar);
      tc_tma_load_2d(b_dst + 64 * TC_BK * 2, &map_w, kt * TC_BK, n0 + n1_offset, bar);
    }
  } else if (warp == 1 && lane == 0) {
    // issuer: four K = 16 instructions per stage, then the stage goes back to the producer
    const unsigned idesc = tc_instr_desc(TC_BM, TC_BN);
    bool ok = true;
    for (int kt = 0; kt < kt_count && ok; ++kt) {
      const int s = kt % TC_STAGES;
      ok = tc_mbar_wait(tc_smem(&sh->full[s]), (kt / TC_STAGES) & 1, abort_flag, 2);
      if (!ok) break;
      tc_fence_after();
      const unsigned a_src = tc_smem(tiles + s * TC_STAGE_BYTES);
      const unsigned b_src = a_src + TC_BM * TC_BK * 2;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k)
        tc_mma(tmem, tc_smem_desc(a_src + k * 32), tc_smem_desc(b_src + k * 32), idesc, (kt | k) != 0);
      tc_commit(tc_smem(&sh->empty[s]));
    }
    if (ok) tc_commit(tc_smem(&sh->done));
  } else if (warp >= 2) {
    // epilogue: a warp reads the 32 accumulator rows (lanes) it may touch, thread = row
    if (tc_mbar_wait(tc_smem(&sh->done), 0, abort_flag, 3)) {
      tc_fence_after();
      const int group = warp & 3;
      const int m = m0 + group * 32 + lane;
      const unsigned row_addr = tmem + ((unsigned)(group * 32) << 16);
      if (EPI == TC_EPI_SILU_MUL) {
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
          float g[32], u[32];
          tc_ld32(row_addr + c, g);
          tc_ld32(row_addr + 64 + c, u);
          if (m < M && n0 + c < N) {
#pragma unroll
            for (int i = 0; i < 32; ++i) g[i] = g[i] / (1.f + expf(-g[i])) * u[i];
            tc_store_row_bf16(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n0 + c, g, N - n0 - c);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < TC_BN; c += 32) {
          float v[32];
          tc_ld32(row_addr + c, v);
          if (m < M) {
            if (EPI == TC_EPI_F32) {
              float* dst = reinterpret_cast<float*>(out) + (size_t)m * ldo + n0 + c;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (n0 + c + i < N) dst[i] = v[i];
            } else if (n0 + c < N) {
              tc_store_row_bf16(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n0 + c, v, N - n0 - c);
            }
          }
        }
      }
    }
  }
  // leave together; after a wait that gave up, give the copies in flight time to land before the
  // shared memory goes away
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TC_BN) : "memory");
  }
}

// ------------------------------------------------------------------------------------ host

typedef CUresult (*TcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TcEncodeFn tc_encode_fn() {
  static TcEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (TcEncodeFn)p;
  }
  return fn;
}

// A map over a row-major bfloat16 matrix [rows, cols] (row stride ld elements) with boxes of box_rows x 64.
static int tc_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  TcEncodeFn fn = tc_encode_fn();
  MS_REQUIRE(fn != nullptr, "gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MS_REQUIRE(r == CUDA_SUCCESS, "gemm_tcgen05: cuTensorMapEncodeTiled failed with %d (base %p rows %d cols %d ld %d)", (int)r,
             base, rows, cols, ld);
  return 0;
}

template <int EPI>
static int tc_launch(const CUtensorMap& mx, const CUtensorMap& mw, void* out, int ldo, int M, int N, int K, int n1_offset,
                     dim3 grid, cudaStream_t stream) {
  const size_t smem = (size_t)TC_STAGES * TC_STAGE_BYTES + sizeof(TcShared) + 1024;
  auto kern = gemm_tcgen05_kernel<EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      ms_set_error("gemm_tcgen05: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  kern<<<grid, TC_THREADS, smem, stream>>>(mx, mw, out, ldo, M, N, K, n1_offset);
  MS_LAUNCH_CHECK("gemm_tcgen05");
  return 0;
}

MS_API int ms_gemm_tc_supports(int M, int N, int K) { return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0; }

// 0 if no block ever gave up a wait; else the code of the first that did (1 producer, 2 issuer, 3 epilogue).
// Synchronizes the device.  `reset` clears the code.
MS_API int ms_gemm_tc_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
  if (reset && v) {
    int z = 0;
    cudaMemcpyToSymbol(g_tc_error, &z, sizeof(int));
  }
  return v;
}

// A wait that runs out, in the form that cannot hang: one thread waits `polls` polls on a barrier in its own
// shared memory that nothing arrives on, through the helper that every wait of the kernels here uses; no
// copy and no tensor memory is involved.  Leaves code 9 for ms_gemm_tc_status.
__global__ void tc_wait_probe_kernel(int polls) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc_mbar_init(tc_smem(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    tc_mbar_wait(tc_smem(&bar), 0, &abort_flag, 9, polls);
  }
}
MS_API int ms_gemm_tc_wait_probe(int polls, cudaStream_t stream) {
  MS_REQUIRE(polls >= 1 && polls <= 100000, "gemm_tc_wait_probe: 1 to 100000 polls");
  tc_wait_probe_kernel<<<1, 32, 0, stream>>>(polls);
  MS_LAUNCH_CHECK("gemm_tc_wait_probe");
  return 0;
}

// out[M, N] = x[M, K] . w[N, K]^T; x, w bfloat16 (row strides ldx, K); out bfloat16 or float32.
MS_API int ms_gemm_tc(const void* x, int ldx, const void* w, void* out, int out_dtype, int ldo, int M, int N, int K,
                      cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ms_gemm_tc_supports(M, N, K), "gemm_tcgen05: M=%d N=%d K=%d (a multiple of 8) is not covered", M, N, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ldo >= N && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0),
             "gemm_tcgen05: operands must be 16-byte aligned with row strides that are multiples of 8");
  CUtensorMap mx, mw;
  if (int rc = tc_make_map(&mx, x, M, K, ldx, TC_BM)) return rc;
  if (int rc = tc_make_map(&mw, w, N, K, K, 64)) return rc;
  dim3 grid((N + TC_BN - 1) / TC_BN, (M + TC_BM - 1) / TC_BM);
  if (out_dtype == MS_F32) return tc_launch<TC_EPI_F32>(mx, mw, out, ldo, M, N, K, 64, grid, stream);
  MS_REQUIRE(out_dtype == MS_BF16, "gemm_tcgen05: unknown out dtype %d", out_dtype);
  return tc_launch<TC_EPI_BF16>(mx, mw, out, ldo, M, N, K, 64, grid, stream);
}

// out[M, I] = silu(x . w[0:I]^T) * (x . w[I:2I]^T); w is [2I, K] with the gate rows first; out bfloat16.
MS_API int ms_gemm_tc_silu_mul(const void* x, int ldx, const void* w_gate_up, void* out, int ldo, int M, int I, int K,
                               cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ms_gemm_tc_supports(M, I, K), "gemm_tcgen05_silu_mul: M=%d I=%d K=%d (a multiple of 8) is not covered", M, I, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ldo >= I && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w_gate_up % 16 == 0),
             "gemm_tcgen05_silu_mul: operands must be 16-byte aligned with row strides that are multiples of 8");
  CUtensorMap mx, mw;
  if (int rc = tc_make_map(&mx, x, M, K, ldx, TC_BM)) return rc;
  // one map over all 2I rows: a block's first box holds 64 gate rows, its second the up rows of the same
  // outputs; where I is no multiple of 64 the last block's boxes run past their half, into columns of the
  // accumulator that the epilogue does not store
  if (int rc = tc_make_map(&mw, w_gate_up, 2 * I, K, K, 64)) return rc;
  dim3 grid((I + 63) / 64, (M + TC_BM - 1) / TC_BM);
  return tc_launch<TC_EPI_SILU_MUL>(mx, mw, out, ldo, M, I, K, I, grid, stream);
}

// ------------------------------------------------------------------------------------------------
// The second operand given as [K, N] (N contiguous): "MN-major" for the tensor core.  This is how the
// values of attention lie in the cache ([key][head_dim]) when they multiply the probabilities, so this
// small product pins down the descriptor for that layout.  One block, one 128 x 64 output tile per
// 64-wide column block, K in steps of 64.
__device__ __forceinline__ unsigned long long tc_smem_desc_mn(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
  d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kn_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_b,
                       float* __restrict__ out, int ldo, int M, int N, int K, unsigned lbo_bytes, unsigned sbo_bytes,
                       unsigned kadv_bytes) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // the tiles sit in the middle of a generous allocation: an operand fetch that strays while the descriptor
  // fields are being established still reads this block's own shared memory
  unsigned char* a_tile = tiles + 65536;            // [128 rows][64 k] K-major, 16 KB
  unsigned char* b_tile = tiles + 65536 + 16384;    // [64 k][64 n] N contiguous, 8 KB
  TcShared* sh = reinterpret_cast<TcShared*>(tiles);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * 64;
  const int kt_count = (K + 63) / 64;
  if (threadIdx.x == 0) {
    tc_mbar_init(tc_smem(&sh->full[0]), 1);
    tc_mbar_init(tc_smem(&sh->empty[0]), 1);
    tc_mbar_init(tc_smem(&sh->done), 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(&sh->tmem_base)), "r"(64) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = sh->tmem_base;
  if (warp == 0 && lane == 0) {
    for (int kt = 0; kt < kt_count; ++kt) {  // one stage: load, wait for its use, load again
      if (kt > 0 && !tc_mbar_wait(tc_smem(&sh->empty[0]), (kt - 1) & 1, abort_flag, 1)) break;
      const unsigned bar = tc_smem(&sh->full[0]);
      tc_mbar_expect_tx(bar, 16384 + 8192);
      tc_tma_load_2d(tc_smem(a_tile), &map_x, kt * 64, m0, bar);
      tc_tma_load_2d(tc_smem(b_tile), &map_b, n0, kt * 64, bar);
    }
  } else if (warp == 1 && lane == 0) {
    // as tc_instr_desc, N = 64, with bit 16 set: the second operand is MN-major
    const unsigned idesc = tc_instr_desc(TC_BM, 64) | (1u << 16);
    bool ok = true;
    for (int kt = 0; kt < kt_count && ok; ++kt) {
      ok = tc_mbar_wait(tc_smem(&sh->full[0]), kt & 1, abort_flag, 2);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < 4; ++k)
        tc_mma(tmem, tc_smem_desc(tc_smem(a_tile) + k * 32), tc_smem_desc_mn(tc_smem(b_tile) + k * kadv_bytes, lbo_bytes, sbo_bytes),
               idesc, (kt | k) != 0);
      tc_commit(tc_smem(&sh->empty[0]));
    }
    if (ok) tc_commit(tc_smem(&sh->done));
  } else if (warp >= 2) {
    if (tc_mbar_wait(tc_smem(&sh->done), 0, abort_flag, 3)) {
      tc_fence_after();
      const int group = warp & 3;
      const int m = m0 + group * 32 + lane;
      for (int c = 0; c < 64; c += 32) {
        float v[32];
        tc_ld32(tmem + ((unsigned)(group * 32) << 16) + c, v);
        if (m < M)
          for (int i = 0; i < 32; ++i)
            if (n0 + c + i < N) out[(size_t)m * ldo + n0 + c + i] = v[i];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(64) : "memory");
}

// out[M, N] (float32) = x[M, K] . b[K, N]; x bfloat16 [M, K], b bfloat16 [K, N] with N contiguous (row stride ldb).
// lbo/sbo/kadv: the descriptor fields for b's tiles (bytes); 0, 1024, 2048 are the values the engine uses.
MS_API int ms_gemm_tc_kn(const void* x, int ldx, const void* b, int ldb, float* out, int ldo, int M, int N, int K,
                         int lbo_bytes, int sbo_bytes, int kadv_bytes, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(M >= 1 && N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0, "gemm_tcgen05_kn: M=%d N=%d K=%d (N and K multiples of 8)", M, N, K);
  MS_REQUIRE(ldx % 8 == 0 && ldb % 8 == 0 && ldx >= K && ldb >= N && ldo >= N, "gemm_tcgen05_kn: bad row strides");
  CUtensorMap mx, mb;
  if (int rc = tc_make_map(&mx, x, M, K, ldx, TC_BM)) return rc;
  if (int rc = tc_make_map(&mb, b, K, N, ldb, 64)) return rc;
  const size_t smem = 200 * 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    MS_REQUIRE(e == cudaSuccess, "gemm_tcgen05_kn: cannot get shared memory: %s", cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((N + 63) / 64, (M + TC_BM - 1) / TC_BM);
  gemm_tcgen05_kn_kernel<<<grid, TC_THREADS, smem, stream>>>(mx, mb, out, ldo, M, N, K, (unsigned)lbo_bytes, (unsigned)sbo_bytes,
                                                              (unsigned)kadv_bytes);
  MS_LAUNCH_CHECK("gemm_tcgen05_kn");
  return 0;
}

// ================================================================================================
// The product for few rows (decoding with up to 64 requests) the other way round: the WEIGHTS are the
// 128-row operand of tcgen05.mma and the batch is its N = 16, 32 or 64, so a tile of 128 weight rows is
// streamed once through a ring of TMA stages while the tensor core multiplies it with all batch rows:
//
//     acc[128 weight rows, NB batch rows] += W[n0 .. n0+127, k .. k+63] . x[0 .. NB-1, k .. k+63]^T
//
// The k range of a tile is split over the blocks of a thread-block cluster when there are few tiles.
// Warp 0 (one thread) requests the weights of its first stages BEFORE it waits for the preceding kernel
// of the stream (they do not depend on it) and the batch rows after; warp 1 (one thread) issues the
// instructions; warps 2-5 take the accumulator out of tensor memory, thread = weight row.  Every block
// then puts its sums for a share of the tile's rows into the shared memory of the block that owns that
// share (distributed shared memory, stores only), one cluster barrier makes them visible, and the owner
// adds them in rank order and runs the epilogue for its rows, so the result does not depend on timing:
//   plain            out[m][n] (bfloat16 or float32), optionally divided by rms of residual row m
//   SiLU-mul         a tile holds 64 gate rows and the 64 up rows of the same outputs
//   residual add     residual[m][n] += product; sums of squares per row and block of 16 columns; bfloat16 copy
// These are the epilogues of gemm_small_m.cu, whose products this kernel takes over where the matrices
// are large or the rows more than 16.  Every mbarrier wait is bounded (code 4 producer, 5 issuer,
// 6 epilogue for ms_gemm_tc_status).
#include <cooperative_groups.h>

#include "launch.cuh"

namespace cg = cooperative_groups;

#define RT_BM 128
#define RT_BK 64
#define RT_THREADS 192
#define RT_W_BYTES (RT_BM * RT_BK * 2)
#define RT_MAX_STAGES 8
#define RT_MAX_CLUSTER 8

enum { RT_EPI_BF16 = 0, RT_EPI_F32 = 1, RT_EPI_SILU_MUL = 2, RT_EPI_RESADD = 3 };

struct RtExtra {
  const float* stats_in;  // row scaling: sums of squares [M][stats_in_nb] of the rows the activations were rounded from
  int stats_in_nb;
  float eps;
  int scale_k;            // the width of those rows (the mean of squares is over it)
  float* residual;        // residual epilogue: float32 [M][ldr], added into in place
  int ldr;
  float* stats_out;       // [M][ceil(N / 16)]
  __nv_bfloat16* copy_out;  // optional: the new residual rounded, [M][ldc]
  int ldc;
};

struct RtShared {
  unsigned long long full[RT_MAX_STAGES];
  unsigned long long empty[RT_MAX_STAGES];
  unsigned long long done;
  unsigned tmem_base;
  int abort_flag;
  float inv_rms[64];
};

__device__ __forceinline__ void rt_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared memory: [stages x (W tile 16 KB | x tile NB x 128 B)] [gather: RT_BM rows x (NB + 1) floats] [RtShared].
// The gathering buffer holds, for the rows this block owns, every cluster block's sums: [rank][row of the share][NB + 1].
template <int NB, int EPI, int SCALE>
__global__ void __launch_bounds__(RT_THREADS, 2)
gemm_rows_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                    const __grid_constant__ CUtensorMap map_x, void* __restrict__ out, int ldo, int M, int N, int K,
                    int cluster_size, int stages, RtExtra ex) {
  constexpr int X_BYTES = NB * RT_BK * 2;
  constexpr int STAGE_BYTES = RT_W_BYTES + X_BYTES;
  constexpr int GROW = NB + 4;  // floats per gathered row: 16-byte rows whose quarter-warps fall into different banks
  constexpr int TMEM_COLS = NB < 32 ? 32 : NB;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* gather = reinterpret_cast<float*>(tiles + (size_t)stages * STAGE_BYTES);  // (only with a cluster)
  RtShared* sh = reinterpret_cast<RtShared*>(gather + (cluster_size > 1 ? RT_BM * GROW : 0));
  volatile int* abort_flag = &sh->abort_flag;

  ms_pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / cluster_size, rank = blockIdx.x - tile * cluster_size;
  // the tile's weight rows: 128 consecutive ones, or 64 gate rows and the 64 up rows of the same outputs
  const int n0 = tile * (EPI == RT_EPI_SILU_MUL ? 64 : RT_BM);
  const int kt_count = (K + RT_BK - 1) / RT_BK;
  const int kt_per = (kt_count + cluster_size - 1) / cluster_size;
  const int kt0 = rank * kt_per;
  const int my_kt = max(0, min(kt_count, kt0 + kt_per) - kt0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc_mbar_init(tc_smem(&sh->full[s]), 1);
      tc_mbar_init(tc_smem(&sh->empty[s]), 1);
    }
    tc_mbar_init(tc_smem(&sh->done), 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(&sh->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = sh->tmem_base;

  if (warp == 0 && lane == 0) {
    // producer.  The weights of the first stages go out before the wait for the preceding kernel; the batch rows,
    // which it wrote, after.  A stage's barrier counts the bytes of both.
    const int first = my_kt < stages ? my_kt : stages;
    for (int kt = 0; kt < first; ++kt) {
      const unsigned dst = tc_smem(tiles + kt * STAGE_BYTES), bar = tc_smem(&sh->full[kt]);
      tc_mbar_expect_tx(bar, STAGE_BYTES);
      if (EPI == RT_EPI_SILU_MUL) {
        tc_tma_load_2d(dst, &map_w, (kt0 + kt) * RT_BK, n0, bar);
        tc_tma_load_2d(dst + 64 * RT_BK * 2, &map_w2, (kt0 + kt) * RT_BK, n0, bar);
      } else {
        tc_tma_load_2d(dst, &map_w, (kt0 + kt) * RT_BK, n0, bar);
        tc_tma_load_2d(dst + 64 * RT_BK * 2, &map_w, (kt0 + kt) * RT_BK, n0 + 64, bar);
      }
    }
    ms_pdl_wait();
    for (int kt = 0; kt < first; ++kt)
      tc_tma_load_2d(tc_smem(tiles + kt * STAGE_BYTES + RT_W_BYTES), &map_x, (kt0 + kt) * RT_BK, 0, tc_smem(&sh->full[kt]));
    for (int kt = first; kt < my_kt; ++kt) {
      const int s = kt % stages;
      if (!tc_mbar_wait(tc_smem(&sh->empty[s]), ((kt / stages) - 1) & 1, abort_flag, 4)) break;
      const unsigned dst = tc_smem(tiles + s * STAGE_BYTES), bar = tc_smem(&sh->full[s]);
      tc_mbar_expect_tx(bar, STAGE_BYTES);
      if (EPI == RT_EPI_SILU_MUL) {
        tc_tma_load_2d(dst, &map_w, (kt0 + kt) * RT_BK, n0, bar);
        tc_tma_load_2d(dst + 64 * RT_BK * 2, &map_w2, (kt0 + kt) * RT_BK, n0, bar);
      } else {
        tc_tma_load_2d(dst, &map_w, (kt0 + kt) * RT_BK, n0, bar);
        tc_tma_load_2d(dst + 64 * RT_BK * 2, &map_w, (kt0 + kt) * RT_BK, n0 + 64, bar);
      }
      tc_tma_load_2d(dst + RT_W_BYTES, &map_x, (kt0 + kt) * RT_BK, 0, bar);
    }
  } else if (warp == 1 && lane == 0) {
    // issuer: four K = 16 instructions per stage, then the stage goes back to the producer
    const unsigned idesc = tc_instr_desc(RT_BM, NB);
    bool ok = true;
    for (int kt = 0; kt < my_kt && ok; ++kt) {
      const int s = kt % stages;
      ok = tc_mbar_wait(tc_smem(&sh->full[s]), (kt / stages) & 1, abort_flag, 5);
      if (!ok) break;
      tc_fence_after();
      const unsigned a_src = tc_smem(tiles + s * STAGE_BYTES);
      const unsigned b_src = a_src + RT_W_BYTES;
#pragma unroll
      for (int k = 0; k < RT_BK / 16; ++k)
        tc_mma(tmem, tc_smem_desc(a_src + k * 32), tc_smem_desc(b_src + k * 32), idesc, (kt | k) != 0);
      tc_commit(tc_smem(&sh->empty[s]));
    }
    if (ok && my_kt > 0) tc_commit(tc_smem(&sh->done));
  } else if (warp >= 2) {
    // epilogue: the row scaling's 1 / rms first (it needs only what the preceding kernel left)
    ms_pdl_wait();
    const int et = threadIdx.x - 64;  // 0..127
    if (SCALE == 1) {
      if (et < NB) {
        float ss = 0.f;
        if (et < M)
          for (int b = 0; b < ex.stats_in_nb; ++b) ss += ex.stats_in[(size_t)et * ex.stats_in_nb + b];
        sh->inv_rms[et] = rsqrtf(ss / (float)ex.scale_k + ex.eps);
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
    }
    const bool have = my_kt == 0 || tc_mbar_wait(tc_smem(&sh->done), 0, abort_flag, 6);
    const int group = warp & 3;
    const int row = group * 32 + lane;  // the accumulator lane = weight row of the tile
    const unsigned row_addr = tmem + ((unsigned)(group * 32) << 16);
    if (have) tc_fence_after();
    if (cluster_size == 1) {
      // one block has the whole k range: straight from tensor memory to the output, 16 batch rows at a time; a warp's
      // lanes are 32 consecutive outputs of a batch row
      float* up_s = reinterpret_cast<float*>(tiles);  // gated form: the up rows' values for the gate rows' threads
      if (EPI == RT_EPI_SILU_MUL) {                    // (the stages are free: every product has been done)
        if (have && row >= 64) {
#pragma unroll
          for (int c = 0; c < NB; c += 16) {
            float v[16];
            rt_ld16(row_addr + c, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) up_s[(row - 64) * GROW + c + j] = v[j];
          }
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
      }
      const int n = n0 + (EPI == RT_EPI_SILU_MUL ? (row & 63) : row);
      if (have && !(EPI == RT_EPI_SILU_MUL && row >= 64)) {
#pragma unroll
        for (int c = 0; c < NB; c += 16) {
          float v[16];
          if (my_kt > 0) {
            rt_ld16(row_addr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c + j;
            const bool ok = m < M && n < N;
            const float rs = SCALE == 1 ? sh->inv_rms[m] : 1.f;
            if (EPI == RT_EPI_SILU_MUL) {
              const float gate = v[j] * rs, up = up_s[row * GROW + m] * rs;
              if (ok) reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
            } else if (EPI == RT_EPI_RESADD) {
              float r = 0.f;
              if (ok) {
                r = ex.residual[(size_t)m * ex.ldr + n] + v[j];
                ex.residual[(size_t)m * ex.ldr + n] = r;
                if (ex.copy_out) ex.copy_out[(size_t)m * ex.ldc + n] = __float2bfloat16_rn(r);
              }
              float ss = r * r;  // the sum of squares of 16 consecutive columns: 16 consecutive lanes
#pragma unroll
              for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off, 16);
              if ((lane & 15) == 0 && ok) ex.stats_out[(size_t)m * ((N + 15) / 16) + n / 16] = ss;
            } else if (ok) {
              if (EPI == RT_EPI_F32)
                reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = v[j] * rs;
              else
                reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v[j] * rs);
            }
          }
        }
      }
    } else if (have) {
      // the k range is split over a cluster: this block's sums go to the blocks that own the rows.  The rows are
      // shared out in runs: run `owner` belongs to the cluster's block `owner`.  The gated form pairs gate row i with
      // up row 64 + i, so both halves are cut alike.
      const int half = EPI == RT_EPI_SILU_MUL ? 64 : RT_BM;
      const int run = half / cluster_size;
      const int i = EPI == RT_EPI_SILU_MUL ? (row & 63) : row;
      const int owner = i / run;
      const int local = (i - owner * run) + ((EPI == RT_EPI_SILU_MUL && row >= 64) ? run : 0);
      cg::cluster_group cluster = cg::this_cluster();
      const int rows_owned = EPI == RT_EPI_SILU_MUL ? 2 * run : run;
      float* dst = cluster.map_shared_rank(gather, owner) + ((size_t)rank * rows_owned + local) * GROW;
#pragma unroll
      for (int c = 0; c < NB; c += 16) {
        float v[16];
        if (my_kt > 0) {
          rt_ld16(row_addr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(dst + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    }
  }
  tc_fence_before();
  if (cluster_size > 1) {
    cg::this_cluster().sync();
  } else {
    __syncthreads();
  }
  if (cluster_size > 1 && warp >= 2 && !*abort_flag) {
    // the rows this block owns, summed over the cluster's blocks in rank order
    const int et = threadIdx.x - 64;
    const int half = EPI == RT_EPI_SILU_MUL ? 64 : RT_BM;
    const int run = half / cluster_size;
    const int rows_owned = EPI == RT_EPI_SILU_MUL ? 2 * run : run;
    const int first = n0 + rank * run;  // the first output column (weight row) of this block's run
    for (int e = et; e < run * NB; e += 128) {
      const int m = e / run, i = e - m * run;  // consecutive threads: consecutive outputs of one batch row
      float a = 0.f, b = 0.f;
      for (int k = 0; k < cluster_size; ++k) {
        a += gather[((size_t)k * rows_owned + i) * GROW + m];
        if (EPI == RT_EPI_SILU_MUL) b += gather[((size_t)k * rows_owned + run + i) * GROW + m];
      }
      const int n = first + i;
      const bool ok = m < M && n < N;
      const float rs = SCALE == 1 ? sh->inv_rms[m] : 1.f;
      if (EPI == RT_EPI_SILU_MUL) {
        const float gate = a * rs, up = b * rs;
        if (ok) reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      } else if (EPI == RT_EPI_RESADD) {
        float v = 0.f;
        if (ok) {
          v = ex.residual[(size_t)m * ex.ldr + n] + a;
          ex.residual[(size_t)m * ex.ldr + n] = v;
          if (ex.copy_out) ex.copy_out[(size_t)m * ex.ldc + n] = __float2bfloat16_rn(v);
        }
        // the sum of squares of each 16 consecutive columns of a row: 16 consecutive lanes (a run is a multiple of 16)
        float ss = v * v;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off, 16);
        if ((lane & 15) == 0 && ok) ex.stats_out[(size_t)m * ((N + 15) / 16) + n / 16] = ss;
      } else if (ok) {
        if (EPI == RT_EPI_F32)
          reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = a * rs;
        else
          reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(a * rs);
      }
    }
  }
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------ host

struct RtPlan {
  int nb, cluster, stages;
  size_t smem;
};

// How a product is spread over the GPU: tiles of 128 weight rows (64 outputs of the gated form), the k range of a
// tile split over a cluster while that leaves every block at least two steps of 64 and all blocks resident at once
// (two blocks per SM), and as many stages as the block's share of an SM's shared memory holds.
static RtPlan rt_plan(int M, int tiles, int K, int sm_count) {
  RtPlan p;
  p.nb = M <= 16 ? 16 : M <= 32 ? 32 : 64;
  const int kt = (K + RT_BK - 1) / RT_BK;
  p.cluster = 1;
  while (p.cluster * 2 <= RT_MAX_CLUSTER && (long long)tiles * p.cluster * 2 <= 2LL * sm_count && kt / (p.cluster * 2) >= 2) p.cluster *= 2;
  const int per = (kt + p.cluster - 1) / p.cluster;
  const size_t stage = RT_W_BYTES + (size_t)p.nb * RT_BK * 2;
  const size_t fixed = (p.cluster > 1 ? (size_t)RT_BM * (p.nb + 4) * sizeof(float) : 0) + sizeof(RtShared) + 1024;
  const size_t budget = ((long long)tiles * p.cluster <= sm_count ? 200 : 104) * 1024;
  int stages = (int)((budget - fixed) / stage);
  if (stages > per) stages = per;
  if (stages > RT_MAX_STAGES) stages = RT_MAX_STAGES;
  if (stages < 1) stages = 1;
  p.stages = stages;
  p.smem = (size_t)stages * stage + fixed;
  return p;
}

template <int NB, int EPI, int SCALE>
static int rt_launch_nb(const CUtensorMap& mw, const CUtensorMap& mw2, const CUtensorMap& mx, void* out, int ldo, int M, int N,
                        int K, int tiles, const RtPlan& p, const RtExtra& ex, cudaStream_t stream) {
  auto kern = gemm_rows_tc_kernel<NB, EPI, SCALE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
    if (e != cudaSuccess) {
      ms_set_error("gemm_rows_tc: cannot configure shared memory: %s", cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  MS_LAUNCH_RESULT("gemm_rows_tc", ms_launch(kern, dim3(tiles * p.cluster), dim3(RT_THREADS), p.smem, stream, p.cluster, true, mw, mw2,
                                            mx, out, ldo, M, N, K, p.cluster, p.stages, ex));
  return 0;
}

template <int EPI, int SCALE>
static int rt_launch(const void* x, int ldx, const void* w, const void* w2, void* out, int ldo, int M, int N, int K,
                     const RtExtra& ex, int sm_count, cudaStream_t stream) {
  MS_REQUIRE(M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0, "gemm_rows_tc: M=%d (1..64), N=%d, K=%d (a multiple of 8) is not covered", M, N, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)w2 % 16 == 0),
             "gemm_rows_tc: operands must be 16-byte aligned with row strides that are multiples of 8");
  const int tiles = EPI == RT_EPI_SILU_MUL ? (N + 63) / 64 : (N + RT_BM - 1) / RT_BM;
  const RtPlan p = rt_plan(M, tiles, K, sm_count);
  CUtensorMap mw, mw2, mx;
  if (int rc = tc_make_map(&mw, w, N, K, K, 64)) return rc;
  if (int rc = tc_make_map(&mw2, w2 ? w2 : w, N, K, K, 64)) return rc;
  if (int rc = tc_make_map(&mx, x, M, K, ldx, p.nb)) return rc;
  if (p.nb == 16) return rt_launch_nb<16, EPI, SCALE>(mw, mw2, mx, out, ldo, M, N, K, tiles, p, ex, stream);
  if (p.nb == 32) return rt_launch_nb<32, EPI, SCALE>(mw, mw2, mx, out, ldo, M, N, K, tiles, p, ex, stream);
  return rt_launch_nb<64, EPI, SCALE>(mw, mw2, mx, out, ldo, M, N, K, tiles, p, ex, stream);
}

MS_API int ms_gemm_rows_tc_supports(int M, int N, int K) { return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0; }

// out[M, N] = x[M, K] . w[N, K]^T for M <= 64; out bfloat16 or float32.
MS_API int ms_gemm_rows_tc(const void* x, int ldx, const void* w, void* out, int out_dtype, int ldo, int M, int N, int K,
                           int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ldo >= N, "gemm_rows_tc: out row stride %d is shorter than N = %d", ldo, N);
  if (out_dtype == MS_F32) return rt_launch<RT_EPI_F32, 0>(x, ldx, w, nullptr, out, ldo, M, N, K, RtExtra{}, sm_count, stream);
  MS_REQUIRE(out_dtype == MS_BF16, "gemm_rows_tc: unknown out dtype %d", out_dtype);
  return rt_launch<RT_EPI_BF16, 0>(x, ldx, w, nullptr, out, ldo, M, N, K, RtExtra{}, sm_count, stream);
}

// out[M, I] = silu(x . w_gate^T) * (x . w_up^T); w_gate, w_up [I, K]; out bfloat16.
MS_API int ms_gemm_rows_tc_silu_mul(const void* x, int ldx, const void* w_gate, const void* w_up, void* out, int ldo, int M,
                                    int I, int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ldo >= I && w_up != nullptr, "gemm_rows_tc_silu_mul: bad arguments");
  return rt_launch<RT_EPI_SILU_MUL, 0>(x, ldx, w_gate, w_up, out, ldo, M, I, K, RtExtra{}, sm_count, stream);
}

// out = (x . w^T) / rms(row), or silu(. / rms) * (. / rms) with w_up: x is the residual rounded to bfloat16 [M, K],
// stats_in [M][stats_nb] the sums of squares of its rows (see ms_gemm_rows_tc_resadd).  out bfloat16.
MS_API int ms_gemm_rows_tc_scaled(const void* x, int ldx, const float* stats_in, int stats_nb, float eps, const void* w,
                                  const void* w_up, void* out, int ldo, int M, int N, int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ldo >= N && stats_in != nullptr && stats_nb >= 1, "gemm_rows_tc_scaled: bad arguments");
  RtExtra ex = {};
  ex.stats_in = stats_in;
  ex.stats_in_nb = stats_nb;
  ex.eps = eps;
  ex.scale_k = K;
  if (w_up) return rt_launch<RT_EPI_SILU_MUL, 1>(x, ldx, w, w_up, out, ldo, M, N, K, ex, sm_count, stream);
  return rt_launch<RT_EPI_BF16, 1>(x, ldx, w, nullptr, out, ldo, M, N, K, ex, sm_count, stream);
}

// residual[M, N] += x[M, K] . w[N, K]^T in place (float32); stats_out[m][b] = the sum of squares of the new residual's
// row m over columns [16 b, 16 b + 16); copy_out (optional, bfloat16 [M][ldc]) = the new residual rounded.
MS_API int ms_gemm_rows_tc_resadd(const void* x, int ldx, const void* w, float* residual, int ldr, float* stats_out,
                                  void* copy_out, int ldc, int M, int N, int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(residual != nullptr && stats_out != nullptr && ldr >= N && (copy_out == nullptr || ldc >= N), "gemm_rows_tc_resadd: bad arguments");
  RtExtra ex = {};
  ex.residual = residual;
  ex.ldr = ldr;
  ex.stats_out = stats_out;
  ex.copy_out = (__nv_bfloat16*)copy_out;
  ex.ldc = ldc;
  return rt_launch<RT_EPI_RESADD, 0>(x, ldx, w, nullptr, nullptr, 0, M, N, K, ex, sm_count, stream);
}

// ------------------------------------------------------------------------------------------------
// The product for many rows with PAIRS of SMs on one tile (tcgen05 cta_group::2): a cluster of two resident blocks
// goes through its tiles of the output one after the other.  A tile is 256 rows x BN columns (256, or 128 when that
// leaves too few tiles); each block of the pair holds its own 128 rows of the activations and HALF of the tile's
// weight rows in its shared memory, block 0 issues the instructions for both, and each block's tensor memory
// receives the accumulators of its own 128 rows.  A block alone cannot feed the tensor core from its shared memory
// (operand reads and TMA writes of a 128 x 256 tile add up to 192 bytes a cycle against the 128 it has); with the
// weights split over the pair they fit.  K goes in steps of 64 through a ring of stages that runs on across tiles,
// and there are TWO accumulators in tensor memory, so that the epilogue warps drain tile i while the tensor core
// works on tile i + 1.  Tiles that share weight rows are neighbours in the order.
// Both blocks copy with TMA into their own shared memory and count the bytes on block 0's barrier (no load uses
// cluster multicast); block 0's commits reach both blocks' barriers; the epilogue threads of both blocks arrive on
// block 0's barrier when they have drained an accumulator.  Every wait is bounded as above.
// Epilogues as in the few-row kernels (gemm_small_m.cu), so that a pre-norm block needs no kernel between its
// products:
//   plain      out = acc (bfloat16)
//   SCALE      every output row times 1 / rms of the row the activations were rounded from, made from the
//              sums of squares that RESADD left: the RMS norm for a matrix with the norm's weight folded in
//   SILU_MUL   block 0 holds BN/2 gate rows, block 1 the BN/2 up rows of the same outputs; out = silu(gate) * up
//   RESADD     residual (float32) += acc in place; a bfloat16 copy of the new residual; its sums of squares
//              per row and half tile of columns (a consumer adds up all of a row's sums, however many there are)
#define PR_BK 64
#define PR_THREADS 320  // a copying warp, an issuing warp, eight epilogue warps
#define PR_MAX_STAGES 8
// where a warp's 32 rows x 32 columns change hands in the epilogue: rows of 144 bytes (float32) or of 80 (bfloat16)
#define PR_EXCHANGE_BYTES(EPI) ((EPI) == PR_EPI_RESADD ? 32 * 144 : 32 * 80)
// stages of the ring: what the exchange leaves of the shared memory
#define PR_STAGES(BN, EPI) ((BN) == 256 ? ((EPI) == PR_EPI_RESADD ? 5 : 6) : ((EPI) == PR_EPI_RESADD ? 7 : 8))
#define PR_PEER_MASK 0xFEFFFFFFu  // a shared::cluster address with this bit cleared is block 0's copy of the same place
enum { PR_EPI_BF16 = 0, PR_EPI_SILU_MUL = 1, PR_EPI_RESADD = 2 };

struct PrExtra {
  const float* stats_in;  // SCALE: [M][stats_in_nb] sums of squares of the rows the activations were rounded from
  int stats_in_nb;
  float eps;
  int up_offset;          // SILU_MUL: rows between a gate row and its up row in the weight matrix
  float* residual;        // RESADD: float32 [M][ldr], added into in place
  int ldr;
  float* stats_out;       // RESADD: [M][stats_out_nb]
  int stats_out_nb;
  __nv_bfloat16* copy_out;  // RESADD, optional: [M][ldc]
  int ldc;
};

struct PrShared {
  unsigned long long full[PR_MAX_STAGES], empty[PR_MAX_STAGES], acc_full[2], acc_empty[2];
  unsigned tmem_base;
  int abort_flag;
};

__device__ __forceinline__ unsigned pr_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void pr_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A copy into this block's shared memory whose bytes are counted on block 0's barrier at the same place.
__device__ __forceinline__ void pr_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar & PR_PEER_MASK)
      : "memory");
}
__device__ __forceinline__ void pr_mma(unsigned tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
  const unsigned z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// When the instructions issued so far are done, one arrival on the barrier at this place in both blocks of the pair.
__device__ __forceinline__ void pr_commit_both(unsigned bar) {
  const unsigned short both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(bar),
               "h"(both)
               : "memory");
}
// 32 floats of a row, with 16-byte loads where the row allows it; what lies past `valid` reads as zero.
__device__ __forceinline__ void pr_load32(float (&dst)[32], const float* src, int valid) {
  if (valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 r = *reinterpret_cast<const float4*>(src + i);
      dst[i] = r.x; dst[i + 1] = r.y; dst[i + 2] = r.z; dst[i + 3] = r.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) dst[i] = i < valid ? src[i] : 0.f;
  }
}
__device__ __forceinline__ void pr_arrive_block0(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(bar & PR_PEER_MASK) : "memory");
}

template <int BN, int EPI, int SCALE>
__global__ void __launch_bounds__(PR_THREADS, 1)
gemm_pair_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    __nv_bfloat16* __restrict__ out, int ldo, int M, int N, int K, int tiles_m, int num_tiles, PrExtra ex) {
  constexpr int HALF = BN / 2;                          // weight rows a block holds of a tile
  constexpr int STAGE_BYTES = (128 + HALF) * PR_BK * 2;  // per block
  constexpr int STAGES = PR_STAGES(BN, EPI);
  constexpr int OUT_COLS = EPI == PR_EPI_SILU_MUL ? HALF : BN;  // output columns of a tile
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  PrShared* sh = reinterpret_cast<PrShared*>(tiles + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)pr_cluster_rank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int kt_count = (K + PR_BK - 1) / PR_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc_mbar_init(tc_smem(&sh->full[s]), 1);   // block 0's: its own announcement of the bytes; both blocks' copies count on it
      tc_mbar_init(tc_smem(&sh->empty[s]), 1);  // each block's own: block 0's commit arrives on both
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(tc_smem(&sh->acc_full[b]), 1);     // each block's own
      tc_mbar_init(tc_smem(&sh->acc_empty[b]), 512);  // block 0's: the epilogue threads of both blocks
    }
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {  // the same warp of both blocks: the accumulators of a pair lie at the same columns
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc_smem(&sh->tmem_base)),
                 "r"(2 * BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  pr_cluster_sync();  // the other block's barriers exist before anything arrives on them
  tc_fence_after();
  const unsigned tmem = sh->tmem_base;

  if (warp == 0 && lane == 0) {
    // producer (both blocks): the ring of stages runs on from tile to tile
    int it = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int mt = tile % tiles_m, nt = tile / tiles_m;
      const int m0 = mt * 256 + rank * 128;
      const int w0 = EPI == PR_EPI_SILU_MUL ? nt * HALF + rank * ex.up_offset : nt * BN + rank * HALF;
      for (int kt = 0; kt < kt_count; ++kt, ++it) {
        const int s = it % STAGES;
        if (it >= STAGES && !tc_mbar_wait(tc_smem(&sh->empty[s]), ((it / STAGES) - 1) & 1, abort_flag, 21)) {
          ok = false;
          break;
        }
        const unsigned a_dst = tc_smem(tiles + s * STAGE_BYTES);
        const unsigned b_dst = a_dst + 128 * PR_BK * 2;
        const unsigned bar = tc_smem(&sh->full[s]);
        if (rank == 0) tc_mbar_expect_tx(bar, 2 * STAGE_BYTES);
        pr_tma_load_2d(a_dst, &map_x, kt * PR_BK, m0, bar);
        pr_tma_load_2d(b_dst, &map_w, kt * PR_BK, w0, bar);
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // issuer (block 0): four K = 16 instructions of 256 x BN per stage, into the accumulator both epilogues have drained
    const unsigned idesc = tc_instr_desc(256, BN);
    int it = 0, count = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++count) {
      const int buf = count & 1;
      if (count >= 2) {
        ok = tc_mbar_wait(tc_smem(&sh->acc_empty[buf]), ((count >> 1) - 1) & 1, abort_flag, 22);
        if (!ok) break;
        tc_fence_after();
      }
      const unsigned acc = tmem + buf * BN;
      for (int kt = 0; kt < kt_count; ++kt, ++it) {
        const int s = it % STAGES;
        ok = tc_mbar_wait(tc_smem(&sh->full[s]), (it / STAGES) & 1, abort_flag, 22);
        if (!ok) break;
        tc_fence_after();
        const unsigned a_src = tc_smem(tiles + s * STAGE_BYTES);
        const unsigned b_src = a_src + 128 * PR_BK * 2;
#pragma unroll
        for (int k = 0; k < PR_BK / 16; ++k)
          pr_mma(acc, tc_smem_desc(a_src + k * 32), tc_smem_desc(b_src + k * 32), idesc, (kt | k) != 0);
        pr_commit_both(tc_smem(&sh->empty[s]));
      }
      if (ok) pr_commit_both(tc_smem(&sh->acc_full[buf]));
    }
  } else if (warp >= 2) {
    // epilogue (both blocks).  A warp may touch the 32 lanes of tensor memory that its number allows: it takes 32 rows
    // of the block's half of the tile, 32 columns at a time, a row per thread; the values then change hands through
    // the warp's piece of shared memory so that a thread holds consecutive columns of few rows and global memory is
    // read and written in whole rows of the chunk (a row per thread would cost a transaction per thread and access).
    // Eight warps: two for each group of 32 rows, one for the left half of the tile's columns and one for the right.
    const int group = warp & 3;
    const int c_begin = warp >= 6 ? OUT_COLS / 2 : 0, c_end = c_begin + OUT_COLS / 2;
    unsigned char* stage = reinterpret_cast<unsigned char*>(sh) + 1024 + (warp - 2) * PR_EXCHANGE_BYTES(EPI);
    int count = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++count) {
      const int mt = tile % tiles_m, nt = tile / tiles_m;
      const int m_warp = mt * 256 + rank * 128 + group * 32;  // the warp's first row
      const int m = m_warp + lane, n0 = nt * OUT_COLS;
      float inv = 1.f;
      if (SCALE && m < M) {  // while the tensor core still works on the tile; eight loads in flight at a time
        const float* st = ex.stats_in + (size_t)m * ex.stats_in_nb;
        float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int b = 0; b < ex.stats_in_nb; b += 8) {
#pragma unroll
          for (int i = 0; i < 8; ++i) part[i] += b + i < ex.stats_in_nb ? st[b + i] : 0.f;
        }
        inv = rsqrtf((((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]))) / (float)K + ex.eps);
      }
      // RESADD, after the exchange: thread = (row 4 i + lane / 8, columns 4 (lane % 8) .. + 3) for i = 0 .. 7
      const int rr = lane >> 3, rq = lane & 7;
      float4 rold[8];  // the old residual of the chunk to come, requested a chunk ahead
      float ss[8];     // sums of squares of the new residual, per row of this thread, over the tile
      if (EPI == PR_EPI_RESADD) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ss[i] = 0.f;
          const int row = m_warp + 4 * i + rr, col = n0 + c_begin + 4 * rq;
          rold[i] = (row < M && col < N) ? *reinterpret_cast<const float4*>(ex.residual + (size_t)row * ex.ldr + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      const int buf = count & 1;
      ok = tc_mbar_wait(tc_smem(&sh->acc_full[buf]), (count >> 1) & 1, abort_flag, 23);
      if (!ok) break;
      tc_fence_after();
      const unsigned row_addr = tmem + buf * BN + ((unsigned)(group * 32) << 16);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 32) {
        float v[32];
        tc_ld32(row_addr + c, v);
        if (EPI == PR_EPI_SILU_MUL) {
          float u[32];
          tc_ld32(row_addr + OUT_COLS + c, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float gate = v[i] * inv;
            v[i] = gate * __frcp_rn(1.f + __expf(-gate)) * (u[i] * inv);  // (a reciprocal of infinity is zero: no NaN far left)
          }
        } else if (SCALE) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= inv;
        }
        const int n = n0 + c;
        if (EPI == PR_EPI_RESADD) {
          // float32 through the exchange: rows of 144 bytes (16-byte accesses of a quarter warp fall into different banks)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(stage + lane * 144 + 16 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = m_warp + 4 * i + rr, col = n + 4 * rq;
            const float4 acc = *reinterpret_cast<const float4*>(stage + (4 * i + rr) * 144 + 16 * rq);
            const float4 old = rold[i];
            if (c + 32 < c_end)
              rold[i] = (row < M && col + 32 < N) ? *reinterpret_cast<const float4*>(ex.residual + (size_t)row * ex.ldr + col + 32)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < M && col < N) {
              const float4 nw = make_float4(old.x + acc.x, old.y + acc.y, old.z + acc.z, old.w + acc.w);
              *reinterpret_cast<float4*>(ex.residual + (size_t)row * ex.ldr + col) = nw;
              if (ex.copy_out) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(nw.x, nw.y), hi = __floats2bfloat162_rn(nw.z, nw.w);
                *reinterpret_cast<uint2*>(ex.copy_out + (size_t)row * ex.ldc + col) =
                    make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
              }
              ss[i] += (nw.x * nw.x + nw.y * nw.y) + (nw.z * nw.z + nw.w * nw.w);
            }
          }
          __syncwarp();
        } else {
          // bfloat16 through the exchange: rows of 80 bytes
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 pk;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
            *reinterpret_cast<uint4*>(stage + lane * 80 + 16 * j) = pk;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = m_warp + 8 * i + (lane >> 2), col = n + 8 * (lane & 3);
            const uint4 pk = *reinterpret_cast<const uint4*>(stage + (8 * i + (lane >> 2)) * 80 + 16 * (lane & 3));
            if (row < M && col < N) *reinterpret_cast<uint4*>(out + (size_t)row * ldo + col) = pk;
          }
          __syncwarp();
        }
      }
      if (EPI == PR_EPI_RESADD) {
        // a row's eight threads add up their sums (in a fixed order) and one of them writes the row's sum for this tile
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float t = ss[i];
          t += __shfl_xor_sync(0xffffffffu, t, 1);
          t += __shfl_xor_sync(0xffffffffu, t, 2);
          t += __shfl_xor_sync(0xffffffffu, t, 4);
          const int row = m_warp + 4 * i + rr;
          if (rq == 0 && row < M) ex.stats_out[(size_t)row * ex.stats_out_nb + 2 * nt + (warp >= 6 ? 1 : 0)] = t;
        }
      }
      tc_fence_before();
      pr_arrive_block0(tc_smem(&sh->acc_empty[buf]));
    }
  }
  // leave together: neither block's shared memory, barriers or tensor memory may go while the other still uses them
  tc_fence_before();
  __syncthreads();
  pr_cluster_sync();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * BN) : "memory");
  }
}

template <int BN, int EPI, int SCALE>
static int pr_launch(const CUtensorMap& mx, const CUtensorMap& mw, void* out, int ldo, int M, int N, int K, const PrExtra& ex,
                     int sm_count, cudaStream_t stream) {
  constexpr int STAGES = PR_STAGES(BN, EPI);
  const size_t smem = (size_t)STAGES * (128 + BN / 2) * PR_BK * 2 + 1024 + 8 * PR_EXCHANGE_BYTES(EPI) + 1024;
  auto kern = gemm_pair_tc_kernel<BN, EPI, SCALE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      ms_set_error("gemm_pair_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return 2;
    }
    configured = true;
  }
  constexpr int OUT_COLS = EPI == PR_EPI_SILU_MUL ? BN / 2 : BN;
  const int tiles_m = (M + 255) / 256, tiles_n = (N + OUT_COLS - 1) / OUT_COLS;
  const int num_tiles = tiles_m * tiles_n;
  const int pairs = num_tiles < sm_count / 2 ? num_tiles : sm_count / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(PR_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MS_LAUNCH_RESULT("gemm_pair_tc", cudaLaunchKernelEx(&cfg, kern, mx, mw, (__nv_bfloat16*)out, ldo, M, N, K, tiles_m, num_tiles, ex));
  return 0;
}

// Tiles of 256 or of 128 columns: by the rounds the pairs of SMs need for all tiles, times what a step of K costs with
// that width (the tensor core is fed fully only by the wide tiles: a narrow one costs 0.72 of a wide one, not half).
static bool pr_wide(int M, int N, int sm_count) {
  const long long tm = (M + 255) / 256, pairs = sm_count / 2;
  const long long wide = (tm * ((N + 255) / 256) + pairs - 1) / pairs, narrow = (tm * ((N + 127) / 128) + pairs - 1) / pairs;
  return wide * 100 <= narrow * 72;
}

static int pr_maps(CUtensorMap* mx, CUtensorMap* mw, const void* x, int ldx, const void* w, int M, int w_rows, int K, int w_box) {
  MS_REQUIRE(M >= 1 && w_rows >= 8 && w_rows % 8 == 0 && K >= 8 && K % 8 == 0,
             "gemm_pair_tc: M=%d N=%d K=%d (N and K multiples of 8) is not covered", M, w_rows, K);
  MS_REQUIRE(ldx % 8 == 0 && ldx >= K && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0),
             "gemm_pair_tc: operands must be 16-byte aligned with row strides that are multiples of 8");
  if (int rc = tc_make_map(mx, x, M, K, ldx, 128)) return rc;
  return tc_make_map(mw, w, w_rows, K, K, w_box);
}

// out[M, N] = x[M, K] . w[N, K]^T, all bfloat16.  stats_in (or null): [M][stats_nb] sums of squares of the rows that
// x was rounded from; every output row is then divided by that row's rms (K values, eps inside the root).
MS_API int ms_gemm_pair_tc(const void* x, int ldx, const void* w, void* out, int ldo, int M, int N, int K,
                           const float* stats_in, int stats_nb, float eps, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ldo >= N && ldo % 8 == 0 && (uintptr_t)out % 16 == 0 && sm_count >= 2 && (stats_in == nullptr || stats_nb >= 1),
             "gemm_pair_tc: bad sizes ldo=%d (a multiple of 8, rows 16-byte aligned)", ldo);
  const bool wide = pr_wide(M, N, sm_count);
  CUtensorMap mx, mw;
  if (int rc = pr_maps(&mx, &mw, x, ldx, w, M, N, K, wide ? 128 : 64)) return rc;
  PrExtra ex = {stats_in, stats_nb, eps, 0, nullptr, 0, nullptr, 0, nullptr, 0};
  if (stats_in)
    return wide ? pr_launch<256, PR_EPI_BF16, 1>(mx, mw, out, ldo, M, N, K, ex, sm_count, stream)
                : pr_launch<128, PR_EPI_BF16, 1>(mx, mw, out, ldo, M, N, K, ex, sm_count, stream);
  return wide ? pr_launch<256, PR_EPI_BF16, 0>(mx, mw, out, ldo, M, N, K, ex, sm_count, stream)
              : pr_launch<128, PR_EPI_BF16, 0>(mx, mw, out, ldo, M, N, K, ex, sm_count, stream);
}

// out[M, I] = silu(x . w[0:I]^T) * (x . w[I:2I]^T); w is [2I, K] with the gate rows first; row scaling as above.
MS_API int ms_gemm_pair_tc_silu_mul(const void* x, int ldx, const void* w_gate_up, void* out, int ldo, int M, int I, int K,
                                    const float* stats_in, int stats_nb, float eps, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(ldo >= I && ldo % 8 == 0 && I % 8 == 0 && (uintptr_t)out % 16 == 0 && sm_count >= 2 && (stats_in == nullptr || stats_nb >= 1),
             "gemm_pair_tc_silu_mul: bad sizes I=%d ldo=%d (multiples of 8, rows 16-byte aligned)", I, ldo);
  CUtensorMap mx, mw;
  if (int rc = pr_maps(&mx, &mw, x, ldx, w_gate_up, M, 2 * I, K, 128)) return rc;
  PrExtra ex = {stats_in, stats_nb, eps, I, nullptr, 0, nullptr, 0, nullptr, 0};
  if (stats_in) return pr_launch<256, PR_EPI_SILU_MUL, 1>(mx, mw, out, ldo, M, I, K, ex, sm_count, stream);
  return pr_launch<256, PR_EPI_SILU_MUL, 0>(mx, mw, out, ldo, M, I, K, ex, sm_count, stream);
}

// How many sums of squares a row of ms_gemm_pair_tc_resadd's stats_out has (two per tile of columns: one per epilogue warp).
MS_API int ms_gemm_pair_tc_stats_blocks(int M, int N, int sm_count) { return 2 * (pr_wide(M, N, sm_count) ? (N + 255) / 256 : (N + 127) / 128); }

// residual[M, N] (float32) += x[M, K] . w[N, K]^T in place; stats_out[m][b] = the sum of squares of the new
// residual's row m over its b-th tile of columns (ms_gemm_pair_tc_stats_blocks of them a row); copy_out (or null):
// the new residual rounded to bfloat16.
MS_API int ms_gemm_pair_tc_resadd(const void* x, int ldx, const void* w, float* residual, int ldr, float* stats_out,
                                  void* copy_out, int ldc, int M, int N, int K, int sm_count, cudaStream_t stream) {
  if (M == 0) return 0;
  MS_REQUIRE(residual != nullptr && stats_out != nullptr && ldr >= N && ldr % 4 == 0 && (uintptr_t)residual % 16 == 0 && sm_count >= 2 &&
                 (copy_out == nullptr || (ldc >= N && ldc % 4 == 0 && (uintptr_t)copy_out % 8 == 0)),
             "gemm_pair_tc_resadd: bad sizes ldr=%d ldc=%d (multiples of 4, aligned rows)", ldr, ldc);
  const bool wide = pr_wide(M, N, sm_count);
  CUtensorMap mx, mw;
  if (int rc = pr_maps(&mx, &mw, x, ldx, w, M, N, K, wide ? 128 : 64)) return rc;
  PrExtra ex = {nullptr, 0, 0.f, 0, residual, ldr, stats_out, ms_gemm_pair_tc_stats_blocks(M, N, sm_count), (__nv_bfloat16*)copy_out, ldc};
  return wide ? pr_launch<256, PR_EPI_RESADD, 0>(mx, mw, nullptr, 0, M, N, K, ex, sm_count, stream)
              : pr_launch<128, PR_EPI_RESADD, 0>(mx, mw, nullptr, 0, M, N, K, ex, sm_count, stream);
}
