// Bias add, rotary position encoding of q and k, and the write of k and v into
// the paged cache, in one kernel.
//
// Counterparts in gqf2008/machserve (crates/mach-model/src/kernels.rs): add_bias
// :151-160, rope_batched :589-660, kv_store_paged :1148-1168.  The reference
// computes powf/cosf/sinf per element in float32; here the angles come from a
// table of (cos, sin) built on the host in float64 and rounded once, indexed by
// absolute position.  All arithmetic is float32; the bias is added before the
// rotation (crates/mach-model/src/batched.rs:3622-3678).
//
// Cache layout: pages[page][kv_head][slot in page][head_dim].
#include "launch.cuh"

template <typename TA, typename TC>
__global__ void rope_kv_store_kernel(const TA* __restrict__ qkv, int ld, const float* __restrict__ bias,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int max_pages, int num_pages,
                                     const float2* __restrict__ cos_sin, int rot, int interleaved,
                                     TA* __restrict__ q_out, TC* __restrict__ k_pages, TC* __restrict__ v_pages,
                                     int hq, int hkv, int hd, int page_size) {
  ms_pdl_trigger();
  ms_pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  if (seq < 0) return;  // padding row
  const int pos = positions[t];
  const TA* row = qkv + (size_t)t * ld;
  const int half = hd / 2, rhalf = rot / 2;
  const int qw = hq * hd, kw = hkv * hd;

  size_t cache_base = 0;
  bool store = hkv > 0;
  if (store) {
    const int page = block_table[(size_t)seq * max_pages + pos / page_size];
    store = page >= 0 && page < num_pages;
    cache_base = (size_t)(store ? page : 0) * hkv * page_size * hd + (size_t)(pos % page_size) * hd;
  }
  const float2* cs = cos_sin + (size_t)pos * rhalf;

  // q and k: one pair of coordinates per iteration
  const int npairs = (hq + hkv) * half;
  for (int e = threadIdx.x; e < npairs; e += blockDim.x) {
    const int head = e / half, j = e - head * half;
    int d0, d1;
    const bool rotate = j < rhalf;
    if (rotate) {
      d0 = interleaved ? 2 * j : j;
      d1 = interleaved ? 2 * j + 1 : j + rhalf;
    } else {  // coordinates past the rotary part pass through
      d0 = interleaved ? 2 * j : rot + 2 * (j - rhalf);
      d1 = d0 + 1;
    }
    const int col0 = head * hd + d0, col1 = head * hd + d1;  // columns within [q | k]
    float a = ms_to_float(row[col0]), b = ms_to_float(row[col1]);
    if (bias) {
      a += bias[col0];
      b += bias[col1];
    }
    float ra = a, rb = b;
    if (rotate) {
      const float2 c = cs[j];
      ra = a * c.x - b * c.y;
      rb = a * c.y + b * c.x;
    }
    if (head < hq) {
      q_out[(size_t)t * qw + col0] = ms_from_float<TA>(ra);
      q_out[(size_t)t * qw + col1] = ms_from_float<TA>(rb);
    } else if (store) {
      const int kvh = head - hq;
      TC* dst = k_pages + cache_base + (size_t)kvh * page_size * hd;
      dst[d0] = ms_from_float<TC>(ra);
      dst[d1] = ms_from_float<TC>(rb);
    }
  }
  // v: bias and copy
  if (store) {
    for (int e = threadIdx.x; e < kw; e += blockDim.x) {
      const int kvh = e / hd, dd = e - kvh * hd;
      float v = ms_to_float(row[qw + kw + e]);
      if (bias) v += bias[qw + kw + e];
      v_pages[cache_base + (size_t)kvh * page_size * hd + dd] = ms_from_float<TC>(v);
    }
  }
}

// The common case, bfloat16 everywhere, full rotary with half pairing, head_dim a multiple of 16: a thread
// takes 8 consecutive pairs (j .. j+7, j+half .. j+7+half) of one head, or 8 values of v, with 16-byte
// accesses.  Same arithmetic as above.
__global__ void rope_kv_store_vec_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, const float* __restrict__ bias,
                                         const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int max_pages, int num_pages,
                                         const float2* __restrict__ cos_sin, __nv_bfloat16* __restrict__ q_out,
                                         __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, int hq,
                                         int hkv, int hd, int page_size) {
  ms_pdl_trigger();
  const int t = blockIdx.x;
  const int half = hd / 2, per_head = half / 8;
  const int qw = hq * hd, kw = hkv * hd;
  const int rot_items = (hq + hkv) * per_head, v_items = kw / 8;
  // what does not depend on the kernel before: the row's sequence and position, its page, its angles
  const int seq = seq_of_token[t];
  const int pos = positions[t];
  size_t cache_base = 0;
  bool store = hkv > 0 && seq >= 0;
  if (store) {
    const int page = block_table[(size_t)seq * max_pages + pos / page_size];
    store = page >= 0 && page < num_pages;
    cache_base = (size_t)(store ? page : 0) * hkv * page_size * hd + (size_t)(pos % page_size) * hd;
  }
  ms_pdl_wait();
  if (seq < 0) return;  // padding row
  const __nv_bfloat16* row = qkv + (size_t)t * ld;
  const float2* cs = cos_sin + (size_t)pos * half;
  for (int e = threadIdx.x; e < rot_items + v_items; e += blockDim.x) {
    if (e < rot_items) {
      const int head = e / per_head, j = (e - head * per_head) * 8;
      const int col = head * hd + j;
      // all loads of the item first (two of the row, four of the angles, four of the bias), then the arithmetic
      const uint4 ua = *reinterpret_cast<const uint4*>(row + col), ub = *reinterpret_cast<const uint4*>(row + col + half);
      float4 c[4], ba[2], bb[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = *reinterpret_cast<const float4*>(cs + j + 2 * i);  // (cos, sin) of two pairs
      if (bias) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          ba[i] = *reinterpret_cast<const float4*>(bias + col + 4 * i);
          bb[i] = *reinterpret_cast<const float4*>(bias + col + half + 4 * i);
        }
      } else {
        ba[0] = ba[1] = bb[0] = bb[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      const float* fa = reinterpret_cast<const float*>(ba);
      const float* fb = reinterpret_cast<const float*>(bb);
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ua);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&ub);
      uint4 oa, ob;
      __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&oa);
      __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(ha[i]), b = __bfloat1622float2(hb[i]);
        a.x += fa[2 * i];
        a.y += fa[2 * i + 1];
        b.x += fb[2 * i];
        b.y += fb[2 * i + 1];
        const float2 c0 = make_float2(c[i].x, c[i].y), c1 = make_float2(c[i].z, c[i].w);
        pa[i] = __floats2bfloat162_rn(a.x * c0.x - b.x * c0.y, a.y * c1.x - b.y * c1.y);
        pb[i] = __floats2bfloat162_rn(a.x * c0.y + b.x * c0.x, a.y * c1.y + b.y * c1.x);
      }
      if (head < hq) {
        *reinterpret_cast<uint4*>(q_out + (size_t)t * qw + col) = oa;
        *reinterpret_cast<uint4*>(q_out + (size_t)t * qw + col + half) = ob;
      } else if (store) {
        __nv_bfloat16* dst = k_pages + cache_base + (size_t)(head - hq) * page_size * hd + j;
        *reinterpret_cast<uint4*>(dst) = oa;
        *reinterpret_cast<uint4*>(dst + half) = ob;
      }
    } else if (store) {
      const int c = (e - rot_items) * 8;
      const int kvh = c / hd, dd = c - kvh * hd;
      const uint4 u = *reinterpret_cast<const uint4*>(row + qw + kw + c);
      float4 bv[2];
      if (bias) {
        bv[0] = *reinterpret_cast<const float4*>(bias + qw + kw + c);
        bv[1] = *reinterpret_cast<const float4*>(bias + qw + kw + c + 4);
      } else {
        bv[0] = bv[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      const float* fv = reinterpret_cast<const float*>(bv);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      uint4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        po[i] = __floats2bfloat162_rn(f.x + fv[2 * i], f.y + fv[2 * i + 1]);
      }
      *reinterpret_cast<uint4*>(v_pages + cache_base + (size_t)kvh * page_size * hd + dd) = o;
    }
  }
}

// qkv: [tokens, ld] with q in columns [0, hq*hd), k in the next hkv*hd, v in the next hkv*hd.
// hkv == 0: only q is encoded and nothing is stored (a layer that reads another layer's cache).
// rot == 0: no rotation (bias and store only).  cos_sin: [table_len, rot/2] pairs.
MS_API int ms_rope_kv_store(const void* qkv, int act_dtype, int ld, const float* bias, const int* positions,
                            const int* seq_of_token, const int* block_table, int max_pages, int num_pages,
                            const float* cos_sin, int rot, int interleaved, void* q_out, void* k_pages,
                            void* v_pages, int cache_dtype, int tokens, int hq, int hkv, int hd, int page_size,
                            cudaStream_t stream) {
  if (tokens == 0) return 0;
  MS_REQUIRE(tokens > 0 && hq > 0 && hkv >= 0 && hd > 0 && hd % 2 == 0, "rope_kv_store: bad sizes tokens=%d hq=%d hkv=%d hd=%d",
             tokens, hq, hkv, hd);
  MS_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "rope_kv_store: rotary size %d must be even and at most head_dim %d", rot, hd);
  MS_REQUIRE(ld >= (hq + 2 * hkv) * hd, "rope_kv_store: row stride %d is shorter than q|k|v = %d", ld, (hq + 2 * hkv) * hd);
  MS_REQUIRE(hkv == 0 || (page_size > 0 && max_pages > 0 && num_pages > 0), "rope_kv_store: bad cache sizes");
  MS_REQUIRE(rot == 0 || cos_sin != nullptr, "rope_kv_store: rotation without a table");
  if (act_dtype == MS_BF16 && cache_dtype == MS_BF16 && rot == hd && !interleaved && hd % 16 == 0 && ld % 8 == 0 &&
      ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)bias | (uintptr_t)cos_sin) % 16 == 0) {
    int items = (hq + hkv) * (hd / 16) + hkv * hd / 8;
    int vthreads = (items + 31) / 32 * 32;
    vthreads = vthreads > 256 ? 256 : vthreads;
    MS_LAUNCH_RESULT("rope_kv_store",
                     ms_launch(rope_kv_store_vec_kernel, dim3(tokens), dim3(vthreads), 0, stream, 1, true,
                               (const __nv_bfloat16*)qkv, ld, bias, positions, seq_of_token, block_table, max_pages, num_pages,
                               (const float2*)cos_sin, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
                               hq, hkv, hd, page_size));
    return 0;
  }
  int threads = ((hq + hkv) * hd / 2 + 31) / 32 * 32;
  threads = threads > 256 ? 256 : threads;
#define MS_ROPE_CASE(TA, TC)                                                                                         \
  MS_LAUNCH_RESULT("rope_kv_store",                                                                                  \
                   ms_launch(rope_kv_store_kernel<TA, TC>, dim3(tokens), dim3(threads), 0, stream, 1, true,          \
                             (const TA*)qkv, ld, bias, positions, seq_of_token, block_table, max_pages, num_pages,   \
                             (const float2*)cos_sin, rot, interleaved, (TA*)q_out, (TC*)k_pages, (TC*)v_pages, hq,   \
                             hkv, hd, page_size))
  if (act_dtype == MS_F32 && cache_dtype == MS_F32)
    MS_ROPE_CASE(float, float);
  else if (act_dtype == MS_BF16 && cache_dtype == MS_BF16)
    MS_ROPE_CASE(__nv_bfloat16, __nv_bfloat16);
  else if (act_dtype == MS_F32 && cache_dtype == MS_BF16)
    MS_ROPE_CASE(float, __nv_bfloat16);
  else
    MS_REQUIRE(false, "rope_kv_store: unsupported dtypes act=%d cache=%d", act_dtype, cache_dtype);
#undef MS_ROPE_CASE
  return 0;
}
