// The fused form of the decode attention (attention_decode_cluster.cuh): bias, rotation and cache write inside the kernel.
#include "attention_decode_cluster.cuh"

MS_TIMELINE_SETTER(ms_timeline_set_attention_decode_cluster_rope)

// The fused form: reads rows of q|k|v as the projection left them (bfloat16, row stride ld, a multiple of 8),
// adds the bias (float32, or null), rotates q and k with the table cos_sin [positions][hd/2] (pairs j, j + hd/2),
// writes k and v of each row's position into the cache when `store` is set (the row then has hq + 2 hkv heads,
// else hq and the cache holds the position already), and attends.  Stands for ms_rope_kv_store followed by
// ms_attention_decode_cluster when every row is alone in its sequence.
MS_API int ms_attention_decode_cluster_rope(const void* qkv, int ld, const float* bias, const float* cos_sin, int store,
                                            void* k_pages, void* v_pages, void* out, const int* rows,
                                            const int* positions, const int* slot_of_token, const int* block_table,
                                            int max_pages, int num_pages, int tokens, int hq, int hkv, int hd,
                                            int page_size, int window, float scale, int num_splits, int stages,
                                            int warps, int keys_per_warp, int parts, float* scratch, long long scratch_words,
                                       int* counters, int num_counters, cudaStream_t stream) {
  MS_REQUIRE(qkv != nullptr && cos_sin != nullptr, "attention_decode_cluster_rope: no rows or no rotary table");
  MS_REQUIRE(ld % 8 == 0 && ld >= (hq + (store ? 2 * hkv : 0)) * hd, "attention_decode_cluster_rope: row stride %d (a multiple of 8, at least %d)",
             ld, (hq + (store ? 2 * hkv : 0)) * hd);
  MS_REQUIRE(((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0 && (uintptr_t)cos_sin % 8 == 0,
             "attention_decode_cluster_rope: rows and pages must be 16-byte aligned");
  const DclRaw raw = {(const __nv_bfloat16*)qkv, ld, bias, (const float2*)cos_sin, store ? 1 : 0};
  return decode_cluster_dispatch<true>(nullptr, &raw, k_pages, v_pages, out, rows, positions, slot_of_token, block_table,
                                 max_pages, num_pages, tokens, hq, hkv, hd, page_size, window, scale, num_splits, stages,
                                 warps, keys_per_warp, parts, scratch, scratch_words, counters, num_counters, stream);
}
