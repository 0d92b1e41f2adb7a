// The decode attention whose splits meet inside a thread-block cluster (attention_decode_cluster.cuh): the form that is
// given encoded queries.  The fused form (bias, rotation and cache write inside) is built from
// attention_decode_cluster_rope.cu, so that the two halves of the kernel's many shapes compile side by side.
#include "attention_decode_cluster.cuh"

MS_TIMELINE_SETTER(ms_timeline_set_attention_decode_cluster)

// The most tiles a block can hold at once for a head size.
MS_API int ms_attention_decode_cluster_max_stages(int hd) { return dcl_max_stages(hd); }

// How many blocks with `stages` tiles an SM holds at once (by shared memory and by threads).
MS_API int ms_attention_decode_cluster_blocks_per_sm(int hd, int stages, int warps) {
  const size_t per_block = dcl_smem_bytes(hd, stages, warps) + 1024 + 16 * (size_t)hd * 4 + 1200;  // + the system's share and the static arrays
  int n = (int)((size_t)233472 / per_block);
  const int by_threads = 2048 / (warps * 32);
  n = n > by_threads ? by_threads : n;
  return n > 32 ? 32 : n;
}

MS_API long long ms_attention_decode_cluster_scratch_words(int tokens, int hq, int hkv, int hd, int parts) {
  return parts > 1 && hkv > 0 ? (long long)tokens * hkv * parts * ((hq / hkv) * hd + 32) : 0;
}

// As ms_attention_decode, with clusters in place of scratch memory for up to 8 runs of keys.  num_splits: 1, 2, 4 or 8 (the cluster size).
// stages: tiles of 64 keys a block holds at once, 1 .. ms_attention_decode_cluster_max_stages(hd).
// warps: 4, or 8 (for the few blocks of a small batch: half a tile per warp, or a quarter when the run goes through a ring).  keys_per_warp: the part of a tile a
// warp takes at a time with four warps, 16, 32 or 64; 0 chooses by the number of stages.
// parts: clusters a (row, kv head) pair's keys are spread over (1: none of what follows; up to 16, with clusters of more
// than one block): then `scratch` holds ms_attention_decode_cluster_scratch_words(...) float32 words and `counters`
// tokens * hkv int32 that are zero before the first launch (every launch leaves them zero).
MS_API int ms_attention_decode_cluster(const void* q, const void* k_pages, const void* v_pages, void* out,
                                       const int* rows, const int* positions, const int* slot_of_token,
                                       const int* block_table, int max_pages, int num_pages, int tokens, int hq, int hkv,
                                       int hd, int page_size, int window, float scale, int num_splits, int stages,
                                       int warps, int keys_per_warp, int parts, float* scratch, long long scratch_words,
                                       int* counters, int num_counters, cudaStream_t stream) {
  return decode_cluster_dispatch<false>(q, nullptr, const_cast<void*>(k_pages), const_cast<void*>(v_pages), out, rows, positions,
                                 slot_of_token, block_table, max_pages, num_pages, tokens, hq, hkv, hd, page_size, window,
                                 scale, num_splits, stages, warps, keys_per_warp, parts, scratch, scratch_words, counters, num_counters, stream);
}
