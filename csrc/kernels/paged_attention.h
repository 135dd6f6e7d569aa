// C interface of the paged KV-cache kernels (paged_attention.cu).
// Cache layout per layer: [num_blocks, block_size, kv_heads, head_dim] bf16 for K and for V.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// Copies new keys / values into their cache slots.  k_new / v_new: [tokens, kv_heads, head_dim] with row pitch
// ld_k / ld_v (so they may be column ranges of a packed QKV projection).  slot_mapping[t] = block * block_size + offset,
// negative slots are skipped.
int rb_kv_append(const void* k_new, long long ld_k, const void* v_new, long long ld_v, void* k_cache, void* v_cache,
                 const long long* slot_mapping, long long tokens, int kv_heads, int head_dim, long long num_slots,
                 void* stream);
// Decode attention: one query token per sequence.
//   q [batch, heads, head_dim] (row pitch ld_q), out [batch, heads, head_dim] (row pitch ld_o), both bf16
//   block_tables [batch, max_blocks] int32, context_lens [batch] int32 (tokens already in the cache, incl. the new one)
//   scratch: fp32 [rb_paged_attention_scratch_floats(...)] for the per-slice partial results of the split-KV kernel
long long rb_paged_attention_scratch_floats(int batch, int heads, int head_dim, int max_blocks, int block_size);
int rb_paged_attention_decode(const void* q, long long ld_q, void* out, long long ld_o, const void* k_cache,
                              const void* v_cache, const int* block_tables, int max_blocks, const int* context_lens,
                              int batch, int heads, int kv_heads, int head_dim, int block_size, long long num_blocks,
                              float scale, float* scratch, void* stream);
#ifdef __cplusplus
}
#endif
