// C interface of the embedding kernels (embedding.cu).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// out[t, :] = wte[ids[t], :] (+ wpe[t % seq_len, :] when wpe != NULL); bf16 tables and output.
int rb_embedding_fwd(const long long* ids, const void* wte, const void* wpe, void* out, long long tokens, int dim,
                     int seq_len, long long vocab, void* stream);
// Ints of scratch rb_embedding_bwd needs for `tokens` ids over a table of `vocab` rows.
long long rb_embedding_bwd_scratch_ints(long long tokens, long long vocab);
// dwte[ids[t], :] += dy[t, :] (fp32 accumulate, rows visited in ascending t: bit-reproducible);
// dwpe[s, :] += sum_b dy[b*seq_len + s, :] when dwpe != NULL.  dy is bf16 [tokens, dim].
int rb_embedding_bwd(const long long* ids, const void* dy, float* dwte, float* dwpe, int* scratch, long long tokens,
                     int dim, int seq_len, long long vocab, void* stream);
#ifdef __cplusplus
}
#endif
