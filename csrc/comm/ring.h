// C interface of the ring / context-parallel attention helpers (ring.cu): copies between this GPU's memory and a
// peer's symmetric buffer, and the log-sum-exp merge of attention partial results.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// Copies `bytes` (a multiple of 16, both addresses 16-byte aligned) from `src` to `dst`; either side may be a peer's
// symmetric buffer mapped into this process.  `ctas` bounds the grid (0 = 32) so that the copy shares the GPU with
// the attention kernel of the previous block instead of displacing it; ctas < 0 hands the copy to a copy engine.
int rb_peer_copy(void* dst, const void* src, long long bytes, int ctas, void* stream);
// Folds one attention partial (o_new bf16 [B, S, H, D] dense, lse_new fp32 [B, H, S]) into the running result
// (o_acc fp32 [B, S, H, D], lse_acc fp32 [B, H, S]):
//   lse = log(exp(lse_acc) + exp(lse_new));  o_acc = o_acc * exp(lse_acc - lse) + o_new * exp(lse_new - lse)
// Rows whose lse_new is -inf (fully masked in this block) leave the running result untouched.  first != 0: the
// running result is uninitialised and is overwritten.  D must be a multiple of 8.
int rb_attn_merge(float* o_acc, float* lse_acc, const void* o_new, const float* lse_new, int B, int S, int H, int D,
                  int first, void* stream);
// out[i] (bf16) = sum, in rank order and in fp32, of slots[r * slot_elems + i] (bf16) over the ranks r with bit r of
// `mask` set: the owner-side fold of the key / value gradients that the ranks deposited for this rank's block.
// slot_elems must be a multiple of 4.
int rb_ring_fold(const void* slots, int world, unsigned int mask, long long slot_elems, void* out, void* stream);
#ifdef __cplusplus
}
#endif
