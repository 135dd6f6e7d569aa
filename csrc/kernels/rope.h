// C interface of the rotary-embedding and SwiGLU kernels (rope.cu).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// In-place rotary position embedding on bf16 x viewed as [tokens, heads, head_dim] with row pitch ld
// (head h starts at column h*head_dim).  Pairs are (i, i + head_dim/2) ("rotate half").  The position of
// token t is positions[t] when positions != NULL, else pos_offset + (t % seq_len).  inverse = 1 applies the
// transposed rotation, which is the backward pass.
int rb_rope(void* x, long long ld, const long long* positions, long long tokens, int heads, int head_dim, int seq_len,
            long long pos_offset, float theta, int inverse, void* stream);
// h[t, f] = silu(gu[t, f]) * gu[t, F + f]   with gu [tokens, 2F] (gate | up), bf16
int rb_swiglu_fwd(const void* gu, long long ld_gu, void* h, long long ld_h, long long tokens, int F, void* stream);
// dgu[t, f] = dh * up * silu'(gate);  dgu[t, F + f] = dh * silu(gate)
int rb_swiglu_bwd(const void* dh, long long ld_dh, const void* gu, long long ld_gu, void* dgu, long long ld_dgu,
                  long long tokens, int F, void* stream);
#ifdef __cplusplus
}
#endif
