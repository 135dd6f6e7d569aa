// C interface of the flash-attention kernels (attention.cu).  bf16 tensors addressed by element
// strides {batch, row, head}; the head dimension is contiguous.  lse / delta are fp32 [batch, heads, seq_q].
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
typedef struct RbAttnArgs {
  const void* q; const void* k; const void* v;
  void* o;                 // forward: output; backward: the forward output (read)
  const void* d_o;         // backward: gradient of o (same strides as o)
  void* dq; void* dk; void* dv;
  float* lse;              // forward: written (may be NULL); backward: read
  float* delta;            // backward scratch, fp32 [batch, heads, seq_q]
  long long q_strides[3], k_strides[3], v_strides[3], o_strides[3];
  long long dq_strides[3], dk_strides[3], dv_strides[3];
  int batch, heads, kv_heads, seq_q, seq_k, head_dim;
  int causal;              // with seq_q < seq_k the queries are aligned to the end of the keys
  float scale;             // softmax scale, usually 1/sqrt(head_dim)
  const int* kv_lens;      // optional [batch]: keys at positions >= kv_lens[b] are padding and invisible (NULL: all seq_k
                           // keys are real).  Taken by the "tc2" kernels; the others return -9 when it is set.
} RbAttnArgs;
int rb_attention_fwd(const RbAttnArgs* args, void* stream);
int rb_attention_bwd(const RbAttnArgs* args, void* stream);
// tcgen05 paths (attention_tc.cu, attention_fwd2.cu, attention_bwd_tc.cu, attention_bwd2.cu); -9: shape not taken
int rb_attention_fwd_tc(const RbAttnArgs* args, void* stream);
int rb_attention_fwd_tc2(const RbAttnArgs* args, int poly_every, void* stream);
int rb_attention_bwd_tc(const RbAttnArgs* args, void* stream);
int rb_attention_delta_tc(const RbAttnArgs* args, void* stream);
int rb_attention_bwd_tc2(const RbAttnArgs* args, void* stream);
#ifdef __cplusplus
}
#endif
