// C interface of the NVLink-multicast (NVLS) data-plane kernels (nvls.cu).  `mc` is the multicast address of a buffer
// that every rank has bound to one multicast object; the same offsets address the same elements on every rank.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// dst[i] (+)= sum over all ranks of buffer[elem_offset + i], i < n, fp32 (n and elem_offset multiples of 4).
int rb_mc_reduce_f32(const void* mc, long long elem_offset, void* dst, long long n, int accumulate, int max_ctas, void* stream);
// In place: bytes [byte_offset, byte_offset + nbytes) of EVERY rank's buffer become the sum over ranks (fp32 elements, or
// bf16 pairs accumulated in fp32).  Each rank calls it on its own disjoint range.
int rb_mc_allreduce(void* mc, long long byte_offset, long long nbytes, int bf16, int max_ctas, void* stream);
// Copies nbytes from local memory `src` to offset byte_offset of every rank's buffer.
int rb_mc_broadcast(const void* src, void* mc, long long byte_offset, long long nbytes, int max_ctas, void* stream);
// One-shot all-reduce for tensor-parallel inference: out = sum over ranks of the staged [rows, cols] bf16 tensor at the
// multicast address `mc_stage` (+ residual).  Flags as in rb_tp_allreduce (signal pad, device-resident epoch, bounded wait).
int rb_tp_allreduce_mc(const void* mc_stage, void* const* pad_ptrs_dev, const void* local_pad, int world, int rank, int channel,
                       const unsigned int* epoch_dev, int limit_ms, const void* residual, void* out, int rows, int cols, void* stream);
#ifdef __cplusplus
}
#endif
