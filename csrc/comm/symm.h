// C interface of the peer-memory communication layer (symm.cu): symmetric allocations shared between
// the ranks of one node through CUDA IPC, bounded-wait signal flags, and the fused ZeRO kernels that
// reduce gradients, update the sharded optimizer state and publish parameters over NVLink from inside
// one kernel.  All waits are bounded and report through the status buffer (rb_status_read).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// ---- symmetric memory ------------------------------------------------------------------------------
void* rb_symm_alloc(long long bytes);            // device allocation, zero-filled; NULL on failure
int rb_symm_free(void* ptr);
int rb_ipc_export(void* ptr, unsigned char* handle64);          // fills 64 bytes
void* rb_ipc_import(const unsigned char* handle64);            // maps a peer's allocation; NULL on failure
int rb_ipc_close(void* ptr);

// ---- signals -----------------------------------------------------------------------------------------
// Every rank owns a signal pad of RB_SIGNAL_SLOTS u32 words per peer: pad[channel * world + src_rank].
// rb_signal_all: write `value` into slot (channel, my_rank) of every rank's pad (peer stores, release order).
// rb_wait_all:   wait until all `world` slots of `channel` in the LOCAL pad are >= value (acquire loads),
//                at most limit_ms milliseconds; on expiry sets kStatusFlagTimeout and returns.
int rb_signal_all(void* const* pad_ptrs_dev, int world, int my_rank, int channel, unsigned int value, void* stream);
int rb_wait_all(const void* local_pad, int world, int channel, unsigned int value, int limit_ms, void* stream);

// ---- fused ZeRO step -----------------------------------------------------------------------------------
typedef struct RbZeroArgs {
  void* const* grad_ptrs_dev;   // [world] device array: every rank's FULL fp32 gradient buffer (peer-mapped)
  void* const* lowp_ptrs_dev;   // [world] device array: every rank's FULL bf16 parameter buffer (peer-mapped)
  void* const* pad_ptrs_dev;    // [world] device array: every rank's signal pad
  void* local_pad;              // this rank's signal pad
  float* norm_slots;            // local fp32 [world]: per-rank partial sums of squares land here (peer-written)
  void* const* norm_ptrs_dev;   // [world] device array: every rank's norm_slots
  float* grad_shard;            // local fp32 [shard_len]: the reduced gradient shard
  float* master;                // local fp32 [shard_len]
  float* m;                     // local fp32 [shard_len]
  float* v;                     // local fp32 [shard_len]
  float* partials;              // local fp32 scratch [2048], zero-filled once by the caller: per-CTA partial sums in
                                // [0, 1024), two u32 "last CTA" counters at [1536] and [1537] (the kernels reset them)
  long long shard_off;          // first flat index this rank owns
  long long shard_len;
  long long decay_end;          // flat indices below this get weight decay
  int world, rank;
  unsigned int epoch;           // strictly increasing per step; flag values are derived from it
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_grad_norm;
  int limit_ms;
} RbZeroArgs;
// Phase 1: wait for every peer's "gradients ready" flag, sum this rank's shard over all peers' gradient
// buffers (fixed rank order, fp32), store it, and publish this shard's sum of squares to every rank.
// Phase 2: wait for all partial norms, clip, AdamW on the fp32 master shard, push the bf16 parameters into
// every rank's working copy, then raise the "parameters pushed" flag on every peer.
int rb_zero_reduce(const RbZeroArgs* args, void* stream);
int rb_zero_adam_push(const RbZeroArgs* args, void* stream);
// out[rows, n] = sum over `world` receive slots (dense, slot_elems bf16 each, rank order) (+ residual): the owner-side
// tail of the fused GEMM -> reduce-scatter (peer_mode 2 of rb_gemm_bf16).
int rb_tp_reduce_slots(const void* slots, int world, long long slot_elems, const void* residual, void* out, void* stream);
// One-shot all-reduce / all-gather for small tensor-parallel activations (decode steps, short prefills).
// Every rank has written its [rows, cols] bf16 contribution into its own symmetric staging buffer (stage_ptrs_dev[r]
// is rank r's, peer-mapped).  The kernel raises this rank's flag on every peer, waits (bounded, limit_ms) for all
// flags of (channel, epoch), then
//   gather == 0: out[rows, cols]           = sum over ranks (rank order, fp32) (+ residual[rows, cols])
//   gather == 1: out[rows, world * cols]   = the contributions side by side, rank r in columns [r*cols, (r+1)*cols)
// Callers alternate between two staging buffers from call to call; a flag for call n+1 is only raised after the
// rank has finished reading call n, so a buffer is never overwritten while a peer still reads it.
// `epoch_dev` (optional): device word holding the epoch, advanced by the caller with a kernel earlier in the stream;
// it replaces the `epoch` argument, so that a call captured in a CUDA graph sees a new epoch at every replay.
int rb_tp_allreduce(void* const* stage_ptrs_dev, void* const* pad_ptrs_dev, const void* local_pad, int world, int rank,
                    int channel, unsigned int epoch, const unsigned int* epoch_dev, int limit_ms, const void* residual,
                    void* out, int rows, int cols, int gather, void* stream);
#ifdef __cplusplus
}
#endif
