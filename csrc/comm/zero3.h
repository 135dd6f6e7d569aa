// C interface of the ZeRO-3 data plane (zero3.cu): parameters, gradients and optimizer state are cut into buckets
// (one per transformer block plus one for the embeddings); every rank owns a 1/world slice of each bucket.
//
//   rb_zero3_gather   all-gather of one bucket's bf16 parameters: every rank pulls the peers' slices out of their
//                     symmetric shard buffers into a local landing buffer (peer loads over NVLink).
//   rb_zero3_reduce   reduce-scatter of one bucket's fp32 gradients: every rank raises "my gradients of this bucket are
//                     written", waits for the same flag of all peers, pulls ITS slice out of every peer's symmetric
//                     gradient buffer, sums in rank order and adds the result to its gradient shard; the last CTA tells
//                     every peer that this rank is done reading their buffer.
//   rb_zero3_wait     stream-ordered bounded wait for a flag channel (used before a gradient buffer is reused).
//   rb_zero3_publish  exchanges this rank's partial sum of squares and loss sum with all peers.
//   rb_zero3_adam     waits for all partial norms, clips, applies AdamW to the owned slices of all buckets, writes the
//                     bf16 slices into this rank's symmetric shard buffer and raises "parameters of step k are ready".
//
// Flags live in a signal pad per rank: pad[channel * world + source_rank] (u32, monotonically increasing values).
// Kernels that run inside CUDA graphs read the value to signal / wait for from device memory (`epoch_dev`), which the
// host advances with rb_epoch_advance earlier in the same stream.  Every wait is bounded by `limit_ms`; on expiry the
// kernel sets the flag-timeout bit of the device status word (rb_status_read) and skips its data movement.
// No TMA multicast and no multimem instruction is used in this file: plain peer loads and stores only.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int rb_epoch_advance(unsigned int* epoch_dev, void* stream);       // *epoch_dev += 1 (one thread)

typedef struct RbZero3Gather {
  void* const* lowp_ptrs_dev;      // [world] device array: every rank's bf16 parameter-shard buffer (peer-mapped)
  const void* local_pad;           // this rank's signal pad
  const unsigned int* epoch_dev;   // number of optimizer steps this rank has completed; peers' flags must reach it
  int channel;                     // "parameters ready" channel
  long long shard_off;             // element offset of this bucket's slice inside every shard buffer
  long long n_per_rank;            // elements per rank in this bucket (multiple of 8)
  void* dst;                       // local bf16 landing buffer [world * n_per_rank]
  int world, rank, limit_ms, max_ctas;
  int threads;                     // threads per CTA: 64, 128 or 256 (anything else: 256)
} RbZero3Gather;
int rb_zero3_gather(const RbZero3Gather* a, void* stream);

typedef struct RbZero3Reduce {
  void* const* grad_ptrs_dev;      // [world] device array: every rank's fp32 gradient buffer holding this bucket
  void* const* pad_ptrs_dev;       // [world] device array: every rank's signal pad
  const void* local_pad;
  const unsigned int* epoch_dev;   // micro-batch counter of this rank
  int ready_channel, consumed_channel;
  long long n_per_rank;            // elements per rank (multiple of 4); this rank reads [rank * n_per_rank, +n_per_rank)
  float* shard_dst;                // this rank's fp32 gradient shard for this bucket [n_per_rank]
  int accumulate;                  // 0: shard_dst = sum; 1: shard_dst += sum
  unsigned int* counter;           // one u32, zero before the first call; the kernel resets it
  int world, rank, limit_ms, max_ctas;
  int threads;                     // threads per CTA: 64, 128 or 256 (anything else: 256)
} RbZero3Reduce;
int rb_zero3_reduce(const RbZero3Reduce* a, void* stream);

// Writes *epoch_dev into slot (channel, rank) of every rank's pad (release order after a system-scope fence): everything
// this stream wrote before is visible to a peer that sees the flag.  One tiny CTA.
int rb_zero3_signal(void* const* pad_ptrs_dev, int world, int rank, int channel, const unsigned int* epoch_dev, void* stream);

// dst[i] (+)= src[0][i] + src[1][i] + ... (fixed order, fp32), n a multiple of 4: the local half of a reduce-scatter
// whose remote slices were brought in by the copy engines.
typedef struct RbZero3Sum {
  const float* src[16];
  float* dst;
  long long n;
  int num_src;
  int accumulate;
} RbZero3Sum;
int rb_zero3_sum(const RbZero3Sum* a, void* stream);

// Waits until all `world` flags of `channel` in the local pad are >= *epoch_dev + delta (delta <= 0).
int rb_zero3_wait(const void* local_pad, int world, int channel, const unsigned int* epoch_dev, int delta, int limit_ms,
                  void* stream);

typedef struct RbZero3Step {
  void* const* pad_ptrs_dev;       // [world]
  const void* local_pad;
  void* const* slots_ptrs_dev;     // [world] device array: every rank's exchange slots, fp32 [2 * world] (sumsq, loss)
  const float* local_slots;
  const float* sumsq_local;        // device scalar: sum of squares of this rank's gradient shard
  const float* loss_local;         // device scalar: this rank's summed loss
  float* loss_out;                 // device scalar: sum of all ranks' loss sums (rank order) * loss_scale
  float loss_scale;
  int norm_channel, params_channel;
  unsigned int step;               // 1, 2, ...: value of the flags of this step
  unsigned int* step_epoch_dev;    // device word set to `step` once this rank's parameters are written
  // shard-wide views
  float* master; float* m; float* v; const float* grad; void* lowp_shard;   // [shard_len] each (lowp is bf16)
  long long shard_len;
  // bucket table (device arrays of `num_buckets` entries): first shard element of the bucket, and how many of this
  // rank's elements of that bucket take weight decay (the decayed parameters come first inside a bucket)
  const long long* bucket_shard_start;
  const long long* bucket_decay_count;
  int num_buckets;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_grad_norm;
  unsigned int* counter;           // one u32, zero before the first call; the kernel resets it
  int world, rank, limit_ms;
} RbZero3Step;
int rb_zero3_publish(const RbZero3Step* a, void* stream);
int rb_zero3_adam(const RbZero3Step* a, void* stream);

#ifdef __cplusplus
}
#endif
