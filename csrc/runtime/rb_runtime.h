// C interface of the host runtime library (librb200_runtime.so): paged-KV block allocator, continuous-batching
// scheduler core, tile-configuration search, a memory-mapped token loader with a background batch prefetcher, and an asynchronous checkpoint file writer.  No GPU code; bound with ctypes.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
// ---- paged KV block allocator --------------------------------------------------------------------------------
typedef struct RbBlockAllocator RbBlockAllocator;
RbBlockAllocator* rb_ba_create(int num_blocks, int block_size);
void rb_ba_destroy(RbBlockAllocator* a);
int rb_ba_num_free(const RbBlockAllocator* a);
int rb_ba_num_blocks(const RbBlockAllocator* a);
int rb_ba_block_size(const RbBlockAllocator* a);
// Grows sequence `seq_id` so that it can hold `num_tokens` tokens in total (allocating ceil(n / block_size) blocks
// minus what it already owns).  Returns the number of newly allocated blocks, or -1 when there are not enough free
// blocks (nothing is allocated in that case).  A second call for the same sequence EXTENDS its table.
int rb_ba_reserve(RbBlockAllocator* a, int64_t seq_id, int num_tokens);
// Can `num_tokens` more tokens be held for this sequence (existing or new) without running out of blocks?
int rb_ba_can_reserve(const RbBlockAllocator* a, int64_t seq_id, int num_tokens);
int rb_ba_free(RbBlockAllocator* a, int64_t seq_id);           // returns the number of blocks released
int rb_ba_table_len(const RbBlockAllocator* a, int64_t seq_id);
int rb_ba_table(const RbBlockAllocator* a, int64_t seq_id, int32_t* out, int max_out);   // copies the table; returns its length
int64_t rb_ba_slot(const RbBlockAllocator* a, int64_t seq_id, int token_index);          // block * block_size + offset, -1 if unmapped
int rb_ba_num_sequences(const RbBlockAllocator* a);

// ---- tile-configuration search (autotuner core) --------------------------------------------------------------
// A search space is a list of dimensions, each with a list of integer choices.  Strategies: 0 grid, 1 random,
// 2 evolutionary, 3 bayesian-style (explore / exploit around the incumbent).  The caller measures each proposed
// configuration and reports the time; the searcher never runs kernels itself.
typedef struct RbSearch RbSearch;
RbSearch* rb_search_create(int strategy, int num_dims, const int* dim_sizes, const int* choices_flat, uint64_t seed,
                           int max_evals);
void rb_search_destroy(RbSearch* s);
int rb_search_next(RbSearch* s, int* config_out);                 // 1 = config_out filled, 0 = search complete
void rb_search_report(RbSearch* s, const int* config, double time_us);
int rb_search_best(const RbSearch* s, int* config_out, double* time_us_out);   // 1 if any result was reported
int rb_search_num_evals(const RbSearch* s);

// ---- memory-mapped token dataset ----------------------------------------------------------------------------------
typedef struct RbTokenFile RbTokenFile;
RbTokenFile* rb_tokens_open(const char* path, int bytes_per_token);      // 2 (uint16) or 4 (int32)
void rb_tokens_close(RbTokenFile* f);
int64_t rb_tokens_len(const RbTokenFile* f);
// Fills out[batch, seq_len + 1] (int64) with windows starting at the given offsets; returns 0 on success.
int rb_tokens_gather(const RbTokenFile* f, const int64_t* offsets, int batch, int seq_len_plus1, int64_t* out);
// Deterministic window offsets for (seed, step): uniform over valid starts.
void rb_tokens_sample_offsets(const RbTokenFile* f, uint64_t seed, uint64_t step, int batch, int seq_len_plus1,
                              int64_t* offsets_out);

// ---- background batch prefetcher over a token file -------------------------------------------------------------------
// A worker thread fills `depth` caller-provided buffers (each batch * seq_len_plus1 int64, typically pinned host
// memory) with the batches of steps first_step, first_step + 1, ... exactly as rb_tokens_sample_offsets +
// rb_tokens_gather produce them for (seed, step).  next: blocks until the batch of the next step in order is ready and
// returns its buffer index (step_out receives the step), -2 on timeout (timeout_ms < 0 waits for ever), -3 when the
// worker failed.  release: hands the buffer back once the caller has consumed it.  The file must outlive the prefetcher.
typedef struct RbPrefetcher RbPrefetcher;
RbPrefetcher* rb_prefetch_create(const RbTokenFile* f, uint64_t seed, uint64_t first_step, int batch, int seq_len_plus1,
                                 int depth, int64_t* const* buffers);
int rb_prefetch_next(RbPrefetcher* p, int timeout_ms, uint64_t* step_out);
int rb_prefetch_release(RbPrefetcher* p, int index);
void rb_prefetch_destroy(RbPrefetcher* p);

// ---- continuous-batching scheduler core -----------------------------------------------------------------------------
// Decisions of one serving iteration over the block allocator `alloc` (not owned): retire finished requests, resume
// paused ones, admit waiting ones while blocks and the prefill budget last, preempt a LOW-priority request when memory
// has run out and something more urgent waits.  policy: 0 first come first served, 1 shortest remaining first,
// 2 priority.  Request states: 0 waiting, 1 prefill, 2 generating, 3 paused, 4 completed.
typedef struct RbScheduler RbScheduler;
RbScheduler* rb_sched_create(RbBlockAllocator* alloc, int max_batch, int policy, double preemption_threshold,
                             int max_prefill_tokens);
void rb_sched_destroy(RbScheduler* s);
int64_t rb_sched_add(RbScheduler* s, int prompt_len, int max_tokens, int priority, int has_eos, int64_t eos_id);  // id
int rb_sched_has_work(const RbScheduler* s);
void rb_sched_retire(RbScheduler* s);
// Runs one iteration and fills the batch (policy order): ids, 1 where the whole prefix must be (re)computed, tokens in
// the cache after the step.  Returns the batch size, -2 when cap is too small.
int rb_sched_schedule(RbScheduler* s, int64_t* ids, int32_t* is_prefill, int32_t* seq_lens, int cap);
int rb_sched_take_retired(RbScheduler* s, int64_t* ids, int cap);           // ids retired since the last call
// Records one sampled token per request and grows its block table.  result[i]: 0 ignored (not running), 1 recorded,
// 2 recorded and paused for lack of blocks.  Returns the number paused.
int rb_sched_update(RbScheduler* s, const int64_t* ids, const int64_t* tokens, int n, int32_t* result);
int rb_sched_state(const RbScheduler* s, int64_t id);                       // -1 unknown
void rb_sched_stats(const RbScheduler* s, int64_t* out4);                   // completed, preempted, admitted, generated tokens
int rb_sched_list(const RbScheduler* s, int which, int64_t* ids, int cap);  // which: 0 pending, 1 running, 2 paused; returns count
void rb_sched_forget(RbScheduler* s, int64_t id);                           // drops the record of a completed request
// Removes an unfinished request from whichever queue holds it, frees its blocks and drops its record.  Returns 1 when
// a request was removed, 0 when it had already completed, -1 when the id is unknown.
int rb_sched_abort(RbScheduler* s, int64_t id);

// ---- asynchronous checkpoint file writer ----------------------------------------------------------------------------
// Worker threads write each job to "<path>.partial", fsync and rename it into place.  submit_* return a ticket (> 0)
// or -1.  `copy` jobs duplicate the bytes at submission; `borrowed` jobs read the caller's buffer until the ticket
// has been waited on.  wait: 0 done, 1 timed out (timeout_ms < 0 waits for ever).  flush: number of failed jobs since
// the last take_error, -2 when still busy after timeout_ms.  take_error copies the latest message and clears the count.
typedef struct RbAsyncWriter RbAsyncWriter;
RbAsyncWriter* rb_aw_create(int num_threads);
void rb_aw_destroy(RbAsyncWriter* w);                           // drains the queue first
int64_t rb_aw_submit_copy(RbAsyncWriter* w, const char* path, const void* data, long long bytes);
int64_t rb_aw_submit_borrowed(RbAsyncWriter* w, const char* path, const void* data, long long bytes);
int rb_aw_wait(RbAsyncWriter* w, int64_t ticket, int timeout_ms);
int rb_aw_flush(RbAsyncWriter* w, int timeout_ms);
int rb_aw_pending(RbAsyncWriter* w);
long long rb_aw_bytes_written(RbAsyncWriter* w);
int rb_aw_take_error(RbAsyncWriter* w, char* buf, int buf_len);
#ifdef __cplusplus
}
#endif
