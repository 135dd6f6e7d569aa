// Background batch prefetcher for token files: a worker thread gathers the windows of consecutive training steps
// into a ring of caller-provided buffers (pinned host memory, so the host-to-device copy of step i + 1 can run under
// the compute of step i), in step order, ahead of the consumer.  The batches are the ones rb_tokens_sample_offsets /
// rb_tokens_gather would produce for the same (seed, step), so a run with and without the prefetcher sees identical data.
// The reference's DataLoader builds every batch on the calling thread (crates/data/src/lib.rs).
#include <chrono>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

#include "rb_runtime.h"

struct RbPrefetcher {
  const RbTokenFile* file;
  uint64_t seed, next_fill_step, next_take_step;
  int batch, width, depth;
  std::vector<int64_t*> buffers;
  std::vector<int> state;             // 0 free, 1 filled (waiting for the consumer), 2 held by the consumer
  std::vector<uint64_t> step_of;
  std::vector<int64_t> offsets;
  std::mutex mu;
  std::condition_variable cv_free, cv_ready;
  std::thread worker;
  bool stop = false;
  int error = 0;

  void run() {
    for (;;) {
      int slot = -1;
      uint64_t step = 0;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_free.wait(lk, [&] {
          if (stop) return true;
          for (int i = 0; i < depth; ++i)
            if (state[i] == 0) return true;
          return false;
        });
        if (stop) return;
        for (int i = 0; i < depth; ++i)
          if (state[i] == 0) { slot = i; break; }
        step = next_fill_step++;
        state[slot] = 3;                   // being filled
      }
      rb_tokens_sample_offsets(file, seed, step, batch, width, offsets.data());
      const int rc = rb_tokens_gather(file, offsets.data(), batch, width, buffers[slot]);
      {
        std::lock_guard<std::mutex> lk(mu);
        if (rc != 0) error = rc;
        step_of[slot] = step;
        state[slot] = 1;
      }
      cv_ready.notify_all();
    }
  }
};

extern "C" {

RbPrefetcher* rb_prefetch_create(const RbTokenFile* f, uint64_t seed, uint64_t first_step, int batch, int seq_len_plus1,
                                 int depth, int64_t* const* buffers) {
  if (!f || batch <= 0 || seq_len_plus1 <= 1 || depth < 1 || depth > 64 || !buffers) return nullptr;
  if (rb_tokens_len(f) < seq_len_plus1) return nullptr;
  for (int i = 0; i < depth; ++i)
    if (!buffers[i]) return nullptr;
  RbPrefetcher* p = new RbPrefetcher();
  p->file = f;
  p->seed = seed;
  p->next_fill_step = p->next_take_step = first_step;
  p->batch = batch;
  p->width = seq_len_plus1;
  p->depth = depth;
  p->buffers.assign(buffers, buffers + depth);
  p->state.assign(depth, 0);
  p->step_of.assign(depth, 0);
  p->offsets.assign(batch, 0);
  p->worker = std::thread([p] { p->run(); });
  return p;
}

int rb_prefetch_next(RbPrefetcher* p, int timeout_ms, uint64_t* step_out) {
  if (!p) return -1;
  std::unique_lock<std::mutex> lk(p->mu);
  int slot = -1;
  auto ready = [&] {
    if (p->error) return true;
    for (int i = 0; i < p->depth; ++i)
      if (p->state[i] == 1 && p->step_of[i] == p->next_take_step) { slot = i; return true; }
    return false;
  };
  if (timeout_ms < 0) {
    p->cv_ready.wait(lk, ready);
  } else if (!p->cv_ready.wait_for(lk, std::chrono::milliseconds(timeout_ms), ready)) {
    return -2;                             // nothing ready in time
  }
  if (slot < 0) return -3;                 // the worker hit an error (window out of range)
  p->state[slot] = 2;
  if (step_out) *step_out = p->next_take_step;
  ++p->next_take_step;
  return slot;
}

int rb_prefetch_release(RbPrefetcher* p, int index) {
  if (!p || index < 0 || index >= p->depth) return -1;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    if (p->state[index] != 2) return -1;
    p->state[index] = 0;
  }
  p->cv_free.notify_one();
  return 0;
}

void rb_prefetch_destroy(RbPrefetcher* p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    p->stop = true;
  }
  p->cv_free.notify_all();
  if (p->worker.joinable()) p->worker.join();
  delete p;
}

}  // extern "C"
