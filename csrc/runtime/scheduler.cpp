// Iteration-level (continuous-batching) request scheduler core: queues, ordering policy, admission against the paged
// KV block allocator, preemption under memory pressure and retirement.  The serving engine calls it once per model
// step; token storage and timing stay with the caller, which passes in only what decisions need (lengths, priority,
// the sampled token).  Same decisions as the reference scheduler (crates/nn/src/continuous_batching.rs:170-439),
// except that the scheduling policy is honoured and the end-of-sequence id is per request.
#include "rb_runtime.h"

#include <algorithm>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

enum State { kWaiting = 0, kPrefill = 1, kGenerating = 2, kPaused = 3, kCompleted = 4 };

struct Req {
  int64_t id;
  int prompt_len, max_tokens, priority;
  bool has_eos;
  int64_t eos_id;
  int generated = 0;
  int64_t last_token = 0;
  int state = kWaiting;
  int total_len() const { return prompt_len + generated; }
  int remaining() const { return max_tokens - generated; }
  bool should_complete() const {
    if (generated >= max_tokens) return true;
    return has_eos && generated > 0 && last_token == eos_id;
  }
};

}  // namespace

struct RbScheduler {
  RbBlockAllocator* alloc;
  int max_batch, policy, max_prefill;
  double threshold;
  std::unordered_map<int64_t, Req> reqs;
  std::deque<int64_t> pending, paused;
  std::vector<int64_t> running;                 // in the order requests entered the running set
  std::vector<int64_t> retired;                 // retired since the last take
  int64_t next_id = 0;
  int64_t n_completed = 0, n_preempted = 0, n_admitted = 0, n_generated = 0;

  bool reserve(int64_t id, int tokens) { return rb_ba_reserve(alloc, id, tokens) >= 0; }

  template <class It>
  std::vector<int64_t> ordered(It first, It last) const {
    std::vector<int64_t> v(first, last);
    if (policy == 1) {          // shortest remaining tokens first
      std::stable_sort(v.begin(), v.end(), [&](int64_t a, int64_t b) {
        const Req &x = reqs.at(a), &y = reqs.at(b);
        const long kx = x.remaining() + (x.generated ? 0 : x.prompt_len), ky = y.remaining() + (y.generated ? 0 : y.prompt_len);
        return kx != ky ? kx < ky : a < b;
      });
    } else if (policy == 2) {   // priority
      std::stable_sort(v.begin(), v.end(), [&](int64_t a, int64_t b) {
        const Req &x = reqs.at(a), &y = reqs.at(b);
        return x.priority != y.priority ? x.priority > y.priority : a < b;
      });
    }
    return v;
  }

  void drop_running(int64_t id) { running.erase(std::find(running.begin(), running.end(), id)); }

  void retire() {
    std::vector<int64_t> done;
    for (int64_t id : running)
      if (reqs.at(id).should_complete()) done.push_back(id);
    for (int64_t id : done) {
      Req& r = reqs.at(id);
      drop_running(id);
      r.state = kCompleted;
      rb_ba_free(alloc, id);
      retired.push_back(id);
      ++n_completed;
      n_generated += r.generated;
    }
  }

  void try_resume() {
    const size_t n = paused.size();
    for (size_t i = 0; i < n; ++i) {
      if (static_cast<int>(running.size()) >= max_batch) break;
      Req& r = reqs.at(paused.front());
      if (!reserve(r.id, r.total_len() + 1)) break;
      paused.pop_front();
      r.state = kPrefill;                       // its cache was released: the whole prefix is recomputed
      running.push_back(r.id);
    }
  }

  void admit() {
    int budget = max_prefill;
    for (int64_t id : ordered(pending.begin(), pending.end())) {
      Req& r = reqs.at(id);
      if (static_cast<int>(running.size()) >= max_batch) break;
      if (r.prompt_len > budget && budget < max_prefill) break;
      if (!reserve(id, r.prompt_len + 1)) break;        // head-of-line: keep the order when memory is short
      pending.erase(std::find(pending.begin(), pending.end(), id));
      r.state = kPrefill;
      running.push_back(id);
      ++n_admitted;
      budget -= r.prompt_len;
    }
  }

  void maybe_preempt() {
    if (pending.empty() || running.size() <= 1) return;
    const int free_blocks = rb_ba_num_free(alloc);
    if (free_blocks > 0 && static_cast<double>(running.size()) / max_batch <= threshold) return;
    int waiting_best = 0;
    for (int64_t id : pending) waiting_best = std::max(waiting_best, reqs.at(id).priority);
    int64_t victim = -1;
    for (int64_t id : running) {
      const Req& r = reqs.at(id);
      if (r.priority < waiting_best && r.priority == 0) victim = std::max(victim, id);
    }
    if (victim < 0 || free_blocks > 0) return;
    drop_running(victim);
    rb_ba_free(alloc, victim);
    reqs.at(victim).state = kPaused;
    paused.push_back(victim);
    ++n_preempted;
  }
};

extern "C" {

RbScheduler* rb_sched_create(RbBlockAllocator* alloc, int max_batch, int policy, double preemption_threshold,
                             int max_prefill_tokens) {
  if (!alloc || max_batch <= 0 || policy < 0 || policy > 2 || max_prefill_tokens <= 0) return nullptr;
  RbScheduler* s = new RbScheduler();
  s->alloc = alloc;
  s->max_batch = max_batch;
  s->policy = policy;
  s->threshold = preemption_threshold;
  s->max_prefill = max_prefill_tokens;
  return s;
}

void rb_sched_destroy(RbScheduler* s) { delete s; }

int64_t rb_sched_add(RbScheduler* s, int prompt_len, int max_tokens, int priority, int has_eos, int64_t eos_id) {
  if (!s || prompt_len < 0 || max_tokens < 0) return -1;
  Req r;
  r.id = s->next_id++;
  r.prompt_len = prompt_len;
  r.max_tokens = max_tokens;
  r.priority = priority;
  r.has_eos = has_eos != 0;
  r.eos_id = eos_id;
  s->reqs.emplace(r.id, r);
  s->pending.push_back(r.id);
  return r.id;
}

int rb_sched_has_work(const RbScheduler* s) { return s && (!s->pending.empty() || !s->running.empty() || !s->paused.empty()); }

void rb_sched_retire(RbScheduler* s) {
  if (s) s->retire();
}

int rb_sched_schedule(RbScheduler* s, int64_t* ids, int32_t* is_prefill, int32_t* seq_lens, int cap) {
  if (!s) return -1;
  s->retire();
  s->try_resume();
  s->admit();
  s->maybe_preempt();
  const std::vector<int64_t> order = s->ordered(s->running.begin(), s->running.end());
  if (static_cast<int>(order.size()) > cap) return -2;
  for (size_t i = 0; i < order.size(); ++i) {
    const Req& r = s->reqs.at(order[i]);
    ids[i] = r.id;
    is_prefill[i] = r.state == kPrefill;
    seq_lens[i] = r.total_len();
  }
  return static_cast<int>(order.size());
}

int rb_sched_take_retired(RbScheduler* s, int64_t* ids, int cap) {
  if (!s) return -1;
  const int n = static_cast<int>(std::min<size_t>(s->retired.size(), static_cast<size_t>(cap < 0 ? 0 : cap)));
  for (int i = 0; i < n; ++i) ids[i] = s->retired[i];
  s->retired.erase(s->retired.begin(), s->retired.begin() + n);
  return n;
}

int rb_sched_update(RbScheduler* s, const int64_t* ids, const int64_t* tokens, int n, int32_t* result) {
  if (!s) return -1;
  int paused_now = 0;
  for (int i = 0; i < n; ++i) {
    auto it = s->reqs.find(ids[i]);
    if (it == s->reqs.end() || (it->second.state != kPrefill && it->second.state != kGenerating)) {
      if (result) result[i] = 0;                // not running: ignored
      continue;
    }
    Req& r = it->second;
    ++r.generated;
    r.last_token = tokens[i];
    r.state = kGenerating;
    if (result) result[i] = 1;
    if (!r.should_complete() && !s->reserve(r.id, r.total_len() + 1)) {
      s->drop_running(r.id);                    // out of blocks: pause this request instead of failing the batch
      rb_ba_free(s->alloc, r.id);
      r.state = kPaused;
      s->paused.push_back(r.id);
      ++s->n_preempted;
      ++paused_now;
      if (result) result[i] = 2;
    }
  }
  return paused_now;
}

int rb_sched_state(const RbScheduler* s, int64_t id) {
  if (!s) return -1;
  auto it = s->reqs.find(id);
  return it == s->reqs.end() ? -1 : it->second.state;
}

void rb_sched_stats(const RbScheduler* s, int64_t* out4) {
  if (!s || !out4) return;
  out4[0] = s->n_completed;
  out4[1] = s->n_preempted;
  out4[2] = s->n_admitted;
  out4[3] = s->n_generated;
}

int rb_sched_list(const RbScheduler* s, int which, int64_t* ids, int cap) {
  if (!s) return -1;
  std::vector<int64_t> v;
  if (which == 0) v.assign(s->pending.begin(), s->pending.end());
  else if (which == 1) v = s->running;
  else if (which == 2) v.assign(s->paused.begin(), s->paused.end());
  else return -1;
  const int n = static_cast<int>(v.size());
  if (ids)
    for (int i = 0; i < n && i < cap; ++i) ids[i] = v[i];
  return n;
}

int rb_sched_abort(RbScheduler* s, int64_t id) {
  if (!s) return -1;
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  Req& r = it->second;
  if (r.state == kCompleted) return 0;
  auto drop = [&](std::deque<int64_t>& q) {
    auto p = std::find(q.begin(), q.end(), id);
    if (p != q.end()) q.erase(p);
  };
  drop(s->pending);
  drop(s->paused);
  auto p = std::find(s->running.begin(), s->running.end(), id);
  if (p != s->running.end()) s->running.erase(p);
  rb_ba_free(s->alloc, id);                     // no-op when the request holds no blocks
  s->reqs.erase(it);
  return 1;
}

void rb_sched_forget(RbScheduler* s, int64_t id) {
  if (!s) return;
  auto it = s->reqs.find(id);
  if (it != s->reqs.end() && it->second.state == kCompleted) s->reqs.erase(it);
}

}  // extern "C"
