// Asynchronous file writer for checkpoints: a small pool of worker threads takes (path, bytes) jobs from a queue,
// writes each to "<path>.partial", fsyncs and renames it into place, so that a reader never sees a torn file and the
// training loop does not wait for the disk.  Jobs either copy the caller's bytes at submission or borrow the caller's
// buffer (pinned host memory that a device-to-host copy has filled) until the job's ticket is waited on.
// Counterpart of the reference's writer thread (crates/distributed/src/checkpoint.rs:271-308), which serialises
// through one channel and has no completion tickets.
#include "rb_runtime.h"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

struct Job {
  int64_t ticket;
  std::string path;
  std::vector<uint8_t> owned;      // copy mode
  const uint8_t* data;             // borrowed mode (owned empty) or owned.data()
  size_t bytes;
};

bool write_all(int fd, const uint8_t* p, size_t n) {
  while (n > 0) {
    const ssize_t w = ::write(fd, p, n > (1u << 30) ? (1u << 30) : n);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}

}  // namespace

struct RbAsyncWriter {
  std::mutex mu;
  std::condition_variable cv_work, cv_done;
  std::deque<Job> queue;
  std::vector<std::thread> workers;
  int64_t next_ticket = 1;
  int64_t in_flight = 0;
  std::vector<int64_t> running;    // tickets being written right now
  int64_t completed_below = 1;     // every ticket < this has finished (kept exact by `finished`)
  std::vector<int64_t> finished;   // finished tickets >= completed_below
  int errors = 0;
  std::string last_error;
  long long bytes_written = 0;
  bool stop = false;

  void mark_done(int64_t t) {
    finished.push_back(t);
    bool moved = true;
    while (moved) {
      moved = false;
      for (size_t i = 0; i < finished.size(); ++i) {
        if (finished[i] == completed_below) {
          finished[i] = finished.back();
          finished.pop_back();
          ++completed_below;
          moved = true;
          break;
        }
      }
    }
  }
  bool is_done(int64_t t) const {
    if (t < completed_below) return true;
    for (int64_t f : finished)
      if (f == t) return true;
    return false;
  }

  void run() {
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_work.wait(lk, [&] { return stop || !queue.empty(); });
        if (queue.empty()) return;              // stop requested and nothing left
        job = std::move(queue.front());
        queue.pop_front();
        if (!job.owned.empty()) job.data = job.owned.data();
      }
      std::string err;
      const std::string tmp = job.path + ".partial";
      const int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
      if (fd < 0) {
        err = "open " + tmp + ": " + strerror(errno);
      } else {
        if (!write_all(fd, job.data, job.bytes)) err = "write " + tmp + ": " + strerror(errno);
        if (err.empty() && ::fsync(fd) != 0) err = "fsync " + tmp + ": " + strerror(errno);
        ::close(fd);
        if (err.empty() && ::rename(tmp.c_str(), job.path.c_str()) != 0) err = "rename " + tmp + ": " + strerror(errno);
        if (!err.empty()) ::unlink(tmp.c_str());
      }
      {
        std::lock_guard<std::mutex> lk(mu);
        if (!err.empty()) {
          ++errors;
          last_error = err;
        } else {
          bytes_written += static_cast<long long>(job.bytes);
        }
        --in_flight;
        mark_done(job.ticket);
      }
      cv_done.notify_all();
    }
  }
};

extern "C" {

RbAsyncWriter* rb_aw_create(int num_threads) {
  if (num_threads < 1) num_threads = 1;
  if (num_threads > 16) num_threads = 16;
  RbAsyncWriter* w = new RbAsyncWriter();
  for (int i = 0; i < num_threads; ++i) w->workers.emplace_back([w] { w->run(); });
  return w;
}

void rb_aw_destroy(RbAsyncWriter* w) {
  if (!w) return;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    w->stop = true;
  }
  w->cv_work.notify_all();
  for (auto& t : w->workers) t.join();       // workers drain the queue before they leave
  delete w;
}

static int64_t submit(RbAsyncWriter* w, const char* path, const void* data, long long bytes, bool copy) {
  if (!w || !path || bytes < 0 || (bytes > 0 && !data)) return -1;
  Job job;
  job.path = path;
  job.bytes = static_cast<size_t>(bytes);
  job.data = static_cast<const uint8_t*>(data);
  if (copy && bytes > 0) {
    job.owned.assign(job.data, job.data + job.bytes);
    job.data = nullptr;                        // re-pointed at owned.data() by the worker (the vector may move)
  }
  int64_t ticket;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    if (w->stop) return -1;
    ticket = job.ticket = w->next_ticket++;
    ++w->in_flight;
    w->queue.push_back(std::move(job));
  }
  w->cv_work.notify_one();
  return ticket;
}

int64_t rb_aw_submit_copy(RbAsyncWriter* w, const char* path, const void* data, long long bytes) {
  return submit(w, path, data, bytes, true);
}

int64_t rb_aw_submit_borrowed(RbAsyncWriter* w, const char* path, const void* data, long long bytes) {
  return submit(w, path, data, bytes, false);
}

int rb_aw_wait(RbAsyncWriter* w, int64_t ticket, int timeout_ms) {
  if (!w || ticket <= 0) return -1;
  std::unique_lock<std::mutex> lk(w->mu);
  if (ticket >= w->next_ticket) return -1;
  auto done = [&] { return w->is_done(ticket); };
  if (timeout_ms < 0) {
    w->cv_done.wait(lk, done);
    return 0;
  }
  return w->cv_done.wait_for(lk, std::chrono::milliseconds(timeout_ms), done) ? 0 : 1;
}

int rb_aw_flush(RbAsyncWriter* w, int timeout_ms) {
  if (!w) return -1;
  std::unique_lock<std::mutex> lk(w->mu);
  auto idle = [&] { return w->in_flight == 0; };
  if (timeout_ms < 0) {
    w->cv_done.wait(lk, idle);
  } else if (!w->cv_done.wait_for(lk, std::chrono::milliseconds(timeout_ms), idle)) {
    return -2;                                 // still busy
  }
  return w->errors;
}

int rb_aw_pending(RbAsyncWriter* w) {
  if (!w) return -1;
  std::lock_guard<std::mutex> lk(w->mu);
  return static_cast<int>(w->in_flight);
}

long long rb_aw_bytes_written(RbAsyncWriter* w) {
  if (!w) return -1;
  std::lock_guard<std::mutex> lk(w->mu);
  return w->bytes_written;
}

int rb_aw_take_error(RbAsyncWriter* w, char* buf, int buf_len) {
  if (!w) return -1;
  std::lock_guard<std::mutex> lk(w->mu);
  const int n = w->errors;
  if (buf && buf_len > 0) snprintf(buf, static_cast<size_t>(buf_len), "%s", w->last_error.c_str());
  w->errors = 0;
  w->last_error.clear();
  return n;
}

}  // extern "C"
