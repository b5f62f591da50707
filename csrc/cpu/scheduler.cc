// Request scheduler core of the data-parallel serving path: per-worker (per-GPU) ticket queues,
// least-loaded dispatch, dynamic batching with a queueing-delay bound, request deadlines,
// cancellation, hand-over of a dead worker's queue, and the counters behind /metrics.
//
// The payloads stay in the caller's language: this core only moves 64-bit tickets. A worker thread
// blocks in fdb_sched_next_batch WITHOUT holding the interpreter lock, which is what lets eight
// workers of one Python process keep eight GPUs busy.
//
// The reference leaves all of this to Triton (dynamic_batching / instance_group of a model's
// config.pbtxt, consumed in serving/src/fastdeploy_runtime.cc:972-1144 ProcessRequests) and has no
// scheduler of its own; its Python server serialises requests with one lock per model
// (python/fastdeploy/serving/model_manager.py:52-57).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <vector>

#include "fdb_cpu.h"

namespace {

using Clock = std::chrono::steady_clock;

inline int64_t now_us() {
  return std::chrono::duration_cast<std::chrono::microseconds>(Clock::now().time_since_epoch()).count();
}

struct Ticket {
  int64_t id;
  int64_t t_enqueue_us;
  int64_t deadline_us;   // absolute, 0 = none
};

constexpr int kHistBuckets = 12;   // batch sizes 1, 2, 3-4, 5-8, ... , > 1024

struct WorkerState {
  std::deque<Ticket> q;
  std::condition_variable cv;
  bool alive = true;
  int in_flight = 0;              // tickets handed out and not yet reported done
  // counters
  int64_t requests = 0, batches = 0, failed = 0, expired = 0, cancelled = 0;
  int64_t queue_wait_us = 0, compute_us = 0, batch_size_sum = 0;
  int64_t hist[kHistBuckets] = {0};
};

struct Sched {
  std::mutex mu;
  std::vector<WorkerState> w;
  int max_batch, max_delay_us;
  bool closed = false;
  int64_t next_id = 1;
  int rr = 0;
  std::deque<int64_t> orphaned;   // tickets that lost their last worker: the caller fails them
  explicit Sched(int n) : w(n) {}
};

int hist_bucket(int n) {
  int b = 0;
  int cap = 1;
  while (n > cap && b < kHistBuckets - 1) { cap <<= 1; ++b; }
  return b;
}

// least loaded alive worker (queued + in flight); ties rotate
int pick_worker(Sched* s) {
  const int n = static_cast<int>(s->w.size());
  int best = -1;
  long best_load = 0;
  s->rr = (s->rr + 1) % n;
  for (int k = 0; k < n; ++k) {
    const int i = (s->rr + k) % n;
    if (!s->w[i].alive) continue;
    const long load = static_cast<long>(s->w[i].q.size()) + s->w[i].in_flight;
    if (best < 0 || load < best_load) { best = i; best_load = load; }
  }
  return best;
}

}  // namespace

FDB_CPU_API void* fdb_sched_create(int num_workers, int max_batch, int max_delay_us) {
  if (num_workers < 1 || max_batch < 1 || max_delay_us < 0) {
    fdbcpu::set_error("scheduler: need at least one worker, max_batch >= 1, max_delay_us >= 0");
    return nullptr;
  }
  auto* s = new Sched(num_workers);
  s->max_batch = max_batch;
  s->max_delay_us = max_delay_us;
  return s;
}

FDB_CPU_API void fdb_sched_destroy(void* h) { delete static_cast<Sched*>(h); }

// Enqueues `count` requests at once. With together = 0 every request goes to the worker that is least
// loaded at that moment, so a burst spreads out; with together = 1 the whole burst goes to ONE worker,
// chosen once (requests that belong together - the frames of one pinned batch buffer - then stay adjacent
// in a batch). timeout_us > 0 sets a deadline relative to now. Writes the tickets and the chosen workers;
// returns the number enqueued (0 when closed or no worker is alive).
FDB_CPU_API int fdb_sched_submit(void* h, int count, int64_t timeout_us, int together, int64_t* tickets, int* workers) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  if (s->closed) { fdbcpu::set_error("scheduler is closed"); return 0; }
  const int64_t t = now_us();
  int done = 0;
  int fixed = -1;
  for (; done < count; ++done) {
    const int wi = (together && fixed >= 0) ? fixed : pick_worker(s);
    fixed = wi;
    if (wi < 0) { fdbcpu::set_error("all workers have failed"); break; }
    Ticket tk{s->next_id++, t, timeout_us > 0 ? t + timeout_us : 0};
    s->w[wi].q.push_back(tk);
    tickets[done] = tk.id;
    if (workers != nullptr) workers[done] = wi;
    if (s->w[wi].q.size() == 1 || static_cast<int>(s->w[wi].q.size()) >= s->max_batch) s->w[wi].cv.notify_one();
  }
  return done;
}

// Blocks (at most wait_us; < 0 = until something happens) for the next batch of worker `wi`: returns as
// soon as max_batch tickets are queued, or max_delay_us after the first one arrived. Tickets whose deadline
// has passed are not run: they come back in `expired` (n_expired). Returns the batch size, 0 on timeout,
// -1 when the scheduler is closed or the worker has been marked dead.
FDB_CPU_API int fdb_sched_next_batch(void* h, int wi, int64_t wait_us, int64_t* out, int cap, int64_t* expired,
                                     int expired_cap, int* n_expired) {
  auto* s = static_cast<Sched*>(h);
  std::unique_lock<std::mutex> lk(s->mu);
  WorkerState& w = s->w[wi];
  *n_expired = 0;
  const auto t_end = Clock::now() + std::chrono::microseconds(wait_us < 0 ? 0 : wait_us);
  for (;;) {
    if (s->closed || !w.alive) return -1;
    // drop what has expired at the head of the queue
    const int64_t t = now_us();
    while (!w.q.empty() && w.q.front().deadline_us != 0 && w.q.front().deadline_us <= t && *n_expired < expired_cap) {
      expired[(*n_expired)++] = w.q.front().id;
      w.q.pop_front();
      ++w.expired;
    }
    if (*n_expired > 0 && w.q.empty()) return 0;      // let the caller fail them now
    if (!w.q.empty()) {
      const int limit = std::min(cap, s->max_batch);
      const int64_t first_age = t - w.q.front().t_enqueue_us;
      if (static_cast<int>(w.q.size()) >= limit || first_age >= s->max_delay_us) {
        int n = 0;
        while (n < limit && !w.q.empty()) {
          const Ticket tk = w.q.front();
          w.q.pop_front();
          if (tk.deadline_us != 0 && tk.deadline_us <= t) {
            if (*n_expired < expired_cap) expired[(*n_expired)++] = tk.id;
            ++w.expired;
            continue;
          }
          w.queue_wait_us += t - tk.t_enqueue_us;
          out[n++] = tk.id;
        }
        if (n == 0) continue;
        w.in_flight += n;
        return n;
      }
      // wait for more requests, but no longer than the delay bound of the first one
      w.cv.wait_for(lk, std::chrono::microseconds(s->max_delay_us - first_age));
      continue;
    }
    if (wait_us < 0) {
      w.cv.wait(lk);
    } else {
      if (Clock::now() >= t_end) return 0;
      w.cv.wait_until(lk, t_end);
    }
  }
}

// Reports a finished batch of `n` tickets (ok = 0 when the model raised).
FDB_CPU_API void fdb_sched_done(void* h, int wi, int n, int ok, int64_t compute_us) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  WorkerState& w = s->w[wi];
  w.in_flight = std::max(0, w.in_flight - n);
  w.requests += n;
  w.batches += 1;
  w.batch_size_sum += n;
  w.compute_us += compute_us;
  w.hist[hist_bucket(n)] += 1;
  if (!ok) w.failed += n;
}

// Removes a ticket that has not been handed to a worker yet. Returns 1 when it was removed.
FDB_CPU_API int fdb_sched_cancel(void* h, int64_t ticket) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  for (auto& w : s->w) {
    for (auto it = w.q.begin(); it != w.q.end(); ++it) {
      if (it->id == ticket) {
        w.q.erase(it);
        ++w.cancelled;
        return 1;
      }
    }
  }
  return 0;
}

// Takes worker `wi` out of rotation and moves its queue to the living workers. Tickets that cannot be
// placed (no worker left) are appended to the orphan list. Returns the number of tickets moved.
FDB_CPU_API int fdb_sched_mark_dead(void* h, int wi) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  WorkerState& w = s->w[wi];
  w.alive = false;
  int moved = 0;
  while (!w.q.empty()) {
    const Ticket tk = w.q.front();
    w.q.pop_front();
    const int to = pick_worker(s);
    if (to < 0) {
      s->orphaned.push_back(tk.id);
    } else {
      s->w[to].q.push_back(tk);
      s->w[to].cv.notify_one();
      ++moved;
    }
  }
  w.cv.notify_all();
  return moved;
}

// Pops up to `cap` orphaned tickets (their requests can no longer be served).
FDB_CPU_API int fdb_sched_take_orphans(void* h, int64_t* out, int cap) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  int n = 0;
  while (n < cap && !s->orphaned.empty()) {
    out[n++] = s->orphaned.front();
    s->orphaned.pop_front();
  }
  return n;
}

FDB_CPU_API int fdb_sched_alive(void* h, int wi) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  return s->w[wi].alive ? 1 : 0;
}

FDB_CPU_API int fdb_sched_pending(void* h, int wi) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  return static_cast<int>(s->w[wi].q.size());
}

// Closes the scheduler: wakes every worker (next_batch returns -1) and moves everything still queued to
// the orphan list.
FDB_CPU_API void fdb_sched_close(void* h) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  s->closed = true;
  for (auto& w : s->w) {
    while (!w.q.empty()) {
      s->orphaned.push_back(w.q.front().id);
      w.q.pop_front();
    }
    w.cv.notify_all();
  }
}

// out[0..7] = requests, batches, failed, expired, cancelled, queue_wait_us, compute_us, batch_size_sum;
// out[8] = queued now, out[9] = in flight now, out[10] = alive; out[11 .. 11 + 12) = batch-size histogram
// (upper bounds 1, 2, 4, ..., 1024, +inf).
FDB_CPU_API int fdb_sched_stats(void* h, int wi, int64_t* out, int cap) {
  auto* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  if (cap < 11 + kHistBuckets) return -1;
  const WorkerState& w = s->w[wi];
  const int64_t v[11] = {w.requests, w.batches, w.failed, w.expired, w.cancelled, w.queue_wait_us, w.compute_us,
                         w.batch_size_sum, static_cast<int64_t>(w.q.size()), w.in_flight, w.alive ? 1 : 0};
  std::memcpy(out, v, sizeof(v));
  std::memcpy(out + 11, w.hist, sizeof(w.hist));
  return 11 + kHistBuckets;
}
