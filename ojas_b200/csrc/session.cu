// An owner-thread session: the shape ojas-capi gives a backend whose handle may only be used from one thread (its Metal
// session keeps the device on a thread of its own and sends work to it, ojas-capi/src/owner.rs; the CUDA runtime of the
// reference is `!Send` for the same reason, ojas-cuda/src/backend.rs:27-31). A session starts a thread that opens the backend
// and is the only thread that ever touches it; any other thread hands it a call and waits for the answer. The open itself is
// waited for with a limit, so a caller that gives up does not hang on a device that never answers: the abandoned thread
// closes what it opened when it gets there.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <memory>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace {

struct Job {
  ojc_session_fn fn = nullptr;
  void* arg = nullptr;
  ojc_status status = OJC_OK;
  std::string error;
  bool done = false;
};

struct Shared {
  std::mutex m;
  std::condition_variable wake, answered;
  std::deque<Job*> queue;
  bool opened = false, closing = false, abandoned = false;
  ojc_status open_status = OJC_OK;
  std::string open_error;
  ojc_backend* be = nullptr;
};

void owner_main(std::shared_ptr<Shared> sh, int32_t device, uint64_t budget) {
  ojc_backend* be = nullptr;
  const ojc_status st = ojc_open(device, budget, &be);
  {
    std::lock_guard<std::mutex> lock(sh->m);
    sh->open_status = st;
    if (st != OJC_OK) sh->open_error = ojc_last_error();
    sh->be = be;
    sh->opened = true;
    if (sh->abandoned) {                     // nobody is waiting any more: give the device back and leave
      if (be) ojc_close(be);
      return;
    }
  }
  sh->answered.notify_all();
  if (st != OJC_OK) return;
  while (true) {
    Job* job = nullptr;
    {
      std::unique_lock<std::mutex> lock(sh->m);
      sh->wake.wait(lock, [&] { return sh->closing || !sh->queue.empty(); });
      if (sh->queue.empty()) break;          // closing, and every queued call has been answered
      job = sh->queue.front();
      sh->queue.pop_front();
    }
    const ojc_status js = (ojc_status)job->fn(be, job->arg);
    {
      std::lock_guard<std::mutex> lock(sh->m);
      job->status = js;
      if (js != OJC_OK) job->error = ojc_last_error();
      job->done = true;
    }
    sh->answered.notify_all();
  }
  ojc_close(be);
}

}  // namespace

struct ojc_session {
  std::shared_ptr<Shared> sh;
  std::thread owner;
};

extern "C" {

ojc_status ojc_session_open(int32_t device_ordinal, uint64_t budget_bytes, uint64_t open_timeout_ms, ojc_session** out) {
  const char* op = "session_open";
  if (!out) return ojc_fail(OJC_ERR_BACKEND, op, "null out pointer");
  *out = nullptr;
  ojc_session* s = new ojc_session();
  s->sh = std::make_shared<Shared>();
  s->owner = std::thread(owner_main, s->sh, device_ordinal, budget_bytes);
  std::unique_lock<std::mutex> lock(s->sh->m);
  const bool in_time = s->sh->answered.wait_for(lock, std::chrono::milliseconds(open_timeout_ms), [&] { return s->sh->opened; });
  if (!in_time) {
    s->sh->abandoned = true;                 // the owner thread closes whatever it opens and exits on its own
    lock.unlock();
    s->owner.detach();
    delete s;
    return ojc_fail(OJC_ERR_WAIT_TIMEOUT, op, "the device did not open within the limit");
  }
  const ojc_status st = s->sh->open_status;
  const std::string err = s->sh->open_error;
  lock.unlock();
  if (st != OJC_OK) {
    s->owner.join();
    delete s;
    return ojc_fail(st, op, err);
  }
  *out = s;
  return OJC_OK;
}

ojc_status ojc_session_call(ojc_session* s, ojc_session_fn fn, void* arg) {
  const char* op = "session_call";
  if (!s || !fn) return ojc_fail(OJC_ERR_BACKEND, op, "null session or function");
  if (std::this_thread::get_id() == s->owner.get_id()) return (ojc_status)fn(s->sh->be, arg);   // a call made from inside a call runs in place
  Job job;
  job.fn = fn; job.arg = arg;
  {
    std::unique_lock<std::mutex> lock(s->sh->m);
    if (s->sh->closing) return ojc_fail(OJC_ERR_BACKEND, op, "the session is closing");
    s->sh->queue.push_back(&job);
    s->sh->wake.notify_one();
    s->sh->answered.wait(lock, [&] { return job.done; });
  }
  if (job.status != OJC_OK) return ojc_fail(job.status, "session", job.error);   // the owner thread's message, on the caller's thread
  return OJC_OK;
}

ojc_status ojc_session_close(ojc_session* s) {
  if (!s) return OJC_OK;
  {
    std::lock_guard<std::mutex> lock(s->sh->m);
    s->sh->closing = true;
  }
  s->sh->wake.notify_all();
  if (s->owner.joinable()) s->owner.join();
  delete s;
  return OJC_OK;
}

// ---- the training ops ojas-capi routes to a session (OP_TRAIN_OPEN, OP_TRAIN_STEP: ojas-capi/src/train.rs), as calls on the owner thread
namespace {
struct TrainOpenArgs { const ojc_model_spec* spec; const ojc_train_config* cfg; int64_t batch, seq; ojc_trainer** out; };
struct TrainRunArgs { ojc_trainer* tr; const uint32_t* const* ids; const uint32_t* const* targets; int64_t k; ojc_step_report* report; };
}  // namespace

ojc_status ojc_session_train_open(ojc_session* s, const ojc_model_spec* spec, const ojc_train_config* cfg, int64_t batch, int64_t seq, ojc_trainer** out) {
  TrainOpenArgs a{spec, cfg, batch, seq, out};
  return ojc_session_call(s, [](ojc_backend* be, void* p) -> int32_t { auto* t = (TrainOpenArgs*)p; return ojc_trainer_open(be, t->spec, t->cfg, t->batch, t->seq, t->out); }, &a);
}

ojc_status ojc_session_train_run(ojc_session* s, ojc_trainer* tr, const uint32_t* const* ids_host, const uint32_t* const* targets_host, int64_t k, ojc_step_report* report) {
  TrainRunArgs a{tr, ids_host, targets_host, k, report};
  return ojc_session_call(s, [](ojc_backend*, void* p) -> int32_t { auto* t = (TrainRunArgs*)p; return ojc_trainer_run(t->tr, t->ids, t->targets, t->k, t->report); }, &a);
}

ojc_status ojc_session_train_close(ojc_session* s, ojc_trainer* tr) {
  return ojc_session_call(s, [](ojc_backend*, void* p) -> int32_t { return ojc_trainer_close((ojc_trainer*)p); }, tr);
}

}  // extern "C"
