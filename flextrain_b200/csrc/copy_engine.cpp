// Copy engine: pinned-host <-> HBM transfers on dedicated CUDA streams, submitted from a worker thread.
//
// The reference moves weights, gradients, optimizer state and activations with one Python-issued
// Tensor.copy_ per tensor on three streams (flextrain/engine/buffers.py:1088-1164,
// flextrain/core/activation_schema.py:483-519).  Here Python hands over a *batch* of coalesced
// transfers (one per ring slot or activation slot) and returns at once; a worker thread issues the
// cudaMemcpyAsync calls, the cross-stream waits and the event records, so the interpreter never sits
// between a DMA and the compute that depends on it.
//
//   streams   0 = inbound (H2D), 1 = outbound (D2H), 2 = context (window refills)
//   events    keyed by a caller-chosen 64-bit id; waiting on a key that was never recorded is an error
//             (-5), never a silent pass or a hang
//   device<0  host-only mode: the same queue and event bookkeeping with memcpy, for CPU tests
//
// One cudaMemcpyAsync per transfer: the batched-memcpy driver entry points are not used.
#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

struct Job {
  void* dst;
  const void* src;
  size_t nbytes;
  int stream;            // 0..2
  uint64_t wait_key;     // 0 = none: engine event this transfer must wait for
  void* wait_external;   // cudaEvent_t recorded by the caller (e.g. on the compute stream), or null
  uint64_t record_key;   // 0 = none: engine event recorded after this transfer
};

struct Engine {
  int device;
  cudaStream_t streams[3] = {nullptr, nullptr, nullptr};
  std::unordered_map<uint64_t, cudaEvent_t> events;     // recorded engine events
  std::unordered_map<uint64_t, bool> host_events;       // host-only mode
  std::mutex mu;
  std::condition_variable cv_work, cv_done;
  std::deque<std::pair<uint64_t, std::vector<Job>>> queue;
  uint64_t next_ticket = 1, done_ticket = 0;
  std::atomic<int> error{0};
  std::atomic<uint64_t> bytes_moved{0}, copies{0};
  bool stop = false;
  std::thread worker;
};

void run_batch(Engine* e, std::vector<Job>& jobs) {
  for (Job& j : jobs) {
    if (e->device < 0) {
      if (j.wait_key) {
        std::lock_guard<std::mutex> g(e->mu);
        if (!e->host_events.count(j.wait_key)) { e->error = -5; continue; }
      }
      if (j.nbytes) std::memcpy(j.dst, j.src, j.nbytes);
      if (j.record_key) {
        std::lock_guard<std::mutex> g(e->mu);
        e->host_events[j.record_key] = true;
      }
    } else {
      cudaStream_t s = e->streams[j.stream];
      if (j.wait_external) cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(j.wait_external), 0);
      if (j.wait_key) {
        cudaEvent_t ev = nullptr;
        {
          std::lock_guard<std::mutex> g(e->mu);
          auto it = e->events.find(j.wait_key);
          if (it != e->events.end()) ev = it->second;
        }
        if (ev == nullptr) { e->error = -5; continue; }
        cudaStreamWaitEvent(s, ev, 0);
      }
      if (j.nbytes) {
        cudaError_t rc = cudaMemcpyAsync(j.dst, j.src, j.nbytes, cudaMemcpyDefault, s);
        if (rc != cudaSuccess) { e->error = -100 - static_cast<int>(rc); continue; }
      }
      if (j.record_key) {
        cudaEvent_t ev = nullptr;
        {
          std::lock_guard<std::mutex> g(e->mu);
          auto it = e->events.find(j.record_key);
          if (it != e->events.end()) ev = it->second;
        }
        if (ev == nullptr) {
          cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
          std::lock_guard<std::mutex> g(e->mu);
          e->events[j.record_key] = ev;
        }
        cudaEventRecord(ev, s);
      }
    }
    e->bytes_moved += j.nbytes;
    e->copies += 1;
  }
}

void worker_main(Engine* e) {
  if (e->device >= 0) cudaSetDevice(e->device);
  for (;;) {
    std::pair<uint64_t, std::vector<Job>> item;
    {
      std::unique_lock<std::mutex> lk(e->mu);
      e->cv_work.wait(lk, [&] { return e->stop || !e->queue.empty(); });
      if (e->queue.empty()) return;
      item = std::move(e->queue.front());
      e->queue.pop_front();
    }
    run_batch(e, item.second);
    {
      std::lock_guard<std::mutex> g(e->mu);
      e->done_ticket = item.first;
    }
    e->cv_done.notify_all();
  }
}

}  // namespace

extern "C" {

void* ftb_ce_create(int device) {
  Engine* e = new Engine();
  e->device = device;
  if (device >= 0) {
    if (cudaSetDevice(device) != cudaSuccess) { delete e; return nullptr; }
    for (int i = 0; i < 3; ++i)
      if (cudaStreamCreateWithFlags(&e->streams[i], cudaStreamNonBlocking) != cudaSuccess) { delete e; return nullptr; }
  }
  e->worker = std::thread(worker_main, e);
  return e;
}

void ftb_ce_destroy(void* h) {
  Engine* e = static_cast<Engine*>(h);
  {
    std::lock_guard<std::mutex> g(e->mu);
    e->stop = true;
  }
  e->cv_work.notify_all();
  if (e->worker.joinable()) e->worker.join();
  if (e->device >= 0) {
    cudaSetDevice(e->device);
    for (auto& kv : e->events) cudaEventDestroy(kv.second);
    for (int i = 0; i < 3; ++i)
      if (e->streams[i]) cudaStreamDestroy(e->streams[i]);
  }
  delete e;
}

// Enqueue `n` transfers (parallel arrays). Returns a ticket (> 0); the transfers are issued in order.
uint64_t ftb_ce_submit(void* h, int n, void** dst, void** src, const uint64_t* nbytes, const int* stream,
                       const uint64_t* wait_key, void** wait_external, const uint64_t* record_key) {
  Engine* e = static_cast<Engine*>(h);
  std::vector<Job> jobs(n);
  for (int i = 0; i < n; ++i)
    jobs[i] = Job{dst[i], src[i], static_cast<size_t>(nbytes[i]), stream[i], wait_key ? wait_key[i] : 0,
                  wait_external ? wait_external[i] : nullptr, record_key ? record_key[i] : 0};
  uint64_t t;
  {
    std::lock_guard<std::mutex> g(e->mu);
    t = e->next_ticket++;
    e->queue.emplace_back(t, std::move(jobs));
  }
  e->cv_work.notify_one();
  return t;
}

// Block the calling host thread until the worker has ISSUED every transfer up to `ticket` (not until the
// copies have completed on the device).
int ftb_ce_flush(void* h, uint64_t ticket) {
  Engine* e = static_cast<Engine*>(h);
  std::unique_lock<std::mutex> lk(e->mu);
  e->cv_done.wait(lk, [&] { return e->done_ticket >= ticket; });
  return e->error.load();
}

// Make `stream` (any CUDA stream, e.g. the framework's compute stream) wait for engine event `key`.
// `ticket` is the submission that records it. Returns -5 if the key was never recorded.
int ftb_ce_stream_wait(void* h, uint64_t key, uint64_t ticket, void* stream) {
  Engine* e = static_cast<Engine*>(h);
  ftb_ce_flush(h, ticket);
  if (e->device < 0) {
    std::lock_guard<std::mutex> g(e->mu);
    return e->host_events.count(key) ? 0 : -5;
  }
  cudaEvent_t ev = nullptr;
  {
    std::lock_guard<std::mutex> g(e->mu);
    auto it = e->events.find(key);
    if (it != e->events.end()) ev = it->second;
  }
  if (ev == nullptr) return -5;
  return -static_cast<int>(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), ev, 0));
}

// Wait on the host until all three copy streams are idle.
int ftb_ce_synchronize(void* h) {
  Engine* e = static_cast<Engine*>(h);
  uint64_t last;
  {
    std::lock_guard<std::mutex> g(e->mu);
    last = e->next_ticket - 1;
  }
  ftb_ce_flush(h, last);
  if (e->device >= 0)
    for (int i = 0; i < 3; ++i) cudaStreamSynchronize(e->streams[i]);
  return e->error.load();
}

void ftb_ce_forget(void* h, uint64_t key) {
  Engine* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  e->host_events.erase(key);
  // device events are kept and re-recorded: cudaEventRecord on an existing event is cheap
}

void ftb_ce_stats(void* h, uint64_t* bytes, uint64_t* copies) {
  Engine* e = static_cast<Engine*>(h);
  *bytes = e->bytes_moved.load();
  *copies = e->copies.load();
}

int ftb_ce_error(void* h) { return static_cast<Engine*>(h)->error.exchange(0); }

}  // extern "C"
