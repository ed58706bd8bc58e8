// CPU model of the persistent kernel's scheduling protocol: std::atomic + threads instead of PTX
// acquire/release + CTAs, same structure as csrc/maco_kernel.cu:
//
//   * monotonic event counters, launch `epoch` waits for events[e] >= epoch * count
//   * STATIC mode: per-worker queues in global topological order, each task waits for itself
//   * DYNAMIC mode: a scheduler thread polls dispatch groups in a 32-group window and pushes ready
//     tasks into per-worker rings (slot first, then head with release); workers publish tails;
//     back-pressure when a ring is full; TERMINATE closes each ring
//   * every wait is bounded; on expiry the waiter records {status, task, event}, raises the
//     abort word, and everybody drains
//
// It exists so that the protocol can be exercised on a machine without a GPU (and under
// -fsanitize=thread): dependency resolution, ring wrap-around and back-pressure, re-execution
// across epochs, and injected faults - a worker that stalls, a producer that never signals.
// The reference has no such model; its device protocol is untested (no test touches
// maco_simple_persistent_kernel or the scheduler CTA).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr uint32_t kTerminate = 0xffffffffu;
enum Status : uint32_t { OK = 0, TIMEOUT = 1, BAD_TASK = 2, QUEUE_OVERFLOW = 4 };

struct SimTask {            // mirrors the scheduling part of MacoTaskDesc
  int32_t wait_event[2];
  uint32_t wait_count[2];
  int32_t signal_event[2];
  uint32_t work_us;         // simulated task duration
  uint32_t stall;           // fault injection: 1 = this task never finishes (worker stalls until abort)
};

struct SimGroup { uint32_t first_task, num_tasks; int32_t wait_event[2]; uint32_t wait_count[2]; };

struct Sim {
  const SimTask* tasks; uint32_t num_tasks;
  const SimGroup* groups; uint32_t num_groups;
  uint32_t num_workers, ring_size, mode, epoch;
  uint64_t budget_us;
  std::vector<std::atomic<uint32_t>> events, heads, tails, ring;
  const uint32_t* static_queue; const uint32_t* static_count; uint32_t static_stride;
  std::atomic<uint32_t> abort_word{0}, status{0}, fail_task{0}, fail_event{0}, completed{0}, order_pos{0};
  uint32_t* order;          // completion order (task indices), may be null
  Sim(uint32_t ne, uint32_t nw, uint32_t rs) : events(ne), heads(nw), tails(nw), ring((size_t)nw * rs) {
    for (auto& e : events) e.store(0);
    for (auto& h : heads) h.store(0);
    for (auto& t : tails) t.store(0);
  }
};

using Clock = std::chrono::steady_clock;

bool aborted(Sim& s) { return s.abort_word.load(std::memory_order_relaxed) == s.epoch; }

void report(Sim& s, uint32_t st, uint32_t task, uint32_t event) {
  uint32_t expected = s.abort_word.load(std::memory_order_relaxed);
  if (expected != s.epoch && s.abort_word.compare_exchange_strong(expected, s.epoch)) {
    s.fail_task.store(task); s.fail_event.store(event);
  }
  s.status.fetch_or(st);
}

bool wait_ge(Sim& s, std::atomic<uint32_t>& flag, uint32_t expect) {
  auto t0 = Clock::now();
  uint32_t spins = 0;
  while ((int32_t)(flag.load(std::memory_order_acquire) - expect) < 0) {
    if ((++spins & 63u) == 0) {
      if (aborted(s)) return false;
      if ((uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(Clock::now() - t0).count() > s.budget_us) return false;
      std::this_thread::yield();
    }
  }
  return true;
}

bool wait_deps(Sim& s, const SimTask& d, uint32_t task) {
  for (int j = 0; j < 2; ++j) {
    int e = d.wait_event[j];
    if (e < 0) continue;
    if (!wait_ge(s, s.events[e], s.epoch * d.wait_count[j])) { report(s, TIMEOUT, task, (uint32_t)e); return false; }
  }
  return true;
}

bool fetch(Sim& s, uint32_t w, uint32_t i, uint32_t q_base, uint32_t& task) {
  if (s.mode == 0) {
    task = i < s.static_count[w] ? s.static_queue[(size_t)w * s.static_stride + i] : kTerminate;
    return true;
  }
  uint32_t pos = q_base + i;
  if (!wait_ge(s, s.heads[w], pos + 1)) { report(s, TIMEOUT, 0xfffffffeu, w); return false; }
  task = s.ring[(size_t)w * s.ring_size + (pos % s.ring_size)].load(std::memory_order_relaxed);
  return true;
}

void worker(Sim& s, uint32_t w) {
  const uint32_t q_base = s.mode == 1 ? s.tails[w].load(std::memory_order_relaxed) : 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t task;
    if (!fetch(s, w, i, q_base, task)) return;
    if (task == kTerminate) { if (s.mode == 1) s.tails[w].store(q_base + i + 1, std::memory_order_release); return; }
    if (task >= s.num_tasks) { report(s, BAD_TASK, task, 0); return; }
    const SimTask& d = s.tasks[task];
    if (!wait_deps(s, d, task)) return;
    if (d.stall) {                                   // injected fault: hold the task until somebody aborts
      auto t0 = Clock::now();
      while (!aborted(s)) {
        if ((uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(Clock::now() - t0).count() > 4 * s.budget_us) break;
        std::this_thread::yield();
      }
      return;
    }
    if (d.work_us) std::this_thread::sleep_for(std::chrono::microseconds(d.work_us));
    if (s.order) s.order[s.order_pos.fetch_add(1)] = task;
    for (int j = 0; j < 2; ++j) if (d.signal_event[j] >= 0) s.events[d.signal_event[j]].fetch_add(1, std::memory_order_release);
    s.completed.fetch_add(1);
    if (s.mode == 1) s.tails[w].store(q_base + i + 1, std::memory_order_release);
    if (aborted(s)) return;
  }
}

bool push(Sim& s, std::vector<uint32_t>& heads_local, uint32_t w, uint32_t task) {
  uint32_t head = heads_local[w];
  if (!wait_ge(s, s.tails[w], head + 1 - s.ring_size)) return false;       // back-pressure
  s.ring[(size_t)w * s.ring_size + (head % s.ring_size)].store(task, std::memory_order_relaxed);   // slot first
  s.heads[w].store(head + 1, std::memory_order_release);                                         // then publish
  heads_local[w] = head + 1;
  return true;
}

void scheduler(Sim& s) {
  std::vector<uint32_t> heads_local(s.num_workers);
  for (uint32_t w = 0; w < s.num_workers; ++w) heads_local[w] = s.heads[w].load(std::memory_order_relaxed);
  uint32_t base = 0, window_done = 0, rr = 0;
  auto last = Clock::now();
  bool ok = true;
  while (ok && base < s.num_groups) {
    bool progress = false;
    for (uint32_t lane = 0; lane < 32 && ok; ++lane) {
      uint32_t g = base + lane;
      if (g >= s.num_groups || ((window_done >> lane) & 1u)) continue;
      const SimGroup& gd = s.groups[g];
      bool ready = true;
      for (int j = 0; j < 2; ++j) {
        int e = gd.wait_event[j];
        if (e >= 0 && (int32_t)(s.events[e].load(std::memory_order_acquire) - s.epoch * gd.wait_count[j]) < 0) ready = false;
      }
      if (!ready) continue;
      for (uint32_t t = 0; t < gd.num_tasks; ++t) {
        if (!push(s, heads_local, (rr + t) % s.num_workers, gd.first_task + t)) { report(s, QUEUE_OVERFLOW, gd.first_task, 0); ok = false; break; }
      }
      rr = (rr + gd.num_tasks) % s.num_workers;
      window_done |= 1u << lane;
      progress = true;
    }
    if (progress) {
      last = Clock::now();
      while (window_done & 1u) { window_done >>= 1; ++base; }
    } else {
      if (aborted(s) || (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(Clock::now() - last).count() > s.budget_us) {
        report(s, TIMEOUT, 0xfffffffdu, base);
        ok = false;
      }
      std::this_thread::yield();
    }
  }
  for (uint32_t w = 0; w < s.num_workers; ++w) push(s, heads_local, w, kTerminate);
}

}  // namespace

extern "C" {

// Runs `epochs` launches of the program. result[0] = status bits, [1] = failing task, [2] = failing
// event, [3] = tasks completed over all launches. `order` (optional) receives the completion order.
int maco_host_sim_run(const SimTask* tasks, uint32_t num_tasks, const SimGroup* groups, uint32_t num_groups,
                      uint32_t num_events, uint32_t num_workers, uint32_t ring_size, uint32_t mode,
                      const uint32_t* static_queue, const uint32_t* static_count, uint32_t static_stride,
                      uint32_t epochs, uint64_t budget_us, uint32_t* order, uint32_t* result) {
  if (num_workers == 0 || ring_size == 0) return -1;
  Sim s(num_events ? num_events : 1, num_workers, ring_size);
  s.tasks = tasks; s.num_tasks = num_tasks; s.groups = groups; s.num_groups = num_groups;
  s.num_workers = num_workers; s.ring_size = ring_size; s.mode = mode; s.budget_us = budget_us;
  s.static_queue = static_queue; s.static_count = static_count; s.static_stride = static_stride; s.order = order;
  for (uint32_t ep = 1; ep <= epochs; ++ep) {
    s.epoch = ep;
    std::vector<std::thread> th;
    for (uint32_t w = 0; w < num_workers; ++w) th.emplace_back(worker, std::ref(s), w);
    if (mode == 1) th.emplace_back(scheduler, std::ref(s));
    for (auto& t : th) t.join();
    if (s.status.load() != 0) break;
  }
  result[0] = s.status.load(); result[1] = s.fail_task.load(); result[2] = s.fail_event.load(); result[3] = s.completed.load();
  return 0;
}

int maco_host_sim_sizes(int* task, int* group) { *task = sizeof(SimTask); *group = sizeof(SimGroup); return 0; }

}  // extern "C"
