// Host operands and results in ordinary (pageable) memory.
//
// A JVM hands its arrays over from the Java heap (GetPrimitiveArrayCritical, utils/NativeHelper.java:361-418 is the
// reference's own bridge of that kind), i.e. as pageable memory. cudaMemcpyAsync from or to such memory is staged by
// the driver through one internal buffer by one thread, at about a fifth of the PCIe rate. The copies here do that
// staging themselves: a ring of pinned slices per handle, filled (or drained) by a few host threads in parallel while
// the DMA engine moves the slices already filled. Pinned or registered host memory, small transfers and handles
// without a ring take the plain cudaMemcpyAsync.
#include "cla_common.cuh"
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <sched.h>
#include <thread>

namespace cla {

constexpr size_t STAGE_SLICE = 2u << 20;   // bytes per ring slot
constexpr int STAGE_SLOTS = 16;            // 32 MB of pinned memory per handle that ever sees a pageable operand
constexpr size_t STAGE_MIN = 4u << 20;     // smaller transfers are not worth the threads

struct HostStage {
  char* ring = nullptr;
  cudaEvent_t ev[STAGE_SLOTS] = {};
  int threads = 1;
};

static int stage_threads() {
  static const int t = [] {
    if (const char* e = getenv("CLA_STAGE_THREADS")) return std::max(0, std::min(32, atoi(e)));
    cpu_set_t set;
    int n = 1;
    if (sched_getaffinity(0, sizeof(set), &set) == 0) n = CPU_COUNT(&set);
    return std::max(1, std::min(6, n / 2));  // the copy rate levels off at four to six threads (measured 1..16)
  }();
  return t;  // 0 switches the staging off
}

bool host_is_pageable(const void* p) {
  cudaPointerAttributes a;
  const cudaError_t e = cudaPointerGetAttributes(&a, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return true;
  }
  return a.type == cudaMemoryTypeUnregistered;
}

static HostStage* stage_of(Matrix* m) {
  if (m->hostStage) return m->hostStage;
  if (stage_threads() == 0) return nullptr;
  auto* st = new HostStage();
  if (cudaHostAlloc((void**)&st->ring, STAGE_SLICE * STAGE_SLOTS, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    delete st;
    return nullptr;  // no pinned memory to be had: the driver's own staging still works
  }
  for (auto& e : st->ev)
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      for (auto& f : st->ev)
        if (f) cudaEventDestroy(f);
      cudaFreeHost(st->ring);
      delete st;
      return nullptr;
    }
  st->threads = stage_threads();
  m->hostStage = st;
  return st;
}

void host_stage_free(Matrix* m) {
  HostStage* st = m->hostStage;
  if (!st) return;
  for (auto& e : st->ev)
    if (e) cudaEventDestroy(e);
  if (st->ring) cudaFreeHost(st->ring);
  delete st;
  m->hostStage = nullptr;
}

bool host_copy_staged(Matrix* m, const void* host, size_t bytes) {
  return bytes >= STAGE_MIN && stage_threads() > 0 && host_is_pageable(host) && stage_of(m) != nullptr;
}

// Shared state of one transfer. Slice j lives in ring slot j % STAGE_SLOTS. `ready[j]`: the workers have filled slice
// j (upload) or the coordinator has recorded the event of its device->host copy (download). `freed[j]`: the slot may
// be reused -- upload: the coordinator has recorded the event of the slice's host->device copy (a worker then waits
// for that event); download: a worker has drained the slice.
struct Transfer {
  size_t n = 0;
  std::unique_ptr<std::atomic<int>[]> ready, freed;
  std::atomic<size_t> next{0};
  std::atomic<bool> abort{false};
  explicit Transfer(size_t slices) : n(slices), ready(new std::atomic<int>[slices]), freed(new std::atomic<int>[slices]) {
    for (size_t i = 0; i < slices; i++) {
      ready[i].store(0);
      freed[i].store(0);
    }
  }
};

static inline bool wait_flag(const std::atomic<int>& f, const std::atomic<bool>& abort) {
  while (!f.load(std::memory_order_acquire)) {
    if (abort.load(std::memory_order_relaxed)) return false;
    std::this_thread::yield();
  }
  return true;
}

// Host -> device. `enqueued(b)` is called (on the calling thread) every time more bytes have been put on `cs`, with
// the number of leading bytes enqueued so far; it may launch work that depends on them. Returns CLA_OK or an error.
int64_t host_to_device_staged(Matrix* m, void* dDst, const void* host, size_t bytes, cudaStream_t cs,
                              const std::function<int64_t(size_t)>& enqueued) {
  HostStage* st = stage_of(m);
  if (!st) return fail(CLA_ERR_STATE, "host staging ring missing");
  const size_t n = (bytes + STAGE_SLICE - 1) / STAGE_SLICE;
  Transfer tr(n);
  const char* src = (const char*)host;
  const int device = m->device;
  auto worker = [&]() {
    cudaSetDevice(device);
    for (;;) {
      const size_t j = tr.next.fetch_add(1);
      if (j >= n || tr.abort.load()) break;
      const int slot = (int)(j % STAGE_SLOTS);
      if (j >= (size_t)STAGE_SLOTS) {  // the slot's previous slice must have left for the device
        if (!wait_flag(tr.freed[j - STAGE_SLOTS], tr.abort)) break;
        if (cudaEventSynchronize(st->ev[slot]) != cudaSuccess) {
          tr.abort.store(true);
          break;
        }
      }
      const size_t off = j * STAGE_SLICE, len = std::min(STAGE_SLICE, bytes - off);
      memcpy(st->ring + (size_t)slot * STAGE_SLICE, src + off, len);
      tr.ready[j].store(1, std::memory_order_release);
    }
  };
  std::vector<std::thread> pool;
  const int nThreads = (int)std::min<size_t>((size_t)st->threads, n);
  for (int t = 0; t < nThreads; t++) pool.emplace_back(worker);
  int64_t rc = CLA_OK;
  for (size_t j = 0; j < n && rc == CLA_OK; j++) {
    if (!wait_flag(tr.ready[j], tr.abort)) {
      rc = fail(CLA_ERR_CUDA, "host staging: a worker failed");
      break;
    }
    const int slot = (int)(j % STAGE_SLOTS);
    const size_t off = j * STAGE_SLICE, len = std::min(STAGE_SLICE, bytes - off);
    cudaError_t e = cudaMemcpyAsync((char*)dDst + off, st->ring + (size_t)slot * STAGE_SLICE, len, cudaMemcpyHostToDevice, cs);
    if (e == cudaSuccess) e = cudaEventRecord(st->ev[slot], cs);
    if (e != cudaSuccess) {
      rc = fail(CLA_ERR_CUDA, std::string("host staging upload: ") + cudaGetErrorString(e));
      break;
    }
    tr.freed[j].store(1, std::memory_order_release);
    if (enqueued) rc = enqueued(off + len);
  }
  if (rc != CLA_OK) tr.abort.store(true);
  for (auto& t : pool) t.join();
  return rc;
}

// Device -> host, after the work already on `s`. Returns when `host` holds the data.
int64_t device_to_host_staged(Matrix* m, void* host, const void* dSrc, size_t bytes, cudaStream_t s) {
  HostStage* st = stage_of(m);
  if (!st) return fail(CLA_ERR_STATE, "host staging ring missing");
  const size_t n = (bytes + STAGE_SLICE - 1) / STAGE_SLICE;
  Transfer tr(n);
  char* dst = (char*)host;
  const int device = m->device;
  auto worker = [&]() {
    cudaSetDevice(device);
    for (;;) {
      const size_t j = tr.next.fetch_add(1);
      if (j >= n || tr.abort.load()) break;
      const int slot = (int)(j % STAGE_SLOTS);
      if (!wait_flag(tr.ready[j], tr.abort)) break;
      if (cudaEventSynchronize(st->ev[slot]) != cudaSuccess) {
        tr.abort.store(true);
        break;
      }
      const size_t off = j * STAGE_SLICE, len = std::min(STAGE_SLICE, bytes - off);
      memcpy(dst + off, st->ring + (size_t)slot * STAGE_SLICE, len);
      tr.freed[j].store(1, std::memory_order_release);
    }
  };
  std::vector<std::thread> pool;
  const int nThreads = (int)std::min<size_t>((size_t)st->threads, n);
  for (int t = 0; t < nThreads; t++) pool.emplace_back(worker);
  int64_t rc = CLA_OK;
  for (size_t j = 0; j < n; j++) {
    const int slot = (int)(j % STAGE_SLOTS);
    if (j >= (size_t)STAGE_SLOTS && !wait_flag(tr.freed[j - STAGE_SLOTS], tr.abort)) {  // the slot has been drained
      rc = fail(CLA_ERR_CUDA, "host staging: a worker failed");
      break;
    }
    const size_t off = j * STAGE_SLICE, len = std::min(STAGE_SLICE, bytes - off);
    cudaError_t e = cudaMemcpyAsync(st->ring + (size_t)slot * STAGE_SLICE, (const char*)dSrc + off, len, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaEventRecord(st->ev[slot], s);
    if (e != cudaSuccess) {
      rc = fail(CLA_ERR_CUDA, std::string("host staging download: ") + cudaGetErrorString(e));
      break;
    }
    tr.ready[j].store(1, std::memory_order_release);
  }
  if (rc != CLA_OK) tr.abort.store(true);
  for (auto& t : pool) t.join();
  if (rc == CLA_OK && tr.abort.load()) rc = fail(CLA_ERR_CUDA, "host staging: a worker failed");
  return rc;
}

}  // namespace cla
