// knj_residency.cu -- CUDA implementations of the residency gates declared in
// include/knj_residency.h (the reference's SlotAllocator / TransferEngine /
// HostArena, src/residency/residency.h:144-215; its HIP models are the fixed slot
// pool and the copy-stream engine of tools/bench/q4k_stream_ffn.hip:219-674).
//
// Slot pool: one device allocation cut into equal slots; a slot is "loaded" when
// every transfer registered for it has finished and a released slot returns to
// the free list only then. Transfer engine: device copies go out immediately on
// one of two non-blocking streams (demand at the higher priority) with an event
// each; file reads and writes are done by one worker thread that always serves
// the demand queue first. Nothing here blocks the caller.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <iterator>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "knj_residency.h"

namespace knj {
namespace {

class CudaHostArena final : public HostArena {
 public:
  void *alloc(uint64_t bytes) override {
    void *p = nullptr;
    if (bytes == 0 || cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return p;
  }
  void free(void *p) override {
    if (p) cudaFreeHost(p);
  }
};

class SlotPool final : public CudaSlotAllocator {
 public:
  SlotPool(int n, uint64_t bytes) : slot_bytes_(bytes), slots_(n) {
    if (n > 0 && bytes > 0 && cudaMalloc(&base_, (size_t)n * bytes) != cudaSuccess) {
      cudaGetLastError();
      base_ = nullptr;
    }
  }
  ~SlotPool() override {
    if (base_) cudaFree(base_);
  }
  SlotHandle acquire(uint32_t layer, uint32_t index, uint64_t byte_size) override {
    if (!base_ || byte_size > slot_bytes_) return kNoSlot;
    reap();
    for (size_t i = 0; i < slots_.size(); ++i) {
      Slot &s = slots_[i];
      if (s.state == kFree) {
        s = Slot{};
        s.state = kHeld;
        s.layer = layer;
        s.index = index;
        s.bytes = byte_size;
        return (SlotHandle)i;
      }
    }
    return kNoSlot;
  }
  void release(SlotHandle h) override {
    if (!valid(h) || slots_[h].state != kHeld || slots_[h].pins > 0) return;
    slots_[h].state = kRetiring;
    reap();
  }
  bool released(SlotHandle h) const override {
    if (!valid(h)) return true;
    const_cast<SlotPool *>(this)->reap();
    return slots_[h].state == kFree;
  }
  void pin(SlotHandle h) override {
    if (valid(h) && slots_[h].state == kHeld) ++slots_[h].pins;
  }
  void unpin(SlotHandle h) override {
    if (valid(h) && slots_[h].pins > 0) --slots_[h].pins;
  }
  bool load_event_fired(SlotHandle h) const override {
    if (!valid(h) || slots_[h].state != kHeld) return false;
    return transfers_done(slots_[h]);
  }
  void *vram_ptr(SlotHandle h) const override {
    return valid(h) && slots_[h].state != kFree ? static_cast<char *>(base_) + (size_t)h * slot_bytes_ : nullptr;
  }
  uint64_t byte_size(SlotHandle h) const override { return valid(h) ? slots_[h].bytes : 0; }
  void watch(SlotHandle h, const TransferEngine *engine, TransferId id) override {
    if (valid(h) && engine && id != kNoTransfer) slots_[h].loads.push_back({engine, id});
  }
  SlotHandle slot_of(const void *p) const override {
    if (!base_ || !p || slot_bytes_ == 0) return kNoSlot;
    const char *c = static_cast<const char *>(p), *b = static_cast<const char *>(base_);
    if (c < b || c >= b + slots_.size() * slot_bytes_) return kNoSlot;
    const SlotHandle h = (SlotHandle)((c - b) / slot_bytes_);
    return slots_[h].state != kFree ? h : kNoSlot;
  }

 private:
  enum State { kFree, kHeld, kRetiring };
  struct Load {
    const TransferEngine *engine;
    TransferId id;
  };
  struct Slot {
    State state = kFree;
    uint32_t layer = 0, index = 0;
    uint64_t bytes = 0;
    int pins = 0;
    std::vector<Load> loads;
  };
  bool valid(SlotHandle h) const { return h >= 0 && (size_t)h < slots_.size(); }
  static bool transfers_done(const Slot &s) {
    for (const Load &l : s.loads)
      if (l.engine->poll(l.id) == TransferState::PENDING) return false;
    return true;
  }
  // retiring slots whose transfers have all finished become free
  void reap() {
    for (Slot &s : slots_)
      if (s.state == kRetiring && transfers_done(s)) s = Slot{};
  }
  void *base_ = nullptr;
  uint64_t slot_bytes_;
  std::vector<Slot> slots_;
};

class CopyEngine final : public TransferEngine {
 public:
  explicit CopyEngine(const char *path, CudaSlotAllocator *slots = nullptr) : slots_(slots) {
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);  // hi is the numerically smallest = most urgent
    ok_ = cudaStreamCreateWithPriority(&demand_, cudaStreamNonBlocking, hi) == cudaSuccess &&
          cudaStreamCreateWithPriority(&prefetch_, cudaStreamNonBlocking, lo) == cudaSuccess;
    if (!ok_) cudaGetLastError();
    if (path) fd_ = ::open(path, O_RDWR);
    worker_ = std::thread([this] { run(); });
  }
  ~CopyEngine() override {
    {
      std::lock_guard<std::mutex> g(m_);
      stop_ = true;
    }
    cv_.notify_all();
    worker_.join();
    if (ok_) {
      cudaStreamSynchronize(demand_);
      cudaStreamSynchronize(prefetch_);
    }
    for (auto &kv : dev_) cudaEventDestroy(kv.second);
    if (ok_) {
      cudaStreamDestroy(demand_);
      cudaStreamDestroy(prefetch_);
    }
    if (fd_ >= 0) ::close(fd_);
  }
  TransferId submit_nvme_read(void *dst, uint64_t off, uint64_t bytes, IoClass io) override {
    return fd_ >= 0 && dst ? enqueue_file({false, dst, nullptr, off, bytes}, io) : kNoTransfer;
  }
  TransferId submit_nvme_write(const void *src, uint64_t off, uint64_t bytes, IoClass io) override {
    return fd_ >= 0 && src ? enqueue_file({true, nullptr, src, off, bytes}, io) : kNoTransfer;
  }
  TransferId submit_h2d(void *dst, const void *src, uint64_t bytes, IoClass io) override {
    return note(dst, device_copy(dst, src, bytes, cudaMemcpyHostToDevice, io));
  }
  TransferId submit_d2h(void *dst, const void *src, uint64_t bytes, IoClass io) override {
    return note(src, device_copy(dst, src, bytes, cudaMemcpyDeviceToHost, io));
  }
  TransferState poll(TransferId id) const override {
    std::lock_guard<std::mutex> g(m_);
    auto d = dev_.find(id);
    if (d != dev_.end()) {
      const cudaError_t e = cudaEventQuery(d->second);
      if (e == cudaSuccess) {  // finished copies keep only their state, not their event
        cudaEventDestroy(d->second);
        dev_.erase(d);
        file_[id] = TransferState::DONE;
        return TransferState::DONE;
      }
      if (e == cudaErrorNotReady) return TransferState::PENDING;
      cudaGetLastError();
      return TransferState::FAILED;
    }
    auto f = file_.find(id);
    return f == file_.end() ? TransferState::FAILED : f->second;
  }
  bool cancel(TransferId id) override {  // only file work that has not started can still be withdrawn
    std::lock_guard<std::mutex> g(m_);
    for (std::deque<Job> *q : {&q_demand_, &q_prefetch_})
      for (auto it = q->begin(); it != q->end(); ++it)
        if (it->id == id) {
          q->erase(it);
          file_[id] = TransferState::CANCELLED;
          return true;
        }
    return false;
  }
  // work enqueued on `s` afterwards waits for the device copy `id`
  bool wait_on_stream(TransferId id, cudaStream_t s) {
    std::lock_guard<std::mutex> g(m_);
    auto d = dev_.find(id);
    if (d != dev_.end()) return cudaStreamWaitEvent(s, d->second, 0) == cudaSuccess;
    auto f = file_.find(id);  // a copy already seen finished needs no wait
    return f != file_.end() && f->second == TransferState::DONE;
  }

 private:
  struct FileOp {
    bool write;
    void *dst;
    const void *src;
    uint64_t off, bytes;
  };
  struct Job {
    TransferId id;
    FileOp op;
  };
  // a copy whose device side lies in a slot of the bound pool is registered with that slot
  TransferId note(const void *dev, TransferId id) {
    if (slots_ && id != kNoTransfer) {
      const SlotHandle h = slots_->slot_of(dev);
      if (h != kNoSlot) slots_->watch(h, this, id);
    }
    return id;
  }
  CudaSlotAllocator *slots_ = nullptr;
  TransferId device_copy(void *dst, const void *src, uint64_t bytes, cudaMemcpyKind kind, IoClass io) {
    if (!ok_ || !dst || !src) return kNoTransfer;
    cudaStream_t st = io == IoClass::DEMAND ? demand_ : prefetch_;
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaMemcpyAsync(dst, src, bytes, kind, st) != cudaSuccess || cudaEventRecord(ev, st) != cudaSuccess) {
      cudaGetLastError();
      if (ev) cudaEventDestroy(ev);
      return kNoTransfer;
    }
    std::lock_guard<std::mutex> g(m_);
    const TransferId id = next_++;
    dev_[id] = ev;
    forget_old(id);
    return id;
  }
  // States are kept for the most recent kKept transfers: finished ones older than that are forgotten (a poll of
  // them answers FAILED, as for an id never handed out), so a long run does not grow the tables. Called locked.
  static constexpr TransferId kKept = 1u << 16;
  void forget_old(TransferId newest) {
    if ((newest & 0xfffu) != 0 || newest <= kKept) return;
    const TransferId limit = newest - kKept;
    for (auto it = file_.begin(); it != file_.end();)
      it = (it->first < limit && it->second != TransferState::PENDING) ? file_.erase(it) : std::next(it);
    for (auto it = dev_.begin(); it != dev_.end();) {
      if (it->first < limit && cudaEventQuery(it->second) == cudaSuccess) {
        cudaEventDestroy(it->second);
        it = dev_.erase(it);
      } else {
        ++it;
      }
    }
  }
  TransferId enqueue_file(FileOp op, IoClass io) {
    std::lock_guard<std::mutex> g(m_);
    const TransferId id = next_++;
    forget_old(id);
    file_[id] = TransferState::PENDING;
    (io == IoClass::DEMAND ? q_demand_ : q_prefetch_).push_back({id, op});
    cv_.notify_one();
    return id;
  }
  void run() {
    for (;;) {
      Job job;
      {
        std::unique_lock<std::mutex> g(m_);
        cv_.wait(g, [this] { return stop_ || !q_demand_.empty() || !q_prefetch_.empty(); });
        if (q_demand_.empty() && q_prefetch_.empty()) return;  // stop requested and nothing left
        std::deque<Job> &q = !q_demand_.empty() ? q_demand_ : q_prefetch_;  // demand first, always
        job = q.front();
        q.pop_front();
      }
      bool good = true;
      uint64_t done = 0;
      while (good && done < job.op.bytes) {
        const ssize_t n = job.op.write
                              ? ::pwrite(fd_, static_cast<const char *>(job.op.src) + done, job.op.bytes - done, (off_t)(job.op.off + done))
                              : ::pread(fd_, static_cast<char *>(job.op.dst) + done, job.op.bytes - done, (off_t)(job.op.off + done));
        if (n <= 0) good = false;
        else done += (uint64_t)n;
      }
      std::lock_guard<std::mutex> g(m_);
      file_[job.id] = good ? TransferState::DONE : TransferState::FAILED;
    }
  }

  bool ok_ = false;
  cudaStream_t demand_ = nullptr, prefetch_ = nullptr;
  int fd_ = -1;
  mutable std::mutex m_;
  std::condition_variable cv_;
  bool stop_ = false;
  TransferId next_ = 1;
  mutable std::unordered_map<TransferId, cudaEvent_t> dev_;
  mutable std::unordered_map<TransferId, TransferState> file_;
  std::deque<Job> q_demand_, q_prefetch_;
  std::thread worker_;

  friend int ::knj_res_wait_on_stream(void *, uint64_t, void *);
};

}  // namespace

std::unique_ptr<HostArena> make_cuda_host_arena() { return std::unique_ptr<HostArena>(new CudaHostArena()); }
std::unique_ptr<CudaSlotAllocator> make_cuda_slot_allocator(int n_slots, uint64_t slot_bytes) {
  return std::unique_ptr<CudaSlotAllocator>(new SlotPool(n_slots, slot_bytes));
}
std::unique_ptr<TransferEngine> make_cuda_transfer_engine(const char *backing_path, CudaSlotAllocator *slots) {
  return std::unique_ptr<TransferEngine>(new CopyEngine(backing_path, slots));
}

}  // namespace knj

using namespace knj;

extern "C" {

void *knj_res_arena_create(void) { return make_cuda_host_arena().release(); }
void *knj_res_arena_alloc(void *a, uint64_t bytes) { return a ? static_cast<HostArena *>(a)->alloc(bytes) : nullptr; }
void knj_res_arena_free(void *a, void *p) { if (a) static_cast<HostArena *>(a)->free(p); }
void knj_res_arena_destroy(void *a) { delete static_cast<HostArena *>(a); }

void *knj_res_slots_create(int n, uint64_t bytes) { return make_cuda_slot_allocator(n, bytes).release(); }
int knj_res_slot_acquire(void *s, uint32_t layer, uint32_t index, uint64_t bytes) {
  return s ? static_cast<CudaSlotAllocator *>(s)->acquire(layer, index, bytes) : kNoSlot;
}
void knj_res_slot_release(void *s, int h) { if (s) static_cast<CudaSlotAllocator *>(s)->release(h); }
int knj_res_slot_released(void *s, int h) { return s && static_cast<CudaSlotAllocator *>(s)->released(h) ? 1 : 0; }
void knj_res_slot_pin(void *s, int h) { if (s) static_cast<CudaSlotAllocator *>(s)->pin(h); }
void knj_res_slot_unpin(void *s, int h) { if (s) static_cast<CudaSlotAllocator *>(s)->unpin(h); }
int knj_res_slot_load_fired(void *s, int h) { return s && static_cast<CudaSlotAllocator *>(s)->load_event_fired(h) ? 1 : 0; }
void *knj_res_slot_ptr(void *s, int h) { return s ? static_cast<CudaSlotAllocator *>(s)->vram_ptr(h) : nullptr; }
uint64_t knj_res_slot_bytes(void *s, int h) { return s ? static_cast<CudaSlotAllocator *>(s)->byte_size(h) : 0; }
void knj_res_slot_watch(void *s, int h, void *engine, uint64_t id) {
  if (s) static_cast<CudaSlotAllocator *>(s)->watch(h, static_cast<TransferEngine *>(engine), id);
}
void knj_res_slots_destroy(void *s) { delete static_cast<CudaSlotAllocator *>(s); }

void *knj_res_engine_create(const char *path) { return make_cuda_transfer_engine(path).release(); }
uint64_t knj_res_submit_nvme_read(void *e, void *dst, uint64_t off, uint64_t bytes, int io) {
  return e ? static_cast<TransferEngine *>(e)->submit_nvme_read(dst, off, bytes, io ? IoClass::PREFETCH : IoClass::DEMAND) : 0;
}
uint64_t knj_res_submit_nvme_write(void *e, const void *src, uint64_t off, uint64_t bytes, int io) {
  return e ? static_cast<TransferEngine *>(e)->submit_nvme_write(src, off, bytes, io ? IoClass::PREFETCH : IoClass::DEMAND) : 0;
}
uint64_t knj_res_submit_h2d(void *e, void *dst, const void *src, uint64_t bytes, int io) {
  return e ? static_cast<TransferEngine *>(e)->submit_h2d(dst, src, bytes, io ? IoClass::PREFETCH : IoClass::DEMAND) : 0;
}
uint64_t knj_res_submit_d2h(void *e, void *dst, const void *src, uint64_t bytes, int io) {
  return e ? static_cast<TransferEngine *>(e)->submit_d2h(dst, src, bytes, io ? IoClass::PREFETCH : IoClass::DEMAND) : 0;
}
int knj_res_poll(void *e, uint64_t id) { return e ? (int)static_cast<TransferEngine *>(e)->poll(id) : 2; }
int knj_res_cancel(void *e, uint64_t id) { return e && static_cast<TransferEngine *>(e)->cancel(id) ? 1 : 0; }
int knj_res_wait_on_stream(void *e, uint64_t id, void *stream) {
  if (!e) return -1;
  return static_cast<CopyEngine *>(static_cast<TransferEngine *>(e))->wait_on_stream(id, static_cast<cudaStream_t>(stream)) ? 0 : -1;
}
void knj_res_engine_destroy(void *e) { delete static_cast<TransferEngine *>(e); }

}  // extern "C"
