/* knj_residency.h -- CUDA back ends for the three gates the reference's residency
 * state machine drives through injected interfaces (src/residency/residency.h:
 * SlotAllocator :144-172, TransferEngine :174-203, HostArena :205-215). The state
 * machine itself is host code that needs no change; what it lacked on this
 * hardware were implementations of the gates. Names, arguments and meanings of
 * the virtual functions are the reference's, so its ResidencyManager is
 * constructed over these objects unchanged (oracle/ref_residency_check.cpp does
 * exactly that with the reference's residency.cpp).
 *
 * All experts fit in HBM on a B200, so none of this is on the timed path; it
 * exists so that the "experts streamed through a few slots" mode produces the
 * same bits as the resident mode (tests/test_gpu_residency.py).
 */
#ifndef KNJ_RESIDENCY_BACKENDS_H
#define KNJ_RESIDENCY_BACKENDS_H

#include <stdint.h>

#ifdef __cplusplus
#include <memory>

namespace knj {

/* The reference's own header (src/residency/residency.h, include guard KNJ_RESIDENCY_H) declares the same three
 * abstract classes and their enums under the same names. A translation unit that constructs the reference's
 * ResidencyManager over these back ends includes the reference header FIRST (or defines
 * KNJ_HAVE_REFERENCE_RESIDENCY, which makes this header include it by its project-relative path); the
 * declarations below are then skipped and the factories return implementations of the reference's classes. */
#if defined(KNJ_HAVE_REFERENCE_RESIDENCY) && !defined(KNJ_RESIDENCY_H)
#include "src/residency/residency.h"
#endif
#ifndef KNJ_RESIDENCY_H

using SlotHandle = int32_t;
constexpr SlotHandle kNoSlot = -1;

using TransferId = uint64_t;
constexpr TransferId kNoTransfer = 0;
enum class TransferState : uint8_t { PENDING = 0, DONE, FAILED, CANCELLED };
enum class IoClass : uint8_t { DEMAND = 0, PREFETCH = 1 };

/* Asynchronous copies only; every call returns a handle to poll (the CUDA engine keeps the state of the most
 * recent 65536 transfers; older finished ones poll as FAILED, like an unknown id). Demand traffic
 * runs on a higher-priority stream / ahead of queued prefetch work. */
class TransferEngine {
 public:
  virtual ~TransferEngine() = default;
  virtual TransferId submit_nvme_read(void *dst_host, uint64_t src_offset, uint64_t bytes, IoClass io) = 0;
  virtual TransferId submit_nvme_write(const void *src_host, uint64_t dst_offset, uint64_t bytes, IoClass io) = 0;
  virtual TransferId submit_h2d(void *dst_device, const void *src_host, uint64_t bytes, IoClass io) = 0;
  virtual TransferId submit_d2h(void *dst_host, const void *src_device, uint64_t bytes, IoClass io) = 0;
  virtual TransferState poll(TransferId id) const = 0;
  virtual bool cancel(TransferId id) = 0;
};

/* Fixed pool of equal device slots. A slot's copy is "loaded" once the transfers
 * registered for it have finished, and a released slot is reusable only then. */
class SlotAllocator {
 public:
  virtual ~SlotAllocator() = default;
  virtual SlotHandle acquire(uint32_t layer, uint32_t index, uint64_t byte_size) = 0;  /* kNoSlot: no room now */
  virtual void release(SlotHandle slot) = 0;
  virtual bool released(SlotHandle slot) const = 0;
  virtual void pin(SlotHandle slot) = 0;
  virtual void unpin(SlotHandle slot) = 0;
  virtual bool load_event_fired(SlotHandle slot) const = 0;
  virtual void *vram_ptr(SlotHandle slot) const = 0;
  virtual uint64_t byte_size(SlotHandle slot) const = 0;
};

/* Pinned (page-locked) staging memory of the RAM tier. */
class HostArena {
 public:
  virtual ~HostArena() = default;
  virtual void *alloc(uint64_t bytes) = 0;
  virtual void free(void *p) = 0;
};

#endif /* !KNJ_RESIDENCY_H: the interface declarations */

/* The CUDA slot pool additionally learns which transfers read or fill a slot: a slot's load event has fired, and
 * a released slot is reusable, only when all of them have finished. Not synchronised: one host thread drives a
 * pool (the thread that drives the state machine); the engine's worker thread never touches it. */
class CudaSlotAllocator : public SlotAllocator {
 public:
  virtual void watch(SlotHandle slot, const TransferEngine *engine, TransferId id) = 0;
  /* the held or retiring slot that contains device address p, else kNoSlot */
  virtual SlotHandle slot_of(const void *p) const = 0;
};

std::unique_ptr<HostArena> make_cuda_host_arena();
std::unique_ptr<CudaSlotAllocator> make_cuda_slot_allocator(int n_slots, uint64_t slot_bytes);
/* backing_path may be null: then the NVMe calls return kNoTransfer. With `slots`, every device copy whose device
 * side lies in one of the pool's slots registers itself there (watch), which is the bookkeeping the state machine
 * expects from the pool; the pool must outlive the engine's last submit. */
std::unique_ptr<TransferEngine> make_cuda_transfer_engine(const char *backing_path, CudaSlotAllocator *slots = nullptr);

}  // namespace knj

extern "C" {
#endif

/* C view of the same objects (opaque pointers), for hosts without C++. io: 0 demand, 1 prefetch.
 * poll: 0 pending, 1 done, 2 failed, 3 cancelled. */
void *knj_res_arena_create(void);
void *knj_res_arena_alloc(void *arena, uint64_t bytes);
void knj_res_arena_free(void *arena, void *p);
void knj_res_arena_destroy(void *arena);

void *knj_res_slots_create(int n_slots, uint64_t slot_bytes);
int knj_res_slot_acquire(void *slots, uint32_t layer, uint32_t index, uint64_t bytes);
void knj_res_slot_release(void *slots, int slot);
int knj_res_slot_released(void *slots, int slot);
void knj_res_slot_pin(void *slots, int slot);
void knj_res_slot_unpin(void *slots, int slot);
int knj_res_slot_load_fired(void *slots, int slot);
void *knj_res_slot_ptr(void *slots, int slot);
uint64_t knj_res_slot_bytes(void *slots, int slot);
void knj_res_slot_watch(void *slots, int slot, void *engine, uint64_t transfer);
void knj_res_slots_destroy(void *slots);

void *knj_res_engine_create(const char *backing_path);
uint64_t knj_res_submit_nvme_read(void *engine, void *dst_host, uint64_t src_offset, uint64_t bytes, int io);
uint64_t knj_res_submit_nvme_write(void *engine, const void *src_host, uint64_t dst_offset, uint64_t bytes, int io);
uint64_t knj_res_submit_h2d(void *engine, void *dst_device, const void *src_host, uint64_t bytes, int io);
uint64_t knj_res_submit_d2h(void *engine, void *dst_host, const void *src_device, uint64_t bytes, int io);
int knj_res_poll(void *engine, uint64_t transfer);
int knj_res_cancel(void *engine, uint64_t transfer);
/* Work enqueued on `stream` after this call starts only when the device copy `transfer` has finished. */
int knj_res_wait_on_stream(void *engine, uint64_t transfer, void *stream);
void knj_res_engine_destroy(void *engine);

#ifdef __cplusplus
}
#endif
#endif /* KNJ_RESIDENCY_BACKENDS_H */
