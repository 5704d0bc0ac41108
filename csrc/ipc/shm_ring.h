// Single-producer / single-consumer ring of fixed-size slots living in shared memory.
// Plays the part of the reference's `shmem-ipc` work and completion queues
// (src/ipc/core/src/customer.rs:20-21: depth 32, busy polled). Producer and consumer
// indices sit on separate cache lines; slots are copied by value. The geometry (depth,
// slot size) is kept in the Ring object of each side, never re-read from the shared
// header, so that a peer who scribbles over the header cannot make this side index
// outside the segment; the indices themselves are only ever used modulo the depth.
#pragma once
#include <stdint.h>
#include <string.h>

#include <atomic>

namespace mccs {
namespace ipc {

struct alignas(64) RingHeader {
  std::atomic<uint64_t> head;   // next slot the consumer reads
  uint8_t pad0[56];
  std::atomic<uint64_t> tail;   // next slot the producer writes
  uint8_t pad1[56];
  uint32_t depth;               // power of two
  uint32_t slot_bytes;
  uint8_t pad2[56];
};
static_assert(sizeof(RingHeader) == 192, "ring header layout is part of the ABI");

class Ring {
 public:
  Ring() : hdr_(nullptr), slots_(nullptr), depth_(0), slot_bytes_(0) {}
  // `mem` must be 64-byte aligned and bytes_needed(depth, slot) large.
  static size_t bytes_needed(uint32_t depth, uint32_t slot_bytes) {
    return sizeof(RingHeader) + (size_t)depth * slot_bytes;
  }
  // Creator side: formats the header.
  void init(void* mem, uint32_t depth, uint32_t slot_bytes) {
    hdr_ = reinterpret_cast<RingHeader*>(mem);
    slots_ = reinterpret_cast<uint8_t*>(mem) + sizeof(RingHeader);
    hdr_->head.store(0, std::memory_order_relaxed);
    hdr_->tail.store(0, std::memory_order_relaxed);
    hdr_->depth = depth;
    hdr_->slot_bytes = slot_bytes;
    depth_ = depth;
    slot_bytes_ = slot_bytes;
    std::atomic_thread_fence(std::memory_order_release);
  }
  // Peer side: adopts an already formatted ring (geometry read once, here).
  void attach(void* mem) {
    hdr_ = reinterpret_cast<RingHeader*>(mem);
    slots_ = reinterpret_cast<uint8_t*>(mem) + sizeof(RingHeader);
    depth_ = hdr_->depth;
    slot_bytes_ = hdr_->slot_bytes;
  }
  bool valid() const { return hdr_ != nullptr && depth_ != 0 && (depth_ & (depth_ - 1)) == 0; }
  uint32_t depth() const { return depth_; }
  uint32_t slot_bytes() const { return slot_bytes_; }

  // Producer. Returns false when the ring is full.
  bool try_push(const void* item) {
    const uint64_t t = hdr_->tail.load(std::memory_order_relaxed);
    const uint64_t h = hdr_->head.load(std::memory_order_acquire);
    if (t - h >= depth_) return false;
    memcpy(slots_ + (size_t)(t & (depth_ - 1)) * slot_bytes_, item, slot_bytes_);
    hdr_->tail.store(t + 1, std::memory_order_release);
    return true;
  }
  // Consumer. Returns false when the ring is empty.
  bool try_pop(void* item) {
    const uint64_t h = hdr_->head.load(std::memory_order_relaxed);
    const uint64_t t = hdr_->tail.load(std::memory_order_acquire);
    if (h == t) return false;
    memcpy(item, slots_ + (size_t)(h & (depth_ - 1)) * slot_bytes_, slot_bytes_);
    hdr_->head.store(h + 1, std::memory_order_release);
    return true;
  }
  // Consumer: look at the oldest entry without removing it.
  bool peek(void* item) const {
    const uint64_t h = hdr_->head.load(std::memory_order_relaxed);
    const uint64_t t = hdr_->tail.load(std::memory_order_acquire);
    if (h == t) return false;
    memcpy(item, slots_ + (size_t)(h & (depth_ - 1)) * slot_bytes_, slot_bytes_);
    return true;
  }
  void drop() { hdr_->head.store(hdr_->head.load(std::memory_order_relaxed) + 1, std::memory_order_release); }
  uint64_t size() const {
    return hdr_->tail.load(std::memory_order_acquire) - hdr_->head.load(std::memory_order_acquire);
  }
  bool empty() const { return size() == 0; }

 private:
  RingHeader* hdr_;
  uint8_t* slots_;
  uint32_t depth_;
  uint32_t slot_bytes_;
};

}  // namespace ipc
}  // namespace mccs
