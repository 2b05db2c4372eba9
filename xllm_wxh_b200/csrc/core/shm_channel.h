// Single-writer / multi-reader broadcast channel in POSIX shared memory.
//
// Carries the packed step inputs from the scheduler process to the rank processes on the
// same host (and small results back through a second channel).  The design follows the
// reference's version-stamped shared-memory buffer polled by the workers
// (xllm/core/runtime/forward_shared_memory_manager.h:32-100,
//  xllm/core/distributed_runtime/shm_channel.cpp): the writer bumps a sequence number
// after the payload is in place; each reader acknowledges the sequence it consumed, and
// the writer does not overwrite before every reader has acknowledged.  Every wait has a
// timeout so that a dead peer shows up as an error code instead of a hang.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>

namespace xl {

class ShmChannel {
 public:
  static constexpr int kMaxReaders = 64;
  struct Header {
    std::atomic<uint64_t> seq;
    std::atomic<uint64_t> size;
    std::atomic<uint64_t> closed;
    uint64_t capacity;
    std::atomic<uint64_t> acks[kMaxReaders];
  };

  ShmChannel(const std::string& name, size_t capacity_bytes, int num_readers, bool create)
      : name_(name), capacity_(capacity_bytes), readers_(num_readers), owner_(create) {
    if (num_readers < 1 || num_readers > kMaxReaders) throw std::invalid_argument("ShmChannel: bad reader count");
    total_ = sizeof(Header) + capacity_;
    int fd = -1;
    if (create) {
      shm_unlink(name.c_str());
      fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
      if (fd < 0) throw std::runtime_error("shm_open(create) failed for " + name);
      if (ftruncate(fd, static_cast<off_t>(total_)) != 0) {
        ::close(fd);
        throw std::runtime_error("ftruncate failed for " + name);
      }
    } else {
      // the creator may not be up yet: retry for a bounded time
      for (int i = 0; i < 3000 && fd < 0; ++i) {
        fd = shm_open(name.c_str(), O_RDWR, 0600);
        if (fd >= 0) {
          struct stat st;
          if (fstat(fd, &st) == 0 && static_cast<size_t>(st.st_size) >= total_) break;
          ::close(fd);
          fd = -1;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
      }
      if (fd < 0) throw std::runtime_error("shm_open(attach) timed out for " + name);
    }
    void* p = mmap(nullptr, total_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) throw std::runtime_error("mmap failed for " + name);
    hdr_ = static_cast<Header*>(p);
    payload_ = reinterpret_cast<uint8_t*>(p) + sizeof(Header);
    if (create) {
      hdr_->seq.store(0);
      hdr_->size.store(0);
      hdr_->closed.store(0);
      hdr_->capacity = capacity_;
      for (int i = 0; i < kMaxReaders; ++i) hdr_->acks[i].store(0);
    }
    for (int i = 0; i < kMaxReaders; ++i) local_seq_[i] = 0;
  }
  ~ShmChannel() {
    if (hdr_) munmap(hdr_, total_);
    if (owner_) shm_unlink(name_.c_str());
  }

  // 0 ok, 1 timeout (a reader did not acknowledge), 2 too large, 3 closed
  int write(const void* data, size_t n, double timeout_s) {
    if (n > capacity_) return 2;
    if (hdr_->closed.load(std::memory_order_acquire)) return 3;
    const uint64_t cur = hdr_->seq.load(std::memory_order_acquire);
    if (!wait([&] {
          for (int r = 0; r < readers_; ++r)
            if (hdr_->acks[r].load(std::memory_order_acquire) < cur) return false;
          return true;
        }, timeout_s))
      return hdr_->closed.load() ? 3 : 1;
    std::memcpy(payload_, data, n);
    hdr_->size.store(n, std::memory_order_relaxed);
    hdr_->seq.store(cur + 1, std::memory_order_release);
    return 0;
  }

  // 0 ok, 1 timeout, 2 destination too small, 3 closed
  int read_into(int reader, void* dst, size_t cap, double timeout_s, size_t* got = nullptr) {
    if (reader < 0 || reader >= readers_) return 2;
    const uint64_t want = local_seq_[reader] + 1;
    if (!wait([&] { return hdr_->seq.load(std::memory_order_acquire) >= want; }, timeout_s))
      return hdr_->closed.load() ? 3 : 1;
    size_t n = hdr_->size.load(std::memory_order_relaxed);
    if (n > cap) return 2;
    std::memcpy(dst, payload_, n);
    if (got) *got = n;
    local_seq_[reader] = want;
    hdr_->acks[reader].store(want, std::memory_order_release);
    return static_cast<int>(0);
  }
  int read(int reader, std::string& out, double timeout_s) {
    if (reader < 0 || reader >= readers_) return 2;
    const uint64_t want = local_seq_[reader] + 1;
    if (!wait([&] { return hdr_->seq.load(std::memory_order_acquire) >= want; }, timeout_s))
      return hdr_->closed.load() ? 3 : 1;
    size_t n = hdr_->size.load(std::memory_order_relaxed);
    out.assign(reinterpret_cast<const char*>(payload_), n);
    local_seq_[reader] = want;
    hdr_->acks[reader].store(want, std::memory_order_release);
    return 0;
  }
  void close() { hdr_->closed.store(1, std::memory_order_release); }
  static void unlink(const std::string& name) { shm_unlink(name.c_str()); }

 private:
  template <class Pred>
  bool wait(Pred&& ready, double timeout_s) {
    using clock = std::chrono::steady_clock;
    const auto deadline = clock::now() + std::chrono::duration<double>(timeout_s);
    int spins = 0;
    while (!ready()) {
      if (hdr_->closed.load(std::memory_order_acquire)) return false;
      if (++spins < 2000) {
#if defined(__x86_64__)
        __builtin_ia32_pause();
#endif
      } else {
        if (clock::now() > deadline) return false;
        std::this_thread::sleep_for(std::chrono::microseconds(spins < 20000 ? 1 : 50));
      }
    }
    return true;
  }

  std::string name_;
  size_t capacity_, total_ = 0;
  int readers_;
  bool owner_;
  Header* hdr_ = nullptr;
  uint8_t* payload_ = nullptr;
  uint64_t local_seq_[kMaxReaders];
};

}  // namespace xl
