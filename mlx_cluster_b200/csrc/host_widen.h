// Host half of the narrow transport used by the host-buffer entry points: walk matrices whose
// ids fit 32 bits cross PCIe as int32 and are widened to the caller's int64 buffer by a small
// pool of host threads, which halves the bytes on the bus.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <mutex>
#include <thread>
#include <vector>

namespace walk_b200 {

// dst[i] = (int64_t)src[i] for i in [0, count). Uses AVX2 non-temporal stores when the CPU has them.
void widen_i32_to_i64(const int32_t* src, int64_t* dst, int64_t count);

// Fixed set of worker threads; widen() splits one array into equal contiguous pieces, one per
// worker plus one for the calling thread, and returns when all pieces are written.
class WidenPool {
 public:
  explicit WidenPool(int workers);
  ~WidenPool();
  WidenPool(const WidenPool&) = delete;
  WidenPool& operator=(const WidenPool&) = delete;
  void widen(const int32_t* src, int64_t* dst, int64_t count);
  int workers() const { return (int)threads_.size(); }

 private:
  void worker_main(int index);
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_job_, cv_done_;
  uint64_t generation_ = 0;
  int finished_ = 0;
  bool stop_ = false;
  const int32_t* src_ = nullptr;
  int64_t* dst_ = nullptr;
  int64_t count_ = 0;
};

}  // namespace walk_b200
