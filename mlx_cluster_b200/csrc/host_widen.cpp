// Host threads that widen int32 walk matrices, landed in pinned staging memory, into the
// caller's int64 buffers. See host_widen.h.
#include "host_widen.h"

#include <immintrin.h>

namespace walk_b200 {

namespace {

constexpr int64_t kStreamingMin = 1 << 15;  // below this many elements plain stores keep the data in cache

void widen_scalar(const int32_t* src, int64_t* dst, int64_t count) {
  for (int64_t i = 0; i < count; i++) dst[i] = src[i];
}

#if defined(__x86_64__)
__attribute__((target("avx2"))) void widen_avx2(const int32_t* src, int64_t* dst, int64_t count) {
  int64_t i = 0;
  while (i < count && (reinterpret_cast<uintptr_t>(dst + i) & 31)) {
    dst[i] = src[i];
    i++;
  }
  for (; i + 8 <= count; i += 8) {
    const __m128i lo = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i));
    const __m128i hi = _mm_loadu_si128(reinterpret_cast<const __m128i*>(src + i + 4));
    _mm256_stream_si256(reinterpret_cast<__m256i*>(dst + i), _mm256_cvtepi32_epi64(lo));
    _mm256_stream_si256(reinterpret_cast<__m256i*>(dst + i + 4), _mm256_cvtepi32_epi64(hi));
  }
  for (; i < count; i++) dst[i] = src[i];
  _mm_sfence();
}
#endif

// piece k of `parts` equal pieces of [0, count), cut at multiples of 8 elements
void piece_bounds(int64_t count, int parts, int k, int64_t* b, int64_t* e) {
  const int64_t per = ((count + parts - 1) / parts + 7) & ~int64_t(7);
  *b = per * k < count ? per * k : count;
  *e = per * (k + 1) < count ? per * (k + 1) : count;
}

}  // namespace

void widen_i32_to_i64(const int32_t* src, int64_t* dst, int64_t count) {
#if defined(__x86_64__)
  static const bool have_avx2 = __builtin_cpu_supports("avx2");
  if (have_avx2 && count >= kStreamingMin) {
    widen_avx2(src, dst, count);
    return;
  }
#endif
  widen_scalar(src, dst, count);
}

WidenPool::WidenPool(int workers) {
  if (workers < 0) workers = 0;
  threads_.reserve(workers);
  for (int k = 0; k < workers; k++) threads_.emplace_back([this, k] { worker_main(k); });
}

WidenPool::~WidenPool() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_ = true;
  }
  cv_job_.notify_all();
  for (auto& t : threads_) t.join();
}

void WidenPool::worker_main(int index) {
  uint64_t seen = 0;
  for (;;) {
    const int32_t* src;
    int64_t* dst;
    int64_t count;
    {
      std::unique_lock<std::mutex> lock(mu_);
      cv_job_.wait(lock, [&] { return stop_ || generation_ != seen; });
      if (stop_) return;
      seen = generation_;
      src = src_; dst = dst_; count = count_;
    }
    int64_t b, e;
    piece_bounds(count, (int)threads_.size() + 1, index, &b, &e);
    if (e > b) widen_i32_to_i64(src + b, dst + b, e - b);
    {
      std::lock_guard<std::mutex> lock(mu_);
      finished_++;
    }
    cv_done_.notify_one();
  }
}

void WidenPool::widen(const int32_t* src, int64_t* dst, int64_t count) {
  if (count <= 0) return;
  const int workers = (int)threads_.size();
  if (workers == 0 || count < 4 * kStreamingMin) {
    widen_i32_to_i64(src, dst, count);
    return;
  }
  {
    std::lock_guard<std::mutex> lock(mu_);
    src_ = src; dst_ = dst; count_ = count;
    finished_ = 0;
    generation_++;
  }
  cv_job_.notify_all();
  int64_t b, e;
  piece_bounds(count, workers + 1, workers, &b, &e);  // the calling thread takes the last piece
  if (e > b) widen_i32_to_i64(src + b, dst + b, e - b);
  std::unique_lock<std::mutex> lock(mu_);
  cv_done_.wait(lock, [&] { return finished_ == workers; });
}

}  // namespace walk_b200
