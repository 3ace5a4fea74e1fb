// Minimal stand-in for the parts of the MLX C++ API that the reference's two
// walk primitives touch. Test infrastructure only: it lets the reference's own
// RandomWalk.cpp / BiasedRandomWalk.cpp be compiled unmodified on Linux so that
// their eval_cpu loops can serve as the parity oracle and the CPU baseline.
// Storage and scheduling only; no walk arithmetic lives here.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <memory>
#include <ostream>
#include <stdexcept>
#include <utility>
#include <vector>

namespace mlx::core {

struct Dtype {
  enum Kind { int32, int64, float32 } kind;
  bool operator==(const Dtype& o) const { return kind == o.kind; }
};
static constexpr Dtype int64{Dtype::int64};
static constexpr Dtype float32{Dtype::float32};

struct Device {
  enum Type { cpu, gpu } type = cpu;
  int index = 0;
};
struct Stream {
  int index = 0;
  Device device{};
};
struct StreamOrDevice {
  Stream stream{};
  StreamOrDevice() = default;
  StreamOrDevice(Stream s) : stream(s) {}
};
inline Stream to_stream(StreamOrDevice s) { return s.stream; }

namespace allocator {
struct Buffer {
  void* ptr = nullptr;
  bool owned = false;
};
inline Buffer malloc_or_wait(size_t nbytes) {
  return Buffer{std::malloc(nbytes ? nbytes : 1), true};
}
}  // namespace allocator

class Primitive;

class array {
 public:
  array() : st_(std::make_shared<State>()) {}
  // Borrow caller memory (inputs).
  array(void* data, size_t size, Dtype dtype) : st_(std::make_shared<State>()) {
    st_->buf.ptr = data;
    st_->buf.owned = false;
    st_->size = size;
    st_->dtype = dtype;
  }
  array(std::vector<int> shape, Dtype dtype) : st_(std::make_shared<State>()) {
    size_t s = 1;
    for (int d : shape) s *= static_cast<size_t>(d);
    st_->size = s;
    st_->dtype = dtype;
    st_->shape = std::move(shape);
  }
  size_t size() const { return st_->size; }
  Dtype dtype() const { return st_->dtype; }
  const std::vector<int>& shape() const { return st_->shape; }
  void set_data(allocator::Buffer b) {
    st_->release();
    st_->buf = b;
  }
  template <typename T>
  T* data() { return static_cast<T*>(st_->buf.ptr); }
  template <typename T>
  const T* data() const { return static_cast<const T*>(st_->buf.ptr); }

  static std::vector<array> make_arrays(
      std::vector<std::vector<int>> shapes,
      const std::vector<Dtype>& dtypes,
      const std::shared_ptr<Primitive>& primitive,
      const std::vector<array>& inputs) {
    std::vector<array> outs;
    for (size_t i = 0; i < shapes.size(); i++) {
      array a(shapes[i], dtypes[i]);
      a.st_->primitive = primitive;
      a.st_->inputs = inputs;
      outs.push_back(a);
    }
    return outs;
  }
  std::shared_ptr<Primitive> primitive() const { return st_->primitive; }
  const std::vector<array>& inputs() const { return st_->inputs; }

 private:
  struct State {
    allocator::Buffer buf{};
    size_t size = 0;
    Dtype dtype{Dtype::int64};
    std::vector<int> shape;
    std::shared_ptr<Primitive> primitive;
    std::vector<array> inputs;
    void release() {
      if (buf.owned && buf.ptr) std::free(buf.ptr);
      buf = allocator::Buffer{};
    }
    ~State() { release(); }
  };
  std::shared_ptr<State> st_;
};

}  // namespace mlx::core
