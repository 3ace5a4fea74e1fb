// Stand-in for mlx/primitives.h: the abstract node type the reference subclasses.
#pragma once
#include "mlx/array.h"

namespace mlx::core {

class Primitive {
 public:
  explicit Primitive(Stream stream) : stream_(stream) {}
  virtual ~Primitive() = default;
  const Stream& stream() { return stream_; }
  virtual void eval_cpu(const std::vector<array>& inputs, std::vector<array>& outputs) = 0;
  virtual void eval_gpu(const std::vector<array>& inputs, std::vector<array>& outputs) = 0;
  virtual std::vector<array> jvp(
      const std::vector<array>& primals,
      const std::vector<array>& tangents,
      const std::vector<int>& argnums) = 0;
  virtual std::vector<array> vjp(
      const std::vector<array>& primals,
      const std::vector<array>& cotangents,
      const std::vector<int>& argnums,
      const std::vector<array>& outputs) = 0;
  virtual std::pair<std::vector<array>, std::vector<int>> vmap(
      const std::vector<array>& inputs,
      const std::vector<int>& axes) = 0;
  virtual void print(std::ostream& os) = 0;
  virtual bool is_equivalent(const Primitive& other) const = 0;
  virtual std::vector<std::vector<int>> output_shapes(const std::vector<array>& inputs) = 0;

 private:
  Stream stream_;
};

}  // namespace mlx::core
