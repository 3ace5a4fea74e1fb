// Test infrastructure, not product code.
//
// C entry points around the reference's own eval_cpu loops
// (random_walks/RandomWalk.cpp:18-62 and random_walks/BiasedRandomWalk.cpp:30-102),
// which are compiled UNMODIFIED from the reference checkout against the header
// stand-ins in mlx_stub/. Nothing here computes a walk: the harness wraps caller
// buffers as arrays, calls eval_cpu, times that call alone and copies the two
// outputs back.
//
// Two holes of the reference on a non-Metal build are papered over here:
//  * RandomWalk::eval_gpu is declared (random_walks/RandomWalk.h:15-16) but only
//    defined under _METAL_ (random_walks/RandomWalk.cpp:72-109); the vtable needs
//    a definition, so one that throws is supplied.
//  * BiasedRandomWalk::eval_cpu binds inputs[3] (random_walks/BiasedRandomWalk.cpp:34,50)
//    although its factory passes three inputs (:191); a dummy fourth array is
//    passed so that the vector access stays in range. Its value is never used.
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <vector>

#include "random_walks/BiasedRandomWalk.h"
#include "random_walks/RandomWalk.h"

namespace mlx::core {
void RandomWalk::eval_gpu(const std::vector<array>&, std::vector<array>&) {
  throw std::runtime_error("RandomWalk::eval_gpu: no Metal on this build");
}
}  // namespace mlx::core

namespace {
using namespace mlx::core;

struct CoutSilencer {
  // The reference prints progress lines to std::cout inside the op path
  // (random_walks/RandomWalk.cpp:40,140); keep test logs clean.
  std::streambuf* saved;
  CoutSilencer() : saved(std::cout.rdbuf(nullptr)) {}
  ~CoutSilencer() {
    std::cout.rdbuf(saved);
    std::cout.clear();
  }
};

double now_s() {
  using clk = std::chrono::steady_clock;
  return std::chrono::duration<double>(clk::now().time_since_epoch()).count();
}
}  // namespace

extern "C" {

// Runs RandomWalk::eval_cpu. n_out: [n, L+1], e_out: [n, L] (either may be NULL).
// Returns the seconds spent inside eval_cpu (output malloc included, as in the reference).
double ref_random_walk(const int64_t* rowptr, int64_t n_rowptr, const int64_t* col, int64_t nnz,
                       const int64_t* start, int64_t n, const float* rand, int walk_length,
                       int64_t* n_out, int64_t* e_out) {
  CoutSilencer quiet;
  std::vector<array> inputs = {
      array(const_cast<int64_t*>(rowptr), (size_t)n_rowptr, int64),
      array(const_cast<int64_t*>(col), (size_t)nnz, int64),
      array(const_cast<int64_t*>(start), (size_t)n, int64),
      array(const_cast<float*>(rand), (size_t)n * (size_t)walk_length, float32),
  };
  std::vector<array> outputs = {
      array({(int)n, walk_length + 1}, int64),
      array({(int)n, walk_length}, int64),
  };
  RandomWalk prim(walk_length, Stream{});
  double t0 = now_s();
  prim.eval_cpu(inputs, outputs);
  double t1 = now_s();
  if (n_out) std::memcpy(n_out, outputs[0].data<int64_t>(), sizeof(int64_t) * (size_t)n * (walk_length + 1));
  if (e_out) std::memcpy(e_out, outputs[1].data<int64_t>(), sizeof(int64_t) * (size_t)n * walk_length);
  return t1 - t0;
}

// Runs BiasedRandomWalk::eval_cpu after srand(srand_seed) (the reference draws
// from the C library's global rand(); seeding it here makes a run repeatable on
// one libc). walk_length must be >= 1 (the reference writes column 1 unconditionally).
double ref_rejection_sampling(const int64_t* rowptr, int64_t n_rowptr, const int64_t* col, int64_t nnz,
                              const int64_t* start, int64_t n, int walk_length, double p, double q,
                              unsigned srand_seed, int64_t* n_out, int64_t* e_out) {
  CoutSilencer quiet;
  float dummy = 0.f;
  std::vector<array> inputs = {
      array(const_cast<int64_t*>(rowptr), (size_t)n_rowptr, int64),
      array(const_cast<int64_t*>(col), (size_t)nnz, int64),
      array(const_cast<int64_t*>(start), (size_t)n, int64),
      array(&dummy, 1, float32),
  };
  std::vector<array> outputs = {
      array({(int)n, walk_length + 1}, int64),
      array({(int)n, walk_length}, int64),
  };
  BiasedRandomWalk prim(Stream{}, walk_length, p, q);
  std::srand(srand_seed);
  double t0 = now_s();
  prim.eval_cpu(inputs, outputs);
  double t1 = now_s();
  if (n_out) std::memcpy(n_out, outputs[0].data<int64_t>(), sizeof(int64_t) * (size_t)n * (walk_length + 1));
  if (e_out) std::memcpy(e_out, outputs[1].data<int64_t>(), sizeof(int64_t) * (size_t)n * walk_length);
  return t1 - t0;
}

// Shape metadata of the lazy node the reference factories build
// (random_walks/RandomWalk.cpp:138-148, random_walks/BiasedRandomWalk.cpp:183-193).
void ref_factory_shapes(int64_t n, int walk_length, int which, int* out4) {
  CoutSilencer quiet;
  int64_t one = 0;
  float f = 0.f;
  array rowptr(&one, 1, int64), col(&one, 1, int64), rand(&f, 1, float32);
  std::vector<int64_t> st((size_t)n, 0);
  array start(st.data(), (size_t)n, int64);
  array out = which == 0 ? random_walk(rowptr, col, start, rand, walk_length, {})
                         : rejection_sampling(rowptr, col, start, walk_length, 1.0, 1.0, {});
  out4[0] = out.shape()[0];
  out4[1] = out.shape()[1];
  out4[2] = (int)out.inputs().size();
  out4[3] = out.dtype() == int64 ? 1 : 0;
}

int ref_rand_max(void) { return RAND_MAX; }
}
