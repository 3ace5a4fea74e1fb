// Philox4x32-10 (Salmon et al., SC'11) for host and device, and the node2vec walk
// stream built on it: key = seed, counter = (walk lo32, step, attempt, walk hi32).
#pragma once
#include <cstdint>

namespace walk_b200 {

constexpr uint32_t kPhiloxM0 = 0xD2511F53u;
constexpr uint32_t kPhiloxM1 = 0xCD9E8D57u;
constexpr uint32_t kPhiloxW0 = 0x9E3779B9u;
constexpr uint32_t kPhiloxW1 = 0xBB67AE85u;

struct Philox4 {
  uint32_t x, y, z, w;
};

__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2,
                                                          uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; r++) {
    // one 32x32->64 multiply per product (a single wide multiply-add on the device)
    const uint64_t p0 = (uint64_t)kPhiloxM0 * c0;
    const uint64_t p1 = (uint64_t)kPhiloxM1 * c2;
    const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    const uint32_t n0 = hi1 ^ c1 ^ k0;
    const uint32_t n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += kPhiloxW0;
    k1 += kPhiloxW1;
  }
  return Philox4{c0, c1, c2, c3};
}

// Only the two words the walk consumes: candidate draw (word 0 >> 1) and accept draw
// (word 1 >> 1), both 31-bit like glibc rand().
__host__ __device__ __forceinline__ void node2vec_draw(uint32_t k0, uint32_t k1, uint64_t walk,
                                                       uint32_t step, uint32_t attempt,
                                                       uint32_t& cand31, uint32_t& acc31) {
  const Philox4 o = philox4x32_10((uint32_t)walk, step, attempt, (uint32_t)(walk >> 32), k0, k1);
  cand31 = o.x >> 1;
  acc31 = o.y >> 1;
}

// Draws of the uniform walk when the caller supplies no rand array: one Philox block serves four
// consecutive steps. counter = (walk lo32, step >> 2, kUniformTag, walk hi32), word (step & 3),
// r = (word >> 8) * 2^-24: a float32 in [0, 1), never 1.
constexpr uint32_t kUniformTag = 0x554E4946u;

__host__ __device__ __forceinline__ Philox4 uniform_block(uint32_t k0, uint32_t k1, uint64_t walk, uint32_t step_quad) {
  return philox4x32_10((uint32_t)walk, step_quad, kUniformTag, (uint32_t)(walk >> 32), k0, k1);
}

__host__ __device__ __forceinline__ float uniform_from_word(uint32_t w) {
  return (float)(w >> 8) * (1.0f / 16777216.0f);
}

// Negative samples of the skip-gram loss: draw k of row g is word (k & 3) of the block with
// counter = (g lo32, k >> 2, kNegativeTag, g hi32); node = (word * num_nodes) >> 32.
constexpr uint32_t kNegativeTag = 0x4E454753u;

__host__ __device__ __forceinline__ Philox4 negative_block(uint32_t k0, uint32_t k1, uint64_t row, uint32_t quad) {
  return philox4x32_10((uint32_t)row, quad, kNegativeTag, (uint32_t)(row >> 32), k0, k1);
}

__host__ __device__ __forceinline__ int64_t negative_from_word(uint32_t w, uint64_t num_nodes) {
  return (int64_t)(((uint64_t)w * num_nodes) >> 32);
}

}  // namespace walk_b200
