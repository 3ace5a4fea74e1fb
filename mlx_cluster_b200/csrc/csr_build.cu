// Edge list -> CSR on the device: the step in front of the walk generators.
//
// The reference's demos sort the edge index on the host and derive rowptr from the counts of the
// row ids that occur, which drops isolated nodes (tests/test_random_walk.py:22-28 of the reference
// project). Here the number of nodes is an argument, rowptr always has num_nodes + 1 entries, and
// the work is laid out for the GPU instead of as one global sort:
//   1. count    one atomicAdd per directed edge into its row's counter (the counters of a 16 M node
//               graph fit L2);
//   2. scan     counters -> row offsets (three small launches, no block waits for another);
//   3. fill     every edge takes a slot of its row (atomicSub on the same counters) and stores its
//               32-bit column there: rows are complete but unordered;
//   4. sort     each row on its own: up to 64 entries by one warp in registers (bitonic network over
//               two values per lane), longer rows by one block with a least-significant-digit radix
//               sort whose warps own contiguous pieces of the row (stable without any cross-warp
//               ordering inside a pass); duplicates are dropped and the row is compacted in place;
//   5. scan     surviving entries per row -> rowptr;
//   6. emit     rows are copied to their final place as int64.
// Everything is stream-ordered; nothing is read back to the host. Sorted, duplicate-free rows are
// what the node2vec membership test needs.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/walk_b200.h"
#include "host_common.h"

namespace walk_b200 {
namespace {

constexpr int kBuildBlock = 256;
constexpr int kBuildWarps = kBuildBlock / 32;
constexpr uint32_t kSmallRow = 64;         // rows up to this many raw entries: one warp, registers
constexpr uint32_t kMediumRow = 2048;      // rows up to this many: one warp, radix sort; longer: one block
constexpr uint32_t kPadKey = 0xffffffffu;  // sorts behind every node id (ids are below 2^31)
constexpr unsigned kFullMask = 0xffffffffu;
constexpr int kScanItems = 16;             // items per thread of one scan tile
constexpr int kScanTile = kBuildBlock * kScanItems;

__device__ __forceinline__ void raise(uint32_t* flags, uint32_t bit) {
  if (flags) atomicOr(flags, bit);
}

// ---- 1. count / 3. fill ------------------------------------------------------------------------
// FILL = false: count the entries of every row. FILL = true: place them; by then the scan has
// turned each counter into its row's end offset (32 bits are enough: there are fewer than 2^32
// slots), so one atomicSub both claims a slot and says where it is. Afterwards the counters are
// free for the per-row results of the sort.
template <bool FILL>
__global__ void __launch_bounds__(kBuildBlock) csr_edges_kernel(const int64_t* __restrict__ src,
                                                                const int64_t* __restrict__ dst, int64_t m,
                                                                int64_t num_nodes, uint32_t options,
                                                                uint32_t* __restrict__ counters,
                                                                uint32_t* __restrict__ raw_col,
                                                                uint32_t* __restrict__ flags) {
  const bool sym = (options & WALK_B200_BUILD_SYMMETRIZE) != 0;
  const bool drop_self = (options & WALK_B200_BUILD_DROP_SELF_LOOPS) != 0;
  const int64_t stride = (int64_t)gridDim.x * kBuildBlock;
  for (int64_t i = (int64_t)blockIdx.x * kBuildBlock + threadIdx.x; i < m; i += stride) {
    const int64_t u = __ldcs(src + i), v = __ldcs(dst + i);
    if ((uint64_t)u >= (uint64_t)num_nodes || (uint64_t)v >= (uint64_t)num_nodes) {
      if (!FILL) raise(flags, WALK_B200_FLAG_BAD_NODE);
      continue;  // the edge is left out
    }
    if (drop_self && u == v) continue;
    if (!FILL) {
      atomicAdd(counters + u, 1u);
      if (sym && u != v) atomicAdd(counters + v, 1u);
    } else {
      raw_col[atomicSub(counters + u, 1u) - 1u] = (uint32_t)v;
      if (sym && u != v) raw_col[atomicSub(counters + v, 1u) - 1u] = (uint32_t)u;
    }
  }
}

// ---- 2./5. exclusive scan of uint32 counts into int64 offsets ------------------------------------
__device__ __forceinline__ uint64_t block_exclusive_scan(uint64_t x, uint64_t* total, uint64_t* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t inc = x;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint64_t y = __shfl_up_sync(kFullMask, inc, o);
    if (lane >= o) inc += y;
  }
  __syncthreads();  // warp_sums may still be read from the previous call
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  uint64_t before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kBuildWarps; w++) {
    const uint64_t s = warp_sums[w];
    if (w < warp) before += s;
    all += s;
  }
  *total = all;
  return before + inc - x;
}

__global__ void __launch_bounds__(kBuildBlock) scan_tile_sums_kernel(const uint32_t* __restrict__ in, int64_t n,
                                                                     uint64_t* __restrict__ tile_sums) {
  __shared__ uint64_t warp_sums[kBuildWarps];
  const int64_t base = (int64_t)blockIdx.x * kScanTile;
  uint64_t mine = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; j++) {
    const int64_t i = base + (int64_t)j * kBuildBlock + threadIdx.x;
    if (i < n) mine += in[i];
  }
  uint64_t total;
  block_exclusive_scan(mine, &total, warp_sums);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

// one block: tile sums -> exclusive offsets, in place
__global__ void __launch_bounds__(kBuildBlock) scan_tile_offsets_kernel(uint64_t* __restrict__ tile_sums, int64_t tiles) {
  __shared__ uint64_t warp_sums[kBuildWarps];
  uint64_t carry = 0;
  for (int64_t b = 0; b < tiles; b += kBuildBlock) {
    const int64_t i = b + threadIdx.x;
    const uint64_t x = i < tiles ? tile_sums[i] : 0;
    uint64_t total;
    const uint64_t ex = block_exclusive_scan(x, &total, warp_sums);
    if (i < tiles) tile_sums[i] = carry + ex;
    carry += total;
  }
}

// ENDS: the count of row i is replaced by the low 32 bits of the row's end offset (the fill's cursor).
template <bool ENDS>
__global__ void __launch_bounds__(kBuildBlock) scan_write_kernel(uint32_t* __restrict__ in, int64_t n,
                                                                 const uint64_t* __restrict__ tile_offsets,
                                                                 int64_t* __restrict__ out /* [n + 1] */) {
  __shared__ uint64_t warp_sums[kBuildWarps];
  const int64_t base = (int64_t)blockIdx.x * kScanTile;
  uint64_t carry = tile_offsets[blockIdx.x];
#pragma unroll 1
  for (int j = 0; j < kScanItems; j++) {
    const int64_t i = base + (int64_t)j * kBuildBlock + threadIdx.x;
    const uint64_t x = i < n ? in[i] : 0;
    uint64_t total;
    const uint64_t ex = block_exclusive_scan(x, &total, warp_sums);
    if (i < n) out[i] = (int64_t)(carry + ex);
    if (ENDS && i < n) in[i] = (uint32_t)(carry + ex + x);
    if (i == n - 1) out[n] = (int64_t)(carry + ex + x);
    carry += total;
  }
}

// ---- 4a. rows of up to 64 entries: one warp, two values per lane ----------------------------------
__device__ __forceinline__ uint32_t cmp_swap(uint32_t v, uint32_t other, bool keep_min) {
  return keep_min ? min(v, other) : max(v, other);
}

__global__ void __launch_bounds__(kBuildBlock) csr_sort_small_kernel(const int64_t* __restrict__ raw_rowptr,
                                                                     int64_t num_nodes, uint32_t options,
                                                                     uint32_t* __restrict__ raw_col,
                                                                     uint32_t* __restrict__ kept,
                                                                     uint32_t* __restrict__ medium_rows,
                                                                     uint32_t* __restrict__ long_rows,
                                                                     unsigned long long* __restrict__ list_counts) {
  const bool dedupe = (options & WALK_B200_BUILD_DEDUPE) != 0;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * kBuildWarps;
  for (int64_t r = (int64_t)blockIdx.x * kBuildWarps + (threadIdx.x >> 5); r < num_nodes; r += warps) {
    const int64_t s = raw_rowptr[r];
    const uint64_t d = (uint64_t)(raw_rowptr[r + 1] - s);
    if (d == 0) {
      if (lane == 0) kept[r] = 0;
      continue;
    }
    if (d > kSmallRow) {  // not this kernel's: append to the list of the kernel that sorts it
      if (lane == 0) {
        if (d <= kMediumRow) medium_rows[atomicAdd(list_counts + 0, 1ull)] = (uint32_t)r;
        else long_rows[atomicAdd(list_counts + 1, 1ull)] = (uint32_t)r;
      }
      continue;
    }
    uint32_t a = (uint32_t)lane < d ? raw_col[s + lane] : kPadKey;
    uint32_t b = (uint32_t)lane + 32u < d ? raw_col[s + 32 + lane] : kPadKey;
    // bitonic network over the 64 values a[0..31], b[0..31] (value index = lane, lane + 32)
    const int top = d > 32 ? 64 : 32;
    for (int size = 2; size <= top; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        if (stride == 32) {
          const uint32_t lo = min(a, b), hi = max(a, b);
          a = lo; b = hi;
        } else {
          const uint32_t oa = __shfl_xor_sync(kFullMask, a, stride);
          const uint32_t ob = __shfl_xor_sync(kFullMask, b, stride);
          const bool lower = (lane & stride) == 0;
          a = cmp_swap(a, oa, lower == ((lane & size) == 0));
          b = cmp_swap(b, ob, lower == (((lane + 32) & size) == 0));
        }
      }
    }
    // with top == 32 only `a` was a full ascending run; b is all padding then
    uint32_t prev_a = __shfl_up_sync(kFullMask, a, 1);
    uint32_t prev_b = __shfl_up_sync(kFullMask, b, 1);
    const uint32_t last_a = __shfl_sync(kFullMask, a, 31);
    if (lane == 0) prev_b = last_a;
    const bool keep_a = a != kPadKey && (!dedupe || lane == 0 || a != prev_a);
    const bool keep_b = b != kPadKey && (!dedupe || b != prev_b);
    const unsigned ma = __ballot_sync(kFullMask, keep_a), mb = __ballot_sync(kFullMask, keep_b);
    const unsigned lt = (1u << lane) - 1u;
    __syncwarp();
    if (keep_a) raw_col[s + __popc(ma & lt)] = a;
    if (keep_b) raw_col[s + __popc(ma) + __popc(mb & lt)] = b;
    if (lane == 0) kept[r] = (uint32_t)(__popc(ma) + __popc(mb));
  }
}

// ---- 4b. rows of 65 .. kMediumRow entries: one warp, LSD radix sort between the row and its twin ----
// Same passes as the block kernel below with a team of one warp: no block barrier anywhere, a
// 256-bin histogram per warp, lane l owns bins 8l .. 8l+7 in the scan.
__global__ void __launch_bounds__(kBuildBlock) csr_sort_medium_kernel(const int64_t* __restrict__ raw_rowptr,
                                                                      uint32_t options, int32_t passes, int32_t digit_bits,
                                                                      uint32_t* __restrict__ raw_col,
                                                                      uint32_t* __restrict__ tmp,
                                                                      uint32_t* __restrict__ kept,
                                                                      const uint32_t* __restrict__ medium_rows,
                                                                      const unsigned long long* __restrict__ medium_count) {
  __shared__ uint32_t hist[kBuildWarps][256];
  const bool dedupe = (options & WALK_B200_BUILD_DEDUPE) != 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  const uint32_t digit_mask = (1u << digit_bits) - 1u;
  uint32_t* bins = hist[warp];
  const unsigned long long rows = *medium_count;
  const unsigned long long warps = (unsigned long long)gridDim.x * kBuildWarps;
  for (unsigned long long w = (unsigned long long)blockIdx.x * kBuildWarps + warp; w < rows; w += warps) {
    const uint32_t r = medium_rows[w];
    const int64_t s = raw_rowptr[r];
    const uint32_t d = (uint32_t)(raw_rowptr[r + 1] - s);
    uint32_t* cur = raw_col + s;
    uint32_t* alt = tmp + s;
    for (int32_t pass = 0; pass < passes; pass++) {
      const int shift = pass * digit_bits;
#pragma unroll
      for (int k = 0; k < 8; k++) bins[lane + 32 * k] = 0;
      __syncwarp();
      for (uint32_t i = lane; i < d; i += 32) atomicAdd(&bins[(cur[i] >> shift) & digit_mask], 1u);
      __syncwarp();
      {  // exclusive scan of the 256 bins
        uint32_t c[8], sum = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) { c[k] = bins[lane * 8 + k]; sum += c[k]; }
        uint32_t inc = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t y = __shfl_up_sync(kFullMask, inc, o);
          if (lane >= o) inc += y;
        }
        uint32_t run = inc - sum;
#pragma unroll
        for (int k = 0; k < 8; k++) { bins[lane * 8 + k] = run; run += c[k]; }
      }
      __syncwarp();
      uint32_t v_next = lane < d ? cur[lane] : 0u;
      for (uint32_t i0 = 0; i0 < d; i0 += 32) {
        const uint32_t i = i0 + lane;
        const bool valid = i < d;
        const uint32_t v = v_next;
        if (i + 32 < d) v_next = cur[i + 32];
        const uint32_t digit = valid ? ((v >> shift) & digit_mask) : 0xffffffffu;
        const unsigned same = __match_any_sync(kFullMask, digit);
        const uint32_t rank = (uint32_t)__popc(same & lt);
        uint32_t base = 0;
        if (valid) base = bins[digit];
        __syncwarp();
        if (valid) {
          alt[base + rank] = v;
          if (rank == 0) bins[digit] = base + (uint32_t)__popc(same);
        }
        __syncwarp();
      }
      uint32_t* t = cur; cur = alt; alt = t;
    }
    // drop duplicates, compact to the front of the row in raw_col (in place when cur is the row:
    // a survivor never moves up, and a step's reads come before its writes)
    uint32_t* out = raw_col + s;
    uint32_t written = 0;
    for (uint32_t i0 = 0; i0 < d; i0 += 32) {
      const uint32_t i = i0 + lane;
      uint32_t v = 0;
      bool keep = false;
      if (i < d) {
        v = cur[i];
        keep = !dedupe || i == 0 || cur[i - 1] != v;
      }
      const unsigned m = __ballot_sync(kFullMask, keep);
      if (keep) out[written + (uint32_t)__popc(m & lt)] = v;
      written += (uint32_t)__popc(m);
      __syncwarp();
    }
    if (lane == 0) kept[r] = written;
  }
}

// ---- 4c. longer rows: one block, LSD radix sort between the row and its twin in `tmp` -------------
// Warp w owns the contiguous piece [w * piece, (w + 1) * piece) of the row. A pass counts digits per
// warp, turns the counts into one start offset per (digit, warp) -- all of digit k before digit k+1,
// within a digit warp 0's entries before warp 1's -- and then every warp scatters its piece in order,
// 32 entries at a time, ranking equal digits inside the 32 with match_any. Stable, and no warp waits
// for another inside the scatter.
__global__ void __launch_bounds__(kBuildBlock) csr_sort_long_kernel(const int64_t* __restrict__ raw_rowptr,
                                                                    uint32_t options, int32_t passes, int32_t digit_bits,
                                                                    uint32_t* __restrict__ raw_col,
                                                                    uint32_t* __restrict__ tmp,
                                                                    uint32_t* __restrict__ kept,
                                                                    const uint32_t* __restrict__ long_rows,
                                                                    const unsigned long long* __restrict__ long_count) {
  __shared__ uint32_t offs[kBuildWarps][256];
  __shared__ uint64_t warp_sums[kBuildWarps];
  __shared__ uint32_t tile_warp_kept[kBuildWarps];
  const bool dedupe = (options & WALK_B200_BUILD_DEDUPE) != 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  const uint32_t digit_mask = (1u << digit_bits) - 1u;
  const unsigned long long rows = *long_count;
  for (unsigned long long w = blockIdx.x; w < rows; w += gridDim.x) {
    const uint32_t r = long_rows[w];
    const int64_t s = raw_rowptr[r];
    const uint32_t d = (uint32_t)(raw_rowptr[r + 1] - s);
    const uint64_t piece = ((((uint64_t)d + kBuildWarps - 1) / kBuildWarps) + 31u) & ~(uint64_t)31;
    const uint32_t p_begin = (uint32_t)min((uint64_t)d, piece * (uint64_t)warp);
    const uint32_t p_end = (uint32_t)min((uint64_t)d, piece * (uint64_t)(warp + 1));
    uint32_t* cur = raw_col + s;
    uint32_t* alt = tmp + s;
    for (int32_t pass = 0; pass < passes; pass++) {
      const int shift = pass * digit_bits;
      for (int k = threadIdx.x; k < kBuildWarps * 256; k += kBuildBlock) (&offs[0][0])[k] = 0;
      __syncthreads();
      for (uint32_t i = p_begin + lane; i < p_end; i += 32) atomicAdd(&offs[warp][(cur[i] >> shift) & digit_mask], 1u);
      __syncthreads();
      {  // thread t is digit t: exclusive offsets over (digit, warp)
        uint64_t total = 0;
#pragma unroll
        for (int k = 0; k < kBuildWarps; k++) total += offs[k][threadIdx.x];
        uint64_t all;
        uint32_t run = (uint32_t)block_exclusive_scan(total, &all, warp_sums);
#pragma unroll
        for (int k = 0; k < kBuildWarps; k++) {
          const uint32_t c = offs[k][threadIdx.x];
          offs[k][threadIdx.x] = run;
          run += c;
        }
      }
      __syncthreads();
      uint32_t v_next = p_begin + lane < p_end ? cur[p_begin + lane] : 0u;  // fetched one step ahead
      for (uint32_t i0 = p_begin; i0 < p_end; i0 += 32) {
        const uint32_t i = i0 + lane;
        const bool valid = i < p_end;
        const uint32_t v = v_next;
        if ((uint64_t)i + 32 < p_end) v_next = cur[i + 32];
        const uint32_t digit = valid ? ((v >> shift) & digit_mask) : 0xffffffffu;
        const unsigned same = __match_any_sync(kFullMask, digit);
        const uint32_t rank = (uint32_t)__popc(same & lt);
        uint32_t base = 0;
        if (valid) base = offs[warp][digit];
        __syncwarp();
        if (valid) {
          alt[base + rank] = v;
          if (rank == 0) offs[warp][digit] = base + (uint32_t)__popc(same);
        }
        __syncwarp();
      }
      __syncthreads();
      uint32_t* t = cur; cur = alt; alt = t;
    }
    // `cur` is sorted. Drop duplicates and write the survivors to the front of the row in raw_col.
    // In place this is safe: a survivor moves to an index not above its own, tiles go in order, and
    // the element a tile compares its first entry with is read after the earlier tiles' writes,
    // none of which can have changed it.
    uint32_t* out = raw_col + s;
    uint32_t written = 0;
    for (uint32_t i0 = 0; i0 < d; i0 += kBuildBlock) {
      const uint32_t i = i0 + threadIdx.x;
      uint32_t v = 0;
      bool keep = false;
      if (i < d) {
        v = cur[i];
        keep = !dedupe || i == 0 || cur[i - 1] != v;
      }
      const unsigned m = __ballot_sync(kFullMask, keep);
      __syncthreads();  // all reads of this tile are done; tile_warp_kept is free again
      if (lane == 0) tile_warp_kept[warp] = (uint32_t)__popc(m);
      __syncthreads();
      uint32_t before = 0, all = 0;
#pragma unroll
      for (int k = 0; k < kBuildWarps; k++) {
        const uint32_t c = tile_warp_kept[k];
        if (k < warp) before += c;
        all += c;
      }
      if (keep) out[written + before + (uint32_t)__popc(m & lt)] = v;
      written += all;
    }
    if (threadIdx.x == 0) kept[r] = written;
    __syncthreads();
  }
}

// ---- 6. emit ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBuildBlock) csr_emit_small_kernel(const int64_t* __restrict__ raw_rowptr,
                                                                     const uint32_t* __restrict__ raw_col,
                                                                     const int64_t* __restrict__ rowptr,
                                                                     int64_t num_nodes, int64_t* __restrict__ col) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * kBuildWarps;
  for (int64_t r = (int64_t)blockIdx.x * kBuildWarps + (threadIdx.x >> 5); r < num_nodes; r += warps) {
    const int64_t s = raw_rowptr[r];
    if ((uint64_t)(raw_rowptr[r + 1] - s) > kMediumRow) continue;  // a long row: the block kernel's
    const int64_t o = rowptr[r];
    const int64_t k = rowptr[r + 1] - o;
    for (int64_t j = lane; j < k; j += 32) col[o + j] = (int64_t)raw_col[s + j];
  }
}

__global__ void __launch_bounds__(kBuildBlock) csr_emit_long_kernel(const int64_t* __restrict__ raw_rowptr,
                                                                    const uint32_t* __restrict__ raw_col,
                                                                    const int64_t* __restrict__ rowptr,
                                                                    const uint32_t* __restrict__ long_rows,
                                                                    const unsigned long long* __restrict__ long_count,
                                                                    int64_t* __restrict__ col) {
  const unsigned long long rows = *long_count;
  for (unsigned long long w = blockIdx.x; w < rows; w += gridDim.x) {
    const uint32_t r = long_rows[w];
    const int64_t s = raw_rowptr[r], o = rowptr[r];
    const int64_t k = rowptr[r + 1] - o;
    for (int64_t j = threadIdx.x; j < k; j += kBuildBlock) col[o + j] = (int64_t)raw_col[s + j];
  }
}

// ---- scratch layout ----------------------------------------------------------------------------------
struct BuildLayout {
  size_t counters, raw_rowptr, tile_sums, raw_col, tmp, medium_rows, long_rows, list_counts, total;
};

size_t align_up(size_t x) { return (x + 255) & ~size_t(255); }

BuildLayout build_layout(int64_t m, int64_t num_nodes, uint32_t options) {
  const size_t slots = (size_t)m * ((options & WALK_B200_BUILD_SYMMETRIZE) ? 2 : 1);
  const size_t tiles = ((size_t)num_nodes + kScanTile - 1) / kScanTile + 1;
  BuildLayout L{};
  size_t at = 0;
  L.counters = at;   at += align_up((size_t)num_nodes * 4 + 4);
  L.raw_rowptr = at; at += align_up(((size_t)num_nodes + 1) * 8);
  L.tile_sums = at;  at += align_up(tiles * 8);
  L.raw_col = at;    at += align_up(slots * 4 + 4);
  L.tmp = at;        at += align_up(slots * 4 + 4);
  L.medium_rows = at; at += align_up((slots / (kSmallRow + 1) + 1) * 4);
  L.long_rows = at;   at += align_up((slots / (kMediumRow + 1) + 1) * 4);
  L.list_counts = at; at += align_up(16);
  L.total = at;
  return L;
}

int check_build_args(int64_t m, int64_t num_nodes, uint32_t options) {
  if (m < 0 || num_nodes < 0) return host::fail(WALK_B200_ERR_INVALID_ARG, "negative edge or node count");
  if (options & ~(uint32_t)(WALK_B200_BUILD_SYMMETRIZE | WALK_B200_BUILD_DROP_SELF_LOOPS | WALK_B200_BUILD_DEDUPE))
    return host::fail(WALK_B200_ERR_INVALID_ARG, "unknown build option bits 0x%x", options);
  if (num_nodes >= (1ll << 31))
    return host::fail(WALK_B200_ERR_UNSUPPORTED, "the CSR builder needs num_nodes < 2^31");
  if (m >= (1ll << 31))
    return host::fail(WALK_B200_ERR_UNSUPPORTED, "the CSR builder needs fewer than 2^31 input edges");
  return WALK_B200_OK;
}

int scan_counts(uint32_t* counts, int64_t n, uint64_t* tile_sums, int64_t* out, bool ends, cudaStream_t s) {
  if (n == 0) {
    WALK_CUDA_TRY(cudaMemsetAsync(out, 0, 8, s));
    return WALK_B200_OK;
  }
  const int64_t tiles = (n + kScanTile - 1) / kScanTile;
  scan_tile_sums_kernel<<<(unsigned)tiles, kBuildBlock, 0, s>>>(counts, n, tile_sums);
  if (int rc = host::check_launch("scan_tile_sums_kernel")) return rc;
  scan_tile_offsets_kernel<<<1, kBuildBlock, 0, s>>>(tile_sums, tiles);
  if (int rc = host::check_launch("scan_tile_offsets_kernel")) return rc;
  if (ends) scan_write_kernel<true><<<(unsigned)tiles, kBuildBlock, 0, s>>>(counts, n, tile_sums, out);
  else scan_write_kernel<false><<<(unsigned)tiles, kBuildBlock, 0, s>>>(counts, n, tile_sums, out);
  return host::check_launch("scan_write_kernel");
}

unsigned capped_grid(int64_t items_per_block_units, int per_sm) {
  int64_t cap = (int64_t)host::sm_count() * per_sm;
  int64_t g = items_per_block_units < cap ? items_per_block_units : cap;
  return (unsigned)(g < 1 ? 1 : g);
}

}  // namespace
}  // namespace walk_b200

using namespace walk_b200;

extern "C" {

int walk_b200_csr_build_scratch_bytes(int64_t num_input_edges, int64_t num_nodes, uint32_t options,
                                      uint64_t* bytes) {
  if (!bytes) return host::fail(WALK_B200_ERR_INVALID_ARG, "bytes is NULL");
  if (int rc = check_build_args(num_input_edges, num_nodes, options)) return rc;
  *bytes = build_layout(num_input_edges, num_nodes, options).total;
  return WALK_B200_OK;
}

int walk_b200_csr_build(const int64_t* src, const int64_t* dst, int64_t num_input_edges, int64_t num_nodes,
                        uint32_t options, void* scratch, uint64_t scratch_bytes, int64_t* rowptr,
                        int64_t* col, uint32_t* status_flags, void* stream) {
  if (int rc = check_build_args(num_input_edges, num_nodes, options)) return rc;
  if (!rowptr) return host::fail(WALK_B200_ERR_INVALID_ARG, "rowptr is NULL");
  if (num_input_edges > 0 && (!src || !dst || !col))
    return host::fail(WALK_B200_ERR_INVALID_ARG, "src, dst or col is NULL");
  const BuildLayout L = build_layout(num_input_edges, num_nodes, options);
  if (!scratch || scratch_bytes < L.total)
    return host::fail(WALK_B200_ERR_INVALID_ARG, "scratch too small: %llu bytes given, %llu needed",
                      (unsigned long long)scratch_bytes, (unsigned long long)L.total);
  if ((reinterpret_cast<uintptr_t>(scratch) & 255) != 0)
    return host::fail(WALK_B200_ERR_INVALID_ARG, "scratch must be 256-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  char* base = static_cast<char*>(scratch);
  uint32_t* counters = reinterpret_cast<uint32_t*>(base + L.counters);
  int64_t* raw_rowptr = reinterpret_cast<int64_t*>(base + L.raw_rowptr);
  uint64_t* tile_sums = reinterpret_cast<uint64_t*>(base + L.tile_sums);
  uint32_t* raw_col = reinterpret_cast<uint32_t*>(base + L.raw_col);
  uint32_t* tmp = reinterpret_cast<uint32_t*>(base + L.tmp);
  uint32_t* medium_rows = reinterpret_cast<uint32_t*>(base + L.medium_rows);
  uint32_t* long_rows = reinterpret_cast<uint32_t*>(base + L.long_rows);
  unsigned long long* list_counts = reinterpret_cast<unsigned long long*>(base + L.list_counts);
  unsigned long long* long_count = list_counts + 1;

  if (num_nodes == 0 || num_input_edges == 0) {
    WALK_CUDA_TRY(cudaMemsetAsync(rowptr, 0, ((size_t)num_nodes + 1) * 8, s));
    return WALK_B200_OK;
  }
  WALK_CUDA_TRY(cudaMemsetAsync(counters, 0, (size_t)num_nodes * 4, s));
  WALK_CUDA_TRY(cudaMemsetAsync(list_counts, 0, 16, s));

  const unsigned edge_grid = capped_grid((num_input_edges + kBuildBlock - 1) / kBuildBlock, 16);
  csr_edges_kernel<false><<<edge_grid, kBuildBlock, 0, s>>>(src, dst, num_input_edges, num_nodes, options, counters,
                                                            nullptr, status_flags);
  if (int rc = host::check_launch("csr_edges_kernel<count>")) return rc;
  if (int rc = scan_counts(counters, num_nodes, tile_sums, raw_rowptr, true, s)) return rc;
  csr_edges_kernel<true><<<edge_grid, kBuildBlock, 0, s>>>(src, dst, num_input_edges, num_nodes, options, counters,
                                                           raw_col, status_flags);
  if (int rc = host::check_launch("csr_edges_kernel<fill>")) return rc;

  const unsigned row_grid = capped_grid((num_nodes + kBuildWarps - 1) / kBuildWarps, 16);
  csr_sort_small_kernel<<<row_grid, kBuildBlock, 0, s>>>(raw_rowptr, num_nodes, options, raw_col, counters, medium_rows,
                                                         long_rows, list_counts);
  if (int rc = host::check_launch("csr_sort_small_kernel")) return rc;
  int key_bits = 1;
  while (key_bits < 31 && (1ll << key_bits) < num_nodes) key_bits++;
  const int passes = (key_bits + 7) / 8;
  const int digit_bits = (key_bits + passes - 1) / passes;
  const unsigned long_grid = (unsigned)host::sm_count() * 8;
  csr_sort_medium_kernel<<<long_grid, kBuildBlock, 0, s>>>(raw_rowptr, options, passes, digit_bits, raw_col, tmp, counters,
                                                           medium_rows, list_counts);
  if (int rc = host::check_launch("csr_sort_medium_kernel")) return rc;
  csr_sort_long_kernel<<<long_grid, kBuildBlock, 0, s>>>(raw_rowptr, options, passes, digit_bits, raw_col, tmp, counters,
                                                         long_rows, long_count);
  if (int rc = host::check_launch("csr_sort_long_kernel")) return rc;

  if (int rc = scan_counts(counters, num_nodes, tile_sums, rowptr, false, s)) return rc;
  csr_emit_small_kernel<<<row_grid, kBuildBlock, 0, s>>>(raw_rowptr, raw_col, rowptr, num_nodes, col);
  if (int rc = host::check_launch("csr_emit_small_kernel")) return rc;
  csr_emit_long_kernel<<<long_grid, kBuildBlock, 0, s>>>(raw_rowptr, raw_col, rowptr, long_rows, long_count, col);
  return host::check_launch("csr_emit_long_kernel");
}

}  // extern "C"
