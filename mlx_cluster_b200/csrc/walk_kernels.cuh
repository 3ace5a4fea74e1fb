// sm_100a kernels of the two CSR walk generators.
//
// Both walks are chains of dependent 8-byte gathers (row bounds -> col entry), so the
// kernels are organised around memory behaviour, not arithmetic:
//   * every divergent (one-sector-per-lane) memory instruction costs a warp 32 L1 tag
//     cycles, so the per-step count of such instructions is kept minimal: one 8-byte
//     row descriptor instead of a rowptr pair, and rand / walk-matrix traffic staged
//     through shared memory so that its global side is coalesced row segments;
//   * latency is hidden by occupancy (one walk per thread, >= 1536 threads per SM),
//     not by anything clever inside one walk: a walk's steps are inherently serial;
//   * node2vec runs as a per-thread state machine that issues exactly one gather per
//     loop trip whatever the walk is doing (row fetch, candidate draw, binary-search
//     probe), so lanes of a warp never wait for each other's rejection loops.
// No tensor cores: there is no dense contraction anywhere in this path.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <type_traits>

#include "../../include/walk_b200.h"
#include "philox.cuh"

namespace walk_b200 {

constexpr int kBlock = 256;
constexpr int kWarpsPerBlock = kBlock / 32;
constexpr int kDescStartBits = 36;
constexpr uint64_t kDescStartMask = (1ull << kDescStartBits) - 1;
constexpr uint64_t kDescMaxDeg = (1ull << (64 - kDescStartBits)) - 1;

__device__ __forceinline__ void raise_flag(uint32_t* flags, uint32_t bit) {
  if (flags) atomicOr(flags, bit);
}

// ---- L2 eviction policies ---------------------------------------------------------
// Row bounds are re-read all the time (accesses are skewed to hub nodes) while col
// gathers, rand and the walk matrix stream through once: the former are loaded with an
// evict-last policy, the latter with evict-first, so that the stream does not flush the
// row descriptors out of L2. `hints` bit 0 enables the former, bit 1 the latter.
struct L2Policy {
  uint64_t keep, stream, normal;
};

__device__ __forceinline__ L2Policy make_policies(int hints) {
  L2Policy p;
  if (hints & 4) {  // no explicit policy at all (0 selects the plain load forms below)
    p.keep = p.stream = p.normal = 0;
    return p;
  }
  asm("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p.normal));
  p.keep = p.normal;
  p.stream = p.normal;
  if (hints & 1) asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p.keep));
  if (hints & 2) asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p.stream));
  return p;
}

// Read-only 8-byte random gather with an L2 policy (inputs never change during a launch).
// On this part a missing gather pulls a whole 128-byte line from DRAM by default; the
// 64-byte prefetch size halves that (measured: 123 -> 63 bytes of DRAM per gather).
__device__ __forceinline__ int64_t ld8(const void* addr, uint64_t policy) {
  int64_t v;
  if (policy) asm("ld.global.nc.L2::cache_hint.L2::64B.b64 %0, [%1], %2;" : "=l"(v) : "l"(addr), "l"(policy));
  else asm("ld.global.nc.L2::64B.b64 %0, [%1];" : "=l"(v) : "l"(addr));
  return v;
}
__device__ __forceinline__ uint32_t ld4(const void* addr, uint64_t policy) {
  uint32_t v;
  if (policy) asm("ld.global.nc.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(v) : "l"(addr), "l"(policy));
  else asm("ld.global.nc.b32 %0, [%1];" : "=r"(v) : "l"(addr));
  return v;
}
__device__ __forceinline__ ulonglong2 ld16(const void* addr, uint64_t policy) {
  ulonglong2 v;
  if (policy) asm("ld.global.nc.L2::cache_hint.L2::64B.v2.b64 {%0, %1}, [%2], %3;" : "=l"(v.x), "=l"(v.y) : "l"(addr), "l"(policy));
  else asm("ld.global.nc.L2::64B.v2.b64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(addr));
  return v;
}
__device__ __forceinline__ void st8(void* addr, int64_t v, uint64_t policy) {
  if (policy) asm volatile("st.global.L2::cache_hint.b64 [%0], %1, %2;" ::"l"(addr), "l"(v), "l"(policy) : "memory");
  else asm volatile("st.global.b64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}

// Row bounds of node v: one 8-byte load when a packed descriptor exists.
template <bool USE_DESC>
__device__ __forceinline__ void load_row(const int64_t* __restrict__ rowptr,
                                         const uint64_t* __restrict__ desc, int64_t v,
                                         uint64_t policy, int64_t& row_start, int64_t& deg) {
  if (USE_DESC) {
    const uint64_t d = (uint64_t)ld8(desc + v, policy);
    row_start = (int64_t)(d & kDescStartMask);
    deg = (int64_t)(d >> kDescStartBits);
  } else {
    const int64_t a = ld8(rowptr + v, policy);
    const int64_t b = ld8(rowptr + v + 1, policy);
    row_start = a;
    deg = b - a;
  }
}

// ---------------------------------------------------------------------------------
// gather_probe: what this device sustains in dependent random 8-byte gathers that miss L2.
// Each thread chases a pseudo-random chain through a large array, one gather in flight
// per thread, exactly the access pattern of a walk step. The walks cannot beat this rate
// per DRAM-missing gather, whatever their byte counts say.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z ^= z >> 30; z *= 0xbf58476d1ce4e5b9ull;
  z ^= z >> 27; z *= 0x94d049bb133111ebull;
  z ^= z >> 31;
  return z;
}

// CHAINS independent chains per thread (that many gathers in flight per thread), BYTES per gather
// (8, 16 or 32, naturally aligned), and the amount the L2 fetches from DRAM on a miss (64-byte
// prefetch size as the walks use, or the part's default of a whole 128-byte line).
template <int CHAINS, int BYTES, bool FETCH64>
__global__ void __launch_bounds__(kBlock) gather_probe_kernel(const int64_t* __restrict__ data,
                                                              uint64_t num_elems, int iters,
                                                              int64_t* sink) {
  static_assert(BYTES == 8 || BYTES == 16 || BYTES == 32, "gather width");
  constexpr int kWords = BYTES / 8;
  const uint64_t tid = (uint64_t)blockIdx.x * kBlock + threadIdx.x;
  uint64_t idx[CHAINS];
  int64_t acc[CHAINS];
#pragma unroll
  for (int c = 0; c < CHAINS; c++) { idx[c] = splitmix64(tid * CHAINS + c + 1); acc[c] = 0; }
  const uint64_t slots = num_elems / kWords;
  for (int i = 0; i < iters; i++) {
#pragma unroll
    for (int c = 0; c < CHAINS; c++) {
      idx[c] = splitmix64(idx[c] + (uint64_t)acc[c]);
      const int64_t* addr = data + __umul64hi(idx[c], slots) * kWords;
      int64_t a = 0, b = 0, d = 0, e = 0;
      if (BYTES == 8) {
        if (FETCH64) asm volatile("ld.global.nc.L2::64B.b64 %0, [%1];" : "=l"(a) : "l"(addr));
        else asm volatile("ld.global.nc.b64 %0, [%1];" : "=l"(a) : "l"(addr));
      } else {
        if (FETCH64) asm volatile("ld.global.nc.L2::64B.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(addr));
        else asm volatile("ld.global.nc.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(addr));
        if (BYTES == 32) {
          if (FETCH64) asm volatile("ld.global.nc.L2::64B.v2.b64 {%0, %1}, [%2];" : "=l"(d), "=l"(e) : "l"(addr + 2));
          else asm volatile("ld.global.nc.v2.b64 {%0, %1}, [%2];" : "=l"(d), "=l"(e) : "l"(addr + 2));
        }
      }
      acc[c] += a + b + d + e;
    }
  }
  int64_t total = 0;
#pragma unroll
  for (int c = 0; c < CHAINS; c++) total += acc[c];
  if (total == 0x7fffffffffffffffll) *sink = total;  // never true on a zeroed array; keeps the chains alive
}

// ---------------------------------------------------------------------------------
// rowdesc_pack: rowptr -> (start | degree << 36). Streaming, one thread per node.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock) rowdesc_pack_kernel(const int64_t* __restrict__ rowptr,
                                                              int64_t num_nodes, int64_t num_edges,
                                                              uint64_t* __restrict__ desc,
                                                              uint32_t* flags) {
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t v = (int64_t)blockIdx.x * kBlock + threadIdx.x; v < num_nodes; v += stride) {
    const int64_t a = rowptr[v];
    const int64_t b = rowptr[v + 1];
    int64_t deg = b - a;
    uint32_t bad = 0;
    if (a < 0 || b < a || b > num_edges) { bad |= WALK_B200_FLAG_BAD_ROWPTR; deg = 0; }
    if ((uint64_t)a > kDescStartMask || (uint64_t)deg > kDescMaxDeg) {
      bad |= WALK_B200_FLAG_DESC_OVERFLOW;
      deg = 0;
    }
    if (bad) raise_flag(flags, bad);
    desc[v] = ((uint64_t)a & kDescStartMask) | ((uint64_t)deg << kDescStartBits);
  }
}

// ---------------------------------------------------------------------------------
// csr_validate: grid-stride over nodes, edges and starts.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock) csr_validate_kernel(const int64_t* __restrict__ rowptr,
                                                              const int64_t* __restrict__ col,
                                                              int64_t num_nodes, int64_t num_edges,
                                                              const int64_t* __restrict__ start,
                                                              int64_t num_walks, int check_sorted,
                                                              uint32_t* flags) {
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  const int64_t tid = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  uint32_t bad = 0;
  if (tid == 0) {
    if (rowptr[0] != 0 || rowptr[num_nodes] != num_edges) bad |= WALK_B200_FLAG_BAD_ROWPTR;
  }
  for (int64_t v = tid; v < num_nodes; v += stride) {
    const int64_t a = rowptr[v], b = rowptr[v + 1];
    if (a < 0 || b < a || b > num_edges) {
      bad |= WALK_B200_FLAG_BAD_ROWPTR;
    } else if (check_sorted) {
      // rows are short on average; hub rows are walked by one thread, acceptable for a checker
      for (int64_t e = a + 1; e < b; e++)
        if (col[e - 1] >= col[e]) { bad |= WALK_B200_FLAG_UNSORTED_ROW; break; }
    }
  }
  for (int64_t e = tid; e < num_edges; e += stride) {
    const int64_t c = col[e];
    if (c < 0 || c >= num_nodes) bad |= WALK_B200_FLAG_BAD_NODE;
  }
  if (start) {
    for (int64_t w = tid; w < num_walks; w += stride) {
      const int64_t s = start[w];
      if (s < 0 || s >= num_nodes) bad |= WALK_B200_FLAG_BAD_NODE;
    }
  }
  if (bad) raise_flag(flags, bad);
}

// ---------------------------------------------------------------------------------
// uniform walk
// ---------------------------------------------------------------------------------
// fused edge records: fused[e] = (col[e], row descriptor of col[e]). One 16-byte gather then
// yields the next node *and* its row bounds, so a uniform step is one dependent DRAM access
// instead of two (col entry, then the target's row descriptor).
__global__ void __launch_bounds__(kBlock) fused_build_kernel(const int64_t* __restrict__ col,
                                                             const uint64_t* __restrict__ desc,
                                                             int64_t num_nodes, int64_t num_edges,
                                                             ulonglong2* __restrict__ fused, uint32_t* flags) {
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t e = (int64_t)blockIdx.x * kBlock + threadIdx.x; e < num_edges; e += stride) {
    const int64_t c = col[e];
    ulonglong2 rec;
    rec.x = (unsigned long long)c;
    if ((uint64_t)c >= (uint64_t)num_nodes) {
      raise_flag(flags, WALK_B200_FLAG_BAD_NODE);
      rec.y = 0;  // degree 0: a walk that lands here parks
    } else {
      rec.y = __ldg(desc + c);
    }
    fused[e] = rec;
  }
}

// col and reverse position in one 8-byte word: colrev[e] = col[e] | revpos[e] << 32. The gather of a
// candidate then also brings the position of the edge back from it, which is what the step after an
// accepted candidate needs; the separate 4-byte gather of revpos per step disappears.
__global__ void __launch_bounds__(kBlock) colrev_build_kernel(const int64_t* __restrict__ col,
                                                              const uint32_t* __restrict__ revpos,
                                                              int64_t num_nodes, int64_t num_edges,
                                                              uint64_t* __restrict__ colrev, uint32_t* flags) {
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t e = (int64_t)blockIdx.x * kBlock + threadIdx.x; e < num_edges; e += stride) {
    const int64_t c = col[e];
    if ((uint64_t)c >= (uint64_t)num_nodes) {
      raise_flag(flags, WALK_B200_FLAG_BAD_NODE);
      colrev[e] = 0xffffffffull | (0xfffffffeull << 32);  // out of range for the walk to flag; edge back unknown
    } else {
      colrev[e] = (uint64_t)(uint32_t)c | ((uint64_t)revpos[e] << 32);
    }
  }
}

struct UniformParams {
  const int64_t* rowptr;
  const int64_t* col;
  const uint64_t* desc;
  const ulonglong2* fused;
  int64_t num_nodes, num_edges;
  const int64_t* start;
  const float* rand;
  int64_t num_walks;
  int32_t walk_length;
  int32_t hints;
  int64_t* n_out;
  int64_t* e_out;
  uint32_t* flags;
  int32_t generate;           // draws come from the kernel's own Philox stream instead of `rand`
  uint32_t key0, key1;        // its key
  uint64_t walk_index_base, walk_index_stride;
};

// One uniform step from `cur` with draw r. Same float32 arithmetic as the reference:
// degree converted to float32 (round to nearest), float32 product, truncation.
// A node without out-edges parks the walk for good (its row can never gain an edge).
template <bool USE_DESC>
__device__ __forceinline__ int64_t uniform_step(const UniformParams& P, const L2Policy& pol, int64_t& cur,
                                                bool& parked, float r) {
  int64_t rs, deg;
  load_row<USE_DESC>(P.rowptr, P.desc, cur, pol.keep, rs, deg);
  if (deg <= 0) {
    if (deg < 0) raise_flag(P.flags, WALK_B200_FLAG_BAD_ROWPTR);
    parked = true;
    return -1;
  }
  const float prod = __fmul_rn(r, __ll2float_rn(deg));
  int64_t e = rs + __float2ll_rz(prod);
  if ((uint64_t)e >= (uint64_t)P.num_edges) {  // rand >= 1, NaN, negative, or corrupt rowptr
    raise_flag(P.flags, WALK_B200_FLAG_BAD_EDGE);
    if (P.num_edges <= 0) {  // nothing to clamp to (col may be NULL): park instead of gathering
      parked = true;
      return -1;
    }
    e = e < 0 ? 0 : P.num_edges - 1;
  }
  const int64_t nxt = ld8(P.col + e, pol.stream);
  if ((uint64_t)nxt >= (uint64_t)P.num_nodes) {
    raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);  // park: keep cur
    parked = true;
  } else {
    cur = nxt;
  }
  return e;
}

// Same step on fused edge records: the lane carries the row bounds of `cur` and gets the next
// node together with that node's bounds from one 16-byte gather.
__device__ __forceinline__ int64_t uniform_step_fused(const UniformParams& P, const L2Policy& pol, int64_t& cur,
                                                      int64_t& rs, int64_t& deg, bool& parked, float r) {
  if (deg <= 0) {
    parked = true;
    return -1;
  }
  const float prod = __fmul_rn(r, __ll2float_rn(deg));
  int64_t e = rs + __float2ll_rz(prod);
  if ((uint64_t)e >= (uint64_t)P.num_edges) {
    raise_flag(P.flags, WALK_B200_FLAG_BAD_EDGE);
    if (P.num_edges <= 0) {
      parked = true;
      return -1;
    }
    e = e < 0 ? 0 : P.num_edges - 1;
  }
  const ulonglong2 rec = ld16(P.fused + e, pol.stream);
  if (rec.x >= (uint64_t)P.num_nodes) {
    raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);  // park: keep cur
    parked = true;
  } else {
    cur = (int64_t)rec.x;
    rs = (int64_t)(rec.y & kDescStartMask);
    deg = (int64_t)(rec.y >> kDescStartBits);
  }
  return e;
}

// Plain variant: every thread reads its own rand entries and writes its own row with
// 8-byte strided accesses. Kept as the baseline the staged kernel is measured against
// (it is what the reference's Metal kernel does) and for walk lengths below one chunk.
template <bool USE_DESC, bool HAS_EOUT>
__global__ void __launch_bounds__(kBlock) uniform_walk_direct_kernel(const UniformParams P) {
  const int64_t w = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  if (w >= P.num_walks) return;
  const L2Policy pol = make_policies(P.hints);
  const int64_t L = P.walk_length;
  int64_t cur = P.start[w];
  int64_t* out = P.n_out + w * (L + 1);
  out[0] = cur;
  bool parked = false;
  if ((uint64_t)cur >= (uint64_t)P.num_nodes) {
    raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
    parked = true;
  }
  for (int64_t l = 0; l < L; l++) {
    int64_t e = -1;
    if (!parked) e = uniform_step<USE_DESC>(P, pol, cur, parked, __ldg(P.rand + w * L + l));
    out[l + 1] = cur;
    if (HAS_EOUT) P.e_out[w * L + l] = e;
  }
}

// Staged variant. A warp owns 32 consecutive walks, i.e. one contiguous span of rand
// and of the walk matrix. Steps are processed in chunks of S: the chunk's rand values
// are fetched as row segments (S consecutive floats per walk, lanes along the segment)
// into a shared tile, each lane then walks its S steps out of the tile, overwriting
// every consumed rand slot with the node it reached, and the tile is flushed as row
// segments of S consecutive int64. Global traffic on both sides is whole sectors; the
// only divergent accesses left per step are the row fetch and the col gather. The next
// chunk's rand is prefetched into registers while the current chunk walks.
// GEN: no rand array; lane w draws step l from the Philox stream of its global walk index
// (uniform_block / uniform_from_word), four steps per block, so nothing is read for the draws.
template <int S, int MIN_BLOCKS, bool USE_DESC, bool HAS_EOUT, bool FUSED = false, bool GEN = false>
__global__ void __launch_bounds__(kBlock, MIN_BLOCKS) uniform_walk_staged_kernel(const UniformParams P) {
  static_assert(!FUSED || USE_DESC, "fused edge records carry row descriptors");
  static_assert(S % 4 == 0, "a Philox block serves four steps");
  constexpr int kPitch = 33;  // 8-byte slots per tile row: 32 lanes + 1 pad
  __shared__ unsigned long long tiles[kWarpsPerBlock][S][kPitch];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  unsigned long long (*tile)[kPitch] = tiles[wib];
  const int64_t w0 = ((int64_t)blockIdx.x * kWarpsPerBlock + wib) * 32;
  if (w0 >= P.num_walks) return;  // whole warp leaves together
  const L2Policy pol = make_policies(P.hints);
  const int64_t L = P.walk_length;
  const int nw = (int)min((int64_t)32, P.num_walks - w0);
  const bool live = lane < nw;
  const int64_t w = w0 + lane;

  int64_t cur = 0;
  int64_t cur_rs = 0, cur_deg = 0;  // FUSED: row bounds of cur travel with the lane
  bool parked = !live;
  if (live) {
    cur = P.start[w];
    P.n_out[w * (L + 1)] = cur;
    if ((uint64_t)cur >= (uint64_t)P.num_nodes) {
      raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
      parked = true;
    } else if (FUSED) {
      load_row<true>(P.rowptr, P.desc, cur, pol.keep, cur_rs, cur_deg);
    }
  }

  const float* rand_span = P.rand + w0 * L;           // [nw, L] contiguous
  int64_t* out_span = P.n_out + w0 * (L + 1);          // [nw, L+1] contiguous
  int64_t* eout_span = HAS_EOUT ? P.e_out + w0 * L : nullptr;

  // Element k*32+lane of a chunk maps to (walk wi = idx / sc, step j = idx % sc).
  uint32_t pre[S];
  auto prefetch = [&](int64_t l0) {
    const int sc = (int)min((int64_t)S, L - l0);
    const int total = nw * sc;
#pragma unroll
    for (int k = 0; k < S; k++) {
      const int idx = k * 32 + lane;
      uint32_t bits = 0;
      if (idx < total) {
        const int wi = (sc == S) ? idx / S : idx / sc;
        const int j = idx - wi * sc;
        bits = ld4(rand_span + (int64_t)wi * L + l0 + j, pol.stream);
      }
      pre[k] = bits;
    }
  };

  const uint64_t gw = P.walk_index_base + (uint64_t)w * P.walk_index_stride;
  if (!GEN) prefetch(0);
  for (int64_t l0 = 0; l0 < L; l0 += S) {
    const int sc = (int)min((int64_t)S, L - l0);
    const int total = nw * sc;
    if (!GEN) {
#pragma unroll
      for (int k = 0; k < S; k++) {
        const int idx = k * 32 + lane;
        if (idx < total) {
          const int wi = (sc == S) ? idx / S : idx / sc;
          const int j = idx - wi * sc;
          tile[j][wi] = pre[k];
        }
      }
      __syncwarp();
      if (l0 + S < L) prefetch(l0 + S);
    }
    if (live) {
      Philox4 blk = {0, 0, 0, 0};
      for (int j = 0; j < sc; j++) {
        int64_t e = -1;
        if (!parked) {
          float r;
          if (GEN) {
            if ((j & 3) == 0) blk = uniform_block(P.key0, P.key1, gw, (uint32_t)((l0 + j) >> 2));
            const uint32_t word = (j & 3) == 0 ? blk.x : (j & 3) == 1 ? blk.y : (j & 3) == 2 ? blk.z : blk.w;
            r = uniform_from_word(word);
          } else {
            r = __uint_as_float((uint32_t)tile[j][lane]);
          }
          e = FUSED ? uniform_step_fused(P, pol, cur, cur_rs, cur_deg, parked, r)
                    : uniform_step<USE_DESC>(P, pol, cur, parked, r);
        }
        tile[j][lane] = (unsigned long long)cur;
        if (HAS_EOUT) eout_span[(int64_t)lane * L + l0 + j] = e;
      }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < S; k++) {
      const int idx = k * 32 + lane;
      if (idx < total) {
        const int wi = (sc == S) ? idx / S : idx / sc;
        const int j = idx - wi * sc;
        st8(out_span + (int64_t)wi * (L + 1) + 1 + l0 + j, (int64_t)tile[j][wi], pol.stream);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------
// edge hash set: exact membership "is (x -> t) an edge" in about one 32-byte probe
// ---------------------------------------------------------------------------------
// Open addressing over buckets of 4 x 8-byte slots (one 32-byte sector, aligned);
// key = (x << 32) | t, empty = all ones. A key lives in the first bucket of its probe
// sequence that had room when it was inserted, so a lookup may stop at the first bucket
// that still has an empty slot. Load factor <= 0.5 by construction of the table size.
constexpr uint64_t kEdgeEmpty = ~0ull;
constexpr int kEdgeSlotsPerBucket = 4;
constexpr int kEdgeMaxProbe = 4096;  // buckets; far beyond anything a half-full table produces

__host__ __device__ __forceinline__ uint64_t edge_key(uint64_t x, uint64_t t) { return (x << 32) | t; }

__device__ __forceinline__ uint64_t edge_bucket(uint64_t key, uint64_t num_buckets) {
  uint64_t z = key;
  z ^= z >> 30; z *= 0xbf58476d1ce4e5b9ull;
  z ^= z >> 27; z *= 0x94d049bb133111ebull;
  z ^= z >> 31;
  return __umul64hi(z, num_buckets);
}

__global__ void __launch_bounds__(kBlock) edgeset_build_kernel(const int64_t* __restrict__ rowptr,
                                                               const int64_t* __restrict__ col,
                                                               int64_t num_nodes, int64_t num_edges,
                                                               unsigned long long* __restrict__ table,
                                                               uint64_t num_buckets, uint32_t* flags) {
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t e = (int64_t)blockIdx.x * kBlock + threadIdx.x; e < num_edges; e += stride) {
    // source row of edge e: last v with rowptr[v] <= e
    int64_t lo = 0, hi = num_nodes;
    while (hi - lo > 1) {
      const int64_t mid = lo + (hi - lo) / 2;
      if (__ldg(rowptr + mid) <= e) lo = mid; else hi = mid;
    }
    const int64_t t = __ldg(col + e);
    if ((uint64_t)t >= (uint64_t)num_nodes) { raise_flag(flags, WALK_B200_FLAG_BAD_NODE); continue; }
    const uint64_t key = edge_key((uint64_t)lo, (uint64_t)t);
    uint64_t b = edge_bucket(key, num_buckets);
    bool placed = false;
    for (int probe = 0; probe < kEdgeMaxProbe && !placed; probe++) {
      unsigned long long* slot = table + b * kEdgeSlotsPerBucket;
#pragma unroll
      for (int k = 0; k < kEdgeSlotsPerBucket && !placed; k++) {
        const unsigned long long old = atomicCAS(slot + k, kEdgeEmpty, key);
        if (old == kEdgeEmpty || old == key) placed = true;
      }
      if (++b == num_buckets) b = 0;
    }
    if (!placed) raise_flag(flags, WALK_B200_FLAG_EDGESET_FULL);
  }
}

// ---------------------------------------------------------------------------------
// reverse positions: revpos[e] for edge e = (u -> v) is the index in col of (v -> u)
// ---------------------------------------------------------------------------------
// With it a node2vec step knows, without touching col, whether a drawn edge leads back to
// the previous node. Needs rows strictly ascending (binary search, and "x == t" must mean
// "this very edge"); a violation raises WALK_B200_FLAG_UNSORTED_ROW and the array must not
// be used. kNoEdge marks edges without a reverse.
constexpr uint32_t kNoEdge = 0xffffffffu;       // the reverse edge does not exist
constexpr uint32_t kUnknownEdge = 0xfffffffeu;  // not looked up: the shortcut must not be taken

__global__ void __launch_bounds__(kBlock) revpos_build_kernel(const int64_t* __restrict__ rowptr,
                                                              const int64_t* __restrict__ col,
                                                              int64_t num_nodes, int64_t num_edges,
                                                              uint32_t* __restrict__ revpos, uint32_t* flags) {
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t e = (int64_t)blockIdx.x * kBlock + threadIdx.x; e < num_edges; e += stride) {
    int64_t lo = 0, hi = num_nodes;  // source row u of edge e: last u with rowptr[u] <= e
    while (hi - lo > 1) {
      const int64_t mid = lo + (hi - lo) / 2;
      if (__ldg(rowptr + mid) <= e) lo = mid; else hi = mid;
    }
    const int64_t u = lo;
    const int64_t v = __ldg(col + e);
    uint32_t pos = kNoEdge;
    if ((uint64_t)v >= (uint64_t)num_nodes) {
      raise_flag(flags, WALK_B200_FLAG_BAD_NODE);
    } else {
      if (e > __ldg(rowptr + u) && __ldg(col + e - 1) >= v) raise_flag(flags, WALK_B200_FLAG_UNSORTED_ROW);
      int64_t a = __ldg(rowptr + v), b = __ldg(rowptr + v + 1);
      while (a < b) {
        const int64_t mid = a + (b - a) / 2;
        const int64_t w = __ldg(col + mid);
        if (w == u) { pos = (uint32_t)mid; break; }
        if (w < u) a = mid + 1; else b = mid;
      }
    }
    revpos[e] = pos;
  }
}

// ---------------------------------------------------------------------------------
// triangle filter: per directed edge, which positions of the target's row hold common neighbours
// ---------------------------------------------------------------------------------
// colrev16[e] = {colrev[e], filter(e)}. For e = (a -> b), bit k of filter(e) is set iff some w in N(a) & N(b)
// sits at a position p of b's row with p mod 64 == k: a walk that came from a and stands on b need not look at
// a candidate drawn at a position whose bit is clear to know that it is not a neighbour of a.
// Work is done once per undirected edge, from the end with the shorter row (ties: the smaller id): one warp
// walks that row, asks the edge hash set for each entry whether it is a neighbour of the other end, and for
// the hits sets the bit of the entry's position in its own row (filter of the edge back) and, after a binary
// search, of its position in the other end's row (filter of the edge itself). An edge whose shorter row
// exceeds max_row, a self-loop and an edge without a reverse keep the all-ones word the host wrote before the
// launch: no filtering. Warps take chunks of 64 edges from a counter.
__device__ __forceinline__ bool edge_lookup(const uint64_t* __restrict__ table, uint64_t num_buckets, uint64_t key) {
  uint64_t b = edge_bucket(key, num_buckets);
  for (int probe = 0; probe < kEdgeMaxProbe; probe++) {
    const ulonglong2 h0 = ld16(table + b * kEdgeSlotsPerBucket, 0), h1 = ld16(table + b * kEdgeSlotsPerBucket + 2, 0);
    if (h0.x == key || h0.y == key || h1.x == key || h1.y == key) return true;
    if (h0.x == kEdgeEmpty || h0.y == kEdgeEmpty || h1.x == kEdgeEmpty || h1.y == kEdgeEmpty) return false;
    if (++b == num_buckets) b = 0;
  }
  return true;  // a chain that long does not occur in a table at most half full; "maybe" is the safe answer
}

__global__ void __launch_bounds__(kBlock) trifilter_build_kernel(const int64_t* __restrict__ rowptr,
                                                                 const int64_t* __restrict__ col,
                                                                 const uint64_t* __restrict__ colrev,
                                                                 const uint64_t* __restrict__ edgeset, uint64_t edgeset_buckets,
                                                                 int64_t num_nodes, int64_t num_edges, int64_t max_row,
                                                                 ulonglong2* __restrict__ colrev16,
                                                                 unsigned long long* queue) {
  constexpr unsigned kFull = 0xffffffffu;
  constexpr int64_t kChunk = 64;
  const int lane = threadIdx.x & 31;
  while (true) {
    unsigned long long chunk = 0;
    if (lane == 0) chunk = atomicAdd(queue, 1ull);
    chunk = __shfl_sync(kFull, chunk, 0);
    const int64_t e0 = (int64_t)chunk * kChunk;
    if (e0 >= num_edges) break;
    const int64_t e1 = min(e0 + kChunk, num_edges);
    // source row of e0: last a with rowptr[a] <= e0; later edges of the chunk move on from there
    int64_t lo = 0, hi = num_nodes;
    while (hi - lo > 1) {
      const int64_t mid = lo + (hi - lo) / 2;
      if (__ldg(rowptr + mid) <= e0) lo = mid; else hi = mid;
    }
    int64_t a = lo;
    int64_t a_end = __ldg(rowptr + a + 1);
    for (int64_t e = e0; e < e1; e++) {
      while (e >= a_end) { a++; a_end = __ldg(rowptr + a + 1); }
      const uint64_t cr = colrev[e];
      if (lane == 0) colrev16[e].x = cr;
      const int64_t b = (int64_t)(cr & 0xffffffffull);
      const uint32_t rev = (uint32_t)(cr >> 32);
      if (rev >= 0xfffffffeu || b == a || (uint64_t)b >= (uint64_t)num_nodes) continue;  // no edge back, or a self-loop
      const int64_t a_rs = __ldg(rowptr + a), b_rs = __ldg(rowptr + b);
      const int64_t da = a_end - a_rs, db = __ldg(rowptr + b + 1) - b_rs;
      if (!(da < db || (da == db && a < b))) continue;  // done from the other end
      if (max_row > 0 && da > max_row) continue;
      unsigned long long here = 0, there = 0;  // bits of positions in a's row / in b's row
      for (int64_t i = lane; i < da; i += 32) {
        const int64_t w = __ldg(col + a_rs + i);
        if (!edge_lookup(edgeset, edgeset_buckets, edge_key((uint64_t)b, (uint64_t)w))) continue;
        here |= 1ull << (i & 63);
        int64_t p = b_rs, q = b_rs + db;  // position of w in b's row (it is there: the set just said so)
        while (p < q) {
          const int64_t mid = p + (q - p) / 2;
          const int64_t c = __ldg(col + mid);
          if (c == w) { there |= 1ull << ((mid - b_rs) & 63); break; }
          if (c < w) p = mid + 1; else q = mid;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        here |= __shfl_xor_sync(kFull, here, o);
        there |= __shfl_xor_sync(kFull, there, o);
      }
      if (lane == 0) {
        colrev16[e].y = there;    // standing on b, came from a: candidates are positions of b's row
        colrev16[rev].y = here;   // standing on a, came from b
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// node2vec walk
// ---------------------------------------------------------------------------------
struct Node2vecParams {
  const int64_t* rowptr;
  const int64_t* col;
  const uint64_t* desc;
  const uint64_t* edgeset;
  uint64_t edgeset_buckets;
  const uint64_t* colrev;  // REV kernels: col[e] | revpos[e] << 32
  const ulonglong2* colrev16;  // triangle-filter kernel: {colrev[e], filter word of e}
  int64_t num_nodes, num_edges;
  const int64_t* start;
  int64_t num_walks;
  int32_t walk_length;
  int32_t hints;
  uint32_t cut0, cut1, cut2;  // accept31 < cut_k  <=>  r < prob_k
  uint32_t key0, key1;
  uint64_t walk_index_base;
  uint64_t walk_index_stride;
  uint32_t max_attempts;
  int32_t batch_lanes, batch_trips;  // batching of the rare state paths (see the kernel)
  int32_t draw_loop;                 // REV: memory-free rejections consumed per trip
  int64_t* n_out;
  int64_t* e_out;
  uint32_t* flags;
  unsigned long long* counters;
  unsigned long long* queue;  // launch-wide chunk counter, zero at launch
  // HOST kernels only (HOST_NARROW: n_out / e_out point at int32 matrices): finished walks are counted per slab of
  // 2^slab_shift consecutive rows in slab_done (zero at launch); the walk that completes a slab sets
  // slab_flags[slab] (mapped host memory), after which the host may copy that slab's rows out while
  // the launch goes on.
  int32_t slab_shift;
  uint32_t* slab_done;
  volatile uint32_t* slab_flags;
};

enum : int { ST_IDLE = 0, ST_START, ST_ROW, ST_ACCEPTED, ST_ATTEMPT, ST_XROW, ST_SEARCH, ST_HASH };
enum : int { MEMBER_SEARCH_PREV = 0, MEMBER_SEARCH_CAND = 1, MEMBER_HASH = 2 };
// HOST template argument of the node2vec kernels: the single-launch mode of the host-buffer entry point.
// HOST_NARROW: the matrices are int32 (ids fit; half the bytes cross the bus, host threads widen them);
// HOST_WIDE: int64, copied straight into the caller's buffer. Both count finished walks per slab.
enum : int { HOST_NONE = 0, HOST_NARROW = 1, HOST_WIDE = 2 };

// Persistent warps; one walk per lane; one gather per loop trip whatever the lane is doing.
//   ST_START     fetch the start node of a freshly assigned walk
//   ST_ROW       fetch the bounds of the current node's row (REV: and the reverse position)
//   ST_ACCEPTED  a step was decided: write it, advance, then continue as ST_ROW in the same trip
//   ST_ATTEMPT   draw a candidate edge (Philox), classify it, gather col[e] if needed
//   ST_XROW      (MEMBER_SEARCH_CAND) fetch the bounds of the candidate's row
//   ST_SEARCH    one binary-search probe of the membership test
//   ST_HASH      (MEMBER_HASH) one 32-byte bucket of the edge hash set
// A warp executes the union of the paths its lanes are on, so a path that only one or two
// lanes need costs as many issue slots as one all 32 need. The draw path (ST_ATTEMPT) is by far
// the most frequent; the others are rare per lane but almost always present somewhere in the
// warp. They are therefore batched: lanes that reach ST_HASH, or ST_ACCEPTED/ST_ROW/ST_START,
// wait in that state until batch_lanes lanes of the warp are there (or batch_trips trips have
// passed, or no lane has heavy work), and then the path runs once for all of them. Most trips
// execute the draw path alone.
// A lane whose walk ends takes the next unassigned walk of its warp's current chunk of
// 32; a warp whose chunk is used up takes the next chunk from a launch-wide counter
// (one atomicAdd per 32 walks). Walk cost varies by orders of magnitude (isolated start:
// two trips; hub-heavy walk under strong rejection: thousands) and is tied to the bits
// of the start id on generated graphs, so any static deal of walks to warps leaves part
// of the machine idle for a good part of the launch. Draws are indexed by the walk's
// global row, so which lane runs which walk does not change any result.
// The membership test is only entered when it can change the outcome: the accept draw
// is already known to be >= cut2 (not accepted outright), not accepted by the
// return-to-previous rule, and < cut1. MEMBER_SEARCH_PREV (undirected graphs) searches
// the candidate x in the previous node's sorted row; MEMBER_SEARCH_CAND searches the
// previous node t in the candidate's row, as the reference's is_neighbor(x, t) does;
// MEMBER_HASH asks the edge hash set for (x -> t).
//
// REV (with MEMBER_HASH, row descriptors and 32-bit indices): the lane also carries ret_e, the
// index in col of the edge back to the previous node, and in_e, the index of the edge it arrived by.
// Candidates are gathered from colrev, whose upper half is the position of the edge back from the
// candidate: accepting it makes that the next ret_e. An attempt whose drawn edge is ret_e knows its
// candidate (x = t) without a gather, and accepting it just swaps ret_e and in_e; an attempt whose
// accept draw is >= cut1 can only be accepted by the return rule: if its edge is not ret_e it is
// rejected without touching memory at all. At (p, q) = (0.25, 4) that is three attempts in four.
// Same draws, same decisions, fewer gathers.
//
// HOST (the host-buffer entry point's single-launch mode): finished walks are counted per slab of
// 2^slab_shift rows, so the host can copy a slab out as soon as its last walk is done; with HOST_NARROW
// the walk and edge matrices are int32 (P.n_out / P.e_out point at int32 storage; the ids fit).
template <typename idx_t, int MEMBER, bool USE_DESC, bool HAS_EOUT, bool COUNT, bool REV = false, int HOST = HOST_NONE>
__global__ void __launch_bounds__(kBlock, COUNT ? 1 : 6) node2vec_walk_kernel(const Node2vecParams P) {
  static_assert(!REV || (MEMBER == MEMBER_HASH && USE_DESC && sizeof(idx_t) == 4), "REV needs hash membership, row descriptors, 32-bit indices");
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const L2Policy pol = make_policies(P.hints);
  const int32_t L = P.walk_length;
  const int64_t n = P.num_walks;
  const int64_t* __restrict__ col = P.col;

  // warp-uniform queue of walks: [q_next, q_end) of the current chunk of 32
  const int64_t n_chunks = (n + 31) / 32;
  int64_t q_next = 0, q_end = 0;  // empty: the first trip fetches a chunk
  bool drained = false;           // the launch-wide counter has run past the last chunk
  int wait_hash = 0, wait_row = 0;  // trips the batched paths have been held back

  uint32_t c_loads = 0, c_attempts = 0, c_member = 0, c_probes = 0, c_formula = 0;
  uint32_t c_deg0 = 0, c_deg1 = 0, c_sampled = 0, c_first = 0;

  int64_t i = 0;                  // walk (row of this launch) the lane is working on
  idx_t t = 0, v = 0, x = 0;      // previous node, current node, candidate
  idx_t v_rs = 0, v_re = 0;       // row [start, end) of v
  idx_t t_rs = 0, t_re = 0;       // row [start, end) of t (MEMBER_SEARCH_PREV range)
  uint32_t v_deg = 0;             // degree of v saturated at 2^31 (enough for "u % deg" with 31-bit u)
  uint32_t v_inv = 0;             // floor((2^32 - 1) / v_deg): "u % v_deg" as a multiply and one fix-up
  using uidx_t = typename std::conditional<sizeof(idx_t) == 4, uint32_t, uint64_t>::type;
  uidx_t lo = 0, hi = 0;          // search window / hash bucket + probe count / parked accept draw
  idx_t e = 0;                    // sampled edge index
  idx_t ret_e = (idx_t)kUnknownEdge;  // REV: index of the edge v -> t (kNoEdge: there is none)
  idx_t in_e = (idx_t)kUnknownEdge;   // REV: index of the edge t -> v the walk arrived by
  uint32_t x_rev = kUnknownEdge;      // REV: index of the edge x -> v, gathered with the candidate x
  int32_t l = 0;                  // step being produced
  uint32_t a = 0;                 // attempt counter of this step
  int state = ST_IDLE;
  bool finished = false;          // the lane completed a walk in the last trip (progress reporting)

  auto put_node = [&](int64_t row, int32_t k, int64_t node) {
    if (HOST == HOST_NARROW) reinterpret_cast<int32_t*>(P.n_out)[row * ((int64_t)L + 1) + k] = (int32_t)node;
    else st8(P.n_out + row * ((int64_t)L + 1) + k, node, pol.stream);
  };
  auto put_edge = [&](int64_t row, int32_t k, int64_t edge) {
    if (HOST == HOST_NARROW) reinterpret_cast<int32_t*>(P.e_out)[row * (int64_t)L + k] = (int32_t)edge;
    else P.e_out[row * (int64_t)L + k] = edge;
  };

  while (true) {
    // ---- progress reporting: a finished walk's rows are made visible, then counted for its slab
    if (HOST && finished) {
      __threadfence();
      const int64_t slab = i >> P.slab_shift;
      const int64_t rows_in_slab = min((int64_t)1 << P.slab_shift, n - (slab << P.slab_shift));
      if ((int64_t)atomicAdd(P.slab_done + slab, 1u) + 1 == rows_in_slab) {
        __threadfence_system();
        P.slab_flags[slab] = 1u;
      }
    }
    if (HOST) finished = false;

    // ---- hand walks to idle lanes (all lanes of the warp pass here together)
    const unsigned idle = __ballot_sync(kFull, state == ST_IDLE);
    if (idle) {
      if (q_next >= q_end && !drained) {  // chunk used up: take the next one of the launch
        unsigned long long chunk = 0;
        if (lane == 0) chunk = atomicAdd(P.queue, 1ull);
        chunk = __shfl_sync(kFull, chunk, 0);
        if ((int64_t)chunk < n_chunks) {
          q_next = (int64_t)chunk * 32;
          q_end = min(q_next + 32, n);
        } else {
          drained = true;
        }
      }
      if (q_next < q_end) {
        const int avail = (int)(q_end - q_next);
        const int rank = __popc(idle & ((1u << lane) - 1u));
        if (state == ST_IDLE && rank < avail) {
          i = q_next + rank;
          state = ST_START;
        }
        q_next += min(__popc(idle), avail);
      } else if (idle == kFull) {
        break;  // nothing left to hand out and nobody is working
      }
    }

    // ---- which batched paths run this trip (warp-uniform decisions)
    const bool heavy = state == ST_ATTEMPT || state == ST_SEARCH || state == ST_XROW;
    const bool in_hash = state == ST_HASH;
    const bool in_row = state == ST_ROW || state == ST_ACCEPTED || state == ST_START;
    const unsigned m_heavy = __ballot_sync(kFull, heavy);
    const unsigned m_hash = __ballot_sync(kFull, in_hash);
    const unsigned m_row = __ballot_sync(kFull, in_row);
    bool go_hash = false, go_row = false;
    if (m_hash) {
      go_hash = __popc(m_hash) >= P.batch_lanes || !m_heavy || ++wait_hash >= P.batch_trips;
      if (go_hash) wait_hash = 0;
    }
    if (m_row) {
      go_row = __popc(m_row) >= P.batch_lanes || !m_heavy || ++wait_row >= P.batch_trips;
      if (go_row) wait_row = 0;
    }

    if (heavy || (in_hash && go_hash) || (in_row && go_row)) {
      bool accept = false, reject = false;
      bool need_load = true;  // REV: some attempts are decided without touching memory

      if (state == ST_ACCEPTED) {  // write the decided step, advance, go on to the next row fetch
        put_node(i, l + 1, (int64_t)x);
        if (HAS_EOUT) put_edge(i, l, (a >= P.max_attempts) ? -1 : (int64_t)e);
        if (REV) {
          if (e == (idx_t)kUnknownEdge) { ret_e = (idx_t)kUnknownEdge; in_e = (idx_t)kUnknownEdge; }  // stood still
          else if (e == ret_e) { const idx_t back = ret_e; ret_e = in_e; in_e = back; }              // went back
          else { in_e = e; ret_e = (idx_t)x_rev; }
        }
        t = v; t_rs = v_rs; t_re = v_re;
        v = x;
        l++;
        if (l == L) { state = ST_IDLE; finished = true; need_load = false; }
        else state = ST_ROW;
      }

      // ---- address of this trip's gather
      const void* addr = nullptr;
      uint64_t policy = pol.stream;
      if (state == ST_START) {
        addr = P.start + i;
      } else if (state == ST_ROW) {
        addr = USE_DESC ? (const void*)(P.desc + (int64_t)v) : (const void*)(P.rowptr + (int64_t)v);
        policy = pol.keep;
      } else if (state == ST_ATTEMPT) {
        if (v_deg == 1) {
          e = v_rs;  // forced move: no draw (deg-1 shortcut of the reference; also exact at step 0)
        } else {
          // REV: attempts that are rejected without touching memory (not the way back, accept draw
          // above cut1 and cut2) are consumed right here, up to draw_loop of them per trip, instead
          // of costing a whole trip of the state machine each.
          const uint64_t gw = P.walk_index_base + (uint64_t)i * P.walk_index_stride;
          const bool may_skip = REV && l > 0 && ret_e != (idx_t)kUnknownEdge;
          uint32_t cand, acc;
          for (int k = 1;; k++) {
            node2vec_draw(P.key0, P.key1, gw, (uint32_t)l, a, cand, acc);
            // cand % v_deg, exactly: the quotient estimate is at most one too small for a 31-bit cand
            uint32_t rem = cand - __umulhi(cand, v_inv) * v_deg;
            if (rem >= v_deg) rem -= v_deg;
            e = v_rs + (idx_t)rem;
            if (!may_skip || e == ret_e || acc < P.cut2 || acc < P.cut1) break;
            if (k >= P.draw_loop || a + 1 >= P.max_attempts) break;  // leave it to the regular path below
            if (COUNT) c_attempts++;
            a++;
          }
          lo = acc;  // parked until the candidate arrives
        }
        addr = REV ? (const void*)(P.colrev + (int64_t)e) : (const void*)(col + (int64_t)e);
        if (REV && l > 0 && ret_e != (idx_t)kUnknownEdge) {
          const bool is_ret = (e == ret_e);
          if (v_deg == 1) {
            if (is_ret) { x = t; accept = true; need_load = false; }
          } else {
            const uint32_t acc = (uint32_t)lo;
            if (is_ret) {  // the candidate is the previous node: no gather needed to know it
              need_load = false;
              x = t;
              if (COUNT) c_attempts++;
              if (acc < P.cut2 || acc < P.cut0) accept = true;
              else if (acc < P.cut1) {  // only a self-loop t -> t could still accept: ask the edge set
                if (COUNT) { c_member++; state = ST_XROW; }
                else { lo = (uidx_t)edge_bucket(edge_key((uint64_t)x, (uint64_t)t), P.edgeset_buckets); hi = 0; state = ST_HASH; }
              } else reject = true;
            } else if (acc >= P.cut2 && acc >= P.cut1) {  // not the way back and too large for the other rules
              need_load = false;
              if (COUNT) c_attempts++;
              reject = true;
            }
          }
        }
      } else if (state == ST_XROW) {
        addr = USE_DESC ? (const void*)(P.desc + (int64_t)x) : (const void*)(P.rowptr + (int64_t)x);
        policy = pol.keep;
      } else if (state == ST_SEARCH) {
        addr = col + (int64_t)(lo + (hi - lo) / 2);
        policy = pol.normal;  // upper levels of a hub row's search tree are shared by many walks
      } else if (state == ST_HASH) {
        addr = P.edgeset + (uint64_t)lo * kEdgeSlotsPerBucket;
      }

      int64_t val = 0, val2 = 0;
      ulonglong2 h0 = {0, 0}, h1 = {0, 0};
      if (!need_load) {
        // decided above
      } else if (MEMBER == MEMBER_HASH && state == ST_HASH) {
        h0 = ld16(addr, policy);
        h1 = ld16((const char*)addr + 16, policy);
        if (COUNT) c_loads += 4;
      } else {
        val = ld8(addr, policy);
        const bool pair = !USE_DESC && (state == ST_ROW || state == ST_XROW);
        if (pair) val2 = ld8((const char*)addr + 8, policy);
        // the instrumented kernel's extra look at deg(x) is bookkeeping, not part of the walk
        const bool bookkeeping = COUNT && state == ST_XROW && MEMBER != MEMBER_SEARCH_CAND;
        if (COUNT && !bookkeeping) c_loads += pair ? 2 : 1;
        if (REV && state == ST_ATTEMPT) {
          x_rev = (uint32_t)((uint64_t)val >> 32);
          val = (int64_t)((uint64_t)val & 0xffffffffull);
        }
      }

      // ---- consume it
      if (!need_load) {
        // nothing was loaded
      } else if (state == ST_START) {
        put_node(i, 0, val);
        t = (idx_t)val;
        v = (idx_t)val;
        l = 0;
        if (REV) { ret_e = (idx_t)kUnknownEdge; in_e = (idx_t)kUnknownEdge; }
        if ((uint64_t)val >= (uint64_t)P.num_nodes) {
          raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
          for (int32_t k = 0; k < L; k++) { put_node(i, k + 1, val); if (HAS_EOUT) put_edge(i, k, -1); }
          state = ST_IDLE;
          finished = true;
        } else if (L > 0) {
          state = ST_ROW;
        } else {
          state = ST_IDLE;
          finished = true;
        }
      } else if (state == ST_ROW || state == ST_XROW) {
        int64_t rs, deg;
        if (USE_DESC) { rs = (int64_t)((uint64_t)val & kDescStartMask); deg = (int64_t)((uint64_t)val >> kDescStartBits); }
        else { rs = val; deg = val2 - val; }
        if (deg < 0 || rs < 0 || rs + deg > P.num_edges) { raise_flag(P.flags, WALK_B200_FLAG_BAD_ROWPTR); deg = 0; }
        if (state == ST_ROW) {
          if (deg == 0) {
            // stay in place for every remaining step
            if (COUNT) c_deg0 += (uint32_t)(L - l);
            for (int32_t k = l; k < L; k++) { put_node(i, k + 1, (int64_t)v); if (HAS_EOUT) put_edge(i, k, -1); }
            state = ST_IDLE;
            finished = true;
          } else {
            v_rs = (idx_t)rs;
            v_re = (idx_t)(rs + deg);
            v_deg = deg > 0x7fffffffll ? 0x80000000u : (uint32_t)deg;
            v_inv = 0xffffffffu / v_deg;
            a = 0;
            state = ST_ATTEMPT;
            if (COUNT) { if (l == 0) c_first++; else if (deg == 1) c_deg1++; else c_sampled++; }
          }
        } else {  // ST_XROW: bounds of the candidate's row
          if (COUNT && P.counters) {  // formula term of this membership test: ceil(log2(deg(x) + 1))
            uint32_t bits = 0;
            while ((1ull << bits) < (uint64_t)deg + 1) bits++;
            c_formula += bits;
          }
          if (MEMBER == MEMBER_SEARCH_CAND) {
            lo = (uidx_t)rs; hi = (uidx_t)(rs + deg);
            if (lo < hi) state = ST_SEARCH; else reject = true;
          } else if (MEMBER == MEMBER_SEARCH_PREV) {  // only reached in the instrumented kernel
            lo = (uidx_t)t_rs; hi = (uidx_t)t_re;
            if (lo < hi) state = ST_SEARCH; else reject = true;
          } else {
            lo = (uidx_t)edge_bucket(edge_key((uint64_t)x, (uint64_t)t), P.edgeset_buckets);
            hi = 0;
            state = ST_HASH;
          }
        }
      } else if (state == ST_ATTEMPT) {
        if ((uint64_t)val >= (uint64_t)P.num_nodes) {
          raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
          val = (int64_t)v;  // park on the current node
          if (REV) x_rev = kUnknownEdge;
        }
        x = (idx_t)val;
        if (l == 0 || v_deg == 1) {
          accept = true;
        } else {
          if (COUNT) c_attempts++;
          const uint32_t acc = (uint32_t)lo;
          if (acc < P.cut2) accept = true;
          else if (x == t && acc < P.cut0) accept = true;
          else if (acc < P.cut1) {
            if (COUNT) c_member++;
            if (COUNT || MEMBER == MEMBER_SEARCH_CAND) {
              state = ST_XROW;  // the instrumented kernel always looks at deg(x) for the byte formula
            } else if (MEMBER == MEMBER_SEARCH_PREV) {
              lo = (uidx_t)t_rs; hi = (uidx_t)t_re;
              if (lo < hi) state = ST_SEARCH; else reject = true;
            } else {
              lo = (uidx_t)edge_bucket(edge_key((uint64_t)x, (uint64_t)t), P.edgeset_buckets);
              hi = 0;
              state = ST_HASH;
            }
          } else reject = true;
        }
      } else if (state == ST_SEARCH) {
        if (COUNT) c_probes++;
        const uidx_t mid = lo + (hi - lo) / 2;
        const int64_t key = MEMBER == MEMBER_SEARCH_PREV ? (int64_t)x : (int64_t)t;
        if (val == key) accept = true;       // member, and the draw is known to be < cut1
        else {
          if (val < key) lo = mid + 1; else hi = mid;
          if (!(lo < hi)) reject = true;     // not a member, and the draw is known to be >= cut2
        }
      } else if (state == ST_HASH) {
        if (COUNT) c_probes++;
        const uint64_t key = edge_key((uint64_t)x, (uint64_t)t);
        if (h0.x == key || h0.y == key || h1.x == key || h1.y == key) accept = true;
        else if (h0.x == kEdgeEmpty || h0.y == kEdgeEmpty || h1.x == kEdgeEmpty || h1.y == kEdgeEmpty) reject = true;
        else {
          if (++lo == P.edgeset_buckets) lo = 0;
          if (++hi >= (uidx_t)kEdgeMaxProbe) { raise_flag(P.flags, WALK_B200_FLAG_EDGESET_FULL); reject = true; }
        }
      }

      if (reject) {
        a++;
        state = ST_ATTEMPT;
        if (a >= P.max_attempts) {
          raise_flag(P.flags, WALK_B200_FLAG_ATTEMPT_CAP);
          x = v; accept = true;  // give up on this step: stand still
          if (REV) e = (idx_t)kUnknownEdge;
        }
      }
      if (accept) state = ST_ACCEPTED;  // written and advanced when the row path next runs
    }
  }

  if (COUNT) {
    uint32_t c[WALK_B200_COUNTER_COUNT];
    c[WALK_B200_CNT_LOADS] = c_loads; c[WALK_B200_CNT_ATTEMPTS] = c_attempts;
    c[WALK_B200_CNT_MEMBERSHIP] = c_member; c[WALK_B200_CNT_PROBES] = c_probes;
    c[WALK_B200_CNT_STEPS_DEG0] = c_deg0; c[WALK_B200_CNT_STEPS_DEG1] = c_deg1;
    c[WALK_B200_CNT_STEPS_SAMPLED] = c_sampled; c[WALK_B200_CNT_STEPS_FIRST] = c_first;
    c[WALK_B200_CNT_FORMULA_PROBES] = c_formula;
#pragma unroll
    for (int k = 0; k < WALK_B200_COUNTER_COUNT; k++) {
      unsigned long long s = c[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
      if (lane == 0 && s) atomicAdd(P.counters + k, s);
    }
  }
}

// ---------------------------------------------------------------------------------
// context windows: the step after the walks in a node2vec pipeline
// ---------------------------------------------------------------------------------
// windows[(w * nwin + j) * cs + k] = walks[w * (L + 1) + j + k], nwin = L + 2 - cs: every run of cs
// consecutive nodes of every walk (first column = centre node, the rest = its skip-gram context).
// Streaming: each thread produces two adjacent output elements (one 16-byte store); the reads of
// neighbouring threads overlap and are served by L1. 64-bit index arithmetic is done once per
// walk row (blockIdx.y strides over walks), 32-bit inside a row.
// FAST_DIV: f / cs as a multiply-high with magic = floor(2^32 / cs) + 1, exact for every f the
// launch can produce (the host checks per_walk * (magic * cs - 2^32) < 2^32 before choosing it).
template <bool FAST_DIV>
__global__ void __launch_bounds__(kBlock) context_windows_kernel(const int64_t* __restrict__ walks,
                                                                 int64_t num_walks, int32_t row_len,
                                                                 int32_t cs, uint32_t magic, int32_t per_walk,
                                                                 int64_t* __restrict__ windows, bool base_aligned) {
  const L2Policy pol = make_policies(2);  // the windows stream out once: evict-first
  for (int64_t w = blockIdx.y; w < num_walks; w += gridDim.y) {
    const int64_t* __restrict__ row = walks + w * row_len;
    int64_t* __restrict__ out = windows + w * (int64_t)per_walk;
    // 16-byte alignment of this walk's output (base_aligned: the matrix itself starts on a 16-byte boundary)
    const bool aligned = base_aligned == (((w * (int64_t)per_walk) & 1) == 0);
    for (int32_t f = 2 * (blockIdx.x * kBlock + threadIdx.x); f < per_walk; f += 2 * gridDim.x * kBlock) {
      const int32_t j0 = FAST_DIV ? (int32_t)__umulhi((uint32_t)f, magic) : f / cs;
      const int32_t k0 = f - j0 * cs;
      const int64_t a = __ldg(row + j0 + k0);
      if (f + 1 < per_walk) {
        int32_t j1 = j0, k1 = k0 + 1;
        if (k1 == cs) { j1++; k1 = 0; }
        const int64_t b = __ldg(row + j1 + k1);
        if (aligned) {
          asm volatile("st.global.L2::cache_hint.v2.b64 [%0], {%1, %2}, %3;" ::"l"(out + f), "l"(a), "l"(b), "l"(pol.stream) : "memory");
        } else {
          st8(out + f, a, pol.stream);
          st8(out + f + 1, b, pol.stream);
        }
      } else {
        st8(out + f, a, pol.stream);
      }
    }
  }
}

// Negative rows for the skip-gram loss: out[r, 0] = start[r], out[r, 1 + k] = a node drawn uniformly
// from [0, num_nodes). One thread per Philox block = four consecutive draws of one row; consecutive
// threads write consecutive 32-byte pieces of a row.
__global__ void __launch_bounds__(kBlock) negative_walks_kernel(const int64_t* __restrict__ start, int64_t num_rows,
                                                                int32_t L, uint32_t quads_per_row, uint64_t num_nodes,
                                                                uint32_t key0, uint32_t key1, uint64_t row_base,
                                                                uint64_t row_stride, int64_t* __restrict__ out) {
  const L2Policy pol = make_policies(2);
  const int64_t total = num_rows * (int64_t)quads_per_row;
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t t = (int64_t)blockIdx.x * kBlock + threadIdx.x; t < total; t += stride) {
    const int64_t r = t / quads_per_row;
    const uint32_t quad = (uint32_t)(t - r * quads_per_row);
    int64_t* row = out + r * ((int64_t)L + 1);
    if (quad == 0) st8(row, __ldg(start + r), pol.stream);
    if (L == 0) continue;
    const Philox4 b = negative_block(key0, key1, row_base + (uint64_t)r * row_stride, quad);
    const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int32_t draw = (int32_t)(quad * 4u) + k;
      if (draw < L) st8(row + 1 + draw, negative_from_word(w[k], num_nodes), pol.stream);
    }
  }
}

// Narrow transport of the host entry points: int64 ids that fit 32 bits are packed to int32 before
// they cross PCIe. Four elements per thread and trip (two 16-byte loads, one 16-byte store); both
// arrays start on 16-byte boundaries, the tail goes element by element.
__global__ void __launch_bounds__(kBlock) narrow_i64_kernel(const int64_t* __restrict__ in, int64_t count,
                                                            int32_t* __restrict__ out) {
  const int64_t quads = count >> 2;
  const int64_t stride = (int64_t)gridDim.x * kBlock;
  for (int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x; i < quads; i += stride) {
    const longlong2 a = __ldcs(reinterpret_cast<const longlong2*>(in) + 2 * i);
    const longlong2 b = __ldcs(reinterpret_cast<const longlong2*>(in) + 2 * i + 1);
    reinterpret_cast<int4*>(out)[i] = make_int4((int32_t)a.x, (int32_t)a.y, (int32_t)b.x, (int32_t)b.y);
  }
  const int64_t tail = (quads << 2) + (int64_t)blockIdx.x * kBlock + threadIdx.x;
  if (tail < count) out[tail] = (int32_t)in[tail];
}

}  // namespace walk_b200
