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

// Row bounds of node v: one 8-byte load when a packed descriptor exists.
template <bool USE_DESC>
__device__ __forceinline__ void load_row(const int64_t* __restrict__ rowptr,
                                         const uint64_t* __restrict__ desc, int64_t v,
                                         int64_t& row_start, int64_t& deg) {
  if (USE_DESC) {
    const uint64_t d = __ldg(desc + v);
    row_start = (int64_t)(d & kDescStartMask);
    deg = (int64_t)(d >> kDescStartBits);
  } else {
    const int64_t a = __ldg(rowptr + v);
    const int64_t b = __ldg(rowptr + v + 1);
    row_start = a;
    deg = b - a;
  }
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
struct UniformParams {
  const int64_t* rowptr;
  const int64_t* col;
  const uint64_t* desc;
  int64_t num_nodes, num_edges;
  const int64_t* start;
  const float* rand;
  int64_t num_walks;
  int32_t walk_length;
  int64_t* n_out;
  int64_t* e_out;
  uint32_t* flags;
};

// One uniform step from `cur` with draw r. Same float32 arithmetic as the reference:
// degree converted to float32 (round to nearest), float32 product, truncation.
template <bool USE_DESC>
__device__ __forceinline__ int64_t uniform_step(const UniformParams& P, int64_t& cur, float r) {
  int64_t rs, deg;
  load_row<USE_DESC>(P.rowptr, P.desc, cur, rs, deg);
  if (deg <= 0) {
    if (deg < 0) raise_flag(P.flags, WALK_B200_FLAG_BAD_ROWPTR);
    return -1;
  }
  const float prod = __fmul_rn(r, __ll2float_rn(deg));
  int64_t e = rs + __float2ll_rz(prod);
  if ((uint64_t)e >= (uint64_t)P.num_edges) {  // rand >= 1, NaN, negative, or corrupt rowptr
    raise_flag(P.flags, WALK_B200_FLAG_BAD_EDGE);
    e = e < 0 ? 0 : P.num_edges - 1;
  }
  const int64_t nxt = __ldg(P.col + e);
  if ((uint64_t)nxt >= (uint64_t)P.num_nodes) {
    raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);  // park: keep cur
  } else {
    cur = nxt;
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
    if (!parked) e = uniform_step<USE_DESC>(P, cur, __ldg(P.rand + w * L + l));
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
template <int S, bool USE_DESC, bool HAS_EOUT>
__global__ void __launch_bounds__(kBlock) uniform_walk_staged_kernel(const UniformParams P) {
  constexpr int kPitch = 33;  // 8-byte slots per tile row: 32 lanes + 1 pad
  __shared__ unsigned long long tiles[kWarpsPerBlock][S][kPitch];
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  unsigned long long (*tile)[kPitch] = tiles[wib];
  const int64_t w0 = ((int64_t)blockIdx.x * kWarpsPerBlock + wib) * 32;
  if (w0 >= P.num_walks) return;  // whole warp leaves together
  const int64_t L = P.walk_length;
  const int nw = (int)min((int64_t)32, P.num_walks - w0);
  const bool live = lane < nw;
  const int64_t w = w0 + lane;

  int64_t cur = 0;
  bool parked = !live;
  if (live) {
    cur = P.start[w];
    P.n_out[w * (L + 1)] = cur;
    if ((uint64_t)cur >= (uint64_t)P.num_nodes) {
      raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
      parked = true;
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
        bits = __float_as_uint(__ldg(rand_span + (int64_t)wi * L + l0 + j));
      }
      pre[k] = bits;
    }
  };

  prefetch(0);
  for (int64_t l0 = 0; l0 < L; l0 += S) {
    const int sc = (int)min((int64_t)S, L - l0);
    const int total = nw * sc;
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
    if (live) {
      for (int j = 0; j < sc; j++) {
        int64_t e = -1;
        if (!parked) e = uniform_step<USE_DESC>(P, cur, __uint_as_float((uint32_t)tile[j][lane]));
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
        out_span[(int64_t)wi * (L + 1) + 1 + l0 + j] = (int64_t)tile[j][wi];
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------
// node2vec walk
// ---------------------------------------------------------------------------------
struct Node2vecParams {
  const int64_t* rowptr;
  const int64_t* col;
  const uint64_t* desc;
  int64_t num_nodes, num_edges;
  const int64_t* start;
  int64_t num_walks;
  int32_t walk_length;
  uint32_t cut0, cut1, cut2;  // accept31 < cut_k  <=>  r < prob_k
  uint32_t key0, key1;
  uint64_t walk_index_base;
  uint32_t max_attempts;
  int64_t* n_out;
  int64_t* e_out;
  uint32_t* flags;
  unsigned long long* counters;
};

enum : int { ST_ROW = 0, ST_ATTEMPT = 1, ST_SEARCH = 2, ST_XROW = 3, ST_DONE = 4 };

// One thread per walk; one gather per loop trip.
//   ST_ROW      fetch the bounds of the current node's row
//   ST_ATTEMPT  draw a candidate edge (Philox) and gather col[e]
//   ST_XROW     (general graphs) fetch the bounds of the candidate's row
//   ST_SEARCH   one binary-search probe of the membership test
// The membership test is only entered when it can change the outcome: the draw is
// already known to be >= cut2 (not accepted outright), not accepted by the
// return-to-previous rule, and < cut1. SYM searches the candidate x in the previous
// node's row (bounds already in registers, row hot in cache); otherwise the previous
// node t is searched in the candidate's row, as the reference's is_neighbor(x, t) does.
template <typename idx_t, bool SYM, bool USE_DESC, bool HAS_EOUT, bool COUNT>
__global__ void __launch_bounds__(kBlock) node2vec_walk_kernel(const Node2vecParams P) {
  const int64_t i = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  const bool live = i < P.num_walks;
  if (!COUNT && !live) return;

  uint32_t c_loads = 0, c_attempts = 0, c_member = 0, c_probes = 0;
  uint32_t c_deg0 = 0, c_deg1 = 0, c_sampled = 0, c_first = 0;

  if (live) {
    const int32_t L = P.walk_length;
    const uint64_t gw = P.walk_index_base + (uint64_t)i;
    int64_t* out = P.n_out + i * ((int64_t)L + 1);
    int64_t* eout = HAS_EOUT ? P.e_out + i * (int64_t)L : nullptr;
    const int64_t* __restrict__ col = P.col;

    idx_t t, v, x = 0;              // previous node, current node, candidate
    idx_t v_rs = 0, v_re = 0;       // row [start, end) of v
    idx_t t_rs = 0, t_re = 0;       // row [start, end) of t (SYM search range)
    uint32_t v_deg = 0;             // degree of v saturated at 2^31 (enough for "u % deg" with 31-bit u)
    idx_t lo = 0, hi = 0;           // binary-search window
    idx_t e = 0;                    // sampled edge index
    int32_t l = 0;                  // step being produced
    uint32_t a = 0;                 // attempt counter of this step
    int state = ST_ROW;

    const int64_t s0 = P.start[i];
    out[0] = s0;
    if ((uint64_t)s0 >= (uint64_t)P.num_nodes) {
      raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
      for (int32_t k = 0; k < L; k++) { out[k + 1] = s0; if (HAS_EOUT) eout[k] = -1; }
      state = ST_DONE;
    }
    if (L == 0) state = ST_DONE;
    t = (idx_t)s0;
    v = (idx_t)s0;

    while (state != ST_DONE) {
      // ---- address of this trip's gather
      const int64_t* addr;
      if (state == ST_ROW) {
        addr = USE_DESC ? (const int64_t*)(P.desc + (int64_t)v) : P.rowptr + (int64_t)v;
      } else if (state == ST_ATTEMPT) {
        if (v_deg == 1) {
          e = v_rs;  // forced move: no draw (deg-1 shortcut of the reference; also exact at step 0)
        } else {
          uint32_t cand, acc;
          node2vec_draw(P.key0, P.key1, gw, (uint32_t)l, a, cand, acc);
          e = v_rs + (idx_t)(cand % v_deg);
          lo = (idx_t)acc;  // parked in `lo` until the candidate arrives
        }
        addr = col + (int64_t)e;
      } else if (state == ST_XROW) {
        addr = USE_DESC ? (const int64_t*)(P.desc + (int64_t)x) : P.rowptr + (int64_t)x;
      } else {  // ST_SEARCH
        addr = col + (int64_t)(lo + (hi - lo) / 2);
      }

      int64_t val = __ldg(addr);
      int64_t val2 = 0;
      if (!USE_DESC && (state == ST_ROW || state == ST_XROW)) val2 = __ldg(addr + 1);
      if (COUNT) c_loads += (!USE_DESC && (state == ST_ROW || state == ST_XROW)) ? 2 : 1;

      // ---- consume it
      bool accept = false, reject = false;
      if (state == ST_ROW) {
        int64_t rs, deg;
        if (USE_DESC) { rs = (int64_t)((uint64_t)val & kDescStartMask); deg = (int64_t)((uint64_t)val >> kDescStartBits); }
        else { rs = val; deg = val2 - val; }
        if (deg < 0 || rs < 0 || rs + deg > P.num_edges) { raise_flag(P.flags, WALK_B200_FLAG_BAD_ROWPTR); deg = 0; }
        if (deg == 0) {
          // stay in place for every remaining step
          if (COUNT) c_deg0 += (uint32_t)(L - l);
          for (int32_t k = l; k < L; k++) { out[k + 1] = (int64_t)v; if (HAS_EOUT) eout[k] = -1; }
          state = ST_DONE;
        } else {
          v_rs = (idx_t)rs;
          v_re = (idx_t)(rs + deg);
          v_deg = deg > 0x7fffffffll ? 0x80000000u : (uint32_t)deg;
          a = 0;
          state = ST_ATTEMPT;
          if (COUNT) { if (l == 0) c_first++; else if (deg == 1) c_deg1++; else c_sampled++; }
        }
      } else if (state == ST_ATTEMPT) {
        if ((uint64_t)val >= (uint64_t)P.num_nodes) {
          raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
          val = (int64_t)v;  // park on the current node
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
            if (SYM) {
              lo = t_rs; hi = t_re;
              if (COUNT) c_member++;
              if (lo < hi) state = ST_SEARCH; else reject = true;
            } else {
              state = ST_XROW;
              if (COUNT) c_member++;
            }
          } else reject = true;
        }
      } else if (state == ST_XROW) {
        int64_t rs, deg;
        if (USE_DESC) { rs = (int64_t)((uint64_t)val & kDescStartMask); deg = (int64_t)((uint64_t)val >> kDescStartBits); }
        else { rs = val; deg = val2 - val; }
        if (deg < 0 || rs < 0 || rs + deg > P.num_edges) { raise_flag(P.flags, WALK_B200_FLAG_BAD_ROWPTR); deg = 0; }
        lo = (idx_t)rs; hi = (idx_t)(rs + deg);
        if (lo < hi) state = ST_SEARCH; else { reject = true; }
      } else {  // ST_SEARCH
        if (COUNT) c_probes++;
        const idx_t mid = lo + (hi - lo) / 2;
        const int64_t key = SYM ? (int64_t)x : (int64_t)t;
        if (val == key) accept = true;       // member, and the draw is known to be < cut1
        else {
          if (val < key) lo = mid + 1; else hi = mid;
          if (!(lo < hi)) reject = true;     // not a member, and the draw is known to be >= cut2
        }
      }

      if (reject) {
        a++;
        state = ST_ATTEMPT;
        if (a >= P.max_attempts) {
          raise_flag(P.flags, WALK_B200_FLAG_ATTEMPT_CAP);
          x = v; e = v_rs; accept = true;  // give up on this step: stand still
        }
      }
      if (accept) {
        out[l + 1] = (int64_t)x;
        if (HAS_EOUT) eout[l] = (x == v && a >= P.max_attempts) ? -1 : (int64_t)e;
        t = v; t_rs = v_rs; t_re = v_re;
        v = x;
        l++;
        state = (l == L) ? ST_DONE : ST_ROW;
      }
    }
  }

  if (COUNT) {
    uint32_t c[WALK_B200_COUNTER_COUNT];
    c[WALK_B200_CNT_LOADS] = c_loads; c[WALK_B200_CNT_ATTEMPTS] = c_attempts;
    c[WALK_B200_CNT_MEMBERSHIP] = c_member; c[WALK_B200_CNT_PROBES] = c_probes;
    c[WALK_B200_CNT_STEPS_DEG0] = c_deg0; c[WALK_B200_CNT_STEPS_DEG1] = c_deg1;
    c[WALK_B200_CNT_STEPS_SAMPLED] = c_sampled; c[WALK_B200_CNT_STEPS_FIRST] = c_first;
#pragma unroll
    for (int k = 0; k < WALK_B200_COUNTER_COUNT; k++) {
      unsigned long long s = c[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if ((threadIdx.x & 31) == 0 && s) atomicAdd(P.counters + k, s);
    }
  }
}

}  // namespace walk_b200
