// node2vec walk, pooled form with a triangle filter: node2vec_pool_kernel (n2v_pool.cuh) plus one 64-bit word
// per walk that answers most membership tests without touching memory.
//
// The test "is the previous node t a neighbour of the candidate x" (is_neighbor of the reference,
// random_walks/BiasedRandomWalk.cpp:20-28,88) needs x, i.e. the gather of the candidate, and then the edge
// hash set: two dependent DRAM accesses, and nine times in ten the answer is no. On an undirected graph the
// answer can only be yes when x is a common neighbour of t and v, the node the walk stands on. So every
// directed edge (t -> v) carries a filter word: bit b is set iff some common neighbour of t and v sits at a
// position p of v's row with p mod 64 == b. A walk that arrived by that edge draws a position in v's row; if
// its bit is clear the candidate is certainly not a neighbour of t, and an attempt that only the membership
// rule could accept is rejected before anything is gathered. The words live beside col and the reverse
// positions in 16-byte records (colrev16[e] = {col[e] | revpos[e] << 32, filter of e}), so the gather of a
// candidate that is accepted outright brings the filter of the next step with it; after a step accepted
// through the hash set, or a step back along the edge the walk came by, the word is fetched with the row
// descriptor. Exact: the filter only ever says "certainly not". Same Philox draws, same decisions, same
// outputs as the other kernels.
//
// A kernel of its own rather than a template flag of node2vec_pool_kernel: that kernel's speed depends on its exact
// code shape (see its header) and it remains the kernel for graphs without a filter, so it is left untouched.
//
// Requires what node2vec_pool_kernel requires, a graph the caller declares undirected (WALK_B200_CSR_SYMMETRIC),
// the records from walk_b200_trifilter_build, and walk_length < 32768.
#pragma once
#include "n2v_pool.cuh"

namespace walk_b200 {

enum : int { PF_BL0 = PF_COUNT, PF_BL1, PF_TRI_COUNT };  // the filter word of the edge the walk arrived by
constexpr uint32_t kFetchFilter = 0x80000000u;           // PF_LS bit: the word of the accepted edge is not at hand

// COUNT: the instrumented instantiation (untimed): counts what the kernel reads into P.counters.
template <bool HAS_EOUT, int HOST, bool COUNT = false, int SLOTS = kPoolSlots>
__global__ void __launch_bounds__(kBlock, COUNT ? 1 : 6) node2vec_pool_tri_kernel(const Node2vecParams P) {
  uint32_t c_loads = 0, c_attempts = 0, c_member = 0, c_probes = 0, c_gathers = 0, c_filtered = 0;
  static_assert(SLOTS % 32 == 0 && SLOTS >= 32 && SLOTS <= 96, "whole slots per lane, within static shared memory");
  __shared__ uint32_t pool[PF_TRI_COUNT][kWarpsPerBlock][SLOTS];
  __shared__ uint8_t sel[kWarpsPerBlock][SLOTS];
  constexpr unsigned kFull = 0xffffffffu;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  const L2Policy pol = make_policies(P.hints);
  const int32_t L = P.walk_length;
  const int64_t n = P.num_walks;
  const int64_t n_chunks = (n + 31) / 32;
#define FLD(f, s) pool[f][warp][s]

  auto put_node = [&](int64_t row, int32_t k, int64_t node) {
    if (HOST == HOST_NARROW) reinterpret_cast<int32_t*>(P.n_out)[row * ((int64_t)L + 1) + k] = (int32_t)node;
    else st8(P.n_out + row * ((int64_t)L + 1) + k, node, pol.stream);
  };
  auto put_edge = [&](int64_t row, int32_t k, int64_t edge) {
    if (HOST == HOST_NARROW) reinterpret_cast<int32_t*>(P.e_out)[row * (int64_t)L + k] = (int32_t)edge;
    else P.e_out[row * (int64_t)L + k] = edge;
  };
  // a finished walk's rows are made visible, then counted for its slab (host single-launch mode)
  auto report_finished = [&](int64_t row) {
    if (!HOST) return;
    __threadfence();
    const int64_t slab = row >> P.slab_shift;
    const int64_t rows_in_slab = min((int64_t)1 << P.slab_shift, n - (slab << P.slab_shift));
    if ((int64_t)atomicAdd(P.slab_done + slab, 1u) + 1 == rows_in_slab) {
      __threadfence_system();
      P.slab_flags[slab] = 1u;
    }
  };

  constexpr int K = SLOTS / 32;  // slots per lane: slot lane + 32 k, k < K
#pragma unroll
  for (int k = 0; k < K; k++) FLD(PF_LS, lane + 32 * k) = PS_IDLE;
  __syncwarp();
  int64_t q_next = 0, q_end = 0;  // current chunk of 32 walks of the launch-wide queue
  bool drained = false;

  while (true) {
    int st[K];
#pragma unroll
    for (int k = 0; k < K; k++) st[k] = (int)(FLD(PF_LS, lane + 32 * k) & 7u);

    // ---- hand unassigned walks to idle slots
    unsigned idle[K];
    int n_idle = 0;
#pragma unroll
    for (int k = 0; k < K; k++) { idle[k] = __ballot_sync(kFull, st[k] == PS_IDLE); n_idle += __popc(idle[k]); }
    if (n_idle && !drained) {
      int rank[K], before = 0;
#pragma unroll
      for (int k = 0; k < K; k++) { rank[k] = before + __popc(idle[k] & lt); before += __popc(idle[k]); }
      int given = 0;
      while (given < n_idle) {
        if (q_next >= q_end) {
          unsigned long long chunk = 0;
          if (lane == 0) chunk = atomicAdd(P.queue, 1ull);
          chunk = __shfl_sync(kFull, chunk, 0);
          if ((int64_t)chunk >= n_chunks) { drained = true; break; }
          q_next = (int64_t)chunk * 32;
          q_end = min(q_next + 32, n);
        }
        const int take = min((int)(q_end - q_next), n_idle - given);
#pragma unroll
        for (int k = 0; k < K; k++) {
          if (st[k] == PS_IDLE && rank[k] >= given && rank[k] < given + take) {
            FLD(PF_I, lane + 32 * k) = (uint32_t)(q_next + (rank[k] - given));
            FLD(PF_LS, lane + 32 * k) = PS_START;
            st[k] = PS_START;
          }
        }
        q_next += take;
        given += take;
      }
      __syncwarp();
    }

    // ---- pick the class most slots are in
    unsigned mA[K], mH[K], mR[K];
    int nA = 0, nH = 0, nR = 0;
#pragma unroll
    for (int k = 0; k < K; k++) {
      mA[k] = __ballot_sync(kFull, st[k] == PS_ATTEMPT);
      mH[k] = __ballot_sync(kFull, st[k] == PS_HASH);
      mR[k] = __ballot_sync(kFull, st[k] >= PS_START && st[k] <= PS_ACCEPTED);
      nA += __popc(mA[k]); nH += __popc(mH[k]); nR += __popc(mR[k]);
    }
    if (nA + nH + nR == 0) break;  // every slot idle: the queue is drained (idle slots are refilled above otherwise)
    int cls;
    if (nA >= nH && nA >= nR) cls = PS_ATTEMPT;
    else if (nH >= nR) cls = PS_HASH;
    else cls = PS_ROW;
    int cnt = 0;
#pragma unroll
    for (int k = 0; k < K; k++) {
      const unsigned m = cls == PS_ATTEMPT ? mA[k] : (cls == PS_HASH ? mH[k] : mR[k]);
      if ((m >> lane) & 1u) sel[warp][cnt + __popc(m & lt)] = (uint8_t)(lane + 32 * k);
      cnt += __popc(m);
    }
    __syncwarp();

    // the slots of the class, 32 at a time (the choice above is paid once for all rounds); a last
    // round that would fill less than half the warp is left for a later trip
    for (int base = 0; base < cnt && (base == 0 || cnt - base >= 16); base += 32)
    if (base + lane < cnt) {
      const int s = sel[warp][base + lane];
      const int64_t i = (int64_t)FLD(PF_I, s);
      uint32_t ls = FLD(PF_LS, s);
      int32_t l = (int32_t)((ls >> 16) & 0x7fffu);

      if (cls == PS_ROW) {
        // -------- START / ACCEPTED, then the row fetch of the node the walk now stands on
        int st = (int)(ls & 7u);
        uint32_t v = 0;
        bool done = false;
        uint32_t fetch_edge = kUnknownEdge;  // edge whose filter word must be fetched beside the row descriptor
        if (st == PS_START) {
          const int64_t val = ld8(P.start + i, pol.stream);
          if (COUNT) c_loads++;
          put_node(i, 0, val);
          l = 0;
          if ((uint64_t)val >= (uint64_t)P.num_nodes) {
            raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
            for (int32_t k = 0; k < L; k++) { put_node(i, k + 1, val); if (HAS_EOUT) put_edge(i, k, -1); }
            done = true;
          } else if (L == 0) {
            done = true;
          } else {
            v = (uint32_t)val;
            FLD(PF_T, s) = v;
            FLD(PF_V, s) = v;
            FLD(PF_RET, s) = kUnknownEdge;
            FLD(PF_IN, s) = kUnknownEdge;
            FLD(PF_BL0, s) = 0xffffffffu;  // no edge in: nothing is filtered
            FLD(PF_BL1, s) = 0xffffffffu;
          }
        } else if (st == PS_ACCEPTED) {
          const uint32_t x = FLD(PF_X, s), e = FLD(PF_E, s);
          put_node(i, l + 1, (int64_t)x);
          if (HAS_EOUT) put_edge(i, l, FLD(PF_A, s) >= P.max_attempts ? -1 : (int64_t)e);
          const uint32_t ret_e = FLD(PF_RET, s);
          if (e == kUnknownEdge) {  // stood still
            FLD(PF_RET, s) = kUnknownEdge; FLD(PF_IN, s) = kUnknownEdge;
            FLD(PF_BL0, s) = 0xffffffffu; FLD(PF_BL1, s) = 0xffffffffu;
          } else if (e == ret_e) {  // went back: the edge in is the old edge back, whose word was never gathered
            FLD(PF_RET, s) = FLD(PF_IN, s); FLD(PF_IN, s) = ret_e;
            fetch_edge = ret_e;
          } else {
            FLD(PF_IN, s) = e; FLD(PF_RET, s) = FLD(PF_XREV, s);
            if (ls & kFetchFilter) fetch_edge = e;  // accepted through the hash set: the candidate's word was dropped
          }
          FLD(PF_T, s) = FLD(PF_V, s);
          FLD(PF_V, s) = x;
          v = x;
          l++;
          if (l == L) done = true;
        } else {
          v = FLD(PF_V, s);
        }
        if (!done) {
          const uint64_t d = (uint64_t)ld8(P.desc + (int64_t)v, pol.keep);
          if (COUNT) c_loads += fetch_edge != kUnknownEdge ? 2 : 1;
          if (fetch_edge != kUnknownEdge) {
            const uint64_t word = (uint64_t)ld8(reinterpret_cast<const char*>(P.colrev16 + (int64_t)fetch_edge) + 8, pol.stream);
            FLD(PF_BL0, s) = (uint32_t)word;
            FLD(PF_BL1, s) = (uint32_t)(word >> 32);
          }
          int64_t rs = (int64_t)(d & kDescStartMask), deg = (int64_t)(d >> kDescStartBits);
          if (rs + deg > P.num_edges) { raise_flag(P.flags, WALK_B200_FLAG_BAD_ROWPTR); deg = 0; }
          if (deg == 0) {  // stay in place for every remaining step
            for (int32_t k = l; k < L; k++) { put_node(i, k + 1, (int64_t)v); if (HAS_EOUT) put_edge(i, k, -1); }
            done = true;
          } else {
            const uint32_t v_deg = deg > 0x7fffffffll ? 0x80000000u : (uint32_t)deg;
            FLD(PF_RS, s) = (uint32_t)rs;
            FLD(PF_DEG, s) = v_deg;
            FLD(PF_A, s) = 0;
            FLD(PF_LS, s) = ((uint32_t)l << 16) | PS_ATTEMPT;
          }
        }
        if (done) {
          FLD(PF_LS, s) = PS_IDLE;
          report_finished(i);
        }
      } else if (cls == PS_ATTEMPT) {
        // -------- draw candidates until one needs memory (or is decided), gather it, classify it
        const uint32_t t = FLD(PF_T, s), v = FLD(PF_V, s);
        const uint32_t v_rs = FLD(PF_RS, s), v_deg = FLD(PF_DEG, s);
        const uint32_t v_inv = 0xffffffffu / v_deg;  // recomputed: a slot field less leaves the SM more L1
        const uint32_t ret_e = FLD(PF_RET, s);
        uint32_t a = FLD(PF_A, s);
        uint32_t e, acc = 0, x = 0;
        bool accept = false, reject = false, probe = false, need_load = true;
        const bool known = l > 0 && ret_e != kUnknownEdge;
        // all ones whenever the walk has no edge in (first step, after standing still): then nothing is filtered
        const uint64_t filter = (uint64_t)FLD(PF_BL0, s) | ((uint64_t)FLD(PF_BL1, s) << 32);
        bool filtered = false;  // the attempt in hand needs the membership rule and the filter rules it out
        if (v_deg == 1) {
          e = v_rs;  // forced move: no draw
          if (known && e == ret_e) { x = t; accept = true; need_load = false; }
        } else {
          const uint64_t gw = P.walk_index_base + (uint64_t)i * P.walk_index_stride;
          uint32_t cand;
          for (int k = 1;; k++) {
            node2vec_draw(P.key0, P.key1, gw, (uint32_t)l, a, cand, acc);
            uint32_t rem = cand - __umulhi(cand, v_inv) * v_deg;  // cand % v_deg, exactly
            if (rem >= v_deg) rem -= v_deg;
            e = v_rs + rem;
            filtered = false;
            if (!known || e == ret_e || acc < P.cut2) break;
            if (acc < P.cut1) {  // only the membership rule could accept: is the drawn position one of a common neighbour?
              if ((filter >> (rem & 63u)) & 1ull) break;
              filtered = true;
            }
            if (k >= P.draw_loop || a + 1 >= P.max_attempts) break;
            if (COUNT) { c_attempts++; if (filtered) c_filtered++; }
            a++;  // rejected without touching memory
          }
          if (COUNT && l > 0) { c_attempts++; if (filtered) c_filtered++; }
          if (known) {
            if (e == ret_e) {  // the candidate is the previous node: no gather needed to know it
              need_load = false;
              x = t;
              if (acc < P.cut2 || acc < P.cut0) accept = true;
              else if (acc < P.cut1) probe = true;  // only a self-loop t -> t could still accept
              else reject = true;
            } else if (filtered || (acc >= P.cut2 && acc >= P.cut1)) {  // not the way back, and no other rule can accept
              need_load = false;
              reject = true;
            }
          }
        }
        if (need_load) {
          const ulonglong2 rec = ld16(P.colrev16 + (int64_t)e, pol.stream);
          if (COUNT) { c_loads += 2; c_gathers++; }
          const uint64_t w = rec.x;
          uint64_t x_filter = rec.y;  // the filter of the edge v -> x: the next step's, if x is accepted
          uint32_t x_rev = (uint32_t)(w >> 32);
          x = (uint32_t)w;
          if ((uint64_t)x >= (uint64_t)P.num_nodes) {
            raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
            x = v;  // park on the current node
            x_rev = kUnknownEdge;
            x_filter = ~0ull;
          }
          FLD(PF_XREV, s) = x_rev;
          if (l == 0 || v_deg == 1) accept = true;
          else if (acc < P.cut2) accept = true;
          else if (x == t && acc < P.cut0) accept = true;
          else if (acc < P.cut1) probe = true;
          else reject = true;
          if (COUNT && probe) c_member++;
          if (accept) {  // this step is over: its own filter gives way to the next one's
            FLD(PF_BL0, s) = (uint32_t)x_filter;
            FLD(PF_BL1, s) = (uint32_t)(x_filter >> 32);
          }
        }
        int next = PS_ATTEMPT;
        if (probe) next = PS_HASH;
        if (reject) {
          a++;
          if (a >= P.max_attempts) {
            raise_flag(P.flags, WALK_B200_FLAG_ATTEMPT_CAP);
            x = v; accept = true;  // give up on this step: stand still
            e = kUnknownEdge;
          }
        }
        if (accept) next = PS_ACCEPTED;
        FLD(PF_A, s) = a;
        FLD(PF_E, s) = e;
        FLD(PF_X, s) = x;
        FLD(PF_LS, s) = ((uint32_t)l << 16) | (uint32_t)next;  // buckets probed: 0
      } else {
        // -------- one 32-byte bucket of the edge hash set
        const uint32_t x = FLD(PF_X, s), t = FLD(PF_T, s);
        uint32_t hi = (ls >> 3) & 0x1fffu;  // buckets probed so far: this trip reads bucket (home + hi) mod buckets
        const uint64_t key = edge_key((uint64_t)x, (uint64_t)t);
        uint64_t lo = edge_bucket(key, P.edgeset_buckets) + hi;
        while (lo >= P.edgeset_buckets) lo -= P.edgeset_buckets;
        const void* addr = P.edgeset + lo * kEdgeSlotsPerBucket;
        const ulonglong2 h0 = ld16(addr, pol.stream), h1 = ld16((const char*)addr + 16, pol.stream);
        if (COUNT) { c_loads += 4; c_probes++; }
        bool accept = false, reject = false;
        if (h0.x == key || h0.y == key || h1.x == key || h1.y == key) accept = true;
        else if (h0.x == kEdgeEmpty || h0.y == kEdgeEmpty || h1.x == kEdgeEmpty || h1.y == kEdgeEmpty) reject = true;
        else if (++hi >= (uint32_t)kEdgeMaxProbe) { raise_flag(P.flags, WALK_B200_FLAG_EDGESET_FULL); reject = true; }
        int next = PS_HASH;
        if (reject) {
          uint32_t a = FLD(PF_A, s) + 1;
          next = PS_ATTEMPT;
          hi = 0;
          if (a >= P.max_attempts) {
            raise_flag(P.flags, WALK_B200_FLAG_ATTEMPT_CAP);
            FLD(PF_X, s) = FLD(PF_V, s);  // stand still
            FLD(PF_E, s) = kUnknownEdge;
            next = PS_ACCEPTED;
          }
          FLD(PF_A, s) = a;
        }
        uint32_t fetch = 0;
        if (accept) { next = PS_ACCEPTED; hi = 0; fetch = kFetchFilter; }
        FLD(PF_LS, s) = fetch | ((uint32_t)l << 16) | (hi << 3) | (uint32_t)next;
      }
    }
    __syncwarp();
  }
#undef FLD
  if (COUNT) {
    uint32_t c[WALK_B200_COUNTER_COUNT] = {};
    c[WALK_B200_CNT_LOADS] = c_loads; c[WALK_B200_CNT_ATTEMPTS] = c_attempts;
    c[WALK_B200_CNT_MEMBERSHIP] = c_member; c[WALK_B200_CNT_PROBES] = c_probes;
    c[WALK_B200_CNT_GATHERS16] = c_gathers; c[WALK_B200_CNT_FILTERED] = c_filtered;
#pragma unroll
    for (int k = 0; k < WALK_B200_COUNTER_COUNT; k++) {
      unsigned long long sum = c[k];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
      if (lane == 0 && sum) atomicAdd(P.counters + k, sum);
    }
  }
}

}  // namespace walk_b200
