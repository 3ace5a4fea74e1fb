// node2vec walk, pooled form: the state of a walk lives in shared memory, not in the registers of a
// fixed lane. A warp owns a pool of 64 walk slots. Every trip it looks at the states of its slots,
// picks the state class most of them are in (drawing candidates / probing the edge hash set /
// finishing a step and fetching the next row), deals up to 32 slots of that class to its lanes and
// runs that one path for all of them. In node2vec_walk_kernel a warp executes the union of the paths
// its 32 fixed lanes are on and about 12 lanes do useful work per instruction; here a trip executes one
// path with most lanes busy. Same Philox draws, same decisions, same outputs.
//
// The kernel runs at the register limit of six blocks per SM (40) with no spill, and its speed is sensitive to
// its code shape well beyond what the source suggests (measured: a 32-bit instead of a 64-bit chunk window,
// or one more shared-memory store in the refill branch, each cost 3-4 % of the launch): re-measure after any edit.
//
// Requires the configuration the bench uses: 32-bit indices, row descriptors, the edge hash set and
// colrev (col joined with the reverse positions); fewer than 2^32 walks, walk_length < 65536.
#pragma once
#include "walk_kernels.cuh"

namespace walk_b200 {

constexpr int kPoolSlots = 64;  // walk slots per warp. Measured at R-MAT 24, (0.25, 4): 32 slots 141 ms, 64 slots 124 ms,
                                // 96 slots 181 ms (its shared memory leaves the SM too little L1 for the misses in flight)
enum : int {
  PF_I = 0,   // walk (row of this launch)
  PF_T,       // previous node
  PF_V,       // current node
  PF_RS,      // row start of v
  PF_DEG,     // degree of v (saturated at 2^31)
  PF_RET,     // index of the edge v -> t (kNoEdge / kUnknownEdge)
  PF_IN,      // index of the edge t -> v the walk arrived by
  PF_X,       // candidate
  PF_XREV,    // index of the edge x -> v, gathered with x
  PF_E,       // drawn edge
  PF_A,       // attempt counter of this step
  PF_LS,      // state (bits 0-2) | buckets probed (bits 3-15) | step (bits 16-31)
  PF_COUNT
};
enum : int { PS_IDLE = 0, PS_START, PS_ROW, PS_ACCEPTED, PS_ATTEMPT, PS_HASH };

template <bool HAS_EOUT, int HOST, int SLOTS = kPoolSlots>
__global__ void __launch_bounds__(kBlock, 6) node2vec_pool_kernel(const Node2vecParams P) {
  static_assert(SLOTS % 32 == 0 && SLOTS >= 32 && SLOTS <= 96, "whole slots per lane, within static shared memory");
  __shared__ uint32_t pool[PF_COUNT][kWarpsPerBlock][SLOTS];
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
      int32_t l = (int32_t)(ls >> 16);

      if (cls == PS_ROW) {
        // -------- START / ACCEPTED, then the row fetch of the node the walk now stands on
        int st = (int)(ls & 7u);
        uint32_t v = 0;
        bool done = false;
        if (st == PS_START) {
          const int64_t val = ld8(P.start + i, pol.stream);
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
          }
        } else if (st == PS_ACCEPTED) {
          const uint32_t x = FLD(PF_X, s), e = FLD(PF_E, s);
          put_node(i, l + 1, (int64_t)x);
          if (HAS_EOUT) put_edge(i, l, FLD(PF_A, s) >= P.max_attempts ? -1 : (int64_t)e);
          const uint32_t ret_e = FLD(PF_RET, s);
          if (e == kUnknownEdge) { FLD(PF_RET, s) = kUnknownEdge; FLD(PF_IN, s) = kUnknownEdge; }      // stood still
          else if (e == ret_e) { FLD(PF_RET, s) = FLD(PF_IN, s); FLD(PF_IN, s) = ret_e; }               // went back
          else { FLD(PF_IN, s) = e; FLD(PF_RET, s) = FLD(PF_XREV, s); }
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
            if (!known || e == ret_e || acc < P.cut2 || acc < P.cut1) break;
            if (k >= P.draw_loop || a + 1 >= P.max_attempts) break;
            a++;  // rejected without touching memory
          }
          if (known) {
            if (e == ret_e) {  // the candidate is the previous node: no gather needed to know it
              need_load = false;
              x = t;
              if (acc < P.cut2 || acc < P.cut0) accept = true;
              else if (acc < P.cut1) probe = true;  // only a self-loop t -> t could still accept
              else reject = true;
            } else if (acc >= P.cut2 && acc >= P.cut1) {  // not the way back, too large for the other rules
              need_load = false;
              reject = true;
            }
          }
        }
        if (need_load) {
          const uint64_t w = (uint64_t)ld8(P.colrev + (int64_t)e, pol.stream);
          uint32_t x_rev = (uint32_t)(w >> 32);
          x = (uint32_t)w;
          if ((uint64_t)x >= (uint64_t)P.num_nodes) {
            raise_flag(P.flags, WALK_B200_FLAG_BAD_NODE);
            x = v;  // park on the current node
            x_rev = kUnknownEdge;
          }
          FLD(PF_XREV, s) = x_rev;
          if (l == 0 || v_deg == 1) accept = true;
          else if (acc < P.cut2) accept = true;
          else if (x == t && acc < P.cut0) accept = true;
          else if (acc < P.cut1) probe = true;
          else reject = true;
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
        if (accept) { next = PS_ACCEPTED; hi = 0; }
        FLD(PF_LS, s) = ((uint32_t)l << 16) | (hi << 3) | (uint32_t)next;
      }
    }
    __syncwarp();
  }
#undef FLD
}

}  // namespace walk_b200
