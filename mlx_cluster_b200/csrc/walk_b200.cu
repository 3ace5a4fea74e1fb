// Host launch/stream layer and C ABI of the B200 walk generators (see include/walk_b200.h).
//
// Everything a framework binds lives behind extern "C": argument checks, threshold
// arithmetic, kernel selection, launches on the caller's stream, the resident-graph
// handle and the slab pipeline for host buffers. No torch types, no exceptions.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <thread>

#include "../../include/walk_b200.h"
#include "host_common.h"
#include "host_widen.h"
#include "walk_kernels.cuh"
#include "n2v_pool.cuh"
#include "n2v_pool_tri.cuh"

namespace {

using namespace walk_b200;

thread_local std::string g_last_error;
thread_local const char* g_last_kernel = "";  // name of the kernel this thread launched last (string literals only)
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define CUDA_TRY(expr)                                                                      \
  do {                                                                                      \
    cudaError_t err__ = (expr);                                                             \
    if (err__ != cudaSuccess)                                                               \
      return fail(WALK_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));   \
  } while (0)

int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess)
    return fail(WALK_B200_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(err));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  g_last_kernel = what;
  return WALK_B200_OK;
}

// ---- tuning knobs (experiments; defaults are the measured best) ------------------
struct Tuning {
  std::atomic<int32_t> uniform_variant{0};  // 0 auto (7; 1 for walk_length < 4), 1 direct, staged: 2 S=8, 3 S=16,
                                            // 4 S=4, 5 S=16 @6 blocks/SM, 6 S=8 @8, 7 S=16 @4, 8 S=16 @5, 9 S=8 @6
  std::atomic<int32_t> uniform_fused{1};    // use fused edge records when the graph has them
  std::atomic<int32_t> n2v_idx{0};          // 0 auto (32-bit indices when they fit), 1 force 64-bit
  std::atomic<int32_t> n2v_member{0};       // 0 auto (hash set when the graph has one), 1 ignore the hash set
  std::atomic<int32_t> n2v_batch_lanes{4};  // rare state paths wait for this many lanes of a warp ...
  std::atomic<int32_t> n2v_batch_trips{4};  // ... or this many trips (measured best: 4/4)
  std::atomic<int32_t> n2v_draw_loop{3};    // memory-free rejections consumed per trip (reverse-position kernel;
                                            // measured: 1 -> 193 ms, 2 -> 169, 3 -> 166, 4 -> 170, 8 -> 207)
  std::atomic<int32_t> n2v_rev{1};          // 1 auto (reverse positions when they pay), 0 never, 2 whenever available
  std::atomic<int32_t> n2v_pool{1};         // 1: pooled kernel (walk state in shared memory, one state class per trip)
  std::atomic<int32_t> n2v_blocks_per_sm{0};  // 0 = what the occupancy calculator allows
  std::atomic<int32_t> n2v_tri{1};          // 1: use the triangle filter when the graph carries one (undirected graphs), 0 never
  std::atomic<int32_t> n2v_tri_draw_loop{5};  // ... and consume up to this many memory-free rejections per trip there
                                            // (most attempts are: 2 -> 102.9 ms, 3 -> 91.4, 5 -> 87.3, 8 -> 89.5)
  std::atomic<int32_t> trifilter_max_row{1024};  // resident graphs: edges whose shorter row is longer go unfiltered
                                                 // (1024: 2.0 s to build and 92.0 ms per launch at R-MAT 24; none: 8.6 s, 91.4 ms)
  std::atomic<int32_t> n2v_count_kernel{0}; // which kernel a call with counters instruments (0 per-lane, 1 triangle filter)
  std::atomic<int32_t> edgeset_slots_per_edge{4};  // size of the edge hash set a resident graph builds: 2 = half full
                                                   // (the minimum), 4 = a quarter full (fewer second buckets read)
  std::atomic<int32_t> n2v_max_attempts{(int32_t)WALK_B200_MAX_ATTEMPTS};  // rejections after which a step gives up
  std::atomic<int32_t> l2_hints{3};         // bit 0: evict-last row bounds, bit 1: evict-first streams
  std::atomic<int32_t> l2_fetch_granularity{0};  // set only through walk_b200_set_tuning (applies the CUDA limit)
  std::atomic<int32_t> host_slab_mb{256};   // walk-matrix bytes per pipeline slab of the host entry points
  std::atomic<int32_t> use_rowdesc{1};      // host entry points: build and use the packed row descriptor
  std::atomic<int32_t> host_narrow{2};      // host entry points: 1 ids that fit int32 cross PCIe as int32, 0 never,
                                            // 2 whichever a short measurement at graph creation finds faster
  std::atomic<int32_t> host_threads{0};     // host threads that widen them again; 0 = min(16, hardware threads)
  std::atomic<int32_t> host_single_launch{1};  // node2vec host entry: one launch over all rows, slabs copied out
                                               // behind it as they complete (needs host_narrow)
  std::atomic<int32_t> host_resident_mb{65536};  // ... while the int32 matrices fit this many MiB of device memory
} g_tuning;

std::atomic<int32_t>* tuning_slot(const char* key) {
  if (!key) return nullptr;
  if (!strcmp(key, "uniform_variant")) return &g_tuning.uniform_variant;
  if (!strcmp(key, "uniform_fused")) return &g_tuning.uniform_fused;
  if (!strcmp(key, "n2v_idx")) return &g_tuning.n2v_idx;
  if (!strcmp(key, "n2v_member")) return &g_tuning.n2v_member;
  if (!strcmp(key, "n2v_rev")) return &g_tuning.n2v_rev;
  if (!strcmp(key, "n2v_pool")) return &g_tuning.n2v_pool;
  if (!strcmp(key, "n2v_batch_lanes")) return &g_tuning.n2v_batch_lanes;
  if (!strcmp(key, "n2v_batch_trips")) return &g_tuning.n2v_batch_trips;
  if (!strcmp(key, "n2v_draw_loop")) return &g_tuning.n2v_draw_loop;
  if (!strcmp(key, "n2v_blocks_per_sm")) return &g_tuning.n2v_blocks_per_sm;
  if (!strcmp(key, "n2v_tri")) return &g_tuning.n2v_tri;
  if (!strcmp(key, "n2v_tri_draw_loop")) return &g_tuning.n2v_tri_draw_loop;
  if (!strcmp(key, "n2v_count_kernel")) return &g_tuning.n2v_count_kernel;
  if (!strcmp(key, "trifilter_max_row")) return &g_tuning.trifilter_max_row;
  if (!strcmp(key, "n2v_max_attempts")) return &g_tuning.n2v_max_attempts;
  if (!strcmp(key, "edgeset_slots_per_edge")) return &g_tuning.edgeset_slots_per_edge;
  if (!strcmp(key, "l2_hints")) return &g_tuning.l2_hints;
  if (!strcmp(key, "l2_fetch_granularity")) return &g_tuning.l2_fetch_granularity;
  if (!strcmp(key, "host_slab_mb")) return &g_tuning.host_slab_mb;
  if (!strcmp(key, "use_rowdesc")) return &g_tuning.use_rowdesc;
  if (!strcmp(key, "host_narrow")) return &g_tuning.host_narrow;
  if (!strcmp(key, "host_threads")) return &g_tuning.host_threads;
  if (!strcmp(key, "host_single_launch")) return &g_tuning.host_single_launch;
  if (!strcmp(key, "host_resident_mb")) return &g_tuning.host_resident_mb;
  return nullptr;
}

int check_csr(const walk_b200_csr* g) {
  if (!g) return fail(WALK_B200_ERR_INVALID_ARG, "csr descriptor is NULL");
  if (g->num_nodes < 0 || g->num_edges < 0)
    return fail(WALK_B200_ERR_INVALID_ARG, "negative graph size (num_nodes=%lld, num_edges=%lld)",
                (long long)g->num_nodes, (long long)g->num_edges);
  if (!g->rowptr) return fail(WALK_B200_ERR_INVALID_ARG, "rowptr is NULL");
  if (g->num_edges > 0 && !g->col) return fail(WALK_B200_ERR_INVALID_ARG, "col is NULL");
  return WALK_B200_OK;
}

int check_walk_sizes(int64_t num_walks, int32_t walk_length, const void* start, const void* n_out) {
  if (num_walks < 0) return fail(WALK_B200_ERR_INVALID_ARG, "num_walks is negative");
  if (walk_length < 0) return fail(WALK_B200_ERR_INVALID_ARG, "walk_length is negative");
  if (num_walks > 0 && (!start || !n_out))
    return fail(WALK_B200_ERR_INVALID_ARG, "start or n_out is NULL");
  // row pitch * rows must stay inside int64 element indices
  if (num_walks > 0 && (int64_t)(walk_length + 1ll) > (INT64_MAX / 8) / num_walks)
    return fail(WALK_B200_ERR_INVALID_ARG, "num_walks * (walk_length + 1) overflows");
  return WALK_B200_OK;
}

int64_t blocks_for(int64_t n) { return (n + kBlock - 1) / kBlock; }

// ---- thresholds -------------------------------------------------------------------
constexpr double kRandMax = 2147483647.0;

uint32_t accept_cut(double prob) {
  // smallest 31-bit draw w with (double)w / RAND_MAX >= prob; 2^31 if there is none
  uint64_t lo = 0, hi = (uint64_t)2147483647 + 1;
  while (lo < hi) {
    const uint64_t mid = lo + (hi - lo) / 2;
    if ((double)mid / kRandMax >= prob) hi = mid; else lo = mid + 1;
  }
  return (uint32_t)lo;
}

int thresholds(double p, double q, double prob[3], uint32_t cuts[3]) {
  if (!(p > 0.0) || !(q > 0.0) || !std::isfinite(p) || !std::isfinite(q))
    return fail(WALK_B200_ERR_BAD_PQ, "p and q must be finite and > 0 (got p=%g, q=%g)", p, q);
  const double max_prob = std::fmax(std::fmax(1. / p, 1.), 1. / q);
  prob[0] = 1. / p / max_prob;
  prob[1] = 1. / max_prob;
  prob[2] = 1. / q / max_prob;
  // prob_2 applies to every candidate, so it bounds the expected attempts of a step by 1 / prob_2
  // whatever the graph looks like; below 2^-16 a step can take longer than anyone will wait
  if (!(prob[2] >= 1.0 / 65536.0))
    return fail(WALK_B200_ERR_BAD_PQ,
                "p=%g, q=%g give prob_2 = %g (< 2^-16): the rejection loop would need more than 65536 attempts per step",
                p, q, prob[2]);
  for (int k = 0; k < 3; k++) cuts[k] = accept_cut(prob[k]);
  return WALK_B200_OK;
}

// ---- launches ---------------------------------------------------------------------
template <bool USE_DESC, bool HAS_EOUT>
int launch_uniform_t(const UniformParams& P, cudaStream_t s) {
  int variant = g_tuning.uniform_variant.load();
  if (variant == 0) variant = P.walk_length >= 4 ? 7 : 1;
  const unsigned grid = (unsigned)blocks_for(P.num_walks);
  if (P.generate) {  // draws generated in the kernel: the staged kernel only
    if (USE_DESC && P.fused && g_tuning.uniform_fused.load() != 0) {
      uniform_walk_staged_kernel<16, 4, true, HAS_EOUT, true, true><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<16,4,fused,gen>");
    }
    uniform_walk_staged_kernel<16, 4, USE_DESC, HAS_EOUT, false, true><<<grid, kBlock, 0, s>>>(P);
    return check_launch("uniform_walk_staged_kernel<16,4,gen>");
  }
  if (USE_DESC && P.fused && variant != 1 && g_tuning.uniform_fused.load() != 0) {
    if (variant == 2) {
      uniform_walk_staged_kernel<8, 1, true, HAS_EOUT, true><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<8,fused>");
    }
    uniform_walk_staged_kernel<16, 4, true, HAS_EOUT, true><<<grid, kBlock, 0, s>>>(P);
    return check_launch("uniform_walk_staged_kernel<16,4,fused>");
  }
  switch (variant) {
    case 1:
      uniform_walk_direct_kernel<USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_direct_kernel");
    case 2:
      uniform_walk_staged_kernel<8, 1, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<8>");
    case 4:
      uniform_walk_staged_kernel<4, 1, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<4>");
    case 5:
      uniform_walk_staged_kernel<16, 6, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<16,6>");
    case 6:
      uniform_walk_staged_kernel<8, 8, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<8,8>");
    case 7:
      uniform_walk_staged_kernel<16, 4, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<16,4>");
    case 8:
      uniform_walk_staged_kernel<16, 5, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<16,5>");
    case 9:
      uniform_walk_staged_kernel<8, 6, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<8,6>");
    case 3:
    default:
      uniform_walk_staged_kernel<16, 1, USE_DESC, HAS_EOUT><<<grid, kBlock, 0, s>>>(P);
      return check_launch("uniform_walk_staged_kernel<16>");
  }
}

int launch_uniform(const UniformParams& P, cudaStream_t s) {
  const bool d = P.desc != nullptr, e = P.e_out != nullptr;
  if (d) return e ? launch_uniform_t<true, true>(P, s) : launch_uniform_t<true, false>(P, s);
  return e ? launch_uniform_t<false, true>(P, s) : launch_uniform_t<false, false>(P, s);
}

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cached[dev].load();
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev].store(v);
  }
  return v;
}

// Launch-wide chunk counters of the node2vec kernel. Each launch takes the next slot of
// this ring, clears it on its stream and hands it to the kernel. The ring lives in the
// library's device image, so a launch allocates nothing. A slot is reused after
// kQueueSlots further launches on the same device: more node2vec launches than that in
// flight at once (across streams) are not supported.
constexpr int kQueueSlots = 4096;
__device__ unsigned long long g_queue_slots[kQueueSlots];
std::mutex g_queue_mu;
unsigned long long* g_queue_base[64] = {};
std::atomic<uint32_t> g_queue_next{0};

int next_queue_slot(unsigned long long** out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(WALK_B200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  {
    std::lock_guard<std::mutex> lock(g_queue_mu);
    if (!g_queue_base[dev]) {
      void* p = nullptr;
      CUDA_TRY(cudaGetSymbolAddress(&p, g_queue_slots));
      g_queue_base[dev] = static_cast<unsigned long long*>(p);
    }
  }
  *out = g_queue_base[dev] + (g_queue_next.fetch_add(1) % kQueueSlots);
  return WALK_B200_OK;
}

// Persistent launch: as many blocks as fit on the device at once (or fewer, if the batch is small).
template <typename K>
int launch_n2v_kernel(K kernel, const Node2vecParams& P0, cudaStream_t s, const char* name = "node2vec_walk_kernel") {
  Node2vecParams P = P0;
  if (int rc = next_queue_slot(&P.queue)) return rc;
  CUDA_TRY(cudaMemsetAsync(P.queue, 0, sizeof(unsigned long long), s));
  int per_sm = g_tuning.n2v_blocks_per_sm.load();
  if (per_sm <= 0) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, 0) != cudaSuccess || per_sm <= 0) {
      (void)cudaGetLastError();
      per_sm = 4;
    }
  }
  int64_t grid = (int64_t)sm_count() * per_sm;
  const int64_t needed = (P.num_walks + kBlock - 1) / kBlock;  // one chunk of 32 walks per warp at least
  if (grid > needed) grid = needed;
  if (grid < 1) grid = 1;
  kernel<<<(unsigned)grid, kBlock, 0, s>>>(P);
  return check_launch(name);
}

template <typename idx_t, int MEMBER, bool USE_DESC>
int launch_n2v_t(const Node2vecParams& P, cudaStream_t s) {
  const bool e = P.e_out != nullptr, c = P.counters != nullptr;
  if (c) {
    if (e) return launch_n2v_kernel(node2vec_walk_kernel<idx_t, MEMBER, USE_DESC, true, true>, P, s);
    return launch_n2v_kernel(node2vec_walk_kernel<idx_t, MEMBER, USE_DESC, false, true>, P, s);
  }
  if (e) return launch_n2v_kernel(node2vec_walk_kernel<idx_t, MEMBER, USE_DESC, true, false>, P, s);
  return launch_n2v_kernel(node2vec_walk_kernel<idx_t, MEMBER, USE_DESC, false, false>, P, s);
}

template <typename idx_t>
int launch_n2v_i(const Node2vecParams& P, int member, cudaStream_t s) {
  const bool d = P.desc != nullptr;
  switch (member) {
    case MEMBER_HASH:
      return d ? launch_n2v_t<idx_t, MEMBER_HASH, true>(P, s) : launch_n2v_t<idx_t, MEMBER_HASH, false>(P, s);
    case MEMBER_SEARCH_PREV:
      return d ? launch_n2v_t<idx_t, MEMBER_SEARCH_PREV, true>(P, s) : launch_n2v_t<idx_t, MEMBER_SEARCH_PREV, false>(P, s);
    default:
      return d ? launch_n2v_t<idx_t, MEMBER_SEARCH_CAND, true>(P, s) : launch_n2v_t<idx_t, MEMBER_SEARCH_CAND, false>(P, s);
  }
}

// The reverse-position shortcut costs one more 4-byte gather per step and saves the col gather of
// every attempt whose accept draw lies above both cut1 and cut2. Measured on R-MAT scale 24:
// (p,q)=(0.25,4) 266 -> 199 ms, (0.5,2) 92 -> 88 ms, but (1,2) 64 -> 80 ms and (1,1) 27 -> 45 ms,
// where no attempt can be skipped. It is used when at least half of the attempts are skippable.
bool rev_pays(const Node2vecParams& P) {
  const int mode = g_tuning.n2v_rev.load();
  if (mode == 0) return false;
  if (mode == 2) return true;
  const uint32_t top = P.cut1 > P.cut2 ? P.cut1 : P.cut2;
  return top <= (1u << 30);  // max(prob_1, prob_2) <= 0.5
}

// The pooled kernel covers the configuration with every per-graph structure present. It wins where
// steps are long (many rejected attempts per step, i.e. where the reverse positions pay: 123 vs
// 164 ms at (p, q) = (0.25, 4) on R-MAT 24) and loses where almost every first candidate is accepted
// and a step is three short trips (8.9 vs 7.9 ms at (1, 2) on R-MAT 22): 1 = where it wins, 2 = always.
bool pool_possible(const Node2vecParams& P, int member) {  // what the pooled kernels are built for
  return g_tuning.n2v_pool.load() != 0 && member == MEMBER_HASH && P.colrev && P.desc && !P.counters &&
         P.num_nodes <= 0x7fffffffll && P.num_edges < 0xfffffffell && P.edgeset_buckets < 0xffffffffull &&
         P.num_walks < 0xffffffffll && P.walk_length < 65536 && g_tuning.n2v_idx.load() != 1 &&
         g_tuning.n2v_rev.load() != 0;
}

bool pool_applies(const Node2vecParams& P, int member) {
  return pool_possible(P, member) && (g_tuning.n2v_pool.load() == 2 || rev_pays(P));
}

// The triangle filter speaks about "x is a neighbour of t"; the walk asks "t is a neighbour of x": undirected
// graphs only. With the filter the pooled form wins wherever membership tests occur at all, i.e. whenever
// prob_1 > prob_2 (q > 1): 6.26 against 7.16 ms for the per-lane kernel at (p, q) = (1, 2) on R-MAT 22, where the
// unfiltered pooled kernel needs 7.89. With counters it runs only when the caller asked for this kernel's own counts.
bool tri_applies(const Node2vecParams& P0, int member, bool sym) {
  if (!P0.colrev16 || !sym || P0.walk_length >= 32768 || g_tuning.n2v_tri.load() == 0) return false;
  Node2vecParams P = P0;
  if (P.counters) {
    if (g_tuning.n2v_count_kernel.load() != 1) return false;
    P.counters = nullptr;  // the pooled kernels leave instrumented launches to the per-lane kernel
  }
  return pool_possible(P, member) && (g_tuning.n2v_pool.load() == 2 || P.cut1 > P.cut2);
}

int launch_n2v(const Node2vecParams& P, bool sym, cudaStream_t s) {
  int member = sym ? MEMBER_SEARCH_PREV : MEMBER_SEARCH_CAND;
  if (P.edgeset && P.edgeset_buckets > 0 && g_tuning.n2v_member.load() != 1) member = MEMBER_HASH;
  // the triangle filter speaks about "x is a neighbour of t"; the walk asks "t is a neighbour of x": undirected graphs only
  if (tri_applies(P, member, sym)) {
    Node2vecParams T = P;
    T.draw_loop = g_tuning.n2v_tri_draw_loop.load() < 1 ? 1 : g_tuning.n2v_tri_draw_loop.load();
    if (T.counters) {
      if (T.e_out) return launch_n2v_kernel(node2vec_pool_tri_kernel<true, HOST_NONE, true>, T, s, "node2vec_pool_tri_kernel");
      return launch_n2v_kernel(node2vec_pool_tri_kernel<false, HOST_NONE, true>, T, s, "node2vec_pool_tri_kernel");
    }
    if (T.e_out) return launch_n2v_kernel(node2vec_pool_tri_kernel<true, HOST_NONE>, T, s, "node2vec_pool_tri_kernel");
    return launch_n2v_kernel(node2vec_pool_tri_kernel<false, HOST_NONE>, T, s, "node2vec_pool_tri_kernel");
  }
  if (pool_applies(P, member)) {
    if (P.e_out) return launch_n2v_kernel(node2vec_pool_kernel<true, false>, P, s, "node2vec_pool_kernel");
    return launch_n2v_kernel(node2vec_pool_kernel<false, false>, P, s, "node2vec_pool_kernel");
  }
  const bool fits32 = P.num_nodes <= 0x7fffffffll && P.num_edges <= 0xffffffffll;
  if (member == MEMBER_HASH && P.colrev && P.desc && fits32 && P.num_edges < 0xfffffffell &&
      g_tuning.n2v_idx.load() != 1 && rev_pays(P)) {
    const bool e = P.e_out != nullptr, c = P.counters != nullptr;
    if (c) {
      if (e) return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, true, true, true>, P, s);
      return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, false, true, true>, P, s);
    }
    if (e) return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, true, false, true>, P, s);
    return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, false, false, true>, P, s);
  }
  if (fits32 && g_tuning.n2v_idx.load() != 1) return launch_n2v_i<uint32_t>(P, member, s);
  return launch_n2v_i<int64_t>(P, member, s);
}

// Single-launch mode of the host entry point: kernels that report finished slabs and write int32 matrices
// (narrow transport) or int64 ones (wide). Built for 32-bit indices with row descriptors; returns
// kNoHostKernel for any other configuration (the caller then runs the slab pipeline).
constexpr int kNoHostKernel = -1;

template <int HOST>
int launch_n2v_host_t(const Node2vecParams& P, bool sym, cudaStream_t s) {
  const bool fits32 = P.num_nodes <= 0x7fffffffll && P.num_edges < 0x7fffffffll;
  if (!fits32 || !P.desc || P.counters || g_tuning.n2v_idx.load() == 1) return kNoHostKernel;
  const bool e = P.e_out != nullptr;
  int member = sym ? MEMBER_SEARCH_PREV : MEMBER_SEARCH_CAND;
  if (P.edgeset && P.edgeset_buckets > 0 && g_tuning.n2v_member.load() != 1) member = MEMBER_HASH;
  if (tri_applies(P, member, sym)) {
    Node2vecParams T = P;
    T.draw_loop = g_tuning.n2v_tri_draw_loop.load() < 1 ? 1 : g_tuning.n2v_tri_draw_loop.load();
    if (e) return launch_n2v_kernel(node2vec_pool_tri_kernel<true, HOST>, T, s, "node2vec_pool_tri_kernel");
    return launch_n2v_kernel(node2vec_pool_tri_kernel<false, HOST>, T, s, "node2vec_pool_tri_kernel");
  }
  if (pool_applies(P, member)) {
    if (e) return launch_n2v_kernel(node2vec_pool_kernel<true, HOST>, P, s, "node2vec_pool_kernel");
    return launch_n2v_kernel(node2vec_pool_kernel<false, HOST>, P, s, "node2vec_pool_kernel");
  }
  if (member == MEMBER_HASH && P.colrev && rev_pays(P)) {
    if (e) return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, true, false, true, HOST>, P, s);
    return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, false, false, true, HOST>, P, s);
  }
  switch (member) {
    case MEMBER_HASH:
      if (e) return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, true, false, false, HOST>, P, s);
      return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_HASH, true, false, false, false, HOST>, P, s);
    case MEMBER_SEARCH_PREV:
      if (e) return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_SEARCH_PREV, true, true, false, false, HOST>, P, s);
      return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_SEARCH_PREV, true, false, false, false, HOST>, P, s);
    default:
      if (e) return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_SEARCH_CAND, true, true, false, false, HOST>, P, s);
      return launch_n2v_kernel(node2vec_walk_kernel<uint32_t, MEMBER_SEARCH_CAND, true, false, false, false, HOST>, P, s);
  }
}

int launch_n2v_host(const Node2vecParams& P, bool sym, bool narrow, cudaStream_t s) {
  return narrow ? launch_n2v_host_t<HOST_NARROW>(P, sym, s) : launch_n2v_host_t<HOST_WIDE>(P, sym, s);
}

// Argument checks and kernel parameters shared by the device-pointer entry and the host entry.
int prepare_n2v(const walk_b200_csr* g, const int64_t* start, int64_t num_walks, int32_t walk_length,
                double p, double q, uint64_t seed, uint64_t walk_index_base, uint64_t walk_index_stride,
                int64_t* n_out, int64_t* e_out, uint32_t* status_flags, uint64_t* counters,
                Node2vecParams* out) {
  if (int rc = check_csr(g)) return rc;
  if (int rc = check_walk_sizes(num_walks, walk_length, start, n_out)) return rc;
  double prob[3];
  uint32_t cuts[3];
  if (int rc = thresholds(p, q, prob, cuts)) return rc;
  Node2vecParams P{};
  P.rowptr = g->rowptr; P.col = g->col; P.desc = g->rowdesc;
  P.num_nodes = g->num_nodes; P.num_edges = g->num_edges;
  P.start = start; P.num_walks = num_walks; P.walk_length = walk_length;
  P.cut0 = cuts[0]; P.cut1 = cuts[1]; P.cut2 = cuts[2];
  P.key0 = (uint32_t)seed; P.key1 = (uint32_t)(seed >> 32);
  P.walk_index_base = walk_index_base;
  P.walk_index_stride = walk_index_stride ? walk_index_stride : 1;
  {
    const int32_t cap = g_tuning.n2v_max_attempts.load();
    P.max_attempts = cap < 1 ? 1u : (uint32_t)cap > WALK_B200_MAX_ATTEMPTS ? WALK_B200_MAX_ATTEMPTS : (uint32_t)cap;
  }
  P.batch_lanes = g_tuning.n2v_batch_lanes.load();
  P.batch_trips = g_tuning.n2v_batch_trips.load();
  if (P.batch_lanes < 1) P.batch_lanes = 1;
  if (P.batch_trips < 1) P.batch_trips = 1;
  P.draw_loop = g_tuning.n2v_draw_loop.load();
  if (P.draw_loop < 1) P.draw_loop = 1;
  P.n_out = n_out; P.e_out = walk_length > 0 ? e_out : nullptr;
  P.flags = status_flags; P.counters = (unsigned long long*)counters;
  P.hints = g_tuning.l2_hints.load();
  if (g->edgeset && g->edgeset_buckets > 0) {
    if (g->num_nodes >= 0xffffffffll)
      return fail(WALK_B200_ERR_UNSUPPORTED, "the edge hash set needs num_nodes < 2^32 - 1");
    if ((reinterpret_cast<uintptr_t>(g->edgeset) & 31) != 0)
      return fail(WALK_B200_ERR_INVALID_ARG, "edgeset must be 32-byte aligned");
    P.edgeset = g->edgeset; P.edgeset_buckets = g->edgeset_buckets;
    P.colrev = g->colrev;
    if (g->colrev16 && g->colrev) {
      if ((reinterpret_cast<uintptr_t>(g->colrev16) & 15) != 0)
        return fail(WALK_B200_ERR_INVALID_ARG, "colrev16 must be 16-byte aligned");
      P.colrev16 = static_cast<const ulonglong2*>(g->colrev16);
    }
  }
  *out = P;
  return WALK_B200_OK;
}

int grid_for_streaming(int64_t n) {
  int64_t b = blocks_for(n);
  const int64_t cap = 148 * 16;  // 16 resident blocks' worth per SM of a 148-SM part
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace

namespace walk_b200 {
namespace host {

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int check_launch(const char* what) { return ::check_launch(what); }

int sm_count() { return ::sm_count(); }

}  // namespace host
}  // namespace walk_b200

// ======================================================================================
// C ABI
// ======================================================================================
extern "C" {

int walk_b200_abi_version(void) { return WALK_B200_ABI_VERSION; }

const char* walk_b200_last_error(void) { return g_last_error.c_str(); }

uint64_t walk_b200_launch_count(void) { return g_launches.load(); }

const char* walk_b200_last_kernel(void) { return g_last_kernel; }

int walk_b200_set_tuning(const char* key, int32_t value) {
  auto* slot = tuning_slot(key);
  if (!slot) return fail(WALK_B200_ERR_INVALID_ARG, "unknown tuning key '%s'", key ? key : "(null)");
  if (slot == &g_tuning.l2_fetch_granularity) {
    // per-context hint to the L2 on how much to fetch from DRAM per miss (32, 64 or 128 bytes)
    if (value != 32 && value != 64 && value != 128)
      return fail(WALK_B200_ERR_INVALID_ARG, "l2_fetch_granularity must be 32, 64 or 128");
    CUDA_TRY(cudaDeviceSetLimit(cudaLimitMaxL2FetchGranularity, (size_t)value));
  }
  slot->store(value);
  return WALK_B200_OK;
}

int walk_b200_get_tuning(const char* key, int32_t* value) {
  auto* slot = tuning_slot(key);
  if (!slot || !value) return fail(WALK_B200_ERR_INVALID_ARG, "unknown tuning key '%s'", key ? key : "(null)");
  *value = slot->load();
  return WALK_B200_OK;
}

void walk_b200_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
  const Philox4 o = philox4x32_10(counter[0], counter[1], counter[2], counter[3], key[0], key[1]);
  out[0] = o.x; out[1] = o.y; out[2] = o.z; out[3] = o.w;
}

void walk_b200_node2vec_draw(uint64_t seed, uint64_t walk, uint32_t step, uint32_t attempt,
                             uint32_t* candidate31, uint32_t* accept31) {
  uint32_t c, a;
  node2vec_draw((uint32_t)seed, (uint32_t)(seed >> 32), walk, step, attempt, c, a);
  if (candidate31) *candidate31 = c;
  if (accept31) *accept31 = a;
}

int walk_b200_node2vec_thresholds(double p, double q, double prob[3], uint32_t cuts[3]) {
  double pr[3];
  uint32_t cu[3];
  int rc = thresholds(p, q, pr, cu);
  if (rc) return rc;
  for (int k = 0; k < 3; k++) {
    if (prob) prob[k] = pr[k];
    if (cuts) cuts[k] = cu[k];
  }
  return WALK_B200_OK;
}

int walk_b200_shard_range(int64_t num_walks, int32_t world_size, int32_t rank, int64_t* begin, int64_t* end) {
  if (num_walks < 0 || world_size < 1 || rank < 0 || rank >= world_size || !begin || !end)
    return fail(WALK_B200_ERR_INVALID_ARG, "bad shard request (num_walks=%lld, world_size=%d, rank=%d)",
                (long long)num_walks, world_size, rank);
  const int64_t per = (num_walks + world_size - 1) / world_size;
  int64_t b = per * rank, e = b + per;
  if (b > num_walks) b = num_walks;
  if (e > num_walks) e = num_walks;
  *begin = b;
  *end = e;
  return WALK_B200_OK;
}

int walk_b200_shard_count_cyclic(int64_t num_walks, int32_t world_size, int32_t rank, int64_t* count) {
  if (num_walks < 0 || world_size < 1 || rank < 0 || rank >= world_size || !count)
    return fail(WALK_B200_ERR_INVALID_ARG, "bad shard request (num_walks=%lld, world_size=%d, rank=%d)",
                (long long)num_walks, world_size, rank);
  *count = num_walks > rank ? (num_walks - rank + world_size - 1) / world_size : 0;
  return WALK_B200_OK;
}

namespace {
int uniform_walk_impl(const walk_b200_csr* g, const int64_t* start, const float* rand, bool generate,
                      uint64_t seed, uint64_t base, uint64_t stride, int64_t num_walks, int32_t walk_length,
                      int64_t* n_out, int64_t* e_out, uint32_t* status_flags, void* stream);
}

int walk_b200_uniform_walk(const walk_b200_csr* g, const int64_t* start, const float* rand,
                           int64_t num_walks, int32_t walk_length, int64_t* n_out, int64_t* e_out,
                           uint32_t* status_flags, void* stream) {
  return uniform_walk_impl(g, start, rand, false, 0, 0, 1, num_walks, walk_length, n_out, e_out, status_flags, stream);
}

int walk_b200_uniform_walk_philox(const walk_b200_csr* g, const int64_t* start, int64_t num_walks,
                                  int32_t walk_length, uint64_t seed, uint64_t walk_index_base,
                                  uint64_t walk_index_stride, int64_t* n_out, int64_t* e_out,
                                  uint32_t* status_flags, void* stream) {
  return uniform_walk_impl(g, start, nullptr, true, seed, walk_index_base, walk_index_stride ? walk_index_stride : 1,
                           num_walks, walk_length, n_out, e_out, status_flags, stream);
}

void walk_b200_uniform_draw(uint64_t seed, uint64_t walk, uint32_t step, float* r) {
  const Philox4 b = uniform_block((uint32_t)seed, (uint32_t)(seed >> 32), walk, step >> 2);
  const uint32_t w = (step & 3) == 0 ? b.x : (step & 3) == 1 ? b.y : (step & 3) == 2 ? b.z : b.w;
  if (r) *r = uniform_from_word(w);
}

void walk_b200_uniform_draws(uint64_t seed, uint64_t walk_index_base, uint64_t walk_index_stride,
                             int64_t num_walks, int32_t walk_length, float* out) {
  if (!out || num_walks <= 0 || walk_length <= 0) return;
  if (walk_index_stride == 0) walk_index_stride = 1;
  for (int64_t w = 0; w < num_walks; w++) {
    const uint64_t gw = walk_index_base + (uint64_t)w * walk_index_stride;
    for (int32_t l = 0; l < walk_length; l += 4) {
      const Philox4 b = uniform_block((uint32_t)seed, (uint32_t)(seed >> 32), gw, (uint32_t)l >> 2);
      const uint32_t words[4] = {b.x, b.y, b.z, b.w};
      for (int k = 0; k < 4 && l + k < walk_length; k++) out[w * walk_length + l + k] = uniform_from_word(words[k]);
    }
  }
}

namespace {
int uniform_walk_impl(const walk_b200_csr* g, const int64_t* start, const float* rand, bool generate,
                      uint64_t seed, uint64_t base, uint64_t stride, int64_t num_walks, int32_t walk_length,
                      int64_t* n_out, int64_t* e_out, uint32_t* status_flags, void* stream) {
  if (int rc = check_csr(g)) return rc;
  if (int rc = check_walk_sizes(num_walks, walk_length, start, n_out)) return rc;
  if (!generate && num_walks > 0 && walk_length > 0 && !rand) return fail(WALK_B200_ERR_INVALID_ARG, "rand is NULL");
  if (num_walks == 0) return WALK_B200_OK;
  UniformParams P{};
  P.key0 = (uint32_t)seed; P.key1 = (uint32_t)(seed >> 32);
  P.walk_index_base = base; P.walk_index_stride = stride;
  P.rowptr = g->rowptr; P.col = g->col; P.desc = g->rowdesc;
  P.num_nodes = g->num_nodes; P.num_edges = g->num_edges;
  P.start = start; P.rand = rand; P.num_walks = num_walks; P.walk_length = walk_length;
  P.n_out = n_out; P.e_out = walk_length > 0 ? e_out : nullptr; P.flags = status_flags;
  P.hints = g_tuning.l2_hints.load();
  if (g->fused && g->rowdesc) {
    if ((reinterpret_cast<uintptr_t>(g->fused) & 15) != 0)
      return fail(WALK_B200_ERR_INVALID_ARG, "fused edge records must be 16-byte aligned");
    P.fused = static_cast<const ulonglong2*>(g->fused);
  }
  P.generate = generate ? 1 : 0;
  return launch_uniform(P, (cudaStream_t)stream);
}
}  // namespace

int walk_b200_node2vec_walk(const walk_b200_csr* g, const int64_t* start, int64_t num_walks,
                            int32_t walk_length, double p, double q, uint64_t seed,
                            uint64_t walk_index_base, uint64_t walk_index_stride, int64_t* n_out,
                            int64_t* e_out, uint32_t* status_flags, uint64_t* counters, void* stream) {
  Node2vecParams P{};
  if (int rc = prepare_n2v(g, start, num_walks, walk_length, p, q, seed, walk_index_base, walk_index_stride,
                           n_out, e_out, status_flags, counters, &P))
    return rc;
  if (num_walks == 0) return WALK_B200_OK;
  return launch_n2v(P, (g->flags & WALK_B200_CSR_SYMMETRIC) != 0, (cudaStream_t)stream);
}

int walk_b200_rowdesc_pack(const int64_t* rowptr, int64_t num_nodes, int64_t num_edges,
                           uint64_t* rowdesc, uint32_t* status_flags, void* stream) {
  if (num_nodes < 0 || num_edges < 0) return fail(WALK_B200_ERR_INVALID_ARG, "negative graph size");
  if (!rowptr || (num_nodes > 0 && !rowdesc)) return fail(WALK_B200_ERR_INVALID_ARG, "rowptr or rowdesc is NULL");
  if (num_nodes == 0) return WALK_B200_OK;
  rowdesc_pack_kernel<<<grid_for_streaming(num_nodes), kBlock, 0, (cudaStream_t)stream>>>(
      rowptr, num_nodes, num_edges, rowdesc, status_flags);
  return check_launch("rowdesc_pack_kernel");
}

int walk_b200_edgeset_buckets(int64_t num_edges, uint64_t* buckets) {
  if (num_edges < 0 || !buckets) return fail(WALK_B200_ERR_INVALID_ARG, "bad edge count or NULL result");
  // load factor 0.5: two slots per edge, four slots per bucket; never empty
  uint64_t b = ((uint64_t)num_edges * 2 + kEdgeSlotsPerBucket - 1) / kEdgeSlotsPerBucket;
  *buckets = b < 64 ? 64 : b;
  return WALK_B200_OK;
}

int walk_b200_edgeset_build(const walk_b200_csr* g, uint64_t* table, uint64_t buckets,
                            uint32_t* status_flags, void* stream) {
  if (int rc = check_csr(g)) return rc;
  if (!table || buckets == 0) return fail(WALK_B200_ERR_INVALID_ARG, "edge set table is NULL or empty");
  if ((reinterpret_cast<uintptr_t>(table) & 31) != 0)
    return fail(WALK_B200_ERR_INVALID_ARG, "edge set table must be 32-byte aligned");
  if (g->num_nodes >= 0xffffffffll)
    return fail(WALK_B200_ERR_UNSUPPORTED, "the edge hash set needs num_nodes < 2^32 - 1");
  if (buckets * kEdgeSlotsPerBucket < (uint64_t)g->num_edges + (uint64_t)g->num_edges / 4)
    return fail(WALK_B200_ERR_INVALID_ARG, "edge set table too small: %llu buckets for %lld edges",
                (unsigned long long)buckets, (long long)g->num_edges);
  CUDA_TRY(cudaMemsetAsync(table, 0xff, buckets * kEdgeSlotsPerBucket * sizeof(uint64_t), (cudaStream_t)stream));
  if (g->num_edges == 0) return WALK_B200_OK;
  edgeset_build_kernel<<<grid_for_streaming(g->num_edges), kBlock, 0, (cudaStream_t)stream>>>(
      g->rowptr, g->col, g->num_nodes, g->num_edges, (unsigned long long*)table, buckets, status_flags);
  return check_launch("edgeset_build_kernel");
}

int walk_b200_fused_build(const walk_b200_csr* g, void* fused, uint32_t* status_flags, void* stream) {
  if (int rc = check_csr(g)) return rc;
  if (!g->rowdesc) return fail(WALK_B200_ERR_INVALID_ARG, "fused edge records need the row descriptors (rowdesc is NULL)");
  if (g->num_edges > 0 && !fused) return fail(WALK_B200_ERR_INVALID_ARG, "fused is NULL");
  if ((reinterpret_cast<uintptr_t>(fused) & 15) != 0)
    return fail(WALK_B200_ERR_INVALID_ARG, "fused edge records must be 16-byte aligned");
  if (g->num_edges == 0) return WALK_B200_OK;
  fused_build_kernel<<<grid_for_streaming(g->num_edges), kBlock, 0, (cudaStream_t)stream>>>(
      g->col, g->rowdesc, g->num_nodes, g->num_edges, static_cast<ulonglong2*>(fused), status_flags);
  return check_launch("fused_build_kernel");
}

int walk_b200_colrev_build(const walk_b200_csr* g, uint64_t* colrev, uint32_t* status_flags, void* stream) {
  if (int rc = check_csr(g)) return rc;
  if (!g->revpos) return fail(WALK_B200_ERR_INVALID_ARG, "colrev is built from the reverse positions (revpos is NULL)");
  if (g->num_edges > 0 && !colrev) return fail(WALK_B200_ERR_INVALID_ARG, "colrev is NULL");
  if (g->num_nodes >= 0xffffffffll) return fail(WALK_B200_ERR_UNSUPPORTED, "colrev needs num_nodes < 2^32 - 1");
  if (g->num_edges == 0) return WALK_B200_OK;
  colrev_build_kernel<<<grid_for_streaming(g->num_edges), kBlock, 0, (cudaStream_t)stream>>>(
      g->col, g->revpos, g->num_nodes, g->num_edges, colrev, status_flags);
  return check_launch("colrev_build_kernel");
}

int walk_b200_trifilter_build(const walk_b200_csr* g, void* colrev16, int64_t max_row, uint32_t* status_flags,
                              void* stream) {
  (void)status_flags;
  if (int rc = check_csr(g)) return rc;
  if (!(g->flags & WALK_B200_CSR_SYMMETRIC))
    return fail(WALK_B200_ERR_INVALID_ARG, "the triangle filter is only valid on a graph declared undirected (WALK_B200_CSR_SYMMETRIC)");
  if (!g->colrev || !g->edgeset || g->edgeset_buckets == 0)
    return fail(WALK_B200_ERR_INVALID_ARG, "the triangle filter is built from colrev and the edge hash set (one of them is NULL)");
  if (g->num_edges > 0 && !colrev16) return fail(WALK_B200_ERR_INVALID_ARG, "colrev16 is NULL");
  if ((reinterpret_cast<uintptr_t>(colrev16) & 15) != 0 || (reinterpret_cast<uintptr_t>(g->edgeset) & 31) != 0)
    return fail(WALK_B200_ERR_INVALID_ARG, "colrev16 must be 16-byte aligned (and the edge set 32-byte aligned)");
  if (max_row < 0) return fail(WALK_B200_ERR_INVALID_ARG, "max_row is negative");
  if (g->num_edges == 0) return WALK_B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // all ones = "maybe" for every position: what an edge keeps when the kernel leaves it out
  CUDA_TRY(cudaMemsetAsync(colrev16, 0xff, (size_t)g->num_edges * 16, s));
  unsigned long long* queue = nullptr;
  if (int rc = next_queue_slot(&queue)) return rc;
  CUDA_TRY(cudaMemsetAsync(queue, 0, sizeof(unsigned long long), s));
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, trifilter_build_kernel, kBlock, 0) != cudaSuccess || per_sm <= 0) {
    (void)cudaGetLastError();
    per_sm = 4;
  }
  int64_t grid = (int64_t)sm_count() * per_sm;
  const int64_t needed = (g->num_edges + 64 * kWarpsPerBlock - 1) / (64 * kWarpsPerBlock);
  if (grid > needed) grid = needed;
  trifilter_build_kernel<<<(unsigned)grid, kBlock, 0, s>>>(g->rowptr, g->col, g->colrev, g->edgeset, g->edgeset_buckets,
                                                          g->num_nodes, g->num_edges, max_row,
                                                          static_cast<ulonglong2*>(colrev16), queue);
  return check_launch("trifilter_build_kernel");
}

int walk_b200_revpos_build(const walk_b200_csr* g, uint32_t* revpos, uint32_t* status_flags, void* stream) {
  if (int rc = check_csr(g)) return rc;
  if (g->num_edges > 0 && !revpos) return fail(WALK_B200_ERR_INVALID_ARG, "revpos is NULL");
  if (g->num_edges >= 0xfffffffell)
    return fail(WALK_B200_ERR_UNSUPPORTED, "reverse positions are 32-bit: num_edges must be below 2^32 - 2");
  if (g->num_edges == 0) return WALK_B200_OK;
  revpos_build_kernel<<<grid_for_streaming(g->num_edges), kBlock, 0, (cudaStream_t)stream>>>(
      g->rowptr, g->col, g->num_nodes, g->num_edges, revpos, status_flags);
  return check_launch("revpos_build_kernel");
}

int walk_b200_csr_validate(const walk_b200_csr* g, const int64_t* start, int64_t num_walks,
                           int32_t check_sorted, uint32_t* status_flags, void* stream) {
  if (int rc = check_csr(g)) return rc;
  if (!status_flags) return fail(WALK_B200_ERR_INVALID_ARG, "status_flags is required");
  if (num_walks < 0) return fail(WALK_B200_ERR_INVALID_ARG, "num_walks is negative");
  int64_t work = g->num_nodes;
  if (g->num_edges > work) work = g->num_edges;
  if (num_walks > work) work = num_walks;
  csr_validate_kernel<<<grid_for_streaming(work), kBlock, 0, (cudaStream_t)stream>>>(
      g->rowptr, g->col, g->num_nodes, g->num_edges, start, start ? num_walks : 0, check_sorted, status_flags);
  return check_launch("csr_validate_kernel");
}

// ---- consumer of the walk matrix ----------------------------------------------------
int walk_b200_context_windows(const int64_t* walks, int64_t num_walks, int32_t walk_length,
                              int32_t context_size, int64_t* windows, void* stream) {
  if (num_walks < 0 || walk_length < 0) return fail(WALK_B200_ERR_INVALID_ARG, "negative size");
  if (context_size < 1 || context_size > walk_length + 1)
    return fail(WALK_B200_ERR_INVALID_ARG, "context_size must be in [1, walk_length + 1] (got %d for walk_length %d)",
                context_size, walk_length);
  const int64_t nwin = (int64_t)walk_length + 2 - context_size;
  const int64_t per_walk = nwin * context_size;
  if (per_walk > 0x7fffffffll) return fail(WALK_B200_ERR_UNSUPPORTED, "one walk yields more than 2^31 window elements");
  if (num_walks == 0) return WALK_B200_OK;
  if (!walks || !windows) return fail(WALK_B200_ERR_INVALID_ARG, "walks or windows is NULL");
  const int64_t bx = (per_walk + 2 * kBlock - 1) / (2 * kBlock);
  dim3 grid((unsigned)(bx < 64 ? bx : 64), (unsigned)(num_walks < 65535 ? num_walks : 65535), 1);
  // division by context_size as a multiply-high when that is exact for every element index of a walk
  const uint64_t magic = (1ull << 32) / (uint64_t)context_size + 1;
  const bool fast = magic <= 0xffffffffull &&
                    (uint64_t)per_walk * (magic * (uint64_t)context_size - (1ull << 32)) < (1ull << 32);
  if ((reinterpret_cast<uintptr_t>(walks) & 7) != 0 || (reinterpret_cast<uintptr_t>(windows) & 7) != 0)
    return fail(WALK_B200_ERR_INVALID_ARG, "walks and windows must be 8-byte aligned");
  // the kernel stores pairs of elements with one 16-byte store where the pair starts on a 16-byte boundary;
  // which pairs do depends on where the caller's matrix starts (a view that begins at an odd element is fine)
  const bool base_aligned = (reinterpret_cast<uintptr_t>(windows) & 15) == 0;
  if (fast)
    context_windows_kernel<true><<<grid, kBlock, 0, (cudaStream_t)stream>>>(
        walks, num_walks, walk_length + 1, context_size, (uint32_t)magic, (int32_t)per_walk, windows, base_aligned);
  else
    context_windows_kernel<false><<<grid, kBlock, 0, (cudaStream_t)stream>>>(
        walks, num_walks, walk_length + 1, context_size, 0u, (int32_t)per_walk, windows, base_aligned);
  return check_launch("context_windows_kernel");
}

int walk_b200_negative_walks(const int64_t* start, int64_t num_rows, int32_t walk_length, int64_t num_nodes,
                             uint64_t seed, uint64_t row_index_base, uint64_t row_index_stride, int64_t* out,
                             void* stream) {
  if (num_rows < 0 || walk_length < 0) return fail(WALK_B200_ERR_INVALID_ARG, "negative size");
  if (num_nodes < 1 || num_nodes > (1ll << 32))
    return fail(WALK_B200_ERR_UNSUPPORTED, "negative sampling draws from [0, num_nodes) with 1 <= num_nodes <= 2^32");
  if (num_rows == 0) return WALK_B200_OK;
  if (!start || !out) return fail(WALK_B200_ERR_INVALID_ARG, "start or out is NULL");
  const uint32_t quads = walk_length > 0 ? (uint32_t)((walk_length + 3) / 4) : 1u;
  if (num_rows > INT64_MAX / 8 / ((int64_t)walk_length + 1)) return fail(WALK_B200_ERR_INVALID_ARG, "matrix too large");
  int64_t blocks = blocks_for(num_rows * (int64_t)quads);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  negative_walks_kernel<<<(unsigned)blocks, kBlock, 0, (cudaStream_t)stream>>>(
      start, num_rows, walk_length, quads, (uint64_t)num_nodes, (uint32_t)seed, (uint32_t)(seed >> 32), row_index_base,
      row_index_stride ? row_index_stride : 1, out);
  return check_launch("negative_walks_kernel");
}

int walk_b200_negative_draw(uint64_t seed, uint64_t row, uint32_t k, int64_t num_nodes, int64_t* node) {
  if (!node) return fail(WALK_B200_ERR_INVALID_ARG, "node is NULL");
  if (num_nodes < 1 || num_nodes > (1ll << 32)) return fail(WALK_B200_ERR_UNSUPPORTED, "num_nodes must be in [1, 2^32]");
  const Philox4 b = negative_block((uint32_t)seed, (uint32_t)(seed >> 32), row, k >> 2);
  const uint32_t w[4] = {b.x, b.y, b.z, b.w};
  *node = negative_from_word(w[k & 3], (uint64_t)num_nodes);
  return WALK_B200_OK;
}

}  // extern "C"

// ---- device probe -------------------------------------------------------------------
namespace {
typedef void (*ProbeKernel)(const int64_t*, uint64_t, int, int64_t*);

template <int CHAINS>
ProbeKernel probe_kernel_for(int bytes, bool fetch64) {
  if (bytes == 8) return fetch64 ? gather_probe_kernel<CHAINS, 8, true> : gather_probe_kernel<CHAINS, 8, false>;
  if (bytes == 16) return fetch64 ? gather_probe_kernel<CHAINS, 16, true> : gather_probe_kernel<CHAINS, 16, false>;
  return fetch64 ? gather_probe_kernel<CHAINS, 32, true> : gather_probe_kernel<CHAINS, 32, false>;
}
}  // namespace

extern "C" {

int walk_b200_gather_probe_ex(size_t array_bytes, int32_t iters, int32_t chains, int32_t gather_bytes,
                              int32_t fetch_bytes, int32_t threads_per_sm, double* gathers_per_second) {
  if (!gathers_per_second || iters < 1 || array_bytes < (1u << 20))
    return fail(WALK_B200_ERR_INVALID_ARG, "gather probe needs an array of at least 1 MiB and iters >= 1");
  if (chains != 1 && chains != 2 && chains != 4)
    return fail(WALK_B200_ERR_INVALID_ARG, "gather probe: chains must be 1, 2 or 4");
  if (gather_bytes != 8 && gather_bytes != 16 && gather_bytes != 32)
    return fail(WALK_B200_ERR_INVALID_ARG, "gather probe: gather_bytes must be 8, 16 or 32");
  if (fetch_bytes != 64 && fetch_bytes != 128)
    return fail(WALK_B200_ERR_INVALID_ARG, "gather probe: fetch_bytes must be 64 or 128");
  if (threads_per_sm != 0 && (threads_per_sm < kBlock || threads_per_sm > 2048 || threads_per_sm % kBlock))
    return fail(WALK_B200_ERR_INVALID_ARG, "gather probe: threads_per_sm must be 0 or a multiple of %d up to 2048", kBlock);
  *gathers_per_second = 0.0;
  const ProbeKernel kernel = chains == 1 ? probe_kernel_for<1>(gather_bytes, fetch_bytes == 64)
                           : chains == 2 ? probe_kernel_for<2>(gather_bytes, fetch_bytes == 64)
                                         : probe_kernel_for<4>(gather_bytes, fetch_bytes == 64);
  int64_t* data = nullptr;
  int64_t* sink = nullptr;
  cudaEvent_t a = nullptr, b = nullptr;
  const uint64_t n = array_bytes / 32 * 4;  // whole 32-byte pieces, so that every gather width divides the array
  // threads_per_sm = 0: 2^22 threads, several waves of full occupancy; otherwise one wave of that many per SM
  const int64_t threads = threads_per_sm ? (int64_t)sm_count() * threads_per_sm : (int64_t)1 << 22;
  int rc = WALK_B200_OK;
  auto cleanup = [&]() {
    if (a) cudaEventDestroy(a);
    if (b) cudaEventDestroy(b);
    if (data) cudaFree(data);
    if (sink) cudaFree(sink);
  };
#define P_TRY(expr)                                                                                    \
  do {                                                                                                 \
    cudaError_t err__ = (expr);                                                                        \
    if (err__ != cudaSuccess) {                                                                        \
      rc = fail(WALK_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));                \
      cleanup();                                                                                       \
      return rc;                                                                                       \
    }                                                                                                  \
  } while (0)
  P_TRY(cudaMalloc((void**)&data, n * 8));
  P_TRY(cudaMalloc((void**)&sink, 8));
  P_TRY(cudaMemset(data, 0, n * 8));
  P_TRY(cudaEventCreate(&a));
  P_TRY(cudaEventCreate(&b));
  const unsigned grid = (unsigned)(threads / kBlock);
  kernel<<<grid, kBlock>>>(data, n, iters, sink);  // warm-up
  if ((rc = check_launch("gather_probe_kernel"))) { cleanup(); return rc; }
  P_TRY(cudaEventRecord(a));
  kernel<<<grid, kBlock>>>(data, n, iters, sink);
  if ((rc = check_launch("gather_probe_kernel"))) { cleanup(); return rc; }
  P_TRY(cudaEventRecord(b));
  P_TRY(cudaEventSynchronize(b));
  float ms = 0.f;
  P_TRY(cudaEventElapsedTime(&ms, a, b));
#undef P_TRY
  cleanup();
  if (ms > 0.f) *gathers_per_second = (double)threads * iters * chains / (ms * 1e-3);
  return WALK_B200_OK;
}

int walk_b200_gather_probe(size_t array_bytes, int32_t iters, double* gathers_per_second) {
  return walk_b200_gather_probe_ex(array_bytes, iters, 1, 8, 64, 0, gathers_per_second);
}

// ---- L2 residency hint -------------------------------------------------------------
int walk_b200_l2_window_set(const void* ptr, size_t bytes, float hit_ratio, void* stream, size_t* granted_bytes) {
  if (granted_bytes) *granted_bytes = 0;
  if (!ptr || bytes == 0) return fail(WALK_B200_ERR_INVALID_ARG, "empty L2 window");
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  int max_window = 0, max_persist = 0;
  CUDA_TRY(cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, dev));
  CUDA_TRY(cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, dev));
  if (max_window <= 0 || max_persist <= 0) return WALK_B200_OK;  // nothing on offer: not an error
  const size_t carve = bytes < (size_t)max_persist ? bytes : (size_t)max_persist;
  if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, carve) != cudaSuccess) {
    (void)cudaGetLastError();  // carve-out refused (e.g. a shared-context configuration): run without the hint
    return WALK_B200_OK;
  }
  size_t win = bytes < (size_t)max_window ? bytes : (size_t)max_window;
  cudaStreamAttrValue attr;
  memset(&attr, 0, sizeof(attr));
  attr.accessPolicyWindow.base_ptr = const_cast<void*>(ptr);
  attr.accessPolicyWindow.num_bytes = win;
  float ratio = hit_ratio;
  if (!(ratio > 0.f) || ratio > 1.f) {
    // fill the carve-out once: hit the fraction of the window that fits
    ratio = win <= (size_t)max_persist ? 1.f : (float)max_persist / (float)win;
  }
  attr.accessPolicyWindow.hitRatio = ratio;
  attr.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
  attr.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
  CUDA_TRY(cudaStreamSetAttribute((cudaStream_t)stream, cudaStreamAttributeAccessPolicyWindow, &attr));
  if (granted_bytes) *granted_bytes = win;
  return WALK_B200_OK;
}

int walk_b200_l2_window_clear(void* stream) {
  cudaStreamAttrValue attr;
  memset(&attr, 0, sizeof(attr));
  attr.accessPolicyWindow.num_bytes = 0;
  attr.accessPolicyWindow.hitProp = cudaAccessPropertyNormal;
  attr.accessPolicyWindow.missProp = cudaAccessPropertyNormal;
  CUDA_TRY(cudaStreamSetAttribute((cudaStream_t)stream, cudaStreamAttributeAccessPolicyWindow, &attr));
  CUDA_TRY(cudaCtxResetPersistingL2Cache());
  // give the carve-out back: while it is set aside, ordinary traffic has that much less L2
  if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, 0) != cudaSuccess) (void)cudaGetLastError();
  return WALK_B200_OK;
}

}  // extern "C"

// ======================================================================================
// Entry point that allocates nothing
// ======================================================================================
// Scratch for callers that cannot allocate: the packed row descriptors live in this
// fixed array of the library's device image instead of caller or pool memory. In host
// code the name below is only a handle for the runtime, never a device address; the
// address each device gave the array is looked up once and cached in noalloc_scratch().
static __device__ __align__(256) unsigned long long g_noalloc_rowdesc[WALK_B200_NOALLOC_MAX_NODES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
uint64_t* g_noalloc_ptr[kMaxDevices] = {};

// Device address of g_noalloc_rowdesc on the current device (set-up on first use).
int noalloc_scratch(uint64_t** out) {
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(WALK_B200_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_rowdesc));
    if (!p) return fail(WALK_B200_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_noalloc_ptr[dev] = static_cast<uint64_t*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return WALK_B200_OK;
}

}  // namespace

extern "C" int walk_b200_uniform_walk_noalloc(const int64_t* rowptr, const int64_t* col, int64_t num_nodes,
                                              int64_t num_edges, const int64_t* start, const float* rand,
                                              int64_t num_walks, int32_t walk_length, int64_t* n_out,
                                              int64_t* e_out, uint32_t* status_flags, void* stream) {
  walk_b200_csr g{};
  g.rowptr = rowptr; g.col = col; g.num_nodes = num_nodes; g.num_edges = num_edges;
  if (int rc = check_csr(&g)) return rc;
  if (int rc = check_walk_sizes(num_walks, walk_length, start, n_out)) return rc;
  if (num_walks > 0 && walk_length > 0 && !rand) return fail(WALK_B200_ERR_INVALID_ARG, "rand is NULL");
  if (num_nodes > WALK_B200_NOALLOC_MAX_NODES)
    return fail(WALK_B200_ERR_UNSUPPORTED,
                "graph has %lld nodes; the built-in scratch of walk_b200_uniform_walk_noalloc holds %d "
                "(use walk_b200_uniform_walk with caller-provided rowdesc, or rowdesc = NULL)",
                (long long)num_nodes, WALK_B200_NOALLOC_MAX_NODES);
  if ((uint64_t)num_edges > kDescStartMask)
    return fail(WALK_B200_ERR_UNSUPPORTED, "graph has %lld edges; row descriptors address at most 2^36",
                (long long)num_edges);
  if (num_walks == 0) return WALK_B200_OK;
  uint64_t* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  if (num_nodes > 0) {
    // rewrites entries [0, num_nodes): whatever an earlier call left there is never read
    rowdesc_pack_kernel<<<grid_for_streaming(num_nodes), kBlock, 0, (cudaStream_t)stream>>>(
        rowptr, num_nodes, num_edges, scratch, status_flags);
    if (int rc = check_launch("rowdesc_pack_kernel")) return rc;
  }
  UniformParams P{};
  P.walk_index_stride = 1;
  P.rowptr = rowptr; P.col = col; P.desc = num_nodes > 0 ? scratch : nullptr;
  P.num_nodes = num_nodes; P.num_edges = num_edges;
  P.start = start; P.rand = rand; P.num_walks = num_walks; P.walk_length = walk_length;
  P.n_out = n_out; P.e_out = walk_length > 0 ? e_out : nullptr; P.flags = status_flags;
  P.hints = g_tuning.l2_hints.load();
  return launch_uniform(P, (cudaStream_t)stream);
}

// ======================================================================================
// Resident graph + host-buffer entry points
// ======================================================================================
struct walk_b200_graph {
  int device = 0;
  int64_t num_nodes = 0, num_edges = 0;
  uint32_t csr_flags = 0;
  int64_t* d_rowptr = nullptr;
  int64_t* d_col = nullptr;
  uint64_t* d_desc = nullptr;
  uint64_t* d_edgeset = nullptr;
  uint64_t edgeset_buckets = 0;
  uint64_t* d_colrev = nullptr;
  void* d_colrev16 = nullptr;
  void* d_fused = nullptr;
  uint32_t* d_flags = nullptr;
  static constexpr int kLanes = 4;  // slabs in flight: copy-in, kernel, copy-out, host widening
  cudaStream_t streams[kLanes] = {};
  cudaEvent_t landed[kLanes] = {};  // narrow transport: the slab's int32 copy is in host staging
  int64_t* d_start[kLanes] = {};
  float* d_rand[kLanes] = {};
  int64_t* d_out[kLanes] = {};
  int64_t* d_eout[kLanes] = {};
  int32_t* d_pack[kLanes] = {};     // narrow transport: int32 copies of d_out / d_eout ...
  int32_t* d_epack[kLanes] = {};
  int32_t* h_pack[kLanes] = {};     // ... and their pinned host staging
  int32_t* h_epack[kLanes] = {};
  size_t cap_start = 0, cap_rand = 0, cap_out = 0, cap_eout = 0;  // bytes per lane
  size_t cap_pack = 0, cap_epack = 0, cap_hpack = 0, cap_hepack = 0;
  // single-launch mode of the node2vec host entry: all start rows, the whole int32 walk (and edge)
  // matrix, per-slab counters of finished walks, and the per-slab flags the kernel sets (mapped host memory)
  int64_t* d_start_all = nullptr;
  int32_t* d_all = nullptr;
  int32_t* d_eall = nullptr;
  uint32_t* d_slab_done = nullptr;
  uint32_t* h_slab_flags = nullptr;
  size_t cap_start_all = 0, cap_all = 0, cap_eall = 0, cap_slab_done = 0, cap_slab_flags = 0;
  std::unique_ptr<WidenPool> pool;
  // transport of the walk matrices to host buffers, measured once at creation (host_narrow = 2):
  // pinned device-to-host copy rate and the widening threads' output rate, both in GB/s
  bool prefer_narrow = true;
  double measured_d2h_gbs = 0.0, measured_widen_gbs = 0.0;
  std::mutex mu;
};

namespace {

struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) ok = true;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

template <typename T>
int grow(T** bufs, size_t* cap, size_t need) {
  if (need <= *cap) return WALK_B200_OK;
  for (int k = 0; k < walk_b200_graph::kLanes; k++) {
    if (bufs[k]) cudaFree(bufs[k]);
    bufs[k] = nullptr;
  }
  *cap = 0;
  for (int k = 0; k < walk_b200_graph::kLanes; k++) CUDA_TRY(cudaMalloc((void**)&bufs[k], need));
  *cap = need;
  return WALK_B200_OK;
}

int grow_pinned(int32_t** bufs, size_t* cap, size_t need) {
  if (need <= *cap) return WALK_B200_OK;
  for (int k = 0; k < walk_b200_graph::kLanes; k++) {
    if (bufs[k]) cudaFreeHost(bufs[k]);
    bufs[k] = nullptr;
  }
  *cap = 0;
  for (int k = 0; k < walk_b200_graph::kLanes; k++) CUDA_TRY(cudaHostAlloc((void**)&bufs[k], need, cudaHostAllocDefault));
  *cap = need;
  return WALK_B200_OK;
}

template <typename T>
int grow_one(T** buf, size_t* cap, size_t need) {
  if (need <= *cap) return WALK_B200_OK;
  if (*buf) cudaFree(*buf);
  *buf = nullptr;
  *cap = 0;
  CUDA_TRY(cudaMalloc((void**)buf, need));
  *cap = need;
  return WALK_B200_OK;
}

int ensure_pool(walk_b200_graph* g) {
  int want_threads = g_tuning.host_threads.load();
  if (want_threads <= 0) {
    want_threads = (int)std::thread::hardware_concurrency();
    if (want_threads > 16) want_threads = 16;
    if (want_threads < 1) want_threads = 1;
  }
  if (!g->pool || g->pool->workers() != want_threads - 1) g->pool.reset(new WidenPool(want_threads - 1));
  return WALK_B200_OK;
}

int launch_narrow(const int64_t* in, int64_t count, int32_t* out, cudaStream_t s) {
  if (count <= 0) return WALK_B200_OK;
  int64_t blocks = blocks_for((count + 3) / 4);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  narrow_i64_kernel<<<(unsigned)blocks, kBlock, 0, s>>>(in, count, out);
  return check_launch("narrow_i64_kernel");
}

int flags_to_status(uint32_t f) {
  if (!f) return WALK_B200_OK;
  return fail(WALK_B200_ERR_DEVICE_FLAGS,
              "kernel raised status flags 0x%x:%s%s%s%s%s%s%s", f,
              (f & WALK_B200_FLAG_BAD_NODE) ? " node id out of range;" : "",
              (f & WALK_B200_FLAG_BAD_EDGE) ? " edge index out of range (rand outside [0,1)?);" : "",
              (f & WALK_B200_FLAG_ATTEMPT_CAP) ? " rejection attempt cap hit;" : "",
              (f & WALK_B200_FLAG_BAD_ROWPTR) ? " rowptr malformed;" : "",
              (f & WALK_B200_FLAG_DESC_OVERFLOW) ? " row descriptor overflow;" : "",
              (f & WALK_B200_FLAG_UNSORTED_ROW) ? " row not strictly ascending;" : "",
              (f & WALK_B200_FLAG_EDGESET_FULL) ? " edge hash set overflow;" : "");
}

// Which transport a call uses for matrices whose ids fit 31 bits: the tuning decides, or (host_narrow = 2)
// the measurement taken when the graph was created.
bool use_narrow(const walk_b200_graph* g, bool ids_fit) {
  const int mode = g_tuning.host_narrow.load();
  if (!ids_fit || mode == 0) return false;
  if (mode == 1) return true;
  return g->prefer_narrow;
}

// node2vec over host buffers as ONE launch: all start rows go up, the kernel writes matrices that stay on
// the device, counts finished walks per slab of 2^shift rows and sets a flag in mapped host memory when a
// slab is complete. The host copies each complete slab out on a second stream while the launch goes on.
// Narrow transport: the matrices are int32, a slab lands in pinned staging and host threads widen it into
// the caller's int64 buffers. Wide transport: the matrices are int64 and a slab is copied straight into the
// caller's buffers (pinned ones, or the copy does not overlap). Against one launch per slab this removes the
// drain at the end of every launch (each costs about as long as the slowest walk of the slab; consecutive
// launches of a persistent kernel barely overlap). The kernel never waits for the host. Returns
// kNoHostKernel (before doing anything) when this mode does not apply; the caller then runs the slab
// pipeline. Called with g->mu held and the graph's device current.
int run_host_n2v_single(walk_b200_graph* g, const walk_b200_csr& csr, bool narrow, const int64_t* h_start, int64_t n,
                        int32_t L, double p, double q, uint64_t seed, uint64_t base, uint64_t stride, int64_t* h_n_out,
                        int64_t* h_e_out) {
  constexpr int kLanes = walk_b200_graph::kLanes;
  const bool want_e = h_e_out && L > 0;
  if (!g->d_desc || g->num_nodes >= (1ll << 31) || g->num_edges >= (1ll << 31) - 1) return kNoHostKernel;
  const size_t elem = narrow ? 4 : 8;
  const size_t row_b = (size_t)(L + 1) * elem;
  const size_t need = (size_t)n * row_b + (want_e ? (size_t)n * L * elem : 0);
  if (need > ((size_t)g_tuning.host_resident_mb.load() << 20)) return kNoHostKernel;
  if (g_tuning.n2v_idx.load() == 1) return kNoHostKernel;
  {  // the matrices must fit what the device has left (buffers kept from earlier calls count as free)
    size_t free_b = 0, total_b = 0;
    CUDA_TRY(cudaMemGetInfo(&free_b, &total_b));
    const size_t kept = g->cap_all + g->cap_eall + g->cap_start_all;
    if (need + (size_t)n * 8 + ((size_t)64 << 20) > free_b + kept) return kNoHostKernel;
  }

  // slab: the largest power of two of rows whose copy is at most an eighth of the slab tuning
  // (small slabs keep the staging copy cache-warm for the widening threads and shorten the exposed tail)
  int shift = 10;
  const size_t target = ((size_t)g_tuning.host_slab_mb.load() << 20) / 8 * (narrow ? 1 : 2);
  while (shift < 30 && ((size_t)2 << shift) * row_b <= target) shift++;
  const int64_t slab_rows = (int64_t)1 << shift;
  const int64_t slabs = (n + slab_rows - 1) / slab_rows;

  if (int rc = grow_one(&g->d_start_all, &g->cap_start_all, (size_t)n * 8)) return rc;
  if (int rc = grow_one(&g->d_all, &g->cap_all, (size_t)n * row_b)) return rc;
  if (want_e) if (int rc = grow_one(&g->d_eall, &g->cap_eall, (size_t)n * L * elem)) return rc;
  if (int rc = grow_one(&g->d_slab_done, &g->cap_slab_done, (size_t)slabs * 4)) return rc;
  if ((size_t)slabs * 4 > g->cap_slab_flags) {
    if (g->h_slab_flags) cudaFreeHost(g->h_slab_flags);
    g->h_slab_flags = nullptr;
    g->cap_slab_flags = 0;
    CUDA_TRY(cudaHostAlloc((void**)&g->h_slab_flags, (size_t)slabs * 4, cudaHostAllocMapped));
    g->cap_slab_flags = (size_t)slabs * 4;
  }
  if (narrow) {
    const size_t slab_bytes = (size_t)(slab_rows < n ? slab_rows : n) * row_b;
    if (int rc = grow_pinned(g->h_pack, &g->cap_hpack, slab_bytes)) return rc;
    if (want_e) if (int rc = grow_pinned(g->h_epack, &g->cap_hepack, (size_t)(slab_rows < n ? slab_rows : n) * L * 4)) return rc;
    if (int rc = ensure_pool(g)) return rc;
  }
  uint32_t* d_slab_flags = nullptr;
  CUDA_TRY(cudaHostGetDevicePointer((void**)&d_slab_flags, g->h_slab_flags, 0));

  cudaStream_t work = g->streams[0], copy = g->streams[1];
  // idle after a normal call; after a call that returned early with an error they may not be, and a
  // launch still running must not set flags of this call
  CUDA_TRY(cudaStreamSynchronize(work));
  CUDA_TRY(cudaStreamSynchronize(copy));
  volatile uint32_t* flags = g->h_slab_flags;
  for (int64_t k = 0; k < slabs; k++) flags[k] = 0;
  CUDA_TRY(cudaMemsetAsync(g->d_flags, 0, sizeof(uint32_t), work));
  CUDA_TRY(cudaMemsetAsync(g->d_slab_done, 0, (size_t)slabs * 4, work));
  CUDA_TRY(cudaMemcpyAsync(g->d_start_all, h_start, (size_t)n * 8, cudaMemcpyHostToDevice, work));

  Node2vecParams P{};
  if (int rc = prepare_n2v(&csr, g->d_start_all, n, L, p, q, seed, base, stride, reinterpret_cast<int64_t*>(g->d_all),
                           want_e ? reinterpret_cast<int64_t*>(g->d_eall) : nullptr, g->d_flags, nullptr, &P))
    return rc;
  P.slab_shift = shift;
  P.slab_done = g->d_slab_done;
  P.slab_flags = d_slab_flags;
  {
    const int rc = launch_n2v_host(P, (csr.flags & WALK_B200_CSR_SYMMETRIC) != 0, narrow, work);
    if (rc == kNoHostKernel) {  // nothing was launched; leave the stream idle for the fallback
      CUDA_TRY(cudaStreamSynchronize(work));
      return kNoHostKernel;
    }
    if (rc) return rc;
  }

  auto rows_of = [&](int64_t k) { return (n - k * slab_rows < slab_rows) ? n - k * slab_rows : slab_rows; };
  auto widen = [&](int64_t k) -> int {
    const int lane = (int)(k % kLanes);
    CUDA_TRY(cudaEventSynchronize(g->landed[lane]));
    g->pool->widen(g->h_pack[lane], h_n_out + k * slab_rows * (L + 1), rows_of(k) * (L + 1));
    if (want_e) g->pool->widen(g->h_epack[lane], h_e_out + k * slab_rows * L, rows_of(k) * L);
    return WALK_B200_OK;
  };

  bool kernel_done = false;
  for (int64_t k = 0; k < slabs; k++) {
    // Wait for the slab's flag. The launch is finite (every walk has an attempt cap), so the wait
    // ends at the latest when the work stream has drained; then every slab is complete.
    for (uint32_t spins = 0; !kernel_done && flags[k] == 0; spins++) {
      if ((spins & 63) == 63) {
        const cudaError_t st = cudaStreamQuery(work);
        if (st == cudaSuccess) kernel_done = true;
        else if (st != cudaErrorNotReady) return fail(WALK_B200_ERR_CUDA, "node2vec launch failed: %s", cudaGetErrorString(st));
      }
      std::this_thread::yield();
    }
    if (narrow) {
      const int lane = (int)(k % kLanes);
      // the lane's staging was widened kLanes - 1 slabs ago (the widen below trails by one slab)
      CUDA_TRY(cudaMemcpyAsync(g->h_pack[lane], g->d_all + k * slab_rows * (L + 1), (size_t)rows_of(k) * row_b,
                               cudaMemcpyDeviceToHost, copy));
      if (want_e)
        CUDA_TRY(cudaMemcpyAsync(g->h_epack[lane], g->d_eall + k * slab_rows * L, (size_t)rows_of(k) * L * 4,
                                 cudaMemcpyDeviceToHost, copy));
      CUDA_TRY(cudaEventRecord(g->landed[lane], copy));
      if (k >= 1) if (int rc = widen(k - 1)) return rc;
    } else {
      const int64_t* d_all64 = reinterpret_cast<const int64_t*>(g->d_all);
      CUDA_TRY(cudaMemcpyAsync(h_n_out + k * slab_rows * (L + 1), d_all64 + k * slab_rows * (L + 1),
                               (size_t)rows_of(k) * row_b, cudaMemcpyDeviceToHost, copy));
      if (want_e)
        CUDA_TRY(cudaMemcpyAsync(h_e_out + k * slab_rows * L, reinterpret_cast<const int64_t*>(g->d_eall) + k * slab_rows * L,
                                 (size_t)rows_of(k) * L * 8, cudaMemcpyDeviceToHost, copy));
    }
  }
  if (narrow) if (int rc = widen(slabs - 1)) return rc;
  CUDA_TRY(cudaStreamSynchronize(work));
  CUDA_TRY(cudaStreamSynchronize(copy));
  uint32_t f = 0;
  CUDA_TRY(cudaMemcpy(&f, g->d_flags, sizeof(f), cudaMemcpyDeviceToHost));
  return flags_to_status(f);
}

// Runs one walk over host buffers in slabs: H2D(start[, rand]) -> kernel -> D2H(walks)
// per slab, slabs round-robin over kLanes streams so copies in both directions overlap
// the kernels of neighbouring slabs. When every id fits int32 (and the tuning allows it) the
// slab is packed to int32 on the device, lands in pinned staging owned by the graph and is widened
// into the caller's buffer by host threads while later slabs run: half the bytes on the bus, and
// the caller's output buffers need not be pinned.
int run_host_walk(walk_b200_graph* g, bool biased, const int64_t* h_start, const float* h_rand,
                  int64_t n, int32_t L, double p, double q, uint64_t seed, uint64_t base, uint64_t stride,
                  int64_t* h_n_out, int64_t* h_e_out) {
  if (stride == 0) stride = 1;
  if (!g) return fail(WALK_B200_ERR_INVALID_ARG, "graph handle is NULL");
  if (int rc = check_walk_sizes(n, L, h_start, h_n_out)) return rc;
  if (!biased && n > 0 && L > 0 && !h_rand) return fail(WALK_B200_ERR_INVALID_ARG, "rand is NULL");
  double prob[3];
  uint32_t cuts[3];
  if (biased) if (int rc = thresholds(p, q, prob, cuts)) return rc;
  if (n == 0) return WALK_B200_OK;

  std::lock_guard<std::mutex> lock(g->mu);
  DeviceGuard dg(g->device);
  if (!dg.ok) return fail(WALK_B200_ERR_CUDA, "cannot select device %d", g->device);

  constexpr int kLanes = walk_b200_graph::kLanes;
  const bool want_e = h_e_out && L > 0;
  const bool narrow = use_narrow(g, g->num_nodes < (1ll << 31) && (!want_e || g->num_edges < (1ll << 31)));
  walk_b200_csr csr{};
  csr.rowptr = g->d_rowptr; csr.col = g->d_col; csr.num_nodes = g->num_nodes; csr.num_edges = g->num_edges;
  csr.rowdesc = g->d_desc; csr.flags = g->csr_flags;
  csr.edgeset = g->d_edgeset; csr.edgeset_buckets = g->edgeset_buckets;
  csr.colrev = g->d_colrev;
  csr.colrev16 = g->d_colrev16;
  csr.fused = g->d_fused;

  if (biased && g_tuning.host_single_launch.load() != 0) {
    const int rc = run_host_n2v_single(g, csr, narrow, h_start, n, L, p, q, seed, base, stride, h_n_out, h_e_out);
    if (rc != kNoHostKernel) return rc;
  }

  const size_t row_bytes = (size_t)(L + 1) * 8;
  int64_t slab_rows = (int64_t)(((size_t)g_tuning.host_slab_mb.load() << 20) / row_bytes);
  if (slab_rows < 1024) slab_rows = 1024;
  slab_rows = (slab_rows + 255) / 256 * 256;
  if (slab_rows > n) slab_rows = n;
  if (int rc = grow(g->d_start, &g->cap_start, (size_t)slab_rows * 8)) return rc;
  if (int rc = grow(g->d_out, &g->cap_out, (size_t)slab_rows * row_bytes)) return rc;
  if (!biased && L > 0) if (int rc = grow(g->d_rand, &g->cap_rand, (size_t)slab_rows * L * 4)) return rc;
  if (want_e) if (int rc = grow(g->d_eout, &g->cap_eout, (size_t)slab_rows * L * 8)) return rc;
  if (narrow) {
    if (int rc = grow(g->d_pack, &g->cap_pack, (size_t)slab_rows * row_bytes / 2)) return rc;
    if (int rc = grow_pinned(g->h_pack, &g->cap_hpack, (size_t)slab_rows * row_bytes / 2)) return rc;
    if (want_e) {
      if (int rc = grow(g->d_epack, &g->cap_epack, (size_t)slab_rows * L * 4)) return rc;
      if (int rc = grow_pinned(g->h_epack, &g->cap_hepack, (size_t)slab_rows * L * 4)) return rc;
    }
    if (int rc = ensure_pool(g)) return rc;
  }

  CUDA_TRY(cudaMemsetAsync(g->d_flags, 0, sizeof(uint32_t), g->streams[0]));
  CUDA_TRY(cudaStreamSynchronize(g->streams[0]));

  // widen slab `i` (narrow transport) once its staging copy has landed
  auto finish = [&](int64_t i) -> int {
    const int lane = (int)(i % kLanes);
    const int64_t r0 = i * slab_rows;
    const int64_t rows = (n - r0 < slab_rows) ? n - r0 : slab_rows;
    CUDA_TRY(cudaEventSynchronize(g->landed[lane]));
    g->pool->widen(g->h_pack[lane], h_n_out + r0 * (L + 1), rows * (L + 1));
    if (want_e) g->pool->widen(g->h_epack[lane], h_e_out + r0 * L, rows * L);
    return WALK_B200_OK;
  };

  const int64_t slabs = (n + slab_rows - 1) / slab_rows;
  constexpr int64_t kLag = kLanes - 1;  // slabs queued on the device while the host widens an older one
  for (int64_t i = 0; i < slabs; i++) {
    const int lane = (int)(i % kLanes);
    const int64_t r0 = i * slab_rows;
    const int64_t rows = (n - r0 < slab_rows) ? n - r0 : slab_rows;
    cudaStream_t s = g->streams[lane];
    CUDA_TRY(cudaMemcpyAsync(g->d_start[lane], h_start + r0, (size_t)rows * 8, cudaMemcpyHostToDevice, s));
    int64_t* d_e = want_e ? g->d_eout[lane] : nullptr;
    int rc;
    if (biased) {
      rc = walk_b200_node2vec_walk(&csr, g->d_start[lane], rows, L, p, q, seed, base + (uint64_t)r0 * stride,
                                   stride, g->d_out[lane], d_e, g->d_flags, nullptr, s);
    } else {
      if (L > 0)
        CUDA_TRY(cudaMemcpyAsync(g->d_rand[lane], h_rand + r0 * L, (size_t)rows * L * 4, cudaMemcpyHostToDevice, s));
      rc = walk_b200_uniform_walk(&csr, g->d_start[lane], g->d_rand[lane], rows, L, g->d_out[lane], d_e,
                                  g->d_flags, s);
    }
    if (rc) return rc;
    if (narrow) {
      if (int rc2 = launch_narrow(g->d_out[lane], rows * (L + 1), g->d_pack[lane], s)) return rc2;
      CUDA_TRY(cudaMemcpyAsync(g->h_pack[lane], g->d_pack[lane], (size_t)rows * (L + 1) * 4, cudaMemcpyDeviceToHost, s));
      if (d_e) {
        if (int rc2 = launch_narrow(d_e, rows * L, g->d_epack[lane], s)) return rc2;
        CUDA_TRY(cudaMemcpyAsync(g->h_epack[lane], g->d_epack[lane], (size_t)rows * L * 4, cudaMemcpyDeviceToHost, s));
      }
      CUDA_TRY(cudaEventRecord(g->landed[lane], s));
      if (i >= kLag) if (int rc2 = finish(i - kLag)) return rc2;  // frees the lane slab i + 1 will use
    } else {
      CUDA_TRY(cudaMemcpyAsync(h_n_out + r0 * (L + 1), g->d_out[lane], (size_t)rows * row_bytes, cudaMemcpyDeviceToHost, s));
      if (d_e) CUDA_TRY(cudaMemcpyAsync(h_e_out + r0 * L, d_e, (size_t)rows * L * 8, cudaMemcpyDeviceToHost, s));
    }
  }
  if (narrow)
    for (int64_t i = (slabs > kLag ? slabs - kLag : 0); i < slabs; i++)
      if (int rc2 = finish(i)) return rc2;
  for (int k = 0; k < kLanes; k++) CUDA_TRY(cudaStreamSynchronize(g->streams[k]));
  uint32_t f = 0;
  CUDA_TRY(cudaMemcpy(&f, g->d_flags, sizeof(f), cudaMemcpyDeviceToHost));
  return flags_to_status(f);
}

// Which transport serves this process best is a property of the box and of what else runs on it (the ranks of
// one machine share its host memory): time a pinned device-to-host copy and the widening of as many elements,
// once, at graph creation, when every rank of a job is doing the same. Per byte of int64 output the narrow
// transport costs max(half a byte over the bus, one byte through the widening threads), the wide one a byte
// over the bus.
int measure_transport(walk_b200_graph* g) {
  const size_t elems = (size_t)8 << 20;  // 32 MiB of int32, 64 MiB of int64
  int32_t* h32 = nullptr;
  int64_t* h64 = nullptr;
  int64_t* d64 = nullptr;
  int rc = WALK_B200_OK;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  auto cleanup = [&]() {
    if (h32) cudaFreeHost(h32);
    if (h64) cudaFreeHost(h64);
    if (d64) cudaFree(d64);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
  };
#define M_TRY(expr)                                                                                  \
  do {                                                                                               \
    cudaError_t err__ = (expr);                                                                      \
    if (err__ != cudaSuccess) {                                                                      \
      rc = fail(WALK_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));              \
      cleanup();                                                                                     \
      return rc;                                                                                     \
    }                                                                                                \
  } while (0)
  M_TRY(cudaHostAlloc((void**)&h32, elems * 4, cudaHostAllocDefault));
  M_TRY(cudaHostAlloc((void**)&h64, elems * 8, cudaHostAllocDefault));
  M_TRY(cudaMalloc((void**)&d64, elems * 8));
  M_TRY(cudaEventCreate(&e0));
  M_TRY(cudaEventCreate(&e1));
  cudaStream_t s = g->streams[0];
  M_TRY(cudaMemsetAsync(d64, 0, elems * 8, s));
  M_TRY(cudaMemcpyAsync(h64, d64, elems * 8, cudaMemcpyDeviceToHost, s));  // warm-up, touches the pages
  M_TRY(cudaEventRecord(e0, s));
  const int reps = 4;
  for (int r = 0; r < reps; r++) M_TRY(cudaMemcpyAsync(h64, d64, elems * 8, cudaMemcpyDeviceToHost, s));
  M_TRY(cudaEventRecord(e1, s));
  M_TRY(cudaEventSynchronize(e1));
  float ms = 0.f;
  M_TRY(cudaEventElapsedTime(&ms, e0, e1));
#undef M_TRY
  if ((rc = ensure_pool(g))) { cleanup(); return rc; }
  memset(h32, 1, elems * 4);
  g->pool->widen(h32, h64, (int64_t)elems);
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < reps; r++) g->pool->widen(h32, h64, (int64_t)elems);
  const double wsecs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  cleanup();
  g->measured_d2h_gbs = ms > 0.f ? (double)reps * elems * 8 / (ms * 1e-3) / 1e9 : 0.0;
  g->measured_widen_gbs = wsecs > 0 ? (double)reps * elems * 8 / wsecs / 1e9 : 0.0;
  if (g->measured_d2h_gbs > 0 && g->measured_widen_gbs > 0) {
    const double narrow_cost = std::fmax(0.5 / g->measured_d2h_gbs, 1.0 / g->measured_widen_gbs);
    const double wide_cost = 1.0 / g->measured_d2h_gbs;
    g->prefer_narrow = narrow_cost * 1.1 < wide_cost;
  }
  return WALK_B200_OK;
}

}  // namespace

extern "C" {

int walk_b200_graph_create(const int64_t* h_rowptr, const int64_t* h_col, int64_t num_nodes,
                           int64_t num_edges, uint32_t csr_flags, int32_t validate, walk_b200_graph** out) {
  if (!out) return fail(WALK_B200_ERR_INVALID_ARG, "out is NULL");
  *out = nullptr;
  if (num_nodes < 0 || num_edges < 0 || !h_rowptr || (num_edges > 0 && !h_col))
    return fail(WALK_B200_ERR_INVALID_ARG, "bad graph arguments");
  walk_b200_graph* g = new (std::nothrow) walk_b200_graph();
  if (!g) return fail(WALK_B200_ERR_INVALID_ARG, "out of host memory");
  auto bail = [&](int rc) { std::string keep = g_last_error; walk_b200_graph_destroy(g); g_last_error = keep; return rc; };
#define G_TRY(expr)                                                                                   \
  do {                                                                                                \
    cudaError_t err__ = (expr);                                                                       \
    if (err__ != cudaSuccess)                                                                         \
      return bail(fail(WALK_B200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)));       \
  } while (0)
  G_TRY(cudaGetDevice(&g->device));
  g->num_nodes = num_nodes; g->num_edges = num_edges; g->csr_flags = csr_flags;
  for (int k = 0; k < walk_b200_graph::kLanes; k++) {
    G_TRY(cudaStreamCreateWithFlags(&g->streams[k], cudaStreamNonBlocking));
    G_TRY(cudaEventCreateWithFlags(&g->landed[k], cudaEventDisableTiming));
  }
  G_TRY(cudaMalloc((void**)&g->d_rowptr, (size_t)(num_nodes + 1) * 8));
  G_TRY(cudaMalloc((void**)&g->d_col, (size_t)(num_edges > 0 ? num_edges : 1) * 8));
  G_TRY(cudaMalloc((void**)&g->d_flags, 256));
  cudaStream_t s = g->streams[0];
  G_TRY(cudaMemsetAsync(g->d_flags, 0, 256, s));
  G_TRY(cudaMemcpyAsync(g->d_rowptr, h_rowptr, (size_t)(num_nodes + 1) * 8, cudaMemcpyHostToDevice, s));
  if (num_edges > 0) G_TRY(cudaMemcpyAsync(g->d_col, h_col, (size_t)num_edges * 8, cudaMemcpyHostToDevice, s));
  uint32_t f = 0;
  if (validate) {
    walk_b200_csr csr{};
    csr.rowptr = g->d_rowptr; csr.col = g->d_col; csr.num_nodes = num_nodes; csr.num_edges = num_edges;
    if (int rc = walk_b200_csr_validate(&csr, nullptr, 0, validate == 2 ? 0 : 1, g->d_flags, s)) return bail(rc);
    G_TRY(cudaMemcpyAsync(&f, g->d_flags, 4, cudaMemcpyDeviceToHost, s));
    G_TRY(cudaStreamSynchronize(s));
    if (f) { flags_to_status(f); return bail(fail(WALK_B200_ERR_CSR_INVALID, "graph failed validation: %s", std::string(g_last_error).c_str())); }
  }
  if (g_tuning.use_rowdesc.load() && num_nodes > 0) {
    G_TRY(cudaMalloc((void**)&g->d_desc, (size_t)num_nodes * 8));
    if (int rc = walk_b200_rowdesc_pack(g->d_rowptr, num_nodes, num_edges, g->d_desc, g->d_flags, s)) return bail(rc);
    G_TRY(cudaMemcpyAsync(&f, g->d_flags, 4, cudaMemcpyDeviceToHost, s));
    G_TRY(cudaStreamSynchronize(s));
    if (f & WALK_B200_FLAG_BAD_ROWPTR) { return bail(fail(WALK_B200_ERR_CSR_INVALID, "rowptr is not a monotone prefix array ending at num_edges")); }
    if (f & WALK_B200_FLAG_DESC_OVERFLOW) {  // graph too large for the packed form: walk from rowptr
      cudaFree(g->d_desc);
      g->d_desc = nullptr;
    }
  }
  if ((csr_flags & WALK_B200_CSR_WANT_EDGESET) && num_edges > 0 && num_nodes < 0xffffffffll) {
    walk_b200_csr csr{};
    csr.rowptr = g->d_rowptr; csr.col = g->d_col; csr.num_nodes = num_nodes; csr.num_edges = num_edges;
    if (int rc = walk_b200_edgeset_buckets(num_edges, &g->edgeset_buckets)) return bail(rc);
    {  // a sparser table answers more membership tests from their first bucket; taken when it fits comfortably
      int32_t spe = g_tuning.edgeset_slots_per_edge.load();
      if (spe < 2) spe = 2;
      if (spe > 16) spe = 16;
      size_t free_b = 0, total_b = 0;
      G_TRY(cudaMemGetInfo(&free_b, &total_b));
      const uint64_t want = g->edgeset_buckets * (uint64_t)spe / 2;
      const uint64_t rest = (uint64_t)num_edges * 12;  // reverse positions and their join with col, built next
      // (behind the triangle filter few tests reach the set: the minimum size does as well there)
      const bool filtered = (csr_flags & WALK_B200_CSR_WANT_TRIFILTER) && (csr_flags & WALK_B200_CSR_SYMMETRIC);
      if (!filtered && want * kEdgeSlotsPerBucket * sizeof(uint64_t) + rest < free_b / 2) g->edgeset_buckets = want;
    }
    G_TRY(cudaMalloc((void**)&g->d_edgeset, g->edgeset_buckets * kEdgeSlotsPerBucket * sizeof(uint64_t)));
    if (int rc = walk_b200_edgeset_build(&csr, g->d_edgeset, g->edgeset_buckets, g->d_flags, s)) return bail(rc);
    G_TRY(cudaMemcpyAsync(&f, g->d_flags, 4, cudaMemcpyDeviceToHost, s));
    G_TRY(cudaStreamSynchronize(s));
    if (f) { flags_to_status(f); return bail(fail(WALK_B200_ERR_CSR_INVALID, "edge set build failed: %s", std::string(g_last_error).c_str())); }
    // reverse positions ride on the edge set; rows that are not strictly ascending simply go without
    if (num_edges < 0xfffffffell) {
      uint32_t* d_revpos = nullptr;
      G_TRY(cudaMalloc((void**)&d_revpos, (size_t)num_edges * sizeof(uint32_t)));
      int rc = walk_b200_revpos_build(&csr, d_revpos, g->d_flags, s);
      cudaError_t ce = rc ? cudaSuccess : cudaMemcpyAsync(&f, g->d_flags, 4, cudaMemcpyDeviceToHost, s);
      if (!rc && ce == cudaSuccess) ce = cudaStreamSynchronize(s);
      if (!rc && ce == cudaSuccess && !f) {  // join them with col: the array the kernel gathers from
        csr.revpos = d_revpos;
        ce = cudaMalloc((void**)&g->d_colrev, (size_t)num_edges * sizeof(uint64_t));
        if (ce == cudaSuccess) rc = walk_b200_colrev_build(&csr, g->d_colrev, g->d_flags, s);
        if (!rc && ce == cudaSuccess) ce = cudaStreamSynchronize(s);
      }
      cudaFree(d_revpos);
      if (rc) return bail(rc);
      if (ce != cudaSuccess) return bail(fail(WALK_B200_ERR_CUDA, "reverse-position build failed: %s", cudaGetErrorString(ce)));
      if (f) G_TRY(cudaMemsetAsync(g->d_flags, 0, 4, s));
    }
  }
  if ((csr_flags & WALK_B200_CSR_WANT_TRIFILTER) && (csr_flags & WALK_B200_CSR_SYMMETRIC) && g->d_colrev && g->d_desc) {
    walk_b200_csr csr{};
    csr.rowptr = g->d_rowptr; csr.col = g->d_col; csr.num_nodes = num_nodes; csr.num_edges = num_edges;
    csr.rowdesc = g->d_desc; csr.flags = csr_flags; csr.edgeset = g->d_edgeset; csr.edgeset_buckets = g->edgeset_buckets;
    csr.colrev = g->d_colrev;
    G_TRY(cudaMalloc(&g->d_colrev16, (size_t)num_edges * 16));
    if (int rc = walk_b200_trifilter_build(&csr, g->d_colrev16, g_tuning.trifilter_max_row.load(), g->d_flags, s)) return bail(rc);
    G_TRY(cudaStreamSynchronize(s));
  }
  if ((csr_flags & WALK_B200_CSR_WANT_FUSED) && num_edges > 0 && g->d_desc) {
    walk_b200_csr csr{};
    csr.rowptr = g->d_rowptr; csr.col = g->d_col; csr.num_nodes = num_nodes; csr.num_edges = num_edges;
    csr.rowdesc = g->d_desc;
    G_TRY(cudaMalloc(&g->d_fused, (size_t)num_edges * 16));
    if (int rc = walk_b200_fused_build(&csr, g->d_fused, g->d_flags, s)) return bail(rc);
    G_TRY(cudaMemcpyAsync(&f, g->d_flags, 4, cudaMemcpyDeviceToHost, s));
    G_TRY(cudaStreamSynchronize(s));
    if (f) { flags_to_status(f); return bail(fail(WALK_B200_ERR_CSR_INVALID, "fused record build failed: %s", std::string(g_last_error).c_str())); }
  }
  G_TRY(cudaStreamSynchronize(s));
#undef G_TRY
  if (g_tuning.host_narrow.load() == 2 && num_nodes < (1ll << 31)) {
    if (int rc = measure_transport(g)) return bail(rc);
  }
  *out = g;
  return WALK_B200_OK;
}

int walk_b200_graph_host_transport(const walk_b200_graph* g, int32_t* narrow, double* d2h_gbs, double* widen_gbs) {
  if (!g) return fail(WALK_B200_ERR_INVALID_ARG, "graph is NULL");
  if (narrow) *narrow = use_narrow(g, g->num_nodes < (1ll << 31)) ? 1 : 0;
  if (d2h_gbs) *d2h_gbs = g->measured_d2h_gbs;
  if (widen_gbs) *widen_gbs = g->measured_widen_gbs;
  return WALK_B200_OK;
}

int walk_b200_host_widen_probe(size_t out_bytes, double* out_gbs) {
  if (!out_gbs || out_bytes < (1u << 20)) return fail(WALK_B200_ERR_INVALID_ARG, "widen probe needs at least 1 MiB and a result");
  *out_gbs = 0.0;
  int threads = g_tuning.host_threads.load();
  if (threads <= 0) {
    threads = (int)std::thread::hardware_concurrency();
    if (threads > 16) threads = 16;
    if (threads < 1) threads = 1;
  }
  const int64_t count = (int64_t)(out_bytes / 8);
  std::unique_ptr<int32_t[]> src(new (std::nothrow) int32_t[count]);
  std::unique_ptr<int64_t[]> dst(new (std::nothrow) int64_t[count]);
  if (!src || !dst) return fail(WALK_B200_ERR_INVALID_ARG, "out of host memory");
  memset(src.get(), 1, (size_t)count * 4);
  WidenPool pool(threads - 1);
  pool.widen(src.get(), dst.get(), count);  // touches the pages
  const auto t0 = std::chrono::steady_clock::now();
  const int reps = 3;
  for (int r = 0; r < reps; r++) pool.widen(src.get(), dst.get(), count);
  const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  if (secs > 0) *out_gbs = (double)reps * (double)count * 8.0 / secs / 1e9;
  return WALK_B200_OK;
}

int walk_b200_graph_destroy(walk_b200_graph* g) {
  if (!g) return WALK_B200_OK;
  {
    DeviceGuard dg(g->device);
    for (int k = 0; k < walk_b200_graph::kLanes; k++) {
      if (g->streams[k]) { cudaStreamSynchronize(g->streams[k]); cudaStreamDestroy(g->streams[k]); }
      if (g->d_start[k]) cudaFree(g->d_start[k]);
      if (g->d_rand[k]) cudaFree(g->d_rand[k]);
      if (g->d_out[k]) cudaFree(g->d_out[k]);
      if (g->d_eout[k]) cudaFree(g->d_eout[k]);
      if (g->d_pack[k]) cudaFree(g->d_pack[k]);
      if (g->d_epack[k]) cudaFree(g->d_epack[k]);
      if (g->h_pack[k]) cudaFreeHost(g->h_pack[k]);
      if (g->h_epack[k]) cudaFreeHost(g->h_epack[k]);
      if (g->landed[k]) cudaEventDestroy(g->landed[k]);
    }
    if (g->d_rowptr) cudaFree(g->d_rowptr);
    if (g->d_col) cudaFree(g->d_col);
    if (g->d_desc) cudaFree(g->d_desc);
    if (g->d_edgeset) cudaFree(g->d_edgeset);
    if (g->d_colrev) cudaFree(g->d_colrev);
    if (g->d_colrev16) cudaFree(g->d_colrev16);
    if (g->d_fused) cudaFree(g->d_fused);
    if (g->d_flags) cudaFree(g->d_flags);
    if (g->d_start_all) cudaFree(g->d_start_all);
    if (g->d_all) cudaFree(g->d_all);
    if (g->d_eall) cudaFree(g->d_eall);
    if (g->d_slab_done) cudaFree(g->d_slab_done);
    if (g->h_slab_flags) cudaFreeHost(g->h_slab_flags);
  }
  delete g;
  return WALK_B200_OK;
}

int walk_b200_graph_csr(const walk_b200_graph* g, walk_b200_csr* out) {
  if (!g || !out) return fail(WALK_B200_ERR_INVALID_ARG, "graph or out is NULL");
  memset(out, 0, sizeof(*out));
  out->rowptr = g->d_rowptr; out->col = g->d_col; out->num_nodes = g->num_nodes; out->num_edges = g->num_edges;
  out->rowdesc = g->d_desc; out->flags = g->csr_flags;
  out->edgeset = g->d_edgeset; out->edgeset_buckets = g->edgeset_buckets;
  out->colrev = g->d_colrev;
  out->colrev16 = g->d_colrev16;
  out->fused = g->d_fused;
  return WALK_B200_OK;
}

int walk_b200_graph_device_bytes(const walk_b200_graph* g, int64_t* bytes) {
  if (!g || !bytes) return fail(WALK_B200_ERR_INVALID_ARG, "graph or bytes is NULL");
  *bytes = (g->num_nodes + 1) * 8 + g->num_edges * 8 + (g->d_desc ? g->num_nodes * 8 : 0) +
           (int64_t)(g->d_edgeset ? g->edgeset_buckets * kEdgeSlotsPerBucket * 8 : 0) +
           (g->d_colrev ? g->num_edges * 8 : 0) + (g->d_colrev16 ? g->num_edges * 16 : 0) +
           (g->d_fused ? g->num_edges * 16 : 0);
  return WALK_B200_OK;
}

int walk_b200_uniform_walk_host(walk_b200_graph* g, const int64_t* h_start, const float* h_rand,
                                int64_t num_walks, int32_t walk_length, int64_t* h_n_out, int64_t* h_e_out) {
  return run_host_walk(g, false, h_start, h_rand, num_walks, walk_length, 1.0, 1.0, 0, 0, 1, h_n_out, h_e_out);
}

int walk_b200_node2vec_walk_host(walk_b200_graph* g, const int64_t* h_start, int64_t num_walks,
                                 int32_t walk_length, double p, double q, uint64_t seed,
                                 uint64_t walk_index_base, uint64_t walk_index_stride, int64_t* h_n_out,
                                 int64_t* h_e_out) {
  return run_host_walk(g, true, h_start, nullptr, num_walks, walk_length, p, q, seed, walk_index_base,
                       walk_index_stride, h_n_out, h_e_out);
}

}  // extern "C"
