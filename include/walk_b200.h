/*
 * walk_b200.h -- C ABI of the B200 (sm_100a) CSR walk generators.
 *
 * This is the boundary a host framework binds in place of the reference's two
 * primitives. Plain pointers and sizes only; no exceptions cross it; every entry
 * point returns a WALK_B200_* status (0 = success) and leaves a message behind for
 * walk_b200_last_error(). There is no CPU implementation behind any of these
 * calls: without a CUDA device they fail with WALK_B200_ERR_CUDA.
 *
 * Conventions
 *   - "device pointer" = memory of the CUDA device that is current on the calling
 *     thread. All launches are asynchronous on `stream` (a cudaStream_t passed as
 *     void*, NULL = the legacy default stream); outputs are valid in stream order.
 *   - CSR arrays are int64, as in the reference: rowptr[num_nodes+1], col[num_edges].
 *   - Walk matrix n_out is int64 [num_walks, walk_length+1], row-major; the optional
 *     edge matrix e_out is int64 [num_walks, walk_length] (-1 where the walk stood still).
 *   - A node without out-edges keeps the walk in place for all remaining steps.
 *   - status_flags (optional device uint32) is OR-ed with WALK_B200_FLAG_* bits when
 *     a kernel meets malformed input; the kernel never faults on it: it parks the
 *     walk or clamps the index and carries on.
 */
#ifndef WALK_B200_H_
#define WALK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WALK_B200_ABI_VERSION 9

/* ---- return codes ---- */
#define WALK_B200_OK 0
#define WALK_B200_ERR_INVALID_ARG 1 /* null pointer, negative size, size overflow */
#define WALK_B200_ERR_BAD_PQ 2      /* p or q not finite, not > 0, or prob_2 = (1/q)/max(1/p, 1, 1/q) below 2^-16 */
#define WALK_B200_ERR_CUDA 3        /* a CUDA runtime call failed (message has the CUDA error) */
#define WALK_B200_ERR_CSR_INVALID 4 /* walk_b200_csr_validate / host entry points found a malformed graph */
#define WALK_B200_ERR_UNSUPPORTED 5 /* e.g. row descriptor cannot represent this graph */
#define WALK_B200_ERR_DEVICE_FLAGS 6 /* host entry point: the kernel raised status flags (see message) */

/* ---- device status flag bits ---- */
#define WALK_B200_FLAG_BAD_NODE 0x1u      /* a start or col value outside [0, num_nodes) */
#define WALK_B200_FLAG_BAD_EDGE 0x2u      /* a sampled edge index outside [0, num_edges) (rand >= 1, NaN, bad rowptr) */
#define WALK_B200_FLAG_ATTEMPT_CAP 0x4u   /* node2vec: WALK_B200_MAX_ATTEMPTS rejections in one step */
#define WALK_B200_FLAG_BAD_ROWPTR 0x8u    /* rowptr not monotone, or rowptr[0] != 0, or rowptr[N] != num_edges */
#define WALK_B200_FLAG_DESC_OVERFLOW 0x10u /* a row start >= 2^36 or a degree >= 2^28: no packed descriptor */
#define WALK_B200_FLAG_UNSORTED_ROW 0x20u /* csr_validate: a row is not strictly ascending */
#define WALK_B200_FLAG_WAIT_TIMEOUT 0x40u /* reserved */
#define WALK_B200_FLAG_EDGESET_FULL 0x80u /* edge hash set too small for the graph (build) or a probe chain ran away (lookup) */

#define WALK_B200_MAX_ATTEMPTS (1u << 22)

/* ---- graph description ---- */
#define WALK_B200_CSR_SYMMETRIC 0x1u /* caller asserts (u,v) in E <=> (v,u) in E: lets node2vec search the previous
                                        node's row instead of the candidate's; results are identical on such graphs */

#define WALK_B200_CSR_WANT_EDGESET 0x2u /* walk_b200_graph_create only: also build the edge hash set and, when rows are
                                           strictly ascending, col joined with the reverse positions */

#define WALK_B200_CSR_WANT_FUSED 0x4u /* walk_b200_graph_create only: also build the fused edge records */

#define WALK_B200_CSR_WANT_TRIFILTER 0x8u /* walk_b200_graph_create only, with _SYMMETRIC and _WANT_EDGESET: also build the
                                             triangle filter (walk_b200_trifilter_build; tuning trifilter_max_row) */

typedef struct walk_b200_csr {
  const int64_t* rowptr;   /* device, [num_nodes + 1] */
  const int64_t* col;      /* device, [num_edges]; node2vec needs each row sorted ascending */
  int64_t num_nodes;
  int64_t num_edges;
  const uint64_t* rowdesc; /* device, [num_nodes], from walk_b200_rowdesc_pack, or NULL (kernels then read rowptr) */
  uint32_t flags;          /* WALK_B200_CSR_* */
  uint32_t reserved;
  const uint64_t* edgeset; /* device, [4 * edgeset_buckets], from walk_b200_edgeset_build, or NULL: node2vec then
                              runs its membership test as a binary search over col */
  uint64_t edgeset_buckets;
  const uint32_t* revpos;  /* device, [num_edges], from walk_b200_revpos_build, or NULL: input of
                              walk_b200_colrev_build, not read by the walks */
  const void* fused;       /* device, [num_edges] 16-byte records from walk_b200_fused_build, or NULL; the uniform
                              walk then makes one gather per step; needs rowdesc */
  const uint64_t* colrev;  /* device, [num_edges], from walk_b200_colrev_build, or NULL; only used together with
                              edgeset and rowdesc */
  const void* colrev16;    /* device, [num_edges] 16-byte records from walk_b200_trifilter_build, or NULL; only used
                              together with colrev, edgeset and rowdesc on a graph flagged WALK_B200_CSR_SYMMETRIC */
} walk_b200_csr;

/* node2vec instrumentation slots (device uint64[WALK_B200_COUNTER_COUNT], caller zeroes them) */
enum {
  WALK_B200_CNT_LOADS = 0,      /* 8-byte gathers issued (rowptr/rowdesc/col), all states */
  WALK_B200_CNT_ATTEMPTS,       /* candidate draws in the rejection loop (steps >= 1, degree >= 2) */
  WALK_B200_CNT_MEMBERSHIP,     /* membership tests actually run */
  WALK_B200_CNT_PROBES,         /* binary-search probes (or hash buckets read) of those tests */
  WALK_B200_CNT_STEPS_DEG0,
  WALK_B200_CNT_STEPS_DEG1,
  WALK_B200_CNT_STEPS_SAMPLED,
  WALK_B200_CNT_STEPS_FIRST,
  WALK_B200_CNT_FORMULA_PROBES, /* sum over membership tests of ceil(log2(deg(candidate) + 1)): what a binary search
                                   of the candidate's row, the reference's is_neighbor(x, t) done in log time, would probe */
  WALK_B200_CNT_GATHERS16,      /* triangle-filter kernel only: 16-byte candidate gathers (each also counted as 2 loads) */
  WALK_B200_CNT_FILTERED,       /* triangle-filter kernel only: attempts the filter rejected without a gather */
  WALK_B200_COUNTER_COUNT
};

/* ---- library ---- */
int walk_b200_abi_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char* walk_b200_last_error(void);
/* Number of kernels this library has launched in this process (all threads). */
uint64_t walk_b200_launch_count(void);
/* Name of the kernel the calling thread launched last through this library ("" before the first launch),
 * e.g. "node2vec_pool_kernel": lets a host check which variant a call selected. */
const char* walk_b200_last_kernel(void);

/*
 * Uniform CSR walk. Replaces RandomWalk::eval_cpu (random_walks/RandomWalk.cpp:18-62),
 * the Metal kernel (random_walks/random_walk.metal:5-35) and its host launch
 * RandomWalk::eval_gpu (random_walks/RandomWalk.cpp:73-108). Step l of walk w takes
 * col[rowptr[v] + (int64)(rand[w*L+l] * (float)deg(v))], float32 product truncated
 * toward zero, bit-for-bit as the reference. e_out and status_flags may be NULL.
 */
int walk_b200_uniform_walk(const walk_b200_csr* g, const int64_t* start, const float* rand,
                           int64_t num_walks, int32_t walk_length, int64_t* n_out,
                           int64_t* e_out, uint32_t* status_flags, void* stream);

/*
 * The same uniform walk with its draws generated in the kernel instead of read from a caller's
 * rand array (the reference always takes rand_data from the caller, tests/test_random_walk.py:31;
 * this variant removes that [n, L] float32 input, 4 bytes per step of reads and, on the largest
 * workloads, an array bigger than the GPU). Draw of step l of global walk w (= walk_index_base +
 * row * walk_index_stride): Philox4x32-10, key = seed, counter = (w lo32, l >> 2, 0x554E4946, w hi32),
 * word (l & 3), r = (word >> 8) * 2^-24. walk_b200_uniform_draws fills the matching rand array on
 * the host, so the result equals walk_b200_uniform_walk on that array bit for bit.
 */
int walk_b200_uniform_walk_philox(const walk_b200_csr* g, const int64_t* start, int64_t num_walks,
                                  int32_t walk_length, uint64_t seed, uint64_t walk_index_base,
                                  uint64_t walk_index_stride, int64_t* n_out, int64_t* e_out,
                                  uint32_t* status_flags, void* stream);
void walk_b200_uniform_draw(uint64_t seed, uint64_t walk, uint32_t step, float* r);
void walk_b200_uniform_draws(uint64_t seed, uint64_t walk_index_base, uint64_t walk_index_stride,
                             int64_t num_walks, int32_t walk_length, float* out);

/*
 * node2vec biased walk by rejection sampling. Replaces BiasedRandomWalk::eval_cpu
 * (random_walks/BiasedRandomWalk.cpp:30-102, is_neighbor :20-28); the reference has
 * no GPU version (eval_gpu throws, :150-155). Draws come from Philox4x32-10 with
 * key = seed and counter = (walk lo32, step, attempt, walk hi32), walk =
 * walk_index_base + row * walk_index_stride (stride 0 is read as 1; a rank that holds every
 * G-th start row passes base = its rank, stride = G): word0>>1 picks the candidate (mod degree), word1>>1 is the
 * accept draw r = w / 2147483647 compared against prob_0/1/2 of the reference
 * (:52-55). Same accept/reject decisions as the reference loop fed with that stream.
 * counters (device uint64[WALK_B200_COUNTER_COUNT]) selects the instrumented kernel
 * when non-NULL. e_out, status_flags, counters may be NULL. walk_length 0 returns
 * the start column only (the reference requires walk_length >= 1).
 */
int walk_b200_node2vec_walk(const walk_b200_csr* g, const int64_t* start, int64_t num_walks,
                            int32_t walk_length, double p, double q, uint64_t seed,
                            uint64_t walk_index_base, uint64_t walk_index_stride, int64_t* n_out,
                            int64_t* e_out, uint32_t* status_flags, uint64_t* counters, void* stream);

/*
 * Pack rowptr into one 8-byte descriptor per node: bits 0..35 = rowptr[v],
 * bits 36..63 = degree. One 8-byte load then replaces the rowptr pair read of
 * random_walks/RandomWalk.cpp:45-46 / BiasedRandomWalk.cpp:71. rowdesc is caller
 * scratch of num_nodes * 8 bytes. Raises WALK_B200_FLAG_DESC_OVERFLOW / _BAD_ROWPTR
 * in status_flags when the graph does not fit (then pass rowdesc = NULL to the walks).
 */
int walk_b200_rowdesc_pack(const int64_t* rowptr, int64_t num_nodes, int64_t num_edges,
                           uint64_t* rowdesc, uint32_t* status_flags, void* stream);

/*
 * Edge hash set: an exact set of all directed edges, so that node2vec's membership test
 * "is t a neighbour of x" (is_neighbor, random_walks/BiasedRandomWalk.cpp:20-28, a linear
 * scan there) costs about one 32-byte read instead of a binary search over col.
 * walk_b200_edgeset_buckets gives the smallest table size for a graph (16 bytes per edge: load
 * factor 0.5); any larger bucket count works too, and a sparser table answers more tests from
 * their first bucket (measured on R-MAT 24 at p=0.25, q=4: 1.22 buckets read per test half full,
 * 1.02 a quarter full, 4.5 % off the launch); table is caller scratch of 32 * buckets bytes, 32-byte aligned. Needs
 * num_nodes < 2^32 - 1 (else WALK_B200_ERR_UNSUPPORTED). Works for any CSR, directed or
 * not, sorted or not. Put the pointer and bucket count into walk_b200_csr.
 */
int walk_b200_edgeset_buckets(int64_t num_edges, uint64_t* buckets);
int walk_b200_edgeset_build(const walk_b200_csr* g, uint64_t* table, uint64_t buckets,
                            uint32_t* status_flags, void* stream);

/*
 * Fused edge records for the uniform walk: fused[e] = (col[e], row descriptor of col[e]), 16 bytes per
 * edge (caller scratch of 16 * num_edges bytes, 16-byte aligned; g->rowdesc must be set). The step
 * "col[rowptr[v] + idx] then rowptr pair of the new node" (random_walks/RandomWalk.cpp:45-54) becomes
 * one 16-byte gather, i.e. one DRAM access instead of two on graphs whose row bounds do not stay in L2.
 * Results are identical with and without it.
 */
int walk_b200_fused_build(const walk_b200_csr* g, void* fused, uint32_t* status_flags, void* stream);

/*
 * Reverse positions: revpos[e] for the edge e = (u -> v) is the index in col of (v -> u), or
 * 0xffffffff if the graph has no such edge. With it (and the edge hash set and row descriptors) a
 * node2vec step knows without a gather whether a drawn edge leads back to the previous node --
 * the "x == t" test of random_walks/BiasedRandomWalk.cpp:86 -- and skips the col gather of every
 * attempt that only the return rule could accept (three in four at p=0.25, q=4). revpos is caller
 * scratch of 4 * num_edges bytes. Needs every row strictly ascending (else
 * WALK_B200_FLAG_UNSORTED_ROW is raised and the array must not be used) and num_edges < 2^32 - 2.
 * Results are identical with and without it.
 */
int walk_b200_revpos_build(const walk_b200_csr* g, uint32_t* revpos, uint32_t* status_flags, void* stream);

/*
 * colrev[e] = col[e] | revpos[e] << 32 (g->revpos must be set; num_nodes < 2^32 - 1; caller scratch
 * of 8 * num_edges bytes). This is the array the node2vec kernel reads when it uses reverse
 * positions: the gather of a candidate also brings the position of the edge back from it, so a step
 * needs no separate look-up of the reverse position. revpos itself may be freed afterwards.
 */
int walk_b200_colrev_build(const walk_b200_csr* g, uint64_t* colrev, uint32_t* status_flags, void* stream);

/*
 * Triangle filter for node2vec on an undirected graph: colrev16[e] = {colrev[e], filter word of e} (caller scratch
 * of 16 * num_edges bytes, 16-byte aligned; g needs colrev, edgeset and WALK_B200_CSR_SYMMETRIC). The membership
 * test "is the previous node t a neighbour of the candidate x" (is_neighbor, random_walks/BiasedRandomWalk.cpp:20-28,
 * called at :88) can only say yes when x is a common neighbour of t and the node v the walk stands on. Bit k of the
 * word of edge (t -> v) is set iff such a common neighbour sits at a position p of v's row with p mod 64 == k, so a
 * walk that arrived by that edge knows from the position it drew alone, before gathering the candidate, that an
 * attempt which only the membership rule could accept fails. With it a launch at p=0.25, q=4 gathers about half as
 * much. Building it costs one edge-set look-up per entry of the shorter row of every undirected edge (seconds on a
 * graph of 5e8 edges; worth it for a graph that is walked many times); edges whose shorter row exceeds max_row
 * (0 = no limit) keep an all-ones word, i.e. go unfiltered. Results are identical with and without it.
 */
int walk_b200_trifilter_build(const walk_b200_csr* g, void* colrev16, int64_t max_row, uint32_t* status_flags,
                              void* stream);

/*
 * Full check the reference never makes (it reinterprets whatever it is given,
 * random_walks/RandomWalk.cpp:33-38): rowptr[0]==0, monotone, rowptr[N]==num_edges,
 * 0 <= col < N, 0 <= start < N, and (check_sorted != 0) rows strictly ascending.
 * Findings are OR-ed into status_flags (required, device). start may be NULL.
 */
int walk_b200_csr_validate(const walk_b200_csr* g, const int64_t* start, int64_t num_walks,
                           int32_t check_sorted, uint32_t* status_flags, void* stream);

/*
 * Host-side Philox4x32-10 block and the walk stream built on it, so a caller can
 * reproduce every draw of walk_b200_node2vec_walk without a GPU.
 */
void walk_b200_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]);
void walk_b200_node2vec_draw(uint64_t seed, uint64_t walk, uint32_t step, uint32_t attempt,
                             uint32_t* candidate31, uint32_t* accept31);
/* thresholds prob_0/1/2 (BiasedRandomWalk.cpp:52-55) and their exact integer cuts:
 * "r < prob_k" <=> "accept31 < cuts[k]". Returns WALK_B200_ERR_BAD_PQ on bad p/q. */
int walk_b200_node2vec_thresholds(double p, double q, double prob[3], uint32_t cuts[3]);

/* Contiguous block partition of num_walks start rows over world_size ranks. */
int walk_b200_shard_range(int64_t num_walks, int32_t world_size, int32_t rank,
                          int64_t* begin, int64_t* end);
/* Cyclic partition: rank r holds rows r, r + world_size, ...; returns how many that is. Balances
 * ranks on graphs whose node ids are correlated with degree (block shards of an R-MAT graph differ
 * by 25 % in work). */
int walk_b200_shard_count_cyclic(int64_t num_walks, int32_t world_size, int32_t rank, int64_t* count);

/* ---- edge list -> CSR on the device ----------------------------------------------
 * The step in front of the walks. The reference's demos sort the edge index on the
 * host and derive rowptr from the counts of the row ids that occur, which loses
 * isolated nodes (tests/test_random_walk.py:22-28 of the reference project); here
 * num_nodes is an argument and rowptr always has num_nodes + 1 entries.
 * src/dst: int64 [num_input_edges] device arrays. Output: rowptr int64 [num_nodes + 1],
 * col int64 with room for num_input_edges entries (twice that with
 * WALK_B200_BUILD_SYMMETRIZE); rows come out sorted ascending; the number of edges
 * written is rowptr[num_nodes] (read it from the device after the stream has caught
 * up). Edges with an endpoint outside [0, num_nodes) are left out and raise
 * WALK_B200_FLAG_BAD_NODE. Needs num_nodes < 2^31 and num_input_edges < 2^31.
 * scratch: device memory, 256-byte aligned, walk_b200_csr_build_scratch_bytes() bytes,
 * free again when the stream has passed the call. Nothing is read back to the host.
 */
#define WALK_B200_BUILD_SYMMETRIZE 0x1u      /* also insert every edge reversed */
#define WALK_B200_BUILD_DROP_SELF_LOOPS 0x2u /* leave out u -> u */
#define WALK_B200_BUILD_DEDUPE 0x4u          /* keep one copy of a repeated edge */

int walk_b200_csr_build_scratch_bytes(int64_t num_input_edges, int64_t num_nodes, uint32_t options,
                                      uint64_t* bytes);
int walk_b200_csr_build(const int64_t* src, const int64_t* dst, int64_t num_input_edges,
                        int64_t num_nodes, uint32_t options, void* scratch, uint64_t scratch_bytes,
                        int64_t* rowptr, int64_t* col, uint32_t* status_flags, void* stream);

/* ---- resident graph + host-buffer entry points ---------------------------------
 * For callers whose arrays live in host memory. The graph is uploaded once and stays
 * resident on the device that was current at creation; each walk call then moves
 * only its own batch: start (+ rand) host->device and the walk matrix device->host,
 * in slabs so that copies overlap the kernel. start and rand should be pinned
 * (cudaHostAlloc / cudaHostRegister) for the uploads to overlap.
 * When every id fits 31 bits the matrices can cross the bus as int32 into pinned staging
 * owned by the graph, host threads of the library widening them into the caller's
 * int64 buffers (which may then be pageable): half the bytes on the bus, twice the
 * traffic in host memory. Which of the two transports is faster depends on the machine
 * and on how many processes share its host memory, so by default (host_narrow = 2) a
 * short measurement at graph creation decides. node2vec runs as one launch whose
 * finished slabs are copied out while it goes on, and keeps the matrices in
 * device memory for the duration of the call. Results are identical either way. A
 * call returns when the caller's buffers are written; on a non-zero return their
 * contents are unspecified.
 */
typedef struct walk_b200_graph walk_b200_graph;

/* validate: 0 = trust the arrays; 1 = run walk_b200_csr_validate with the sorted-rows check on the uploaded graph
 * and fail with WALK_B200_ERR_CSR_INVALID on any finding (what node2vec without the edge hash set needs: its
 * membership test is then a binary search); 2 = the same without the sorted-rows check. */
int walk_b200_graph_create(const int64_t* h_rowptr, const int64_t* h_col, int64_t num_nodes,
                           int64_t num_edges, uint32_t csr_flags, int32_t validate,
                           walk_b200_graph** out);
int walk_b200_graph_destroy(walk_b200_graph* g);
/* Device view of a resident graph (pointers owned by the graph). */
int walk_b200_graph_csr(const walk_b200_graph* g, walk_b200_csr* out);
int walk_b200_graph_device_bytes(const walk_b200_graph* g, int64_t* bytes);

/* Transport the host entry points use for this graph's walk matrices (1 = int32 on the bus plus widening threads,
 * 0 = int64 straight into the caller's buffers) under the current host_narrow tuning, and the two rates measured
 * when the graph was created (GB/s; 0 if host_narrow was not 2 then): pinned device-to-host copy, and int64
 * output of the widening threads. Any result pointer may be NULL. */
int walk_b200_graph_host_transport(const walk_b200_graph* g, int32_t* narrow, double* d2h_gbs, double* widen_gbs);
/* Output rate (GB/s of int64 written) of the widening threads on `out_bytes` of int64, with the current
 * host_threads tuning: the host-side ceiling of the int32 transport on this machine right now. */
int walk_b200_host_widen_probe(size_t out_bytes, double* out_gbs);

int walk_b200_uniform_walk_host(walk_b200_graph* g, const int64_t* h_start, const float* h_rand,
                                int64_t num_walks, int32_t walk_length, int64_t* h_n_out,
                                int64_t* h_e_out);
int walk_b200_node2vec_walk_host(walk_b200_graph* g, const int64_t* h_start, int64_t num_walks,
                                 int32_t walk_length, double p, double q, uint64_t seed,
                                 uint64_t walk_index_base, uint64_t walk_index_stride, int64_t* h_n_out,
                                 int64_t* h_e_out);

/* ---- L2 residency hint ----------------------------------------------------------
 * Marks [ptr, ptr+bytes) (typically rowdesc or rowptr: the array whose accesses are
 * skewed to hub nodes) as persisting in L2 for work launched on `stream` afterwards.
 * Per-context, per-stream state only; walk_b200_l2_window_clear undoes it, carve-out included.
 * Measured on B200 with these kernels: the carve-out takes L2 away from the col gathers and made
 * every workload slower (uniform scale 22: 5.9 -> 11.8 ms); the kernels' own per-load eviction
 * policies do the job instead. Kept for hosts that want to experiment; off unless called.
 * granted_bytes (optional) receives the window actually set (0 if the device or
 * driver configuration offers none).
 */
int walk_b200_l2_window_set(const void* ptr, size_t bytes, float hit_ratio, void* stream,
                            size_t* granted_bytes);
int walk_b200_l2_window_clear(void* stream);

/* ---- entry point that allocates nothing ----------------------------------------
 * No counterpart in the reference (its primitives always allocate their outputs and
 * know nothing of scratch memory).
 *
 * Same walk, same results as walk_b200_uniform_walk with a packed row descriptor, for
 * callers that must not allocate device memory at call time: code that runs where a
 * cudaMalloc would stall the device it shares with latency-critical work (cudaMalloc
 * synchronises the whole device), hosts whose own memory pool already owns all of the
 * GPU so that a driver allocation may simply fail, and plug-in layers that are only
 * handed raw pointers and have no allocator to ask. Such a caller still passes the
 * CSR, the inputs and the outputs; the one piece of scratch the fast path needs -- the
 * 8-byte row descriptor per node -- lives in a fixed array inside the library's own
 * device image (WALK_B200_NOALLOC_MAX_NODES entries = 8 MiB, resident on every GPU
 * that loads the library until the process exits). The call packs rowptr into that
 * array and then walks, both on `stream`; it calls no cudaMalloc / cudaFree / pool
 * routine. Graphs with more than WALK_B200_NOALLOC_MAX_NODES nodes (or more than 2^36
 * edges) are rejected with WALK_B200_ERR_UNSUPPORTED.
 *
 * The first call on each device looks up the array's device address (a one-off
 * set-up that may make the driver load this library's device code), so make that
 * first call outside of any stream capture. All calls on a device share the one
 * array and it keeps the previous call's descriptors: every call rewrites the
 * entries it reads before reading them, so nothing has to be cleared, but two calls
 * whose work overlaps on the GPU (different streams, no ordering between them) race
 * on it -- order them. e_out and status_flags may be NULL.
 */
#define WALK_B200_NOALLOC_MAX_NODES (1 << 20)
int walk_b200_uniform_walk_noalloc(const int64_t* rowptr, const int64_t* col, int64_t num_nodes,
                                   int64_t num_edges, const int64_t* start, const float* rand,
                                   int64_t num_walks, int32_t walk_length, int64_t* n_out,
                                   int64_t* e_out, uint32_t* status_flags, void* stream);

/*
 * Consumer of the walk matrix, the step that follows the walks in a node2vec pipeline (no counterpart
 * in the reference, whose README lists further algorithms as future work, README.md:65-69): all runs of
 * context_size consecutive nodes of every walk, windows[(w * nwin + j) * cs + k] = walks[w, j + k] with
 * nwin = walk_length + 2 - context_size; column 0 is the centre node, the rest its skip-gram context.
 * windows is int64 [num_walks * nwin, context_size], device, caller-allocated; like walks it only needs the
 * 8-byte alignment of its element type (a view that starts at an odd element of a larger buffer is fine).
 */
int walk_b200_context_windows(const int64_t* walks, int64_t num_walks, int32_t walk_length,
                              int32_t context_size, int64_t* windows, void* stream);

/*
 * Negative samples of the skip-gram loss, shaped like walks so that walk_b200_context_windows applies
 * to them unchanged (no counterpart in the reference): out[r, 0] = start[r], out[r, 1 + k] = a node id
 * drawn uniformly from [0, num_nodes), k < walk_length. out is int64 [num_rows, walk_length + 1], device.
 * Draw k of global row g = row_index_base + r * row_index_stride (stride 0 means 1) is word (k & 3) of
 * Philox4x32-10 with key = seed and counter = (g low 32, k >> 2, 0x4E454753, g high 32);
 * node = (word * num_nodes) >> 32. Needs 1 <= num_nodes <= 2^32. walk_b200_negative_draw replays one
 * draw on the host.
 */
int walk_b200_negative_walks(const int64_t* start, int64_t num_rows, int32_t walk_length,
                             int64_t num_nodes, uint64_t seed, uint64_t row_index_base,
                             uint64_t row_index_stride, int64_t* out, void* stream);
int walk_b200_negative_draw(uint64_t seed, uint64_t row, uint32_t k, int64_t num_nodes, int64_t* node);

/*
 * Device probe (diagnostic; allocates and frees array_bytes of device memory itself):
 * the rate of dependent random 8-byte gathers over an array much larger than L2, one
 * gather in flight per thread -- the access pattern of a walk step. On B200 this rate,
 * not the byte bandwidth, bounds the walks: about 5e10 DRAM-missing gathers per second
 * whether a miss moves 64 or 128 bytes. No counterpart in the reference.
 */
int walk_b200_gather_probe(size_t array_bytes, int32_t iters, double* gathers_per_second);
/* The same probe with its shape exposed, to tell a limit of the memory system from a limit of the
 * probe: `chains` (1, 2 or 4) independent chains per thread, i.e. that many gathers in flight per
 * thread; `gather_bytes` (8, 16 or 32) per gather; `fetch_bytes` 64 (the L2 fetches half a line per
 * miss, as the walks ask for) or 128 (the part's default, a whole line); `threads_per_sm` 0 for 2^22
 * threads in several full waves, else one wave of that many resident threads per SM (a multiple of 256
 * up to 2048). The plain probe above is (1, 8, 64, 0). */
int walk_b200_gather_probe_ex(size_t array_bytes, int32_t iters, int32_t chains, int32_t gather_bytes,
                              int32_t fetch_bytes, int32_t threads_per_sm, double* gathers_per_second);

/* Kernel variant and transport selection; unknown keys fail. None of them changes a result (but see n2v_max_attempts).
 *   uniform_variant, uniform_fused, l2_hints, l2_fetch_granularity, use_rowdesc
 *   n2v_idx, n2v_member, n2v_rev, n2v_pool (0 per-lane kernel, 1 pooled kernel where it wins, 2 always),
 *   n2v_batch_lanes, n2v_batch_trips, n2v_draw_loop, n2v_blocks_per_sm, n2v_tri (0: ignore a graph's triangle filter),
 *   edgeset_slots_per_edge (size of the edge hash set a resident graph builds for itself, in 8-byte slots per
 *   edge: 2 = half full, the minimum; default 4, taken when the table fits half of the free device memory),
 *   n2v_max_attempts (rejections after which a step gives up, at most WALK_B200_MAX_ATTEMPTS: the one key that
 *   can change a result, and only for steps that reach the cap, which raise WALK_B200_FLAG_ATTEMPT_CAP)
 *   host_slab_mb, host_narrow (1 int32 on the bus, 0 int64, 2 measured at graph creation), host_threads (widening threads, 0 = min(16, cores)),
 *   host_single_launch (node2vec host entry as one launch), host_resident_mb (its device-memory limit) */
int walk_b200_set_tuning(const char* key, int32_t value);
int walk_b200_get_tuning(const char* key, int32_t* value);

#ifdef __cplusplus
}
#endif
#endif /* WALK_B200_H_ */
