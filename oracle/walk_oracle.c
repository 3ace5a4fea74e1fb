/*
 * CPU restatement of the reference's two walk generators. TEST INFRASTRUCTURE ONLY:
 * this file is the checker for the CUDA path (tests, the smoke check and the
 * bench's cpu_baseline leg may call it); no product code path may route through it.
 *
 * Parity status: PINNED. tests/test_oracle.py checks
 *   - oracle_uniform_walk bit-for-bit against the reference's own
 *     RandomWalk::eval_cpu (compiled unmodified into oracle/_ref) and against the
 *     golden fixtures that build produced;
 *   - oracle_node2vec_walk in draw mode 0 (libc rand(), same call order as the
 *     reference) bit-for-bit against the reference's BiasedRandomWalk::eval_cpu
 *     after the same srand(); draw mode 1 replaces only the source of the two
 *     draws per attempt with a Philox4x32-10 counter stream.
 *
 * Reference lines followed (paths inside the reference project):
 *   random_walks/RandomWalk.cpp:41-60           uniform walk loop
 *   random_walks/BiasedRandomWalk.cpp:20-28     is_neighbor (linear scan)
 *   random_walks/BiasedRandomWalk.cpp:52-55     thresholds prob_0 / prob_1 / prob_2
 *   random_walks/BiasedRandomWalk.cpp:57-99     biased walk loop
 * Philox4x32-10 is the published counter-based generator of Salmon et al.
 * (SC'11), restated here from its definition.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_RAND_MAX 2147483647 /* glibc RAND_MAX, the divisor at BiasedRandomWalk.cpp:84 */

/* ---- Philox4x32-10 -------------------------------------------------------- */

static inline void philox_round(uint32_t c[4], const uint32_t k[2]) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0];
  const uint32_t n1 = (uint32_t)p1;
  const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1];
  const uint32_t n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
  uint32_t k[2] = {key[0], key[1]};
  for (int r = 0; r < 10; r++) {
    if (r) { k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u; }
    philox_round(c, k);
  }
  memcpy(out, c, sizeof(c));
}

/* The walk stream: key = seed, counter = (walk lo, step, attempt, walk hi).
 * Word 0 >> 1 is the candidate draw, word 1 >> 1 the accept draw; both are 31-bit,
 * the range of glibc rand(). */
static inline void walk_draw(uint64_t seed, uint64_t walk, uint32_t step, uint32_t attempt,
                             uint32_t* cand, uint32_t* acc) {
  uint32_t ctr[4] = {(uint32_t)walk, step, attempt, (uint32_t)(walk >> 32)};
  uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  uint32_t o[4];
  oracle_philox4x32_10(ctr, key, o);
  *cand = o[0] >> 1;
  *acc = o[1] >> 1;
}

/* ---- uniform walk: random_walks/RandomWalk.cpp:41-60 ---------------------- */

void oracle_uniform_walk(const int64_t* rowptr, const int64_t* col, const int64_t* start,
                         const float* rnd, int64_t n, int walk_length,
                         int64_t* n_out, int64_t* e_out /* may be NULL */) {
  const int64_t L = walk_length;
  for (int64_t w = 0; w < n; w++) {
    int64_t cur = start[w];
    n_out[w * (L + 1)] = cur;
    for (int64_t l = 0; l < L; l++) {
      const int64_t rs = rowptr[cur], re = rowptr[cur + 1];
      int64_t e;
      if (re - rs == 0) {
        e = -1; /* stay in place */
      } else {
        const float r = rnd[w * L + l];
        /* int64 degree -> float32, float32 product, truncation toward zero */
        const float prod = r * (float)(re - rs);
        e = rs + (int64_t)prod;
        cur = col[e];
      }
      n_out[w * (L + 1) + l + 1] = cur;
      if (e_out) e_out[w * L + l] = e;
    }
  }
}

/* ---- node2vec biased walk ------------------------------------------------- */

void oracle_node2vec_thresholds(double p, double q, double out[3]) {
  /* random_walks/BiasedRandomWalk.cpp:52-55 */
  const double max_prob = fmax(fmax(1. / p, 1.), 1. / q);
  out[0] = 1. / p / max_prob;
  out[1] = 1. / max_prob;
  out[2] = 1. / q / max_prob;
}

/* Smallest 31-bit draw w with (double)w / RAND_MAX >= prob, i.e. "r < prob" <=> "w < cut".
 * Returns 2^31 when every draw is below prob. Independent of the product's copy. */
uint32_t oracle_accept_cut(double prob) {
  uint64_t lo = 0, hi = (uint64_t)ORACLE_RAND_MAX + 1; /* first w with r(w) >= prob in [lo, hi] */
  while (lo < hi) {
    const uint64_t mid = lo + (hi - lo) / 2;
    const double r = (double)mid / (double)ORACLE_RAND_MAX;
    if (r >= prob) hi = mid; else lo = mid + 1;
  }
  return (uint32_t)lo;
}

static inline int linear_is_neighbor(const int64_t* rowptr, const int64_t* col, int64_t v, int64_t w,
                                     int64_t* scanned) {
  /* random_walks/BiasedRandomWalk.cpp:20-28 */
  const int64_t rs = rowptr[v], re = rowptr[v + 1];
  for (int64_t i = rs; i < re; i++) {
    (*scanned)++;
    if (col[i] == w) return 1;
  }
  return 0;
}

static inline int ceil_log2_u64(uint64_t x) { /* ceil(log2(x)) for x >= 1 */
  int b = 0;
  while (((uint64_t)1 << b) < x) b++;
  return b;
}

enum {
  CNT_ATTEMPTS = 0,      /* candidate draws inside the rejection loop (steps l >= 1, deg >= 2) */
  CNT_MEMBERSHIP_REF,    /* is_neighbor calls the reference makes */
  CNT_MEMBERSHIP_NEEDED, /* attempts whose outcome depends on the membership test */
  CNT_SCAN_ELEMS,        /* elements the reference's linear scans touch */
  CNT_BSEARCH_PROBES,    /* sum over needed tests of ceil(log2(deg(x)+1)) */
  CNT_STEPS_DEG0,
  CNT_STEPS_DEG1,
  CNT_STEPS_SAMPLED,     /* steps l >= 1 with deg >= 2 */
  CNT_STEPS_FIRST,       /* step 0 with deg >= 1 */
  CNT_STEPS_CAPPED,      /* steps given up after max_attempts rejections (never with max_attempts = 0) */
  CNT_COUNT
};

int oracle_counter_count(void) { return CNT_COUNT; }

/*
 * draw_mode 0: libc rand() in the reference's call order (caller seeds with srand()).
 * draw_mode 1: Philox stream above with global walk index walk_index_base + row * walk_index_stride.
 * counters: CNT_COUNT int64 slots, may be NULL.
 * max_attempts: 0 = the reference's unbounded while(true) (random_walks/BiasedRandomWalk.cpp:80). A positive
 * value restates the one deviation of the CUDA path: a step whose first max_attempts candidates are all
 * rejected stands still (x = v, edge id -1), where the reference would keep drawing.
 */
void oracle_node2vec_walk(const int64_t* rowptr, const int64_t* col, const int64_t* start,
                          int64_t n, int walk_length, double p, double q,
                          int draw_mode, uint64_t seed, uint64_t walk_index_base,
                          uint64_t walk_index_stride, int64_t* n_out, int64_t* e_out /* may be NULL */,
                          int64_t* counters /* may be NULL */, uint32_t max_attempts) {
  const int64_t L = walk_length;
  double prob[3];
  oracle_node2vec_thresholds(p, q, prob);
  const double prob_0 = prob[0], prob_1 = prob[1], prob_2 = prob[2];
  int64_t cnt[CNT_COUNT];
  memset(cnt, 0, sizeof(cnt));

  for (int64_t w = 0; w < n; w++) {
    const uint64_t gw = walk_index_base + (uint64_t)w * (walk_index_stride ? walk_index_stride : 1);
    int64_t t = start[w], v, x = 0, e;
    n_out[w * (L + 1)] = t;
    if (L < 1) continue; /* the reference writes column 1 unconditionally; L >= 1 is its precondition */
    int64_t rs = rowptr[t], re = rowptr[t + 1];
    if (re - rs == 0) {
      e = -1;
      v = t;
      cnt[CNT_STEPS_DEG0]++;
    } else {
      uint32_t u, unused;
      if (draw_mode == 0) u = (uint32_t)rand();
      else walk_draw(seed, gw, 0u, 0u, &u, &unused);
      e = rs + (int64_t)(u % (uint64_t)(re - rs));
      v = col[e];
      cnt[CNT_STEPS_FIRST]++;
    }
    n_out[w * (L + 1) + 1] = v;
    if (e_out) e_out[w * L] = e;
    for (int64_t l = 1; l < L; l++) {
      rs = rowptr[v]; re = rowptr[v + 1];
      if (re - rs == 0) {
        e = -1;
        x = v;
        cnt[CNT_STEPS_DEG0]++;
      } else if (re - rs == 1) {
        e = rs;
        x = col[e];
        cnt[CNT_STEPS_DEG1]++;
      } else {
        cnt[CNT_STEPS_SAMPLED]++;
        for (uint32_t a = 0;; a++) {
          uint32_t u, wdraw;
          if (draw_mode == 0) { u = (uint32_t)rand(); }
          else walk_draw(seed, gw, (uint32_t)l, a, &u, &wdraw);
          e = rs + (int64_t)(u % (uint64_t)(re - rs));
          x = col[e];
          if (draw_mode == 0) wdraw = (uint32_t)rand();
          const double r = (double)wdraw / (double)ORACLE_RAND_MAX;
          cnt[CNT_ATTEMPTS]++;
          /* lazy-evaluation bookkeeping (does not alter the decision) */
          const int pre_accept = (r < prob_2) || (x == t && r < prob_0);
          if (!pre_accept && r < prob_1) {
            cnt[CNT_MEMBERSHIP_NEEDED]++;
            cnt[CNT_BSEARCH_PROBES] += ceil_log2_u64((uint64_t)(rowptr[x + 1] - rowptr[x]) + 1);
          }
          if (x == t && r < prob_0) break;
          cnt[CNT_MEMBERSHIP_REF]++;
          if (linear_is_neighbor(rowptr, col, x, t, &cnt[CNT_SCAN_ELEMS]) && r < prob_1) break;
          if (r < prob_2) break;
          if (max_attempts && a + 1 >= max_attempts) { /* not in the reference: give up, stand still */
            x = v;
            e = -1;
            cnt[CNT_STEPS_CAPPED]++;
            break;
          }
        }
      }
      n_out[w * (L + 1) + l + 1] = x;
      if (e_out) e_out[w * L + l] = e;
      t = v;
      v = x;
    }
  }
  if (counters) memcpy(counters, cnt, sizeof(cnt));
}
