/*
 * mac_oracle.c -- CPU restatement of the reference's MAC decode path.
 *
 * TEST INFRASTRUCTURE.  This file is the checker for the CUDA path: only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark may
 * build, load or call it.  The product library never links or falls back to it.
 *
 * Parity pin: the decision logic has no CPU implementation in the reference
 * (it exists only as CUDA), so this restatement is pinned three ways:
 *  (1) against golden vectors produced by importing the reference's own
 *      PyTorch FP32 helpers (_ref_attention/_merge,
 *      attention/tools/check_mac_persistent_decode.py:9-51) on the recipes of
 *      the reference's kernel tests (tests/golden/, generator committed there);
 *  (2) against the reference's Python mirror of its synthetic-decision hash
 *      (benchmark/bench_mac_vs_flashinfer_direct.py:79-211), also as golden
 *      vectors;
 *  (3) on a GPU box, against the reference CUDA kernel itself, compiled for
 *      sm_100a from its own source file by oracle/build_ref.py.
 *
 * All buffers here are HOST pointers; the argument structs are the ones of
 * include/mac_b200.h so a test can fill one struct and hand it to both sides.
 * Paths below are relative to the reference project; DEC.cu =
 * attention/src/mac_attention/integrations/sglang/csrc/mac_decode_persistent.cu,
 * PRE.cu = .../csrc/mac_prefill_update_cache.cu.
 */
#define _GNU_SOURCE
#include <math.h>
#include <limits.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "../include/mac_b200.h"

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------- host threading -- */
/* Plain pthreads work queue (no OpenMP runtime in this image): items are
 * handed out one at a time through an atomic counter. */
typedef void (*item_fn)(void* ctx, int item);
typedef struct ParallelJob {
  item_fn fn;
  void* ctx;
  int n;
  atomic_int next;
} ParallelJob;

static void* parallel_worker(void* arg) {
  ParallelJob* job = (ParallelJob*)arg;
  for (;;) {
    int i = atomic_fetch_add(&job->next, 1);
    if (i >= job->n) break;
    job->fn(job->ctx, i);
  }
  return NULL;
}

static int oracle_threads(void) {
  const char* e = getenv("MAC_ORACLE_THREADS");
  int t = e ? atoi(e) : (int)sysconf(_SC_NPROCESSORS_ONLN);
  if (t < 1) t = 1;
  if (t > 256) t = 256;
  return t;
}

static void parallel_for(int n, item_fn fn, void* ctx) {
  int t = oracle_threads();
  if (t > n) t = n;
  ParallelJob job;
  job.fn = fn;
  job.ctx = ctx;
  job.n = n;
  atomic_init(&job.next, 0);
  if (t <= 1) {
    parallel_worker(&job);
    return;
  }
  pthread_t th[256];
  int started = 0;
  for (int i = 0; i < t - 1; ++i)
    if (pthread_create(&th[started], NULL, parallel_worker, &job) == 0) started++;
  parallel_worker(&job);
  for (int i = 0; i < started; ++i) pthread_join(th[i], NULL);
}

/* Threads the last call could use (reported next to CPU timings). */
ORACLE_API int mac_oracle_num_threads(void) { return oracle_threads(); }

/* ------------------------------------------------------------------ bf16 -- */
static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = ((uint32_t)v) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
/* round-to-nearest-even, NaN kept quiet: what __float2bfloat16_rn does */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* ------------------------------------------------------ ring positions -- */
/* DEC.cu:798-807 */
static inline int ring_slot_to_pos(int past_len, int M, int slot) {
  if (past_len < M) return slot;
  int base = past_len - M;
  int tail = past_len % M;
  int order = slot - tail;
  if (order < 0) order += M;
  return base + order;
}
/* DEC.cu:837-848 */
static inline int pos_to_ring_slot(int past_len, int M, int pos) {
  if (past_len < M) return pos;
  int base = past_len - M;
  int tail = past_len % M;
  int slot = (pos - base) + tail;
  if (slot >= M) slot -= M;
  if (slot < 0) slot += M;
  return slot;
}
/* DEC.cu:713-716 */
static inline int cache_end_for_pos(int p, int S) {
  int e = p + 1 - S;
  return e > 0 ? e : 0;
}
/* DEC.cu:809-811 */
static inline int better_pair(float d, int pos, float bd, int bp) {
  return (d < bd) || (d == bd && pos < bp);
}
/* DEC.cu:221-230 */
static inline int request_ready(const MacB200DecodeArgs* a, int req) {
  if (a->cache_ready == NULL) return 1;
  if (req < 0) return 0;
  if (a->cache_ready[req] == 0) return 0;
  if (a->cache_epoch != NULL && a->request_epoch != NULL &&
      a->cache_epoch[req] != a->request_epoch[req])
    return 0;
  return 1;
}

/* --------------------------------------------------- synthetic decisions -- */
/* DEC.cu:817-835 */
static inline uint32_t mix_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
static inline float uniform01_u32(uint32_t x) {
  return (float)(mix_u32(x) & 0x00ffffffu) * (1.0f / 16777216.0f);
}
static inline float pseudo_normal_u32(uint32_t x) {
  float s = uniform01_u32(x);
  s = s + uniform01_u32(x ^ 0x9e3779b9u);
  s = s + uniform01_u32(x ^ 0x85ebca6bu);
  s = s + uniform01_u32(x ^ 0xc2b2ae35u);
  return (s - 2.0f) * 1.7320508075688772f;
}
static inline float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }
/* DEC.cu:375-388.  The device compiler contracts a*b+c into one fused
 * multiply-add, so the rounding point is written out with fmaf here. */
static int bench_target_miss_units(const MacB200DecodeArgs* a, int unit_total) {
  if (unit_total <= 0) return 0;
  float miss_rate = 1.0f - a->bench_hit_rate;
  miss_rate = clampf(miss_rate, 0.0f, 1.0f);
  int miss_units;
  if (a->bench_exact_quota != 0 && a->bench_hit_rate_std == 0.0f)
    miss_units = (int)floorf(fmaf(miss_rate, (float)unit_total, 0.5f));
  else
    miss_units = (int)ceilf(miss_rate * (float)unit_total);
  if (miss_units < 0) miss_units = 0;
  if (miss_units > unit_total) miss_units = unit_total;
  return miss_units;
}

static inline float threshold_distance(const MacB200DecodeArgs* a) {
  /* DEC.cu:5342, evaluated in float, left to right */
  float t = 2.0f * (float)a->D;
  t = t * (1.0f - a->threshold);
  t = t * (1.0f - a->threshold);
  return t;
}

/* ------------------------------------------------------------ match scan -- */
/* Squared L2 distance in the exact operation order of DEC.cu:1062-1069 with
 * the 16-lane xor butterfly of DEC.cu:343-349: lane t owns dims [8t,8t+8),
 * sums them with sequential fmaf from 0, then the lanes are combined
 * pairwise at distance 8, 4, 2, 1. */
static float ring_distance(const uint16_t* q, const uint16_t* c) {
  float lane[16];
  for (int t = 0; t < 16; ++t) {
    float acc = 0.0f;
    for (int i = 0; i < 8; ++i) {
      float diff = bf16_to_f32(q[t * 8 + i]) - bf16_to_f32(c[t * 8 + i]);
      acc = fmaf(diff, diff, acc);
    }
    lane[t] = acc;
  }
  for (int off = 8; off > 0; off >>= 1) {
    float nxt[16];
    for (int t = 0; t < 16; ++t) nxt[t] = lane[t] + lane[t ^ off];
    memcpy(lane, nxt, sizeof(lane));
  }
  return lane[0];
}

typedef struct HeadDecision {
  int hit, mslot, mpos, prefix_end, rect_start, new_end;
} HeadDecision;

static int request_bad(const MacB200DecodeArgs* a, int n) {
  int req = a->req_ids[n];
  int P = a->past_lens[n];
  if (req < 0 || req >= a->R || req >= a->req_to_token_rows) return 1;
  if (P < 0 || P > a->req_to_token_stride) return 1;
  return 0;
}

/* Per-head decision: DEC.cu:942-1099 (scan), 1142-1302 (hit test, synthetic
 * override, front-sink demotion). */
static void decide_head(const MacB200DecodeArgs* a, int n, int hq, HeadDecision* out) {
  const uint16_t* q_pre = (const uint16_t*)a->q_pre;
  const uint16_t* qc = (const uint16_t*)a->query_cache;
  const int M = a->M, Hq = a->Hq, D = a->D, Tm = a->max_match_tiles;
  const int P = a->past_lens[n];
  const int req = a->req_ids[n];
  int cand_begin = P - M > 0 ? P - M : 0;
  int cand_end = P;
  if (a->candidate_mode == 1) {
    cand_end = P - a->lookback_right;
    if (cand_end < cand_begin) cand_end = cand_begin;
  }
  int eligible = P >= a->gen_min_limit && cand_end > cand_begin && request_ready(a, req);

  float best_d = INFINITY;
  int best_p = INT_MAX, best_s = -1;
  for (int tile = 0; tile < Tm; ++tile) {
    float td = INFINITY;
    int tp = INT_MAX, ts = -1;
    int s0 = tile * a->match_tile_slots;
    int s1 = s0 + a->match_tile_slots;
    if (s1 > M) s1 = M;
    for (int slot = s0; slot < s1 && eligible; ++slot) {
      int pos = ring_slot_to_pos(P, M, slot);
      if (pos < cand_begin || pos >= cand_end) continue;
      const uint16_t* c = qc + (((int64_t)req * M + slot) * Hq + hq) * D;
      float d = ring_distance(q_pre + ((int64_t)n * Hq + hq) * D, c);
      if (better_pair(d, pos, td, tp)) {
        td = d;
        tp = pos;
        ts = slot;
      }
    }
    int64_t off = ((int64_t)n * Hq + hq) * Tm + tile;
    if (a->match_dist) a->match_dist[off] = td;
    if (a->match_pos) a->match_pos[off] = tp;
    if (a->match_slot) a->match_slot[off] = ts;
    if (better_pair(td, tp, best_d, best_p)) {
      best_d = td;
      best_p = tp;
      best_s = ts;
    }
  }
  int hit = eligible && best_s >= 0 && best_d < threshold_distance(a);

  const int S = a->semantic_pos_ahead;
  if (a->bench_mode != 0 || a->bench_miss_mask >= 0) {
    /* DEC.cu:1184-1269 */
    int G = a->Hq / a->Hkv;
    int hkv = hq / G;
    int lane_i = hq - hkv * G;
    uint32_t unit_id = (a->bench_mode == 2) ? (uint32_t)hkv : (uint32_t)hq;
    uint32_t base_key = (uint32_t)a->bench_seed ^ ((uint32_t)a->bench_layer_id * 0x9e3779b9u) ^
                        ((uint32_t)P * 0x85ebca6bu);
    uint32_t key = base_key ^ ((uint32_t)n * 0xc2b2ae35u) ^ (unit_id * 0x27d4eb2fu);
    float hit_rate = clampf(
        fmaf(a->bench_hit_rate_std, pseudo_normal_u32(key ^ 0x4cf5ad43u), a->bench_hit_rate),
        0.0f, 1.0f);
    if (a->bench_miss_mask >= 0) {
      int miss = lane_i >= 0 && lane_i < 30 && (((a->bench_miss_mask >> lane_i) & 1) != 0);
      hit = eligible && P > 0 && M > 0 && !miss;
    } else if (a->bench_exact_quota != 0 && a->bench_hit_rate_std == 0.0f) {
      int unit_total = (a->bench_mode == 2) ? a->N * a->Hkv : a->N * a->Hq;
      int unit = (a->bench_mode == 2) ? n * a->Hkv + hkv : n * a->Hq + hq;
      int miss_units = bench_target_miss_units(a, unit_total);
      int offset = unit_total > 0 ? (int)(base_key % (uint32_t)unit_total) : 0;
      int rotated = unit + offset;
      if (rotated >= unit_total) rotated -= unit_total;
      hit = eligible && P > 0 && M > 0 && !(rotated < miss_units);
    } else {
      hit = eligible && P > 0 && M > 0 && uniform01_u32(key ^ 0x165667b1u) < hit_rate;
    }
    if (hit) {
      int max_lag = M < P ? M : P;
      int new_end_tmp = cache_end_for_pos(P, S);
      float lag_f = fmaf(a->bench_match_lag_std, pseudo_normal_u32(key ^ 0xd3a2646cu),
                         a->bench_match_lag_mean);
      int requested_skip = 0;
      if (a->bench_skip_ratio >= 0.0f) {
        requested_skip = 1;
        float skip = clampf(fmaf(a->bench_skip_ratio_std, pseudo_normal_u32(key ^ 0xfd7046c5u),
                                 a->bench_skip_ratio),
                            0.0f, 0.999999f);
        int target = (int)roundf(skip * (float)P);
        if (target > new_end_tmp - 1) target = new_end_tmp - 1;
        if (target < 0) target = 0;
        lag_f = (float)(new_end_tmp - target);
      }
      int lag = (int)roundf(lag_f);
      if (lag < 1) lag = 1;
      if (requested_skip) {
        if (lag > P) lag = P;
      } else if (lag > max_lag) {
        lag = max_lag;
      }
      if (max_lag <= 0 || new_end_tmp <= 0) {
        hit = 0;
        best_p = INT_MAX;
        best_s = -1;
      } else {
        best_p = P - lag;
        if (best_p < 0) best_p = 0;
        best_s = pos_to_ring_slot(P, M, best_p);
        /* benchmark extension: a synthetic match older than the ring's span stands in a
         * slot of its own (position mod M) instead of an out-of-range one */
        if (a->bench_long_band != 0 && best_p < P - M) best_s = best_p % M;
        best_d = 0.0f;
      }
    } else {
      best_p = INT_MAX;
      best_s = -1;
      best_d = INFINITY;
    }
  }

  int prefix_end = 0, rect_start = 0, mpos = -1, mslot = -1;
  if (hit) {
    mpos = best_p;
    mslot = best_s;
    prefix_end = cache_end_for_pos(mpos, S);
    rect_start = prefix_end;
  }
  int F = a->front_sink_tokens > 0 ? a->front_sink_tokens : 0;
  if (hit && F > 0 && prefix_end < F) { /* DEC.cu:1285-1291 */
    hit = 0;
    mpos = -1;
    mslot = -1;
    prefix_end = 0;
    rect_start = 0;
  }
  out->hit = hit;
  out->mslot = mslot;
  out->mpos = mpos;
  out->prefix_end = prefix_end;
  out->rect_start = rect_start;
  out->new_end = cache_end_for_pos(P, S);
}

/* ------------------------------------------------------------- attention -- */
typedef struct State {
  double o[128];
  double lse; /* natural log; -inf = empty */
} State;

static void state_empty(State* s) {
  memset(s->o, 0, sizeof(s->o));
  s->lse = -INFINITY;
}

static inline int64_t physical_token(const MacB200DecodeArgs* a, int n, int req, int pos, int P) {
  /* DEC.cu:850-864 */
  if (pos == P) {
    return a->out_cache_loc_is_i64 ? (int64_t)((const int64_t*)a->out_cache_loc)[n]
                                   : (int64_t)((const int32_t*)a->out_cache_loc)[n];
  }
  return a->req_to_token[(int64_t)req * a->req_to_token_stride + pos];
}

/* Softmax attention of query head hq over logical positions [t0,t1):
 * normalised o and natural-log LSE (tools/check_mac_persistent_decode.py:9-29,
 * with the accumulation kept in double). */
static void attend_range(const MacB200DecodeArgs* a, int n, int hq, int t0, int t1, State* st) {
  state_empty(st);
  if (t1 <= t0) return;
  const uint16_t* q = (const uint16_t*)a->q_post + ((int64_t)n * a->Hq + hq) * a->D;
  const uint16_t* K = (const uint16_t*)a->k_buffer;
  const uint16_t* V = (const uint16_t*)a->v_buffer;
  const int G = a->Hq / a->Hkv, hkv = hq / G, D = a->D;
  const int req = a->req_ids[n], P = a->past_lens[n];
  float qf[128];
  for (int d = 0; d < D; ++d) qf[d] = bf16_to_f32(q[d]);
  int len = t1 - t0;
  double* logit = (double*)malloc(sizeof(double) * (size_t)len);
  double mx = -INFINITY;
  for (int i = 0; i < len; ++i) {
    int64_t tok = physical_token(a, n, req, t0 + i, P);
    const uint16_t* kr = K + (tok * a->Hkv + hkv) * D;
    double acc = 0.0;
    for (int d = 0; d < D; ++d) acc += (double)qf[d] * (double)bf16_to_f32(kr[d]);
    logit[i] = acc * (double)a->sm_scale;
    if (logit[i] > mx) mx = logit[i];
  }
  double denom = 0.0;
  double o[128];
  memset(o, 0, sizeof(o));
  for (int i = 0; i < len; ++i) {
    double p = exp(logit[i] - mx);
    denom += p;
    int64_t tok = physical_token(a, n, req, t0 + i, P);
    const uint16_t* vr = V + (tok * a->Hkv + hkv) * D;
    for (int d = 0; d < D; ++d) o[d] += p * (double)bf16_to_f32(vr[d]);
  }
  free(logit);
  for (int d = 0; d < D; ++d) st->o[d] = o[d] / denom;
  st->lse = mx + log(denom);
}

/* LSE merge: tools/check_mac_persistent_decode.py:31-51, DEC.cu:866-890 */
static void state_merge(State* s, const State* t) {
  if (!isfinite(t->lse)) return;
  if (!isfinite(s->lse)) {
    *s = *t;
    return;
  }
  double m = s->lse > t->lse ? s->lse : t->lse;
  double ws = exp(s->lse - m), wt = exp(t->lse - m);
  double den = ws + wt;
  for (int d = 0; d < 128; ++d) s->o[d] = (ws * s->o[d] + wt * t->o[d]) / den;
  s->lse = m + log(den);
}

typedef struct StepCtx {
  const MacB200DecodeArgs* a;
  HeadDecision* hd;
  int* bad;
  State* prefix;
  float* out_f32;
  float* ring_o_f32;
} StepCtx;

static void decide_item(void* ctx, int idx) {
  StepCtx* c = (StepCtx*)ctx;
  int n = idx / c->a->Hq, hq = idx % c->a->Hq;
  if (c->bad[n]) return;
  decide_head(c->a, n, hq, &c->hd[idx]);
}

/* attention + merge + ring write + output of one (row, head):
 * DEC.cu:4346-4365 (prefix state), 4485-4497 (ring write before the sink
 * merge), 4500-4520 (sink, output only), 4640-4672 (tail, output). */
static void attend_item(void* ctx, int idx) {
  StepCtx* c = (StepCtx*)ctx;
  const MacB200DecodeArgs* a = c->a;
  HeadDecision* hd = c->hd;
  int* bad = c->bad;
  State* prefix = c->prefix;
  float* out_f32 = c->out_f32;
  float* ring_o_f32 = c->ring_o_f32;
  const int Hq = a->Hq, D = a->D, M = a->M;
  const int F = a->front_sink_tokens > 0 ? a->front_sink_tokens : 0;
  uint16_t* out = (uint16_t*)a->out;
  uint16_t* qcache = (uint16_t*)a->query_cache;
  uint16_t* acache = (uint16_t*)a->attn_cache;
  const uint16_t* q_pre = (const uint16_t*)a->q_pre;
    int n = idx / Hq, hq = idx % Hq;
    int64_t ho = idx;
    if (bad[n]) {
      for (int d = 0; d < D; ++d) {
        out[ho * D + d] = 0;
        if (out_f32) out_f32[ho * D + d] = 0.0f;
        if (ring_o_f32) ring_o_f32[ho * D + d] = 0.0f;
      }
      if (a->optional_lse) a->optional_lse[ho] = -INFINITY;
      return;
    }
    const int req = a->req_ids[n], P = a->past_lens[n];
    HeadDecision* h = &hd[idx];
    const int new_end = h->new_end;
    int band_lo = h->rect_start;
    int sink_hi = F < new_end ? F : new_end; /* head_front_sink_end, DEC.cu:725-731 */
    if (sink_hi > band_lo) sink_hi = band_lo;
    if (sink_hi < 0) sink_hi = 0;

    State st = prefix[idx], part;
    attend_range(a, n, hq, band_lo, new_end, &part);
    state_merge(&st, &part);
    /* ring write (only rows of ready requests) */
    if (request_ready(a, req)) {
      int dest = P % M;
      int64_t base = (((int64_t)req * M + dest) * Hq + hq) * D;
      int ok = isfinite(st.lse);
      for (int d = 0; d < D; ++d) {
        qcache[base + d] = q_pre[ho * D + d];
        acache[base + d] = ok ? f32_to_bf16((float)st.o[d]) : 0;
      }
      a->lse_cache[((int64_t)req * M + dest) * Hq + hq] = ok ? (float)st.lse : -INFINITY;
    }
    if (ring_o_f32)
      for (int d = 0; d < D; ++d) ring_o_f32[ho * D + d] = isfinite(st.lse) ? (float)st.o[d] : 0.0f;
    attend_range(a, n, hq, 0, sink_hi, &part);
    state_merge(&st, &part);
    attend_range(a, n, hq, new_end, P + 1, &part);
    state_merge(&st, &part);
    int ok = isfinite(st.lse);
    for (int d = 0; d < D; ++d) {
      out[ho * D + d] = ok ? f32_to_bf16((float)st.o[d]) : 0;
      if (out_f32) out_f32[ho * D + d] = ok ? (float)st.o[d] : 0.0f;
    }
    if (a->optional_lse) a->optional_lse[ho] = ok ? (float)st.lse : -INFINITY;
}

/* --------------------------------------------------------- decode step -- */
/*
 * One full MAC decode step on the CPU.  Writes everything the CUDA entry
 * point writes (out, optional_lse, ring row P % M of ready requests, decision
 * arrays, task_counts[5], [6]).  out_f32 / ring_o_f32 (optional, [N,Hq,D])
 * receive the un-rounded output and ring state for tolerance checks.
 * Returns the number of rows skipped as malformed (those rows get zeros).
 */
/*
 * row_mask (optional, [N] bytes): rows whose byte is 0 are left out of the step
 * entirely (no decisions, no attention, zero outputs, not counted anywhere)
 * while N and the row indices of the other rows stay what they are -- the
 * synthetic-decision hash depends on both.  Lets a test check a sample of a
 * large batch without holding every request's K/V on the host.
 */
ORACLE_API int mac_oracle_decode_step_rows(const MacB200DecodeArgs* a, float* out_f32,
                                           float* ring_o_f32, const uint8_t* row_mask) {
  const int N = a->N, Hq = a->Hq, Hkv = a->Hkv, D = a->D, M = a->M;
  if (D != 128 || Hkv <= 0 || Hq % Hkv != 0) return -1;
  const int G = Hq / Hkv;
  const int S = a->semantic_pos_ahead;
  const int F = a->front_sink_tokens > 0 ? a->front_sink_tokens : 0;
  int bad_rows = 0;
  HeadDecision* hd = (HeadDecision*)calloc((size_t)N * Hq, sizeof(HeadDecision));
  int* gmode = (int*)calloc((size_t)N * Hkv, sizeof(int));
  int* bad = (int*)calloc((size_t)N, sizeof(int));
  int nonhit = 0, full = 0;

  for (int n = 0; n < N; ++n) {
    if (row_mask && !row_mask[n]) {
      bad[n] = 2; /* left out on request */
      continue;
    }
    bad[n] = request_bad(a, n);
    bad_rows += bad[n];
  }

  {
    StepCtx c0 = {a, hd, bad, NULL, out_f32, ring_o_f32};
    parallel_for(N * Hq, decide_item, &c0);
  }

  /* group classification: DEC.cu:1305-1402 */
  for (int n = 0; n < N; ++n) {
    if (bad[n]) continue;
    const int req = a->req_ids[n], P = a->past_lens[n];
    const int new_end = cache_end_for_pos(P, S);
    const int fs = F < new_end ? F : new_end; /* clamp_front_sink_end, DEC.cu:718-723 */
    for (int hkv = 0; hkv < Hkv; ++hkv) {
      int valid[16];
      int vcount = 0, begin = INT_MAX;
      for (int l = 0; l < G; ++l) {
        int hq = hkv * G + l;
        HeadDecision* h = &hd[n * Hq + hq];
        int v = h->hit && h->mslot >= 0 && h->new_end == new_end;
        int clen = h->new_end - h->rect_start;
        if (v) {
          float pl = a->lse_cache[((int64_t)req * M + h->mslot) * Hq + hq];
          /* bench_long_band: benchmark extension of the C ABI, lifts the "<= M" rule for
           * synthetic decisions only (no counterpart in the reference) */
          v = isfinite(pl) && clen >= 0 &&
              (clen <= M || (a->bench_long_band != 0 && a->bench_mode != 0));
        }
        valid[l] = v;
        if (v) {
          vcount++;
          if (h->rect_start < begin) begin = h->rect_start;
        }
      }
      int mode = 1;
      if (vcount == G)
        mode = 0;
      else if (vcount > 0 && a->mixed_group_fallback != 0)
        mode = 2;
      if (mode != 0) {
        begin = fs;
        for (int l = 0; l < G; ++l) {
          if (mode == 2 && valid[l]) continue;
          HeadDecision* h = &hd[n * Hq + hkv * G + l];
          h->hit = 0;
          h->mslot = -1;
          h->mpos = -1;
          h->prefix_end = 0;
          h->rect_start = fs;
          h->new_end = new_end;
        }
      }
      if (begin > new_end) begin = new_end;
      if (begin < 0) begin = 0;
      int64_t go = (int64_t)n * Hkv + hkv;
      gmode[go] = mode;
      if (a->group_rect_begin) a->group_rect_begin[go] = begin;
      if (a->group_rect_end) a->group_rect_end[go] = new_end;
      if (a->group_tail_begin) a->group_tail_begin[go] = new_end;
      if (a->group_tail_end) a->group_tail_end[go] = P + 1;
      if (a->group_mode) a->group_mode[go] = mode;
      if (mode != 0) nonhit++;
      if (mode == 1) full++;
    }
    for (int hq = 0; hq < Hq; ++hq) {
      int64_t ho = (int64_t)n * Hq + hq;
      HeadDecision* h = &hd[ho];
      if (a->head_hit) a->head_hit[ho] = h->hit;
      if (a->head_match_slot) a->head_match_slot[ho] = h->mslot;
      if (a->head_match_pos) a->head_match_pos[ho] = h->mpos;
      if (a->head_prefix_end) a->head_prefix_end[ho] = h->prefix_end;
      if (a->head_rect_start) a->head_rect_start[ho] = h->rect_start;
      if (a->head_new_end) a->head_new_end[ho] = h->new_end;
    }
  }
  if (a->task_counts) {
    a->task_counts[5] = nonhit;
    a->task_counts[6] = full;
  }

  /* attention + merge + ring write + output: DEC.cu:4346-4365 (prefix state),
   * 4485-4497 (ring write before the sink merge), 4500-4520 (sink, output only),
   * 4640-4672 (tail, output). */
  uint16_t* acache = (uint16_t*)a->attn_cache;
  /* The ring row read on a hit may be the row written this step (oldest
   * candidate); take all prefix states before any write. */
  State* prefix = (State*)malloc(sizeof(State) * (size_t)N * Hq);
  for (int idx = 0; idx < N * Hq; ++idx) {
    int n = idx / Hq, hq = idx % Hq;
    state_empty(&prefix[idx]);
    if (bad[n]) continue;
    HeadDecision* h = &hd[idx];
    if (h->hit && h->mslot >= 0) {
      int req = a->req_ids[n];
      float pl = a->lse_cache[((int64_t)req * M + h->mslot) * Hq + hq];
      if (isfinite(pl)) {
        const uint16_t* row = acache + (((int64_t)req * M + h->mslot) * Hq + hq) * D;
        for (int d = 0; d < D; ++d) prefix[idx].o[d] = (double)bf16_to_f32(row[d]);
        prefix[idx].lse = (double)pl;
      }
    }
  }

  {
    StepCtx c1 = {a, hd, bad, prefix, out_f32, ring_o_f32};
    parallel_for(N * Hq, attend_item, &c1);
  }

  free(prefix);
  free(hd);
  free(gmode);
  free(bad);
  return bad_rows;
}

ORACLE_API int mac_oracle_decode_step(const MacB200DecodeArgs* a, float* out_f32,
                                      float* ring_o_f32) {
  return mac_oracle_decode_step_rows(a, out_f32, ring_o_f32, NULL);
}

/* Decisions only (no attention): for large-shape decision parity. */
ORACLE_API int mac_oracle_decide(const MacB200DecodeArgs* a, int32_t* hit, int32_t* mslot,
                                 int32_t* mpos) {
  const int N = a->N, Hq = a->Hq;
  for (int idx = 0; idx < N * Hq; ++idx) {
    HeadDecision h;
    decide_head(a, idx / Hq, idx % Hq, &h);
    hit[idx] = h.hit;
    mslot[idx] = h.mslot;
    mpos[idx] = h.mpos;
  }
  return 0;
}

/* -------------------------------------------------------- prefill side -- */
/* PRE.cu:201-269 */
ORACLE_API int mac_oracle_prefill_update_cache(const MacB200PrefillArgs* p) {
  if (p->M <= 0 || p->B <= 0) return 0;
  const size_t row_bf16 = (size_t)p->H * p->D * 2, row_f32 = (size_t)p->H * 4;
  for (int b = 0; b < p->B; ++b) {
    int req = p->req_ids[b];
    int Ni = p->lens[b];
    if (Ni <= 0) continue;
    if (req < 0 || req >= p->R) continue;
    int start = Ni > p->M ? Ni - p->M : 0;
    int keep = Ni - start;
    int base_off = p->offsets[b];
    if (base_off < 0 || base_off + Ni > p->src_rows) continue;
    int L = p->request_length_by_batch ? p->request_length[b] : p->request_length[req];
    if (L < 0) L = 0;
    int base_dest = (int)(((int64_t)L + start) % p->M);
    for (int i = 0; i < keep; ++i) {
      int dest = base_dest + i;
      if (dest >= p->M) dest -= p->M;
      size_t src = (size_t)(base_off + start + i);
      size_t dst = (size_t)req * p->M + dest;
      memcpy((uint8_t*)p->q_cache + dst * row_bf16, (const uint8_t*)p->src_q + src * row_bf16,
             row_bf16);
      memcpy((uint8_t*)p->attn_cache + dst * row_bf16,
             (const uint8_t*)p->src_attn + src * row_bf16, row_bf16);
      memcpy((uint8_t*)p->lse_cache + dst * row_f32, (const uint8_t*)p->src_lse + src * row_f32,
             row_f32);
      if (p->q_post_cache) {
        uint16_t* r = (uint16_t*)((uint8_t*)p->q_post_cache + dst * row_bf16);
        for (int e = 0; e < p->H * p->D; ++e) r[e] = 0x7fc0;
      }
    }
    if (!p->request_length_by_batch) p->request_length[req] += Ni;
  }
  return 0;
}

/* PRE.cu:271-283 */
ORACLE_API int mac_oracle_mark_persistent_ready(uint8_t* ready, int64_t* cache_epoch,
                                                const int64_t* request_epoch,
                                                const int32_t* req_ids, int32_t B, int32_t R) {
  for (int i = 0; i < B; ++i) {
    int req = req_ids[i];
    if (req < 0 || req >= R) continue;
    cache_epoch[req] = request_epoch[req];
    ready[req] = 1;
  }
  return 0;
}
/* PRE.cu:285-298 */
ORACLE_API int mac_oracle_invalidate_persistent_ready(uint8_t* ready, int64_t* cache_epoch,
                                                      int64_t* request_epoch,
                                                      const int32_t* req_ids, int32_t B,
                                                      int32_t R) {
  for (int i = 0; i < B; ++i) {
    int req = req_ids[i];
    if (req < 0 || req >= R) continue;
    ready[req] = 0;
    cache_epoch[req] = -1;
    request_epoch[req] += 1;
  }
  return 0;
}
/* PRE.cu:300-320 */
ORACLE_API int mac_oracle_update_request_state(int32_t* req_len, int32_t* match_req_len,
                                               int32_t* cache_lens, const int32_t* req_ids,
                                               const int32_t* seq_lens, const int32_t* cur_lens,
                                               int32_t B, int32_t R) {
  for (int i = 0; i < B; ++i) {
    int32_t c = seq_lens[i] - cur_lens[i];
    if (c < 0) c = 0;
    cache_lens[i] = c;
    int req = req_ids[i];
    if (req < 0 || req >= R) continue;
    req_len[req] = seq_lens[i];
    match_req_len[req] = c;
  }
  return 0;
}

/* Helpers exported for unit tests of the position algebra and the hash. */
ORACLE_API int mac_oracle_ring_slot_to_pos(int past_len, int M, int slot) {
  return ring_slot_to_pos(past_len, M, slot);
}
ORACLE_API int mac_oracle_pos_to_ring_slot(int past_len, int M, int pos) {
  return pos_to_ring_slot(past_len, M, pos);
}
ORACLE_API float mac_oracle_ring_distance(const uint16_t* q, const uint16_t* c) {
  return ring_distance(q, c);
}
ORACLE_API float mac_oracle_threshold_distance(float threshold, int D) {
  MacB200DecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.threshold = threshold;
  a.D = D;
  return threshold_distance(&a);
}
ORACLE_API int mac_oracle_abi_struct_size(void) { return (int)sizeof(MacB200DecodeArgs); }
ORACLE_API int mac_oracle_build_struct_size(void) { return (int)sizeof(MacB200PrefillBuildArgs); }
ORACLE_API int mac_oracle_build_struct_tail_offset(void) {
  return (int)offsetof(MacB200PrefillBuildArgs, req_to_token);
}

/* ----------------------------------------------- decode RoPE + q preserve -- */
/* attention/src/mac_attention/integrations/sglang/csrc/mac_decode_rope_preserve.cu:35-156.
 * The rotation is evaluated the way the device compiler evaluates
 * x0*c - x1*s and x1*c + x0*s: second product rounded, first fused. */
static inline int64_t load_index(const void* p, int is_i64, int64_t n) {
  return is_i64 ? ((const int64_t*)p)[n] : (int64_t)((const int32_t*)p)[n];
}
ORACLE_API int mac_oracle_decode_rope_preserve(const MacB200RopeArgs* a) {
  const int64_t D = a->head_dim, R = a->rotary_dim, half = R / 2;
  uint16_t* q = (uint16_t*)a->q;
  uint16_t* k = (uint16_t*)a->k;
  const uint16_t* v = (const uint16_t*)a->v;
  uint16_t* q_pre = (uint16_t*)a->q_pre;
  uint16_t* kb = (uint16_t*)a->k_buffer;
  uint16_t* vb = (uint16_t*)a->v_buffer;
  for (int64_t n = 0; n < a->N; ++n) {
    const int64_t pos = load_index(a->positions, a->positions_i64, n);
    const int64_t loc = load_index(a->cache_locs, a->cache_locs_i64, n);
    const int pool_ok = loc >= 0 && loc < a->kv_pool_tokens;
    const float* cs = a->cos_sin_cache + pos * a->cos_sin_stride0;
    for (int which = 0; which < 2; ++which) {
      const int64_t H = which ? a->Hkv : a->Hq;
      for (int64_t h = 0; h < H; ++h) {
        uint16_t* row = which ? k + n * a->k_stride0 + h * D : q + n * a->q_stride0 + h * D;
        if (!which)
          for (int64_t d = 0; d < D; ++d) q_pre[(n * a->Hq + h) * D + d] = row[d];
        for (int64_t pair = 0; pair < half; ++pair) {
          const int64_t d0 = a->is_neox ? pair : 2 * pair, d1 = a->is_neox ? pair + half : d0 + 1;
          const float x0 = bf16_to_f32(row[d0]), x1 = bf16_to_f32(row[d1]);
          const float c = cs[pair], s = cs[half + pair];
          const float y0 = fmaf(x0, c, -(x1 * s));
          const float y1 = fmaf(x1, c, x0 * s);
          row[d0] = f32_to_bf16(y0);
          row[d1] = f32_to_bf16(y1);
        }
        if (which && pool_ok)
          for (int64_t d = 0; d < D; ++d) kb[(loc * a->Hkv + h) * D + d] = row[d];
      }
    }
    if (pool_ok)
      for (int64_t h = 0; h < a->Hkv; ++h)
        for (int64_t d = 0; d < D; ++d)
          vb[(loc * a->Hkv + h) * D + d] = v[n * a->v_stride0 + h * D + d];
  }
  return 0;
}

/* ------------------------------------------------------ prefill downdate -- */
/* attention/src/mac_attention/integrations/sglang/csrc/mac_merge_downdate_cache.cu:116-288,
 * float32 LSE only (the element types only change how the scalar is loaded). */
static void downdate_scalars_f(float l1, float l2, float* ret, float* t, float* scale) {
  const float diff = l2 - l1;
  const float em1 = expm1f(diff);
  const int last_block = fabsf(em1) <= 1e-7f;
  const int invalid = (diff > 0.0f) && !last_block;
  if (last_block) {
    *ret = -INFINITY; *t = 0.f; *scale = 0.f;
  } else if (invalid) {
    *ret = l1; *t = 0.f; *scale = 1.f;
  } else {
    const float one_minus = 1.f - expf(diff);
    *ret = l1 + logf(fmaxf(one_minus + 1e-7f, 1e-30f));
    *t = expf(diff);
    *scale = expf(l1 - *ret);
  }
}

ORACLE_API int mac_oracle_update_then_downdate(const uint16_t* out1, const float* lse1,
                                               uint16_t* out2, float* lse2, int64_t rows,
                                               int32_t D) {
  for (int64_t r = 0; r < rows; ++r) {
    float ret, t, scale;
    downdate_scalars_f(lse1[r], lse2[r], &ret, &t, &scale);
    for (int d = 0; d < D; ++d) {
      const float o = (bf16_to_f32(out1[r * D + d]) - t * bf16_to_f32(out2[r * D + d])) * scale;
      out2[r * D + d] = f32_to_bf16(o);
    }
    lse2[r] = ret;
  }
  return 0;
}

/* ------------------------------------------------ one-pass prefill build -- */
/* The ring contents the reference hook's operator sequence leaves
 * (attention/src/mac_attention/integrations/sglang/flashinfer_hooks.py:2459-2492:
 * band-LSE scale, downdate, ring copy, ready mark; -inf LSE under front sink,
 * 2205-2215), restated per ring row; float32 LSE inputs only.
 * MAC_B200_SINK_EXCLUDE has no reference implementation: it restates the
 * invariant the reference's comment gives -- a ring row covers exactly
 * [min(F, E), E) -- by removing the row's attention over the sink tokens
 * [0, min(F, E)), evaluated here in double precision, with a second downdate;
 * rows with E <= F hold the empty state (0, -inf), as decode-written rows do
 * (DEC.cu:4485-4497). */
typedef struct {
  const MacB200PrefillBuildArgs* a;
  int b, req, start, keep, base_off, base_dest, L;
} BuildCtx;

static void build_row_item(void* ctx, int i) {
  const BuildCtx* c = (const BuildCtx*)ctx;
  const MacB200PrefillBuildArgs* a = c->a;
  const MacB200PrefillArgs* p = &a->ring;
  const int H = p->H, D = p->D;
  int dest = c->base_dest + i;
  if (dest >= p->M) dest -= p->M;
  const size_t src = (size_t)(c->base_off + c->start + i);
  const size_t dst = (size_t)c->req * p->M + dest;
  const uint16_t* full = (const uint16_t*)p->src_attn + src * H * D;
  const uint16_t* band = (const uint16_t*)a->band_attn + src * H * D;
  uint16_t* orow = (uint16_t*)p->attn_cache + dst * H * D;
  memcpy((uint16_t*)p->q_cache + dst * H * D, (const uint16_t*)p->src_q + src * H * D,
         (size_t)H * D * 2);
  if (p->q_post_cache) {
    uint16_t* r = (uint16_t*)p->q_post_cache + dst * H * D;
    for (int e = 0; e < H * D; ++e) r[e] = 0x7fc0;
  }
  const int64_t pos = (int64_t)c->L + c->start + i;
  int64_t E = pos + 1 - a->semantic_pos_ahead;
  if (E < 0) E = 0;
  const int F = a->front_sink_tokens;
  double* osink = (double*)malloc(sizeof(double) * D);
  double* sc = (double*)malloc(sizeof(double) * (F > 0 ? F : 1));
  for (int h = 0; h < H; ++h) {
    float ret, t, scale;
    downdate_scalars_f(((const float*)p->src_lse)[src * H + h],
                       ((const float*)a->band_lse)[src * H + h] * a->band_lse_scale, &ret, &t,
                       &scale);
    if (a->sink_mode != MAC_B200_SINK_EXCLUDE) {
      for (int d = 0; d < D; ++d)
        orow[h * D + d] = f32_to_bf16(
            (bf16_to_f32(full[h * D + d]) - t * bf16_to_f32(band[h * D + d])) * scale);
      p->lse_cache[dst * H + h] = a->sink_mode == MAC_B200_SINK_UNMATCHABLE ? -INFINITY : ret;
      continue;
    }
    if (E <= F) {
      for (int d = 0; d < D; ++d) orow[h * D + d] = 0;
      p->lse_cache[dst * H + h] = -INFINITY;
      continue;
    }
    const int kh = h / (H / a->Hkv);
    const uint16_t* q = (const uint16_t*)a->q_post + (src * H + h) * D;
    double m = -INFINITY;
    for (int j = 0; j < F; ++j) {
      const int64_t tok = a->req_to_token[(int64_t)c->req * a->req_to_token_stride + j];
      const uint16_t* k = (const uint16_t*)a->k_buffer + (tok * a->Hkv + kh) * D;
      double dot = 0.0;
      for (int d = 0; d < D; ++d) dot += (double)bf16_to_f32(q[d]) * (double)bf16_to_f32(k[d]);
      sc[j] = dot * (double)a->sm_scale;
      if (sc[j] > m) m = sc[j];
    }
    double sum = 0.0;
    for (int d = 0; d < D; ++d) osink[d] = 0.0;
    for (int j = 0; j < F; ++j) {
      const int64_t tok = a->req_to_token[(int64_t)c->req * a->req_to_token_stride + j];
      const uint16_t* v = (const uint16_t*)a->v_buffer + (tok * a->Hkv + kh) * D;
      const double w = exp(sc[j] - m);
      sum += w;
      for (int d = 0; d < D; ++d) osink[d] += w * (double)bf16_to_f32(v[d]);
    }
    const float lse_sink = (float)(m + log(sum));
    float ret2, t2, scale2;
    downdate_scalars_f(ret, lse_sink, &ret2, &t2, &scale2);
    for (int d = 0; d < D; ++d) {
      const float mid = (bf16_to_f32(full[h * D + d]) - t * bf16_to_f32(band[h * D + d])) * scale;
      const float sk = sum > 0.0 ? (float)(osink[d] / sum) : 0.f;   /* F == 0: no sink at all */
      orow[h * D + d] = f32_to_bf16((mid - t2 * sk) * scale2);
    }
    p->lse_cache[dst * H + h] = ret2;
  }
  free(sc);
  free(osink);
}

ORACLE_API int mac_oracle_prefill_build(const MacB200PrefillBuildArgs* a) {
  const MacB200PrefillArgs* p = &a->ring;
  if (p->M <= 0 || p->B <= 0) return 0;
  for (int b = 0; b < p->B; ++b) {
    BuildCtx c;
    c.a = a;
    c.b = b;
    c.req = p->req_ids[b];
    const int Ni = p->lens[b];
    if (Ni <= 0) continue;
    if (c.req < 0 || c.req >= p->R) continue;
    c.start = Ni > p->M ? Ni - p->M : 0;
    c.keep = Ni - c.start;
    c.base_off = p->offsets[b];
    if (c.base_off < 0 || c.base_off + Ni > p->src_rows) continue;
    c.L = p->request_length_by_batch ? p->request_length[b] : p->request_length[c.req];
    if (c.L < 0) c.L = 0;
    c.base_dest = (int)(((int64_t)c.L + c.start) % p->M);
    parallel_for(c.keep, build_row_item, &c);
    if (!p->request_length_by_batch) p->request_length[c.req] += Ni;
  }
  if (a->ready)
    mac_oracle_mark_persistent_ready(a->ready, a->cache_epoch, a->request_epoch, p->req_ids, p->B,
                                     p->R);
  return 0;
}
