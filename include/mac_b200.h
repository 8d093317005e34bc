/*
 * mac_b200.h -- C ABI of the B200-native MAC-Attention fused decode path.
 *
 * Plain C: raw device pointers, int32/int64 sizes and scalars, no torch types.
 * Every entry point returns 0 on success or a negative MAC_B200_E* code; the
 * text of the last error on the calling thread is at mac_b200_last_error().
 * Nothing here synchronises the host with the device; work is queued on the
 * stream that is passed in (a cudaStream_t carried as void*; NULL = legacy
 * default stream) on the device that is current on the calling thread.
 *
 * Each entry point replaces one operator of the reference's PyTorch extension
 * modules (paths relative to the reference project,
 * attention/src/mac_attention/integrations/sglang/csrc/):
 *
 *   mac_b200_persistent_decode_bf16       mac_decode_persistent.cu:4962-5524
 *   mac_b200_prefill_update_cache         mac_prefill_update_cache.cu:324-372
 *   mac_b200_mark_persistent_ready        mac_prefill_update_cache.cu:374-409
 *   mac_b200_invalidate_persistent_ready  mac_prefill_update_cache.cu:411-446
 *   mac_b200_update_request_state         mac_prefill_update_cache.cu:448-495
 *   mac_b200_decode_rope_preserve_q_bf16  mac_decode_rope_preserve.cu:174-269
 *   mac_b200_update_then_downdate_bf16_inplace  mac_merge_downdate_cache.cu:320-401
 *
 * Notation: N batch rows, Hq query heads, Hkv KV heads, G = Hq/Hkv (1..8),
 * D = 128, M ring capacity, R ring rows, P = past_lens[n] (tokens already in
 * the KV pool, excluding the current one), S = semantic_pos_ahead,
 * F = front_sink_tokens.
 */
#ifndef MAC_B200_H_
#define MAC_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAC_B200_ABI_VERSION 2

/* Error codes (negative). */
#define MAC_B200_OK 0
#define MAC_B200_EINVAL (-1)      /* bad argument: shape, dtype flag, null pointer          */
#define MAC_B200_EUNSUPPORTED (-2)/* valid for the reference API but outside this build      */
#define MAC_B200_ECUDA (-3)       /* a CUDA runtime call failed (text has the CUDA error)    */
#define MAC_B200_ECAPTURE (-4)    /* scratch must grow but the stream is being captured      */
#define MAC_B200_ESIZE (-5)       /* request exceeds a stated fixed capacity                 */

/* Bits of the device status word (see mac_b200_query_status). */
#define MAC_B200_STATUS_BARRIER_TIMEOUT 0x1u /* a bounded grid-barrier wait ran out         */
#define MAC_B200_STATUS_BAD_REQUEST 0x2u     /* req id / length outside the tables; row zeroed */
#define MAC_B200_STATUS_SCHED_OVERFLOW 0x4u  /* internal schedule exceeded its arena         */
#define MAC_B200_STATUS_COPY_TIMEOUT 0x8u    /* a bounded wait on a bulk copy ran out          */

/*
 * Arguments of one fused MAC decode step.
 * Replaces the 68 positional arguments of the reference operator
 * mac_persistent_decode_bf16 (mac_decode_persistent.cu:4962-5030).  All
 * pointers are device pointers unless stated otherwise; "bf16" buffers are
 * passed as void*.  Tensors are contiguous, row-major, with the shapes given.
 *
 * The reference's task-list and partial-result workspaces (its arguments
 * complete_task_go .. partial_tail_lse) are private scratch of the old
 * kernel's scheduler; the host shim validates them for signature
 * compatibility and this kernel does not need them.
 */
typedef struct MacB200DecodeArgs {
  /* ---- sizes ---- */
  int32_t N;                   /* decode rows in this step                                  */
  int32_t Hq;                  /* query heads                                               */
  int32_t Hkv;                 /* KV heads                                                  */
  int32_t D;                   /* head dim, must be 128                                     */
  int32_t M;                   /* ring capacity (slots per request)                         */
  int32_t R;                   /* ring rows = query_cache.size(0)                           */
  int32_t req_to_token_rows;   /* rows of req_to_token                                      */
  int32_t req_to_token_stride; /* columns of req_to_token                                   */
  int64_t kv_tokens;           /* rows of k_buffer / v_buffer                               */
  int32_t ws_batch;            /* N' >= N: leading dim of the decision workspaces           */
  int32_t max_match_tiles;     /* Tm = match_dist.size(2) >= ceil(M / match_tile_slots)     */

  /* ---- scalars, same meaning as the reference operator's ---- */
  int32_t max_context;
  int32_t tile_tokens;         /* accepted; only used for reported counters                 */
  int32_t match_tile_slots;
  int32_t semantic_pos_ahead;  /* S */
  int32_t front_sink_tokens;   /* F (negative is treated as 0)                              */
  int32_t gen_min_limit;
  int32_t lookback_right;
  int32_t candidate_mode;
  float threshold;             /* hit iff dist < 2*D*(1-threshold)^2 (strict)               */
  float sm_scale;
  int32_t debug_enabled;       /* >= 2: write timestamps into phase_cycles                  */
  int32_t bench_mode;          /* 0 off, 1 synthetic per head, 2 synthetic per KV group     */
  float bench_hit_rate;
  float bench_hit_rate_std;
  float bench_skip_ratio;
  float bench_skip_ratio_std;
  float bench_match_lag_mean;
  float bench_match_lag_std;
  int32_t bench_seed;
  int32_t bench_miss_mask;     /* < 0 off */
  int32_t bench_layer_id;
  /* Result-affecting launcher knobs the reference reads from the environment
   * (mac_decode_persistent.cu:5229, 5337). */
  int32_t mixed_group_fallback; /* MAC_PERSISTENT_MIXED_GROUP_FALLBACK, default 1           */
  int32_t bench_exact_quota;    /* MAC_BENCH_EXACT_QUOTA, default 1                         */
  int32_t out_cache_loc_is_i64; /* 0: int32, 1: int64                                       */
  int32_t phase_cycles_count;   /* elements of phase_cycles (>= 6)                          */
  int32_t grid_cap;             /* > 0 caps the persistent grid (MAC_PERSISTENT_COOP_CTAS)  */
  /* Benchmark extension, no counterpart in the reference: with synthetic decisions
   * (bench_mode != 0) a reused entry may lie further back than the ring is long, i.e.
   * the rule "new_end - prefix_end <= M" (mac_decode_persistent.cu:1323-1328) is lifted,
   * so that bench_skip_ratio can place the matched prefix anywhere in the context.
   * 0 (default) keeps the reference's rule and its decisions. */
  int32_t bench_long_band;

  /* ---- inputs ----
   * Every pointer is an address the device can access.  q_post, q_pre and out may also be
   * page-locked host memory mapped into the device's address space: out is written once per
   * row, which saves the copy of the result back to the host; q_pre is read once per scanned
   * ring tile, so a step that scans should keep it in device memory. */
  const void* q_post;          /* [N,Hq,D] bf16, post-RoPE query (attention)                */
  const void* q_pre;           /* [N,Hq,D] bf16, pre-RoPE query (matching, ring write)      */
  const void* k_buffer;        /* [kv_tokens,Hkv,D] bf16                                    */
  const void* v_buffer;        /* [kv_tokens,Hkv,D] bf16                                    */
  const int32_t* req_to_token; /* [rows,stride] logical position -> KV pool row             */
  const int32_t* req_ids;      /* [>=N]                                                     */
  const int32_t* past_lens;    /* [>=N]                                                     */
  const void* out_cache_loc;   /* [>=N] int32 or int64: pool row of the current token       */
  /* ---- MAC ring (read and written) ---- */
  void* query_cache;           /* [R,M,Hq,D] bf16                                           */
  void* attn_cache;            /* [R,M,Hq,D] bf16                                           */
  float* lse_cache;            /* [R,M,Hq] f32, natural log                                 */
  /* ---- outputs ---- */
  void* out;                   /* [N,Hq,D] bf16                                             */
  float* optional_lse;         /* [N,Hq] f32 natural log, or NULL                           */
  /* ---- observable workspace outputs (all int32 unless noted) ---- */
  float* match_dist;           /* [N',Hq,Tm] f32 */
  int32_t* match_pos;          /* [N',Hq,Tm] */
  int32_t* match_slot;         /* [N',Hq,Tm] */
  int32_t* head_hit;           /* [N',Hq] */
  int32_t* head_match_slot;
  int32_t* head_match_pos;
  int32_t* head_prefix_end;
  int32_t* head_rect_start;
  int32_t* head_new_end;
  int32_t* group_rect_begin;   /* [N',Hkv] */
  int32_t* group_rect_end;
  int32_t* group_rect_tiles;
  int32_t* group_tail_begin;
  int32_t* group_tail_end;
  int32_t* group_tail_tiles;
  int32_t* group_mode;         /* 0 all heads reuse, 1 full attention, 2 mixed              */
  int32_t* task_counts;        /* [>=9] */
  int64_t* phase_cycles;       /* [phase_cycles_count] int64 */
  /* ---- readiness gate: NULL cache_ready = every request ready ---- */
  const uint8_t* cache_ready;  /* [R] bool/u8 */
  const int64_t* cache_epoch;  /* [R] or NULL */
  const int64_t* request_epoch;/* [R] or NULL */
} MacB200DecodeArgs;

/*
 * One fused MAC decode step: ring match scan, hit/miss/demoted scheduling,
 * partial attention, LSE merge, ring update and output, one persistent launch.
 * Replaces mac_persistent_decode_bf16 (mac_decode_persistent.cu:4962-5524).
 *
 * Scratch: a small per-device arena owned by the library holds split-KV
 * partials and scheduler words.  It is allocated (or grown) on the first call
 * that needs it, which therefore must not happen while `stream` is being
 * captured into a CUDA graph: make one eager call first.  Later calls allocate
 * nothing.  Launches of this entry point that overlap on one device race on
 * that arena; keep them on one stream or order them with events.
 */
int mac_b200_persistent_decode_bf16(const MacB200DecodeArgs* args, void* stream);

/*
 * The same decode step for hosts that cannot allocate device memory.
 * No counterpart in the reference (its operator takes all scratch from the
 * caller).
 *
 * Who needs it: a process whose own pool allocator owns all of HBM, a plugin
 * loaded under a sandbox that filters the driver's allocation calls, or code
 * that is already inside a region where allocating is illegal.  This entry
 * point never calls cudaMalloc, cudaFree or any allocating library routine:
 * its scratch (split-KV partials, scheduler words) is one fixed 8 MiB block
 * of device memory built into the library image, which every GPU that loads
 * the library keeps until the process exits.
 *
 * Limit: a step whose scratch need exceeds the block is refused with
 * MAC_B200_ESIZE and a message that names the need.  With a grid of 148 CTAs
 * the need is roughly (296 + 3*N*Hkv) * (Hq/Hkv) * 512 bytes, so e.g. 64
 * requests x 8 KV heads with 4..8 query heads per KV head fit.
 *
 * The first call on a device looks up the block's device address and sets the
 * kernel's attributes; make that first call outside of any stream capture.
 * All calls on a device share the block and it keeps the previous call's
 * contents (the kernel clears the words that must start at zero), so two of
 * these calls -- or one of these and one mac_b200_persistent_decode_bf16 --
 * that overlap on the GPU race; keep them on one stream or order them.
 */
int mac_b200_persistent_decode_bf16_noalloc(const MacB200DecodeArgs* args, void* stream);

/*
 * Arguments of the prefill-side ring build.
 * Replaces the 14 arguments of mac_prefill_update_cache
 * (mac_prefill_update_cache.cu:324-337).
 */
typedef struct MacB200PrefillArgs {
  int32_t R, M, H, D;            /* ring geometry: q_cache is [R,M,H,D]                       */
  int32_t B;                     /* batch rows = req_ids.size(0)                              */
  int32_t src_rows;              /* rows of src_q / src_attn / src_lse                        */
  int32_t request_length_by_batch; /* 1: request_length is [B] (read only); 0: [R], bumped    */
  void* q_cache;                 /* [R,M,H,D] bf16 */
  void* attn_cache;              /* [R,M,H,D] bf16 */
  float* lse_cache;              /* [R,M,H] f32    */
  void* q_post_cache;            /* [R,M,H,D] bf16 or NULL: rows get the bf16 NaN 0x7fc0      */
  int32_t* request_length;       /* [R] or [B] */
  const int32_t* req_ids;        /* [B] */
  const void* src_q;             /* [src_rows,H,D] bf16 */
  const void* src_attn;          /* [src_rows,H,D] bf16 */
  const float* src_lse;          /* [src_rows,H] f32 */
  const int32_t* offsets;        /* [B+1] row offsets into src_* */
  const int32_t* lens;           /* [B] */
} MacB200PrefillArgs;

/* Replaces mac_prefill_update_cache (mac_prefill_update_cache.cu:324-372). */
int mac_b200_prefill_update_cache(const MacB200PrefillArgs* args, void* stream);

/* Replaces mac_mark_persistent_ready (mac_prefill_update_cache.cu:374-409):
 * for each valid req: cache_epoch[req] = request_epoch[req]; ready[req] = 1. */
int mac_b200_mark_persistent_ready(uint8_t* ready, int64_t* cache_epoch,
                                   const int64_t* request_epoch, const int32_t* req_ids,
                                   int32_t B, int32_t R, void* stream);

/* Replaces mac_invalidate_persistent_ready (mac_prefill_update_cache.cu:411-446):
 * ready[req] = 0; cache_epoch[req] = -1; request_epoch[req] += 1. */
int mac_b200_invalidate_persistent_ready(uint8_t* ready, int64_t* cache_epoch,
                                         int64_t* request_epoch, const int32_t* req_ids,
                                         int32_t B, int32_t R, void* stream);

/* Replaces mac_update_request_state (mac_prefill_update_cache.cu:448-495). */
int mac_b200_update_request_state(int32_t* req_len, int32_t* match_req_len,
                                  int32_t* cache_lens, const int32_t* req_ids,
                                  const int32_t* seq_lens, const int32_t* cur_lens,
                                  int32_t B, int32_t R, void* stream);

/*
 * One-pass prefill ring build: LSE downdate + ring write + readiness mark.
 *
 * The reference's prefill hook (flashinfer_hooks.py:2459-2492) runs, per layer,
 *   band_lse *= ln 2                                   (elementwise, all rows)
 *   mac_update_then_downdate_bf16_inplace(full, band)  (all rows, in place)
 *   mac_prefill_update_cache(ring, q, band, band_lse)  (last min(len, M) rows)
 *   mac_mark_persistent_ready(...)
 * and, when front_sink_tokens > 0, first overwrites the LSE with -inf so that
 * prefill rows can never match (flashinfer_hooks.py:2205-2215).  Only the last
 * min(len, M) rows of a request ever reach the ring, so this entry point
 * downdates just those rows on their way into the ring and marks the requests
 * ready, in one pass over the data.  The ring contents are those of the
 * sequence above; the band tensors are NOT modified (the reference overwrites
 * them with the downdated state and never reads them again).
 *
 * sink_mode selects what front-sink handling the ring rows get:
 *   MAC_B200_SINK_NONE        F == 0: ring row = full - band.
 *   MAC_B200_SINK_UNMATCHABLE the reference's behaviour for F > 0: same state,
 *                             LSE = -inf (row can never be reused).
 *   MAC_B200_SINK_EXCLUDE     no counterpart in the reference (its comment at
 *                             flashinfer_hooks.py:2205-2215 describes it as not
 *                             implemented): the attention of each row's post-RoPE
 *                             query over the sink tokens [0, min(F, E)),
 *                             E = max(pos + 1 - S, 0), is computed in the kernel
 *                             and subtracted too, so the ring row covers exactly
 *                             [min(F, E), E) as decode-written rows do and is
 *                             matchable at once.  Needs D = 128, F <= 128, H / Hkv in
 *                             {1, 2, 4, 8, 16}, sm_scale > 0 and 16-byte aligned tensors
 *                             (else MAC_B200_EUNSUPPORTED / MAC_B200_EINVAL).
 */
#define MAC_B200_SINK_NONE 0
#define MAC_B200_SINK_UNMATCHABLE 1
#define MAC_B200_SINK_EXCLUDE 2

typedef struct MacB200PrefillBuildArgs {
  MacB200PrefillArgs ring;       /* ring.src_attn / ring.src_lse: state of the FULL prefix of
                                    each row; ring.src_lse holds full_lse_dtype elements      */
  const void* band_attn;         /* [src_rows,H,D] bf16: state of each row's trailing window  */
  const void* band_lse;          /* [src_rows,H], band_lse_dtype elements                     */
  int32_t full_lse_dtype;        /* MAC_B200_LSE_*                                            */
  int32_t band_lse_dtype;        /* MAC_B200_LSE_*                                            */
  float band_lse_scale;          /* band LSE is multiplied by this first (ln 2 for a log2-
                                    domain producer, 1 otherwise)                             */
  int32_t sink_mode;             /* MAC_B200_SINK_*                                           */
  uint8_t* ready;                /* [R] or NULL: readiness gate to mark (all three or none)   */
  int64_t* cache_epoch;          /* [R]                                                       */
  const int64_t* request_epoch;  /* [R]                                                       */
  /* MAC_B200_SINK_EXCLUDE only */
  int32_t Hkv;                   /* KV heads; H % Hkv == 0                                    */
  int32_t front_sink_tokens;     /* F                                                         */
  int32_t semantic_pos_ahead;    /* S: a row at position pos has prefix end E = pos + 1 - S   */
  int32_t req_to_token_rows;
  int32_t req_to_token_stride;
  float sm_scale;
  int64_t kv_tokens;             /* rows of k_buffer / v_buffer                               */
  const void* q_post;            /* [src_rows,H,D] bf16 post-RoPE queries                     */
  const void* k_buffer;          /* [kv_tokens,Hkv,D] bf16                                    */
  const void* v_buffer;          /* [kv_tokens,Hkv,D] bf16                                    */
  const int32_t* req_to_token;   /* [rows,stride] logical position -> KV pool row             */
} MacB200PrefillBuildArgs;

int mac_b200_prefill_downdate_update_cache(const MacB200PrefillBuildArgs* args, void* stream);

/*
 * Arguments of the decode-time fused "preserve pre-RoPE q + RoPE(q,k) + KV-pool
 * write".  Replaces the 11 arguments of mac_decode_rope_preserve_q_bf16
 * (mac_decode_rope_preserve.cu:174-186).  Strides are in elements; the last
 * dimension of q, k, v is contiguous.
 */
typedef struct MacB200RopeArgs {
  int64_t N;                 /* decode tokens                                             */
  int32_t Hq, Hkv;           /* heads of q and of k/v                                     */
  int32_t head_dim;          /* D                                                         */
  int32_t rotary_dim;        /* = cos_sin_cache.size(1), even, <= D                       */
  int32_t is_neox;           /* 1: pairs (d, d + rotary_dim/2); 0: pairs (2p, 2p+1)       */
  int32_t positions_i64;     /* 0: int32, 1: int64                                        */
  int32_t cache_locs_i64;    /* 0: int32, 1: int64                                        */
  int32_t reserved;
  int64_t q_stride0, k_stride0, v_stride0;  /* row strides of q, k, v                     */
  int64_t cos_sin_stride0;   /* row stride of cos_sin_cache                               */
  int64_t kv_pool_tokens;    /* rows of k_buffer / v_buffer                               */
  void* q;                   /* [N, Hq*D] bf16, rotated in place                          */
  void* k;                   /* [N, Hkv*D] bf16, rotated in place                         */
  const void* v;             /* [N, Hkv*D] bf16                                           */
  void* q_pre;               /* [>=N, Hq, D] bf16: q before rotation                      */
  void* k_buffer;            /* [T, Hkv, D] bf16: row cache_locs[n] <- rotated k          */
  void* v_buffer;            /* [T, Hkv, D] bf16: row cache_locs[n] <- v                  */
  const float* cos_sin_cache;/* [max_pos, rotary_dim] f32: cos | sin                      */
  const void* positions;     /* [>=N] int32|int64                                         */
  const void* cache_locs;    /* [>=N] int32|int64                                         */
} MacB200RopeArgs;

/* Replaces mac_decode_rope_preserve_q_bf16 (mac_decode_rope_preserve.cu:174-269).
 * Rows of cache_locs outside [0, kv_pool_tokens) are not written to the pool. */
int mac_b200_decode_rope_preserve_q_bf16(const MacB200RopeArgs* args, void* stream);

/* LSE element types of the downdate operator. */
#define MAC_B200_LSE_F32 0
#define MAC_B200_LSE_F16 1
#define MAC_B200_LSE_BF16 2

/*
 * Replaces mac_update_then_downdate_bf16_inplace (mac_merge_downdate_cache.cu:320-401):
 * for each of `rows` (token, head) rows, (out2, lse2) <- (out1, lse1) minus (out2, lse2):
 *   lse2 <- lse1 + log(1 - exp(lse2 - lse1)),  out2 <- (out1 - exp(lse2 - lse1) * out2) * scale,
 * with the reference's guards (window equal to the whole -> empty state; window
 * larger than the whole -> keep (out1, lse1)).  out1/out2: [rows, D] bf16
 * contiguous; lse1/lse2: [rows] of the given element types, natural log.
 */
int mac_b200_update_then_downdate_bf16_inplace(const void* out1, const void* lse1,
                                               int32_t lse1_dtype, void* out2, void* lse2,
                                               int32_t lse2_dtype, int64_t rows, int32_t D,
                                               void* stream);

/* Text of the last error raised on the calling thread ("" if none).
 * Stands in for the c10::Error text of the reference's TORCH_CHECKs. */
const char* mac_b200_last_error(void);

/* MAC_B200_ABI_VERSION the library was built with. */
int mac_b200_abi_version(void);

/*
 * Reads (and clears) the sticky device status word of the current device:
 * synchronises `stream`, copies the word back, resets barrier state if a
 * bounded wait ran out.  Not on the hot path; tests and health checks poll it.
 * No counterpart in the reference (its kernel has no bounded waits).
 */
int mac_b200_query_status(uint32_t* status_out, void* stream);

/*
 * Self-test of the kernels' bounded waits (no counterpart in the reference,
 * whose grid.sync() cannot time out).  Runs a two-CTA kernel that waits at a
 * barrier which nothing completes, with a 2 ms limit, on barrier words of its
 * own: both CTAs must give up and return.  Reports how many CTAs gave up and
 * the status word they left (read and cleared like mac_b200_query_status).
 * Synchronises the stream; a health check, not a hot-path call.
 */
int mac_b200_selftest_bounded_wait(uint32_t* status_out, int32_t* ctas_gave_up, void* stream);

/*
 * Static launch facts of the decode kernel on the current device, for logs
 * and benchmarks (the reference prints the same under
 * MAC_PERSISTENT_DEBUG_LAUNCH, mac_decode_persistent.cu:5406-5419).
 */
typedef struct MacB200LaunchInfo {
  int32_t sm_count;
  int32_t ctas_per_sm;
  int32_t block_threads;
  int32_t dynamic_smem_bytes;
  int32_t regs_per_thread;
  int32_t last_grid;            /* grid of the most recent decode launch on this device      */
  int64_t arena_bytes;          /* current size of the per-device scratch arena              */
  int64_t kernel_launches;      /* decode + prefill + gate kernels launched by this process  */
} MacB200LaunchInfo;
int mac_b200_launch_info(MacB200LaunchInfo* info);

#ifdef __cplusplus
}
#endif
#endif /* MAC_B200_H_ */
