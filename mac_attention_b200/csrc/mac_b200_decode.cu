// Fused MAC decode step for B200 (sm_100a): one persistent, CUDA-graph-safe launch.
//
// What one launch does, for every decode row n and query head:
//   A. match scan    squared-L2 distance between the pre-RoPE query and every
//                    candidate row of the request's recent-query ring; per
//                    match tile argmin with (distance, then older position)
//                    ordering.
//   B. classify      per head hit test / synthetic benchmark override /
//                    front-sink demotion; per KV group mode (all heads reuse,
//                    full attention, mixed); per group token rows
//                    sink | band | tail and their cost.
//   C. attend+merge  the rows of all groups are laid end to end in a "cost
//                    space" ordered demoted -> miss -> hit queue and cut into
//                    equal pieces, a whole multiple of the grid (wave-quantised);
//                    CTAs pull pieces by ticket.  Each (piece x row) segment is
//                    streamed through a per-warp cp.async ring of 16-token bf16
//                    K/V blocks and contracted with mma.sync m16n8k16 (the GQA
//                    group's query rows padded to 16).  The CTA that retires a
//                    group's last segment LSE-merges prefix state + partials,
//                    writes the ring row and the output.
// Phases are separated by two grid barriers (bounded spins, cooperative launch
// guarantees co-residency); nothing else waits on another CTA.
//
// Semantics follow the reference kernel
// attention/src/mac_attention/integrations/sglang/csrc/mac_decode_persistent.cu
// (cited as DEC.cu below); structure, scheduling and data flow are new.
#include <cuda.h>
#include <cuda_bf16.h>

#include <climits>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "mac_b200_common.h"

namespace mac_b200 {
namespace {

// ----------------------------------------------------------------- constants
constexpr int kD = 128;                    // head dim (fixed, as in the reference)
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;                 // per-warp cp.async ring depth
constexpr int kBlkTok = 16;                // tokens per warp block (one mma K step of P.V)
constexpr int kRowBytes = kD * 2;          // one bf16 K or V row
constexpr int kStageBytes = 2 * kBlkTok * kRowBytes;     // K block + V block = 8 KB
constexpr int kWarpRingBytes = kStages * kStageBytes;    // 24 KB
constexpr int kRingBytes = kWarps * kWarpRingBytes;      // 192 KB
constexpr int kMaxGroups = 4096;           // N * Hkv upper bound of one launch
constexpr int kMaxHq = 128;
constexpr int kOvhTok = 256;               // cost of opening a row, in token equivalents (G <= 4)
constexpr int kMinPieceTok = 1536;          // smallest streaming piece worth its fixed cost
constexpr int kMaxWaves = 4;                // most pieces per CTA the arena is sized for
constexpr unsigned kFuseMaxCost = 8192;       // groups up to this cost are never split over pieces
constexpr int kCombineRow = kD + 8;        // padded fp32 row of the cross-warp combine buffer
constexpr int kSmemPerm = kMaxGroups * 2;              // u16 gperm[]
constexpr int kSmemPrefix = (kMaxGroups + 1) * 4;      // u32 cost prefix
constexpr int kSmemMisc = 1024;
constexpr int kSmemBytes = kRingBytes + kSmemPerm + kSmemPrefix + 12 + kSmemMisc;
// mbarrier words of the bulk-copy scan (64-byte aligned, inside the kSmemMisc tail)
constexpr int kSmemBars = (kRingBytes + kSmemPerm + kSmemPrefix + 12 + 63) / 64 * 64;
static_assert(kSmemBars + 64 <= kSmemBytes, "mbarrier words must fit the tail");
constexpr unsigned long long kBarrierLimitNs = 2000000000ull;  // a grid-barrier wait gives up after 2 s
constexpr float kLog2e = 1.4426950408889634074f;
constexpr float kLn2 = 0.6931471805599453094f;

// Cross-launch state: the grid barrier words and the sticky status word.  Zero
// at module load; the barrier leaves its counter at zero after every use.
__device__ unsigned g_bar_count = 0;
__device__ unsigned g_bar_gen = 0;
__device__ unsigned g_status = 0;

struct GroupPlan {
  int32_t sink_hi;   // sink row  [0, sink_hi)
  int32_t band_lo;   // band row  [band_lo, new_end)
  int32_t new_end;   // tail row  [new_end, kv_len)
  int32_t kv_len;
  int32_t cls;       // 0 demoted queue, 1 miss queue, 2 hit queue
  int32_t cost;      // token equivalents, sum over non-empty rows of (len + kOvhTok)
  int32_t mode;
  int32_t req;       // ring / page-table row of the request (-1 for a malformed row)
};

struct Arena {
  uint32_t* ticket;      // [1] piece ticket of phase C
  int32_t* garrive;      // [NG] segments retired per group
  GroupPlan* plan;       // [NG]
  float* part_o;         // [slots][G][kD]
  float* part_lse;       // [slots][8]
  int32_t slots;
};

struct DecodeParams {
  MacB200DecodeArgs a;
  Arena ar;
  float thr_dist;
  float scale_log2;      // sm_scale * log2(e)
  int32_t G;
  int32_t NG;
  int32_t F;             // front_sink_tokens clamped at 0
  int32_t tm_used;       // ceil(M / match_tile_slots)
  int32_t max_pieces;
  int32_t force_waves;   // 0: pick by size; 1, 2 or 4: tuning override (MAC_B200_PIECE_WAVES)
  int32_t ovh_tok;       // cost of opening a row, in token equivalents (kOvhTok unless overridden)
  int32_t min_piece;     // smallest piece worth its fixed cost (kMinPieceTok unless overridden)
  int32_t fuse_max;      // groups up to this cost are never split (kFuseMaxCost unless overridden)
  int32_t scan_mode;     // 0: per-thread cp.async staging; 1 / 2: bulk tensor copies, 64 B / 128 B probe
};

// ------------------------------------------------------------- small helpers
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                            uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col).  Rows 8..15 of A are
// always zero here (at most 8 query heads share a KV head), so a1 = a3 = 0.
__device__ __forceinline__ void mma_bf16_rows8(float (&c)[4], uint32_t a0, uint32_t a2,
                                               uint32_t b0, uint32_t b1) {
  const uint32_t z = 0u;
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}

// DEC.cu:798-807
__device__ __forceinline__ int ring_slot_to_pos(int past_len, int M, int slot) {
  if (past_len < M) return slot;
  int order = slot - past_len % M;
  if (order < 0) order += M;
  return past_len - M + order;
}
// DEC.cu:837-848
__device__ __forceinline__ int pos_to_ring_slot(int past_len, int M, int pos) {
  if (past_len < M) return pos;
  int slot = (pos - (past_len - M)) + past_len % M;
  if (slot >= M) slot -= M;
  if (slot < 0) slot += M;
  return slot;
}
__device__ __forceinline__ int cache_end_for_pos(int p, int S) {
  const int e = p + 1 - S;
  return e > 0 ? e : 0;
}
__device__ __forceinline__ bool better_pair(float d, int pos, float bd, int bp) {
  return (d < bd) || (d == bd && pos < bp);
}
// DEC.cu:221-230
__device__ __forceinline__ bool request_ready(const MacB200DecodeArgs& a, int req) {
  if (a.cache_ready == nullptr) return true;
  if (req < 0) return false;
  if (a.cache_ready[req] == 0) return false;
  if (a.cache_epoch != nullptr && a.request_epoch != nullptr &&
      a.cache_epoch[req] != a.request_epoch[req])
    return false;
  return true;
}
__device__ __forceinline__ bool request_bad(const MacB200DecodeArgs& a, int n) {
  const int req = a.req_ids[n];
  const int P = a.past_lens[n];
  return req < 0 || req >= a.R || req >= a.req_to_token_rows || P < 0 ||
         P > a.req_to_token_stride;
}
__device__ __forceinline__ void candidate_window(const MacB200DecodeArgs& a, int P, int& begin,
                                                 int& end) {
  begin = P - a.M > 0 ? P - a.M : 0;
  end = P;
  if (a.candidate_mode == 1) {
    end = P - a.lookback_right;
    if (end < begin) end = begin;
  }
}

// Synthetic-decision hash of the reference's benchmark mode, DEC.cu:817-835.
__device__ __forceinline__ uint32_t mix_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float uniform01_u32(uint32_t x) {
  return static_cast<float>(mix_u32(x) & 0x00ffffffu) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ float pseudo_normal_u32(uint32_t x) {
  float s = uniform01_u32(x);
  s = __fadd_rn(s, uniform01_u32(x ^ 0x9e3779b9u));
  s = __fadd_rn(s, uniform01_u32(x ^ 0x85ebca6bu));
  s = __fadd_rn(s, uniform01_u32(x ^ 0xc2b2ae35u));
  return __fmul_rn(__fadd_rn(s, -2.0f), 1.7320508075688772f);
}
__device__ __forceinline__ float clampf(float v, float lo, float hi) {
  return fminf(fmaxf(v, lo), hi);
}
// DEC.cu:375-388 (the a*b+c there is one fused multiply-add on the device)
__device__ __forceinline__ int bench_target_miss_units(const MacB200DecodeArgs& a, int total) {
  if (total <= 0) return 0;
  float miss_rate = clampf(__fadd_rn(1.0f, -a.bench_hit_rate), 0.0f, 1.0f);
  int miss;
  if (a.bench_exact_quota != 0 && a.bench_hit_rate_std == 0.0f)
    miss = static_cast<int>(floorf(__fmaf_rn(miss_rate, static_cast<float>(total), 0.5f)));
  else
    miss = static_cast<int>(ceilf(__fmul_rn(miss_rate, static_cast<float>(total))));
  if (miss < 0) miss = 0;
  if (miss > total) miss = total;
  return miss;
}

// ------------------------------------------------------------- grid barrier
// Sense-reversing barrier on two device words.  The wait is bounded by wall
// time (%globaltimer): when it runs out the CTA records
// MAC_B200_STATUS_BARRIER_TIMEOUT and the kernel returns (every CTA observes the
// failure through the return value; none is left spinning).
__device__ __forceinline__ unsigned long long global_ns_u64() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ bool grid_barrier_on(unsigned nblocks, unsigned* count, unsigned* gen_word,
                                unsigned long long limit_ns) {
  __shared__ int sh_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    const unsigned gen = ld_acquire_u32(gen_word);
    __threadfence();
    const unsigned prev = atomicAdd(count, 1u);
    if (prev == nblocks - 1) {
      *count = 0;
      __threadfence();
      atomicAdd(gen_word, 1u);
    } else {
      const unsigned long long t0 = global_ns_u64();
      unsigned polls = 0;
      while (ld_acquire_u32(gen_word) == gen) {
        __nanosleep(40);
        if ((++polls & 31u) == 0u && global_ns_u64() - t0 > limit_ns) {
          atomicOr(&g_status, MAC_B200_STATUS_BARRIER_TIMEOUT);
          ok = 0;
          break;
        }
      }
    }
    __threadfence();
    sh_ok = ok;
  }
  __syncthreads();
  return sh_ok != 0;
}
__device__ bool grid_barrier(unsigned nblocks) {
  return grid_barrier_on(nblocks, &g_bar_count, &g_bar_gen, kBarrierLimitNs);
}

// Self-test of the bounded wait: two CTAs meet at a barrier that expects three,
// on words of their own, with a 2 ms limit.  Nothing ever completes it; both
// give up, set the status bit and return.
__device__ unsigned g_selftest_count = 0;
__device__ unsigned g_selftest_gen = 0;
__global__ void bounded_wait_selftest_kernel(int* gave_up) {
  const bool ok = grid_barrier_on(gridDim.x + 1, &g_selftest_count, &g_selftest_gen, 2000000ull);
  if (threadIdx.x == 0 && !ok) atomicAdd(gave_up, 1);
}

// ---------------------------------------------------------------- phase A
// Match scan.  The CTA owns match tiles blockIdx.x, blockIdx.x + grid, ... of
// the (tile, request) grid.  Eight lanes (an "octet") own one (slot, head) ring
// row at a time; lane j holds dims [8j, 8j+8) and, for rows that survive the
// probe, dims [64+8j, 64+8j+8).
//
//  * Probe: only the first 128 bytes of every candidate row are fetched and
//    their 64-dim partial distance is estimated in packed bf16 arithmetic with
//    a proven relative error below 2.4 %.  The partial distance is a lower
//    bound of the full one, so a row whose estimate is >= 1.0625 x the hit
//    threshold can never be a hit and is dropped; like the reference's probe
//    (DEC.cu:996-1059) this never changes a decision.
//  * Survivors: the second 128 bytes are fetched and the full distance is
//    formed as in the reference (DEC.cu:1062-1069, 343-349): per-lane sums of 8
//    sequential FMAs, then pairwise at lane distance 8 (here: in-lane, first
//    half + second half), 4, 2, 1 -- bit-identical results, so thresholds and
//    (distance, older position) ties resolve identically.
//  * Rows reach the lanes through a per-thread cp.async ring in shared memory
//    (a batch = 8 rows x 16 bytes + the two query chunks, kScanDepth-1 batches
//    in flight).  A lane only reads back bytes it copied itself: no barrier.
//  * The probe sums of a batch are reduced with a halving exchange (7 shuffles
//    for 8 rows): after steps at lane distance 4, 2, 1 lane j holds row j.
constexpr int kScanU = 8;
constexpr int kScanDepth = 4;
constexpr int kScanLaneChunks = kScanU + 2;                          // 8 rows + 2 query chunks
constexpr int kScanStageBytes = kScanLaneChunks * 16 * kThreads;     // 40 KB
constexpr int kScanRoundTiles = 32;   // tiles per round when sub-results are combined in smem
static_assert(kScanDepth * kScanStageBytes + kScanRoundTiles * (32 * 12 + 48) <= kRingBytes,
              "scan ring must fit");

struct ScanCursor {
  int k, hi, b;                 // tile of the round, head of this octet, batch of the tile
  int n, tile, P, req, cbeg, cend, s_begin, s_end;
  int tail, off_lo, off_hi;     // logical position of slot s: s + (s < tail ? off_lo : off_hi)
  bool elig;
};

// ring_slot_to_pos (DEC.cu:798-807) with the modulo hoisted out of the slot loop.
__device__ __forceinline__ int scan_slot_pos(const ScanCursor& c, int s) {
  return s + (s < c.tail ? c.off_lo : c.off_hi);
}

// Tile descriptors of a round live in shared memory: they are worked out once
// (one thread per tile) instead of inside the streaming loop.
struct ScanTileInfo {
  int n, tile, P, req, cbeg, cend, s_begin, s_end, tail, off_lo, off_hi, elig;
};
__device__ __forceinline__ void scan_fetch_tile(const ScanTileInfo* info, int k, ScanCursor& c) {
  const int4* src = reinterpret_cast<const int4*>(info + k);
  const int4 w0 = src[0], w1 = src[1], w2 = src[2];
  c.n = w0.x; c.tile = w0.y; c.P = w0.z; c.req = w0.w;
  c.cbeg = w1.x; c.cend = w1.y; c.s_begin = w1.z; c.s_end = w1.w;
  c.tail = w2.x; c.off_lo = w2.y; c.off_hi = w2.z; c.elig = w2.w != 0;
}

__device__ __forceinline__ void scan_load_tile(const MacB200DecodeArgs& a, int g, ScanCursor& c) {
  c.tile = g / a.N;
  c.n = g - c.tile * a.N;
  c.s_begin = c.tile * a.match_tile_slots;
  c.s_end = min(a.M, c.s_begin + a.match_tile_slots);
  c.elig = false;
  c.P = 0; c.req = 0; c.cbeg = 0; c.cend = 0;
  c.tail = 0; c.off_lo = 0; c.off_hi = 0;
  if (!request_bad(a, c.n)) {
    c.P = a.past_lens[c.n];
    c.req = a.req_ids[c.n];
    candidate_window(a, c.P, c.cbeg, c.cend);
    c.elig = c.P >= a.gen_min_limit && c.cend > c.cbeg && request_ready(a, c.req);
    if (c.P >= a.M) {
      c.tail = c.P % a.M;
      c.off_lo = c.P - c.tail;          // slots before the write cursor hold the newest positions
      c.off_hi = c.P - a.M - c.tail;    // slots from the cursor on hold the oldest
    }
  }
}

// sum over 8 dims of (q - c)^2, sequential FMAs from 0 (one lane's share of a row)
__device__ __forceinline__ float scan_dist8(const float (&q)[8], const uint4& raw) {
  float t = 0.0f, diff;
  diff = q[0] - bf16_lo(raw.x); t = __fmaf_rn(diff, diff, t);
  diff = q[1] - bf16_hi(raw.x); t = __fmaf_rn(diff, diff, t);
  diff = q[2] - bf16_lo(raw.y); t = __fmaf_rn(diff, diff, t);
  diff = q[3] - bf16_hi(raw.y); t = __fmaf_rn(diff, diff, t);
  diff = q[4] - bf16_lo(raw.z); t = __fmaf_rn(diff, diff, t);
  diff = q[5] - bf16_hi(raw.z); t = __fmaf_rn(diff, diff, t);
  diff = q[6] - bf16_lo(raw.w); t = __fmaf_rn(diff, diff, t);
  diff = q[7] - bf16_hi(raw.w); t = __fmaf_rn(diff, diff, t);
  return t;
}
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
  f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// 8-dim partial distance in packed bf16 (probe only; see its error bound at the use).
__device__ __forceinline__ float scan_probe8(const uint4& q, const uint4& c) {
  const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&q);
  const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c);
  __nv_bfloat162 acc = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 d = __hsub2(q2[i], c2[i]);
    acc = __hfma2(d, d, acc);
  }
  const uint32_t bits = *reinterpret_cast<const uint32_t*>(&acc);
  return bf16_lo(bits) + bf16_hi(bits);
}

// Exact distance of the rows of a batch that passed the probe (bits of `live`):
// first half re-read from the staged copy, second 128 bytes fetched, per-lane
// fp32 sums of 8 sequential FMAs, lane distance 8 = in-lane add of the two
// halves, then lane distances 4, 2, 1 (DEC.cu:1062-1069, 343-349).  Kept out of
// line: it runs for a handful of rows per request and would otherwise double
// the size of the streaming loop.
struct ScanBest {
  float d;
  int p, s;
};
__device__ __noinline__ ScanBest scan_survivors(unsigned live, const uint8_t* stage,
                                                const char* rows, int64_t slot_stride,
                                                unsigned oct_mask, int s_first, int spar,
                                                int tail, int off_lo, int off_hi, float bd,
                                                int bp, int bs) {
  float qlo[8], qhi[8];
  unpack8(*reinterpret_cast<const uint4*>(stage + kScanU * (kThreads * 16)), qlo);
  unpack8(*reinterpret_cast<const uint4*>(stage + (kScanU + 1) * (kThreads * 16)), qhi);
  uint4 raw2[kScanU];
#pragma unroll
  for (int u = 0; u < kScanU; ++u)
    if ((live >> u) & 1u) raw2[u] = ld_stream16(rows + u * slot_stride);
#pragma unroll
  for (int u = 0; u < kScanU; ++u) {
    if (!((live >> u) & 1u)) continue;
    const float lo = scan_dist8(qlo, *reinterpret_cast<const uint4*>(stage + u * (kThreads * 16)));
    float d = __fadd_rn(lo, scan_dist8(qhi, raw2[u]));               // lane distance 8
    d = __fadd_rn(d, __shfl_xor_sync(oct_mask, d, 4, 8));
    d = __fadd_rn(d, __shfl_xor_sync(oct_mask, d, 2, 8));
    d = __fadd_rn(d, __shfl_xor_sync(oct_mask, d, 1, 8));
    const int s = s_first + u * spar;
    const int pos = s + (s < tail ? off_lo : off_hi);
    if (better_pair(d, pos, bd, bp)) { bd = d; bp = pos; bs = s; }
  }
  ScanBest r;
  r.d = bd; r.p = bp; r.s = bs;
  return r;
}

__device__ void phase_match_scan(const DecodeParams& p, uint8_t* smem) {
  const MacB200DecodeArgs& a = p.a;
  const int tid = threadIdx.x;
  // control words used after the barriers
  if (blockIdx.x == 0) {
    if (tid < 9) a.task_counts[tid] = 0;
    if (tid == 9) *p.ar.ticket = gridDim.x;   // pieces 0 .. grid-1 go to their CTA without a ticket
  }
  for (int g = blockIdx.x * kThreads + tid; g < p.NG; g += gridDim.x * kThreads)
    p.ar.garrive[g] = 0;

  const int Hq = a.Hq, M = a.M, Tm = a.max_match_tiles;
  int p2 = 1;
  while (p2 < Hq && p2 < 32) p2 <<= 1;   // heads scanned side by side
  const int spar = 32 / p2;              // slots scanned side by side (only when Hq < 32)
  const int oct = tid >> 3, j = tid & 7;
  const int hslot = oct % p2, sub = oct / p2;
  const int oct_shift = ((tid & 31) >> 3) * 8;
  const unsigned oct_mask = 0xffu << oct_shift;
  const int nh = hslot < Hq ? (Hq - hslot + p2 - 1) / p2 : 0;          // heads of this octet
  const int nb = (a.match_tile_slots + kScanU * spar - 1) / (kScanU * spar);  // batches per tile
  const int total_tiles = a.N * Tm;
  const int my_tiles = static_cast<int>(blockIdx.x) < total_tiles
                           ? (total_tiles - static_cast<int>(blockIdx.x) +
                              static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)
                           : 0;
  const int round_tiles = kScanRoundTiles;
  const char* ring = static_cast<const char*>(a.query_cache);
  const char* qsrc = static_cast<const char*>(a.q_pre);
  const uint32_t lane_base = smem_u32(smem) + tid * 16;
  const uint8_t* lane_ptr = smem + tid * 16;
  const int64_t slot_stride = static_cast<int64_t>(Hq) * kRowBytes * spar;  // bytes between rows of a batch
  const float thr_probe = p.thr_dist * 1.0625f;   // see the probe's error bound below
  // partial (per sub) results of a round, only used when spar > 1
  float* part_d = reinterpret_cast<float*>(smem + kScanDepth * kScanStageBytes);
  int* part_p = reinterpret_cast<int*>(part_d + kScanRoundTiles * 32);
  int* part_s = part_p + kScanRoundTiles * 32;
  ScanTileInfo* tinfo = reinterpret_cast<ScanTileInfo*>(part_s + kScanRoundTiles * 32);

  for (int r0 = 0; r0 < my_tiles; r0 += round_tiles) {
    const int rt = min(round_tiles, my_tiles - r0);
    const int nseq = rt * nh * nb;
    if (tid < rt) {
      ScanCursor c;
      scan_load_tile(a, blockIdx.x + (r0 + tid) * gridDim.x, c);
      ScanTileInfo ti;
      ti.n = c.n; ti.tile = c.tile; ti.P = c.P; ti.req = c.req; ti.cbeg = c.cbeg; ti.cend = c.cend;
      ti.s_begin = c.s_begin; ti.s_end = c.s_end; ti.tail = c.tail; ti.off_lo = c.off_lo;
      ti.off_hi = c.off_hi; ti.elig = c.elig ? 1 : 0;
      tinfo[tid] = ti;
    }
    __syncthreads();
    ScanCursor ci, cc;   // issue side, consume side
    ci.k = ci.hi = ci.b = 0;
    scan_fetch_tile(tinfo, 0, ci);
    cc = ci;
    auto advance = [&](ScanCursor& c) {
      if (++c.b == nb) {
        c.b = 0;
        if (++c.hi == nh) {
          c.hi = 0;
          if (++c.k < rt) scan_fetch_tile(tinfo, c.k, c);
        }
      }
    };
    // first slot of the cursor's batch, address of its first row chunk for this lane
    auto batch_first_slot = [&](const ScanCursor& c) { return c.s_begin + sub + c.b * kScanU * spar; };
    auto row_ptr = [&](const ScanCursor& c, int s, int h) {
      return ring + ((static_cast<int64_t>(c.req) * M + s) * Hq + h) * kRowBytes + j * 16;
    };
    auto batch_all_valid = [&](const ScanCursor& c, int s_first) {
      const int s_last = s_first + (kScanU - 1) * spar;
      return s_last < c.s_end && ((s_first < c.tail) == (s_last < c.tail)) &&
             scan_slot_pos(c, s_first) >= c.cbeg && scan_slot_pos(c, s_last) < c.cend;
    };
    auto issue = [&](int seq) {
      if (ci.elig) {
        const int h = hslot + ci.hi * p2;
        const uint32_t dst = lane_base + (seq % kScanDepth) * kScanStageBytes;
        const int s_first = batch_first_slot(ci);
        const char* src = row_ptr(ci, s_first, h);
        bool any = false;
        if (__builtin_expect(batch_all_valid(ci, s_first), 1)) {
#pragma unroll
          for (int u = 0; u < kScanU; ++u)
            cp_async16(dst + u * (kThreads * 16), src + u * slot_stride, 16);
          any = true;
        } else {
#pragma unroll 1
          for (int u = 0; u < kScanU; ++u) {
            const int s = s_first + u * spar;
            const int pos = scan_slot_pos(ci, s);
            if (s < ci.s_end && pos >= ci.cbeg && pos < ci.cend) {
              cp_async16(dst + u * (kThreads * 16), src + u * slot_stride, 16);
              any = true;
            }
          }
        }
        if (any) {
          const char* q = qsrc + (static_cast<int64_t>(ci.n) * Hq + h) * kRowBytes + j * 16;
          cp_async16(dst + kScanU * (kThreads * 16), q, 16);
          cp_async16(dst + (kScanU + 1) * (kThreads * 16), q + 128, 16);
        }
      }
      advance(ci);
    };

#pragma unroll
    for (int s = 0; s < kScanDepth - 1; ++s) {
      if (s < nseq) issue(s);
      cp_async_commit();
    }
    float bd = INFINITY;
    int bp = INT_MAX, bs = -1;
    for (int seq = 0; seq < nseq; ++seq) {
      cp_async_wait<kScanDepth - 2>();
      if (cc.b == 0) { bd = INFINITY; bp = INT_MAX; bs = -1; }
      if (cc.elig) {
        const uint8_t* src = lane_ptr + (seq % kScanDepth) * kScanStageBytes;
        // Probe in packed bf16 arithmetic (two dims per instruction).  Each lane's
        // 8-dim sum carries a relative error below 6 * 2^-8 = 2.4 % (one rounding
        // of the difference, squared, plus four roundings of the running sum), so
        // comparing against the threshold widened by 1/16 can only let extra rows
        // through to the exact evaluation, never drop a row whose exact distance
        // is below the threshold.
        const uint4 qv = *reinterpret_cast<const uint4*>(src + kScanU * (kThreads * 16));
        float acc[kScanU];
#pragma unroll
        for (int u = 0; u < kScanU; ++u)
          acc[u] = scan_probe8(qv, *reinterpret_cast<const uint4*>(src + u * (kThreads * 16)));
        // halving exchange over the octet: lane j ends with the probe sum of row j
        const bool b2 = (j & 4) != 0, b1 = (j & 2) != 0, b0 = (j & 1) != 0;
        float w4[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float send = b2 ? acc[r] : acc[r + 4];
          const float keep = b2 ? acc[r + 4] : acc[r];
          w4[r] = __fadd_rn(keep, __shfl_xor_sync(oct_mask, send, 4, 8));
        }
        float w2[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float send = b1 ? w4[r] : w4[r + 2];
          const float keep = b1 ? w4[r + 2] : w4[r];
          w2[r] = __fadd_rn(keep, __shfl_xor_sync(oct_mask, send, 2, 8));
        }
        const float send0 = b0 ? w2[0] : w2[1];
        const float keep0 = b0 ? w2[1] : w2[0];
        const float probe = __fadd_rn(keep0, __shfl_xor_sync(oct_mask, send0, 1, 8));
        const int s_first = batch_first_slot(cc);
        const int s_mine = s_first + j * spar;
        const int pos_mine = scan_slot_pos(cc, s_mine);
        const bool survive = s_mine < cc.s_end && pos_mine >= cc.cbeg && pos_mine < cc.cend &&
                             probe < thr_probe;   // NaN probes drop out here as well
        const unsigned live = (__ballot_sync(oct_mask, survive) >> oct_shift) & 0xffu;
        if (__builtin_expect(live != 0u, 0)) {   // octet-uniform; rare unless the ring holds near rows
          const int h = hslot + cc.hi * p2;
          const ScanBest nb_ = scan_survivors(
              live, src, row_ptr(cc, s_first, h) + 128, slot_stride, oct_mask, s_first, spar,
              cc.tail, cc.off_lo, cc.off_hi, bd, bp, bs);
          bd = nb_.d; bp = nb_.p; bs = nb_.s;
        }
      }
      if (cc.b == nb - 1 && j == 0) {
        const int h = hslot + cc.hi * p2;
        if (spar == 1) {
          const int64_t off = (static_cast<int64_t>(cc.n) * Hq + h) * Tm + cc.tile;
          a.match_dist[off] = bd;
          a.match_pos[off] = bp;
          a.match_slot[off] = bs;
        } else {
          const int e = cc.k * 32 + h * spar + sub;
          part_d[e] = bd; part_p[e] = bp; part_s[e] = bs;
        }
      }
      advance(cc);
      const int nxt = seq + kScanDepth - 1;
      if (nxt < nseq) issue(nxt);
      cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();   // everyone is done with the tile descriptors of this pass
    if (spar > 1) {
      for (int t = tid; t < rt * Hq; t += kThreads) {
        const int k = t / Hq, h = t - k * Hq;
        float d0 = INFINITY;
        int p0 = INT_MAX, s0 = -1;
        for (int s = 0; s < spar; ++s) {
          const int e = k * 32 + h * spar + s;
          if (better_pair(part_d[e], part_p[e], d0, p0)) { d0 = part_d[e]; p0 = part_p[e]; s0 = part_s[e]; }
        }
        const int g = blockIdx.x + (r0 + k) * gridDim.x;
        const int tile = g / a.N, n = g - tile * a.N;
        const int64_t off = (static_cast<int64_t>(n) * Hq + h) * Tm + tile;
        a.match_dist[off] = d0;
        a.match_pos[off] = p0;
        a.match_slot[off] = s0;
      }
      __syncthreads();
    }
  }
}


// ------------------------------------------------- phase A, bulk-copy variant
// The same match scan with the ring rows brought in by the copy engine instead
// of by per-thread cp.async: the ring is viewed as a 2-D tensor [R*M*Hq rows,
// 128 bf16] and ONE elected thread issues a tiled bulk copy
// (cp.async.bulk.tensor.2d, completion on an mbarrier) of the probe columns of
// 256 consecutive rows -- one row per thread.  The rows of a (request, match
// tile) are consecutive in that view, so a tile is a handful of such boxes.
// The other 255 threads issue no address arithmetic and no copy instructions
// at all; each evaluates the probe of its own row straight from shared memory
// (swizzled by the copy engine, so the 256 row reads are bank-conflict free).
//
//  * Probe width kChunks * 16 bytes (64 B = dims 0..31, or 128 B = dims 0..63):
//    the partial distance over a prefix of the dims is a lower bound of the
//    full one whatever the prefix, and it is formed per 16-byte chunk in packed
//    bf16 exactly as in the cp.async variant (same error bound, same widened
//    threshold), the chunk sums added in fp32.
//  * A row that passes the probe is re-read whole from global memory by its
//    thread and its exact distance formed in the reference's order
//    (DEC.cu:1062-1069, 343-349): sixteen 8-dim sums of sequential FMAs, then
//    pairwise at chunk distance 8, 4, 2, 1.  The per-(tile, head) minimum with
//    the (distance, older position) order is kept by a 64-bit atomicMin in
//    shared memory on (distance bits << 32 | position): distances are
//    non-negative, so their bit patterns order like the values, NaNs order
//    above +inf and never win.
//  * Every wait on a copy is bounded (wall time); on expiry the CTA records
//    MAC_B200_STATUS_COPY_TIMEOUT, waits (bounded again) for the copies it still
//    has in flight and the kernel returns.
constexpr int kTmaBoxRows = 256;
constexpr unsigned long long kCopyWaitLimitNs = 2000000000ull;
constexpr unsigned long long kCopyDrainLimitNs = 50000000ull;
constexpr unsigned long long kNoMatchKey = (0x7f800000ull << 32) | 0x7fffffffull;   // (+inf, INT_MAX)

struct BoxTile {
  int n, tile, P, cbeg, cend, s_begin, nrows, tail, off_lo, off_hi, nbox, row0;
};
static_assert(sizeof(BoxTile) == 48, "three int4 loads");

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns_u64();
  unsigned polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 63u) == 0u && global_ns_u64() - t0 > limit_ns) return false;
  }
  return true;
}
__device__ __forceinline__ void bulk_tensor_load_2d(uint32_t dst, const CUtensorMap* map, int x,
                                                    int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, "
      "%3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Exact distance of one ring row (global memory) to one query row, reference
// summation order; updates the per-(tile, head) minimum.
__device__ __noinline__ void scan_exact_row(const char* row, const char* qrow, int pos,
                                            unsigned long long* best) {
  float sum[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    const uint4 rv = ld_stream16(row + c * 16);
    const uint4 qv = __ldg(reinterpret_cast<const uint4*>(qrow + c * 16));
    float qf[8];
    unpack8(qv, qf);
    sum[c] = scan_dist8(qf, rv);
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) sum[c] = __fadd_rn(sum[c], sum[c + 8]);
#pragma unroll
  for (int c = 0; c < 4; ++c) sum[c] = __fadd_rn(sum[c], sum[c + 4]);
  sum[0] = __fadd_rn(sum[0], sum[2]);
  sum[1] = __fadd_rn(sum[1], sum[3]);
  const float d = __fadd_rn(sum[0], sum[1]);
  const unsigned long long key =
      (static_cast<unsigned long long>(__float_as_uint(d)) << 32) | static_cast<unsigned>(pos);
  atomicMin(best, key);
}

template <int kChunks>
__device__ bool phase_match_scan_bulk(const DecodeParams& p, const CUtensorMap* ring_map,
                                      uint8_t* smem) {
  constexpr int kProbeBytes = kChunks * 16;
  constexpr int kBoxBytes = kTmaBoxRows * kProbeBytes;
  constexpr int kStagesB = kChunks == 4 ? 8 : 5;
  static_assert(kStagesB * kBoxBytes + 1024 + kScanRoundTiles * 48 <= kRingBytes, "scan stages must fit");
  static_assert(2 * kMaxHq * 8 <= kSmemPerm, "best-match words must fit");
  const MacB200DecodeArgs& a = p.a;
  const int tid = threadIdx.x;
  if (blockIdx.x == 0) {
    if (tid < 9) a.task_counts[tid] = 0;
    if (tid == 9) *p.ar.ticket = gridDim.x;   // pieces 0 .. grid-1 go to their CTA without a ticket
  }
  for (int g = blockIdx.x * kThreads + tid; g < p.NG; g += gridDim.x * kThreads)
    p.ar.garrive[g] = 0;

  const int Hq = a.Hq, M = a.M, Tm = a.max_match_tiles;
  const int total_tiles = a.N * Tm;
  const int my_tiles = static_cast<int>(blockIdx.x) < total_tiles
                           ? (total_tiles - static_cast<int>(blockIdx.x) +
                              static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)
                           : 0;
  const uint32_t base_u32 = smem_u32(smem);
  const uint32_t pad = (1024u - (base_u32 & 1023u)) & 1023u;
  uint8_t* stage0 = smem + pad;
  const uint32_t stage0_u32 = base_u32 + pad;
  BoxTile* tinfo = reinterpret_cast<BoxTile*>(stage0 + kStagesB * kBoxBytes);
  unsigned long long* best = reinterpret_cast<unsigned long long*>(smem + kRingBytes);  // [2][kMaxHq]
  const uint32_t bars_u32 = smem_u32(smem + kSmemBars);
  const float thr_probe = p.thr_dist * 1.0625f;   // see the probe's error bound in scan_probe8's user
  const bool fixed_head = (kTmaBoxRows % Hq) == 0;   // a thread then keeps one head for every box
  const char* ring = static_cast<const char*>(a.query_cache);
  const char* qsrc = static_cast<const char*>(a.q_pre);
  const int swz = kChunks == 4 ? ((tid >> 1) & 3) : (tid & 7);
  const uint8_t* my_row = stage0 + tid * kProbeBytes;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kStagesB; ++s) mbar_init(bars_u32 + s * 8, 1);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int i = tid; i < 2 * kMaxHq; i += kThreads) best[i] = kNoMatchKey;
  __syncthreads();

  unsigned seq_base = 0;   // boxes consumed in earlier rounds (stage and parity carry over)
  bool failed = false;
  for (int r0 = 0; r0 < my_tiles && !failed; r0 += kScanRoundTiles) {
    const int rt = min(kScanRoundTiles, my_tiles - r0);
    if (tid < rt) {
      ScanCursor c;
      scan_load_tile(a, blockIdx.x + (r0 + tid) * gridDim.x, c);
      BoxTile t;
      t.n = c.n; t.tile = c.tile; t.P = c.P; t.cbeg = c.cbeg; t.cend = c.cend;
      t.s_begin = c.s_begin; t.nrows = (c.s_end - c.s_begin) * Hq;
      t.tail = c.tail; t.off_lo = c.off_lo; t.off_hi = c.off_hi;
      t.row0 = (c.req * M + c.s_begin) * Hq;
      bool any = false;
      if (c.elig)
        for (int s = c.s_begin; s < c.s_end; ++s) {
          const int pos = scan_slot_pos(c, s);
          any = any || (pos >= c.cbeg && pos < c.cend);
        }
      t.nbox = any ? (t.nrows + kTmaBoxRows - 1) / kTmaBoxRows : 0;
      tinfo[tid] = t;
    }
    __syncthreads();
    int nact = 0;
    for (int k = 0; k < rt; ++k) nact += tinfo[k].nbox;
    // tiles without a candidate row report "no match" (the classifier reads every tile)
    for (int k = 0; k < rt; ++k) {
      if (tinfo[k].nbox != 0 || tid >= Hq) continue;
      const int64_t off = (static_cast<int64_t>(tinfo[k].n) * Hq + tid) * Tm + tinfo[k].tile;
      a.match_dist[off] = INFINITY;
      a.match_pos[off] = INT_MAX;
      a.match_slot[off] = -1;
    }
    // producer cursor (thread 0) and consumer cursor (every thread) over the active boxes
    int pk = 0, pb = -1, ck = 0, cb = -1;
    auto advance = [&](int& k, int& b) {
      ++b;
      while (k < rt && b >= tinfo[k].nbox) { ++k; b = 0; }
    };
    unsigned issued = 0;
    auto issue = [&](unsigned i) {   // thread 0: box pk/pb into stage (seq_base + i) % kStagesB
      const unsigned sq = seq_base + i;
      const uint32_t bar = bars_u32 + (sq % kStagesB) * 8;
      mbar_expect_tx(bar, kBoxBytes);
      bulk_tensor_load_2d(stage0_u32 + (sq % kStagesB) * kBoxBytes, ring_map, 0,
                          tinfo[pk].row0 + pb * kTmaBoxRows, bar);
    };
    if (tid == 0) {
      advance(pk, pb);
      while (issued < static_cast<unsigned>(min(kStagesB, nact))) {
        issue(issued);
        ++issued;
        advance(pk, pb);
      }
    }
    uint4 q[kChunks], qn[kChunks];   // this tile's query chunks, the next active tile's (in flight)
    bool have_qn = false;
    int my_h = 0;
    auto load_q = [&](int n, uint4 (&dst)[kChunks]) {
      const uint4* qp = reinterpret_cast<const uint4*>(
          qsrc + (static_cast<int64_t>(n) * Hq + my_h) * kRowBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) dst[c] = __ldg(qp + c);
    };
    int job = 0;   // active tiles seen so far in this pass (selects the best-match buffer)
    BoxTile t{};
    advance(ck, cb);
    for (int i = 0; i < nact; ++i) {
      const unsigned sq = seq_base + static_cast<unsigned>(i);
      if (cb == 0) {
        const int4* src = reinterpret_cast<const int4*>(tinfo + ck);
        const int4 w0 = src[0], w1 = src[1], w2 = src[2];
        t.n = w0.x; t.tile = w0.y; t.P = w0.z; t.cbeg = w0.w;
        t.cend = w1.x; t.s_begin = w1.y; t.nrows = w1.z; t.tail = w1.w;
        t.off_lo = w2.x; t.off_hi = w2.y; t.nbox = w2.z; t.row0 = w2.w;
        if (fixed_head) {
          my_h = tid % Hq;
          if (have_qn) {
#pragma unroll
            for (int c = 0; c < kChunks; ++c) q[c] = qn[c];
          } else {
            load_q(t.n, q);
          }
          int nk = ck + 1;   // the next tile's query is fetched a whole tile ahead
          while (nk < rt && tinfo[nk].nbox == 0) ++nk;
          have_qn = nk < rt;
          if (have_qn) load_q(tinfo[nk].n, qn);
        }
      }
      const int r_local = cb * kTmaBoxRows + tid;
      bool cand = false;
      int pos = 0, slot = 0;
      if (r_local < t.nrows) {
        const int so = r_local / Hq;
        slot = t.s_begin + so;
        if (!fixed_head) my_h = r_local - so * Hq;
        pos = slot + (slot < t.tail ? t.off_lo : t.off_hi);
        cand = pos >= t.cbeg && pos < t.cend;
      }
      if (!fixed_head && cand) load_q(t.n, q);
      const bool ok = mbar_wait_bounded(bars_u32 + (sq % kStagesB) * 8, (sq / kStagesB) & 1u,
                                        kCopyWaitLimitNs);
      if (ok && cand) {
        const uint8_t* rowp = my_row + (sq % kStagesB) * kBoxBytes;
        float probe = 0.0f;
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          probe += scan_probe8(q[c], *reinterpret_cast<const uint4*>(rowp + ((c ^ swz) << 4)));
        if (__builtin_expect(probe < thr_probe, 0)) {   // NaN probes drop out here as well
          scan_exact_row(ring + static_cast<int64_t>(t.row0 + r_local) * kRowBytes,
                         qsrc + (static_cast<int64_t>(t.n) * Hq + my_h) * kRowBytes, pos,
                         best + (job & 1) * kMaxHq + my_h);
        }
      }
      const bool last_box = cb == t.nbox - 1;
      if (__syncthreads_or(ok ? 0 : 1)) {   // some thread's wait ran out: give up as one CTA
        failed = true;
        if (tid == 0) {
          atomicOr(&g_status, MAC_B200_STATUS_COPY_TIMEOUT);
          for (unsigned j = static_cast<unsigned>(i) + 1; j < issued; ++j)   // copies still in flight
            mbar_wait_bounded(bars_u32 + ((seq_base + j) % kStagesB) * 8,
                              ((seq_base + j) / kStagesB) & 1u, kCopyDrainLimitNs);
        }
        __syncthreads();
        break;
      }
      if (tid == 0 && issued < static_cast<unsigned>(nact)) {   // the stage just read is free again
        issue(issued);
        ++issued;
        advance(pk, pb);
      }
      if (last_box) {
        if (tid < Hq) {
          unsigned long long* slotp = best + (job & 1) * kMaxHq + tid;
          const unsigned long long key = *slotp;
          *slotp = kNoMatchKey;
          const int64_t off = (static_cast<int64_t>(t.n) * Hq + tid) * Tm + t.tile;
          const int bpos = static_cast<int>(key & 0xffffffffull);
          a.match_dist[off] = __uint_as_float(static_cast<unsigned>(key >> 32));
          a.match_pos[off] = bpos;
          a.match_slot[off] = key == kNoMatchKey ? -1 : pos_to_ring_slot(t.P, M, bpos);
        }
        ++job;
      }
      advance(ck, cb);
    }
    seq_base += static_cast<unsigned>(nact);
    __syncthreads();   // everyone is done with the tile descriptors of this pass
  }
  return !failed;
}


// ---------------------------------------------------------------- phase B
// One warp per KV group: cross-tile argmin per head, hit test, synthetic
// override, front-sink demotion, group mode, reported arrays, and the group's
// plan for phase C.  Decision rules: DEC.cu:1142-1402.
__device__ void phase_classify(const DecodeParams& p) {
  const MacB200DecodeArgs& a = p.a;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = p.G, Hq = a.Hq, Hkv = a.Hkv, M = a.M, Tm = a.max_match_tiles;
  int gp2 = 1;
  while (gp2 < G) gp2 <<= 1;
  const int L = 32 / gp2;        // lanes cooperating on one head
  const int hl = lane / L;       // head index inside the group
  const int sub = lane % L;
  const int S = a.semantic_pos_ahead;

  for (int g = blockIdx.x * kWarps + warp; g < p.NG; g += gridDim.x * kWarps) {
    const int n = g / Hkv, hkv = g - n * Hkv;
    const int64_t go = static_cast<int64_t>(n) * Hkv + hkv;
    GroupPlan plan;
    if (request_bad(a, n)) {
      // Malformed row: zero output, no ring access, sticky status bit.
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.out);
      for (int i = lane; i < G * kD; i += 32)
        out[(static_cast<int64_t>(n) * Hq + hkv * G) * kD + i] = __float2bfloat16_rn(0.0f);
      if (lane < G) {
        const int64_t ho = static_cast<int64_t>(n) * Hq + hkv * G + lane;
        if (a.optional_lse) a.optional_lse[ho] = -INFINITY;
        a.head_hit[ho] = 0; a.head_match_slot[ho] = -1; a.head_match_pos[ho] = -1;
        a.head_prefix_end[ho] = 0; a.head_rect_start[ho] = 0; a.head_new_end[ho] = 0;
      }
      if (lane == 0) {
        atomicOr(&g_status, MAC_B200_STATUS_BAD_REQUEST);
        a.group_rect_begin[go] = 0; a.group_rect_end[go] = 0; a.group_rect_tiles[go] = 0;
        a.group_tail_begin[go] = 0; a.group_tail_end[go] = 0; a.group_tail_tiles[go] = 0;
        a.group_mode[go] = 1;
        plan.sink_hi = 0; plan.band_lo = 0; plan.new_end = 0; plan.kv_len = 0;
        plan.cls = 0; plan.cost = 0; plan.mode = 1; plan.req = -1;
        p.ar.plan[g] = plan;
      }
      continue;
    }
    const int P = a.past_lens[n], req = a.req_ids[n];
    int cbeg, cend;
    candidate_window(a, P, cbeg, cend);
    const bool ready = request_ready(a, req);
    const bool eligible = P >= a.gen_min_limit && cend > cbeg && ready;
    const int hq = hkv * G + hl;
    const bool head_lane = hl < G;

    float bd = INFINITY;
    int bp = INT_MAX, bs = -1;
    if (head_lane && eligible) {
      const int64_t base = (static_cast<int64_t>(n) * Hq + hq) * Tm;
      for (int t = sub; t < p.tm_used; t += L) {
        const float d = __ldcg(a.match_dist + base + t);
        const int pp = __ldcg(a.match_pos + base + t);
        const int ss = __ldcg(a.match_slot + base + t);
        if (better_pair(d, pp, bd, bp)) { bd = d; bp = pp; bs = ss; }
      }
    }
    for (int off = L >> 1; off > 0; off >>= 1) {
      const float od = __shfl_xor_sync(0xffffffffu, bd, off);
      const int op = __shfl_xor_sync(0xffffffffu, bp, off);
      const int os = __shfl_xor_sync(0xffffffffu, bs, off);
      if (better_pair(od, op, bd, bp)) { bd = od; bp = op; bs = os; }
    }
    bool hit = eligible && bs >= 0 && bd < p.thr_dist;

    if (a.bench_mode != 0 || a.bench_miss_mask >= 0) {
      // DEC.cu:1184-1269
      const uint32_t unit_id = (a.bench_mode == 2) ? static_cast<uint32_t>(hkv)
                                                   : static_cast<uint32_t>(hq);
      const uint32_t base_key = static_cast<uint32_t>(a.bench_seed) ^
                                (static_cast<uint32_t>(a.bench_layer_id) * 0x9e3779b9u) ^
                                (static_cast<uint32_t>(P) * 0x85ebca6bu);
      const uint32_t key = base_key ^ (static_cast<uint32_t>(n) * 0xc2b2ae35u) ^
                           (unit_id * 0x27d4eb2fu);
      if (a.bench_miss_mask >= 0) {
        const bool miss = hl >= 0 && hl < 30 && (((a.bench_miss_mask >> hl) & 1) != 0);
        hit = eligible && P > 0 && M > 0 && !miss;
      } else if (a.bench_exact_quota != 0 && a.bench_hit_rate_std == 0.0f) {
        const int total = (a.bench_mode == 2) ? a.N * Hkv : a.N * Hq;
        const int unit = (a.bench_mode == 2) ? n * Hkv + hkv : n * Hq + hq;
        const int miss_units = bench_target_miss_units(a, total);
        const int offset = total > 0 ? static_cast<int>(base_key % static_cast<uint32_t>(total)) : 0;
        int rotated = unit + offset;
        if (rotated >= total) rotated -= total;
        hit = eligible && P > 0 && M > 0 && !(rotated < miss_units);
      } else {
        const float rate = clampf(__fmaf_rn(a.bench_hit_rate_std,
                                            pseudo_normal_u32(key ^ 0x4cf5ad43u),
                                            a.bench_hit_rate), 0.0f, 1.0f);
        hit = eligible && P > 0 && M > 0 && uniform01_u32(key ^ 0x165667b1u) < rate;
      }
      if (hit) {
        const int max_lag = M < P ? M : P;
        const int new_end_tmp = cache_end_for_pos(P, S);
        float lag_f = __fmaf_rn(a.bench_match_lag_std, pseudo_normal_u32(key ^ 0xd3a2646cu),
                                a.bench_match_lag_mean);
        bool requested_skip = false;
        if (a.bench_skip_ratio >= 0.0f) {
          requested_skip = true;
          const float skip = clampf(__fmaf_rn(a.bench_skip_ratio_std,
                                              pseudo_normal_u32(key ^ 0xfd7046c5u),
                                              a.bench_skip_ratio), 0.0f, 0.999999f);
          int target = static_cast<int>(roundf(__fmul_rn(skip, static_cast<float>(P))));
          if (target > new_end_tmp - 1) target = new_end_tmp - 1;
          if (target < 0) target = 0;
          lag_f = static_cast<float>(new_end_tmp - target);
        }
        int lag = static_cast<int>(roundf(lag_f));
        if (lag < 1) lag = 1;
        if (requested_skip) {
          if (lag > P) lag = P;
        } else if (lag > max_lag) {
          lag = max_lag;
        }
        if (max_lag <= 0 || new_end_tmp <= 0) {
          hit = false; bp = INT_MAX; bs = -1;
        } else {
          bp = P - lag;
          if (bp < 0) bp = 0;
          bs = pos_to_ring_slot(P, M, bp);
          // benchmark extension: a synthetic match older than the ring's span stands in a
          // slot of its own (position mod M) instead of an out-of-range one
          if (a.bench_long_band != 0 && bp < P - M) bs = bp % M;
          bd = 0.0f;
        }
      } else {
        bp = INT_MAX; bs = -1; bd = INFINITY;
      }
    }

    int prefix_end = 0, rect_start = 0, mpos = -1, mslot = -1;
    if (hit) {
      mpos = bp; mslot = bs;
      prefix_end = cache_end_for_pos(mpos, S);
      rect_start = prefix_end;
    }
    if (hit && p.F > 0 && prefix_end < p.F) {  // DEC.cu:1285-1291
      hit = false; mpos = -1; mslot = -1; prefix_end = 0; rect_start = 0;
    }
    const int new_end = cache_end_for_pos(P, S);
    // reusable ("valid") head: DEC.cu:1323-1328
    bool valid = head_lane && hit && mslot >= 0;
    if (valid) {
      const float pl = a.lse_cache[(static_cast<int64_t>(req) * M + mslot) * Hq + hq];
      const int clen = new_end - rect_start;
      const bool any_lag = a.bench_long_band != 0 && a.bench_mode != 0;   // benchmark extension
      valid = isfinite(pl) && clen >= 0 && (clen <= M || any_lag);
    }
    const bool rep = head_lane && sub == 0;  // one representative lane per head
    const unsigned vmask = __ballot_sync(0xffffffffu, valid && rep);
    const int vcount = __popc(vmask);
    int mode = 1;
    if (vcount == G) mode = 0;
    else if (vcount > 0 && a.mixed_group_fallback != 0) mode = 2;
    int fs = p.F < new_end ? p.F : new_end;
    if (mode != 0 && !(mode == 2 && valid)) {
      hit = false; mslot = -1; mpos = -1; prefix_end = 0; rect_start = fs;
    }
    // group rows
    int sink_hi = fs < rect_start ? fs : rect_start;   // DEC.cu:725-731
    int my_lo = head_lane ? rect_start : INT_MAX;
    int my_sink = head_lane ? sink_hi : 0;
    for (int off = 16; off > 0; off >>= 1) {
      my_lo = min(my_lo, __shfl_xor_sync(0xffffffffu, my_lo, off));
      my_sink = max(my_sink, __shfl_xor_sync(0xffffffffu, my_sink, off));
    }
    int band_lo = my_lo;
    if (band_lo > new_end) band_lo = new_end;
    if (band_lo < 0) band_lo = 0;
    if (rep) {
      const int64_t ho = static_cast<int64_t>(n) * Hq + hq;
      a.head_hit[ho] = hit ? 1 : 0;
      a.head_match_slot[ho] = mslot;
      a.head_match_pos[ho] = mpos;
      a.head_prefix_end[ho] = prefix_end;
      a.head_rect_start[ho] = rect_start;
      a.head_new_end[ho] = new_end;
    }
    if (lane == 0) {
      const int kv_len = P + 1;
      const int tile = a.tile_tokens > 0 ? a.tile_tokens : 1;
      const int band_tok = new_end - band_lo;
      a.group_rect_begin[go] = band_lo;
      a.group_rect_end[go] = new_end;
      a.group_rect_tiles[go] = (band_tok + tile - 1) / tile;
      a.group_tail_begin[go] = new_end;
      a.group_tail_end[go] = kv_len;
      a.group_tail_tiles[go] = (kv_len - new_end + tile - 1) / tile;
      a.group_mode[go] = mode;
      if (mode != 0) atomicAdd(&a.task_counts[5], 1);
      if (mode == 1) atomicAdd(&a.task_counts[6], 1);
      if (mode != 0 && band_tok > tile) atomicAdd(&a.task_counts[3], 1);
      if (kv_len > new_end) atomicAdd(&a.task_counts[1], 1);
      plan.sink_hi = my_sink;
      plan.band_lo = band_lo;
      plan.new_end = new_end;
      plan.kv_len = kv_len;
      plan.mode = mode;
      plan.req = req;
      plan.cls = (mode == 0) ? 2 : (eligible ? 1 : 0);
      int cost = 0;
      if (my_sink > 0) cost += my_sink + p.ovh_tok;
      if (band_tok > 0) cost += band_tok + p.ovh_tok;
      if (kv_len > new_end) cost += kv_len - new_end + p.ovh_tok;
      plan.cost = cost;
      p.ar.plan[g] = plan;
    }
  }
}

// ---------------------------------------------------------------- phase C
struct Schedule {
  uint16_t* gperm;   // [NG] cost-space order -> group id
  uint32_t* cpre;    // [NG+1] exclusive prefix of group cost in cost-space order
  uint32_t W;        // total cost
  uint32_t ps;       // piece size
  uint32_t pieces;
};

// Block-wide exclusive scan of one 64-bit value per thread; returns the
// thread's prefix and the block total.  `warp_tot` is a [kWarps] smem scratch.
__device__ __forceinline__ unsigned long long block_scan_excl(unsigned long long v,
                                                              unsigned long long* warp_tot,
                                                              unsigned long long& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long o = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += o;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  unsigned long long base = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const unsigned long long t = warp_tot[w];
    if (w < warp) base += t;
    tot += t;
  }
  total = tot;
  return base + inc - v;
}

// Every CTA derives the same schedule from the group plans: order groups by
// queue (demoted, miss, hit), prefix-sum their cost, cut into pieces.
__device__ void build_schedule(const DecodeParams& p, Schedule& sc, unsigned long long* scan_sm,
                               uint32_t* tmp) {
  const int tid = threadIdx.x;
  const int NG = p.NG;
  // pass 1: one load per group (queue class and cost, kept in shared memory for the two
  // passes that follow) and the class totals
  unsigned long long totals = 0;
  for (int base = 0; base < NG; base += kThreads) {
    const int g = base + tid;
    unsigned long long v = 0;
    if (g < NG) {
      const int2 cc = __ldcg(reinterpret_cast<const int2*>(&p.ar.plan[g].cls));   // cls, cost
      tmp[g] = static_cast<uint32_t>(cc.y) | (static_cast<uint32_t>(cc.x) << 30);
      v = 1ull << (21 * cc.x);
    }
    unsigned long long t;
    block_scan_excl(v, scan_sm, t);
    totals += t;
  }
  const unsigned t0 = static_cast<unsigned>(totals & 0x1fffffull);
  const unsigned t1 = static_cast<unsigned>((totals >> 21) & 0x1fffffull);
  // pass 2: rank inside class -> permutation; costs move to cost-space order
  unsigned long long carry = 0;
  for (int base = 0; base < NG; base += kThreads) {
    const int g = base + tid;
    int cls = 0;
    uint32_t cost = 0;
    unsigned long long v = 0;
    if (g < NG) {
      cls = static_cast<int>(tmp[g] >> 30);
      cost = tmp[g] & 0x3fffffffu;
      v = 1ull << (21 * cls);
    }
    unsigned long long t;
    const unsigned long long ex = block_scan_excl(v, scan_sm, t) + carry;
    carry += t;
    if (g < NG) {
      const unsigned r = static_cast<unsigned>((ex >> (21 * cls)) & 0x1fffffull);
      const unsigned v_idx = (cls == 0) ? r : (cls == 1 ? t0 + r : t0 + t1 + r);
      sc.gperm[v_idx] = static_cast<uint16_t>(g);
      sc.cpre[v_idx] = cost;
    }
  }
  __syncthreads();
  // pass 3: cost prefix in cost-space order (in place)
  unsigned long long ccarry = 0;
  for (int base = 0; base < NG; base += kThreads) {
    const int v_idx = base + tid;
    unsigned long long c = 0;
    if (v_idx < NG) {
      c = static_cast<unsigned long long>(sc.cpre[v_idx]);
      // bits 40.. count the groups small enough to be finished in one fused pass
      if (c > 0 && c <= static_cast<unsigned long long>(p.fuse_max)) c |= 1ull << 40;
    }
    unsigned long long t;
    const unsigned long long ex = block_scan_excl(c, scan_sm, t) + ccarry;
    ccarry += t;
    if (v_idx < NG) sc.cpre[v_idx] = static_cast<uint32_t>(ex & 0xffffffffffull);
  }
  const unsigned n_small = static_cast<unsigned>(ccarry >> 40);
  ccarry &= 0xffffffffffull;
  if (tid == 0) sc.cpre[NG] = static_cast<uint32_t>(ccarry);
  __syncthreads();
  sc.W = static_cast<uint32_t>(ccarry);
  // Wave-quantised piece count: as many pieces as keep a piece above
  // kMinPieceTok; once there is a piece per CTA, exactly one per CTA.
  // ... but never fewer pieces than there are small groups (up to one per half such
  // piece): those are latency-bound and want a CTA each, whatever their cost adds up to.
  unsigned pieces = sc.W / static_cast<unsigned>(p.min_piece);
  unsigned small_pieces = 2u * sc.W / static_cast<unsigned>(p.min_piece);
  if (small_pieces > n_small) small_pieces = n_small;
  if (pieces < small_pieces) pieces = small_pieces;
  if (pieces < 1) pieces = 1;
  if (pieces > gridDim.x) {
    // One piece per CTA.  Interleaved A/B runs on B200 (1, 2 and 4 waves of pieces with
    // dynamic tickets) had one wave fastest in all but the very largest steps, where four
    // waves won by under 1 %: a second piece costs a CTA another row opening and another
    // set of partials to merge, which outweighs the better tail.  The override stays for
    // tuning.
    unsigned waves = 1u;
    if (p.force_waves > 0) waves = static_cast<unsigned>(p.force_waves);
    pieces = waves * gridDim.x;
  }
  if (pieces > static_cast<unsigned>(p.max_pieces)) pieces = p.max_pieces;
  sc.pieces = pieces;
  sc.ps = (sc.W + pieces - 1) / pieces;
  if (sc.ps < 1) sc.ps = 1;
}

struct RowGeom {
  int tok_begin;   // first logical position of the row
  int len;         // tokens
  uint32_t a;      // start of the row in cost space
  uint32_t c;      // cost of the row (0 if empty)
};

__device__ __forceinline__ void group_rows(const GroupPlan& pl, uint32_t a0, int ovh,
                                           RowGeom (&rows)[3]) {
  rows[0].tok_begin = 0;          rows[0].len = pl.sink_hi;
  rows[1].tok_begin = pl.band_lo; rows[1].len = pl.new_end - pl.band_lo;
  rows[2].tok_begin = pl.new_end; rows[2].len = pl.kv_len - pl.new_end;
  uint32_t a = a0;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    if (rows[r].len < 0) rows[r].len = 0;
    rows[r].a = a;
    rows[r].c = rows[r].len > 0 ? static_cast<uint32_t>(rows[r].len + ovh) : 0u;
    a += rows[r].c;
  }
}

// Token sub-range of a row that falls into cost interval [x0, x1).  The first
// kOvhTok cost units of a row stand for the fixed cost of opening it; cut
// points are rounded down to whole 16-token blocks so neighbours agree.
__device__ __forceinline__ void segment_tokens(const RowGeom& row, int ovh, uint32_t x0,
                                               uint32_t x1, int& lo, int& hi) {
  const uint32_t end = row.a + row.c;
  int l = 0, h = row.len;
  if (x0 > row.a) {
    const int rel = static_cast<int>(x0 - row.a) - ovh;
    l = rel > 0 ? (rel & ~(kBlkTok - 1)) : 0;
  }
  if (x1 < end) {
    const int rel = static_cast<int>(x1 - row.a) - ovh;
    h = rel > 0 ? (rel & ~(kBlkTok - 1)) : 0;
  }
  if (h > row.len) h = row.len;
  if (l > h) l = h;
  lo = row.tok_begin + l;
  hi = row.tok_begin + h;
}

__device__ __forceinline__ void row_piece_span(const RowGeom& row, uint32_t ps, int& p_lo,
                                               int& p_hi) {
  p_lo = static_cast<int>(row.a / ps);
  p_hi = static_cast<int>((row.a + row.c - 1) / ps);
}

// One warp's share of a token row: 16-token blocks first, first+stride, ... of
// logical positions [t0, t1).  row_kind: 0 sink, 1 band, 2 tail (decides each
// head's own sub-range inside [t0, t1)).
struct WarpWork {
  int t0, t1, row_kind, first, stride;
};

// Streams the warp's blocks of request n through KV head hkv for the G query
// heads of the group: per-warp cp.async K/V ring, mma.sync contraction, online
// softmax.  Leaves the warp's un-normalised accumulators (rows = heads), running
// max (log2 domain) and denominator (already summed over the quad).
__device__ __forceinline__ void warp_stream(const DecodeParams& p, uint8_t* smem, int n, int hkv,
                                            int req, int P, const WarpWork& w,
                                            float (&oacc)[16][4], float& m_run, float& l_run) {
  const MacB200DecodeArgs& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.G;
  const int hrow = lane >> 2, quad = lane & 3;
  const bool has_head = hrow < G;
  const int hq = hkv * G + (has_head ? hrow : 0);
  const int t0 = w.t0, t1 = w.t1;

  // this head's own range inside the row
  int lo = t0, hi = t1;
  if (has_head) {
    const int rs = __ldcg(a.head_rect_start + static_cast<int64_t>(n) * a.Hq + hq);
    if (w.row_kind == 1) {
      lo = max(t0, rs);
    } else if (w.row_kind == 0) {
      const int ne = cache_end_for_pos(P, a.semantic_pos_ahead);
      int sh = p.F < ne ? p.F : ne;
      if (sh > rs) sh = rs;
      hi = min(t1, sh);
    }
  } else {
    hi = lo;  // padded rows see nothing
  }

  // Q fragments: rows = heads of the group, 8 K-steps of 16 dims
  uint32_t qa0[8], qa2[8];
  {
    const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
        static_cast<const char*>(a.q_post) + (static_cast<int64_t>(n) * a.Hq + hq) * kRowBytes);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa0[kk] = has_head ? __ldg(qrow + kk * 8 + quad) : 0u;
      qa2[kk] = has_head ? __ldg(qrow + kk * 8 + 4 + quad) : 0u;
    }
  }

#pragma unroll
  for (int j = 0; j < 16; ++j) { oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.0f; }
  m_run = -INFINITY;
  l_run = 0.0f;

  const int nblk = (t1 - t0 + kBlkTok - 1) / kBlkTok;
  const int mine = (w.stride > 0 && w.first < nblk) ? (nblk - w.first + w.stride - 1) / w.stride : 0;
  uint8_t* ring = smem + warp * kWarpRingBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const char* kbase = static_cast<const char*>(a.k_buffer) + static_cast<int64_t>(hkv) * kRowBytes;
  const char* vbase = static_cast<const char*>(a.v_buffer) + static_cast<int64_t>(hkv) * kRowBytes;
  const int64_t tok_stride = static_cast<int64_t>(a.Hkv) * kRowBytes;
  const int32_t* table = a.req_to_token + static_cast<int64_t>(req) * a.req_to_token_stride;

  // pool row of the lane's token (lanes 0..15) of this warp's j-th block; -1 = past the end
  // (Page-table entries are followed as they are, like in the reference: a bounds check here
  // was measured at 0.6-1.2 % of the whole step, a check inside issue_block at 16 %.)
  // (pool rows travel as 32-bit values -- the launcher refuses pools of 2^31 rows or more --
  // so that handing a row to the other lanes is one shuffle; every instruction of the
  // copy-issue loop below is worth 0.2-0.5 % of a full-attention step)
  auto load_token = [&](int j) -> int {
    const int pos = t0 + (w.first + j * w.stride) * kBlkTok + (lane & 15);
    if (pos >= t1) return 0;   // never copied (see issue_block); any valid row will do
    if (pos == P) {
      return a.out_cache_loc_is_i64
                 ? static_cast<int>(static_cast<const int64_t*>(a.out_cache_loc)[n])
                 : static_cast<const int32_t*>(a.out_cache_loc)[n];
    }
    return __ldg(table + pos);
  };
  const char* kb_lane = kbase + (lane & 15) * 16;
  const char* vb_lane = vbase + (lane & 15) * 16;
  const uint32_t stride32 = static_cast<uint32_t>(tok_stride);
  auto issue_block = [&](int j, int tok_reg) {
    const uint32_t st = ring_u32 + (j % kStages) * kStageBytes;
    const int chunk = lane & 15;
    // rows of this block that lie inside [t0, t1): all 16 except in the last block of a row
    const int nvalid = t1 - (t0 + (w.first + j * w.stride) * kBlkTok);
    if (nvalid >= kBlkTok) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = (lane >> 4) + 2 * i;
        const uint32_t tok = static_cast<uint32_t>(__shfl_sync(0xffffffffu, tok_reg, r));
        const uint64_t off = static_cast<uint64_t>(tok) * stride32;
        const uint32_t dst = st + r * kRowBytes + ((chunk ^ (r & 7)) << 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(kb_lane + off) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + kBlkTok * kRowBytes), "l"(vb_lane + off) : "memory");
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = (lane >> 4) + 2 * i;
        const uint32_t tok = static_cast<uint32_t>(__shfl_sync(0xffffffffu, tok_reg, r));
        const int bytes = r < nvalid ? 16 : 0;   // rows past the end are zero-filled
        const uint64_t off = static_cast<uint64_t>(tok) * stride32;
        const uint32_t dst = st + r * kRowBytes + ((chunk ^ (r & 7)) << 4);
        cp_async16(dst, kb_lane + off, bytes);
        cp_async16(dst + kBlkTok * kRowBytes, vb_lane + off, bytes);
      }
    }
  };

  int tok_next = -1;
#pragma unroll
  for (int j = 0; j < kStages - 1; ++j) {
    if (j < mine) issue_block(j, load_token(j));
    cp_async_commit();
  }
  if (kStages - 1 < mine) tok_next = load_token(kStages - 1);

  for (int j = 0; j < mine; ++j) {
    cp_async_wait<kStages - 2>();
    __syncwarp();
    const uint32_t kst = ring_u32 + (j % kStages) * kStageBytes;
    const uint32_t vst = kst + kBlkTok * kRowBytes;
    const int tb = t0 + (w.first + j * w.stride) * kBlkTok;

    // S = Q K^T for 16 tokens: two n-blocks of 8 tokens
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int mi = lane >> 3;
      const int r = ((mi >> 1) << 3) + (lane & 7);
      const uint32_t row_addr = kst + r * kRowBytes;
      const int rx = r & 7;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const int chunk = 2 * kk + (mi & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(row_addr + ((chunk ^ rx) << 4), b0, b1, b2, b3);
        mma_bf16_rows8(s0, qa0[kk], qa2[kk], b0, b1);
        mma_bf16_rows8(s1, qa0[kk], qa2[kk], b2, b3);
      }
    }
    // online softmax in the log2 domain
    const int pos0 = tb + quad * 2;
    float sv[4];
    sv[0] = (pos0 >= lo && pos0 < hi) ? s0[0] * p.scale_log2 : -INFINITY;
    sv[1] = (pos0 + 1 >= lo && pos0 + 1 < hi) ? s0[1] * p.scale_log2 : -INFINITY;
    sv[2] = (pos0 + 8 >= lo && pos0 + 8 < hi) ? s1[0] * p.scale_log2 : -INFINITY;
    sv[3] = (pos0 + 9 >= lo && pos0 + 9 < hi) ? s1[1] * p.scale_log2 : -INFINITY;
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
    const float alpha = ex2(m_run - m_use);
    const float p0 = ex2(sv[0] - m_use), p1 = ex2(sv[1] - m_use);
    const float p2 = ex2(sv[2] - m_use), p3 = ex2(sv[3] - m_use);
    l_run = l_run * alpha + ((p0 + p1) + (p2 + p3));
    m_run = m_new;
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) { oacc[jj][0] *= alpha; oacc[jj][1] *= alpha; }
    const uint32_t pa0 = pack_bf16x2(p0, p1);
    const uint32_t pa2 = pack_bf16x2(p2, p3);
    // O += P V
    {
      const int mi = lane >> 3;
      const int r = ((mi & 1) << 3) + (lane & 7);
      const uint32_t row_addr = vst + r * kRowBytes;
      const int rx = r & 7;
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int chunk = 2 * jj + (mi >> 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(row_addr + ((chunk ^ rx) << 4), b0, b1, b2, b3);
        mma_bf16_rows8(oacc[2 * jj], pa0, pa2, b0, b1);
        mma_bf16_rows8(oacc[2 * jj + 1], pa0, pa2, b2, b3);
      }
    }
    __syncwarp();
    const int jn = j + kStages - 1;
    if (jn < mine) issue_block(jn, tok_next);
    cp_async_commit();
    if (jn + 1 < mine) tok_next = load_token(jn + 1);
  }
  cp_async_wait<0>();
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
}

// Cross-warp combine buffer in shared memory (aliases the idle K/V ring).
struct CombineBuf {
  float* o;   // [kWarps][8][kCombineRow]
  float* m;   // [kWarps][8]
  float* l;   // [kWarps][8]
};
__device__ __forceinline__ CombineBuf combine_buf(uint8_t* smem) {
  CombineBuf c;
  c.o = reinterpret_cast<float*>(smem);
  c.m = c.o + kWarps * 8 * kCombineRow;
  c.l = c.m + kWarps * 8;
  return c;
}
// Every warp publishes its accumulators; returns after the CTA-wide barrier.
__device__ __forceinline__ void combine_publish(uint8_t* smem, const float (&oacc)[16][4],
                                                float m_run, float l_run) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hrow = lane >> 2, quad = lane & 3;
  __syncthreads();  // every warp is done with its K/V ring
  const CombineBuf cb = combine_buf(smem);
  float* dst = cb.o + (warp * 8 + hrow) * kCombineRow + quad * 2;
#pragma unroll
  for (int jj = 0; jj < 16; ++jj)
    *reinterpret_cast<float2*>(dst + jj * 8) = make_float2(oacc[jj][0], oacc[jj][1]);
  if (quad == 0) {
    cb.m[warp * 8 + hrow] = m_run;
    cb.l[warp * 8 + hrow] = l_run;
  }
  __syncthreads();
}
// Head h's normalised partial over warps [w_lo, w_hi): lane owns dims [4*lane, 4*lane+4);
// lse is the natural-log LSE, -inf when the warps saw no token of the head.
__device__ __forceinline__ void combine_reduce(uint8_t* smem, int h, int w_lo, int w_hi,
                                               float4& acc, float& lse) {
  const int lane = threadIdx.x & 31;
  const CombineBuf cb = combine_buf(smem);
  float mx = -INFINITY;
  for (int w = w_lo; w < w_hi; ++w) mx = fmaxf(mx, cb.m[w * 8 + h]);
  float lsum = 0.0f;
  acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (mx != -INFINITY) {
    for (int w = w_lo; w < w_hi; ++w) {
      const float wgt = ex2(cb.m[w * 8 + h] - mx);
      lsum += cb.l[w * 8 + h] * wgt;
      const float4 o = *reinterpret_cast<const float4*>(cb.o + (w * 8 + h) * kCombineRow + lane * 4);
      acc.x += o.x * wgt; acc.y += o.y * wgt; acc.z += o.z * wgt; acc.w += o.w * wgt;
    }
  }
  lse = -INFINITY;
  if (lsum > 0.0f) {
    const float inv = 1.0f / lsum;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    lse = (mx + lg2(lsum)) * kLn2;
  } else {
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// One segment by the whole CTA: warp w takes blocks w, w+8, ...; the normalised
// partial (o, natural-log LSE) of every head goes to arena slot `slot`.
__device__ void attend_segment(const DecodeParams& p, uint8_t* smem, int n, int hkv, int req, int P,
                               int t0, int t1, int row_kind, int slot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float oacc[16][4];
  float m_run, l_run;
  const WarpWork w{t0, t1, row_kind, warp, kWarps};
  warp_stream(p, smem, n, hkv, req, P, w, oacc, m_run, l_run);
  combine_publish(smem, oacc, m_run, l_run);
  if (warp < p.G) {
    float4 acc;
    float lse;
    combine_reduce(smem, warp, 0, kWarps, acc, lse);
    float* po = p.ar.part_o + (static_cast<int64_t>(slot) * p.G + warp) * kD + lane * 4;
    __stcg(reinterpret_cast<float4*>(po), acc);
    if (lane == 0) __stcg(p.ar.part_lse + static_cast<int64_t>(slot) * 8 + warp, lse);
  }
  __syncthreads();  // combine buffer is free again
}

// LSE merge of (o, lse) with another partial; natural log (DEC.cu:866-890).
__device__ __forceinline__ void merge_state(float4& o, float& lse, const float4& o2, float lse2) {
  if (!isfinite(lse2)) return;
  if (!isfinite(lse)) {
    o = o2;
    lse = lse2;
    return;
  }
  const float m = fmaxf(lse, lse2);
  const float es = expf(lse - m), eo = expf(lse2 - m);
  const float den = es + eo;
  const float ws = es / den, wo = eo / den;
  o.x = ws * o.x + wo * o2.x; o.y = ws * o.y + wo * o2.y;
  o.z = ws * o.z + wo * o2.z; o.w = ws * o.w + wo * o2.w;
  lse = m + logf(den);
}

// Reused prefix state of head hq (warp-wide; lane owns 4 dims): the matched
// ring row if the head is a hit with a finite LSE, else empty (DEC.cu:4346-4365).
__device__ __forceinline__ void load_prefix_state(const MacB200DecodeArgs& a, int n, int hq,
                                                  int req, float4& o, float& lse) {
  const int lane = threadIdx.x & 31;
  const int64_t ho = static_cast<int64_t>(n) * a.Hq + hq;
  o = make_float4(0.f, 0.f, 0.f, 0.f);
  lse = -INFINITY;
  const int hit = __ldcg(a.head_hit + ho);
  const int mslot = __ldcg(a.head_match_slot + ho);
  if (hit != 0 && mslot >= 0) {
    const int64_t row = (static_cast<int64_t>(req) * a.M + mslot) * a.Hq + hq;
    const float pl_lse = a.lse_cache[row];
    if (isfinite(pl_lse)) {
      const uint2 raw = *reinterpret_cast<const uint2*>(
          static_cast<const char*>(a.attn_cache) + row * kRowBytes + lane * 8);
      o = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
      lse = pl_lse;
    }
  }
}

// Ring row P mod M of this step (query, state, LSE); only for requests whose
// cache passes the readiness gate (DEC.cu:4485-4497).
__device__ __forceinline__ void write_ring_row(const MacB200DecodeArgs& a, int n, int hq, int req,
                                               int P, const float4& o, float lse) {
  const int lane = threadIdx.x & 31;
  if (!request_ready(a, req)) return;
  const int64_t ho = static_cast<int64_t>(n) * a.Hq + hq;
  const int dest = P % a.M;
  const int64_t row = (static_cast<int64_t>(req) * a.M + dest) * a.Hq + hq;
  const bool ok = isfinite(lse);
  const uint2 qv = *reinterpret_cast<const uint2*>(static_cast<const char*>(a.q_pre) +
                                                   ho * kRowBytes + lane * 8);
  *reinterpret_cast<uint2*>(static_cast<char*>(a.query_cache) + row * kRowBytes + lane * 8) = qv;
  uint2 ov = make_uint2(0u, 0u);
  if (ok) {
    ov.x = pack_bf16x2(o.x, o.y);
    ov.y = pack_bf16x2(o.z, o.w);
  }
  *reinterpret_cast<uint2*>(static_cast<char*>(a.attn_cache) + row * kRowBytes + lane * 8) = ov;
  if (lane == 0) a.lse_cache[row] = ok ? lse : -INFINITY;
}

__device__ __forceinline__ void write_output(const MacB200DecodeArgs& a, int n, int hq,
                                             const float4& o, float lse) {
  const int lane = threadIdx.x & 31;
  const int64_t ho = static_cast<int64_t>(n) * a.Hq + hq;
  const bool ok = isfinite(lse);
  uint2 ov = make_uint2(0u, 0u);
  if (ok) {
    ov.x = pack_bf16x2(o.x, o.y);
    ov.y = pack_bf16x2(o.z, o.w);
  }
  *reinterpret_cast<uint2*>(static_cast<char*>(a.out) + ho * kRowBytes + lane * 8) = ov;
  if (lane == 0 && a.optional_lse) a.optional_lse[ho] = ok ? lse : -INFINITY;
}

// Runs in the CTA that retired the group's last segment (all 256 threads): prefix
// state (+) band partials -> ring row; (+) sink (+) tail partials -> output.  Warp h < G
// owns head h, lane owns 4 dims.  Order of operations: DEC.cu:4346-4365, 4485-4520.
//
// A row that spans several pieces left one partial per piece in the arena.  A long
// context on a small batch spans dozens; loading them one after the other (each load
// an L2 round trip) was a tail of tens of microseconds.  So the partial rows of up to
// kMergeChunk pieces at a time are copied into the idle K/V ring in shared memory by
// the whole CTA (cp.async, double-buffered: as many loads in flight as there are rows), and each head's
// warp then accumulates them from shared memory with softmax weights taken from all of
// the row's LSEs at once.
constexpr int kMergeChunk = 32;
constexpr int kMergeStagedMin = 6;   // rows with fewer partials are merged by direct loads
static_assert(2 * kMergeChunk * 4 * kRowBytes * 2 <= kRingBytes &&
                  2 * (kMergeChunk / 2) * 8 * kRowBytes * 2 <= kRingBytes,
              "two merge staging buffers must fit the ring");

__device__ void merge_group(const DecodeParams& p, uint8_t* smem, const Schedule& sc, int v_idx,
                            int g, const GroupPlan& pl) {
  const MacB200DecodeArgs& a = p.a;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.G;
  const bool active = warp < G;
  const int n = g / a.Hkv, hkv = g - n * a.Hkv;
  const int hq = hkv * G + (active ? warp : 0);
  RowGeom rows[3];
  group_rows(pl, sc.cpre[v_idx], p.ovh_tok, rows);

  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  float lse = -INFINITY;
  if (active) load_prefix_state(a, n, hq, pl.req, o, lse);
  const uint32_t stage_u32 = smem_u32(smem);
  auto merge_row = [&](int r) {     // control flow is uniform over the CTA
    if (rows[r].c == 0) return;
    int p_lo, p_hi;
    row_piece_span(rows[r], sc.ps, p_lo, p_hi);
    const int np = p_hi - p_lo + 1;
    const int64_t slot0 = static_cast<int64_t>(p_lo) + 3 * v_idx + r;
    if (np < kMergeStagedMin) {   // a few partials: straight loads, no barrier
      if (active) {
        for (int b = 0; b < np; ++b) {
          const float l2 = __ldcg(p.ar.part_lse + (slot0 + b) * 8 + warp);
          if (!isfinite(l2)) continue;
          const float4 o2 = __ldcg(reinterpret_cast<const float4*>(
              p.ar.part_o + ((slot0 + b) * G + warp) * kD + lane * 4));
          merge_state(o, lse, o2, l2);
        }
      }
      return;
    }
    float mx = -INFINITY;
    if (active) {
      for (int b = lane; b < np; b += 32) {
        const float l2 = __ldcg(p.ar.part_lse + (slot0 + b) * 8 + warp);
        if (isfinite(l2)) mx = fmaxf(mx, l2);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    const int units_per_piece = G * (kRowBytes * 2 / 16);   // 16-byte units of one piece's G fp32 rows
    // two staging buffers of `chunk` pieces each (64 KB apiece): the next chunk is in
    // flight while this one is accumulated
    const int chunk = G <= 4 ? kMergeChunk : kMergeChunk / 2;
    const uint32_t buf_bytes = static_cast<uint32_t>(chunk) * units_per_piece * 16;
    auto stage = [&](int base, int which) {
      const int cnt = min(chunk, np - base);
      const char* src = reinterpret_cast<const char*>(p.ar.part_o + (slot0 + base) * G * kD);
      for (int u = tid; u < cnt * units_per_piece; u += kThreads)
        cp_async16(stage_u32 + which * buf_bytes + u * 16, src + static_cast<size_t>(u) * 16, 16);
      cp_async_commit();
    };
    stage(0, 0);
    int which = 0;
    for (int base = 0; base < np; base += chunk, which ^= 1) {
      const int cnt = min(chunk, np - base);
      const bool more = base + chunk < np;
      if (more) stage(base + chunk, which ^ 1);
      float w_mine = 0.f;
      if (active && lane < cnt && mx != -INFINITY) {
        const float l2 = __ldcg(p.ar.part_lse + (slot0 + base + lane) * 8 + warp);
        if (isfinite(l2)) w_mine = expf(l2 - mx);
      }
      den += w_mine;
      if (more) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncthreads();
      if (active) {
        const float4* rowp =
            reinterpret_cast<const float4*>(smem + which * buf_bytes) + warp * 32 + lane;
        for (int j = 0; j < cnt; ++j) {
          const float w = __shfl_sync(0xffffffffu, w_mine, j);
          if (w != 0.f) {   // warp-uniform
            const float4 v = rowp[j * G * 32];
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
          }
        }
      }
      __syncthreads();   // this buffer is refilled two chunks from now
    }
    if (active && mx != -INFINITY) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) den += __shfl_xor_sync(0xffffffffu, den, off);
      const float inv = 1.0f / den;   // den >= 1: the piece that holds the maximum has weight 1
      merge_state(o, lse, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv),
                  mx + logf(den));
    }
  };
  merge_row(1);
  if (active) write_ring_row(a, n, hq, pl.req, pl.kv_len - 1, o, lse);
  merge_row(0);
  merge_row(2);
  if (active) write_output(a, n, hq, o, lse);
}

// A group whose three rows all fall inside one piece is finished by this CTA
// alone in a single pass: the 8 warps are split over the rows in proportion to
// their 16-token blocks, all rows stream at once, and after one shared-memory
// combine warp h merges head h in registers (prefix (+) band -> ring row;
// (+) sink (+) tail -> output).  No arena traffic, no arrival counter.
__device__ void attend_group_fused(const DecodeParams& p, uint8_t* smem, int n, int hkv,
                                   const GroupPlan& pl) {
  const MacB200DecodeArgs& a = p.a;
  const int warp = threadIdx.x >> 5;
  const int G = p.G;
  const int begin[3] = {0, pl.band_lo, pl.new_end};
  const int end[3] = {pl.sink_hi, pl.new_end, pl.kv_len};
  int nblk[3], nw[3] = {0, 0, 0};
  int left = kWarps;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const int len = end[r] - begin[r];
    nblk[r] = len > 0 ? (len + kBlkTok - 1) / kBlkTok : 0;
    if (nblk[r] > 0) { nw[r] = 1; --left; }
  }
  while (left > 0) {  // next warp goes to the row with the most blocks per warp
    int best = -1;
    float load = 0.0f;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      if (nw[r] == 0) continue;
      const float l = static_cast<float>(nblk[r]) / static_cast<float>(nw[r]);
      if (l > load) { load = l; best = r; }
    }
    if (best < 0 || load <= 1.0f) break;
    ++nw[best];
    --left;
  }
  const int base[3] = {0, nw[0], nw[0] + nw[1]};
  WarpWork w{0, 0, 2, 0, 0};
#pragma unroll
  for (int r = 0; r < 3; ++r)
    if (warp >= base[r] && warp < base[r] + nw[r]) w = WarpWork{begin[r], end[r], r, warp - base[r], nw[r]};

  // the reused prefix state is fetched up front so its latency hides behind the stream
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  float lse = -INFINITY;
  const int hq = hkv * G + (warp < G ? warp : 0);
  if (warp < G) load_prefix_state(a, n, hq, pl.req, o, lse);

  float oacc[16][4];
  float m_run, l_run;
  warp_stream(p, smem, n, hkv, pl.req, pl.kv_len - 1, w, oacc, m_run, l_run);
  combine_publish(smem, oacc, m_run, l_run);
  if (warp < G) {
    float4 o2;
    float l2;
    if (nw[1] > 0) { combine_reduce(smem, warp, base[1], base[1] + nw[1], o2, l2); merge_state(o, lse, o2, l2); }
    write_ring_row(a, n, hq, pl.req, pl.kv_len - 1, o, lse);
    if (nw[0] > 0) { combine_reduce(smem, warp, base[0], base[0] + nw[0], o2, l2); merge_state(o, lse, o2, l2); }
    if (nw[2] > 0) { combine_reduce(smem, warp, base[2], base[2] + nw[2], o2, l2); merge_state(o, lse, o2, l2); }
    write_output(a, n, hq, o, lse);
  }
  __syncthreads();  // combine buffer is free again
}

__device__ void phase_attend(const DecodeParams& p, uint8_t* smem) {
  __shared__ unsigned long long scan_sm[kWarps];
  __shared__ int sh_piece;
  __shared__ int sh_last;
  Schedule sc;
  sc.gperm = reinterpret_cast<uint16_t*>(smem + kRingBytes);
  sc.cpre = reinterpret_cast<uint32_t*>(smem + kRingBytes + kSmemPerm);
  build_schedule(p, sc, scan_sm, reinterpret_cast<uint32_t*>(smem));   // the idle K/V ring is the scratch
  const int tid = threadIdx.x;
  const int NG = p.NG;
  if (blockIdx.x == 0 && tid == 0) {
    p.a.task_counts[4] = static_cast<int32_t>(sc.ps);
    p.a.task_counts[0] = static_cast<int32_t>(sc.pieces);
  }
  if (sc.W == 0) return;

  // CTA b takes piece b; further pieces (only with more than one wave of pieces) by ticket.
  for (bool first = true;; first = false) {
    int piece = static_cast<int>(blockIdx.x);
    if (!first) {
      __syncthreads();
      if (tid == 0) sh_piece = static_cast<int>(atomicAdd(p.ar.ticket, 1u));
      __syncthreads();
      piece = sh_piece;
    }
    if (piece >= static_cast<int>(sc.pieces)) break;
    const uint32_t x0 = static_cast<uint32_t>(piece) * sc.ps;
    uint32_t x1 = x0 + sc.ps;
    if (x1 > sc.W) x1 = sc.W;
    if (x0 >= x1) continue;
    // first group whose cost range ends after x0
    int lo = 0, hi = NG;  // find smallest v with cpre[v+1] > x0
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (sc.cpre[mid + 1] > x0) hi = mid; else lo = mid + 1;
    }
    for (int v = lo; v < NG && sc.cpre[v] < x1; ++v) {
      if (sc.cpre[v + 1] == sc.cpre[v]) continue;  // empty group (malformed row)
      const int g = sc.gperm[v];
      GroupPlan pl;
      {
        const int4* src = reinterpret_cast<const int4*>(&p.ar.plan[g]);
        const int4 w0 = __ldcg(src), w1 = __ldcg(src + 1);
        pl.sink_hi = w0.x; pl.band_lo = w0.y; pl.new_end = w0.z; pl.kv_len = w0.w;
        pl.cls = w1.x; pl.cost = w1.y; pl.mode = w1.z; pl.req = w1.w;
      }
      const int n = g / p.a.Hkv, hkv = g - n * p.a.Hkv;
      // A small group is never split: it belongs to the piece that holds its
      // first cost unit and is finished there in one fused pass.
      const uint32_t gcost = sc.cpre[v + 1] - sc.cpre[v];
      if (gcost <= static_cast<uint32_t>(p.fuse_max) && gcost <= 2u * sc.ps) {
        if (sc.cpre[v] >= x0) attend_group_fused(p, smem, n, hkv, pl);
        continue;
      }
      RowGeom rows[3];
      group_rows(pl, sc.cpre[v], p.ovh_tok, rows);
      int expected = 0, done_here = 0;
#pragma unroll 1
      for (int r = 0; r < 3; ++r) {
        if (rows[r].c == 0) continue;
        int p_lo, p_hi;
        row_piece_span(rows[r], sc.ps, p_lo, p_hi);
        expected += p_hi - p_lo + 1;
        if (piece < p_lo || piece > p_hi) continue;
        int t0, t1;
        segment_tokens(rows[r], p.ovh_tok, x0, x1, t0, t1);
        const int slot = piece + 3 * v + r;
        if (slot < p.ar.slots) {
          attend_segment(p, smem, n, hkv, pl.req, pl.kv_len - 1, t0, t1, r, slot);
        } else if (tid == 0) {
          atomicOr(&g_status, MAC_B200_STATUS_SCHED_OVERFLOW);
        }
        done_here += 1;
      }
      if (done_here == 0) continue;
      // publish partials, then count this CTA's segments against the group
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int prev = atomicAdd(&p.ar.garrive[g], done_here);
        sh_last = (prev + done_here == expected) ? 1 : 0;
      }
      __syncthreads();
      if (sh_last) {
        __threadfence();
        merge_group(p, smem, sc, v, g, pl);
      }
    }
  }
}

// ------------------------------------------------------------------- kernel
__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// The three phases; returns early when a bounded wait ran out.  kBulkScan selects the match
// scan at compile time: the two variants are separate kernels, because merely carrying the
// bulk-copy scan in the same kernel cost the cp.async variant 2-13 us per step on B200
// (measured with interleaved runs of both builds; the code is never executed there).
template <bool kBulkScan>
__device__ __forceinline__ void decode_phases(const DecodeParams& p, const CUtensorMap* ring_map,
                                              uint8_t* smem) {
  const bool stamp = p.a.debug_enabled >= 2 && blockIdx.x == 0 && threadIdx.x == 0;
  if (stamp) p.a.phase_cycles[0] = global_ns();
  if constexpr (kBulkScan) {
    if (p.scan_mode == 1) {
      if (!phase_match_scan_bulk<4>(p, ring_map, smem)) return;
    } else {
      if (!phase_match_scan_bulk<8>(p, ring_map, smem)) return;
    }
  } else {
    phase_match_scan(p, smem);
  }
  if (!grid_barrier(gridDim.x)) return;
  if (stamp) p.a.phase_cycles[1] = global_ns();
  phase_classify(p);
  if (!grid_barrier(gridDim.x)) return;
  if (stamp) p.a.phase_cycles[2] = global_ns();
  phase_attend(p, smem);
  if (stamp) {
    const long long t = global_ns();
    for (int i = 3; i < p.a.phase_cycles_count; ++i) p.a.phase_cycles[i] = t;
  }
}

__global__ void __launch_bounds__(kThreads, 1)
mac_decode_persistent_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  decode_phases<false>(p, nullptr, smem);
}

// The same step with the bulk-copy match scan (MAC_B200_SCAN=bulk64 / bulk128).
__global__ void __launch_bounds__(kThreads, 1)
mac_decode_persistent_bulk_scan_kernel(const DecodeParams p,
                                       const __grid_constant__ CUtensorMap ring_map) {
  extern __shared__ __align__(128) uint8_t smem[];
  decode_phases<true>(p, &ring_map, smem);
}

// --------------------------------------------------------------- host state
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int ctas_per_sm = 0;
  int regs = 0;
  int last_grid = 0;
  void* arena = nullptr;
  size_t arena_bytes = 0;
};
std::mutex g_mu;
DeviceState g_dev[64];

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tuning override of the number of piece waves, read at every launch (0 = automatic).
int piece_waves_override() {
  const char* e = std::getenv("MAC_B200_PIECE_WAVES");
  if (!e) return 0;
  const int v = std::atoi(e);
  return (v == 1 || v == 2 || v == 4) ? v : 0;
}

// Tuning overrides read at every launch.
int env_int_or(const char* name, int dflt, int lo, int hi) {
  const char* e = std::getenv(name);
  if (!e) return dflt;
  const int v = std::atoi(e);
  return (v >= lo && v <= hi) ? v : dflt;
}

// Cost of opening a row in token equivalents; MAC_B200_OVH_TOK overrides it for tuning.
// Measured on B200 (one piece per CTA): 256 is the flat optimum for G <= 4 (128 and 192 are
// 10-30 % slower, 384 is 1-3 % slower), 384 for G = 8 (256 is 3-9 % slower there: a
// fused small group moves twice the heads).
int row_overhead_tokens(int G) {
  const int dflt = G <= 4 ? kOvhTok : kOvhTok + 32 * (G - 4);
  const char* e = std::getenv("MAC_B200_OVH_TOK");
  if (!e) return dflt;
  const int v = std::atoi(e);
  return (v >= 16 && v <= 4096) ? (v & ~15) : dflt;
}

struct ArenaLayout {
  size_t ticket, garrive, plan, part_lse, part_o, total;
  int slots;
};
ArenaLayout arena_layout(int NG, int G, int max_pieces) {
  ArenaLayout L;
  L.slots = max_pieces + 3 * NG;
  size_t off = 0;
  L.ticket = off; off = align_up(off + 64, 256);
  L.garrive = off; off = align_up(off + sizeof(int32_t) * NG, 256);
  L.plan = off; off = align_up(off + sizeof(GroupPlan) * NG, 256);
  L.part_lse = off; off = align_up(off + sizeof(float) * 8 * L.slots, 256);
  L.part_o = off; off = align_up(off + sizeof(float) * static_cast<size_t>(L.slots) * G * kD, 256);
  L.total = off;
  return L;
}

// Checks shared by the decode entry points: the shape rules of the reference
// launcher (mac_decode_persistent.cu:5080-5153) and this build's limits.
// Returns MAC_B200_OK with *empty = true for an empty batch.
int validate_decode_args(const MacB200DecodeArgs& a, bool* empty) {
  *empty = false;
  MAC_REQUIRE(a.D == kD, "persistent decode supports D=128 only");
  MAC_REQUIRE(a.Hkv > 0 && a.Hq > 0 && a.Hq % a.Hkv == 0, "Hq must be divisible by Hkv");
  const int G = a.Hq / a.Hkv;
  MAC_REQUIRE(G > 0 && G <= 8, "unsupported GQA group size");
  MAC_REQUIRE(a.N >= 0, "negative batch");
  MAC_REQUIRE(a.M > 0 && a.R > 0, "ring tensors must not be empty");
  MAC_REQUIRE(a.match_tile_slots > 0, "match_tile_slots must be positive");
  MAC_REQUIRE(a.max_match_tiles >= (a.M + a.match_tile_slots - 1) / a.match_tile_slots,
              "match workspace too small");
  MAC_REQUIRE(a.ws_batch >= a.N, "decision workspaces are smaller than the batch");
  MAC_REQUIRE(a.bench_mode == 0 || a.bench_mode == 1 || a.bench_mode == 2,
              "unsupported synthetic MAC bench mode");
  MAC_REQUIRE(a.phase_cycles_count >= 6 && a.phase_cycles,
              "phase_cycles must have at least 6 elements");
  MAC_REQUIRE(a.q_post && a.q_pre && a.k_buffer && a.v_buffer && a.req_to_token && a.req_ids &&
                  a.past_lens && a.out_cache_loc && a.query_cache && a.attn_cache && a.lse_cache &&
                  a.out,
              "input/output tensors must not be null");
  MAC_REQUIRE(a.match_dist && a.match_pos && a.match_slot && a.head_hit && a.head_match_slot &&
                  a.head_match_pos && a.head_prefix_end && a.head_rect_start && a.head_new_end &&
                  a.group_rect_begin && a.group_rect_end && a.group_rect_tiles &&
                  a.group_tail_begin && a.group_tail_end && a.group_tail_tiles && a.group_mode &&
                  a.task_counts,
              "workspace tensors must not be null");
  if (a.N == 0) {
    *empty = true;
    return MAC_B200_OK;
  }
  if (a.Hq > kMaxHq)
    return fail(MAC_B200_EUNSUPPORTED, "Hq=%d exceeds this build's limit of %d", a.Hq, kMaxHq);
  const long long NGll = static_cast<long long>(a.N) * a.Hkv;
  if (NGll > kMaxGroups)
    return fail(MAC_B200_EUNSUPPORTED, "N*Hkv=%lld exceeds this build's limit of %d", NGll,
                kMaxGroups);
  if (a.kv_tokens >= (int64_t(1) << 31))
    return fail(MAC_B200_EUNSUPPORTED, "KV pool of %lld rows exceeds this build's limit of 2^31 - 1",
                static_cast<long long>(a.kv_tokens));
  return MAC_B200_OK;
}

// Kernel parameters of a validated step on a grid of `grid` CTAs whose scratch
// block starts at `arena` and is laid out for `max_pieces` pieces.
DecodeParams make_decode_params(const MacB200DecodeArgs& a, void* arena, int max_pieces) {
  DecodeParams p;
  p.a = a;
  p.G = a.Hq / a.Hkv;
  p.NG = a.N * a.Hkv;
  p.F = a.front_sink_tokens > 0 ? a.front_sink_tokens : 0;
  p.tm_used = (a.M + a.match_tile_slots - 1) / a.match_tile_slots;
  p.max_pieces = max_pieces;
  p.force_waves = piece_waves_override();
  p.ovh_tok = row_overhead_tokens(p.G);
  p.min_piece = env_int_or("MAC_B200_MIN_PIECE", kMinPieceTok, 64, 1 << 20);
  p.fuse_max = env_int_or("MAC_B200_FUSE_MAX", static_cast<int>(kFuseMaxCost), 0, 1 << 24);
  {
    float t = 2.0f * static_cast<float>(a.D);   // mac_decode_persistent.cu:5342, in float
    t = t * (1.0f - a.threshold);
    t = t * (1.0f - a.threshold);
    p.thr_dist = t;
  }
  p.scale_log2 = a.sm_scale * kLog2e;
  p.scan_mode = 0;   // set by launch_decode once the ring's tensor map exists
  const ArenaLayout L = arena_layout(p.NG, p.G, max_pieces);
  char* base = static_cast<char*>(arena);
  p.ar.ticket = reinterpret_cast<uint32_t*>(base + L.ticket);
  p.ar.garrive = reinterpret_cast<int32_t*>(base + L.garrive);
  p.ar.plan = reinterpret_cast<GroupPlan*>(base + L.plan);
  p.ar.part_lse = reinterpret_cast<float*>(base + L.part_lse);
  p.ar.part_o = reinterpret_cast<float*>(base + L.part_o);
  p.ar.slots = L.slots;
  return p;
}

// One-time facts of the decode kernel on a device (the device is current).
int query_kernel_facts(int device, int* sm_count, int* ctas_per_sm, int* regs) {
  int coop = 0;
  MAC_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device));
  if (!coop) return fail(MAC_B200_EUNSUPPORTED, "device does not support cooperative launch");
  MAC_CUDA(cudaFuncSetAttribute(mac_decode_persistent_kernel,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  MAC_CUDA(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device));
  MAC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(ctas_per_sm, mac_decode_persistent_kernel,
                                                         kThreads, kSmemBytes));
  if (*ctas_per_sm < 1) return fail(MAC_B200_ECUDA, "decode kernel has zero occupancy");
  cudaFuncAttributes fa{};
  MAC_CUDA(cudaFuncGetAttributes(&fa, mac_decode_persistent_kernel));
  *regs = fa.numRegs;
  return MAC_B200_OK;
}

// Decode launches of one device share its barrier words and scratch, so two of
// them must never run at the same time.  Launches on one stream are ordered by
// the stream; a launch on ANOTHER stream while the previous one has not
// finished is refused instead of being left to race.  (Not checked while a
// stream is being captured: a graph's launches run when it is replayed.)
struct InFlight {
  cudaEvent_t done = nullptr;
  cudaStream_t stream = nullptr;
  bool recorded = false;
};
std::mutex g_inflight_mu;
InFlight g_inflight[64];

// Tensor map of the query ring for the bulk-copy scan: rows = (request, slot,
// head), 128 bf16 each; one box = the probe columns of 256 consecutive rows,
// swizzled so that 256 threads can each read their own row without bank
// conflicts.  cuTensorMapEncodeTiled is a host-side computation; it is looked
// up through the runtime so the library does not link against the driver.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Scan variant.  MAC_B200_SCAN picks one for A/B runs:
//   cpasync            per-thread cp.async staging, 128 B probe, eight lanes per row (0; default)
//   bulk64 / bulk128   bulk tensor copies into shared memory, 64 B / 128 B probe (1 / 2)
// Measured on B200: DRAM delivers whole 128-byte lines whatever part of a ring row is asked
// for (ncu: the same dram__bytes_read for the 64 B and the 128 B probe), so the narrower
// probe saves no traffic; the variants land within a few percent of each other at batch 64
// and cpasync wins at small batches (no mbarrier set-up, no barrier per box).
int scan_mode_wanted() {
  const char* e = std::getenv("MAC_B200_SCAN");
  if (!e) return 0;
  if (!std::strcmp(e, "bulk64")) return 1;
  if (!std::strcmp(e, "bulk128")) return 2;
  return 0;
}

// Returns the scan mode that can run and fills `map` for the bulk-copy modes: they need a
// 16-byte aligned ring, row indices that fit 31 bits and the driver's tensor-map encoder.
// Otherwise: cp.async staging.
int make_ring_map(const MacB200DecodeArgs& a, CUtensorMap* map) {
  std::memset(map, 0, sizeof(*map));
  const int mode = scan_mode_wanted();
  if (mode == 0) return 0;
  const unsigned long long rows = static_cast<unsigned long long>(a.R) * a.M * a.Hq;
  if ((reinterpret_cast<uintptr_t>(a.query_cache) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(a.q_pre) & 15u) != 0 || rows >= (1ull << 31))
    return 0;
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return 0;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(kRowBytes)};
  const cuuint32_t box[2] = {mode == 1 ? 32u : 64u, static_cast<cuuint32_t>(kTmaBoxRows)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.query_cache, dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          mode == 1 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? mode : 0;
}

int launch_decode(int device, const DecodeParams& p, int grid, cudaStream_t stream) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  MAC_CUDA(cudaStreamIsCapturing(stream, &cs));
  const bool capturing = cs != cudaStreamCaptureStatusNone;
  std::lock_guard<std::mutex> lock(g_inflight_mu);
  InFlight& f = g_inflight[device];
  if (!capturing && f.recorded && f.stream != stream) {
    const cudaError_t q = cudaEventQuery(f.done);
    if (q == cudaErrorNotReady)
      return fail(MAC_B200_EINVAL,
                  "a decode step is still running on another stream of this device; decode "
                  "launches share per-device scratch and must not overlap (order them with an "
                  "event or use one stream)");
    if (q != cudaSuccess) return cuda_fail(q, "cudaEventQuery");
  }
  DecodeParams params = p;
  alignas(64) CUtensorMap ring_map;
  params.scan_mode = make_ring_map(p.a, &ring_map);
  if (params.scan_mode != 0) {
    static std::once_flag bulk_attr[64];
    cudaError_t attr_rc = cudaSuccess;
    std::call_once(bulk_attr[device], [&] {   // per device; this kernel shares the default one's shape
      attr_rc = cudaFuncSetAttribute(mac_decode_persistent_bulk_scan_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    });
    if (attr_rc != cudaSuccess) return cuda_fail(attr_rc, "cudaFuncSetAttribute");
    void* kargs[] = {&params, &ring_map};
    MAC_CUDA(cudaLaunchCooperativeKernel(
        reinterpret_cast<void*>(mac_decode_persistent_bulk_scan_kernel), dim3(grid), dim3(kThreads),
        kargs, kSmemBytes, stream));
  } else {
    void* kargs[] = {&params};
    MAC_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(mac_decode_persistent_kernel),
                                         dim3(grid), dim3(kThreads), kargs, kSmemBytes, stream));
  }
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  if (!capturing) {
    if (f.done == nullptr) MAC_CUDA(cudaEventCreateWithFlags(&f.done, cudaEventDisableTiming));
    MAC_CUDA(cudaEventRecord(f.done, stream));
    f.stream = stream;
    f.recorded = true;
  }
  return MAC_B200_OK;
}

}  // namespace
}  // namespace mac_b200

using namespace mac_b200;

extern "C" int mac_b200_persistent_decode_bf16(const MacB200DecodeArgs* args, void* stream_v) {
  MAC_REQUIRE(args != nullptr, "decode args must not be null");
  const MacB200DecodeArgs& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  bool empty = false;
  if (const int rc = validate_decode_args(a, &empty)) return rc;
  if (empty) return MAC_B200_OK;
  const int G = a.Hq / a.Hkv;
  const int NG = a.N * a.Hkv;

  int device = 0;
  MAC_CUDA(cudaGetDevice(&device));
  MAC_REQUIRE(device >= 0 && device < 64, "device index out of range");
  DeviceState st;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState& ds = g_dev[device];
    if (!ds.ready) {
      if (const int rc = query_kernel_facts(device, &ds.sm_count, &ds.ctas_per_sm, &ds.regs))
        return rc;
      ds.ready = true;
    }
    int grid = ds.sm_count * ds.ctas_per_sm;
    if (a.grid_cap > 0 && a.grid_cap < grid) grid = a.grid_cap;
    const int max_pieces = kMaxWaves * grid;
    const ArenaLayout L = arena_layout(NG, G, max_pieces);
    if (L.total > ds.arena_bytes) {
      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
      MAC_CUDA(cudaStreamIsCapturing(stream, &cs));
      if (cs != cudaStreamCaptureStatusNone)
        return fail(MAC_B200_ECAPTURE,
                    "scratch arena must grow to %zu bytes but the stream is being captured; "
                    "run one eager call with this shape first", L.total);
      // Launches still in flight may be using the old arena.
      MAC_CUDA(cudaDeviceSynchronize());
      if (ds.arena) MAC_CUDA(cudaFree(ds.arena));
      ds.arena = nullptr;
      ds.arena_bytes = 0;
      const size_t want = align_up(L.total + L.total / 4, 1 << 20);
      MAC_CUDA(cudaMalloc(&ds.arena, want));
      ds.arena_bytes = want;
    }
    ds.last_grid = grid;
    st = ds;
  }
  const DecodeParams p = make_decode_params(a, st.arena, kMaxWaves * st.last_grid);
  return launch_decode(device, p, st.last_grid, stream);
}

// ---------------------------------------------------------------------------
// Decode entry point that never allocates.
//
// Some hosts of this library must not create or free device memory: a serving
// process that hands all of HBM to its own pool allocator up front, a plugin
// that runs under a sandbox which filters the driver's allocation calls, or a
// caller that is already inside a region where allocation is illegal.  For
// them the split-KV partials and scheduler words live in one fixed block of
// device memory that is part of the library image itself.
namespace mac_b200 {
namespace {

constexpr size_t kNoAllocArenaBytes = size_t(8) << 20;  // 8 MiB, resident on every GPU that loads the library
static __device__ __align__(256) unsigned char g_noalloc_arena[kNoAllocArenaBytes];

struct NoAllocDeviceState {
  bool ready = false;
  int sm_count = 0;
  int ctas_per_sm = 0;
  void* arena = nullptr;  // device address of g_noalloc_arena on this device
};
std::mutex g_noalloc_mu;
NoAllocDeviceState g_noalloc_dev[64];

}  // namespace
}  // namespace mac_b200

extern "C" int mac_b200_persistent_decode_bf16_noalloc(const MacB200DecodeArgs* args,
                                                       void* stream_v) {
  MAC_REQUIRE(args != nullptr, "decode args must not be null");
  const MacB200DecodeArgs& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  bool empty = false;
  if (const int rc = validate_decode_args(a, &empty)) return rc;
  if (empty) return MAC_B200_OK;
  const int G = a.Hq / a.Hkv;
  const long long NGll = static_cast<long long>(a.N) * a.Hkv;

  int device = 0;
  MAC_CUDA(cudaGetDevice(&device));
  MAC_REQUIRE(device >= 0 && device < 64, "device index out of range");
  NoAllocDeviceState st;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDeviceState& ds = g_noalloc_dev[device];
    if (!ds.ready) {
      // One-time set-up for this device (it is the current one): kernel
      // attributes, occupancy, and the device address of the fixed block.  In
      // host code the array's name is only a handle for the runtime; the
      // address a kernel can use comes from cudaGetSymbolAddress.
      int regs = 0;
      if (const int rc = query_kernel_facts(device, &ds.sm_count, &ds.ctas_per_sm, &regs)) return rc;
      void* sym = nullptr;
      MAC_CUDA(cudaGetSymbolAddress(&sym, g_noalloc_arena));
      if (sym == nullptr) return fail(MAC_B200_ECUDA, "fixed scratch block has no device address");
      ds.arena = sym;
      ds.ready = true;
    }
    st = ds;
  }
  int grid = st.sm_count * st.ctas_per_sm;
  if (a.grid_cap > 0 && a.grid_cap < grid) grid = a.grid_cap;
  // the fixed block is sized for two pieces per CTA (the kernel clamps a tuning override to it)
  const int max_pieces = 2 * grid;
  const ArenaLayout L = arena_layout(static_cast<int>(NGll), G, max_pieces);
  if (L.total > kNoAllocArenaBytes)
    return fail(MAC_B200_ESIZE,
                "this step needs %zu bytes of scratch (N*Hkv=%lld groups, %d query heads per "
                "group) but the fixed block holds %zu; use mac_b200_persistent_decode_bf16 or a "
                "smaller batch",
                L.total, NGll, G, kNoAllocArenaBytes);
  // The block keeps whatever the previous call left in it.  The words that
  // must start at zero (piece ticket, per-group arrival counters) are cleared
  // by the kernel's first phase before any CTA reads them; everything else is
  // written before it is read within one launch.
  const DecodeParams p = make_decode_params(a, st.arena, max_pieces);
  return launch_decode(device, p, grid, stream);
}

extern "C" int mac_b200_query_status(uint32_t* status_out, void* stream_v) {
  MAC_REQUIRE(status_out != nullptr, "status_out must not be null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  MAC_CUDA(cudaStreamSynchronize(stream));
  unsigned v = 0;
  MAC_CUDA(cudaMemcpyFromSymbol(&v, g_status, sizeof(v)));
  unsigned build_bits = 0;
  if (const int rc = take_prefill_build_status(&build_bits)) return rc;
  *status_out = v | build_bits;
  if (v != 0) {
    const unsigned zero = 0;
    MAC_CUDA(cudaDeviceSynchronize());
    MAC_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(zero)));
    if (v & MAC_B200_STATUS_BARRIER_TIMEOUT) {
      MAC_CUDA(cudaMemcpyToSymbol(g_bar_count, &zero, sizeof(zero)));
    }
  }
  return MAC_B200_OK;
}

extern "C" int mac_b200_selftest_bounded_wait(uint32_t* status_out, int32_t* ctas_gave_up,
                                              void* stream_v) {
  MAC_REQUIRE(status_out != nullptr && ctas_gave_up != nullptr, "outputs must not be null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int* d_count = nullptr;
  MAC_CUDA(cudaMalloc(&d_count, sizeof(int)));
  MAC_CUDA(cudaMemsetAsync(d_count, 0, sizeof(int), stream));
  bounded_wait_selftest_kernel<<<2, 32, 0, stream>>>(d_count);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  MAC_CUDA(cudaStreamSynchronize(stream));
  int gave_up = 0;
  MAC_CUDA(cudaMemcpy(&gave_up, d_count, sizeof(int), cudaMemcpyDeviceToHost));
  MAC_CUDA(cudaFree(d_count));
  *ctas_gave_up = gave_up;
  const unsigned zero = 0;
  MAC_CUDA(cudaMemcpyToSymbol(g_selftest_count, &zero, sizeof(zero)));
  return mac_b200_query_status(status_out, stream_v);
}

extern "C" int mac_b200_launch_info(MacB200LaunchInfo* info) {
  MAC_REQUIRE(info != nullptr, "info must not be null");
  int device = 0;
  MAC_CUDA(cudaGetDevice(&device));
  MAC_REQUIRE(device >= 0 && device < 64, "device index out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  const DeviceState& ds = g_dev[device];
  info->sm_count = ds.sm_count;
  info->ctas_per_sm = ds.ctas_per_sm;
  info->block_threads = kThreads;
  info->dynamic_smem_bytes = kSmemBytes;
  info->regs_per_thread = ds.regs;
  info->last_grid = ds.last_grid;
  info->arena_bytes = static_cast<int64_t>(ds.arena_bytes);
  info->kernel_launches = g_kernel_launches.load(std::memory_order_relaxed);
  return MAC_B200_OK;
}
