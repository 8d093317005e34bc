// Sink-exclusive prefill ring build on the fifth-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory, operands staged by TMA).
//
// Same operator and same arithmetic as prefill_sink_exclusive_ring_kernel in
// mac_b200_prefill_build.cu (which stays as the fallback): a ring row must
// cover [min(F, E), E); the prefill producers give the state of [0, pos] and of
// the trailing window [E, pos]; what is left to remove is the row's attention
// over the sink tokens [0, F), computed here, inside the pass that streams the
// row through both downdates into the ring.  No counterpart in the reference,
// which stamps such rows unmatchable instead
// (attention/src/mac_attention/integrations/sglang/flashinfer_hooks.py:2205-2215).
//
// Why a second implementation: the products of a tile leave the warps altogether (one thread
// issues them, the copy engine stages every operand and every row), which takes a fifth of the
// instruction stream away; what is left -- softmax, row factors, element-wise combine -- is
// inherent to the rows.
//
// CTA = (slice of a request's ring rows, one KV head), 256 threads, one CTA per SM.  The sink K
// (key-major) and V (transposed: dim-major) of the (request, KV head) are staged once per CTA
// in the 128-byte-swizzled operand layout.  The CTA works through 128-row tiles (128/G tokens x
// the G query heads of the KV head); two threads share a row, each taking 64 of its columns
// (both reach the row's tensor-memory lane: warps w and w + 4 address the same lanes):
//   1. the tile's q_post, full and band rows arrive by bulk tensor copies (3-D boxes of 64 dims
//      x G heads x 128/G tokens, 128-byte swizzle, completion on mbarriers): q_post two tiles
//      ahead into a two-stage operand buffer, full / band one tile ahead; the rows that come
//      through registers (q_pre) are pulled into L2 two tiles ahead;
//   2. S = Q K^T was issued while the previous tile was being finished (eight
//      tcgen05.mma 128x128x16 products into one of two score stages in tensor memory);
//   3. every thread reads its 64 score columns with tcgen05.ld, the two halves of a row exchange
//      their maxima through shared memory, and the bf16 weights go over the dead q_post rows as
//      the next operand (64 keys = one operand atom per thread half);
//   4. one thread issues O = P V and, right after, the next tile's S = Q K^T; meanwhile the
//      q_pre rows are stored to the ring and the two threads of a row exchange the sums of their
//      weights and each fold both downdates into the row's three factors
//      (state = full*A - band*B - sink*C);
//   5. every thread reads its 64 columns of O and combines them with its half of the staged full
//      and band rows IN PLACE (the staged rows lie in the operand layout: a thread's 16-byte
//      chunks are swizzled with its row, so row-per-thread access is free of bank conflicts and
//      no transposition through shared memory is needed);
//   6. the finished rows go to the ring in whole 256-byte rows, and the next tile's full / band
//      rows are requested.
// Every wait on a copy or a product is bounded by wall time; on expiry the CTA records
// MAC_B200_STATUS_COPY_TIMEOUT, leaves its tile loop at the next common point, frees its
// tensor memory and returns.
#include <cuda.h>

#include <cstdlib>

#include "mac_b200_common.h"
#include "mac_b200_state_math.cuh"

namespace mac_b200 {
namespace {

constexpr int kTcRowBytes = 256;                 // D = 128 bf16
constexpr int kTcTileRows = 128;                 // MMA M
constexpr int kTcMaxF = 128;                     // MMA N of the first product
constexpr int kTcThreads = 256;                  // two threads per row: each takes 64 columns
constexpr int kTcAtomBytes = 128 * 128;          // 128 rows x 64 bf16, swizzled: one operand atom
constexpr int kTcOperandBytes = 2 * kTcAtomBytes;
constexpr int kTcSmemK = 0;
constexpr int kTcSmemVt = kTcSmemK + kTcOperandBytes;
constexpr int kTcSmemQ = kTcSmemVt + kTcOperandBytes;               // two stages of q_post rows / weights
constexpr int kTcSmemFull = kTcSmemQ + 2 * kTcOperandBytes;         // full rows, then the finished rows
constexpr int kTcSmemBand = kTcSmemFull + kTcOperandBytes;
constexpr int kTcSmemXch = kTcSmemBand + kTcOperandBytes;           // float2 per row
constexpr int kTcSmemBars = kTcSmemXch + kTcTileRows * 8;
constexpr int kTcSmemBytes = kTcSmemBars + 128 + 1024;   // + room to align the base to 1024 bytes
constexpr int kTcTmemCols = 512;                 // two stages of S (128 columns each) and O (128)
constexpr unsigned long long kTcWaitLimitNs = 2000000000ull;

// instruction descriptor of both products: bf16 x bf16 -> fp32, both operands K-major, M 128, N 128
constexpr uint32_t kTcIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ unsigned g_tc_status = 0;

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long tc_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// false when the limit ran out
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  if (tc_mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = tc_now_ns();
  for (unsigned spins = 1;; ++spins) {
    if (tc_mbar_try_wait(bar, parity)) return true;   // each try may itself block for a while
    if ((spins & 63u) == 0u && tc_now_ns() - t0 > kTcWaitLimitNs) return false;
  }
}
__device__ __forceinline__ void tc_fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_operand_desc(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(2) << 61);
}
// D[tmem] (+)= A[smem] * B[smem]^T, 128 x 128 x 16, issued by one thread
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kTcIdesc), "r"(accumulate), "r"(0u), "r"(0u),
      "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// 32 consecutive fp32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// the same without the wait: several loads can be in flight before one tc_ld_wait()
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float tc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tc_tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                               int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, "
      "%4}], [%5];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

// Softmax of one thread's share of its score row: kQ * 32 columns starting at column
// h * kQ * 32 of the row in tensor memory.  The two threads of a row exchange their maxima
// through `xch` (one __syncthreads inside: every thread of the CTA calls this), then each writes
// the bf16 weights of its columns into the operand layout (row r of `opnd`: 16-byte chunks of 8
// keys, atom = chunk / 8, chunk swizzled with the row) and returns the scaled row maximum and
// the sum of its own weights.
template <int kQ>
__device__ __forceinline__ void tc_softmax_share(uint32_t trow, int h, int r, int F, float scale_log2,
                                                 float2* xch, uint8_t* opnd, float& ms, float& psum) {
  const int col0 = h * kQ * 32;
  uint32_t su[kQ][32];
#pragma unroll
  for (int q = 0; q < kQ; ++q) tc_ld32_nowait(trow + col0 + q * 32, su[q]);
  tc_ld_wait();
  float sv[kQ][32];
#pragma unroll
  for (int q = 0; q < kQ; ++q)
#pragma unroll
    for (int i = 0; i < 32; ++i) sv[q][i] = __uint_as_float(su[q][i]);
  if (F < 2 * kQ * 32) {
#pragma unroll
    for (int q = 0; q < kQ; ++q)
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + q * 32 + i >= F) sv[q][i] = -INFINITY;
  }
  float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int q = 0; q < kQ; ++q)
#pragma unroll
    for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], sv[q][i]);
  reinterpret_cast<float*>(&xch[r])[h] = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
  __syncthreads();                                      // both shares' maxima are there
  const float2 mm = xch[r];
  const float m = fmaxf(mm.x, mm.y);
  ms = m == -INFINITY ? 0.f : m * scale_log2;           // -inf only when there is no sink key at all
  uint8_t* prow = opnd + r * 128;
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int q = 0; q < kQ; ++q) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {                       // 8 keys = one 16-byte chunk of weights
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float e0 = tc_ex2(fmaf(sv[q][c * 8 + 2 * e], scale_log2, -ms));
        const float e1 = tc_ex2(fmaf(sv[q][c * 8 + 2 * e + 1], scale_log2, -ms));
        sum4[e] += e0 + e1;
        w[e] = pack2(e0, e1);
      }
      const int key_chunk = (col0 >> 3) + q * 4 + c;
      *reinterpret_cast<uint4*>(prow + (key_chunk >> 3) * kTcAtomBytes +
                                (((key_chunk & 7) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  psum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

struct TcRowSpan {
  int req, keep, start, base_off, base_dest;
  bool ok;
};
// Which rows of request b go where (mac_prefill_update_cache.cu:214-236).
__device__ __forceinline__ TcRowSpan tc_row_span(const MacB200PrefillArgs& p, int b) {
  TcRowSpan s{};
  s.ok = false;
  s.req = p.req_ids[b];
  const int Ni = p.lens[b];
  if (Ni <= 0 || p.M <= 0) return s;
  if (s.req < 0 || s.req >= p.R) return s;
  s.start = Ni > p.M ? Ni - p.M : 0;
  s.keep = Ni - s.start;
  s.base_off = p.offsets[b];
  if (s.base_off < 0 || s.base_off + Ni > p.src_rows) return s;
  int L_before = p.request_length_by_batch ? p.request_length[b] : p.request_length[s.req];
  if (L_before < 0) L_before = 0;
  s.base_dest = static_cast<int>((static_cast<int64_t>(L_before) + s.start) % p.M);
  s.ok = true;
  return s;
}

// grid = (slices, Hkv, B); G = query heads per KV head
template <int G>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_sink_exclusive_tc_kernel(const MacB200PrefillBuildArgs a,
                                 const __grid_constant__ CUtensorMap q_map,
                                 const __grid_constant__ CUtensorMap f_map,
                                 const __grid_constant__ CUtensorMap b_map) {
  extern __shared__ __align__(1024) uint8_t tc_smem_raw[];
  // the swizzled operand layout repeats every 1024 bytes of the shared-memory ADDRESS
  uint8_t* tc_smem = tc_smem_raw + ((1024u - (tc_smem_u32(tc_smem_raw) & 1023u)) & 1023u);
  constexpr int TG = kTcTileRows / G;               // tokens per tile
  const MacB200PrefillArgs& p = a.ring;
  const TcRowSpan sp = tc_row_span(p, blockIdx.z);
  if (!sp.ok) return;
  if (sp.req >= a.req_to_token_rows) {              // no page-table row: not built, not marked ready
    if (threadIdx.x == 0) atomicOr(&g_tc_status, MAC_B200_STATUS_BAD_REQUEST);
    return;
  }
  const int H = p.H, Hkv = a.Hkv;
  const int kh = blockIdx.y;
  const int F = a.front_sink_tokens;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int r = tid & 127;                           // row of the tile (= tensor-memory lane)
  const int h = tid >> 7;                            // column half this thread works on
  const uint32_t smem0 = tc_smem_u32(tc_smem);
  uint32_t* tmem_word = reinterpret_cast<uint32_t*>(tc_smem + kTcSmemBars + 96);
  uint32_t* abort_word = reinterpret_cast<uint32_t*>(tc_smem + kTcSmemBars + 100);
  const uint32_t bar_q0 = smem0 + kTcSmemBars;       // q_post rows of stage 0 / 1: +0, +8
  const uint32_t bar_s0 = bar_q0 + 16;               // first product into S[0] / S[1]: +16, +24
  const uint32_t bar_o = bar_q0 + 32;                // second product
  const uint32_t bar_fb = bar_q0 + 40;               // full and band rows

  // ---- tensor memory, barriers
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     tc_smem_u32(tmem_word)),
                 "r"(kTcTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int k = 0; k < 6; ++k) tc_mbar_init(bar_q0 + k * 8, 1);
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // ---- sink K (key-major) and V (dim-major) of this (request, KV head): operand layout, zero
  // rows for keys >= F and for positions without a valid pool row
  {
    const int32_t* table = a.req_to_token + static_cast<int64_t>(sp.req) * a.req_to_token_stride;
    const char* kb = static_cast<const char*>(a.k_buffer) + static_cast<int64_t>(kh) * kTcRowBytes;
    const char* vb = static_cast<const char*>(a.v_buffer) + static_cast<int64_t>(kh) * kTcRowBytes;
    const int64_t tok_stride = static_cast<int64_t>(Hkv) * kTcRowBytes;
    for (int task = tid; task < kTcMaxF * 16; task += kTcThreads) {
      const int c = task >> 7, j = task & 127;  // 16-byte chunk (8 dims) of the row of key j: keys
                                                // vary across the lanes, so the transposing
                                                // 2-byte stores of a warp land in a few words
      int64_t tok = -1;
      if (j < F && j < a.req_to_token_stride) tok = table[j];
      const bool ok = tok >= 0 && tok < a.kv_tokens;
      if (j < F && !ok && c == 0) atomicOr(&g_tc_status, MAC_B200_STATUS_BAD_REQUEST);
      uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = kv;
      if (ok) {
        kv = *reinterpret_cast<const uint4*>(kb + tok * tok_stride + c * 16);
        vv = *reinterpret_cast<const uint4*>(vb + tok * tok_stride + c * 16);
      }
      // K: atom = dims / 64, row = key, chunk of the row swizzled with the row
      *reinterpret_cast<uint4*>(tc_smem + kTcSmemK + (c >> 3) * kTcAtomBytes + j * 128 +
                                (((c & 7) ^ (j & 7)) << 4)) = kv;
      // V transposed: atom = key / 64, row = dim, element = key % 64
      const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
      uint8_t* vt = tc_smem + kTcSmemVt + (j >> 6) * kTcAtomBytes + ((j & 7) << 1);
      const int kc = (j & 63) >> 3;             // 16-byte chunk of the key inside the dim's row
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = c * 8 + e;
        const uint16_t val = static_cast<uint16_t>((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xffffu));
        *reinterpret_cast<uint16_t*>(vt + d * 128 + ((kc ^ (d & 7)) << 4)) = val;
      }
    }
  }
  tc_fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_word;
  const uint32_t tmem_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
  const uint32_t tmem_o = tmem_base + 256;           // S[0] at +0, S[1] at +128

  uint8_t* fullS = tc_smem + kTcSmemFull;
  uint8_t* bandS = tc_smem + kTcSmemBand;
  float2* xch = reinterpret_cast<float2*>(tc_smem + kTcSmemXch);   // per row: the halves' maxima, then sums
  const uint64_t desc_k = tc_operand_desc(smem0 + kTcSmemK);
  const uint64_t desc_vt = tc_operand_desc(smem0 + kTcSmemVt);

  const int ntiles = (sp.keep + TG - 1) / TG;
  const size_t row_bf16 = static_cast<size_t>(H) * kTcRowBytes;
  const char* qpre = static_cast<const char*>(p.src_q);
  const char* fsrc = static_cast<const char*>(p.src_attn);
  const char* bsrc = static_cast<const char*>(a.band_attn);
  char* qc = static_cast<char*>(p.q_cache) + static_cast<size_t>(sp.req) * p.M * row_bf16;
  char* ac = static_cast<char*>(p.attn_cache) + static_cast<size_t>(sp.req) * p.M * row_bf16;
  char* pc = p.q_post_cache
                 ? static_cast<char*>(p.q_post_cache) + static_cast<size_t>(sp.req) * p.M * row_bf16
                 : nullptr;
  float* lc = p.lse_cache + static_cast<size_t>(sp.req) * p.M * H;
  const float scale_log2 = a.sm_scale * 1.4426950408889634f;
  const int64_t pos0 = static_cast<int64_t>(p.request_length_by_batch
                                                ? p.request_length[blockIdx.z]
                                                : p.request_length[sp.req]);
  const int64_t pos_base = (pos0 < 0 ? 0 : pos0) + sp.start;
  const uint32_t nanw = 0x7fc07fc0u;
  const uint4 nan4 = make_uint4(nanw, nanw, nanw, nanw);
  const int nk2 = (F + 15) >> 4;                     // k-steps of the second product
  const int tok_r = r / G, head_r = kh * G + (r % G);   // token of the tile and head of this thread's row

  // what this thread moves in the coalesced passes: 16-byte piece `c16` of the 256-byte rows
  // it*16 + tid/16
  const int c16 = tid & 15, row16 = tid >> 4;
  auto head_off16 = [&](int rr) {
    return static_cast<size_t>(kh * G + rr % G) * kTcRowBytes + c16 * 16;
  };
  auto src_tok_of = [&](int tile_x) { return sp.base_off + sp.start + tile_x * TG; };
  // The copy-engine requests and the products are issued by single threads; each costs its
  // thread a few hundred cycles, and every other thread meets it at the next barrier.  So the
  // duties are spread over threads of different warps: thread 0 arms the barriers and issues
  // the second product, thread 128 issues the next tile's first product, and the boxes of a
  // request are issued one per warp.
  auto request_q_rows = [&](int tile_x, int stage) {   // threads 0 and 128: q_post rows -> operand layout
    const uint32_t dst = smem0 + kTcSmemQ + stage * kTcOperandBytes, bar = bar_q0 + stage * 8;
    if (tid == 0) {
      tc_mbar_expect_tx(bar, kTcOperandBytes);
      tc_tma_load_3d(dst, &q_map, 0, kh * G, src_tok_of(tile_x), bar);
    } else if (tid == 128) {
      tc_tma_load_3d(dst + kTcAtomBytes, &q_map, 64, kh * G, src_tok_of(tile_x), bar);
    }
  };
  auto request_state_rows = [&](int tile_x) {          // threads 0, 32, 64, 96: full and band rows
    if (tid == 0) {
      tc_mbar_expect_tx(bar_fb, 2 * kTcOperandBytes);
      tc_tma_load_3d(smem0 + kTcSmemFull, &f_map, 0, kh * G, src_tok_of(tile_x), bar_fb);
    } else if (tid == 32) {
      tc_tma_load_3d(smem0 + kTcSmemFull + kTcAtomBytes, &f_map, 64, kh * G, src_tok_of(tile_x), bar_fb);
    } else if (tid == 64) {
      tc_tma_load_3d(smem0 + kTcSmemBand, &b_map, 0, kh * G, src_tok_of(tile_x), bar_fb);
    } else if (tid == 96) {
      tc_tma_load_3d(smem0 + kTcSmemBand + kTcAtomBytes, &b_map, 64, kh * G, src_tok_of(tile_x), bar_fb);
    }
  };
  auto issue_first_product = [&](int stage) {          // one thread: S[stage] = Q[stage] K^T
    const uint64_t desc_q = tc_operand_desc(smem0 + kTcSmemQ + stage * kTcOperandBytes);
    tc_fence_after_sync();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint64_t off = static_cast<uint64_t>(((k >> 2) * kTcAtomBytes + (k & 3) * 32) >> 4);
      tc_mma(tmem_base + stage * 128, desc_q + off, desc_k + off, k > 0 ? 1u : 0u);
    }
    tc_commit(bar_s0 + stage * 8);
  };
  // Rows that come through registers (q_pre) or the copy engine (q_post, full, band) are pulled
  // into L2 two tiles ahead: one prefetch per (tensor, token) of the G heads' contiguous rows.
  auto prefetch_rows = [&](int tile_x) {
    if (tile_x >= ntiles) return;
    const int ip = tile_x * TG;
    for (int t = tid; t < 3 * TG; t += kTcThreads) {
      const int which = t / TG, tk = t - which * TG;
      if (ip + tk >= sp.keep) continue;
      const char* base = which == 0 ? qpre : which == 1 ? fsrc : bsrc;
      const char* src = base + static_cast<size_t>(src_tok_of(tile_x) + tk) * row_bf16 +
                        static_cast<size_t>(kh * G) * kTcRowBytes;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(G * kTcRowBytes)
                   : "memory");
    }
  };

  const int tile_step = gridDim.x;
  const int tile0 = blockIdx.x;
  bool good = true;
  if (tile0 < ntiles) {
    prefetch_rows(tile0);
    prefetch_rows(tile0 + tile_step);
    request_q_rows(tile0, 0);
    if (tile0 + tile_step < ntiles) request_q_rows(tile0 + tile_step, 1);
    request_state_rows(tile0);
    if (tid == 0) {
      good &= tc_mbar_wait(bar_q0, 0);
      issue_first_product(0);
    }
    __syncwarp();
  }

  int k = 0;
  for (int tile = tile0; tile < ntiles; tile += tile_step, ++k) {
    if (*reinterpret_cast<volatile uint32_t*>(abort_word) != 0u) break;
    const int s = k & 1;                                   // stage of this tile's q_post rows and scores
    const uint32_t ph2 = static_cast<uint32_t>(k >> 1) & 1u, ph1 = static_cast<uint32_t>(k) & 1u;
    const int i0 = tile * TG;
    const int src_tok0 = src_tok_of(tile);                 // source row of the tile's first token
    const int nrows_tok = sp.keep - i0;                    // tokens of the tile that exist (may exceed TG)
    const bool has_next = tile + tile_step < ntiles;
    uint8_t* opnd = tc_smem + kTcSmemQ + s * kTcOperandBytes;   // q_post rows, then the weights
    prefetch_rows(tile + 2 * tile_step);

    // ---- 1. this row's LSEs; the q_pre rows on their way to the ring (stored after the softmax)
    const bool row_ok = tok_r < nrows_tok;
    float l_full = 0.f, l_band = 0.f;
    if (row_ok) {
      const size_t li = static_cast<size_t>(src_tok0 + tok_r) * H + head_r;
      l_full = load_lse(p.src_lse, a.full_lse_dtype, li);
      l_band = load_lse(a.band_lse, a.band_lse_dtype, li);
    }
    uint4 qv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int rr = u * 16 + row16;
      if (rr / G < nrows_tok)
        qv[u] = ld_stream16(qpre + static_cast<size_t>(src_tok0 + rr / G) * row_bf16 + head_off16(rr));
    }

    // ---- 2. softmax of this thread's share of its row: 64 of the 128 score columns, or 32 of
    // the first 64 when the sink has at most 64 keys (the columns beyond F hold no key; the
    // second product only reads the k-steps that do)
    good &= tc_mbar_wait(bar_s0 + s * 8, ph2);
    tc_fence_after_sync();
    float ms, psum;
    if (F > 64)
      tc_softmax_share<2>(tmem_base + s * 128 + tmem_lane, h, r, F, scale_log2, xch, opnd, ms, psum);
    else
      tc_softmax_share<1>(tmem_base + s * 128 + tmem_lane, h, r, F, scale_log2, xch, opnd, ms, psum);
    tc_fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();                                    // sync 2: weights written, maxima consumed
    reinterpret_cast<float*>(&xch[r])[h] = psum;        // read after sync 3

    // ---- 3. O = P V, and at once the next tile's S = Q K^T; meanwhile the q_pre rows are
    // stored and the row factors worked out
    if (tid == 0) {
      const uint64_t desc_p = tc_operand_desc(smem0 + kTcSmemQ + s * kTcOperandBytes);
      tc_fence_after_sync();
      for (int kk = 0; kk < nk2; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * kTcAtomBytes + (kk & 3) * 32) >> 4);
        tc_mma(tmem_o, desc_p + off, desc_vt + off, kk > 0 ? 1u : 0u);
      }
      tc_commit(bar_o);
    } else if (tid == 128 && has_next) {
      good &= tc_mbar_wait(bar_q0 + (s ^ 1) * 8, static_cast<uint32_t>((k + 1) >> 1) & 1u);
      issue_first_product(s ^ 1);
    }
    __syncwarp();
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int rr = u * 16 + row16;
      if (rr / G < nrows_tok) {
        int d = sp.base_dest + i0 + rr / G;
        if (d >= p.M) d -= p.M;
        const size_t doff = static_cast<size_t>(d) * row_bf16 + head_off16(rr);
        st_stream16(qc + doff, qv[u]);
        if (pc) st_stream16(pc + doff, nan4);
      }
    }
    __syncthreads();                                    // sync 3: both halves' sums are there
    // both threads of a row work out its factors (the second one would only wait otherwise):
    // no hand-over through shared memory, one barrier fewer
    float4 k4 = make_float4(0.f, 0.f, 0.f, 1.f);
    if (row_ok) {
      const float2 ss = xch[r];
      const float sum = ss.x + ss.y;
      float ret1, t1, s1;
      downdate_scalars(l_full, __fmul_rn(l_band, a.band_lse_scale), ret1, t1, s1);
      int64_t E = pos_base + i0 + tok_r + 1 - a.semantic_pos_ahead;
      if (E < 0) E = 0;
      float ret2 = -INFINITY;
      if (E > F) {
        const float lse_sink = sum > 0.f ? (ms + log2f(sum)) * 0.6931471805599453f : -INFINITY;
        float t2, s2;
        downdate_scalars(ret1, lse_sink, ret2, t2, s2);
        k4.x = s1 * s2;
        k4.y = t1 * k4.x;
        k4.z = sum > 0.f ? t2 * s2 / sum : 0.f;
        k4.w = 0.f;
      }
      if (h == 0) {
        int dest_r = sp.base_dest + i0 + tok_r;           // ring row of this thread's row
        if (dest_r >= p.M) dest_r -= p.M;
        lc[static_cast<size_t>(dest_r) * H + head_r] = ret2;
      }
    }
    good &= tc_mbar_wait(bar_o, ph1);
    good &= tc_mbar_wait(bar_fb, ph1);
    tc_fence_after_sync();
    // the operand buffer of this stage is free (threads 0 and 128 have seen the second product
    // finish themselves): the q_post rows of the tile after the next
    if (tile + 2 * tile_step < ntiles) request_q_rows(tile + 2 * tile_step, s);
    __syncwarp();

    // ---- 4. this thread's half of its row: state = full*A - band*B - sink*C, written in place
    // over the staged full row (both rows lie in the operand layout: a thread's 16-byte chunks
    // are swizzled with its row, so the eight rows of a quarter-warp never share a bank)
    {
      uint8_t* frow = fullS + h * kTcAtomBytes + r * 128;
      const uint8_t* brow = bandS + h * kTcAtomBytes + r * 128;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t ou[32];
        tc_ld32_nowait(tmem_o + tmem_lane + h * 64 + q * 32, ou);
        tc_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c) {                   // 8 columns = one 16-byte chunk of bf16
          const int pos = ((q * 4 + c) ^ (r & 7)) << 4;
          const uint4 f4 = *reinterpret_cast<const uint4*>(frow + pos);
          const uint4 b4 = *reinterpret_cast<const uint4*>(brow + pos);
          const uint32_t x[4] = {f4.x, f4.y, f4.z, f4.w};
          const uint32_t y[4] = {b4.x, b4.y, b4.z, b4.w};
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float s0 = nk2 == 0 ? 0.f : __uint_as_float(ou[c * 8 + 2 * i]);
            const float s1 = nk2 == 0 ? 0.f : __uint_as_float(ou[c * 8 + 2 * i + 1]);
            const float r0 = fmaf(lo_f(x[i]), k4.x, fmaf(-lo_f(y[i]), k4.y, -(s0 * k4.z)));
            const float r1 = fmaf(hi_f(x[i]), k4.x, fmaf(-hi_f(y[i]), k4.y, -(s1 * k4.z)));
            w[i] = k4.w != 0.f ? 0u : pack2(r0, r1);
          }
          *reinterpret_cast<uint4*>(frow + pos) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    tc_fence_before_sync();
    if (!good) {
      atomicOr(&g_tc_status, MAC_B200_STATUS_COPY_TIMEOUT);
      *reinterpret_cast<volatile uint32_t*>(abort_word) = 1u;   // read after the syncs below
    }
    __syncthreads();                                    // sync 5: the finished rows are in place

    // ---- 5. the rows go to the ring in whole 256-byte rows
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int rr = u * 16 + row16;
      if (rr / G >= nrows_tok) continue;
      const uint4 w4 = *reinterpret_cast<const uint4*>(fullS + (c16 >> 3) * kTcAtomBytes + rr * 128 +
                                                       (((c16 & 7) ^ (rr & 7)) << 4));
      int d = sp.base_dest + i0 + rr / G;
      if (d >= p.M) d -= p.M;
      st_stream16(ac + static_cast<size_t>(d) * row_bf16 + head_off16(rr), w4);
    }
    tc_fence_async_smem();                              // the copy engine writes these rows next
    __syncthreads();                                    // sync 6: the staged rows are free
    if (has_next) request_state_rows(tile + tile_step);
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTcTmemCols)
                 : "memory");
  }
}

typedef CUresult (*TcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TcEncodeTiledFn tc_encode_tiled_fn() {
  static TcEncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<TcEncodeTiledFn>(ptr);
  }();
  return fn;
}

}  // namespace

int take_prefill_sink_tc_status(unsigned* bits) {
  unsigned v = 0;
  MAC_CUDA(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(v)));
  if (v != 0) {
    const unsigned zero = 0;
    MAC_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(zero)));
  }
  *bits = v;
  return MAC_B200_OK;
}

// Launches the tensor-memory kernel when the step fits it; `launched` tells the caller.
// The caller has validated the arguments of the sink-exclusive mode.
int launch_prefill_sink_exclusive_tc(const MacB200PrefillBuildArgs& a, int sms, cudaStream_t stream,
                                     bool* launched) {
  *launched = false;
  const MacB200PrefillArgs& p = a.ring;
  const int G = p.H / a.Hkv;
  if (G < 1 || G > 16 || (16 % G) != 0 || p.src_rows <= 0) return MAC_B200_OK;
  // CTAs per (request, KV head): every CTA restages the sink K/V, so as few as fill the GPU in
  // whole waves -- the count in 1..8 whose last wave is fullest.
  const int TG = kTcTileRows / G;
  const int max_tiles = ((p.M < 1 ? 1 : p.M) + TG - 1) / TG;
  const int max_slices = max_tiles;
  const int pairs = p.B * a.Hkv;
  int slices = 1;
  double best = -1.0;
  for (int sl = 1; sl <= 8 && sl <= max_slices; ++sl) {
    const long long total = static_cast<long long>(sl) * pairs;
    const long long waves = (total + sms - 1) / sms;
    const double eff = static_cast<double>(total) / static_cast<double>(waves * sms);
    if (eff > best + 1e-9) { best = eff; slices = sl; }
  }
  if (const char* e = std::getenv("MAC_B200_SINK_SLICES")) {
    const int v = std::atoi(e);
    if (v >= 1 && v <= max_slices) slices = v;
  }
  TcEncodeTiledFn enc = tc_encode_tiled_fn();
  if (enc == nullptr) return MAC_B200_OK;
  // q_post, full and band rows share one geometry: [src_rows][H][128] bf16, box = 64 dims x the G
  // heads of a KV head x 128/G tokens, 128-byte swizzle (a box lands as one operand atom)
  alignas(64) CUtensorMap q_map, f_map, b_map;
  const cuuint64_t dims[3] = {128u, static_cast<cuuint64_t>(p.H), static_cast<cuuint64_t>(p.src_rows)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kTcRowBytes),
                                 static_cast<cuuint64_t>(p.H) * kTcRowBytes};
  const cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(G), static_cast<cuuint32_t>(kTcTileRows / G)};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const void* bases[3] = {a.q_post, p.src_attn, a.band_attn};
  CUtensorMap* maps[3] = {&q_map, &f_map, &b_map};
  for (int i = 0; i < 3; ++i) {
    if (enc(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(bases[i]), dims, strides,
            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return MAC_B200_OK;
  }
  void (*kernel)(MacB200PrefillBuildArgs, CUtensorMap, CUtensorMap, CUtensorMap) =
      G == 1 ? prefill_sink_exclusive_tc_kernel<1>
      : G == 2 ? prefill_sink_exclusive_tc_kernel<2>
      : G == 4 ? prefill_sink_exclusive_tc_kernel<4>
      : G == 8 ? prefill_sink_exclusive_tc_kernel<8>
               : prefill_sink_exclusive_tc_kernel<16>;
  MAC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
  dim3 grid(slices, a.Hkv, p.B);
  kernel<<<grid, kTcThreads, kTcSmemBytes, stream>>>(a, q_map, f_map, b_map);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  *launched = true;
  return MAC_B200_OK;
}

}  // namespace mac_b200
