// One-pass prefill ring build (sm_100a): LSE downdate + ring write + readiness
// mark for the rows that reach the ring.
//
// The reference's prefill hook
// (attention/src/mac_attention/integrations/sglang/flashinfer_hooks.py:2459-2492)
// scales the band LSE, downdates EVERY prompt row in place
// (csrc/mac_merge_downdate_cache.cu:116-288), copies the last min(len, M) rows of
// each request into its ring (csrc/mac_prefill_update_cache.cu:201-269) and marks
// the requests ready (same file, 374-409): four launches and, for a 32K prompt
// with a 2K ring, sixteen times more downdate traffic than the ring needs.  Here
// the rows bound for the ring are downdated on their way into it: each
// (row, head) state is read once from the full-prefix and band tensors and
// written once, to the ring.  The band tensors are left as they were.
#include <cstdlib>

#include "mac_b200_common.h"
#include "mac_b200_state_math.cuh"

namespace mac_b200 {
namespace {

constexpr int kBuildThreads = 256;
constexpr int kBuildMaxH = 256;  // heads whose row scalars fit the shared-memory tables

struct RowSpan {
  int req, keep, start, base_off, base_dest;
  bool ok;
};

// Which rows of request b go where (mac_prefill_update_cache.cu:214-236).
__device__ __forceinline__ RowSpan row_span(const MacB200PrefillArgs& p, int b) {
  RowSpan s{};
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

struct ChunkLoads {
  uint4 q[2][2], full[2][2], band[2][2];  // [row of the pair][chunk c, chunk c + blockDim]
};

__device__ __forceinline__ uint4 downdate_chunk(uint4 x4, uint4 y4, float t, float scale) {
  const uint32_t x[4] = {x4.x, x4.y, x4.z, x4.w};
  const uint32_t y[4] = {y4.x, y4.y, y4.z, y4.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float r0 = (lo_f(x[i]) - t * lo_f(y[i])) * scale;
    const float r1 = (hi_f(x[i]) - t * hi_f(y[i])) * scale;
    o[i] = pack2(r0, r1);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// grid = (ctas_per_request, B); CTA x of request b handles row pairs x, x+gridDim.x, ...
__global__ void __launch_bounds__(kBuildThreads, 2)
prefill_downdate_ring_kernel(const MacB200PrefillBuildArgs a) {
  const MacB200PrefillArgs& p = a.ring;
  const RowSpan sp = row_span(p, blockIdx.y);
  if (!sp.ok) return;
  const int H = p.H, D = p.D;
  const size_t row_bf16 = static_cast<size_t>(H) * D * 2;
  uint8_t* qc = static_cast<uint8_t*>(p.q_cache) + static_cast<size_t>(sp.req) * p.M * row_bf16;
  uint8_t* ac = static_cast<uint8_t*>(p.attn_cache) + static_cast<size_t>(sp.req) * p.M * row_bf16;
  float* lc = p.lse_cache + static_cast<size_t>(sp.req) * p.M * H;
  uint8_t* pc = p.q_post_cache
                    ? static_cast<uint8_t*>(p.q_post_cache) + static_cast<size_t>(sp.req) * p.M * row_bf16
                    : nullptr;
  const uint8_t* qs = static_cast<const uint8_t*>(p.src_q);
  const uint8_t* fs = static_cast<const uint8_t*>(p.src_attn);
  const uint8_t* bs = static_cast<const uint8_t*>(a.band_attn);
  const bool unmatchable = a.sink_mode == MAC_B200_SINK_UNMATCHABLE;
  const uint32_t nanw = 0x7fc07fc0u;
  const uint4 nan4 = make_uint4(nanw, nanw, nanw, nanw);

  const bool vec = D % 8 == 0 && H <= kBuildMaxH &&
                   ((reinterpret_cast<uintptr_t>(qc) | reinterpret_cast<uintptr_t>(ac) |
                     reinterpret_cast<uintptr_t>(qs) | reinterpret_cast<uintptr_t>(fs) |
                     reinterpret_cast<uintptr_t>(bs) | reinterpret_cast<uintptr_t>(pc)) & 15u) == 0;
  if (!vec) {
    // Element-wise path for odd head sizes or unaligned bases.
    const __nv_bfloat16* f16 = reinterpret_cast<const __nv_bfloat16*>(fs);
    const __nv_bfloat16* b16 = reinterpret_cast<const __nv_bfloat16*>(bs);
    const uint16_t* q16 = reinterpret_cast<const uint16_t*>(qs);
    for (int i = blockIdx.x; i < sp.keep; i += gridDim.x) {
      int dest = sp.base_dest + i;
      if (dest >= p.M) dest -= p.M;
      const size_t srow = static_cast<size_t>(sp.base_off + sp.start + i);
      for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
        const int h = e / D;
        float ret, t, scale;
        downdate_scalars(load_lse(p.src_lse, a.full_lse_dtype, srow * H + h),
                         __fmul_rn(load_lse(a.band_lse, a.band_lse_dtype, srow * H + h),
                                   a.band_lse_scale),  // rounded product, as a separate scale op
                         ret, t, scale);
        const float r = (__bfloat162float(f16[srow * H * D + e]) -
                         t * __bfloat162float(b16[srow * H * D + e])) * scale;
        reinterpret_cast<__nv_bfloat16*>(ac)[static_cast<size_t>(dest) * H * D + e] =
            __float2bfloat16_rn(r);
        reinterpret_cast<uint16_t*>(qc)[static_cast<size_t>(dest) * H * D + e] = q16[srow * H * D + e];
        if (pc) reinterpret_cast<uint16_t*>(pc)[static_cast<size_t>(dest) * H * D + e] = 0x7fc0;
        if (e == h * D) lc[static_cast<size_t>(dest) * H + h] = unmatchable ? -INFINITY : ret;
      }
    }
    return;
  }

  __shared__ float s_t[2][2 * kBuildMaxH];
  __shared__ float s_scale[2][2 * kBuildMaxH];
  const int chunks = static_cast<int>(row_bf16 / 16);
  const int cph = D / 8;  // 16-byte chunks per head
  int par = 0;
  for (int i = 2 * blockIdx.x; i < sp.keep; i += 2 * gridDim.x, par ^= 1) {
    const bool two = i + 1 < sp.keep;
    int d0 = sp.base_dest + i;
    if (d0 >= p.M) d0 -= p.M;
    int d1 = d0 + 1;
    if (d1 >= p.M) d1 -= p.M;
    const size_t s0 = static_cast<size_t>(sp.base_off + sp.start + i), s1 = s0 + 1;

    // First pass of row loads goes out before the LSE arithmetic, so that the
    // exp/log chain of the scalars overlaps the memory latency.
    ChunkLoads L;
    auto issue = [&](int c) {
      const int c2 = c + blockDim.x;
      const bool more = c2 < chunks;
      L.q[0][0] = ld_stream16(qs + s0 * row_bf16 + static_cast<size_t>(c) * 16);
      L.full[0][0] = ld_stream16(fs + s0 * row_bf16 + static_cast<size_t>(c) * 16);
      L.band[0][0] = ld_stream16(bs + s0 * row_bf16 + static_cast<size_t>(c) * 16);
      if (more) {
        L.q[0][1] = ld_stream16(qs + s0 * row_bf16 + static_cast<size_t>(c2) * 16);
        L.full[0][1] = ld_stream16(fs + s0 * row_bf16 + static_cast<size_t>(c2) * 16);
        L.band[0][1] = ld_stream16(bs + s0 * row_bf16 + static_cast<size_t>(c2) * 16);
      }
      if (two) {
        L.q[1][0] = ld_stream16(qs + s1 * row_bf16 + static_cast<size_t>(c) * 16);
        L.full[1][0] = ld_stream16(fs + s1 * row_bf16 + static_cast<size_t>(c) * 16);
        L.band[1][0] = ld_stream16(bs + s1 * row_bf16 + static_cast<size_t>(c) * 16);
        if (more) {
          L.q[1][1] = ld_stream16(qs + s1 * row_bf16 + static_cast<size_t>(c2) * 16);
          L.full[1][1] = ld_stream16(fs + s1 * row_bf16 + static_cast<size_t>(c2) * 16);
          L.band[1][1] = ld_stream16(bs + s1 * row_bf16 + static_cast<size_t>(c2) * 16);
        }
      }
    };
    auto finish = [&](int c) {
      const int c2 = c + blockDim.x;
      const bool more = c2 < chunks;
      const int h0 = c / cph, h1 = c2 / cph;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r == 1 && !two) break;
        const size_t drow = static_cast<size_t>(r ? d1 : d0) * row_bf16;
        st_stream16(qc + drow + static_cast<size_t>(c) * 16, L.q[r][0]);
        st_stream16(ac + drow + static_cast<size_t>(c) * 16,
                    downdate_chunk(L.full[r][0], L.band[r][0], s_t[par][r * H + h0],
                                   s_scale[par][r * H + h0]));
        if (pc) st_stream16(pc + drow + static_cast<size_t>(c) * 16, nan4);
        if (more) {
          st_stream16(qc + drow + static_cast<size_t>(c2) * 16, L.q[r][1]);
          st_stream16(ac + drow + static_cast<size_t>(c2) * 16,
                      downdate_chunk(L.full[r][1], L.band[r][1], s_t[par][r * H + h1],
                                     s_scale[par][r * H + h1]));
          if (pc) st_stream16(pc + drow + static_cast<size_t>(c2) * 16, nan4);
        }
      }
    };

    const bool first = static_cast<int>(threadIdx.x) < chunks;
    if (first) issue(threadIdx.x);
    for (int idx = threadIdx.x; idx < (two ? 2 : 1) * H; idx += blockDim.x) {
      const int r = idx >= H ? 1 : 0;
      const int h = idx - r * H;
      const size_t srow = r ? s1 : s0;
      const int drow = r ? d1 : d0;
      float ret, t, scale;
      downdate_scalars(load_lse(p.src_lse, a.full_lse_dtype, srow * H + h),
                       __fmul_rn(load_lse(a.band_lse, a.band_lse_dtype, srow * H + h),
                                 a.band_lse_scale),  // rounded product, as a separate scale op
                       ret, t, scale);
      s_t[par][idx] = t;
      s_scale[par][idx] = scale;
      lc[static_cast<size_t>(drow) * H + h] = unmatchable ? -INFINITY : ret;
    }
    __syncthreads();
    if (first) finish(threadIdx.x);
    for (int c = threadIdx.x + 2 * blockDim.x; c < chunks; c += 2 * blockDim.x) {
      issue(c);
      finish(c);
    }
  }
}

// ------------------------------------------------------------------------
// Sink-exclusive build (MAC_B200_SINK_EXCLUDE).
//
// A ring row must cover [min(F, E), E).  The prefill producers give the state
// of [0, pos] and of the trailing window [E, pos]; what is left to remove is
// the row's attention over the sink tokens [0, F), which nobody has computed.
// It is a small dense problem -- 16 query rows x F <= 128 keys x D = 128 per
// warp tile -- done here on the tensor cores (mma.sync m16n8k16, bf16 in, fp32
// accumulate) straight from shared memory, inside the pass that also streams
// the row through the two downdates into the ring.  Its HBM traffic is the
// stream of the rows alone; the sink K/V of a (request, KV head) are read once
// per CTA.
//
// CTA = (slice of a request's ring rows, one KV head); 8 independent warps.  A
// warp tile is 16 MMA rows = 16/G consecutive tokens x the G query heads of the
// KV head.  Per tile the warp
//   1. cp.asyncs its full and band rows into its own staging and fetches the
//      rows' LSEs (lane r < 16 owns MMA row r); the q_post and q_pre rows were
//      requested while the previous tile was still being worked on,
//   2. S = Q K^T over the sink keys; as soon as the staged q rows are dead the
//      NEXT tile's q rows are requested into the same staging, so that a tile
//      never starts by waiting for DRAM; softmax (log2 domain), O = P V,
//   3. folds both downdates into three factors per row, one row per lane:
//      state = full*A - band*B - sink_unnormalised*C,
//   4. applies them in the accumulators' own layout, in place over the staged
//      full rows, and streams the rows to the ring in 16-byte chunks.
// With 246 registers per thread (64 score + 64 output accumulators) only eight
// warps fit an SM, so the kernel is bound by issue latency rather than by HBM
// or the tensor pipe; anything the warp does on a few lanes only (the row
// factors' exp/log chains) costs as much as if all lanes did it.
constexpr int kSxD = 128;
constexpr int kSxRowBytes = kSxD * 2;
constexpr int kSxMaxF = 128;
constexpr int kSxWarps = 8;
constexpr int kSxThreads = kSxWarps * 32;
constexpr int kSxRegionRows = 16 * kSxRowBytes;        // one staged 16-row tensor
constexpr int kSxRegionA = 2 * kSxRegionRows;          // q_post + q_pre staging of one tile
constexpr int kSxWarpBytes = kSxRegionA + 2 * kSxRegionRows + 16 * 16;
constexpr int kSxKvBytes = 2 * kSxMaxF * kSxRowBytes;
constexpr int kSxSmemBytes = kSxKvBytes + kSxWarps * kSxWarpBytes;

__device__ __forceinline__ uint32_t sx_smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void sx_cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void sx_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void sx_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void sx_ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                               uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void sx_ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                     uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void sx_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float sx_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Sticky status bits raised by the kernels of this file (read and cleared
// through mac_b200_query_status together with the decode kernel's word).
__device__ unsigned g_build_status = 0;

// A request whose id has no row in req_to_token cannot have its sink attention
// computed: its ring rows are not built and it is not marked ready.
__device__ __forceinline__ bool sink_request_out_of_table(const MacB200PrefillBuildArgs& a, int req) {
  return a.sink_mode == MAC_B200_SINK_EXCLUDE && req >= a.req_to_token_rows;
}

// grid = (slices, Hkv, B); G = query heads per KV head
template <int G>
__global__ void __launch_bounds__(kSxThreads, 1)
prefill_sink_exclusive_ring_kernel(const MacB200PrefillBuildArgs a) {
  extern __shared__ __align__(128) uint8_t sx_smem[];
  constexpr int TG = 16 / G;                        // tokens per warp tile
  const MacB200PrefillArgs& p = a.ring;
  const RowSpan sp = row_span(p, blockIdx.z);
  if (!sp.ok) return;
  if (sink_request_out_of_table(a, sp.req)) {
    if (threadIdx.x == 0) atomicOr(&g_build_status, MAC_B200_STATUS_BAD_REQUEST);
    return;
  }
  const int H = p.H, Hkv = a.Hkv;
  const int kh = blockIdx.y;
  const int F = a.front_sink_tokens;
  const int nkb = (F + 15) >> 4;  // 16-key blocks
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = lane & 3, rlo = lane >> 2, rhi = rlo + 8;

  // ---- sink K/V of this (request, KV head) -> shared memory, swizzled rows
  uint8_t* ks = sx_smem;
  uint8_t* vs = sx_smem + kSxMaxF * kSxRowBytes;
  {
    const int32_t* table = a.req_to_token + static_cast<int64_t>(sp.req) * a.req_to_token_stride;
    const char* kb = static_cast<const char*>(a.k_buffer) + static_cast<int64_t>(kh) * kSxRowBytes;
    const char* vb = static_cast<const char*>(a.v_buffer) + static_cast<int64_t>(kh) * kSxRowBytes;
    const int64_t tok_stride = static_cast<int64_t>(Hkv) * kSxRowBytes;
    for (int task = tid; task < nkb * 16 * 16; task += kSxThreads) {
      const int j = task >> 4, c = task & 15;
      int64_t tok = -1;
      if (j < F && j < a.req_to_token_stride) tok = table[j];
      const bool ok = tok >= 0 && tok < a.kv_tokens;
      if (j < F && !ok && c == 0)   // a sink position without a valid pool row reads as zeros
        atomicOr(&g_build_status, MAC_B200_STATUS_BAD_REQUEST);
      const int64_t off = (ok ? tok : 0) * tok_stride + c * 16;
      const uint32_t dst = j * kSxRowBytes + ((c ^ (j & 7)) << 4);
      sx_cp_async16(sx_smem_u32(ks) + dst, kb + off, ok ? 16 : 0);
      sx_cp_async16(sx_smem_u32(vs) + dst, vb + off, ok ? 16 : 0);
    }
    sx_commit();
    sx_wait<0>();
    __syncthreads();
  }

  uint8_t* wbase = sx_smem + kSxKvBytes + warp * kSxWarpBytes;
  uint8_t* regA = wbase;                           // q_post rows | q_pre rows, later the sink state
  uint8_t* fullS = wbase + kSxRegionA;
  uint8_t* bandS = fullS + kSxRegionRows;
  float4* scal = reinterpret_cast<float4*>(bandS + kSxRegionRows);  // per row: A, B, C, empty flag
  const uint32_t regA_u32 = sx_smem_u32(regA), full_u32 = sx_smem_u32(fullS),
                 band_u32 = sx_smem_u32(bandS);
  const uint32_t ks_u32 = sx_smem_u32(ks), vs_u32 = sx_smem_u32(vs);

  const int ntiles = (sp.keep + TG - 1) / TG;
  const size_t row_bf16 = static_cast<size_t>(H) * kSxRowBytes;
  const char* qpost = static_cast<const char*>(a.q_post);
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

  // What this lane moves in the 16-byte passes: chunk c of MMA rows 2j + (lane >> 4).
  // MMA row r = token r / G of the tile, head kh * G + r % G.
  const int c = lane & 15;
  const int r_half = lane >> 4;
  const size_t src_base = static_cast<size_t>(sp.base_off + sp.start) * row_bf16 +
                          static_cast<size_t>(kh * G) * kSxRowBytes + c * 16;
  const size_t head_base = static_cast<size_t>(kh * G) * kSxRowBytes + c * 16;
  const int mi = lane >> 3, l7 = lane & 7;

  // q_post (swizzled, an MMA operand) and q_pre (linear, copied through) rows of a tile
  auto stage_q_rows = [&](int tile_q) {
    const int iq = tile_q * TG;
    const size_t tsrc = src_base + static_cast<size_t>(iq) * row_bf16;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = 2 * j + r_half;
      const bool ok = tile_q < ntiles && iq + r / G < sp.keep;
      const size_t so = ok ? tsrc + static_cast<size_t>(r / G) * row_bf16 + (r % G) * kSxRowBytes : 0;
      sx_cp_async16(regA_u32 + r * kSxRowBytes + ((c ^ (r & 7)) << 4), qpost + so, ok ? 16 : 0);
      sx_cp_async16(regA_u32 + kSxRegionRows + r * kSxRowBytes + c * 16, qpre + so, ok ? 16 : 0);
    }
    sx_commit();
  };
  const int tile_step = gridDim.x * kSxWarps;
  if (static_cast<int>(blockIdx.x) * kSxWarps + warp < ntiles)
    stage_q_rows(blockIdx.x * kSxWarps + warp);

  for (int tile = blockIdx.x * kSxWarps + warp; tile < ntiles; tile += tile_step) {
    const int i0 = tile * TG;
    const size_t tile_src = src_base + static_cast<size_t>(i0) * row_bf16;
    int dbase = sp.base_dest + i0;                  // ring row of the tile's first token
    if (dbase >= p.M) dbase -= p.M;

    // ---- 1. stage the tile: full and band rows now; the q rows are already on their way
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = 2 * j + r_half;
      const bool ok = i0 + r / G < sp.keep;
      const size_t so = ok ? tile_src + static_cast<size_t>(r / G) * row_bf16 + (r % G) * kSxRowBytes : 0;
      const uint32_t dst = r * kSxRowBytes + ((c ^ (r & 7)) << 4);
      sx_cp_async16(full_u32 + dst, fsrc + so, ok ? 16 : 0);
      sx_cp_async16(band_u32 + dst, bsrc + so, ok ? 16 : 0);
    }
    sx_commit();
    // LSEs of the row whose factors this lane works out later (lane r < 16 owns MMA row r):
    // fetched now so that their latency hides behind the tensor-core work
    float l_full = 0.f, l_band = 0.f;
    {
      const int tk = i0 + lane / G;
      if (lane < 16 && tk < sp.keep) {
        const size_t li = static_cast<size_t>(sp.base_off + sp.start + tk) * H + kh * G + (lane % G);
        l_full = load_lse(p.src_lse, a.full_lse_dtype, li);
        l_band = load_lse(a.band_lse, a.band_lse_dtype, li);
      }
    }
    sx_wait<1>();
    __syncwarp();

    // q_pre rows go to the ring as they are; the NaN stamp of q_post_cache too
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = 2 * j + r_half;
      if (i0 + r / G < sp.keep) {
        const uint4 v = *reinterpret_cast<const uint4*>(regA + kSxRegionRows + r * kSxRowBytes + c * 16);
        int d = dbase + r / G;
        if (d >= p.M) d -= p.M;
        const size_t doff = static_cast<size_t>(d) * row_bf16 + head_base + (r % G) * kSxRowBytes;
        st_stream16(qc + doff, v);
        if (pc) st_stream16(pc + doff, nan4);
      }
    }

    // ---- 2. S = Q K^T (k-step outermost: 2 * nkb independent accumulators per step)
    float s[8][2][4];
#pragma unroll
    for (int kb = 0; kb < 8; ++kb)
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) s[kb][nb][0] = s[kb][nb][1] = s[kb][nb][2] = s[kb][nb][3] = 0.f;
    {
      const uint32_t qrow = regA_u32 + (((mi & 1) << 3) + l7) * kSxRowBytes;
      const uint32_t krow = ks_u32 + (((mi >> 1) << 3) + l7) * kSxRowBytes;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t q0, q1, q2, q3;
        sx_ldmatrix_x4(qrow + (((2 * kk + (mi >> 1)) ^ l7) << 4), q0, q1, q2, q3);
        const uint32_t ksw = ((2 * kk + (mi & 1)) ^ l7) << 4;
#pragma unroll
        for (int kb = 0; kb < 8; ++kb) {
          if (kb < nkb) {
            uint32_t b0, b1, b2, b3;
            sx_ldmatrix_x4(krow + kb * 16 * kSxRowBytes + ksw, b0, b1, b2, b3);
            sx_mma(s[kb][0], q0, q1, q2, q3, b0, b1);
            sx_mma(s[kb][1], q0, q1, q2, q3, b2, b3);
          }
        }
      }
    }
    // The staged q rows are dead (q_pre went to the ring above, q_post into S): request the next
    // tile's into the same staging now, a tile's worth of work ahead of their use.
    __syncwarp();
    if (tile + tile_step < ntiles) stage_q_rows(tile + tile_step); else sx_commit();

    // softmax over the F sink keys, log2 domain; keys >= F only exist in the last block
    if (F & 15) {
#pragma unroll
      for (int kb = 0; kb < 8; ++kb)
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            s[kb][nb][e] = kb * 16 + nb * 8 + quad * 2 + (e & 1) >= F ? -INFINITY : s[kb][nb][e];
    }
    float m_lo = -INFINITY, m_hi = -INFINITY;
#pragma unroll
    for (int kb = 0; kb < 8; ++kb) {
      if (kb < nkb) {
        m_lo = fmaxf(m_lo, fmaxf(fmaxf(s[kb][0][0], s[kb][0][1]), fmaxf(s[kb][1][0], s[kb][1][1])));
        m_hi = fmaxf(m_hi, fmaxf(fmaxf(s[kb][0][2], s[kb][0][3]), fmaxf(s[kb][1][2], s[kb][1][3])));
      }
    }
    m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 1));
    m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 2));
    m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 1));
    m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 2));
    // scaled maxima (sm_scale > 0); -inf only when there is no sink key at all
    const float ms_lo = m_lo == -INFINITY ? 0.f : m_lo * scale_log2;
    const float ms_hi = m_hi == -INFINITY ? 0.f : m_hi * scale_log2;
    float sum_lo = 0.f, sum_hi = 0.f;   // fp32 sums of the unrounded weights: the second downdate
                                        // is sensitive to the denominator when the sink holds
                                        // nearly all of a row's mass
    uint32_t pa[8][4];
#pragma unroll
    for (int kb = 0; kb < 8; ++kb) {
      if (kb < nkb) {
        float e[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          e[nb][0] = sx_ex2(fmaf(s[kb][nb][0], scale_log2, -ms_lo));
          e[nb][1] = sx_ex2(fmaf(s[kb][nb][1], scale_log2, -ms_lo));
          e[nb][2] = sx_ex2(fmaf(s[kb][nb][2], scale_log2, -ms_hi));
          e[nb][3] = sx_ex2(fmaf(s[kb][nb][3], scale_log2, -ms_hi));
        }
        sum_lo += (e[0][0] + e[0][1]) + (e[1][0] + e[1][1]);
        sum_hi += (e[0][2] + e[0][3]) + (e[1][2] + e[1][3]);
        pa[kb][0] = pack2(e[0][0], e[0][1]);
        pa[kb][1] = pack2(e[0][2], e[0][3]);
        pa[kb][2] = pack2(e[1][0], e[1][1]);
        pa[kb][3] = pack2(e[1][2], e[1][3]);
      }
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    // O = P V (unnormalised)
    float o[16][4];
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) o[jj][0] = o[jj][1] = o[jj][2] = o[jj][3] = 0.f;
    {
      const uint32_t vrow = vs_u32 + (((mi & 1) << 3) + l7) * kSxRowBytes;
#pragma unroll
      for (int kb = 0; kb < 8; ++kb) {
        if (kb < nkb) {
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            uint32_t b0, b1, b2, b3;
            sx_ldmatrix_x4_trans(vrow + kb * 16 * kSxRowBytes + (((2 * jj + (mi >> 1)) ^ l7) << 4),
                                 b0, b1, b2, b3);
            sx_mma(o[2 * jj], pa[kb][0], pa[kb][1], pa[kb][2], pa[kb][3], b0, b1);
            sx_mma(o[2 * jj + 1], pa[kb][0], pa[kb][1], pa[kb][2], pa[kb][3], b2, b3);
          }
        }
      }
    }

    // ---- 3. both downdates folded into three factors per row, lane r < 16 for MMA row r:
    //   state = full * A - band * B - sink_unnormalised * C
    {
      // row r's scaled maximum and denominator live in the quad 4 * (r & 7): rows 0..7 in
      // the "lo" values, rows 8..15 in the "hi" values
      const int src_lane = (lane & 7) << 2;
      const float ms_a = __shfl_sync(0xffffffffu, ms_lo, src_lane);
      const float ms_b = __shfl_sync(0xffffffffu, ms_hi, src_lane);
      const float su_a = __shfl_sync(0xffffffffu, sum_lo, src_lane);
      const float su_b = __shfl_sync(0xffffffffu, sum_hi, src_lane);
      const int r = lane;
      const int tk = i0 + r / G;
      if (r < 16 && tk < sp.keep) {
        const float ms = (r & 8) ? ms_b : ms_a, sum = (r & 8) ? su_b : su_a;
        const int h = kh * G + (r % G);
        float ret1, t1, s1;
        downdate_scalars(l_full, __fmul_rn(l_band, a.band_lse_scale), ret1, t1, s1);
        int64_t E = pos_base + tk + 1 - a.semantic_pos_ahead;
        if (E < 0) E = 0;
        float ret2 = -INFINITY, fa = 0.f, fb = 0.f, fc = 0.f, empty = 1.f;
        if (E > F) {
          const float lse_sink = sum > 0.f ? (ms + log2f(sum)) * 0.6931471805599453f : -INFINITY;
          float t2, s2;
          downdate_scalars(ret1, lse_sink, ret2, t2, s2);
          fa = s1 * s2;
          fb = t1 * fa;
          fc = sum > 0.f ? t2 * s2 / sum : 0.f;
          empty = 0.f;
        }
        scal[r] = make_float4(fa, fb, fc, empty);
        int d = dbase + r / G;
        if (d >= p.M) d -= p.M;
        lc[static_cast<size_t>(d) * H + h] = ret2;
      }
    }
    // ---- 4. apply the factors where the sink state lies (the accumulators' layout: rows rlo
    // and rhi, columns jj * 8 + quad * 2 + {0, 1}), in place over the staged full rows, then
    // stream the rows to the ring
    sx_wait<1>();   // full and band rows have landed; the next tile's q rows may still be in flight
    __syncwarp();   // and every lane sees them and the row factors
    {
      const float4 klo = scal[rlo], khi = scal[rhi];
      uint8_t* f_lo = fullS + rlo * kSxRowBytes + quad * 4;
      const uint8_t* b_lo = bandS + rlo * kSxRowBytes + quad * 4;
      constexpr int kHi = 8 * kSxRowBytes;   // row rhi = rlo + 8 has the same swizzle (rhi & 7 == rlo)
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const int ch = (jj ^ rlo) << 4;
        uint32_t* fl = reinterpret_cast<uint32_t*>(f_lo + ch);
        uint32_t* fh = reinterpret_cast<uint32_t*>(f_lo + kHi + ch);
        const uint32_t xl = *fl, xh = *fh;
        const uint32_t yl = *reinterpret_cast<const uint32_t*>(b_lo + ch);
        const uint32_t yh = *reinterpret_cast<const uint32_t*>(b_lo + kHi + ch);
        const float l0 = fmaf(lo_f(xl), klo.x, fmaf(-lo_f(yl), klo.y, -(o[jj][0] * klo.z)));
        const float l1 = fmaf(hi_f(xl), klo.x, fmaf(-hi_f(yl), klo.y, -(o[jj][1] * klo.z)));
        const float h0 = fmaf(lo_f(xh), khi.x, fmaf(-lo_f(yh), khi.y, -(o[jj][2] * khi.z)));
        const float h1 = fmaf(hi_f(xh), khi.x, fmaf(-hi_f(yh), khi.y, -(o[jj][3] * khi.z)));
        *fl = klo.w != 0.f ? 0u : pack2(l0, l1);
        *fh = khi.w != 0.f ? 0u : pack2(h0, h1);
      }
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = 2 * j + r_half;
      if (i0 + r / G >= sp.keep) continue;
      const uint4 w4 = *reinterpret_cast<const uint4*>(fullS + r * kSxRowBytes + ((c ^ (r & 7)) << 4));
      int d = dbase + r / G;
      if (d >= p.M) d -= p.M;
      st_stream16(ac + static_cast<size_t>(d) * row_bf16 + head_base + (r % G) * kSxRowBytes, w4);
    }
    __syncwarp();   // the next tile's staging overwrites what other lanes just read
  }
}

// Runs after every CTA of the build kernel has read L_before (stream order):
// bumps request_length in the by-request mode and marks the requests ready
// (mac_prefill_update_cache.cu:262-267 and 374-409).
__global__ void prefill_build_finish_kernel(const MacB200PrefillBuildArgs a) {
  const MacB200PrefillArgs& p = a.ring;
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= p.B) return;
  const int req = p.req_ids[b];
  if (req < 0 || req >= p.R) return;
  if (sink_request_out_of_table(a, req)) return;   // rows were not built: not ready, length kept
  if (a.ready) {
    a.cache_epoch[req] = a.request_epoch[req];
    a.ready[req] = 1;
  }
  if (p.request_length_by_batch) return;
  const int Ni = p.lens[b];
  if (Ni <= 0 || p.M <= 0) return;
  const int base_off = p.offsets[b];
  if (base_off < 0 || base_off + Ni > p.src_rows) return;
  atomicAdd(&p.request_length[req], Ni);
}

}  // namespace

int take_prefill_build_status(unsigned* bits) {
  unsigned v = 0;
  MAC_CUDA(cudaMemcpyFromSymbol(&v, g_build_status, sizeof(v)));
  if (v != 0) {
    const unsigned zero = 0;
    MAC_CUDA(cudaMemcpyToSymbol(g_build_status, &zero, sizeof(zero)));
  }
  unsigned tc = 0;
  if (const int rc = take_prefill_sink_tc_status(&tc)) return rc;
  *bits = v | tc;
  return MAC_B200_OK;
}

}  // namespace mac_b200

using namespace mac_b200;

extern "C" int mac_b200_prefill_downdate_update_cache(const MacB200PrefillBuildArgs* args,
                                                      void* stream_v) {
  MAC_REQUIRE(args != nullptr, "prefill build args must not be null");
  const MacB200PrefillBuildArgs& a = *args;
  const MacB200PrefillArgs& p = a.ring;
  if (p.M <= 0 || p.B <= 0) return MAC_B200_OK;
  MAC_REQUIRE(p.R > 0, "R must be > 0");
  MAC_REQUIRE(p.H > 0 && p.D > 0, "num_heads and head_dim must be > 0");
  MAC_REQUIRE(p.q_cache && p.attn_cache && p.lse_cache, "ring tensors must not be null");
  MAC_REQUIRE(p.request_length && p.req_ids && p.offsets && p.lens,
              "batch metadata must not be null");
  MAC_REQUIRE(p.src_rows == 0 || (p.src_q && p.src_attn && p.src_lse && a.band_attn && a.band_lse),
              "source tensors must not be null");
  MAC_REQUIRE(a.full_lse_dtype >= 0 && a.full_lse_dtype <= 2 && a.band_lse_dtype >= 0 &&
                  a.band_lse_dtype <= 2,
              "lse must be float32, bfloat16, or float16");
  MAC_REQUIRE(a.sink_mode >= MAC_B200_SINK_NONE && a.sink_mode <= MAC_B200_SINK_EXCLUDE,
              "unknown sink_mode");
  const bool gate_any = a.ready || a.cache_epoch || a.request_epoch;
  const bool gate_all = a.ready && a.cache_epoch && a.request_epoch;
  MAC_REQUIRE(!gate_any || gate_all, "ready, cache_epoch and request_epoch go together");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (a.sink_mode == MAC_B200_SINK_EXCLUDE) {
    MAC_REQUIRE(a.q_post && a.k_buffer && a.v_buffer && a.req_to_token,
                "sink-exclusive build needs q_post, k_buffer, v_buffer and req_to_token");
    MAC_REQUIRE(a.Hkv > 0 && p.H % a.Hkv == 0, "H must be divisible by Hkv");
    MAC_REQUIRE(a.front_sink_tokens >= 0 && a.semantic_pos_ahead >= 0, "negative F or S");
    MAC_REQUIRE(a.req_to_token_rows > 0 && a.req_to_token_stride >= a.front_sink_tokens,
                "req_to_token has fewer columns than front_sink_tokens");
    const int G = p.H / a.Hkv;
    if (p.D != kSxD)
      return fail(MAC_B200_EUNSUPPORTED, "sink-exclusive build supports D=128 only (got %d)", p.D);
    if (a.front_sink_tokens > kSxMaxF)
      return fail(MAC_B200_EUNSUPPORTED, "front_sink_tokens=%d exceeds this build's limit of %d",
                  a.front_sink_tokens, kSxMaxF);
    if (G > 16 || (16 % G) != 0)
      return fail(MAC_B200_EUNSUPPORTED, "sink-exclusive build needs a GQA group of 1, 2, 4, 8 or 16");
    const uintptr_t bits = reinterpret_cast<uintptr_t>(p.q_cache) | reinterpret_cast<uintptr_t>(p.attn_cache) |
                           reinterpret_cast<uintptr_t>(p.q_post_cache) | reinterpret_cast<uintptr_t>(p.src_q) |
                           reinterpret_cast<uintptr_t>(p.src_attn) | reinterpret_cast<uintptr_t>(a.band_attn) |
                           reinterpret_cast<uintptr_t>(a.q_post) | reinterpret_cast<uintptr_t>(a.k_buffer) |
                           reinterpret_cast<uintptr_t>(a.v_buffer);
    MAC_REQUIRE((bits & 15u) == 0, "sink-exclusive build needs 16-byte aligned tensors");
    MAC_REQUIRE(a.sm_scale > 0.f, "sm_scale must be positive");
    int device = 0;
    MAC_CUDA(cudaGetDevice(&device));
    void (*kernel)(MacB200PrefillBuildArgs) =
        G == 1 ? prefill_sink_exclusive_ring_kernel<1>
        : G == 2 ? prefill_sink_exclusive_ring_kernel<2>
        : G == 4 ? prefill_sink_exclusive_ring_kernel<4>
        : G == 8 ? prefill_sink_exclusive_ring_kernel<8>
                 : prefill_sink_exclusive_ring_kernel<16>;
    // the attribute is per device: set it on every call (cheap, no synchronisation)
    MAC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSxSmemBytes));
    const int sms = device_sm_count(device);
    // MAC_B200_SINK_KERNEL=tcgen05 takes the tensor-memory kernel (mac_b200_prefill_sink_tc.cu)
    if (const char* k = std::getenv("MAC_B200_SINK_KERNEL")) {
      if (k[0] == 't') {
        bool launched = false;
        if (const int rc = launch_prefill_sink_exclusive_tc(a, sms, stream, &launched)) return rc;
        if (launched) {
          if (!p.request_length_by_batch || a.ready) {
            prefill_build_finish_kernel<<<(p.B + 127) / 128, 128, 0, stream>>>(a);
            MAC_CUDA(cudaGetLastError());
            g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
          }
          return MAC_B200_OK;
        }
      }
    }
    const int TG = 16 / G;
    const int max_tiles = ((p.M < 1 ? 1 : p.M) + TG - 1) / TG;
    const int pairs = p.B * a.Hkv;
    // Slices per (request, KV head): between three and eight CTAs per SM in all, and among
    // those the count that leaves the last wave fullest (fewest slices on a tie: every CTA
    // reloads the sink K/V).  MAC_B200_SINK_SLICES overrides it for tuning.
    const int max_slices = (max_tiles + kSxWarps - 1) / kSxWarps;
    int lo = (3 * sms + pairs - 1) / pairs, hi = (8 * sms + pairs - 1) / pairs;
    if (lo < 1) lo = 1;
    if (hi > max_slices) hi = max_slices;
    if (lo > hi) lo = hi;
    int slices = lo;
    double best = -1.0;
    for (int sl = lo; sl <= hi; ++sl) {
      const long long total = static_cast<long long>(sl) * pairs;
      const long long waves = (total + sms - 1) / sms;
      const double eff = static_cast<double>(total) / static_cast<double>(waves * sms);
      if (eff > best + 1e-9) { best = eff; slices = sl; }
    }
    if (const char* e = std::getenv("MAC_B200_SINK_SLICES")) {
      const int v = std::atoi(e);
      if (v >= 1 && v <= max_slices) slices = v;
    }
    if (slices < 1) slices = 1;
    dim3 grid(slices, a.Hkv, p.B);
    kernel<<<grid, kSxThreads, kSxSmemBytes, stream>>>(a);
    MAC_CUDA(cudaGetLastError());
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    if (!p.request_length_by_batch || a.ready) {
      prefill_build_finish_kernel<<<(p.B + 127) / 128, 128, 0, stream>>>(a);
      MAC_CUDA(cudaGetLastError());
      g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return MAC_B200_OK;
  }
  int per_req = (p.M + 1) / 2 < 64 ? (p.M + 1) / 2 : 64;
  if (p.B >= 32 && per_req > 32) per_req = 32;
  if (per_req < 1) per_req = 1;
  dim3 grid(per_req, p.B);
  prefill_downdate_ring_kernel<<<grid, kBuildThreads, 0, stream>>>(a);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  if (!p.request_length_by_batch || a.ready) {
    prefill_build_finish_kernel<<<(p.B + 127) / 128, 128, 0, stream>>>(a);
    MAC_CUDA(cudaGetLastError());
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  }
  return MAC_B200_OK;
}
