// Prefill-side ring build and readiness-gate kernels (sm_100a).
//
// mac_b200_prefill_update_cache copies the last min(len, M) rows of each
// request's (pre-RoPE query, prefix attention state, LSE) into that request's
// ring at slot (L_before + start + i) mod M, optionally stamps the matching
// rows of q_post_cache with the bf16 NaN sentinel 0x7fc0, and (when
// request_length is indexed by request) bumps request_length[req] by len.
// Semantics follow the reference operator
// attention/src/mac_attention/integrations/sglang/csrc/mac_prefill_update_cache.cu:201-269;
// the launch geometry does not.  The reference walks each request's rows with
// ONE CTA; here the rows of a request are spread over many CTAs so that a
// handful of long prompts still saturates HBM, every access is a 16-byte
// streaming load/store, and the request_length bump runs as a second tiny
// kernel so it cannot race the reads of L_before.
#include "mac_b200_common.h"
#include "mac_b200_state_math.cuh"

namespace mac_b200 {
namespace {

constexpr int kCopyThreads = 256;

struct PrefillParams {
  MacB200PrefillArgs a;
  int ctas_per_request;
};

// Copies `bytes` from src to dst with 16-byte vectors when both are aligned,
// else with the widest unit that divides everything.
__device__ __forceinline__ void copy_row(uint8_t* dst, const uint8_t* src, size_t bytes) {
  const bool vec = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) &
                    15u) == 0;
  if (vec) {
    for (size_t i = threadIdx.x; i < bytes / 16; i += blockDim.x)
      st_stream16(dst + i * 16, ld_stream16(src + i * 16));
  } else if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 3u) ==
             0) {
    for (size_t i = threadIdx.x; i < bytes / 4; i += blockDim.x)
      reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
  } else {
    for (size_t i = threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
  }
}

__device__ __forceinline__ void fill_row_u16(uint8_t* dst, size_t bytes, uint16_t pattern) {
  const uint32_t w = (static_cast<uint32_t>(pattern) << 16) | pattern;
  if (((reinterpret_cast<uintptr_t>(dst) | bytes) & 15u) == 0) {
    const uint4 v = make_uint4(w, w, w, w);
    for (size_t i = threadIdx.x; i < bytes / 16; i += blockDim.x) st_stream16(dst + i * 16, v);
  } else {
    for (size_t i = threadIdx.x; i < bytes / 2; i += blockDim.x)
      reinterpret_cast<uint16_t*>(dst)[i] = pattern;
  }
}

// grid = (ctas_per_request, B); CTA x of request b copies rows x, x+gridDim.x, ...
__global__ void __launch_bounds__(kCopyThreads, 3)
prefill_ring_copy_kernel(const PrefillParams pp) {
  const MacB200PrefillArgs& p = pp.a;
  const int b = blockIdx.y;
  const int req = p.req_ids[b];
  const int Ni = p.lens[b];
  if (Ni <= 0 || p.M <= 0) return;
  if (req < 0 || req >= p.R) return;
  const int start = Ni > p.M ? Ni - p.M : 0;
  const int keep = Ni - start;
  const int base_off = p.offsets[b];
  if (base_off < 0 || base_off + Ni > p.src_rows) return;
  int L_before = p.request_length_by_batch ? p.request_length[b] : p.request_length[req];
  if (L_before < 0) L_before = 0;
  const int base_dest = static_cast<int>((static_cast<int64_t>(L_before) + start) % p.M);

  const size_t row_bf16 = static_cast<size_t>(p.H) * p.D * 2;
  const size_t row_f32 = static_cast<size_t>(p.H) * 4;
  uint8_t* qc = static_cast<uint8_t*>(p.q_cache) + static_cast<size_t>(req) * p.M * row_bf16;
  uint8_t* ac = static_cast<uint8_t*>(p.attn_cache) + static_cast<size_t>(req) * p.M * row_bf16;
  uint8_t* lc = reinterpret_cast<uint8_t*>(p.lse_cache) + static_cast<size_t>(req) * p.M * row_f32;
  uint8_t* pc = p.q_post_cache
                    ? static_cast<uint8_t*>(p.q_post_cache) + static_cast<size_t>(req) * p.M * row_bf16
                    : nullptr;
  const uint8_t* qs = static_cast<const uint8_t*>(p.src_q);
  const uint8_t* as = static_cast<const uint8_t*>(p.src_attn);
  const uint8_t* ls = reinterpret_cast<const uint8_t*>(p.src_lse);

  const bool vec = ((reinterpret_cast<uintptr_t>(qc) | reinterpret_cast<uintptr_t>(ac) |
                     reinterpret_cast<uintptr_t>(qs) | reinterpret_cast<uintptr_t>(as) |
                     reinterpret_cast<uintptr_t>(pc) | row_bf16) & 15u) == 0;
  if (vec) {
    // Two ring rows per pass: all 16-byte loads of a pass (two chunks of q and
    // of the state for both rows) are issued before the first store, so a
    // thread keeps up to 128 bytes in flight.
    const size_t chunks = row_bf16 / 16;
    for (int i = 2 * blockIdx.x; i < keep; i += 2 * gridDim.x) {
      const bool two = i + 1 < keep;
      int d0 = base_dest + i;
      if (d0 >= p.M) d0 -= p.M;
      int d1 = d0 + 1;
      if (d1 >= p.M) d1 -= p.M;
      const size_t s0 = static_cast<size_t>(base_off + start + i), s1 = s0 + 1;
      // LSE rows of the pair: one float per thread, loaded before the row chunks so that
      // all of a pass's loads are in flight together
      float lse_v[2] = {0.f, 0.f};
      const int lse_n = (two ? 2 : 1) * p.H;
      const bool lse_small = lse_n <= 2 * static_cast<int>(blockDim.x);
      if (lse_small) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int idx = threadIdx.x + k * blockDim.x;
          if (idx < lse_n)
            lse_v[k] = p.src_lse[(idx >= p.H ? s1 : s0) * p.H + (idx >= p.H ? idx - p.H : idx)];
        }
      }
      for (size_t c = threadIdx.x; c < chunks; c += 2 * blockDim.x) {
        const size_t c2 = c + blockDim.x;
        const bool more = c2 < chunks;
        uint4 q00 = ld_stream16(qs + s0 * row_bf16 + c * 16);
        uint4 a00 = ld_stream16(as + s0 * row_bf16 + c * 16);
        uint4 q01 = q00, a01 = a00, q10 = q00, a10 = a00, q11 = q00, a11 = a00;
        if (more) {
          q01 = ld_stream16(qs + s0 * row_bf16 + c2 * 16);
          a01 = ld_stream16(as + s0 * row_bf16 + c2 * 16);
        }
        if (two) {
          q10 = ld_stream16(qs + s1 * row_bf16 + c * 16);
          a10 = ld_stream16(as + s1 * row_bf16 + c * 16);
          if (more) {
            q11 = ld_stream16(qs + s1 * row_bf16 + c2 * 16);
            a11 = ld_stream16(as + s1 * row_bf16 + c2 * 16);
          }
        }
        const uint32_t nanw = 0x7fc07fc0u;
        const uint4 nan4 = make_uint4(nanw, nanw, nanw, nanw);
        st_stream16(qc + d0 * row_bf16 + c * 16, q00);
        st_stream16(ac + d0 * row_bf16 + c * 16, a00);
        if (pc) st_stream16(pc + d0 * row_bf16 + c * 16, nan4);
        if (more) {
          st_stream16(qc + d0 * row_bf16 + c2 * 16, q01);
          st_stream16(ac + d0 * row_bf16 + c2 * 16, a01);
          if (pc) st_stream16(pc + d0 * row_bf16 + c2 * 16, nan4);
        }
        if (two) {
          st_stream16(qc + d1 * row_bf16 + c * 16, q10);
          st_stream16(ac + d1 * row_bf16 + c * 16, a10);
          if (pc) st_stream16(pc + d1 * row_bf16 + c * 16, nan4);
          if (more) {
            st_stream16(qc + d1 * row_bf16 + c2 * 16, q11);
            st_stream16(ac + d1 * row_bf16 + c2 * 16, a11);
            if (pc) st_stream16(pc + d1 * row_bf16 + c2 * 16, nan4);
          }
        }
      }
      if (lse_small) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int idx = threadIdx.x + k * blockDim.x;
          if (idx < lse_n)
            p.lse_cache[(static_cast<size_t>(req) * p.M + (idx >= p.H ? d1 : d0)) * p.H +
                        (idx >= p.H ? idx - p.H : idx)] = lse_v[k];
        }
      } else {
        copy_row(lc + d0 * row_f32, ls + s0 * row_f32, row_f32);
        if (two) copy_row(lc + d1 * row_f32, ls + s1 * row_f32, row_f32);
      }
    }
    return;
  }
  for (int i = blockIdx.x; i < keep; i += gridDim.x) {
    int dest = base_dest + i;
    if (dest >= p.M) dest -= p.M;
    const size_t src_row = static_cast<size_t>(base_off + start + i);
    copy_row(qc + dest * row_bf16, qs + src_row * row_bf16, row_bf16);
    copy_row(ac + dest * row_bf16, as + src_row * row_bf16, row_bf16);
    copy_row(lc + dest * row_f32, ls + src_row * row_f32, row_f32);
    if (pc) fill_row_u16(pc + dest * row_bf16, row_bf16, 0x7fc0);
  }
}

// Second launch of the legacy mode: request_length[req] += len, after every
// copy CTA of the first launch has read L_before (stream order).
__global__ void prefill_bump_length_kernel(const MacB200PrefillArgs p) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= p.B) return;
  const int req = p.req_ids[b];
  const int Ni = p.lens[b];
  if (Ni <= 0 || p.M <= 0) return;
  if (req < 0 || req >= p.R) return;
  const int base_off = p.offsets[b];
  if (base_off < 0 || base_off + Ni > p.src_rows) return;
  atomicAdd(&p.request_length[req], Ni);
}

__global__ void mark_ready_kernel(uint8_t* ready, int64_t* cache_epoch,
                                  const int64_t* request_epoch, const int32_t* req_ids, int B,
                                  int R) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const int req = req_ids[i];
  if (req < 0 || req >= R) return;
  cache_epoch[req] = request_epoch[req];
  ready[req] = 1;
}

__global__ void invalidate_ready_kernel(uint8_t* ready, int64_t* cache_epoch,
                                        int64_t* request_epoch, const int32_t* req_ids, int B,
                                        int R) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const int req = req_ids[i];
  if (req < 0 || req >= R) return;
  ready[req] = 0;
  cache_epoch[req] = -1;
  request_epoch[req] += 1;
}

__global__ void update_request_state_kernel(int32_t* req_len, int32_t* match_req_len,
                                            int32_t* cache_lens, const int32_t* req_ids,
                                            const int32_t* seq_lens, const int32_t* cur_lens,
                                            int B, int R) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const int32_t seq = seq_lens[i];
  int32_t cache_len = seq - cur_lens[i];
  if (cache_len < 0) cache_len = 0;
  cache_lens[i] = cache_len;
  const int req = req_ids[i];
  if (req < 0 || req >= R) return;
  req_len[req] = seq;
  match_req_len[req] = cache_len;
}

}  // namespace
}  // namespace mac_b200

using namespace mac_b200;

extern "C" int mac_b200_prefill_update_cache(const MacB200PrefillArgs* a, void* stream_v) {
  MAC_REQUIRE(a != nullptr, "prefill args must not be null");
  if (a->M <= 0 || a->B <= 0) return MAC_B200_OK;  // reference: silent no-op
  MAC_REQUIRE(a->R > 0, "R must be > 0");
  MAC_REQUIRE(a->H > 0 && a->D > 0, "num_heads and head_dim must be > 0");
  MAC_REQUIRE(a->q_cache && a->attn_cache && a->lse_cache, "ring tensors must not be null");
  MAC_REQUIRE(a->request_length && a->req_ids && a->offsets && a->lens,
              "batch metadata must not be null");
  MAC_REQUIRE(a->src_rows == 0 || (a->src_q && a->src_attn && a->src_lse),
              "source tensors must not be null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  PrefillParams pp;
  pp.a = *a;
  // Enough CTAs per request that one long prompt alone covers the machine,
  // few enough that 64 requests do not queue tens of thousands of idle CTAs.
  int per_req = (a->M + 1) / 2 < 64 ? (a->M + 1) / 2 : 64;
  if (a->B >= 32 && per_req > 32) per_req = 32;
  if (per_req < 1) per_req = 1;
  pp.ctas_per_request = per_req;
  dim3 grid(per_req, a->B);
  prefill_ring_copy_kernel<<<grid, kCopyThreads, 0, stream>>>(pp);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  if (!a->request_length_by_batch) {
    prefill_bump_length_kernel<<<(a->B + 127) / 128, 128, 0, stream>>>(*a);
    MAC_CUDA(cudaGetLastError());
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  }
  return MAC_B200_OK;
}

extern "C" int mac_b200_mark_persistent_ready(uint8_t* ready, int64_t* cache_epoch,
                                              const int64_t* request_epoch,
                                              const int32_t* req_ids, int32_t B, int32_t R,
                                              void* stream_v) {
  if (B <= 0) return MAC_B200_OK;
  MAC_REQUIRE(ready && cache_epoch && request_epoch && req_ids, "gate tensors must not be null");
  mark_ready_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream_v)>>>(
      ready, cache_epoch, request_epoch, req_ids, B, R);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return MAC_B200_OK;
}

extern "C" int mac_b200_invalidate_persistent_ready(uint8_t* ready, int64_t* cache_epoch,
                                                    int64_t* request_epoch,
                                                    const int32_t* req_ids, int32_t B, int32_t R,
                                                    void* stream_v) {
  if (B <= 0) return MAC_B200_OK;
  MAC_REQUIRE(ready && cache_epoch && request_epoch && req_ids, "gate tensors must not be null");
  invalidate_ready_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream_v)>>>(
      ready, cache_epoch, request_epoch, req_ids, B, R);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return MAC_B200_OK;
}

extern "C" int mac_b200_update_request_state(int32_t* req_len, int32_t* match_req_len,
                                             int32_t* cache_lens, const int32_t* req_ids,
                                             const int32_t* seq_lens, const int32_t* cur_lens,
                                             int32_t B, int32_t R, void* stream_v) {
  if (B <= 0) return MAC_B200_OK;
  MAC_REQUIRE(req_len && match_req_len && cache_lens && req_ids && seq_lens && cur_lens,
              "request-state tensors must not be null");
  update_request_state_kernel<<<(B + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream_v)>>>(
      req_len, match_req_len, cache_lens, req_ids, seq_lens, cur_lens, B, R);
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return MAC_B200_OK;
}
