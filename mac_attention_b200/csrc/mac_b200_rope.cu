// Decode-time fused "preserve pre-RoPE q + RoPE(q, k) + KV-pool write" (sm_100a).
//
// Per decode token n: q_pre[n] <- q[n] (before rotation), q[n] and k[n] are
// rotated in place with the (cos | sin) row of positions[n], the rotated k and
// the untouched v are scattered into the KV pool at row cache_locs[n].
// Semantics follow the reference operator
// attention/src/mac_attention/integrations/sglang/csrc/mac_decode_rope_preserve.cu:35-156, 174-269.
// The reference assigns one element pair per thread and walks five task
// classes with a grid-stride loop; here one thread owns a 16-byte chunk (8 bf16)
// of a head together with its rotation partner chunk, every global access is a
// 16-byte vector, and the three roles (q heads, k heads, v heads) are spread
// over the grid so the whole step is one wave of small CTAs.
#include <cuda_bf16.h>

#include "mac_b200_common.h"

namespace mac_b200 {
namespace {

constexpr int kRopeThreads = 128;

__device__ __forceinline__ float lo_f(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float hi_f(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// y0 = x0*c - x1*s, y1 = x1*c + x0*s, evaluated as the reference's compiler
// evaluates them: one product rounded, the other fused into the add.
__device__ __forceinline__ void rotate(float x0, float x1, float c, float s, float& y0, float& y1) {
  y0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
  y1 = __fmaf_rn(x1, c, __fmul_rn(x0, s));
}

__device__ __forceinline__ int64_t load_index(const void* p, int is_i64, int64_t n) {
  return is_i64 ? static_cast<const int64_t*>(p)[n]
                : static_cast<int64_t>(static_cast<const int32_t*>(p)[n]);
}

// One work unit = (token, head of q|k|v, chunk).  For rotated dims under the
// NeoX layout a unit covers chunk c of the first half and chunk c of the second
// half (partners d and d + rotary_dim/2); under the interleaved layout and for
// pass-through dims and v it covers one chunk.
__global__ void __launch_bounds__(kRopeThreads)
rope_preserve_vec_kernel(const MacB200RopeArgs a) {
  const int D = a.head_dim, R = a.rotary_dim, half = R >> 1;
  const int heads = a.Hq + 2 * a.Hkv;
  const int rot_units = a.is_neox ? half / 8 : R / 8;
  const int pass_units = (D - R) / 8;
  const int units_qk = rot_units + pass_units;     // per q or k head
  const int units_v = D / 8;
  const int64_t per_token = static_cast<int64_t>(a.Hq + a.Hkv) * units_qk +
                            static_cast<int64_t>(a.Hkv) * units_v;
  const int64_t total = a.N * per_token;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= total) return;
  (void)heads;
  const int64_t n = t / per_token;
  int64_t r = t - n * per_token;
  const int64_t q_units = static_cast<int64_t>(a.Hq) * units_qk;
  const int64_t k_units = static_cast<int64_t>(a.Hkv) * units_qk;

  if (r >= q_units + k_units) {                    // ---- v head: copy into the pool
    r -= q_units + k_units;
    const int h = static_cast<int>(r / units_v), c = static_cast<int>(r - static_cast<int64_t>(h) * units_v);
    const int64_t loc = load_index(a.cache_locs, a.cache_locs_i64, n);
    if (loc < 0 || loc >= a.kv_pool_tokens) return;
    const uint4 v = *reinterpret_cast<const uint4*>(
        static_cast<const char*>(a.v) + (n * a.v_stride0 + static_cast<int64_t>(h) * D + c * 8) * 2);
    *reinterpret_cast<uint4*>(static_cast<char*>(a.v_buffer) +
                              ((loc * a.Hkv + h) * D + c * 8) * 2) = v;
    return;
  }
  const bool is_k = r >= q_units;
  if (is_k) r -= q_units;
  const int h = static_cast<int>(r / units_qk);
  const int u = static_cast<int>(r - static_cast<int64_t>(h) * units_qk);
  char* row = is_k ? static_cast<char*>(a.k) + (n * a.k_stride0 + static_cast<int64_t>(h) * D) * 2
                   : static_cast<char*>(a.q) + (n * a.q_stride0 + static_cast<int64_t>(h) * D) * 2;
  char* pre = is_k ? nullptr
                   : static_cast<char*>(a.q_pre) + ((n * a.Hq + h) * static_cast<int64_t>(D)) * 2;
  char* pool = nullptr;
  if (is_k) {
    const int64_t loc = load_index(a.cache_locs, a.cache_locs_i64, n);
    if (loc >= 0 && loc < a.kv_pool_tokens)
      pool = static_cast<char*>(a.k_buffer) + ((loc * a.Hkv + h) * static_cast<int64_t>(D)) * 2;
  }
  if (u >= rot_units) {                            // ---- pass-through dims
    const int d = R + (u - rot_units) * 8;
    const uint4 x = *reinterpret_cast<const uint4*>(row + d * 2);
    if (pre) *reinterpret_cast<uint4*>(pre + d * 2) = x;
    if (pool) *reinterpret_cast<uint4*>(pool + d * 2) = x;
    return;
  }
  const int64_t pos = load_index(a.positions, a.positions_i64, n);
  const float* cs = a.cos_sin_cache + pos * a.cos_sin_stride0;
  if (a.is_neox) {
    const int d0 = u * 8, d1 = half + u * 8;
    const uint4 x0 = *reinterpret_cast<const uint4*>(row + d0 * 2);
    const uint4 x1 = *reinterpret_cast<const uint4*>(row + d1 * 2);
    if (pre) {
      *reinterpret_cast<uint4*>(pre + d0 * 2) = x0;
      *reinterpret_cast<uint4*>(pre + d1 * 2) = x1;
    }
    const float4 c0 = *reinterpret_cast<const float4*>(cs + d0), c1 = *reinterpret_cast<const float4*>(cs + d0 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + half + d0),
                 s1 = *reinterpret_cast<const float4*>(cs + half + d0 + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t a0[4] = {x0.x, x0.y, x0.z, x0.w}, a1[4] = {x1.x, x1.y, x1.z, x1.w};
    uint32_t y0[4], y1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float p0, p1, q0, q1;
      rotate(lo_f(a0[i]), lo_f(a1[i]), c[2 * i], s[2 * i], p0, p1);
      rotate(hi_f(a0[i]), hi_f(a1[i]), c[2 * i + 1], s[2 * i + 1], q0, q1);
      y0[i] = pack2(p0, q0);
      y1[i] = pack2(p1, q1);
    }
    const uint4 o0 = make_uint4(y0[0], y0[1], y0[2], y0[3]);
    const uint4 o1 = make_uint4(y1[0], y1[1], y1[2], y1[3]);
    *reinterpret_cast<uint4*>(row + d0 * 2) = o0;
    *reinterpret_cast<uint4*>(row + d1 * 2) = o1;
    if (pool) {
      *reinterpret_cast<uint4*>(pool + d0 * 2) = o0;
      *reinterpret_cast<uint4*>(pool + d1 * 2) = o1;
    }
  } else {                                         // interleaved pairs (2p, 2p+1)
    const int d0 = u * 8, p0i = d0 >> 1;
    const uint4 x = *reinterpret_cast<const uint4*>(row + d0 * 2);
    if (pre) *reinterpret_cast<uint4*>(pre + d0 * 2) = x;
    const float4 c = *reinterpret_cast<const float4*>(cs + p0i);
    const float4 s = *reinterpret_cast<const float4*>(cs + half + p0i);
    const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
    const uint32_t xa[4] = {x.x, x.y, x.z, x.w};
    uint32_t y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float r0, r1;
      rotate(lo_f(xa[i]), hi_f(xa[i]), cc[i], ss[i], r0, r1);
      y[i] = pack2(r0, r1);
    }
    const uint4 o = make_uint4(y[0], y[1], y[2], y[3]);
    *reinterpret_cast<uint4*>(row + d0 * 2) = o;
    if (pool) *reinterpret_cast<uint4*>(pool + d0 * 2) = o;
  }
}

// Element-pair fallback for shapes or alignments the vector kernel cannot take
// (head_dim or rotary_dim not multiples of 8/16, odd strides, unaligned bases).
__global__ void __launch_bounds__(kRopeThreads)
rope_preserve_scalar_kernel(const MacB200RopeArgs a) {
  const int64_t D = a.head_dim, R = a.rotary_dim, half = R >> 1;
  const int64_t q_pair = a.N * a.Hq * half, k_pair = a.N * a.Hkv * half;
  const int64_t q_pass = a.N * a.Hq * (D - R), k_pass = a.N * a.Hkv * (D - R);
  const int64_t v_tot = a.N * a.Hkv * D;
  const int64_t total = q_pair + k_pair + q_pass + k_pass + v_tot;
  __nv_bfloat16* q = static_cast<__nv_bfloat16*>(a.q);
  __nv_bfloat16* k = static_cast<__nv_bfloat16*>(a.k);
  const __nv_bfloat16* v = static_cast<const __nv_bfloat16*>(a.v);
  __nv_bfloat16* q_pre = static_cast<__nv_bfloat16*>(a.q_pre);
  __nv_bfloat16* kb = static_cast<__nv_bfloat16*>(a.k_buffer);
  __nv_bfloat16* vb = static_cast<__nv_bfloat16*>(a.v_buffer);
  for (int64_t task = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; task < total;
       task += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t t = task;
    if (t < q_pair + k_pair) {
      const bool is_k = t >= q_pair;
      if (is_k) t -= q_pair;
      const int64_t H = is_k ? a.Hkv : a.Hq;
      const int64_t pair = t % half, tmp = t / half, h = tmp % H, n = tmp / H;
      const int64_t pos = load_index(a.positions, a.positions_i64, n);
      const float* cs = a.cos_sin_cache + pos * a.cos_sin_stride0;
      const int64_t d0 = a.is_neox ? pair : (pair << 1), d1 = a.is_neox ? pair + half : d0 + 1;
      __nv_bfloat16* row = is_k ? k + n * a.k_stride0 + h * D : q + n * a.q_stride0 + h * D;
      const __nv_bfloat16 b0 = row[d0], b1 = row[d1];
      if (!is_k) {
        q_pre[(n * a.Hq + h) * D + d0] = b0;
        q_pre[(n * a.Hq + h) * D + d1] = b1;
      }
      float y0, y1;
      rotate(__bfloat162float(b0), __bfloat162float(b1), cs[pair], cs[half + pair], y0, y1);
      const __nv_bfloat16 o0 = __float2bfloat16_rn(y0), o1 = __float2bfloat16_rn(y1);
      row[d0] = o0;
      row[d1] = o1;
      if (is_k) {
        const int64_t loc = load_index(a.cache_locs, a.cache_locs_i64, n);
        if (loc >= 0 && loc < a.kv_pool_tokens) {
          kb[(loc * a.Hkv + h) * D + d0] = o0;
          kb[(loc * a.Hkv + h) * D + d1] = o1;
        }
      }
      continue;
    }
    t -= q_pair + k_pair;
    if (t < q_pass) {
      const int64_t d = R + t % (D - R), tmp = t / (D - R), h = tmp % a.Hq, n = tmp / a.Hq;
      q_pre[(n * a.Hq + h) * D + d] = q[n * a.q_stride0 + h * D + d];
      continue;
    }
    t -= q_pass;
    if (t < k_pass) {
      const int64_t d = R + t % (D - R), tmp = t / (D - R), h = tmp % a.Hkv, n = tmp / a.Hkv;
      const int64_t loc = load_index(a.cache_locs, a.cache_locs_i64, n);
      if (loc >= 0 && loc < a.kv_pool_tokens)
        kb[(loc * a.Hkv + h) * D + d] = k[n * a.k_stride0 + h * D + d];
      continue;
    }
    t -= k_pass;
    const int64_t d = t % D, tmp = t / D, h = tmp % a.Hkv, n = tmp / a.Hkv;
    const int64_t loc = load_index(a.cache_locs, a.cache_locs_i64, n);
    if (loc >= 0 && loc < a.kv_pool_tokens)
      vb[(loc * a.Hkv + h) * D + d] = v[n * a.v_stride0 + h * D + d];
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace mac_b200

using namespace mac_b200;

extern "C" int mac_b200_decode_rope_preserve_q_bf16(const MacB200RopeArgs* args, void* stream_v) {
  MAC_REQUIRE(args != nullptr, "rope args must not be null");
  const MacB200RopeArgs& a = *args;
  MAC_REQUIRE(a.N >= 0, "negative batch");
  MAC_REQUIRE(a.head_dim > 0 && a.Hq > 0 && a.Hkv > 0, "invalid head_dim");
  MAC_REQUIRE(a.rotary_dim > 0 && a.rotary_dim <= a.head_dim && (a.rotary_dim % 2) == 0,
              "invalid rotary_dim");
  if (a.N == 0) return MAC_B200_OK;
  MAC_REQUIRE(a.q && a.k && a.v && a.q_pre && a.k_buffer && a.v_buffer && a.cos_sin_cache &&
                  a.positions && a.cache_locs,
              "rope tensors must not be null");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int D = a.head_dim, R = a.rotary_dim;
  const bool vec = D % 8 == 0 && R % (a.is_neox ? 16 : 8) == 0 && a.q_stride0 % 8 == 0 &&
                   a.k_stride0 % 8 == 0 && a.v_stride0 % 8 == 0 && a.cos_sin_stride0 % 4 == 0 &&
                   aligned16(a.q) && aligned16(a.k) && aligned16(a.v) && aligned16(a.q_pre) &&
                   aligned16(a.k_buffer) && aligned16(a.v_buffer) && aligned16(a.cos_sin_cache);
  if (vec) {
    const int rot_units = a.is_neox ? (R / 2) / 8 : R / 8;
    const int units_qk = rot_units + (D - R) / 8;
    const int64_t per_token = static_cast<int64_t>(a.Hq + a.Hkv) * units_qk +
                              static_cast<int64_t>(a.Hkv) * (D / 8);
    const int64_t total = a.N * per_token;
    const int64_t blocks = (total + kRopeThreads - 1) / kRopeThreads;
    MAC_REQUIRE(blocks < (int64_t(1) << 31), "rope problem too large");
    rope_preserve_vec_kernel<<<static_cast<unsigned>(blocks), kRopeThreads, 0, stream>>>(a);
  } else {
    const int64_t total = a.N * (static_cast<int64_t>(a.Hq + a.Hkv) * (D - R / 2) +
                                 static_cast<int64_t>(a.Hkv) * D);
    int64_t blocks = (total + kRopeThreads - 1) / kRopeThreads;
    int device = 0;
    MAC_CUDA(cudaGetDevice(&device));
    const int64_t max_blocks = static_cast<int64_t>(device_sm_count(device)) * 16;
    if (blocks > max_blocks) blocks = max_blocks;
    if (blocks < 1) blocks = 1;
    rope_preserve_scalar_kernel<<<static_cast<unsigned>(blocks), kRopeThreads, 0, stream>>>(a);
  }
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return MAC_B200_OK;
}
