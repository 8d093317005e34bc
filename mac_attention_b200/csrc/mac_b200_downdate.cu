// Prefill-side LSE downdate, in place (sm_100a).
//
// For every (token, head) row: the state of the whole prefix (out1, lse1) minus
// the state of the trailing window (out2, lse2) gives the state of the prefix
// without that window, written over (out2, lse2).  Formula and guards follow the
// reference kernel
// attention/src/mac_attention/integrations/sglang/csrc/mac_merge_downdate_cache.cu:116-288.
// The reference spends one 256-thread CTA with a double-buffered shared-memory
// stage on each 256-byte row; here a row is a handful of 16-byte chunks owned by
// neighbouring lanes (16 lanes for D = 128); the scalars of the 8..32 rows a warp
// handles per pass are worked out one row per lane and handed to the chunk lanes
// by shuffle, and each thread keeps four rows in flight.
#include "mac_b200_common.h"
#include "mac_b200_state_math.cuh"

namespace mac_b200 {
namespace {

constexpr int kDownThreads = 256;
constexpr int kDownUnroll = 4;

struct DowndateParams {
  const char* out1;
  char* out2;
  const void* lse1;
  void* lse2;
  int64_t rows;
  int32_t D, chunks, lanes_per_row, unroll, dt1, dt2;
};

__global__ void __launch_bounds__(kDownThreads)
downdate_inplace_kernel(const DowndateParams p) {
  const int lpr = p.lanes_per_row;                   // power of two <= 32
  const int lane = threadIdx.x & 31;
  const int sub = lane & (lpr - 1);                  // chunk lane inside the row group
  const int rows_per_warp = 32 / lpr;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t row_bytes = static_cast<int64_t>(p.D) * 2;

  const int unroll = p.unroll;                             // <= kDownUnroll, and such that
  const int rows_per_iter = rows_per_warp * unroll;        // <= 32: one lane per row for the scalars
  for (int64_t base = warp_global * rows_per_iter; base < p.rows; base += warps_total * rows_per_iter) {
    // lane r works out the three scalars of row base + r (all lanes busy), the
    // chunk lanes fetch them by shuffle; the row's LSE is replaced right away
    // (only this lane reads it).
    float my_t = 0.f, my_scale = 0.f;
    {
      const int64_t row = base + lane;
      if (lane < rows_per_iter && row < p.rows) {
        float ret;
        downdate_scalars(load_lse(p.lse1, p.dt1, row), load_lse(p.lse2, p.dt2, row), ret, my_t,
                         my_scale);
        store_lse(p.lse2, p.dt2, row, ret);
      }
    }
    for (int c0 = 0; c0 < p.chunks; c0 += lpr) {
      const int c = c0 + sub;
      uint4 a[kDownUnroll], b[kDownUnroll];
      bool live[kDownUnroll];
#pragma unroll
      for (int u = 0; u < kDownUnroll; ++u) {
        const int64_t row = base + u * rows_per_warp + lane / lpr;
        live[u] = u < unroll && row < p.rows && c < p.chunks;
        if (live[u]) {
          a[u] = *reinterpret_cast<const uint4*>(p.out1 + row * row_bytes + c * 16);
          b[u] = *reinterpret_cast<const uint4*>(p.out2 + row * row_bytes + c * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < kDownUnroll; ++u) {
        const int src = u * rows_per_warp + lane / lpr;    // the lane that owns this row's scalars
        const float t = __shfl_sync(0xffffffffu, my_t, src);
        const float scale = __shfl_sync(0xffffffffu, my_scale, src);
        if (!live[u]) continue;
        const int64_t row = base + u * rows_per_warp + lane / lpr;
        const uint32_t x[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
        const uint32_t y[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float r0 = (lo_f(x[i]) - t * lo_f(y[i])) * scale;
          const float r1 = (hi_f(x[i]) - t * hi_f(y[i])) * scale;
          o[i] = pack2(r0, r1);
        }
        *reinterpret_cast<uint4*>(p.out2 + row * row_bytes + c * 16) =
            make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// D not a multiple of 8 or unaligned bases: one thread per element pair stride.
__global__ void __launch_bounds__(kDownThreads)
downdate_inplace_scalar_kernel(const DowndateParams p) {
  const __nv_bfloat16* o1 = reinterpret_cast<const __nv_bfloat16*>(p.out1);
  __nv_bfloat16* o2 = reinterpret_cast<__nv_bfloat16*>(p.out2);
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp_global; row < p.rows; row += warps_total) {
    float ret, t, scale;
    downdate_scalars(load_lse(p.lse1, p.dt1, row), load_lse(p.lse2, p.dt2, row), ret, t, scale);
    __syncwarp();
    for (int d = lane; d < p.D; d += 32) {
      const float r = (__bfloat162float(o1[row * p.D + d]) - t * __bfloat162float(o2[row * p.D + d])) * scale;
      o2[row * p.D + d] = __float2bfloat16_rn(r);
    }
    __syncwarp();
    if (lane == 0) store_lse(p.lse2, p.dt2, row, ret);
  }
}

}  // namespace
}  // namespace mac_b200

using namespace mac_b200;

extern "C" int mac_b200_update_then_downdate_bf16_inplace(const void* out1, const void* lse1,
                                                          int32_t lse1_dtype, void* out2,
                                                          void* lse2, int32_t lse2_dtype,
                                                          int64_t rows, int32_t D,
                                                          void* stream_v) {
  MAC_REQUIRE(rows >= 0 && D > 0, "invalid downdate shape");
  if (rows == 0) return MAC_B200_OK;
  MAC_REQUIRE(out1 && lse1 && out2 && lse2, "downdate tensors must not be null");
  MAC_REQUIRE(lse1_dtype >= 0 && lse1_dtype <= 2 && lse2_dtype >= 0 && lse2_dtype <= 2,
              "lse must be float32, bfloat16, or float16");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  DowndateParams p;
  p.out1 = static_cast<const char*>(out1);
  p.out2 = static_cast<char*>(out2);
  p.lse1 = lse1;
  p.lse2 = lse2;
  p.rows = rows;
  p.D = D;
  p.dt1 = lse1_dtype;
  p.dt2 = lse2_dtype;
  int device = 0;
  MAC_CUDA(cudaGetDevice(&device));
  const int64_t max_blocks = static_cast<int64_t>(device_sm_count(device)) * 32;
  const bool vec = D % 8 == 0 && ((reinterpret_cast<uintptr_t>(out1) | reinterpret_cast<uintptr_t>(out2)) & 15u) == 0;
  if (vec) {
    p.chunks = D / 8;
    int lpr = 1;
    while (lpr < p.chunks && lpr < 32) lpr <<= 1;
    p.lanes_per_row = lpr;
    p.unroll = kDownUnroll;
    while ((32 / lpr) * p.unroll > 32) p.unroll >>= 1;   // narrow rows: fewer rows in flight per lane
    const int64_t rows_per_cta = static_cast<int64_t>(kDownThreads / 32) * (32 / lpr) * p.unroll;
    int64_t blocks = (rows + rows_per_cta - 1) / rows_per_cta;
    if (blocks > max_blocks) blocks = max_blocks;
    downdate_inplace_kernel<<<static_cast<unsigned>(blocks), kDownThreads, 0, stream>>>(p);
  } else {
    p.chunks = 0;
    p.unroll = 1;
    p.lanes_per_row = 32;
    int64_t blocks = (rows + 7) / 8;
    if (blocks > max_blocks) blocks = max_blocks;
    downdate_inplace_scalar_kernel<<<static_cast<unsigned>(blocks), kDownThreads, 0, stream>>>(p);
  }
  MAC_CUDA(cudaGetLastError());
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return MAC_B200_OK;
}
