// Torch-extension shim of the decode operator: the pybind module the reference
// ships for mac_persistent_decode_bf16 (mac_decode_persistent.cu:4962-5030 and
// 5526-5529 in the reference project), re-expressed over the C ABI.
//
// It takes torch.Tensors, checks what the reference launcher checks (same
// messages, before any launch), extracts pointers and sizes into
// MacB200DecodeArgs and calls the C-ABI entry point on torch's current CUDA
// stream of the tensors' device.  Nothing else happens here: no allocation, no
// kernel, no torch op.  Failures are reported by return code, not by C++
// exceptions: kShimCheckFailed with the text at last_error() for a failed
// check (the Python operator raises the RuntimeError the reference's
// TORCH_CHECK would), else the C ABI's own status code.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/mac_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

constexpr int kShimCheckFailed = -1000;

std::string& shim_error() {
  static thread_local std::string text;
  return text;
}

template <typename... Parts>
int shim_fail(const Parts&... parts) {
  shim_error() = c10::str(parts...);
  return kShimCheckFailed;
}

// A failed requirement leaves its message at last_error() and makes the enclosing function
// return kShimCheckFailed.
#define REQUIRE(cond, ...)                         \
  do {                                             \
    if (!(cond)) return shim_fail(__VA_ARGS__);    \
  } while (0)
#define REQUIRE_OK(call)                           \
  do {                                             \
    if (const int rc_ = (call)) return rc_;        \
  } while (0)

int check(const Tensor& t, const char* name, at::ScalarType dtype, int64_t dim) {
  REQUIRE(t.is_cuda(), name, " must be CUDA");
  REQUIRE(t.is_contiguous(), name, " must be contiguous");
  REQUIRE(t.scalar_type() == dtype, name, " has wrong dtype");
  REQUIRE(t.dim() == dim, name, " has wrong rank");
  return 0;
}

// The step's own inputs and its output (q_post, q_pre, out) may also lie in pinned host memory
// (torch's pin_memory(): page-locked by the CUDA runtime, one address on host and device): the
// kernel then reads the queries and writes the output over the bus itself, and a caller whose
// queries are produced on the host, or who wants the output there, needs no staging copy.
int check_step_io(const Tensor& t, const char* name, at::ScalarType dtype, int64_t dim) {
  REQUIRE(t.is_cuda() || (t.device().is_cpu() && t.is_pinned()), name,
          " must be CUDA or pinned host memory");
  REQUIRE(t.is_contiguous(), name, " must be contiguous");
  REQUIRE(t.scalar_type() == dtype, name, " has wrong dtype");
  REQUIRE(t.dim() == dim, name, " has wrong rank");
  return 0;
}

int check_partial_o(const Tensor& t, const char* name) {
  REQUIRE(t.is_cuda(), name, " must be CUDA");
  REQUIRE(t.is_contiguous(), name, " must be contiguous");
  REQUIRE(t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16, name,
          " must be float32 or bfloat16");
  REQUIRE(t.dim() == 5, name, " has wrong rank");
  return 0;
}

int env_flag(const char* name, int dflt) {
  const char* raw = std::getenv(name);
  if (raw == nullptr) return dflt;
  char* end = nullptr;
  const long v = std::strtol(raw, &end, 10);
  if (end == raw) return 0;
  return v != 0 ? 1 : 0;
}

int env_positive_int(const char* name, int dflt) {
  const char* raw = std::getenv(name);
  if (raw == nullptr) return dflt;
  char* end = nullptr;
  const long v = std::strtol(raw, &end, 10);
  return (end != raw && v > 0) ? static_cast<int>(v) : dflt;
}

bool present(const OptTensor& t) { return t.has_value() && t->defined() && t->numel() > 0; }

enum Entry { kDecode = 0, kDecodeNoAlloc = 1 };

// `lean` callers pass no task lists and no partial buffers (None for those arguments).
// Returns the C ABI's status code (0 = launched); the caller turns a non-zero code into a
// RuntimeError carrying mac_b200_last_error() of this thread.
int decode(
    int entry, const Tensor& q_post, const Tensor& q_pre, const Tensor& k_buffer,
    const Tensor& v_buffer, const Tensor& req_to_token, const Tensor& req_ids,
    const Tensor& past_lens, const Tensor& out_cache_loc, const Tensor& query_cache,
    const Tensor& attn_cache, const Tensor& lse_cache, const Tensor& out, const Tensor& optional_lse,
    const Tensor& match_dist, const Tensor& match_pos, const Tensor& match_slot,
    const Tensor& head_hit, const Tensor& head_match_slot, const Tensor& head_match_pos,
    const Tensor& head_prefix_end, const Tensor& head_rect_start, const Tensor& head_new_end,
    const Tensor& group_rect_begin, const Tensor& group_rect_end, const Tensor& group_rect_tiles,
    const Tensor& group_tail_begin, const Tensor& group_tail_end, const Tensor& group_tail_tiles,
    const Tensor& group_mode, const OptTensor& complete_task_go, const OptTensor& complete_task_tile,
    const OptTensor& tail_task_go, const OptTensor& tail_task_tile,
    const OptTensor& hit_tail_task_ho, const OptTensor& hit_tail_task_tile,
    const Tensor& task_counts, const OptTensor& partial_rect_o, const OptTensor& partial_rect_lse,
    const OptTensor& partial_rect_reduced_o, const OptTensor& partial_rect_reduced_lse,
    const OptTensor& partial_tail_o, const OptTensor& partial_tail_lse, const Tensor& phase_cycles,
    int64_t max_context, int64_t tile_tokens, int64_t match_tile_slots, int64_t semantic_pos_ahead,
    int64_t front_sink_tokens, int64_t gen_min_limit, int64_t lookback_right,
    int64_t candidate_mode, double threshold, double sm_scale, int64_t debug_enabled,
    int64_t bench_mode, double bench_hit_rate, double bench_hit_rate_std, double bench_skip_ratio,
    double bench_skip_ratio_std, double bench_match_lag_mean, double bench_match_lag_std,
    int64_t bench_seed, int64_t bench_miss_mask, int64_t bench_layer_id,
    const OptTensor& query_post_cache, const OptTensor& mac_cache_ready,
    const OptTensor& mac_cache_epoch, const OptTensor& mac_request_epoch) {
  REQUIRE_OK(check_step_io(q_post, "q_post", at::kBFloat16, 3));
  REQUIRE_OK(check_step_io(q_pre, "q_pre", at::kBFloat16, 3));
  REQUIRE_OK(check(k_buffer, "k_buffer", at::kBFloat16, 3));
  REQUIRE_OK(check(v_buffer, "v_buffer", at::kBFloat16, 3));
  REQUIRE_OK(check(req_to_token, "req_to_token", at::kInt, 2));
  REQUIRE_OK(check(req_ids, "req_ids", at::kInt, 1));
  REQUIRE_OK(check(past_lens, "past_lens", at::kInt, 1));
  REQUIRE(out_cache_loc.is_cuda(), "out_cache_loc must be CUDA");
  REQUIRE(out_cache_loc.is_contiguous(), "out_cache_loc must be contiguous");
  REQUIRE(out_cache_loc.dim() == 1, "out_cache_loc has wrong rank");
  REQUIRE(out_cache_loc.scalar_type() == at::kInt || out_cache_loc.scalar_type() == at::kLong,
              "out_cache_loc must be int32 or int64");
  REQUIRE_OK(check(query_cache, "query_cache", at::kBFloat16, 4));
  if (present(query_post_cache)) REQUIRE_OK(check(*query_post_cache, "query_post_cache", at::kBFloat16, 4));
  REQUIRE_OK(check(attn_cache, "attn_cache", at::kBFloat16, 4));
  REQUIRE_OK(check(lse_cache, "lse_cache", at::kFloat, 3));
  REQUIRE_OK(check_step_io(out, "out", at::kBFloat16, 3));
  REQUIRE(optional_lse.is_cuda(), "optional_lse must be CUDA");
  REQUIRE(optional_lse.is_contiguous(), "optional_lse must be contiguous");
  REQUIRE(optional_lse.numel() == 0 || optional_lse.scalar_type() == at::kFloat,
              "optional_lse must be empty or float32");
  REQUIRE(phase_cycles.is_cuda(), "phase_cycles must be CUDA");
  REQUIRE(phase_cycles.is_contiguous(), "phase_cycles must be contiguous");
  REQUIRE(phase_cycles.scalar_type() == at::kLong, "phase_cycles must be int64");
  REQUIRE(phase_cycles.numel() >= 6, "phase_cycles must have at least 6 elements");
  REQUIRE_OK(check(match_dist, "match_dist", at::kFloat, 3));
  REQUIRE_OK(check(match_pos, "match_pos", at::kInt, 3));
  REQUIRE_OK(check(match_slot, "match_slot", at::kInt, 3));
  const Tensor* head_ws[6] = {&head_hit,        &head_match_slot, &head_match_pos,
                              &head_prefix_end, &head_rect_start, &head_new_end};
  const char* head_names[6] = {"head_hit",        "head_match_slot", "head_match_pos",
                               "head_prefix_end", "head_rect_start", "head_new_end"};
  const Tensor* group_ws[7] = {&group_rect_begin, &group_rect_end, &group_rect_tiles,
                               &group_tail_begin, &group_tail_end, &group_tail_tiles, &group_mode};
  const char* group_names[7] = {"group_rect_begin", "group_rect_end", "group_rect_tiles",
                                "group_tail_begin", "group_tail_end", "group_tail_tiles",
                                "group_mode"};
  for (int i = 0; i < 6; ++i) REQUIRE_OK(check(*head_ws[i], head_names[i], at::kInt, 2));
  for (int i = 0; i < 7; ++i) REQUIRE_OK(check(*group_ws[i], group_names[i], at::kInt, 2));
  REQUIRE_OK(check(task_counts, "task_counts", at::kInt, 1));
  const bool lean = !partial_rect_o.has_value();
  if (!lean) {
    REQUIRE(complete_task_go && complete_task_tile && tail_task_go && tail_task_tile &&
                    hit_tail_task_ho && hit_tail_task_tile && partial_rect_lse &&
                    partial_rect_reduced_o && partial_rect_reduced_lse && partial_tail_o &&
                    partial_tail_lse,
                "task lists and partial workspaces go together");
    REQUIRE_OK(check(*complete_task_go, "complete_task_go", at::kInt, 1));
    REQUIRE_OK(check(*complete_task_tile, "complete_task_tile", at::kInt, 1));
    REQUIRE_OK(check(*tail_task_go, "tail_task_go", at::kInt, 1));
    REQUIRE_OK(check(*tail_task_tile, "tail_task_tile", at::kInt, 1));
    REQUIRE_OK(check(*hit_tail_task_ho, "hit_tail_task_ho", at::kInt, 1));
    REQUIRE_OK(check(*hit_tail_task_tile, "hit_tail_task_tile", at::kInt, 1));
    REQUIRE_OK(check_partial_o(*partial_rect_o, "partial_rect_o"));
    REQUIRE_OK(check(*partial_rect_lse, "partial_rect_lse", at::kFloat, 4));
    REQUIRE_OK(check_partial_o(*partial_rect_reduced_o, "partial_rect_reduced_o"));
    REQUIRE_OK(check(*partial_rect_reduced_lse, "partial_rect_reduced_lse", at::kFloat, 4));
    REQUIRE_OK(check_partial_o(*partial_tail_o, "partial_tail_o"));
    REQUIRE_OK(check(*partial_tail_lse, "partial_tail_lse", at::kFloat, 4));
    REQUIRE(partial_rect_reduced_o->scalar_type() == partial_rect_o->scalar_type() &&
                    partial_tail_o->scalar_type() == partial_rect_o->scalar_type(),
                "all partial output workspaces must use the same dtype");
  }

  const int64_t N = q_post.size(0), Hq = q_post.size(1), D = q_post.size(2);
  const int64_t Hkv = k_buffer.size(1);
  REQUIRE(D == 128, "persistent decode v1 supports D=128 only");
  REQUIRE(q_pre.sizes() == q_post.sizes(), "q_pre/q_post shape mismatch");
  REQUIRE(v_buffer.sizes() == k_buffer.sizes(), "k/v shape mismatch");
  REQUIRE(Hkv > 0 && Hq % Hkv == 0, "Hq must be divisible by Hkv");
  const int64_t G = Hq / Hkv;
  REQUIRE(G > 0 && G <= 8, "unsupported GQA group size");
  REQUIRE(req_ids.size(0) >= N && past_lens.size(0) >= N && out_cache_loc.size(0) >= N,
              "batch metadata too small");
  REQUIRE(out.sizes() == q_post.sizes(), "out shape mismatch");
  const int64_t R = query_cache.size(0), M = query_cache.size(1);
  REQUIRE(query_cache.size(2) == Hq && query_cache.size(3) == D, "query_cache shape mismatch");
  REQUIRE(attn_cache.sizes() == query_cache.sizes(), "attn_cache shape mismatch");
  REQUIRE(lse_cache.size(0) == R && lse_cache.size(1) == M && lse_cache.size(2) == Hq,
              "lse_cache shape mismatch");
  REQUIRE(tile_tokens > 0 && match_tile_slots > 0, "tile sizes must be positive");
  const int64_t Tm = match_dist.size(2);
  REQUIRE(Tm >= (M + match_tile_slots - 1) / match_tile_slots, "match workspace too small");
  REQUIRE(group_mode.size(0) >= N && group_mode.size(1) >= Hkv, "group_mode workspace too small");
  REQUIRE(task_counts.numel() >= 9, "task_counts must have at least nine elements");
  REQUIRE(bench_mode >= 0 && bench_mode <= 2, "unsupported synthetic MAC bench mode");
  if (!lean) {
    const int64_t Tc = partial_rect_lse->size(2), Tr = partial_rect_reduced_lse->size(2),
                  Tt = partial_tail_lse->size(2);
    REQUIRE(Tc >= (max_context + tile_tokens - 1) / tile_tokens, "rect workspace too small");
    REQUIRE(Tr >= (max_context + tile_tokens * 32 - 1) / (tile_tokens * 32),
                "reduced rect workspace too small");
    REQUIRE(Tt >= (semantic_pos_ahead + tile_tokens - 1) / tile_tokens,
                "tail workspace too small");
    auto shape5 = [&](const Tensor& t, int64_t tiles) {
      return t.size(0) >= N && t.size(1) == Hkv && t.size(2) == tiles && t.size(3) == G &&
             t.size(4) == D;
    };
    auto shape4 = [&](const Tensor& t, int64_t tiles) {
      return t.size(0) >= N && t.size(1) == Hkv && t.size(2) == tiles && t.size(3) == G;
    };
    REQUIRE(shape5(*partial_rect_o, Tc), "rect output workspace has wrong shape");
    REQUIRE(shape4(*partial_rect_lse, Tc), "rect lse workspace has wrong shape");
    REQUIRE(shape5(*partial_rect_reduced_o, Tr), "reduced rect output workspace has wrong shape");
    REQUIRE(shape4(*partial_rect_reduced_lse, Tr), "reduced rect lse workspace has wrong shape");
    REQUIRE(shape5(*partial_tail_o, Tt), "tail output workspace has wrong shape");
    REQUIRE(shape4(*partial_tail_lse, Tt), "tail lse workspace has wrong shape");
    REQUIRE(complete_task_tile->numel() == complete_task_go->numel(), "complete task shape mismatch");
    REQUIRE(tail_task_tile->numel() == tail_task_go->numel(), "tail task shape mismatch");
    REQUIRE(hit_tail_task_tile->numel() == hit_tail_task_ho->numel(), "hit tail task shape mismatch");
    REQUIRE(complete_task_go->numel() >= N * Hq * Tc, "complete task workspace too small");
    REQUIRE(tail_task_go->numel() >= N * Hkv * Tt, "tail task workspace too small");
    REQUIRE(hit_tail_task_ho->numel() >= N * Hq * Tt, "hit tail task workspace too small");
  }
  int64_t ws_batch = match_dist.size(0);
  const Tensor* match_ws[3] = {&match_dist, &match_pos, &match_slot};
  const char* match_names[3] = {"match_dist", "match_pos", "match_slot"};
  for (int i = 0; i < 3; ++i)
    REQUIRE(match_ws[i]->size(0) >= N && match_ws[i]->size(1) == Hq && match_ws[i]->size(2) == Tm,
                match_names[i], " workspace has wrong shape");
  for (int i = 0; i < 6; ++i) {
    REQUIRE(head_ws[i]->size(0) >= N && head_ws[i]->size(1) == Hq, head_names[i],
                " workspace has wrong shape");
    ws_batch = std::min(ws_batch, head_ws[i]->size(0));
  }
  for (int i = 0; i < 7; ++i) {
    REQUIRE(group_ws[i]->size(0) >= N && group_ws[i]->size(1) == Hkv, group_names[i],
                " workspace has wrong shape");
    ws_batch = std::min(ws_batch, group_ws[i]->size(0));
  }

  MacB200DecodeArgs a;
  std::memset(&a, 0, sizeof(a));
  if (present(mac_cache_ready)) {
    const Tensor& ready = *mac_cache_ready;
    REQUIRE(ready.is_cuda(), "mac_cache_ready must be CUDA");
    REQUIRE(ready.is_contiguous(), "mac_cache_ready must be contiguous");
    REQUIRE(ready.scalar_type() == at::kBool || ready.scalar_type() == at::kByte,
                "mac_cache_ready must be bool or uint8");
    REQUIRE(ready.numel() >= R, "mac_cache_ready is smaller than the ring");
    a.cache_ready = static_cast<const uint8_t*>(ready.data_ptr());
    if (present(mac_cache_epoch) && present(mac_request_epoch)) {
      REQUIRE_OK(check(*mac_cache_epoch, "mac_cache_epoch", at::kLong, 1));
      REQUIRE_OK(check(*mac_request_epoch, "mac_request_epoch", at::kLong, 1));
      REQUIRE(mac_cache_epoch->numel() >= R && mac_request_epoch->numel() >= R,
                  "epoch tensors are smaller than the ring");
      a.cache_epoch = mac_cache_epoch->data_ptr<int64_t>();
      a.request_epoch = mac_request_epoch->data_ptr<int64_t>();
    }
  }
  if (optional_lse.numel() > 0) {
    REQUIRE(optional_lse.numel() >= N * Hq, "optional_lse is smaller than [N,Hq]");
    a.optional_lse = optional_lse.data_ptr<float>();
  }
  a.N = static_cast<int32_t>(N);
  a.Hq = static_cast<int32_t>(Hq);
  a.Hkv = static_cast<int32_t>(Hkv);
  a.D = static_cast<int32_t>(D);
  a.M = static_cast<int32_t>(M);
  a.R = static_cast<int32_t>(R);
  a.req_to_token_rows = static_cast<int32_t>(req_to_token.size(0));
  a.req_to_token_stride = static_cast<int32_t>(req_to_token.size(1));
  a.kv_tokens = k_buffer.size(0);
  a.ws_batch = static_cast<int32_t>(ws_batch);
  a.max_match_tiles = static_cast<int32_t>(Tm);
  a.max_context = static_cast<int32_t>(max_context);
  a.tile_tokens = static_cast<int32_t>(tile_tokens);
  a.match_tile_slots = static_cast<int32_t>(match_tile_slots);
  a.semantic_pos_ahead = static_cast<int32_t>(semantic_pos_ahead);
  a.front_sink_tokens = static_cast<int32_t>(front_sink_tokens);
  a.gen_min_limit = static_cast<int32_t>(gen_min_limit);
  a.lookback_right = static_cast<int32_t>(lookback_right);
  a.candidate_mode = static_cast<int32_t>(candidate_mode);
  a.threshold = static_cast<float>(threshold);
  a.sm_scale = static_cast<float>(sm_scale);
  a.debug_enabled = static_cast<int32_t>(debug_enabled);
  a.bench_mode = static_cast<int32_t>(bench_mode);
  a.bench_hit_rate = static_cast<float>(bench_hit_rate);
  a.bench_hit_rate_std = static_cast<float>(bench_hit_rate_std);
  a.bench_skip_ratio = static_cast<float>(bench_skip_ratio);
  a.bench_skip_ratio_std = static_cast<float>(bench_skip_ratio_std);
  a.bench_match_lag_mean = static_cast<float>(bench_match_lag_mean);
  a.bench_match_lag_std = static_cast<float>(bench_match_lag_std);
  a.bench_seed = static_cast<int32_t>(static_cast<uint32_t>(bench_seed & 0xffffffffll));
  a.bench_miss_mask = static_cast<int32_t>(bench_miss_mask);
  a.bench_layer_id = static_cast<int32_t>(static_cast<uint32_t>(bench_layer_id & 0xffffffffll));
  // The reference reads these knobs from the environment on every launch
  // (mac_decode_persistent.cu:5229, 5337, 5403).
  a.mixed_group_fallback = env_flag("MAC_PERSISTENT_MIXED_GROUP_FALLBACK", 1);
  a.bench_exact_quota = env_flag("MAC_BENCH_EXACT_QUOTA", 1);
  a.grid_cap = env_positive_int("MAC_PERSISTENT_COOP_CTAS", 0);
  a.bench_long_band = env_flag("MAC_B200_BENCH_LONG_BAND", 0);   // benchmark extension, default off
  a.out_cache_loc_is_i64 = out_cache_loc.scalar_type() == at::kLong ? 1 : 0;
  a.phase_cycles_count = static_cast<int32_t>(phase_cycles.numel());
  a.q_post = q_post.data_ptr();   // pinned host memory has the same address on the device
  a.q_pre = q_pre.data_ptr();
  a.out = out.data_ptr();
  a.k_buffer = k_buffer.data_ptr();
  a.v_buffer = v_buffer.data_ptr();
  a.req_to_token = req_to_token.data_ptr<int32_t>();
  a.req_ids = req_ids.data_ptr<int32_t>();
  a.past_lens = past_lens.data_ptr<int32_t>();
  a.out_cache_loc = out_cache_loc.data_ptr();
  a.query_cache = query_cache.data_ptr();
  a.attn_cache = attn_cache.data_ptr();
  a.lse_cache = lse_cache.data_ptr<float>();
  a.match_dist = match_dist.data_ptr<float>();
  a.match_pos = match_pos.data_ptr<int32_t>();
  a.match_slot = match_slot.data_ptr<int32_t>();
  a.head_hit = head_hit.data_ptr<int32_t>();
  a.head_match_slot = head_match_slot.data_ptr<int32_t>();
  a.head_match_pos = head_match_pos.data_ptr<int32_t>();
  a.head_prefix_end = head_prefix_end.data_ptr<int32_t>();
  a.head_rect_start = head_rect_start.data_ptr<int32_t>();
  a.head_new_end = head_new_end.data_ptr<int32_t>();
  a.group_rect_begin = group_rect_begin.data_ptr<int32_t>();
  a.group_rect_end = group_rect_end.data_ptr<int32_t>();
  a.group_rect_tiles = group_rect_tiles.data_ptr<int32_t>();
  a.group_tail_begin = group_tail_begin.data_ptr<int32_t>();
  a.group_tail_end = group_tail_end.data_ptr<int32_t>();
  a.group_tail_tiles = group_tail_tiles.data_ptr<int32_t>();
  a.group_mode = group_mode.data_ptr<int32_t>();
  a.task_counts = task_counts.data_ptr<int32_t>();
  a.phase_cycles = phase_cycles.data_ptr<int64_t>();

  const c10::cuda::CUDAGuard guard(k_buffer.device());   // q_post may be host memory
  void* stream = static_cast<void*>(c10::cuda::getCurrentCUDAStream(k_buffer.device().index()).stream());
  return entry == kDecodeNoAlloc ? mac_b200_persistent_decode_bf16_noalloc(&a, stream)
                                 : mac_b200_persistent_decode_bf16(&a, stream);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "torch.Tensor front end of the B200 MAC decode step (pointer/shape extraction only)";
  m.def("last_error", [] { return shim_error(); },
        "text of the last failed check on the calling thread");
  m.attr("CHECK_FAILED") = kShimCheckFailed;
  m.def("decode", &decode,
        "entry (0: allocating, 1: fixed scratch block) followed by the reference operator's 68 "
        "positional arguments; task lists and partial buffers may be None (lean call); returns "
        "the C ABI's status code");
}
