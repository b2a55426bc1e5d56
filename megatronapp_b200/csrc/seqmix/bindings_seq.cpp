// PyTorch bindings of the sequence-mixing kernels (pybind11 module megatronapp_b200._C_seq).
#include <torch/extension.h>
#include <algorithm>
#include <atomic>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "seqmix_api.h"

using torch::Tensor;

namespace {

std::atomic<int64_t> g_launches{0};
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void count(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool act_is_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kFloat, name, " must be bf16 or fp32, got ", t.scalar_type());
  return t.scalar_type() == at::kBFloat16;
}
void check_f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), name, " must be a contiguous fp32 CUDA tensor");
}
void check_i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), name, " must be a contiguous int32 CUDA tensor");
}
void check_rows(const Tensor& t, const char* name) {   // [T, ...] with contiguous trailing dims and a free row stride
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1 && t.stride(1) == t.size(2), name, " must be [T, heads, dim] with contiguous heads");
}
void check_last_error(const char* what) {
  cudaError_t e = cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

void add_rms_norm(Tensor x, c10::optional<Tensor> delta, const Tensor& w, Tensor y, double eps) {
  check_f32(x, "x");
  const bool bf16 = act_is_bf16(y, "y");
  TORCH_CHECK(x.dim() == 2 && y.is_contiguous() && y.sizes() == x.sizes(), "x / y must be [rows, cols]");
  TORCH_CHECK(w.scalar_type() == y.scalar_type() && w.is_contiguous() && w.numel() == x.size(1), "weight must match y's dtype and cols");
  TORCH_CHECK(x.size(1) * sizeof(float) <= 48 * 1024, "row too wide");
  const void* d = nullptr;
  if (delta.has_value() && delta->defined()) {
    TORCH_CHECK(delta->scalar_type() == y.scalar_type() && delta->is_contiguous() && delta->sizes() == x.sizes(),
                "delta must be contiguous, shaped like x, in y's dtype");
    d = delta->data_ptr();
  }
  c10::cuda::CUDAGuard g(x.device());
  b200seq::add_rms_norm(x.data_ptr<float>(), d, w.data_ptr(), y.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                        static_cast<float>(eps), bf16, cur_stream());
  count(); check_last_error("add_rms_norm");
}

void gated_head_rms_norm(const Tensor& o, const Tensor& w, c10::optional<Tensor> gate, Tensor y, double eps) {
  check_f32(o, "o");
  TORCH_CHECK(o.dim() == 3, "o must be [T, H, dv]");
  const bool bf16 = act_is_bf16(y, "y");
  const int T = static_cast<int>(o.size(0)), H = static_cast<int>(o.size(1)), dv = static_cast<int>(o.size(2));
  TORCH_CHECK(y.is_contiguous() && y.numel() == o.numel(), "y must be [T, H * dv]");
  TORCH_CHECK(w.scalar_type() == y.scalar_type() && w.is_contiguous() && (w.numel() == dv || w.numel() == H * dv), "bad weight");
  const void* gp = nullptr;
  if (gate.has_value() && gate->defined()) {
    TORCH_CHECK(gate->scalar_type() == y.scalar_type() && gate->is_contiguous() && gate->numel() == o.numel(), "bad gate");
    gp = gate->data_ptr();
  }
  c10::cuda::CUDAGuard g(o.device());
  b200seq::gated_head_rms_norm(o.data_ptr<float>(), w.data_ptr(), gp, y.data_ptr(), T, H, dv, w.numel() != dv || H == 1, eps, bf16,
                               cur_stream());
  count(); check_last_error("gated_head_rms_norm");
}

void causal_conv_silu(const Tensor& x, const Tensor& w, const Tensor& cu, const Tensor& rows, const Tensor& tok_seq, Tensor window,
                      Tensor y, int64_t max_len) {
  const bool bf16 = act_is_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "x must be [T, C] with unit inner stride");
  const int T = static_cast<int>(x.size(0)), C = static_cast<int>(x.size(1)), taps = static_cast<int>(w.size(1));
  TORCH_CHECK(w.scalar_type() == x.scalar_type() && w.is_contiguous() && w.size(0) == C, "bad conv weight");
  TORCH_CHECK(y.scalar_type() == x.scalar_type() && y.is_contiguous() && y.sizes() == x.sizes(), "bad y");
  TORCH_CHECK(window.scalar_type() == x.scalar_type() && window.is_contiguous() && window.dim() == 3 && window.size(1) == taps - 1 &&
              window.size(2) == C, "window must be [rows, taps - 1, C]");
  check_i32(cu, "cu"); check_i32(rows, "rows"); check_i32(tok_seq, "tok_seq");
  TORCH_CHECK(tok_seq.numel() == T && cu.numel() == rows.numel() + 1, "bad packed-batch tensors");
  c10::cuda::CUDAGuard g(x.device());
  b200seq::causal_conv_silu(x.data_ptr(), x.stride(0), w.data_ptr(), cu.data_ptr<int>(), rows.data_ptr<int>(), tok_seq.data_ptr<int>(),
                            window.data_ptr(), y.data_ptr(), T, static_cast<int>(rows.numel()), C, taps, static_cast<int>(max_len), bf16,
                            cur_stream());
  count(2); check_last_error("causal_conv_silu");
}

void delta_rule_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& log_decay, const Tensor& beta, const Tensor& cu,
                     const Tensor& rows, Tensor state, Tensor out, double unit_eps, double q_scale, int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q / k / v dtypes differ");
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  check_f32(log_decay, "log_decay"); check_f32(beta, "beta"); check_f32(state, "state"); check_f32(out, "out");
  check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::DeltaArgs p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.ldq = q.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0);
  p.H = static_cast<int>(v.size(1)); p.KH = static_cast<int>(q.size(1)); p.d = static_cast<int>(q.size(2)); p.dv = static_cast<int>(v.size(2));
  TORCH_CHECK(p.H % p.KH == 0 && k.size(1) == p.KH && k.size(2) == p.d, "bad head layout");
  TORCH_CHECK(log_decay.numel() == q.size(0) * p.H * p.d && beta.numel() == q.size(0) * p.H, "bad decay / beta shape");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == p.H && state.size(2) == p.d && state.size(3) == p.dv, "bad state shape");
  TORCH_CHECK(out.numel() == q.size(0) * p.H * p.dv, "bad out shape");
  p.log_decay = log_decay.data_ptr<float>(); p.beta = beta.data_ptr<float>();
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>();
  p.state = state.data_ptr<float>(); p.out = out.data_ptr<float>();
  p.unit_eps = static_cast<float>(unit_eps); p.q_scale = static_cast<float>(q_scale);
  p.max_len = max_len > 0 ? static_cast<int>(max_len) : (1 << 30);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(b200seq::delta_rule_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "delta_rule_scan: key dim ", p.d,
              " above the largest kernel instance (256)");
  count(); check_last_error("delta_rule_scan");
}

void mlstm_scan(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& log_i, const Tensor& log_f, const Tensor& cu,
                const Tensor& rows, Tensor state, Tensor norm_state, Tensor max_state, Tensor out, double q_scale, double denom_eps,
                int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q / k / v dtypes differ");
  check_rows(q, "q"); check_rows(k, "k"); check_rows(v, "v");
  check_f32(log_i, "log_i"); check_f32(log_f, "log_f"); check_f32(state, "state"); check_f32(norm_state, "norm_state");
  check_f32(max_state, "max_state"); check_f32(out, "out");
  check_i32(cu, "cu"); check_i32(rows, "rows");
  b200seq::MlstmArgs p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.ldq = q.stride(0); p.ldk = k.stride(0); p.ldv = v.stride(0);
  p.H = static_cast<int>(v.size(1)); p.d = static_cast<int>(q.size(2)); p.dv = static_cast<int>(v.size(2));
  TORCH_CHECK(q.size(1) == p.H && k.size(1) == p.H && k.size(2) == p.d, "bad head layout");
  TORCH_CHECK(log_i.numel() == q.size(0) * p.H && log_f.numel() == q.size(0) * p.H, "bad gate shape");
  TORCH_CHECK(state.dim() == 4 && state.size(1) == p.H && state.size(2) == p.d && state.size(3) == p.dv, "bad state shape");
  TORCH_CHECK(norm_state.numel() == state.size(0) * p.H * p.d && max_state.numel() == state.size(0) * p.H, "bad n / m shape");
  TORCH_CHECK(out.numel() == q.size(0) * p.H * p.dv, "bad out shape");
  p.log_i = log_i.data_ptr<float>(); p.log_f = log_f.data_ptr<float>();
  p.cu = cu.data_ptr<int>(); p.rows = rows.data_ptr<int>();
  p.state = state.data_ptr<float>(); p.norm_state = norm_state.data_ptr<float>(); p.max_state = max_state.data_ptr<float>();
  p.out = out.data_ptr<float>();
  p.q_scale = static_cast<float>(q_scale); p.denom_eps = static_cast<float>(denom_eps);
  p.max_len = max_len > 0 ? static_cast<int>(max_len) : (1 << 30);
  c10::cuda::CUDAGuard g(q.device());
  TORCH_CHECK(b200seq::mlstm_scan(p, static_cast<int>(rows.numel()), bf16, cur_stream()), "mlstm_scan: key dim ", p.d,
              " above the largest kernel instance (256)");
  count(); check_last_error("mlstm_scan");
}

void latent_attention_paged(const Tensor& q, const Tensor& cache, const Tensor& block_table, const Tensor& tok_req, const Tensor& tok_len,
                            Tensor out, int64_t block_size, double scale, int64_t max_len) {
  const bool bf16 = act_is_bf16(q, "q_lat");
  TORCH_CHECK(q.dim() == 3 && q.is_contiguous(), "q_lat must be contiguous [T, H, r]");
  TORCH_CHECK(cache.scalar_type() == q.scalar_type() && cache.dim() == 2 && cache.is_contiguous() && cache.size(1) == q.size(2),
              "cache must be [slots, r] in q_lat's dtype");
  check_i32(block_table, "block_table"); check_i32(tok_req, "tok_req"); check_i32(tok_len, "tok_len"); check_f32(out, "out");
  TORCH_CHECK(block_table.dim() == 2 && tok_req.numel() == q.size(0) && tok_len.numel() == q.size(0) && out.numel() == q.numel(),
              "bad shapes");
  b200seq::LatentAttnArgs p{};
  p.q = q.data_ptr(); p.cache = cache.data_ptr();
  p.block_table = block_table.data_ptr<int>(); p.tok_req = tok_req.data_ptr<int>(); p.tok_len = tok_len.data_ptr<int>();
  p.out = out.data_ptr<float>();
  p.H = static_cast<int>(q.size(1)); p.r = static_cast<int>(q.size(2)); p.block_size = static_cast<int>(block_size);
  p.max_blocks = static_cast<int>(block_table.size(1)); p.scale = static_cast<float>(scale);
  c10::cuda::CUDAGuard g(q.device());
  p.n_splits = b200seq::latent_attention_splits(p.H, p.r, static_cast<int>(q.size(0)), static_cast<int>(max_len));
  const int64_t vec = 16 / static_cast<int64_t>(cache.element_size());
  p.vec_ok = (p.r % vec == 0 && reinterpret_cast<uintptr_t>(cache.data_ptr()) % 16 == 0) ? 1 : 0;
  Tensor ws;
  if (p.n_splits > 1) {
    ws = torch::empty({q.size(0), q.size(1), p.n_splits, q.size(2) + 2}, out.options());
    p.ws = ws.data_ptr<float>();
  }
  TORCH_CHECK(b200seq::latent_attention_paged(p, static_cast<int>(q.size(0)), bf16, cur_stream()), "latent_attention_paged: rank ", p.r,
              " above the largest kernel instance (1024)");
  count(p.n_splits > 1 ? 2 : 1); check_last_error("latent_attention_paged");
}

void group_limited_router(const Tensor& logits, Tensor probs, Tensor rmap, int64_t topk, int64_t groups, int64_t keep, bool renorm) {
  check_f32(logits, "logits"); check_f32(probs, "probs");
  TORCH_CHECK(logits.dim() == 2 && probs.sizes() == logits.sizes() && rmap.sizes() == logits.sizes() && rmap.scalar_type() == at::kBool &&
              rmap.is_contiguous(), "bad shapes");
  c10::cuda::CUDAGuard g(logits.device());
  TORCH_CHECK(b200seq::group_limited_router(logits.data_ptr<float>(), probs.data_ptr<float>(), rmap.data_ptr<bool>(),
                                            static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)), static_cast<int>(topk),
                                            static_cast<int>(groups), static_cast<int>(keep), renorm, cur_stream()),
              "group_limited_router: unsupported sizes (experts ", logits.size(1), ", groups ", groups, ", top ", topk, ")");
  count(); check_last_error("group_limited_router");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("add_rms_norm", &add_rms_norm);
  m.def("gated_head_rms_norm", &gated_head_rms_norm);
  m.def("causal_conv_silu", &causal_conv_silu);
  m.def("delta_rule_scan", &delta_rule_scan);
  m.def("mlstm_scan", &mlstm_scan);
  m.def("latent_attention_paged", &latent_attention_paged);
  m.def("group_limited_router", &group_limited_router);
  m.def("launch_count", []() { return g_launches.load(); });
  m.def("reset_launch_count", []() { g_launches.store(0); });
}
