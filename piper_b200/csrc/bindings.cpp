// torch.ops.piper_c.*: thin tensor-level wrappers over the launchers in this
// directory.  Each wrapper validates shapes/dtypes, takes the current CUDA
// stream, and writes into caller-allocated outputs; none of them allocates
// device memory.  Higher-level autograd-aware ops live in piper_b200/ops.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <torch/library.h>

#include <atomic>
#include <cmath>

#include "attention_sm100.h"
#include "elementwise.h"
#include "gemm_sm100.h"
#include "moe.h"
#include "ep_exchange.h"
#include "zero_fused.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<at::Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}

// Number of kernels of this library launched by this process (benchmarks report it).
std::atomic<int64_t> g_kernel_launches{0};

void check_rc(int rc, const char* what, int kernels = 1) {
  TORCH_CHECK(rc == 0, "piper_c::", what, " failed with code ", rc);
  g_kernel_launches.fetch_add(kernels, std::memory_order_relaxed);
}

int64_t kernel_launch_count() { return g_kernel_launches.load(std::memory_order_relaxed); }

const void* opt_ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }
float* opt_f32(const OptTensor& t) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->scalar_type() == at::kFloat, "expected float32 tensor");
  return t->data_ptr<float>();
}

// C[M,N] = A * B^T.  a: [M,K] (a_mn=false) or [K,M] (a_mn=true); b: [N,K]
// (b_mn=false) or [K,N] (b_mn=true).  c bf16 -> store; c fp32 -> store or
// accumulate.
void gemm_tiled(const Tensor& a, const Tensor& b, Tensor c, bool a_mn, bool b_mn, bool accumulate, Tensor status,
                int64_t tile) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2, "gemm expects 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1, "inner stride must be 1");
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm contraction mismatch: ", K, " vs ", Kb);
  TORCH_CHECK(c.size(0) == M && c.size(1) == N, "gemm output shape mismatch");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "row strides must be multiples of 8");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(c.data_ptr()) % 16 == 0,
              "gemm operands must be 16-byte aligned");
  piper::GemmArgs g;
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.c = c.data_ptr();
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.ldc = c.stride(0);
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.a_mn_major = a_mn;
  g.b_mn_major = b_mn;
  if (c.scalar_type() == at::kBFloat16) {
    TORCH_CHECK(!accumulate, "bf16 output cannot accumulate");
    TORCH_CHECK(c.stride(0) % 8 == 0, "bf16 output row stride must be a multiple of 8");
    g.epilogue = piper::kEpiStoreBf16;
  } else {
    TORCH_CHECK(c.scalar_type() == at::kFloat, "gemm output must be bf16 or fp32");
    TORCH_CHECK(c.stride(0) % 4 == 0, "fp32 output row stride must be a multiple of 4");
    g.epilogue = piper::kEpiAccumF32;
  }
  g.accumulate = accumulate ? 1 : 0;
  g.status = status.data_ptr<int>();
  TORCH_CHECK(tile == 0 || tile == 128 || tile == 256, "gemm tile must be 0 (auto), 128 or 256");
  g.tile = static_cast<int>(tile);
  check_rc(piper::gemm_bf16_launch(g, num_sms(), cur_stream()), "gemm");
}

void gemm(const Tensor& a, const Tensor& b, Tensor c, bool a_mn, bool b_mn, bool accumulate, Tensor status) {
  gemm_tiled(a, b, c, a_mn, b_mn, accumulate, status, 0);
}

void rmsnorm_fwd(const Tensor& x, const OptTensor& res, const Tensor& w, Tensor y, const OptTensor& h_out,
                 Tensor rstd, double eps) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous(), "rmsnorm expects contiguous tensors");
  const int64_t D = x.size(-1);
  const int64_t T = x.numel() / D;
  TORCH_CHECK(res.has_value() == h_out.has_value(), "res and h_out go together");
  check_rc(piper::rmsnorm_fwd(x.data_ptr(), opt_ptr(res), w.data_ptr(), y.data_ptr(),
                              h_out.has_value() ? h_out->data_ptr() : nullptr, rstd.data_ptr<float>(), T,
                              static_cast<int>(D), static_cast<float>(eps), cur_stream()),
           "rmsnorm_fwd");
}

int64_t rmsnorm_bwd_num_partials(int64_t T) { return piper::rmsnorm_bwd_num_partials(T); }

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, const OptTensor& dres,
                 Tensor dx, Tensor dw_partial, const OptTensor& dw_f32, const OptTensor& dw_bf16,
                 bool accumulate) {
  check_bf16(dy, "dy");
  check_bf16(x, "x");
  const int64_t D = x.size(-1);
  const int64_t T = x.numel() / D;
  TORCH_CHECK(dw_partial.numel() >= piper::rmsnorm_bwd_num_partials(T) * D, "dw_partial too small");
  check_rc(piper::rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), opt_ptr(dres),
                              dx.data_ptr(), dw_partial.data_ptr<float>(), opt_f32(dw_f32),
                              dw_bf16.has_value() ? dw_bf16->data_ptr() : nullptr, accumulate ? 1 : 0, T,
                              static_cast<int>(D), cur_stream()),
           "rmsnorm_bwd", 2);
}

void qk_rope_fwd(const Tensor& qkv, Tensor out, const Tensor& cos, const Tensor& sin, const OptTensor& qw,
                 const OptTensor& kw, int64_t S, int64_t Hq, int64_t Hkv, int64_t hd, bool interleaved,
                 double eps) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(qkv.is_contiguous() && out.is_contiguous(), "qk_rope expects contiguous tensors");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat, "cos/sin must be fp32");
  TORCH_CHECK(cos.size(0) >= S && cos.size(-1) == hd / 2, "cos/sin must be [>=S, hd/2]");
  const int64_t T = qkv.numel() / ((Hq + 2 * Hkv) * hd);
  check_rc(piper::qk_rope_fwd(qkv.data_ptr(), out.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(),
                              opt_ptr(qw), opt_ptr(kw), T, static_cast<int>(S), static_cast<int>(Hq),
                              static_cast<int>(Hkv), static_cast<int>(hd), interleaved ? 1 : 0,
                              static_cast<float>(eps), cur_stream()),
           "qk_rope_fwd");
}

void qk_rope_bwd(const Tensor& dout, const Tensor& qkv, Tensor din, const Tensor& cos, const Tensor& sin,
                 const OptTensor& qw, const OptTensor& kw, const OptTensor& dqw, const OptTensor& dkw,
                 int64_t S, int64_t Hq, int64_t Hkv, int64_t hd, bool interleaved, double eps) {
  check_bf16(dout, "dout");
  const int64_t T = dout.numel() / ((Hq + 2 * Hkv) * hd);
  check_rc(piper::qk_rope_bwd(dout.data_ptr(), qkv.data_ptr(), din.data_ptr(), cos.data_ptr<float>(),
                              sin.data_ptr<float>(), opt_ptr(qw), opt_ptr(kw), opt_f32(dqw), opt_f32(dkw), T,
                              static_cast<int>(S), static_cast<int>(Hq), static_cast<int>(Hkv),
                              static_cast<int>(hd), interleaved ? 1 : 0, static_cast<float>(eps),
                              cur_stream()),
           "qk_rope_bwd");
}

void swiglu_fwd(const Tensor& h13, Tensor act) {
  check_bf16(h13, "h13");
  TORCH_CHECK(h13.is_contiguous() && act.is_contiguous(), "swiglu expects contiguous tensors");
  const int64_t F = act.size(-1);
  check_rc(piper::swiglu_fwd(h13.data_ptr(), act.data_ptr(), act.numel() / F, static_cast<int>(F), cur_stream()),
           "swiglu_fwd");
}

void swiglu_bwd(const Tensor& h13, const Tensor& dact, Tensor dh13) {
  check_bf16(h13, "h13");
  check_bf16(dact, "dact");
  TORCH_CHECK(dact.is_contiguous() && dh13.is_contiguous(), "swiglu expects contiguous tensors");
  const int64_t F = dact.size(-1);
  check_rc(piper::swiglu_bwd(h13.data_ptr(), dact.data_ptr(), dh13.data_ptr(), dact.numel() / F,
                             static_cast<int>(F), cur_stream()),
           "swiglu_bwd");
}

void embedding_fwd(const Tensor& tokens, const Tensor& table, Tensor out, Tensor status) {
  check_bf16(table, "table");
  TORCH_CHECK(tokens.scalar_type() == at::kLong && tokens.is_contiguous(), "tokens must be contiguous int64");
  check_rc(piper::embedding_fwd(reinterpret_cast<const long long*>(tokens.data_ptr<int64_t>()), table.data_ptr(),
                                out.data_ptr(), tokens.numel(), static_cast<int>(table.size(1)),
                                static_cast<int>(table.size(0)), status.data_ptr<int>(), cur_stream()),
           "embedding_fwd");
}

void embedding_bwd(const Tensor& tokens, const Tensor& dout, Tensor dtable) {
  check_bf16(dout, "dout");
  TORCH_CHECK(dtable.scalar_type() == at::kFloat, "dtable must be fp32");
  check_rc(piper::embedding_bwd(reinterpret_cast<const long long*>(tokens.data_ptr<int64_t>()), dout.data_ptr(),
                                dtable.data_ptr<float>(), tokens.numel(), static_cast<int>(dtable.size(1)),
                                static_cast<int>(dtable.size(0)), cur_stream()),
           "embedding_bwd");
}

void ce_fwd(const Tensor& logits, const Tensor& labels, Tensor loss, Tensor lse, int64_t ignore_index) {
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "logits must be [T, V] with unit inner stride");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous(), "labels must be contiguous int64");
  check_rc(piper::ce_fwd(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                         loss.data_ptr<float>(), lse.data_ptr<float>(), logits.size(0),
                         static_cast<int>(logits.size(1)), logits.stride(0), ignore_index, cur_stream()),
           "ce_fwd");
}

void ce_bwd(const Tensor& logits, const Tensor& labels, const Tensor& lse, const Tensor& gscale, double row_scale,
            Tensor out, int64_t ignore_index) {
  check_bf16(logits, "logits");
  TORCH_CHECK(out.stride(0) == logits.stride(0), "out must share the row stride of logits");
  TORCH_CHECK(gscale.scalar_type() == at::kFloat, "gscale must be fp32");
  check_rc(piper::ce_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                         lse.data_ptr<float>(), gscale.data_ptr<float>(), static_cast<float>(row_scale),
                         out.data_ptr(), logits.size(0), static_cast<int>(logits.size(1)), logits.stride(0),
                         ignore_index, cur_stream()),
           "ce_bwd");
}

void adam_flat(Tensor master, Tensor m, Tensor v, const Tensor& grad, const OptTensor& param_bf16, double lr,
               double b1, double b2, double eps, double wd, int64_t step, double grad_scale, bool decoupled) {
  TORCH_CHECK(master.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat, "adam buffers are fp32");
  TORCH_CHECK(master.is_contiguous() && m.is_contiguous() && v.is_contiguous() && grad.is_contiguous(),
              "adam buffers must be contiguous");
  check_rc(piper::adam_flat(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                            grad.data_ptr<float>(), param_bf16.has_value() ? param_bf16->data_ptr() : nullptr,
                            master.numel(), static_cast<float>(lr), static_cast<float>(b1),
                            static_cast<float>(b2), static_cast<float>(eps), static_cast<float>(wd),
                            static_cast<int>(step), static_cast<float>(grad_scale), decoupled ? 1 : 0,
                            cur_stream()),
           "adam_flat");
}

void cast_f32_to_bf16(const Tensor& in, Tensor out, double scale) {
  check_rc(piper::cast_f32_to_bf16(in.data_ptr<float>(), out.data_ptr(), in.numel(), static_cast<float>(scale),
                                   cur_stream()),
           "cast_f32_to_bf16");
}

void add_bf16(const Tensor& a, const Tensor& b, Tensor out) {
  check_bf16(a, "a");
  check_bf16(b, "b");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && out.is_contiguous() && a.numel() == b.numel(),
              "add_bf16 expects contiguous tensors of equal size");
  check_rc(piper::add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), cur_stream()), "add_bf16");
}

void accum_bf16_into_f32(const Tensor& g, Tensor acc) {
  check_bf16(g, "g");
  TORCH_CHECK(g.is_contiguous() && acc.is_contiguous() && g.numel() == acc.numel(), "accum shape mismatch");
  check_rc(piper::accum_bf16_into_f32(g.data_ptr(), acc.data_ptr<float>(), g.numel(), cur_stream()),
           "accum_bf16_into_f32");
}

void attn_fwd(const Tensor& qkv, Tensor out, Tensor lse, int64_t B, int64_t S, int64_t Hq, int64_t Hkv,
              int64_t hd, double scale, Tensor status) {
  check_bf16(qkv, "qkv");
  TORCH_CHECK(qkv.is_contiguous() && out.is_contiguous(), "attention expects contiguous tensors");
  TORCH_CHECK(qkv.numel() == B * S * (Hq + 2 * Hkv) * hd, "qkv has the wrong size");
  check_rc(piper::attn_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), static_cast<int>(B),
                           static_cast<int>(S), static_cast<int>(Hq), static_cast<int>(Hkv),
                           static_cast<int>(hd), static_cast<float>(scale), status.data_ptr<int>(),
                           cur_stream()),
           "attn_fwd");
}

void attn_bwd(const Tensor& qkv, const Tensor& out, const Tensor& dout, const Tensor& lse, Tensor delta,
              Tensor dqkv, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t hd, double scale,
              Tensor status) {
  check_bf16(qkv, "qkv");
  check_bf16(dout, "dout");
  TORCH_CHECK(dout.is_contiguous() && dqkv.is_contiguous(), "attention expects contiguous tensors");
  check_rc(piper::attn_bwd(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(),
                           delta.data_ptr<float>(), dqkv.data_ptr(), static_cast<int>(B), static_cast<int>(S),
                           static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<int>(hd),
                           static_cast<float>(scale), status.data_ptr<int>(), cur_stream()),
           "attn_bwd", 3);
}

}  // namespace

#include "bindings_moe.inc"
#include "bindings_fused.inc"

TORCH_LIBRARY(piper_c, m) {
  m.def("kernel_launch_count", &kernel_launch_count);
  m.def("gemm", &gemm);
  m.def("gemm_tiled", &gemm_tiled);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd_num_partials", &rmsnorm_bwd_num_partials);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("qk_rope_fwd", &qk_rope_fwd);
  m.def("qk_rope_bwd", &qk_rope_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd", &ce_bwd);
  m.def("adam_flat", &adam_flat);
  m.def("cast_f32_to_bf16", &cast_f32_to_bf16);
  m.def("accum_bf16_into_f32", &accum_bf16_into_f32);
  m.def("add_bf16", &add_bf16);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  register_moe_ops(m);
  register_fused_ops(m);
}
