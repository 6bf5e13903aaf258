// Python bindings (pybind11 through torch's extension machinery) for the sm_100a kernels.
// Tensors are validated here (device, dtype, contiguity, alignment) so that kernels can assume their layout.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>

#include "gemm_sm100.h"
#include "kernels.h"
#include "ext_api.h"

namespace {

using torch::Tensor;

int num_sms() {
    static int n = 0;
    if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    return n;
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_cuda(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}
void check_bf16(const Tensor& t, const char* name) {
    check_cuda(t, name);
    TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bf16");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
const float* opt_f32(const c10::optional<Tensor>& t) {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat, "scale/amax tensors must be CUDA fp32");
    return t->data_ptr<float>();
}
float* opt_f32_mut(const c10::optional<Tensor>& t) { return const_cast<float*>(opt_f32(t)); }
const void* opt_ptr(const c10::optional<Tensor>& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }

int64_t g_launches = 0;  // kernels of this extension launched so far (host-side count)
int64_t launch_count() { return g_launches; }
Tensor error_flag_tensor();

Tensor g_error_flag;
int* error_flag_ptr() {
    if (!g_error_flag.defined()) g_error_flag = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA));
    return g_error_flag.data_ptr<int>();
}

// fmt: bf16 -> 1 ; float8_e4m3fn -> 0 ; float8_e5m2 -> 1 (uint8 tensors take the explicit *_fmt argument)
int fp8_fmt_of(const Tensor& t, int64_t explicit_fmt) {
    if (t.scalar_type() == at::kFloat8_e5m2) return 1;
    if (t.scalar_type() == at::kFloat8_e4m3fn) return 0;
    return static_cast<int>(explicit_fmt);
}

// D = alpha * sa * sb * op(A) op(B)^T (+ D).   a: [M,K] (a_mn=false) or [K,M] (a_mn=true); b: [N,K] or [K,N].
void gemm(const Tensor& a, const Tensor& b, Tensor& d, bool a_mn, bool b_mn, bool accumulate, double alpha, const c10::optional<Tensor>& scale_a,
          const c10::optional<Tensor>& scale_b, const c10::optional<Tensor>& amax_out, int64_t a_fmt, int64_t b_fmt, int64_t tile_n) {
    check_cuda(a, "a");
    check_cuda(b, "b");
    check_cuda(d, "d");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2, "gemm operands must be 2-D");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "gemm operands need a contiguous inner dimension");
    TORCH_CHECK(a.element_size() == b.element_size(), "gemm operands must have the same element width");
    const int es = static_cast<int>(a.element_size());
    TORCH_CHECK(es == 1 || (es == 2 && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16), "gemm inputs must be bf16 or fp8");
    TORCH_CHECK(d.scalar_type() == at::kBFloat16 || d.scalar_type() == at::kFloat, "gemm output must be bf16 or fp32");
    const c10::cuda::CUDAGuard guard(a.device());
    sg::GemmParams p{};
    p.M = static_cast<int>(a_mn ? a.size(1) : a.size(0));
    p.K = static_cast<int>(a_mn ? a.size(0) : a.size(1));
    p.N = static_cast<int>(b_mn ? b.size(1) : b.size(0));
    const int64_t kb = b_mn ? b.size(0) : b.size(1);
    TORCH_CHECK(kb == p.K, "gemm: contraction sizes differ (", p.K, " vs ", kb, ")");
    TORCH_CHECK(d.size(0) == p.M && d.size(1) == p.N, "gemm: output must be [", p.M, ", ", p.N, "]");
    p.elem_bytes = es;
    p.a_fmt = es == 2 ? 1 : fp8_fmt_of(a, a_fmt);
    p.b_fmt = es == 2 ? 1 : fp8_fmt_of(b, b_fmt);
    p.a_mn = a_mn;
    p.b_mn = b_mn;
    p.D = d.data_ptr();
    p.ldd = static_cast<int>(d.stride(0));
    p.out_fp32 = d.scalar_type() == at::kFloat;
    p.accumulate = accumulate;
    p.alpha = static_cast<float>(alpha);
    p.scale_a = opt_f32(scale_a);
    p.scale_b = opt_f32(scale_b);
    p.amax_out = opt_f32_mut(amax_out);
    p.error_flag = error_flag_ptr();
    p.tile_n = static_cast<int>(tile_n);
    if (const char* v = std::getenv("SUROGATE_GEMM_PREFETCH")) p.pair_prefetch = std::atoi(v);   // tuning aids; unset = the kernel's defaults
    if (const char* v = std::getenv("SUROGATE_GEMM_GROUP_M")) p.pair_group_m = std::atoi(v);
    sg::GemmOperand A{a.data_ptr(), static_cast<uint64_t>(a.stride(0)) * es};
    sg::GemmOperand B{b.data_ptr(), static_cast<uint64_t>(b.stride(0)) * es};
    g_launches += 1;
    const char* err = sg::gemm_sm100(A, B, p, num_sms(), cur_stream());
    TORCH_CHECK(err == nullptr, err ? err : "");
}

Tensor error_flag_tensor() {
    error_flag_ptr();
    return g_error_flag;
}

int64_t read_error_flag(bool reset) {
    if (!g_error_flag.defined()) return 0;
    const int64_t v = g_error_flag.item<int>();
    if (reset && v) g_error_flag.zero_();
    return v;
}

std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& residual, const Tensor& w, double eps, bool want_y,
                                const c10::optional<Tensor>& fp8_scale, const c10::optional<Tensor>& amax_out, bool want_fp8) {
    check_bf16(x, "x");
    check_bf16(w, "w");
    const int C = static_cast<int>(x.size(-1));
    TORCH_CHECK(C % 8 == 0 && w.numel() == C, "rmsnorm: C must be a multiple of 8 and match the weight");
    const int rows = static_cast<int>(x.numel() / C);
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor res_out, y, y8;
    if (residual.has_value() && residual->defined()) {
        check_bf16(*residual, "residual");
        res_out = torch::empty_like(x);
    }
    if (want_y) y = torch::empty_like(x);
    if (want_fp8) y8 = torch::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
    auto lead = x.sizes().vec();
    lead.pop_back();
    Tensor rstd = torch::empty(lead, x.options().dtype(at::kFloat));
    g_launches += 1;
    sg::rmsnorm_fwd(x.data_ptr(), opt_ptr(residual), w.data_ptr(), res_out.defined() ? res_out.data_ptr() : nullptr, y.defined() ? y.data_ptr() : nullptr,
                    rstd.data_ptr<float>(), y8.defined() ? y8.data_ptr() : nullptr, opt_f32(fp8_scale), opt_f32_mut(amax_out), rows, C,
                    static_cast<float>(eps), cur_stream());
    return {res_out, y, rstd, y8};
}

std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, const c10::optional<Tensor>& d_res) {
    check_bf16(dy, "dy");
    check_bf16(x, "x");
    check_bf16(w, "w");
    const int C = static_cast<int>(x.size(-1));
    TORCH_CHECK(C % 8 == 0 && C <= 16384, "rmsnorm_bwd: C must be a multiple of 8 and <= 16384");
    const int rows = static_cast<int>(x.numel() / C);
    const c10::cuda::CUDAGuard guard(x.device());
    if (d_res.has_value() && d_res->defined()) check_bf16(*d_res, "d_res");
    Tensor dx = torch::empty_like(x);
    const int blocks = sg::rmsnorm_bwd_blocks_wide(rows, C, num_sms());
    Tensor partial = torch::empty({blocks, C}, x.options().dtype(at::kFloat));
    Tensor dw = torch::empty({C}, x.options().dtype(at::kFloat));
    g_launches += 2;
    sg::rmsnorm_bwd_n(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), opt_ptr(d_res), dx.data_ptr(), partial.data_ptr<float>(),
                      dw.data_ptr<float>(), rows, C, blocks, cur_stream());
    return {dx, dw};
}

static const int* opt_i32(const c10::optional<Tensor>& t) {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->numel() >= 1, "expected a CUDA int32 tensor");
    return t->data_ptr<int>();
}

// rows_limit (optional, one CUDA int32): only that many leading rows are in use; the rest of the (worst-case sized) buffer is not touched
std::vector<Tensor> swiglu_fwd(const Tensor& x, bool want_y, const c10::optional<Tensor>& fp8_scale, const c10::optional<Tensor>& amax_out, bool want_fp8,
                               const c10::optional<Tensor>& rows_limit) {
    check_bf16(x, "x");
    const int M = static_cast<int>(x.size(-1) / 2);
    TORCH_CHECK(M % 8 == 0, "swiglu: M must be a multiple of 8");
    const size_t rows = x.numel() / (2 * M);
    const c10::cuda::CUDAGuard guard(x.device());
    auto shape = x.sizes().vec();
    shape.back() = M;
    Tensor y, y8;
    if (want_y) y = torch::empty(shape, x.options());
    if (want_fp8) y8 = torch::empty(shape, x.options().dtype(at::kFloat8_e4m3fn));
    g_launches += 1;
    sg::swiglu_fwd(x.data_ptr(), y.defined() ? y.data_ptr() : nullptr, y8.defined() ? y8.data_ptr() : nullptr, opt_f32(fp8_scale), opt_f32_mut(amax_out),
                   rows, M, num_sms(), cur_stream(), opt_i32(rows_limit));
    return {y, y8};
}

Tensor swiglu_bwd(const Tensor& dy, const Tensor& x, const c10::optional<Tensor>& rows_limit) {
    check_bf16(dy, "dy");
    check_bf16(x, "x");
    const int M = static_cast<int>(x.size(-1) / 2);
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor dx = torch::empty_like(x);
    g_launches += 1;
    sg::swiglu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel() / (2 * M), M, num_sms(), cur_stream(), opt_i32(rows_limit));
    return dx;
}

// The gradient as E5M2 only (its reader is an FP8 GEMM): scaled by `fp8_scale`, abs-max of the unscaled values recorded in `amax_out`.
Tensor swiglu_bwd_fp8(const Tensor& dy, const Tensor& x, const Tensor& fp8_scale, const Tensor& amax_out) {
    check_bf16(dy, "dy");
    check_bf16(x, "x");
    const int M = static_cast<int>(x.size(-1) / 2);
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor dx8 = torch::empty(x.sizes(), x.options().dtype(at::kFloat8_e5m2));
    g_launches += 1;
    sg::swiglu_bwd(dy.data_ptr(), x.data_ptr(), nullptr, x.numel() / (2 * M), M, num_sms(), cur_stream(), nullptr, dx8.data_ptr(), fp8_scale.data_ptr<float>(),
                   amax_out.data_ptr<float>());
    return dx8;
}

void zero_empty_groups(Tensor& out, const Tensor& offsets) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.dim() >= 2 && offsets.is_cuda() && offsets.scalar_type() == at::kInt, "out [G, ...] and CUDA int32 offsets");
    const int64_t G = out.size(0);
    TORCH_CHECK(offsets.numel() >= G + 1, "offsets needs G + 1 entries");
    const size_t bytes = static_cast<size_t>(out.numel() / G) * out.element_size();
    TORCH_CHECK(bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "group matrices must be multiples of 16 bytes");
    const c10::cuda::CUDAGuard guard(out.device());
    g_launches += 1;
    sg::zero_empty_groups(out.data_ptr(), offsets.data_ptr<int>(), static_cast<int>(G), bytes, cur_stream());
}

// ``pos`` is [tokens] int32, or [3, tokens] (temporal / height / width rows) when sec_h or sec_w is non-zero: frequency j then
// reads the height row if j % 3 == 1 and j < 3 * sec_h, the width row if j % 3 == 2 and j < 3 * sec_w.
std::vector<Tensor> qk_norm_rope_fwd(const Tensor& qkv, const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw, const Tensor& pos, int64_t Hq,
                                     int64_t Hkv, int64_t D, double eps, double theta, int64_t sec_h, int64_t sec_w) {
    check_bf16(qkv, "qkv");
    TORCH_CHECK(D == 128, "qk_norm_rope kernel supports head_dim 128");
    TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kInt && pos.is_contiguous(), "position_ids must be contiguous CUDA int32");
    const size_t tokens = qkv.numel() / ((Hq + 2 * Hkv) * D);
    const bool multi_axis = sec_h > 0 || sec_w > 0;
    TORCH_CHECK(static_cast<size_t>(pos.numel()) == (multi_axis ? 3 : 1) * tokens, "position_ids must have one entry per token (three rows of them for multi-axis positions)");
    const c10::cuda::CUDAGuard guard(qkv.device());
    Tensor out = torch::empty_like(qkv);
    const bool norm = qw.has_value() && qw->defined();
    Tensor q_rstd, k_rstd;
    if (norm) {
        check_bf16(*qw, "q_norm_weight");
        check_bf16(*kw, "k_norm_weight");
        auto lead = qkv.sizes().vec();
        lead.back() = Hq;
        q_rstd = torch::empty(lead, qkv.options().dtype(at::kFloat));
        lead.back() = Hkv;
        k_rstd = torch::empty(lead, qkv.options().dtype(at::kFloat));
    }
    g_launches += 1;
    sg::qk_norm_rope_fwd(qkv.data_ptr(), opt_ptr(qw), opt_ptr(kw), pos.data_ptr<int>(), out.data_ptr(), norm ? q_rstd.data_ptr<float>() : nullptr,
                         norm ? k_rstd.data_ptr<float>() : nullptr, tokens, static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<float>(eps),
                         static_cast<float>(theta), static_cast<int>(3 * sec_h), static_cast<int>(3 * sec_w), num_sms(), cur_stream());
    return {out, q_rstd, k_rstd};
}

std::vector<Tensor> qk_norm_rope_bwd(const Tensor& d_out, const Tensor& qkv_pre, const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw,
                                     const c10::optional<Tensor>& q_rstd, const c10::optional<Tensor>& k_rstd, const Tensor& pos, int64_t Hq,
                                     int64_t Hkv, int64_t D, double eps, double theta, int64_t sec_h, int64_t sec_w) {
    check_bf16(d_out, "d_out");
    check_bf16(qkv_pre, "qkv");
    TORCH_CHECK(D == 128, "qk_norm_rope kernel supports head_dim 128");
    const size_t tokens = d_out.numel() / ((Hq + 2 * Hkv) * D);
    TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kInt && pos.is_contiguous() &&
                    static_cast<size_t>(pos.numel()) == ((sec_h > 0 || sec_w > 0) ? 3 : 1) * tokens,
                "position_ids must be contiguous CUDA int32 with one entry per token (three rows for multi-axis positions)");
    const c10::cuda::CUDAGuard guard(d_out.device());
    Tensor dx = torch::empty_like(d_out);
    const bool norm = qw.has_value() && qw->defined();
    Tensor dqw, dkw;
    if (norm) {
        dqw = torch::zeros({D}, d_out.options().dtype(at::kFloat));
        dkw = torch::zeros({D}, d_out.options().dtype(at::kFloat));
    }
    g_launches += 1;
    sg::qk_norm_rope_bwd(d_out.data_ptr(), qkv_pre.data_ptr(), opt_ptr(qw), opt_ptr(kw), pos.data_ptr<int>(), dx.data_ptr(), opt_f32_mut(q_rstd),
                         opt_f32_mut(k_rstd), norm ? dqw.data_ptr<float>() : nullptr, norm ? dkw.data_ptr<float>() : nullptr, tokens,
                         static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<float>(eps), static_cast<float>(theta), static_cast<int>(3 * sec_h),
                         static_cast<int>(3 * sec_w), num_sms(), cur_stream());
    return {dx, dqw, dkw};
}

Tensor embedding_fwd(const Tensor& tokens, const Tensor& table) {
    check_bf16(table, "table");
    TORCH_CHECK(tokens.is_cuda() && tokens.scalar_type() == at::kInt && tokens.is_contiguous(), "tokens must be contiguous CUDA int32");
    const int C = static_cast<int>(table.size(1));
    TORCH_CHECK(C % 8 == 0, "embedding: C must be a multiple of 8");
    const c10::cuda::CUDAGuard guard(table.device());
    auto shape = tokens.sizes().vec();
    shape.push_back(C);
    Tensor out = torch::empty(shape, table.options());
    g_launches += 1;
    sg::embedding_fwd(tokens.data_ptr<int>(), table.data_ptr(), out.data_ptr(), tokens.numel(), C, static_cast<int>(table.size(0)), error_flag_ptr(), num_sms(),
                      cur_stream());
    return out;
}

// deterministic = true: positions sorted by token id, one CTA per run of equal ids, fp32 sums, no atomics (bit-reproducible);
// false: bf16 / fp32 atomic adds in arrival order.
void embedding_bwd(const Tensor& tokens, const Tensor& d_out, Tensor& d_table, bool deterministic) {
    check_bf16(d_out, "d_out");
    if (deterministic) {
        TORCH_CHECK(d_table.is_cuda() && d_table.is_contiguous() && (d_table.scalar_type() == at::kFloat || d_table.scalar_type() == at::kBFloat16) &&
                        d_table.size(1) % 2 == 0,
                    "d_table: contiguous fp32 / bf16 [V, C]");
        const c10::cuda::CUDAGuard guard(d_out.device());
        auto sorted = tokens.reshape({-1}).sort(/*stable=*/true, /*dim=*/0, /*descending=*/false);
        Tensor ids = std::get<0>(sorted).contiguous(), order = std::get<1>(sorted).contiguous();
        g_launches += 1;
        sg::embedding_bwd_sorted(ids.data_ptr<int>(), reinterpret_cast<const long long*>(order.data_ptr<int64_t>()), d_out.data_ptr(), d_table.data_ptr(),
                                 d_table.scalar_type() == at::kFloat, static_cast<int>(ids.numel()), static_cast<int>(d_table.size(1)),
                                 static_cast<int>(d_table.size(0)), cur_stream());
        return;
    }
    TORCH_CHECK(d_table.is_cuda() && d_table.is_contiguous(), "d_table must be contiguous CUDA");
    TORCH_CHECK(d_table.scalar_type() == at::kFloat || d_table.scalar_type() == at::kBFloat16, "d_table must be fp32 or bf16");
    const int C = static_cast<int>(d_table.size(1));
    const c10::cuda::CUDAGuard guard(d_out.device());
    g_launches += 1;
    sg::embedding_bwd(tokens.data_ptr<int>(), d_out.data_ptr(), d_table.data_ptr(), d_table.scalar_type() == at::kFloat, tokens.numel(), C, num_sms(),
                      cur_stream());
}

// logits [rows, V] bf16 (row stride ld) are overwritten with d_logits when write_grad; returns per-row losses.
Tensor cross_entropy_fwd_bwd(Tensor& logits, const Tensor& targets, const c10::optional<Tensor>& scale, double scale_host, bool write_grad,
                             const c10::optional<Tensor>& row_weight, const c10::optional<Tensor>& kd_idx, const c10::optional<Tensor>& kd_logp,
                             double kd_weight, const c10::optional<Tensor>& kd_loss_out) {
    check_cuda(logits, "logits");
    TORCH_CHECK(logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "logits must be 2-D bf16 with contiguous rows");
    TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kInt && targets.is_contiguous(), "targets must be contiguous CUDA int32");
    const int rows = static_cast<int>(logits.size(0)), V = static_cast<int>(logits.size(1)), ld = static_cast<int>(logits.stride(0));
    TORCH_CHECK(V % 8 == 0 && ld % 8 == 0, "cross_entropy: V and row stride must be multiples of 8");
    TORCH_CHECK(targets.numel() == rows, "one target per row");
    const c10::cuda::CUDAGuard guard(logits.device());
    Tensor loss = torch::empty({rows}, logits.options().dtype(at::kFloat));
    const float* rw = nullptr;
    if (row_weight.has_value() && row_weight->defined()) {
        TORCH_CHECK(row_weight->is_cuda() && row_weight->scalar_type() == at::kFloat && row_weight->is_contiguous() && row_weight->numel() == rows,
                    "row_weight must be contiguous CUDA float32 with one value per row");
        rw = row_weight->data_ptr<float>();
    }
    const int* ki = nullptr;
    const float* kl = nullptr;
    float* ko = nullptr;
    int K = 0;
    if (kd_idx.has_value() && kd_idx->defined()) {
        TORCH_CHECK(kd_logp.has_value() && kd_logp->defined(), "kd_idx needs kd_logp");
        TORCH_CHECK(kd_idx->is_cuda() && kd_idx->scalar_type() == at::kInt && kd_idx->is_contiguous() && kd_idx->dim() == 2 && kd_idx->size(0) == rows,
                    "kd_idx must be contiguous CUDA int32 [rows, K]");
        TORCH_CHECK(kd_logp->is_cuda() && kd_logp->scalar_type() == at::kFloat && kd_logp->is_contiguous() && kd_logp->sizes() == kd_idx->sizes(),
                    "kd_logp must be contiguous CUDA float32 [rows, K]");
        K = static_cast<int>(kd_idx->size(1));
        ki = kd_idx->data_ptr<int>();
        kl = kd_logp->data_ptr<float>();
        if (kd_loss_out.has_value() && kd_loss_out->defined()) {
            TORCH_CHECK(kd_loss_out->is_cuda() && kd_loss_out->scalar_type() == at::kFloat && kd_loss_out->numel() == rows, "kd_loss_out: float32 [rows]");
            ko = kd_loss_out->data_ptr<float>();
        }
    }
    g_launches += 1;
    sg::cross_entropy_fwd_bwd(logits.data_ptr(), targets.data_ptr<int>(), loss.data_ptr<float>(), opt_f32(scale), static_cast<float>(scale_host), rows, V,
                              ld, write_grad, rw, ki, kl, K, static_cast<float>(kd_weight), ko, cur_stream());
    return loss;
}

Tensor quantize_fp8(const Tensor& x, const c10::optional<Tensor>& scale, const c10::optional<Tensor>& amax_out, bool e5m2,
                    const c10::optional<Tensor>& rows_limit, const c10::optional<Tensor>& out) {
    check_bf16(x, "x");
    TORCH_CHECK(x.numel() % 8 == 0, "quantize_fp8: numel must be a multiple of 8");
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor q;
    if (out.has_value() && out->defined()) {   // caller-owned destination (a slice of a peer-visible buffer): one byte per element
        TORCH_CHECK(out->is_cuda() && out->is_contiguous() && out->element_size() == 1 && out->numel() == x.numel(), "quantize_fp8: out must hold numel bytes");
        TORCH_CHECK(reinterpret_cast<uintptr_t>(out->data_ptr()) % 8 == 0, "quantize_fp8: out must be 8-byte aligned");
        q = *out;
    } else {
        q = torch::empty(x.sizes(), x.options().dtype(e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn));
    }
    g_launches += 1;
    sg::quantize_fp8(x.data_ptr(), q.data_ptr(), opt_f32(scale), opt_f32_mut(amax_out), x.numel(), e5m2, num_sms(), cur_stream(), opt_i32(rows_limit),
                     static_cast<int>(x.size(-1)));
    return q;
}

void amax(const Tensor& x, Tensor& amax_out, const c10::optional<Tensor>& rows_limit) {
    check_bf16(x, "x");
    TORCH_CHECK(x.numel() % 8 == 0, "amax: numel must be a multiple of 8");
    const c10::cuda::CUDAGuard guard(x.device());
    g_launches += 1;
    sg::amax_bf16(x.data_ptr(), amax_out.data_ptr<float>(), x.numel(), num_sms(), cur_stream(), opt_i32(rows_limit), static_cast<int>(x.size(-1)));
}

Tensor sumsq(const Tensor& x) {
    check_cuda(x, "x");
    TORCH_CHECK(x.is_contiguous() && (x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16), "sumsq: contiguous fp32/bf16");
    const c10::cuda::CUDAGuard guard(x.device());
    const int nblocks = num_sms() * 2;
    Tensor partial = torch::empty({nblocks}, x.options().dtype(at::kFloat));
    g_launches += 1;
    sg::sumsq(x.data_ptr(), x.scalar_type() == at::kFloat, partial.data_ptr<float>(), nblocks, x.numel(), cur_stream());
    return partial.sum();
}

void adamw_step(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const c10::optional<Tensor>& mask, const Tensor& hp) {
    check_cuda(p, "p");
    TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw: contiguous tensors");
    TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && hp.scalar_type() == at::kFloat && hp.numel() >= 8, "adamw: fp32 state");
    TORCH_CHECK(p.numel() % 8 == 0, "adamw: element count must be a multiple of 8");
    const c10::cuda::CUDAGuard guard(p.device());
    g_launches += 1;
    sg::adamw_fp32(p.data_ptr(), p.scalar_type() == at::kFloat, g.data_ptr(), g.scalar_type() == at::kFloat, m.data_ptr<float>(), v.data_ptr<float>(),
                   static_cast<const uint8_t*>(opt_ptr(mask)), hp.data_ptr<float>(), p.numel(), num_sms(), cur_stream());
}

void adamw8_step(Tensor& p, const Tensor& g, Tensor& m8, Tensor& v8, Tensor& ms, Tensor& vs, const c10::optional<Tensor>& mask, const Tensor& hp) {
    check_cuda(p, "p");
    TORCH_CHECK(p.is_contiguous() && g.is_contiguous(), "adamw8: contiguous tensors");
    TORCH_CHECK(m8.scalar_type() == at::kChar && v8.scalar_type() == at::kByte && ms.scalar_type() == at::kHalf && vs.scalar_type() == at::kHalf,
                "adamw8: state dtypes int8/uint8/fp16/fp16");
    TORCH_CHECK(static_cast<size_t>(ms.numel()) * 32 >= static_cast<size_t>(p.numel()), "adamw8: one scale per 32 elements");
    TORCH_CHECK(p.numel() % 32 == 0, "adamw8: element count must be a multiple of 32");
    const c10::cuda::CUDAGuard guard(p.device());
    int block_mask = 0;  // the weight-decay mask is one byte per parameter, or one byte per 128 parameters
    if (mask.has_value() && mask->defined()) {
        TORCH_CHECK(mask->scalar_type() == at::kByte && mask->is_contiguous(), "adamw8: mask must be contiguous uint8");
        if (mask->numel() != p.numel()) {
            TORCH_CHECK(p.numel() % 128 == 0 && mask->numel() * 128 == p.numel(), "adamw8: mask needs one byte per parameter or per 128 parameters");
            block_mask = 1;
        }
    }
    g_launches += 1;
    sg::adamw_8bit(p.data_ptr(), p.scalar_type() == at::kFloat, g.data_ptr(), g.scalar_type() == at::kFloat, m8.data_ptr(), v8.data_ptr(), ms.data_ptr(),
                   vs.data_ptr(), static_cast<const uint8_t*>(opt_ptr(mask)), block_mask, hp.data_ptr<float>(), p.numel(), num_sms(), cur_stream());
}

}  // namespace

void sg_count_launch(int n) { g_launches += n; }
int* sg_error_flag() { return error_flag_ptr(); }

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("error_flag_tensor", &error_flag_tensor, "the device int32 word kernels set when a bounded wait runs out");
    m.def("gemm", &gemm, "tcgen05 GEMM");
    m.def("read_error_flag", &read_error_flag);
    m.def("launch_count", &launch_count, "number of kernels this extension has launched");
    m.def("rmsnorm_fwd", &rmsnorm_fwd);
    m.def("rmsnorm_bwd", &rmsnorm_bwd);
    m.def("swiglu_fwd", &swiglu_fwd, pybind11::arg("x"), pybind11::arg("want_y"), pybind11::arg("fp8_scale"), pybind11::arg("amax_out"), pybind11::arg("want_fp8"),
          pybind11::arg("rows_limit") = c10::optional<Tensor>());
    m.def("swiglu_bwd", &swiglu_bwd, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("rows_limit") = c10::optional<Tensor>());
    m.def("swiglu_bwd_fp8", &swiglu_bwd_fp8);
    m.def("zero_empty_groups", &zero_empty_groups, "zero the [G, ...] slices of groups that own no rows");
    m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd, py::arg("qkv"), py::arg("q_norm_weight"), py::arg("k_norm_weight"), py::arg("position_ids"), py::arg("num_q_heads"),
          py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("eps"), py::arg("theta"), py::arg("sec_h") = 0, py::arg("sec_w") = 0);
    m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd, py::arg("d_out"), py::arg("qkv"), py::arg("q_norm_weight"), py::arg("k_norm_weight"), py::arg("q_rstd"),
          py::arg("k_rstd"), py::arg("position_ids"), py::arg("num_q_heads"), py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("eps"), py::arg("theta"),
          py::arg("sec_h") = 0, py::arg("sec_w") = 0);
    m.def("embedding_fwd", &embedding_fwd);
    m.def("embedding_bwd", &embedding_bwd, py::arg("tokens"), py::arg("d_out"), py::arg("d_table"), py::arg("deterministic") = true);
    m.def("cross_entropy_fwd_bwd", &cross_entropy_fwd_bwd, py::arg("logits"), py::arg("targets"), py::arg("scale"), py::arg("scale_host"),
          py::arg("write_grad"), py::arg("row_weight") = py::none(), py::arg("kd_idx") = py::none(), py::arg("kd_logp") = py::none(),
          py::arg("kd_weight") = 0.0, py::arg("kd_loss_out") = py::none());
    m.def("quantize_fp8", &quantize_fp8, pybind11::arg("x"), pybind11::arg("scale"), pybind11::arg("amax_out"), pybind11::arg("e5m2"),
          pybind11::arg("rows_limit") = c10::optional<Tensor>(), pybind11::arg("out") = c10::optional<Tensor>());
    m.def("amax", &amax, pybind11::arg("x"), pybind11::arg("amax_out"), pybind11::arg("rows_limit") = c10::optional<Tensor>());
    m.def("sumsq", &sumsq);
    m.def("adamw_step", &adamw_step);
    m.def("adamw8_step", &adamw8_step);
    sg_register_extra(m);
    sg_register_device_io(m);
}
