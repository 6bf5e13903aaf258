// Bindings for the peer-memory communication kernels (and, below, attention / MoE / NVFP4 as they are added).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <string>

#include "attention_sm100.h"
#include "conv1d_kernels.h"
#include "normuon_kernels.h"
#include "qlora_kernels.h"
#include "comm_kernels.h"
#include "ep_kernels.h"
#include "gemm_sm100.h"
#include "moe_kernels.h"
#include "nvfp4_kernels.h"
#include "ext_api.h"

namespace {
using torch::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

sg::PeerPtrs to_peers(const std::vector<int64_t>& ptrs, int64_t byte_offset = 0) {
    TORCH_CHECK(!ptrs.empty() && ptrs.size() <= sg::kMaxPeers, "1..8 peer pointers expected");
    sg::PeerPtrs p{};
    for (size_t i = 0; i < ptrs.size(); ++i) p.p[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]) + byte_offset);
    return p;
}

void symm_barrier(const std::vector<int64_t>& pads, int64_t rank, int64_t epoch, int64_t slot_base, Tensor& error_flag, double budget_s) {
    sg_count_launch(1);
    sg::symm_barrier(to_peers(pads), static_cast<int>(rank), static_cast<int>(pads.size()), static_cast<uint32_t>(epoch), static_cast<int>(slot_base),
                     error_flag.data_ptr<int>(), budget_s, cur_stream());
}

// bufs: base pointers of every rank's arena; byte_offset: where this bucket's full gradient buffer starts inside the arena.
void reduce_scatter_fused(const std::vector<int64_t>& bufs, int64_t byte_offset, int64_t shard_elems, int64_t rank, double scale, Tensor& out,
                          bool accumulate, const c10::optional<Tensor>& sumsq_out, int64_t max_blocks) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == shard_elems, "reduce_scatter: out must be a contiguous shard");
    TORCH_CHECK(shard_elems % 8 == 0 && byte_offset % 16 == 0, "reduce_scatter: shard must be a multiple of 8 elements, 16-byte aligned");
    TORCH_CHECK(out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16, "reduce_scatter: out must be fp32 or bf16");
    TORCH_CHECK(!accumulate || out.scalar_type() == at::kFloat, "reduce_scatter: accumulate needs an fp32 shard");
    float* ss = (sumsq_out.has_value() && sumsq_out->defined()) ? sumsq_out->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::reduce_scatter_fused(to_peers(bufs, byte_offset), 0, static_cast<size_t>(shard_elems), static_cast<int>(rank), static_cast<int>(bufs.size()),
                             static_cast<float>(scale), out.data_ptr(), out.scalar_type() == at::kFloat, accumulate, ss, static_cast<int>(max_blocks),
                             cur_stream());
}

void reduce_scatter_multimem(int64_t mc_base, int64_t byte_offset, int64_t shard_elems, int64_t rank, double scale, Tensor& out,
                             const c10::optional<Tensor>& sumsq_out, int64_t max_blocks) {
    TORCH_CHECK(mc_base != 0, "reduce_scatter_multimem: no multicast mapping");
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == shard_elems && shard_elems % 8 == 0 && byte_offset % 16 == 0, "bad shard");
    float* ss = (sumsq_out.has_value() && sumsq_out->defined()) ? sumsq_out->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::reduce_scatter_multimem(reinterpret_cast<const void*>(static_cast<uintptr_t>(mc_base) + byte_offset), 0, static_cast<size_t>(shard_elems),
                                static_cast<int>(rank), static_cast<float>(scale), out.data_ptr(), out.scalar_type() == at::kFloat, ss,
                                static_cast<int>(max_blocks), cur_stream());
}

// shards: arena bases; byte_offset: where this bucket's master shard starts.  Gathers elements [seg_begin, seg_end) of the bucket.
void all_gather_fused(const std::vector<int64_t>& shards, int64_t byte_offset, int64_t shard_elems, int64_t seg_begin, int64_t seg_end,
                      const c10::optional<Tensor>& out_bf16, const c10::optional<Tensor>& out_fp8, const c10::optional<Tensor>& scale,
                      int64_t max_blocks) {
    TORCH_CHECK(seg_begin % 8 == 0 && seg_end % 8 == 0 && shard_elems % 8 == 0 && byte_offset % 16 == 0, "all_gather: ranges must be multiples of 8");
    void* o16 = nullptr;
    void* o8 = nullptr;
    if (out_bf16.has_value() && out_bf16->defined()) {
        TORCH_CHECK(out_bf16->scalar_type() == at::kBFloat16 && out_bf16->is_contiguous() && out_bf16->numel() >= seg_end, "all_gather: bf16 output");
        o16 = out_bf16->data_ptr();
    }
    if (out_fp8.has_value() && out_fp8->defined()) {
        TORCH_CHECK(out_fp8->element_size() == 1 && out_fp8->is_contiguous() && out_fp8->numel() >= seg_end, "all_gather: fp8 output");
        o8 = out_fp8->data_ptr();
    }
    const float* sc = (scale.has_value() && scale->defined()) ? scale->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::all_gather_fused(to_peers(shards, byte_offset), 0, static_cast<size_t>(shard_elems), static_cast<size_t>(seg_begin),
                         static_cast<size_t>(seg_end), o16, o8, sc, static_cast<int>(max_blocks), cur_stream());
}

void all_reduce_small(const std::vector<int64_t>& arenas, const std::vector<int64_t>& pads, int64_t slot_byte_offset, Tensor& data, int64_t op,
                      int64_t rank, int64_t epoch, int64_t slot_base, Tensor& error_flag, double budget_s) {
    TORCH_CHECK(data.is_cuda() && data.scalar_type() == at::kFloat && data.is_contiguous() && data.numel() <= 1024, "all_reduce_small: <=1024 fp32");
    sg_count_launch(1);
    sg::all_reduce_small(to_peers(arenas, slot_byte_offset), to_peers(pads), 0, data.data_ptr<float>(), static_cast<int>(data.numel()),
                         static_cast<int>(op), static_cast<int>(rank), static_cast<int>(arenas.size()), static_cast<uint32_t>(epoch),
                         static_cast<int>(slot_base), error_flag.data_ptr<int>(), budget_s, cur_stream());
}


int sms() {
    static int n = 0;
    if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    return n;
}

// ---------------------------------------------------------------------------------------- MoE
// logits fp32 [tokens, E] -> (topk weights fp32 [tokens, K], topk index int32 [tokens, K]); counts / prob_sum / lse_sq are accumulated.
std::vector<Tensor> moe_softmax_topk(const Tensor& logits, int64_t K, bool renorm, Tensor& counts, Tensor& prob_sum, const c10::optional<Tensor>& lse_sq,
                                     bool want_probs) {
    TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.dim() == 2, "logits: fp32 [tokens, E]");
    const int tokens = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
    TORCH_CHECK(E <= 256 && K <= 16 && K <= E, "moe_softmax_topk supports E <= 256, K <= 16");
    TORCH_CHECK(counts.scalar_type() == at::kInt && counts.numel() == E && prob_sum.scalar_type() == at::kFloat && prob_sum.numel() == E, "counts/prob_sum [E]");
    const c10::cuda::CUDAGuard guard(logits.device());
    Tensor w = torch::empty({tokens, K}, logits.options());
    Tensor idx = torch::empty({tokens, K}, logits.options().dtype(at::kInt));
    Tensor probs;
    if (want_probs) probs = torch::empty_like(logits);
    float* lse = (lse_sq.has_value() && lse_sq->defined()) ? lse_sq->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::moe_softmax_topk(logits.data_ptr<float>(), w.data_ptr<float>(), idx.data_ptr<int>(), want_probs ? probs.data_ptr<float>() : nullptr,
                         counts.data_ptr<int>(), prob_sum.data_ptr<float>(), lse, tokens, E, static_cast<int>(K), renorm, sms(), cur_stream());
    return {w, idx, probs};
}

// d_logits (bf16 [tokens, E]) of the router from d(top-k weights) [tokens, K] (optional), the forward's per-expert counts (optional: needed
// with an auxiliary loss) and d_aux, the gradient of the auxiliary loss as a device scalar (optional).
Tensor moe_router_bwd(const Tensor& logits, const Tensor& topk_idx, const c10::optional<Tensor>& d_topk_w, const c10::optional<Tensor>& counts,
                      const c10::optional<Tensor>& d_aux, bool renorm, double aux_coef, double z_coef) {
    TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.dim() == 2, "logits: fp32 [tokens, E]");
    TORCH_CHECK(topk_idx.scalar_type() == at::kInt && topk_idx.is_contiguous(), "topk_idx: contiguous int32");
    const int tokens = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
    const int K = static_cast<int>(topk_idx.numel() / tokens);
    TORCH_CHECK(E <= 256 && K <= 16, "moe_router_bwd supports E <= 256, K <= 16");
    auto fptr = [](const c10::optional<Tensor>& t) -> const float* {
        if (!t.has_value() || !t->defined()) return nullptr;
        TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "expected contiguous fp32");
        return t->data_ptr<float>();
    };
    const int* cp = nullptr;
    if (counts.has_value() && counts->defined()) {
        TORCH_CHECK(counts->scalar_type() == at::kInt && counts->numel() == E, "counts: int32 [E]");
        cp = counts->data_ptr<int>();
    }
    const c10::cuda::CUDAGuard guard(logits.device());
    Tensor d_logits = torch::empty({tokens, E}, logits.options().dtype(at::kBFloat16));
    sg_count_launch(1);
    sg::moe_router_bwd(logits.data_ptr<float>(), topk_idx.data_ptr<int>(), fptr(d_topk_w), cp, fptr(d_aux), d_logits.data_ptr(), tokens, E, K, renorm,
                       static_cast<float>(aux_coef), static_cast<float>(z_coef), sms(), cur_stream());
    return d_logits;
}

// counts int32 [E_local] -> padded offsets int32 [E_local + 1]; cursors zeroed.
void moe_offsets(const Tensor& counts, Tensor& offsets, Tensor& cursors, int64_t capacity_rows, Tensor& error_flag) {
    const int E = static_cast<int>(counts.numel());
    TORCH_CHECK(E <= 256 && offsets.numel() == E + 1 && cursors.numel() >= E, "moe_offsets: E <= 256");
    sg_count_launch(1);
    sg::moe_offsets(counts.data_ptr<int>(), offsets.data_ptr<int>(), cursors.data_ptr<int>(), E, static_cast<int>(capacity_rows),
                    error_flag.data_ptr<int>(), cur_stream());
}

void moe_permute(const Tensor& x, const Tensor& topk_idx, const Tensor& offsets, Tensor& cursors, Tensor& row_map, Tensor& xp, int64_t expert_base,
                 int64_t num_local) {
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && xp.scalar_type() == at::kBFloat16 && xp.is_contiguous(), "bf16 contiguous");
    const int C = static_cast<int>(x.size(-1));
    const int tokens = static_cast<int>(x.numel() / C), K = static_cast<int>(topk_idx.size(-1));
    TORCH_CHECK(C % 8 == 0 && K <= 16 && row_map.numel() == static_cast<int64_t>(tokens) * K, "moe_permute shapes");
    sg_count_launch(1);
    sg::moe_permute(x.data_ptr(), topk_idx.data_ptr<int>(), offsets.data_ptr<int>(), cursors.data_ptr<int>(), row_map.data_ptr<int>(), xp.data_ptr(),
                    tokens, C, K, static_cast<int>(expert_base), static_cast<int>(num_local), static_cast<int>(xp.size(0)), cur_stream());
}

Tensor moe_unpermute(const Tensor& yp, const c10::optional<Tensor>& w, const Tensor& row_map, int64_t tokens, int64_t K) {
    TORCH_CHECK(yp.scalar_type() == at::kBFloat16 && yp.is_contiguous(), "yp: bf16 contiguous");
    const int C = static_cast<int>(yp.size(-1));
    Tensor y = torch::empty({tokens, C}, yp.options());
    const float* wp = (w.has_value() && w->defined()) ? w->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::moe_unpermute(yp.data_ptr(), wp, row_map.data_ptr<int>(), y.data_ptr(), static_cast<int>(tokens), C, static_cast<int>(K), cur_stream());
    return y;
}

std::vector<Tensor> moe_unpermute_bwd(const Tensor& dy, const Tensor& yp, const Tensor& w, const Tensor& row_map) {
    TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && yp.is_contiguous(), "bf16 contiguous");
    const int C = static_cast<int>(yp.size(-1));
    const int tokens = static_cast<int>(dy.numel() / C), K = static_cast<int>(w.size(-1));
    Tensor d_yp = torch::zeros_like(yp);
    Tensor d_w = torch::empty_like(w);
    sg_count_launch(1);
    sg::moe_unpermute_bwd(dy.data_ptr(), yp.data_ptr(), w.data_ptr<float>(), row_map.data_ptr<int>(), d_yp.data_ptr(), d_w.data_ptr<float>(), tokens, C, K,
                          cur_stream());
    return {d_yp, d_w};
}

// Grouped GEMM (see gemm_sm100.h).  mode 1: a [R, K] (rows grouped), b = weights [G, N, K] (b_mn=false) or [G, K, N]-as-stored
// [G, Kc, N] (b_mn=true, contraction Kc); d [R, N].  mode 2: a [R, M], b [R, N] (both MN-major), d [G, M, N].
void gemm_grouped(const Tensor& a, const Tensor& b, Tensor& d, const Tensor& offsets, int64_t mode, bool b_mn, bool accumulate, double alpha,
                  const c10::optional<Tensor>& scale_a, const c10::optional<Tensor>& scale_b, Tensor& error_flag) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && d.is_cuda() && a.is_contiguous() && b.is_contiguous() && d.is_contiguous(), "contiguous CUDA tensors");
    TORCH_CHECK(a.element_size() == b.element_size() && (a.element_size() == 2 || a.element_size() == 1), "bf16 or fp8 operands");
    TORCH_CHECK(offsets.scalar_type() == at::kInt && offsets.is_cuda(), "offsets: CUDA int32");
    const c10::cuda::CUDAGuard guard(a.device());
    const int es = static_cast<int>(a.element_size());
    auto fmt = [&](const Tensor& t) { return es == 2 ? 1 : (t.scalar_type() == at::kFloat8_e5m2 ? 1 : 0); };
    sg::GemmParams p{};
    p.elem_bytes = es;
    p.a_fmt = fmt(a);
    p.b_fmt = fmt(b);
    p.mode = static_cast<int>(mode);
    p.num_groups = static_cast<int>(offsets.numel() - 1);
    p.group_offsets = offsets.data_ptr<int>();
    p.D = d.data_ptr();
    p.out_fp32 = d.scalar_type() == at::kFloat;
    p.accumulate = accumulate;
    p.alpha = static_cast<float>(alpha);
    p.scale_a = (scale_a.has_value() && scale_a->defined()) ? scale_a->data_ptr<float>() : nullptr;
    p.scale_b = (scale_b.has_value() && scale_b->defined()) ? scale_b->data_ptr<float>() : nullptr;
    p.error_flag = error_flag.data_ptr<int>();
    p.tile_n = 0;
    sg::GemmOperand A{a.data_ptr(), 0}, B{b.data_ptr(), 0};
    if (mode == 1) {
        TORCH_CHECK(a.dim() == 2 && b.dim() == 3 && d.dim() == 2 && b.size(0) == p.num_groups, "mode 1: a [R,K], b [G,*,*], d [R,N]");
        p.a_mn = 0;
        p.b_mn = b_mn;
        p.K = static_cast<int>(a.size(1));
        p.N = static_cast<int>(b_mn ? b.size(2) : b.size(1));
        TORCH_CHECK((b_mn ? b.size(1) : b.size(2)) == p.K, "mode 1: contraction mismatch");
        p.M = static_cast<int>(a.size(0));
        TORCH_CHECK(d.size(0) == a.size(0) && d.size(1) == p.N, "mode 1: d must be [R, N]");
        p.a_total_rows = a.size(0);
        p.b_total_rows = b.size(0) * b.size(1);
        A.row_stride_bytes = static_cast<uint64_t>(p.K) * es;
        B.row_stride_bytes = static_cast<uint64_t>(b.size(2)) * es;
        p.ldd = p.N;
    } else {
        TORCH_CHECK(mode == 2 && a.dim() == 2 && b.dim() == 2 && d.dim() == 3 && d.size(0) == p.num_groups && a.size(0) == b.size(0), "mode 2 shapes");
        p.a_mn = 1;
        p.b_mn = 1;
        p.M = static_cast<int>(a.size(1));
        p.N = static_cast<int>(b.size(1));
        p.K = 1;
        TORCH_CHECK(d.size(1) == p.M && d.size(2) == p.N, "mode 2: d must be [G, M, N]");
        p.a_total_rows = a.size(0);
        p.b_total_rows = b.size(0);
        A.row_stride_bytes = static_cast<uint64_t>(p.M) * es;
        B.row_stride_bytes = static_cast<uint64_t>(p.N) * es;
        p.ldd = p.N;
    }
    sg_count_launch(1);
    const char* err = sg::gemm_sm100(A, B, p, sms(), cur_stream());
    TORCH_CHECK(err == nullptr, err ? err : "");
}

// ---------------------------------------------------------------------------------------- expert parallel
void ep_plan(const std::vector<int64_t>& ctrl, int64_t ctrl_byte_offset, const std::vector<int64_t>& pads, const Tensor& counts, Tensor& offsets,
             Tensor& dst_base, Tensor& cursors, int64_t rank, int64_t epoch, int64_t slot_base, int64_t capacity_rows, Tensor& error_flag,
             double budget_s) {
    const int E = static_cast<int>(counts.numel()), world = static_cast<int>(ctrl.size());
    TORCH_CHECK(E <= 256 && E % world == 0 && offsets.numel() == 2 * (E / world) + 2 && dst_base.numel() == E && cursors.numel() == E, "ep_plan shapes");
    sg_count_launch(1);
    sg::ep_plan(to_peers(ctrl, ctrl_byte_offset), to_peers(pads), counts.data_ptr<int>(), offsets.data_ptr<int>(), dst_base.data_ptr<int>(),
                cursors.data_ptr<int>(), E, static_cast<int>(rank), world, static_cast<uint32_t>(epoch), static_cast<int>(slot_base),
                static_cast<int>(capacity_rows), error_flag.data_ptr<int>(), budget_s, cur_stream());
}

void ep_zero_pad_rows(Tensor& buf, const Tensor& offsets, int64_t El, int64_t capacity_rows) {
    TORCH_CHECK(buf.is_cuda() && buf.scalar_type() == at::kBFloat16 && buf.is_contiguous() && buf.dim() == 2 && buf.size(1) % 8 == 0, "buf: bf16 [rows, C]");
    TORCH_CHECK(offsets.scalar_type() == at::kInt && offsets.numel() >= 2 * El + 2 && capacity_rows <= buf.size(0), "offsets / capacity");
    const c10::cuda::CUDAGuard guard(buf.device());
    sg_count_launch(1);
    sg::ep_zero_pad_rows(buf.data_ptr(), offsets.data_ptr<int>(), static_cast<int>(El), static_cast<int>(buf.size(1)), static_cast<int>(capacity_rows), cur_stream());
}

void copy_rows_upto(const Tensor& src, Tensor& dst, const Tensor& n_rows) {
    TORCH_CHECK(src.is_cuda() && dst.is_cuda() && src.is_contiguous() && dst.is_contiguous() && src.dim() == 2 && src.sizes() == dst.sizes(), "same-shape 2-D tensors");
    TORCH_CHECK(src.element_size() == 2 && dst.element_size() == 2 && src.size(1) % 8 == 0, "16-bit elements, row length a multiple of 8");
    TORCH_CHECK(n_rows.scalar_type() == at::kInt && n_rows.is_cuda() && n_rows.numel() == 1, "n_rows: one CUDA int32");
    const c10::cuda::CUDAGuard guard(src.device());
    sg_count_launch(1);
    sg::copy_rows_upto(src.data_ptr(), dst.data_ptr(), n_rows.data_ptr<int>(), static_cast<int>(src.size(1)), sms(), cur_stream());
}

// Deterministic row claim: pos[tok*K+k] = how many earlier (in token order) copies of this rank go to the same expert.
Tensor ep_row_positions(const Tensor& topk_idx, int64_t num_experts) {
    TORCH_CHECK(topk_idx.is_cuda() && topk_idx.scalar_type() == at::kInt && topk_idx.is_contiguous(), "topk_idx: contiguous CUDA int32");
    const c10::cuda::CUDAGuard guard(topk_idx.device());
    Tensor pos = torch::empty_like(topk_idx);
    sg_count_launch(1);
    sg::ep_row_positions(topk_idx.data_ptr<int>(), pos.data_ptr<int>(), static_cast<int>(topk_idx.numel()), static_cast<int>(num_experts), cur_stream());
    return pos;
}

void ep_dispatch(const Tensor& x, const c10::optional<Tensor>& topk_idx, const c10::optional<Tensor>& w, const c10::optional<Tensor>& dst_base,
                 const c10::optional<Tensor>& cursors, Tensor& row_map, const std::vector<int64_t>& recv, int64_t recv_byte_offset, int64_t K,
                 int64_t experts_per_rank, int64_t capacity_rows, bool reuse_map, const c10::optional<Tensor>& q_scale, const c10::optional<Tensor>& amax_out) {
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous(), "x: bf16 contiguous");
    const float* qs = (q_scale.has_value() && q_scale->defined()) ? q_scale->data_ptr<float>() : nullptr;
    float* am = (amax_out.has_value() && amax_out->defined()) ? amax_out->data_ptr<float>() : nullptr;
    TORCH_CHECK(!(qs && w.has_value() && w->defined()), "ep_dispatch: FP8 rows carry no per-row weights");
    const int C = static_cast<int>(x.size(-1));
    const int tokens = static_cast<int>(x.numel() / C);
    TORCH_CHECK(C % 8 == 0 && K <= 16 && row_map.numel() == static_cast<int64_t>(tokens) * K, "ep_dispatch shapes");
    auto iptr = [](const c10::optional<Tensor>& t) { return (t.has_value() && t->defined()) ? t->data_ptr<int>() : nullptr; };
    const float* wp = (w.has_value() && w->defined()) ? w->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::ep_dispatch(x.data_ptr(), iptr(topk_idx), wp, iptr(dst_base), iptr(cursors), row_map.data_ptr<int>(), to_peers(recv, recv_byte_offset), tokens, C,
                    static_cast<int>(K), static_cast<int>(experts_per_rank), static_cast<int>(capacity_rows), reuse_map, qs, am, cur_stream());
}

std::vector<Tensor> ep_combine(const std::vector<int64_t>& outs, int64_t out_byte_offset, const c10::optional<Tensor>& w, const Tensor& row_map,
                               int64_t tokens, int64_t C, int64_t K, int64_t capacity_rows, bool keep_rows) {
    auto opts = torch::TensorOptions().dtype(at::kBFloat16).device(row_map.device());
    Tensor y = torch::empty({tokens, C}, opts);
    Tensor rows;
    if (keep_rows) rows = torch::empty({tokens * K, C}, opts);
    const float* wp = (w.has_value() && w->defined()) ? w->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    sg::ep_combine(to_peers(outs, out_byte_offset), wp, row_map.data_ptr<int>(), y.data_ptr(), keep_rows ? rows.data_ptr() : nullptr,
                   static_cast<int>(tokens), static_cast<int>(C), static_cast<int>(K), static_cast<int>(capacity_rows), cur_stream());
    return {y, rows};
}

Tensor ep_weight_grad(const Tensor& rows, const Tensor& dy, int64_t K) {
    const int C = static_cast<int>(dy.size(-1));
    const int tokens = static_cast<int>(dy.numel() / C);
    Tensor d_w = torch::empty({tokens, K}, dy.options().dtype(at::kFloat));
    sg_count_launch(1);
    sg::ep_weight_grad(rows.data_ptr(), dy.data_ptr(), d_w.data_ptr<float>(), tokens, C, static_cast<int>(K), cur_stream());
    return d_w;
}

// ---------------------------------------------------------------------------------------- NVFP4
int64_t nvfp4_sf_bytes(int64_t rows, int64_t K) { return ((rows + 127) / 128) * ((K / 16 + 3) / 4) * 512; }

// x [rows, K] bf16 -> (packed e2m1 [rows, K/2] uint8, scale factors in atom layout uint8)
std::vector<Tensor> nvfp4_quantize(const Tensor& x, const Tensor& amax, bool stochastic, int64_t seed, bool block2d, bool four_over_six) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: bf16 [rows, K]");
    const int rows = static_cast<int>(x.size(0)), K = static_cast<int>(x.size(1));
    TORCH_CHECK(K % 16 == 0 && (!block2d || rows % 16 == 0), "nvfp4_quantize: K (and rows for 2-D blocks) must be multiples of 16");
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor q = torch::empty({rows, K / 2}, x.options().dtype(at::kByte));
    Tensor sf = torch::zeros({nvfp4_sf_bytes(rows, K)}, x.options().dtype(at::kByte));
    sg_count_launch(1);
    sg::nvfp4_quantize_rows(x.data_ptr(), q.data_ptr(), sf.data_ptr(), amax.data_ptr<float>(), rows, K, stochastic, static_cast<uint32_t>(seed), block2d,
                            sms(), cur_stream(), four_over_six && !stochastic);
    return {q, sf};
}

// x [R, C] bf16 -> quantised transpose: (q [C, R/2], sf for rows = C, K = R); optional random Hadamard along R
std::vector<Tensor> nvfp4_quantize_transpose(const Tensor& x, const Tensor& amax, bool stochastic, bool hadamard, int64_t seed, int64_t sign_mask,
                                             bool four_over_six) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: bf16 [R, C]");
    const int R = static_cast<int>(x.size(0)), C = static_cast<int>(x.size(1));
    TORCH_CHECK(R % 64 == 0 && C % 64 == 0, "nvfp4_quantize_transpose: both dimensions must be multiples of 64");
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor q = torch::empty({C, R / 2}, x.options().dtype(at::kByte));
    Tensor sf = torch::zeros({nvfp4_sf_bytes(C, R)}, x.options().dtype(at::kByte));
    sg_count_launch(1);
    sg::nvfp4_quantize_transpose(x.data_ptr(), q.data_ptr(), sf.data_ptr(), amax.data_ptr<float>(), R, C, stochastic, hadamard,
                                 static_cast<uint32_t>(seed), static_cast<uint32_t>(sign_mask), cur_stream(), four_over_six && !stochastic);
    return {q, sf};
}

Tensor nvfp4_dequantize(const Tensor& q, const Tensor& sf, const Tensor& amax, double amax_div, double encode) {
    const int rows = static_cast<int>(q.size(0)), K = static_cast<int>(q.size(1)) * 2;
    const c10::cuda::CUDAGuard guard(q.device());
    Tensor out = torch::empty({rows, K}, q.options().dtype(at::kBFloat16));
    sg_count_launch(1);
    sg::nvfp4_dequantize(q.data_ptr(), sf.data_ptr(), amax.data_ptr<float>(), static_cast<float>(amax_div), out.data_ptr(), rows, K, sms(), cur_stream(),
                         static_cast<float>(encode));
    return out;
}

// d [M, N] = alpha * sa * sb * dequant(a) . dequant(b)^T on the tensor cores (block scales applied in hardware)
void gemm_nvfp4(const Tensor& a, const Tensor& sfa, const Tensor& b, const Tensor& sfb, Tensor& d, bool accumulate, double alpha,
                const c10::optional<Tensor>& scale_a, const c10::optional<Tensor>& scale_b, Tensor& error_flag) {
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kByte && a.is_contiguous() && b.scalar_type() == at::kByte && b.is_contiguous(), "packed uint8 operands");
    const int M = static_cast<int>(a.size(0)), N = static_cast<int>(b.size(0)), K = static_cast<int>(a.size(1)) * 2;
    TORCH_CHECK(b.size(1) * 2 == K && d.size(0) == M && d.size(1) == N && d.stride(1) == 1, "gemm_nvfp4 shapes");
    TORCH_CHECK(sfa.numel() >= nvfp4_sf_bytes(M, K) && sfb.numel() >= nvfp4_sf_bytes(N, K), "scale-factor buffers too small");
    TORCH_CHECK(d.scalar_type() == at::kBFloat16 || d.scalar_type() == at::kFloat, "output bf16 or fp32");
    const c10::cuda::CUDAGuard guard(a.device());
    const float* sa = (scale_a.has_value() && scale_a->defined()) ? scale_a->data_ptr<float>() : nullptr;
    const float* sb = (scale_b.has_value() && scale_b->defined()) ? scale_b->data_ptr<float>() : nullptr;
    sg_count_launch(1);
    const char* err = sg::gemm_nvfp4_sm100(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), d.data_ptr(), M, N, K, static_cast<int>(d.stride(0)),
                                           d.scalar_type() == at::kFloat, accumulate, static_cast<float>(alpha), sa, sb, error_flag.data_ptr<int>(), sms(),
                                           cur_stream());
    TORCH_CHECK(err == nullptr, err ? err : "");
}

// ---------------------------------------------------------------------------------------- attention
// `lo` (optional int32 [B, T]): first key each query may attend; see attention_fwd64_sm100.cu
static const int* lo_ptr(const c10::optional<Tensor>& lo, const Tensor& qkv) {
    if (!lo.has_value() || !lo->defined()) return nullptr;
    TORCH_CHECK(lo->is_cuda() && lo->scalar_type() == at::kInt && lo->is_contiguous() && lo->dim() == 2 && lo->size(0) == qkv.size(0) &&
                    lo->size(1) == qkv.size(1),
                "attention lower bounds: int32 [B, T] on the device");
    return lo->data_ptr<int>();
}

std::vector<Tensor> flash_attn_fwd(const Tensor& qkv, int64_t Hq, int64_t Hkv, double scale, const c10::optional<Tensor>& lo) {
    TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.is_contiguous() && qkv.dim() == 3, "qkv: bf16 [B, T, (Hq+2Hkv)*128]");
    const int B = static_cast<int>(qkv.size(0)), T = static_cast<int>(qkv.size(1));
    TORCH_CHECK(qkv.size(2) == (Hq + 2 * Hkv) * 128, "flash_attn: head_dim must be 128");
    const c10::cuda::CUDAGuard guard(qkv.device());
    Tensor out = torch::empty({B, T, Hq * 128}, qkv.options());
    Tensor lse = torch::empty({B, T, Hq}, qkv.options().dtype(at::kFloat));
    sg_count_launch(1);
    const char* err = sg::flash_attn_fwd64_sm100(qkv.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), B, T, static_cast<int>(Hq), static_cast<int>(Hkv),
                                                 static_cast<float>(scale), sg_error_flag(), cur_stream(), nullptr, lo_ptr(lo, qkv));
    TORCH_CHECK(err == nullptr, err ? err : "");
    return {out, lse};
}

Tensor flash_attn_fwd_profile(const Tensor& qkv, int64_t Hq, int64_t Hkv, double scale) {
    const int B = static_cast<int>(qkv.size(0)), T = static_cast<int>(qkv.size(1));
    Tensor out = torch::empty({B, T, Hq * 128}, qkv.options());
    Tensor lse = torch::empty({B, T, Hq}, qkv.options().dtype(at::kFloat));
    Tensor prof = torch::zeros({8}, qkv.options().dtype(at::kLong));
    const char* err = sg::flash_attn_fwd64_sm100(qkv.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), B, T, static_cast<int>(Hq), static_cast<int>(Hkv),
                                                 static_cast<float>(scale), sg_error_flag(), cur_stream(), reinterpret_cast<long long*>(prof.data_ptr<int64_t>()));
    TORCH_CHECK(err == nullptr, err ? err : "");
    return prof;
}

Tensor flash_attn_bwd_profile(const Tensor& d_out, const Tensor& qkv, const Tensor& lse, int64_t Hq, int64_t Hkv, double scale) {
    const int B = static_cast<int>(qkv.size(0)), T = static_cast<int>(qkv.size(1));
    Tensor d_qkv = torch::empty_like(qkv);
    Tensor delta = torch::zeros_like(lse);
    Tensor prof = torch::zeros({16}, qkv.options().dtype(at::kLong));
    const char* err = sg::flash_attn_bwd64_sm100(qkv.data_ptr(), d_out.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(), d_qkv.data_ptr(), B, T,
                                                 static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<float>(scale), sg_error_flag(), cur_stream(),
                                                 reinterpret_cast<long long*>(prof.data_ptr<int64_t>()));
    TORCH_CHECK(err == nullptr, err ? err : "");
    return prof;
}

// d_out [B, T, Hq*128], qkv packed, out [B, T, Hq*128], lse [B, T, Hq] -> d_qkv (packed layout).  With `lo`, `kv_qend` (int32
// [B, T/128]) is the exclusive end, in 64-row query tiles, of the queries that attend each 128-key tile.
Tensor flash_attn_bwd(const Tensor& d_out, const Tensor& qkv, const Tensor& out, const Tensor& lse, int64_t Hq, int64_t Hkv, double scale,
                      const c10::optional<Tensor>& lo, const c10::optional<Tensor>& kv_qend) {
    TORCH_CHECK(d_out.is_cuda() && d_out.scalar_type() == at::kBFloat16 && d_out.is_contiguous() && out.is_contiguous() && qkv.is_contiguous(), "bf16 contiguous");
    TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse: fp32 contiguous");
    const int B = static_cast<int>(qkv.size(0)), T = static_cast<int>(qkv.size(1));
    const c10::cuda::CUDAGuard guard(qkv.device());
    const int* lo_p = lo_ptr(lo, qkv);
    const int* qend_p = nullptr;
    if (lo_p) {
        TORCH_CHECK(kv_qend.has_value() && kv_qend->is_cuda() && kv_qend->scalar_type() == at::kInt && kv_qend->is_contiguous() &&
                        kv_qend->numel() == static_cast<int64_t>(B) * (T / 128),
                    "attention backward with lower bounds needs kv_qend: int32 [B, T/128]");
        qend_p = kv_qend->data_ptr<int>();
    }
    Tensor d_qkv = torch::empty_like(qkv);
    Tensor delta = torch::empty_like(lse);
    sg_count_launch(3);
    const char* err = sg::flash_attn_bwd_sm100(qkv.data_ptr(), out.data_ptr(), d_out.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                                               d_qkv.data_ptr(), B, T, static_cast<int>(Hq), static_cast<int>(Hkv), static_cast<float>(scale),
                                               sg_error_flag(), sms(), cur_stream(), lo_p, qend_p);
    TORCH_CHECK(err == nullptr, err ? err : "");
    return d_qkv;
}

// ---------------------------------------------------------------------------------------- NorMuon
// g: gradient of one matrix (bf16 / fp32, flat); m: bf16 momentum (updated); returns (u bf16 = Nesterov blend, sumsq fp32[1])
std::vector<Tensor> normuon_momentum(const Tensor& g, Tensor& m, const Tensor& hp, double mu) {
    TORCH_CHECK(g.is_cuda() && g.is_contiguous() && m.is_contiguous() && m.scalar_type() == at::kBFloat16 && m.numel() == g.numel(), "normuon_momentum operands");
    TORCH_CHECK(g.scalar_type() == at::kFloat || g.scalar_type() == at::kBFloat16, "gradient: fp32 or bf16");
    const c10::cuda::CUDAGuard guard(g.device());
    Tensor u = torch::empty(g.sizes(), g.options().dtype(at::kBFloat16));
    Tensor sumsq = torch::zeros({1}, g.options().dtype(at::kFloat));
    sg_count_launch(1);
    sg::normuon_momentum(g.data_ptr(), g.scalar_type() == at::kFloat, m.data_ptr(), u.data_ptr(), sumsq.data_ptr<float>(), hp.data_ptr<float>(),
                         static_cast<float>(mu), g.numel(), sms(), cur_stream());
    return {u, sumsq};
}
// 8-bit momentum: m8 int8 codes, ms fp16 scales per 128 values (both updated); numel % 128 == 0
std::vector<Tensor> normuon_momentum8(const Tensor& g, Tensor& m8, Tensor& ms, const Tensor& hp, double mu) {
    TORCH_CHECK(g.is_cuda() && g.is_contiguous() && m8.is_contiguous() && m8.scalar_type() == at::kChar && m8.numel() == g.numel() && g.numel() % 128 == 0,
                "normuon_momentum8: int8 codes of the gradient's size, a multiple of 128");
    TORCH_CHECK(ms.is_contiguous() && ms.scalar_type() == at::kHalf && ms.numel() == g.numel() / 128, "normuon_momentum8: one fp16 scale per 128 values");
    TORCH_CHECK(g.scalar_type() == at::kFloat || g.scalar_type() == at::kBFloat16, "gradient: fp32 or bf16");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(g.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(m8.data_ptr()) & 3) == 0, "normuon_momentum8: alignment");
    const c10::cuda::CUDAGuard guard(g.device());
    Tensor u = torch::empty(g.sizes(), g.options().dtype(at::kBFloat16));
    Tensor sumsq = torch::zeros({1}, g.options().dtype(at::kFloat));
    sg_count_launch(1);
    sg::normuon_momentum8(g.data_ptr(), g.scalar_type() == at::kFloat, m8.data_ptr(), ms.data_ptr(), u.data_ptr(), sumsq.data_ptr<float>(), hp.data_ptr<float>(),
                          static_cast<float>(mu), g.numel(), sms(), cur_stream());
    return {u, sumsq};
}
void normuon_normalise(Tensor& x, const Tensor& sumsq) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "x: contiguous bf16");
    const c10::cuda::CUDAGuard guard(x.device());
    sg_count_launch(1);
    sg::normuon_normalise(x.data_ptr(), sumsq.data_ptr<float>(), x.numel(), sms(), cur_stream());
}
// x [R, C] bf16 (the orthogonalised update); v fp32 [R] (updated); returns sums fp32[2]
Tensor normuon_row_stats(const Tensor& x, Tensor& v, const Tensor& hp, double beta2) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && v.scalar_type() == at::kFloat && v.numel() == x.size(0),
                "normuon_row_stats operands");
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor sums = torch::zeros({2}, x.options().dtype(at::kFloat));
    sg_count_launch(1);
    sg::normuon_row_stats(x.data_ptr(), v.data_ptr<float>(), sums.data_ptr<float>(), hp.data_ptr<float>(), static_cast<float>(beta2), static_cast<int>(x.size(0)),
                          static_cast<int>(x.size(1)), cur_stream());
    return sums;
}
// w: the slice [first, first + w.numel()) of the row-major parameter (bf16 / fp32 master), updated in place
void normuon_apply(Tensor& w, const Tensor& x, const Tensor& v, const Tensor& sums, const Tensor& hp, double update_scale, bool cautious, int64_t first) {
    TORCH_CHECK(w.is_cuda() && w.is_contiguous() && (w.scalar_type() == at::kFloat || w.scalar_type() == at::kBFloat16), "w: contiguous fp32 / bf16");
    TORCH_CHECK(x.dim() == 2 && first >= 0 && first + w.numel() <= x.numel(), "normuon_apply: slice outside the matrix");
    const c10::cuda::CUDAGuard guard(w.device());
    sg_count_launch(1);
    sg::normuon_apply(w.data_ptr(), w.scalar_type() == at::kFloat, x.data_ptr(), v.data_ptr<float>(), sums.data_ptr<float>(), hp.data_ptr<float>(),
                      static_cast<float>(update_scale), cautious, static_cast<int>(x.size(1)), static_cast<size_t>(first), static_cast<size_t>(w.numel()), sms(),
                      cur_stream());
}

// ---------------------------------------------------------------------------------------- depth-wise causal conv1d (channels-last)
static void check_conv(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& seq_id) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 3 && (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat), "x: contiguous [B, T, C] bf16 / fp32");
    TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == at::kFloat && w.dim() == 2 && w.size(0) == x.size(2) && w.size(1) >= 1 && w.size(1) <= 4,
                "w: contiguous fp32 [C, K] with K <= 4");
    TORCH_CHECK(x.size(2) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "C must be a multiple of 8 and x 16-byte aligned");
    if (seq_id.has_value() && seq_id->defined())
        TORCH_CHECK(seq_id->is_cuda() && seq_id->is_contiguous() && seq_id->scalar_type() == at::kInt && seq_id->numel() == x.size(0) * x.size(1), "seq_id: int32 [B, T]");
}
Tensor causal_conv1d_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, const c10::optional<Tensor>& seq_id, bool silu) {
    check_conv(x, w, seq_id);
    if (bias.has_value() && bias->defined()) TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == x.size(2), "bias: fp32 [C]");
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor y = torch::empty_like(x);
    sg_count_launch(1);
    sg::causal_conv1d_fwd(x.data_ptr(), w.data_ptr<float>(), (bias.has_value() && bias->defined()) ? bias->data_ptr<float>() : nullptr,
                          (seq_id.has_value() && seq_id->defined()) ? seq_id->data_ptr<int>() : nullptr, y.data_ptr(), x.scalar_type() == at::kFloat,
                          static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), static_cast<int>(x.size(2)), static_cast<int>(w.size(1)), silu, cur_stream());
    return y;
}
// dz: gradient of the convolution output before any activation -> (dx, dw fp32 [C, K], dbias fp32 [C])
std::vector<Tensor> causal_conv1d_bwd(const Tensor& dz, const Tensor& x, const Tensor& w, const c10::optional<Tensor>& seq_id) {
    check_conv(x, w, seq_id);
    TORCH_CHECK(dz.is_cuda() && dz.is_contiguous() && dz.sizes() == x.sizes() && dz.scalar_type() == x.scalar_type() && (reinterpret_cast<uintptr_t>(dz.data_ptr()) & 15) == 0,
                "dz: same shape, type and alignment as x");
    const c10::cuda::CUDAGuard guard(x.device());
    Tensor dx = torch::empty_like(x);
    Tensor dw = torch::zeros_like(w);
    Tensor db = torch::zeros({x.size(2)}, w.options());
    sg_count_launch(1);
    sg::causal_conv1d_bwd(dz.data_ptr(), x.data_ptr(), w.data_ptr<float>(), (seq_id.has_value() && seq_id->defined()) ? seq_id->data_ptr<int>() : nullptr,
                          dx.data_ptr(), dw.data_ptr<float>(), db.data_ptr<float>(), x.scalar_type() == at::kFloat, static_cast<int>(x.size(0)),
                          static_cast<int>(x.size(1)), static_cast<int>(x.size(2)), static_cast<int>(w.size(1)), cur_stream());
    return {dx, dw, db};
}

// ---------------------------------------------------------------------------------------- QLoRA storage -> bf16
// kind: "bnb_nf4" (a = absmax fp32, or a = int8 codes with b = fp32 scales per 256 blocks and c = fp32 offset), "fp8_block" (a = fp32
// scales), "nvfp4" (a = UE4M3 scale bytes, b = fp32 tensor de-scale), "mxfp4" (a = E8M0 scale bytes).
Tensor dequant_blockwise(const std::string& kind, const Tensor& codes, const Tensor& a, const c10::optional<Tensor>& b, const c10::optional<Tensor>& c,
                         int64_t n, int64_t block) {
    TORCH_CHECK(codes.is_cuda() && codes.is_contiguous() && a.is_cuda() && a.is_contiguous(), "contiguous CUDA tensors");
    TORCH_CHECK(n % 8 == 0 && n > 0, "dequant: the element count must be a positive multiple of 8");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(codes.data_ptr()) & 7) == 0, "dequant: codes must be 8-byte aligned");
    const c10::cuda::CUDAGuard guard(codes.device());
    Tensor out = torch::empty({n}, codes.options().dtype(at::kBFloat16));
    sg_count_launch(1);
    if (kind == "bnb_nf4") {
        TORCH_CHECK(codes.numel() * codes.element_size() * 2 >= n && block >= 8 && block % 8 == 0, "nf4: codes too short or bad block");
        if (a.scalar_type() == at::kFloat) {
            sg::dequant_nf4(codes.data_ptr(), a.data_ptr<float>(), nullptr, nullptr, nullptr, out.data_ptr(), n, static_cast<int>(block), sms(), cur_stream());
        } else {
            TORCH_CHECK(a.scalar_type() == at::kChar && b.has_value() && c.has_value() && b->scalar_type() == at::kFloat && c->scalar_type() == at::kFloat,
                        "nf4 double quantisation: int8 codes, fp32 scales, fp32 offset");
            sg::dequant_nf4(codes.data_ptr(), nullptr, a.data_ptr<int8_t>(), b->data_ptr<float>(), c->data_ptr<float>(), out.data_ptr(), n,
                            static_cast<int>(block), sms(), cur_stream());
        }
    } else if (kind == "fp8_block") {
        TORCH_CHECK(codes.numel() * codes.element_size() >= n && a.scalar_type() == at::kFloat && block % 8 == 0, "fp8_block operands");
        sg::dequant_fp8_block(codes.data_ptr(), a.data_ptr<float>(), out.data_ptr(), n, static_cast<int>(block), sms(), cur_stream());
    } else if (kind == "nvfp4") {
        TORCH_CHECK(b.has_value() && b->scalar_type() == at::kFloat && a.element_size() == 1 && a.numel() * 16 >= n, "nvfp4 operands");
        sg::dequant_nvfp4(codes.data_ptr(), a.data_ptr(), b->data_ptr<float>(), out.data_ptr(), n, sms(), cur_stream());
    } else if (kind == "mxfp4") {
        TORCH_CHECK(a.element_size() == 1 && a.numel() * 32 >= n, "mxfp4 operands");
        sg::dequant_mxfp4(codes.data_ptr(), a.data_ptr(), out.data_ptr(), n, sms(), cur_stream());
    } else {
        TORCH_CHECK(false, "unknown storage kind '", kind, "'");
    }
    return out;
}

}  // namespace

void sg_register_extra(pybind11::module_& m) {
    m.def("symm_barrier", &symm_barrier);
    m.def("reduce_scatter_fused", &reduce_scatter_fused);
    m.def("reduce_scatter_multimem", &reduce_scatter_multimem);
    m.def("all_gather_fused", &all_gather_fused);
    m.def("all_reduce_small", &all_reduce_small);
    m.def("moe_softmax_topk", &moe_softmax_topk);
    m.def("moe_router_bwd", &moe_router_bwd);
    m.def("moe_offsets", &moe_offsets);
    m.def("moe_permute", &moe_permute);
    m.def("moe_unpermute", &moe_unpermute);
    m.def("moe_unpermute_bwd", &moe_unpermute_bwd);
    m.def("gemm_grouped", &gemm_grouped);
    m.def("nvfp4_sf_bytes", &nvfp4_sf_bytes);
    m.def("nvfp4_quantize", &nvfp4_quantize, pybind11::arg("x"), pybind11::arg("amax"), pybind11::arg("stochastic"), pybind11::arg("seed"), pybind11::arg("block2d"),
          pybind11::arg("four_over_six") = false);
    m.def("nvfp4_quantize_transpose", &nvfp4_quantize_transpose, pybind11::arg("x"), pybind11::arg("amax"), pybind11::arg("stochastic"), pybind11::arg("hadamard"),
          pybind11::arg("seed"), pybind11::arg("sign_mask"), pybind11::arg("four_over_six") = false);
    m.def("nvfp4_dequantize", &nvfp4_dequantize, pybind11::arg("q"), pybind11::arg("sf"), pybind11::arg("amax"), pybind11::arg("amax_div"),
          pybind11::arg("encode") = 2688.0);
    m.def("gemm_nvfp4", &gemm_nvfp4);
    m.def("flash_attn_fwd", &flash_attn_fwd, pybind11::arg("qkv"), pybind11::arg("Hq"), pybind11::arg("Hkv"), pybind11::arg("scale"),
          pybind11::arg("lo") = c10::optional<Tensor>());
    m.def("flash_attn_bwd", &flash_attn_bwd, pybind11::arg("d_out"), pybind11::arg("qkv"), pybind11::arg("out"), pybind11::arg("lse"), pybind11::arg("Hq"),
          pybind11::arg("Hkv"), pybind11::arg("scale"), pybind11::arg("lo") = c10::optional<Tensor>(), pybind11::arg("kv_qend") = c10::optional<Tensor>());
    m.def("flash_attn_bwd_profile", &flash_attn_bwd_profile, "per-phase cycle counters of the backward passes (development aid)");
    m.def("flash_attn_fwd_profile", &flash_attn_fwd_profile, "per-phase cycle counters of one softmax thread (development aid)");
    m.def("dequant_blockwise", &dequant_blockwise, pybind11::arg("kind"), pybind11::arg("codes"), pybind11::arg("a"), pybind11::arg("b") = c10::optional<Tensor>(),
          pybind11::arg("c") = c10::optional<Tensor>(), pybind11::arg("n"), pybind11::arg("block") = 0);
    m.def("normuon_momentum", &normuon_momentum);
    m.def("normuon_momentum8", &normuon_momentum8);
    m.def("normuon_normalise", &normuon_normalise);
    m.def("normuon_row_stats", &normuon_row_stats);
    m.def("normuon_apply", &normuon_apply);
    m.def("causal_conv1d_fwd", &causal_conv1d_fwd, pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("bias") = c10::optional<Tensor>(),
          pybind11::arg("seq_id") = c10::optional<Tensor>(), pybind11::arg("silu") = false);
    m.def("causal_conv1d_bwd", &causal_conv1d_bwd, pybind11::arg("dz"), pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("seq_id") = c10::optional<Tensor>());
    m.def("ep_plan", &ep_plan);
    m.def("ep_dispatch", &ep_dispatch, pybind11::arg("x"), pybind11::arg("topk_idx"), pybind11::arg("w"), pybind11::arg("dst_base"), pybind11::arg("row_pos"),
          pybind11::arg("row_map"), pybind11::arg("recv"), pybind11::arg("recv_byte_offset"), pybind11::arg("K"), pybind11::arg("experts_per_rank"),
          pybind11::arg("capacity_rows"), pybind11::arg("reuse_map"), pybind11::arg("q_scale") = c10::optional<Tensor>(),
          pybind11::arg("amax_out") = c10::optional<Tensor>());
    m.def("ep_row_positions", &ep_row_positions);
    m.def("ep_zero_pad_rows", &ep_zero_pad_rows);
    m.def("copy_rows_upto", &copy_rows_upto);
    m.def("ep_combine", &ep_combine);
    m.def("ep_weight_grad", &ep_weight_grad);
}
