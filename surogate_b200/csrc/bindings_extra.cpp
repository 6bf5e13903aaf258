// Bindings for the peer-memory communication kernels (and, below, attention / MoE / NVFP4 as they are added).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm_kernels.h"
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

}  // namespace

void sg_register_extra(pybind11::module_& m) {
    m.def("symm_barrier", &symm_barrier);
    m.def("reduce_scatter_fused", &reduce_scatter_fused);
    m.def("reduce_scatter_multimem", &reduce_scatter_multimem);
    m.def("all_gather_fused", &all_gather_fused);
    m.def("all_reduce_small", &all_reduce_small);
}
