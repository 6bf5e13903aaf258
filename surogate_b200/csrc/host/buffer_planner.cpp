// Static buffer planning for the graph compiler: interval colouring of tensor lifetimes into one arena.
//
// Input: per tensor its size in bytes and its lifetime [first, last] in op indices.  Tensors are placed largest first (ties: earlier
// first write, then input order), each at the lowest 256-byte-aligned offset that is free during its whole lifetime; the result is
// the offset of every tensor and the arena size.  The same procedure exists in Python (dsl/graph_compiler.py: _pack) and is the
// oracle of this one; the native form keeps planning of graphs with tens of thousands of tensors (unrolled stacks, long pipelines)
// out of the interpreter.  `validate_plan` checks a plan: alignment, bounds, and that no two tensors alive at the same time overlap.
// Reference counterpart: csrc/src/runtime/dsl/buffer_plan.h, graph_compiler.cpp (region layout / baked offsets).
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <string>
#include <vector>

#include "host_api.h"

namespace sg {

static inline int64_t align256(int64_t n) { return (n + 255) / 256 * 256; }

BufferPlanResult plan_buffer_offsets(const std::vector<int64_t>& nbytes, const std::vector<int64_t>& first, const std::vector<int64_t>& last) {
    const size_t n = nbytes.size();
    BufferPlanResult out;
    out.offsets.assign(n, 0);
    std::vector<size_t> order(n);
    std::iota(order.begin(), order.end(), size_t{0});
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
        if (nbytes[a] != nbytes[b]) return nbytes[a] > nbytes[b];
        return first[a] < first[b];
    });
    std::vector<size_t> placed;
    placed.reserve(n);
    std::vector<std::pair<int64_t, int64_t>> busy;
    for (size_t idx : order) {
        busy.clear();
        for (size_t p : placed)
            if (nbytes[p] > 0 && first[p] <= last[idx] && first[idx] <= last[p]) busy.emplace_back(out.offsets[p], out.offsets[p] + align256(nbytes[p]));
        std::sort(busy.begin(), busy.end());
        int64_t off = 0;
        const int64_t need = align256(nbytes[idx]);
        for (const auto& iv : busy) {
            if (off + need <= iv.first) break;
            off = std::max(off, iv.second);
        }
        out.offsets[idx] = off;
        placed.push_back(idx);
        out.total = std::max(out.total, off + need);
    }
    return out;
}

std::string validate_buffer_plan(const std::vector<int64_t>& nbytes, const std::vector<int64_t>& first, const std::vector<int64_t>& last,
                                 const std::vector<int64_t>& offsets, int64_t total) {
    const size_t n = nbytes.size();
    for (size_t a = 0; a < n; ++a) {
        if (offsets[a] % 256) return "tensor " + std::to_string(a) + " is not 256-byte aligned";
        if (offsets[a] < 0 || offsets[a] + nbytes[a] > total) return "tensor " + std::to_string(a) + " ends outside the arena";
        for (size_t b = a + 1; b < n; ++b) {
            const bool together = first[a] <= last[b] && first[b] <= last[a];
            const bool overlap = offsets[a] < offsets[b] + nbytes[b] && offsets[b] < offsets[a] + nbytes[a];
            if (together && overlap && nbytes[a] > 0 && nbytes[b] > 0) return "tensors " + std::to_string(a) + " and " + std::to_string(b) + " alias while both are alive";
        }
    }
    return "";
}

}  // namespace sg
