// Bookkeeping for device memory handed out in stack order, and a registry of named long-lived allocations.
//
// MemoryStack manages a caller-provided address range (one large device allocation): allocate() bumps a 4 KiB-aligned
// cursor, checkpoint()/restore() bracket a phase (a layer's transients, the LM-head chunks) so that everything the phase took
// is released at once, and the high-water mark says how large the range has to be.  Because a phase always receives the
// same addresses, kernels captured in a CUDA graph keep valid pointers.  AllocationRegistry records what lives outside the
// stack (weights, gradients, optimizer state, staging buffers) by category and memory kind for the memory breakdown.
// Reference counterparts: csrc/src/utilities/stack.{h,cpp} (DeviceMemoryStack), allocator.{h,cpp} (TensorAllocator stats).
#include <algorithm>
#include <string>
#include <stdexcept>

#include "host_api.h"

namespace sg {

MemoryStack::MemoryStack(uint64_t base, uint64_t capacity, uint64_t align) : base_(base), capacity_(capacity), align_(align ? align : 1) {
    if (align_ & (align_ - 1)) throw std::invalid_argument("MemoryStack: alignment must be a power of two");
    if (base_ % align_) throw std::invalid_argument("MemoryStack: base address is not aligned");
}

uint64_t MemoryStack::allocate(uint64_t bytes, const std::string& name) {
    const uint64_t size = (std::max<uint64_t>(bytes, 1) + align_ - 1) / align_ * align_;
    if (used_ + size > capacity_) {
        std::string msg = "MemoryStack: '" + name + "' needs " + std::to_string(size) + " bytes, " + std::to_string(capacity_ - used_) + " of " +
                          std::to_string(capacity_) + " free; live:";
        for (const Block& b : live_) msg += " " + b.name + "=" + std::to_string(b.bytes);
        throw std::runtime_error(msg);
    }
    const uint64_t addr = base_ + used_;
    live_.push_back({name, used_, size});
    used_ += size;
    high_water_ = std::max(high_water_, used_);
    uint64_t& peak = peak_by_name_[name];
    peak = std::max(peak, size);
    ++allocations_;
    return addr;
}

void MemoryStack::restore(size_t checkpoint) {
    if (checkpoint > live_.size()) throw std::invalid_argument("MemoryStack: checkpoint is above the current depth");
    while (live_.size() > checkpoint) {
        used_ = live_.back().offset;
        live_.pop_back();
    }
}

void MemoryStack::free_last(uint64_t address) {
    if (live_.empty() || base_ + live_.back().offset != address) throw std::invalid_argument("MemoryStack: only the most recent allocation can be freed");
    used_ = live_.back().offset;
    live_.pop_back();
}

std::vector<std::pair<std::string, uint64_t>> MemoryStack::live() const {
    std::vector<std::pair<std::string, uint64_t>> out;
    for (const Block& b : live_) out.emplace_back(b.name, b.bytes);
    return out;
}

void AllocationRegistry::record(const std::string& name, const std::string& category, const std::string& kind, uint64_t bytes) {
    static const char* kinds[] = {"device", "managed", "pinned", "write_combined", "host"};
    if (std::find(std::begin(kinds), std::end(kinds), kind) == std::end(kinds)) throw std::invalid_argument("AllocationRegistry: unknown memory kind '" + kind + "'");
    release(name);
    entries_[name] = {category, kind, bytes};
    uint64_t& cur = current_[kind];
    cur += bytes;
    uint64_t& peak = peak_[kind];
    peak = std::max(peak, cur);
}

void AllocationRegistry::release(const std::string& name) {
    auto it = entries_.find(name);
    if (it == entries_.end()) return;
    current_[it->second.kind] -= it->second.bytes;
    entries_.erase(it);
}

std::map<std::string, uint64_t> AllocationRegistry::by_category(const std::string& kind) const {
    std::map<std::string, uint64_t> out;
    for (const auto& kv : entries_)
        if (kind.empty() || kv.second.kind == kind) out[kv.second.category] += kv.second.bytes;
    return out;
}

std::map<std::string, uint64_t> AllocationRegistry::by_kind(bool peak) const { return peak ? peak_ : current_; }

std::vector<std::pair<std::string, uint64_t>> AllocationRegistry::largest(size_t n) const {
    std::vector<std::pair<std::string, uint64_t>> out;
    for (const auto& kv : entries_) out.emplace_back(kv.first, kv.second.bytes);
    std::sort(out.begin(), out.end(), [](const auto& a, const auto& b) { return a.second > b.second || (a.second == b.second && a.first < b.first); });
    if (out.size() > n) out.resize(n);
    return out;
}

}  // namespace sg
