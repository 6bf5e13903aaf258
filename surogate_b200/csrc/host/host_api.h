// Declarations shared by the host runtime sources and their Python bindings.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace sg {

// cpu_optim.cpp
void cpu_adamw_step(float* param, float* m, float* v, const void* grad, bool grad_is_bf16, uint16_t* work_bf16, int64_t n, float lr, float beta1,
                    float beta2, float eps, float weight_decay, float grad_scale, int64_t step, const uint8_t* decay_mask = nullptr);
double cpu_sum_squares(const void* x, bool is_bf16, int64_t n);
struct AdamJob {   // one flat buffer of an update; ``work_bf16`` / ``work_f32``: optional copy of the new values in the streaming dtype
    float *param, *m, *v;
    const void* grad;
    bool grad_is_bf16;
    uint16_t* work_bf16;
    float* work_f32;
    int64_t n;
    const uint8_t* decay_mask;
};
struct AdamHyper {
    float lr, beta1, beta2, eps, weight_decay, grad_scale;
    int64_t step;
};
class AsyncAdamW {   // depth-1 queue + worker thread (overlap) or inline execution (overlap = false)
public:
    explicit AsyncAdamW(bool overlap);
    ~AsyncAdamW();
    AsyncAdamW(const AsyncAdamW&) = delete;
    AsyncAdamW& operator=(const AsyncAdamW&) = delete;
    void submit(std::vector<AdamJob> jobs, const AdamHyper& hyper);
    void drain();
    long completed() const;
    bool overlap() const;

private:
    struct Impl;
    Impl* impl_;
};

// memory_stack.cpp
class MemoryStack {   // stack-ordered sub-allocation of one address range (bookkeeping only: the caller owns the memory)
public:
    MemoryStack(uint64_t base, uint64_t capacity, uint64_t align = 4096);
    uint64_t allocate(uint64_t bytes, const std::string& name);   // address; throws with the live blocks listed when the range is full
    size_t checkpoint() const { return live_.size(); }
    void restore(size_t checkpoint);                              // frees everything allocated after the checkpoint
    void free_last(uint64_t address);
    uint64_t used() const { return used_; }
    uint64_t capacity() const { return capacity_; }
    uint64_t high_water() const { return high_water_; }
    uint64_t allocations() const { return allocations_; }
    std::vector<std::pair<std::string, uint64_t>> live() const;
    const std::map<std::string, uint64_t>& peak_by_name() const { return peak_by_name_; }

private:
    struct Block {
        std::string name;
        uint64_t offset, bytes;
    };
    uint64_t base_, capacity_, align_, used_ = 0, high_water_ = 0, allocations_ = 0;
    std::vector<Block> live_;
    std::map<std::string, uint64_t> peak_by_name_;
};
class AllocationRegistry {   // named long-lived allocations by category (weights, gradients, ...) and memory kind
public:
    void record(const std::string& name, const std::string& category, const std::string& kind, uint64_t bytes);
    void release(const std::string& name);
    std::map<std::string, uint64_t> by_category(const std::string& kind = "") const;
    std::map<std::string, uint64_t> by_kind(bool peak = false) const;
    std::vector<std::pair<std::string, uint64_t>> largest(size_t n) const;
    size_t size() const { return entries_.size(); }

private:
    struct Entry {
        std::string category, kind;
        uint64_t bytes;
    };
    std::map<std::string, Entry> entries_;
    std::map<std::string, uint64_t> current_, peak_;
};

// lpt_planner.cpp
struct ExpertChunk {
    int gpu, token_start, token_end;
};
struct WeightMove {
    int expert, src_rank, dst_rank;
};
struct LptPlan {
    std::vector<std::vector<ExpertChunk>> assignments;  // per expert
    std::vector<WeightMove> moves;
    std::vector<int64_t> gpu_loads;
    std::vector<int> expert_to_gpu;  // rank that handles most of the expert's tokens
    bool uses_lpt = false;
    float imbalance = 1.0f;
};
float imbalance_ratio(const int64_t* counts, int num_experts, int ep_size);
std::vector<int> balanced_placement(const int64_t* counts, int num_experts, int ep_size, const int* current, float tolerance, int* moved_out);
LptPlan compute_lpt_plan(const int64_t* counts, int num_experts, int ep_size, float threshold, float capacity_factor, int min_tokens_per_gemm);

// crash_handler.cpp
void install_crash_handler(const std::string& tag);

// nvml_info.cpp
struct GpuTelemetry {
    bool ok = false;
    std::string name, error;
    unsigned sm_clock_mhz = 0, sm_clock_max_mhz = 0, mem_clock_mhz = 0, power_mw = 0, power_limit_mw = 0, temperature_c = 0, gpu_util = 0, mem_util = 0;
    unsigned long long mem_used = 0, mem_total = 0, throttle_reasons = 0, pcie_rx_kbs = 0, pcie_tx_kbs = 0;
};
GpuTelemetry query_gpu(int index);  // read-only NVML queries through a dlopen'ed libnvidia-ml

// buffer_planner.cpp
struct BufferPlanResult {
    std::vector<int64_t> offsets;
    int64_t total = 0;
};
BufferPlanResult plan_buffer_offsets(const std::vector<int64_t>& nbytes, const std::vector<int64_t>& first, const std::vector<int64_t>& last);
std::string validate_buffer_plan(const std::vector<int64_t>& nbytes, const std::vector<int64_t>& first, const std::vector<int64_t>& last,
                                 const std::vector<int64_t>& offsets, int64_t total);

}  // namespace sg
