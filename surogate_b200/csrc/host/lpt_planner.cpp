// Least-loaded expert-parallel planner: longest-processing-time-first assignment of experts to ranks with token-range
// spilling.  Experts are visited from the most to the least loaded; each stays on the rank that owns its weights while that
// rank has capacity (capacity_factor x the mean load), the overflow goes to whichever rank currently has the least work, in
// pieces of at least min_tokens_per_gemm tokens so no helper receives a GEMM too small to be worth the weight transfer.
// Reference counterpart: csrc/src/runtime/ep/lpt_planner.h:56-80.
#include <algorithm>
#include <numeric>

#include "host_api.h"

namespace sg {

float imbalance_ratio(const int64_t* counts, int E, int ep) {
    const int local = E / ep;
    int64_t total = 0, worst = 0;
    for (int g = 0; g < ep; ++g) {
        int64_t load = 0;
        for (int e = g * local; e < (g + 1) * local; ++e) load += counts[e];
        total += load;
        worst = std::max(worst, load);
    }
    return total == 0 ? 1.0f : static_cast<float>(static_cast<double>(worst) * ep / static_cast<double>(total));
}

LptPlan compute_lpt_plan(const int64_t* counts, int E, int ep, float threshold, float capacity_factor, int min_chunk) {
    LptPlan plan;
    const int local = E / ep;
    plan.assignments.resize(E);
    plan.gpu_loads.assign(ep, 0);
    plan.expert_to_gpu.resize(E);
    plan.imbalance = imbalance_ratio(counts, E, ep);
    int64_t total = 0;
    for (int e = 0; e < E; ++e) total += counts[e];
    if (plan.imbalance <= threshold || ep == 1 || total == 0) {
        for (int e = 0; e < E; ++e) {
            const int g = e / local;
            plan.assignments[e].push_back({g, 0, static_cast<int>(counts[e])});
            plan.gpu_loads[g] += counts[e];
            plan.expert_to_gpu[e] = g;
        }
        return plan;
    }
    plan.uses_lpt = true;
    const int64_t capacity = static_cast<int64_t>(capacity_factor * static_cast<double>(total) / ep) + 1;
    std::vector<int> order(E);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return counts[a] > counts[b]; });
    for (int e : order) {
        const int native = e / local;
        int64_t remaining = counts[e], start = 0;
        auto give = [&](int g, int64_t n) {
            if (n <= 0) return;
            plan.assignments[e].push_back({g, static_cast<int>(start), static_cast<int>(start + n)});
            plan.gpu_loads[g] += n;
            if (g != native) plan.moves.push_back({e, native, g});
            start += n;
            remaining -= n;
        };
        int64_t room = std::max<int64_t>(0, capacity - plan.gpu_loads[native]);
        if (remaining <= room || remaining < 2 * static_cast<int64_t>(min_chunk)) {
            give(native, remaining);  // fits, or too small to be worth splitting
        } else {
            int64_t keep = room >= min_chunk ? std::min(room, remaining - min_chunk) : 0;
            give(native, keep);
            int rounds = 0;
            while (remaining > 0 && rounds++ < 4 * ep) {
                int h = -1;
                for (int g = 0; g < ep; ++g)
                    if (g != native && (h < 0 || plan.gpu_loads[g] < plan.gpu_loads[h])) h = g;
                int64_t take = std::max<int64_t>(capacity - plan.gpu_loads[h], min_chunk);
                take = std::min(take, remaining);
                if (remaining - take < min_chunk) take = remaining;  // never leave a sliver behind
                give(h, take);
            }
            if (remaining > 0) give(native, remaining);
        }
        int best = native;
        int64_t best_n = -1;
        for (auto& c : plan.assignments[e])
            if (c.token_end - c.token_start > best_n) { best_n = c.token_end - c.token_start; best = c.gpu; }
        plan.expert_to_gpu[e] = best;
        if (plan.assignments[e].empty()) plan.assignments[e].push_back({native, 0, 0});
    }
    return plan;
}

// Expert re-placement: every rank keeps exactly E/ep experts, but WHICH experts is chosen so that the per-rank token load is
// even.  Experts are visited from the most to the least loaded; one stays where it is while that rank has a free slot and its
// load stays within (1 + tolerance) of the mean, otherwise it goes to the least-loaded rank that still has a free slot.
// placement[e] = rank * (E/ep) + slot.  Experts that do not change rank keep their slot, so only real moves cost traffic.
std::vector<int> balanced_placement(const int64_t* counts, int E, int ep, const int* current, float tolerance, int* moved_out) {
    const int El = E / ep;
    int64_t total = 0;
    for (int e = 0; e < E; ++e) total += counts[e];
    const double target = static_cast<double>(total) / ep * (1.0 + tolerance);
    std::vector<int> order(E), rank_of(E, -1), free_slots(ep, El);
    std::vector<int64_t> load(ep, 0);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return counts[a] > counts[b]; });
    for (int e : order) {
        const int cur = current[e] / El;
        int pick = -1;
        if (free_slots[cur] > 0 && static_cast<double>(load[cur] + counts[e]) <= target) pick = cur;
        if (pick < 0) {
            for (int r = 0; r < ep; ++r)
                if (free_slots[r] > 0 && (pick < 0 || load[r] < load[pick] || (load[r] == load[pick] && r == cur))) pick = r;
        }
        rank_of[e] = pick;
        load[pick] += counts[e];
        free_slots[pick] -= 1;
    }
    std::vector<int> placement(E, -1);
    std::vector<std::vector<char>> used(ep, std::vector<char>(El, 0));
    int moved = 0;
    for (int e = 0; e < E; ++e)
        if (rank_of[e] == current[e] / El) { placement[e] = current[e]; used[rank_of[e]][current[e] % El] = 1; }
    for (int e = 0; e < E; ++e) {
        if (placement[e] >= 0) continue;
        const int r = rank_of[e];
        int slot = 0;
        while (used[r][slot]) ++slot;
        used[r][slot] = 1;
        placement[e] = r * El + slot;
        ++moved;
    }
    if (moved_out) *moved_out = moved;
    return placement;
}

}  // namespace sg
