// Host-side optimizer kernels for CPU-resident training state: fp32 AdamW over pinned host memory (OpenMP), with the bf16
// working copy written in the same pass so the next host->device weight stream needs no extra conversion sweep.
// Reference counterpart: csrc/src/runtime/optimizers/cpu_adamw.cpp.
#include <cmath>
#include <cstdint>
#include <cstring>

#include "host_api.h"

namespace sg {

static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = static_cast<uint32_t>(v) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
    u += 0x7FFFu + ((u >> 16) & 1u);                                                       // round to nearest even
    return static_cast<uint16_t>(u >> 16);
}

void cpu_adamw_step(float* param, float* m, float* v, const void* grad, bool grad_is_bf16, uint16_t* work_bf16, int64_t n, float lr, float beta1,
                    float beta2, float eps, float weight_decay, float grad_scale, int64_t step, const uint8_t* decay_mask) {
    const float bc1 = 1.0f - std::pow(beta1, static_cast<float>(step));
    const float bc2 = 1.0f - std::pow(beta2, static_cast<float>(step));
    const float step_size = lr / bc1;
    const float inv_sqrt_bc2 = 1.0f / std::sqrt(bc2);
    const float* g32 = static_cast<const float*>(grad);
    const uint16_t* g16 = static_cast<const uint16_t*>(grad);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float g = (grad_is_bf16 ? bf16_to_f32(g16[i]) : g32[i]) * grad_scale;
        const float mi = beta1 * m[i] + (1.0f - beta1) * g;
        const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
        m[i] = mi;
        v[i] = vi;
        float p = param[i];
        if (!decay_mask || decay_mask[i]) p -= lr * weight_decay * p;
        p -= step_size * mi / (std::sqrt(vi) * inv_sqrt_bc2 + eps);
        param[i] = p;
        if (work_bf16) work_bf16[i] = f32_to_bf16(p);
    }
}

double cpu_sum_squares(const void* x, bool is_bf16, int64_t n) {
    double acc = 0.0;
    const float* x32 = static_cast<const float*>(x);
    const uint16_t* x16 = static_cast<const uint16_t*>(x);
#pragma omp parallel for reduction(+ : acc) schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const double t = is_bf16 ? bf16_to_f32(x16[i]) : x32[i];
        acc += t * t;
    }
    return acc;
}

}  // namespace sg
