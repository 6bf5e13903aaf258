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
    if (grad_scale == 0.0f) {   // skipped update (non-finite gradient): weights and moments stay; the streamed copy is still refreshed
        if (work_bf16) {
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) work_bf16[i] = f32_to_bf16(param[i]);
        }
        return;
    }
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

// ---------------------------------------------------------------------------------------------------------------------------
// One-step-stale optimizer worker: a dedicated thread drains a depth-1 queue of AdamW updates so that the host update of step N
// overlaps the device compute of step N+1.  submit() first waits for the previous update, so at most one is in flight and the
// weights a step reads are never more than one update old.  A failure inside the worker is kept and re-thrown by the next
// submit() / drain().  Reference counterpart: csrc/src/runtime/optimizers/async_optimizer.{h,cpp}.
#include <condition_variable>
#include <exception>
#include <mutex>
#include <stdexcept>
#include <thread>

namespace sg {

struct AsyncAdamW::Impl {
    bool overlap;
    std::thread worker;
    std::mutex mu;
    std::condition_variable work_cv, done_cv;
    bool has_job = false, stop = false;
    std::vector<AdamJob> jobs;
    AdamHyper hyper{};
    long submitted = 0, completed = 0;
    std::exception_ptr error;

    static void run(const std::vector<AdamJob>& jobs, const AdamHyper& h) {
        for (const AdamJob& j : jobs) {
            if (!j.param || !j.m || !j.v || !j.grad || j.n < 0) throw std::invalid_argument("async AdamW: null buffer or negative size in a job");
            cpu_adamw_step(j.param, j.m, j.v, j.grad, j.grad_is_bf16, j.work_bf16, j.n, h.lr, h.beta1, h.beta2, h.eps, h.weight_decay, h.grad_scale, h.step,
                           j.decay_mask);
            if (j.work_f32) std::memcpy(j.work_f32, j.param, static_cast<size_t>(j.n) * sizeof(float));
        }
    }

    void loop() {
        std::unique_lock<std::mutex> lock(mu);
        for (;;) {
            work_cv.wait(lock, [&] { return has_job || stop; });
            if (!has_job && stop) return;
            std::vector<AdamJob> mine;
            mine.swap(jobs);
            AdamHyper h = hyper;
            has_job = false;
            lock.unlock();
            std::exception_ptr err;
            try {
                run(mine, h);
            } catch (...) {
                err = std::current_exception();
            }
            lock.lock();
            if (err && !error) error = err;
            ++completed;
            done_cv.notify_all();
        }
    }

    void rethrow_locked() {
        if (error) {
            std::exception_ptr e = error;
            error = nullptr;
            std::rethrow_exception(e);
        }
    }
};

AsyncAdamW::AsyncAdamW(bool overlap) : impl_(new Impl) {
    impl_->overlap = overlap;
    if (overlap) impl_->worker = std::thread([this] { impl_->loop(); });
}

AsyncAdamW::~AsyncAdamW() {
    if (impl_->overlap) {
        {
            std::lock_guard<std::mutex> lock(impl_->mu);
            impl_->stop = true;
        }
        impl_->work_cv.notify_all();
        if (impl_->worker.joinable()) impl_->worker.join();
    }
    delete impl_;
}

void AsyncAdamW::submit(std::vector<AdamJob> jobs, const AdamHyper& hyper) {
    if (!impl_->overlap) {
        Impl::run(jobs, hyper);
        ++impl_->submitted;
        ++impl_->completed;
        return;
    }
    std::unique_lock<std::mutex> lock(impl_->mu);
    impl_->done_cv.wait(lock, [&] { return impl_->completed == impl_->submitted; });  // the previous update is done: depth 1
    impl_->rethrow_locked();
    impl_->jobs = std::move(jobs);
    impl_->hyper = hyper;
    impl_->has_job = true;
    ++impl_->submitted;
    lock.unlock();
    impl_->work_cv.notify_one();
}

void AsyncAdamW::drain() {
    if (!impl_->overlap) return;
    std::unique_lock<std::mutex> lock(impl_->mu);
    impl_->done_cv.wait(lock, [&] { return impl_->completed == impl_->submitted; });
    impl_->rethrow_locked();
}

long AsyncAdamW::completed() const {
    std::lock_guard<std::mutex> lock(impl_->mu);
    return impl_->completed;
}

bool AsyncAdamW::overlap() const { return impl_->overlap; }

}  // namespace sg
