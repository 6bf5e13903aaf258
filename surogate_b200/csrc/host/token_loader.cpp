#include "token_loader.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <numeric>
#include <stdexcept>

namespace sg {

namespace {
constexpr int kHeaderBytes = 1024;
constexpr int32_t kIgnore = -100;
const char kMagic[8] = {'B', 'I', 'N', '.', 'T', 'O', 'K', '\n'};

inline uint64_t splitmix64(uint64_t& s) {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
}  // namespace

std::vector<int64_t> shuffled_order(int64_t n, int64_t seed, int64_t epoch, int64_t salt, bool shuffle) {
    std::vector<int64_t> v(static_cast<size_t>(n));
    std::iota(v.begin(), v.end(), 0);
    if (!shuffle || n < 2) return v;
    uint64_t s = static_cast<uint64_t>(seed) * 0x9E3779B97F4A7C15ull ^ (static_cast<uint64_t>(epoch) + 0x1000) * 0xC2B2AE3D27D4EB4Full ^
                 (static_cast<uint64_t>(salt) + 0x2000) * 0x165667B19E3779F9ull;
    for (int64_t i = n - 1; i > 0; --i) {
        uint64_t j = splitmix64(s) % static_cast<uint64_t>(i + 1);
        std::swap(v[i], v[j]);
    }
    return v;
}

void TokenLoader::open_file(const std::string& path) {
    TokenFile f;
    f.path = path;
    f.fd = ::open(path.c_str(), O_RDONLY);
    if (f.fd < 0) throw std::runtime_error("cannot open token file " + path);
    struct stat st;
    if (fstat(f.fd, &st) != 0 || st.st_size < kHeaderBytes) { ::close(f.fd); throw std::runtime_error(path + ": not a token shard (too small)"); }
    f.bytes = static_cast<size_t>(st.st_size);
    void* m = mmap(nullptr, f.bytes, PROT_READ, MAP_SHARED, f.fd, 0);
    if (m == MAP_FAILED) { ::close(f.fd); throw std::runtime_error("mmap failed for " + path); }
    f.base = static_cast<const uint8_t*>(m);
    if (std::memcmp(f.base, kMagic, 8) != 0) { munmap(m, f.bytes); ::close(f.fd); throw std::runtime_error(path + ": not a token shard (bad magic)"); }
    const int32_t* h = reinterpret_cast<const int32_t*>(f.base);
    f.version = h[2];
    if (f.version < 1 || f.version > 3 || h[3] != 4) { munmap(m, f.bytes); ::close(f.fd); throw std::runtime_error(path + ": unsupported token shard version"); }
    f.n_tokens = static_cast<uint32_t>(h[4]);
    f.vocab = h[5];
    f.has_masks = h[6] != 0;
    f.non_overlapping = h[7] != 0;
    size_t need = kHeaderBytes + 4ull * f.n_tokens + (f.version >= 3 ? 4ull * f.n_tokens : 0) + (f.has_masks ? (f.n_tokens + 7) / 8 : 0);
    if (f.bytes < need) { munmap(m, f.bytes); ::close(f.fd); throw std::runtime_error(path + ": truncated token shard"); }
    f.tokens = reinterpret_cast<const int32_t*>(f.base + kHeaderBytes);
    size_t off = kHeaderBytes + 4ull * f.n_tokens;
    if (f.version >= 3) { f.positions = reinterpret_cast<const int32_t*>(f.base + off); off += 4ull * f.n_tokens; }
    if (f.has_masks) f.mask_bits = f.base + off;
    madvise(m, f.bytes, MADV_RANDOM);
    files_.push_back(f);
}

TokenLoader::TokenLoader(const std::vector<std::string>& files, int batch, int seq_len, int64_t seed, int rank, int world, bool shuffle, int depth)
    : B_(batch), T_(seq_len), rank_(rank), world_(world), depth_(depth < 1 ? 1 : depth), shuffle_(shuffle) {
    if (files.empty()) throw std::runtime_error("TokenLoader needs at least one token file");
    for (auto& p : files) open_file(p);
    cursor_.seed = consumed_.seed = seed;
    int64_t per_rank = 0;
    for (auto& f : files_) per_rank += chunks_in(f) / world_;
    if (per_rank < B_) throw std::runtime_error("token files hold fewer rows than one batch per rank");
    start();
}

TokenLoader::~TokenLoader() {
    stop();
    for (auto& f : files_) {
        if (f.base) munmap(const_cast<uint8_t*>(f.base), f.bytes);
        if (f.fd >= 0) ::close(f.fd);
    }
}

int64_t TokenLoader::chunks_in(const TokenFile& f) const { return f.non_overlapping ? f.n_tokens / T_ : (f.n_tokens > 0 ? (f.n_tokens - 1) / T_ : 0); }

int64_t TokenLoader::total_chunks() const {
    int64_t n = 0;
    for (auto& f : files_) n += chunks_in(f);
    return n;
}

int64_t TokenLoader::steps_per_epoch() const {
    int64_t n = 0;
    for (auto& f : files_) n += chunks_in(f) / world_;
    return n / B_;
}

void TokenLoader::fill_row(const TokenFile& f, int64_t chunk, int32_t* x, int32_t* y, int32_t* p) const {
    const int64_t s = chunk * T_;
    std::memcpy(x, f.tokens + s, sizeof(int32_t) * T_);
    if (f.positions) std::memcpy(p, f.positions + s, sizeof(int32_t) * T_);
    else for (int t = 0; t < T_; ++t) p[t] = t;
    auto mask_at = [&](int64_t i) -> bool { return (f.mask_bits[i >> 3] >> (i & 7)) & 1; };
    if (f.non_overlapping) {
        for (int t = 0; t + 1 < T_; ++t) {
            int32_t v = f.tokens[s + t + 1];
            if (f.positions && p[t + 1] == 0) v = kIgnore;  // first token of the next packed document is not a target
            if (f.has_masks && !mask_at(s + t + 1)) v = kIgnore;
            y[t] = v;
        }
        y[T_ - 1] = kIgnore;
    } else {
        for (int t = 0; t < T_; ++t) {
            int32_t v = f.tokens[s + t + 1];
            if (f.has_masks && !mask_at(s + t + 1)) v = kIgnore;
            y[t] = v;
        }
    }
}

void TokenLoader::assemble(Batch& b) {
    const size_t n = static_cast<size_t>(B_) * T_;
    b.x.resize(n);
    b.y.resize(n);
    b.p.resize(n);
    const int64_t nf = static_cast<int64_t>(files_.size());
    int row = 0, guard = 0;
    while (row < B_) {
        if (order_epoch_ != cursor_.epoch) {
            file_order_ = shuffled_order(nf, cursor_.seed, cursor_.epoch, 0, shuffle_);
            order_epoch_ = cursor_.epoch;
            order_file_ = -1;
        }
        const int64_t fid = file_order_[cursor_.file_index];
        const TokenFile& f = files_[fid];
        if (order_file_ != cursor_.file_index) {
            std::vector<int64_t> full = shuffled_order(chunks_in(f), cursor_.seed, cursor_.epoch, 1 + fid, shuffle_);
            chunk_order_.clear();
            for (size_t k = rank_; k < full.size(); k += world_) chunk_order_.push_back(full[k]);
            order_file_ = cursor_.file_index;
        }
        if (cursor_.chunk_index >= static_cast<int64_t>(chunk_order_.size())) {
            cursor_.file_index += 1;
            cursor_.chunk_index = 0;
            order_file_ = -1;
            if (cursor_.file_index >= nf) { cursor_.file_index = 0; cursor_.epoch += 1; }
            if (++guard > 2 * nf + 2) throw std::runtime_error("token files hold fewer rows than one batch per rank");
            continue;
        }
        const int64_t c = chunk_order_[cursor_.chunk_index++];
        fill_row(f, c, b.x.data() + static_cast<size_t>(row) * T_, b.y.data() + static_cast<size_t>(row) * T_, b.p.data() + static_cast<size_t>(row) * T_);
        ++row;
    }
    b.after = cursor_;
}

void TokenLoader::run() {
    while (true) {
        {
            std::unique_lock<std::mutex> lk(mu_);
            cv_.wait(lk, [&] { return stop_ || static_cast<int>(queue_.size()) < depth_; });
            if (stop_) return;
        }
        Batch b;
        try {
            assemble(b);
        } catch (const std::exception& e) {
            std::lock_guard<std::mutex> lk(mu_);
            error_ = e.what();
            cv_.notify_all();
            return;
        }
        {
            std::lock_guard<std::mutex> lk(mu_);
            queue_.push_back(std::move(b));
        }
        cv_.notify_all();
    }
}

void TokenLoader::start() {
    stop_ = false;
    worker_ = std::thread([this] { run(); });
}

void TokenLoader::stop() {
    {
        std::lock_guard<std::mutex> lk(mu_);
        stop_ = true;
    }
    cv_.notify_all();
    if (worker_.joinable()) worker_.join();
}

void TokenLoader::next(int32_t* x, int32_t* y, int32_t* p) {
    Batch b;
    {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return !queue_.empty() || !error_.empty(); });
        if (queue_.empty()) throw std::runtime_error(error_);
        b = std::move(queue_.front());
        queue_.pop_front();
    }
    cv_.notify_all();
    const size_t bytes = sizeof(int32_t) * static_cast<size_t>(B_) * T_;
    std::memcpy(x, b.x.data(), bytes);
    std::memcpy(y, b.y.data(), bytes);
    std::memcpy(p, b.p.data(), bytes);
    consumed_ = b.after;
}

void TokenLoader::set_state(const LoaderState& s) {
    stop();
    queue_.clear();
    error_.clear();
    cursor_ = consumed_ = s;
    order_epoch_ = order_file_ = -1;
    start();
}

}  // namespace sg
