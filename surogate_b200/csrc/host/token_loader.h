// Streaming reader of token shard files ("BIN.TOK\n" header, int32 tokens, int32 position ids, packed loss-mask bits).
// A background thread assembles the next batches (mmap gather, shifted targets, mask -> -100) while the GPU trains;
// the order is a two-level seeded shuffle (files, then rows of a file) that depends only on (seed, epoch), so a run
// resumes from (seed, epoch, file_index, chunk_index) and rank r of w takes every w-th row of the shuffled order.
// Reference counterpart: csrc/src/runtime/training/dataloader.h:39, dataloader.cpp:183-217.
#pragma once
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace sg {

struct LoaderState {
    int64_t seed = 0, epoch = 0, file_index = 0, chunk_index = 0;
};

struct TokenFile {
    std::string path;
    int fd = -1;
    const uint8_t* base = nullptr;
    size_t bytes = 0;
    int version = 0;
    int64_t n_tokens = 0;
    int vocab = 0;
    bool has_masks = false, non_overlapping = false;
    const int32_t* tokens = nullptr;
    const int32_t* positions = nullptr;
    const uint8_t* mask_bits = nullptr;
};

// Fisher-Yates with splitmix64, identical to the Python fallback (data/loader.py: shuffled_order).
std::vector<int64_t> shuffled_order(int64_t n, int64_t seed, int64_t epoch, int64_t salt, bool shuffle);

class TokenLoader {
public:
    TokenLoader(const std::vector<std::string>& files, int batch, int seq_len, int64_t seed, int rank, int world, bool shuffle, int prefetch_depth);
    ~TokenLoader();
    TokenLoader(const TokenLoader&) = delete;
    TokenLoader& operator=(const TokenLoader&) = delete;

    // Fills three [batch, seq_len] int32 buffers: inputs, targets (-100 = no loss), position ids.
    void next(int32_t* x, int32_t* y, int32_t* p);
    LoaderState state() const { return consumed_; }
    void set_state(const LoaderState& s);
    int64_t steps_per_epoch() const;
    int64_t total_chunks() const;
    int vocab() const { return files_.empty() ? 0 : files_[0].vocab; }

private:
    struct Batch {
        std::vector<int32_t> x, y, p;
        LoaderState after;
    };
    void open_file(const std::string& path);
    int64_t chunks_in(const TokenFile& f) const;
    void assemble(Batch& b);   // producer-side: advances cursor_
    void fill_row(const TokenFile& f, int64_t chunk, int32_t* x, int32_t* y, int32_t* p) const;
    void start();
    void stop();
    void run();

    std::vector<TokenFile> files_;
    int B_, T_, rank_, world_, depth_;
    bool shuffle_;
    LoaderState cursor_, consumed_;
    std::vector<int64_t> file_order_, chunk_order_;
    int64_t order_epoch_ = -1, order_file_ = -1;

    std::thread worker_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<Batch> queue_;
    bool stop_ = false;
    std::string error_;
};

}  // namespace sg
