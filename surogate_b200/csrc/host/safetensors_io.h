// safetensors reader / writer for the host runtime: header parse, multi-threaded pread into caller memory (a pinned staging
// buffer or a parameter shard), row-range reads for sharded loading, and a writer that lays the file out once and fills
// tensors with parallel pwrite.  Reference counterpart: csrc/src/utilities/safetensors.{h,cpp}.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace sg {

struct StEntry {
    std::string name, dtype;
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;  // byte range inside the data section
};

int dtype_size(const std::string& st_dtype);  // "F32" -> 4, "BF16" -> 2, "F8_E4M3" -> 1, ... ; 0 if unknown

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;

    const std::vector<StEntry>& entries() const { return entries_; }
    const StEntry* find(const std::string& name) const;
    const std::map<std::string, std::string>& metadata() const { return metadata_; }
    uint64_t data_start() const { return data_start_; }  // file offset of the data section (entry ranges are relative to it)
    // Copies bytes [offset, offset + nbytes) of the tensor's data into dst using `threads` concurrent preads.
    void read_into(const std::string& name, void* dst, uint64_t nbytes, uint64_t offset, int threads) const;
    // Rows [row_begin, row_end) of dimension 0.
    void read_rows(const std::string& name, void* dst, int64_t row_begin, int64_t row_end, int threads) const;

private:
    std::string path_;
    int fd_ = -1;
    uint64_t data_start_ = 0, file_size_ = 0;
    std::vector<StEntry> entries_;
    std::map<std::string, size_t> index_;
    std::map<std::string, std::string> metadata_;
};

struct StWriteItem {
    std::string name, dtype;
    std::vector<int64_t> shape;
    const void* data = nullptr;
    uint64_t nbytes = 0;
};

// Writes header + tensors (in the given order, each aligned to 8 bytes through header padding only, as the format requires
// contiguous data).  Returns the file size.
uint64_t write_safetensors(const std::string& path, const std::vector<StWriteItem>& items, const std::map<std::string, std::string>& metadata,
                           int threads);

}  // namespace sg
