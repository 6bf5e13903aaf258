#include "safetensors_io.h"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <stdexcept>
#include <thread>

#include "json_min.h"

namespace sg {

int dtype_size(const std::string& d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0") return 1;
    return 0;
}

namespace {
void pread_all(int fd, char* dst, uint64_t n, uint64_t off) {
    while (n > 0) {
        ssize_t r = ::pread(fd, dst, std::min<uint64_t>(n, 1ull << 30), static_cast<off_t>(off));
        if (r < 0) { if (errno == EINTR) continue; throw std::runtime_error(std::string("pread failed: ") + strerror(errno)); }
        if (r == 0) throw std::runtime_error("pread: unexpected end of file");
        dst += r; off += r; n -= r;
    }
}
void pwrite_all(int fd, const char* src, uint64_t n, uint64_t off) {
    while (n > 0) {
        ssize_t r = ::pwrite(fd, src, std::min<uint64_t>(n, 1ull << 30), static_cast<off_t>(off));
        if (r < 0) { if (errno == EINTR) continue; throw std::runtime_error(std::string("pwrite failed: ") + strerror(errno)); }
        src += r; off += r; n -= r;
    }
}
template <class F>
void parallel_chunks(uint64_t nbytes, int threads, F&& fn) {
    constexpr uint64_t kMinChunk = 8ull << 20;
    int nt = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>(threads < 1 ? 1 : threads, nbytes / kMinChunk)));
    if (nt == 1) { fn(0, nbytes); return; }
    uint64_t per = (nbytes / nt + 4095) & ~4095ull;
    std::vector<std::thread> pool;
    std::vector<std::string> errs(nt);
    for (int t = 0; t < nt; ++t) {
        uint64_t a = std::min<uint64_t>(nbytes, per * t), b = std::min<uint64_t>(nbytes, per * (t + 1));
        if (a >= b) continue;
        pool.emplace_back([&, a, b, t] {
            try { fn(a, b - a); } catch (const std::exception& e) { errs[t] = e.what(); }
        });
    }
    for (auto& th : pool) th.join();
    for (auto& e : errs)
        if (!e.empty()) throw std::runtime_error(e);
}
}  // namespace

SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open " + path);
    struct stat st;
    fstat(fd_, &st);
    file_size_ = static_cast<uint64_t>(st.st_size);
    uint64_t hlen = 0;
    if (file_size_ < 8) throw std::runtime_error(path + ": not a safetensors file");
    pread_all(fd_, reinterpret_cast<char*>(&hlen), 8, 0);
    if (hlen > file_size_ - 8 || hlen > (1ull << 31)) throw std::runtime_error(path + ": bad safetensors header length");
    std::string header(hlen, '\0');
    pread_all(fd_, header.data(), hlen, 8);
    data_start_ = 8 + hlen;
    Json root = parse_json(header);
    for (auto& kv : root.obj) {
        if (kv.first == "__metadata__") {
            for (auto& m : kv.second.obj)
                if (m.second.kind == Json::Str) metadata_[m.first] = m.second.str;
            continue;
        }
        StEntry e;
        e.name = kv.first;
        e.dtype = kv.second.at("dtype").as_str();
        for (auto& d : kv.second.at("shape").arr) e.shape.push_back(d.as_int());
        const Json& off = kv.second.at("data_offsets");
        e.begin = static_cast<uint64_t>(off.arr.at(0).as_int());
        e.end = static_cast<uint64_t>(off.arr.at(1).as_int());
        if (e.end < e.begin || data_start_ + e.end > file_size_) throw std::runtime_error(path + ": tensor '" + e.name + "' lies outside the file");
        index_[e.name] = entries_.size();
        entries_.push_back(std::move(e));
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (fd_ >= 0) ::close(fd_);
}

const StEntry* SafetensorsFile::find(const std::string& name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &entries_[it->second];
}

void SafetensorsFile::read_into(const std::string& name, void* dst, uint64_t nbytes, uint64_t offset, int threads) const {
    const StEntry* e = find(name);
    if (!e) throw std::runtime_error(path_ + ": no tensor '" + name + "'");
    if (offset + nbytes > e->end - e->begin) throw std::runtime_error("read beyond the end of tensor '" + name + "'");
    const uint64_t base = data_start_ + e->begin + offset;
    char* out = static_cast<char*>(dst);
    parallel_chunks(nbytes, threads, [&](uint64_t a, uint64_t n) { pread_all(fd_, out + a, n, base + a); });
}

void SafetensorsFile::read_rows(const std::string& name, void* dst, int64_t r0, int64_t r1, int threads) const {
    const StEntry* e = find(name);
    if (!e) throw std::runtime_error(path_ + ": no tensor '" + name + "'");
    if (e->shape.empty() || r0 < 0 || r1 > e->shape[0] || r0 > r1) throw std::runtime_error("bad row range for tensor '" + name + "'");
    uint64_t row_bytes = dtype_size(e->dtype);
    for (size_t d = 1; d < e->shape.size(); ++d) row_bytes *= static_cast<uint64_t>(e->shape[d]);
    read_into(name, dst, row_bytes * static_cast<uint64_t>(r1 - r0), row_bytes * static_cast<uint64_t>(r0), threads);
}

uint64_t write_safetensors(const std::string& path, const std::vector<StWriteItem>& items, const std::map<std::string, std::string>& metadata,
                           int threads) {
    std::string header = "{";
    if (!metadata.empty()) {
        header += "\"__metadata__\":{";
        bool first = true;
        for (auto& kv : metadata) {
            if (!first) header += ",";
            first = false;
            json_escape(header, kv.first);
            header += ":";
            json_escape(header, kv.second);
        }
        header += "},";
    }
    uint64_t off = 0;
    for (size_t i = 0; i < items.size(); ++i) {
        const auto& it = items[i];
        if (i) header += ",";
        json_escape(header, it.name);
        header += ":{\"dtype\":\"" + it.dtype + "\",\"shape\":[";
        for (size_t d = 0; d < it.shape.size(); ++d) header += (d ? "," : "") + std::to_string(it.shape[d]);
        header += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + it.nbytes) + "]}";
        off += it.nbytes;
    }
    header += "}";
    while ((8 + header.size()) % 8 != 0) header.push_back(' ');
    const std::string tmp = path + ".tmp";
    int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) throw std::runtime_error("cannot create " + tmp);
    try {
        uint64_t hlen = header.size();
        pwrite_all(fd, reinterpret_cast<const char*>(&hlen), 8, 0);
        pwrite_all(fd, header.data(), hlen, 8);
        uint64_t base = 8 + hlen;
        for (const auto& it : items) {
            const char* src = static_cast<const char*>(it.data);
            parallel_chunks(it.nbytes, threads, [&](uint64_t a, uint64_t n) { pwrite_all(fd, src + a, n, base + a); });
            base += it.nbytes;
        }
        ::close(fd);
        if (::rename(tmp.c_str(), path.c_str()) != 0) throw std::runtime_error("rename failed for " + path);
        return base;
    } catch (...) {
        ::close(fd);
        ::unlink(tmp.c_str());
        throw;
    }
}

}  // namespace sg
