#include "bpe_tokenizer.h"

#include <algorithm>
#include <atomic>
#include <climits>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <thread>

#include "json_min.h"
#include "unicode_tables.h"  // generated at build time: kLetterRanges / kNumberRanges (sorted, inclusive codepoint ranges)

namespace sg {

namespace {

bool in_ranges(const uint32_t (*ranges)[2], int n, uint32_t cp) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        int mid = (lo + hi) >> 1;
        if (cp < ranges[mid][0]) hi = mid - 1;
        else if (cp > ranges[mid][1]) lo = mid + 1;
        else return true;
    }
    return false;
}

// UTF-8 -> codepoints with the byte offset of each; malformed bytes become single codepoints 0xFFFD-like pieces that
// still map back to the original bytes because offsets, not re-encoding, delimit the output pieces.
void decode_utf8(const std::string& s, std::vector<uint32_t>& cps, std::vector<uint32_t>& offs) {
    size_t i = 0, n = s.size();
    cps.reserve(n);
    offs.reserve(n + 1);
    while (i < n) {
        unsigned char c = static_cast<unsigned char>(s[i]);
        uint32_t cp = c;
        int len = 1;
        if (c >= 0xF0 && c < 0xF8 && i + 3 < n) { cp = c & 0x07; len = 4; }
        else if (c >= 0xE0 && c < 0xF0 && i + 2 < n) { cp = c & 0x0F; len = 3; }
        else if (c >= 0xC0 && c < 0xE0 && i + 1 < n) { cp = c & 0x1F; len = 2; }
        bool ok = true;
        for (int k = 1; k < len; ++k) {
            unsigned char cc = static_cast<unsigned char>(s[i + k]);
            if ((cc & 0xC0) != 0x80) { ok = false; break; }
            cp = (cp << 6) | (cc & 0x3F);
        }
        if (!ok || (len == 1 && c >= 0x80)) { cp = 0xFFFD; len = 1; }
        cps.push_back(cp);
        offs.push_back(static_cast<uint32_t>(i));
        i += len;
    }
    offs.push_back(static_cast<uint32_t>(n));
}

// GPT-2 byte <-> printable-codepoint table used by byte-level vocabularies.
struct ByteMap {
    uint32_t byte_to_cp[256];
    std::unordered_map<uint32_t, uint8_t> cp_to_byte;
    ByteMap() {
        int extra = 0;
        for (int b = 0; b < 256; ++b) {
            bool printable = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
            byte_to_cp[b] = printable ? static_cast<uint32_t>(b) : 256u + extra++;
            cp_to_byte[byte_to_cp[b]] = static_cast<uint8_t>(b);
        }
    }
};
const ByteMap& byte_map() {
    static ByteMap m;
    return m;
}

// Vocabulary strings are written with the printable stand-ins; turn one back into raw bytes.
std::string vocab_string_to_bytes(const std::string& tok) {
    std::vector<uint32_t> cps, offs;
    decode_utf8(tok, cps, offs);
    std::string out;
    out.reserve(cps.size());
    const auto& m = byte_map().cp_to_byte;
    for (size_t i = 0; i < cps.size(); ++i) {
        auto it = m.find(cps[i]);
        if (it != m.end()) out.push_back(static_cast<char>(it->second));
        else out.append(tok, offs[i], offs[i + 1] - offs[i]);  // not a byte-level symbol: keep its UTF-8 bytes
    }
    return out;
}

inline uint32_t lower_ascii(uint32_t c) { return (c >= 'A' && c <= 'Z') ? c + 32 : c; }

// Length in codepoints of a contraction ('s 't 're 've 'm 'll 'd) starting at i, or 0.
int contraction_len(const std::vector<uint32_t>& c, size_t i, bool icase) {
    if (c[i] != '\'' || i + 1 >= c.size()) return 0;
    auto at = [&](size_t k) -> uint32_t { return k < c.size() ? (icase ? lower_ascii(c[k]) : c[k]) : 0; };
    uint32_t a = at(i + 1), b = at(i + 2);
    if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
    if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
    return 0;
}

}  // namespace

bool unicode_is_letter(uint32_t cp) { return in_ranges(kLetterRanges, kNumLetterRanges, cp); }
bool unicode_is_number(uint32_t cp) { return in_ranges(kNumberRanges, kNumNumberRanges, cp); }
bool unicode_is_space(uint32_t cp) {
    return (cp >= 9 && cp <= 13) || cp == 32 || cp == 0x85 || cp == 0xA0 || cp == 0x1680 || (cp >= 0x2000 && cp <= 0x200A) || cp == 0x2028 ||
           cp == 0x2029 || cp == 0x202F || cp == 0x205F || cp == 0x3000;
}

std::vector<std::string> BpeTokenizer::pre_tokenize(const std::string& text) const {
    std::vector<uint32_t> c, off;
    decode_utf8(text, c, off);
    std::vector<std::string> out;
    const size_t n = c.size();
    auto L = [&](size_t k) { return k < n && unicode_is_letter(c[k]); };
    auto N = [&](size_t k) { return k < n && unicode_is_number(c[k]); };
    auto S = [&](size_t k) { return k < n && unicode_is_space(c[k]); };
    auto other = [&](size_t k) { return k < n && !unicode_is_space(c[k]) && !unicode_is_letter(c[k]) && !unicode_is_number(c[k]); };
    auto emit = [&](size_t a, size_t b) { out.emplace_back(text, off[a], off[b] - off[a]); };
    size_t i = 0;
    while (i < n) {
        size_t j = i;
        if (int cl = contraction_len(c, i, style_.contractions_ignore_case)) {
            emit(i, i + cl);
            i += cl;
            continue;
        }
        if (!style_.legacy_gpt2) {
            // [^\r\n\p{L}\p{N}]?\p{L}+
            size_t s = i;
            if (!L(s) && c[s] != '\r' && c[s] != '\n' && !N(s) && L(s + 1)) ++s;
            if (L(s)) {
                j = s;
                while (L(j)) ++j;
                emit(i, j);
                i = j;
                continue;
            }
            // \p{N}{1,k}
            if (N(i)) {
                j = i;
                while (N(j) && (style_.max_digits == 0 || j - i < static_cast<size_t>(style_.max_digits))) ++j;
                emit(i, j);
                i = j;
                continue;
            }
            //  ?[^\s\p{L}\p{N}]+[\r\n]*
            s = i + (c[i] == ' ' ? 1 : 0);
            if (other(s)) {
                j = s;
                while (other(j)) ++j;
                while (j < n && (c[j] == '\r' || c[j] == '\n')) ++j;
                emit(i, j);
                i = j;
                continue;
            }
        } else {
            size_t s = i + (c[i] == ' ' ? 1 : 0);
            if (L(s)) { j = s; while (L(j)) ++j; emit(i, j); i = j; continue; }
            if (N(s)) { j = s; while (N(j)) ++j; emit(i, j); i = j; continue; }
            if (other(s)) { j = s; while (other(j)) ++j; emit(i, j); i = j; continue; }
        }
        if (S(i)) {
            j = i;
            while (S(j)) ++j;  // whitespace run [i, j)
            if (!style_.legacy_gpt2) {
                // \s*[\r\n]+ : up to and including the last newline of the run
                size_t last_nl = SIZE_MAX;
                for (size_t k = i; k < j; ++k)
                    if (c[k] == '\r' || c[k] == '\n') last_nl = k;
                if (last_nl != SIZE_MAX) { emit(i, last_nl + 1); i = last_nl + 1; continue; }
            }
            // \s+(?!\S) : leave the last whitespace for the next piece unless the run ends the text; else \s+
            if (j < n && j - i > 1) { emit(i, j - 1); i = j - 1; continue; }
            emit(i, j);
            i = j;
            continue;
        }
        emit(i, i + 1);  // anything the alternatives above do not cover
        ++i;
    }
    return out;
}

void BpeTokenizer::encode_word(const std::string& word, std::vector<int32_t>& out) const {
    if (word.empty()) return;
    {
        std::lock_guard<std::mutex> g(cache_mu_);
        auto it = cache_.find(word);
        if (it != cache_.end()) { out.insert(out.end(), it->second.begin(), it->second.end()); return; }
    }
    std::vector<int32_t> ids;
    if (ignore_merges_) {
        auto it = bytes_to_id_.find(word);
        if (it != bytes_to_id_.end()) ids.push_back(it->second);
    }
    if (ids.empty()) {
        ids.reserve(word.size());
        for (unsigned char b : word) ids.push_back(byte_id_[b]);
        while (ids.size() > 1) {
            int best_rank = INT_MAX, best_pos = -1, best_id = -1;
            for (size_t k = 0; k + 1 < ids.size(); ++k) {
                auto it = merges_.find((static_cast<uint64_t>(static_cast<uint32_t>(ids[k])) << 32) | static_cast<uint32_t>(ids[k + 1]));
                if (it != merges_.end() && it->second.first < best_rank) { best_rank = it->second.first; best_pos = static_cast<int>(k); best_id = it->second.second; }
            }
            if (best_pos < 0) break;
            ids[best_pos] = best_id;
            ids.erase(ids.begin() + best_pos + 1);
        }
    }
    out.insert(out.end(), ids.begin(), ids.end());
    if (word.size() <= 64) {
        std::lock_guard<std::mutex> g(cache_mu_);
        if (cache_.size() < (1u << 20)) cache_.emplace(word, std::move(ids));
    }
}

void BpeTokenizer::encode_plain(const std::string& text, std::vector<int32_t>& out) const {
    for (const auto& w : pre_tokenize(text)) encode_word(w, out);
}

std::vector<int32_t> BpeTokenizer::encode(const std::string& text, bool allow_added_tokens) const {
    std::vector<int32_t> out;
    if (!allow_added_tokens || added_.empty()) { encode_plain(text, out); return out; }
    size_t pos = 0, seg = 0;
    while (pos < text.size()) {
        int hit = -1;
        for (size_t a = 0; a < added_.size(); ++a) {  // added_ is sorted longest first
            const std::string& t = added_[a].first;
            if (text[pos] == t[0] && text.compare(pos, t.size(), t) == 0) { hit = static_cast<int>(a); break; }
        }
        if (hit < 0) { ++pos; continue; }
        if (pos > seg) encode_plain(text.substr(seg, pos - seg), out);
        out.push_back(added_[hit].second);
        pos += added_[hit].first.size();
        seg = pos;
    }
    if (seg < text.size()) encode_plain(text.substr(seg), out);
    return out;
}

std::vector<std::vector<int32_t>> BpeTokenizer::encode_batch(const std::vector<std::string>& texts, bool allow_added, int threads) const {
    std::vector<std::vector<int32_t>> out(texts.size());
    int nt = std::max(1, std::min<int>(threads > 0 ? threads : static_cast<int>(std::thread::hardware_concurrency()), static_cast<int>(texts.size())));
    if (nt == 1) {
        for (size_t i = 0; i < texts.size(); ++i) out[i] = encode(texts[i], allow_added);
        return out;
    }
    std::atomic<size_t> next{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([&] {
            for (size_t i = next.fetch_add(1); i < texts.size(); i = next.fetch_add(1)) out[i] = encode(texts[i], allow_added);
        });
    for (auto& th : pool) th.join();
    return out;
}

std::string BpeTokenizer::decode(const std::vector<int32_t>& ids, bool skip_special) const {
    std::string out;
    for (int32_t id : ids) {
        if (id < 0 || id >= vocab_size()) continue;
        if (skip_special && special_[id]) continue;
        out += id_to_bytes_[id];
    }
    return out;
}

int32_t BpeTokenizer::token_to_id(const std::string& token_bytes) const {
    auto it = bytes_to_id_.find(token_bytes);
    return it == bytes_to_id_.end() ? -1 : it->second;
}

const std::string& BpeTokenizer::id_to_token(int32_t id) const {
    static const std::string empty;
    return (id >= 0 && id < vocab_size()) ? id_to_bytes_[id] : empty;
}

bool BpeTokenizer::is_special(int32_t id) const { return id >= 0 && id < vocab_size() && special_[id]; }

std::shared_ptr<BpeTokenizer> BpeTokenizer::from_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return from_json(ss.str());
}

static void scan_pattern(const Json& node, PreTokenizerStyle& st, bool& found) {
    if (node.kind == Json::Obj) {
        const Json* type = node.find("type");
        if (type && type->kind == Json::Str && type->str == "Split") {
            const Json* pat = node.find("pattern");
            const Json* rx = pat ? pat->find("Regex") : nullptr;
            if (rx && rx->kind == Json::Str) {
                const std::string& r = rx->str;
                found = true;
                st.legacy_gpt2 = r.find("[^\\r\\n\\p{L}\\p{N}]?") == std::string::npos;
                st.contractions_ignore_case = r.find("(?i:") != std::string::npos;
                if (r.find("\\p{N}{1,3}") != std::string::npos) st.max_digits = 3;
                else if (r.find("\\p{N}+") != std::string::npos) st.max_digits = 0;
                else st.max_digits = 1;
            }
        }
        if (type && type->kind == Json::Str && type->str == "ByteLevel" && !found) {
            const Json* ur = node.find("use_regex");
            if (!ur || ur->kind != Json::Bool || ur->b) { st.legacy_gpt2 = true; st.contractions_ignore_case = false; st.max_digits = 0; }
        }
        for (auto& kv : node.obj) scan_pattern(kv.second, st, found);
    } else if (node.kind == Json::Arr) {
        for (auto& v : node.arr) scan_pattern(v, st, found);
    }
}

std::shared_ptr<BpeTokenizer> BpeTokenizer::from_json(const std::string& text) {
    Json root = parse_json(text);
    const Json& model = root.at("model");
    const Json* mtype = model.find("type");
    if (mtype && mtype->kind == Json::Str && mtype->str != "BPE") throw std::runtime_error("tokenizer.json: only BPE models are supported, got " + mtype->str);
    auto tp = std::make_shared<BpeTokenizer>();
    BpeTokenizer& t = *tp;
    bool found = false;
    if (const Json* pre = root.find("pre_tokenizer")) scan_pattern(*pre, t.style_, found);
    if (const Json* im = model.find("ignore_merges")) t.ignore_merges_ = im->kind == Json::Bool && im->b;

    const Json& vocab = model.at("vocab");
    int32_t max_id = -1;
    for (auto& kv : vocab.obj) max_id = std::max<int32_t>(max_id, static_cast<int32_t>(kv.second.as_int()));
    const Json* added = root.find("added_tokens");
    if (added)
        for (auto& a : added->arr) max_id = std::max<int32_t>(max_id, static_cast<int32_t>(a.at("id").as_int()));
    t.id_to_bytes_.assign(max_id + 1, std::string());
    t.special_.assign(max_id + 1, 0);
    t.bytes_to_id_.reserve(vocab.obj.size() * 2);
    for (auto& kv : vocab.obj) {
        int32_t id = static_cast<int32_t>(kv.second.as_int());
        std::string bytes = vocab_string_to_bytes(kv.first);
        t.id_to_bytes_[id] = bytes;
        t.bytes_to_id_.emplace(std::move(bytes), id);
    }
    for (int b = 0; b < 256; ++b) {
        auto it = t.bytes_to_id_.find(std::string(1, static_cast<char>(b)));
        t.byte_id_[b] = it == t.bytes_to_id_.end() ? -1 : it->second;
    }
    for (int b = 0; b < 256; ++b)
        if (t.byte_id_[b] < 0) throw std::runtime_error("tokenizer.json: vocabulary lacks a single-byte token (not a byte-level BPE)");

    const Json& merges = model.at("merges");
    int rank = 0;
    t.merges_.reserve(merges.arr.size() * 2);
    for (auto& m : merges.arr) {
        std::string a, b;
        if (m.kind == Json::Str) {
            size_t sp = m.str.find(' ');
            if (sp == std::string::npos) { ++rank; continue; }
            a = m.str.substr(0, sp);
            b = m.str.substr(sp + 1);
        } else if (m.kind == Json::Arr && m.arr.size() == 2) {
            a = m.arr[0].as_str();
            b = m.arr[1].as_str();
        }
        std::string ab = vocab_string_to_bytes(a), bb = vocab_string_to_bytes(b);
        auto ia = t.bytes_to_id_.find(ab), ib = t.bytes_to_id_.find(bb), iab = t.bytes_to_id_.find(ab + bb);
        if (ia != t.bytes_to_id_.end() && ib != t.bytes_to_id_.end() && iab != t.bytes_to_id_.end()) {
            uint64_t key = (static_cast<uint64_t>(static_cast<uint32_t>(ia->second)) << 32) | static_cast<uint32_t>(ib->second);
            t.merges_.emplace(key, std::make_pair(rank, iab->second));
        }
        ++rank;
    }
    if (added) {
        for (auto& a : added->arr) {
            int32_t id = static_cast<int32_t>(a.at("id").as_int());
            const std::string& content = a.at("content").as_str();
            const Json* sp = a.find("special");
            t.id_to_bytes_[id] = content;
            t.special_[id] = (sp && sp->kind == Json::Bool && sp->b) ? 1 : 0;
            if (!content.empty()) t.added_.emplace_back(content, id);
        }
        std::stable_sort(t.added_.begin(), t.added_.end(), [](const auto& x, const auto& y) { return x.first.size() > y.first.size(); });
    }
    return tp;
}

}  // namespace sg
