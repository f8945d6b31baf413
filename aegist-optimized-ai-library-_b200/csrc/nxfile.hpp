// Reader for the .nx brain format (writer: aegist/nx.py:70-143; Rust reader: aegist_rs/src/nx.rs).
//   bytes 0..8 magic "AEGISTNX" | 8..12 u32 LE version | 12..20 u64 LE header length H | H bytes JSON
//   data section from the next 64-byte boundary; every tensor 64-byte aligned.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "json.hpp"
#include "sha256.hpp"

namespace b2 {

struct NxTensor {
    std::string dtype;
    std::vector<int64_t> shape;
    size_t offset = 0, nbytes = 0;
    std::string group;
};

class NxFile {
public:
    std::string path;
    JValue header;
    std::map<std::string, NxTensor> tensors;
    size_t data_start = 0;

    ~NxFile() { close(); }
    void close() {
        if (map_) munmap((void*)map_, size_);
        if (fd_ >= 0) ::close(fd_);
        map_ = nullptr;
        fd_ = -1;
    }
    bool open(const std::string& p, std::string& err) {
        path = p;
        fd_ = ::open(p.c_str(), O_RDONLY);
        if (fd_ < 0) { err = "cannot open " + p + ": " + strerror(errno); return false; }
        struct stat st;
        if (fstat(fd_, &st) != 0) { err = "cannot stat " + p; return false; }
        size_ = (size_t)st.st_size;
        if (size_ < 20) { err = p + " is not an .nx file"; return false; }
        map_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (map_ == MAP_FAILED) { map_ = nullptr; err = "cannot map " + p; return false; }
        if (memcmp(map_, "AEGISTNX", 8) != 0 && memcmp(map_, "AUGISTNX", 8) != 0) { err = p + " is not an .nx file"; return false; }
        uint32_t version;
        uint64_t hlen;
        memcpy(&version, map_ + 8, 4);
        memcpy(&hlen, map_ + 12, 8);
        if (version > 1) { err = p + " uses .nx format v" + std::to_string(version) + "; this engine reads up to v1"; return false; }
        if (20 + hlen > size_) { err = p + ": header runs past the end of the file"; return false; }
        std::string jerr;
        JParser parser((const char*)map_ + 20, (size_t)hlen);
        if (!parser.parse(header, jerr)) { err = "bad .nx header: " + jerr; return false; }
        data_start = 20 + hlen + (64 - (20 + hlen) % 64) % 64;
        const JValue* ts = header.get("tensors");
        if (!ts || ts->type != JValue::Obj) { err = "header has no tensors"; return false; }
        for (auto& kv : ts->obj) {
            NxTensor t;
            const JValue& m = kv.second;
            if (auto d = m.get("dtype")) t.dtype = d->str;
            if (auto s = m.get("shape")) for (auto& x : s->arr) t.shape.push_back((int64_t)x.num);
            auto off = m.get("offset"), nb = m.get("nbytes");
            if (!off || !nb) { err = kv.first + ": tensor entry without offset/nbytes"; return false; }
            t.offset = (size_t)off->num;
            t.nbytes = (size_t)nb->num;
            if (auto g = m.get("group")) t.group = g->str; else t.group = "base";
            if (data_start + t.offset + t.nbytes > size_) { err = kv.first + " runs past the end of the file (truncated brain?)"; return false; }
            tensors[kv.first] = t;
        }
        return true;
    }
    const uint8_t* data(const NxTensor& t) const { return map_ + data_start + t.offset; }

    // group -> matches the header's sha256; order (group, name) as the writer hashes
    std::map<std::string, bool> verify() const {
        std::vector<std::pair<std::string, std::string>> order;
        for (auto& kv : tensors) order.emplace_back(kv.second.group, kv.first);
        std::sort(order.begin(), order.end());
        std::map<std::string, Sha256> h;
        for (const char* g : {"base", "engine", "cores"}) h[g];
        for (auto& gn : order) {
            auto it = h.find(gn.first);
            if (it == h.end()) continue;
            const NxTensor& t = tensors.at(gn.second);
            it->second.update(data(t), t.nbytes);
        }
        std::map<std::string, bool> ok;
        const JValue* want = header.get("sha256");
        for (auto& kv : h) {
            const JValue* w = want ? want->get(kv.first) : nullptr;
            ok[kv.first] = w && w->type == JValue::Str && w->str == kv.second.hex();
        }
        return ok;
    }

private:
    int fd_ = -1;
    const uint8_t* map_ = nullptr;
    size_t size_ = 0;
};

}  // namespace b2
