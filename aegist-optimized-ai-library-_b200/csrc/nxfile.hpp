// Reader for the .nx brain format (writer: aegist/nx.py:70-143; Rust reader: aegist_rs/src/nx.rs).
//   bytes 0..8 magic "AEGISTNX" | 8..12 u32 LE version | 12..20 u64 LE header length H | H bytes JSON
//   data section from the next 64-byte boundary; every tensor 64-byte aligned.
// A cores file (aegist_rs/src/nx.rs:82-110) is an .nx file whose header names a base file
// ("base": {"path", "sha256"}) and whose tensors, all of group "cores", replace the base's tensors of the same
// names: opening it opens the base, checks that the base's weights are the ones the cores were learned on, and
// lays the cores over them.
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
    bool overlay = false;     // the bytes live in the cores file laid over this base
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
        delete over_;
        over_ = nullptr;
    }
    // open `p`; when it is a cores file, this object becomes its base with the cores laid over it
    bool open(const std::string& p, std::string& err) {
        if (!open_one(p, err)) return false;
        const JValue* base = header.get("base");
        if (!base || base->type != JValue::Obj) return true;
        const JValue* bp = base->get("path");
        if (!bp || bp->type != JValue::Str) { err = p + ": base has no path"; return false; }
        NxFile* top = new NxFile();
        // this object's mapping moves into `top`; then the base is opened in place
        top->path = path; top->header = header; top->tensors = tensors; top->data_start = data_start;
        top->fd_ = fd_; top->map_ = map_; top->size_ = size_;
        fd_ = -1; map_ = nullptr; size_ = 0;
        const std::string base_path = bp->str;
        const JValue top_base = *base;          // `base` points into the header that is about to be replaced
        base = &top_base;
        tensors.clear();
        header = JValue();
        if (!open_one(base_path, err)) { err = p + " is learned cores over " + base_path + ": " + err; delete top; return false; }
        const JValue* nested = header.get("base");
        if (nested && nested->type == JValue::Obj) { err = p + ": its base " + base_path + " is itself a cores file"; delete top; return false; }
        const JValue* have = header.get("sha256");
        const JValue* hb = have ? have->get("base") : nullptr;
        const JValue* want = base->get("sha256");
        if (!hb || !want || hb->type != JValue::Str || want->type != JValue::Str || hb->str != want->str) {
            err = p + " was learned on a different " + base_path + " (its weights changed since)";
            delete top;
            return false;
        }
        for (auto& kv : top->tensors) {
            NxTensor t = kv.second;
            if (t.group != "cores") { err = p + ": a cores file may only hold cores, not " + kv.first; delete top; return false; }
            auto it = tensors.find(kv.first);
            bool fits = it != tensors.end() && it->second.dtype == t.dtype && it->second.shape.size() == t.shape.size();
            for (size_t i = 1; fits && i < t.shape.size(); i++) fits = it->second.shape[i] == t.shape[i];
            if (!fits) { err = p + ": " + kv.first + " does not fit " + base_path; delete top; return false; }
            t.overlay = true;
            tensors[kv.first] = t;
        }
        over_ = top;
        return true;
    }
    // sha256 over the header's hash object in compact JSON with sorted keys (what serde_json prints), then over the
    // cores file's, first 12 bytes in hex (NxFile::fingerprint, aegist_rs/src/nx.rs:114-124); empty without hashes
    std::string fingerprint() const {
        auto dump = [](const JValue* o) {
            std::vector<std::pair<std::string, std::string>> kv;
            for (auto& e : o->obj) kv.emplace_back(e.first, e.second.str);
            std::sort(kv.begin(), kv.end());
            std::string s = "{";
            for (size_t i = 0; i < kv.size(); i++) s += std::string(i ? "," : "") + "\"" + kv[i].first + "\":\"" + kv[i].second + "\"";
            return s + "}";
        };
        const JValue* h = header.get("sha256");
        if (!h || h->type != JValue::Obj) return "";
        Sha256 sh;
        std::string a = dump(h);
        sh.update((const uint8_t*)a.data(), a.size());
        if (over_) {
            const JValue* oh = over_->header.get("sha256");
            if (oh && oh->type == JValue::Obj) { std::string b = dump(oh); sh.update((const uint8_t*)b.data(), b.size()); }
        }
        return sh.hex().substr(0, 24);
    }
    bool open_one(const std::string& p, std::string& err) {
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
    const uint8_t* data(const NxTensor& t) const {
        if (t.overlay && over_) return over_->map_ + over_->data_start + t.offset;
        return map_ + data_start + t.offset;
    }

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
        for (auto& kv : h) {
            // the cores of a cores file are hashed in that file's header, everything else in the base's
            const JValue* want = (over_ && kv.first == "cores") ? over_->header.get("sha256") : header.get("sha256");
            const JValue* w = want ? want->get(kv.first) : nullptr;
            ok[kv.first] = w && w->type == JValue::Str && w->str == kv.second.hex();
        }
        return ok;
    }

private:
    int fd_ = -1;
    const uint8_t* map_ = nullptr;
    size_t size_ = 0;
    NxFile* over_ = nullptr;      // the cores file laid over this base, if any
};

}  // namespace b2
