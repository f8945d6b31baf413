// b2-debug-logits BRAIN in.json out.bin [--context N] [--kv f32|bf16] [--device D]
//
// The reference's parity entry point (`aegist debug-logits`, aegist_rs/src/main.rs:733-803) over this engine's
// C ABI, reading the same in.json and writing the same out.bin:
//   {"prompt": [ids], "steps": [ids]}            -> f32 logits after the prompt and after each step token,
//                                                   [(1 + steps) x vocab]
//   {"ops": [{"feed": [ids]} | {"snapshot": true} | {"crop": n} | {"save": path} | {"load": path}], "taps": [layers]}
//                                                -> one logits row per feed; each crop prints "crop n -> kept" on
//                                                   stderr; with taps, every feed's last-token state after those
//                                                   layers goes to out.bin.taps
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/b200moe.h"
#include "json.hpp"

using namespace b2;

static int die(const std::string& m) {
    fprintf(stderr, "%s\n", m.c_str());
    return 1;
}
static double now() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static std::vector<uint32_t> ids_of(const JValue* v) {
    std::vector<uint32_t> r;
    if (v && v->type == JValue::Arr)
        for (auto& x : v->arr) r.push_back((uint32_t)x.num);
    return r;
}
static bool write_f32(const std::string& path, const std::vector<float>& rows) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(rows.data(), 4, rows.size(), f) == rows.size();
    return fclose(f) == 0 && ok;
}

int main(int argc, char** argv) {
    std::vector<std::string> pos;
    int context = 2048, device = 0, kv = B2_KV_F32;
    for (int i = 1; i < argc; i++) {
        const std::string a = argv[i];
        if (a == "--context" && i + 1 < argc) context = atoi(argv[++i]);
        else if (a == "--device" && i + 1 < argc) device = atoi(argv[++i]);
        else if (a == "--kv" && i + 1 < argc) kv = std::string(argv[++i]) == "bf16" ? B2_KV_BF16 : B2_KV_F32;
        else pos.push_back(a);
    }
    if (pos.size() != 3) return die("usage: b2-debug-logits BRAIN in.json out.bin [--context N] [--kv f32|bf16] [--device D]");
    const std::string brain = pos[0], inp = pos[1], out = pos[2];
    std::ifstream in(inp);
    if (!in) return die(inp + ": cannot read");
    std::stringstream ss;
    ss << in.rdbuf();
    const std::string text = ss.str();
    JValue spec;
    std::string jerr;
    JParser parser(text.data(), text.size());
    if (!parser.parse(spec, jerr)) return die(inp + ": " + jerr);

    b2_engine* e = nullptr;
    if (b2_open(brain.c_str(), context, device, 1, kv, &e)) {
        const std::string m = e ? b2_last_error(e) : "engine could not be created";
        if (e) b2_close(e);
        return die(m);
    }
    const int V = b2_vocab(e), D = b2_d_model(e);
    auto fail = [&]() { const std::string m = b2_last_error(e); b2_close(e); return die(m); };
    std::vector<float> rows, row((size_t)V);

    if (const JValue* ops = spec.get("ops"); ops && ops->type == JValue::Arr) {
        std::vector<int> taps;
        if (const JValue* t = spec.get("taps"); t && t->type == JValue::Arr)
            for (auto& x : t->arr) taps.push_back((int)x.num);
        if (b2_set_taps(e, taps.data(), (int)taps.size())) return fail();
        std::vector<float> tap_rows, tap((size_t)taps.size() * D);
        for (auto& op : ops->arr) {
            const JValue *f = op.get("feed"), *sn = op.get("snapshot"), *cr = op.get("crop"), *sv = op.get("save"), *ld = op.get("load");
            if (f && f->type == JValue::Arr) {
                const std::vector<uint32_t> ids = ids_of(f);
                if (b2_feed(e, ids.data(), (int)ids.size(), row.data())) return fail();
                rows.insert(rows.end(), row.begin(), row.end());
                if (!taps.empty()) {
                    if (b2_taps(e, tap.data())) return fail();
                    tap_rows.insert(tap_rows.end(), tap.begin(), tap.end());
                }
            } else if (sn && sn->type == JValue::Bool && sn->b) {
                if (b2_snapshot(e)) return fail();
            } else if (cr && cr->is_num()) {
                fprintf(stderr, "crop %d -> %d\n", (int)cr->num, b2_crop(e, (int)cr->num));
            } else if (sv && sv->type == JValue::Str) {
                const double t0 = now();
                if (b2_save_state(e, sv->str.c_str())) return fail();
                fprintf(stderr, "save %d tokens: %.2fs\n", b2_length(e), now() - t0);
            } else if (ld && ld->type == JValue::Str) {
                const double t0 = now();
                int n = 0;
                if (b2_load_state(e, ld->str.c_str(), nullptr, 0, &n)) return fail();
                fprintf(stderr, "load %d tokens: %.2fs\n", n, now() - t0);
            } else {
                b2_close(e);
                return die("unknown op");
            }
        }
        if (!taps.empty() && !write_f32(out + ".taps", tap_rows)) { b2_close(e); return die(out + ".taps: cannot write"); }
        if (!write_f32(out, rows)) { b2_close(e); return die(out + ": cannot write"); }
        b2_close(e);
        return 0;
    }

    const std::vector<uint32_t> prompt = ids_of(spec.get("prompt")), steps = ids_of(spec.get("steps"));
    if (prompt.empty()) { b2_close(e); return die("in.json needs a prompt or ops"); }
    double t0 = now();
    if (b2_feed(e, prompt.data(), (int)prompt.size(), row.data())) return fail();
    rows.insert(rows.end(), row.begin(), row.end());
    const double prefill = now() - t0;
    t0 = now();
    for (uint32_t t : steps) {
        if (b2_feed(e, &t, 1, row.data())) return fail();
        rows.insert(rows.end(), row.begin(), row.end());
    }
    const double dt = now() - t0;
    if (!write_f32(out, rows)) { b2_close(e); return die(out + ": cannot write"); }
    uint64_t hits = 0, page_ins = 0;
    b2_expert_counters(e, &hits, &page_ins);
    fprintf(stderr, "%s; prefill %zu tokens in %.3fs; %zu rows; %zu decode steps in %.3fs (%.1f tok/s); experts %llu hits, %llu copied in\n",
            b2_describe(e), prompt.size(), prefill, 1 + steps.size(), steps.size(), dt, steps.size() / (dt > 1e-9 ? dt : 1e-9),
            (unsigned long long)hits, (unsigned long long)page_ins);
    b2_close(e);
    return 0;
}
