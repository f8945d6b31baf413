// Host side of the decode engine and its C ABI (include/b200moe.h).
//
// What the reference does in aegist_rs/src/hybrid.rs is done here with a different plan:
//   * every tensor, the embedding table and all experts included, is resident in HBM (a slot table
//     [layer][expert] -> device address replaces the LRU pool of hybrid.rs:190-390);
//   * a decode step is one CUDA graph of 6 launches per layer with no host synchronisation inside:
//     token ids, positions, router picks and the arg-max stay on the device (the reference crosses
//     the host boundary 82 times per token, hybrid.rs:743-758, 875, 919, 1000);
//   * the KV cache is paged (64-token pages through a page table) and stored as bf16 or fp32.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/b200moe.h"
#include "kernels.cuh"
#include "nxfile.hpp"

namespace b2 {

#define CU(call)                                                                                       \
    do {                                                                                               \
        cudaError_t e_ = (call);                                                                       \
        if (e_ != cudaSuccess) return fail("%s: %s", #call, cudaGetErrorString(e_));                   \
    } while (0)

// From this many sequences (or prompt tokens) on a step runs on the tcgen05 GEMM family; below it on the GEMV family,
// which re-reads the weights once per pair of sequences. Measured on the 4-layer full-width case at context 8192:
// 0.53 ms per step at 4 sequences, 0.92 at 7 on the GEMV family; 0.74 at 8 on the GEMM family.
constexpr int BATCH_GEMM_MIN = 6;

struct Cfg {
    int V = 0, D = 0, L = 0;
    std::vector<int> attn;
    int H = 0, KV = 0, HD = 0, RD = 0;
    double theta = 0;
    int HK = 0, HV = 0, DK = 0, DV = 0, CK = 0;
    int E = 0, TOPK = 0, I = 0, SH = 0, G = 0;
    float eps = 1e-6f;
    int n1 = 0, n2 = 0, rank = 0, cores_active = 0;
    int C() const { return 2 * HK * DK + HV * DV; }
    int VD() const { return HV * DV; }
    int n_attn() const { int n = 0; for (int a : attn) n += a; return n; }
    int n_delta() const { return L - n_attn(); }
    size_t gu_q() const { return (size_t)2 * I * (D / 2); }
    size_t gu_sm() const { return (size_t)2 * I * (D / G) * 2; }
    size_t dn_q() const { return (size_t)D * (I / 2); }
    size_t dn_sm() const { return (size_t)D * (I / G) * 2; }
    size_t off_gu_s() const { return gu_q(); }
    size_t off_gu_m() const { return gu_q() + gu_sm(); }
    size_t off_dn_q() const { return gu_q() + 2 * gu_sm(); }
    size_t off_dn_s() const { return off_dn_q() + dn_q(); }
    size_t off_dn_m() const { return off_dn_s() + dn_sm(); }
    size_t expert_bytes() const { size_t n = off_dn_m() + dn_sm(); return (n + 63) / 64 * 64; }
};

struct DevTensor {
    void* p = nullptr;
    size_t nbytes = 0;
    std::string dtype;
    std::vector<int64_t> shape;
};

struct QWd { const int8_t* w = nullptr; const uint16_t* s = nullptr; int n = 0, k = 0; };

struct LayerW {
    bool attn = false;
    int slot = 0;
    const uint16_t *norm1 = nullptr, *norm2 = nullptr;
    // attention
    QWd q, k, v, o;
    const uint16_t *q_norm = nullptr, *k_norm = nullptr;
    // DeltaNet
    QWd in_qkv, in_z, out;
    const uint16_t *in_a = nullptr, *in_b = nullptr, *conv = nullptr, *a_log = nullptr, *dt_bias = nullptr, *gnorm = nullptr;
    // MoE
    const uint16_t* router = nullptr;
    QWd sh_gate, sh_up, sh_down;
    const uint16_t* sh_gw = nullptr;
    const uint8_t* experts = nullptr;       // [local experts][expert_bytes]
    const uint8_t** eptr = nullptr;         // device [E]
    float* router_bias = nullptr;           // device [E] or null
    // core engine + the layer's live switchable cores (live_bank, aegist_rs/src/hybrid.rs:1122-1150)
    const uint16_t *key1 = nullptr, *key2 = nullptr;      // [n1][D], [n2][D]; null: the brain has no core engine tensors
    int* live = nullptr;                    // device [n1 * n2]: core id -> index into the bank, or -1
    int n_live = 0;
    const uint16_t *cg = nullptr, *cu = nullptr, *cd = nullptr;   // bank: gate, up [n][D][r], down [n][r][D]
};

static size_t dtype_size(const std::string& d) {
    if (d == "bf16" || d == "f16") return 2;
    if (d == "f32") return 4;
    if (d == "i8" || d == "u8") return 1;
    if (d == "i64") return 8;
    return 0;
}

constexpr int g_tc_warps = 16;   // compute warps per block of k_tcgemv
static int down_row_blocks(int D) { return (D + DOWN_ROWS - 1) / DOWN_ROWS; }

}  // namespace b2

using namespace b2;

struct b2_engine {
    Cfg c;
    int device = 0, B = 1, cap = 0, nsm = 148;
    bool kv_f32 = false;
    int ep_rank = 0, ep_world = 1;
    std::string err, desc;
    std::map<std::string, DevTensor> t;
    std::vector<LayerW> layers;
    const uint16_t *embed = nullptr, *norm = nullptr;
    QWd lm_head;
    bool finished = false;
    size_t weight_bytes = 0;
    std::string gpu_name;

    cudaStream_t stream = nullptr;
    cudaGraphExec_t graph = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int launches = 0;

    // state
    float *conv = nullptr, *state = nullptr;
    size_t conv_bytes = 0, state_bytes = 0;
    float* snap_conv[2] = {nullptr, nullptr};
    float* snap_state[2] = {nullptr, nullptr};
    long snap_pos[2] = {-1, -1};
    void *kpool = nullptr, *vpool = nullptr;
    int* page_table = nullptr;
    int pages_per_seq = 0;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    int length = 0;
    // the tokens fed so far (one sequence), for saved states; unknown after steps whose tokens stayed on the device
    std::vector<uint32_t> toks;
    bool toks_known = true;
    std::string fingerprint;      // names the weights (NxFile::fingerprint); empty when built from tensors

    // per-step device scalars and work buffers
    int *d_tok = nullptr, *d_next = nullptr, *d_pos = nullptr, *d_err = nullptr;
    unsigned int* d_counter = nullptr;      // [B] gemv finishers
    unsigned int* d_acounter = nullptr;     // [B][KV] attention merge
    float *x = nullptr, *big = nullptr, *zbuf = nullptr, *kraw = nullptr, *vraw = nullptr, *beta = nullptr, *gdec = nullptr;
    float *obuf = nullptr, *att = nullptr, *rlogits = nullptr, *sh_act = nullptr, *sgate = nullptr, *act = nullptr, *logits = nullptr;
    int* top_idx = nullptr;                  // [L][B][TOPK]
    float* top_w = nullptr;
    float* part_val = nullptr;
    int* part_idx = nullptr;
    float* attn_part = nullptr;
    __half* xh = nullptr;                    // [Tpad][2][4096] fp16 activations for the tensor-core path
    int xh_tpad = 0;
    int8_t* uq_i = nullptr;                  // [passes][3][64][4096] int8 digit planes for the tcgen05 GEMM
    uint16_t* uq_b = nullptr;                // [passes][3][64][4096] bf16 planes
    float* uq_scale = nullptr;               // [passes * 64]
    int uq_passes = 0;
    // grouped expert GEMM: picks sorted by expert, chunk table, fp16 expert activations, group sums
    int *g_list = nullptr, *g_chunk = nullptr;
    __half* acth = nullptr;
    float *xsum_tok = nullptr, *xsum_act = nullptr;
    int8_t* sq = nullptr; float *sq_scale = nullptr, *sq_sum = nullptr;   // planes of the sorted picks (k_umma_q4)
    int cap_small = 0, cap_big = 0;
    const uint8_t** top_ptr = nullptr;       // [B][TOPK] expert blobs of the current layer's picks (k_moe_gu1 -> k_moe_down1)
    int8_t* actq = nullptr;                  // [B * TOPK][4][I] digit planes of act
    float *asc = nullptr, *asum = nullptr;   // [B * TOPK][I / 32] scale and sum of each 32-value group of act
    unsigned long long* d_trace = nullptr;   // step timeline slots, allocated by the first b2_debug_trace_step
    float* ypart = nullptr;                  // [B][TOPK + 1][D]
    unsigned int* d_dcounter = nullptr;      // [B][row blocks of the expert down projection]
    int nsplit = 1, head_grid = 1;
    int attn_tiles = 1;                      // 64-position tiles a slice of the longest context spans
    uint32_t* h_pin = nullptr;               // pinned staging [B]
    std::vector<int> tap_layers;
    float* tap_buf = nullptr;
    uint64_t hits = 0;
    // core engine: switch-on counts per layer and core, the picks of the current layer, its score rows, the live cores' output
    int* d_counts = nullptr;                 // [L][n1 * n2]
    int* csel = nullptr; float* cselw = nullptr;      // [B][cores_active]
    float *cscore = nullptr, *core_y = nullptr;       // [B][n1 + n2], [B][D]
    int live_cores = 0;
    // expert parallelism (ep_world > 1): NCCL is resolved at run time from the library the process
    // already has loaded (torch's), so that one process never holds two NCCL versions
    void* nccl_lib = nullptr;
    ncclComm_t comm = nullptr;
    ncclResult_t (*p_ncclGetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*p_ncclCommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*p_ncclCommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*p_ncclAllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*p_ncclSend)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*p_ncclRecv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*p_ncclGroupStart)() = nullptr;
    ncclResult_t (*p_ncclGroupEnd)() = nullptr;
    const char* (*p_ncclGetErrorString)(ncclResult_t) = nullptr;
    float *rec_local = nullptr, *rec_all = nullptr, *recv_y = nullptr;
    // exchange by peer stores: rec_all | recv_y | flags are one block that the other ranks map (cudaIpc)
    float* ep_block = nullptr;
    size_t ep_block_floats = 0, ep_flag_off = 0;
    float* ep_peer[EP_MAX_WORLD] = {};
    bool ep_peer_ready = false;
    int* d_ep_seq = nullptr;
    unsigned long long* d_ep_rows = nullptr;
    long ep_steps = 0;
    int load_nccl();
    int ep_exchange_records(cudaStream_t st);
    int ep_exchange_outputs(cudaStream_t st);

    // Prompt chunks (b2_feed of 16 or more tokens): the step's kernels with the chunk's tokens as the columns, on a work
    // buffer set of its own that is allocated when the first such feed arrives.
    struct ChunkBufs {
        int W = 0;                                  // tokens per chunk
        int *tok = nullptr, *vpos = nullptr;        // [W] token ids, positions pos0 + t
        float *x = nullptr, *big = nullptr, *zbuf = nullptr, *kraw = nullptr, *vraw = nullptr, *beta = nullptr, *gdec = nullptr;
        float *obuf = nullptr, *att = nullptr, *rlogits = nullptr, *sh_act = nullptr, *sgate = nullptr, *act = nullptr;
        int* top_idx = nullptr; float* top_w = nullptr;
        float *ypart = nullptr, *attn_part = nullptr;
        unsigned int *dcounter = nullptr, *counter = nullptr;
        __half *xh = nullptr, *acth = nullptr;
        int xh_tpad = 0;
        int8_t* uq_i = nullptr; uint16_t* uq_b = nullptr; float* uq_scale = nullptr; int uq_passes = 0;
        int *g_list = nullptr, *g_chunk = nullptr;
        float *xsum_tok = nullptr, *xsum_act = nullptr;
        int8_t* sq = nullptr; float *sq_scale = nullptr, *sq_sum = nullptr;
        int cap_small = 0, cap_big = 0, nsplit = 1, attn_tiles = 1;
        int* csel = nullptr; float *cselw = nullptr, *cscore = nullptr, *core_y = nullptr;
    } pc;
    cudaGraphExec_t chunk_graph = nullptr;          // a full chunk without the head, captured at its first use
    int ensure_chunk_bufs();
    int feed_chunk(const uint32_t* ids, int T, bool want_head);

    // per-kernel timing (b2_profile_step): one event after every launch of an un-graphed step
    bool profiling = false;
    std::vector<cudaEvent_t> prof_ev;
    std::vector<int> prof_class;
    size_t prof_used = 0;
    void mark(int cls, cudaStream_t st) {
        if (!profiling) return;
        if (prof_used == prof_ev.size()) { cudaEvent_t e; cudaEventCreate(&e); prof_ev.push_back(e); prof_class.push_back(0); }
        prof_class[prof_used] = cls;
        cudaEventRecord(prof_ev[prof_used++], st);
    }
    void class_bytes(double out[8]) const;

    int fail(const char* fmt, ...) {
        char buf[1024];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof(buf), fmt, ap);
        va_end(ap);
        err = buf;
        return 1;
    }
    ~b2_engine();
    int parse_config(const JValue& j);
    int put(const std::string& name, const std::string& dtype, const std::vector<int64_t>& shape, const void* data,
            size_t nbytes, bool on_device);
    int finish();
    int need(const std::string& name, const std::string& dtype, std::vector<int64_t> shape, const void** out);
    int qw(const std::string& prefix, int n, int k, QWd* out);
    int build_graph();
    int enqueue_step(cudaStream_t st, bool count, int chunk_T = 0, bool chunk_head = false);
    int run_steps(int n);
    int check_device_error();
    int reset_state();
    std::string state_key() const;
    struct Piece { char* p; size_t bytes; };
    std::vector<Piece> state_pieces(int n) const;
};

b2_engine::~b2_engine() {
    if (t.empty() && !finished) return;   // nothing was ever allocated (e.g. creation was refused)
    cudaSetDevice(device);
    if (ep_peer_ready) for (int p = 0; p < ep_world; p++) if (p != ep_rank && ep_peer[p]) cudaIpcCloseMemHandle(ep_peer[p]);
    if (graph) cudaGraphExecDestroy(graph);
    if (chunk_graph) cudaGraphExecDestroy(chunk_graph);
    for (auto& kv : t) cudaFree(kv.second.p);
    for (auto& l : layers) { cudaFree((void*)l.eptr); cudaFree(l.router_bias); cudaFree(l.live); }
    void* bufs[] = {conv, state, snap_conv[0], snap_conv[1], snap_state[0], snap_state[1], kpool, vpool, page_table, rope_cos,
                    rope_sin, d_tok, d_next, d_pos, d_err, d_counter, d_acounter, x, big, zbuf, kraw, vraw, beta, gdec, obuf, att,
                    rlogits, sh_act, sgate, act, logits, top_idx, top_w, part_val, part_idx, attn_part, tap_buf, ypart, d_dcounter, rec_local, ep_block, d_ep_seq, d_ep_rows, xh, g_list, g_chunk, acth, xsum_tok, xsum_act, sq, sq_scale, sq_sum, d_trace, (void*)top_ptr, actq, asc, asum, uq_i, uq_b, uq_scale, d_counts, csel, cselw, cscore, core_y};
    for (void* p : bufs) cudaFree(p);
    void* cb[] = {pc.tok, pc.vpos, pc.x, pc.big, pc.zbuf, pc.kraw, pc.vraw, pc.beta, pc.gdec, pc.obuf, pc.att, pc.rlogits, pc.sh_act, pc.sgate,
                  pc.act, pc.top_idx, pc.top_w, pc.ypart, pc.attn_part, pc.dcounter, pc.counter, pc.xh, pc.acth, pc.uq_i, pc.uq_b, pc.uq_scale,
                  pc.g_list, pc.g_chunk, pc.xsum_tok, pc.xsum_act, pc.sq, pc.sq_scale, pc.sq_sum, pc.csel, pc.cselw, pc.cscore, pc.core_y};
    for (void* p : cb) cudaFree(p);
    if (h_pin) cudaFreeHost(h_pin);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    for (cudaEvent_t e : prof_ev) cudaEventDestroy(e);
    if (comm && p_ncclCommDestroy) p_ncclCommDestroy(comm);
    if (stream) cudaStreamDestroy(stream);
}

// HConfig::from_header + check (aegist_rs/src/hybrid.rs:53-120), with this engine's own shape limits.
int b2_engine::parse_config(const JValue& j) {
    auto num = [&](const char* k, double* out) -> bool {
        const JValue* v = j.get(k);
        if (!v || !v->is_num()) { fail("config is missing %s", k); return false; }
        *out = v->num;
        return true;
    };
    double d;
#define GETI(field, key) if (!num(key, &d)) return 1; c.field = (int)d;
    GETI(V, "vocab_size") GETI(D, "d_model") GETI(L, "n_layers") GETI(H, "n_heads") GETI(KV, "n_kv_heads")
    GETI(HD, "head_dim") GETI(RD, "rotary_dim") GETI(HK, "lin_k_heads") GETI(HV, "lin_v_heads") GETI(DK, "lin_k_dim")
    GETI(DV, "lin_v_dim") GETI(CK, "conv_kernel") GETI(E, "n_experts") GETI(TOPK, "experts_active")
    GETI(I, "expert_hidden") GETI(SH, "shared_hidden") GETI(G, "expert_group") GETI(rank, "core_rank")
    GETI(cores_active, "cores_active")
#undef GETI
    if (!num("rope_theta", &c.theta)) return 1;
    if (!num("norm_eps", &d)) return 1;
    c.eps = (float)d;
    const JValue* lt = j.get("layer_types");
    if (!lt || lt->type != JValue::Arr) return fail("config is missing layer_types");
    for (auto& k : lt->arr) c.attn.push_back(k.type == JValue::Str && k.str == "attn");
    const JValue* grid = j.get("core_grid");
    if (!grid || grid->type != JValue::Arr || grid->arr.size() != 2) return fail("config is missing core_grid");
    c.n1 = (int)grid->arr[0].num;
    c.n2 = (int)grid->arr[1].num;
    const JValue* tie = j.get("tie_embeddings");
    if (tie && tie->type == JValue::Bool && tie->b) return fail("this engine build needs an untied output head");
    const JValue* arch = j.get("arch");
    if (arch && arch->type == JValue::Str && arch->str != "hybrid-moe") return fail("arch %s is not hybrid-moe", arch->str.c_str());
    for (const char* k : {"hc_count"}) {
        const JValue* v = j.get(k);
        if (v && v->is_num() && v->num > 1) return fail("this engine does not run brains with hyper-connections (hc_count > 1)");
    }
    const JValue* ef = j.get("expert_format");
    if (ef && ef->type == JValue::Str && ef->str != "q4") return fail("expert_format %s is not q4", ef->str.c_str());

    std::string bad;
    auto add = [&](const std::string& s) { bad += (bad.empty() ? "" : "; ") + s; };
    if ((int)c.attn.size() != c.L) add("layer_types length");
    if (c.V < 1 || c.L < 1) add("empty model");
    if (c.D % 64 != 0 || c.D < 64 || c.D > 2048) add("d_model must be a multiple of 64, at most 2048");
    if (!(c.HD == 64 || c.HD == 128 || c.HD == 256) || c.RD > c.HD || c.RD % 2 != 0 || c.RD < 2) add("head_dim must be 64/128/256 and rotary_dim even <= head_dim");
    if (c.KV < 1 || c.H % std::max(c.KV, 1) != 0 || c.H / std::max(c.KV, 1) > 8) add("n_heads must be a multiple of n_kv_heads with at most 8 query heads per KV head");
    if (!(c.DK == 64 || c.DK == 128) || c.DV % 32 != 0 || c.DV > 256 || c.HK < 1 || c.HV % std::max(c.HK, 1) != 0 || c.CK != 4) add("DeltaNet needs lin_k_dim 64/128, lin_v_dim a multiple of 32, hv % hk == 0, conv kernel 4");
    if (c.H * c.HD > 4096 || c.VD() > 4096 || (c.H * c.HD) % 32 != 0 || c.VD() % 32 != 0) add("mixer width above 4096");
    if (c.C() % 2 != 0) add("odd conv width");
    if (c.E > 256 || c.E < 1 || c.TOPK > 8 || c.TOPK < 1 || c.TOPK > c.E || c.G != 64 || c.I % 64 != 0 || c.I > 512 || c.I < 64) add("experts need n_experts <= 256, top-k <= 8, group 64, hidden a multiple of 64 up to 512");
    if (c.SH % 16 != 0 || c.SH > 512 || c.SH < 16) add("shared_hidden must be a multiple of 16 up to 512");
    if (c.E % ep_world != 0) add("n_experts not divisible by the number of expert-parallel ranks");
    if (c.n1 < 1 || c.n2 < 1 || c.n1 > 128 || c.n2 > 128 || c.cores_active < 1 || c.cores_active > 8 || c.rank < 1 || c.rank > 256)
        add("core engine needs a grid of at most 128 x 128, 1 to 8 active cores, rank up to 256");
    if (!bad.empty()) return fail("this engine build does not support this brain's shape: %s", bad.c_str());
    return 0;
}

int b2_engine::put(const std::string& name, const std::string& dtype, const std::vector<int64_t>& shape, const void* data,
                   size_t nbytes, bool on_device) {
    if (finished) return fail("b2_put_tensor after b2_finish");
    size_t es = dtype_size(dtype);
    if (!es) return fail("%s: unsupported dtype %s", name.c_str(), dtype.c_str());
    size_t n = es;
    for (auto s : shape) n *= (size_t)s;
    if (n != nbytes) return fail("%s: %zu bytes given, shape says %zu", name.c_str(), nbytes, n);
    CU(cudaSetDevice(device));
    DevTensor d;
    d.dtype = dtype;
    d.shape = shape;
    const char* src = (const char*)data;
    // expert-parallel: keep only this rank's rows of the packed experts
    bool is_experts = name.size() > 15 && name.rfind(".moe.experts.q4") == name.size() - 15;
    if (is_experts && ep_world > 1) {
        if (shape.size() != 2 || shape[0] != c.E) return fail("%s: expected [%d, expert_bytes]", name.c_str(), c.E);
        size_t per = (size_t)c.E / ep_world;
        src += per * ep_rank * (size_t)shape[1];
        nbytes = per * (size_t)shape[1];
        d.shape[0] = (int64_t)per;
    }
    d.nbytes = nbytes;
    if (t.count(name)) { cudaFree(t[name].p); weight_bytes -= t[name].nbytes; }
    CU(cudaMalloc(&d.p, std::max<size_t>(nbytes, 16)));
    if (nbytes) CU(cudaMemcpy(d.p, src, nbytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice));
    weight_bytes += nbytes;
    t[name] = d;
    return 0;
}

int b2_engine::need(const std::string& name, const std::string& dtype, std::vector<int64_t> shape, const void** out) {
    auto it = t.find(name);
    if (it == t.end()) return fail("the brain has no tensor %s", name.c_str());
    const DevTensor& d = it->second;
    bool same = d.dtype == dtype && d.shape.size() == shape.size();
    for (size_t i = 0; same && i < shape.size(); i++) same = d.shape[i] == shape[i];
    if (!same) {
        std::string got = d.dtype + " [", want = dtype + " [";
        for (auto s : d.shape) got += std::to_string(s) + ",";
        for (auto s : shape) want += std::to_string(s) + ",";
        return fail("%s is %s], expected %s]", name.c_str(), got.c_str(), want.c_str());
    }
    *out = d.p;
    return 0;
}

int b2_engine::qw(const std::string& prefix, int n, int k, QWd* out) {
    const void *w, *s;
    if (need(prefix + ".qweight", "i8", {n, k}, &w)) return 1;
    if (need(prefix + ".scale", "bf16", {n, 1}, &s)) return 1;
    out->w = (const int8_t*)w;
    out->s = (const uint16_t*)s;
    out->n = n;
    out->k = k;
    return 0;
}

template <typename T>
static cudaError_t dalloc(T** p, size_t n, bool zero = true) {
    cudaError_t e = cudaMalloc((void**)p, std::max<size_t>(n * sizeof(T), 16));
    if (e == cudaSuccess && zero) e = cudaMemset(*p, 0, std::max<size_t>(n * sizeof(T), 16));
    return e;
}

int b2_engine::finish() {
    if (finished) return fail("b2_finish called twice");
    CU(cudaSetDevice(device));
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, device));
    nsm = prop.multiProcessorCount;
    gpu_name = prop.name;
    const void* p;
#define NEED(dst, name, dtype, ...) if (need(name, dtype, {__VA_ARGS__}, &p)) return 1; dst = (decltype(dst))p;
    NEED(embed, "embed.weight", "bf16", c.V, c.D)
    NEED(norm, "norm.weight", "bf16", c.D)
    if (qw("lm_head", c.V, c.D, &lm_head)) return 1;
    int n_attn = 0, n_delta = 0;
    const int per = c.E / ep_world;
    for (int i = 0; i < c.L; i++) {
        LayerW l;
        std::string b = "blocks." + std::to_string(i) + ".";
        l.attn = c.attn[i];
        NEED(l.norm1, b + "norm1.weight", "bf16", c.D)
        NEED(l.norm2, b + "norm2.weight", "bf16", c.D)
        if (l.attn) {
            l.slot = n_attn++;
            NEED(l.q_norm, b + "mixer.q_norm.weight", "bf16", c.HD)
            NEED(l.k_norm, b + "mixer.k_norm.weight", "bf16", c.HD)
            if (qw(b + "mixer.q", 2 * c.H * c.HD, c.D, &l.q) || qw(b + "mixer.k", c.KV * c.HD, c.D, &l.k) ||
                qw(b + "mixer.v", c.KV * c.HD, c.D, &l.v) || qw(b + "mixer.o", c.D, c.H * c.HD, &l.o)) return 1;
        } else {
            l.slot = n_delta++;
            NEED(l.in_a, b + "mixer.in_a.weight", "bf16", c.HV, c.D)
            NEED(l.in_b, b + "mixer.in_b.weight", "bf16", c.HV, c.D)
            NEED(l.conv, b + "mixer.conv", "bf16", c.C(), c.CK)
            NEED(l.a_log, b + "mixer.A_log", "bf16", c.HV)
            NEED(l.dt_bias, b + "mixer.dt_bias", "bf16", c.HV)
            NEED(l.gnorm, b + "mixer.norm.weight", "bf16", c.DV)
            if (qw(b + "mixer.in_qkv", c.C(), c.D, &l.in_qkv) || qw(b + "mixer.in_z", c.VD(), c.D, &l.in_z) ||
                qw(b + "mixer.out", c.D, c.VD(), &l.out)) return 1;
        }
        NEED(l.router, b + "moe.router.weight", "bf16", c.E, c.D)
        NEED(l.sh_gw, b + "moe.shared_gate.weight", "bf16", 1, c.D)
        if (qw(b + "moe.shared.gate", c.SH, c.D, &l.sh_gate) || qw(b + "moe.shared.up", c.SH, c.D, &l.sh_up) ||
            qw(b + "moe.shared.down", c.D, c.SH, &l.sh_down)) return 1;
        NEED(l.experts, b + "moe.experts.q4", "u8", per, (int64_t)c.expert_bytes())
        // the slot table: every expert of this rank is resident at a fixed address
        std::vector<const uint8_t*> tab(c.E, nullptr);
        for (int e = 0; e < per; e++) tab[ep_rank * per + e] = l.experts + (size_t)e * c.expert_bytes();
        CU(cudaMalloc((void**)&l.eptr, c.E * sizeof(void*)));
        CU(cudaMemcpy((void*)l.eptr, tab.data(), c.E * sizeof(void*), cudaMemcpyHostToDevice));
        CU(dalloc(&l.router_bias, c.E));   // zeros: adding them changes no logit; b2_set_router_bias fills them
        if (t.count(b + "engine.key1.weight")) {
            NEED(l.key1, b + "engine.key1.weight", "bf16", c.n1, c.D)
            NEED(l.key2, b + "engine.key2.weight", "bf16", c.n2, c.D)
            // the sparse bank: ids [n] name the cores that are stored; everything else adds nothing
            const int nc = c.n1 * c.n2;
            std::vector<int> map(nc, -1);
            auto it = t.find(b + "cores.ids");
            int n = 0;
            if (it != t.end() && it->second.nbytes) {
                if (it->second.dtype != "i64") return fail("%scores.ids must be i64", b.c_str());
                n = (int)(it->second.nbytes / 8);
                std::vector<int64_t> ids(n);
                CU(cudaMemcpy(ids.data(), it->second.p, (size_t)n * 8, cudaMemcpyDeviceToHost));
                for (int j = 0; j < n; j++) {
                    if (ids[j] < 0 || ids[j] >= nc) return fail("%scores.ids: core id %lld is outside the %d x %d grid", b.c_str(), (long long)ids[j], c.n1, c.n2);
                    map[(size_t)ids[j]] = j;
                }
                NEED(l.cg, b + "cores.gate", "bf16", n, c.D, c.rank)
                NEED(l.cu, b + "cores.up", "bf16", n, c.D, c.rank)
                NEED(l.cd, b + "cores.down", "bf16", n, c.rank, c.D)
            }
            l.n_live = n;
            live_cores += n;
            CU(dalloc(&l.live, nc, false));
            CU(cudaMemcpy(l.live, map.data(), (size_t)nc * 4, cudaMemcpyHostToDevice));
        }
        layers.push_back(l);
    }
#undef NEED
    // context, recurrent state, snapshots (aegist_rs/src/hybrid.rs:606-625)
    if (cap <= 0) cap = 32768;
    pages_per_seq = (cap + KV_PAGE - 1) / KV_PAGE;
    const size_t kv_elems = (size_t)std::max(n_attn, 1) * B * pages_per_seq * c.KV * KV_PAGE * c.HD;
    const size_t kvb = kv_f32 ? 4 : 2;
    cudaError_t e1 = cudaMalloc(&kpool, kv_elems * kvb), e2 = cudaMalloc(&vpool, kv_elems * kvb);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return fail("KV cache for %d tokens x %d sequences: %s", cap, B, cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    CU(cudaMemset(kpool, 0, kv_elems * kvb));
    CU(cudaMemset(vpool, 0, kv_elems * kvb));
    {
        // identity page table: sequence b owns pages [b * pages_per_seq, (b+1) * pages_per_seq) of each layer's pool
        std::vector<int> pt((size_t)B * pages_per_seq);
        for (size_t i = 0; i < pt.size(); i++) pt[i] = (int)i;
        CU(dalloc(&page_table, pt.size(), false));
        CU(cudaMemcpy(page_table, pt.data(), pt.size() * 4, cudaMemcpyHostToDevice));
    }
    conv_bytes = (size_t)std::max(n_delta, 1) * B * c.C() * 3 * 4;
    state_bytes = (size_t)std::max(n_delta, 1) * B * c.HV * c.DK * c.DV * 4;
    CU(dalloc((char**)&conv, conv_bytes));
    CU(dalloc((char**)&state, state_bytes));
    for (int s = 0; s < 2; s++) {
        CU(dalloc((char**)&snap_conv[s], conv_bytes));
        CU(dalloc((char**)&snap_state[s], state_bytes));
    }
    {
        // RoPE tables as the Python reference builds them (aegist/hybrid.py:152-157): fp32 angle =
        // fp32(position) * fp32(1 / fp32(theta^(2j/rd))); the power in double reproduces torch's fp32 pow.
        const int hr = c.RD / 2;
        std::vector<float> cs((size_t)cap * hr), sn((size_t)cap * hr);
        for (int j = 0; j < hr; j++) {
            const float ex = (float)(2 * j) / (float)c.RD;
            const float pw = (float)std::pow((double)(float)c.theta, (double)ex);
            const float inv = 1.0f / pw;
            for (int pos = 0; pos < cap; pos++) {
                const float ang = (float)pos * inv;
                cs[(size_t)pos * hr + j] = (float)std::cos((double)ang);
                sn[(size_t)pos * hr + j] = (float)std::sin((double)ang);
            }
        }
        CU(dalloc(&rope_cos, cs.size(), false));
        CU(dalloc(&rope_sin, sn.size(), false));
        CU(cudaMemcpy(rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice));
        CU(cudaMemcpy(rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice));
    }
    // work buffers
    const int bigw = std::max(2 * c.H * c.HD, c.C());
    CU(dalloc(&d_tok, B)); CU(dalloc(&d_next, B)); CU(dalloc(&d_pos, B)); CU(dalloc(&d_err, 1));
    CU(dalloc(&d_counter, B)); CU(dalloc(&d_acounter, (size_t)B * c.KV));
    CU(dalloc(&x, (size_t)B * c.D)); CU(dalloc(&big, (size_t)B * bigw)); CU(dalloc(&zbuf, (size_t)B * c.VD()));
    CU(dalloc(&kraw, (size_t)B * c.KV * c.HD)); CU(dalloc(&vraw, (size_t)B * c.KV * c.HD));
    CU(dalloc(&beta, (size_t)B * c.HV)); CU(dalloc(&gdec, (size_t)B * c.HV));
    CU(dalloc(&obuf, (size_t)B * c.VD())); CU(dalloc(&att, (size_t)B * c.H * c.HD));
    CU(dalloc(&rlogits, (size_t)B * c.E)); CU(dalloc(&sh_act, (size_t)B * c.SH)); CU(dalloc(&sgate, B));
    const size_t Bg = (size_t)B * ep_world;   // sequences whose picks may land on this GPU's experts
    CU(dalloc(&act, Bg * c.TOPK * c.I)); CU(dalloc(&logits, (size_t)B * c.V));
    CU(dalloc(&top_idx, (size_t)c.L * B * c.TOPK)); CU(dalloc(&top_w, (size_t)c.L * B * c.TOPK));
    CU(dalloc(&top_ptr, (size_t)B * c.TOPK));
    CU(dalloc(&actq, (size_t)B * c.TOPK * M1_PLANES * c.I));
    CU(dalloc(&asc, (size_t)B * c.TOPK * std::max(1, c.I / 32))); CU(dalloc(&asum, (size_t)B * c.TOPK * std::max(1, c.I / 32)));
    head_grid = std::min((c.V + 31) / 32, nsm);
    CU(dalloc(&part_val, (size_t)B * head_grid)); CU(dalloc(&part_idx, (size_t)B * head_grid));
    // attention: enough slices to fill the GPU, but at least 64 positions each at full context. With many sequences the
    // GPU is full anyway; slices of about 8 tiles then keep the blocks short, so that they spread evenly over the SMs
    // (an SM holds one block: 2 x 64 x 2 blocks of 64 tiles each were two uneven waves, 295 us per layer at context 8192)
    nsplit = std::max(1, std::min({64, std::max((2 * nsm) / std::max(1, c.KV * B), (cap + 8 * AM_TILE - 1) / (8 * AM_TILE)), (cap + 63) / 64}));
    if (const char* v = getenv("B2_ATTN_SPLITS")) nsplit = std::max(1, std::min(64, atoi(v)));   // for tests: long slices at short contexts
    attn_tiles = ((cap + nsplit - 1) / nsplit + AM_TILE - 1) / AM_TILE;
    CU(dalloc(&attn_part, (size_t)B * c.KV * nsplit * (c.H / c.KV) * (c.HD + 2)));
    if ((int)Bg >= BATCH_GEMM_MIN) {
        xh_tpad = ((int)Bg + MM_TOK - 1) / MM_TOK * MM_TOK;
        CU(dalloc((uint16_t**)&xh, (size_t)xh_tpad * 2 * 4096));
        uq_passes = ((int)Bg + UM_TOK - 1) / UM_TOK;
        CU(dalloc(&uq_i, (size_t)uq_passes * UM_PI * UM_TOK * 4096));
        CU(dalloc(&uq_b, (size_t)uq_passes * UM_PB * UM_TOK * 4096));
        CU(dalloc(&uq_scale, (size_t)uq_passes * UM_TOK));
        const size_t P = Bg * c.TOPK;
        cap_small = (int)std::min<size_t>(P, c.E / ep_world);
        cap_big = (int)(P / (GQ_SMALL + 1)) + 1;
        CU(dalloc(&g_list, P));
        CU(dalloc(&g_chunk, (size_t)3 * (cap_small + cap_big) + 2));
        CU(dalloc((uint16_t**)&acth, P * 2 * c.I));
        CU(dalloc(&xsum_tok, Bg * (c.D / 64)));
        CU(dalloc(&xsum_act, P * std::max(1, c.I / 64)));
        CU(dalloc(&sq, (size_t)UM_PI * P * std::max(c.D, c.I)));
        CU(dalloc(&sq_scale, P)); CU(dalloc(&sq_sum, P * (size_t)(std::max(c.D, c.I) / 64 + 1)));
    }
    CU(dalloc(&ypart, Bg * (c.TOPK + 1) * c.D));
    CU(dalloc(&d_dcounter, Bg * down_row_blocks(c.D)));
    CU(dalloc(&d_counts, (size_t)c.L * c.n1 * c.n2));
    CU(dalloc(&csel, (size_t)B * c.cores_active)); CU(dalloc(&cselw, (size_t)B * c.cores_active));
    CU(dalloc(&cscore, (size_t)B * (c.n1 + c.n2))); CU(dalloc(&core_y, (size_t)B * c.D));
    if (ep_world > 1) {
        const size_t rw = c.D + 2 * c.TOPK;
        CU(dalloc(&rec_local, (size_t)B * rw));
        const size_t nrec = (Bg * rw + 63) / 64 * 64, ny = Bg * (c.TOPK + 1) * c.D;
        ep_flag_off = nrec + ny;
        ep_block_floats = ep_flag_off + 2 * EP_MAX_WORLD * EP_MAX_BLOCKS;
        CU(dalloc(&ep_block, ep_block_floats));
        CU(cudaMemset(ep_block, 0, ep_block_floats * sizeof(float)));
        rec_all = ep_block; recv_y = ep_block + nrec;
        CU(dalloc(&d_ep_seq, 2)); CU(dalloc(&d_ep_rows, 1));
    }
    CU(cudaMallocHost((void**)&h_pin, (std::max(B, 1) * 2 + 1) * sizeof(uint32_t)));   // ids | arg-max | device error word
    CU(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    CU(cudaEventCreate(&ev0));
    CU(cudaEventCreate(&ev1));
    CU(cudaDeviceSynchronize());
    finished = true;
    char buf[512];
    size_t kv_bytes = 2 * kv_elems * kvb;
    snprintf(buf, sizeof(buf), "%s: %.2f GB of weights in HBM (%d of %d experts resident%s), %d live cores, context %d tokens x %d, KV %s %.2f GB",
             gpu_name.c_str(), weight_bytes / 1e9, c.L * per, c.L * c.E, ep_world > 1 ? " on this rank" : "", live_cores, cap, B,
             kv_f32 ? "fp32" : "bf16", kv_bytes / 1e9);
    desc = buf;
    if (ep_world > 1) return 0;   // the step graph holds NCCL calls: it is built by b2_ep_init
    return build_graph();
}


static int g_launch_count = 0;   // kernels launched so far (a step's count is the difference)

// Step timeline (b2_debug_trace_step): while g_trace_base is set, the launch with index i since g_trace_first
// gets the slot g_trace_base + 16 i in its argument struct (structs with a `trace` member; null otherwise).
static unsigned long long* g_trace_base = nullptr;
static int g_trace_first = 0;
constexpr int TRACE_MAX_LAUNCHES = 4096;
template <typename T>
static auto with_trace(const T& a, int) -> decltype((void)a.trace, T()) {
    T c = a;
    const int i = g_launch_count - 1 - g_trace_first;
    c.trace = (g_trace_base && i >= 0 && i < TRACE_MAX_LAUNCHES) ? g_trace_base + (size_t)16 * i : nullptr;
    return c;
}
template <typename T>
static const T& with_trace(const T& a, long) { return a; }

template <typename... KArgs, typename... Args>
static cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    g_launch_count++;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;   // programmatic dependent launch for every kernel of a step
    return cudaLaunchKernelEx(&cfg, kernel, with_trace(args, 0)...);
}

template <typename F>
static cudaError_t opt_in_smem(F* f, size_t bytes) {
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute((const void*)f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

// k_mma_i8 over `passes` groups of MM_TOK sequences. A grid that gives an SM at most one block (the out projections,
// the MoE-in matrices) is bound by the latency of its K chunks, one after the other: it takes the deeper ring.
static cudaError_t launch_mma_i8(const MmaArgs& m, int passes, int nsm, cudaStream_t st) {
    const dim3 grid(m.total_blocks, passes), block(MM_THREADS);
    const bool deep = m.total_blocks * passes <= nsm && m.K / MM_KC >= MM_STAGES_DEEP;
    const size_t smem = (size_t)(deep ? MM_STAGES_DEEP : MM_STAGES) * MM_STAGE_BYTES;
    cudaError_t e;
    if (deep) { if ((e = opt_in_smem(k_mma_i8<MM_STAGES_DEEP>, smem)) == cudaSuccess) e = launch_k(k_mma_i8<MM_STAGES_DEEP>, grid, block, smem, st, m); }
    else { if ((e = opt_in_smem(k_mma_i8<MM_STAGES>, smem)) == cudaSuccess) e = launch_k(k_mma_i8<MM_STAGES>, grid, block, smem, st, m); }
    return e;
}

// Tensor-core paths for BATCH_GEMM_MIN or more tokens: scratch for the fp16 activations of k_mma_i8, and for the activation planes of
// the tcgen05 GEMM (k_umma: int8 digit planes qi, bf16 planes qb, per-token scales; `passes_max` groups of 64 tokens).
struct BatchCtx { __half* xh; int Tpad; int8_t* qi; uint16_t* qb; float* xscale; int passes_max; };

// cuTensorMapEncodeTiled through the runtime's driver entry point table (no link against libcuda)
static PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        cudaGetLastError();
        return (PFN_cuTensorMapEncodeTiled_v12000)p;
    }();
    return fn;
}
// a [rows][row_bytes] byte matrix as a 2-D tensor of bytes; box = 128 bytes x box_rows, 128-byte swizzle, zeros outside
static bool byte_matrix_map(CUtensorMap* m, const void* p, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    auto enc = tensor_map_encoder();
    if (!enc || !p || ((uintptr_t)p & 15) || row_bytes % 128 != 0 || box_rows > 256) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {UM_BK, box_rows};
    const cuuint32_t es[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(p), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static bool umma_kind(int k) {
    return k == SEG_I8 || k == SEG_I8_CONV || k == SEG_I8_SILU || k == SEG_I8_ACC || k == SEG_I8_GATEUP || k == SEG_I8_ARGMAX ||
           k == SEG_BF || k == SEG_BF_SIGMOID || k == SEG_BF_DECAY;
}
// All segments of a GEMV group for T tokens on the tcgen05 GEMM: planes, then one persistent launch. false = this group
// does not fit it (the caller takes another path); *err carries a launch error.
static long g_umma_launches = 0;      // how many GEMV groups went to k_umma (tests check that the tcgen05 path is the one that runs)
static bool launch_umma(const GemvArgs& a, int T, int nsm, cudaStream_t st, const BatchCtx& bc, cudaError_t* err) {
    *err = cudaSuccess;
    const int passes = (T + UM_TOK - 1) / UM_TOK;
    if (!bc.qi || passes > bc.passes_max || a.K % UM_BK != 0 || a.K > 4096 || a.nseg > GEMV_MAX_SEG || !tensor_map_encoder()) return false;
    UmmaArgs u{};
    bool any_i8 = false, any_bf = false;
    for (int i = 0; i < a.nseg; i++) {
        const Seg& g = a.seg[i];
        if (!umma_kind(g.kind)) return false;
        const bool isbf = g.kind == SEG_BF || g.kind == SEG_BF_SIGMOID || g.kind == SEG_BF_DECAY;
        const bool pair = g.kind == SEG_I8_GATEUP;
        (isbf ? any_bf : any_i8) = true;
        UmmaSeg& d = u.seg[i];
        d.s = g.s; d.s2 = g.s2; d.bias = g.bias; d.out = g.out; d.rows = g.rows; d.out_stride = g.out_stride;
        d.kind = g.kind == SEG_I8_ARGMAX ? (int)SEG_I8 : g.kind;
        d.units = pair ? (g.rows + 63) / 64 : (g.rows + UM_M - 1) / UM_M;
        u.total_units += d.units;
        const uint64_t rb = isbf ? 2ull * a.K : (uint64_t)a.K;
        if (!byte_matrix_map(&u.wmap[i], g.w, g.rows, rb, 64)) return false;
        if (pair && !byte_matrix_map(&u.wmap2[i], g.w2, g.rows, rb, 64)) return false;
    }
    u.nseg = a.nseg;
    // tokens per unit: a block pulls about 110 GB/s out of L2, so few row blocks are split over the tokens too
    int tt = UM_TOK;
    while (tt > 16 && tt / 2 >= T) tt /= 2;      // no wider than the tokens need: narrow tiles move two K chunks per stage
    while (tt > 16 && u.total_units * passes * ((std::min(T, (int)UM_TOK) + tt - 1) / tt) * 2 <= nsm && T > tt / 2) tt /= 2;
    u.tt = tt;
    if (!byte_matrix_map(&u.xmap_i8, bc.qi, (uint64_t)passes * UM_PI * UM_TOK, a.K, tt)) return false;
    if (!byte_matrix_map(&u.xmap_bf, bc.qb, (uint64_t)passes * UM_PB * UM_TOK, 2ull * a.K, tt)) return false;
    PrepQArgs p{};
    p.x = a.x; p.x_stride = a.x_stride; p.norm_w = a.norm_w; p.gn_w = a.gn_w; p.z = a.z; p.DV = a.DV; p.eps = a.eps;
    p.K = a.K; p.T = T; p.qi = any_i8 ? bc.qi : nullptr; p.qb = any_bf ? bc.qb : nullptr; p.xscale = bc.xscale;
    if ((*err = launch_k(k_prep_q, dim3(passes * UM_TOK), dim3(256), 0, st, p)) != cudaSuccess) return true;
    u.K = a.K; u.T = T; u.passes = passes; u.xscale = bc.xscale;
    u.conv_w = a.conv_w; u.conv_state = a.conv_state; u.a_log = a.a_log; u.dt_bias = a.dt_bias; u.err = a.err;
    if ((*err = opt_in_smem(k_umma, UM_SMEM)) != cudaSuccess) return true;
    const int nsub = passes == 1 ? (std::min(T, (int)UM_TOK) + tt - 1) / tt : UM_TOK / tt;      // as the kernel counts them
    const int grid = std::max(1, std::min(u.total_units * passes * nsub, nsm));
    *err = launch_k(k_umma, dim3(grid), dim3(UM_THREADS), UM_SMEM, st, u);
    g_umma_launches++;
    return true;
}
static void seal(GemvArgs& a, int K);

static cudaError_t launch_gemv(const GemvArgs& a0, int B, int nsm, cudaStream_t st, int grid_override = 0,
                               const BatchCtx* bc = nullptr) {
    GemvArgs a = a0;
    if (a.x_stride == 0) a.x_stride = a.K;
    cudaError_t e;
    if (bc && B >= BATCH_GEMM_MIN && launch_umma(a, B, nsm, st, *bc, &e)) {
        // every matrix of the group went to the tcgen05 GEMM; the head's arg-max and the router's top-8 are launches of their own
        if (e != cudaSuccess) return e;
        for (int i = 0; i < a.nseg; i++)
            if (a.seg[i].kind == SEG_I8_ARGMAX && a.finisher == FIN_ARGMAX) {
                e = launch_k(k_argmax_rows, dim3(B), dim3(1024), 0, st, (const float*)a.seg[i].out, a.seg[i].rows, a.seg[i].out_stride, a.next_tok, a.pos);
                if (e != cudaSuccess) return e;
            }
        if (a.finisher == FIN_TOPK)
            e = launch_k(k_router_topk, dim3((B + 7) / 8), dim3(256), 0, st, (const float*)a.seg[0].out, a.seg[0].out_stride, a.E, a.topk,
                         a.top_idx, a.top_w, B, a.core);
        return e;
    }
    if (bc && bc->xh && B >= BATCH_GEMM_MIN && B <= bc->Tpad && a.K % MM_KC == 0) {
        // int8 matrices (except the head with its arg-max) go to the tensor cores; bf16 rows stay on k_rowgemv
        MmaArgs m{};
        GemvArgs rest = a;
        rest.nseg = 0;
        const float* argmax_logits = nullptr;
        int argmax_rows = 0, argmax_stride = 0;
        bool topk_moved = false;
        for (int i = 0; i < a.nseg; i++) {
            const Seg& g = a.seg[i];
            // the head's rows are multiplied like any int8 matrix; its arg-max runs as a kernel of its own over the logits
            const bool i8 = g.kind == SEG_I8 || g.kind == SEG_I8_CONV || g.kind == SEG_I8_SILU || g.kind == SEG_I8_ACC || g.kind == SEG_I8_GATEUP ||
                            (g.kind == SEG_I8_ARGMAX && a.finisher == FIN_ARGMAX) ||
                            // bf16 rows (router, DeltaNet a/b, shared gate) are widened to fp16 in registers; the router's
                            // top-8 then runs as a launch of its own
                            ((g.kind == SEG_BF_SIGMOID || g.kind == SEG_BF_DECAY || g.kind == SEG_BF) && a.K % (MM_KC / 2) == 0);
            if (i8 && m.nseg < 4) {
                if (g.kind == SEG_BF && a.finisher == FIN_TOPK && i == 0) topk_moved = true;
                MmaSeg& d = m.seg[m.nseg++];
                d.w = (const int8_t*)g.w; d.s = g.s; d.w2 = (const int8_t*)g.w2; d.s2 = g.s2; d.out = g.out; d.rows = g.rows; d.bias = g.bias;
                d.kind = g.kind == SEG_I8_ARGMAX ? (int)SEG_I8 : g.kind; d.out_stride = g.out_stride;
                if (g.kind == SEG_I8_ARGMAX) { argmax_logits = g.out; argmax_rows = g.rows; argmax_stride = g.out_stride; }
                const int rpb = g.kind == SEG_I8_GATEUP ? MM_ROWS / 2 : MM_ROWS;
                d.blocks = (g.rows + rpb - 1) / rpb;
                m.total_blocks += d.blocks;
            } else {
                rest.seg[rest.nseg++] = g;
            }
        }
        if (m.nseg > 0) {
            PrepArgs p{};
            p.x = a.x; p.x_stride = a.x_stride; p.norm_w = a.norm_w; p.gn_w = a.gn_w; p.z = a.z; p.DV = a.DV; p.eps = a.eps;
            p.K = a.K; p.T = B; p.out = bc->xh; p.Tpad = (B + MM_TOK - 1) / MM_TOK * MM_TOK;
            e = launch_k(k_prep_x, dim3(p.Tpad), dim3(256), 0, st, p);
            if (e != cudaSuccess) return e;
            m.xh = bc->xh; m.K = a.K; m.T = B; m.conv_w = a.conv_w; m.conv_state = a.conv_state; m.a_log = a.a_log; m.dt_bias = a.dt_bias;
            e = launch_mma_i8(m, p.Tpad / MM_TOK, nsm, st);
            if (e != cudaSuccess) return e;
            if (argmax_logits) {
                e = launch_k(k_argmax_rows, dim3(B), dim3(1024), 0, st, argmax_logits, argmax_rows, argmax_stride, a.next_tok, a.pos);
                if (e != cudaSuccess) return e;
            }
            if (topk_moved) {
                // the picks need every score row: what this kernel did not take (beyond its four matrices) is multiplied first
                if (rest.nseg > 0) {
                    rest.finisher = FIN_NONE;
                    rest.core.score = nullptr;
                    seal(rest, a.K);
                    if ((e = launch_gemv(rest, B, nsm, st, 0, nullptr)) != cudaSuccess) return e;
                }
                return launch_k(k_router_topk, dim3((B + 7) / 8), dim3(256), 0, st, (const float*)a.seg[0].out, a.seg[0].out_stride, a.E, a.topk,
                                a.top_idx, a.top_w, B, a.core);
            }
            if (rest.nseg == 0) return cudaSuccess;
            seal(rest, a.K);
            a = rest;
            grid_override = 0;
        }
    }
    if (tc_shape_ok(a.K, g_tc_warps)) {
        // int8 products on the tensor cores; one block per SM, NB sequences per pass. Rows per tile (r for
        // 2048-byte slots, r / 2 for wide rows and pairs) such that the longest block has the least to stream.
        int best_r = 32;
        long best_cost = -1;
        for (int r = 32; r >= 16; r -= 2) {
            int T = 0;
            for (int i = 0; i < a.nseg; i++) {
                const int tr = rl_tile_rows(a.seg[i].kind, a.K) == 32 ? r : r / 2;
                T += (a.seg[i].rows + tr - 1) / tr;
            }
            const int G = grid_override ? grid_override : std::max(1, std::min(T, nsm));
            const long cost = (long)((T + G - 1) / G) * r;
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_r = r; }
        }
        a.total_jobs = 0;
        for (int i = 0; i < a.nseg; i++) {
            Seg& g = a.seg[i];
            g.tr = rl_tile_rows(g.kind, a.K) == 32 ? best_r : best_r / 2;
            g.jobs = (g.rows + g.tr - 1) / g.tr;
            a.total_jobs += g.jobs;
        }
        const int grid = grid_override ? grid_override : std::max(1, std::min(a.total_jobs, nsm));
        a.jq = a.total_jobs / grid; a.jr = a.total_jobs % grid;
        const int per_block = (a.total_jobs + grid - 1) / grid;
        const int nst = std::max(1, std::min(per_block, TC_MAX_STAGES));   // stages: what the longest block needs
#define TCG(NBv, Wv)                                                                                            \
    {                                                                                                           \
        const size_t smem = tc_smem_bytes(a, NBv, nst, Wv);                                                     \
        e = opt_in_smem(k_tcgemv<NBv, Wv>, smem);                                                               \
        if (e == cudaSuccess)                                                                                   \
            e = launch_k(k_tcgemv<NBv, Wv>, dim3(grid, (B + NBv - 1) / NBv), dim3((Wv + TC_EPI) * 32), smem, st, a, B, nst, tc_stage_bytes(a)); \
    }
        if (B >= 2) TCG(2, 16) else TCG(1, 16)
#undef TCG
        return e;
    }
    {
        // shapes the tensor-core kernel does not take: one block of 1024 threads per SM, NB sequences per pass
        const int grid = grid_override ? grid_override : std::max(1, std::min(a.total_jobs, nsm));
        if (B >= 2) {
            const size_t smem = (size_t)2 * RL_STAGE_BYTES + (size_t)4 * a.K * 4 + (size_t)2 * 4 * RL_WARPS * 32 * 4;
            e = opt_in_smem(k_rowgemv<4, 2>, smem);
            if (e == cudaSuccess) e = launch_k(k_rowgemv<4, 2>, dim3(grid, (B + 3) / 4), RL_THREADS, smem, st, a, B);
        } else {
            const size_t smem = (size_t)3 * RL_STAGE_BYTES + (size_t)a.K * 4 + (size_t)2 * RL_WARPS * 32 * 4;
            e = opt_in_smem(k_rowgemv<1, 3>, smem);
            if (e == cudaSuccess) e = launch_k(k_rowgemv<1, 3>, dim3(grid, 1), RL_THREADS, smem, st, a, B);
        }
        return e;
    }
}

static Seg make_seg(int kind, const void* w, const uint16_t* s, int rows, float* out, int out_stride) {
    Seg g{};
    g.w = w; g.s = s; g.rows = rows; g.kind = kind; g.out = out; g.out_stride = out_stride;
    g.jobs = 0;   // tiles: filled by seal(), which knows K
    return g;
}
static void seal(GemvArgs& a, int K) {
    a.K = K;
    a.total_jobs = 0;
    for (int i = 0; i < a.nseg; i++) {
        Seg& g = a.seg[i];
        g.jobs = (g.rows + rl_tile_rows(g.kind, K) - 1) / rl_tile_rows(g.kind, K);
        a.total_jobs += g.jobs;
    }
}

static void seal(GemvArgs& a, int K);
static Seg make_seg(int kind, const void* w, const uint16_t* s, int rows, float* out, int out_stride);

static void launch_proj(const ProjArgs& a, int B, int nsm, cudaStream_t st, const BatchCtx* bc = nullptr) {
    GemvArgs g{};
    g.seg[0] = make_seg(SEG_I8_ACC, a.w, a.s, a.N, a.x, a.N);
    g.nseg = 1;
    seal(g, a.K);
    g.x = a.in; g.x_stride = a.K; g.norm_w = nullptr; g.eps = a.eps;
    if (a.mode == 0) { g.gn_w = a.gn_w; g.z = a.z; g.DV = a.DV; }
    launch_gemv(g, B, nsm, st, 0, bc);
}

static void launch_delta(const DeltaArgs& a, int DK, int B, cudaStream_t st) {
    dim3 g(a.HV * (a.DV / 32), B);
    if (DK == 64) launch_k(k_delta_step<64>, g, THREADS, 0, st, a);
    else launch_k(k_delta_step<128>, g, THREADS, 0, st, a);
}

static void launch_experts(const ExpertArgs& a, int B, int nsm, cudaStream_t st, b2_engine* prof = nullptr) {
    const int picks = B * a.topk;
    // whole rows per warp: I / 8 warps / blocks; 32 blocks give two rows per warp at I = 512
    const int gx = std::max(1, (a.I + GU_RPW * WARPS - 1) / (GU_RPW * WARPS));   // every warp gets its GU_RPW row pairs
    if (a.D <= 1024) launch_k(k_expert_gu<1>, dim3(gx, picks), THREADS, 0, st, a);
    else launch_k(k_expert_gu<2>, dim3(gx, picks), THREADS, 0, st, a);
    if (prof) prof->mark(5, st);
    launch_k(k_expert_down, dim3(down_row_blocks(a.D), a.topk + 1, B), THREADS, 0, st, a);
    if (prof) prof->mark(6, st);
}

// The experts of one layer for T tokens as a grouped tensor-core GEMM: group the picks, gate/up, down into
// ypart, the shared expert's down projection into ypart's last slot. The caller combines.
struct ExpertMmaCtx {
    int* list; int* chunk; int cap_small, cap_big;
    __half* xh; __half* acth; float* xsum_tok; float* xsum_act;
    // the tcgen05 kernel's operands: planes of the sorted picks, and where this GPU's expert blobs lie
    int8_t* sq; float* sq_scale; float* sq_sum; int slots;
    const uint8_t* experts; size_t expert_bytes; int per, e0;
};
static void chunk_tables(const ExpertMmaCtx& m, ChunkTable& small, ChunkTable& big) {
    int* p = m.chunk;
    small.expert = p; small.start = p + m.cap_small; small.n = p + 2 * m.cap_small; small.cap = m.cap_small;
    p += 3 * m.cap_small;
    big.expert = p; big.start = p + m.cap_big; big.n = p + 2 * m.cap_big; big.cap = m.cap_big;
    p += 3 * m.cap_big;
    small.count = p; big.count = p + 1;
}
static cudaError_t launch_q4(Q4Args q, const ChunkTable& small, const ChunkTable& big, int row_blocks, int nsm, cudaStream_t st) {
    cudaError_t e;
    const size_t sm1 = (size_t)Q4_STAGES * q4_stage_bytes(1), sm4 = (size_t)Q4_STAGES * q4_stage_bytes(4);
    if ((e = opt_in_smem(k_mma_q4<1>, sm1)) != cudaSuccess) return e;
    if ((e = opt_in_smem(k_mma_q4<4>, sm4)) != cudaSuccess) return e;
    // blocks per row block: what fills the SMs at the occupancy each variant reaches (5 and 2 blocks per SM)
    const int gs = std::max(1, std::min(small.cap, (5 * nsm + row_blocks - 1) / row_blocks));
    const int gb = std::max(1, std::min(big.cap, (2 * nsm + row_blocks - 1) / row_blocks));
    q.chunks = small;
    if ((e = launch_k(k_mma_q4<1>, dim3(row_blocks, gs), dim3(Q4_THREADS), sm1, st, q)) != cudaSuccess) return e;
    q.chunks = big;
    return launch_k(k_mma_q4<4>, dim3(row_blocks, gb), dim3(Q4_THREADS), sm4, st, q);
}
// One matrix of the experts (gate/up pairs, or down) on k_umma_q4: planes of the sorted picks, then the grouped GEMM.
static bool umma_q4_fits(const ExpertArgs& a, const ExpertMmaCtx& m, int P) {
    auto ok = [&](int K, size_t off_q, size_t off_s, size_t off_m) {
        return K % UQ_KB == 0 && K <= 64 * UQ_MAXG && (((uintptr_t)m.experts + off_q) & 15) == 0 && (off_s | off_m) % 8 == 0;
    };
    return tensor_map_encoder() && m.sq && m.experts && P <= m.slots && m.expert_bytes % 16 == 0 &&
           ok(a.D, 0, a.off_gu_s, a.off_gu_m) && ok(a.I, a.off_dn_q, a.off_dn_s, a.off_dn_m);
}
// false: a tensor map could not be made, nothing was launched.
static bool launch_umma_q4(const ExpertArgs& a, const ExpertMmaCtx& m, const GroupArgs& g, bool pair, int P, int nsm, cudaStream_t st, cudaError_t* err) {
    auto enc = tensor_map_encoder();
    const int K = pair ? a.D : a.I, rows = pair ? a.I : a.D;
    const size_t off_q = pair ? 0 : a.off_dn_q;
    const uint8_t* base = m.experts + off_q;
    UmmaQ4Args u{};
    {
        const cuuint64_t dims[3] = {(cuuint64_t)K / 2, (cuuint64_t)(pair ? 2 * a.I : a.D), (cuuint64_t)m.per};
        const cuuint64_t strides[2] = {(cuuint64_t)K / 2, (cuuint64_t)m.expert_bytes};
        const cuuint32_t box[3] = {UQ_KB / 2, 64, 1};
        const cuuint32_t es[3] = {1, 1, 1};
        if (enc(&u.wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
    }
    if (!byte_matrix_map(&u.xmap, m.sq, (uint64_t)(K / UM_BK) * m.slots * UM_PI, UM_BK, UQ_NCOL)) return false;
    float* const xsum = m.sq_sum;                            // [slots][K / 64]
    PrepSlotsArgs p{};
    p.src = pair ? a.x : a.act; p.stride = pair ? a.x_stride : a.I; p.by_pick = pair ? 0 : 1; p.topk = a.topk;
    p.norm_w = pair ? a.norm_w : nullptr; p.eps = a.eps; p.K = K; p.P = P; p.list = g.list; p.qi = m.sq; p.slots = m.slots;
    p.xscale = m.sq_scale; p.xsum = xsum;
    if ((*err = launch_k(k_prep_q_slots, dim3(P), dim3(256), 0, st, p)) != cudaSuccess) return true;
    u.eptr = a.eptr; u.list = g.list; u.small = g.small; u.big = g.big; u.topk = a.topk; u.pair = pair ? 1 : 0; u.rows = rows; u.K = K;
    u.up_row0 = a.I; u.e0 = m.e0; u.rbu = std::max(1, 2048 / K);     // about 8 ring steps per unit
    u.off_s = pair ? a.off_gu_s : a.off_dn_s; u.off_m = pair ? a.off_gu_m : a.off_dn_m;
    u.slots = m.slots; u.xscale = m.sq_scale; u.xsum = xsum; u.out = pair ? a.act : a.ypart; u.err = a.err;
    if ((*err = opt_in_smem(k_umma_q4, UQ_SMEM)) != cudaSuccess) return true;
    *err = launch_k(k_umma_q4, dim3(nsm), dim3(UQ_THREADS), UQ_SMEM, st, u);
    g_umma_launches++;
    return true;
}

static cudaError_t launch_experts_mma(const ExpertArgs& a, int T, const ExpertMmaCtx& m, int nsm, cudaStream_t st, b2_engine* prof) {
    cudaError_t e;
    const int P = T * a.topk;
    GroupArgs g{};
    g.top_idx = a.top_idx; g.idx_stride = a.idx_stride; g.T = T; g.topk = a.topk; g.E = a.E; g.eptr = a.eptr;
    g.list = m.list;
    chunk_tables(m, g.small, g.big);
    const bool q4_umma = umma_q4_fits(a, m, P);               // else (K not a multiple of 256, no tensor-map encoder): k_mma_q4
    g.big_n = q4_umma ? UQ_TT : 0;
    if ((e = launch_k(k_group_picks, dim3(1), dim3(1024), 0, st, g)) != cudaSuccess) return e;
    bool gu_done = false, dn_done = false;
    if (q4_umma) {
        gu_done = launch_umma_q4(a, m, g, true, P, nsm, st, &e);
        if (gu_done && e != cudaSuccess) return e;
    }
    if (gu_done) {
        if (prof) prof->mark(5, st);
        dn_done = launch_umma_q4(a, m, g, false, P, nsm, st, &e);
        if (dn_done && e != cudaSuccess) return e;
    }
    Q4Args q{};
    q.eptr = a.eptr; q.list = g.list; q.topk = a.topk;
    if (!gu_done) {
        PrepArgs p{};
        p.x = a.x; p.x_stride = a.x_stride; p.norm_w = a.norm_w; p.eps = a.eps; p.K = a.D; p.T = T; p.Tpad = T; p.out = m.xh;
        p.xsum = m.xsum_tok; p.perm8 = 1;
        if ((e = launch_k(k_prep_x, dim3(T), dim3(256), 0, st, p)) != cudaSuccess) return e;
        q.pair = 1; q.rows = a.I; q.K = a.D; q.off_q = 0; q.off_s = a.off_gu_s; q.off_m = a.off_gu_m; q.up_row0 = a.I;
        q.xh = m.xh; q.xsum = m.xsum_tok; q.by_pick = 0; q.out = a.act; q.row_tiles = 1;
        if ((e = launch_q4(q, g.small, g.big, (a.I + 31) / 32, nsm, st)) != cudaSuccess) return e;
        if (prof) prof->mark(5, st);
    }
    if (!dn_done) {
        PrepArgs p2{};
        p2.x = a.act; p2.x_stride = a.I; p2.K = a.I; p2.T = P; p2.Tpad = P; p2.out = m.acth; p2.xsum = m.xsum_act; p2.perm8 = 1;
        if ((e = launch_k(k_prep_x, dim3(P), dim3(256), 0, st, p2)) != cudaSuccess) return e;
        q.pair = 0; q.rows = a.D; q.K = a.I; q.off_q = a.off_dn_q; q.off_s = a.off_dn_s; q.off_m = a.off_dn_m; q.up_row0 = 0;
        q.xh = m.acth; q.xsum = m.xsum_act; q.by_pick = 1; q.out = a.ypart;
        q.row_tiles = std::max(1, std::min(4, 2048 / a.I));      // keep about 8 ring steps per block
        if ((e = launch_q4(q, g.small, g.big, (a.D + Q4_ROWS * q.row_tiles - 1) / (Q4_ROWS * q.row_tiles), nsm, st)) != cudaSuccess) return e;
    }
    // shared expert down for this GPU's own tokens: int8 [D][SH] on the dense tensor-core kernel
    PrepArgs p3{};
    p3.x = a.sh_act; p3.x_stride = a.SH; p3.K = a.SH; p3.T = a.nlocal; p3.Tpad = (a.nlocal + MM_TOK - 1) / MM_TOK * MM_TOK; p3.out = m.xh;
    if ((e = launch_k(k_prep_x, dim3(p3.Tpad), dim3(256), 0, st, p3)) != cudaSuccess) return e;
    MmaArgs d{};
    d.seg[0].w = a.shd_w; d.seg[0].s = a.shd_s; d.seg[0].rows = a.D; d.seg[0].kind = SEG_I8;
    d.seg[0].out = a.ypart + ((size_t)a.local0 * (a.topk + 1) + a.topk) * a.D; d.seg[0].out_stride = (a.topk + 1) * a.D;
    d.seg[0].blocks = (a.D + MM_ROWS - 1) / MM_ROWS;
    d.nseg = 1; d.total_blocks = d.seg[0].blocks; d.xh = m.xh; d.K = a.SH; d.T = a.nlocal;
    if ((e = launch_mma_i8(d, p3.Tpad / MM_TOK, nsm, st)) != cudaSuccess) return e;
    if (prof) prof->mark(6, st);
    return cudaSuccess;
}

static cudaError_t launch_attn(const AttnArgs& a, int HD, bool f32, int B, cudaStream_t st, int tiles_per_slice, int nsm, b2_engine* prof = nullptr) {
    const int G = a.H / a.KV;
    const size_t smem = (size_t)WARPS * G * HD * 4;
    dim3 g(a.nsplit, a.KV, B);
#define ATT(hd, f)                                                                     \
    {                                                                                  \
        cudaError_t e = opt_in_smem(k_attn<hd, f>, smem);                              \
        if (e != cudaSuccess) return e;                                                \
        launch_k(k_attn<hd, f>, g, THREADS, smem, st, a);                              \
    }
    const int hr = a.RD / 2;
    const bool rope_ok = hr % 32 == 0 || (hr > 0 && hr < 32 && (hr & (hr - 1)) == 0);   // pairs in one lane, or a power of two lanes apart
    if (!f32 && G <= 8 && rope_ok && (HD == 256 || HD == 128 || HD == 64)) {
        // bf16 cache: both contractions on the tensor cores; two tile buffers when a slice can span several tiles
        // with two or more blocks per SM to choose from, two single-buffered blocks on an SM (registers allow two) hide a
        // tile's latency behind each other's products better than one double-buffered block does
        const int nbuf = (tiles_per_slice > 1 && (long)a.nsplit * a.KV * B < 2L * nsm) ? 2 : 1;
        cudaError_t e;
#define ATM(hd)                                                                                     \
    {                                                                                               \
        e = opt_in_smem(k_attn_mma<hd>, am_smem<hd>(nbuf));                                         \
        if (e == cudaSuccess) e = launch_k(k_attn_mma<hd>, g, THREADS, am_smem<hd>(nbuf), st, a, nbuf); \
    }
        if (HD == 256) ATM(256) else if (HD == 128) ATM(128) else ATM(64)
#undef ATM
        if (e != cudaSuccess) return e;
        launch_k(k_attn_merge, dim3(a.H, B), THREADS, 0, st, a, HD);
        return cudaSuccess;
    }
    if (HD == 64) { if (f32) ATT(64, true) else ATT(64, false) }
    else if (HD == 128) { if (f32) ATT(128, true) else ATT(128, false) }
    else { if (f32) ATT(256, true) else ATT(256, false) }
#undef ATT
    launch_k(k_attn_merge, dim3(a.H, B), THREADS, 0, st, a, HD);
    return cudaSuccess;
}

// The expert kernels for fewer than BATCH_GEMM_MIN tokens (moe1.cuh): shapes they take, and their two launches. `x_in` rows are
// normalised with `norm_w` when it is given; the result is added into `xout`.
static bool moe1_shape_ok(const Cfg& c) {
    return (c.D == 512 || c.D == 1024 || c.D == 2048 || c.D == 4096) && c.I >= 128 && c.I <= 2048 && (c.I & (c.I - 1)) == 0 &&
           c.SH % 128 == 0 && c.TOPK <= 8 && c.E <= 256;
}
struct Moe1Ctx { const uint8_t** top_ptr; int8_t* actq; float* asc; float* asum; };
static cudaError_t launch_moe1(const Cfg& c, const float* rlogits, const float* x_in, const uint16_t* norm_w, const uint8_t* const* eptr,
                               int* top_idx, float* top_w, const Moe1Ctx& m, const float* sh_act, const float* sgate, const int8_t* shd_w,
                               const uint16_t* shd_s, float* xout, int* err, int B, cudaStream_t st, b2_engine* prof,
                               const CoreRoute* core = nullptr, const CoresLiveArgs* live = nullptr) {
    Gu1Args g{};
    if (core) g.core = *core;
    g.logits = rlogits; g.x = x_in; g.norm_w = norm_w; g.eps = c.eps; g.eptr = eptr;
    g.off_gu_s = c.off_gu_s(); g.off_gu_m = c.off_gu_m(); g.D = c.D; g.I = c.I; g.E = c.E; g.topk = c.TOPK;
    g.top_idx = top_idx; g.top_w = top_w; g.top_ptr = m.top_ptr; g.actq = m.actq; g.asc = m.asc; g.asum = m.asum; g.err = err;
    const int gx = c.TOPK * c.I / M1_GU_PAIRS;
    cudaError_t ce = opt_in_smem(k_moe_gu1, m1_gu_smem(c.D));
    if (ce == cudaSuccess) ce = launch_k(k_moe_gu1, dim3(gx, B), dim3(M1_GU_THREADS), m1_gu_smem(c.D), st, g);
    if (prof) prof->mark(5, st);
    // the gate/up kernel has made the core engine's picks; the live cores read x before the down kernel writes it
    if (live && ce == cudaSuccess) ce = launch_k(k_cores_live, dim3(B), dim3(256), (size_t)(live->D + live->r) * 4, st, *live);
    Down1Args d{};
    d.top_ptr = m.top_ptr; d.top_w = top_w; d.actq = m.actq; d.asc = m.asc; d.asum = m.asum; d.sh_act = sh_act; d.sg = sgate;
    d.shd_w = shd_w; d.shd_s = shd_s;
    d.off_dn_q = c.off_dn_q(); d.off_dn_s = c.off_dn_s(); d.off_dn_m = c.off_dn_m();
    d.D = c.D; d.I = c.I; d.SH = c.SH; d.topk = c.TOPK; d.xout = xout;
    const size_t dsm = m1_down_smem(c.I, c.SH, c.TOPK);
    if (ce == cudaSuccess) ce = opt_in_smem(k_moe_down1, dsm);
    if (ce == cudaSuccess)
        ce = launch_k(k_moe_down1, dim3((c.D + M1_DOWN_ROWS - 1) / M1_DOWN_ROWS, B), dim3(2 * (c.TOPK + 1) * 32), dsm, st, d);
    if (prof) prof->mark(6, st);
    return ce;
}

// One decode step for all B sequences: token ids in d_tok, positions in d_pos.
// chunk_T > 0: a prompt chunk of chunk_T tokens of the engine's one sequence instead (the tokens are the columns of
// every matrix product; conv, delta rule and attention walk them in order; the head runs for the last token only,
// and only when chunk_head is set).
int b2_engine::enqueue_step(cudaStream_t st, bool count, int chunk_T, bool chunk_head) {
    int n = 0;
    const int launches0 = g_launch_count;
    const bool chunk = chunk_T > 0;
    const int NSEQ = this->B;                     // sequences: what the recurrent state, the conv taps and the KV pages are laid out by
    const int B = chunk ? chunk_T : this->B;      // columns of this step's matrix products
    // the work buffers of this step: the members, or the chunk's own set under the same names
    int* const d_tok = chunk ? pc.tok : this->d_tok;
    int* const d_pos = chunk ? pc.vpos : this->d_pos;
    float* const x = chunk ? pc.x : this->x;
    float* const big = chunk ? pc.big : this->big;
    float* const zbuf = chunk ? pc.zbuf : this->zbuf;
    float* const kraw = chunk ? pc.kraw : this->kraw;
    float* const vraw = chunk ? pc.vraw : this->vraw;
    float* const beta = chunk ? pc.beta : this->beta;
    float* const gdec = chunk ? pc.gdec : this->gdec;
    float* const obuf = chunk ? pc.obuf : this->obuf;
    float* const att = chunk ? pc.att : this->att;
    float* const rlogits = chunk ? pc.rlogits : this->rlogits;
    float* const sh_act = chunk ? pc.sh_act : this->sh_act;
    float* const sgate = chunk ? pc.sgate : this->sgate;
    float* const act = chunk ? pc.act : this->act;
    float* const ypart = chunk ? pc.ypart : this->ypart;
    float* const attn_part = chunk ? pc.attn_part : this->attn_part;
    unsigned int* const d_dcounter = chunk ? pc.dcounter : this->d_dcounter;
    unsigned int* const d_counter = chunk ? pc.counter : this->d_counter;
    __half* const xh = chunk ? pc.xh : this->xh;
    __half* const acth = chunk ? pc.acth : this->acth;
    int* const g_list = chunk ? pc.g_list : this->g_list;
    int* const g_chunk = chunk ? pc.g_chunk : this->g_chunk;
    float* const xsum_tok = chunk ? pc.xsum_tok : this->xsum_tok;
    float* const xsum_act = chunk ? pc.xsum_act : this->xsum_act;
    const int cap_small = chunk ? pc.cap_small : this->cap_small, cap_big = chunk ? pc.cap_big : this->cap_big;
    const int nsplit = chunk ? pc.nsplit : this->nsplit, attn_tiles = chunk ? pc.attn_tiles : this->attn_tiles;
    const BatchCtx bctx = chunk ? BatchCtx{pc.xh, pc.xh_tpad, pc.uq_i, pc.uq_b, pc.uq_scale, pc.uq_passes}
                                : BatchCtx{this->xh, xh_tpad, uq_i, uq_b, uq_scale, uq_passes};
    const BatchCtx* bc = xh ? &bctx : nullptr;
    cudaGetLastError();   // a stale error of an earlier, unrelated call must not be blamed on these launches
    mark(-1, st);
    launch_k(k_embed, dim3(B), dim3(256), 0, st, embed, (const int*)d_tok, x, c.D, c.V, d_err);
    if (chunk) launch_k(k_iota_from, dim3((B + 255) / 256), dim3(256), 0, st, d_pos, (const int*)this->d_pos, B);
    mark(0, st);
    n++;
    const size_t kv_layer = (size_t)NSEQ * pages_per_seq * c.KV * KV_PAGE * c.HD * (kv_f32 ? 4 : 2);
    for (int li = 0; li < c.L; li++) {
        const LayerW& l = layers[li];
        if (l.attn) {
            GemvArgs a{};
            a.seg[0] = make_seg(SEG_I8, l.q.w, l.q.s, l.q.n, big, 2 * c.H * c.HD);
            a.seg[1] = make_seg(SEG_I8, l.k.w, l.k.s, l.k.n, kraw, c.KV * c.HD);
            a.seg[2] = make_seg(SEG_I8, l.v.w, l.v.s, l.v.n, vraw, c.KV * c.HD);
            a.nseg = 3; seal(a, c.D);
            a.x = x; a.norm_w = l.norm1; a.eps = c.eps; a.K = c.D; a.err = d_err;
            launch_gemv(a, B, nsm, st, 0, bc);
            mark(1, st);
            AttnArgs t{};
            t.qraw = big; t.kraw = kraw; t.vraw = vraw; t.qn_w = l.q_norm; t.kn_w = l.k_norm;
            t.rope_cos = rope_cos; t.rope_sin = rope_sin; t.pos = d_pos;
            t.kpool = (char*)kpool + kv_layer * l.slot; t.vpool = (char*)vpool + kv_layer * l.slot;
            t.page_table = page_table; t.pages_per_seq = pages_per_seq; t.pt_stride = chunk ? 0 : pages_per_seq;
            t.H = c.H; t.KV = c.KV; t.RD = c.RD; t.eps = c.eps; t.scale = 1.0f / std::sqrt((float)c.HD);
            t.part = attn_part; t.out = att; t.nsplit = nsplit;
            cudaError_t e = cudaSuccess;
            if (chunk) {
                // every token's key and value row goes into the cache first: a token's blocks then find the rows of the
                // chunk's earlier tokens there (they write their own row again, with the same bytes)
                AttnArgs ap = t;
                ap.append_only = 1;
                e = launch_attn(ap, c.HD, kv_f32, B, st, attn_tiles, nsm);
            }
            if (e == cudaSuccess) e = launch_attn(t, c.HD, kv_f32, B, st, attn_tiles, nsm);
            if (e != cudaSuccess) return fail("attention launch: %s", cudaGetErrorString(e));
            mark(3, st);
            ProjArgs p{};
            p.in = att; p.mode = 1; p.w = l.o.w; p.s = l.o.s; p.x = x; p.N = c.D; p.K = c.H * c.HD; p.eps = c.eps; p.DV = c.DV;
            launch_proj(p, B, nsm, st, bc);
        } else {
            GemvArgs a{};
            a.seg[0] = make_seg(chunk ? SEG_I8 : SEG_I8_CONV, l.in_qkv.w, l.in_qkv.s, l.in_qkv.n, big, c.C());
            a.seg[1] = make_seg(SEG_I8_SILU, l.in_z.w, l.in_z.s, l.in_z.n, zbuf, c.VD());
            a.seg[2] = make_seg(SEG_BF_SIGMOID, l.in_b, nullptr, c.HV, beta, c.HV);
            a.seg[3] = make_seg(SEG_BF_DECAY, l.in_a, nullptr, c.HV, gdec, c.HV);
            a.nseg = 4; seal(a, c.D);
            a.x = x; a.norm_w = l.norm1; a.eps = c.eps; a.K = c.D; a.err = d_err;
            a.conv_w = l.conv; a.conv_state = conv + (size_t)l.slot * NSEQ * c.C() * 3;
            a.a_log = l.a_log; a.dt_bias = l.dt_bias;
            launch_gemv(a, B, nsm, st, 0, bc);
            mark(1, st);
            float* const lstate = state + (size_t)l.slot * NSEQ * c.HV * c.DK * c.DV;
            if (chunk) {
                ConvScanArgs cs{big, l.conv, a.conv_state, c.C(), B};
                launch_k(k_conv_scan, dim3((c.C() + 255) / 256), dim3(256), 0, st, cs);
                DeltaScanArgs ds{big, beta, gdec, lstate, obuf, c.C(), c.HK, c.HV, c.DV, B};
                const dim3 g(c.HV * (c.DV / 32));
                if (c.DK == 64) launch_k(k_delta_scan<64>, g, dim3(THREADS), 0, st, ds);
                else launch_k(k_delta_scan<128>, g, dim3(THREADS), 0, st, ds);
            } else {
            DeltaArgs d{};
            d.y = big; d.beta = beta; d.g = gdec; d.state = lstate;
            d.o = obuf; d.C = c.C(); d.HK = c.HK; d.HV = c.HV; d.DV = c.DV; d.prenormed = 0;
            launch_delta(d, c.DK, B, st);
            }
            mark(2, st);
            ProjArgs p{};
            p.in = obuf; p.z = zbuf; p.gn_w = l.gnorm; p.eps = c.eps; p.DV = c.DV; p.mode = 0;
            p.w = l.out.w; p.s = l.out.s; p.x = x; p.N = c.D; p.K = c.VD();
            launch_proj(p, B, nsm, st, bc);
        }
        mark(4, st);
        n += l.attn ? 4 : 3;
        {
            GemvArgs a{};
            a.seg[0] = make_seg(SEG_BF, l.router, nullptr, c.E, rlogits, c.E);
            a.seg[0].bias = l.router_bias;
            a.seg[1] = make_seg(SEG_I8_GATEUP, l.sh_gate.w, l.sh_gate.s, c.SH, sh_act, c.SH);
            a.seg[1].w2 = l.sh_up.w; a.seg[1].s2 = l.sh_up.s;
            a.seg[2] = make_seg(SEG_BF_SIGMOID, l.sh_gw, nullptr, 1, sgate, 1);
            a.nseg = 3;
            // the core engine's two key tables ride along: their scores, then the picks where the router's are made
            float* const cscore = chunk ? pc.cscore : this->cscore;
            int* const csel = chunk ? pc.csel : this->csel;
            float* const cselw = chunk ? pc.cselw : this->cselw;
            float* const core_y = chunk ? pc.core_y : this->core_y;
            CoreRoute cr{};
            if (l.key1) {
                a.seg[3] = make_seg(SEG_BF, l.key1, nullptr, c.n1, cscore, c.n1 + c.n2);
                a.seg[4] = make_seg(SEG_BF, l.key2, nullptr, c.n2, cscore + c.n1, c.n1 + c.n2);
                a.nseg = 5;
                cr.score = cscore; cr.n1 = c.n1; cr.n2 = c.n2; cr.k = c.cores_active;
                cr.counts = d_counts + (size_t)li * c.n1 * c.n2; cr.sel = csel; cr.selw = cselw;
            }
            seal(a, c.D);
            a.core = cr;
            // the layer's live cores: their output goes to core_y once the picks are known and before the experts write x
            CoresLiveArgs cl{};
            const bool has_live = l.key1 && l.n_live > 0;
            if (has_live) {
                cl.x = x; cl.norm_w = l.norm2; cl.eps = c.eps; cl.live = l.live; cl.cg = l.cg; cl.cu = l.cu; cl.cd = l.cd;
                cl.sel = csel; cl.selw = cselw; cl.y = core_y; cl.D = c.D; cl.r = c.rank; cl.k = c.cores_active;
            }
            auto launch_live = [&]() {
                if (has_live) launch_k(k_cores_live, dim3(B), dim3(256), (size_t)(c.D + c.rank) * 4, st, cl);
            };
            a.x = x; a.norm_w = l.norm2; a.eps = c.eps; a.K = c.D; a.err = d_err;
            // fewer than BATCH_GEMM_MIN tokens on one GPU: the top-8 moves into the expert kernel and the experts are spread over all SMs
            const bool moe1 = ep_world == 1 && B < BATCH_GEMM_MIN && moe1_shape_ok(c);
            a.finisher = moe1 ? FIN_NONE : FIN_TOPK; a.counter = d_counter; a.E = c.E; a.topk = c.TOPK;
            // a chunk's picks live in its own scratch; the last token's are kept where a decode step's are (b2_debug_router)
            a.top_idx = chunk ? pc.top_idx : top_idx + (size_t)li * B * c.TOPK;
            a.top_w = chunk ? pc.top_w : top_w + (size_t)li * B * c.TOPK;
            launch_gemv(a, B, nsm, st, 0, bc);
            if (chunk) {
                cudaMemcpyAsync(top_idx + (size_t)li * NSEQ * c.TOPK, pc.top_idx + (size_t)(B - 1) * c.TOPK, c.TOPK * sizeof(int), cudaMemcpyDeviceToDevice, st);
                cudaMemcpyAsync(top_w + (size_t)li * NSEQ * c.TOPK, pc.top_w + (size_t)(B - 1) * c.TOPK, c.TOPK * sizeof(float), cudaMemcpyDeviceToDevice, st);
            }
            mark(1, st);
            if (!moe1) launch_live();              // the picks were made by the launch above (its finisher, or k_router_topk)
            if (moe1) {
                const Moe1Ctx mc{top_ptr, actq, asc, asum};
                cudaError_t ce = launch_moe1(c, rlogits, x, l.norm2, l.eptr, a.top_idx, a.top_w, mc, sh_act, sgate, (const int8_t*)l.sh_down.w,
                                             l.sh_down.s, x, d_err, B, st, this, &cr, has_live ? &cl : nullptr);
                if (ce != cudaSuccess) return fail("expert kernels: %s", cudaGetErrorString(ce));
                n += 3;
            } else {
            ExpertArgs x2{};
            x2.eptr = l.eptr; x2.topk = c.TOPK; x2.E = c.E; x2.D = c.D; x2.I = c.I;
            x2.off_gu_s = c.off_gu_s(); x2.off_gu_m = c.off_gu_m(); x2.off_dn_q = c.off_dn_q(); x2.off_dn_s = c.off_dn_s(); x2.off_dn_m = c.off_dn_m();
            x2.norm_w = l.norm2; x2.eps = c.eps; x2.act = act; x2.sh_act = sh_act; x2.sg = sgate;
            x2.shd_w = l.sh_down.w; x2.shd_s = l.sh_down.s; x2.SH = c.SH; x2.xout = x; x2.err = d_err;
            x2.ypart = ypart; x2.counter = d_dcounter; x2.null_is_error = ep_world == 1;
            const int Tg = B * ep_world;
            const bool grouped = xh && Tg >= BATCH_GEMM_MIN && Tg * c.TOPK <= GQ_MAXP && c.D % MM_KC == 0 && c.I % MM_KC == 0 &&
                                 c.SH % MM_KC == 0 && c.D <= 2048 && c.I <= 2048 && c.E <= 256;
            const ExpertMmaCtx mctx{g_list, g_chunk, cap_small, cap_big, xh, acth, xsum_tok, xsum_act,
                                    chunk ? pc.sq : sq, chunk ? pc.sq_scale : sq_scale, chunk ? pc.sq_sum : sq_sum, Tg * c.TOPK,
                                    l.experts, c.expert_bytes(), c.E / ep_world, ep_rank * (c.E / ep_world)};
            if (ep_world == 1) {
                x2.x = x; x2.x_stride = c.D; x2.top_idx = a.top_idx; x2.top_w = a.top_w; x2.idx_stride = c.TOPK;
                x2.combine = 1; x2.local0 = 0; x2.nlocal = B;
                if (grouped) {
                    cudaError_t ce = launch_experts_mma(x2, B, mctx, nsm, st, this);
                    if (ce != cudaSuccess) return fail("grouped expert GEMM: %s", cudaGetErrorString(ce));
                    EpArgs ep{};
                    ep.x = x; ep.top_idx = a.top_idx; ep.top_w = a.top_w; ep.recv_y = ypart; ep.sg = sgate; ep.xout = x;
                    ep.D = c.D; ep.topk = c.TOPK; ep.B = B; ep.E = c.E; ep.world = 1; ep.rank = 0; ep.has_shared = 1;
                    launch_k(k_ep_combine, dim3(std::max(1, (c.D + 255) / 256), B), dim3(256), 0, st, ep);
                } else {
                    launch_experts(x2, B, nsm, st, this);
                }
            } else {
                const int rw = c.D + 2 * c.TOPK;
                EpArgs ep{};
                ep.x = x; ep.top_idx = a.top_idx; ep.top_w = a.top_w; ep.rec = rec_local; ep.recv_y = recv_y; ep.sg = sgate; ep.xout = x;
                ep.D = c.D; ep.topk = c.TOPK; ep.B = B; ep.E = c.E; ep.world = ep_world; ep.rank = ep_rank; ep.has_shared = 1;
                EpPushArgs pa{};
                if (ep_peer_ready) {
                    for (int p = 0; p < ep_world; p++) pa.peers.base[p] = ep_peer[p];
                    pa.peers.rec_off = 0; pa.peers.y_off = (size_t)(recv_y - ep_block); pa.peers.flag_off = ep_flag_off;
                    pa.x = x; pa.top_idx = a.top_idx; pa.top_w = a.top_w; pa.ypart = ypart; pa.D = c.D; pa.topk = c.TOPK; pa.B = B; pa.E = c.E;
                    pa.world = ep_world; pa.rank = ep_rank; pa.seq = d_ep_seq; pa.rows_sent = d_ep_rows; pa.err = d_err;
                    const int nb0 = std::min(B, EP_MAX_BLOCKS);
                    launch_k(k_ep_push_records, dim3(nb0), dim3(256), 0, st, pa);
                    launch_k(k_ep_wait, dim3(1), dim3(EP_MAX_WORLD * EP_MAX_BLOCKS), 0, st, EpWaitArgs{nullptr, (int*)ep_block + ep_flag_off, d_ep_seq, 0, ep_world, ep_rank, nb0, 1 << 21, d_err});
                } else {
                    launch_k(k_ep_pack, dim3(B), dim3(256), 0, st, ep);
                    if (ep_exchange_records(st)) return 1;
                }
                x2.x = rec_all; x2.x_stride = rw; x2.top_idx = (const int*)(rec_all + c.D); x2.top_w = rec_all + c.D + c.TOPK; x2.idx_stride = rw;
                x2.combine = 0; x2.local0 = ep_rank * B; x2.nlocal = B;
                if (grouped) {
                    cudaError_t ce = launch_experts_mma(x2, Tg, mctx, nsm, st, this);
                    if (ce != cudaSuccess) return fail("grouped expert GEMM: %s", cudaGetErrorString(ce));
                } else {
                    launch_experts(x2, Tg, nsm, st, this);
                }
                if (ep_peer_ready) {
                    launch_k(k_ep_push_outputs, dim3(EP_MAX_BLOCKS), dim3(256), 0, st, pa);
                    launch_k(k_ep_wait, dim3(1), dim3(EP_MAX_WORLD * EP_MAX_BLOCKS), 0, st, EpWaitArgs{nullptr, (int*)ep_block + ep_flag_off, d_ep_seq, 1, ep_world, ep_rank, EP_MAX_BLOCKS, 1 << 21, d_err});
                } else if (ep_exchange_outputs(st)) return 1;
                launch_k(k_ep_combine, dim3(std::max(1, (c.D + 255) / 256), B), dim3(256), 0, st, ep);
                n += 2;
            }
            n += 3;
            }
        }
        if (l.key1 && l.n_live > 0) {
            float* const cy = chunk ? pc.core_y : this->core_y;
            launch_k(k_add_rows, dim3((B * c.D + 255) / 256), dim3(256), 0, st, x, (const float*)cy, B * c.D);
        }
        for (size_t j = 0; j < tap_layers.size(); j++)
            if (tap_layers[j] == li) {
                // the hidden state after this layer, of every sequence's token; of a chunk's last token
                if (chunk) cudaMemcpyAsync(tap_buf + j * (size_t)NSEQ * c.D, x + (size_t)(B - 1) * c.D, (size_t)c.D * 4, cudaMemcpyDeviceToDevice, st);
                else cudaMemcpyAsync(tap_buf + j * (size_t)B * c.D, x, (size_t)B * c.D * 4, cudaMemcpyDeviceToDevice, st);
            }
    }
    if (!chunk || chunk_head) {
        GemvArgs a{};
        a.seg[0] = make_seg(SEG_I8_ARGMAX, lm_head.w, lm_head.s, c.V, logits, c.V);
        a.nseg = 1; seal(a, c.D);
        a.x = chunk ? x + (size_t)(B - 1) * c.D : x; a.norm_w = norm; a.eps = c.eps; a.K = c.D; a.err = d_err;
        a.finisher = FIN_ARGMAX; a.counter = this->d_counter; a.part_val = part_val; a.part_idx = part_idx;
        a.next_tok = d_next; a.pos = chunk ? nullptr : d_pos;
        // a chunk's head runs for its last token alone (the decode GEMV), and leaves the residual row where a decode step does
        launch_gemv(a, chunk ? 1 : B, nsm, st, head_grid, chunk ? nullptr : bc);
        mark(7, st);
        n++;
    }
    if (chunk) {
        cudaMemcpyAsync(this->x, x + (size_t)(B - 1) * c.D, (size_t)c.D * 4, cudaMemcpyDeviceToDevice, st);
        k_add_i32<<<1, 32, 0, st>>>(this->d_pos, B, NSEQ);                  // the sequence is B positions further
    }
    (void)n;
    if (count) launches = g_launch_count - launches0;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("kernel launch: %s", cudaGetErrorString(e));
    return 0;
}

// ---- prompt chunks ------------------------------------------------------------------------------------------------
constexpr int CHUNK_TOKENS = 128;        // tokens per chunk: what the pick grouping handles at once (GQ_MAXP picks)
constexpr int CHUNK_MIN = 16;            // shorter feeds (and the rest of a longer one) go token by token

int b2_engine::ensure_chunk_bufs() {
    if (pc.W) return 0;
    const int W = CHUNK_TOKENS;
    const int bigw = std::max(2 * c.H * c.HD, c.C());
    const size_t P = (size_t)W * c.TOPK;
    CU(dalloc(&pc.tok, W)); CU(dalloc(&pc.vpos, W));
    CU(dalloc(&pc.x, (size_t)W * c.D)); CU(dalloc(&pc.big, (size_t)W * bigw)); CU(dalloc(&pc.zbuf, (size_t)W * c.VD()));
    CU(dalloc(&pc.kraw, (size_t)W * c.KV * c.HD)); CU(dalloc(&pc.vraw, (size_t)W * c.KV * c.HD));
    CU(dalloc(&pc.beta, (size_t)W * c.HV)); CU(dalloc(&pc.gdec, (size_t)W * c.HV));
    CU(dalloc(&pc.obuf, (size_t)W * c.VD())); CU(dalloc(&pc.att, (size_t)W * c.H * c.HD));
    CU(dalloc(&pc.rlogits, (size_t)W * c.E)); CU(dalloc(&pc.sh_act, (size_t)W * c.SH)); CU(dalloc(&pc.sgate, W));
    CU(dalloc(&pc.act, P * c.I)); CU(dalloc(&pc.top_idx, P)); CU(dalloc(&pc.top_w, P));
    CU(dalloc(&pc.ypart, (size_t)W * (c.TOPK + 1) * c.D));
    CU(dalloc(&pc.dcounter, (size_t)W * down_row_blocks(c.D))); CU(dalloc(&pc.counter, W));
    // one block set per token already fills the GPU: few, long slices
    pc.nsplit = std::max(1, std::min({64, (2 * nsm) / std::max(1, c.KV * W), (cap + 63) / 64}));
    pc.attn_tiles = ((cap + pc.nsplit - 1) / pc.nsplit + AM_TILE - 1) / AM_TILE;
    CU(dalloc(&pc.attn_part, (size_t)W * c.KV * pc.nsplit * (c.H / c.KV) * (c.HD + 2)));
    pc.xh_tpad = (W + MM_TOK - 1) / MM_TOK * MM_TOK;
    CU(dalloc((uint16_t**)&pc.xh, (size_t)pc.xh_tpad * 2 * 4096));
    pc.uq_passes = (W + UM_TOK - 1) / UM_TOK;
    CU(dalloc(&pc.uq_i, (size_t)pc.uq_passes * UM_PI * UM_TOK * 4096));
    CU(dalloc(&pc.uq_b, (size_t)pc.uq_passes * UM_PB * UM_TOK * 4096));
    CU(dalloc(&pc.uq_scale, (size_t)pc.uq_passes * UM_TOK));
    pc.cap_small = (int)std::min<size_t>(P, c.E);
    pc.cap_big = (int)(P / (GQ_SMALL + 1)) + 1;
    CU(dalloc(&pc.g_list, P));
    CU(dalloc(&pc.g_chunk, (size_t)3 * (pc.cap_small + pc.cap_big) + 2));
    CU(dalloc((uint16_t**)&pc.acth, P * 2 * c.I));
    CU(dalloc(&pc.xsum_tok, (size_t)W * (c.D / 64)));
    CU(dalloc(&pc.xsum_act, P * std::max(1, c.I / 64)));
    CU(dalloc(&pc.sq, (size_t)UM_PI * P * std::max(c.D, c.I))); CU(dalloc(&pc.sq_scale, P)); CU(dalloc(&pc.sq_sum, P * (size_t)(std::max(c.D, c.I) / 64 + 1)));
    CU(dalloc(&pc.csel, (size_t)W * c.cores_active)); CU(dalloc(&pc.cselw, (size_t)W * c.cores_active));
    CU(dalloc(&pc.cscore, (size_t)W * (c.n1 + c.n2))); CU(dalloc(&pc.core_y, (size_t)W * c.D));
    pc.W = W;
    return 0;
}

// T (16 .. CHUNK_TOKENS) tokens of the sequence in one pass over the layers (forward_chunk, aegist_rs/src/hybrid.rs:1023-1025)
int b2_engine::feed_chunk(const uint32_t* ids, int T, bool want_head) {
    if (ensure_chunk_bufs()) return 1;
    CU(cudaMemcpyAsync(pc.tok, ids, (size_t)T * 4, cudaMemcpyHostToDevice, stream));
    if (T == CHUNK_TOKENS && !want_head) {
        // the common case of a long prompt: one graph launch instead of some fifteen launches per layer
        if (!chunk_graph) {
            cudaGraph_t g;
            CU(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
            const int rc = enqueue_step(stream, false, T, false);
            const cudaError_t ce = cudaStreamEndCapture(stream, &g);
            if (rc) return rc;
            if (ce != cudaSuccess) return fail("chunk graph capture: %s", cudaGetErrorString(ce));
            const cudaError_t ci = cudaGraphInstantiate(&chunk_graph, g, 0);
            cudaGraphDestroy(g);
            if (ci != cudaSuccess) { chunk_graph = nullptr; return fail("chunk graph instantiate: %s", cudaGetErrorString(ci)); }
        }
        CU(cudaGraphLaunch(chunk_graph, stream));
    } else if (enqueue_step(stream, false, T, want_head)) return 1;
    length += T;
    hits += (uint64_t)T * c.TOPK * c.L;
    for (int i = 0; i < T; i++) toks.push_back(ids[i]);
    return 0;
}

int b2_engine::build_graph() {
    CU(cudaSetDevice(device));
    if (graph) { cudaGraphExecDestroy(graph); graph = nullptr; }
    cudaGraph_t g;
    CU(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_step(stream, true);
    cudaError_t e = cudaStreamEndCapture(stream, &g);
    if (rc) return rc;
    if (e != cudaSuccess) return fail("graph capture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail("graph instantiate: %s", cudaGetErrorString(e));
    return 0;
}

// The device error word travels to page-locked memory on the stream, so a feed pays one synchronisation for its
// results and the check together.
int b2_engine::check_device_error() {
    uint32_t* slot = h_pin + 2 * std::max(B, 1);
    CU(cudaMemcpyAsync(slot, d_err, 4, cudaMemcpyDeviceToHost, stream));
    CU(cudaStreamSynchronize(stream));
    const int h = (int)*slot;
    if (h) {
        cudaMemsetAsync(d_err, 0, 4, stream);
        cudaStreamSynchronize(stream);
        if (h == 1) return fail("a token id is outside the vocabulary (%d)", c.V);
        if (h == 3) return fail("a bulk copy into shared memory did not complete (bounded wait gave up)");
        if (h == 4) return fail("a block waited too long for another block's results (bounded wait gave up)");
        if (h == 5) return fail("another rank's part of the expert exchange did not arrive (bounded wait gave up)");
        return fail("router returned an expert outside 0..%d", c.E - 1);
    }
    return 0;
}

int b2_engine::run_steps(int n) {
    for (int i = 0; i < n; i++) CU(cudaGraphLaunch(graph, stream));
    if (ep_world > 1) ep_steps += n;
    length += n;
    hits += (uint64_t)n * B * c.TOPK * c.L;
    return 0;
}

int b2_engine::reset_state() {
    CU(cudaMemsetAsync(conv, 0, conv_bytes, stream));
    CU(cudaMemsetAsync(state, 0, state_bytes, stream));
    CU(cudaMemsetAsync(d_pos, 0, B * 4, stream));
    length = 0;
    toks.clear();
    toks_known = true;
    snap_pos[0] = snap_pos[1] = -1;
    return 0;
}

int b2_engine::load_nccl() {
    if (p_ncclAllGather) return 0;
    const char* names[] = {getenv("B2_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n) continue;
        nccl_lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD);        // the copy this process already uses, if any
        if (!nccl_lib) nccl_lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (nccl_lib) break;
    }
    if (!nccl_lib) return fail("cannot load NCCL (libnccl.so.2): %s", dlerror());
#define SYM(name) *(void**)(&p_##name) = dlsym(nccl_lib, #name); if (!p_##name) return fail("NCCL has no %s", #name);
    SYM(ncclGetUniqueId) SYM(ncclCommInitRank) SYM(ncclCommDestroy) SYM(ncclAllGather) SYM(ncclSend) SYM(ncclRecv)
    SYM(ncclGroupStart) SYM(ncclGroupEnd) SYM(ncclGetErrorString)
#undef SYM
    return 0;
}
#define NC(call)                                                                                   \
    do {                                                                                           \
        ncclResult_t r_ = (call);                                                                  \
        if (r_ != ncclSuccess) return fail("%s: %s", #call, p_ncclGetErrorString(r_));             \
    } while (0)

// every GPU's records [B][D + 2 topk] -> all records, in rank order
int b2_engine::ep_exchange_records(cudaStream_t st) {
    const size_t n = (size_t)B * (c.D + 2 * c.TOPK);
    NC(p_ncclAllGather(rec_local, rec_all, n, ncclFloat32, comm, st));
    return 0;
}
// block p of ypart (the picks of GPU p's sequences computed here) goes to GPU p; block q of recv_y comes from GPU q
int b2_engine::ep_exchange_outputs(cudaStream_t st) {
    const size_t blk = (size_t)B * (c.TOPK + 1) * c.D;
    NC(p_ncclGroupStart());
    for (int p = 0; p < ep_world; p++) {
        NC(p_ncclSend(ypart + p * blk, blk, ncclFloat32, p, comm, st));
        NC(p_ncclRecv(recv_y + p * blk, blk, ncclFloat32, p, comm, st));
    }
    NC(p_ncclGroupEnd());
    return 0;
}

// Algorithmic bytes of one decode step by kernel class (0 embed, 1 norm+GEMV groups, 2 delta step,
// 3 attention, 4 output projections, 5 expert gate/up, 6 expert down + shared down, 7 head):
// every weight byte once per step, recurrent state read and written, KV read up to the current length,
// min(B * top-k, E) experts per layer. Activations are not counted.
void b2_engine::class_bytes(double out[8]) const {
    for (int i = 0; i < 8; i++) out[i] = 0;
    auto qwb = [](double n, double k) { return n * k + 2 * n; };
    const double nb = B;
    const double uniq = std::min<double>(nb * c.TOPK, c.E / ep_world);
    out[0] = nb * c.D * 2.0;
    for (int i = 0; i < c.L; i++) {
        if (c.attn[i]) {
            out[1] += c.D * 2.0 + qwb(2 * c.H * c.HD, c.D) + 2 * qwb(c.KV * c.HD, c.D);
            out[3] += 2.0 * c.HD * 2 + nb * 2.0 * c.KV * c.HD * (kv_f32 ? 4 : 2) * (length + 1);
            out[4] += qwb(c.D, c.H * c.HD);
        } else {
            out[1] += c.D * 2.0 + qwb(c.C(), c.D) + qwb(c.VD(), c.D) + 2.0 * c.HV * c.D * 2 + c.C() * c.CK * 2.0 + c.HV * 4.0 +
                      nb * 2.0 * c.C() * 3 * 4;
            out[2] += nb * 2.0 * c.HV * c.DK * c.DV * 4;
            out[4] += qwb(c.D, c.VD()) + c.DV * 2.0;
        }
        out[1] += c.D * 2.0 + (double)c.E * c.D * 2 + c.D * 2.0 + 2 * qwb(c.SH, c.D) + (layers[i].key1 ? (c.n1 + c.n2) * c.D * 2.0 : 0.0);
        out[5] += uniq * (double)(c.gu_q() + 2 * c.gu_sm()) + c.D * 2.0;
        out[6] += uniq * (double)(c.dn_q() + 2 * c.dn_sm()) + qwb(c.D, c.SH);
    }
    out[7] = c.D * 2.0 + qwb(c.V, c.D);
}

// ------------------------------------------------------------------------------------------
extern "C" {

int b2_create(const char* config_json, int max_context, int device, int batch, int kv_dtype, int ep_rank, int ep_world,
              b2_engine** out) {
    if (!out) return 1;
    b2_engine* e = new b2_engine();
    *out = e;
    e->device = device;
    e->B = batch < 1 ? 1 : batch;
    e->cap = max_context;
    e->kv_f32 = kv_dtype == B2_KV_F32;
    e->ep_rank = ep_rank;
    e->ep_world = ep_world < 1 ? 1 : ep_world;
    if (ep_rank < 0 || ep_rank >= e->ep_world) return e->fail("expert-parallel rank %d outside 0..%d", ep_rank, e->ep_world - 1);
    int ndev = 0;
    cudaError_t ce = cudaGetDeviceCount(&ndev);
    if (ce != cudaSuccess || ndev == 0) return e->fail("no CUDA device: %s (this engine has no CPU path)", cudaGetErrorString(ce));
    if (device < 0 || device >= ndev) return e->fail("CUDA device %d does not exist (%d visible)", device, ndev);
    JValue j;
    std::string jerr;
    JParser parser(config_json, strlen(config_json));
    if (!parser.parse(j, jerr)) return e->fail("bad config JSON: %s", jerr.c_str());
    return e->parse_config(j);
}

int b2_put_tensor(b2_engine* e, const char* name, const char* dtype, const int64_t* shape, int ndim, const void* data,
                  size_t nbytes, int data_on_device) {
    if (!e) return 1;
    return e->put(name, dtype, std::vector<int64_t>(shape, shape + ndim), data, nbytes, data_on_device != 0);
}

int b2_finish(b2_engine* e) { return e ? e->finish() : 1; }

int b2_ep_unique_id(b2_engine* e, void* id_out, size_t len) {
    if (!e) return 1;
    if (len < sizeof(ncclUniqueId)) return e->fail("the id buffer needs %zu bytes", sizeof(ncclUniqueId));
    if (e->load_nccl()) return 1;
    ncclUniqueId id;
    ncclResult_t r = e->p_ncclGetUniqueId(&id);
    if (r != ncclSuccess) return e->fail("ncclGetUniqueId: %s", e->p_ncclGetErrorString(r));
    memcpy(id_out, &id, sizeof(id));
    return 0;
}

int b2_ep_init(b2_engine* e, const void* id_in, size_t len) {
    if (!e || !e->finished) return 1;
    if (e->ep_world <= 1) return e->fail("this engine was created for a single GPU");
    if (len < sizeof(ncclUniqueId)) return e->fail("the id buffer needs %zu bytes", sizeof(ncclUniqueId));
    if (e->load_nccl()) return 1;
    cudaError_t ce = cudaSetDevice(e->device);
    if (ce != cudaSuccess) return e->fail("cudaSetDevice: %s", cudaGetErrorString(ce));
    ncclUniqueId id;
    memcpy(&id, id_in, sizeof(id));
    ncclResult_t r = e->p_ncclCommInitRank(&e->comm, e->ep_world, id, e->ep_rank);
    if (r != ncclSuccess) return e->fail("ncclCommInitRank: %s", e->p_ncclGetErrorString(r));
    // one exchange of each kind outside the graph: NCCL sets up its channels on first use
    if (e->ep_exchange_records(e->stream) || e->ep_exchange_outputs(e->stream)) return 1;
    ce = cudaStreamSynchronize(e->stream);
    if (ce != cudaSuccess) return e->fail("first exchange: %s", cudaGetErrorString(ce));
    return e->build_graph();
}

int b2_ep_ipc_handle(b2_engine* e, void* out, size_t len) {
    if (!e || !e->finished) return 1;
    if (e->ep_world <= 1 || !e->ep_block) return e->fail("this engine was created for a single GPU");
    if (len < sizeof(cudaIpcMemHandle_t)) return e->fail("the handle buffer needs %zu bytes", sizeof(cudaIpcMemHandle_t));
    cudaIpcMemHandle_t h;
    cudaError_t ce = cudaSetDevice(e->device);
    if (ce == cudaSuccess) ce = cudaIpcGetMemHandle(&h, e->ep_block);
    if (ce != cudaSuccess) return e->fail("cudaIpcGetMemHandle: %s", cudaGetErrorString(ce));
    memcpy(out, &h, sizeof(h));
    return 0;
}

int b2_ep_ipc_attach(b2_engine* e, const void* handles, size_t len_each, int n) {
    if (!e || !e->finished) return 1;
    if (e->ep_world <= 1 || !e->ep_block) return e->fail("this engine was created for a single GPU");
    if (n != e->ep_world || n > EP_MAX_WORLD || len_each < sizeof(cudaIpcMemHandle_t))
        return e->fail("expected %d handles of %zu bytes (at most %d ranks)", e->ep_world, sizeof(cudaIpcMemHandle_t), EP_MAX_WORLD);
    if (e->ep_peer_ready) return e->fail("the peers' blocks are mapped already");
    if (e->c.D % 4 != 0 || (2 * e->c.TOPK) % 4 != 0) return e->fail("the peer-store exchange needs d_model and 2 x experts_active to be multiples of 4 (16-byte rows)");
    cudaError_t ce = cudaSetDevice(e->device);
    if (ce != cudaSuccess) return e->fail("cudaSetDevice: %s", cudaGetErrorString(ce));
    for (int p = 0; p < n; p++) {
        if (p == e->ep_rank) { e->ep_peer[p] = e->ep_block; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)handles + (size_t)p * len_each, sizeof(h));
        void* ptr = nullptr;
        ce = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (ce != cudaSuccess) {
            for (int q = 0; q < p; q++) if (q != e->ep_rank && e->ep_peer[q]) { cudaIpcCloseMemHandle(e->ep_peer[q]); e->ep_peer[q] = nullptr; }
            cudaGetLastError();
            return e->fail("cudaIpcOpenMemHandle (rank %d): %s", p, cudaGetErrorString(ce));
        }
        e->ep_peer[p] = (float*)ptr;
    }
    e->ep_peer_ready = true;
    return e->comm ? e->build_graph() : 0;          // the step graph holds the exchange's launches
}

int b2_open(const char* nx_path, int max_context, int device, int batch, int kv_dtype, b2_engine** out) {
    if (!out) return 1;
    *out = nullptr;
    NxFile nx;
    std::string err;
    if (!nx.open(nx_path, err)) {
        b2_engine* e = new b2_engine();
        *out = e;
        return e->fail("%s", err.c_str());
    }
    const JValue* cfg = nx.header.get("config");
    // re-serialise the config object: find it in the raw header is not needed, rebuild minimal JSON
    std::string js = "{";
    if (cfg && cfg->type == JValue::Obj) {
        bool first = true;
        for (auto& kv : cfg->obj) {
            const JValue& v = kv.second;
            std::string s;
            char buf[64];
            if (v.type == JValue::Num) { snprintf(buf, sizeof(buf), "%.17g", v.num); s = buf; }
            else if (v.type == JValue::Bool) s = v.b ? "true" : "false";
            else if (v.type == JValue::Str) s = "\"" + v.str + "\"";
            else if (v.type == JValue::Arr) {
                s = "[";
                for (size_t i = 0; i < v.arr.size(); i++) {
                    if (i) s += ",";
                    if (v.arr[i].type == JValue::Num) { snprintf(buf, sizeof(buf), "%.17g", v.arr[i].num); s += buf; }
                    else if (v.arr[i].type == JValue::Str) s += "\"" + v.arr[i].str + "\"";
                    else s += "null";
                }
                s += "]";
            } else s = "null";
            js += std::string(first ? "" : ",") + "\"" + kv.first + "\":" + s;
            first = false;
        }
    }
    js += "}";
    int rc = b2_create(js.c_str(), max_context, device, batch, kv_dtype, 0, 1, out);
    if (rc) return rc;
    b2_engine* e = *out;
    e->fingerprint = nx.fingerprint();
    for (auto& kv : nx.tensors) {
        const NxTensor& t = kv.second;
        if (e->put(kv.first, t.dtype, t.shape, nx.data(t), t.nbytes, false)) return 1;
    }
    return e->finish();
}

int b2_verify_file(const char* nx_path, int ok[3], char* err, size_t err_len) {
    NxFile nx;
    std::string msg;
    if (!nx.open(nx_path, msg)) {
        if (err && err_len) snprintf(err, err_len, "%s", msg.c_str());
        return 1;
    }
    auto r = nx.verify();
    ok[0] = r["base"]; ok[1] = r["engine"]; ok[2] = r["cores"];
    return 0;
}

void b2_close(b2_engine* e) { delete e; }

static int feed_checks(b2_engine* e, int n) {
    if (!e) return 1;
    if (!e->finished) return e->fail("the engine is not loaded (b2_finish has not succeeded)");
    if (e->length + n > e->cap) return e->fail("context full: %d + %d tokens > %d", e->length, n, e->cap);
    cudaError_t ce = cudaSetDevice(e->device);
    if (ce != cudaSuccess) return e->fail("cudaSetDevice: %s", cudaGetErrorString(ce));
    return 0;
}
#define CUE(call)                                                                                      \
    do {                                                                                               \
        cudaError_t e_ = (call);                                                                       \
        if (e_ != cudaSuccess) return e->fail("%s: %s", #call, cudaGetErrorString(e_));                \
    } while (0)

int b2_feed(b2_engine* e, const uint32_t* ids, int n, float* logits_out) {
    if (e && e->B != 1) return e->fail("b2_feed needs an engine opened with batch 1 (this one has %d)", e->B);
    if (e && n < 1) return e->fail("b2_feed needs at least one token");
    if (feed_checks(e, n)) return 1;
    for (int i = 0; i < n; i++)
        if (ids[i] >= (uint32_t)e->c.V) return e->fail("token id %u is outside the vocabulary (%d)", ids[i], e->c.V);
    int i0 = 0;
    // whole chunks of the prompt go through the layers together; what is left (fewer than 16 tokens) token by token
    while (n - i0 >= CHUNK_MIN && e->ep_world == 1) {
        const int T = std::min(CHUNK_TOKENS, n - i0);
        if (e->feed_chunk(ids + i0, T, i0 + T == n)) return 1;
        i0 += T;                     // (the caller's ids are read by stream-ordered copies; the stream is drained before we return)
    }
    for (int i = i0; i < n; i++) {
        // the id travels as a kernel-independent 4-byte copy ordered on the stream
        CUE(cudaMemcpyAsync(e->d_tok, ids + i, 4, cudaMemcpyHostToDevice, e->stream));
        if (e->run_steps(1)) return 1;
        e->toks.push_back(ids[i]);
    }
    if (logits_out) CUE(cudaMemcpyAsync(logits_out, e->logits, (size_t)e->c.V * 4, cudaMemcpyDeviceToHost, e->stream));
    return e->check_device_error();
}

void* b2_host_alloc(size_t bytes) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
void b2_host_free(void* p) {
    if (p) cudaFreeHost(p);
}

int b2_feed_batch(b2_engine* e, const uint32_t* ids, uint32_t* next_greedy, float* logits_out) {
    if (feed_checks(e, 1)) return 1;
    for (int b = 0; b < e->B; b++)
        if (ids[b] >= (uint32_t)e->c.V) return e->fail("token id %u is outside the vocabulary (%d)", ids[b], e->c.V);
    memcpy(e->h_pin, ids, (size_t)e->B * 4);
    CUE(cudaMemcpyAsync(e->d_tok, e->h_pin, (size_t)e->B * 4, cudaMemcpyHostToDevice, e->stream));
    if (e->run_steps(1)) return 1;
    if (e->B == 1) e->toks.push_back(ids[0]); else e->toks_known = false;
    if (next_greedy) CUE(cudaMemcpyAsync(e->h_pin + e->B, e->d_next, (size_t)e->B * 4, cudaMemcpyDeviceToHost, e->stream));
    if (logits_out) CUE(cudaMemcpyAsync(logits_out, e->logits, (size_t)e->B * e->c.V * 4, cudaMemcpyDeviceToHost, e->stream));
    if (e->check_device_error()) return 1;
    if (next_greedy) memcpy(next_greedy, e->h_pin + e->B, (size_t)e->B * 4);
    return 0;
}

int b2_decode_greedy(b2_engine* e, const uint32_t* first, int steps, uint32_t* tokens_out, float* device_ms) {
    if (e && steps < 1) return e->fail("b2_decode_greedy needs at least one step");
    if (feed_checks(e, steps)) return 1;
    const int B = e->B;
    for (int b = 0; b < B; b++)
        if (first[b] >= (uint32_t)e->c.V) return e->fail("token id %u is outside the vocabulary (%d)", first[b], e->c.V);
    int* hist = nullptr;
    CUE(cudaMalloc((void**)&hist, (size_t)steps * B * 4));
    memcpy(e->h_pin, first, (size_t)B * 4);
    CUE(cudaMemcpyAsync(e->d_tok, e->h_pin, (size_t)B * 4, cudaMemcpyHostToDevice, e->stream));
    CUE(cudaEventRecord(e->ev0, e->stream));
    for (int s = 0; s < steps; s++) {
        if (e->run_steps(1)) { cudaFree(hist); return 1; }
        // the arg-max becomes the next input and is kept for the caller: two 4*B-byte device copies
        CUE(cudaMemcpyAsync(e->d_tok, e->d_next, (size_t)B * 4, cudaMemcpyDeviceToDevice, e->stream));
        CUE(cudaMemcpyAsync(hist + (size_t)s * B, e->d_next, (size_t)B * 4, cudaMemcpyDeviceToDevice, e->stream));
    }
    CUE(cudaEventRecord(e->ev1, e->stream));
    CUE(cudaMemcpyAsync(tokens_out, hist, (size_t)steps * B * 4, cudaMemcpyDeviceToHost, e->stream));
    CUE(cudaStreamSynchronize(e->stream));
    cudaFree(hist);
    if (B == 1) {                       // fed: the first token, then every arg-max but the last
        e->toks.push_back(first[0]);
        for (int s = 0; s + 1 < steps; s++) e->toks.push_back(tokens_out[s]);
    } else e->toks_known = false;
    if (device_ms) CUE(cudaEventElapsedTime(device_ms, e->ev0, e->ev1));
    return e->check_device_error();
}

// Lm::crop (aegist_rs/src/hybrid.rs:1029-1059)
int b2_crop(b2_engine* e, int n) {
    if (!e || !e->finished) return -1;
    if (n >= e->length) return e->length;
    cudaSetDevice(e->device);
    int best = -1;
    for (int i = 0; i < 2; i++)
        if (e->snap_pos[i] >= 0 && e->snap_pos[i] <= n && (best < 0 || e->snap_pos[i] > e->snap_pos[best])) best = i;
    bool ok = false;
    if (best >= 0) {
        ok = cudaMemcpyAsync(e->conv, e->snap_conv[best], e->conv_bytes, cudaMemcpyDeviceToDevice, e->stream) == cudaSuccess &&
             cudaMemcpyAsync(e->state, e->snap_state[best], e->state_bytes, cudaMemcpyDeviceToDevice, e->stream) == cudaSuccess;
    }
    if (ok) {
        const int p = (int)e->snap_pos[best];
        e->length = p;
        if ((int)e->toks.size() >= p) e->toks.resize(p);
        k_fill_i32<<<(e->B + 255) / 256, 256, 0, e->stream>>>(e->d_pos, p, e->B);
        for (int i = 0; i < 2; i++) if (e->snap_pos[i] > p) e->snap_pos[i] = -1;
    } else {
        e->reset_state();
    }
    cudaStreamSynchronize(e->stream);
    return e->length;
}

// Lm::snapshot (aegist_rs/src/hybrid.rs:1061-1072)
int b2_snapshot(b2_engine* e) {
    if (!e || !e->finished) return 1;
    for (int i = 0; i < 2; i++) if (e->snap_pos[i] == e->length) return 0;
    int i = (e->snap_pos[0] <= e->snap_pos[1]) ? 0 : 1;   // an empty slot (-1), else the oldest
    CUE(cudaSetDevice(e->device));
    CUE(cudaMemcpyAsync(e->snap_conv[i], e->conv, e->conv_bytes, cudaMemcpyDeviceToDevice, e->stream));
    CUE(cudaMemcpyAsync(e->snap_state[i], e->state, e->state_bytes, cudaMemcpyDeviceToDevice, e->stream));
    CUE(cudaStreamSynchronize(e->stream));
    e->snap_pos[i] = e->length;
    return 0;
}

// ---- saved states (trait Lm::state_key / save_state / load_state, aegist_rs/src/model.rs:375-387) ----
// File format of the reference's engines that save states (aegist_rs/src/next.rs:2442-2548): "AEGSTATE", u64 LE
// header length, JSON {"key", "toks"}, then layer by layer what the first n tokens left behind: an attention
// layer's keys and values per KV head (n rows each), a DeltaNet layer's conv taps [C][3] and state [HV][DK][DV].
std::string b2_engine::state_key() const {
    char buf[96];
    snprintf(buf, sizeof(buf), "-%dx%dx%d%s", c.L, c.KV, c.HD, kv_f32 ? "-kvf32" : "");
    return (fingerprint.empty() ? std::string("tensors") : fingerprint) + buf;
}
// (device address, bytes) of every piece in file order; the KV rows of a head are contiguous within a 64-token page
std::vector<b2_engine::Piece> b2_engine::state_pieces(int n) const {
    std::vector<Piece> v;
    const size_t esz = kv_f32 ? 4 : 2;
    const size_t kv_layer = (size_t)B * pages_per_seq * c.KV * KV_PAGE * c.HD * esz;
    for (const LayerW& l : layers) {
        if (l.attn) {
            for (int h = 0; h < c.KV; h++)
                for (int which = 0; which < 2; which++)
                    for (int p0 = 0; p0 < n; p0 += KV_PAGE) {
                        const int rows = std::min(KV_PAGE, n - p0);
                        char* pool = (char*)(which ? vpool : kpool) + kv_layer * l.slot;
                        v.push_back({pool + (((size_t)(p0 / KV_PAGE) * c.KV + h) * KV_PAGE) * c.HD * esz, (size_t)rows * c.HD * esz});
                    }
        } else {
            v.push_back({(char*)(conv + (size_t)l.slot * B * c.C() * 3), (size_t)c.C() * 3 * 4});
            v.push_back({(char*)(state + (size_t)l.slot * B * c.HV * c.DK * c.DV), (size_t)c.HV * c.DK * c.DV * 4});
        }
    }
    return v;
}

const char* b2_state_key(const b2_engine* e) {
    static thread_local std::string k;
    k = e ? e->state_key() : "";
    return k.c_str();
}

int b2_save_state(b2_engine* e, const char* path) {
    if (!e || !e->finished) return 1;
    if (e->B != 1) return e->fail("states are saved for one sequence (this engine has %d)", e->B);
    if (!e->toks_known || (int)e->toks.size() != e->length) return e->fail("the tokens of this context are not all known to the host (device-side steps were run)");
    CUE(cudaSetDevice(e->device));
    CUE(cudaStreamSynchronize(e->stream));
    const int n = e->length;
    std::string head = "{\"key\":\"" + e->state_key() + "\",\"toks\":[";
    for (int i = 0; i < n; i++) head += (i ? "," : "") + std::to_string(e->toks[i]);
    head += "]}";
    const std::string tmp = std::string(path) + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return e->fail("%s: %s", tmp.c_str(), strerror(errno));
    const uint64_t hl = head.size();
    bool ok = fwrite("AEGSTATE", 1, 8, f) == 8 && fwrite(&hl, 8, 1, f) == 1 && fwrite(head.data(), 1, head.size(), f) == head.size();
    std::vector<char> buf;
    for (auto& pc : e->state_pieces(n)) {
        if (!ok) break;
        buf.resize(pc.bytes);
        if (cudaMemcpy(buf.data(), pc.p, pc.bytes, cudaMemcpyDeviceToHost) != cudaSuccess) { ok = false; break; }
        ok = fwrite(buf.data(), 1, pc.bytes, f) == pc.bytes;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) { remove(tmp.c_str()); cudaGetLastError(); return e->fail("%s: could not write the state", tmp.c_str()); }
    if (rename(tmp.c_str(), path) != 0) return e->fail("%s: %s", path, strerror(errno));
    return 0;
}

int b2_load_state(b2_engine* e, const char* path, uint32_t* toks_out, int cap_toks, int* n_out) {
    if (!e || !e->finished) return 1;
    if (e->B != 1) return e->fail("states are loaded for one sequence (this engine has %d)", e->B);
    CUE(cudaSetDevice(e->device));
    // on any error the engine is left empty (model.rs:383-384)
    e->reset_state();
    cudaStreamSynchronize(e->stream);
    FILE* f = fopen(path, "rb");
    if (!f) return e->fail("%s: %s", path, strerror(errno));
    char magic[16];
    if (fread(magic, 1, 16, f) != 16 || memcmp(magic, "AEGSTATE", 8) != 0) { fclose(f); return e->fail("%s: not a saved state", path); }
    uint64_t hl;
    memcpy(&hl, magic + 8, 8);
    if (hl > (1ull << 30)) { fclose(f); return e->fail("%s: not a saved state", path); }
    std::string head(hl, 0);
    if (fread(&head[0], 1, hl, f) != hl) { fclose(f); return e->fail("%s: truncated", path); }
    JValue j;
    std::string jerr;
    JParser parser(head.data(), head.size());
    if (!parser.parse(j, jerr)) { fclose(f); return e->fail("%s: %s", path, jerr.c_str()); }
    const JValue* key = j.get("key");
    if (!key || key->type != JValue::Str || key->str != e->state_key()) { fclose(f); return e->fail("%s: saved by another brain", path); }
    std::vector<uint32_t> toks;
    if (const JValue* t = j.get("toks")) for (auto& x : t->arr) toks.push_back((uint32_t)x.num);
    const int n = (int)toks.size();
    if (n == 0 || n >= e->cap) { fclose(f); return e->fail("%s: %d tokens do not fit a context of %d", path, n, e->cap); }
    std::vector<char> buf;
    for (auto& pc : e->state_pieces(n)) {
        buf.resize(pc.bytes);
        if (fread(buf.data(), 1, pc.bytes, f) != pc.bytes) { fclose(f); e->reset_state(); return e->fail("%s: truncated", path); }
        if (cudaMemcpy(pc.p, buf.data(), pc.bytes, cudaMemcpyHostToDevice) != cudaSuccess) { fclose(f); cudaGetLastError(); e->reset_state(); return e->fail("%s: upload failed", path); }
    }
    fclose(f);
    k_fill_i32<<<1, 32, 0, e->stream>>>(e->d_pos, n, 1);
    CUE(cudaStreamSynchronize(e->stream));
    e->length = n;
    e->toks = toks;
    e->toks_known = true;
    e->snap_pos[0] = e->snap_pos[1] = -1;
    if (b2_snapshot(e)) return 1;
    if (n_out) *n_out = n;
    if (toks_out) memcpy(toks_out, toks.data(), (size_t)std::min(n, cap_toks) * 4);
    return 0;
}

int b2_length(const b2_engine* e) { return e ? e->length : 0; }
int b2_cap(const b2_engine* e) { return e ? e->cap : 0; }
int b2_vocab(const b2_engine* e) { return e ? e->c.V : 0; }
int b2_d_model(const b2_engine* e) { return e ? e->c.D : 0; }

int b2_set_taps(b2_engine* e, const int* layers, int n) {
    if (!e || !e->finished) return 1;
    for (int i = 0; i < n; i++)
        if (layers[i] < 0 || layers[i] >= e->c.L) return e->fail("tap layer %d out of range (the brain has %d layers)", layers[i], e->c.L);
    CUE(cudaSetDevice(e->device));
    CUE(cudaStreamSynchronize(e->stream));
    cudaFree(e->tap_buf);
    e->tap_buf = nullptr;
    e->tap_layers.assign(layers, layers + n);
    if (n) CUE(dalloc(&e->tap_buf, (size_t)n * e->B * e->c.D));
    if (e->chunk_graph) { cudaGraphExecDestroy(e->chunk_graph); e->chunk_graph = nullptr; }      // it holds the old taps' copies
    return e->build_graph();
}

int b2_taps(b2_engine* e, float* out) {
    if (!e || !e->finished) return 1;
    if (e->tap_layers.empty()) return 0;
    CUE(cudaSetDevice(e->device));
    CUE(cudaMemcpyAsync(out, e->tap_buf, e->tap_layers.size() * (size_t)e->B * e->c.D * 4, cudaMemcpyDeviceToHost, e->stream));
    CUE(cudaStreamSynchronize(e->stream));
    return 0;
}

int b2_core_counts(b2_engine* e, int32_t* out) {
    if (!e || !e->finished) return 1;
    CUE(cudaSetDevice(e->device));
    CUE(cudaStreamSynchronize(e->stream));
    CUE(cudaMemcpy(out, e->d_counts, (size_t)e->c.L * e->c.n1 * e->c.n2 * 4, cudaMemcpyDeviceToHost));
    return 0;
}
int b2_reset_counts(b2_engine* e) {
    if (!e || !e->finished) return 1;
    CUE(cudaSetDevice(e->device));
    CUE(cudaMemsetAsync(e->d_counts, 0, (size_t)e->c.L * e->c.n1 * e->c.n2 * 4, e->stream));
    CUE(cudaStreamSynchronize(e->stream));
    return 0;
}

void b2_expert_counters(const b2_engine* e, uint64_t* hits, uint64_t* page_ins) {
    if (hits) *hits = e ? e->hits : 0;
    if (page_ins) *page_ins = 0;
}

const char* b2_describe(const b2_engine* e) { return e ? e->desc.c_str() : ""; }
const char* b2_last_error(const b2_engine* e) { return e ? e->err.c_str() : "no engine"; }

int b2_debug_router(b2_engine* e, int layer, int32_t* idx, float* wts) {
    if (!e || !e->finished) return 1;
    if (layer < 0 || layer >= e->c.L) return e->fail("layer %d out of range", layer);
    CUE(cudaSetDevice(e->device));
    const size_t n = (size_t)e->B * e->c.TOPK;
    CUE(cudaStreamSynchronize(e->stream));
    if (idx) CUE(cudaMemcpy(idx, e->top_idx + layer * n, n * 4, cudaMemcpyDeviceToHost));
    if (wts) CUE(cudaMemcpy(wts, e->top_w + layer * n, n * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int b2_debug_hidden(b2_engine* e, float* out) {
    if (!e || !e->finished) return 1;
    CUE(cudaSetDevice(e->device));
    CUE(cudaStreamSynchronize(e->stream));
    CUE(cudaMemcpy(out, e->x, (size_t)e->B * e->c.D * 4, cudaMemcpyDeviceToHost));
    return 0;
}

int b2_set_router_bias(b2_engine* e, int layer, const float* bias) {
    if (!e || !e->finished) return 1;
    if (layer < 0 || layer >= e->c.L) return e->fail("layer %d out of range", layer);
    CUE(cudaSetDevice(e->device));
    CUE(cudaStreamSynchronize(e->stream));
    LayerW& l = e->layers[layer];
    if (!bias) CUE(cudaMemset(l.router_bias, 0, (size_t)e->c.E * 4));
    else CUE(cudaMemcpy(l.router_bias, bias, (size_t)e->c.E * 4, cudaMemcpyHostToDevice));
    return 0;
}

int b2_launches_per_step(const b2_engine* e) { return e ? e->launches : 0; }
long b2_debug_umma_launches(void) { return g_umma_launches; }

int b2_debug_seek(b2_engine* e, int n) {
    if (!e || !e->finished) return 1;
    if (n < 0 || n > e->cap) return e->fail("cannot seek to %d (context holds %d)", n, e->cap);
    CUE(cudaSetDevice(e->device));
    k_fill_i32<<<(e->B + 255) / 256, 256, 0, e->stream>>>(e->d_pos, n, e->B);
    CUE(cudaStreamSynchronize(e->stream));
    e->length = n;
    e->toks_known = false;
    return 0;
}

double b2_step_bytes(const b2_engine* e) {
    if (!e) return 0;
    double cls[8];
    e->class_bytes(cls);
    double s = 0;
    for (double v : cls) s += v;
    return s;
}

double b2_ep_bytes_per_step(const b2_engine* e) {
    if (!e || e->ep_world <= 1) return 0;
    const Cfg& c = e->c;
    const double peers = e->ep_world - 1;
    const double gather = peers * e->B * (c.D + 2.0 * c.TOPK) * 4;       // this GPU's records, to every peer
    if (e->ep_peer_ready) {
        // peer stores: only the rows of picks computed here for other ranks' tokens travel; counted on the device
        unsigned long long rows = 0;
        cudaMemcpy(&rows, e->d_ep_rows, sizeof(rows), cudaMemcpyDeviceToHost);
        return c.L * gather + (e->ep_steps > 0 ? (double)rows * c.D * 4 / e->ep_steps : 0.0);
    }
    const double back = peers * e->B * (c.TOPK + 1.0) * c.D * 4;         // pick outputs computed here, to their owners
    return c.L * (gather + back);
}

int b2_debug_trace_step(b2_engine* e, unsigned long long* out, int cap_launches, int* n_launches) {
    if (feed_checks(e, 1)) return 1;
    if (!e->d_trace && cudaMalloc(&e->d_trace, (size_t)TRACE_MAX_LAUNCHES * 128) != cudaSuccess) return e->fail("trace buffer: out of memory");
    std::vector<unsigned long long> init((size_t)TRACE_MAX_LAUNCHES * 16, 0ull);
    for (int i = 0; i < TRACE_MAX_LAUNCHES; i++) init[(size_t)16 * i] = ~0ull;
    cudaMemcpyAsync(e->d_trace, init.data(), init.size() * 8, cudaMemcpyHostToDevice, e->stream);
    cudaStreamSynchronize(e->stream);
    // the same step as the decode graph, captured once more with the time stamp slots handed out
    cudaGraph_t g;
    cudaGraphExec_t ge = nullptr;
    g_trace_base = e->d_trace;
    g_trace_first = g_launch_count;
    cudaError_t ce = cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal);
    int rc = ce == cudaSuccess ? e->enqueue_step(e->stream, false) : 1;
    const int n = g_launch_count - g_trace_first;
    g_trace_base = nullptr;
    cudaError_t ce2 = cudaStreamEndCapture(e->stream, &g);
    if (rc || ce != cudaSuccess || ce2 != cudaSuccess) return e->fail("trace step: capture failed");
    ce = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (ce != cudaSuccess) return e->fail("trace step: %s", cudaGetErrorString(ce));
    ce = cudaGraphLaunch(ge, e->stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
    cudaGraphExecDestroy(ge);
    if (ce != cudaSuccess) return e->fail("trace step: %s", cudaGetErrorString(ce));
    e->length += 1;
    e->toks_known = false;
    const int m = std::min(std::min(n, cap_launches), TRACE_MAX_LAUNCHES);
    cudaMemcpy(out, e->d_trace, (size_t)m * 128, cudaMemcpyDeviceToHost);
    *n_launches = m;
    return 0;
}

int b2_profile_step(b2_engine* e, int iters, float ms[8], double bytes[8], int launches[8]) {
    if (feed_checks(e, iters)) return 1;
    for (int i = 0; i < 8; i++) { ms[i] = 0; launches[i] = 0; }
    e->class_bytes(bytes);
    e->profiling = true;
    for (int it = 0; it < iters; it++) {
        e->prof_used = 0;
        if (e->enqueue_step(e->stream, false)) { e->profiling = false; return 1; }
        cudaMemcpyAsync(e->d_tok, e->d_next, (size_t)e->B * 4, cudaMemcpyDeviceToDevice, e->stream);
        cudaError_t ce = cudaStreamSynchronize(e->stream);
        if (ce != cudaSuccess) { e->profiling = false; return e->fail("profile step: %s", cudaGetErrorString(ce)); }
        e->length += 1;
        e->toks_known = false;
        for (size_t k = 1; k < e->prof_used; k++) {
            float t = 0;
            cudaEventElapsedTime(&t, e->prof_ev[k - 1], e->prof_ev[k]);
            ms[e->prof_class[k]] += t;
            launches[e->prof_class[k]] += 1;
        }
    }
    e->profiling = false;
    for (int i = 0; i < 8; i++) { ms[i] /= iters; launches[i] /= iters; }
    return 0;
}

}  // extern "C"

#include "ops.cuh"
#include "noalloc.cuh"
#include "sampler.hpp"
