// b2_moe_forward_static: the MoE layer operator for callers that must not allocate device memory.
//
// Some hosts cannot call cudaMalloc while they run the model: a serving process that has handed
// all of the GPU's free memory to its own arena at start-up (any later cudaMalloc fails or steals
// from the arena's headroom), a real-time loop where an allocation's implicit device
// synchronisation is not acceptable, or a plug-in that lives inside another runtime and is only
// given pointers. The ordinary operator (b2_moe_create / b2_moe_forward) allocates its work buffers
// when it is created. This variant allocates nothing: the caller passes device pointers for every
// weight, the input rows and the outputs, and the kernels' work memory (router logits, shared
// expert activations, expert activations, the per-pick down outputs that the last block sums, the
// block counters) lives in one file-scope device array that every GPU loading this library holds
// until the process exits.
//
// Consequences of the shared array, all documented in the header too:
//  * sizes are capped (B2_STATIC_MAX_* below); larger problems are refused with an error;
//  * the array keeps the previous call's contents, so the counters and the output rows that the
//    kernels add into are cleared at the start of every call;
//  * two calls that overlap on one GPU (two streams, two threads) use the same memory and race;
//  * the first call on a device looks the array's device address up (cudaGetSymbolAddress with that
//    device current); make that first call before any stream capture begins;
//  * every call ends by synchronising `stream` and reading the kernels' error word back, so it must
//    never be made on a stream that is being captured;
//  * every device pointer (h, y, idx, wts and the nine inside *w) must be non-null where required and
//    16-byte aligned: the kernels read them with 128-bit loads. A pointer that fails this is refused
//    with code 3 before anything is launched.
#pragma once

#define B2_STATIC_MAX_TOKENS 8
#define B2_STATIC_MAX_D 2048
#define B2_STATIC_MAX_E 256
#define B2_STATIC_MAX_TOPK 8
#define B2_STATIC_MAX_I 512
#define B2_STATIC_MAX_SH 512

namespace b2 {
// word offsets inside the array
constexpr size_t NA_RLOGITS = 0;
constexpr size_t NA_SHACT = NA_RLOGITS + (size_t)B2_STATIC_MAX_TOKENS * B2_STATIC_MAX_E;
constexpr size_t NA_SGATE = NA_SHACT + (size_t)B2_STATIC_MAX_TOKENS * B2_STATIC_MAX_SH;
constexpr size_t NA_ACT = NA_SGATE + 64;
constexpr size_t NA_YPART = NA_ACT + (size_t)B2_STATIC_MAX_TOKENS * B2_STATIC_MAX_TOPK * B2_STATIC_MAX_I;
constexpr size_t NA_TOPIDX = NA_YPART + (size_t)B2_STATIC_MAX_TOKENS * (B2_STATIC_MAX_TOPK + 1) * B2_STATIC_MAX_D;
constexpr size_t NA_TOPW = NA_TOPIDX + 64;
constexpr size_t NA_ZERO = NA_TOPW + 64;                      // everything from here on starts each call at zero
constexpr size_t NA_COUNTER = NA_ZERO;                        // [tokens] finisher counters of the router launch
constexpr size_t NA_DCOUNTER = NA_COUNTER + 64;               // [tokens][row blocks] of the down projection
constexpr size_t NA_ERR = NA_DCOUNTER + (size_t)B2_STATIC_MAX_TOKENS * (B2_STATIC_MAX_D / DOWN_ROWS);
constexpr size_t NA_WORDS = NA_ERR + 64;
}  // namespace b2

// 748 KB per GPU. In host code this name is only a stand-in for the symbol, never a device address:
// the address the kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_moe_static_scratch[b2::NA_WORDS];

namespace b2 {
constexpr int NA_MAX_DEVICES = 64;
static float* g_na_ptr[NA_MAX_DEVICES] = {nullptr};

// Once per device, with that device current: the device address of the array.
static int na_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return op_fail("cudaGetDevice", e);
    if (dev < 0 || dev >= NA_MAX_DEVICES) { fprintf(stderr, "b200moe: b2_moe_forward_static: device %d out of range\n", dev); return 3; }
    if (!g_na_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_moe_static_scratch);
        if (e != cudaSuccess) return op_fail("cudaGetSymbolAddress(g_moe_static_scratch)", e);
        g_na_ptr[dev] = (float*)p;
    }
    *out = g_na_ptr[dev];
    return 0;
}
}  // namespace b2

extern "C" int b2_moe_forward_static(const b2_moe_device_weights* w, const float* h, int tokens, float* y, int32_t* idx,
                                     float* wts, void* stream) {
    if (!w || !h || !y) { fprintf(stderr, "b200moe: b2_moe_forward_static: null argument\n"); return 3; }
    if (tokens < 1 || tokens > B2_STATIC_MAX_TOKENS || w->d_model > B2_STATIC_MAX_D || w->n_experts > B2_STATIC_MAX_E ||
        w->top_k > B2_STATIC_MAX_TOPK || w->expert_hidden > B2_STATIC_MAX_I || w->shared_hidden > B2_STATIC_MAX_SH) {
        fprintf(stderr, "b200moe: b2_moe_forward_static: %d tokens, d_model %d, %d experts top-%d, hidden %d, shared %d is beyond the "
                        "static work memory (at most %d tokens, %d, %d top-%d, %d, %d)\n",
                tokens, w->d_model, w->n_experts, w->top_k, w->expert_hidden, w->shared_hidden, B2_STATIC_MAX_TOKENS, B2_STATIC_MAX_D,
                B2_STATIC_MAX_E, B2_STATIC_MAX_TOPK, B2_STATIC_MAX_I, B2_STATIC_MAX_SH);
        return 2;
    }
    Cfg c;
    c.D = w->d_model; c.E = w->n_experts; c.TOPK = w->top_k; c.I = w->expert_hidden; c.SH = w->shared_hidden; c.G = 64;
    if (c.D % 64 || c.D < 64 || c.E < 1 || c.TOPK < 1 || c.TOPK > c.E || c.I % 64 || c.I < 64 || c.SH % 16 || c.SH < 16) {
        fprintf(stderr, "b200moe: b2_moe_forward_static: unsupported shape\n");
        return 3;
    }
    {
        // the kernels use 128-bit loads on all of these; a null or misaligned one must be an error code, not a fault
        const void* must[] = {h, y, w->router_bf16, w->expert_ptrs, w->sh_gate_q, w->sh_gate_s, w->sh_up_q, w->sh_up_s,
                              w->sh_down_q, w->sh_down_s, w->shared_gate_bf16};
        const char* names[] = {"h", "y", "router_bf16", "expert_ptrs", "sh_gate_q", "sh_gate_s", "sh_up_q", "sh_up_s",
                               "sh_down_q", "sh_down_s", "shared_gate_bf16"};
        for (int i = 0; i < 11; i++)
            if (!must[i] || ((uintptr_t)must[i] & 15)) {
                fprintf(stderr, "b200moe: b2_moe_forward_static: %s is %s\n", names[i], must[i] ? "not 16-byte aligned" : "null");
                return 3;
            }
        if (((uintptr_t)idx & 3) || ((uintptr_t)wts & 3)) { fprintf(stderr, "b200moe: b2_moe_forward_static: idx / wts misaligned\n"); return 3; }
    }
    float* s = nullptr;
    if (int rc = na_scratch(&s)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    int dev = 0, nsm = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev);
    // what the kernels count in or add into must start at zero; the rest is overwritten before it is read
    OPCU(cudaMemsetAsync(s + NA_ZERO, 0, (NA_WORDS - NA_ZERO) * sizeof(float), st));
    OPCU(cudaMemsetAsync(y, 0, (size_t)tokens * c.D * sizeof(float), st));
    int* top_idx = (int*)(s + NA_TOPIDX);
    float* top_w = s + NA_TOPW;
    GemvArgs a{};
    a.seg[0] = make_seg(SEG_BF, w->router_bf16, nullptr, c.E, s + NA_RLOGITS, c.E);
    a.seg[1] = make_seg(SEG_I8_GATEUP, w->sh_gate_q, w->sh_gate_s, c.SH, s + NA_SHACT, c.SH);
    a.seg[1].w2 = w->sh_up_q; a.seg[1].s2 = w->sh_up_s;
    a.seg[2] = make_seg(SEG_BF_SIGMOID, w->shared_gate_bf16, nullptr, 1, s + NA_SGATE, 1);
    a.nseg = 3; seal(a, c.D);
    a.x = h; a.norm_w = nullptr; a.K = c.D; a.err = (int*)(s + NA_ERR);
    a.finisher = FIN_TOPK; a.counter = (unsigned int*)(s + NA_COUNTER); a.E = c.E; a.topk = c.TOPK; a.top_idx = top_idx; a.top_w = top_w;
    OPCU(launch_gemv(a, tokens, nsm, st));
    ExpertArgs x{};
    x.eptr = w->expert_ptrs; x.top_idx = top_idx; x.top_w = top_w; x.topk = c.TOPK; x.E = c.E; x.D = c.D; x.I = c.I;
    x.idx_stride = c.TOPK; x.x_stride = c.D; x.combine = 1; x.local0 = 0; x.nlocal = tokens;
    x.off_gu_s = c.off_gu_s(); x.off_gu_m = c.off_gu_m(); x.off_dn_q = c.off_dn_q(); x.off_dn_s = c.off_dn_s(); x.off_dn_m = c.off_dn_m();
    x.x = h; x.norm_w = nullptr; x.act = s + NA_ACT; x.sh_act = s + NA_SHACT; x.sg = s + NA_SGATE;
    x.shd_w = w->sh_down_q; x.shd_s = w->sh_down_s; x.SH = c.SH; x.xout = y; x.err = (int*)(s + NA_ERR);
    x.null_is_error = 1; x.ypart = s + NA_YPART; x.counter = (unsigned int*)(s + NA_DCOUNTER);
    launch_experts(x, tokens, nsm, st);
    OPCU(cudaGetLastError());
    if (idx) OPCU(cudaMemcpyAsync(idx, top_idx, (size_t)tokens * c.TOPK * sizeof(int), cudaMemcpyDeviceToDevice, st));
    if (wts) OPCU(cudaMemcpyAsync(wts, top_w, (size_t)tokens * c.TOPK * sizeof(float), cudaMemcpyDeviceToDevice, st));
    // the error word the kernels set (a pick outside the table, a copy that never landed): 4 bytes into a local, no allocation
    int herr = 0;
    OPCU(cudaMemcpyAsync(&herr, s + NA_ERR, sizeof(int), cudaMemcpyDeviceToHost, st));
    OPCU(cudaStreamSynchronize(st));
    if (herr) {
        fprintf(stderr, "b200moe: b2_moe_forward_static: %s\n",
                herr == 3 ? "a bulk copy into shared memory did not complete (bounded wait gave up)"
                          : "the router picked an expert whose table entry is null or out of range");
        return 4;
    }
    return 0;
}
