// Single operators over host buffers (include/b200moe.h, last section): the same kernels the engine
// launches, wrapped so that one op can be checked against the reference's op on the same inputs.
#pragma once

namespace b2 {
struct OpErr { char msg[256]; };
static thread_local OpErr g_op_err;
static int op_fail(const char* what, cudaError_t e) {
    snprintf(g_op_err.msg, sizeof(g_op_err.msg), "%s: %s", what, cudaGetErrorString(e));
    fprintf(stderr, "b200moe: %s\n", g_op_err.msg);
    return 1;
}
#define OPCU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return op_fail(#call, e_); } while (0)

template <typename T>
static cudaError_t upload(T** dst, const T* src, size_t n) {
    cudaError_t e = cudaMalloc((void**)dst, std::max<size_t>(n * sizeof(T), 16));
    if (e != cudaSuccess) return e;
    return cudaMemcpy(*dst, src, n * sizeof(T), cudaMemcpyHostToDevice);
}
}  // namespace b2

struct b2_moe {
    int device, maxT, nsm;
    b2_moe_weights w;
    Cfg c;
    uint16_t *router = nullptr, *sg_s = nullptr, *su_s = nullptr, *sd_s = nullptr, *shared_gate = nullptr;
    uint8_t* experts = nullptr;
    int8_t *sg_q = nullptr, *su_q = nullptr, *sd_q = nullptr;
    const uint8_t** eptr = nullptr;
    float *h = nullptr, *y = nullptr, *rlogits = nullptr, *sh_act = nullptr, *sgate = nullptr, *act = nullptr, *top_w = nullptr;
    int *top_idx = nullptr, *err = nullptr;
    unsigned int* counter = nullptr;
    float* ypart = nullptr;
    unsigned int* dcounter = nullptr;
    // fewer than 8 tokens: the engine's small-batch expert kernels (k_moe_gu1 / k_moe_down1)
    const uint8_t** top_ptr = nullptr;
    int8_t* actq = nullptr;
    float *asc = nullptr, *asum = nullptr;
    int* h_err = nullptr;                    // page-locked copy of the device error word
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
};

// The device error word after an operator's kernels: 2 = a pick outside the expert table, 3 = a bulk copy that
// never landed (bounded wait gave up). Returns non-zero with a message when it is set, and clears it.
static int op_check_err(int* d_err, int* h_err, cudaStream_t st, const char* who) {
    OPCU(cudaMemcpyAsync(h_err, d_err, 4, cudaMemcpyDeviceToHost, st));
    OPCU(cudaStreamSynchronize(st));
    if (*h_err == 0) return 0;
    const int code = *h_err;
    cudaMemsetAsync(d_err, 0, 4, st);
    cudaStreamSynchronize(st);
    snprintf(g_op_err.msg, sizeof(g_op_err.msg), "%s: %s", who,
             code == 3 ? "a bulk copy into shared memory did not complete (bounded wait gave up)"
                       : "the router picked an expert that is not in the table");
    fprintf(stderr, "b200moe: %s\n", g_op_err.msg);
    return 4;
}

struct b2_delta {
    int device, B, H, dk, dv;
    float *state = nullptr, *y = nullptr, *g = nullptr, *beta = nullptr, *o = nullptr;
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    std::vector<float> pack;
};

extern "C" {

int b2_op_linear_i8(int device, const int8_t* q, const uint16_t* scale, int n, int k, const float* x, int tokens, float* y) {
    if (k % 16 != 0 || k > 4096 || n < 1 || tokens < 1) { snprintf(g_op_err.msg, sizeof(g_op_err.msg), "b2_op_linear_i8: k must be a multiple of 16 up to 4096"); return 1; }
    OPCU(cudaSetDevice(device));
    cudaDeviceProp prop;
    OPCU(cudaGetDeviceProperties(&prop, device));
    int8_t* dq = nullptr; uint16_t* ds = nullptr; float *dx = nullptr, *dy = nullptr;
    OPCU(upload(&dq, q, (size_t)n * k));
    OPCU(upload(&ds, scale, (size_t)n));
    OPCU(upload(&dx, x, (size_t)tokens * k));
    OPCU(cudaMalloc((void**)&dy, (size_t)tokens * n * 4));
    OPCU(cudaMemset(dy, 0, (size_t)tokens * n * 4));
    if (k <= 2048) {
        GemvArgs a{};
        a.seg[0] = make_seg(SEG_I8, dq, ds, n, dy, n);
        a.nseg = 1; seal(a, k);
        a.x = dx; a.norm_w = nullptr;
        launch_gemv(a, tokens, prop.multiProcessorCount, 0);
    } else {
        ProjArgs p{};
        p.in = dx; p.mode = 1; p.w = dq; p.s = ds; p.x = dy; p.N = n; p.K = k; p.DV = 32;
        launch_proj(p, tokens, prop.multiProcessorCount, 0);
    }
    OPCU(cudaGetLastError());
    OPCU(cudaMemcpy(y, dy, (size_t)tokens * n * 4, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(ds); cudaFree(dx); cudaFree(dy);
    return 0;
}

int b2_debug_wait_timeout(int device, int polls, int* status) {
    if (!status || polls < 1 || polls > (1 << 22)) return 1;
    OPCU(cudaSetDevice(device));
    int* d = nullptr;
    OPCU(dalloc(&d, 1));
    k_wait_never<<<1, 32>>>(polls, d);
    OPCU(cudaGetLastError());
    OPCU(cudaMemcpy(status, d, sizeof(int), cudaMemcpyDeviceToHost));
    cudaFree(d);
    return 0;
}

int b2_moe_create(int device, const b2_moe_weights* w, int max_tokens, b2_moe** out) {
    b2_moe* m = new b2_moe();
    *out = m;
    m->device = device; m->maxT = max_tokens; m->w = *w;
    Cfg& c = m->c;
    c.D = w->d_model; c.E = w->n_experts; c.TOPK = w->top_k; c.I = w->expert_hidden; c.SH = w->shared_hidden; c.G = w->group;
    if (c.D % 64 || c.D > 2048 || c.E > 256 || c.TOPK > 8 || c.G != 64 || c.I % 64 || c.I > 512 || c.SH % 16 || c.SH > 512) {
        snprintf(g_op_err.msg, sizeof(g_op_err.msg), "b2_moe_create: unsupported shape");
        return 1;
    }
    OPCU(cudaSetDevice(device));
    cudaDeviceProp prop;
    OPCU(cudaGetDeviceProperties(&prop, device));
    m->nsm = prop.multiProcessorCount;
    OPCU(upload(&m->router, w->router_bf16, (size_t)c.E * c.D));
    OPCU(upload(&m->experts, w->experts_q4, (size_t)c.E * c.expert_bytes()));
    OPCU(upload(&m->sg_q, w->sh_gate_q, (size_t)c.SH * c.D)); OPCU(upload(&m->sg_s, w->sh_gate_s, (size_t)c.SH));
    OPCU(upload(&m->su_q, w->sh_up_q, (size_t)c.SH * c.D)); OPCU(upload(&m->su_s, w->sh_up_s, (size_t)c.SH));
    OPCU(upload(&m->sd_q, w->sh_down_q, (size_t)c.D * c.SH)); OPCU(upload(&m->sd_s, w->sh_down_s, (size_t)c.D));
    OPCU(upload(&m->shared_gate, w->shared_gate_bf16, (size_t)c.D));
    std::vector<const uint8_t*> tab(c.E);
    for (int e = 0; e < c.E; e++) tab[e] = m->experts + (size_t)e * c.expert_bytes();
    OPCU(upload(&m->eptr, (const uint8_t* const*)tab.data(), (size_t)c.E));
    const int T = max_tokens;
    OPCU(dalloc(&m->h, (size_t)T * c.D)); OPCU(dalloc(&m->y, (size_t)T * c.D)); OPCU(dalloc(&m->rlogits, (size_t)T * c.E));
    OPCU(dalloc(&m->sh_act, (size_t)T * c.SH)); OPCU(dalloc(&m->sgate, T)); OPCU(dalloc(&m->act, (size_t)T * c.TOPK * c.I));
    OPCU(dalloc(&m->top_w, (size_t)T * c.TOPK)); OPCU(dalloc(&m->top_idx, (size_t)T * c.TOPK)); OPCU(dalloc(&m->err, 1));
    OPCU(dalloc(&m->counter, T));
    OPCU(dalloc(&m->ypart, (size_t)T * (c.TOPK + 1) * c.D));
    OPCU(dalloc(&m->dcounter, (size_t)T * down_row_blocks(c.D)));
    OPCU(dalloc(&m->top_ptr, (size_t)T * c.TOPK));
    OPCU(dalloc(&m->actq, (size_t)T * c.TOPK * M1_PLANES * c.I));
    OPCU(dalloc(&m->asc, (size_t)T * c.TOPK * std::max(1, c.I / 32))); OPCU(dalloc(&m->asum, (size_t)T * c.TOPK * std::max(1, c.I / 32)));
    OPCU(cudaMallocHost((void**)&m->h_err, sizeof(int)));
    OPCU(cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking));
    OPCU(cudaEventCreate(&m->e0)); OPCU(cudaEventCreate(&m->e1));
    return 0;
}

int b2_moe_forward(b2_moe* m, const float* h, int tokens, float* y, int32_t* idx, float* wts, float* device_ms) {
    if (!m || tokens < 1 || tokens > m->maxT) return 1;
    const Cfg& c = m->c;
    OPCU(cudaSetDevice(m->device));
    OPCU(cudaMemcpyAsync(m->h, h, (size_t)tokens * c.D * 4, cudaMemcpyHostToDevice, m->st));
    OPCU(cudaMemsetAsync(m->y, 0, (size_t)tokens * c.D * 4, m->st));
    OPCU(cudaEventRecord(m->e0, m->st));
    GemvArgs a{};
    a.seg[0] = make_seg(SEG_BF, m->router, nullptr, c.E, m->rlogits, c.E);
    a.seg[1] = make_seg(SEG_I8_GATEUP, m->sg_q, m->sg_s, c.SH, m->sh_act, c.SH);
    a.seg[1].w2 = m->su_q; a.seg[1].s2 = m->su_s;
    a.seg[2] = make_seg(SEG_BF_SIGMOID, m->shared_gate, nullptr, 1, m->sgate, 1);
    a.nseg = 3; seal(a, c.D);
    a.x = m->h; a.norm_w = nullptr; a.K = c.D; a.err = m->err;
    // the kernels the engine would run for this many tokens: below 8 the top-8 happens inside the expert kernel
    const bool moe1 = tokens < 8 && moe1_shape_ok(c);
    a.finisher = moe1 ? FIN_NONE : FIN_TOPK; a.counter = m->counter; a.E = c.E; a.topk = c.TOPK; a.top_idx = m->top_idx; a.top_w = m->top_w;
    launch_gemv(a, tokens, m->nsm, m->st);
    if (moe1) {
        const Moe1Ctx mc{m->top_ptr, m->actq, m->asc, m->asum};
        OPCU(launch_moe1(c, m->rlogits, m->h, nullptr, m->eptr, m->top_idx, m->top_w, mc, m->sh_act, m->sgate, m->sd_q, m->sd_s, m->y, m->err,
                         tokens, m->st, nullptr));
    } else {
    ExpertArgs x{};
    x.eptr = m->eptr; x.top_idx = m->top_idx; x.top_w = m->top_w; x.topk = c.TOPK; x.E = c.E; x.D = c.D; x.I = c.I;
    x.idx_stride = c.TOPK; x.x_stride = c.D; x.combine = 1; x.local0 = 0; x.nlocal = tokens;
    x.off_gu_s = c.off_gu_s(); x.off_gu_m = c.off_gu_m(); x.off_dn_q = c.off_dn_q(); x.off_dn_s = c.off_dn_s(); x.off_dn_m = c.off_dn_m();
    x.x = m->h; x.norm_w = nullptr; x.act = m->act; x.sh_act = m->sh_act; x.sg = m->sgate;
    x.shd_w = m->sd_q; x.shd_s = m->sd_s; x.SH = c.SH; x.xout = m->y; x.err = m->err;
    x.null_is_error = 1; x.ypart = m->ypart; x.counter = m->dcounter;
    launch_experts(x, tokens, m->nsm, m->st);
    }
    OPCU(cudaEventRecord(m->e1, m->st));
    OPCU(cudaGetLastError());
    OPCU(cudaMemcpyAsync(y, m->y, (size_t)tokens * c.D * 4, cudaMemcpyDeviceToHost, m->st));
    if (idx) OPCU(cudaMemcpyAsync(idx, m->top_idx, (size_t)tokens * c.TOPK * 4, cudaMemcpyDeviceToHost, m->st));
    if (wts) OPCU(cudaMemcpyAsync(wts, m->top_w, (size_t)tokens * c.TOPK * 4, cudaMemcpyDeviceToHost, m->st));
    if (int rc = op_check_err(m->err, m->h_err, m->st, "b2_moe_forward")) return rc;
    if (device_ms) OPCU(cudaEventElapsedTime(device_ms, m->e0, m->e1));
    return 0;
}

void b2_moe_destroy(b2_moe* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    void* bufs[] = {m->router, m->sg_s, m->su_s, m->sd_s, m->shared_gate, m->experts, m->sg_q, m->su_q, m->sd_q, (void*)m->eptr, m->h, m->y,
                    m->rlogits, m->sh_act, m->sgate, m->act, m->top_w, m->top_idx, m->err, m->counter, m->ypart, m->dcounter,
                    (void*)m->top_ptr, m->actq, m->asc, m->asum};
    for (void* p : bufs) cudaFree(p);
    if (m->h_err) cudaFreeHost(m->h_err);
    if (m->e0) cudaEventDestroy(m->e0);
    if (m->e1) cudaEventDestroy(m->e1);
    if (m->st) cudaStreamDestroy(m->st);
    delete m;
}

int b2_delta_create(int device, int batch, int heads, int dk, int dv, const float* state0, b2_delta** out) {
    b2_delta* d = new b2_delta();
    *out = d;
    d->device = device; d->B = batch; d->H = heads; d->dk = dk; d->dv = dv;
    if (!(dk == 64 || dk == 128) || dv % 32 != 0 || batch < 1 || heads < 1) {
        snprintf(g_op_err.msg, sizeof(g_op_err.msg), "b2_delta_create: dk must be 64 or 128 and dv a multiple of 32");
        return 1;
    }
    OPCU(cudaSetDevice(device));
    const size_t ns = (size_t)batch * heads * dk * dv;
    OPCU(dalloc(&d->state, ns));
    if (state0) OPCU(cudaMemcpy(d->state, state0, ns * 4, cudaMemcpyHostToDevice));
    const int C = heads * (2 * dk + dv);
    OPCU(dalloc(&d->y, (size_t)batch * C)); OPCU(dalloc(&d->g, (size_t)batch * heads)); OPCU(dalloc(&d->beta, (size_t)batch * heads));
    OPCU(dalloc(&d->o, (size_t)batch * heads * dv));
    d->pack.resize((size_t)batch * C);
    OPCU(cudaStreamCreateWithFlags(&d->st, cudaStreamNonBlocking));
    OPCU(cudaEventCreate(&d->e0)); OPCU(cudaEventCreate(&d->e1));
    return 0;
}

int b2_delta_step(b2_delta* d, const float* q, const float* k, const float* v, const float* g, const float* beta, float* out,
                  float* device_ms) {
    if (!d) return 1;
    OPCU(cudaSetDevice(d->device));
    const int B = d->B, H = d->H, dk = d->dk, dv = d->dv, C = H * (2 * dk + dv);
    for (int b = 0; b < B; b++) {   // the engine's row layout: q heads | k heads | v heads
        memcpy(&d->pack[(size_t)b * C], q + (size_t)b * H * dk, (size_t)H * dk * 4);
        memcpy(&d->pack[(size_t)b * C + H * dk], k + (size_t)b * H * dk, (size_t)H * dk * 4);
        memcpy(&d->pack[(size_t)b * C + 2 * H * dk], v + (size_t)b * H * dv, (size_t)H * dv * 4);
    }
    OPCU(cudaMemcpyAsync(d->y, d->pack.data(), (size_t)B * C * 4, cudaMemcpyHostToDevice, d->st));
    OPCU(cudaMemcpyAsync(d->g, g, (size_t)B * H * 4, cudaMemcpyHostToDevice, d->st));
    OPCU(cudaMemcpyAsync(d->beta, beta, (size_t)B * H * 4, cudaMemcpyHostToDevice, d->st));
    DeltaArgs a{};
    a.y = d->y; a.beta = d->beta; a.g = d->g; a.state = d->state; a.o = d->o; a.C = C; a.HK = H; a.HV = H; a.DV = dv; a.prenormed = 1;
    OPCU(cudaEventRecord(d->e0, d->st));
    launch_delta(a, dk, B, d->st);
    OPCU(cudaEventRecord(d->e1, d->st));
    OPCU(cudaGetLastError());
    OPCU(cudaMemcpyAsync(out, d->o, (size_t)B * H * dv * 4, cudaMemcpyDeviceToHost, d->st));
    OPCU(cudaStreamSynchronize(d->st));
    if (device_ms) OPCU(cudaEventElapsedTime(device_ms, d->e0, d->e1));
    return 0;
}

int b2_delta_state(b2_delta* d, float* state_out) {
    if (!d) return 1;
    OPCU(cudaSetDevice(d->device));
    OPCU(cudaMemcpy(state_out, d->state, (size_t)d->B * d->H * d->dk * d->dv * 4, cudaMemcpyDeviceToHost));
    return 0;
}

void b2_delta_destroy(b2_delta* d) {
    if (!d) return;
    cudaSetDevice(d->device);
    cudaFree(d->state); cudaFree(d->y); cudaFree(d->g); cudaFree(d->beta); cudaFree(d->o);
    if (d->e0) cudaEventDestroy(d->e0);
    if (d->e1) cudaEventDestroy(d->e1);
    if (d->st) cudaStreamDestroy(d->st);
    delete d;
}

}  // extern "C"
