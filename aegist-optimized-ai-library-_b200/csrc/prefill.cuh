// Prompt chunks: what differs from a decode step when T tokens of ONE sequence are fed at once
// (HybridEngine::forward_chunk, aegist_rs/src/hybrid.rs:1023-1025; the multi-token loops of delta_scan,
// aegist_rs/kernels/hybrid.cu:240-300, and conv_silu, :205-221).
//
// The linears and the experts of a chunk are the batched-decode kernels with the chunk's tokens as the columns
// (the tcgen05 GEMM, the grouped 4-bit GEMM). What is sequential in the tokens runs here:
//   k_conv_scan    the depthwise causal conv (kernel 4) + SiLU over the chunk, one thread per channel, taps carried
//   k_delta_scan   the gated delta rule over the chunk, state slab in registers: the state crosses HBM once per chunk
// Attention over a chunk is the decode attention kernel with one block set per token: all tokens share the sequence's
// pages, token t sits at position pos0 + t and sees the positions up to its own; the chunk's keys and values are
// appended first by a launch of the same kernel in append-only mode, so every token finds the earlier ones in the cache.
#pragma once

namespace b2 {

struct ConvScanArgs {
    float* y;                 // [T][C] raw in_qkv rows in, silu(conv) out
    const uint16_t* conv_w;   // [C][4] bf16
    float* conv_state;        // [C][3] oldest first
    int C, T;
};

// aegist/hybrid.py:393-398: y = silu(sum_j w[c][j] * taps[j]), taps = the 3 previous inputs and the new one
__global__ void __launch_bounds__(256) k_conv_scan(const ConvScanArgs a) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    grid_dep_launch();
    grid_dep_wait();
    if (c >= a.C) return;
    const uint2 cw = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)c * 4);
    const float w0 = bflo(cw.x), w1 = bfhi(cw.x), w2 = bflo(cw.y), w3 = bfhi(cw.y);
    float* stt = a.conv_state + (size_t)c * 3;
    float s0 = stt[0], s1 = stt[1], s2 = stt[2];
    for (int t = 0; t < a.T; t++) {
        float* p = a.y + (size_t)t * a.C + c;
        const float raw = *p;
        float y = w0 * s0;
        y = fmaf(w1, s1, y);
        y = fmaf(w2, s2, y);
        y = fmaf(w3, raw, y);
        *p = siluf_(y);
        s0 = s1; s1 = s2; s2 = raw;
    }
    stt[0] = s0; stt[1] = s1; stt[2] = s2;
}

struct DeltaScanArgs {
    const float* y;      // [T][C] conv + SiLU output: q | k | v
    const float* beta;   // [T][HV]
    const float* g;      // [T][HV]
    float* state;        // [HV][DK][DV] of the sequence
    float* o;            // [T][HV * DV] raw readout
    int C, HK, HV, DV, T;
};

// k_delta_step's arithmetic (aegist/hybrid.py:314-324, 409-412) for T consecutive tokens on a [DK x 32] column slab of
// one value head's state: S *= exp(g); kv = S^T k; delta = (v - kv) beta; S += k (x) delta; o = S^T q, token after token.
// grid (HV * DV / 32); 256 threads: warp w holds state rows w, w + 8, ..., lane = column.
template <int DK>
__global__ void __launch_bounds__(THREADS) k_delta_scan(const DeltaScanArgs a) {
    constexpr int RPT = DK / WARPS;
    __shared__ float qs[DK], ks[DK];
    __shared__ float red[2][WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nslab = a.DV / 32;
    const int slab = blockIdx.x % nslab, h = blockIdx.x / nslab;
    const int hk = h / (a.HV / a.HK);
    const int key_dim = a.HK * DK;
    const int col = slab * 32 + lane;
    grid_dep_launch();
    grid_dep_wait();
    float* S = a.state + ((size_t)h * DK) * a.DV + col;
    float st[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) st[r] = S[(size_t)(warp + WARPS * r) * a.DV];
    for (int t = 0; t < a.T; t++) {
        const float* yb = a.y + (size_t)t * a.C;
        if (warp < 2) {   // warp 0 normalises q, warp 1 normalises k
            const float* src = yb + (warp == 0 ? 0 : key_dim) + hk * DK;
            float* dst = warp == 0 ? qs : ks;
            float v[DK / 32];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < DK / 32; i++) { v[i] = src[lane + 32 * i]; ss = fmaf(v[i], v[i], ss); }
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
            for (int i = 0; i < DK / 32; i++) {
                float x = v[i] * r;
                if (warp == 0) x *= (DK == 128 ? 0.08838834764831845f : (DK == 64 ? 0.125f : rsqrtf((float)DK)));
                dst[lane + 32 * i] = x;
            }
        }
        const float vj = yb[2 * key_dim + h * a.DV + col];
        const float beta = a.beta[(size_t)t * a.HV + h];
        const float decay = expf(a.g[(size_t)t * a.HV + h]);
        __syncthreads();
        float kv = 0.f;
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            st[r] *= decay;
            kv = fmaf(st[r], ks[warp + WARPS * r], kv);
        }
        red[0][warp][lane] = kv;
        __syncthreads();
        kv = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) kv += red[0][w][lane];
        const float delta = (vj - kv) * beta;
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < RPT; r++) {
            st[r] = fmaf(ks[warp + WARPS * r], delta, st[r]);
            o = fmaf(st[r], qs[warp + WARPS * r], o);
        }
        red[1][warp][lane] = o;
        __syncthreads();                   // also: qs / ks may be rewritten for the next token
        if (warp == 0) {
            o = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) o += red[1][w][lane];
            a.o[(size_t)t * a.HV * a.DV + h * a.DV + col] = o;
        }
    }
#pragma unroll
    for (int r = 0; r < RPT; r++) S[(size_t)(warp + WARPS * r) * a.DV] = st[r];
}

// p[i] = base[0] + i: the positions of a chunk's tokens
__global__ void k_iota_from(int* p, const int* base, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dep_launch();
    grid_dep_wait();
    if (i < n) p[i] = base[0] + i;
}

}  // namespace b2
