// Decode-step kernels for the hybrid-MoE token loop, written for sm_100a.
//
// One decode step of one layer is six launches (the reference's CUDA engine uses 16-18,
// aegist_rs/src/hybrid.rs:787-993); which kernel fills a role depends on the number of sequences:
//
//   DeltaNet layer                                    attention layer
//   GEMV group    norm1 + in_qkv(+conv+SiLU) + in_z    GEMV group    norm1 + q, k, v
//                 + in_b(sigmoid) + in_a(decay)
//   k_delta_step  L2 norm + gated delta rule           k_attn(_mma)  q/k norm + RoPE + KV append +
//                                                      k_attn_merge  split-K attention, merge, gate
//   GEMV group    gated RMSNorm + out, += residual     GEMV group    o, += residual
//   -- then, for every layer --
//   GEMV group    norm2 + router logits + shared gate/up(+SiLU) + shared_gate (+ top-8)
//   expert gate/up, expert down + shared down, += residual
//
// A GEMV group is k_tcgemv (tcgemv.cuh; k_rowgemv, rowgemv.cuh, for shapes it does not take) up to 5
// sequences and k_prep_q + k_umma (ummagemm.cuh; k_prep_x + k_mma_i8, mmagemm.cuh, for shapes it does not take)
// from 6 on; the experts are k_moe_gu1 / k_moe_down1 (moe1.cuh) up to 5 sequences, the grouped GEMM
// (k_group_picks, mmaexperts.cuh + k_umma_q4, ummaq4.cuh; k_mma_q4 for shapes it does not take) from 6 tokens
// on, and k_expert_gu / k_expert_down (this file) wherever none of the faster kernels takes the shape.
//
// All arithmetic is fp32 with fp32 accumulation or exact integer products (the reference's kernels
// are fp32, aegist_rs/kernels/aegist.cu:1-6). Weights stream from HBM exactly once per step.
// Integer-to-float conversion instructions run at a sixteenth of the FMA rate on this part, so the
// CUDA-core kernels widen weights with byte permutes into the mantissa of a magic constant instead
// (q4 codes as 1 + code/16). Grids are sized in multiples of the SM count by the host.
//
// Cross-block steps (router top-8, arg-max over the vocabulary, summing the expert picks) are done
// by whichever block finishes last (a counter and a fence), never by waiting on another block.
//
// Every kernel is written for programmatic dependent launch: it first asks for its successor to be
// scheduled and starts loading its own first weights (which no kernel writes), and only then waits
// for its predecessor's results (grid_dep_wait). Launched without the attribute these are no-ops.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

constexpr int THREADS = 256;
constexpr int WARPS = 8;
constexpr int KV_PAGE = 64;   // tokens per KV-cache page

__device__ __forceinline__ float bf(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ float bflo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bfhi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint16_t f2bf(float f) {   // round to nearest even
    uint32_t u = __float_as_uint(f);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// Programmatic dependent launch: let the next kernel of the stream be scheduled now; and block until
// the previous kernel has completed and its writes are visible. Everything a kernel reads that an
// earlier kernel wrote, and everything it writes, comes after grid_dep_wait().
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Time stamps of a launch for the step timeline (debugging aid; trace is null in normal runs). Per launch
// 16 words: [0] first block in and [4] last block out (ns of the global timer, which is slow to read, so it is
// read only there), [5] kernel code, [6] a shape hint, [7] last block in, [8] block 0's SM cycle counter when it came in,
// [9] .. [15] the same counter at points 1 .. 7 of block 0 (1 past the dependency wait, 2 past the prologue,
// 3 past the main loop; the others as the kernel defines them).
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool trace_block0() { return (blockIdx.x | blockIdx.y | blockIdx.z) == 0; }
__device__ __forceinline__ void trace_in(unsigned long long* p, int code, int hint) {
    if (p && threadIdx.x == 0) {
        const unsigned long long t = gtime();
        atomicMin(p, t);
        atomicMax(p + 7, t);        // when the last block came in
        if (trace_block0()) { p[5] = (unsigned long long)code; p[6] = (unsigned long long)hint; p[8] = (unsigned long long)clock64(); }
    }
}
__device__ __forceinline__ void trace_pt(unsigned long long* p, int i) {
    if (p && threadIdx.x == 0 && trace_block0()) p[8 + i] = (unsigned long long)clock64();
}
__device__ __forceinline__ void trace_out(unsigned long long* p) {
    if (p && threadIdx.x == 0) atomicMax(p + 4, gtime());
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the 256 threads of a block, the same value in every thread; `red` holds 8 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < WARPS; i++) s += red[i];
    return s;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// Streaming 128-bit load of weights that are read once per step.
__device__ __forceinline__ int4 ldw(const void* p) { return __ldcs(reinterpret_cast<const int4*>(p)); }

// Four int8 -> fp32 without conversion instructions: flip the sign bit (q + 128 in 0..255), drop the
// byte into the low mantissa of 2^23 with a byte permute, subtract 2^23 + 128. Exact.
__device__ __forceinline__ float dot16_i8(const int4& w, const float* x) {
    float a[4];
    const int v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {       // four independent chains: a lone FMA chain is latency-bound
        const uint32_t u = (uint32_t)v[i] ^ 0x80808080u;
        a[i] = x[4 * i + 0] * (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f);
        a[i] = fmaf(x[4 * i + 1], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f, a[i]);
        a[i] = fmaf(x[4 * i + 2], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f, a[i]);
        a[i] = fmaf(x[4 * i + 3], __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f, a[i]);
    }
    return (a[0] + a[1]) + (a[2] + a[3]);
}
// 32 four-bit codes (even index in the low nibble) against 32 activations. Each code is placed in
// the top four mantissa bits of 1.0 (a shift and one logic op), giving f = 1 + code/16 exactly; the
// function returns sum f * x, and the caller recovers sum code * x = 16 * (result - sum x).
__device__ __forceinline__ float dot32_q4f(const int4& w, const float* x) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t v[4] = {(uint32_t)w.x, (uint32_t)w.y, (uint32_t)w.z, (uint32_t)w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int n = 0; n < 8; n++) {
            const int sh = 19 - 4 * n;
            const uint32_t t = sh >= 0 ? (v[i] << sh) : (v[i] >> (-sh));
            a[i] = fmaf(x[8 * i + n], __uint_as_float((t & 0x00780000u) | 0x3F800000u), a[i]);
        }
    }
    return (a[0] + a[1]) + (a[2] + a[3]);
}

// ------------------------------------------------------------------------------------------
// k_embed: x[b] = embed[token[b]] widened to fp32 (the reference looks rows up on the host,
// aegist_rs/src/hybrid.rs:743-758). A bad id sets *err and reads row 0.
__global__ void k_embed(const uint16_t* __restrict__ embed, const int* __restrict__ tok, float* __restrict__ x,
                        int D, int V, int* err) {
    const int b = blockIdx.x;
    grid_dep_launch();
    grid_dep_wait();
    int id = tok[b];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicExch(err, 1);
        id = 0;
    }
    const uint16_t* row = embed + (size_t)id * D;
    for (int k = threadIdx.x; k < D; k += blockDim.x) x[(size_t)b * D + k] = bf(row[k]);
}

// ------------------------------------------------------------------------------------------
// A GEMV group: norm prologue + several weight matrices against the same normalised vector.
enum SegKind : int {
    SEG_I8 = 0,        // int8 rows, out = scale * dot
    SEG_I8_CONV = 1,   // int8 rows, then the depthwise causal conv (kernel 4) + SiLU with its state
    SEG_BF_SIGMOID = 2,  // bf16 rows, out = sigmoid(dot)
    SEG_BF_DECAY = 3,  // bf16 rows, out = -exp(A_log) * softplus(dot + dt_bias)
    SEG_BF = 4,        // bf16 rows, out = dot (+ bias[row] if given)
    SEG_I8_GATEUP = 5, // two int8 matrices, out = silu(s1 * dot1) * (s2 * dot2)
    SEG_I8_ARGMAX = 6, // int8 rows, out = scale * dot, and the arg-max over all rows
    SEG_I8_SILU = 7,   // int8 rows, out = silu(scale * dot)
    SEG_I8_ACC = 8     // int8 rows, out += scale * dot (a projection back into the residual stream)
};
enum Finisher : int { FIN_NONE = 0, FIN_TOPK = 1, FIN_ARGMAX = 2 };

struct Seg {
    const void* w;
    const uint16_t* s;
    const void* w2;
    const uint16_t* s2;
    float* out;        // [B][out_stride]
    const float* bias; // SEG_BF only, may be null
    int rows;
    int kind;
    int out_stride;
    int jobs;          // filled by the host: tiles of 8 rows (int8 kinds) or 4 rows (bf16 rows, gate/up pairs)
    int tr;            // k_tcgemv: rows per tile chosen by the host (0 = as many as a stage holds)
};


// The core engine (CoreEngine.forward, aegist/model.py:214-224; the routing half of cores_apply,
// aegist_rs/kernels/aegist.cu:283-322): two score tables of n1 and n2 entries address n1 * n2 switchable cores. The k
// best of each table, the k1 * k2 sums of their pairs, the k best sums (ties to the earlier one), softmax over those.
// Every pick is tallied in counts[core] (Lm::core_counts); picks and weights are kept for the live cores' kernel.
struct CoreRoute {
    const float* score;      // [T][n1 + n2] the two tables' scores of every token (null: this brain has no core engine)
    int n1, n2, k;
    int* counts;             // [n1 * n2] of this layer
    int* sel;                // [T][k]
    float* selw;             // [T][k]
};
// one warp per token; n1 <= 128, n2 <= 128, k <= 8. Everything stays in registers (lane r holds the r-th pick of a
// table, lane c and c + 32 the candidates c): a local array here would give every kernel that calls this a stack frame.
__device__ __forceinline__ void core_route_warp(const CoreRoute& cr, int t, int lane) {
    const float* s = cr.score + (size_t)t * (cr.n1 + cr.n2);
    const int k0 = min(cr.k, cr.n1), k1 = min(cr.k, cr.n2);
    float pv0 = 0.f, pv1 = 0.f;
    int pi0 = 0, pi1 = 0;
#pragma unroll
    for (int tab = 0; tab < 2; tab++) {
        const int n = tab ? cr.n2 : cr.n1, kk = tab ? k1 : k0;
        const float* st = s + (tab ? cr.n1 : 0);
        float m0 = lane < n ? __ldcg(st + lane) : -INFINITY, m1 = lane + 32 < n ? __ldcg(st + lane + 32) : -INFINITY;
        float m2 = lane + 64 < n ? __ldcg(st + lane + 64) : -INFINITY, m3 = lane + 96 < n ? __ldcg(st + lane + 96) : -INFINITY;
        for (int r = 0; r < kk; r++) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            if (lane < n && m0 > bv) { bv = m0; bi = lane; }                     // '>' keeps the lower index
            if (lane + 32 < n && m1 > bv) { bv = m1; bi = lane + 32; }
            if (lane + 64 < n && m2 > bv) { bv = m2; bi = lane + 64; }
            if (lane + 96 < n && m3 > bv) { bv = m3; bi = lane + 96; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == r) { if (tab) { pv1 = bv; pi1 = bi; } else { pv0 = bv; pi0 = bi; } }
            if ((bi & 31) == lane) {
                const int j = bi >> 5;
                if (j == 0) m0 = -INFINITY; else if (j == 1) m1 = -INFINITY; else if (j == 2) m2 = -INFINITY; else m3 = -INFINITY;
            }
        }
    }
    // candidate c = a k1 + b: the first table's pick a outermost (as the reference lists them); at most 64 candidates
    const int nc = k0 * k1, k = min(cr.k, nc);
    float c0, c1;
    int core0, core1;
    {
        const int a0 = lane / k1, b0 = lane - a0 * k1, a1 = (lane + 32) / k1, b1 = (lane + 32) - a1 * k1;
        const float va0 = __shfl_sync(0xffffffffu, pv0, a0 & 31), vb0 = __shfl_sync(0xffffffffu, pv1, b0 & 31);
        const float va1 = __shfl_sync(0xffffffffu, pv0, a1 & 31), vb1 = __shfl_sync(0xffffffffu, pv1, b1 & 31);
        const int ia0 = __shfl_sync(0xffffffffu, pi0, a0 & 31), ib0 = __shfl_sync(0xffffffffu, pi1, b0 & 31);
        const int ia1 = __shfl_sync(0xffffffffu, pi0, a1 & 31), ib1 = __shfl_sync(0xffffffffu, pi1, b1 & 31);
        c0 = lane < nc ? va0 + vb0 : -INFINITY; core0 = ia0 * cr.n2 + ib0;
        c1 = lane + 32 < nc ? va1 + vb1 : -INFINITY; core1 = ia1 * cr.n2 + ib1;
    }
    float myv = 0.f;
    int mycore = 0;
    for (int j = 0; j < k; j++) {            // the j-th best sum goes to lane j; ties to the earlier candidate
        float bv = c0;
        int bc = lane;
        if (c1 > bv) { bv = c1; bc = lane + 32; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oc = __shfl_xor_sync(0xffffffffu, bc, o);
            if (ov > bv || (ov == bv && oc < bc)) { bv = ov; bc = oc; }
        }
        const int core = __shfl_sync(0xffffffffu, (bc >> 5) ? core1 : core0, bc & 31);
        if (lane == j) { myv = bv; mycore = core; }
        if (lane == (bc & 31)) { if (bc >> 5) c1 = -INFINITY; else c0 = -INFINITY; }
    }
    const float top = __shfl_sync(0xffffffffu, myv, 0);
    const float ex = lane < k ? expf(myv - top) : 0.f;
    float sum = 0.f;
    for (int j = 0; j < k; j++) sum += __shfl_sync(0xffffffffu, ex, j);        // summed in pick order, as one thread would
    if (lane < k) {
        cr.sel[(size_t)t * cr.k + lane] = mycore;
        cr.selw[(size_t)t * cr.k + lane] = ex / sum;
        atomicAdd(cr.counts + mycore, 1);
    }
}

constexpr int GEMV_MAX_SEG = 6;     // router + shared gate/up + shared gate + the core engine's two key tables

struct GemvArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    Seg seg[GEMV_MAX_SEG];
    int nseg;
    int total_jobs;
    int jq, jr;              // k_tcgemv: total_jobs = jq * grid + jr; block b starts at b * jq + min(b, jr)
    const float* x;          // [B][x_stride] residual stream
    int x_stride;            // row stride of x (the host sets K when it is left 0)
    const uint16_t* norm_w;  // [K]
    float eps;
    int K;
    // gated RMSNorm prologue instead of the ZNorm one (k_rowgemv only): x holds o, z holds silu(z)
    const uint16_t* gn_w;    // [DV] or null
    const float* z;          // [B][x_stride]
    int DV;
    // SEG_I8_CONV
    const uint16_t* conv_w;  // [C][4]
    float* conv_state;       // [B][C][3], oldest first
    // SEG_BF_DECAY
    const uint16_t* a_log;
    const uint16_t* dt_bias;
    // finishers
    int finisher;
    unsigned int* counter;   // [B], zero before the launch; the finisher puts it back to zero
    // FIN_TOPK
    int E, topk;
    int* top_idx;            // [B][topk]
    float* top_w;            // [B][topk]
    // FIN_ARGMAX
    float* part_val;         // [B][gridDim.x]
    int* part_idx;           // [B][gridDim.x]
    int* next_tok;           // [B]
    int* pos;                // [B] advanced by one by the finisher (may be null)
    int* err;                // set to 3 if a bulk copy never landed (bounded wait gave up)
    CoreRoute core;          // FIN_TOPK: the core engine's picks follow the router's (scores = two of the segments)
};

// Softmax over E router logits and the `topk` largest in descending order, ties to the lower
// index, weights renormalised over the picks (aegist/hybrid.py:641-645; hybrid.cu:317-360).
// One warp per token; E <= 256.
__device__ __forceinline__ void router_topk_warp(const float* __restrict__ logits, int E, int topk,
                                                 int* __restrict__ idx, float* __restrict__ wts, int lane) {
    float p[8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        p[i] = e < E ? __ldcg(logits + e) : -INFINITY;
        mx = fmaxf(mx, p[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = lane + 32 * i;
        p[i] = e < E ? expf(p[i] - mx) : 0.f;
        sum += p[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < 8; i++) p[i] = (lane + 32 * i) < E ? p[i] / sum : -1.f;
    float topv[8];
    int tope[8];
    float tsum = 0.f;
    for (int r = 0; r < topk; r++) {
        float bv = -1.f;
        int be = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; i++) {   // ascending expert id within the lane: '>' keeps the lower id
            if (p[i] > bv) { bv = p[i]; be = lane + 32 * i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        if ((be & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; i++) if (i == (be >> 5)) p[i] = -1.f;
        }
        if (r < 8) { topv[r] = bv; tope[r] = be; }
        tsum += bv;
    }
    if (lane == 0) {
        for (int r = 0; r < topk && r < 8; r++) {
            idx[r] = tope[r];
            wts[r] = topv[r] / tsum;
        }
    }
}

// ---- bulk asynchronous copies (TMA) into a shared-memory ring, tracked by mbarriers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Wait for a phase of an mbarrier of this block. The wait is bounded: if the phase has not completed
// after a very long time (a copy that never lands), *err is set and the caller goes on with whatever
// the buffer holds, so that the kernel always terminates.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int limit = 1 << 22) {
    for (int spin = 0; spin < limit; spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    if (err) atomicExch(err, 3);
    return false;
}
// One contiguous copy global -> shared; src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

}  // namespace b2
#include "rowgemv.cuh"
#include "mmagemm.cuh"
#include "mmaexperts.cuh"
#include "digits.cuh"
#include "tcgemv.cuh"
#include "moe1.cuh"
namespace b2 {

// ------------------------------------------------------------------------------------------
// k_delta_step: L2-normalise q and k, then one step of the gated delta rule on a [DK x 32] column
// slab of one value head's state (aegist/hybrid.py:314-324, 409-412):
//     S *= exp(g);  kv = S^T k;  delta = (v - kv) * beta;  S += k (x) delta;  o = S^T q
// Columns of S never interact, so a head is split over DV/32 blocks. State is [B][HV][DK][DV] fp32
// and crosses HBM once in each direction.
struct DeltaArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const float* y;      // [B][C] conv+SiLU output: q | k | v
    const float* beta;   // [B][HV]
    const float* g;      // [B][HV]
    float* state;        // [B][HV][DK][DV]
    float* o;            // [B][HV*DV] raw readout (the gated norm is applied by the out projection's prologue)
    int C, HK, HV, DV;
    int prenormed;       // 1: q and k come in already normalised and scaled (the bare delta-rule op)
};

template <int DK>
__global__ void __launch_bounds__(THREADS) k_delta_step(const DeltaArgs a) {
    constexpr int RPT = DK / WARPS;   // state rows per thread
    __shared__ float qs[DK], ks[DK];
    __shared__ float red[WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nslab = a.DV / 32;
    const int slab = blockIdx.x % nslab, h = blockIdx.x / nslab, b = blockIdx.y;
    const int hk = h / (a.HV / a.HK);
    const int key_dim = a.HK * DK;
    const int col = slab * 32 + lane;
    grid_dep_launch();
    trace_in(a.trace, 3, gridDim.x);
    grid_dep_wait();        // the state itself is written by this kernel's previous launch
    trace_pt(a.trace, 1);

    float* S = a.state + (((size_t)b * a.HV + h) * DK) * a.DV + col;
    float st[RPT];
#pragma unroll
    for (int r = 0; r < RPT; r++) st[r] = S[(size_t)(warp + WARPS * r) * a.DV];

    const float* yb = a.y + (size_t)b * a.C;
    if (warp < 2) {   // warp 0 normalises q, warp 1 normalises k
        const float* src = yb + (warp == 0 ? 0 : key_dim) + hk * DK;
        float* dst = warp == 0 ? qs : ks;
        float v[DK / 32];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 32; i++) { v[i] = src[lane + 32 * i]; ss = fmaf(v[i], v[i], ss); }
        ss = warp_sum(ss);
        float r = 1.0f;
        if (!a.prenormed) r = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
        for (int i = 0; i < DK / 32; i++) {
            float t = v[i] * r;
            if (warp == 0 && !a.prenormed) t *= (DK == 128 ? 0.08838834764831845f : (DK == 64 ? 0.125f : rsqrtf((float)DK)));
            dst[lane + 32 * i] = t;
        }
    }
    const float vj = yb[2 * key_dim + h * a.DV + col];
    const float beta = a.beta[(size_t)b * a.HV + h];
    const float decay = expf(a.g[(size_t)b * a.HV + h]);
    __syncthreads();

    float kv = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        st[r] *= decay;
        kv = fmaf(st[r], ks[warp + WARPS * r], kv);
    }
    red[warp][lane] = kv;
    __syncthreads();
    kv = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) kv += red[w][lane];
    const float delta = (vj - kv) * beta;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; r++) {
        st[r] = fmaf(ks[warp + WARPS * r], delta, st[r]);
        o = fmaf(st[r], qs[warp + WARPS * r], o);
        S[(size_t)(warp + WARPS * r) * a.DV] = st[r];
    }
    red[warp][lane] = o;
    __syncthreads();
    if (warp == 0) {
        o = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) o += red[w][lane];
        a.o[(size_t)b * a.HV * a.DV + h * a.DV + col] = o;
    }
    trace_out(a.trace);
}

// ------------------------------------------------------------------------------------------
// The mixer's output projection, accumulated into the residual stream (run as a GEMV group).
//   mode 0 (DeltaNet): input = w * rmsnorm_DV(o) * silu(z) per value head (aegist/hybrid.py:133-147);
//                      silu(z) arrives ready-made from the in_z rows' epilogue
//   mode 1 (attention): input is used as it is (already merged and gated by k_attn_merge)
// K up to 4096: two warps share a row, each holding its half of the input in registers. A value
// head (DV values) is DV/16 neighbouring lanes' slices, so its mean square is a short shuffle
// reduction.
struct ProjArgs {
    const float* in;      // [B][K]
    const float* z;       // [B][K]      mode 0: silu(z), applied by the kernel that produced z
    const uint16_t* gn_w; // [DV]        mode 0
    float eps;
    int DV;               // 32, 64, 128 or 256
    int mode;
    const int8_t* w;      // [N][K]
    const uint16_t* s;    // [N]
    float* x;             // [B][N] residual stream, += result
    int N, K;
};

// ------------------------------------------------------------------------------------------
// Experts. One expert's bytes (aegist/hybrid.py:472-480):
//   gu_q u8 [2I][D/2] | gu_s f16 [2I][D/64] | gu_m f16 [2I][D/64] | dn_q u8 [D][I/2] | dn_s | dn_m f16 [D][I/64]
// w = code * scale + min, so a row's dot is  sum_g ( s_g * sum(code * x) + m_g * sum(x) )  over its
// 64-value groups (the factorisation of hybrid.cu:405-406).
struct ExpertArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const uint8_t* const* eptr;   // [E] device address of each resident expert (null: not on this GPU)
    const int* top_idx;           // [tokens][idx_stride] the router's picks
    const float* top_w;           // [tokens][idx_stride]
    int idx_stride;               // top-k on one GPU; the exchange record width under expert parallelism
    int x_stride;                 // d_model on one GPU; the exchange record width under expert parallelism
    int combine;                  // 1: the last block adds the picks into xout; 0: a later kernel does (expert parallel)
    int local0, nlocal;           // tokens [local0, local0 + nlocal) are this GPU's own (they get the shared expert)
    int topk, E;
    int D, I;
    size_t off_gu_s, off_gu_m, off_dn_q, off_dn_s, off_dn_m;
    // gate/up
    const float* x;               // [tokens][x_stride] residual stream (normalised again here)
    const uint16_t* norm_w;
    float eps;
    float* act;                   // [B*topk][I]
    // down + shared down
    const float* sh_act;          // [B][SH]
    const float* sg;              // [B] sigmoid(shared_gate)
    const int8_t* shd_w;          // [D][SH]
    const uint16_t* shd_s;        // [D]
    int SH;
    float* ypart;                 // [B][topk + 1][D] per-pick down outputs (+ the shared expert's)
    unsigned int* counter;        // [B][row blocks]
    float* xout;                  // [B][D] residual stream, += result
    int* err;
    int null_is_error;            // 1: every expert must be in the table (one GPU); 0: a null entry is another rank's expert
};

// act[pick][i] = silu(gate_i . h) * (up_i . h), one warp per (gate, up) row pair.
// grid (blocks per pick, B * topk).
constexpr int GU_RPW = 2;       // (gate, up) row pairs per warp: the grid is sized so that this covers expert_hidden

template <int MAXC>   // 32-code slices per lane: D <= MAXC * 1024
__global__ void __launch_bounds__(THREADS, 2) k_expert_gu(const ExpertArgs a) {
    const int pick = blockIdx.y, b = pick / a.topk;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    grid_dep_launch();
    trace_in(a.trace, 5, gridDim.x);
    grid_dep_wait();              // which expert to read is the previous kernel's result
    trace_pt(a.trace, 1);
    const int e = a.top_idx[(size_t)b * a.idx_stride + pick % a.topk];
    const uint8_t* base = (e >= 0 && e < a.E) ? a.eptr[e] : nullptr;
    if (base == nullptr) {   // not resident here (another rank's expert) or a bad pick
        if (e < 0 || e >= a.E || a.null_is_error) { if (threadIdx.x == 0) atomicExch(a.err, 2); }
        return;
    }
    const int nchunk = a.D >> 5;          // 16-byte slices per row
    const int ngroup = a.D >> 6;
    const int gw = blockIdx.x * WARPS + warp, TW = gridDim.x * WARPS;

    const uint16_t* gs = (const uint16_t*)(base + a.off_gu_s);
    const uint16_t* gm = (const uint16_t*)(base + a.off_gu_m);
    // both (gate, up) row pairs of this warp are requested up front: one round trip to HBM
    int4 wg[GU_RPW][MAXC], wu[GU_RPW][MAXC];
    uint16_t sg_[GU_RPW][MAXC], mg_[GU_RPW][MAXC], su_[GU_RPW][MAXC], mu_[GU_RPW][MAXC];
#pragma unroll
    for (int u = 0; u < GU_RPW; u++) {
        const int i = gw + u * TW;
        const uint8_t* pg = base + (size_t)i * (a.D >> 1);
        const uint8_t* pu = base + (size_t)(a.I + i) * (a.D >> 1);
#pragma unroll
        for (int jj = 0; jj < MAXC; jj++) {
            const int c = lane + 32 * jj;
            if (i < a.I && c < nchunk) {
                wg[u][jj] = ldw(pg + (size_t)c * 16); wu[u][jj] = ldw(pu + (size_t)c * 16);
                const int g = c >> 1;
                sg_[u][jj] = gs[(size_t)i * ngroup + g]; mg_[u][jj] = gm[(size_t)i * ngroup + g];
                su_[u][jj] = gs[(size_t)(a.I + i) * ngroup + g]; mu_[u][jj] = gm[(size_t)(a.I + i) * ngroup + g];
            } else {
                wg[u][jj] = make_int4(0, 0, 0, 0); wu[u][jj] = make_int4(0, 0, 0, 0);
                sg_[u][jj] = mg_[u][jj] = su_[u][jj] = mu_[u][jj] = 0;
            }
        }
    }

    // this lane's 32-value slices of norm2(x): slice jj is values [32 * (lane + 32 jj), +32)
    float xr[MAXC][32];
    float xsum[MAXC];
    {
        const float* xg = a.x + (size_t)b * a.x_stride;
        float ss = 0.f;
#pragma unroll
        for (int jj = 0; jj < MAXC; jj++) {
            const int c = lane + 32 * jj;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < nchunk) t = reinterpret_cast<const float4*>(xg + 32 * c)[q];
                xr[jj][4 * q] = t.x; xr[jj][4 * q + 1] = t.y; xr[jj][4 * q + 2] = t.z; xr[jj][4 * q + 3] = t.w;
                ss = fmaf(t.x, t.x, ss); ss = fmaf(t.y, t.y, ss); ss = fmaf(t.z, t.z, ss); ss = fmaf(t.w, t.w, ss);
            }
        }
        float r = 1.0f;
        if (a.norm_w) {
            ss = warp_sum(ss);
            r = 1.0f / sqrtf(ss / (float)a.D + a.eps);
        }
#pragma unroll
        for (int jj = 0; jj < MAXC; jj++) {
            const int c = lane + 32 * jj;
            xsum[jj] = 0.f;
            if (a.norm_w && c < nchunk) {
                const uint4* pw = reinterpret_cast<const uint4*>(a.norm_w + 32 * c);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 t = pw[q];
                    const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                    for (int n = 0; n < 4; n++) {
                        xr[jj][8 * q + 2 * n] = xr[jj][8 * q + 2 * n] * r * (1.0f + bflo(u[n]));
                        xr[jj][8 * q + 2 * n + 1] = xr[jj][8 * q + 2 * n + 1] * r * (1.0f + bfhi(u[n]));
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 32; q++) xsum[jj] += xr[jj][q];
        }
    }
    float ag[GU_RPW], au[GU_RPW];
#pragma unroll
    for (int u = 0; u < GU_RPW; u++) {
        ag[u] = 0.f; au[u] = 0.f;
#pragma unroll
        for (int jj = 0; jj < MAXC; jj++) {
            // sum code * x = 16 * (sum f * x - sum x), f = 1 + code / 16
            const float fg = dot32_q4f(wg[u][jj], &xr[jj][0]);
            const float fu = dot32_q4f(wu[u][jj], &xr[jj][0]);
            ag[u] += h2f(sg_[u][jj]) * (16.0f * (fg - xsum[jj])) + h2f(mg_[u][jj]) * xsum[jj];
            au[u] += h2f(su_[u][jj]) * (16.0f * (fu - xsum[jj])) + h2f(mu_[u][jj]) * xsum[jj];
        }
    }
#pragma unroll
    for (int u = 0; u < GU_RPW; u++) { ag[u] = warp_sum(ag[u]); au[u] = warp_sum(au[u]); }
    if (lane == 0) {
#pragma unroll
        for (int u = 0; u < GU_RPW; u++) {
            const int i = gw + u * TW;
            if (i < a.I) a.act[(size_t)pick * a.I + i] = siluf_(ag[u]) * au[u];
        }
    }
    trace_out(a.trace);
}

// The down projections. grid (row blocks, topk + 1, B): blockIdx.y < topk computes one pick's
//   ypart[r][o] = down_r[o] . act_r        (4-bit rows, a half-warp per row, act_r in registers)
// and blockIdx.y == topk the shared expert's  ypart[topk][o] = scale[o] * (shared_down[o] . shared_act).
// The block that finishes a row block last adds, in rank order so that the result does not depend
// on scheduling,   x[o] += sum_r w_r * ypart[r][o] + sigmoid(shared_gate) * ypart[topk][o].
// Needs I <= 512 and SH <= 512.
constexpr int DOWN_ROWS = 64;     // output rows per block
__global__ void __launch_bounds__(THREADS, 2) k_expert_down(const ExpertArgs a) {
    const int rb = blockIdx.x, r = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = rb * DOWN_ROWS, row1 = min(a.D, row0 + DOWN_ROWS);
    __shared__ int s_last;
    grid_dep_launch();
    trace_in(a.trace, 6, gridDim.x);
    float* yp = a.ypart + ((size_t)b * (a.topk + 1) + r) * a.D;
    if (r == a.topk) {
        // shared expert: int8 rows of SH values, one warp per row; only for this GPU's own tokens
        if (b < a.local0 || b >= a.local0 + a.nlocal) return;
        const int shchunk = a.SH >> 4;
        constexpr int NIT = DOWN_ROWS / WARPS;        // rows per warp, all requested up front
        int4 w[NIT];
#pragma unroll
        for (int u = 0; u < NIT; u++) {
            const int o = row0 + warp + WARPS * u;
            w[u] = (o < row1 && lane < shchunk) ? ldw(a.shd_w + (size_t)o * a.SH + (size_t)lane * 16) : make_int4(0, 0, 0, 0);
        }
        grid_dep_wait();
        float shx[16];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (lane < shchunk) t = reinterpret_cast<const float4*>(a.sh_act + (size_t)(b - a.local0) * a.SH + 16 * lane)[q];
            shx[4 * q] = t.x; shx[4 * q + 1] = t.y; shx[4 * q + 2] = t.z; shx[4 * q + 3] = t.w;
        }
        float d[NIT];
#pragma unroll
        for (int u = 0; u < NIT; u++) d[u] = dot16_i8(w[u], shx);
#pragma unroll
        for (int u = 0; u < NIT; u++) d[u] = warp_sum(d[u]);
        if (lane == 0) {
#pragma unroll
            for (int u = 0; u < NIT; u++) {
                const int o = row0 + warp + WARPS * u;
                if (o < row1) yp[o] = bf(a.shd_s[o]) * d[u];
            }
        }
    } else {
        grid_dep_wait();
        const int e = a.top_idx[(size_t)b * a.idx_stride + r];
        const uint8_t* base = (e >= 0 && e < a.E) ? a.eptr[e] : nullptr;
        const int nchunk = a.I >> 5;                  // 32-code slices per row (<= 16)
        const int ngroup = a.I >> 6;
        const int hw = lane >> 4, hl = lane & 15;
        if (base != nullptr) {
            const uint8_t* q4 = base + a.off_dn_q;
            const uint16_t* ds = (const uint16_t*)(base + a.off_dn_s);
            const uint16_t* dm = (const uint16_t*)(base + a.off_dn_m);
            constexpr int NIT = DOWN_ROWS / (2 * WARPS);   // a warp covers two rows at a time; all of them requested up front
            int4 w[NIT];
            uint16_t sc[NIT], mn[NIT];
#pragma unroll
            for (int u = 0; u < NIT; u++) {
                const int o = row0 + 2 * warp + hw + 2 * WARPS * u;
                if (o < row1 && hl < nchunk) {
                    w[u] = ldw(q4 + (size_t)o * (a.I >> 1) + (size_t)hl * 16);
                    sc[u] = ds[(size_t)o * ngroup + (hl >> 1)];
                    mn[u] = dm[(size_t)o * ngroup + (hl >> 1)];
                } else { w[u] = make_int4(0, 0, 0, 0); sc[u] = 0; mn[u] = 0; }
            }
            float xv[32];
            float xsum = 0.f;
            const float* ar = a.act + ((size_t)b * a.topk + r) * a.I + 32 * hl;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (hl < nchunk) t = reinterpret_cast<const float4*>(ar)[q];
                xv[4 * q] = t.x; xv[4 * q + 1] = t.y; xv[4 * q + 2] = t.z; xv[4 * q + 3] = t.w;
                xsum += t.x + t.y + t.z + t.w;
            }
            float d[NIT];
#pragma unroll
            for (int u = 0; u < NIT; u++) {
                const float f = dot32_q4f(w[u], xv);
                d[u] = h2f(sc[u]) * (16.0f * (f - xsum)) + h2f(mn[u]) * xsum;
            }
#pragma unroll
            for (int u = 0; u < NIT; u++) {
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) d[u] += __shfl_xor_sync(0xffffffffu, d[u], off);
            }
            if (hl == 0) {
#pragma unroll
                for (int u = 0; u < NIT; u++) {
                    const int o = row0 + 2 * warp + hw + 2 * WARPS * u;
                    if (o < row1) yp[o] = d[u];
                }
            }
        } else {
            if (e < 0 || e >= a.E) { if (threadIdx.x == 0) atomicExch(a.err, 2); }
            if (a.combine)
                for (int o = row0 + threadIdx.x; o < row1; o += THREADS) yp[o] = 0.f;
            // under expert parallelism another GPU computes this pick; nothing is written here
        }
    }
    trace_pt(a.trace, 3);
    if (!a.combine) { trace_out(a.trace); return; }
    // last block of this (sequence, row block): weighted sum in rank order, into the residual stream
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int n = atomicAdd(a.counter + (size_t)b * gridDim.x + rb, 1u);
        s_last = (n == (unsigned int)a.topk);
    }
    __syncthreads();
    if (!s_last) { trace_out(a.trace); return; }
    __threadfence();
    for (int o = row0 + threadIdx.x; o < row1; o += THREADS) {
        const float* base = a.ypart + (size_t)b * (a.topk + 1) * a.D + o;
        float y = 0.f;
        for (int k = 0; k < a.topk; k++) y = fmaf(a.top_w[(size_t)b * a.idx_stride + k], __ldcg(base + (size_t)k * a.D), y);
        if (a.shd_w) y = fmaf(a.sg[b], __ldcg(base + (size_t)a.topk * a.D), y);
        a.xout[(size_t)b * a.D + o] += y;
    }
    if (threadIdx.x == 0) a.counter[(size_t)b * gridDim.x + rb] = 0;
    trace_out(a.trace);
}

// N consecutive cache values (bf16 or fp32) starting at a 4*N- or 2*N-byte aligned address -> fp32.
template <int N, bool F32>
__device__ __forceinline__ void load_kv(const void* base, size_t elem, float (&out)[N]) {
    if (F32) {
        const float* p = (const float*)base + elem;
        if (N % 4 == 0) {
#pragma unroll
            for (int q = 0; q < N / 4; q++) {
                const float4 t = reinterpret_cast<const float4*>(p)[q];
                out[4 * q] = t.x; out[4 * q + 1] = t.y; out[4 * q + 2] = t.z; out[4 * q + 3] = t.w;
            }
        } else {
            const float2 t = *reinterpret_cast<const float2*>(p);
            out[0] = t.x; out[1] = t.y;
        }
    } else {
        const uint16_t* p = (const uint16_t*)base + elem;
        if (N == 8) {
            const uint4 t = *reinterpret_cast<const uint4*>(p);
            out[0] = bflo(t.x); out[1] = bfhi(t.x); out[2] = bflo(t.y); out[3] = bfhi(t.y);
            out[4] = bflo(t.z); out[5] = bfhi(t.z); out[6] = bflo(t.w); out[7] = bfhi(t.w);
        } else if (N == 4) {
            const uint2 t = *reinterpret_cast<const uint2*>(p);
            out[0] = bflo(t.x); out[1] = bfhi(t.x); out[2] = bflo(t.y); out[3] = bfhi(t.y);
        } else {
            const uint32_t t = *reinterpret_cast<const uint32_t*>(p);
            out[0] = bflo(t); out[1] = bfhi(t);
        }
    }
}

// ------------------------------------------------------------------------------------------
// k_attn: gated GQA decode attention over the paged KV cache, split along the context.
// Each block takes one KV head of one sequence and one slice of the positions, for all the query
// heads of the group (so a key/value row is read once, not once per query head as in hybrid.cu:121-173).
// Prologue: per-head zero-centred RMSNorm of q and of the new k, partial RoPE (rotate-half on the
// first RD dims, aegist/hybrid.py:160-166, angles from a host-built table), and the block that owns
// the newest position appends k, v to the cache. Each warp walks its positions four at a time with
// all eight row loads in flight. A block leaves (acc, max, sum) per query head in scratch memory;
// k_attn_merge combines the slices and applies sigmoid(gate).
struct AttnArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const float* qraw;        // [B][H][2*HD]  (query | gate) per head
    const float* kraw;        // [B][KV][HD]
    const float* vraw;        // [B][KV][HD]
    const uint16_t* qn_w;     // [HD]
    const uint16_t* kn_w;     // [HD]
    const float* rope_cos;    // [cap][RD/2]
    const float* rope_sin;
    const int* pos;           // [B] position of the new token
    void* kpool;              // [pages][KV][KV_PAGE][HD] bf16 or fp32
    void* vpool;
    const int* page_table;    // [B][pages per sequence]
    int pages_per_seq;
    int pt_stride;            // page-table row stride per block set: pages_per_seq, or 0 when the block sets are the tokens
                              // of ONE sequence's prompt chunk (position pos[b] each, all on the same pages)
    int append_only;          // 1: write the new key and value rows into the cache and leave
    int H, KV, RD;
    float eps, scale;
    float* part;              // [B][KV][nsplit][G][HD + 2]  scratch
    float* out;               // [B][H*HD]
    int nsplit;
};

constexpr int ATT_PPW = 4;    // positions a warp loads at once

template <int HD, bool KVF32>
__global__ void __launch_bounds__(THREADS) k_attn(const AttnArgs a) {
    constexpr int DPL = HD / 32;              // dims per lane
    constexpr int MAXG = 8;
    const int G = a.H / a.KV;                 // query heads per KV head (<= 8)
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    grid_dep_launch();
    trace_in(a.trace, 7, gridDim.x);
    grid_dep_wait();
    trace_pt(a.trace, 1);
    const int pos = a.pos[b];
    const int L = pos + 1;
    int chunk = (L + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + WARPS * ATT_PPW - 1) / (WARPS * ATT_PPW) * (WARPS * ATT_PPW);
    const int p0 = split * chunk, p1 = min(L, p0 + chunk);
    const size_t pstride = HD + 2;
    float* part = a.part + (((size_t)b * a.KV + kvh) * a.nsplit + split) * G * pstride;
    if (p0 >= p1) {                           // an empty slice: say so and leave
        for (int g = threadIdx.x; g < G; g += THREADS) { part[g * pstride + HD] = -INFINITY; part[g * pstride + HD + 1] = 0.f; }
        return;
    }

    __shared__ float qs[MAXG][HD];
    __shared__ float knew[HD], vnew[HD];
    __shared__ float m_s[WARPS][MAXG], l_s[WARPS][MAXG];
    extern __shared__ float accs[];            // [WARPS][G][HD]

    // prologue: warps 0..G-1 prepare the query heads, the next one the new key and value
    const float* cs = a.rope_cos + (size_t)pos * (a.RD / 2);
    const float* sn = a.rope_sin + (size_t)pos * (a.RD / 2);
    for (int t = warp; t < G + 1; t += WARPS) {
        const bool isq = t < G;
        const float* src = isq ? a.qraw + ((size_t)b * a.H + kvh * G + t) * 2 * HD : a.kraw + ((size_t)b * a.KV + kvh) * HD;
        const uint16_t* nw = isq ? a.qn_w : a.kn_w;
        float* dst = isq ? qs[t] : knew;
        float v[DPL];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) { v[i] = src[lane + 32 * i]; ss = fmaf(v[i], v[i], ss); }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)HD + a.eps);
#pragma unroll
        for (int i = 0; i < DPL; i++) dst[lane + 32 * i] = v[i] * r * (1.0f + bf(nw[lane + 32 * i]));
        __syncwarp();
        const int hr = a.RD / 2;
        for (int j = lane; j < hr; j += 32) {     // pairs (j, j + RD/2)
            const float x0 = dst[j], x1 = dst[j + hr];
            const float c = cs[j], s = sn[j];
            dst[j] = x0 * c - x1 * s;
            dst[j + hr] = x1 * c + x0 * s;
        }
        if (!isq) {
            const float* vs = a.vraw + ((size_t)b * a.KV + kvh) * HD;
            __syncwarp();
            for (int i = lane; i < HD; i += 32) {
                float kx = dst[i], vx = vs[i];
                if (!KVF32) { kx = bf(f2bf(kx)); vx = bf(f2bf(vx)); }   // what a bf16 cache gives back
                knew[i] = kx;
                vnew[i] = vx;
            }
        }
    }
    __syncthreads();
    // the block that owns the newest position appends it
    if (pos >= p0 && pos < p1) {
        const int page = a.page_table[(size_t)b * a.pt_stride + pos / KV_PAGE];
        const size_t off = (((size_t)page * a.KV + kvh) * KV_PAGE + pos % KV_PAGE) * HD;
        for (int i = threadIdx.x; i < HD; i += THREADS) {
            if (KVF32) { ((float*)a.kpool)[off + i] = knew[i]; ((float*)a.vpool)[off + i] = vnew[i]; }
            else { ((uint16_t*)a.kpool)[off + i] = f2bf(knew[i]); ((uint16_t*)a.vpool)[off + i] = f2bf(vnew[i]); }
        }
    }
    if (a.append_only) return;

    // scores are kept in the base-2 domain: q carries 1/sqrt(HD) * log2(e), so p = 2^(s - m)
    float q[MAXG][DPL];
#pragma unroll
    for (int g = 0; g < MAXG; g++)
#pragma unroll
        for (int i = 0; i < DPL; i++) q[g][i] = g < G ? qs[g][lane * DPL + i] * (a.scale * 1.4426950408889634f) : 0.f;
    // running max and sum of head (lane >> 2), the same in the four lanes of a head; acc[g][i] in every lane
    float m_run = -INFINITY, l_run = 0.f;
    float acc[MAXG][DPL];
#pragma unroll
    for (int g = 0; g < MAXG; g++)
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[g][i] = 0.f;
    const int hg = lane >> 2, pu = lane & 3;
    // each lane owns DPL consecutive dims of a row: one 16-byte (bf16, HD 256) load per key.
    // Four positions at a time: 32 partial scores (8 heads x 4 positions) per lane are summed over the
    // lanes by a halving exchange (31 shuffles) that leaves score j in lane j; the softmax bookkeeping
    // is then one value per lane instead of 32 values in every lane.
    const int per_warp = chunk / WARPS;
    const int w0 = p0 + warp * per_warp, w1 = min(p1, w0 + per_warp);
    for (int pb = w0; pb < w1; pb += ATT_PPW) {
        float kk[ATT_PPW][DPL], vv[ATT_PPW][DPL];
#pragma unroll
        for (int u = 0; u < ATT_PPW; u++) {
            const int p = pb + u;
            if (p < w1 && p != pos) {
                const int page = a.page_table[(size_t)b * a.pt_stride + p / KV_PAGE];
                const size_t off = (((size_t)page * a.KV + kvh) * KV_PAGE + p % KV_PAGE) * HD + lane * DPL;
                load_kv<DPL, KVF32>(a.kpool, off, kk[u]);
                load_kv<DPL, KVF32>(a.vpool, off, vv[u]);
            } else {
#pragma unroll
                for (int i = 0; i < DPL; i++) {
                    kk[u][i] = p == pos ? knew[lane * DPL + i] : 0.f;
                    vv[u][i] = p == pos ? vnew[lane * DPL + i] : 0.f;
                }
            }
        }
        float sp[32];
#pragma unroll
        for (int g = 0; g < MAXG; g++)
#pragma unroll
            for (int u = 0; u < ATT_PPW; u++) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < DPL; i++) s = fmaf(q[g][i], kk[u][i], s);
                sp[g * 4 + u] = s;
            }
        // halving exchange: after the step with offset o a lane keeps the half of the values whose index
        // has the same bit o as its lane number
#pragma unroll
        for (int o = 16, n = 16; o > 0; o >>= 1, n >>= 1) {
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < n; i++) {
                const float send = up ? sp[i] : sp[i + n];
                const float keep = up ? sp[i + n] : sp[i];
                sp[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
        }
        const bool valid = hg < G && pb + pu < w1;
        const float s = valid ? sp[0] : -INFINITY;          // score of head hg, position pb + pu
        float mx = fmaxf(s, __shfl_xor_sync(0xffffffffu, s, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float corr = m_new == -INFINITY ? 1.0f : exp2f(m_run - m_new);
        const float pe = valid ? exp2f(s - m_new) : 0.f;
        float ps = pe + __shfl_xor_sync(0xffffffffu, pe, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * corr + ps;
        m_run = m_new;
#pragma unroll
        for (int g = 0; g < MAXG; g++) {
            if (g < G) {
                const float cg = __shfl_sync(0xffffffffu, corr, 4 * g);
#pragma unroll
                for (int i = 0; i < DPL; i++) acc[g][i] *= cg;
#pragma unroll
                for (int u = 0; u < ATT_PPW; u++) {
                    const float pg = __shfl_sync(0xffffffffu, pe, 4 * g + u);
#pragma unroll
                    for (int i = 0; i < DPL; i++) acc[g][i] = fmaf(pg, vv[u][i], acc[g][i]);
                }
            }
        }
    }
    // merge the 8 warps of this block
#pragma unroll
    for (int g = 0; g < MAXG; g++) {
        if (g < G) {
            const float mg = __shfl_sync(0xffffffffu, m_run, 4 * g);
            const float lg = __shfl_sync(0xffffffffu, l_run, 4 * g);
            if (lane == 0) { m_s[warp][g] = mg; l_s[warp][g] = lg; }
#pragma unroll
            for (int i = 0; i < DPL; i++) accs[((size_t)warp * G + g) * HD + lane * DPL + i] = acc[g][i];
        }
    }
    __syncthreads();
    for (int g = 0; g < G; g++) {
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; w++) mx = fmaxf(mx, m_s[w][g]);
        float cw[WARPS];
#pragma unroll
        for (int w = 0; w < WARPS; w++) cw[w] = m_s[w][g] == -INFINITY ? 0.f : exp2f(m_s[w][g] - mx);
        for (int d = threadIdx.x; d < HD; d += THREADS) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) s = fmaf(accs[((size_t)w * G + g) * HD + d], cw[w], s);
            part[g * pstride + d] = s;
        }
        if (threadIdx.x == 0) {
            float lsum = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; w++) lsum += l_s[w][g] * cw[w];
            part[g * pstride + HD] = mx;
            part[g * pstride + HD + 1] = lsum;
        }
    }
    trace_out(a.trace);
}

// out[b][head][d] = (sum_s acc_s[d] * 2^(m_s - m)) / (sum_s l_s * 2^(m_s - m)) * sigmoid(gate[d])
// (the slices keep their maxima in the base-2 domain).
// grid (H, B), one thread per dim (strided when HD > blockDim).
__global__ void __launch_bounds__(THREADS) k_attn_merge(const AttnArgs a, int HD) {
    const int head = blockIdx.x, b = blockIdx.y;
    const int G = a.H / a.KV, kvh = head / G, g = head % G;
    __shared__ float sc[64];
    __shared__ float s_inv;
    grid_dep_launch();
    trace_in(a.trace, 8, gridDim.x);
    grid_dep_wait();
    trace_pt(a.trace, 1);
    const size_t pstride = HD + 2;
    const float* pb = a.part + (((size_t)b * a.KV + kvh) * a.nsplit) * G * pstride + (size_t)g * pstride;
    const size_t sstride = (size_t)G * pstride;
    // everything is requested at once (one round trip): this thread's dim of every slice, the gate, and in warp 0
    // the slices' maxima and sums. A slice that was empty left its old (finite) sums in place; its weight is zero.
    const int d0 = threadIdx.x;
    float v[64];
#pragma unroll
    for (int s = 0; s < 64; s++) v[s] = (s < a.nsplit && d0 < HD) ? __ldcg(pb + s * sstride + d0) : 0.f;
    const float gate0 = d0 < HD ? a.qraw[((size_t)b * a.H + head) * 2 * HD + HD + d0] : 0.f;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float ms[2], ls[2];
        float mx = -INFINITY;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int s = lane + 32 * u;
            ms[u] = s < a.nsplit ? __ldcg(pb + s * sstride + HD) : -INFINITY;
            ls[u] = s < a.nsplit ? __ldcg(pb + s * sstride + HD + 1) : 0.f;
            mx = fmaxf(mx, ms[u]);
        }
        mx = warp_max(mx);
        float lsum = 0.f;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const float c = ms[u] == -INFINITY ? 0.f : exp2f(ms[u] - mx);
            sc[lane + 32 * u] = (lane + 32 * u < a.nsplit) ? c : 0.f;
            lsum += ls[u] * c;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) s_inv = 1.0f / lsum;
    }
    __syncthreads();
    if (d0 < HD) {
        float acc = 0.f;                         // slices in order
#pragma unroll
        for (int s = 0; s < 64; s++) acc = fmaf(sc[s] != 0.f ? v[s] : 0.f, sc[s], acc);
        a.out[(size_t)b * a.H * HD + head * HD + d0] = (acc * s_inv) * sigmoidf_(gate0);
    }
    for (int d = d0 + THREADS; d < HD; d += THREADS) {      // HD > 256 only
        float acc = 0.f;
        for (int s = 0; s < a.nsplit; s++)
            if (sc[s] != 0.f) acc = fmaf(__ldcg(pb + s * sstride + d), sc[s], acc);
        const float gate = a.qraw[((size_t)b * a.H + head) * 2 * HD + HD + d];
        a.out[(size_t)b * a.H * HD + head * HD + d] = (acc * s_inv) * sigmoidf_(gate);
    }
    trace_out(a.trace);
}

}  // namespace b2
#include "attnmma.cuh"
#include "ummagemm.cuh"
#include "ummaq4.cuh"
#include "prefill.cuh"
namespace b2 {

// ------------------------------------------------------------------------------------------
// Expert parallelism. Sequences are split over the GPUs (mixers, router, shared expert local), the
// experts of every layer too (expert e lives on GPU e / (E / world)). Per layer:
//   k_ep_pack     record[b] = x[b] | picks | weights            (this GPU's B sequences)
//   all-gather    records of all world * B sequences
//   k_expert_gu / k_expert_down on every sequence's picks that hit a local expert -> ypart[token][r]
//   all-to-all    block p of ypart (GPU p's sequences) goes to GPU p
//   k_ep_combine  x[b] += sum_r w_r * ypart_from_owner(e_r)[b][r] + shared, picks in rank order: the
//                 same sums in the same order as on one GPU, so the result is bit-identical.
struct EpArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const float* x;        // [B][D]
    const int* top_idx;    // [B][topk]
    const float* top_w;    // [B][topk]
    float* rec;            // [B][D + 2 * topk]
    const float* recv_y;   // [world][B][topk + 1][D]: block p came from GPU p
    const float* sg;       // [B]
    float* xout;           // [B][D]
    int D, topk, B, E, world, rank, has_shared;
};

__global__ void k_ep_pack(const EpArgs a) {
    const int b = blockIdx.x;
    grid_dep_launch();
    grid_dep_wait();
    const int rw = a.D + 2 * a.topk;
    float* r = a.rec + (size_t)b * rw;
    for (int k = threadIdx.x; k < a.D; k += blockDim.x) r[k] = a.x[(size_t)b * a.D + k];
    if (threadIdx.x < a.topk) {
        r[a.D + threadIdx.x] = __int_as_float(a.top_idx[b * a.topk + threadIdx.x]);
        r[a.D + a.topk + threadIdx.x] = a.top_w[b * a.topk + threadIdx.x];
    }
}

__global__ void k_ep_combine(const EpArgs a) {
    const int b = blockIdx.y;
    grid_dep_launch();
    trace_in(a.trace, 13, gridDim.x);
    grid_dep_wait();
    const int per = a.E / a.world;
    const size_t blk = (size_t)a.B * (a.topk + 1) * a.D;      // one GPU's block
    for (int o = blockIdx.x * blockDim.x + threadIdx.x; o < a.D; o += gridDim.x * blockDim.x) {
        float y = 0.f;
        for (int r = 0; r < a.topk; r++) {
            const int e = a.top_idx[b * a.topk + r];
            const int owner = min(max(e, 0), a.E - 1) / per;
            y = fmaf(a.top_w[b * a.topk + r], a.recv_y[owner * blk + ((size_t)b * (a.topk + 1) + r) * a.D + o], y);
        }
        if (a.has_shared) y = fmaf(a.sg[b], a.recv_y[a.rank * blk + ((size_t)b * (a.topk + 1) + a.topk) * a.D + o], y);
        a.xout[(size_t)b * a.D + o] += y;
    }
    trace_out(a.trace);
}

// The same exchange without a library call: every GPU maps every other GPU's exchange block (cudaIpc) and writes
// its records, and afterwards the outputs of the picks it computed, straight into their places there with plain
// peer stores. Every sending block then raises a flag of its own in each receiver's block (one system-scope fence by
// one thread after the block's barrier, then relaxed stores of the exchange's number: fences of all threads, or a
// last-block counter with three fences in a row, cost 15 us per launch). The receiver's one-block kernel polls its
// flags with acquire loads, for a bounded number of polls (then error 5 and on with whatever is there), and the
// kernels after it read the data. Only rows of picks whose expert lives on the sender travel (1 / world of the dense
// block on average). A block is written again only after its reader has answered (records -> outputs -> next
// layer's records), so one buffer does.
constexpr int EP_MAX_WORLD = 8;
constexpr int EP_MAX_BLOCKS = 64;                    // sending blocks per launch, each with its own flag
struct EpPeers {
    float* base[EP_MAX_WORLD];   // every rank's exchange block as this GPU addresses it (its own included)
    size_t rec_off, y_off;       // floats from the base: records [world * B][D + 2 topk], outputs [world][B][topk + 1][D]
    size_t flag_off;             // ints from the base: flags [2 kinds][EP_MAX_WORLD senders][EP_MAX_BLOCKS]
};
struct EpPushArgs {
    unsigned long long* trace;
    EpPeers peers;
    const float* x;              // [B][D]
    const int* top_idx;          // [B][topk]
    const float* top_w;
    const float* ypart;          // [world * B][topk + 1][D] (outputs kind)
    int D, topk, B, E, world, rank;
    const int* seq;              // [2] number of the last completed exchange of each kind
    unsigned long long* rows_sent;
    int* err;
};

// one thread of a block, after the block's stores and a barrier
__device__ __forceinline__ void ep_signal(const EpPushArgs& a, int kind) {
    __threadfence_system();
    const int v = a.seq[kind] + 1;
    for (int p = 0; p < a.world; p++) {
        if (p == a.rank) continue;
        int* f = reinterpret_cast<int*>(a.peers.base[p]) + a.peers.flag_off + (kind * EP_MAX_WORLD + a.rank) * EP_MAX_BLOCKS + blockIdx.x;
        asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(f), "r"(v) : "memory");
    }
}

// records: block b takes the local sequences b, b + gridDim.x, .. and writes each one's record into slot
// rank * B + sequence of every rank's block
__global__ void __launch_bounds__(256) k_ep_push_records(const EpPushArgs a) {
    grid_dep_launch();
    trace_in(a.trace, 18, gridDim.x);
    grid_dep_wait();
    const int rw = a.D + 2 * a.topk;
    for (int b = blockIdx.x; b < a.B; b += gridDim.x) {
        const size_t slot = (size_t)(a.rank * a.B + b) * rw;
        for (int k = threadIdx.x * 4; k < a.D; k += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(a.x + (size_t)b * a.D + k);
            for (int p = 0; p < a.world; p++) *reinterpret_cast<float4*>(a.peers.base[p] + a.peers.rec_off + slot + k) = v;
        }
        if ((int)threadIdx.x < a.topk) {
            const float fi = __int_as_float(a.top_idx[b * a.topk + threadIdx.x]), fw = a.top_w[b * a.topk + threadIdx.x];
            for (int p = 0; p < a.world; p++) {
                float* r = a.peers.base[p] + a.peers.rec_off + slot;
                r[a.D + threadIdx.x] = fi;
                r[a.D + a.topk + threadIdx.x] = fw;
            }
        }
    }
    __syncthreads();                                 // the block's stores happen before thread 0's fence (bar.sync, then a cumulative fence)
    if (threadIdx.x == 0) ep_signal(a, 0);
    trace_out(a.trace);
}

// outputs: a row per (token, rank of the pick) of all world * B tokens, then one per local sequence for the shared
// expert's slot; a row travels only if its expert lives here, to the rank that owns the token. Block b takes the rows
// b, b + gridDim.x, ..
__global__ void __launch_bounds__(256) k_ep_push_outputs(const EpPushArgs a) {
    grid_dep_launch();
    trace_in(a.trace, 19, gridDim.x);
    grid_dep_wait();
    const int T = a.world * a.B, rw = a.D + 2 * a.topk, per = a.E / a.world;
    const float* rec = a.peers.base[a.rank] + a.peers.rec_off;
    unsigned sent = 0;
    for (int row = blockIdx.x; row < T * a.topk + a.B; row += gridDim.x) {
        int t, r, owner;
        bool go;
        if (row < T * a.topk) {
            t = row / a.topk; r = row - t * a.topk;
            const int e = __float_as_int(rec[(size_t)t * rw + a.D + r]);
            go = min(max(e, 0), a.E - 1) / per == a.rank;
            owner = t / a.B;
        } else {
            t = a.rank * a.B + (row - T * a.topk); r = a.topk;         // the shared expert's output of a local sequence
            go = true;
            owner = a.rank;
        }
        if (!go) continue;
        const float* src = a.ypart + ((size_t)t * (a.topk + 1) + r) * a.D;
        float* dst = a.peers.base[owner] + a.peers.y_off + ((size_t)(a.rank * a.B + (t - owner * a.B)) * (a.topk + 1) + r) * a.D;
        for (int k = threadIdx.x * 4; k < a.D; k += blockDim.x * 4) *reinterpret_cast<float4*>(dst + k) = *reinterpret_cast<const float4*>(src + k);
        sent += owner != a.rank;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (sent) atomicAdd(a.rows_sent, (unsigned long long)sent);
        ep_signal(a, 1);
    }
    trace_out(a.trace);
}

// one block: thread (p, b) waits for block b of rank p's launch of this kind; then the exchange's number is kept
struct EpWaitArgs {
    unsigned long long* trace;
    int* flags;                  // this rank's [2][EP_MAX_WORLD][EP_MAX_BLOCKS]
    int* seq;                    // [2]
    int kind, world, rank, nblocks, polls;
    int* err;
};
__global__ void __launch_bounds__(EP_MAX_WORLD * EP_MAX_BLOCKS) k_ep_wait(const EpWaitArgs a) {
    trace_in(a.trace, 20, a.kind);
    grid_dep_wait();                                 // keeps the chain: what follows this kernel also follows what came before it
    trace_pt(a.trace, 1);
    const int want = a.seq[a.kind] + 1;
    const int p = threadIdx.x / EP_MAX_BLOCKS, b = threadIdx.x % EP_MAX_BLOCKS;
    const bool failed = a.err && *reinterpret_cast<volatile int*>(a.err) != 0;     // an earlier wait of this step gave up: do not wait again
    if (!failed && p < a.world && p != a.rank && b < a.nblocks) {
        const int* f = a.flags + (a.kind * EP_MAX_WORLD + p) * EP_MAX_BLOCKS + b;
        bool ok = false;
        for (int i = 0; i < a.polls && !ok; i++) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            ok = v - want >= 0;
        }
        if (!ok && a.err) atomicExch(a.err, 5);
    }
    __syncthreads();
    if (threadIdx.x == 0) { __threadfence_system(); a.seq[a.kind] = want; }
    trace_out(a.trace);
}

// ------------------------------------------------------------------------------------------
// Small helpers for the host: fill and copy.
// next_tok[b] = arg-max of logits[b][0..rows) (the first of equal maxima), pos[b] += 1: the greedy step of a batch
// whose head ran as a plain matrix product. One block per sequence.
__global__ void __launch_bounds__(1024) k_argmax_rows(const float* __restrict__ logits, int rows, int stride, int* __restrict__ next_tok,
                                                      int* __restrict__ pos) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    grid_dep_launch();
    grid_dep_wait();
    const float* row = logits + (size_t)b * stride;
    float v = -INFINITY;
    int ix = 0x7fffffff;
    for (int i = threadIdx.x; i < rows; i += 1024) {         // ascending i: '>' keeps the first
        const float t = row[i];
        if (t > v) { v = t; ix = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
        if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
    }
    if (lane == 0) { s_v[warp] = v; s_i[warp] = ix; }
    __syncthreads();
    if (warp == 0) {
        v = s_v[lane]; ix = s_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
            if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
        if (lane == 0) {
            next_tok[b] = ix;
            if (pos) pos[b] += 1;
        }
    }
}

// A wait that cannot succeed, for testing the bounded wait: the barrier expects bytes that no copy delivers, so
// mbar_wait gives up after `polls` polls, sets *err to 3 and the kernel ends normally.
__global__ void k_wait_never(int polls, int* err) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(&bar, 16);
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(&bar, 0, err, polls);
}

// The live switchable cores of one layer (SparseCoreBank.forward, aegist/hybrid.py:745-771; the second half of
// cores_apply, aegist_rs/kernels/aegist.cu:323-349): for every pick whose core is stored, w * down^T (silu(h gate) * (h up))
// with h = norm2(x), summed into y[t] (which k_add_rows later adds to the residual stream). grid (T), 256 threads,
// dynamic shared memory D + r floats. Launched only for layers that have live cores.
struct CoresLiveArgs {
    const float* x;           // [T][D] residual rows before the experts wrote them
    const uint16_t* norm_w;   // [D]
    float eps;
    const int* live;          // [n cores] index into the bank, or -1
    const uint16_t *cg, *cu, *cd;   // bank: gate [n][D][r], up [n][D][r], down [n][r][D] bf16
    const int* sel;           // [T][k]
    const float* selw;        // [T][k]
    float* y;                 // [T][D]
    int D, r, k;
};
__global__ void __launch_bounds__(256) k_cores_live(const CoresLiveArgs a) {
    extern __shared__ float cl_smem[];
    float* h = cl_smem;              // [D]
    float* z = cl_smem + a.D;        // [r]
    __shared__ float red[8];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    grid_dep_launch();
    grid_dep_wait();
    const float* xr = a.x + (size_t)t * a.D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.D; i += 256) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float rn = 1.0f / sqrtf(ss / (float)a.D + a.eps);
    for (int i = threadIdx.x; i < a.D; i += 256) h[i] = xr[i] * rn * (1.0f + bf(a.norm_w[i]));
    float acc[8];                    // this thread's output dims i = threadIdx.x + 256 j (D <= 2048)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    __syncthreads();
    for (int c = 0; c < a.k; c++) {
        const int li = a.live[a.sel[(size_t)t * a.k + c]];
        if (li < 0) continue;        // the same for the whole block
        const uint16_t* G = a.cg + (size_t)li * a.D * a.r;
        const uint16_t* U = a.cu + (size_t)li * a.D * a.r;
        const uint16_t* Dn = a.cd + (size_t)li * a.r * a.D;
        for (int j = warp; j < a.r; j += 8) {
            float g = 0.f, u = 0.f;
            for (int i = lane; i < a.D; i += 32) {
                g = fmaf(h[i], bf(G[(size_t)i * a.r + j]), g);
                u = fmaf(h[i], bf(U[(size_t)i * a.r + j]), u);
            }
            g = warp_sum(g);
            u = warp_sum(u);
            if (lane == 0) z[j] = siluf_(g) * u;
        }
        __syncthreads();
        const float wc = a.selw[(size_t)t * a.k + c];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int i = threadIdx.x + 256 * j;
            if (i >= a.D) break;
            float s = 0.f;
            for (int q = 0; q < a.r; q++) s = fmaf(z[q], bf(Dn[(size_t)q * a.D + i]), s);
            acc[j] = fmaf(wc, s, acc[j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int i = threadIdx.x + 256 * j;
        if (i < a.D) a.y[(size_t)t * a.D + i] = acc[j];
    }
}
// x[t][i] += y[t][i]
__global__ void k_add_rows(float* x, const float* y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    grid_dep_launch();
    grid_dep_wait();
    if (i < n) x[i] += y[i];
}

__global__ void k_fill_i32(int* p, int v, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
__global__ void k_add_i32(int* p, int v, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] += v;
}

}  // namespace b2
