// k_rowgemv: norm prologue + several weight matrices against the same activation rows, one weight
// row per LANE.
//
// A tile is 32 row slots of up to 2048 bytes (32 int8 rows; 16 bf16 rows of twice the bytes, two
// lanes per row; 16 gate rows + 16 up rows of a pair). It is brought into shared memory by one bulk
// copy per slot, each slot padded by 16 bytes so that the 32 lanes of a warp, reading the same column
// of 32 different slots, hit different banks. The 32 warps of the block split the columns: warp w
// takes the w-th 1/32 of every slot, so all 1024 threads work on one tile at a time. Within a warp
// every lane reads the SAME activations (a shared-memory broadcast), so activations need no
// registers, nothing is shuffled, and a weight, once widened, is used for all NB sequences of the
// pass. The 32 partial sums of a row meet in shared memory; one warp (a different one for every
// tile) adds them in warp order and runs the epilogue with one lane per row.
//
// Tiles are double- or triple-buffered; the block-wide barrier that ends a tile is also what frees its
// buffer, so warp 0 re-arms it right there. The first tiles are requested before grid_dep_wait().
#pragma once

namespace b2 {

constexpr int RL_WARPS = 32;
constexpr int RL_THREADS = RL_WARPS * 32;
constexpr int RL_SLOT_MAX = 2048;                       // bytes of weights per slot
constexpr int RL_SLOT_STRIDE = RL_SLOT_MAX + 16;        // padded
constexpr int RL_SLOT_STRIDE_BF = 2 * RL_SLOT_MAX + 16; // a bf16 row is twice the bytes; 16 of them per tile
constexpr int RL_STAGE_BYTES = 32 * RL_SLOT_STRIDE;     // 66,048

__device__ __host__ __forceinline__ bool rl_is_bf(int kind) { return kind == SEG_BF_SIGMOID || kind == SEG_BF_DECAY || kind == SEG_BF; }
// a row wider than one slot (bf16 rows; int8 rows of more than 2048 values) is shared by lanes l and l + 16
__device__ __host__ __forceinline__ bool rl_two_lanes(int kind, int K) { return rl_is_bf(kind) || K > RL_SLOT_MAX; }
// outputs per tile: 32 int8 rows, 16 wide rows, 16 gate/up pairs
__device__ __host__ __forceinline__ int rl_tile_rows(int kind, int K) {
    return (rl_two_lanes(kind, K) || kind == SEG_I8_GATEUP) ? 16 : 32;
}

template <int NB, int NST>
__global__ void __launch_bounds__(RL_THREADS, 1) k_rowgemv(const GemvArgs a, int nseq) {
    extern __shared__ __align__(128) unsigned char rl_smem[];
    unsigned char* stages = rl_smem;                                        // [NST][RL_STAGE_BYTES]
    float* xs = reinterpret_cast<float*>(rl_smem + (size_t)NST * RL_STAGE_BYTES);   // [NB][K]
    float* part = xs + (size_t)NB * a.K;                                    // [2][NB][RL_WARPS][32]
    __shared__ __align__(8) uint64_t full_bar[NST];
    __shared__ float red[RL_WARPS][NB];
    __shared__ int s_last;
    __shared__ float s_bv[RL_WARPS][NB];
    __shared__ int s_bi[RL_WARPS][NB];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b0 = blockIdx.y * NB;                    // first sequence of this pass
    const int t0 = (int)((long long)blockIdx.x * a.total_jobs / gridDim.x);
    const int t1 = (int)((long long)(blockIdx.x + 1) * a.total_jobs / gridDim.x);
    grid_dep_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) mbar_init(&full_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // tile -> (segment, first row); warp 0 asks for tile t into stage st, one bulk copy per slot
    auto locate = [&](int t, int& s, int& tin) {
        s = 0; tin = t;
        while (s + 1 < a.nseg && tin >= a.seg[s].jobs) { tin -= a.seg[s].jobs; s++; }
    };
    auto request = [&](int t, int st) {
        int s, tin;
        locate(t, s, tin);
        const Seg& sg = a.seg[s];
        const int tr = rl_tile_rows(sg.kind, a.K);
        const int row0 = tin * tr;
        const int n = min(tr, sg.rows - row0);
        const bool pair = sg.kind == SEG_I8_GATEUP;
        const uint32_t rb = rl_is_bf(sg.kind) ? 2u * a.K : (uint32_t)a.K;          // bytes per slot
        const int nslots = pair ? 2 * n : n;
        if (lane == 0) mbar_expect_tx(&full_bar[st], rb * nslots);
        __syncwarp();
        const int sstride = rl_two_lanes(sg.kind, a.K) ? RL_SLOT_STRIDE_BF : RL_SLOT_STRIDE;
        const bool active = pair ? (lane < n || (lane >= 16 && lane < 16 + n)) : lane < n;
        if (active) {
            const char* src = pair ? (lane < 16 ? (const char*)sg.w + (size_t)(row0 + lane) * a.K
                                                : (const char*)sg.w2 + (size_t)(row0 + lane - 16) * a.K)
                                   : (const char*)sg.w + (size_t)(row0 + lane) * rb;
            bulk_load(stages + (size_t)st * RL_STAGE_BYTES + (size_t)lane * sstride, src, rb, &full_bar[st]);
        }
    };
    if (warp == 0)
        for (int i = 0; i < NST && t0 + i < t1; i++) request(t0 + i, i);
    grid_dep_wait();

    // prologue: xs[b] = znorm(x[b]) (or x[b] itself), all 1024 threads; or, for the DeltaNet output
    // projection, w * rmsnorm_DV(o) * silu(z) per value head (aegist/hybrid.py:133-147), one head per warp
    if (a.gn_w) {
        const int nh = a.K / a.DV;
#pragma unroll
        for (int b = 0; b < NB; b++) {
            for (int h = warp; h < nh; h += RL_WARPS) {
                float ss = 0.f;
                const bool live = b0 + b < nseq;
                const float* in = a.x + (size_t)(b0 + b) * a.x_stride + h * a.DV;
                const float* z = a.z + (size_t)(b0 + b) * a.x_stride + h * a.DV;
                if (live) for (int i = lane; i < a.DV; i += 32) { const float v = in[i]; ss = fmaf(v, v, ss); }
                ss = warp_sum(ss);
                const float r = 1.0f / sqrtf(ss / (float)a.DV + a.eps);
                for (int i = lane; i < a.DV; i += 32)
                    xs[b * a.K + h * a.DV + i] = live ? (bf(a.gn_w[i]) * (in[i] * r)) * z[i] : 0.f;
            }
        }
        __syncthreads();
    } else {
        float ss[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            ss[b] = 0.f;
            if (b0 + b < nseq)
                for (int k = threadIdx.x; k < a.K; k += RL_THREADS) {
                    const float v = a.x[(size_t)(b0 + b) * a.x_stride + k];
                    xs[b * a.K + k] = v;
                    ss[b] = fmaf(v, v, ss[b]);
                }
            else
                for (int k = threadIdx.x; k < a.K; k += RL_THREADS) xs[b * a.K + k] = 0.f;
        }
        if (a.norm_w) {
#pragma unroll
            for (int b = 0; b < NB; b++) ss[b] = warp_sum(ss[b]);
            if (lane == 0)
#pragma unroll
                for (int b = 0; b < NB; b++) red[warp][b] = ss[b];
            __syncthreads();
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float t = 0.f;
                for (int w = 0; w < RL_WARPS; w++) t += red[w][b];
                const float r = 1.0f / sqrtf(t / (float)a.K + a.eps);
                for (int k = threadIdx.x; k < a.K; k += RL_THREADS) xs[b * a.K + k] = xs[b * a.K + k] * r * (1.0f + bf(a.norm_w[k]));
            }
        }
        __syncthreads();
    }

    float best_v[NB];
    int best_i[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) { best_v[b] = -INFINITY; best_i[b] = 0x7fffffff; }

    for (int t = t0, i = 0; t < t1; t++, i++) {
        const int st = i % NST;
        int s, tin;
        locate(t, s, tin);
        const Seg& sg = a.seg[s];
        const bool isbf = rl_is_bf(sg.kind);
        const bool two = rl_two_lanes(sg.kind, a.K);
        const int tr = rl_tile_rows(sg.kind, a.K);
        const int row0 = tin * tr;
        // this lane's slot and byte range: wide rows are shared by lanes l and l + 16 (half a row each)
        const int slot = two ? (lane & 15) : lane;
        const int rowbytes = isbf ? 2 * a.K : a.K;
        const int nch = (two ? rowbytes / 2 : rowbytes) >> 4;          // 16-byte chunks this lane could see
        const int cpw = (nch + RL_WARPS - 1) / RL_WARPS;
        const int c_lo = warp * cpw, c_hi = min(nch, c_lo + cpw);
        const int cbase = two ? (lane >> 4) * nch : 0;                 // second half of a wide row
        float* pt = part + (size_t)(i & 1) * NB * RL_WARPS * 32;
        mbar_wait(&full_bar[st], (i / NST) & 1, a.err);
        const unsigned char* src = stages + (size_t)st * RL_STAGE_BYTES + (size_t)slot * (two ? RL_SLOT_STRIDE_BF : RL_SLOT_STRIDE);
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.f;
        for (int c = c_lo; c < c_hi; c++) {
            const int4 wv = *reinterpret_cast<const int4*>(src + (size_t)(cbase + c) * 16);
            if (!isbf) {
                float wf[16];
                const int v[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t u = (uint32_t)v[q] ^ 0x80808080u;
                    wf[4 * q + 0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
                    wf[4 * q + 1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
                    wf[4 * q + 2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
                    wf[4 * q + 3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const float4* px = reinterpret_cast<const float4*>(xs + (size_t)b * a.K + 16 * (cbase + c));
                    float p0 = 0.f, p1 = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; q += 2) {
                        const float4 x0 = px[q], x1 = px[q + 1];
                        p0 = fmaf(x0.x, wf[4 * q + 0], p0); p0 = fmaf(x0.y, wf[4 * q + 1], p0);
                        p0 = fmaf(x0.z, wf[4 * q + 2], p0); p0 = fmaf(x0.w, wf[4 * q + 3], p0);
                        p1 = fmaf(x1.x, wf[4 * q + 4], p1); p1 = fmaf(x1.y, wf[4 * q + 5], p1);
                        p1 = fmaf(x1.z, wf[4 * q + 6], p1); p1 = fmaf(x1.w, wf[4 * q + 7], p1);
                    }
                    acc[b] += p0 + p1;
                }
            } else {
                const uint32_t v[4] = {(uint32_t)wv.x, (uint32_t)wv.y, (uint32_t)wv.z, (uint32_t)wv.w};
                const int k0 = 8 * (cbase + c);
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const float4* px = reinterpret_cast<const float4*>(xs + (size_t)b * a.K + k0);
                    const float4 x0 = px[0], x1 = px[1];
                    float p = x0.x * bflo(v[0]);
                    p = fmaf(x0.y, bfhi(v[0]), p); p = fmaf(x0.z, bflo(v[1]), p); p = fmaf(x0.w, bfhi(v[1]), p);
                    p = fmaf(x1.x, bflo(v[2]), p); p = fmaf(x1.y, bfhi(v[2]), p); p = fmaf(x1.z, bflo(v[3]), p);
                    p = fmaf(x1.w, bfhi(v[3]), p);
                    acc[b] += p;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) pt[((size_t)b * RL_WARPS + warp) * 32 + lane] = acc[b];
        __syncthreads();                       // partials complete; the stage is free
        if (warp == 0 && t + NST < t1) request(t + NST, st);
        if (warp == 1 + (i % (RL_WARPS - 1))) {
            // epilogue: lane j owns output row0 + j (16 outputs for bf16 rows and pairs, 32 for int8)
            const int row = row0 + lane;
            const bool mine = lane < tr && row < sg.rows;
            float e0 = 0.f, e1 = 0.f, e2 = 0.f, e3 = 0.f;
            uint2 ecw = make_uint2(0u, 0u);
            if (mine) {
                switch (sg.kind) {
                case SEG_I8: case SEG_I8_ARGMAX: case SEG_I8_SILU: case SEG_I8_CONV: case SEG_I8_ACC: e0 = bf(sg.s[row]); break;
                case SEG_I8_GATEUP: e0 = bf(sg.s[row]); e1 = bf(sg.s2[row]); break;
                case SEG_BF_DECAY: e0 = bf(a.a_log[row]); e1 = bf(a.dt_bias[row]); break;
                case SEG_BF: e0 = sg.bias ? sg.bias[row] : 0.f; break;
                default: break;
                }
                if (sg.kind == SEG_I8_CONV) ecw = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)row * 4);
            }
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (!mine || b0 + b >= nseq) continue;
                const float* pb = pt + (size_t)b * RL_WARPS * 32;
                float sA = 0.f, sB = 0.f;
                for (int w = 0; w < RL_WARPS; w++) { sA += pb[w * 32 + lane]; if (tr == 16) sB += pb[w * 32 + lane + 16]; }
                float* out = sg.out + (size_t)(b0 + b) * sg.out_stride;
                if (two && !isbf) { sA += sB; sB = 0.f; }          // the two halves of a wide int8 row
                switch (sg.kind) {
                case SEG_I8: out[row] = e0 * sA; break;
                case SEG_I8_ACC: out[row] += e0 * sA; break;
                case SEG_I8_SILU: out[row] = siluf_(e0 * sA); break;
                case SEG_I8_ARGMAX: {
                    const float v0 = e0 * sA;
                    out[row] = v0;
                    if (v0 > best_v[b] || (v0 == best_v[b] && row < best_i[b])) { best_v[b] = v0; best_i[b] = row; }
                } break;
                case SEG_I8_CONV: {
                    // hybrid.py:393-398: y = silu(sum_j w[c][j] * taps[j]), taps = 3 previous inputs + the new one
                    const float raw = e0 * sA;
                    float* stt = a.conv_state + ((size_t)(b0 + b) * sg.rows + row) * 3;
                    e1 = stt[0]; e2 = stt[1]; e3 = stt[2];
                    float y = bflo(ecw.x) * e1;
                    y = fmaf(bfhi(ecw.x), e2, y);
                    y = fmaf(bflo(ecw.y), e3, y);
                    y = fmaf(bfhi(ecw.y), raw, y);
                    stt[0] = e2; stt[1] = e3; stt[2] = raw;
                    out[row] = siluf_(y);
                } break;
                case SEG_BF_SIGMOID: out[row] = sigmoidf_(sA + sB); break;
                case SEG_BF_DECAY: out[row] = -expf(e0) * softplusf_((sA + sB) + e1); break;
                case SEG_BF: out[row] = (sA + sB) + e0; break;
                case SEG_I8_GATEUP: out[row] = siluf_(e0 * sA) * (e1 * sB); break;
                }
            }
        }
    }

    if (a.finisher == FIN_NONE) return;
    // finishers, one pass of NB sequences at a time
    if (a.finisher == FIN_ARGMAX) {
#pragma unroll
        for (int b = 0; b < NB; b++) {          // best over the lanes of a warp, then over the warps
            float v = best_v[b];
            int ix = best_i[b];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
                if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
            }
            if (lane == 0) { s_bv[warp][b] = v; s_bi[warp][b] = ix; }
        }
        __syncthreads();
        if (threadIdx.x < NB && b0 + threadIdx.x < nseq) {
            const int b = threadIdx.x;
            float v = s_bv[0][b];
            int ix = s_bi[0][b];
            for (int w = 1; w < RL_WARPS; w++)
                if (s_bv[w][b] > v || (s_bv[w][b] == v && s_bi[w][b] < ix)) { v = s_bv[w][b]; ix = s_bi[w][b]; }
            a.part_val[(size_t)(b0 + b) * gridDim.x + blockIdx.x] = v;
            a.part_idx[(size_t)(b0 + b) * gridDim.x + blockIdx.x] = ix;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int n = atomicAdd(a.counter + blockIdx.y, 1u);
        s_last = (n == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (warp < NB && b0 + warp < nseq) {
        const int b = b0 + warp;
        if (a.finisher == FIN_TOPK) {
            router_topk_warp(a.seg[0].out + (size_t)b * a.seg[0].out_stride, a.E, a.topk, a.top_idx + (size_t)b * a.topk,
                             a.top_w + (size_t)b * a.topk, lane);
            if (a.core.score) core_route_warp(a.core, b, lane);
        } else {
            float v = -INFINITY;
            int ix = 0x7fffffff;
            for (int g = lane; g < (int)gridDim.x; g += 32) {
                const float pv = __ldcg(a.part_val + (size_t)b * gridDim.x + g);
                const int pi = __ldcg(a.part_idx + (size_t)b * gridDim.x + g);
                if (pv > v || (pv == v && pi < ix)) { v = pv; ix = pi; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
                if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
            }
            if (lane == 0) {
                a.next_tok[b] = ix;
                if (a.pos) a.pos[b] += 1;
            }
        }
    }
    if (threadIdx.x == 0) a.counter[blockIdx.y] = 0;
}

}  // namespace b2
