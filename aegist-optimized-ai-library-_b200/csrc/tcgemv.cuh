// k_tcgemv: the decode GEMV (norm prologue + several weight matrices against the same activation
// rows) with the multiply-adds of the int8 matrices on the tensor cores.
//
// A GEMV streams every weight once, so what limits it besides HBM is the instruction stream that turns
// bytes into products: about 3.3 instructions per int8 weight when each product is an FMA. Here the
// int8 weights go to mma.sync.m16n8k32.s8 exactly as they lie in memory (a warp reads 16 bytes of two
// rows and issues two instructions for 1024 products per sequence), and the activations are split once
// per launch into four int8 digit planes (digits.cuh) that occupy four of the eight B columns per
// sequence, so up to two sequences share a pass. The integer sums are exact.
//
// The tile, its bulk copies and the segment bookkeeping are those of k_rowgemv: 32 row slots of up to
// 2048 bytes (16 slots for rows of up to 4096 bytes: bf16 rows, int8 rows of 4096 values), one bulk
// copy per slot, slots padded by 64 bytes so that the fragment loads of rows r and r + 1 fall into
// different halves of the banks. The W compute warps of a block split a tile into (16-row block, K
// slice) parts and leave their partial sums in shared memory. Two more warps take the tiles in turn:
// they fetch the epilogue operands (scales, convolution taps and state) while the tile is being
// multiplied, wait on a named barrier for its partial sums, re-arm the freed stage with the next bulk
// copies, add the partial sums in slice order and run the epilogue with one lane per row slot, so the
// global-memory round trips of the epilogue are off the compute warps' path. bf16 rows (router,
// DeltaNet a/b projections) keep fp32 FMAs on fp32 activations with the same thread-to-byte mapping.
// The rows of a tile (at most 32, or 16 wide ones) are chosen per launch so that the tiles divide
// evenly among the blocks.
#pragma once

namespace b2 {

constexpr int TC_PAD = 64;
constexpr int TC_SLOT_STRIDE = RL_SLOT_MAX + TC_PAD;              // 2112
constexpr int TC_SLOT_STRIDE_WIDE = 2 * RL_SLOT_MAX + TC_PAD;     // 4160
constexpr int TC_STAGE_BYTES = 32 * TC_SLOT_STRIDE;               // 67,584 (>= 16 * 4160)

__host__ __device__ __forceinline__ bool tc_has_bf(const GemvArgs& a) {
    for (int i = 0; i < a.nseg; i++)
        if (rl_is_bf(a.seg[i].kind)) return true;
    return false;
}
constexpr int TC_EPI = 4;          // epilogue warps = partial-sum buffers: a tile's epilogue may take four tile times
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }
// rows of a tile of this segment: what the host chose, else the most a stage holds
__host__ __device__ __forceinline__ int tc_tile_rows(const Seg& g, int K) { return g.tr > 0 ? g.tr : rl_tile_rows(g.kind, K); }
// bytes of dynamic shared memory: stages | digit planes [NB][4][K + 64] | fp32 activations [NB][K] (only with
// bf16 rows) | partial sums [TC_EPI][NB][W][32]
// bytes of a stage: the slots the largest tile of the launch occupies (the up rows of a pair tile start at slot 16)
__host__ __device__ __forceinline__ int tc_stage_bytes(const GemvArgs& a) {
    int m = 0;
    for (int i = 0; i < a.nseg; i++) {
        const Seg& g = a.seg[i];
        const int tr = tc_tile_rows(g, a.K);
        const int slots = g.kind == SEG_I8_GATEUP ? 16 + tr : tr;
        const int bytes = slots * (rl_two_lanes(g.kind, a.K) ? TC_SLOT_STRIDE_WIDE : TC_SLOT_STRIDE);
        m = bytes > m ? bytes : m;
    }
    return m;
}
__host__ __device__ __forceinline__ size_t tc_smem_bytes(const GemvArgs& a, int NB, int NST, int W) {
    return (size_t)NST * tc_stage_bytes(a) + (size_t)NB * M1_PLANES * (a.K + 64) + (tc_has_bf(a) ? (size_t)NB * a.K * 4 : 0) +
           (size_t)TC_EPI * NB * W * 32 * 4;
}
// the shapes the tensor-core path takes: K slices of whole 64-byte steps
__host__ __device__ __forceinline__ bool tc_shape_ok(int K, int W) { return K % (32 * W) == 0 && K <= 2 * RL_SLOT_MAX && K % 8 == 0; }



// NJ 64-byte steps of a warp's K slice for rows (gid, gid + 8): every load first, then the mma's on NJ
// independent accumulators.
template <int NJ>
__device__ __forceinline__ void tc_i8_steps(const unsigned char* pa, const unsigned char* pb, const int8_t* px, bool colact, int (&c)[4]) {
    uint4 wa[NJ], wb[NJ], xb[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        wa[j] = *reinterpret_cast<const uint4*>(pa + 64 * j);
        wb[j] = *reinterpret_cast<const uint4*>(pb + 64 * j);
        xb[j] = make_uint4(0u, 0u, 0u, 0u);
        if (colact) xb[j] = *reinterpret_cast<const uint4*>(px + 64 * j);
    }
    int cc[NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        cc[j][0] = cc[j][1] = cc[j][2] = cc[j][3] = 0;
        imma16832(cc[j], wa[j].x, wb[j].x, wa[j].y, wb[j].y, xb[j].x, xb[j].y);
    }
#pragma unroll
    for (int j = 0; j < NJ; j++) imma16832(cc[j], wa[j].z, wb[j].z, wa[j].w, wb[j].w, xb[j].z, xb[j].w);
#pragma unroll
    for (int j = 0; j < NJ; j++)
#pragma unroll
        for (int q = 0; q < 4; q++) c[q] += cc[j][q];
}

// NST stages of shared memory (1 .. TC_MAX_STAGES): as many as the longest block has tiles. (Keeping two of these
// blocks, or one and an expert block, on an SM so that the next kernel's first tiles arrive under the previous
// kernel was measured and lost: it costs a stage and 40 registers per thread.)
constexpr int TC_MAX_STAGES = 3;
template <int NB, int W>
__global__ void __launch_bounds__((W + TC_EPI) * 32, 1) k_tcgemv(const GemvArgs a, int nseq, int NST, int stage_bytes) {
    constexpr int WT = W + TC_EPI;                 // all warps
    constexpr int BAR_N = W * 32 + 32;             // the compute warps and the one epilogue warp of a tile
    extern __shared__ __align__(128) unsigned char tc_smem[];
    const bool has_bf = tc_has_bf(a);
    unsigned char* stages = tc_smem;                                                     // [NST][stage_bytes]
    const int XS = a.K + 64;                                                             // plane stride: neighbouring planes in different halves of the banks
    int8_t* xq = reinterpret_cast<int8_t*>(tc_smem + (size_t)NST * stage_bytes);         // [NB][4][XS] digit planes
    float* xs = reinterpret_cast<float*>(xq + (size_t)NB * M1_PLANES * XS);              // [NB][K] when has_bf
    float* part = xs + (has_bf ? (size_t)NB * a.K : 0);                                  // [TC_EPI][NB][W][32]
    __shared__ __align__(8) uint64_t full_bar[TC_MAX_STAGES];
    __shared__ float red[2][WT][NB];
    __shared__ float s_xscale[NB];
    __shared__ int s_last;
    __shared__ float s_bv[TC_EPI][NB];
    __shared__ int s_bi[TC_EPI][NB];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid = lane & 3;
    const int b0 = blockIdx.y * NB;                    // first sequence of this pass
    const int t0 = (int)blockIdx.x * a.jq + min((int)blockIdx.x, a.jr);          // the first jr blocks take one tile more
    const int t1 = t0 + a.jq + ((int)blockIdx.x < a.jr ? 1 : 0);
    grid_dep_launch();
    trace_in(a.trace, 1, a.seg[0].rows);
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) mbar_init(&full_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto locate = [&](int t, int& s, int& tin) {
        s = 0; tin = t;
        while (s + 1 < a.nseg && tin >= a.seg[s].jobs) { tin -= a.seg[s].jobs; s++; }
    };
    // one warp asks for tile t into stage st, one bulk copy per slot
    auto request = [&](int t, int st) {
        int s, tin;
        locate(t, s, tin);
        const Seg& sg = a.seg[s];
        const int tr = tc_tile_rows(sg, a.K);
        const int row0 = tin * tr;
        const int n = min(tr, sg.rows - row0);
        const bool pair = sg.kind == SEG_I8_GATEUP;
        const uint32_t rb = rl_is_bf(sg.kind) ? 2u * a.K : (uint32_t)a.K;          // bytes per slot
        const int nslots = pair ? 2 * n : n;
        if (lane == 0) mbar_expect_tx(&full_bar[st], rb * nslots);
        __syncwarp();
        const int sstride = rl_two_lanes(sg.kind, a.K) ? TC_SLOT_STRIDE_WIDE : TC_SLOT_STRIDE;
        const bool active = pair ? (lane < n || (lane >= 16 && lane < 16 + n)) : lane < n;
        if (active) {
            const char* src = pair ? (lane < 16 ? (const char*)sg.w + (size_t)(row0 + lane) * a.K
                                                : (const char*)sg.w2 + (size_t)(row0 + lane - 16) * a.K)
                                   : (const char*)sg.w + (size_t)(row0 + lane) * rb;
            bulk_load(stages + (size_t)st * stage_bytes + (size_t)lane * sstride, src, rb, &full_bar[st]);
        }
    };
    if (warp == W)
        for (int i = 0; i < NST && t0 + i < t1; i++) request(t0 + i, i);
    grid_dep_wait();
    trace_pt(a.trace, 1);

    // prologue: the normalised activations as int8 digit planes (and fp32 when bf16 rows follow). Thread c takes
    // the 8 consecutive values of chunk c, so every value crosses from global memory once, as two 16-byte loads.
    {
        const int kc = threadIdx.x * 8;
        const bool has = kc < a.K;
        float xv[NB][8];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
            if (has && b0 + b < nseq) {
                v0 = *reinterpret_cast<const float4*>(a.x + (size_t)(b0 + b) * a.x_stride + kc);
                v1 = *reinterpret_cast<const float4*>(a.x + (size_t)(b0 + b) * a.x_stride + kc + 4);
            }
            xv[b][0] = v0.x; xv[b][1] = v0.y; xv[b][2] = v0.z; xv[b][3] = v0.w;
            xv[b][4] = v1.x; xv[b][5] = v1.y; xv[b][6] = v1.z; xv[b][7] = v1.w;
        }
        const bool znorm = a.gn_w == nullptr && a.norm_w != nullptr;
        if (a.gn_w) {
            // DeltaNet output projection: w * rmsnorm_DV(o) * silu(z) per value head (aegist/hybrid.py:133-147);
            // a head is DV / 8 neighbouring lanes
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (has) wv = *reinterpret_cast<const uint4*>(a.gn_w + (kc % a.DV));
            const float gw[8] = {bflo(wv.x), bfhi(wv.x), bflo(wv.y), bfhi(wv.y), bflo(wv.z), bfhi(wv.z), bflo(wv.w), bfhi(wv.w)};
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float4 z0 = make_float4(0.f, 0.f, 0.f, 0.f), z1 = z0;
                if (has && b0 + b < nseq) {
                    z0 = *reinterpret_cast<const float4*>(a.z + (size_t)(b0 + b) * a.x_stride + kc);
                    z1 = *reinterpret_cast<const float4*>(a.z + (size_t)(b0 + b) * a.x_stride + kc + 4);
                }
                const float zz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) ss = fmaf(xv[b][i], xv[b][i], ss);
                for (int o = a.DV >> 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float r = 1.0f / sqrtf(ss / (float)a.DV + a.eps);
#pragma unroll
                for (int i = 0; i < 8; i++) xv[b][i] = (gw[i] * (xv[b][i] * r)) * zz[i];
            }
        } else if (a.norm_w) {
            // (1 + w) * x / rms(x) (aegist/hybrid.py:119-130). The rms is one factor for the whole vector, so the sum of
            // squares and the largest |(1 + w) x| are reduced together, behind one barrier, and the factor joins after it
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (has) wv = *reinterpret_cast<const uint4*>(a.norm_w + kc);
            const float nw[8] = {1.0f + bflo(wv.x), 1.0f + bfhi(wv.x), 1.0f + bflo(wv.y), 1.0f + bfhi(wv.y),
                                 1.0f + bflo(wv.z), 1.0f + bfhi(wv.z), 1.0f + bflo(wv.w), 1.0f + bfhi(wv.w)};
#pragma unroll
            for (int b = 0; b < NB; b++) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) { ss = fmaf(xv[b][i], xv[b][i], ss); xv[b][i] *= nw[i]; }
                ss = warp_sum(ss);
                if (lane == 0) red[0][warp][b] = ss;
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float mx = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(xv[b][i]));
            mx = warp_max(mx);
            if (lane == 0) red[1][warp][b] = mx;
        }
        __syncthreads();
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float mx = 0.f;
#pragma unroll
            for (int w = 0; w < WT; w++) mx = fmaxf(mx, red[1][w][b]);
            if (znorm) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < WT; w++) t += red[0][w][b];
                const float rn = 1.0f / sqrtf(t / (float)a.K + a.eps);
#pragma unroll
                for (int i = 0; i < 8; i++) xv[b][i] *= rn;
                mx *= rn;
            }
            const float inv = mx > 1e-30f ? 127.0f / mx : 0.f;
            if (threadIdx.x == 0) s_xscale[b] = mx / 127.0f;
            if (has) {
                uint2 w[M1_PLANES];
                digits8(xv[b], inv, false, w);
#pragma unroll
                for (int p = 0; p < M1_PLANES; p++) *reinterpret_cast<uint2*>(xq + (size_t)(b * M1_PLANES + p) * XS + kc) = w[p];
                if (has_bf) {
                    *reinterpret_cast<float4*>(xs + (size_t)b * a.K + kc) = make_float4(xv[b][0], xv[b][1], xv[b][2], xv[b][3]);
                    *reinterpret_cast<float4*>(xs + (size_t)b * a.K + kc + 4) = make_float4(xv[b][4], xv[b][5], xv[b][6], xv[b][7]);
                }
            }
        }
    }
    __syncthreads();
    trace_pt(a.trace, 2);

    float best_v[NB];
    int best_i[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) { best_v[b] = -INFINITY; best_i[b] = 0x7fffffff; }

    if (warp < W) {
        // ---- compute warps: partial sums of every tile into part[tile & 1] ----
        // this lane's activation column in the B operand: plane (gid & 3) of sequence (gid >> 2)
        const bool colact = (gid >> 2) < NB;
        const int8_t* xcol = xq + (size_t)gid * XS;
        // what this lane's two result columns (2 tid, 2 tid + 1) weigh: planes 2 (tid & 1), 2 (tid & 1) + 1 of sequence tid >> 1
        const float pw0 = ((tid >> 1) < NB ? s_xscale[(tid >> 1) < NB ? (tid >> 1) : 0] : 0.f) * ((tid & 1) ? (1.0f / 16384.0f) : 1.0f);
        const float pw1 = pw0 * (1.0f / 128.0f);
        int st = 0, ph = 0;                               // stage of tile i and the parity of its use: no divisions per tile
        for (int t = t0, i = 0; t < t1; t++, i++) {
            const int buf = i & (TC_EPI - 1);
            int s, tin;
            locate(t, s, tin);
            const int kind = a.seg[s].kind;
            const bool isbf = rl_is_bf(kind);
            const bool two = rl_two_lanes(kind, a.K);
            const int tr = tc_tile_rows(a.seg[s], a.K);    // slots beyond the tile's rows are not part of the stage: clamp
            float* pt = part + (size_t)buf * NB * W * 32;
            const unsigned char* stage = stages + (size_t)st * stage_bytes;
            if (i >= TC_EPI) bar_sync(1 + TC_EPI + buf, BAR_N);   // the epilogue of tile i - TC_EPI has read this buffer
            mbar_wait(&full_bar[st], ph, a.err);
            if (!isbf) {
                const int nrb = two ? 1 : 2;               // 16-slot blocks in the tile
                const int rbk = warp & (nrb - 1), ks = warp >> (nrb - 1);
                const int slice = two ? a.K / W : a.K / (W / 2);      // bytes = values; a multiple of 64 (constant divisors)
                const int sstride = two ? TC_SLOT_STRIDE_WIDE : TC_SLOT_STRIDE;
                const int slot_hi = (kind == SEG_I8_GATEUP ? rbk * 16 : 0) + tr - 1;       // last slot this row block may read
                const unsigned char* pa = stage + (size_t)min(rbk * 16 + gid, slot_hi) * sstride + ks * slice + tid * 16;
                const unsigned char* pb = stage + (size_t)min(rbk * 16 + gid + 8, slot_hi) * sstride + ks * slice + tid * 16;
                const int8_t* px = xcol + ks * slice + tid * 16;
                int c0[4] = {0, 0, 0, 0};
                int j = 0;
                for (; j + 256 <= slice; j += 256) tc_i8_steps<4>(pa + j, pb + j, px + j, colact, c0);
                if (j + 128 <= slice) { tc_i8_steps<2>(pa + j, pb + j, px + j, colact, c0); j += 128; }
                if (j + 64 <= slice) tc_i8_steps<1>(pa + j, pb + j, px + j, colact, c0);
                // c0[q]: row gid (+8 for q >= 2), column 2 tid + (q & 1); the four planes of a sequence are lanes tid, tid ^ 1
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float v = (float)c0[2 * h] * pw0 + (float)c0[2 * h + 1] * pw1;
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    const int b = tid >> 1;
                    if ((tid & 1) == 0 && b < NB) pt[((size_t)b * W + ks) * 32 + rbk * 16 + gid + h * 8] = v;
                }
            } else {
                // bf16 rows: 16 slots of 2 K bytes; warp -> (8-row half, K slice), lane -> (row, 16-byte unit of a 64-byte step)
                const int rh = warp & 1, ks = warp >> 1;
                const int slice = 2 * a.K / (W / 2);       // bytes
                const unsigned char* pa = stage + (size_t)min(rh * 8 + gid, tr - 1) * TC_SLOT_STRIDE_WIDE + ks * slice + tid * 16;
                float acc[NB];
#pragma unroll
                for (int b = 0; b < NB; b++) acc[b] = 0.f;
#pragma unroll 4
                for (int j = 0; j < slice; j += 64) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(pa + j);
                    const int k0 = (ks * slice + j + tid * 16) >> 1;
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const float4* pxs = reinterpret_cast<const float4*>(xs + (size_t)b * a.K + k0);
                        const float4 x0 = pxs[0], x1 = pxs[1];
                        float p = x0.x * bflo(wv.x);
                        p = fmaf(x0.y, bfhi(wv.x), p); p = fmaf(x0.z, bflo(wv.y), p); p = fmaf(x0.w, bfhi(wv.y), p);
                        p = fmaf(x1.x, bflo(wv.z), p); p = fmaf(x1.y, bfhi(wv.z), p); p = fmaf(x1.z, bflo(wv.w), p);
                        p = fmaf(x1.w, bfhi(wv.w), p);
                        acc[b] += p;
                    }
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    float v = acc[b];
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (tid == 0) pt[((size_t)b * W + ks) * 32 + rh * 8 + gid] = v;
                }
            }
            bar_arrive(1 + buf, BAR_N);            // partial sums written, the stage read
            if (++st == NST) { st = 0; ph ^= 1; }
        }
    } else {
        // ---- epilogue warps: warp W + p takes tiles p, p + 2, ... of this block ----
        const int p = warp - W;
        int st = p % NST;                                  // stage of this warp's next tile
        const int dst = TC_EPI % NST;
        for (int t = t0 + p, i = p; t < t1; t += TC_EPI, i += TC_EPI) {
            int s, tin;
            locate(t, s, tin);
            const Seg& sg = a.seg[s];
            const bool isbf = rl_is_bf(sg.kind);
            const bool two = rl_two_lanes(sg.kind, a.K);
            const bool pair = sg.kind == SEG_I8_GATEUP;
            const int tr = tc_tile_rows(sg, a.K);
            const int np = isbf ? W / 2 : (two ? W : W / 2);       // partial sums per row slot
            const int row = tin * tr + lane;                        // lane j owns output row0 + j
            const bool mine = lane < tr && row < sg.rows;
            const float* pt = part + (size_t)p * NB * W * 32;
            // everything the epilogue needs from global memory is requested before the tile is waited for
            float e0 = 0.f, e1 = 0.f;
            uint2 ecw = make_uint2(0u, 0u);
            float cst[NB][3];
            if (mine) {
                switch (sg.kind) {
                case SEG_I8: case SEG_I8_ARGMAX: case SEG_I8_SILU: case SEG_I8_CONV: case SEG_I8_ACC: e0 = bf(sg.s[row]); break;
                case SEG_I8_GATEUP: e0 = bf(sg.s[row]); e1 = bf(sg.s2[row]); break;
                case SEG_BF_DECAY: e0 = bf(a.a_log[row]); e1 = bf(a.dt_bias[row]); break;
                case SEG_BF: e0 = sg.bias ? sg.bias[row] : 0.f; break;
                default: break;
                }
                if (sg.kind == SEG_I8_CONV) {
                    ecw = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)row * 4);
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        if (b0 + b >= nseq) continue;
                        const float* stt = a.conv_state + ((size_t)(b0 + b) * sg.rows + row) * 3;
                        cst[b][0] = stt[0]; cst[b][1] = stt[1]; cst[b][2] = stt[2];
                    }
                }
            }
            bar_sync(1 + p, BAR_N);                // partial sums of tile i complete; its stage is free
            if (t + NST < t1) request(t + NST, st);
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (!mine || b0 + b >= nseq) continue;
                const float* pb = pt + (size_t)b * W * 32;
                float sA = 0.f, sB = 0.f;
                for (int w = 0; w < np; w++) { sA += pb[w * 32 + lane]; if (pair) sB += pb[w * 32 + lane + 16]; }
                float* out = sg.out + (size_t)(b0 + b) * sg.out_stride;
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
                    float y = bflo(ecw.x) * cst[b][0];
                    y = fmaf(bfhi(ecw.x), cst[b][1], y);
                    y = fmaf(bflo(ecw.y), cst[b][2], y);
                    y = fmaf(bfhi(ecw.y), raw, y);
                    stt[0] = cst[b][1]; stt[1] = cst[b][2]; stt[2] = raw;
                    out[row] = siluf_(y);
                } break;
                case SEG_BF_SIGMOID: out[row] = sigmoidf_(sA); break;
                case SEG_BF_DECAY: out[row] = -expf(e0) * softplusf_(sA + e1); break;
                case SEG_BF: out[row] = sA + e0; break;
                case SEG_I8_GATEUP: out[row] = siluf_(e0 * sA) * (e1 * sB); break;
                }
            }
            if (t + TC_EPI < t1) bar_arrive(1 + TC_EPI + p, BAR_N);     // the buffer may be written again
            st += dst;
            if (st >= NST) st -= NST;
        }
    }
    trace_pt(a.trace, 3);
    if (a.finisher == FIN_NONE) { trace_out(a.trace); return; }
    // finishers, one pass of NB sequences at a time
    if (a.finisher == FIN_ARGMAX) {
        if (warp >= W) {
#pragma unroll
            for (int b = 0; b < NB; b++) {          // best over the lanes of an epilogue warp
                float v = best_v[b];
                int ix = best_i[b];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
                    if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
                }
                if (lane == 0) { s_bv[warp - W][b] = v; s_bi[warp - W][b] = ix; }
            }
        }
        __syncthreads();
        if (threadIdx.x < NB && b0 + threadIdx.x < nseq) {
            const int b = threadIdx.x;
            float v = s_bv[0][b];
            int ix = s_bi[0][b];
            for (int w = 1; w < TC_EPI; w++)
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
    if (!s_last) { trace_out(a.trace); return; }
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
    trace_out(a.trace);
}

}  // namespace b2
