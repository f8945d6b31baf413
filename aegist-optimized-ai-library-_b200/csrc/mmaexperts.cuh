// Batched decode: the 4-bit experts as a grouped tensor-core GEMM (the "expert GEMMs" of the
// reference for more than 8 tokens, aegist_rs/kernels/hybrid.cu:461-549, which tile in shared memory
// on CUDA cores).
//
//   k_group_picks   counting sort of the step's picks by expert (the host code of
//                   aegist_rs/src/hybrid.rs:875-900, on the device): per expert the list of its picks in
//                   pick order, cut into chunks: runs of up to 32 picks (16 for k_umma_q4) go to the "big" table, a rest of
//                   at most 8 picks to the "small" table (most experts of a step have only a few picks)
//   k_mma_q4<NT>    for one chunk (one expert, <= 8 * NT of its picks) and a block of weight rows:
//                   out = rows x picks, codes widened to fp16 (exact), activations as fp16 hi + lo,
//                   mma.sync.m16n8k16 into a per-group accumulator that is then scaled:
//                   sum_k w x = sum_groups ( s_g * sum_k code x  +  m_g * sum_k x )
//                   gate/up mode writes silu(gate) * up per pick; down mode writes the pick's output row
//                   into ypart for the pick-order combine.
//
// The activations are stored with every 8 values in the order 0 4 1 5 2 6 3 7: a 32-bit word of
// eight codes then splits into the half2 pairs (c0,c4) (c1,c5) (c2,c6) (c3,c7) with one logic
// operation and one half2 arithmetic operation each, and the k order inside an mma step is free as
// long as both operands use the same one.
#pragma once

namespace b2 {

constexpr int GQ_MAXP = 1024;     // picks per step the grouping kernel handles (64 sequences x 8 x 2)
constexpr int GQ_BIG = 32;        // picks per big chunk
constexpr int GQ_SMALL = 8;       // picks per small chunk

struct ChunkTable {
    int* expert;                  // [cap]
    int* start;                   // [cap] offset into the pick list
    int* n;                       // [cap]
    int* count;                   // [1]
    int cap;
};

struct GroupArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const int* top_idx;           // [T][idx_stride]
    int idx_stride, T, topk, E;
    const uint8_t* const* eptr;   // only experts resident here are grouped
    int* list;                    // [P] pick ids (t * topk + r) sorted by expert, pick order inside an expert
    ChunkTable small, big;
    int big_n;                    // picks per big chunk (0: GQ_BIG)
};

// one block of 1024 threads. The order of the picks inside an expert's list is whatever the shared-memory atomics
// give: every pick's result goes to its own place in ypart, so the order changes nothing downstream.
__global__ void __launch_bounds__(1024) k_group_picks(const GroupArgs a) {
    __shared__ int s_e[GQ_MAXP];
    __shared__ int s_cnt[256], s_off[256], s_fill[256];
    __shared__ int s_w[3][8];
    grid_dep_launch();
    trace_in(a.trace, 11, gridDim.x);
    grid_dep_wait();
    const int P = a.T * a.topk;
    const int BN = a.big_n > 0 ? a.big_n : GQ_BIG;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < 256) { s_cnt[threadIdx.x] = 0; s_fill[threadIdx.x] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = a.top_idx[(size_t)(p / a.topk) * a.idx_stride + p % a.topk];
        const int ok = (e >= 0 && e < a.E && a.eptr[e] != nullptr) ? e : -1;
        s_e[p] = ok;
        if (ok >= 0) atomicAdd(&s_cnt[ok], 1);
    }
    __syncthreads();
    // per expert: big chunks of up to 32 picks while more than 8 are left, then one small chunk of the rest;
    // exclusive prefix sums over the experts of the pick counts and of the two chunk counts (256 threads)
    int cnt = 0, nb = 0, ns = 0, x0 = 0, x1 = 0, x2 = 0;
    if (threadIdx.x < 256) {
        const int e = threadIdx.x;
        cnt = e < a.E ? s_cnt[e] : 0;
        nb = cnt > GQ_SMALL ? (cnt - GQ_SMALL + BN - 1) / BN : 0;
        ns = (cnt - nb * BN) > 0 ? 1 : 0;
        x0 = cnt; x1 = nb; x2 = ns;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o), y2 = __shfl_up_sync(0xffffffffu, x2, o);
            if (lane >= o) { x0 += y0; x1 += y1; x2 += y2; }
        }
        if (lane == 31) { s_w[0][warp] = x0; s_w[1][warp] = x1; s_w[2][warp] = x2; }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
        const int e = threadIdx.x;
        int b0 = 0, b1 = 0, b2 = 0;
        for (int w = 0; w < warp; w++) { b0 += s_w[0][w]; b1 += s_w[1][w]; b2 += s_w[2][w]; }
        const int off = b0 + x0 - cnt, cb0 = b1 + x1 - nb, cs0 = b2 + x2 - ns;
        s_off[e] = off;
        int s0 = 0, left = cnt;
        for (int k = 0; k < nb; k++) {
            const int n = min(BN, left);
            if (cb0 + k < a.big.cap) { a.big.expert[cb0 + k] = e; a.big.start[cb0 + k] = off + s0; a.big.n[cb0 + k] = n; }
            s0 += n; left -= n;
        }
        if (ns && cs0 < a.small.cap) { a.small.expert[cs0] = e; a.small.start[cs0] = off + s0; a.small.n[cs0] = left; }
        if (e == 255) { *a.big.count = min(cb0 + nb, a.big.cap); *a.small.count = min(cs0 + ns, a.small.cap); }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = s_e[p];
        if (e >= 0) a.list[s_off[e] + atomicAdd(&s_fill[e], 1)] = p;
    }
    trace_out(a.trace);
}

constexpr int Q4_THREADS = 128;             // 4 warps, one 16-row slab each
constexpr int Q4_ROWS = 64;                 // weight rows per tile (16 per warp); a pair tile = 32 gate + 32 up
constexpr int Q4_PA = 160;                  // bytes between code rows in shared memory (128 used)
constexpr int Q4_STAGE_A = Q4_ROWS * Q4_PA; // 10240
constexpr int Q4_STAGE_S = Q4_ROWS * 16;    // per row: 4 groups x (scale, min) f16
constexpr int Q4_STAGES = 2;                // two blocks of the 32-pick variant fit an SM
__host__ __device__ constexpr int q4_stage_bytes(int NT) { return Q4_STAGE_A + Q4_STAGE_S + 16 * NT * MM_PB; }   // 19712 (NT 1), 45056 (NT 4)

struct Q4Args {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const uint8_t* const* eptr;
    const int* list;
    ChunkTable chunks;
    int topk;
    int pair;                 // 1: rows are (gate i, up i) pairs -> act; 0: down rows -> ypart
    int rows, K;              // output rows (I pairs, or D) and contraction length (D, or I)
    int row_tiles;            // tiles of 64 rows (32 pairs) one block walks through
    size_t off_q, off_s, off_m;   // sections of this matrix inside an expert
    int up_row0;              // pair mode: first up row (= I)
    const __half* xh;         // activations: [token or pick][2][K] fp16 hi | lo, 8-permuted
    const float* xsum;        // [token or pick][K / 64] sums of the activations per group
    int by_pick;              // 0: xh / xsum are indexed by token (p / topk); 1: by pick
    float* out;               // pair: act [P][rows]; down: ypart [T][topk + 1][rows]
};

// eight codes (a 32-bit word, code i in bits 4i..4i+3) -> half2 pairs (c0,c4) (c1,c5) (c2,c6) (c3,c7), exact
__device__ __forceinline__ void q4x8_to_h2x4(uint32_t w, uint32_t& p0, uint32_t& p1, uint32_t& p2, uint32_t& p3) {
    const uint32_t magic = 0x64006400u;                // 1024 | code in the low mantissa bits
    const uint32_t k1024 = 0x64006400u, k16th = 0x2C002C00u, km64 = 0xD400D400u;
    uint32_t a = (w & 0x000F000Fu) | magic;
    uint32_t b = (w & 0x00F000F0u) | magic;            // 1024 + 16 * code
    const uint32_t w8 = w >> 8;
    uint32_t c = (w8 & 0x000F000Fu) | magic;
    uint32_t d = (w8 & 0x00F000F0u) | magic;
    const __half2 h1024 = *reinterpret_cast<const __half2*>(&k1024);
    const __half2 h16th = *reinterpret_cast<const __half2*>(&k16th);
    const __half2 hm64 = *reinterpret_cast<const __half2*>(&km64);
    __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), h1024);
    __half2 hb = __hfma2(*reinterpret_cast<__half2*>(&b), h16th, hm64);
    __half2 hc = __hsub2(*reinterpret_cast<__half2*>(&c), h1024);
    __half2 hd = __hfma2(*reinterpret_cast<__half2*>(&d), h16th, hm64);
    p0 = *reinterpret_cast<uint32_t*>(&ha);
    p1 = *reinterpret_cast<uint32_t*>(&hb);
    p2 = *reinterpret_cast<uint32_t*>(&hc);
    p3 = *reinterpret_cast<uint32_t*>(&hd);
}

// grid (row blocks, blocks per row block); NT = 8-pick tiles per chunk (1: small table, 4: big table)
template <int NT>
__global__ void __launch_bounds__(Q4_THREADS) k_mma_q4(const Q4Args a) {
    constexpr int STAGE = q4_stage_bytes(NT);
    constexpr int NCOL = 8 * NT;                  // picks per chunk
    extern __shared__ __align__(128) unsigned char q4_smem[];
    __shared__ int s_pick[NCOL];
    __shared__ int s_src[NCOL], s_dst[NCOL];     // per pick: row of its activations, row of its output (no divisions later)
    __shared__ float s_xsum[NCOL][33];           // [pick of the chunk][group]
    __shared__ float gate_s[2][16][NCOL + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid = lane & 3;
    grid_dep_launch();
    trace_in(a.trace, 12, gridDim.x * 1000 + NT);
    grid_dep_wait();
    // a block walks the chunks blockIdx.y, blockIdx.y + gridDim.y, ...: the grid is sized for the SMs, not for the
    // largest possible number of chunks
    const int nchunk = *a.chunks.count;
    for (int chunk = blockIdx.y; chunk < nchunk; chunk += gridDim.y) {
    const int e = a.chunks.expert[chunk];
    const int n = min(a.chunks.n[chunk], NCOL);
    const uint8_t* base = a.eptr[e];
    if (threadIdx.x < NCOL) {
        const int pk = threadIdx.x < n ? a.list[a.chunks.start[chunk] + threadIdx.x] : -1;
        const int tk = pk < 0 ? 0 : pk / a.topk;
        s_pick[threadIdx.x] = pk;
        s_src[threadIdx.x] = pk < 0 ? 0 : (a.by_pick ? pk : tk);
        s_dst[threadIdx.x] = pk < 0 ? 0 : (a.pair ? pk : tk * (a.topk + 1) + (pk - tk * a.topk));
    }
    __syncthreads();
    const int rows_per_tile = a.pair ? Q4_ROWS / 2 : Q4_ROWS;
    const int row0 = blockIdx.x * rows_per_tile * a.row_tiles;
    const int ngroup = a.K >> 6;                 // <= 32
    for (int p = threadIdx.x; p < n * ngroup; p += Q4_THREADS) {
        const int c = p / ngroup, g = p % ngroup;
        s_xsum[c][g] = a.xsum[(size_t)s_src[c] * ngroup + g];
    }
    const int rowbytes = a.K >> 1;
    const int nk = a.K / MM_KC;
    const int niter = nk * a.row_tiles;

    auto weight_row = [&](int rt, int r) {  // shared-memory row r of tile rt -> row of the matrix
        const int t0 = row0 + rt * rows_per_tile;
        const int g = a.pair ? (r < 32 ? t0 + r : a.up_row0 + t0 + (r - 32)) : t0 + r;
        const int last = a.pair ? (r < 32 ? a.rows - 1 : a.up_row0 + a.rows - 1) : a.rows - 1;
        return min(g, last);
    };
    auto load_stage = [&](int it, int st) {
        const int rt = it / nk, kc = it - rt * nk;
        unsigned char* sa = q4_smem + (size_t)st * STAGE;
        unsigned char* ss = sa + Q4_STAGE_A;
        unsigned char* sb = ss + Q4_STAGE_S;
        for (int p = threadIdx.x; p < Q4_ROWS * 8; p += Q4_THREADS) {          // codes: 64 rows x 128 B
            const int r = p >> 3, c = p & 7;
            cp_async16(sa + r * Q4_PA + c * 16, base + a.off_q + (size_t)weight_row(rt, r) * rowbytes + (size_t)kc * 128 + c * 16);
        }
        {                                                                      // scales and mins: 8 B each per row
            const int r = threadIdx.x >> 1, which = threadIdx.x & 1;
            const uint8_t* src = base + (which ? a.off_m : a.off_s) + ((size_t)weight_row(rt, r) * ngroup + (size_t)kc * 4) * 2;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(ss + r * 16 + which * 8)), "l"(src) : "memory");
        }
        // activations of the chunk's picks only: columns 0..NCOL-1 hi, NCOL..2 NCOL-1 lo; the other
        // columns keep whatever shared memory held (their products are never stored)
        for (int p = threadIdx.x; p < 2 * n * (MM_KC / 8); p += Q4_THREADS) {
            const int j = p / (MM_KC / 8), c = p % (MM_KC / 8);
            const int part = j >= n, tc = part ? j - n : j;
            const int src_row = s_src[tc];
            cp_async16(sb + (part * NCOL + tc) * MM_PB + c * 16, a.xh + ((size_t)src_row * 2 + part) * a.K + (size_t)kc * MM_KC + c * 8);
        }
        cp_async_commit();
    };
    for (int i = 0; i < Q4_STAGES - 1; i++) {
        if (i < niter) load_stage(i, i); else cp_async_commit();
    }
    float acc[2 * NT][4];
#pragma unroll
    for (int j = 0; j < 2 * NT; j++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[j][q] = 0.f;

    const int r0 = warp * 16 + gid, r1 = r0 + 8;
    int kc = 0, rt = 0;
    for (int it = 0; it < niter; it++) {
        cp_async_wait<Q4_STAGES - 2>();
        __syncthreads();
        if (it + Q4_STAGES - 1 < niter) load_stage(it + Q4_STAGES - 1, (it + Q4_STAGES - 1) % Q4_STAGES); else cp_async_commit();
        const unsigned char* sa = q4_smem + (size_t)(it % Q4_STAGES) * STAGE;
        const unsigned char* ss = sa + Q4_STAGE_A;
        const unsigned char* sb = ss + Q4_STAGE_S;
        const uint4 sm0 = *reinterpret_cast<const uint4*>(ss + r0 * 16);      // 4 scales | 4 mins of row r0
        const uint4 sm1 = *reinterpret_cast<const uint4*>(ss + r1 * 16);
        const uint32_t sv0[2] = {sm0.x, sm0.y}, mv0[2] = {sm0.z, sm0.w}, sv1[2] = {sm1.x, sm1.y}, mv1[2] = {sm1.z, sm1.w};
#pragma unroll
        for (int sbk = 0; sbk < 4; sbk++) {            // one 64-value group per super-block
            const uint2 w0 = *reinterpret_cast<const uint2*>(sa + r0 * Q4_PA + sbk * 32 + tid * 8);
            const uint2 w1 = *reinterpret_cast<const uint2*>(sa + r1 * Q4_PA + sbk * 32 + tid * 8);
            uint32_t af[4][4];
            q4x8_to_h2x4(w0.x, af[0][0], af[0][2], af[1][0], af[1][2]);
            q4x8_to_h2x4(w1.x, af[0][1], af[0][3], af[1][1], af[1][3]);
            q4x8_to_h2x4(w0.y, af[2][0], af[2][2], af[3][0], af[3][2]);
            q4x8_to_h2x4(w1.y, af[2][1], af[2][3], af[3][1], af[3][3]);
            const float s0 = h2f((uint16_t)(sv0[sbk >> 1] >> ((sbk & 1) * 16)));
            const float m0 = h2f((uint16_t)(mv0[sbk >> 1] >> ((sbk & 1) * 16)));
            const float s1 = h2f((uint16_t)(sv1[sbk >> 1] >> ((sbk & 1) * 16)));
            const float m1 = h2f((uint16_t)(mv1[sbk >> 1] >> ((sbk & 1) * 16)));
            const int grp = kc * 4 + sbk;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                if (nt * 8 >= n) break;
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    float t[4] = {0.f, 0.f, 0.f, 0.f};
                    const unsigned char* bp = sb + (part * NCOL + nt * 8 + gid) * MM_PB + sbk * 128 + tid * 32;
                    const uint4 x0 = *reinterpret_cast<const uint4*>(bp);
                    const uint4 x1 = *reinterpret_cast<const uint4*>(bp + 16);
                    mma16816(t, af[0], x0.x, x0.y);
                    mma16816(t, af[1], x0.z, x0.w);
                    mma16816(t, af[2], x1.x, x1.y);
                    mma16816(t, af[3], x1.z, x1.w);
                    float* ac = acc[part * NT + nt];
                    ac[0] = fmaf(s0, t[0], ac[0]); ac[1] = fmaf(s0, t[1], ac[1]);
                    ac[2] = fmaf(s1, t[2], ac[2]); ac[3] = fmaf(s1, t[3], ac[3]);
                }
#pragma unroll
                for (int c = 0; c < 2; c++) {           // min term, once per pick
                    const float xs = s_xsum[nt * 8 + 2 * tid + c][grp];
                    acc[nt][c] = fmaf(m0, xs, acc[nt][c]);
                    acc[nt][2 + c] = fmaf(m1, xs, acc[nt][2 + c]);
                }
            }
        }
        if (++kc < nk) continue;
        // a row tile is complete: write it out and start the next one
        kc = 0;
        const int t0 = row0 + rt * rows_per_tile;
        if (a.pair) {
            if (warp < 2) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int q = 0; q < 4; q++) gate_s[warp][gid + (q >> 1) * 8][nt * 8 + 2 * tid + (q & 1)] = acc[nt][q] + acc[NT + nt][q];
            }
            __syncthreads();
        }
        if (!a.pair || warp >= 2) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int rl = gid + (q >> 1) * 8, col = nt * 8 + 2 * tid + (q & 1);
                    const int pk = s_pick[col];
                    const int row = a.pair ? t0 + (warp - 2) * 16 + rl : t0 + warp * 16 + rl;
                    if (pk < 0 || row >= a.rows) continue;
                    const float dot = acc[nt][q] + acc[NT + nt][q];
                    if (a.pair) a.out[(size_t)pk * a.rows + row] = siluf_(gate_s[warp - 2][rl][col]) * dot;
                    else a.out[(size_t)s_dst[col] * a.rows + row] = dot;
                }
        }
#pragma unroll
        for (int j = 0; j < 2 * NT; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[j][q] = 0.f;
        rt++;
    }
    cp_async_wait<0>();
    __syncthreads();                   // the chunk's tables and stages are reused by the next one
    }
    trace_out(a.trace);
}

}  // namespace b2
