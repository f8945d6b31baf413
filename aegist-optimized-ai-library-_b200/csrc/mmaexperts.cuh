// Batched decode: the 4-bit experts as a grouped tensor-core GEMM (the "expert GEMMs" of the
// reference for more than 8 tokens, aegist_rs/kernels/hybrid.cu:461-549, which tile in shared memory
// on CUDA cores).
//
//   k_group_picks   counting sort of the step's picks by expert (the host code of
//                   aegist_rs/src/hybrid.rs:875-900, on the device): per expert the list of its picks in
//                   pick order, cut into chunks of at most 32 for the GEMM grid
//   k_mma_q4        for one chunk (one expert, <= 32 of its tokens) and one block of weight rows:
//                   out = rows x tokens, codes widened to fp16 (exact), activations as fp16 hi + lo,
//                   mma.sync.m16n8k16 into a per-group accumulator that is then scaled:
//                   sum_k w x = sum_groups ( s_g * sum_k code x  +  m_g * sum_k x )
//                   gate/up mode writes silu(gate) * up per pick; down mode writes the pick's output row
//                   into ypart for the pick-order combine.
#pragma once

namespace b2 {

constexpr int GQ_MAXP = 1024;     // picks per step the grouping kernel handles (64 sequences x 8 x 2)
constexpr int GQ_CH = 32;         // tokens per chunk

struct GroupArgs {
    const int* top_idx;           // [T][idx_stride]
    int idx_stride, T, topk, E;
    const uint8_t* const* eptr;   // only experts resident here are grouped
    int* list;                    // [P] pick ids (t * topk + r) sorted by expert, pick order inside an expert
    int* chunk_expert;            // [max chunks]
    int* chunk_start;             // [max chunks] offset into list
    int* chunk_n;                 // [max chunks]
    int* nchunks;                 // [1]
    int max_chunks;
};

// one block of 1024 threads
__global__ void __launch_bounds__(1024) k_group_picks(const GroupArgs a) {
    __shared__ int s_e[GQ_MAXP];
    __shared__ int s_cnt[256], s_off[256];
    grid_dep_launch();
    grid_dep_wait();
    const int P = a.T * a.topk;
    for (int e = threadIdx.x; e < 256; e += blockDim.x) s_cnt[e] = 0;
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = a.top_idx[(size_t)(p / a.topk) * a.idx_stride + p % a.topk];
        s_e[p] = (e >= 0 && e < a.E && a.eptr[e] != nullptr) ? e : -1;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x)
        if (s_e[p] >= 0) atomicAdd(&s_cnt[s_e[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, c = 0;
        for (int e = 0; e < a.E; e++) {
            s_off[e] = off;
            for (int s0 = 0; s0 < s_cnt[e] && c < a.max_chunks; s0 += GQ_CH, c++) {
                a.chunk_expert[c] = e;
                a.chunk_start[c] = off + s0;
                a.chunk_n[c] = min(GQ_CH, s_cnt[e] - s0);
            }
            off += s_cnt[e];
        }
        *a.nchunks = c;
    }
    __syncthreads();
    // position of a pick inside its expert's list = number of earlier picks of the same expert
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = s_e[p];
        if (e < 0) continue;
        int pos = 0;
        for (int q = 0; q < p; q++) pos += (s_e[q] == e);
        a.list[s_off[e] + pos] = p;
    }
}

constexpr int Q4_ROWS = 64;                 // weight rows per block (16 per warp); a pair block = 32 gate + 32 up
constexpr int Q4_PA = 160;                  // bytes between code rows in shared memory (128 used)
constexpr int Q4_STAGE_A = Q4_ROWS * Q4_PA; // 10240
constexpr int Q4_STAGE_S = Q4_ROWS * 16;    // per row: 4 groups x (scale, min) f16
constexpr int Q4_STAGE_B = 2 * MM_TOK * MM_PB;
constexpr int Q4_STAGE_BYTES = Q4_STAGE_A + Q4_STAGE_S + Q4_STAGE_B;    // 45056
constexpr int Q4_STAGES = 3;

struct Q4Args {
    const uint8_t* const* eptr;
    const int* list;
    const int* chunk_expert;
    const int* chunk_start;
    const int* chunk_n;
    const int* nchunks;
    int topk;
    int pair;                 // 1: rows are (gate i, up i) pairs -> act; 0: down rows -> ypart
    int rows, K;              // output rows (I pairs, or D) and contraction length (D, or I)
    size_t off_q, off_s, off_m;   // sections of this matrix inside an expert
    int up_row0;              // pair mode: first up row (= I)
    const __half* xh;         // activations: [token or pick][2][K] fp16 hi | lo
    const float* xsum;        // [token or pick][K / 64] sums of the activations per group
    int by_pick;              // 0: xh / xsum are indexed by token (p / topk); 1: by pick
    float* out;               // pair: act [P][rows]; down: ypart [T][topk + 1][rows]
};

// four codes (two bytes: c0 | c1 << 4, c2 | c3 << 4) -> two half2, exact
__device__ __forceinline__ void q4x4_to_h2x2(uint32_t two_bytes, uint32_t& h01, uint32_t& h23) {
    const uint32_t magic = 0x64006400u, bias = 0x64006400u;     // 1024 + code, minus 1024
    uint32_t a = (two_bytes & 0x0000000Fu) | ((two_bytes << 12) & 0x000F0000u) | magic;
    uint32_t b = ((two_bytes >> 8) & 0x0000000Fu) | ((two_bytes << 4) & 0x000F0000u) | magic;
    __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<const __half2*>(&bias));
    __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), *reinterpret_cast<const __half2*>(&bias));
    h01 = *reinterpret_cast<uint32_t*>(&ha);
    h23 = *reinterpret_cast<uint32_t*>(&hb);
}

// grid (row blocks, max chunks)
__global__ void __launch_bounds__(MM_THREADS) k_mma_q4(const Q4Args a) {
    extern __shared__ __align__(128) unsigned char q4_smem[];
    __shared__ int s_pick[GQ_CH];
    __shared__ float s_xsum[GQ_CH][33];          // [sequence of the chunk][group]
    __shared__ float gate_s[2][16][MM_TOK + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid = lane & 3;
    grid_dep_launch();
    grid_dep_wait();
    const int chunk = blockIdx.y;
    if (chunk >= *a.nchunks) return;
    const int e = a.chunk_expert[chunk];
    const int n = a.chunk_n[chunk];
    const uint8_t* base = a.eptr[e];
    if (threadIdx.x < GQ_CH) s_pick[threadIdx.x] = threadIdx.x < n ? a.list[a.chunk_start[chunk] + threadIdx.x] : -1;
    __syncthreads();
    const int rows_per_block = a.pair ? Q4_ROWS / 2 : Q4_ROWS;
    const int row0 = blockIdx.x * rows_per_block;
    const int ngroup = a.K >> 6;                 // <= 32
    for (int p = threadIdx.x; p < GQ_CH * ngroup; p += MM_THREADS) {
        const int c = p / ngroup, g = p % ngroup;
        const int pk = s_pick[c];
        s_xsum[c][g] = pk < 0 ? 0.f : a.xsum[(size_t)(a.by_pick ? pk : pk / a.topk) * ngroup + g];
    }
    const int rowbytes = a.K >> 1;
    const int nk = a.K / MM_KC;

    auto weight_row = [&](int r) {          // shared-memory row r of the block -> row of the matrix
        int g = a.pair ? (r < 32 ? row0 + r : a.up_row0 + row0 + (r - 32)) : row0 + r;
        const int last = a.pair ? (r < 32 ? a.rows - 1 : a.up_row0 + a.rows - 1) : a.rows - 1;
        return min(g, last);
    };
    auto load_stage = [&](int kc, int st) {
        unsigned char* sa = q4_smem + (size_t)st * Q4_STAGE_BYTES;
        unsigned char* ss = sa + Q4_STAGE_A;
        unsigned char* sb = ss + Q4_STAGE_S;
        for (int p = threadIdx.x; p < Q4_ROWS * 8; p += MM_THREADS) {          // codes: 64 rows x 128 B
            const int r = p >> 3, c = p & 7;
            cp_async16(sa + r * Q4_PA + c * 16, base + a.off_q + (size_t)weight_row(r) * rowbytes + (size_t)kc * 128 + c * 16);
        }
        for (int p = threadIdx.x; p < Q4_ROWS * 2; p += MM_THREADS) {          // scales and mins: 8 B each per row
            const int r = p >> 1, which = p & 1;
            const uint8_t* src = base + (which ? a.off_m : a.off_s) + ((size_t)weight_row(r) * ngroup + (size_t)kc * 4) * 2;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(ss + r * 16 + which * 8)), "l"(src) : "memory");
        }
        for (int p = threadIdx.x; p < 2 * MM_TOK * (MM_KC / 8); p += MM_THREADS) {
            const int col = p / (MM_KC / 8), c = p % (MM_KC / 8);
            const int pk = s_pick[col & (MM_TOK - 1)], part = col >> 5;
            const int src_row = pk < 0 ? 0 : (a.by_pick ? pk : pk / a.topk);     // unused columns read row 0 (never stored)
            cp_async16(sb + col * MM_PB + c * 16, a.xh + ((size_t)src_row * 2 + part) * a.K + (size_t)kc * MM_KC + c * 8);
        }
        cp_async_commit();
    };
    for (int i = 0; i < Q4_STAGES - 1; i++) {
        if (i < nk) load_stage(i, i); else cp_async_commit();
    }
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[j][q] = 0.f;

    for (int kc = 0; kc < nk; kc++) {
        cp_async_wait<Q4_STAGES - 2>();
        __syncthreads();
        if (kc + Q4_STAGES - 1 < nk) load_stage(kc + Q4_STAGES - 1, (kc + Q4_STAGES - 1) % Q4_STAGES); else cp_async_commit();
        const unsigned char* sa = q4_smem + (size_t)(kc % Q4_STAGES) * Q4_STAGE_BYTES;
        const unsigned char* ss = sa + Q4_STAGE_A;
        const unsigned char* sb = ss + Q4_STAGE_S;
        const int r0 = warp * 16 + gid, r1 = r0 + 8;
#pragma unroll
        for (int sbk = 0; sbk < 4; sbk++) {            // one 64-value group per super-block
            const uint2 w0 = *reinterpret_cast<const uint2*>(sa + r0 * Q4_PA + sbk * 32 + tid * 8);
            const uint2 w1 = *reinterpret_cast<const uint2*>(sa + r1 * Q4_PA + sbk * 32 + tid * 8);
            uint32_t af[4][4];
            q4x4_to_h2x2(w0.x & 0xFFFFu, af[0][0], af[0][2]); q4x4_to_h2x2(w0.x >> 16, af[1][0], af[1][2]);
            q4x4_to_h2x2(w0.y & 0xFFFFu, af[2][0], af[2][2]); q4x4_to_h2x2(w0.y >> 16, af[3][0], af[3][2]);
            q4x4_to_h2x2(w1.x & 0xFFFFu, af[0][1], af[0][3]); q4x4_to_h2x2(w1.x >> 16, af[1][1], af[1][3]);
            q4x4_to_h2x2(w1.y & 0xFFFFu, af[2][1], af[2][3]); q4x4_to_h2x2(w1.y >> 16, af[3][1], af[3][3]);
            const float s0 = h2f(*reinterpret_cast<const uint16_t*>(ss + r0 * 16 + sbk * 2));
            const float m0 = h2f(*reinterpret_cast<const uint16_t*>(ss + r0 * 16 + 8 + sbk * 2));
            const float s1 = h2f(*reinterpret_cast<const uint16_t*>(ss + r1 * 16 + sbk * 2));
            const float m1 = h2f(*reinterpret_cast<const uint16_t*>(ss + r1 * 16 + 8 + sbk * 2));
            const int grp = kc * 4 + sbk;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                float t[4] = {0.f, 0.f, 0.f, 0.f};
                const unsigned char* bp = sb + (nt * 8 + gid) * MM_PB + sbk * 128 + tid * 32;
                const uint4 x0 = *reinterpret_cast<const uint4*>(bp);
                const uint4 x1 = *reinterpret_cast<const uint4*>(bp + 16);
                mma16816(t, af[0], x0.x, x0.y);
                mma16816(t, af[1], x0.z, x0.w);
                mma16816(t, af[2], x1.x, x1.y);
                mma16816(t, af[3], x1.z, x1.w);
                acc[nt][0] = fmaf(s0, t[0], acc[nt][0]); acc[nt][1] = fmaf(s0, t[1], acc[nt][1]);
                acc[nt][2] = fmaf(s1, t[2], acc[nt][2]); acc[nt][3] = fmaf(s1, t[3], acc[nt][3]);
            }
#pragma unroll
            for (int nt = 0; nt < 4; nt++)             // min term, once per sequence (hi columns)
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const float xs = s_xsum[nt * 8 + 2 * tid + c][grp];
                    acc[nt][c] = fmaf(m0, xs, acc[nt][c]);
                    acc[nt][2 + c] = fmaf(m1, xs, acc[nt][2 + c]);
                }
        }
    }
    cp_async_wait<0>();

    if (a.pair && warp < 2) {
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int q = 0; q < 4; q++) gate_s[warp][gid + (q >> 1) * 8][nt * 8 + 2 * tid + (q & 1)] = acc[nt][q] + acc[nt + 4][q];
    }
    if (a.pair) __syncthreads();
    if (a.pair && warp < 2) return;
#pragma unroll
    for (int nt = 0; nt < 4; nt++)
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int rl = gid + (q >> 1) * 8, col = nt * 8 + 2 * tid + (q & 1);
            const int pk = s_pick[col];
            const int row = a.pair ? row0 + (warp - 2) * 16 + rl : row0 + warp * 16 + rl;
            if (pk < 0 || row >= a.rows) continue;
            const float dot = acc[nt][q] + acc[nt + 4][q];
            if (a.pair) a.out[(size_t)pk * a.rows + row] = siluf_(gate_s[warp - 2][rl][col]) * dot;
            else a.out[((size_t)(pk / a.topk) * (a.topk + 1) + pk % a.topk) * a.rows + row] = dot;
        }
}

}  // namespace b2
