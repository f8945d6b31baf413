// k_umma_q4: the 4-bit experts of a step (6 or more tokens) as a grouped Blackwell tensor-core GEMM
// (the reference's expert GEMMs for more than 8 tokens, aegist_rs/kernels/hybrid.cu:461-549).
//
// k_group_picks has sorted the step's picks by expert and cut every expert's list into chunks of at most 16 picks. A
// unit of work is (chunk, block of 128 weight rows): out[pick][row] = sum_k w[row][k] x[pick][k] for the chunk's picks,
// with w = code * scale_g + min_g per 64-value group g (aegist/hybrid.py ExpertBank), so
//     sum_k w x = sum_g ( scale_g * sum_{k in g} code x  +  min_g * sum_{k in g} x ).
// The integer sums of a group must not mix with another group's, so every group gets its own accumulator columns in
// tensor memory and the epilogue folds them with the group's fp16 scale:
//
//   producer warp     TMA tensor copies per K step (256 codes = 4 groups): the packed codes of 128 rows (128 bytes each,
//                     straight from the expert's blob through a 3-D tensor map [expert][row][byte]) and the three int8
//                     digit planes of the chunk's picks. The planes are stored in sorted-pick order with the three planes
//                     of a pick's 128 values next to each other, so a chunk's operand tile is 6 KB of consecutive memory
//                     and one copy (as 96 separate 128-byte rows the plane copies took longer than everything else
//                     together). The ring is 5 steps deep: about 80 KB of weights per SM in flight
//   4 converter warps the codes' nibbles -> int8 (0..15) in the 128-byte-swizzled layout tcgen05.mma reads (one of two
//                     buffers), then fence.proxy.async and an mbarrier arrival
//   MMA warp          per group two tcgen05.mma (kind::i8, M 128, N 48, K 32) into that group's 48 columns of one of two
//                     accumulator buffers; tcgen05.commit frees the ring step and the code buffer and hands the
//                     accumulators to the epilogue
//   4 epilogue warps  thread = weight row = TMEM lane: tcgen05.ld of the group's columns, planes combined per pick, times
//                     the row's group scale, plus the group minimum times the pick's group sum; after the last K step the
//                     pick's activation scale, then silu(gate) * up (pairs) or the pick's output row (down)
//
// Every wait is a bounded mbarrier wait; a thread whose wait gave up skips its later waits, the producer stops issuing
// copies and drains those in flight, and the kernel ends normally with the error word set.
#pragma once

namespace b2 {

constexpr int UQ_TT = 16;                        // picks per unit (a chunk of the pick list)
constexpr int UQ_NCOL = UQ_TT * UM_PI;           // 48 accumulator columns per group
constexpr int UQ_KB = 256;                       // codes per ring step: two 128-byte-wide sub-tiles, four groups
constexpr int UQ_RAW = UM_M * UQ_KB / 2;         // 16 KB: packed codes of a step
constexpr int UQ_BSUB = UQ_NCOL * UM_BK;         // 6 KB: one sub-tile of the planes
constexpr int UQ_LOAD = UQ_RAW + 2 * UQ_BSUB;    // 28 KB per ring step
constexpr int UQ_STAGES = 5;
constexpr int UQ_ASUB = UM_M * UM_BK;            // 16 KB: one sub-tile of the codes as int8
constexpr int UQ_ABUF = 2;                       // code buffers
constexpr int UQ_GCOL = 64;                      // columns between the groups' accumulators: a tcgen05.mma whose accumulator does not start on a
                                                 // multiple of the next power of two above N takes about three times as long
constexpr int UQ_ACC = 4 * UQ_GCOL;              // 256 accumulator columns per buffer
constexpr int UQ_THREADS = 320;                  // producer, MMA, 4 converter warps, 4 epilogue warps
constexpr size_t UQ_SMEM = (size_t)UQ_STAGES * UQ_LOAD + (size_t)UQ_ABUF * 2 * UQ_ASUB + 1024;
constexpr int UQ_MAXG = 32;                      // groups of a row (K <= 2048)

struct UmmaQ4Args {
    CUtensorMap wmap;         // this matrix's packed codes of the layer's experts: [expert][row][K / 2 bytes], box 128 B x 64 rows
    CUtensorMap xmap;         // planes [K / 128][slots][3][128 bytes] as rows of 128 bytes; box 48 rows (16 slots), 128-byte swizzle
    unsigned long long* trace;
    const uint8_t* const* eptr;   // [E] expert blobs (for the scale and min rows)
    const int* list;          // pick ids sorted by expert (k_group_picks)
    ChunkTable small, big;
    int topk, pair, rows, K;  // pair: rows = pairs (expert_hidden), gate row i and up row up_row0 + i; else rows = output rows
    int up_row0;
    int rbu;                  // row blocks one unit walks through with the same picks (a short K gives short units otherwise)
    int e0;                   // first expert that lives on this GPU (its blob is index 0 of the tensor map)
    size_t off_s, off_m;      // the matrix's scale and min sections inside an expert blob
    int slots;                // capacity of the planes (rows per plane)
    const float* xscale;      // [slots] scale of each slot's planes
    const float* xsum;        // [slots][K / 64] sum of each 64-value group of the slot's activations
    float* out;               // pair: act [picks][rows]; else ypart [tokens][topk + 1][rows]
    int* err;
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}

__global__ void __launch_bounds__(UQ_THREADS, 1) k_umma_q4(const __grid_constant__ UmmaQ4Args a) {
    extern __shared__ unsigned char uq_raw[];
    __shared__ __align__(8) uint64_t full_bar[UQ_STAGES], empty_bar[UQ_STAGES], conv_bar[UQ_ABUF], a_empty[UQ_ABUF], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) float s_xsum[UQ_TT][UQ_MAXG + 4];
    __shared__ float s_xscale[UQ_TT];
    __shared__ int s_dst[UQ_TT];                     // output row index of each pick of the chunk (-1: not a pick)
    __shared__ float gate_x[64][UQ_TT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* ring = uq_raw + ((1024u - (smem_u32(uq_raw) & 1023u)) & 1023u);
    unsigned char* abuf = ring + (size_t)UQ_STAGES * UQ_LOAD;
    grid_dep_launch();
    trace_in(a.trace, 16, gridDim.x);
    if (threadIdx.x == 0) {
        for (int s = 0; s < UQ_STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < UQ_ABUF; b++) { mbar_init(&conv_bar[b], 4); mbar_init(&a_empty[b], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    grid_dep_wait();                                 // the chunk tables, the planes and the activations are earlier launches' results

    const int nbig = *a.big.count, nsmall = *a.small.count;
    const int RB = a.pair ? (a.rows + 63) / 64 : (a.rows + UM_M - 1) / UM_M;      // row blocks
    const int RBU = max(1, a.rbu), RG = (RB + RBU - 1) / RBU;                     // row blocks per unit, units per chunk
    const int nwork = (nbig + nsmall) * RG;          // big chunks first: they are the long ones
    const int nk = a.K / UQ_KB;                      // ring steps per unit
    const int ngroup = a.K >> 6;
    auto chunk_of = [&](int w, int& e, int& start, int& n, int& rb) {      // rb: the unit's first row block
        const int c = w / RG;
        rb = (w - c * RG) * RBU;
        const ChunkTable& t = c < nbig ? a.big : a.small;
        const int i = c < nbig ? c : c - nbig;
        e = t.expert[i]; start = t.start[i]; n = t.n[i];
    };
    auto wait = [&](uint64_t* bar, uint32_t parity, bool& dead) {
        if (dead) return;
        if (!mbar_wait(bar, parity, a.err, 1 << 21)) dead = true;
    };

    if (warp == 0) {
        // ---- producer: lane 0 waits and announces, lanes 0..3 issue one copy each ----
        int st = 0, ph = 0;
        bool dead = false;
        uint32_t armed_mask = 0, armed_par = 0;
        for (int w = blockIdx.x; w < nwork; w += gridDim.x) {
            int e, start, n, rb;
            chunk_of(w, e, start, n, rb);
            for (int rbi = 0; rbi < RBU && rb + rbi < RB && !dead; rbi++) {
            const int r0 = rb + rbi;
            const int y = a.pair ? (lane == 0 ? r0 * 64 : a.up_row0 + r0 * 64) : r0 * UM_M + lane * 64;      // lanes 0, 1: the two row halves
            for (int kc = 0; kc < nk; kc++) {
                if (lane == 0) {
                    wait(&empty_bar[st], ph ^ 1, dead);
                    if (!dead) mbar_expect_tx(&full_bar[st], UQ_LOAD);
                }
                dead = __shfl_sync(0xffffffffu, (int)dead, 0) != 0;
                if (dead) break;
                unsigned char* sb = ring + (size_t)st * UQ_LOAD;
                if (lane < 2) tma_load_3d(sb + lane * (UQ_RAW / 2), &a.wmap, kc * (UQ_KB / 2), y, e - a.e0, &full_bar[st]);
                else if (lane < 4) tma_load_2d(sb + UQ_RAW + (lane - 2) * UQ_BSUB, &a.xmap, 0, ((kc * 2 + lane - 2) * a.slots + start) * UM_PI, &full_bar[st]);
                armed_mask |= 1u << st;
                armed_par = (armed_par & ~(1u << st)) | ((uint32_t)ph << st);
                if (++st == UQ_STAGES) { st = 0; ph ^= 1; }
            }
            }
            if (dead) break;
        }
        __syncwarp();
        if (lane == 0 && dead)
            for (int i = 0; i < UQ_STAGES; i++)
                if (armed_mask >> i & 1) mbar_wait(&full_bar[i], (armed_par >> i) & 1u, nullptr, 1 << 16);
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            int st = 0, ph = 0, n = 0;
            bool dead = false;
            const uint32_t idesc = umma_idesc(2, 1, UM_M, UQ_NCOL);
            for (int w = blockIdx.x; w < nwork; w += gridDim.x) {
                int e, start, cn, rb;
                chunk_of(w, e, start, cn, rb);
                const int steps = nk * min(RBU, RB - rb);
                for (int kc = 0; kc < steps; kc++, n++) {
                    const int buf = n & 1;
                    wait(&acc_empty[buf], ((n >> 1) & 1) ^ 1, dead);        // the epilogue has folded this buffer's groups
                    wait(&conv_bar[buf], (n >> 1) & 1, dead);               // codes converted (and, before that, planes landed)
                    tc_fence_after();
                    const uint32_t sa = smem_u32(abuf + (size_t)buf * 2 * UQ_ASUB), sb = smem_u32(ring + (size_t)st * UQ_LOAD + UQ_RAW);
#pragma unroll
                    for (int g = 0; g < 4; g++) {    // group g: sub-tile g / 2, bytes 64 (g % 2) .. + 63 of its rows, two K 32 steps
                        const uint64_t ad = umma_desc_sw128(sa + (g >> 1) * UQ_ASUB) + 4 * (g & 1), bd = umma_desc_sw128(sb + (g >> 1) * UQ_BSUB) + 4 * (g & 1);
                        umma_i8(tmem + (uint32_t)buf * UQ_ACC + (uint32_t)g * UQ_GCOL, ad, bd, idesc, 0u);
                        umma_i8(tmem + (uint32_t)buf * UQ_ACC + (uint32_t)g * UQ_GCOL, ad + 2, bd + 2, idesc, 1u);
                    }
                    umma_commit(&empty_bar[st]);
                    umma_commit(&a_empty[buf]);
                    umma_commit(&acc_full[buf]);
                    if (++st == UQ_STAGES) { st = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp < 6) {
        // ---- converters: 16 packed bytes -> 32 int8 codes, written where the 128-byte swizzle puts them ----
        const int cw = warp - 2;
        int st = 0, ph = 0, n = 0;
        bool dead = false;
        for (int w = blockIdx.x; w < nwork; w += gridDim.x) {
            int e, start, cn, rb;
            chunk_of(w, e, start, cn, rb);
            const int steps = nk * min(RBU, RB - rb);
            for (int kc = 0; kc < steps; kc++, n++) {
                const int buf = n & 1;
                wait(&full_bar[st], ph, dead);
                wait(&a_empty[buf], ((n >> 1) & 1) ^ 1, dead);              // the MMAs that read this code buffer are done
                const unsigned char* raw = ring + (size_t)st * UQ_LOAD;
                unsigned char* ab = abuf + (size_t)buf * 2 * UQ_ASUB;
                // eight neighbouring lanes take two rows and, of each, the four 16-byte pieces of one sub-tile: their loads
                // cover all 32 banks once, and so do their swizzled stores (rows r and r + 1 differ in the low swizzle bit).
                // 16 bytes q of row r are codes 32 q .. 32 q + 31. All loads first: the stores cannot be proven not to alias.
                const int hf = (lane >> 2) & 1;
                uint4 pk[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int r = cw * 32 + (j >> 1) * 8 + (lane >> 3) * 2 + hf, q = (lane & 3) + 4 * (hf ^ (j & 1));
                    pk[j] = *reinterpret_cast<const uint4*>(raw + r * 128 + q * 16);
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int r = cw * 32 + (j >> 1) * 8 + (lane >> 3) * 2 + hf, q = (lane & 3) + 4 * (hf ^ (j & 1));
                    const uint32_t pw[4] = {pk[j].x, pk[j].y, pk[j].z, pk[j].w};
                    uint32_t o[8];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t lo = pw[i] & 0x0F0F0F0Fu, hi = (pw[i] >> 4) & 0x0F0F0F0Fu;    // even codes | odd codes
                        o[2 * i] = __byte_perm(lo, hi, 0x5140);
                        o[2 * i + 1] = __byte_perm(lo, hi, 0x7362);
                    }
                    unsigned char* row = ab + (q >> 2) * UQ_ASUB + r * UM_BK;
                    const int u = 2 * (q & 3);
                    *reinterpret_cast<uint4*>(row + ((u ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4*>(row + (((u + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the tensor core reads through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&conv_bar[buf]);
                if (++st == UQ_STAGES) { st = 0; ph ^= 1; }
            }
        }
    } else {
        // ---- epilogue: warp w may touch TMEM lanes 32 (w % 4) .. + 31 ----
        const int q = warp & 3;
        const int vrow = q * 32 + lane;
        const int et = threadIdx.x - 6 * 32;         // 0..127 among the epilogue threads
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        int n = 0;
        bool dead = false;
        // a unit's picks are fetched into registers while the unit before it runs
        struct Pre { int e, start, cn, rb, p; float xs; const uint8_t* blob; float v[4], vs[4]; } P;
        auto prefetch = [&](int w) {
            P.cn = 0; P.e = -1; P.blob = nullptr;
            if (w >= nwork) return;
            chunk_of(w, P.e, P.start, P.cn, P.rb);
            P.blob = a.eptr[P.e];
            const bool live = et < P.cn;                                         // et >= 16 is never live
            P.p = live ? a.list[P.start + et] : -1;
            P.xs = live ? a.xscale[P.start + et] : 0.f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int i = et + 128 * j, t = i / ngroup, g = i - t * ngroup;
                const bool ok = i < UQ_TT * ngroup && t < P.cn;
                P.v[j] = ok ? a.xsum[(size_t)(P.start + t) * ngroup + g] : 0.f;
                P.vs[j] = ok ? a.xscale[P.start + t] : 0.f;
            }
        };
        prefetch(blockIdx.x);
        for (int w = blockIdx.x; w < nwork; w += gridDim.x) {
            const int cn = P.cn, rb0 = P.rb;
            const uint8_t* blob = P.blob;
            asm volatile("bar.sync 3, 128;" ::: "memory");                      // the previous unit's readers are done
            if (et < UQ_TT) {
                s_xscale[et] = P.xs;
                s_dst[et] = P.p >= 0 ? (a.pair ? P.p : (P.p / a.topk) * (a.topk + 1) + P.p % a.topk) : -1;
            }
            // group sums in units of the pick's scale, so that the scale multiplies once at the end
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int i = et + 128 * j, t = i / ngroup, g = i - t * ngroup;
                if (i < UQ_TT * ngroup) s_xsum[t][g] = P.vs[j] > 0.f ? P.v[j] / P.vs[j] : 0.f;
            }
            asm volatile("bar.sync 3, 128;" ::: "memory");
            prefetch(w + gridDim.x);
            for (int rbi = 0; rbi < RBU && rb0 + rbi < RB; rbi++) {
                const int rb = rb0 + rbi;
                const int row = a.pair ? (vrow < 64 ? rb * 64 + vrow : a.up_row0 + rb * 64 + vrow - 64) : rb * UM_M + vrow;
                const int orow = a.pair ? rb * 64 + (vrow & 63) : rb * UM_M + vrow;      // row of the output
                const bool rok = a.pair ? orow < a.rows : row < a.rows;
                const uint16_t* srow = reinterpret_cast<const uint16_t*>(blob + a.off_s) + (size_t)(rok ? row : 0) * ngroup;
                const uint16_t* mrow = reinterpret_cast<const uint16_t*>(blob + a.off_m) + (size_t)(rok ? row : 0) * ngroup;
                // a step's four groups of the row: scale and min (fp16), requested one step ahead
                uint2 s4n = *reinterpret_cast<const uint2*>(srow), m4n = *reinterpret_cast<const uint2*>(mrow);
                float acc[UQ_TT];
#pragma unroll
                for (int t = 0; t < UQ_TT; t++) acc[t] = 0.f;
                for (int kc = 0; kc < nk; kc++, n++) {
                    const int buf = n & 1;
                    const uint2 s4 = s4n, m4 = m4n;
                    if (kc + 1 < nk) { s4n = *reinterpret_cast<const uint2*>(srow + 4 * (kc + 1)); m4n = *reinterpret_cast<const uint2*>(mrow + 4 * (kc + 1)); }
                    wait(&acc_full[buf], (n >> 1) & 1, dead);
                    tc_fence_after();
                    float xs4[UQ_TT][4];             // the picks' sums of this step's four groups
#pragma unroll
                    for (int i = 0; i < UQ_TT; i++) {
                        const float4 t4 = *reinterpret_cast<const float4*>(&s_xsum[i][4 * kc]);
                        xs4[i][0] = t4.x; xs4[i][1] = t4.y; xs4[i][2] = t4.z; xs4[i][3] = t4.w;
                    }
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        // the three plane sums of a group are below 2^16 in magnitude (64 codes of at most 15 times digits of
                        // at most 64), so d0 2^14 + d1 2^7 + d2 fits an int; 2^-14 goes into the row's scale
                        const uint32_t sw = g < 2 ? s4.x : s4.y, mw = g < 2 ? m4.x : m4.y;
                        const float sc = h2f((uint16_t)(g & 1 ? sw >> 16 : sw & 0xFFFFu)) * (1.0f / 16384.0f), mn = h2f((uint16_t)(g & 1 ? mw >> 16 : mw & 0xFFFFu));
                        const uint32_t base = tmem + lane_addr + (uint32_t)buf * UQ_ACC + (uint32_t)g * UQ_GCOL;
                        uint32_t d[3][16];               // column 3 t + p: plane p of pick t
                        tmem_ld16(base, d[0]);
                        tmem_ld16(base + 16, d[1]);
                        tmem_ld16(base + 32, d[2]);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const int c = 3 * i;
                            const int v = (int)d[c >> 4][c & 15] * 16384 + ((int)d[(c + 1) >> 4][(c + 1) & 15] * 128 + (int)d[(c + 2) >> 4][(c + 2) & 15]);
                            acc[i] = fmaf(sc, (float)v, fmaf(mn, xs4[i][g], acc[i]));
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                    if (kc == 0 && rbi == 0 && P.blob) {
                        // the next unit's scale and min rows towards L2 (they are touched nowhere else before)
                        for (int k = 0; k < RBU && P.rb + k < RB; k++) {
                            const int r2 = a.pair ? (vrow < 64 ? (P.rb + k) * 64 + vrow : a.up_row0 + (P.rb + k) * 64 + vrow - 64) : (P.rb + k) * UM_M + vrow;
                            if (a.pair ? (P.rb + k) * 64 + (vrow & 63) < a.rows : r2 < a.rows) {
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(P.blob + a.off_s + (size_t)r2 * ngroup * 2));
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(P.blob + a.off_m + (size_t)r2 * ngroup * 2));
                            }
                        }
                    }
                }
#pragma unroll
                for (int t = 0; t < UQ_TT; t++) acc[t] *= s_xscale[t];
                // results: act = silu(gate) * up per pick (pairs), or the pick's row of ypart
                if (a.pair) {
                    if (rbi > 0) asm volatile("bar.sync 3, 128;" ::: "memory");     // the previous row block's readers of gate_x
                    if (vrow < 64) {
#pragma unroll
                        for (int t = 0; t < UQ_TT; t++) gate_x[vrow][t] = acc[t];
                    }
                    asm volatile("bar.sync 3, 128;" ::: "memory");
                    if (vrow >= 64 && rok) {
#pragma unroll
                        for (int t = 0; t < UQ_TT; t++)
                            if (s_dst[t] >= 0) a.out[(size_t)s_dst[t] * a.rows + orow] = siluf_(gate_x[vrow - 64][t]) * acc[t];
                    }
                } else if (rok) {
#pragma unroll
                    for (int t = 0; t < UQ_TT; t++)
                        if (s_dst[t] >= 0) a.out[(size_t)s_dst[t] * a.rows + orow] = acc[t];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { __syncwarp(); tmem_dealloc(tmem, 512); }
    trace_out(a.trace);
}

// ---- the activations of the sorted picks as planes -----------------------------------------------------------
struct PrepSlotsArgs {
    unsigned long long* trace;
    const float* src;         // [rows][stride]: by_pick ? one row per pick : one row per token
    int stride, by_pick, topk;
    const uint16_t* norm_w;   // ZNorm weight [K] or null
    float eps;
    int K, P;                 // P = pick slots
    const int* list;          // [P] pick ids in sorted order (entries past the step's picks are stale but in range)
    int8_t* qi;               // [K / 128][slots][3][128]: the three planes of a slot's 128 values lie together, a chunk's picks in a row
    int slots;
    float* xscale;            // [slots]
    float* xsum;              // [slots][K / 64]
};

// one block of 256 threads per slot; K <= 2048
__global__ void __launch_bounds__(256) k_prep_q_slots(const PrepSlotsArgs a) {
    __shared__ float red[2][8];
    const int s = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    grid_dep_launch();
    trace_in(a.trace, 17, gridDim.x);
    grid_dep_wait();
    const int p = min(max(a.list[s], 0), a.P - 1);
    const float* x = a.src + (size_t)(a.by_pick ? p : p / a.topk) * a.stride;
    const int k = threadIdx.x * 8;
    float xv[8];
    float ss = 0.f;
    {
        float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
        if (k < a.K) { v0 = *reinterpret_cast<const float4*>(x + k); v1 = *reinterpret_cast<const float4*>(x + k + 4); }
        xv[0] = v0.x; xv[1] = v0.y; xv[2] = v0.z; xv[3] = v0.w; xv[4] = v1.x; xv[5] = v1.y; xv[6] = v1.z; xv[7] = v1.w;
        if (a.norm_w) {
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (k < a.K) wv = *reinterpret_cast<const uint4*>(a.norm_w + k);
            const float nw[8] = {1.0f + bflo(wv.x), 1.0f + bfhi(wv.x), 1.0f + bflo(wv.y), 1.0f + bfhi(wv.y),
                                 1.0f + bflo(wv.z), 1.0f + bfhi(wv.z), 1.0f + bflo(wv.w), 1.0f + bfhi(wv.w)};
#pragma unroll
            for (int i = 0; i < 8; i++) { ss = fmaf(xv[i], xv[i], ss); xv[i] *= nw[i]; }
        }
    }
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(xv[i]));
    ss = warp_sum(ss);
    mx = warp_max(mx);
    if (lane == 0) { red[0][warp] = ss; red[1][warp] = mx; }
    __syncthreads();
    ss = 0.f; mx = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) { ss += red[0][w]; mx = fmaxf(mx, red[1][w]); }
    if (a.norm_w) {
        const float rn = 1.0f / sqrtf(ss / (float)a.K + a.eps);
#pragma unroll
        for (int i = 0; i < 8; i++) xv[i] *= rn;
        mx *= rn;
    }
    const float inv = mx > 1e-30f ? 127.0f / mx : 0.f;
    if (threadIdx.x == 0) a.xscale[s] = mx / 127.0f;
    // the sum of a 64-value group: 8 neighbouring lanes, values in index order within a lane
    float s8 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) s8 += xv[i];
    s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
    s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
    s8 += __shfl_xor_sync(0xffffffffu, s8, 4);
    if (k < a.K) {
        if ((lane & 7) == 0) a.xsum[(size_t)s * (a.K >> 6) + (k >> 6)] = s8;
        uint32_t w[UM_PI][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int qv = __float2int_rn(xv[i] * inv * 16384.0f);
            const int d2 = ((qv + 64) & 127) - 64;
            qv = (qv - d2) >> 7;
            const int d1 = ((qv + 64) & 127) - 64;
            const int d0 = (qv - d1) >> 7;
            const int sh = 8 * (i & 3);
            w[0][i >> 2] |= (uint32_t)(d0 & 255) << sh; w[1][i >> 2] |= (uint32_t)(d1 & 255) << sh; w[2][i >> 2] |= (uint32_t)(d2 & 255) << sh;
        }
#pragma unroll
        for (int pl = 0; pl < UM_PI; pl++)
            *reinterpret_cast<uint2*>(a.qi + ((((size_t)(k >> 7) * a.slots + s) * UM_PI + pl) << 7) + (k & 127)) = make_uint2(w[pl][0], w[pl][1]);
    }
    trace_out(a.trace);
}

}  // namespace b2
