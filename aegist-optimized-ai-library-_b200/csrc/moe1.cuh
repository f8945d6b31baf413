// The routed experts of one layer for a handful of tokens (fewer than 6 in the engine, up to 7), as two kernels whose work
// is spread evenly over the GPU instead of one block per pick:
//
//   k_moe_gu1    every block: router softmax + top-8 from the logits (redundantly, which replaces a
//                last-block finisher and its fence + atomic + reload), norm2(x) as int8 digit planes, then
//                32 of the token's topk * I (gate, up) row pairs, fetched in one go with 16-byte
//                asynchronous copies and multiplied on the tensor cores; act = silu(gate) * up leaves the
//                block as digit planes of its own (one scale per 32 values) for the down projection
//   k_moe_down1  one block per 16 output rows: two warps per pick multiply those rows of the pick's down
//                matrix with its act planes, two more the shared expert's rows, and the block adds the 9
//                parts in rank order into the residual stream (no cross-block combine)
//
// Arithmetic: the 4-bit codes (0..15) and the int8 weights go to mma.sync.m16n8k32.s8 unchanged; the
// activations are split into four int8 digit planes, x = scale * (d0 + d1/128 + d2/128^2 + d3/128^3)
// with scale = max|x| / 127, which holds every fp32 activation to 2^-22 of the largest one; the planes
// are four of the eight B columns. The integer sums are exact; per 64-value group they are scaled by
// the group's fp16 scale, and the group minimum times the group's activation sum is added
// (w = code * s + m, aegist/hybrid.py ExpertBank).
#pragma once

namespace b2 {

constexpr int M1_GU_WARPS = 32;           // 4 blocks of 8 pairs x 8 eighths of K
constexpr int M1_GU_THREADS = M1_GU_WARPS * 32;
constexpr int M1_GU_PAIRS = 32;           // pairs per block of k_moe_gu1: one 32-value group of act
constexpr int M1_DOWN_ROWS = 16;
constexpr int M1_DOWN_WARPS = 18;         // (8 picks + shared) x 2 halves of K

// n fp16 values global -> shared: asynchronous 16-byte pieces when n is a multiple of 8, plain loads otherwise;
// piece `c` of the (n * 2 + 15) / 16 pieces of the row
__device__ __forceinline__ void copy_f16_piece(uint16_t* dst, const uint8_t* src, int n, int c) {
    if ((n & 7) == 0) {
        cp_async16(reinterpret_cast<unsigned char*>(dst) + c * 16, src + (size_t)c * 16);
    } else {
        const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
        for (int i = 8 * c; i < min(n, 8 * c + 8); i++) dst[i] = s[i];
    }
}
// Scale rows in shared memory: per row [scales | mins] of ngroup fp16 each, in 16-byte pieces; piece q of row
// `slot` sits at position q ^ (slot & mask), so that the same piece of 8 neighbouring rows covers all banks.
// mask = pieces per row - 1 (at most 7) when the pieces per row are a power of two, else 0.
__device__ __forceinline__ int sc_mask(int ngroup) {
    const int npq = 2 * ((ngroup * 2 + 15) >> 4);
    return ((ngroup & 7) == 0 && (npq & (npq - 1)) == 0) ? min(npq, 8) - 1 : 0;
}
// address (in fp16 units, relative to the row) of value g of part `which` (0 scales, 1 mins)
__device__ __forceinline__ int sc_pos(int ngroup, int mask, int slot, int which, int g) {
    if (mask == 0) return which * ngroup + g;
    const int q = which * (ngroup >> 3) + (g >> 3);
    return ((q ^ (slot & mask)) << 3) + (g & 7);
}
// Softmax over E <= 256 router logits and the topk <= 8 largest in descending order, ties to the lower
// index, weights renormalised over the picks (aegist/hybrid.py:641-645); one warp, the same values as
// router_topk_warp. A probability is positive, so its bits order like an unsigned integer: a round is two
// warp-wide integer reductions (largest key, then lowest expert holding it) instead of shuffle ladders.
// Pick r ends up in lane r.
__device__ __forceinline__ void router_topk_lanes(const float* __restrict__ logits, int E, int topk, int lane, int& my_e, float& my_w) {
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
    uint32_t key[8];                     // bits of the probability + 1; 0 = not available
#pragma unroll
    for (int i = 0; i < 8; i++) key[i] = (lane + 32 * i) < E ? __float_as_uint(p[i] / sum) + 1u : 0u;
    float tsum = 0.f, myv = 0.f;
    my_e = -1;
#pragma unroll 1
    for (int r = 0; r < topk; r++) {
        uint32_t bk = 0u;
        int bi = 0;
#pragma unroll
        for (int i = 0; i < 8; i++)       // ascending expert id within the lane: '>' keeps the lower id
            if (key[i] > bk) { bk = key[i]; bi = i; }
        const uint32_t m = __reduce_max_sync(0xffffffffu, bk);
        const uint32_t cand = (bk == m && m != 0u) ? (uint32_t)(lane + 32 * bi) : 0x7fffffffu;
        const int e = (int)__reduce_min_sync(0xffffffffu, cand);
        if ((e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; i++) if (i == (e >> 5)) key[i] = 0u;
        }
        const float v = m ? __uint_as_float(m - 1u) : 0.f;
        if (lane == r) { myv = v; my_e = e; }
        tsum += v;
    }
    my_w = myv / tsum;
}

// top-k of every sequence's router logits, one warp per sequence (batched decode, after the logits came from a
// matrix product). grid (ceil(B / 8)), 256 threads.
__global__ void __launch_bounds__(256) k_router_topk(const float* __restrict__ logits, int stride, int E, int topk, int* __restrict__ top_idx,
                                                     float* __restrict__ top_w, int B, const CoreRoute core) {
    const int lane = threadIdx.x & 31, b = blockIdx.x * 8 + (threadIdx.x >> 5);
    grid_dep_launch();
    grid_dep_wait();
    if (b >= B) return;
    int e;
    float w;
    router_topk_lanes(logits + (size_t)b * stride, E, topk, lane, e, w);
    if (lane < topk) { top_idx[(size_t)b * topk + lane] = e; top_w[(size_t)b * topk + lane] = w; }
    if (core.score) core_route_warp(core, b, lane);       // the core engine's picks of the same token
}

struct Gu1Args {
    unsigned long long* trace;
    const float* logits;          // [B][E] router logits (bias included)
    const float* x;               // [B][D] residual stream
    const uint16_t* norm_w;       // [D]
    float eps;
    const uint8_t* const* eptr;   // [E] resident experts
    size_t off_gu_s, off_gu_m;
    int D, I, E, topk;
    int* top_idx;                 // [B][topk] out (block 0 of every token)
    float* top_w;                 // [B][topk] out
    const uint8_t** top_ptr;      // [B][topk] out: the picks' expert blobs, for k_moe_down1
    int8_t* actq;                 // [B * topk][PLANES][I] out: digit planes of act, even/odd order within 8
    float* asc;                   // [B * topk][I / 32] out: scale of each 32-value group of act
    float* asum;                  // [B * topk][I / 32] out: sum of each 32-value group of act
    int* err;
    CoreRoute core;               // the core engine's picks: one otherwise idle warp of every token's first block makes them
};

// dynamic shared memory: rows | scales | digit planes of x | group sums of x
__host__ __device__ __forceinline__ size_t m1_gu_smem(int D) {
    return (size_t)2 * M1_GU_PAIRS * ((D >> 1) + 32) + (size_t)2 * M1_GU_PAIRS * 2 * (D >> 6) * 2 + (size_t)M1_PLANES * (D + 64) + (size_t)(D >> 6) * 4;
}

// grid (topk * I / 32, B); 32 warps. Prologue: warps 0-7 rank the experts (one thread per expert: every warp
// lists the 8 best of its 32 by counting, for each, the ones that beat it; the 64 listed are ranked the same
// way), warps 8-15 normalise x and split it into digit planes, 8 consecutive values per thread.
__global__ void __launch_bounds__(M1_GU_THREADS) k_moe_gu1(const Gu1Args a) {
    extern __shared__ __align__(128) unsigned char m1_smem[];
    const int D = a.D, half = D >> 1;                   // bytes of codes per row
    const int pitch = half + 32;                        // rows r .. r+3 fall into different quarters of the banks
    const int ngroup = D >> 6;
    unsigned char* s_rows = m1_smem;                                            // [2 * M1_GU_PAIRS][pitch]
    uint16_t* s_sc = reinterpret_cast<uint16_t*>(s_rows + (size_t)2 * M1_GU_PAIRS * pitch);   // [2 * PAIRS][2][ngroup]: scales | mins
    const int XS = D + 64;                              // plane stride: planes p, p+1 in different halves of the banks
    int8_t* s_xq = reinterpret_cast<int8_t*>(s_sc + (size_t)2 * M1_GU_PAIRS * 2 * ngroup);    // [PLANES][XS], even/odd order
    float* s_xsum = reinterpret_cast<float*>(s_xq + (size_t)M1_PLANES * XS);                  // [ngroup]
    __shared__ __align__(16) uint32_t s_key[64];        // the 8 best keys of each of the 8 ranking warps
    __shared__ __align__(16) int s_cand[64];            // and their experts
    __shared__ const uint8_t* s_eptr[256];              // the layer's expert table (E <= 256)
    __shared__ int s_top[8];
    __shared__ float s_topv[8];
    __shared__ float s_red[2][8];
    __shared__ float s_part[8][4][16][2];               // [K eighth][row block][row][gate | up]
    __shared__ float s_scale;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid = lane & 3;
    const int b = blockIdx.y;
    grid_dep_launch();
    trace_in(a.trace, 5, gridDim.x);
    // the expert table is written at load time only: read it while the previous kernel still runs
    if (threadIdx.x < a.E && threadIdx.x < 256) s_eptr[threadIdx.x] = a.eptr[threadIdx.x];
    if (threadIdx.x < 8) { s_top[threadIdx.x] = -1; s_topv[threadIdx.x] = 0.f; }
    grid_dep_wait();
    trace_pt(a.trace, 1);

    if (warp < 8) {
        // aegist/hybrid.py:641-645: softmax, the topk largest in descending order (ties to the lower index)
        const int e = threadIdx.x;
        const float v = e < a.E ? __ldcg(a.logits + (size_t)b * a.E + e) : -INFINITY;
        float mx = warp_max(v);
        if (lane == 0) s_red[0][warp] = mx;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        mx = s_red[0][0];
#pragma unroll
        for (int w = 1; w < 8; w++) mx = fmaxf(mx, s_red[0][w]);
        const float p = e < a.E ? expf(v - mx) : 0.f;
        float sum = warp_sum(p);
        if (lane == 0) s_red[1][warp] = sum;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) sum += s_red[1][w];
        const float prob = p / sum;
        const uint32_t key = e < a.E ? __float_as_uint(prob) + 1u : 0u;      // positive floats order like their bits
        // two rounds of rank counting (independent compares instead of a chain of reductions): every warp ranks its
        // 32 experts among themselves over 31 rotations and lists its 8 best, then the 64 listed are ranked, four
        // threads per candidate. Order: larger key first, equal keys by the lower expert number.
        {
            int rank = 0;
#pragma unroll
            for (int s = 1; s < 32; s++) {
                const uint32_t o = __shfl_sync(0xffffffffu, key, (lane + s) & 31);
                const bool lower = lane + s >= 32;                  // the other lane holds a lower expert number
                rank += (o > key || (o == key && lower)) ? 1 : 0;
            }
            if (rank < 8) { s_key[warp * 8 + rank] = key; s_cand[warp * 8 + rank] = key ? e : 0x7fffffff; }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        {
            const int c = threadIdx.x >> 2, q = threadIdx.x & 3;
            const uint32_t kc = s_key[c];
            const int ec = s_cand[c];
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint4 kk = *reinterpret_cast<const uint4*>(s_key + q * 16 + j * 4);
                const int4 ee = *reinterpret_cast<const int4*>(s_cand + q * 16 + j * 4);
                cnt += (kk.x > kc || (kk.x == kc && ee.x < ec)) ? 1 : 0;
                cnt += (kk.y > kc || (kk.y == kc && ee.y < ec)) ? 1 : 0;
                cnt += (kk.z > kc || (kk.z == kc && ee.z < ec)) ? 1 : 0;
                cnt += (kk.w > kc || (kk.w == kc && ee.w < ec)) ? 1 : 0;
            }
            cnt += __shfl_xor_sync(0xffffffffu, cnt, 1);
            cnt += __shfl_xor_sync(0xffffffffu, cnt, 2);
            if (q == 0 && cnt < a.topk) {
                s_top[cnt] = ec < 0x7fffffff ? ec : -1;
                s_topv[cnt] = kc ? __uint_as_float(kc - 1u) : 0.f;
            }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (blockIdx.x == 0 && threadIdx.x < a.topk) {
            float tsum = 0.f;
            for (int r = 0; r < a.topk; r++) tsum += s_topv[r];
            const int ex = s_top[threadIdx.x];
            a.top_idx[(size_t)b * a.topk + threadIdx.x] = ex;
            a.top_w[(size_t)b * a.topk + threadIdx.x] = s_topv[threadIdx.x] / tsum;
            a.top_ptr[(size_t)b * a.topk + threadIdx.x] = (ex >= 0 && ex < a.E) ? s_eptr[ex] : nullptr;
        }
        trace_pt(a.trace, 2);
    } else if (warp == 16) {
        if (blockIdx.x == 0 && a.core.score) core_route_warp(a.core, b, lane);
    } else if (warp < 16) {
        // norm2(x) -> digit planes and group sums; D / 8 chunks over 256 threads
        const int xt = threadIdx.x - 256;
        constexpr int XC = 2;                           // turns: D <= 256 * 8 * 2
        float xv[XC][8], nw[XC][8];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < XC; j++) {
            const int k = (xt + j * 256) * 8;
            if (k < D) {
                const float4 v0 = *reinterpret_cast<const float4*>(a.x + (size_t)b * D + k);
                const float4 v1 = *reinterpret_cast<const float4*>(a.x + (size_t)b * D + k + 4);
                xv[j][0] = v0.x; xv[j][1] = v0.y; xv[j][2] = v0.z; xv[j][3] = v0.w;
                xv[j][4] = v1.x; xv[j][5] = v1.y; xv[j][6] = v1.z; xv[j][7] = v1.w;
                uint4 wv = make_uint4(0u, 0u, 0u, 0u);
                if (a.norm_w) wv = *reinterpret_cast<const uint4*>(a.norm_w + k);
                nw[j][0] = 1.0f + bflo(wv.x); nw[j][1] = 1.0f + bfhi(wv.x); nw[j][2] = 1.0f + bflo(wv.y); nw[j][3] = 1.0f + bfhi(wv.y);
                nw[j][4] = 1.0f + bflo(wv.z); nw[j][5] = 1.0f + bfhi(wv.z); nw[j][6] = 1.0f + bflo(wv.w); nw[j][7] = 1.0f + bfhi(wv.w);
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) { xv[j][i] = 0.f; nw[j][i] = 1.0f; }
            }
#pragma unroll
            for (int i = 0; i < 8; i++) { ss = fmaf(xv[j][i], xv[j][i], ss); xv[j][i] *= nw[j][i]; }
        }
        // the rms is one factor for the whole vector: the sum of squares and the largest |(1 + w) x| are reduced
        // together, behind one barrier
        float* red = &s_part[0][0][0][0];               // scratch until the main part starts
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < XC; j++)
#pragma unroll
            for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(xv[j][i]));
        ss = warp_sum(ss);
        mx = warp_max(mx);
        if (lane == 0) { red[warp] = ss; red[16 + warp] = mx; }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        mx = 0.f;
        float t = 0.f;
#pragma unroll
        for (int w = 8; w < 16; w++) { mx = fmaxf(mx, red[16 + w]); t += red[w]; }
        if (a.norm_w) {
            const float r = 1.0f / sqrtf(t / (float)D + a.eps);
#pragma unroll
            for (int j = 0; j < XC; j++)
#pragma unroll
                for (int i = 0; i < 8; i++) xv[j][i] *= r;
            mx *= r;
        }
        const float inv = mx > 1e-30f ? 127.0f / mx : 0.f;
        if (xt == 0) s_scale = mx / 127.0f;
#pragma unroll
        for (int j = 0; j < XC; j++) {
            const int k = (xt + j * 256) * 8;
            // the sum of a 64-value group: 8 neighbouring lanes, values in index order within a lane
            float s8 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) s8 += xv[j][i];
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
            s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
            s8 += __shfl_xor_sync(0xffffffffu, s8, 4);
            if (k < D) {
                uint2 w[M1_PLANES];
                digits8(xv[j], inv, true, w);
#pragma unroll
                for (int p = 0; p < M1_PLANES; p++) *reinterpret_cast<uint2*>(s_xq + (size_t)p * XS + k) = w[p];
                if ((lane & 7) == 0) s_xsum[k >> 6] = s8;
            }
        }
    }
    __syncthreads();
    trace_pt(a.trace, 3);

    // this block's 32 pairs: rows i0 .. i0 + 31 of pick rnk
    const int p0 = blockIdx.x * M1_GU_PAIRS;
    const int rnk = p0 / a.I, i0 = p0 - rnk * a.I;
    const int e = s_top[rnk];
    const uint8_t* base = (e >= 0 && e < a.E) ? s_eptr[e] : nullptr;
    if (base == nullptr) {                               // a bad pick: say so, nothing to compute
        if (threadIdx.x == 0) atomicExch(a.err, 2);
        trace_out(a.trace);
        return;
    }
    // slot of pair s: block s / 8, gate in row s % 8 of the block's 16 rows, up in row 8 + s % 8; a warp
    // fetches two whole rows, a lane 16-byte pieces of them
    const int chunks = half >> 4;
    const int sch = (ngroup * 2 + 15) >> 4;              // 16-byte pieces of a row's scales (ngroup fp16)
    const int scm = sc_mask(ngroup);
    const int which = lane / sch, ch = lane - which * sch;      // this lane's piece of a row's scales | mins
#pragma unroll
    for (int it = 0; it < 2 * M1_GU_PAIRS / M1_GU_WARPS; it++) {
        const int rowi = warp + it * M1_GU_WARPS;
        const int s = rowi >> 1, up = rowi & 1;
        const int slot = (s >> 3) * 16 + up * 8 + (s & 7);
        const size_t grow = (size_t)(up * a.I + i0 + s);
        const uint8_t* src = base + grow * half;
        unsigned char* dst = s_rows + (size_t)slot * pitch;
        for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 16, src + (size_t)c * 16);
        if (lane < 2 * sch) {
            const uint8_t* ssrc = base + (which ? a.off_gu_m : a.off_gu_s) + grow * ngroup * 2;
            uint16_t* srow = s_sc + (size_t)slot * 2 * ngroup;
            if (scm) cp_async16(reinterpret_cast<unsigned char*>(srow + (((which * sch + ch) ^ (slot & scm)) << 3)), ssrc + (size_t)ch * 16);
            else copy_f16_piece(srow + which * ngroup, ssrc, ngroup, ch);
        }
    }
    cp_async_commit();
    trace_pt(a.trace, 4);
    cp_async_wait<0>();
    __syncthreads();
    trace_pt(a.trace, 5);

    // warp -> (block of 8 pairs, eighth of K); lane (gid, tid) -> rows gid (gate) and gid + 8 (up) of the block,
    // 16 codes of every 64-code group. A warp's ge = ngroup / 8 groups (1, 2, 4 or 8) lie inside one 16-byte piece of
    // a scale row, so their scales and mins are at consecutive positions from a base computed once.
    const int rb = warp & 3, ke = warp >> 2;
    const int ge = ngroup >> 3;
    float accg[2] = {0.f, 0.f}, accu[2] = {0.f, 0.f};   // planes 2 tid and 2 tid + 1
    float mng = 0.f, mnu = 0.f;
    {
        const int gf = ke * ge;
        const int slg = rb * 16 + gid, slu = slg + 8;
        const unsigned char* pg = s_rows + (size_t)slg * pitch + tid * 8 + gf * 32;
        const unsigned char* pu = pg + (size_t)8 * pitch;
        const uint16_t* sgs = s_sc + (size_t)slg * 2 * ngroup + sc_pos(ngroup, scm, slg, 0, gf);
        const uint16_t* sgm = s_sc + (size_t)slg * 2 * ngroup + sc_pos(ngroup, scm, slg, 1, gf);
        const uint16_t* sus = s_sc + (size_t)slu * 2 * ngroup + sc_pos(ngroup, scm, slu, 0, gf);
        const uint16_t* sum_ = s_sc + (size_t)slu * 2 * ngroup + sc_pos(ngroup, scm, slu, 1, gf);
        const int8_t* px = s_xq + (size_t)(gid & 3) * XS + tid * 16 + gf * 64;
        const float* pxs = s_xsum + gf;
        const bool colact = gid < M1_PLANES;
#pragma unroll 2
        for (int g = 0; g < ge; g++) {
            const uint2 wg = *reinterpret_cast<const uint2*>(pg + g * 32);
            const uint2 wu = *reinterpret_cast<const uint2*>(pu + g * 32);
            uint4 xb = make_uint4(0u, 0u, 0u, 0u);
            if (colact) xb = *reinterpret_cast<const uint4*>(px + g * 64);
            const float sgv = h2f(sgs[g]), suv = h2f(sus[g]), mgv = h2f(sgm[g]), muv = h2f(sum_[g]);
            const float xs = pxs[g];
            int t[4] = {0, 0, 0, 0};
            imma16832(t, wg.x & 0x0F0F0F0Fu, wu.x & 0x0F0F0F0Fu, (wg.x >> 4) & 0x0F0F0F0Fu, (wu.x >> 4) & 0x0F0F0F0Fu, xb.x, xb.y);
            imma16832(t, wg.y & 0x0F0F0F0Fu, wu.y & 0x0F0F0F0Fu, (wg.y >> 4) & 0x0F0F0F0Fu, (wu.y >> 4) & 0x0F0F0F0Fu, xb.z, xb.w);
            accg[0] = fmaf(sgv, small_int_to_float(t[0]), accg[0]); accg[1] = fmaf(sgv, small_int_to_float(t[1]), accg[1]);
            accu[0] = fmaf(suv, small_int_to_float(t[2]), accu[0]); accu[1] = fmaf(suv, small_int_to_float(t[3]), accu[1]);
            mng = fmaf(mgv, xs, mng);
            mnu = fmaf(muv, xs, mnu);
        }
    }
    {
        float w0, w1;
        plane_weights(tid, s_scale, w0, w1);
        float vg = accg[0] * w0 + accg[1] * w1, vu = accu[0] * w0 + accu[1] * w1;
        vg += __shfl_xor_sync(0xffffffffu, vg, 1); vu += __shfl_xor_sync(0xffffffffu, vu, 1);
        if (tid == 0) { s_part[ke][rb][gid][0] = vg + mng; s_part[ke][rb][gid][1] = vu + mnu; }
    }
    __syncthreads();
    trace_pt(a.trace, 6);
    if (warp == 0) {
        // act of pair `lane`, then this 32-value group of act as digit planes with its own scale
        const int s = lane;
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) { g += s_part[q][s >> 3][s & 7][0]; u += s_part[q][s >> 3][s & 7][1]; }
        const float v = siluf_(g) * u;
        const float mx = warp_max(fabsf(v));
        const float inv = mx > 1e-30f ? 127.0f / mx : 0.f;
        int d[M1_PLANES];
        to_digits(v, inv, d);
        const size_t pick = (size_t)b * a.topk + rnk;
        const int pos = i0 + ((s & ~7) | ((s & 1) << 2) | ((s & 7) >> 1));      // even ones first within 8
#pragma unroll
        for (int p = 0; p < M1_PLANES; p++) a.actq[(pick * M1_PLANES + p) * a.I + pos] = (int8_t)d[p];
        const float sm = warp_sum(v);
        if (lane == 0) {
            a.asc[pick * (a.I >> 5) + (i0 >> 5)] = mx / 127.0f;
            a.asum[pick * (a.I >> 5) + (i0 >> 5)] = sm;
        }
    }
    trace_pt(a.trace, 7);
    trace_out(a.trace);
}

struct Down1Args {
    unsigned long long* trace;
    const uint8_t* const* top_ptr;   // [B][topk] the picks' expert blobs (null: not resident)
    const float* top_w;              // [B][topk]
    const int8_t* actq;              // [B * topk][PLANES][I] digit planes of act (k_moe_gu1)
    const float* asc;                // [B * topk][I / 32]
    const float* asum;               // [B * topk][I / 32]
    const float* sh_act;             // [B][SH]
    const float* sg;                 // [B] sigmoid(shared gate)
    const int8_t* shd_w;             // [D][SH] shared down, or null
    const uint16_t* shd_s;           // [D]
    size_t off_dn_q, off_dn_s, off_dn_m;
    int D, I, SH, topk;
    float* xout;                     // [B][D] residual stream, += result
};

// per pick warp (a half of K): 16 rows x (I / 4 + 16) codes | scales [16][2][I / 64] | planes [4][I / 2] | 2 x [I / 64] group scales
// and sums; per shared warp: 16 rows x (SH / 2 + 64) | planes [4][SH / 2]
__host__ __device__ __forceinline__ size_t m1_down_pick_bytes(int I) {
    return (size_t)M1_DOWN_ROWS * ((I >> 2) + 16) + (size_t)M1_DOWN_ROWS * 2 * (I >> 6) * 2 + (size_t)M1_PLANES * (I >> 1) + (size_t)2 * (I >> 5) * 4;
}
__host__ __device__ __forceinline__ size_t m1_down_shared_bytes(int SH) { return (size_t)M1_DOWN_ROWS * ((SH >> 1) + 64) + (size_t)M1_PLANES * (SH >> 1); }
__host__ __device__ __forceinline__ size_t m1_down_smem(int I, int SH, int topk) {
    return (size_t)2 * topk * m1_down_pick_bytes(I) + 2 * m1_down_shared_bytes(SH);
}

// grid (D / 16, B); 2 * (topk + 1) warps: warp 2 r + h = half h of K of pick r, the last two the shared expert
__global__ void __launch_bounds__(M1_DOWN_WARPS * 32) k_moe_down1(const Down1Args a) {
    extern __shared__ __align__(128) unsigned char m1d_smem[];
    __shared__ float s_y[M1_DOWN_WARPS][M1_DOWN_ROWS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid = lane & 3;
    const int b = blockIdx.y;
    const int row0 = blockIdx.x * M1_DOWN_ROWS;
    const int I = a.I, SH = a.SH;
    const int r = warp >> 1, kh = warp & 1;
    grid_dep_launch();
    trace_in(a.trace, 6, gridDim.x);
    float y0 = 0.f, y1 = 0.f;             // rows gid and gid + 8 (valid in lanes with tid == 0)
    // what the final sum needs from global memory is requested by its threads right after the wait, not at the end
    float cw[8], csg = 0.f, cx = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) cw[k] = 0.f;
    const bool comb = threadIdx.x < M1_DOWN_ROWS && row0 + threadIdx.x < a.D;
    if (r < a.topk) {
        const int halfk = I >> 2;                        // bytes of codes of this warp's half of a row
        const int pitch = halfk + 16;                    // 8 rows x 16 bytes cover all banks
        const int ngroup = I >> 6, gh = ngroup >> 1;     // groups per half
        unsigned char* s_rows = m1d_smem + (size_t)warp * m1_down_pick_bytes(I);
        uint16_t* s_sc = reinterpret_cast<uint16_t*>(s_rows + (size_t)M1_DOWN_ROWS * pitch);     // [16][2][ngroup]
        int8_t* s_xq = reinterpret_cast<int8_t*>(s_sc + (size_t)M1_DOWN_ROWS * 2 * ngroup);      // [PLANES][I / 2]
        float* s_as = reinterpret_cast<float*>(s_xq + (size_t)M1_PLANES * (I >> 1));             // [2 gh] scales | [2 gh] sums
        grid_dep_wait();
        trace_pt(a.trace, 1);
        if (comb) {
#pragma unroll
            for (int k = 0; k < 8; k++) cw[k] = k < a.topk ? a.top_w[(size_t)b * a.topk + k] : 0.f;
            csg = a.shd_w ? a.sg[b] : 0.f;
            cx = a.xout[(size_t)b * a.D + row0 + threadIdx.x];
        }
        const size_t pick = (size_t)b * a.topk + r;
        const uint8_t* base = a.top_ptr[pick];
        if (base != nullptr) {
            // I is a power of two: pieces per row are too, so rows and pieces come from shifts
            const int chunks = halfk >> 4, csh = __ffs(chunks) - 1;
            for (int c = lane; c < M1_DOWN_ROWS * chunks; c += 32) {
                const int rr = c >> csh, ch = c & (chunks - 1);
                if (row0 + rr < a.D)
                    cp_async16(s_rows + (size_t)rr * pitch + ch * 16, base + a.off_dn_q + (size_t)(row0 + rr) * (I >> 1) + (size_t)kh * halfk + (size_t)ch * 16);
            }
            const int sch = (ngroup * 2 + 15) >> 4, ssh = __ffs(sch) - 1;
            for (int c = lane; c < M1_DOWN_ROWS * 2 * sch; c += 32) {
                const int q = c >> ssh, ch = c & (sch - 1);
                const int rr = q >> 1, which = q & 1;
                if (row0 + rr < a.D)
                    copy_f16_piece(s_sc + ((size_t)rr * 2 + which) * ngroup, base + (which ? a.off_dn_m : a.off_dn_s) + ((size_t)(row0 + rr) * ngroup) * 2, ngroup, ch);
            }
            const int pch = (I >> 1) >> 4, psh = __ffs(pch) - 1;   // 16-byte pieces of a plane's half
            for (int c = lane; c < M1_PLANES * pch; c += 32) {
                const int p = c >> psh, ch = c & (pch - 1);
                cp_async16(s_xq + (size_t)p * (I >> 1) + ch * 16, a.actq + (pick * M1_PLANES + p) * I + (size_t)kh * (I >> 1) + (size_t)ch * 16);
            }
            cp_async_commit();
            for (int c = lane; c < 2 * gh; c += 32) {
                s_as[c] = a.asc[pick * (I >> 5) + kh * 2 * gh + c];
                s_as[2 * gh + c] = a.asum[pick * (I >> 5) + kh * 2 * gh + c];
            }
            cp_async_wait<0>();
            __syncwarp();
            const unsigned char* p0 = s_rows + (size_t)gid * pitch + tid * 4;
            const unsigned char* p1 = p0 + (size_t)8 * pitch;
            const uint16_t* s0 = s_sc + (size_t)gid * 2 * ngroup + kh * gh;
            const uint16_t* s1 = s0 + (size_t)8 * 2 * ngroup;
            const int8_t* px = s_xq + (size_t)(gid & 3) * (I >> 1) + tid * 8;
            const bool colact = gid < M1_PLANES;
            float pw0, pw1;
            plane_weights(tid, 1.0f, pw0, pw1);
            float m0 = 0.f, m1 = 0.f;
            for (int g = 0; g < gh; g++) {
                const uint32_t a00 = *reinterpret_cast<const uint32_t*>(p0 + g * 32), a01 = *reinterpret_cast<const uint32_t*>(p0 + g * 32 + 16);
                const uint32_t a10 = *reinterpret_cast<const uint32_t*>(p1 + g * 32), a11 = *reinterpret_cast<const uint32_t*>(p1 + g * 32 + 16);
                uint2 xb0 = make_uint2(0u, 0u), xb1 = xb0;
                if (colact) {
                    xb0 = *reinterpret_cast<const uint2*>(px + g * 64);
                    xb1 = *reinterpret_cast<const uint2*>(px + g * 64 + 32);
                }
                int t0[4] = {0, 0, 0, 0}, t1[4] = {0, 0, 0, 0};
                imma16832(t0, a00 & 0x0F0F0F0Fu, a10 & 0x0F0F0F0Fu, (a00 >> 4) & 0x0F0F0F0Fu, (a10 >> 4) & 0x0F0F0F0Fu, xb0.x, xb0.y);
                imma16832(t1, a01 & 0x0F0F0F0Fu, a11 & 0x0F0F0F0Fu, (a01 >> 4) & 0x0F0F0F0Fu, (a11 >> 4) & 0x0F0F0F0Fu, xb1.x, xb1.y);
                const float c0 = s_as[2 * g], c1 = s_as[2 * g + 1];           // scales of the two 32-value groups
                const float xs = s_as[2 * gh + 2 * g] + s_as[2 * gh + 2 * g + 1];
                const float v0 = c0 * (small_int_to_float(t0[0]) * pw0 + small_int_to_float(t0[1]) * pw1) +
                                 c1 * (small_int_to_float(t1[0]) * pw0 + small_int_to_float(t1[1]) * pw1);
                const float v1 = c0 * (small_int_to_float(t0[2]) * pw0 + small_int_to_float(t0[3]) * pw1) +
                                 c1 * (small_int_to_float(t1[2]) * pw0 + small_int_to_float(t1[3]) * pw1);
                y0 = fmaf(h2f(s0[g]), v0, y0);
                y1 = fmaf(h2f(s1[g]), v1, y1);
                m0 = fmaf(h2f(s0[ngroup + g]), xs, m0);
                m1 = fmaf(h2f(s1[ngroup + g]), xs, m1);
            }
            y0 += __shfl_xor_sync(0xffffffffu, y0, 1); y1 += __shfl_xor_sync(0xffffffffu, y1, 1);
            y0 += m0; y1 += m1;
        }
    } else {
        // shared expert: int8 rows of SH values against sh_act, this warp's half of SH
        const int hk = SH >> 1, pitch = hk + 64;
        unsigned char* s_rows = m1d_smem + (size_t)2 * a.topk * m1_down_pick_bytes(I) + (size_t)kh * m1_down_shared_bytes(SH);
        int8_t* s_xq = reinterpret_cast<int8_t*>(s_rows + (size_t)M1_DOWN_ROWS * pitch);
        if (a.shd_w) {
            const int chunks = hk >> 4;
            for (int c = lane; c < M1_DOWN_ROWS * chunks; c += 32) {          // weights do not depend on the previous kernel
                const int rr = c / chunks, ch = c - rr * chunks;               // (before the wait: not on the critical path)
                if (row0 + rr < a.D)
                    cp_async16(s_rows + (size_t)rr * pitch + ch * 16, (const unsigned char*)a.shd_w + (size_t)(row0 + rr) * SH + (size_t)kh * hk + (size_t)ch * 16);
            }
            cp_async_commit();
        }
        grid_dep_wait();
        if (a.shd_w) {
            // this half of sh_act as digit planes with its own scale: 8 consecutive values per lane and turn
            const float* src = a.sh_act + (size_t)b * SH + kh * hk;
            float mx = 0.f;
            for (int k = lane * 8; k < hk; k += 256)
#pragma unroll
                for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(src[k + i]));
            mx = warp_max(mx);
            const float inv = mx > 1e-30f ? 127.0f / mx : 0.f;
            for (int k = lane * 8; k < hk; k += 256) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = src[k + i];
                uint2 w[M1_PLANES];
                digits8(v, inv, false, w);
#pragma unroll
                for (int p = 0; p < M1_PLANES; p++) *reinterpret_cast<uint2*>(s_xq + (size_t)p * hk + k) = w[p];
            }
            cp_async_wait<0>();
            __syncwarp();
            const unsigned char* p0 = s_rows + (size_t)gid * pitch + tid * 16;
            const unsigned char* p1 = p0 + (size_t)8 * pitch;
            const int8_t* px = s_xq + (size_t)(gid & 3) * hk + tid * 16;
            const bool colact = gid < M1_PLANES;
            int t[4] = {0, 0, 0, 0};
            for (int k = 0; k < hk; k += 64) {
                const uint4 w0 = *reinterpret_cast<const uint4*>(p0 + k);
                const uint4 w1 = *reinterpret_cast<const uint4*>(p1 + k);
                uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                if (colact) xb = *reinterpret_cast<const uint4*>(px + k);
                imma16832(t, w0.x, w1.x, w0.y, w1.y, xb.x, xb.y);
                imma16832(t, w0.z, w1.z, w0.w, w1.w, xb.z, xb.w);
            }
            float w0f, w1f;
            plane_weights(tid, mx / 127.0f, w0f, w1f);
            y0 = (float)t[0] * w0f + (float)t[1] * w1f;
            y1 = (float)t[2] * w0f + (float)t[3] * w1f;
            y0 += __shfl_xor_sync(0xffffffffu, y0, 1); y1 += __shfl_xor_sync(0xffffffffu, y1, 1);
            if (row0 + gid < a.D) y0 *= bf(a.shd_s[row0 + gid]);
            if (row0 + gid + 8 < a.D) y1 *= bf(a.shd_s[row0 + gid + 8]);
        }
    }
    if (tid == 0) { s_y[warp][gid] = y0; s_y[warp][gid + 8] = y1; }
    __syncthreads();
    trace_pt(a.trace, 3);
    // x[o] += sum_r w_r * y_r[o] + sigmoid(shared gate) * y_shared[o], picks in rank order
    if (comb) {
        const int o = threadIdx.x;
        float y = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++)
            if (k < a.topk) y = fmaf(cw[k], s_y[2 * k][o] + s_y[2 * k + 1][o], y);
        if (a.shd_w) y = fmaf(csg, s_y[2 * a.topk][o] + s_y[2 * a.topk + 1][o], y);
        a.xout[(size_t)b * a.D + row0 + o] = cx + y;
    }
    trace_out(a.trace);
}

}  // namespace b2
