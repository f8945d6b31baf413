// k_attn_mma: the decode attention of k_attn (same prologue, same slices, same partial results for
// k_attn_merge) for a bf16 KV cache, with the two contractions on the tensor cores.
//
// A block takes one KV head of one sequence and one slice of the context, in tiles of 64 positions
// (one cache page). Per tile, with the G <= 8 query heads of the group as the rows of a 16-row operand:
//   S = Q K^T    mma.sync.m16n8k16.bf16: Q as three bf16 planes (hi + mid + lo = the fp32 value to 2^-24),
//                K as it lies in the cache; warp w takes positions 8 w .. 8 w + 7
//   softmax      online, base-2, maxima and sums of the 8 warps meet in shared memory
//   O += P V     P as three bf16 planes (exact to 2^-24), V through ldmatrix.trans; warp w takes HD / 8 output dims
// K and V tiles come in by 16-byte cp.async, double-buffered when the slice has more than one tile. The
// exact fp32 arithmetic of k_attn (used for an fp32 cache) differs from this only by summation order: the
// three-plane splits of Q and P carry all 24 significant bits.
#pragma once

namespace b2 {

constexpr int AM_TILE = 64;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)) : "memory");
}
// v = hi + mid + lo with three bf16 values (truncation, so every remainder is exact)
__device__ __forceinline__ void split3_bf16(float v, uint16_t& hi, uint16_t& mid, uint16_t& lo) {
    const uint32_t h = __float_as_uint(v) & 0xFFFF0000u;
    const float r1 = v - __uint_as_float(h);
    const uint32_t m = __float_as_uint(r1) & 0xFFFF0000u;
    const float r2 = r1 - __uint_as_float(m);
    hi = (uint16_t)(h >> 16); mid = (uint16_t)(m >> 16); lo = (uint16_t)(__float_as_uint(r2) >> 16);
}

template <int HD>
__host__ __device__ constexpr int am_kpitch() { return HD * 2 + 64; }   // rows r, r + 1 in different halves of the banks
template <int HD>
__host__ __device__ constexpr int am_vpitch() { return HD * 2 + 16; }   // 8 consecutive rows cover all banks (ldmatrix)
// dynamic shared memory: [nbuf] K tiles | [nbuf] V tiles | Q planes [3][8][HD + 32] bf16 | P planes [3][8][72] bf16
template <int HD>
__host__ __device__ constexpr size_t am_smem(int nbuf) {
    return (size_t)nbuf * AM_TILE * (am_kpitch<HD>() + am_vpitch<HD>()) + (size_t)3 * 8 * (HD + 32) * 2 + (size_t)3 * 8 * 72 * 2;
}

// grid (nsplit, KV, B); the slice length is a multiple of 64
template <int HD>
__global__ void __launch_bounds__(THREADS) k_attn_mma(const AttnArgs a, int nbuf) {
    constexpr int KP = am_kpitch<HD>(), VP = am_vpitch<HD>(), QP = HD + 32, PP = 72;
    constexpr int NTV = HD / 64;                // 8-dim output tiles per warp
    constexpr int DPL = HD / 32;
    const int G = a.H / a.KV;                   // query heads per KV head (<= 8)
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid = lane & 3;
    extern __shared__ __align__(128) unsigned char am_smem_raw[];
    unsigned char* Ks = am_smem_raw;                                         // [nbuf][64][KP]
    unsigned char* Vs = Ks + (size_t)nbuf * AM_TILE * KP;                    // [nbuf][64][VP]
    uint16_t* Qh = reinterpret_cast<uint16_t*>(Vs + (size_t)nbuf * AM_TILE * VP);   // [3][8][QP]
    uint16_t* Ps = Qh + 3 * 8 * QP;                                          // [3][8][PP]
    __shared__ float knew[HD], vnew[HD];
    __shared__ float s_max[WARPS][8], s_sum[WARPS][8];
    grid_dep_launch();
    trace_in(a.trace, 7, gridDim.x);
    grid_dep_wait();
    trace_pt(a.trace, 1);
    const int pos = a.pos[b];
    const int L = pos + 1;
    int chunk = (L + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + AM_TILE - 1) / AM_TILE * AM_TILE;
    const int p0 = split * chunk, p1 = min(L, p0 + chunk);
    const size_t pstride = HD + 2;
    float* part = a.part + (((size_t)b * a.KV + kvh) * a.nsplit + split) * G * pstride;
    if (p0 >= p1) {                           // an empty slice: say so and leave
        for (int g = threadIdx.x; g < G; g += THREADS) { part[g * pstride + HD] = -INFINITY; part[g * pstride + HD + 1] = 0.f; }
        trace_out(a.trace);
        return;
    }
    const uint16_t* kpool = (const uint16_t*)a.kpool;
    const uint16_t* vpool = (const uint16_t*)a.vpool;
    // a tile is one cache page: 64 rows of HD bf16 for this KV head, contiguous; rows past the slice are not needed
    // but must hold finite numbers (their probabilities are zero), so the last valid row is loaded in their place
    auto load_tile = [&](int t0, int buf) {
        const int page = a.page_table[(size_t)b * a.pt_stride + t0 / KV_PAGE];
        const size_t base = ((size_t)page * a.KV + kvh) * KV_PAGE * HD;
        constexpr int CPR = HD * 2 / 16;        // 16-byte pieces per row
        const int last = min(AM_TILE, p1 - t0) - 1;
        for (int c = threadIdx.x; c < AM_TILE * CPR; c += THREADS) {
            const int r = c / CPR, ch = c - r * CPR;
            const int rs = min(r, last);
            cp_async16(Ks + ((size_t)buf * AM_TILE + r) * KP + ch * 16, kpool + base + (size_t)rs * HD + ch * 8);
            cp_async16(Vs + ((size_t)buf * AM_TILE + r) * VP + ch * 16, vpool + base + (size_t)rs * HD + ch * 8);
        }
        cp_async_commit();
    };
    // prologue: warps 0..G-1 prepare the query heads (ZNorm, partial RoPE), the next one the new key and value.
    // Everything a warp needs is requested at once; a lane holds dims lane + 32 i, so with RD / 2 a multiple of 32
    // the two halves of a rotation pair are in one lane, and for a shorter rotation they are RD / 2 lanes apart.
    const int hr = a.RD / 2;
    for (int t = warp; t < G + 1; t += WARPS) {
        const bool isq = t < G;
        const float* src = isq ? a.qraw + ((size_t)b * a.H + kvh * G + t) * 2 * HD : a.kraw + ((size_t)b * a.KV + kvh) * HD;
        const uint16_t* nw = isq ? a.qn_w : a.kn_w;
        const float* vs = a.vraw + ((size_t)b * a.KV + kvh) * HD;
        float v[DPL], w[DPL], vv[DPL], c[DPL], s[DPL];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const int d = lane + 32 * i;
            v[i] = src[d];
            w[i] = 1.0f + bf(nw[d]);
            vv[i] = isq ? 0.f : vs[d];
            const int j = d < hr ? d : d - hr;          // index of the pair this dim belongs to (dims below RD only)
            c[i] = d < a.RD ? a.rope_cos[(size_t)pos * hr + j] : 1.0f;
            s[i] = d < a.RD ? a.rope_sin[(size_t)pos * hr + j] : 0.f;
            ss = fmaf(v[i], v[i], ss);
        }
        if (t == warp) load_tile(p0, 0);               // the first tile's copies go out while those loads are in flight
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)HD + a.eps);
#pragma unroll
        for (int i = 0; i < DPL; i++) v[i] = v[i] * r * w[i];
        // rotate-half on the first RD dims (aegist/hybrid.py:160-166): (x0, x1) -> (x0 c - x1 s, x1 c + x0 s)
        float y[DPL];
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const int d = lane + 32 * i;
            float other = __shfl_xor_sync(0xffffffffu, v[i], hr & 31);   // hr < 32: only register 0 holds rotated dims
            if (hr >= 32) {
                const int pi = d < hr ? i + (hr >> 5) : i - (hr >> 5);    // the partner is hr / 32 registers away, same lane
                other = 0.f;
#pragma unroll
                for (int k = 0; k < DPL; k++) other = k == pi ? v[k] : other;
            }
            y[i] = d < hr ? v[i] * c[i] - other * s[i] : (d < a.RD ? v[i] * c[i] + other * s[i] : v[i]);
        }
        if (isq) {
            // scores are kept in the base-2 domain: q carries 1/sqrt(HD) * log2(e)
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                uint16_t h, m, l;
                split3_bf16(y[i] * (a.scale * 1.4426950408889634f), h, m, l);
                const int d = lane + 32 * i;
                Qh[(0 * 8 + t) * QP + d] = h; Qh[(1 * 8 + t) * QP + d] = m; Qh[(2 * 8 + t) * QP + d] = l;
            }
        } else {
#pragma unroll
            for (int i = 0; i < DPL; i++) { knew[lane + 32 * i] = bf(f2bf(y[i])); vnew[lane + 32 * i] = bf(f2bf(vv[i])); }   // what the cache gives back
        }
    }
    if (warp >= G + 1) load_tile(p0, 0);                // warps without a prologue row
    for (int t = G + warp; t < 8; t += WARPS)             // unused query rows are zero
        for (int i = lane; i < HD; i += 32) { Qh[(0 * 8 + t) * QP + i] = 0; Qh[(1 * 8 + t) * QP + i] = 0; Qh[(2 * 8 + t) * QP + i] = 0; }
    __syncthreads();
    // the block that owns the newest position appends it
    if (pos >= p0 && pos < p1) {
        const int page = a.page_table[(size_t)b * a.pt_stride + pos / KV_PAGE];
        const size_t off = (((size_t)page * a.KV + kvh) * KV_PAGE + pos % KV_PAGE) * HD;
        for (int i = threadIdx.x; i < HD; i += THREADS) { ((uint16_t*)a.kpool)[off + i] = f2bf(knew[i]); ((uint16_t*)a.vpool)[off + i] = f2bf(vnew[i]); }
    }
    if (a.append_only) {
        cp_async_wait<0>();                     // the first tile's copies were already sent
        trace_out(a.trace);
        return;
    }
    trace_pt(a.trace, 2);

    float m_run = -INFINITY, l_run = 0.f;       // of head gid, the same in the four lanes of a row
    float o[NTV][4];
#pragma unroll
    for (int n = 0; n < NTV; n++) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

    const int ntile = (p1 - p0 + AM_TILE - 1) / AM_TILE;
    for (int it = 0; it < ntile; it++) {
        const int t0 = p0 + it * AM_TILE;
        const int buf = nbuf == 2 ? (it & 1) : 0;
        if (nbuf == 1 && it > 0) load_tile(t0, 0);
        if (nbuf == 2 && it + 1 < ntile) { load_tile(t0 + AM_TILE, buf ^ 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        // the newest position is not in the cache yet (or was written by this block a moment ago): patch the tile
        if (pos >= t0 && pos < t0 + AM_TILE) {
            const int r = pos - t0;
            for (int i = threadIdx.x; i < HD; i += THREADS) {
                reinterpret_cast<uint16_t*>(Ks + ((size_t)buf * AM_TILE + r) * KP)[i] = f2bf(knew[i]);
                reinterpret_cast<uint16_t*>(Vs + ((size_t)buf * AM_TILE + r) * VP)[i] = f2bf(vnew[i]);
            }
            __syncthreads();
        }
        // S = Q K^T for positions t0 + 8 warp + (2 tid, 2 tid + 1) and head gid. Within a 32-dim step a lane
        // takes 8 consecutive dims of both operands (the order of k inside an mma step is free).
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const unsigned char* kr = Ks + ((size_t)buf * AM_TILE + warp * 8 + gid) * KP + tid * 16;
            const uint16_t* q0 = Qh + (0 * 8 + gid) * QP + tid * 8;
            const uint16_t* q1 = Qh + (1 * 8 + gid) * QP + tid * 8;
            const uint16_t* q2 = Qh + (2 * 8 + gid) * QP + tid * 8;
#pragma unroll
            for (int c = 0; c < HD / 32; c++) {
                const uint4 kk = *reinterpret_cast<const uint4*>(kr + c * 64);
                const uint4 a0 = *reinterpret_cast<const uint4*>(q0 + c * 32);
                const uint4 a1 = *reinterpret_cast<const uint4*>(q1 + c * 32);
                const uint4 a2 = *reinterpret_cast<const uint4*>(q2 + c * 32);
                mma_bf16(s4, a0.x, 0u, a0.y, 0u, kk.x, kk.y); mma_bf16(s4, a0.z, 0u, a0.w, 0u, kk.z, kk.w);
                mma_bf16(s4, a1.x, 0u, a1.y, 0u, kk.x, kk.y); mma_bf16(s4, a1.z, 0u, a1.w, 0u, kk.z, kk.w);
                mma_bf16(s4, a2.x, 0u, a2.y, 0u, kk.x, kk.y); mma_bf16(s4, a2.z, 0u, a2.w, 0u, kk.z, kk.w);
            }
        }
        const int pa = t0 + warp * 8 + 2 * tid;
        float s0 = pa < p1 ? s4[0] : -INFINITY, s1 = pa + 1 < p1 ? s4[1] : -INFINITY;
        float mx = fmaxf(s0, s1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (tid == 0) s_max[warp][gid] = mx;
        __syncthreads();
        float m_new = m_run;
#pragma unroll
        for (int w = 0; w < WARPS; w++) m_new = fmaxf(m_new, s_max[w][gid]);
        const float corr = m_run == -INFINITY ? 0.f : exp2f(m_run - m_new);
        const float e0 = s0 == -INFINITY ? 0.f : exp2f(s0 - m_new), e1 = s1 == -INFINITY ? 0.f : exp2f(s1 - m_new);
        float ps = e0 + e1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        if (tid == 0) s_sum[warp][gid] = ps;
        {   // P as hi + mid + lo bf16 planes (truncations, so the remainders are exact), [plane][head][position in the tile]
            uint16_t a0, a1, a2, b0, b1, b2;
            split3_bf16(e0, a0, a1, a2);
            split3_bf16(e1, b0, b1, b2);
            const int pc = warp * 8 + 2 * tid;
            *reinterpret_cast<uint32_t*>(Ps + (0 * 8 + gid) * PP + pc) = (uint32_t)a0 | ((uint32_t)b0 << 16);
            *reinterpret_cast<uint32_t*>(Ps + (1 * 8 + gid) * PP + pc) = (uint32_t)a1 | ((uint32_t)b1 << 16);
            *reinterpret_cast<uint32_t*>(Ps + (2 * 8 + gid) * PP + pc) = (uint32_t)a2 | ((uint32_t)b2 << 16);
        }
        __syncthreads();
        float lt = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) lt += s_sum[w][gid];
        l_run = l_run * corr + lt;
        m_run = m_new;
        // O = O * corr + P V for this warp's HD / 8 output dims
#pragma unroll
        for (int n = 0; n < NTV; n++) { o[n][0] *= corr; o[n][1] *= corr; }
#pragma unroll
        for (int ks = 0; ks < AM_TILE / 16; ks++) {
            const uint32_t ph0 = *reinterpret_cast<const uint32_t*>(Ps + (0 * 8 + gid) * PP + ks * 16 + 2 * tid);
            const uint32_t ph2 = *reinterpret_cast<const uint32_t*>(Ps + (0 * 8 + gid) * PP + ks * 16 + 8 + 2 * tid);
            const uint32_t pl0 = *reinterpret_cast<const uint32_t*>(Ps + (1 * 8 + gid) * PP + ks * 16 + 2 * tid);
            const uint32_t pl2 = *reinterpret_cast<const uint32_t*>(Ps + (1 * 8 + gid) * PP + ks * 16 + 8 + 2 * tid);
            const uint32_t pm0 = *reinterpret_cast<const uint32_t*>(Ps + (2 * 8 + gid) * PP + ks * 16 + 2 * tid);
            const uint32_t pm2 = *reinterpret_cast<const uint32_t*>(Ps + (2 * 8 + gid) * PP + ks * 16 + 8 + 2 * tid);
            const unsigned char* vr = Vs + ((size_t)buf * AM_TILE + ks * 16 + (lane & 15)) * VP + (size_t)warp * (HD / 8) * 2;
#pragma unroll
            for (int n = 0; n < NTV; n++) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(b0, b1, vr + n * 16);
                mma_bf16(o[n], pm0, 0u, pm2, 0u, b0, b1);       // smallest parts first
                mma_bf16(o[n], pl0, 0u, pl2, 0u, b0, b1);
                mma_bf16(o[n], ph0, 0u, ph2, 0u, b0, b1);
            }
        }
        __syncthreads();                     // the tile, P and the per-warp maxima may be overwritten
    }
    trace_pt(a.trace, 3);
    // (acc, max, sum) of this slice per query head, for k_attn_merge
    if (gid < G) {
#pragma unroll
        for (int n = 0; n < NTV; n++) {
            const int d = warp * (HD / 8) + n * 8 + 2 * tid;
            part[gid * pstride + d] = o[n][0];
            part[gid * pstride + d + 1] = o[n][1];
        }
        if (warp == 0 && tid == 0) { part[gid * pstride + HD] = m_run; part[gid * pstride + HD + 1] = l_run; }
    }
    trace_out(a.trace);
}

}  // namespace b2
