// Batched decode (6 or more sequences per GPU): the int8 linears as a tensor-core contraction.
//
// With B sequences the linears are [rows x K] x [K x B] products: real dense contractions, and on
// CUDA cores they are bound by the FMA rate, not by HBM (64 sequences x 1.7 G weights = 110 GFMA per
// step). Here each warp multiplies a 16-row slab of int8 weights, widened exactly to fp16 in
// registers (byte permute into 1024 + q + 128, minus 1152), with the activations split into two fp16
// halves, x = hi + lo (about 22 bits of x), by mma.sync.m16n8k16 with fp32 accumulation. Products of
// an fp16 integer and an fp16 value are exact in fp32, so the result differs from the fp32 GEMV only
// by the 2^-22 relative truncation of x and the order of the additions.
//
//   k_prep_x   activations -> normalised fp16 (hi | lo) rows [T][2][K] (ZNorm, gated RMSNorm or none)
//   k_mma_i8   out[t][row] = epilogue(scale[row] * sum_k W[row][k] x[t][k]) for up to 3 matrices
//
// A block is 4 warps = 64 weight rows; the K dimension is streamed in 256-wide chunks through a
// 3-stage cp.async ring holding the 64 x 256 int8 weight tile (row pitch 320 B) and the fp16
// activation tile of 32 sequences (64 columns x 256, column pitch 528 B); both pitches make the
// fragment loads bank-conflict free. The k index inside a 16-wide mma step is permuted identically on
// both operands (a thread takes 4 consecutive bytes / halves per step), which lets a thread fetch
// its A bytes for four steps with one 16-byte load.
#pragma once
#include <cuda_fp16.h>

namespace b2 {

constexpr int MM_ROWS = 64;          // weight rows per block (16 per warp)
constexpr int MM_KC = 256;           // K chunk
constexpr int MM_TOK = 32;           // sequences per pass (64 columns: hi and lo)
constexpr int MM_PA = 320;           // bytes between weight rows in shared memory
constexpr int MM_PB = 528;           // bytes between activation columns in shared memory
constexpr int MM_STAGES = 2;          // two blocks of 4 warps fit an SM (2 x 106 KB); with 3 stages only one did, and it ran slower
constexpr int MM_STAGES_DEEP = 4;     // for grids of at most one block per SM: 212 KB, three K chunks in flight
constexpr int MM_STAGE_BYTES = MM_ROWS * MM_PA + 2 * MM_TOK * MM_PB;   // 20480 + 33792
constexpr int MM_THREADS = 256;       // 8 warps: warp = (half of the sequences) x (16-row slab)

struct PrepArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    const float* x;          // [T][x_stride]
    int x_stride;
    const uint16_t* norm_w;  // ZNorm weight [K] or null
    const uint16_t* gn_w;    // gated RMSNorm weight [DV] or null (then z is silu(z))
    const float* z;
    int DV;
    float eps;
    int K, T;
    __half* out;             // [Tpad][2][K]; rows T..Tpad-1 are zero
    int Tpad;
    float* xsum;             // optional [T][K / 64]: the sum of each 64-value group (for the 4-bit min term)
    int perm8;               // store every 8 values in the order 0 4 1 5 2 6 3 7 (what the 4-bit unpacking yields)
};

// one block per sequence
__global__ void __launch_bounds__(256) k_prep_x(const PrepArgs a) {
    __shared__ float red[8];
    __shared__ float vs[4096];
    const int t = blockIdx.x;
    grid_dep_launch();
    trace_in(a.trace, 9, gridDim.x);
    grid_dep_wait();
    __half* hi = a.out + (size_t)t * 2 * a.K;
    __half* lo = hi + a.K;
    if (t >= a.T) {
        for (int k = threadIdx.x; k < a.K; k += 256) { hi[k] = __float2half(0.f); lo[k] = __float2half(0.f); }
        trace_out(a.trace);
        return;
    }
    const float* x = a.x + (size_t)t * a.x_stride;
    if (a.gn_w) {
        // DeltaNet output projection input: w * rmsnorm_DV(o) * silu(z) per value head. A thread takes 8 consecutive
        // values per turn, all of its loads in flight together; a head is DV / 8 neighbouring lanes.
        const float* z = a.z + (size_t)t * a.x_stride;
        constexpr int TURNS = 2;                        // K <= 256 threads * 8 * 2
        float xv[TURNS][8], zv[TURNS][8], gw[TURNS][8];
#pragma unroll
        for (int j = 0; j < TURNS; j++) {
            const int k = (threadIdx.x + j * 256) * 8;
            const bool has = k < a.K;
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0, z0 = v0, z1 = v0;
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (has) {
                v0 = *reinterpret_cast<const float4*>(x + k); v1 = *reinterpret_cast<const float4*>(x + k + 4);
                z0 = *reinterpret_cast<const float4*>(z + k); z1 = *reinterpret_cast<const float4*>(z + k + 4);
                wv = *reinterpret_cast<const uint4*>(a.gn_w + (k % a.DV));
            }
            xv[j][0] = v0.x; xv[j][1] = v0.y; xv[j][2] = v0.z; xv[j][3] = v0.w; xv[j][4] = v1.x; xv[j][5] = v1.y; xv[j][6] = v1.z; xv[j][7] = v1.w;
            zv[j][0] = z0.x; zv[j][1] = z0.y; zv[j][2] = z0.z; zv[j][3] = z0.w; zv[j][4] = z1.x; zv[j][5] = z1.y; zv[j][6] = z1.z; zv[j][7] = z1.w;
            gw[j][0] = bflo(wv.x); gw[j][1] = bfhi(wv.x); gw[j][2] = bflo(wv.y); gw[j][3] = bfhi(wv.y);
            gw[j][4] = bflo(wv.z); gw[j][5] = bfhi(wv.z); gw[j][6] = bflo(wv.w); gw[j][7] = bfhi(wv.w);
        }
#pragma unroll
        for (int j = 0; j < TURNS; j++) {
            const int k = (threadIdx.x + j * 256) * 8;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) ss = fmaf(xv[j][i], xv[j][i], ss);
            for (int o = a.DV >> 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float r = 1.0f / sqrtf(ss / (float)a.DV + a.eps);
            if (k < a.K) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float v = (gw[j][i] * (xv[j][i] * r)) * zv[j][i];
                    const __half h1 = __float2half(v);
                    hi[k + i] = h1;
                    lo[k + i] = __float2half(v - __half2float(h1));
                }
            }
        }
        trace_out(a.trace);
        return;
    }
    float r = 1.0f;
    if (a.norm_w) {
        float ss = 0.f;
        for (int k = threadIdx.x; k < a.K; k += 256) { const float v = x[k]; ss = fmaf(v, v, ss); }
        ss = block_sum(ss, red);
        r = 1.0f / sqrtf(ss / (float)a.K + a.eps);
    }
    for (int k = threadIdx.x; k < a.K; k += 256) {
        float v = x[k];
        if (a.norm_w) v = v * r * (1.0f + bf(a.norm_w[k]));
        vs[k] = v;
        const __half h1 = __float2half(v);
        const int ks = a.perm8 ? ((k & ~7) | ((k & 3) << 1) | ((k >> 2) & 1)) : k;
        hi[ks] = h1;
        lo[ks] = __float2half(v - __half2float(h1));
    }
    if (a.xsum) {
        __syncthreads();
        for (int g = threadIdx.x; g < a.K / 64; g += 256) {
            float s = 0.f;
            for (int i = 0; i < 64; i++) s += vs[64 * g + i];
            a.xsum[(size_t)t * (a.K / 64) + g] = s;
        }
    }
    trace_out(a.trace);
}

struct MmaSeg {
    const int8_t* w;         // [rows][K] int8, or [rows][K] bf16 for the SEG_BF* kinds
    const uint16_t* s;       // bf16 scale per row
    const int8_t* w2;        // SEG_I8_GATEUP: the up matrix
    const uint16_t* s2;
    const float* bias;       // SEG_BF only, may be null
    float* out;              // [T][out_stride]
    int rows, kind, out_stride;
    int blocks;              // ceil(rows / MM_ROWS), filled by the host
};

struct MmaArgs {
    unsigned long long* trace;   // step timeline slot of this launch, or null
    MmaSeg seg[4];
    int nseg, total_blocks;
    const __half* xh;        // [Tpad][2][K]
    int K, T;
    // SEG_I8_CONV
    const uint16_t* conv_w;
    float* conv_state;       // [T][C][3]
    // SEG_BF_DECAY
    const uint16_t* a_log;
    const uint16_t* dt_bias;
};

// eight bf16 (a 16-byte piece of a row) -> four half2. Exact for magnitudes from 2^-14 up; smaller ones round to
// the fp16 subnormal grid (absolute error below 2^-25).
__device__ __forceinline__ void bf16x8_to_h2x4(const uint4& w, uint32_t (&h)[4]) {
    const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 t = __floats2half2_rn(__uint_as_float(v[i] << 16), __uint_as_float(v[i] & 0xFFFF0000u));
        h[i] = *reinterpret_cast<const uint32_t*>(&t);
    }
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// four int8 -> two half2 (exact): bytes (0,1) and (2,3) of w
__device__ __forceinline__ void i8x4_to_h2x2(uint32_t w, uint32_t& h01, uint32_t& h23) {
    const uint32_t u = w ^ 0x80808080u;
    const uint32_t bias = 0x64806480u;                       // (1152, 1152)
    uint32_t a = __byte_perm(u, 0x64646464u, 0x4140);        // 1024 + (q0 + 128), 1024 + (q1 + 128)
    uint32_t b = __byte_perm(u, 0x64646464u, 0x4342);
    __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<const __half2*>(&bias));
    __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), *reinterpret_cast<const __half2*>(&bias));
    h01 = *reinterpret_cast<uint32_t*>(&ha);
    h23 = *reinterpret_cast<uint32_t*>(&hb);
}

// grid (total_blocks, passes of MM_TOK sequences). NS = stages of the K-chunk ring (the same sums in the same
// order for every NS). Warps 0-3 take sequences 0-15 of the pass, warps 4-7 sequences 16-31, each its 16-row slab:
// a block alone on an SM (matrices of few rows) then still has two warps per scheduler to hide the conversion and
// mma latencies, which is what bounds these launches.
template <int NS>
__global__ void __launch_bounds__(MM_THREADS) k_mma_i8(const MmaArgs a) {
    extern __shared__ __align__(128) unsigned char mm_smem[];
    const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) & 3, half = threadIdx.x >> 7;
    const int gid = lane >> 2, tid = lane & 3;
    const int t0 = blockIdx.y * MM_TOK;
    // this warp's four n-tiles of the 64 columns: hi parts 2 half, 2 half + 1, lo parts 4 + 2 half, 5 + 2 half
    const int ntile[4] = {2 * half, 2 * half + 1, 2 * half + 4, 2 * half + 5};
    grid_dep_launch();
    trace_in(a.trace, 10, gridDim.x);
    // which matrix and which 64 rows
    int s = 0, blk = blockIdx.x;
    while (s + 1 < a.nseg && blk >= a.seg[s].blocks) { blk -= a.seg[s].blocks; s++; }
    const MmaSeg sg = a.seg[s];
    const bool pair = sg.kind == SEG_I8_GATEUP;
    const bool isbf = sg.kind == SEG_BF || sg.kind == SEG_BF_SIGMOID || sg.kind == SEG_BF_DECAY;
    const int kcw = isbf ? MM_KC / 2 : MM_KC;         // weights per K chunk: a chunk is 256 bytes of a row either way
    // a pair block covers 32 gate rows and the same 32 up rows: warps 0,1 gate, warps 2,3 up
    const int rows_per_block = pair ? MM_ROWS / 2 : MM_ROWS;
    const int row0 = blk * rows_per_block;
    const int nk = a.K / kcw;

    auto load_stage = [&](int kc, int st) {
        unsigned char* sa = mm_smem + (size_t)st * MM_STAGE_BYTES;
        unsigned char* sb = sa + MM_ROWS * MM_PA;
        // weights: 64 rows x 256 B = 1024 16-byte pieces
        for (int p = threadIdx.x; p < MM_ROWS * (MM_KC / 16); p += MM_THREADS) {
            const int r = p / (MM_KC / 16), c = p % (MM_KC / 16);
            int grow;
            const int8_t* base;
            if (pair) { base = r < 32 ? sg.w : sg.w2; grow = row0 + (r & 31); }
            else { base = sg.w; grow = row0 + r; }
            grow = min(grow, sg.rows - 1);                    // rows past the end repeat the last row (never stored)
            cp_async16(sa + r * MM_PA + c * 16, base + ((size_t)grow * a.K + (size_t)kc * kcw) * (isbf ? 2 : 1) + c * 16);
        }
        // activations: 64 columns (32 sequences x hi, lo) x 256 halves = 2048 pieces
        const int pcs = kcw / 8, psh = isbf ? 4 : 5;                           // 16-byte pieces per column: 16 or 32
        for (int p = threadIdx.x; p < 2 * MM_TOK * pcs; p += MM_THREADS) {
            const int col = p >> psh, c = p & (pcs - 1);
            const int tok = t0 + (col & (MM_TOK - 1)), part = col >> 5;        // columns 0..31 hi, 32..63 lo
            cp_async16(sb + col * MM_PB + c * 16, a.xh + ((size_t)tok * 2 + part) * a.K + (size_t)kc * kcw + c * 8);
        }
        cp_async_commit();
    };

    grid_dep_wait();          // the activations are the previous kernel's output
    for (int i = 0; i < NS - 1; i++) {
        if (i < nk) load_stage(i, i); else cp_async_commit();
    }
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[j][q] = 0.f;

    for (int kc = 0; kc < nk; kc++) {
        cp_async_wait<NS - 2>();
        __syncthreads();
        if (kc + NS - 1 < nk) load_stage(kc + NS - 1, (kc + NS - 1) % NS); else cp_async_commit();
        const unsigned char* sa = mm_smem + (size_t)(kc % NS) * MM_STAGE_BYTES;
        const unsigned char* sb = sa + MM_ROWS * MM_PA;
        const unsigned char* ar0 = sa + (warp * 16 + gid) * MM_PA;
        const unsigned char* ar1 = ar0 + 8 * MM_PA;
        if (isbf) {
            // bf16 rows: 64 bytes of a row are 32 weights = two k16 steps; a lane takes 8 consecutive weights
#pragma unroll
            for (int sbk = 0; sbk < MM_KC / 64; sbk++) {
                const uint4 w0 = *reinterpret_cast<const uint4*>(ar0 + sbk * 64 + tid * 16);
                const uint4 w1 = *reinterpret_cast<const uint4*>(ar1 + sbk * 64 + tid * 16);
                uint32_t h0[4], h1[4];
                bf16x8_to_h2x4(w0, h0);
                bf16x8_to_h2x4(w1, h1);
                const uint32_t afa[4] = {h0[0], h1[0], h0[1], h1[1]}, afb[4] = {h0[2], h1[2], h0[3], h1[3]};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint4 x0 = *reinterpret_cast<const uint4*>(sb + (ntile[j] * 8 + gid) * MM_PB + sbk * 64 + tid * 16);
                    mma16816(acc[j], afa, x0.x, x0.y);
                    mma16816(acc[j], afb, x0.z, x0.w);
                }
            }
            continue;
        }
#pragma unroll
        for (int sbk = 0; sbk < MM_KC / 64; sbk++) {
            // this thread's 16 bytes of rows gid and gid + 8 cover four k16 steps
            const uint4 w0 = *reinterpret_cast<const uint4*>(ar0 + sbk * 64 + tid * 16);
            const uint4 w1 = *reinterpret_cast<const uint4*>(ar1 + sbk * 64 + tid * 16);
            const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w}, wb[4] = {w1.x, w1.y, w1.z, w1.w};
            uint32_t af[4][4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                i8x4_to_h2x2(wa[j], af[j][0], af[j][2]);
                i8x4_to_h2x2(wb[j], af[j][1], af[j][3]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                // column 8 nt + gid: 16 halves = this thread's k range of the super-block
                const unsigned char* bp = sb + (ntile[j] * 8 + gid) * MM_PB + sbk * 128 + tid * 32;
                const uint4 x0 = *reinterpret_cast<const uint4*>(bp);
                const uint4 x1 = *reinterpret_cast<const uint4*>(bp + 16);
                mma16816(acc[j], af[0], x0.x, x0.y);
                mma16816(acc[j], af[1], x0.z, x0.w);
                mma16816(acc[j], af[2], x1.x, x1.y);
                mma16816(acc[j], af[3], x1.z, x1.w);
            }
        }
    }
    cp_async_wait<0>();

    // epilogue. Thread holds rows (gid, gid + 8) of its warp's slab and, in n-tile nt, columns 2 tid, 2 tid + 1:
    // sequences 8 nt + 2 tid (+1) for nt < 4 (hi, acc[0], acc[1]) and the same sequences' lo parts (acc[2], acc[3]).
    __shared__ float gate_s[2][16][MM_TOK + 1];     // pairs: the gate warps hand their sums to the up warps
    if (pair && warp < 2) {
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int r = gid + (q >> 1) * 8, col = ntile[j] * 8 + 2 * tid + (q & 1);
                gate_s[warp][r][col] = acc[j][q] + acc[j + 2][q];
            }
    }
    if (pair) __syncthreads();
    if (pair && warp < 2) { trace_out(a.trace); return; }
#pragma unroll
    for (int j = 0; j < 2; j++) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int rl = gid + (q >> 1) * 8;                               // row inside the warp's slab
            const int col = ntile[j] * 8 + 2 * tid + (q & 1);
            const int tok = t0 + col;
            const int row = pair ? row0 + (warp - 2) * 16 + rl : row0 + warp * 16 + rl;
            if (tok >= a.T || row >= sg.rows) continue;
            const float dot = acc[j][q] + acc[j + 2][q];
            float* out = sg.out + (size_t)tok * sg.out_stride;
            switch (sg.kind) {
            case SEG_I8: out[row] = bf(sg.s[row]) * dot; break;
            case SEG_I8_SILU: out[row] = siluf_(bf(sg.s[row]) * dot); break;
            case SEG_I8_ACC: out[row] += bf(sg.s[row]) * dot; break;
            case SEG_I8_GATEUP: out[row] = siluf_(bf(sg.s[row]) * gate_s[warp - 2][rl][col]) * (bf(sg.s2[row]) * dot); break;
            case SEG_I8_CONV: {
                const float raw = bf(sg.s[row]) * dot;
                float* stt = a.conv_state + ((size_t)tok * sg.rows + row) * 3;
                const uint2 cw = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)row * 4);
                const float s0 = stt[0], s1 = stt[1], s2 = stt[2];
                float y = bflo(cw.x) * s0;
                y = fmaf(bfhi(cw.x), s1, y);
                y = fmaf(bflo(cw.y), s2, y);
                y = fmaf(bfhi(cw.y), raw, y);
                stt[0] = s1; stt[1] = s2; stt[2] = raw;
                out[row] = siluf_(y);
            } break;
            case SEG_BF: out[row] = dot + (sg.bias ? sg.bias[row] : 0.f); break;
            case SEG_BF_SIGMOID: out[row] = sigmoidf_(dot); break;
            case SEG_BF_DECAY: out[row] = -expf(bf(a.a_log[row])) * softplusf_(dot + bf(a.dt_bias[row])); break;
            default: break;
            }
        }
    }
    trace_out(a.trace);
}

}  // namespace b2
