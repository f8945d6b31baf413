// k_umma: the int8 (and bf16-row) linears for many tokens as a Blackwell tensor-core GEMM.
//
//   out[t][row] = epilogue(scale[row] * sum_k W[row][k] x[t][k])        rows x K weights, T tokens
//
// With 6 or more tokens (batched decode, prompt chunks) the linears are dense contractions. The fifth-generation
// tensor cores take both operands straight from shared memory and keep the accumulator in tensor memory, so no
// warp touches a weight byte:
//
//   producer warp   one elected lane: TMA tensor copies (cp.async.bulk.tensor, 128-byte swizzle) of a 128-row x 128-byte
//                   weight box and of the activation planes of the unit's tokens into a 5-stage ring, mbarrier-tracked
//   MMA warp        one elected lane: tcgen05.mma (M 128, N tokens x planes, K 32 bytes) four times per stage, operands
//                   described by shared-memory descriptors, accumulators in TMEM; tcgen05.commit releases the stage and,
//                   after the last K chunk, hands the accumulator to the epilogue. Two accumulators alternate, so the
//                   products of the next unit run under the epilogue of this one.
//   8 epilogue warps  thread = weight row = TMEM lane (two warps per quarter of the lanes, 16 tokens at a time each): tcgen05.ld, the planes of a token combined, row scale, the
//                   launch's epilogue (SiLU, gate * up, conv with its state, += residual, ...), coalesced stores
//
// Arithmetic. int8 weights are multiplied as stored (kind::i8, s32 accumulators: exact) with the activations split
// into three int8 digit planes per token, x = s (d0 + d1/128 + d2/128^2) (the small-batch kernels carry a fourth plane,
// digits.cuh), which holds every activation to 2^-21 of the token's largest. bf16 rows (router, DeltaNet a/b, shared gate) are multiplied as stored (kind::f16, f32 accumulators)
// with the activations as three bf16 planes, x = hi + mid + lo exactly; every product is exact in fp32.
//
// The K loop walks 128-byte chunks of a row (128 int8 or 64 bf16 weights). A unit of work is (128 weight rows, tt
// tokens), tt = 64, 32 or 16: a block pulls at most about 110 GB/s out of L2, so a matrix of few rows is split over
// the tokens as well until the units fill the SMs. A block walks units blockIdx.x, + gridDim.x, ... Every wait is a bounded mbarrier wait (mbar_wait): on a
// time-out the error word is set and the thread skips its later waits; the producer stops issuing copies and waits
// (bounded) for those in flight; the kernel runs to its end, frees its tensor memory and returns.
#pragma once
#include <cuda.h>

namespace b2 {

constexpr int UM_MAX_STAGES = 12;          // the ring holds as many stages as fit: what a block has in flight bounds what it pulls
constexpr int UM_M = 128;                  // weight rows per unit = TMEM lanes
constexpr int UM_TOK = 64;                 // tokens per unit
constexpr int UM_BK = 128;                 // bytes of a row per K chunk (the swizzle span)
constexpr int UM_PI = 3;                   // int8 digit planes: x = s (d0 + d1/128 + d2/128^2), 2^-21 of the token's largest value
constexpr int UM_PB = 3;                   // bf16 planes
constexpr int UM_A_BYTES = UM_M * UM_BK;                     // 16 KB
constexpr int UM_RING_BYTES = 200 * 1024;
// A stage holds KC K chunks (each a 128-row x 128-byte weight box + the tokens' planes): the hand-over of a stage between
// the producer and the MMA lane (two mbarrier operations on either side) costs about 400 cycles whatever it carries, more
// than four products over few tokens take, so units of 32 or 16 tokens move two chunks per stage.
__host__ __device__ constexpr int um_kc(int tt) { return tt >= 64 ? 1 : 2; }
__host__ __device__ constexpr int um_chunk_bytes(int tt) { return UM_A_BYTES + tt * UM_PI * UM_BK; }      // 40, 28 or 22 KB
__host__ __device__ constexpr int um_stage_bytes(int tt) { return um_kc(tt) * um_chunk_bytes(tt); }       // 40, 56 or 44 KB
__host__ __device__ constexpr int um_stages(int tt) { return UM_RING_BYTES / um_stage_bytes(tt) < UM_MAX_STAGES ? UM_RING_BYTES / um_stage_bytes(tt) : UM_MAX_STAGES; }
static_assert(UM_PI == UM_PB, "int8 and bf16 rows share the stage layout");
constexpr int UM_THREADS = 320;            // producer, MMA, 8 epilogue warps (two per quarter of the TMEM lanes)
constexpr int UM_TMEM_COLS = 512;          // two accumulators of up to 256 columns
constexpr size_t UM_SMEM = (size_t)UM_RING_BYTES + 1024;                // + room to align the ring to 1024 bytes

struct UmmaSeg {
    const uint16_t* s;       // bf16 scale per row (int8 kinds)
    const uint16_t* s2;      // SEG_I8_GATEUP: the up matrix's scales
    const float* bias;       // SEG_BF only, may be null
    float* out;              // [T][out_stride]
    int rows, kind, out_stride;
    int units;               // row blocks: ceil(rows / 128), or ceil(rows / 64) for a gate/up pair
};

struct UmmaArgs {
    CUtensorMap wmap[GEMV_MAX_SEG];     // weights of each segment as a [rows][K bytes] tensor, box 128 bytes x 64 rows
    CUtensorMap wmap2[GEMV_MAX_SEG];    // SEG_I8_GATEUP: the up matrix
    CUtensorMap xmap_i8;     // int8 planes [passes * 3 * 64][K], box 128 bytes x tt rows (one box per plane)
    CUtensorMap xmap_bf;     // bf16 planes [passes * 3 * 64][2 K bytes], box 128 bytes x tt rows
    unsigned long long* trace;
    UmmaSeg seg[GEMV_MAX_SEG];
    int nseg, total_units;   // total_units = sum of seg units
    int K, T, passes;        // passes = ceil(T / 64)
    int tt;                  // tokens per unit of work: 64, 32 or 16 (the planes' tensor maps have boxes of `tt` rows)
    const float* xscale;     // [passes * 64] scale of each token's int8 planes
    const uint16_t* conv_w;  // SEG_I8_CONV (decode: one token per sequence, state per sequence)
    float* conv_state;       // [T][C][3]
    const uint16_t* a_log;   // SEG_BF_DECAY
    const uint16_t* dt_bias;
    int* err;
};

// ---- tcgen05 / TMA wrappers -------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// the mbarrier gets one arrival when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; `accumulate` = 0 overwrites D
__device__ __forceinline__ void umma_i8(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(adesc),
                 "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(adesc),
                 "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand in 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride byte offset), leading byte offset unused (1), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: dense, D format (0 f16, 1 f32, 2 s32) at bit 4, A format at 7, B format at 10, both K-major,
// N / 8 at bit 17, M / 16 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t dfmt, uint32_t abfmt, uint32_t M, uint32_t N) {
    return (dfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

__global__ void __launch_bounds__(UM_THREADS, 1) k_umma(const __grid_constant__ UmmaArgs a) {
    extern __shared__ unsigned char um_raw[];
    __shared__ __align__(8) uint64_t full_bar[UM_MAX_STAGES], empty_bar[UM_MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ float gate_x[2][64][17];              // gate/up pairs: the gate rows' values of 16 tokens, per half of the tokens
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* ring = um_raw + ((1024u - (smem_u32(um_raw) & 1023u)) & 1023u);
    grid_dep_launch();
    trace_in(a.trace, 14, gridDim.x);
    if (threadIdx.x == 0) {
        for (int s = 0; s < UM_MAX_STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&tmem_slot, UM_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int NST = um_stages(a.tt), STAGE = um_stage_bytes(a.tt), KC = um_kc(a.tt), CHUNK = um_chunk_bytes(a.tt);
    // token groups of a pass; with a single pass only the groups that hold tokens are counted, so that the work items
    // that exist spread over all blocks
    const int nsub = a.passes == 1 ? (min(a.T, UM_TOK) + a.tt - 1) / a.tt : UM_TOK / a.tt;
    const int nwork = a.total_units * a.passes * nsub;       // (row block, pass of 64 tokens, token group), token groups innermost
    // work item w -> unit, pass, first token; false when the group holds no token at all (every role skips it alike)
    auto decode = [&](int w, int& unit, int& pass, int& sub) {
        sub = w % nsub;
        const int r = w / nsub;
        pass = r % a.passes;
        unit = r / a.passes;
        return pass * UM_TOK + sub * a.tt < a.T;
    };
    // activations (and residuals, conv state) are earlier launches' results; the weights are not, so the producer warp
    // sends the weight copies of its first stages before it waits
    if (warp != 0) grid_dep_wait();

    // step-timeline points of block 0 (any thread may stamp): 1 past the dependency wait, 2 the producer has issued its
    // last copy, 3 the MMA lane has committed its last unit, 4 the epilogue got its first accumulator, 5 the epilogue is done
    auto stamp = [&](int i) {
        if (a.trace && blockIdx.x == 0) a.trace[8 + i] = (unsigned long long)clock64();
    };
    // A bounded wait. `dead` is the caller's own flag: after one of its waits has given up, a thread skips the rest
    // and runs to the end of its loops; the other roles' waits then give up the same way.
    auto wait = [&](uint64_t* bar, uint32_t parity, bool& dead) {
        if (dead) return;
        if (!mbar_wait(bar, parity, a.err, 1 << 21)) dead = true;
    };
    auto locate = [&](int unit, int& s, int& blk) {
        s = 0; blk = unit;
        while (s + 1 < a.nseg && blk >= a.seg[s].units) { blk -= a.seg[s].units; s++; }
    };

    if (warp == 0) {
        // ---- producer: lane 0 waits for the stage and announces the bytes, then lanes 0 .. 5 KC - 1 issue one tensor copy
        // each: per K chunk the two 64-row halves of the weight box and the three planes ----
        int st = 0, ph = 0;
        bool dead = false;
        uint32_t armed_mask = 0, armed_par = 0;     // stages with a copy group sent, and the parity of the latest one
        const int ck = lane / 5, which = lane - ck * 5;      // this lane's chunk of the stage and its copy within the chunk
        // what a lane copies for a work item: its tensor map, row coordinate and place in the stage
        struct Item { const CUtensorMap* map; int y, off, nk; bool ok; };
        auto item = [&](int w) {
            Item it{nullptr, 0, 0, 0, false};
            int unit, pass, sub;
            if (!decode(w, unit, pass, sub)) return it;
            int s, blk;
            locate(unit, s, blk);
            const int kind = a.seg[s].kind;
            const bool isbf = kind == SEG_BF || kind == SEG_BF_SIGMOID || kind == SEG_BF_DECAY;
            const bool pair = kind == SEG_I8_GATEUP;
            it.nk = (isbf ? 2 * a.K : a.K) / UM_BK;                   // K chunks of the unit
            it.map = which >= 2 ? (isbf ? &a.xmap_bf : &a.xmap_i8) : (pair && which == 1 ? &a.wmap2[s] : &a.wmap[s]);
            it.y = which >= 2 ? (pass * UM_PI + (which - 2)) * UM_TOK + sub * a.tt : (pair ? blk * 64 : blk * UM_M + which * 64);
            it.off = ck * CHUNK + (which >= 2 ? UM_A_BYTES + (which - 2) * a.tt * UM_BK : which * 64 * UM_BK);
            it.ok = true;
            return it;
        };
        // before the wait: the weight copies (lanes with which < 2) of the first work item's first stages, whose barriers
        // are armed for the whole stage; after it, the plane copies of the same stages. The loop below goes on from there.
        int w_first = blockIdx.x, pre = 0;
        while (w_first < nwork && !item(w_first).ok) w_first += gridDim.x;
        if (w_first < nwork) {
            const Item it = item(w_first);
            for (int k0 = 0; k0 < it.nk && pre < NST; k0 += KC, pre++) {
                const int nch = min(KC, it.nk - k0);
                if (lane == 0) mbar_expect_tx(&full_bar[pre], (uint32_t)nch * CHUNK);
                __syncwarp();
                if (lane < 5 * nch && which < 2) tma_load_2d(ring + (size_t)pre * STAGE + it.off, it.map, (k0 + ck) * UM_BK, it.y, &full_bar[pre]);
            }
            grid_dep_wait();
            if (lane == 0) stamp(1);
            for (int j = 0; j < pre; j++) {
                const int k0 = j * KC, nch = min(KC, it.nk - k0);
                if (lane < 5 * nch && which >= 2) tma_load_2d(ring + (size_t)j * STAGE + it.off, it.map, (k0 + ck) * UM_BK, it.y, &full_bar[j]);
                armed_mask |= 1u << j;                                  // parity 0: the first use of these stages
            }
            st = pre == NST ? 0 : pre;
            ph = pre == NST ? 1 : 0;
        } else {
            grid_dep_wait();
            if (lane == 0) stamp(1);
        }
        for (int w = w_first; w < nwork; w += gridDim.x) {
            const Item it = item(w);
            if (!it.ok) continue;
            for (int k0 = (w == w_first ? pre * KC : 0); k0 < it.nk; k0 += KC) {
                const int nch = min(KC, it.nk - k0);                    // chunks in this stage
                if (lane == 0) {
                    wait(&empty_bar[st], ph ^ 1, dead);
                    if (!dead) mbar_expect_tx(&full_bar[st], (uint32_t)nch * CHUNK);
                }
                dead = __shfl_sync(0xffffffffu, (int)dead, 0) != 0;
                if (dead) break;
                if (lane < 5 * nch) tma_load_2d(ring + (size_t)st * STAGE + it.off, it.map, (k0 + ck) * UM_BK, it.y, &full_bar[st]);
                armed_mask |= 1u << st;
                armed_par = (armed_par & ~(1u << st)) | ((uint32_t)ph << st);
                if (++st == NST) { st = 0; ph ^= 1; }
            }
            if (dead) break;
        }
        __syncwarp();
        if (lane == 0) {
            stamp(2);
            if (dead)                                // copies still in flight must land before the block may leave
                for (int i = 0; i < UM_MAX_STAGES; i++)
                    if (armed_mask >> i & 1) mbar_wait(&full_bar[i], (armed_par >> i) & 1u, nullptr, 1 << 16);
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            int st = 0, ph = 0, n = 0;
            bool dead = false;
            for (int w = blockIdx.x; w < nwork; w += gridDim.x) {
                int unit, pass, sub;
                if (!decode(w, unit, pass, sub)) continue;
                int s, blk;
                locate(unit, s, blk);
                const int kind = a.seg[s].kind;
                const bool isbf = kind == SEG_BF || kind == SEG_BF_SIGMOID || kind == SEG_BF_DECAY;
                const int nk = (isbf ? 2 * a.K : a.K) / UM_BK;
                const uint32_t idesc = isbf ? umma_idesc(1, 1, UM_M, a.tt * UM_PB) : umma_idesc(2, 1, UM_M, a.tt * UM_PI);
                const int buf = n & 1;
                wait(&acc_empty[buf], ((n >> 1) & 1) ^ 1, dead);            // the epilogue has read this accumulator
                tc_fence_after();
                const uint32_t d = tmem + (uint32_t)buf * 256u;
                for (int k0 = 0; k0 < nk; k0 += KC) {
                    wait(&full_bar[st], ph, dead);
                    tc_fence_after();
                    const int nch = min(KC, nk - k0);
                    for (int c = 0; c < nch; c++) {
                        const uint32_t sa = smem_u32(ring + (size_t)st * STAGE + (size_t)c * CHUNK);
                        const uint64_t ad = umma_desc_sw128(sa), bd = umma_desc_sw128(sa + UM_A_BYTES);
#pragma unroll
                        for (int k = 0; k < UM_BK / 32; k++) {
                            // 32 bytes further along K inside the swizzle span: + 2 in the descriptor's address field
                            const uint32_t acc = (k0 + c != 0 || k != 0) ? 1u : 0u;
                            if (isbf) umma_f16(d, ad + 2 * k, bd + 2 * k, idesc, acc);
                            else umma_i8(d, ad + 2 * k, bd + 2 * k, idesc, acc);
                        }
                    }
                    umma_commit(&empty_bar[st]);                          // the stage may be refilled once these have read it
                    if (++st == NST) { st = 0; ph ^= 1; }
                }
                umma_commit(&acc_full[buf]);
                n++;
            }
            stamp(3);
        }
    } else {
        // ---- epilogue: warp w may touch TMEM lanes 32 (w % 4) .. + 31 ----
        // warps 2..5 take tokens 0..31 of the unit, warps 6..9 tokens 32..63
        const int q = warp & 3, th = (warp - 2) >> 2;
        const int vrow = q * 32 + lane;                                  // row of the unit = TMEM lane
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        int n = 0;
        bool dead = false;
        for (int w = blockIdx.x; w < nwork; w += gridDim.x) {
            int unit, pass, sub;
            if (!decode(w, unit, pass, sub)) continue;
            int s, blk;
            locate(unit, s, blk);
            const UmmaSeg& sg = a.seg[s];
            const int kind = sg.kind;
            const bool isbf = kind == SEG_BF || kind == SEG_BF_SIGMOID || kind == SEG_BF_DECAY;
            const bool pair = kind == SEG_I8_GATEUP;
            const int row = pair ? blk * 64 + (vrow & 63) : blk * UM_M + vrow;
            const bool rok = row < sg.rows;
            const int buf = n & 1;
            // what the epilogue needs from global memory, asked for before the accumulator is waited for
            float rs = 1.f, e1 = 0.f;
            uint2 cw = make_uint2(0u, 0u);
            if (rok) {
                if (!isbf) rs = bf(pair && vrow >= 64 ? sg.s2[row] : sg.s[row]);
                if (kind == SEG_BF) rs = sg.bias ? sg.bias[row] : 0.f;
                if (kind == SEG_BF_DECAY) { rs = bf(a.a_log[row]); e1 = bf(a.dt_bias[row]); }
                if (kind == SEG_I8_CONV) cw = *reinterpret_cast<const uint2*>(a.conv_w + (size_t)row * 4);
            }
            wait(&acc_full[buf], (n >> 1) & 1, dead);
            tc_fence_after();
            if (n == 0 && threadIdx.x == 64) stamp(4);
            const uint32_t base = tmem + lane_addr + (uint32_t)buf * 256u;
            for (int c = th; c < a.tt / 16; c += 2) {                   // the two warps of a lane quarter take the chunks in turn
                const int t0 = pass * UM_TOK + sub * a.tt + c * 16;
                if (n == 0 && c == 1 && threadIdx.x == 64) stamp(7);
                if (t0 >= a.T) break;                                    // uniform over the block
                float v[16];
                {
                    uint32_t d0[16], d1[16], d2[16];
                    tmem_ld16(base + 0 * a.tt + c * 16, d0);
                    tmem_ld16(base + 1 * a.tt + c * 16, d1);
                    tmem_ld16(base + 2 * a.tt + c * 16, d2);
                    tmem_ld_wait();
                    if (n == 0 && c == 0 && threadIdx.x == 64) stamp(6);
                    if (isbf) {
#pragma unroll
                        for (int i = 0; i < 16; i++) v[i] = (__uint_as_float(d2[i]) + __uint_as_float(d1[i])) + __uint_as_float(d0[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const float f = (float)(int)d2[i] * (1.0f / 128.0f) + (float)(int)d1[i];
                            v[i] = (f * (1.0f / 128.0f) + (float)(int)d0[i]) * __ldg(a.xscale + t0 + i);
                        }
                    }
                }
                if (pair) {
                    if (vrow < 64) {
#pragma unroll
                        for (int i = 0; i < 16; i++) gate_x[th][vrow][i] = rs * v[i];
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + th) : "memory");
                    if (vrow >= 64 && rok) {
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            if (t0 + i < a.T) sg.out[(size_t)(t0 + i) * sg.out_stride + row] = siluf_(gate_x[th][vrow - 64][i]) * (rs * v[i]);
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + th) : "memory");
                    continue;
                }
                if (!rok) continue;
                // one thread owns a row for all 64 tokens: what it reads from global memory for the 16 tokens of a chunk is
                // requested together (16 independent loads in flight), never one token after the other
                if (kind == SEG_I8_CONV) {
                    // aegist/hybrid.py:393-398: y = silu(sum_j w[c][j] * taps[j]), taps = 3 previous inputs + the new one
                    float s0[16], s1[16], s2[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int t = min(t0 + i, a.T - 1);
                        const float* stt = a.conv_state + ((size_t)t * sg.rows + row) * 3;
                        s0[i] = stt[0]; s1[i] = stt[1]; s2[i] = stt[2];
                    }
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int t = t0 + i;
                        if (t >= a.T) break;
                        const float raw = rs * v[i];
                        float y = bflo(cw.x) * s0[i];
                        y = fmaf(bfhi(cw.x), s1[i], y);
                        y = fmaf(bflo(cw.y), s2[i], y);
                        y = fmaf(bfhi(cw.y), raw, y);
                        float* stt = a.conv_state + ((size_t)t * sg.rows + row) * 3;
                        stt[0] = s1[i]; stt[1] = s2[i]; stt[2] = raw;
                        sg.out[(size_t)t * sg.out_stride + row] = siluf_(y);
                    }
                    continue;
                }
                if (kind == SEG_I8_ACC) {
                    float old[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) old[i] = sg.out[(size_t)min(t0 + i, a.T - 1) * sg.out_stride + row];
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        if (t0 + i < a.T) sg.out[(size_t)(t0 + i) * sg.out_stride + row] = old[i] + rs * v[i];
                    continue;
                }
                // the remaining kinds only store: the value first (kind is uniform over the block), then 16 predicated stores
                float y[16];
                if (kind == SEG_I8_SILU) {
#pragma unroll
                    for (int i = 0; i < 16; i++) y[i] = siluf_(rs * v[i]);
                } else if (kind == SEG_BF) {
#pragma unroll
                    for (int i = 0; i < 16; i++) y[i] = v[i] + rs;
                } else if (kind == SEG_BF_SIGMOID) {
#pragma unroll
                    for (int i = 0; i < 16; i++) y[i] = sigmoidf_(v[i]);
                } else if (kind == SEG_BF_DECAY) {
                    const float ea = -expf(rs);
#pragma unroll
                    for (int i = 0; i < 16; i++) y[i] = ea * softplusf_(v[i] + e1);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) y[i] = rs * v[i];
                }
                float* out = sg.out + (size_t)t0 * sg.out_stride + row;
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (t0 + i < a.T) out[(size_t)i * sg.out_stride] = y[i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            n++;
        }
        if (threadIdx.x == 64) stamp(5);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { __syncwarp(); tmem_dealloc(tmem, UM_TMEM_COLS); }
    trace_out(a.trace);
}

// ---- activations -> planes ------------------------------------------------------------------------------------
struct PrepQArgs {
    unsigned long long* trace;
    const float* x;          // [T][x_stride]
    int x_stride;
    const uint16_t* norm_w;  // ZNorm weight [K] or null
    const uint16_t* gn_w;    // gated RMSNorm weight [DV] or null (then z is silu(z))
    const float* z;
    int DV;
    float eps;
    int K, T;
    int8_t* qi;              // [passes][3][64][K] int8 digit planes, or null
    uint16_t* qb;            // [passes][3][64][K] bf16 planes, or null
    float* xscale;           // [passes * 64]
};

// one block of 256 threads per token slot (passes * 64 slots; slots past T are zero); K <= 4096
__global__ void __launch_bounds__(256) k_prep_q(const PrepQArgs a) {
    __shared__ float red[2][8];
    const int t = blockIdx.x, pass = t / UM_TOK, tt = t % UM_TOK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    grid_dep_launch();
    trace_in(a.trace, 15, gridDim.x);
    grid_dep_wait();
    constexpr int TURNS = 2;                             // K <= 256 threads * 8 * 2
    float xv[TURNS][8];
    const bool live = t < a.T;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < TURNS; j++) {
        const int k = (threadIdx.x + j * 256) * 8;
        float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
        if (live && k < a.K) {
            v0 = *reinterpret_cast<const float4*>(a.x + (size_t)t * a.x_stride + k);
            v1 = *reinterpret_cast<const float4*>(a.x + (size_t)t * a.x_stride + k + 4);
        }
        xv[j][0] = v0.x; xv[j][1] = v0.y; xv[j][2] = v0.z; xv[j][3] = v0.w; xv[j][4] = v1.x; xv[j][5] = v1.y; xv[j][6] = v1.z; xv[j][7] = v1.w;
        if (a.gn_w) {
            // DeltaNet out projection input: w * rmsnorm_DV(o) * silu(z) per value head (aegist/hybrid.py:133-147); a head is DV / 8 lanes
            float4 z0 = make_float4(0.f, 0.f, 0.f, 0.f), z1 = z0;
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (live && k < a.K) {
                z0 = *reinterpret_cast<const float4*>(a.z + (size_t)t * a.x_stride + k);
                z1 = *reinterpret_cast<const float4*>(a.z + (size_t)t * a.x_stride + k + 4);
                wv = *reinterpret_cast<const uint4*>(a.gn_w + (k % a.DV));
            }
            const float zz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
            const float gw[8] = {bflo(wv.x), bfhi(wv.x), bflo(wv.y), bfhi(wv.y), bflo(wv.z), bfhi(wv.z), bflo(wv.w), bfhi(wv.w)};
            float s8 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) s8 = fmaf(xv[j][i], xv[j][i], s8);
            for (int o = a.DV >> 4; o > 0; o >>= 1) s8 += __shfl_xor_sync(0xffffffffu, s8, o);
            const float r = 1.0f / sqrtf(s8 / (float)a.DV + a.eps);
#pragma unroll
            for (int i = 0; i < 8; i++) xv[j][i] = (gw[i] * (xv[j][i] * r)) * zz[i];
        } else if (a.norm_w) {
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (k < a.K) wv = *reinterpret_cast<const uint4*>(a.norm_w + k);
            const float nw[8] = {1.0f + bflo(wv.x), 1.0f + bfhi(wv.x), 1.0f + bflo(wv.y), 1.0f + bfhi(wv.y),
                                 1.0f + bflo(wv.z), 1.0f + bfhi(wv.z), 1.0f + bflo(wv.w), 1.0f + bfhi(wv.w)};
#pragma unroll
            for (int i = 0; i < 8; i++) { ss = fmaf(xv[j][i], xv[j][i], ss); xv[j][i] *= nw[i]; }
        }
    }
    float mx = 0.f;
#pragma unroll
    for (int j = 0; j < TURNS; j++)
#pragma unroll
        for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(xv[j][i]));
    ss = warp_sum(ss);
    mx = warp_max(mx);
    if (lane == 0) { red[0][warp] = ss; red[1][warp] = mx; }
    __syncthreads();
    ss = 0.f; mx = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) { ss += red[0][w]; mx = fmaxf(mx, red[1][w]); }
    if (a.norm_w && !a.gn_w) {
        // (1 + w) * x / rms(x) (aegist/hybrid.py:119-130): the rms is one factor for the whole row
        const float rn = 1.0f / sqrtf(ss / (float)a.K + a.eps);
#pragma unroll
        for (int j = 0; j < TURNS; j++)
#pragma unroll
            for (int i = 0; i < 8; i++) xv[j][i] *= rn;
        mx *= rn;
    }
    const float inv = mx > 1e-30f ? 127.0f / mx : 0.f;
    if (threadIdx.x == 0 && a.xscale) a.xscale[t] = mx / 127.0f;
#pragma unroll
    for (int j = 0; j < TURNS; j++) {
        const int k = (threadIdx.x + j * 256) * 8;
        if (k >= a.K) continue;
        if (a.qi) {
            // q = v * inv (|q| <= 127) rounded once to a multiple of 2^-14, then split into balanced base-128 digits:
            // d1, d2 in [-64, 63], d0 what remains (|d0| <= 127)
            uint32_t w[UM_PI][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int qv = __float2int_rn(xv[j][i] * inv * 16384.0f);
                const int d2 = ((qv + 64) & 127) - 64;
                qv = (qv - d2) >> 7;
                const int d1 = ((qv + 64) & 127) - 64;
                const int d0 = (qv - d1) >> 7;
                const int sh = 8 * (i & 3);
                w[0][i >> 2] |= (uint32_t)(d0 & 255) << sh; w[1][i >> 2] |= (uint32_t)(d1 & 255) << sh; w[2][i >> 2] |= (uint32_t)(d2 & 255) << sh;
            }
#pragma unroll
            for (int p = 0; p < UM_PI; p++)
                *reinterpret_cast<uint2*>(a.qi + (((size_t)pass * UM_PI + p) * UM_TOK + tt) * a.K + k) = make_uint2(w[p][0], w[p][1]);
        }
        if (a.qb) {
            uint32_t h[4], m[4], l[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint16_t h0, m0, l0, h1, m1, l1;
                split3_bf16(xv[j][2 * i], h0, m0, l0);
                split3_bf16(xv[j][2 * i + 1], h1, m1, l1);
                h[i] = (uint32_t)h0 | ((uint32_t)h1 << 16); m[i] = (uint32_t)m0 | ((uint32_t)m1 << 16); l[i] = (uint32_t)l0 | ((uint32_t)l1 << 16);
            }
            uint16_t* b0 = a.qb + (((size_t)pass * UM_PB + 0) * UM_TOK + tt) * a.K + k;
            *reinterpret_cast<uint4*>(b0) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4*>(b0 + (size_t)UM_TOK * a.K) = make_uint4(m[0], m[1], m[2], m[3]);
            *reinterpret_cast<uint4*>(b0 + (size_t)2 * UM_TOK * a.K) = make_uint4(l[0], l[1], l[2], l[3]);
        }
    }
    trace_out(a.trace);
}

}  // namespace b2
