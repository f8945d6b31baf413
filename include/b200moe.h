/* b200moe: C ABI of the B200-native decode engine for the hybrid-MoE token loop.
 *
 * Every entry point replaces one piece of the reference's Rust engine (paths are relative to
 * aegist-fast-35b/ in the reference tree). The boundary is `trait Lm` (aegist_rs/src/model.rs:363-427)
 * as implemented by `HybridEngine` (aegist_rs/src/hybrid.rs:1015-1119): plain pointers and sizes,
 * ids are u32, logits are f32[vocab], errors are a non-zero return code plus a message
 * (`b2_last_error`), never an abort.
 *
 * Threading: one engine is used by one thread at a time (the reference takes `&mut self`).
 * All functions returning int return 0 on success.
 */
#ifndef B200MOE_H
#define B200MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b2_engine b2_engine;

enum { B2_KV_BF16 = 0, B2_KV_F32 = 1 };

/* -- loading ------------------------------------------------------------------------------- */

/* HybridEngine::load / load_on (aegist_rs/src/hybrid.rs:505-711): open an .nx brain, check the
 * config, upload every tensor, allocate context for `max_context` tokens (0 = 32768) for `batch`
 * sequences. All experts become resident (the reference's LRU pool, hybrid.rs:190-390, is replaced
 * by a full slot table). `kv_dtype`: B2_KV_BF16 is what the reference engine stores
 * (kernels/hybrid.cu:113-114); B2_KV_F32 matches the Python reference's fp32 cache. */
int b2_open(const char* nx_path, int max_context, int device, int batch, int kv_dtype, b2_engine** out);

/* The same engine built from tensors already in memory (host or device pointers), for callers that
 * produce a brain without writing a file: b2_create with the header's "config" JSON, one
 * b2_put_tensor per tensor named as in the .nx file (hybrid.rs:546-602), then b2_finish.
 * `ep_rank`/`ep_world` select which experts this engine keeps (expert e lives on rank
 * e / (n_experts / ep_world)); use 0, 1 for a single GPU. */
int b2_create(const char* config_json, int max_context, int device, int batch, int kv_dtype,
              int ep_rank, int ep_world, b2_engine** out);
int b2_put_tensor(b2_engine* e, const char* name, const char* dtype, const int64_t* shape, int ndim,
                  const void* data, size_t nbytes, int data_on_device);
int b2_finish(b2_engine* e);

/* Expert parallelism over `ep_world` GPUs of one node, one process per GPU, each with an engine made
 * by b2_create(..., ep_rank, ep_world) for its own `batch` sequences: the experts of every layer are
 * split over the GPUs and the picks travel by NCCL (an all-gather of the routed tokens and an
 * all-to-all of the expert outputs per layer). Rank 0 calls b2_ep_unique_id and hands the 128 bytes
 * to every rank by any means; then all ranks call b2_ep_init together, and from then on
 * b2_feed_batch / b2_decode_greedy together, step for step. The reference engine is single-GPU
 * (aegist_rs/src/hybrid.rs:511-514 only picks which one); this has no counterpart there. */
int b2_ep_unique_id(b2_engine* e, void* id_out, size_t len);
int b2_ep_init(b2_engine* e, const void* id_in, size_t len);

/* The same exchange by plain peer stores instead of NCCL calls (optional, after b2_ep_init): every rank gets the
 * 64-byte handle of its exchange block (cudaIpc), the handles of all ranks in rank order travel to every rank by any
 * means, and b2_ep_ipc_attach maps them. From then on a rank writes its records, and the outputs of the picks it
 * computed (only those: 1 / ep_world of the dense block on average), straight into the other ranks' blocks and raises
 * a flag there; the receiving rank waits for the flags a bounded number of polls (about a second; then the step
 * fails with a message, it does not hang). Results are the same sums in the same order as with NCCL and as on one
 * GPU. All ranks attach, or none. No counterpart in the reference. */
int b2_ep_ipc_handle(b2_engine* e, void* handle_out, size_t len);
int b2_ep_ipc_attach(b2_engine* e, const void* handles, size_t len_each, int n);

/* NxFile::verify (aegist_rs/src/nx.rs:164-184): recompute the per-group SHA-256 of a brain file.
 * ok[0..2] = base, engine, cores (1 = matches the header). */
int b2_verify_file(const char* nx_path, int ok[3], char* err, size_t err_len);

void b2_close(b2_engine* e);

/* -- the token loop ------------------------------------------------------------------------ */

/* Lm::feed (hybrid.rs:1016-1027): feed `n` tokens of sequence 0 (batch must be 1) and return the
 * logits after the last one in `logits_out` (f32[vocab], host; may be NULL). Fails with
 * "context full" when length + n > cap, and on a token id outside the vocabulary. */
int b2_feed(b2_engine* e, const uint32_t* ids, int n, float* logits_out);

/* Page-locked host memory for `logits_out` and `ids`: copies to and from it are plain DMA, where pageable memory
 * is staged by the driver (0.1 ms per feed for the 35B vocabulary's 608 KB of logits). Not part of the reference
 * interface, whose feed returns a fresh Vec<f32>; a binding keeps one such buffer per engine and copies out of it
 * only if its caller keeps the logits. NULL when the allocation fails. */
void* b2_host_alloc(size_t bytes);
void b2_host_free(void* p);

/* One token for each of the `batch` sequences. `next_greedy` (u32[batch], host, optional) receives
 * the arg-max of each row (first maximum wins, as chat.rs:239); `logits_out` (f32[batch][vocab],
 * host, optional). New entry point: the reference engine has no batch. */
int b2_feed_batch(b2_engine* e, const uint32_t* ids, uint32_t* next_greedy, float* logits_out);

/* The greedy loop of Chat::step / debug_logits (chat.rs:485-488, main.rs:780-791) kept on the
 * device: feed `first` (u32[batch]), then `steps - 1` times feed each sequence its own arg-max.
 * `tokens_out` (u32[steps][batch], host) receives the arg-max after every feed. `device_ms`
 * (optional) receives the time of the whole loop measured with CUDA events on the engine's stream. */
int b2_decode_greedy(b2_engine* e, const uint32_t* first, int steps, uint32_t* tokens_out, float* device_ms);

/* Lm::crop / snapshot / length / cap (hybrid.rs:1029-1076). b2_crop returns the length kept
 * (>= 0) or a negative error. */
int b2_crop(b2_engine* e, int n);
int b2_snapshot(b2_engine* e);

/* Lm::state_key / save_state / load_state (aegist_rs/src/model.rs:375-387). The reference's hybrid engine
 * keeps the trait's defaults (it cannot save); its other engines write the file format used here
 * (aegist_rs/src/next.rs:2442-2548): "AEGSTATE", u64 LE header length, JSON {"key", "toks"}, then per layer the
 * keys and values of the first n positions (per KV head) or the conv taps [C][3] and the recurrent state
 * [HV][DK][DV]. The key is `<fingerprint of the brain file>-<layers>x<kv heads>x<head dim>` (+ "-kvf32" for an
 * fp32 cache), so a state only loads into the brain that wrote it. One sequence only. b2_load_state returns the
 * saved tokens (`toks_out` holds up to `cap_toks`, `*n_out` their number), takes a snapshot at that length, and
 * leaves the engine empty on any error. b2_save_state needs every token of the context to have passed through
 * the host (b2_feed, b2_feed_batch, b2_decode_greedy). */
const char* b2_state_key(const b2_engine* e);
int b2_save_state(b2_engine* e, const char* path);
int b2_load_state(b2_engine* e, const char* path, uint32_t* toks_out, int cap_toks, int* n_out);
int b2_length(const b2_engine* e);
int b2_cap(const b2_engine* e);

/* Lm::set_taps / taps (hybrid.rs:1078-1093): keep the residual stream after the given layers for
 * the last token of every feed. b2_taps writes f32[n_taps][batch][d_model]. */
int b2_set_taps(b2_engine* e, const int* layers, int n);
int b2_taps(b2_engine* e, float* out);

/* Lm::core_counts / reset_counts (hybrid.rs:1095-1101): per-layer switch-on counts of the core
 * engine, i32[layers][n_cores]. The engine runs the reference's core engine in every layer of every token
 * (cores_apply, kernels/aegist.cu:283-350): product-key routing over the two key tables, one count per pick, and the
 * output of the picks whose core is live (stored in the brain file or a cores file laid over it). */
int b2_core_counts(b2_engine* e, int32_t* out);
int b2_reset_counts(b2_engine* e);

/* Lm::expert_counters (hybrid.rs:1103-1105): (expert uses served from device memory, experts
 * copied in). With every expert resident the second number stays 0. */
void b2_expert_counters(const b2_engine* e, uint64_t* hits, uint64_t* page_ins);

/* Lm::describe (hybrid.rs:1107-1118) and the message of the last failed call. */
const char* b2_describe(const b2_engine* e);
const char* b2_last_error(const b2_engine* e);
int b2_vocab(const b2_engine* e);
int b2_d_model(const b2_engine* e);

/* chat.rs:238-272 `sample`: top-k, then nucleus, then inverse CDF with the splitmix64 generator of
 * chat.rs:221-235; temperature <= 0 is greedy. `rng_state` is advanced in place. */
uint32_t b2_sample(const float* logits, int vocab, float temperature, float top_p, int top_k, uint64_t* rng_state);

/* -- parity and measurement hooks ---------------------------------------------------------- */

/* Router picks and weights of the latest step for one layer: i32[batch][k], f32[batch][k]
 * (the reference exposes them through $AEGIST_ROUTE_TRACE, hybrid.rs:163-181). */
int b2_debug_router(b2_engine* e, int layer, int32_t* idx, float* wts);
/* The residual stream after the last layer, before the final norm: f32[batch][d_model]
 * ($AEGIST_DUMP_FINAL, hybrid.rs:771-781). */
int b2_debug_hidden(b2_engine* e, float* out);
/* Add `bias` (f32[n_experts], host; NULL removes it) to one layer's router logits before the
 * softmax: shapes expert popularity for load-balance measurements. No reference counterpart. */
int b2_set_router_bias(b2_engine* e, int layer, const float* bias);
/* Set the context length without feeding tokens: positions 0..n-1 of the KV cache keep whatever they
 * hold (zeros after loading) and the recurrent state is untouched. For timing a step at a given
 * context length; the logits that follow are not those of any real prompt. No reference counterpart. */
int b2_debug_seek(b2_engine* e, int n);
/* Number of kernel launches in one decode step (all sequences). */
int b2_launches_per_step(const b2_engine* e);
/* How many launches of the tcgen05 GEMM (k_umma) this process has enqueued so far, graph captures included: lets a
 * test see that the Blackwell tensor-core path, not a fall-back, is what ran. No counterpart in the reference. */
long b2_debug_umma_launches(void);
/* Algorithmic bytes one decode step moves (weights once, recurrent state read + written, KV read
 * up to the current length), for roofline arithmetic. */
double b2_step_bytes(const b2_engine* e);

/* Run `iters` decode steps (each sequence is fed its own arg-max) outside the CUDA graph with an
 * event after every launch, and report per kernel class the mean device time per step (ms), the
 * algorithmic bytes per step and the launches per step. Classes: 0 embedding gather, 1 norm + GEMV
 * groups, 2 DeltaNet step, 3 attention, 4 output projections, 5 expert gate/up, 6 expert down +
 * shared down, 7 head. */
int b2_profile_step(b2_engine* e, int iters, float ms[8], double bytes[8], int launches[8]);
/* Bytes this GPU sends to its peers in one decode step of an expert-parallel engine (0 on one GPU): the per-layer
 * records (all-gather) and the pick outputs computed here for other GPUs' sequences. No counterpart in the reference. */
double b2_ep_bytes_per_step(const b2_engine* e);

/* Timeline of one decode step as the CUDA graph runs it (debugging aid, no reference counterpart; the step
 * feeds the current tokens and advances the length by one). Per launch 16 words: [0] first block entered and
 * [4] last block left, in ns of the GPU's global timer; [5] kernel code (1 GEMV, 3 DeltaNet step, 5 expert
 * gate/up, 6 expert down, 7 attention, 8 attention merge; 0 = a kernel that records nothing); [6] a shape hint
 * (rows of the first matrix, or the grid); [8] the SM cycle counter of block 0 when it entered and [9]..[15]
 * the same counter at its points 1..7 (1 past the wait for the previous kernel, 2 past the prologue, 3 past the
 * main loop, others kernel-specific). `out` holds 16 * cap_launches words. */
int b2_debug_trace_step(b2_engine* e, unsigned long long* out, int cap_launches, int* n_launches);

/* -- single operators, host buffers in and out (the reference's per-op semantics) ----------- */

/* QLinear.forward (aegist/model.py:92-93; gemv_i8, kernels/aegist.cu:84-91): y[t][n] = scale[n] * sum_k x[t][k] q[n][k]. */
int b2_op_linear_i8(int device, const int8_t* q, const uint16_t* scale_bf16, int n, int k,
                    const float* x, int tokens, float* y);
/* MoE.forward (aegist/hybrid.py:641-652; router_topk + moe_*_gemv + shared expert, hybrid.rs:863-975)
 * on `tokens` rows of h: y = experts(h) + sigmoid(shared_gate h) * shared(h). Weight pointers are
 * host memory in the .nx layouts. idx/wts (optional) receive the router's picks. It runs the kernels the
 * engine runs for that many tokens (below 8 the top-8 happens inside the expert kernel). Returns 4 when
 * the kernels set their error word (a bad pick, a copy that never landed). */
typedef struct {
    int d_model, n_experts, top_k, expert_hidden, shared_hidden, group;
    const uint16_t* router_bf16;      /* [E][D] */
    const uint8_t* experts_q4;        /* [E][expert_bytes] */
    const int8_t* sh_gate_q; const uint16_t* sh_gate_s;   /* [SH][D], [SH] */
    const int8_t* sh_up_q;   const uint16_t* sh_up_s;
    const int8_t* sh_down_q; const uint16_t* sh_down_s;   /* [D][SH], [D] */
    const uint16_t* shared_gate_bf16; /* [D] */
} b2_moe_weights;
typedef struct b2_moe b2_moe;
int b2_moe_create(int device, const b2_moe_weights* w, int max_tokens, b2_moe** out);
int b2_moe_forward(b2_moe* m, const float* h, int tokens, float* y, int32_t* idx, float* wts, float* device_ms);
void b2_moe_destroy(b2_moe* m);

/* The same MoE layer operator for callers that must not allocate device memory (a process whose own
 * arena already owns the GPU's free memory, a loop that cannot afford an allocation's device-wide
 * synchronisation, a plug-in that is only ever handed pointers). It has no counterpart in the
 * reference. It calls no cudaMalloc / cudaFree and no allocating library routine: every pointer below
 * is DEVICE memory supplied by the caller (`expert_ptrs` is a device array of n_experts device
 * addresses, one packed expert row each), and the kernels' work memory is a fixed array inside the
 * library, 748 KB on every GPU that loads it. Limits: at most 8 tokens, d_model 2048, 256 experts,
 * top-8, expert_hidden 512, shared_hidden 512; anything larger returns 2 with a message on stderr
 * (3: bad argument, 1: CUDA error). All calls share that array, which keeps the last call's contents
 * (the function clears what must start at zero, y included): calls that overlap on one GPU race, so
 * run them one after the other. The first call on a device looks the array's address up; make it
 * before any stream capture begins. Work is queued on `stream` (a cudaStream_t, NULL = default); every
 * call then synchronises that stream and reads the kernels' error word back, so it must never be made on
 * a stream that is being captured. h, y and the nine pointers inside *w must be non-null and 16-byte
 * aligned (the kernels use 128-bit loads), idx / wts 4-byte aligned: otherwise 3 is returned and nothing
 * runs. 4 = the kernels reported an error (a pick whose table entry is null, a copy that never landed).
 * idx / wts are optional outputs. */
typedef struct {
    int d_model, n_experts, top_k, expert_hidden, shared_hidden;
    const uint16_t* router_bf16;            /* [E][D] */
    const uint8_t* const* expert_ptrs;      /* [E] device addresses of the packed experts */
    const int8_t* sh_gate_q; const uint16_t* sh_gate_s;
    const int8_t* sh_up_q;   const uint16_t* sh_up_s;
    const int8_t* sh_down_q; const uint16_t* sh_down_s;
    const uint16_t* shared_gate_bf16;       /* [D] */
} b2_moe_device_weights;
int b2_moe_forward_static(const b2_moe_device_weights* w, const float* h, int tokens, float* y, int32_t* idx,
                          float* wts, void* stream);

/* Runs a kernel whose only wait can never succeed (an mbarrier that expects bytes no copy delivers) with a
 * limit of `polls` polls, and returns the device error word in *status: 3 = the bounded wait gave up and the
 * kernel ended normally. This is how the time-out path of every bulk-copy wait is tested without a hang.
 * No counterpart in the reference. */
int b2_debug_wait_timeout(int device, int polls, int* status);

/* delta_rule_step (aegist/hybrid.py:318-324; delta_scan, kernels/hybrid.cu:240-300) with the state
 * kept on the device between calls. q, k [B][H][dk] (already normalised and scaled), v [B][H][dv],
 * g, beta [B][H]; out [B][H][dv]. */
typedef struct b2_delta b2_delta;
int b2_delta_create(int device, int batch, int heads, int dk, int dv, const float* state0, b2_delta** out);
int b2_delta_step(b2_delta* d, const float* q, const float* k, const float* v, const float* g, const float* beta,
                  float* out, float* device_ms);
int b2_delta_state(b2_delta* d, float* state_out);
void b2_delta_destroy(b2_delta* d);

#ifdef __cplusplus
}
#endif
#endif
