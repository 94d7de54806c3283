/* b200w4 -- C ABI of the B200 (sm_100a) W4G128 / W4A8 matmul path.
 *
 * Plain pointers and sizes only.  Every function returns 0 on success or a
 * negative B2W4_E_* code; b2w4_last_error() gives the text of the last failure
 * on that context.  Nothing here throws, and nothing falls back to the CPU: if
 * no sm_100 device is usable, b2w4_ctx_create fails.
 *
 * Each entry point names the reference interface (mollm, path:line) it stands
 * in for.  Weights arrive as the reference's canonical BG128 blocks
 * (kernels/quant_layouts.h:9-14): block (n8,g) at index n8*(K/128)+g, 8 fp32
 * row scales then q[4][8][16] nibble bytes; 544 bytes per 8 rows x 128 k.
 *
 * Tensors follow the reference's matmul convention (engine/cuda_backend.cu:
 * 1032-1045): activations x are fp32 [M rows][K], row stride lda elements;
 * outputs y are fp32 [M rows][N], row stride ldc elements.
 */
#ifndef B200W4_H
#define B200W4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    B2W4_OK = 0,
    B2W4_E_INVALID = -1,   /* bad argument / unsupported shape              */
    B2W4_E_CUDA = -2,      /* a CUDA call failed                            */
    B2W4_E_NO_DEVICE = -3, /* no usable sm_100 device                       */
    B2W4_E_NOMEM = -4,
    B2W4_E_TIMEOUT = -5    /* a bounded device-side wait gave up            */
};

/* Activation-quantisation rule (reference kernels/matmul_w4.cpp:1058-1075 for
 * M==1, :1125-1154 for M>1). */
enum {
    B2W4_ACT_G128 = 128, /* one int8 scale per 128 values, applied row by row */
    B2W4_ACT_G32 = 32    /* one int8 scale per 32 values                      */
};

/* Post-matmul activation, same numbering as the reference's Activation enum
 * (kernels/activations.h:28-35). */
enum { B2W4_NONE = 0, B2W4_SILU = 1, B2W4_GELU = 2, B2W4_RELU = 3, B2W4_RELU_SQUARED = 4 };

typedef struct b2w4_ctx b2w4_ctx;
typedef struct b2w4_weight b2w4_weight;

/* ---- context -------------------------------------------------------------
 * Replaces CudaBackend::Impl construction (engine/cuda_backend.cu:394-409):
 * binds a device, owns scratch for quantised activations.  `stream` is a
 * cudaStream_t (NULL = the legacy default stream the reference uses). */
int b2w4_ctx_create(int device, b2w4_ctx** out);
void b2w4_ctx_destroy(b2w4_ctx* ctx);
int b2w4_ctx_set_stream(b2w4_ctx* ctx, void* stream);
int b2w4_sync(b2w4_ctx* ctx); /* end_graph(), engine/cuda_backend.cu:631-639 */
/* Bound of the device-side waits for ANOTHER GPU's stores (the exchanges inside
 * the kernels, below), 1..10000 ms, default about 2 s.  It must cover the skew
 * between the ranks' host threads -- a peer still loading a kernel's code while
 * this rank's consumer already spins -- not only the flight of the stores.  No
 * counterpart in the reference (one process, one device). */
int b2w4_ctx_set_peer_wait_ms(b2w4_ctx* ctx, int milliseconds);
const char* b2w4_last_error(const b2w4_ctx* ctx);
const char* b2w4_version(void);

/* ---- weights -------------------------------------------------------------
 * Replaces CudaBackend::wrap_weight_int4 (engine/cuda_backend.cu:462-487) and
 * its upload helper (:147-175): validates K%128==0, copies the blocks (the
 * caller may free or overwrite them afterwards) and repacks them on the device
 * into the streaming layout the kernels read (nibble plane + scale plane).
 * `host_blocks` holds ((N+7)/8)*(K/128)*544 bytes. */
int b2w4_weight_upload(b2w4_ctx* ctx, const void* host_blocks, int n, int k,
                       b2w4_weight** out);
/* Same, from blocks already in device memory (weights generated on the GPU). */
int b2w4_weight_from_device(b2w4_ctx* ctx, const void* device_blocks, int n, int k,
                            b2w4_weight** out);
void b2w4_weight_free(b2w4_ctx* ctx, b2w4_weight* w);
int b2w4_weight_shape(const b2w4_weight* w, int* n, int* k);
/* 1 if every group scale is exactly representable in fp16 (the device scale
 * plane is then fp16), 0 if the plane had to stay fp32. */
int b2w4_weight_scales_fp16(const b2w4_weight* w);
/* Bytes of device memory one full pass over the weight reads. */
size_t b2w4_weight_stream_bytes(const b2w4_weight* w);

/* ---- matmul --------------------------------------------------------------
 * Replaces CudaBackend::Impl::run_matmul_device (engine/cuda_backend.cu:
 * 212-337): y[M,N] = act(x[M,K] * W^T), device pointers, asynchronous on the
 * context's stream.  Arithmetic is the reference's W4A8 kernels': int8
 * activations per `act_rule` group, int32 dot per group, then
 * y = fma(float(dot), fp32(wscale*ascale), y) in ascending group order
 * (kernels/matmul_w4.cpp:211-295, :785-901).  `activation` is applied to
 * columns [act_n_begin, act_n_begin+act_n_len); act_n_len < 0 = all columns
 * (kernels/matmul_internal.h:73-119). */
int b2w4_matmul(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda,
                float* y_dev, int ldc, int m, int act_rule, int activation,
                int act_n_begin, int act_n_len);

/* Replaces CudaBackend::Impl::run_matmul (host tensors staged through the
 * device, engine/cuda_backend.cu:339-359) and CudaBackend::lm_head_gemv
 * (:1393-1400): host x, host y, synchronous. */
int b2w4_matmul_host(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_host,
                     int lda, float* y_host, int ldc, int m, int act_rule,
                     int activation, int act_n_begin, int act_n_len);

/* No counterpart in the reference.  Some callers of this library cannot allocate
 * device memory at the time they run a matmul: code inside a real-time or
 * latency-critical serving loop that forbids cudaMalloc (it synchronises the
 * device), code running while a stream capture is open, or a host runtime whose
 * memory budget was fixed at start-up.  b2w4_matmul quantises the activations
 * into a pool that grows with cudaMalloc on demand; this variant runs the same
 * tensor-core kernel with that buffer in a fixed 2.6 MiB array inside the
 * library image, and calls no cudaMalloc, cudaFree or other allocating routine.
 * Limits: 5 <= m <= 256 rows, K <= 10240; anything else is B2W4_E_INVALID.
 * Same arithmetic and bits as b2w4_matmul (per-128 rule only).
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current: make that first call before
 * any stream capture.  All calls share the array, which keeps the previous
 * call's contents (nothing in it needs to start at zero); calls that overlap on
 * the GPU race on it.  Every GPU that uses the library holds the array until
 * the process exits. */
int b2w4_matmul_static_scratch(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev,
                               int lda, float* y_dev, int ldc, int m, int activation,
                               int act_n_begin, int act_n_len);

/* Parity hook with no reference counterpart in the CUDA backend: writes the
 * int32 group accumulators of the same kernels, [M][N][K/128] for
 * B2W4_ACT_G128 or [M][N][K/32] for B2W4_ACT_G32, to device memory. */
int b2w4_debug_group_sums(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev,
                          int lda, int m, int act_rule, int32_t* sums_dev);

/* Parity hook: the device activation quantiser alone (reference
 * kernels/matmul_quant.cpp:578-641 and :280-329).  q_dev receives int8 [M][K]
 * in natural k order, scales_dev fp32 [M][K/act_rule]. */
int b2w4_quantize_activations(b2w4_ctx* ctx, const float* x_dev, int lda, int m,
                              int k, int act_rule, int8_t* q_dev, float* scales_dev);

/* Activation rule of the routed-MoE expert matmuls.  B2W4_ACT_G32 (default) is the
 * reference's: an expert that was handed several rows runs the multi-row W4A8
 * kernel, one activation scale per 32 values (kernels/moe.cpp:1055-1058 ->
 * kernels/matmul_w4.cpp:1125-1154), an expert with a single row the one-row
 * kernel, one scale per 128 values (:1058-1075).  B2W4_ACT_G128 applies the
 * one-row rule to every row (a deviation from the reference, somewhat faster). */
int b2w4_ctx_set_moe_rule(b2w4_ctx* ctx, int act_rule);

/* ---- routed MoE ----------------------------------------------------------
 * Replaces kernel_qwen3_moe (kernels/moe.cpp:576-1129) as dispatched for
 * OpType::MOE (graph/cpu_backend.cpp:169-206) in the Qwen3-MoE configuration:
 * softmax top-k routing over raw logits with ties to the lower expert id
 * (kernels/moe_routing.cpp:129-166), fp16 router weight [E,H], expert
 * aggregates gate_up [E*2I, H] and down [E*H, I] as BG128 weights, no shared
 * expert.  hidden fp32 [tokens][H] (row stride ldx), out fp32 [tokens][H]
 * (row stride ldo); all device pointers.  Optional outputs (NULL to skip):
 * logits [tokens][E], indices int32 / weights fp32 [tokens][top_k]. */
int b2w4_moe_forward(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens,
                     int hidden_size, const void* router_fp16_dev, int num_experts,
                     int top_k, int intermediate, const b2w4_weight* gate_up,
                     const b2w4_weight* down, float* out_dev, int ldo,
                     float* logits_dev, int32_t* indices_dev, float* weights_dev);

/* Routing alone: select_moe_routes, score_func 0 (kernels/moe_routing.cpp:
 * 25-169).  logits fp32 [tokens][E] on the device. */
int b2w4_moe_select_routes(b2w4_ctx* ctx, const float* logits_dev, int tokens,
                           int num_experts, int top_k, int32_t* indices_dev,
                           float* weights_dev);

/* ---- expert-parallel MoE ---------------------------------------------------
 * No counterpart in the reference, which runs one process on one device; the op
 * is kernel_qwen3_moe (kernels/moe.cpp:576-1129) split at the point where the
 * experts' outputs meet.  Rank r of P holds the aggregates of experts
 * [expert_begin, expert_begin+expert_count) only (gate_up_local
 * [expert_count*2I, H], down_local [expert_count*H, I]); hidden and the router
 * weight are replicated, so every rank derives the same routes without an
 * exchange.  b2w4_moe_expert_outputs writes route_out fp32 [tokens*top_k][H]:
 * row t*top_k+j is the down-projection output of token t's j-th route when its
 * expert is held here, zeros otherwise, and indices / weights [tokens][top_k]
 * as b2w4_moe_forward does.  The caller sums route_out over the ranks (an
 * all-reduce: each row has one owner, the sum adds only zeros and changes no
 * bit) and calls b2w4_moe_combine, which applies out[t] = fma(w, y, out[t])
 * over the token's routes in ascending expert id (kernels/moe.cpp:1100-1110):
 * the result equals b2w4_moe_forward's bit for bit. */
int b2w4_moe_expert_outputs(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens,
                            int hidden_size, const void* router_fp16_dev, int num_experts,
                            int top_k, int intermediate, const b2w4_weight* gate_up_local,
                            const b2w4_weight* down_local, int expert_begin,
                            int expert_count, float* route_out_dev, int32_t* indices_dev,
                            float* weights_dev);
int b2w4_moe_combine(b2w4_ctx* ctx, const float* route_out_dev, int tokens, int hidden_size,
                     int top_k, const int32_t* indices_dev, const float* weights_dev,
                     float* out_dev, int ldo);

/* ---- lm_head with the greedy token picked on the device -----------------------
 * Replaces the pair "lm_head matmul, copy N logits to the host, argmax_token"
 * (engine/sampler.cpp:31-77) of a greedy decode step, as the reference's Metal
 * backend does with lm_head_argmax_device_and_end_graph and its small-batch form
 * (engine/metal_backend.h:159-176; engine/engine.cpp:792-803, :1189): the
 * matmul's epilogue reduces the logits of each of the m <= 8 activation rows to
 * token_dev[row] = the first index of the maximum (a NaN never wins, except at
 * index 0 where nothing beats it -- the scalar loop's behaviour).  y_dev may be
 * NULL (logits not written at all) or fp32 [m][ldc].  Per-128 activation rule. */
int b2w4_matmul_argmax(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda, int m,
                       float* y_dev, int ldc, int32_t* token_dev);

/* ---- exchanges inside the kernels: tensor-parallel matmul, expert-parallel MoE --
 * No counterpart in the reference (one process, one device).  Instead of a
 * kernel followed by a collective call, the producing kernel stores each value,
 * paired with the number of the exchange in one 8-byte word, straight into every
 * rank's staging buffer through peer mappings, and the consuming kernel takes an
 * entry once it carries the current exchange number (bounded wait, see
 * b2w4_ctx_set_peer_wait_ms; then B2W4_E_TIMEOUT through b2w4_sync, and every
 * output value whose entry never arrived is a quiet NaN -- a token: -1 -- never
 * a stale value of an earlier exchange; the exchange count still advances, so
 * the group stays in step, and callers must check b2w4_sync before they use the
 * outputs of a step).  A word is written whole, so no fence or flag write
 * follows the data and the exchange costs one trip over the link.
 * stage_peers[p] = rank p's staging buffer as mapped into this process (e.g. the
 * buffer_ptrs of a symmetric-memory rendezvous), 16-byte aligned, all zero before
 * first use: uint64[2 + 2 * half] with word 0 the count of completed exchanges
 * and two halves that alternate, so that a rank may run one exchange ahead of
 * its peers.  Every rank issues the same sequence of calls on a group, and a
 * staging buffer serves one kind of call with one half size. */
typedef struct b2w4_tp_group {
    int rank, world;       /* world <= 8 */
    void* stage_peers[8];
} b2w4_tp_group;

/* Tensor-parallel decode matmul with the all-gather inside: rank r holds the rows
 * [n_offset, n_offset + N_shard) of a weight (8-row tiles whole), the shards cover
 * [0, ldc), and every rank needs the full rows.  b2w4_matmul_tp is b2w4_matmul
 * (per-128 activation rule) for m <= 8 activation rows x_dev [m][lda] whose
 * epilogue stores into every rank's staging buffer (half = 8 * ldc whatever m
 * is); b2w4_tp_gather, with the same m, waits for every entry of the current
 * half, unpacks the rows into y_dev [m][ldc] and advances the count.  Same
 * arithmetic and bits as b2w4_matmul on the unsharded weight. */
int b2w4_matmul_tp(b2w4_ctx* ctx, const b2w4_weight* w_shard, const float* x_dev, int lda,
                   int m, int ldc, int n_offset, const b2w4_tp_group* group, int activation,
                   int act_n_begin, int act_n_len);
int b2w4_tp_gather(b2w4_ctx* ctx, const b2w4_tp_group* group, float* y_dev, int m, int ldc);

/* Tensor-parallel lm_head with the greedy token picked on the devices: every rank
 * reduces its rows to one (maximum, index in the unsharded weight) pair per
 * activation row and hands it to every rank as two tagged words (staging buffer
 * uint64[2 + 2 * 128]); b2w4_tp_gather_token takes the largest of the world's
 * pairs -- the token b2w4_matmul_argmax gives on the unsharded weight -- into
 * token_dev [m] and advances the count.  No logits leave a GPU. */
int b2w4_matmul_argmax_tp(b2w4_ctx* ctx, const b2w4_weight* w_shard, const float* x_dev, int lda,
                          int m, int n_offset, const b2w4_tp_group* group);
int b2w4_tp_gather_token(b2w4_ctx* ctx, const b2w4_tp_group* group, int32_t* token_dev, int m);

/* Expert-parallel MoE with the hand-over inside: b2w4_moe_expert_outputs, the sum
 * over the ranks and b2w4_moe_combine as one call.  The owner of a route stores
 * its down-projection row into every rank's staging buffer (half = stage_rows *
 * H words, stage_rows >= tokens * top_k and the same on every call of the group)
 * and the combine takes the rows from there.  out equals b2w4_moe_forward's bit
 * for bit.  Meant for decode steps: it moves 8 bytes per value to every peer. */
int b2w4_moe_forward_ep(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens,
                        int hidden_size, const void* router_fp16_dev, int num_experts,
                        int top_k, int intermediate, const b2w4_weight* gate_up_local,
                        const b2w4_weight* down_local, int expert_begin, int expert_count,
                        const b2w4_tp_group* group, int stage_rows, float* out_dev, int ldo,
                        int32_t* indices_dev, float* weights_dev);

/* ---- a list of decode GEMVs as one persistent kernel ------------------------------
 * Stands in for the walk over a decode graph's MATMUL nodes with one activation
 * row (graph/execute.cpp:651-669, one dispatch per weight) and for the batch entry
 * point that runs several one-row GEMVs in one dispatch
 * (kernel_matmul_int4_gemv_batch, kernels/matmul_w4.cpp:381-493).  Every op is
 * b2w4_matmul with m == 1 and the per-128 activation rule -- same arithmetic, same
 * bits -- but the whole list is ONE cooperative kernel, one CTA per SM: the weights
 * of later ops stream into shared memory while earlier ops compute, and an op that
 * consumes an earlier op's output picks it up on the device as soon as it is
 * written (tagged 8-byte words, no kernel boundary, no barrier).
 * Op i computes y_i[N_i] = act(W_i * x_i), where x_i[K_i] is
 *   x_from >= 0 : elements [x_offset, x_offset + K_i) of op x_from's output (an
 *                 earlier op of the list), or
 *   x_from == -1: x_dev (fp32 on the device, ready before the run starts), or, when
 *                 x_dev is NULL, the chain's own input vector (b2w4_chain_input /
 *                 the x_host of b2w4_chain_run_host).
 * y_dev (optional) receives the plain fp32 row; the last op's row is also kept in
 * the chain's own output buffer when it names no y_dev (b2w4_chain_output).
 * Limits: 1..4096 ops; K such that one 8-row tile of a weight (K/128 * 528 bytes)
 * plus the quantised activations fit an SM's shared memory (K <= 32768 or so).
 * All device-side waits are bounded (about 2 s); on expiry b2w4_sync returns
 * B2W4_E_TIMEOUT and the outputs of that run are undefined. */
typedef struct b2w4_chain_op {
    const b2w4_weight* w;
    int x_from;          /* -1, or the index of an earlier op */
    int x_offset;        /* first element of that op's output used as input */
    const float* x_dev;  /* x_from == -1 only; NULL = the chain's input vector */
    float* y_dev;        /* NULL = not written out */
    int activation, act_n_begin, act_n_len; /* as b2w4_matmul */
} b2w4_chain_op;
typedef struct b2w4_chain b2w4_chain;
int b2w4_chain_create(b2w4_ctx* ctx, const b2w4_chain_op* ops, int count, b2w4_chain** out);
void b2w4_chain_destroy(b2w4_ctx* ctx, b2w4_chain* chain);
/* Tensor-parallel form (no counterpart in the reference: one process, one device).
 * Every rank builds the same list on its row shard of every weight: op i's weight
 * here holds the rows [n_offset, n_offset + N_shard) of a full row of n_full
 * values (8-row tiles whole).  The all-gather is inside the kernel: a value is
 * stored, tagged, into EVERY rank's scratch over the peer mappings, and an op that
 * consumes an earlier op's output polls its own rank's scratch -- it sees the full
 * row, exactly as on one GPU, with no collective call and no extra launch; x_offset
 * and K refer to the full row.  y_peers[p] (optional, all or none) is rank p's
 * plain fp32 row [n_full] as mapped here: the kernel stores this rank's columns
 * into every one of them.  y_dev must be NULL.  group->stage_peers[p] is rank p's
 * scratch: uint64[b2w4_chain_scratch_words(...)], zeroed before the chain is
 * created, 16-byte aligned, used by this chain only.  Every rank issues the same
 * sequence of runs.  A rank that runs ahead is held by the bounded waits for its
 * peers' values; plain y_peers rows of a run are complete on every rank once
 * every rank has synchronised after that run. */
typedef struct b2w4_chain_shard {
    int n_offset, n_full;
    void* y_peers[8];
} b2w4_chain_shard;
int b2w4_chain_create_tp(b2w4_ctx* ctx, const b2w4_chain_op* ops,
                         const b2w4_chain_shard* shards, int count,
                         const b2w4_tp_group* group, b2w4_chain** out);
size_t b2w4_chain_scratch_words(const b2w4_chain_shard* shards, int count);
/* Asynchronous on the context's stream. */
int b2w4_chain_run(b2w4_ctx* ctx, b2w4_chain* chain);
/* One decode step from host memory: x_host[x_len] goes to the chain's input
 * vector, the list runs, the chain's own output (the last op's row) comes back in
 * y_host[y_len]; one upload, one kernel, one download, one synchronisation.
 * Replaces a sequence of CudaBackend::lm_head_gemv-style host calls
 * (engine/cuda_backend.cu:1393-1400). */
int b2w4_chain_run_host(b2w4_ctx* ctx, b2w4_chain* chain, const float* x_host, int x_len,
                        float* y_host, int y_len);
/* Profiling hook, no reference counterpart: while trace_dev is non-NULL, CTA `cta`
 * of every run writes 8 int64 time stamps (cycles of that CTA's SM) per op to
 * trace_dev[op*8 ..]:
 * 0 op begins, 1 its activations have arrived, 2 quantised, 5 about to wait for
 * its first tile, 3 that tile's weights are in shared memory, 4 its last tile done
 * (all compute warp 0); 6 the copy of the op's last tile was issued, 7 cycles
 * the producer thread waited for ring space during the op's copies. */
int b2w4_chain_set_trace(b2w4_chain* chain, long long* trace_dev, int cta);
float* b2w4_chain_input(b2w4_chain* chain);   /* device pointer, may be NULL */
float* b2w4_chain_output(b2w4_chain* chain);  /* device pointer, may be NULL */
size_t b2w4_chain_weight_bytes(const b2w4_chain* chain);

/* ---- the operators between a decoder layer's matmuls ---------------------------------
 * Device kernels for the operators a dense decoder layer runs between its W4G128
 * matmuls, so that a decode step needs no host round trip.  All tensors fp32 on the
 * device, rows = tokens, features contiguous; asynchronous on the context's stream.
 * Sums over a row are tree reductions (the reference's scalar loops are
 * sequential): agreement with the reference is to fp32 rounding of a reassociated
 * sum; the element-wise arithmetic keeps the reference's operation order.
 *   b2w4_rms_norm      OpType::RMS_NORM, kernel_rms_norm (kernels/norm.cpp:13-31,
 *                      :95-121): out = (x * 1/sqrt(mean(x^2) + eps)) * weight
 *   b2w4_add_rms_norm  OpType::ADD_RMS_NORM, kernel_add_rms_norm (:123-190):
 *                      residual += update (written back), out = rms_norm(residual)
 *   b2w4_swiglu        OpType::SWIGLU (kernels/elementwise.cpp:529-570): merged row
 *                      [2I] = gate | up; out[i] = (gate[i] / (1+exp(-gate[i]))) * up[i]
 *   b2w4_elementwise   OpType::ADD / MUL on equal-shaped contiguous tensors
 *   b2w4_rope          OpType::ROTARY_EMBED, kernel_rope with interleave == 0
 *                      (kernels/rope.cpp:11-50, :155-195): x [tokens][heads][dim];
 *                      cos / sin are tables [positions][rope_dim/2] (filled on the
 *                      host as engine/input_prep.cpp:18-31 does) and token t takes row
 *                      first_position + t, or *position_dev + t when position_dev is
 *                      given; in place when out == x
 *   b2w4_attention     OpType::SDPA with a KV cache (kernels/attention.cpp:1043-1057
 *                      for the cache layout [kv_head][capacity][dim], fp32;
 *                      kernels/attention_x86_avx512.cpp:47-109 for the arithmetic):
 *                      appends the new tokens' k, v [tokens][kv_heads][dim] at
 *                      positions past.., then causal attention of q
 *                      [tokens][heads][dim] over keys 0 .. past + t, full-row softmax,
 *                      P*V accumulated in ascending key order (dim <= 256; the scores
 *                      of all visible keys are held in shared memory, which bounds
 *                      them near 45,000; runs of eight or more tokens take a tiled
 *                      form -- one block per kv head and tile of query tokens, keys
 *                      and values staged once per tile, the same bits -- while a
 *                      tile's scores fit, about 1,400 keys); past_dev (optional)
 *                      gives `past` from device memory instead
 *                      k_dev and v_dev both NULL: nothing is appended, the cache rows
 *                      past .. past + tokens - 1 are in place already (b2w4_qkv_prepare)
 *   b2w4_qkv_prepare   what sits between the fused qkv matmul and attention, in one
 *                      launch: rows of the merged output [tokens][(heads + 2 kv_heads)
 *                      * dim] -- Q and K rows get the per-head RMSNorm (weights may be
 *                      NULL: none) and the rotary embedding over the whole head
 *                      (engine/cuda_attention.cu:8-55 fuses the two likewise), Q lands
 *                      in q_out [tokens][heads][dim], K and V in their cache rows
 *                      past + t.  Bit-identical to b2w4_rms_norm + b2w4_rope +
 *                      the append of b2w4_attention.  dim a multiple of 64, <= 256
 *   b2w4_advance       *counter_dev += by, after history_dev[*counter_dev] = *token_dev
 *                      (both optional).  With the position on the device a decode
 *                      step is the same sequence of launches for every token and can
 *                      be captured once in a CUDA graph and replayed (the reference
 *                      keeps its decode graph static for the same reason,
 *                      engine/model_loader.cpp:1111) -- no counterpart as an operator
 *   b2w4_copy_rows     OpType::CONTIGUOUS for a block of rows: a strided window (e.g.
 *                      the q, k or v columns of a fused qkv output) made contiguous
 *   b2w4_embed_rows    rows ids[r] of an fp16 table [vocab][dim] widened to fp32 */
int b2w4_rms_norm(b2w4_ctx* ctx, const float* x_dev, int ldx, int rows, int dim,
                  const float* weight_dev, float eps, float* out_dev, int ldo);
int b2w4_add_rms_norm(b2w4_ctx* ctx, float* residual_dev, int ldr, const float* update_dev,
                      int ldu, int rows, int dim, const float* weight_dev, float eps,
                      float* out_dev, int ldo);
int b2w4_swiglu(b2w4_ctx* ctx, const float* merged_dev, int ldm, int rows, int intermediate,
                float* out_dev, int ldo);
int b2w4_elementwise(b2w4_ctx* ctx, const float* a_dev, const float* b_dev, float* out_dev,
                     size_t count, int multiply);
int b2w4_rope(b2w4_ctx* ctx, const float* x_dev, float* out_dev, int tokens, int heads, int dim,
              const float* cos_dev, const float* sin_dev, int rope_dim, int first_position,
              const int* position_dev);
int b2w4_attention(b2w4_ctx* ctx, const float* q_dev, const float* k_dev, const float* v_dev,
                   float* k_cache_dev, float* v_cache_dev, float* out_dev, int tokens, int heads,
                   int kv_heads, int dim, int past, const int* past_dev, int capacity,
                   float scale);
int b2w4_qkv_prepare(b2w4_ctx* ctx, const float* qkv_dev, int ld, int tokens, int heads,
                     int kv_heads, int dim, const float* q_weight_dev, const float* k_weight_dev,
                     float eps, const float* cos_dev, const float* sin_dev, int past,
                     const int* past_dev, float* q_out_dev, float* k_cache_dev, float* v_cache_dev,
                     int capacity);
int b2w4_advance(b2w4_ctx* ctx, int* counter_dev, int by, const int32_t* token_dev,
                 int32_t* history_dev, int history_len);
int b2w4_copy_rows(b2w4_ctx* ctx, const float* src_dev, int ld_src, float* dst_dev, int ld_dst,
                   int rows, int cols);
/* Host function (no device, no context): cos / sin tables [positions][rope_dim / 2] for
 * b2w4_rope / b2w4_qkv_prepare, filled as the reference's engine fills them
 * (engine/input_prep.cpp:18-31), in fp32 through the host libm's float functions. */
int b2w4_rope_tables(float* cos_host, float* sin_host, int positions, int first_position,
                     int rope_dim, float theta);
int b2w4_embed_rows(b2w4_ctx* ctx, const void* table_fp16_dev, const int32_t* ids_dev, int rows,
                    int dim, float* out_dev, int ldo);

/* Launch counter: how many of this library's kernels have been launched on the
 * context since creation (for benchmark bookkeeping). */
uint64_t b2w4_kernel_launches(const b2w4_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* B200W4_H */
