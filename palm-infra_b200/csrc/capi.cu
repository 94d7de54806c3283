// extern "C" entry points of libb200w4 (declared in include/b200w4.h): argument checks,
// context and weight lifetime, and dispatch to the kernels' launchers.  No arithmetic here.
#include "b200w4_internal.cuh"

#include <math.h>

#include <cstdlib>
#include <cstring>
#include <new>

int b2w4_fail(b2w4_ctx* ctx, int code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

int b2w4_reserve(b2w4_ctx* ctx, int slot, size_t bytes, void** out) {
    if (ctx->scratch_cap[slot] < bytes) {
        // the old block may still be read by queued kernels
        B2W4_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->scratch[slot])
            cudaFree(ctx->scratch[slot]);
        ctx->scratch[slot] = nullptr;
        ctx->scratch_cap[slot] = 0;
        size_t cap = bytes + bytes / 4 + 4096;
        cudaError_t e = cudaMalloc(&ctx->scratch[slot], cap);
        if (e != cudaSuccess)
            return b2w4_fail(ctx, B2W4_E_NOMEM, "cudaMalloc(%zu): %s", cap,
                             cudaGetErrorString(e));
        ctx->scratch_cap[slot] = cap;
    }
    *out = ctx->scratch[slot];
    return B2W4_OK;
}

extern "C" {

const char* b2w4_version(void) { return "b200w4 0.1 (sm_100a)"; }

// Host function, no device involved: the rotary-embedding tables as the reference's engine
// fills them (engine/input_prep.cpp:18-31) -- theta_i = 1 / theta^(2i / rope_dim), angle =
// position * theta_i, cosine and sine of the angle, every step in fp32 through the host
// libm's float functions, so that on the same host the tables carry the engine's bits
// (the float cosine and sine of a libm are within an ulp of the exact value, not always equal
// to it, and differ between implementations).
int b2w4_rope_tables(float* cos_host, float* sin_host, int positions, int first_position,
                     int rope_dim, float theta) {
    if (!cos_host || !sin_host || positions <= 0 || first_position < 0 || rope_dim <= 0 ||
        (rope_dim & 1) || !(theta > 0.f))
        return B2W4_E_INVALID;
    const int half = rope_dim / 2;
    for (int n = 0; n < positions; ++n) {
        const int pos = first_position + n;
        for (int i = 0; i < half; ++i) {
            const float inv = 1.0f / powf(theta, 2.0f * i / rope_dim);
            const float angle = pos * inv;
            cos_host[(size_t)n * half + i] = cosf(angle);
            sin_host[(size_t)n * half + i] = sinf(angle);
        }
    }
    return B2W4_OK;
}

int b2w4_ctx_create(int device, b2w4_ctx** out) {
    if (!out)
        return B2W4_E_INVALID;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count ||
        device >= kMaxDevices)
        return B2W4_E_NO_DEVICE;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess)
        return B2W4_E_NO_DEVICE;
    if (prop.major != 10)  // the kernels are built for sm_100a only
        return B2W4_E_NO_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess)
        return B2W4_E_CUDA;
    b2w4_ctx* ctx = new (std::nothrow) b2w4_ctx();
    if (!ctx)
        return B2W4_E_NOMEM;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->peer_wait_cycles = kTpWaitLimitCycles;
    const char* pdl = getenv("B2W4_PDL");
    ctx->pdl = !(pdl && pdl[0] == '0');
    const char* tpc = getenv("B2W4_GEMV_TPC");  // tuning: cap on tiles per GEMV CTA
    if (tpc && atoi(tpc) > 0)
        ctx->gemv_tpc_override = atoi(tpc);
    const char* gk = getenv("B2W4_GEMM");  // tuning: "tc" / "mma" force one many-row kernel
    if (gk && gk[0] == 't')
        ctx->gemm_kind = 1;
    if (gk && gk[0] == 'm')
        ctx->gemm_kind = 2;
    const char* at = getenv("B2W4_ATTN");  // debug: "row" keeps the one-row attention kernel
    if (at && at[0] == 'r')
        ctx->attn_tiles = false;
    const char* gmr = getenv("B2W4_GEMV_MAX_ROWS");  // tuning/debug: rows kept on the GEMV
    if (gmr && atoi(gmr) > 0)
        ctx->gemv_max_rows = atoi(gmr);
    if (cudaMalloc(reinterpret_cast<void**>(&ctx->flag_dev), 256) != cudaSuccess ||
        cudaMemset(ctx->flag_dev, 0, 256) != cudaSuccess) {
        delete ctx;
        return B2W4_E_NOMEM;
    }
    if (cudaHostAlloc(reinterpret_cast<void**>(&ctx->status_host), 64, cudaHostAllocMapped) !=
            cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->status_dev), ctx->status_host,
                                 0) != cudaSuccess) {
        if (ctx->status_host)
            cudaFreeHost(ctx->status_host);
        cudaFree(ctx->flag_dev);
        delete ctx;
        return B2W4_E_NOMEM;
    }
    *ctx->status_host = 0;
    *out = ctx;
    return B2W4_OK;
}

void b2w4_ctx_destroy(b2w4_ctx* ctx) {
    if (!ctx)
        return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 8; ++i)
        if (ctx->scratch[i])
            cudaFree(ctx->scratch[i]);
    if (ctx->flag_dev)
        cudaFree(ctx->flag_dev);
    if (ctx->status_host)
        cudaFreeHost(ctx->status_host);
    delete ctx;
}

int b2w4_ctx_set_stream(b2w4_ctx* ctx, void* stream) {
    if (!ctx)
        return B2W4_E_INVALID;
    ctx->stream = static_cast<cudaStream_t>(stream);
    return B2W4_OK;
}

int b2w4_ctx_set_peer_wait_ms(b2w4_ctx* ctx, int milliseconds) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (milliseconds < 1 || milliseconds > 10000)
        return b2w4_fail(ctx, B2W4_E_INVALID, "peer wait: 1..10000 ms (got %d)", milliseconds);
    int khz = 0;  // SM clock in kHz: the kernels count SM cycles
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device);
    if (khz <= 0)
        khz = 1965000;
    ctx->peer_wait_cycles = (unsigned long long)milliseconds * (unsigned long long)khz;
    return B2W4_OK;
}

int b2w4_ctx_set_moe_rule(b2w4_ctx* ctx, int act_rule) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (act_rule != B2W4_ACT_G128 && act_rule != B2W4_ACT_G32)
        return b2w4_fail(ctx, B2W4_E_INVALID, "moe rule must be 128 or 32");
    ctx->moe_rule = act_rule;
    return B2W4_OK;
}

// Drains the stream and reads the status word a kernel sets when one of its bounded waits
// gave up; clears it so that the context stays usable.
static int drain_and_check(b2w4_ctx* ctx) {
    B2W4_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int status = *reinterpret_cast<volatile int*>(ctx->status_host);
    if (status != 0) {
        *reinterpret_cast<volatile int*>(ctx->status_host) = 0;
        cudaMemset(ctx->flag_dev + 2, 0, sizeof(int));  // the persistent kernel's abort word
        return b2w4_fail(ctx, status, "a device-side wait ran out of iterations");
    }
    return B2W4_OK;
}

int b2w4_sync(b2w4_ctx* ctx) {
    if (!ctx)
        return B2W4_E_INVALID;
    return drain_and_check(ctx);
}

const char* b2w4_last_error(const b2w4_ctx* ctx) { return ctx ? ctx->err : "no context"; }

uint64_t b2w4_kernel_launches(const b2w4_ctx* ctx) { return ctx ? ctx->launches : 0; }

// ---- weights -----------------------------------------------------------------------

static int weight_create(b2w4_ctx* ctx, const void* dev_blocks, int n, int k,
                         b2w4_weight** out) {
    b2w4_weight* w = new (std::nothrow) b2w4_weight();
    if (!w)
        return b2w4_fail(ctx, B2W4_E_NOMEM, "out of host memory");
    w->n = n;
    w->k = k;
    w->tiles = (n + 7) / 8;
    w->groups = k / 128;
    int rc = b2w4_launch_repack(ctx, dev_blocks, w);
    if (rc != B2W4_OK) {
        if (w->nib)
            cudaFree(w->nib);
        if (w->scl)
            cudaFree(w->scl);
        delete w;
        return rc;
    }
    *out = w;
    return B2W4_OK;
}

static int check_weight_shape(b2w4_ctx* ctx, const void* blocks, int n, int k,
                              b2w4_weight** out) {
    if (!ctx || !out)
        return B2W4_E_INVALID;
    *out = nullptr;
    if (!blocks || n <= 0 || k <= 0 || k % 128 != 0)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "weight: need blocks, n>0 and k a positive multiple of 128 "
                         "(n=%d k=%d)", n, k);
    return B2W4_OK;
}

int b2w4_weight_upload(b2w4_ctx* ctx, const void* host_blocks, int n, int k,
                       b2w4_weight** out) {
    int rc = check_weight_shape(ctx, host_blocks, n, k, out);
    if (rc != B2W4_OK)
        return rc;
    const size_t bytes = (size_t)((n + 7) / 8) * (k / 128) * 544;
    void* staging = nullptr;
    cudaError_t e = cudaMalloc(&staging, bytes);
    if (e != cudaSuccess)
        return b2w4_fail(ctx, B2W4_E_NOMEM, "cudaMalloc(%zu): %s", bytes,
                         cudaGetErrorString(e));
    e = cudaMemcpyAsync(staging, host_blocks, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(staging);
        return b2w4_fail(ctx, B2W4_E_CUDA, "H2D weight copy: %s", cudaGetErrorString(e));
    }
    rc = weight_create(ctx, staging, n, k, out);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(staging);
    return rc;
}

int b2w4_weight_from_device(b2w4_ctx* ctx, const void* device_blocks, int n, int k,
                            b2w4_weight** out) {
    int rc = check_weight_shape(ctx, device_blocks, n, k, out);
    if (rc != B2W4_OK)
        return rc;
    return weight_create(ctx, device_blocks, n, k, out);
}

void b2w4_weight_free(b2w4_ctx* ctx, b2w4_weight* w) {
    if (!w)
        return;
    if (ctx)
        cudaStreamSynchronize(ctx->stream);
    if (w->nib)
        cudaFree(w->nib);
    if (w->scl)
        cudaFree(w->scl);
    delete w;
}

int b2w4_weight_shape(const b2w4_weight* w, int* n, int* k) {
    if (!w)
        return B2W4_E_INVALID;
    if (n)
        *n = w->n;
    if (k)
        *k = w->k;
    return B2W4_OK;
}

int b2w4_weight_scales_fp16(const b2w4_weight* w) { return w ? w->scales_fp16 : 0; }

size_t b2w4_weight_stream_bytes(const b2w4_weight* w) {
    return w ? w->nib_bytes + w->scl_bytes : 0;
}

// ---- matmul ------------------------------------------------------------------------

static int check_matmul(b2w4_ctx* ctx, const b2w4_weight* w, const void* x, int lda,
                        const void* y, int ldc, int m, int act_rule, int activation) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!w || !x || !y)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul: null weight or tensor");
    if (m <= 0 || lda < w->k || ldc < w->n)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "matmul: bad shape m=%d lda=%d (k=%d) ldc=%d (n=%d)", m, lda,
                         w->k, ldc, w->n);
    if (act_rule != B2W4_ACT_G128 && act_rule != B2W4_ACT_G32)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul: act_rule must be 128 or 32");
    if (activation < B2W4_NONE || activation > B2W4_RELU_SQUARED)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul: unknown activation %d", activation);
    return B2W4_OK;
}

// Up to eight activation rows stream the weight once through the GEMV kernels (one row:
// dp4a; two to eight: the warp-level int8 tensor instruction); more rows go to the tcgen05
// kernel (K <= 10240).  All produce the same bits for the same activation rule.
static int matmul_dispatch(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                           float* y, int ldc, int m, int act_rule, int activation,
                           int act_n_begin, int act_n_len) {
    const bool rows = m > ctx->gemv_max_rows;
    // unaligned activation rows: the tcgen05 path's quantiser reads scalars
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (lda & 3) == 0;
    const bool tc = rows && w->groups <= 80;
    // mma.sync with register accumulators: when asked for, or when the tensor-core kernel
    // cannot take the call; of itself under the per-128 rule for weights whose CTAs are all
    // resident at once, and under the per-32 rule for up to 32 rows (measured: a quarter of
    // a token block does not pay for the tensor-memory pipeline)
    const bool mma = rows && vec && b2w4_gemm_mma_fits(w, m, act_rule) &&
                     (ctx->gemm_kind == 2 || !tc ||
                      (ctx->gemm_kind == 0 &&
                       (act_rule == B2W4_ACT_G128
                            ? b2w4_gemm_mma_resident(w, m, act_rule, ctx->sm_count)
                            : m <= 32)));
    if (mma)
        return b2w4_launch_gemm_mma(ctx, w, x, lda, y, ldc, m, act_rule, activation, act_n_begin,
                                    act_n_len);
    if (tc)
        return b2w4_launch_gemm_tc(ctx, w, x, lda, y, ldc, m, act_rule, activation, act_n_begin,
                                   act_n_len);
    return b2w4_launch_gemv(ctx, w, x, lda, y, ldc, m, act_rule, activation, act_n_begin,
                            act_n_len, nullptr);
}

int b2w4_matmul(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda,
                float* y_dev, int ldc, int m, int act_rule, int activation,
                int act_n_begin, int act_n_len) {
    int rc = check_matmul(ctx, w, x_dev, lda, y_dev, ldc, m, act_rule, activation);
    if (rc != B2W4_OK)
        return rc;
    return matmul_dispatch(ctx, w, x_dev, lda, y_dev, ldc, m, act_rule, activation,
                           act_n_begin, act_n_len);
}

int b2w4_matmul_host(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_host, int lda,
                     float* y_host, int ldc, int m, int act_rule, int activation,
                     int act_n_begin, int act_n_len) {
    int rc = check_matmul(ctx, w, x_host, lda, y_host, ldc, m, act_rule, activation);
    if (rc != B2W4_OK)
        return rc;
    void *xd = nullptr, *yd = nullptr;
    const size_t xb = sizeof(float) * (size_t)m * w->k, yb = sizeof(float) * (size_t)m * w->n;
    if ((rc = b2w4_reserve(ctx, SCR_STAGE_X, xb, &xd)) != B2W4_OK ||
        (rc = b2w4_reserve(ctx, SCR_STAGE_Y, yb, &yd)) != B2W4_OK)
        return rc;
    // contiguous rows (always the case for one row) take the plain 1-D copy
    if (m == 1 || lda == w->k)
        B2W4_CUDA(ctx, cudaMemcpyAsync(xd, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
    else
        B2W4_CUDA(ctx, cudaMemcpy2DAsync(xd, sizeof(float) * w->k, x_host, sizeof(float) * lda,
                                         sizeof(float) * w->k, m, cudaMemcpyHostToDevice,
                                         ctx->stream));
    // A small result in mapped pinned host memory is stored by the kernel itself, straight
    // across the host link: no second copy-engine hop before the host may read it (measured on
    // the decode GEMV: 21 us per call instead of 28 us).  Large results keep the copy engine.
    if (yb <= (1u << 20)) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, y_host) == cudaSuccess &&
            at.type == cudaMemoryTypeHost && at.devicePointer) {
            rc = matmul_dispatch(ctx, w, static_cast<const float*>(xd), w->k,
                                 static_cast<float*>(at.devicePointer), ldc, m, act_rule,
                                 activation, act_n_begin, act_n_len);
            if (rc != B2W4_OK)
                return rc;
            return drain_and_check(ctx);  // a kernel's time-out is this call's return value
        }
        cudaGetLastError();  // pageable memory: not an error, take the staged path
    }
    rc = matmul_dispatch(ctx, w, static_cast<const float*>(xd), w->k,
                         static_cast<float*>(yd), w->n, m, act_rule, activation, act_n_begin,
                         act_n_len);
    if (rc != B2W4_OK)
        return rc;
    if (m == 1 || ldc == w->n)
        B2W4_CUDA(ctx, cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, ctx->stream));
    else
        B2W4_CUDA(ctx, cudaMemcpy2DAsync(y_host, sizeof(float) * ldc, yd, sizeof(float) * w->n,
                                         sizeof(float) * w->n, m, cudaMemcpyDeviceToHost,
                                         ctx->stream));
    return drain_and_check(ctx);
}

int b2w4_matmul_tp(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda, int m,
                   int ldc, int n_offset, const b2w4_tp_group* group, int activation,
                   int act_n_begin, int act_n_len) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!w || !x_dev || !group || group->world < 1 || group->world > kTpMaxWorld ||
        group->rank < 0 || group->rank >= group->world || n_offset < 0 ||
        ldc < n_offset + w->n || m < 1 || m > kTpMaxRows || lda < w->k)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_tp: bad argument");
    if (activation < B2W4_NONE || activation > B2W4_RELU_SQUARED)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_tp: unknown activation %d", activation);
    b2w4_tp_args tp = {};
    for (int p = 0; p < group->world; ++p) {
        if (!group->stage_peers[p] || (reinterpret_cast<uintptr_t>(group->stage_peers[p]) & 7))
            return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_tp: null or unaligned peer pointer");
        tp.stage_peer[p] = static_cast<unsigned long long*>(group->stage_peers[p]);
    }
    tp.world = group->world;
    tp.rank = group->rank;
    tp.n_offset = n_offset;
    return b2w4_launch_gemv(ctx, w, x_dev, lda, nullptr, ldc, m, B2W4_ACT_G128, activation,
                            act_n_begin, act_n_len, nullptr, &tp);
}

// One word per activation row for the fused greedy token (zero between uses).
static unsigned long long* top1_cells(b2w4_ctx* ctx) {
    return reinterpret_cast<unsigned long long*>(ctx->flag_dev + 16);
}

int b2w4_matmul_argmax(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda, int m,
                       float* y_dev, int ldc, int32_t* token_dev) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!w || !x_dev || !token_dev || m < 1 || m > kTop1MaxRows || lda < w->k ||
        (y_dev && ldc < w->n))
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_argmax: bad argument (1..%d rows)",
                         kTop1MaxRows);
    b2w4_top1_args top1;
    top1.cells = top1_cells(ctx);
    int rc = b2w4_launch_gemv(ctx, w, x_dev, lda, y_dev, ldc, m, B2W4_ACT_G128, B2W4_NONE, 0, -1,
                              nullptr, nullptr, &top1);
    if (rc != B2W4_OK)
        return rc;
    return b2w4_launch_top1_token(ctx, top1.cells, token_dev, m);
}

static int tp_args_from_group(b2w4_ctx* ctx, const b2w4_tp_group* group, int n_offset,
                              b2w4_tp_args* tp, const char* who) {
    if (!group || group->world < 1 || group->world > kTpMaxWorld || group->rank < 0 ||
        group->rank >= group->world || n_offset < 0)
        return b2w4_fail(ctx, B2W4_E_INVALID, "%s: bad group", who);
    *tp = b2w4_tp_args();
    for (int p = 0; p < group->world; ++p) {
        if (!group->stage_peers[p] || (reinterpret_cast<uintptr_t>(group->stage_peers[p]) & 7))
            return b2w4_fail(ctx, B2W4_E_INVALID, "%s: null or unaligned peer pointer", who);
        tp->stage_peer[p] = static_cast<unsigned long long*>(group->stage_peers[p]);
    }
    tp->world = group->world;
    tp->rank = group->rank;
    tp->n_offset = n_offset;
    return B2W4_OK;
}

int b2w4_matmul_argmax_tp(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda,
                          int m, int n_offset, const b2w4_tp_group* group) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!w || !x_dev || m < 1 || m > kTop1MaxRows || lda < w->k)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_argmax_tp: bad argument (1..%d rows)",
                         kTop1MaxRows);
    b2w4_tp_args tp;
    int rc = tp_args_from_group(ctx, group, n_offset, &tp, "matmul_argmax_tp");
    if (rc != B2W4_OK)
        return rc;
    b2w4_tp_args offset_only = b2w4_tp_args();  // the matmul only needs n_offset
    offset_only.n_offset = n_offset;
    b2w4_top1_args top1;
    top1.cells = top1_cells(ctx);
    rc = b2w4_launch_gemv(ctx, w, x_dev, lda, nullptr, 0, m, B2W4_ACT_G128, B2W4_NONE, 0, -1,
                          nullptr, &offset_only, &top1);
    if (rc != B2W4_OK)
        return rc;
    return b2w4_launch_tp_send_token(ctx, top1.cells, tp, m);
}

int b2w4_tp_gather_token(b2w4_ctx* ctx, const b2w4_tp_group* group, int32_t* token_dev, int m) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!token_dev || m < 1 || m > kTop1MaxRows)
        return b2w4_fail(ctx, B2W4_E_INVALID, "tp_gather_token: bad argument");
    b2w4_tp_args tp;
    int rc = tp_args_from_group(ctx, group, 0, &tp, "tp_gather_token");
    if (rc != B2W4_OK)
        return rc;
    return b2w4_launch_tp_gather_token(ctx, tp.stage_peer[tp.rank], token_dev, m, tp.world);
}

int b2w4_tp_gather(b2w4_ctx* ctx, const b2w4_tp_group* group, float* y_dev, int m, int ldc) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!group || !y_dev || ldc <= 0 || m < 1 || m > kTpMaxRows || group->world < 1 || group->world > kTpMaxWorld ||
        group->rank < 0 || group->rank >= group->world || !group->stage_peers[group->rank])
        return b2w4_fail(ctx, B2W4_E_INVALID, "tp_gather: bad argument");
    return b2w4_launch_tp_gather(
        ctx, static_cast<unsigned long long*>(group->stage_peers[group->rank]), y_dev, m, ldc);
}

int b2w4_debug_group_sums(b2w4_ctx* ctx, const b2w4_weight* w, const float* x_dev, int lda,
                          int m, int act_rule, int32_t* sums_dev) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!w || !x_dev || !sums_dev || m <= 0 || lda < w->k)
        return b2w4_fail(ctx, B2W4_E_INVALID, "group_sums: bad argument");
    if (act_rule != B2W4_ACT_G128 && act_rule != B2W4_ACT_G32)
        return b2w4_fail(ctx, B2W4_E_INVALID, "group_sums: act_rule must be 128 or 32");
    void* yd = nullptr;
    int rc = b2w4_reserve(ctx, SCR_STAGE_Y, sizeof(float) * (size_t)m * w->n, &yd);
    if (rc != B2W4_OK)
        return rc;
    return b2w4_launch_gemv(ctx, w, x_dev, lda, static_cast<float*>(yd), w->n, m, act_rule,
                            B2W4_NONE, 0, -1, sums_dev);
}

int b2w4_quantize_activations(b2w4_ctx* ctx, const float* x_dev, int lda, int m, int k,
                              int act_rule, int8_t* q_dev, float* scales_dev) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!x_dev || !q_dev || !scales_dev)
        return b2w4_fail(ctx, B2W4_E_INVALID, "quantize: null pointer");
    return b2w4_launch_quantize(ctx, x_dev, lda, m, k, act_rule, q_dev, scales_dev,
                                QLAYOUT_NATURAL);
}

}  // extern "C"
