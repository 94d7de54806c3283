// Internal declarations shared by the b200w4 translation units (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "b200w4.h"

// ---------------------------------------------------------------------------
// Device weight: the canonical BG128 stream split into two planes.
//   nib: [tiles][groups][32] uint4 -- for 8-row tile t and 128-k group g, 32
//        16-byte chunks in the block's own order: chunk (sub*8 + row) holds
//        k = g*128 + sub*32 .. +31 of row t*8+row, low nibble = even k.
//   scl: [tiles][groups][8] fp16 (or fp32 when a scale is not fp16-exact).
// One 8x128 block is 512 B + 16 B: 4.125 bits per weight.
// ---------------------------------------------------------------------------
struct b2w4_weight {
    int n = 0, k = 0, tiles = 0, groups = 0;
    int scales_fp16 = 1;
    uint4* nib = nullptr;
    void* scl = nullptr;
    size_t nib_bytes = 0, scl_bytes = 0;
};

struct b2w4_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    bool pdl = true;  // programmatic dependent launch between consecutive kernels
    int gemv_max_rows = 8;  // activation rows up to which the GEMV kernels are used
    // 0 = mma.sync GEMM when its resident mode fits (few tokens), else the tcgen05 GEMM;
    // tuning: 1 = always the tcgen05 GEMM, 2 = the mma.sync GEMM whenever the shape fits it
    int gemm_kind = 0;
    bool attn_tiles = true;  // a run of tokens takes the tile attention kernel
    int gemv_tpc_override = 0;  // tuning: cap on 8-row tiles per GEMV CTA (0 = heuristic)
    // Routed MoE: B2W4_ACT_G32 = the reference's rule (an expert that holds several rows
    // quantises its activations per 32 values, a lone row per 128); B2W4_ACT_G128 = per 128
    // for every row.
    int moe_rule = B2W4_ACT_G32;
    unsigned long long peer_wait_cycles = 0;  // bound of waits for a peer's stores (set at create)
    char err[512] = {0};
    // grow-only scratch (quantised activations, MoE work lists, staging)
    void* scratch[8] = {nullptr};
    size_t scratch_cap[8] = {0};
    int* flag_dev = nullptr;  // device words: arrival counters, greedy-token cells
    // The status word a kernel sets when a bounded wait gives up lives in mapped pinned HOST
    // memory: the host reads it after a stream synchronise with no copy.  status_dev is the
    // same word's device address.
    int* status_host = nullptr;
    int* status_dev = nullptr;
};

enum ScratchSlot {
    SCR_QA = 0,      // quantised activations
    SCR_AS = 1,      // activation scales
    SCR_STAGE_X = 2, // host-call staging: x
    SCR_STAGE_Y = 3, // host-call staging: y
    SCR_MOE_A = 4,
    SCR_MOE_B = 5,
    SCR_MOE_C = 6,
    SCR_MOE_D = 7,
};

int b2w4_fail(b2w4_ctx* ctx, int code, const char* fmt, ...);
int b2w4_reserve(b2w4_ctx* ctx, int slot, size_t bytes, void** out);

#define B2W4_CUDA(ctx, call)                                                      \
    do {                                                                          \
        cudaError_t e__ = (call);                                                 \
        if (e__ != cudaSuccess)                                                   \
            return b2w4_fail((ctx), B2W4_E_CUDA, "%s: %s", #call,                 \
                             cudaGetErrorString(e__));                            \
    } while (0)

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of a kernel PER
// DEVICE: a cache of what has been configured is indexed by the context's device.
constexpr int kMaxDevices = 64;
struct b2w4_smem_optin {
    size_t bytes[kMaxDevices];  // zero-initialised as a function-local static
};
template <typename Kernel>
inline cudaError_t b2w4_opt_in_smem(b2w4_ctx* ctx, Kernel kern, size_t smem,
                                    b2w4_smem_optin& cache) {
    size_t& have = cache.bytes[ctx->device];
    if (smem <= 48 * 1024 || smem <= have)
        return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e == cudaSuccess)
        have = smem;
    return e;
}

// kernels' host launchers (defined in the .cu files)
int b2w4_launch_repack(b2w4_ctx* ctx, const void* dev_blocks, b2w4_weight* w);
int b2w4_launch_quantize(b2w4_ctx* ctx, const float* x, int lda, int m, int k,
                         int act_rule, int8_t* q, float* scales, int layout);
// 9..256 rows per launch on mma.sync with register accumulators (gemm_mma.cu)
bool b2w4_gemm_mma_fits(const b2w4_weight* w, int m, int act_rule);
bool b2w4_gemm_mma_resident(const b2w4_weight* w, int m, int act_rule, int sm_count);
int b2w4_launch_gemm_mma(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                         float* y, int ldc, int m, int act_rule, int activation,
                         int act_n_begin, int act_n_len);
int b2w4_launch_quantize_mma(b2w4_ctx* ctx, const float* x, int lda, int m, int k, int m_pad,
                             int act_rule, int8_t* q, float* scales_t, int32_t* es_t);
// Tensor-parallel epilogue of the one-row GEMV: the kernel stores its rows into every rank's
// copy of the output and the launch's last CTA bumps this rank's arrival counter on every
// rank.  world == 0: off.
constexpr int kTpMaxWorld = 8;
// Staging buffer of a peer exchange (uint64 words): word 0 counts completed exchanges, word 1
// is unused, then two halves that alternate between exchanges.  Every data word is
// (exchange number << 32 | fp32 bits), written whole, so a reader needs no fence.
constexpr int kTpStageHeader = 2;
constexpr int kTpMaxRows = 8;  // activation rows per tensor-parallel matmul; half = 8 * ldc words
// Default bound of a wait for another GPU's stores, in SM cycles: about 2 s, the same order
// as the bound of the waits on this GPU's own copies.  It has to cover the skew between the
// ranks' host threads (a peer that is still loading a kernel's code, or growing a scratch
// buffer, when this rank's consumer already spins), not only the flight of the stores.
// b2w4_ctx_set_peer_wait_ms changes it per context.
constexpr unsigned long long kTpWaitLimitCycles = 4000000000ull;
struct b2w4_tp_args {
    unsigned long long* stage_peer[kTpMaxWorld];  // rank p's staging buffer, mapped on this GPU
    int world, rank, n_offset;  // n_offset: first output column of this rank's rows
};

// Fused greedy-token epilogue of the decode matmul (engine/sampler.cpp:72-77: best = 0, then
// every i with logits[i] > logits[best] takes over -- the first maximum wins, a NaN never
// wins unless it sits at index 0, where nothing can beat it).  Each output becomes the 64-bit
// word (order-preserving key of the value << 32 | ~index); the maximum word over a row is its
// token.  cells[8]: one word per activation row, zero between uses: every CTA of the matmul
// folds its maximum in with one fire-and-forget atomic per row and exits -- no fence, no
// counter, so the epilogue adds no latency to a CTA -- and the small kernel that follows in
// the stream reads the cells, clears them and writes the tokens.
constexpr int kTop1MaxRows = 8;
// Tensor-parallel form: every rank's (row, rank) maximum goes to every rank's staging buffer
// as two tagged words (key, ~global index); half = rows * ranks * 2 words.
constexpr int kTop1StageHalf = kTop1MaxRows * kTpMaxWorld * 2;
struct b2w4_top1_args {
    unsigned long long* cells;
};
#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long b2w4_top1_word(float v, int n) {
    unsigned bits = __float_as_uint(v), key;
    if (v != v) {
        key = n == 0 ? 0xFFFFFFFFu : 0u;
    } else {
        if (bits == 0x80000000u)
            bits = 0u;  // -0 == +0: the lower index wins
        key = (bits & 0x80000000u) ? ~bits : bits | 0x80000000u;  // -inf -> 0x007FFFFF > 0
    }
    return ((unsigned long long)key << 32) | (0xFFFFFFFFu - (unsigned)n);
}
// After the output loop, every thread of the CTA: `best` is the thread's maximum word for
// activation row mi (the 8 lanes of a group share mi), s_top1[8] was zeroed at kernel start.
__device__ __forceinline__ void b2w4_top1_finish(const b2w4_top1_args& t, unsigned long long best,
                                                 int mi, int m, unsigned long long* s_top1) {
#pragma unroll
    for (int o = 1; o <= 4; o <<= 1) {
        const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 7) == 0 && mi < m)
        atomicMax(&s_top1[mi], best);
    __syncthreads();
    if ((int)threadIdx.x < m)
        atomicMax(t.cells + threadIdx.x, s_top1[threadIdx.x]);
}
#endif


int b2w4_launch_gemv(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                     float* y, int ldc, int m, int act_rule, int activation,
                     int act_n_begin, int act_n_len, int32_t* sums,
                     const b2w4_tp_args* tp = nullptr, const b2w4_top1_args* top1 = nullptr);
int b2w4_launch_tp_gather(b2w4_ctx* ctx, unsigned long long* stage_local, float* y, int m,
                          int ldc);
int b2w4_launch_top1_token(b2w4_ctx* ctx, unsigned long long* cells, int32_t* token, int m);
int b2w4_launch_tp_send_token(b2w4_ctx* ctx, unsigned long long* cells, const b2w4_tp_args& tp,
                              int m);
int b2w4_launch_tp_gather_token(b2w4_ctx* ctx, unsigned long long* stage_local, int32_t* token,
                                int m, int world);
// 2..8 activation rows per pass on the int8 tensor instruction (gemv_mma.cu)
int b2w4_launch_gemv_mma(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                     float* y, int ldc, int m, int act_rule, int activation,
                     int act_n_begin, int act_n_len, int32_t* sums,
                     const b2w4_tp_args* tp = nullptr, const b2w4_top1_args* top1 = nullptr);

int b2w4_launch_quantize_umma(b2w4_ctx* ctx, const float* x, int lda, int m, int k, int m_pad,
                              int act_rule, int8_t* q, float* scales);
int b2w4_launch_gemm_tc(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                        float* y, int ldc, int m, int act_rule, int activation, int act_n_begin,
                        int act_n_len);

// activation-quantiser output layouts
enum {
    QLAYOUT_NATURAL = 0,  // int8 [M][K], k ascending
    QLAYOUT_EVEN_ODD = 1, // int8 [M][K], each 32-block stored as even16|odd16
    // int8 [M][K]; inside each 128-group: [word position p 0..3][32 bytes], the 32 bytes
    // being the even-k codes 4p..4p+3 of the four 32-blocks (16 bytes) then the odd-k ones:
    // the B-operand words of one lane of the m16n8k32 tensor instruction, contiguous
    QLAYOUT_MMA = 2,
};

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float b2w4_activation(float v, int act) {
    // scalar forms of the reference's fused activations
    // (kernels/activations.h:76-99): SILU = x * 1/(1+exp(-x)), GELU tanh form.
    switch (act) {
    case B2W4_SILU: {
        // exp in fp64 then one rounding: agrees with a correctly rounded expf
        float e = (float)exp(-(double)v);
        float s = __fdiv_rn(1.f, __fadd_rn(1.f, e));
        return __fmul_rn(v, s);
    }
    case B2W4_GELU: {
        const float c = 0.7978845608f;
        float v3 = __fmul_rn(__fmul_rn(v, v), v);
        float inner = __fmul_rn(c, __fadd_rn(v, __fmul_rn(0.044715f, v3)));
        float th = (float)tanh((double)inner);
        return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.f, th));
    }
    case B2W4_RELU:
        return v > 0.f ? v : 0.f;
    case B2W4_RELU_SQUARED: {
        float r = v > 0.f ? v : 0.f;
        return __fmul_rn(r, r);
    }
    default:
        return v;
    }
}

__device__ __forceinline__ bool b2w4_act_applies(int n, int act, int begin, int len,
                                                 int n_total) {
    if (act == B2W4_NONE || len == 0)
        return false;
    if (len < 0 || (begin == 0 && len >= n_total))
        return true;
    return n >= begin && n < begin + len;
}

// One activation group: amax -> scale / inverse -> round-to-nearest-even codes.
// Same rounding points as the reference quantisers
// (kernels/matmul_quant.cpp:602-603, :628-633).
__device__ __forceinline__ void b2w4_quant_params(float amax, float& scale, float& inv) {
    scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
    inv = amax > 0.f ? __fdiv_rn(127.f, amax) : 0.f;
}

__device__ __forceinline__ int b2w4_quant_code(float v, float inv) {
    int q = __float2int_rn(__fmul_rn(v, inv));
    return max(-127, min(127, q));
}

__device__ __forceinline__ uint4 b2w4_ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// A bounded wait gave up: a plain store (every writer stores the same value) into the
// host-mapped status word.  The store drains at the latest at the end of the grid, which is
// before the host's stream synchronise returns.
__device__ __forceinline__ void b2w4_report_timeout(int* status) {
    *reinterpret_cast<volatile int*>(status) = B2W4_E_TIMEOUT;
}

__device__ __forceinline__ void b2w4_pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void b2w4_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// First statements of a small kernel in a chain of dependent launches: let the next kernel's
// CTAs be scheduled now, then wait until everything the previous kernel wrote is visible.
// Nothing may touch memory before this.  (Without the launch attribute both are no-ops.)
__device__ __forceinline__ void b2w4_pdl_chain_entry() {
    b2w4_pdl_launch_dependents();
    b2w4_pdl_wait();
}

// Launch with programmatic stream serialisation: the kernel may become resident while its
// predecessor in the stream still runs (it must call b2w4_pdl_wait / b2w4_pdl_chain_entry
// before touching memory).  Shortens the gap between short dependent kernels.
template <typename... KArgs, typename... Args>
inline cudaError_t b2w4_launch_chained(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                       size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
