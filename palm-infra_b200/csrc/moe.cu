// Routed mixture-of-experts op on the GPU, Qwen3-MoE configuration (softmax top-k routing,
// no shared expert).  Stands in for kernel_qwen3_moe (reference kernels/moe.cpp:576-1129)
// and select_moe_routes (kernels/moe_routing.cpp:25-169):
//   1 router logits          hidden[T,H] x router[E,H]^T, fp16 router, fp64 accumulation
//   2 route selection        top-k by raw logit, ties to the lower expert id, softmax over
//                            the k selected logits
//   3 compaction             counting sort of the T*k routes by expert, tokens ascending
//   4 activation quantiser   int8 per 128 values, once per token (shared by its routes)
//   5 grouped gate_up GEMV   per expert, over its ragged route list  -> [routes][2I]
//   6 SwiGLU + quantiser     silu(gate) * up, int8 per 128 values    -> [routes][I]
//   7 grouped down GEMV                                              -> [routes][H]
//   8 combine                out[t] = sum_e w * y, experts in ascending id, sequential fma
// Expert matmuls use the same W4A8 arithmetic as the dense path (per-128 rule, int32 group
// sums, fp32 chain in group order), so a route's result equals a one-row GEMV of that
// expert's weight slice.  Nothing is atomically accumulated: every output is written by one
// thread in a fixed order.
#include "b200w4_internal.cuh"

namespace {

constexpr unsigned kSpinLimit = 1u << 22;
constexpr unsigned long long kWaitLimitCycles = 4000000000ull;  // SM cycles: about 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// SM cycle counter: cheap to read (the global nanosecond timer is not), good enough to
// bound a wait
__device__ __forceinline__ unsigned long long wait_clock() {
    return (unsigned long long)clock64();
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar) {
    if (mbar_try_wait(bar, 0))
        return true;
    const unsigned long long t0 = wait_clock();
    for (unsigned spins = 0; spins < kSpinLimit; ++spins) {
        if (mbar_try_wait(bar, 0))
            return true;
        if ((spins & 63) == 63 && wait_clock() - t0 > kWaitLimitCycles)
            return false;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- 1. router logits: one warp per (4 tokens, EPW experts) -----------------------------
// fp32 activation times fp16 weight is exact in fp64 and a few thousand such terms of
// similar magnitude add without rounding, so the fp64 sum does not depend on its order;
// one rounding to fp32 at the end (the oracle accumulates the same way).  A lane takes 8
// consecutive columns per step (one 16-byte load of router halves, two of each token's
// activations); the warp's router rows are reused for its 4 tokens.
constexpr int kRouterTok = 4;
// logits of tokens t0..t0+NT-1 against experts e0..e0+EPW-1, computed by one warp.  The K loop
// is unrolled so that several steps' loads are in flight at once: with one token and one
// expert per warp (decode) the warp is a pure latency chain otherwise.
template <int EPW, int NT>
__device__ __forceinline__ void router_logits_warp(const float* __restrict__ hidden, int ldx,
                                                   int tokens, int hidden_size,
                                                   const __half* __restrict__ router,
                                                   int num_experts, float* __restrict__ logits,
                                                   int t0, int e0, int lane) {
    double acc[NT][EPW];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < EPW; ++j)
            acc[i][j] = 0.0;
#pragma unroll (NT == 1 ? 8 : 2)
    for (int d = lane * 8; d < hidden_size; d += 256) {
        float xv[NT][8];
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            // rows past the last token repeat it: loaded, never stored
            const float* x = hidden + (size_t)min(t0 + i, tokens - 1) * ldx + d;
            const float4 lo = *reinterpret_cast<const float4*>(x);
            const float4 hi = *reinterpret_cast<const float4*>(x + 4);
            xv[i][0] = lo.x, xv[i][1] = lo.y, xv[i][2] = lo.z, xv[i][3] = lo.w;
            xv[i][4] = hi.x, xv[i][5] = hi.y, xv[i][6] = hi.z, xv[i][7] = hi.w;
        }
#pragma unroll
        for (int j = 0; j < EPW; ++j) {
            const int e = min(e0 + j, num_experts - 1);
            const uint4 raw = *reinterpret_cast<const uint4*>(router + (size_t)e * hidden_size + d);
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float2 r = __half22float2(h2[c]);
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    acc[i][j] += (double)xv[i][2 * c] * (double)r.x;
                    acc[i][j] += (double)xv[i][2 * c + 1] * (double)r.y;
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < EPW; ++j) {
            double v = acc[i][j];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && t0 + i < tokens && e0 + j < num_experts)
                logits[(size_t)(t0 + i) * num_experts + e0 + j] = (float)v;
        }
}

template <int EPW>
__global__ void moe_router_logits_kernel(const float* __restrict__ hidden, int ldx, int tokens,
                                         int hidden_size, const __half* __restrict__ router,
                                         int num_experts, float* __restrict__ logits) {
    b2w4_pdl_chain_entry();
    const int eblocks = (num_experts + EPW - 1) / EPW;
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int tblocks = (tokens + kRouterTok - 1) / kRouterTok;
    if (wid >= (long long)tblocks * eblocks)
        return;
    const int t0 = (int)(wid / eblocks) * kRouterTok, e0 = (int)(wid % eblocks) * EPW;
    router_logits_warp<EPW, kRouterTok>(hidden, ldx, tokens, hidden_size, router, num_experts,
                                        logits, t0, e0, lane);
}

// Fallback for activations whose rows are not 16-byte aligned: one warp per (token, expert),
// scalar loads.
__global__ void moe_router_logits_scalar_kernel(const float* __restrict__ hidden, int ldx,
                                                int tokens, int hidden_size,
                                                const __half* __restrict__ router,
                                                int num_experts, float* __restrict__ logits) {
    b2w4_pdl_chain_entry();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)tokens * num_experts)
        return;
    const int t = (int)(wid / num_experts), e = (int)(wid % num_experts);
    const float* x = hidden + (size_t)t * ldx;
    const __half* r = router + (size_t)e * hidden_size;
    double acc = 0.0;
    for (int d = lane; d < hidden_size; d += 32)
        acc += (double)x[d] * (double)__half2float(r[d]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0)
        logits[(size_t)t * num_experts + e] = (float)acc;
}

// ---- 2. route selection: one warp per token ---------------------------------------------
// The reference selects by insertion with strict '>' (kernels/moe_routing.cpp:129-142): the
// result is the k largest logits in descending order, equal logits in ascending expert id,
// and a logit that is -inf or NaN never displaces the initial (expert 0, -inf) slot.  Here
// that is k rounds of a warp-wide arg-max over (logit descending, expert id ascending) with
// taken experts masked out; a round is two warp reductions (redux.sync) on integer keys.  Then the softmax over the selected logits: exp(l - l_max),
// sequential fp32 sum, times 1/sum (:157-166).
constexpr int kMaxTopK = 16;
constexpr int kSelectMaxExperts = 1024;  // 32 lanes x 32 logits in registers

// routes of token t, by one warp; also returns lane j's expert (lanes >= top_k: undefined).
// NS = logits per lane (32 * NS >= experts).
template <int NS>
__device__ __forceinline__ int select_routes_warp(const float* logits, int t,
                                                  int num_experts, int top_k,
                                                  int32_t* __restrict__ idx,
                                                  float* __restrict__ weights, int lane) {
    const float* row = logits + (size_t)t * num_experts;
    // the lane's logits (experts lane, lane+32, ...) stay in registers for all k rounds
    float mine[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s)
        mine[s] = lane + 32 * s < num_experts ? row[lane + 32 * s] : NAN;
    float my_v = -INFINITY;   // lane j keeps the j-th selected logit
    int my_e = 0;
    // Order-preserving integer key of a logit: larger float <=> larger key, -0 counted as +0
    // like the float comparison does; NaN and -inf get key 0, which never qualifies (the
    // insertion's strict '>' against its initial -inf).
    uint32_t key[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        const float v = __fadd_rn(mine[s], 0.f);
        const uint32_t u = __float_as_uint(v);
        key[s] = !(v > -INFINITY) ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
    }
    for (int j = 0; j < top_k; ++j) {
        uint32_t bk = 0u;
        int bs = 0;
#pragma unroll
        for (int s = 0; s < NS; ++s)
            if (key[s] > bk) {  // strict: of equal logits the lower expert id stays
                bk = key[s];
                bs = s;
            }
        // two warp reductions: the largest key, then the lowest expert id that holds it
        const uint32_t wk = __reduce_max_sync(0xffffffffu, bk);
        const uint32_t we = __reduce_min_sync(
            0xffffffffu, (wk != 0u && bk == wk) ? (uint32_t)(lane + 32 * bs) : 0xffffffffu);
        if (wk != 0u && (int)(we & 31u) == lane) {
#pragma unroll
            for (int s = 0; s < NS; ++s)
                if (s == (int)(we >> 5))
                    key[s] = 0u;  // taken
        }
        if (lane == j && wk != 0u) {  // the key gives the logit back, bit for bit
            my_v = __uint_as_float((wk & 0x80000000u) ? (wk ^ 0x80000000u) : ~wk);
            my_e = (int)we;
        }
    }
    const float maximum = __shfl_sync(0xffffffffu, my_v, 0);
    // exp in fp64 and one rounding: agrees with a correctly rounded expf
    const float ex = lane < top_k ? (float)exp((double)__fsub_rn(my_v, maximum)) : 0.f;
    float sum = 0.f;
    for (int j = 0; j < top_k; ++j)
        sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, ex, j));
    const float inverse = sum > 0.f ? __fdiv_rn(1.f, sum) : 0.f;
    if (lane < top_k) {
        idx[(size_t)t * top_k + lane] = my_e;
        weights[(size_t)t * top_k + lane] = __fmul_rn(ex, inverse);
    }
    return my_e;
}

// dispatch on the number of experts
__device__ __forceinline__ int select_routes_any(const float* logits, int t, int num_experts,
                                                 int top_k, int32_t* __restrict__ idx,
                                                 float* __restrict__ weights, int lane) {
    if (num_experts <= 128)
        return select_routes_warp<4>(logits, t, num_experts, top_k, idx, weights, lane);
    if (num_experts <= 256)
        return select_routes_warp<8>(logits, t, num_experts, top_k, idx, weights, lane);
    if (num_experts <= 512)
        return select_routes_warp<16>(logits, t, num_experts, top_k, idx, weights, lane);
    return select_routes_warp<kSelectMaxExperts / 32>(logits, t, num_experts, top_k, idx, weights,
                                                      lane);
}

__global__ void moe_select_routes_kernel(const float* __restrict__ logits, int tokens,
                                         int num_experts, int top_k, int32_t* __restrict__ idx,
                                         float* __restrict__ weights) {
    b2w4_pdl_chain_entry();
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= tokens)
        return;
    select_routes_any(logits, t, num_experts, top_k, idx, weights, lane);
}

// ---- 3. compaction: one block ------------------------------------------------------------
// counts, exclusive offsets, and per expert its routes in ascending token order
// (kernels/moe.cpp:759-776).  pos[t][j] = the compact position of token t's j-th route;
// slots[y] = (expert, first route, one past its last route) of the y-th expert that has routes,
// ascending; empty (0, 0, 0) from the number of such experts on: what a grouped-matmul CTA
// needs to start, in one 16-byte load.
// Stable placement, a chunk of routes at a time (one route per thread): lanes of a warp that
// hold the same expert find each other with match.any, the lowest of them records the warp's
// count for that expert, a scan over the warps turns the counts into first slots, and every
// route lands at its warp's first slot plus its rank among the matching lanes.
constexpr int kCompactThreads = 1024;
constexpr int kCompactTableInts = 8192;  // warps x experts count table
__global__ void __launch_bounds__(kCompactThreads)
moe_compact_kernel(const int32_t* __restrict__ idx, int tokens, int top_k, int num_experts,
                   int32_t* __restrict__ offsets, int32_t* __restrict__ route_token,
                   int32_t* __restrict__ pos, int4* __restrict__ slots) {
    b2w4_pdl_chain_entry();
    extern __shared__ int s_int[];
    const int E = num_experts;
    const int nw = min(kCompactThreads / 32, max(1, kCompactTableInts / E));  // warps placing
    int* s_cnt = s_int;             // [E+1] counts
    int* s_cursor = s_cnt + E + 1;  // [E] next free slot per expert
    int* s_wc = s_cursor + E;       // [nw][E]
    const int routes = tokens * top_k;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned lt = (1u << lane) - 1u;
    for (int e = threadIdx.x; e <= E; e += blockDim.x)
        s_cnt[e] = 0;
    for (int y = threadIdx.x; y < E; y += blockDim.x)
        slots[y] = make_int4(0, 0, 0, 0);  // experts with routes overwrite theirs below
    __syncthreads();
    for (int i0 = 0; i0 < routes; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        const int e = i < routes ? idx[i] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (peers & lt) == 0)
            atomicAdd(&s_cnt[e], __popc(peers));  // integer counts: order-free
    }
    __syncthreads();
    // exclusive offsets and the list of experts with routes: entry e sums the counts below it
    for (int e = threadIdx.x; e <= E; e += blockDim.x) {
        int run = 0, rank = 0;
        for (int q = 0; q < e; ++q) {
            const int c = s_cnt[q];
            run += c;
            rank += c > 0;
        }
        offsets[e] = run;
        if (e < E) {
            s_cursor[e] = run;
            if (s_cnt[e] > 0)
                slots[rank] = make_int4(e, run, run + s_cnt[e], 0);
        }
    }
    __syncthreads();
    const int chunk = nw * 32;
    for (int c0 = 0; c0 < routes; c0 += chunk) {
        for (int w = threadIdx.x; w < nw * E; w += blockDim.x)
            s_wc[w] = 0;
        __syncthreads();
        const int i = c0 + threadIdx.x;
        int e = -1;
        unsigned peers = 0;
        if (warp < nw) {  // warp-uniform
            e = i < routes ? idx[i] : -1;
            peers = __match_any_sync(0xffffffffu, e);
            if (e >= 0 && (peers & lt) == 0)
                s_wc[warp * E + e] = __popc(peers);
        }
        __syncthreads();
        for (int x = threadIdx.x; x < E; x += blockDim.x) {
            int run = s_cursor[x];
            for (int w = 0; w < nw; ++w) {
                const int c = s_wc[w * E + x];
                s_wc[w * E + x] = run;
                run += c;
            }
            s_cursor[x] = run;
        }
        __syncthreads();
        if (e >= 0) {
            const int slot = s_wc[warp * E + e] + __popc(peers & lt);
            route_token[slot] = i / top_k;
            pos[i] = slot;
        }
        __syncthreads();
    }
}

size_t compact_smem(int num_experts) {
    int nw = kCompactTableInts / num_experts;
    nw = nw < 1 ? 1 : (nw > kCompactThreads / 32 ? kCompactThreads / 32 : nw);
    return sizeof(int) * ((size_t)2 * num_experts + 1 + (size_t)nw * num_experts);
}

// ---- 1-4 fused for a few tokens (decode) ---------------------------------------------------
// One launch instead of four: every warp of the grid quantises its share of the hidden rows
// and computes its share of the router logits; the block that arrives last at a counter (no
// block waits for another) selects the routes, one warp per token, and compacts them.  Same
// device functions, same bits as the separate kernels.
constexpr int kFusedSwigluTokens = 4;
constexpr int kFusedTokens = 8;
constexpr int kFusedRoutes = 128;
constexpr int kFusedThreads = 128;
__global__ void __launch_bounds__(kFusedThreads)
moe_route_fused_kernel(const float* __restrict__ hidden, int ldx, int tokens, int hidden_size,
                       const __half* __restrict__ router, int num_experts, int top_k,
                       float* logits, int32_t* __restrict__ idx, float* __restrict__ weights,
                       int32_t* __restrict__ offsets, int32_t* __restrict__ route_token,
                       int32_t* __restrict__ pos, int4* __restrict__ slots,
                       int8_t* __restrict__ q_hidden, float* __restrict__ as_hidden,
                       int* __restrict__ arrivals) {
    b2w4_pdl_chain_entry();
    __shared__ int s_last;
    __shared__ int s_route[kFusedRoutes];  // expert of route i = (token, j)
    extern __shared__ int s_cnt[];         // [E+1]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gwarp = blockIdx.x * (kFusedThreads / 32) + warp;
    const int nwarps = gridDim.x * (kFusedThreads / 32);
    // hidden rows -> int8, one warp per (token, 128-group), codes in tensor-operand order
    const int G = hidden_size >> 7;
    for (int task = gwarp; task < tokens * G; task += nwarps) {
        const int row = task / G, g = task - row * G;
        const float4 v = *reinterpret_cast<const float4*>(hidden + (size_t)row * ldx +
                                                          (size_t)g * 128 + lane * 4);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        float scale, inv;
        b2w4_quant_params(amax, scale, inv);
        const int c0 = b2w4_quant_code(v.x, inv), c1 = b2w4_quant_code(v.y, inv);
        const int c2 = b2w4_quant_code(v.z, inv), c3 = b2w4_quant_code(v.w, inv);
        if (lane == 0)
            as_hidden[(size_t)row * G + g] = scale;
        int8_t* blk = q_hidden + (size_t)row * hidden_size + (size_t)g * 128 +
                      ((lane & 7) >> 1) * 32 + (lane >> 3) * 4 + (lane & 1) * 2;
        *reinterpret_cast<char2*>(blk) = make_char2((signed char)c0, (signed char)c2);
        *reinterpret_cast<char2*>(blk + 16) = make_char2((signed char)c1, (signed char)c3);
    }
    // router logits, one warp per expert and block of four tokens
    for (int e = gwarp; e < num_experts; e += nwarps) {
        if (tokens == 1)
            router_logits_warp<1, 1>(hidden, ldx, tokens, hidden_size, router, num_experts, logits,
                                     0, e, lane);
        else
            for (int t0 = 0; t0 < tokens; t0 += kRouterTok)
                router_logits_warp<1, kRouterTok>(hidden, ldx, tokens, hidden_size, router,
                                                  num_experts, logits, t0, e, lane);
    }
    // arrival: the last block to get here sees every block's logits
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(arrivals, 1) == (int)gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    for (int t = warp; t < tokens; t += kFusedThreads / 32) {
        const int e = select_routes_any(logits, t, num_experts, top_k, idx, weights, lane);
        if (lane < top_k)
            s_route[t * top_k + lane] = e;
    }
    for (int e = threadIdx.x; e <= num_experts; e += kFusedThreads)
        s_cnt[e] = 0;
    for (int y = threadIdx.x; y < num_experts; y += kFusedThreads)
        slots[y] = make_int4(0, 0, 0, 0);  // experts with routes overwrite theirs below
    __syncthreads();
    const int routes = tokens * top_k;
    if (threadIdx.x < routes)
        atomicAdd(&s_cnt[s_route[threadIdx.x]], 1);  // integer counts: order-free
    __syncthreads();
    // exclusive scan of the counts (and of "has routes") over the experts, a block-wide chunk
    // of experts at a time; then thread e places its routes in token order
    __shared__ int s_wsum[kFusedThreads / 32][2];
    int carry_run = 0, carry_rank = 0;
    for (int base = 0; base <= num_experts; base += kFusedThreads) {
        const int e = base + threadIdx.x;
        const int c = e < num_experts ? s_cnt[e] : 0;
        int run = c, rank = c > 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {  // inclusive scan inside the warp
            const int r = __shfl_up_sync(0xffffffffu, run, off);
            const int k = __shfl_up_sync(0xffffffffu, rank, off);
            if (lane >= off) {
                run += r;
                rank += k;
            }
        }
        if (lane == 31) {
            s_wsum[warp][0] = run;
            s_wsum[warp][1] = rank;
        }
        __syncthreads();
        int wrun = carry_run, wrank = carry_rank, trun = 0, trank = 0;
#pragma unroll
        for (int w = 0; w < kFusedThreads / 32; ++w) {
            if (w < warp) {
                wrun += s_wsum[w][0];
                wrank += s_wsum[w][1];
            }
            trun += s_wsum[w][0];
            trank += s_wsum[w][1];
        }
        run += wrun - c;          // exclusive
        rank += wrank - (c > 0);
        if (e <= num_experts) {
            offsets[e] = run;
            if (e < num_experts && c > 0) {
                slots[rank] = make_int4(e, run, run + c, 0);
                for (int i = 0; i < routes; ++i)
                    if (s_route[i] == e) {
                        route_token[run] = i / top_k;
                        pos[i] = run;
                        ++run;
                    }
            }
        }
        carry_run += trun;
        carry_rank += trank;
        __syncthreads();
    }
    if (threadIdx.x == 0)
        *arrivals = 0;  // ready for the next launch
}

// ---- 6. SwiGLU + quantiser: one warp per (route, 128-wide group of I) ------------------
// inter = (g * 1/(1+exp(-g))) * u with gate = columns [0,I), up = [I,2I)
// (kernels/moe.cpp:160-183), then the per-128 quantiser; codes in tensor-operand order.
// one warp: 128 values of one route, written to `group_dst` (the 128 code bytes of the group)
// and `scale_dst`
// a32: one scale per 32 values (scale_dst[0..3], the lane's block is lane / 8) instead of one
// per 128 (scale_dst[0])
__device__ __forceinline__ void swiglu_quant_warp(const float* __restrict__ gate_row,
                                                  const float* __restrict__ up_row, int lane,
                                                  int8_t* group_dst, float* scale_dst,
                                                  bool a32 = false) {
    const float* gp = gate_row + lane * 4;
    const float* up = up_row + lane * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float gate = gp[i];
        const float e = (float)exp(-(double)gate);
        const float s = __fdiv_rn(1.f, __fadd_rn(1.f, e));
        v[i] = __fmul_rn(__fmul_rn(gate, s), up[i]);
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int off = 4; off > 0; off >>= 1)  // the lane's 32-block: eight lanes
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (!a32) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
    }
    float scale, inv;
    b2w4_quant_params(amax, scale, inv);
    const int c0 = b2w4_quant_code(v[0], inv), c1 = b2w4_quant_code(v[1], inv);
    const int c2 = b2w4_quant_code(v[2], inv), c3 = b2w4_quant_code(v[3], inv);
    if (a32) {
        if ((lane & 7) == 0)
            scale_dst[lane >> 3] = scale;
    } else if (lane == 0) {
        *scale_dst = scale;
    }
    // tensor-operand order inside the group: [word position][even words of the four
    // 32-blocks, then the odd words]; the lane holds k = 4*lane..+3: 32-block lane/8, even
    // codes at even index 2*(lane%8), 2*(lane%8)+1
    int8_t* blk = group_dst + ((lane & 7) >> 1) * 32 + (lane >> 3) * 4 + (lane & 1) * 2;
    *reinterpret_cast<char2*>(blk) = make_char2((signed char)c0, (signed char)c2);
    *reinterpret_cast<char2*>(blk + 16) = make_char2((signed char)c1, (signed char)c3);
}

// scales: [routes][scale_stride].  offsets (null = per-128 everywhere): first compact route of
// every expert, [num_experts + 1]; a route whose expert holds several routes is quantised per
// 32 values (scales[r][4*g + block]), a lone route per 128 (scales[r][g]).
__global__ void moe_swiglu_quant_kernel(const float* __restrict__ gu, int routes,
                                        int intermediate, int8_t* __restrict__ q,
                                        float* __restrict__ scales, int scale_stride,
                                        const int32_t* __restrict__ offsets, int num_experts,
                                        const int32_t* __restrict__ route_lo,
                                        const int32_t* __restrict__ route_hi) {
    b2w4_pdl_chain_entry();
    const int groups = intermediate >> 7;
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)routes * groups)
        return;
    const int r = (int)(wid / groups), g = (int)(wid % groups);
    // expert-parallel runs only own the compact positions of their experts
    if (route_lo && (r < *route_lo || r >= *route_hi))
        return;
    bool a32 = false;
    if (offsets) {  // the expert of compact route r: offsets[e] <= r < offsets[e + 1]
        int lo = 0, hi = num_experts;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (offsets[mid] <= r)
                lo = mid;
            else
                hi = mid;
        }
        a32 = offsets[lo + 1] - offsets[lo] >= 2;
    }
    const float* gp = gu + (size_t)r * 2 * intermediate + (size_t)g * 128;
    swiglu_quant_warp(gp, gp + intermediate, lane,
                      q + (size_t)r * intermediate + (size_t)g * 128,
                      scales + (size_t)r * scale_stride + (a32 ? g * 4 : g), a32);
}

// ---- 8. combine: one block per (token, 512 hidden columns) -------------------------------
// out[t] starts at 0 and takes fma(w, y, out) for the token's experts in ascending id
// (kernels/moe.cpp:642-645, :966, :1100-1110).  The token's k routes are put in that order
// once per block; pos == nullptr reads route rows in (token, route) order.
constexpr int kCombineThreads = 128;
__global__ void __launch_bounds__(kCombineThreads)
moe_combine_kernel(const float* __restrict__ dn, const int32_t* __restrict__ idx,
                   const float* __restrict__ weights, const int32_t* __restrict__ pos,
                   int tokens, int top_k, int hidden_size, float* __restrict__ out, int ldo) {
    b2w4_pdl_chain_entry();
    __shared__ int s_row[kMaxTopK];
    __shared__ float s_w[kMaxTopK];
    const int t = blockIdx.y;
    if (threadIdx.x < top_k) {
        // rank of this route among the token's routes by expert id (ids are distinct, except
        // for the repeated placeholder slots of a degenerate row: ties go to the lower slot)
        const int j = threadIdx.x;
        const int key = idx[(size_t)t * top_k + j];
        // loaded before the rank is known: one memory round trip instead of two
        const int row = pos ? pos[(size_t)t * top_k + j] : t * top_k + j;
        const float w = weights[(size_t)t * top_k + j];
        int rank = 0;
        for (int o = 0; o < top_k; ++o) {
            const int other = idx[(size_t)t * top_k + o];
            rank += other < key || (other == key && o < j);
        }
        s_row[rank] = row;
        s_w[rank] = w;
    }
    __syncthreads();
    const int d = (blockIdx.x * kCombineThreads + threadIdx.x) * 4;
    if (d >= hidden_size)
        return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < top_k; ++j) {
        const float w = s_w[j];
        const float4 y = *reinterpret_cast<const float4*>(dn + (size_t)s_row[j] * hidden_size + d);
        acc.x = __fmaf_rn(w, y.x, acc.x);
        acc.y = __fmaf_rn(w, y.y, acc.y);
        acc.z = __fmaf_rn(w, y.z, acc.z);
        acc.w = __fmaf_rn(w, y.w, acc.w);
    }
    float* o = out + (size_t)t * ldo + d;
    o[0] = acc.x, o[1] = acc.y, o[2] = acc.z, o[3] = acc.w;  // ldo need not be a multiple of 4
}

// ---- expert-parallel hand-over: route outputs in (token, route) order -------------------
// Row t*top_k+j takes the down-projection output of token t's j-th route when that route's
// expert is one of this rank's, zeros otherwise; summed over the ranks (each row has exactly
// one owner, so the sum only adds zeros) the buffer holds every route's output.
__global__ void moe_scatter_routes_kernel(const float* __restrict__ dn,
                                          const int32_t* __restrict__ idx,
                                          const int32_t* __restrict__ pos, int routes,
                                          int hidden_size, int expert_begin, int expert_count,
                                          float* __restrict__ route_out) {
    b2w4_pdl_chain_entry();
    const int r = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (r >= routes || d >= hidden_size)
        return;
    const int e = idx[r] - expert_begin;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e >= 0 && e < expert_count)
        v = *reinterpret_cast<const float4*>(dn + (size_t)pos[r] * hidden_size + d);
    *reinterpret_cast<float4*>(route_out + (size_t)r * hidden_size + d) = v;
}

// ---- expert-parallel hand-over inside the kernels ---------------------------------------
// Instead of a zero-padded buffer summed by an all-reduce call, the owner of a route stores its
// output row into every rank's staging buffer over peer mappings, each value paired with the
// exchange number in one 8-byte word (the same protocol as the tensor-parallel matmul's
// all-gather); rows of other ranks' experts are left to their owners.
__global__ void moe_scatter_routes_peers_kernel(const float* __restrict__ dn,
                                                const int32_t* __restrict__ idx,
                                                const int32_t* __restrict__ pos, int routes,
                                                int hidden_size, int expert_begin,
                                                int expert_count, int stage_rows,
                                                const b2w4_tp_args peers) {
    b2w4_pdl_chain_entry();
    const int r = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (r >= routes || d >= hidden_size)
        return;
    const int e = idx[r] - expert_begin;
    if (e < 0 || e >= expert_count)
        return;
    const unsigned exchange =
        *reinterpret_cast<const volatile unsigned*>(peers.stage_peer[peers.rank]) + 1u;
    const float4 v = *reinterpret_cast<const float4*>(dn + (size_t)pos[r] * hidden_size + d);
    const unsigned long long tag = (unsigned long long)exchange << 32;
    const ulonglong2 w01 = make_ulonglong2(tag | __float_as_uint(v.x), tag | __float_as_uint(v.y));
    const ulonglong2 w23 = make_ulonglong2(tag | __float_as_uint(v.z), tag | __float_as_uint(v.w));
    const size_t at = kTpStageHeader + (size_t)(exchange & 1) * stage_rows * hidden_size +
                      (size_t)r * hidden_size + d;
#pragma unroll
    for (int p = 0; p < kTpMaxWorld; ++p)
        if (p < peers.world) {
            ulonglong2* dst = reinterpret_cast<ulonglong2*>(peers.stage_peer[p] + at);
            dst[0] = w01;
            dst[1] = w23;
        }
}

// Combine over the staging buffer: as moe_combine_kernel, but every value is taken from the
// current exchange's half once it carries the exchange number (bounded wait: `wait_limit` SM
// cycles).  The last block advances the count of completed exchanges.  An output that lacks
// one of its rows becomes a quiet NaN, never a sum over stale rows.
__global__ void __launch_bounds__(kCombineThreads)
moe_combine_staged_kernel(unsigned long long* stage, int stage_rows,
                          const int32_t* __restrict__ idx, const float* __restrict__ weights,
                          const int32_t* __restrict__ pos, int tokens, int top_k, int hidden_size,
                          float* __restrict__ out, int ldo, unsigned* done, int* status,
                          unsigned long long wait_limit) {
    b2w4_pdl_chain_entry();
    __shared__ int s_row[kMaxTopK];
    __shared__ float s_w[kMaxTopK];
    const int t = blockIdx.y;
    unsigned* count = reinterpret_cast<unsigned*>(stage);
    const unsigned exchange = *reinterpret_cast<volatile unsigned*>(count) + 1u;
    if (threadIdx.x < top_k) {
        const int j = threadIdx.x;
        const int key = idx[(size_t)t * top_k + j];
        const float w = weights[(size_t)t * top_k + j];
        int rank = 0;
        for (int o = 0; o < top_k; ++o) {
            const int other = idx[(size_t)t * top_k + o];
            rank += other < key || (other == key && o < j);
        }
        // rows in compact order (stored by the down-projection itself) or in (token, route)
        // order (stored by the scatter kernel)
        s_row[rank] = pos ? pos[(size_t)t * top_k + j] : t * top_k + j;
        s_w[rank] = w;
    }
    __syncthreads();
    const int d = (blockIdx.x * kCombineThreads + threadIdx.x) * 4;
    if (d < hidden_size) {
        const unsigned long long* half =
            stage + kTpStageHeader + (size_t)(exchange & 1) * stage_rows * hidden_size;
        const long long t0 = clock64();
        bool gave_up = false;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < top_k; ++j) {
            const volatile unsigned long long* src = half + (size_t)s_row[j] * hidden_size + d;
            unsigned long long w0, w1, w2, w3;
            for (;;) {
                w0 = src[0], w1 = src[1], w2 = src[2], w3 = src[3];
                if (((unsigned)(w0 >> 32) == exchange && (unsigned)(w1 >> 32) == exchange &&
                     (unsigned)(w2 >> 32) == exchange && (unsigned)(w3 >> 32) == exchange) ||
                    gave_up)
                    break;
                if ((unsigned long long)(clock64() - t0) > wait_limit) {
                    b2w4_report_timeout(status);
                    gave_up = true;
                }
            }
            if (gave_up) {
                acc = make_float4(__uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u),
                                  __uint_as_float(0x7FC00000u), __uint_as_float(0x7FC00000u));
                break;
            }
            const float w = s_w[j];
            acc.x = __fmaf_rn(w, __uint_as_float((unsigned)w0), acc.x);
            acc.y = __fmaf_rn(w, __uint_as_float((unsigned)w1), acc.y);
            acc.z = __fmaf_rn(w, __uint_as_float((unsigned)w2), acc.z);
            acc.w = __fmaf_rn(w, __uint_as_float((unsigned)w3), acc.w);
        }
        float* o = out + (size_t)t * ldo + d;
        o[0] = acc.x, o[1] = acc.y, o[2] = acc.z, o[3] = acc.w;
    }
    __syncthreads();  // every thread of the block has read the count
    if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x * gridDim.y - 1) {
        *done = 0;  // ready for the next launch
        *count = exchange;
    }
}

// ---- 5 / 7 (few tokens). grouped expert matmul, decode variant -------------------------
// Used for up to kFusedSwigluTokens tokens, where an expert has one or two routes: items
// (tile pair, group) are spread over all warps, the integer sums go through shared memory and
// a second phase runs the fp32 chains; SwiGLU and its quantiser can run in the prologue.  The
// variant below (register accumulators) is faster from a few routes per expert on; this one
// is faster for a decode step (measured on a Qwen3-30B-shaped layer: 26.9 us against 29.0 us
// per layer for one token, 341 us against 272 us for 256 tokens).
// grid = (CTAs per expert, experts that have routes).  CTA (c, y) owns `tpc` 8-row tiles of
// one expert's slice of the aggregate weight and every route of that expert.  The slice's
// nibble stream is bulk-copied into shared memory once and reused for all of the expert's
// routes, eight at a time: the routes are the eight columns of the warp-level int8 tensor
// instruction (mma.sync m16n8k32), the 16 weight rows of a tile pair its rows.  The math is
// the dense small-batch kernel's: phase 1 integer group sums (a weight word w of 8 nibbles
// splits into hi = w & 0xF0F0F0F0, odd k as 16*q, and lo = (w ^ 0x08080808) & 0x0F0F0F0F,
// even k as q+8; sum = mma(lo, a_even) - 8*sum(a_even) + mma(hi, a_odd)/16), phase 2 the
// fp32 chain per (tile, route, weight row) in ascending group order.
constexpr int kSW = 8;          // warps
constexpr int kST = kSW * 32;
constexpr int kSR = 8;          // routes per pass

struct GroupedSmallArgs {
    const uint8_t* nib;
    const void* scl;
    const int8_t* qa;         // [rows][K] int8, tensor-operand order inside each group
    const float* as;          // [rows][G]
    const float* gate_up;     // if set (few routes): the activations are silu(gate)*up of these
                              // fp32 [routes][2K] rows, quantised here instead of read from qa
    const int4* slots;        // y-th expert with routes: (expert, first route, end), else empty
    int num_experts_all;      // experts routed over
    int expert_begin;         // first expert whose weights this aggregate holds
    int expert_count;         // experts held
    const int32_t* row_map;   // route -> activation row, or null for identity
    float* out;               // [routes][n_e]
    int* status;
    int k, groups, n_e, tiles_e, tpc, d_stride;
    b2w4_tp_args peers;       // world != 0: rows go, tagged, to every rank's staging buffer
    int stage_rows;           // rows per half of that buffer
};

template <bool U>
__device__ __forceinline__ void moe_small_mma(int (&d)[4], uint32_t a0, uint32_t a1,
                                                uint32_t a2, uint32_t a3, uint32_t b0,
                                                uint32_t b1) {
    // lane (gid = lane/4, tid = lane%4): a0 row gid, k 4*tid..+3; a1 row gid+8; a2/a3 k+16;
    // b0 k 4*tid..+3 of column gid, b1 k+16; d0/d1 row gid, columns 2*tid, 2*tid+1; d2/d3 row
    // gid+8
    if (U)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SCL16>
__global__ void __launch_bounds__(kST, 2)
moe_grouped_small_kernel(const GroupedSmallArgs a) {
    b2w4_pdl_chain_entry();
    extern __shared__ __align__(128) uint8_t smem[];
    // blockIdx.y walks the experts that have routes, not all experts: a decode token
    // touches top_k of them
    const int4 slot = a.slots[blockIdx.y];
    const int e_all = slot.x, r0 = slot.y, r1 = slot.z;
    const int e = e_all - a.expert_begin;  // index inside the aggregate held here
    if (e < 0 || e >= a.expert_count)
        return;
    const int tl0 = blockIdx.x * a.tpc;
    const int ntile = min(a.tpc, a.tiles_e - tl0);
    if (r0 >= r1 || ntile <= 0)
        return;
    const int G = a.groups, K = a.k;
    const int tile_bytes = G * 512;
    const int scl_tile_bytes = G * 8 * (SCL16 ? 2 : 4);
    uint8_t* s_w = smem;
    uint8_t* s_scl = s_w + (size_t)a.tpc * tile_bytes;
    uint4* s_qa = reinterpret_cast<uint4*>(s_scl + (size_t)a.tpc * scl_tile_bytes);  // [kSR][K]
    float* s_as = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_qa) + (size_t)kSR * K);
    int* s_es = reinterpret_cast<int*>(s_as + kSR * G);  // -8 * sum of the even-k codes
    float* s_d = reinterpret_cast<float*>(s_es + kSR * G);  // [tpc][G][kSR][8] + pad
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(
        (reinterpret_cast<uintptr_t>(s_d + (size_t)a.tpc * a.d_stride) + 7) & ~uintptr_t(7));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tid = lane & 3;
    const size_t gtile0 = (size_t)e * a.tiles_e + tl0;  // tile index in the aggregate

    if (warp == 0) {
        if (lane == 0)
            mbar_init(&s_bar[0], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            const uint32_t wb = (uint32_t)ntile * tile_bytes, sb = (uint32_t)ntile * scl_tile_bytes;
            mbar_expect_tx(&s_bar[0], wb + sb);
            bulk_g2s(s_w, a.nib + gtile0 * tile_bytes, wb, &s_bar[0]);
            bulk_g2s(s_scl, reinterpret_cast<const uint8_t*>(a.scl) + gtile0 * scl_tile_bytes, sb,
                     &s_bar[0]);
        }
    }
    const int npair = (ntile + 1) >> 1;
    const int n_items = npair * G;
    const uint32_t* s_w32 = reinterpret_cast<const uint32_t*>(s_w);
    const int tile_words = tile_bytes >> 2;
    bool weights_ready = false;

    for (int base = r0; base < r1; base += kSR) {
        const int mc = min(kSR, r1 - base);
        // quantised activations of this pass's routes
        if (a.gate_up) {
            // every CTA of the expert repeats this for the expert's routes: cheap for the few
            // routes of a decode step, and it saves a launch
            for (int task = warp; task < mc * G; task += kSW) {
                const int mi = task / G, g = task - mi * G;
                const float* gp = a.gate_up + (size_t)(base + mi) * 2 * K + (size_t)g * 128;
                swiglu_quant_warp(gp, gp + K, lane,
                                  reinterpret_cast<int8_t*>(s_qa) + (size_t)mi * K + (size_t)g * 128,
                                  s_as + mi * G + g);
            }
        } else {
            for (int i = threadIdx.x; i < mc * (K / 16); i += kST) {
                const int mi = i / (K / 16), c = i - mi * (K / 16);
                const int src_row = a.row_map ? a.row_map[base + mi] : base + mi;
                s_qa[mi * (K / 16) + c] =
                    reinterpret_cast<const uint4*>(a.qa + (size_t)src_row * K)[c];
            }
            for (int i = threadIdx.x; i < mc * G; i += kST) {
                const int mi = i / G, g = i - mi * G;
                const int src_row = a.row_map ? a.row_map[base + mi] : base + mi;
                s_as[mi * G + g] = a.as[(size_t)src_row * G + g];
            }
        }
        __syncthreads();
        // -8 * (sum of the even-k codes) per (route, group): the even words of a group are
        // uint4 0, 2, 4, 6 of its 8
        for (int i = threadIdx.x; i < mc * G; i += kST) {
            const uint4* q = s_qa + (size_t)i * 8;
            int sum = 0;
#pragma unroll
            for (int c = 0; c < 8; c += 2) {
                const uint4 v = q[c];
                sum = __dp4a(0x01010101, (int)v.x, sum);
                sum = __dp4a(0x01010101, (int)v.y, sum);
                sum = __dp4a(0x01010101, (int)v.z, sum);
                sum = __dp4a(0x01010101, (int)v.w, sum);
            }
            s_es[i] = -8 * sum;
        }
        if (!weights_ready) {
            if (!mbar_wait_bounded(&s_bar[0])) {
                if (lane == 0)
                    b2w4_report_timeout(a.status);
                return;  // every thread sees the same barrier: the exit is CTA-uniform
            }
            weights_ready = true;
        }
        __syncthreads();
        // phase 1: item = (pair of tiles = 16 weight rows, group); columns = routes
        const int bcol = gid < mc ? gid : 0;  // unused columns repeat route 0, never read back
        const int qa_base = bcol * (K >> 4) + tid * 2;
#pragma unroll 2
        for (int it = warp; it < n_items; it += kSW) {
            const int tp = it / G;
            const int g = it - tp * G;
            const int t0 = tp * 2;
            const bool two = t0 + 1 < ntile;
            // word `lane` of the 128 bytes of (tile, group, 32-block s): row gid, k 8*tid..+7
            const int wbase = t0 * tile_words + g * 128 + lane;
            uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t u = s_w32[wbase + s * 32];
                const uint32_t v = two ? s_w32[wbase + tile_words + s * 32] : 0u;  // q = 0
                lo0[s] = (u ^ 0x08080808u) & 0x0F0F0F0Fu;
                hi0[s] = u & 0xF0F0F0F0u;
                lo1[s] = (v ^ 0x08080808u) & 0x0F0F0F0Fu;
                hi1[s] = v & 0xF0F0F0F0u;
            }
            const uint4 be = s_qa[qa_base + g * 8], bo = s_qa[qa_base + g * 8 + 1];
            int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
            moe_small_mma<true>(cl, lo0[0], lo1[0], lo0[1], lo1[1], be.x, be.y);
            moe_small_mma<false>(ch, hi0[0], hi1[0], hi0[1], hi1[1], bo.x, bo.y);
            moe_small_mma<true>(cl, lo0[2], lo1[2], lo0[3], lo1[3], be.z, be.w);
            moe_small_mma<false>(ch, hi0[2], hi1[2], hi0[3], hi1[3], bo.z, bo.w);
            const int dbase = t0 * a.d_stride + g * (kSR * 8) + gid;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int mi = tid * 2 + c;
                if (mi < mc) {
                    const int e8 = s_es[mi * G + g];
                    // ch sums 16*q4*a: an exact multiple of 16
                    s_d[dbase + mi * 8] = (float)(cl[c] + e8 + (ch[c] >> 4));
                    if (two)
                        s_d[dbase + a.d_stride + mi * 8] =
                            (float)(cl[2 + c] + e8 + (ch[2 + c] >> 4));
                }
            }
        }
        __syncthreads();
        // phase 2
#pragma unroll 1
        for (int t = threadIdx.x; t < ntile * kSR * 8; t += kST) {
            const int rr = t & 7, mi = (t >> 3) % kSR, tl = t / (8 * kSR);
            if (mi >= mc)
                continue;
            const float* dsrc = s_d + tl * a.d_stride + mi * 8 + rr;
            const float* as = s_as + mi * G;
            float acc = 0.f;
#pragma unroll 4
            for (int g = 0; g < G; ++g) {
                const float ws =
                    SCL16 ? __half2float(
                                reinterpret_cast<const __half*>(s_scl)[(tl * G + g) * 8 + rr])
                          : reinterpret_cast<const float*>(s_scl)[(tl * G + g) * 8 + rr];
                acc = __fmaf_rn(dsrc[g * kSR * 8], __fmul_rn(ws, as[g]), acc);
            }
            const int n = (tl0 + tl) * 8 + rr;
            if (n < a.n_e) {
                if (a.peers.world == 0) {
                    a.out[(size_t)(base + mi) * a.n_e + n] = acc;
                } else {
                    // expert-parallel hand-over: the row (its compact position is the same
                    // on every rank) goes to every rank's staging buffer, each value tagged
                    // with the exchange number in one 8-byte word
                    const unsigned exchange =
                        *reinterpret_cast<const volatile unsigned*>(
                            a.peers.stage_peer[a.peers.rank]) + 1u;
                    const unsigned long long word =
                        ((unsigned long long)exchange << 32) | __float_as_uint(acc);
                    const size_t at = kTpStageHeader +
                                      (size_t)(exchange & 1) * a.stage_rows * a.n_e +
                                      (size_t)(base + mi) * a.n_e + n;
#pragma unroll
                    for (int p = 0; p < kTpMaxWorld; ++p)
                        if (p < a.peers.world)
                            a.peers.stage_peer[p][at] = word;
                }
            }
        }
        __syncthreads();
    }
}

int grouped_small_d_stride(int groups) { return groups * kSR * 8 + 8; }

size_t grouped_small_smem(int k, int groups, int tpc, bool scl16) {
    return (size_t)tpc * groups * 512 + (size_t)tpc * groups * 8 * (scl16 ? 2 : 4) +
           (size_t)kSR * k + 2 * sizeof(float) * kSR * groups +
           sizeof(float) * (size_t)tpc * grouped_small_d_stride(groups) + 8 + 16;
}

// ---- 5 / 7. grouped expert matmul over ragged route lists ------------------------------
// grid = (CTAs per expert, experts that have routes).  CTA (c, y) owns `tpc` 8-row tiles of
// one expert's slice of the aggregate weight and every route of that expert.  The slice's
// nibble stream is bulk-copied into shared memory once and reused for all of the expert's
// routes, sixteen at a time.  The integer sums come from the warp-level int8 tensor
// instruction (mma.sync m16n8k32): 16 weight rows of a tile pair are its rows, eight routes
// its columns.  A warp owns one tile pair and one or two column blocks and runs the whole K
// loop on its own: per 128-k group it splits its weight words into unsigned bytes q+8
// (lo = (w ^ 0x08080808) & 0x0F0F0F0F for even k, hi = ((w >> 4) ^ 0x08080808) & 0x0F0F0F0F
// for odd k), accumulates four instructions into an int32 that starts at
// 0x4B400000 - 8*sum(codes) and therefore ends as the bit pattern of the float 12582912 + D,
// and folds D into fp32 chain values  y = fma(float(D), fp32(ws*as), y)  that stay in its
// registers until the last group: no shared-memory hand-off, no barrier inside the K loop.
// The math is the dense kernels', route by route.
constexpr int kGW = 8;          // warps
constexpr int kGT = kGW * 32;
constexpr int kGR = 16;         // routes per pass: two column blocks
constexpr int kRowPad = 16;     // bytes added to a staged activation row: conflict-free reads

struct GroupedArgs {
    const uint8_t* nib;
    const void* scl;
    const int8_t* qa;         // [rows][K] int8, tensor-operand order inside each group
    const float* as;          // [rows][as_stride]: one scale per 128 values at [g]
    // The reference's rule for an expert that holds SEVERAL rows (kernels/moe.cpp:1055-1058
    // -> kernels/matmul_w4.cpp:1125-1154): one activation scale per 32 values.  qa32 / as32
    // are those rows quantised that way (as32[r][4*g + block]); null = per-128 for every
    // expert.  An expert with a single row keeps the per-128 rule (:1058-1075).
    const int8_t* qa32;
    const float* as32;
    int as_stride, as32_stride;
    const int4* slots;        // y-th expert with routes: (expert, first route, end), else empty
    int num_experts_all;      // experts routed over
    int expert_begin;         // first expert whose weights this aggregate holds
    int expert_count;         // experts held
    const int32_t* row_map;   // route -> activation row, or null for identity
    float* out;               // [routes][n_e]
    int* status;
    int k, groups, n_e, tiles_e, tpc;
};

__device__ __forceinline__ void moe_mma_16x8x32(int (&d)[4], uint32_t a0, uint32_t a1,
                                                uint32_t a2, uint32_t a3, uint32_t b0,
                                                uint32_t b1) {
    // lane (gid = lane/4, tid = lane%4): a0 row gid, k 4*tid..+3; a1 row gid+8; a2/a3 k+16;
    // b0 k 4*tid..+3 of column gid, b1 k+16; d0/d1 row gid, columns 2*tid, 2*tid+1; d2/d3 row
    // gid+8.  A unsigned bytes, B signed bytes.
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SCL16>
__global__ void __launch_bounds__(kGT, 2)
moe_grouped_gemv_kernel(const GroupedArgs a) {
    b2w4_pdl_chain_entry();
    extern __shared__ __align__(128) uint8_t smem[];
    // blockIdx.y walks the experts that have routes, not all experts: a decode token
    // touches top_k of them
    const int4 slot = a.slots[blockIdx.y];
    const int e_all = slot.x, r0 = slot.y, r1 = slot.z;
    const int e = e_all - a.expert_begin;  // index inside the aggregate held here
    if (e < 0 || e >= a.expert_count)
        return;
    const int tl0 = blockIdx.x * a.tpc;
    const int ntile = min(a.tpc, a.tiles_e - tl0);
    if (r0 >= r1 || ntile <= 0)
        return;
    const int G = a.groups, K = a.k;
    const int tile_bytes = G * 512;
    const int scl_tile_bytes = G * 8 * (SCL16 ? 2 : 4);
    const int row_bytes = K + kRowPad;
    uint8_t* s_w = smem;
    uint8_t* s_scl = s_w + (size_t)a.tpc * tile_bytes;
    uint8_t* s_qa = s_scl + (size_t)a.tpc * scl_tile_bytes;                         // [kGR][K+pad]
    // per (group or 32-block, route): activation scale and accumulator bias; sized for the
    // per-32 rule (four entries per group)
    float* s_as = reinterpret_cast<float*>(s_qa + (size_t)kGR * row_bytes);         // [4G][kGR]
    int* s_bias = reinterpret_cast<int*>(s_as + kGR * G * 4);                       // [4G][kGR]
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(
        (reinterpret_cast<uintptr_t>(s_bias + kGR * G * 4) + 7) & ~uintptr_t(7));
    // the expert's rule: per 32 values when it holds several rows
    const bool a32 = a.qa32 != nullptr && (r1 - r0) >= 2;
    const int8_t* const qa_src = a32 ? a.qa32 : a.qa;
    const float* const as_src = a32 ? a.as32 : a.as;
    const int as_stride = a32 ? a.as32_stride : a.as_stride;
    const int SPG = a32 ? 4 : 1;  // scales per group

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tid = lane & 3;
    const size_t gtile0 = (size_t)e * a.tiles_e + tl0;  // tile index in the aggregate

    if (warp == 0) {
        if (lane == 0)
            mbar_init(&s_bar[0], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            const uint32_t wb = (uint32_t)ntile * tile_bytes, sb = (uint32_t)ntile * scl_tile_bytes;
            mbar_expect_tx(&s_bar[0], wb + sb);
            bulk_g2s(s_w, a.nib + gtile0 * tile_bytes, wb, &s_bar[0]);
            bulk_g2s(s_scl, reinterpret_cast<const uint8_t*>(a.scl) + gtile0 * scl_tile_bytes, sb,
                     &s_bar[0]);
        }
    }
    // this warp's tile pair and column blocks: with fewer pairs than warps the two column
    // blocks of a pass go to different warps, otherwise a warp takes both (one split of the
    // weight words serves both)
    const int npair = (ntile + 1) >> 1;
    const int npair_cap = (a.tpc + 1) >> 1;
    const int wpp = npair_cap < kGW ? (kGW / npair_cap >= 2 ? 2 : 1) : 1;  // warps per pair
    const uint32_t* s_w32 = reinterpret_cast<const uint32_t*>(s_w);
    const int tile_words = tile_bytes >> 2;
    bool weights_ready = false;

    for (int base = r0; base < r1; base += kGR) {
        const int mc = min(kGR, r1 - base);
        // quantised activations of this pass's routes
        for (int i = threadIdx.x; i < mc * (K / 16); i += kGT) {
            const int mi = i / (K / 16), c = i - mi * (K / 16);
            const int src_row = a.row_map ? a.row_map[base + mi] : base + mi;
            *reinterpret_cast<uint4*>(s_qa + (size_t)mi * row_bytes + c * 16) =
                reinterpret_cast<const uint4*>(qa_src + (size_t)src_row * K)[c];
        }
        for (int i = threadIdx.x; i < mc * G * SPG; i += kGT) {
            const int mi = i / (G * SPG), gs = i - mi * (G * SPG);
            const int src_row = a.row_map ? a.row_map[base + mi] : base + mi;
            s_as[gs * kGR + mi] = as_src[(size_t)src_row * as_stride + gs];
        }
        __syncthreads();
        // accumulator bias per (route, group): 0x4B400000 - 8 * (sum of the group's codes);
        // per-32 rule: per (route, 32-block).  In tensor-operand order the codes of 32-block
        // b are word b of each of the eight 16-byte chunks of the group.
        for (int i = threadIdx.x; i < mc * G; i += kGT) {
            const int mi = i / G, g = i - mi * G;
            const uint4* q = reinterpret_cast<const uint4*>(s_qa + (size_t)mi * row_bytes + g * 128);
            int sum[4] = {0, 0, 0, 0};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 v = q[c];
                sum[0] = __dp4a(0x01010101, (int)v.x, sum[0]);
                sum[1] = __dp4a(0x01010101, (int)v.y, sum[1]);
                sum[2] = __dp4a(0x01010101, (int)v.z, sum[2]);
                sum[3] = __dp4a(0x01010101, (int)v.w, sum[3]);
            }
            if (a32) {
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    s_bias[(g * 4 + b) * kGR + mi] = 0x4B400000 - 8 * sum[b];
            } else {
                s_bias[g * kGR + mi] = 0x4B400000 - 8 * (sum[0] + sum[1] + sum[2] + sum[3]);
            }
        }
        if (!weights_ready) {
            if (!mbar_wait_bounded(&s_bar[0])) {
                if (lane == 0)
                    b2w4_report_timeout(a.status);
                return;  // every thread sees the same barrier: the exit is CTA-uniform
            }
            weights_ready = true;
        }
        __syncthreads();
        const int ncb = (mc + 7) >> 3;  // column blocks in this pass: 1 or 2
#pragma unroll 1
        for (int pair = warp / wpp; pair < npair; pair += kGW / wpp) {
            const int wj = warp % wpp;
            // column blocks of this warp: both, or the one matching its position in the pair;
            // with a single column block (decode) the pair's two warps take one tile each
            // instead (half of the instruction's rows idle, no warp idle)
            const bool split_tiles = wpp == 2 && ncb == 1;
            const int cb_lo = split_tiles ? 0 : (wpp == 2 ? wj : 0);
            const int cb_hi = split_tiles ? 1 : (wpp == 2 ? wj + 1 : 2);
            const int t0 = split_tiles ? pair * 2 + wj : pair * 2;
            if (cb_lo >= ncb || t0 >= ntile)
                continue;
            const bool two = !split_tiles && t0 + 1 < ntile;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
            for (int g = 0; g < G; ++g) {
                // word `lane` of the 128 bytes of (tile, group, 32-block s): row gid, k 8*tid..+7
                const int wbase = t0 * tile_words + g * 128 + lane;
                uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
#pragma unroll
                for (int sb = 0; sb < 4; ++sb) {
                    const uint32_t u = s_w32[wbase + sb * 32];
                    const uint32_t v = two ? s_w32[wbase + tile_words + sb * 32] : 0u;  // q = 0
                    lo0[sb] = (u ^ 0x08080808u) & 0x0F0F0F0Fu;
                    hi0[sb] = ((u >> 4) ^ 0x08080808u) & 0x0F0F0F0Fu;
                    lo1[sb] = (v ^ 0x08080808u) & 0x0F0F0F0Fu;
                    hi1[sb] = ((v >> 4) ^ 0x08080808u) & 0x0F0F0F0Fu;
                }
                const int si = (t0 * G + g) * 8 + gid;
                const float ws0 = SCL16 ? __half2float(reinterpret_cast<const __half*>(s_scl)[si])
                                        : reinterpret_cast<const float*>(s_scl)[si];
                const float ws1 =
                    !two ? 0.f
                         : (SCL16 ? __half2float(
                                        reinterpret_cast<const __half*>(s_scl)[si + G * 8])
                                  : reinterpret_cast<const float*>(s_scl)[si + G * 8]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int cb = cb_lo + j;
                    if (cb < cb_hi && cb < ncb) {  // warp-uniform
                        // unused columns of the last block read stale rows: never stored
                        const uint4* bp = reinterpret_cast<const uint4*>(
                            s_qa + (size_t)(cb * 8 + gid) * row_bytes + g * 128 + tid * 32);
                        const uint4 be = bp[0], bo = bp[1];
                        if (a32) {
                            // one instruction = one 32-block: its own accumulator, bias and
                            // activation scale, folded into the chain in ascending block order
                            // (kernels/matmul_w4.cpp:785-901)
                            const uint32_t bev[4] = {be.x, be.y, be.z, be.w};
                            const uint32_t bov[4] = {bo.x, bo.y, bo.z, bo.w};
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                const int tk = (g * 4 + b) * kGR + cb * 8 + tid * 2;
                                const int2 bias = *reinterpret_cast<const int2*>(s_bias + tk);
                                const float2 asv = *reinterpret_cast<const float2*>(s_as + tk);
                                int c[4] = {bias.x, bias.y, bias.x, bias.y};
                                moe_mma_16x8x32(c, lo0[b], lo1[b], hi0[b], hi1[b], bev[b], bov[b]);
                                acc[j][0] = __fmaf_rn(__fsub_rn(__int_as_float(c[0]), 12582912.f),
                                                      __fmul_rn(ws0, asv.x), acc[j][0]);
                                acc[j][1] = __fmaf_rn(__fsub_rn(__int_as_float(c[1]), 12582912.f),
                                                      __fmul_rn(ws0, asv.y), acc[j][1]);
                                acc[j][2] = __fmaf_rn(__fsub_rn(__int_as_float(c[2]), 12582912.f),
                                                      __fmul_rn(ws1, asv.x), acc[j][2]);
                                acc[j][3] = __fmaf_rn(__fsub_rn(__int_as_float(c[3]), 12582912.f),
                                                      __fmul_rn(ws1, asv.y), acc[j][3]);
                            }
                            continue;
                        }
                        const int tk = g * kGR + cb * 8 + tid * 2;  // routes of this lane's columns
                        const int2 bias = *reinterpret_cast<const int2*>(s_bias + tk);
                        const float2 asv = *reinterpret_cast<const float2*>(s_as + tk);
                        // two chains of two instructions (latency), joined by one add
                        int c[4] = {bias.x, bias.y, bias.x, bias.y}, c2[4] = {0, 0, 0, 0};
                        moe_mma_16x8x32(c, lo0[0], lo1[0], hi0[0], hi1[0], be.x, bo.x);
                        moe_mma_16x8x32(c2, lo0[1], lo1[1], hi0[1], hi1[1], be.y, bo.y);
                        moe_mma_16x8x32(c, lo0[2], lo1[2], hi0[2], hi1[2], be.z, bo.z);
                        moe_mma_16x8x32(c2, lo0[3], lo1[3], hi0[3], hi1[3], be.w, bo.w);
                        // c + c2 = 0x4B400000 + D: as a float 12582912 + D, exactly
                        acc[j][0] = __fmaf_rn(
                            __fsub_rn(__int_as_float(c[0] + c2[0]), 12582912.f),
                            __fmul_rn(ws0, asv.x), acc[j][0]);
                        acc[j][1] = __fmaf_rn(
                            __fsub_rn(__int_as_float(c[1] + c2[1]), 12582912.f),
                            __fmul_rn(ws0, asv.y), acc[j][1]);
                        acc[j][2] = __fmaf_rn(
                            __fsub_rn(__int_as_float(c[2] + c2[2]), 12582912.f),
                            __fmul_rn(ws1, asv.x), acc[j][2]);
                        acc[j][3] = __fmaf_rn(
                            __fsub_rn(__int_as_float(c[3] + c2[3]), 12582912.f),
                            __fmul_rn(ws1, asv.y), acc[j][3]);
                    }
                }
            }
            // out[route][n]: the eight lanes of a quarter-warp hold eight consecutive n
            const int n0 = (tl0 + t0) * 8 + gid, n1 = n0 + 8;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int cb = cb_lo + j;
                if (cb < cb_hi && cb < ncb) {
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int mi = cb * 8 + tid * 2 + cc;
                        if (mi < mc) {
                            float* o = a.out + (size_t)(base + mi) * a.n_e;
                            if (n0 < a.n_e)
                                o[n0] = acc[j][cc];
                            if (two && n1 < a.n_e)
                                o[n1] = acc[j][2 + cc];
                        }
                    }
                }
            }
        }
        __syncthreads();  // the staged rows are overwritten by the next pass
    }
}

size_t grouped_smem(int k, int groups, int tpc, bool scl16) {
    return (size_t)tpc * groups * 512 + (size_t)tpc * groups * 8 * (scl16 ? 2 : 4) +
           (size_t)kGR * (k + kRowPad) + 2 * sizeof(float) * kGR * groups * 4 + 8 + 16;
}

// `decode` (few tokens): the shared-memory variant, optionally with SwiGLU + quantiser fused
// into its prologue (fused_gate_up = the gate_up matmul's fp32 output).
// qa32 / as32: the same rows quantised per 32 values, for experts that hold several routes
// (null: per-128 for all); as_stride / as32_stride: floats per row of as / as32.
int launch_grouped(b2w4_ctx* ctx, const b2w4_weight* w, int num_experts_all, int expert_begin,
                   int expert_count, int routes, const int8_t* qa, const float* as,
                   int as_stride, const int8_t* qa32, const float* as32, int as32_stride,
                   const int4* slots, const int32_t* row_map, float* out, bool decode,
                   const float* fused_gate_up = nullptr, const b2w4_tp_args* peers = nullptr,
                   int stage_rows = 0) {
    const int n_e = w->n / expert_count;
    const bool scl16 = w->scales_fp16 != 0;
    const int slots_y = routes < num_experts_all ? routes : num_experts_all;  // grid.y
    if (decode) {
        GroupedSmallArgs a = {};
        a.nib = reinterpret_cast<const uint8_t*>(w->nib);
        a.scl = w->scl;
        a.qa = qa;
        a.as = as;
        a.slots = slots;
        a.gate_up = fused_gate_up;
        a.num_experts_all = num_experts_all;
        a.expert_begin = expert_begin;
        a.expert_count = expert_count;
        a.row_map = row_map;
        a.out = out;
        a.status = ctx->status_dev;
        if (peers) {
            a.peers = *peers;
            a.stage_rows = stage_rows;
        }
        a.k = w->k;
        a.groups = w->groups;
        a.n_e = n_e;
        a.tiles_e = n_e / 8;
        int tpc = 16;
        while (tpc > 2 && grouped_small_smem(w->k, w->groups, tpc, scl16) > 113 * 1024)
            tpc -= 2;  // even: tiles are taken in pairs
        a.tpc = tpc;
        a.d_stride = grouped_small_d_stride(w->groups);
        const size_t smem = grouped_small_smem(w->k, w->groups, tpc, scl16);
        if (smem > 220 * 1024)
            return b2w4_fail(ctx, B2W4_E_INVALID, "moe: K=%d needs %zu B shared memory", w->k,
                             smem);
        auto kern = scl16 ? moe_grouped_small_kernel<true> : moe_grouped_small_kernel<false>;
        static b2w4_smem_optin configured[2];  // per instantiation and device
        B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, kern, smem, configured[scl16]));
        dim3 grid((a.tiles_e + tpc - 1) / tpc, slots_y);
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, kern, grid, dim3(kST), smem, ctx->stream, a));
        ctx->launches++;
        return B2W4_OK;
    }
    GroupedArgs a = {};
    a.nib = reinterpret_cast<const uint8_t*>(w->nib);
    a.scl = w->scl;
    a.qa = qa;
    a.as = as;
    a.as_stride = as_stride;
    a.qa32 = qa32;
    a.as32 = as32;
    a.as32_stride = as32_stride;
    a.slots = slots;
    a.num_experts_all = num_experts_all;
    a.expert_begin = expert_begin;
    a.expert_count = expert_count;
    a.row_map = row_map;
    a.out = out;
    a.status = ctx->status_dev;
    a.k = w->k;
    a.groups = w->groups;
    a.n_e = n_e;
    a.tiles_e = n_e / 8;
    int tpc = 16;
    while (tpc > 2 && grouped_smem(w->k, w->groups, tpc, scl16) > 113 * 1024)
        tpc -= 2;  // even: tiles are taken in pairs
    a.tpc = tpc;
    const size_t smem = grouped_smem(w->k, w->groups, tpc, scl16);
    if (smem > 220 * 1024)
        return b2w4_fail(ctx, B2W4_E_INVALID, "moe: K=%d needs %zu B shared memory", w->k, smem);
    auto kern = scl16 ? moe_grouped_gemv_kernel<true> : moe_grouped_gemv_kernel<false>;
    static b2w4_smem_optin configured[2];  // per instantiation and device
    B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, kern, smem, configured[scl16]));
    dim3 grid((a.tiles_e + tpc - 1) / tpc, slots_y);
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, kern, grid, dim3(kGT), smem, ctx->stream, a));
    ctx->launches++;
    return B2W4_OK;
}

}  // namespace

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

extern "C" {

int b2w4_moe_select_routes(b2w4_ctx* ctx, const float* logits_dev, int tokens,
                           int num_experts, int top_k, int32_t* indices_dev,
                           float* weights_dev) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!logits_dev || !indices_dev || !weights_dev || tokens <= 0 || num_experts <= 0 ||
        top_k <= 0 || top_k > num_experts || top_k > kMaxTopK ||
        num_experts > kSelectMaxExperts)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "select_routes: need 0 < top_k <= min(experts, %d), experts <= %d "
                         "(tokens=%d experts=%d top_k=%d)", kMaxTopK, kSelectMaxExperts, tokens,
                         num_experts, top_k);
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_select_routes_kernel, dim3((tokens + 3) / 4),
                                       dim3(128), 0, ctx->stream, logits_dev, tokens,
                                       num_experts, top_k, indices_dev, weights_dev));
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}

}  // extern "C"

// The whole MoE op.  With route_out == nullptr it computes every expert and combines into
// out_dev.  With route_out set it is one rank of an expert-parallel group: routing runs over
// all num_experts (replicated), the aggregates hold experts [expert_begin, expert_begin +
// expert_count) only, and the rank's route outputs go to route_out in (token, route) order.
static int moe_run(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens, int hidden_size,
                   const void* router_fp16_dev, int num_experts, int top_k, int intermediate,
                   const b2w4_weight* gate_up, const b2w4_weight* down, int expert_begin,
                   int expert_count, float* out_dev, int ldo, float* route_out,
                   float* logits_dev, int32_t* indices_dev, float* weights_dev,
                   const b2w4_tp_args* peers = nullptr, int stage_rows = 0) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!hidden_dev || !router_fp16_dev || !gate_up || !down || (!out_dev && !route_out))
        return b2w4_fail(ctx, B2W4_E_INVALID, "moe: null argument");
    if (tokens <= 0 || num_experts <= 0 || num_experts > kSelectMaxExperts || top_k <= 0 ||
        top_k > num_experts || top_k > kMaxTopK || hidden_size % 128 || intermediate % 128 || ldx < hidden_size ||
        (out_dev && ldo < hidden_size))
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "moe: bad shape tokens=%d hidden=%d experts=%d top_k=%d inter=%d",
                         tokens, hidden_size, num_experts, top_k, intermediate);
    if (expert_begin < 0 || expert_count <= 0 || expert_begin + expert_count > num_experts)
        return b2w4_fail(ctx, B2W4_E_INVALID, "moe: experts [%d, %d) outside [0, %d)",
                         expert_begin, expert_begin + expert_count, num_experts);
    if (gate_up->k != hidden_size || gate_up->n != expert_count * 2 * intermediate ||
        down->k != intermediate || down->n != expert_count * hidden_size)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "moe: expert aggregates must be gate_up [E*2I, H] and down [E*H, I] "
                         "for the %d experts held", expert_count);
    const int routes = tokens * top_k;
    const int gh = hidden_size / 128, gi = intermediate / 128;
    // small routing state in one block
    const size_t o_logits = 0;
    const size_t o_idx = align_up(o_logits + sizeof(float) * tokens * num_experts, 256);
    const size_t o_w = align_up(o_idx + sizeof(int32_t) * routes, 256);
    const size_t o_off = align_up(o_w + sizeof(float) * routes, 256);
    const size_t o_rt = align_up(o_off + sizeof(int32_t) * (num_experts + 1), 256);
    const size_t o_pos = align_up(o_rt + sizeof(int32_t) * routes, 256);
    const size_t o_act = align_up(o_pos + sizeof(int32_t) * routes, 256);
    const size_t small_bytes = align_up(o_act + sizeof(int4) * num_experts, 256);
    // quantised hidden (per token) and quantised SwiGLU output (per route)
    // The reference's rule (ctx->moe_rule == B2W4_ACT_G32): an expert that holds several routes
    // quantises per 32 values, a lone route per 128; with one token every expert holds one
    // route.  B2W4_ACT_G128: per 128 for every route.
    const bool rule32 = ctx->moe_rule == B2W4_ACT_G32 && tokens >= 2;
    const size_t o_qh = 0;
    const size_t o_ash = align_up(o_qh + (size_t)tokens * hidden_size, 256);
    const size_t o_qi = align_up(o_ash + sizeof(float) * tokens * gh, 256);
    const size_t o_asi = align_up(o_qi + (size_t)routes * intermediate, 256);
    const size_t o_qh32 = align_up(o_asi + sizeof(float) * routes * gi * 4, 256);
    const size_t o_ash32 = align_up(o_qh32 + (rule32 ? (size_t)tokens * hidden_size : 0), 256);
    const size_t quant_bytes =
        align_up(o_ash32 + (rule32 ? sizeof(float) * tokens * gh * 4 : 0), 256);
    void *sm = nullptr, *qb = nullptr, *gu = nullptr, *dn = nullptr;
    int rc;
    if ((rc = b2w4_reserve(ctx, SCR_MOE_A, small_bytes, &sm)) != B2W4_OK ||
        (rc = b2w4_reserve(ctx, SCR_MOE_B, quant_bytes, &qb)) != B2W4_OK ||
        (rc = b2w4_reserve(ctx, SCR_MOE_C, sizeof(float) * (size_t)routes * 2 * intermediate,
                           &gu)) != B2W4_OK ||
        (rc = b2w4_reserve(ctx, SCR_MOE_D, sizeof(float) * (size_t)routes * hidden_size,
                           &dn)) != B2W4_OK)
        return rc;
    uint8_t* smb = static_cast<uint8_t*>(sm);
    uint8_t* qbb = static_cast<uint8_t*>(qb);
    float* logits = reinterpret_cast<float*>(smb + o_logits);
    int32_t* idx = reinterpret_cast<int32_t*>(smb + o_idx);
    float* wts = reinterpret_cast<float*>(smb + o_w);
    int32_t* offsets = reinterpret_cast<int32_t*>(smb + o_off);
    int32_t* route_token = reinterpret_cast<int32_t*>(smb + o_rt);
    int32_t* pos = reinterpret_cast<int32_t*>(smb + o_pos);
    int4* slots = reinterpret_cast<int4*>(smb + o_act);
    int8_t* q_hidden = reinterpret_cast<int8_t*>(qbb + o_qh);
    float* as_hidden = reinterpret_cast<float*>(qbb + o_ash);
    int8_t* q_inter = reinterpret_cast<int8_t*>(qbb + o_qi);
    float* as_inter = reinterpret_cast<float*>(qbb + o_asi);  // [routes][4 * gi]
    int8_t* q_hidden32 = rule32 ? reinterpret_cast<int8_t*>(qbb + o_qh32) : nullptr;
    float* as_hidden32 = rule32 ? reinterpret_cast<float*>(qbb + o_ash32) : nullptr;
    cudaStream_t st = ctx->stream;

    const __half* router = static_cast<const __half*>(router_fp16_dev);
    const bool aligned =
        (reinterpret_cast<uintptr_t>(hidden_dev) | reinterpret_cast<uintptr_t>(router)) % 16 == 0 &&
        ldx % 4 == 0;
    const bool fused = aligned && tokens <= kFusedTokens && routes <= kFusedRoutes;
    if (fused) {
        // enough blocks to spread the router rows over the SMs, one warp per expert
        const int blocks = (num_experts + kFusedThreads / 32 - 1) / (kFusedThreads / 32);
        B2W4_CUDA(ctx, b2w4_launch_chained(
                           ctx->pdl, moe_route_fused_kernel, dim3(blocks), dim3(kFusedThreads),
                           sizeof(int) * (num_experts + 1), st, hidden_dev, ldx, tokens,
                           hidden_size, router, num_experts, top_k, logits, idx, wts, offsets,
                           route_token, pos, slots, q_hidden, as_hidden, ctx->flag_dev + 4));
        ctx->launches++;
    } else {
        if (!aligned) {
            const long long threads = (long long)tokens * num_experts * 32;
            B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_router_logits_scalar_kernel,
                                               dim3((int)((threads + 255) / 256)), dim3(256), 0, st,
                                               hidden_dev, ldx, tokens, hidden_size, router,
                                               num_experts, logits));
        } else if (tokens <= 8) {  // decode: one expert per warp keeps every SM busy
            const long long warps = (long long)((tokens + kRouterTok - 1) / kRouterTok) * num_experts;
            B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_router_logits_kernel<1>,
                                               dim3((int)((warps * 32 + 127) / 128)), dim3(128), 0, st,
                                               hidden_dev, ldx, tokens, hidden_size, router,
                                               num_experts, logits));
        } else {
            const long long warps =
                (long long)((tokens + kRouterTok - 1) / kRouterTok) * ((num_experts + 3) / 4);
            B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_router_logits_kernel<4>,
                                               dim3((int)((warps * 32 + 127) / 128)), dim3(128), 0, st,
                                               hidden_dev, ldx, tokens, hidden_size, router,
                                               num_experts, logits));
        }
        ctx->launches++;
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_select_routes_kernel, dim3((tokens + 3) / 4),
                                           dim3(128), 0, st, logits, tokens, num_experts, top_k, idx,
                                           wts));
        ctx->launches++;
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_compact_kernel, dim3(1),
                                           dim3(kCompactThreads), compact_smem(num_experts), st, idx,
                                           tokens, top_k, num_experts, offsets, route_token, pos,
                                           slots));
        ctx->launches++;
        B2W4_CUDA(ctx, cudaGetLastError());
        if ((rc = b2w4_launch_quantize(ctx, hidden_dev, ldx, tokens, hidden_size, B2W4_ACT_G128,
                                       q_hidden, as_hidden, QLAYOUT_MMA)) != B2W4_OK)
            return rc;
    }
    if (rule32 && (rc = b2w4_launch_quantize(ctx, hidden_dev, ldx, tokens, hidden_size,
                                             B2W4_ACT_G32, q_hidden32, as_hidden32,
                                             QLAYOUT_MMA)) != B2W4_OK)
        return rc;
    // which grouped-matmul variant: the few-token one implements the per-128 rule only
    const bool decode = rule32 ? false : tokens <= kFusedSwigluTokens;
    // compact positions stay global; the grouped kernels skip experts held elsewhere
    const int32_t* local_offsets = offsets + expert_begin;
    const bool partial = expert_count != num_experts;
    if ((rc = launch_grouped(ctx, gate_up, num_experts, expert_begin, expert_count, routes,
                             q_hidden, as_hidden, gh, q_hidden32, as_hidden32, gh * 4, slots,
                             route_token, static_cast<float*>(gu), decode)) != B2W4_OK)
        return rc;
    // few routes: SwiGLU and its quantiser run inside the down-projection's CTAs
    const bool fuse_swiglu = decode;
    if (!fuse_swiglu) {
        const long long threads = (long long)routes * gi * 32;
        B2W4_CUDA(ctx, b2w4_launch_chained(
                           ctx->pdl, moe_swiglu_quant_kernel, dim3((int)((threads + 255) / 256)),
                           dim3(256), 0, st, static_cast<const float*>(gu), routes, intermediate,
                           q_inter, as_inter, gi * 4,
                           rule32 ? static_cast<const int32_t*>(offsets) : nullptr, num_experts,
                           partial ? local_offsets : nullptr,
                           partial ? local_offsets + expert_count : nullptr));
        ctx->launches++;
    }
    // decode steps hand the rows over from the down-projection's own epilogue
    const bool fused_handover = peers != nullptr && decode;
    // a route's SwiGLU row was quantised by its own expert's rule: one code buffer serves both
    if ((rc = launch_grouped(ctx, down, num_experts, expert_begin, expert_count, routes, q_inter,
                             as_inter, gi * 4, rule32 ? q_inter : nullptr,
                             rule32 ? as_inter : nullptr, gi * 4, slots, nullptr,
                             static_cast<float*>(dn), decode,
                             fuse_swiglu ? static_cast<const float*>(gu) : nullptr,
                             fused_handover ? peers : nullptr, stage_rows)) != B2W4_OK)
        return rc;
    if (route_out) {
        dim3 grid((hidden_size / 4 + 255) / 256, routes);
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_scatter_routes_kernel, grid, dim3(256), 0,
                                           st, static_cast<const float*>(dn), idx, pos, routes,
                                           hidden_size, expert_begin, expert_count, route_out));
        ctx->launches++;
    }
    if (peers) {
        if (!fused_handover) {
            dim3 sgrid((hidden_size / 4 + 255) / 256, routes);
            B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_scatter_routes_peers_kernel, sgrid,
                                               dim3(256), 0, st, static_cast<const float*>(dn),
                                               idx, pos, routes, hidden_size, expert_begin,
                                               expert_count, stage_rows, *peers));
            ctx->launches++;
        }
        dim3 cgrid((hidden_size / 4 + kCombineThreads - 1) / kCombineThreads, tokens);
        B2W4_CUDA(ctx, b2w4_launch_chained(
                           ctx->pdl, moe_combine_staged_kernel, cgrid, dim3(kCombineThreads), 0, st,
                           peers->stage_peer[peers->rank], stage_rows, idx, wts,
                           fused_handover ? static_cast<const int32_t*>(pos) : nullptr, tokens,
                           top_k, hidden_size, out_dev, ldo,
                           reinterpret_cast<unsigned*>(ctx->flag_dev + 6), ctx->status_dev,
                           ctx->peer_wait_cycles));
        ctx->launches++;
    } else if (out_dev) {
        dim3 grid((hidden_size / 4 + kCombineThreads - 1) / kCombineThreads, tokens);
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_combine_kernel, grid,
                                           dim3(kCombineThreads), 0, st,
                                           static_cast<const float*>(dn), idx, wts, pos, tokens,
                                           top_k, hidden_size, out_dev, ldo));
        ctx->launches++;
    }
    B2W4_CUDA(ctx, cudaGetLastError());
    if (logits_dev)
        B2W4_CUDA(ctx, cudaMemcpyAsync(logits_dev, logits,
                                       sizeof(float) * (size_t)tokens * num_experts,
                                       cudaMemcpyDeviceToDevice, st));
    if (indices_dev)
        B2W4_CUDA(ctx, cudaMemcpyAsync(indices_dev, idx, sizeof(int32_t) * (size_t)routes,
                                       cudaMemcpyDeviceToDevice, st));
    if (weights_dev)
        B2W4_CUDA(ctx, cudaMemcpyAsync(weights_dev, wts, sizeof(float) * (size_t)routes,
                                       cudaMemcpyDeviceToDevice, st));
    return B2W4_OK;
}

extern "C" {

int b2w4_moe_forward(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens,
                     int hidden_size, const void* router_fp16_dev, int num_experts, int top_k,
                     int intermediate, const b2w4_weight* gate_up, const b2w4_weight* down,
                     float* out_dev, int ldo, float* logits_dev, int32_t* indices_dev,
                     float* weights_dev) {
    if (ctx && !out_dev)
        return b2w4_fail(ctx, B2W4_E_INVALID, "moe: null argument");
    return moe_run(ctx, hidden_dev, ldx, tokens, hidden_size, router_fp16_dev, num_experts,
                   top_k, intermediate, gate_up, down, 0, num_experts, out_dev, ldo, nullptr,
                   logits_dev, indices_dev, weights_dev);
}

int b2w4_moe_expert_outputs(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens,
                            int hidden_size, const void* router_fp16_dev, int num_experts,
                            int top_k, int intermediate, const b2w4_weight* gate_up_local,
                            const b2w4_weight* down_local, int expert_begin, int expert_count,
                            float* route_out_dev, int32_t* indices_dev, float* weights_dev) {
    if (ctx && (!route_out_dev || !indices_dev || !weights_dev))
        return b2w4_fail(ctx, B2W4_E_INVALID, "moe: null argument");
    return moe_run(ctx, hidden_dev, ldx, tokens, hidden_size, router_fp16_dev, num_experts,
                   top_k, intermediate, gate_up_local, down_local, expert_begin, expert_count,
                   nullptr, 0, route_out_dev, nullptr, indices_dev, weights_dev);
}

int b2w4_moe_forward_ep(b2w4_ctx* ctx, const float* hidden_dev, int ldx, int tokens,
                        int hidden_size, const void* router_fp16_dev, int num_experts, int top_k,
                        int intermediate, const b2w4_weight* gate_up_local,
                        const b2w4_weight* down_local, int expert_begin, int expert_count,
                        const b2w4_tp_group* group, int stage_rows, float* out_dev, int ldo,
                        int32_t* indices_dev, float* weights_dev) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!out_dev || !group || group->world < 1 || group->world > kTpMaxWorld ||
        group->rank < 0 || group->rank >= group->world || tokens <= 0 || top_k <= 0 ||
        stage_rows < tokens * top_k)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "moe_forward_ep: bad group, or fewer staging rows than routes");
    b2w4_tp_args peers = {};
    for (int p = 0; p < group->world; ++p) {
        if (!group->stage_peers[p] || (reinterpret_cast<uintptr_t>(group->stage_peers[p]) & 15))
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "moe_forward_ep: null peer pointer, or not 16-byte aligned");
        peers.stage_peer[p] = static_cast<unsigned long long*>(group->stage_peers[p]);
    }
    peers.world = group->world;
    peers.rank = group->rank;
    return moe_run(ctx, hidden_dev, ldx, tokens, hidden_size, router_fp16_dev, num_experts,
                   top_k, intermediate, gate_up_local, down_local, expert_begin, expert_count,
                   out_dev, ldo, nullptr, nullptr, indices_dev, weights_dev, &peers, stage_rows);
}

int b2w4_moe_combine(b2w4_ctx* ctx, const float* route_out_dev, int tokens, int hidden_size,
                     int top_k, const int32_t* indices_dev, const float* weights_dev,
                     float* out_dev, int ldo) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!route_out_dev || !indices_dev || !weights_dev || !out_dev || tokens <= 0 ||
        hidden_size <= 0 || hidden_size % 4 || top_k <= 0 || top_k > kMaxTopK ||
        ldo < hidden_size || reinterpret_cast<uintptr_t>(route_out_dev) % 16)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "moe_combine: bad argument (hidden a multiple of 4, route rows "
                         "16-byte aligned)");
    dim3 grid((hidden_size / 4 + kCombineThreads - 1) / kCombineThreads, tokens);
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, moe_combine_kernel, grid, dim3(kCombineThreads),
                                       0, ctx->stream, route_out_dev, indices_dev, weights_dev,
                                       static_cast<const int32_t*>(nullptr), tokens, top_k,
                                       hidden_size, out_dev, ldo));
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}

}  // extern "C"
