// The operators that sit between the W4G128 matmuls of a decoder layer, as device kernels, so
// that a decode step needs no trip to the host between its matmuls: RMSNorm, residual add +
// RMSNorm, SwiGLU, add / multiply, rotary embedding, KV-cache append, scaled-dot-product
// attention over the cache, embedding-row lookup.  Semantics follow the reference's CPU
// operators (the x86 build: its scalar and AVX-512 paths), cited per kernel.  Sums over a row
// are tree reductions here where the reference's scalar loops are sequential, so these ops
// agree with the reference to fp32 rounding of a reassociated sum, not bit for bit; everything
// that is element-wise (rotary embedding, add, multiply, the P*V accumulation in key order)
// uses the reference's operation order with no contraction.
// All tensors are fp32, rows = tokens, features contiguous.
#include "b200w4_internal.cuh"

namespace {

constexpr int kNormThreads = 256;
constexpr int kAttnMaxDim = 256;  // widest attention head

__device__ __forceinline__ float block_sum(float v, float* s_part) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // s_part may still be read from a previous call
    if (lane == 0)
        s_part[warp] = v;
    __syncthreads();
    float t = 0.f;
    const int warps = (blockDim.x + 31) >> 5;
    for (int w = 0; w < warps; ++w)  // every thread adds in the same order
        t = __fadd_rn(t, s_part[w]);
    return t;
}

__device__ __forceinline__ float block_max(float v, float* s_part) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0)
        s_part[warp] = v;
    __syncthreads();
    float t = s_part[0];
    const int warps = (blockDim.x + 31) >> 5;
    for (int w = 1; w < warps; ++w)
        t = fmaxf(t, s_part[w]);
    return t;
}

// kernel_rms_norm (kernels/norm.cpp:13-31, :95-121): r = 1/sqrt(sum(x^2)/D + eps),
// out = (x * r) * w.  With `update`: kernel_add_rms_norm (:123-190): the sum x + update is
// written back into x (the residual stream) first.  One block per row.
__global__ void __launch_bounds__(kNormThreads)
rms_norm_kernel(float* __restrict__ x, int ldx, const float* __restrict__ update, int ldu,
                int dim, const float* __restrict__ weight, float eps, float* __restrict__ out,
                int ldo) {
    b2w4_pdl_chain_entry();
    __shared__ float s_part[kNormThreads / 32];
    float* xr = x + (size_t)blockIdx.x * ldx;
    const float* ur = update ? update + (size_t)blockIdx.x * ldu : nullptr;
    float* orow = out + (size_t)blockIdx.x * ldo;
    // up to kNormHeld values per thread stay in registers between the two passes, all their
    // loads in flight together; longer rows re-read the row
    constexpr int kNormHeld = 16;
    float ss = 0.f;
    if (dim <= kNormHeld * kNormThreads) {
        float v[kNormHeld], w[kNormHeld];
#pragma unroll
        for (int u = 0; u < kNormHeld; ++u) {
            const int d = threadIdx.x + kNormThreads * u;
            v[u] = d < dim ? xr[d] : 0.f;
            w[u] = d < dim ? weight[d] : 0.f;
        }
        if (ur) {
#pragma unroll
            for (int u = 0; u < kNormHeld; ++u) {
                const int d = threadIdx.x + kNormThreads * u;
                if (d < dim) {
                    v[u] = __fadd_rn(v[u], ur[d]);
                    xr[d] = v[u];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kNormHeld; ++u)  // the same per-thread order as the strided loop
            if (threadIdx.x + kNormThreads * u < dim)
                ss = __fadd_rn(ss, __fmul_rn(v[u], v[u]));
        ss = block_sum(ss, s_part);
        const float r = __fdiv_rn(1.f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
#pragma unroll
        for (int u = 0; u < kNormHeld; ++u) {
            const int d = threadIdx.x + kNormThreads * u;
            if (d < dim)
                orow[d] = __fmul_rn(__fmul_rn(v[u], r), w[u]);
        }
        return;
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float v = xr[d];
        if (ur) {
            v = __fadd_rn(v, ur[d]);
            xr[d] = v;
        }
        ss = __fadd_rn(ss, __fmul_rn(v, v));
    }
    ss = block_sum(ss, s_part);
    const float r = __fdiv_rn(1.f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
        orow[d] = __fmul_rn(__fmul_rn(xr[d], r), weight[d]);
}

// Small rows (the per-head Q/K norm: 128 values): one warp per row.
__global__ void rms_norm_warp_kernel(const float* __restrict__ x, int ldx, int rows, int dim,
                                     const float* __restrict__ weight, float eps,
                                     float* __restrict__ out, int ldo) {
    b2w4_pdl_chain_entry();
    const int row = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows)
        return;
    const float* xr = x + (size_t)row * ldx;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32)
        ss = __fadd_rn(ss, __fmul_rn(xr[d], xr[d]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
    const float r = __fdiv_rn(1.f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    float* orow = out + (size_t)row * ldo;
    for (int d = lane; d < dim; d += 32)
        orow[d] = __fmul_rn(__fmul_rn(xr[d], r), weight[d]);
}

// SWIGLU of kernel_elementwise (kernels/elementwise.cpp:529-570): a merged row [2I] holds gate
// = [0, I) and up = [I, 2I); out[i] = (g / (1 + exp(-g))) * up[i] -- a division, unlike the
// MoE op's and the matmul epilogue's g * (1 / (1 + exp(-g))).
__global__ void swiglu_kernel(const float* __restrict__ merged, int ldm, int rows, int inter,
                              float* __restrict__ out, int ldo) {
    b2w4_pdl_chain_entry();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * inter)
        return;
    const int r = (int)(i / inter), c = (int)(i - (size_t)r * inter);
    const float g = merged[(size_t)r * ldm + c];
    const float u = merged[(size_t)r * ldm + inter + c];
    const float e = (float)exp(-(double)g);  // in double, rounded once
    out[(size_t)r * ldo + c] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.f, e)), u);
}

__global__ void binary_kernel(const float* __restrict__ a, const float* __restrict__ b,
                              float* __restrict__ out, size_t count, int multiply) {
    b2w4_pdl_chain_entry();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count)
        out[i] = multiply ? __fmul_rn(a[i], b[i]) : __fadd_rn(a[i], b[i]);
}

// kernel_rope, halves form (kernels/rope.cpp:11-50, interleave == false as the Qwen3 graphs
// use it, models/qwen3.py:332-333): out[i] = x0*c - x1*s, out[i+half] = x0*s + x1*c with
// x0 = x[i], x1 = x[i+half]; features beyond rope_dim are copied.  x: [tokens][heads][dim],
// cos / sin: tables [positions][rope_dim/2]; token t uses row pos0 + t, or *pos_dev + t when
// the position lives on the device (a decode step captured once in a CUDA graph and replayed
// for every position).  In place when out == x.
__global__ void rope_kernel(const float* __restrict__ x, float* __restrict__ out, int tokens,
                            int heads, int dim, const float* __restrict__ cosv,
                            const float* __restrict__ sinv, int rope_dim, int pos0,
                            const int* __restrict__ pos_dev) {
    b2w4_pdl_chain_entry();
    const int half = rope_dim >> 1;
    const int pos = pos_dev ? *pos_dev : pos0;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t per_row = (size_t)half + (size_t)(dim - rope_dim);
    if (i >= (size_t)tokens * heads * per_row)
        return;
    const size_t rowi = i / per_row;
    const int j = (int)(i - rowi * per_row);
    const int t = pos + (int)(rowi / heads);
    const float* xr = x + rowi * dim;
    float* orow = out + rowi * dim;
    if (j < half) {
        const float x0 = xr[j], x1 = xr[j + half];
        const float c = cosv[(size_t)t * half + j], s = sinv[(size_t)t * half + j];
        orow[j] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        orow[j + half] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    } else {
        orow[rope_dim + (j - half)] = xr[rope_dim + (j - half)];
    }
}

// KV-cache append: the new tokens' keys and values [tokens][kv_heads][dim] go to positions
// past .. past+tokens-1 of a cache laid out [kv_head][capacity][dim], the layout of the
// reference's cache after its header (kernels/attention.cpp:1043-1057).
__global__ void kv_append_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                 float* __restrict__ k_cache, float* __restrict__ v_cache,
                                 int tokens, int kv_heads, int dim, int past0,
                                 const int* __restrict__ past_dev, int capacity) {
    b2w4_pdl_chain_entry();
    const int past = past_dev ? min(*past_dev, capacity - tokens) : past0;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)tokens * kv_heads * dim)
        return;
    const int d = (int)(i % dim);
    const int h = (int)((i / dim) % kv_heads);
    const int t = (int)(i / ((size_t)dim * kv_heads));
    const size_t dst = ((size_t)h * capacity + past + t) * dim + d;
    k_cache[dst] = k[i];
    v_cache[dst] = v[i];
}

// The step between the fused qkv matmul and attention in one launch (the reference's CUDA
// backend fuses Q/K norm and rotary embedding the same way, engine/cuda_attention.cu:8-55):
// per (token, head) row of the merged qkv output -- a warp each -- the Q and K rows get the
// per-head RMSNorm (weights optional) and the rotary embedding, with exactly the operations of
// rms_norm_warp_kernel and rope_kernel in their order, Q goes to q_out [tokens][heads][dim],
// K and V go straight to their cache rows.  Needs rope over the whole head and dim / 2 a
// multiple of 32, so that both halves of a rotary pair sit in one lane.
__global__ void qkv_prepare_kernel(const float* __restrict__ qkv, int ld, int tokens, int heads,
                                   int kv_heads, int dim, const float* __restrict__ q_weight,
                                   const float* __restrict__ k_weight, float eps,
                                   const float* __restrict__ cosv, const float* __restrict__ sinv,
                                   int pos0, const int* __restrict__ pos_dev,
                                   float* __restrict__ q_out, float* __restrict__ k_cache,
                                   float* __restrict__ v_cache, int capacity) {
    b2w4_pdl_chain_entry();
    const int slots = heads + 2 * kv_heads;
    const size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= (size_t)tokens * slots)
        return;
    const int pos = pos_dev ? min(*pos_dev, capacity - tokens) : pos0;
    const int t = (int)(row / slots), slot = (int)(row % slots);
    const float* xr = qkv + (size_t)t * ld + (size_t)slot * dim;
    constexpr int kPer = kAttnMaxDim / 32;
    float v[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i)
        v[i] = lane + 32 * i < dim ? xr[lane + 32 * i] : 0.f;
    if (slot >= heads + kv_heads) {  // a value row: copied to its cache row
        float* dst = v_cache + ((size_t)(slot - heads - kv_heads) * capacity + pos + t) * dim;
#pragma unroll
        for (int i = 0; i < kPer; ++i)
            if (lane + 32 * i < dim)
                dst[lane + 32 * i] = v[i];
        return;
    }
    const bool is_q = slot < heads;
    const float* w = is_q ? q_weight : k_weight;
    if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kPer; ++i)
            if (lane + 32 * i < dim)
                ss = __fadd_rn(ss, __fmul_rn(v[i], v[i]));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
        const float r = __fdiv_rn(1.f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
#pragma unroll
        for (int i = 0; i < kPer; ++i)
            if (lane + 32 * i < dim)
                v[i] = __fmul_rn(__fmul_rn(v[i], r), w[lane + 32 * i]);
    }
    const int half = dim >> 1, hi = half >> 5;  // v[i] pairs with v[i + hi]
    float* dst = is_q ? q_out + ((size_t)t * heads + slot) * dim
                      : k_cache + ((size_t)(slot - heads) * capacity + pos + t) * dim;
#pragma unroll
    for (int i = 0; i < kPer / 2; ++i) {
        if (i < hi) {
            const int j = lane + 32 * i;
            const float c = cosv[(size_t)(pos + t) * half + j];
            const float sn = sinv[(size_t)(pos + t) * half + j];
            float x0 = 0.f, x1 = 0.f;
#pragma unroll
            for (int u = 0; u < kPer; ++u) {  // register picks with compile-time indices
                if (u == i)
                    x0 = v[u];
                if (u == i + hi)
                    x1 = v[u];
            }
            dst[j] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
            dst[j + half] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
        }
    }
}

// Scaled-dot-product attention of one (query token, head) over the cache, the x86 reference's
// arithmetic (kernels/attention_x86_avx512.cpp:47-109): scores = dot(q, k_j) * scale for the
// visible keys (causal: keys 0 .. past + t), full-row softmax (max, exp, sum, times 1/sum),
// then out = sum_j p_j * v_j accumulated key by key in ascending order with one fused
// multiply-add per key and feature, as the reference's loop does.  One block per (token,
// head).  Scores: a warp per key, four keys' loads in flight at a time.  P*V: thread d owns
// output feature d and walks the keys in order; the value rows come through shared memory in
// chunks that all threads fetch together, the next chunk's loads in flight while the current
// one is consumed, so that the ordered sum does not wait on memory once per key.
constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnStage = 4096;                       // floats of V per chunk
constexpr int kAttnPerThread = kAttnStage / kAttnThreads;
__global__ void __launch_bounds__(kAttnThreads)
attention_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                 const float* __restrict__ v_cache, float* __restrict__ out, int tokens,
                 int heads, int kv_heads, int dim, int past0, const int* __restrict__ past_dev,
                 int capacity, float scale, int score_slots) {
    b2w4_pdl_chain_entry();
    const int past = past_dev ? min(*past_dev, capacity - tokens) : past0;
    extern __shared__ float s_dyn[];
    float* s_scores = s_dyn;                // [score_slots] >= visible keys
    float* s_stage = s_dyn + score_slots;   // [kAttnStage]
    __shared__ float s_part[kAttnWarps];
    const int t = blockIdx.x / heads, h = blockIdx.x % heads;
    const int kvh = h / (heads / kv_heads);
    const int visible = past + t + 1;
    const float* qr = q + ((size_t)t * heads + h) * dim;
    const float* kc = k_cache + (size_t)kvh * capacity * dim;
    const float* vc = v_cache + (size_t)kvh * capacity * dim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    constexpr int kQ = kAttnMaxDim / 32, kKeys = 4;
    float qv[kQ];
#pragma unroll
    for (int i = 0; i < kQ; ++i)
        qv[i] = lane + 32 * i < dim ? qr[lane + 32 * i] : 0.f;
    for (int j0 = warp * kKeys; j0 < visible; j0 += kAttnWarps * kKeys) {
        float kv[kKeys][kQ];
#pragma unroll
        for (int u = 0; u < kKeys; ++u)
#pragma unroll
            for (int i = 0; i < kQ; ++i)
                kv[u][i] = (j0 + u < visible && lane + 32 * i < dim)
                               ? kc[(size_t)(j0 + u) * dim + lane + 32 * i] : 0.f;
#pragma unroll
        for (int u = 0; u < kKeys; ++u) {
            float p = 0.f;
#pragma unroll
            for (int i = 0; i < kQ; ++i)
                if (32 * i < dim)  // lanes past the last feature add +0 products
                    p = __fmaf_rn(qv[i], kv[u][i], p);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                p = __fadd_rn(p, __shfl_xor_sync(0xffffffffu, p, off));
            if (lane == 0 && j0 + u < visible)
                s_scores[j0 + u] = __fmul_rn(p, scale);
        }
    }
    __syncthreads();
    float m = -INFINITY;
    for (int j = threadIdx.x; j < visible; j += blockDim.x)
        m = fmaxf(m, s_scores[j]);
    m = block_max(m, s_part);
    float sum = 0.f;
    for (int j = threadIdx.x; j < visible; j += blockDim.x) {
        const float e = (float)exp((double)__fsub_rn(s_scores[j], m));
        s_scores[j] = e;
        sum = __fadd_rn(sum, e);
    }
    sum = block_sum(sum, s_part);
    const float inv = __fdiv_rn(1.f, sum);

    const int chunk = kAttnStage / dim;  // keys per chunk
    float r[kAttnPerThread];
    auto fetch = [&](int j0) {
        const int n = min(chunk, visible - j0) * dim;
        const float* src = vc + (size_t)j0 * dim;
#pragma unroll
        for (int u = 0; u < kAttnPerThread; ++u) {
            const int i = threadIdx.x + kAttnThreads * u;
            r[u] = i < n ? src[i] : 0.f;
        }
    };
    fetch(0);
    float acc = 0.f;
    for (int j0 = 0; j0 < visible; j0 += chunk) {
        __syncthreads();  // the previous chunk has been consumed (and the scores are final)
#pragma unroll
        for (int u = 0; u < kAttnPerThread; ++u)
            s_stage[threadIdx.x + kAttnThreads * u] = r[u];
        __syncthreads();
        if (j0 + chunk < visible)
            fetch(j0 + chunk);
        if (threadIdx.x < dim) {
            const int nk = min(chunk, visible - j0);
            for (int j = 0; j < nk; ++j) {
                const float p = __fmul_rn(s_scores[j0 + j], inv);
                if (p != 0.f)
                    acc = __fmaf_rn(s_stage[j * dim + threadIdx.x], p, acc);
            }
        }
    }
    if (threadIdx.x < dim)
        out[((size_t)t * heads + h) * dim + threadIdx.x] = acc;
}

// The same attention for a run of new tokens (prefill): one block per (kv head, tile of query
// tokens) serves every query head of that kv head -- up to kTileRows (token, head) rows --
// so that a chunk of keys or values is fetched into shared memory once per tile instead of
// once per row.  Every row's arithmetic is attention_kernel's, operation for operation (the
// lanes' partial dot products and their xor-tree, the softmax sums per 256 strided partials,
// the ordered P*V), so both kernels give the same bits.
//   scores   warp w owns rows 4w .. 4w+3.  For eight keys at a time it forms the 32 partial
//            products (4 rows x 8 keys) per lane, then a butterfly exchange that halves the
//            items a lane holds at each of the xor-tree's five levels -- the same sums in the
//            same order as five shuffles per item, for one shuffle per item
//   softmax  per row by its warp; probabilities e_j / sum are stored back, zero past the
//            row's last visible key
//   P*V      thread (group, d): feature d of DIM/8 rows, keys in ascending order
constexpr int kTileRows = 32;
template <int DIM>
__global__ void __launch_bounds__(kAttnThreads)
attention_tile_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                      const float* __restrict__ v_cache, float* __restrict__ out, int tokens,
                      int heads, int kv_heads, int past0, const int* __restrict__ past_dev,
                      int capacity, float scale, int slots, int tq) {
    b2w4_pdl_chain_entry();
    const int past = past_dev ? min(*past_dev, capacity - tokens) : past0;
    extern __shared__ float s_dyn[];
    float* s_sc = s_dyn;                           // [kTileRows][slots]
    float* s_stage = s_dyn + kTileRows * slots;    // [kAttnStage]
    constexpr int kQ = DIM / 32;                   // features per lane
    constexpr int kChunk = kAttnStage / DIM;       // keys per staged chunk
    const int rep = heads / kv_heads;
    // the last tiles see the most keys: they go first
    const int kvh = blockIdx.y, t0 = (int)(gridDim.x - 1 - blockIdx.x) * tq;
    const int t_end = min(t0 + tq, tokens);
    const int vis_max = past + t_end;              // keys the tile's last token sees
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* kc = k_cache + (size_t)kvh * capacity * DIM;
    const float* vc = v_cache + (size_t)kvh * capacity * DIM;
    // row r of the tile: token t0 + r / rep, head kvh * rep + r % rep; rows past the tile's
    // tokens see no key
    auto row_token = [&](int r) { return t0 + r / rep; };
    auto row_visible = [&](int r) {
        return (r < tq * rep && row_token(r) < tokens) ? past + row_token(r) + 1 : 0;
    };

    float r[kAttnPerThread];
    auto fetch = [&](const float* base, int j0) {
        const int n = min(kChunk, vis_max - j0) * DIM;
        const float* src = base + (size_t)j0 * DIM;
#pragma unroll
        for (int u = 0; u < kAttnPerThread; ++u) {
            const int i = threadIdx.x + kAttnThreads * u;
            r[u] = i < n ? src[i] : 0.f;
        }
    };
    auto stage = [&]() {
        __syncthreads();  // the previous chunk has been consumed
#pragma unroll
        for (int u = 0; u < kAttnPerThread; ++u)
            s_stage[threadIdx.x + kAttnThreads * u] = r[u];
        __syncthreads();
    };

    // ---- scores ----
    float qv[4][kQ];
    int vis[4], vis_warp = 0;
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
        const int row = warp * 4 + rr;
        vis[rr] = row_visible(row);
        vis_warp = max(vis_warp, vis[rr]);
        const float* qr = q + ((size_t)row_token(row) * heads + kvh * rep + row % rep) * DIM;
#pragma unroll
        for (int i = 0; i < kQ; ++i)
            qv[rr][i] = vis[rr] ? qr[lane + 32 * i] : 0.f;
    }
    fetch(kc, 0);
    for (int j0 = 0; j0 < vis_max; j0 += kChunk) {
        stage();
        if (j0 + kChunk < vis_max)
            fetch(kc, j0 + kChunk);
        for (int sub = 0; sub < kChunk / 8 && j0 + sub * 8 < vis_warp; ++sub) {
            float v[32];  // item rr * 8 + kk: row rr of the warp, key kk of the eight
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                float kr[kQ];
#pragma unroll
                for (int i = 0; i < kQ; ++i)
                    kr[i] = s_stage[(sub * 8 + kk) * DIM + lane + 32 * i];
#pragma unroll
                for (int rr = 0; rr < 4; ++rr) {
                    float p = 0.f;
#pragma unroll
                    for (int i = 0; i < kQ; ++i)
                        p = __fmaf_rn(qv[rr][i], kr[i], p);
                    v[rr * 8 + kk] = p;
                }
            }
            // xor-tree levels 16, 8, 4, 2, 1; after level `off` a lane keeps the half of its
            // items selected by that bit of its index, so it ends with item `lane`
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const bool up = lane & off;
#pragma unroll
                for (int i = 0; i < off; ++i) {
                    const float send = up ? v[i] : v[i + off];
                    const float keep = up ? v[i + off] : v[i];
                    v[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, off));
                }
            }
            const int rr = lane >> 3, key = j0 + sub * 8 + (lane & 7);
            int my_vis = vis[0];
            my_vis = rr == 1 ? vis[1] : my_vis;
            my_vis = rr == 2 ? vis[2] : my_vis;
            my_vis = rr == 3 ? vis[3] : my_vis;
            if (key < my_vis)
                s_sc[(warp * 4 + rr) * slots + key] = __fmul_rn(v[0], scale);
        }
    }
    __syncwarp();

    // ---- softmax, a row at a time by the warp that owns it ----
#pragma unroll 1
    for (int rr = 0; rr < 4; ++rr) {
        float* sc = s_sc + (warp * 4 + rr) * slots;
        const int n = vis[rr];
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32)
            m = fmaxf(m, sc[j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        // the sum of attention_kernel: 256 partials of stride 256, a tree per 32 of them,
        // the eight results added in order
        float sum = 0.f;
#pragma unroll 1
        for (int w = 0; w < kAttnWarps; ++w) {
            float part = 0.f;
            for (int j = w * 32 + lane; j < n; j += kAttnThreads) {
                const float e = (float)exp((double)__fsub_rn(sc[j], m));
                sc[j] = e;
                part = __fadd_rn(part, e);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
            sum = __fadd_rn(sum, part);
        }
        const float inv = __fdiv_rn(1.f, sum);
        for (int j = lane; j < ((vis_max + 3) & ~3); j += 32)  // P*V reads four at a time
            sc[j] = j < n ? __fmul_rn(sc[j], inv) : 0.f;
    }

    // ---- P*V ----
    constexpr int kGroups = kAttnThreads / DIM, kRG = kTileRows / kGroups;
    const int grp = threadIdx.x / DIM, d = threadIdx.x % DIM;
    float acc[kRG];
#pragma unroll
    for (int i = 0; i < kRG; ++i)
        acc[i] = 0.f;
    fetch(vc, 0);
    for (int j0 = 0; j0 < vis_max; j0 += kChunk) {
        stage();  // its first barrier also orders the probabilities before their use
        if (j0 + kChunk < vis_max)
            fetch(vc, j0 + kChunk);
        const int nk = min(kChunk, vis_max - j0);
        const float* pr = s_sc + grp * kRG * slots + j0;
        // four keys at a time; a zero probability leaves the sum as it is (values are
        // finite), which is what attention_kernel's skip does
        for (int j = 0; j < nk; j += 4) {
            const float v0 = s_stage[j * DIM + d], v1 = s_stage[(j + 1) * DIM + d];
            const float v2 = s_stage[(j + 2) * DIM + d], v3 = s_stage[(j + 3) * DIM + d];
#pragma unroll
            for (int i = 0; i < kRG; ++i) {
                const float4 p = *reinterpret_cast<const float4*>(pr + i * slots + j);
                acc[i] = __fmaf_rn(v0, p.x, acc[i]);
                acc[i] = __fmaf_rn(v1, p.y, acc[i]);
                acc[i] = __fmaf_rn(v2, p.z, acc[i]);
                acc[i] = __fmaf_rn(v3, p.w, acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kRG; ++i) {
        const int row = grp * kRG + i;
        if (row_visible(row))
            out[((size_t)row_token(row) * heads + kvh * rep + row % rep) * DIM + d] = acc[i];
    }
}

// A position counter on the device: *counter += by (after a decode step of a replayed graph),
// and the step's token appended to a history so that the host may read all of them at the end.
__global__ void advance_kernel(int* counter, int by, const int32_t* token, int32_t* history,
                               int history_len) {
    b2w4_pdl_chain_entry();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int at = *counter;
        if (history && token && at >= 0 && at < history_len)
            history[at] = *token;
        *counter = at + by;
    }
}

// OpType::CONTIGUOUS for a block of rows (kernels/layout.cpp materialises a strided view the
// same way): dst[r][c] = src[r][c], each side with its own row stride.
__global__ void copy_rows_kernel(const float* __restrict__ src, int ld_src,
                                 float* __restrict__ dst, int ld_dst, int rows, int cols) {
    b2w4_pdl_chain_entry();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * cols)
        return;
    const int r = (int)(i / cols), c = (int)(i - (size_t)r * cols);
    dst[(size_t)r * ld_dst + c] = src[(size_t)r * ld_src + c];
}

// Embedding lookup: rows of an fp16 table widened to fp32 (the reference's EMBEDDING input
// path widens fp16 rows the same way, engine/engine.cpp:637-672 uploads "hidden").
__global__ void embed_rows_kernel(const __half* __restrict__ table, const int32_t* __restrict__ ids,
                                  int rows, int dim, float* __restrict__ out, int ldo) {
    b2w4_pdl_chain_entry();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * dim)
        return;
    const int r = (int)(i / dim), d = (int)(i - (size_t)r * dim);
    out[(size_t)r * ldo + d] = __half2float(table[(size_t)ids[r] * dim + d]);
}

}  // namespace

extern "C" {

int b2w4_rms_norm(b2w4_ctx* ctx, const float* x_dev, int ldx, int rows, int dim,
                  const float* weight_dev, float eps, float* out_dev, int ldo) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!x_dev || !weight_dev || !out_dev || rows <= 0 || dim <= 0 || ldx < dim || ldo < dim)
        return b2w4_fail(ctx, B2W4_E_INVALID, "rms_norm: bad argument");
    if (dim <= 256) {
        const size_t threads = (size_t)rows * 32;
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, rms_norm_warp_kernel,
                                           dim3((unsigned)((threads + 255) / 256)), dim3(256), 0,
                                           ctx->stream, x_dev, ldx, rows, dim, weight_dev, eps,
                                           out_dev, ldo));
    } else {
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, rms_norm_kernel, dim3(rows),
                                           dim3(kNormThreads), 0, ctx->stream,
                                           const_cast<float*>(x_dev), ldx,
                                           static_cast<const float*>(nullptr), 0, dim, weight_dev,
                                           eps, out_dev, ldo));
    }
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_add_rms_norm(b2w4_ctx* ctx, float* residual_dev, int ldr, const float* update_dev,
                      int ldu, int rows, int dim, const float* weight_dev, float eps,
                      float* out_dev, int ldo) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!residual_dev || !update_dev || !weight_dev || !out_dev || rows <= 0 || dim <= 0 ||
        ldr < dim || ldu < dim || ldo < dim)
        return b2w4_fail(ctx, B2W4_E_INVALID, "add_rms_norm: bad argument");
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, rms_norm_kernel, dim3(rows), dim3(kNormThreads), 0,
                                       ctx->stream, residual_dev, ldr, update_dev, ldu, dim,
                                       weight_dev, eps, out_dev, ldo));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_swiglu(b2w4_ctx* ctx, const float* merged_dev, int ldm, int rows, int intermediate,
                float* out_dev, int ldo) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!merged_dev || !out_dev || rows <= 0 || intermediate <= 0 || ldm < 2 * intermediate ||
        ldo < intermediate)
        return b2w4_fail(ctx, B2W4_E_INVALID, "swiglu: bad argument");
    const size_t n = (size_t)rows * intermediate;
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, swiglu_kernel, dim3((unsigned)((n + 255) / 256)),
                                       dim3(256), 0, ctx->stream, merged_dev, ldm, rows,
                                       intermediate, out_dev, ldo));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_elementwise(b2w4_ctx* ctx, const float* a_dev, const float* b_dev, float* out_dev,
                     size_t count, int multiply) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!a_dev || !b_dev || !out_dev || count == 0)
        return b2w4_fail(ctx, B2W4_E_INVALID, "elementwise: bad argument");
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, binary_kernel,
                                       dim3((unsigned)((count + 255) / 256)), dim3(256), 0,
                                       ctx->stream, a_dev, b_dev, out_dev, count, multiply));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_rope(b2w4_ctx* ctx, const float* x_dev, float* out_dev, int tokens, int heads, int dim,
              const float* cos_dev, const float* sin_dev, int rope_dim, int first_position,
              const int* position_dev) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!x_dev || !out_dev || !cos_dev || !sin_dev || tokens <= 0 || heads <= 0 || dim <= 0 ||
        rope_dim <= 0 || rope_dim > dim || (rope_dim & 1) || first_position < 0)
        return b2w4_fail(ctx, B2W4_E_INVALID, "rope: bad argument");
    const size_t n = (size_t)tokens * heads * ((size_t)rope_dim / 2 + (dim - rope_dim));
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, rope_kernel, dim3((unsigned)((n + 255) / 256)),
                                       dim3(256), 0, ctx->stream, x_dev, out_dev, tokens, heads,
                                       dim, cos_dev, sin_dev, rope_dim, first_position,
                                       position_dev));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_attention(b2w4_ctx* ctx, const float* q_dev, const float* k_dev, const float* v_dev,
                   float* k_cache_dev, float* v_cache_dev, float* out_dev, int tokens, int heads,
                   int kv_heads, int dim, int past, const int* past_dev, int capacity,
                   float scale) {
    if (!ctx)
        return B2W4_E_INVALID;
    const bool append = k_dev || v_dev;  // neither: the cache rows are in place already
    if (!q_dev || (append && (!k_dev || !v_dev)) || !k_cache_dev || !v_cache_dev || !out_dev ||
        tokens <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 ||
        dim > kAttnMaxDim || past < 0 || past + tokens > capacity)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "attention: bad argument (tokens=%d past=%d capacity=%d heads=%d/%d)",
                         tokens, past, capacity, heads, kv_heads);
    const int keys = past_dev ? capacity : past + tokens;  // position on the device: sized
                                                           // for a full cache
    const int rep = heads / kv_heads;
    // a run of tokens takes the tile kernel while a tile's scores fit in shared memory
    const int tile_slots = ((keys + 31) & ~31) + 8;  // rows 8 banks apart
    const size_t tile_smem = sizeof(float) * ((size_t)kTileRows * tile_slots + kAttnStage);
    const bool tiles = tokens >= 8 && ctx->attn_tiles && rep <= kTileRows &&
                       (dim == 64 || dim == 128 || dim == 256) && tile_smem <= 200 * 1024;
    const int score_slots = (keys + 3) & ~3;
    const size_t row_smem = sizeof(float) * ((size_t)score_slots + kAttnStage);
    if (!tiles && row_smem > 200 * 1024)
        return b2w4_fail(ctx, B2W4_E_INVALID, "attention: %d keys exceed the score buffer", keys);
    if (append) {
        const size_t n = (size_t)tokens * kv_heads * dim;
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, kv_append_kernel,
                                           dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                           ctx->stream, k_dev, v_dev, k_cache_dev, v_cache_dev,
                                           tokens, kv_heads, dim, past, past_dev, capacity));
        ctx->launches++;
    }
    const float* kc = k_cache_dev;
    const float* vc = v_cache_dev;
    if (tiles) {
        const int tq = kTileRows / rep;
        const dim3 grid((tokens + tq - 1) / tq, kv_heads);
#define B2W4_TILE(D)                                                                          \
    do {                                                                                      \
        static b2w4_smem_optin cfg;                                                           \
        B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, attention_tile_kernel<D>, tile_smem, cfg));      \
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, attention_tile_kernel<D>, grid,          \
                                           dim3(kAttnThreads), tile_smem, ctx->stream, q_dev, \
                                           kc, vc, out_dev, tokens, heads, kv_heads, past,    \
                                           past_dev, capacity, scale, tile_slots, tq));       \
    } while (0)
        if (dim == 64)
            B2W4_TILE(64);
        else if (dim == 128)
            B2W4_TILE(128);
        else
            B2W4_TILE(256);
#undef B2W4_TILE
    } else {
        static b2w4_smem_optin configured;
        B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, attention_kernel, row_smem, configured));
        B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, attention_kernel, dim3(tokens * heads),
                                           dim3(kAttnThreads), row_smem, ctx->stream, q_dev, kc,
                                           vc, out_dev, tokens, heads, kv_heads, dim, past,
                                           past_dev, capacity, scale, score_slots));
    }
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_qkv_prepare(b2w4_ctx* ctx, const float* qkv_dev, int ld, int tokens, int heads,
                     int kv_heads, int dim, const float* q_weight_dev, const float* k_weight_dev,
                     float eps, const float* cos_dev, const float* sin_dev, int past,
                     const int* past_dev, float* q_out_dev, float* k_cache_dev, float* v_cache_dev,
                     int capacity) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!qkv_dev || !cos_dev || !sin_dev || !q_out_dev || !k_cache_dev || !v_cache_dev ||
        tokens <= 0 || heads <= 0 || kv_heads <= 0 || dim <= 0 || dim > kAttnMaxDim || dim % 64 ||
        ld < (heads + 2 * kv_heads) * dim || past < 0 || past + tokens > capacity)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "qkv_prepare: bad argument (tokens=%d past=%d capacity=%d dim=%d)", tokens,
                         past, capacity, dim);
    const size_t threads = (size_t)tokens * (heads + 2 * kv_heads) * 32;
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, qkv_prepare_kernel,
                                       dim3((unsigned)((threads + 255) / 256)), dim3(256), 0,
                                       ctx->stream, qkv_dev, ld, tokens, heads, kv_heads, dim,
                                       q_weight_dev, k_weight_dev, eps, cos_dev, sin_dev, past,
                                       past_dev, q_out_dev, k_cache_dev, v_cache_dev, capacity));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_advance(b2w4_ctx* ctx, int* counter_dev, int by, const int32_t* token_dev,
                 int32_t* history_dev, int history_len) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!counter_dev)
        return b2w4_fail(ctx, B2W4_E_INVALID, "advance: no counter");
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, advance_kernel, dim3(1), dim3(32), 0, ctx->stream,
                                       counter_dev, by, token_dev, history_dev, history_len));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_copy_rows(b2w4_ctx* ctx, const float* src_dev, int ld_src, float* dst_dev, int ld_dst,
                   int rows, int cols) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!src_dev || !dst_dev || rows <= 0 || cols <= 0 || ld_src < cols || ld_dst < cols)
        return b2w4_fail(ctx, B2W4_E_INVALID, "copy_rows: bad argument");
    const size_t n = (size_t)rows * cols;
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, copy_rows_kernel,
                                       dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                       ctx->stream, src_dev, ld_src, dst_dev, ld_dst, rows, cols));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_embed_rows(b2w4_ctx* ctx, const void* table_fp16_dev, const int32_t* ids_dev, int rows,
                    int dim, float* out_dev, int ldo) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!table_fp16_dev || !ids_dev || !out_dev || rows <= 0 || dim <= 0 || ldo < dim)
        return b2w4_fail(ctx, B2W4_E_INVALID, "embed_rows: bad argument");
    const size_t n = (size_t)rows * dim;
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, embed_rows_kernel,
                                       dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                       ctx->stream, static_cast<const __half*>(table_fp16_dev),
                                       ids_dev, rows, dim, out_dev, ldo));
    ctx->launches++;
    return B2W4_OK;
}

}  // extern "C"
