// Stand-alone activation quantiser: fp32 rows -> int8 codes + one fp32 scale per group.
// Follows the reference quantisers' rounding points exactly
// (kernels/matmul_quant.cpp:578-641 per 128 values, :280-329 per 32 values): amax over the
// group, scale = amax/127 (1 when amax == 0), codes = clamp(rint(x * (127/amax)), +-127).
#include "b200w4_internal.cuh"

namespace {

// one warp per (row, 128-group); lane holds k = 4*lane .. 4*lane+3 of the group
template <int RULE, int LAYOUT>
__global__ void quantize_rows_kernel(const float* __restrict__ x, int lda, int m, int k,
                                     int8_t* __restrict__ q, float* __restrict__ scales) {
    b2w4_pdl_chain_entry();
    const int groups = k >> 7;
    long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)m * groups)
        return;
    const int row = (int)(wid / groups), g = (int)(wid % groups);
    const float* src = x + (size_t)row * lda + (size_t)g * 128 + lane * 4;
    float v0 = src[0], v1 = src[1], v2 = src[2], v3 = src[3];
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
    // max is exact and order-free, so a butterfly gives the sequential loop's value
    const int span = RULE == 128 ? 32 : 8;
#pragma unroll
    for (int off = span / 2; off > 0; off >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float scale, inv;
    b2w4_quant_params(amax, scale, inv);
    const int c0 = b2w4_quant_code(v0, inv), c1 = b2w4_quant_code(v1, inv);
    const int c2 = b2w4_quant_code(v2, inv), c3 = b2w4_quant_code(v3, inv);
    if (RULE == 128) {
        if (lane == 0)
            scales[(size_t)row * groups + g] = scale;
    } else if ((lane & 7) == 0) {
        scales[(size_t)row * (groups * 4) + g * 4 + (lane >> 3)] = scale;
    }
    int8_t* dst = q + (size_t)row * k + (size_t)g * 128;
    if (LAYOUT == QLAYOUT_NATURAL) {
        char4 packed = make_char4((signed char)c0, (signed char)c1, (signed char)c2,
                                  (signed char)c3);
        *reinterpret_cast<char4*>(dst + lane * 4) = packed;
    } else if (LAYOUT == QLAYOUT_MMA) {
        // the lane holds k = 4*lane..+3: 32-block lane/8, even-k indices 2*(lane%8) and +1
        int8_t* blk = dst + ((lane & 7) >> 1) * 32 + (lane >> 3) * 4 + (lane & 1) * 2;
        *reinterpret_cast<char2*>(blk) = make_char2((signed char)c0, (signed char)c2);
        *reinterpret_cast<char2*>(blk + 16) = make_char2((signed char)c1, (signed char)c3);
    } else {
        // 32-block `sub` = lane/8 stored as 16 even-k codes then 16 odd-k codes
        int8_t* blk = dst + (lane >> 3) * 32;
        const int j = (lane & 7) * 2;
        *reinterpret_cast<char2*>(blk + j) = make_char2((signed char)c0, (signed char)c2);
        *reinterpret_cast<char2*>(blk + 16 + j) =
            make_char2((signed char)c1, (signed char)c3);
    }
}

// Same quantiser, output laid out for the tensor-core kernel: per 128-k group a plane of
// [m_pad tokens][128 bytes]; inside a token's 128 bytes the 32-block `sub` is the 16-byte
// chunk pair (2*sub: even k, 2*sub+1: odd k), and chunk c is stored at position
// c ^ (token % 8): the 128-byte swizzle the MMA's shared-memory descriptor expects, so the
// plane can be bulk-copied into shared memory as is.  Scales: fp32 [groups][m_pad]; with one
// scale per 32 values (A32) [groups][m_pad][4], a token's four block scales side by side.
template <bool A32>
__global__ void quantize_rows_umma_kernel(const float* __restrict__ x, int lda, int m, int k,
                                          int m_pad, int8_t* __restrict__ q,
                                          float* __restrict__ scales) {
    const int groups = k >> 7;
    long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)m * groups)
        return;
    const int row = (int)(wid / groups), g = (int)(wid % groups);
    const float* src = x + (size_t)row * lda + (size_t)g * 128 + lane * 4;
    float v0 = src[0], v1 = src[1], v2 = src[2], v3 = src[3];
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
    // per 128 values: all 32 lanes; per 32 values: the 8 lanes of a 32-block
#pragma unroll
    for (int off = A32 ? 4 : 16; off > 0; off >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float scale, inv;
    b2w4_quant_params(amax, scale, inv);
    const int c0 = b2w4_quant_code(v0, inv), c1 = b2w4_quant_code(v1, inv);
    const int c2 = b2w4_quant_code(v2, inv), c3 = b2w4_quant_code(v3, inv);
    if (A32) {
        if ((lane & 7) == 0)
            scales[((size_t)g * m_pad + row) * 4 + (lane >> 3)] = scale;
    } else if (lane == 0) {
        scales[(size_t)g * m_pad + row] = scale;
    }
    int8_t* tokp = q + ((size_t)g * m_pad + row) * 128;
    const int sub = lane >> 3, j = (lane & 7) * 2, sw = row & 7;
    *reinterpret_cast<char2*>(tokp + (((2 * sub) ^ sw) << 4) + j) =
        make_char2((signed char)c0, (signed char)c2);
    *reinterpret_cast<char2*>(tokp + (((2 * sub + 1) ^ sw) << 4) + j) =
        make_char2((signed char)c1, (signed char)c3);
}

// Same quantiser for the mma.sync GEMM: codes int8 [m][K] in tensor-operand order
// (QLAYOUT_MMA), scales and the accumulator bias 0x4B400000 - 8 * (sum of the group's codes)
// transposed to [groups][m_pad] (per-32 rule: [groups*4][m_pad], one entry per 32-block) so
// that one group of all tokens is contiguous.  (The kernel
// multiplies unsigned nibbles q+8; starting its int32 accumulator at the bias makes it end as
// 0x4B400000 + D, the bit pattern of the float 12582912 + D.)
template <bool A32>
__global__ void quantize_rows_mma_kernel(const float* __restrict__ x, int lda, int m, int k,
                                         int m_pad, int8_t* __restrict__ q,
                                         float* __restrict__ scales_t,
                                         int32_t* __restrict__ es_t) {
    b2w4_pdl_launch_dependents();  // the GEMM behind may start fetching its weights
    const int groups = k >> 7;
    long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)m * groups)
        return;
    const int row = (int)(wid / groups), g = (int)(wid % groups);
    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)row * lda + (size_t)g * 128 +
                                                      lane * 4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    // per 128 values: all 32 lanes; per 32 values: the 8 lanes of a 32-block
#pragma unroll
    for (int off = A32 ? 4 : 16; off > 0; off >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float scale, inv;
    b2w4_quant_params(amax, scale, inv);
    const int c0 = b2w4_quant_code(v.x, inv), c1 = b2w4_quant_code(v.y, inv);
    const int c2 = b2w4_quant_code(v.z, inv), c3 = b2w4_quant_code(v.w, inv);
    int esum = c0 + c1 + c2 + c3;  // integer: order-free
#pragma unroll
    for (int off = A32 ? 4 : 16; off > 0; off >>= 1)
        esum += __shfl_xor_sync(0xffffffffu, esum, off);
    if (A32) {
        if ((lane & 7) == 0) {
            const size_t at = (size_t)(g * 4 + (lane >> 3)) * m_pad + row;
            scales_t[at] = scale;
            es_t[at] = 0x4B400000 - 8 * esum;
        }
    } else if (lane == 0) {
        scales_t[(size_t)g * m_pad + row] = scale;
        es_t[(size_t)g * m_pad + row] = 0x4B400000 - 8 * esum;
    }
    // the lane holds k = 4*lane..+3: 32-block lane/8, even-k indices 2*(lane%8) and +1
    int8_t* blk = q + (size_t)row * k + (size_t)g * 128 + ((lane & 7) >> 1) * 32 +
                  (lane >> 3) * 4 + (lane & 1) * 2;
    *reinterpret_cast<char2*>(blk) = make_char2((signed char)c0, (signed char)c2);
    *reinterpret_cast<char2*>(blk + 16) = make_char2((signed char)c1, (signed char)c3);
}

}  // namespace

int b2w4_launch_quantize_mma(b2w4_ctx* ctx, const float* x, int lda, int m, int k, int m_pad,
                             int act_rule, int8_t* q, float* scales_t, int32_t* es_t) {
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (lda & 3))
        return b2w4_fail(ctx, B2W4_E_INVALID, "quantize: rows must be 16-byte aligned");
    long long warps = (long long)m * (k / 128);
    int grid = (int)((warps * 32 + 255) / 256);
    if (act_rule == B2W4_ACT_G32)
        quantize_rows_mma_kernel<true><<<grid, 256, 0, ctx->stream>>>(x, lda, m, k, m_pad, q,
                                                                      scales_t, es_t);
    else
        quantize_rows_mma_kernel<false><<<grid, 256, 0, ctx->stream>>>(x, lda, m, k, m_pad, q,
                                                                       scales_t, es_t);
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}

int b2w4_launch_quantize_umma(b2w4_ctx* ctx, const float* x, int lda, int m, int k, int m_pad,
                              int act_rule, int8_t* q, float* scales) {
    long long warps = (long long)m * (k / 128);
    int grid = (int)((warps * 32 + 255) / 256);
    if (act_rule == B2W4_ACT_G32)
        quantize_rows_umma_kernel<true><<<grid, 256, 0, ctx->stream>>>(x, lda, m, k, m_pad, q,
                                                                       scales);
    else
        quantize_rows_umma_kernel<false><<<grid, 256, 0, ctx->stream>>>(x, lda, m, k, m_pad, q,
                                                                        scales);
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}

int b2w4_launch_quantize(b2w4_ctx* ctx, const float* x, int lda, int m, int k,
                         int act_rule, int8_t* q, float* scales, int layout) {
    if (k <= 0 || k % 128 != 0 || m <= 0 || lda < k)
        return b2w4_fail(ctx, B2W4_E_INVALID, "quantize: bad shape m=%d k=%d lda=%d", m,
                         k, lda);
    if (act_rule != B2W4_ACT_G128 && act_rule != B2W4_ACT_G32)
        return b2w4_fail(ctx, B2W4_E_INVALID, "quantize: act_rule must be 128 or 32");
    long long warps = (long long)m * (k / 128);
    int grid = (int)((warps * 32 + 255) / 256);
#define LAUNCH(R, L)                                                                         \
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, quantize_rows_kernel<R, L>, dim3(grid),        \
                                       dim3(256), 0, ctx->stream, x, lda, m, k, q, scales))
    if (act_rule == 128 && layout == QLAYOUT_NATURAL)
        LAUNCH(128, QLAYOUT_NATURAL);
    else if (act_rule == 128 && layout == QLAYOUT_MMA)
        LAUNCH(128, QLAYOUT_MMA);
    else if (act_rule == 128)
        LAUNCH(128, QLAYOUT_EVEN_ODD);
    else if (layout == QLAYOUT_NATURAL)
        LAUNCH(32, QLAYOUT_NATURAL);
    else if (layout == QLAYOUT_MMA)
        LAUNCH(32, QLAYOUT_MMA);
    else
        LAUNCH(32, QLAYOUT_EVEN_ODD);
#undef LAUNCH
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}
