// Weight upload hook: canonical BG128 blocks -> device nibble plane + scale plane.
// Stands in for the copy the reference makes in CudaBackend::wrap_weight_int4
// (engine/cuda_backend.cu:462-487 with upload_weight :147-175); the reference keeps the
// 544-byte blocks as they are, this backend splits them so the nibble stream is a
// sequence of aligned 512-byte chunks and the scales narrow to fp16 when that is exact.
#include "b200w4_internal.cuh"

namespace {

constexpr int kBlockBytes = 544;

// sets *flag when any group scale changes value on a round trip through fp16
__global__ void scales_fp16_exact_kernel(const uint8_t* __restrict__ blocks,
                                         long long nblocks, int* flag) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblocks * 8)
        return;
    const float* s = reinterpret_cast<const float*>(blocks + (i >> 3) * kBlockBytes);
    float v = s[i & 7];
    if (__half2float(__float2half_rn(v)) != v)
        atomicOr(flag, 1);
}

// one warp per block: 32 lanes move the 32 16-byte nibble chunks, 8 lanes the scales
template <bool SCL16>
__global__ void repack_bg128_kernel(const uint8_t* __restrict__ blocks, long long nblocks,
                                    uint4* __restrict__ nib, void* __restrict__ scl) {
    long long b = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (b >= nblocks)
        return;
    const uint8_t* src = blocks + b * kBlockBytes;
    // 544 = 34 * 16, so every chunk of every block stays 16-byte aligned
    nib[b * 32 + lane] = *reinterpret_cast<const uint4*>(src + 32 + lane * 16);
    if (lane < 8) {
        float v = reinterpret_cast<const float*>(src)[lane];
        if (SCL16)
            reinterpret_cast<__half*>(scl)[b * 8 + lane] = __float2half_rn(v);
        else
            reinterpret_cast<float*>(scl)[b * 8 + lane] = v;
    }
}

}  // namespace

int b2w4_launch_repack(b2w4_ctx* ctx, const void* dev_blocks, b2w4_weight* w) {
    const long long nblocks = (long long)w->tiles * w->groups;
    if ((reinterpret_cast<uintptr_t>(dev_blocks) & 15) != 0)
        return b2w4_fail(ctx, B2W4_E_INVALID, "BG128 blocks must be 16-byte aligned");
    B2W4_CUDA(ctx, cudaMemsetAsync(ctx->flag_dev, 0, sizeof(int), ctx->stream));
    {
        long long threads = nblocks * 8;
        int grid = (int)((threads + 255) / 256);
        scales_fp16_exact_kernel<<<grid, 256, 0, ctx->stream>>>(
            static_cast<const uint8_t*>(dev_blocks), nblocks, ctx->flag_dev);
        ctx->launches++;
    }
    int inexact = 0;
    B2W4_CUDA(ctx, cudaMemcpyAsync(&inexact, ctx->flag_dev, sizeof(int),
                                   cudaMemcpyDeviceToHost, ctx->stream));
    B2W4_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    w->scales_fp16 = inexact ? 0 : 1;
    w->nib_bytes = (size_t)nblocks * 512;
    w->scl_bytes = (size_t)nblocks * 8 * (w->scales_fp16 ? 2 : 4);
    B2W4_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&w->nib), w->nib_bytes));
    B2W4_CUDA(ctx, cudaMalloc(&w->scl, w->scl_bytes));
    {
        long long threads = nblocks * 32;
        int grid = (int)((threads + 255) / 256);
        if (w->scales_fp16)
            repack_bg128_kernel<true><<<grid, 256, 0, ctx->stream>>>(
                static_cast<const uint8_t*>(dev_blocks), nblocks, w->nib, w->scl);
        else
            repack_bg128_kernel<false><<<grid, 256, 0, ctx->stream>>>(
                static_cast<const uint8_t*>(dev_blocks), nblocks, w->nib, w->scl);
        ctx->launches++;
    }
    B2W4_CUDA(ctx, cudaGetLastError());
    B2W4_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return B2W4_OK;
}
