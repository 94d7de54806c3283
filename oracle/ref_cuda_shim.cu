// Test / benchmark infrastructure only: a thin extern "C" window onto the UNMODIFIED CUDA
// kernels of the reference (engine/cuda_matmul.cu, compiled from the reference tree for
// sm_100 by oracle/Makefile into oracle/_ref/libref_cuda.so).  They are the GPU comparator of
// the benchmark -- "the reference's own CUDA path on the same box" -- and are never on the
// product path.  No arithmetic happens here: every function forwards to the reference's
// launchers in the order CudaBackend::Impl::run_matmul_device uses them
// (engine/cuda_backend.cu:212-337):
//   M == 1: launch_q4_g128_dense_gemv            engine/cuda_matmul.cu:141-170, :234-243
//   M  > 1: launch_dequantize_q4_g128_dense_weight (:85-111, :214-221) into an fp16 [N,K]
//           scratch, launch_fp32_to_fp16 (:10-16, :176-181) of the activations, then
//           run_dense_matmul = cublasGemmEx, fp16 operands, fp32 accumulate (:245-260).
// All work goes to the legacy default stream, as in the reference.
#include "engine/cuda_internal.h"

#include <cstdio>

namespace {
cublasHandle_t g_cublas = nullptr;
void* g_weight_scratch = nullptr;
size_t g_weight_scratch_bytes = 0;
void* g_act_scratch = nullptr;
size_t g_act_scratch_bytes = 0;

bool reserve(void*& p, size_t& have, size_t need) {
    if (have >= need)
        return true;
    if (p)
        cudaFree(p);
    p = nullptr;
    have = 0;
    if (cudaMalloc(&p, need) != cudaSuccess)
        return false;
    have = need;
    return true;
}
}  // namespace

extern "C" {

// y[n] = W[n,k] * x[k], W as canonical BG128 blocks in device memory, x and y fp32 on the
// device.  Returns 0 on success.
int refcuda_gemv_g128(const float* x_dev, const void* blocks_dev, float* y_dev, int n, int k) {
    mollm_cuda::launch_q4_g128_dense_gemv(x_dev, static_cast<const Q4B8G128Block*>(blocks_dev),
                                          y_dev, n, k);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// y[m,n] = x[m,k] * W^T through the reference's M > 1 sequence (dequantise the whole weight to
// fp16, cast the activations, cuBLAS).  The two scratch buffers grow on demand, as the
// reference's do; call once before timing.
int refcuda_gemm_g128(const float* x_dev, int lda, const void* blocks_dev, float* y_dev, int m,
                      int n, int k) {
    if (!g_cublas && cublasCreate(&g_cublas) != CUBLAS_STATUS_SUCCESS)
        return -2;
    if (!reserve(g_weight_scratch, g_weight_scratch_bytes, sizeof(__half) * (size_t)n * k) ||
        !reserve(g_act_scratch, g_act_scratch_bytes, sizeof(__half) * (size_t)m * lda))
        return -3;
    const size_t packed_count = static_cast<size_t>((n + 7) / 8) * (k / 128) * 4 * 8 * 16;
    mollm_cuda::launch_dequantize_q4_g128_dense_weight(
        static_cast<const Q4B8G128Block*>(blocks_dev),
        reinterpret_cast<__half2*>(g_weight_scratch), packed_count, n, k / 128);
    mollm_cuda::launch_fp32_to_fp16(x_dev, static_cast<__half*>(g_act_scratch),
                                    static_cast<size_t>(m) * lda);
    if (cudaGetLastError() != cudaSuccess)
        return -1;
    return mollm_cuda::run_dense_matmul(g_cublas, g_weight_scratch, CUDA_R_16F, g_act_scratch,
                                        CUDA_R_16F, y_dev, m, n, k, lda)
               ? 0
               : -4;
}

void refcuda_release(void) {
    if (g_weight_scratch)
        cudaFree(g_weight_scratch);
    if (g_act_scratch)
        cudaFree(g_act_scratch);
    g_weight_scratch = g_act_scratch = nullptr;
    g_weight_scratch_bytes = g_act_scratch_bytes = 0;
    if (g_cublas)
        cublasDestroy(g_cublas);
    g_cublas = nullptr;
}

}  // extern "C"
