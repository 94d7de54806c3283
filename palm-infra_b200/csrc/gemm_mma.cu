// W4G128 x int8 GEMM for 9..256 activation rows per launch (batched decode, prefill) on the
// warp-level int8 tensor instruction (mma.sync m16n8k32) with register accumulators.
//
// Arithmetic = the reference's NEON W4A8 kernels: the GEMV applied row by row
// (kernels/matmul_w4.cpp:211-295 with the per-128 quantiser, kernels/matmul_quant.cpp:578-641)
//   per 128-k group g:  D = sum q4*q8 (int32);  y = fma(float(D), fp32(ws*as[g]), y)
// groups ascending, or the M > 1 rule (kernels/matmul_w4.cpp:785-901 with the per-32 quantiser,
// kernels/matmul_quant.cpp:280-329): the same step per 32-k block with one activation scale
// per block, blocks ascending.  The contract needs every group's exact int32 sum before the next fp32
// step, so an accumulator cannot run across K: each group's sums are produced, converted and
// folded into the fp32 chain, and the chain value of every (token, weight row) stays in one
// register of one thread for the whole K loop.  With mma.sync the int32 sums come back in
// registers, so that per-group step costs a handful of instructions and no hand-off.
//
// Work split.  The 8-row tiles of the weight are dealt to the CTAs in contiguous runs (one
// CTA per SM); a CTA's nibbles and scales are brought into shared memory once by per-thread
// cp.async, before the kernel waits for the quantiser in front of it (programmatic dependent
// launch).  The int8 activations stream through a two-stage ring, one 128-k group of all
// tokens per stage.  A warp owns one pair of tiles (16 weight rows = the rows of the tensor
// instruction) and a range of 8-token column blocks; per group it splits its weight words
// once into unsigned bytes q+8 (lo = (w ^ 0x08080808) & 0x0F0F0F0F: even k;
// hi = ((w >> 4) ^ 0x08080808) & 0x0F0F0F0F: odd k) and issues four u8 x s8 instructions per
// column block into ONE accumulator that starts at  bias = 0x4B400000 - 8*sum(codes)  (per
// token and group, from the quantiser): the accumulator ends as 0x4B400000 + D, which read as
// a float is 12582912 + D exactly (|D| < 2^22), so D costs one subtraction and no integer
// instruction.  The activation stages form a cp.async ring with one barrier per
// group.  The ring is as deep as shared memory allows (up to 8): with few tokens a group takes
// far less time to compute than a stage takes to arrive.
#include <algorithm>

#include "b200w4_internal.cuh"

namespace {

constexpr int kGemmWarps = 16;
constexpr int kGemmThreads = kGemmWarps * 32;
constexpr int kRowBytes = 144;  // a token's 128 bytes of a stage + 16: conflict-free 16-byte reads
constexpr int kMaxRows = 256;   // tokens per launch

struct GemmMmaArgs {
    const uint8_t* nib;
    const void* scl;
    const int8_t* qa;    // [m][K] int8, tensor-operand order inside each group
    const float* as_t;   // [G*spg][m_pad] activation scales (spg = 1: per 128, 4: per 32-block)
    const int32_t* es_t; // [G*spg][m_pad] 0x4B400000 - 8 * sum of the group's (block's) codes
    int spg;
    float* y;
    int ldc, m, m_pad, n, k, groups, tiles;
    int tiles_base, tiles_rem, tile_cap;
    int stages;  // depth of the activation ring (3..8), or the number of groups: all resident
    int activation, act_n_begin, act_n_len;
};

__device__ __forceinline__ uint32_t gm_smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void gm_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(gm_smem_u32(dst)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void gm_cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(gm_smem_u32(dst)), "l"(src)
                 : "memory");
}
// lane (gid = lane/4, tid = lane%4): a0 row gid, k 4*tid..+3; a1 row gid+8; a2/a3 k+16;
// b0 k 4*tid..+3 of column gid, b1 k+16; d0/d1 row gid, columns 2*tid, 2*tid+1; d2/d3 row gid+8
__device__ __forceinline__ void gm_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __noinline__ float gm_activation(float v, int act) { return b2w4_activation(v, act); }

constexpr int kMinStages = 3, kMaxStages = 8;

// wait until at most n of this thread's cp.async groups are still in flight (n is CTA-uniform)
__device__ __forceinline__ void gm_wait_groups(int n) {
    switch (n) {
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    }
}

// one stage = one 128-k group of every token: codes, scales, accumulator biases
template <int SPG>
__device__ __forceinline__ void load_stage(const GemmMmaArgs& a, int g, uint8_t* s_b, float* s_as,
                                           int* s_es) {
    const int chunks = a.m * 8;  // 16-byte chunks
    for (int i = threadIdx.x; i < chunks; i += kGemmThreads) {
        const int t = i >> 3, c = i & 7;
        gm_cp_async16(s_b + t * kRowBytes + c * 16,
                      a.qa + (size_t)t * a.k + (size_t)g * 128 + c * 16);
    }
    const int m8 = (a.m + 7) & ~7;
#pragma unroll
    for (int sb = 0; sb < SPG; ++sb)
        for (int t = threadIdx.x; t < a.m; t += kGemmThreads) {
            gm_cp_async4(s_as + sb * m8 + t, a.as_t + (size_t)(g * SPG + sb) * a.m_pad + t);
            gm_cp_async4(s_es + sb * m8 + t, a.es_t + (size_t)(g * SPG + sb) * a.m_pad + t);
        }
}

template <int CB, bool SCL16, bool A32>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_w4a8_mma_kernel(const GemmMmaArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int G = a.groups;
    const int tile_bytes = G * 512;
    const int scl_tile_bytes = G * 8 * (SCL16 ? 2 : 4);
    const int m8 = (a.m + 7) & ~7;
    uint8_t* s_w = smem;                                      // [cap][G][512]
    uint8_t* s_scl = s_w + (size_t)a.tile_cap * tile_bytes;   // [cap][G][8]
    const int S = a.stages;
    uint8_t* s_b = s_scl + (size_t)a.tile_cap * scl_tile_bytes;  // [S][m8][kRowBytes]
    constexpr int SPG = A32 ? 4 : 1;  // scales / biases per group
    float* s_as = reinterpret_cast<float*>(s_b + S * (size_t)m8 * kRowBytes);  // [S][SPG][m8]
    int* s_es = reinterpret_cast<int*>(s_as + S * SPG * m8);                    // [S][SPG][m8]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tid = lane & 3;
    const int cta = blockIdx.x;
    const int ntile = a.tiles_base + (cta < a.tiles_rem ? 1 : 0);
    const int tile0 = cta * a.tiles_base + min(cta, a.tiles_rem);

    b2w4_pdl_launch_dependents();
    // the CTA's weights: independent of the quantiser running in front of this kernel
    {
        const uint8_t* src = a.nib + (size_t)tile0 * tile_bytes;
        const int n16 = ntile * (tile_bytes >> 4);
        for (int i = threadIdx.x; i < n16; i += kGemmThreads)
            gm_cp_async16(s_w + (size_t)i * 16, src + (size_t)i * 16);
        const uint8_t* ssrc =
            reinterpret_cast<const uint8_t*>(a.scl) + (size_t)tile0 * scl_tile_bytes;
        const int s16 = ntile * (scl_tile_bytes >> 4);
        for (int i = threadIdx.x; i < s16; i += kGemmThreads)
            gm_cp_async16(s_scl + (size_t)i * 16, ssrc + (size_t)i * 16);
    }
    b2w4_pdl_wait();  // quantised activations come from the previous kernel
    // Ring mode: stages 0 .. S-2 in flight, one barrier per group.  Resident mode (S >= G,
    // few tokens): every group is loaded up front, one barrier in all, and the warps run
    // their K loops without meeting again.  The first copies also carry the weights.
    const bool resident = S >= G;
    const int pre = resident ? G : S - 1;
    for (int g = 0; g < pre; ++g) {
        if (g < G)
            load_stage<SPG>(a, g, s_b + (size_t)g * m8 * kRowBytes, s_as + g * SPG * m8,
                       s_es + g * SPG * m8);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (resident) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
    }

    // this warp's pair of tiles and its range of 8-token column blocks
    const int npair = (ntile + 1) >> 1;
    const int wpp = kGemmWarps / ((a.tile_cap + 1) >> 1);  // warps per pair (same in every CTA)
    const int pair = warp / wpp, wj = warp - pair * wpp;
    const bool busy = pair < npair;
    const int ncb = m8 >> 3;
    const int cb0 = wj * ncb / wpp, cb1 = busy ? (wj + 1) * ncb / wpp : cb0;
    const int t0 = pair * 2;
    const bool two = t0 + 1 < ntile;
    const uint32_t* s_w32 = reinterpret_cast<const uint32_t*>(s_w);
    const int tile_words = tile_bytes >> 2;

    float acc[CB][4];
#pragma unroll
    for (int j = 0; j < CB; ++j)
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

#pragma unroll 1
    for (int g = 0; g < G; ++g) {
        if (!resident) {
            gm_wait_groups(S - 2);
            __syncthreads();  // stage g visible to all; everyone is done with stage g-1
            if (g + S - 1 < G) {
                const int sn = (g + S - 1) % S;  // the slot stage g-1 used
                load_stage<SPG>(a, g + S - 1, s_b + (size_t)sn * m8 * kRowBytes, s_as + sn * SPG * m8,
                           s_es + sn * SPG * m8);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        const int st = resident ? g : g % S;
        if (cb0 < cb1) {
            const uint8_t* b = s_b + (size_t)st * m8 * kRowBytes;
            const float* as = s_as + st * SPG * m8;
            const int* es = s_es + st * SPG * m8;
            // word `lane` of the 128 bytes of (tile, group, 32-block s): row gid, k 8*tid..+7
            const int wbase = t0 * tile_words + g * 128 + lane;
            uint32_t lo0[4], hi0[4], lo1[4], hi1[4];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t u = s_w32[wbase + s * 32];
                const uint32_t v = two ? s_w32[wbase + tile_words + s * 32] : 0u;  // q = 0
                lo0[s] = (u ^ 0x08080808u) & 0x0F0F0F0Fu;
                hi0[s] = ((u >> 4) ^ 0x08080808u) & 0x0F0F0F0Fu;
                lo1[s] = (v ^ 0x08080808u) & 0x0F0F0F0Fu;
                hi1[s] = ((v >> 4) ^ 0x08080808u) & 0x0F0F0F0Fu;
            }
            const int si = (t0 * G + g) * 8 + gid;
            const float ws0 = SCL16 ? __half2float(reinterpret_cast<const __half*>(s_scl)[si])
                                    : reinterpret_cast<const float*>(s_scl)[si];
            const float ws1 =
                !two ? 0.f
                     : (SCL16 ? __half2float(reinterpret_cast<const __half*>(s_scl)[si + G * 8])
                              : reinterpret_cast<const float*>(s_scl)[si + G * 8]);
            const uint8_t* bl = b + gid * kRowBytes + tid * 32;
#pragma unroll
            for (int j = 0; j < CB; ++j) {
                const int cb = cb0 + j;
                if (cb < cb1) {  // warp-uniform
                    const uint4* bp = reinterpret_cast<const uint4*>(bl + cb * (8 * kRowBytes));
                    const uint4 be = bp[0], bo = bp[1];
                    const int tk = cb * 8 + tid * 2;  // tokens of this lane's accumulators
                    if (A32) {
                        // per 32-block: one instruction (even k | odd k), its own bias and
                        // activation scale; blocks folded into the chain in ascending order
                        const uint32_t bev[4] = {be.x, be.y, be.z, be.w};
                        const uint32_t bov[4] = {bo.x, bo.y, bo.z, bo.w};
#pragma unroll
                        for (int sb = 0; sb < 4; ++sb) {
                            const int2 bias = *reinterpret_cast<const int2*>(es + sb * m8 + tk);
                            const float2 asv = *reinterpret_cast<const float2*>(as + sb * m8 + tk);
                            int c[4] = {bias.x, bias.y, bias.x, bias.y};
                            gm_mma(c, lo0[sb], lo1[sb], hi0[sb], hi1[sb], bev[sb], bov[sb]);
                            acc[j][0] = __fmaf_rn(__fsub_rn(__int_as_float(c[0]), 12582912.f),
                                                  __fmul_rn(ws0, asv.x), acc[j][0]);
                            acc[j][1] = __fmaf_rn(__fsub_rn(__int_as_float(c[1]), 12582912.f),
                                                  __fmul_rn(ws0, asv.y), acc[j][1]);
                            acc[j][2] = __fmaf_rn(__fsub_rn(__int_as_float(c[2]), 12582912.f),
                                                  __fmul_rn(ws1, asv.x), acc[j][2]);
                            acc[j][3] = __fmaf_rn(__fsub_rn(__int_as_float(c[3]), 12582912.f),
                                                  __fmul_rn(ws1, asv.y), acc[j][3]);
                        }
                    } else {
                        const int2 bias = *reinterpret_cast<const int2*>(es + tk);
                        const float2 asv = *reinterpret_cast<const float2*>(as + tk);
                        // two chains of two instructions (latency), joined by one add
                        int c[4] = {bias.x, bias.y, bias.x, bias.y}, c2[4] = {0, 0, 0, 0};
                        gm_mma(c, lo0[0], lo1[0], lo0[1], lo1[1], be.x, be.y);
                        gm_mma(c2, hi0[0], hi1[0], hi0[1], hi1[1], bo.x, bo.y);
                        gm_mma(c, lo0[2], lo1[2], lo0[3], lo1[3], be.z, be.w);
                        gm_mma(c2, hi0[2], hi1[2], hi0[3], hi1[3], bo.z, bo.w);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            c[i] += c2[i];
                        // c = 0x4B400000 + D: as a float 12582912 + D, exactly
                        acc[j][0] = __fmaf_rn(__fsub_rn(__int_as_float(c[0]), 12582912.f),
                                              __fmul_rn(ws0, asv.x), acc[j][0]);
                        acc[j][1] = __fmaf_rn(__fsub_rn(__int_as_float(c[1]), 12582912.f),
                                              __fmul_rn(ws0, asv.y), acc[j][1]);
                        acc[j][2] = __fmaf_rn(__fsub_rn(__int_as_float(c[2]), 12582912.f),
                                              __fmul_rn(ws1, asv.x), acc[j][2]);
                        acc[j][3] = __fmaf_rn(__fsub_rn(__int_as_float(c[3]), 12582912.f),
                                              __fmul_rn(ws1, asv.y), acc[j][3]);
                    }
                }
            }
        }
    }

    // y[token][n]: for one token, the eight lanes of a quarter-warp hold eight consecutive n
    if (cb0 < cb1) {
        const int n0 = (tile0 + t0) * 8 + gid, n1 = n0 + 8;
        const bool act0 = b2w4_act_applies(n0, a.activation, a.act_n_begin, a.act_n_len, a.n);
        const bool act1 = b2w4_act_applies(n1, a.activation, a.act_n_begin, a.act_n_len, a.n);
#pragma unroll
        for (int j = 0; j < CB; ++j) {
            const int cb = cb0 + j;
            if (cb < cb1) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int t = cb * 8 + tid * 2 + c;
                    if (t < a.m) {
                        if (n0 < a.n) {
                            float v = acc[j][c];
                            if (act0)
                                v = gm_activation(v, a.activation);
                            a.y[(size_t)t * a.ldc + n0] = v;
                        }
                        if (two && n1 < a.n) {
                            float v = acc[j][2 + c];
                            if (act1)
                                v = gm_activation(v, a.activation);
                            a.y[(size_t)t * a.ldc + n1] = v;
                        }
                    }
                }
            }
        }
    }
}

size_t gemm_mma_smem(int groups, int cap, int m8, bool scl16, int spg, int stages = kMinStages) {
    return (size_t)cap * groups * 512 + (size_t)cap * groups * 8 * (scl16 ? 2 : 4) +
           stages * ((size_t)m8 * kRowBytes + 2 * sizeof(float) * (size_t)m8 * spg) + 16;
}

template <int CB, bool SCL16, bool A32>
int gemm_mma_launch(b2w4_ctx* ctx, const GemmMmaArgs& a, size_t smem, int ctas) {
    auto kern = gemm_w4a8_mma_kernel<CB, SCL16, A32>;
    static b2w4_smem_optin configured;  // per instantiation and device
    B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, kern, smem, configured));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B2W4_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, a));
    ctx->launches++;
    return B2W4_OK;
}

template <int CB>
int gemm_mma_launch_cb(b2w4_ctx* ctx, const GemmMmaArgs& a, bool scl16, size_t smem, int ctas) {
    if (a.spg == 4)
        return scl16 ? gemm_mma_launch<CB, true, true>(ctx, a, smem, ctas)
                     : gemm_mma_launch<CB, false, true>(ctx, a, smem, ctas);
    return scl16 ? gemm_mma_launch<CB, true, false>(ctx, a, smem, ctas)
                 : gemm_mma_launch<CB, false, false>(ctx, a, smem, ctas);
}

}  // namespace

// True when the shape fits this kernel: a tile (8 rows x K) plus the activation ring must fit
// one SM's shared memory.
bool b2w4_gemm_mma_fits(const b2w4_weight* w, int m, int act_rule) {
    const int m8 = (std::min(m, kMaxRows) + 7) & ~7;
    const int spg = act_rule == B2W4_ACT_G32 ? 4 : 1;
    return gemm_mma_smem(w->groups, 2, m8, w->scales_fp16 != 0, spg) <= 220 * 1024;
}

// True when, with one CTA per SM, the CTA's weights and ALL groups of the activations fit in
// shared memory together: the regime this kernel is the fastest in (measured on config 2:
// 16 rows 14 us against 19 us on the tcgen05 kernel; from 64 rows on the tcgen05 kernel wins).
bool b2w4_gemm_mma_resident(const b2w4_weight* w, int m, int act_rule, int sm_count) {
    if (m > kMaxRows)
        return false;
    const int m8 = (m + 7) & ~7;
    const int cap = (w->tiles + sm_count - 1) / sm_count;
    const int spg = act_rule == B2W4_ACT_G32 ? 4 : 1;
    return gemm_mma_smem(w->groups, cap, m8, w->scales_fp16 != 0, spg, w->groups) <= 220 * 1024;
}

int b2w4_launch_gemm_mma(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                         float* y, int ldc, int m, int act_rule, int activation,
                         int act_n_begin, int act_n_len) {
    const int G = w->groups;
    const int spg = act_rule == B2W4_ACT_G32 ? 4 : 1;
    const bool scl16 = w->scales_fp16 != 0;
    for (int m0 = 0; m0 < m; m0 += kMaxRows) {
        const int mc = std::min(kMaxRows, m - m0);
        const int m8 = (mc + 7) & ~7;
        void *qa = nullptr, *sc = nullptr;
        int rc;
        if ((rc = b2w4_reserve(ctx, SCR_QA, (size_t)mc * w->k, &qa)) != B2W4_OK ||
            (rc = b2w4_reserve(ctx, SCR_AS, 2 * sizeof(float) * (size_t)G * spg * m8, &sc)) !=
                B2W4_OK)
            return rc;
        float* as_t = static_cast<float*>(sc);
        int32_t* es_t = reinterpret_cast<int32_t*>(as_t + (size_t)G * spg * m8);
        if ((rc = b2w4_launch_quantize_mma(ctx, x + (size_t)m0 * lda, lda, mc, w->k, m8, act_rule,
                                           static_cast<int8_t*>(qa), as_t, es_t)) != B2W4_OK)
            return rc;
        // tiles per CTA: what fits beside the activation ring, one CTA per SM when possible
        // (a warp keeps at most 12 column blocks of accumulators: enough warps per tile pair)
        const int ncb = m8 / 8;
        const int min_wpp = (ncb + 11) / 12;
        int cap = std::min(16, 2 * (kGemmWarps / min_wpp));
        while (cap > 1 && gemm_mma_smem(G, cap, m8, scl16, spg) > 220 * 1024)
            --cap;
        if (gemm_mma_smem(G, cap, m8, scl16, spg) > 220 * 1024)
            return b2w4_fail(ctx, B2W4_E_INVALID, "gemm: K=%d needs too much shared memory", w->k);
        const int sms = ctx->sm_count;
        int ctas = (w->tiles + sms - 1) / sms <= cap ? std::min(w->tiles, sms)
                                                     : (w->tiles + cap - 1) / cap;
        GemmMmaArgs a;
        a.nib = reinterpret_cast<const uint8_t*>(w->nib);
        a.scl = w->scl;
        a.qa = static_cast<const int8_t*>(qa);
        a.as_t = as_t;
        a.es_t = es_t;
        a.y = y + (size_t)m0 * ldc;
        a.ldc = ldc;
        a.m = mc;
        a.m_pad = m8;
        a.spg = spg;
        a.n = w->n;
        a.k = w->k;
        a.groups = G;
        a.tiles = w->tiles;
        a.tiles_base = w->tiles / ctas;
        a.tiles_rem = w->tiles % ctas;
        a.tile_cap = a.tiles_base + (a.tiles_rem ? 1 : 0);
        a.activation = activation;
        a.act_n_begin = act_n_begin;
        a.act_n_len = act_n_len;
        a.stages = kMinStages;
        if (gemm_mma_smem(G, a.tile_cap, m8, scl16, spg, G) <= 220 * 1024)
            a.stages = G;  // few tokens: all groups resident, no per-group barrier
        else
            while (a.stages < kMaxStages &&
                   gemm_mma_smem(G, a.tile_cap, m8, scl16, spg, a.stages + 1) <= 220 * 1024)
                ++a.stages;
        const size_t smem = gemm_mma_smem(G, a.tile_cap, m8, scl16, spg, a.stages);
        // column blocks per warp: 16 warps over the CTA's tile pairs
        const int wpp = kGemmWarps / ((a.tile_cap + 1) / 2);
        const int need = (ncb + wpp - 1) / wpp;
        if (need > 12)
            return b2w4_fail(ctx, B2W4_E_INVALID, "gemm: internal: %d column blocks per warp",
                             need);
        rc = need <= 1   ? gemm_mma_launch_cb<1>(ctx, a, scl16, smem, ctas)
             : need <= 2 ? gemm_mma_launch_cb<2>(ctx, a, scl16, smem, ctas)
             : need <= 4 ? gemm_mma_launch_cb<4>(ctx, a, scl16, smem, ctas)
             : need <= 8 ? gemm_mma_launch_cb<8>(ctx, a, scl16, smem, ctas)
                         : gemm_mma_launch_cb<12>(ctx, a, scl16, smem, ctas);
        if (rc != B2W4_OK)
            return rc;
    }
    return B2W4_OK;
}
