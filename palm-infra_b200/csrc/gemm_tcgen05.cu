// W4G128 x int8 GEMM for 5..256+ activation rows (batched decode, prefill) on the 5th-gen
// tensor cores: tcgen05.mma kind::i8 with int32 accumulators in tensor memory.
//
// Arithmetic = the reference's W4A8 kernels with one activation scale per 128 values
// (kernels/matmul_w4.cpp:211-295 applied row by row, kernels/matmul_quant.cpp:578-641):
//   per 128-k group g:  D = sum q4*q8 (int32);  y = fma(float(D), fp32(ws*as[g]), y)
// groups ascending.  The int32 group sums are exact on any hardware; the tensor cores
// produce them, and the order-sensitive fp32 chain runs on the CUDA cores, so the result
// is bit-identical to the row-by-row GEMV.
//
// Tile.  A CTA owns R consecutive weight rows (a multiple of 8, at most RP) and up to 256
// tokens.  Tokens sit on the MMA's M side (two blocks of 128 = the 128 TMEM lanes), weight
// rows on its N side: D[token][row] for one group is one 128 x RP int32 tile per token
// block.  R is chosen so that one wave of CTAs covers the weight (N / #SMs rounded up to a
// tile), which no power-of-two tile would do for N = 9728 on 148 SMs.
//
// Pipeline per 128-k group (stage = group, ring of kStages):
//   producer warp   bulk-copies (TMA engine) the group's nibble chunks of the CTA's row
//                   tiles and the pre-quantised, pre-swizzled int8 activations
//   unpack warps    nibbles -> int8 (left-aligned: 16*q4) into the B operand's K-major,
//                   128-byte-swizzled layout; a 128-k group is exactly one swizzle row
//   MMA warp        one thread issues 4 x tcgen05.mma (K = 32 each) per token block into
//                   the group's TMEM accumulator, then tcgen05.commit
//   epilogue warps  tcgen05.ld the int32 sums (thread = token, columns = weight rows),
//                   shift out the factor 16, and run the fp32 chain in registers
// TMEM holds two group accumulators, so the MMAs of group g+1 overlap the chain of group g.
// Every wait is bounded; on a timeout the kernel flags the status word and drains.
#include "b200w4_internal.cuh"

namespace {

constexpr int kStages = 3;
constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kUnpackWarp0 = 2, kUnpackWarps = 4;
constexpr int kEpiWarp0 = 6, kEpiWarps = 8;
constexpr int kThreads = (kEpiWarp0 + kEpiWarps) * 32;  // 448
constexpr unsigned kSpinLimit = 1u << 24;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

struct GemmArgs {
    const uint8_t* nib;  // [tiles][G][512]
    const void* scl;     // [tiles][G][8] fp16|fp32
    const int8_t* qa;    // [G][m_pad][128] int8, 16-byte chunks swizzled by token%8
    const float* as;     // [G][m_pad]
    float* y;
    int* status;
    int ldc, m, m_pad, n, groups, tiles;
    int rows_per_cta;  // R
    int activation, act_n_begin, act_n_len;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// false when the iteration or the time limit runs out
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity))
        return true;
    const unsigned long long t0 = global_ns();
    for (unsigned spins = 0; spins < kSpinLimit; ++spins) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((spins & 255) == 255 && global_ns() - t0 > kWaitLimitNs)
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

// K-major operand, 128-byte swizzle, 8-row atoms of 1024 bytes packed back to back:
// start address >> 4 in bits [0,14), leading byte offset (unused for swizzled K-major) = 1
// in [16,30), stride byte offset 1024 >> 4 in [32,46), descriptor version 1 in [46,48),
// layout type SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::i8, int32 accumulate, signed 8-bit A and B, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_i8(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
          "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __noinline__ float gemm_activation(float v, int act) {
    return b2w4_activation(v, act);
}

// shared-memory plan; stage buffers are 1024-byte aligned (swizzle atoms)
template <int RP>
struct Smem {
    static constexpr int kActStage = 256 * 128;       // two token blocks of 128 x 128 B
    static constexpr int kBStage = RP * 128;          // int8 weights, swizzled
    static constexpr int kRawStage = (RP / 8) * 512;  // nibble chunks
    static constexpr int kActOff = 0;
    static constexpr int kBOff = kActOff + kStages * kActStage;
    static constexpr int kRawOff = kBOff + kStages * kBStage;
    static constexpr int kWsOff = kRawOff + kStages * kRawStage;  // fp32 [G][RP], G <= kMaxG
    static constexpr int kMaxG = 80;  // K <= 10240
    static constexpr int kSclRawOff = kWsOff + kMaxG * RP * 4;    // raw scale chunk
    static constexpr int kBarOff = kSclRawOff + (RP / 8) * kMaxG * 32;
    static constexpr int kTotal = kBarOff + 256 + 1024;  // + slack to align the base
};

template <int RP, bool SCL16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_tc_kernel(const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // swizzle atoms need a 1024-byte aligned base
    uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
    using S = Smem<RP>;
    const int G = a.groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = min(a.rows_per_cta, a.n - blockIdx.x * a.rows_per_cta);  // may be ragged
    const int r_tiles = (R + 7) / 8;
    const int tile0 = blockIdx.x * (a.rows_per_cta / 8);
    const int tok0 = blockIdx.y * 256;
    const int m_here = min(256, a.m - tok0);
    const int n_blocks = (m_here + 127) / 128;  // token blocks of 128 in this CTA

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
    uint64_t* raw_full = bars;                 // [kStages] nibbles + activations landed
    uint64_t* b_full = bars + kStages;         // [kStages] unpack done
    uint64_t* stage_free = bars + 2 * kStages; // [kStages] MMAs that read the stage retired
    uint64_t* acc_full = bars + 3 * kStages;   // [2] group accumulator complete
    uint64_t* acc_free = acc_full + 2;         // [2] epilogue has read it
    uint64_t* scl_full = acc_free + 2;         // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(scl_full + 1);
    volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&b_full[s], kUnpackWarps);
            mbar_init(&stage_free[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_free[b], kEpiWarps);
        }
        mbar_init(scl_full, 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {  // one warp owns the TMEM allocation: 512 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // accumulator b, token block mb: columns [b*256 + mb*RP, +RP)
    auto fail = [&]() {
        *s_abort = 1;
        atomicExch(a.status, B2W4_E_TIMEOUT);
    };

    if (warp == kProducerWarp) {
        // =============================== producer ===================================
        if (lane == 0) {
            // weight scales of the CTA's row tiles: [r_tiles][G][8], one contiguous run
            const uint32_t scl_bytes = (uint32_t)r_tiles * G * 8 * (SCL16 ? 2 : 4);
            mbar_expect_tx(scl_full, scl_bytes);
            bulk_g2s(smem + S::kSclRawOff,
                     reinterpret_cast<const uint8_t*>(a.scl) +
                         (size_t)tile0 * G * 8 * (SCL16 ? 2 : 4),
                     scl_bytes, scl_full);
            for (int g = 0; g < G; ++g) {
                const int s = g % kStages, round = g / kStages;
                if (round > 0 && !mbar_wait(&stage_free[s], (round - 1) & 1)) {
                    fail();
                    break;
                }
                const uint32_t act_bytes = (uint32_t)n_blocks * 128 * 128;
                mbar_expect_tx(&raw_full[s], (uint32_t)r_tiles * 512 + act_bytes);
                for (int t = 0; t < r_tiles; ++t)
                    bulk_g2s(smem + S::kRawOff + s * S::kRawStage + t * 512,
                             a.nib + ((size_t)(tile0 + t) * G + g) * 512, 512, &raw_full[s]);
                bulk_g2s(smem + S::kActOff + s * S::kActStage,
                         a.qa + ((size_t)g * a.m_pad + tok0) * 128, act_bytes, &raw_full[s]);
            }
        }
    } else if (warp == kMmaWarp) {
        // =============================== MMA issue ===================================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(RP);
            for (int g = 0; g < G; ++g) {
                const int s = g % kStages, round = g / kStages;
                const int b = g & 1, use = g >> 1;
                if (!mbar_wait(&b_full[s], round & 1) ||
                    (use > 0 && !mbar_wait(&acc_free[b], (use - 1) & 1))) {
                    fail();
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t b_addr = smem_u32(smem + S::kBOff + s * S::kBStage);
                for (int mb = 0; mb < n_blocks; ++mb) {
                    const uint32_t a_addr =
                        smem_u32(smem + S::kActOff + s * S::kActStage + mb * 128 * 128);
                    const uint32_t d = tmem_base + (uint32_t)(b * 256 + mb * RP);
#pragma unroll
                    for (int j = 0; j < 4; ++j)  // four K = 32 steps inside the swizzle row
                        umma_i8(d, umma_desc_k_sw128(a_addr + j * 32),
                                umma_desc_k_sw128(b_addr + j * 32), idesc, j > 0 ? 1u : 0u);
                }
                umma_commit(&stage_free[s]);  // the stage's operands may be overwritten
                umma_commit(&acc_full[b]);    // the group's sums are complete
            }
        }
    } else if (warp < kEpiWarp0) {
        // =============================== unpack ======================================
        const int ut = (warp - kUnpackWarp0) * 32 + lane;  // 0..127
        for (int g = 0; g < G; ++g) {
            const int s = g % kStages, round = g / kStages;
            // raw_full also orders us after stage_free: the producer waited for it
            if (*s_abort || !mbar_wait(&raw_full[s], round & 1)) {
                if (lane == 0)
                    fail();
                break;
            }
            const uint4* raw = reinterpret_cast<const uint4*>(smem + S::kRawOff + s * S::kRawStage);
            uint8_t* bst = smem + S::kBOff + s * S::kBStage;
            // chunk c of tile t: sub = c/8, row = c%8 -> 32 k of weight row t*8+row
            for (int c = ut; c < r_tiles * 32; c += kUnpackWarps * 32) {
                const uint4 w = raw[c];
                const int t = c >> 5, sub = (c >> 3) & 3, row = c & 7;
                uint4 ev, od;
                ev.x = (w.x << 4) & 0xF0F0F0F0u;
                od.x = w.x & 0xF0F0F0F0u;
                ev.y = (w.y << 4) & 0xF0F0F0F0u;
                od.y = w.y & 0xF0F0F0F0u;
                ev.z = (w.z << 4) & 0xF0F0F0F0u;
                od.z = w.z & 0xF0F0F0F0u;
                ev.w = (w.w << 4) & 0xF0F0F0F0u;
                od.w = w.w & 0xF0F0F0F0u;
                // weight row r = t*8+row: atom t (1024 B), row `row` (128 B), 16-byte
                // chunks 2*sub (even k) and 2*sub+1 (odd k), XOR-swizzled with the row
                uint8_t* rowp = bst + t * 1024 + row * 128;
                *reinterpret_cast<uint4*>(rowp + (((2 * sub) ^ row) << 4)) = ev;
                *reinterpret_cast<uint4*>(rowp + (((2 * sub + 1) ^ row) << 4)) = od;
            }
            // make the generic-proxy writes visible to the tensor core's async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&b_full[s]);
        }
    } else {
        // =============================== epilogue ====================================
        const int ew = warp - kEpiWarp0;   // 0..7
        const int mb = ew >> 2;            // token block of this warpgroup
        const int lq = warp & 3;           // TMEM lane quarter this warp may read
        const int tok = tok0 + mb * 128 + lq * 32 + lane;
        const bool active = mb < n_blocks;
        float acc[RP];
#pragma unroll
        for (int c = 0; c < RP; ++c)
            acc[c] = 0.f;
        // weight scales -> fp32 [G][RP] (column = row of the CTA), shared by all tokens
        if (!mbar_wait(scl_full, 0)) {
            if (lane == 0)
                fail();
        } else {
            float* wsf = reinterpret_cast<float*>(smem + S::kWsOff);
            const int et = ew * 32 + lane;
            for (int i = et; i < G * RP; i += kEpiWarps * 32) {
                const int g = i / RP, c = i - g * RP;
                float v = 0.f;
                if (c < r_tiles * 8) {
                    const int idx = ((c >> 3) * G + g) * 8 + (c & 7);
                    v = SCL16 ? __half2float(reinterpret_cast<const __half*>(
                                    smem + S::kSclRawOff)[idx])
                              : reinterpret_cast<const float*>(smem + S::kSclRawOff)[idx];
                }
                wsf[i] = v;
            }
        }
        // named barrier among the 8 epilogue warps only
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
        const float* wsf = reinterpret_cast<const float*>(smem + S::kWsOff);
        const bool has_tok = active && tok < a.m;
        float a_next = has_tok ? a.as[tok] : 0.f;  // group 0; later groups one ahead
        for (int g = 0; g < G; ++g) {
            const int b = g & 1, use = g >> 1;
            const float a_s = a_next;
            if (g + 1 < G && has_tok)
                a_next = a.as[(size_t)(g + 1) * a.m_pad + tok];
            if (*s_abort || !mbar_wait(&acc_full[b], use & 1)) {
                if (lane == 0)
                    fail();
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (active) {
                const uint32_t taddr =
                    tmem_base + ((uint32_t)(lq * 32) << 16) + (uint32_t)(b * 256 + mb * RP);
#pragma unroll
                for (int c0 = 0; c0 < RP; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + c0, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const float4 w4 = *reinterpret_cast<const float4*>(wsf + g * RP + c0 + i);
                        // the nibbles were left-aligned (16*q4): the sum is an exact
                        // multiple of 16
                        acc[c0 + i + 0] = __fmaf_rn((float)((int)r[i + 0] >> 4),
                                                    __fmul_rn(w4.x, a_s), acc[c0 + i + 0]);
                        acc[c0 + i + 1] = __fmaf_rn((float)((int)r[i + 1] >> 4),
                                                    __fmul_rn(w4.y, a_s), acc[c0 + i + 1]);
                        acc[c0 + i + 2] = __fmaf_rn((float)((int)r[i + 2] >> 4),
                                                    __fmul_rn(w4.z, a_s), acc[c0 + i + 2]);
                        acc[c0 + i + 3] = __fmaf_rn((float)((int)r[i + 3] >> 4),
                                                    __fmul_rn(w4.w, a_s), acc[c0 + i + 3]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_free[b]);
        }
        if (active && tok < a.m && !*s_abort) {
            const int n0 = blockIdx.x * a.rows_per_cta;
            float* dst = a.y + (size_t)tok * a.ldc + n0;
#pragma unroll
            for (int c = 0; c < RP; ++c) {
                if (c < R) {
                    float v = acc[c];
                    if (b2w4_act_applies(n0 + c, a.activation, a.act_n_begin, a.act_n_len, a.n))
                        v = gemm_activation(v, a.activation);
                    dst[c] = v;
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(512)
                     : "memory");
    }
}

template <int RP>
int launch_rp(b2w4_ctx* ctx, const GemmArgs& a, bool scl16, dim3 grid) {
    using S = Smem<RP>;
    auto kern = scl16 ? gemm_w4a8_tc_kernel<RP, true> : gemm_w4a8_tc_kernel<RP, false>;
    static bool configured[2] = {false, false};
    if (!configured[scl16]) {
        B2W4_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            S::kTotal));
        configured[scl16] = true;
    }
    kern<<<grid, kThreads, S::kTotal, ctx->stream>>>(a);
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}

}  // namespace

// Quantises the activations (separate launch), then runs the tensor-core kernel.
int b2w4_launch_gemm_tc(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                        float* y, int ldc, int m, int activation, int act_n_begin,
                        int act_n_len) {
    const int G = w->groups;
    if (G > 80)
        return b2w4_fail(ctx, B2W4_E_INVALID, "gemm: K=%d exceeds the scale staging (K<=10240)",
                         w->k);
    const int m_pad = (m + 127) / 128 * 128;
    void *qa = nullptr, *as = nullptr;
    int rc;
    if ((rc = b2w4_reserve(ctx, SCR_QA, (size_t)G * m_pad * 128, &qa)) != B2W4_OK ||
        (rc = b2w4_reserve(ctx, SCR_AS, sizeof(float) * (size_t)G * m_pad, &as)) != B2W4_OK)
        return rc;
    if ((rc = b2w4_launch_quantize_umma(ctx, x, lda, m, w->k, m_pad, static_cast<int8_t*>(qa),
                                        static_cast<float*>(as))) != B2W4_OK)
        return rc;
    // rows per CTA: one wave of CTAs over the SMs when the token extent is one block
    const int token_blocks = (m + 255) / 256;
    int per_sm = (w->tiles * token_blocks + ctx->sm_count - 1) / ctx->sm_count;
    int r_tiles = (per_sm + token_blocks - 1) / token_blocks;
    r_tiles = max(1, min(r_tiles, 10));  // at most 80 accumulator columns per thread
    const int R = r_tiles * 8;
    GemmArgs a;
    a.nib = reinterpret_cast<const uint8_t*>(w->nib);
    a.scl = w->scl;
    a.qa = static_cast<const int8_t*>(qa);
    a.as = static_cast<const float*>(as);
    a.y = y;
    a.status = ctx->flag_dev + 1;
    a.ldc = ldc;
    a.m = m;
    a.m_pad = m_pad;
    a.n = w->n;
    a.groups = G;
    a.tiles = w->tiles;
    a.rows_per_cta = R;
    a.activation = activation;
    a.act_n_begin = act_n_begin;
    a.act_n_len = act_n_len;
    dim3 grid((w->tiles + r_tiles - 1) / r_tiles, token_blocks);
    const bool scl16 = w->scales_fp16 != 0;
    if (R <= 32)
        return launch_rp<32>(ctx, a, scl16, grid);
    if (R <= 64)
        return launch_rp<64>(ctx, a, scl16, grid);
    return launch_rp<80>(ctx, a, scl16, grid);
}
