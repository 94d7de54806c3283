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
// Pipeline per 128-k group:
//   producer warp   bulk-copies (TMA engine) the pre-quantised, pre-swizzled int8
//                   activations of the group (one copy), and, once per chunk of kGC groups,
//                   the nibble stream of the CTA's row tiles (one copy per tile: a tile's
//                   groups are contiguous).  Issuing a bulk copy costs ~60 ns, so the
//                   number of copies per group, not their size, bounds the producer.
//   unpack warps    nibbles -> sign-extended int8 into the B operand's K-major,
//                   128-byte-swizzled layout; a 128-k group is exactly one swizzle row
//   MMA warp        one thread issues 4 x tcgen05.mma (K = 32 each) per token block into
//                   the group's TMEM accumulator, then tcgen05.commit
//   epilogue warps  tcgen05.ld the int32 sums (thread = token, columns = half of the
//                   CTA's weight rows) and run the fp32 chain in registers
// TMEM holds three to six group accumulators, so the MMAs run ahead of the fp32 chain.
// Every wait is bounded; on a timeout the kernel flags the status word and drains.
//
// The reference's rule for several rows (kernels/matmul_w4.cpp:785-901 with the per-32
// quantiser, kernels/matmul_quant.cpp:280-329) is the A32 form of the same kernel: one
// activation scale per 32 values, and per 32-k block b of a group
//   D_b = sum q4*q8 over the block;  y = fma(float(D_b), fp32(ws*as[g][b]), y)
// blocks ascending inside groups ascending.  A 32-k block is exactly one K = 32 MMA step, so
// the four steps of a group go to four accumulators of their own instead of adding up in
// one; the fp32 chain then has four times the steps per group and becomes the stage that
// paces the kernel, which is why that form runs one token block per CTA with all sixteen
// epilogue warps on the chain (four column ranges), and hands the accumulators over half a
// group at a time so that four to eight such halves fit in tensor memory.
#include "b200w4_internal.cuh"

namespace {

constexpr int kProducerWarp = 0;
constexpr int kMmaWarp = 1;
constexpr int kUnpackWarp0 = 2, kUnpackWarps = 4;
// four epilogue warpgroups: (token block, column half); a warp's TMEM lane quarter is its
// warp index mod 4
constexpr int kEpiWarp0 = 6, kEpiWarps = 16;
constexpr int kThreads = (kEpiWarp0 + kEpiWarps) * 32;  // 704
constexpr unsigned kSpinLimit = 1u << 24;
constexpr unsigned long long kWaitLimitCycles = 4000000000ull;  // SM cycles: about 2 s

struct GemmArgs {
    const uint8_t* nib;  // [tiles][G][512]
    const void* scl;     // [tiles][G][8] fp16|fp32
    const int8_t* qa;    // [G][m_pad][128] int8, 16-byte chunks swizzled by token%8
    const float* as;     // [G][m_pad]; per-32 rule: [G][m_pad][4], one scale per 32-k block
    float* y;
    int* status;
    int ldc, m, m_pad, n, groups, tiles;
    int rows_per_cta;  // R
    int activation, act_n_begin, act_n_len;
};

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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// The hint lets the hardware park the thread until the phase completes (or about 20 us pass)
// instead of having it spin through the issue slots the fp32 chain needs.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
// false when the iteration or the time limit runs out
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity))
        return true;
    const unsigned long long t0 = wait_clock();
    for (unsigned spins = 0; spins < kSpinLimit; ++spins) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((spins & 255) == 255 && wait_clock() - t0 > kWaitLimitCycles)
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
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, "
        "%11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
          "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
// float(d) for |d| < 2^22 without the conversion pipe: 0x4B400000 is 1.5 * 2^23, whose
// ulp is 1, so adding d to its bit pattern adds d to its value; the subtraction is exact.
// A group sum is at most 128 * 8 * 127 = 130048 in magnitude.
__device__ __forceinline__ float int_to_float_exact(int d) {
    return __fsub_rn(__int_as_float(0x4B400000 + d), 12582912.0f);
}

// Two fp32 lanes per instruction (sm_100's packed single-precision arithmetic): each lane is
// the IEEE round-to-nearest operation of its scalar counterpart, so the chain's bits do not
// change; the fp32 pipes, which pace the per-32 form, see half the instructions.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// float(d0), float(d1) as a pair, by the same route as int_to_float_exact
__device__ __forceinline__ uint64_t ints_to_float2_exact(uint32_t d0, uint32_t d1) {
    return sub2(pack2(__int_as_float(0x4B400000 + (int)d0), __int_as_float(0x4B400000 + (int)d1)),
                pack2(12582912.0f, 12582912.0f));
}

__device__ __noinline__ float gemm_activation(float v, int act) {
    return b2w4_activation(v, act);
}

constexpr int kGC = 4;      // groups per raw-weight chunk
constexpr int kBStages = 3; // unpacked-weight (B operand) ring

// shared-memory plan; operand buffers are 1024-byte aligned (swizzle atoms).  NB = token
// blocks of 128 per CTA: one block leaves room for a deeper activation ring.
template <int RP, int NB>
struct Smem {
    static constexpr int kAStages = NB == 2 ? 3 : 4;
    static constexpr int kRawSlots = NB == 2 ? 2 : 4;    // nibble chunks in flight
    static constexpr int kActStage = NB * 128 * 128;        // NB token blocks of 128 x 128 B
    static constexpr int kBStage = RP * 128;                // int8 weights, swizzled
    static constexpr int kRawSlot = (RP / 8) * kGC * 512;   // nibbles: [tile][kGC][512]
    static constexpr int kActOff = 0;
    static constexpr int kBOff = kActOff + kAStages * kActStage;
    static constexpr int kRawOff = kBOff + kBStages * kBStage;
    static constexpr int kWsOff = kRawOff + kRawSlots * kRawSlot;  // fp32 [G][RP], G <= kMaxG
    static constexpr int kMaxG = 80;  // K <= 10240
    static constexpr int kBarOff = kWsOff + kMaxG * RP * 4;
    static constexpr int kTotal = kBarOff + 512 + 1024;  // barriers, + slack to align the base
};

template <int RP, int NB, bool SCL16, bool A32>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a8_tc_kernel(const GemmArgs a) {
    static_assert(!A32 || NB == 1, "the per-32 form runs one token block per CTA");
    constexpr int kAStages = Smem<RP, NB>::kAStages;
    constexpr int kRawSlots = Smem<RP, NB>::kRawSlots;
    constexpr int kSplit = A32 ? 4 : 2;  // column ranges the epilogue warpgroups split
    constexpr int CH = RP / kSplit;      // accumulator columns per epilogue thread
    // The unit that the MMA warp hands to the epilogue: a group's accumulator (NB token
    // blocks of RP columns), or (A32) half a group -- two 32-k blocks with an accumulator of
    // RP columns each -- so that the MMAs of a group's second half, and of the next groups,
    // run while the chain still works on the first.  TMEM holds kAcc units (512 columns).
    constexpr int kAccCols = A32 ? 2 * RP : NB * RP;
    constexpr int kAccMax = A32 ? 8 : 6;
    constexpr int kAcc = 512 / kAccCols > kAccMax ? kAccMax : 512 / kAccCols;
    static_assert(kAcc >= 2, "no accumulator to run ahead into");
    static_assert(!A32 || CH == 8 || CH == 12 || CH == 16, "epilogue load widths");
    // With one token block and the per-128 rule only two of the four epilogue warpgroups
    // have accumulator rows; the other two unpack weights instead (the unpack stage bounds
    // the pipeline there).
    constexpr int kEpiActive = (NB == 2 || A32) ? kEpiWarps : kEpiWarps / 2;
    constexpr int kUnpackAll = kUnpackWarps + (kEpiWarps - kEpiActive);
    extern __shared__ uint8_t smem_raw[];
    // swizzle atoms need a 1024-byte aligned base
    uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
    using S = Smem<RP, NB>;
    const int G = a.groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = min(a.rows_per_cta, a.n - blockIdx.x * a.rows_per_cta);  // may be ragged
    const int r_tiles = (R + 7) / 8;
    const int tile0 = blockIdx.x * (a.rows_per_cta / 8);
    const int tok0 = blockIdx.y * (NB * 128);
    const int m_here = min(NB * 128, a.m - tok0);
    const int n_blocks = (m_here + 127) / 128;  // token blocks of 128 in this CTA

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
    uint64_t* act_full = bars;                  // [kAStages] activations of a group landed
    uint64_t* act_free = act_full + kAStages;   // [kAStages] MMAs that read them retired
    uint64_t* b_full = act_free + kAStages;     // [kBStages] unpack done
    uint64_t* b_free = b_full + kBStages;       // [kBStages] MMAs that read it retired
    uint64_t* raw_full = b_free + kBStages;     // [kRawSlots] nibble chunk landed
    uint64_t* raw_free = raw_full + kRawSlots;  // [kRawSlots] unpack warps are done with it
    uint64_t* acc_full = raw_free + kRawSlots;          // [kAcc] group accumulator complete
    uint64_t* acc_free = acc_full + kAcc;       // [kAcc] epilogue has read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + kAcc);
    volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&act_full[s], 1);
            mbar_init(&act_free[s], 1);
        }
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(&b_full[s], kUnpackAll);
            mbar_init(&b_free[s], 1);
        }
        for (int b = 0; b < kRawSlots; ++b) {
            mbar_init(&raw_full[b], 1);
            mbar_init(&raw_free[b], kUnpackAll);
        }
        for (int b = 0; b < kAcc; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_free[b], kEpiActive);
        }
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
        b2w4_report_timeout(a.status);
    };

    if (warp == kProducerWarp) {
        // =============================== producer ===================================
        // lane t copies row tile t's share of a nibble chunk, lane 31 a group's activations
        bool ok = true;
        for (int g = 0; g < G; ++g) {
            if (g % kGC == 0) {
                const int chunk = g / kGC, slot = chunk % kRawSlots, use = chunk / kRawSlots;
                const int gc = min(kGC, G - g);
                if (use > 0 && !mbar_wait(&raw_free[slot], (use - 1) & 1))
                    ok = false;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                if (lane == 0)
                    mbar_expect_tx(&raw_full[slot], (uint32_t)r_tiles * gc * 512);
                __syncwarp();
                if (lane < r_tiles)
                    bulk_g2s(smem + S::kRawOff + slot * S::kRawSlot + lane * (kGC * 512),
                             a.nib + ((size_t)(tile0 + lane) * G + g) * 512, (uint32_t)gc * 512,
                             &raw_full[slot]);
            }
            const int s = g % kAStages, round = g / kAStages;
            if (round > 0 && !mbar_wait(&act_free[s], (round - 1) & 1))
                ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if (lane == 31) {
                // only the 8-token atoms that hold real tokens are copied; the MMA reads
                // whatever the rest of the 128-token block holds and the epilogue ignores
                // those accumulator rows
                const uint32_t act_bytes = (uint32_t)((m_here + 7) / 8) * 1024;
                mbar_expect_tx(&act_full[s], act_bytes);
                bulk_g2s(smem + S::kActOff + s * S::kActStage,
                         a.qa + ((size_t)g * a.m_pad + tok0) * 128, act_bytes, &act_full[s]);
            }
        }
        if (!ok && lane == 0)
            fail();
    } else if (warp == kMmaWarp) {
        // =============================== MMA issue ===================================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(RP);
            for (int g = 0; g < G; ++g) {
                const int sa = g % kAStages, ra = g / kAStages;
                const int sb = g % kBStages, rb = g / kBStages;
                if (!mbar_wait(&b_full[sb], rb & 1) || !mbar_wait(&act_full[sa], ra & 1)) {
                    fail();
                    break;
                }
                const uint32_t b_addr = smem_u32(smem + S::kBOff + sb * S::kBStage);
                bool ok = true;
                if constexpr (A32) {
                    const uint32_t a_addr = smem_u32(smem + S::kActOff + sa * S::kActStage);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {  // blocks 2h and 2h + 1: one unit
                        const int u = 2 * g + h, b = u % kAcc, use = u / kAcc;
                        if (use > 0 && !mbar_wait(&acc_free[b], (use - 1) & 1)) {
                            ok = false;
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {  // a K = 32 step = a 32-k block
                            const int j = 2 * h + jj;
                            umma_i8(tmem_base + (uint32_t)(b * kAccCols + jj * RP),
                                    umma_desc_k_sw128(a_addr + j * 32),
                                    umma_desc_k_sw128(b_addr + j * 32), idesc, 0u);
                        }
                        umma_commit(&acc_full[b]);  // the two blocks' sums are complete
                    }
                } else {
                    const int b = g % kAcc, use = g / kAcc;
                    if (use > 0 && !mbar_wait(&acc_free[b], (use - 1) & 1))
                        ok = false;
                    if (ok) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        for (int mb = 0; mb < n_blocks; ++mb) {
                            const uint32_t a_addr = smem_u32(smem + S::kActOff +
                                                             sa * S::kActStage + mb * 128 * 128);
                            const uint32_t d = tmem_base + (uint32_t)(b * kAccCols + mb * RP);
#pragma unroll
                            for (int j = 0; j < 4; ++j)  // four K = 32 steps inside the
                                                         // swizzle row, summed in one accumulator
                                umma_i8(d, umma_desc_k_sw128(a_addr + j * 32),
                                        umma_desc_k_sw128(b_addr + j * 32), idesc,
                                        j > 0 ? 1u : 0u);
                        }
                        umma_commit(&acc_full[b]);  // the group's sums are complete
                    }
                }
                if (!ok) {
                    fail();
                    break;
                }
                // a commit fires when every MMA issued so far has retired
                umma_commit(&act_free[sa]);  // the activation stage may be refilled
                umma_commit(&b_free[sb]);    // the unpacked weights may be overwritten
            }
        }
    } else if (warp < kEpiWarp0 || warp >= kEpiWarp0 + kEpiActive) {
        // =============================== unpack ======================================
        const int uw = warp < kEpiWarp0 ? warp - kUnpackWarp0
                                        : kUnpackWarps + (warp - kEpiWarp0 - kEpiActive);
        const int ut = uw * 32 + lane;
        for (int g = 0; g < G; ++g) {
            const int chunk = g / kGC, slot = chunk % kRawSlots, cuse = chunk / kRawSlots;
            const int gi = g % kGC;
            const int sb = g % kBStages, rb = g / kBStages;
            bool ok = !*s_abort;
            if (ok && gi == 0)
                ok = mbar_wait(&raw_full[slot], cuse & 1);   // the chunk's nibbles landed
            if (ok && rb > 0)
                ok = mbar_wait(&b_free[sb], (rb - 1) & 1);   // MMAs left this B stage
            if (!ok) {
                if (lane == 0)
                    fail();
                break;
            }
            // raw slot: [tile][kGC groups][32 chunks of 16 B]
            const uint4* raw =
                reinterpret_cast<const uint4*>(smem + S::kRawOff + slot * S::kRawSlot) + gi * 32;
            uint8_t* bst = smem + S::kBOff + sb * S::kBStage;
            // chunk c of tile t: sub = c/8, row = c%8 -> 32 k of weight row t*8+row
            for (int c = ut; c < r_tiles * 32; c += kUnpackAll * 32) {
                const int t = c >> 5, sub = (c >> 3) & 3, row = c & 7;
                const uint4 w = raw[t * (kGC * 32) + (c & 31)];
                // low nibbles = even k, high nibbles = odd k; a nibble with bit 3 set is
                // negative: OR in 0xF0 (0x08 * 30 = 0xF0, no carry between bytes)
                uint4 ev, od;
                {
                    uint32_t t;
                    t = w.x & 0x0F0F0F0Fu; ev.x = t | ((t & 0x08080808u) * 30u);
                    t = (w.x >> 4) & 0x0F0F0F0Fu; od.x = t | ((t & 0x08080808u) * 30u);
                    t = w.y & 0x0F0F0F0Fu; ev.y = t | ((t & 0x08080808u) * 30u);
                    t = (w.y >> 4) & 0x0F0F0F0Fu; od.y = t | ((t & 0x08080808u) * 30u);
                    t = w.z & 0x0F0F0F0Fu; ev.z = t | ((t & 0x08080808u) * 30u);
                    t = (w.z >> 4) & 0x0F0F0F0Fu; od.z = t | ((t & 0x08080808u) * 30u);
                    t = w.w & 0x0F0F0F0Fu; ev.w = t | ((t & 0x08080808u) * 30u);
                    t = (w.w >> 4) & 0x0F0F0F0Fu; od.w = t | ((t & 0x08080808u) * 30u);
                }
                // weight row r = t*8+row: atom t (1024 B), row `row` (128 B), 16-byte
                // chunks 2*sub (even k) and 2*sub+1 (odd k), XOR-swizzled with the row
                uint8_t* rowp = bst + t * 1024 + row * 128;
                *reinterpret_cast<uint4*>(rowp + (((2 * sub) ^ row) << 4)) = ev;
                *reinterpret_cast<uint4*>(rowp + (((2 * sub + 1) ^ row) << 4)) = od;
            }
            // make the generic-proxy writes visible to the tensor core's async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&b_full[sb]);
                if (gi == kGC - 1 || g == G - 1)
                    mbar_arrive(&raw_free[slot]);  // this warp is done with the chunk
            }
        }
    } else {
        // =============================== epilogue ====================================
        const int ew = warp - kEpiWarp0;       // 0..15
        const int eg = ew >> 2;                // warpgroup
        const int mb = eg % NB;                // its token block
        const int ch = eg / NB;                // its column half
        const int lq = warp & 3;               // TMEM lane quarter this warp may read
        const int tok = tok0 + mb * 128 + lq * 32 + lane;
        // a warp whose 32 tokens all lie past the last row has no chain to run
        const bool active = ch < kSplit && mb < n_blocks && mb * 128 + lq * 32 < m_here;
        float acc[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c)
            acc[c] = 0.f;
        // weight scales -> fp32 [G][RP] (column = row of the CTA), shared by all tokens
        {
            float* wsf = reinterpret_cast<float*>(smem + S::kWsOff);
            const int et = ew * 32 + lane;
            for (int i = et; i < G * RP; i += kEpiActive * 32) {
                const int g = i / RP, c = i - g * RP;
                float v = 0.f;
                if (c < r_tiles * 8) {
                    const size_t idx = ((size_t)(tile0 + (c >> 3)) * G + g) * 8 + (c & 7);
                    v = SCL16 ? __half2float(reinterpret_cast<const __half*>(a.scl)[idx])
                              : reinterpret_cast<const float*>(a.scl)[idx];
                }
                wsf[i] = v;
            }
        }
        // named barrier among the epilogue warps only
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiActive * 32) : "memory");
        const float* wsf = reinterpret_cast<const float*>(smem + S::kWsOff) + ch * CH;
        const bool has_tok = active && tok < a.m;
        if constexpr (A32) {
            // the token's four block scales of a group are one 16-byte load, fetched two
            // groups ahead (a group's chain is long enough to cover the load)
            const float4* as4 = reinterpret_cast<const float4*>(a.as);
            auto load_as = [&](int g) {
                return (has_tok && g < G) ? as4[(size_t)g * a.m_pad + tok]
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            };
            float4 a0 = load_as(0), a1 = load_as(1);
            uint64_t acc2[CH / 2];  // the chain values, columns (2i, 2i + 1) side by side
#pragma unroll
            for (int i = 0; i < CH / 2; ++i)
                acc2[i] = 0ull;
            bool live = true;
            for (int g = 0; g < G && live; ++g) {
                const float asv[4] = {a0.x, a0.y, a0.z, a0.w};
                a0 = a1;
                a1 = load_as(g + 2);
#pragma unroll
                for (int h = 0; h < 2; ++h) {  // the group's two units: blocks 2h, 2h + 1
                    const int u = 2 * g + h, b = u % kAcc, use = u / kAcc;
                    if (*s_abort || !mbar_wait(&acc_full[b], use & 1)) {
                        if (lane == 0)
                            fail();
                        live = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (active) {
                        const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) +
                                               (uint32_t)(b * kAccCols + ch * CH);
                        uint32_t r[2][CH];
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {  // the widest loads that tile CH
                            const uint32_t tb = taddr + jj * RP;
                            if constexpr (CH == 16) {
                                tmem_ld16(tb, *reinterpret_cast<uint32_t(*)[16]>(&r[jj][0]));
                            } else {
                                tmem_ld8(tb, *reinterpret_cast<uint32_t(*)[8]>(&r[jj][0]));
                                if constexpr (CH == 12)
                                    tmem_ld4(tb + 8,
                                             *reinterpret_cast<uint32_t(*)[4]>(&r[jj][8]));
                            }
                        }
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int c = 0; c < CH; c += 4) {
                            const float4 w4 =
                                *reinterpret_cast<const float4*>(wsf + g * RP + c);
                            const uint64_t w_lo = pack2(w4.x, w4.y), w_hi = pack2(w4.z, w4.w);
#pragma unroll
                            for (int jj = 0; jj < 2; ++jj) {  // blocks in ascending order
                                const float s_b = asv[2 * h + jj];
                                const uint64_t s2 = pack2(s_b, s_b);
                                acc2[c / 2] = fma2(ints_to_float2_exact(r[jj][c], r[jj][c + 1]),
                                                   mul2(w_lo, s2), acc2[c / 2]);
                                acc2[c / 2 + 1] =
                                    fma2(ints_to_float2_exact(r[jj][c + 2], r[jj][c + 3]),
                                         mul2(w_hi, s2), acc2[c / 2 + 1]);
                            }
                        }
                    }
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&acc_free[b]);
                }
            }
#pragma unroll
            for (int i = 0; i < CH / 2; ++i)
                unpack2(acc2[i], acc[2 * i], acc[2 * i + 1]);
        } else {
            // the token's activation scales are fetched four groups ahead: a global load takes
            // about as long as a whole group, so a shorter distance would pace the loop
            auto load_as = [&](int g) {
                return (has_tok && g < G) ? a.as[(size_t)g * a.m_pad + tok] : 0.f;
            };
            float a0 = load_as(0), a1 = load_as(1), a2 = load_as(2), a3 = load_as(3);
            // Two token blocks: sixteen warps share the chain and packed arithmetic pays.  One
            // block: eight warps with twice the columns each, where the register pairs it
            // needs cost more than the instructions it saves.
            constexpr bool kPacked = NB == 2;
            uint64_t acc2[kPacked ? CH / 2 : 1];  // chain values, columns (2i, 2i + 1) paired
#pragma unroll
            for (int i = 0; i < (kPacked ? CH / 2 : 1); ++i)
                acc2[i] = 0ull;
            for (int g = 0; g < G; ++g) {
                const int b = g % kAcc, use = g / kAcc;
                const float a_s = a0;
                const uint64_t as2 = pack2(a0, a0);
                a0 = a1;
                a1 = a2;
                a2 = a3;
                a3 = load_as(g + 4);
                if (*s_abort || !mbar_wait(&acc_full[b], use & 1)) {
                    if (lane == 0)
                        fail();
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (active) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(lq * 32) << 16) +
                                           (uint32_t)(b * kAccCols + mb * RP + ch * CH);
                    // columns are requested in batches of up to 24 before one wait: the TMEM read
                    // latency is paid once or twice per group, not once per 8 columns
                    constexpr int kBatch = 24;
#pragma unroll
                    for (int b0 = 0; b0 < CH; b0 += kBatch) {
                        constexpr int kMaxB = kBatch;
                        uint32_t r[kMaxB];
#pragma unroll
                        for (int c0 = 0; c0 < kMaxB; c0 += 8)
                            if (b0 + c0 < CH)
                                tmem_ld8(taddr + b0 + c0, *reinterpret_cast<uint32_t(*)[8]>(&r[c0]));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int c = 0; c < kMaxB; c += 4) {
                            if (b0 + c < CH) {
                                const float4 w4 =
                                    *reinterpret_cast<const float4*>(wsf + g * RP + b0 + c);
                                if constexpr (kPacked) {
                                    acc2[(b0 + c) / 2] =
                                        fma2(ints_to_float2_exact(r[c], r[c + 1]),
                                             mul2(pack2(w4.x, w4.y), as2), acc2[(b0 + c) / 2]);
                                    acc2[(b0 + c) / 2 + 1] = fma2(
                                        ints_to_float2_exact(r[c + 2], r[c + 3]),
                                        mul2(pack2(w4.z, w4.w), as2), acc2[(b0 + c) / 2 + 1]);
                                } else {
                                    acc[b0 + c + 0] =
                                        __fmaf_rn(int_to_float_exact((int)r[c + 0]),
                                                  __fmul_rn(w4.x, a_s), acc[b0 + c + 0]);
                                    acc[b0 + c + 1] =
                                        __fmaf_rn(int_to_float_exact((int)r[c + 1]),
                                                  __fmul_rn(w4.y, a_s), acc[b0 + c + 1]);
                                    acc[b0 + c + 2] =
                                        __fmaf_rn(int_to_float_exact((int)r[c + 2]),
                                                  __fmul_rn(w4.z, a_s), acc[b0 + c + 2]);
                                    acc[b0 + c + 3] =
                                        __fmaf_rn(int_to_float_exact((int)r[c + 3]),
                                                  __fmul_rn(w4.w, a_s), acc[b0 + c + 3]);
                                }
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&acc_free[b]);
            }
            if constexpr (kPacked) {
#pragma unroll
                for (int i = 0; i < CH / 2; ++i)
                    unpack2(acc2[i], acc[2 * i], acc[2 * i + 1]);
            }
        }
        // Output: a thread holds one token's CH columns, which lie CH*4 bytes apart from the
        // next token's in y.  Stage the warp's 32 x CH block in shared memory (the operand
        // ring is idle: the last accumulator was complete, so every MMA and copy has
        // retired) and store token rows with the lanes running along the columns.
        if (active && !*s_abort) {
            constexpr int SP = CH + 4;  // row pitch: 16-byte aligned, conflict-free float4s
            float* stage = reinterpret_cast<float*>(smem + S::kActOff) + ew * (32 * SP);
            const int n0 = blockIdx.x * a.rows_per_cta + ch * CH;
#pragma unroll
            for (int c = 0; c < CH; c += 4) {
                float4 v = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
                if (a.activation != B2W4_NONE) {
                    float* e = &v.x;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (b2w4_act_applies(n0 + c + i, a.activation, a.act_n_begin,
                                             a.act_n_len, a.n))
                            e[i] = gemm_activation(e[i], a.activation);
                }
                *reinterpret_cast<float4*>(stage + lane * SP + c) = v;
            }
            __syncwarp();
            const int tok_w = tok0 + mb * 128 + lq * 32;  // first token of this warp
            const int rows_w = min(32, a.m - tok_w);
            const bool vec_ok = (a.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0;
            constexpr int V = CH / 4;  // float4s per token row
#pragma unroll 4
            for (int i = lane; i < rows_w * V; i += 32) {
                const int r = i / V, c = (i - r * V) * 4;
                const float4 v = *reinterpret_cast<const float4*>(stage + r * SP + c);
                float* dst = a.y + (size_t)(tok_w + r) * a.ldc + n0 + c;
                const int left = R - (ch * CH + c);  // valid columns from here on
                if (left >= 4 && vec_ok) {
                    *reinterpret_cast<float4*>(dst) = v;
                } else {
                    if (left > 0) dst[0] = v.x;
                    if (left > 1) dst[1] = v.y;
                    if (left > 2) dst[2] = v.z;
                    if (left > 3) dst[3] = v.w;
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

template <int RP, int NB, bool A32 = false>
int launch_rp(b2w4_ctx* ctx, const GemmArgs& a, bool scl16, dim3 grid) {
    using S = Smem<RP, NB>;
    auto kern = scl16 ? gemm_w4a8_tc_kernel<RP, NB, true, A32>
                      : gemm_w4a8_tc_kernel<RP, NB, false, A32>;
    static b2w4_smem_optin configured[2];  // per instantiation and device
    B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, kern, S::kTotal, configured[scl16]));
    kern<<<grid, kThreads, S::kTotal, ctx->stream>>>(a);
    ctx->launches++;
    B2W4_CUDA(ctx, cudaGetLastError());
    return B2W4_OK;
}

template <int NB>
int launch_nb(b2w4_ctx* ctx, const GemmArgs& a, bool scl16, dim3 grid, int rows) {
    if (rows <= 32)
        return launch_rp<32, NB>(ctx, a, scl16, grid);
    if (rows <= 64)
        return launch_rp<64, NB>(ctx, a, scl16, grid);
    return launch_rp<80, NB>(ctx, a, scl16, grid);
}

// The per-32 form: one token block per CTA, 32 / 48 / 64 accumulator columns per block.
int launch_a32(b2w4_ctx* ctx, const GemmArgs& a, bool scl16, dim3 grid, int rows) {
    if (rows <= 32)
        return launch_rp<32, 1, true>(ctx, a, scl16, grid);
    if (rows <= 48)
        return launch_rp<48, 1, true>(ctx, a, scl16, grid);
    return launch_rp<64, 1, true>(ctx, a, scl16, grid);
}

// Rows per CTA for the per-32 form.  The fp32 chain paces a CTA, so its time grows with the
// accumulator columns of its instantiation (plus a fixed part per group); the launch takes
// as many rounds as the CTAs need on the SMs.  Pick the tile count with the least product.
int a32_row_tiles(int tiles, int token_blocks, int sm_count) {
    int best = 1;
    long best_cost = -1;
    for (int r = 1; r <= 8; ++r) {
        const long ctas = (long)((tiles + r - 1) / r) * token_blocks;
        const long rounds = (ctas + sm_count - 1) / sm_count;
        const int cols = r <= 4 ? 32 : r <= 6 ? 48 : 64;
        const long cost = rounds * (cols + 12);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = r;
        }
    }
    return best;
}

}  // namespace

// Quantises the activations (separate launch), then runs the tensor-core kernel.
int b2w4_launch_gemm_tc(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                        float* y, int ldc, int m, int act_rule, int activation, int act_n_begin,
                        int act_n_len) {
    const int G = w->groups;
    const bool a32 = act_rule == B2W4_ACT_G32;
    const int spg = a32 ? 4 : 1;  // activation scales per group
    if (G > 80)
        return b2w4_fail(ctx, B2W4_E_INVALID, "gemm: K=%d exceeds the scale staging (K<=10240)",
                         w->k);
    const int m_pad = (m + 127) / 128 * 128;
    void *qa = nullptr, *as = nullptr;
    int rc;
    if ((rc = b2w4_reserve(ctx, SCR_QA, (size_t)G * m_pad * 128, &qa)) != B2W4_OK ||
        (rc = b2w4_reserve(ctx, SCR_AS, sizeof(float) * (size_t)G * m_pad * spg, &as)) !=
            B2W4_OK)
        return rc;
    if ((rc = b2w4_launch_quantize_umma(ctx, x, lda, m, w->k, m_pad, act_rule,
                                        static_cast<int8_t*>(qa), static_cast<float*>(as))) !=
        B2W4_OK)
        return rc;
    // rows per CTA: one wave of CTAs over the SMs when the token extent is one block
    const int nb = (m > 128 && !a32) ? 2 : 1;  // token blocks of 128 per CTA
    const int token_blocks = (m + nb * 128 - 1) / (nb * 128);
    int per_sm = (w->tiles * token_blocks + ctx->sm_count - 1) / ctx->sm_count;
    int r_tiles = (per_sm + token_blocks - 1) / token_blocks;
    r_tiles = max(1, min(r_tiles, 10));  // at most 80 accumulator columns per thread
    if (a32)
        r_tiles = a32_row_tiles(w->tiles, token_blocks, ctx->sm_count);
    const int R = r_tiles * 8;
    GemmArgs a;
    a.nib = reinterpret_cast<const uint8_t*>(w->nib);
    a.scl = w->scl;
    a.qa = static_cast<const int8_t*>(qa);
    a.as = static_cast<const float*>(as);
    a.y = y;
    a.status = ctx->status_dev;
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
    if (a32)
        return launch_a32(ctx, a, scl16, grid, R);
    return nb == 2 ? launch_nb<2>(ctx, a, scl16, grid, R) : launch_nb<1>(ctx, a, scl16, grid, R);
}

// ---------------------------------------------------------------------------------------
// b2w4_matmul_static_scratch: the tensor-core matmul for callers that may not allocate.
//
// The tensor-core kernel reads activations that a first kernel has quantised into device
// memory.  b2w4_matmul takes that buffer from a grow-on-demand cudaMalloc pool; this variant
// takes it from the fixed array below, so the call issues no cudaMalloc / cudaFree and no
// other allocating routine.  The array is part of the library image: every GPU on which the
// library is used holds these 2.6 MiB until the process exits.
//
// Limits: 5 <= M <= 256 activation rows and K <= 10240 (80 groups of 128).
// The array is shared by every call and keeps the last call's contents.  Nothing in it has
// to start at zero: the quantiser rewrites every (group, row < M) entry each call, and rows
// M..M_pad only feed accumulator lanes that are never read.  Two calls that overlap on the
// GPU (different streams, or different contexts on one device) race on it.
namespace {

constexpr int kStaticMaxRows = 256;
constexpr int kStaticMaxGroups = 80;
constexpr size_t kStaticCodeBytes = (size_t)kStaticMaxGroups * kStaticMaxRows * 128;
constexpr size_t kStaticScaleBytes = sizeof(float) * kStaticMaxGroups * kStaticMaxRows;
constexpr int kStaticMaxDevices = 64;

static __device__ __align__(256) uint8_t g_static_scratch[kStaticCodeBytes + kStaticScaleBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, per device.
void* g_static_scratch_addr[kStaticMaxDevices] = {nullptr};

}  // namespace

extern "C" int b2w4_matmul_static_scratch(b2w4_ctx* ctx, const b2w4_weight* w,
                                          const float* x_dev, int lda, float* y_dev, int ldc,
                                          int m, int activation, int act_n_begin,
                                          int act_n_len) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!w || !x_dev || !y_dev)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_static_scratch: null weight or tensor");
    if (m < 5 || m > kStaticMaxRows)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "matmul_static_scratch: M=%d is outside 5..%d (the fixed scratch "
                         "holds %d rows; use b2w4_matmul for other sizes)",
                         m, kStaticMaxRows, kStaticMaxRows);
    if (w->groups > kStaticMaxGroups)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "matmul_static_scratch: K=%d exceeds %d (the fixed scratch holds %d "
                         "groups of 128)", w->k, kStaticMaxGroups * 128, kStaticMaxGroups);
    if (lda < w->k || ldc < w->n)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_static_scratch: lda=%d (k=%d) ldc=%d (n=%d)",
                         lda, w->k, ldc, w->n);
    if (activation < B2W4_NONE || activation > B2W4_RELU_SQUARED)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_static_scratch: unknown activation %d",
                         activation);
    if (ctx->device < 0 || ctx->device >= kStaticMaxDevices)
        return b2w4_fail(ctx, B2W4_E_INVALID, "matmul_static_scratch: device index %d",
                         ctx->device);
    // one-time set-up per device, done by the first call on that device (so that first call
    // should be made before any stream capture begins)
    if (!g_static_scratch_addr[ctx->device]) {
        int current = -1;
        B2W4_CUDA(ctx, cudaGetDevice(&current));
        if (current != ctx->device)
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "matmul_static_scratch: device %d must be current (it is %d)",
                             ctx->device, current);
        void* addr = nullptr;
        B2W4_CUDA(ctx, cudaGetSymbolAddress(&addr, g_static_scratch));
        g_static_scratch_addr[ctx->device] = addr;
    }
    uint8_t* base = static_cast<uint8_t*>(g_static_scratch_addr[ctx->device]);
    int8_t* qa = reinterpret_cast<int8_t*>(base);
    float* as = reinterpret_cast<float*>(base + kStaticCodeBytes);
    const int G = w->groups;
    const int m_pad = (m + 127) / 128 * 128;
    int rc = b2w4_launch_quantize_umma(ctx, x_dev, lda, m, w->k, m_pad, B2W4_ACT_G128, qa, as);
    if (rc != B2W4_OK)
        return rc;
    const int nb = m > 128 ? 2 : 1;
    const int token_blocks = 1;  // M <= 256: one CTA row of token blocks
    int r_tiles = (w->tiles + ctx->sm_count - 1) / ctx->sm_count;
    r_tiles = max(1, min(r_tiles, 10));
    GemmArgs a;
    a.nib = reinterpret_cast<const uint8_t*>(w->nib);
    a.scl = w->scl;
    a.qa = qa;
    a.as = as;
    a.y = y_dev;
    a.status = ctx->status_dev;
    a.ldc = ldc;
    a.m = m;
    a.m_pad = m_pad;
    a.n = w->n;
    a.groups = G;
    a.tiles = w->tiles;
    a.rows_per_cta = r_tiles * 8;
    a.activation = activation;
    a.act_n_begin = act_n_begin;
    a.act_n_len = act_n_len;
    dim3 grid((w->tiles + r_tiles - 1) / r_tiles, token_blocks);
    const bool scl16 = w->scales_fp16 != 0;
    return nb == 2 ? launch_nb<2>(ctx, a, scl16, grid, r_tiles * 8)
                   : launch_nb<1>(ctx, a, scl16, grid, r_tiles * 8);
}
