// W4G128 x int8 GEMV for one activation row (decode): HBM-bound weight streaming.
// (Two and more rows go to the tensor-instruction kernel in gemv_mma.cu; the row-count
// template parameter below is kept at 1.)
//
// Arithmetic = the reference's NEON W4A8 GEMV (kernels/matmul_w4.cpp:211-295) applied row
// by row, with the activation quantiser (kernels/matmul_quant.cpp:578-641) fused in:
//   per 128-k group g:  D = sum q4*q8 (int32);  y = fma(float(D), fp32(ws*as[g]), y)
// groups ascending.  The per-32 rule (kernels/matmul_w4.cpp:785-901) is the same loop
// with one D and one activation scale per 32-k block.
//
// Data movement.  A CTA owns `tpc` consecutive 8-row tiles; their nibble stream
// (tpc * K/128 * 512 bytes, contiguous in the nibble plane) and their scales are brought
// into shared memory by bulk async copies (cp.async.bulk, one per tile, completion on an
// mbarrier per tile) that one thread issues as the first thing the kernel does.  Nothing
// is staged in registers, so the whole weight of a launch is in flight within the first
// microsecond.  A CTA uses under half of an SM's shared memory, registers and threads: two
// CTAs are resident per SM, and with programmatic dependent launch the CTAs of the NEXT
// kernel in the stream become resident and start their copies while this kernel still
// computes.  Weights never depend on the previous kernel's output; only the activation
// read waits on the predecessor (griddepcontrol.wait).
//
// Math, phase 1.  An item is four consecutive groups of one tile; warp w takes items w,
// w+W, ... of the CTA in a short, not unrolled loop (the kernel is latency-sensitive and
// runs a few microseconds: its code has to stay resident in the instruction cache).  In an
// item, lane (gl = lane/8, row = lane%8) owns group gl for one weight row, reads its four
// 16-byte chunks (a quarter warp reads 128 contiguous bytes: no bank conflicts) and the
// even/odd de-interleaved int8 activations (broadcast), and gets the group's int32 sum from
// 32 dp4a with no cross-lane reduction.  A weight word w holds 8 nibbles; two logic
// instructions split it without shifts:
//   hi = w & 0xF0F0F0F0                  odd k, bytes = 16*q as int8
//   lo = (w ^ 0x08080808) & 0x0F0F0F0F   even k, bytes = q+8 as uint8
// sum(q*a) = dp4a.u8.s8(lo, a_even) - 8*sum(a_even) + dp4a.s8.s8(hi, a_odd)/16: the last
// term is an exact multiple of 16 (like the NEON kernel's sdot on left-aligned nibbles and
// its fixed-point convert) and sum(a_even) comes from the quantiser, one per group.  The
// integer sum (as a float: exact) and the scale product fp32(ws*as) go to shared memory.
// Phase 2, after one barrier: one thread per (tile, weight row, activation row) runs the
// order-sensitive chain of fused multiply-adds over the groups in ascending order.
#include "b200w4_internal.cuh"

namespace {

// one activation row: 16 warps of <= 64 registers; more rows keep more integer sums in
// registers: 8 warps of <= 128 registers.  Either way two CTAs share an SM.
__host__ __device__ constexpr int gemv_warps(int mt) { return mt == 1 ? 16 : 8; }
constexpr int kMaxTpc = 16;
constexpr unsigned kSpinLimit = 1u << 22;  // bounded waits: give up, flag, return
constexpr unsigned long long kWaitLimitCycles = 4000000000ull;  // SM cycles: about 2 s
constexpr int kTpGatherThreads = 256;

struct GemvArgs {
    const uint4* nib;
    const void* scl;
    const float* x;
    float* y;
    int32_t* sums;  // optional [m][n][groups or 4*groups]
    int* status;    // device status word: set when a bounded wait gives up
    int lda, ldc, m, n, k, groups, tiles;
    int tpc;       // tiles per CTA
    int ipt_magic; // item / items-per-tile == (item * ipt_magic) >> 16, or 0: divide
    int d_stride;  // ints between the integer sums of consecutive tiles (padded)
    int activation, act_n_begin, act_n_len;
    b2w4_tp_args tp;  // tensor-parallel epilogue (world == 0: off)
    b2w4_top1_args top1;  // greedy-token epilogue (MODE 2)
};
// Kernel modes: plain, with the int32 group sums written out, with the greedy-token epilogue.
constexpr int kModePlain = 0, kModeSums = 1, kModeTop1 = 2;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
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
// global -> shared bulk copy (the TMA engine, untiled form); both addresses 16-byte
// aligned, size a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// SM cycle counter: cheap to read (the global nanosecond timer is not), good enough to
// bound a wait
__device__ __forceinline__ unsigned long long wait_clock() {
    return (unsigned long long)clock64();
}
// Waits for phase 0 of an mbarrier; false when the iteration or the time limit runs out.
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

// uint8 x int8 dot of four byte pairs
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// the fused activations carry fp64 exp / tanh code: keep one out-of-line copy
__device__ __noinline__ float gemv_activation(float v, int act) {
    return b2w4_activation(v, act);
}

template <int MT, bool SCL16, bool A32, int MODE>
__global__ void __launch_bounds__(gemv_warps(MT) * 32, 2)
gemv_w4a8_kernel(const GemvArgs a) {
    constexpr int kWarps = gemv_warps(MT);
    constexpr int kThreads = kWarps * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int SPG = A32 ? 4 : 1;  // integer sums per group
    const int G = a.groups, K = a.k;
    const int tile_bytes = G * 512;
    const int scl_tile_bytes = G * 8 * (SCL16 ? 2 : 4);
    // shared-memory carve-up (every region a multiple of 16 bytes)
    uint8_t* s_w = smem;                                   // [tpc][G][512]
    uint8_t* s_scl = s_w + (size_t)a.tpc * tile_bytes;     // [tpc][G][8] fp16|fp32
    uint4* s_qa = reinterpret_cast<uint4*>(s_scl + (size_t)a.tpc * scl_tile_bytes);  // [MT][K]
    float* s_as = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_qa) + (size_t)MT * K);
    // per (tile, group, [32-block], activation row, weight row): the integer sum as a float
    // (exact: |sum| < 2^24) and the scale product it is multiplied with
    int* s_es = reinterpret_cast<int*>(s_as + MT * G * SPG);  // -8 * sum of the even-k codes
    float* s_d = reinterpret_cast<float*>(s_es + MT * G * SPG);  // [tpc][G][SPG][MT][8] + pad
    float* s_sc = s_d + (size_t)a.tpc * a.d_stride;        // same shape
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(
        (reinterpret_cast<uintptr_t>(s_sc + (size_t)a.tpc * a.d_stride) + 7) & ~uintptr_t(7));

    constexpr bool SUMS = MODE == kModeSums;
    __shared__ unsigned long long s_top1[8];
    if (MODE == kModeTop1 && threadIdx.x < 8)
        s_top1[threadIdx.x] = 0ull;  // barriers follow before the epilogue uses it
    unsigned long long top1_best = 0ull;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gl = lane >> 3, row = lane & 7;
    const int tile0 = blockIdx.x * a.tpc;
    const int ntile = min(a.tpc, a.tiles - tile0);

    // Let the next kernel in the stream become resident and start its own weight copies.
    b2w4_pdl_launch_dependents();

    // ---- weight stream: issued before anything else, independent of the predecessor ----
    if (warp == 0) {
        // lane t arms and fills tile t's barrier; lane ntile does the scales
        if (lane <= ntile)
            mbar_init(&s_bar[lane], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
        if (lane < ntile) {
            mbar_expect_tx(&s_bar[lane], (uint32_t)tile_bytes);
            bulk_g2s(s_w + (size_t)lane * tile_bytes,
                     reinterpret_cast<const uint8_t*>(a.nib) +
                         (size_t)(tile0 + lane) * tile_bytes,
                     (uint32_t)tile_bytes, &s_bar[lane]);
        } else if (lane == ntile) {
            mbar_expect_tx(&s_bar[ntile], (uint32_t)(ntile * scl_tile_bytes));
            bulk_g2s(s_scl,
                     reinterpret_cast<const uint8_t*>(a.scl) + (size_t)tile0 * scl_tile_bytes,
                     (uint32_t)(ntile * scl_tile_bytes), &s_bar[ntile]);
        }
    }

    b2w4_pdl_wait();  // activations come from the previous kernel

    // Tensor-parallel exchange number: one more than the count of completed gathers, kept in
    // the first word of this rank's staging buffer (written by the gather kernel).
    unsigned tp_exchange = 0;
    if (a.tp.world != 0)
        tp_exchange =
            *reinterpret_cast<const volatile unsigned*>(a.tp.stage_peer[a.tp.rank]) + 1u;

    // ---- fused activation quantiser: one half-warp per (activation row, group) ----------
    // lane h of the half-warp holds k = 8h .. 8h+7 of the group (a quarter of a 32-block)
    {
        const int half = lane >> 4, h = lane & 15;
        const int n_q = a.m * G;
        const bool vec_x = (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (a.lda & 3) == 0;
        // the trip count is the same for both halves of the warp (the shuffles below name
        // all 32 lanes); a half without an item works on zeros and stores nothing
#pragma unroll 1
        for (int base = warp * 2; base < n_q; base += kWarps * 2) {
            const int item = base + half;
            const bool live = item < n_q;
            const int mi = live ? item / G : 0, g = live ? item % G : 0;
            const float* src = a.x + (size_t)mi * a.lda + (size_t)g * 128 + h * 8;
            float v[8];
            if (live && vec_x) {  // two 16-byte loads instead of eight scalar ones
                const float4 lo = *reinterpret_cast<const float4*>(src);
                const float4 hi = *reinterpret_cast<const float4*>(src + 4);
                v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
                v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    v[i] = live ? src[i] : 0.f;
            }
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                amax = fmaxf(amax, fabsf(v[i]));
            // max is exact and order-free: the butterfly gives the sequential loop's value
#pragma unroll
            for (int off = (A32 ? 2 : 8); off > 0; off >>= 1)
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            float scale, inv;
            b2w4_quant_params(amax, scale, inv);
            int c[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                c[i] = b2w4_quant_code(v[i], inv);
            int esum = c[0] + c[2] + c[4] + c[6];  // integer: order-free
#pragma unroll
            for (int off = (A32 ? 2 : 8); off > 0; off >>= 1)
                esum += __shfl_xor_sync(0xffffffffu, esum, off);
            if (!live)
                continue;
            if (A32) {
                if ((h & 3) == 0) {
                    s_as[mi * G * 4 + g * 4 + (h >> 2)] = scale;
                    s_es[mi * G * 4 + g * 4 + (h >> 2)] = -8 * esum;
                }
            } else if (h == 0) {
                s_as[mi * G + g] = scale;
                s_es[mi * G + g] = -8 * esum;
            }
            // 32-block h/4 is stored as 16 even-k codes then 16 odd-k codes
            uint8_t* blk = reinterpret_cast<uint8_t*>(s_qa) + (size_t)mi * K + (size_t)g * 128 +
                           (h >> 2) * 32;
            const int j = (h & 3) * 4;
            *reinterpret_cast<char4*>(blk + j) = make_char4(
                (signed char)c[0], (signed char)c[2], (signed char)c[4], (signed char)c[6]);
            *reinterpret_cast<char4*>(blk + 16 + j) = make_char4(
                (signed char)c[1], (signed char)c[3], (signed char)c[5], (signed char)c[7]);
        }
    }
    __syncthreads();  // quantised activations and barrier inits visible to all

    // ---- phase 1: integer group sums ---------------------------------------------------
    const int ipt = (G + 3) >> 2;
    const int n_items = ntile * ipt;
    bool timed_out = !mbar_wait_bounded(&s_bar[ntile]);  // weight scales
#pragma unroll 1
    for (int it = warp; it < n_items && !timed_out; it += kWarps) {
        const int tl = a.ipt_magic ? (it * a.ipt_magic) >> 16 : it / ipt;
        const int g = (it - tl * ipt) * 4 + gl;
        if (!mbar_wait_bounded(&s_bar[tl])) {
            timed_out = true;
            break;
        }
        if (g < G) {
            const uint4* wt =
                reinterpret_cast<const uint4*>(s_w) + (tl * tile_bytes >> 4) + g * 32 + row;
            // a weight word holds 8 nibbles; two logic instructions split it without shifts:
            // odd k as 16*q (int8), even k as q+8 (uint8)
            uint32_t wl[16], wh[16];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint4 w = wt[s * 8];
                wl[s * 4 + 0] = (w.x ^ 0x08080808u) & 0x0F0F0F0Fu;
                wh[s * 4 + 0] = w.x & 0xF0F0F0F0u;
                wl[s * 4 + 1] = (w.y ^ 0x08080808u) & 0x0F0F0F0Fu;
                wh[s * 4 + 1] = w.y & 0xF0F0F0F0u;
                wl[s * 4 + 2] = (w.z ^ 0x08080808u) & 0x0F0F0F0Fu;
                wh[s * 4 + 2] = w.z & 0xF0F0F0F0u;
                wl[s * 4 + 3] = (w.w ^ 0x08080808u) & 0x0F0F0F0Fu;
                wh[s * 4 + 3] = w.w & 0xF0F0F0F0u;
            }
            const int slot = tl * a.d_stride + g * SPG * MT * 8 + row;
            float* dst = s_d + slot;
            float* dsc = s_sc + slot;
            const float ws =
                SCL16 ? __half2float(reinterpret_cast<const __half*>(s_scl)[(tl * G + g) * 8 + row])
                      : reinterpret_cast<const float*>(s_scl)[(tl * G + g) * 8 + row];
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
                if (mi < a.m) {
                    const uint4* qa = s_qa + ((mi * K + g * 128) >> 4);
                    int pt = 0, qt = 0;
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const uint4 ae = qa[s * 2], ao = qa[s * 2 + 1];
                        // two independent chains per sub-block hide dp4a latency
                        int p = dp4a_us(wl[s * 4 + 0], ae.x, 0);
                        int q = __dp4a((int)wh[s * 4 + 0], (int)ao.x, 0);
                        p = dp4a_us(wl[s * 4 + 1], ae.y, p);
                        q = __dp4a((int)wh[s * 4 + 1], (int)ao.y, q);
                        p = dp4a_us(wl[s * 4 + 2], ae.z, p);
                        q = __dp4a((int)wh[s * 4 + 2], (int)ao.z, q);
                        p = dp4a_us(wl[s * 4 + 3], ae.w, p);
                        q = __dp4a((int)wh[s * 4 + 3], (int)ao.w, q);
                        if (A32) {
                            // q sums 16*q4*a: an exact multiple of 16
                            dst[(s * MT + mi) * 8] =
                                (float)(p + s_es[mi * G * 4 + g * 4 + s] + (q >> 4));
                            dsc[(s * MT + mi) * 8] =
                                __fmul_rn(ws, s_as[mi * G * 4 + g * 4 + s]);
                        } else {
                            pt += p;
                            qt += q;
                        }
                    }
                    if (!A32) {
                        dst[mi * 8] = (float)(pt + s_es[mi * G + g] + (qt >> 4));
                        dsc[mi * 8] = __fmul_rn(ws, s_as[mi * G + g]);
                    }
                }
            }
        }
    }
    if (timed_out && lane == 0)
        b2w4_report_timeout(a.status);
    __syncthreads();

    // ---- phase 2: fp32 chain, one thread per (tile, activation row, weight row) ---------
#pragma unroll 1
    for (int t = threadIdx.x; t < ntile * MT * 8; t += kThreads) {
        const int rr = t & 7, mi = (t >> 3) % MT, tl = t / (8 * MT);
        if (mi >= a.m)
            continue;
        const int n = (tile0 + tl) * 8 + rr;
        const float* dsrc = s_d + (size_t)tl * a.d_stride + mi * 8 + rr;
        const float* csrc = s_sc + (size_t)tl * a.d_stride + mi * 8 + rr;
        float acc = 0.f;
        // only the fused multiply-add depends on the previous step; the loads do not
#pragma unroll 10
        for (int j = 0; j < G * SPG; ++j) {
            const float dv = dsrc[j * MT * 8];
            acc = __fmaf_rn(dv, csrc[j * MT * 8], acc);
            if (SUMS && n < a.n)
                a.sums[((size_t)mi * a.n + n) * (G * SPG) + j] = (int)dv;
        }
        if (n < a.n) {
            if (b2w4_act_applies(n, a.activation, a.act_n_begin, a.act_n_len, a.n))
                acc = gemv_activation(acc, a.activation);
            if (MODE == kModeTop1) {
                // the index is the row of the unsharded weight (n_offset is 0 on one GPU)
                const unsigned long long word = b2w4_top1_word(acc, a.tp.n_offset + n);
                top1_best = word > top1_best ? word : top1_best;
                if (a.y)
                    a.y[(size_t)mi * a.ldc + n] = acc;
            } else if (a.tp.world == 0) {
                a.y[(size_t)mi * a.ldc + n] = acc;
            } else {
                // The all-gather is this store: every rank's staging buffer, this GPU's own
                // included, gets (value, exchange number) as one 8-byte word over peer
                // mappings.  The word is written whole, so the reader needs no fence: an
                // entry that carries the current exchange number carries its value.
                const unsigned long long word =
                    ((unsigned long long)tp_exchange << 32) | __float_as_uint(acc);
                const size_t at = kTpStageHeader +
                                  (size_t)(tp_exchange & 1) * kTpMaxRows * a.ldc +
                                  (size_t)mi * a.ldc + a.tp.n_offset + n;
#pragma unroll
                for (int p = 0; p < kTpMaxWorld; ++p)
                    if (p < a.tp.world)
                        a.tp.stage_peer[p][at] = word;
            }
        }
    }
    if (MODE == kModeTop1)
        b2w4_top1_finish(a.top1, top1_best, (threadIdx.x >> 3) % MT, a.m, s_top1);
}

// Second half of the tensor-parallel exchange: waits (bounded) until every entry of the
// current exchange's half of the staging buffer carries the exchange number -- written by this
// GPU's own matmul (complete: this kernel is ordered after it) and by the peers' -- and unpacks
// the values into the plain output row.  The last block then advances the exchange count.
// An entry that never arrives within `wait_limit` SM cycles becomes a quiet NaN in y (never a
// stale value of an earlier exchange) and the status word reports the time-out.
__global__ void __launch_bounds__(kTpGatherThreads)
tp_gather_kernel(unsigned long long* stage, float* y, int m, int ldc, unsigned* done,
                 int* status, unsigned long long wait_limit) {
    b2w4_pdl_chain_entry();
    unsigned* count = reinterpret_cast<unsigned*>(stage);
    const unsigned exchange = *reinterpret_cast<volatile unsigned*>(count) + 1u;
    const volatile unsigned long long* src =
        stage + kTpStageHeader + (size_t)(exchange & 1) * kTpMaxRows * ldc;
    const unsigned long long t0 = wait_clock();
    bool gave_up = false;
    // the m rows of the exchange are contiguous in the half and in y
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m * ldc;
         i += gridDim.x * blockDim.x) {
        unsigned long long word = src[i];
        while ((unsigned)(word >> 32) != exchange && !gave_up) {
            if (wait_clock() - t0 > wait_limit) {
                b2w4_report_timeout(status);
                gave_up = true;
            }
            word = src[i];
        }
        y[i] = (unsigned)(word >> 32) == exchange ? __uint_as_float((unsigned)word)
                                                  : __uint_as_float(0x7FC00000u);
    }
    __syncthreads();  // every thread of the block has read the count
    if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {
        *done = 0;  // ready for the next launch
        *count = exchange;
    }
}

// Second half of the fused greedy token on one GPU: the matmul before it in the stream left
// each row's maximum word in the cells; write the tokens and clear the cells.
__global__ void top1_token_kernel(unsigned long long* cells, int32_t* token, int m) {
    b2w4_pdl_chain_entry();
    if ((int)threadIdx.x < m) {
        const unsigned long long w = atomicExch(cells + threadIdx.x, 0ull);
        token[threadIdx.x] = (int32_t)(0xFFFFFFFFu - (unsigned)w);
    }
}

// Tensor-parallel greedy token, hand-over: this rank's maximum word of every row (left in the
// cells by the matmul, with indices of the unsharded weight) goes to every rank as two tagged
// words; the cells are cleared.  Thread (row r, rank q) stores to rank q.
__global__ void __launch_bounds__(kTop1MaxRows* kTpMaxWorld)
tp_send_token_kernel(unsigned long long* cells, const b2w4_tp_args tp, int m) {
    b2w4_pdl_chain_entry();
    __shared__ unsigned long long s_word[kTop1MaxRows];
    if ((int)threadIdx.x < m)
        s_word[threadIdx.x] = atomicExch(cells + threadIdx.x, 0ull);  // read and clear
    __syncthreads();
    const unsigned exchange =
        *reinterpret_cast<const volatile unsigned*>(tp.stage_peer[tp.rank]) + 1u;
    const unsigned long long tag = (unsigned long long)exchange << 32;
    const int r = threadIdx.x / kTpMaxWorld, q = threadIdx.x % kTpMaxWorld;
    if (r < m && q < tp.world) {
        const size_t slot = kTpStageHeader + (size_t)(exchange & 1) * kTop1StageHalf +
                            ((size_t)r * kTpMaxWorld + tp.rank) * 2;
        tp.stage_peer[q][slot] = tag | (s_word[r] >> 32);
        tp.stage_peer[q][slot + 1] = tag | (s_word[r] & 0xFFFFFFFFull);
    }
}

// ... and the pick: thread (row r, rank p) waits (bounded) for rank p's words of row r, the
// block takes the largest per row -- the one-GPU order -- and advances the count.
__global__ void __launch_bounds__(kTop1MaxRows* kTpMaxWorld)
tp_gather_token_kernel(unsigned long long* stage, int32_t* token, int m, int world, int* status,
                       unsigned long long wait_limit) {
    b2w4_pdl_chain_entry();
    __shared__ unsigned long long s_best[kTop1MaxRows];
    __shared__ int s_missing[kTop1MaxRows];  // a rank's words of this row never arrived
    unsigned* count = reinterpret_cast<unsigned*>(stage);
    const unsigned exchange = *reinterpret_cast<volatile unsigned*>(count) + 1u;
    const int r = threadIdx.x / kTpMaxWorld, p = threadIdx.x % kTpMaxWorld;
    if (threadIdx.x < kTop1MaxRows) {
        s_best[threadIdx.x] = 0ull;
        s_missing[threadIdx.x] = 0;
    }
    __syncthreads();
    if (r < m && p < world) {
        const volatile unsigned long long* src =
            stage + kTpStageHeader + (size_t)(exchange & 1) * kTop1StageHalf +
            ((size_t)r * kTpMaxWorld + p) * 2;
        const unsigned long long t0 = wait_clock();
        unsigned long long hi = src[0], lo = src[1];
        bool arrived = true;
        while ((unsigned)(hi >> 32) != exchange || (unsigned)(lo >> 32) != exchange) {
            if (wait_clock() - t0 > wait_limit) {
                b2w4_report_timeout(status);
                arrived = false;
                break;
            }
            hi = src[0], lo = src[1];
        }
        if (arrived)
            atomicMax(&s_best[r], (hi << 32) | (lo & 0xFFFFFFFFull));
        else
            s_missing[r] = 1;
    }
    __syncthreads();
    // a row that lacks a rank's maximum has no token: -1, never a guess from stale words
    if ((int)threadIdx.x < m)
        token[threadIdx.x] = s_missing[threadIdx.x]
                                 ? -1
                                 : (int32_t)(0xFFFFFFFFu - (unsigned)s_best[threadIdx.x]);
    if (threadIdx.x == 0)
        *count = exchange;
}

int gemv_d_stride(int mt, int groups, bool a32) {
    // +8 ints: consecutive tiles start 8 banks apart, so phase 2's warps read without
    // bank conflicts
    return groups * (a32 ? 4 : 1) * mt * 8 + 8;
}

size_t gemv_smem_bytes(int mt, int k, int groups, int tpc, bool scl16, bool a32) {
    const int spg = a32 ? 4 : 1;
    return (size_t)tpc * groups * 512 + (size_t)tpc * groups * 8 * (scl16 ? 2 : 4) +
           (size_t)mt * k + 2 * sizeof(float) * mt * groups * spg +
           2 * sizeof(float) * (size_t)tpc * gemv_d_stride(mt, groups, a32) + 8 +
           sizeof(uint64_t) * (tpc + 1);
}

template <int MT, bool SCL16, bool A32, int MODE>
int launch_one(b2w4_ctx* ctx, const GemvArgs& a, size_t smem) {
    auto kern = gemv_w4a8_kernel<MT, SCL16, A32, MODE>;
    static b2w4_smem_optin configured;  // per instantiation and device
    B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, kern, smem, configured));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.tiles + a.tpc - 1) / a.tpc);
    cfg.blockDim = dim3(gemv_warps(MT) * 32);
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

template <int MT>
int launch_mt(b2w4_ctx* ctx, const GemvArgs& a, bool scl16, bool a32, size_t smem) {
    const int mode = a.sums ? kModeSums : (a.top1.cells ? kModeTop1 : kModePlain);
#define B2W4_GEMV_MODES(S, A)                                              \
    (mode == kModeSums   ? launch_one<MT, S, A, kModeSums>(ctx, a, smem)   \
     : mode == kModeTop1 ? launch_one<MT, S, A, kModeTop1>(ctx, a, smem)   \
                         : launch_one<MT, S, A, kModePlain>(ctx, a, smem))
    if (scl16)
        return a32 ? B2W4_GEMV_MODES(true, true) : B2W4_GEMV_MODES(true, false);
    return a32 ? B2W4_GEMV_MODES(false, true) : B2W4_GEMV_MODES(false, false);
#undef B2W4_GEMV_MODES
}

}  // namespace

// Rows are processed four at a time; each pass streams the weight once.
int b2w4_launch_gemv(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                     float* y, int ldc, int m, int act_rule, int activation,
                     int act_n_begin, int act_n_len, int32_t* sums, const b2w4_tp_args* tp,
                     const b2w4_top1_args* top1) {
    if (tp && m > kTpMaxRows)
        return b2w4_fail(ctx, B2W4_E_INVALID, "tensor-parallel epilogue: at most %d rows",
                         kTpMaxRows);
    if (m > 1)  // several rows share one pass over the weight on the tensor instruction
        return b2w4_launch_gemv_mma(ctx, w, x, lda, y, ldc, m, act_rule, activation, act_n_begin,
                                    act_n_len, sums, tp, top1);
    const bool a32 = act_rule == B2W4_ACT_G32;
    const int spg = a32 ? 4 : 1;
    const bool scl16 = w->scales_fp16 != 0;
    for (int m0 = 0; m0 < m; m0 += 4) {
        const int mc = min(4, m - m0);
        const int mt = mc == 1 ? 1 : (mc == 2 ? 2 : 4);
        GemvArgs a;
        a.nib = w->nib;
        a.scl = w->scl;
        a.x = x + (size_t)m0 * lda;
        a.y = y ? y + (size_t)m0 * ldc : nullptr;
        a.sums = sums ? sums + (size_t)m0 * w->n * w->groups * spg : nullptr;
        a.status = ctx->status_dev;
        a.lda = lda;
        a.ldc = ldc;
        a.m = mc;
        a.n = w->n;
        a.k = w->k;
        a.groups = w->groups;
        a.tiles = w->tiles;
        a.activation = activation;
        a.act_n_begin = act_n_begin;
        a.act_n_len = act_n_len;
        a.tp = b2w4_tp_args();
        if (tp)
            a.tp = *tp;
        else
            a.tp.world = 0;
        a.top1 = b2w4_top1_args();
        if (top1)
            a.top1 = *top1;
        // Tiles per CTA: a CTA's shared memory stays under half an SM's so that two CTAs share
        // an SM, and the launch is one wave of at most 1.75 CTAs per SM.  Measured on the
        // decode shapes of a 4B dense model (148 SMs): N=9728 K=2560 (1216 tiles) 244 CTAs
        // 4.26 us (152 CTAs 6.0, 304 CTAs needing a second wave 6.6); N=6144 (768 tiles) 256
        // CTAs 3.55 us against 192 CTAs 4.08; N=19456 (2432 tiles) 271 CTAs 7.0 us against 304
        // CTAs 8.65.
        const int per_tile = w->groups * (512 + (scl16 ? 16 : 32)) +
                             8 * gemv_d_stride(mt, w->groups, a32);
        const int budget = 113 * 1024 - mt * w->k - 8 * mt * w->groups * spg - 1024;
        int tpc = max(1, min(budget / per_tile, kMaxTpc));
        const int wave_ctas = ctx->sm_count * 7 / 4;
        const int one_wave = (w->tiles + wave_ctas - 1) / wave_ctas;
        tpc = min(tpc, max(1, one_wave));
        if (ctx->gemv_tpc_override > 0)
            tpc = min(tpc, ctx->gemv_tpc_override);
        a.tpc = tpc;
        {
            const int ipt = (w->groups + 3) / 4;
            a.ipt_magic = 65536 / ipt + 1;
            for (int it = 0; it < tpc * ipt; ++it)  // exact for every item of a CTA?
                if (((it * a.ipt_magic) >> 16) != it / ipt)
                    a.ipt_magic = 0;
        }
        a.d_stride = gemv_d_stride(mt, w->groups, a32);
        const size_t smem = gemv_smem_bytes(mt, w->k, w->groups, tpc, scl16, a32);
        if (smem > 220 * 1024)
            return b2w4_fail(ctx, B2W4_E_INVALID, "gemv: K=%d needs %zu B shared memory",
                             w->k, smem);
        int rc = launch_mt<1>(ctx, a, scl16, a32, smem);  // mt == 1: see the top
        if (rc != B2W4_OK)
            return rc;
    }
    return B2W4_OK;
}

int b2w4_launch_top1_token(b2w4_ctx* ctx, unsigned long long* cells, int32_t* token, int m) {
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, top1_token_kernel, dim3(1), dim3(32), 0,
                                       ctx->stream, cells, token, m));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_launch_tp_send_token(b2w4_ctx* ctx, unsigned long long* cells, const b2w4_tp_args& tp,
                              int m) {
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, tp_send_token_kernel, dim3(1),
                                       dim3(kTop1MaxRows * kTpMaxWorld), 0, ctx->stream, cells,
                                       tp, m));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_launch_tp_gather_token(b2w4_ctx* ctx, unsigned long long* stage_local, int32_t* token,
                                int m, int world) {
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, tp_gather_token_kernel, dim3(1),
                                       dim3(kTop1MaxRows * kTpMaxWorld), 0, ctx->stream,
                                       stage_local, token, m, world, ctx->status_dev,
                                       ctx->peer_wait_cycles));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_launch_tp_gather(b2w4_ctx* ctx, unsigned long long* stage_local, float* y, int m,
                          int ldc) {
    const int blocks = max(1, min((m * ldc + kTpGatherThreads - 1) / kTpGatherThreads,
                                  ctx->sm_count));
    B2W4_CUDA(ctx, b2w4_launch_chained(ctx->pdl, tp_gather_kernel, dim3(blocks),
                                       dim3(kTpGatherThreads), 0, ctx->stream, stage_local, y,
                                       m, ldc, reinterpret_cast<unsigned*>(ctx->flag_dev + 6),
                                       ctx->status_dev, ctx->peer_wait_cycles));
    ctx->launches++;
    return B2W4_OK;
}
