// W4G128 x int8 matmul for 2..8 activation rows (batched decode): HBM-bound weight
// streaming, integer sums on the warp-level int8 tensor instruction (mma.sync m16n8k32).
//
// Arithmetic = the reference's NEON W4A8 kernels applied row by row (kernels/matmul_w4.cpp:
// 211-295 for the per-128 rule, :785-901 for the per-32 rule), with the activation quantiser
// (kernels/matmul_quant.cpp:578-641, :280-329) fused in:
//   per group (32-block) g:  D = sum q4*q8 (int32);  y = fma(float(D), fp32(ws*as[g]), y)
// groups ascending.  Integer sums are exact in any order, so the tensor instruction gives
// the same bits as the scalar loop.
//
// Data movement.  The 8-row tiles of the weight are dealt to the CTAs in contiguous runs
// (as even as possible); a CTA's run of the nibble plane and of the scale plane is brought
// into shared memory by 16-byte cp.async copies that all its threads issue as the first
// thing the kernel does, before it waits for the previous kernel in the stream (programmatic
// dependent launch): weights never depend on the predecessor's output, only the activation
// read does.  The copies are per-thread cp.async on purpose: bulk copies (cp.async.bulk)
// issued by a dependent launch before its predecessor has finished were measured not to
// complete until the predecessor's grid ends (in-kernel timestamps: issued 9 us early,
// landed with the dependency), while per-thread cp.async issued at the same point lands
// within 1.3 us.
//
// Math, phase 1.  An item is (two tiles = 16 weight rows, one group of 128 k); warp w takes
// items w, w+W, ...  The 16x128 weights are the A operand of four m16n8k32 instructions, the
// activation rows are the columns of B (up to 8 rows for the price of one; unused columns
// repeat row 0 and are never read back).  Because a dot product does not care about the
// order of k, a lane's A registers are simply the words it loads: word `lane` of each
// 128-byte row block holds 8 nibbles of row lane/4, and two logic instructions split it
// without shifts:
//   hi = w & 0xF0F0F0F0                  odd k, bytes = 16*q as int8
//   lo = (w ^ 0x08080808) & 0x0F0F0F0F   even k, bytes = q+8 as uint8
// sum(q*a) = mma.u8.s8(lo, a_even) - 8*sum(a_even) + mma.s8.s8(hi, a_odd)/16: the last term
// is an exact multiple of 16 and -8*sum(a_even) comes from the quantiser, one per group.
// The quantiser lays the int8 codes out so that a lane's eight B words of a group are two
// 16-byte loads.  The integer sums go to shared memory as floats (exact: |sum| < 2^24).
// Phase 2, after one barrier: one thread per (tile, weight row, activation row) runs the
// order-sensitive chain of fused multiply-adds over the groups in ascending order.
#include "b200w4_internal.cuh"

namespace {

constexpr int kMmaWarps = 16;  // <= 64 registers per thread: two CTAs share an SM
constexpr int kMaxTilesPerCta = 16;
constexpr size_t kSmemPerCta = 113 * 1024;  // two CTAs per SM

struct MmaArgs {
    const uint4* nib;
    const void* scl;
    const float* x;
    float* y;
    int32_t* sums;  // optional [m][n][groups or 4*groups]
    int lda, ldc, m, n, k, groups, tiles;
    int tiles_base, tiles_rem;  // CTA c owns tiles_base + (c < tiles_rem) tiles
    int tile_cap;               // shared memory is laid out for this many tiles
    int g_magic;                // item / groups == (item * g_magic) >> 16, or 0: divide
    int d_stride;  // floats between the integer sums of consecutive tiles (padded)
    int activation, act_n_begin, act_n_len;
    b2w4_tp_args tp;  // world != 0: the rows go to every rank's staging buffer instead of y
    b2w4_top1_args top1;  // greedy-token epilogue (MODE 2)
};
// Kernel modes: plain, with the int32 group sums written out, with the greedy-token epilogue.
constexpr int kModePlain = 0, kModeSums = 1, kModeTop1 = 2;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src)
                 : "memory");
}
// One warp-wide int8 tensor instruction: D[16x8] += A[16x32] * B[32x8], A unsigned (U) or
// signed bytes, B signed bytes.  Lane (gid = lane/4, tid = lane%4) holds
//   a0: row gid, k = 4*tid..+3     a1: row gid+8, same k     a2/a3: the same rows, k + 16
//   b0: k = 4*tid..+3, column gid  b1: k + 16
//   d0/d1: row gid, columns 2*tid, 2*tid+1     d2/d3: row gid+8
template <bool U>
__device__ __forceinline__ void mma_16x8x32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
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

// the fused activations carry fp64 exp / tanh code: keep one out-of-line copy
__device__ __noinline__ float mma_gemv_activation(float v, int act) {
    return b2w4_activation(v, act);
}

template <int MT, bool SCL16, bool A32, int MODE>
__global__ void __launch_bounds__(kMmaWarps * 32, 2)
gemv_w4a8_mma_kernel(const MmaArgs a) {
    constexpr int kWarps = kMmaWarps;
    constexpr int kThreads = kWarps * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int SPG = A32 ? 4 : 1;  // integer sums per group
    const int G = a.groups, K = a.k;
    const int tile_bytes = G * 512;
    const int scl_tile_bytes = G * 8 * (SCL16 ? 2 : 4);
    // shared-memory carve-up (every region a multiple of 16 bytes)
    uint8_t* s_w = smem;                                      // [cap][G][512]
    uint8_t* s_scl = s_w + (size_t)a.tile_cap * tile_bytes;   // [cap][G][8] fp16|fp32
    uint4* s_qa = reinterpret_cast<uint4*>(s_scl + (size_t)a.tile_cap * scl_tile_bytes);  // [MT][K]
    float* s_as = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_qa) + (size_t)MT * K);
    int* s_es = reinterpret_cast<int*>(s_as + MT * G * SPG);  // -8 * sum of the even-k codes
    // per (tile, group, [32-block], activation row, weight row): the integer sum as a float
    // (exact: |sum| < 2^24)
    float* s_d = reinterpret_cast<float*>(s_es + MT * G * SPG);  // [cap][G][SPG][MT][8] + pad

    constexpr bool SUMS = MODE == kModeSums;
    __shared__ unsigned long long s_top1[8];
    if (MODE == kModeTop1 && threadIdx.x < 8)
        s_top1[threadIdx.x] = 0ull;  // barriers follow before the epilogue uses it
    unsigned long long top1_best = 0ull;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gl = lane >> 3, row = lane & 7;
    const int cta = blockIdx.x;
    const int ntile = a.tiles_base + (cta < a.tiles_rem ? 1 : 0);
    const int tile0 = cta * a.tiles_base + min(cta, a.tiles_rem);

    // Let the next kernel in the stream become resident and start its own weight copies.
    b2w4_pdl_launch_dependents();

    // ---- weight stream: issued before anything else, independent of the predecessor ----
    {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(a.nib) + (size_t)tile0 * tile_bytes;
        const int n16 = ntile * (tile_bytes >> 4);
        for (int i = threadIdx.x; i < n16; i += kThreads)
            cp_async16(s_w + (size_t)i * 16, src + (size_t)i * 16);
        const uint8_t* ssrc =
            reinterpret_cast<const uint8_t*>(a.scl) + (size_t)tile0 * scl_tile_bytes;
        const int s16 = ntile * (scl_tile_bytes >> 4);
        for (int i = threadIdx.x; i < s16; i += kThreads)
            cp_async16(s_scl + (size_t)i * 16, ssrc + (size_t)i * 16);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    b2w4_pdl_wait();  // activations come from the previous kernel

    // Tensor-parallel exchange number: one more than the count of completed gathers (first
    // word of this rank's staging buffer, written by the gather kernel).
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
            // The lane's four even-k codes are one B-operand word of phase 1, its four
            // odd-k codes another.  Group layout: [word position h%4][even words of the four
            // 32-blocks, then the odd words], so a phase-1 lane reads its eight words of a
            // group as two 16-byte loads.
            uint8_t* blk = reinterpret_cast<uint8_t*>(s_qa) + (size_t)mi * K + (size_t)g * 128 +
                           (h & 3) * 32 + (h >> 2) * 4;
            *reinterpret_cast<char4*>(blk) = make_char4(
                (signed char)c[0], (signed char)c[2], (signed char)c[4], (signed char)c[6]);
            *reinterpret_cast<char4*>(blk + 16) = make_char4(
                (signed char)c[1], (signed char)c[3], (signed char)c[5], (signed char)c[7]);
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();  // every thread's copies and the quantised activations are visible

    // ---- phase 1: integer group sums on the int8 tensor instruction ----------------------
    // An item is (pair of tiles = 16 weight rows, group).  Activation row mi is column mi of
    // the B operand; columns past the last row repeat row 0 and are never read back.
    // Shared memory is indexed with 32-bit word offsets throughout.
    {
        const int gid = lane >> 2, tid = lane & 3;
        const int npair = (ntile + 1) >> 1;
        const int n_items = npair * G;
        const int bcol = gid < a.m ? gid : 0;
        const uint32_t* s_w32 = reinterpret_cast<const uint32_t*>(s_w);
        const int tile_words = tile_bytes >> 2;
        const int qa_base = (bcol * K >> 4) + tid * 2;  // uint4 index of this lane's B words
        const int mi0 = tid * 2;                        // columns held in the accumulators
#pragma unroll 2
        for (int it = warp; it < n_items; it += kWarps) {
            const int tp = a.g_magic ? (it * a.g_magic) >> 16 : it / G;
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
            const int dbase = t0 * a.d_stride + gid;
            if (A32) {
                const uint32_t bev[4] = {be.x, be.y, be.z, be.w}, bov[4] = {bo.x, bo.y, bo.z, bo.w};
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
                    mma_16x8x32<true>(cl, lo0[s], lo1[s], 0u, 0u, bev[s], 0u);
                    mma_16x8x32<false>(ch, hi0[s], hi1[s], 0u, 0u, bov[s], 0u);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int mi = mi0 + c;
                        if (c < MT && mi < a.m) {
                            const int e8 = s_es[(mi * G + g) * 4 + s];
                            const int slot = dbase + ((g * 4 + s) * MT + mi) * 8;
                            // ch sums 16*q4*a: an exact multiple of 16
                            s_d[slot] = (float)(cl[c] + e8 + (ch[c] >> 4));
                            if (two)
                                s_d[slot + a.d_stride] = (float)(cl[2 + c] + e8 + (ch[2 + c] >> 4));
                        }
                    }
                }
            } else {
                int cl[4] = {0, 0, 0, 0}, ch[4] = {0, 0, 0, 0};
                mma_16x8x32<true>(cl, lo0[0], lo1[0], lo0[1], lo1[1], be.x, be.y);
                mma_16x8x32<false>(ch, hi0[0], hi1[0], hi0[1], hi1[1], bo.x, bo.y);
                mma_16x8x32<true>(cl, lo0[2], lo1[2], lo0[3], lo1[3], be.z, be.w);
                mma_16x8x32<false>(ch, hi0[2], hi1[2], hi0[3], hi1[3], bo.z, bo.w);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int mi = mi0 + c;
                    if (c < MT && mi < a.m) {
                        const int e8 = s_es[mi * G + g];
                        const int slot = dbase + (g * MT + mi) * 8;
                        // ch sums 16*q4*a: an exact multiple of 16
                        s_d[slot] = (float)(cl[c] + e8 + (ch[c] >> 4));
                        if (two)
                            s_d[slot + a.d_stride] = (float)(cl[2 + c] + e8 + (ch[2 + c] >> 4));
                    }
                }
            }
        }
    }
    __syncthreads();

    // ---- phase 2: fp32 chain, one thread per (tile, activation row, weight row) ---------
    // acc = fma(float(D), fp32(ws * as), acc), groups (32-blocks) ascending.  Only the fused
    // multiply-add depends on the previous step; the loads and the scale product do not.
#pragma unroll 1
    for (int t = threadIdx.x; t < ntile * MT * 8; t += kThreads) {
        const int rr = t & 7, mi = (t >> 3) % MT, tl = t / (8 * MT);
        if (mi >= a.m)
            continue;
        const int n = (tile0 + tl) * 8 + rr;
        const float* dsrc = s_d + tl * a.d_stride + mi * 8 + rr;
        const float* asrc = s_as + mi * G * SPG;
        float acc = 0.f;
#pragma unroll 4
        for (int g = 0; g < G; ++g) {
            const float ws =
                SCL16 ? __half2float(reinterpret_cast<const __half*>(s_scl)[(tl * G + g) * 8 + rr])
                      : reinterpret_cast<const float*>(s_scl)[(tl * G + g) * 8 + rr];
#pragma unroll
            for (int s = 0; s < SPG; ++s) {
                const int j = g * SPG + s;
                const float dv = dsrc[j * MT * 8];
                acc = __fmaf_rn(dv, __fmul_rn(ws, asrc[j]), acc);
                if (SUMS && n < a.n)
                    a.sums[((size_t)mi * a.n + n) * (G * SPG) + j] = (int)dv;
            }
        }
        if (n < a.n) {
            if (b2w4_act_applies(n, a.activation, a.act_n_begin, a.act_n_len, a.n))
                acc = mma_gemv_activation(acc, a.activation);
            if (MODE == kModeTop1) {
                // the index is the row of the unsharded weight (n_offset is 0 on one GPU)
                const unsigned long long word = b2w4_top1_word(acc, a.tp.n_offset + n);
                top1_best = word > top1_best ? word : top1_best;
                if (a.y)
                    a.y[(size_t)mi * a.ldc + n] = acc;
            } else if (a.tp.world == 0) {
                a.y[(size_t)mi * a.ldc + n] = acc;
            } else {
                // (value, exchange number) as one 8-byte word into every rank's staging buffer
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
    // kThreads / 8 is a multiple of MT: a thread's activation row is the same in every pass
    if (MODE == kModeTop1)
        b2w4_top1_finish(a.top1, top1_best, (threadIdx.x >> 3) % MT, a.m, s_top1);
}

int mma_d_stride(int mt, int groups, bool a32) {
    // + 8 floats: consecutive tiles start in different banks
    return groups * (a32 ? 4 : 1) * mt * 8 + 8;
}

size_t mma_smem_bytes(int mt, int k, int groups, int cap, bool scl16, bool a32) {
    const int spg = a32 ? 4 : 1;
    return (size_t)cap * groups * 512 + (size_t)cap * groups * 8 * (scl16 ? 2 : 4) +
           (size_t)mt * k + 2 * sizeof(float) * (size_t)mt * groups * spg +
           sizeof(float) * (size_t)cap * mma_d_stride(mt, groups, a32) + 16;
}

template <int MT, bool SCL16, bool A32, int MODE>
int mma_launch_one(b2w4_ctx* ctx, const MmaArgs& a, size_t smem, int ctas) {
    auto kern = gemv_w4a8_mma_kernel<MT, SCL16, A32, MODE>;
    static b2w4_smem_optin configured;  // per instantiation and device
    B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, kern, smem, configured));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kMmaWarps * 32);
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
int mma_launch_mt(b2w4_ctx* ctx, const MmaArgs& a, bool scl16, bool a32, size_t smem, int ctas) {
    const int mode = a.sums ? kModeSums : (a.top1.cells ? kModeTop1 : kModePlain);
#define B2W4_MMA_MODES(S, A)                                                        \
    (mode == kModeSums   ? mma_launch_one<MT, S, A, kModeSums>(ctx, a, smem, ctas)   \
     : mode == kModeTop1 ? mma_launch_one<MT, S, A, kModeTop1>(ctx, a, smem, ctas)   \
                         : mma_launch_one<MT, S, A, kModePlain>(ctx, a, smem, ctas))
    if (scl16)
        return a32 ? B2W4_MMA_MODES(true, true) : B2W4_MMA_MODES(true, false);
    return a32 ? B2W4_MMA_MODES(false, true) : B2W4_MMA_MODES(false, false);
#undef B2W4_MMA_MODES
}

}  // namespace

// Rows are processed eight at a time (the columns of one tensor instruction); each pass
// streams the weight once.
int b2w4_launch_gemv_mma(b2w4_ctx* ctx, const b2w4_weight* w, const float* x, int lda,
                         float* y, int ldc, int m, int act_rule, int activation,
                         int act_n_begin, int act_n_len, int32_t* sums,
                         const b2w4_tp_args* tp, const b2w4_top1_args* top1) {
    const bool a32 = act_rule == B2W4_ACT_G32;
    const int spg = a32 ? 4 : 1;
    const bool scl16 = w->scales_fp16 != 0;
    for (int m0 = 0; m0 < m; m0 += 8) {
        const int mc = min(8, m - m0);
        const int mt = mc <= 2 ? 2 : (mc <= 4 ? 4 : 8);
        MmaArgs a;
        a.nib = w->nib;
        a.scl = w->scl;
        a.x = x + (size_t)m0 * lda;
        a.y = y ? y + (size_t)m0 * ldc : nullptr;
        a.sums = sums ? sums + (size_t)m0 * w->n * w->groups * spg : nullptr;
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
        a.top1 = b2w4_top1_args();
        if (top1)
            a.top1 = *top1;
        // Tiles per CTA.  `cap` tiles fit while two CTAs still share an SM.  A weight small
        // enough gets one CTA per SM (the next launch's CTAs are then resident beside this
        // one's and their weights land early); a larger one gets two per SM in one balanced
        // wave; beyond that, whole waves of CTAs near the cap.
        int cap = kMaxTilesPerCta;
        while (cap > 1 && mma_smem_bytes(mt, w->k, w->groups, cap, scl16, a32) > kSmemPerCta)
            --cap;
        const int sms = ctx->sm_count;
        int ctas;
        if ((w->tiles + sms - 1) / sms <= cap)
            ctas = min(w->tiles, sms);
        else if ((w->tiles + 2 * sms - 1) / (2 * sms) <= cap)
            ctas = 2 * sms;
        else
            ctas = ((w->tiles + cap - 1) / cap + 2 * sms - 1) / (2 * sms) * (2 * sms);
        if (ctx->gemv_tpc_override > 0)  // tuning: tiles per CTA
            ctas = (w->tiles + min(cap, ctx->gemv_tpc_override) - 1) /
                   min(cap, ctx->gemv_tpc_override);
        a.tiles_base = w->tiles / ctas;
        a.tiles_rem = w->tiles % ctas;
        a.tile_cap = a.tiles_base + (a.tiles_rem ? 1 : 0);
        a.g_magic = 65536 / w->groups + 1;
        for (int it = 0; it < (a.tile_cap + 1) / 2 * w->groups; ++it)  // exact for every item?
            if (((it * a.g_magic) >> 16) != it / w->groups)
                a.g_magic = 0;
        a.d_stride = mma_d_stride(mt, w->groups, a32);
        const size_t smem = mma_smem_bytes(mt, w->k, w->groups, a.tile_cap, scl16, a32);
        if (smem > 220 * 1024)
            return b2w4_fail(ctx, B2W4_E_INVALID, "gemv: K=%d needs %zu B shared memory",
                             w->k, smem);
        int rc = mt == 2 ? mma_launch_mt<2>(ctx, a, scl16, a32, smem, ctas)
                 : mt == 4 ? mma_launch_mt<4>(ctx, a, scl16, a32, smem, ctas)
                           : mma_launch_mt<8>(ctx, a, scl16, a32, smem, ctas);
        if (rc != B2W4_OK)
            return rc;
    }
    return B2W4_OK;
}
