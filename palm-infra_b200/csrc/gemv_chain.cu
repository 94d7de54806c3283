// A list of one-row W4G128 x int8 GEMVs as ONE persistent kernel (decode steps).
//
// What it replaces.  A decode step of the reference is a walk over the graph's nodes, one
// MATMUL dispatch per weight with M == 1 (graph/execute.cpp:651-669 ->
// matmul_int4_q8dot_neon_gemv_g128_range, kernels/matmul_w4.cpp:211-295), and its batch entry
// point runs several such GEMVs in one dispatch (kernel_matmul_int4_gemv_batch,
// kernels/matmul_w4.cpp:381-493).  Arithmetic per GEMV is exactly that kernel's: activations
// quantised per 128 values (kernels/matmul_quant.cpp:578-641), D = sum q4*q8 in int32 per
// (row, group), y = fma(float(D), fp32(ws*as), y) with the groups in ascending order.
//
// Why one kernel.  A 13 MB GEMV is 2 us of HBM time; launched one by one, each GEMV pays the
// dependency on its predecessor (launch boundary, activation read, quantiser, integer sums,
// fp32 chain) with the memory system idle in between.  Here one CTA per SM stays resident for
// the whole list:
//   * a producer thread walks the CTA's share of EVERY op's weight tiles, in order, and keeps a
//     ring of shared memory (about 180 KB per SM, two ops' worth of a 13 MB weight) full with
//     bulk async copies -- weights never depend on activations, so the stream of op i+1 and
//     i+2 flows while op i is still being computed and while its result crosses to the other
//     SMs;
//   * an op's output row goes to a scratch buffer as tagged 8-byte words (tag << 32 | fp32
//     bits).  An aligned 8-byte store is written whole, so a reader that sees the tag sees the
//     value: the consumer op's quantiser simply polls the words it needs.  No grid barrier, no
//     fence, no counter: the hand-over costs one store and one load through L2;
//   * compute warps work in teams on a tile; the order-sensitive fp32 chain of a row runs in
//     registers and is handed from one team member to the next through shared memory.
// Every wait (tagged words, mbarriers) is bounded; on expiry the kernel raises the status
// word, stops waiting everywhere (all CTAs see the abort word) and runs to its end.
//
// The kernel is launched cooperatively (all CTAs co-resident: they wait for one another).
#include "b200w4_internal.cuh"

#include <algorithm>
#include <cstring>
#include <new>
#include <vector>

namespace {

constexpr int kComputeWarps = 18;
constexpr int kChainThreads = (kComputeWarps + 1) * 32;  // + one producer warp
constexpr int kEntries = 32;          // ring entries (tiles in flight per CTA)
constexpr unsigned kEmptyCount = 840; // lcm(1..8): a member arrives with 840 / team size
// Quantised activations: a group's 128 codes sit 144 bytes apart, so that the four groups a
// warp reads with one 16-byte load per lane fall into four different bank groups (at 128 bytes
// apart they share one and the load takes four passes through the shared-memory pipe, which
// this kernel keeps busier than any other unit).
constexpr int kXqStride = 144;
constexpr int kOpSlots = 4;           // op records resident in shared memory
constexpr int kTpiMax = 4;            // 8-row tiles per ring item (one pair of bulk copies)
constexpr uint32_t kItemBytesCap = 48 * 1024;
constexpr int kMaxTeamSize = 8;
constexpr unsigned long long kChainWaitCycles = 4000000000ull;  // about 2 s

// Device record of one GEMV.  Everything a warp would otherwise have to divide for is
// precomputed on the host.
struct __align__(16) ChainOp {
    const uint8_t* nib;
    const uint8_t* scl;
    const float* x_ext;                  // plain fp32 input, or
    const unsigned long long* x_tag;     // tagged words of an earlier op's output
    unsigned long long* y_tag;           // this op's tagged output [n]
    float* y_ext;                        // optional plain output [n]
    int n, groups;
    int tiles_q, tiles_r;                // tiles / CTAs and tiles % CTAs
    int scl_group_bytes;                 // 16 (fp16 scales) or 32 (fp32)
    int team, teams;                     // warps per tile, teams per CTA
    int tpi;                             // tiles per ring item
    unsigned team_magic, tpi_magic;      // x / d == (x * magic) >> 16 for the small x used here
    unsigned tag_in, tag_out;            // relative to the run's tag base
    int activation, act_n_begin, act_n_len;
    int ipt;                             // iterations (4 groups) per tile
    int reuse_x;                         // same input vector as the op before: already quantised
    // Tensor-parallel form (world >= 1; 0 = off): this rank holds the rows [n_offset, n_offset + n) of
    // the full row; the tagged words go to every rank's scratch at word tag_off + row, the
    // plain values (optional) to every rank's y at n_offset + row.
    int world, n_offset;
    int pad_;
    unsigned long long tag_off;          // word offset of this op's shard in a rank's scratch
    float* y_peers[kTpMaxWorld];
};
static_assert(sizeof(ChainOp) == 208, "op record size");
constexpr int kOpRecordQuads = sizeof(ChainOp) / 16;

struct ChainArgs {
    const ChainOp* ops;
    int count;
    unsigned tag_base;
    int* status;       // host-mapped status word
    int* abort_word;   // device word: non-zero = some wait gave up, nobody waits any more
    int ring_bytes;    // shared-memory ring
    int kmax;          // largest K of the list (sizes the quantised-activation buffers)
    // Profiling hook (NULL = off): CTA trace_cta writes, per op, kTraceSlots time stamps in SM
    // cycles (clock64 of that SM: cheap to read, comparable within the CTA): 0 op begins, 1 its activations have arrived, 2 quantised
    // (past the barrier), 5 about to wait for its first tile, 3 that tile's weights are in
    // shared memory, 4 its last tile done (all compute warp 0); 6 the producer issued the
    // op's last copy, 7 cycles the producer waited for ring space during the op.
    long long* trace;
    int trace_cta;
    unsigned long long* scratch_peers[kTpMaxWorld];  // every rank's tagged scratch (world > 1)
};
constexpr int kTraceSlots = 8;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
                 : "memory");
}
// The hint lets the hardware park the thread until the phase completes (or about 20 us pass)
// instead of having it spin through the issue slots the compute warps need.
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
// shared-space loads with 32-bit addresses (volatile: they stay behind the barrier waits)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// (a ^ b) & c in one logic instruction
__device__ __forceinline__ uint32_t xor_and(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x28;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Integer sum of one (weight row, 128-k group): 64 bytes of nibbles at w_addr + {0, 128, 256,
// 384} (the row's chunk of each 32-k block), 128 int8 codes at x_addr (per 32-block: 16 even-k
// codes, 16 odd-k codes).  A weight word w holds 8 nibbles: hi = w & 0xF0F0F0F0 is the odd k
// as 16*q (int8), lo = (w ^ 0x08080808) & 0x0F0F0F0F the even k as q+8 (uint8);
// sum q*a = dp4a.u8.s8(lo, a_even) - 8*sum(a_even) + dp4a.s8.s8(hi, a_odd) / 16 (exact).
__device__ __forceinline__ int group_dot(uint32_t w_addr, uint32_t x_addr, int minus8_esum) {
    int p0 = 0, p1 = 0, q0 = 0, q1 = 0;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint4 w = lds128(w_addr + s * 128);
        const uint4 ae = lds128(x_addr + s * 32);
        const uint4 ao = lds128(x_addr + s * 32 + 16);
        p0 = dp4a_us(xor_and(w.x, 0x08080808u, 0x0F0F0F0Fu), ae.x, p0);
        q0 = __dp4a((int)(w.x & 0xF0F0F0F0u), (int)ao.x, q0);
        p1 = dp4a_us(xor_and(w.y, 0x08080808u, 0x0F0F0F0Fu), ae.y, p1);
        q1 = __dp4a((int)(w.y & 0xF0F0F0F0u), (int)ao.y, q1);
        p0 = dp4a_us(xor_and(w.z, 0x08080808u, 0x0F0F0F0Fu), ae.z, p0);
        q0 = __dp4a((int)(w.z & 0xF0F0F0F0u), (int)ao.z, q0);
        p1 = dp4a_us(xor_and(w.w, 0x08080808u, 0x0F0F0F0Fu), ae.w, p1);
        q1 = __dp4a((int)(w.w & 0xF0F0F0F0u), (int)ao.w, q1);
    }
    return (p0 + p1) + minus8_esum + ((q0 + q1) >> 4);
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void compute_barrier() {  // the compute warps only
    asm volatile("bar.sync 1, %0;" ::"n"(kComputeWarps * 32) : "memory");
}
__device__ __noinline__ float chain_activation(float v, int act) {
    return b2w4_activation(v, act);
}

// Shared state of one CTA's waits: once any wait anywhere gave up, nothing waits any more.
struct WaitCtx {
    int* status;
    int* abort_word;
    bool aborted;
};
__device__ __forceinline__ void give_up(WaitCtx& wc) {
    b2w4_report_timeout(wc.status);
    *reinterpret_cast<volatile int*>(wc.abort_word) = 1;
    wc.aborted = true;
}
// sleep_ns > 0: the waiter is not on anybody's critical path (the producer waiting for ring
// space) and pauses between looks instead of taking issue slots from the compute warps.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, WaitCtx& wc,
                                          unsigned sleep_ns = 0) {
    if (wc.aborted)
        return;
    const long long t0 = clock64();
    for (;;) {
        // a short inner loop of nothing but the look: a waiting warp shares its scheduler
        // with warps that work
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity))
                return;
            if (sleep_ns)
                __nanosleep(sleep_ns);
        }
        if (*reinterpret_cast<volatile int*>(wc.abort_word) != 0) {
            wc.aborted = true;
            return;
        }
        if ((unsigned long long)(clock64() - t0) > kChainWaitCycles) {
            give_up(wc);
            return;
        }
    }
}

// tiles [t0, t1) of an op that CTA c owns: the first tiles_r CTAs take one tile more
__device__ __forceinline__ void tile_range(const ChainOp& op, int c, int& t0, int& t1) {
    t0 = c * op.tiles_q + min(c, op.tiles_r);
    t1 = t0 + op.tiles_q + (c < op.tiles_r ? 1 : 0);
}
// The op record into registers: independent 16-byte loads.
__device__ __forceinline__ ChainOp load_op(const ChainOp* p) {
    union U {
        ChainOp op;
        uint4 q[kOpRecordQuads];
        __device__ U() {}
    } u;
    const uint4* src = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < kOpRecordQuads; ++i)
        u.q[i] = __ldg(src + i);
    return u.op;
}
__device__ __forceinline__ int div_magic(int x, unsigned magic) {
    return (int)(((unsigned)x * magic) >> 16);
}

__global__ void __launch_bounds__(kChainThreads, 1) gemv_chain_kernel(const ChainArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    // ---- shared-memory carve-up (offsets from the base: the pointers stay shared-space) ---
    constexpr int kOffEmpty = 8 * kEntries;
    constexpr int kOffHfull = kOffEmpty + 8 * kEntries;
    constexpr int kOffHempty = kOffHfull + 8 * kComputeWarps;
    constexpr int kOffItemVbeg = kOffHempty + 8 * kComputeWarps;
    constexpr int kOffItemOff = kOffItemVbeg + 8 * kEntries;
    constexpr int kOffHand = kOffItemOff + 4 * kEntries;
    constexpr int kOffHandSent = kOffHand + 4 * 8 * kComputeWarps;
    // A ring of op records: the producer thread, which runs ahead of the compute warps, copies
    // record i in when it starts on op i's weights, so that no compute warp waits on a global
    // load for a field (the compiler sinks such loads to their first use).
    constexpr int kOffOpBars = (kOffHandSent + 4 * kComputeWarps + 7) & ~7;
    constexpr int kOffOps = (kOffOpBars + 2 * 8 * kOpSlots + 15) & ~15;
    constexpr int kOffQs = kOffOps + kOpSlots * (int)sizeof(ChainOp);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);                  // [kEntries]
    uint64_t* empty = reinterpret_cast<uint64_t*>(smem + kOffEmpty);     // [kEntries]
    uint64_t* hfull = reinterpret_cast<uint64_t*>(smem + kOffHfull);     // [kComputeWarps]
    uint64_t* hempty = reinterpret_cast<uint64_t*>(smem + kOffHempty);   // [kComputeWarps]
    unsigned long long* item_vbeg =
        reinterpret_cast<unsigned long long*>(smem + kOffItemVbeg);      // [kEntries]
    uint32_t* item_off = reinterpret_cast<uint32_t*>(smem + kOffItemOff);  // [kEntries]
    float* hand = reinterpret_cast<float*>(smem + kOffHand);             // [kComputeWarps][8]
    // hand-overs sent to each warp so far (the phase of its `hempty` barrier); one sender at a
    // time per receiver, senders of different ops are ordered by the per-op barrier
    volatile uint32_t* hand_sent = reinterpret_cast<volatile uint32_t*>(smem + kOffHandSent);
    const int gmax = a.kmax / 128;
    // per group: {activation scale, -8 * sum of the even-k codes}, two buffers (op parity)
    int2* s_qs = reinterpret_cast<int2*>(smem + kOffQs);                 // [2][gmax]
    const int off_xq = kOffQs + 2 * 8 * gmax;             // [2][gmax * kXqStride], 16-aligned
    uint8_t* s_xq = smem + off_xq;
    const int xq_bytes = gmax * kXqStride;
    const int off_ring = (off_xq + 2 * xq_bytes + 127) & ~127;
    uint8_t* ring = smem + off_ring;
    const uint32_t smem_base = smem_u32(smem);
    ChainOp* s_ops = reinterpret_cast<ChainOp*>(smem + kOffOps);
    uint64_t* ops_full = reinterpret_cast<uint64_t*>(smem + kOffOpBars);   // [kOpSlots]
    uint64_t* ops_empty = ops_full + kOpSlots;                             // [kOpSlots]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    WaitCtx wc = {a.status, a.abort_word, false};

    if (threadIdx.x == 0) {
        for (int e = 0; e < kEntries; ++e) {
            mbar_init(&full[e], 1);
            mbar_init(&empty[e], kEmptyCount * kTpiMax);
        }
        for (int w = 0; w < kComputeWarps; ++w) {
            mbar_init(&hfull[w], 1);
            mbar_init(&hempty[w], 1);
            hand_sent[w] = 0;
        }
        for (int i = 0; i < kOpSlots; ++i) {
            mbar_init(&ops_full[i], 1);
            mbar_init(&ops_empty[i], kComputeWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int cta = blockIdx.x;

    // =============================== producer warp ====================================
    if (warp == kComputeWarps) {
        if (lane != 0)
            return;
        // One thread does all of this once per tile: no division anywhere (a 64-bit modulo by
        // a run-time value costs hundreds of cycles on one thread and throttled the stream).
        unsigned long long head_v = 0;  // virtual ring position (monotonic, gaps included)
        uint32_t head_off = 0;          // the same position inside the ring
        unsigned j = 0, tail = 0;       // next item, oldest item not yet released
        const uint32_t R = (uint32_t)a.ring_bytes;
        for (int oi = 0; oi < a.count; ++oi) {
            const ChainOp op = load_op(a.ops + oi);
            {
                const int slot = oi & (kOpSlots - 1);
                if (oi >= kOpSlots)  // every compute warp is done with the record that was here
                    mbar_wait(&ops_empty[slot], ((unsigned)oi / kOpSlots - 1u) & 1u, wc, 100);
                s_ops[slot] = op;
                mbar_arrive(&ops_full[slot], 1);
            }
            int t0, t1;
            tile_range(op, cta, t0, t1);
            const uint32_t nib_bytes = (uint32_t)op.groups * 512u;
            const uint32_t scl_bytes = (uint32_t)op.groups * (uint32_t)op.scl_group_bytes;
            const uint8_t* const nib = op.nib;
            const uint8_t* const scl = op.scl;
            const int tpi = op.tpi;
            const bool traced = a.trace != nullptr && cta == a.trace_cta;
            long long waited = 0;
            // an item = up to tpi consecutive tiles: their nibble streams are one contiguous
            // run of the nibble plane, their scales one run of the scale plane
            for (int t = t0; t < t1; t += tpi) {
                const int nt = min(tpi, t1 - t);
                const uint32_t size = (uint32_t)nt * (nib_bytes + scl_bytes);
                const int e = (int)(j & (kEntries - 1));
                unsigned long long v0 = head_v;
                uint32_t off = head_off;
                if (off + size > R) {  // no item straddles the end of the ring
                    v0 += R - off;
                    off = 0;
                }
                const unsigned long long v1 = v0 + size;
                // space: everything from the oldest unreleased item's begin up to v1 must fit
                while (tail < j && (v1 - item_vbeg[tail & (kEntries - 1)] > R ||
                                    j - tail >= (unsigned)kEntries)) {
                    const long long w0 = traced ? clock64() : 0;
                    mbar_wait(&empty[tail & (kEntries - 1)], (tail / kEntries) & 1u, wc, 200);
                    if (traced)
                        waited += clock64() - w0;
                    ++tail;
                }
                item_vbeg[e] = head_v;
                item_off[e] = off;
                head_v = v1;
                head_off = off + size;  // <= R; the next item wraps if it does not fit
                mbar_expect_tx(&full[e], size);
                bulk_g2s(ring + off, nib + (size_t)t * nib_bytes, (uint32_t)nt * nib_bytes,
                         &full[e]);
                bulk_g2s(ring + off + (uint32_t)nt * nib_bytes, scl + (size_t)t * scl_bytes,
                         (uint32_t)nt * scl_bytes, &full[e]);
                // the release count of an entry is that of a full item: make up for the
                // tiles this one does not have
                if (nt < kTpiMax)
                    mbar_arrive(&empty[e], kEmptyCount * (unsigned)(kTpiMax - nt));
                ++j;
                if (traced && t + tpi >= t1)
                    a.trace[oi * kTraceSlots + 7] = waited;
            }
        }
        // Shared memory must not be released under copies in flight: the consumers wait for
        // every item in the normal course; after an abort they do not, so wait here (bounded).
        if (*reinterpret_cast<volatile int*>(a.abort_word) != 0) {
            for (unsigned q = (j > (unsigned)kEntries ? j - kEntries : 0); q < j; ++q) {
                const long long t0c = clock64();
                while (!mbar_try_wait(&full[q & (kEntries - 1)], (q / kEntries) & 1u))
                    if ((unsigned long long)(clock64() - t0c) > kChainWaitCycles)
                        break;
            }
        }
        return;
    }

    // =============================== compute warps ====================================
    const int gl = lane >> 3, row = lane & 7;
    const int half = lane >> 4, h = lane & 15;
    unsigned j_base = 0;      // item index of this CTA's first tile of the current op
    unsigned recv_count = 0;  // hand-overs this warp has received (phase of its `hfull`)
    int buf = 1;              // quantised-activation buffer in use (flips before each quantisation)

    for (int oi = 0; oi < a.count; ++oi) {
        mbar_wait(&ops_full[oi & (kOpSlots - 1)], ((unsigned)oi / kOpSlots) & 1u, wc);
        const ChainOp& op = s_ops[oi & (kOpSlots - 1)];
        const int G = op.groups;
        // Consecutive ops on one input vector share its quantisation, as the reference's batch
        // entry point does (kernels/matmul_w4.cpp:438-462): the buffer flips only when a new
        // vector is quantised.
        if (!op.reuse_x)
            buf ^= 1;
        uint8_t* xq = s_xq + buf * xq_bytes;
        int2* qs_b = s_qs + buf * gmax;
        const uint32_t xq_addr = smem_base + (uint32_t)(off_xq + buf * xq_bytes);
        const uint32_t qs_addr = smem_base + (uint32_t)(kOffQs + buf * gmax * 8);

        const bool traced = a.trace != nullptr && cta == a.trace_cta && threadIdx.x == 0;
        // time stamps stay in registers until the op is over: a store would queue behind the
        // shared-memory traffic and distort what it measures
        long long ts0 = 0, ts1 = 0, ts2 = 0, ts3 = 0, ts5 = 0;
        if (traced)
            ts0 = clock64();
        // ---- activations of this op: wait for them (tagged words), quantise per 128 ------
        // A half-warp takes a group; lane h holds k = 32*i + 2h and 32*i + 2h + 1 for the four
        // 32-blocks i, so that each of its four loads covers 256 (tagged) or 128 (plain)
        // contiguous bytes per half-warp.  (148 SMs all read the whole vector: with one lane
        // per 64-byte stretch every load touched 32 sectors and the L2's request rate, not its
        // bandwidth, set the hand-over time.)
        if (!op.reuse_x) {
            const unsigned want = a.tag_base + op.tag_in;
            const long long t0 = clock64();
#pragma unroll 1
            for (int base = warp * 2; base < G; base += kComputeWarps * 2) {
                const int g = base + half;
                const bool live = g < G;
                float v[8];  // v[2i] even k, v[2i+1] odd k of 32-block i
                if (op.x_tag != nullptr) {
                    const volatile ulonglong2* src = reinterpret_cast<const volatile ulonglong2*>(
                        op.x_tag + (size_t)(live ? g : 0) * 128 + h * 2);
                    // While the producers still run, only the first lane of the half-warp looks,
                    // at one word, with a pause between looks.
                    unsigned spins = 0;
                    for (;;) {
                        bool seen = h != 0 || !live || wc.aborted ||
                                    (unsigned)(src[48].y >> 32) == want;
                        if (__all_sync(0xffffffffu, seen))
                            break;
                        __nanosleep(40);
                        if ((++spins & 15u) == 0) {
                            if (*reinterpret_cast<volatile int*>(wc.abort_word) != 0)
                                wc.aborted = true;
                            else if ((unsigned long long)(clock64() - t0) > kChainWaitCycles)
                                give_up(wc);
                        }
                    }
                    for (;;) {
                        bool ok = true;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            unsigned long long w0, w1;  // one 16-byte load: words k, k+1
                            asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];"
                                         : "=l"(w0), "=l"(w1)
                                         : "l"(src + i * 16));
                            ok = ok && (unsigned)(w0 >> 32) == want && (unsigned)(w1 >> 32) == want;
                            v[2 * i] = __uint_as_float((unsigned)w0);
                            v[2 * i + 1] = __uint_as_float((unsigned)w1);
                        }
                        ok = ok || !live || wc.aborted;
                        if (__all_sync(0xffffffffu, ok))
                            break;
                        __nanosleep(20);
                        if ((++spins & 15u) == 0) {
                            if (*reinterpret_cast<volatile int*>(wc.abort_word) != 0)
                                wc.aborted = true;
                            else if ((unsigned long long)(clock64() - t0) > kChainWaitCycles)
                                give_up(wc);
                        }
                    }
                } else {
                    const float* src = op.x_ext + (size_t)(live ? g : 0) * 128 + h * 2;
                    if ((reinterpret_cast<uintptr_t>(op.x_ext) & 7) == 0) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 p = *reinterpret_cast<const float2*>(src + i * 32);
                            v[2 * i] = p.x;
                            v[2 * i + 1] = p.y;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            v[2 * i] = src[i * 32];
                            v[2 * i + 1] = src[i * 32 + 1];
                        }
                    }
                }
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    amax = fmaxf(amax, fabsf(v[i]));
                // max is exact and order-free: the butterfly gives the sequential loop's value
#pragma unroll
                for (int off = 8; off > 0; off >>= 1)
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                float scale, inv;
                b2w4_quant_params(amax, scale, inv);
                int c[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    c[i] = b2w4_quant_code(v[i], inv);
                int esum = c[0] + c[2] + c[4] + c[6];  // the even-k codes; integer: order-free
#pragma unroll
                for (int off = 8; off > 0; off >>= 1)
                    esum += __shfl_xor_sync(0xffffffffu, esum, off);
                if (live) {
                    if (h == 0)
                        qs_b[g] = make_int2(__float_as_int(scale), -8 * esum);
                    // 32-block i is stored as 16 even-k codes then 16 odd-k codes
                    signed char* blk = reinterpret_cast<signed char*>(xq) + g * kXqStride + h;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        blk[i * 32] = (signed char)c[2 * i];
                        blk[i * 32 + 16] = (signed char)c[2 * i + 1];
                    }
                }
            }
        }
        // Codes and scales visible to every warp, and every warp is done with the buffer the
        // NEXT quantisation will overwrite.  Ops that reuse the vector need no barrier: the
        // warps run on, held only by the arrival of their tiles.
        if (!op.reuse_x)
            compute_barrier();
        long long ts2b = 0;
        if (traced) {
            ts2 = clock64();
            const uint32_t probe = lds32(smem_base + kOffOps);  // one shared-memory load
            if (probe != 0x12345678u)  // the clock is read once the load has returned
                ts2b = clock64();
        }

        // ---- this CTA's tiles of the op ---------------------------------------------------
        int t0, t1;
        tile_range(op, cta, t0, t1);
        const int L = t1 - t0;
        // A team = `team` consecutive warps on one tile; member m owns a contiguous range of the
        // tile's iterations (4 groups each).
        const int team = op.team;
        const int teams = op.teams;
        const int my_team = div_magic(warp, op.team_magic);
        // In a team of two, which warp of the pair is member 0 alternates so that the four warp
        // schedulers (warp % 4) see the same mix of short and long members.
        const int member = team == 2 ? ((warp + (warp >> 2)) & 1) : warp - my_team * team;
        const int ipt = op.ipt;
        // floor split: when the iterations do not divide evenly the LATER members get one more.
        // A later member needs the chain value of the earlier ones after its own integer sums
        // are done; with less work upstream the value is there when it looks for it.
        const int ib = div_magic(member * ipt, op.team_magic);
        const int ie = div_magic((member + 1) * ipt, op.team_magic);
        const uint32_t nib_bytes = (uint32_t)G * 512u;
        const uint32_t scl_bytes = (uint32_t)G * (uint32_t)op.scl_group_bytes;
        const int tpi = op.tpi;
        const bool scl16 = op.scl_group_bytes == 16;
        const unsigned tag_out = a.tag_base + op.tag_out;
        const int n_out = op.n, act = op.activation, act_b = op.act_n_begin, act_l = op.act_n_len;
        unsigned long long* const y_tag = op.y_tag;
        float* const y_ext = op.y_ext;
        const int world = op.world;

        if (traced)
            ts1 = clock64();
        if (my_team < teams) {
#pragma unroll 1
            for (int lt = my_team; lt < L; lt += teams) {
                const int item = div_magic(lt, op.tpi_magic), ti = lt - item * tpi;
                const int nt = min(tpi, L - item * tpi);
                const unsigned j = j_base + (unsigned)item;
                const int e = (int)(j & (kEntries - 1));
                if (traced && lt == my_team)
                    ts5 = clock64();
                mbar_wait(&full[e], (j / kEntries) & 1u, wc);
                if (traced && lt == my_team)
                    ts3 = clock64();
                const uint32_t item_addr = smem_base + (uint32_t)off_ring + item_off[e];
                // this lane's row inside the tile's nibble stream / scale block
                const uint32_t w_row = item_addr + (uint32_t)ti * nib_bytes + (uint32_t)row * 16u;
                const uint32_t s_row = item_addr + (uint32_t)nt * nib_bytes +
                                       (uint32_t)ti * scl_bytes + (uint32_t)row * (scl16 ? 2u : 4u);
                // One iteration = groups 4*it .. 4*it+3, one per 8-lane group slot.  The integer
                // work of iteration it+1 is issued before the order-sensitive fp32 chain of
                // iteration it: a member that must wait for the chain value of the groups
                // before its own has its integer sums ready when the value arrives.
                float acc = 0.f;
                bool have_acc = member == 0, released = false;
                float df, sc;
                {
                    const int g = min(ib * 4 + gl, G - 1);
                    const uint2 qs = lds64(qs_addr + (uint32_t)g * 8u);
                    df = (float)group_dot(w_row + (uint32_t)g * 512u,
                                          xq_addr + (uint32_t)(g * kXqStride), (int)qs.y);
                    const float ws = scl16 ? __half2float(__ushort_as_half((unsigned short)lds16(
                                                 s_row + (uint32_t)g * 16u)))
                                           : __uint_as_float(lds32(s_row + (uint32_t)g * 32u));
                    sc = __fmul_rn(ws, __uint_as_float(qs.x));
                }
#pragma unroll 1
                for (int it = ib; it < ie; ++it) {
                    float df_n = 0.f, sc_n = 0.f;
                    if (it + 1 < ie) {
                        const int g = min((it + 1) * 4 + gl, G - 1);
                        const uint2 qs = lds64(qs_addr + (uint32_t)g * 8u);
                        df_n = (float)group_dot(w_row + (uint32_t)g * 512u,
                                                xq_addr + (uint32_t)(g * kXqStride), (int)qs.y);
                        const float ws =
                            scl16 ? __half2float(__ushort_as_half(
                                        (unsigned short)lds16(s_row + (uint32_t)g * 16u)))
                                  : __uint_as_float(lds32(s_row + (uint32_t)g * 32u));
                        sc_n = __fmul_rn(ws, __uint_as_float(qs.x));
                    }
                    if (!released && it + 2 >= ie) {
                        // this member's last read of the slot is behind it
                        released = true;
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&empty[e], kEmptyCount / (unsigned)team);
                    }
                    if (!have_acc) {  // the chain value of the groups before mine
                        mbar_wait(&hfull[warp], recv_count & 1u, wc);
                        acc = hand[warp * 8 + row];
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&hempty[warp], 1);
                        ++recv_count;
                        have_acc = true;
                    }
                    // the four groups of the iteration meet in the lanes of group slot 0 and
                    // are folded in ascending order
                    const float d1 = __shfl_down_sync(0xffffffffu, df, 8);
                    const float d2 = __shfl_down_sync(0xffffffffu, df, 16);
                    const float d3 = __shfl_down_sync(0xffffffffu, df, 24);
                    const float s1 = __shfl_down_sync(0xffffffffu, sc, 8);
                    const float s2 = __shfl_down_sync(0xffffffffu, sc, 16);
                    const float s3 = __shfl_down_sync(0xffffffffu, sc, 24);
                    const int g0 = it * 4;
                    acc = __fmaf_rn(df, sc, acc);
                    if (g0 + 1 < G)
                        acc = __fmaf_rn(d1, s1, acc);
                    if (g0 + 2 < G)
                        acc = __fmaf_rn(d2, s2, acc);
                    if (g0 + 3 < G)
                        acc = __fmaf_rn(d3, s3, acc);
                    df = df_n;
                    sc = sc_n;
                }
                if (member + 1 < team) {
                    // hand the chain value to the member that owns the next groups
                    const int next = team == 2 ? (warp ^ 1) : warp + 1;
                    const uint32_t sent = hand_sent[next];
                    mbar_wait(&hempty[next], (sent & 1u) ^ 1u, wc);
                    if (gl == 0)
                        hand[next * 8 + row] = acc;
                    __syncwarp();
                    if (lane == 0) {
                        hand_sent[next] = sent + 1u;
                        mbar_arrive(&hfull[next], 1);
                    }
                } else if (gl == 0) {
                    const int n = (t0 + lt) * 8 + row;
                    if (n < n_out) {
                        if (b2w4_act_applies(n, act, act_b, act_l, n_out))
                            acc = chain_activation(acc, act);
                        const unsigned long long word =
                            ((unsigned long long)tag_out << 32) | __float_as_uint(acc);
                        if (world == 0) {
                            y_tag[n] = word;
                            if (y_ext)
                                y_ext[n] = acc;
                        } else {
                            // the all-gather is this store: every rank's scratch (this one's
                            // included) gets the tagged word over the peer mappings, and a
                            // consumer op on any rank polls its own scratch as on one GPU
                            const unsigned long long at = op.tag_off + (unsigned)n;
#pragma unroll
                            for (int p = 0; p < kTpMaxWorld; ++p)
                                if (p < world) {
                                    a.scratch_peers[p][at] = word;
                                    if (op.y_peers[p])
                                        op.y_peers[p][op.n_offset + n] = acc;
                                }
                        }
                    }
                }
            }
        }
        j_base += (unsigned)div_magic(L + tpi - 1, op.tpi_magic);
        __syncwarp();
        if (lane == 0)  // this warp is done with the op's record
            mbar_arrive(&ops_empty[oi & (kOpSlots - 1)], 1);
        if (traced) {
            long long* tr = a.trace + oi * kTraceSlots;
            tr[0] = ts0, tr[1] = ts1, tr[2] = ts2, tr[3] = ts3, tr[5] = ts5;
            tr[4] = clock64();
            tr[6] = ts2b;
        }
    }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct b2w4_chain {
    int count = 0;
    int device = 0;
    ChainOp* ops_dev = nullptr;
    unsigned long long* tagged = nullptr;  // all ops' tagged outputs, back to back
    size_t tagged_words = 0;
    float* x_in = nullptr;   // chain-owned input vector (ops that name no x)
    int x_in_len = 0;
    float* y_out = nullptr;  // chain-owned plain output of the last op (when it names no y)
    int y_out_len = 0;
    int kmax = 0;
    int ring_bytes = 0;
    size_t smem_bytes = 0;
    unsigned next_tag = 0;   // tags used so far (the buffer is zeroed when they run out)
    size_t weight_bytes = 0;
    long long* trace = nullptr;  // profiling hook, see ChainArgs
    int trace_cta = 0;
    // tensor-parallel form: the tagged scratch belongs to the caller (peer-mapped buffers)
    int world = 1;
    unsigned long long* scratch_peers[kTpMaxWorld] = {nullptr};
};

namespace {

size_t chain_fixed_smem(int kmax) {  // everything before the ring, as the kernel lays it out
    const int gmax = kmax / 128;
    size_t b = 8 * kEntries * 3 + 8 * kComputeWarps * 2 + 4 * kEntries + 4 * 8 * kComputeWarps +
               4 * kComputeWarps;
    b = (b + 15) & ~size_t(15);
    b += 2 * 8 * kOpSlots + 16 + kOpSlots * sizeof(ChainOp) + 2 * 8 * (size_t)gmax + 2 * (size_t)gmax * kXqStride;
    return (b + 127) & ~size_t(127);
}

// warps per tile: as many as keep every compute warp busy on the op's tiles per CTA, and no
// more than the tile has iterations (every member then owns at least one)
int chain_team_size(int tiles, int groups, int ctas) {
    const int per_cta = (tiles + ctas - 1) / ctas;
    const int ipt = (groups + 3) / 4;
    const int team = std::max(1, std::min(kMaxTeamSize, kComputeWarps / std::max(1, per_cta)));
    return std::min(team, ipt);
}

}  // namespace

namespace {

// Builds a chain; shards / group are null for one GPU.
int chain_create(b2w4_ctx* ctx, const b2w4_chain_op* ops, const b2w4_chain_shard* shards,
                 const b2w4_tp_group* group, int count, b2w4_chain** out) {
    if (!ctx || !out)
        return B2W4_E_INVALID;
    *out = nullptr;
    if (!ops || count < 1 || count > 4096)
        return b2w4_fail(ctx, B2W4_E_INVALID, "chain: 1..4096 ops (got %d)", count);
    const bool tp = group != nullptr;
    if (tp) {
        if (!shards || group->world < 1 || group->world > kTpMaxWorld || group->rank < 0 ||
            group->rank >= group->world)
            return b2w4_fail(ctx, B2W4_E_INVALID, "chain_tp: bad group or no shard table");
        for (int p = 0; p < group->world; ++p)
            if (!group->stage_peers[p] || (reinterpret_cast<uintptr_t>(group->stage_peers[p]) & 15))
                return b2w4_fail(ctx, B2W4_E_INVALID, "chain_tp: null or unaligned scratch of rank %d",
                                 p);
    }
    std::vector<ChainOp> dev(count);
    std::vector<size_t> y_at(count);
    size_t words = 0;
    int kmax = 0, x_in_len = 0;
    uint32_t max_item = 0;
    size_t weight_bytes = 0;
    auto full_n = [&](int i) { return tp ? shards[i].n_full : ops[i].w->n; };
    for (int i = 0; i < count; ++i) {
        const b2w4_chain_op& o = ops[i];
        if (!o.w)
            return b2w4_fail(ctx, B2W4_E_INVALID, "chain: op %d has no weight", i);
        if (o.activation < B2W4_NONE || o.activation > B2W4_RELU_SQUARED)
            return b2w4_fail(ctx, B2W4_E_INVALID, "chain: op %d: unknown activation %d", i,
                             o.activation);
        if (tp && (shards[i].n_offset < 0 || shards[i].n_offset + o.w->n > shards[i].n_full ||
                   o.y_dev))
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "chain_tp: op %d: rows [%d, %d) of %d (and y_dev must be NULL: plain "
                             "rows go to y_peers)", i, shards[i].n_offset,
                             shards[i].n_offset + o.w->n, shards[i].n_full);
        if (o.x_from >= i || o.x_from < -1)
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "chain: op %d takes its input from op %d (must be an earlier op, "
                             "or -1 for x_dev / the chain's input vector)", i, o.x_from);
        if (o.x_from >= 0 && (o.x_offset < 0 || o.x_offset + o.w->k > full_n(o.x_from)))
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "chain: op %d reads [%d, %d) of op %d's %d outputs", i, o.x_offset,
                             o.x_offset + o.w->k, o.x_from, full_n(o.x_from));
        y_at[i] = words;
        words += (size_t)((full_n(i) + 1) & ~1);  // 16-byte aligned rows
        kmax = std::max(kmax, o.w->k);
        if (o.x_from < 0 && !o.x_dev)
            x_in_len = std::max(x_in_len, o.w->k);
        max_item = std::max(max_item, (uint32_t)o.w->groups * (512u + (o.w->scales_fp16 ? 16u : 32u)));
        weight_bytes += o.w->nib_bytes + o.w->scl_bytes;
    }
    if (words * 8 > (size_t)1 << 30)
        return b2w4_fail(ctx, B2W4_E_INVALID, "chain: %zu output values exceed the 1 GiB scratch",
                         words);
    const size_t fixed = chain_fixed_smem(kmax);
    const size_t budget = 227 * 1024;
    if (fixed + max_item > budget)
        return b2w4_fail(ctx, B2W4_E_INVALID, "chain: K=%d does not fit one SM's shared memory",
                         kmax);
    b2w4_chain* c = new (std::nothrow) b2w4_chain();
    if (!c)
        return b2w4_fail(ctx, B2W4_E_NOMEM, "out of host memory");
    c->count = count;
    c->device = ctx->device;
    c->kmax = kmax;
    c->ring_bytes = (int)((budget - fixed) & ~size_t(127));
    c->smem_bytes = fixed + c->ring_bytes;
    c->tagged_words = words;
    c->weight_bytes = weight_bytes;
    c->x_in_len = x_in_len;
    const b2w4_chain_op& last = ops[count - 1];
    c->y_out_len = (last.y_dev || tp) ? 0 : last.w->n;
    cudaError_t e = cudaSuccess;
    unsigned long long* scratch = nullptr;
    if (tp) {
        c->world = group->world;
        for (int p = 0; p < group->world; ++p)
            c->scratch_peers[p] = static_cast<unsigned long long*>(group->stage_peers[p]);
        scratch = c->scratch_peers[group->rank];
    } else {
        e = cudaMalloc(reinterpret_cast<void**>(&c->tagged), words * 8);
        if (e == cudaSuccess)
            e = cudaMemset(c->tagged, 0, words * 8);
        scratch = c->tagged;
    }
    if (e == cudaSuccess)
        e = cudaMalloc(reinterpret_cast<void**>(&c->ops_dev), sizeof(ChainOp) * count);
    if (e == cudaSuccess && c->x_in_len)
        e = cudaMalloc(reinterpret_cast<void**>(&c->x_in), sizeof(float) * c->x_in_len);
    if (e == cudaSuccess && c->y_out_len)
        e = cudaMalloc(reinterpret_cast<void**>(&c->y_out), sizeof(float) * c->y_out_len);
    if (e != cudaSuccess) {
        b2w4_chain_destroy(ctx, c);
        return b2w4_fail(ctx, B2W4_E_NOMEM, "chain: device allocation: %s", cudaGetErrorString(e));
    }
    for (int i = 0; i < count; ++i) {
        const b2w4_chain_op& o = ops[i];
        ChainOp& d = dev[i];
        memset(&d, 0, sizeof(d));
        d.nib = reinterpret_cast<const uint8_t*>(o.w->nib);
        d.scl = reinterpret_cast<const uint8_t*>(o.w->scl);
        if (o.x_from >= 0) {
            d.x_tag = scratch + y_at[o.x_from] + o.x_offset;
            d.tag_in = (unsigned)o.x_from + 1u;
        } else {
            d.x_ext = o.x_dev ? o.x_dev : c->x_in;
        }
        d.y_tag = scratch + y_at[i];
        d.y_ext = o.y_dev ? o.y_dev : (i == count - 1 ? c->y_out : nullptr);
        d.n = o.w->n;
        d.groups = o.w->groups;
        d.tiles_q = o.w->tiles / ctx->sm_count;
        d.tiles_r = o.w->tiles % ctx->sm_count;
        d.ipt = (o.w->groups + 3) / 4;
        d.scl_group_bytes = o.w->scales_fp16 ? 16 : 32;
        d.team = chain_team_size(o.w->tiles, o.w->groups, ctx->sm_count);
        d.teams = kComputeWarps / d.team;
        d.team_magic = 65536u / (unsigned)d.team + 1u;
        {
            const uint32_t tile_bytes = (uint32_t)o.w->groups * (512u + (o.w->scales_fp16 ? 16u : 32u));
            d.tpi = (int)std::max(1u, std::min((uint32_t)kTpiMax, kItemBytesCap / tile_bytes));
            d.tpi_magic = 65536u / (unsigned)d.tpi + 1u;
        }
        d.tag_out = (unsigned)i + 1u;
        d.activation = o.activation;
        d.act_n_begin = o.act_n_begin;
        d.act_n_len = o.act_n_len;
        d.reuse_x = i > 0 && o.x_from < 0 && ops[i - 1].x_from < 0 &&
                    (o.x_dev ? o.x_dev : c->x_in) == (ops[i - 1].x_dev ? ops[i - 1].x_dev : c->x_in) &&
                    o.w->k == ops[i - 1].w->k;
        d.world = tp ? group->world : 0;  // 0: the one-GPU epilogue
        if (tp) {
            d.n_offset = shards[i].n_offset;
            d.tag_off = y_at[i] + (size_t)shards[i].n_offset;
            for (int p = 0; p < group->world; ++p)
                d.y_peers[p] = static_cast<float*>(shards[i].y_peers[p]);
        }
    }
    e = cudaMemcpy(c->ops_dev, dev.data(), sizeof(ChainOp) * count, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        b2w4_chain_destroy(ctx, c);
        return b2w4_fail(ctx, B2W4_E_CUDA, "chain: upload of the op list: %s",
                         cudaGetErrorString(e));
    }
    *out = c;
    return B2W4_OK;
}

}  // namespace

extern "C" {

int b2w4_chain_create(b2w4_ctx* ctx, const b2w4_chain_op* ops, int count, b2w4_chain** out) {
    return chain_create(ctx, ops, nullptr, nullptr, count, out);
}

int b2w4_chain_create_tp(b2w4_ctx* ctx, const b2w4_chain_op* ops, const b2w4_chain_shard* shards,
                         int count, const b2w4_tp_group* group, b2w4_chain** out) {
    if (!group)
        return ctx ? b2w4_fail(ctx, B2W4_E_INVALID, "chain_tp: no group") : B2W4_E_INVALID;
    return chain_create(ctx, ops, shards, group, count, out);
}

size_t b2w4_chain_scratch_words(const b2w4_chain_shard* shards, int count) {
    size_t words = 0;
    for (int i = 0; shards && i < count; ++i)
        words += (size_t)((shards[i].n_full + 1) & ~1);
    return words;
}

void b2w4_chain_destroy(b2w4_ctx* ctx, b2w4_chain* c) {
    if (!c)
        return;
    if (ctx)
        cudaStreamSynchronize(ctx->stream);
    if (c->tagged)
        cudaFree(c->tagged);
    if (c->ops_dev)
        cudaFree(c->ops_dev);
    if (c->x_in)
        cudaFree(c->x_in);
    if (c->y_out)
        cudaFree(c->y_out);
    delete c;
}

int b2w4_chain_run(b2w4_ctx* ctx, b2w4_chain* c) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!c || c->device != ctx->device)
        return b2w4_fail(ctx, B2W4_E_INVALID, "chain_run: no chain, or a chain of another device");
    // tags: one per op and run; when the 32-bit space runs out the scratch goes back to zero
    if (c->next_tag > 0xFFFFFFFFu - (unsigned)c->count - 1u) {
        if (c->world > 1)  // the scratch is the caller's and every rank would have to agree
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "chain_run: tag space of a tensor-parallel chain exhausted; "
                             "recreate the chain on zeroed scratch buffers");
        B2W4_CUDA(ctx, cudaMemsetAsync(c->tagged, 0, c->tagged_words * 8, ctx->stream));
        c->next_tag = 0;
    }
    ChainArgs a;
    a.ops = c->ops_dev;
    a.count = c->count;
    a.tag_base = c->next_tag;
    a.status = ctx->status_dev;
    a.abort_word = ctx->flag_dev + 2;
    a.ring_bytes = c->ring_bytes;
    a.kmax = c->kmax;
    a.trace = c->trace;
    a.trace_cta = c->trace_cta;
    for (int p = 0; p < kTpMaxWorld; ++p)
        a.scratch_peers[p] = c->scratch_peers[p];
    c->next_tag += (unsigned)c->count;
    static b2w4_smem_optin configured;
    B2W4_CUDA(ctx, b2w4_opt_in_smem(ctx, gemv_chain_kernel, c->smem_bytes, configured));
    static int resident[kMaxDevices] = {0};  // co-residency checked once per device
    if (!resident[ctx->device]) {
        int per_sm = 0;
        B2W4_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                           &per_sm, gemv_chain_kernel, kChainThreads, c->smem_bytes));
        if (per_sm < 1)
            return b2w4_fail(ctx, B2W4_E_INVALID,
                             "chain_run: the kernel does not fit an SM (%zu B shared memory)",
                             c->smem_bytes);
        resident[ctx->device] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->sm_count);
    cfg.blockDim = dim3(kChainThreads);
    cfg.dynamicSmemBytes = c->smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident: they wait for each other
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B2W4_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_chain_kernel, a));
    ctx->launches++;
    return B2W4_OK;
}

int b2w4_chain_run_host(b2w4_ctx* ctx, b2w4_chain* c, const float* x_host, int x_len,
                        float* y_host, int y_len) {
    if (!ctx)
        return B2W4_E_INVALID;
    if (!c)
        return b2w4_fail(ctx, B2W4_E_INVALID, "chain_run_host: no chain");
    if ((x_len > 0 && (!x_host || x_len > c->x_in_len)) || x_len < 0)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "chain_run_host: x_len=%d, the chain's input vector holds %d", x_len,
                         c->x_in_len);
    if ((y_len > 0 && (!y_host || y_len > c->y_out_len)) || y_len < 0)
        return b2w4_fail(ctx, B2W4_E_INVALID,
                         "chain_run_host: y_len=%d, the chain's own output holds %d", y_len,
                         c->y_out_len);
    if (x_len > 0)
        B2W4_CUDA(ctx, cudaMemcpyAsync(c->x_in, x_host, sizeof(float) * x_len,
                                       cudaMemcpyHostToDevice, ctx->stream));
    int rc = b2w4_chain_run(ctx, c);
    if (rc != B2W4_OK)
        return rc;
    if (y_len > 0)
        B2W4_CUDA(ctx, cudaMemcpyAsync(y_host, c->y_out, sizeof(float) * y_len,
                                       cudaMemcpyDeviceToHost, ctx->stream));
    return b2w4_sync(ctx);
}

int b2w4_chain_set_trace(b2w4_chain* c, long long* trace_dev, int cta) {
    if (!c || cta < 0)
        return B2W4_E_INVALID;
    c->trace = trace_dev;
    c->trace_cta = cta;
    return B2W4_OK;
}

float* b2w4_chain_input(b2w4_chain* c) { return c ? c->x_in : nullptr; }
float* b2w4_chain_output(b2w4_chain* c) { return c ? c->y_out : nullptr; }
size_t b2w4_chain_weight_bytes(const b2w4_chain* c) { return c ? c->weight_bytes : 0; }

}  // extern "C"
