// Implicit-GEMM convolution on the Blackwell tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA), int8 (s8 x s8 -> s32) and FP8 E4M3 (-> f32), with the
// requantise / bias / activation epilogue fused.
//
// GEMM view of runtime/forward_layers.rs:646-695:
//     D[pixel, filter] = sum over (ky, kx, c) of X[pixel shifted by tap (ky,kx), c] * Wt[filter, (ky,kx,c)]
// Activations are NHWC 8-bit; weights are [filters][ky][kx][c].  One CTA tile is 128 output pixels
// (a TW x TH x TN box of the output, TW*TH*TN = 128) by BN filters.  For every tap and every block of
// BK channels the producer issues two TMA loads: the input box shifted by the tap (out-of-image taps
// are zero-filled by the TMA unit, which is the reference's "skip taps outside the image") and the
// matching weight slab.  Stride-2 convolutions use one tensor map per input parity class so that the
// strided gather is again a dense box.  Every CTA fetches its own operands.
//
// Roles: warp 0 = TMA producer, warp 1 (and warp 2 in the two-issuer form, see "Pipelines" below) = MMA issuer, warp 1 owns TMEM;
// then sixteen epilogue warps (four per TMEM lane quadrant, each group of four warps taking every fourth unit of work, so every
// scheduler has four warps to hide latency with; the per-filter {multiplier, bias} table lives in shared memory so that the
// epilogue fits in 96 registers).  576 threads with one issuer, 640 with two.
// The accumulator is double buffered in TMEM so the epilogue of tile t overlaps the main loop of t+1.
// Every mbarrier wait is bounded: when it gives up it raises a status word the host reads, and all
// roles leave their loops, TMEM is released and the kernel returns.
#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "ln_conv_plan.h"

namespace {

constexpr int kMaxStages = 8;
#ifndef LN_EPILOGUE_GROUPS
#define LN_EPILOGUE_GROUPS 4
#endif
constexpr int kEpilogueGroups = LN_EPILOGUE_GROUPS;   // groups of four epilogue warps (one warp per TMEM lane quadrant); group g takes the tiles t with t % groups == g
constexpr int kEpilogueWarps = 4 * kEpilogueGroups;
// A kernel with PIPES producer / issuer pipelines has 2 * PIPES role warps (producer and MMA issuer of pipeline i are warps 2 i and
// 2 i + 1) followed by the epilogue warps; an epilogue warp's TMEM lane quadrant is its warp index modulo 4 either way.
constexpr int conv_threads(int pipes) { return 32 * (2 * pipes + kEpilogueWarps); }
constexpr int kMaxAccBufs = 8;       // accumulator tiles in TMEM: 512 columns / BN, at most 8
constexpr uint32_t kWaitLimit = 1u << 20;
// Role timing of CTA 0 (clock reads in the hot loops) is compiled in only with -DLN_CONV_ROLE_TIMING.
#ifdef LN_CONV_ROLE_TIMING
constexpr bool kRoleTiming = true;
#else
constexpr bool kRoleTiming = false;
#endif
constexpr uint32_t kWaitHintNs = 2000;  // how long one try_wait may sleep in hardware before it reports "not yet"

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the wait was abandoned (own limit reached, or another role
// already raised the CTA's abort flag).
template <bool BACKOFF = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          long long* waited = nullptr) {
    const long long t0 = kRoleTiming && waited ? clock64() : 0;
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) {
            if (kRoleTiming && waited) *waited += clock64() - t0;
            return true;
        }
        if (BACKOFF && it > 4u) __nanosleep(40);  // single-lane roles: stop stealing issue slots from the epilogue warps of this scheduler
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(status, code);
    return false;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

// CTA-pair forms (clusters of two CTAs, tcgen05 with cta_group::2), used by the tensor-pipe probe only: measured, an M = 256
// instruction over a pair takes as long as an M = 128 one on each SM, so pairs buy the convolution nothing.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once all MMAs issued so far have finished
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}
// M = 256 over the pair: rows 0..127 of A and of the accumulator live in the first CTA, 128..255 in the second; each CTA holds
// half of the N rows of B at the same shared-memory offset.
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    const uint32_t z = 0u;  // no output lane disabled
    if (KIND == LN_KIND_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
            : "memory");
    } else if (KIND == LN_KIND_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
            : "memory");
    }
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if (KIND == LN_KIND_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if (KIND == LN_KIND_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives the columns of TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
// n / d for n * d < 2^40 with the precomputed multiplier ceil(2^40 / d): one wide multiply and a shift
__device__ __forceinline__ int fast_div(int n, unsigned long long magic) { return (int)(((unsigned long long)(unsigned)n * magic) >> 40); }

// 16-byte read from shared memory (the table it reads is written once, before the epilogue warps' barrier)
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
    float4 v;
    asm("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


// int32 -> f32 (round to nearest even) on the FMA/ALU pipes only: the conversion unit shares its issue port with
// ex2/rcp, which the transcendental epilogues need.  Exact: both halves convert exactly, the fma rounds once.
__device__ __forceinline__ float i2f_alu(int v) {
    const float lo = __fadd_rn(__uint_as_float(0x4B000000u | ((uint32_t)v & 0xFFFFu)), -8388608.0f);
    const float hi = __fadd_rn(__uint_as_float(0x4B008000u ^ ((uint32_t)v >> 16)), -8421376.0f);  // (v >> 16) as a signed value
    return __fmaf_rn(hi, 65536.0f, lo);
}
// rne(a * inv_s) clamped to +-127, returned in the low byte (two's complement) of the result; no conversion unit.
__device__ __forceinline__ uint32_t quant_i8_magic(float a, float inv_s) {
    float t = __fmul_rn(a, inv_s);
    t = fminf(fmaxf(t, -127.0f), 127.0f);  // NaN -> -127
    return __float_as_uint(__fadd_rn(t, 12582912.0f));
}
__device__ __forceinline__ uint32_t pack4_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// d = a * b + c on two binary32 values with one instruction (packed f32x2 arithmetic of sm_100)
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    unsigned long long a, b, c, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(c0), "f"(c1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}

// d = a * b and d = a + b in the same packed form (each half rounds like the scalar instruction)
__device__ __forceinline__ void fmul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    unsigned long long a, b, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    unsigned long long a, b, d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
// The four signed bytes of w as floats: w ^ 0x80808080 holds byte + 128 as unsigned numbers, each placed under the exponent of
// 2^23 by one byte permute; the subtraction of 2^23 + 128 is exact.
__device__ __forceinline__ void s8x4_to_float(uint32_t w, float (&f)[4]) {
    const uint32_t x = w ^ 0x80808080u;
    float u[4];
    u[0] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650));
    u[1] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7651));
    u[2] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7652));
    u[3] = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7653));
    fadd2(f[0], f[1], u[0], u[1], -8388736.0f, -8388736.0f);
    fadd2(f[2], f[3], u[2], u[3], -8388736.0f, -8388736.0f);
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are BK bytes wide and swizzled
// with a BK-byte pattern (BK in {32, 64, 128}); groups of 8 rows are 8*BK bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, int bk) {
    const uint64_t layout = bk == 128 ? 2ull : (bk == 64 ? 4ull : 6ull);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);          // start address
    d |= 1ull << 16;                                   // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)((8u * (uint32_t)bk) >> 4) << 32;   // stride byte offset between 8-row groups
    d |= 1ull << 46;                                   // descriptor version
    d |= layout << 61;
    return d;
}


// (block index and grid size are read where they are used, not once at the top of the kernel: two values fewer to keep alive
// across the roles' loops; hoisting them cost the layers with many channels 12 %)
#define LN_FIRST_UNIT ((int)blockIdx.x)
#define LN_UNIT_STEP ((int)gridDim.x)

// Pipelines: issuing one tcgen05.mma costs its thread about 100 cycles whatever the instruction's size (the tensor pipe needs 64
// for N = 128, 136 for N = 256), and the waits and commits around every k-block cost the thread as much again, so one issuing
// thread leaves the tensor pipe idle half of the time or more.  With two pipelines (PIPES = 2) the CTA takes its tiles two at
// a time: a stage holds the activation tiles of both and the weight tile they share (consecutive tiles of a CTA have the same
// filter tile: the grid is a multiple of tiles_f), one producer fills it, and two issuing threads (warps 1 and 2) each multiply
// their own activation tile by the shared weights into their own accumulator buffer (tile t uses buffer t % nbuf, nbuf is
// even).  The two instruction streams overlap in the tensor pipe.  The epilogue takes the tiles in order, as before.
// The roles are inlined into the kernel: as functions of their own they would read the parameters through a pointer instead of
// as constant-bank operands, which costs the single-thread loops 20 to 50 % (measured).
template <int PIPES>
__device__ __forceinline__ void conv_producer_role(const ln_conv_umma_params& p) {
#include "ln_conv_layout.inc"
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        long long w_empty = 0;
        long long* pw = p.debug ? &w_empty : nullptr;
        const long long t_start = kRoleTiming ? clock64() : 0;
        if (b_res && LN_FIRST_UNIT < p.num_units) {
            mbar_arrive_expect_tx(bres_bar, (uint32_t)kblocks * b_bytes);
            for (int kb = 0; kb < kblocks; ++kb) {
                const int tap = kb / p.cblocks, c0 = (kb - tap * p.cblocks) * bk;
                tma_load_2d(bres_base + (uint32_t)kb * b_bytes, &p.tmB, tap * p.cpad + c0, 0, bres_bar);
            }
        }
        int astage = 0;
        uint32_t aphase = 0;
        for (int unit = LN_FIRST_UNIT; ok && unit < p.num_units; unit += PIPES * LN_UNIT_STEP) {
            const int tile = unit;
            const int q1 = fast_div(tile, p.magic_f), tf = tile - q1 * p.tiles_f;
            const int q2 = fast_div(q1, p.magic_w), tw = q1 - q2 * p.tiles_w;
            const int tn = fast_div(q2, p.magic_h), th = q2 - tn * p.tiles_h;
            const int ow0 = tw * p.TW, oh0 = th * p.TH, n0 = tn * p.TN, f0 = tf * bn;
            // two pipelines: the CTA's next tile as well (the same filter tile: the grid is a multiple of tiles_f), unless this was the last
            const bool has1 = PIPES == 2 && unit + LN_UNIT_STEP < p.num_units;
            int ow1 = 0, oh1 = 0, n1 = 0;
            if (has1) {
                const int u1 = fast_div(unit + LN_UNIT_STEP, p.magic_f);
                const int u2 = fast_div(u1, p.magic_w), uw = u1 - u2 * p.tiles_w;
                const int un = fast_div(u2, p.magic_h), uh = u2 - un * p.tiles_h;
                ow1 = uw * p.TW; oh1 = uh * p.TH; n1 = un * p.TN;
            }
            if (halo) {
                // per channel block: box s, then (unless the weights are resident) the weight tiles of the taps that read it
                for (int c0 = 0; ok && c0 < p.cpad; c0 += bk)
                    for (int s = 0; ok && s < 3; ++s) {
                        if (!(ok = mbar_wait(aempty_bar(astage), aphase ^ 1u, abort_flag, p.status, LN_STATUS_PRODUCER_TIMEOUT, pw))) break;
                        mbar_arrive_expect_tx(afull_bar(astage), box_bytes);
                        tma_load_4d(ring_base + (uint32_t)astage * box_bytes, &p.tmA[0], c0, ow0 - p.pad + s, oh0 - p.pad, n0, afull_bar(astage));
                        if (++astage == p.a_stages) { astage = 0; aphase ^= 1u; }
                        if (b_res) continue;
                        for (int r = 0; r < 3; ++r) {
                            if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, LN_STATUS_PRODUCER_TIMEOUT, pw))) break;
                            mbar_arrive_expect_tx(full_bar(stage), b_bytes);
                            tma_load_2d(bring_base + (uint32_t)stage * b_bytes, &p.tmB, (r * 3 + s) * p.cpad + c0, f0, full_bar(stage));
                            if (++stage == stages) { stage = 0; phase ^= 1u; }
                        }
                    }
                continue;
            }
            // taps and channel blocks in nested loops: no division on this single thread's critical path
            int wcol = 0;  // first column of the k-block in the weight matrix: tap * cpad + c0
            for (int r = 0; ok && r < p.R; ++r) {
                for (int s = 0; ok && s < p.S; ++s) {
                    int ty = r - p.pad, tx = s - p.pad, map = 0;
                    if (p.stride == 2) {
                        const int py = ty & 1, px = tx & 1;  // parity class of the tap (two's complement & 1 is non-negative)
                        ty = (ty - py) >> 1;
                        tx = (tx - px) >> 1;
                        map = py * 2 + px;
                    }
                    for (int c0 = 0; c0 < p.cpad; c0 += bk, wcol += bk) {
                        if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, LN_STATUS_PRODUCER_TIMEOUT, pw))) break;
                        const uint32_t sa = ring_base + (uint32_t)stage * stage_bytes;
                        // a stage: the activation tile (both pipelines' tiles when there are two), then the weight tile they share
                        mbar_arrive_expect_tx(full_bar(stage), PIPES == 2 && !has1 ? stage_bytes - a_bytes : stage_bytes);
                        tma_load_4d(sa, &p.tmA[map], c0, ow0 + tx, oh0 + ty, n0, full_bar(stage));
                        if (has1) tma_load_4d(sa + a_bytes, &p.tmA[map], c0, ow1 + tx, oh1 + ty, n1, full_bar(stage));
                        if (!b_res) tma_load_2d(sa + PIPES * a_bytes, &p.tmB, wcol, f0, full_bar(stage));
                        if (++stage == stages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
        if (kRoleTiming && p.debug && blockIdx.x == 0) { p.debug[0] = clock64() - t_start; p.debug[1] = w_empty; }
    }
}

template <int KIND, int PIPES>
__device__ __forceinline__ void conv_mma_role(const ln_conv_umma_params& p) {
#include "ln_conv_layout.inc"
    const uint32_t tmem_base = *tmem_slot;
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
        // instruction descriptor: accumulator type (bits 4-5: 1 = f32, 2 = s32), A and B types (bits 7-9, 10-12: 0 = E4M3 / binary16
        // depending on the kind, 1 = signed 8-bit), N / 8 and M / 16; both operands K-major
        const uint32_t idesc = (KIND == LN_KIND_I8 ? ((2u << 4) | (1u << 7) | (1u << 10)) : (1u << 4)) | ((uint32_t)(bn >> 3) << 17) |
                               ((128u >> 4) << 24);
        int stage = 0, astage = 0;
        uint32_t phase = 0, aphase = 0;
        const uint64_t desc_base = make_smem_desc(0u, bk);
        const uint32_t a_off = (uint32_t)pipe * a_bytes;  // this issuer's activation tile inside a stage
        int t = pipe;  // the CTA's tile counter: pipeline i takes the tiles t = i, i + pipes, ...
        bool ok = true;
        long long w_tempty = 0, w_full = 0, t_issue = 0, t_commit = 0;
        long long* pw1 = p.debug ? &w_tempty : nullptr;
        long long* pw2 = p.debug ? &w_full : nullptr;
        const long long t_start = kRoleTiming ? clock64() : 0;
        if (b_res && LN_FIRST_UNIT < p.num_units) ok = mbar_wait(bres_bar, 0u, abort_flag, p.status, LN_STATUS_MMA_TIMEOUT);
        for (int unit = LN_FIRST_UNIT; ok && unit < p.num_units; unit += PIPES * LN_UNIT_STEP, t += PIPES) {
            // (two pipelines: this issuer's tile is the pair's first or second; a last pair may lack the second, whose issuer then
            // only hands the stages back)
            const bool has = PIPES == 1 || unit + pipe * LN_UNIT_STEP < p.num_units;
            const int buf = t % nbuf;
            const uint32_t acc_phase = (uint32_t)(t / nbuf) & 1u;
            if (has && !(ok = mbar_wait(tempty_bar(buf), acc_phase ^ 1u, abort_flag, p.status, LN_STATUS_MMA_TIMEOUT, pw1))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * bn);
            if (halo) {
                uint32_t accumulate = 0;
                for (int cb = 0; ok && cb < p.cblocks; ++cb)
                    for (int s = 0; ok && s < 3; ++s) {
                        if (!(ok = mbar_wait(afull_bar(astage), aphase, abort_flag, p.status, LN_STATUS_MMA_TIMEOUT, pw2))) break;
                        const uint32_t sa = ring_base + (uint32_t)astage * box_bytes;
                        for (int r = 0; r < 3; ++r) {
                            uint32_t sb;
                            if (b_res) sb = bres_base + (uint32_t)((r * 3 + s) * p.cblocks + cb) * b_bytes;
                            else {
                                if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, LN_STATUS_MMA_TIMEOUT, pw2))) break;
                                sb = bring_base + (uint32_t)stage * b_bytes;
                            }
                            // the box from its row r on: 128 consecutive rows of bk bytes, aligned to the 8-row swizzle pattern
                            const uint64_t a_desc = desc_base + ((sa + (uint32_t)(r * p.TW * bk)) >> 4), b_desc = desc_base + (sb >> 4);
                            tc_mma<KIND>(d_tmem, a_desc, b_desc, idesc, accumulate);
                            if (bk == 64) tc_mma<KIND>(d_tmem, a_desc + 2u, b_desc + 2u, idesc, 1u);  // (this mode runs with 32 or 64 bytes per row)
                            accumulate = 1u;
                            if (!b_res) {
                                tc_commit(empty_bar(stage));
                                if (++stage == stages) { stage = 0; phase ^= 1u; }
                            }
                        }
                        if (!ok) break;
                        tc_commit(aempty_bar(astage));  // arrives when the MMAs above have finished reading the box
                        if (++astage == p.a_stages) { astage = 0; aphase ^= 1u; }
                    }
                if (!ok) break;
                tc_commit(tfull_bar(buf));
                continue;
            }
            for (int kb = 0; kb < kblocks; ++kb) {
                if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, LN_STATUS_MMA_TIMEOUT, pw2))) break;
                if (PIPES == 2 && !has) {
                    mbar_arrive(empty_bar(stage));
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                    continue;
                }
                const long long ti0 = kRoleTiming && p.debug ? clock64() : 0;
                // (no tcgen05 fence here: the operands were written by the TMA unit and its completion on the barrier just waited for
                // makes them visible to the tensor core; the fence after the accumulator wait above orders the MMAs behind the
                // epilogue's TMEM reads)
                // descriptors: the constant part plus the operand's address in units of 16 bytes (shared-memory addresses stay below
                // 2^18, so the sum never carries out of the 14-bit field); one instruction consumes 32 bytes of K = +2 units
                const uint32_t sa = ring_base + (uint32_t)stage * stage_bytes;
                const uint64_t a_desc = desc_base + ((sa + a_off) >> 4),
                               b_desc = desc_base + ((b_res ? bres_base + (uint32_t)kb * b_bytes : sa + PIPES * a_bytes) >> 4);
                const uint32_t acc0 = (uint32_t)(kb != 0);
                if (bk == 128) {
                    tc_mma<KIND>(d_tmem, a_desc, b_desc, idesc, acc0);
                    tc_mma<KIND>(d_tmem, a_desc + 2u, b_desc + 2u, idesc, 1u);
                    tc_mma<KIND>(d_tmem, a_desc + 4u, b_desc + 4u, idesc, 1u);
                    tc_mma<KIND>(d_tmem, a_desc + 6u, b_desc + 6u, idesc, 1u);
                } else {
                    tc_mma<KIND>(d_tmem, a_desc, b_desc, idesc, acc0);
                    if (bk == 64) tc_mma<KIND>(d_tmem, a_desc + 2u, b_desc + 2u, idesc, 1u);
                }
                const long long ti1 = kRoleTiming && p.debug ? clock64() : 0;
                tc_commit(empty_bar(stage));  // arrives when the MMAs above have finished reading this stage
                if (++stage == stages) { stage = 0; phase ^= 1u; }
                if (kRoleTiming && p.debug) { t_issue += ti1 - ti0; t_commit += clock64() - ti1; }
            }
            if (!ok) break;
            if (has) tc_commit(tfull_bar(buf));
        }
        if (kRoleTiming && p.debug && blockIdx.x == 0 && pipe == 0) { p.debug[2] = clock64() - t_start; p.debug[3] = w_tempty; p.debug[4] = w_full; p.debug[5] = t; p.debug[25] = t_issue; p.debug[26] = t_commit; }
    }
}

template <int KIND, int ACT, bool EXACT, int PIPES>
__device__ __forceinline__ void conv_epilogue_role(const ln_conv_umma_params& p) {
#include "ln_conv_layout.inc"
    const uint32_t tmem_base = *tmem_slot;
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;          // TMEM lanes 32*quad .. 32*quad+31 are the ones this warp may read
    // Which of the warps of the quadrant.  The work of the epilogue is cut into units: an accumulator tile is `subs` units of
    // bn / subs columns each (subs > 1 when TMEM holds fewer tiles than there are groups, so that all groups stay busy), and
    // group g takes the units u with u % groups == g, u counting (tile, sub) pairs in order.  Never more groups than
    // nbuf * subs: a group that starts waiting for a unit of tile t has finished its unit `groups` earlier, a unit of tile
    // t - ceil(groups / subs) or later; tiles are committed in order, so the previous use of this buffer (tile t - nbuf) has
    // been accumulated in full, which a parity wait needs.
    const int group = (warp - 2 * PIPES) >> 2;
    const int subs = p.subs, sub_cols = bn / subs;
    const int groups = nbuf * subs < kEpilogueGroups ? nbuf * subs : kEpilogueGroups;
    const int row = quad * 32 + lane;
    const int pw = row & (p.TW - 1), ph = (row >> p.log_tw) & (p.TH - 1), pn = row >> (p.log_tw + p.log_th);
    constexpr bool kTranscendental = ACT == LN_ACT_MISH || ACT == LN_ACT_SWISH || ACT == LN_ACT_LOGISTIC;
    const bool folded = !EXACT && p.mb_folded != nullptr;
    {
        // the epilogue warps bring the table in while the producer and the MMA issuer fill the pipeline
        const uint4* src = reinterpret_cast<const uint4*>(folded ? p.mb_folded : p.mb);
        for (int i = (int)threadIdx.x - 64 * PIPES; i < p.tab_bytes / 16; i += 32 * kEpilogueWarps) {
            const uint4 v = __ldg(src + i);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tab_base + 16u * (uint32_t)i), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
        asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpilogueWarps) : "memory");
    }
    int t = 0;
    bool ok = true;
    long long w_tfull = 0, dbg_ld = 0, dbg_math = 0, dbg_st = 0;
    long long* pwe = p.debug ? &w_tfull : nullptr;
    const long long t_start = kRoleTiming ? clock64() : 0;
    int turn = 0;  // unit counter modulo groups
    for (int unit = LN_FIRST_UNIT; ok && group < groups && unit < p.num_units; unit += LN_UNIT_STEP, ++t)
    for (int sub = 0; ok && sub < subs; ++sub, turn = turn + 1 == groups ? 0 : turn + 1) {
        if (turn != group) continue;  // another group of epilogue warps takes this unit
        const int tile = unit;
        const int c_begin = sub * sub_cols, c_end = c_begin + sub_cols;
        const int q1 = fast_div(tile, p.magic_f), tf = tile - q1 * p.tiles_f;
        const int q2 = fast_div(q1, p.magic_w), tw = q1 - q2 * p.tiles_w;
        const int tn = fast_div(q2, p.magic_h), th = q2 - tn * p.tiles_h;
        const int ow = tw * p.TW + pw, oh = th * p.TH + ph, n = tn * p.TN + pn, f0 = tf * bn;
        const bool valid = ow < p.OW && oh < p.OH && n < p.N;
        const int buf = t % nbuf;
        const uint32_t acc_phase = (uint32_t)(t / nbuf) & 1u;
        if (!(ok = mbar_wait<false>(tfull_bar(buf), acc_phase, abort_flag, p.status, LN_STATUS_EPILOGUE_TIMEOUT, pwe))) break;
        tc_fence_after();
        const uint32_t taddr0 = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * bn);
        const int64_t pix = ((int64_t)n * p.OH + oh) * p.OW + ow;
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
            uint32_t acc[32];
            const long long tq0 = kRoleTiming && p.debug ? clock64() : 0;
            tmem_ld_32x32(taddr0 + (uint32_t)c0, acc);
            const bool fast = KIND == LN_KIND_I8 && p.out_kind == LN_OUT_Q && f0 + c0 + 32 <= p.F;
            // where this chunk goes: with pixel-group packing the columns [j * f_real, (j + 1) * f_real) are the filters of the
            // j-th pixel of the row's group (f_real is a multiple of 32 then, so a chunk never straddles two pixels)
            int64_t opix = pix;
            int fo = f0 + c0;
            if (p.pack > 1) {
                int j = 0;
                while (fo >= p.f_real) { fo -= p.f_real; ++j; }
                opix = pix * p.pack + j;
            }
            if (fast) {
                // ---- fast path: 32 valid filters, int8 out.  The {mult, bias} pairs (two per 16-byte load) are fetched
                // while the TMEM load is in flight, so the arithmetic below runs from registers only.
                const uint32_t mtab = tab_base + 8u * (uint32_t)(f0 + c0);
                uint4 r0 = make_uint4(0u, 0u, 0u, 0u), r1 = r0;
                if (p.res != nullptr && valid) {  // residual codes of the fused shortcut, fetched while TMEM is read
                    const uint4* rp = (const uint4*)((const uint8_t*)p.res + opix * p.res_pixel_stride + fo);
                    r0 = __ldg(rp);
                    r1 = __ldg(rp + 1);
                }
                tmem_ld_wait();
                const long long tq1 = kRoleTiming && p.debug ? clock64() : 0;
                if (kRoleTiming && p.debug) dbg_ld += tq1 - tq0;
                if (!valid) continue;
                uint32_t packed[8];
                // Four values at a time, each loop body fetching its own two table entries from shared memory, so that few
                // values are live at once (the kernel has to fit in 96 registers).
                if (folded) {
                    // Fast mode, accumulators below 2^22.  Adding an accumulator to the bits of 1.5 * 2^23 gives the float
                    // 1.5 * 2^23 + accumulator; the table holds {mult 2i, mult 2i+1, bias 2i, bias 2i+1} divided by the output scale,
                    // the bias carrying -1.5 * 2^23 * mult, so one packed FMA yields two pre-activations in code units;
                    // activation and rounding run in packed binary16.
                    // Accumulators that may reach 2^22 lose their low p.acc_shift bits first (the table carries the larger
                    // multiplier and the mean of what is dropped); the planner allows that only where it moves a
                    // pre-activation by no more than 0.02 of a code.
                    const __half2 kh = __float2half2_rn(p.sy_log2e), inv_h = __float2half2_rn(p.inv_sy);
                    const int sh = p.acc_shift;
                    if (sh == 0) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 ma = lds_f4(mtab + 32u * j), mc = lds_f4(mtab + 32u * j + 16u);
                            float t0, t1, t2, t3;
                            ffma2(t0, t1, __int_as_float(0x4B400000 + (int)acc[4 * j]), __int_as_float(0x4B400000 + (int)acc[4 * j + 1]), ma.x, ma.y, ma.z, ma.w);
                            ffma2(t2, t3, __int_as_float(0x4B400000 + (int)acc[4 * j + 2]), __int_as_float(0x4B400000 + (int)acc[4 * j + 3]), mc.x, mc.y, mc.z, mc.w);
                            packed[j] = ln_h2_pack(ln_h2_code<ACT>(t0, t1, kh, inv_h), ln_h2_code<ACT>(t2, t3, kh, inv_h));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 ma = lds_f4(mtab + 32u * j), mc = lds_f4(mtab + 32u * j + 16u);
                            float t0, t1, t2, t3;
                            ffma2(t0, t1, __int_as_float(0x4B400000 + ((int)acc[4 * j] >> sh)), __int_as_float(0x4B400000 + ((int)acc[4 * j + 1] >> sh)), ma.x, ma.y, ma.z, ma.w);
                            ffma2(t2, t3, __int_as_float(0x4B400000 + ((int)acc[4 * j + 2] >> sh)), __int_as_float(0x4B400000 + ((int)acc[4 * j + 3] >> sh)), mc.x, mc.y, mc.z, mc.w);
                            packed[j] = ln_h2_pack(ln_h2_code<ACT>(t0, t1, kh, inv_h), ln_h2_code<ACT>(t2, t3, kh, inv_h));
                        }
                    }
                } else {
                    // int32 -> f32: below 2^22 through the bits of 1.5 * 2^23 (two FMA-pipe instructions, exact); otherwise the
                    // conversion unit, or, for the transcendental epilogues that need that unit for ex2 / rcp, an exact ALU sequence
                    const bool small = p.small_acc != 0;
                    const __half2 inv_h = __float2half2_rn(p.inv_sy);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 ma = lds_f4(mtab + 32u * j), mc = lds_f4(mtab + 32u * j + 16u);
                        float x[4];
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const int a = (int)acc[4 * j + b];
                            x[b] = small ? __fadd_rn(__int_as_float(0x4B400000 + a), -12582912.0f) : (kTranscendental ? i2f_alu(a) : __int2float_rn(a));
                        }
                        const float v0 = __fmaf_rn(x[0], ma.x, ma.y), v1 = __fmaf_rn(x[1], ma.z, ma.w), v2 = __fmaf_rn(x[2], mc.x, mc.y), v3 = __fmaf_rn(x[3], mc.z, mc.w);
                        if (EXACT)
                            packed[j] = pack4_low_bytes(quant_i8_magic(ln_epilogue_act<true>(ACT, v0), p.inv_sy), quant_i8_magic(ln_epilogue_act<true>(ACT, v1), p.inv_sy),
                                                        quant_i8_magic(ln_epilogue_act<true>(ACT, v2), p.inv_sy), quant_i8_magic(ln_epilogue_act<true>(ACT, v3), p.inv_sy));
                        else
                            packed[j] = ln_h2_pack(ln_h2_act_quant<ACT>(v0, v1, inv_h), ln_h2_act_quant<ACT>(v2, v3, inv_h));
                    }
                }
                if (p.res != nullptr) {
                    // fused shortcut, the arithmetic of the stand-alone shortcut kernel applied to the codes just produced
                    const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
                    // (two values per instruction where the packed f32x2 forms exist: every product, sum and fma rounds exactly
                    // like its scalar twin, so the codes are those of the stand-alone kernel)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float c[4], r[4], v[4];
                        s8x4_to_float(packed[j], c);
                        s8x4_to_float(rw[j], r);
                        uint32_t u[4];
#pragma unroll
                        for (int b = 0; b < 4; b += 2) {
                            fmul2(v[b], v[b + 1], c[b], c[b + 1], p.s_c, p.s_c);
                            ffma2(v[b], v[b + 1], r[b], r[b + 1], p.s_res, p.s_res, v[b], v[b + 1]);
                            fmul2(v[b], v[b + 1], v[b], v[b + 1], p.inv_sy2, p.inv_sy2);
                            v[b] = fminf(fmaxf(v[b], -127.0f), 127.0f);  // NaN -> -127, as in quant_i8_magic
                            v[b + 1] = fminf(fmaxf(v[b + 1], -127.0f), 127.0f);
                            fadd2(v[b], v[b + 1], v[b], v[b + 1], 12582912.0f, 12582912.0f);
                            u[b] = __float_as_uint(v[b]);
                            u[b + 1] = __float_as_uint(v[b + 1]);
                        }
                        packed[j] = pack4_low_bytes(u[0], u[1], u[2], u[3]);
                    }
                }
                const long long tq2 = kRoleTiming && p.debug ? clock64() : 0;
                uint4* o = (uint4*)((uint8_t*)p.out + opix * p.out_pixel_stride + fo);
                o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                if (kRoleTiming && p.debug) { dbg_math += tq2 - tq1; dbg_st += clock64() - tq2; }
                continue;
            }
            if (KIND == LN_KIND_F8 && folded && p.out_kind == LN_OUT_Q) {
                // ---- FP8 fast path (the planner folds only when every chunk has its 32 filters): pre-activations in units of the
                // output scale by one packed fma on the binary32 accumulators, activation in packed binary16, two E4M3 codes
                // per conversion
                const uint32_t mtab = tab_base + 8u * (uint32_t)(f0 + c0);
                tmem_ld_wait();
                if (!valid) continue;
                const __half2 kh = __float2half2_rn(p.sy_log2e), inv_h = __float2half2_rn(p.inv_sy);
                uint32_t packed[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 ma = lds_f4(mtab + 32u * j), mc = lds_f4(mtab + 32u * j + 16u);
                    float t0, t1, t2, t3;
                    ffma2(t0, t1, __uint_as_float(acc[4 * j]), __uint_as_float(acc[4 * j + 1]), ma.x, ma.y, ma.z, ma.w);
                    ffma2(t2, t3, __uint_as_float(acc[4 * j + 2]), __uint_as_float(acc[4 * j + 3]), mc.x, mc.y, mc.z, mc.w);
                    packed[j] = ln_h2_to_e4m3x2(ln_h2_value<ACT>(t0, t1, kh, inv_h)) | (ln_h2_to_e4m3x2(ln_h2_value<ACT>(t2, t3, kh, inv_h)) << 16);
                }
                uint4* o = (uint4*)((uint8_t*)p.out + opix * p.out_pixel_stride + fo);
                o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                continue;
            }
            // ---- general path: f32 / raw-accumulator outputs (NCHW), FP8, and int8 chunks with fewer than 32 real filters.
            // The {mult, bias} pairs come two per 16-byte load (the table is padded to a multiple of 32 filters).
            const int nf = p.F - (f0 + c0);  // real filters from this chunk's first column on (32 or more: all of the chunk)
            tmem_ld_wait();
            if (!valid || nf <= 0) continue;
            if (p.out_kind == LN_OUT_ACC) {
                // NCHW, raw accumulator bits (int32 or f32): consecutive lanes are consecutive pixels of a row, one plane per filter
                const int64_t plane = (int64_t)p.OH * p.OW;
                int32_t* o = (int32_t*)p.out + ((int64_t)n * p.F + (f0 + c0)) * plane + (int64_t)oh * p.OW + ow;
#pragma unroll
                for (int j = 0; j < 32; ++j, o += plane)
                    if (j < nf) *o = (int32_t)acc[j];
                continue;
            }
            float a[32];
            const uint32_t mtab = tab_base + 8u * (uint32_t)(f0 + c0);  // (never the folded table: that one needs int8 output and full chunks)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float4 mj = lds_f4(mtab + 16u * j);
                const float x0 = KIND == LN_KIND_I8 ? __int2float_rn((int)acc[2 * j]) : __uint_as_float(acc[2 * j]);
                const float x1 = KIND == LN_KIND_I8 ? __int2float_rn((int)acc[2 * j + 1]) : __uint_as_float(acc[2 * j + 1]);
                a[2 * j] = ln_epilogue_act<EXACT>(ACT, __fmaf_rn(x0, mj.x, mj.y));
                a[2 * j + 1] = ln_epilogue_act<EXACT>(ACT, __fmaf_rn(x1, mj.z, mj.w));
            }
            if (p.out_kind == LN_OUT_F32) {
                const int64_t plane = (int64_t)p.OH * p.OW;
                float* o = (float*)p.out + ((int64_t)n * p.F + (f0 + c0)) * plane + (int64_t)oh * p.OW + ow;  // NCHW
#pragma unroll
                for (int j = 0; j < 32; ++j, o += plane)
                    if (j < nf) *o = a[j];
            } else {
                if (KIND == LN_KIND_F16) {
                    // binary16 NHWC: 32 filters = 64 bytes per pixel, rounded to nearest even, infinities kept
                    uint32_t hw[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const __half2 h = __floats2half2_rn(2 * j < nf ? a[2 * j] : 0.0f, 2 * j + 1 < nf ? a[2 * j + 1] : 0.0f);
                        hw[j] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    uint4* o = (uint4*)((uint8_t*)p.out + opix * p.out_pixel_stride + 2 * fo);
#pragma unroll
                    for (int j = 0; j < 4; ++j) o[j] = make_uint4(hw[4 * j], hw[4 * j + 1], hw[4 * j + 2], hw[4 * j + 3]);
                    continue;
                }
                uint32_t packed[8];
                if (KIND == LN_KIND_I8) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t v = 0;
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const int q = 4 * j + b < nf ? ln_quant_i8(a[4 * j + b], p.inv_sy) : 0;
                            v |= ((uint32_t)q & 0xFFu) << (8 * b);
                        }
                        packed[j] = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a[4 * j] * p.inv_sy, a[4 * j + 1] * p.inv_sy), __NV_SATFINITE, __NV_E4M3);
                        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(a[4 * j + 2] * p.inv_sy, a[4 * j + 3] * p.inv_sy), __NV_SATFINITE, __NV_E4M3);
                        uint32_t w = lo | (hi << 16);
                        const int left = nf - 4 * j;  // codes of filters that do not exist are zero
                        if (left < 4) w = left <= 0 ? 0u : (w & (0xFFFFFFFFu >> (8 * (4 - left))));
                        packed[j] = w;
                    }
                }
                uint4* o = (uint4*)((uint8_t*)p.out + opix * p.out_pixel_stride + fo);
                o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
    if (p.debug && blockIdx.x == 0 && lane == 0 && warp - 2 * PIPES < 8) {  // (the counter block has room for eight epilogue warps)
        p.debug[6 + 2 * (warp - 2 * PIPES)] = clock64() - t_start;
        p.debug[7 + 2 * (warp - 2 * PIPES)] = w_tfull;
        if (warp == 2 * PIPES) { p.debug[22] = dbg_ld; p.debug[23] = dbg_math; p.debug[24] = dbg_st; }
    }
}

// PIPES (1 or 2): the number of producer / issuer pipelines, a compile-time constant so that the single-pipeline kernel carries
// none of the other's index arithmetic in its single-thread loops.
template <int KIND, int ACT, bool EXACT, int PIPES>
__global__ void __launch_bounds__(conv_threads(PIPES), 1) conv_umma_kernel(const __grid_constant__ ln_conv_umma_params p) {
#include "ln_conv_layout.inc"
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), PIPES);  // every issuer hands the stage back
        }
        for (int b = 0; b < nbuf; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 4 * p.subs);  // the four warps of each group that drained one of the tile's column units
        }
        mbar_init(bres_bar, 1);
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(afull_bar(s), 1);
            mbar_init(aempty_bar(s), 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;


    if (warp < 2 * PIPES) {
        if (warp == 0) conv_producer_role<PIPES>(p);
        else if (warp <= PIPES) conv_mma_role<KIND, PIPES>(p);
    } else {
        conv_epilogue_role<KIND, ACT, EXACT, PIPES>(p);
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        // a wait was abandoned: give copies that may still be in flight time to land before the CTA's
        // shared memory is handed to another CTA
        for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

#undef LN_FIRST_UNIT
#undef LN_UNIT_STEP

// Tensor-pipe peak probe: one CTA per SM, one thread issuing tcgen05.mma (M = 128, N = n, 32 bytes of K per instruction)
// back to back on operand tiles that stay in shared memory, no loads, no epilogue.  What it measures is the rate the tensor
// cores sustain when nothing else limits them: the denominator of the convolution's roofline.  PAIR: clusters of two CTAs,
// the first one issuing M = 256 instructions for both (tcgen05.mma.cta_group::2).
template <int KIND, bool PAIR>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters, int n, int variant, int* status) {
    // variant bit 0: a tcgen05.commit (to a barrier nobody waits for) after every four instructions, as a pipelined main loop
    // releases its stages; bit 1: the operands rotate through four tile sets instead of staying on one
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    constexpr uint32_t kSet = (128u + 256u) * 128u;  // one A tile + one B tile
    const uint32_t sets = (variant & 2) ? 4u : 1u;
    // variant bit 2: a second warp issues the same stream into its own accumulator (its own barriers, 16 bytes further on)
    const uint32_t issuer = threadIdx.x >> 5;  // warp 0, and warp 1 when two warps issue
    const uint32_t bar = base + sets * kSet + 16u * issuer, bar2 = bar + 8u;
    uint8_t* g = smem_raw + (base - smem_u32(smem_raw));
    for (uint32_t i = threadIdx.x; i < sets * kSet / 16u; i += blockDim.x) reinterpret_cast<uint4*>(g)[i] = make_uint4(0u, 0u, 0u, 0u);
    volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(g + sets * kSet + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(g + sets * kSet + 48);
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < 4u; ++i) mbar_init(base + sets * kSet + 8u * i, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the zeroed tiles are read through the async proxy
    if (threadIdx.x < 32) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_all = *slot, tmem = tmem_all + 256u * issuer;
    if ((threadIdx.x == 0 || ((variant & 4) && threadIdx.x == 32)) && rank == 0) {
        const uint32_t idesc = (KIND == LN_KIND_I8 ? ((2u << 4) | (1u << 7) | (1u << 10)) : (1u << 4)) | (((uint32_t)n >> 3) << 17) |
                               (((PAIR ? 256u : 128u) >> 4) << 24);
        uint32_t phase = 0;
        bool ok = true;
        for (int it = 0; ok && it < iters; ++it) {
            const uint32_t set = (uint32_t)it & (sets - 1u);
            const uint64_t a_desc = make_smem_desc(base + set * kSet, 128), b_desc = make_smem_desc(base + set * kSet + 128u * 128u, 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (PAIR) tc_mma_pair<KIND>(tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (uint32_t)((it | k) != 0));
                else tc_mma<KIND>(tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (uint32_t)((it | k) != 0));
            }
            if (variant & 1) {
                if (PAIR) tc_commit_pair(bar2);
                else tc_commit(bar2);
            }
            if ((it & 63) == 63 || it + 1 == iters) {  // keep the queue bounded: wait for every 256th instruction
                if (PAIR) tc_commit_pair(bar);
                else tc_commit(bar);
                ok = mbar_wait(bar, phase, abort_flag, status, LN_STATUS_MMA_TIMEOUT);
                phase ^= 1u;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    if (threadIdx.x < 32) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_all), "r"(512u) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_all), "r"(512u) : "memory");
    }
}

constexpr int kMaxDynamicSmem = 227 * 1024;
constexpr uint32_t kMaxTableBytes = 32u * 1024u;  // {multiplier, bias} pairs of at most 4096 filters

template <int KIND, bool EXACT, int PIPES>
cudaError_t launch_act(ln_ctx* ctx, const ln_conv_umma_params& p, int grid, size_t smem, cudaStream_t stream) {
#define LN_LAUNCH_ACT(A)                                                                                             \
    case A: {                                                                                                        \
        auto k = conv_umma_kernel<KIND, A, EXACT, PIPES>;                                                              \
        if (!ctx->configured_kernels.count((const void*)k)) { /* once per kernel per context */                      \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);   \
            if (e != cudaSuccess) return e;                                                                          \
            ctx->configured_kernels.insert((const void*)k);                                                          \
        }                                                                                                            \
        k<<<grid, conv_threads(PIPES), smem, stream>>>(p);                                                                           \
        return cudaGetLastError();                                                                                   \
    }
    switch (p.act) {
        LN_LAUNCH_ACT(LN_ACT_LINEAR)
        LN_LAUNCH_ACT(LN_ACT_LOGISTIC)
        LN_LAUNCH_ACT(LN_ACT_LEAKY)
        LN_LAUNCH_ACT(LN_ACT_MISH)
        LN_LAUNCH_ACT(LN_ACT_SWISH)
        LN_LAUNCH_ACT(LN_ACT_RELU)
    }
#undef LN_LAUNCH_ACT
    return cudaErrorInvalidValue;
}

__global__ void make_mb_kernel(const float* __restrict__ wscale, const float* __restrict__ bias, float x_scale, int F, int fpad,
                               float2* __restrict__ mb) {
    int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= fpad) return;
    mb[f] = f < F ? make_float2(__fmul_rn(x_scale, wscale[f]), bias[f]) : make_float2(0.0f, 0.0f);
}

// Block-diagonal weights of a pixel-group-packed 1x1 convolution: row j * F + f holds filter f in bytes [j * cpad, (j + 1) * cpad)
// of a 128-byte row and zeros elsewhere, so that one 128-byte activation row (pack = 128 / cpad consecutive pixels)
// yields the outputs of all its pixels.  mb2[j * F + f] = mb[f].
__global__ void pack_group_weights_kernel(const uint8_t* __restrict__ w, int cpad, int F, int pack, int fpad2, uint8_t* __restrict__ w2,
                                          const float2* __restrict__ mb, float2* __restrict__ mb2) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 4 bytes of w2
    if (i >= fpad2 * 32) return;
    const int row = i >> 5, b = (i & 31) * 4;
    const int j = row / F, f = row - j * F;
    uint32_t v = 0;
    if (j < pack && b >= j * cpad && b < (j + 1) * cpad) v = *reinterpret_cast<const uint32_t*>(w + (size_t)f * cpad + (b - j * cpad));
    *reinterpret_cast<uint32_t*>(w2 + (size_t)row * 128 + b) = v;
    if ((i & 31) == 0) mb2[row] = j < pack ? mb[f] : make_float2(0.0f, 0.0f);
}

// The same for a 3x3 stride-1 pad-1 convolution: a 128-byte row is `pack` consecutive pixels of one image row, the output row the
// same `pack` pixels.  In units of pixel groups the taps are again 3x3 with pad 1; tap (r, s') of output pixel j_out reads input
// pixel j_in of group X + s' - 1, which is column offset s = pack (s' - 1) + j_in - j_out + 1 of the original 3x3 (zero weight
// when that is outside 0..2).  w is [fpad][3][3][cpad], w2 [fpad2][3][3][pack * cpad].
__global__ void pack_group_weights_k3_kernel(const uint8_t* __restrict__ w, int cpad, int F, int pack, int fpad2, uint8_t* __restrict__ w2,
                                             const float2* __restrict__ mb, float2* __restrict__ mb2) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 4 bytes of w2
    const int rw = pack * cpad / 4;                      // words of one row of `pack` pixels (32 for a 128-byte row)
    if (i >= fpad2 * 9 * rw) return;
    const int row = i / (9 * rw), rem = i - row * 9 * rw, tap = rem / rw, b = (rem - tap * rw) * 4;
    const int r = tap / 3, sp = tap - r * 3;
    const int j_out = row / F, f = row - j_out * F, j_in = b / cpad, c = b - j_in * cpad;
    const int s = pack * (sp - 1) + j_in - j_out + 1;
    uint32_t v = 0;
    if (j_out < pack && s >= 0 && s <= 2) v = *reinterpret_cast<const uint32_t*>(w + (((size_t)f * 3 + r) * 3 + s) * cpad + c);
    *reinterpret_cast<uint32_t*>(w2 + (size_t)i * 4) = v;
    if (rem == 0) mb2[row] = j_out < pack ? mb[f] : make_float2(0.0f, 0.0f);
}

// Weights of a 3x3 stride-2 pad-1 convolution over 32 channels, rearranged for its 2x2 stride-1 form over the 2x2
// space-to-depth image: w2[f][ty][tx][(qy * 2 + qx) * 32 + c] = w[f][2 ty + qy - 1][2 tx + qx - 1][c], zero where that tap does
// not exist (input row 2 (oy + ty - 1) + qy is row 2 oy + r - 1 of the original with r = 2 ty + qy - 1).
__global__ void pack_s2d_weights_kernel(const uint8_t* __restrict__ w, int fpad, uint8_t* __restrict__ w2) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 4 bytes of w2: [fpad][2][2][128]
    if (i >= fpad * 4 * 32) return;
    const int f = i / 128, rem = i - f * 128, tap = rem >> 5, b = (rem & 31) * 4;
    const int ty = tap >> 1, tx = tap & 1, q = b >> 5, c = b & 31;
    const int r = 2 * ty + (q >> 1) - 1, sx = 2 * tx + (q & 1) - 1;
    uint32_t v = 0;
    if (r >= 0 && sx >= 0) v = *reinterpret_cast<const uint32_t*>(w + (((size_t)f * 3 + r) * 3 + sx) * 32 + c);
    *reinterpret_cast<uint32_t*>(w2 + (size_t)i * 4) = v;
}

// Table of the folded fast epilogue, one float4 per pair of filters: {m0, m1, b0, b1} with m = mult / s_y and
// b = bias / s_y - 1.5 * 2^23 * m, so that fma(float with the bits 0x4B400000 + accumulator, m, b) is the pre-activation in
// units of the output scale.
__global__ void fold_mb_kernel(const float2* __restrict__ mb, int n, float inv_sy, int shift, float2* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;  // pair index
    if (2 * i >= n) return;
    // with `shift` low accumulator bits dropped (floor) the multiplier grows by 2^shift and the bias takes the mean of what was
    // dropped, (2^shift - 1) / 2 accumulator units
    // (shift < 0: binary32 accumulators, FP8 layers -- nothing dropped and no 1.5 * 2^23 to take out)
    const bool f32acc = shift < 0;
    if (f32acc) shift = 0;
    const float up = (float)(1 << shift), mean = 0.5f * (float)((1 << shift) - 1);
    const float u0 = __fmul_rn(mb[2 * i].x, inv_sy), u1 = __fmul_rn(mb[2 * i + 1].x, inv_sy);  // codes per accumulator unit
    const float m0 = __fmul_rn(u0, up), m1 = __fmul_rn(u1, up);
    const float c0 = __fmaf_rn(mean, u0, __fmul_rn(mb[2 * i].y, inv_sy)), c1 = __fmaf_rn(mean, u1, __fmul_rn(mb[2 * i + 1].y, inv_sy));
    const float b0 = f32acc ? c0 : __fmaf_rn(-12582912.0f, m0, c0), b1 = f32acc ? c1 : __fmaf_rn(-12582912.0f, m1, c1);
    out[2 * i] = make_float2(m0, m1);
    out[2 * i + 1] = make_float2(b0, b1);
}

int ilog2(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return l;
}

}  // namespace

bool ln_conv_umma_supported(int64_t channels_padded, int64_t k, int64_t stride_x, int64_t stride_y, int64_t dilation, int64_t groups,
                            int64_t in_w, int64_t in_h) {
    if (groups != 1 || dilation != 1) return false;
    if (stride_x != stride_y || (stride_x != 1 && stride_x != 2)) return false;
    if (channels_padded % 32 != 0 || k < 1 || k > 7) return false;
    (void)in_w;
    (void)in_h;
    return true;
}

// Picks the output box: TW*TH*TN = 128, all powers of two, minimising the number of tiles (ties: wider in w).
// `wide`: planar (NCHW) outputs are written one filter plane at a time, 32 lanes = 32 consecutive pixels, so the box
// must be at least 32 pixels wide for those stores to coalesce.
static void choose_box(int OW, int OH, int N, bool wide, int* TW, int* TH, int* TN) {
    int64_t best = -1;
    for (int lw = wide ? 5 : 0; lw <= 7; ++lw)
        for (int lh = 0; lw + lh <= 7; ++lh) {
            int tw = 1 << lw, th = 1 << lh, tn = 128 >> (lw + lh);
            int64_t tiles = (int64_t)((OW + tw - 1) / tw) * ((OH + th - 1) / th) * ((N + tn - 1) / tn);
            if (best < 0 || tiles < best || (tiles == best && tw > *TW)) {
                best = tiles;
                *TW = tw; *TH = th; *TN = tn;
            }
        }
}

void ln_conv_umma_plan_release(ln_ctx* ctx, ln_conv_umma_plan* plan) {
    if (plan->aux_w) ln_pool_free(ctx, plan->aux_w, plan->aux_w_bytes);
    if (plan->aux_mb) ln_pool_free(ctx, plan->aux_mb, plan->aux_mb_bytes);
    if (plan->aux_mbf) ln_pool_free(ctx, plan->aux_mbf, plan->aux_mbf_bytes);
    plan->aux_mbf = nullptr;
    plan->aux_w = nullptr;
    plan->aux_mb = nullptr;
}

int ln_conv_umma_plan_build(ln_ctx* ctx, ln_conv_umma_plan* plan, const ln_conv_geom& g_in) {
    ln_conv_umma_params& p = plan->p;
    memset(&p, 0, sizeof p);
    ln_conv_geom g = g_in;
    float2* mb = plan->mb;
    int pack = 1;
    // LN_CONV_DISABLE=pack,halo switches the two layout modes off (for A/B measurements)
    const char* disable = getenv("LN_CONV_DISABLE");
    const bool allow_pack = !(disable && strstr(disable, "pack")), allow_halo = !(disable && strstr(disable, "halo"));
    const bool allow_resident = !(disable && strstr(disable, "resident"));
    const char* rms = getenv("LN_CONV_RESIDENT_MIN_STAGES");
    const uint32_t res_min_stages = rms && atoi(rms) >= 2 ? (uint32_t)atoi(rms) : 4u;
    // Space-to-depth input (see ln_conv_geom::s2d_input): 4 taps of 128-byte rows instead of 9 taps of 32-byte rows.
    if (g.s2d_input) {
        if (!(g.k == 3 && g.stride == 2 && g.pad == 1 && g.cpad == 32 && g.H % 2 == 0 && g.W % 2 == 0 && g.x_pixel_stride == 32 && g.res == nullptr))
            return ln_fail(ctx, LN_ERR_UNSUPPORTED, "tensor-core convolution: a space-to-depth input needs 3x3 stride 2 pad 1 over 32 channels and even sizes");
        plan->aux_w_bytes = (size_t)g.fpad * 4 * 128;
        plan->aux_w = ln_pool_alloc(ctx, plan->aux_w_bytes);
        if (!plan->aux_w) return LN_ERR_CUDA;
        pack_s2d_weights_kernel<<<(g.fpad * 128 + 255) / 256, 256, 0, ctx->stream>>>((const uint8_t*)g.w, g.fpad, (uint8_t*)plan->aux_w);
        LN_LAUNCHED(ctx);
        g.w = plan->aux_w;
        g.k = 2; g.stride = 1; g.pad = 1;
        g.cpad = 128; g.C = 128; g.x_pixel_stride = 128;
        g.H /= 2; g.W /= 2;
    }
    // Pixel-group packing.  The TMA unit spends about as long on a 32- or 64-byte row as on a 128-byte one, and a 1x1
    // convolution over a dense NHWC tensor is a plain GEMM over pixels: read `pack` = 128 / C consecutive pixels as one
    // 128-byte row and multiply by block-diagonal weights (pack x F virtual filters).  The tensor core does `pack` times the
    // arithmetic, which it has to spare at these sizes; the loads are `pack` times fewer rows.
    {
        const int64_t P = (int64_t)g.N * g.H * g.W;
        const int pk = g.cpad < 128 ? 128 / g.cpad : 1;
        if (allow_pack && pk > 1 && g.k == 1 && g.stride == 1 && g.pad == 0 && g.x_pixel_stride == g.cpad && P % pk == 0 && g.out_kind == LN_OUT_Q &&
            g.res == nullptr && g.F % 32 == 0 && pk * g.F <= 256 && (((uintptr_t)g.x) & 127) == 0 && P / pk < (1ll << 30)) {
            const int F2 = pk * g.F, bn2 = ln_conv_choose_bn(F2), fpad2 = (int)ln_round_up(F2, bn2);
            plan->aux_w_bytes = (size_t)fpad2 * 128;
            plan->aux_mb_bytes = (size_t)fpad2 * sizeof(float2);
            plan->aux_w = ln_pool_alloc(ctx, plan->aux_w_bytes);
            plan->aux_mb = (float2*)ln_pool_alloc(ctx, plan->aux_mb_bytes);
            if (!plan->aux_w || !plan->aux_mb) return LN_ERR_CUDA;
            pack_group_weights_kernel<<<(fpad2 * 32 + 255) / 256, 256, 0, ctx->stream>>>((const uint8_t*)g.w, g.cpad, g.F, pk, fpad2, (uint8_t*)plan->aux_w,
                                                                                     plan->mb, plan->aux_mb);
            LN_LAUNCHED(ctx);
            pack = pk;
            g.w = plan->aux_w; g.fpad = fpad2; g.F = F2;
            g.cpad = 128; g.C = 128; g.x_pixel_stride = 128;
            g.W = (int)(P / pk); g.H = 1; g.N = 1; g.OW = g.W; g.OH = 1;
            mb = plan->aux_mb;
        }
    }
    // Pixel groups for 3x3 stride-1 layers with few channels: `pack` consecutive pixels of an image row per 128-byte row on both
    // sides, nine taps in units of groups (see pack_group_weights_k3_kernel).  The tensor core multiplies mostly zeros -- `pack`
    // times the arithmetic -- but it is idle at these sizes, and the loads become `pack` times fewer 128-byte rows.
    {
        // two pixels per row at most: with 32 channels that is a 64-byte row and 2 x zeros for the tensor core instead of a 128-byte
        // row and 4 x (3x3 C32 -> K64 at 304x304 x16: 113 -> 103 us, and the 128 virtual filters then run with two issuers)
        int pk = g.cpad < 128 ? 128 / g.cpad : 1;
        if (pk > 2) pk = 2;
        if (const char* e = getenv("LN_CONV_PACK3_MAX")) {  // (A/B measurements: 4, 2 or 1 pixels per row)
            const int v = atoi(e);
            if (v >= 1 && v * g.cpad <= 128) pk = v;
        }
        const int rb = pk * g.cpad;  // bytes of one row of pk pixels
        if (allow_pack && pack == 1 && pk > 1 && !g.s2d_input && g.k == 3 && g.stride == 1 && g.pad == 1 && g.x_pixel_stride == g.cpad && g.W % pk == 0 &&
            g.OW == g.W && g.OH == g.H && g.out_kind == LN_OUT_Q && g.F % 32 == 0 && pk * g.F <= 256 && (((uintptr_t)g.x) & 127) == 0) {
            const int F2 = pk * g.F, bn2 = ln_conv_choose_bn(F2), fpad2 = (int)ln_round_up(F2, bn2);
            plan->aux_w_bytes = (size_t)fpad2 * 9 * rb;
            plan->aux_mb_bytes = (size_t)fpad2 * sizeof(float2);
            plan->aux_w = ln_pool_alloc(ctx, plan->aux_w_bytes);
            plan->aux_mb = (float2*)ln_pool_alloc(ctx, plan->aux_mb_bytes);
            if (!plan->aux_w || !plan->aux_mb) return LN_ERR_CUDA;
            pack_group_weights_k3_kernel<<<(fpad2 * 9 * (rb / 4) + 255) / 256, 256, 0, ctx->stream>>>((const uint8_t*)g.w, g.cpad, g.F, pk, fpad2, (uint8_t*)plan->aux_w,
                                                                                           plan->mb, plan->aux_mb);
            LN_LAUNCHED(ctx);
            pack = pk;
            g.w = plan->aux_w; g.fpad = fpad2; g.F = F2;
            g.cpad = rb; g.C = rb; g.x_pixel_stride = rb;
            g.W /= pk; g.OW /= pk;
            mb = plan->aux_mb;
        }
    }
    if (!ln_conv_umma_supported(g.cpad, g.k, g.stride, g.stride, 1, 1, g.W, g.H))
        return ln_fail(ctx, LN_ERR_UNSUPPORTED, "tensor-core convolution: unsupported geometry (cpad %d k %d stride %d)", g.cpad, g.k, g.stride);
    if (((uintptr_t)g.x & 15) || (g.x_pixel_stride & 15) || ((uintptr_t)g.w & 15))
        return ln_fail(ctx, LN_ERR_ARG, "tensor-core convolution: operands must be 16-byte aligned with 16-byte pixel strides");
    if (g.out_kind == LN_OUT_Q && ((((uintptr_t)g.out) & 15) || (g.out_pixel_stride & 15)))
        return ln_fail(ctx, LN_ERR_ARG, "tensor-core convolution: 8-bit output must be 16-byte aligned");
    int bk = g.cpad % 128 == 0 ? 128 : (g.cpad % 64 == 0 ? 64 : 32);
    if (const char* e = getenv("LN_CONV_BK")) {  // (A/B measurements: a smaller channel block, 64 or 32 bytes)
        const int v = atoi(e);
        if ((v == 64 || v == 32) && v < bk) bk = v;
    }
    int bn = ln_conv_choose_bn(g.F);  // filter tile: least padding, ties to the larger tile
    if (const char* e = getenv("LN_CONV_BN")) {  // (A/B measurements: a smaller filter tile)
        const int v = atoi(e);
        if ((v == 128 || v == 64) && v < bn && g.fpad % v == 0) bn = v;
    }
    if (g.fpad % bn != 0) return ln_fail(ctx, LN_ERR_ARG, "tensor-core convolution: weights are padded to %d filters, tile needs a multiple of %d", g.fpad, bn);
    p.bk = bk; p.bn = bn;
    p.R = g.k; p.S = g.k; p.stride = g.stride; p.pad = g.pad;
    p.cblocks = g.cpad / bk; p.cpad = g.cpad;
    p.OW = g.OW; p.OH = g.OH; p.N = g.N; p.F = g.F;
    p.fpad_used = (int)ln_round_up(g.F, 32);
    p.nbuf = 512 / bn > kMaxAccBufs ? kMaxAccBufs : 512 / bn;
    p.pipes = 1;
    p.subs = p.nbuf >= kEpilogueGroups ? 1 : (kEpilogueGroups + p.nbuf - 1) / p.nbuf;  // column units per tile: keeps every epilogue group busy
    while (p.subs > 1 && (bn % (32 * p.subs)) != 0) --p.subs;
    p.small_acc = g.small_acc ? 1 : 0;
    p.pack = pack; p.f_real = g_in.F;
    choose_box(g.OW, g.OH, g.N, g.out_kind != LN_OUT_Q, &p.TW, &p.TH, &p.TN);
    // Row-shifted boxes for 3x3 stride-1 layers.  The nine taps of a tile read overlapping windows of the same input patch; one
    // box per tap re-reads that patch nine times from L2, which is what bounds these layers (the TMA unit's row rate for few
    // channels, L2 bandwidth for many).  Three boxes of TW x (TH + 2) pixels, shifted by 0 / 1 / 2 pixels in x, hold every
    // tap's operand as 128 consecutive rows starting at row r of box s -- still aligned to the 8-row swizzle pattern because TW
    // is a multiple of 8 -- so a tile and channel block costs 3 loads instead of 9.  The tile has to be TW x TH pixels of one
    // image; the mode is used when that shape wastes at most 15 % of the rows, and only for layers of at most 64 channels:
    // measured, it gains 10 % there and loses with 128 and more (the larger boxes complete later than per-tap boxes do).
    // {multiplier, bias} pairs of every filter tile, kept in shared memory behind the barrier block
    const uint32_t tab_bytes = (uint32_t)(ln_round_up(g.F, bn) * sizeof(float2));
    if (tab_bytes > kMaxTableBytes) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "tensor-core convolution: %d filters exceed the %u the epilogue table holds", g.F, kMaxTableBytes / 8u);
    p.tab_bytes = (int)tab_bytes;
    const uint32_t smem_budget = (uint32_t)kMaxDynamicSmem - 1024u - 512u - tab_bytes;
    if (allow_halo && g.k == 3 && g.stride == 1 && pack == 1 && g.out_kind != LN_OUT_F32 && g.cpad <= 64) {
        int best_tw = 0, best_th = 0;
        int64_t best_tiles = -1;
        for (int lw = 3; lw <= 7; ++lw) {
            const int tw = 1 << lw, th = 128 >> lw;
            const int64_t tiles = (int64_t)((g.OW + tw - 1) / tw) * ((g.OH + th - 1) / th);
            if (best_tiles < 0 || tiles < best_tiles) { best_tiles = tiles; best_tw = tw; best_th = th; }
        }
        const uint32_t box_bytes = (uint32_t)(best_th + 2) * best_tw * bk;
        const uint32_t b_all = (uint32_t)(9 * (g.cpad / bk)) * (uint32_t)bn * bk;
        const bool one_ftile = ln_round_up(g.F, bn) / bn == 1;
        const bool resident = one_ftile && b_all + 4u * box_bytes <= smem_budget;      // resident weights + at least four boxes
        const bool ring_fits = 4u * box_bytes + 4u * (uint32_t)bn * bk <= smem_budget;  // four boxes + four weight tiles
        if (best_tiles * 128 * 100 <= (int64_t)g.OW * g.OH * 115 && (resident || ring_fits)) {
            p.halo = 1; p.box_bytes = (int)box_bytes;
            p.TW = best_tw; p.TH = best_th; p.TN = 1;
        }
    }
    p.log_tw = ilog2(p.TW); p.log_th = ilog2(p.TH);
    p.tiles_w = (g.OW + p.TW - 1) / p.TW;
    p.tiles_h = (g.OH + p.TH - 1) / p.TH;
    p.tiles_n = (g.N + p.TN - 1) / p.TN;
    p.tiles_f = (int)(ln_round_up(g.F, bn) / bn);
    p.num_tiles = p.tiles_w * p.tiles_h * p.tiles_n * p.tiles_f;
    p.num_units = p.num_tiles;
    auto magic = [](int d) { return ((1ull << 40) + (unsigned long long)d - 1) / (unsigned long long)d; };
    p.magic_f = magic(p.tiles_f); p.magic_w = magic(p.tiles_w); p.magic_h = magic(p.tiles_h);
    if ((long long)p.num_tiles * p.num_tiles >= (1ll << 40)) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "tensor-core convolution: %d tiles", p.num_tiles);
    p.act = g.act; p.inv_sy = g.inv_sy; p.out_kind = g.out_kind;
    p.out_esize = g.kind == LN_KIND_F16 ? 2 : 1;
    p.out = g.out; p.out_pixel_stride = g.out_pixel_stride;
    p.res = g.res; p.res_pixel_stride = g.res_pixel_stride; p.s_c = g.s_c; p.s_res = g.s_res; p.inv_sy2 = g.inv_sy2;
    if (g.res && (g.out_kind != LN_OUT_Q || g.kind != LN_KIND_I8 || g.F % 32 != 0 || (((uintptr_t)g.res) & 15) || (g.res_pixel_stride & 15)))
        return ln_fail(ctx, LN_ERR_UNSUPPORTED, "tensor-core convolution: a fused shortcut needs int8 output, filters a multiple of 32 and 16-byte aligned residuals");
    p.status = ctx->d_status;
    p.debug = ctx->debug_cycles;
    p.mb = mb;
    p.mb_folded = nullptr;
    p.sy_log2e = 1.44269504f / g.inv_sy;
    // (the folded epilogue drops the lower clamp of the activations that are bounded below: needs 0.31 / s_y <= 127)
    const int acc_shift = g.small_acc ? 0 : g.acc_shift;  // (callers that do not set acc_shift leave it 0 with small_acc false: no fold)
    p.acc_shift = 0;
    // FP8 layers with 8-bit output and whole 32-filter chunks take the same packed binary16 epilogue (binary32 accumulators go
    // straight into the fma; the conversion to E4M3 saturates by itself)
    const bool fold_f8 = g.kind == LN_KIND_F8 && g.out_kind == LN_OUT_Q && g.F % 32 == 0 && !(getenv("LN_CONV_F8_FOLD") && atoi(getenv("LN_CONV_F8_FOLD")) == 0);
    if (fold_f8 || (g.kind == LN_KIND_I8 && (g.small_acc || acc_shift > 0) && g.out_kind == LN_OUT_Q && g.inv_sy <= 400.0f && g.F % 32 == 0)) {
        p.acc_shift = acc_shift;
        plan->aux_mbf_bytes = (size_t)g.fpad * sizeof(float2);
        plan->aux_mbf = (float2*)ln_pool_alloc(ctx, plan->aux_mbf_bytes);
        if (!plan->aux_mbf) return LN_ERR_CUDA;
        fold_mb_kernel<<<(g.fpad / 2 + 127) / 128, 128, 0, ctx->stream>>>(mb, g.fpad, g.inv_sy, fold_f8 ? -1 : acc_shift, plan->aux_mbf);
        LN_LAUNCHED(ctx);
        p.mb_folded = plan->aux_mbf;
    }

    const int b_rows = bn;
    const uint32_t b_total = (uint32_t)(g.k * g.k * (g.cpad / bk)) * (uint32_t)b_rows * bk;  // all weights of one filter tile (this CTA's part)
    // weights stay in shared memory when there is a single filter tile and they leave room for at least four activation stages
    if (p.halo) {
        const uint32_t box = (uint32_t)p.box_bytes, b_bytes = (uint32_t)bn * bk;
        p.b_resident = (p.tiles_f == 1 && b_total + 4u * box <= smem_budget) ? 1 : 0;
        int a_stages, stages;
        if (p.b_resident) {
            a_stages = (int)((smem_budget - b_total) / box);
            stages = 1;
        } else {
            // split what is left between boxes and weight tiles, three weight tiles per box (one box serves three taps)
            a_stages = (int)(smem_budget / (box + 3u * b_bytes));
            if (a_stages < 4) a_stages = 4;
            if (a_stages > kMaxStages) a_stages = kMaxStages;
            stages = (int)((smem_budget - (uint32_t)a_stages * box) / b_bytes);
        }
        if (a_stages > kMaxStages) a_stages = kMaxStages;
        if (stages > kMaxStages) stages = kMaxStages;
        p.a_stages = a_stages;
        p.stages = stages;
        plan->smem = (size_t)a_stages * box + (p.b_resident ? b_total : (size_t)stages * b_bytes) + 1024 /*alignment slack*/ + 512 /*barriers*/;
    } else {
    p.b_resident = (allow_resident && p.tiles_f == 1 && b_total + res_min_stages * 128u * bk <= smem_budget) ? 1 : 0;
    uint32_t ring_budget = (p.b_resident ? smem_budget : 200u * 1024u - tab_bytes) - (p.b_resident ? b_total : 0u);
    // Two pipelines (see the kernel) where one issuing thread cannot keep the tensor pipe busy and two double stages fit; the
    // tiles of a pair must share their filter tile, so the grid has to be a multiple of tiles_f.
    // LN_CONV_PIPES = 1 / 2 forces one / two wherever possible (for A/B measurements).
    const char* pipes_env = getenv("LN_CONV_PIPES");
    const int pipes_forced = pipes_env ? atoi(pipes_env) : 0;
    uint32_t stage2_bytes = 256u * bk + (p.b_resident ? 0u : (uint32_t)bn * bk);
    int grid = p.num_tiles < ctx->sm_count ? p.num_tiles : ctx->sm_count;
    // Measured (us, one -> two issuers): 3x3 C128 -> K128 at 76x76 x64 106 -> 83; 3x3 stride 2 C64 -> K128 at 304x304 x16 88 -> 65;
    // 3x3 C256 -> K512 at 38x38 x64 94 -> 92; 1x1 C512 -> K256 27 -> 35; the packed 3x3 C32 -> K64 (256 virtual filters) 111 -> 129:
    // filter tiles of 256 keep one issuer (their instructions are long enough, and three 64 KB stages are too few).
    const bool pipes_rule = bn <= 128 && g.k * g.k * (g.cpad / 32) >= 16;
    bool streamed_for_pipes = false;
    // Two issuers drain a stage twice as fast, so the ring has to be deeper: where resident weights would leave fewer than four
    // double stages and streaming them leaves four, stream them (3x3 C128 -> K128 at 76x76 x64: 77.8 -> 73.7 us).
    if (p.b_resident && pipes_forced != 1 && (pipes_rule || pipes_forced == 2) && ring_budget / stage2_bytes < 4 &&
        (200u * 1024u - tab_bytes) / (256u * bk + (uint32_t)bn * bk) >= 4) {
        streamed_for_pipes = true;
        p.b_resident = 0;
        ring_budget = 200u * 1024u - tab_bytes;
        stage2_bytes = 256u * bk + (uint32_t)bn * bk;
    }
    if (ring_budget / stage2_bytes >= 2 && p.num_tiles >= 2 * grid && pipes_forced != 1 && (pipes_rule || pipes_forced == 2)) {
        const int grid2 = grid - grid % p.tiles_f;
        if (grid2 > 0 && grid2 * 20 >= grid * 19) {  // (giving up more than 5 % of the SMs for the alignment is not worth it)
            p.pipes = 2;
            grid = grid2;
        }
    }
    if (streamed_for_pipes && p.pipes != 2) {  // one issuer after all: back to the resident weights
        p.b_resident = 1;
        ring_budget = smem_budget - b_total;
    }
    const uint32_t stage_bytes = p.pipes == 2 ? stage2_bytes : (p.b_resident ? 128u * bk : (uint32_t)(128 + b_rows) * bk);
    int stages = (int)(ring_budget / stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return ln_fail(ctx, LN_ERR_UNSUPPORTED, "tensor-core convolution: stage of %u bytes does not fit", stage_bytes);
    p.stages = stages;
    plan->grid = grid;
    plan->smem = (size_t)stages * stage_bytes + (p.b_resident ? b_total : 0u) + 1024 /*alignment slack*/ + 512 /*barriers*/;
    }
    plan->smem += tab_bytes;
    if (p.halo) plan->grid = p.num_tiles < ctx->sm_count ? p.num_tiles : ctx->sm_count;
    plan->kind = g.kind;

    const CUtensorMapSwizzle swz = bk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (bk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    const int nmaps = g.stride == 2 ? 4 : 1;
    for (int m = 0; m < nmaps; ++m) {
        const int py = m >> 1, px = m & 1;
        // sub-lattice of input pixels (y, x) with y % stride == py, x % stride == px
        int64_t Wm = (g.W - px + g.stride - 1) / g.stride, Hm = (g.H - py + g.stride - 1) / g.stride;
        if (Wm < 1) Wm = 1;
        if (Hm < 1) Hm = 1;
        cuuint64_t dims[4] = {(cuuint64_t)g.cpad, (cuuint64_t)Wm, (cuuint64_t)Hm, (cuuint64_t)g.N};
        cuuint64_t strides[3] = {(cuuint64_t)g.stride * g.x_pixel_stride, (cuuint64_t)g.stride * g.W * g.x_pixel_stride,
                                 (cuuint64_t)g.H * g.W * g.x_pixel_stride};
        cuuint32_t box[4] = {(cuuint32_t)bk, (cuuint32_t)p.TW, (cuuint32_t)(p.halo ? p.TH + 2 : p.TH), (cuuint32_t)p.TN};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        void* base = (uint8_t*)g.x + ((int64_t)py * g.W + px) * g.x_pixel_stride;
        CUresult r = ctx->encode_tiled(&p.tmA[m], CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, dims, strides, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return ln_fail(ctx, LN_ERR_CUDA, "cuTensorMapEncodeTiled(activations, map %d) failed with %d", m, (int)r);
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)g.k * g.k * g.cpad, (cuuint64_t)g.fpad};
        cuuint64_t strides[1] = {(cuuint64_t)g.k * g.k * g.cpad};
        cuuint32_t box[2] = {(cuuint32_t)bk, (cuuint32_t)b_rows};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = ctx->encode_tiled(&p.tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)g.w, dims, strides, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return ln_fail(ctx, LN_ERR_CUDA, "cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
    }
    if (getenv("LN_DEBUG_PLAN"))
        fprintf(stderr, "plan: bk %d bn %d stages %d nbuf %d subs %d b_res %d halo %d a_stages %d box %d TW %d TH %d TN %d tiles %d f %d grid %d smem %zu tab %d kind %d small %d folded %d pack %d%s\n",
                p.bk, p.bn, p.stages, p.nbuf, p.subs, p.b_resident, p.halo, p.a_stages, p.box_bytes, p.TW, p.TH, p.TN, p.num_tiles, p.tiles_f, plan->grid,
                plan->smem, p.tab_bytes, plan->kind, p.small_acc, p.mb_folded != nullptr, p.pack, (p.pipes == 2 ? " 2 pipelines" : ""));
    return LN_OK;
}

int ln_conv_umma_make_mb(ln_ctx* ctx, const float* wscale_dev, const float* bias_dev, float x_scale, int F, int fpad, float2* mb_dev) {
    make_mb_kernel<<<(fpad + 127) / 128, 128, 0, ctx->stream>>>(wscale_dev, bias_dev, x_scale, F, fpad, mb_dev);
    LN_LAUNCHED(ctx);
    return LN_OK;
}

static int32_t mma_peak_run(ln_ctx* ctx, int32_t dtype, int32_t n, int32_t pair_and_variant, int32_t iters, float* tops, const char* who) {
    const int pair = pair_and_variant & 1, variant = (pair_and_variant >> 1) & 7;
    if (!ctx || !tops || iters < 1 || iters > (1 << 20)) return ln_fail(ctx, LN_ERR_ARG, "%s: bad argument", who);
    if (dtype != LN_Q8 && dtype != LN_F8 && dtype != LN_F16) return ln_fail(ctx, LN_ERR_ARG, "%s: dtype must be LN_Q8, LN_F8 or LN_F16", who);
    if (n < 32 || n > 256 || n % 32 != 0) return ln_fail(ctx, LN_ERR_ARG, "%s: N must be a multiple of 32 up to 256", who);
    cudaSetDevice(ctx->device);
    const size_t smem = (size_t)((variant & 2) ? 4 : 1) * (128 + 256) * 128 + 1024 + 64;
    const int grid = pair ? 2 * (ctx->sm_count / 2) : ctx->sm_count;
    auto launch = [&](int it) -> cudaError_t {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = pair ? 2 : 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        ctx->launches++;
#define LN_PEAK(K)                                                                                                           \
    {                                                                                                                        \
        cudaError_t e;                                                                                                       \
        if (pair) {                                                                                                          \
            e = cudaFuncSetAttribute(mma_peak_kernel<K, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
            if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, mma_peak_kernel<K, true>, it, (int)n, variant, ctx->d_status);         \
        } else {                                                                                                             \
            e = cudaFuncSetAttribute(mma_peak_kernel<K, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
            if (e == cudaSuccess) e = cudaLaunchKernelEx(&cfg, mma_peak_kernel<K, false>, it, (int)n, variant, ctx->d_status);        \
        }                                                                                                                    \
        return e;                                                                                                            \
    }
        if (dtype == LN_Q8) LN_PEAK(LN_KIND_I8)
        if (dtype == LN_F8) LN_PEAK(LN_KIND_F8)
        LN_PEAK(LN_KIND_F16)
#undef LN_PEAK
    };
    cudaEvent_t e0, e1;
    LN_CUDA(ctx, cudaEventCreate(&e0));
    LN_CUDA(ctx, cudaEventCreate(&e1));
    cudaError_t e = launch(iters < 64 ? iters : 64);  // warm-up
    cudaEventRecord(e0, ctx->stream);
    if (e == cudaSuccess) e = launch(iters);
    cudaEventRecord(e1, ctx->stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "%s: %s", who, cudaGetErrorString(e));
    int rc = ln_check_status(ctx, who);
    if (rc) return rc;
    // one instruction is M x N x (32 bytes of K) multiply-adds: 32 per row pair for the 8-bit types, 16 for binary16
    const double k_elems = dtype == LN_F16 ? 16.0 : 32.0;
    const double issuers = (pair ? grid / 2 : grid) * ((variant & 4) ? 2.0 : 1.0), m = pair ? 256.0 : 128.0;
    *tops = (float)(2.0 * m * (double)n * k_elems * 4.0 * (double)iters * issuers / (ms * 1e-3) / 1e12);
    return LN_OK;
}

extern "C" int32_t ln_debug_mma_peak(ln_ctx* ctx, int32_t dtype, int32_t iters, float* tops) {
    return mma_peak_run(ctx, dtype, 256, 0, iters, tops, "ln_debug_mma_peak");
}

extern "C" int32_t ln_debug_mma_peak_shape(ln_ctx* ctx, int32_t dtype, int32_t n, int32_t pair, int32_t iters, float* tops) {
    return mma_peak_run(ctx, dtype, n, pair, iters, tops, "ln_debug_mma_peak_shape");
}

int ln_conv_umma_launch(ln_ctx* ctx, const ln_conv_umma_plan* plan) {
    cudaError_t e;
    const bool exact = ctx->exact_epilogue;
    const bool two = plan->p.pipes == 2;
#define LN_LAUNCH_KIND(K, X) (two ? launch_act<K, X, 2>(ctx, plan->p, plan->grid, plan->smem, ctx->stream) : launch_act<K, X, 1>(ctx, plan->p, plan->grid, plan->smem, ctx->stream))
    if (plan->kind == LN_KIND_I8) e = exact ? LN_LAUNCH_KIND(LN_KIND_I8, true) : LN_LAUNCH_KIND(LN_KIND_I8, false);
    else if (plan->kind == LN_KIND_F16) e = LN_LAUNCH_KIND(LN_KIND_F16, false);  // activations with the hardware ex2 / rcp (2 ulp of binary32, far below one binary16 rounding)
    else e = exact ? LN_LAUNCH_KIND(LN_KIND_F8, true) : LN_LAUNCH_KIND(LN_KIND_F8, false);
#undef LN_LAUNCH_KIND
    ctx->launches++;
    if (e != cudaSuccess) return ln_fail(ctx, LN_ERR_CUDA, "tensor-core convolution launch: %s", cudaGetErrorString(e));
    return LN_OK;
}
