// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (tiled loads, bulk stores), cp.async, tcgen05 (TMEM
// allocation, UMMA issue/commit, TMEM loads) and the shared-memory / instruction descriptors
// the UMMA unit consumes.  Everything here is device-only and header-only.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace smla {

// ---------------------------------------------------------------------------------------------
// Error reporting for bounded waits.  A wait that runs out publishes a code in global memory
// and raises a CTA-wide abort flag in shared memory (and in the partner CTA of a 2-CTA cluster);
// every later wait in the CTA returns at once, so the kernel drains and exits instead of
// hanging the device.
// ---------------------------------------------------------------------------------------------
struct WaitCtx {
    int* g_err;             // global error word (0 = ok; the first code recorded stays)
    volatile int* s_abort;  // CTA-local abort flag in shared memory
    long long limit;        // cycles a wait may take before it gives up
    uint32_t peer_abort;    // shared::cluster address of the partner CTA's abort flag, 0 if there is none
};

constexpr long long kWaitLimitCycles = 2000000000LL;  // default limit: ~1 s at B200 clocks

// Give up: flag this CTA and its partner, record the code (the first one wins).
__device__ __forceinline__ void wait_give_up(const WaitCtx& ctx, int code) {
    *ctx.s_abort = 1;
    if (ctx.peer_abort) asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(ctx.peer_abort), "r"(1) : "memory");
    atomicCAS(ctx.g_err, 0, code);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe: returns at once, so a spin on it reacts within tens of cycles, whereas try_wait may
// park the warp and wake it late.  Costs issue slots: only for the few latency-critical waiters.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __noinline__ bool mbar_spin_slow(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
    const long long t0 = clock64();
    int it = 0;
    while (true) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((++it & 255) == 0) {
            if (*ctx.s_abort) return false;
            if (clock64() - t0 > ctx.limit) {
                wait_give_up(ctx, code);
                return false;
            }
        }
    }
}
// Bounded low-latency wait (hot spin).
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
    if (mbar_test_wait(bar, parity)) return true;
    return mbar_spin_slow(bar, parity, ctx, code);
}
// Bounded wait.  Returns false if it gave up (error `code` recorded) or the CTA is aborting.
// `sleep_ns` > 0 makes the waiter yield its issue slots between polls: many warps spinning on barriers
// otherwise starve the single thread that issues the UMMAs of the scheduler they share.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code, unsigned sleep_ns) {
    const long long t0 = clock64();
    int it = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((++it & 31) == 0) {
            if (*ctx.s_abort) return false;
            if (clock64() - t0 > ctx.limit) {
                wait_give_up(ctx, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code,
                                          unsigned sleep_ns = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, ctx, code, sleep_ns);
}

// Wait used only while a CTA winds down after an abort: ignores the abort flag, still bounded.
__device__ __noinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity, long long limit) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(64);
        if (clock64() - t0 > limit) return;
    }
}

// ---- plain shared-memory counter as a hand-over between two threads of a CTA ------------------------------
// An mbarrier arrival takes ~180 cycles to become visible to a poller; a volatile word takes a few tens.
__device__ __forceinline__ void flag_store(uint32_t saddr, uint32_t v) {
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(saddr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t flag_load(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr) : "memory");
    return v;
}
// Bounded wait until the counter at `saddr` reaches `want` (counters only grow).
__device__ __noinline__ bool flag_wait_slow(uint32_t saddr, uint32_t want, const WaitCtx& ctx, int code) {
    const long long t0 = clock64();
    int it = 0;
    while (true) {
        if (static_cast<int32_t>(flag_load(saddr) - want) >= 0) return true;
        if ((++it & 255) == 0) {
            if (*ctx.s_abort) return false;
            if (clock64() - t0 > ctx.limit) {
                wait_give_up(ctx, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool flag_wait(uint32_t saddr, uint32_t want, const WaitCtx& ctx, int code) {
    if (static_cast<int32_t>(flag_load(saddr) - want) >= 0) return true;
    return flag_wait_slow(saddr, want, ctx, code);
}

// ---- proxies / fences -------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- L2 eviction policies ------------------------------------------------------------------------
// kv rows are re-read by every query and should stay in L2; scratch and per-query operands stream through.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// ---- TMA ---------------------------------------------------------------------------------------
// Tiled loads: box as encoded in the tensor map, coordinates {c0 = innermost element, c1 = row, ...}.
// c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const void* tmap, int c0, int c1, uint32_t bar,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_hint(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}
// Bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned) from this CTA's shared memory to global,
// tracked by the thread's bulk-group; the source may be reused after bulk_wait_read().
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t ssrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(ssrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Copies `src_bytes` (0 or 16) bytes and fills the rest of the 16 with zeros: with 0 nothing is read from global.
__device__ __forceinline__ void cp_async16_zfill_hint(uint32_t dst, const void* src, uint32_t src_bytes, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(src_bytes),
                 "l"(policy)
                 : "memory");
}
// Arrive on `bar` (one pending arrival of its expected count) once every cp.async this thread has
// issued so far has landed in shared memory.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- TMEM allocation (one CTA) ---------------------------------------------------------------
// Must be executed by one full warp; the base address is written to `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- UMMA descriptors --------------------------------------------------------------------------
enum : uint32_t { kSwizzleNone = 0, kSwizzle128 = 2, kSwizzle64 = 4, kSwizzle32 = 6 };

// Shared-memory matrix descriptor: start address, leading/stride byte offsets (all >> 4),
// descriptor version 1, swizzle mode in the top three bits.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle) {
    return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) |
           (static_cast<uint64_t>(swizzle) << 61);
}
// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
// a_mn / b_mn: 0 = operand is K-major in shared memory, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn) << 15) |
           (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
           (static_cast<uint32_t>(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, one K=16 step, issued by a single thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on `bar` once every UMMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- TMEM loads --------------------------------------------------------------------------------
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- thread-block clusters and two-CTA (cta_group::2) tcgen05 ------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs: arrive + wait on the hardware cluster barrier.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// Same without the cluster-scope release: that release costs the issuing thread about a thousand cycles per
// call, which a thread relaying one signal per pipeline step cannot afford.  Only for signals whose data is
// already in place by other means: shared memory of the signalling CTA filled by copies this thread has seen
// complete (and fenced to the async proxy), or tensor-memory reads this warp has waited for.
// The PTX memory model promises this ordering only for the release form; that the relaxed form is enough here rests
// on the two cases above and on measurement (a build with -DSMLA_RELEASE_ARRIVE gives bit-identical S, dS and dQ).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_bar) {
#ifdef SMLA_RELEASE_ARRIVE
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
#else
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
#endif
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Pair UMMA, issued by one thread of the even-ranked CTA: D[256 x N] (+)= A[256 x 16] * B[N x 16]^T where each
// CTA supplies 128 rows of A and N/2 rows of B from the same shared-memory offsets, and keeps its 128 rows of D.
__device__ __forceinline__ void umma_ss_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same, delivered to the barrier at this shared-memory offset in every CTA of `cta_mask` (bit per cluster rank).
// This is an mbarrier arrival, not a data transfer.
__device__ __forceinline__ void umma_commit_2cta_mask(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void st_global_v4_hint(void* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                                  uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(addr), "r"(a), "r"(b), "r"(c), "r"(d),
                 "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void st_global_v8(void* addr, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

// ---- small helpers -----------------------------------------------------------------------------
// Reductions over the 32 lanes of a warp in one instruction (every lane receives the result).
__device__ __forceinline__ float redux_max_f32(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ unsigned redux_add_u32(unsigned v) {
    unsigned r;
    asm volatile("redux.sync.add.u32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two fp32 -> packed bf16x2 (round to nearest even); `lo` goes to the low half
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// The same under a predicate inside one asm block (`row` >= 0), so that a run of them compiles to predicated
// instructions and not to a chain of branches around each one.
__device__ __forceinline__ void red_add_f32_if_row(float* addr, float v, int row) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ge.s32 p, %2, 0;\n\t"
        "@p red.global.add.f32 [%0], %1;\n\t}"
        ::"l"(addr), "f"(v), "r"(row)
        : "memory");
}

// A plain store under the same predicate (the staged, reproducible form of the dKV scatter).
__device__ __forceinline__ void st_global_f32_if_row(float* addr, float v, int row) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ge.s32 p, %2, 0;\n\t"
        "@p st.global.f32 [%0], %1;\n\t}"
        ::"l"(addr), "f"(v), "r"(row)
        : "memory");
}
// The same with an L2 eviction policy: the accumulator rows are touched again by later queries and should
// outlive the operands that only stream through.
__device__ __forceinline__ void red_add_f32_if_row_hint(float* addr, float v, int row, uint64_t policy) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ge.s32 p, %2, 0;\n\t"
        "@p red.global.add.L2::cache_hint.f32 [%0], %1, %3;\n\t}"
        ::"l"(addr), "f"(v), "r"(row), "l"(policy)
        : "memory");
}

}  // namespace smla
