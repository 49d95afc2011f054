// Device kernels of the sparse MLA backward for sm_100a.
//
// The backward of one query token is a chain of five contractions around a softmax-gradient
// step.  It is split into four kernels that hand bf16 S / dS through a scratch buffer:
//
//   delta      Delta[q,h] = sum_j O[q,h,j] * dO[q,h,j]                         (HBM-bound)
//   recompute  P^T = K_g Q^T, dP^T = V_g dO^T  (tcgen05, keys on the M axis),
//              S = exp2(P*scale*log2e - lse), dS = S*(dP - Delta)*scale -> bf16 scratch
//   dkv        dKV^T[d, key] = dO^T S + Q^T dS (tcgen05, d on the M axis), then one coalesced
//              fp32 reduction per (key, 32 consecutive d) straight from TMEM registers
//   dq         dQ[head, d] = dS^T K_g (tcgen05, heads on the M axis, d on N) accumulated over all keys
//
// The forward (o, lse for the same indices) has a logits kernel of its own (2-CTA pairs with Q resident and two tiles
// in flight), run once to find every row's maximum logit and once to write E = exp2(logit - max) and the row sums, and
// reuses the dq kernel on the V columns, dividing by the sums on the way out.
//
// Heads are padded to HP = 64 or 128, so h_q = 16 / 64 / 128 use the same code.  Gathered kv rows and
// Q / dO are held as 128-byte-swizzled [rows x 64 bf16] chunks (kv rows by 16-byte cp.async, Q / dO by
// TMA); S / dS tiles arrive by TMA in the no-swizzle core-matrix order.  A chunk is read K-major or
// MN-major by choosing the descriptor, never by moving data.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>

#include "sm100_ptx.cuh"

namespace smla {

constexpr unsigned kPollSleepNs = 32;   // back-off of producer / consumer warps waiting on mbarriers
constexpr int kDQK = 576;
constexpr int kDV = 512;
constexpr int kQChunks = kDQK / 64;   // 9 column chunks of 64
constexpr int kVChunks = kDV / 64;    // 8
constexpr int kDqChunks = 3;          // dq: three d-parts of three column chunks (192 columns) each

struct KParams {
    const __nv_bfloat16* kv;  // [s_kv, 576]
    const int32_t* indices;   // [s_q, topk]
    const float* lse;         // [s_q, h_q]
    const float* delta;       // [s_q, h_q]
    __nv_bfloat16* s_scr;     // [q_chunk][HP/8 head blocks][topk_pad keys][8 heads], see scratch_offset
    __nv_bfloat16* ds_scr;    // likewise
    float* dKV;               // [s_kv, 576]
    float* staging;           // reproducible mode: [q_chunk][topk_pad slots][576] fp32, one row per slot
    __nv_bfloat16* dQ;        // [s_q, h_q, 576]
    // forward only
    int* m_ord;               // [s_q, h_q] row maximum of the raw logits Q.K, as order-preserving integers
    unsigned long long* l_fix;// [s_q, h_q] row sum of exp2(logit - max) in 2^-22 fixed point
    float* lse_out;           // [s_q, h_q]
    float lse_out_mult;       // 1 (base 2) or ln 2 (natural log)
    // dq-style kernel: where the result goes (dQ with pitch 576, or o with pitch 512)
    __nv_bfloat16* gout;      // [s_q, h_q, 576] (dQ) or [s_q, h_q, 512] (o)
    int* g_err;
    int q0;                   // first query (global row) of this launch
    int nq;                   // queries in this launch
    int scr0;                 // scratch row of query q0 (a launch may cover a part of the queries a scratch holds)
    int s_q, s_kv, h_q, topk, topk_pad;
    float sm_scale, scale_log2e, lse_mult;
    int q_start, causal;
    const int4* qmeta;        // optional per query {first kv row of its sequence, kv rows of its sequence,
                              // position for the causal rule, top-k slots in use}; null: one sequence
    long long wait_limit;     // cycles a bounded wait may take
};

// What a query may attend to: rows [kv_base, kv_base + kv_len) of kv, index values relative to kv_base.
struct QMeta {
    int kv_base, kv_len, q_pos, topk_len;
};
__device__ __forceinline__ QMeta load_qmeta(const KParams& p, int q_global) {
    if (p.qmeta) {
        const int4 m = __ldg(p.qmeta + q_global);
        return QMeta{m.x, m.y, m.z, m.w};
    }
    return QMeta{0, p.s_kv, p.q_start + q_global, p.topk};
}
// kv row a slot gathers from, -1 when the index is outside the query's sequence (nothing is read then)
__device__ __forceinline__ int gather_row(int idx, const QMeta& m, const KParams& p) {
    const int row = m.kv_base + idx;
    return (idx >= 0 && idx < m.kv_len && row < p.s_kv) ? row : -1;
}
// After a bounded wait has given up: let this thread's own cp.async land and leave in-flight TMA loads (they
// depend on nothing and complete within microseconds) the time to land before the CTA gives up its shared memory.
__device__ __forceinline__ void abort_wind_down(volatile int* s_abort) {
    if (*s_abort) {
        cp_async_wait_all();
        for (int i = 0; i < 32; ++i) __nanosleep(1000);
    }
}

// S / dS scratch of one query: [HP/8 head blocks][topk_pad keys][8 heads] bf16, i.e. the UMMA core matrices
// (8 keys x 16 bytes) of the no-swizzle layouts stored one after another.  A warp of the recompute kernel holds 32
// consecutive keys, so each of its stores writes 512 consecutive bytes (four full cache lines) instead of 32
// scattered sectors; the consumers fetch [head block][keys of a tile][8 heads] with one TMA box of 512-byte rows.
__device__ __forceinline__ size_t scratch_offset(int key, int head, int topk_pad) {
    return (static_cast<size_t>(head >> 3) * topk_pad + key) * 8 + (head & 7);
}


// error codes recorded by bounded waits: 100*kernel + site
enum { kErrRecompute = 100, kErrDkv = 200, kErrDq = 300, kErrFwd = 400 };

__device__ __forceinline__ bool slot_valid(int idx, int key, const QMeta& m, const KParams& p) {
    return key < m.topk_len && idx >= 0 && idx < m.kv_len && m.kv_base + idx < p.s_kv && (!p.causal || idx <= m.q_pos);
}

// fp32 <-> integers that compare like the floats they came from (so that integer max instructions and atomics work
// on them); -inf maps to the smallest value used
__device__ __forceinline__ int float_to_ordered(float x) {
    const int i = __float_as_int(x);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float ordered_to_float(int o) {
    return __int_as_float(o ^ ((o >> 31) & 0x7fffffff));
}
constexpr int kOrderedNegInf = static_cast<int>(0xff800000u ^ 0x7fffffffu);   // float_to_ordered(-inf)
constexpr float kFixScale = 4194304.f;                                           // 2^22

// =============================================================================================
// Delta = rowsum(O * dO).  One warp per (query, head) row of 512 bf16; each lane reads 2 x 16 B
// of each tensor, so a warp reads 2 x 1 KB fully coalesced.
// =============================================================================================
__global__ void __launch_bounds__(256) smla_delta_kernel(const uint4* __restrict__ O, const uint4* __restrict__ dO,
                                                         float* __restrict__ delta, int n_rows) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const uint4* o = O + static_cast<size_t>(row) * (kDV / 8);
    const uint4* g = dO + static_cast<size_t>(row) * (kDV / 8);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 a = __ldg(o + lane + 32 * i);
        uint4 b = __ldg(g + lane + 32 * i);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 x = __bfloat1622float2(pa[k]);
            float2 y = __bfloat1622float2(pb[k]);
            acc = fmaf(x.x, y.x, acc);
            acc = fmaf(x.y, y.y, acc);
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) delta[row] = acc;
}

// =============================================================================================
// recompute: persistent 2-CTA clusters, 19 warps per CTA; cluster c works on queries c, c + #clusters, ...
// The pair works on 256-key tiles with cta_group::2 UMMAs of shape M = 256 keys x N = 2*HP:
//   A  each CTA gathers ITS 128 keys of the tile (every kv row is fetched once per query, not once
//      per head group), chunk by chunk through a 5-slot ring of [128 keys x 64 col] chunks;
//   B  each CTA holds the Q and dO rows of ITS half of the heads, stored per column chunk as
//      [Q_j | dO_j] so that one UMMA of N = 2*HP yields P^T and dP^T side by side
//      (chunk 8 has no V columns: its dO half is a block of zeros);
//   D  each CTA ends up with [its 128 keys] x [P^T | dP^T of all heads] in its own TMEM, columns
//      ordered (head half 0: P, dP), (head half 1: P, dP); two buffers.
//   warps 0-7   softmax-gradient on the CTA's own keys: warp w -> TMEM lane quarter w % 4, head half w / 4
//   warps 8-15  gather producers (cp.async 16 B, swizzled); completion arrives on the slot's mbarrier
//   warps 16,17 even CTA: the two UMMA issuers for the pair, taking alternate chunks.  A thread that issues a
//               tcgen05.mma is held until the tensor pipe takes it, and whatever else it executes (barrier
//               polls, commits) is time the pipe idles; with two threads handing over through a counter, one
//               waits for its next chunk and commits while the other's UMMAs run.
//               odd CTA: warp 16 forwards "my slot is full" to the even CTA (cp.async cannot signal remotely)
//   warp 18     TMA of the CTA's Q / dO chunks, one barrier per column chunk
// Slot-free, chunk-free and accumulator-ready signals are tcgen05.commit arrivals delivered to both CTAs.
// Nothing is drained between queries: the ring, the two accumulator buffers and the counters behind their
// barrier phases run on, the Q / dO chunk j of the next query is fetched as soon as the last tile's UMMAs
// on chunk j have finished, and the softmax of a query's last tile overlaps the next query's first UMMAs.
// =============================================================================================
namespace rp {
constexpr int kThreads = 608;
constexpr int kProducerThreads = 256;
constexpr int kTileKeys = 256;             // per pair; 128 per CTA
constexpr int kChunkA = 128 * 128;         // 16 KB gathered chunk
template <int HP> struct Cfg {
    static constexpr int NH = HP / 2;                  // heads whose Q / dO rows this CTA holds
    static constexpr int kStages = HP == 128 ? 5 : 9;  // what the stacked Q / dO leaves of the shared memory
    static constexpr int kBHalf = NH * 128;            // one [NH heads x 64 col] chunk
    static constexpr int kBChunk = 2 * kBHalf;         // stacked [Q_j | dO_j]
    static constexpr int kOffB = 0;
    static constexpr int kOffRing = kQChunks * kBChunk;
    static constexpr int kOffMisc = kOffRing + kStages * kChunkA;
    static constexpr int kSmemBytes = kOffMisc + 1024 + 512 + 1024;   // lse/delta + barriers + alignment slack
    static constexpr int kAccCols = 2 * HP;                        // one accumulator buffer: [S | dP]
    static constexpr int kTmemCols = 2 * kAccCols;                 // two buffers
};
}  // namespace rp

template <int HP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(rp::kThreads, 1)
smla_recompute_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                           const KParams p) {
    using namespace rp;
    using C = Cfg<HP>;
    constexpr int NH = C::NH;
    constexpr int kStages = C::kStages;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    uint8_t* misc = smem + C::kOffMisc;
    float* lse_s = reinterpret_cast<float*>(misc);          // [HP] base-2 lse, +inf for padded heads
    float* delta_s = lse_s + HP;                            // [HP] Delta * sm_scale
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc + 1024);
    const uint32_t bar_full = smem_u32(bars);               // [kStages] gathered chunk landed (even CTA: in both CTAs)
    const uint32_t bar_empty = bar_full + 8 * kStages;      // [kStages] pair UMMAs reading the slot finished
    const uint32_t bar_bfull = bar_empty + 8 * kStages;     // [9] Q / dO column chunk of the current query landed
    const uint32_t bar_bfree = bar_bfull + 8 * kQChunks;    // [9] the query's last UMMAs on the chunk finished
    const uint32_t bar_tfull = bar_bfree + 8 * kQChunks;    // [2] accumulator buffer complete
    const uint32_t bar_tempty = bar_tfull + 16;             // [2] (even CTA) both CTAs have read the buffer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 1024 + 8 * (2 * kStages + 2 * kQChunks + 4));
    volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t tok = smem_u32(tmem_slot + 2);           // (even CTA) chunks issued so far, the issuers' hand-over
    const uint32_t bar_drain = smem_u32(tmem_slot + 4);     // [2] one per issuer, used only while winding down after an abort
    static_assert(8 * (2 * kStages + 2 * kQChunks + 4) + 16 + 16 <= 512, "barrier area");
    const WaitCtx wc{p.g_err, s_abort, p.wait_limit, map_to_cta(smem_u32(tmem_slot + 1), rank ^ 1)};

    if (threadIdx.x == 0) {
        *s_abort = 0;
        tmem_slot[2] = 0;
        for (int i = 0; i < kStages; ++i) {
            // the even CTA's "full" also counts one arrival forwarded from the odd CTA
            mbar_init(bar_full + 8 * i, kProducerThreads + (rank == 0 ? 1 : 0));
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < kQChunks; ++i) {
            mbar_init(bar_bfull + 8 * i, 1);
            mbar_init(bar_bfree + 8 * i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 16);   // 8 softmax warps in each CTA
            mbar_init(bar_drain + 8 * i, 1);
        }
        fence_mbar_init();
    }
    {   // zero block standing in for the dO half of column chunk 8 (never overwritten)
        uint4* z = reinterpret_cast<uint4*>(smem + C::kOffB + 8 * C::kBChunk + C::kBHalf);
        for (int i = threadIdx.x; i < C::kBHalf / 16; i += kThreads) z[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async_smem();
    }
    if (warp == 16) {
        tmem_alloc_2cta(smem_u32(tmem_slot), C::kTmemCols);
        tmem_relinquish_2cta();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // barriers of both CTAs are initialised before anyone signals across
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int n_tiles = p.topk_pad / kTileKeys;
    const int nq = p.nq;

    if (warp >= 8 && warp < 16) {
        // ------------------------------------------------------------------ gather producers
        const int pt = threadIdx.x - 256;   // 0..255
        const int u = pt & 7;               // 16-byte unit inside a 128-byte chunk row
        const int r0 = pt >> 3;             // rows r0, r0+32, r0+64, r0+96 of this CTA's 128 keys
        const uint32_t dst0 = s_base + C::kOffRing + r0 * 128 + ((u ^ (r0 & 7)) << 4);
        const char* kvb = reinterpret_cast<const char*>(p.kv) + u * 16;
        const uint64_t pol_keep = l2_policy_evict_last();
        // index of slot (tile, row i) of query ql, -1 past the top-k; the loads for the next tile are issued
        // before the current tile's copies so that their latency never stalls the ring
        // (raw values: nothing may depend on a load here, or the wait for it would sit in front of the copies; they are
        // turned into kv rows one tile later, when they are used)
        QMeta qm_next = load_qmeta(p, p.q0 + (pair < nq ? pair : 0));
        auto load_idx = [&](int ql, int tile, int (&idx)[4]) {
            if (ql >= nq) {
                idx[0] = idx[1] = idx[2] = idx[3] = -1;
                return;
            }
            if (tile == 0) qm_next = load_qmeta(p, p.q0 + ql);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = tile * kTileKeys + rank * 128 + r0 + 32 * i;
                idx[i] = key < p.topk ? __ldg(p.indices + static_cast<size_t>(p.q0 + ql) * p.topk + key) : -1;
            }
        };
        int idx_next[4];
        load_idx(pair, 0, idx_next);
        int s = 0;
        uint32_t ph = 1;                    // parity that means "slot free" for the current pass over the ring
        for (int ql = pair; ql < nq; ql += n_pairs) {
            for (int tile = 0; tile < n_tiles; ++tile) {
                // A slot whose index is out of range reads nothing and lands as zeros (its S, dS are forced to 0
                // anyway).  Sending all of them to one stand-in row instead would make that row's cache lines a
                // hot spot that every SM queues on.
                const char* src[4];
                uint32_t nb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = gather_row(idx_next[i], qm_next, p);
                    nb[i] = row >= 0 ? 16u : 0u;
                    src[i] = kvb + static_cast<size_t>(row >= 0 ? row : 0) * (kDQK * 2);
                }
                if (tile + 1 < n_tiles) load_idx(ql, tile + 1, idx_next);
                else load_idx(ql + n_pairs, 0, idx_next);
                for (int j = 0; j < kQChunks; ++j) {
                    mbar_wait(bar_empty + 8 * s, ph, wc, kErrRecompute + 11, kPollSleepNs);
                    const uint32_t d = dst0 + s * kChunkA;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        cp_async16_zfill_hint(d + i * 32 * 128, src[i] + j * 128, nb[i], pol_keep);
                    cp_async_mbar_arrive_noinc(bar_full + 8 * s);
                    if (++s == kStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 18) {
        // ------------------------------------------------------------------ Q / dO chunks of this CTA's heads
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_do);
            const uint64_t pol_stream = l2_policy_evict_first();
            uint32_t qpar = 1;              // parity of "chunk free" left by the previous query
            for (int ql = pair; ql < nq; ql += n_pairs, qpar ^= 1) {
                const int row0 = (p.q0 + ql) * p.h_q + NH * rank;
                for (int j = 0; j < kQChunks; ++j) {
                    if (ql != pair) mbar_wait(bar_bfree + 8 * j, qpar, wc, kErrRecompute + 16, kPollSleepNs);
                    const bool with_do = j < kVChunks;
                    mbar_arrive_expect_tx(bar_bfull + 8 * j, (with_do ? 2 : 1) * C::kBHalf);
                    tma_load_2d_hint(s_base + C::kOffB + j * C::kBChunk, &tm_q, 64 * j, row0, bar_bfull + 8 * j, pol_stream);
                    if (with_do)
                        tma_load_2d_hint(s_base + C::kOffB + j * C::kBChunk + C::kBHalf, &tm_do, 64 * j, row0,
                                         bar_bfull + 8 * j, pol_stream);
                }
            }
        }
    } else if (warp == 16 || warp == 17) {
        if (lane == 0) {
            if (rank == 1) {
                if (warp == 16) {
                // -------------------------------------------------------------- forward slot-full to the even CTA
                int s = 0;
                uint32_t ph = 0, qpar = 0;
                for (int ql = pair; ql < nq; ql += n_pairs, qpar ^= 1) {
                    for (int tile = 0; tile < n_tiles; ++tile) {
                        for (int j = 0; j < kQChunks; ++j) {
                            // this CTA's half of Q / dO is part of what "full" promises
                            if (tile == 0) mbar_wait(bar_bfull + 8 * j, qpar, wc, kErrRecompute + 15);
                            mbar_spin(bar_full + 8 * s, ph, wc, kErrRecompute + 17);
                            // The copies have landed in this CTA's shared memory (the wait above saw them complete);
                            // make them visible to the tensor core's proxy here, then signal without a cluster-scope
                            // release, which would cost this thread about a thousand cycles per chunk.
                            fence_proxy_async_smem();
                            mbar_arrive_cluster_relaxed(map_to_cta(bar_full + 8 * s, 0));
                            if (++s == kStages) {
                                s = 0;
                                ph ^= 1;
                            }
                        }
                    }
                }
                }
            } else {
                // -------------------------------------------------------------- UMMA issuers for the pair
                // Issuer x takes the chunks whose running number is x mod 2.  For a chunk it waits until the data is
                // there, then until the other issuer has issued the chunk before (a counter in shared memory: the
                // UMMAs enter the pipe in chunk order, so every accumulator is summed in one fixed order and the
                // results are reproducible bit for bit), issues 4 UMMAs (512 cycles of math on both SMs), bumps the
                // counter and commits.  The UMMAs of one accumulator form a dependency chain, so the commit behind a
                // tile's last chunk covers the whole tile.
                const int x = warp - 16;
                constexpr uint32_t idesc = make_idesc_bf16(256, C::kAccCols, 0, 0);
                const uint64_t desc_hi = make_smem_desc(0, 16, 1024, kSwizzle128) & 0xFFFFFFFF00000000ull;
                const uint32_t desc_lo = static_cast<uint32_t>(make_smem_desc(0, 16, 1024, kSwizzle128));
                const uint32_t a_lo0 = desc_lo + ((s_base + C::kOffRing) >> 4);
                const uint32_t b_lo0 = desc_lo + ((s_base + C::kOffB) >> 4);
                const int n_queries = (nq - pair + n_pairs - 1) / n_pairs;
                const int total = n_queries * n_tiles * kQChunks;
                int j = x, tile = 0, gt = 0;    // running chunk `it` = column chunk j of tile `tile` of a query; gt counts tiles
                uint32_t qpar = 0;
                int s = x % kStages;
                uint32_t ph = 0;
                for (int it = x; it < total; it += 2) {
                    const int b = gt & 1;
                    if (j == 0) mbar_spin(bar_tempty + 8 * b, ((gt >> 1) & 1) ^ 1, wc, kErrRecompute + 13);
                    if (tile == 0) mbar_wait(bar_bfull + 8 * j, qpar, wc, kErrRecompute + 12);
                    mbar_spin(bar_full + 8 * s, ph, wc, kErrRecompute + 14);
                    flag_wait(tok, static_cast<uint32_t>(it), wc, kErrRecompute + 19);
                    tc_fence_after_sync();
                    const uint32_t d = tmem + b * C::kAccCols;
                    const uint32_t a_lo = a_lo0 + s * (kChunkA >> 4);
                    const uint32_t b_lo = b_lo0 + j * (C::kBChunk >> 4);
                    umma_ss_2cta(d, desc_hi | a_lo, desc_hi | b_lo, idesc, j != 0);
#pragma unroll
                    for (int kk = 1; kk < 4; ++kk)   // 32 bytes further along K = +2 in the address field
                        umma_ss_2cta(d, desc_hi | (a_lo + 2 * kk), desc_hi | (b_lo + 2 * kk), idesc, 1);
                    tc_fence_before_sync();
                    flag_store(tok, static_cast<uint32_t>(it + 1));
                    umma_commit_2cta_mask(bar_empty + 8 * s, 3);
                    if (tile == n_tiles - 1) umma_commit_2cta_mask(bar_bfree + 8 * j, 3);   // the next query's chunk may come in
                    if (j == kQChunks - 1) umma_commit_2cta_mask(bar_tfull + 8 * b, 3);
                    j += 2;
                    if (j >= kQChunks) {
                        j -= kQChunks;
                        ++gt;
                        if (++tile == n_tiles) {
                            tile = 0;
                            qpar ^= 1;
                        }
                    }
                    s += 2;
                    if (s >= kStages) {
                        s -= kStages;
                        ph ^= 1;
                    }
                }
                if (*s_abort) {   // winding down: nothing of this thread's may still be in the tensor pipe at dealloc
                    umma_commit_2cta_mask(bar_drain + 8 * x, 1);
                    mbar_wait_drain(bar_drain + 8 * x, 0, p.wait_limit);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax gradient (own 128 keys)
        const int quarter = warp & 3;
        const int g = warp >> 2;            // head half
        const int row = quarter * 32 + lane;
        const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
        const uint64_t pol_stream = l2_policy_evict_first();
        // lse (threads 0..HP-1) and Delta (threads HP..2HP-1) of a query go through shared memory; the value for
        // the next query is fetched one query ahead
        const int t = threadIdx.x;
        auto load_stat = [&](int ql) -> float {
            if (ql >= nq) return 0.f;
            const int h = t < HP ? t : t - HP;
            if (t >= 2 * HP) return 0.f;
            if (h >= p.h_q) return t < HP ? __int_as_float(0x7f800000) : 0.f;
            const size_t o = static_cast<size_t>(p.q0 + ql) * p.h_q + h;
            return t < HP ? p.lse[o] * p.lse_mult : p.delta[o] * p.sm_scale;
        };
        float stat_next = load_stat(pair);
        int gt = 0;
        for (int ql = pair; ql < nq; ql += n_pairs) {
            const int qg = p.q0 + ql;
            const QMeta qm = load_qmeta(p, qg);
            asm volatile("bar.sync 1, 256;" ::: "memory");      // every softmax warp is done with the previous query
            if (t < 2 * HP) lse_s[t] = stat_next;              // delta_s follows lse_s
            asm volatile("bar.sync 1, 256;" ::: "memory");
            stat_next = load_stat(ql + n_pairs);
            for (int tile = 0; tile < n_tiles; ++tile, ++gt) {
                const int key = tile * kTileKeys + rank * 128 + row;
                const int idx = key < p.topk ? __ldg(p.indices + static_cast<size_t>(qg) * p.topk + key) : -1;
                const bool valid = slot_valid(idx, key, qm, p);
                const int b = gt & 1;
                mbar_wait(bar_tfull + 8 * b, (gt >> 1) & 1, wc, kErrRecompute + 18, kPollSleepNs);
                tc_fence_after_sync();
                {
                    const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + b * C::kAccCols + g * 2 * NH;
                    // the 32 lanes hold consecutive keys: 32 x 16 bytes of consecutive addresses per store
                    const size_t off = static_cast<size_t>(p.scr0 + ql) * p.topk_pad * HP + scratch_offset(key, g * NH, p.topk_pad);
                    __nv_bfloat16* s_out = p.s_scr + off;
                    __nv_bfloat16* ds_out = p.ds_scr + off;
                    const uint32_t vmask = valid ? 0xFFFFFFFFu : 0u;
                    // 16 heads at a time (loading the next 16 columns under the work on these was measured: no change)
                    auto work = [&](int c0, const uint32_t (&pv)[16], const uint32_t (&dpv)[16]) {
                        uint32_t so[8], dso[8];
                        const float4* l4 = reinterpret_cast<const float4*>(lse_s + g * NH + c0);     // 16 heads: 4 + 4 vector loads
                        const float4* d4 = reinterpret_cast<const float4*>(delta_s + g * NH + c0);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const float4 l = l4[v], dl = d4[v];
                            const float lv[4] = {l.x, l.y, l.z, l.w}, dv[4] = {dl.x, dl.y, dl.z, dl.w};
                            float sv[4], dsv[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int c = 4 * v + e;
                                // dv holds Delta * sm_scale: dS = S * (dP - Delta) * sm_scale in two instructions
                                const float sx = ex2_approx(fmaf(__uint_as_float(pv[c]), p.scale_log2e, -lv[e]));
                                sv[e] = sx;
                                dsv[e] = sx * fmaf(__uint_as_float(dpv[c]), p.sm_scale, -dv[e]);
                            }
                            // an unused slot is masked after packing (one AND per two values; also wipes the
                            // NaN / inf its never-gathered operand row may have produced)
                            so[2 * v] = pack_bf16x2(sv[0], sv[1]) & vmask;
                            so[2 * v + 1] = pack_bf16x2(sv[2], sv[3]) & vmask;
                            dso[2 * v] = pack_bf16x2(dsv[0], dsv[1]) & vmask;
                            dso[2 * v + 1] = pack_bf16x2(dsv[2], dsv[3]) & vmask;
                        }
                        // 16 heads = two blocks of 8; a block is topk_pad * 8 elements further
                        __nv_bfloat16* s0 = s_out + static_cast<size_t>(c0) * p.topk_pad;
                        __nv_bfloat16* d0 = ds_out + static_cast<size_t>(c0) * p.topk_pad;
                        const size_t blk = static_cast<size_t>(p.topk_pad) * 8;
                        st_global_v4_hint(s0, so[0], so[1], so[2], so[3], pol_stream);
                        st_global_v4_hint(s0 + blk, so[4], so[5], so[6], so[7], pol_stream);
                        st_global_v4_hint(d0, dso[0], dso[1], dso[2], dso[3], pol_stream);
                        st_global_v4_hint(d0 + blk, dso[4], dso[5], dso[6], dso[7], pol_stream);
                    };
#pragma unroll 1
                    for (int c0 = 0; c0 < NH; c0 += 16) {
                        uint32_t pv[16], dpv[16];
                        tmem_ld_32x16(taddr + c0, pv);
                        tmem_ld_32x16(taddr + NH + c0, dpv);
                        tmem_ld_wait();
                        work(c0, pv, dpv);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                // The accumulator reads have completed (tcgen05.wait::ld above), which is all the issuer needs to know;
                // the stores to the scratch are ordered by the kernel boundary.  A cluster-scope release here would hold
                // the warp for about a thousand cycles per tile.
                if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * b);
            }
        }
    }
    abort_wind_down(s_abort);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves while the other may still signal it or read its operands
    if (warp == 16) tmem_dealloc_2cta(tmem, C::kTmemCols);
}

// =============================================================================================
// forward logits as persistent 2-CTA clusters: one pair per query (queries round-robin).
//
// With B = Q only there is no dO to share the shared memory with: a CTA holds Q of HALF the heads (9 chunks of
// [HP/2 heads x 64 col], 72 KB at 128 heads), which leaves nine ring slots for the gathered keys.
//   cta_group::2 UMMAs of M = 256 keys (128 gathered by each CTA) x N = HP heads (HP/2 supplied by each CTA) x K = 16;
//   D  this CTA's [128 keys] x [HP heads] in TMEM, four buffers of HP columns
//   warps 0-7   row statistics / exponentials on the CTA's own keys: warp w -> TMEM lane quarter w % 4, head half w / 4
//   warps 8-15  gather producers (cp.async 16 B, swizzled), one group of four warps per tile stream
//   warps 16-19 even CTA: the four UMMA issuers for the pair; odd CTA: warp 16 forwards "my slot is full"
//   warp 20     TMA of the CTA's Q chunks
// Two 256-key tiles are in flight at a time, as two independent streams (the even tiles and the odd tiles): each stream
// has its own producer group, its own ring slots (five and four), its own pair of accumulator buffers (one is read by
// the statistics warps while the other fills) and two issuers; the streams share only the tensor pipe.  Ring slots of
// its own matter: a producer group that fills a slot has then itself seen the slot's previous use, so its wait on the
// phase parity of "slot free" cannot be satisfied by the phase before last (with one ring shared by the two groups a
// group that ran ahead of the other overwrote a slot in use and arrived twice on one barrier phase).
// A thread that issues UMMAs executes everything slowly (cycle counters: ~450 cycles for the four UMMAs of a chunk,
// ~270 for its commits, ~230 for advancing a handful of counters, against 256 cycles of tensor-pipe time), so a stream
// is shared by two issuers that take alternate chunks and hand over through a counter in shared memory: the UMMAs of an
// accumulator enter the pipe in chunk order and the result is reproducible bit for bit.
// Slot-free, chunk-free and accumulator-ready signals are tcgen05.commit arrivals delivered to both CTAs.
// kMode 1: row maxima only (atomicMax per head at the end of a query); kMode 2: E = exp2(logit - max) as bf16 into the
// scratch (the backward's S layout) and the row sums in 2^-22 fixed point.
// =============================================================================================
namespace fp {
constexpr int kProducerWarps = 8;
constexpr int kProducerThreads = 32 * kProducerWarps;
constexpr int kRowStep = 2 * kProducerWarps;              // a producer thread copies rows r0 + kRowStep * i of its tile
constexpr int kRowsPerThread = 128 / kRowStep;
constexpr int kIssuerWarp = 8 + kProducerWarps;           // the first issuer warp
constexpr int kIssuersPerStream = 2;
constexpr int kIssuers = 2 * kIssuersPerStream;
constexpr int kThreads = 256 + kProducerThreads + 32 * kIssuers + 32;   // statistics, producers, issuers, Q loader
constexpr int kTileKeys = 256;             // per pair; 128 per CTA
constexpr int kChunkA = 128 * 128;
template <int HP> struct Cfg {
    static constexpr int kBChunk = (HP / 2) * 128;                 // Q_j of this CTA's heads
    static constexpr int kStages = HP == 128 ? 9 : 11;
    // every tile stream has ring slots of its own (a slot is then always filled by the same producer group, which has
    // seen its previous use: waits on a barrier's phase parity cannot be taken for the phase before last)
    static constexpr int kStages0 = (kStages + 1) / 2;             // stream 0: slots [0, kStages0)
    static constexpr int kStages1 = kStages / 2;                   // stream 1: slots [kStages0, kStages)
    static constexpr int kOffB = 0;
    static constexpr int kOffRing = kQChunks * kBChunk;
    static constexpr int kOffMisc = kOffRing + kStages * kChunkA;
    static constexpr int kSmemBytes = kOffMisc + 1024 + 512 + 1024;   // row maxima + barriers + alignment slack
    static constexpr int kTmemCols = 4 * HP;                       // two pairs of accumulator buffers
    static_assert(kSmemBytes <= 232448, "shared memory of one SM");
};
}  // namespace fp

template <int HP, int kMode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(fp::kThreads, 1)
smla_fwd_logits_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const KParams p) {
    using namespace fp;
    using C = Cfg<HP>;
    constexpr int NH = HP / 2;
    constexpr int kStages = C::kStages;
    const uint32_t rank = cluster_ctarank();
    const int cta = blockIdx.x >> 1;         // the pair
    const int n_ctas = gridDim.x >> 1;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    uint8_t* misc = smem + C::kOffMisc;
    float* m2_s = reinterpret_cast<float*>(misc);             // [HP] row maximum in base-2 units, +inf for padded heads
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc + 1024);
    const uint32_t bar_full = smem_u32(bars);               // [kStages] gathered chunk landed
    const uint32_t bar_empty = bar_full + 8 * kStages;      // [kStages] the UMMAs reading the slot finished
    const uint32_t bar_bfull = bar_empty + 8 * kStages;     // [9] Q column chunk of the current query landed
    const uint32_t bar_bfree = bar_bfull + 8 * kQChunks;    // [9] the query's last UMMAs on the chunk finished
    const uint32_t bar_tfull = bar_bfree + 8 * kQChunks;    // [4] accumulator buffer complete
    const uint32_t bar_tempty = bar_tfull + 32;             // [4] the softmax warps have read the buffer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 1024 + 8 * (2 * kStages + 2 * kQChunks + 8));
    volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t tok = smem_u32(tmem_slot + 2);           // [2] chunks issued so far in each stream: the issuers' hand-over
    const uint32_t bar_drain = smem_u32(tmem_slot + 4);     // [kIssuers] used only while winding down after an abort
    static_assert(8 * (2 * kStages + 2 * kQChunks + 8) + 16 + 8 * kIssuers <= 512, "barrier area");
    const WaitCtx wc{p.g_err, s_abort, p.wait_limit, map_to_cta(smem_u32(tmem_slot + 1), rank ^ 1)};

    if (threadIdx.x == 0) {
        *s_abort = 0;
        tmem_slot[2] = tmem_slot[3] = 0;
        for (int i = 0; i < kStages; ++i) {
            // the even CTA's "full" also counts one arrival forwarded from the odd CTA
            mbar_init(bar_full + 8 * i, kProducerThreads / 2 + (rank == 0 ? 1 : 0));   // one producer group per slot
            mbar_init(bar_empty + 8 * i, 1);
        }
        for (int i = 0; i < kQChunks; ++i) {
            mbar_init(bar_bfull + 8 * i, 1);
            mbar_init(bar_bfree + 8 * i, 2);     // both issuers' last UMMAs on the chunk
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(bar_tfull + 8 * i, 1);
            mbar_init(bar_tempty + 8 * i, 16);   // eight statistics warps in each CTA
        }
        for (int i = 0; i < kIssuers; ++i) mbar_init(bar_drain + 8 * i, 1);
        fence_mbar_init();
    }
    if (warp == kIssuerWarp) {
        tmem_alloc_2cta(smem_u32(tmem_slot), C::kTmemCols);
        tmem_relinquish_2cta();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // barriers of both CTAs are initialised before anyone signals across
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int n_tp = p.topk_pad / (2 * kTileKeys);      // tile pairs; the forward pads the top-k to a multiple of 512
    const int nq = p.nq;

    if (warp >= 8 && warp < kIssuerWarp) {
        // ------------------------------------------------------------------ gather producers
        // Two groups of kProducerWarps / 2 warps, one per tile stream: group x fills every second ring position, the
        // chunks of tile 2t + x, so a warp waits and arrives once per two positions and the streams do not hold each
        // other up.
        const int grp = (warp - 8) / (kProducerWarps / 2);
        const int pt = threadIdx.x - 256 - grp * (kProducerThreads / 2);
        const int u = pt & 7;               // 16-byte unit inside a 128-byte chunk row
        const int r0 = pt >> 3;             // rows r0 + kRowStep * i of the CTA's 128 keys
        const uint32_t dst0 = s_base + C::kOffRing + r0 * 128 + ((u ^ (r0 & 7)) << 4);
        const char* kvb = reinterpret_cast<const char*>(p.kv) + u * 16;
        const uint64_t pol_keep = l2_policy_evict_last();
        // raw index values, loaded one tile ahead and turned into kv rows when they are used
        QMeta qm_next = load_qmeta(p, p.q0 + (cta < nq ? cta : 0));
        int idx_next[kRowsPerThread];
        auto load_idx = [&](int ql, int tp) {
            if (ql >= nq) {
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) idx_next[i] = -1;
                return;
            }
            if (tp == 0) qm_next = load_qmeta(p, p.q0 + ql);
#pragma unroll
            for (int i = 0; i < kRowsPerThread; ++i) {
                const int key = (2 * tp + grp) * kTileKeys + static_cast<int>(rank) * 128 + r0 + kRowStep * i;
                idx_next[i] = key < p.topk ? __ldg(p.indices + static_cast<size_t>(p.q0 + ql) * p.topk + key) : -1;
            }
        };
        load_idx(cta, 0);
        const int ring0 = grp ? C::kStages0 : 0, ring_n = grp ? C::kStages1 : C::kStages0;
        int rs = 0;                         // slot of the group's ring
        uint32_t ph = 1;                    // parity that means "slot free" for the current pass over the ring
        for (int ql = cta; ql < nq; ql += n_ctas) {
            for (int tp = 0; tp < n_tp; ++tp) {
                const char* src[kRowsPerThread];
                uint32_t nb[kRowsPerThread];    // 0: slot out of range, read nothing and land zeros
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) {
                    const int row = gather_row(idx_next[i], qm_next, p);
                    nb[i] = row >= 0 ? 16u : 0u;
                    src[i] = kvb + static_cast<size_t>(row >= 0 ? row : 0) * (kDQK * 2);
                }
                if (tp + 1 < n_tp) load_idx(ql, tp + 1);
                else load_idx(ql + n_ctas, 0);
                for (int j = 0; j < kQChunks; ++j) {
                    const int s = ring0 + rs;
                    mbar_wait(bar_empty + 8 * s, ph, wc, kErrFwd + 11, kPollSleepNs);
                    const uint32_t d = dst0 + s * kChunkA;
#pragma unroll
                    for (int i = 0; i < kRowsPerThread; ++i)
                        cp_async16_zfill_hint(d + i * kRowStep * 128, src[i] + j * 128, nb[i], pol_keep);
                    cp_async_mbar_arrive_noinc(bar_full + 8 * s);
                    if (++rs == ring_n) {
                        rs = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == kIssuerWarp + kIssuers) {
        // ------------------------------------------------------------------ Q chunks of the query (all heads)
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            const uint64_t pol_stream = l2_policy_evict_first();
            uint32_t qpar = 1;              // parity of "chunk free" left by the previous query
            for (int ql = cta; ql < nq; ql += n_ctas, qpar ^= 1) {
                const int row0 = (p.q0 + ql) * p.h_q + NH * static_cast<int>(rank);
                for (int j = 0; j < kQChunks; ++j) {
                    if (ql != cta) mbar_wait(bar_bfree + 8 * j, qpar, wc, kErrFwd + 16, kPollSleepNs);
                    mbar_arrive_expect_tx(bar_bfull + 8 * j, C::kBChunk);
                    tma_load_2d_hint(s_base + C::kOffB + j * C::kBChunk, &tm_q, 64 * j, row0, bar_bfull + 8 * j, pol_stream);
                }
            }
        }
    } else if (warp >= kIssuerWarp && warp < kIssuerWarp + kIssuers) {
        if (lane == 0 && rank == 1) {
            if (warp == kIssuerWarp) {
                // -------------------------------------------------------------- forward slot-full to the even CTA
                int rs[2] = {0, 0};
                uint32_t ph[2] = {0, 0}, qpar = 0;
                for (int ql = cta; ql < nq; ql += n_ctas, qpar ^= 1) {
                    for (int tp = 0; tp < n_tp; ++tp) {
                        for (int j = 0; j < kQChunks; ++j) {
                            // this CTA's half of Q is part of what "full" promises
                            if (tp == 0) mbar_wait(bar_bfull + 8 * j, qpar, wc, kErrFwd + 15);
#pragma unroll
                            for (int sub = 0; sub < 2; ++sub) {
                                const int s = (sub ? C::kStages0 : 0) + rs[sub];
                                mbar_spin(bar_full + 8 * s, ph[sub], wc, kErrFwd + 17);
                                // The copies have landed in this CTA's shared memory (the wait above saw them
                                // complete); make them visible to the tensor core's proxy here, then signal without
                                // a cluster-scope release (hundreds of cycles per call).
                                fence_proxy_async_smem();
                                mbar_arrive_cluster_relaxed(map_to_cta(bar_full + 8 * s, 0));
                                if (++rs[sub] == (sub ? C::kStages1 : C::kStages0)) {
                                    rs[sub] = 0;
                                    ph[sub] ^= 1;
                                }
                            }
                        }
                    }
                }
            }
        } else if (lane == 0) {
            // ------------------------------------------------------------------ UMMA issuers for the pair
            // Issuer i takes the ring positions i, i + kIssuers, ...: chunks y, y + kIssuersPerStream, ... (y = i / 2) of
            // stream x = i % 2, the tiles 2t + x, accumulated into buffer 2 * (pair parity) + x.
            const int i = warp - kIssuerWarp;
            const int x = i & 1, y = i >> 1;
            constexpr uint32_t idesc = make_idesc_bf16(256, HP, 0, 0);
            const uint64_t desc_hi = make_smem_desc(0, 16, 1024, kSwizzle128) & 0xFFFFFFFF00000000ull;
            const uint32_t desc_lo = static_cast<uint32_t>(make_smem_desc(0, 16, 1024, kSwizzle128));
            const uint32_t a_lo0 = desc_lo + ((s_base + C::kOffRing) >> 4);
            const uint32_t b_lo0 = desc_lo + ((s_base + C::kOffB) >> 4);
            const int n_queries = nq > cta ? (nq - cta + n_ctas - 1) / n_ctas : 0;
            const int total = n_queries * n_tp * kQChunks;      // chunks of a stream
            const uint32_t my_tok = tok + 4 * x;
            int j = y, tp = 0, gtp = 0;
            uint32_t qpar = 0;
            const int ring0 = x ? C::kStages0 : 0, ring_n = x ? C::kStages1 : C::kStages0;
            static_assert(kIssuersPerStream < C::kStages1, "an issuer meets a slot again only after the stream's other issuers");
            int rs = y;                     // chunk c of the stream sits in slot c mod ring_n of the stream's ring
            uint32_t ph = 0;
            for (int c = y; c < total; c += kIssuersPerStream) {
                const int s = ring0 + rs;
                const int b = 2 * (gtp & 1) + x;
                if (j == 0) mbar_spin(bar_tempty + 8 * b, ((gtp >> 1) & 1) ^ 1, wc, kErrFwd + 13);
                if (tp == 0) mbar_wait(bar_bfull + 8 * j, qpar, wc, kErrFwd + 12);
                mbar_spin(bar_full + 8 * s, ph, wc, kErrFwd + 14);
                fence_proxy_async_smem();        // the chunk was written by cp.async, the tensor core reads it
                flag_wait(my_tok, static_cast<uint32_t>(c), wc, kErrFwd + 19);
                tc_fence_after_sync();
                const uint32_t d = tmem + b * HP;
                const uint32_t a_lo = a_lo0 + s * (kChunkA >> 4);
                const uint32_t b_lo = b_lo0 + j * (C::kBChunk >> 4);
                umma_ss_2cta(d, desc_hi | a_lo, desc_hi | b_lo, idesc, j != 0);
#pragma unroll
                for (int kk = 1; kk < 4; ++kk)   // 32 bytes further along K = +2 in the address field
                    umma_ss_2cta(d, desc_hi | (a_lo + 2 * kk), desc_hi | (b_lo + 2 * kk), idesc, 1);
                tc_fence_before_sync();
                flag_store(my_tok, static_cast<uint32_t>(c + 1));
                // The UMMAs on one accumulator complete in the order they were issued, so the commit behind a tile's
                // last chunk covers the chunks the stream's other issuer put in before it.
                umma_commit_2cta_mask(bar_empty + 8 * s, 3);
                if (tp == n_tp - 1) umma_commit_2cta_mask(bar_bfree + 8 * j, 3);
                if (j == kQChunks - 1) umma_commit_2cta_mask(bar_tfull + 8 * b, 3);
                j += kIssuersPerStream;
                if (j >= kQChunks) {
                    j -= kQChunks;
                    ++gtp;
                    if (++tp == n_tp) {
                        tp = 0;
                        qpar ^= 1;
                    }
                }
                rs += kIssuersPerStream;
                if (rs >= ring_n) {
                    rs -= ring_n;
                    ph ^= 1;
                }
            }
            if (*s_abort) {
                umma_commit_2cta_mask(bar_drain + 8 * i, 1);
                mbar_wait_drain(bar_drain + 8 * i, 0, p.wait_limit);
            }
        }
    } else {
        // ------------------------------------------------------------------ row statistics / exponentials
        const int quarter = warp & 3;
        const int g = warp >> 2;            // head half
        const int row = quarter * 32 + lane;
        const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
        const uint64_t pol_stream = l2_policy_evict_first();
        const int t = threadIdx.x;
        // second pass: the row maximum found by the first pass, in base-2 units, fetched one query ahead
        auto load_stat = [&](int ql) -> float {
            if (kMode == 1 || ql >= nq || t >= HP) return 0.f;
            if (t >= p.h_q) return __int_as_float(0x7f800000);
            return ordered_to_float(p.m_ord[static_cast<size_t>(p.q0 + ql) * p.h_q + t]) * p.scale_log2e;
        };
        float stat_next = load_stat(cta);
        int gt = 0;                         // tiles so far: pair gt >> 1, tile gt & 1 of the pair
        const int n_tiles = 2 * n_tp;
        for (int ql = cta; ql < nq; ql += n_ctas) {
            const int qg = p.q0 + ql;
            const QMeta qm = load_qmeta(p, qg);
            if constexpr (kMode == 2) {
                asm volatile("bar.sync 1, 256;" ::: "memory");      // every softmax warp is done with the previous query
                if (t < HP) m2_s[t] = stat_next;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                stat_next = load_stat(ql + n_ctas);
            }
            // what this lane keeps for heads g * NH + lane and g * NH + 32 + lane over the query's tiles
            float keep_max[2] = {__int_as_float(0xff800000), __int_as_float(0xff800000)};
            unsigned long long keep_sum[2] = {0ull, 0ull};
            for (int tile = 0; tile < n_tiles; ++tile, ++gt) {
                const int key = tile * kTileKeys + static_cast<int>(rank) * 128 + row;
                const int idx = key < p.topk ? __ldg(p.indices + static_cast<size_t>(qg) * p.topk + key) : -1;
                const bool valid = slot_valid(idx, key, qm, p);
                const int b = gt & 3;               // 2 * (pair parity) + tile of the pair
                mbar_wait(bar_tfull + 8 * b, (gt >> 2) & 1, wc, kErrFwd + 18, kPollSleepNs);
                tc_fence_after_sync();
                const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + b * HP + g * NH;
                if constexpr (kMode == 1) {
                    // the maximum over the warp's 32 keys of every head: one warp reduction per head
                    const float ninf = __int_as_float(0xff800000);
#pragma unroll 1
                    for (int c0 = 0; c0 < NH; c0 += 32) {
                        uint32_t pv[32];
                        tmem_ld_32x32(taddr + c0, pv);
                        tmem_ld_wait();
                        float mine = ninf;
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const float r = redux_max_f32(valid ? __uint_as_float(pv[c]) : ninf);
                            if (lane == c) mine = r;
                        }
                        if (c0 == 0) keep_max[0] = fmaxf(keep_max[0], mine);
                        else keep_max[1] = fmaxf(keep_max[1], mine);
                    }
                } else {
                    const size_t off = static_cast<size_t>(p.scr0 + ql) * p.topk_pad * HP + scratch_offset(key, g * NH, p.topk_pad);
                    __nv_bfloat16* s_out = p.s_scr + off;
                    const uint32_t vmask = valid ? 0xFFFFFFFFu : 0u;
                    const uint32_t fxmask = valid ? 0x007FFFFFu : 0u;
#pragma unroll 1
                    for (int c0 = 0; c0 < NH; c0 += 16) {
                        uint32_t pv[16];
                        tmem_ld_32x16(taddr + c0, pv);
                        tmem_ld_wait();
                        uint32_t so[8];
                        const float4* l4 = reinterpret_cast<const float4*>(m2_s + g * NH + c0);
                        unsigned mine = 0;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const float4 l = l4[v];
                            const float lv[4] = {l.x, l.y, l.z, l.w};
                            float sv[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int c = 4 * v + e;
                                // E <= 1 (+ one rounding): the same logits produced the maximum in the first pass
                                const float ex = ex2_approx(fmaf(__uint_as_float(pv[c]), p.scale_log2e, -lv[e]));
                                sv[e] = ex;
                                // Row sums in 2^-22 fixed point: integer warp reductions and integer atomics add in
                                // any order to the same result.  E + 2.0f lies in [2, 4), where one unit of the mantissa
                                // is 2^-22: the low 23 bits of the sum's bit pattern are E in fixed point, rounded to
                                // nearest, without a conversion instruction (conversions, exponentials and warp
                                // reductions share one quarter-rate pipe).  2048 terms lose at most 2^-12 of a sum >= 1.
                                const unsigned fx = __float_as_uint(ex + 2.0f) & fxmask;
                                const unsigned r = redux_add_u32(fx);
                                if (lane == ((c0 + c) & 31)) mine = r;
                            }
                            so[2 * v] = pack_bf16x2(sv[0], sv[1]) & vmask;
                            so[2 * v + 1] = pack_bf16x2(sv[2], sv[3]) & vmask;
                        }
                        // columns c0 .. c0 + 15 went to lanes (c0 & 31) .. (c0 & 31) + 15
                        if (static_cast<unsigned>(lane - (c0 & 31)) < 16u) {
                            if (c0 < 32) keep_sum[0] += mine;
                            else keep_sum[1] += mine;
                        }
                        __nv_bfloat16* s0 = s_out + static_cast<size_t>(c0) * p.topk_pad;
                        const size_t blk = static_cast<size_t>(p.topk_pad) * 8;
                        st_global_v4_hint(s0, so[0], so[1], so[2], so[3], pol_stream);
                        st_global_v4_hint(s0 + blk, so[4], so[5], so[6], so[7], pol_stream);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                // the accumulator reads have completed (tcgen05.wait::ld), which is all the issuers need to know
                if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * b);
            }
            // this warp's share of the query's row statistics: integer atomics, so the order in which the warps
            // arrive does not change the result
#pragma unroll
            for (int k = 0; k < NH / 32; ++k) {
                const int head = g * NH + 32 * k + lane;
                if (head < p.h_q) {
                    const size_t o = static_cast<size_t>(qg) * p.h_q + head;
                    if constexpr (kMode == 1) atomicMax(p.m_ord + o, float_to_ordered(keep_max[k]));
                    else atomicAdd(p.l_fix + o, keep_sum[k]);
                }
            }
        }
    }
    abort_wind_down(s_abort);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves while the other may still signal it or read its operands
    if (warp == kIssuerWarp) tmem_dealloc_2cta(tmem, C::kTmemCols);
}

// Row statistics of the forward start at -inf (maximum) and 0 (sum).
__global__ void smla_fwd_stats_init_kernel(int* m_ord, unsigned long long* l_fix, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        m_ord[i] = kOrderedNegInf;
        l_fix[i] = 0ull;
    }
}

// =============================================================================================
// dkv as persistent 2-CTA clusters: one pair per query, all 576 columns of d.
//
//   dKV^T[d, key] = dO^T . S + Q^T . dS with cta_group::2 UMMAs of M = 256 rows of d (128 per CTA) x N = 128 keys
//   (64 supplied by each CTA): a CTA reads 4 KB of A and 2 KB of B per 64 cycles of math, where the single-CTA
//   128x128x16 form reads 8 KB, which is all the shared-memory bandwidth there is.  The S / dS scratch of a query is
//   read once (half a tile per CTA) instead of once per d-part.
//
//   blocks of d   0: [0,256)   1: [256,512)   2: [512,576) (Q^T . dS only: V has 512 columns)
//   CTA r holds rows [128 r, 128 r + 128) of blocks 0 and 1 as resident Q^T / dO^T chunk pairs.  Block 2 is issued
//   from the slot pair (3, 4) in both CTAs: slot 4 holds chunk 8 in both, so both compute the same 64 real rows in
//   lanes 64-127 (lanes 0-63 repeat chunk 3's rows and are dropped); CTA (tile & 1) drains them, which keeps the
//   reductions of the two CTAs equal over two tiles.
//   warp 0      producer: resident chunks per query; per 128-key tile this CTA's 64 keys of S and dS, two stages
//   warp 1      even CTA: UMMA issuer for the pair; odd CTA: relays "my half landed" to the even CTA's barriers
//   warps 2-17  drain, two groups of eight on alternate accumulator units (ring of four 128-column units per CTA):
//               lane = d row, one predicated fp32 reduction per key = 128 contiguous bytes of dKV
// =============================================================================================
namespace dp {
constexpr int kThreads = 576;
constexpr int kTileKeys = 128;
constexpr int kUnits = 4;
constexpr int kTileStages = 2;
template <int HP> struct Cfg {
    static constexpr int kChunk = HP * 128;                 // resident chunk [HP heads x 64 d] bytes
    static constexpr int kHalfMat = HP * 128;               // S (or dS) of 64 keys: [HP/8][64 keys][8 heads]
    static constexpr int kStage = 2 * kHalfMat;             // S then dS
    static constexpr int kOffQ = 0;                         // 5 slots
    static constexpr int kOffDO = 5 * kChunk;               // 4 slots
    static constexpr int kOffStage = 9 * kChunk;
    static constexpr int kOffMisc = kOffStage + kTileStages * kStage;
    static constexpr int kOffIdx = kOffMisc + 256;          // [2 groups][2 tile parities][2 key halves][64] int
    static constexpr int kSmemBytes = kOffMisc + 256 + 2048 + 1024;
};
}  // namespace dp

// kStaged: instead of adding a slot's [576] contribution into dKV with fp32 reductions (whose order, and therefore
// rounding, changes from run to run), write it to the slot's own row of a staging buffer; smla_dkv_segment_sum_kernel
// then adds the rows that belong to one kv row in a fixed order.
template <int HP, bool kStaged = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(dp::kThreads, 1)
smla_dkv_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_ds, const KParams p) {
    using namespace dp;
    using C = Cfg<HP>;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;
    const int nq = p.nq;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffMisc);
    const uint32_t bar_tfull = smem_u32(bars);                        // [2] tile stage landed (even CTA: in both CTAs)
    const uint32_t bar_tempty = bar_tfull + 8 * kTileStages;          // [2] the tile's UMMAs finished
    const uint32_t bar_res = bar_tempty + 8 * kTileStages;            // 1  resident chunks landed (even CTA: in both CTAs)
    const uint32_t bar_resfree = bar_res + 8;                         // 1  all UMMAs of the query finished
    const uint32_t bar_ufull = bar_resfree + 8;                       // [kUnits] accumulator unit complete
    const uint32_t bar_uempty = bar_ufull + 8 * kUnits;               // [kUnits] (even CTA) both CTAs have drained the unit
    const uint32_t bar_drain = bar_uempty + 8 * kUnits;               // 1  used only while winding down after an abort
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::kOffMisc + 8 * (2 * kTileStages + 3 + 2 * kUnits));
    static_assert(8 * (2 * kTileStages + 3 + 2 * kUnits) + 8 <= 256, "barrier area");
    volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const WaitCtx wc{p.g_err, s_abort, p.wait_limit, map_to_cta(smem_u32(tmem_slot + 1), rank ^ 1)};

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int i = 0; i < kTileStages; ++i) {
            mbar_init(bar_tfull + 8 * i, rank == 0 ? 2 : 1);   // own expect_tx arrival (+ the odd CTA's relayed one)
            mbar_init(bar_tempty + 8 * i, 1);
        }
        mbar_init(bar_res, rank == 0 ? 2 : 1);
        mbar_init(bar_resfree, 1);
        mbar_init(bar_drain, 1);
        for (int i = 0; i < kUnits; ++i) {
            mbar_init(bar_ufull + 8 * i, 1);
            mbar_init(bar_uempty + 8 * i, 16);                 // eight drain warps of the unit's group in each CTA
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_2cta(smem_u32(tmem_slot), 512);
        tmem_relinquish_2cta();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // barriers of both CTAs are initialised before anyone signals across
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int n_tiles = p.topk_pad / kTileKeys;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_do);
            tma_prefetch_desc(&tm_s);
            tma_prefetch_desc(&tm_ds);
            const uint64_t pol_stream = l2_policy_evict_first();
            int s = 0;
            uint32_t ph = 1, k = 0;        // ph: parity that means "stage free" in the current pass over the ring
            for (int ql = pair; ql < nq; ql += n_pairs, ++k) {
                // the resident operands are replaced once the previous query's UMMAs are done; the drain warps
                // meanwhile still work through the accumulator ring, so the reductions do not pause
                if (k) mbar_wait(bar_resfree, (k - 1) & 1, wc, kErrDkv + 6, kPollSleepNs);
                mbar_arrive_expect_tx(bar_res, 9 * C::kChunk);
                const int row0 = (p.q0 + ql) * p.h_q;
                for (int j = 0; j < 4; ++j) {          // slots 0..3: chunks {2r, 2r+1} of block 0 and block 1
                    const int chunk = (j >> 1) * 4 + 2 * static_cast<int>(rank) + (j & 1);
                    tma_load_2d_hint(s_base + C::kOffQ + j * C::kChunk, &tm_q, 64 * chunk, row0, bar_res, pol_stream);
                    tma_load_2d_hint(s_base + C::kOffDO + j * C::kChunk, &tm_do, 64 * chunk, row0, bar_res, pol_stream);
                }
                tma_load_2d_hint(s_base + C::kOffQ + 4 * C::kChunk, &tm_q, 64 * 8, row0, bar_res, pol_stream);
                for (int tile = 0; tile < n_tiles; ++tile) {
                    mbar_wait(bar_tempty + 8 * s, ph, wc, kErrDkv + 1, kPollSleepNs);
                    mbar_arrive_expect_tx(bar_tfull + 8 * s, C::kStage);
                    const uint32_t dst = s_base + C::kOffStage + s * C::kStage;
                    // box = this CTA's 64 keys of every head block -> [HP/8][64 keys][8 heads]
                    const int kb = tile * (kTileKeys / 32) + 2 * static_cast<int>(rank);
                    tma_load_4d_hint(dst, &tm_s, 0, kb, 0, p.scr0 + ql, bar_tfull + 8 * s, pol_stream);
                    tma_load_4d_hint(dst + C::kHalfMat, &tm_ds, 0, kb, 0, p.scr0 + ql, bar_tfull + 8 * s, pol_stream);
                    if (++s == kTileStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            if (rank == 1) {
                // -------------------------------------------------------------- relay "landed" to the even CTA
                // TMA wrote the data (async proxy) and the tensor core reads it (async proxy): no proxy fence; the
                // relaxed arrive costs a few cycles where a cluster-scope release costs hundreds.
                int s = 0;
                uint32_t ph = 0, k = 0;
                for (int ql = pair; ql < nq; ql += n_pairs, ++k) {
                    mbar_wait(bar_res, k & 1, wc, kErrDkv + 10);
                    mbar_arrive_cluster_relaxed(map_to_cta(bar_res, 0));
                    for (int tile = 0; tile < n_tiles; ++tile) {
                        mbar_spin(bar_tfull + 8 * s, ph, wc, kErrDkv + 11);
                        mbar_arrive_cluster_relaxed(map_to_cta(bar_tfull + 8 * s, 0));
                        if (++s == kTileStages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                }
            } else {
                // -------------------------------------------------------------- UMMA issuer for the pair
                constexpr uint32_t idesc = make_idesc_bf16(256, 128, 1, 0);   // A MN-major (d contiguous), B K-major
                int s = 0;
                uint32_t ph = 0, k = 0, unit = 0;
                for (int ql = pair; ql < nq; ql += n_pairs, ++k) {
                    mbar_wait(bar_res, k & 1, wc, kErrDkv + 2);
                    for (int tile = 0; tile < n_tiles; ++tile) {
                        mbar_wait(bar_tfull + 8 * s, ph, wc, kErrDkv + 4);
                        const uint32_t st_s = s_base + C::kOffStage + s * C::kStage;
                        const uint32_t st_ds = st_s + C::kHalfMat;
                        for (int blk = 0; blk < 3; ++blk, ++unit) {
                            const int us = unit % kUnits;
                            mbar_wait(bar_uempty + 8 * us, ((unit / kUnits) & 1) ^ 1, wc, kErrDkv + 3);
                            tc_fence_after_sync();
                            const uint32_t d = tmem + us * 128;
                            // each CTA's 128 rows: slot pair (0,1), (2,3) or, for block 2, (3,4)
                            const int slot = blk == 2 ? 3 : 2 * blk;
                            if (blk < 2) {
                                const uint32_t a_do = s_base + C::kOffDO + slot * C::kChunk;
#pragma unroll
                                for (int ks = 0; ks < HP / 16; ++ks)
                                    umma_ss_2cta(d, make_smem_desc(a_do + ks * 2048, C::kChunk, 1024, kSwizzle128),
                                                 make_smem_desc(st_s + ks * 2048, 1024, 128, kSwizzleNone), idesc, ks != 0);
                            }
                            const uint32_t a_q = s_base + C::kOffQ + slot * C::kChunk;
#pragma unroll
                            for (int ks = 0; ks < HP / 16; ++ks)
                                umma_ss_2cta(d, make_smem_desc(a_q + ks * 2048, C::kChunk, 1024, kSwizzle128),
                                             make_smem_desc(st_ds + ks * 2048, 1024, 128, kSwizzleNone), idesc,
                                             blk < 2 || ks != 0);
                            umma_commit_2cta_mask(bar_ufull + 8 * us, 3);
                        }
                        umma_commit_2cta_mask(bar_tempty + 8 * s, 3);
                        if (++s == kTileStages) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    umma_commit_2cta_mask(bar_resfree, 3);
                }
                if (*s_abort) {   // winding down: nothing of this thread's may still be in the tensor pipe at dealloc
                    umma_commit_2cta_mask(bar_drain, 1);
                    mbar_wait_drain(bar_drain, 0, p.wait_limit);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ drain (this CTA's 128 rows of every unit)
        // Two groups of eight warps take alternate units: one group's fixed cost per unit (wait, accumulator load,
        // indices) runs under the other group's reductions.
        const int dw = warp - 2;                // 0..15
        const int grp = dw >> 3;
        const int quarter = warp & 3;           // the TMEM lane quarter a warp may read is warp % 4
        const int e = (dw >> 2) & 1;            // which 64 keys of the 128-key tile this warp scatters
        const int member = dw & 3;              // the four warps of a (group, key half) share one index buffer
        const int upq = n_tiles * 3;            // units per query: even, because top-k is padded to 256 keys
        // index buffers [group][tile parity][key half][64]: filled by member 0 from registers it loaded one tile ahead,
        // published with a named barrier of the four warps.  Every tile shows up in both groups' unit sequences and
        // the barrier keeps the four within one tile of each other, so two buffers per (group, key half) suffice.
        int* idx_base = reinterpret_cast<int*>(smem + C::kOffIdx) + (grp * 4 + e) * 64;
        const int bar_id = 1 + grp * 2 + e;
        const uint32_t uempty0 = map_to_cta(bar_uempty, 0);
#ifdef SMLA_RED_EVICT_LAST
        const uint64_t pol_keep = l2_policy_evict_last();
#endif
        int pf[2] = {-1, -1};
        // (the dKV row a valid slot adds to, -1 for an unused slot)
        auto fetch_idx = [&](int ql, int tile) {
            if (ql >= nq) {
                pf[0] = pf[1] = -1;
                return;
            }
            const int qg = p.q0 + ql;
            const QMeta qm = load_qmeta(p, qg);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int key = tile * kTileKeys + 64 * e + 32 * i + lane;
                const int idx = key < p.topk ? __ldg(p.indices + static_cast<size_t>(qg) * p.topk + key) : -1;
                pf[i] = slot_valid(idx, key, qm, p) ? qm.kv_base + idx : -1;
            }
        };
        if (member == 0) fetch_idx(pair, 0);
        uint32_t qn = 0;
        for (int ql = pair; ql < nq; ql += n_pairs, ++qn) {
            int last_tile = -1;
            for (int ul = grp; ul < upq; ul += 2) {
                const int tile = ul / 3, blk = ul - tile * 3;
                const uint32_t unit = qn * upq + ul;
                const int us = unit % kUnits;
                int* idx_s = idx_base + (tile & 1) * 128;
                if (tile != last_tile) {
                    last_tile = tile;
                    if (member == 0) {
                        idx_s[lane] = pf[0];
                        idx_s[32 + lane] = pf[1];
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                    if (member == 0) {
                        if (tile + 1 < n_tiles) fetch_idx(ql, tile + 1);
                        else fetch_idx(ql + n_pairs, 0);
                    }
                }
                mbar_wait(bar_ufull + 8 * us, (unit / kUnits) & 1, wc, kErrDkv + 5, kPollSleepNs);
                tc_fence_after_sync();
                // blocks 0, 1: every row is real (d = 256 blk + 128 rank + row).  Block 2: rows 64..127 are d 512..575
                // in both CTAs; the CTA whose turn it is drains them.
                const bool mine = blk < 2 || (quarter >= 2 && static_cast<uint32_t>(tile & 1) == rank);
                if (mine) {
                    const int d0 = blk < 2 ? 256 * blk + 128 * static_cast<int>(rank) : 512 - 64;
                    float* out = p.dKV + d0 + quarter * 32 + lane;
                    // staged form: the row of slot (query, first key of this warp's 64) in the staging buffer
                    float* sout = nullptr;
                    if constexpr (kStaged)
                        sout = p.staging + (static_cast<size_t>(p.scr0 + ql) * p.topk_pad + tile * kTileKeys + 64 * e) * kDQK +
                               d0 + quarter * 32 + lane;
                    const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + us * 128 + 64 * e;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        uint32_t r[32];
                        tmem_ld_32x32(taddr + 32 * i, r);
                        int ix[32];
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            const int4 t = reinterpret_cast<const int4*>(idx_s)[8 * i + v];
                            ix[4 * v] = t.x; ix[4 * v + 1] = t.y; ix[4 * v + 2] = t.z; ix[4 * v + 3] = t.w;
                        }
                        tmem_ld_wait();
                        if constexpr (kStaged) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                st_global_f32_if_row(sout + static_cast<size_t>(32 * i + j) * kDQK, __uint_as_float(r[j]), ix[j]);
                        } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
#ifdef SMLA_RED_EVICT_LAST
                            red_add_f32_if_row_hint(out + static_cast<size_t>(static_cast<unsigned>(ix[j])) * kDQK,
                                                    __uint_as_float(r[j]), ix[j], pol_keep);
#else
                            red_add_f32_if_row(out + static_cast<size_t>(static_cast<unsigned>(ix[j])) * kDQK,
                                               __uint_as_float(r[j]), ix[j]);
#endif
                        }
                    }
                }
                // the accumulator reads have completed (tcgen05.wait::ld), which is all the issuer needs to know
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(uempty0 + 8 * us);
            }
        }
    }
    abort_wind_down(s_abort);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves while the other may still signal it or read its operands
    if (warp == 1) tmem_dealloc_2cta(tmem, 512);
}


// =============================================================================================
// Reproducible dKV, second half: one warp per kv row walks the row's slots in the index inverse (CSR by kv row, flat
// slot ids ascending) and adds their staged [576] contributions in that order, so a row's sum is rounded the same way
// in every run.  A pass covers the queries [q_lo, q_hi); a row's slots of that range are a contiguous piece of its
// CSR segment (found by binary search), and passes follow one another in a fixed order.
// =============================================================================================
__global__ void __launch_bounds__(256) smla_dkv_segment_sum_kernel(const int* __restrict__ row_ptr,
                                                                   const int* __restrict__ entries,
                                                                   const float* __restrict__ staging, float* __restrict__ dKV,
                                                                   int s_kv, int topk, int topk_pad, int q_lo, int q_hi) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= s_kv) return;
    const int b = __ldg(row_ptr + row), e = __ldg(row_ptr + row + 1);
    auto lower = [&](long long flat) {      // first position in [b, e) whose flat slot id is >= flat
        int lo = b, hi = e;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(entries + mid) < flat) lo = mid + 1;
            else hi = mid;
        }
        return lo;
    };
    const int i0 = lower(static_cast<long long>(q_lo) * topk), i1 = lower(static_cast<long long>(q_hi) * topk);
    if (i1 <= i0) return;
    constexpr int kPer = kDQK / 32;          // 18 elements per lane
    float acc[kPer];
#pragma unroll
    for (int k = 0; k < kPer; ++k) acc[k] = 0.f;
    auto src_of = [&](int i) {
        const int flat = __ldg(entries + i);
        const int q = flat / topk;
        return staging + (static_cast<size_t>(q - q_lo) * topk_pad + (flat - q * topk)) * kDQK + lane;
    };
    int i = i0;
    for (; i + 1 < i1; i += 2) {             // two slots in flight; the additions keep the slot order
        const float* s0 = src_of(i);
        const float* s1 = src_of(i + 1);
        float v0[kPer], v1[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            v0[k] = __ldcs(s0 + 32 * k);
            v1[k] = __ldcs(s1 + 32 * k);
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k) acc[k] = (acc[k] + v0[k]) + v1[k];
    }
    if (i < i1) {
        const float* s0 = src_of(i);
#pragma unroll
        for (int k = 0; k < kPer; ++k) acc[k] += __ldcs(s0 + 32 * k);
    }
    float* out = dKV + static_cast<size_t>(row) * kDQK + lane;
#pragma unroll
    for (int k = 0; k < kPer; ++k) out[32 * k] += acc[k];
}

// =============================================================================================
// dq: one CTA per (query, d-part of kSplit column chunks); 14 warps; two CTAs per SM, so that one's start-up (TMEM,
// first gathers) and epilogue run under the other's tiles.
//   warps 0-3   epilogue: TMEM -> bf16 -> dQ[q, head, d]; lane = head, so a thread stores whole 64-byte pieces of
//               its head's row
//   warps 4-11  producers: per 64-key tile the part's columns of the kv rows picked by index (16-byte
//               cp.async into the swizzled layout)
//   warp 13     TMA: the dS scratch tile
//   warp 12     UMMA issuer: acc[128 heads, d of the part] += dS^T . Kg  (both operands MN-major: the key index is
//               the contraction and runs along shared-memory rows).  Heads are the M side so that N can be 256
//               columns of d: a 128x256x16 UMMA reads 12 KB of shared memory per 128 cycles of math, whereas the
//               transposed 128x128x16 form reads 8 KB per 64 cycles, which is all the bandwidth there is (measured
//               ~100 cycles per UMMA instead of 64).  With HP = 64 the upper 64 accumulator rows are computed from
//               whatever follows the dS tile in shared memory and never read.
//               (Two issuers taking alternate tiles, handing over through a counter, changed nothing at one CTA
//               per SM: the kernel waits for its gathers, not for the issuer.)
// =============================================================================================
namespace dq {
constexpr int kThreads = 448;
constexpr int kProducerWarps = 8;
constexpr int kTileKeys = 64;
template <int HP, int kSplit> struct Cfg {
    static constexpr int kStages = (HP == 64 && kSplit <= 3) ? 3 : 2;   // what fits twice into an SM's shared memory
    static_assert(kSplit >= 1 && kSplit <= 4, "one UMMA covers the part: N = 64 kSplit <= 256");
    static constexpr int kKgBytes = kSplit * 8192;
    static constexpr int kDsBytes = (HP / 64) * 8192;
    static constexpr int kStage = kKgBytes + kDsBytes;     // dS right after Kg
    static constexpr int kOffMisc = kStages * kStage;
    // the A operand always spans 128 heads: with HP = 64 its upper half reads 8 KB past the dS tile
    static constexpr int kSmemBytes = kOffMisc + 256 + 1024 + (HP == 64 ? 8192 : 0);
    static_assert(2 * (kSmemBytes + 1024) <= 233472, "two CTAs per SM");
    static constexpr int kTmemCols = 256;                  // up to 256 columns of d; two CTAs share the SM's 512
    static constexpr int kRowBytes = kSplit * 128 + 16;    // epilogue staging of one head's row
    static_assert(128 * kRowBytes <= kOffMisc, "the epilogue stages its rows in the pipeline's memory");
};
}  // namespace dq

// kNorm (forward, o = S.V): the scratch holds unnormalised E = exp2(logit - max); every head's row is divided by its
// row sum on the way out, and the CTA of d-part 0 writes lse = max + log2(sum).
template <int HP, int kSplit, int kTotal, bool kNorm = false>
__global__ void __launch_bounds__(dq::kThreads, 2)
smla_dq_kernel(const __grid_constant__ CUtensorMap tm_ds, const KParams p) {
    using namespace dq;
    using C = Cfg<HP, kSplit>;
    constexpr int kStages = C::kStages;
    constexpr int kParts = (kTotal + kSplit - 1) / kSplit;
    const int part = blockIdx.x % kParts;
    const int ql = blockIdx.x / kParts;
    const int qg = p.q0 + ql;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // d-part i gathers kv column chunks [i kSplit, (i + 1) kSplit): 3 x 3 of 9 for dQ, 2 x 4 of 8 for o = S.V
    const int chunk0 = part * kSplit;
    const int n_ch = kTotal - chunk0 < kSplit ? kTotal - chunk0 : kSplit;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t s_base = smem_u32(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffMisc);
    const uint32_t bar_full = smem_u32(bars);             // [kStages]
    const uint32_t bar_empty = bar_full + 8 * kStages;    // [kStages]
    const uint32_t bar_acc = bar_empty + 8 * kStages;     // 1
    const uint32_t bar_drain = bar_acc + 8;               // 1  used only while winding down after an abort
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::kOffMisc + 8 * (2 * kStages + 2));
    volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const WaitCtx wc{p.g_err, s_abort, p.wait_limit, 0u};

    if (threadIdx.x == 0) {
        *s_abort = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(bar_full + 8 * i, kProducerWarps * 32 + 1);   // cp.async threads + the TMA expect_tx arrival
            mbar_init(bar_empty + 8 * i, 1);
        }
        mbar_init(bar_acc, 1);
        mbar_init(bar_drain, 1);
        fence_mbar_init();
    }
    if (warp == 12) {
        tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int n_tiles = p.topk_pad / kTileKeys;

    if (warp >= 4 && warp < 12) {
        const int pt = threadIdx.x - 128;   // 0..255
        const int u = pt & 7;
        const int r0 = pt >> 3;             // rows r0 and r0+32 of the tile
        const uint32_t dst0 = s_base + r0 * 128 + ((u ^ (r0 & 7)) << 4);
        const char* kvb = reinterpret_cast<const char*>(p.kv) + chunk0 * 128 + u * 16;
        const uint64_t pol_keep = l2_policy_evict_last();
        // the indices of a tile are loaded one tile ahead, so that their latency is never in front of the copies
        // (raw values, turned into kv rows when they are used: nothing may depend on a load here)
        int idx_next[2];
        const QMeta qm = load_qmeta(p, qg);
        auto load_idx = [&](int tile) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int key = tile * kTileKeys + r0 + 32 * i;
                idx_next[i] = (tile < n_tiles && key < p.topk) ? __ldg(p.indices + static_cast<size_t>(qg) * p.topk + key) : -1;
            }
        };
        load_idx(0);
        int s = 0;
        uint32_t ph = 1;                    // parity that means "stage free" for the current pass over the ring
        for (int tile = 0; tile < n_tiles; ++tile) {
            const char* src[2];
            uint32_t nb[2];   // 0: slot out of range, read nothing and land zeros (no shared stand-in row: it would be a hot spot)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = gather_row(idx_next[i], qm, p);
                nb[i] = row >= 0 ? 16u : 0u;
                src[i] = kvb + static_cast<size_t>(row >= 0 ? row : 0) * (kDQK * 2);
            }
            load_idx(tile + 1);
            mbar_wait(bar_empty + 8 * s, ph, wc, kErrDq + 1, kPollSleepNs);
            const uint32_t d = dst0 + s * C::kStage;
            for (int c = 0; c < n_ch; ++c) {
                cp_async16_zfill_hint(d + c * 8192, src[0] + c * 128, nb[0], pol_keep);
                cp_async16_zfill_hint(d + c * 8192 + 32 * 128, src[1] + c * 128, nb[1], pol_keep);
            }
            cp_async_mbar_arrive_noinc(bar_full + 8 * s);
            if (++s == kStages) {
                s = 0;
                ph ^= 1;
            }
        }
    } else if (warp == 13) {
        if (lane == 0) tma_prefetch_desc(&tm_ds);
        const uint64_t pol_stream = l2_policy_evict_first();
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 1;
            for (int tile = 0; tile < n_tiles; ++tile) {
                mbar_wait(bar_empty + 8 * s, ph, wc, kErrDq + 4, kPollSleepNs);
                const uint32_t dst = s_base + s * C::kStage;
                mbar_arrive_expect_tx(bar_full + 8 * s, C::kDsBytes);
                // box = 64 keys of every head block -> [HP/8][64 keys][8 heads]
                tma_load_4d_hint(dst + C::kKgBytes, &tm_ds, 0, tile * (kTileKeys / 32), 0, p.scr0 + ql, bar_full + 8 * s, pol_stream);
                if (++s == kStages) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
    } else if (warp == 12) {
        if (lane == 0) {
            // N = the part's column chunks (up to 256 d) in one UMMA
            const uint32_t idesc1 = make_idesc_bf16(128, n_ch * 64, 1, 1);
            // A = dS^T: [HP/8 head blocks][64 keys][8 heads], 8-key groups 128 B apart, head blocks 1 KB apart.
            // Descriptors: the fixed fields once, the address (16-byte units, the low 14 bits) added per UMMA.
            const uint64_t a_hi = make_smem_desc(0, 128, 1024, kSwizzleNone) & 0xFFFFFFFF00000000ull;
            const uint32_t a_lo0 = static_cast<uint32_t>(make_smem_desc(0, 128, 1024, kSwizzleNone)) + ((s_base + C::kKgBytes) >> 4);
            const uint64_t b_hi = make_smem_desc(0, 8192, 1024, kSwizzle128) & 0xFFFFFFFF00000000ull;
            const uint32_t b_lo0 = static_cast<uint32_t>(make_smem_desc(0, 8192, 1024, kSwizzle128)) + (s_base >> 4);
            int s = 0;
            uint32_t ph = 0;
            for (int tile = 0; tile < n_tiles; ++tile) {
                mbar_spin(bar_full + 8 * s, ph, wc, kErrDq + 2);
                fence_proxy_async_smem();
                tc_fence_after_sync();
                const uint32_t a_lo = a_lo0 + s * (C::kStage >> 4), b_lo = b_lo0 + s * (C::kStage >> 4);
#pragma unroll
                for (int ks = 0; ks < kTileKeys / 16; ++ks) {
                    const uint64_t a = a_hi | (a_lo + ks * (256 >> 4));
                    umma_ss(tmem, a, b_hi | (b_lo + ks * (2048 >> 4)), idesc1, (tile | ks) != 0);
                }
                umma_commit(bar_empty + 8 * s);
                if (++s == kStages) {
                    s = 0;
                    ph ^= 1;
                }
            }
            umma_commit(bar_acc);
            if (*s_abort) {   // winding down: nothing of this thread's may still be in the tensor pipe at dealloc
                umma_commit(bar_drain);
                mbar_wait_drain(bar_drain, 0, p.wait_limit);
            }
        }
    } else {
        const int quarter = warp;
        mbar_wait(bar_acc, 0, wc, kErrDq + 3, kPollSleepNs);
        tc_fence_after_sync();
        // lane = head, columns = d of the part.  Each thread converts its head's row to bf16 in shared memory (the
        // pipeline stages are idle by now; rows 16 bytes apart modulo 128 so that the 16-byte stores of a warp
        // spread over all banks) and sends it off as one bulk copy: whole cache lines instead of 32 scattered
        // 16-byte pieces per store instruction.
        constexpr int kPitch = kTotal * 64;      // 576 for dQ, 512 for o
        constexpr int kRowBytes = C::kRowBytes;
        const int head = quarter * 32 + lane;
        const uint32_t row_s = s_base + head * kRowBytes;
        float inv = 1.f;
        if constexpr (kNorm) {
            if (head < p.h_q) {
                const size_t o = static_cast<size_t>(qg) * p.h_q + head;
                const float l = static_cast<float>(p.l_fix[o]) * (1.f / kFixScale);
                inv = l > 0.f ? 1.f / l : 0.f;               // no valid slot: o = 0, lse = +inf
                if (part == 0)
                    p.lse_out[o] = (l > 0.f ? fmaf(ordered_to_float(p.m_ord[o]), p.scale_log2e, __log2f(l))
                                            : __int_as_float(0x7f800000)) * p.lse_out_mult;
            }
        }
        if (quarter * 32 < p.h_q) {               // warp-uniform: heads are padded to a multiple of 8 only
            const uint32_t taddr = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int cg = 0; cg < n_ch * 4; ++cg) {   // 16 columns at a time: two CTAs per SM leave 64 registers a thread
                uint32_t r[16];
                tmem_ld_32x16(taddr + cg * 16, r);
                tmem_ld_wait();
                if constexpr (kNorm) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * inv);
                }
#pragma unroll
                for (int v = 0; v < 2; ++v)
                    st_shared_v4(row_s + cg * 32 + v * 16,
                                 pack_bf16x2(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1])),
                                 pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                                 pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                                 pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
            }
            if (head < p.h_q) {
                fence_proxy_async_smem();         // this thread's row only: no one else touches it
                bulk_store(p.gout + (static_cast<size_t>(qg) * p.h_q + head) * kPitch + chunk0 * 64, row_s, n_ch * 128);
                bulk_commit();
                bulk_wait_read();
            }
        }
    }
    abort_wind_down(s_abort);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 12) tmem_dealloc(tmem, C::kTmemCols);
}

// =============================================================================================
// Self-test of the bounded waits: one CTA waits on a barrier (or a counter) that nothing ever signals, with a
// short limit.  The wait must give up, record `code`, raise the abort flag, and the kernel must return
// normally; a second wait must then return at once.  out[0] = what the first wait returned, out[1] = what
// the second returned, out[2] = cycles the first wait took.
// =============================================================================================
__global__ void __launch_bounds__(32) smla_selftest_wait_kernel(int* g_err, long long* out, int which, long long limit,
                                                                int code) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    __shared__ uint32_t counter;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        counter = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const WaitCtx wc{g_err, &abort_flag, limit, 0u};
        const long long t0 = clock64();
        bool a;
        if (which == 0) a = mbar_wait(smem_u32(&bar), 0, wc, code, kPollSleepNs);
        else if (which == 1) a = mbar_spin(smem_u32(&bar), 0, wc, code);
        else a = flag_wait(smem_u32(&counter), 1u, wc, code);
        const long long t1 = clock64();
        const bool b = mbar_wait(smem_u32(&bar), 0, wc, code + 1);
        out[0] = a ? 1 : 0;
        out[1] = b ? 1 : 0;
        out[2] = t1 - t0;
    }
}

}  // namespace smla
