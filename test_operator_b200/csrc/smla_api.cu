// C ABI and host launchers of the sparse MLA backward (see include/smla_bwd.h).
// Host side only: argument checks, workspace carving, TMA descriptor encoding, kernel launches.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <map>
#include <mutex>

#include "../../include/smla_bwd.h"
#include "smla_kernels.cuh"
#include "smla_index_inverse.cuh"

namespace {

using smla::KParams;

constexpr size_t kAlign = 256;
constexpr size_t kDefaultBudget = size_t(6) << 30;  // scratch budget when the caller gives none

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

thread_local int g_last_launches = 0;
thread_local int g_last_device_code = 0;

// ---- schedule of one backward pass ------------------------------------------------------------------------
// chunks == 0: the four kernels one after another on the caller's stream.
// chunks >= 2: the queries of a pass are cut into `chunks` parts; recompute and dq of part c run on the caller's
//   stream while the dkv kernel of part c - 1 runs on a second (internal, higher-priority) stream with a grid of
//   `dkv_pairs` clusters, the recompute kernels taking the remaining clusters.  The dkv kernel is bound by the
//   chip's fp32 reduction rate, not by its SMs, so it loses little on fewer SMs, and the SMs it leaves do the
//   tensor-core work of the other two kernels meanwhile.
constexpr int kMaxChunks = 16;
std::atomic<int> g_sched_chunks{-2};      // -2: not yet read from the environment; -1: chosen per head count
std::atomic<int> g_sched_dkv_pairs{0};
constexpr int kDefaultChunks = -1;        // chosen from the head count, see auto_chunks
constexpr int kDefaultDkvPairs = 0;       // 0: chosen from the head count, see auto_dkv_pairs
std::atomic<long long> g_wait_limit{smla::kWaitLimitCycles};

void schedule(int* chunks, int* dkv_pairs) {
    int c = g_sched_chunks.load();
    if (c < -1) {
        int cc = kDefaultChunks, dp = kDefaultDkvPairs;
        if (const char* e = std::getenv("SMLA_SCHEDULE")) {      // "chunks,dkv_pairs"
            int a = 0, b = 0;
            if (std::sscanf(e, "%d,%d", &a, &b) == 2 && a >= -1 && a != 1 && a <= kMaxChunks && b >= 0) {
                cc = a;
                dp = b;
            }
        }
        g_sched_dkv_pairs.store(dp);
        g_sched_chunks.store(cc);
        c = cc;
    }
    *chunks = c;
    *dkv_pairs = g_sched_dkv_pairs.load();
}

// Clusters for the dkv kernel when the caller leaves the choice to the library: its share of the three kernels'
// time, measured with each kernel alone on a whole B200 (top-k 2048; dkv 3.8 ms at either head count, recompute +
// dq 3.4 ms at 128 heads and 2.65 ms at 64).  The step time is flat within +-3 clusters of these.
// Measured on B200, alternating the schedules on one GPU: with 64 heads two overlapped parts beat one kernel after the
// other by 4 % (5.89 against 6.16 ms; three parts and more lose to two, each launch has its own tail); with 128 heads the
// kernels one after the other are 2.5 % faster than any overlapped form (7.39 against 7.60 ms, 8.64 against 8.85 ms over
// a second of steps): there the recompute and dQ kernels want all of the SMs more than the dKV kernel minds having them.
int auto_chunks(int h_pad) { return h_pad > 64 ? 0 : 2; }

int auto_dkv_pairs(int h_pad, int resident) {
    const double share = h_pad > 64 ? 0.50 : 0.60;
    int n = static_cast<int>(resident * share + 0.5);
    if (n < 1) n = 1;
    if (n > resident - 1) n = resident - 1;
    return n;
}

// Second stream and the events that order it against the caller's stream, one set per device, created on the first
// call that needs them.  The mutex is held while a call enqueues, so that two host threads do not interleave their
// records and waits on the shared events.
struct DevSched {
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_part[kMaxChunks] = {};
    bool ready = false;
};
std::mutex g_dev_sched_mutex;
DevSched g_dev_sched[64];

DevSched* dev_sched_locked() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    DevSched& d = g_dev_sched[dev];
    if (d.ready) return &d;
    int lo = 0, hi = 0;
    if (cudaDeviceGetStreamPriorityRange(&lo, &hi) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithPriority(&d.side, cudaStreamNonBlocking, hi) != cudaSuccess) return nullptr;
    bool ok = cudaEventCreateWithFlags(&d.ev_fork, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&d.ev_join, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < kMaxChunks && ok; ++i) ok = cudaEventCreateWithFlags(&d.ev_part[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) return nullptr;
    d.ready = true;
    return &d;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link-time libcuda dependency,
// so the library also loads on a machine without a driver (symbol checks on a CPU-only box).
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
    });
    return fn;
}

// 2-D bf16 tensor [rows, cols] with row pitch `pitch_bytes`, box {box_cols, box_rows}, 128-byte swizzle.
bool make_map_2d(CUtensorMap* m, const void* base, uint64_t cols, uint64_t rows, uint64_t pitch_bytes, uint32_t box_cols,
                 uint32_t box_rows) {
    EncodeFn enc = get_encode_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// S / dS scratch [queries][h_pad/8 head blocks][topk_pad keys][8 heads] bf16 as a 4-D tensor whose rows are 32 keys
// of one head block (512 contiguous bytes); a box takes `box_keys` keys of every head block of one query and lands
// as [head block][keys][8 heads], the no-swizzle core-matrix order.
bool make_map_scratch(CUtensorMap* m, const void* base, uint64_t queries, int topk_pad, int h_pad, uint32_t box_keys) {
    EncodeFn enc = get_encode_fn();
    if (!enc) return false;
    const uint64_t head_blocks = uint64_t(h_pad) / 8;
    cuuint64_t dims[4] = {256, uint64_t(topk_pad) / 32, head_blocks, queries};
    cuuint64_t strides[3] = {512, uint64_t(topk_pad) * 16, head_blocks * uint64_t(topk_pad) * 16};
    cuuint32_t box[4] = {256, box_keys / 32, static_cast<cuuint32_t>(head_blocks), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

struct Plan {
    int h_pad;       // heads padded to 64 or 128
    int topk_pad;    // top-k padded to a multiple of 256
    int q_chunk;     // queries per pass
    size_t err_off, delta_off, s_off, ds_off, total;
};

bool check_params(const smla_bwd_params* p) {
    if (!p) return false;
    if (p->s_q <= 0 || p->s_kv <= 0 || p->topk <= 0) return false;
    if (p->h_q <= 0 || p->h_q > 128 || (p->h_q % 8) != 0) return false;
    // int32 row coordinates in the TMA descriptors
    if (static_cast<long long>(p->s_q) * p->h_q > INT_MAX) return false;
    if (reinterpret_cast<uintptr_t>(p->query_meta) & 15) return false;
    return true;
}

bool make_plan(const smla_bwd_params* p, size_t budget, Plan* pl) {
    if (!check_params(p)) return false;
    pl->h_pad = p->h_q <= 64 ? 64 : 128;
    pl->topk_pad = (p->topk + 255) / 256 * 256;   // the pair recompute kernel walks 256-key tiles
    const size_t per_q = size_t(pl->topk_pad) * pl->h_pad * 2 /*bf16*/ * 2 /*S and dS*/;
    pl->err_off = 0;
    pl->delta_off = kAlign;
    const size_t fixed = align_up(pl->delta_off + size_t(p->s_q) * p->h_q * 4, kAlign);
    if (budget == 0) budget = kDefaultBudget;
    size_t qc = budget > fixed ? (budget - fixed) / per_q : 0;
    if (qc < 1) qc = 1;
    if (qc > size_t(p->s_q)) qc = p->s_q;
    // scratch rows are TMA row coordinates (int32)
    while (qc > 1 && qc * size_t(pl->topk_pad) > size_t(INT_MAX)) qc /= 2;
    pl->q_chunk = int(qc);
    pl->s_off = fixed;
    pl->ds_off = align_up(pl->s_off + qc * per_q / 2, kAlign);
    pl->total = align_up(pl->ds_off + qc * per_q / 2, kAlign);
    return true;
}

// Largest q_chunk that fits a given workspace (layout must match what run() will use).
bool plan_for_workspace(const smla_bwd_params* p, size_t ws_bytes, Plan* pl) {
    if (!make_plan(p, ws_bytes, pl)) return false;
    while (pl->total > ws_bytes && pl->q_chunk > 1) {
        Plan t = *pl;
        const size_t per_q = size_t(pl->topk_pad) * pl->h_pad * 4;
        size_t over = pl->total - ws_bytes;
        int dec = int(over / per_q) + 1;
        t.q_chunk = pl->q_chunk - dec < 1 ? 1 : pl->q_chunk - dec;
        t.ds_off = align_up(t.s_off + size_t(t.q_chunk) * per_q / 2, kAlign);
        t.total = align_up(t.ds_off + size_t(t.q_chunk) * per_q / 2, kAlign);
        *pl = t;
    }
    return pl->total <= ws_bytes;
}

template <typename K>
bool set_smem(K kernel, int bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
}

// How many 2-CTA clusters of `kernel` the current device runs at once: the grid of a persistent kernel.  A
// cluster needs two free SMs of one GPC, so this can be less than half the SM count.  Looked up once per
// (kernel, device).
template <typename K>
int resident_pairs(K kernel, int threads, int smem_bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return 0;
    const std::pair<const void*, int> key(reinterpret_cast<const void*>(kernel), dev);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int n = 0;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) return 0;
        n = sms / 2;
    }
    cache[key] = n;
    return n;
}

template <int HP>
int launch_chain(const smla_bwd_params* p, const Plan& pl, uint8_t* ws, cudaStream_t st, int stages, bool allow_overlap,
                 const smla_bwd_det_params* det = nullptr) {
    using namespace smla;
    __nv_bfloat16* s_scr = reinterpret_cast<__nv_bfloat16*>(ws + pl.s_off);
    __nv_bfloat16* ds_scr = reinterpret_cast<__nv_bfloat16*>(ws + pl.ds_off);
    float* delta = reinterpret_cast<float*>(ws + pl.delta_off);

    CUtensorMap tm_qnh, tm_donh, tm_qhp, tm_dohp, tm_s, tm_ds;
    const uint64_t qrows = uint64_t(p->s_q) * p->h_q;
    bool ok = true;
    ok &= make_map_2d(&tm_qnh, p->q, kDQK, qrows, kDQK * 2, 64, HP / 2);
    ok &= make_map_2d(&tm_donh, p->dO, kDV, qrows, kDV * 2, 64, HP / 2);
    ok &= make_map_2d(&tm_qhp, p->q, kDQK, qrows, kDQK * 2, 64, HP);
    ok &= make_map_2d(&tm_dohp, p->dO, kDV, qrows, kDV * 2, 64, HP);
    // S / dS scratch: the dkv kernel loads [128 keys x 64 heads] boxes, the dq kernel [64 keys x 64 heads]
    ok &= make_map_scratch(&tm_s, s_scr, uint64_t(pl.q_chunk), pl.topk_pad, HP, 64);
    ok &= make_map_scratch(&tm_ds, ds_scr, uint64_t(pl.q_chunk), pl.topk_pad, HP, 64);
    if (!ok) return SMLA_ERR_LAUNCH;

    // per device, so set on every call (cheap) rather than once per process
    bool attr_ok = set_smem(smla_recompute_pair_kernel<HP>, rp::Cfg<HP>::kSmemBytes);
    attr_ok &= set_smem(smla_dkv_pair_kernel<HP>, dp::Cfg<HP>::kSmemBytes);
    if (det) attr_ok &= set_smem(smla_dkv_pair_kernel<HP, true>, dp::Cfg<HP>::kSmemBytes);
    attr_ok &= set_smem(smla_dq_kernel<HP, kDqChunks, kQChunks>, dq::Cfg<HP, kDqChunks>::kSmemBytes);
    if (!attr_ok) return SMLA_ERR_LAUNCH;

    KParams kp{};
    kp.kv = reinterpret_cast<const __nv_bfloat16*>(p->kv);
    kp.indices = p->indices;
    kp.lse = p->lse;
    kp.delta = delta;
    kp.s_scr = s_scr;
    kp.ds_scr = ds_scr;
    kp.dKV = p->dKV;
    kp.dQ = reinterpret_cast<__nv_bfloat16*>(p->dQ);
    kp.gout = kp.dQ;
    kp.g_err = reinterpret_cast<int*>(ws + pl.err_off);
    kp.s_q = p->s_q;
    kp.s_kv = p->s_kv;
    kp.h_q = p->h_q;
    kp.topk = p->topk;
    kp.topk_pad = pl.topk_pad;
    kp.sm_scale = p->sm_scale > 0.f ? p->sm_scale : 1.0f / sqrtf(float(kDQK));
    kp.scale_log2e = kp.sm_scale * 1.4426950408889634f;
    kp.lse_mult = p->lse_is_base2 ? 1.0f : 1.4426950408889634f;
    kp.causal = p->q_start_index_s != SMLA_NO_CAUSAL;
    kp.q_start = kp.causal ? p->q_start_index_s : 0;

    kp.qmeta = reinterpret_cast<const int4*>(p->query_meta);
    kp.wait_limit = g_wait_limit.load();
    kp.staging = det ? det->staging : nullptr;

    if (stages & SMLA_STAGE_DELTA) {
        const int n_rows = p->s_q * p->h_q;
        smla_delta_kernel<<<(n_rows + 7) / 8, 256, 0, st>>>(reinterpret_cast<const uint4*>(p->O),
                                                          reinterpret_cast<const uint4*>(p->dO), delta, n_rows);
        ++g_last_launches;
    }
    const int pairs_r = resident_pairs(smla_recompute_pair_kernel<HP>, rp::kThreads, rp::Cfg<HP>::kSmemBytes);
    const int pairs_d = resident_pairs(smla_dkv_pair_kernel<HP>, dp::kThreads, dp::Cfg<HP>::kSmemBytes);
    if (pairs_r <= 0 || pairs_d <= 0) return SMLA_ERR_LAUNCH;
    auto launch_recompute = [&](cudaStream_t s_, int pairs) {
        smla_recompute_pair_kernel<HP><<<2 * (kp.nq < pairs ? kp.nq : pairs), rp::kThreads, rp::Cfg<HP>::kSmemBytes, s_>>>(tm_qnh, tm_donh, kp);
        ++g_last_launches;
    };
    auto launch_dkv = [&](cudaStream_t s_, int pairs) {
        const int grid = 2 * (kp.nq < pairs ? kp.nq : pairs);
        if (det) {
            // reproducible form: per-slot contributions to the staging rows, then one warp per kv row adds its slots
            // of this pass in CSR order
            smla_dkv_pair_kernel<HP, true><<<grid, dp::kThreads, dp::Cfg<HP>::kSmemBytes, s_>>>(tm_qhp, tm_dohp, tm_s, tm_ds, kp);
            smla_dkv_segment_sum_kernel<<<(p->s_kv + 7) / 8, 256, 0, s_>>>(det->row_ptr, det->entries, det->staging, p->dKV, p->s_kv,
                                                                           p->topk, pl.topk_pad, kp.q0, kp.q0 + kp.nq);
            g_last_launches += 2;
            return;
        }
        smla_dkv_pair_kernel<HP><<<grid, dp::kThreads, dp::Cfg<HP>::kSmemBytes, s_>>>(tm_qhp, tm_dohp, tm_s, tm_ds, kp);
        ++g_last_launches;
    };
    auto launch_dq = [&](cudaStream_t s_) {
        smla_dq_kernel<HP, kDqChunks, kQChunks><<<kp.nq * (kQChunks / kDqChunks), dq::kThreads, dq::Cfg<HP, kDqChunks>::kSmemBytes, s_>>>(tm_ds, kp);
        ++g_last_launches;
    };

    int chunks = 0, dkv_pairs = 0;
    schedule(&chunks, &dkv_pairs);
    if (chunks < 0) chunks = auto_chunks(HP);
    const int all = SMLA_STAGE_RECOMPUTE | SMLA_STAGE_DKV | SMLA_STAGE_DQ;
    if (dkv_pairs <= 0) dkv_pairs = auto_dkv_pairs(HP, pairs_d < pairs_r ? pairs_d : pairs_r);
    if (!allow_overlap || det || (stages & all) != all || dkv_pairs >= pairs_d || dkv_pairs >= pairs_r) chunks = 0;

    for (int q0 = 0; q0 < p->s_q; q0 += pl.q_chunk) {
        const int nq = (p->s_q - q0 < pl.q_chunk) ? p->s_q - q0 : pl.q_chunk;
        // a part must keep every cluster of both kernels busy for a few queries, or cutting costs more than it hides
        int parts = chunks;
        while (parts >= 2 && nq / parts < 4 * pairs_r) --parts;
        if (parts < 2) {
            kp.q0 = q0;
            kp.nq = nq;
            kp.scr0 = 0;
            if (stages & SMLA_STAGE_RECOMPUTE) launch_recompute(st, pairs_r);
            if (stages & SMLA_STAGE_DKV) launch_dkv(st, pairs_d);
            if (stages & SMLA_STAGE_DQ) launch_dq(st);
            continue;
        }
        std::lock_guard<std::mutex> lock(g_dev_sched_mutex);
        DevSched* ds = dev_sched_locked();
        if (!ds) return SMLA_ERR_LAUNCH;
        // the second stream starts behind everything the caller's stream holds so far (dKV cleared, Delta, the
        // previous pass's readers of the scratch)
        if (cudaEventRecord(ds->ev_fork, st) != cudaSuccess || cudaStreamWaitEvent(ds->side, ds->ev_fork, 0) != cudaSuccess)
            return SMLA_ERR_LAUNCH;
        for (int c = 0; c < parts; ++c) {
            const int a0 = static_cast<int>(static_cast<long long>(nq) * c / parts);
            const int a1 = static_cast<int>(static_cast<long long>(nq) * (c + 1) / parts);
            kp.q0 = q0 + a0;
            kp.nq = a1 - a0;
            kp.scr0 = a0;
            launch_recompute(st, c == 0 ? pairs_r : pairs_r - dkv_pairs);
            if (cudaEventRecord(ds->ev_part[c], st) != cudaSuccess ||
                cudaStreamWaitEvent(ds->side, ds->ev_part[c], 0) != cudaSuccess)
                return SMLA_ERR_LAUNCH;
            launch_dkv(ds->side, c == parts - 1 ? pairs_d : dkv_pairs);
            launch_dq(st);
        }
        if (cudaEventRecord(ds->ev_join, ds->side) != cudaSuccess || cudaStreamWaitEvent(st, ds->ev_join, 0) != cudaSuccess)
            return SMLA_ERR_LAUNCH;
    }
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- forward ---------------------------------------------------------------------------------------------
// Workspace: error word | row maxima [s_q, h_q] i32 | row sums [s_q, h_q] u64 | E scratch (bf16, one matrix per query).
struct FwdPlan {
    int h_pad, topk_pad, q_chunk;
    size_t err_off, m_off, l_off, s_off, total;
};

bool check_fwd_params(const smla_fwd_params* p) {
    if (!p) return false;
    if (p->s_q <= 0 || p->s_kv <= 0 || p->topk <= 0) return false;
    if (p->h_q <= 0 || p->h_q > 128 || (p->h_q % 8) != 0) return false;
    if (static_cast<long long>(p->s_q) * p->h_q > INT_MAX) return false;
    if (reinterpret_cast<uintptr_t>(p->query_meta) & 15) return false;
    return true;
}

void fwd_layout(const smla_fwd_params* p, FwdPlan* pl, size_t qc) {
    const size_t unit = size_t(pl->topk_pad) * pl->h_pad * 2;   // one bf16 matrix per query
    const size_t rows = size_t(p->s_q) * p->h_q;
    pl->q_chunk = int(qc);
    pl->err_off = 0;
    pl->m_off = kAlign;
    pl->l_off = align_up(pl->m_off + rows * 4, kAlign);
    pl->s_off = align_up(pl->l_off + rows * 8, kAlign);
    pl->total = align_up(pl->s_off + qc * unit, kAlign);
}

bool make_fwd_plan(const smla_fwd_params* p, size_t budget, FwdPlan* pl) {
    if (!check_fwd_params(p)) return false;
    pl->h_pad = p->h_q <= 64 ? 64 : 128;
    pl->topk_pad = (p->topk + 511) / 512 * 512;   // the logits kernel walks pairs of 256-key tiles
    const size_t unit = size_t(pl->topk_pad) * pl->h_pad * 2;
    if (budget == 0) budget = kDefaultBudget;
    fwd_layout(p, pl, 1);
    const size_t fixed = pl->s_off;
    size_t qc = budget > fixed ? (budget - fixed) / unit : 0;
    if (qc < 1) qc = 1;
    if (qc > size_t(p->s_q)) qc = p->s_q;
    while (qc > 1 && qc * size_t(pl->topk_pad) > size_t(INT_MAX)) qc /= 2;
    fwd_layout(p, pl, qc);
    return true;
}

bool fwd_plan_for_workspace(const smla_fwd_params* p, size_t ws_bytes, FwdPlan* pl) {
    if (!make_fwd_plan(p, ws_bytes, pl)) return false;
    const size_t unit = size_t(pl->topk_pad) * pl->h_pad * 2;
    while (pl->total > ws_bytes && pl->q_chunk > 1) {
        const size_t over = pl->total - ws_bytes;
        const int dec = int(over / unit) + 1;
        fwd_layout(p, pl, pl->q_chunk - dec < 1 ? 1 : pl->q_chunk - dec);
    }
    return pl->total <= ws_bytes;
}

// Three passes over the queries: row maxima of the logits (nothing but 4 bytes per row is written); E = exp2(logit -
// max) as bf16 into the scratch plus its row sums; o = E.V divided by the sum on the way out, and lse.  The logits are
// computed twice (576 of the forward's 1088 multiply-adds per slot) in exchange for never existing in memory.
template <int HP>
int launch_fwd_chain(const smla_fwd_params* p, const FwdPlan& pl, uint8_t* ws, cudaStream_t st) {
    using namespace smla;
    __nv_bfloat16* s_scr = reinterpret_cast<__nv_bfloat16*>(ws + pl.s_off);
    CUtensorMap tm_qnh, tm_s;
    const uint64_t qrows = uint64_t(p->s_q) * p->h_q;
    bool ok = true;
    ok &= make_map_2d(&tm_qnh, p->q, kDQK, qrows, kDQK * 2, 64, HP / 2);
    ok &= make_map_scratch(&tm_s, s_scr, uint64_t(pl.q_chunk), pl.topk_pad, HP, 64);
    if (!ok) return SMLA_ERR_LAUNCH;
    bool attr_ok = set_smem(smla_fwd_logits_pair_kernel<HP, 1>, fp::Cfg<HP>::kSmemBytes);
    attr_ok &= set_smem(smla_fwd_logits_pair_kernel<HP, 2>, fp::Cfg<HP>::kSmemBytes);
    // o = E.V: the two d-parts gather V column chunks [0,4) and [4,8)
    attr_ok &= set_smem(smla_dq_kernel<HP, kVChunks / 2, kVChunks, true>, dq::Cfg<HP, kVChunks / 2>::kSmemBytes);
    if (!attr_ok) return SMLA_ERR_LAUNCH;

    KParams kp{};
    kp.kv = reinterpret_cast<const __nv_bfloat16*>(p->kv);
    kp.indices = p->indices;
    kp.s_scr = s_scr;
    kp.m_ord = reinterpret_cast<int*>(ws + pl.m_off);
    kp.l_fix = reinterpret_cast<unsigned long long*>(ws + pl.l_off);
    kp.lse_out = p->lse;
    kp.lse_out_mult = p->lse_is_base2 ? 1.0f : 0.6931471805599453f;
    kp.g_err = reinterpret_cast<int*>(ws + pl.err_off);
    kp.s_q = p->s_q;
    kp.s_kv = p->s_kv;
    kp.h_q = p->h_q;
    kp.topk = p->topk;
    kp.topk_pad = pl.topk_pad;
    kp.sm_scale = p->sm_scale > 0.f ? p->sm_scale : 1.0f / sqrtf(float(kDQK));
    kp.scale_log2e = kp.sm_scale * 1.4426950408889634f;
    kp.causal = p->q_start_index_s != SMLA_NO_CAUSAL;
    kp.q_start = kp.causal ? p->q_start_index_s : 0;
    kp.gout = reinterpret_cast<__nv_bfloat16*>(p->o);
    kp.qmeta = reinterpret_cast<const int4*>(p->query_meta);
    kp.wait_limit = g_wait_limit.load();
    kp.scr0 = 0;
    const int n_rows = p->s_q * p->h_q;
    smla_fwd_stats_init_kernel<<<(n_rows + 255) / 256, 256, 0, st>>>(kp.m_ord, kp.l_fix, n_rows);
    ++g_last_launches;
    const int pairs_1 = resident_pairs(smla_fwd_logits_pair_kernel<HP, 1>, fp::kThreads, fp::Cfg<HP>::kSmemBytes);
    const int pairs_2 = resident_pairs(smla_fwd_logits_pair_kernel<HP, 2>, fp::kThreads, fp::Cfg<HP>::kSmemBytes);
    if (pairs_1 <= 0 || pairs_2 <= 0) return SMLA_ERR_LAUNCH;
    for (int q0 = 0; q0 < p->s_q; q0 += pl.q_chunk) {
        const int nq = (p->s_q - q0 < pl.q_chunk) ? p->s_q - q0 : pl.q_chunk;
        kp.q0 = q0;
        kp.nq = nq;
        // persistent 2-CTA clusters, one per SM pair (each CTA takes the whole shared memory of its SM)
        smla_fwd_logits_pair_kernel<HP, 1><<<2 * (nq < pairs_1 ? nq : pairs_1), fp::kThreads, fp::Cfg<HP>::kSmemBytes, st>>>(tm_qnh, kp);
        smla_fwd_logits_pair_kernel<HP, 2><<<2 * (nq < pairs_2 ? nq : pairs_2), fp::kThreads, fp::Cfg<HP>::kSmemBytes, st>>>(tm_qnh, kp);
        smla_dq_kernel<HP, kVChunks / 2, kVChunks, true><<<nq * 2, dq::kThreads, dq::Cfg<HP, kVChunks / 2>::kSmemBytes, st>>>(tm_s, kp);
        g_last_launches += 3;
    }
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

// ---- workspace that lives in the library image (smla_bwd_run_noalloc) -----------------------------------
// Every GPU that loads the library carries these bytes until the process exits.
constexpr size_t kStaticWorkspaceBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_ws_mutex;
void* g_static_ws_ptr[kMaxDevices] = {};   // device address of g_static_workspace, per device ordinal

// The array's name is only a host-side handle; the kernels need its device address, which is looked up
// once per device (with that device current) and cached.
int static_workspace_ptr(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SMLA_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_static_ws_mutex);
    if (!g_static_ws_ptr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_workspace) != cudaSuccess || !ptr) return SMLA_ERR_LAUNCH;
        g_static_ws_ptr[dev] = ptr;
    }
    *out = g_static_ws_ptr[dev];
    return SMLA_OK;
}

}  // namespace

extern "C" {

size_t smla_bwd_workspace_size(const smla_bwd_params* p, size_t budget_bytes) {
    Plan pl;
    if (!make_plan(p, budget_bytes, &pl)) return 0;
    return pl.total;
}

int smla_bwd_get_workspace_layout(const smla_bwd_params* p, size_t workspace_bytes, smla_bwd_workspace_layout* out) {
    Plan pl;
    if (!out || !check_params(p)) return SMLA_ERR_BAD_ARG;
    if (!plan_for_workspace(p, workspace_bytes, &pl)) return SMLA_ERR_WORKSPACE;
    out->err_offset = pl.err_off;
    out->delta_offset = pl.delta_off;
    out->s_offset = pl.s_off;
    out->ds_offset = pl.ds_off;
    out->q_chunk = pl.q_chunk;
    out->topk_pad = pl.topk_pad;
    out->h_pad = pl.h_pad;
    out->total_bytes = pl.total;
    return SMLA_OK;
}

namespace {
int run_stages_impl(const smla_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream, int stage_mask,
                    bool allow_overlap, const smla_bwd_det_params* det = nullptr) {
    g_last_launches = 0;
    if (!check_params(p) || !workspace) return SMLA_ERR_BAD_ARG;
    if (!p->q || !p->kv || !p->dO || !p->lse || !p->O || !p->indices || !p->dQ || !p->dKV) return SMLA_ERR_BAD_ARG;
    // TMA needs 16-byte aligned bases; vector loads/stores need the same for the rest
    if (!aligned16(p->q) || !aligned16(p->kv) || !aligned16(p->dO) || !aligned16(p->O) || !aligned16(p->dQ) ||
        !aligned16(p->dKV) || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)))
        return SMLA_ERR_BAD_ARG;
    Plan pl;
    if (!plan_for_workspace(p, workspace_bytes, &pl)) return SMLA_ERR_WORKSPACE;
    if (det) {
        // a pass may hold no more queries than the staging buffer has rows for
        if (p->query_meta || !det->row_ptr || !det->entries || !det->staging || !aligned16(det->staging)) return SMLA_ERR_BAD_ARG;
        const size_t per_q = size_t(pl.topk_pad) * SMLA_D_QK * sizeof(float);
        const size_t fit = det->staging_bytes / per_q;
        if (fit < 1) return SMLA_ERR_WORKSPACE;
        if (size_t(pl.q_chunk) > fit) pl.q_chunk = int(fit);
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    if (stage_mask & SMLA_STAGE_ZERO) {
        if (cudaMemsetAsync(p->dKV, 0, size_t(p->s_kv) * SMLA_D_QK * sizeof(float), st) != cudaSuccess)
            return SMLA_ERR_LAUNCH;
    }
    return pl.h_pad == 64 ? launch_chain<64>(p, pl, ws, st, stage_mask, allow_overlap, det)
                          : launch_chain<128>(p, pl, ws, st, stage_mask, allow_overlap, det);
}
}  // namespace

int smla_bwd_run_deterministic(const smla_bwd_params* p, const smla_bwd_det_params* det, void* workspace,
                               size_t workspace_bytes, void* stream, int stage_mask) {
    if (!det) return SMLA_ERR_BAD_ARG;
    return run_stages_impl(p, workspace, workspace_bytes, stream, stage_mask, false, det);
}

size_t smla_bwd_staging_bytes_per_query(const smla_bwd_params* p) {
    Plan pl;
    if (!make_plan(p, 0, &pl)) return 0;
    return size_t(pl.topk_pad) * SMLA_D_QK * sizeof(float);
}

int smla_bwd_run_stages(const smla_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream, int stage_mask) {
    return run_stages_impl(p, workspace, workspace_bytes, stream, stage_mask, true);
}

int smla_bwd_workspace_init(void* workspace, void* stream) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1))) return SMLA_ERR_BAD_ARG;
    return cudaMemsetAsync(workspace, 0, kAlign, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

int smla_bwd_set_schedule(int chunks, int dkv_pairs) {
    if (chunks < -1 || chunks > kMaxChunks || chunks == 1 || dkv_pairs < 0) return SMLA_ERR_BAD_ARG;   // -1 / 0 pairs: automatic
    g_sched_dkv_pairs.store(dkv_pairs);
    g_sched_chunks.store(chunks);
    return SMLA_OK;
}

void smla_bwd_get_schedule(int* chunks, int* dkv_pairs) {
    int c = 0, d = 0;
    schedule(&c, &d);
    if (chunks) *chunks = c;
    if (dkv_pairs) *dkv_pairs = d;
}

int smla_bwd_run(const smla_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
    return smla_bwd_run_stages(p, workspace, workspace_bytes, stream, SMLA_STAGE_ALL);
}

int smla_bwd_run_noalloc(const smla_bwd_params* p, void* stream) {
    g_last_launches = 0;
    Plan pl;
    if (!check_params(p)) return SMLA_ERR_BAD_ARG;
    // the fixed part (error word, Delta) plus the S / dS scratch of at least one query must fit the built-in array
    if (!plan_for_workspace(p, kStaticWorkspaceBytes, &pl)) return SMLA_ERR_TOO_LARGE_FOR_STATIC;
    void* ws = nullptr;
    const int st = static_workspace_ptr(&ws);
    if (st != SMLA_OK) return st;
    // one stream only: this entry point creates nothing, streams and events included
    return run_stages_impl(p, ws, kStaticWorkspaceBytes, stream, SMLA_STAGE_ALL, false);
}

size_t smla_bwd_noalloc_capacity(void) { return kStaticWorkspaceBytes; }

int smla_bwd_noalloc_status(void* stream) {
    void* ws = nullptr;
    const int st = static_workspace_ptr(&ws);
    if (st != SMLA_OK) return st;
    return smla_bwd_status(ws, stream);
}

size_t smla_fwd_workspace_size(const smla_fwd_params* p, size_t budget_bytes) {
    FwdPlan pl;
    if (!make_fwd_plan(p, budget_bytes, &pl)) return 0;
    return pl.total;
}

int smla_fwd_run(const smla_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream) {
    g_last_launches = 0;
    if (!check_fwd_params(p) || !workspace) return SMLA_ERR_BAD_ARG;
    if (!p->q || !p->kv || !p->indices || !p->o || !p->lse) return SMLA_ERR_BAD_ARG;
    if (!aligned16(p->q) || !aligned16(p->kv) || !aligned16(p->o) || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)))
        return SMLA_ERR_BAD_ARG;
    FwdPlan pl;
    if (!fwd_plan_for_workspace(p, workspace_bytes, &pl)) return SMLA_ERR_WORKSPACE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    return pl.h_pad == 64 ? launch_fwd_chain<64>(p, pl, ws, st) : launch_fwd_chain<128>(p, pl, ws, st);
}

int smla_bwd_delta(const void* O, const void* dO, float* delta, int32_t s_q, int32_t h_q, void* stream) {
    if (!O || !dO || !delta || s_q <= 0 || h_q <= 0 || !aligned16(O) || !aligned16(dO)) return SMLA_ERR_BAD_ARG;
    if (static_cast<long long>(s_q) * h_q > INT_MAX) return SMLA_ERR_BAD_ARG;
    const int n_rows = s_q * h_q;
    smla::smla_delta_kernel<<<(n_rows + 7) / 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(O), reinterpret_cast<const uint4*>(dO), delta, n_rows);
    g_last_launches = 1;
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

int smla_bwd_status(void* workspace, void* stream) {
    if (!workspace) return SMLA_ERR_BAD_ARG;
    int flag = 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&flag, workspace, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return SMLA_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return SMLA_ERR_LAUNCH;
    g_last_device_code = flag;
    if (flag == 0) return SMLA_OK;
    // reported once: the word is cleared so that the workspace can be used again
    if (cudaMemsetAsync(workspace, 0, 4, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) return SMLA_ERR_LAUNCH;
    return SMLA_ERR_DEVICE_TIMEOUT;
}

int smla_bwd_last_device_code(void) { return g_last_device_code; }

int smla_debug_set_wait_limit_cycles(long long cycles) {
    g_wait_limit.store(cycles > 0 ? cycles : smla::kWaitLimitCycles);
    return SMLA_OK;
}

int smla_selftest_wait_timeout(void* workspace, int which, long long limit_cycles, long long* out3, void* stream) {
    if (!workspace || !out3 || which < 0 || which > 2 || limit_cycles <= 0) return SMLA_ERR_BAD_ARG;
    smla::smla_selftest_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<int*>(workspace), out3, which, limit_cycles, 900 + 10 * which);
    g_last_launches = 1;
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

// ---- index inverse (CSR by kv row) -------------------------------------------------------------
namespace {
inline size_t up256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }
struct InvLayout { size_t keys_a, keys_b, vals_tmp, hist, totals, total; };
inline InvLayout inv_layout(int64_t n, const inv::Plan& pl) {
    InvLayout l;
    size_t off = 0;
    l.keys_a = off; off += up256(static_cast<size_t>(n) * 4);
    l.keys_b = off; off += up256(static_cast<size_t>(n) * 4);
    l.vals_tmp = off; off += up256(static_cast<size_t>(n) * 4);
    l.hist = off; off += up256(static_cast<size_t>(inv::kMaxRadix) * pl.n_blocks * 4);
    l.totals = off; off += up256(inv::kMaxRadix * 4);
    l.total = off;
    return l;
}
inline bool inv_shape_ok(int32_t s_q, int32_t topk, int32_t s_kv) {
    return s_q >= 0 && topk > 0 && s_kv > 0 && s_kv < INT32_MAX &&
           static_cast<int64_t>(s_q) * topk <= static_cast<int64_t>(INT32_MAX);
}
}  // namespace

size_t smla_index_inverse_workspace_size(int32_t s_q, int32_t topk, int32_t s_kv) {
    if (!inv_shape_ok(s_q, topk, s_kv)) return 0;
    const int64_t n = static_cast<int64_t>(s_q) * topk;
    return inv_layout(n, inv::make_plan(n, s_kv)).total + 256;
}

int smla_index_inverse(const int32_t* indices, int32_t s_q, int32_t topk, int32_t s_kv, int32_t q_start_index_s,
                       int32_t* row_ptr, int32_t* entries, void* workspace, size_t workspace_bytes, void* stream) {
    if (!inv_shape_ok(s_q, topk, s_kv) || !row_ptr) return SMLA_ERR_BAD_ARG;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t n = static_cast<int64_t>(s_q) * topk;
    g_last_launches = 0;
    if (n == 0) {
        if (cudaMemsetAsync(row_ptr, 0, (static_cast<size_t>(s_kv) + 1) * 4, st) != cudaSuccess) return SMLA_ERR_LAUNCH;
        return SMLA_OK;
    }
    if (!indices || !entries || !workspace) return SMLA_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return SMLA_ERR_BAD_ARG;
    const inv::Plan pl = inv::make_plan(n, s_kv);
    const InvLayout l = inv_layout(n, pl);
    if (workspace_bytes < l.total) return SMLA_ERR_WORKSPACE;
    if (cudaFuncSetAttribute(inv::scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, inv::kScatterDynSmem) !=
        cudaSuccess)
        return SMLA_ERR_LAUNCH;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint32_t* kbuf[2] = {reinterpret_cast<uint32_t*>(ws + l.keys_a), reinterpret_cast<uint32_t*>(ws + l.keys_b)};
    int32_t* vtmp = reinterpret_cast<int32_t*>(ws + l.vals_tmp);
    uint32_t* hist = reinterpret_cast<uint32_t*>(ws + l.hist);
    uint32_t* totals = reinterpret_cast<uint32_t*>(ws + l.totals);
    const uint32_t mask = (1u << pl.digit_bits) - 1u;
    const int radix = 1 << pl.digit_bits;
    const int causal = q_start_index_s != SMLA_NO_CAUSAL;
    int launches = 0;
    const int32_t* vin = nullptr;
    for (int pass = 0; pass < pl.passes; ++pass) {
        const int shift = pass * pl.digit_bits;
        if (pass == 0)
            inv::make_keys_kernel<<<pl.n_blocks, inv::kThreads, 0, st>>>(indices, kbuf[0], hist, n, topk, s_kv, causal,
                                                                         causal ? q_start_index_s : 0, mask, pl.n_blocks);
        else
            inv::histogram_kernel<<<pl.n_blocks, inv::kThreads, 0, st>>>(kbuf[pass & 1], hist, n, shift, mask, pl.n_blocks);
        inv::scan_rows_kernel<<<radix, 1024, 0, st>>>(hist, totals, pl.n_blocks);
        // the last pass must land in `entries`: passes alternate between the temporary and the output
        int32_t* vout = ((pl.passes - 1 - pass) & 1) ? vtmp : entries;
        inv::scatter_kernel<<<pl.n_blocks, inv::kThreads, inv::kScatterDynSmem, st>>>(kbuf[pass & 1], vin, kbuf[(pass + 1) & 1], vout, hist,
                                                                   totals, n, shift, mask, pl.n_blocks);
        vin = vout;
        launches += 3;
    }
    const int rows = s_kv + 1;
    inv::row_ptr_kernel<<<(rows + 255) / 256, 256, 0, st>>>(kbuf[pl.passes & 1], row_ptr, n, s_kv);
    g_last_launches = launches + 1;
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

// ---- sum of the ranks' partial dKV over NVLink (query-sharded runs) ---------------------------------------------
// Rank r owns kv rows [r * rows, (r + 1) * rows).  Every CTA walks a slice of the owned rows, loads the same 16 bytes
// from every rank's partial buffer (its own from HBM, the others' through NVLink with plain loads: no TMA, no
// multicast), adds them in rank order (so the result does not depend on timing) and stores the sum.  With
// `zero_sources` it also writes zeros back over what it has read, in every rank's buffer: each row of every partial
// is read by exactly one rank, its owner, so after all ranks have run the kernel every partial is clear for the next
// step and no separate memset is needed.  The caller orders the kernel between two cross-rank barriers.
namespace {
constexpr int kMaxRanks = 16;
struct PeerPtrs {
    float4* p[kMaxRanks];
};
__global__ void __launch_bounds__(256) pull_reduce_kernel(PeerPtrs peers, int world, int rank, float4* __restrict__ out,
                                                          size_t n4, size_t first4, int zero_sources) {
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < world) v[r] = peers.p[r][first4 + i];
        float4 acc = v[0];
#pragma unroll
        for (int r = 1; r < kMaxRanks; ++r)
            if (r < world) {
                acc.x += v[r].x;
                acc.y += v[r].y;
                acc.z += v[r].z;
                acc.w += v[r].w;
            }
        out[i] = acc;
        if (zero_sources) {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < world) peers.p[r][first4 + i] = zero;
        }
    }
}
// The same sum taken inside the NVSwitch: one multimem.ld_reduce on the multicast mapping of the partial buffers
// returns the sum over all ranks of 16 bytes, so a rank receives only its reduced rows (1/R of what the pull form
// moves), and one multimem.st clears those 16 bytes in every rank's buffer at once.
__global__ void __launch_bounds__(256) multimem_reduce_kernel(float4* __restrict__ mc, float4* __restrict__ out, size_t n4,
                                                              size_t first4, int zero_sources) {
    constexpr int kUnroll = 4;              // independent reductions in flight per thread
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i0 = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < n4; i0 += kUnroll * stride) {
        float4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < n4)
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(v[u].x), "=f"(v[u].y), "=f"(v[u].z), "=f"(v[u].w)
                             : "l"(mc + first4 + i)
                             : "memory");
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = i0 + u * stride;
            if (i < n4) {
                out[i] = v[u];
                if (zero_sources)
                    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc + first4 + i), "f"(0.f),
                                 "f"(0.f), "f"(0.f), "f"(0.f)
                                 : "memory");
            }
        }
    }
}
}  // namespace

int smla_dkv_multimem_reduce(void* multicast_partial, int32_t world, int32_t rank, int32_t s_kv, float* out,
                             int32_t zero_sources, void* stream) {
    if (!multicast_partial || !out || world < 1 || rank < 0 || rank >= world || s_kv <= 0 || s_kv % world) return SMLA_ERR_BAD_ARG;
    if (!aligned16(multicast_partial) || !aligned16(out)) return SMLA_ERR_BAD_ARG;
    const size_t rows = static_cast<size_t>(s_kv) / world;
    const size_t n4 = rows * (SMLA_D_QK / 4);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return SMLA_ERR_LAUNCH;
    size_t blocks = (n4 + 255) / 256;
    const size_t cap = static_cast<size_t>(sms) * 8;
    if (blocks > cap) blocks = cap;
    multimem_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<float4*>(multicast_partial), reinterpret_cast<float4*>(out), n4, static_cast<size_t>(rank) * n4, zero_sources);
    g_last_launches = 1;
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

int smla_dkv_pull_reduce(const void* const* partials, int32_t world, int32_t rank, int32_t s_kv, float* out,
                         int32_t zero_sources, void* stream) {
    if (!partials || !out || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || s_kv <= 0 || s_kv % world)
        return SMLA_ERR_BAD_ARG;
    PeerPtrs pp{};
    for (int r = 0; r < world; ++r) {
        if (!partials[r] || !aligned16(partials[r])) return SMLA_ERR_BAD_ARG;
        pp.p[r] = reinterpret_cast<float4*>(const_cast<void*>(partials[r]));
    }
    if (!aligned16(out)) return SMLA_ERR_BAD_ARG;
    const size_t rows = static_cast<size_t>(s_kv) / world;
    const size_t n4 = rows * (SMLA_D_QK / 4);
    const size_t first4 = static_cast<size_t>(rank) * n4;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return SMLA_ERR_LAUNCH;
    size_t blocks = (n4 + 255) / 256;
    const size_t cap = static_cast<size_t>(sms) * 8;
    if (blocks > cap) blocks = cap;
    pull_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        pp, world, rank, reinterpret_cast<float4*>(out), n4, first4, zero_sources);
    g_last_launches = 1;
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

// ---- SM clock probe ------------------------------------------------------------------------------------------
namespace {
__global__ void clock_probe_kernel(unsigned long long* out, int n_sm) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (static_cast<int>(smid) < n_sm) {
        out[2 * smid] = static_cast<unsigned long long>(clock64());
        out[2 * smid + 1] = t;
    }
}
// fp32 reductions the way the dkv kernel issues them (one red.global.add.f32 per lane, 32 lanes = 128 consecutive bytes)
// on rows picked at random: a warp per row, rows_per_cta rows per block.
__global__ void reduction_rate_probe_kernel(float* dst, uint32_t n_rows, int row_floats, int rows_per_cta) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int r = warp; r < rows_per_cta; r += n_warps) {
        uint32_t h = blockIdx.x * 1315423911u + static_cast<uint32_t>(r) * 2654435761u + 12345u;
        h ^= h >> 16; h *= 0x7feb352du; h ^= h >> 15; h *= 0x846ca68bu; h ^= h >> 16;
        float* g = dst + static_cast<size_t>(h % n_rows) * row_floats;
        for (int v = lane; v < row_floats; v += 32) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(g + v), "f"(1.f) : "memory");
    }
}
}  // namespace

int smla_reduction_rate_probe(float* dst, int32_t n_rows, int32_t row_floats, int32_t rows_per_cta, int32_t n_ctas, void* stream) {
    if (!dst || n_rows <= 0 || row_floats <= 0 || rows_per_cta <= 0 || n_ctas <= 0) return SMLA_ERR_BAD_ARG;
    reduction_rate_probe_kernel<<<n_ctas, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dst, static_cast<uint32_t>(n_rows), row_floats,
                                                                                          rows_per_cta);
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

int smla_clock_probe(unsigned long long* out, int n_sm, void* stream) {
    if (!out || n_sm <= 0) return SMLA_ERR_BAD_ARG;
    clock_probe_kernel<<<4 * n_sm, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, n_sm);
    return cudaGetLastError() == cudaSuccess ? SMLA_OK : SMLA_ERR_LAUNCH;
}

int smla_bwd_last_launch_count(void) { return g_last_launches; }

const char* smla_status_string(int status) {
    switch (status) {
        case SMLA_OK: return "ok";
        case SMLA_ERR_BAD_ARG: return "bad argument (null/misaligned pointer or unsupported shape)";
        case SMLA_ERR_LAUNCH: return "CUDA launch or driver call failed";
        case SMLA_ERR_WORKSPACE: return "workspace too small";
        case SMLA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out; results are invalid";
        case SMLA_ERR_TOO_LARGE_FOR_STATIC:
            return "problem too large for the library's built-in 32 MiB workspace (Delta + one query of S/dS must fit); "
                   "use smla_bwd_run with a caller-provided workspace";
        default: return "unknown status";
    }
}

}  // extern "C"
