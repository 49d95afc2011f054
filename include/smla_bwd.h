/* C ABI of the B200 sparse MLA attention backward.
 *
 * Plain pointers and sizes only; every pointer is a device pointer unless stated.  The
 * library never allocates device memory: the caller passes a workspace whose size it asks
 * for first.  All entry points enqueue on the given CUDA stream and return without a host
 * synchronisation except smla_bwd_status().
 *
 * Replaces, in the reference project MrChen314/test_operator:
 *   - the host launchers `launch_preprocess_delta` and `launch_test_mla_bwd`
 *     (mla_bwd/mla_bwd.cu:802-819, 822-969; prototype mla_bwd/mla_bwd.cuh:284-298), and
 *   - the operator body `mla_bwd_forward` (mla_bwd/mla_bwd.cu:972-1058) apart from tensor
 *     allocation, which stays with the caller.
 */
#ifndef SMLA_BWD_H_
#define SMLA_BWD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMLA_D_QK 576          /* 512 latent + 64 rope (mla_bwd/mla_bwd.cuh:44-47) */
#define SMLA_D_V 512
#define SMLA_NO_CAUSAL INT32_MIN /* q_start_index_s value that switches the causal bound off */

/* status codes */
#define SMLA_OK 0
#define SMLA_ERR_BAD_ARG 1        /* shape / alignment / null pointer (reference: TORCH_CHECKs, mla_bwd.cu:975-1015,1040) */
#define SMLA_ERR_LAUNCH 2         /* a CUDA runtime or driver call failed (reference prints and ignores, mla_bwd.cu:814-818,965-968) */
#define SMLA_ERR_WORKSPACE 3      /* workspace too small */
#define SMLA_ERR_DEVICE_TIMEOUT 4 /* a bounded wait inside a kernel ran out; results are invalid */
#define SMLA_ERR_TOO_LARGE_FOR_STATIC 5 /* smla_bwd_run_noalloc: does not fit the built-in workspace */

/* stages of smla_bwd_run_stages (bit mask) */
#define SMLA_STAGE_ZERO 1      /* clear dKV                           (reference: torch::zeros, mla_bwd.cu:1027) */
#define SMLA_STAGE_DELTA 2     /* Delta = rowsum(O * dO)              (reference: preprocess_delta_kernel, mla_bwd.cu:51-95) */
#define SMLA_STAGE_RECOMPUTE 4 /* S, dS (bf16) from P = QK^T, dP = dO V^T (reference: mla_bwd.cu:225-320, 700-718) */
#define SMLA_STAGE_DKV 8       /* dKV += S^T dO + dS^T Q, scattered by index (reference: mla_bwd.cu:493-618, 720-753) */
#define SMLA_STAGE_DQ 16       /* dQ = dS K_gathered                  (reference: mla_bwd.cu:322-404, 729-737) */
#define SMLA_STAGE_ALL 31

typedef struct smla_bwd_params {
    /* inputs, all contiguous (reference tensor contract: mla_bwd/mla_bwd.cu:975-1015) */
    const void* q;          /* bf16 [s_q, h_q, 576] */
    const void* kv;         /* bf16 [s_kv, 576] */
    const void* dO;         /* bf16 [s_q, h_q, 512] */
    const float* lse;       /* f32  [s_q, h_q]  log-sum-exp of the scaled logits */
    const void* O;          /* bf16 [s_q, h_q, 512] */
    const int32_t* indices; /* i32  [s_q, topk]; a value outside [0, s_kv) marks an unused slot */
    /* outputs */
    void* dQ;               /* bf16 [s_q, h_q, 576], fully overwritten */
    float* dKV;             /* f32  [s_kv, 576], accumulated into; cleared first when SMLA_STAGE_ZERO runs */
    int32_t s_q, s_kv, h_q, topk;
    float sm_scale;          /* <= 0 selects 1/sqrt(576) (reference: mla_bwd/test_mla_bwd.py:38) */
    int32_t q_start_index_s; /* slot valid only if idx <= q_start_index_s + query row (reference uses 0,
                                mla_bwd.cu:122,772); SMLA_NO_CAUSAL disables the bound */
    int32_t lse_is_base2;    /* 1: lse in base-2 units as the reference operator expects (mla_bwd.cu:262-270); 0: natural log */
    /* Optional (null: one sequence, every slot in use): i32 [s_q][4], 16-byte aligned, per query
     *   {first kv row of the query's sequence, kv rows of that sequence, position for the causal rule, top-k slots in use}.
     * Index values are then relative to the sequence's first row and valid in [0, rows of the sequence); slot j of a
     * query takes part only if j < slots in use; with the causal rule on, only if idx <= position (q_start_index_s
     * then only switches the rule on or off).  s_kv stays the total number of kv / dKV rows.  This is how packed
     * (variable-length) and batched inputs run as one launch chain; the fields follow the per-query ones of the
     * reference's richer parameter block (dq_test/dq_phase_capture.cuh:107-109). */
    const int32_t* query_meta;
} smla_bwd_params;

/* Workspace (device memory) needed for `p`, never more than about `budget_bytes` when that is
 * non-zero (the query dimension is then processed in several passes).  0 on bad arguments. */
size_t smla_bwd_workspace_size(const smla_bwd_params* p, size_t budget_bytes);

/* Whole backward: clear dKV, Delta, recompute, dKV, dQ.  `stream` is a cudaStream_t. */
int smla_bwd_run(const smla_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Same with a stage mask (SMLA_STAGE_*): lets a caller skip the clear (to accumulate partial
 * dKV over several calls) and lets tests and profilers run one kernel at a time. */
int smla_bwd_run_stages(const smla_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream,
                        int stage_mask);

/* Whole backward with a REPRODUCIBLE dKV: the same inputs give the same bits in every run.  (No counterpart in the
 * reference, whose scatter is an order-dependent reduce-add as well: mla_bwd/mla_bwd.cu:23-26,527-537.)
 * The regular entry points add every slot's contribution into dKV with fp32 reductions, whose order - and so the
 * rounding of a row's sum - differs from run to run (dQ is reproducible either way).  Here the dKV kernel writes every
 * slot's [576] fp32 contribution to the slot's own row of `staging`, and a second kernel walks the index inverse of the
 * sparse pattern (smla_index_inverse: CSR by kv row, flat slot ids ascending) and adds a kv row's slots in that order.
 * Costs one extra write and read of 2304 bytes per slot (about 39 GB on the 4096-query x top-k 2048 workload).
 *   row_ptr / entries: what smla_index_inverse returned for the same indices, s_kv and q_start_index_s;
 *   staging: device memory, 16-byte aligned; a pass over the queries holds staging_bytes /
 *            smla_bwd_staging_bytes_per_query(p) queries (at least one must fit), so a small buffer means more passes;
 *   stage_mask as in smla_bwd_run_stages; without SMLA_STAGE_ZERO the sums are added to what dKV holds.
 * query_meta must be null (one sequence).  Runs the kernels one after the other on `stream`. */
typedef struct smla_bwd_det_params {
    const int32_t* row_ptr; /* [s_kv + 1] */
    const int32_t* entries; /* [s_q * topk] */
    float* staging;
    size_t staging_bytes;
} smla_bwd_det_params;
int smla_bwd_run_deterministic(const smla_bwd_params* p, const smla_bwd_det_params* det, void* workspace,
                               size_t workspace_bytes, void* stream, int stage_mask);
size_t smla_bwd_staging_bytes_per_query(const smla_bwd_params* p);

/* Whole backward for callers that must not allocate device memory.  (No counterpart in the reference, whose
 * operator allocates delta, dQ and dKV itself on every call.)
 *
 * Who needs it: host code that runs where a cudaMalloc is off limits -- a plugin inside a process whose
 * framework has already reserved the GPU's memory for its own pool (a raw allocation there fails or
 * fragments the pool), or a latency-bound loop that cannot take the device-wide synchronisation an
 * allocation or free may imply.  Such a caller still owns q, kv, dO, lse, O, indices, dQ and dKV; what it cannot
 * provide is the scratch for Delta and the bf16 S / dS.  This entry point takes that scratch from a
 * 32 MiB array compiled into the library (smla_bwd_noalloc_capacity()), resident on every GPU that loads
 * the library until the process exits.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 * Limits and rules:
 *  - 256 + 4*s_q*h_q bytes of Delta plus the S/dS of at least one query (4 * topk_pad * h_pad bytes, topk
 *    rounded up to 256, heads to 64 or 128) must fit in the 32 MiB; otherwise SMLA_ERR_TOO_LARGE_FOR_STATIC.
 *    Larger s_q simply takes more passes over the query dimension (about 31 queries per pass at
 *    h_q 128 / topk 2048), so this path trades speed for not allocating.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 *    device current) and caches it; make that first call before any stream capture begins.
 *  - All calls on a device share the one array.  It keeps whatever the previous call left; every byte that
 *    is read is rewritten first (Delta and the S/dS rows of a pass are fully overwritten before use; the
 *    error word starts at zero with the library image and is cleared again when a timeout has been reported).  Two calls whose kernels overlap on the GPU (different streams, or threads)
 *    race on it: serialise them.
 *  - Status of the last call: smla_bwd_noalloc_status(stream) (synchronises the stream). */
int smla_bwd_run_noalloc(const smla_bwd_params* p, void* stream);
size_t smla_bwd_noalloc_capacity(void);
int smla_bwd_noalloc_status(void* stream);

/* ---- forward (the step before this path) ---------------------------------------------------------------
 * o = softmax(scale * q K_g^T) V_g and the log-sum-exp the backward consumes, for the same top-k indices.
 * The reference has no forward kernel; its tests build o / lse with fp32 torch code
 * (dq_test/test_dq_phase.py:53-59), which is what this entry point reproduces on the GPU. */
typedef struct smla_fwd_params {
    const void* q;          /* bf16 [s_q, h_q, 576] */
    const void* kv;         /* bf16 [s_kv, 576] */
    const int32_t* indices; /* i32  [s_q, topk] */
    void* o;                /* bf16 [s_q, h_q, 512], fully overwritten (0 for a query without a valid slot) */
    float* lse;             /* f32  [s_q, h_q] (+inf for a query without a valid slot) */
    int32_t s_q, s_kv, h_q, topk;
    float sm_scale;          /* <= 0 selects 1/sqrt(576) */
    int32_t q_start_index_s; /* as in smla_bwd_params */
    int32_t lse_is_base2;    /* 1: write lse in base-2 units (what smla_bwd_run expects by default); 0: natural log */
    const int32_t* query_meta; /* as in smla_bwd_params */
} smla_fwd_params;
size_t smla_fwd_workspace_size(const smla_fwd_params* p, size_t budget_bytes);
int smla_fwd_run(const smla_fwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Delta only: delta[s_q, h_q] = sum_j O[.., j] * dO[.., j]   (reference: launch_preprocess_delta). */
int smla_bwd_delta(const void* O, const void* dO, float* delta, int32_t s_q, int32_t h_q, void* stream);

/* Where the pieces of the workspace live, for stage-by-stage checks.  Offsets in bytes. */
typedef struct smla_bwd_workspace_layout {
    size_t err_offset;    /* int32 device error word */
    size_t delta_offset;  /* f32 [s_q, h_q] */
    size_t s_offset;      /* bf16 [q_chunk, h_pad/8, topk_pad, 8]  S  of the LAST query chunk processed; per query: */
    size_t ds_offset;     /* bf16 [q_chunk, h_pad/8, topk_pad, 8]  dS    block of 8 heads, key, head in block      */
    int32_t q_chunk, topk_pad, h_pad;
    size_t total_bytes;
} smla_bwd_workspace_layout;
int smla_bwd_get_workspace_layout(const smla_bwd_params* p, size_t workspace_bytes, smla_bwd_workspace_layout* out);

/* Index inverse of the sparse pattern (a reusable pre-pass; the reference has no such operator, its validity rule
 * is the one of mla_bwd/mla_bwd.cu:765-789): CSR by kv row of the valid slots.
 *   row_ptr [s_kv + 1] i32: entries[row_ptr[r] .. row_ptr[r+1]) are the slots that chose kv row r;
 *   entries [s_q * topk] i32: flat slot ids q * topk + slot, ascending inside a row (a fixed order: the result is
 *     reproducible bit for bit); behind row_ptr[s_kv] follow the unused slots in ascending flat order.
 * s_q * topk must fit in 31 bits.  q_start_index_s has the meaning it has in the backward's parameter block; SMLA_NO_CAUSAL: no causal bound.
 * `workspace`: device memory, 256-byte aligned, at least smla_index_inverse_workspace_size() bytes (0 = bad shape). */
size_t smla_index_inverse_workspace_size(int32_t s_q, int32_t topk, int32_t s_kv);
int smla_index_inverse(const int32_t* indices, int32_t s_q, int32_t topk, int32_t s_kv, int32_t q_start_index_s,
                       int32_t* row_ptr, int32_t* entries, void* workspace, size_t workspace_bytes, void* stream);

/* The first 256 bytes of a workspace hold the device error word.  Clear them once before the workspace's first
 * use (this call, or any memset); the run entry points do not, so that a timeout recorded by any call of a
 * sequence is still there when the status is read. */
int smla_bwd_workspace_init(void* workspace, void* stream);

/* Synchronises `stream`, reads the device error word in the workspace and returns SMLA_OK or
 * SMLA_ERR_DEVICE_TIMEOUT (or SMLA_ERR_LAUNCH if the stream reports a CUDA error).  A recorded timeout is
 * reported once: the word is cleared on the way out.  The reference swallows device-side failures
 * (mla_bwd/mla_bwd.cu:814-818,965-968); this is the replacement. */
int smla_bwd_status(void* workspace, void* stream);
/* The raw word the last smla_bwd_status on this thread read: 0, or 100 * kernel + the site of the wait that gave up. */
int smla_bwd_last_device_code(void);

/* How one pass of the backward is scheduled.  chunks = 0: the kernels one after another on the caller's stream.
 * chunks >= 2: the queries of a pass are cut into that many parts and the dKV kernel of a part runs on a second
 * stream owned by the library, on `dkv_pairs` 2-SM clusters (0: chosen by the library from the head count), beside
 * the recompute and dQ kernels of the next part: the dKV kernel keeps the load/store path busy and the tensor cores
 * a third of the time, the other two the reverse.  chunks = -1 (the default): chosen by the library from the head
 * count - two overlapped parts up to 64 heads, one after another with 128, which is what measured faster on B200.
 * A pass falls back to one-after-the-other when it has too few queries to keep every cluster busy in every part.
 * The second stream and its events are created by the first call that needs them on a device: make that call before a
 * stream capture begins.  Process-wide; the environment variable SMLA_SCHEDULE="chunks,dkv_pairs" sets the initial
 * value.  smla_bwd_get_schedule returns what was set (-1 for automatic), not what a head count resolves to. */
int smla_bwd_set_schedule(int chunks, int dkv_pairs);
void smla_bwd_get_schedule(int* chunks, int* dkv_pairs);

/* Test hooks for the bounded waits inside the kernels (every wait on a barrier or a flag gives up after a limit,
 * records a code and lets the kernel return).  smla_debug_set_wait_limit_cycles changes the limit for later
 * launches (<= 0 restores the default of about a second).  smla_selftest_wait_timeout launches a one-warp kernel
 * that waits, with the given limit, on something nothing ever signals (which = 0: sleeping barrier wait, 1:
 * spinning barrier wait, 2: counter wait) and writes {first wait returned, second wait returned, cycles waited}
 * to out3 (device memory, 3 x int64); the code 900 + 10 * which lands in the workspace's error word. */
int smla_debug_set_wait_limit_cycles(long long cycles);
int smla_selftest_wait_timeout(void* workspace, int which, long long limit_cycles, long long* out3, void* stream);

/* Query-sharded runs (one long sequence, queries split over `world` GPUs of one node, every rank holding a full-size
 * fp32 partial dKV): sum the partials' rows [rank * s_kv / world, (rank + 1) * s_kv / world) into `out`
 * ([s_kv / world, 576] fp32, this GPU's memory).  `partials[r]` is rank r's partial buffer as mapped into THIS process
 * (its own for r == rank, peer mappings otherwise; `partials` itself is a host array).  The kernel reads peers with
 * plain loads over NVLink and adds in rank order.  With zero_sources != 0 it clears what it has read, in every
 * rank's buffer, so that after all ranks have run it every partial is zero for the next step.  The caller must order
 * it between two cross-rank barriers on the stream (all partials complete before; nobody reuses a partial before
 * everyone has finished).  No counterpart in the reference, which has no multi-GPU code; it stands in for
 * ncclReduceScatter on this path. */
int smla_dkv_pull_reduce(const void* const* partials, int32_t world, int32_t rank, int32_t s_kv, float* out,
                         int32_t zero_sources, void* stream);

/* The same sum taken inside the NVSwitch, for buffers that also have a multicast (NVLS) mapping: `multicast_partial`
 * is the multicast address of the partial buffers (what torch's symmetric memory calls multicast_ptr, offset to the
 * buffer).  One multimem.ld_reduce returns the sum over all ranks, so a rank receives only its own reduced rows, and
 * with zero_sources != 0 one multimem.st clears them in every rank's buffer.  Same barrier rules as above. */
int smla_dkv_multimem_reduce(void* multicast_partial, int32_t world, int32_t rank, int32_t s_kv, float* out,
                             int32_t zero_sources, void* stream);

/* Measurement aid: every SM that gets a block writes {its cycle counter, the global nanosecond timer} to
 * out[2 * smid], out[2 * smid + 1] (device memory, 2 * n_sm x u64; SMs that got none keep what was there).  Two probes
 * around a timed region give the average SM clock inside it: delta cycles / delta ns per SM. */
int smla_clock_probe(unsigned long long* out, int n_sm, void* stream);

/* Measurement aid (no counterpart in the reference): n_ctas blocks of 256 threads add 1.0f to every element of
 * rows_per_cta rows each, picked at random among dst's n_rows rows of row_floats floats, with the instruction form the
 * dKV scatter uses (red.global.add.f32, a warp per row, 128 consecutive bytes per instruction).  Timed by the caller,
 * n_ctas * rows_per_cta * row_floats * 4 bytes / time is the rate at which this GPU takes fp32 reductions: the ceiling
 * the dKV kernel is measured against. */
int smla_reduction_rate_probe(float* dst, int32_t n_rows, int32_t row_floats, int32_t rows_per_cta, int32_t n_ctas, void* stream);

/* Number of kernels (own kernels, memset excluded) the last smla_bwd_run_stages on this thread launched. */
int smla_bwd_last_launch_count(void);

const char* smla_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* SMLA_BWD_H_ */
