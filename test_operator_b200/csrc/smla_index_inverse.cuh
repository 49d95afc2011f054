// Index inverse of the sparse attention pattern: from indices [s_q, topk] (kv row chosen by each slot of each
// query) to a CSR by kv row -- row_ptr [s_kv + 1] and entries [s_q * topk], where the entries of a row are the flat
// slot ids q * topk + slot of the valid slots that chose it, in ascending order.  The order is fixed (not the
// arrival order of atomics), so the result is reproducible bit for bit.
//
// Method: a stable least-significant-digit radix sort of (key = kv row, value = flat slot id).  The values start in
// ascending order, so a stable sort by key alone yields (row, flat id) order.  Unused slots get the key s_kv and end
// up behind row_ptr[s_kv] in flat order.  Per pass three kernels: digit histogram per block, exclusive scan of the
// [digit][block] matrix, stable scatter.  All of it is integer work bound by HBM: 4 B read + 4 B written per slot
// to form the keys, then 8 B read + 8 B written per slot and pass.
//
// The reference has no such operator; the validity rule is the one of its kernel (mla_bwd/mla_bwd.cu:765-789).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace inv {

constexpr int kThreads = 512;
constexpr int kItems = 16;                       // entries per thread
constexpr int kBlockItems = kThreads * kItems;   // entries per block, contiguous
constexpr int kWarps = kThreads / 32;
constexpr int kMaxRadix = 256;

struct Plan {
    int passes;      // 1..4
    int digit_bits;  // <= 8
    int n_blocks;
};

inline Plan make_plan(int64_t n, int32_t s_kv) {
    int bits = 1;
    while ((static_cast<int64_t>(1) << bits) <= static_cast<int64_t>(s_kv)) ++bits;   // keys are 0..s_kv inclusive
    Plan pl;
    pl.passes = (bits + 7) / 8;
    pl.digit_bits = (bits + pl.passes - 1) / pl.passes;
    pl.n_blocks = static_cast<int>((n + kBlockItems - 1) / kBlockItems);
    return pl;
}

__device__ __forceinline__ uint32_t digit_of(uint32_t key, int shift, uint32_t mask) { return (key >> shift) & mask; }

// keys[i] = kv row of flat slot i, or s_kv for an unused slot; also the first pass's digit histogram.
__global__ void __launch_bounds__(kThreads)
make_keys_kernel(const int32_t* __restrict__ indices, uint32_t* __restrict__ keys, uint32_t* __restrict__ hist,
                 int64_t n, int32_t topk, int32_t s_kv, int32_t causal, int32_t q_start, uint32_t mask, int n_blocks) {
    __shared__ uint32_t h[kMaxRadix];
    for (int i = threadIdx.x; i <= static_cast<int>(mask); i += kThreads) h[i] = 0;
    __syncthreads();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kBlockItems;
#pragma unroll 4
    for (int t = 0; t < kItems; ++t) {
        const int64_t i = base + static_cast<int64_t>(t) * kThreads + threadIdx.x;
        if (i < n) {
            const int idx = indices[i];
            const int q = static_cast<int>(i / topk);
            const bool valid = idx >= 0 && idx < s_kv && (!causal || idx <= q_start + q);
            const uint32_t key = valid ? static_cast<uint32_t>(idx) : static_cast<uint32_t>(s_kv);
            keys[i] = key;
            atomicAdd(&h[key & mask], 1u);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= static_cast<int>(mask); i += kThreads) hist[static_cast<size_t>(i) * n_blocks + blockIdx.x] = h[i];
}

__global__ void __launch_bounds__(kThreads)
histogram_kernel(const uint32_t* __restrict__ keys, uint32_t* __restrict__ hist, int64_t n, int shift, uint32_t mask,
                 int n_blocks) {
    __shared__ uint32_t h[kMaxRadix];
    for (int i = threadIdx.x; i <= static_cast<int>(mask); i += kThreads) h[i] = 0;
    __syncthreads();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kBlockItems;
#pragma unroll 4
    for (int t = 0; t < kItems; ++t) {
        const int64_t i = base + static_cast<int64_t>(t) * kThreads + threadIdx.x;
        if (i < n) atomicAdd(&h[digit_of(keys[i], shift, mask)], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= static_cast<int>(mask); i += kThreads) hist[static_cast<size_t>(i) * n_blocks + blockIdx.x] = h[i];
}

// Block-wide exclusive scan of one value per thread (blockDim.x a multiple of 32, at most 1024); returns the
// exclusive prefix and leaves the block total in *total_out (shared).  `warp_sums` holds 32 words.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_sums, uint32_t* total_out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const uint32_t w = lane < n_warps ? warp_sums[lane] : 0u;
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += up;
        }
        warp_sums[lane] = wi - w;
        if (lane == 31) *total_out = wi;
    }
    __syncthreads();
    const uint32_t r = warp_sums[warp] + incl - v;
    __syncthreads();   // warp_sums may be reused by the caller's next call
    return r;
}

// One block per digit: hist[digit][0..n_blocks) becomes its exclusive prefix over the blocks; the digit's total goes
// to totals[digit].  The scatter kernel adds the prefix over the digits itself (at most 256 values).
__global__ void __launch_bounds__(1024)
scan_rows_kernel(uint32_t* __restrict__ hist, uint32_t* __restrict__ totals, int n_blocks) {
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t tile_total;
    uint32_t* row = hist + static_cast<size_t>(blockIdx.x) * n_blocks;
    uint32_t carry = 0;
    for (int base = 0; base < n_blocks; base += 1024) {
        const int i = base + threadIdx.x;
        const uint32_t v = i < n_blocks ? row[i] : 0u;
        const uint32_t ex = block_exclusive_scan(v, warp_sums, &tile_total);
        if (i < n_blocks) row[i] = carry + ex;
        carry += tile_total;
        __syncthreads();
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}

// Stable scatter of one pass.  Warp w of a block owns the contiguous entries [w * kWarpItems, (w + 1) * kWarpItems)
// of the block's range, so (warp, step, lane) order is flat order.
//   1. every warp counts the digits of its entries (private shared-memory counters);
//   2. the counts are prefixed over the warps and over the digits: block-local position of every (digit, warp) run;
//   3. every warp places its entries, step by step, into a shared-memory copy of the block's output in digit order
//      (position = running base of (warp, digit) + rank among the lanes of the step with the same digit);
//   4. the staged entries go out in that order: entry j of digit d lands at global base of (d, block) + j - local
//      base of d, so consecutive threads write consecutive addresses inside a digit's run (about kBlockItems / radix
//      entries) instead of 32 different lines per warp instruction.
// vals_in == nullptr means the values are the flat positions themselves (first pass).
constexpr int kScatterDynSmem = kBlockItems * 8;   // staged keys + values

// Lanes of the warp whose digit (below 256) equals this lane's, among the active lanes.  Eight ballots: the
// `match.any` instruction gives the same mask but runs on a pipe that takes a warp every ~64 cycles per SM, which
// bounded the whole sort (70 % pipe utilisation under ncu) when it was used.
__device__ __forceinline__ uint32_t same_digit_lanes(uint32_t d, bool active) {
    uint32_t peers = __ballot_sync(0xffffffffu, active);
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        const bool bit = (d >> b) & 1u;
        const uint32_t m = __ballot_sync(0xffffffffu, bit);
        peers &= bit ? m : ~m;
    }
    return peers;
}

__global__ void __launch_bounds__(kThreads, 2)
scatter_kernel(const uint32_t* __restrict__ keys_in, const int32_t* __restrict__ vals_in,
               uint32_t* __restrict__ keys_out, int32_t* __restrict__ vals_out, const uint32_t* __restrict__ hist,
               const uint32_t* __restrict__ totals, int64_t n, int shift, uint32_t mask, int n_blocks) {
    constexpr int kWarpItems = kBlockItems / kWarps;   // 512
    constexpr int kSteps = kWarpItems / 32;            // 16
    extern __shared__ __align__(16) uint32_t staged[];
    uint32_t* skeys = staged;
    int32_t* svals = reinterpret_cast<int32_t*>(staged + kBlockItems);
    __shared__ uint32_t global_base[kMaxRadix];   // first output position of (digit, this block)
    __shared__ uint32_t local_base[kMaxRadix];    // first staged position of the digit
    __shared__ uint32_t warp_count[kWarps][kMaxRadix];
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t total;
    const int radix = static_cast<int>(mask) + 1;
    for (int i = threadIdx.x; i < kWarps * kMaxRadix; i += kThreads) (&warp_count[0][0])[i] = 0;
    {
        // exclusive prefix of the digit totals (radix <= 256 <= kThreads: one value per thread)
        const uint32_t t = threadIdx.x < radix ? totals[threadIdx.x] : 0u;
        const uint32_t ex = block_exclusive_scan(t, warp_sums, &total);
        if (threadIdx.x < radix) global_base[threadIdx.x] = ex + hist[static_cast<size_t>(threadIdx.x) * n_blocks + blockIdx.x];
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lanes_below = (1u << lane) - 1u;
    const int64_t block0 = static_cast<int64_t>(blockIdx.x) * kBlockItems;
    const int64_t first = block0 + static_cast<int64_t>(warp) * kWarpItems + lane;
    uint32_t* mine = warp_count[warp];
#pragma unroll
    for (int t = 0; t < kSteps; ++t) {
        const int64_t i = first + t * 32;
        const bool active = i < n;
        if (active) atomicAdd(&mine[digit_of(keys_in[i], shift, mask)], 1u);   // counts only: order does not matter
    }
    __syncthreads();
    {
        // per digit: counts of the warps -> offsets inside the digit's run; the run lengths -> local bases
        uint32_t run = 0;
        if (threadIdx.x < radix) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const uint32_t c = warp_count[w][threadIdx.x];
                warp_count[w][threadIdx.x] = run;
                run += c;
            }
        }
        const uint32_t lb = block_exclusive_scan(run, warp_sums, &total);
        if (threadIdx.x < radix) {
            local_base[threadIdx.x] = lb;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) warp_count[w][threadIdx.x] += lb;
        }
    }
    __syncthreads();
    // second read of the warp's 2 KB of keys (L1 / L2), all of it in flight before the dependent ranking starts
    uint32_t keys[kSteps];
    int32_t vals[kSteps];
#pragma unroll
    for (int t = 0; t < kSteps; ++t) {
        const int64_t i = first + t * 32;
        keys[t] = i < n ? keys_in[i] : 0u;
        vals[t] = (vals_in && i < n) ? vals_in[i] : static_cast<int32_t>(i);
    }
#pragma unroll
    for (int t = 0; t < kSteps; ++t) {
        const int64_t i = first + t * 32;
        const bool active = i < n;
        const uint32_t key = keys[t];
        const uint32_t d = active ? digit_of(key, shift, mask) : 0u;
        const uint32_t peers = same_digit_lanes(d, active);
        const uint32_t rank = __popc(peers & lanes_below);
        uint32_t pos = 0;
        if (active) pos = mine[d] + rank;
        __syncwarp();
        if (active && rank == 0) mine[d] += __popc(peers);
        __syncwarp();
        if (active) {
            skeys[pos] = key;
            svals[pos] = vals[t];
        }
    }
    __syncthreads();
    const int64_t left = n - block0;
    const int count = left < kBlockItems ? static_cast<int>(left) : kBlockItems;
#pragma unroll 4
    for (int j = threadIdx.x; j < count; j += kThreads) {
        const uint32_t key = skeys[j];
        const uint32_t d = digit_of(key, shift, mask);
        const uint32_t pos = global_base[d] + (static_cast<uint32_t>(j) - local_base[d]);
        keys_out[pos] = key;
        vals_out[pos] = svals[j];
    }
}

// row_ptr[r] = number of sorted keys below r = first position whose key is >= r, for r in [0, s_kv].
__global__ void row_ptr_kernel(const uint32_t* __restrict__ sorted_keys, int32_t* __restrict__ row_ptr, int64_t n,
                               int32_t s_kv) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r > s_kv) return;
    int64_t lo = 0, hi = n;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (sorted_keys[mid] < static_cast<uint32_t>(r)) lo = mid + 1; else hi = mid;
    }
    row_ptr[r] = static_cast<int32_t>(lo);
}

}  // namespace inv
