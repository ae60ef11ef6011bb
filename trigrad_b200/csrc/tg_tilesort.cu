// Per-tile sort of the (depth, triangle) entries: the segmented counterpart of the device-wide radix
// sort.  The reference sorts (tile << 32 | depth) keys with a stable device-wide sort
// (cub::DeviceSegmentedSort::StableSortPairs, render.cu:272-284); because every triangle occurs at most once per tile and entries are emitted in
// triangle order, sorting each tile's segment by (depth, triangle) gives the same permutation.
//
// Entries are uint64 words (ordered depth << 32 | triangle), already grouped by tile:
// tile t owns entries[offsets[t] .. offsets[t+1]).
//   n <= 128     one warp per tile, rank sort: every element counts the smaller ones (no exchange steps)
//   n <= 1024    a CTA of 128 threads per tile (work list): bitonic network in shared memory, 8 words per
//                thread kept in registers between trips to shared memory
//   n <= 16384   the same network in 136 KB of shared memory, 1024 threads with 8 or 16 words each;
//                tiles taken from a work list
//   beyond       the same CTA sorts 16384-entry chunks in shared memory and runs the network's wide
//                steps on the segment in global memory
// No kernel here waits on another CTA.
#include <atomic>

#include "tg_radix.cuh"

namespace tg {

constexpr int kTileSortWarps = 4;                      // tiles per CTA of the short kernel
constexpr int kTileSortThreads = 32 * kTileSortWarps;
constexpr int kTileSortRank = 128;
constexpr int kTileSortShort = 1024;
constexpr int kTileSortLongThreads = 1024;
constexpr int kTileSortChunk = 16384;

// Pair q of a step with stride j: the lower index, i.e. q with a zero bit inserted at position log2(j).
__device__ __forceinline__ uint32_t pair_low(uint32_t q, uint32_t j) { return ((q & ~(j - 1)) << 1) | (q & (j - 1)); }

// ---- register-blocked bitonic network -----------------------------------------------------------------
// The array of P = 1 << logP words lives in shared memory.  P >> LOGE threads take part; each keeps
// E = 1 << LOGE words in registers per round - the words whose indices differ only in LOGE chosen
// bits [LO, LO + LOGE) - and so runs up to LOGE steps of the network between two trips to shared memory.
// One spare word after every E keeps the rounds free of bank conflicts: for a fixed register slot the
// sixteen lanes of a half-warp then fall on sixteen different 8-byte banks whatever LO is.
// Every thread of the CTA must call (barriers inside).
template <int LOGE>
__device__ __forceinline__ int padded(int i) { return i + (i >> LOGE); }
constexpr int kMidSmemWords = kTileSortShort + (kTileSortShort >> 3);
constexpr int kLongSmemWords = kTileSortChunk + (kTileSortChunk >> 3);   // covers 8192 + 8192/8 and 16384 + 16384/16

template <int E>
__device__ __forceinline__ void exchange_in_registers(uint64_t (&v)[E], int bit, int r, bool desc) {
    const uint64_t x = v[r], y = v[r | (1 << bit)];
    const bool sw = (x > y) != desc;
    v[r] = sw ? y : x;
    v[r | (1 << bit)] = sw ? x : y;
}

// One round: index bits [LO, LO + LOGE) in registers, steps for the NB highest... lowest of them
// (NB == LOGE except in the last round of a phase, where LO == 0 and only bits NB-1 .. 0 remain).
// LO and NB are compile-time so that all shared-memory offsets are immediates.
template <int LOGE, int LO, int NB>
__device__ __forceinline__ void blocked_round(uint64_t* s, int tid, bool desc) {
    constexpr int E = 1 << LOGE;
    const int base = ((tid >> LO) << (LO + LOGE)) | (tid & ((1 << LO) - 1));
    // base has zero bits in [LO, LO + LOGE): padded(base + (r << LO)) = padded(base) + (r << LO) + ((r << LO) >> LOGE)
    uint64_t* p = s + padded<LOGE>(base);
    uint64_t v[E];
#pragma unroll
    for (int r = 0; r < E; r++) v[r] = p[(r << LO) + ((r << LO) >> LOGE)];
#pragma unroll
    for (int bit = NB - 1; bit >= 0; bit--) {
#pragma unroll
        for (int r = 0; r < E; r++) {
            if (r & (1 << bit)) continue;
            exchange_in_registers<E>(v, bit, r, desc);
        }
    }
#pragma unroll
    for (int r = 0; r < E; r++) p[(r << LO) + ((r << LO) >> LOGE)] = v[r];
}

template <int LOGE, int LO>
__device__ __forceinline__ void blocked_round_lo(uint64_t* s, int tid, int lo, bool desc) {
    if constexpr (LO > 14 - LOGE) {
        return;                               // logP <= 14: no round starts higher
    } else {
        if (lo == LO) blocked_round<LOGE, LO, LOGE>(s, tid, desc);
        else blocked_round_lo<LOGE, LO + 1>(s, tid, lo, desc);
    }
}

template <int LOGE, int NB>
__device__ __forceinline__ void blocked_round_last(uint64_t* s, int tid, int nb, bool desc) {
    if constexpr (NB > LOGE) {
        return;
    } else {
        if (nb == NB) blocked_round<LOGE, 0, NB>(s, tid, desc);
        else blocked_round_last<LOGE, NB + 1>(s, tid, nb, desc);
    }
}

// Steps for index bits b_top .. 0 of the phase that merges runs of 1 << kb words (kb > LOGE).  Direction
// of a pair: ascending where bit kb of the index is clear (classic bitonic sort), always ascending with
// all_asc (the merge tail of the all-ascending network used on segments that span several chunks).
template <int LOGE>
__device__ __forceinline__ void blocked_steps(uint64_t* s, int tid, int logP, int kb, int b_top, bool all_asc) {
    const bool active = tid < (1 << (logP - LOGE));
    int b = b_top;
    while (b >= 0) {
        const int lo = (b - LOGE + 1 > 0) ? b - LOGE + 1 : 0;
        if (active) {
            // bit kb lies above the bits held in registers: one direction per thread and round
            const int base = ((tid >> lo) << (lo + LOGE)) | (tid & ((1 << lo) - 1));
            const bool desc = !all_asc && ((base >> kb) & 1);
            if (lo > 0) blocked_round_lo<LOGE, 1>(s, tid, lo, desc);
            else blocked_round_last<LOGE, 1>(s, tid, b + 1, desc);
        }
        __syncthreads();
        b = lo - 1;
    }
}

// Whole ascending sort of the padded array of 1 << logP words (data in place, barrier passed),
// LOGE <= logP <= 14.
template <int LOGE>
__device__ __forceinline__ void blocked_sort(uint64_t* s, int tid, int logP) {
    constexpr int E = 1 << LOGE;
    if (tid < (1 << (logP - LOGE))) {   // phases 1 .. LOGE touch only the thread's own E consecutive words: one trip
        const int base = tid << LOGE;
        uint64_t* p = s + padded<LOGE>(base);
        uint64_t v[E];
#pragma unroll
        for (int r = 0; r < E; r++) v[r] = p[r];
#pragma unroll
        for (int kb = 1; kb <= LOGE; kb++) {
#pragma unroll
            for (int bit = kb - 1; bit >= 0; bit--) {
#pragma unroll
                for (int r = 0; r < E; r++) {
                    if (r & (1 << bit)) continue;
                    exchange_in_registers<E>(v, bit, r, ((base + r) >> kb) & 1);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < E; r++) p[r] = v[r];
    }
    __syncthreads();
    for (int kb = LOGE + 1; kb <= logP; kb++) blocked_steps<LOGE>(s, tid, logP, kb, kb - 1, false);
}

// Loads seg[0..n) (padding with the largest word up to 1 << logP), sorts, hands the result out.
template <int LOGE, int NT>
__device__ __forceinline__ void sort_segment_in_smem(uint64_t* s, uint64_t* seg, uint32_t n, int logP, int32_t* ids_out,
                                                     bool write_back, int tid) {
    for (int i = tid; i < (1 << logP); i += NT) s[padded<LOGE>(i)] = ((uint32_t)i < n) ? seg[i] : ~0ull;
    __syncthreads();
    blocked_sort<LOGE>(s, tid, logP);
    for (uint32_t i = tid; i < n; i += NT) {
        const uint64_t x = s[padded<LOGE>((int)i)];
        if (ids_out) ids_out[i] = (int32_t)(uint32_t)x;
        if (write_back) seg[i] = x;
    }
    __syncthreads();
}

__device__ __forceinline__ int log2_at_least(uint32_t n) {
    int b = 0;
    while ((1u << b) < n) b++;
    return b;
}

// Work lists in the sort's scratch: [0] long tiles, [1] next long item to hand out in the first round,
// [2] mid tiles, [3] next mid item, [4] next long item of the second round, [5] unused (all zero before
// tile_sort_kernel), then `tiles` slots of long items and `tiles` slots of mid items.
constexpr int kListHead = 6;
__device__ __forceinline__ uint32_t* long_items(uint32_t* lists) { return lists + kListHead; }
__device__ __forceinline__ uint32_t* mid_items(uint32_t* lists, int tiles) { return lists + kListHead + tiles; }

// Rank sort of n <= 32 * PER words by one warp: every lane counts, for each of its PER words, the words
// of the segment that are smaller, which is the word's final position (all words differ).
template <int PER>
__device__ __forceinline__ void rank_sort_warp(uint64_t* s, uint64_t* __restrict__ entries, int32_t* __restrict__ sorted_ids,
                                               int beg, int n, int lane, int write_back) {
    uint64_t mine[PER];
#pragma unroll
    for (int r = 0; r < PER; r++) {
        const int i = lane + r * 32;
        mine[r] = (i < n) ? entries[beg + i] : ~0ull;
        if (i < n) s[i] = mine[r];
    }
    __syncwarp();
    int below[PER] = {};
    for (int j = 0; j < n; j++) {
        const uint64_t other = s[j];
#pragma unroll
        for (int r = 0; r < PER; r++) below[r] += (other < mine[r]) ? 1 : 0;
    }
#pragma unroll
    for (int r = 0; r < PER; r++) {
        if (lane + r * 32 < n) {
            sorted_ids[beg + below[r]] = (int32_t)(uint32_t)mine[r];
            if (write_back) entries[beg + below[r]] = mine[r];
        }
    }
}

// One warp per tile: rank sort of the tiles with at most kTileSortRank entries, the others go to the
// work list of their length class.
__global__ void __launch_bounds__(kTileSortThreads) tile_sort_kernel(uint64_t* __restrict__ entries,
                                                                     const int32_t* __restrict__ offsets, int tiles,
                                                                     int32_t* __restrict__ sorted_ids,
                                                                     uint32_t* __restrict__ lists, int write_back) {
    __shared__ uint64_t s_all[kTileSortWarps][kTileSortRank];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile = blockIdx.x * kTileSortWarps + warp;
    if (tile >= tiles) return;
    const int edge = (lane < 2) ? offsets[tile + lane] : 0;
    const int beg = __shfl_sync(0xffffffffu, edge, 0);
    const int n = __shfl_sync(0xffffffffu, edge, 1) - beg;
    if (n <= 0) return;
    if (n > kTileSortRank) {
        if (lane == 0) {
            if (n > kTileSortShort) long_items(lists)[atomicAdd(&lists[0], 1u)] = (uint32_t)tile;
            else mid_items(lists, tiles)[atomicAdd(&lists[2], 1u)] = (uint32_t)tile;
        }
        return;
    }
    uint64_t* s = s_all[warp];
    if (n <= 32) rank_sort_warp<1>(s, entries, sorted_ids, beg, n, lane, write_back);
    else if (n <= 64) rank_sort_warp<2>(s, entries, sorted_ids, beg, n, lane, write_back);
    else rank_sort_warp<kTileSortRank / 32>(s, entries, sorted_ids, beg, n, lane, write_back);
}

// Tiles of kTileSortRank < n <= kTileSortShort entries: persistent CTAs of 128 threads, next free item first.
__global__ void __launch_bounds__(kTileSortThreads) tile_sort_mid_kernel(uint64_t* entries,
                                                                         const int32_t* __restrict__ offsets, int tiles,
                                                                         int32_t* __restrict__ sorted_ids, uint32_t* lists,
                                                                         int write_back) {
    __shared__ uint64_t s_mid[kMidSmemWords];
    __shared__ uint32_t s_item;
    const int tid = threadIdx.x;
    const uint32_t count = lists[2];
    while (true) {
        if (tid == 0) s_item = atomicAdd(&lists[3], 1u);
        __syncthreads();
        const uint32_t w = s_item;
        __syncthreads();
        if (w >= count) break;
        const int tile = (int)mid_items(lists, tiles)[w];
        const int beg = offsets[tile];
        const uint32_t n = (uint32_t)(offsets[tile + 1] - beg);
        sort_segment_in_smem<3, kTileSortThreads>(s_mid, entries + beg, n, log2_at_least(n), sorted_ids + beg,
                                                  write_back != 0, tid);
    }
}

// One wide step of the network on a segment in global memory: pairs (i, l) with l >= n do nothing.
template <bool MIRROR>
__device__ __forceinline__ void global_step(uint64_t* seg, uint32_t n, uint32_t P, uint32_t j, uint32_t k, int tid) {
    for (uint32_t q = tid; q < (P >> 1); q += kTileSortLongThreads) {
        const uint32_t i = pair_low(q, j), l = MIRROR ? (i ^ (k - 1)) : (i | j);
        if (l < n) {
            uint64_t a = seg[i], b = seg[l];
            if (a > b) {
                seg[i] = b;
                seg[l] = a;
            }
        }
    }
    __syncthreads();
}

// Persistent CTAs (one per SM) take the long tiles from the work list, next free item first.
__global__ void __launch_bounds__(kTileSortLongThreads) tile_sort_long_kernel(uint64_t* entries,
                                                                              const int32_t* __restrict__ offsets,
                                                                              int32_t* __restrict__ sorted_ids,
                                                                              uint32_t* lists, int write_back) {
    extern __shared__ __align__(16) uint64_t s_long[];
    __shared__ uint32_t s_item;
    constexpr int kLogChunk = 14;
    static_assert((1 << kLogChunk) == kTileSortChunk && kTileSortLongThreads == 1024, "chunk = 1024 threads x 16 words");
    const int tid = threadIdx.x;
    const uint32_t count = lists[0];
    // Two rounds over the list: the tiles above 8192 entries first, the shorter ones afterwards, so that
    // the kernel does not end on a few SMs that drew a long tile late.
    for (int round = 0; round < 2; round++)
    while (true) {
        if (tid == 0) s_item = atomicAdd(&lists[round == 0 ? 1 : 4], 1u);
        __syncthreads();
        const uint32_t w = s_item;
        __syncthreads();
        if (w >= count) break;
        const int tile = (int)long_items(lists)[w];
        const int beg = offsets[tile];
        const uint32_t n = (uint32_t)(offsets[tile + 1] - beg);
        if ((n > 8192u) != (round == 0)) continue;
        uint64_t* seg = entries + beg;
        if (n <= 8192u) {            // 8 words per thread: 256, 512 or 1024 threads take part
            sort_segment_in_smem<3, kTileSortLongThreads>(s_long, seg, n, log2_at_least(n), sorted_ids + beg,
                                                          write_back != 0, tid);
        } else if (n <= (uint32_t)kTileSortChunk) {
            sort_segment_in_smem<4, kTileSortLongThreads>(s_long, seg, n, kLogChunk, sorted_ids + beg, write_back != 0,
                                                          tid);
        } else {
            // Chunks sorted in shared memory; the steps wider than a chunk run on the segment in global
            // memory.  This network compares towards the same side everywhere (the first step of a merge
            // pairs mirrored positions), so the words missing beyond n act as padding without being stored.
            uint32_t P = (uint32_t)kTileSortChunk;
            while (P < n) P <<= 1;
            for (uint32_t base = 0; base < n; base += kTileSortChunk) {
                const uint32_t m = (n - base < (uint32_t)kTileSortChunk) ? n - base : (uint32_t)kTileSortChunk;
                sort_segment_in_smem<4, kTileSortLongThreads>(s_long, seg + base, m, kLogChunk, nullptr, true, tid);
            }
            for (uint32_t k = 2u * kTileSortChunk; k <= P && k != 0; k <<= 1) {
                global_step<true>(seg, n, P, k >> 1, k, tid);
                for (uint32_t j = k >> 2; j >= (uint32_t)kTileSortChunk; j >>= 1) global_step<false>(seg, n, P, j, k, tid);
                for (uint32_t base = 0; base < n; base += kTileSortChunk) {
                    for (int i = tid; i < kTileSortChunk; i += kTileSortLongThreads)
                        s_long[padded<4>(i)] = (base + i < n) ? seg[base + i] : ~0ull;
                    __syncthreads();
                    blocked_steps<4>(s_long, tid, kLogChunk, kLogChunk, kLogChunk - 1, true);
                    for (int i = tid; i < kTileSortChunk; i += kTileSortLongThreads)
                        if (base + i < n) seg[base + i] = s_long[padded<4>(i)];
                    __syncthreads();
                }
            }
            for (uint32_t i = tid; i < n; i += kTileSortLongThreads) sorted_ids[beg + i] = (int32_t)(uint32_t)seg[i];
            __syncthreads();
        }
    }
}

}  // namespace tg

namespace tg_host {

size_t tile_sort_scratch_bytes(int tiles) { return sizeof(uint32_t) * (2 * (size_t)(tiles > 0 ? tiles : 0) + tg::kListHead); }

// `scratch_prepared`: the caller has zeroed the first six words of `lists`.  `longest`: an upper bound
// of the longest tile list when the caller knows one (the kernels of the length classes above it are
// not launched), UINT32_MAX otherwise.
int sort_tile_lists(uint64_t* entries, const int32_t* offsets, int tiles, int32_t* sorted_ids, uint32_t* lists,
                    bool scratch_prepared, bool write_back, uint32_t longest, cudaStream_t s) {
    TG_REQUIRE(tiles >= 0, "tiles < 0");
    if (tiles == 0) return TG_OK;
    TG_REQUIRE(entries && offsets && sorted_ids && lists, "null pointer");
    if (!scratch_prepared) TG_CUDA(cudaMemsetAsync(lists, 0, tg::kListHead * sizeof(uint32_t), s));
    tg::tile_sort_kernel<<<(tiles + tg::kTileSortWarps - 1) / tg::kTileSortWarps, tg::kTileSortThreads, 0, s>>>(
        entries, offsets, tiles, sorted_ids, lists, write_back ? 1 : 0);
    TG_LAUNCH_CHECK("tile_sort_kernel");
    if (longest > (uint32_t)tg::kTileSortRank) {
        const int grid = tiles < 148 * 12 ? tiles : 148 * 12;
        tg::tile_sort_mid_kernel<<<grid, tg::kTileSortThreads, 0, s>>>(entries, offsets, tiles, sorted_ids, lists,
                                                                        write_back ? 1 : 0);
        TG_LAUNCH_CHECK("tile_sort_mid_kernel");
    }
    if (longest > (uint32_t)tg::kTileSortShort) {
        constexpr int kMaxDevices = 64;
        static std::atomic<bool> attr_set[kMaxDevices];   // zero-initialised; setting the attribute twice is harmless
        const size_t long_smem = sizeof(uint64_t) * tg::kLongSmemWords;
        int dev = 0;
        TG_CUDA(cudaGetDevice(&dev));
        TG_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index outside the supported range");
        if (!attr_set[dev].load(std::memory_order_acquire)) {
            TG_CUDA(cudaFuncSetAttribute(tg::tile_sort_long_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)long_smem));
            attr_set[dev].store(true, std::memory_order_release);
        }
        const int grid = tiles < 148 ? tiles : 148;
        tg::tile_sort_long_kernel<<<grid, tg::kTileSortLongThreads, long_smem, s>>>(entries, offsets, sorted_ids, lists,
                                                                                     write_back ? 1 : 0);
        TG_LAUNCH_CHECK("tile_sort_long_kernel");
    }
    return TG_OK;
}

}  // namespace tg_host

extern "C" {

size_t tg_tile_sort_scratch_bytes(int tiles) { return tg_host::tile_sort_scratch_bytes(tiles); }

int tg_sort_tile_lists(uint64_t* entries, const int32_t* offsets, int tiles, int32_t* sorted_ids, void* scratch,
                       size_t scratch_bytes, tg_stream_t stream) {
    if (scratch_bytes < tg_host::tile_sort_scratch_bytes(tiles)) {
        tg_host::set_error("tile sort scratch: need %zu bytes, got %zu", tg_host::tile_sort_scratch_bytes(tiles),
                           scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    TG_REQUIRE(((uintptr_t)scratch & 3) == 0 && ((uintptr_t)entries & 7) == 0, "alignment");
    return tg_host::sort_tile_lists(entries, offsets, tiles, sorted_ids, (uint32_t*)scratch, false, true, UINT32_MAX,
                                    (cudaStream_t)stream);
}

}  // extern "C"
