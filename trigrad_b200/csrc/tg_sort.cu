// Stage 4: onesweep least-significant-digit radix sort of (uint64 key, uint32 value) pairs.
//
// The digits of every pass are counted in a single read of the keys (here, or on the fly by the
// key-emission kernel) and turned into global digit offsets.  Then one kernel per pass: each CTA
// takes a tile of pairs (ticket order), ranks them stably by the pass digit (per-warp ballots, one
// per digit bit), publishes its per-digit counts, obtains the counts of all earlier tiles by
// decoupled look-back (one thread per digit, bounded waits) and scatters keys and values through
// shared memory so that global writes are contiguous runs per digit.  Every pass reads 12 B and
// writes 12 B per pair: HBM-bound.
#include "tg_radix.cuh"

#ifndef TG_SORT_THREADS
#define TG_SORT_THREADS 256
#endif
#ifndef TG_SORT_ITEMS
#define TG_SORT_ITEMS 16
#endif
#ifndef TG_SORT_MIN_CTAS
#define TG_SORT_MIN_CTAS 3
#endif

namespace tg {

// Tile shape of a pass.  Measured on a B200 at 2^27 pairs (GB/s of algorithmic traffic): 256 threads x 16
// pairs 2551, 512x12 2396, 512x8 2254, 256x8 2014, 512x6 2069, 1024x4 1608 - more pairs per thread (fewer,
// larger tiles: less look-back and per-tile overhead) beats more resident warps.
constexpr int kPassThreads = TG_SORT_THREADS;
constexpr int kPassWarps = kPassThreads / 32;
constexpr int kPassItems = TG_SORT_ITEMS;
constexpr int kSortTile = kPassThreads * kPassItems;
constexpr uint32_t kSortSpinLimit = 1u << 22;
constexpr uint64_t kFlagAggregate = 1ull << 32;
constexpr uint64_t kFlagInclusive = 2ull << 32;
static_assert(kPassThreads >= kRadix && kPassThreads % 32 == 0, "one thread per digit is needed");
static_assert(32 * kPassItems <= 65535, "per-warp digit counters are 16 bit");

__global__ void __launch_bounds__(kSortThreads) sort_histogram_kernel(const uint64_t* __restrict__ keys, uint32_t n,
                                                                      HistArgs h) {
    __shared__ uint32_t s_hist[kMaxPasses * kRadix];
    __shared__ uint32_t s_warp_tot[kSortWarps];
    __shared__ bool s_last;
    for (int i = threadIdx.x; i < h.passes * kRadix; i += kSortThreads) s_hist[i] = 0;
    __syncthreads();
    const uint32_t stride = gridDim.x * kSortThreads;
    for (uint32_t i = blockIdx.x * kSortThreads + threadIdx.x; i < n; i += stride) hist_count(s_hist, keys[i], h);
    __syncthreads();
    hist_flush_and_finish(s_hist, s_warp_tot, &s_last, h);
}

__device__ __forceinline__ uint64_t ld_word(const uint64_t* p) { return *(const volatile uint64_t*)p; }
__device__ __forceinline__ void st_word(uint64_t* p, uint64_t v) { *(volatile uint64_t*)p = v; }

template <int THREADS, int ITEMS>
struct SortSmemT {
    uint64_t keys[THREADS * ITEMS];
    uint32_t vals[THREADS * ITEMS];
    uint16_t warp_hist[THREADS / 32][kRadix];   // per-warp digit counts, then offsets of the warp inside the digit
    uint32_t digit_start[kRadix];
    uint32_t bin_offset[kRadix];
    uint32_t warp_tot[8];
    uint32_t part;
    uint32_t fail;
};
using SortSmem = SortSmemT<kPassThreads, kPassItems>;
// Shape of the single-launch path for small inputs.  Measured on config 3 (338k pairs): 256x16 tiles 13 us
// per pass, 512x16 with all peer masks computed up front 15 us - the per-item ballot + offset chain
// (about 0.25 us per item and warp) and the prefix chain between tiles dominate, not the launches.
constexpr int kSmallThreads = 256;
constexpr int kSmallItems = 16;
constexpr int kSmallTile = kSmallThreads * kSmallItems;
using SortSmemSmall = SortSmemT<kSmallThreads, kSmallItems>;


// One tile of one pass.  `p` is the tile's position in the order in which tiles resolve their prefixes.
// PIPE marks the single-launch (all passes) variant.
template <int THREADS, int ITEMS, bool PIPE>
__device__ __forceinline__ void onesweep_tile(SortSmemT<THREADS, ITEMS>& sm, uint32_t p, const uint64_t* __restrict__ keys_in,
                                              const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out,
                                              uint32_t* __restrict__ vals_out, uint32_t n, int shift, int bits,
                                              const uint32_t* __restrict__ digit_offsets,
                                              uint64_t* __restrict__ lookback /*[parts][256]*/,
                                              uint32_t* __restrict__ status) {
    const int tid = threadIdx.x, warp = tid >> 5;
    const unsigned lane = lane_id();
    const uint32_t digit_mask = (1u << bits) - 1u;
    const uint64_t tile_base = (uint64_t)p * (THREADS * ITEMS);
    const uint32_t valid = (uint32_t)min((uint64_t)(THREADS * ITEMS), (uint64_t)n - tile_base);

    // warp-striped load: warp w owns a contiguous run of 32*ITEMS pairs, lane l takes items i*32 + l
    uint64_t key[ITEMS];
    uint32_t val[ITEMS];
    uint32_t rank2[(ITEMS + 1) / 2];   // two 16-bit ranks per register
#pragma unroll
    for (int i = 0; i < (ITEMS + 1) / 2; i++) rank2[i] = 0;
    const uint32_t warp_base = warp * (32 * ITEMS);
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const uint32_t idx = warp_base + i * 32 + lane;
        if (idx < valid) {
            if (PIPE) {   // single-launch path: other SMs rewrote the buffers in the previous pass, read through L2
                key[i] = __ldcg(keys_in + tile_base + idx);
                val[i] = __ldcg(vals_in + tile_base + idx);
            } else {
                key[i] = keys_in[tile_base + idx];
                val[i] = vals_in[tile_base + idx];
            }
        } else {
            key[i] = ~0ull;
            val[i] = 0;
        }
    }
    // Stable ranking inside the warp.  The lanes holding the same digit are found with one ballot per
    // digit bit (match.any costs several times more on this part when the digits of a warp are mostly
    // distinct).  Slots past the end of the input take the largest digit: they sit at the end of the last
    // tile, so they rank behind every real key and only inflate a count nobody reads.
    const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const uint32_t idx = warp_base + i * 32 + lane;
        const bool ok = idx < valid;
        const uint32_t d = ok ? ((uint32_t)(key[i] >> shift) & digit_mask) : digit_mask;
        unsigned peers = 0xffffffffu;
        for (int b = 0; b < bits; b++) {
            const bool bit = (d >> b) & 1u;
            const unsigned v = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? v : ~v;
        }
        const int leader = __ffs(peers) - 1;
        uint32_t old = 0;
        if ((int)lane == leader) {
            old = sm.warp_hist[warp][d];
            sm.warp_hist[warp][d] = (uint16_t)(old + __popc(peers));
        }
        old = __shfl_sync(0xffffffffu, old, leader);
        rank2[i >> 1] |= ((old + __popc(peers & lt_mask)) & 0xffffu) << (16 * (i & 1));
        __syncwarp();
    }
    __syncthreads();

    // per digit (thread d < 256): offsets of each warp inside the digit, CTA count, CTA start, look-back
    uint32_t cta_count = 0;
    if (THREADS == kRadix || tid < kRadix) {
        uint32_t run = 0;
#pragma unroll
        for (int w = 0; w < (THREADS / 32); w++) {
            const uint32_t c = sm.warp_hist[w][tid];
            sm.warp_hist[w][tid] = (uint16_t)run;
            run += c;
        }
        cta_count = run;
    }
    const uint32_t dstart = block_exclusive_scan_256(cta_count, sm.warp_tot);   // threads >= 256 contribute 0
    if (THREADS == kRadix || tid < kRadix) {
        uint64_t* mine = lookback + (size_t)p * kRadix + tid;
        uint32_t excl = 0;
        bool failed = false;
        if (p == 0) {
            st_word(mine, kFlagInclusive | cta_count);
        } else {
            st_word(mine, kFlagAggregate | cta_count);
            for (int64_t q = (int64_t)p - 1; q >= 0; --q) {
                const uint64_t* w = lookback + (size_t)q * kRadix + tid;
                uint64_t word = 0;
                uint32_t it = 0;
                for (; it < kSortSpinLimit; ++it) {
                    word = ld_word(w);
                    if (word >> 32) break;
                    if (it > 64) __nanosleep(100);
                }
                if (it == kSortSpinLimit) { failed = true; break; }
                excl += (uint32_t)word;
                if ((word >> 32) == 2u) break;
            }
            st_word(mine, kFlagInclusive | (uint64_t)(excl + cta_count));
        }
        if (failed) { sm.fail = 1; atomicExch(status, 2u); }
        sm.digit_start[tid] = dstart;
        sm.bin_offset[tid] = digit_offsets[tid] + excl - dstart;   // modulo 2^32 on purpose
    }
    __syncthreads();
    if (sm.fail) return;   // uniform: nothing is written by this tile

    // scatter into CTA-sorted order in shared memory
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const uint32_t idx = warp_base + i * 32 + lane;
        if (idx < valid) {
            const uint32_t d = (uint32_t)(key[i] >> shift) & digit_mask;
            const uint32_t r = sm.digit_start[d] + sm.warp_hist[warp][d] + ((rank2[i >> 1] >> (16 * (i & 1))) & 0xffffu);
            sm.keys[r] = key[i];
            sm.vals[r] = val[i];
        }
    }
    __syncthreads();
    // coalesced runs out to global memory
    for (uint32_t k = tid; k < valid; k += THREADS) {
        const uint64_t kk = sm.keys[k];
        const uint32_t d = (uint32_t)(kk >> shift) & digit_mask;
        const uint32_t dst = sm.bin_offset[d] + k;
        keys_out[dst] = kk;
        vals_out[dst] = sm.vals[k];
    }
}

// One pass, tiles taken in ticket order: a tile only ever waits for tiles that already run.
__global__ void __launch_bounds__(kPassThreads, TG_SORT_MIN_CTAS) onesweep_pass_kernel(
    const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out,
    uint32_t* __restrict__ vals_out, uint32_t n, int shift, int bits, const uint32_t* __restrict__ digit_offsets,
    uint32_t* __restrict__ ticket, uint64_t* __restrict__ lookback, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SortSmem& sm = *reinterpret_cast<SortSmem*>(smem_raw);
    if (threadIdx.x == 0) { sm.part = atomicAdd(ticket, 1u); sm.fail = 0; }
    for (int i = threadIdx.x; i < kPassWarps * kRadix / 2; i += kPassThreads) reinterpret_cast<uint32_t*>(&sm.warp_hist[0][0])[i] = 0;
    __syncthreads();
    const uint32_t p = sm.part;
    if ((uint64_t)p * kSortTile >= n) return;
    onesweep_tile<kPassThreads, kPassItems, false>(sm, p, keys_in, vals_in, keys_out, vals_out, n, shift, bits, digit_offsets, lookback,
                                                 status);
}

// Bounded grid-wide barrier for a cooperative launch: a counter that only grows.
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t target, uint32_t* status) {
    __shared__ uint32_t s_ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        uint32_t it = 0;
        for (; it < kSortSpinLimit; ++it) {
            if (*(volatile uint32_t*)counter >= target) break;
            if (it > 64) __nanosleep(40);
        }
        s_ok = it < kSortSpinLimit;
        if (!s_ok) atomicExch(status, 3u);
        __threadfence();
    }
    __syncthreads();
    return s_ok != 0;
}

// All passes in one cooperative launch (every tile resident at once): for small inputs the per-pass launch,
// ticket and drain latencies dominate, and a grid barrier between passes is cheaper than a new kernel.
__global__ void __launch_bounds__(kSmallThreads, 1) onesweep_all_passes_kernel(
    uint64_t* __restrict__ keys_a, uint32_t* __restrict__ vals_a, uint64_t* __restrict__ keys_b,
    uint32_t* __restrict__ vals_b, uint32_t n, int begin_bit, int end_bit, int passes,
    const uint32_t* __restrict__ digit_offsets /*[passes][256]*/, uint64_t* __restrict__ lookback /*[passes][parts][256]*/,
    uint32_t* __restrict__ barrier_counter, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SortSmemSmall& sm = *reinterpret_cast<SortSmemSmall*>(smem_raw);
    const uint32_t parts = gridDim.x;
    for (int pass = 0; pass < passes; pass++) {
        const int shift = begin_bit + pass * kRadixBits;
        const int bits = min(kRadixBits, end_bit - shift);
        if (threadIdx.x == 0) sm.fail = 0;
        for (int i = threadIdx.x; i < (kSmallThreads / 32) * kRadix / 2; i += kSmallThreads) reinterpret_cast<uint32_t*>(&sm.warp_hist[0][0])[i] = 0;
        __syncthreads();
        const bool odd = pass & 1;
        onesweep_tile<kSmallThreads, kSmallItems, true>(sm, blockIdx.x, odd ? keys_b : keys_a, odd ? vals_b : vals_a, odd ? keys_a : keys_b,
                      odd ? vals_a : vals_b, n, shift, bits, digit_offsets + pass * kRadix,
                      lookback + (size_t)pass * parts * kRadix, status);
        if (pass + 1 < passes && !grid_barrier(barrier_counter, (uint32_t)(pass + 1) * parts, status)) return;
    }
}

}  // namespace tg

namespace tg_host {

static inline int sort_passes(int begin_bit, int end_bit) { return (end_bit - begin_bit + tg::kRadixBits - 1) / tg::kRadixBits; }
static inline size_t sort_parts(uint32_t n) { return ((size_t)n + tg::kSortTile - 1) / tg::kSortTile; }

size_t sort_scratch_clear_bytes(uint32_t n, int passes) {
    return tg::kHistBytes + tg::kCtrBytes + (size_t)passes * sort_parts(n) * tg::kRadix * sizeof(uint64_t);
}

// scratch_prepared: the caller has zeroed sort_scratch_clear_bytes(>= n) bytes and filled the digit
// offsets (the key-emission kernel counts digits as it writes keys); then no clearing and no
// histogram pass are needed here.
int sort_pairs(uint64_t* keys_a, uint64_t* keys_b, uint32_t* vals_a, uint32_t* vals_b, uint32_t n, int begin_bit,
               int end_bit, void* scratch, size_t scratch_bytes, uint32_t* status, int* result_in_b_host,
               bool scratch_prepared, cudaStream_t s) {
    TG_REQUIRE(begin_bit >= 0 && end_bit <= 64 && begin_bit < end_bit, "bit range");
    TG_REQUIRE(n < 0x80000000u, "n must stay below 2^31");
    const int passes = sort_passes(begin_bit, end_bit);
    TG_REQUIRE(passes <= tg::kMaxPasses, "too many passes");
    if (result_in_b_host) *result_in_b_host = 0;
    if (n == 0) return TG_OK;
    TG_REQUIRE(keys_a && keys_b && vals_a && vals_b && scratch && status, "null pointer");
    TG_REQUIRE(((uintptr_t)scratch & 15) == 0, "scratch must be 16-byte aligned");
    const size_t parts = sort_parts(n);
    const size_t need = sort_scratch_clear_bytes(n, passes);
    if (scratch_bytes < need) {
        set_error("sort scratch: need %zu bytes, got %zu", need, scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    uint32_t* hist = (uint32_t*)scratch;
    uint32_t* ctr = (uint32_t*)((char*)scratch + tg::kHistBytes);   // [0..7] tickets, [8] histogram-done
    uint64_t* lookback = (uint64_t*)((char*)scratch + tg::kHistBytes + tg::kCtrBytes);
    if (!scratch_prepared) {
        TG_CUDA(cudaMemsetAsync(scratch, 0, need, s));
        int hist_grid = (int)((n + tg::kSortThreads * 16 - 1) / (tg::kSortThreads * 16));
        if (hist_grid > 148 * 8) hist_grid = 148 * 8;
        if (hist_grid < 1) hist_grid = 1;
        const tg::HistArgs h = {hist, ctr + tg::kHistDoneWord, begin_bit, end_bit, passes};
        tg::sort_histogram_kernel<<<hist_grid, tg::kSortThreads, 0, s>>>(keys_a, n, h);
        TG_LAUNCH_CHECK("sort_histogram_kernel");
    }
    static thread_local int cfg_device = -1;
    static thread_local size_t max_resident = 0;      // tiles that can be resident at once (cooperative launch limit)
    int dev = 0;
    TG_CUDA(cudaGetDevice(&dev));
    if (cfg_device != dev) {
        TG_CUDA(cudaFuncSetAttribute(tg::onesweep_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)sizeof(tg::SortSmem)));
        TG_CUDA(cudaFuncSetAttribute(tg::onesweep_all_passes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)sizeof(tg::SortSmemSmall)));
        int per_sm = 0, sms = 0, coop = 0;
        TG_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tg::onesweep_all_passes_kernel, tg::kSmallThreads,
                                                              sizeof(tg::SortSmemSmall)));
        TG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        TG_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        max_resident = coop ? (size_t)per_sm * sms : 0;
        cfg_device = dev;
    }
    const size_t small_parts = ((size_t)n + tg::kSmallTile - 1) / tg::kSmallTile;
    if (small_parts <= max_resident && passes > 1) {
        // small input: every (large) tile fits on the GPU at once, all passes in one cooperative launch
        uint32_t* barrier_counter = ctr + tg::kHistDoneWord + 1;
        int bb = begin_bit, eb = end_bit, np = passes;
        uint32_t nn = n;
        void* args[] = {&keys_a, &vals_a, &keys_b, &vals_b, &nn, &bb, &eb, &np, &hist, &lookback, &barrier_counter, &status};
        TG_CUDA(cudaLaunchCooperativeKernel((const void*)tg::onesweep_all_passes_kernel, dim3((unsigned)small_parts),
                                            dim3(tg::kSmallThreads), args, sizeof(tg::SortSmemSmall), s));
        TG_LAUNCH_CHECK("onesweep_all_passes_kernel");
        if (result_in_b_host) *result_in_b_host = passes & 1;
        return TG_OK;
    }
    uint64_t* kin = keys_a; uint64_t* kout = keys_b;
    uint32_t* vin = vals_a; uint32_t* vout = vals_b;
    for (int p = 0; p < passes; p++) {
        const int shift = begin_bit + p * tg::kRadixBits;
        const int bits = (end_bit - shift < tg::kRadixBits) ? (end_bit - shift) : tg::kRadixBits;
        uint64_t* lb = lookback + (size_t)p * parts * tg::kRadix;
        tg::onesweep_pass_kernel<<<(unsigned)parts, tg::kPassThreads, sizeof(tg::SortSmem), s>>>(
            kin, vin, kout, vout, n, shift, bits, hist + p * tg::kRadix, ctr + p, lb, status);
        TG_LAUNCH_CHECK("onesweep_pass_kernel");
        uint64_t* tk = kin; kin = kout; kout = tk;
        uint32_t* tv = vin; vin = vout; vout = tv;
    }
    if (result_in_b_host) *result_in_b_host = passes & 1;
    return TG_OK;
}

}  // namespace tg_host

extern "C" {


size_t tg_sort_scratch_bytes(uint32_t n) { return tg_host::sort_scratch_clear_bytes(n, tg::kMaxPasses); }

int tg_sort_pairs(uint64_t* keys_a, uint64_t* keys_b, uint32_t* vals_a, uint32_t* vals_b, uint32_t n, int begin_bit,
                  int end_bit, void* scratch, size_t scratch_bytes, uint32_t* status, int* result_in_b_host,
                  tg_stream_t stream) {
    return tg_host::sort_pairs(keys_a, keys_b, vals_a, vals_b, n, begin_bit, end_bit, scratch, scratch_bytes, status,
                               result_in_b_host, false, (cudaStream_t)stream);
}

}  // extern "C"
