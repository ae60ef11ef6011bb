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

struct SortSmem {
    uint64_t keys[kSortTile];
    uint32_t vals[kSortTile];
    uint16_t warp_hist[kPassWarps][kRadix];   // per-warp digit counts, then offsets of the warp inside the digit
    uint32_t digit_start[kRadix];
    uint32_t bin_offset[kRadix];
    uint32_t warp_tot[8];
    uint32_t part;
    uint32_t fail;
};

__global__ void __launch_bounds__(kPassThreads, TG_SORT_MIN_CTAS) onesweep_pass_kernel(
    const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint64_t* __restrict__ keys_out,
    uint32_t* __restrict__ vals_out, uint32_t n, int shift, int bits, const uint32_t* __restrict__ digit_offsets,
    uint32_t* __restrict__ ticket, uint64_t* __restrict__ lookback /*[parts][256]*/, uint32_t* __restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    SortSmem& sm = *reinterpret_cast<SortSmem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5;
    const unsigned lane = lane_id();
    const uint32_t digit_mask = (1u << bits) - 1u;

    if (tid == 0) { sm.part = atomicAdd(ticket, 1u); sm.fail = 0; }
    for (int i = tid; i < kPassWarps * kRadix / 2; i += kPassThreads) reinterpret_cast<uint32_t*>(&sm.warp_hist[0][0])[i] = 0;
    __syncthreads();
    const uint32_t p = sm.part;
    const uint64_t tile_base = (uint64_t)p * kSortTile;
    if (tile_base >= n) return;
    const uint32_t valid = (uint32_t)min((uint64_t)kSortTile, (uint64_t)n - tile_base);

    // warp-striped load: warp w owns a contiguous run of 32*kPassItems pairs, lane l takes items i*32 + l
    uint64_t key[kPassItems];
    uint32_t val[kPassItems];
    uint16_t rank[kPassItems];
    const uint32_t warp_base = warp * (32 * kPassItems);
#pragma unroll
    for (int i = 0; i < kPassItems; i++) {
        const uint32_t idx = warp_base + i * 32 + lane;
        if (idx < valid) {
            key[i] = keys_in[tile_base + idx];
            val[i] = vals_in[tile_base + idx];
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
    for (int i = 0; i < kPassItems; i++) {
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
        rank[i] = (uint16_t)(old + __popc(peers & lt_mask));
        __syncwarp();
    }
    __syncthreads();

    // per digit (thread d < 256): offsets of each warp inside the digit, CTA count, CTA start, look-back
    uint32_t cta_count = 0;
    if (tid < kRadix) {
        uint32_t run = 0;
#pragma unroll
        for (int w = 0; w < kPassWarps; w++) {
            const uint32_t c = sm.warp_hist[w][tid];
            sm.warp_hist[w][tid] = (uint16_t)run;
            run += c;
        }
        cta_count = run;
    }
    const uint32_t dstart = block_exclusive_scan_256(cta_count, sm.warp_tot);   // threads >= 256 contribute 0
    if (tid < kRadix) {
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
    if (sm.fail) return;

    // scatter into CTA-sorted order in shared memory
#pragma unroll
    for (int i = 0; i < kPassItems; i++) {
        const uint32_t idx = warp_base + i * 32 + lane;
        if (idx < valid) {
            const uint32_t d = (uint32_t)(key[i] >> shift) & digit_mask;
            const uint32_t r = sm.digit_start[d] + sm.warp_hist[warp][d] + rank[i];
            sm.keys[r] = key[i];
            sm.vals[r] = val[i];
        }
    }
    __syncthreads();
    // coalesced runs out to global memory
    for (uint32_t k = tid; k < valid; k += kPassThreads) {
        const uint64_t kk = sm.keys[k];
        const uint32_t d = (uint32_t)(kk >> shift) & digit_mask;
        const uint32_t dst = sm.bin_offset[d] + k;
        keys_out[dst] = kk;
        vals_out[dst] = sm.vals[k];
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
    static thread_local int smem_set_device = -1;
    int dev = 0;
    TG_CUDA(cudaGetDevice(&dev));
    if (smem_set_device != dev) {
        TG_CUDA(cudaFuncSetAttribute(tg::onesweep_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)sizeof(tg::SortSmem)));
        smem_set_device = dev;
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
