// Radix-sort constants and the digit-histogram helpers shared by the sort kernels and by the key
// emission kernel (which can count the digits of the keys it writes, saving one read of them).
#pragma once
#include "tg_common.cuh"

namespace tg {

constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kMaxPasses = 8;
constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;

// scratch layout (bytes): [0, 8 KB) digit histograms / offsets [kMaxPasses][256] uint32,
// [8 KB, 8 KB + 64) tickets[kMaxPasses] + histogram-done counter (word 8), then the look-back words
// [passes][parts][256] uint64.
constexpr size_t kHistBytes = (size_t)kMaxPasses * kRadix * sizeof(uint32_t);
constexpr size_t kCtrBytes = 64;
constexpr int kHistDoneWord = 8;
// Up to this many tiles the CTA that finishes the fused preprocess kernel last scans the tile counts itself.
constexpr int kTileScanByLastCta = 65536;
// Top bit of the longest-list word the binning kernel reports: a launch order of the tiles was written.
constexpr uint32_t kOrderWrittenBit = 0x80000000u;

// Exclusive scan of one value per thread over the first 256 threads of a CTA (all threads of the CTA
// must call it; threads beyond 256 pass 0 and ignore the result).
__device__ __forceinline__ uint32_t block_exclusive_scan_256(uint32_t v, uint32_t* s_warp_tot /*[8]*/) {
    uint32_t incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane_id() >= (unsigned)d) incl += y;
    }
    const int warp = threadIdx.x >> 5;
    __syncthreads();   // protect s_warp_tot from a previous use
    if (lane_id() == 31 && warp < kSortWarps) s_warp_tot[warp] = incl;
    __syncthreads();
    uint32_t off = 0;
#pragma unroll
    for (int w = 0; w < kSortWarps; w++) {
        uint32_t x = s_warp_tot[w];
        if (w < warp) off += x;
    }
    return off + incl - v;
}

struct HistArgs {
    uint32_t* hist;           // [kMaxPasses][256] global counts, zeroed by the host; NULL = no histogram
    uint32_t* done_counter;   // zeroed by the host
    int begin_bit, end_bit, passes;
};

// Count the digits of one key into the CTA's shared histogram.
__device__ __forceinline__ void hist_count(uint32_t* s_hist, uint64_t key, const HistArgs& h) {
    for (int p = 0; p < h.passes; p++) {
        const int shift = h.begin_bit + p * kRadixBits;
        const int bits = min(kRadixBits, h.end_bit - shift);
        atomicAdd(&s_hist[p * kRadix + ((uint32_t)(key >> shift) & ((1u << bits) - 1u))], 1u);
    }
}

// Add the CTA's histogram to the global one; the last CTA to arrive turns the global counts into
// exclusive digit offsets, per pass.  Call with all 256 threads of every CTA, after a barrier.
__device__ __forceinline__ void hist_flush_and_finish(uint32_t* s_hist, uint32_t* s_warp_tot, bool* s_last,
                                                      const HistArgs& h) {
    for (int i = threadIdx.x; i < h.passes * kRadix; i += kSortThreads) {
        const uint32_t c = s_hist[i];
        if (c) atomicAdd(&h.hist[i], c);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *s_last = (atomicAdd(h.done_counter, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    for (int p = 0; p < h.passes; p++) {
        const uint32_t c = __ldcg(&h.hist[p * kRadix + threadIdx.x]);
        const uint32_t e = block_exclusive_scan_256(c, s_warp_tot);
        h.hist[p * kRadix + threadIdx.x] = e;
    }
}

}  // namespace tg

namespace tg_host {
// Internal (not part of the C ABI): the pieces tg_render_forward strings together.
int emit_keys(const float* vertices, const int32_t* indices, int T, int W, int H, int tw, int th,
              const uint32_t* tri_offsets, uint64_t* keys, uint32_t* ids, uint32_t capacity, const tg::HistArgs& hist,
              cudaStream_t stream);
int sort_pairs(uint64_t* keys_a, uint64_t* keys_b, uint32_t* vals_a, uint32_t* vals_b, uint32_t n, int begin_bit,
               int end_bit, void* scratch, size_t scratch_bytes, uint32_t* status, int* result_in_b_host,
               bool scratch_prepared, cudaStream_t stream);
size_t sort_scratch_clear_bytes(uint32_t n, int passes);
size_t preprocess_scan_scratch_bytes(int T);
int preprocess_scan(const float* vertices, const int32_t* indices, const float* colors, const float* opacities, int T,
                    int W, int H, int tw, int th, float* tri_geo, float* tri_attr, uint32_t* tri_offsets, void* scratch,
                    uint32_t* status, uint32_t* tile_cursor, int32_t* offsets, void* tile_scan_scratch, bool cull,
                    bool packed, uint32_t* tile_order, cudaStream_t stream);
int emit_entries(const float* vertices, const int32_t* indices, int T, int W, int H, int tw, int th,
                 const uint32_t* tri_offsets, const void* scan_scratch, uint32_t* tile_cursor, uint64_t* entries,
                 uint32_t capacity, const float* tri_geo_for_cull, bool packed, cudaStream_t stream);
void set_tile_order(const uint32_t* order, uint32_t longest_list = 0);
size_t tile_sort_scratch_bytes(int tiles);
int sort_tile_lists(uint64_t* entries, const int32_t* offsets, int tiles, int32_t* sorted_ids, uint32_t* lists,
                    bool scratch_prepared, bool write_back, uint32_t longest, cudaStream_t stream);
}  // namespace tg_host
