// Binning stages: per-triangle preprocess, device-wide scan, key emission, tile ranges.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "tg_radix.cuh"

namespace tg {

// ================================================================================================
// Stage 1: preprocess.  One thread per triangle: gathers its three vertices and attributes,
// counts the tiles its bounding box touches and writes the two packed records the compositing
// kernels stream.  HBM-bound: reads 12 B + 3 gathers of (16+12+4) B, writes 4 + 64 + 96 B.
__device__ __forceinline__ uint32_t preprocess_triangle(int t, const float4* __restrict__ vertices,
                                                        const int* __restrict__ indices,
                                                        const float* __restrict__ colors,
                                                        const float* __restrict__ opacities, int W, int H, int tw,
                                                        int th, int tiles_x, int tiles_y, int4* __restrict__ tri_rects,
                                                        float4* __restrict__ tri_geo, float4* __restrict__ tri_attr,
                                                        Rect& r, float* m_out = nullptr, bool packed = false) {
    // packed inputs: faces as [T,4] int32 and colours as [V,4] (r, g, b, opacity), one 16-byte load each instead
    // of the reference's 12-byte strides (util.h:457-573); the branch is uniform over the grid
    int ia, ib, ic;
    if (packed) {
        const int4 f = reinterpret_cast<const int4*>(indices)[t];
        ia = f.x; ib = f.y; ic = f.z;
    } else {
        ia = indices[3 * (size_t)t]; ib = indices[3 * (size_t)t + 1]; ic = indices[3 * (size_t)t + 2];
    }
    float4 a = vertices[ia], b = vertices[ib], c = vertices[ic];

    bool ok = tile_rect(a.x, a.y, b.x, b.y, c.x, c.y, W, H, tw, th, tiles_x, tiles_y, r);
    const uint32_t count = ok ? (uint32_t)(r.x1 - r.x0 + 1) * (uint32_t)(r.y1 - r.y0 + 1) : 0u;
    if (tri_rects) tri_rects[t] = make_int4(r.x0, r.y0, r.x1, r.y1);

    // barycentric matrix, reference render.cu:324-336: plain mul/sub/div
    float denom = add(add(mul(a.x, sub(b.y, c.y)), mul(b.x, sub(c.y, a.y))), mul(c.x, sub(a.y, b.y)));
    if (fabsf(denom) < kEffZero) denom = 1.0f;
    float m0 = div(sub(b.y, c.y), denom);
    float m1 = div(sub(c.x, b.x), denom);
    float m2 = div(sub(mul(b.x, c.y), mul(c.x, b.y)), denom);
    float m3 = div(sub(c.y, a.y), denom);
    float m4 = div(sub(a.x, c.x), denom);
    float m5 = div(sub(mul(c.x, a.y), mul(a.x, c.y)), denom);
    float m6 = div(sub(a.y, b.y), denom);
    float m7 = div(sub(b.x, a.x), denom);
    float m8 = div(sub(mul(a.x, b.y), mul(b.x, a.y)), denom);
    if (m_out) {
        m_out[0] = m0; m_out[1] = m1; m_out[2] = m2; m_out[3] = m3; m_out[4] = m4; m_out[5] = m5; m_out[6] = m6;
        m_out[7] = m7; m_out[8] = m8;
    }

    // Lower bound of the per-pixel sort depth: with weights of one sign the interpolated depth is
    // a convex combination of the vertex depths; a relative margin covers fp32 rounding.
    float zlow = -INFINITY;
    bool same_sign = (a.w > 0.f && b.w > 0.f && c.w > 0.f) || (a.w < 0.f && b.w < 0.f && c.w < 0.f);
    if (same_sign) {
        float zmin = fminf(fminf(a.z, b.z), c.z);
        float zabs = fmaxf(fmaxf(fabsf(a.z), fabsf(b.z)), fabsf(c.z));
        float lo = zmin - 4e-6f * zabs;
        if (isfinite(lo)) zlow = lo;
    }

    float4* g = tri_geo + 4 * (size_t)t;
    g[0] = make_float4(m0, m1, m2, m3);
    g[1] = make_float4(m4, m5, m6, m7);
    g[2] = make_float4(m8, a.z, b.z, c.z);
    g[3] = make_float4(a.w, b.w, c.w, zlow);

    float4* q = tri_attr + 6 * (size_t)t;
    float4 ra, rb, rc;   // (r, g, b, opacity) of the three vertices
    if (packed) {
        const float4* rgba = reinterpret_cast<const float4*>(colors);
        ra = rgba[ia]; rb = rgba[ib]; rc = rgba[ic];
    } else {
        const float* ca = colors + 3 * (size_t)ia;
        const float* cb = colors + 3 * (size_t)ib;
        const float* cc = colors + 3 * (size_t)ic;
        ra = make_float4(ca[0], ca[1], ca[2], opacities[ia]);
        rb = make_float4(cb[0], cb[1], cb[2], opacities[ib]);
        rc = make_float4(cc[0], cc[1], cc[2], opacities[ic]);
    }
    q[0] = make_float4(ra.w, rb.w, rc.w, ra.x);
    q[1] = make_float4(ra.y, ra.z, rb.x, rb.y);
    q[2] = make_float4(rb.z, rc.x, rc.y, rc.z);
    q[3] = make_float4(div(1.f, a.w), div(1.f, b.w), div(1.f, c.w), __int_as_float(ia));
    q[4] = make_float4(__int_as_float(ib), __int_as_float(ic), a.x, a.y);
    q[5] = make_float4(b.x, b.y, c.x, c.y);
    return count;
}

__global__ void __launch_bounds__(256) preprocess_kernel(const float4* __restrict__ vertices,
                                                         const int* __restrict__ indices,
                                                         const float* __restrict__ colors,
                                                         const float* __restrict__ opacities, int T, int W, int H,
                                                         int tw, int th, int tiles_x, int tiles_y,
                                                         uint32_t* __restrict__ tri_counts, int4* __restrict__ tri_rects,
                                                         float4* __restrict__ tri_geo, float4* __restrict__ tri_attr) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    Rect r;
    tri_counts[t] = preprocess_triangle(t, vertices, indices, colors, opacities, W, H, tw, th, tiles_x, tiles_y, tri_rects,
                                        tri_geo, tri_attr, r);
}

// ================================================================================================
// Stage 2: single-pass exclusive scan with decoupled look-back.
// scratch: word 0 = ticket counter (uint32, padded to 8 bytes), then one uint64 per partition:
// (flag << 32) | value, flag 0 = nothing yet, 1 = partition aggregate, 2 = inclusive prefix.
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;
constexpr uint32_t kSpinLimit = 1u << 22;   // bounded wait: ~ seconds with the nanosleep below

__device__ __forceinline__ uint64_t ld_volatile(const uint64_t* p) { return *(const volatile uint64_t*)p; }
__device__ __forceinline__ void st_volatile(uint64_t* p, uint64_t v) { *(volatile uint64_t*)p = v; }

// Wait (bounded) until the partition word has a non-zero flag.  Returns false if the wait ran out.
__device__ __forceinline__ bool wait_flag(const uint64_t* p, uint64_t& word, uint32_t spin_limit) {
    for (uint32_t it = 0; it < spin_limit; ++it) {
        word = ld_volatile(p);
        if ((word >> 32) != 0) return true;
        if (it > 64) __nanosleep(100);
    }
    return false;
}

// Decoupled look-back, executed by ONE WARP of partition p: publishes the partition's total, sums the
// totals of all earlier partitions (32 words per step) until one of them already carries an inclusive
// prefix, publishes its own inclusive prefix and returns the exclusive one.
__device__ __forceinline__ uint32_t lookback_exclusive(int p, uint32_t total, uint64_t* part_status, uint32_t* status,
                                                       uint32_t spin_limit = kSpinLimit) {
    uint32_t excl = 0;
    if (p == 0) {
        if (lane_id() == 0) st_volatile(&part_status[0], (2ull << 32) | total);
        return 0;
    }
    if (lane_id() == 0) st_volatile(&part_status[p], (1ull << 32) | total);
    int q = p - 1 - (int)lane_id();
    bool failed = false;
    while (true) {
        uint64_t word = 2ull << 32;   // virtual partitions before 0: inclusive prefix 0
        if (q >= 0 && !wait_flag(&part_status[q], word, spin_limit)) { failed = true; word = 2ull << 32; }
        const uint32_t flag = (uint32_t)(word >> 32), val = (uint32_t)word;
        const unsigned incl_mask = __ballot_sync(0xffffffffu, flag == 2u);
        uint32_t contrib = val;
        if (incl_mask) {
            const int first = __ffs(incl_mask) - 1;
            if ((int)lane_id() > first) contrib = 0;
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, d);
        excl += contrib;
        if (incl_mask) break;
        q -= 32;
    }
    if (__any_sync(0xffffffffu, failed) && lane_id() == 0) atomicExch(status, 1u);
    if (lane_id() == 0) st_volatile(&part_status[p], (2ull << 32) | (uint64_t)(excl + total));
    return excl;
}

__global__ void __launch_bounds__(kScanThreads) scan_kernel(const uint32_t* __restrict__ in,
                                                            uint32_t* __restrict__ out, int n, int num_parts,
                                                            uint32_t* ticket, uint64_t* part_status,
                                                            uint32_t* status) {
    __shared__ uint32_t s_part;
    __shared__ uint32_t s_warp[kScanThreads / 32];
    __shared__ uint32_t s_excl;
    if (threadIdx.x == 0) s_part = atomicAdd(ticket, 1u);
    __syncthreads();
    const int p = (int)s_part;
    if (p >= num_parts) return;
    const int base = p * kScanTile + threadIdx.x * kScanItems;

    uint32_t v[kScanItems];
    uint32_t sum = 0;
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        v[i] = (base + i < n) ? in[base + i] : 0u;
        sum += v[i];
    }
    // block exclusive scan of `sum`
    uint32_t incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane_id() >= (unsigned)d) incl += y;
    }
    const int warp = threadIdx.x >> 5;
    if (lane_id() == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t warp_off = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; w++) {
        uint32_t x = s_warp[w];
        if (w < warp) warp_off += x;
        total += x;
    }
    uint32_t thread_excl = warp_off + incl - sum;

    if (warp == 0) {
        const uint32_t excl = lookback_exclusive(p, total, part_status, status);
        if (lane_id() == 0) {
            s_excl = excl;
            if (p == num_parts - 1) out[n] = excl + total;
        }
    }
    __syncthreads();
    uint32_t run = s_excl + thread_excl;
#pragma unroll
    for (int i = 0; i < kScanItems; i++) {
        if (base + i < n) out[base + i] = run;
        run += v[i];
    }
}

// Self-test of the bounded wait: ONE warp plays partition 1 of a scan whose partition 0 never publishes
// anything (its word stays zero), with a spin limit of a few polls.  The wait runs out, the warp raises the
// status word and returns; nothing waits for anything else, so the launch always ends.
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(uint64_t* part_status /*[2], zero*/, uint32_t* status,
                                                                  uint32_t spin_limit, uint32_t* excl_out) {
    const uint32_t excl = lookback_exclusive(1, 7u, part_status, status, spin_limit);
    if (lane_id() == 0) *excl_out = excl;
}

// Stages 1 and 2 as the forward path runs them: the CTA that preprocesses 256 triangles scans their
// tile counts among themselves (`tri_offsets[t]` = entries of the CTA's earlier triangles) and leaves
// its total in `part_total`; no CTA waits for another.  The writer of the entries only needs these local
// offsets, because it places every entry through its tile's cursor.
//
// The CTA also counts its (triangle, tile) entries per tile, one thread per entry, and the CTA that
// finishes last adds up the totals (K) and turns the tile counts into the exclusive tile offsets, in place
// (`tile_cursor[t]` = first slot of tile t, advanced later by the entry writer) and in `bin.offsets`.
struct TileBinArgs {
    uint32_t* tile_cursor;   // [tiles], zero on entry
    int32_t* offsets;        // [tiles + 1], written when scan_here
    uint32_t* done;          // zero on entry: counts finished CTAs
    int tiles;
    int scan_here;           // 1: the last CTA scans the tile counts; 0: the host launches a scan
    uint32_t* longest;       // written when scan_here: the largest tile count
    uint32_t* part_total;    // [CTAs] entries of each CTA's triangles
    uint32_t* k_out;         // K = all entries
    uint32_t* order;         // [tiles] or null: tiles by descending list-length class, written when scan_here and
                             // the lists are long and uneven enough to matter; *longest then carries kOrderWrittenBit
};

// Exclusive scan of cursor[0..tiles) by one CTA of 256 threads, in place, copy in offsets[0..tiles].
// Rounds of 2048 counts: coalesced loads into shared memory, eight consecutive counts per thread,
// coalesced stores (a single SM issues too few memory requests per clock for anything strided).
constexpr int kTileScanRound = 2048;
__device__ uint32_t tile_offsets_by_one_cta(uint32_t* cursor, int32_t* offsets, int tiles, uint32_t* longest,
                                        uint32_t* s_buf /*[2048]*/, uint32_t* s_warp /*[8]*/,
                                        uint32_t* k_out = nullptr) {
    constexpr int kPer = kTileScanRound / 256;
    const int tid = threadIdx.x, warp = tid >> 5;
    uint32_t carry = 0, biggest = 0;
    for (int base = 0; base < tiles; base += kTileScanRound) {
        __syncthreads();                      // s_buf and s_warp free again
#pragma unroll
        for (int k = 0; k < kPer; k++) {
            const int i = base + k * 256 + tid;
            s_buf[k * 256 + tid] = (i < tiles) ? __ldcg(cursor + i) : 0u;
        }
        __syncthreads();
        uint32_t v[kPer], mine = 0;
#pragma unroll
        for (int k = 0; k < kPer; k++) {
            v[k] = s_buf[tid * kPer + k];
            mine += v[k];
            biggest = max(biggest, v[k]);
        }
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane_id() >= (unsigned)d) incl += y;
        }
        if (lane_id() == 31) s_warp[warp] = incl;
        __syncthreads();
        uint32_t warp_off = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) {
            uint32_t x = s_warp[w];
            if (w < warp) warp_off += x;
            total += x;
        }
        uint32_t run = carry + warp_off + incl - mine;
#pragma unroll
        for (int k = 0; k < kPer; k++) {
            s_buf[tid * kPer + k] = run;
            run += v[k];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kPer; k++) {
            const int i = base + k * 256 + tid;
            if (i < tiles) {
                const uint32_t x = s_buf[k * 256 + tid];
                cursor[i] = x;
                offsets[i] = (int32_t)x;
            }
        }
        carry += total;
    }
    if (tid == 0) {
        offsets[tiles] = (int32_t)carry;
        if (k_out) *k_out = carry;
    }
    biggest = __reduce_max_sync(0xffffffffu, biggest);
    __syncthreads();
    if (lane_id() == 0) s_warp[warp] = biggest;
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int w = 1; w < 8; w++) biggest = max(biggest, s_warp[w]);
        *longest = biggest;
        s_warp[0] = biggest;
    }
    __syncthreads();
    return s_warp[0];
}

// Launch order for the compositing kernel: tiles grouped by the class floor(log2(length)) + 1 of their list length,
// longest class first (empty tiles last).  With one CTA per tile in scan order a tile whose list is as long as
// everything else an SM processes can start late and leave the other SMs idle (a view of a fine mesh: 28 % of the
// SM time); long lists first removes that tail.  Worth its two passes over the offsets only when lists are long and
// uneven and the tiles are few enough for one CTA (a 1920x1080 image: 8160 tiles, 5 us).
constexpr uint32_t kOrderMinLongest = 256;
constexpr int kOrderMaxTiles = 16384;
constexpr uint32_t kOrderMinMean = 64;
__device__ void tile_order_by_one_cta(const int32_t* offsets, int tiles, uint32_t* order, uint32_t* s_hist /*[33]*/) {
    const int tid = threadIdx.x;
    const unsigned lane = lane_id(), lt_mask = (1u << lane) - 1u;
    if (tid < 33) s_hist[tid] = 0;
    __syncthreads();
    const int padded = (tiles + 255) & ~255;
    for (int i = tid; i < padded; i += 256) {
        const int cls = (i < tiles) ? 32 - __clz((uint32_t)(offsets[i + 1] - offsets[i])) : 33;
        const unsigned peers = __match_any_sync(0xffffffffu, cls);          // one shared-memory atomic per class and warp
        if (cls <= 32 && (peers & lt_mask) == 0) atomicAdd(&s_hist[cls], (uint32_t)__popc(peers));
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t run = 0;
        for (int c = 32; c >= 0; c--) { const uint32_t n = s_hist[c]; s_hist[c] = run; run += n; }
    }
    __syncthreads();
    for (int i = tid; i < padded; i += 256) {
        const int cls = (i < tiles) ? 32 - __clz((uint32_t)(offsets[i + 1] - offsets[i])) : 33;
        const unsigned peers = __match_any_sync(0xffffffffu, cls);
        const int leader = __ffs(peers) - 1;
        uint32_t base = 0;
        if (cls <= 32 && (int)lane == leader) base = atomicAdd(&s_hist[cls], (uint32_t)__popc(peers));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (cls <= 32) order[base + __popc(peers & lt_mask)] = (uint32_t)i;
    }
}

// CULL: a (triangle, tile) pair of the bounding rectangle is counted only if the triangle can cover the centre of
// some pixel of the tile (rect_may_cover on the tile's pixel-centre rectangle): the exact test the reference
// leaves open (render.cu:110).  K is then the sum of the tile counts, not of the rectangle sizes.
// MINB: CTAs per SM the register budget is set for.  Six (40 registers) keeps a mesh of up to 888 x 256 triangles
// resident in a single wave; larger meshes run several waves anyway and gain from more registers per thread
// (more of a triangle's gathers in flight at once).
#ifndef TG_PREPROCESS_MINB_LARGE
#define TG_PREPROCESS_MINB_LARGE 5
#endif
template <bool CULL, int MINB>
__global__ void __launch_bounds__(256, MINB) preprocess_count_kernel(const float4* __restrict__ vertices,
                                                               const int* __restrict__ indices,
                                                               const float* __restrict__ colors,
                                                               const float* __restrict__ opacities, int T, int W, int H,
                                                               int tw, int th, int tiles_x, int tiles_y,
                                                               float4* __restrict__ tri_geo, float4* __restrict__ tri_attr,
                                                               uint32_t* __restrict__ tri_offsets /*[T], CTA-local*/,
                                                               TileBinArgs bin, int packed) {
    __shared__ uint32_t s_warp[8];
    __shared__ uint32_t s_buf[kTileScanRound];
    uint32_t* s_loc = s_buf;                 // [257] exclusive offsets of the CTA's triangles within the CTA
    int* s_rect = (int*)s_buf + 257;         // [768] x0, y0, rows of each triangle's tile rectangle
    __shared__ bool s_last;
    __shared__ uint32_t s_k_upper;
    __shared__ float s_m[CULL ? 9 * 256 : 1];   // barycentric matrices of the CTA's triangles, component-major
    const int tid = threadIdx.x;
    const int p = blockIdx.x, num_parts = gridDim.x;
    const int t = p * 256 + tid;
    Rect r = {0, 0, 0, 0};
    float m[9];
    const uint32_t count = (t < T) ? preprocess_triangle(t, vertices, indices, colors, opacities, W, H, tw, th, tiles_x,
                                                         tiles_y, nullptr, tri_geo, tri_attr, r, CULL ? m : nullptr, packed != 0)
                                   : 0u;
    if (CULL && count) {
#pragma unroll
        for (int k = 0; k < 9; k++) s_m[k * 256 + tid] = m[k];
    }
    uint32_t incl = count;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane_id() >= (unsigned)d) incl += y;
    }
    const int warp = tid >> 5;
    if (lane_id() == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t warp_off = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; w++) {
        uint32_t x = s_warp[w];
        if (w < warp) warp_off += x;
        total += x;
    }
    const uint32_t local_excl = warp_off + incl - count;
    s_loc[tid] = local_excl;
    s_rect[3 * tid] = r.x0;
    s_rect[3 * tid + 1] = r.y0;
    s_rect[3 * tid + 2] = r.y1 - r.y0 + 1;
    if (tid == 0) {
        s_loc[256] = total;
        bin.part_total[p] = total;
    }
    if (t < T) tri_offsets[t] = local_excl;
    __syncthreads();

    for (uint32_t e = tid; e < total; e += 256) {
        int lo = 0, hi = 256;                 // largest i with s_loc[i] <= e
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_loc[mid] <= e) lo = mid; else hi = mid;
        }
        const uint32_t local = e - s_loc[lo];
        const uint32_t ny = (uint32_t)s_rect[3 * lo + 2];
        const int tx = s_rect[3 * lo] + (int)(local / ny), ty = s_rect[3 * lo + 1] + (int)(local % ny);
        if (CULL) {
            float mm[9];
#pragma unroll
            for (int k = 0; k < 9; k++) mm[k] = s_m[k * 256 + lo];
            if (!rect_may_cover(mm, tile_pixel_rect(tx, ty, W, H, tw, th))) continue;
        }
        atomicAdd(&bin.tile_cursor[ty * tiles_x + tx], 1u);
    }
    __syncthreads();                          // the CTA's counts are issued; one cumulative fence publishes them
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(bin.done, 1u) == (uint32_t)num_parts - 1u);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // K: sum of the CTA totals
    uint32_t k = 0;
    for (int i = tid; i < num_parts; i += 256) k += __ldcg(bin.part_total + i);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) k += __shfl_xor_sync(0xffffffffu, k, d);
    __syncthreads();
    if (lane_id() == 0) s_warp[warp] = k;
    __syncthreads();
    if (tid == 0) {
        k = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) k += s_warp[w];
        if (!CULL) *bin.k_out = k;
        s_k_upper = k;                       // with culling an upper bound of K (sum of the rectangle sizes)
    }
    __syncthreads();
    if (bin.scan_here) {
        const uint32_t biggest = tile_offsets_by_one_cta(bin.tile_cursor, bin.offsets, bin.tiles, bin.longest, s_buf, s_warp,
                                                         CULL ? bin.k_out : nullptr);
        // the launch order costs two more passes over the offsets: only for images of at most 16384 tiles whose
        // lists are long on average (from the rectangle sizes) and uneven (the longest one at least 256 entries)
        if (bin.order && bin.tiles <= kOrderMaxTiles && s_k_upper >= kOrderMinMean * (uint32_t)bin.tiles &&
            biggest >= kOrderMinLongest) {
            __syncthreads();                      // the offsets written above are read back by other threads
            tile_order_by_one_cta(bin.offsets, bin.tiles, bin.order, s_buf);
            // the host reads the longest list length together with K: its top bit says "an order was written"
            // (lengths stay below 2^31), so that the compositing kernel is given the order only when there is one
            if (tid == 0) *bin.longest = biggest | kOrderWrittenBit;
        }
    }
}

// ================================================================================================
// Stage 3: key emission.
struct Plane { float A, B, C; };

// reference render.cu:140-152, `1.0 / det` in double.
__device__ __forceinline__ Plane depth_plane(float ax, float ay, float az, float bx, float by, float bz, float cx,
                                             float cy, float cz) {
    float det = add(add(mul(ax, sub(by, cy)), mul(bx, sub(cy, ay))), mul(cx, sub(ay, by)));
    float id = (float)__ddiv_rn(1.0, (double)det);
    Plane p;
    p.A = mul(add(add(mul(az, sub(by, cy)), mul(bz, sub(cy, ay))), mul(cz, sub(ay, by))), id);
    p.B = mul(add(add(mul(ax, sub(bz, cz)), mul(bx, sub(cz, az))), mul(cx, sub(az, bz))), id);
    p.C = mul(add(add(mul(ax, sub(mul(by, cz), mul(cy, bz))), mul(bx, sub(mul(cy, az), mul(ay, cz)))),
                  mul(cx, sub(mul(ay, bz), mul(by, az)))),
              id);
    return p;
}

__device__ __forceinline__ float plane_depth(const Plane& p, float x, float y) { return fma_(p.A, x, fma_(p.B, y, p.C)); }

// One Sutherland-Hodgman pass against an axis-aligned half-plane (reference render.cu:159-189).
template <int AXIS>
__device__ __forceinline__ int clip_pass(const float2* in, int n_in, float2* out, float bound) {
    auto dist = [&](const float2& p) -> float {
        if (AXIS == 0) return sub(p.x, bound);
        if (AXIS == 1) return sub(bound, p.x);
        if (AXIS == 2) return sub(p.y, bound);
        return sub(bound, p.y);
    };
    int n_out = 0;
    float2 p0 = in[n_in - 1];
    float d0 = dist(p0);
    bool in0 = d0 >= 0.f;
    for (int i = 0; i < n_in; i++) {
        float2 p1 = in[i];
        float d1 = dist(p1);
        bool in1 = d1 >= 0.f;
        if (in1 != in0) {
            float t = div(d0, sub(d0, d1));
            out[n_out++] = make_float2(fma_(t, sub(p1.x, p0.x), p0.x), fma_(t, sub(p1.y, p0.y), p0.y));
        }
        if (in1) out[n_out++] = p1;
        p0 = p1; d0 = d1; in0 = in1;
    }
    return n_out;
}

struct TriXYZ { float ax, ay, az, bx, by, bz, cx, cy, cz; };

__device__ float tile_key(const TriXYZ& v, const Plane& pl, int tx, int ty, int W, int H, int tw, int th) {
    const float xmin = sub(mul(div((float)(tx * tw), (float)W), 2.f), 1.f);
    const float xmax = sub(mul(div((float)((tx + 1) * tw), (float)W), 2.f), 1.f);
    const float ymin = sub(mul(div((float)(ty * th), (float)H), 2.f), 1.f);
    const float ymax = sub(mul(div((float)((ty + 1) * th), (float)H), 2.f), 1.f);
    // triangle entirely inside the tile: the clipper would return it unchanged
    const float lox = fminf(fminf(v.ax, v.bx), v.cx), hix = fmaxf(fmaxf(v.ax, v.bx), v.cx);
    const float loy = fminf(fminf(v.ay, v.by), v.cy), hiy = fmaxf(fmaxf(v.ay, v.by), v.cy);
    if (sub(lox, xmin) >= 0.f && sub(xmax, hix) >= 0.f && sub(loy, ymin) >= 0.f && sub(ymax, hiy) >= 0.f) {
        float md0 = fminf(FLT_MAX, plane_depth(pl, v.ax, v.ay));
        md0 = fminf(md0, plane_depth(pl, v.bx, v.by));
        return fminf(md0, plane_depth(pl, v.cx, v.cy));
    }
    float2 poly[8], buf[8];
    poly[0] = make_float2(v.ax, v.ay);
    poly[1] = make_float2(v.bx, v.by);
    poly[2] = make_float2(v.cx, v.cy);
    int n = clip_pass<0>(poly, 3, buf, xmin);
    if (n <= 0) return 1e30f;
    n = clip_pass<1>(buf, n, poly, xmax);
    if (n <= 0) return 1e30f;
    n = clip_pass<2>(poly, n, buf, ymin);
    if (n <= 0) return 1e30f;
    n = clip_pass<3>(buf, n, poly, ymax);
    if (n <= 0) return 1e30f;
    float md = FLT_MAX;
    for (int i = 0; i < n; i++) md = fminf(md, plane_depth(pl, poly[i].x, poly[i].y));
    return md;
}

// One CTA takes 256 consecutive triangles.  Phase 1 (a thread per triangle) gathers the vertices and
// stages rectangle, depth plane and first output slot in shared memory.  Phase 2 (a thread per
// OUTPUT entry) finds its triangle by binary search over the staged offsets, so that a triangle
// touching many tiles is spread over the whole CTA and no lane idles behind a long neighbour.
// When `hist.hist` is set the digits of the written keys are counted on the fly, which saves the
// radix sort its own histogram pass over the keys.
struct __align__(16) EmitTri {
    float ax, ay, az, bx, by, bz, cx, cy, cz;
    float A, B, C;
    int x0, y0, ny, pad;
};
struct EmitMat { float m[9]; };   // CULL only: the triangle's barycentric matrix (from its packed record)
constexpr int kEmitThreads = 256;

//
// DIRECT: the tile offsets are known already; every entry takes the next free slot of its tile
// (`tile_cursor`, arrival order) and is stored there as (ordered depth << 32 | triangle), ready for the
// per-tile sort.  `keys` is that array, `ids` is unused.
// CULL (with DIRECT): pairs that the culling preprocess_count_kernel did not count are skipped by the same test.
template <bool DIRECT, bool CULL>
__global__ void __launch_bounds__(kEmitThreads) emit_keys_kernel(const float4* __restrict__ vertices,
                                                                 const int* __restrict__ indices, int T, int W, int H,
                                                                 int tw, int th, int tiles_x, int tiles_y,
                                                                 const uint32_t* __restrict__ tri_offsets,
                                                                 uint64_t* __restrict__ keys, uint32_t* __restrict__ ids,
                                                                 uint32_t capacity, HistArgs hist,
                                                                 uint32_t* __restrict__ tile_cursor,
                                                                 const uint32_t* __restrict__ part_total,
                                                                 const float4* __restrict__ tri_geo, int packed) {
    __shared__ EmitTri s_tri[kEmitThreads];
    __shared__ EmitMat s_mat[CULL ? kEmitThreads : 1];
    __shared__ uint32_t s_off[kEmitThreads + 1];
    __shared__ uint32_t s_hist[DIRECT ? 1 : kMaxPasses * kRadix];     // digit counts of the radix route only
    __shared__ uint32_t s_warp_tot[kSortWarps];
    __shared__ bool s_last;
    const int tid = threadIdx.x;
    const int t0 = blockIdx.x * kEmitThreads;
    const int ntri = min(kEmitThreads, T - t0);
    if (!DIRECT && hist.hist)
        for (int i = tid; i < hist.passes * kRadix; i += kEmitThreads) s_hist[i] = 0;
    if (tid < ntri) {
        const int t = t0 + tid;
        int ia, ib, ic;
        if (packed) {
            const int4 f = reinterpret_cast<const int4*>(indices)[t];
            ia = f.x; ib = f.y; ic = f.z;
        } else {
            ia = indices[3 * (size_t)t]; ib = indices[3 * (size_t)t + 1]; ic = indices[3 * (size_t)t + 2];
        }
        const float4 a = vertices[ia], b = vertices[ib], c = vertices[ic];
        EmitTri e;
        e.ax = a.x; e.ay = a.y; e.az = a.z; e.bx = b.x; e.by = b.y; e.bz = b.z; e.cx = c.x; e.cy = c.y; e.cz = c.z;
        Rect r;
        if (tile_rect(a.x, a.y, b.x, b.y, c.x, c.y, W, H, tw, th, tiles_x, tiles_y, r)) {
            const Plane pl = depth_plane(a.x, a.y, a.z, b.x, b.y, b.z, c.x, c.y, c.z);
            e.A = pl.A; e.B = pl.B; e.C = pl.C;
        } else {
            e.A = e.B = e.C = 0.f;
        }
        e.x0 = r.x0; e.y0 = r.y0; e.ny = r.y1 - r.y0 + 1; e.pad = 0;
        s_tri[tid] = e;
        s_off[tid] = tri_offsets[t];
        if (CULL) {
            const float4 g0 = tri_geo[4 * (size_t)t], g1 = tri_geo[4 * (size_t)t + 1], g2 = tri_geo[4 * (size_t)t + 2];
            s_mat[tid] = {{g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w, g2.x}};
        }
    }
    // DIRECT: the offsets are local to the 256 triangles of the CTA and its total stands in a separate array
    if (tid == 0) s_off[ntri] = DIRECT ? part_total[blockIdx.x] : tri_offsets[t0 + ntri];
    __syncthreads();
    const uint32_t first = s_off[0], total = s_off[ntri] - first;
    for (uint32_t e = tid; e < total; e += kEmitThreads) {
        const uint32_t ge = first + e;
        // largest i in [0, ntri) with s_off[i] <= ge (triangles without entries have equal offsets)
        int lo = 0, hi = ntri;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= ge) lo = mid; else hi = mid;
        }
        const EmitTri& tr = s_tri[lo];
        const uint32_t local = ge - s_off[lo];
        const int tx = tr.x0 + (int)(local / (uint32_t)tr.ny), ty = tr.y0 + (int)(local % (uint32_t)tr.ny);
        if (CULL && !rect_may_cover(s_mat[lo].m, tile_pixel_rect(tx, ty, W, H, tw, th))) continue;
        const TriXYZ v = {tr.ax, tr.ay, tr.az, tr.bx, tr.by, tr.bz, tr.cx, tr.cy, tr.cz};
        const Plane pl = {tr.A, tr.B, tr.C};
        // DIRECT: the slot does not depend on the key, so its atomic (a round trip to L2) is issued first and
        // travels while the polygon is clipped
        uint32_t pos = 0;
        if (DIRECT) pos = atomicAdd(&tile_cursor[ty * tiles_x + tx], 1u);
        const float depth = tile_key(v, pl, tx, ty, W, H, tw, th);
        if (DIRECT) {
            if (pos < capacity) keys[pos] = ((uint64_t)float_to_ordered(depth) << 32) | (uint32_t)(t0 + lo);
            continue;
        }
        const uint64_t key = ((uint64_t)(uint32_t)(ty * tiles_x + tx) << 32) | float_to_ordered(depth);
        if (ge < capacity) {                       // the host guarantees K <= capacity before the result is used
            keys[ge] = key;
            ids[ge] = (uint32_t)(t0 + lo);
            if (hist.hist) hist_count(s_hist, key, hist);
        }
    }
    if (!DIRECT && hist.hist) {
        __syncthreads();
        hist_flush_and_finish(s_hist, s_warp_tot, &s_last, hist);
    }
}

// Inputs in the packed layout: colours and opacities as one [V,4] array, faces as [T,4] (fourth word 0).
__global__ void __launch_bounds__(256) pack_inputs_kernel(const float* __restrict__ colors,
                                                          const float* __restrict__ opacities,
                                                          const int* __restrict__ indices, int V, int T,
                                                          float4* __restrict__ rgba, int4* __restrict__ faces) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < V) rgba[i] = make_float4(colors[3 * (size_t)i], colors[3 * (size_t)i + 1], colors[3 * (size_t)i + 2], opacities[i]);
    if (i < T) faces[i] = make_int4(indices[3 * (size_t)i], indices[3 * (size_t)i + 1], indices[3 * (size_t)i + 2], 0);
}

// ================================================================================================
// Stage 5: tile ranges from the sorted keys.  Thread i looks at the boundary before entry i.
__global__ void __launch_bounds__(256) tile_ranges_kernel(const uint64_t* __restrict__ keys, uint32_t n, int tiles,
                                                          int* __restrict__ offsets) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > n) return;
    const int prev = (i == 0) ? -1 : (int)(keys[i - 1] >> 32);
    int cur = (i == n) ? tiles : (int)(keys[i] >> 32);
    if (cur > tiles) cur = tiles;
    for (int t = prev + 1; t <= cur; t++) offsets[t] = (int)i;
}

}  // namespace tg

// ================================================================================================
// host side
namespace tg_host {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
    return TG_ERR_CUDA;
}
const char* last_error() { return g_err; }

static int check_dims_internal(int T, int W, int H, int tw, int th) {
    TG_REQUIRE(T >= 0, "T < 0");
    TG_REQUIRE(W > 0 && H > 0, "image size must be positive");
    TG_REQUIRE(tw > 0 && th > 0, "tile size must be positive");
    TG_REQUIRE(tw * th <= 1024, "tile_width * tile_height must be <= 1024");
    return TG_OK;
}

// finished-CTA counter (4, zero on entry) + pad (4) + one total per CTA of 256 triangles
size_t preprocess_scan_scratch_bytes(int T) { return 8 + 4 * ((size_t)(T > 0 ? (T + 255) / 256 : 0) + 1); }

// Per-triangle records, CTA-local triangle offsets (`tri_offsets[T + 2]`: [t] local to the triangle's
// CTA of 256, [T] = K, [T + 1] = longest tile list), tile offsets in `tile_cursor[tiles]` and
// `offsets[tiles + 1]`.  The first word of `scratch` and `tile_cursor` must have been zeroed by the caller.
// Beyond kTileScanByLastCta tiles a device-wide scan makes the tile offsets, for which `tile_scan_scratch`
// (zeroed, tg_scan_scratch_bytes(tiles) bytes) is needed, and [T + 1] is set to UINT32_MAX (not known).
int preprocess_scan(const float* vertices, const int32_t* indices, const float* colors, const float* opacities, int T,
                    int W, int H, int tw, int th, float* tri_geo, float* tri_attr, uint32_t* tri_offsets, void* scratch,
                    uint32_t* status, uint32_t* tile_cursor, int32_t* offsets, void* tile_scan_scratch, bool cull,
                    bool packed, uint32_t* tile_order, cudaStream_t stream) {
    if (int s = check_dims_internal(T, W, H, tw, th)) return s;
    TG_REQUIRE(tri_offsets && scratch && status && tile_cursor && offsets, "null pointer");
    const int tiles_x = (W + tw - 1) / tw, tiles_y = (H + th - 1) / th;
    const int tiles = tiles_x * tiles_y;
    if (T == 0) {
        TG_CUDA(cudaMemsetAsync(tri_offsets, 0, sizeof(uint32_t) * 2, stream));
        TG_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int32_t) * ((size_t)tiles + 1), stream));
        return TG_OK;
    }
    TG_REQUIRE(vertices && indices && colors && (packed || opacities) && tri_geo && tri_attr, "null pointer");
    TG_REQUIRE(((uintptr_t)vertices & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 && ((uintptr_t)tri_attr & 15) == 0,
               "vertices / tri_geo / tri_attr must be 16-byte aligned");
    TG_REQUIRE(!packed || ((((uintptr_t)indices | (uintptr_t)colors) & 15) == 0),
               "packed faces [T,4] and colours [V,4] must be 16-byte aligned");
    const bool by_last_cta = tiles <= tg::kTileScanByLastCta;
    TG_REQUIRE(by_last_cta || tile_scan_scratch, "null tile scan scratch");
    const tg::TileBinArgs bin = {tile_cursor, offsets, (uint32_t*)scratch, tiles, by_last_cta ? 1 : 0,
                                 tri_offsets + T + 1, (uint32_t*)scratch + 2, tri_offsets + T,
                                 by_last_cta ? tile_order : nullptr};
    TG_REQUIRE(!cull || by_last_cta, "tile culling is limited to 65536 tiles");
    const int grid = (T + 255) / 256;
    const bool one_wave = grid <= 148 * 6;      // all CTAs resident at once at six per SM
#define TG_LAUNCH_PREPROCESS(CULLV, MINBV)                                                                             \
    tg::preprocess_count_kernel<CULLV, MINBV><<<grid, 256, 0, stream>>>(                                               \
        (const float4*)vertices, indices, colors, opacities, T, W, H, tw, th, tiles_x, tiles_y, (float4*)tri_geo,      \
        (float4*)tri_attr, tri_offsets, bin, packed ? 1 : 0)
    if (cull) {
        if (one_wave) TG_LAUNCH_PREPROCESS(true, 6); else TG_LAUNCH_PREPROCESS(true, TG_PREPROCESS_MINB_LARGE);
    } else {
        if (one_wave) TG_LAUNCH_PREPROCESS(false, 6); else TG_LAUNCH_PREPROCESS(false, TG_PREPROCESS_MINB_LARGE);
    }
#undef TG_LAUNCH_PREPROCESS
    TG_LAUNCH_CHECK("preprocess_count_kernel");
    if (!by_last_cta) {
        // counts -> offsets by the device-wide scan, then the cursors start at the offsets
        const int parts = (tiles + tg::kScanTile - 1) / tg::kScanTile;
        tg::scan_kernel<<<parts, tg::kScanThreads, 0, stream>>>(tile_cursor, (uint32_t*)offsets, tiles, parts,
                                                                 (uint32_t*)tile_scan_scratch,
                                                                 (uint64_t*)((char*)tile_scan_scratch + 8), status);
        TG_LAUNCH_CHECK("scan_kernel");
        TG_CUDA(cudaMemcpyAsync(tile_cursor, offsets, sizeof(uint32_t) * (size_t)tiles, cudaMemcpyDeviceToDevice, stream));
        TG_CUDA(cudaMemsetAsync(tri_offsets + T + 1, 0xff, sizeof(uint32_t), stream));
    }
    return TG_OK;
}

int emit_keys(const float* vertices, const int32_t* indices, int T, int W, int H, int tw, int th,
              const uint32_t* tri_offsets, uint64_t* keys, uint32_t* ids, uint32_t capacity, const tg::HistArgs& hist,
              cudaStream_t stream) {
    if (int s = check_dims_internal(T, W, H, tw, th)) return s;
    if (T == 0) return TG_OK;
    TG_REQUIRE(vertices && indices && tri_offsets && keys && ids, "null pointer");
    const int tiles_x = (W + tw - 1) / tw, tiles_y = (H + th - 1) / th;
    tg::emit_keys_kernel<false, false><<<(T + tg::kEmitThreads - 1) / tg::kEmitThreads, tg::kEmitThreads, 0, stream>>>(
        (const float4*)vertices, indices, T, W, H, tw, th, tiles_x, tiles_y, tri_offsets, keys, ids, capacity, hist,
        nullptr, nullptr, nullptr, 0);
    TG_LAUNCH_CHECK("emit_keys_kernel");
    return TG_OK;
}

// Entries written straight into their tile's segment of `entries` (capacity slots), unsorted within it.
// `tri_offsets` and `scan_scratch` as preprocess_scan left them (CTA-local offsets, CTA totals).
int emit_entries(const float* vertices, const int32_t* indices, int T, int W, int H, int tw, int th,
                 const uint32_t* tri_offsets, const void* scan_scratch, uint32_t* tile_cursor, uint64_t* entries,
                 uint32_t capacity, const float* tri_geo_for_cull, bool packed, cudaStream_t stream) {
    if (int s = check_dims_internal(T, W, H, tw, th)) return s;
    if (T == 0 || capacity == 0) return TG_OK;
    TG_REQUIRE(vertices && indices && tri_offsets && scan_scratch && tile_cursor && entries, "null pointer");
    const int tiles_x = (W + tw - 1) / tw, tiles_y = (H + th - 1) / th;
    const tg::HistArgs none = {nullptr, nullptr, 0, 0, 0};
    const int grid = (T + tg::kEmitThreads - 1) / tg::kEmitThreads;
    if (tri_geo_for_cull)
        tg::emit_keys_kernel<true, true><<<grid, tg::kEmitThreads, 0, stream>>>(
            (const float4*)vertices, indices, T, W, H, tw, th, tiles_x, tiles_y, tri_offsets, entries, nullptr, capacity,
            none, tile_cursor, (const uint32_t*)scan_scratch + 2, (const float4*)tri_geo_for_cull, packed ? 1 : 0);
    else
        tg::emit_keys_kernel<true, false><<<grid, tg::kEmitThreads, 0, stream>>>(
            (const float4*)vertices, indices, T, W, H, tw, th, tiles_x, tiles_y, tri_offsets, entries, nullptr, capacity,
            none, tile_cursor, (const uint32_t*)scan_scratch + 2, nullptr, packed ? 1 : 0);
    TG_LAUNCH_CHECK("emit_entries_kernel");
    return TG_OK;
}
static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace tg_host

extern "C" {

int tg_version(void) { return 1; }

unsigned long long tg_launch_count(void) { return tg_host::g_launches.load(std::memory_order_relaxed); }

const char* tg_last_error(void) { return tg_host::last_error(); }

const char* tg_status_string(int s) {
    switch (s) {
        case TG_OK: return "ok";
        case TG_ERR_BAD_ARG: return "bad argument";
        case TG_ERR_WORKSPACE: return "workspace too small";
        case TG_ERR_CAPACITY: return "list capacity exceeded";
        case TG_ERR_DEVICE_FLAG: return "device error flag set (a bounded wait ran out)";
        case TG_ERR_CUDA: return "CUDA error";
        default: return "unknown status";
    }
}

static int check_dims(int T, int W, int H, int tw, int th) {
    TG_REQUIRE(T >= 0, "T < 0");
    TG_REQUIRE(W > 0 && H > 0, "image size must be positive");
    TG_REQUIRE(tw > 0 && th > 0, "tile size must be positive");
    TG_REQUIRE(tw * th <= 1024, "tile_width * tile_height must be <= 1024");
    return TG_OK;
}

int tg_preprocess(const float* vertices, const int32_t* indices, const float* colors, const float* opacities, int T,
                  int W, int H, int tw, int th, uint32_t* tri_counts, int32_t* tri_rects, float* tri_geo,
                  float* tri_attr, tg_stream_t stream) {
    if (int s = check_dims(T, W, H, tw, th)) return s;
    if (T == 0) return TG_OK;
    TG_REQUIRE(vertices && indices && colors && opacities && tri_counts && tri_geo && tri_attr, "null pointer");
    TG_REQUIRE(((uintptr_t)vertices & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 && ((uintptr_t)tri_attr & 15) == 0 &&
                   ((uintptr_t)tri_rects & 15) == 0,
               "vertices / tri_geo / tri_attr / tri_rects must be 16-byte aligned");
    const int tiles_x = (W + tw - 1) / tw, tiles_y = (H + th - 1) / th;
    tg::preprocess_kernel<<<(T + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        (const float4*)vertices, indices, colors, opacities, T, W, H, tw, th, tiles_x, tiles_y, tri_counts,
        (int4*)tri_rects, (float4*)tri_geo, (float4*)tri_attr);
    TG_LAUNCH_CHECK("preprocess_kernel");
    return TG_OK;
}

size_t tg_scan_scratch_bytes(int n) {
    size_t parts = (size_t)((n > 0 ? n : 0) + tg::kScanTile - 1) / tg::kScanTile;
    return 8 + 8 * (parts + 1);
}

int tg_scan(const uint32_t* in, uint32_t* out, int n, void* scratch, size_t scratch_bytes, uint32_t* status,
            tg_stream_t stream) {
    TG_REQUIRE(n >= 0, "n < 0");
    TG_REQUIRE(out && scratch && status, "null pointer");
    TG_REQUIRE(((uintptr_t)scratch & 7) == 0, "scratch must be 8-byte aligned");
    if (scratch_bytes < tg_scan_scratch_bytes(n)) {
        tg_host::set_error("scan scratch: need %zu bytes, got %zu", tg_scan_scratch_bytes(n), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        TG_CUDA(cudaMemsetAsync(out, 0, sizeof(uint32_t), s));
        return TG_OK;
    }
    TG_REQUIRE(in != nullptr, "null pointer");
    const int parts = (n + tg::kScanTile - 1) / tg::kScanTile;
    TG_CUDA(cudaMemsetAsync(scratch, 0, tg_scan_scratch_bytes(n), s));
    tg::scan_kernel<<<parts, tg::kScanThreads, 0, s>>>(in, out, n, parts, (uint32_t*)scratch,
                                                      (uint64_t*)((char*)scratch + 8), status);
    TG_LAUNCH_CHECK("scan_kernel");
    return TG_OK;
}

// ---- prefix scan without caller-provided scratch ------------------------------------------------
// Some hosts of this library may not allocate device memory at the point where they need a scan:
// code running under a fixed memory budget that was carved up at start-up, a real-time loop that
// must not touch the allocator, or a plugin whose embedding application owns every allocation.
// For them the partition words of the look-back scan live in a fixed array inside the library
// image.  Every GPU that loads the library holds these 64 KB + 256 B until the process exits.
constexpr int kStaticScanMaxN = 1 << 24;                                         // elements per call
constexpr int kStaticScanMaxParts = (kStaticScanMaxN + tg::kScanTile - 1) / tg::kScanTile;
constexpr size_t kStaticScanBytes = 256 + 8 * ((size_t)kStaticScanMaxParts + 1);  // ticket (padded) + words
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScanBytes];

// In host code the array's name is only a handle; the device address has to be asked for, once per
// device, with that device current.
static int static_scan_scratch_address(void** out) {
    constexpr int kMaxDevices = 64;
    static std::atomic<void*> cache[kMaxDevices];
    int dev = 0;
    TG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        tg_host::set_error("device index %d outside the supported range", dev);
        return TG_ERR_BAD_ARG;
    }
    void* p = cache[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        TG_CUDA(cudaGetSymbolAddress(&p, g_static_scan_scratch));
        cache[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return TG_OK;
}

int tg_scan_static(const uint32_t* in, uint32_t* out, int n, uint32_t* status, tg_stream_t stream) {
    TG_REQUIRE(n >= 0, "n < 0");
    TG_REQUIRE(out && status, "null pointer");
    if (n > kStaticScanMaxN) {
        tg_host::set_error("tg_scan_static handles at most %d elements per call (got %d); use tg_scan with caller scratch",
                           kStaticScanMaxN, n);
        return TG_ERR_CAPACITY;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        TG_CUDA(cudaMemsetAsync(out, 0, sizeof(uint32_t), s));
        return TG_OK;
    }
    TG_REQUIRE(in != nullptr, "null pointer");
    void* scratch = nullptr;
    if (int st = static_scan_scratch_address(&scratch)) return st;
    const int parts = (n + tg::kScanTile - 1) / tg::kScanTile;
    // the array keeps what the previous call left: clear the ticket and the words this call uses
    TG_CUDA(cudaMemsetAsync(scratch, 0, 256 + 8 * ((size_t)parts + 1), s));
    tg::scan_kernel<<<parts, tg::kScanThreads, 0, s>>>(in, out, n, parts, (uint32_t*)scratch,
                                                      (uint64_t*)((char*)scratch + 256), status);
    TG_LAUNCH_CHECK("scan_kernel (static scratch)");
    return TG_OK;
}

int tg_pack_inputs(const float* colors, const float* opacities, const int32_t* indices, int V, int T, float* rgba,
                   int32_t* faces, tg_stream_t stream) {
    TG_REQUIRE(V >= 0 && T >= 0, "negative size");
    if (V == 0 && T == 0) return TG_OK;
    TG_REQUIRE((V == 0 || (colors && opacities && rgba)) && (T == 0 || (indices && faces)), "null pointer");
    TG_REQUIRE((((uintptr_t)rgba | (uintptr_t)faces) & 15) == 0, "rgba / faces must be 16-byte aligned");
    const int n = V > T ? V : T;
    tg::pack_inputs_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(colors, opacities, indices, V, T,
                                                                              (float4*)rgba, (int4*)faces);
    TG_LAUNCH_CHECK("pack_inputs_kernel");
    return TG_OK;
}

int tg_selftest_bounded_wait(void* scratch, size_t scratch_bytes, uint32_t* status, uint32_t spin_limit,
                             tg_stream_t stream) {
    TG_REQUIRE(scratch && status, "null pointer");
    TG_REQUIRE(((uintptr_t)scratch & 7) == 0 && scratch_bytes >= 32, "scratch: 32 bytes, 8-byte aligned");
    TG_REQUIRE(spin_limit >= 1 && spin_limit <= 4096, "spin_limit must be in 1..4096");
    cudaStream_t s = (cudaStream_t)stream;
    TG_CUDA(cudaMemsetAsync(scratch, 0, 32, s));
    tg::bounded_wait_selftest_kernel<<<1, 32, 0, s>>>((uint64_t*)scratch, status, spin_limit, (uint32_t*)scratch + 6);
    TG_LAUNCH_CHECK("bounded_wait_selftest_kernel");
    return TG_OK;
}

int tg_emit_keys(const float* vertices, const int32_t* indices, int T, int W, int H, int tw, int th,
                 const uint32_t* tri_offsets, uint64_t* keys, uint32_t* ids, uint32_t capacity, tg_stream_t stream) {
    const tg::HistArgs no_hist = {nullptr, nullptr, 0, 0, 0};
    return tg_host::emit_keys(vertices, indices, T, W, H, tw, th, tri_offsets, keys, ids, capacity, no_hist,
                              (cudaStream_t)stream);
}

int tg_tile_ranges(const uint64_t* sorted_keys, uint32_t n, int tiles, int32_t* offsets, tg_stream_t stream) {
    TG_REQUIRE(tiles > 0 && offsets, "bad tiles / offsets");
    TG_REQUIRE(n == 0 || sorted_keys, "null keys");
    TG_REQUIRE(n < 0x80000000u, "K must stay below 2^31");
    const uint32_t threads = n + 1;
    tg::tile_ranges_kernel<<<(threads + 255) / 256, 256, 0, (cudaStream_t)stream>>>(sorted_keys, n, tiles, offsets);
    TG_LAUNCH_CHECK("tile_ranges_kernel");
    return TG_OK;
}

}  // extern "C"
