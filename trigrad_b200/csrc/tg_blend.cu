// Stages 6 and 7: per-tile forward compositing and the backward (gradient) kernel.
//
// One CTA per tile, one thread per pixel (tile_w*tile_h threads rounded up to a warp multiple); a
// warp owns an 8x4 pixel block when the tile size allows it.  The tile's depth-sorted triangle
// list is streamed through shared memory in coalesced, vectorised chunks of packed 64-byte
// geometry records.  For every staged chunk each warp first rejects, with one lane per record, the
// records that cannot cover any of its 32 pixels (exact corner test on the same rounded
// arithmetic as the per-pixel test); only the survivors are tested per pixel.
//
// per_pixel_sort = true  (the reference default): each pixel keeps the nearest <= 32 covering
//     fragments by (interpolated depth, list position) and blends them in that order; further
//     batches of 32 follow while transmittance > threshold and blended < max_layers.  The ids of
//     the blended fragments can be saved per pixel so that the backward pass need not search again.
// per_pixel_sort = false: fragments are blended in list order; a pixel stops once its
//     transmittance is <= threshold, a warp skips chunks once all its lanes stopped (ballot) and
//     the CTA leaves the list as soon as every warp voted "done".
//
// Backward: per pixel the recorded fragments are walked last to first with the reference's
// recurrences; every lane adds its contribution with 128-bit vector reductions
// (red.global.add.v4.f32) into a packed per-vertex buffer (x, y, w, opacity | r, g, b, -) that a
// small kernel then unpacks into grad_vertices / grad_colors / grad_opacities.
#include "tg_common.cuh"

namespace tg {

constexpr int kChunk = 64;   // records staged per step (64 bytes each, 80 bytes apart in shared memory)

struct BlendParams {
    const float4* geo;
    const float4* attr;
    const int* ids;
    const int* offsets;
    int W, H, tw, th, tiles_x;
    float thr;
    int max_layers;
    // Optional launch order of the tiles (longest lists first, so that no heavy tile starts late): CTA b handles tile
    // order[b], or tile b when there is none (the stage entry points; lists too short or too even to bother).
    const uint32_t* order;
};

__device__ __forceinline__ int tile_of_block(const BlendParams& P) {
    return P.order != nullptr ? (int)P.order[blockIdx.x] : (int)blockIdx.x;
}

struct PixelAcc {
    float alpha = 1.f, r = 0.f, g = 0.f, b = 0.f, depth = 0.f, weight = 0.f;
    int blended = 0;
};

// Load the geometry record of triangle `id` straight from global memory (L1/L2 resident).
__device__ __forceinline__ void load_geo(const float4* geo, int id, float* m, float* w) {
    const float4 g0 = __ldg(geo + 4 * (size_t)id), g1 = __ldg(geo + 4 * (size_t)id + 1);
    const float4 g2 = __ldg(geo + 4 * (size_t)id + 2), g3 = __ldg(geo + 4 * (size_t)id + 3);
    m[0] = g0.x; m[1] = g0.y; m[2] = g0.z; m[3] = g0.w; m[4] = g1.x; m[5] = g1.y; m[6] = g1.z; m[7] = g1.w; m[8] = g2.x;
    w[0] = g3.x; w[1] = g3.y; w[2] = g3.z;
}

constexpr int kAttrQuads = TG_ATTR_WORDS / 4;
struct AttrRec { float o[3]; float c[9]; float iw[3]; int vid[3]; float xy[6]; };

// FULL = false loads only what the forward pass needs (opacities, colours, 1/w).
template <bool FULL>
__device__ __forceinline__ AttrRec load_attr(const float4* attr, int id) {
    const float4* q = attr + kAttrQuads * (size_t)id;
    const float4 q0 = __ldg(q), q1 = __ldg(q + 1), q2 = __ldg(q + 2), q3 = __ldg(q + 3);
    AttrRec a;
    a.o[0] = q0.x; a.o[1] = q0.y; a.o[2] = q0.z;
    a.c[0] = q0.w; a.c[1] = q1.x; a.c[2] = q1.y; a.c[3] = q1.z; a.c[4] = q1.w; a.c[5] = q2.x; a.c[6] = q2.y; a.c[7] = q2.z;
    a.c[8] = q2.w;
    a.iw[0] = q3.x; a.iw[1] = q3.y; a.iw[2] = q3.z;
    if (FULL) {
        const float4 q4 = __ldg(q + 4), q5 = __ldg(q + 5);
        a.vid[0] = __float_as_int(q3.w); a.vid[1] = __float_as_int(q4.x); a.vid[2] = __float_as_int(q4.y);
        a.xy[0] = q4.z; a.xy[1] = q4.w; a.xy[2] = q5.x; a.xy[3] = q5.y; a.xy[4] = q5.z; a.xy[5] = q5.w;
    }
    return a;
}

// process_forward of the reference (render.cu:417-453); every operation rounded separately, in the
// oracle's order, so that the image agrees bit for bit with it.  The four weighted interpolations
// share one correctly rounded reciprocal of their common denominator.
struct BlendedValues { float o_raw, cr, cg, cb, z, den; };

__device__ __forceinline__ BlendedValues blend_one(const Bary& b, const float* w, const AttrRec& a, PixelAcc& acc) {
    BlendedValues v;
    v.den = fma_(b.z, w[2], fma_(b.y, w[1], mul(b.x, w[0])));
    const float inv = __frcp_rn(v.den);
    auto weighted = [&](float a0, float a1, float a2) -> float {
        float nom = mul(mul(b.x, a0), w[0]);
        nom = fma_(mul(b.y, a1), w[1], nom);
        nom = fma_(mul(b.z, a2), w[2], nom);
        return mul(nom, inv);
    };
    v.o_raw = weighted(a.o[0], a.o[1], a.o[2]);
    const float o = fminf(fmaxf(v.o_raw, 0.f), kMaxOpacity);
    v.cr = weighted(a.c[0], a.c[3], a.c[6]);
    v.cg = weighted(a.c[1], a.c[4], a.c[7]);
    v.cb = weighted(a.c[2], a.c[5], a.c[8]);
    v.z = interp_rn(b, a.iw[0], a.iw[1], a.iw[2], 1.f, 1.f, 1.f);
    const float ao = mul(acc.alpha, o);
    acc.depth = add(acc.depth, mul(ao, v.z));
    acc.weight = add(acc.weight, ao);
    acc.r = add(acc.r, mul(ao, v.cr));
    acc.g = add(acc.g, mul(ao, v.cg));
    acc.b = add(acc.b, mul(ao, v.cb));
    acc.alpha = mul(acc.alpha, sub(1.f, o));
    acc.blended++;
    return v;
}

// NDC extent (pixel centres) of the active pixels of one warp.
using WarpRect = PixelRect;

struct TileCtx {
    int tile, start, end, ix, iy;
    bool active;
    float px, py;
    WarpRect rect;
};

// Pixel-centre coordinates need double arithmetic (one rounding, reference render.cu:561-562); the
// tile_w + tile_h distinct values of a tile are computed once by its first threads and shared.
constexpr int kMaxTileCoords = 1026;

__device__ __forceinline__ TileCtx tile_context(const BlendParams& P, float* s_coord) {
    TileCtx c;
    c.tile = tile_of_block(P);
    const int tx = c.tile % P.tiles_x, ty = c.tile / P.tiles_x;
    for (int i = threadIdx.x; i < P.tw + P.th; i += blockDim.x)
        s_coord[i] = (i < P.tw) ? pixel_coord(tx * P.tw + i, P.W) : pixel_coord(ty * P.th + (i - P.tw), P.H);
    int lx, ly;
    const bool blocks = (P.tw & 7) == 0 && (P.th & 3) == 0;
    int bx0 = 0, by0 = 0;
    if (blocks) {
        // a warp owns an 8x4 block of the tile: compact footprint, fewer records survive its cull
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, bpr = P.tw >> 3;
        bx0 = (warp % bpr) * 8;
        by0 = (warp / bpr) * 4;
        lx = bx0 + (lane & 7);
        ly = by0 + (lane >> 3);
    } else {
        lx = threadIdx.x % P.tw;
        ly = threadIdx.x / P.tw;
    }
    c.ix = tx * P.tw + lx;
    c.iy = ty * P.th + ly;
    c.active = (int)threadIdx.x < P.tw * P.th && c.ix < P.W && c.iy < P.H;
    // (a caller that walks no tile list - the queued backward, whose blocks need not be the forward's tiles - passes none)
    c.start = P.offsets ? P.offsets[c.tile] : 0;
    c.end = P.offsets ? P.offsets[c.tile + 1] : 0;
    __syncthreads();
    c.px = s_coord[min(lx, P.tw - 1)];
    c.py = s_coord[P.tw + min(ly, P.th - 1)];
    if (blocks) {
        // the coordinates grow with the index, so the extent of the block's pixels inside the image is given by
        // its first and last valid column and row
        const int nx = min(8, P.W - tx * P.tw - bx0), ny = min(4, P.H - ty * P.th - by0);
        if (nx > 0 && ny > 0 && (int)threadIdx.x < P.tw * P.th)
            c.rect = {s_coord[bx0], s_coord[bx0 + nx - 1], s_coord[P.tw + by0], s_coord[P.tw + by0 + ny - 1]};
        else
            c.rect = {INFINITY, -INFINITY, INFINITY, -INFINITY};
        return c;
    }
    float x0 = c.active ? c.px : INFINITY, x1 = c.active ? c.px : -INFINITY;
    float y0 = c.active ? c.py : INFINITY, y1 = c.active ? c.py : -INFINITY;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        x0 = fminf(x0, __shfl_xor_sync(0xffffffffu, x0, d));
        x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, d));
        y0 = fminf(y0, __shfl_xor_sync(0xffffffffu, y0, d));
        y1 = fmaxf(y1, __shfl_xor_sync(0xffffffffu, y1, d));
    }
    c.rect = {x0, x1, y0, y1};
    return c;
}

// Stage `n` records of the list starting at `first` into shared memory (ids + geometry).
// Staged records are 80 bytes apart (64 bytes of record, 16 of padding): with that stride the 32 lanes of a warp can
// each read "their" record with 16-byte loads without shared-memory bank conflicts (a 64-byte stride puts every
// second lane on the same banks), and the words of a record keep constant offsets from its base.
constexpr int kStagedQuads = 5;
__device__ __forceinline__ int staged_quad(int r, int q) { return kStagedQuads * r + q; }

__device__ __forceinline__ void stage_chunk(const BlendParams& P, int first, int n, float4* s_geo, int* s_id) {
    for (int i = threadIdx.x; i < n * 4; i += blockDim.x) {
        const int rec = i >> 2, q = i & 3;
        const int id = P.ids[first + rec];
        if (q == 0) s_id[rec] = id;
        s_geo[staged_quad(rec, q)] = __ldg(P.geo + 4 * (size_t)id + q);
    }
}

// The attribute quads the forward blend needs (opacities, colours, 1/w: the first four of the six), staged next to
// the geometry when the whole tile list fits in one chunk: the blend of the selected fragments then reads its
// records from shared memory instead of gathering 128 bytes per fragment and lane through L1.  Same 80-byte pitch.
__device__ __forceinline__ void stage_attr_chunk(const BlendParams& P, int first, int n, float4* s_attr) {
    for (int i = threadIdx.x; i < n * 4; i += blockDim.x) {
        const int rec = i >> 2, q = i & 3;
        const int id = P.ids[first + rec];
        s_attr[staged_quad(rec, q)] = __ldg(P.attr + kAttrQuads * (size_t)id + q);
    }
}
__device__ __forceinline__ AttrRec staged_attr(const float4* s_attr, int r) {
    const float4 q0 = s_attr[staged_quad(r, 0)], q1 = s_attr[staged_quad(r, 1)], q2 = s_attr[staged_quad(r, 2)],
                 q3 = s_attr[staged_quad(r, 3)];
    AttrRec a;
    a.o[0] = q0.x; a.o[1] = q0.y; a.o[2] = q0.z;
    a.c[0] = q0.w; a.c[1] = q1.x; a.c[2] = q1.y; a.c[3] = q1.z; a.c[4] = q1.w; a.c[5] = q2.x; a.c[6] = q2.y; a.c[7] = q2.z;
    a.c[8] = q2.w;
    a.iw[0] = q3.x; a.iw[1] = q3.y; a.iw[2] = q3.z;
    return a;
}

// A staged geometry record in registers (only the parts a caller uses are actually loaded).
struct StagedGeo {
    float m[9];
    float z[3];
    float w[3];
    float zlow;
};
__device__ __forceinline__ StagedGeo load_staged(const float4* s_geo, int r) {
    const float4 a = s_geo[staged_quad(r, 0)], b = s_geo[staged_quad(r, 1)], c = s_geo[staged_quad(r, 2)],
                 d = s_geo[staged_quad(r, 3)];
    StagedGeo g;
    g.m[0] = a.x; g.m[1] = a.y; g.m[2] = a.z; g.m[3] = a.w; g.m[4] = b.x; g.m[5] = b.y; g.m[6] = b.z; g.m[7] = b.w;
    g.m[8] = c.x; g.z[0] = c.y; g.z[1] = c.z; g.z[2] = c.w; g.w[0] = d.x; g.w[1] = d.y; g.w[2] = d.z; g.zlow = d.w;
    return g;
}

// Bit mask (64 records) of the staged records that may matter to this warp: the triangle may cover one
// of its pixels (corner test) and, when `depth_cut` is finite, its depth lower bound is below the cut
// (every lane already holds a full batch of nearer fragments otherwise).
__device__ __forceinline__ unsigned long long warp_cull(const float4* s_geo, int n, const WarpRect& R,
                                                        float depth_cut = INFINITY) {
    const int lane = lane_id();
    bool k0 = false, k1 = false;
    if (lane < n) {
        const StagedGeo g = load_staged(s_geo, lane);
        k0 = g.zlow < depth_cut && rect_may_cover(g.m, R);
    }
    if (lane + 32 < n) {
        const StagedGeo g = load_staged(s_geo, lane + 32);
        k1 = g.zlow < depth_cut && rect_may_cover(g.m, R);
    }
    const unsigned m0 = __ballot_sync(0xffffffffu, k0), m1 = __ballot_sync(0xffffffffu, k1);
    return (unsigned long long)m0 | ((unsigned long long)m1 << 32);
}

// 16-byte asynchronous copy global -> shared (completion awaited with cp_async_wait_all by the issuing thread, then
// made visible to the CTA by a barrier).
__device__ __forceinline__ void cp_async16(float4* smem_dst, const float4* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One selection sweep over the whole tile list (select_next_k_in_tile, reference render.cu:375-415):
// keeps the `bs` covered fragments smallest in (depth, j) among those after (lastDepth, lastJ).
// All threads of the CTA must call it; `go` says whether this thread collects.
// `s_attr`, when given, receives the attribute quads of the chunk as well (stage_attr_chunk).
// `s_geo2` / `s_id2`, when given, are a second pair of staging buffers: a list of more than one chunk is then streamed
// (CTAs of 256 threads: one quad per thread and chunk) - the records of chunk k + 1 travel by asynchronous copies
// while chunk k is processed, their ids having been fetched one iteration earlier still, and one barrier per chunk
// replaces the two of the load-then-process loop.
// (STREAM is a template parameter so that callers which never stream carry none of its state.)
template <bool STREAM = false>
__device__ __forceinline__ int select_sweep(const BlendParams& P, const TileCtx& c, bool go, int bs, float lastDepth,
                                            int lastJ, float* dl, int* jl, float4* s_geo, int* s_id,
                                            float4* s_attr = nullptr, float4* s_geo2 = nullptr, int* s_id2 = nullptr) {
    int found = 0;
    float dfar = -INFINITY;     // dl[found - 1]; -inf while the batch is empty, so the first fragment is appended
    const bool warp_go = __any_sync(0xffffffffu, go);
    const bool streamed = STREAM && s_geo2 != nullptr && c.end - c.start > kChunk && blockDim.x == 4 * kChunk;
    const int my_rec = threadIdx.x >> 2, my_q = threadIdx.x & 3;
    int id_ahead = -1;          // streamed: id of this thread's record in the chunk after the one being copied
    if (streamed) {
        __syncthreads();        // whoever read the buffers before (an earlier sweep) is done
        const int id = P.ids[c.start + my_rec];                       // chunk 0 is full: the list is longer
        if (my_q == 0) s_id[my_rec] = id;
        cp_async16(s_geo + staged_quad(my_rec, my_q), P.geo + 4 * (size_t)id + my_q);
        cp_async_commit();
        if (my_rec < c.end - c.start - kChunk) id_ahead = P.ids[c.start + kChunk + my_rec];
    }
    int chunk = 0;
    for (int first = c.start; first < c.end; first += kChunk, chunk++) {
        const int n = min(kChunk, c.end - first);
        const float4* geo_now = s_geo;          // the staged records of this chunk
        if (streamed) {
            float4* other_geo = s_geo2;         // buffers the next chunk is copied into
            int* other_id = s_id2;
            if (chunk & 1) { geo_now = s_geo2; other_geo = s_geo; other_id = s_id; }
            cp_async_wait_all();
            __syncthreads();    // this chunk has landed for everyone, and everyone has left the chunk before
            if (first + kChunk < c.end) {
                if (id_ahead >= 0) {
                    if (my_q == 0) other_id[my_rec] = id_ahead;
                    cp_async16(other_geo + staged_quad(my_rec, my_q), P.geo + 4 * (size_t)id_ahead + my_q);
                }
                cp_async_commit();
                const int first2 = first + 2 * kChunk;
                id_ahead = (first2 < c.end && my_rec < c.end - first2) ? P.ids[first2 + my_rec] : -1;
            }
        } else {
            __syncthreads();
            stage_chunk(P, first, n, s_geo, s_id);
            if (s_attr) stage_attr_chunk(P, first, n, s_attr);
            __syncthreads();
        }
        if (!warp_go) continue;
        // Once every collecting lane of the warp holds a full batch, a record whose depth lower bound is
        // not below the farthest kept depth of any lane cannot enter any lane's batch (ties lose).
        float cut = go ? ((found == bs) ? dfar : INFINITY) : -INFINITY;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) cut = fmaxf(cut, __shfl_xor_sync(0xffffffffu, cut, d));
        const unsigned long long mask = warp_cull(geo_now, n, c.rect, cut);
        // the two 32-bit halves of the mask one after the other: bit scans on 32-bit words are cheaper than on the
        // 64-bit one, and this loop runs once per surviving record and warp
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            unsigned bits = half ? (unsigned)(mask >> 32) : (unsigned)mask;
            while (bits) {
                const int r = __ffs((int)bits) - 1 + 32 * half;
                bits &= bits - 1;
                // all lanes read the same record: broadcast 16-byte loads
                const float4* rec = geo_now + kStagedQuads * r;
                const float4 q0 = rec[0], q1 = rec[1], q2 = rec[2];
                const float m[9] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x};
                const Bary b = apply_bary(m, c.px, c.py);
                // one minimum instead of three comparisons: fminf skips NaN operands, so the result is below
                // kEffZero exactly when one of the three is (and NaN, i.e. "covered", when all three are NaN)
                if (!go || fminf(fminf(b.x, b.y), b.z) < kEffZero) continue;
                const float4 q3 = rec[3];
                const float d = interp_rn(b, q2.y, q2.z, q2.w, q3.x, q3.y, q3.z);
                const int j = first + r;
                if (d < lastDepth) continue;
                if (d == lastDepth && j <= lastJ) continue;
                // the farthest kept depth stays in a register: lists come roughly front to back, so most
                // fragments go to the end of the batch (ties keep list order) or, once it is full, nowhere
                if (d >= dfar) {
                    if (found == bs) continue;
                    dl[found] = d;
                    jl[found] = j;
                    dfar = d;
                    found++;
                    continue;
                }
                int pos = (found < bs) ? found : (bs - 1);
                while (pos > 0 && d < dl[pos - 1]) {
                    dl[pos] = dl[pos - 1];
                    jl[pos] = jl[pos - 1];
                    pos--;
                }
                dl[pos] = d;
                jl[pos] = j;
                if (found < bs) found++;
                dfar = dl[found - 1];
            }
        }
    }
    return found;
}

__device__ __forceinline__ void store_pixel(const TileCtx& c, const BlendParams& P, PixelAcc& acc, float4* image,
                                            float* depthmap, float* final_w, int* ends) {
    if (!c.active) return;
    const size_t index = (size_t)c.iy * P.W + c.ix;
    float dm;
    if (acc.weight > kEffZero) dm = div(acc.depth, acc.weight);
    else { dm = INFINITY; acc.weight = 0.f; }
    depthmap[index] = dm;
    final_w[index] = acc.weight;
    ends[index] = acc.blended;
    image[index] = make_float4(acc.r, acc.g, acc.b, acc.alpha);
}

// sel: optional [planes][H*W] int32; plane k of a pixel receives the triangle id of its k-th blended
// fragment (k < ends).  Only written when it is not null (per-pixel mode, max_layers <= 32).
// STREAM: lists of more than one chunk are streamed through two staging buffers (select_sweep); instantiated
// separately because the state it carries costs the one-chunk tiles a few spilled registers.
template <bool SORT, int MAXT, bool STREAM = false>
__global__ void __launch_bounds__(MAXT, MAXT <= 256 ? 5 : 1) blend_forward_kernel(BlendParams P, float4* __restrict__ image,
                                                             float* __restrict__ depthmap, float* __restrict__ final_w,
                                                             int* __restrict__ ends, int* __restrict__ sel) {
    __shared__ float4 s_geo[kChunk * kStagedQuads];
    __shared__ float4 s_attr[SORT ? kChunk * kStagedQuads : 1];   // one-chunk lists: attributes; longer ones: 2nd buffer
    __shared__ int s_id[kChunk];
    __shared__ int s_id2[STREAM ? kChunk : 1];
    __shared__ float s_coord[kMaxTileCoords];
    const int this_tile = tile_of_block(P);
    if (P.offsets[this_tile] == P.offsets[this_tile + 1]) {
        // a tile without entries: background, and no need for pixel-centre coordinates (any pixel order will do)
        const int tx = this_tile % P.tiles_x, ty = this_tile / P.tiles_x;
        const int ix = tx * P.tw + (int)threadIdx.x % P.tw, iy = ty * P.th + (int)threadIdx.x / P.tw;
        if ((int)threadIdx.x < P.tw * P.th && ix < P.W && iy < P.H) {
            const size_t index = (size_t)iy * P.W + ix;
            depthmap[index] = INFINITY;
            final_w[index] = 0.f;
            ends[index] = 0;
            image[index] = make_float4(0.f, 0.f, 0.f, 1.f);
        }
        return;
    }
    const TileCtx c = tile_context(P, s_coord);
    PixelAcc acc;

    if (SORT) {
        float dl[kBatchLayers];
        int jl[kBatchLayers];
        float lastDepth = -INFINITY;
        int lastJ = -1;
        bool want = c.active;
        const size_t plane = (size_t)P.W * P.H, index = (size_t)c.iy * P.W + c.ix;
        while (true) {
            const bool go = want && acc.alpha > P.thr && acc.blended < P.max_layers;
            if (!__syncthreads_or(go)) break;
            const int bs = min(kBatchLayers, P.max_layers - acc.blended);
            // A list of one chunk is still in shared memory after the sweep, and then its attribute quads were staged
            // with it (while the geometry loads were in flight anyway): the blend reads its records from shared memory
            // instead of gathering 128 bytes per fragment and lane through L1.  (Deciding after the sweep, from the
            // number of pixels that found something, whether staging the attributes pays was slower: the loads then
            // wait alone behind a barrier.)
            const bool one_chunk = c.end - c.start <= kChunk;
            const int found = select_sweep<STREAM>(P, c, go, bs, lastDepth, lastJ, dl, jl, s_geo, s_id,
                                                   one_chunk ? s_attr : nullptr, one_chunk ? nullptr : s_attr, s_id2);
            if (go) {
                const int n = min(found, P.max_layers - acc.blended);
                for (int i = 0; i < n; i++) {
                    if (one_chunk) {
                        const int r = jl[i] - c.start;
                        const StagedGeo g = load_staged(s_geo, r);
                        const Bary b = apply_bary(g.m, c.px, c.py);
                        const AttrRec a = staged_attr(s_attr, r);
                        if (sel) sel[(size_t)acc.blended * plane + index] = s_id[r];
                        blend_one(b, g.w, a, acc);
                        continue;
                    }
                    const int id = P.ids[jl[i]];
                    float m[9], w[3];
                    load_geo(P.geo, id, m, w);
                    const Bary b = apply_bary(m, c.px, c.py);
                    const AttrRec a = load_attr<false>(P.attr, id);
                    if (sel) sel[(size_t)acc.blended * plane + index] = id;
                    blend_one(b, w, a, acc);
                }
                if (n > 0) {
                    lastDepth = dl[n - 1];
                    lastJ = jl[n - 1];
                }
                // fewer than a full batch found: the sweep saw every remaining fragment, nothing is left
                if (found < bs) want = false;
            }
            if (P.max_layers <= kBatchLayers) break;   // a single batch is all there can be: no second vote
        }
    } else {
        bool done = !c.active;
        for (int first = c.start; first < c.end; first += kChunk) {
            const int n = min(kChunk, c.end - first);
            __syncthreads();
            stage_chunk(P, first, n, s_geo, s_id);
            __syncthreads();
            // a warp whose lanes have all stopped skips the chunk
            if (!__all_sync(0xffffffffu, done)) {
                const unsigned long long mask = warp_cull(s_geo, n, c.rect);
#pragma unroll 1
                for (int half = 0; half < 2; half++) {      // 32-bit bit scans, as in select_sweep
                    unsigned bits = half ? (unsigned)(mask >> 32) : (unsigned)mask;
                    while (bits) {
                        const int r = __ffs((int)bits) - 1 + 32 * half;
                        bits &= bits - 1;
                        if (done) continue;
                        if (!(acc.alpha > P.thr && acc.blended < P.max_layers)) { done = true; continue; }
                        const float* g = reinterpret_cast<const float*>(s_geo + kStagedQuads * r);
                        const Bary b = apply_bary(g, c.px, c.py);
                        if (!covered(b)) continue;
                        const AttrRec a = load_attr<false>(P.attr, s_id[r]);
                        blend_one(b, g + 12, a, acc);
                    }
                }
                if (!(acc.alpha > P.thr && acc.blended < P.max_layers)) done = true;
            }
            if (__syncthreads_and(done)) break;
        }
    }
    store_pixel(c, P, acc, image, depthmap, final_w, ends);
}

// ------------------------------------------------------------------------------------------------
// Backward.

struct BackState { float alpha, sr = 0.f, sg = 0.f, sb = 0.f, oa = 0.f, zoa = 0.f; };

struct PixelGrad {
    float gr, gg, gb, ga, gd;          // upstream gradients of this pixel
    float final_alpha, final_weight, final_depth;
};

// Approximate reciprocal (1 ulp, one MUFU instruction): gradients carry a 1e-4 tolerance and float
// atomics already make their last bits run-dependent.
__device__ __forceinline__ float rcp_fast(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// One fragment's contribution to its triangle's three vertices: (x, y, w, opacity, r, g, b) each.
struct Contrib {
    float v[3][7];
    int vid[3];
};

// Packed per-vertex gradient accumulator: slot 0 = (d/dx, d/dy, d/dw, d/dopacity), slot 1 = (d/dr, d/dg, d/db, 0).
__device__ __forceinline__ void red_add_v4(float4* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d));
}

// process_backward of the reference (render.cu:455-538) for one fragment of one pixel; adds this
// pixel's contribution for the triangle's three vertices into `gpack`.  The interpolation VJPs
// (util.h:299-355) share 1/den; vertex-position gradients follow the reference's expanded partial
// derivatives (util.h:405-455) term by term: for small triangles their fp32 cancellation is
// systematic and part of what "the same result" means.
__device__ __forceinline__ void emit_contrib(const Contrib& c, float4* __restrict__ gpack) {
#pragma unroll
    for (int k = 0; k < 3; k++) {
        red_add_v4(gpack + 2 * (size_t)c.vid[k], c.v[k][0], c.v[k][1], c.v[k][2], c.v[k][3]);
        red_add_v4(gpack + 2 * (size_t)c.vid[k] + 1, c.v[k][4], c.v[k][5], c.v[k][6], 0.f);
    }
}

__device__ __forceinline__ void backward_one(const float* w, const AttrRec& a, const Bary& b, float px, float py,
                                             const PixelGrad& pg, BackState& st, Contrib& out) {
    const float bw0 = b.x * w[0], bw1 = b.y * w[1], bw2 = b.z * w[2];
    const float den = bw0 + bw1 + bw2;
    const bool ok = !(den * den < kEffZero);
    const float inv = rcp_fast(den);
    const float o_raw = (bw0 * a.o[0] + bw1 * a.o[1] + bw2 * a.o[2]) * inv;
    const float o = fminf(fmaxf(o_raw, 0.f), kMaxOpacity);
    const float cr = (bw0 * a.c[0] + bw1 * a.c[3] + bw2 * a.c[6]) * inv;
    const float cg = (bw0 * a.c[1] + bw1 * a.c[4] + bw2 * a.c[7]) * inv;
    const float cb = (bw0 * a.c[2] + bw1 * a.c[5] + bw2 * a.c[8]) * inv;
    const float iw0 = a.iw[0], iw1 = a.iw[1], iw2 = a.iw[2];
    const float denz = b.x + b.y + b.z;
    const bool okz = !(denz * denz < kEffZero);
    const float invz = rcp_fast(denz);
    const float z = (b.x * iw0 + b.y * iw1 + b.z * iw2) * invz;
    const float iom = rcp_fast(1.f - o);

    const float drgb_do = ((cr * st.alpha - st.sr) * pg.gr + (cg * st.alpha - st.sg) * pg.gg + (cb * st.alpha - st.sb) * pg.gb -
                           pg.ga * pg.final_alpha) * iom;
    st.alpha = st.alpha * iom;
    const float ao = st.alpha * o;
    st.sr += cr * ao;
    st.sg += cg * ao;
    st.sb += cb * ao;
    const float ddw_do = st.alpha - st.oa * iom;
    const float dud_do = st.alpha * z - st.zoa * iom;
    st.oa += ao;
    st.zoa += z * ao;
    const bool has_w = !(pg.final_weight < kEffZero);
    const float inv_fw = has_w ? rcp_fast(pg.final_weight) : 0.f;
    const float dd_do = (dud_do - pg.final_depth * ddw_do) * inv_fw * pg.gd;
    const float d_do = drgb_do + (has_w ? dd_do : 0.f);

    // upstream of the four weighted interpolations (0 where the reference's guard returns zeros)
    const float uo = ok ? d_do * inv : 0.f;
    const float ur = ok ? ao * pg.gr * inv : 0.f, ug = ok ? ao * pg.gg * inv : 0.f, ub = ok ? ao * pg.gb * inv : 0.f;
    // e_k = sum over attributes of upstream * (a_k - value): d/d(b_k w_k) of the interpolated values
    const float e0 = uo * (a.o[0] - o_raw) + ur * (a.c[0] - cr) + ug * (a.c[1] - cg) + ub * (a.c[2] - cb);
    const float e1 = uo * (a.o[1] - o_raw) + ur * (a.c[3] - cr) + ug * (a.c[4] - cg) + ub * (a.c[5] - cb);
    const float e2 = uo * (a.o[2] - o_raw) + ur * (a.c[6] - cr) + ug * (a.c[7] - cg) + ub * (a.c[8] - cb);
    // depth interpolation (values 1/w, unit weights)
    const float uz = (okz && has_w) ? ao * pg.gd * inv_fw * invz : 0.f;
    const float z0 = uz * (iw0 - z), z1 = uz * (iw1 - z), z2 = uz * (iw2 - z);
    const float g0 = w[0] * e0 + z0, g1 = w[1] * e1 + z1, g2 = w[2] * e2 + z2;       // d/d bary
    // d/dw: weighted interpolations, plus (as the reference does, render.cu:530) the gradient w.r.t. the unit
    // weights of the depth interpolation, plus the chain through the values 1/w
    const float gw0 = b.x * e0 + b.x * z0 - uz * b.x * iw0 * iw0;
    const float gw1 = b.y * e1 + b.y * z1 - uz * b.y * iw1 * iw1;
    const float gw2 = b.z * e2 + b.z * z2 - uz * b.z * iw2 * iw2;

    // barycentric_backward: l by cross products, then the expanded partials
    const float ax = a.xy[0], ay = a.xy[1], bx = a.xy[2], by = a.xy[3], cx = a.xy[4], cy = a.xy[5];
    float gxy[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float d = ax * (by - cy) + bx * (-ay + cy) + cx * (ay - by);
    if (!(fabsf(d) < kEffZero)) {
        const float iT = rcp_fast((bx - ax) * (cy - ay) - (by - ay) * (cx - ax));
        const float lx = ((bx - px) * (cy - py) - (by - py) * (cx - px)) * iT;
        const float ly = ((cx - px) * (ay - py) - (cy - py) * (ax - px)) * iT;
        const float lz = ((ax - px) * (by - py) - (ay - py) * (bx - px)) * iT;
        const float id = rcp_fast(d);
        gxy[0] = (g0 * (lx * (-by + cy)) + g1 * (-cy - ly * (by - cy) + py) + g2 * (by - lz * (by - cy) - py)) * id;
        gxy[1] = (g0 * (lx * (bx - cx)) + g1 * (cx + ly * (bx - cx) - px) + g2 * (-bx + lz * (bx - cx) + px)) * id;
        gxy[2] = (g0 * (cy + lx * (ay - cy) - py) + g1 * (ly * (ay - cy)) + g2 * (-ay + lz * (ay - cy) + py)) * id;
        gxy[3] = (g0 * (-cx - lx * (ax - cx) + px) + g1 * (ly * (-ax + cx)) + g2 * (ax - lz * (ax - cx) - px)) * id;
        gxy[4] = (g0 * (-by - lx * (ay - by) + py) + g1 * (ay - ly * (ay - by) - py) + g2 * (lz * (-ay + by))) * id;
        gxy[5] = (g0 * (bx + lx * (ax - bx) - px) + g1 * (-ax + ly * (ax - bx) + px) + g2 * (lz * (ax - bx))) * id;
    }
    const float gw[3] = {gw0, gw1, gw2}, bwk[3] = {bw0, bw1, bw2};
#pragma unroll
    for (int k = 0; k < 3; k++) {
        out.vid[k] = a.vid[k];
        out.v[k][0] = gxy[2 * k];
        out.v[k][1] = gxy[2 * k + 1];
        out.v[k][2] = gw[k];
        out.v[k][3] = uo * bwk[k];
        out.v[k][4] = ur * bwk[k];
        out.v[k][5] = ug * bwk[k];
        out.v[k][6] = ub * bwk[k];
    }
}

struct BackwardIn {
    const float4* gimage;
    const float* gdepth;
    const float4* image;
    const float* depthmap;
    const float* final_w;
    const int* ends;
    // fused mean-squared-error loss: when l2_target is set, the upstream gradient of the image is
    // l2_grad_scale * (image - target), the depth-map gradient is zero and the squared differences are
    // summed into l2_partials[64] (no gradient image is ever materialised)
    const float4* l2_target;
    float l2_grad_scale;
    float* l2_partials;
    // the same target as 8-bit RGBA (value / 255, correctly rounded division: what `u8.float() / 255` gives);
    // at most one of l2_target / l2_target_u8 is set
    const uchar4* l2_target_u8;
};
constexpr int kLossPartials = 64;

__device__ __forceinline__ int load_pixel_state(const TileCtx& c, const BlendParams& P, const BackwardIn& in,
                                                PixelGrad& pg, BackState& st, float* sq_diff = nullptr) {
    pg = PixelGrad{};
    st.alpha = 1.f;
    if (sq_diff) *sq_diff = 0.f;
    if (!c.active) return 0;
    const size_t index = (size_t)c.iy * P.W + c.ix;
    const float4 img = in.image[index];
    if (in.l2_target || in.l2_target_u8) {
        float4 t;
        if (in.l2_target_u8) {
            const uchar4 u = in.l2_target_u8[index];
            t = make_float4(__fdiv_rn((float)u.x, 255.f), __fdiv_rn((float)u.y, 255.f), __fdiv_rn((float)u.z, 255.f),
                            __fdiv_rn((float)u.w, 255.f));
        } else {
            t = in.l2_target[index];
        }
        const float dr = img.x - t.x, dg = img.y - t.y, db = img.z - t.z, da = img.w - t.w;
        pg.gr = in.l2_grad_scale * dr; pg.gg = in.l2_grad_scale * dg; pg.gb = in.l2_grad_scale * db;
        pg.ga = in.l2_grad_scale * da;
        pg.gd = 0.f;
        if (sq_diff) *sq_diff = dr * dr + dg * dg + db * db + da * da;
    } else {
        const float4 gi = in.gimage[index];
        pg.gr = gi.x; pg.gg = gi.y; pg.gb = gi.z; pg.ga = gi.w;
        pg.gd = in.gdepth ? in.gdepth[index] : 0.f;      // no depth-map gradient given: zero
    }
    pg.final_alpha = img.w;
    pg.final_weight = in.final_w[index];
    pg.final_depth = in.depthmap[index];
    st.alpha = pg.final_alpha;
    return min(in.ends[index], P.max_layers);
}

// Default mode with the per-pixel fragment ids saved by the forward pass: no list search, no shared
// memory, no barriers - every thread walks its own fragments last to first.
template <int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT <= 256 ? 4 : 1) blend_backward_saved_kernel(BlendParams P, BackwardIn in,
                                                                    const int* __restrict__ sel,
                                                                    float4* __restrict__ gpack) {
    __shared__ float s_coord[kMaxTileCoords];
    const TileCtx c = tile_context(P, s_coord);
    PixelGrad pg;
    BackState st;
    float sq = 0.f;
    const int n = load_pixel_state(c, P, in, pg, st, &sq);
    const size_t plane = (size_t)P.W * P.H, index = (size_t)c.iy * P.W + c.ix;
    const int lane = lane_id();
    if (in.l2_target || in.l2_target_u8) {
        // loss: warp sum, then one atomic per warp into one of 64 partial sums (spread addresses)
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
        if (lane == 0 && sq != 0.f) atomicAdd(in.l2_partials + ((blockIdx.x * 8 + (threadIdx.x >> 5)) & (kLossPartials - 1)), sq);
    }
    int nmax = n;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, d));
    // 2x2 pixel quads of the warp's 8x4 block: lanes L, L^1, L^8, L^9
    const unsigned quad = 0x303u << (lane & ~9);
    // ids are fetched one fragment ahead of their use
    int id_next = (n > 0) ? sel[(size_t)(n - 1) * plane + index] : 0;
    for (int s = 0; s < nmax; s++) {
        const int k = n - 1 - s;
        const bool has = k >= 0;
        const int id = has ? id_next : -1 - lane;          // distinct negatives never match
        if (k > 0) id_next = sel[(size_t)(k - 1) * plane + index];
        Contrib ct;
#pragma unroll
        for (int j = 0; j < 3; j++) {
            ct.vid[j] = 0;
#pragma unroll
            for (int q = 0; q < 7; q++) ct.v[j][q] = 0.f;
        }
        if (has) {
            float m[9], w[3];
            load_geo(P.geo, id, m, w);
            const AttrRec a = load_attr<true>(P.attr, id);
            const Bary b = apply_bary(m, c.px, c.py);
            backward_one(w, a, b, c.px, c.py, pg, st, ct);
        }
        // Pixels of one quad that hold the same triangle are summed with two shuffle rounds and one
        // lane issues the reductions: fewer, fuller vector atomics.
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        const bool full4 = has && ((peers & quad) == quad);
#pragma unroll
        for (int j = 0; j < 3; j++) {
#pragma unroll
            for (int q = 0; q < 7; q++) {
                float t = ct.v[j][q];
                t += __shfl_xor_sync(0xffffffffu, t, 1);
                t += __shfl_xor_sync(0xffffffffu, t, 8);
                if (full4) ct.v[j][q] = t;
            }
        }
        if (has && (!full4 || (lane & 9) == 0)) emit_contrib(ct, gpack);
    }
}

// ---- default mode, two-part gradient with a per-warp queue ------------------------------------------
// The pixels of a warp blend different numbers of fragments (on average fewer than half the lanes have
// one in a given round), and only the transmittance recurrence ties a pixel's fragments together.  So
// the work is split: part A (per pixel, back to front) runs the recurrence and produces the upstream
// gradients of the fragment's interpolations; these go into a queue in shared memory; part B (the
// expensive barycentric partials and the 21 per-vertex outputs) pops 32 queued fragments at a time and
// so runs with full warps.  The arithmetic per fragment is that of backward_one.  A warp whose lanes are
// busy anyway (deep overlap, or one opaque layer everywhere) skips the queue.
struct QueuedFragment {
    float px, py;
    int id;
    float bx, by, bz;
    float o_raw, cr, cg, cb, z;
    float uo, ur, ug, ub, uz;
};
constexpr int kQueueFields = 16, kQueueSlots = 64;

// Part A, second half: the transmittance recurrence of render.cu:455-538 for one fragment (back to
// front) and the upstream gradients of its interpolations.  inv_den / inv_denz are the reciprocals of
// the interpolation denominators, or 0 where the reference's guard returns zero gradients.
__device__ __forceinline__ void backward_recurrence(float o_raw, float cr, float cg, float cb, float z, float inv_den,
                                                    float inv_denz, const PixelGrad& pg, BackState& st,
                                                    QueuedFragment& f) {
    const float o = fminf(fmaxf(o_raw, 0.f), kMaxOpacity);
    const float iom = rcp_fast(1.f - o);
    const float drgb_do = ((cr * st.alpha - st.sr) * pg.gr + (cg * st.alpha - st.sg) * pg.gg + (cb * st.alpha - st.sb) * pg.gb -
                           pg.ga * pg.final_alpha) * iom;
    st.alpha = st.alpha * iom;
    const float ao = st.alpha * o;
    st.sr += cr * ao;
    st.sg += cg * ao;
    st.sb += cb * ao;
    const float ddw_do = st.alpha - st.oa * iom;
    const float dud_do = st.alpha * z - st.zoa * iom;
    st.oa += ao;
    st.zoa += z * ao;
    const bool has_w = !(pg.final_weight < kEffZero);
    const float inv_fw = has_w ? rcp_fast(pg.final_weight) : 0.f;
    const float dd_do = (dud_do - pg.final_depth * ddw_do) * inv_fw * pg.gd;
    const float d_do = drgb_do + (has_w ? dd_do : 0.f);
    f.o_raw = o_raw; f.cr = cr; f.cg = cg; f.cb = cb; f.z = z;
    f.uo = d_do * inv_den;
    f.ur = ao * pg.gr * inv_den;
    f.ug = ao * pg.gg * inv_den;
    f.ub = ao * pg.gb * inv_den;
    f.uz = has_w ? ao * pg.gd * inv_fw * inv_denz : 0.f;
}

// Part A: interpolations of the fragment (approximate reciprocals), then the recurrence.
__device__ __forceinline__ void backward_state(const float* w, const AttrRec& a, const Bary& b, const PixelGrad& pg,
                                               BackState& st, QueuedFragment& f) {
    const float bw0 = b.x * w[0], bw1 = b.y * w[1], bw2 = b.z * w[2];
    const float den = bw0 + bw1 + bw2;
    const bool ok = !(den * den < kEffZero);
    const float inv = rcp_fast(den);
    const float o_raw = (bw0 * a.o[0] + bw1 * a.o[1] + bw2 * a.o[2]) * inv;
    const float cr = (bw0 * a.c[0] + bw1 * a.c[3] + bw2 * a.c[6]) * inv;
    const float cg = (bw0 * a.c[1] + bw1 * a.c[4] + bw2 * a.c[7]) * inv;
    const float cb = (bw0 * a.c[2] + bw1 * a.c[5] + bw2 * a.c[8]) * inv;
    const float denz = b.x + b.y + b.z;
    const bool okz = !(denz * denz < kEffZero);
    const float invz = rcp_fast(denz);
    const float z = (b.x * a.iw[0] + b.y * a.iw[1] + b.z * a.iw[2]) * invz;
    f.bx = b.x; f.by = b.y; f.bz = b.z;
    backward_recurrence(o_raw, cr, cg, cb, z, ok ? inv : 0.f, okz ? invz : 0.f, pg, st, f);
}

// Part B: from the upstream gradients to the contribution for the triangle's three vertices.
__device__ __forceinline__ void backward_outputs(const float* w, const AttrRec& a, const QueuedFragment& f, Contrib& out) {
    const float uo = f.uo, ur = f.ur, ug = f.ug, ub = f.ub, uz = f.uz;
    const float e0 = uo * (a.o[0] - f.o_raw) + ur * (a.c[0] - f.cr) + ug * (a.c[1] - f.cg) + ub * (a.c[2] - f.cb);
    const float e1 = uo * (a.o[1] - f.o_raw) + ur * (a.c[3] - f.cr) + ug * (a.c[4] - f.cg) + ub * (a.c[5] - f.cb);
    const float e2 = uo * (a.o[2] - f.o_raw) + ur * (a.c[6] - f.cr) + ug * (a.c[7] - f.cg) + ub * (a.c[8] - f.cb);
    const float iw0 = a.iw[0], iw1 = a.iw[1], iw2 = a.iw[2];
    const float z0 = uz * (iw0 - f.z), z1 = uz * (iw1 - f.z), z2 = uz * (iw2 - f.z);
    const float g0 = w[0] * e0 + z0, g1 = w[1] * e1 + z1, g2 = w[2] * e2 + z2;
    const float gw0 = f.bx * e0 + f.bx * z0 - uz * f.bx * iw0 * iw0;
    const float gw1 = f.by * e1 + f.by * z1 - uz * f.by * iw1 * iw1;
    const float gw2 = f.bz * e2 + f.bz * z2 - uz * f.bz * iw2 * iw2;
    const float px = f.px, py = f.py;
    const float ax = a.xy[0], ay = a.xy[1], bx = a.xy[2], by = a.xy[3], cx = a.xy[4], cy = a.xy[5];
    float gxy[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float d = ax * (by - cy) + bx * (-ay + cy) + cx * (ay - by);
    if (!(fabsf(d) < kEffZero)) {
        const float iT = rcp_fast((bx - ax) * (cy - ay) - (by - ay) * (cx - ax));
        const float lx = ((bx - px) * (cy - py) - (by - py) * (cx - px)) * iT;
        const float ly = ((cx - px) * (ay - py) - (cy - py) * (ax - px)) * iT;
        const float lz = ((ax - px) * (by - py) - (ay - py) * (bx - px)) * iT;
        const float id = rcp_fast(d);
        gxy[0] = (g0 * (lx * (-by + cy)) + g1 * (-cy - ly * (by - cy) + py) + g2 * (by - lz * (by - cy) - py)) * id;
        gxy[1] = (g0 * (lx * (bx - cx)) + g1 * (cx + ly * (bx - cx) - px) + g2 * (-bx + lz * (bx - cx) + px)) * id;
        gxy[2] = (g0 * (cy + lx * (ay - cy) - py) + g1 * (ly * (ay - cy)) + g2 * (-ay + lz * (ay - cy) + py)) * id;
        gxy[3] = (g0 * (-cx - lx * (ax - cx) + px) + g1 * (ly * (-ax + cx)) + g2 * (ax - lz * (ax - cx) - px)) * id;
        gxy[4] = (g0 * (-by - lx * (ay - by) + py) + g1 * (ay - ly * (ay - by) - py) + g2 * (lz * (-ay + by))) * id;
        gxy[5] = (g0 * (bx + lx * (ax - bx) - px) + g1 * (-ax + ly * (ax - bx) + px) + g2 * (lz * (ax - bx))) * id;
    }
    const float gw[3] = {gw0, gw1, gw2}, bwk[3] = {f.bx * w[0], f.by * w[1], f.bz * w[2]};
#pragma unroll
    for (int k = 0; k < 3; k++) {
        out.vid[k] = a.vid[k];
        out.v[k][0] = gxy[2 * k];
        out.v[k][1] = gxy[2 * k + 1];
        out.v[k][2] = gw[k];
        out.v[k][3] = uo * bwk[k];
        out.v[k][4] = ur * bwk[k];
        out.v[k][5] = ug * bwk[k];
        out.v[k][6] = ub * bwk[k];
    }
}

// Part B for the fragments in queue slots first .. first + count - 1 (count <= 32), one per lane.
// Consecutive slots that hold the same triangle (neighbouring pixels mostly do) are summed over runs of
// up to four with two shuffle rounds before the vector reductions are issued (a third round, runs of
// eight, costs more in shuffles than it saves in reductions).
__device__ __forceinline__ void drain_queue(const BlendParams& P, float (*q)[kQueueSlots], int first, int count,
                                            float4* __restrict__ gpack) {
    const int lane = lane_id();
    const bool valid = lane < count;
    QueuedFragment f;
    const int slot = first + (valid ? lane : 0);
    f.px = q[0][slot]; f.py = q[1][slot]; f.id = __float_as_int(q[2][slot]);
    f.bx = q[3][slot]; f.by = q[4][slot]; f.bz = q[5][slot];
    f.o_raw = q[6][slot]; f.cr = q[7][slot]; f.cg = q[8][slot]; f.cb = q[9][slot]; f.z = q[10][slot];
    f.uo = q[11][slot]; f.ur = q[12][slot]; f.ug = q[13][slot]; f.ub = q[14][slot]; f.uz = q[15][slot];
    const int id = valid ? f.id : -1 - lane;
    Contrib ct;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        ct.vid[j] = 0;
#pragma unroll
        for (int k = 0; k < 7; k++) ct.v[j][k] = 0.f;
    }
    if (valid) {
        const float4 g3 = __ldg(P.geo + 4 * (size_t)id + 3);
        const float w[3] = {g3.x, g3.y, g3.z};
        const AttrRec a = load_attr<true>(P.attr, id);
        backward_outputs(w, a, f, ct);
    }
    // runs of equal triangle ids in lane order
    const int prev = __shfl_up_sync(0xffffffffu, id, 1);
    const unsigned heads = __ballot_sync(0xffffffffu, lane == 0 || prev != id);
    const unsigned above = (lane == 31) ? 1u : (heads >> (lane + 1));      // head flags of lanes lane+1 .. (bit 0 = next lane)
    const bool same1 = (above & 1u) == 0 && lane + 1 < 32;
    const bool same2 = (above & 3u) == 0 && lane + 2 < 32;
    const int run_start = 31 - __clz(heads & (0xffffffffu >> (31 - lane)));
#pragma unroll
    for (int j = 0; j < 3; j++) {
#pragma unroll
        for (int k = 0; k < 7; k++) {
            float t = ct.v[j][k], u;
            u = __shfl_down_sync(0xffffffffu, t, 1); if (same1) t += u;
            u = __shfl_down_sync(0xffffffffu, t, 2); if (same2) t += u;
            ct.v[j][k] = t;
        }
    }
    if (valid && ((lane - run_start) & 3) == 0) emit_contrib(ct, gpack);
}

// Whole fragments per round, for warps whose lanes are busy anyway.  Pixels of one 2x2 quad (lanes L, L^1,
// L^8, L^9 of the warp's 8x4 block) that hold the same triangle are summed before one lane issues the
// reductions.  Kept out of line so that it does not weigh on the register allocation of the queued path.
__device__ __noinline__ void backward_rounds_direct(const BlendParams& P, float px, float py, PixelGrad pg, BackState st,
                                                    int n, int nmax, int id_next, const int* __restrict__ sel_pixel,
                                                    size_t plane, float4* __restrict__ gpack) {
    const int lane = lane_id();
    const unsigned quad = 0x303u << (lane & ~9);
    for (int s = 0; s < nmax; s++) {
        const int k = n - 1 - s;
        const bool has = k >= 0;
        const int id = has ? id_next : -1 - lane;          // distinct negatives never match
        if (k > 0) id_next = sel_pixel[(size_t)(k - 1) * plane];
        Contrib ct;
#pragma unroll
        for (int j = 0; j < 3; j++) {
            ct.vid[j] = 0;
#pragma unroll
            for (int i = 0; i < 7; i++) ct.v[j][i] = 0.f;
        }
        if (has) {
            float m[9], w[3];
            load_geo(P.geo, id, m, w);
            const AttrRec a = load_attr<true>(P.attr, id);
            const Bary b = apply_bary(m, px, py);
            backward_one(w, a, b, px, py, pg, st, ct);
        }
        const unsigned peers = __match_any_sync(0xffffffffu, id);
        const bool full4 = has && ((peers & quad) == quad);
#pragma unroll
        for (int j = 0; j < 3; j++) {
#pragma unroll
            for (int i = 0; i < 7; i++) {
                float t = ct.v[j][i];
                t += __shfl_xor_sync(0xffffffffu, t, 1);
                t += __shfl_xor_sync(0xffffffffu, t, 8);
                if (full4) ct.v[j][i] = t;
            }
        }
        if (has && (!full4 || (lane & 9) == 0)) emit_contrib(ct, gpack);
    }
}

template <int MAXT>
__global__ void __launch_bounds__(MAXT, 1024 / MAXT) blend_backward_queued_kernel(BlendParams P, BackwardIn in,
                                                                        const int* __restrict__ sel,
                                                                        float4* __restrict__ gpack) {
    static_assert(MAXT % 32 == 0 && MAXT <= 256, "one queue per warp, at most 8 warps");
    __shared__ float s_coord[MAXT + 2];      // tile_w + tile_h <= tile_w * tile_h + 1 <= MAXT + 1
    __shared__ float s_queue[MAXT / 32][kQueueFields][kQueueSlots];
    const TileCtx c = tile_context(P, s_coord);
    PixelGrad pg;
    BackState st;
    float sq = 0.f;
    const int n = load_pixel_state(c, P, in, pg, st, &sq);
    const size_t plane = (size_t)P.W * P.H, index = (size_t)c.iy * P.W + c.ix;
    const int lane = lane_id();
    float (*q)[kQueueSlots] = s_queue[threadIdx.x >> 5];
    if (in.l2_target || in.l2_target_u8) {
        // loss: warp sum, then one atomic per warp into one of 64 partial sums (spread addresses)
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
        if (lane == 0 && sq != 0.f) atomicAdd(in.l2_partials + ((blockIdx.x * 8 + (threadIdx.x >> 5)) & (kLossPartials - 1)), sq);
    }
    int nmax = n;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, d));
    int nsum = n;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) nsum += __shfl_xor_sync(0xffffffffu, nsum, d);
    int id_next = (n > 0) ? sel[(size_t)(n - 1) * plane + index] : 0;   // ids are fetched one fragment ahead
    if (nsum * 10 >= nmax * 32 * 9) {
        // Nearly all lanes have a fragment in every round (90 % or more): the queue would cost more than the idle
        // lanes do.
        backward_rounds_direct(P, c.px, c.py, pg, st, n, nmax, id_next, sel + index, plane, gpack);
        return;
    }
    int queued = 0;                                    // uniform over the warp
    for (int s = 0; s < nmax; s++) {
        const int k = n - 1 - s;
        const bool has = k >= 0;
        const int id = id_next;
        if (k > 0) id_next = sel[(size_t)(k - 1) * plane + index];
        const unsigned pushing = __ballot_sync(0xffffffffu, has);
        if (has) {
            float m[9], w[3];
            load_geo(P.geo, id, m, w);
            const AttrRec a = load_attr<false>(P.attr, id);
            const Bary b = apply_bary(m, c.px, c.py);
            QueuedFragment f;
            backward_state(w, a, b, pg, st, f);
            const int slot = queued + __popc(pushing & ((1u << lane) - 1u));
            q[0][slot] = c.px; q[1][slot] = c.py; q[2][slot] = __int_as_float(id);
            q[3][slot] = f.bx; q[4][slot] = f.by; q[5][slot] = f.bz;
            q[6][slot] = f.o_raw; q[7][slot] = f.cr; q[8][slot] = f.cg; q[9][slot] = f.cb; q[10][slot] = f.z;
            q[11][slot] = f.uo; q[12][slot] = f.ur; q[13][slot] = f.ug; q[14][slot] = f.ub; q[15][slot] = f.uz;
        }
        queued += __popc(pushing);
        __syncwarp();
        if (queued >= 32) {
            queued -= 32;
            drain_queue(P, q, queued, 32, gpack);
            __syncwarp();
        }
    }
    if (queued > 0) drain_queue(P, q, 0, queued, gpack);
}

// ---- one optimisation step of one view in a single kernel -------------------------------------------
// Forward compositing (default mode, max_layers <= 32: a single batch) followed, in the same thread, by
// the backward of mean((image - target)^2).  The values the forward interpolates for every blended
// fragment (opacity, colour, 1/w, barycentrics) are kept in local memory and feed the recurrence
// directly: no second pass over geometry and attributes for it, no selection planes, no re-read of the
// image; the per-vertex outputs go through the per-warp queue as in blend_backward_queued_kernel.
template <int MAXT>
__global__ void __launch_bounds__(MAXT, 4) blend_step_l2_kernel(BlendParams P, float4* __restrict__ image,
                                                                float* __restrict__ depthmap, float* __restrict__ final_w,
                                                                int* __restrict__ ends, const float4* __restrict__ target,
                                                                float grad_scale, float* __restrict__ l2_partials,
                                                                float4* __restrict__ gpack) {
    static_assert(MAXT == 256, "the per-warp queues are sized for 8 warps");
    __shared__ float4 s_geo[kChunk * kStagedQuads];
    __shared__ int s_id[kChunk];
    __shared__ float s_coord[kMaxTileCoords];
    __shared__ float s_queue[MAXT / 32][kQueueFields][kQueueSlots];
    const TileCtx c = tile_context(P, s_coord);
    const int lane = lane_id();
    PixelAcc acc;
    float4 kept[kBatchLayers][3];   // per blended fragment: (b.x, b.y, b.z, o_raw), (cr, cg, cb, z), (1/den, 1/denz, id, -)
    int n = 0;
    {
        float dl[kBatchLayers];
        int jl[kBatchLayers];
        const bool go = c.active && acc.alpha > P.thr && P.max_layers > 0;
        if (__syncthreads_or(go)) {
            const int bs = min(kBatchLayers, P.max_layers);
            const int found = select_sweep(P, c, go, bs, -INFINITY, -1, dl, jl, s_geo, s_id);
            if (go) {
                n = min(found, P.max_layers);
                for (int i = 0; i < n; i++) {
                    const int id = P.ids[jl[i]];
                    float m[9], w[3];
                    load_geo(P.geo, id, m, w);
                    const Bary b = apply_bary(m, c.px, c.py);
                    const AttrRec a = load_attr<false>(P.attr, id);
                    const BlendedValues v = blend_one(b, w, a, acc);
                    const float denz = b.x + b.y + b.z;
                    kept[i][0] = make_float4(b.x, b.y, b.z, v.o_raw);
                    kept[i][1] = make_float4(v.cr, v.cg, v.cb, v.z);
                    kept[i][2] = make_float4((v.den * v.den < kEffZero) ? 0.f : rcp_fast(v.den),
                                             (denz * denz < kEffZero) ? 0.f : rcp_fast(denz), __int_as_float(id), 0.f);
                }
            }
        }
    }
    const float final_alpha = acc.alpha, out_r = acc.r, out_g = acc.g, out_b = acc.b;
    store_pixel(c, P, acc, image, depthmap, final_w, ends);   // normalises acc.weight to 0 where no depth exists

    // upstream gradient of the image and the pixel's squared error
    PixelGrad pg = PixelGrad{};
    BackState st;
    st.alpha = final_alpha;
    float sq = 0.f;
    if (c.active) {
        const float4 t = target[(size_t)c.iy * P.W + c.ix];
        const float dr = out_r - t.x, dg = out_g - t.y, db = out_b - t.z, da = final_alpha - t.w;
        pg.gr = grad_scale * dr; pg.gg = grad_scale * dg; pg.gb = grad_scale * db; pg.ga = grad_scale * da;
        pg.gd = 0.f;
        pg.final_alpha = final_alpha;
        pg.final_weight = acc.weight;
        pg.final_depth = (acc.weight > kEffZero) ? div(acc.depth, acc.weight) : INFINITY;
        sq = dr * dr + dg * dg + db * db + da * da;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
    if (lane == 0 && sq != 0.f) atomicAdd(l2_partials + ((blockIdx.x * 8 + (threadIdx.x >> 5)) & (kLossPartials - 1)), sq);

    float (*q)[kQueueSlots] = s_queue[threadIdx.x >> 5];
    int nmax = n;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, d));
    int queued = 0;                                    // uniform over the warp
    for (int s = 0; s < nmax; s++) {
        const int k = n - 1 - s;
        const bool has = k >= 0;
        const unsigned pushing = __ballot_sync(0xffffffffu, has);
        if (has) {
            const float4 k0 = kept[k][0], k1 = kept[k][1], k2 = kept[k][2];
            QueuedFragment f;
            f.bx = k0.x; f.by = k0.y; f.bz = k0.z;
            backward_recurrence(k0.w, k1.x, k1.y, k1.z, k1.w, k2.x, k2.y, pg, st, f);
            const int slot = queued + __popc(pushing & ((1u << lane) - 1u));
            q[0][slot] = c.px; q[1][slot] = c.py; q[2][slot] = k2.z;
            q[3][slot] = f.bx; q[4][slot] = f.by; q[5][slot] = f.bz;
            q[6][slot] = f.o_raw; q[7][slot] = f.cr; q[8][slot] = f.cg; q[9][slot] = f.cb; q[10][slot] = f.z;
            q[11][slot] = f.uo; q[12][slot] = f.ur; q[13][slot] = f.ug; q[14][slot] = f.ub; q[15][slot] = f.uz;
        }
        queued += __popc(pushing);
        __syncwarp();
        if (queued >= 32) {
            queued -= 32;
            drain_queue(P, q, queued, 32, gpack);
            __syncwarp();
        }
    }
    if (queued > 0) drain_queue(P, q, 0, queued, gpack);
}

// General path (any max_layers, both modes): searches the list again as the reference does.
template <bool SORT, int MAXT>
__global__ void __launch_bounds__(MAXT) blend_backward_kernel(BlendParams P, BackwardIn in, float4* __restrict__ gpack) {
    __shared__ float4 s_geo[kChunk * kStagedQuads];
    __shared__ int s_id[kChunk];
    __shared__ float s_coord[kMaxTileCoords];
    const TileCtx c = tile_context(P, s_coord);
    PixelGrad pg;
    BackState st;
    const int limit = load_pixel_state(c, P, in, pg, st);

    if (SORT) {
        float dl[kBatchLayers];
        int jl[kBatchLayers];
        float lastDepth = -INFINITY;
        int lastJ = -1;
        int remaining = limit;
        while (true) {
            const bool go = remaining > 0;
            if (!__syncthreads_or(go)) break;
            const int bs = min(kBatchLayers, remaining);
            const int found = select_sweep(P, c, go, bs, lastDepth, lastJ, dl, jl, s_geo, s_id);
            if (go) {
                const int n = min(found, remaining);
                for (int i = n - 1; i >= 0; --i) {          // reference render.cu:684-688
                    const int id = P.ids[jl[i]];
                    float m[9], w[3];
                    load_geo(P.geo, id, m, w);
                    const Bary b = apply_bary(m, c.px, c.py);
                    const AttrRec a = load_attr<true>(P.attr, id);
                    Contrib ct;
                    backward_one(w, a, b, c.px, c.py, pg, st, ct);
                    emit_contrib(ct, gpack);
                }
                if (n > 0) {
                    lastDepth = dl[n - 1];
                    lastJ = jl[n - 1];
                    remaining -= n;
                } else {
                    remaining = 0;
                }
            }
        }
    } else {
        // reference render.cu:659-666: the first `limit` list entries, front to back
        __shared__ int s_lim;
        if (threadIdx.x == 0) s_lim = 0;
        __syncthreads();
        if (limit > 0) atomicMax(&s_lim, limit);
        __syncthreads();
        const int cta_lim = min(s_lim, c.end - c.start);
        for (int first = 0; first < cta_lim; first += kChunk) {
            const int n = min(kChunk, cta_lim - first);
            __syncthreads();
            stage_chunk(P, c.start + first, n, s_geo, s_id);
            __syncthreads();
            if (!__any_sync(0xffffffffu, first < limit)) continue;
            unsigned long long mask = warp_cull(s_geo, n, c.rect);
            while (mask) {
                const int r = __ffsll((long long)mask) - 1;
                mask &= mask - 1;
                if (first + r >= limit) continue;
                const float* g = reinterpret_cast<const float*>(s_geo + kStagedQuads * r);
                const Bary b = apply_bary(g, c.px, c.py);
                if (!covered(b)) continue;
                const AttrRec a = load_attr<true>(P.attr, s_id[r]);
                Contrib ct;
                backward_one(g + 12, a, b, c.px, c.py, pg, st, ct);
                emit_contrib(ct, gpack);
            }
        }
    }
}

// ---- corrected gradients outside the default mode (an extension, not reference behaviour) -----------
// The reference's recurrences (render.cu:478-497) are written for a walk over a pixel's blended fragments from
// the last one to the first.  Its kernel does that only in the default mode: with per_pixel_sort = false it
// visits the first `ends` list entries front to back (render.cu:659-666), and beyond 32 layers it reverses the
// order inside each batch of 32 only (render.cu:673-693).  This kernel computes the gradient of what the forward
// pass actually blended, for any mode and any number of layers, without storing the sequence: it walks the
// fragments in FORWARD order and obtains the sums over the fragments behind the current one - the only thing
// the back-to-front walk is needed for - as (final value - running prefix), the final values being the forward
// outputs (image, final weight, depth map * final weight).
struct PrefixState { float alpha = 1.f, sr = 0.f, sg = 0.f, sb = 0.f, oa = 0.f, zoa = 0.f; };
struct PixelFinals { float r, g, b, depth_sum; };

__device__ __forceinline__ void backward_one_prefix(const float* w, const AttrRec& a, const Bary& b, float px, float py,
                                                    const PixelGrad& pg, const PixelFinals& fin, PrefixState& pf,
                                                    Contrib& out) {
    const float bw0 = b.x * w[0], bw1 = b.y * w[1], bw2 = b.z * w[2];
    const float den = bw0 + bw1 + bw2;
    const bool ok = !(den * den < kEffZero);
    const float inv = rcp_fast(den);
    QueuedFragment f;
    f.px = px; f.py = py; f.id = 0;
    f.bx = b.x; f.by = b.y; f.bz = b.z;
    f.o_raw = (bw0 * a.o[0] + bw1 * a.o[1] + bw2 * a.o[2]) * inv;
    f.cr = (bw0 * a.c[0] + bw1 * a.c[3] + bw2 * a.c[6]) * inv;
    f.cg = (bw0 * a.c[1] + bw1 * a.c[4] + bw2 * a.c[7]) * inv;
    f.cb = (bw0 * a.c[2] + bw1 * a.c[5] + bw2 * a.c[8]) * inv;
    const float denz = b.x + b.y + b.z;
    const bool okz = !(denz * denz < kEffZero);
    const float invz = rcp_fast(denz);
    f.z = (b.x * a.iw[0] + b.y * a.iw[1] + b.z * a.iw[2]) * invz;
    const float o = fminf(fmaxf(f.o_raw, 0.f), kMaxOpacity);
    const float iom = rcp_fast(1.f - o);
    const float alpha = pf.alpha;              // transmittance in front of this fragment
    const float ao = alpha * o;
    pf.sr += f.cr * ao; pf.sg += f.cg * ao; pf.sb += f.cb * ao;
    pf.oa += ao;
    pf.zoa += f.z * ao;
    pf.alpha = alpha * (1.f - o);
    // sums over the fragments behind this one
    const float sr = fin.r - pf.sr, sg = fin.g - pf.sg, sb = fin.b - pf.sb;
    const float oa = pg.final_weight - pf.oa, zoa = fin.depth_sum - pf.zoa;
    const float drgb_do = (f.cr * alpha - sr * iom) * pg.gr + (f.cg * alpha - sg * iom) * pg.gg +
                          (f.cb * alpha - sb * iom) * pg.gb - pg.ga * pg.final_alpha * iom;
    const float ddw_do = alpha - oa * iom;
    const float dud_do = alpha * f.z - zoa * iom;
    const bool has_w = !(pg.final_weight < kEffZero);
    const float inv_fw = has_w ? rcp_fast(pg.final_weight) : 0.f;
    const float d_do = drgb_do + (has_w ? (dud_do - pg.final_depth * ddw_do) * inv_fw * pg.gd : 0.f);
    const float inv_den = ok ? inv : 0.f;
    f.uo = d_do * inv_den;
    f.ur = ao * pg.gr * inv_den;
    f.ug = ao * pg.gg * inv_den;
    f.ub = ao * pg.gb * inv_den;
    f.uz = (has_w && okz) ? ao * pg.gd * inv_fw * invz : 0.f;
    backward_outputs(w, a, f, out);
}

template <bool SORT, int MAXT>
__global__ void __launch_bounds__(MAXT) blend_backward_corrected_kernel(BlendParams P, BackwardIn in,
                                                                        float4* __restrict__ gpack) {
    __shared__ float4 s_geo[kChunk * kStagedQuads];
    __shared__ int s_id[kChunk];
    __shared__ float s_coord[kMaxTileCoords];
    const TileCtx c = tile_context(P, s_coord);
    PixelGrad pg;
    BackState unused;
    const int limit = load_pixel_state(c, P, in, pg, unused);
    PixelFinals fin = {0.f, 0.f, 0.f, 0.f};
    if (c.active) {
        const float4 img = in.image[(size_t)c.iy * P.W + c.ix];
        fin.r = img.x; fin.g = img.y; fin.b = img.z;
        fin.depth_sum = (pg.final_weight < kEffZero) ? 0.f : pg.final_depth * pg.final_weight;
    }
    PrefixState pf;

    if (SORT) {
        float dl[kBatchLayers];
        int jl[kBatchLayers];
        float lastDepth = -INFINITY;
        int lastJ = -1;
        int remaining = limit;
        while (true) {
            const bool go = remaining > 0;
            if (!__syncthreads_or(go)) break;
            const int bs = min(kBatchLayers, remaining);
            const int found = select_sweep(P, c, go, bs, lastDepth, lastJ, dl, jl, s_geo, s_id);
            if (go) {
                const int n = min(found, remaining);
                for (int i = 0; i < n; ++i) {
                    const int id = P.ids[jl[i]];
                    float m[9], w[3];
                    load_geo(P.geo, id, m, w);
                    const Bary b = apply_bary(m, c.px, c.py);
                    const AttrRec a = load_attr<true>(P.attr, id);
                    Contrib ct;
                    backward_one_prefix(w, a, b, c.px, c.py, pg, fin, pf, ct);
                    emit_contrib(ct, gpack);
                }
                if (n > 0) {
                    lastDepth = dl[n - 1];
                    lastJ = jl[n - 1];
                    remaining -= n;
                } else {
                    remaining = 0;
                }
            }
        }
    } else {
        // the forward's walk (render.cu:578-581): list order, covered entries only, until `limit` are done
        int processed = 0;
        bool done = limit <= 0;
        for (int first = c.start; first < c.end; first += kChunk) {
            const int n = min(kChunk, c.end - first);
            __syncthreads();
            stage_chunk(P, first, n, s_geo, s_id);
            __syncthreads();
            if (!__all_sync(0xffffffffu, done)) {
                unsigned long long mask = warp_cull(s_geo, n, c.rect);
                while (mask) {
                    const int r = __ffsll((long long)mask) - 1;
                    mask &= mask - 1;
                    if (done) continue;
                    const float* g = reinterpret_cast<const float*>(s_geo + kStagedQuads * r);
                    const Bary b = apply_bary(g, c.px, c.py);
                    if (!covered(b)) continue;
                    const AttrRec a = load_attr<true>(P.attr, s_id[r]);
                    Contrib ct;
                    backward_one_prefix(g + 12, a, b, c.px, c.py, pg, fin, pf, ct);
                    emit_contrib(ct, gpack);
                    if (++processed >= limit) done = true;
                }
            }
            if (__syncthreads_and(done)) break;
        }
    }
}

// Packed accumulator -> the three gradient tensors of the reference (render.cu:789-791).
__global__ void __launch_bounds__(256) unpack_gradients_kernel(const float4* __restrict__ gpack, int V,
                                                               float4* __restrict__ gV, float* __restrict__ gC,
                                                               float* __restrict__ gO, int accumulate,
                                                               const float* __restrict__ l2_partials, float l2_loss_scale,
                                                               float* __restrict__ l2_loss_out) {
    if (l2_loss_out && blockIdx.x == 0 && threadIdx.x < 32) {
        float x = l2_partials[threadIdx.x] + l2_partials[threadIdx.x + 32];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
        if (threadIdx.x == 0) *l2_loss_out = (accumulate ? *l2_loss_out : 0.f) + x * l2_loss_scale;
    }
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    const float4 a = gpack[2 * (size_t)v], b = gpack[2 * (size_t)v + 1];
    float4 ov = make_float4(a.x, a.y, 0.f, a.z);
    float c0 = b.x, c1 = b.y, c2 = b.z, o = a.w;
    if (accumulate) {
        const float4 old = gV[v];
        ov.x += old.x; ov.y += old.y; ov.z = old.z; ov.w += old.w;
        c0 += gC[3 * (size_t)v]; c1 += gC[3 * (size_t)v + 1]; c2 += gC[3 * (size_t)v + 2];
        o += gO[v];
    }
    gV[v] = ov;
    gC[3 * (size_t)v] = c0; gC[3 * (size_t)v + 1] = c1; gC[3 * (size_t)v + 2] = c2;
    gO[v] = o;
}

// The same for the packed input layout: colour and opacity gradients as one [V,4] array (dr, dg, db, dopacity).
__global__ void __launch_bounds__(256) unpack_gradients_rgba_kernel(const float4* __restrict__ gpack, int V,
                                                                    float4* __restrict__ gV, float4* __restrict__ gRGBA,
                                                                    int accumulate, const float* __restrict__ l2_partials,
                                                                    float l2_loss_scale, float* __restrict__ l2_loss_out) {
    if (l2_loss_out && blockIdx.x == 0 && threadIdx.x < 32) {
        float x = l2_partials[threadIdx.x] + l2_partials[threadIdx.x + 32];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
        if (threadIdx.x == 0) *l2_loss_out = (accumulate ? *l2_loss_out : 0.f) + x * l2_loss_scale;
    }
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    const float4 a = gpack[2 * (size_t)v], b = gpack[2 * (size_t)v + 1];
    float4 ov = make_float4(a.x, a.y, 0.f, a.z), oc = make_float4(b.x, b.y, b.z, a.w);
    if (accumulate) {
        const float4 pv = gV[v], pc = gRGBA[v];
        ov.x += pv.x; ov.y += pv.y; ov.z = pv.z; ov.w += pv.w;
        oc.x += pc.x; oc.y += pc.y; oc.z += pc.z; oc.w += pc.w;
    }
    gV[v] = ov;
    gRGBA[v] = oc;
}

}  // namespace tg

extern "C" {

static int blend_args(int W, int H, int tw, int th, int max_layers) {
    TG_REQUIRE(W > 0 && H > 0 && tw > 0 && th > 0, "sizes must be positive");
    TG_REQUIRE(tw * th <= 1024, "tile_width * tile_height must be <= 1024");
    TG_REQUIRE(max_layers >= 1, "max_layers must be >= 1");
    return TG_OK;
}

static tg::BlendParams make_params(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids,
                                   const int32_t* offsets, int W, int H, int tw, int th, float thr, int max_layers) {
    tg::BlendParams P;
    P.geo = (const float4*)tri_geo; P.attr = (const float4*)tri_attr; P.ids = sorted_ids; P.offsets = offsets;
    P.W = W; P.H = H; P.tw = tw; P.th = th; P.tiles_x = (W + tw - 1) / tw;
    P.thr = thr; P.max_layers = max_layers;
    P.order = nullptr;
    return P;
}

int tg_selection_planes(int per_pixel_sort, int max_layers) {
    return (per_pixel_sort && max_layers >= 1 && max_layers <= tg::kBatchLayers) ? max_layers : 0;
}

}  // extern "C"

namespace tg_host {
// Set by tg_render_forward / tg_render_step_l2 around their compositing call (same thread): the tile order the
// binning kernel left in the workspace.  The stage entry points run with the identity order.
static thread_local const uint32_t* g_tile_order = nullptr;
static thread_local uint32_t g_longest_list = 0;
void set_tile_order(const uint32_t* order, uint32_t longest_list) {
    g_tile_order = order;
    g_longest_list = longest_list;
}
}  // namespace tg_host

extern "C" {

int tg_blend_forward(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                     int W, int H, int tw, int th, float thr, int per_pixel_sort, int max_layers, float* image,
                     float* depthmap, float* final_weights, int32_t* ends, int32_t* selection, tg_stream_t stream) {
    if (int s = blend_args(W, H, tw, th, max_layers)) return s;
    TG_REQUIRE(offsets && image && depthmap && final_weights && ends, "null pointer");
    TG_REQUIRE(((uintptr_t)image & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 && ((uintptr_t)tri_attr & 15) == 0,
               "image / tri_geo / tri_attr must be 16-byte aligned");
    if (tg_selection_planes(per_pixel_sort, max_layers) == 0) selection = nullptr;
    tg::BlendParams P = make_params(tri_geo, tri_attr, sorted_ids, offsets, W, H, tw, th, thr, max_layers);
    P.order = tg_host::g_tile_order;
    const int tiles = P.tiles_x * ((H + th - 1) / th);
    const int threads = ((tw * th + 31) / 32) * 32;
    cudaStream_t s = (cudaStream_t)stream;
    float4* img = (float4*)image;
    if (threads <= 256) {
        // lists well beyond one staged chunk (the binning kernel of the same call reported the longest): stream them
        if (per_pixel_sort && threads == 256 && tg_host::g_longest_list > 2u * tg::kChunk)
            tg::blend_forward_kernel<true, 256, true><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends, selection);
        else if (per_pixel_sort) tg::blend_forward_kernel<true, 256><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends, selection);
        else tg::blend_forward_kernel<false, 256><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends, nullptr);
    } else {
        if (per_pixel_sort) tg::blend_forward_kernel<true, 1024><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends, selection);
        else tg::blend_forward_kernel<false, 1024><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends, nullptr);
    }
    TG_LAUNCH_CHECK("blend_forward_kernel");
    return TG_OK;
}

size_t tg_backward_scratch_bytes(int V) { return (size_t)(V > 0 ? V : 0) * 32 + 512; }

static int backward_impl(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                         int V, int W, int H, int tw, int th, int per_pixel_sort, int max_layers,
                         const float* grad_image, const float* grad_depthmap, const void* l2_target, bool target_u8,
                         float l2_grad_scale,
                         float l2_loss_scale, float* l2_loss_out, const float* image, const float* depthmap,
                         const float* final_weights, const int32_t* ends, const int32_t* selection, float* grad_vertices,
                         float* grad_colors, float* grad_opacities, int accumulate, void* scratch, size_t scratch_bytes,
                         tg_stream_t stream) {
    if (int s = blend_args(W, H, tw, th, max_layers)) return s;
    TG_REQUIRE(V >= 0, "V < 0");
    TG_REQUIRE(offsets && image && depthmap && final_weights && ends, "null pointer");
    TG_REQUIRE(l2_target || grad_image, "null upstream gradient");
    if (V == 0) return TG_OK;
    const bool packed = accumulate == TG_ACCUMULATE_PACKED;   // gradients stay in the scratch, which keeps accumulating
    TG_REQUIRE(scratch && (packed || (grad_vertices && grad_colors && grad_opacities)), "null gradient / scratch pointer");
    TG_REQUIRE(((uintptr_t)image & 15) == 0 && ((uintptr_t)grad_image & 15) == 0 &&
                   ((uintptr_t)l2_target & (target_u8 ? 3 : 15)) == 0 &&
                   ((uintptr_t)tri_geo & 15) == 0 && ((uintptr_t)tri_attr & 15) == 0 &&
                   ((uintptr_t)grad_vertices & 15) == 0 && ((uintptr_t)scratch & 15) == 0,
               "image / grad_image / target / tri_geo / tri_attr / grad_vertices / scratch must be 16-byte aligned");
    if (scratch_bytes < tg_backward_scratch_bytes(V)) {
        tg_host::set_error("backward scratch: need %zu bytes, got %zu", tg_backward_scratch_bytes(V), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    const bool saved = selection != nullptr && tg_selection_planes(per_pixel_sort, max_layers) > 0;
    TG_REQUIRE(!l2_target || saved, "the fused L2 backward needs the selection saved by the forward pass (default mode)");
    cudaStream_t s = (cudaStream_t)stream;
    float4* gpack = (float4*)scratch;
    float* partials = (float*)((char*)scratch + (size_t)V * 32);
    if (!packed) TG_CUDA(cudaMemsetAsync(gpack, 0, (size_t)V * 32 + sizeof(float) * tg::kLossPartials, s));
    const tg::BlendParams P = make_params(tri_geo, tri_attr, sorted_ids, offsets, W, H, tw, th, 0.f, max_layers);
    const int tiles = P.tiles_x * ((H + th - 1) / th);
    const int threads = ((tw * th + 31) / 32) * 32;
    const tg::BackwardIn in = {(const float4*)grad_image, grad_depthmap, (const float4*)image, depthmap, final_weights,
                               ends, target_u8 ? nullptr : (const float4*)l2_target, l2_grad_scale, partials,
                               target_u8 ? (const uchar4*)l2_target : nullptr};
    if (threads <= 256) {
        if (saved) {
            // The queued kernel walks the per-pixel selection, not the tile lists, so its blocks need not be the
            // forward's tiles: 16x8 pixels (four warps) finish more evenly than whole tiles do, and a block's
            // registers come free only when its slowest warp is done (config 3: 179 -> 173 µs; 64 threads the
            // same, 32 threads slower again).
            tg::BlendParams Q = P;
            Q.tw = 16; Q.th = 8;
            Q.tiles_x = (W + Q.tw - 1) / Q.tw;
            Q.offsets = nullptr; Q.ids = nullptr; Q.order = nullptr;
            const int blocks = Q.tiles_x * ((H + Q.th - 1) / Q.th);
            tg::blend_backward_queued_kernel<128><<<blocks, 128, 0, s>>>(Q, in, selection, gpack);
        }
        else if (per_pixel_sort) tg::blend_backward_kernel<true, 256><<<tiles, threads, 0, s>>>(P, in, gpack);
        else tg::blend_backward_kernel<false, 256><<<tiles, threads, 0, s>>>(P, in, gpack);
    } else {
        if (saved) tg::blend_backward_saved_kernel<1024><<<tiles, threads, 0, s>>>(P, in, selection, gpack);
        else if (per_pixel_sort) tg::blend_backward_kernel<true, 1024><<<tiles, threads, 0, s>>>(P, in, gpack);
        else tg::blend_backward_kernel<false, 1024><<<tiles, threads, 0, s>>>(P, in, gpack);
    }
    TG_LAUNCH_CHECK("blend_backward_kernel");
    if (packed) return TG_OK;
    tg::unpack_gradients_kernel<<<(V + 255) / 256, 256, 0, s>>>(gpack, V, (float4*)grad_vertices, grad_colors,
                                                              grad_opacities, accumulate, partials, l2_loss_scale,
                                                              l2_target ? l2_loss_out : nullptr);
    TG_LAUNCH_CHECK("unpack_gradients_kernel");
    return TG_OK;
}

int tg_blend_step_l2(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets, int V,
                     int W, int H, int tw, int th, float thr, int max_layers, const float* target, float grad_scale,
                     float loss_scale, float* loss_out, float* image, float* depthmap, float* final_weights, int32_t* ends,
                     float* grad_vertices, float* grad_colors, float* grad_opacities, int accumulate, void* scratch,
                     size_t scratch_bytes, tg_stream_t stream) {
    if (int s = blend_args(W, H, tw, th, max_layers)) return s;
    TG_REQUIRE(tw * th <= 256 && max_layers <= tg::kBatchLayers,
               "the one-kernel step needs tiles of at most 256 pixels and max_layers <= 32 "
               "(otherwise: tg_blend_forward + tg_blend_backward_l2)");
    TG_REQUIRE(V > 0, "V must be positive");
    const bool packed = accumulate == TG_ACCUMULATE_PACKED;
    TG_REQUIRE(offsets && image && depthmap && final_weights && ends && target && (packed || loss_out), "null pointer");
    TG_REQUIRE(scratch && (packed || (grad_vertices && grad_colors && grad_opacities)), "null gradient / scratch pointer");
    TG_REQUIRE(((uintptr_t)image & 15) == 0 && ((uintptr_t)target & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 &&
                   ((uintptr_t)tri_attr & 15) == 0 && ((uintptr_t)grad_vertices & 15) == 0 && ((uintptr_t)scratch & 15) == 0,
               "image / target / tri_geo / tri_attr / grad_vertices / scratch must be 16-byte aligned");
    if (scratch_bytes < tg_backward_scratch_bytes(V)) {
        tg_host::set_error("backward scratch: need %zu bytes, got %zu", tg_backward_scratch_bytes(V), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    float4* gpack = (float4*)scratch;
    float* partials = (float*)((char*)scratch + (size_t)V * 32);
    if (!packed) TG_CUDA(cudaMemsetAsync(gpack, 0, (size_t)V * 32 + sizeof(float) * tg::kLossPartials, s));
    tg::BlendParams P = make_params(tri_geo, tri_attr, sorted_ids, offsets, W, H, tw, th, thr, max_layers);
    P.order = tg_host::g_tile_order;
    const int tiles = P.tiles_x * ((H + th - 1) / th);
    const int threads = ((tw * th + 31) / 32) * 32;
    tg::blend_step_l2_kernel<256><<<tiles, threads, 0, s>>>(P, (float4*)image, depthmap, final_weights, ends,
                                                            (const float4*)target, grad_scale, partials, gpack);
    TG_LAUNCH_CHECK("blend_step_l2_kernel");
    if (packed) return TG_OK;
    tg::unpack_gradients_kernel<<<(V + 255) / 256, 256, 0, s>>>(gpack, V, (float4*)grad_vertices, grad_colors,
                                                              grad_opacities, accumulate, partials, loss_scale, loss_out);
    TG_LAUNCH_CHECK("unpack_gradients_kernel");
    return TG_OK;
}

int tg_unpack_gradients(const void* scratch, size_t scratch_bytes, int V, float loss_scale, float* loss_out,
                        float* grad_vertices, float* grad_colors, float* grad_opacities, int accumulate,
                        tg_stream_t stream) {
    TG_REQUIRE(V > 0, "V must be positive");
    TG_REQUIRE(scratch && grad_vertices && grad_colors && grad_opacities, "null pointer");
    TG_REQUIRE(accumulate == 0 || accumulate == 1, "accumulate must be 0 or 1");
    TG_REQUIRE(((uintptr_t)grad_vertices & 15) == 0 && ((uintptr_t)scratch & 15) == 0,
               "grad_vertices / scratch must be 16-byte aligned");
    if (scratch_bytes < tg_backward_scratch_bytes(V)) {
        tg_host::set_error("backward scratch: need %zu bytes, got %zu", tg_backward_scratch_bytes(V), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    const float* partials = (const float*)((const char*)scratch + (size_t)V * 32);
    tg::unpack_gradients_kernel<<<(V + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        (const float4*)scratch, V, (float4*)grad_vertices, grad_colors, grad_opacities, accumulate, partials, loss_scale,
        loss_out);
    TG_LAUNCH_CHECK("unpack_gradients_kernel");
    return TG_OK;
}

int tg_unpack_gradients_rgba(const void* scratch, size_t scratch_bytes, int V, float loss_scale, float* loss_out,
                             float* grad_vertices, float* grad_rgba, int accumulate, tg_stream_t stream) {
    TG_REQUIRE(V > 0, "V must be positive");
    TG_REQUIRE(scratch && grad_vertices && grad_rgba, "null pointer");
    TG_REQUIRE(accumulate == 0 || accumulate == 1, "accumulate must be 0 or 1");
    TG_REQUIRE((((uintptr_t)grad_vertices | (uintptr_t)grad_rgba | (uintptr_t)scratch) & 15) == 0,
               "grad_vertices / grad_rgba / scratch must be 16-byte aligned");
    if (scratch_bytes < tg_backward_scratch_bytes(V)) {
        tg_host::set_error("backward scratch: need %zu bytes, got %zu", tg_backward_scratch_bytes(V), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    const float* partials = (const float*)((const char*)scratch + (size_t)V * 32);
    tg::unpack_gradients_rgba_kernel<<<(V + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        (const float4*)scratch, V, (float4*)grad_vertices, (float4*)grad_rgba, accumulate, partials, loss_scale, loss_out);
    TG_LAUNCH_CHECK("unpack_gradients_rgba_kernel");
    return TG_OK;
}

int tg_blend_backward(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                      int V, int W, int H, int tw, int th, int per_pixel_sort, int max_layers, const float* grad_image,
                      const float* grad_depthmap, const float* image, const float* depthmap, const float* final_weights,
                      const int32_t* ends, const int32_t* selection, float* grad_vertices, float* grad_colors,
                      float* grad_opacities, int accumulate, void* scratch, size_t scratch_bytes, tg_stream_t stream) {
    TG_REQUIRE(grad_image, "null upstream gradient");
    return backward_impl(tri_geo, tri_attr, sorted_ids, offsets, V, W, H, tw, th, per_pixel_sort, max_layers, grad_image,
                         grad_depthmap, nullptr, false, 0.f, 0.f, nullptr, image, depthmap, final_weights, ends, selection,
                         grad_vertices, grad_colors, grad_opacities, accumulate, scratch, scratch_bytes, stream);
}

int tg_blend_backward_corrected(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids,
                                const int32_t* offsets, int V, int W, int H, int tw, int th, int per_pixel_sort,
                                int max_layers, const float* grad_image, const float* grad_depthmap, const float* image,
                                const float* depthmap, const float* final_weights, const int32_t* ends,
                                float* grad_vertices, float* grad_colors, float* grad_opacities, int accumulate,
                                void* scratch, size_t scratch_bytes, tg_stream_t stream) {
    if (int s = blend_args(W, H, tw, th, max_layers)) return s;
    TG_REQUIRE(V >= 0, "V < 0");
    TG_REQUIRE(offsets && image && depthmap && final_weights && ends && grad_image, "null pointer");
    if (V == 0) return TG_OK;
    TG_REQUIRE(accumulate == 0 || accumulate == 1, "accumulate must be 0 or 1");
    TG_REQUIRE(scratch && grad_vertices && grad_colors && grad_opacities, "null gradient / scratch pointer");
    TG_REQUIRE(((uintptr_t)image & 15) == 0 && ((uintptr_t)grad_image & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 &&
                   ((uintptr_t)tri_attr & 15) == 0 && ((uintptr_t)grad_vertices & 15) == 0 && ((uintptr_t)scratch & 15) == 0,
               "image / grad_image / tri_geo / tri_attr / grad_vertices / scratch must be 16-byte aligned");
    if (scratch_bytes < tg_backward_scratch_bytes(V)) {
        tg_host::set_error("backward scratch: need %zu bytes, got %zu", tg_backward_scratch_bytes(V), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    float4* gpack = (float4*)scratch;
    float* partials = (float*)((char*)scratch + (size_t)V * 32);
    TG_CUDA(cudaMemsetAsync(gpack, 0, (size_t)V * 32 + sizeof(float) * tg::kLossPartials, s));
    const tg::BlendParams P = make_params(tri_geo, tri_attr, sorted_ids, offsets, W, H, tw, th, 0.f, max_layers);
    const int tiles = P.tiles_x * ((H + th - 1) / th);
    const int threads = ((tw * th + 31) / 32) * 32;
    const tg::BackwardIn in = {(const float4*)grad_image, grad_depthmap, (const float4*)image, depthmap, final_weights,
                               ends, nullptr, 0.f, partials, nullptr};
    if (threads <= 256) {
        if (per_pixel_sort) tg::blend_backward_corrected_kernel<true, 256><<<tiles, threads, 0, s>>>(P, in, gpack);
        else tg::blend_backward_corrected_kernel<false, 256><<<tiles, threads, 0, s>>>(P, in, gpack);
    } else {
        if (per_pixel_sort) tg::blend_backward_corrected_kernel<true, 1024><<<tiles, threads, 0, s>>>(P, in, gpack);
        else tg::blend_backward_corrected_kernel<false, 1024><<<tiles, threads, 0, s>>>(P, in, gpack);
    }
    TG_LAUNCH_CHECK("blend_backward_corrected_kernel");
    tg::unpack_gradients_kernel<<<(V + 255) / 256, 256, 0, s>>>(gpack, V, (float4*)grad_vertices, grad_colors,
                                                              grad_opacities, accumulate, partials, 0.f, nullptr);
    TG_LAUNCH_CHECK("unpack_gradients_kernel");
    return TG_OK;
}

int tg_blend_backward_l2(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                         int V, int W, int H, int tw, int th, int per_pixel_sort, int max_layers, const float* target,
                         float grad_scale, float loss_scale, float* loss_out, const float* image, const float* depthmap,
                         const float* final_weights, const int32_t* ends, const int32_t* selection, float* grad_vertices,
                         float* grad_colors, float* grad_opacities, int accumulate, void* scratch, size_t scratch_bytes,
                         tg_stream_t stream) {
    TG_REQUIRE(target && (loss_out || accumulate == TG_ACCUMULATE_PACKED), "null target / loss pointer");
    return backward_impl(tri_geo, tri_attr, sorted_ids, offsets, V, W, H, tw, th, per_pixel_sort, max_layers, nullptr,
                         nullptr, target, false, grad_scale, loss_scale, loss_out, image, depthmap, final_weights, ends,
                         selection, grad_vertices, grad_colors, grad_opacities, accumulate, scratch, scratch_bytes, stream);
}

int tg_blend_backward_l2_u8(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                            int V, int W, int H, int tw, int th, int per_pixel_sort, int max_layers,
                            const uint8_t* target_rgba8, float grad_scale, float loss_scale, float* loss_out,
                            const float* image, const float* depthmap, const float* final_weights, const int32_t* ends,
                            const int32_t* selection, float* grad_vertices, float* grad_colors, float* grad_opacities,
                            int accumulate, void* scratch, size_t scratch_bytes, tg_stream_t stream) {
    TG_REQUIRE(target_rgba8 && (loss_out || accumulate == TG_ACCUMULATE_PACKED), "null target / loss pointer");
    return backward_impl(tri_geo, tri_attr, sorted_ids, offsets, V, W, H, tw, th, per_pixel_sort, max_layers, nullptr,
                         nullptr, target_rgba8, true, grad_scale, loss_scale, loss_out, image, depthmap, final_weights, ends,
                         selection, grad_vertices, grad_colors, grad_opacities, accumulate, scratch, scratch_bytes, stream);
}

}  // extern "C"
