// Stages 6 and 7: per-tile forward compositing and the backward (gradient) kernel.
//
// One CTA per tile, one thread per pixel (tile_w*tile_h threads rounded up to a warp multiple).
// The tile's depth-sorted triangle list is streamed through shared memory in coalesced,
// vectorised chunks of packed 64-byte geometry records; every pixel tests every staged record.
//
// per_pixel_sort = true  (the reference default): each pixel keeps the nearest <= 32 covering
//     fragments by (interpolated depth, list position), then blends them in that order; further
//     batches of 32 follow while transmittance > threshold and blended < max_layers.
// per_pixel_sort = false: fragments are blended in list order; a pixel stops once its
//     transmittance is <= threshold, a whole warp skips records once all its lanes stopped and the
//     CTA leaves the list as soon as every warp voted "done".
#include "tg_common.cuh"

namespace tg {

constexpr int kChunk = 64;   // records staged per step: 64 x 64 B = 4 KB

struct BlendParams {
    const float4* geo;
    const float4* attr;
    const int* ids;
    const int* offsets;
    int W, H, tw, th, tiles_x;
    float thr;
    int max_layers;
};

struct PixelAcc {
    float alpha = 1.f, r = 0.f, g = 0.f, b = 0.f, depth = 0.f, weight = 0.f;
    int blended = 0;
};

struct Frag {
    Bary bary;
    float w0, w1, w2;
};

// Load the geometry record of triangle `id` straight from global memory (L1/L2 resident).
__device__ __forceinline__ void load_geo(const float4* geo, int id, float* m, float* z, float* w) {
    const float4 g0 = __ldg(geo + 4 * (size_t)id), g1 = __ldg(geo + 4 * (size_t)id + 1);
    const float4 g2 = __ldg(geo + 4 * (size_t)id + 2), g3 = __ldg(geo + 4 * (size_t)id + 3);
    m[0] = g0.x; m[1] = g0.y; m[2] = g0.z; m[3] = g0.w; m[4] = g1.x; m[5] = g1.y; m[6] = g1.z; m[7] = g1.w; m[8] = g2.x;
    z[0] = g2.y; z[1] = g2.z; z[2] = g2.w;
    w[0] = g3.x; w[1] = g3.y; w[2] = g3.z;
}

constexpr int kAttrQuads = TG_ATTR_WORDS / 4;
struct AttrRec { float o[3]; float c[9]; int vid[3]; float xy[6]; };

// FULL = false loads only what the forward pass needs (opacities and colours).
template <bool FULL>
__device__ __forceinline__ AttrRec load_attr(const float4* attr, int id) {
    const float4* q = attr + kAttrQuads * (size_t)id;
    const float4 q0 = __ldg(q), q1 = __ldg(q + 1), q2 = __ldg(q + 2);
    AttrRec a;
    a.o[0] = q0.x; a.o[1] = q0.y; a.o[2] = q0.z;
    a.c[0] = q0.w; a.c[1] = q1.x; a.c[2] = q1.y; a.c[3] = q1.z; a.c[4] = q1.w; a.c[5] = q2.x; a.c[6] = q2.y; a.c[7] = q2.z;
    a.c[8] = q2.w;
    if (FULL) {
        const float4 q3 = __ldg(q + 3), q4 = __ldg(q + 4), q5 = __ldg(q + 5);
        a.vid[0] = __float_as_int(q3.x); a.vid[1] = __float_as_int(q3.y); a.vid[2] = __float_as_int(q3.z);
        a.xy[0] = q4.x; a.xy[1] = q4.y; a.xy[2] = q4.z; a.xy[3] = q4.w; a.xy[4] = q5.x; a.xy[5] = q5.y;
    }
    return a;
}

// process_forward of the reference (render.cu:417-453); every operation rounded separately so the
// image agrees bit for bit with the oracle.
__device__ __forceinline__ void blend_one(const Bary& b, const float* w, const AttrRec& a, PixelAcc& acc) {
    float o = interp_rn(b, a.o[0], a.o[1], a.o[2], w[0], w[1], w[2]);
    o = fminf(fmaxf(o, 0.f), kMaxOpacity);
    const float cr = interp_rn(b, a.c[0], a.c[3], a.c[6], w[0], w[1], w[2]);
    const float cg = interp_rn(b, a.c[1], a.c[4], a.c[7], w[0], w[1], w[2]);
    const float cb = interp_rn(b, a.c[2], a.c[5], a.c[8], w[0], w[1], w[2]);
    const float zv = interp_rn(b, div(1.f, w[0]), div(1.f, w[1]), div(1.f, w[2]), 1.f, 1.f, 1.f);
    const float ao = mul(acc.alpha, o);
    acc.depth = add(acc.depth, mul(ao, zv));
    acc.weight = add(acc.weight, ao);
    acc.r = add(acc.r, mul(ao, cr));
    acc.g = add(acc.g, mul(ao, cg));
    acc.b = add(acc.b, mul(ao, cb));
    acc.alpha = mul(acc.alpha, sub(1.f, o));
    acc.blended++;
}

struct TileCtx {
    int tile, start, end, ix, iy;
    bool active;
    float px, py;
};

__device__ __forceinline__ TileCtx tile_context(const BlendParams& P) {
    TileCtx c;
    c.tile = blockIdx.x;
    const int tx = c.tile % P.tiles_x, ty = c.tile / P.tiles_x;
    const int lx = threadIdx.x % P.tw, ly = threadIdx.x / P.tw;
    c.ix = tx * P.tw + lx;
    c.iy = ty * P.th + ly;
    c.active = (int)threadIdx.x < P.tw * P.th && c.ix < P.W && c.iy < P.H;
    c.start = P.offsets[c.tile];
    c.end = P.offsets[c.tile + 1];
    c.px = pixel_coord(c.ix, P.W);
    c.py = pixel_coord(c.iy, P.H);
    return c;
}

// Stage `n` records of the list starting at `first` into shared memory (ids + geometry).
__device__ __forceinline__ void stage_chunk(const BlendParams& P, int first, int n, float4* s_geo, int* s_id) {
    for (int i = threadIdx.x; i < n * 4; i += blockDim.x) {
        const int rec = i >> 2, q = i & 3;
        const int id = P.ids[first + rec];
        if (q == 0) s_id[rec] = id;
        s_geo[i] = __ldg(P.geo + 4 * (size_t)id + q);
    }
}

// One selection sweep over the whole tile list (select_next_k_in_tile, reference render.cu:375-415):
// keeps the `bs` covered fragments smallest in (depth, j) among those after (lastDepth, lastJ).
// All threads of the CTA must call it; `go` says whether this thread collects.
__device__ __forceinline__ int select_sweep(const BlendParams& P, const TileCtx& c, bool go, int bs, float lastDepth,
                                            int lastJ, float* dl, int* jl, float4* s_geo, int* s_id) {
    int found = 0;
    for (int first = c.start; first < c.end; first += kChunk) {
        const int n = min(kChunk, c.end - first);
        __syncthreads();
        stage_chunk(P, first, n, s_geo, s_id);
        __syncthreads();
        if (!go) continue;
        for (int r = 0; r < n; r++) {
            const float* g = reinterpret_cast<const float*>(s_geo + 4 * r);
            const Bary b = apply_bary(g, c.px, c.py);
            if (!covered(b)) continue;
            const float d = interp_rn(b, g[9], g[10], g[11], g[12], g[13], g[14]);
            const int j = first + r;
            if (d < lastDepth) continue;
            if (d == lastDepth && j <= lastJ) continue;
            if (found == bs && d >= dl[bs - 1]) continue;
            int pos = (found < bs) ? found : (bs - 1);
            while (pos > 0 && d < dl[pos - 1]) {
                dl[pos] = dl[pos - 1];
                jl[pos] = jl[pos - 1];
                pos--;
            }
            dl[pos] = d;
            jl[pos] = j;
            if (found < bs) found++;
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

template <bool SORT, int MAXT>
__global__ void __launch_bounds__(MAXT) blend_forward_kernel(BlendParams P, float4* __restrict__ image,
                                                             float* __restrict__ depthmap, float* __restrict__ final_w,
                                                             int* __restrict__ ends) {
    __shared__ float4 s_geo[kChunk * 4];
    __shared__ int s_id[kChunk];
    const TileCtx c = tile_context(P);
    PixelAcc acc;

    if (SORT) {
        float dl[kBatchLayers];
        int jl[kBatchLayers];
        float lastDepth = -INFINITY;
        int lastJ = -1;
        bool want = c.active;
        while (true) {
            const bool go = want && acc.alpha > P.thr && acc.blended < P.max_layers;
            if (!__syncthreads_or(go)) break;
            const int bs = min(kBatchLayers, P.max_layers - acc.blended);
            const int found = select_sweep(P, c, go, bs, lastDepth, lastJ, dl, jl, s_geo, s_id);
            if (go) {
                if (found == 0) want = false;
                else {
                    const int n = min(found, P.max_layers - acc.blended);
                    for (int i = 0; i < n; i++) {
                        const int id = P.ids[jl[i]];
                        float m[9], z[3], w[3];
                        load_geo(P.geo, id, m, z, w);
                        const Bary b = apply_bary(m, c.px, c.py);
                        const AttrRec a = load_attr<false>(P.attr, id);
                        blend_one(b, w, a, acc);
                    }
                    lastDepth = dl[n - 1];
                    lastJ = jl[n - 1];
                }
            }
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
                for (int r = 0; r < n && !done; r++) {
                    if (!(acc.alpha > P.thr && acc.blended < P.max_layers)) { done = true; break; }
                    const float* g = reinterpret_cast<const float*>(s_geo + 4 * r);
                    const Bary b = apply_bary(g, c.px, c.py);
                    if (!covered(b)) continue;
                    const AttrRec a = load_attr<false>(P.attr, s_id[r]);
                    blend_one(b, g + 12, a, acc);
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

// Gradient contributions of one fragment: per vertex (x, y, w, r, g, b, o).
struct FragGrad { float v[21]; };

// Scalar interpolation VJP (reference util.h:299-317).
__device__ __forceinline__ void interp_bwd(float g, const Bary& b, float a0, float a1, float a2, float w0, float w1,
                                           float w2, float* gbary, float* gvals, float* gw) {
    const float nom = b.x * w0 * a0 + b.y * w1 * a1 + b.z * w2 * a2;
    const float den = b.x * w0 + b.y * w1 + b.z * w2;
    if (den * den < kEffZero) {
        gbary[0] = gbary[1] = gbary[2] = 0.f;
        gvals[0] = gvals[1] = gvals[2] = 0.f;
        gw[0] = gw[1] = gw[2] = 0.f;
        return;
    }
    const float inv = 1.f / den, inv2 = inv * inv;
    const float e0 = (a0 * den - nom) * inv2, e1 = (a1 * den - nom) * inv2, e2 = (a2 * den - nom) * inv2;
    gbary[0] = g * w0 * e0; gbary[1] = g * w1 * e1; gbary[2] = g * w2 * e2;
    gvals[0] = g * b.x * w0 * inv; gvals[1] = g * b.y * w1 * inv; gvals[2] = g * b.z * w2 * inv;
    gw[0] = g * b.x * e0; gw[1] = g * b.y * e1; gw[2] = g * b.z * e2;
}

// process_backward of the reference (render.cu:455-538).  Vertex-position gradients follow the
// reference's expanded partial derivatives (util.h:405-455) term by term: for small triangles
// their fp32 rounding is systematic and part of what "the same result" means.
__device__ __forceinline__ void backward_one(const float* w, const AttrRec& a, const Bary& b, float px, float py,
                                             const PixelGrad& pg, BackState& st, FragGrad& out) {
    float o = interp_rn(b, a.o[0], a.o[1], a.o[2], w[0], w[1], w[2]);
    o = fminf(fmaxf(o, 0.f), kMaxOpacity);
    const float cr = interp_rn(b, a.c[0], a.c[3], a.c[6], w[0], w[1], w[2]);
    const float cg = interp_rn(b, a.c[1], a.c[4], a.c[7], w[0], w[1], w[2]);
    const float cb = interp_rn(b, a.c[2], a.c[5], a.c[8], w[0], w[1], w[2]);
    const float iw0 = 1.f / w[0], iw1 = 1.f / w[1], iw2 = 1.f / w[2];
    const float z = interp_rn(b, iw0, iw1, iw2, 1.f, 1.f, 1.f);
    const float om = 1.f - o, iom = 1.f / om;

    const float drgb_do = ((cr * st.alpha - st.sr) * iom * pg.gr + (cg * st.alpha - st.sg) * iom * pg.gg +
                           (cb * st.alpha - st.sb) * iom * pg.gb) -
                          pg.ga * pg.final_alpha * iom;
    st.alpha = st.alpha * iom;
    st.sr += cr * o * st.alpha;
    st.sg += cg * o * st.alpha;
    st.sb += cb * o * st.alpha;
    const float ddw_do = st.alpha - st.oa * iom;
    const float dud_do = st.alpha * z - st.zoa * iom;
    st.oa += o * st.alpha;
    st.zoa += z * o * st.alpha;
    const bool has_w = !(pg.final_weight < kEffZero);
    const float inv_fw = has_w ? 1.f / pg.final_weight : 0.f;
    const float dd_do = has_w ? (dud_do - pg.final_depth * ddw_do) * inv_fw * pg.gd : 0.f;
    const float d_do = drgb_do + dd_do;

    float gb_o[3], gv_o[3], gw_o[3];
    interp_bwd(d_do, b, a.o[0], a.o[1], a.o[2], w[0], w[1], w[2], gb_o, gv_o, gw_o);

    const float ao = st.alpha * o;
    float gbary[3] = {gb_o[0], gb_o[1], gb_o[2]};
    float gw[3] = {gw_o[0], gw_o[1], gw_o[2]};
    float gcol[9];
    {
        // colour: vector VJP = three scalar VJPs sharing bary / w
        const float dcs[3] = {ao * pg.gr, ao * pg.gg, ao * pg.gb};
#pragma unroll
        for (int ch = 0; ch < 3; ch++) {
            float gb_c[3], gv_c[3], gw_c[3];
            interp_bwd(dcs[ch], b, a.c[ch], a.c[3 + ch], a.c[6 + ch], w[0], w[1], w[2], gb_c, gv_c, gw_c);
#pragma unroll
            for (int k = 0; k < 3; k++) {
                gbary[k] += gb_c[k];
                gw[k] += gw_c[k];
                gcol[3 * k + ch] = gv_c[k];
            }
        }
    }
    {
        const float dd_dz = has_w ? ao * pg.gd * inv_fw : 0.f;
        float gb_z[3], gv_z[3], gw_z[3];
        interp_bwd(dd_dz, b, iw0, iw1, iw2, 1.f, 1.f, 1.f, gb_z, gv_z, gw_z);
        gbary[0] += gb_z[0]; gbary[1] += gb_z[1]; gbary[2] += gb_z[2];
        // the reference also adds the gradient w.r.t. the unit weights of this interpolation to the
        // w gradient (render.cu:530); kept for identical results
        gw[0] += gw_z[0] - gv_z[0] * iw0 * iw0;
        gw[1] += gw_z[1] - gv_z[1] * iw1 * iw1;
        gw[2] += gw_z[2] - gv_z[2] * iw2 * iw2;
    }
    // barycentric_backward: l by cross products, then the expanded partials
    const float ax = a.xy[0], ay = a.xy[1], bx = a.xy[2], by = a.xy[3], cx = a.xy[4], cy = a.xy[5];
    float gxy[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float d = ax * (by - cy) + bx * (-ay + cy) + cx * (ay - by);
    if (!(fabsf(d) < kEffZero)) {
        const float Tt = (bx - ax) * (cy - ay) - (by - ay) * (cx - ax);
        const float lx = ((bx - px) * (cy - py) - (by - py) * (cx - px)) / Tt;
        const float ly = ((cx - px) * (ay - py) - (cy - py) * (ax - px)) / Tt;
        const float lz = ((ax - px) * (by - py) - (ay - py) * (bx - px)) / Tt;
        const float id = 1.f / d;
        const float g0 = gbary[0], g1 = gbary[1], g2 = gbary[2];
        gxy[0] = (g0 * (lx * (-by + cy)) + g1 * (-cy - ly * (by - cy) + py) + g2 * (by - lz * (by - cy) - py)) * id;
        gxy[1] = (g0 * (lx * (bx - cx)) + g1 * (cx + ly * (bx - cx) - px) + g2 * (-bx + lz * (bx - cx) + px)) * id;
        gxy[2] = (g0 * (cy + lx * (ay - cy) - py) + g1 * (ly * (ay - cy)) + g2 * (-ay + lz * (ay - cy) + py)) * id;
        gxy[3] = (g0 * (-cx - lx * (ax - cx) + px) + g1 * (ly * (-ax + cx)) + g2 * (ax - lz * (ax - cx) - px)) * id;
        gxy[4] = (g0 * (-by - lx * (ay - by) + py) + g1 * (ay - ly * (ay - by) - py) + g2 * (lz * (-ay + by))) * id;
        gxy[5] = (g0 * (bx + lx * (ax - bx) - px) + g1 * (-ax + ly * (ax - bx) + px) + g2 * (lz * (ax - bx))) * id;
    }
#pragma unroll
    for (int k = 0; k < 3; k++) {
        out.v[7 * k + 0] = gxy[2 * k + 0];
        out.v[7 * k + 1] = gxy[2 * k + 1];
        out.v[7 * k + 2] = gw[k];
        out.v[7 * k + 3] = gcol[3 * k + 0];
        out.v[7 * k + 4] = gcol[3 * k + 1];
        out.v[7 * k + 5] = gcol[3 * k + 2];
        out.v[7 * k + 6] = gv_o[k];
    }
}

struct GradOut { float* gV; float* gC; float* gO; };

// Warp-level reduction before atomics: lanes holding the same triangle are summed with shuffles
// and one lane issues the 21 atomics of that triangle.
__device__ __forceinline__ void warp_accumulate(bool has, int tri, const int* vid, const FragGrad& fg, const GradOut& G) {
    unsigned todo = __ballot_sync(0xffffffffu, has);
    while (todo) {
        const int leader = __ffs(todo) - 1;
        const int tsel = __shfl_sync(0xffffffffu, tri, leader);
        const bool mine = has && tri == tsel;
        const unsigned grp = __ballot_sync(0xffffffffu, mine);
        todo &= ~grp;
        float s[21];
#pragma unroll
        for (int k = 0; k < 21; k++) {
            float x = mine ? fg.v[k] : 0.f;
            if (grp != (1u << leader)) {
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
            }
            s[k] = x;
        }
        if ((int)lane_id() == leader) {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const int v = vid[k];
                atomicAdd(G.gV + 4 * (size_t)v + 0, s[7 * k + 0]);
                atomicAdd(G.gV + 4 * (size_t)v + 1, s[7 * k + 1]);
                atomicAdd(G.gV + 4 * (size_t)v + 3, s[7 * k + 2]);
                atomicAdd(G.gC + 3 * (size_t)v + 0, s[7 * k + 3]);
                atomicAdd(G.gC + 3 * (size_t)v + 1, s[7 * k + 4]);
                atomicAdd(G.gC + 3 * (size_t)v + 2, s[7 * k + 5]);
                atomicAdd(G.gO + v, s[7 * k + 6]);
            }
        }
    }
}

template <bool SORT, int MAXT>
__global__ void __launch_bounds__(MAXT) blend_backward_kernel(BlendParams P, const float4* __restrict__ gimage,
                                                              const float* __restrict__ gdepth,
                                                              const float4* __restrict__ image,
                                                              const float* __restrict__ depthmap,
                                                              const float* __restrict__ final_w,
                                                              const int* __restrict__ ends, GradOut G) {
    __shared__ float4 s_geo[kChunk * 4];
    __shared__ int s_id[kChunk];
    const TileCtx c = tile_context(P);
    PixelGrad pg = {};
    BackState st;
    st.alpha = 1.f;
    int limit = 0;
    if (c.active) {
        const size_t index = (size_t)c.iy * P.W + c.ix;
        const float4 gi = gimage[index];
        pg.gr = gi.x; pg.gg = gi.y; pg.gb = gi.z; pg.ga = gi.w;
        pg.gd = gdepth[index];
        pg.final_alpha = image[index].w;
        pg.final_weight = final_w[index];
        pg.final_depth = depthmap[index];
        st.alpha = pg.final_alpha;
        limit = min(ends[index], P.max_layers);
    }

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
            int n = 0;
            if (go) {
                if (found == 0) remaining = 0;
                else n = min(found, remaining);
            }
            // walk the batch back to front; the warp iterates together so that lanes can be reduced
            int nmax = n;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, d));
            for (int s = 0; s < nmax; s++) {
                const bool has = s < n;
                int id = -1;
                FragGrad fg;
                AttrRec a;
                a.vid[0] = a.vid[1] = a.vid[2] = 0;
                if (has) {
                    id = P.ids[jl[n - 1 - s]];
                    float m[9], z[3], w[3];
                    load_geo(P.geo, id, m, z, w);
                    const Bary b = apply_bary(m, c.px, c.py);
                    a = load_attr<true>(P.attr, id);
                    backward_one(w, a, b, c.px, c.py, pg, st, fg);
                }
                warp_accumulate(has, id, a.vid, fg, G);
            }
            if (n > 0) {
                lastDepth = dl[n - 1];
                lastJ = jl[n - 1];
                remaining -= n;
            }
        }
    } else {
        // reference render.cu:659-666: the first `limit` list entries, front to back
        int lim_max = limit;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) lim_max = max(lim_max, __shfl_xor_sync(0xffffffffu, lim_max, d));
        __shared__ int s_lim;
        if (threadIdx.x == 0) s_lim = 0;
        __syncthreads();
        if (lane_id() == 0) atomicMax(&s_lim, lim_max);
        __syncthreads();
        const int cta_lim = min(s_lim, c.end - c.start);
        for (int first = 0; first < cta_lim; first += kChunk) {
            const int n = min(kChunk, cta_lim - first);
            __syncthreads();
            stage_chunk(P, c.start + first, n, s_geo, s_id);
            __syncthreads();
            const int warp_n = min(n, lim_max - first);
            for (int r = 0; r < warp_n; r++) {
                const float* g = reinterpret_cast<const float*>(s_geo + 4 * r);
                bool has = (first + r) < limit;
                Bary b = {0.f, 0.f, 0.f};
                if (has) {
                    b = apply_bary(g, c.px, c.py);
                    has = covered(b);
                }
                const int id = s_id[r];
                FragGrad fg;
                AttrRec a;
                a.vid[0] = a.vid[1] = a.vid[2] = 0;
                if (__any_sync(0xffffffffu, has)) {
                    a = load_attr<true>(P.attr, id);
                    if (has) backward_one(g + 12, a, b, c.px, c.py, pg, st, fg);
                    warp_accumulate(has, id, a.vid, fg, G);
                }
            }
        }
    }
}

}  // namespace tg

extern "C" {

static int blend_args(int W, int H, int tw, int th, int max_layers) {
    TG_REQUIRE(W > 0 && H > 0 && tw > 0 && th > 0, "sizes must be positive");
    TG_REQUIRE(tw * th <= 1024, "tile_width * tile_height must be <= 1024");
    TG_REQUIRE(max_layers >= 1, "max_layers must be >= 1");
    return TG_OK;
}

int tg_blend_forward(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                     int W, int H, int tw, int th, float thr, int per_pixel_sort, int max_layers, float* image,
                     float* depthmap, float* final_weights, int32_t* ends, tg_stream_t stream) {
    if (int s = blend_args(W, H, tw, th, max_layers)) return s;
    TG_REQUIRE(offsets && image && depthmap && final_weights && ends, "null pointer");
    TG_REQUIRE(((uintptr_t)image & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 && ((uintptr_t)tri_attr & 15) == 0,
               "image / tri_geo / tri_attr must be 16-byte aligned");
    tg::BlendParams P;
    P.geo = (const float4*)tri_geo; P.attr = (const float4*)tri_attr; P.ids = sorted_ids; P.offsets = offsets;
    P.W = W; P.H = H; P.tw = tw; P.th = th; P.tiles_x = (W + tw - 1) / tw;
    P.thr = thr; P.max_layers = max_layers;
    const int tiles = P.tiles_x * ((H + th - 1) / th);
    const int threads = ((tw * th + 31) / 32) * 32;
    cudaStream_t s = (cudaStream_t)stream;
    float4* img = (float4*)image;
    if (threads <= 256) {
        if (per_pixel_sort) tg::blend_forward_kernel<true, 256><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends);
        else tg::blend_forward_kernel<false, 256><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends);
    } else {
        if (per_pixel_sort) tg::blend_forward_kernel<true, 1024><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends);
        else tg::blend_forward_kernel<false, 1024><<<tiles, threads, 0, s>>>(P, img, depthmap, final_weights, ends);
    }
    TG_LAUNCH_CHECK("blend_forward_kernel");
    return TG_OK;
}

int tg_blend_backward(const float* tri_geo, const float* tri_attr, const int32_t* sorted_ids, const int32_t* offsets,
                      int V, int W, int H, int tw, int th, int per_pixel_sort, int max_layers, const float* grad_image,
                      const float* grad_depthmap, const float* image, const float* depthmap, const float* final_weights,
                      const int32_t* ends, float* grad_vertices, float* grad_colors, float* grad_opacities,
                      int accumulate, tg_stream_t stream) {
    if (int s = blend_args(W, H, tw, th, max_layers)) return s;
    TG_REQUIRE(V >= 0, "V < 0");
    TG_REQUIRE(offsets && grad_image && grad_depthmap && image && depthmap && final_weights && ends, "null pointer");
    TG_REQUIRE(V == 0 || (grad_vertices && grad_colors && grad_opacities), "null gradient pointer");
    TG_REQUIRE(((uintptr_t)image & 15) == 0 && ((uintptr_t)grad_image & 15) == 0 && ((uintptr_t)tri_geo & 15) == 0 &&
                   ((uintptr_t)tri_attr & 15) == 0,
               "image / grad_image / tri_geo / tri_attr must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    if (!accumulate && V > 0) {
        TG_CUDA(cudaMemsetAsync(grad_vertices, 0, sizeof(float) * 4 * (size_t)V, s));
        TG_CUDA(cudaMemsetAsync(grad_colors, 0, sizeof(float) * 3 * (size_t)V, s));
        TG_CUDA(cudaMemsetAsync(grad_opacities, 0, sizeof(float) * (size_t)V, s));
    }
    tg::BlendParams P;
    P.geo = (const float4*)tri_geo; P.attr = (const float4*)tri_attr; P.ids = sorted_ids; P.offsets = offsets;
    P.W = W; P.H = H; P.tw = tw; P.th = th; P.tiles_x = (W + tw - 1) / tw;
    P.thr = 0.f; P.max_layers = max_layers;
    const int tiles = P.tiles_x * ((H + th - 1) / th);
    const int threads = ((tw * th + 31) / 32) * 32;
    tg::GradOut G = {grad_vertices, grad_colors, grad_opacities};
    const float4* gi = (const float4*)grad_image;
    const float4* im = (const float4*)image;
    if (threads <= 256) {
        if (per_pixel_sort)
            tg::blend_backward_kernel<true, 256><<<tiles, threads, 0, s>>>(P, gi, grad_depthmap, im, depthmap, final_weights, ends, G);
        else
            tg::blend_backward_kernel<false, 256><<<tiles, threads, 0, s>>>(P, gi, grad_depthmap, im, depthmap, final_weights, ends, G);
    } else {
        if (per_pixel_sort)
            tg::blend_backward_kernel<true, 1024><<<tiles, threads, 0, s>>>(P, gi, grad_depthmap, im, depthmap, final_weights, ends, G);
        else
            tg::blend_backward_kernel<false, 1024><<<tiles, threads, 0, s>>>(P, gi, grad_depthmap, im, depthmap, final_weights, ends, G);
    }
    TG_LAUNCH_CHECK("blend_backward_kernel");
    return TG_OK;
}

}  // extern "C"
