// Near-plane triangle splitter fused with the world -> render-space projection, and its vector-Jacobian
// product: the step before the rasteriser for cameras that sit inside or close to the mesh.
//
// The reference does this in its notebook with a Python loop over triangles (`split_clipped`,
// notebooks/renderer.ipynb cell "Clip Test"): clip-space vertices, signed distance d = z + w to the near plane,
// a triangle with all three vertices inside (d >= 0) is kept, one with none is dropped, one inside vertex gives
// one smaller triangle (in, new1, new2), two inside vertices give a quad split into (in1, in2, new1) and
// (new1, in2, new2); a new vertex is a + t (b - a) with t = d_a / (d_a - d_b) from the inside vertex a to the
// outside vertex b, and colours and opacities are interpolated with the same t.  The result is a triangle
// soup.  Here one thread handles one input triangle and owns two output slots (6 vertices), so the order of
// the reference's soup is kept and nothing has to be counted or compacted: slots that are not needed are
// filled with a degenerate triangle (all vertices (0,0,0,1)), which the rasteriser's preprocess drops.
// Output vertices are already divided: (x/w, y/w, z/w, 1/w), the render format (viewer.py:271-278).
#include "tg_common.cuh"

namespace tg {

struct ClipMat { float m[16]; };   // row-major projection * view

struct ClipVertex { float x, y, z, w; };

__device__ __forceinline__ ClipVertex to_clip(const float* __restrict__ points, int v, const ClipMat& pv) {
    const float x = points[3 * (size_t)v], y = points[3 * (size_t)v + 1], z = points[3 * (size_t)v + 2];
    float c[4];
#pragma unroll
    for (int r = 0; r < 4; r++) c[r] = fma_(pv.m[4 * r + 2], z, fma_(pv.m[4 * r + 1], y, fma_(pv.m[4 * r], x, pv.m[4 * r + 3])));
    return {c[0], c[1], c[2], c[3]};
}

// Which case a triangle is, and the rotation (in, out1, out2) / (out, in1, in2) the reference uses.
struct ClipCase {
    int inside;      // number of inside vertices
    int k0, k1, k2;  // inside == 1: (in, out1, out2); inside == 2: (out, in1, in2); else (0, 1, 2)
};

__device__ __forceinline__ ClipCase classify(float d0, float d1, float d2) {
    const bool i0 = d0 >= 0.f, i1 = d1 >= 0.f, i2 = d2 >= 0.f;
    ClipCase c;
    c.inside = (int)i0 + (int)i1 + (int)i2;
    c.k0 = 0; c.k1 = 1; c.k2 = 2;
    if (c.inside == 1) {
        if (i0) { c.k0 = 0; c.k1 = 1; c.k2 = 2; }
        else if (i1) { c.k0 = 1; c.k1 = 2; c.k2 = 0; }
        else { c.k0 = 2; c.k1 = 0; c.k2 = 1; }
    } else if (c.inside == 2) {
        if (!i0) { c.k0 = 0; c.k1 = 1; c.k2 = 2; }
        else if (!i1) { c.k0 = 1; c.k1 = 2; c.k2 = 0; }
        else { c.k0 = 2; c.k1 = 0; c.k2 = 1; }
    }
    return c;
}

struct SoupVertex { ClipVertex v; float r, g, b, o; };

// a + t (b - a), every operation rounded separately (what the tensor expression of the reference evaluates to)
__device__ __forceinline__ float lerp_rn(float a, float b, float t) { return add(a, mul(t, sub(b, a))); }

__device__ __forceinline__ SoupVertex lerp_vertex(const SoupVertex& a, const SoupVertex& b, float t) {
    SoupVertex n;
    n.v = {lerp_rn(a.v.x, b.v.x, t), lerp_rn(a.v.y, b.v.y, t), lerp_rn(a.v.z, b.v.z, t), lerp_rn(a.v.w, b.v.w, t)};
    n.r = lerp_rn(a.r, b.r, t); n.g = lerp_rn(a.g, b.g, t); n.b = lerp_rn(a.b, b.b, t);
    n.o = lerp_rn(a.o, b.o, t);
    return n;
}

__device__ __forceinline__ void store_soup(const SoupVertex& s, int slot, float4* __restrict__ out_vertices,
                                           float* __restrict__ out_colors, float* __restrict__ out_opacities) {
    out_vertices[slot] = make_float4(div(s.v.x, s.v.w), div(s.v.y, s.v.w), div(s.v.z, s.v.w), div(1.f, s.v.w));
    out_colors[3 * (size_t)slot] = s.r; out_colors[3 * (size_t)slot + 1] = s.g; out_colors[3 * (size_t)slot + 2] = s.b;
    out_opacities[slot] = s.o;
}

__device__ __forceinline__ void store_unused(int slot, float4* __restrict__ out_vertices, float* __restrict__ out_colors,
                                             float* __restrict__ out_opacities) {
    out_vertices[slot] = make_float4(0.f, 0.f, 0.f, 1.f);
    out_colors[3 * (size_t)slot] = 0.f; out_colors[3 * (size_t)slot + 1] = 0.f; out_colors[3 * (size_t)slot + 2] = 0.f;
    out_opacities[slot] = 0.f;
}

__global__ void __launch_bounds__(256) project_clip_kernel(const float* __restrict__ points, const int* __restrict__ indices,
                                                           const float* __restrict__ colors,
                                                           const float* __restrict__ opacities, int T, ClipMat pv,
                                                           float4* __restrict__ out_vertices, int* __restrict__ out_indices,
                                                           float* __restrict__ out_colors,
                                                           float* __restrict__ out_opacities) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    SoupVertex s[3];
    float d[3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        const int v = indices[3 * (size_t)t + k];
        s[k].v = to_clip(points, v, pv);
        s[k].r = colors[3 * (size_t)v]; s[k].g = colors[3 * (size_t)v + 1]; s[k].b = colors[3 * (size_t)v + 2];
        s[k].o = opacities[v];
        d[k] = add(s[k].v.z, s[k].v.w);
    }
    const int base = 6 * t;
#pragma unroll
    for (int k = 0; k < 6; k++) out_indices[base + k] = base + k;
    const ClipCase cc = classify(d[0], d[1], d[2]);
    SoupVertex o[6];
    int used = 0;
    if (cc.inside == 3) {
        o[0] = s[0]; o[1] = s[1]; o[2] = s[2];
        used = 3;
    } else if (cc.inside == 1) {
        const SoupVertex& in = s[cc.k0];
        const float t1 = div(d[cc.k0], sub(d[cc.k0], d[cc.k1])), t2 = div(d[cc.k0], sub(d[cc.k0], d[cc.k2]));
        o[0] = in; o[1] = lerp_vertex(in, s[cc.k1], t1); o[2] = lerp_vertex(in, s[cc.k2], t2);
        used = 3;
    } else if (cc.inside == 2) {
        const SoupVertex &out = s[cc.k0], &in1 = s[cc.k1], &in2 = s[cc.k2];
        const float t1 = div(d[cc.k1], sub(d[cc.k1], d[cc.k0])), t2 = div(d[cc.k2], sub(d[cc.k2], d[cc.k0]));
        const SoupVertex n1 = lerp_vertex(in1, out, t1), n2 = lerp_vertex(in2, out, t2);
        o[0] = in1; o[1] = in2; o[2] = n1;
        o[3] = n1; o[4] = in2; o[5] = n2;
        used = 6;
    }
#pragma unroll
    for (int k = 0; k < 6; k++) {
        if (k < used) store_soup(o[k], base + k, out_vertices, out_colors, out_opacities);
        else store_unused(base + k, out_vertices, out_colors, out_opacities);
    }
}

// ---- vector-Jacobian product ---------------------------------------------------------------------
// Gradient record of one ORIGINAL vertex of the triangle: clip-space position, colour, opacity.
struct VertexGrad { float x = 0.f, y = 0.f, z = 0.f, w = 0.f, r = 0.f, g = 0.f, b = 0.f, o = 0.f; };

struct SoupGrad { float x, y, z, w, r, g, b, o; };   // upstream gradient of one soup vertex, position already in clip space

// render-space gradient (of x/w, y/w, z/w, 1/w) -> clip-space gradient at clip vertex c
__device__ __forceinline__ SoupGrad load_soup_grad(const ClipVertex& c, int slot, const float4* __restrict__ gv,
                                                   const float* __restrict__ gc, const float* __restrict__ go) {
    const float4 g = gv[slot];
    const float iw = 1.f / c.w;
    SoupGrad s;
    s.x = g.x * iw; s.y = g.y * iw; s.z = g.z * iw;
    s.w = -(s.x * c.x + s.y * c.y + s.z * c.z + g.w * iw) * iw;
    s.r = gc[3 * (size_t)slot]; s.g = gc[3 * (size_t)slot + 1]; s.b = gc[3 * (size_t)slot + 2];
    s.o = go[slot];
    return s;
}

__device__ __forceinline__ void add_grad(VertexGrad& a, const SoupGrad& g, float f) {
    a.x += f * g.x; a.y += f * g.y; a.z += f * g.z; a.w += f * g.w;
    a.r += f * g.r; a.g += f * g.g; a.b += f * g.b; a.o += f * g.o;
}

// new = a + t (b - a), t = da / (da - db), d = z + w: the gradient g of `new` goes to a and b, also through t
__device__ __forceinline__ void lerp_backward(const SoupVertex& a, const SoupVertex& b, float da, float db, float t,
                                              const SoupGrad& g, VertexGrad& ga, VertexGrad& gb) {
    add_grad(ga, g, 1.f - t);
    add_grad(gb, g, t);
    const float gt = g.x * (b.v.x - a.v.x) + g.y * (b.v.y - a.v.y) + g.z * (b.v.z - a.v.z) + g.w * (b.v.w - a.v.w) +
                     g.r * (b.r - a.r) + g.g * (b.g - a.g) + g.b * (b.b - a.b) + g.o * (b.o - a.o);
    const float inv = 1.f / (da - db);
    const float gda = gt * (-db) * inv * inv, gdb = gt * da * inv * inv;
    ga.z += gda; ga.w += gda;
    gb.z += gdb; gb.w += gdb;
}

__global__ void __launch_bounds__(256) project_clip_backward_kernel(
    const float* __restrict__ points, const int* __restrict__ indices, const float* __restrict__ colors,
    const float* __restrict__ opacities, int T, ClipMat pv, const float4* __restrict__ grad_out_vertices,
    const float* __restrict__ grad_out_colors, const float* __restrict__ grad_out_opacities,
    float* __restrict__ grad_points, float* __restrict__ grad_colors, float* __restrict__ grad_opacities) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    SoupVertex s[3];
    float d[3];
    int vid[3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        const int v = indices[3 * (size_t)t + k];
        vid[k] = v;
        s[k].v = to_clip(points, v, pv);
        s[k].r = colors[3 * (size_t)v]; s[k].g = colors[3 * (size_t)v + 1]; s[k].b = colors[3 * (size_t)v + 2];
        s[k].o = opacities[v];
        d[k] = add(s[k].v.z, s[k].v.w);
    }
    const ClipCase cc = classify(d[0], d[1], d[2]);
    if (cc.inside == 0) return;
    const int base = 6 * t;
    VertexGrad g[3];
    if (cc.inside == 3) {
#pragma unroll
        for (int k = 0; k < 3; k++)
            add_grad(g[k], load_soup_grad(s[k].v, base + k, grad_out_vertices, grad_out_colors, grad_out_opacities), 1.f);
    } else if (cc.inside == 1) {
        const SoupVertex &in = s[cc.k0], &o1 = s[cc.k1], &o2 = s[cc.k2];
        const float t1 = div(d[cc.k0], sub(d[cc.k0], d[cc.k1])), t2 = div(d[cc.k0], sub(d[cc.k0], d[cc.k2]));
        const SoupVertex n1 = lerp_vertex(in, o1, t1), n2 = lerp_vertex(in, o2, t2);
        add_grad(g[cc.k0], load_soup_grad(in.v, base, grad_out_vertices, grad_out_colors, grad_out_opacities), 1.f);
        lerp_backward(in, o1, d[cc.k0], d[cc.k1], t1,
                      load_soup_grad(n1.v, base + 1, grad_out_vertices, grad_out_colors, grad_out_opacities), g[cc.k0], g[cc.k1]);
        lerp_backward(in, o2, d[cc.k0], d[cc.k2], t2,
                      load_soup_grad(n2.v, base + 2, grad_out_vertices, grad_out_colors, grad_out_opacities), g[cc.k0], g[cc.k2]);
    } else {
        const SoupVertex &out = s[cc.k0], &in1 = s[cc.k1], &in2 = s[cc.k2];
        const float t1 = div(d[cc.k1], sub(d[cc.k1], d[cc.k0])), t2 = div(d[cc.k2], sub(d[cc.k2], d[cc.k0]));
        const SoupVertex n1 = lerp_vertex(in1, out, t1), n2 = lerp_vertex(in2, out, t2);
        // soup: (in1, in2, n1), (n1, in2, n2)
        add_grad(g[cc.k1], load_soup_grad(in1.v, base, grad_out_vertices, grad_out_colors, grad_out_opacities), 1.f);
        add_grad(g[cc.k2], load_soup_grad(in2.v, base + 1, grad_out_vertices, grad_out_colors, grad_out_opacities), 1.f);
        add_grad(g[cc.k2], load_soup_grad(in2.v, base + 4, grad_out_vertices, grad_out_colors, grad_out_opacities), 1.f);
        SoupGrad gn1 = load_soup_grad(n1.v, base + 2, grad_out_vertices, grad_out_colors, grad_out_opacities);
        const SoupGrad gn1b = load_soup_grad(n1.v, base + 3, grad_out_vertices, grad_out_colors, grad_out_opacities);
        gn1.x += gn1b.x; gn1.y += gn1b.y; gn1.z += gn1b.z; gn1.w += gn1b.w;
        gn1.r += gn1b.r; gn1.g += gn1b.g; gn1.b += gn1b.b; gn1.o += gn1b.o;
        lerp_backward(in1, out, d[cc.k1], d[cc.k0], t1, gn1, g[cc.k1], g[cc.k0]);
        lerp_backward(in2, out, d[cc.k2], d[cc.k0], t2,
                      load_soup_grad(n2.v, base + 5, grad_out_vertices, grad_out_colors, grad_out_opacities), g[cc.k2], g[cc.k0]);
    }
#pragma unroll
    for (int k = 0; k < 3; k++) {
        const int v = vid[k];
        // clip -> world: clip = PV (p, 1)
#pragma unroll
        for (int j = 0; j < 3; j++)
            atomicAdd(grad_points + 3 * (size_t)v + j,
                      g[k].x * pv.m[j] + g[k].y * pv.m[4 + j] + g[k].z * pv.m[8 + j] + g[k].w * pv.m[12 + j]);
        atomicAdd(grad_colors + 3 * (size_t)v, g[k].r);
        atomicAdd(grad_colors + 3 * (size_t)v + 1, g[k].g);
        atomicAdd(grad_colors + 3 * (size_t)v + 2, g[k].b);
        atomicAdd(grad_opacities + v, g[k].o);
    }
}

}  // namespace tg

extern "C" {

int tg_project_clip(const float* points, const int32_t* indices, const float* colors, const float* opacities, int T,
                    const float* pv_host, float* out_vertices, int32_t* out_indices, float* out_colors,
                    float* out_opacities, tg_stream_t stream) {
    TG_REQUIRE(T >= 0, "T < 0");
    if (T == 0) return TG_OK;
    TG_REQUIRE(T <= 0x7fffffff / 6, "T too large for 6 T soup vertices");
    TG_REQUIRE(points && indices && colors && opacities && pv_host && out_vertices && out_indices && out_colors &&
                   out_opacities, "null pointer");
    TG_REQUIRE(((uintptr_t)out_vertices & 15) == 0, "out_vertices must be 16-byte aligned");
    tg::ClipMat pv;
    for (int i = 0; i < 16; i++) pv.m[i] = pv_host[i];
    tg::project_clip_kernel<<<(T + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        points, indices, colors, opacities, T, pv, (float4*)out_vertices, out_indices, out_colors, out_opacities);
    TG_LAUNCH_CHECK("project_clip_kernel");
    return TG_OK;
}

int tg_project_clip_backward(const float* points, const int32_t* indices, const float* colors, const float* opacities,
                             int T, const float* pv_host, const float* grad_out_vertices, const float* grad_out_colors,
                             const float* grad_out_opacities, float* grad_points, float* grad_colors,
                             float* grad_opacities, tg_stream_t stream) {
    TG_REQUIRE(T >= 0, "T < 0");
    if (T == 0) return TG_OK;
    TG_REQUIRE(points && indices && colors && opacities && pv_host && grad_out_vertices && grad_out_colors &&
                   grad_out_opacities && grad_points && grad_colors && grad_opacities, "null pointer");
    TG_REQUIRE(((uintptr_t)grad_out_vertices & 15) == 0, "grad_out_vertices must be 16-byte aligned");
    tg::ClipMat pv;
    for (int i = 0; i < 16; i++) pv.m[i] = pv_host[i];
    tg::project_clip_backward_kernel<<<(T + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        points, indices, colors, opacities, T, pv, (const float4*)grad_out_vertices, grad_out_colors, grad_out_opacities,
        grad_points, grad_colors, grad_opacities);
    TG_LAUNCH_CHECK("project_clip_backward_kernel");
    return TG_OK;
}

}  // extern "C"
