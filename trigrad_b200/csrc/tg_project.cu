// World -> render-space projection of the vertices and its vector-Jacobian product: the step right
// before the rasteriser in a multi-view optimisation.  The reference does it with torch tensor
// operations in its viewer (viewer.py:271-278: clip = PV * (x, y, z, 1); vertex = (clip.xyz / clip.w,
// 1 / clip.w)); here one kernel each way, so that a view's render-space vertices and the world-space
// gradient need no intermediate tensors.
#include "tg_common.cuh"

namespace tg {

struct Mat4 { float m[16]; };   // row-major

__global__ void __launch_bounds__(256) project_kernel(const float* __restrict__ points, int V, Mat4 pv,
                                                      float4* __restrict__ vertices) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    const float x = points[3 * (size_t)v], y = points[3 * (size_t)v + 1], z = points[3 * (size_t)v + 2];
    float c[4];
#pragma unroll
    for (int r = 0; r < 4; r++) c[r] = fma_(pv.m[4 * r + 2], z, fma_(pv.m[4 * r + 1], y, fma_(pv.m[4 * r], x, pv.m[4 * r + 3])));
    vertices[v] = make_float4(div(c[0], c[3]), div(c[1], c[3]), div(c[2], c[3]), div(1.f, c[3]));
}

// grad_points[v] (+)= J^T grad_vertices[v], J = d(x/w, y/w, z/w, 1/w) / d(point).
__global__ void __launch_bounds__(256) project_backward_kernel(const float* __restrict__ points, int V, Mat4 pv,
                                                               const float4* __restrict__ grad_vertices,
                                                               float* __restrict__ grad_points, int accumulate) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    const float x = points[3 * (size_t)v], y = points[3 * (size_t)v + 1], z = points[3 * (size_t)v + 2];
    float c[4];
#pragma unroll
    for (int r = 0; r < 4; r++) c[r] = fma_(pv.m[4 * r + 2], z, fma_(pv.m[4 * r + 1], y, fma_(pv.m[4 * r], x, pv.m[4 * r + 3])));
    const float4 g = grad_vertices[v];
    const float iw = div(1.f, c[3]);
    // d/dclip: the first three outputs are clip.k / clip.w, the fourth is 1 / clip.w
    const float d0 = g.x * iw, d1 = g.y * iw, d2 = g.z * iw;
    const float d3 = -(d0 * c[0] + d1 * c[1] + d2 * c[2] + g.w * iw) * iw;
#pragma unroll
    for (int k = 0; k < 3; k++) {
        const float gk = d0 * pv.m[k] + d1 * pv.m[4 + k] + d2 * pv.m[8 + k] + d3 * pv.m[12 + k];
        float* out = grad_points + 3 * (size_t)v + k;
        *out = accumulate ? *out + gk : gk;
    }
}

// The packed accumulator of ONE view (what the gradient kernels leave with TG_ACCUMULATE_PACKED: per vertex
// (d/dx, d/dy, d/dw, d/dopacity | d/dr, d/dg, d/db, -), then 64 loss partials) straight to world space: the
// render-space vertex gradient goes through the projection's VJP and is ADDED to grad_points, colours and
// opacities are added as they are, and the accumulator is cleared on the way out so that the next view needs no
// memset.  All additions are atomic reductions: several streams may add their views into the same three
// tensors.  Vertices that received nothing (hidden, off-screen) cost one 32-byte read.
__global__ void __launch_bounds__(256) unpack_project_backward_kernel(float4* __restrict__ gpack, int V,
                                                                      const float* __restrict__ points, Mat4 pv,
                                                                      float* __restrict__ grad_points,
                                                                      float* __restrict__ grad_colors,
                                                                      float* __restrict__ grad_opacities,
                                                                      float* __restrict__ partials, float loss_scale,
                                                                      float* __restrict__ loss_out) {
    if (blockIdx.x == 0 && threadIdx.x < 32) {
        float x = partials[threadIdx.x] + partials[threadIdx.x + 32];
        partials[threadIdx.x] = 0.f;
        partials[threadIdx.x + 32] = 0.f;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
        if (threadIdx.x == 0 && loss_out) atomicAdd(loss_out, x * loss_scale);
    }
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    const float4 a = gpack[2 * (size_t)v], b = gpack[2 * (size_t)v + 1];
    if (a.x == 0.f && a.y == 0.f && a.z == 0.f && a.w == 0.f && b.x == 0.f && b.y == 0.f && b.z == 0.f) return;
    gpack[2 * (size_t)v] = make_float4(0.f, 0.f, 0.f, 0.f);
    gpack[2 * (size_t)v + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
    const float x = points[3 * (size_t)v], y = points[3 * (size_t)v + 1], z = points[3 * (size_t)v + 2];
    float c[4];
#pragma unroll
    for (int r = 0; r < 4; r++) c[r] = fma_(pv.m[4 * r + 2], z, fma_(pv.m[4 * r + 1], y, fma_(pv.m[4 * r], x, pv.m[4 * r + 3])));
    const float iw = div(1.f, c[3]);
    // render-space gradient (x, y, z = 0, w) -> clip space -> world space, as project_backward_kernel
    const float d0 = a.x * iw, d1 = a.y * iw;
    const float d3 = -(d0 * c[0] + d1 * c[1] + a.z * iw) * iw;
#pragma unroll
    for (int k = 0; k < 3; k++)
        atomicAdd(grad_points + 3 * (size_t)v + k, d0 * pv.m[k] + d1 * pv.m[4 + k] + d3 * pv.m[12 + k]);
    atomicAdd(grad_colors + 3 * (size_t)v, b.x);
    atomicAdd(grad_colors + 3 * (size_t)v + 1, b.y);
    atomicAdd(grad_colors + 3 * (size_t)v + 2, b.z);
    atomicAdd(grad_opacities + v, a.w);
}

}  // namespace tg

extern "C" {

int tg_project(const float* points, int V, const float* pv_host, float* vertices, tg_stream_t stream) {
    TG_REQUIRE(V >= 0, "V < 0");
    if (V == 0) return TG_OK;
    TG_REQUIRE(points && pv_host && vertices, "null pointer");
    TG_REQUIRE(((uintptr_t)vertices & 15) == 0, "vertices must be 16-byte aligned");
    tg::Mat4 pv;
    for (int i = 0; i < 16; i++) pv.m[i] = pv_host[i];
    tg::project_kernel<<<(V + 255) / 256, 256, 0, (cudaStream_t)stream>>>(points, V, pv, (float4*)vertices);
    TG_LAUNCH_CHECK("project_kernel");
    return TG_OK;
}

int tg_project_backward(const float* points, int V, const float* pv_host, const float* grad_vertices, float* grad_points,
                        int accumulate, tg_stream_t stream) {
    TG_REQUIRE(V >= 0, "V < 0");
    if (V == 0) return TG_OK;
    TG_REQUIRE(points && pv_host && grad_vertices && grad_points, "null pointer");
    TG_REQUIRE(((uintptr_t)grad_vertices & 15) == 0, "grad_vertices must be 16-byte aligned");
    tg::Mat4 pv;
    for (int i = 0; i < 16; i++) pv.m[i] = pv_host[i];
    tg::project_backward_kernel<<<(V + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        points, V, pv, (const float4*)grad_vertices, grad_points, accumulate);
    TG_LAUNCH_CHECK("project_backward_kernel");
    return TG_OK;
}

int tg_unpack_project_backward(void* scratch, size_t scratch_bytes, int V, const float* points, const float* pv_host,
                               float loss_scale, float* loss_out, float* grad_points, float* grad_colors,
                               float* grad_opacities, tg_stream_t stream) {
    TG_REQUIRE(V > 0, "V must be positive");
    TG_REQUIRE(scratch && points && pv_host && grad_points && grad_colors && grad_opacities, "null pointer");
    TG_REQUIRE(((uintptr_t)scratch & 15) == 0, "scratch must be 16-byte aligned");
    if (scratch_bytes < tg_backward_scratch_bytes(V)) {
        tg_host::set_error("backward scratch: need %zu bytes, got %zu", tg_backward_scratch_bytes(V), scratch_bytes);
        return TG_ERR_WORKSPACE;
    }
    tg::Mat4 pv;
    for (int i = 0; i < 16; i++) pv.m[i] = pv_host[i];
    float* partials = (float*)((char*)scratch + (size_t)V * 32);
    tg::unpack_project_backward_kernel<<<(V + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        (float4*)scratch, V, points, pv, grad_points, grad_colors, grad_opacities, partials, loss_scale, loss_out);
    TG_LAUNCH_CHECK("unpack_project_backward_kernel");
    return TG_OK;
}

}  // extern "C"
