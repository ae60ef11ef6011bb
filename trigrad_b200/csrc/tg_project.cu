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

}  // extern "C"
