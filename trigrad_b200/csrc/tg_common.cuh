// Shared device helpers for the trigrad_b200 kernels (sm_100a).
//
// "Decision arithmetic" - everything that feeds an integer or an ordering decision (tile
// rectangle, sort key, coverage test, per-pixel sort depth) - is written with explicit
// round-to-nearest intrinsics so that nvcc never fuses or reorders it.  The sequences are the
// ones the CPU oracle fixes, which makes those stages bit-comparable.  Value arithmetic
// (blending, gradients) is left to the compiler.
#pragma once
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../../include/trigrad_b200.h"

namespace tg {

constexpr float kEffZero = FLT_MIN;       // reference util.h:24
constexpr float kMaxOpacity = 0.9999f;    // reference util.h:22
constexpr int kBatchLayers = 32;          // reference render.cu:570,655

// ---- rn math -------------------------------------------------------------------------------
__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float fma_(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }

// Order-preserving float -> uint32 (ascending floats give ascending unsigned); -0 folds to +0.
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    f = __fadd_rn(f, 0.0f);
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Rect { int x0, y0, x1, y1; };

// Tile rectangle of a triangle's bounding box; returns false for degenerate / non-finite input.
// Same rule as reference render.cu:51-76: float add, then double multiply/divide, cast, clamp,
// truncate.
__device__ __forceinline__ bool tile_rect(float ax, float ay, float bx, float by, float cx, float cy, int W, int H,
                                          int tw, int th, int tiles_x, int tiles_y, Rect& r) {
    float ux = sub(bx, ax), uy = sub(by, ay), vx = sub(cx, ax), vy = sub(cy, ay);
    float v = sub(mul(ux, vy), mul(uy, vx));
    if (fabsf(v) < kEffZero || isnan(v) || isinf(v)) {
        r = {0, -1, 0, -1};
        return false;
    }
    float minx = fminf(fminf(ax, bx), cx), miny = fminf(fminf(ay, by), cy);
    float maxx = fmaxf(fmaxf(ax, bx), cx), maxy = fmaxf(fmaxf(ay, by), cy);
    auto to_tile = [](float m, int extent, int tile, int ntiles) -> int {
        double d = __ddiv_rn(__dmul_rn(__dmul_rn((double)add(m, 1.0f), 0.5), (double)extent), (double)tile);
        float f = (float)d;
        float hi = (float)(ntiles - 1);
        f = (f < 0.0f) ? 0.0f : ((hi < f) ? hi : f);
        return (int)f;
    };
    r.x0 = to_tile(minx, W, tw, tiles_x);
    r.y0 = to_tile(miny, H, th, tiles_y);
    r.x1 = to_tile(maxx, W, tw, tiles_x);
    r.y1 = to_tile(maxy, H, th, tiles_y);
    return true;
}

// Pixel-centre NDC coordinate, computed in double and rounded once (reference render.cu:561-562).
__device__ __forceinline__ float pixel_coord(int i, int extent) {
    return (float)(__dsub_rn(__dmul_rn(__ddiv_rn(__dadd_rn((double)i, 0.5), (double)extent), 2.0), 1.0));
}

// Packed per-triangle records -------------------------------------------------------------------
struct __align__(16) Geo {
    float m[9];     // cartesian -> barycentric matrix, row major
    float z[3];     // vertex z (sort depth source)
    float w[3];     // vertex w
    float zlow;     // lower bound of the per-pixel sort depth over the triangle (-inf if none)
};
struct __align__(16) Attr {
    float o[3];     // vertex opacities
    float c[9];     // vertex colours a.rgb b.rgb c.rgb
    float iw[3];    // 1 / vertex w (correctly rounded), the values of the depth-map interpolation
    int vid[3];     // vertex ids
    float xy[6];    // a.xy b.xy c.xy (backward: vertex-position gradients)
};
static_assert(sizeof(Geo) == 4 * TG_GEO_WORDS, "Geo layout");
static_assert(sizeof(Attr) == 4 * TG_ATTR_WORDS, "Attr layout");

struct Bary { float x, y, z; };

// bary = M * (px, py, 1): two nested FMAs per row (the oracle's placement).
__device__ __forceinline__ Bary apply_bary(const float* m, float px, float py) {
    Bary b;
    b.x = fma_(m[0], px, fma_(m[1], py, m[2]));
    b.y = fma_(m[3], px, fma_(m[4], py, m[5]));
    b.z = fma_(m[6], px, fma_(m[7], py, m[8]));
    return b;
}
__device__ __forceinline__ bool covered(const Bary& b) {
    return !(b.x < kEffZero || b.y < kEffZero || b.z < kEffZero);
}

// Perspective-weighted interpolation, (b*a)*w products, FMA-accumulated (the oracle's placement).
__device__ __forceinline__ float interp_rn(const Bary& b, float a0, float a1, float a2, float w0, float w1, float w2) {
    float den = fma_(b.z, w2, fma_(b.y, w1, mul(b.x, w0)));
    float nom = mul(mul(b.x, a0), w0);
    nom = fma_(mul(b.y, a1), w1, nom);
    nom = fma_(mul(b.z, a2), w2, nom);
    return div(nom, den);
}

// NDC extent of the pixel centres of a block of pixels (a warp's 8x4 block, a whole tile).
struct PixelRect { float x0, x1, y0, y1; };

// Can the triangle with matrix m cover any pixel centre inside R?  Each barycentric is evaluated at
// the corner of R that maximises it, with the very operations of the per-pixel test; correctly
// rounded FMAs are monotone, so a pixel inside R can never get a larger value than the corner.
__device__ __forceinline__ bool rect_may_cover(const float* m, const PixelRect& R) {
#pragma unroll
    for (int k = 0; k < 3; k++) {
        const float cx = (m[3 * k] >= 0.f) ? R.x1 : R.x0;
        const float cy = (m[3 * k + 1] >= 0.f) ? R.y1 : R.y0;
        const float v = fma_(m[3 * k], cx, fma_(m[3 * k + 1], cy, m[3 * k + 2]));
        if (v < kEffZero) return false;
    }
    return true;
}

// Pixel-centre rectangle of tile (tx, ty); the last row / column of tiles may be cut by the image border.
__device__ __forceinline__ PixelRect tile_pixel_rect(int tx, int ty, int W, int H, int tw, int th) {
    PixelRect R;
    R.x0 = pixel_coord(tx * tw, W);
    R.x1 = pixel_coord(min((tx + 1) * tw, W) - 1, W);
    R.y0 = pixel_coord(ty * th, H);
    R.y1 = pixel_coord(min((ty + 1) * th, H) - 1, H);
    return R;
}

__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31u; }

}  // namespace tg

// Host-side helpers shared by the .cu files -------------------------------------------------------
namespace tg_host {
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void count_launch();
}  // namespace tg_host

#define TG_CUDA(call)                                                   \
    do {                                                                \
        cudaError_t e__ = (call);                                       \
        if (e__ != cudaSuccess) return tg_host::cuda_fail(e__, #call);  \
    } while (0)
#define TG_LAUNCH_CHECK(name)                                           \
    do {                                                                \
        tg_host::count_launch();                                        \
        cudaError_t e__ = cudaGetLastError();                           \
        if (e__ != cudaSuccess) return tg_host::cuda_fail(e__, name);   \
    } while (0)
#define TG_REQUIRE(cond, msg)                                           \
    do {                                                                \
        if (!(cond)) {                                                  \
            tg_host::set_error("bad argument: %s", msg);                \
            return TG_ERR_BAD_ARG;                                      \
        }                                                               \
    } while (0)
