"""ctypes front end of the CPU oracle (``oracle/trigrad_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the benchmark's
``cpu_baseline`` / reference arm, never by the shipped render path.

Two ways to the per-tile lists are offered and must agree (``tests/test_oracle.py``):

* ``build_lists``            - native: per-tile counts, cumulative offsets, ``std::stable_sort``
                               per tile, i.e. the reference's own objects (``render.cu:286-308``);
* ``build_lists_staged``     - the new pipeline's objects restated with numpy: per-triangle counts,
                               exclusive scan, 64-bit ``tile<<32 | ord(depth)`` keys in triangle
                               order, one global stable sort, tile ranges.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        import build as _build  # oracle/build.py

        path = _build.LIB
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            path = _build.build()
        _lib = C.CDLL(path)
        _lib.tgo_build_lists_f32.restype = C.c_longlong
        _lib.tgo_build_lists_f64.restype = C.c_longlong
        _lib.tgo_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().tgo_num_threads())


def set_num_threads(n: int) -> None:
    lib().tgo_set_num_threads(C.c_int(n))


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _suf(dtype) -> str:
    return "f32" if np.dtype(dtype) == np.float32 else "f64"


def _fn(name: str, dtype):
    return getattr(lib(), f"{name}_{_suf(dtype)}")


def _sc(dtype, x):
    return C.c_float(x) if np.dtype(dtype) == np.float32 else C.c_double(x)


def float_to_ordered_u32(x: np.ndarray) -> np.ndarray:
    """Order-preserving float32 -> uint32 map used in the 64-bit sort keys.

    Negative floats have all bits flipped, non-negative ones the sign bit set; -0.0 is first
    mapped to +0.0 so that the two zeros compare equal, as they do in a float comparison.
    """
    x = np.asarray(x, dtype=np.float32) + np.float32(0.0)  # -0.0 + 0.0 = +0.0
    u = x.view(np.uint32)
    neg = (u >> np.uint32(31)).astype(bool)
    return np.where(neg, ~u, u | np.uint32(0x80000000)).astype(np.uint32)


def ordered_u32_to_float(u: np.ndarray) -> np.ndarray:
    u = np.asarray(u, dtype=np.uint32)
    pos = (u >> np.uint32(31)).astype(bool)
    return np.where(pos, u & np.uint32(0x7FFFFFFF), ~u).astype(np.uint32).view(np.float32)


@dataclass
class Lists:
    offsets: np.ndarray   # [tiles+1] int32
    ids: np.ndarray       # [K] int32, sorted per tile
    keys: np.ndarray      # [K] float, sorted per tile


@dataclass
class Staged:
    rects: np.ndarray        # [T,4] int32 (x0,y0,x1,y1), empty = (0,-1,0,-1)
    counts: np.ndarray       # [T] int32
    tri_offsets: np.ndarray  # [T+1] int64 exclusive scan of counts
    keys_unsorted: np.ndarray  # [K] uint64 (float32 only)
    ids_unsorted: np.ndarray   # [K] int32
    keys_sorted: np.ndarray    # [K] uint64
    ids_sorted: np.ndarray     # [K] int32
    offsets: np.ndarray        # [tiles+1] int32
    depth_keys_unsorted: np.ndarray  # [K] float


def num_tiles(W, H, tw, th):
    return ((W + tw - 1) // tw) * ((H + th - 1) // th)


def tile_rects(verts, idx, W, H, tw, th):
    verts = np.ascontiguousarray(verts)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    T = idx.shape[0]
    rects = np.empty((T, 4), np.int32)
    counts = np.empty(T, np.int32)
    _fn("tgo_tile_rects", verts.dtype)(_p(verts), _p(idx), T, W, H, tw, th, _p(rects), _p(counts))
    return rects, counts


def build_lists_staged(verts, idx, W, H, tw, th) -> Staged:
    verts = np.ascontiguousarray(verts)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    T = idx.shape[0]
    rects, counts = tile_rects(verts, idx, W, H, tw, th)
    tri_offsets = np.zeros(T + 1, np.int64)
    np.cumsum(counts, out=tri_offsets[1:])
    K = int(tri_offsets[-1])
    depth = np.empty(K, verts.dtype)
    tiles = np.empty(K, np.int32)
    tris = np.empty(K, np.int32)
    _fn("tgo_emit_keys", verts.dtype)(_p(verts), _p(idx), T, W, H, tw, th, _p(rects), _p(tri_offsets), _p(depth),
                                      _p(tiles), _p(tris))
    nt = num_tiles(W, H, tw, th)
    if verts.dtype == np.float32:
        keys = (tiles.astype(np.uint64) << np.uint64(32)) | float_to_ordered_u32(depth).astype(np.uint64)
        order = np.argsort(keys, kind="stable")
        keys_sorted = keys[order]
    else:
        keys = np.zeros(K, np.uint64)
        order = np.lexsort((np.arange(K), depth, tiles))  # tile, then depth, then emission order
        keys_sorted = keys
    ids_sorted = tris[order]
    tiles_sorted = tiles[order]
    offsets = np.searchsorted(tiles_sorted, np.arange(nt + 1), side="left").astype(np.int32)
    return Staged(rects, counts, tri_offsets, keys, tris, keys_sorted, np.ascontiguousarray(ids_sorted), offsets, depth)


def build_lists(verts, idx, W, H, tw, th, cull: bool = False) -> Lists:
    """Per-tile sorted lists.  ``cull`` drops the (triangle, tile) pairs whose triangle provably covers no pixel centre of
    the tile (an extension; the reference lists every tile of the bounding box, ``render.cu:110``)."""
    verts = np.ascontiguousarray(verts)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    T = idx.shape[0]
    nt = num_tiles(W, H, tw, th)
    offsets = np.empty(nt + 1, np.int32)
    f = _fn("tgo_build_lists", verts.dtype)
    K = f(_p(verts), _p(idx), T, W, H, tw, th, _p(offsets), None, None, C.c_longlong(0), int(cull))
    ids = np.empty(max(K, 1), np.int32)
    keys = np.empty(max(K, 1), verts.dtype)
    K2 = f(_p(verts), _p(idx), T, W, H, tw, th, _p(offsets), _p(ids), _p(keys), C.c_longlong(K), int(cull))
    assert K2 == K
    return Lists(offsets, ids[:K], keys[:K])


def bary_matrices(verts, idx):
    verts = np.ascontiguousarray(verts)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    M = np.empty((idx.shape[0], 3, 3), verts.dtype)
    _fn("tgo_bary_matrices", verts.dtype)(_p(verts), _p(idx), idx.shape[0], _p(M))
    return M


def depth_planes(verts, idx):
    verts = np.ascontiguousarray(verts)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    P = np.empty((idx.shape[0], 3), verts.dtype)
    _fn("tgo_depth_planes", verts.dtype)(_p(verts), _p(idx), idx.shape[0], _p(P))
    return P


@dataclass
class ForwardOut:
    image: np.ndarray
    depthmap: np.ndarray
    final_weights: np.ndarray
    ends: np.ndarray
    lists: Lists
    M: np.ndarray


def forward(verts, idx, colors, opac, W, H, tw=16, th=16, thr=1 / 256, per_pixel_sort=True, max_layers=32,
            lists: Lists | None = None, tile_stride: int = 1) -> ForwardOut:
    dt = np.asarray(verts).dtype
    verts = np.ascontiguousarray(verts, dtype=dt)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    colors = np.ascontiguousarray(colors, dtype=dt)
    opac = np.ascontiguousarray(opac, dtype=dt)
    T = idx.shape[0]
    if max_layers <= 0:
        max_layers = T + 1          # reference src/trigrad/wrapper.py:35-36
    if lists is None:
        lists = build_lists(verts, idx, W, H, tw, th)
    M = bary_matrices(verts, idx)
    image = np.zeros((H, W, 4), dt)
    depth = np.zeros((H, W), dt)
    fw = np.zeros((H, W), dt)
    ends = np.zeros((H, W), np.int32)
    ids = np.ascontiguousarray(lists.ids)
    _fn("tgo_forward", dt)(_p(verts), _p(idx), _p(colors), _p(opac), T, W, H, tw, th, _p(ids), _p(lists.offsets), _p(M),
                           _sc(dt, thr), int(bool(per_pixel_sort)), int(max_layers), _p(image), _p(depth), _p(fw),
                           _p(ends), int(tile_stride))
    return ForwardOut(image, depth, fw, ends, lists, M)


def backward(verts, idx, colors, opac, W, H, fwd: ForwardOut, grad_image, grad_depth, tw=16, th=16,
             per_pixel_sort=True, max_layers=32, tile_stride: int = 1, corrected: bool = False):
    """Gradients (gV [V,4], gC [V,3], gO [V]).  ``corrected=False`` restates the reference literally, including its
    behaviour outside the default mode (``render.cu:659-666``, ``:673-693``); ``corrected=True`` visits the blended
    fragments last to first in every mode (an extension; identical in the default mode)."""
    dt = np.asarray(verts).dtype
    verts = np.ascontiguousarray(verts, dtype=dt)
    idx = np.ascontiguousarray(idx, dtype=np.int32)
    colors = np.ascontiguousarray(colors, dtype=dt)
    opac = np.ascontiguousarray(opac, dtype=dt)
    gi = np.ascontiguousarray(grad_image, dtype=dt)
    gd = np.ascontiguousarray(grad_depth, dtype=dt)
    T = idx.shape[0]
    if max_layers <= 0:
        max_layers = T + 1
    gV = np.zeros_like(verts)
    gC = np.zeros_like(colors)
    gO = np.zeros_like(opac)
    ids = np.ascontiguousarray(fwd.lists.ids)
    _fn("tgo_backward", dt)(_p(verts), _p(idx), _p(colors), _p(opac), T, W, H, tw, th, _p(ids), _p(fwd.lists.offsets),
                            _p(fwd.M), int(bool(per_pixel_sort)), int(max_layers), _p(gi), _p(gd), _p(fwd.image),
                            _p(fwd.depthmap), _p(fwd.final_weights), _p(fwd.ends), _p(gV), _p(gC), _p(gO), int(tile_stride),
                            int(bool(corrected)))
    return gV, gC, gO


def sampled_pixels(scene, tile_stride: int) -> int:
    """Number of image pixels inside the tiles a ``tile_stride`` sample renders."""
    tx = (scene.width + scene.tile_width - 1) // scene.tile_width
    ty = (scene.height + scene.tile_height - 1) // scene.tile_height
    t = np.arange(0, tx * ty, max(1, tile_stride))
    w = np.minimum(scene.tile_width, scene.width - (t % tx) * scene.tile_width)
    h = np.minimum(scene.tile_height, scene.height - (t // tx) * scene.tile_height)
    return int((w * h).sum())


def render_l2(scene, dtype=np.float32, per_pixel_sort=True, max_layers=32, thr=1 / 256, target=None, tile_stride=1):
    """fwd + bwd of ``mean((image - target)**2)`` on a ``trigrad_b200.scenes.Scene``; the timed CPU step.

    ``tile_stride`` > 1 composites only every tile_stride-th tile (binning and sorting still run in
    full): a bounded sample of the workload for timing; outputs outside the sampled tiles stay zero."""
    v = scene.vertices.astype(dtype)
    c = scene.colors.astype(dtype)
    o = scene.opacities.astype(dtype)
    if target is None:
        target = scene.target()
    target = target.astype(dtype)
    f = forward(v, scene.indices, c, o, scene.width, scene.height, scene.tile_width, scene.tile_height, thr,
                per_pixel_sort, max_layers, tile_stride=tile_stride)
    diff = f.image - target
    loss = float(np.mean(diff.astype(np.float64) ** 2))
    gi = (diff * dtype(2.0 / diff.size)).astype(dtype)
    gd = np.zeros((scene.height, scene.width), dtype)
    g = backward(v, scene.indices, c, o, scene.width, scene.height, f, gi, gd, scene.tile_width, scene.tile_height,
                 per_pixel_sort, max_layers, tile_stride=tile_stride)
    return loss, f, g


def project(points, pv):
    """World points [V,3] -> render vertices (x/w, y/w, z/w, 1/w) with clip = PV (x, y, z, 1); in the dtype of `points`.

    Restates the tensor operations of the reference's viewer (``viewer.py:271-278``).
    """
    pts = np.asarray(points)
    dt = pts.dtype
    h = np.concatenate([pts, np.ones((pts.shape[0], 1), dt)], axis=1)
    clip = h @ np.asarray(pv, dt).T
    out = np.empty_like(clip)
    out[:, :3] = clip[:, :3] / clip[:, 3:4]
    out[:, 3] = dt.type(1) / clip[:, 3]
    return out


def project_vjp(points, pv, grad_vertices):
    """Vector-Jacobian product of `project`: gradient w.r.t. the points [V,3] given the gradient w.r.t. the vertices [V,4]."""
    pts = np.asarray(points)
    dt = pts.dtype
    pvm = np.asarray(pv, dt)
    g = np.asarray(grad_vertices, dt)
    h = np.concatenate([pts, np.ones((pts.shape[0], 1), dt)], axis=1)
    clip = h @ pvm.T
    iw = dt.type(1) / clip[:, 3]
    d = np.empty_like(clip)
    d[:, :3] = g[:, :3] * iw[:, None]
    d[:, 3] = -(np.sum(d[:, :3] * clip[:, :3], axis=1) + g[:, 3] * iw) * iw
    return (d @ pvm)[:, :3]


# ---------------------------------------------------------------------------------------------------------
# Near-plane triangle splitting (reference: ``split_clipped`` in notebooks/renderer.ipynb, cell "Clip Test").
# Plain Python loops: small cases only.  Pinned by tests/golden/clip_near_plane.npz, which holds outputs and
# autograd gradients of the reference's own function (run on CPU torch by tests/golden/make_clip_golden.py).
def split_clipped(clip, idx, colors, opac):
    """Restatement of the reference's ``split_clipped``: triangles cut at the plane ``z + w = 0`` of clip space.

    Returns ``(verts [3N,4], colors [3N,C], opac [3N], slots [N], plan)`` in the dtype of ``clip``: the triangle soup in
    the reference's order, for every output triangle the slot ``2 t + k`` (k-th output of input triangle t), and
    ``plan``: per soup vertex ``(a, b, t)`` meaning ``vertex = in[a] + t (in[b] - in[a])`` (``b = -1``: a copy of a).
    """
    clip = np.asarray(clip)
    dt = clip.dtype
    colors = np.asarray(colors, dt)
    opac = np.asarray(opac, dt).reshape(-1)
    out_v, out_c, out_o, slots, plan = [], [], [], [], []

    def copy(i):
        out_v.append(clip[i]); out_c.append(colors[i]); out_o.append(opac[i]); plan.append((int(i), -1, dt.type(0)))

    def lerp(a, b, t):
        out_v.append(clip[a] + t * (clip[b] - clip[a]))
        out_c.append(colors[a] + t * (colors[b] - colors[a]))
        out_o.append(opac[a] + t * (opac[b] - opac[a]))
        plan.append((int(a), int(b), t))

    for t_id, tri in enumerate(np.asarray(idx)):
        i0, i1, i2 = (int(x) for x in tri)
        d = [clip[i][2] + clip[i][3] for i in (i0, i1, i2)]
        inside = [x >= 0 for x in d]
        n = sum(inside)
        if n == 3:
            copy(i0); copy(i1); copy(i2)
            slots.append(2 * t_id)
        elif n == 1:
            if inside[0]:
                a, b, c, da, db, dc = i0, i1, i2, d[0], d[1], d[2]
            elif inside[1]:
                a, b, c, da, db, dc = i1, i2, i0, d[1], d[2], d[0]
            else:
                a, b, c, da, db, dc = i2, i0, i1, d[2], d[0], d[1]
            t1, t2 = da / (da - db), da / (da - dc)
            copy(a); lerp(a, b, t1); lerp(a, c, t2)
            slots.append(2 * t_id)
        elif n == 2:
            if not inside[0]:
                o, a, b, do, da, db = i0, i1, i2, d[0], d[1], d[2]
            elif not inside[1]:
                o, a, b, do, da, db = i1, i2, i0, d[1], d[2], d[0]
            else:
                o, a, b, do, da, db = i2, i0, i1, d[2], d[0], d[1]
            t1, t2 = da / (da - do), db / (db - do)
            copy(a); copy(b); lerp(a, o, t1)
            lerp(a, o, t1); copy(b); lerp(b, o, t2)
            slots += [2 * t_id, 2 * t_id + 1]
    C_ = colors.shape[1] if colors.ndim == 2 else 3
    if not out_v:
        return np.zeros((0, 4), dt), np.zeros((0, C_), dt), np.zeros((0,), dt), np.zeros((0,), np.int64), plan
    return (np.stack(out_v).astype(dt), np.stack(out_c).astype(dt), np.asarray(out_o, dt), np.asarray(slots, np.int64), plan)


def split_clipped_vjp(clip, colors, opac, plan, g_verts, g_colors, g_opac):
    """Vector-Jacobian product of ``split_clipped`` (float64): gradients w.r.t. clip vertices, colours and opacities
    given the gradients of the soup; the interpolation parameter ``t = d_a / (d_a - d_b)``, ``d = z + w``, is
    differentiated too (what torch autograd does with the reference's tensor expression)."""
    clip, colors, opac = (np.asarray(x, np.float64) for x in (clip, colors, opac))
    opac = opac.reshape(-1)
    gv, gc, go = np.zeros_like(clip), np.zeros_like(colors), np.zeros_like(opac)
    for k, (a, b, t) in enumerate(plan):
        t = float(t)
        if b < 0:
            gv[a] += g_verts[k]; gc[a] += g_colors[k]; go[a] += g_opac[k]
            continue
        gv[a] += (1 - t) * g_verts[k]; gv[b] += t * g_verts[k]
        gc[a] += (1 - t) * g_colors[k]; gc[b] += t * g_colors[k]
        go[a] += (1 - t) * g_opac[k]; go[b] += t * g_opac[k]
        gt = (g_verts[k] @ (clip[b] - clip[a]) + g_colors[k] @ (colors[b] - colors[a]) + g_opac[k] * (opac[b] - opac[a]))
        da, db = clip[a][2] + clip[a][3], clip[b][2] + clip[b][3]
        gda, gdb = gt * (-db) / (da - db) ** 2, gt * da / (da - db) ** 2
        gv[a][2] += gda; gv[a][3] += gda
        gv[b][2] += gdb; gv[b][3] += gdb
    return gv, gc, go


def to_clip(points, pv):
    """clip = PV (x, y, z, 1) in the dtype of ``points`` (reference ``viewer.py:271-274``)."""
    points = np.asarray(points)
    h = np.concatenate([points, np.ones((points.shape[0], 1), points.dtype)], axis=1)
    return h @ np.asarray(pv, points.dtype).T


def project_clip(points, pv, idx, colors, opac):
    """World mesh -> render-space soup clipped at the near plane: ``to_clip``, ``split_clipped``, then the division
    ``(x/w, y/w, z/w, 1/w)`` of ``viewer.py:275-278``.  Returns (verts, colors, opac, slots, plan, clip_soup)."""
    clip = to_clip(points, pv)
    sv, sc, so, slots, plan = split_clipped(clip, idx, colors, opac)
    out = np.empty_like(sv)
    if sv.shape[0]:
        out[:, :3] = sv[:, :3] / sv[:, 3:4]
        out[:, 3] = 1 / sv[:, 3]
    return out, sc, so, slots, plan, sv


def project_clip_vjp(points, pv, colors, opac, plan, clip_soup, g_verts, g_colors, g_opac):
    """VJP of ``project_clip`` (float64) w.r.t. world points, colours and opacities."""
    points = np.asarray(points, np.float64)
    pv = np.asarray(pv, np.float64)
    cs = np.asarray(clip_soup, np.float64)
    g = np.asarray(g_verts, np.float64)
    iw = 1.0 / cs[:, 3]
    gclip = np.empty_like(cs)
    gclip[:, :3] = g[:, :3] * iw[:, None]
    gclip[:, 3] = -(np.sum(gclip[:, :3] * cs[:, :3], axis=1) + g[:, 3] * iw) * iw
    gv, gc, go = split_clipped_vjp(to_clip(points, pv), colors, opac, plan, gclip, np.asarray(g_colors, np.float64),
                                   np.asarray(g_opac, np.float64))
    return gv @ pv[:, :3], gc, go
