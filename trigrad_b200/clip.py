"""Near-plane triangle splitting fused with the world -> render-space projection (``tg_project_clip``).

The reference's notebook clips with a Python loop over triangles (``split_clipped``,
``notebooks/renderer.ipynb``, cell "Clip Test") before dividing by w: a triangle that crosses the plane
``z + w = 0`` in clip space is cut into one or two triangles, one behind it is dropped, and the result is a
triangle soup with interpolated colours and opacities.  ``project_clip`` does the projection, the splitting and the
division in one kernel and is differentiable: its backward (``tg_project_clip_backward``) carries the gradients of
the soup back to world positions, colours and opacities, also through the interpolation parameters.

The soup has a fixed layout: input triangle t owns output triangles 2t and 2t+1 (vertices 6t .. 6t+5); slots that
are not needed hold a degenerate triangle that the rasteriser drops, so nothing is counted or compacted and the
reference's triangle order is kept.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
from torch.autograd import Function

from . import _native as N
from . import wrapper as _w


def _pv_host(pv):
    if isinstance(pv, torch.Tensor):
        pv = pv.detach().cpu().numpy()
    m = np.ascontiguousarray(pv, dtype=np.float32)
    if m.shape != (4, 4):
        raise ValueError("pv must be a 4x4 matrix")
    return m


class ProjectClip(Function):
    @staticmethod
    def forward(ctx, points, indices, colors, opacities, pv):
        V, T = points.shape[0], indices.shape[0]
        _w.check_tensor(points, "points", (V, 3))
        _w.check_tensor(indices, "indices", (T, 3), torch.int32)
        _w.check_tensor(colors, "colors", (V, 3))
        _w.check_tensor(opacities, "opacities", (V,))
        m = _pv_host(pv)
        points, indices, colors, opacities = (x.contiguous() for x in (points, indices, colors, opacities))
        dev = points.device
        out_v = torch.empty((6 * T, 4), dtype=torch.float32, device=dev)
        out_i = torch.empty((2 * T, 3), dtype=torch.int32, device=dev)
        out_c = torch.empty((6 * T, 3), dtype=torch.float32, device=dev)
        out_o = torch.empty((6 * T,), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            p = _w._ptr
            N.check("project_clip", N.lib().tg_project_clip(p(points), p(indices), p(colors), p(opacities), T,
                                                            m.ctypes.data_as(C.c_void_p), p(out_v), p(out_i), p(out_c),
                                                            p(out_o), C.c_void_p(stream)))
        ctx.save_for_backward(points, indices, colors, opacities)
        ctx.pv = m
        ctx.mark_non_differentiable(out_i)
        return out_v, out_i, out_c, out_o

    @staticmethod
    def backward(ctx, g_v, g_i, g_c, g_o):
        points, indices, colors, opacities = ctx.saved_tensors
        T = indices.shape[0]
        dev = points.device
        gp, gc, go = torch.zeros_like(points), torch.zeros_like(colors), torch.zeros_like(opacities)
        zeros = lambda shape: torch.zeros(shape, dtype=torch.float32, device=dev)   # noqa: E731
        g_v = zeros((6 * T, 4)) if g_v is None else g_v.contiguous()
        g_c = zeros((6 * T, 3)) if g_c is None else g_c.contiguous()
        g_o = zeros((6 * T,)) if g_o is None else g_o.contiguous()
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            p = _w._ptr
            N.check("project_clip_backward", N.lib().tg_project_clip_backward(
                p(points), p(indices), p(colors), p(opacities), T, ctx.pv.ctypes.data_as(C.c_void_p), p(g_v), p(g_c),
                p(g_o), p(gp), p(gc), p(go), C.c_void_p(stream)))
        return gp, None, gc, go, None


def project_clip(points: torch.Tensor, indices: torch.Tensor, colors: torch.Tensor, opacities: torch.Tensor, pv):
    """World-space mesh -> render-space triangle soup clipped at the near plane.

        points (V,3) float32, indices (T,3) int32, colors (V,3), opacities (V,), pv: 4x4 projection * view (host)

    Returns ``(vertices (6T,4), indices (2T,3), colors (6T,3), opacities (6T,))`` ready for ``render``; differentiable
    with respect to points, colours and opacities.
    """
    return ProjectClip.apply(points, indices, colors, opacities, pv)
