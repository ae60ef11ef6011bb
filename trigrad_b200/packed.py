"""Packed 16-byte input layout: faces as ``[T,4]`` int32 and per-vertex attributes as ``[V,4]`` (r, g, b, opacity).

The reference passes colours as ``[V,3]`` and faces as ``[T,3]`` and reads them through packed 3-word types
(``color3``, ``id3``, ``src/trigrad/util.h:457-573``): 12-byte strides that no vector load fits.  A caller that owns
its parameter tensors can keep them in the packed layout instead - one tensor ``rgba`` to optimise instead of
``colors`` and ``opacities`` - and call ``render_packed``: same rasteriser, same results, gradients returned in
the same layout (``tg_unpack_gradients_rgba``).
"""
from __future__ import annotations

import ctypes as C

import torch
from torch.autograd import Function

from . import _native as N
from . import wrapper as _w


def pack_mesh(colors: torch.Tensor, opacities: torch.Tensor, indices: torch.Tensor):
    """``(colors [V,3], opacities [V], indices [T,3] int32)`` -> ``(rgba [V,4], faces [T,4] int32)`` (one kernel)."""
    V, T = colors.shape[0], indices.shape[0]
    _w.check_tensor(colors, "colors", (V, 3))
    _w.check_tensor(opacities, "opacities", (V,))
    _w.check_tensor(indices, "indices", (T, 3), torch.int32)
    dev = colors.device
    rgba = torch.empty((V, 4), dtype=torch.float32, device=dev)
    faces = torch.empty((T, 4), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        p = _w._ptr
        N.check("pack_inputs", N.lib().tg_pack_inputs(p(colors.contiguous()), p(opacities.contiguous()),
                                                      p(indices.contiguous()), V, T, p(rgba), p(faces),
                                                      C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return rgba, faces


class RendererPacked(Function):
    @staticmethod
    def forward(ctx, vertices, faces, rgba, width=500, height=500, tile_width=16, tile_height=16,
                early_stopping_threshold=1 / 256, record_timing=False, per_pixel_sort=True, max_layers=32):
        n, _ = vertices.shape
        _w.check_tensor(vertices, "vertices", (n, 4))
        _w.check_tensor(rgba, "rgba", (n, 4))
        m, _ = faces.shape
        _w.check_tensor(faces, "faces", (m, 4), torch.int32)
        if max_layers <= 0:
            max_layers = m + 1
        ctx.num_vertices = n
        ctx.args = (width, height, tile_width, tile_height, bool(per_pixel_sort), int(max_layers))
        if m < 1:
            ctx.skipped = True
            image = torch.zeros((height, width, 4), dtype=rgba.dtype, device=rgba.device)
            image[..., 3] = 1.0
            depthmap = torch.full((height, width), float("inf"), dtype=rgba.dtype, device=rgba.device)
            timings = None
            ctx.save_for_backward(vertices, rgba)
        else:
            ctx.skipped = False
            (image, depthmap, final_weights, sorted_ids, offsets, tri_geo, tri_attr, ends, selection,
             timings) = _w.forward_native(vertices.contiguous(), faces.contiguous(), rgba.contiguous(), None, width, height,
                                          tile_width, tile_height, early_stopping_threshold, record_timing, per_pixel_sort,
                                          max_layers, cull_tiles=bool(per_pixel_sort) and _w.CULL_TILES, packed_inputs=True)
            ctx.has_selection = selection is not None
            saved = [sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends]
            ctx.save_for_backward(*(saved + ([selection] if selection is not None else [])))
        if record_timing:
            return image, depthmap, timings
        return image, depthmap

    @staticmethod
    def backward(ctx, grad_image, grad_depthmap, grad_timings=None):
        if ctx.skipped:
            vertices, rgba = ctx.saved_tensors
            return (torch.zeros_like(vertices), None, torch.zeros_like(rgba)) + (None,) * 8
        saved = tuple(ctx.saved_tensors) + (() if ctx.has_selection else (None,))
        sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends, selection = saved
        width, height, tile_width, tile_height, per_pixel_sort, max_layers = ctx.args
        V = ctx.num_vertices
        device = image.device
        lib = N.lib()
        with torch.cuda.device(device):
            stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            st = _w._state(device)
            st.check_error_word(st.last_slot)
            nscratch = lib.tg_backward_scratch_bytes(V)
            scratch = torch.zeros(nscratch, dtype=torch.uint8, device=device)
            gV = torch.empty((V, 4), dtype=torch.float32, device=device)
            gRGBA = torch.empty((V, 4), dtype=torch.float32, device=device)
            gi, gd = grad_image.contiguous(), grad_depthmap.contiguous()
            p = _w._ptr
            # the sums stay in the packed accumulator, which already has the layout wanted here
            N.check("blend_backward", lib.tg_blend_backward(
                p(tri_geo), p(tri_attr), p(sorted_ids), p(offsets), V, width, height, tile_width, tile_height,
                int(per_pixel_sort), int(max_layers), p(gi), p(gd), p(image), p(depthmap), p(final_weights), p(ends),
                p(selection), None, None, None, N.TG_ACCUMULATE_PACKED, p(scratch), nscratch, stream))
            N.check("unpack_gradients_rgba", lib.tg_unpack_gradients_rgba(p(scratch), nscratch, V, 0.0, None, p(gV), p(gRGBA),
                                                                          0, stream))
        return (gV, None, gRGBA) + (None,) * 8


def render_packed(vertices: torch.Tensor, faces: torch.Tensor, rgba: torch.Tensor, width: int = 500, height: int = 500,
                  tile_width: int = 16, tile_height: int = 16, early_stopping_threshold: float = 1 / 256,
                  record_timing: bool = False, per_pixel_sort: bool = True, max_layers: int = 32):
    """``render`` for the packed layout: ``faces`` is ``[T,4]`` int32 (fourth column ignored), ``rgba`` is ``[V,4]``
    (r, g, b, opacity).  Same outputs as ``render(vertices, faces[:, :3], rgba[:, :3], rgba[:, 3], ...)``; gradients
    flow to ``vertices`` and ``rgba``."""
    if tile_width * tile_height > 1024:
        raise ValueError("tile_width * tile_height must be <= 1024")
    return RendererPacked.apply(vertices, faces, rgba, width, height, tile_width, tile_height, early_stopping_threshold,
                                record_timing, per_pixel_sort, max_layers)
