"""``render_corrected``: the reference's ``render`` with gradients that are right in every mode.

The reference's backward kernel is only consistent with its forward in the default mode.  With
``per_pixel_sort=False`` it visits the first ``ends`` list entries front to back although its recurrences are
written for a walk from the last blended fragment to the first and ``ends`` counts blended fragments
(``src/trigrad/render.cu:659-666`` against ``:478-497``); with more than 32 layers it reverses the order inside
each batch of 32 only (``:673-693``).  ``trigrad_b200.render`` reproduces both literally (drop-in means identical
results).  This module is the opt-in alternative: same arguments, same forward results, and a backward
(``tg_blend_backward_corrected``) that differentiates what the forward blended, whatever the mode and the
number of layers.  In the default mode both functions return the same gradients.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch.autograd import Function

from . import _native as N
from . import wrapper as _w


class RendererCorrected(Function):
    @staticmethod
    def forward(ctx, vertices, indices, colors, opacities, width=500, height=500, tile_width=16, tile_height=16,
                early_stopping_threshold=1 / 256, record_timing=False, per_pixel_sort=True, max_layers=32):
        n, _ = vertices.shape
        _w.check_tensor(vertices, "vertices", (n, 4))
        _w.check_tensor(colors, "colors", (n, 3))
        _w.check_tensor(opacities, "opacities", (n,))
        ctx.num_vertices = n
        m, _ = indices.shape
        _w.check_tensor(indices, "indices", (m, 3), torch.int32)
        if max_layers <= 0:
            max_layers = m + 1
        ctx.args = (width, height, tile_width, tile_height, bool(per_pixel_sort), int(max_layers))
        if m < 1:
            ctx.skipped = True
            image = torch.zeros((height, width, 4), dtype=colors.dtype, device=colors.device)
            image[..., 3] = 1.0
            depthmap = torch.full((height, width), float("inf"), dtype=colors.dtype, device=colors.device)
            timings = None
            ctx.save_for_backward(vertices, colors, opacities)
        else:
            ctx.skipped = False
            (image, depthmap, final_weights, sorted_ids, offsets, tri_geo, tri_attr, ends, _, timings) = _w.forward_native(
                vertices.contiguous(), indices.contiguous(), colors.contiguous(), opacities.contiguous(), width, height,
                tile_width, tile_height, early_stopping_threshold, record_timing, per_pixel_sort, max_layers,
                save_selection=False, cull_tiles=_w.CULL_TILES)
            ctx.save_for_backward(sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends)
        if record_timing:
            return image, depthmap, timings
        return image, depthmap

    @staticmethod
    def backward(ctx, grad_image, grad_depthmap, grad_timings=None):
        if ctx.skipped:
            vertices, colors, opacities = ctx.saved_tensors
            return (torch.zeros_like(vertices), None, torch.zeros_like(colors), torch.zeros_like(opacities)) + (None,) * 8
        sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends = ctx.saved_tensors
        width, height, tile_width, tile_height, per_pixel_sort, max_layers = ctx.args
        V = ctx.num_vertices
        device = image.device
        lib = N.lib()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            st = _w._state(device)
            st.check_error_word(st.last_slot)
            nscratch = lib.tg_backward_scratch_bytes(V)
            scratch = torch.empty(nscratch, dtype=torch.uint8, device=device)
            f32 = dict(dtype=torch.float32, device=device)
            gV, gC, gO = torch.empty((V, 4), **f32), torch.empty((V, 3), **f32), torch.empty((V,), **f32)
            gi, gd = grad_image.contiguous(), grad_depthmap.contiguous()
            p = _w._ptr
            N.check("blend_backward_corrected", lib.tg_blend_backward_corrected(
                p(tri_geo), p(tri_attr), p(sorted_ids), p(offsets), V, width, height, tile_width, tile_height,
                int(per_pixel_sort), int(max_layers), p(gi), p(gd), p(image), p(depthmap), p(final_weights), p(ends),
                p(gV), p(gC), p(gO), 0, p(scratch), nscratch, C.c_void_p(stream)))
        return (gV, None, gC, gO) + (None,) * 8


def render_corrected(vertices, indices, colors, opacities, width=500, height=500, tile_width=16, tile_height=16,
                     early_stopping_threshold=1 / 256, record_timing=False, per_pixel_sort=True, max_layers=32):
    """Same contract as ``trigrad_b200.render`` (and the reference's ``trigrad.render``); the gradients are those of
    the rendered image in every mode, see the module docstring."""
    if tile_width * tile_height > 1024:
        raise ValueError("tile_width * tile_height must be <= 1024")
    return RendererCorrected.apply(vertices, indices, colors, opacities, width, height, tile_width, tile_height,
                                   early_stopping_threshold, record_timing, per_pixel_sort, max_layers)
