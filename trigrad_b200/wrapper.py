"""Python entry point: ``render`` and the ``Renderer`` autograd function.

Mirrors the public interface of the reference (``src/trigrad/wrapper.py:12-158``): same argument
order and defaults, same exceptions (``TypeError`` for device / dtype, ``ValueError`` for shapes and
oversized tiles), same outputs ``(image, depthmap[, timings])`` and the same twelve gradient slots.
The work itself is done by hand-written sm_100a kernels behind the C ABI of
``include/trigrad_b200.h``; this module only allocates tensors and passes raw pointers and the
current CUDA stream.  There is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch
from torch.autograd import Function

from . import _native as N
from .util import create_check

precision = torch.float32
check_tensor = create_check("cuda", precision)

TIMING_KEYS = ("init", "per_tile_lists", "sorting", "bary_transforms", "rasterization")

# In the default mode the forward saves, per pixel, the ids of the fragments it blended (max_layers int32 planes
# of the image size: 265 MB at 1920x1080, 1.06 GB at 3840x2160, alive until the backward of that render has
# run) so that the backward need not search the tile lists again.  A render whose planes would exceed this many
# bytes saves nothing and its backward searches the lists as the reference does (same gradients, slower).
SELECTION_MAX_BYTES = 1 << 30

# With per_pixel_sort (the default) ``render`` lists a (triangle, tile) pair only when the triangle can cover the
# centre of a pixel of that tile - the exact test the reference leaves as a TODO (``render.cu:110``).  A pair that is
# dropped covers no pixel, so image, depth map and gradients are bit-identical either way; only the private tile
# lists are shorter than the reference's.  Tile-order mode keeps the reference's lists because its backward indexes
# them by position.  Set to False to build the reference's lists in every mode.
CULL_TILES = True


class _DeviceState:
    """Per (device, stream) reusable buffers: workspace, pinned read-back slots, K estimate."""

    SLOTS = 256

    def __init__(self, device: torch.device):
        self.device = device
        self.workspace = torch.empty(0, dtype=torch.uint8, device=device)
        self.info = torch.zeros((self.SLOTS, 4), dtype=torch.int32).pin_memory()   # K, longest list, error word, -
        self.slot = 0
        self.last_slot = -1      # slot of the previous native call on this stream (its error word may still travel)
        self.k_estimate = 0

    def next_slot(self) -> int:
        s = self.slot
        self.slot = (self.slot + 1) % self.SLOTS
        return s

    def check_error_word(self, slot: int) -> None:
        """Raise if the kernels of the call that used `slot` raised the device error word (a bounded wait ran
        out inside a kernel, so its outputs are not valid).  The word arrives by an asynchronous copy at the
        end of that call: it is certain to be there once a later event of the same stream has completed."""
        if slot < 0:
            return
        stale = int(self.info[slot, 2])
        if stale:
            self.info[slot, 2] = 0
            raise RuntimeError(f"trigrad_b200: an earlier render reported device error word {stale} "
                               "(a bounded wait ran out inside a kernel); its outputs are not valid")

    def finish_call(self, slot: int) -> None:
        """After a native forward call that used `slot` has returned: the call waited for an event recorded after
        the previous call's work on this stream, so the previous call's error word has arrived - check it."""
        prev, self.last_slot = self.last_slot, slot
        if prev != slot:
            self.check_error_word(prev)

    def ensure_workspace(self, nbytes: int) -> torch.Tensor:
        if self.workspace.numel() < nbytes:
            self.workspace = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=self.device)
        return self.workspace


_states: dict = {}


def _state(device: torch.device) -> _DeviceState:
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    st = _states.get(key)
    if st is None:
        st = _states[key] = _DeviceState(device)
    return st


def check_device_errors(device=None) -> None:
    """Synchronise the current stream of `device` and raise if the last render on it reported a device error
    word.  ``render`` checks the word of a call when the next call on the same stream returns, and (without
    waiting) when its backward starts; this is the explicit check for the last call of a program."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.current_stream(device).synchronize()
    with torch.cuda.device(device):
        st = _state(device)
    st.check_error_word(st.last_slot)


def _ptr(t: torch.Tensor | None):
    return None if t is None else C.c_void_p(t.data_ptr())


def forward_native(vertices, indices, colors, opacities, width, height, tile_width, tile_height,
                   early_stopping_threshold, record_timing, per_pixel_sort, max_layers, save_selection=True,
                   cull_tiles=False, packed_inputs=False):
    """Run the whole forward path.  Returns the public outputs and the state saved for backward.

    ``save_selection=False`` (or planes larger than ``SELECTION_MAX_BYTES``) skips the per-pixel record of the
    blended fragment ids; the backward then searches the tile lists again.  ``cull_tiles`` lists a (triangle, tile)
    pair only if the triangle can cover a pixel centre of the tile (``TG_FORWARD_CULL_TILES``): same image, same
    gradients, shorter lists than the reference's.  ``packed_inputs``: ``indices`` is ``[T,4]`` int32 and ``colors`` is
    ``[V,4]`` (r, g, b, opacity), ``opacities`` is None (``TG_INPUT_PACKED``)."""
    lib = N.lib()
    device = vertices.device
    T = indices.shape[0]
    tiles = ((width + tile_width - 1) // tile_width) * ((height + tile_height - 1) // tile_height)
    with torch.cuda.device(device):
        st = _state(device)
        stream = torch.cuda.current_stream(device).cuda_stream
        f32 = dict(dtype=torch.float32, device=device)
        image = torch.empty((height, width, 4), **f32)
        depthmap = torch.empty((height, width), **f32)
        final_weights = torch.empty((height, width), **f32)
        ends = torch.empty((height, width), dtype=torch.int32, device=device)
        tri_geo = torch.empty((T, N.GEO_WORDS), **f32)
        tri_attr = torch.empty((T, N.ATTR_WORDS), **f32)
        offsets = torch.empty(tiles + 1, dtype=torch.int32, device=device)
        planes = lib.tg_selection_planes(int(bool(per_pixel_sort)), int(max_layers))
        if not save_selection or planes * height * width * 4 > SELECTION_MAX_BYTES:
            planes = 0
        selection = torch.empty((planes, height, width), dtype=torch.int32, device=device) if planes else None
        stage_ms = (C.c_float * 5)() if record_timing else None
        cap = max(int(st.k_estimate * 1.25) + 1024, 2 * T + 1024)
        while True:
            sorted_ids = torch.empty(cap, dtype=torch.int32, device=device)
            ws = st.ensure_workspace(lib.tg_forward_workspace_bytes(T, tiles, cap))
            base = (ws.data_ptr() + 255) // 256 * 256
            slot = st.next_slot()
            info = st.info[slot]
            status = lib.tg_render_forward(
                _ptr(vertices), _ptr(indices), _ptr(colors), _ptr(opacities), T, width, height, tile_width,
                tile_height, float(early_stopping_threshold), int(bool(per_pixel_sort)), int(max_layers),
                _ptr(image), _ptr(depthmap), _ptr(final_weights), _ptr(ends), _ptr(selection), _ptr(tri_geo), _ptr(tri_attr),
                _ptr(sorted_ids), cap, _ptr(offsets), C.c_void_p(base), ws.numel() - (base - ws.data_ptr()),
                C.c_void_p(info.data_ptr()), stage_ms,
                (N.TG_FORWARD_CULL_TILES if cull_tiles else 0) | (N.TG_INPUT_PACKED if packed_inputs else 0),
                C.c_void_p(stream))
            K = int(info[0])
            if status == N.TG_ERR_CAPACITY:
                cap = int(K * 1.25) + 1024
                continue
            N.check("render_forward", status)
            st.finish_call(slot)
            break
        st.k_estimate = K
        timings = None
        if record_timing:
            timings = {k: float(stage_ms[i]) / 1000.0 for i, k in enumerate(TIMING_KEYS)}
    return image, depthmap, final_weights, sorted_ids[:K], offsets, tri_geo, tri_attr, ends, selection, timings


def backward_native(grad_image, grad_depthmap, saved, V, width, height, tile_width, tile_height, per_pixel_sort,
                    max_layers, out=None):
    """Gradient kernel.  ``out`` = (gV, gC, gO) to accumulate into, or None to get fresh tensors."""
    lib = N.lib()
    sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends, selection = saved
    device = image.device
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        # the forward's error word, if it has arrived by now (no waiting here): lists built by a kernel whose
        # bounded wait ran out must not be walked
        st = _state(device)
        st.check_error_word(st.last_slot)
        nscratch = lib.tg_backward_scratch_bytes(V)
        scratch = torch.empty(nscratch, dtype=torch.uint8, device=device)
        if grad_image is None:       # only the depth map was used downstream
            grad_image = torch.zeros_like(image)
        grad_image = grad_image.contiguous()
        grad_depthmap = None if grad_depthmap is None else grad_depthmap.contiguous()     # None: taken as zero by the kernel
        accumulate = out is not None
        if out is None:
            f32 = dict(dtype=torch.float32, device=device)
            out = (torch.empty((V, 4), **f32), torch.empty((V, 3), **f32), torch.empty((V,), **f32))
        gV, gC, gO = out
        status = lib.tg_blend_backward(
            _ptr(tri_geo), _ptr(tri_attr), _ptr(sorted_ids), _ptr(offsets), V, width, height, tile_width, tile_height,
            int(bool(per_pixel_sort)), int(max_layers), _ptr(grad_image), _ptr(grad_depthmap), _ptr(image),
            _ptr(depthmap), _ptr(final_weights), _ptr(ends), _ptr(selection), _ptr(gV), _ptr(gC), _ptr(gO),
            int(accumulate), _ptr(scratch), nscratch, C.c_void_p(stream))
        N.check("blend_backward", status)
    return gV, gC, gO


def backward_l2_native(target, saved, V, width, height, tile_width, tile_height, per_pixel_sort, max_layers, out,
                       loss_out, accumulate=True, packed_scratch=None):
    """Backward of ``mean((image - target)**2)`` fused into the gradient kernel (no gradient image is formed).

    ``saved`` is the tuple ``forward_native`` returned for backward (it must contain the selection, i.e. the
    default per-pixel mode with ``max_layers <= 32``); ``out`` = (gV [V,4], gC [V,3], gO [V]) and the 0-d float32
    ``loss_out`` are overwritten, or added to when ``accumulate`` is true.  With ``packed_scratch`` (a zeroed uint8
    tensor of ``tg_backward_scratch_bytes(V)`` bytes shared by the views of a step) nothing is written but that
    accumulator; ``unpack_gradients_native`` turns it into the three tensors later.  ``target`` is float32
    ``[H,W,4]`` or uint8 ``[H,W,4]`` (8-bit RGBA, read as value / 255).
    """
    lib = N.lib()
    sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends, selection = saved
    if selection is None:
        raise ValueError("the fused L2 backward needs per_pixel_sort=True and max_layers <= 32")
    device = image.device
    n = float(width * height * 4)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        nscratch = lib.tg_backward_scratch_bytes(V)
        if packed_scratch is not None:
            scratch, mode, (gV, gC, gO), loss_out = packed_scratch, N.TG_ACCUMULATE_PACKED, (None, None, None), None
        else:
            scratch, mode, (gV, gC, gO) = torch.empty(nscratch, dtype=torch.uint8, device=device), int(bool(accumulate)), out
        entry = lib.tg_blend_backward_l2_u8 if target.dtype == torch.uint8 else lib.tg_blend_backward_l2
        status = entry(
            _ptr(tri_geo), _ptr(tri_attr), _ptr(sorted_ids), _ptr(offsets), V, width, height, tile_width, tile_height,
            int(bool(per_pixel_sort)), int(max_layers), _ptr(target.contiguous()), 2.0 / n, 1.0 / n, _ptr(loss_out),
            _ptr(image), _ptr(depthmap), _ptr(final_weights), _ptr(ends), _ptr(selection), _ptr(gV), _ptr(gC), _ptr(gO),
            mode, _ptr(scratch), nscratch, C.c_void_p(stream))
        N.check("blend_backward_l2", status)
    return gV, gC, gO


def unpack_gradients_native(packed_scratch, V, width, height, out, loss_out, accumulate=False):
    """Packed accumulator of a step's views -> (gV [V,4], gC [V,3], gO [V]) and the summed mean squared error."""
    lib = N.lib()
    gV, gC, gO = out
    device = gV.device
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        N.check("unpack_gradients", lib.tg_unpack_gradients(
            _ptr(packed_scratch), packed_scratch.numel(), V, 1.0 / float(width * height * 4), _ptr(loss_out), _ptr(gV),
            _ptr(gC), _ptr(gO), int(bool(accumulate)), C.c_void_p(stream)))
    return out


def step_l2_native(vertices, indices, colors, opacities, target, width, height, tile_width, tile_height,
                   early_stopping_threshold, max_layers, out, loss_out, accumulate=True, record_timing=False,
                   packed_scratch=None, cull_tiles=False):
    """One view of an optimisation step in one native call: tile lists, forward, ``mean((image - target)**2)``
    and its gradients (forward and backward run in a single kernel).

    Default per-pixel mode with ``1 <= max_layers <= 32`` and tiles of at most 256 pixels.  ``out`` = (gV [V,4],
    gC [V,3], gO [V]) and the 0-d float32 ``loss_out`` are overwritten, or added to when ``accumulate`` is true.
    Returns (image, depthmap, final_weights, ends, timings).
    """
    lib = N.lib()
    device = vertices.device
    T, V = indices.shape[0], vertices.shape[0]
    tiles = ((width + tile_width - 1) // tile_width) * ((height + tile_height - 1) // tile_height)
    npix = float(width * height * 4)
    with torch.cuda.device(device):
        st = _state(device)
        stream = torch.cuda.current_stream(device).cuda_stream
        f32 = dict(dtype=torch.float32, device=device)
        image = torch.empty((height, width, 4), **f32)
        depthmap = torch.empty((height, width), **f32)
        final_weights = torch.empty((height, width), **f32)
        ends = torch.empty((height, width), dtype=torch.int32, device=device)
        tri_geo = torch.empty((T, N.GEO_WORDS), **f32)
        tri_attr = torch.empty((T, N.ATTR_WORDS), **f32)
        offsets = torch.empty(tiles + 1, dtype=torch.int32, device=device)
        nscratch = lib.tg_backward_scratch_bytes(V)
        if packed_scratch is not None:   # the views of a step share one accumulator, see backward_l2_native
            scratch, mode, (gV, gC, gO), loss_out = packed_scratch, N.TG_ACCUMULATE_PACKED, (None, None, None), None
        else:
            scratch, mode, (gV, gC, gO) = torch.empty(nscratch, dtype=torch.uint8, device=device), int(bool(accumulate)), out
        stage_ms = (C.c_float * 5)() if record_timing else None
        target = target.contiguous()
        cap = max(int(st.k_estimate * 1.25) + 1024, 2 * T + 1024)
        while True:
            sorted_ids = torch.empty(cap, dtype=torch.int32, device=device)
            ws = st.ensure_workspace(lib.tg_forward_workspace_bytes(T, tiles, cap))
            base = (ws.data_ptr() + 255) // 256 * 256
            slot = st.next_slot()
            info = st.info[slot]
            status = lib.tg_render_step_l2(
                _ptr(vertices), _ptr(indices), _ptr(colors), _ptr(opacities), T, V, width, height, tile_width, tile_height,
                float(early_stopping_threshold), int(max_layers), _ptr(target), 2.0 / npix, 1.0 / npix, _ptr(loss_out),
                _ptr(image), _ptr(depthmap), _ptr(final_weights), _ptr(ends), _ptr(tri_geo), _ptr(tri_attr),
                _ptr(sorted_ids), cap, _ptr(offsets), _ptr(gV), _ptr(gC), _ptr(gO), mode,
                C.c_void_p(base), ws.numel() - (base - ws.data_ptr()), _ptr(scratch), nscratch,
                C.c_void_p(info.data_ptr()), stage_ms, N.TG_FORWARD_CULL_TILES if cull_tiles else 0, C.c_void_p(stream))
            K = int(info[0])
            if status == N.TG_ERR_CAPACITY:
                cap = int(K * 1.25) + 1024
                continue
            N.check("render_step_l2", status)
            st.finish_call(slot)
            break
        st.k_estimate = K
        timings = None
        if record_timing:
            timings = {k: float(stage_ms[i]) / 1000.0 for i, k in enumerate(TIMING_KEYS)}
    return image, depthmap, final_weights, ends, timings


class Renderer(Function):
    @staticmethod
    def forward(ctx, vertices: torch.Tensor, indices: torch.Tensor, colors: torch.Tensor, opacities: torch.Tensor,
                width: int = 500, height: int = 500, tile_width: int = 16, tile_height: int = 16,
                early_stopping_threshold: float = 1 / 256, record_timing: bool = False, per_pixel_sort: bool = True,
                max_layers: int = 32):
        n, _ = vertices.shape
        check_tensor(vertices, "vertices", (n, 4))
        check_tensor(colors, "colors", (n, 3))
        check_tensor(opacities, "opacities", (n,))
        ctx.num_vertices = n
        n, _ = indices.shape
        check_tensor(indices, "indices", (n, 3), torch.int32)
        if max_layers <= 0:
            max_layers = n + 1
        ctx.width, ctx.height = width, height
        ctx.tile_width, ctx.tile_height = tile_width, tile_height
        # an output that was not used downstream arrives in backward as None instead of a tensor of zeros that
        # autograd would have to fill and the kernel to read (the depth map, in the usual image-only loss)
        ctx.set_materialize_grads(False)
        ctx.per_pixel_sort, ctx.max_layers = per_pixel_sort, max_layers
        if n < 1:
            ctx.skipped = True
            image = torch.zeros((height, width, 4), dtype=colors.dtype, device=colors.device)
            image[..., 3] = 1.0
            depthmap = torch.full((height, width), float("inf"), dtype=colors.dtype, device=colors.device)
            timings = None
            ctx.save_for_backward(vertices, colors, opacities)
        else:
            ctx.skipped = False
            (image, depthmap, final_weights, sorted_ids, offsets, tri_geo, tri_attr, ends, selection,
             timings) = forward_native(
                vertices.contiguous(), indices.contiguous(), colors.contiguous(), opacities.contiguous(), width, height,
                tile_width, tile_height, early_stopping_threshold, record_timing, per_pixel_sort, max_layers,
                cull_tiles=bool(per_pixel_sort) and CULL_TILES)
            ctx.has_selection = selection is not None
            saved = [sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends]
            ctx.save_for_backward(*(saved + ([selection] if selection is not None else [])))
        if record_timing:
            return image, depthmap, timings
        return image, depthmap

    @staticmethod
    def backward(ctx, grad_image: torch.Tensor, grad_depthmap: torch.Tensor, grad_timings=None):
        if ctx.skipped or (grad_image is None and grad_depthmap is None):
            if ctx.skipped:
                vertices, colors, opacities = ctx.saved_tensors
                gV, gC, gO = torch.zeros_like(vertices), torch.zeros_like(colors), torch.zeros_like(opacities)
            else:
                dev, V = ctx.saved_tensors[4].device, ctx.num_vertices
                gV, gC, gO = (torch.zeros((V, 4), device=dev), torch.zeros((V, 3), device=dev), torch.zeros((V,), device=dev))
        else:
            saved = tuple(ctx.saved_tensors) + (() if ctx.has_selection else (None,))
            gV, gC, gO = backward_native(grad_image, grad_depthmap, saved, ctx.num_vertices, ctx.width,
                                         ctx.height, ctx.tile_width, ctx.tile_height, ctx.per_pixel_sort, ctx.max_layers)
        return (gV, None, gC, gO, None, None, None, None, None, None, None, None)


def render(vertices: torch.Tensor, indices: torch.Tensor, colors: torch.Tensor, opacities: torch.Tensor,
           width: int = 500, height: int = 500, tile_width: int = 16, tile_height: int = 16,
           early_stopping_threshold: float = 1 / 256, record_timing: bool = False, per_pixel_sort: bool = True,
           max_layers: int = 32) -> Tuple[torch.Tensor, torch.Tensor] | Tuple[torch.Tensor, torch.Tensor, dict]:
    """Render semi-transparent triangles (same contract as the reference ``trigrad.render``).

        vertices  : (N, 4) float32 CUDA tensor (x'/w', y'/w', z'/w', 1/w') in [-1, 1] clip space
        indices   : (M, 3) int32 triangle vertex indices
        colors    : (N, 3) vertex colours, opacities : (N,) vertex opacities
        per_pixel_sort : sort fragments per pixel (default) or blend in per-tile order
        max_layers     : maximum number of layers composited per pixel, <= 0 for no limit

    Returns ``image`` (height, width, 4) whose alpha channel holds the remaining translucency,
    ``depthmap`` (height, width) and, with ``record_timing``, a dict of stage times in seconds.

    Memory: in the default mode (``per_pixel_sort`` and ``max_layers <= 32``) autograd keeps ``max_layers`` int32
    planes of the image size alive per render until its backward has run (265 MB at 1920x1080), see
    ``SELECTION_MAX_BYTES`` in this module for the switch to the list-searching backward.
    """
    if tile_width * tile_height > 1024:
        raise ValueError("tile_width * tile_height must be <= 1024")
    return Renderer.apply(vertices, indices, colors, opacities, width, height, tile_width, tile_height,
                          early_stopping_threshold, record_timing, per_pixel_sort, max_layers)
