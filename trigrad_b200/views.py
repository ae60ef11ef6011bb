"""Batches of views over several GPUs: contiguous view sharding and one all-reduce of the gradients.

The reference renders one view per call and has no multi-device code.  Views are independent, so a
batch shards with no data-path exchange: rank r of N renders views [r*B/N, (r+1)*B/N) of the same
mesh (every GPU holds the whole mesh).  World-space gradients of positions, colours and opacities
accumulate over the rank's views into ONE contiguous fp32 buffer laid out as
``[gP (V,3) | gC (V,3) | gO (V) | loss]``; a single ``all_reduce(SUM)`` over NCCL then runs in place on that
buffer.  The projection world -> NDC (the reference viewer's tensor operations, ``viewer.py:274-280``) and its
VJP are one kernel each (``tg_project`` / ``tg_project_backward``, used by ``l2_world_view_step``); ``project``
is the same map in torch operations for callers that want autograd through it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

import torch

from . import wrapper as _w
from .wrapper import render as _render


def shard_views(n_views: int, rank: int, world_size: int) -> range:
    """Contiguous block of views of `rank`; blocks differ by at most one view and cover [0, n_views)."""
    if not (0 <= rank < world_size):
        raise ValueError("rank out of range")
    base, extra = divmod(n_views, world_size)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def project(points: torch.Tensor, pv: torch.Tensor) -> torch.Tensor:
    """World points (V,3) -> render vertices (x/w', y/w', z/w', 1/w'), differentiable."""
    ones = torch.ones((points.shape[0], 1), dtype=points.dtype, device=points.device)
    clip = torch.cat([points, ones], dim=1) @ pv.T
    inv_w = 1.0 / clip[:, 3:4]
    return torch.cat([clip[:, :3] * inv_w, inv_w], dim=1).contiguous()


@dataclass
class GradBuffer:
    """One contiguous fp32 buffer holding the three gradients, with typed views into it."""

    flat: torch.Tensor
    points: torch.Tensor     # (V,3) or (V,4) view
    colors: torch.Tensor     # (V,3) view
    opacities: torch.Tensor  # (V,)  view
    loss: torch.Tensor       # 0-d view of the last element: the summed loss rides along in the same all-reduce

    @staticmethod
    def allocate(num_vertices: int, device, position_components: int = 3) -> "GradBuffer":
        """position_components = 3 for world-space positions, 4 for render-space (x, y, z, w) vertices."""
        V, p = num_vertices, position_components
        flat = torch.zeros((p + 4) * V + 1, dtype=torch.float32, device=device)
        return GradBuffer(flat, flat[:p * V].view(V, p), flat[p * V:(p + 3) * V].view(V, 3), flat[(p + 3) * V:(p + 4) * V],
                          flat[(p + 4) * V])

    def zero_(self) -> None:
        self.flat.zero_()


class PackedGradients:
    """One accumulator for the gradients and the loss of all views of a step (``tg_unpack_gradients``).

    The gradient kernels add into it with atomic vector reductions, from any number of streams; it is cleared once
    per step and unpacked once per step instead of once per view.  Render-space gradients only: views that need
    their own vertex gradient (a projection VJP per view) cannot share it for the positions.
    """

    def __init__(self, num_vertices: int, device):
        from . import _native as N

        self.num_vertices = num_vertices
        self.scratch = torch.zeros(N.lib().tg_backward_scratch_bytes(num_vertices), dtype=torch.uint8, device=device)

    def zero_(self) -> None:
        self.scratch.zero_()

    def unpack(self, width: int, height: int, grad_vertices: torch.Tensor, grad_colors: torch.Tensor,
               grad_opacities: torch.Tensor, loss: torch.Tensor, accumulate: bool = False) -> None:
        """Writes (or adds) the sums; ``loss`` receives the sum of the views' mean squared errors."""
        _w.unpack_gradients_native(self.scratch, self.num_vertices, width, height,
                                   (grad_vertices, grad_colors, grad_opacities), loss, accumulate)


def render_views_l2(points: torch.Tensor, indices: torch.Tensor, colors: torch.Tensor, opacities: torch.Tensor,
                    pvs: torch.Tensor, targets: Sequence[torch.Tensor] | torch.Tensor, view_ids: Sequence[int],
                    width: int, height: int, grads: GradBuffer, render_fn: Callable = _render,
                    **render_kwargs) -> torch.Tensor:
    """Render the given views, accumulate d(sum of per-view MSE)/d(points, colors, opacities) into `grads`.

    Returns the summed loss (a 0-d tensor on the device).  `targets[k]` is the (H,W,4) target of view k.
    """
    total = torch.zeros((), dtype=torch.float32, device=points.device)
    for k in view_ids:
        p = points.detach().requires_grad_(True)
        c = colors.detach().requires_grad_(True)
        o = opacities.detach().requires_grad_(True)
        verts = project(p, pvs[k])
        out = render_fn(verts, indices, c, o, width, height, **render_kwargs)
        image = out[0]
        loss = torch.mean((image - targets[k]) ** 2)
        gp, gc, go = torch.autograd.grad(loss, (p, c, o))
        grads.points += gp
        grads.colors += gc
        grads.opacities += go
        total = total + loss.detach()
    return total


def l2_view_step(vertices: torch.Tensor, indices: torch.Tensor, colors: torch.Tensor, opacities: torch.Tensor,
                 target: torch.Tensor, width: int, height: int, grad_vertices: torch.Tensor, grad_colors: torch.Tensor,
                 grad_opacities: torch.Tensor, loss: torch.Tensor, tile_width: int = 16, tile_height: int = 16,
                 early_stopping_threshold: float = 1 / 256, max_layers: int = 32, one_kernel: bool = False,
                 packed: "PackedGradients | None" = None, cull_tiles: bool = True) -> torch.Tensor:
    """One view of a multi-view optimisation step without autograd: forward, then the backward of
    ``mean((image - target)**2)`` fused into the gradient kernel.  With ``one_kernel`` (tiles of up to 256 pixels)
    both directions run in one compositing kernel: a few percent faster for a single stream of views and on scenes
    with long tile lists, slower when several streams of views overlap on one GPU (measured on B200).

    Adds the view's gradients to ``grad_vertices [V,4]`` (render-space x, y, z, w), ``grad_colors [V,3]``,
    ``grad_opacities [V]`` and its loss to the 0-d float32 tensor ``loss`` - no gradient image, no per-view
    gradient tensors, no elementwise kernels.  Default per-pixel mode only (``max_layers`` in 1..32); use
    ``render`` with autograd for anything else.  Returns the rendered image.

    With ``packed`` the gradients and the loss go into that accumulator instead (the four gradient / loss arguments
    may be None): no clearing and no unpacking per view, see ``PackedGradients``.  ``cull_tiles`` (default) keeps
    (triangle, tile) pairs that cannot cover a pixel out of the tile lists; results are identical either way.
    """
    if not (1 <= max_layers <= 32):
        raise ValueError("l2_view_step needs 1 <= max_layers <= 32")
    n, _ = vertices.shape
    _w.check_tensor(vertices, "vertices", (n, 4))
    _w.check_tensor(colors, "colors", (n, 3))
    _w.check_tensor(opacities, "opacities", (n,))
    m, _ = indices.shape
    _w.check_tensor(indices, "indices", (m, 3), torch.int32)
    if target.dtype == torch.uint8:
        # 8-bit RGBA target (value / 255): a quarter of the bytes per view; the two-kernel path reads it directly
        if one_kernel:
            raise ValueError("the one-kernel step takes a float32 target")
        _w.check_tensor(target, "target", (height, width, 4), torch.uint8)
    else:
        _w.check_tensor(target, "target", (height, width, 4))
    if tile_width * tile_height > 1024:
        raise ValueError("tile_width * tile_height must be <= 1024")
    if m < 1:
        if packed is not None:
            raise ValueError("a mesh without triangles cannot use the packed accumulator")
        tf = target.float() / 255 if target.dtype == torch.uint8 else target
        loss += torch.mean((torch.tensor([0.0, 0.0, 0.0, 1.0], device=target.device) - tf) ** 2)
        return None
    grads = (grad_vertices, grad_colors, grad_opacities)
    if one_kernel and tile_width * tile_height <= 256:
        # forward, loss and gradients in one native call (one compositing kernel for both directions)
        return _w.step_l2_native(vertices.contiguous(), indices.contiguous(), colors.contiguous(), opacities.contiguous(),
                                 target, width, height, tile_width, tile_height, early_stopping_threshold, max_layers,
                                 grads, loss, accumulate=True,
                                 packed_scratch=None if packed is None else packed.scratch, cull_tiles=cull_tiles)[0]
    (image, depthmap, final_weights, sorted_ids, offsets, tri_geo, tri_attr, ends, selection, _) = _w.forward_native(
        vertices.contiguous(), indices.contiguous(), colors.contiguous(), opacities.contiguous(), width, height,
        tile_width, tile_height, early_stopping_threshold, False, True, max_layers, cull_tiles=cull_tiles)
    saved = (sorted_ids, offsets, tri_geo, tri_attr, image, depthmap, final_weights, ends, selection)
    _w.backward_l2_native(target, saved, n, width, height, tile_width, tile_height, True, max_layers, grads, loss,
                          accumulate=True, packed_scratch=None if packed is None else packed.scratch)
    return image


def _pv_host(pv):
    """Row-major 4x4 float32 matrix in host memory (a CUDA tensor is copied down, which synchronises)."""
    import numpy as np

    if isinstance(pv, torch.Tensor):
        pv = pv.detach().cpu().numpy()
    m = np.ascontiguousarray(pv, dtype=np.float32)
    if m.shape != (4, 4):
        raise ValueError("pv must be a 4x4 matrix")
    return m


def project_native(points: torch.Tensor, pv) -> torch.Tensor:
    """World points (V,3) -> render vertices (V,4) in one kernel (``tg_project``); ``pv`` best given on the host."""
    import ctypes as C

    from . import _native as N

    _w.check_tensor(points, "points", (points.shape[0], 3))
    m = _pv_host(pv)
    out = torch.empty((points.shape[0], 4), dtype=torch.float32, device=points.device)
    with torch.cuda.device(points.device):
        stream = torch.cuda.current_stream(points.device).cuda_stream
        N.check("project", N.lib().tg_project(C.c_void_p(points.data_ptr()), points.shape[0], m.ctypes.data_as(C.c_void_p),
                                              C.c_void_p(out.data_ptr()), C.c_void_p(stream)))
    return out


def project_backward_native(points: torch.Tensor, pv, grad_vertices: torch.Tensor, grad_points: torch.Tensor,
                            accumulate: bool = True) -> torch.Tensor:
    """``grad_points (V,3)`` += (or =) the vector-Jacobian product of ``project_native`` with ``grad_vertices (V,4)``."""
    import ctypes as C

    from . import _native as N

    V = points.shape[0]
    _w.check_tensor(points, "points", (V, 3))
    _w.check_tensor(grad_vertices, "grad_vertices", (V, 4))
    _w.check_tensor(grad_points, "grad_points", (V, 3))
    m = _pv_host(pv)
    with torch.cuda.device(points.device):
        stream = torch.cuda.current_stream(points.device).cuda_stream
        N.check("project_backward", N.lib().tg_project_backward(
            C.c_void_p(points.data_ptr()), V, m.ctypes.data_as(C.c_void_p), C.c_void_p(grad_vertices.data_ptr()),
            C.c_void_p(grad_points.data_ptr()), int(bool(accumulate)), C.c_void_p(stream)))
    return grad_points


def l2_world_view_step(points: torch.Tensor, pv, indices: torch.Tensor, colors: torch.Tensor, opacities: torch.Tensor,
                       target: torch.Tensor, width: int, height: int, grad_points: torch.Tensor, grad_colors: torch.Tensor,
                       grad_opacities: torch.Tensor, loss: torch.Tensor, tile_width: int = 16, tile_height: int = 16,
                       early_stopping_threshold: float = 1 / 256, max_layers: int = 32,
                       one_kernel: bool = False, packed: "PackedGradients | None" = None) -> torch.Tensor:
    """``l2_view_step`` for a mesh in world space seen through the 4x4 matrix ``pv``: projection, rendering step and
    the projection's VJP without torch tensor operations.  ``grad_points [V,3]`` accumulates the world-space
    gradient; the other arguments are those of ``l2_view_step``.  Returns the rendered image.

    With ``packed`` (a ``PackedGradients`` that is all zero, one per stream) the view's gradients stay in that
    accumulator through the backward kernel and one more kernel (``tg_unpack_project_backward``) carries them
    through the projection's VJP into the three tensors and ``loss`` with atomic additions and leaves the
    accumulator zero again: no per-view clear, no render-space gradient tensor, and views on several streams may
    add into the same tensors."""
    m = _pv_host(pv)
    verts = project_native(points, m)
    if packed is not None:
        import ctypes as C

        from . import _native as N

        image = l2_view_step(verts, indices, colors, opacities, target, width, height, None, None, None, None, tile_width,
                             tile_height, early_stopping_threshold, max_layers, one_kernel, packed=packed)
        with torch.cuda.device(points.device):
            stream = torch.cuda.current_stream(points.device).cuda_stream
            N.check("unpack_project_backward", N.lib().tg_unpack_project_backward(
                C.c_void_p(packed.scratch.data_ptr()), packed.scratch.numel(), points.shape[0],
                C.c_void_p(points.data_ptr()), m.ctypes.data_as(C.c_void_p), 1.0 / float(width * height * 4),
                C.c_void_p(loss.data_ptr()), C.c_void_p(grad_points.data_ptr()), C.c_void_p(grad_colors.data_ptr()),
                C.c_void_p(grad_opacities.data_ptr()), C.c_void_p(stream)))
        return image
    gverts = torch.zeros_like(verts)
    image = l2_view_step(verts, indices, colors, opacities, target, width, height, gverts, grad_colors, grad_opacities, loss,
                         tile_width, tile_height, early_stopping_threshold, max_layers, one_kernel)
    project_backward_native(points, m, gverts, grad_points, accumulate=True)
    return image


def allreduce_gradients(grads: GradBuffer, loss: torch.Tensor | None = None, group=None) -> None:
    """Sum the gradient buffer (and optionally the loss) over all ranks, in place, with one collective each."""
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    dist.all_reduce(grads.flat, op=dist.ReduceOp.SUM, group=group)
    if loss is not None:
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
