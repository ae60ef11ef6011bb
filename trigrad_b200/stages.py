"""Stage-level access to the CUDA path: thin torch-tensor wrappers over the C-ABI stage entry points.

Each function allocates its outputs with torch, passes raw pointers and the current stream to one
``tg_*`` entry point of ``include/trigrad_b200.h`` and raises on a non-zero status.  Used by the
parity tests (one stage at a time against the oracle) and by the benchmark's per-stage timing.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _native as N


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def scene_tensors(sc):
    return (cuda(sc.vertices), cuda(sc.indices), cuda(sc.colors), cuda(sc.opacities))


def num_tiles(sc):
    return ((sc.width + sc.tile_width - 1) // sc.tile_width) * ((sc.height + sc.tile_height - 1) // sc.tile_height)


def preprocess(sc, tensors=None):
    v, i, c, o = tensors or scene_tensors(sc)
    T = i.shape[0]
    counts = torch.empty(T, dtype=torch.int32, device="cuda")
    rects = torch.empty((T, 4), dtype=torch.int32, device="cuda")
    geo = torch.empty((T, N.GEO_WORDS), dtype=torch.float32, device="cuda")
    attr = torch.empty((T, N.ATTR_WORDS), dtype=torch.float32, device="cuda")
    N.check("preprocess", N.lib().tg_preprocess(ptr(v), ptr(i), ptr(c), ptr(o), T, sc.width, sc.height, sc.tile_width,
                                                sc.tile_height, ptr(counts), ptr(rects), ptr(geo), ptr(attr), stream()))
    return counts, rects, geo, attr


def scan(counts: torch.Tensor):
    n = counts.numel()
    out = torch.empty(n + 1, dtype=torch.int32, device="cuda")
    nb = N.lib().tg_scan_scratch_bytes(n)
    scratch = torch.empty(nb + 16, dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    N.check("scan", N.lib().tg_scan(ptr(counts), ptr(out), n, ptr(scratch), nb, ptr(status), stream()))
    assert int(status[0]) == 0
    return out


def emit_keys(sc, tri_offsets, K, tensors=None):
    v, i, c, o = tensors or scene_tensors(sc)
    keys = torch.empty(max(K, 1), dtype=torch.int64, device="cuda")
    ids = torch.empty(max(K, 1), dtype=torch.int32, device="cuda")
    N.check("emit", N.lib().tg_emit_keys(ptr(v), ptr(i), i.shape[0], sc.width, sc.height, sc.tile_width, sc.tile_height,
                                         ptr(tri_offsets), ptr(keys), ptr(ids), K, stream()))
    return keys[:K], ids[:K]


class SortBuffers:
    """Ping-pong buffers and scratch for ``tg_sort_pairs`` on n pairs."""

    def __init__(self, n: int):
        self.n = n
        self.ka = torch.empty(max(n, 1), dtype=torch.int64, device="cuda")
        self.kb = torch.empty_like(self.ka)
        self.va = torch.empty(max(n, 1), dtype=torch.int32, device="cuda")
        self.vb = torch.empty_like(self.va)
        self.nbytes = N.lib().tg_sort_scratch_bytes(n)
        self.scratch = torch.empty(self.nbytes + 16, dtype=torch.uint8, device="cuda")
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")

    def load(self, keys: torch.Tensor, vals: torch.Tensor) -> None:
        self.ka[:self.n].copy_(keys)
        self.va[:self.n].copy_(vals)

    def sort(self, begin_bit: int, end_bit: int):
        """Asynchronous: launches the sort on the current stream; returns (keys, vals) views of the result."""
        in_b = C.c_int(0)
        N.check("sort", N.lib().tg_sort_pairs(ptr(self.ka), ptr(self.kb), ptr(self.va), ptr(self.vb), self.n, begin_bit,
                                              end_bit, ptr(self.scratch), self.nbytes, ptr(self.status), C.byref(in_b),
                                              stream()))
        return (self.kb[:self.n], self.vb[:self.n]) if in_b.value else (self.ka[:self.n], self.va[:self.n])


def sort_pairs(keys: torch.Tensor, vals: torch.Tensor, begin_bit=0, end_bit=64):
    n = keys.numel()
    ka = keys.clone()
    va = vals.clone()
    kb = torch.empty_like(ka)
    vb = torch.empty_like(va)
    nb = N.lib().tg_sort_scratch_bytes(n)
    scratch = torch.empty(nb + 16, dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    in_b = C.c_int(0)
    N.check("sort", N.lib().tg_sort_pairs(ptr(ka), ptr(kb), ptr(va), ptr(vb), n, begin_bit, end_bit, ptr(scratch), nb,
                                          ptr(status), C.byref(in_b), stream()))
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    return (kb, vb) if in_b.value else (ka, va)


def tile_ranges(sorted_keys: torch.Tensor, tiles: int):
    off = torch.empty(tiles + 1, dtype=torch.int32, device="cuda")
    N.check("ranges", N.lib().tg_tile_ranges(ptr(sorted_keys), sorted_keys.numel(), tiles, ptr(off), stream()))
    return off


def sort_tile_lists(entries: torch.Tensor, offsets: torch.Tensor):
    """Sorts every tile's segment of `entries` (uint64 as int64 storage) in place; returns the low words."""
    tiles = offsets.numel() - 1
    ids = torch.empty(entries.numel(), dtype=torch.int32, device="cuda")
    nscratch = N.lib().tg_tile_sort_scratch_bytes(tiles)
    scratch = torch.empty(nscratch, dtype=torch.uint8, device="cuda")
    N.check("sort_tile_lists", N.lib().tg_sort_tile_lists(ptr(entries), ptr(offsets), tiles, ptr(ids), ptr(scratch),
                                                          nscratch, stream()))
    return ids


def blend_forward(sc, geo, attr, ids, offsets, thr=1 / 256, per_pixel_sort=True, max_layers=32, save_selection=True):
    """Returns (image, depthmap, final_weights, ends, selection); selection is None when not applicable."""
    H, W = sc.height, sc.width
    planes = N.lib().tg_selection_planes(int(per_pixel_sort), int(max_layers)) if save_selection else 0
    sel = torch.empty((planes, H, W), dtype=torch.int32, device="cuda") if planes else None
    image = torch.empty((H, W, 4), dtype=torch.float32, device="cuda")
    depth = torch.empty((H, W), dtype=torch.float32, device="cuda")
    fw = torch.empty((H, W), dtype=torch.float32, device="cuda")
    ends = torch.empty((H, W), dtype=torch.int32, device="cuda")
    N.check("blend_forward", N.lib().tg_blend_forward(ptr(geo), ptr(attr), ptr(ids), ptr(offsets), W, H, sc.tile_width,
                                                      sc.tile_height, float(thr), int(per_pixel_sort), int(max_layers),
                                                      ptr(image), ptr(depth), ptr(fw), ptr(ends), ptr(sel), stream()))
    return image, depth, fw, ends, sel


def blend_step_l2(sc, geo, attr, ids, offsets, target, thr=1 / 256, max_layers=32):
    """Forward + backward of mean((image - target)^2) in one kernel.
    Returns (image, depthmap, final_weights, ends), (gV, gC, gO), loss."""
    H, W, V = sc.height, sc.width, sc.num_vertices
    image = torch.empty((H, W, 4), dtype=torch.float32, device="cuda")
    depth = torch.empty((H, W), dtype=torch.float32, device="cuda")
    fw = torch.empty((H, W), dtype=torch.float32, device="cuda")
    ends = torch.empty((H, W), dtype=torch.int32, device="cuda")
    gV = torch.zeros((V, 4), dtype=torch.float32, device="cuda")
    gC = torch.zeros((V, 3), dtype=torch.float32, device="cuda")
    gO = torch.zeros((V,), dtype=torch.float32, device="cuda")
    loss = torch.zeros((), dtype=torch.float32, device="cuda")
    nscratch = N.lib().tg_backward_scratch_bytes(V)
    scratch = torch.empty(nscratch, dtype=torch.uint8, device="cuda")
    npix = float(W * H * 4)
    N.check("blend_step_l2", N.lib().tg_blend_step_l2(
        ptr(geo), ptr(attr), ptr(ids), ptr(offsets), V, W, H, sc.tile_width, sc.tile_height, float(thr), int(max_layers),
        ptr(target), 2.0 / npix, 1.0 / npix, ptr(loss), ptr(image), ptr(depth), ptr(fw), ptr(ends), ptr(gV), ptr(gC),
        ptr(gO), 0, ptr(scratch), nscratch, stream()))
    return (image, depth, fw, ends), (gV, gC, gO), loss


def blend_backward(sc, geo, attr, ids, offsets, fwd, gimage, gdepth, per_pixel_sort=True, max_layers=32):
    image, depth, fw, ends, sel = fwd
    V = sc.num_vertices
    nscratch = N.lib().tg_backward_scratch_bytes(V)
    scratch = torch.empty(nscratch, dtype=torch.uint8, device="cuda")
    gV = torch.empty((V, 4), dtype=torch.float32, device="cuda")
    gC = torch.empty((V, 3), dtype=torch.float32, device="cuda")
    gO = torch.empty((V,), dtype=torch.float32, device="cuda")
    N.check("blend_backward", N.lib().tg_blend_backward(
        ptr(geo), ptr(attr), ptr(ids), ptr(offsets), V, sc.width, sc.height, sc.tile_width, sc.tile_height,
        int(per_pixel_sort), int(max_layers), ptr(gimage), ptr(gdepth), ptr(image), ptr(depth), ptr(fw), ptr(ends),
        ptr(sel), ptr(gV), ptr(gC), ptr(gO), 0, ptr(scratch), nscratch, stream()))
    return gV, gC, gO


