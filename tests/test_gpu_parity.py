"""GPU parity tests proper: every stage of the CUDA path, called through the C ABI, against the CPU oracle.

Bars (from the task's north star): tile counts, sort keys, sorted order and tile ranges bit-exact;
forward image within 1e-5 relative; gradients within 1e-4 relative.  Because the kernels mirror the
oracle's decision arithmetic operation by operation, fragment selection (``ends``) is also required to
be identical and the forward image is additionally checked for exact equality.
"""
import numpy as np
import pytest
import torch

import helpers as Hh
import oracle as O
from trigrad_b200 import scenes as S

pytestmark = pytest.mark.gpu

IMG_TOL = 1e-5        # forward image, relative to the image maximum
GRAD_TOL = 1e-4       # gradients, relative L2 error (the parity bar)
GRAD_TOL_MAX = 1e-3   # sanity bound on the worst element, relative to the tensor maximum: fp32 atomics
                      # accumulate in a run-dependent order and the expanded barycentric partials cancel


def edge_case_scene():
    """Degenerate, off-screen, huge and sliver triangles plus negative / mixed-sign depths."""
    v = np.array([
        [0.0, 0.0, 1.0], [0.0, 0.0, 1.0], [0.0, 0.0, 1.0],          # 0: all vertices equal (degenerate)
        [-0.5, -0.5, 2.0], [0.0, 0.0, 2.0], [0.5, 0.5, 2.0],        # 1: collinear (degenerate)
        [2.0, -0.2, 1.5], [3.0, -0.2, 1.5], [2.5, 0.4, 1.5],        # 2: right of the screen (clamped onto border)
        [-9.0, -7.0, 3.0], [9.0, -7.0, 3.0], [0.0, 11.0, 3.0],      # 3: covers everything
        [-0.9, 0.31, 0.7], [0.9, 0.3101, 0.7], [0.0, 0.3125, 0.7],  # 4: sliver across many tiles
        [-0.3, -0.8, -1.0], [0.4, -0.7, -2.0], [0.1, -0.1, -1.5],   # 5: negative depths
        [-0.8, 0.5, 1.0], [-0.2, 0.6, 4.0], [-0.5, 0.95, 2.0],      # 6: strongly varying depth
        [0.2, 0.2, 1e-3], [0.6, 0.25, 1e-3], [0.4, 0.7, 1e-3],      # 7: tiny depth (huge w)
    ], dtype=np.float32)
    idx = np.arange(24, dtype=np.int32).reshape(8, 3)
    rng = np.random.default_rng(21)
    col = rng.random((24, 3), dtype=np.float32)
    op = rng.uniform(0.2, 0.95, 24).astype(np.float32)
    return S.Scene("edge_cases", S.add_w(v), idx, col, op, 200, 120, 16, 16)


SCENES = {
    "cfg1": lambda: S.config1_icosphere(),
    "cfg2": lambda: S.config2_random10k(),
    "cfg3_small": lambda: S.config3_random200k(T=20_000, width=640, height=360),
    "cfg5_small": lambda: S.config5_overlap(T=4_000, width=320, height=192),
    "squares": lambda: S.overlapping_squares(10),
    "large": lambda: S.large_triangles(3),
    "depth_overlap": lambda: S.depth_overlap(),
    "layers40": lambda: S.full_screen_layers(40, width=48, height=40),
    "edge": edge_case_scene,
    "odd_tiles": lambda: S.random_triangles(3000, 333, 217, 0.05, 0.6, name="odd"),
}
# depth complexity far above 32 in the centre: exercises the full-batch depth cut of the selection sweep
SCENES["deep_overlap"] = lambda: S.random_triangles(12_000, 256, 160, 0.08, 0.5, centroid="gauss", centroid_sigma=0.2,
                                                    name="deep_overlap")
SCENES["odd_tiles_5x7"] = lambda: (lambda s: (setattr(s, "tile_width", 5), setattr(s, "tile_height", 7), s)[2])(
    S.random_triangles(3000, 333, 217, 0.05, 0.6, name="odd57"))
SCENES["big_tile_32x32"] = lambda: (lambda s: (setattr(s, "tile_width", 32), setattr(s, "tile_height", 32), s)[2])(
    S.random_triangles(2000, 256, 160, 0.08, 0.6, name="big32"))


@pytest.fixture(scope="module", params=list(SCENES))
def pipeline(request):
    """Run every stage once per scene through the C ABI and the oracle."""
    sc = SCENES[request.param]()
    tens = Hh.scene_tensors(sc)
    counts, rects, geo, attr = Hh.preprocess(sc, tens)
    tri_off = Hh.scan(counts)
    K = int(tri_off[-1])
    keys, ids = Hh.emit_keys(sc, tri_off, K, tens)
    tiles = Hh.num_tiles(sc)
    end_bit = 32 + max(0, int(np.ceil(np.log2(tiles)))) if tiles > 1 else 32
    skeys, sids = Hh.sort_pairs(keys, ids, 0, end_bit)
    offsets = Hh.tile_ranges(skeys, tiles)
    st = O.build_lists_staged(sc.vertices, sc.indices, sc.width, sc.height, sc.tile_width, sc.tile_height)
    return dict(sc=sc, tens=tens, counts=counts, rects=rects, geo=geo, attr=attr, tri_off=tri_off, K=K, keys=keys,
                ids=ids, skeys=skeys, sids=sids, offsets=offsets, st=st, tiles=tiles)


def test_preprocess_counts_and_rects_bit_exact(pipeline):
    p = pipeline
    assert np.array_equal(p["counts"].cpu().numpy(), p["st"].counts)
    assert np.array_equal(p["rects"].cpu().numpy(), p["st"].rects)


def test_preprocess_records_bit_exact(pipeline):
    p, sc = pipeline, pipeline["sc"]
    M = O.bary_matrices(sc.vertices, sc.indices).reshape(-1, 9)
    geo = p["geo"].cpu().numpy()
    assert np.array_equal(geo[:, :9].view(np.uint32), M.view(np.uint32))
    v = sc.vertices[sc.indices]                      # [T,3,4]
    assert np.array_equal(geo[:, 9:12], v[:, :, 2])
    assert np.array_equal(geo[:, 12:15], v[:, :, 3])
    attr = p["attr"].cpu().numpy()
    assert np.array_equal(attr[:, 0:3], sc.opacities[sc.indices])
    assert np.array_equal(attr[:, 3:12], sc.colors[sc.indices].reshape(-1, 9))
    assert np.array_equal(attr[:, 12:15], np.float32(1) / v[:, :, 3])
    assert np.array_equal(attr[:, 15:18].view(np.int32), sc.indices)
    assert np.array_equal(attr[:, 18:24], v[:, :, :2].reshape(-1, 6))


def test_scan_bit_exact(pipeline):
    p = pipeline
    assert np.array_equal(p["tri_off"].cpu().numpy().astype(np.int64), p["st"].tri_offsets)


def test_emitted_keys_bit_exact(pipeline):
    p = pipeline
    assert p["K"] == p["st"].keys_unsorted.shape[0]
    assert np.array_equal(p["keys"].cpu().numpy().view(np.uint64), p["st"].keys_unsorted)
    assert np.array_equal(p["ids"].cpu().numpy(), p["st"].ids_unsorted)


def test_sorted_keys_and_ids_bit_exact(pipeline):
    p = pipeline
    assert np.array_equal(p["skeys"].cpu().numpy().view(np.uint64), p["st"].keys_sorted)
    assert np.array_equal(p["sids"].cpu().numpy(), p["st"].ids_sorted)


def test_tile_ranges_bit_exact(pipeline):
    p = pipeline
    assert np.array_equal(p["offsets"].cpu().numpy(), p["st"].offsets)
    # and they are the reference's objects: per-tile counts cumulated (oracle native path)
    sc = p["sc"]
    li = O.build_lists(sc.vertices, sc.indices, sc.width, sc.height, sc.tile_width, sc.tile_height)
    assert np.array_equal(p["offsets"].cpu().numpy(), li.offsets)
    assert np.array_equal(p["sids"].cpu().numpy(), li.ids)


def _forward_entry_lists(sc):
    """Sorted ids and tile offsets as the whole-forward entry point builds them (fused binning, per-tile sort)."""
    from trigrad_b200 import wrapper as Wr

    t = Hh.scene_tensors(sc)
    out = Wr.forward_native(*t, sc.width, sc.height, sc.tile_width,
                            sc.tile_height, 1 / 256, False, True, 32)
    torch.cuda.synchronize()
    return out[3].cpu().numpy(), out[4].cpu().numpy(), out[0].cpu().numpy()


def test_forward_entry_lists_bit_exact(pipeline):
    """tg_render_forward takes another route to the lists (counts per tile, segmented sort): same result."""
    p = pipeline
    ids, offsets, _ = _forward_entry_lists(p["sc"])
    assert np.array_equal(offsets, p["st"].offsets)
    assert np.array_equal(ids, p["st"].ids_sorted)


def test_forward_entry_more_tiles_than_one_cta_scans():
    """Beyond 65536 tiles the tile offsets come from the device-wide scan instead of the last CTA."""
    sc = S.random_triangles(6000, 2100, 2100, 0.02, 0.6, name="many_tiles")
    sc.tile_width = sc.tile_height = 8
    assert Hh.num_tiles(sc) > 65536
    ids, offsets, _ = _forward_entry_lists(sc)
    li = O.build_lists(sc.vertices, sc.indices, sc.width, sc.height, sc.tile_width, sc.tile_height)
    assert np.array_equal(offsets, li.offsets)
    assert np.array_equal(ids, li.ids)


def test_forward_entry_very_long_tile_lists():
    """One tile with more than 16384 entries: chunks sorted in shared memory, wide steps in global memory."""
    sc = S.random_triangles(50_000, 32, 32, 0.5, 0.3, name="one_tile_50k")
    ids, offsets, image = _forward_entry_lists(sc)
    li = O.build_lists(sc.vertices, sc.indices, sc.width, sc.height, sc.tile_width, sc.tile_height)
    assert np.diff(li.offsets).max() > 16384
    assert np.array_equal(offsets, li.offsets)
    assert np.array_equal(ids, li.ids)
    of = O.forward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, sc.tile_width, sc.tile_height,
                   1 / 256, True, 32)
    assert np.array_equal(image.view(np.uint32), of.image.view(np.uint32))


@pytest.mark.parametrize("lengths", [
    [0, 1, 2, 31, 32, 33, 0, 255, 256, 257, 1023, 1024, 1025, 0, 4096, 5000, 16384],
    [16385, 3, 40_000, 0, 70_001, 1],
    [300_000],
], ids=["short_and_medium", "beyond_one_chunk", "single_300k"])
def test_sort_tile_lists_segment_lengths(lengths):
    """Segmented sort alone: every length class of the kernels, duplicates of the high word included."""
    rng = np.random.default_rng(len(lengths))
    offsets = np.zeros(len(lengths) + 1, np.int32)
    np.cumsum(lengths, out=offsets[1:])
    n = int(offsets[-1])
    hi = rng.integers(0, 1 << 32, n, dtype=np.uint64)
    hi[::3] = hi[0] if n else 0                                   # equal depths: the low word decides
    entries = np.empty(n, np.uint64)
    expect = np.empty(n, np.uint64)
    for a, b in zip(offsets[:-1], offsets[1:]):
        lo = rng.permutation(int(b - a)).astype(np.uint64)        # unique within a segment, like triangle ids
        entries[a:b] = (hi[a:b] << np.uint64(32)) | lo
        expect[a:b] = np.sort(entries[a:b])
    dev = Hh.cuda(entries.view(np.int64))
    ids = Hh.sort_tile_lists(dev, Hh.cuda(offsets))
    torch.cuda.synchronize()
    assert np.array_equal(dev.cpu().numpy().view(np.uint64), expect)
    assert np.array_equal(ids.cpu().numpy().view(np.uint32), (expect & np.uint64(0xFFFFFFFF)).astype(np.uint32))


MODES = [
    dict(per_pixel_sort=True, max_layers=32, thr=1 / 256),    # the reference default
    dict(per_pixel_sort=False, max_layers=32, thr=1 / 256),
    dict(per_pixel_sort=True, max_layers=7, thr=1 / 256),
    dict(per_pixel_sort=True, max_layers=0, thr=1 / 256),     # <= 0 means unlimited (T+1)
    dict(per_pixel_sort=False, max_layers=0, thr=0.2),
    dict(per_pixel_sort=True, max_layers=40, thr=0.5),        # second batch only while alpha > thr
]


@pytest.mark.parametrize("mode", MODES, ids=lambda m: f"sort{int(m['per_pixel_sort'])}_L{m['max_layers']}_t{m['thr']:.3f}")
def test_forward_and_backward_vs_oracle(pipeline, mode):
    p, sc = pipeline, pipeline["sc"]
    T = sc.num_triangles
    ml = mode["max_layers"] if mode["max_layers"] > 0 else T + 1
    fwd = Hh.blend_forward(sc, p["geo"], p["attr"], p["sids"], p["offsets"], mode["thr"], mode["per_pixel_sort"], ml)
    image, depth, fw, ends = [t.cpu().numpy() for t in fwd[:4]]
    of = O.forward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, sc.tile_width,
                   sc.tile_height, mode["thr"], mode["per_pixel_sort"], ml)
    assert np.array_equal(ends, of.ends), "fragment selection differs"
    assert Hh.rel_err(image, of.image) <= IMG_TOL
    assert np.array_equal(np.isinf(depth), np.isinf(of.depthmap))
    fin = np.isfinite(of.depthmap)
    assert Hh.rel_err(depth[fin], of.depthmap[fin]) <= IMG_TOL if fin.any() else True
    assert Hh.rel_err(fw, of.final_weights) <= IMG_TOL
    # the kernels mirror the oracle's arithmetic: the result is in fact identical
    assert np.array_equal(image.view(np.uint32), of.image.view(np.uint32))
    assert np.array_equal(depth.view(np.uint32), of.depthmap.view(np.uint32))

    rng = np.random.default_rng(7)
    gi = rng.normal(size=image.shape).astype(np.float32)
    gd = rng.normal(size=depth.shape).astype(np.float32)
    g = Hh.blend_backward(sc, p["geo"], p["attr"], p["sids"], p["offsets"], fwd, Hh.cuda(gi), Hh.cuda(gd),
                          mode["per_pixel_sort"], ml)
    og = O.backward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, of, gi, gd, sc.tile_width,
                    sc.tile_height, mode["per_pixel_sort"], ml)
    checks = [("saved selection" if fwd[4] is not None else "list search", g)]
    if fwd[4] is not None:
        # the same gradients without the ids saved by the forward pass (lists searched again)
        checks.append(("list search", Hh.blend_backward(sc, p["geo"], p["attr"], p["sids"], p["offsets"], fwd[:4] + (None,),
                                                        Hh.cuda(gi), Hh.cuda(gd), mode["per_pixel_sort"], ml)))
    for path, gg in checks:
      for name, a, b in zip(("vertices", "colors", "opacities"), gg, og):
        a = a.cpu().numpy()
        assert np.all(a[:, 2] == 0) if name == "vertices" else True
        err, err_max = Hh.rel_l2(a, b), Hh.rel_err(a, b)
        assert err <= GRAD_TOL, f"grad_{name} ({path}): relative L2 error {err:.3e}"
        assert err_max <= GRAD_TOL_MAX, f"grad_{name} ({path}): worst element {err_max:.3e}"


@pytest.mark.parametrize("max_layers", [32, 5])
def test_one_kernel_step_vs_oracle(pipeline, max_layers):
    """tg_blend_step_l2 (forward + backward of the mean squared error in one kernel): image identical to the
    oracle's forward, loss and gradients equal to the oracle's backward of the same loss."""
    p, sc = pipeline, pipeline["sc"]
    if sc.tile_width * sc.tile_height > 256:
        pytest.skip("the one-kernel step needs tiles of at most 256 pixels")
    rng = np.random.default_rng(11)
    target = rng.random((sc.height, sc.width, 4), dtype=np.float32)
    (image, depth, fw, ends), grads, loss = Hh.blend_step_l2(sc, p["geo"], p["attr"], p["sids"], p["offsets"],
                                                            Hh.cuda(target), 1 / 256, max_layers)
    of = O.forward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, sc.tile_width,
                   sc.tile_height, 1 / 256, True, max_layers)
    assert np.array_equal(ends.cpu().numpy(), of.ends)
    assert np.array_equal(image.cpu().numpy().view(np.uint32), of.image.view(np.uint32))
    assert np.array_equal(depth.cpu().numpy().view(np.uint32), of.depthmap.view(np.uint32))
    assert np.array_equal(fw.cpu().numpy().view(np.uint32), of.final_weights.view(np.uint32))
    n = np.float32(sc.width * sc.height * 4)
    diff = of.image - target
    ref_loss = float(np.sum(diff.astype(np.float64) ** 2) / n)
    assert abs(float(loss) - ref_loss) <= 1e-5 * ref_loss
    gi = (diff * (np.float32(2) / n)).astype(np.float32)
    og = O.backward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, of, gi,
                    np.zeros((sc.height, sc.width), np.float32), sc.tile_width, sc.tile_height, True, max_layers)
    # A gradient that is analytically zero (triangles with one colour and one opacity: no dependence on the
    # vertex positions) comes out of fp32 as cancellation noise, 1e-8 against 1e-2 for the colours.  The fp64
    # oracle tells which gradients are of that kind; those only have to be negligible here as well.
    f64 = [np.asarray(x, np.float64) for x in (sc.vertices, sc.colors, sc.opacities)]
    of64 = O.forward(f64[0], sc.indices, f64[1], f64[2], sc.width, sc.height, sc.tile_width, sc.tile_height, 1 / 256, True,
                     max_layers)
    gi64 = (of64.image - target) * (2.0 / float(n))
    og64 = O.backward(f64[0], sc.indices, f64[1], f64[2], sc.width, sc.height, of64, gi64,
                      np.zeros((sc.height, sc.width)), sc.tile_width, sc.tile_height, True, max_layers)
    whole = float(np.sqrt(sum(float(np.sum(g ** 2)) for g in og64)))
    for name, a, b, b64 in zip(("vertices", "colors", "opacities"), grads, og, og64):
        a = a.cpu().numpy()
        if float(np.linalg.norm(b64)) < 1e-4 * whole:
            assert float(np.linalg.norm(a.astype(np.float64))) <= 1e-4 * whole, f"grad_{name} should be negligible"
            continue
        err, err_max = Hh.rel_l2(a, b), Hh.rel_err(a, b)
        assert err <= GRAD_TOL, f"grad_{name}: relative L2 error {err:.3e}"
        assert err_max <= GRAD_TOL_MAX, f"grad_{name}: worst element {err_max:.3e}"


def test_large_sort_random_keys():
    """Sort alone on 3M random 45-bit keys, odd length, against numpy's stable sort."""
    rng = np.random.default_rng(3)
    n = 3_000_017
    keys = rng.integers(0, 1 << 45, n, dtype=np.int64)
    keys[::7] = keys[3]           # many duplicates: stability matters
    vals = np.arange(n, dtype=np.int32)
    sk, sv = Hh.sort_pairs(Hh.cuda(keys), Hh.cuda(vals), 0, 45)
    order = np.argsort(keys, kind="stable")
    assert np.array_equal(sk.cpu().numpy(), keys[order])
    assert np.array_equal(sv.cpu().numpy(), vals[order])


@pytest.mark.parametrize("n", [0, 1, 255, 2048, 2049, 100_000, 5_000_001])
def test_scan_sizes(n):
    rng = np.random.default_rng(n)
    x = rng.integers(0, 50, n, dtype=np.int32)
    out = Hh.scan(Hh.cuda(x)).cpu().numpy().astype(np.int64)
    ref = np.zeros(n + 1, np.int64)
    np.cumsum(x, out=ref[1:])
    assert np.array_equal(out, ref)


@pytest.mark.parametrize("n,bits", [(1, 64), (4096, 64), (4097, 40), (12345, 33), (70_000, 64)])
def test_sort_sizes(n, bits):
    rng = np.random.default_rng(n)
    keys = rng.integers(0, 1 << min(bits, 62), n, dtype=np.int64)
    vals = rng.integers(0, 1 << 31, n, dtype=np.int32)
    sk, sv = Hh.sort_pairs(Hh.cuda(keys), Hh.cuda(vals), 0, bits)
    order = np.argsort(keys, kind="stable")
    assert np.array_equal(sk.cpu().numpy(), keys[order])
    assert np.array_equal(sv.cpu().numpy(), vals[order])
