"""GPU tests of what goes beyond the reference's behaviour: pixel-centre tile culling (the reference's TODO at
``render.cu:110``), corrected gradients outside the default mode, and the near-plane triangle splitter fused with
the projection (the reference's notebook function ``split_clipped``).  Each is checked against the CPU oracle's
restatement, which the CPU tests pin (finite differences, invariance of the render, the reference's own function).
"""
import numpy as np
import pytest
import torch

import helpers as Hh
import oracle as O
import trigrad_b200
from trigrad_b200 import scenes as S
from trigrad_b200 import views
from trigrad_b200 import wrapper as Wr

pytestmark = pytest.mark.gpu


# ---- tile culling -------------------------------------------------------------------------------------------
CULL_SCENES = {
    "cfg1": S.config1_icosphere,
    "cfg2": S.config2_random10k,
    "cfg3_small": lambda: S.config3_random200k(T=20_000, width=640, height=360),
    "cfg5_small": lambda: S.config5_overlap(T=4_000, width=320, height=192),
    "odd_tiles": lambda: S.random_triangles(3000, 333, 217, 0.05, 0.6, name="odd"),
    "odd_tiles_5x7": lambda: (lambda s: (setattr(s, "tile_width", 5), setattr(s, "tile_height", 7), s)[2])(
        S.random_triangles(3000, 333, 217, 0.05, 0.6, name="odd57")),
    "depth_overlap": S.depth_overlap,
    "sphere_view": lambda: S.config4_view(S.displaced_sphere(5), S.camera_ring(8)[3], 640, 360),
}


@pytest.mark.parametrize("name", list(CULL_SCENES))
def test_culled_lists_bit_exact_and_render_unchanged(name):
    sc = CULL_SCENES[name]()
    t = Hh.scene_tensors(sc)
    args = (sc.width, sc.height, sc.tile_width, sc.tile_height, 1 / 256, False, True, 32)
    plain = Wr.forward_native(*t, *args)
    culled = Wr.forward_native(*t, *args, cull_tiles=True)
    torch.cuda.synchronize()
    li = O.build_lists(sc.vertices, sc.indices, sc.width, sc.height, sc.tile_width, sc.tile_height, cull=True)
    assert np.array_equal(culled[4].cpu().numpy(), li.offsets)
    assert np.array_equal(culled[3].cpu().numpy(), li.ids)
    assert culled[3].numel() <= plain[3].numel()
    for k in (0, 1, 2, 7):          # image, depth map, final weights, ends
        assert torch.equal(plain[k], culled[k])


@pytest.mark.parametrize("one_kernel", [False, True])
def test_view_step_gradients_do_not_depend_on_culling(one_kernel):
    sc = S.config2_random10k()
    v, i, c, o = Hh.scene_tensors(sc)
    V = sc.num_vertices
    target = Hh.cuda(sc.target())
    out = []
    for cull in (False, True):
        gV, gC, gO = torch.zeros((V, 4), device="cuda"), torch.zeros((V, 3), device="cuda"), torch.zeros((V,), device="cuda")
        loss = torch.zeros((), device="cuda")
        img = views.l2_view_step(v, i, c, o, target, sc.width, sc.height, gV, gC, gO, loss, one_kernel=one_kernel,
                                 cull_tiles=cull)
        out.append((img, float(loss), gV.cpu().numpy(), gC.cpu().numpy(), gO.cpu().numpy()))
    assert torch.equal(out[0][0], out[1][0])
    assert abs(out[0][1] - out[1][1]) <= 1e-6 * out[0][1]
    for a, b in zip(out[0][2:], out[1][2:]):
        assert Hh.rel_l2(a, b) <= 1e-5


# ---- corrected gradients ----------------------------------------------------------------------------------------
CORRECTED_CASES = {
    "layers60_tileorder": (lambda: S.full_screen_layers(60, width=48, height=40), dict(per_pixel_sort=False, max_layers=61, thr=1 / 256)),
    "layers40_per_pixel": (lambda: S.full_screen_layers(40, width=48, height=40, reverse=True), dict(per_pixel_sort=True, max_layers=40, thr=0.0)),
    "deep_overlap_per_pixel_unlimited": (lambda: S.random_triangles(6000, 128, 96, 0.08, 0.5, centroid="gauss", centroid_sigma=0.2,
                                                                    name="deep"), dict(per_pixel_sort=True, max_layers=0, thr=1 / 256)),
    "random_tileorder": (lambda: S.random_triangles(3000, 333, 217, 0.05, 0.6, name="odd"), dict(per_pixel_sort=False, max_layers=0, thr=0.05)),
    "default_mode": (S.config2_random10k, dict(per_pixel_sort=True, max_layers=32, thr=1 / 256)),
}


def _render_grads(fn, sc, mode, gi, gd):
    v, i, c, o = Hh.scene_tensors(sc)
    v.requires_grad_(), c.requires_grad_(), o.requires_grad_()
    image, depth = fn(v, i, c, o, sc.width, sc.height, sc.tile_width, sc.tile_height, mode["thr"], False,
                      mode["per_pixel_sort"], mode["max_layers"])
    d0 = torch.where(torch.isfinite(depth), depth, torch.zeros_like(depth))
    ((image * Hh.cuda(gi)).sum() + (d0 * Hh.cuda(gd)).sum()).backward()
    return image.detach().cpu().numpy(), [x.grad.cpu().numpy() for x in (v, c, o)]


@pytest.mark.parametrize("name", list(CORRECTED_CASES))
def test_corrected_gradients_match_the_oracle(name):
    make, mode = CORRECTED_CASES[name]
    sc = make()
    rng = np.random.default_rng(7)
    gi = rng.normal(size=(sc.height, sc.width, 4)).astype(np.float32)
    gd = rng.normal(size=(sc.height, sc.width)).astype(np.float32)
    image, grads = _render_grads(trigrad_b200.render_corrected, sc, mode, gi, gd)
    # truth: the fp64 oracle's corrected backward (which the CPU tests hold against finite differences)
    f64 = [np.asarray(x, np.float64) for x in (sc.vertices, sc.colors, sc.opacities)]
    of = O.forward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, sc.tile_width, sc.tile_height,
                   mode["thr"], mode["per_pixel_sort"], mode["max_layers"])
    assert np.array_equal(image.view(np.uint32), of.image.view(np.uint32))
    of64 = O.forward(f64[0], sc.indices, f64[1], f64[2], sc.width, sc.height, sc.tile_width, sc.tile_height, mode["thr"],
                     mode["per_pixel_sort"], mode["max_layers"])
    if not np.array_equal(of64.ends, of.ends):
        pytest.skip("fp32 and fp64 blend different fragments on this scene")
    og = O.backward(f64[0], sc.indices, f64[1], f64[2], sc.width, sc.height, of64, gi.astype(np.float64),
                    gd.astype(np.float64), sc.tile_width, sc.tile_height, mode["per_pixel_sort"], mode["max_layers"],
                    corrected=True)
    whole = float(np.sqrt(sum(float(np.sum(g ** 2)) for g in og)))
    for nm, a, b in zip(("vertices", "colors", "opacities"), grads, og):
        if float(np.linalg.norm(b)) < 1e-4 * whole:      # analytically (almost) zero: only has to be negligible
            assert float(np.linalg.norm(a.astype(np.float64))) <= 1e-3 * whole, nm
            continue
        assert Hh.rel_l2(a, b) <= 2e-4, f"grad_{nm}: {Hh.rel_l2(a, b):.3e}"


def test_corrected_gradients_equal_render_gradients_in_the_default_mode():
    sc = S.config2_random10k()
    mode = dict(per_pixel_sort=True, max_layers=32, thr=1 / 256)
    rng = np.random.default_rng(8)
    gi = rng.normal(size=(sc.height, sc.width, 4)).astype(np.float32)
    gd = rng.normal(size=(sc.height, sc.width)).astype(np.float32)
    ia, a = _render_grads(trigrad_b200.render, sc, mode, gi, gd)
    ib, b = _render_grads(trigrad_b200.render_corrected, sc, mode, gi, gd)
    assert np.array_equal(ia, ib)
    for x, y in zip(a, b):
        assert Hh.rel_l2(x, y) <= 1e-4


def test_literal_gradients_differ_from_corrected_ones_in_tile_order_mode():
    """render() keeps the reference's behaviour (drop-in); the corrected variant is a different number there."""
    make, mode = CORRECTED_CASES["layers60_tileorder"]
    sc = make()
    rng = np.random.default_rng(7)
    gi = rng.normal(size=(sc.height, sc.width, 4)).astype(np.float32)
    gd = np.zeros((sc.height, sc.width), np.float32)
    _, a = _render_grads(trigrad_b200.render, sc, mode, gi, gd)
    _, b = _render_grads(trigrad_b200.render_corrected, sc, mode, gi, gd)
    assert Hh.rel_l2(a[1], b[1]) > 1e-2


# ---- near-plane splitting -------------------------------------------------------------------------------------
def _camera_inside_mesh():
    """A displaced sphere seen from a camera INSIDE it, looking along +z: many triangles cross the near plane."""
    mesh = S.displaced_sphere(3)
    P = S.perspective(60.0, 0.1, 100.0, 320, 192)
    pv = (P @ S.lookat([0.0, 0.0, 0.35], target=(0.0, 0.0, 5.0))).astype(np.float32)
    return mesh, pv


def test_project_clip_matches_the_oracle():
    mesh, pv = _camera_inside_mesh()
    pts, i, c, o = Hh.cuda(mesh.points), Hh.cuda(mesh.indices), Hh.cuda(mesh.colors), Hh.cuda(mesh.opacities)
    ov, oi, oc, oo = trigrad_b200.project_clip(pts, i, c, o, pv)
    torch.cuda.synchronize()
    T = mesh.indices.shape[0]
    assert ov.shape == (6 * T, 4) and oi.shape == (2 * T, 3)
    assert np.array_equal(oi.cpu().numpy().reshape(-1), np.arange(6 * T))
    rv, rc, ro, slots, plan, _ = O.project_clip(mesh.points.astype(np.float64), pv.astype(np.float64), mesh.indices,
                                                mesh.colors.astype(np.float64), mesh.opacities.astype(np.float64))
    n_cut = sum(1 for (_, b, _) in plan if b >= 0)
    assert n_cut > 50 and len(slots) < 2 * T          # the case is not trivial: cuts and drops both occur
    got_v = ov.cpu().numpy().reshape(2 * T, 3, 4)
    got_c = oc.cpu().numpy().reshape(2 * T, 3, 3)
    got_o = oo.cpu().numpy().reshape(2 * T, 3)
    assert Hh.rel_err(got_v[slots].reshape(-1, 4), rv) <= 2e-5
    assert Hh.rel_err(got_c[slots].reshape(-1, 3), rc) <= 1e-5
    assert Hh.rel_err(got_o[slots].reshape(-1), ro) <= 1e-5
    unused = np.setdiff1d(np.arange(2 * T), slots)
    assert np.all(got_v[unused] == np.array([0, 0, 0, 1], np.float32)) and np.all(got_o[unused] == 0)


def test_project_clip_backward_matches_the_oracle_vjp():
    mesh, pv = _camera_inside_mesh()
    pts, i = Hh.cuda(mesh.points).requires_grad_(), Hh.cuda(mesh.indices)
    c, o = Hh.cuda(mesh.colors).requires_grad_(), Hh.cuda(mesh.opacities).requires_grad_()
    ov, oi, oc, oo = trigrad_b200.project_clip(pts, i, c, o, pv)
    T = mesh.indices.shape[0]
    rng = np.random.default_rng(12)
    p64 = mesh.points.astype(np.float64)
    rv, rc, ro, slots, plan, clip_soup = O.project_clip(p64, pv.astype(np.float64), mesh.indices,
                                                        mesh.colors.astype(np.float64), mesh.opacities.astype(np.float64))
    n = rv.shape[0]
    up_v, up_c, up_o = rng.normal(size=(n, 4)), rng.normal(size=(n, 3)), rng.normal(size=(n,))
    # the same upstream gradients on the kernel's fixed two-slots-per-triangle layout (zero on unused slots)
    gv = np.zeros((2 * T, 3, 4), np.float32); gv[slots] = up_v.reshape(-1, 3, 4)
    gc = np.zeros((2 * T, 3, 3), np.float32); gc[slots] = up_c.reshape(-1, 3, 3)
    go = np.zeros((2 * T, 3), np.float32); go[slots] = up_o.reshape(-1, 3)
    torch.autograd.backward((ov, oc, oo), (Hh.cuda(gv.reshape(-1, 4)), Hh.cuda(gc.reshape(-1, 3)), Hh.cuda(go.reshape(-1))))
    ref = O.project_clip_vjp(p64, pv.astype(np.float64), mesh.colors, mesh.opacities, plan, clip_soup,
                             gv[slots].reshape(-1, 4), gc[slots].reshape(-1, 3), go[slots].reshape(-1))
    for nm, a, b in zip(("points", "colors", "opacities"), (pts.grad, c.grad, o.grad), ref):
        assert Hh.rel_l2(a.cpu().numpy(), b) <= 1e-4, nm


def test_render_of_a_clipped_mesh_matches_the_oracle_and_is_differentiable():
    """project_clip -> render -> loss -> backward to world space; the image equals the oracle's render of the same soup."""
    mesh, pv = _camera_inside_mesh()
    W, H = 320, 192
    pts, i = Hh.cuda(mesh.points).requires_grad_(), Hh.cuda(mesh.indices)
    c, o = Hh.cuda(mesh.colors).requires_grad_(), Hh.cuda(mesh.opacities).requires_grad_()
    v, idx, cc, oo = trigrad_b200.project_clip(pts, i, c, o, pv)
    image, _ = trigrad_b200.render(v, idx, cc, oo, W, H)
    target = torch.rand((H, W, 4), device="cuda")
    torch.mean((image - target) ** 2).backward()
    torch.cuda.synchronize()
    assert torch.isfinite(image).all() and float((image[..., 3] < 1).float().mean()) > 0.5     # the mesh fills the view
    of = O.forward(v.detach().cpu().numpy(), idx.cpu().numpy(), cc.detach().cpu().numpy(), oo.detach().cpu().numpy(), W, H)
    assert np.array_equal(image.detach().cpu().numpy().view(np.uint32), of.image.view(np.uint32))
    for g in (pts.grad, c.grad, o.grad):
        assert torch.isfinite(g).all() and float(g.abs().sum()) > 0


# ---- packed input layout and the OBJ reader ---------------------------------------------------------------------
@pytest.mark.parametrize("mode", [dict(per_pixel_sort=True, max_layers=32), dict(per_pixel_sort=False, max_layers=0),
                                  dict(per_pixel_sort=True, max_layers=40)], ids=["default", "tile_order", "40_layers"])
def test_render_packed_equals_render(mode):
    """faces [T,4] + rgba [V,4] through ``render_packed`` against the reference layout through ``render``: identical
    image and depth map, gradients equal up to the order of the float atomics."""
    sc = S.config2_random10k()
    v, i, c, o = Hh.scene_tensors(sc)
    rgba, faces = trigrad_b200.pack_mesh(c, o, i)
    assert torch.equal(rgba[:, :3], c) and torch.equal(rgba[:, 3], o) and torch.equal(faces[:, :3], i)
    rng = np.random.default_rng(4)
    gi = Hh.cuda(rng.normal(size=(sc.height, sc.width, 4)).astype(np.float32))
    gd = Hh.cuda(rng.normal(size=(sc.height, sc.width)).astype(np.float32))

    def loss(image, depth):
        d0 = torch.where(torch.isfinite(depth), depth, torch.zeros_like(depth))
        return (image * gi).sum() + (d0 * gd).sum()

    va, ca, oa = v.clone().requires_grad_(), c.clone().requires_grad_(), o.clone().requires_grad_()
    ia, da = trigrad_b200.render(va, i, ca, oa, sc.width, sc.height, 16, 16, 1 / 256, False, **mode)
    loss(ia, da).backward()
    vb, rb = v.clone().requires_grad_(), rgba.clone().requires_grad_()
    ib, db = trigrad_b200.render_packed(vb, faces, rb, sc.width, sc.height, 16, 16, 1 / 256, False, **mode)
    loss(ib, db).backward()
    assert torch.equal(ia, ib) and torch.equal(da, db)
    assert Hh.rel_l2(vb.grad.cpu().numpy(), va.grad.cpu().numpy()) <= 1e-5
    assert Hh.rel_l2(rb.grad[:, :3].cpu().numpy(), ca.grad.cpu().numpy()) <= 1e-5
    assert Hh.rel_l2(rb.grad[:, 3].cpu().numpy(), oa.grad.cpu().numpy()) <= 1e-5


def test_obj_mesh_renders_like_the_oracle():
    """A mesh read from OBJ text (an octahedron written out here) through project_native + render, against the oracle."""
    text = "\n".join(["v 1 0 0", "v -1 0 0", "v 0 1 0", "v 0 -1 0", "v 0 0 1", "v 0 0 -1",
                      "f 1 3 5", "f 3 2 5", "f 2 4 5", "f 4 1 5", "f 3 1 6", "f 2 3 6", "f 4 2 6", "f 1 4 6"])
    pts, faces = trigrad_b200.loads_obj(text)
    assert pts.shape == (6, 3) and faces.shape == (8, 3)
    pv = S.camera_ring(8, width=256, height=192)[1]
    verts = views.project_native(Hh.cuda(pts), pv)
    rng = np.random.default_rng(6)
    col, op = rng.random((6, 3), dtype=np.float32), rng.uniform(0.3, 0.9, 6).astype(np.float32)
    image, depth = trigrad_b200.render(verts, Hh.cuda(faces), Hh.cuda(col), Hh.cuda(op), 256, 192)
    of = O.forward(verts.cpu().numpy(), faces, col, op, 256, 192)
    assert np.array_equal(image.cpu().numpy().view(np.uint32), of.image.view(np.uint32))
    assert int(of.ends.max()) == 2          # front and back face
