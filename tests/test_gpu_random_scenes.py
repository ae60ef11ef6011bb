"""Seeded random scenes through the whole forward entry point and both optimisation-step paths against the oracle:
triangle counts, image and tile sizes and triangle sizes drawn at random (tiny meshes, ragged image borders, tiles
of 16 to 1024 pixels, lists from empty to thousands of entries)."""
import numpy as np
import pytest
import torch

import helpers as Hh
import oracle as O
from trigrad_b200 import scenes as S
from trigrad_b200 import views
from trigrad_b200 import wrapper as Wr

pytestmark = pytest.mark.gpu


def _random_case(seed):
    rng = np.random.default_rng(1000 + seed)
    T = int(rng.choice([1, 2, 7, 60, 500, 3000, 9000]))
    W, H = int(rng.integers(5, 300)), int(rng.integers(5, 200))
    tw, th = int(rng.choice([4, 8, 16, 32])), int(rng.choice([4, 8, 16, 32]))
    edge = float(rng.choice([0.01, 0.05, 0.3, 1.5]))
    centroid = "gauss" if rng.random() < 0.4 else "uniform"
    sc = S.random_triangles(T, W, H, edge, 0.7, centroid=centroid, centroid_sigma=0.3, name=f"rand{seed}", seed=seed)
    sc.tile_width, sc.tile_height = tw, th
    return sc


@pytest.mark.parametrize("seed", range(24))
def test_random_scene_lists_image_and_step(seed):
    sc = _random_case(seed)
    t = Hh.scene_tensors(sc)
    out = Wr.forward_native(*t, sc.width, sc.height, sc.tile_width, sc.tile_height, 1 / 256, False, True, 32)
    torch.cuda.synchronize()
    li = O.build_lists(sc.vertices, sc.indices, sc.width, sc.height, sc.tile_width, sc.tile_height)
    assert np.array_equal(out[4].cpu().numpy(), li.offsets)
    assert np.array_equal(out[3].cpu().numpy(), li.ids)
    of = O.forward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, sc.tile_width, sc.tile_height,
                   1 / 256, True, 32)
    assert np.array_equal(out[7].cpu().numpy(), of.ends)
    assert np.array_equal(out[0].cpu().numpy().view(np.uint32), of.image.view(np.uint32))

    rng = np.random.default_rng(seed)
    target = rng.random((sc.height, sc.width, 4), dtype=np.float32)
    n = np.float32(sc.width * sc.height * 4)
    gi = ((of.image - target) * (np.float32(2) / n)).astype(np.float32)
    og = O.backward(sc.vertices, sc.indices, sc.colors, sc.opacities, sc.width, sc.height, of, gi,
                    np.zeros((sc.height, sc.width), np.float32), sc.tile_width, sc.tile_height, True, 32)
    whole = float(np.sqrt(sum(float(np.sum(np.asarray(g, np.float64) ** 2)) for g in og)))
    V = sc.num_vertices
    for one_kernel in (False, True):
        gV, gC, gO = torch.zeros((V, 4), device="cuda"), torch.zeros((V, 3), device="cuda"), torch.zeros((V,), device="cuda")
        loss = torch.zeros((), device="cuda")
        img = views.l2_view_step(*t, Hh.cuda(target), sc.width, sc.height, gV, gC, gO, loss, sc.tile_width, sc.tile_height,
                                 one_kernel=one_kernel)
        torch.cuda.synchronize()
        assert np.array_equal(img.cpu().numpy().view(np.uint32), of.image.view(np.uint32))
        for name, a, b in zip(("vertices", "colors", "opacities"), (gV, gC, gO), og):
            err = float(np.linalg.norm(a.cpu().numpy().astype(np.float64) - b)) / max(float(np.linalg.norm(b)), 1e-3 * whole, 1e-30)
            assert err <= 1e-4, f"seed {seed}, one_kernel {one_kernel}: grad_{name} relative L2 error {err:.3e}"
