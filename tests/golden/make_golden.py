"""Record golden vectors from the reference's own CUDA build.

The reference (Davidxdydz/trigrad) ships no golden vectors and runs only on a GPU.  This script is
meant to be executed on a machine with a CUDA device where ``oracle/_ref/`` holds the reference
extension built by ``oracle/build_ref.py`` from the unmodified reference sources.  For a few small
seeded scenes it calls the reference's ``render_forward`` / ``render_backward``
(``src/trigrad/module.cu:8-9``) and stores inputs-independent outputs as compressed ``.npz``:

    image, depthmap, final_weights, ends, offsets, sorted_ids, grad_vertices, grad_colors, grad_opacities

The scenes themselves are regenerated from ``trigrad_b200.scenes`` (seeded) by the tests, so only the
outputs are stored.  The upstream gradients are seeded N(0,1) draws (seed 7).

Usage (on the GPU machine):  python tests/golden/make_golden.py <output_dir>
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

from trigrad_b200 import scenes as S  # noqa: E402


def golden_scenes():
    """name -> (scene, mode kwargs).  Kept small: the vectors are committed."""
    out = {}
    out["squares_default"] = (S.overlapping_squares(10), dict(per_pixel_sort=True, max_layers=32, thr=1 / 256))
    out["large_default"] = (S.large_triangles(3), dict(per_pixel_sort=True, max_layers=32, thr=1 / 256))
    out["depth_overlap_default"] = (S.depth_overlap(), dict(per_pixel_sort=True, max_layers=32, thr=1 / 256))
    out["layers40_default"] = (S.full_screen_layers(40, width=48, height=40), dict(per_pixel_sort=True, max_layers=32, thr=1 / 256))
    out["layers60_tileorder"] = (S.full_screen_layers(60, width=48, height=40), dict(per_pixel_sort=False, max_layers=61, thr=1 / 256))
    out["cfg1_128_default"] = (S.config1_icosphere(width=128, height=128), dict(per_pixel_sort=True, max_layers=32, thr=1 / 256))
    out["cfg1_128_tileorder"] = (S.config1_icosphere(width=128, height=128), dict(per_pixel_sort=False, max_layers=32, thr=1 / 256))
    out["random2k_default"] = (S.random_triangles(2000, 160, 160, 0.05, 0.6, name="random2k"),
                               dict(per_pixel_sort=True, max_layers=32, thr=1 / 256))
    out["overlap3k_L8"] = (S.config5_overlap(T=3000, width=160, height=96), dict(per_pixel_sort=True, max_layers=8, thr=1 / 256))
    return out


def upstream(scene):
    rng = np.random.default_rng(7)
    gi = rng.normal(size=(scene.height, scene.width, 4)).astype(np.float32)
    gd = rng.normal(size=(scene.height, scene.width)).astype(np.float32)
    return gi, gd


def main(outdir: str) -> None:
    import torch

    import build_ref

    ref = build_ref.load()
    if ref is None:
        raise SystemExit("oracle/_ref is not built; run oracle/build_ref.py where the reference checkout is mounted")
    os.makedirs(outdir, exist_ok=True)
    dev = "cuda"
    for name, (sc, mode) in golden_scenes().items():
        v = torch.from_numpy(sc.vertices).to(dev)
        i = torch.from_numpy(sc.indices).to(dev)
        c = torch.from_numpy(sc.colors).to(dev)
        o = torch.from_numpy(sc.opacities).to(dev)
        ml = mode["max_layers"]
        image, depth, fw, ids, offsets, bary, ends, _ = ref.render_forward(
            v, i, c, o, sc.width, sc.height, sc.tile_width, sc.tile_height, mode["thr"], True, mode["per_pixel_sort"], ml)
        gi, gd = upstream(sc)
        gV, gC, gO = ref.render_backward(torch.from_numpy(gi).to(dev), torch.from_numpy(gd).to(dev), v, i, c, o, ids,
                                         offsets, bary, image, depth, fw, ends, sc.width, sc.height, sc.tile_width,
                                         sc.tile_height, mode["thr"], mode["per_pixel_sort"], ml)
        torch.cuda.synchronize()
        np.savez_compressed(
            os.path.join(outdir, name + ".npz"),
            image=image.cpu().numpy(), depthmap=depth.cpu().numpy(), final_weights=fw.cpu().numpy(),
            ends=ends.cpu().numpy(), offsets=offsets.cpu().numpy(), sorted_ids=ids.cpu().numpy(),
            grad_vertices=gV.cpu().numpy(), grad_colors=gC.cpu().numpy(), grad_opacities=gO.cpu().numpy(),
            per_pixel_sort=np.int32(mode["per_pixel_sort"]), max_layers=np.int32(ml), thr=np.float32(mode["thr"]))
        print(f"[golden] {name}: K={ids.numel()} ends max {int(ends.max())}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
