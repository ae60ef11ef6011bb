"""Record golden vectors for the near-plane triangle splitter from the reference's OWN function.

The reference implements ``split_clipped`` in a notebook cell (``notebooks/renderer.ipynb``, cell "Clip Test").  This
script reads that cell from the reference checkout, executes only the definition of ``split_clipped`` (on CPU torch),
runs it on a seeded mesh whose triangles fall into every case (kept, dropped, one or two vertices behind the plane)
and stores inputs, outputs and - through torch autograd with seeded upstream gradients - the gradients with respect
to clip vertices, colours and opacities in ``tests/golden/clip_near_plane.npz``.

    python tests/golden/make_clip_golden.py [/path/to/reference]
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_split_clipped(reference_root):
    nb = json.load(open(os.path.join(reference_root, "notebooks", "renderer.ipynb")))
    for cell in nb["cells"]:
        src = "".join(cell["source"])
        if "def split_clipped" in src:
            start = src.index("def split_clipped")
            end = src.index("proj = getProjectionMatrix")
            ns = {"torch": torch, "np": np}
            exec(src[start:end], ns)
            return ns["split_clipped"]
    raise SystemExit("split_clipped not found in the notebook")


def seeded_inputs():
    rng = np.random.default_rng(31)
    V, T = 40, 64
    clip = np.empty((V, 4), np.float32)
    clip[:, :2] = rng.uniform(-2, 2, (V, 2))
    clip[:, 3] = rng.uniform(0.2, 3.0, V)
    clip[:, 2] = rng.uniform(-2.5, 2.0, V) * clip[:, 3]          # z + w changes sign for about a third of the vertices
    idx = rng.integers(0, V, (T, 3)).astype(np.int32)
    idx = idx[(idx[:, 0] != idx[:, 1]) & (idx[:, 1] != idx[:, 2]) & (idx[:, 0] != idx[:, 2])]
    colors = rng.random((V, 3), dtype=np.float32)
    opac = rng.uniform(0.1, 0.9, (V, 1)).astype(np.float32)
    return clip, idx, colors, opac


def main(reference_root=os.environ.get("TRIGRAD_REFERENCE", os.path.join(os.sep, "root", "reference"))):
    split = reference_split_clipped(reference_root)
    clip, idx, colors, opac = seeded_inputs()
    tc = torch.tensor(clip, requires_grad=True)
    tcol = torch.tensor(colors, requires_grad=True)
    top = torch.tensor(opac, requires_grad=True)
    v, i, c, o = split(tc, torch.tensor(idx), tcol, top)
    rng = np.random.default_rng(32)
    gv = rng.normal(size=tuple(v.shape)).astype(np.float32)
    gc = rng.normal(size=tuple(c.shape)).astype(np.float32)
    go = rng.normal(size=tuple(o.shape)).astype(np.float32)
    ((v * torch.tensor(gv)).sum() + (c * torch.tensor(gc)).sum() + (o * torch.tensor(go)).sum()).backward()
    np.savez_compressed(os.path.join(HERE, "clip_near_plane.npz"), clip=clip, indices=idx, colors=colors, opacities=opac,
                        out_vertices=v.detach().numpy(), out_indices=i.numpy(), out_colors=c.detach().numpy(),
                        out_opacities=o.detach().numpy(), up_vertices=gv, up_colors=gc, up_opacities=go,
                        grad_clip=tc.grad.numpy(), grad_colors=tcol.grad.numpy(), grad_opacities=top.grad.numpy())
    print(f"[golden] clip_near_plane: {idx.shape[0]} triangles in, {v.shape[0] // 3} out")


if __name__ == "__main__":
    main(*sys.argv[1:2])
