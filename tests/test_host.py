"""Host-side logic that needs no GPU: argument checks, scene generators, view sharding, the 2-rank exchange."""
import os
import sys

import numpy as np
import pytest
import torch

import trigrad_b200
from trigrad_b200 import scenes as S
from trigrad_b200 import views
from trigrad_b200.util import create_check


def _scene_tensors(sc):
    return (torch.from_numpy(sc.vertices), torch.from_numpy(sc.indices), torch.from_numpy(sc.colors),
            torch.from_numpy(sc.opacities))


def test_render_rejects_cpu_tensors_like_the_reference():
    v, i, c, o = _scene_tensors(S.large_triangles(2))
    with pytest.raises(TypeError, match="must be on cuda"):
        trigrad_b200.render(v, i, c, o, 32, 32)


def test_render_rejects_oversized_tiles():
    v, i, c, o = _scene_tensors(S.large_triangles(2))
    with pytest.raises(ValueError, match="<= 1024"):
        trigrad_b200.render(v, i, c, o, 64, 64, 64, 32)


def test_check_tensor_semantics():
    check = create_check("cpu", torch.float32)
    t = torch.zeros(5, 4)
    check(t, "t", (5, 4))
    check(torch.zeros(3), "t", 3)
    with pytest.raises(ValueError):
        check(t, "t", (5, 3))
    with pytest.raises(TypeError):
        check(t.double(), "t", (5, 4))
    with pytest.raises(TypeError):
        check(torch.zeros(5, 3, dtype=torch.int64), "idx", (5, 3), torch.int32)
    with pytest.raises(TypeError):
        create_check("cuda", torch.float32)(t, "t", (5, 4))


def test_scene_generators_are_seeded_and_sized():
    a, b = S.config1_icosphere(), S.config1_icosphere()
    assert a.num_triangles == 1280 and a.num_vertices == 642
    assert np.array_equal(a.vertices, b.vertices) and np.array_equal(a.colors, b.colors)
    assert abs(np.abs(a.vertices[:, :2]).max() - 0.8) < 1e-6
    assert np.allclose(a.vertices[:, 3], 1 / a.vertices[:, 2])
    c2 = S.config2_random10k()
    assert c2.num_triangles == 10_000 and c2.num_vertices == 30_000 and (c2.width, c2.height) == (512, 512)
    assert c2.opacities.min() >= 0.1 and c2.opacities.max() <= 0.9
    pts, faces = S.icosphere(4)
    assert pts.shape[0] == 10 * 4 ** 4 + 2 and faces.shape[0] == 20 * 4 ** 4
    # closed mesh: every edge is shared by exactly two faces
    e = np.sort(np.concatenate([faces[:, [0, 1]], faces[:, [1, 2]], faces[:, [2, 0]]]), axis=1)
    _, counts = np.unique(e, axis=0, return_counts=True)
    assert np.all(counts == 2)


def test_camera_ring_projection_keeps_the_sphere_in_view():
    mesh = S.displaced_sphere(3)
    pvs = S.camera_ring(8, width=192, height=108)
    for k in (0, 3):
        v = S.project_numpy(mesh.points, pvs[k])
        assert np.all(np.abs(v[:, :2]) < 1.0) and np.all(v[:, 3] > 0)
    p = torch.from_numpy(mesh.points)
    assert np.allclose(views.project(p, torch.from_numpy(pvs[1])).numpy(), S.project_numpy(mesh.points, pvs[1]),
                       rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("n,world", [(64, 1), (64, 2), (64, 8), (10, 4), (3, 8)])
def test_shard_views_partitions_the_batch(n, world):
    seen = []
    for r in range(world):
        blk = views.shard_views(n, r, world)
        seen += list(blk)
        assert len(blk) in (n // world, n // world + 1)
    assert seen == list(range(n))


def _fake_render(vertices, indices, colors, opacities, width, height, **kw):
    """CPU stand-in with the render() signature: a smooth function of all differentiable inputs."""
    tri = vertices[indices.long()]                               # [T,3,4]
    s = (tri[..., :2].sum() + tri[..., 3].sum()) * 1e-3
    img = (colors.mean(0) * opacities.mean()).repeat(height, width, 1)
    img = torch.cat([img, torch.ones(height, width, 1)], dim=2) + s
    return img, torch.zeros(height, width)


def _worker(rank, world, port, tmpdir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mesh = S.displaced_sphere(2)
    pvs = torch.from_numpy(S.camera_ring(6, width=16, height=8))
    targets = torch.rand(6, 8, 16, 4, generator=torch.Generator().manual_seed(3))
    p, i = torch.from_numpy(mesh.points), torch.from_numpy(mesh.indices)
    c, o = torch.from_numpy(mesh.colors), torch.from_numpy(mesh.opacities)
    g = views.GradBuffer.allocate(p.shape[0], "cpu")
    ids = views.shard_views(6, rank, world)
    loss = views.render_views_l2(p, i, c, o, pvs, targets, ids, 16, 8, g, render_fn=_fake_render)
    views.allreduce_gradients(g, loss)
    torch.save((g.flat.clone(), loss.clone()), os.path.join(tmpdir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_two_rank_view_sharding_and_allreduce_matches_single_rank(tmp_path):
    """world_size 2 over gloo on CPU: summed gradients equal the single-process result over all views."""
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    g0, l0 = torch.load(tmp_path / "r0.pt")
    g1, l1 = torch.load(tmp_path / "r1.pt")
    assert torch.equal(g0, g1) and torch.equal(l0, l1)
    mesh = S.displaced_sphere(2)
    pvs = torch.from_numpy(S.camera_ring(6, width=16, height=8))
    targets = torch.rand(6, 8, 16, 4, generator=torch.Generator().manual_seed(3))
    g = views.GradBuffer.allocate(mesh.points.shape[0], "cpu")
    loss = views.render_views_l2(torch.from_numpy(mesh.points), torch.from_numpy(mesh.indices),
                                 torch.from_numpy(mesh.colors), torch.from_numpy(mesh.opacities), pvs, targets,
                                 range(6), 16, 8, g, render_fn=_fake_render)
    assert torch.allclose(g.flat, g0, rtol=1e-5, atol=1e-8)
    assert torch.allclose(loss, l0, rtol=1e-6)
    assert g.points.data_ptr() == g.flat.data_ptr()      # one buffer, typed views


def test_obj_loader_reads_triangles_quads_and_relative_indices():
    from trigrad_b200 import loads_obj
    text = """# a unit square as one quad, then a triangle addressed with negative and slashed indices
mtllib ignored.mtl
v 0 0 0
v 1 0 0
v 1 1 0 1.0
v 0 1 0
vn 0 0 1
vt 0.5 0.5
f 1/1/1 2/1/1 3//1 4
v 0.5 0.5 1
g tip
f -1 1 2/7
"""
    pts, faces = loads_obj(text)
    assert pts.dtype == np.float32 and pts.shape == (5, 3)
    assert faces.dtype == np.int32
    assert faces.tolist() == [[0, 1, 2], [0, 2, 3], [4, 0, 1]]
    assert pts[2].tolist() == [1.0, 1.0, 0.0] and pts[4].tolist() == [0.5, 0.5, 1.0]


def test_obj_loader_rejects_bad_records(tmp_path):
    from trigrad_b200 import load_obj, loads_obj
    with pytest.raises(ValueError):
        loads_obj("v 0 0 0\nf 1 2 3\n")            # indices beyond the vertices read so far
    with pytest.raises(ValueError):
        loads_obj("v 0 0\n")
    p = tmp_path / "tri.obj"
    p.write_text("v 0 0 0\nv 1 0 0\nv 0 1 0\nf 1 2 3\n")
    pts, faces = load_obj(str(p))
    assert pts.shape == (3, 3) and faces.tolist() == [[0, 1, 2]]
