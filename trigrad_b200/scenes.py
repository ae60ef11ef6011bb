"""Seeded synthetic scenes (numpy only) for the benchmark configurations and the parity tests.

These stand in for any external mesh or dataset: the reference measures on no public suite, and
none is used here.  Everything is float32 / int32 and reproducible from fixed seeds
(geometry 0, colours 1, opacities 2, loss target 3).

Vertex format is the one ``trigrad.render`` expects (reference ``src/trigrad/wrapper.py:131``):
``(x, y, z, w)`` with x, y in NDC [-1, 1].  The random-triangle scenes use the reference
fixtures' convention ``z = view depth d, w = 1/d`` (reference ``tests/testcases.py:5-9``); the
camera-ring scene uses the viewer's ``(x/w', y/w', z/w', 1/w')`` (reference ``viewer.py:274-280``).

The small fixtures at the end restate the scene *conventions* of the reference's test fixtures
(``tests/testcases.py``) with seeded colours so that they can serve as golden-vector inputs.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

SEED_GEOMETRY, SEED_COLOR, SEED_OPACITY, SEED_TARGET = 0, 1, 2, 3


@dataclass
class Scene:
    """One view ready for ``render``: all arrays are C-contiguous numpy."""

    name: str
    vertices: np.ndarray   # [V,4] float32
    indices: np.ndarray    # [T,3] int32
    colors: np.ndarray     # [V,3] float32
    opacities: np.ndarray  # [V]   float32
    width: int
    height: int
    tile_width: int = 16
    tile_height: int = 16
    meta: dict = field(default_factory=dict)

    @property
    def num_triangles(self) -> int:
        return int(self.indices.shape[0])

    @property
    def num_vertices(self) -> int:
        return int(self.vertices.shape[0])

    def target(self) -> np.ndarray:
        """Seeded U(0,1) loss target ``[H,W,4]`` float32."""
        rng = np.random.default_rng(SEED_TARGET)
        return rng.random((self.height, self.width, 4), dtype=np.float32)


def add_w(xyz: np.ndarray) -> np.ndarray:
    """Append w = 1/z (the reference fixtures' convention, ``tests/testcases.py:5-9``)."""
    xyz = np.asarray(xyz, dtype=np.float32)
    return np.ascontiguousarray(np.concatenate([xyz, (np.float32(1) / xyz[:, 2:3])], axis=1), dtype=np.float32)


# ----------------------------------------------------------------------------------------------
# icosphere


def icosphere(subdivisions: int) -> tuple[np.ndarray, np.ndarray]:
    """Unit icosphere: returns (points [V,3] float64, faces [T,3] int32) with shared vertices.

    V = 10*4^s + 2, T = 20*4^s.
    """
    phi = (1.0 + 5.0 ** 0.5) / 2.0
    pts = np.array(
        [[-1, phi, 0], [1, phi, 0], [-1, -phi, 0], [1, -phi, 0], [0, -1, phi], [0, 1, phi],
         [0, -1, -phi], [0, 1, -phi], [phi, 0, -1], [phi, 0, 1], [-phi, 0, -1], [-phi, 0, 1]],
        dtype=np.float64,
    )
    pts /= np.linalg.norm(pts, axis=1, keepdims=True)
    faces = np.array(
        [[0, 11, 5], [0, 5, 1], [0, 1, 7], [0, 7, 10], [0, 10, 11], [1, 5, 9], [5, 11, 4], [11, 10, 2],
         [10, 7, 6], [7, 1, 8], [3, 9, 4], [3, 4, 2], [3, 2, 6], [3, 6, 8], [3, 8, 9], [4, 9, 5],
         [2, 4, 11], [6, 2, 10], [8, 6, 7], [9, 8, 1]],
        dtype=np.int64,
    )
    for _ in range(subdivisions):
        nv = pts.shape[0]
        e = np.concatenate([faces[:, [0, 1]], faces[:, [1, 2]], faces[:, [2, 0]]], axis=0)
        e.sort(axis=1)
        key = e[:, 0] * nv + e[:, 1]
        uniq, inv = np.unique(key, return_inverse=True)
        mid = pts[uniq // nv] + pts[uniq % nv]
        mid /= np.linalg.norm(mid, axis=1, keepdims=True)
        pts = np.concatenate([pts, mid], axis=0)
        nf = faces.shape[0]
        m01, m12, m20 = nv + inv[:nf], nv + inv[nf:2 * nf], nv + inv[2 * nf:]
        a, b, c = faces[:, 0], faces[:, 1], faces[:, 2]
        faces = np.concatenate(
            [np.stack([a, m01, m20], 1), np.stack([b, m12, m01], 1), np.stack([c, m20, m12], 1),
             np.stack([m01, m12, m20], 1)], axis=0)
    return pts, np.ascontiguousarray(faces.astype(np.int32))


def _vertex_attributes(nv: int, o_lo: float, o_hi: float) -> tuple[np.ndarray, np.ndarray]:
    colors = np.random.default_rng(SEED_COLOR).random((nv, 3), dtype=np.float32)
    op = np.random.default_rng(SEED_OPACITY).random(nv, dtype=np.float32)
    opac = (np.float32(o_lo) + np.float32(o_hi - o_lo) * op).astype(np.float32)
    return np.ascontiguousarray(colors), np.ascontiguousarray(opac)


def config1_icosphere(subdivisions: int = 3, width: int = 256, height: int = 256) -> Scene:
    """Jittered closed icosphere, T = 1280 at 3 subdivisions; depth d = 2 - z."""
    rng = np.random.default_rng(SEED_GEOMETRY)
    pts, faces = icosphere(subdivisions)
    pts = pts + rng.normal(0.0, 0.02, pts.shape)
    pts = pts * (0.8 / np.abs(pts[:, :2]).max())
    xyz = np.stack([pts[:, 0], pts[:, 1], 2.0 - pts[:, 2]], axis=1)
    colors, opac = _vertex_attributes(pts.shape[0], 0.3, 0.9)
    return Scene("cfg1_icosphere", add_w(xyz), faces, colors, opac, width, height)


def random_triangles(T: int, width: int, height: int, edge_mu: float, edge_sigma: float,
                     centroid: str = "uniform", centroid_sigma: float = 0.1, name: str = "random",
                     seed: int = SEED_GEOMETRY) -> Scene:
    """T independent equilateral triangles (V = 3T) in NDC.

    centroid ~ U[-1,1]^2 (or N(0, sigma^2) per axis), edge L ~ LogNormal(ln edge_mu, edge_sigma),
    circumradius L/sqrt(3), rotation ~ U[0, 2pi), per-triangle depth d0 ~ U(0.1, 10) and per-vertex
    depth d0 * (1 + 0.05 U(-1,1)); RGB ~ U(0,1), opacity ~ U(0.1, 0.9).
    """
    rng = np.random.default_rng(seed)
    if centroid == "uniform":
        cen = rng.uniform(-1.0, 1.0, (T, 2))
    else:
        cen = rng.normal(0.0, centroid_sigma, (T, 2))
    L = rng.lognormal(np.log(edge_mu), edge_sigma, T)
    rot = rng.uniform(0.0, 2.0 * np.pi, T)
    d0 = rng.uniform(0.1, 10.0, T)
    dv = d0[:, None] * (1.0 + 0.05 * rng.uniform(-1.0, 1.0, (T, 3)))
    ang = rot[:, None] + np.arange(3)[None, :] * (2.0 * np.pi / 3.0)
    r = (L / np.sqrt(3.0))[:, None]
    x = cen[:, 0:1] + r * np.cos(ang)
    y = cen[:, 1:2] + r * np.sin(ang)
    xyz = np.stack([x.reshape(-1), y.reshape(-1), dv.reshape(-1)], axis=1)
    faces = np.arange(3 * T, dtype=np.int32).reshape(T, 3)
    colors, opac = _vertex_attributes(3 * T, 0.1, 0.9)
    return Scene(name, add_w(xyz), np.ascontiguousarray(faces), colors, opac, width, height)


def config2_random10k() -> Scene:
    return random_triangles(10_000, 512, 512, 0.02, 0.5, name="cfg2_random10k")


def config3_random200k(T: int = 200_000, width: int = 1920, height: int = 1080) -> Scene:
    return random_triangles(T, width, height, 0.005, 0.7, name="cfg3_random200k")


def config5_overlap(T: int = 2_000_000, width: int = 3840, height: int = 2160) -> Scene:
    return random_triangles(T, width, height, 0.01, 0.5, centroid="gauss", centroid_sigma=0.1,
                            name="cfg5_overlap")


# ----------------------------------------------------------------------------------------------
# config 4: displaced sphere seen from a ring of cameras


def _lattice_noise(p: np.ndarray, seed: int, octaves: int = 4) -> np.ndarray:
    """Smooth seeded lattice noise in [-1, 1] (trilinear, smoothstep-faded, `octaves` octaves)."""
    rng = np.random.default_rng(seed)
    n = 32
    out = np.zeros(p.shape[0])
    amp, freq, norm = 1.0, 2.0, 0.0
    for _ in range(octaves):
        lat = rng.uniform(-1.0, 1.0, (n, n, n))
        q = p * freq
        i0 = np.floor(q).astype(np.int64)
        f = q - i0
        f = f * f * (3.0 - 2.0 * f)
        acc = np.zeros(p.shape[0])
        for dx in (0, 1):
            for dy in (0, 1):
                for dz in (0, 1):
                    wgt = (f[:, 0] if dx else 1 - f[:, 0]) * (f[:, 1] if dy else 1 - f[:, 1]) * \
                          (f[:, 2] if dz else 1 - f[:, 2])
                    acc += wgt * lat[(i0[:, 0] + dx) % n, (i0[:, 1] + dy) % n, (i0[:, 2] + dz) % n]
        out += amp * acc
        norm += amp
        amp *= 0.5
        freq *= 2.0
    return out / norm


@dataclass
class WorldMesh:
    """World-space mesh + attributes for the multi-view configuration."""

    points: np.ndarray     # [V,3] float32 world positions
    indices: np.ndarray    # [T,3] int32
    colors: np.ndarray     # [V,3] float32
    opacities: np.ndarray  # [V]   float32


def displaced_sphere(subdivisions: int = 8, amplitude: float = 0.1) -> WorldMesh:
    pts, faces = icosphere(subdivisions)
    r = 1.0 + amplitude * _lattice_noise(pts, SEED_GEOMETRY)
    pts = (pts * r[:, None]).astype(np.float32)
    colors, opac = _vertex_attributes(pts.shape[0], 0.1, 0.9)
    return WorldMesh(np.ascontiguousarray(pts), faces, colors, opac)


def perspective(fov_y_deg: float, near: float, far: float, width: int, height: int) -> np.ndarray:
    """Projection matrix with the layout of the reference viewer (``viewer.py:96-111``)."""
    t = np.tan(np.radians(fov_y_deg) / 2.0) * near
    r = t * width / height
    f, n = far, near
    return np.array([[n / r, 0, 0, 0], [0, n / t, 0, 0],
                     [0, 0, -(f + n) / (f - n), -(2 * f * n) / (f - n)], [0, 0, -1, 0]], dtype=np.float64)


def lookat(eye, target=(0.0, 0.0, 0.0), up=(0.0, 1.0, 0.0)) -> np.ndarray:
    """View matrix as in the reference viewer (``viewer.py:128-144``)."""
    eye = np.asarray(eye, dtype=np.float64)
    fwd = eye - np.asarray(target, dtype=np.float64)
    fwd /= np.linalg.norm(fwd)
    upv = np.asarray(up, dtype=np.float64)
    upv = upv / np.linalg.norm(upv)
    right = np.cross(upv, fwd)
    right /= np.linalg.norm(right)
    up2 = np.cross(fwd, right)
    V = np.eye(4)
    V[0, :3], V[1, :3], V[2, :3] = right, up2, fwd
    V[0, 3], V[1, 3], V[2, 3] = -right @ eye, -up2 @ eye, -fwd @ eye
    return V


def camera_ring(n_views: int = 64, radius: float = 3.0, fov_y_deg: float = 45.0, near: float = 0.1,
                far: float = 100.0, width: int = 1920, height: int = 1080) -> np.ndarray:
    """``[n_views, 4, 4]`` float32 projection*view matrices, cameras on a ring in the xz-plane."""
    P = perspective(fov_y_deg, near, far, width, height)
    out = np.empty((n_views, 4, 4), dtype=np.float32)
    for i in range(n_views):
        a = 2.0 * np.pi * i / n_views
        out[i] = (P @ lookat([radius * np.sin(a), 0.0, radius * np.cos(a)])).astype(np.float32)
    return out


def project_numpy(points: np.ndarray, pv: np.ndarray) -> np.ndarray:
    """World -> render vertex format ``(x/w', y/w', z/w', 1/w')`` (reference ``viewer.py:274-280``)."""
    h = np.concatenate([points.astype(np.float32), np.ones((points.shape[0], 1), np.float32)], axis=1)
    clip = h @ pv.astype(np.float32).T
    out = np.empty_like(clip)
    out[:, :3] = clip[:, :3] / clip[:, 3:4]
    out[:, 3] = np.float32(1) / clip[:, 3]
    return np.ascontiguousarray(out)


def config4_view(mesh: WorldMesh, pv: np.ndarray, width: int = 1920, height: int = 1080, name: str = "cfg4_view") -> Scene:
    return Scene(name, project_numpy(mesh.points, pv), mesh.indices, mesh.colors, mesh.opacities, width, height)


# ----------------------------------------------------------------------------------------------
# small fixtures following the conventions of the reference's tests/testcases.py, seeded


def overlapping_squares(n: int = 10, lo: float = 0.1, hi: float = 0.9, seed: int = 11) -> Scene:
    """n concentric squares (2 triangles each) at depths 1..n, one colour per square.

    Same construction as reference ``tests/testcases.py:12-36`` (x scaled by 1.00001, all by 2).
    """
    rng = np.random.default_rng(seed)
    v, idx, col = [], [], []
    for i, s in enumerate(np.linspace(lo, hi, n, dtype=np.float32)):
        s = float(s) / 2
        f = 1.00001
        v += [[-f * s, -s, i + 1], [f * s, -s, i + 1], [f * s, s, i + 1], [-f * s, s, i + 1]]
        a = 4 * i
        idx += [[a, a + 1, a + 2], [a, a + 2, a + 3]]
        c = rng.random(3).tolist()
        col += [c, c, c, c]
    verts = np.asarray(v, dtype=np.float32) * np.float32(2)
    sc = Scene("overlapping_squares", add_w(verts), np.asarray(idx, dtype=np.int32),
               np.asarray(col, dtype=np.float32), np.full(4 * n, 0.99, np.float32), 50, 50, 4, 4)
    return sc


def large_triangles(n: int = 3, r: float = 4.0, seed: int = 12, opacity: float = 0.99) -> Scene:
    """n screen-covering triangles at depths 1..n (reference ``tests/testcases.py:73-102``)."""
    rng = np.random.default_rng(seed)
    v, idx, col = [], [], []
    for i in range(n):
        ang = rng.uniform(0, 2 * np.pi)
        for k in range(3):
            v.append([np.cos(ang + k * 2 * np.pi / 3) * r + 0.5, np.sin(ang + k * 2 * np.pi / 3) * r + 0.5, i + 1])
            col.append(rng.random(3).tolist())
        idx.append([3 * i, 3 * i + 1, 3 * i + 2])
    return Scene("large_triangles", add_w(np.asarray(v, dtype=np.float32)), np.asarray(idx, dtype=np.int32),
                 np.asarray(col, dtype=np.float32), np.full(3 * n, opacity, np.float32), 50, 50, 4, 4)


def depth_overlap() -> Scene:
    """Two intersecting triangles (reference ``tests/testcases.py:39-70``)."""
    v = np.array([[-1.0, -1, 3], [1, -1, 3], [0, 1, 2], [-1, 1, 3], [1, 1, 3], [0, -1, 2]], dtype=np.float32)
    col = np.array([[1, 0, 0]] * 3 + [[0, 0, 1]] * 3, dtype=np.float32)
    return Scene("depth_overlap", add_w(v), np.array([[0, 1, 2], [3, 4, 5]], np.int32), col,
                 np.ones(6, np.float32), 64, 64, 16, 16)


def full_screen_layers(n: int, opacity: float = 0.1, width: int = 32, height: int = 32, seed: int = 13,
                       tile: int = 16, reverse: bool = False) -> Scene:
    """n constant-depth triangles that each cover the whole screen, depths 1..n (or n..1)."""
    rng = np.random.default_rng(seed)
    v, idx, col = [], [], []
    for i in range(n):
        d = float(n - i if reverse else i + 1)
        v += [[-4.0, -3.0, d], [4.0, -3.0, d], [0.0, 5.0, d]]
        c = rng.random(3).tolist()
        col += [c, c, c]
        idx.append([3 * i, 3 * i + 1, 3 * i + 2])
    return Scene("full_screen_layers", add_w(np.asarray(v, np.float32)), np.asarray(idx, np.int32),
                 np.asarray(col, np.float32), np.full(3 * n, opacity, np.float32), width, height, tile, tile)
