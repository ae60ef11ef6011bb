"""Wavefront OBJ reader for smoke scenes (the reference ships ``monkey.obj`` for its viewer, ``viewer.py``).

Only what a triangle renderer needs: ``v`` records (x y z, an optional w is ignored) and ``f`` records with any of
the index forms ``i``, ``i/t``, ``i//n``, ``i/t/n``, positive (1-based) or negative (relative to the vertices read so
far); polygons are triangulated as fans.  Everything else (normals, texture coordinates, groups, materials, smoothing
groups, comments) is skipped.
"""
from __future__ import annotations

import io
from typing import Tuple

import numpy as np


def load_obj(source) -> Tuple[np.ndarray, np.ndarray]:
    """``source``: a path, or a file-like object with text lines.  Returns ``(points [V,3] float32, faces [T,3] int32)``."""
    own = isinstance(source, (str, bytes)) or hasattr(source, "__fspath__")
    f = open(source, "r") if own else source
    try:
        pts, faces = [], []
        for lineno, line in enumerate(f, 1):
            parts = line.split("#", 1)[0].split()
            if not parts:
                continue
            if parts[0] == "v":
                if len(parts) < 4:
                    raise ValueError(f"line {lineno}: a vertex needs three coordinates")
                pts.append((float(parts[1]), float(parts[2]), float(parts[3])))
            elif parts[0] == "f":
                if len(parts) < 4:
                    raise ValueError(f"line {lineno}: a face needs at least three vertices")
                ids = []
                for tok in parts[1:]:
                    i = int(tok.split("/", 1)[0])
                    i = i - 1 if i > 0 else len(pts) + i
                    if not (0 <= i < len(pts)):
                        raise ValueError(f"line {lineno}: vertex index {tok} out of range")
                    ids.append(i)
                for k in range(1, len(ids) - 1):
                    faces.append((ids[0], ids[k], ids[k + 1]))
    finally:
        if own:
            f.close()
    return (np.asarray(pts, dtype=np.float32).reshape(-1, 3), np.asarray(faces, dtype=np.int32).reshape(-1, 3))


def loads_obj(text: str) -> Tuple[np.ndarray, np.ndarray]:
    """``load_obj`` on a string."""
    return load_obj(io.StringIO(text))
