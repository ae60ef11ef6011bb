"""Argument validation shared by the Python entry points.

Same behaviour as the reference helper (``src/trigrad/util.py:1-16``): a wrong device or dtype is a
``TypeError``, a wrong shape a ``ValueError``.
"""
from __future__ import annotations


def create_check(default_device: str, default_dtype):
    def check_tensor(tensor, name, shape=None, dtype=None, device=None):
        if shape is not None and not isinstance(shape, tuple):
            shape = (shape,)
        want_device = default_device if device is None else device
        if tensor.device.type != want_device:
            raise TypeError(f"{name} must be on {want_device}, but got {tensor.device.type}")
        want_dtype = default_dtype if dtype is None else dtype
        if tensor.dtype != want_dtype:
            raise TypeError(f"{name} must be of type {want_dtype}, but got {tensor.dtype}")
        if shape is not None and tuple(tensor.shape) != shape:
            raise ValueError(f"{name} must be of shape {shape}, but got {tuple(tensor.shape)}")

    return check_tensor
