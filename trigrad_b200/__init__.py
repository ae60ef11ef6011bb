"""trigrad_b200: B200-native (sm_100a) differentiable triangle rasterisation behind trigrad's ``render`` API."""
from .clip import project_clip
from .corrected import render_corrected
from .obj import load_obj, loads_obj
from .packed import pack_mesh, render_packed
from .wrapper import Renderer, check_device_errors, precision, render

__all__ = ["render", "Renderer", "precision", "check_device_errors", "render_corrected", "project_clip",
           "render_packed", "pack_mesh", "load_obj", "loads_obj"]
__version__ = "0.1.0"
