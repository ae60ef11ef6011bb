"""trigrad_b200: B200-native (sm_100a) differentiable triangle rasterisation behind trigrad's ``render`` API."""
from .clip import project_clip
from .corrected import render_corrected
from .wrapper import Renderer, check_device_errors, precision, render

__all__ = ["render", "Renderer", "precision", "check_device_errors", "render_corrected", "project_clip"]
__version__ = "0.1.0"
