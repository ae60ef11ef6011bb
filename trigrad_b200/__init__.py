"""trigrad_b200: B200-native (sm_100a) differentiable triangle rasterisation behind trigrad's ``render`` API."""
from .wrapper import Renderer, precision, render

__all__ = ["render", "Renderer", "precision"]
__version__ = "0.1.0"
