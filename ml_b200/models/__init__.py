from .decoder import GPT  # noqa: F401
from .vision import VisionTower  # noqa: F401
