from .config import LeroraxConfig, LeroraxLayerConfig  # noqa: F401
from .loader import load_lerorax_weights, load_model_dir  # noqa: F401
from .model import LeroraxModel  # noqa: F401
