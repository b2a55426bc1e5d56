from .config import ZikunexConfig, ZikunexLayerConfig  # noqa: F401
from .loader import load_zikunex_weights, read_safetensors, read_safetensors_header  # noqa: F401
from .model import ZikunexModel  # noqa: F401
