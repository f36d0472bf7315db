from .config import PRESETS, ModelConfig, get_config  # noqa: F401
from .decoder import Block, DecoderLM, build_model  # noqa: F401
