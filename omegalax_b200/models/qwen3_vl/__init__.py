from . import config, model  # noqa: F401
from .config import Qwen3VLConfig, Qwen3VLVisionConfig, make_vl_config, make_vl_config_from_hf  # noqa: F401
from .model import Qwen3VL, get_rope_index  # noqa: F401
