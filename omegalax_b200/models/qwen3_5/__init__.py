from . import config, model  # noqa: F401
from .config import Qwen3_5Config, Qwen3_5TextConfig, Qwen3_5VisionConfig  # noqa: F401
from .model import Qwen3_5ForCausalLM, Qwen3_5ForConditionalGeneration  # noqa: F401
