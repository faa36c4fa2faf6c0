from .llama import PRESETS, DecoderConfig, DecoderLayer, DecoderLM, get_config
from .toy import ToyConfig, ToyTransformer
from . import hf  # noqa: F401  (Hugging Face Llama / Qwen2 checkpoint conversion)
