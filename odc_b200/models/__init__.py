from .llama import PRESETS, DecoderConfig, DecoderLayer, DecoderLM, get_config
from .toy import ToyConfig, ToyTransformer
