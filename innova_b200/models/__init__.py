from .config import TransformerConfig, PRESETS, gpt2_small, tiny_dense, llama_7b, dense_13b, moe_24l  # noqa: F401
from .dense import DenseModel  # noqa: F401
from .moe import MoEModel  # noqa: F401
