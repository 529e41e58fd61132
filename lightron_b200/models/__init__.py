from .llama import LightronTransformer, TransformerBlock, Attention, MLP, RMSNorm, init_weights, flatten_parameters  # noqa: F401
from .moe import MoEFeedForward  # noqa: F401
