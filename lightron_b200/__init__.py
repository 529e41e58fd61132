"""lightron_b200: a Blackwell-native 4-D-parallel LLM training framework."""
from .config import ModelArgs, RunConfig, load_config, parse_config, build_model_args  # noqa: F401

__version__ = "0.1.0"
