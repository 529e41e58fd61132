from .eval import evaluate  # noqa: F401
from .hf import convert_hf_llama_state_dict, export_hf_llama_state_dict, load_hf_llama_weights  # noqa: F401
