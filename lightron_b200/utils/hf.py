"""Hugging Face Llama <-> lightron_b200 weight mapping.

Parity with the reference's ``utils/hf_utils.py:7-64`` (key-by-key copy of an HF Llama
state_dict into the model: ``model.embed_tokens`` -> ``tok_embeddings``, ``self_attn.{q,k,v,o}_proj``
-> ``attention.{wq,wk,wv,wo}``, ``mlp.{gate,up,down}_proj`` -> ``feed_forward.{w1,w3,w2}``,
``input_layernorm`` / ``post_attention_layernorm`` -> ``attention_norm`` / ``ffn_norm``, ``model.norm``,
``lm_head`` -> ``output``).  The reference copies whole tensors and therefore only works unsharded
and without GQA; here the full tensors go through ``checkpoint.load_full_state_dict`` which slices
TP shards and skips layers of other pipeline stages.  HF stores q/k in the "rotate-half" RoPE
layout; this model uses interleaved pairs (the reference's convention), so q/k rows are permuted.
"""
from __future__ import annotations

from typing import Dict

import torch

_LAYER_MAP = {
    "self_attn.q_proj.weight": "attention.wq.weight", "self_attn.k_proj.weight": "attention.wk.weight",
    "self_attn.v_proj.weight": "attention.wv.weight", "self_attn.o_proj.weight": "attention.wo.weight",
    "mlp.gate_proj.weight": "feed_forward.w1.weight", "mlp.up_proj.weight": "feed_forward.w3.weight",
    "mlp.down_proj.weight": "feed_forward.w2.weight", "input_layernorm.weight": "attention_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
}
_TOP_MAP = {"model.embed_tokens.weight": "tok_embeddings.weight", "model.norm.weight": "norm.weight",
            "lm_head.weight": "output.weight"}


def _to_interleaved(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """[h*d, in] rows from rotate-half order (first half | second half) to (x0, x1) pairs."""
    hd = w.shape[0] // n_heads
    return w.view(n_heads, 2, hd // 2, -1).transpose(1, 2).reshape(w.shape)


def _from_interleaved(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    hd = w.shape[0] // n_heads
    return w.view(n_heads, hd // 2, 2, -1).transpose(1, 2).reshape(w.shape)


def convert_hf_llama_state_dict(hf_sd: Dict[str, torch.Tensor], n_heads: int, n_kv_heads: int,
                                permute_rope: bool = True) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for k, v in hf_sd.items():
        if k in _TOP_MAP:
            out[_TOP_MAP[k]] = v
        elif k.startswith("model.layers."):
            _, _, idx, rest = k.split(".", 3)
            if rest in _LAYER_MAP:
                t = v
                if permute_rope and rest == "self_attn.q_proj.weight":
                    t = _to_interleaved(v, n_heads)
                elif permute_rope and rest == "self_attn.k_proj.weight":
                    t = _to_interleaved(v, n_kv_heads)
                out[f"layers.{idx}.{_LAYER_MAP[rest]}"] = t
    if "output.weight" not in out and "tok_embeddings.weight" in out:       # tied embeddings
        out["output.weight"] = out["tok_embeddings.weight"]
    return out


def export_hf_llama_state_dict(sd: Dict[str, torch.Tensor], n_heads: int, n_kv_heads: int,
                               permute_rope: bool = True) -> Dict[str, torch.Tensor]:
    inv_top = {v: k for k, v in _TOP_MAP.items()}
    inv_layer = {v: k for k, v in _LAYER_MAP.items()}
    out: Dict[str, torch.Tensor] = {}
    for k, v in sd.items():
        if k in inv_top:
            out[inv_top[k]] = v
        elif k.startswith("layers."):
            _, idx, rest = k.split(".", 2)
            if rest in inv_layer:
                t = v
                if permute_rope and rest == "attention.wq.weight":
                    t = _from_interleaved(v, n_heads)
                elif permute_rope and rest == "attention.wk.weight":
                    t = _from_interleaved(v, n_kv_heads)
                out[f"model.layers.{idx}.{inv_layer[rest]}"] = t
    return out


def load_hf_llama_weights(model, hf_model_or_state_dict, permute_rope: bool = True):
    """Copy HF Llama weights into ``model`` (any TP / PP layout).  Accepts an HF model or its
    state_dict.  Returns the model."""
    from ..checkpoint import load_full_state_dict
    sd = hf_model_or_state_dict.state_dict() if hasattr(hf_model_or_state_dict, "state_dict") else hf_model_or_state_dict
    args = getattr(model, "args", None) or model.stage.args
    full = convert_hf_llama_state_dict(sd, args.n_heads, args.n_kv_heads, permute_rope)
    load_full_state_dict(model, full, strict=True)
    return model
