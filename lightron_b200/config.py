"""Configuration: the ``ModelArgs`` dataclass and the four-section JSON run config.

Parity with the reference: ``config/config.py:6-27`` (``ModelArgs`` fields and defaults),
``trainer.py:79-90`` (JSON sections ``distributed / model / dataset / training`` and the
``TP_SIZE/DP_SIZE/CP_SIZE/PP_SIZE/EP_SIZE`` environment overrides), ``trainer.py:149-164``
(HF config -> ``ModelArgs`` mapping) and ``model/model.py:53-57`` (SwiGLU hidden size rule).

Extensions that the reference lacks (it needs the HF hub for every run): inline model
dimensions, explicit ``intermediate_size`` and ``rope_theta``, ``dataset.name = "synthetic"``,
``distributed.{cp_mode, sequence_parallel, fsdp, fused_comm}``, ``training.{dtype, save_interval,
resume, master_weights}``.  Both ``pp_engine`` and the sample file's ``engine`` spelling are read.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, Optional


@dataclass
class ModelArgs:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = None
    moe_num_experts: int = 0
    moe_topk: int = 0
    moe_layer_freq: int = 2
    vocab_size: int = 32000
    multiple_of: int = 256
    ffn_dim_multiplier: Optional[float] = None
    norm_eps: float = 1e-5
    max_seq_len: int = 2048
    tp_size: int = 1
    cp_size: int = 1
    device_mesh_shape: tuple = (1, 1)
    # --- extensions (absent from the reference) ---
    intermediate_size: Optional[int] = None   # overrides the multiple_of rule when set
    rope_theta: float = 10000.0
    moe_aux_loss_coef: float = 0.01
    moe_capacity_factor: float = 2.0          # rows an expert-parallel rank can receive = factor x its own copies
    ep_size: int = 1
    sequence_parallel: bool = False
    cp_mode: str = "ring"                     # "ring" | "allgather" (both zig-zag causal) | "ulysses"

    def __post_init__(self):
        if self.n_kv_heads is None:
            self.n_kv_heads = self.n_heads
        if self.dim % self.n_heads:
            raise ValueError(f"dim {self.dim} not divisible by n_heads {self.n_heads}")
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if self.cp_mode not in ("ring", "ulysses", "allgather"):
            raise ValueError(f"cp_mode must be ring|ulysses|allgather, got {self.cp_mode}")

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def ffn_hidden(self) -> int:
        """SwiGLU hidden size (reference rule: model/model.py:53-57)."""
        if self.intermediate_size is not None:
            return int(self.intermediate_size)
        hidden = int(2 * (4 * self.dim) / 3)
        if self.ffn_dim_multiplier is not None:
            hidden = int(self.ffn_dim_multiplier * hidden)
        m = self.multiple_of
        return m * ((hidden + m - 1) // m)

    def is_moe_layer(self, layer_id: int) -> bool:
        """Reference rule (model/model.py:219): MoE on layers with id % freq == 1.  freq <= 1 (which
        the reference's rule can never satisfy) means every layer is MoE (Mixtral style)."""
        if self.moe_num_experts <= 1:
            return False
        return self.moe_layer_freq <= 1 or layer_id % self.moe_layer_freq == 1

    def num_active_params(self) -> int:
        """Parameters a token actually visits (top-k experts only): the N of the 6*N*tokens rule."""
        mlp = 3 * self.dim * self.ffn_hidden
        n_moe = sum(1 for i in range(self.n_layers) if self.is_moe_layer(i))
        return self.num_params() - n_moe * max(self.moe_num_experts - max(self.moe_topk, 1), 0) * mlp

    def num_params(self) -> int:
        d, kv = self.dim, self.n_kv_heads * self.head_dim
        attn = 2 * d * d + 2 * d * kv
        mlp = 3 * d * self.ffn_hidden
        total = 2 * self.vocab_size * d + d
        for i in range(self.n_layers):
            total += attn + 2 * d
            if self.is_moe_layer(i):
                total += self.moe_num_experts * mlp + d * self.moe_num_experts
            else:
                total += mlp
        return total


# Named shapes usable as ``model.name`` without the HF hub.
PRESETS: Dict[str, Dict[str, Any]] = {
    "tiny": dict(dim=256, n_layers=4, n_heads=8, n_kv_heads=8, vocab_size=8192,
                 intermediate_size=688, norm_eps=1e-5, rope_theta=10000.0),
    "llama-1.1b": dict(dim=2048, n_layers=22, n_heads=32, n_kv_heads=4, vocab_size=32000,
                       intermediate_size=5632, norm_eps=1e-5, rope_theta=10000.0),
    # the 1.1B shape with as many KV heads as query heads: the nearest shape that the reference's
    # stock attention (no GQA) can run; used for like-for-like comparisons only
    "llama-1.1b-mha": dict(dim=2048, n_layers=22, n_heads=32, n_kv_heads=32, vocab_size=32000,
                           intermediate_size=5632, norm_eps=1e-5, rope_theta=10000.0),
    "llama-8b": dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256,
                     intermediate_size=14336, norm_eps=1e-5, rope_theta=500000.0),
    "moe-8x": dict(dim=4096, n_layers=16, n_heads=32, n_kv_heads=8, vocab_size=32000,
                   intermediate_size=14336, norm_eps=1e-5, rope_theta=10000.0,
                   moe_num_experts=8, moe_topk=2, moe_layer_freq=1),
}

_HF_KEYS = {
    "hidden_size": "dim", "num_hidden_layers": "n_layers", "num_attention_heads": "n_heads",
    "num_key_value_heads": "n_kv_heads", "rms_norm_eps": "norm_eps", "vocab_size": "vocab_size",
    "intermediate_size": "intermediate_size", "rope_theta": "rope_theta",
}


@dataclass
class DistributedConfig:
    tp_size: int = 1
    dp_size: int = 1
    cp_size: int = 1
    pp_size: int = 1
    ep_size: int = 1
    pp_engine: str = "1f1b"
    cp_mode: str = "ring"
    sequence_parallel: bool = False
    fsdp: bool = False           # True: parameters, gradients and optimizer state sharded per block over dp
                                 # (parallel.fsdp engine); False: replicated bf16 parameters + sharded optimizer (ZeRO-1)
    fused_comm: bool = True      # use the peer-memory fused kernels when on CUDA

    @property
    def world_size(self) -> int:
        return self.tp_size * self.dp_size * self.cp_size * self.pp_size


@dataclass
class TrainingConfig:
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    seq_length: int = 2048
    learning_rate: float = 3e-4
    total_steps: int = 10
    weight_decay: float = 0.01
    log_interval: int = 10
    max_samples: Optional[int] = None
    seed: int = 42
    dtype: str = "bf16"          # "bf16" (fp32 master weights) | "fp32"
    save_interval: int = 0       # 0 = only at the end (reference behaviour, trainer.py:330-338)
    save_dir: str = "."
    save_final: bool = True      # the reference always writes a checkpoint after the last step
    resume: Optional[str] = None
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    grad_clip: float = 0.0
    jsonl_log: Optional[str] = None
    heartbeat_timeout_s: float = 600.0   # a rank without a heartbeat for this long is reported (0 disables)
    profile_steps: Optional[tuple] = None   # (first, last): torch.profiler trace of these steps on the log rank
    profile_dir: str = "."               # where the chrome trace (lightron_trace_rank<r>.json) goes


@dataclass
class DatasetConfig:
    name: str = "synthetic"
    split: str = "train"
    num_workers: int = 0
    tokenizer: Optional[str] = None


@dataclass
class RunConfig:
    distributed: DistributedConfig = field(default_factory=DistributedConfig)
    model: Dict[str, Any] = field(default_factory=dict)
    dataset: DatasetConfig = field(default_factory=DatasetConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)

    def to_dict(self) -> Dict[str, Any]:
        return {"distributed": asdict(self.distributed), "model": dict(self.model),
                "dataset": asdict(self.dataset), "training": asdict(self.training)}


def _take(cls, d: Dict[str, Any], section: str):
    known = {f for f in cls.__dataclass_fields__}
    extra = set(d) - known
    if extra:
        raise ValueError(f"unknown key(s) {sorted(extra)} in config section '{section}'")
    return cls(**d)


def parse_config(raw: Dict[str, Any], env: Optional[Dict[str, str]] = None) -> RunConfig:
    """Validate a raw JSON dict.  Unknown keys raise (the reference silently ignores them)."""
    env = os.environ if env is None else env
    for sec in ("distributed", "model", "training"):
        if sec not in raw:
            raise ValueError(f"config is missing section '{sec}'")
    dist_raw = dict(raw["distributed"])
    if "engine" in dist_raw:                       # sample file spelling (config_tinystories.json:8)
        dist_raw.setdefault("pp_engine", dist_raw.pop("engine"))
        dist_raw.pop("engine", None)
    for key in ("tp_size", "dp_size", "cp_size", "pp_size", "ep_size"):
        if key.upper() in env:
            dist_raw[key] = int(env[key.upper()])
    dcfg = _take(DistributedConfig, dist_raw, "distributed")
    dcfg.pp_engine = dcfg.pp_engine.lower()
    if dcfg.pp_engine not in ("afab", "1f1b"):
        raise ValueError(f"Invalid pp_engine: {dcfg.pp_engine}")
    if dcfg.dp_size % dcfg.ep_size:
        raise ValueError(f"DP size ({dcfg.dp_size}) must be divisible by EP size ({dcfg.ep_size})")
    tr = dict(raw["training"])
    for req in ("micro_batch_size", "gradient_accumulation_steps", "seq_length", "learning_rate", "total_steps"):
        if req not in tr:
            raise ValueError(f"training.{req} is required")
    if "betas" in tr:
        tr["betas"] = tuple(tr["betas"])
    tcfg = _take(TrainingConfig, tr, "training")
    if tcfg.dtype not in ("bf16", "fp32"):
        raise ValueError("training.dtype must be bf16|fp32")
    if tcfg.seq_length % dcfg.cp_size:
        raise ValueError("seq_length must be divisible by cp_size")
    dscfg = _take(DatasetConfig, dict(raw.get("dataset", {})), "dataset")
    return RunConfig(distributed=dcfg, model=dict(raw["model"]), dataset=dscfg, training=tcfg)


def load_config(path: str) -> RunConfig:
    with open(path, "r") as f:
        return parse_config(json.load(f))


def _hf_config_dict(name: str) -> Optional[Dict[str, Any]]:
    """Resolve ``model.name``: a preset, a local dir / config.json, or (online) the HF hub."""
    if name in PRESETS:
        return None
    path = name
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f)
    try:  # last resort, like trainer.py:135 of the reference (needs a cache or network)
        from transformers import AutoConfig
        return AutoConfig.from_pretrained(name).to_dict()
    except Exception as e:  # pragma: no cover - offline box
        raise ValueError(f"cannot resolve model.name={name!r}: not a preset {sorted(PRESETS)}, "
                         f"not a local config, and the HF hub is unreachable ({type(e).__name__})")


def build_model_args(cfg: RunConfig) -> ModelArgs:
    """Model section -> ModelArgs.  Precedence: inline dims > HF config / preset."""
    m = dict(cfg.model)
    name = m.pop("name", None)
    kw: Dict[str, Any] = {}
    if name is not None:
        if name in PRESETS:
            kw.update(PRESETS[name])
        else:
            hf = _hf_config_dict(name)
            for hk, ak in _HF_KEYS.items():
                if hf.get(hk) is not None:
                    kw[ak] = hf[hk]
            if "n_embd" in hf:        # gpt2-style configs, as in the reference sample run
                kw.update(dim=hf["n_embd"], n_layers=hf["n_layer"], n_heads=hf["n_head"])
                kw.pop("intermediate_size", None)
    for hk, ak in _HF_KEYS.items():
        if hk in m:
            kw[ak] = m.pop(hk)
    valid = set(ModelArgs.__dataclass_fields__)
    for k in list(m):
        if k not in valid:
            raise ValueError(f"unknown key '{k}' in config section 'model'")
        kw[k] = m.pop(k)
    kw.setdefault("moe_num_experts", 1)
    kw.setdefault("moe_topk", 2)
    d = cfg.distributed
    vocab = kw.get("vocab_size", 32000)
    if d.tp_size > 1 and vocab % d.tp_size:        # trainer.py:137-145
        vocab = (vocab // d.tp_size + 1) * d.tp_size
    kw["vocab_size"] = vocab
    kw.update(max_seq_len=cfg.training.seq_length, tp_size=d.tp_size, cp_size=d.cp_size,
              ep_size=d.ep_size, sequence_parallel=d.sequence_parallel, cp_mode=d.cp_mode)
    return ModelArgs(**kw)
