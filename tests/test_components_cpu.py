"""Single-process CPU tests: config schema, data slicing, HF key mapping, evaluation, checkpoint files."""
import copy
import json
import os

import pytest
import torch

from lightron_b200 import mesh
from lightron_b200.config import ModelArgs, PRESETS, build_model_args, parse_config
from lightron_b200.data import MicroBatchDataLoader, cp_slice_indices

RAW = {
    "distributed": {"tp_size": 1, "dp_size": 1, "engine": "afab"},
    "model": {"name": "tiny"},
    "dataset": {"name": "synthetic"},
    "training": {"micro_batch_size": 2, "gradient_accumulation_steps": 1, "seq_length": 64, "learning_rate": 3e-4,
                 "total_steps": 3, "dtype": "fp32", "log_interval": 1},
}


def test_config_schema_env_overrides_and_engine_alias():
    cfg = parse_config(copy.deepcopy(RAW), env={"TP_SIZE": "2", "DP_SIZE": "4"})
    assert cfg.distributed.tp_size == 2 and cfg.distributed.dp_size == 4
    assert cfg.distributed.pp_engine == "afab"            # the sample file's "engine" spelling is honoured
    with pytest.raises(ValueError):
        bad = copy.deepcopy(RAW)
        bad["training"]["no_such_key"] = 1
        parse_config(bad, env={})
    with pytest.raises(ValueError):
        bad = copy.deepcopy(RAW)
        del bad["training"]["total_steps"]
        parse_config(bad, env={})
    with pytest.raises(ValueError):
        parse_config({**copy.deepcopy(RAW), "distributed": {"dp_size": 3, "ep_size": 2}}, env={})


def test_model_args_ffn_rule_and_presets():
    assert ModelArgs(dim=2048, n_heads=32).ffn_hidden == 5632                    # reference rule, multiple_of 256
    assert ModelArgs(dim=4096, n_heads=32, ffn_dim_multiplier=1.3).ffn_hidden == 14336
    assert ModelArgs(dim=256, n_heads=8, multiple_of=16).ffn_hidden == 688
    a = ModelArgs(**PRESETS["llama-1.1b"])
    assert abs(a.num_params() - 1.100e9) < 2e6
    cfg = parse_config({**copy.deepcopy(RAW), "model": {"hidden_size": 128, "num_hidden_layers": 2,
                                                        "num_attention_heads": 4, "vocab_size": 1001}},
                       env={"TP_SIZE": "2"})
    args = build_model_args(cfg)
    assert args.dim == 128 and args.vocab_size == 1002                          # padded to a multiple of tp


def test_hf_style_local_config_dir(tmp_path):
    d = tmp_path / "hfmodel"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
                                               "num_key_value_heads": 2, "vocab_size": 512, "rms_norm_eps": 1e-6,
                                               "intermediate_size": 176, "rope_theta": 500000.0}))
    raw = copy.deepcopy(RAW)
    raw["model"] = {"name": str(d)}
    args = build_model_args(parse_config(raw, env={}))
    assert (args.dim, args.n_kv_heads, args.ffn_hidden, args.rope_theta, args.norm_eps) == (64, 2, 176, 500000.0, 1e-6)


def test_cp_slices_partition_the_sequence():
    for mode in ("contiguous", "zigzag"):
        seen = torch.cat([cp_slice_indices(64, 4, r, mode) for r in range(4)])
        assert sorted(seen.tolist()) == list(range(64))
    z = cp_slice_indices(16, 2, 0, "zigzag").tolist()
    assert z == [0, 1, 2, 3, 12, 13, 14, 15]


def test_dataloader_shapes_targets_and_resume():
    mesh.set_context(None)
    dl = MicroBatchDataLoader(micro_batch_size=4, seq_length=128, grad_acc_steps=2, vocab_size=1000, seed=0)
    assert dl.global_batch_size == 8 and dl.seq_length_per_gpu == 128
    b0 = next(dl)
    assert b0["input_ids"].shape == (4, 128) and b0["input_ids"].dtype == torch.int64
    assert torch.equal(b0["input_ids"][:, 1:], b0["target_ids"][:, :-1])        # labels = inputs shifted by one
    b1 = next(dl)
    dl2 = MicroBatchDataLoader(micro_batch_size=4, seq_length=128, grad_acc_steps=2, vocab_size=1000, seed=0)
    dl2.load_state_dict({"cursor": 1})
    assert torch.equal(next(dl2)["input_ids"], b1["input_ids"])


def test_synthetic_samples_do_not_depend_on_the_batching():
    """Sample i is a function of (seed, i): one micro-batch of 8 holds the rows of 8 micro-batches of 1, and of
    the micro-batches two data-parallel ranks would draw."""
    from lightron_b200.data import SyntheticTokens
    ds = SyntheticTokens(1000, 32, seed=3)
    whole = ds.batch(16, 8)
    singles = torch.cat([ds.batch(16 + i, 1) for i in range(8)])
    halves = torch.cat([ds.batch(16, 4), ds.batch(20, 4)])
    assert torch.equal(whole, singles) and torch.equal(whole, halves)
    assert not torch.equal(whole[0], whole[1])
    assert not torch.equal(SyntheticTokens(1000, 32, seed=4).batch(16, 8), whole)


def test_swiglu_mlp_fallback_matches_the_composed_ops():
    """Off the GPU ``swiglu_mlp`` is the three composed ops (and the oracle formula)."""
    from lightron_b200.ops import functional as OF
    g = torch.Generator().manual_seed(0)
    x = torch.randn(12, 16, generator=g, requires_grad=True)
    w1, w3 = torch.randn(24, 16, generator=g) * 0.1, torch.randn(24, 16, generator=g) * 0.1
    w2 = torch.randn(16, 24, generator=g) * 0.1
    y = OF.swiglu_mlp(x, w1, w3, w2)
    want = (torch.nn.functional.silu(x @ w1.t()) * (x @ w3.t())) @ w2.t()
    assert torch.allclose(y, want, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()


def test_hf_key_mapping_roundtrip_and_rope_layout():
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.utils import convert_hf_llama_state_dict, export_hf_llama_state_dict, load_hf_llama_weights
    mesh.set_context(None)
    a = ModelArgs(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, intermediate_size=96, max_seq_len=16)
    m = LightronTransformer(a)
    init_weights(m, 0)
    hf = export_hf_llama_state_dict(m.state_dict(), 4, 2)
    assert "model.layers.1.self_attn.q_proj.weight" in hf and "lm_head.weight" in hf
    back = convert_hf_llama_state_dict(hf, 4, 2)
    for k, v in m.state_dict().items():
        assert torch.equal(back[k], v), k
    # rotate-half RoPE on the exported q equals interleaved RoPE on ours, up to the same permutation
    m2 = LightronTransformer(a)
    load_hf_llama_weights(m2, hf)
    tok = torch.randint(0, 128, (1, 16))
    assert torch.allclose(m(tok), m2(tok))


def test_evaluate_reports_loss_and_perplexity():
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.utils import evaluate
    mesh.set_context(None)
    a = ModelArgs(dim=64, n_layers=1, n_heads=4, vocab_size=128, intermediate_size=96, max_seq_len=32)
    m = LightronTransformer(a)
    init_weights(m, 0)
    dl = MicroBatchDataLoader(micro_batch_size=2, seq_length=32, vocab_size=128)
    out = evaluate(m, dl, torch.device("cpu"), max_batches=3)
    assert out["batches"] == 3 and abs(out["loss"] - 4.85) < 0.3 and out["perplexity"] > 50


def test_checkpoint_save_resume_and_corruption(tmp_path):
    from lightron_b200.trainer import Trainer
    mesh.set_context(None)
    raw = copy.deepcopy(RAW)
    raw["distributed"] = {}
    raw["training"].update(total_steps=4, save_dir=str(tmp_path), save_interval=2)
    tr = Trainer(parse_config(raw, env={}))
    out = tr.fit()
    assert os.path.exists(out["checkpoint"]) and os.path.exists(tmp_path / "ckpt_step_2_tpsize_1_dpsize_1")
    payload = torch.load(out["checkpoint"], weights_only=False)
    assert set(payload) >= {"model", "optimizer", "trained_steps", "trained_tokens"}
    assert payload["trained_steps"] == 4 and "layers.0.attention.wq.weight" in payload["model"]
    # resume from step 2 and replay steps 3..4: same final weights as the uninterrupted run
    mesh.set_context(None)
    raw2 = copy.deepcopy(raw)
    raw2["training"].update(resume=str(tmp_path / "ckpt_step_2_tpsize_1_dpsize_1"), save_dir=str(tmp_path / "b"))
    os.makedirs(tmp_path / "b")
    tr2 = Trainer(parse_config(raw2, env={}))
    assert tr2.step == 2
    out2 = tr2.fit()
    a, b = payload["model"], torch.load(out2["checkpoint"], weights_only=False)["model"]
    for k in a:
        assert torch.allclose(a[k], b[k], atol=1e-6), k
    # a truncated file is reported, not silently loaded
    path = out["checkpoint"]
    with open(path, "r+b") as f:
        f.truncate(os.path.getsize(path) // 2)
    mesh.set_context(None)
    raw3 = copy.deepcopy(raw)
    raw3["training"].update(resume=path)
    with pytest.raises(RuntimeError, match="unreadable"):
        Trainer(parse_config(raw3, env={}))
    mesh.set_context(None)


def test_profiler_window_writes_a_trace(tmp_path):
    """``training.profile_steps`` runs the chosen steps under torch.profiler and leaves a chrome trace."""
    import json
    from lightron_b200.trainer import Trainer
    mesh.set_context(None)
    raw = copy.deepcopy(RAW)
    raw["distributed"] = {}
    raw["training"].update(total_steps=4, save_final=False, profile_steps=[2, 3], profile_dir=str(tmp_path))
    out = Trainer(parse_config(raw, env={})).fit()
    assert out["steps"] == 4
    trace = tmp_path / "lightron_trace_rank0.json"
    assert trace.exists()
    events = json.loads(trace.read_text())["traceEvents"]
    assert len(events) > 10
    mesh.set_context(None)


def test_two_runs_with_one_seed_end_bitwise_equal():
    """Repeated-run determinism of the whole loop (data order, init, optimizer) on the oracle ops."""
    from lightron_b200.trainer import Trainer
    finals = []
    for _ in range(2):
        mesh.set_context(None)
        raw = copy.deepcopy(RAW)
        raw["distributed"] = {}
        raw["training"].update(total_steps=3, save_final=False)
        tr = Trainer(parse_config(raw, env={}))
        tr.fit()
        finals.append({k: v.clone() for k, v in tr.model.state_dict().items()})
    mesh.set_context(None)
    for k in finals[0]:
        assert torch.equal(finals[0][k], finals[1][k]), k
