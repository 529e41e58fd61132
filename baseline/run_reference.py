"""Reference arm of bench.py.

Runs the UNMODIFIED reference, installed with pip under ``baseline/_ref`` (top-level packages
``config``, ``model``, ``layers``, ``parallel``), through its own public modules, following the
sequence of its ``trainer.py:74-345``: ``setup_distributed`` -> ``ModelArgs`` -> meta-device
``LightronTransformer`` -> ``apply_fsdp2`` when dp > 1 -> ``to_empty`` + N(0, 0.02) init -> RoPE
table recompute -> ``model.to(bfloat16)`` -> ``torch.optim.AdamW`` -> its ``train_step_single``
(``F.cross_entropy`` on gathered logits, ``loss.item()`` per micro-batch).  Only the pieces that
need the network are replaced: the HF ``AutoConfig`` lookup by explicit dimensions and the HF
dataset by synthetic uniform-random tokens of the same shape.  None of lightron_b200's models,
kernels or engine is imported here.

If the stock code cannot run the named config (for instance its GQA view bug,
``model/model.py:166-167``, raises for n_kv_heads < n_heads) the arm prints
``{"impl": "reference", "unavailable": "..."}`` and exits 0.
"""
from __future__ import annotations

import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

SHAPES = {
    "llama-1.1b": dict(dim=2048, n_layers=22, n_heads=32, n_kv_heads=4, vocab_size=32000),
    "llama-1.1b-mha": dict(dim=2048, n_layers=22, n_heads=32, n_kv_heads=32, vocab_size=32000),
    "tiny": dict(dim=256, n_layers=4, n_heads=8, n_kv_heads=8, vocab_size=8192, multiple_of=16),
}


def _unavailable(why: str, rank: int = 0):
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


LIKE_FOR_LIKE = {"llama-1.1b": "llama-1.1b-mha"}     # nearest shape the stock attention can run (no GQA)


def _describe(e: Exception, model: str) -> str:
    tb = traceback.extract_tb(e.__traceback__)
    where = next((f"{os.path.relpath(f.filename, REF)}:{f.lineno}" for f in reversed(tb) if f.filename.startswith(REF)), "")
    return f"unmodified reference raised {type(e).__name__} at {where} on {model}: {e}".replace("\n", " ")[:400]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if not os.path.isdir(os.path.join(REF, "model")):
        return _unavailable("reference not installed under baseline/_ref", rank)
    if args.model not in SHAPES:
        return _unavailable(f"no reference shape for model {args.model}", rank)
    # the reference's packages are top-level names: they must win over anything in the repo root
    sys.path[:] = [REF] + [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(HERE)]
    for name in ("config", "tests", "data", "model", "parallel", "layers", "utils"):
        sys.modules.pop(name, None)
    try:
        line = None
        try:
            line = _run(args, args.model)
        except Exception as e:  # stock code path raised: report, do not patch
            line = {"impl": "reference", "unavailable": _describe(e, args.model)}
        # the same steps on the nearest shape the stock code runs, so that every record carries a
        # same-box, same-shape pair next to the headline config
        other = LIKE_FOR_LIKE.get(args.model)
        if other is not None and not getattr(args, "no_like_for_like", False):
            try:
                import gc
                import torch
                gc.collect()
                torch.cuda.empty_cache()
                full = _run(args, other)
                like = None if full is None else {"model": other, "value": full["value"], "unit": "tokens/s",
                                                  "ms_per_step": full["ms_per_step"],
                                                  "e2e": {"value": full["e2e"]["value"], "ms_per_step": full["e2e"]["ms_per_step"]}}
            except Exception as e:
                like = {"model": other, "unavailable": _describe(e, other)}
            if line is not None and like is not None:
                line["like_for_like"] = like
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        try:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:
            pass


_DIST_READY = False


def _run(args, model_name):
    """Builds and times one model shape; returns the JSON record on rank 0 (None elsewhere)."""
    global _DIST_READY
    import datetime
    import statistics  # noqa: F401
    import torch
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F
    from config.config import ModelArgs
    from layers.layers import precompute_freqs_cis
    from model.model import LightronTransformer
    from parallel.distributed import setup_distributed

    n = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert n == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={n}"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    tp = args.tp if args.tp is not None else (2 if n >= 2 else 1)
    dp = n // tp
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if not _DIST_READY:
        dist.init_process_group(backend="nccl", init_method="env://", rank=rank, world_size=n,
                                timeout=datetime.timedelta(minutes=10))
        setup_distributed(tp_size=tp, pp_size=1, cp_size=1, ep_size=1, dp_size=dp)
        _DIST_READY = True

    shape = dict(SHAPES[model_name])
    model_args = ModelArgs(max_seq_len=args.seq, norm_eps=1e-5, tp_size=tp, cp_size=1, moe_num_experts=1, moe_topk=2,
                           moe_layer_freq=2, **shape)
    with torch.device("meta"):
        base_model = LightronTransformer(model_args)

    def robust_init_weights(m):       # the reference's initialiser (trainer.py:172-193)
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
        elif "Norm" in m.__class__.__name__:
            if getattr(m, "weight", None) is not None:
                nn.init.ones_(m.weight)
        elif getattr(m, "weight", None) is not None and len(list(m.children())) == 0:
            nn.init.normal_(m.weight, mean=0.0, std=0.02)

    if dp > 1:
        from parallel.parallel_fsdp import apply_fsdp2
        base_model = apply_fsdp2(base_model)
        base_model = base_model.to_empty(device="cuda")
        torch.manual_seed(42)
        base_model.apply(robust_init_weights)
    else:
        base_model = base_model.to_empty(device="cuda")
        base_model.apply(robust_init_weights)
    with torch.no_grad():
        base_model.freqs_cis.copy_(precompute_freqs_cis(model_args.dim // model_args.n_heads, model_args.max_seq_len).to("cuda"))
    model = base_model.to(torch.bfloat16)
    model.train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.01)

    def train_step_single(batch):     # trainer.py:48-55 of the reference, grad_acc_steps = 1
        input_ids = batch["input_ids"].to(device)
        target_ids = batch["target_ids"].to(device)
        logits = model(input_ids)
        loss = F.cross_entropy(logits.view(-1, logits.size(-1)), target_ids.view(-1), reduction="mean")
        loss.backward()
        return loss.item()

    dp_rank = rank // tp
    g = torch.Generator().manual_seed(1234 + dp_rank)

    def host_batch():
        blk = torch.randint(0, shape["vocab_size"], (args.mbs, args.seq + 1), generator=g, dtype=torch.int64)
        return {"input_ids": blk[:, :-1].contiguous().pin_memory(), "target_ids": blk[:, 1:].contiguous().pin_memory()}

    def step(batch):
        optimizer.zero_grad(set_to_none=True)
        loss = train_step_single(batch)
        optimizer.step()
        return loss

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    resident = [{k: v.to(device) for k, v in host_batch().items()} for _ in range(4)]
    for i in range(args.warmup):
        step(resident[i % 4])
    barrier()
    sys.path.insert(0, os.path.dirname(HERE))
    from bench import ClockSampler, METRIC   # the sampler only shells out to nvidia-smi
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(resident[i % 4])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        lv = step(host_batch())
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=device)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    tokens_per_step = args.mbs * dp * args.seq
    del model, base_model, optimizer, resident
    if rank == 0:
        return ({
            "impl": "reference", "metric": METRIC, "value": tokens_per_step / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": n, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (no fp32 master: stock model.to(bfloat16))",
            "data": "synthetic uniform-random token ids, random-init N(0,0.02) weights",
            "config": {"model": model_name, "global_batch": args.mbs * dp, "seq_len": args.seq,
                       "parallelism": f"tp{tp}dp{dp}" if n > 1 else "single",
                       "l2": "working set far exceeds the 126 MB L2"},
            "clocks": clocks, "gpu_launches": 0, "final_loss": loss,
            "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 2 * args.mbs * args.seq * 8, "d2h_bytes_per_step": 4, "last_loss": lv},
        })
    return None
