"""gloo multi-process tests: ring collectives vs library collectives, FSDP / DDP parity with a
single process, TP checkpoint gather + re-shard, host-side failure detection."""
import copy
import os

import pytest
import torch

from dist_utils import run_distributed


def _ring_worker(rank, world):
    import torch.distributed as dist
    from lightron_b200.parallel.collectives import ring_all_gather, ring_all_reduce, ring_p2p, ring_reduce_scatter
    g = dist.new_group(list(range(world)))
    torch.manual_seed(rank)
    x = torch.randn(1000 + 3)                                   # not divisible by the world size
    want = x.clone()
    dist.all_reduce(want, group=g)
    got = ring_all_reduce(x.clone(), g)
    assert (got - want).abs().max() < 1e-5
    y = torch.randn(5, 7)
    outs = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(outs, y, group=g)
    assert torch.equal(ring_all_gather(y, g), torch.cat(outs))
    chunks = [torch.randn(4, 3) for _ in range(world)]
    total = torch.stack(chunks).clone()
    dist.all_reduce(total, group=g)
    assert (ring_reduce_scatter(chunks, g) - total[rank]).abs().max() < 1e-5
    t = torch.full((3,), float(rank))
    ring_p2p(t, src=0, dst=world - 1, group=g)
    if rank == world - 1:
        assert torch.equal(t, torch.zeros(3))
    return True


@pytest.mark.parametrize("world", [2, 4])
def test_ring_collectives_match_library(world):
    assert all(run_distributed(_ring_worker, world))


ARGS = dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=256, intermediate_size=96, max_seq_len=32)


def _batches(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 256, (2, 32), generator=g) for _ in range(n)]


def _single_reference(steps, world):
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    mesh.set_context(None)
    m = LightronTransformer(ModelArgs(**ARGS))
    init_weights(m, 1)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3, weight_decay=0.01)
    data = _batches(steps * world)
    for s in range(steps):
        opt.zero_grad()
        for r in range(world):
            tok = data[s * world + r]
            (m.loss(tok, torch.roll(tok, -1, 1)) / world).backward()
        opt.step()
    return {k: v.detach().clone() for k, v in m.state_dict().items()}


def _fsdp_worker(rank, world, steps, strategy):
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.parallel import apply_fsdp1
    ctx = mesh.setup_distributed(dp_size=world)
    m = LightronTransformer(ModelArgs(**ARGS), ctx)
    init_weights(m, 1)
    apply_fsdp1(m, strategy=strategy, ctx=ctx)
    numel_local = sum(p.numel() for p in m._fsdp.parameters())
    opt = m._fsdp.make_optimizer(lr=1e-3, weight_decay=0.01)
    data = _batches(steps * world)
    for s in range(steps):
        opt.zero_grad()
        tok = data[s * world + rank]
        m.loss(tok, torch.roll(tok, -1, 1)).backward()
        opt.step()
    return {k: v.numpy().copy() for k, v in m._fsdp.full_state_dict().items()}, numel_local      # numpy pickles by value


@pytest.mark.parametrize("strategy", ["full", "grad_op"])
def test_fsdp_matches_single_process(strategy):
    want = _single_reference(3, 2)
    (got, numel_local), _ = run_distributed(_fsdp_worker, 2, 3, strategy)
    total = sum(v.numel() for v in want.values())
    assert numel_local < 0.6 * total                       # each rank really holds about half
    for k, v in want.items():
        assert torch.allclose(torch.from_numpy(got[k]), v, atol=2e-5), k


def _ddp_worker(rank, world, steps):
    from lightron_b200 import mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    from lightron_b200.parallel import DataParallel
    ctx = mesh.setup_distributed(dp_size=world)
    m = LightronTransformer(ModelArgs(**ARGS), ctx)
    init_weights(m, 1)
    ddp = DataParallel(m, group=ctx.dp_group, bucket_mb=0.05)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3, weight_decay=0.01)
    data = _batches(steps * world)
    for s in range(steps):
        opt.zero_grad()
        tok = data[s * world + rank]
        ddp.loss(tok, torch.roll(tok, -1, 1)).backward()
        ddp.finish_grad_sync()
        opt.step()
    return {k: v.detach().numpy().copy() for k, v in m.state_dict().items()}


def test_ddp_buckets_match_single_process():
    want = _single_reference(3, 2)
    got = run_distributed(_ddp_worker, 2, 3)[0]
    for k, v in want.items():
        assert torch.allclose(torch.from_numpy(got[k]), v, atol=2e-5), k


def _ckpt_worker(rank, world, tmp):
    from lightron_b200 import checkpoint as ckpt, mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer, init_weights
    ctx = mesh.setup_distributed(tp_size=world)
    args = ModelArgs(**ARGS, tp_size=world)
    m = LightronTransformer(args, ctx)
    init_weights(m, 5)
    path = os.path.join(tmp, "ck")
    ckpt.save(path, m, None, 7, 123, None, ctx)
    full = torch.load(path, weights_only=False)
    m2 = LightronTransformer(args, ctx)
    ckpt.load(path, m2, None, None, ctx)
    same = all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
    return {k: tuple(v.shape) for k, v in full["model"].items()}, full["trained_steps"], same


def test_tp_checkpoint_holds_full_tensors_and_reshards(tmp_path):
    shapes, steps, same = run_distributed(_ckpt_worker, 2, str(tmp_path))[0]
    assert steps == 7 and same
    assert shapes["layers.0.attention.wq.weight"] == (64, 64)          # unsharded, loadable by the reference layout
    assert shapes["layers.0.feed_forward.w2.weight"] == (64, 96)
    assert shapes["tok_embeddings.weight"] == (256, 64)
    # the same file loads into a single-process (tp=1) model
    from lightron_b200 import checkpoint as ckpt, mesh
    from lightron_b200.config import ModelArgs
    from lightron_b200.models import LightronTransformer
    mesh.set_context(None)
    m = LightronTransformer(ModelArgs(**ARGS))
    meta = ckpt.load(os.path.join(str(tmp_path), "ck"), m)
    assert meta["trained_tokens"] == 123


def _failure_worker(rank, world):
    """Rank 1 'dies' between steps (stops beating, never joins the next collective)."""
    import time
    import torch.distributed as dist
    from lightron_b200.health import Heartbeat, RankFailure, check_config_agreement, guarded
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world)
    out = {}
    try:
        check_config_agreement({"lr": 1e-3 if rank != 1 else 2e-3})
        out["mismatch"] = False
    except RankFailure as e:
        out["mismatch"] = "ranks [1]" in str(e)
    hb.beat()
    dist.barrier()
    if rank == 1:
        time.sleep(2.5)                      # no more beats, no more collectives for a while
        out["dead"] = None
    else:
        time.sleep(1.2)
        hb.beat()
        out["dead"] = hb.dead_ranks(max_age_s=1.0)
        t = torch.zeros(1)
        try:
            guarded(lambda: dist.all_reduce(t), timeout_s=0.5, what="all_reduce")
            out["guard"] = "returned"
        except RankFailure:
            out["guard"] = "timeout"
    return out


def test_host_side_failure_detection():
    res = run_distributed(_failure_worker, 2)
    assert res[0]["mismatch"] and res[1]["mismatch"]
    assert res[0]["dead"] == [1]
    assert res[0]["guard"] == "timeout"


_RESHARD = {
    "distributed": {},
    "model": {"name": "tiny"},
    "dataset": {"name": "synthetic"},
    "training": {"micro_batch_size": 2, "gradient_accumulation_steps": 1, "seq_length": 64, "learning_rate": 3e-4,
                 "total_steps": 2, "seed": 0, "dtype": "fp32", "log_interval": 1000},
}


def _reshard_worker(rank, world, tmp, phase):
    import copy
    import warnings
    from lightron_b200.config import parse_config
    from lightron_b200.trainer import Trainer
    raw = copy.deepcopy(_RESHARD)
    if phase == "save":
        raw["distributed"]["tp_size"] = 2
        raw["training"]["save_dir"] = tmp
        out = Trainer(parse_config(raw, env={})).fit()
        return out["checkpoint"]
    raw["distributed"]["dp_size"] = 2
    raw["training"].update(resume=os.path.join(tmp, "ckpt_step_2_tpsize_2_dpsize_1"), total_steps=3, save_final=False)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        tr = Trainer(parse_config(raw, env={}))
    warned = any("parallel layout" in str(x.message) for x in w)
    loss = float(tr.train_step())
    return warned, tr.step, tr.dataloader.cursor, loss, int(tr.optimizer.step_count)


def test_checkpoint_resumes_under_another_layout(tmp_path):
    """Saved at tp=2, resumed at dp=2: the per-rank optimizer shards, RNG state and data cursor of
    the old layout must not be loaded into ranks that mean something else now."""
    run_distributed(_reshard_worker, 2, str(tmp_path), "save")
    res = run_distributed(_reshard_worker, 2, str(tmp_path), "load")
    for warned, step, cursor, loss, opt_steps in res:
        assert warned
        assert step == 3 and cursor == 3          # cursor recomputed from the step count (2), then one more batch
        assert opt_steps == 1                       # moments restarted
        assert loss == loss and loss < 20.0


def _recovery_worker(rank, world, tmp, phase):
    """dp2 run of 4 steps with a checkpoint every 2.  'full': uninterrupted.  'crash': rank 1 raises before
    step 3 (host-side injection, nothing in flight).  'resume': relaunch from the step-2 checkpoint."""
    import copy
    from lightron_b200 import health
    from lightron_b200.config import parse_config
    from lightron_b200.trainer import Trainer
    raw = copy.deepcopy(_RESHARD)
    raw["distributed"]["dp_size"] = 2
    raw["training"].update(total_steps=4, save_interval=2, save_final=False, log_interval=1, heartbeat_timeout_s=60.0,
                           save_dir=os.path.join(tmp, "full" if phase == "full" else "crash"))
    os.makedirs(raw["training"]["save_dir"], exist_ok=True)
    os.environ.pop("LIGHTRON_INJECT_FAILURE", None)
    if phase == "crash":
        os.environ["LIGHTRON_INJECT_FAILURE"] = "1:3"
    if phase == "resume":
        raw["training"]["resume"] = os.path.join(tmp, "crash", "ckpt_step_2_tpsize_1_dpsize_2")
    tr = Trainer(parse_config(raw, env={}))
    try:
        tr.fit()
    except health.InjectedFailure as e:
        return "injected", str(e), tr.step
    except health.RankFailure as e:
        return "rank_failure", str(e), tr.step
    return "done", {k: v.float().numpy() for k, v in tr.model.state_dict().items()}, tr.step


def test_injected_rank_failure_is_reported_and_recovered_from_the_last_checkpoint(tmp_path):
    """A rank dies between steps (host-side injection): the survivor's collective times out, the survivor names
    the rank that failed first, and a relaunch from the last periodic checkpoint ends with the weights of the
    uninterrupted run."""
    import numpy as np
    full = run_distributed(_recovery_worker, 2, str(tmp_path), "full")
    assert full[0][0] == "done" and full[0][2] == 4
    crash = run_distributed(_recovery_worker, 2, str(tmp_path), "crash", pg_timeout_s=8)
    assert crash[1][0] == "injected" and crash[1][2] == 2
    assert crash[0][0] == "rank_failure" and "rank(s) [1] failed first" in crash[0][1] and "InjectedFailure" in crash[0][1]
    assert os.path.exists(tmp_path / "crash" / "ckpt_step_2_tpsize_1_dpsize_2")
    resumed = run_distributed(_recovery_worker, 2, str(tmp_path), "resume")
    assert resumed[0][0] == "done" and resumed[0][2] == 4
    for k, v in full[0][1].items():
        assert np.allclose(v, resumed[0][1][k], atol=1e-6), k
