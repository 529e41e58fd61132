"""Training engine behind ``trainer.py --config X.json``.

Follows the reference's ``trainer.py:74-345`` step by step (config sections, env overrides,
distributed set-up, ModelArgs, model build + N(0, 0.02) init, data loader, AdamW, gradient
accumulation, PP engines, TPS line every ``log_interval`` steps, final checkpoint) with these
intended differences: the loss is never pulled to the host inside the step (the reference calls
``loss.item()`` per micro-batch, trainer.py:55); throughput is timed on the device and reduced
with MAX over ranks, next to the reference's wall-clock TPS; bf16 runs keep fp32 master weights;
periodic checkpoints and exact resume exist; PP composes with DP; a JSONL metrics log is written.
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from . import checkpoint as ckpt
from . import mesh as _mesh
from .config import RunConfig, build_model_args, load_config
from .data import MicroBatchDataLoader
from .models.llama import LightronTransformer, init_weights
from .ops import native
from .optim import DistributedAdamW
from .parallel import fused
from .parallel.pp import PipelineParallel, init_pp_group_manager, train_step_pipeline_1f1b, train_step_pipeline_afab
from .timing import StepTimer


class InfiniteDataIterator:
    """``next()`` never raises StopIteration and exposes ``grad_acc_steps`` (trainer.py:58-71)."""

    def __init__(self, dataloader, grad_acc_steps: int):
        self.dataloader, self.grad_acc_steps = dataloader, grad_acc_steps
        self._it = iter(dataloader)

    def __next__(self):
        try:
            return next(self._it)
        except StopIteration:
            self._it = iter(self.dataloader)
            return next(self._it)


def train_step_single(model, batch, grad_acc_steps: int, device, positions=None) -> torch.Tensor:
    """One micro-batch forward + backward.  Returns the (already divided) loss as a device scalar."""
    input_ids = batch["input_ids"].to(device, non_blocking=True)
    target_ids = batch["target_ids"].to(device, non_blocking=True)
    loss = model.loss(input_ids, target_ids, positions=positions) / grad_acc_steps
    loss.backward()
    return loss.detach()


class Trainer:
    def __init__(self, cfg: RunConfig, ctx: Optional[_mesh.ParallelContext] = None):
        self.cfg = cfg
        d, t = cfg.distributed, cfg.training
        self.ctx = ctx or _mesh.setup_distributed(tp_size=d.tp_size, pp_size=d.pp_size, cp_size=d.cp_size,
                                                  ep_size=d.ep_size, dp_size=d.dp_size)
        ctx = self.ctx
        self.device = ctx.device
        fused.set_fused(d.fused_comm)
        init_pp_group_manager(ctx)
        from . import health
        health.check_config_agreement(cfg.to_dict())        # a rank started with another JSON fails here
        self.args = build_model_args(cfg)
        self.dtype = torch.bfloat16 if t.dtype == "bf16" else torch.float32
        torch.manual_seed(t.seed)
        if d.pp_size > 1:
            self.model = PipelineParallel(self.args, ctx=ctx, dtype=self.dtype, device=self.device)
            net = self.model.stage
        else:
            self.model = LightronTransformer(self.args, ctx, dtype=self.dtype, device=self.device)
            net = self.model
        self.net = net
        init_weights(net, seed=t.seed)
        net.train()
        self.optimizer = self._build_engine(net)
        cp_mode = "zigzag" if (d.cp_size > 1 and d.cp_mode in ("ring", "allgather")) else "contiguous"
        self.dataloader = MicroBatchDataLoader(
            micro_batch_size=t.micro_batch_size, seq_length=t.seq_length, dataset_name=cfg.dataset.name,
            tokenizer_name=cfg.dataset.tokenizer or cfg.model.get("name"), grad_acc_steps=t.gradient_accumulation_steps,
            vocab_size=self.args.vocab_size, split=cfg.dataset.split, max_samples=t.max_samples, seed=t.seed,
            num_workers=cfg.dataset.num_workers, cp_mode=cp_mode, ctx=ctx, pin_memory=self.device.type == "cuda")
        self.data_iter = InfiniteDataIterator(self.dataloader, t.gradient_accumulation_steps)
        self.positions = self.dataloader.positions.to(self.device) if d.cp_size > 1 else None
        rows = t.micro_batch_size * self.dataloader.seq_length_per_gpu
        if self.args.sequence_parallel and d.tp_size > 1:
            rows //= d.tp_size
        self.tensor_shapes = (rows, self.args.dim)
        if self.args.sequence_parallel and d.tp_size > 1 and d.fused_comm and self.device.type == "cuda":
            from .parallel import symm
            tokens = t.micro_batch_size * self.dataloader.seq_length_per_gpu
            if symm.supported(ctx.tp_group) and symm.shapes_ok(tokens, ctx.tp_group):
                n_layers = len(net.layers)
                per_mb = 2 * n_layers + (1 if net.last_stage else 0)
                in_flight = 1 if d.pp_size == 1 else (d.pp_size if d.pp_engine == "1f1b" else t.gradient_accumulation_steps)
                symm.presize(ctx.tp_group, tokens, self.args.dim, self.device, fwd_gathers_in_flight=per_mb * in_flight)
        self.step = 0
        self.tokens_seen = 0
        # MFU denominator: the bf16 matmul rate measured on this machine under sustained load when the
        # measurement file is present, else the nominal dense figure
        peaks = native.measured_peaks()
        self.peak_flops = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]) * 1e12
        self.peak_source = peaks["source"]
        self.timer = StepTimer(self.device)
        # liveness: every rank publishes a beat in the rendezvous store at each log interval and looks
        # at the others' (health.Heartbeat); a rank that stopped beating is reported on the host before
        # the next collective would hang on it
        self.heartbeat = None
        if dist.is_initialized() and ctx.world_size > 1 and t.heartbeat_timeout_s > 0:
            try:
                store = dist.distributed_c10d._get_default_store()
                self.heartbeat = health.Heartbeat(store, ctx.rank, ctx.world_size)
                self.heartbeat.beat()
            except Exception:
                self.heartbeat = None
        if t.resume:
            meta = ckpt.load(t.resume, self.model, self.optimizer, self.dataloader, ctx)
            self.step, self.tokens_seen = meta["trained_steps"], meta["trained_tokens"]

    def _build_engine(self, net):
        """Data-parallel engine.  Default: replicated bf16 parameters, optimizer state sharded over the
        replicas (``DistributedAdamW``).  ``distributed.fsdp``: parameters, gradients and optimizer
        state sharded per transformer block (the reference wires ``apply_fsdp2`` whenever dp > 1,
        trainer.py:198-203): the peer-memory engine when the layout allows it, else the
        library-collective one."""
        d, t, ctx = self.cfg.distributed, self.cfg.training, self.ctx
        if d.fsdp and ctx.grad_replicas > 1:
            from .parallel import fsdp as fsdp_lib, fsdp_native
            why_not = fsdp_native.supported(net, ctx, self.dtype, t.grad_clip)
            if why_not is None:
                self.engine = "fsdp (peer-memory kernels)"
                return fsdp_native.NativeFSDP(net, ctx, lr=t.learning_rate, weight_decay=t.weight_decay, betas=t.betas, eps=t.eps)
            if d.pp_size == 1 and not any(getattr(p, "is_expert", False) for p in net.parameters()):
                self.engine = f"fsdp (library collectives: {why_not})"
                fsdp_lib.apply_fsdp2(net, ctx=ctx, param_dtype=self.dtype)
                return fsdp_lib.FSDPOptimizer(net, lr=t.learning_rate, weight_decay=t.weight_decay, betas=t.betas, eps=t.eps)
            if ctx.rank == 0:
                print(f"[lightron] distributed.fsdp ignored for this layout ({why_not}); using the sharded-optimizer engine",
                      flush=True)
        self.engine = "sharded optimizer (replicated bf16 parameters)"
        return DistributedAdamW(net, lr=t.learning_rate, weight_decay=t.weight_decay, betas=t.betas, eps=t.eps, ctx=ctx,
                                grad_clip=t.grad_clip)

    # ------------------------------------------------------------------------------------------
    def train_step(self) -> torch.Tensor:
        """One optimizer step (all micro-batches).  Returns the summed loss as a device scalar."""
        d, t = self.cfg.distributed, self.cfg.training
        ga = t.gradient_accumulation_steps
        self.optimizer.zero_grad()
        if d.pp_size > 1:
            fn = train_step_pipeline_afab if d.pp_engine == "afab" else train_step_pipeline_1f1b
            loss = fn(self.model, self.data_iter, self.tensor_shapes, self.device, self.dtype,
                      optimizer=self.optimizer, positions=self.positions)
        else:
            loss = torch.zeros((), dtype=torch.float32, device=self.device)
            for i in range(ga):
                batch = next(self.data_iter)
                assert batch["input_ids"].shape[1] == self.dataloader.seq_length_per_gpu
                self.optimizer.set_requires_gradient_sync(i == ga - 1)
                loss += train_step_single(self.model, batch, ga, self.device, self.positions).float()
        self.optimizer.step()
        self.step += 1
        self.tokens_seen += self.dataloader.global_batch_size * t.seq_length
        return loss

    def _check_liveness(self) -> None:
        """Beat, then fail loudly if a rank has not beaten for ``heartbeat_timeout_s`` (it died or is
        stuck between steps; the survivors would otherwise sit in the next collective until its timeout)."""
        hb = self.heartbeat
        if hb is None:
            return
        from . import health
        hb.beat()
        dead = hb.dead_ranks(self.cfg.training.heartbeat_timeout_s)
        if dead:
            raise health.RankFailure(f"ranks {dead} have not published a heartbeat for more than "
                                     f"{self.cfg.training.heartbeat_timeout_s:.0f} s")

    def save(self, path: Optional[str] = None) -> str:
        d = self.cfg.distributed
        path = path or ckpt.ckpt_name(self.step, d.tp_size, d.dp_size, self.cfg.training.save_dir)
        if self.device.type == "cuda" and native.available():
            native.raise_on_device_status()        # never checkpoint state that a timed-out kernel may have skipped
        ckpt.save(path, self.model, self.optimizer, self.step, self.tokens_seen, self.dataloader, self.ctx)
        return path

    def fit(self) -> Dict[str, Any]:
        """The training loop.  A rank that leaves it with an exception announces that in the store; a rank
        whose own step then fails names the rank that failed first as the cause."""
        from . import health
        hb = self.heartbeat
        try:
            return self._fit()
        except health.RankFailure:
            raise
        except Exception as e:
            if hb is not None:
                first = health.failed_ranks(hb.store, hb.world, exclude=hb.rank)
                if first:
                    raise health.RankFailure(f"rank(s) {sorted(first)} failed first ({'; '.join(first.values())}); this rank's "
                                             f"own error was {type(e).__name__}: {str(e)[:200]}") from e
                health.announce_failure(hb.store, hb.rank, f"{type(e).__name__}: {e}")
            raise

    def _fit(self) -> Dict[str, Any]:
        from . import health
        t, ctx = self.cfg.training, self.ctx
        is_log = ctx.rank == ctx.log_rank
        tokens_per_step = self.dataloader.global_batch_size * t.seq_length
        log_f = open(t.jsonl_log, "a") if (t.jsonl_log and is_log) else None
        if ctx.rank == 0:
            n = sum(p.numel() for p in self.net.parameters())
            print(f"Model initialized. Local parameters: {n / 1e9:.3f}B | {ctx.describe()} | engine: {self.engine}", flush=True)
            print("\n=== Start Training ===", flush=True)
        start = time.time()
        first_step, tokens0 = self.step, self.tokens_seen
        last_loss = float("nan")
        prof = None
        while self.step < t.total_steps:
            # optional torch.profiler window (training.profile_steps = [first, last], log rank only): the
            # steps inside it run under the profiler and are not representative of the step time
            if t.profile_steps and is_log and prof is None and self.step + 1 == int(t.profile_steps[0]):
                acts = [torch.profiler.ProfilerActivity.CPU]
                if self.device.type == "cuda":
                    acts.append(torch.profiler.ProfilerActivity.CUDA)
                prof = torch.profiler.profile(activities=acts)
                prof.__enter__()
            health.maybe_inject_failure(self.step + 1, ctx.rank)
            self.timer.start()
            if self.device.type == "cuda":
                torch.cuda.nvtx.range_push(f"step {self.step + 1}")
            loss = self.train_step()
            if self.device.type == "cuda":
                torch.cuda.nvtx.range_pop()
            self.timer.stop()
            if prof is not None and (self.step >= int(t.profile_steps[1]) or self.step == t.total_steps):
                prof.__exit__(None, None, None)
                trace = os.path.join(t.profile_dir, f"lightron_trace_rank{ctx.rank}.json")
                prof.export_chrome_trace(trace)
                print(f"profiler trace of steps {t.profile_steps[0]}-{self.step} written to {trace}", flush=True)
                prof, t.profile_steps = None, None
            if self.step % t.log_interval == 0 or self.step == t.total_steps:
                ms = self.timer.mean_ms_max_over_ranks()          # device time, MAX over ranks
                # the reference prints rank 0's local loss (trainer.py:308-314); here it is the mean
                # over the dp x cp replicas, taken from the last pipeline stage
                if ctx.grad_replicas > 1:
                    dist.all_reduce(loss, group=ctx.dpcp_group)
                    loss = loss / ctx.grad_replicas
                last_loss = float(loss)                            # the only host sync, once per log interval
                if self.device.type == "cuda" and native.available():
                    native.raise_on_device_status()                # bounded waits that ran out inside a kernel
                    dropped = native.take_moe_dropped()
                    if dropped["events"]:
                        print(f"[rank {ctx.rank}] step {self.step}: expert capacity exceeded, {dropped['events']} routed copies / plans "
                              f"dropped (largest demand {dropped['max_rows']} rows; raise model.moe_capacity_factor)", flush=True)
                self._check_liveness()
                if is_log:
                    tps_wall = (self.tokens_seen - tokens0) / max(time.time() - start, 1e-9)
                    tps_dev = tokens_per_step / (ms / 1e3) if ms > 0 else float("nan")
                    # model FLOPs: 6 N per token for the matmuls + causal attention (fwd + bwd)
                    a = self.args
                    flops_tok = 6.0 * a.num_active_params() + 6.0 * a.n_layers * a.dim * t.seq_length
                    mfu = flops_tok * tps_dev / (ctx.world_size * self.peak_flops) if ms > 0 else float("nan")
                    print(f"Step {self.step}/{t.total_steps} | Loss: {last_loss:.4f} | TPS: {tps_wall:.2f} tokens/s"
                          f" | device TPS: {tps_dev:.2f} | step {ms:.2f} ms | MFU {mfu * 100:.1f}%", flush=True)
                    if log_f:
                        log_f.write(json.dumps({"step": self.step, "loss": last_loss, "tokens_per_s_wall": tps_wall,
                                                "tokens_per_s_device": tps_dev, "step_ms": ms, "mfu": mfu, "mfu_peak_tflops": self.peak_flops / 1e12,
                                                "mfu_peak_source": self.peak_source,
                                                "tokens_seen": self.tokens_seen}) + "\n")
                        log_f.flush()
                self.timer.reset()
            if t.save_interval and self.step % t.save_interval == 0 and self.step < t.total_steps:
                self.save()
        path = self.save() if (t.save_final and (t.total_steps > first_step or not t.resume)) else None
        if is_log:
            print("Training Finished!", flush=True)
        if log_f:
            log_f.close()
        return {"loss": last_loss, "steps": self.step, "tokens": self.tokens_seen, "checkpoint": path}


def main(argv=None) -> Dict[str, Any]:
    import argparse
    parser = argparse.ArgumentParser(description="lightron-b200 training script")
    parser.add_argument("--config", type=str, required=True, help="Path to JSON config file")
    a = parser.parse_args(argv)
    cfg = load_config(a.config)
    if int(os.environ.get("RANK", 0)) == 0:
        print(f"Starting training with config: {a.config}", flush=True)
    trainer = Trainer(cfg)
    try:
        return trainer.fit()
    finally:
        _mesh.destroy()
