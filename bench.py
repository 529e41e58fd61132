"""Headline benchmark: training tokens/s of the Llama-style 1.1B model (bf16, fp32 master weights,
AdamW, seq 2048, micro-batch 8 per data-parallel rank, synthetic uniform-random tokens).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 10 --warmup 3

Layout per GPU count: 1 -> single GPU; 2 -> TP2; 4 -> TP2 x DP2; 8 -> TP2 x DP4 (the named config).
With the default model both arms also time `llama-1.1b-mha` (32 KV heads: the nearest shape the
unmodified reference runs, since its attention cannot do GQA) and report it under `like_for_like`.
Rank 0 prints ONE JSON line.  `value` times K optimizer steps on the device (CUDA events, barrier
and synchronize on both sides, MAX over ranks) with batches already resident on the GPU; `e2e`
runs the same steps through the public Trainer API with the data loader's pinned host batches
copied to the device every step and the loss read back to the host every step.
`--impl reference` runs the unmodified reference (installed under baseline/_ref) instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "train tokens/sec (device-timed, max over ranks)"


def layout_for(n: int, tp: int | None):
    if tp is None:
        tp = 2 if n >= 2 else 1
    assert n % tp == 0
    return tp, n // tp


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def _measure_ours(args, model_name, ctx):
    """One model on the current process group: device-timed steps, then the end-to-end steps."""
    import gc
    import torch
    import torch.distributed as dist
    from lightron_b200.config import parse_config
    from lightron_b200.ops import native
    from lightron_b200.trainer import Trainer

    n = int(os.environ.get("WORLD_SIZE", "1"))
    tp, dp = layout_for(n, args.tp)
    raw = {
        "distributed": {"tp_size": tp, "dp_size": dp, "sequence_parallel": bool(args.sp) and tp > 1,
                        "fused_comm": not args.no_fused},
        "model": {"name": model_name},
        "dataset": {"name": "synthetic"},
        "training": {"micro_batch_size": args.mbs, "gradient_accumulation_steps": 1, "seq_length": args.seq,
                     "learning_rate": 3e-4, "total_steps": 10 ** 9, "dtype": "bf16", "seed": 0, "log_interval": 10 ** 9},
    }
    tr = Trainer(parse_config(raw, env={}), ctx=ctx)
    dev = tr.device
    rank = tr.ctx.rank
    tokens_per_step = tr.dataloader.global_batch_size * args.seq

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed: batches resident on the GPU ----
    host_iter = tr.data_iter

    class Resident:
        grad_acc_steps = 1

        def __init__(self, k):
            self.b = [{kk: v.to(dev) for kk, v in next(host_iter).items()} for _ in range(k)]
            self.i = 0

        def __next__(self):
            self.i += 1
            return self.b[self.i % len(self.b)]

    tr.data_iter = Resident(4)
    for _ in range(args.warmup):
        tr.train_step()
    barrier()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    launches0 = native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = tr.train_step()
    e1.record()
    barrier()
    launches = native.launch_count() - launches0
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    final_loss = float(loss)
    native.raise_on_device_status()          # a bounded wait that ran out inside a kernel invalidates the number

    # ---- end to end: pinned host batch -> H2D every step, loss -> host every step ----
    tr.data_iter = host_iter
    for _ in range(2):
        float(tr.train_step())
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        l = tr.train_step()          # Trainer copies this step's pinned input_ids / target_ids to the device
        lv = float(l)                # device -> host read of the loss
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    h2d = 2 * args.mbs * args.seq * 8
    d2h = 4
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    out = {
        "model": model_name, "tokens_per_step": tokens_per_step, "ms": ms, "e2e_ms": e2e_ms, "clocks": clocks,
        "launches": launches, "final_loss": final_loss, "last_loss": lv, "h2d": h2d, "d2h": d2h,
        "global_batch": tr.dataloader.global_batch_size, "tp": tp, "dp": dp, "rank": rank,
    }
    # free this model before the next one is built (arenas, optimizer state, workspaces stay cached per group)
    del tr, host_iter
    gc.collect()
    torch.cuda.empty_cache()
    return out


LIKE_FOR_LIKE = {"llama-1.1b": "llama-1.1b-mha"}     # nearest shape the unmodified reference can run (it cannot run GQA)


def run_ours(args):
    from lightron_b200 import mesh

    n = int(os.environ.get("WORLD_SIZE", "1"))
    assert n == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={n} (launch with torch.distributed.run for N>1)"
    tp, dp = layout_for(n, args.tp)
    ctx = mesh.setup_distributed(tp_size=tp, pp_size=1, cp_size=1, ep_size=1, dp_size=dp)
    m = _measure_ours(args, args.model, ctx)
    like = None
    if args.model in LIKE_FOR_LIKE and not args.no_like_for_like:
        try:
            lm = _measure_ours(args, LIKE_FOR_LIKE[args.model], ctx)
            like = {"model": lm["model"], "value": lm["tokens_per_step"] / (lm["ms"] / 1e3), "unit": "tokens/s",
                    "ms_per_step": lm["ms"], "e2e": {"value": lm["tokens_per_step"] / (lm["e2e_ms"] / 1e3),
                                                     "ms_per_step": lm["e2e_ms"]},
                    "note": "same steps / warmup / layout on the shape the stock reference runs (32 KV heads)"}
        except Exception as e:           # the headline number stands on its own
            like = {"model": LIKE_FOR_LIKE[args.model], "unavailable": f"{type(e).__name__}: {e}"[:300]}
    if m["rank"] == 0:
        ms, e2e_ms, tokens_per_step = m["ms"], m["e2e_ms"], m["tokens_per_step"]
        out = {
            "metric": METRIC, "value": tokens_per_step / (ms / 1e3), "unit": "tokens/s", "n_gpus": n,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if dp == 1 else "weak",
            "scaling_note": "1 -> 2 GPUs splits the same 16384-token batch over TP2 (strong scaling); every further "
                            "pair of GPUs is one more data-parallel replica with its own 16384-token batch (weak scaling)",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init N(0,0.02) weights",
            "impl": "lightron_b200",
            "config": {"model": args.model, "global_batch": m["global_batch"], "seq_len": args.seq,
                       "micro_batch_per_dp_rank": args.mbs, "parallelism": f"tp{tp}dp{dp}" if n > 1 else "single",
                       "sequence_parallel": bool(args.sp) and tp > 1, "optimizer": "AdamW fp32 master (ZeRO-1 over dp)",
                       "l2": "working set (>= 2.2 GB of weights + activations per step) far exceeds the 126 MB L2"},
            "clocks": m["clocks"], "gpu_launches": m["launches"], "final_loss": m["final_loss"],
            "e2e": {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"], "last_loss": m["last_loss"]},
        }
        if like is not None:
            out["like_for_like"] = like
        print(json.dumps(out), flush=True)
    mesh.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-1.1b")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--mbs", type=int, default=8)
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--sp", type=int, default=1, help="sequence parallelism inside the TP group (default on)")
    ap.add_argument("--no-fused", action="store_true", help="library collectives instead of the fused peer-memory kernels")
    ap.add_argument("--no-like-for-like", action="store_true",
                    help="skip the extra measurement of the shape that the unmodified reference can run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        from baseline.run_reference import run_reference
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
