"""Evaluation loop: mean loss and perplexity over at most ``max_batches`` batches.

Parity with the reference's ``utils/utils.py:4-29`` (``evaluate(model, dataloader, device,
max_batches)`` -> loss / perplexity).  Uses the model's vocab-parallel loss, keeps the running
sum on the device (one host read at the end) and averages over the data-parallel group.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.distributed as dist


@torch.no_grad()
def evaluate(model, dataloader, device, max_batches: Optional[int] = 50, positions=None, group=None) -> Dict[str, float]:
    was_training = model.training
    model.eval()
    total = torch.zeros((), dtype=torch.float64, device=device)
    n = 0
    for i, batch in enumerate(dataloader):
        if max_batches is not None and i >= max_batches:
            break
        loss = model.loss(batch["input_ids"].to(device), batch["target_ids"].to(device), positions=positions)
        total += loss.double()
        n += 1
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        t = torch.stack((total, torch.tensor(float(n), dtype=torch.float64, device=device)))
        dist.all_reduce(t, group=group)
        total, n = t[0], float(t[1])
    mean = float(total) / max(n, 1)
    if was_training:
        model.train()
    return {"loss": mean, "perplexity": math.exp(min(mean, 50.0)), "batches": n}
