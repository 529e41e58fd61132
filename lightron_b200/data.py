"""Data: micro-batch loader with data-parallel sampling and context-parallel slicing.

Parity with the reference ``data/dataloader.py``: ``MicroBatchDataLoader`` yields
``{"input_ids", "target_ids"}`` of shape ``[micro_batch, seq/cp]`` int64 (``:140-181``), exposes
``global_batch_size = mbs * grad_acc * dp`` (``:44``), ``seq_length_per_gpu`` (``:47``) and
``grad_acc_steps``; text datasets are tokenised, concatenated and cut into blocks of ``seq+1``
tokens (``:96-138``) and sampled per DP rank.  Additions: a ``synthetic`` dataset (uniform random
token ids, no network), zig-zag CP slicing for causal ring attention (rank r owns chunks r and
2c-1-r so that every rank does the same causal work), the global positions of the local slice, a
resumable cursor, and pinned host batches.
"""
from __future__ import annotations

from typing import Dict, Iterator, Optional

import torch

from . import mesh as _mesh


def cp_slice_indices(seq_len: int, cp_size: int, cp_rank: int, mode: str = "contiguous") -> torch.Tensor:
    """Global positions [seq_len / cp] owned by ``cp_rank``."""
    if cp_size == 1:
        return torch.arange(seq_len)
    if mode == "contiguous":
        n = seq_len // cp_size
        return torch.arange(cp_rank * n, (cp_rank + 1) * n)
    if mode == "zigzag":
        assert seq_len % (2 * cp_size) == 0, "zig-zag needs seq_len divisible by 2*cp"
        n = seq_len // (2 * cp_size)
        a = torch.arange(cp_rank * n, (cp_rank + 1) * n)
        b = torch.arange((2 * cp_size - 1 - cp_rank) * n, (2 * cp_size - cp_rank) * n)
        return torch.cat((a, b))
    raise ValueError(f"unknown cp slicing mode {mode}")


class SyntheticTokens:
    """Sample i is ``seq_len + 1`` uniform ids in [0, vocab) drawn from a generator seeded by
    (seed, i): any rank can produce any sample, and a run can resume at any cursor."""

    def __init__(self, vocab_size: int, seq_len: int, seed: int = 0, num_samples: int = 1 << 30):
        self.vocab_size, self.seq_len, self.seed, self.num_samples = vocab_size, seq_len, seed, num_samples

    def __len__(self):
        return self.num_samples

    def batch(self, first: int, count: int) -> torch.Tensor:
        # sample i is a function of (seed, i) alone: the same global batch holds the same rows however
        # it is cut into micro-batches or spread over data-parallel ranks
        g = torch.Generator()
        rows = []
        for i in range(first, first + count):
            g.manual_seed(self.seed * 1_000_003 + i)
            rows.append(torch.randint(0, self.vocab_size, (self.seq_len + 1,), generator=g, dtype=torch.int64))
        return torch.stack(rows)


class TokenBlocks:
    """A tokenised corpus cut into blocks of seq_len + 1 (the reference's map-style pipeline)."""

    def __init__(self, ids: torch.Tensor, seq_len: int):
        n = (ids.numel() - 1) // (seq_len + 1)
        self.blocks = ids[: n * (seq_len + 1)].view(n, seq_len + 1)

    def __len__(self):
        return self.blocks.shape[0]

    def batch(self, first: int, count: int) -> torch.Tensor:
        idx = (torch.arange(first, first + count)) % len(self)
        return self.blocks[idx]


def load_text_dataset(name: str, tokenizer_name: str, split: str, seq_len: int, max_samples: Optional[int]):
    """HF ``datasets`` + tokenizer path (needs a local cache or network; absent offline)."""
    try:
        from datasets import load_dataset
        from transformers import AutoTokenizer
    except ImportError as e:
        raise RuntimeError(f"dataset '{name}' needs the `datasets` package ({e}); use dataset.name='synthetic'")
    tok = AutoTokenizer.from_pretrained(tokenizer_name)
    ds = load_dataset(name, split=split)
    if max_samples:
        ds = ds.select(range(min(max_samples, len(ds))))
    ids = []
    for row in ds:
        ids.extend(tok(row["text"])["input_ids"])
        ids.append(tok.eos_token_id or 0)
    return TokenBlocks(torch.tensor(ids, dtype=torch.int64), seq_len)


class MicroBatchDataLoader:
    def __init__(self, micro_batch_size: int, seq_length: int, dataset_name: str = "synthetic",
                 tokenizer_name: Optional[str] = None, grad_acc_steps: int = 1, vocab_size: int = 32000,
                 split: str = "train", max_samples: Optional[int] = None, seed: int = 42, num_workers: int = 0,
                 cp_mode: str = "contiguous", ctx: Optional[_mesh.ParallelContext] = None, pin_memory: bool = False):
        ctx = ctx or _mesh.get_context()
        self.ctx = ctx
        self.micro_batch_size, self.seq_length, self.grad_acc_steps = micro_batch_size, seq_length, grad_acc_steps
        self.dp_world_size, self.dp_rank = ctx.dp_size, ctx.dp_rank
        self.cp_world_size, self.cp_rank = ctx.cp_size, ctx.cp_rank
        self.global_batch_size = micro_batch_size * grad_acc_steps * self.dp_world_size
        assert seq_length % self.cp_world_size == 0
        self.seq_length_per_gpu = seq_length // self.cp_world_size
        if dataset_name == "synthetic":
            self.dataset = SyntheticTokens(vocab_size, seq_length, seed=seed)
        else:
            self.dataset = load_text_dataset(dataset_name, tokenizer_name, split, seq_length, max_samples)
        self.positions = cp_slice_indices(seq_length, self.cp_world_size, self.cp_rank, cp_mode)
        self.cursor = 0                    # micro-batches consumed by this rank
        self.pin_memory = pin_memory and torch.cuda.is_available()

    def state_dict(self) -> Dict[str, int]:
        return {"cursor": self.cursor}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.cursor = int(sd["cursor"])

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        # global sample order: micro-batch m of dp rank r covers samples (m*dp + r)*mbs ...
        first = (self.cursor * self.dp_world_size + self.dp_rank) * self.micro_batch_size
        self.cursor += 1
        blk = self.dataset.batch(first, self.micro_batch_size)
        inp = blk[:, :-1].index_select(1, self.positions).contiguous()
        tgt = blk[:, 1:].index_select(1, self.positions).contiguous()
        if self.pin_memory:
            inp, tgt = inp.pin_memory(), tgt.pin_memory()
        return {"input_ids": inp, "target_ids": tgt}
