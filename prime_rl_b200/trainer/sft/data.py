"""SFT data: samples -> packed rows of ``seq_len`` tokens with document boundaries.

``FakeDataset``     synthetic ids (fixed or variable lengths);
``JsonlDataset``    local ``.jsonl`` rows (token ids + mask, or prompt/completion ids);
``PackedDataset``   concatenates samples into rows of exactly ``seq_len`` tokens (the
                    reference's CatDataset, src/prime_rl/trainer/sft/data.py), resumable.
Each data-parallel rank takes every ``world``-th sample, so ranks never see the same data.
"""

from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Iterator

import torch


class FakeDataset:
    def __init__(self, cfg, vocab_size: int):
        self.cfg, self.vocab = cfg, min(vocab_size, 50000)

    def __iter__(self) -> Iterator[dict]:
        rng = random.Random(self.cfg.seed)
        i = 0
        while True:
            n = self.cfg.seq_len if self.cfg.length == "fixed" else rng.randint(max(2, self.cfg.seq_len // 8), self.cfg.seq_len)
            if self.cfg.input_ids == "increasing":
                ids = [(i + j) % self.vocab for j in range(n)]
            else:
                ids = [rng.randrange(self.vocab) for _ in range(n)]
            yield {"input_ids": ids, "loss_mask": [True] * n}
            i += 1


class JsonlDataset:
    def __init__(self, cfg, tokenizer=None):
        p = Path(cfg.name)
        self.files = sorted(p.glob("*.jsonl")) if p.is_dir() else [p]
        if not self.files or not self.files[0].exists():
            raise FileNotFoundError(f"SFT dataset '{cfg.name}' not found (expected a local .jsonl file or directory; "
                                    "there is no dataset hub access in this build)")
        self.cfg, self.tokenizer = cfg, tokenizer

    def _rows(self):
        for f in self.files:
            with open(f) as fh:
                for line in fh:
                    if line.strip():
                        yield json.loads(line)

    def _convert(self, row: dict) -> dict:
        if "input_ids" in row:
            return {"input_ids": row["input_ids"], "loss_mask": row.get("loss_mask", [True] * len(row["input_ids"]))}
        if "prompt_ids" in row:
            p, c = row["prompt_ids"], row["completion_ids"]
            return {"input_ids": p + c, "loss_mask": [False] * len(p) + [True] * len(c)}
        if "messages" in row and self.tokenizer is not None:
            ids, mask = [], []
            lm = self.cfg.loss_mask
            for i, m in enumerate(row["messages"]):
                upto = self.tokenizer.apply_chat_template(row["messages"][: i + 1], tokenize=True)
                new = upto[len(ids):]
                ids = list(upto)
                mask.extend([bool(getattr(lm, m["role"], False))] * len(new))
            return {"input_ids": ids, "loss_mask": mask}
        raise ValueError("unsupported SFT row format")

    def __iter__(self):
        epoch = 0
        while True:
            rows = list(self._rows())
            if self.cfg.shuffle:
                random.Random(self.cfg.seed + epoch).shuffle(rows)
            for r in rows:
                yield self._convert(r)
            epoch += 1


class PackedDataset:
    """Rows of exactly ``seq_len`` tokens; a sample that does not fit is split across rows."""

    def __init__(self, dataset, seq_len: int, rank: int = 0, world: int = 1):
        self.dataset, self.seq_len, self.rank, self.world = dataset, seq_len, rank, world
        self.samples_seen = 0

    def state_dict(self):
        return {"samples_seen": self.samples_seen}

    def load_state_dict(self, sd):
        self.samples_seen = sd.get("samples_seen", 0)

    def __iter__(self):
        ids, mask, lens = [], [], []
        skip = self.samples_seen
        for n, s in enumerate(self.dataset):
            if n % self.world != self.rank:
                continue
            if skip > 0:
                skip -= 1
                continue
            self.samples_seen += 1
            sid, sm = list(s["input_ids"]), list(s["loss_mask"])
            while sid:
                room = self.seq_len - len(ids)
                take = min(room, len(sid))
                ids.extend(sid[:take]); mask.extend(sm[:take]); lens.append(take)
                sid, sm = sid[take:], sm[take:]
                if len(ids) == self.seq_len:
                    pos = [j for L in lens for j in range(L)]
                    yield {"input_ids": torch.tensor(ids), "loss_mask": torch.tensor(mask),
                           "position_ids": torch.tensor(pos, dtype=torch.int32), "sequence_lengths": lens}
                    ids, mask, lens = [], [], []


def setup_dataset(cfg, vocab_size: int, rank: int, world: int, tokenizer=None) -> PackedDataset:
    base = FakeDataset(cfg, vocab_size) if cfg.type == "fake" else JsonlDataset(cfg, tokenizer)
    return PackedDataset(base, cfg.seq_len, rank, world)
