"""Data pipelines.

``SyntheticTokens``: uniform random token ids of a fixed shape, reproducible per (seed, index);
``labels = input_ids`` like the reference's grouped LM data.
``load_text_dataset``: the reference's HF pipeline (tokenise everything, concatenate, cut into
``seq_length`` blocks, ``labels = input_ids.copy()``; reference: train.py:316-371).  It needs the
``datasets`` package, a tokenizer and network or a local cache, so it is imported lazily.
"""
from __future__ import annotations

import multiprocessing
from itertools import chain

import torch
from torch.utils.data import Dataset


class SyntheticTokens(Dataset):
    def __init__(self, vocab_size: int, seq_length: int, num_samples: int = 1 << 16, seed: int = 0):
        self.vocab_size, self.seq_length, self.num_samples, self.seed = vocab_size, seq_length, num_samples, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx: int):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        ids = torch.randint(0, self.vocab_size, (self.seq_length,), generator=g, dtype=torch.int64)
        return {"input_ids": ids, "labels": ids.clone()}


def collate(batch):
    return {k: torch.stack([b[k] for b in batch]) for k in batch[0]}


def load_text_dataset(dataset_name: str, dataset_subset, tokenizer_name: str, seq_length: int,
                      max_position_embeddings: int):
    import datasets  # noqa: lazy, optional dependency
    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(tokenizer_name)
    data = datasets.load_dataset(dataset_name, dataset_subset)
    cols = data["train"].column_names
    text_col = "text" if "text" in cols else cols[0]
    tokenized = data.map(lambda ex: tokenizer(ex[text_col]), batched=True, remove_columns=cols,
                         num_proc=multiprocessing.cpu_count(), load_from_cache_file=True,
                         desc="Running tokenizer on dataset")
    seq_length = seq_length or tokenizer.model_max_length
    if seq_length > max_position_embeddings:
        seq_length = min(1024, max_position_embeddings)

    def group(ex):
        cat = {k: list(chain(*ex[k])) for k in ex.keys()}
        total = len(cat[list(ex.keys())[0]])
        if total > seq_length:
            total = (total // seq_length) * seq_length
        out = {k: [t[i:i + seq_length] for i in range(0, total, seq_length)] for k, t in cat.items()}
        out["labels"] = out["input_ids"].copy()
        return out

    lm = tokenized.map(group, batched=True, num_proc=multiprocessing.cpu_count(), load_from_cache_file=True,
                       desc=f"Grouping texts in chunks of {seq_length}")
    return lm["train"].with_format("torch")
