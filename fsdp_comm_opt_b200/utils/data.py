"""Data pipelines.

``SyntheticTokens``: uniform random token ids of a fixed shape, reproducible per (seed, index);
``labels = input_ids`` like the reference's grouped LM data.
``load_text_dataset``: the reference's HF pipeline (tokenise everything, concatenate, cut into
``seq_length`` blocks, ``labels = input_ids.copy()``; reference: train.py:316-371).  The dataset
name may be a hub id (needs network or a local cache) or a local ``.txt`` / ``.json`` / ``.jsonl`` /
``.csv`` file or a directory of them; the tokenizer may be a hub id, a local directory, or
``"bytes"`` for the built-in byte-level tokenizer (ids 0..255), so the pipeline also runs offline.
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


class ByteTokenizer:
    """Byte-level tokenizer: UTF-8 bytes as ids 0..255.  Needs no files; any vocabulary of at least
    256 entries can train on it."""

    model_max_length = 1 << 30

    def __call__(self, texts):
        if isinstance(texts, str):
            texts = [texts]
        ids = [list(t.encode("utf-8")) for t in texts]
        return {"input_ids": ids, "attention_mask": [[1] * len(i) for i in ids]}


def _load_raw(dataset_name: str, dataset_subset):
    import os

    import datasets  # noqa: lazy, optional dependency

    kinds = {".txt": "text", ".json": "json", ".jsonl": "json", ".csv": "csv"}
    if os.path.isdir(dataset_name):
        files = sorted(os.path.join(dataset_name, f) for f in os.listdir(dataset_name)
                       if os.path.splitext(f)[1] in kinds)
        if not files:
            raise FileNotFoundError(f"no .txt/.json/.jsonl/.csv files in {dataset_name}")
        return datasets.load_dataset(kinds[os.path.splitext(files[0])[1]], data_files={"train": files})
    if os.path.isfile(dataset_name):
        return datasets.load_dataset(kinds[os.path.splitext(dataset_name)[1]], data_files={"train": dataset_name})
    return datasets.load_dataset(dataset_name, dataset_subset)


def load_text_dataset(dataset_name: str, dataset_subset, tokenizer_name: str, seq_length: int,
                      max_position_embeddings: int, vocab_size: int | None = None, num_proc: int | None = None):
    if tokenizer_name == "bytes":
        tokenizer = ByteTokenizer()
    else:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(tokenizer_name)
    n_tok = 256 if tokenizer_name == "bytes" else len(tokenizer)
    if vocab_size is not None and n_tok > vocab_size:
        raise ValueError(f"tokenizer has {n_tok} ids but the model's vocabulary is {vocab_size}")
    data = _load_raw(dataset_name, dataset_subset)
    cols = data["train"].column_names
    text_col = "text" if "text" in cols else cols[0]
    num_proc = num_proc or multiprocessing.cpu_count()
    tokenized = data.map(lambda ex: tokenizer(ex[text_col]), batched=True, remove_columns=cols,
                         num_proc=num_proc, load_from_cache_file=True,
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

    lm = tokenized.map(group, batched=True, num_proc=num_proc, load_from_cache_file=True,
                       desc=f"Grouping texts in chunks of {seq_length}")
    return lm["train"].with_format("torch")
