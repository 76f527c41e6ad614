"""Text file -> token chunks -> data-parallel loaders, with no download and no tokenizer
package: bytes are the tokens (ids 0 .. 255, 256 = end of document).

Parity: examples/data_util.py of the reference (Hugging Face dataset + tokenizer, concatenation
into fixed-length chunks, ``DistributedSampler`` loaders); the steps are the same, the source is
a local file.
"""
from __future__ import annotations

import os
import sys

import torch
from torch.utils.data import Dataset

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from slapo_b200.data import DevicePrefetcher, build_dataloader, pack_documents  # noqa: E402

BYTE_VOCAB = 257      # 256 byte values + end of document
EOS = 256


def read_documents(path, min_chars=1):
    """Paragraphs (blank-line separated) of a UTF-8 text file as lists of byte ids."""
    with open(path, "rb") as fh:
        raw = fh.read()
    docs = [list(part.strip()) for part in raw.split(b"\n\n")]
    return [d for d in docs if len(d) >= min_chars]


class ChunkDataset(Dataset):
    """Rows of ``seq_len`` tokens; ``kind="causal"``: labels = inputs (the model shifts them),
    ``kind="mlm"``: 15 % of the positions keep their token as label, the rest is -100."""

    def __init__(self, rows, kind="causal", mlm_prob=0.15, seed=0):
        self.rows, self.kind, self.mlm_prob, self.seed = rows, kind, mlm_prob, seed

    def __len__(self):
        return self.rows.shape[0]

    def __getitem__(self, idx):
        ids = self.rows[idx]
        if self.kind == "causal":
            return ids, ids.clone()
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        labels = torch.full_like(ids, -100)
        pick = torch.rand(ids.shape[0], generator=g) < self.mlm_prob
        labels[pick] = ids[pick]
        return ids, labels


def get_dataloaders(path, seq_len, micro_batch_size, mesh=None, kind="causal", val_fraction=0.1,
                    seed=0, device=None):
    """(train loader, validation loader, train sampler): every data-parallel replica of ``mesh``
    reads its own share, tensor- / pipeline-parallel ranks of a replica read the same rows.
    With ``device`` the loaders prefetch onto it on a side stream."""
    rows = pack_documents(read_documents(path), seq_len, eos_id=EOS)
    if rows.shape[0] < 2:
        raise ValueError(f"{path} holds {rows.shape[0]} rows of {seq_len} tokens; need at least 2")
    n_val = max(1, int(rows.shape[0] * val_fraction))
    train, val = rows[:-n_val], rows[-n_val:]
    t_loader, sampler = build_dataloader(ChunkDataset(train, kind, seed=seed), micro_batch_size,
                                         mesh=mesh, shuffle=True, seed=seed)
    v_loader, _ = build_dataloader(ChunkDataset(val, kind, seed=seed + 1), micro_batch_size,
                                   mesh=mesh, shuffle=False, drop_last=False)
    if device is not None:
        t_loader, v_loader = DevicePrefetcher(t_loader, device), DevicePrefetcher(v_loader, device)
    return t_loader, v_loader, sampler


class LossTestDataset(Dataset):
    """``fn(entry)`` applied to every entry of ``dataset`` on access (the wrapper the
    reference's scripts put around a tokenised dataset, examples/data_util.py:13-24 there)."""

    def __init__(self, dataset, fn):
        self.dataset, self.fn = dataset, fn

    def __len__(self):
        return len(self.dataset)

    def __getitem__(self, index):
        return self.fn(self.dataset[index])


def get_dataloader(model_name, dataset_name, micro_batch_size, enable_pipeline=False,
                   cache_dir=None, mpu=None, max_seq_length=1024):
    """``(train loader, validation loader)`` under the call the reference's scripts make
    (examples/data_util.py:27-68 there).  ``dataset_name`` is the path of a local text file
    (nothing is downloaded: bytes are the tokens); ``model_name`` picks the objective (masked
    language modelling for the BERT family, next-token prediction otherwise); ``mpu`` is the
    :class:`DeviceMesh` that tells which rows this data-parallel replica reads.  ``cache_dir``
    and ``enable_pipeline`` are accepted for compatibility: batches are ``[input_ids, labels]``
    in both cases (``engine.train_batch(input_ids, labels=labels)``)."""
    del cache_dir, enable_pipeline
    kind = "mlm" if any(k in model_name.lower() for k in ("bert", "roberta", "albert")) else "causal"
    train, val, _ = get_dataloaders(dataset_name, max_seq_length, micro_batch_size, mesh=mpu,
                                    kind=kind)
    return train, val
