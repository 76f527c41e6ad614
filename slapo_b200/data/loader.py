"""Datasets, sampler wiring and the device prefetcher (see the package docstring)."""
from __future__ import annotations

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, DistributedSampler


def pack_documents(documents, seq_len, eos_id=None, drop_remainder=True):
    """Concatenate token lists (``eos_id`` between documents) and cut the
    stream into rows of ``seq_len`` tokens: ``[n_rows, seq_len]`` int64."""
    stream = []
    for doc in documents:
        stream.extend(int(t) for t in doc)
        if eos_id is not None:
            stream.append(int(eos_id))
    n_rows = len(stream) // seq_len
    if not drop_remainder and len(stream) % seq_len:
        pad = (n_rows + 1) * seq_len - len(stream)
        stream.extend([eos_id if eos_id is not None else 0] * pad)
        n_rows += 1
    return torch.tensor(stream[:n_rows * seq_len], dtype=torch.long).view(n_rows, seq_len)


class TokenFileDataset(Dataset):
    """Rows of ``seq_len`` tokens from a flat binary token file (memory-mapped,
    ``uint16`` or ``int32``).  ``kind``: ``"causal"`` -> ``(ids, ids)``,
    ``"mlm"`` -> ``(ids, labels)`` with 15 % of the positions kept as labels."""

    def __init__(self, path, seq_len, dtype="uint16", kind="causal", mlm_prob=0.15, seed=0):
        self.tokens = np.memmap(path, dtype=np.dtype(dtype), mode="r")
        self.seq_len = seq_len
        self.kind, self.mlm_prob, self.seed = kind, mlm_prob, seed
        self.n = len(self.tokens) // seq_len

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        lo = idx * self.seq_len
        ids = torch.from_numpy(self.tokens[lo:lo + self.seq_len].astype(np.int64))
        if self.kind == "causal":
            return ids, ids.clone()
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        labels = torch.full_like(ids, -100)
        pick = torch.rand(self.seq_len, generator=g) < self.mlm_prob
        labels[pick] = ids[pick]
        return ids, labels


class SyntheticDataset(Dataset):
    """Deterministic random samples of a model spec's benchmark shape."""

    def __init__(self, spec, size, seq=None, seq_dec=None, seed=0):
        self.spec, self.size, self.seq, self.seq_dec, self.seed = spec, size, seq, seq_dec, seed

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        inputs, labels = self.spec.make_batch(1, self.seq, self.seq_dec, seed=self.seed + idx)
        return tuple(t[0] for t in inputs) + (labels[0],)


def build_dataloader(dataset, micro_batch_size, mesh=None, dp_rank=None, dp_size=None,
                     shuffle=True, seed=0, drop_last=True, num_workers=0, pin_memory=None):
    """``DataLoader`` whose sampler gives every data-parallel replica its own
    share; tensor- and pipeline-parallel ranks of one replica see the same
    samples (their ``dp_rank`` is equal).  Returns ``(loader, sampler)`` - call
    ``sampler.set_epoch(e)`` at the start of every epoch."""
    if mesh is not None:
        dp_rank, dp_size = mesh.dp_rank, mesh.dp_size
    dp_rank = 0 if dp_rank is None else dp_rank
    dp_size = 1 if dp_size is None else dp_size
    sampler = DistributedSampler(dataset, num_replicas=dp_size, rank=dp_rank, shuffle=shuffle,
                                 seed=seed, drop_last=drop_last)
    if pin_memory is None:
        pin_memory = torch.cuda.is_available()
    loader = DataLoader(dataset, batch_size=micro_batch_size, sampler=sampler,
                        num_workers=num_workers, pin_memory=pin_memory, drop_last=drop_last)
    return loader, sampler


class DevicePrefetcher:
    """Iterates a loader one batch ahead: the next batch is copied from pinned
    host memory on a side stream while the caller computes on the current
    one.  On CPU it is a plain pass-through."""

    def __init__(self, loader, device):
        self.loader = loader
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def _move(self, batch):
        if self.stream is None:
            return batch
        with torch.cuda.stream(self.stream):
            return tuple(t.to(self.device, non_blocking=True) if torch.is_tensor(t) else t
                         for t in batch)

    def __len__(self):
        return len(self.loader)

    def __iter__(self):
        it = iter(self.loader)
        try:
            nxt = self._move(tuple(next(it)))
        except StopIteration:
            return
        while nxt is not None:
            if self.stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self.stream)
                for t in nxt:
                    if torch.is_tensor(t):
                        t.record_stream(torch.cuda.current_stream(self.device))
            cur = nxt
            try:
                nxt = self._move(tuple(next(it)))
            except StopIteration:
                nxt = None
            yield cur
