"""Input pipeline: packing, token files, data-parallel sharding, prefetcher."""
import numpy as np
import torch

from slapo_b200.data import (DevicePrefetcher, SyntheticDataset, TokenFileDataset,
                             build_dataloader, pack_documents)
from slapo_b200.models.zoo import get_model_spec


def test_pack_documents():
    rows = pack_documents([[1, 2, 3], [4, 5], [6, 7, 8, 9]], seq_len=4, eos_id=0)
    assert rows.tolist() == [[1, 2, 3, 0], [4, 5, 0, 6], [7, 8, 9, 0]]
    rows = pack_documents([[1, 2, 3, 4, 5]], seq_len=4, eos_id=None, drop_remainder=False)
    assert rows.shape == (2, 4) and rows[1].tolist() == [5, 0, 0, 0]


def test_token_file_dataset_and_dp_sharding(tmp_path):
    path = tmp_path / "tokens.bin"
    np.arange(0, 64 * 16, dtype=np.uint16).tofile(path)
    ds = TokenFileDataset(str(path), seq_len=16, kind="mlm", seed=3)
    assert len(ds) == 64
    ids, labels = ds[2]
    assert ids.tolist() == list(range(32, 48))
    kept = labels != -100
    assert torch.equal(labels[kept], ids[kept]) and 0 < kept.sum() < 16
    assert torch.equal(ds[2][1], labels)                       # deterministic masking
    seen = []
    for dp_rank in range(4):
        loader, sampler = build_dataloader(ds, 4, dp_rank=dp_rank, dp_size=4, seed=1,
                                           pin_memory=False)
        sampler.set_epoch(0)
        batches = list(loader)
        assert len(batches) == 4 and batches[0][0].shape == (4, 16)
        seen += [int(row[0]) for b in batches for row in b[0]]
    assert sorted(seen) == [16 * i for i in range(64)]         # a partition of the data set
    causal = TokenFileDataset(str(path), seq_len=16, kind="causal")
    assert torch.equal(*causal[5])


def test_synthetic_dataset_and_prefetcher():
    spec = get_model_spec("t5-base")
    ds = SyntheticDataset(spec, size=8, seq=12, seq_dec=6, seed=2)
    enc, dec, labels = ds[0]
    assert enc.shape == (12,) and dec.shape == (6,) and labels.shape == (6,)
    loader, _ = build_dataloader(ds, 2, shuffle=False, pin_memory=False)
    got = list(DevicePrefetcher(loader, "cpu"))
    assert len(got) == 4 and got[0][0].shape == (2, 12)
    assert torch.equal(got[0][0][0], enc)
