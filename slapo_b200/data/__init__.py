"""Input pipeline: fixed-length token chunks, data-parallel sampling, pinned
host buffers and copies on a side stream.

The reference tokenises a Hugging Face dataset, concatenates it and cuts it
into ``seq_len`` chunks behind a ``DistributedSampler``
(examples/data_util.py:25-137).  Here the same three steps work from token
arrays (no downloads): ``pack_documents`` / ``TokenFileDataset`` make the
chunks, ``build_dataloader`` shards them over the data-parallel ranks of a
mesh, ``DevicePrefetcher`` keeps the next batch's host-to-device copy in
flight on its own CUDA stream while the current step computes.
"""
from .loader import (DevicePrefetcher, SyntheticDataset, TokenFileDataset,  # noqa: F401
                     build_dataloader, pack_documents)
