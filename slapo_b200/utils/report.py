"""Memory / performance reports and model-FLOPs calculators.

Parity: slapo/utils/report.py:17-108 and the per-sample FLOPs formula of
benchmark/bench_single_node.py:72-130 of the reference.
"""
from __future__ import annotations

import gc

import psutil
import torch

from ..logger import get_logger

logger = get_logger("report")


def report_memory(msg: str = "", report_gc: bool = False) -> dict:
    """Log and return host RSS and device peak memory (MiB)."""
    rss = psutil.Process().memory_info().rss / 2**20
    out = {"cpu_rss_mib": rss, "gpu_allocated_mib": 0.0, "gpu_peak_mib": 0.0}
    if torch.cuda.is_available():
        out["gpu_allocated_mib"] = torch.cuda.memory_allocated() / 2**20
        out["gpu_peak_mib"] = torch.cuda.max_memory_allocated() / 2**20
        torch.cuda.reset_peak_memory_stats()
    logger.info(
        "%s CPU RSS %.0f MiB | GPU allocated %.0f MiB peak %.0f MiB",
        msg, out["cpu_rss_mib"], out["gpu_allocated_mib"], out["gpu_peak_mib"],
    )
    if report_gc:
        count = 0
        for obj in gc.get_objects():
            try:
                if torch.is_tensor(obj):
                    count += 1
            except Exception:
                continue
        out["live_tensors"] = count
        logger.info("%s live tensors: %d", msg, count)
    return out


def profile_perf(model, inputs, backward: bool = False, row_limit: int = 25):
    """Run one step under ``torch.profiler`` and return the kernel table."""
    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(ProfilerActivity.CUDA)
    with profile(activities=acts, record_shapes=True) as prof:
        out = model(*inputs)
        if backward:
            first = out[0] if isinstance(out, (tuple, list)) else out
            if isinstance(first, dict):
                first = next(iter(first.values()))
            first.float().mean().backward()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    key = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
    table = prof.key_averages().table(sort_by=key, row_limit=row_limit)
    logger.info("\n%s", table)
    return table


def calc_decoder_tflops(batch, seq, layers, hidden, vocab, elapsed_s, n_gpus=1, ckpt=False):
    """Megatron-style model TFLOP/s per GPU for a decoder-only model."""
    factor = 96 if ckpt else 72
    flops = factor * batch * seq * layers * hidden**2 * (
        1 + seq / (6 * hidden) + vocab / (12 * hidden * layers)
    )
    return flops / elapsed_s / n_gpus / 1e12


def transformer_train_flops_per_sample(layers, hidden, seq, vocab, ffn=None):
    """fwd+bwd FLOPs of one sample: 3 x (L(4hs^2 + 8sh^2 + 4*s*h*ffn) + 2shv)."""
    ffn = 4 * hidden if ffn is None else ffn
    per_layer = 4 * hidden * seq**2 + 8 * seq * hidden**2 + 4 * seq * hidden * ffn
    return 3 * (layers * per_layer + 2 * seq * hidden * vocab)


def t5_train_flops_per_sample(enc_layers, dec_layers, d_model, d_attn, d_ff, enc_seq, dec_seq,
                              vocab, gated=False):
    """fwd+bwd FLOPs of one encoder-decoder sample."""
    def attn(sq, sk):
        proj = 2 * d_model * d_attn * (2 * sq + 2 * sk)
        return proj + 4 * sq * sk * d_attn

    n_in = 2 if gated else 1
    def ffn(s):
        return 2 * s * d_model * d_ff * (n_in + 1)

    enc = enc_layers * (attn(enc_seq, enc_seq) + ffn(enc_seq))
    dec = dec_layers * (attn(dec_seq, dec_seq) + attn(dec_seq, enc_seq) + ffn(dec_seq))
    head = 2 * dec_seq * d_model * vocab
    return 3 * (enc + dec + head)
