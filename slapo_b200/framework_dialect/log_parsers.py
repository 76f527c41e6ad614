"""Training-log parsers used by the auto-tuner.

Every parser returns ``(param_per_gpu_M, samples_per_sec, gpu_mem_MB,
error_code)`` with error code 0 = ok, 1 = out of memory, 2 = failed.  The
``native`` parser reads the one-line JSON records this framework's engine
and ``bench.py`` print; the ``deepspeed`` / ``megatron`` parsers read those
tools' log formats.

Parity: slapo/framework_dialect/deepspeed/utils.py:9-46 and
megatron/utils.py:9-65 of the reference.
"""
from __future__ import annotations

import json
import re

from .registry import register_framework_dialect


def _read(log_file):
    with open(log_file, "r", errors="replace") as fh:
        return fh.read()


def _failure_code(text):
    if "CUDA out of memory" in text or "OutOfMemoryError" in text:
        return 1
    return 2


@register_framework_dialect("native", "log_parser")
class NativeLogParser:
    @staticmethod
    def parse_log(log_file):
        text = _read(log_file)
        samples, mem, params = [], 0.0, 0.0
        for line in text.splitlines():
            line = line.strip()
            if not (line.startswith("{") and line.endswith("}")):
                continue
            try:
                rec = json.loads(line)
            except json.JSONDecodeError:
                continue
            if "samples_per_sec" in rec:
                samples.append(float(rec["samples_per_sec"]))
            elif rec.get("unit") == "samples/s" and "value" in rec:
                samples.append(float(rec["value"]))
            mem = max(mem, float(rec.get("max_mem_mb", 0.0)))
            params = float(rec.get("param_per_gpu_m", params))
        if not samples:
            return params, 0.0, mem, _failure_code(text)
        if len(samples) > 2:
            samples = samples[1:]  # first record includes warm-up
        return params, sum(samples) / len(samples), mem, 0


@register_framework_dialect("deepspeed", "log_parser")
class DeepSpeedLogParser:
    @staticmethod
    def parse_log(log_file):
        text = _read(log_file)
        thr = [float(x) for x in re.findall(r"SamplesPerSec=([\d.]+)", text)]
        mems = [float(x) for x in re.findall(r"MaxMemAllocated=([\d.]+)\s*GB", text)]
        params = re.findall(r"param(?:eter)?s? per gpu[^\d]*([\d.]+)", text, re.I)
        param = float(params[-1]) if params else 0.0
        if not thr:
            return param, 0.0, 0.0, _failure_code(text)
        if len(thr) > 2:
            thr = thr[1:]
        return param, sum(thr) / len(thr), (max(mems) * 1024 if mems else 0.0), 0


@register_framework_dialect("megatron", "log_parser")
class MegatronLogParser:
    @staticmethod
    def parse_log(log_file):
        text = _read(log_file)
        times = [float(x) for x in re.findall(r"elapsed time per iteration \(ms\):\s*([\d.]+)", text)]
        batch = re.findall(r"global batch size:\s*(\d+)", text)
        mems = [float(x) for x in re.findall(r"max allocated:\s*([\d.]+)", text)]
        params = re.findall(r"number of parameters on \(tensor, pipeline\) model parallel rank "
                            r"\(0, 0\):\s*(\d+)", text)
        param = float(params[-1]) / 1e6 if params else 0.0
        if not times or not batch:
            return param, 0.0, 0.0, _failure_code(text)
        if len(times) > 1:
            times = times[1:]
        avg_ms = sum(times) / len(times)
        return param, int(batch[-1]) / (avg_ms / 1e3), (max(mems) if mems else 0.0), 0
