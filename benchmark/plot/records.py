"""Readers shared by the plotting scripts: benchmark records come as JSON lines (one object per
line: the line ``bench.py`` prints, or the record of ``python -m slapo_b200.bench.train``), as the
TSV of ``bench_single_node.py sweep``, or as the JSON database of the auto-tuner."""
from __future__ import annotations

import json


def _norm(rec):
    """One flat record: model, impl, gpus, layout, samples_per_sec."""
    if "metric" in rec:            # bench.py
        cfg = rec.get("config", {})
        return {"model": cfg.get("model", "?"), "impl": rec.get("impl", "native"),
                "gpus": int(rec.get("n_gpus", 1)), "layout": cfg.get("parallelism", ""),
                "samples_per_sec": float(rec.get("value") or 0.0), "label": rec.get("label", "")}
    if "samples_per_sec" in rec:   # bench/train.py, sweep rows
        gpus = rec.get("gpus")
        if gpus is None:
            gpus = int(rec.get("tp", 1)) * int(rec.get("pp", 1)) * int(rec.get("dp", 1))
        layout = rec.get("layout") or "tp{tp}pp{pp}dp{dp}".format(
            tp=rec.get("tp", 1), pp=rec.get("pp", 1), dp=rec.get("dp", 1))
        try:
            thr = float(rec["samples_per_sec"])
        except (TypeError, ValueError):      # "oom" / "fail"
            thr = 0.0
        return {"model": rec.get("model", "?"), "impl": rec.get("impl", "native"), "gpus": int(gpus),
                "layout": layout, "samples_per_sec": thr, "label": rec.get("label", "")}
    return None


def read_records(path):
    """Records of a ``.jsonl`` / ``.log`` (lines that are not JSON objects are skipped) or ``.tsv``."""
    out = []
    with open(path, encoding="utf-8") as fh:
        if path.endswith(".tsv"):
            header = fh.readline().rstrip("\n").split("\t")
            for line in fh:
                cells = line.rstrip("\n").split("\t")
                if len(cells) == len(header):
                    rec = _norm(dict(zip(header, cells)))
                    if rec:
                        out.append(rec)
            return out
        for line in fh:
            line = line.strip()
            if not line.startswith("{"):
                continue
            try:
                rec = _norm(json.loads(line))
            except json.JSONDecodeError:
                continue
            if rec:
                out.append(rec)
    return out


def read_tuner_db(path):
    """[(cfg dict, samples/s, error code)] in the order the tuner visited the points."""
    with open(path, encoding="utf-8") as fh:
        db = json.load(fh)
    out = []
    for key, val in db.items():
        cfg = {}
        for part in key.strip("() ").split(","):      # "(batch_size: 8, ckpt_ratio: 0.5)"
            if ":" in part:
                k, v = (x.strip() for x in part.split(":", 1))
                try:
                    cfg[k] = float(v) if "." in v else int(v)
                except ValueError:
                    cfg[k] = v
        out.append((cfg, float(val.get("thrpt") or 0.0), int(val.get("error_code", 0))))
    return out
