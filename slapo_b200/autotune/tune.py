"""Auto-tuner for schedule hyper-parameters (batch size x checkpoint ratio).

Pieces:

* ``Symbol`` / ``Space`` - a *dependent* search space: symbols are fixed one
  after the other and a user ``update_space_fn(args, space)`` may re-create
  the not-yet-fixed symbols whose candidates depend on the fixed ones;
  comparisons on a symbol are false until it is fixed.
* ``Database`` - JSON record of every evaluated point, rewritten on each
  commit so that a killed search can be inspected and resumed.
* ``tune`` - the search: evaluate the largest batch size; if it does not fit
  (throughput 0) binary-search the largest one that does; then for each batch
  size, largest first, binary-search the checkpoint ratio (the fraction of
  layers checkpointed: less = faster until memory runs out) reusing the
  previous position as the lower bound; stop after 5 evaluations in a row that do not
  improve the best throughput.
* evaluation - either a training *script* run as a subprocess with the
  symbols substituted textually into its arguments and exported as
  environment variables (its log is parsed by the target's ``log_parser``),
  or an in-process ``eval_fn(cfg) -> samples/s`` (no process start-up per
  point, which matters when a point takes seconds on a B200).

CLI: ``python -m slapo_b200.autotune.tune --config CFG.py [--db DB.json]
[--error-stop none|symbol|all] [--target native] TRAIN_SCRIPT [ARGS...]`` where
``CFG.py`` defines ``get_bs_range(args) -> (min, max, step)``.

Parity: slapo/autotune/tune.py:22-447 of the reference.
"""
from __future__ import annotations

import argparse
import copy
import importlib.util
import json
import os
import re
import shlex
import subprocess
import sys

from ..logger import get_logger

logger = get_logger("autotune")

CKPT_RATIOS = [1.0, 0.92, 0.84, 0.67, 0.5, 0.34, 0.25]
PATIENCE = 5


class Symbol:
    """A tunable name with candidate values; unusable in comparisons until fixed."""

    def __init__(self, name, vals):
        self.name = name
        self.vals = list(vals)
        self.fixed_idx = -1

    def is_fixed(self):
        return self.fixed_idx != -1

    @property
    def value(self):
        if not self.is_fixed():
            raise ValueError(f"symbol {self.name} is not fixed yet")
        return self.vals[self.fixed_idx]

    def fix_at(self, idx):
        if not 0 <= idx < len(self.vals):
            raise ValueError(f"cannot fix {self.name} ({len(self.vals)} values) at index {idx}")
        self.fixed_idx = idx

    def add(self, val):
        if val not in self.vals:
            self.vals.append(val)

    def __len__(self):
        return len(self.vals)

    def _cmp(self, other, op):
        return self.is_fixed() and op(self.value, other)

    def __gt__(self, other):
        return self._cmp(other, lambda a, b: a > b)

    def __ge__(self, other):
        return self._cmp(other, lambda a, b: a >= b)

    def __lt__(self, other):
        return self._cmp(other, lambda a, b: a < b)

    def __le__(self, other):
        return self._cmp(other, lambda a, b: a <= b)

    def __repr__(self):
        return f"Symbol({self.name}, {self.value if self.is_fixed() else self.vals})"


class Space:
    def __init__(self):
        self.space: dict[str, Symbol] = {}
        self.idx_to_name: list[str] = []
        self.fixed_idx = -1

    def create_symbol(self, name, vals):
        """New symbol, or - if it exists and is not fixed yet - the same name
        with new candidates (they may depend on symbols fixed meanwhile)."""
        if name in self.space and self.space[name].is_fixed():
            return self.space[name]
        if name not in self.space:
            self.idx_to_name.append(name)
        self.space[name] = Symbol(name, vals)
        return self.space[name]

    def next(self):
        if self.fixed_idx + 1 < len(self.space):
            self.fixed_idx += 1
            return self.space[self.idx_to_name[self.fixed_idx]]
        return None

    def reset(self):
        self.fixed_idx = -1
        for sym in self.space.values():
            sym.fixed_idx = -1

    def to_dict(self):
        return {sym.name: sym.value for sym in self.space.values()}

    def clone(self):
        return copy.deepcopy(self)

    @staticmethod
    def cfg_dict_to_str(cfg):
        return "(" + ", ".join(f"{k}: {v}" for k, v in cfg.items()) + ")"

    def enumerate(self, args, update_space_fn):
        """All complete assignments reachable under ``update_space_fn``."""
        out = []

        def rec(space):
            sym = space.next()
            if sym is None:
                out.append(space.to_dict())
                return
            for idx in range(len(sym.vals)):
                sym.fix_at(idx)
                nxt = update_space_fn(args, space) if update_space_fn else space
                rec(nxt.clone())

        rec(self.clone())
        return out

    def log_space(self, training_script_args, update_space_fn):
        points = self.enumerate(training_script_args, update_space_fn)
        logger.info("Enumerating the search space:")
        for p in points:
            logger.info("\t%s", self.cfg_dict_to_str(p))
        logger.info("Space size: %d", len(points))
        return len(points)

    def __repr__(self):
        rows = [f"\t{s.name}: {str(s.value) + ' (fixed)' if s.is_fixed() else s.vals}"
                for s in self.space.values()]
        return "Space(\n" + ",\n".join(rows) + ")"


class Database:
    def __init__(self, db_file_name=None):
        self.db_file_name = db_file_name
        self.db = {}

    def load(self):
        if self.db_file_name and os.path.exists(self.db_file_name):
            with open(self.db_file_name, "r", encoding="utf-8") as fh:
                self.db = json.load(fh)
            logger.info("loaded %d tuning records from %s", len(self.db), self.db_file_name)
        return self.db

    def commit(self, key, data):
        self.db[key] = data
        if self.db_file_name:
            tmp = self.db_file_name + ".tmp"
            with open(tmp, "w", encoding="utf-8") as fh:
                json.dump(self.db, fh, indent=2)
            os.replace(tmp, self.db_file_name)


# ---------------------------------------------------------------------- #
def convert_nargs_to_dict(nargs):
    """``["--a", "1", "--flag", "pos"]`` -> ``{"a": 1, "flag": 1, "pos": 1}``."""

    def infer(val):
        try:
            num = float(val)
        except ValueError:
            return val
        return int(num) if num == int(num) else num

    out, i = {}, 0
    nargs = list(nargs or [])
    while i < len(nargs):
        name = nargs[i]
        i += 1
        key = name.lstrip("-")
        if not name.startswith("-") or i == len(nargs) or nargs[i].startswith("-"):
            out[key] = 1
            continue
        vals = []
        while i < len(nargs) and not nargs[i].startswith("-"):
            vals.append(infer(nargs[i]))
            i += 1
        out[key] = vals[0] if len(vals) == 1 else vals
    return out


def tune(training_script_args, get_bs_range, eval_fn, tune_ckpt=True, is_valid=None,
         ckpt_ratios=None, patience=PATIENCE):
    """Search batch size then checkpoint ratio; returns ``(best_cfg, best_thrpt, trace)``.

    ``eval_fn(cfg) -> samples/s`` must return 0 for a point that fails (OOM)."""
    min_bs, max_bs, step = get_bs_range(training_script_args)
    bs_range = list(range(min_bs, max_bs + 1, step))
    ratios = list(ckpt_ratios or CKPT_RATIOS)
    state = {"stale": 0, "best": (None, -1.0)}
    trace = []

    def evaluate(cfg):
        valid = is_valid(cfg) if is_valid else True
        thr = float(eval_fn(dict(cfg))) if valid else 0.0
        trace.append((dict(cfg), thr))
        logger.info("- %s -> %.2f samples/s", Space.cfg_dict_to_str(cfg), thr)
        if thr > state["best"][1]:
            state["best"] = (dict(cfg), thr)
            state["stale"] = 0
        else:
            state["stale"] += 1
        return thr

    def bisect(values, cfg, key, lo=0, hi=None):
        """Largest index whose point runs (values are ordered from cheapest in
        memory to most expensive); None as throughput = stopped early."""
        hi = len(values) - 1 if hi is None else hi
        mid, thr = lo, 0.0
        while lo <= hi:
            mid = (lo + hi) // 2
            cfg[key] = values[mid]
            thr = evaluate(cfg)
            if thr < 0.01:
                hi = mid - 1
            else:
                lo = mid + 1
            if state["stale"] >= patience:
                return mid, None
        if thr < 0.01:
            mid -= 1
        return max(mid, 0), thr

    cfg = {"batch_size": max_bs, "ckpt_ratio": ratios[0]}
    thr = evaluate(cfg)
    pos = 0
    if thr == 0:  # the largest batch does not fit even with full checkpointing
        idx, thr = bisect(bs_range, cfg, "batch_size")
        max_bs = bs_range[idx]
    logger.info("largest batch size that runs with full checkpointing: %d", max_bs)
    if tune_ckpt:
        # the ratio is the fraction of layers that are checkpointed: 1.0
        # (index 0) needs the least memory and is slowest, so a larger index
        # is faster until it no longer fits.  A smaller batch can only afford
        # a larger index, hence the search resumes from the last position.
        for bs in reversed(bs_range):
            cfg["batch_size"] = bs
            pos, thr = bisect(ratios, cfg, "ckpt_ratio", lo=pos)
            if thr is None:
                break
    best_cfg, best_thr = state["best"]
    return best_cfg, best_thr, trace


# ---------------------------------------------------------------------- #
def load_config(config_file):
    spec = importlib.util.spec_from_file_location("slapo_tune_cfg", os.path.abspath(config_file))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    if not hasattr(module, "get_bs_range"):
        raise ValueError("the tuning config must define get_bs_range(args)")
    return module


def run_training_script(script, script_args, cfg, log_file="run_script.log", timeout=None):
    """Run ``python script args`` with symbols substituted and exported."""
    text = " ".join(script_args)
    for key, val in cfg.items():
        text = re.sub(rf"\b{re.escape(key)}\b", str(val), text)
    env = dict(os.environ)
    env.update({k: str(v) for k, v in cfg.items()})
    cmd = [sys.executable, script] + shlex.split(text)
    logger.info("\trunning: %s", " ".join(cmd))
    with open(log_file, "w", encoding="utf-8") as fh:
        try:
            subprocess.run(cmd, stdout=fh, stderr=subprocess.STDOUT, env=env, timeout=timeout,
                           check=False)
        except subprocess.TimeoutExpired:
            fh.write("\nTIMEOUT\n")
    return log_file


def parse_args(argv=None):
    parser = argparse.ArgumentParser("slapo_b200 auto-tuner")
    parser.add_argument("--config", required=True, help="python file defining get_bs_range(args)")
    parser.add_argument("--db", default=None, help="JSON file receiving every evaluated point")
    parser.add_argument("--error-stop", default="none", choices=["none", "symbol", "all"])
    parser.add_argument("--target", default="native",
                        help="log parser to use: native | deepspeed | megatron")
    parser.add_argument("--log-file", default=None,
                        help="log written by the training script (default: its stdout)")
    parser.add_argument("training_script")
    parser.add_argument("training_script_args", nargs=argparse.REMAINDER)
    return parser.parse_args(argv)


def main(argv=None):
    from ..framework_dialect import get_dialect_cls

    args = parse_args(argv)
    config = load_config(args.config)
    db = Database(args.db)
    db.load()
    parser = get_dialect_cls("log_parser", args.target)
    script_args = convert_nargs_to_dict(args.training_script_args)

    def eval_fn(cfg):
        key = Space.cfg_dict_to_str(cfg)
        if key in db.db and db.db[key].get("error_code") == 0:
            return db.db[key]["thrpt"]
        stdout_log = run_training_script(args.training_script, args.training_script_args, cfg)
        log_file = args.log_file or stdout_log
        _, thrpt, mem, code = parser.parse_log(log_file)
        with open(stdout_log, "r", encoding="utf-8", errors="replace") as fh:
            tail = fh.read()[-4000:]
        db.commit(key, {"error_code": code, "thrpt": thrpt, "mem_mb": mem, "log": tail})
        if args.error_stop == "all" and code != 0:
            raise RuntimeError(f"stop tuning: {key} failed with code {code}")
        return thrpt if code == 0 else 0.0

    is_valid = getattr(config, "is_valid", None)
    valid = (lambda cfg: is_valid(script_args, cfg)) if is_valid else None
    best, thr, _ = tune(script_args, config.get_bs_range, eval_fn, is_valid=valid,
                        tune_ckpt=getattr(config, "TUNE_CKPT", True))
    logger.info("best config: %s (%.2f samples/s)", best, thr)
    print(json.dumps({"best": best, "samples_per_sec": thr}))
    return best


if __name__ == "__main__":
    main()
