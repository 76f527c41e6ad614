"""Utilities: rank-filtered logger, env.execute, hook helpers, functional<->module mapping,
version helpers, memory / FLOP reports, init_empty_weights."""
import logging

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

import slapo_b200 as slapo
from slapo_b200 import env
from slapo_b200.utils import common, mapping, report, versions

from dist_utils import run_distributed


def _logger_worker(rank, world):
    records = []

    class Capture(logging.Handler):
        def emit(self, record):
            records.append(record.getMessage())

    logger = slapo.get_logger("unit-test-logger")
    logger.logger.addHandler(Capture())
    logger.info("everyone %d", 1)
    logger.info("only zero", ranks=0)
    logger.info("only one", ranks=[1])
    assert f"[Rank {rank}] everyone 1" in records
    assert (f"[Rank {rank}] only zero" in records) == (rank == 0)
    assert (f"[Rank {rank}] only one" in records) == (rank == 1)


def test_logger_filters_by_rank():
    run_distributed(_logger_worker, 2)
    assert slapo.get_logger("x") is slapo.get_logger("x")      # per-name singleton


def _env_fn(rank, world, path):
    env.setup(rank, world, backend="gloo", port=29588)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t)
    if rank == 0:
        with open(path, "w") as fh:
            fh.write(str(float(t)))
    env.cleanup()


def test_env_execute_spawns_a_world(tmp_path):
    out = tmp_path / "sum.txt"
    env.execute(_env_fn, args=(2, str(out)), world_size=2)
    assert out.read_text() == "3.0"


def test_hook_helpers():
    a, b = nn.Linear(2, 2), nn.Linear(2, 2)
    assert not common.has_hook(a, "fwd_pre")
    a.register_forward_pre_hook(lambda m, i: None)
    a.register_forward_hook(lambda m, i, o: None)
    assert common.has_hook(a, "fwd_pre") and common.has_hook(a, "fwd_post")
    assert not common.has_hook(a, "bwd_post")
    hooks = common.get_hooks(a)
    assert len(hooks["fwd_pre"]) == 1 and len(hooks["fwd_post"]) == 1
    common.transfer_hooks(a, b, ["fwd_pre"])
    assert common.has_hook(b, "fwd_pre") and not common.has_hook(b, "fwd_post")
    assert common.is_module_list(nn.ModuleList([a])) and not common.is_module_list(a)
    assert common.is_lambda_function(lambda: 0) and not common.is_lambda_function(test_hook_helpers)
    assert common.importlib_or_none("definitely_not_a_module") is None
    assert common.importlib_or_none("math") is not None


def test_functional_module_mapping():
    pairs = mapping.MAPPING_FROM_FUNCTIONAL_TO_MODULE
    assert pairs[F.relu] is nn.ReLU and pairs[F.layer_norm] is nn.LayerNorm
    assert pairs[F.linear] is nn.Linear and pairs[F.gelu] is nn.GELU
    assert len(pairs) >= 11


def test_versions_and_reports():
    assert versions.compare_versions("1.2.3", ">=", "1.2.0")
    assert not versions.compare_versions("1.2.3", "<", "1.0")
    assert versions.is_torch_version(">=", "2.0")
    mem = report.report_memory("unit test")
    assert mem["cpu_rss_mib"] > 0
    # 72 * B * s * L * h^2 * (1 + s/(6h) + V/(12hL)) per second, in TFLOP/s
    tf = report.calc_decoder_tflops(8, 1024, 24, 2048, 50257, elapsed_s=1.0)
    base = 72 * 8 * 1024 * 24 * 2048**2 / 1e12
    assert base < tf < base * 1.4
    assert report.calc_decoder_tflops(8, 1024, 24, 2048, 50257, 1.0, ckpt=True) > tf
    table = report.profile_perf(nn.Linear(4, 4), [torch.randn(2, 4)], backward=True)
    assert "aten::" in table


def test_init_empty_weights():
    with slapo.init_empty_weights():
        m = nn.Linear(1024, 1024)
        assert m.weight.is_meta
    assert not nn.Linear(2, 2).weight.is_meta
    with slapo.init_empty_weights(enable=False):
        assert not nn.Linear(2, 2).weight.is_meta
    with slapo.init_empty_weights(include_buffers=True):
        bn = nn.BatchNorm1d(4)
        assert bn.running_mean.is_meta


def test_profile_switch_annotates_modules_and_is_harmless_on_cpu():
    """``EngineConfig(profile=True)``: NVTX ranges are requested and the scheduled modules get
    range hooks; without CUDA everything stays a no-op and training is unchanged."""
    import copy

    import torch
    from torch import nn

    from slapo_b200.ops.linear import LinearWithSyncFunc
    from slapo_b200.runtime.engine import TrainEngine
    from slapo_b200.utils import nvtx

    torch.manual_seed(0)
    model = nn.Sequential(LinearWithSyncFunc(8, 8), nn.ReLU(), nn.Linear(8, 1))
    plain = TrainEngine(copy.deepcopy(model), config={"lr": 1e-2})
    prof = TrainEngine(model, config={"lr": 1e-2, "profile": True})
    assert getattr(model[0], "_slapo_nvtx", False) and not getattr(model[2], "_slapo_nvtx", False)
    assert nvtx.annotate_modules(model) == 0          # idempotent
    x = torch.randn(4, 8)
    a = plain.train_batch(x)
    b = prof.train_batch(x)
    torch.testing.assert_close(a, b)
    assert prof.phase_times() == {}                   # device timing needs CUDA
    with nvtx.range("anything"):
        pass
    nvtx.enable(False)
