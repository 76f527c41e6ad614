"""fp16 loss scaling of the native engine: the scaled backward gives the same update as an
unscaled one, an overflow skips the step and halves the scale, clean steps grow it back, the
DeepSpeed ``fp16`` block configures it, and the scale travels with the optimizer state.

Parity: the reference trains fp16 models through DeepSpeed's dynamic loss scaler
(``"fp16": {"enabled": true, "initial_scale_power": 12}``, examples/utils.py:33-47 of the
reference); here the engine does it."""
import copy

import pytest
import torch
from torch import nn

from slapo_b200.runtime.engine import EngineConfig, TrainEngine


def _net():
    torch.manual_seed(5)
    return nn.Sequential(nn.Linear(8, 16), nn.GELU(), nn.Linear(16, 4))


def _loss(out, labels):
    return nn.functional.mse_loss(out, labels)


def test_static_scale_gives_the_unscaled_update():
    x, y = torch.randn(6, 8), torch.randn(6, 4)
    plain = TrainEngine(_net(), {"lr": 1e-2, "clip_grad": 0.5}, loss_fn=_loss)
    scaled = TrainEngine(_net(), {"lr": 1e-2, "clip_grad": 0.5, "loss_scale": 1024.0},
                         loss_fn=_loss)
    assert scaled.scaling and not scaled.dynamic_scale and not plain.scaling
    for _ in range(3):
        a = plain.train_batch(x, labels=y)
        b = scaled.train_batch(x, labels=y)
        torch.testing.assert_close(a, b)            # the reported loss is the unscaled one
    torch.testing.assert_close(scaled.last_grad_norm, plain.last_grad_norm, rtol=1e-5, atol=1e-7)
    for p, q in zip(plain.model.parameters(), scaled.model.parameters()):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def test_overflow_skips_the_step_and_halves_the_scale():
    x, y = torch.randn(6, 8), torch.randn(6, 4)
    eng = TrainEngine(_net(), {"lr": 1e-2, "clip_grad": 0.0, "loss_scale": 0,
                               "initial_scale_power": 4, "loss_scale_window": 2,
                               "min_loss_scale": 4.0}, loss_fn=_loss)
    assert eng.dynamic_scale and eng.loss_scale == 16.0
    before = copy.deepcopy(eng.model.state_dict())
    bad = x.clone()
    bad[0, 0] = float("inf")
    eng.train_batch(bad, labels=y)
    assert eng.loss_scale == 8.0 and eng.step_count == 0 and eng.skipped_steps == 1
    for k, v in eng.model.state_dict().items():
        torch.testing.assert_close(v, before[k])                 # nothing moved
    assert float(eng.flat_grad.abs().sum()) == 0.0               # and nothing is left behind
    eng.train_batch(bad, labels=y)
    eng.train_batch(bad, labels=y)
    assert eng.loss_scale == 4.0                                 # never below the floor
    eng.train_batch(x, labels=y)
    assert eng.step_count == 1 and eng.loss_scale == 4.0
    eng.train_batch(x, labels=y)
    assert eng.step_count == 2 and eng.loss_scale == 8.0         # two clean steps: doubled
    state = eng.optimizer_state()
    other = TrainEngine(_net(), {"loss_scale": 0}, loss_fn=_loss)
    other.load_optimizer_state(state)
    assert other.loss_scale == 8.0 and other.step_count == 2


def test_deepspeed_fp16_block_and_dtype_default():
    cfg = EngineConfig.from_dict({"fp16": {"enabled": True, "initial_scale_power": 12,
                                           "loss_scale_window": 500},
                                  "gradient_clipping": 1.0})
    assert cfg.initial_scale_power == 12 and cfg.loss_scale_window == 500 and cfg.clip_grad == 1.0
    assert "fp16" not in cfg.extra
    half = TrainEngine(_net().half(), cfg, loss_fn=_loss)
    assert half.dynamic_scale and half.loss_scale == 4096.0      # fp16 parameters: on by default
    full = TrainEngine(_net(), cfg, loss_fn=_loss)
    assert not full.scaling and full.loss_scale == 1.0           # other dtypes: off


def _pp_worker(rank, world):
    """Two stages, static scale: same losses as without scaling, and an overflow on the last
    stage is seen by the first one (one norm for the whole model)."""
    from test_train_equivalence_cpu import _tiny_spec

    import slapo_b200 as slapo
    from slapo_b200.parallel.mesh import DeviceMesh

    losses = {}
    for scale in (None, 256.0):
        torch.manual_seed(21)
        spec = _tiny_spec("gpt-neo-125m")
        model = spec.build().init_weights()
        mesh = DeviceMesh(pp=2, dp=1, tp=1)
        sch = slapo.model_schedule.apply_schedule(
            model, spec.schedule_key, model_config=spec.config, group=mesh.schedule_group,
            attn_op_name="reference", pipeline_cuts=[1])
        engine, _ = slapo.build(
            sch, target="native", mesh=mesh, init_weights=False, num_micro_batches=2,
            loss_fn=spec.loss_fn(None, False),
            config={"lr": 1e-2, "clip_grad": 1.0, "weight_decay": 0.0, "loss_scale": scale})
        inputs, labels = spec.make_batch(4, seq=32, seed=3)
        losses[scale] = [float(engine.train_batch(*inputs, labels=labels)) for _ in range(3)]
        if scale is not None:
            # an absurd scale overflows the last stage's fp32 gradients: both stages skip
            engine.inner.loss_scale, engine.inner.dynamic_scale = 1e38, True
            count = engine.inner.step_count
            engine.train_batch(*inputs, labels=labels)
            assert engine.inner.step_count == count and engine.inner.skipped_steps == 1
            assert engine.inner.loss_scale == 5e37
    assert losses[None] == pytest.approx(losses[256.0], rel=1e-4)


def test_pipeline_stages_scale_and_skip_together():
    from dist_utils import run_distributed

    run_distributed(_pp_worker, 2)


def test_fused_data_parallel_path_is_decided_after_the_loss_scale(monkeypatch):
    """The choice between the peer-memory and the NCCL data-parallel path is made while the
    flat buffers are built and reads the scaling state: it must exist by then.  (On a CPU
    the decision returns early; here it is replayed as on a CUDA device with two replicas.)"""
    from types import SimpleNamespace

    from slapo_b200.runtime import engine as engine_mod

    calls = []
    real = TrainEngine._want_fused_dp

    def spy(self):
        calls.append(hasattr(self, "scaling"))
        return real(self)

    monkeypatch.setattr(TrainEngine, "_want_fused_dp", spy)
    eng = TrainEngine(_net().half(), {"loss_scale": 0}, loss_fn=_loss)
    assert calls and all(calls)
    monkeypatch.setattr(TrainEngine, "_want_fused_dp", real)
    monkeypatch.setattr(engine_mod.native, "available", lambda: True)
    eng.device, eng.dp_size = SimpleNamespace(type="cuda"), 2
    assert eng.scaling and eng._want_fused_dp() is False          # fp16: NCCL path
    plain = TrainEngine(_net().bfloat16(), None, loss_fn=_loss)
    plain.device, plain.dp_size = SimpleNamespace(type="cuda"), 2
    assert not plain.scaling
    assert plain._want_fused_dp() == hasattr(torch.ops.slapo_b200, "dp_grad_rs")
