"""The whole training step replayed from one CUDA graph: same losses as the eager engine
(dropout off), step-dependent optimizer scalars read from device memory, dropout masks that
differ from replay to replay, activation checkpointing inside the captured step."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(dropout):
    import slapo_b200 as slapo
    from slapo_b200.models import BertConfig, BertForMaskedLM, mlm_loss

    cfg = BertConfig(vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                     intermediate_size=1024, hidden_dropout_prob=dropout,
                     attention_probs_dropout_prob=dropout)
    torch.manual_seed(0)
    slapo.set_random_seed(11)
    model = BertForMaskedLM(cfg).init_weights().cuda().bfloat16()
    sch = slapo.model_schedule.apply_schedule(model, "bert", model_config=cfg, group=False,
                                              ckpt_ratio=0.5)
    engine, _ = slapo.build(sch, target="native", init_weights=False,
                            config={"lr": 1e-3, "clip_grad": 1.0},
                            loss_fn=lambda out, lab: mlm_loss(out["logits"], lab))
    return engine


def _batch(seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1024, (8, 128), generator=g).cuda()
    labels = ids.clone()
    labels[:, ::2] = -100
    return ids, labels


def test_captured_step_matches_eager_engine():
    from slapo_b200.ops import native

    eager = _engine(0.0)
    graphed_engine = _engine(0.0)           # same seeds: identical weights
    ids, labels = _batch(0)
    graphed = graphed_engine.capture_step(ids, labels=labels, warmup=3)
    assert graphed.kernels_per_step > 20
    for _ in range(3):                      # the eager twin takes the same three warm-up steps
        eager.train_batch(ids, labels=labels)
    assert graphed_engine.step_count == eager.step_count == 3
    for step in range(5):
        ids, labels = _batch(step + 1)
        l_g = float(graphed(ids, labels=labels))
        l_e = float(eager.train_batch(ids, labels=labels))
        assert abs(l_g - l_e) < 2e-2 * max(1.0, abs(l_e)), (step, l_g, l_e)
    assert graphed_engine.step_count == eager.step_count == 8
    torch.testing.assert_close(graphed_engine.flat_param.float(), eager.flat_param.float(),
                               rtol=2e-2, atol=2e-2)
    assert native.ops().device_status() == 0


def test_captured_step_draws_fresh_dropout_masks_and_learns():
    engine = _engine(0.1)
    ids, labels = _batch(0)
    graphed = engine.capture_step(ids, labels=labels, warmup=3)
    losses = [float(graphed(ids, labels=labels)) for _ in range(12)]
    assert all(l == l for l in losses)                    # finite
    assert len({round(l, 5) for l in losses}) > 6         # not one frozen mask / frozen weights
    assert losses[-1] < losses[0]
