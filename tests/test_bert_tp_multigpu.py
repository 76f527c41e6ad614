"""BERT through the native engine on 2 GPUs with the fused TP kernels: the
tensor+sequence-parallel model must track the single-GPU model (same weights,
same data) in loss and in the gathered output."""
import copy

import pytest
import torch

from dist_utils import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world, sequence_parallel):
    import torch.distributed as dist

    import slapo_b200 as slapo
    from slapo_b200.models import BertConfig, BertForMaskedLM, mlm_loss
    from slapo_b200.ops import native
    from slapo_b200.ops.linear import LinearWithSyncFunc

    dev = torch.device("cuda", rank)
    cfg = BertConfig(vocab_size=4096, hidden_size=256, num_hidden_layers=2,
                     num_attention_heads=4, intermediate_size=1024,
                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(11)
    ref = BertForMaskedLM(cfg).init_weights().to(dev).bfloat16()
    ids = torch.randint(0, cfg.vocab_size, (8, 128), device=dev)
    labels = ids.clone()
    labels[:, ::3] = -100
    # single-GPU model through the same kernels
    sch1 = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "bert", model_config=cfg,
                                               group=False)
    m1, _ = slapo.build(sch1, init_weights=False)
    loss1 = mlm_loss(m1(ids)["logits"], labels)
    # tensor parallel over both GPUs
    slapo.set_random_seed(3, tp_rank=rank, always_enable_tp_seed=sequence_parallel)
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "bert", model_config=cfg,
                                              sequence_parallel=sequence_parallel)
    engine, _ = slapo.build(sch, target="native", init_weights=False,
                            config={"lr": 1e-4, "clip_grad": 1.0},
                            loss_fn=lambda out, lab: mlm_loss(out["logits"], lab, None, True))
    fused = [m for m in engine.model.modules() if isinstance(m, LinearWithSyncFunc)
             and (m.fused_pre or m.fused_post or m.fused_bwd)]
    assert len(fused) >= 8, "the TP linears were not lowered to fused kernels"
    before = native.launch_count()
    loss_tp = mlm_loss(engine.model(ids)["logits"], labels, None, True)
    assert native.launch_count() > before
    torch.testing.assert_close(loss_tp.float(), loss1.float(), rtol=2e-2, atol=2e-2)
    losses = [float(engine.train_batch(ids, labels=labels)) for _ in range(4)]
    assert native.ops().device_status() == 0
    assert losses[-1] < losses[0], losses
    dist.barrier()


@pytest.mark.parametrize("sequence_parallel", [False, True])
def test_bert_tp2_fused_matches_single_gpu(sequence_parallel):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed(_worker, 2, sequence_parallel, backend="nccl")
