"""shard / sync on two gloo ranks: column+row parallel MLP, attribute fix-ups,
tied weights, hook ordering, validation errors, every sync op's numerics and
the nine reshard schemes with their backward."""
import copy

import pytest
import torch
from torch import nn

import slapo_b200 as slapo
from slapo_b200.parallel import reshard_ops, sync_ops

from dist_utils import run_distributed


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(16, 32)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(32, 16)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


def _mlp_worker(rank, world):
    torch.manual_seed(0)
    ref = MLP()
    x = torch.randn(4, 16, requires_grad=True)
    y_ref = ref(x)
    y_ref.sum().backward()
    gx_ref = x.grad.clone()
    x.grad = None

    sch = slapo.create_schedule(copy.deepcopy(ref))
    sch["fc1"].shard("weight", axis=0)
    sch["fc1"].shard("bias", axis=0)
    sch["fc1"].sync("bwd_post", "all_reduce")
    sch["fc2"].shard("weight", axis=1)
    sch["fc2"].sync("fwd_post", "all_reduce")
    model, _ = slapo.build(sch, init_weights=False)
    assert model.fc1.out_features == 16 and model.fc2.in_features == 16
    assert model.fc1.weight.shape == (16, 16) and model.fc2.weight.shape == (16, 16)
    torch.testing.assert_close(model.fc1.weight, ref.fc1.weight.chunk(world)[rank])
    y = model(x)
    torch.testing.assert_close(y, y_ref, rtol=1e-5, atol=1e-5)   # bias added once
    y.sum().backward()
    torch.testing.assert_close(x.grad, gx_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(model.fc2.weight.grad, ref.fc2.weight.grad.chunk(world, 1)[rank],
                               rtol=1e-5, atol=1e-5)
    assert getattr(model.fc1.weight, "orig_shape", None) == (32, 16)


def test_column_row_parallel_mlp():
    run_distributed(_mlp_worker, 2)


def _validation_worker(rank, world):
    sch = slapo.create_schedule(MLP())
    sch["fc1"].shard("weight", axis=0)
    with pytest.raises(Exception):   # column-parallel output is a partition: no all_reduce
        sch["fc1"].sync("fwd_post", "all_reduce")
    with pytest.raises(Exception):   # conflicting second shard
        sch["fc1"].shard("weight", axis=1)
    sch["fc2"].shard("weight", axis=1)
    with pytest.raises(Exception):   # partial sums cannot be all-gathered
        sch["fc2"].sync("fwd_post", "all_gather", axis=1)
    with pytest.raises(Exception):
        sch["fc2"].sync("fwd_pre", "all_gather", axis=1)
    with pytest.raises(Exception):
        sch["fc2"].sync("no_such_mode", "all_reduce")
    with pytest.raises(Exception):
        sch["act"].shard("weight", axis=0)      # no such parameter
    odd = slapo.create_schedule(nn.Linear(16, 15))
    with pytest.raises(Exception):
        odd.shard("weight", axis=0)             # 15 rows over 2 ranks


def test_shard_sync_validation():
    run_distributed(_validation_worker, 2)


class Tied(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(32, 8)
        self.head = nn.Linear(8, 32, bias=False)
        self.head.weight = self.emb.weight

    def forward(self, ids):
        return self.head(self.emb(ids))


def _tied_worker(rank, world):
    sch = slapo.create_schedule(Tied())
    sch["emb"].shard("weight", axis=0)
    sch["head"].shard("weight", axis=0)
    assert sch.mod.emb.weight is sch.mod.head.weight
    assert sch.mod.emb.weight.shape == (16, 8)
    assert sch.mod.emb.num_embeddings == 16 and sch.mod.head.out_features == 16


def test_shard_tied_weights_share_new_parameter():
    run_distributed(_tied_worker, 2)


def _hook_order_worker(rank, world):
    order = []
    lin = nn.Linear(4, 4)
    sch = slapo.create_schedule(lin)

    def first(module, inputs):
        order.append("custom")
        return inputs

    sch.sync("fwd_pre", first)
    sch.sync("fwd_pre", "all_gather", axis=0)
    x = torch.full((2, 4), float(rank))
    out = sch.mod(x)
    assert order == ["custom"]
    assert out.shape == (2 * world, 4)      # gathered along axis 0 after the custom hook


def test_sync_hooks_run_in_registration_order():
    run_distributed(_hook_order_worker, 2)


def _sync_ops_worker(rank, world):
    full = torch.arange(8.0).reshape(2, 4)
    # all_gather of per-rank column shards rebuilds the full tensor; the backward
    # hands each rank its slice of the gradient (x world when grads are replicas)
    shard = full.chunk(world, 1)[rank].clone().requires_grad_(True)
    out = sync_ops.all_gather_forward_output(shard, 1, None)
    torch.testing.assert_close(out, full)
    out.backward(torch.ones_like(out) * (rank + 1))
    torch.testing.assert_close(shard.grad, torch.full((2, 2), float(sum(range(1, world + 1)))))
    shard.grad = None
    out = sync_ops.all_gather_forward_output(shard, 1, None, tensor_parallel_output_grad=False)
    out.backward(torch.ones_like(out) * (rank + 1))
    torch.testing.assert_close(shard.grad, torch.full((2, 2), float(rank + 1)))

    # reduce_scatter: sum over ranks, keep own slice; backward all-gathers
    x = (full * (rank + 1)).requires_grad_(True)
    out = sync_ops.reduce_scatter_forward_output(x, 1, None)
    torch.testing.assert_close(out, (full * 3).chunk(world, 1)[rank])
    out.backward(torch.full_like(out, float(rank + 1)))
    want = torch.cat([torch.full((2, 2), 1.0), torch.full((2, 2), 2.0)], 1)
    torch.testing.assert_close(x.grad, want)

    # scatter: keep own slice; backward all-gathers the slices of the gradient
    x = full.clone().requires_grad_(True)
    out = sync_ops.scatter_forward_output(x, 0, None)
    torch.testing.assert_close(out, full.chunk(world, 0)[rank])
    out.backward(torch.full_like(out, float(rank + 1)))
    torch.testing.assert_close(x.grad, torch.tensor([[1.0] * 4, [2.0] * 4]))

    # all_reduce forward / identity backward, and the mirror image
    x = (full * (rank + 1)).requires_grad_(True)
    out = sync_ops.reduce_forward_output(x, None)
    torch.testing.assert_close(out, full * 3)
    out.backward(torch.ones_like(out))
    torch.testing.assert_close(x.grad, torch.ones_like(full))
    x = full.clone().requires_grad_(True)
    out = sync_ops.reduce_backward_grad(x, None)
    torch.testing.assert_close(out, full)
    out.backward(torch.full_like(out, float(rank + 1)))
    torch.testing.assert_close(x.grad, torch.full_like(full, 3.0))


def test_sync_op_numerics():
    run_distributed(_sync_ops_worker, 2)


def _reshard_worker(rank, world):
    torch.manual_seed(1)
    full = torch.randn(2, 4, 6)         # [batch, seq, hidden]: "S" on seq (axis 1) or hidden (axis -1)
    seq_shard = full.chunk(world, 1)[rank]
    hid_shard = full.chunk(world, 2)[rank]
    cases = {
        "RR->RS": (full, hid_shard), "RR->SR": (full, seq_shard),
        "RS->RR": (hid_shard, full), "SR->RR": (seq_shard, full),
        "RS->SR": (hid_shard, seq_shard), "SR->RS": (seq_shard, hid_shard),
        "RR->RR": (full, full), "RS->RS": (hid_shard, hid_shard), "SR->SR": (seq_shard, seq_shard),
    }
    for scheme, (src, want) in cases.items():
        x = src.clone().requires_grad_(True)
        out = reshard_ops.reshard(scheme, x, None)
        torch.testing.assert_close(out, want, msg=scheme)
        # the backward is the inverse layout change of the gradient
        g = torch.randn(2, 4, 6)
        g_out = {"R": g, "RS": g.chunk(world, 2)[rank], "SR": g.chunk(world, 1)[rank]}[
            scheme.split("->")[1].replace("RR", "R")]
        out.backward(g_out.contiguous())
        src_kind = scheme.split("->")[0]
        if src_kind == "RR":
            # every rank holds a replica: gradients of the sliced copies are gathered
            want_g = g if scheme != "RR->RR" else g
        elif src_kind == "RS":
            want_g = g.chunk(world, 2)[rank]
        else:
            want_g = g.chunk(world, 1)[rank]
        torch.testing.assert_close(x.grad, want_g, msg=scheme + " backward")
    with pytest.raises(Exception):
        reshard_ops.reshard("SS->RR", full, None)


def test_reshard_schemes():
    run_distributed(_reshard_worker, 2)


def _sync_string_reshard_worker(rank, world):
    lin = nn.Linear(6, 6)
    sch = slapo.create_schedule(lin)
    sch.sync("fwd_post", "RR->SR")
    out = sch.mod(torch.randn(2, 4, 6))
    assert out.shape == (2, 4 // world, 6)


def test_sync_accepts_reshard_strings():
    run_distributed(_sync_string_reshard_worker, 2)
