"""Schedule tree: paths, primitive registry, whole-module replace with hook
transfer, replace_all, annotations and tied-weight sharding (single rank)."""
import pytest
import torch
from torch import nn

import slapo_b200 as slapo


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(8, 16)
        self.act = nn.ReLU()
        self.fc2 = nn.Linear(16, 8)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = nn.ModuleList([Block() for _ in range(3)])
        self.seq = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return self.seq(x)


def test_paths_and_lookup():
    sch = slapo.create_schedule(Net())
    assert sch[""] is sch
    assert isinstance(sch["layers.0"].mod, Block)
    assert sch["layers.1.fc1"].mod is sch.mod.layers[1].fc1
    assert sch["layers.1"]["fc1"] is sch["layers.1.fc1"]
    # nn.Sequential: a normal child whose elements are reached either way
    assert sch["seq"]["0"].mod is sch.mod.seq[0]
    assert sch["seq.0"].mod is sch.mod.seq[0]
    assert "layers.2.fc2" in sch and "layers.3" not in sch and "nothing" not in sch
    with pytest.raises(KeyError):
        sch["layers.7"]
    assert sch["layers.0.fc1"].get_top_schedule() is sch
    assert sch["layers.0.fc1"].parent is sch["layers.0"]
    assert sch["layers.0.fc1"].path == "layers.0.fc1" and sch["layers.0.fc1"].name == "fc1"
    assert sch.get_module("layers.0.fc1") is sch.mod.layers[0].fc1
    names = [n for n, _ in sch.named_schedules()]
    assert "layers.0.fc1" in names and "seq.2" in names
    assert sch.world_size == 1 and sch.rank == 0


def test_primitive_registry():
    names = slapo.list_primitives()
    for want in ("replace", "shard", "sync", "fork_rng", "annotate", "checkpoint", "fuse",
                 "decompose", "cut_pipeline_stage", "replace_all"):
        assert want in names, want
    table = slapo.list_primitives(name_only=False)
    assert set(table) == set(names)

    from slapo_b200.primitives.base import Primitive, register_primitive

    @register_primitive()
    class CountParams(Primitive):
        @staticmethod
        def name():
            return "count_params_for_test"

        @staticmethod
        def apply(sch):
            return sum(p.numel() for p in sch.mod.parameters())

    sch = slapo.create_schedule(Block())
    assert sch.count_params_for_test() == 8 * 16 + 16 + 16 * 8 + 8
    with pytest.raises(Exception):
        @register_primitive()
        class Again(Primitive):  # duplicate name
            @staticmethod
            def name():
                return "count_params_for_test"

            @staticmethod
            def apply(sch):
                return 0
    with pytest.raises(Exception):
        @register_primitive()
        class NotAPrimitive:  # wrong base class
            pass
    with pytest.raises(AttributeError):
        sch.no_such_primitive()


def test_replace_module_transfers_hooks_and_updates_tree():
    model = Net()
    calls = []
    model.layers[0].fc1.register_forward_pre_hook(lambda m, i: calls.append("pre"))
    model.layers[0].fc1.register_forward_hook(lambda m, i, o: calls.append("post"))
    model.layers[0].fc1.register_full_backward_hook(lambda m, gi, go: calls.append("bwd"))
    sch = slapo.create_schedule(model)
    new = nn.Linear(8, 16)
    sch["layers.0.fc1"].replace(new)
    assert sch.mod.layers[0].fc1 is new and sch["layers.0.fc1"].mod is new
    sch.mod(torch.randn(2, 8, requires_grad=True)).sum().backward()
    assert calls == ["pre", "post", "bwd"]
    # a replaced Sequential element
    sch["seq"]["1"].replace(nn.GELU())
    assert isinstance(sch.mod.seq[1], nn.GELU)


def test_replace_all():
    sch = slapo.create_schedule(Net())

    def make(name, mod, scale=1):
        new = nn.Linear(mod.in_features, mod.out_features * scale)
        new.tag = name
        return new

    sch.replace_all(nn.ReLU, lambda name, mod: nn.Tanh())
    assert all(isinstance(b.act, nn.Tanh) for b in sch.mod.layers)
    assert isinstance(sch.mod.seq[1], nn.Tanh)
    sch["layers.0"].replace_all(nn.Linear, make, scale=1)
    assert sch.mod.layers[0].fc1.tag.endswith("fc1")
    assert not hasattr(sch.mod.layers[1].fc1, "tag")


def test_annotate_survives_build():
    sch = slapo.create_schedule(Net())
    sch["layers.0.fc1"].annotate("weight", "my_tag", 7)
    model, _ = slapo.build(sch, init_weights=False)
    assert model.layers[0].fc1.weight.my_tag == 7


class Tied(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(16, 8)
        self.head = nn.Linear(8, 16, bias=False)
        self.head.weight = self.emb.weight

    def forward(self, ids):
        return self.head(self.emb(ids))


def test_tie_weight_analysis():
    from slapo_b200.pipeline import analyze_tie_weights
    ties = analyze_tie_weights(Tied(), False)
    assert len(ties) == 1
    (names,) = ties.values()
    assert sorted(n for n, _ in names) == ["emb.weight", "head.weight"]


def test_checkpoint_hands_catch_all_keyword_arguments_on_by_name():
    """A layer whose forward ends in ``**kwargs`` (the Hugging Face convention): named
    arguments are checkpointed positionally, what falls into ``**kwargs`` is passed by name -
    unless it carries a gradient."""
    import pytest as _pytest

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(4, 4)

        def forward(self, x, scale=1.0, **kwargs):
            return self.fc(x) * scale + kwargs.get("shift", 0.0)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.layer = Layer()

        def forward(self, x, shift):
            return self.layer(x, scale=2.0, shift=shift, flag=True)

    torch.manual_seed(0)
    net = Net()
    x = torch.randn(3, 4, requires_grad=True)
    shift = torch.randn(3, 4)
    want = net(x, shift)
    want.sum().backward()
    weight = net.layer.fc.weight
    grad = weight.grad.clone()
    net.zero_grad()
    sch = slapo.create_schedule(net)
    sch["layer"].checkpoint()
    got = sch.mod(x, shift)
    torch.testing.assert_close(got, want)
    got.sum().backward()
    torch.testing.assert_close(weight.grad, grad)
    with _pytest.raises(ValueError, match="carry gradients"):
        sch.mod(x, shift.clone().requires_grad_(True))


def test_checkpoint_refuses_a_key_value_cache():
    """A stateful cache handed into a recomputed layer would be appended to twice."""
    import pytest as _pytest

    class Cache:
        def get_seq_length(self):
            return 0

        def update(self, *a):
            return a

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.layer = nn.Linear(4, 4)

        def forward(self, x, cache=None):
            return self.layer(x)

    class Top(nn.Module):
        def __init__(self):
            super().__init__()
            self.net = Net()

        def forward(self, x, cache=None):
            return self.net(x, cache=cache)

    sch = slapo.create_schedule(Top())
    sch["net"].checkpoint()
    x = torch.randn(2, 4, requires_grad=True)
    assert sch.mod(x).shape == (2, 4)
    with _pytest.raises(ValueError, match="use_cache"):
        sch.mod(x, cache=Cache())
