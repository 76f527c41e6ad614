"""Static-graph path: hierarchical / flattened tracing, pattern search,
vertical and horizontal replacement, fusion and decomposition."""
import operator

import pytest
import torch
import torch.nn.functional as F
from torch import fx, nn

import slapo_b200 as slapo
from slapo_b200.pattern import ModulePattern, Pattern, call_module


class SelfAttn(nn.Module):
    def __init__(self):
        super().__init__()
        self.query = nn.Linear(16, 16)
        self.key = nn.Linear(16, 16)
        self.value = nn.Linear(16, 16)

    def forward(self, x):
        q, k, v = self.query(x), self.key(x), self.value(x)
        return F.softmax(q @ k.transpose(-1, -2), dim=-1) @ v


class Untraceable(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(16, 16)

    def forward(self, x):
        if x.sum() > 0:   # data-dependent control flow
            return self.lin(x)
        return x


class Layer(nn.Module):
    def __init__(self, bad=False):
        super().__init__()
        self.attn = SelfAttn()
        self.dense = nn.Linear(16, 16)
        self.act = nn.ReLU()
        self.extra = Untraceable() if bad else nn.Identity()

    def forward(self, x):
        y = self.act(self.dense(self.attn(x)))
        return self.extra(y) + x


class Model(nn.Module):
    def __init__(self, bad=False):
        super().__init__()
        self.layers = nn.ModuleList([Layer(bad) for _ in range(2)])

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


def test_hierarchical_trace_keeps_untraceable_children():
    model = Model(bad=True)
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    assert sch.trace(recursive=True)
    assert isinstance(sch.mod, fx.GraphModule)
    assert isinstance(sch["layers.0"].mod, fx.GraphModule)
    assert isinstance(sch["layers.0.attn"].mod, fx.GraphModule)
    assert isinstance(sch["layers.0.extra"].mod, Untraceable)  # left alone, no exception
    torch.testing.assert_close(sch.mod(x), want)


def test_flatten_trace():
    model = Layer()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    sch.trace(flatten=True)
    targets = [n.target for n in sch.mod.graph.nodes if n.op == "call_module"]
    assert "attn.query" in targets and "dense" in targets
    with pytest.raises(KeyError):
        sch["attn"]["query"]
    assert isinstance(sch.get_module("attn.query"), nn.Linear)
    torch.testing.assert_close(sch.mod(x), want)


def test_leaf_modules_by_class_name():
    sch = slapo.create_schedule(Layer())
    sch.trace(flatten=True, leaf_modules=["SelfAttn"])
    targets = [n.target for n in sch.mod.graph.nodes if n.op == "call_module"]
    assert "attn" in targets and "attn.query" not in targets


def test_find_regex_and_predicate():
    sch = slapo.create_schedule(Layer())
    sub = sch["attn"]
    sub.trace()
    found = sub.find(r"query|key|value")
    assert len(found) == 3
    nodes = sub.find_node(lambda n: n.op == "call_function" and n.target is F.softmax)
    assert len(nodes) == 1


def test_find_functional_pattern_matches_module_call():
    sch = slapo.create_schedule(Layer())
    sch.trace(flatten=True)

    def pattern(x):
        return F.relu(call_module("dense", x))

    matches = sch.find(pattern)
    assert len(matches) == 1
    assert [n.target for _, n in matches[0]] == ["dense", "act"]


def test_find_pattern_class_and_module_pattern():
    class QK(Pattern):
        def __init__(self):
            super().__init__()
            self.lin = ModulePattern(r"query|key")

        def forward(self, x):
            return self.lin(x)

    sch = slapo.create_schedule(SelfAttn())
    sch.trace()
    matches = sch.find(QK())
    assert len(matches) == 2


def test_vertical_replace_names_and_numerics():
    model = Layer()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    sch.trace(flatten=True)

    def pattern(x):
        return F.relu(call_module("dense", x))

    class DenseRelu(nn.Module):
        def __init__(self, lin):
            super().__init__()
            self.lin = lin

        def forward(self, x):
            return F.relu(self.lin(x))

    sub = sch.find(pattern)
    sch.replace(DenseRelu(sch.get_module("dense")), sub, name="DenseRelu")
    targets = [n.target for n in sch.mod.graph.nodes if n.op == "call_module"]
    assert "DenseRelu_0" in targets and "dense" not in targets and "act" not in targets
    assert "DenseRelu_0" in sch.child
    torch.testing.assert_close(sch.mod(x), want)


def test_horizontal_replace_fuses_parallel_matches():
    model = SelfAttn()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    sch.trace()
    matches = sch.find(lambda x: call_module(r"query|key|value", x))
    assert len(matches) == 3 and all(len(m) == 1 for m in matches)

    class QKV(nn.Module):
        def __init__(self, q, k, v):
            super().__init__()
            self.fused = nn.Linear(16, 48)
            with torch.no_grad():
                self.fused.weight.copy_(torch.cat([q.weight, k.weight, v.weight]))
                self.fused.bias.copy_(torch.cat([q.bias, k.bias, v.bias]))

        def forward(self, x):
            return self.fused(x).chunk(3, dim=-1)

    sch.replace(QKV(model.query, model.key, model.value), matches, name="QKV")
    calls = [n for n in sch.mod.graph.nodes if n.op == "call_module"]
    assert [c.target for c in calls] == ["QKV_0"]
    items = [n for n in sch.mod.graph.nodes if n.op == "call_function" and n.target is operator.getitem]
    assert [n.args[1] for n in items] == [0, 1, 2]
    torch.testing.assert_close(sch.mod(x), want, rtol=1e-5, atol=1e-5)


def test_replace_function():
    model = SelfAttn()
    x = torch.randn(2, 4, 16)
    sch = slapo.create_schedule(model)
    sch.trace()
    node = sch.find_node(lambda n: n.op == "call_function" and n.target is F.softmax)

    def my_softmax(t, dim=-1, **_kw):
        return torch.softmax(t * 1.0, dim=dim)

    sch.replace(my_softmax, node)
    assert any(n.op == "call_function" and n.target is my_softmax for n in sch.mod.graph.nodes)
    torch.testing.assert_close(sch.mod(x), model(x))


def test_fuse_none_compiler_and_decompose():
    model = Layer()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    sch["dense"].decompose()
    sch.trace(flatten=True)

    def pattern(x, bias):
        return F.relu(x + bias)

    sub = sch.find(pattern)
    assert len(sub) == 1
    sch.fuse(sub, compiler=None, name="BiasRelu")
    fused = sch.get_module("BiasRelu_0")
    assert isinstance(fused, nn.Sequential) and type(fused).__name__ == "BiasRelu"
    built, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(built(x), want)
    # decompose keeps the very same Parameter objects
    assert any(p is model.dense.weight for p in built.parameters())
    assert any(p is model.dense.bias for p in built.parameters())


def test_fuse_none_keeps_chain_members():
    class ConvRelu(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = nn.Conv2d(3, 8, 3)
            self.relu = nn.ReLU()

        def forward(self, x):
            return self.relu(self.conv(x)) + 1

    model = ConvRelu()
    x = torch.randn(1, 3, 8, 8)
    want = model(x)
    sch = slapo.create_schedule(model)
    sub = sch.find(lambda x: F.relu(call_module("conv", x)))
    assert len(sub[0]) == 2
    sch.fuse(sub, compiler=None, name="FusedConvReLU")
    fused = sch.mod.FusedConvReLU_0
    assert type(fused).__name__ == "FusedConvReLU"
    assert isinstance(fused[0], nn.Conv2d) and isinstance(fused[1], nn.ReLU)
    torch.testing.assert_close(sch.mod(x), want)


def test_fuse_torchscript():
    model = Layer()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    sch["dense"].decompose()
    sch.trace(flatten=True)
    sub = sch.find(lambda x, bias: F.relu(x + bias))
    sch.fuse(sub, compiler="TorchScript", name="FusedBiasRelu")
    torch.testing.assert_close(sch.mod(x), want)


def test_fuse_native_bias_gelu_and_dropout_add_ln():
    """compiler="native": the chain is recognised and replaced by the module that
    calls the fused kernel (on CPU the same module runs its PyTorch fallback)."""
    from slapo_b200.ops.fusion_patterns import NativeBiasAct, NativeBiasDropoutAdd

    class FFN(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1 = nn.Linear(16, 32)
            self.fc2 = nn.Linear(32, 16)
            self.drop = nn.Dropout(0.0)
            self.ln = nn.LayerNorm(16)

        def forward(self, x):
            h = F.gelu(self.fc1(x), approximate="tanh")
            return self.ln(self.drop(self.fc2(h)) + x)

    model = FFN()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(model)
    sch["fc1"].decompose()
    sch["fc2"].decompose()
    sch.trace(flatten=True)

    sub = sch.find(lambda x, b: F.gelu(x + b, approximate="tanh"))
    assert len(sub) == 1
    sch.fuse(sub, compiler="native", name="BiasGelu")
    assert isinstance(sch.get_module("BiasGelu_0"), NativeBiasAct)

    def tail(x, b, res):
        return call_module("ln", call_module("drop", x + b) + res)

    sub = sch.find(tail)
    assert len(sub) == 1 and len(sub[0]) == 4
    sch.fuse(sub, compiler="native", name="DropAddLN")
    fused = sch.get_module("DropAddLN_0")
    assert isinstance(fused, NativeBiasDropoutAdd) and fused.layer_norm is model.ln
    torch.testing.assert_close(sch.mod(x), want, rtol=1e-5, atol=1e-5)

    with pytest.raises(NotImplementedError):
        sch2 = slapo.create_schedule(Layer())
        sch2.trace(flatten=True)
        sch2.fuse(sch2.find(lambda x: F.relu(call_module("dense", x))), compiler="native")


def test_dynamo_and_huggingface_tracer_names():
    model = SelfAttn()
    x = torch.randn(2, 4, 16)
    want = model(x)
    sch = slapo.create_schedule(SelfAttn())
    sch.mod.load_state_dict(model.state_dict())
    assert sch.trace(tracer="huggingface")
    torch.testing.assert_close(sch.mod(x), want)
    sch2 = slapo.create_schedule(SelfAttn())
    sch2.mod.load_state_dict(model.state_dict())
    assert sch2.trace(tracer="dynamo", concrete_args={"example_inputs": (x,)})
    assert isinstance(sch2.mod, fx.GraphModule)
    torch.testing.assert_close(sch2.mod(x), want)
    sch3 = slapo.create_schedule(SelfAttn())
    sch3.mod.load_state_dict(model.state_dict())
    assert sch3.trace(tracer="dynamo", concrete_args={"x": x})       # the reference's spelling
    torch.testing.assert_close(sch3.mod(x), want)
    assert not slapo.create_schedule(SelfAttn()).trace(tracer="no-such-tracer")


def test_checkpoint_of_a_matched_subgraph():
    """``sch.checkpoint(subgraph)``: the matched chain (dense -> bias add -> relu) becomes its
    own module under activation checkpointing; outputs and gradients are those of the plain
    model and the chain's activations are recomputed in backward."""
    from slapo_b200.primitives.checkpoint import CheckPointWrapper

    torch.manual_seed(0)
    model = Layer()
    x = torch.randn(2, 4, 16, requires_grad=True)
    want = model(x)
    want.sum().backward()
    want_grad = x.grad.clone()
    want_wgrad = model.dense.weight.grad.clone()
    x.grad = None
    model.zero_grad()

    sch = slapo.create_schedule(model)
    sch.trace(flatten=True)
    sub = sch.find(lambda x: F.relu(call_module("dense", x)))
    assert len(sub) == 1 and len(sub[0]) == 2
    sch.checkpoint(sub)
    wrappers = [m for m in sch.mod.modules() if isinstance(m, CheckPointWrapper)]
    assert len(wrappers) == 1
    calls = {"n": 0}
    wrappers[0].mod.register_forward_hook(lambda *_: calls.__setitem__("n", calls["n"] + 1))
    built, _ = slapo.build(sch, init_weights=False)
    got = built(x)
    torch.testing.assert_close(got, want)
    assert calls["n"] == 1
    got.sum().backward()
    assert calls["n"] == 2            # recomputed once in backward
    torch.testing.assert_close(x.grad, want_grad)
    torch.testing.assert_close(model.dense.weight.grad, want_wgrad)
    with pytest.raises(ValueError, match="exactly one"):
        sch.checkpoint([sub[0], sub[0]])


class ShapeDependent(nn.Module):
    """Python control flow on tensor shapes: untraceable for plain fx, fine once the proxies
    carry meta tensors."""

    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(50, 16)
        self.proj = nn.Linear(16, 16)
        self.attn = SelfAttn()

    def forward(self, input_ids, attention_mask=None):
        x = self.emb(input_ids)
        bsz, seq = input_ids.size()
        if seq > 4:                         # needs a concrete size
            x = self.proj(x)
        if attention_mask is not None:
            x = x * attention_mask.unsqueeze(-1)
        x = x.view(bsz, seq, -1)
        return self.attn(x)


def test_huggingface_tracer_propagates_meta_tensors():
    torch.manual_seed(0)
    model = ShapeDependent()
    ids = torch.randint(0, 50, (2, 16))
    want = model(ids)
    # the plain engine gives up on the shape-dependent branch and keeps the module eager
    plain = slapo.create_schedule(ShapeDependent())
    plain.mod.load_state_dict(model.state_dict())
    plain.trace(tracer="pytorch")
    assert not isinstance(plain.mod, fx.GraphModule)
    # the meta engine resolves it; hierarchy and numerics are preserved
    sch = slapo.create_schedule(ShapeDependent())
    sch.mod.load_state_dict(model.state_dict())
    assert sch.trace(tracer="huggingface", config={"seq_len": 16, "hidden_size": 16})
    assert isinstance(sch.mod, fx.GraphModule)
    torch.testing.assert_close(sch.mod(ids), want)
    assert "attn" in sch.child and isinstance(sch["attn"].mod, fx.GraphModule)
    shapes = {n.name: n.meta.get("shape") for n in sch.mod.graph.nodes}
    assert shapes["emb"] == (2, 16, 16) and shapes["input_ids"] == (2, 16)
    assert [n for n in sch.mod.graph.nodes if n.op == "call_module" and n.target == "proj"]
