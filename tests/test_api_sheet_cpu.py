"""The public surface a user of the reference relies on exists under the same names and takes
the same parameters (positional order and keyword names)."""
import importlib
import inspect

import pytest

import slapo_b200 as slapo


def _params(obj):
    return list(inspect.signature(obj).parameters)


def _has(obj, *names):
    have = _params(obj)
    missing = [n for n in names if n not in have]
    assert not missing, f"{obj}: missing parameters {missing} (has {have})"


def test_top_level():
    assert _params(slapo.create_schedule)[:5] == ["root", "name", "path", "parent", "group"]
    assert _params(slapo.build)[:3] == ["sch", "target", "init_weights"]
    assert _params(slapo.list_primitives) == ["name_only"]
    assert callable(slapo.register_primitive)
    _has(slapo.Verify, "sch", "example_inputs", "device", "eval_mode", "enable")
    assert _params(slapo.checkpoint)[0] == "function"
    _has(slapo.checkpoint, "use_reentrant")
    assert _params(slapo.set_random_seed) == ["seed", "dp_rank", "pp_rank", "tp_rank",
                                              "always_enable_tp_seed"]
    assert callable(slapo.get_cuda_rng_tracker) and callable(slapo.is_random_seed_set)
    assert _params(slapo.init_empty_weights) == ["enable", "include_buffers"]
    assert _params(slapo.get_logger)[:2] == ["name", "level"]
    env = importlib.import_module("slapo_b200.env")
    assert _params(env.setup)[:3] == ["rank", "world_size", "backend"]
    assert callable(env.cleanup) and _params(env.execute)[:2] == ["fn", "args"]


def test_schedule_methods():
    from slapo_b200.schedule import Schedule

    for name in ("get_top_schedule", "get_module", "named_schedules", "trace", "trace_until", "find",
                 "find_node", "find_subgraph", "replace", "replace_all", "shard", "sync", "fork_rng",
                 "annotate", "checkpoint", "fuse", "decompose", "cut_pipeline_stage"):
        assert hasattr(Schedule, name) or name in slapo.list_primitives(), name
    for attr in ("__getitem__", "__contains__"):
        assert hasattr(Schedule, attr)
    prims = slapo.list_primitives(name_only=False)
    for name in ("replace", "replace_all", "shard", "sync", "fork_rng", "annotate", "checkpoint",
                 "fuse", "decompose", "cut_pipeline_stage"):
        assert name in prims, name


def test_sub_packages():
    pattern = importlib.import_module("slapo_b200.pattern")
    assert {"Pattern", "ModulePattern", "call_module"} <= set(dir(pattern))
    op = importlib.import_module("slapo_b200.op")
    _has(op.FlashAttention, "hidden_size", "num_attention_heads", "attn_pdrop", "resid_pdrop",
         "attn_op_name", "bias", "output_proj", "fused_qkv")
    _has(op.FlashAttentionOp, "attn_op_name", "apply_causal_mask", "scale")
    assert _params(op.FlashAttentionOp.forward)[1:6] == ["query_layer", "key_layer", "value_layer",
                                                          "attention_mask", "p"]
    _has(op.ParallelCrossEntropy, "group")
    assert _params(op.FusedQKV)[:3] == ["hidden_size", "num_heads", "world_size"]
    _has(op.LinearWithSyncFunc, "in_features", "out_features", "bias", "device", "dtype", "sync_fn")
    assert _params(op.FusedMLP)[:4] == ["hidden_size", "intermediate_size", "orig_act", "resid_pdrop"]
    for name in ("LinearWithSeparateBias", "Print"):
        assert hasattr(op, name), name
    sharding = importlib.import_module("slapo_b200.sharding")
    _has(sharding.all_gather_forward_output, "inp", "dim", "group", "tensor_parallel_output_grad")
    for name in ("reduce_scatter_forward_output", "scatter_forward_output"):
        assert _params(getattr(sharding, name))[:3] == ["inp", "dim", "group"], name
    for name in ("reduce_forward_output", "reduce_backward_grad"):
        assert _params(getattr(sharding, name))[:2] == ["inp", "group"], name
    for name in ("register_shard_method", "ShardMethod", "apply_shard_method", "apply_sync_method",
                 "new_or_get_tied_param"):
        assert hasattr(sharding, name), name
    pipeline = importlib.import_module("slapo_b200.pipeline")
    assert _params(pipeline.analyze_tie_weights)[:2] == ["top_mod", "is_pipeline_partitioned"]
    assert _params(pipeline.generate_pipeline_partition)[:1] == ["sch"]
    assert _params(pipeline.build_pipeline_model)[:2] == ["sch", "target"]
    assert _params(pipeline.analyze_pipeline_module)[:1] == ["top_mod"]
    ms = importlib.import_module("slapo_b200.model_schedule")
    assert _params(ms.apply_schedule)[:2] == ["model", "schedule_key"]
    reg = importlib.import_module("slapo_b200.model_schedule.registry")
    assert callable(reg.register_schedule) and callable(reg.get_schedule)
    fd = importlib.import_module("slapo_b200.framework_dialect")
    assert _params(fd.register_framework_dialect)[:2] == ["target", "cls_type"]
    assert _params(fd.get_dialect_cls)[:3] == ["cls_type", "target", "allow_none"]
    assert _params(fd.get_all_dialects)[:1] == ["cls_type"]
    report = importlib.import_module("slapo_b200.utils.report")
    assert _params(report.report_memory)[:2] == ["msg", "report_gc"]
    assert _params(report.profile_perf)[:3] == ["model", "inputs", "backward"]
    assert callable(report.calc_decoder_tflops)
    common = importlib.import_module("slapo_b200.utils.common")
    for name in ("get_hooks", "has_hook", "transfer_hooks", "transfer_hooks_for_fusion",
                 "transfor_param_tags", "is_module_list", "importlib_or_none"):
        assert hasattr(common, name), name
    tune = importlib.import_module("slapo_b200.autotune.tune")
    assert _params(tune.Database)[:1] == ["db_file_name"]
    for name in ("load", "commit"):
        assert hasattr(tune.Database, name)
    for name in ("create_symbol", "next", "reset", "to_dict", "clone", "log_space"):
        assert hasattr(tune.Space, name), name
    assert _params(tune.Symbol)[:2] == ["name", "vals"]


@pytest.mark.parametrize("mode,op", [("fwd_post", "all_gather"), ("fwd_post", "reduce_scatter"),
                                     ("fwd_post", "scatter"), ("fwd_post", "all_reduce"),
                                     ("fwd_post", "RS->SR"), ("fwd_pre", "all_gather"),
                                     ("fwd_pre", "SR->RS"), ("bwd_post", "all_reduce")])
def test_sync_accepts_the_documented_string_ops(mode, op):
    import torch
    from torch import nn

    sch = slapo.create_schedule(nn.Sequential(nn.Linear(4, 4)), group=False)
    kwargs = {"axis": 0} if op in ("all_gather", "reduce_scatter", "scatter") else {}
    sch["0"].sync(mode, op, **kwargs)
    assert torch.is_tensor(sch.mod(torch.zeros(2, 4)))
