"""Reference arm of ``bench.py``: the unmodified reference package.

The reference (installed offline into ``baseline/_ref``) is driven through its
own public API and stock code:

* model: Hugging Face ``BertForMaskedLM`` built from a config (random init);
* ``slapo.create_schedule`` on it, then - for TP > 1 - the reference's own
  recipe functions ``shard_mlp`` and ``shard_word_embedding`` from
  ``slapo.model_schedule.bert`` plus ``shard`` / ``sync`` on the attention
  projections exactly as its recipe's ``shard_attention`` does, and
  ``.checkpoint()`` on the first ``int(L * ratio)`` layers (its recipe's
  ``checkpoint``);
* ``slapo.build(sch, init_weights=False)`` with the default dialect, then the
  plain PyTorch AdamW loop of the reference's ``examples/utils.py``
  (``train_with_torch``), because DeepSpeed and Megatron-LM are not installed.

What is *not* live on this box: the reference's flash-attention replacement
(``replace_and_shard_attention`` needs xFormers or flash-attn's pre-2.0
``flash_attn_unpadded_func``); Hugging Face's own SDPA attention runs instead.
None of this framework's code is on this path.
"""
from __future__ import annotations

import json
import os
import sys


def _shard_attention(sch, layers, prefix):
    for idx in range(layers):
        base = f"{prefix}.encoder.layer.{idx}.attention"
        for name in ("query", "key", "value"):
            sub = sch[f"{base}.self.{name}"]
            sub.shard("weight", axis=0)
            sub.shard("bias", axis=0)
            sub.sync(mode="bwd_post", sync_op_or_fn="all_reduce")
        sch[f"{base}.output.dense"].shard("weight", axis=1)
        sch[f"{base}.output.dense"].sync(mode="fwd_post", sync_op_or_fn="all_reduce")


def run(args, ref_root, model_dims, dist_setup, make_batch, timed_loop, clock_sampler_cls,
        make_config):
    import torch

    sys.path.insert(0, ref_root)
    try:
        import slapo  # the reference
        from slapo.model_schedule import bert as ref_bert
        from transformers import BertConfig, BertForMaskedLM
    except Exception as err:
        print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {err}"}))
        return
    if not os.path.abspath(slapo.__file__).startswith(os.path.abspath(ref_root)):
        print(json.dumps({"impl": "reference",
                          "unavailable": "a different slapo package shadows baseline/_ref"}))
        return

    world, rank, local = dist_setup(args)
    device = torch.device("cuda", local)
    tp = world
    vocab = (model_dims["vocab"] + 8 * tp - 1) // (8 * tp) * (8 * tp)
    cfg = BertConfig(vocab_size=vocab, hidden_size=model_dims["hidden"],
                     num_hidden_layers=args.layers, num_attention_heads=model_dims["heads"],
                     intermediate_size=model_dims["ffn"],
                     max_position_embeddings=max(512, args.seq))
    torch.manual_seed(2013)
    model = BertForMaskedLM(cfg).to(torch.bfloat16).to(device)
    sch = slapo.create_schedule(model)
    prefix = "bert"
    if tp > 1:
        _shard_attention(sch, args.layers, prefix)
        ref_bert.shard_mlp(sch[prefix], cfg)
        ref_bert.shard_word_embedding(sch[prefix], cfg.vocab_size)
    # the reference recipe's checkpoint(): the first int(L * ratio) layers.  The
    # primitive's own `order_args_fn` hook is used because Hugging Face 5.x
    # passes BertLayer extra keyword arguments that cannot be replayed
    # positionally (only hidden_states and attention_mask are live here).
    def order_args(*a, **kw):
        mask = a[1] if len(a) > 1 else kw.get("attention_mask")
        return [a[0], mask]

    n_ckpt = int(args.layers * args.ckpt_ratio) if args.ckpt_ratio > 0 else 0
    for idx in range(n_ckpt):
        sch[f"{prefix}.encoder.layer.{idx}"].checkpoint(order_args_fn=order_args)
    model, _ = slapo.build(sch, init_weights=False)
    model.train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)

    local_batch = args.batch_per_gpu * tp  # every TP rank consumes the whole batch
    ids, labels = make_batch(vocab, local_batch, args.seq, 1234, device)

    def step_on(i_ids, i_labels):
        out = model(input_ids=i_ids, labels=i_labels)
        loss = out.loss if hasattr(out, "loss") else out[0]
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss

    def step(_i):
        step_on(ids, labels)

    for i in range(args.warmup):
        step(i)
    sampler = clock_sampler_cls(local)
    sampler.start()
    ms = timed_loop(step, args.steps, device, world)
    clocks = sampler.finish()
    value = local_batch * args.steps / (ms / 1e3)

    e2e = None
    losses = []
    if not args.no_e2e:
        host = [make_batch(vocab, local_batch, args.seq, 77 + i, "cpu", pin=True) for i in range(2)]
        h2d = sum(t.numel() * t.element_size() for t in host[0])

        def e2e_step(i):
            hi, hl = host[i % 2]
            loss = step_on(hi.to(device, non_blocking=True), hl.to(device, non_blocking=True))
            losses.append(float(loss.item()))
            return losses[-1]

        e2e_step(0)
        ms_e = timed_loop(e2e_step, args.steps, device, world)
        e2e = {"value": local_batch * args.steps / (ms_e / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
               "ms_per_step": ms_e / args.steps}
    if rank == 0:
        print(json.dumps({
            "metric": "train samples/sec, BERT-large MLM", "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": make_config("bert-large", args.layers, local_batch, args.seq,
                                  f"tp{tp}" if tp > 1 else "single", args.ckpt_ratio, local_batch),
            "notes": {"checkpointed_layers": n_ckpt, "optimizer_impl": "torch.optim.AdamW",
                      "attention": "HF sdpa (reference flash path needs xformers/flash-attn<2)"},
            "loss": {"first": losses[0] if losses else None, "last": losses[-1] if losses else None},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
            "max_mem_mb": torch.cuda.max_memory_allocated() / 2**20,
        }), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
def _shard_opt(sch, cfg, ref_opt, world):
    """Tensor parallelism of a Hugging Face ``OPTForCausalLM`` with the reference's primitives.

    The reference recipe (``slapo.model_schedule.opt``) first swaps the attention for its own
    ``FlashAttention`` module, which cannot be built on this box (xFormers / flash-attn < 2
    are absent); the projections of the stock attention are sharded instead, the way the
    recipe shards its fused QKV (columns + ``bwd_post`` all-reduce, output rows + ``fwd_post``
    all-reduce).  MLP, word embedding and checkpointing are the recipe's own functions."""
    for idx in range(cfg.num_hidden_layers):
        attn = sch[f"model.decoder.layers.{idx}.self_attn"]
        for name in ("q_proj", "k_proj", "v_proj"):
            attn[name].shard("weight", axis=0)
            attn[name].shard("bias", axis=0)
            attn[name].sync(mode="bwd_post", sync_op_or_fn="all_reduce")
        attn["out_proj"].shard("weight", axis=1)
        attn["out_proj"].sync(mode="fwd_post", sync_op_or_fn="all_reduce")
        attn.mod.num_heads //= world          # the module reshapes to its local heads
        if hasattr(attn.mod, "embed_dim"):
            attn.mod.embed_dim //= world
    ref_opt.replace_and_shard_mlp(sch["model"], cfg, delay_init=False)
    ref_opt.shard_word_embedding(sch["model"], sch["lm_head"], cfg.vocab_size)


def run_opt(args, ref_root, dims, dist_setup, timed_loop, clock_sampler_cls, make_config):
    """OPT-2.7B-shaped causal LM through the unmodified reference: TP = all GPUs (the
    reference's pipeline path needs DeepSpeed, which is not installed), gradient accumulation
    over micro-batches of 4, plain PyTorch AdamW loop."""
    import torch

    sys.path.insert(0, ref_root)
    try:
        import slapo  # the reference
        from slapo.model_schedule import opt as ref_opt
        from transformers import OPTConfig, OPTForCausalLM
    except Exception as err:
        print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {err}"}))
        return
    if not os.path.abspath(slapo.__file__).startswith(os.path.abspath(ref_root)):
        print(json.dumps({"impl": "reference",
                          "unavailable": "a different slapo package shadows baseline/_ref"}))
        return
    world, rank, local = dist_setup(args)
    device = torch.device("cuda", local)
    tp = world
    cfg = OPTConfig(vocab_size=dims["vocab"], hidden_size=dims["hidden"],
                    num_hidden_layers=args.layers, ffn_dim=dims["ffn"],
                    num_attention_heads=dims["heads"], max_position_embeddings=max(2048, args.seq),
                    word_embed_proj_dim=dims["hidden"], activation_function="relu",
                    do_layer_norm_before=True, tie_word_embeddings=True)
    torch.manual_seed(2013)
    model = OPTForCausalLM(cfg).to(torch.bfloat16).to(device)
    sch = slapo.create_schedule(model)
    vocab_parallel = False
    if tp > 1:
        _shard_opt(sch, cfg, ref_opt, world)
        vocab_parallel = True
    # the reference recipe's checkpoint(): the first int(L * ratio) layers; the primitive's own
    # `order_args_fn` hook is used because Hugging Face 5.x passes the decoder layer keyword
    # arguments that the recipe's positional replay would misplace
    def order_args(*a, **kw):
        mask = a[1] if len(a) > 1 else kw.get("attention_mask")
        return [a[0], mask]

    n_ckpt = int(cfg.num_hidden_layers * args.ckpt_ratio) if args.ckpt_ratio > 0 else 0
    for idx in range(n_ckpt):
        sch[f"model.decoder.layers.{idx}"].checkpoint(order_args_fn=order_args)
    model, _ = slapo.build(sch, init_weights=False)
    model.train()
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    micro = dims["micro_batch"]
    global_batch = args.batch_per_gpu * world       # every TP rank consumes the whole batch
    n_micro = max(global_batch // micro, 1)

    def make(seed, dev, pin=False):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg.vocab_size, (micro, args.seq), generator=g)
        if pin:
            ids = ids.pin_memory()
        return ids.to(dev)

    loss_parallel = None
    if vocab_parallel:
        from slapo.op import ParallelCrossEntropy

        loss_parallel = ParallelCrossEntropy(group=None)

    def micro_step(ids):
        if vocab_parallel:
            logits = model(input_ids=ids).logits            # [B, S, V / tp]
            loss = loss_parallel(logits[:, :-1].contiguous().float(), ids[:, 1:].contiguous())
            loss = loss.mean()
        else:
            loss = model(input_ids=ids, labels=ids).loss
        (loss / n_micro).backward()
        return loss

    def finish_step():
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)

    dev_batches = [make(1234 + i, device) for i in range(n_micro)]

    def step(_i):
        for ids in dev_batches:
            micro_step(ids)
        finish_step()

    for i in range(args.warmup):
        step(i)
    sampler = clock_sampler_cls(local)
    sampler.start()
    ms = timed_loop(step, args.steps, device, world)
    clocks = sampler.finish()
    value = global_batch * args.steps / (ms / 1e3)
    e2e, losses = None, []
    if not args.no_e2e:
        host = [[make(77 + 10 * j + i, "cpu", pin=True) for i in range(n_micro)] for j in range(2)]
        h2d = sum(t.numel() * t.element_size() for t in host[0])

        def e2e_step(i):
            loss = None
            for ids in host[i % 2]:
                loss = micro_step(ids.to(device, non_blocking=True))
            finish_step()
            losses.append(float(loss.item()))
            return losses[-1]

        e2e_step(0)
        ms_e = timed_loop(e2e_step, args.steps, device, world)
        e2e = {"value": global_batch * args.steps / (ms_e / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
               "ms_per_step": ms_e / args.steps}
    if rank == 0:
        print(json.dumps({
            "metric": "train samples/sec, OPT-2.7B causal LM", "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": make_config("opt-2.7b", args.layers, global_batch, args.seq,
                                  f"tp{tp}" if tp > 1 else "single", args.ckpt_ratio, micro),
            "notes": {"micro_batches": n_micro, "checkpointed_layers": n_ckpt,
                      "pipeline": "not available in the reference without DeepSpeed: TP only",
                      "attention": "HF sdpa (reference flash path needs xformers/flash-attn<2)"},
            "loss": {"first": losses[0] if losses else None, "last": losses[-1] if losses else None},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
            "max_mem_mb": torch.cuda.max_memory_allocated() / 2**20,
        }), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
