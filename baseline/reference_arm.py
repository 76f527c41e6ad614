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


def run(args, ref_root, model_dims, dist_setup, make_batch, timed_loop, clock_sampler_cls):
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
        print(json.dumps({"impl": "reference", "unavailable": "a different slapo package shadows baseline/_ref"}))
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
    if not args.no_e2e:
        host = [make_batch(vocab, local_batch, args.seq, 77 + i, "cpu", pin=True) for i in range(2)]
        h2d = sum(t.numel() * t.element_size() for t in host[0])

        def e2e_step(i):
            hi, hl = host[i % 2]
            loss = step_on(hi.to(device, non_blocking=True), hl.to(device, non_blocking=True))
            return float(loss.item())

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
            "config": {"model": "bert-large", "layers": args.layers, "global_batch": local_batch,
                       "seq_len": args.seq, "parallelism": f"tp{tp}" if tp > 1 else "single",
                       "ckpt_ratio": args.ckpt_ratio, "checkpointed_layers": n_ckpt,
                       "optimizer": "torch.optim.AdamW",
                       "attention": "HF sdpa (reference flash path needs xformers/flash-attn<2)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
            "max_mem_mb": torch.cuda.max_memory_allocated() / 2**20,
        }), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
