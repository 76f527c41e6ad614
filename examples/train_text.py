"""Train a small GPT-style or BERT-style model on a local text file, every step written out:
mesh, model on the meta device, schedule recipe, ``build``, data loaders, training loop with
validation, sharded checkpoint and resume.

    python examples/train_text.py --text README.md --steps 50                       # one process
    torchrun --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        examples/train_text.py --text README.md --tp 2 --dp 2 --family bert --save ckpt/

Runs on CPU ranks (gloo) as well as on GPUs (NCCL, native kernels).  Parity: the flow of the
reference's examples/<model>/deepspeed_hf.py (init, topology, ``apply_schedule``, ``slapo.build``,
data loader, ``train_batch`` loop), with this library's own engine as the target.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import data_util  # noqa: E402

import slapo_b200 as slapo  # noqa: E402
from slapo_b200 import ckpt  # noqa: E402
from slapo_b200.models import (BertConfig, BertForMaskedLM, GPT2LMHeadModel, GPTConfig,  # noqa: E402
                               causal_lm_loss, mlm_loss)
from slapo_b200.parallel.mesh import DeviceMesh  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--text", required=True, help="UTF-8 text file; its bytes are the tokens")
    ap.add_argument("--family", default="gpt", choices=["gpt", "bert"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--batch-size", type=int, default=8, help="samples per step and replica")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=0, help="0 = world size / tp")
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--ckpt-ratio", type=float, default=0.0)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--eval-every", type=int, default=10)
    ap.add_argument("--save", default=None, help="directory of the sharded checkpoint written at the end")
    ap.add_argument("--resume", default=None, help="directory of a checkpoint to continue from")
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def init_distributed():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    return world, rank, device


def build_model(args, tp_group):
    """(config, model class, recipe name, loss).  With tensor parallelism the logits stay
    sharded over the vocabulary and the loss is the vocabulary-parallel cross entropy."""
    vocab = 320        # 257 byte tokens, padded so that every tensor-parallel shard is whole
    vp = args.tp > 1
    if args.family == "bert":
        cfg = BertConfig(vocab_size=vocab, hidden_size=args.hidden, num_hidden_layers=args.layers,
                         num_attention_heads=args.heads, intermediate_size=4 * args.hidden,
                         max_position_embeddings=args.seq_len)
        return cfg, BertForMaskedLM, "bert", lambda out, lab: mlm_loss(out["logits"], lab, tp_group, vp)
    cfg = GPTConfig(vocab_size=vocab, hidden_size=args.hidden, num_layers=args.layers,
                    num_heads=args.heads, n_positions=args.seq_len)
    return cfg, GPT2LMHeadModel, "gpt2", lambda out, lab: causal_lm_loss(out["logits"], lab, tp_group, vp)


@torch.no_grad()
def evaluate(engine, loader, loss_fn, device):
    model = engine.model
    was_training = model.training
    model.eval()
    total, count = 0.0, 0
    for ids, labels in loader:
        out = model(ids.to(device))
        total += float(loss_fn(out, labels.to(device)))
        count += 1
    model.train(was_training)
    return total / max(count, 1)


def main(argv=None):
    args = parse_args(argv)
    world, rank, device = init_distributed()
    dp = args.dp or world // args.tp
    mesh = DeviceMesh(pp=1, dp=dp, tp=args.tp) if world > 1 else None
    slapo.set_random_seed(args.seed, dp_rank=mesh.dp_rank if mesh else 0, tp_rank=mesh.tp_rank if mesh else 0)

    # 1. the model: on GPUs it is created on the meta device (no memory until the schedule has
    #    sharded it), on CPU ranks with real weights
    cfg, cls, recipe, loss_fn = build_model(args, mesh.tp_group if mesh else None)
    on_gpu = device.type == "cuda"
    if on_gpu:
        with slapo.init_empty_weights():
            model = cls(cfg)
    else:
        model = cls(cfg).init_weights()
    # 2. the schedule recipe: tensor / sequence parallelism, fused kernels, checkpointing
    sch = slapo.model_schedule.apply_schedule(
        model, recipe, model_config=cfg, group=mesh.schedule_group if mesh else None, bf16=on_gpu,
        sequence_parallel=args.sequence_parallel and args.tp > 1, sequence_parallel_axis=0,
        ckpt_ratio=args.ckpt_ratio)
    # 3. materialise the shards and wrap them in the engine (ZeRO-1 data parallelism, fused AdamW)
    engine, _ = slapo.build(sch, target="native", mesh=mesh, loss_fn=loss_fn,
                            init_weights=model._init_weights if on_gpu else False,
                            config={"lr": args.lr, "weight_decay": 0.01, "clip_grad": 1.0})
    start = 0
    if args.resume:
        start = ckpt.load_checkpoint(args.resume, engine.model, engine, mesh=mesh)["step"]
    # 4. data: every data-parallel replica reads its own rows
    kind = "mlm" if args.family == "bert" else "causal"
    train_loader, val_loader, sampler = data_util.get_dataloaders(
        args.text, args.seq_len, args.batch_size, mesh=mesh, kind=kind, seed=args.seed,
        device=device if device.type == "cuda" else None)
    # 5. the loop
    step, epoch, t0 = start, 0, time.time()
    history = []
    while step < start + args.steps:
        sampler.set_epoch(epoch)
        for ids, labels in train_loader:
            loss = engine.train_batch(ids.to(device), labels=labels.to(device))
            step += 1
            history.append(float(loss))
            if step % args.eval_every == 0 or step == start + args.steps:
                # every rank takes part (tensor-parallel layers communicate); rank 0 reports
                # the validation loss of its own data-parallel share
                val = evaluate(engine, val_loader, loss_fn, device)
                if rank == 0:
                    print(f"step {step}: loss {history[-1]:.4f}  validation {val:.4f}  "
                          f"{(time.time() - t0) / (step - start):.3f} s/step", flush=True)
            if step >= start + args.steps:
                break
        epoch += 1
    if args.save:
        engine.step_count = step
        ckpt.save_checkpoint(args.save, engine.model, engine, mesh=mesh)
    if world > 1:
        dist.barrier()
    return history


if __name__ == "__main__":
    main()
