"""A Hugging Face ``transformers`` model on pipeline x tensor x data parallelism, written the way
the example scripts of the reference are (examples/<model>/deepspeed_hf.py there): distributed
set-up, topology and tensor-parallel group, the model built without memory under
``init_empty_weights``, the family's recipe with pipeline cuts, ``build(target="deepspeed",
config=ds_config, topology=...)``, a training loop on synthetic tokens.  The ``"deepspeed"``
target (and ``--target megatron``, the counterpart of the reference's ``megatron_hf.py``
scripts) resolves to this framework's own engines, so nothing but PyTorch (and
``transformers`` for the model definition) is needed.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/deepspeed_hf.py \
        --family opt --hidden 2560 --layers 32 --heads 32 --pmp 2 --tmp 4 \
        --batch-size 64 --micro-batch-size 4 --seq-len 1024 --sequence-parallel

Runs on CPU ranks as well (``--device cpu``, gloo), which is how its test drives it.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import utils  # noqa: E402  (adds the repository root to sys.path)

import slapo_b200 as slapo  # noqa: E402
from slapo_b200.models import causal_lm_loss, mlm_loss, seq2seq_loss  # noqa: E402

FAMILIES = ("bert", "roberta", "albert", "gpt2", "gpt_neo", "opt", "t5")


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--family", default="opt", choices=FAMILIES)
    ap.add_argument("--hidden", type=int, default=768)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--vocab", type=int, default=50272)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--dec-seq-len", type=int, default=128, help="decoder length (t5)")
    ap.add_argument("--batch-size", type=int, default=16, help="samples per step and data-parallel replica")
    ap.add_argument("--micro-batch-size", type=int, default=4)
    ap.add_argument("--pmp", type=int, default=1, help="pipeline stages")
    ap.add_argument("--tmp", type=int, default=1, help="tensor-parallel ranks")
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--checkpoint", type=float, default=0.0, help="fraction of layers recomputed")
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "fp16", "fp32"))
    ap.add_argument("--iter-nums", type=int, default=10)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=2013)
    ap.add_argument("--target", default="deepspeed", choices=("deepspeed", "megatron", "native"),
                    help="runtime dialect named in build(); all three run the native engines")
    return ap.parse_args(argv)


def hf_model(args):
    """The configuration and an un-materialised model of the family (``transformers`` reads no
    file: every size comes from the command line)."""
    import transformers as tr

    h, n, a, v, s = args.hidden, args.layers, args.heads, args.vocab, args.seq_len
    if args.family in ("bert", "roberta", "albert"):
        kw = dict(vocab_size=v, hidden_size=h, num_hidden_layers=n, num_attention_heads=a,
                  intermediate_size=4 * h, max_position_embeddings=s + 2)
        config, cls = {"bert": (tr.BertConfig(**kw), tr.BertForMaskedLM),
                       "roberta": (tr.RobertaConfig(**kw), tr.RobertaForMaskedLM),
                       "albert": (tr.AlbertConfig(embedding_size=128, **kw),
                                  tr.AlbertForMaskedLM)}[args.family]
    elif args.family == "gpt2":
        config, cls = tr.GPT2Config(vocab_size=v, n_embd=h, n_layer=n, n_head=a,
                                    n_positions=s), tr.GPT2LMHeadModel
    elif args.family == "gpt_neo":
        config = tr.GPTNeoConfig(vocab_size=v, hidden_size=h, num_layers=n, num_heads=a,
                                 attention_types=[[["global"], n]], max_position_embeddings=s)
        cls = tr.GPTNeoForCausalLM
    elif args.family == "t5":
        config = tr.T5Config(vocab_size=v, d_model=h, d_kv=h // a, d_ff=4 * h, num_layers=n,
                             num_decoder_layers=n, num_heads=a)
        cls = tr.T5ForConditionalGeneration
    else:
        config = tr.OPTConfig(vocab_size=v, hidden_size=h, num_hidden_layers=n, ffn_dim=4 * h,
                              num_attention_heads=a, max_position_embeddings=s,
                              word_embed_proj_dim=h)
        cls = tr.OPTForCausalLM
    config.use_cache = False
    with slapo.init_empty_weights():
        model = cls(config)
    return config, model


def train(args):
    on_gpu = args.device == "cuda"
    if not dist.is_initialized():
        rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl" if on_gpu else "gloo", rank=rank, world_size=world)
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    device = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")

    # topology: pipeline stages x tensor-parallel ranks, the rest is data parallel
    topology, tp_group = utils.create_dist_group_for_pipeline(args.pmp, args.tmp)
    mesh = topology
    sp = args.sequence_parallel and args.tmp > 1
    slapo.set_random_seed(args.seed, dp_rank=mesh.dp_rank, pp_rank=mesh.pp_rank,
                          tp_rank=mesh.tp_rank, always_enable_tp_seed=sp)

    config, model = hf_model(args)
    utils.logger.info("%s: %.1f M parameters, %d stage(s) x TP %d x DP %d", args.family,
                      sum(p.numel() for p in model.parameters()) / 1e6, args.pmp, args.tmp,
                      mesh.dp_size, ranks=0)

    # the family's recipe; with pipeline stages it traces the model on the micro-batch's shapes
    sch_config = dict(model_config=config, group=mesh.schedule_group, ckpt_ratio=args.checkpoint,
                      bf16=args.dtype == "bf16", fp16=args.dtype == "fp16",
                      attn_op_name="auto" if on_gpu else "reference")
    seq2seq = args.family == "t5"
    if args.family not in ("albert", "t5"):
        sch_config.update(sequence_parallel=sp, sequence_parallel_axis=0)
    if args.pmp > 1:
        shapes = {"batch_size": args.micro_batch_size, "seq_len": args.seq_len}
        if seq2seq:
            shapes = {"input_shapes": {
                "input_ids": (args.micro_batch_size, args.seq_len),
                "decoder_input_ids": (args.micro_batch_size, args.dec_seq_len)}}
        sch_config.update(
            pipeline_cuts=utils.generate_pipeline_cuts(args.layers, args.pmp,
                                                       is_encoder_decoder=seq2seq),
            trace_config=shapes)
    sch = slapo.model_schedule.apply_schedule(model, args.family, **sch_config)

    kind = "seq2seq" if seq2seq else (
        "causal" if args.family in ("gpt2", "gpt_neo", "opt") else "mlm")
    loss_of = {"causal": causal_lm_loss, "mlm": mlm_loss, "seq2seq": seq2seq_loss}[kind]

    def loss_fn(out, labels):
        logits = out["logits"] if isinstance(out, dict) else out.logits
        return loss_of(logits, labels, tp_group, args.tmp > 1)

    micro_batches = max(1, args.batch_size // args.micro_batch_size)
    ds_config = utils.get_ds_config(args.batch_size * mesh.dp_size, args.micro_batch_size,
                                    fp16=args.dtype == "fp16", bf16=args.dtype == "bf16",
                                    zero_stage=1 if mesh.dp_size > 1 else 0,
                                    desc=f"{args.family} with pipeline" if args.pmp > 1 else args.family,
                                    sequence_parallel=sp)
    if args.pmp == 1:
        ds_config["gradient_accumulation_steps"] = micro_batches
    # weights are created here, shard by shard, on the device (the model was built empty)
    engine, _ = slapo.build(sch, target=args.target, config=ds_config,
                            **({"mesh": mesh} if args.target == "native" else {"topology": topology}),
                            loss_fn=loss_fn, init_weights=model._init_weights, device=device,
                            **({"num_micro_batches": micro_batches} if args.pmp > 1 else {}))

    # synthetic tokens, another stream per data-parallel replica
    gen = torch.Generator().manual_seed(args.seed + mesh.dp_rank)
    per_call = args.batch_size if args.pmp > 1 else args.micro_batch_size
    calls_per_step = 1 if args.pmp > 1 else micro_batches

    def batches():
        while True:
            ids = torch.randint(0, args.vocab, (per_call, args.seq_len), generator=gen)
            if kind == "seq2seq":
                dec = torch.randint(0, args.vocab, (per_call, args.dec_seq_len), generator=gen)
                yield {"input_ids": ids, "decoder_input_ids": dec}, dec.clone()
                continue
            if kind == "causal":
                labels = ids.clone()
            else:
                labels = torch.full_like(ids, -100)
                pick = torch.rand(ids.shape, generator=gen) < 0.15
                labels[pick] = ids[pick]
            yield (ids,), labels

    losses = utils.train_with_engine(engine, batches(), steps=args.iter_nums * calls_per_step,
                                     device=device)
    return losses[calls_per_step - 1::calls_per_step]        # one loss per optimizer step


if __name__ == "__main__":
    train(parse_args())
    if dist.is_initialized():
        dist.destroy_process_group()
