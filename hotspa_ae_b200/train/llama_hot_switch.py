"""Command-line training entry: Llama with parallelism hot switching (or one static strategy).

    torchrun --nproc-per-node 8 -m hotspa_ae_b200.train.llama_hot_switch --model_size 7b \\
        --bucket_sizes "32768 16384 4096 0" --strategies "1,4,2 2,2,2 8,1,1" --zero --bf16 \\
        --global_tokens 262144 --steps 10

``--strategies`` lists one "dp,tp,pp" per bucket, longest bucket first (the first one is the home strategy).
``--ds_parallel_config`` takes strategy JSON files instead, in the reference's order (home first, then the
strategy of the shortest bucket ... the strategy of the second-longest bucket).  One strategy and two bounds
give static-parallel training.  Data is synthetic (lognormal lengths, uniform token ids) unless ``--json_file``
names a jsonl file with a ``--json_key`` text field and a vocab/merges pair for the GPT-2 BPE tokenizer.
Reference entry points: hotspa/llama_hot_switch.py:489-594, hotspa/scripts/llama_hot_switch.sh,
hotspa/scripts/llama_static_parallel.sh.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

from ..parallel import mesh as M
from ..utils import data as D
from .trainer import build_trainer_from_args, timed_steps


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model_size", default="7b", help="tiny | 3b | 7b | 13b | 32b")
    ap.add_argument("--hot_switch", action="store_true", help="accepted for compatibility: several strategies switch")
    ap.add_argument("--strategies", default="1,1,1", help='"dp,tp,pp" per bucket, longest bucket first')
    ap.add_argument("--reference_order", action="store_true",
                    help="--strategies is in the reference's order (home, shortest ... second longest)")
    ap.add_argument("--ds_parallel_config", default="", help="comma/space separated strategy JSON files")
    ap.add_argument("--num_strategy", type=int, default=0, help="accepted for compatibility")
    ap.add_argument("--bucket_sizes", default="32768 0")
    ap.add_argument("--zero", action="store_true", help="shard optimizer state over data-parallel ranks (ZeRO-1)")
    ap.add_argument("--global_tokens", type=int, default=0, help="synthetic tokens per step (whole job)")
    ap.add_argument("--fixed_len", type=int, default=0,
                    help="synthetic data: global_batch_size sequences of exactly this length per step")
    ap.add_argument("--micro_batch_tokens", type=int, default=0,
                    help="token budget of a micro-batch (0: one packed row of the bucket's length per micro-batch)")
    ap.add_argument("--global_batch_size", type=int, default=64, help="sequences per step when reading a dataset")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("-e", "--epochs", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--adam_weight_decay", type=float, default=0.0)
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--no_recompute", action="store_true")
    ap.add_argument("--keep_activations", default=None,
                    help="blocks per rank that keep their activations although blocks recompute: one count, or one "
                         "per strategy (\"16,16,18\")")
    ap.add_argument("--switch_mode", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--vocab_size", type=int, default=0)
    ap.add_argument("--hidden_size", type=int, default=0)
    ap.add_argument("--ffn_hidden_size", type=int, default=0)
    ap.add_argument("--num_hidden_layers", type=int, default=0)
    ap.add_argument("-a", "--num_attention_heads", type=int, default=0)
    ap.add_argument("-s", "--seq_length", type=int, default=0, help="maximum sequence length (default: first bucket)")
    ap.add_argument("--json_file", default="")
    ap.add_argument("--json_key", default="content")
    ap.add_argument("--vocab_file", default="")
    ap.add_argument("--merge_file", default="")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--log_file", default="", help="append one JSON line per step (rank 0)")
    ap.add_argument("--save_checkpoint", default="", help="directory to write a checkpoint into after training")
    ap.add_argument("--load_checkpoint", default="", help="directory (or .bin file) to load weights from")
    ap.add_argument("--use_flash_attn", action="store_true", help="accepted for compatibility (always on)")
    ap.add_argument("--no_sequence_parallel", action="store_true",
                    help="tensor parallelism with all-reduce instead of Megatron sequence parallelism")
    ap.add_argument("--run_memory_experiment", action="store_true",
                    help="run the first step only and write this rank's memory figures to --memory_file")
    ap.add_argument("--memory_file", default="", help="result file of --run_memory_experiment (JSON)")
    ap.add_argument("--test_func", action="store_true", help="accepted for compatibility (unused by the reference too)")
    ap.add_argument("--micro_batch_size", type=int, default=1,
                    help="accepted for compatibility: micro-batches are packed rows / token budgets here")
    ap.add_argument("--dataset", default="", help="dataset name, for log lines only")
    ap.add_argument("--hidden_act", default="silu", help="accepted for compatibility: the Llama MLP is SwiGLU")
    ap.add_argument("--dropout_prob", type=float, default=0.0, help="accepted for compatibility: Llama has no dropout")
    return ap.parse_args(argv)


def memory_experiment(trainer, first_batch, path: str) -> dict:
    """One step, then this rank's memory: allocator peaks, device usage as the driver library reports it (reference:
    --run_memory_experiment with HETU_MEMORY_LOG_FILE, hotspa/llama_hot_switch.py:403-419)."""
    import torch
    from ..utils.profiler import CUDAProfiler
    res = trainer.step(first_batch)
    rec = {"rank": M.mesh().rank, "loss": res.loss, "tokens": res.tokens, "buckets": res.buckets}
    rec.update(CUDAProfiler().memory_info())
    if torch.cuda.is_available():
        st = torch.cuda.memory_stats()
        rec["allocated_peak_mb"] = st["allocated_bytes.all.peak"] / 2**20
        rec["reserved_peak_mb"] = st["reserved_bytes.all.peak"] / 2**20
    if path:
        root, ext = os.path.splitext(path)
        with open(f"{root}_rank{M.mesh().rank}{ext or '.json'}", "w") as f:
            json.dump(rec, f)
    return rec


def batches(args, trainer):
    bounds = [int(x) for x in args.bucket_sizes.split()]
    max_len = args.seq_length or bounds[0]
    vocab = trainer.config.vocab_size
    if args.json_file:
        from ..utils.dataset import LlamaJsonDataset, global_batches
        ds = LlamaJsonDataset(args.json_file, args.json_key, max_len, args.vocab_file, args.merge_file)
        yield from global_batches(ds, args.global_batch_size, args.steps * args.epochs, seed=args.seed)
        return
    world = M.mesh().world_size
    tokens = args.global_tokens or 32768 * world
    if args.fixed_len:
        for i in range(args.steps * args.epochs):
            yield D.synthetic_sequences([args.fixed_len] * args.global_batch_size, vocab, seed=args.seed + i)
        return
    for i in range(args.steps * args.epochs):
        lens = D.lognormal_lengths(tokens, seed=args.seed + i, max_len=max_len)
        yield D.synthetic_sequences(lens, vocab, seed=args.seed + i)


def main(argv=None):
    args = parse_args(argv)
    trainer = build_trainer_from_args(args)
    rank = M.mesh().rank
    if args.load_checkpoint:
        from ..utils.checkpoint import load_checkpoint
        load_checkpoint(trainer.model, args.load_checkpoint, graph=trainer.graph)
    if args.run_memory_experiment:
        rec = memory_experiment(trainer, next(iter(batches(args, trainer))), args.memory_file)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        return 0
    logf = open(args.log_file, "a") if (args.log_file and rank == 0) else None

    def log(msg):
        print(msg, flush=True)

    for i, (res, dt) in enumerate(timed_steps(trainer, batches(args, trainer), log)):
        if logf is not None:
            logf.write(json.dumps({"step": i, "loss": res.loss, "time_s": dt, "tokens": res.tokens,
                                   "tokens_per_s": res.tokens / dt, "buckets": res.buckets}) + "\n")
            logf.flush()
    if args.save_checkpoint:
        from ..utils.checkpoint import save_checkpoint
        save_checkpoint(trainer.model, args.save_checkpoint, graph=trainer.graph)
    if logf is not None:
        logf.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
