"""Static-parallel training entry: one (dp, tp, pp) strategy for the whole run.

    torchrun --nproc-per-node 8 -m hotspa_ae_b200.train.llama_static_parallel --model_size 7b --dp 2 --tp 2 --pp 2 \\
        --zero --bf16 --seq_length 4096 --global_batch_size 64 --fixed_len 4096 --steps 10

Same options as ``llama_hot_switch`` plus ``--dp/--tp/--pp``; it is that entry point with a single bucket
(reference: hotspa/scripts/llama_static_parallel.sh, hotspa/llama_hot_switch.py test_static).
"""
from __future__ import annotations

import sys

from . import llama_hot_switch as H


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    vals = {"--dp": "1", "--tp": "1", "--pp": "1"}
    rest, i = [], 0
    while i < len(argv):
        if argv[i] in vals:
            vals[argv[i]] = argv[i + 1]
            i += 2
        else:
            rest.append(argv[i])
            i += 1
    seq = "4096"
    if "--seq_length" in rest:
        seq = rest[rest.index("--seq_length") + 1]
    elif "-s" in rest:
        seq = rest[rest.index("-s") + 1]
    rest += ["--strategies", f"{vals['--dp']},{vals['--tp']},{vals['--pp']}", "--bucket_sizes", f"{seq} 0"]
    return H.main(rest)


if __name__ == "__main__":
    sys.exit(main())
