"""Launcher shared by the multi-process CPU tests: tests/<script> on `world` gloo ranks under torchrun."""
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def torchrun_cpu(script, world, args=(), marker=None, timeout=900):
    """The rendezvous port is picked by binding port 0 and releasing it, so another process can take it before
    torchrun binds: a failed launch is repeated once on a fresh port, and the output of both attempts is shown if the
    second one fails too.  Returns the output of the successful run."""
    env = dict(os.environ, OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    outputs = []
    for _ in range(2):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(HERE, script),
               *[str(a) for a in args]]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, env=env)
        if proc.returncode == 0 and (marker is None or marker in proc.stdout):
            return proc.stdout
        outputs.append(proc.stdout[-3000:])
    raise AssertionError("\n======== second attempt ========\n".join(outputs))
