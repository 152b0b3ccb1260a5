"""Host-side sharding logic, including a world_size-2 gloo run of the rank protocol bench.py uses."""
import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np

from tensorrt_b200.sharding import shard_by_tokens, shard_even

ROOT = Path(__file__).resolve().parents[1]


def test_shard_even_covers_batch():
    for batch in (0, 1, 7, 64, 65):
        for ws in (1, 2, 4, 8):
            parts = [list(shard_even(batch, ws, r)) for r in range(ws)]
            assert sum(parts, []) == list(range(batch))
            assert max(map(len, parts)) - min(map(len, parts)) <= 1
    assert [len(shard_even(64, n, 0)) for n in (1, 2, 4, 8)] == [64, 32, 16, 8]


def test_shard_by_tokens_balances():
    rng = np.random.default_rng(1)
    lengths = rng.integers(32, 385, size=256)
    for ws in (1, 2, 4, 8):
        parts = shard_by_tokens(lengths, ws)
        assert sorted(sum(parts, [])) == list(range(256))
        loads = [int(lengths[p].sum()) for p in parts]
        assert max(loads) - min(loads) <= 384  # LPT bound: at most one longest item apart
    assert shard_by_tokens([], 2) == [[], []]
    assert shard_by_tokens([5], 2) == [[0], []]


def test_two_rank_gloo_protocol(tmp_path):
    """Two CPU ranks shard a batch, 'process' their shard, and agree on max-over-ranks time and total count
    with the same reductions bench.py uses."""
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent("""
        import os, sys
        sys.path.insert(0, %r)
        import torch, torch.distributed as dist
        from tensorrt_b200.sharding import shard_even
        dist.init_process_group("gloo")
        r, ws = dist.get_rank(), dist.get_world_size()
        mine = shard_even(64, ws, r)
        ms = torch.tensor([10.0 + 5 * r], dtype=torch.float64)
        n = torch.tensor([len(mine)], dtype=torch.int64)
        dist.barrier()
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(n, op=dist.ReduceOp.SUM)
        assert ms.item() == 15.0 and n.item() == 64, (ms, n)
        if r == 0:
            print("OK", ms.item(), n.item())
        dist.destroy_process_group()
    """ % str(ROOT)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "OK 15.0 64" in r.stdout
