"""World-size-2 (and 3) gloo runs of the KV-sharded decode host logic on CPU: sharding arithmetic,
the all-gather of partials and the merge order, with numpy stand-ins (the oracle) for the two
kernels.  The CUDA kernels themselves are covered by the GPU tests."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, T, result_dir):
    for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "grilly-next_b200", "python")):
        sys.path.insert(0, p)
    from grilly_next.parallel import ShardedDecoder, partial_floats, shard_range
    from oracle import attention_oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, Hq, Hkv, D = 2, 8, 2, 32
    rng = np.random.default_rng(5)                      # same data on every rank
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    lo, hi = shard_range(T, world, rank)
    g, scale, rows = Hq // Hkv, 1.0 / np.sqrt(D), B * Hq

    class NumpyOps:                                      # what the two kernels compute, in numpy
        def partial(self, q_):
            o = np.zeros((rows, D), np.float32); m = np.full(rows, -1e30, np.float32); l = np.zeros(rows, np.float32)
            if hi > lo:
                for b in range(B):
                    for h in range(Hq):
                        s = (k[b, lo:hi, h // g] @ q_[b, 0, h]) * scale
                        m[b * Hq + h] = s.max()
                        p = np.exp(s - s.max())
                        l[b * Hq + h] = p.sum()
                        o[b * Hq + h] = p @ v[b, lo:hi, h // g]
            return torch.from_numpy(np.concatenate([o.reshape(-1), m, l]))

        def merge(self, gathered, n_parts):
            a = gathered.numpy().reshape(n_parts, -1)
            o = a[:, :rows * D].reshape(n_parts, rows, D); m = a[:, rows * D:rows * D + rows]; l = a[:, rows * D + rows:]
            return orc.lse_merge(o, m, l).reshape(B, 1, Hq, D)

    dec = ShardedDecoder(dist, NumpyOps(), lambda n, m: torch.empty((n, m), dtype=torch.float32))
    out = dec.step(q)
    assert partial_floats(rows, D) == rows * (D + 2)
    want = orc.gqa_decode_attention(q, k, v, Hq, Hkv, D)
    np.save(os.path.join(result_dir, f"err{rank}.npy"), np.abs(out - want).max())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,T", [(2, 257), (3, 2), (2, 1)])
def test_sharded_decode_over_gloo(tmp_path, world, T):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, T, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) <= 2e-6


def test_shard_ranges_partition_the_sequence():
    sys.path.insert(0, os.path.join(ROOT, "grilly-next_b200", "python"))
    from grilly_next.parallel import owner_of_new_token, shard_range
    for T in (0, 1, 7, 64, 131072, 131075):
        for world in (1, 2, 4, 8):
            r = [shard_range(T, world, g) for g in range(world)]
            assert r[0][0] == 0 and r[-1][1] == T
            assert all(r[i][1] == r[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in r]
            assert max(sizes) - min(sizes) <= 1
    assert owner_of_new_token(8) == 7
