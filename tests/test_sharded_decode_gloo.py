"""World-size-2 (and 3) runs of the KV-sharded decode host logic on CPU: sharding arithmetic, the
exchange of partials and the merge order, with numpy stand-ins (the oracle) for the kernels.  The
ranks meet once over torch.distributed's gloo backend (wrapped as a host channel) and once over the
package's own TcpChannel.  The CUDA kernels themselves are covered by the GPU tests."""
import multiprocessing
import os
import pickle
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class GlooChannel:
    """torch.distributed (gloo) as the host channel: a host-memory stand-in for the ranks' meeting point."""

    def __init__(self, dist):
        self.dist, self.rank, self.world = dist, dist.get_rank(), dist.get_world_size()

    def all_gather_bytes(self, payload):
        out = [None] * self.world
        self.dist.all_gather_object(out, bytes(payload))
        return out

    def barrier(self):
        self.dist.barrier()


def _run_rank(channel, T, result_dir):
    from grilly_next.parallel import ShardedDecoder, partial_floats, shard_range
    from oracle import attention_oracle as orc
    rank, world = channel.rank, channel.world
    B, Hq, Hkv, D = 2, 8, 2, 32
    rng = np.random.default_rng(5)                      # same data on every rank
    q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    lo, hi = shard_range(T, world, rank)
    g, scale, rows = Hq // Hkv, 1.0 / np.sqrt(D), B * Hq

    class NumpyOps:                                      # what the kernels compute, in numpy
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
            return np.concatenate([o.reshape(-1), m, l])

        def allgather_merge(self, part):                 # the collective form: all-gather, then merge in rank order
            parts = [np.frombuffer(b, np.float32) for b in channel.all_gather_bytes(part.astype(np.float32).tobytes())]
            a = np.stack(parts)
            o = a[:, :rows * D].reshape(world, rows, D); m = a[:, rows * D:rows * D + rows]; l = a[:, rows * D + rows:]
            return orc.lse_merge(o, m, l).reshape(B, 1, Hq, D)

    dec = ShardedDecoder(channel, NumpyOps())
    out = dec.step(q)
    assert partial_floats(rows, D) == rows * (D + 2)
    want = orc.gqa_decode_attention(q, k, v, Hq, Hkv, D)
    np.save(os.path.join(result_dir, f"err{rank}.npy"), np.abs(out - want).max())
    channel.barrier()


def _paths():
    for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "grilly-next_b200", "python")):
        sys.path.insert(0, p)


def _gloo_worker(rank, world, port, T, result_dir):
    _paths()
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    _run_rank(GlooChannel(dist), T, result_dir)
    dist.destroy_process_group()


def _tcp_worker(rank, world, port, T, result_dir):
    _paths()
    from grilly_next.parallel import TcpChannel, max_over_ranks
    ch = TcpChannel(rank, world, "127.0.0.1", port)
    assert ch.all_gather_bytes(pickle.dumps(rank * 7)) == [pickle.dumps(r * 7) for r in range(world)]
    assert max_over_ranks(ch, float(rank)) == float(world - 1)
    _run_rank(ch, T, result_dir)
    ch.close()


@pytest.mark.parametrize("world,T", [(2, 257), (3, 2), (2, 1)])
def test_sharded_decode_over_gloo(tmp_path, world, T):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_gloo_worker, args=(world, port, T, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) <= 2e-6


@pytest.mark.parametrize("world,T", [(2, 257), (4, 9)])
def test_sharded_decode_over_tcp_channel(tmp_path, world, T):
    ctx = multiprocessing.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_tcp_worker, args=(r, world, port, T, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
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


def test_package_needs_no_framework():
    """The product path is the C ABI: nothing under the package imports torch."""
    pkg = os.path.join(ROOT, "grilly-next_b200")
    for d, _, fs in os.walk(pkg):
        for f in fs:
            if f.endswith((".py", ".cpp", ".h", ".cu", ".cuh")):
                text = open(os.path.join(d, f), errors="ignore").read()
                assert "import torch" not in text and "#include <torch" not in text, os.path.join(d, f)
