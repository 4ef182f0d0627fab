"""Two-GPU check of the KV-sharded decode against the oracle, every form of the exchange: NCCL all-gather +
merge through grl_group_*, the exchange kernel in its flag and {value, step} forms, the exchange inside the
decode kernel, and the op layer's grilly_core.sharded_decode_step.  One process per GPU, meeting over the
package's TcpChannel.  Skipped unless two CUDA devices are visible."""
import ctypes as C
import multiprocessing
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result_dir):
    for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "grilly-next_b200", "python")):
        sys.path.insert(0, p)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["GRILLY_GPU_INDEX"] = str(rank)
    from grilly_next import cabi
    from grilly_next.parallel import CudaShardOps, ShardedDecoder, TcpChannel, shard_range
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc
    ch = TcpChannel(rank, world, "127.0.0.1", port)
    dev = cabi.Device(rank)
    B, Hq, Hkv, D, T = 1, 32, 8, 128, 1000
    rng = np.random.default_rng(7)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    lo, hi = shard_range(T, world, rank)
    pc = PagedCache(dev, B, Hkv, D, hi - lo + 64, dtype=cabi.BF16)
    pc.append(k[:, lo:hi], v[:, lo:hi])
    kb, vb = orc.round_bf16(k), orc.round_bf16(v)
    errs = []

    def run(dec, ops, steps):
        for _ in range(steps):
            q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
            qd = dev.upload(q)
            out_ptr = dec.step(qd)
            dev.sync()
            out = dev.download(out_ptr, (B, 1, Hq, D), np.float32)
            dev.free(qd)
            errs.append(float(np.abs(out - orc.gqa_decode_attention(q, kb, vb, Hq, Hkv, D)).max()))

    # NCCL all-gather + merge behind the C ABI
    ops = CudaShardOps(cabi, dev, pc.layout(), Hq, hi - lo)
    ops.setup_nccl(ch)
    dec = ShardedDecoder(ch, ops)
    run(dec, ops, 3)
    # the {value, step} pair form: first the exchange + merge kernel, then decode + exchange + merge as one launch;
    # several steps each (both inbox parities); both share the inboxes and the step counter
    fused = ops.setup_p2p(ch)
    assert ops.one_launch
    for one_launch in (False, True):
        ops.one_launch = one_launch
        run(dec, ops, 5)
    # the flag-and-fence form of the exchange kernel
    ops2 = CudaShardOps(cabi, dev, pc.layout(), Hq, hi - lo)
    assert ops2.setup_p2p(ch, one_launch=False, low_latency=False) == fused
    run(ShardedDecoder(ch, ops2), ops2, 5)
    ops.close()
    dev.sync()

    # the op layer: grilly_core.ShardGroup + sharded_decode_step on host arrays
    import grilly_core
    ctx = grilly_core.Device()
    raw = ch.all_gather_bytes(grilly_core.shard_group_unique_id() if rank == 0 else b"")[0]
    group = grilly_core.ShardGroup(ctx, raw, rank, world)
    assert (group.rank, group.world) == (rank, world)
    assert tuple(grilly_core.shard_range(T, world, rank)) == (lo, hi)
    kv = grilly_core.create_kv_cache(ctx, num_heads=Hkv, head_dim=D, compression_ratio=1, max_cache_tokens=hi - lo + 64,
                                     use_h2o=False, batch_size=B, page_tokens=64, dtype="bf16")
    grilly_core.kv_cache_append(ctx, kv, k[:, lo:hi], v[:, lo:hi])
    for _ in range(2):
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        out = grilly_core.sharded_decode_step(ctx, kv, group, q)
        errs.append(float(np.abs(out - orc.gqa_decode_attention(q, kb, vb, Hq, Hkv, D)).max()))
    ch.barrier()
    del group
    grilly_core.destroy_kv_cache(ctx, kv)
    np.save(os.path.join(result_dir, f"res{rank}.npy"), np.array(errs + [1.0 if fused else 0.0]))
    ch.barrier()
    dev.close()
    ch.close()


def test_sharded_decode_two_gpus(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "grilly-next_b200", "python"))
    from grilly_next import cabi
    n = C.c_int()
    cabi.lib().grl_device_count(C.byref(n))
    if n.value < 2:
        pytest.skip("needs two GPUs")
    ctx = multiprocessing.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(2):
        res = np.load(tmp_path / f"res{r}.npy")
        assert len(res) == 3 + 10 + 5 + 2 + 1
        assert res[-1] == 1.0, "peer inboxes could not be mapped"
        assert np.all(res[:-1] <= 5e-3), res
