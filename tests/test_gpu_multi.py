"""Two-GPU check of the KV-sharded decode: NCCL all-gather + merge against the fused NVLink exchange +
merge, both against the oracle.  Skipped unless two CUDA devices are visible."""
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
    import ctypes as C
    import torch
    import torch.distributed as dist
    from grilly_next import cabi
    from grilly_next.parallel import CudaShardOps, ShardedDecoder, shard_range, torch_stream_handle
    from gpu_helpers import PagedCache
    from oracle import attention_oracle as orc
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dev = cabi.Device(rank)
    cabi.check(dev.L.grl_device_use_stream(dev.h, torch_stream_handle(torch)))
    B, Hq, Hkv, D, T = 1, 32, 8, 128, 1000
    rng = np.random.default_rng(7)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, T, Hkv, D), dtype=np.float32)
    lo, hi = shard_range(T, world, rank)
    pc = PagedCache(dev, B, Hkv, D, hi - lo + 64, dtype=cabi.BF16)
    pc.append(k[:, lo:hi], v[:, lo:hi])
    ops = CudaShardOps(cabi, dev, pc.layout(), Hq, hi - lo, torch)
    dec = ShardedDecoder(dist, ops, lambda n, m: torch.empty((n, m), dtype=torch.float32, device="cuda"))
    errs = []
    for step in range(3):                       # NCCL path
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        out = dec.step(torch.from_numpy(q).cuda()).cpu().numpy()
        want = orc.gqa_decode_attention(q, orc.round_bf16(k), orc.round_bf16(v), Hq, Hkv, D)
        errs.append(float(np.abs(out - want).max()))
    fused = ops.setup_p2p(dist)
    assert ops.one_launch
    for step in range(10):
        # several steps each (both inbox parities): first the exchange fused with the merge kernel, then
        # decode + exchange + merge as one launch; both share the inboxes and the step counter
        ops.one_launch = step >= 5
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        out = dec.step(torch.from_numpy(q).cuda()).cpu().numpy()
        want = orc.gqa_decode_attention(q, orc.round_bf16(k), orc.round_bf16(v), Hq, Hkv, D)
        errs.append(float(np.abs(out - want).max()))
    # the flag-and-fence form of the exchange kernel (the default above is the {value, step} pair form)
    ops2 = CudaShardOps(cabi, dev, pc.layout(), Hq, hi - lo, torch)
    assert ops2.setup_p2p(dist, one_launch=False, low_latency=False) == fused
    dec2 = ShardedDecoder(dist, ops2, lambda n, m: torch.empty((n, m), dtype=torch.float32, device="cuda"))
    for step in range(5):
        q = rng.standard_normal((B, 1, Hq, D), dtype=np.float32)
        out = dec2.step(torch.from_numpy(q).cuda()).cpu().numpy()
        want = orc.gqa_decode_attention(q, orc.round_bf16(k), orc.round_bf16(v), Hq, Hkv, D)
        errs.append(float(np.abs(out - want).max()))
    dev.sync()
    np.save(os.path.join(result_dir, f"res{rank}.npy"), np.array(errs + [1.0 if fused else 0.0]))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_decode_two_gpus(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = np.load(tmp_path / f"res{r}.npy")
        assert np.all(res[:-1] <= 5e-3), res
