"""The column-sharded mul on two GPUs, one process per GPU over NCCL: every rank computes its column shard and the
epilogue delivers it into every rank's copy of the destination, by stores into the peer's buffer (CUDA IPC mapping) and,
where the platform offers NVLink multicast mappings, by one multimem store per piece; the launch ends with the flag
exchange.  Needs two GPUs (skipped otherwise); the host logic of the sharding is covered on CPU by test_sharding.py."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    import ruy_b200
    import util
    from ruy_b200 import cases, peer
    from ruy_b200.api import Rounding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    stream = torch.cuda.Stream(device=dev)
    results = {}
    with torch.cuda.stream(stream):
        ctx = ruy_b200.Context(rank, stream=stream.cuda_stream)
        rows, depth, cols = 512, 384, 1024                  # 512-column shards: two-CTA tiles, two halves per tile
        shard = cols // world
        case = cases.config3(rows=rows, depth=depth, cols=cols, dst="int8", col_begin=rank * shard, col_count=shard)
        whole = cases.config3(rows=rows, depth=depth, cols=cols, dst="int8")
        want = np.ascontiguousarray(util.run_oracle(whole, Rounding.kReference).T).reshape(-1)   # column-major storage
        nbytes, shard_bytes = rows * cols, rows * shard
        flags = peer.StepFlags(dev)
        modes = {"peer_stores": peer.PeerBuffer(nbytes, dev)}
        try:
            modes["multicast"] = peer.MulticastBuffer(nbytes, dev)
        except Exception as e:                              # no multicast mapping here: the other mode is still checked
            results["multicast"] = f"unavailable: {type(e).__name__}"
        ok = torch.tensor([1 if "multicast" in modes else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok[0]) == 0 and "multicast" in modes:
            modes.pop("multicast").close()
        step = 0
        for name, buf in modes.items():
            full = buf.tensor.view(torch.int8)
            full.zero_()
            mine = full[rank * shard_bytes:(rank + 1) * shard_bytes]
            lhs, rhs, p, d, keep = case.bind(mine, device=dev, rounding=Rounding.kReference)
            stream.synchronize()
            dist.barrier()
            for _ in range(2):                              # twice: the second launch finds the finished-CTA counter rewound
                step += 1
                if name == "multicast":
                    peer.mul_async_multicast(lhs, rhs, p, ctx, d, buf.multicast_ptr + rank * shard_bytes, flags, step)
                else:
                    mirrors = [q + rank * shard_bytes for r_, q in enumerate(buf.ptrs) if r_ != rank]
                    peer.mul_async_mirrored(lhs, rhs, p, ctx, d, mirrors, flags=flags, value=step)
                ctx.sync()                                  # the exchange has told this rank that every shard has landed
                got = full.cpu().numpy()
                results[name] = bool(np.array_equal(got, want))
                dist.barrier()                              # nobody overwrites a buffer that a peer is still reading
        np.save(os.path.join(out_dir, f"rank{rank}.npy"), np.array([f"{k}={v}" for k, v in results.items()]))
        flags.close()
        for buf in modes.values():
            buf.close()
        ctx.close()
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gather_inside_the_launch(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        res = dict(item.split("=", 1) for item in np.load(os.path.join(str(tmp_path), f"rank{rank}.npy")))
        assert res.get("peer_stores") == "True", (rank, res)
        assert res.get("multicast", "True") == "True" or res["multicast"].startswith("unavailable"), (rank, res)
