"""Sequence-sharded decode on two GPUs (skipped where fewer are visible): the fused
peer-store exchange and the NCCL all-gather variant both reproduce the oracle."""

import math
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import oracle
    from probjax_b200 import dist as pjd

    c = oracle.make_config(4, B=3, cap=3000)
    c["kv_lengths"][0] = 7  # shorter than a page: one rank holds nothing of this sequence
    page = 128
    kl = pjd.shard_cache(c["k"], rank, world, page).to(dev)
    vl = pjd.shard_cache(c["v"], rank, world, page).to(dev)
    want, want_lse = oracle.xla_attention(c["q"], c["k"], c["v"], kv_lengths=c["kv_lengths"], sm_scale=c["sm_scale"],
                                          return_lse=True)
    res = {}
    for name, dec in (("fused", pjd.FusedShardedDecoder(c["q"].to(dev), kl, vl, c["kv_lengths"], page=page, sm_scale=c["sm_scale"])),
                      ("nccl", pjd.ShardedDecoder(c["q"].to(dev), kl, vl, c["kv_lengths"], page=page, sm_scale=c["sm_scale"]))):
        for _ in range(3):  # several steps: the exchange buffers alternate
            o, lse = dec(return_lse=True)
        torch.cuda.synchronize(dev)
        if name == "fused":
            dec.check_status()
        res[name] = (float((o.float().cpu() - want.float()).abs().max()), float((lse.cpu() - want_lse).abs().max()))
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_decode_two_gpus(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(os.path.join(str(tmp_path), f"r{r}.pt"))
        for name, (err, err_lse) in res.items():
            assert err <= 2e-2 and err_lse <= 1e-3, (name, err, err_lse)
