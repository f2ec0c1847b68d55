"""Tensor-parallel Newton-Schulz on two GPUs: the Gram all-reduce fused into the SYRK epilogue against exact integer
sums, against the NCCL all-reduce path and against single-device Newton-Schulz on the gathered matrix."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
from emerging_optimizers_b200.utils import fp32_matmul_precision


pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _randn(*shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def _worker(rank, world, port, out, multicast="1"):
    # EO_MULTICAST=0 keeps the exchange on plain peer loads / stores (what a box without NVLS support runs)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", EO_MULTICAST=multicast)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    group = dist.group.WORLD
    from emerging_optimizers_b200.distributed import tensor_parallel as tp

    res = {}
    # 1. the exchange alone, integer-valued shards: every partial and the sum are exact in bf16
    for m, k, tile_m in ((128, 64, 0), (200, 64, 0), (1000, 64, 0), (512, 128, 0), (1000, 64, 256), (512, 128, 256),
                         (264, 64, 256)):  # fmt: skip
        nat.set_option("gemm_tile_m", tile_m)  # 256: the pushing kernel runs with 256-row tiles (two inbox tiles each)
        g = torch.Generator(device="cpu").manual_seed(100 + m)
        full = torch.randint(-1, 2, (m, world * k), generator=g).to(torch.bfloat16)
        for trans in (False, True):
            shard = full[:, rank * k : (rank + 1) * k].contiguous().to(dev)
            if trans:
                shard = shard.T.contiguous().T
            for rep in range(2):  # second call reuses inbox, flags and Gram buffer with the next sequence number
                a = tp.fused_gram(shard, group).clone()
            want = (full.float() @ full.float().T).to(dev)
            res[f"gram.{m}.{int(trans)}.{tile_m}"] = bool(torch.equal(a.float(), want)) and bool(torch.equal(a, a.T))
    nat.set_option("gemm_tile_m", 0)
    # 2. full tensor-parallel Newton-Schulz, both partition dims, fused exchange vs NCCL vs single device
    for shape, pdim in (((512, 2048), 1), ((2048, 512), 0), ((256, 1024), 1)):
        x = _randn(*shape, seed=7)
        shard = x.chunk(world, dim=pdim)[rank].contiguous().to(dev)
        with fp32_matmul_precision("medium"):
            y_fused = muon_utils.newton_schulz_tp(shard, 5, "quintic", group, partition_dim=pdim,
                                                  tp_mode="distributed", use_syrk=True)  # fmt: skip
            os.environ["EO_TP_GRAM"] = "nccl"
            y_nccl = muon_utils.newton_schulz_tp(shard, 5, "quintic", group, partition_dim=pdim,
                                                 tp_mode="distributed", use_syrk=True)  # fmt: skip
            os.environ["EO_TP_GRAM"] = "auto"
            y_full = muon_utils.newton_schulz(x.to(dev), 5, "quintic", use_syrk=True)
        ref = y_full.chunk(world, dim=pdim)[rank]
        res[f"ns.{shape}.{pdim}"] = (_rel(y_fused, ref), _rel(y_nccl, ref), tuple(y_fused.shape) == tuple(shard.shape))
    # 3. S = b A + c A^2 computed in row blocks per rank and all-gathered: same bits as the redundant computation
    x = _randn(512, 2048, seed=9)
    shard = x.chunk(world, dim=1)[rank].contiguous().to(dev)
    with fp32_matmul_precision("medium"):
        y_plain = muon_utils.newton_schulz_tp(shard, 5, "quintic", group, partition_dim=1, tp_mode="distributed", use_syrk=True)
        saved = muon_utils.TP_SHARD_GRAM_POLY_MIN_WORLD
        muon_utils.TP_SHARD_GRAM_POLY_MIN_WORLD = 2
        try:
            y_sharded = muon_utils.newton_schulz_tp(shard, 5, "quintic", group, partition_dim=1, tp_mode="distributed", use_syrk=True)
        finally:
            muon_utils.TP_SHARD_GRAM_POLY_MIN_WORLD = saved
    res["sharded_poly"] = bool(torch.equal(y_plain, y_sharded))
    res["multicast"] = bool(tp._exchange(512, group, dev).multicast)
    torch.cuda.synchronize()
    res["status"] = nat.read_device_status(dev)
    out[rank] = res
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("multicast", ["1", "0"])
def test_fused_gram_exchange_and_tp_newton_schulz_two_gpus(multicast):
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out, multicast), nprocs=world, join=True)
        results = dict(out)
    for rank in range(world):
        res = results[rank]
        assert res["status"] == 0
        if multicast == "0":
            assert not res["multicast"]
        for key, val in res.items():
            if key.startswith("gram."):
                assert val, (rank, key)
            elif key == "sharded_poly":
                assert val, (rank, key)
            elif key.startswith("ns."):
                err_fused, err_nccl, shape_ok = val
                assert shape_ok
                # bf16 path tolerance against single-device Newton-Schulz on the gathered matrix
                assert err_fused <= 2e-2 and err_nccl <= 2e-2, (rank, key, val)
