"""The N > 1 host path on CPU: lane assignment, key-range splitting and the split-KV record
exchange over a world-size-2 gloo group, with the CPU oracle standing in for the device kernels."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from tatara_b200 import sharding  # noqa: E402


def test_assign_lanes_partitions_and_balances():
    rng = np.random.default_rng(0)
    contexts = [int(c) for c in rng.integers(4096, 32769, size=32)]
    for world in (1, 2, 4, 8):
        owned = sharding.assign_lanes(contexts, world)
        flat = sorted(l for r in owned for l in r)
        assert flat == list(range(32))
        loads = [sum(contexts[l] for l in r) for r in owned]
        assert max(loads) - min(loads) <= max(contexts)
        assert owned == sharding.assign_lanes(contexts, world)   # deterministic


def test_split_kv_ranges_cover_exactly():
    for n in (1, 15, 16, 17, 4097, 262144, 262145):
        for world in (1, 2, 4, 8):
            ranges = sharding.split_kv_ranges(n, world)
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            for (b0, e0), (b1, e1) in zip(ranges, ranges[1:]):
                assert e0 == b1 and b0 <= e0
            assert all(b % 16 == 0 or b == n for b, _ in ranges)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_keys, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from tatara_b200 import synthetic as syn
    rng = np.random.default_rng(123)                      # every rank builds the same lane
    keys, values = syn.attn_cache(rng, n_keys, n_keys)
    q, gate = syn.attn_query(rng, np.array([n_keys - 1]))
    begin, end = sharding.split_kv_ranges(n_keys, world)[rank]

    def partial():
        if begin == end:
            rec = np.zeros((16, 258), np.float32)
            rec[:, 256] = -np.inf
            return torch.from_numpy(rec)
        return torch.from_numpy(oracle.attn_partial(q[0], keys, values, begin, end, n_keys))

    out = {}

    def combine(gathered):
        rec = np.ascontiguousarray(gathered.numpy().transpose(1, 0, 2))   # [head][rank][258]
        out["bits"] = oracle.attn_combine(rec, gate[0])

    gathered = torch.zeros((world, 16, 258))
    sharding.split_kv_decode(dist, world, partial, gathered, combine)
    whole = oracle.attn_decode(q[0], gate[0], keys, values, n_keys - 1, n_keys)
    err = np.max(np.abs(syn.from_bf16(out["bits"]) - syn.from_bf16(whole)))
    # every rank must hold the same merged bits
    mine = torch.from_numpy(out["bits"].astype(np.int32))
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    same = all(torch.equal(everyone[0], e) for e in everyone)
    if rank == 0:
        np.save(result_path, np.array([err, float(same)]))
    dist.destroy_process_group()


@pytest.mark.parametrize("n_keys", [1000, 5])
def test_split_kv_exchange_world2_gloo(tmp_path, n_keys):
    world, port = 2, _free_port()
    result = str(tmp_path / "result.npy")
    mp.spawn(_worker, args=(world, port, n_keys, result), nprocs=world, join=True)
    err, same = np.load(result)
    assert same == 1.0
    assert err <= 2e-2
