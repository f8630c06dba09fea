"""The multi-GPU partitioning on CPU ranks: two gloo processes each compute
their shard (with the CPU oracle standing in for the kernel) and the
all-gather of column-major C blocks / attention slabs reproduces the unsharded
result."""
import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_arithmetic():
    sh = importlib.import_module("7_b200.sharding")
    for n, world in ((8192, 8), (28672, 3), (48, 2), (16, 4)):
        spans = [sh.column_shard(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(b % 16 == 0 and e % 16 == 0 for b, e in spans)
    assert [sh.head_shard(512, 8, r) for r in (0, 7)] == [(0, 64), (448, 512)]
    assert [sh.head_shard(5, 2, r) for r in (0, 1)] == [(0, 3), (3, 5)]
    with pytest.raises(ValueError):
        sh.column_shard(100, 2, 0)
    with pytest.raises(ValueError):
        sh.head_shard(8, 2, 2)


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    from oracle import oracle
    sh = importlib.import_module("7_b200.sharding")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # GEMM: A replicated, B split by rows (= C columns), column-major C blocks gathered
        M, N, K = 64, 64, 96
        a = oracle.make_input_bits(M, K, oracle.BF16, 3, 0, oracle.MODE_LCG)
        b = oracle.make_input_bits(N, K, oracle.BF16, 3, 1, oracle.MODE_LCG)
        n0, n1 = sh.column_shard(N, world, rank)
        c_block = oracle.gemm_ref(a, b[n0:n1], oracle.BF16)                 # [M, n1-n0]
        local = torch.from_numpy(np.ascontiguousarray(c_block.T))           # column-major block: [n1-n0, M]
        full_cm = sh.all_gather_shards(local, dist).reshape(N, M).numpy()   # n*M + m
        assert np.array_equal(full_cm.T, oracle.gemm_ref(a, b, oracle.BF16))
        # the replicated A reaches every rank as row blocks exchanged by an all-gather
        a_t = torch.from_numpy(a.view(np.uint8).reshape(M, 2 * K))  # 16-bit patterns as bytes: gloo has no int16
        r0, r1 = sh.row_shard(M, world, rank)
        assert (r1 - r0) * world == M
        a_rows = sh.all_gather_shards(a_t[r0:r1], dist).reshape(M, 2 * K)
        assert torch.equal(a_rows, a_t)
        # attention: (batch*head) slabs
        BH, S, D = 4, 32, 128
        q, k, v = (oracle.baseline_inputs((BH, S, D), "normal", 7, i, oracle.BF16) for i in range(3))
        h0, h1 = sh.head_shard(BH, world, rank)
        o = oracle.fa_ref(q[h0:h1], k[h0:h1], v[h0:h1], oracle.BF16, 0.1, causal=True)
        full = sh.all_gather_shards(torch.from_numpy(o), dist).reshape(BH, S, D).numpy()
        assert np.array_equal(full, oracle.fa_ref(q, k, v, oracle.BF16, 0.1, causal=True))
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_gather(tmp_path):
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")
