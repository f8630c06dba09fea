"""The N-column-sharded GEMM on two GPUs, one process per GPU (NCCL): the
blocks gathered three ways -- ncclAllGather after the kernel, peer stores out
of the kernel's epilogue (wave_cuda_gemm_multi_output) and NVLink multicast
stores (wave_cuda_gemm_multicast_output) -- must all leave the oracle's full C
on every rank, the sharded host-buffer call must return each rank's block, and
the (batch, head)-sharded attention must gather its slabs the same three ways.
Skipped on a machine with fewer than two GPUs (the single-GPU tests cover the
epilogue's copy logic with local buffers standing in for peers, and the gloo
test the host arithmetic)."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    from oracle import oracle
    pkg = importlib.import_module("7_b200")
    wc, sh = pkg.wave_cuda, importlib.import_module("7_b200.sharding")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        M, N, K = 1024, 2048, 512
        a = oracle.make_input_bits(M, K, oracle.BF16, 5, 0, oracle.MODE_LCG)
        b = oracle.make_input_bits(N, K, oracle.BF16, 5, 1, oracle.MODE_LCG)
        want = oracle.round_output(oracle.gemm_ref(a, b, oracle.BF16), "bf16")          # [M, N]
        dev = lambda bits: torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()
        n0, n1 = sh.column_shard(N, world, rank, 256)
        da, db = dev(a), dev(b[n0:n1])
        desc = wc.gemm_desc(M, n1 - n0, K, bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4, in_type=wc.BF16,
                            out_type=wc.BF16, out_layout=wc.COL_MAJOR)
        stream = torch.cuda.current_stream().cuda_stream
        as_f32 = lambda t: t.float().cpu().numpy().reshape(N, M).T  # column-major -> [M, N]

        # 1. kernel, then ncclAllGather of the contiguous column-major blocks
        c_block = torch.full(((n1 - n0) * M,), float("nan"), dtype=torch.bfloat16, device="cuda")
        wc.gemm(desc, da.data_ptr(), db.data_ptr(), c_block.data_ptr(), 0, stream)
        full = sh.all_gather_shards(c_block, dist)
        assert np.array_equal(as_f32(full), want)

        # 2. the gather fused into the kernel: peer stores, then multicast stores
        out = sh.PeerMappedOutput((N, M), torch.bfloat16, dist, rank, world)
        offset = n0 * M * 2
        out.local.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        wc.gemm_multi_output(desc, da.data_ptr(), db.data_ptr(), out.block_targets(offset), stream)
        out.settle()
        torch.cuda.synchronize()
        wc.check_device_status()
        assert np.array_equal(out.local.float().cpu().numpy().T, want)
        dist.barrier()
        if out.multicast_ptr:
            out.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            wc.gemm_multicast_output(desc, da.data_ptr(), db.data_ptr(), out.ptrs[rank] + offset,
                                     out.multicast_ptr + offset, stream)
            out.settle()
            torch.cuda.synchronize()
            wc.check_device_status()
            assert np.array_equal(out.local.float().cpu().numpy().T, want)
            dist.barrier()

        # 3. host buffers: A's rows exchanged over NVLink, B and C blocks through the host call
        a_host = torch.from_numpy(a.view(np.int16)).pin_memory()
        b_host = torch.from_numpy(np.ascontiguousarray(b[n0:n1]).view(np.int16)).pin_memory()
        c_host = torch.zeros((n1 - n0) * M, dtype=torch.int16).pin_memory()
        a_dev = torch.empty((M, K), dtype=torch.int16, device="cuda")
        sh.sharded_gemm_host(wc, desc, a_dev, a_host, b_host, c_host, dist, rank, world, stream)
        wc.check_device_status()
        got = oracle.from_bits(c_host.numpy().view(np.uint16), oracle.BF16).reshape(n1 - n0, M).T
        assert np.array_equal(got, want[:, n0:n1])
        # 4. attention: (batch, head) slabs, gathered by NCCL and inside the kernel (both forms)
        BH, S, D = 8, 512, 128
        q, k, v = (oracle.baseline_inputs((BH, S, D), "normal", 9, i, oracle.BF16) for i in range(3))
        want_o = None
        h0, h1 = sh.head_shard(BH, world, rank)
        fd = wc.fa_desc(1, h1 - h0, S, S, D, causal=True, io_type=wc.BF16)
        dq, dk, dv = (dev(x[h0:h1]) for x in (q, k, v))
        o_slab = torch.full((h1 - h0, S, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        wc.flash_attention_fwd(fd, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), o_slab.data_ptr(), 0, stream)
        want_o = sh.all_gather_shards(o_slab, dist).reshape(BH, S, D).float().cpu().numpy()
        ref = oracle.fa_ref(q, k, v, oracle.BF16, 1.0 / np.sqrt(D), causal=True)
        assert np.abs(want_o - ref).max() <= 3.0e-2
        full_o = sh.PeerMappedOutput((BH, S, D), torch.bfloat16, dist, rank, world)
        o_off = h0 * S * D * 2
        forms = [lambda: wc.flash_attention_fwd_multi_output(fd, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                                              full_o.block_targets(o_off), 0, stream)]
        if full_o.multicast_ptr:
            forms.append(lambda: wc.flash_attention_fwd_multicast_output(
                fd, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), full_o.ptrs[rank] + o_off,
                full_o.multicast_ptr + o_off, 0, stream))
        for form in forms:
            full_o.local.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            form()
            full_o.settle()
            torch.cuda.synchronize()
            wc.check_device_status()
            assert np.array_equal(full_o.local.float().cpu().numpy(), want_o)  # the plain call's bits, from every rank
            dist.barrier()
        open(os.path.join(tmpdir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_gpu_column_shards_three_gathers(cuda, tmp_path):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")
