"""Stream-K GEMM on the library's built-in workspace (wave_cuda_gemm_streamk_static).

That entry point exists for callers that cannot give the GEMM a workspace: a
host written to the reference's plain {A, B, C, trip} argument list has no slot
for one, and a process whose device memory belongs to another allocator, or a
path where a device allocation must not happen, cannot create one.  It must
return exactly what wave_cuda_gemm returns with a caller-allocated workspace,
call after call (the built-in area is shared and keeps the previous call's
contents), and must refuse launches that need more than the area holds.

This file is named to be collected last, so that a run that stops at the first
failure has already run every other test; it also passes when run alone.
"""
import numpy as np
import pytest

from _util import device_out, out_to_f32, to_device_bits

pytestmark = pytest.mark.gpu


def _inputs(oracle, M, N, K, seed):
    t = oracle.BF16
    a = oracle.baseline_inputs((M, K), "normal", seed, 0, t)
    b = oracle.baseline_inputs((N, K), "normal", seed, 1, t, scale=K ** -0.5)
    return a, b


@pytest.mark.parametrize("M,N,K,workers,knobs", [
    (16, 4096, 4096, 148, dict(bn=1)),                                        # skinny, operands swapped
    (256, 512, 2048, 7, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),    # 128 x 256 tiles
])
def test_static_workspace_matches_caller_workspace_twice(cuda, wc, oracle, M, N, K, workers, knobs):
    torch = cuda
    a_bits, b_bits = _inputs(oracle, M, N, K, seed=M + workers)
    a, b = to_device_bits(torch, a_bits), to_device_bits(torch, b_bits)
    desc = wc.gemm_desc(M, N, K, in_type=wc.BF16, out_type=wc.F32, streamk_workers=workers, **knobs)
    scratch, counters = wc.gemm_workspace_bytes(desc)
    assert 0 < scratch + counters <= wc.STATIC_WORKSPACE_BYTES
    stream = torch.cuda.current_stream().cuda_stream

    # existing entry point, workspace allocated by the caller
    ws = torch.zeros(scratch + counters, dtype=torch.uint8, device="cuda")
    c_ref = device_out(torch, M * N, "f32")
    wc.gemm(desc, a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), ws.data_ptr(), stream)
    wc.check_device_status()
    want = out_to_f32(torch, c_ref)
    assert not np.isnan(want).any()

    # new entry point: nothing allocated, two calls in a row on the shared area
    for call in range(2):
        c = device_out(torch, M * N, "f32")  # NaN-filled, so stale or missing writes show
        wc.gemm_streamk_static(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)
        wc.check_device_status()
        got = out_to_f32(torch, c)
        assert np.array_equal(got, want), f"call {call}: max abs diff {np.nanmax(np.abs(got - want))}"

    # and it is the right answer, not merely the same one
    ref = oracle.gemm_ref(a_bits, b_bits, oracle.BF16).reshape(-1)
    assert np.all(np.abs(want - ref) <= 1.0e-2 + 1.0e-3 * np.abs(ref))


def test_static_workspace_refuses_oversized_launch(cuda, wc):
    torch = cuda
    M = N = K = 4096
    desc = wc.gemm_desc(M, N, K, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4, streamk_workers=148)
    scratch, counters = wc.gemm_workspace_bytes(desc)
    assert scratch + counters > wc.STATIC_WORKSPACE_BYTES
    x = torch.zeros(M * K, dtype=torch.float16, device="cuda")
    c = torch.zeros(M * N, dtype=torch.float32, device="cuda")
    with pytest.raises(wc.WaveCudaError) as err:
        wc.gemm_streamk_static(desc, x.data_ptr(), x.data_ptr(), c.data_ptr())
    assert err.value.code == wc.E_INVALID
    assert "built-in workspace holds" in err.value.message


CASES = [
    (16, 4096, 4096, 148, dict(bn=1)),
    (256, 512, 2048, 7, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
]


def test_static_workspace_allocates_nothing_and_survives_alternating_shapes(cuda, wc, oracle):
    """The two properties the entry point exists for.  Free device memory, as
    the driver reports it, does not move across the calls (after one warm-up
    call per shape, which loads the kernels).  And two descriptors with
    different scratch sizes, called alternately, still give the caller-workspace
    bits: the counters sit behind the partial tiles, so their offset inside the
    shared area moves from call to call and each call finds the other shape's
    leftovers where its own counters belong."""
    torch = cuda
    stream = torch.cuda.current_stream().cuda_stream
    prepared = []
    for M, N, K, workers, knobs in CASES:
        a_bits, b_bits = _inputs(oracle, M, N, K, seed=3 * M + workers)
        a, b = to_device_bits(torch, a_bits), to_device_bits(torch, b_bits)
        desc = wc.gemm_desc(M, N, K, in_type=wc.BF16, out_type=wc.F32, streamk_workers=workers, **knobs)
        scratch, counters = wc.gemm_workspace_bytes(desc)
        ws = torch.zeros(scratch + counters, dtype=torch.uint8, device="cuda")
        c_ref = device_out(torch, M * N, "f32")
        wc.gemm(desc, a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), ws.data_ptr(), stream)
        c = device_out(torch, M * N, "f32")
        wc.gemm_streamk_static(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)  # warm-up
        prepared.append((desc, a, b, c, out_to_f32(torch, c_ref), scratch))
    assert prepared[0][5] != prepared[1][5], "the two cases must place their counters at different offsets"
    wc.check_device_status()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        for desc, a, b, c, want, _ in prepared:
            c.fill_(float("nan"))
            wc.gemm_streamk_static(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)
            torch.cuda.synchronize()
            assert np.array_equal(out_to_f32(torch, c), want)
    free_after, _ = torch.cuda.mem_get_info()
    wc.check_device_status()
    assert free_after == free_before, f"device memory in use moved by {free_before - free_after} bytes"


def test_static_workspace_automatic_plan_falls_back_to_whole_tiles(cuda, wc, oracle):
    """streamk_workers = 0 leaves the choice to the library.  Where its
    automatic Stream-K plan needs more than the built-in area holds, the call
    runs as whole tiles (no workspace, nothing allocated) instead of being
    refused, and returns the caller-workspace result."""
    torch = cuda
    stream = torch.cuda.current_stream().cuda_stream
    # (skinny: the automatic plan splits K over every SM with 128 x 16 partial tiles and fits the area;
    #  100 tiles of 128 x 256 on 148 SMs: the automatic plan wants 148 x 2 partial tiles, 38.8 MB, and does not)
    for M2, N2, K2, knobs, fits in [(16, 28672, 1024, dict(bn=1), True),
                                    (1280, 2560, 1024, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4), False)]:
        a_bits, b_bits = _inputs(oracle, M2, N2, K2, seed=77 + M2)
        a, b = to_device_bits(torch, a_bits), to_device_bits(torch, b_bits)
        desc = wc.gemm_desc(M2, N2, K2, in_type=wc.BF16, out_type=wc.F32, streamk_workers=0, **knobs)
        scratch, counters = wc.gemm_workspace_bytes(desc)
        assert scratch > 0 and (scratch + counters <= wc.STATIC_WORKSPACE_BYTES) == fits
        ws = torch.zeros(max(scratch + counters, 16), dtype=torch.uint8, device="cuda")
        c_ref = device_out(torch, M2 * N2, "f32")
        wc.gemm(desc, a.data_ptr(), b.data_ptr(), c_ref.data_ptr(), ws.data_ptr(), stream)
        c = device_out(torch, M2 * N2, "f32")
        wc.gemm_streamk_static(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream)
        wc.check_device_status()
        got, want = out_to_f32(torch, c), out_to_f32(torch, c_ref)
        assert not np.isnan(got).any()
        # whole tiles and Stream-K add the same products in a different grouping
        assert np.all(np.abs(got - want) <= 1.0e-2 + 1.0e-3 * np.abs(want))
