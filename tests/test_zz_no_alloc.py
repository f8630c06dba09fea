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
