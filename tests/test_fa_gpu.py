"""GPU parity of the flash-attention forward against the f64 CPU oracle,
through the C ABI.

Mirrors the reference's runtime checks: the gfx950 runner compares sampled
heads/rows with a f64 reference and passes on max-abs <= 3e-2
(tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp:204-232, 384-394;
test/Integration/wave_flash_attention_gfx950_runtime.mlir:3-22).  Causal
masking, a caller-supplied scale, f16 I/O and ragged lengths are extensions
and are checked against the oracle's labelled extensions.
"""
import os

import numpy as np
import pytest

from _util import env_knobs, to_device_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["pingpong", "stream", "pair", "decoupled"], autouse=True)
def fa_kernel(request, wc):
    """Every test runs on all four attention kernels (two Q tiles ping-ponging;
    one Q tile with double-buffered scores; CTA pairs on 512-row work items;
    80-key blocks with P beside S in tensor memory).  Left alone, the library
    takes the last one."""
    with env_knobs(wc, WAVE_CUDA_FA_KERNEL=request.param):
        yield request.param

REFERENCE_MAX_ABS = 3.0e-2  # wave-fa-gfx950-runner.cpp:388


def run_fa(torch, wc, q_bits, k_bits, v_bits, io_name, batch, heads, causal, scale=0.0, want_lse=False,
           out_f32=False, qk_max_abs=0.0):
    BH, Sq, D = q_bits.shape
    Sk = k_bits.shape[1]
    assert BH == batch * heads
    desc = wc.fa_desc(batch, heads, Sq, Sk, D, scale=scale, causal=causal, io_type=wc.TYPE_BY_NAME[io_name],
                      out_f32=out_f32, qk_max_abs=qk_max_abs)
    q, k, v = (to_device_bits(torch, x) for x in (q_bits, k_bits, v_bits))
    dt = torch.float32 if out_f32 else torch.bfloat16 if io_name == "bf16" else torch.float16
    o = torch.full((BH, Sq, D), float("nan"), dtype=dt, device="cuda")
    lse = torch.full((BH, Sq), float("nan"), dtype=torch.float32, device="cuda") if want_lse else None
    wc.flash_attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                           lse.data_ptr() if want_lse else 0, torch.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    out = o.float().cpu().numpy()
    return (out, lse.cpu().numpy()) if want_lse else out


def lcg_qkv(oracle, BH, Sq, Sk, D, t, seed, input_scale=1):
    q = oracle.fa_input_bits(BH * Sq * D, t, seed, 0, 0.125 * input_scale).reshape(BH, Sq, D)
    k = oracle.fa_input_bits(BH * Sk * D, t, seed, 1, 0.125 * input_scale).reshape(BH, Sk, D)
    v = oracle.fa_input_bits(BH * Sk * D, t, seed, 2, 0.25).reshape(BH, Sk, D)
    return q, k, v


def normal_qkv(oracle, BH, Sq, Sk, D, t, seed):
    return (oracle.baseline_inputs((BH, Sq, D), "normal", seed, 0, t),
            oracle.baseline_inputs((BH, Sk, D), "normal", seed, 1, t),
            oracle.baseline_inputs((BH, Sk, D), "normal", seed, 2, t))


def check(got, want, tag=""):
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert not np.isnan(got).any(), f"{tag}: NaN in output"
    worst = float(diff.max())
    assert worst <= REFERENCE_MAX_ABS, f"{tag}: max abs {worst}"
    # stated tolerance for 16-bit inputs with f32 accumulation:
    # |d| <= 1e-2 + 1e-2*|exp| per element, mean absolute error <= 1e-3
    assert (diff <= 1.0e-2 + 1.0e-2 * np.abs(want)).all(), f"{tag}: max abs {worst}"
    assert float(diff.mean()) <= 1.0e-3, f"{tag}: mean abs {diff.mean()}"


@pytest.mark.parametrize("batch,heads,S,causal,seed", [
    (1, 1, 256, False, 0),
    (1, 2, 256, False, 7),
    (1, 2, 512, False, 3),
    (2, 2, 512, True, 5),
    (1, 1, 1024, True, 1),
    (1, 3, 768, False, 2),
])
def test_runner_inputs_all_rows(cuda, wc, oracle, batch, heads, S, causal, seed):
    """Inputs of the reference runner (bf16 LCG, Q/K x0.125, V x0.25), every
    row checked (the runner checks all rows when S <= 512)."""
    BH, D, t = batch * heads, 128, oracle.BF16
    q, k, v = lcg_qkv(oracle, BH, S, S, D, t, seed)
    got = run_fa(cuda, wc, q, k, v, "bf16", batch, heads, causal)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal)
    check(got, want, f"S={S} causal={causal}")


@pytest.mark.parametrize("causal", [False, True])
def test_normal_inputs_config_shape_small(cuda, wc, oracle, causal):
    """N(0,1) Q/K/V, scale 1/sqrt(128): the benchmark's distribution at
    B=1, H=2, S=512, every row checked."""
    t = oracle.BF16
    q, k, v = normal_qkv(oracle, 2, 512, 512, 128, t, seed=17)
    got, lse = run_fa(cuda, wc, q, k, v, "bf16", 1, 2, causal, want_lse=True)
    want, want_lse = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal, want_lse=True)
    check(got, want, f"normal causal={causal}")
    assert np.abs(lse.astype(np.float64) - want_lse).max() <= 2e-3


@pytest.mark.parametrize("Sq,Sk,causal", [(144, 400, False), (272, 272, True), (16, 16, True), (128, 128, False),
                                          (400, 144, False),
                                          # around multiples of 80 keys (the decoupled kernel's block) and of 128
                                          (80, 80, True), (96, 96, True), (176, 160, False), (336, 336, True),
                                          (640, 640, True), (256, 1040, False)])
def test_ragged_lengths(cuda, wc, oracle, Sq, Sk, causal):
    """Lengths that are not whole numbers of K/V blocks or Q tiles, for every
    kernel: the last block is partly past the end of K, the causal diagonal
    crosses blocks at every offset, a work item may have one tile only."""
    t = oracle.BF16
    q, k, v = normal_qkv(oracle, 3, Sq, Sk, 128, t, seed=Sq + Sk)
    got = run_fa(cuda, wc, q, k, v, "bf16", 1, 3, causal)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal)
    check(got, want, f"{Sq}x{Sk} causal={causal}")


def test_f16_io_and_custom_scale(cuda, wc, oracle):
    t = oracle.F16
    q, k, v = normal_qkv(oracle, 2, 384, 384, 128, t, seed=23)
    got = run_fa(cuda, wc, q, k, v, "f16", 2, 1, True, scale=0.05)
    want = oracle.fa_ref(q, k, v, t, float(np.float32(0.05)), causal=True)
    check(got, want, "f16")


@pytest.mark.parametrize("S,causal,io_name,bound", [
    (256, False, "bf16", 1.0),
    (512, True, "bf16", 1.0),
    (1024, False, "bf16", 1.5),
    (768, True, "bf16", 1.9609375),   # the widest bound the span check admits
    (1280, True, "f16", 1.0),
])
def test_fixed_reference_matches_the_softmax(cuda, wc, oracle, S, causal, io_name, bound):
    """`qk_max_abs` replaces the running row maximum by a constant
    (wave_flash_attention.py:108-113, 602-609); the result is the same softmax.
    Runner inputs with --input-scale=1, whose Q and K reach 1 in magnitude
    (the range the reference's driver wants covered, wave-fa-gfx950.py:77-78)."""
    BH, D = 2, 128
    t = oracle.BF16 if io_name == "bf16" else oracle.F16
    q, k, v = lcg_qkv(oracle, BH, S, S, D, t, seed=S)
    assert np.abs(oracle.from_bits(q, t)).max() <= 1.0 and np.abs(oracle.from_bits(k, t)).max() <= 1.0
    got, lse = run_fa(cuda, wc, q, k, v, io_name, 1, BH, causal, want_lse=True, qk_max_abs=bound)
    want, want_lse = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal, want_lse=True)
    check(got, want, f"fixed reference S={S} causal={causal} bound={bound}")
    assert np.abs(lse.astype(np.float64) - want_lse).max() <= 2e-3


def test_fixed_reference_ragged_and_small_inputs(cuda, wc, oracle):
    """Uniform [-1, 1) inputs under the bound 1, lengths that are not multiples
    of the 128-row tiles, separate query and key lengths."""
    t = oracle.BF16
    for Sq, Sk, causal in ((144, 400, False), (272, 272, True), (16, 16, True), (400, 144, False)):
        q = oracle.baseline_inputs((3, Sq, 128), "uniform", Sq, 0, t)
        k = oracle.baseline_inputs((3, Sk, 128), "uniform", Sq, 1, t)
        v = oracle.baseline_inputs((3, Sk, 128), "uniform", Sq, 2, t)
        got = run_fa(cuda, wc, q, k, v, "bf16", 1, 3, causal, qk_max_abs=1.0)
        want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal)
        check(got, want, f"fixed reference {Sq}x{Sk} causal={causal}")


def test_fixed_reference_at_the_edge_of_the_bf16_range(cuda, wc, oracle):
    """All scores at minus the bound, with the largest bf16 bound the span
    check admits at scale 1/sqrt(128): the probabilities are 2^-125.5, still
    normal bf16 numbers, and every output row is the mean of V
    (integrations/tlx/tests/test_backend.py:10207-10257)."""
    BH, S, D, t = 1, 256, 128, oracle.BF16
    bound = 1.9609375
    q = oracle.to_bits(np.full((BH, S, D), bound, dtype=np.float32), t)
    k = oracle.to_bits(np.full((BH, S, D), -bound, dtype=np.float32), t)
    v = oracle.baseline_inputs((BH, S, D), "uniform", 0, 2, t)
    got = run_fa(cuda, wc, q, k, v, "bf16", 1, 1, False, qk_max_abs=bound)
    mean = oracle.from_bits(v, t).astype(np.float64).mean(axis=1, keepdims=True)
    assert np.isfinite(got).all()
    assert np.abs(got - mean).max() <= 2e-2


def test_fixed_reference_long_sequence_sampled(cuda, wc, oracle):
    """The perf-golden shape's sequence length (B2 H64 N8192 runs with
    --qk-max-abs=1, test_gfx950_fa_b2_h64_n8192_d128_bf16_8wave.py:44) on 2
    heads, on the runner's sample of rows."""
    t = oracle.BF16
    BH, S = 2, 8192
    q, k, v = lcg_qkv(oracle, BH, S, S, 128, t, seed=17)
    got = run_fa(cuda, wc, q, k, v, "bf16", 1, BH, False, qk_max_abs=1.0)
    hs, rs = list(range(BH)), oracle.fa_sample_rows(S)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=False, heads=hs, rows=rs)
    check(got[np.ix_(hs, rs)], want, "fixed reference S=8192")


@pytest.mark.parametrize("causal", [False, True])
def test_long_sequence_sampled(cuda, wc, oracle, causal):
    """S=4096 (the benchmark's sequence length) on 6 heads, checked on the
    reference runner's sample of heads and rows
    (wave-fa-gfx950-runner.cpp:204-232)."""
    t = oracle.BF16
    batch, heads, S = 2, 3, 4096
    q, k, v = normal_qkv(oracle, batch * heads, S, S, 128, t, seed=4)
    got = run_fa(cuda, wc, q, k, v, "bf16", batch, heads, causal)
    hs, rs = oracle.fa_sample_heads(batch * heads), oracle.fa_sample_rows(S)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal, heads=hs, rows=rs)
    check(got[np.ix_(hs, rs)], want, f"S=4096 causal={causal}")


def test_rows_are_convex_combinations(cuda, wc, oracle):
    """Size-independent property: with V constant along keys, every output row
    equals that constant whatever the scores are."""
    t = oracle.BF16
    BH, S = 4, 1024
    q, k, _ = normal_qkv(oracle, BH, S, S, 128, t, seed=8)
    vrow = oracle.baseline_inputs((BH, 1, 128), "normal", 8, 5, t)
    v = np.ascontiguousarray(np.broadcast_to(vrow, (BH, S, 128)))
    got = run_fa(cuda, wc, q, k, v, "bf16", 1, BH, True)
    want = np.broadcast_to(oracle.from_bits(vrow, t), (BH, S, 128))
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()


@pytest.mark.parametrize("D,causal", [(64, True), (64, False), (32, False), (96, True), (16, False)])
def test_smaller_head_dims_run_zero_padded(cuda, wc, oracle, D, causal):
    t = oracle.BF16
    q, k, v = normal_qkv(oracle, 2, 384, 384, D, t, seed=D)
    got = run_fa(cuda, wc, q, k, v, "bf16", 1, 2, causal)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(float(D)), causal=causal)
    check(got, want, f"D={D} causal={causal}")


def test_toy_kernel_surface_matches_reference_golden(cuda, wc, oracle):
    """The reference's toy kernel `flash_attention_f32` (16 query rows, f16 in,
    f32 out, Q pre-multiplied by log2(e)/sqrt(d), exp2 of the bare scores;
    python/mlir/dialects/wave_attention.py:225-278) against the outputs recorded
    from the reference's own Python reference, at the toy runner's tolerance
    3e-3 (tools/wave-fa-calibrate/wave-fa-calibrate-runner.cpp:263)."""
    import json
    import os
    from test_oracle import toy_fa_inputs
    with open(os.path.join(os.path.dirname(__file__), "golden", "fa_toy_golden.json")) as f:
        cases = json.load(f)["cases"]
    for entry in cases:
        c = entry["case"]
        q, k, v = toy_fa_inputs(oracle, c["block_m"], c["head_dim"], c["seq_n"], c["random_seed"])
        got = run_fa(cuda, wc, q, k, v, "f16", 1, 1, False, scale=float(np.log(2.0)), out_f32=True)
        want = np.asarray(entry["out"], np.float64).reshape(got.shape)
        assert np.abs(got - want).max() <= 3.0e-3, c


def test_host_buffer_call_pipelined_by_head_groups(cuda, wc, oracle):
    """Large host-buffer calls run group of heads by group of heads, copies
    overlapped with compute; the result must equal the one-piece call's."""
    import importlib
    wa = importlib.import_module("7_b200.wave_attention")
    t = oracle.BF16
    BH, S = 64, 1024  # 3 x 16 MiB of inputs: above the pipelining threshold
    q, k, v = normal_qkv(oracle, BH, S, S, 128, t, seed=31)
    got = oracle.from_bits(wa.run_attention_host(q, k, v, 4, 16, causal=True), t)
    hs, rs = oracle.fa_sample_heads(BH), oracle.fa_sample_rows(S)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=True, heads=hs, rows=rs)
    check(got[np.ix_(hs, rs)], want, "host pipelined")
    dev = run_fa(cuda, wc, q, k, v, "bf16", 4, 16, True)
    assert np.array_equal(got, dev)


def test_launches_overlapping_on_two_streams(cuda, wc, oracle):
    """Launches that overlap on the GPU (two streams) each draw their work items
    from a counter of their own; both results must be the single-stream ones."""
    t = oracle.BF16
    BH, S = 8, 1024
    q, k, v = normal_qkv(oracle, BH, S, S, 128, t, seed=41)
    want = run_fa(cuda, wc, q, k, v, "bf16", 2, 4, True)
    desc = wc.fa_desc(2, 4, S, S, 128, causal=True, io_type=wc.TYPE_BY_NAME["bf16"])
    dq, dk, dv = (to_device_bits(cuda, x) for x in (q, k, v))
    streams = [cuda.cuda.Stream(), cuda.cuda.Stream()]
    outs = [cuda.empty((BH, S, 128), dtype=cuda.bfloat16, device="cuda") for _ in streams]
    cuda.cuda.synchronize()
    for _ in range(20):
        for st, o in zip(streams, outs):
            wc.flash_attention_fwd(desc, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), o.data_ptr(), 0, st.cuda_stream)
    cuda.cuda.synchronize()
    wc.check_device_status()
    for o in outs:
        assert np.array_equal(o.float().cpu().numpy(), want)


def test_more_queued_launches_than_ticket_counters(cuda, wc, oracle):
    """The work-item counters are a ring of 64 per GPU.  With more launches
    queued than that (70 per stream on 4 streams, each launch with an output of
    its own), the launch that comes round to a counter is ordered behind the one
    that used it before, so no launch may lose or repeat work items: every one
    of the 280 outputs must be the single-stream result."""
    t = oracle.BF16
    BH, S = 4, 512
    q, k, v = normal_qkv(oracle, BH, S, S, 128, t, seed=43)
    want = run_fa(cuda, wc, q, k, v, "bf16", 1, 4, True)
    desc = wc.fa_desc(1, 4, S, S, 128, causal=True, io_type=wc.TYPE_BY_NAME["bf16"])
    dq, dk, dv = (to_device_bits(cuda, x) for x in (q, k, v))
    streams = [cuda.cuda.Stream() for _ in range(4)]
    per_stream = 70
    outs = cuda.full((len(streams), per_stream, BH, S, 128), float("nan"), dtype=cuda.bfloat16, device="cuda")
    cuda.cuda.synchronize()
    for i in range(per_stream):
        for s_idx, st in enumerate(streams):
            wc.flash_attention_fwd(desc, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), outs[s_idx, i].data_ptr(), 0,
                                   st.cuda_stream)
    cuda.cuda.synchronize()
    wc.check_device_status()
    got = outs.float().cpu().numpy()
    assert np.array_equal(got, np.broadcast_to(want, got.shape))


@pytest.mark.parametrize("BH,S,D,causal,out_f32", [
    (6, 512, 128, True, False),
    (3, 384, 64, False, False),     # head dimension below 128: only the first 64 columns exist
    (2, 272, 128, True, True),      # ragged length, f32 output
    (3, 400, 96, True, False),      # ragged length and a narrow head in the 16-bit type
    (80, 1024, 128, True, False),   # more work items than SMs: a CTA's items share its staging area in turn
    (80, 512, 128, False, False),   # ... with both tiles of an item finishing together
])
def test_multi_output_writes_every_target(cuda, wc, oracle, BH, S, D, causal, out_f32):
    """wave_cuda_flash_attention_fwd_multi_output: O lands in every target (on
    one GPU: three local buffers stand in for peer GPUs' copies), each bit for
    bit what the plain call writes; here the slab sits in the middle of a larger
    buffer, as a rank's (batch, head) slab sits inside the gathered O, and the
    rest of that buffer must stay untouched."""
    t = oracle.BF16
    q, k, v = normal_qkv(oracle, BH, S, S, D, t, seed=53)
    want = run_fa(cuda, wc, q, k, v, "bf16", 1, BH, causal, out_f32=out_f32)
    desc = wc.fa_desc(1, BH, S, S, D, causal=causal, io_type=wc.BF16, out_f32=out_f32)
    dq, dk, dv = (to_device_bits(cuda, x) for x in (q, k, v))
    dt = cuda.float32 if out_f32 else cuda.bfloat16
    pad = 2 * S * D  # elements before and after the slab
    targets = [cuda.full((pad + BH * S * D + pad,), float("nan"), dtype=dt, device="cuda") for _ in range(3)]
    esize = 4 if out_f32 else 2
    wc.flash_attention_fwd_multi_output(desc, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                        [x.data_ptr() + pad * esize for x in targets], 0,
                                        cuda.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    for x in targets:
        got = x.float().cpu().numpy()
        assert np.array_equal(got[pad:pad + BH * S * D].reshape(BH, S, D), want)
        assert np.isnan(got[:pad]).all() and np.isnan(got[pad + BH * S * D:]).all()


def _operator_case(cuda, oracle, q_bits, k_bits, v_bits, **kwargs):
    """Runs the torch-tensor operator (the mirror of the reference's
    `attention`, integrations/tlx/workloads/amd_fa_wave.py:1671-1720) on
    (1, H, N, D) tensors built from bit patterns; returns f32 [H, N, D]."""
    import importlib
    wa = importlib.import_module("7_b200.wave_attention")
    q, k, v = (to_device_bits(cuda, x).view(cuda.bfloat16).unsqueeze(0) for x in (q_bits, k_bits, v_bits))
    out = wa.attention(q, k, v, **kwargs)
    cuda.cuda.synchronize()
    importlib.import_module("7_b200.wave_cuda").check_device_status()
    return out[0].float().cpu().numpy()


@pytest.mark.parametrize("mode,sm_scale,qk_max_abs", [
    ("adaptive-negative", -1.0 / np.sqrt(128.0), None),
    ("bounded-negative", -0.3357431655837235, 1.0),
    ("adaptive-zero", 0.0, None),
    ("bounded-negative-zero", -0.0, 1.0),
    ("adaptive-positive", 0.05, None),
])
def test_operator_signed_scale(cuda, oracle, mode, sm_scale, qk_max_abs):
    """Any finite softmax scale, as the reference's operator takes it: constant
    queries, keys whose sign flips every 32 tokens, values the opposite sign
    (integrations/tlx/tests/test_backend.py:10281-10333)."""
    t, S, D = oracle.BF16, 256, 128
    magnitude = 2.0 if mode == "adaptive-negative" else 1.0
    sign = np.where(np.arange(S) % 64 < 32, magnitude, -magnitude).astype(np.float32)
    q = oracle.to_bits(np.full((1, S, D), magnitude, np.float32), t)
    k = oracle.to_bits(np.broadcast_to(sign[None, :, None], (1, S, D)), t)
    v = oracle.to_bits(np.broadcast_to(np.where(sign > 0, -1.0, 1.0).astype(np.float32)[None, :, None], (1, S, D)), t)
    got = _operator_case(cuda, oracle, q, k, v, sm_scale=sm_scale, qk_max_abs=qk_max_abs)
    want = oracle.fa_ref(q, k, v, t, float(sm_scale), causal=False)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-2  # the reference's tolerance for this case


@pytest.mark.parametrize("qk_max_abs", [None, 1.0], ids=["adaptive", "bounded"])
@pytest.mark.parametrize("causal", [False, True])
def test_operator_runner_inputs(cuda, oracle, qk_max_abs, causal):
    t = oracle.BF16
    q, k, v = lcg_qkv(oracle, 3, 512, 512, 128, t, seed=11)
    got = _operator_case(cuda, oracle, q, k, v, causal=causal, qk_max_abs=qk_max_abs)
    want = oracle.fa_ref(q, k, v, t, 1.0 / np.sqrt(128.0), causal=causal)
    check(got, want, f"operator causal={causal} bound={qk_max_abs}")


def test_operator_rejects_what_the_reference_rejects(cuda, oracle):
    """amd_fa_wave.py:1582-1611; test_backend.py:10195-10202, 10260-10277."""
    import importlib
    wa = importlib.import_module("7_b200.wave_attention")
    x = cuda.zeros((1, 1, 256, 128), dtype=cuda.bfloat16, device="cuda")
    for bad in (float("inf"), float("-inf"), float("nan")):
        with pytest.raises(ValueError, match="sm_scale must be finite"):
            wa.attention(x, x, x, sm_scale=bad)
        with pytest.raises(ValueError, match="qk_max_abs must be finite and greater than zero"):
            wa.attention(x, x, x, qk_max_abs=bad)
    with pytest.raises(ValueError, match="qk_max_abs must be finite and greater than zero"):
        wa.attention(x, x, x, qk_max_abs=0.0)
    with pytest.raises(ValueError, match="fixed reference exceeds BF16 range"):
        wa.attention(x, x, x, qk_max_abs=2.0)
    with pytest.raises(ValueError, match="CUDA tensors"):
        wa.attention(x.cpu(), x.cpu(), x.cpu())
