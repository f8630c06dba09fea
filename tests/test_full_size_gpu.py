"""The benchmark configurations at their full sizes, checked on the GPU.

A full CPU reference of 8192^3 or of 512 heads x 4096^2 attention takes minutes,
so these follow the reference's own precedent for large shapes: the gfx950
attention runner checks a fixed sample of heads and rows against its f64
reference (tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp:204-232), and here
the GEMMs are checked on a sample of complete output rows against the oracle
plus one size-independent property (every output row of a GEMM whose B rows
are all equal is constant along n)."""
import numpy as np
import pytest

from _util import runner_tolerance_ok, to_device_bits

pytestmark = pytest.mark.gpu


def _gemm(torch, wc, a_bits, b_bits, in_type, out_name, streamk=1, **knobs):
    M, K = a_bits.shape
    N = b_bits.shape[0]
    desc = wc.gemm_desc(M, N, K, in_type=in_type, out_type=wc.TYPE_BY_NAME[out_name], streamk_workers=streamk, **knobs)
    a, b = to_device_bits(torch, a_bits), to_device_bits(torch, b_bits)
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[out_name]
    c = torch.full((M, N), float("nan"), dtype=dt, device="cuda")
    s, cn = wc.gemm_workspace_bytes(desc)
    ws = torch.zeros(s + cn, dtype=torch.uint8, device="cuda") if s + cn else None
    wc.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), ws.data_ptr() if ws is not None else 0,
            torch.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    return c


def test_config2_square_4096_f16(cuda, wc, oracle):
    """M=N=K=4096, A and B uniform in [-1,1) rounded to f16, f32 accumulate, f16 output."""
    n = 4096
    a = oracle.baseline_inputs((n, n), "uniform", 2, 0, oracle.F16)
    b = oracle.baseline_inputs((n, n), "uniform", 2, 1, oracle.F16)
    c = _gemm(cuda, wc, a, b, wc.F16, "f16", bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)
    rows = np.unique(np.concatenate([np.arange(0, n, 67), [n - 1]])).astype(np.int32)
    want = oracle.round_output(oracle.gemm_ref(a, b, oracle.F16, rows=rows), "f16")
    got = c[rows.tolist()].float().cpu().numpy()
    # outputs are O(sqrt(4096/3)) ~ 37: one f16 ulp there is 2**-5, inside 1e-2 + 1e-3*|exp|
    ok, worst, nbad = runner_tolerance_ok(got, want, "f16")
    assert ok, f"{nbad} of {got.size} sampled elements out of tolerance, worst {worst}"
    assert not cuda.isnan(c).any()


def test_config3_square_8192_bf16(cuda, wc, oracle):
    """M=N=K=8192, A and B ~ N(0,1)/sqrt(K) rounded to bf16, f32 accumulate, bf16
    output, on the CTA-pair kernel; sampled rows against the oracle, mean
    absolute error, and no element left unwritten."""
    n = 8192
    a = oracle.baseline_inputs((n, n), "normal", 3, 0, oracle.BF16, scale=n ** -0.5)
    b = oracle.baseline_inputs((n, n), "normal", 3, 1, oracle.BF16, scale=n ** -0.5)
    c = _gemm(cuda, wc, a, b, wc.BF16, "bf16", bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)
    rows = np.unique(np.concatenate([np.arange(0, n, 257), [127, 128, 255, 256, n - 1]])).astype(np.int32)
    want = oracle.round_output(oracle.gemm_ref(a, b, oracle.BF16, rows=rows), "bf16")
    got = c[rows.tolist()].float().cpu().numpy()
    ok, worst, nbad = runner_tolerance_ok(got, want, "bf16")
    assert ok, f"{nbad} of {got.size} sampled elements out of tolerance, worst {worst}"
    assert float(np.mean(np.abs(got - want))) <= 1e-3
    assert not cuda.isnan(c).any()


def test_config3_constant_b_rows_property(cuda, wc, oracle):
    """Size-independent property at 8192^3: if every row of B (stored N x K) is
    the same vector, C[m, :] is constant along n and equals A[m, :] . b."""
    n = 8192
    a = oracle.baseline_inputs((n, n), "normal", 5, 0, oracle.BF16, scale=n ** -0.5)
    brow = oracle.baseline_inputs((1, n), "normal", 5, 1, oracle.BF16)
    b = np.ascontiguousarray(np.broadcast_to(brow, (n, n)))
    c = _gemm(cuda, wc, a, b, wc.BF16, "f32", bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)
    assert bool((c == c[:, :1]).all()), "rows of C are not constant along n"
    want = oracle.gemm_ref(a, brow, oracle.BF16)[:, 0]
    ok, worst, nbad = runner_tolerance_ok(c[:, 0].cpu().numpy(), want)
    assert ok, f"{nbad} rows out of tolerance, worst {worst}"


def test_config5_skinny_decode_full_check(cuda, wc, oracle):
    """M=16, N=28672, K=8192, A ~ N(0,1), B ~ N(0,1)/sqrt(K), bf16, f32 accumulate,
    Stream-K chosen automatically; every element checked; two launches identical."""
    M, N, K = 16, 28672, 8192
    a = oracle.baseline_inputs((M, K), "normal", 7, 0, oracle.BF16)
    b = oracle.baseline_inputs((N, K), "normal", 7, 1, oracle.BF16, scale=K ** -0.5)
    c1 = _gemm(cuda, wc, a, b, wc.BF16, "f32", streamk=0, bn=1)
    c2 = _gemm(cuda, wc, a, b, wc.BF16, "f32", streamk=0, bn=1)
    assert bool((c1 == c2).all())
    ok, worst, nbad = runner_tolerance_ok(c1.cpu().numpy(), oracle.gemm_ref(a, b, oracle.BF16))
    assert ok, f"{nbad} elements out of tolerance, worst {worst}"


def test_config4_attention_full_size_sampled(cuda, wc, oracle):
    """Causal forward, batch 16, heads 32, S=4096, D=128, Q/K/V ~ N(0,1) in bf16,
    scale 1/sqrt(128): the runner's sample of heads {0, mid, last} and rows
    {0, 31, 32, 127, S/2, S-128, S-1} against the f64 oracle (max-abs <= 3e-2),
    plus the convex-combination bound |O| <= max|V| on every element."""
    torch = cuda
    B, H, S, D = 16, 32, 4096, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(4)
    q, k, v = (torch.randn(B * H, S, D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    o = torch.full_like(q, float("nan"))
    desc = wc.fa_desc(B, H, S, S, D, causal=True)
    wc.flash_attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 0,
                           torch.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    assert not torch.isnan(o).any()
    assert float(o.float().abs().max()) <= float(v.float().abs().max()) * (1 + 2.0 ** -7)
    heads, rows = oracle.fa_sample_heads(B * H), oracle.fa_sample_rows(S)
    bits = lambda x: x[heads.tolist()].cpu().view(torch.int16).numpy().view(np.uint16)
    want = oracle.fa_ref(bits(q), bits(k), bits(v), oracle.BF16, 1.0 / np.sqrt(D), causal=True, rows=rows)
    got = o[heads.tolist()].float().cpu().numpy()[:, rows]
    diff = np.abs(got - want)
    assert diff.max() <= 3.0e-2 and diff.mean() <= 1.0e-3, (diff.max(), diff.mean())
