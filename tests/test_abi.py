"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, validates descriptors with the reference's rules and messages
(python/mlir/dialects/wave_matmul.py:533-619; the reference checks ~25
argument failures the same way, test/Integration/wave_matmul_rand_int_inputs.mlir:29-64),
sizes the Stream-K workspace like the reference runner, and fails loudly --
never silently falls back -- when asked to compute without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = "".join(open(os.path.join(ROOT, "include", name)).read()
                   for name in sorted(os.listdir(os.path.join(ROOT, "include"))) if name.endswith(".h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(wave_cuda_\w+|_mlir_ciface_\w+|mgpu[A-Z]\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(wc):
    lib = wc.lib()
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/wave_cuda.h but not exported"
    assert sorted(wc.EXPORTS) == names
    assert b"sm_100a" in lib.wave_cuda_version()


@pytest.mark.parametrize("kwargs,message", [
    (dict(M=33), "M must be a positive multiple of 16; got 33"),
    (dict(N=0), "N must be a positive multiple of 16; got 0"),
    (dict(K=-16), "K must be a positive multiple of 16; got -16"),
    (dict(bm=0), "BM and BN must be >= 1; got BM=0, BN=2"),
    (dict(bn=3), "BN must be a positive power of two (for the wave-id decomposition); got BN=3"),
    (dict(wave_k_tiles=0), "wave_m_tiles, wave_n_tiles and wave_k_tiles must be >= 1; got wave_m_tiles=1, "
                           "wave_n_tiles=1, wave_k_tiles=0"),
    (dict(bm=3), "BM * wave_m_tiles (=3) must divide M/16 (=4)"),
    (dict(bn=4, wave_n_tiles=3), "BN * wave_n_tiles (=12) must divide N/16 (=4)"),
    (dict(wave_k_tiles=3), "wave_k_tiles (=3) must divide K/16 (=4)"),
    (dict(M=1024, N=1024, bm=8, bn=8), "BM * BN must be <= 32 (RDNA3 workgroup wave cap); got BM=8, BN=8 (product=64)"),
    (dict(cta_group_m=0), "cta_group_m must be >= 1; got 0"),
    (dict(cta_group_m=3), "cta_group_m currently requires M_blocks to divide evenly; got M_blocks=4, cta_group_m=3"),
    (dict(out_layout=6), "output_layout must be one of row-major, column-major, tile-packed; got 6"),
    (dict(out_layout=4, ldc=64), "ldc must be 0 with tile-packed output"),
    (dict(out_layout=2, ldc=64), "ldc must be 0 with tile-packed output"),
    (dict(in_type=2), "input_type must be one of f16, bf16; got 2"),
    (dict(ldc=72), "ldc must be 0 or a multiple of 16"),
])
def test_gemm_validation_messages(wc, kwargs, message):
    base = dict(M=64, N=64, K=64)
    base.update(kwargs)
    M, N, K = base.pop("M"), base.pop("N"), base.pop("K")
    with pytest.raises(wc.WaveCudaError) as err:
        wc.gemm_validate(wc.gemm_desc(M, N, K, **base))
    assert message in err.value.message
    assert err.value.code in (wc.E_INVALID, wc.E_UNSUPPORTED)


def test_valid_descriptors_pass(wc):
    wc.gemm_validate(wc.gemm_desc(32, 32, 64, bm=2, bn=2, wave_k_tiles=2))  # the reference's --compare-cpu case
    wc.gemm_validate(wc.gemm_desc(8192, 8192, 8192, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4, in_type=wc.BF16,
                                  out_type=wc.BF16, cta_group_m=4))
    d = wc.GemmDesc()
    wc.lib().wave_cuda_gemm_desc_init(C.byref(d), 32, 32, 32)
    assert (d.bm, d.bn, d.in_type, d.out_type, d.streamk_workers) == (1, 2, wc.F16, wc.F32, 1)
    wc.gemm_validate(d)


def test_streamk_workspace_sizes(wc, oracle):
    """Scratch = workers * 2 slots * tile * 4 bytes and one counter per output
    tile, the reference's formula (runner.cpp:393-408) with this backend's
    128 x tile_n tile in place of 256 x 256."""
    d = wc.gemm_desc(512, 768, 1024, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4, streamk_workers=5)
    scratch, counters = wc.gemm_workspace_bytes(d)
    assert scratch == 5 * 2 * 128 * 256 * 4
    assert counters == (512 // 128) * (768 // 256) * 4
    assert wc.gemm_workspace_bytes(wc.gemm_desc(512, 768, 1024, streamk_workers=1)) == (0, 0)
    with pytest.raises(wc.WaveCudaError) as err:
        wc.gemm_workspace_bytes(wc.gemm_desc(128, 256, 64, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4,
                                             streamk_workers=9))
    assert "workers must be in [1, total_iterations]" in err.value.message
    R = oracle.ref_lib()
    if R is not None:  # the reference's own sizing for its 256x256 tiles
        assert R.wave_ref_streamk_scratch_bytes(5) == 5 * 2 * 256 * 256 * 4
        assert R.wave_ref_streamk_counter_elements(512, 768) == 6


@pytest.mark.parametrize("kwargs,message", [
    (dict(batch=0), "batch and heads must be positive"),
    (dict(seq_q=100), "sequence lengths must be positive multiples of 16"),
    (dict(head_dim=72), "head_dim must be a multiple of 16 between 16 and 128"),
    (dict(head_dim=256), "head_dim must be a multiple of 16 between 16 and 128"),
    (dict(io_type=2), "io_type must be bf16 or f16"),
    (dict(causal=True, seq_k=512), "causal attention requires seq_q == seq_k"),
    (dict(scale=-1.0), "scale must be finite"),
    # wave_flash_attention.py:64-75
    (dict(qk_max_abs=-1.0), "qk_max_abs must be finite and positive; got -1"),
    (dict(qk_max_abs=float("inf")), "qk_max_abs must be finite and positive; got inf"),
    (dict(qk_max_abs=float("nan")), "qk_max_abs must be finite and positive; got nan"),
    (dict(qk_max_abs=2.0), "qk_max_abs fixed reference exceeds BF16 range; use adaptive reference"),
    # the first bf16 value whose score span passes 126 at scale 1/sqrt(128) (test_backend.py:10217-10224)
    (dict(qk_max_abs=1.96875), "qk_max_abs fixed reference exceeds BF16 range"),
    (dict(qk_max_abs=1.0, scale=1.0), "qk_max_abs fixed reference exceeds BF16 range"),
])
def test_attention_validation_messages(wc, kwargs, message):
    base = dict(batch=1, heads=2, seq_q=256, seq_k=256, head_dim=128)
    base.update(kwargs)
    with pytest.raises(wc.WaveCudaError) as err:
        wc.fa_validate(wc.fa_desc(base.pop("batch"), base.pop("heads"), base.pop("seq_q"), base.pop("seq_k"),
                                  base.pop("head_dim"), **base))
    assert message in err.value.message


@pytest.mark.parametrize("kwargs", [
    dict(qk_max_abs=1.0),                      # the bound the reference's published numbers use
    dict(qk_max_abs=1.9609375),                # the last bf16 value inside the span (test_backend.py:10217)
    dict(qk_max_abs=8.0, scale=1.0 / 1024.0),  # a small scale widens the admissible bound
    dict(qk_max_abs=0.0),                      # 0 = adaptive reference
])
def test_fixed_reference_bounds_that_pass(wc, kwargs):
    wc.fa_validate(wc.fa_desc(1, 2, 256, 256, 128, **kwargs))


def test_memref_shims_return_data_plus_offset(wc):
    """runtime/wave_runtime.cpp:35-40: data + offset, in elements."""
    class MemRef(C.Structure):
        _fields_ = [("base", C.c_void_p), ("data", C.c_void_p), ("offset", C.c_int64), ("size", C.c_int64),
                    ("stride", C.c_int64)]
    lib = wc.lib()
    m = MemRef(0x1000, 0x2000, 3, 16, 1)
    for name, width in (("i8", 1), ("f16", 2), ("bf16", 2), ("i32", 4), ("f32", 4), ("i64", 8), ("f64", 8)):
        fn = getattr(lib, f"_mlir_ciface_wave_memref_to_ptr_global_{name}")
        assert fn(C.byref(m)) == 0x2000 + 3 * width


def test_unknown_kernel_name_is_rejected(wc):
    fn = C.c_void_p()
    d = wc.gemm_desc(64, 64, 64)
    rc = wc.lib().wave_cuda_module_get_function(b"no_such_kernel", C.byref(d), C.byref(fn))
    assert rc == wc.E_NOT_FOUND and b"no kernel named" in wc.lib().wave_cuda_last_error()


def test_compute_without_a_device_fails_loudly(wc):
    """No CPU fallback: on a machine without a CUDA device the host-buffer GEMM
    returns WAVE_E_CUDA instead of computing anything."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import numpy as np
    a = np.zeros((16, 16), np.uint16)
    c = np.zeros((16, 16), np.float32)
    with pytest.raises(wc.WaveCudaError) as err:
        wc.gemm_host(wc.gemm_desc(16, 16, 16, bn=1), a.ctypes.data, a.ctypes.data, c.ctypes.data)
    assert err.value.code == wc.E_CUDA


def test_memref_region_with_any_strides(wc):
    """The host range behind a ranked memref descriptor, which is what the
    mgpuMemHostRegisterMemRef wrapper registers: from the lowest to the highest
    addressed element.  A negative stride reaches below the element at index
    zero, so the range must start there, not at aligned + offset."""
    lib = wc.lib()

    def region(offset, sizes, strides, elem):
        rank = len(sizes)
        buf = (C.c_int64 * (3 + 2 * rank))()
        base = 1 << 20
        buf[0], buf[1], buf[2] = base, base, offset
        for i, (sz, st) in enumerate(zip(sizes, strides)):
            buf[3 + i], buf[3 + rank + i] = sz, st
        first, nbytes = C.c_void_p(), C.c_size_t()
        assert lib.wave_cuda_memref_region(rank, buf, elem, C.byref(first), C.byref(nbytes)) == wc.OK
        return (first.value or 0) - base, nbytes.value

    assert region(0, [4, 8], [8, 1], 2) == (0, 64)               # dense row-major 4 x 8 f16
    assert region(5, [10], [1], 4) == (20, 40)                   # a window at an offset
    assert region(0, [4, 8], [16, 2], 2) == (0, (3 * 16 + 7 * 2 + 1) * 2)   # strided, with holes
    assert region(9, [10], [-1], 4) == (0, 40)                   # reversed vector: lowest byte below index zero
    assert region(31, [4, 8], [-8, -1], 2) == (0, 64)            # both dimensions reversed
    assert region(24, [4, 8], [-8, 1], 2) == (0, 64)             # rows reversed only
    assert region(3, [0, 8], [8, 1], 2) == (6, 0)                # empty
    assert region(7, [], [], 8) == (56, 8)                       # rank 0: one element
    assert lib.wave_cuda_memref_region(1, None, 4, None, None) == wc.E_INVALID


PAIR = dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)


@pytest.mark.parametrize("shape,kwargs,sms,workspace,want", [
    # the benchmark's GEMM and its N-column shards on a 148-SM part (column-major C runs as C^T: swapped)
    ((8192, 8192, 8192), dict(in_type=1, out_type=1, out_layout=1, streamk_workers=0, **PAIR), 148, True,
     dict(tile_m=256, tile_n=256, grid=148, streamk_workers=0, swapped=True)),
    ((8192, 4096, 8192), dict(in_type=1, out_type=1, out_layout=1, streamk_workers=0, **PAIR), 148, True,
     dict(tile_m=256, tile_n=256, grid=148, streamk_workers=0, swapped=True)),
    ((8192, 2048, 8192), dict(in_type=1, out_type=1, out_layout=1, streamk_workers=0, **PAIR), 148, True,
     dict(tile_m=256, tile_n=256, streamk_workers=0, swapped=True)),      # 3 rounds + 34 tiles as 68 half-width items
    ((8192, 1024, 8192), dict(in_type=1, out_type=1, out_layout=1, streamk_workers=0, **PAIR), 148, True,
     dict(tile_m=256, tile_n=224, grid=148, streamk_workers=0, swapped=True)),   # 148 tiles of 224 columns: two full rounds
    # row-major, same problem: not swapped
    ((8192, 8192, 8192), dict(in_type=1, out_type=1, **PAIR), 148, False,
     dict(tile_m=256, tile_n=256, grid=148, streamk_workers=0, swapped=False)),
    # knobs that ask for 128-row tiles stay on the one-CTA kernel
    ((8192, 8192, 8192), dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4), 148, False,
     dict(tile_m=128, tile_n=256, grid=148, streamk_workers=0, swapped=False)),
    # one round of tiles either way: the one-CTA kernel's shorter tail
    ((2048, 2048, 4096), PAIR, 148, False, dict(tile_m=128, tile_n=256, swapped=False)),
    # the decode-shaped GEMM: operands swapped, K split over every SM when there is a workspace
    ((16, 28672, 8192), dict(in_type=1, bn=1, streamk_workers=0), 148, True,
     dict(tile_m=128, tile_n=16, grid=148, streamk_workers=148, swapped=True, scratch_bytes=148 * 2 * 128 * 16 * 4,
          counter_bytes=224 * 4)),
    ((16, 28672, 8192), dict(in_type=1, bn=1, streamk_workers=0), 148, False,
     dict(tile_m=128, tile_n=16, streamk_workers=0, swapped=True, scratch_bytes=0)),
    # explicit worker counts are pure Stream-K on the one-CTA kernel, whatever the part
    ((512, 768, 1024), dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4, streamk_workers=5), 132, True,
     dict(tile_m=128, tile_n=256, grid=5, streamk_workers=5, scratch_bytes=5 * 2 * 128 * 256 * 4, counter_bytes=12 * 4)),
    # a smaller part: 66 pairs
    ((8192, 8192, 8192), dict(in_type=1, out_type=1, **PAIR), 132, False, dict(tile_m=256, tile_n=256, grid=132)),
])
def test_gemm_planner_without_a_device(wc, shape, kwargs, sms, workspace, want):
    """What the backend would launch on a part of a given SM count: kernel
    (one CTA per 128-row tile, or CTA pairs on 256-row tiles), tile width,
    grid, Stream-K workers and workspace -- decided on the host, testable here."""
    plan = wc.gemm_plan_for_sms(wc.gemm_desc(*shape, **kwargs), sms, workspace)
    for key, value in want.items():
        assert plan[key] == value, (key, plan)


def test_gemm_planner_follows_the_environment_knobs(wc):
    import os
    desc = wc.gemm_desc(8192, 1024, 8192, in_type=1, out_type=1, out_layout=1, streamk_workers=0, **PAIR)
    old = {k: os.environ.get(k) for k in ("WAVE_CUDA_GEMM_PAIR_TILE_N", "WAVE_CUDA_GEMM_STREAMK_TAIL",
                                          "WAVE_CUDA_GEMM_KERNEL", "WAVE_CUDA_GEMM_COL_SWAP")}
    try:
        os.environ["WAVE_CUDA_GEMM_PAIR_TILE_N"] = "256"
        wc.reload_env()
        assert wc.gemm_plan_for_sms(desc, 148)["tile_n"] == 256
        os.environ.update(WAVE_CUDA_GEMM_STREAMK_TAIL="force", WAVE_CUDA_GEMM_KERNEL="pair")
        wc.reload_env()
        plan = wc.gemm_plan_for_sms(desc, 148)  # 74 whole tiles, then 54 tiles' K iterations over 74 pairs
        assert plan["streamk_workers"] == 74 and plan["grid"] == 148
        assert plan["scratch_bytes"] == 74 * 2 * 256 * 256 * 4 and plan["counter_bytes"] == 54 * 2 * 4
        assert wc.gemm_plan_for_sms(desc, 148, have_workspace=False)["streamk_workers"] == 0
        os.environ["WAVE_CUDA_GEMM_COL_SWAP"] = "0"
        wc.reload_env()
        assert wc.gemm_plan_for_sms(desc, 148)["swapped"] is False
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        wc.reload_env()
    assert wc.gemm_plan_for_sms(desc, 148)["tile_n"] == 224
