"""CPU tests of the host side: the C-ABI library loads and exports what the header declares,
argument errors come back as codes without any launch, and the tile selector is sane."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_fp8_mm.h")


def header_functions():
    """Every function any header under include/ declares."""
    names = set()
    inc = os.path.dirname(HEADER)
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text = re.sub(r"/\*.*?\*/", "", open(os.path.join(inc, f)).read(), flags=re.S)
            names |= set(re.findall(r"\b(b200_(?:fp8_mm|mla)\w*)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(built_library):
    from amd_developer_challenge_2025_b200 import _lib

    lib = ctypes.CDLL(built_library)
    declared = header_functions()
    assert "b200_fp8_mm" in declared and "b200_fp8_mm_describe" in declared
    for name in declared:
        assert hasattr(lib, name), name
    assert sorted(_lib.EXPORTS) == [d for d in declared if d in _lib.EXPORTS]
    assert set(declared) <= set(_lib.EXPORTS) | {"b200_fp8_mm_plan"}
    assert _lib.load().b200_fp8_mm_abi_version() == _lib.ABI_VERSION


def test_error_codes_without_launch(built_library):
    from amd_developer_challenge_2025_b200 import _lib

    lib = _lib.load()
    one = ctypes.c_void_p(4096)  # never dereferenced: every check below fails first

    def call(a=one, b=one, a_s=one, b_s=one, c=one, m=128, n=128, k=128, lda=None, ldb=None, ldc=None, phase=0):
        return lib.b200_fp8_mm(a, b, a_s, b_s, c, m, n, k, lda or k, ldb or k, k // 128 or 1, 1, k // 128 or 1, 1,
                               ldc or n, phase, None, 0, None, None)

    assert call(a=None) == 1 and call(c=None) == 1
    assert call(k=100) == 2 and call(m=0) == 2 and call(n=-5) == 2
    assert call(lda=130) == 3 and call(ldb=64) == 3 and call(ldc=64) == 3
    assert call(a=ctypes.c_void_p(4100)) == 4
    assert call(phase=128) == 5 and call(phase=16) == 5 and call(phase=-32) == 5
    for code in range(0, 10):
        assert len(_lib.strerror(code)) > 0
    assert "unknown" in _lib.strerror(99)


def test_error_codes_of_the_strided_and_grouped_entry_points(built_library):
    from amd_developer_challenge_2025_b200 import _lib

    lib = _lib.load()
    one = ctypes.c_void_p(4096)  # never dereferenced: every check below fails first

    def strided(a=one, m=128, n=128, k=128, a_sm=None, a_sk=1, b_sn=None, b_sk=1, plan=None):
        return lib.b200_fp8_mm_strided(a, one, one, one, one, m, n, k, k if a_sm is None else a_sm, a_sk,
                                       k if b_sn is None else b_sn, b_sk, 1, 1, 1, 1, n, 0, None, 0, None, None, plan)

    assert strided(a=None) == 1 and strided(k=64) == 2
    assert strided(a_sm=2, a_sk=2) == 3             # neither K nor M contiguous
    assert strided(a_sm=1, a_sk=120) == 3           # MN-major with a pitch smaller than M
    assert strided(a_sm=1, a_sk=136) == 3           # MN-major pitch not a multiple of 16
    assert strided(b_sn=1, b_sk=100) == 3

    def grouped(a=one, g=2, m=128, n=128, k=128, lda=None, a_g=None, ldb=None, b_g=None, ldc=None, c_g=None,
                plan=None):
        lda, ldb, ldc = lda or k, ldb or k, ldc or n
        return lib.b200_fp8_mm_grouped(a, one, one, one, one, g, m, n, k, lda, a_g or m * lda, ldb, b_g or n * ldb,
                                       m, 1, 1, 1, 1, 1, ldc, c_g or m * ldc, None, None, None, plan)

    assert grouped(a=None) == 1
    assert grouped(g=0) == 2 and grouped(k=100) == 2 and grouped(m=0) == 2
    assert grouped(lda=100) == 3 and grouped(a_g=1000) == 3 and grouped(c_g=64) == 3
    assert grouped(a=ctypes.c_void_p(4104)) == 4
    assert len(_lib.strerror(10)) > 0


def test_grouped_wrapper_rejects_cpu_tensors(built_library):
    import amd_developer_challenge_2025_b200 as pkg

    parts = [pkg.make_inputs(8, 128, 128, seed=i) for i in range(2)]
    a, b, a_s, b_s, c = (torch.stack([p[j] for p in parts]) for j in range(5))
    with pytest.raises(ValueError, match="CUDA"):
        pkg.fp8_mm_grouped(a, b, a_s, b_s, c)


def test_python_wrapper_rejects_cpu_tensors_and_bad_shapes(built_library):
    import amd_developer_challenge_2025_b200 as pkg

    a, b, a_s, b_s, c = pkg.make_inputs(8, 128, 128, seed=1)
    with pytest.raises(ValueError, match="CUDA"):
        pkg.custom_kernel((a, b, a_s, b_s, c))


def test_selector_is_pure_and_sane(built_library):
    import amd_developer_challenge_2025_b200 as pkg

    shapes = [(m, n, k) for m in (256, 512, 2048, 8192, 16384)
              for (n, k) in ((1536, 7168), (3072, 1536), (576, 7168), (7168, 256), (7168, 2048), (4608, 7168),
                             (7168, 2304), (512, 7168), (4096, 512))]
    for (m, n, k) in shapes:
        p1, p2 = pkg.describe(m, n, k), pkg.describe(m, n, k)
        assert p1 == p2
        assert p1.block_m == 128 and p1.block_n in (64, 128, 192, 256)
        assert 1 <= p1.split_k <= k // 128
        assert 2 <= p1.stages <= 8 and p1.smem_bytes <= 232448
        assert p1.store_bufs in (0, 1, 2, 3, 4) and 0 <= p1.full_tiles <= p1.tiles
        assert (p1.full_tiles == p1.tiles) == (p1.split_k == 1)
        assert (p1.store_bufs == 0) == (p1.full_tiles == 0)
        tiles = -(-m // (p1.block_m * (2 if p1.cta_pair else 1))) * -(-n // p1.block_n)
        assert p1.tiles == tiles
        assert 1 <= p1.grid <= 148 and p1.grid <= tiles * p1.split_k * (2 if p1.cta_pair else 1)
        # the size covers both this plan and the single-CTA plan that MN-major operands would get
        ws = pkg.workspace_bytes(m, n, k)
        single = pkg.workspace_bytes(m, n, k, pkg.Plan(cta_pair=-1))
        assert ws >= single and (ws == 0) == (p1.split_k == 1 and single == 0)
        if p1.split_k > 1:
            assert ws >= 4096 + (p1.tiles - p1.full_tiles) * p1.split_k * 128 * p1.block_n * 4
    with pytest.raises(Exception):
        pkg.describe(128, 128, 100)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from amd_developer_challenge_2025_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_product_never_imports_oracle():
    pkg_dir = os.path.join(ROOT, "amd_developer_challenge_2025_b200")
    for dirpath, _, files in os.walk(pkg_dir):
        for f in files:
            if f.endswith((".py", ".cu", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("oracle and", "").replace("CPU oracle", ""), f


def test_runner_spec_parser_and_grid():
    from amd_developer_challenge_2025_b200 import runner

    cases = runner.parse_spec("m: 1024; n: 576 ; k: 7168; seed: 7\n\n# comment\nm: 8; n: 16; k: 128\n")
    assert cases == [(1024, 576, 7168, 7), (8, 16, 128, 0)]
    with pytest.raises(ValueError):
        runner.parse_spec("m: 8; n: 16")
    grid = runner.competition_cases()
    assert len(grid) == 18 and all(k % 128 == 0 for (_, _, k, _) in grid)
    # two values of m times the same nine (n, k) pairs, every case with a seed of its own
    assert sorted({m for (m, _, _, _) in grid}) == [1024, 6144]
    assert {(n, k) for (m, n, k, _) in grid if m == 1024} == {(n, k) for (m, n, k, _) in grid if m == 6144}
    assert len({(n, k) for (_, n, k, _) in grid}) == 9 and len({s for (*_, s) in grid}) == 18


def test_host_row_ranges_cover_the_rows_in_order():
    from amd_developer_challenge_2025_b200.fp8_mm import host_row_chunks
    for m in (1, 128, 512, 640, 1024, 2304, 8192, 8192 + 128, 16384):
        for chunk in (256, 512, 1024, 4096):
            ranges = host_row_chunks(m, chunk)
            assert ranges[0][0] == 0 and ranges[-1][1] == m
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            assert all(r0 < r1 for r0, r1 in ranges)
            assert all(r0 % 128 == 0 for r0, _ in ranges)
            if m > 512:
                assert ranges[0] == (0, 256)                 # the first copy back can start early
                assert ranges[-1][1] - ranges[-1][0] <= max(256, chunk // 2) or chunk <= 256
