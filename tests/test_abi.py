"""CPU-side checks of the drop-in boundary: the library builds for sm_100a, loads, exports
every symbol the header declares, and refuses to work without a device (no CPU path)."""
import re
from pathlib import Path

import pytest

import lex_gpu_b200 as L
from lex_gpu_b200 import build, device

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return L.load_library()


def test_every_declared_symbol_is_exported(lib):
    header = (ROOT / "include" / "lexb.h").read_text()
    declared = re.findall(r"LEXB_API\s+[\w\s\*]+?\b(lexb_\w+)\s*\(", header)
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in lexb.h but not exported"
    assert set(declared) == set(device.SYMBOLS)


def test_version_string(lib):
    assert b"sm_100a" in lib.lexb_version()


def test_shard_rows_partitions_whole_tiles():
    for n, world in [(17408, 8), (17408, 4), (17408, 2), (5120, 8), (5120, 4), (5120, 2), (640, 3), (128, 4)]:
        spans = [L.shard_rows(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0
        assert all((hi - lo) % 128 == 0 for lo, hi in spans)
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 128
    assert L.shard_rows(17408, 8, 3) == (6528, 8704)


def test_shard_rows_rejects_bad_arguments():
    with pytest.raises(L.LexbError) as e:
        L.shard_rows(100, 2, 0)
    assert "128" in str(e.value)
    with pytest.raises(L.LexbError):
        L.shard_rows(1024, 2, 2)
    with pytest.raises(L.LexbError):
        L.shard_rows(1024, 0, 0)


def test_open_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(L.LexbError) as e:
        L.Gpu(0)
    assert "no CPU path" in str(e.value)


def test_product_package_does_not_touch_the_oracle():
    """The oracle is test infrastructure: nothing under the package may import, load or call it."""
    banned = re.compile(r"from\s+oracle|import\s+oracle|liblexoracle|lexo_")
    for p in (ROOT / "lex_gpu_b200").rglob("*"):
        if p.suffix in {".py", ".cu", ".cuh", ".h"}:
            assert not banned.search(p.read_text()), p
