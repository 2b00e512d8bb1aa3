"""The C-ABI library loads and exports exactly what include/ncnn_b200.h declares.
No compute call is made here: without a GPU the library must refuse loudly."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT, fixture


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ncnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ncnn_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("ncnn_b200_load", "ncnn_b200_free", "ncnn_b200_last_error", "ncnn_b200_run",
                 "ncnn_b200_run_batch", "ncnn_b200_run_batch_device", "ncnn_b200_describe",
                 "ncnn_b200_op_quantize", "ncnn_b200_op_dequantize", "ncnn_b200_op_requantize",
                 "ncnn_b200_emit_stub"):
        assert must in names


def test_library_exports_every_declared_symbol_and_nothing_else(pkg):
    lib = ctypes.CDLL(pkg.lib_path())
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", pkg.lib_path()], capture_output=True, text=True).stdout
    exported = sorted(line.split()[-1] for line in out.splitlines() if " T " in line)
    assert exported == declared_symbols()  # only the C ABI leaves the library


def test_null_arguments_are_rejected_without_a_gpu(pkg):
    lib = pkg.load_library()
    assert lib.ncnn_b200_load(b"x.param", b"x.bin", None, None) == 1
    assert lib.ncnn_b200_input_count(None) == -1
    assert lib.ncnn_b200_run(None, None, None) == 1
    assert lib.ncnn_b200_op_quantize(None, None, 4, 1, 1, None, 1, None) == 1


@pytest.mark.skipif(os.path.exists("/dev/nvidia0"), reason="checks the behaviour of a box without a GPU")
def test_load_fails_loudly_without_a_gpu(pkg):
    param, bin_ = fixture("convolution")
    with pytest.raises(pkg.NcnnB200Error) as e:
        pkg.Model(param, bin_)
    assert e.value.status == 6
    assert "no CPU path" in e.value.message


def test_missing_library_is_an_error_not_a_fallback(pkg, monkeypatch):
    from ncnn_compiler_b200 import runtime
    monkeypatch.setattr(runtime, "_LIB", None)
    monkeypatch.setattr(runtime, "lib_path", lambda: "/nonexistent/libncnn_b200.so")
    with pytest.raises(pkg.NcnnB200Error):
        runtime.load_library()


def test_shard_range_covers_the_batch_exactly(pkg):
    for total in (0, 1, 7, 64, 256, 257):
        for world in (1, 2, 3, 4, 8):
            spans = [pkg.shard_range(total, world, r) for r in range(world)]
            covered = [i for b, e in spans for i in range(b, e)]
            assert covered == list(range(total))
            assert max(e - b for b, e in spans) == -(-total // world) if total else True
    with pytest.raises(ValueError):
        pkg.shard_range(4, 2, 2)


def test_multi_device_partition_is_contiguous_and_complete(pkg):
    """The shards ncnn_b200_multi_run_batch hands to its devices: contiguous, ceil(n / devices) images each, the
    last ones short or empty, every image exactly once (pure arithmetic: no GPU)."""
    for n in (1, 2, 7, 32, 255, 256, 1000):
        for parts in (1, 2, 3, 4, 8):
            shards = pkg.multi_partition(n, parts)
            per = -(-n // parts)
            assert len(shards) == parts
            covered = []
            for first, count in shards:
                assert 0 <= count <= per
                covered.extend(range(first, first + count))
            assert covered == list(range(n))
            assert all(c == per for _, c in shards[:n // per])
    import pytest as _pytest
    with _pytest.raises(pkg.NcnnB200Error):
        pkg.multi_partition(4, 0)
