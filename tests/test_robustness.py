"""Host-side robustness of the boundary: malformed graphs are refused with a message (never a crash or an
exception across the C ABI), generated stubs survive awkward paths, and the loader is clean under
AddressSanitizer + UndefinedBehaviorSanitizer on the reference's fixtures, its malformed inputs, truncated
weight files and byte-flipped graphs (the reference's own CI runs its tests under the same sanitizers,
.github/workflows/ci.yml:49-62).  None of this needs a GPU."""
import glob
import os
import subprocess

import pytest

from conftest import FIXTURES, ROOT, fixture


def _write(tmp_path, name, lines):
    path = tmp_path / (name + ".param")
    path.write_text("7767517\n%d %d\n" % (len(lines), 8) + "\n".join(lines) + "\n")
    (tmp_path / (name + ".bin")).write_bytes(b"")
    return str(path), str(tmp_path / (name + ".bin"))


@pytest.mark.parametrize("layer", ["Pooling pool 0 1 out 0=0 1=2", "Softmax sm 0 1 out 0=0", "ReLU relu 1 0 data 0=0.0",
                                   "Eltwise add 0 1 out 0=1", "Convolution c 0 1 out 0=2 1=1 6=2",
                                   "InnerProduct ip 0 1 out 0=2 2=2", "Concat cat 0 1 out 0=0"])
def test_layers_without_blobs_are_refused_not_dereferenced(pkg, tmp_path, layer):
    param, bin_ = _write(tmp_path, "m", ["Input input 0 1 data 0=4 1=4 2=1", layer])
    with pytest.raises(pkg.NcnnB200Error) as err:
        pkg.Model(param, bin_, plan_only=True)
    assert err.value.status in (6, 8) and str(err.value)


def test_rank4_shapes_are_planned_and_declared(pkg, tmp_path):
    """Rank-4 results [c,d,h,w] of Reshape / Permute / Slice / Concat (the reference's permute_rank4, slice_rank4 and
    concat_rank4 fixtures): shapes through the four-extent accessors, RANK 4 and DIM0..DIM3 in the emitted header,
    and a loud refusal for layers that do not take rank-4 input."""
    for name, shapes in (("permute_rank4", [(2, 2, 2, 3)]), ("slice_rank4", [(4, 1, 1, 2), (4, 1, 1, 4)]),
                         ("concat_rank4", [(1, 2, 2, 4)])):
        m = pkg.Model(*fixture(name), plan_only=True)
        assert m.output_shapes == shapes
        m.emit_stub(name, *fixture(name), str(tmp_path))
        m.close()
    header = (tmp_path / "permute_rank4.h").read_text()
    assert "PERMUTE_RANK4_OUTPUT1_RANK 4" in header and "PERMUTE_RANK4_OUTPUT1_DIM3 INT64_C(3)" in header
    assert "PERMUTE_RANK4_OUTPUT1_ELEMENTS" in header
    param, bin_ = _write(tmp_path, "p", ["Input input 0 1 data 0=4 1=2 2=3", "Reshape r 1 1 data m 0=2 1=2 11=3 2=2",
                                         "Pooling pool 1 1 m out 0=0 1=2"])
    with pytest.raises(pkg.NcnnB200Error) as err:
        pkg.Model(param, bin_, plan_only=True)
    assert err.value.status == 8 and "rank-4" in str(err.value)


def test_stub_escapes_quotes_and_backslashes_in_paths(pkg, tmp_path):
    param, bin_ = fixture("convolution")
    m = pkg.Model(param, bin_, plan_only=True)
    awkward_param = 'dir with "quotes"\\and\\backslashes/model.param'
    m.emit_stub("conv", awkward_param, "weights\\\".bin", str(tmp_path))
    m.close()
    text = (tmp_path / "conv.c").read_text()
    assert 'dir with \\"quotes\\"\\\\and\\\\backslashes/model.param' in text
    assert 'weights\\\\\\".bin' in text
    # and it is still C
    subprocess.check_call(["gcc", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(tmp_path / "conv.c")])


def test_loader_is_clean_under_address_and_undefined_sanitizers(tmp_path):
    exe = tmp_path / "loader_sanitize"
    src = os.path.join(ROOT, "tests", "sanitize", "loader_sanitize_main.cpp")
    loader = os.path.join(ROOT, "ncnn-compiler_b200", "csrc", "loader.cpp")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
                           "-fno-omit-frame-pointer", "-o", str(exe), src, loader])
    params = sorted(glob.glob(os.path.join(FIXTURES, "*.param")) + glob.glob(os.path.join(FIXTURES, "_malformed", "*.param")))
    assert len(params) > 100
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    out = subprocess.run([str(exe), str(tmp_path)] + params, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "failures without a message 0" in out.stdout
