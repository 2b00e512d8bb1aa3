"""Fixed-rank dynamic input shapes: the `--input-shape=1x?x4` half of the reference's C ABI
(`int f(const float*, const int64_t shape[3], float*, uint64_t capacity)` plus
`f_infer_output_shapes`), its status codes in the wrapper's order (GenerateCAPI.cpp:1053-1480), and
the cases of test/Numerical/operators/dynamic_ops_test.cpp that sit on this path.  Planning and
shape inference need no GPU; running does."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import FIXTURES, ROOT, fixture, rel_l2

TOOL = os.path.join(ROOT, "ncnn-compiler_b200", "ncnn-b200-compile")
EMPTY_BIN = os.path.join(FIXTURES, "relu.bin")


def dyn_fixture(name):
    return os.path.join(FIXTURES, name + ".param")


# ------------------------------------------------------------------ CPU: planning, shapes, statuses
def test_inner_product_dynamic_m_shapes(pkg):
    """dynamic_ops_test.cpp:526-552: [1, rows, 4] -> Squeeze -> InnerProduct -> [rows, 3]."""
    param, bin_ = fixture("inner_product_dynamic_m")
    m = pkg.DynamicModel(param, bin_, [[1, None, 4]], [(0, 1, 1, 1)])
    assert m.input_shapes == [(1, -1, 4)] and m.output_shapes == [(-1, 3)]
    for rows in (3, 7, 1, 640):
        assert m.infer_status([[1, rows, 4]]) == (0, [(rows, 3)])


def test_status_codes_follow_the_wrapper_order(pkg):
    m = pkg.DynamicModel(dyn_fixture("relu_dynamic"), EMPTY_BIN, [[3, None, None]], [(0, 1, 4, 4), (0, 2, 1, 1)])
    assert m.infer_status([[3, 8, 5]]) == (0, [(3, 8, 5)])
    assert m.infer_status([[3, 0, 5]])[0] == 2       # dynamic extent must be positive
    assert m.infer_status([[3, -4, 5]])[0] == 2
    assert m.infer_status([[2, 8, 5]])[0] == 2       # static extent must match
    assert m.infer_status([[3, 6, 5]])[0] == 3       # not a multiple of 4
    assert m.infer_status([[3, 2, 5]])[0] == 3       # below the minimum (and not a multiple)
    assert m.infer_status([[2, 6, 5]])[0] == 2       # an invalid shape is reported before a violated constraint
    assert m.infer_status([[3, 2 ** 40, 2 ** 40]])[0] == 4   # element count overflows
    assert m.infer_status([[3, 4, 2 ** 40]])[0] == 4         # beyond what the planner addresses
    assert m.infer_status([[3, 6, 2 ** 62]])[0] == 3         # a violated constraint is reported before overflow
    assert m.infer_status([None])[0] == 1


def test_constraints_are_checked_at_load_like_the_compile_step(pkg):
    """docs/ncnn-compile-command-line.md 2.6: a constraint must name a `?` dimension of an existing
    input, once, with positive minimum and multiple."""
    args = (dyn_fixture("relu_dynamic"), EMPTY_BIN, [[3, None, None]])
    for bad, why in [((0, 0, 1, 1), "dynamic dimension"), ((0, 3, 1, 1), "dynamic dimension"), ((1, 1, 1, 1), "does not exist"),
                     ((0, 1, 0, 1), "positive"), ((0, 1, 1, -2), "positive")]:
        with pytest.raises(pkg.NcnnB200Error, match=why):
            pkg.DynamicModel(*args, [bad])
    with pytest.raises(pkg.NcnnB200Error, match="repeated"):
        pkg.DynamicModel(*args, [(0, 1, 1, 1), (0, 1, 2, 2)])
    with pytest.raises(pkg.NcnnB200Error, match="number of input shape overrides"):
        pkg.DynamicModel(dyn_fixture("relu_dynamic"), EMPTY_BIN, [[3, None, None], [3, None, None]])


@pytest.mark.parametrize("name,template,shape,want", [
    ("sigmoid_dynamic", [3, None, None], [3, 5, 7], [(3, 5, 7)]),
    ("pooling_global_average_dynamic", [3, None, None], [3, 9, 4], [(3,)]),
    ("pooling_padded_max_dynamic", [3, None, None], [3, 9, 10], None),
    ("pooling_adaptive_average_dynamic", [3, None, None], [3, 9, 10], [(3, 2, 3)]),
    ("pooling_adaptive_max_dynamic", [3, None, None], [3, 9, 10], [(3, 2, 10)]),
    ("slice_dynamic", [3, None, None], [3, 4, 6], [(2, 4, 6), (1, 4, 6)]),
    ("squeeze_dynamic", [1, None, None], [1, 5, 6], [(5, 6)]),
    ("permute_dynamic", [1, None, None], [1, 5, 6], [(6, 5)]),
    ("expand_dims_dynamic", [1, None, None], [1, 5, 6], [(1, 5, 6)]),
    ("reshape_spec_dynamic", [3, None, None], [3, 2, 5], None),
    ("softmax_dynamic", [3, None, None], [3, 2, 5], [(3, 2, 5)]),
    ("interp_dynamic", [4, None, None], [4, 3, 5], None),
    ("padding_dynamic", [2, None, None], [2, 3, 5], None),
])
def test_output_shapes_of_the_reference_dynamic_fixtures(pkg, oracle, name, template, shape, want):
    """Shapes planned for a concrete extent equal the oracle's result shapes (and the literal ones
    the reference's tests expect where they state them)."""
    m = pkg.DynamicModel(dyn_fixture(name), EMPTY_BIN, [template])
    status, got = m.infer_status([shape])
    assert status == 0
    x = np.zeros(shape, np.float32)
    ref = [y.shape for y in oracle.Model(dyn_fixture(name), EMPTY_BIN, input_shapes=[shape]).run([x])]
    assert got == ref
    if want is not None:
        assert got == want
    # output extents that follow the input are marked dynamic, the others keep their value
    for planned, concrete in zip(m.output_shapes, got):
        assert len(planned) == len(concrete) and all(p in (-1, c) for p, c in zip(planned, concrete))


def compile_dynamic(param, out_dir, name, shape, constraints=(), bin_=None):
    cmd = [TOOL, param, f"--output-dir={out_dir}", f"--model-name={name}", f"--input-shape={shape}"]
    cmd += [f"--input-dim-constraint={c}" for c in constraints]
    if bin_:
        cmd.append(f"--bin={bin_}")
    return subprocess.run(cmd, capture_output=True, text=True)


def test_compile_tool_emits_the_dynamic_entry_points(pkg, tmp_path):
    """Same flags as the reference's fixture build (test/Numerical/CMakeLists.txt:785-790), same two
    prototypes as its header writer (tools/ncnn-compile.cpp:1108-1215)."""
    param, _ = fixture("inner_product_dynamic_m")
    out = tmp_path / "ipm"
    r = compile_dynamic(param, str(out), "inner_product_dynamic_m", "1x?x4", ["0:1:min=1,multiple=1"])
    assert r.returncode == 0, r.stderr
    header = (out / "inner_product_dynamic_m.h").read_text()
    assert ("int inner_product_dynamic_m(const float *input1, const int64_t input1_shape[3], float *output1, "
            "uint64_t output1_capacity);") in header
    assert "int inner_product_dynamic_m_infer_output_shapes(const int64_t input1_shape[3], int64_t output1_shape[2]);" in header
    for macro in ("#define INNER_PRODUCT_DYNAMIC_M_INPUT1_DIM1 NCNN_DYNAMIC_DIM", "#define INNER_PRODUCT_DYNAMIC_M_INPUT1_DYNAMIC_DIM_MASK UINT32_C(0x2)",
                  "#define INNER_PRODUCT_DYNAMIC_M_INPUT1_DIM1_MINIMUM INT64_C(1)", "#define INNER_PRODUCT_DYNAMIC_M_OUTPUT1_DIM0 NCNN_DYNAMIC_DIM",
                  "#define INNER_PRODUCT_DYNAMIC_M_OUTPUT1_DIM1 INT64_C(3)", "#define INNER_PRODUCT_DYNAMIC_M_OUTPUT1_DYNAMIC_DIM_MASK UINT32_C(0x1)"):
        assert macro in header
    assert "OUTPUT1_ELEMENTS" not in header  # only static arguments have an element count
    nm = subprocess.run(["nm", "-D", "--defined-only", str(out / "libinner_product_dynamic_m.so")], capture_output=True, text=True).stdout
    assert sorted(l.split()[-1] for l in nm.splitlines() if " T " in l) == ["inner_product_dynamic_m", "inner_product_dynamic_m_infer_output_shapes"]
    # shape inference through the generated library needs no GPU
    lib = ctypes.CDLL(str(out / "libinner_product_dynamic_m.so"))
    infer = lib.inner_product_dynamic_m_infer_output_shapes
    infer.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    for rows in (3, 7):
        dims, res = (ctypes.c_int64 * 3)(1, rows, 4), (ctypes.c_int64 * 2)()
        assert infer(dims, res) == 0 and list(res) == [rows, 3]
    assert infer((ctypes.c_int64 * 3)(1, 0, 4), (ctypes.c_int64 * 2)()) == 2
    assert infer(None, (ctypes.c_int64 * 2)()) == 1


def test_compile_tool_fixed_output_has_no_capacity_or_infer_entry(pkg, tmp_path):
    """A dynamic input with a static result (the reference's classifier case): shape array, no
    capacity, no inference entry (numerical_test_support.cpp:218-229)."""
    param, bin_ = pkg.zoo.dynamic_convnet(str(tmp_path / "cls"), classes=10)
    out = tmp_path / "out"
    r = compile_dynamic(param, str(out), "cls", "3x?x?", ["0:1:min=8,multiple=1", "0:2:min=8,multiple=1"])
    assert r.returncode == 0, r.stderr
    header = (out / "cls.h").read_text()
    assert "int cls(const float *input1, const int64_t input1_shape[3], float *output1);" in header
    assert "infer_output_shapes" not in header and "#define CLS_OUTPUT1_ELEMENTS UINT64_C(10)" in header
    r = compile_dynamic(param, str(tmp_path / "bad"), "cls", "3x?x?", ["0:0:min=1,multiple=1"])
    assert r.returncode != 0 and "dynamic dimension" in r.stderr
    r = compile_dynamic(param, str(tmp_path / "bad2"), "cls", "3x32x32", ["0:1:min=1,multiple=1"])
    assert r.returncode != 0


# ------------------------------------------------------------------------------- GPU: running
@pytest.mark.gpu
def test_inner_product_dynamic_m_matches_the_oracle(pkg, oracle):
    param, bin_ = fixture("inner_product_dynamic_m")
    m = pkg.DynamicModel(param, bin_, [[1, None, 4]], [(0, 1, 1, 1)])
    rng = np.random.default_rng(0x1AAE2)
    for rows in (3, 7, 3, 300):
        x = rng.uniform(-1, 1, (1, rows, 4)).astype(np.float32)
        got = m.run(x)[0]
        want = oracle.Model(param, bin_, input_shapes=[[1, rows, 4]]).run([x])[0]
        assert got.shape == (rows, 3)
        assert np.allclose(got, want, rtol=0, atol=1e-5)  # the reference's tolerance for this case


@pytest.mark.gpu
def test_rejects_insufficient_capacity(pkg):
    """dynamic_ops_test.cpp:554-561: 3x3x5 needs 45 elements, 44 are offered -> status 5; nothing is written."""
    m = pkg.DynamicModel(dyn_fixture("relu_dynamic"), EMPTY_BIN, [[3, None, None]], [(0, 1, 1, 1), (0, 2, 1, 1)])
    x = np.full((3, 3, 5), -1.0, np.float32)
    y = np.full(45, 7.0, np.float32)
    assert m.run_status([x], [[3, 3, 5]], [y], [44]) == 5 and np.all(y == 7.0)
    assert m.run_status([x], [[3, 3, 5]], [y], [45]) == 0 and np.all(y == 0.0)
    assert m.run_status([x], [[3, 0, 5]], [y], [45]) == 2


@pytest.mark.gpu
@pytest.mark.parametrize("name,template,shapes", [
    ("relu_dynamic", [3, None, None], [[3, 3, 5], [3, 17, 9]]),
    ("sigmoid_dynamic", [3, None, None], [[3, 4, 4], [3, 5, 12]]),
    ("softmax_dynamic", [3, None, None], [[3, 4, 4], [3, 5, 12]]),
    ("pooling_global_average_dynamic", [3, None, None], [[3, 6, 6], [3, 9, 4]]),
    ("pooling_padded_max_dynamic", [3, None, None], [[3, 6, 6], [3, 9, 10]]),
    ("pooling_adaptive_average_dynamic", [3, None, None], [[3, 6, 6], [3, 9, 10], [3, 1, 2]]),
    ("pooling_adaptive_max_dynamic", [3, None, None], [[3, 6, 6], [3, 9, 10], [3, 1, 2]]),
    ("slice_dynamic", [3, None, None], [[3, 4, 6], [3, 8, 5]]),
    ("squeeze_dynamic", [1, None, None], [[1, 5, 6], [1, 2, 9]]),
    ("permute_dynamic", [1, None, None], [[1, 5, 6], [1, 2, 9]]),
    ("expand_dims_dynamic", [1, None, None], [[1, 5, 6], [1, 2, 9]]),
    ("interp_dynamic", [4, None, None], [[4, 3, 5], [4, 6, 6]]),
    ("padding_dynamic", [2, None, None], [[2, 3, 5], [2, 6, 6]]),
])
def test_dynamic_fixtures_match_the_oracle_across_shapes(pkg, oracle, name, template, shapes):
    m = pkg.DynamicModel(dyn_fixture(name), EMPTY_BIN, [template])
    rng = np.random.default_rng(11)
    for shape in shapes + shapes[:1]:  # the first shape again: replayed from the table
        x = rng.uniform(-2, 2, shape).astype(np.float32)
        got = m.run(x)
        want = oracle.Model(dyn_fixture(name), EMPTY_BIN, input_shapes=[shape]).run([x])
        assert len(got) == len(want)
        for g, w in zip(got, want):
            assert g.shape == w.shape and np.allclose(g, w, rtol=0, atol=2e-6)


@pytest.mark.gpu
def test_dynamic_convolution_network_through_the_generated_library(pkg, oracle, tmp_path):
    """A fully convolutional network compiled with `--input-shape=3x?x?` and called through dlopen
    with the reference's dynamic signature; the result extents follow the input ([8, H/2, W/2])."""
    param, bin_ = pkg.zoo.dynamic_convnet(str(tmp_path / "fcn"))
    out = tmp_path / "out"
    r = compile_dynamic(param, str(out), "fcn", "3x?x?", ["0:1:min=8,multiple=2", "0:2:min=8,multiple=2"])
    assert r.returncode == 0, r.stderr
    lib = ctypes.CDLL(str(out / "libfcn.so"))
    lib.fcn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_uint64]
    lib.fcn_infer_output_shapes.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    rng = np.random.default_rng(5)
    for h, w in [(32, 48), (64, 40), (32, 48)]:
        dims, res = (ctypes.c_int64 * 3)(3, h, w), (ctypes.c_int64 * 3)()
        assert lib.fcn_infer_output_shapes(dims, res) == 0 and list(res) == [8, h // 2, w // 2]
        x = rng.uniform(-1, 1, (3, h, w)).astype(np.float32)
        y = np.empty(list(res), np.float32)
        assert lib.fcn(x.ctypes.data, dims, y.ctypes.data, y.size) == 0
        want = oracle.Model(param, bin_, input_shapes=[[3, h, w]]).run([x])[0]
        assert rel_l2(y, want) <= 1e-4  # fp32 contraction tolerance: rel-L2 <= 1e-3 required, ~1e-5 achieved
        assert lib.fcn(x.ctypes.data, dims, y.ctypes.data, y.size - 1) == 5
    assert lib.fcn(x.ctypes.data, (ctypes.c_int64 * 3)(3, 33, 48), y.ctypes.data, y.size) == 3  # multiple of 2
    assert lib.fcn(x.ctypes.data, (ctypes.c_int64 * 3)(3, 4, 48), y.ctypes.data, y.size) == 3   # minimum 8
    assert lib.fcn(None, dims, y.ctypes.data, y.size) == 1 and lib.fcn(x.ctypes.data, None, y.ctypes.data, y.size) == 1


@pytest.mark.gpu
def test_dynamic_classifier_keeps_a_fixed_output(pkg, oracle, tmp_path):
    param, bin_ = pkg.zoo.dynamic_convnet(str(tmp_path / "cls"), classes=10)
    m = pkg.DynamicModel(param, bin_, [[3, None, None]], [(0, 1, 8, 1), (0, 2, 8, 1)])
    assert m.output_shapes == [(10,)]
    rng = np.random.default_rng(6)
    for h, w in [(24, 24), (57, 31)]:
        x = rng.uniform(-1, 1, (3, h, w)).astype(np.float32)
        got = m.run(x)[0]
        want = oracle.Model(param, bin_, input_shapes=[[3, h, w]]).run([x])[0]
        assert rel_l2(got, want) <= 1e-4
