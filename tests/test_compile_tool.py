"""ncnn-b200-compile, the sm_100a counterpart of the reference's `ncnn-compile` driver:
model.param/.bin -> lib<model>.so + <model>.h + <model>.json with the reference's entry
signature, header layout and export rule.  Emission needs no GPU; running the stub does."""
import ctypes
import json
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, fixture, rel_l2

TOOL = os.path.join(ROOT, "ncnn-compiler_b200", "ncnn-b200-compile")


def compile_model(param, out_dir, name=None, extra=()):
    cmd = [TOOL, param, f"--output-dir={out_dir}", *extra]
    if name:
        cmd.append(f"--model-name={name}")
    return subprocess.run(cmd, capture_output=True, text=True)


def test_emits_reference_shaped_artifacts_without_a_gpu(pkg, tmp_path):
    param, _ = fixture("relu")
    out = tmp_path / "relu_all"
    r = compile_model(param, str(out), "relu_all", ["--threads=4", "--march=native", "-O3"])  # CPU flags are ignored
    assert r.returncode == 0, r.stderr
    header = (out / "relu_all.h").read_text()
    # the reference records 1217 bytes for this very artifact (test/Native/static_artifact_baseline.json:10-13)
    assert len(header.encode()) == 1217
    assert "int relu_all(const float *input1, float *output1);" in header
    for macro in ("#define NCNN_STATUS_NULL_POINTER 1", "#define RELU_ALL_INPUT_COUNT 1", "#define RELU_ALL_OUTPUT1_RANK 3",
                  "#define RELU_ALL_INPUT1_DIM0 INT64_C(3)", "#define RELU_ALL_OUTPUT1_SHAPE_DEPENDS_ON_DATA 0"):
        assert macro in header
    manifest = json.loads((out / "relu_all.json").read_text())
    assert manifest["function"] == "relu_all"
    assert manifest["inputs"] == [{"name": "input1", "shape": [3, 4, 5], "element_type": "f32", "dynamic_dim_mask": 0}]
    assert manifest["target"]["cpu"] == "sm_100a"
    nm = subprocess.run(["nm", "-D", "--defined-only", str(out / "librelu_all.so")], capture_output=True, text=True).stdout
    assert [l.split()[-1] for l in nm.splitlines() if " T " in l] == ["relu_all"]  # the entry symbol and nothing else


def test_whole_network_compiles_and_int8_keeps_an_f32_abi(pkg, tmp_path):
    param, _ = pkg.zoo.resnet18(str(tmp_path / "resnet-18"), int8=True, size=64)
    out = tmp_path / "out"
    r = compile_model(param, str(out))
    assert r.returncode == 0, r.stderr
    header = (out / "resnet_18.h").read_text()  # resnet-18 -> resnet_18, as the reference sanitises names
    assert "int resnet_18(const float *input1, float *output1);" in header
    assert "int8_t" not in header and "#define RESNET_18_OUTPUT1_ELEMENTS UINT64_C(1000)" in header


@pytest.mark.parametrize("given,want", [("resnet-50", "resnet_50"), ("123model", "ncnn_123model"), ("main", "ncnn_main"),
                                        ("_x", "ncnn__x"), ("a..b  c", "a_b_c"), ("float", "ncnn_float")])
def test_model_name_sanitising_follows_the_reference(pkg, given, want):
    r = subprocess.run([TOOL, "whatever.param", f"--model-name={given}", "--print-model-name"], capture_output=True, text=True)
    assert r.stdout.strip() == want


def test_rejects_what_the_runtime_cannot_run(pkg, tmp_path):
    from conftest import FIXTURES
    r = compile_model(os.path.join(FIXTURES, "detection_output.param"), str(tmp_path / "o"), extra=[f"--bin={fixture('relu')[1]}"])
    assert r.returncode != 0 and "outside the supported path" in r.stderr
    r = compile_model(fixture("relu")[0], str(tmp_path / "o2"), extra=["--target=x86_64"])
    assert r.returncode != 0


def test_plan_only_models_refuse_to_run(pkg):
    param, bin_ = fixture("relu")
    m = pkg.Model(param, bin_, plan_only=True)
    assert m.input_shapes == [(3, 4, 5)]
    x = np.zeros((1, 3, 4, 5), np.float32)
    assert m.run_raw(1, [x.ctypes.data], [x.ctypes.data]) == 6


@pytest.mark.gpu
def test_generated_library_is_a_drop_in_for_the_reference_entry(pkg, oracle, tmp_path):
    """dlopen lib<model>.so, call `int model(const float*, float*)` exactly as the reference's
    test harness does (numerical_test_support.cpp:161-202), compare with the oracle."""
    param, bin_ = pkg.zoo.single_conv(str(tmp_path / "conv"), h=24, w=20)
    out = tmp_path / "out"
    r = compile_model(param, str(out), "conv")
    assert r.returncode == 0, r.stderr
    lib = ctypes.CDLL(str(out / "libconv.so"))
    lib.conv.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    x = np.random.default_rng(8).uniform(-1, 1, (64, 24, 20)).astype(np.float32)
    y = np.empty((64, 24, 20), np.float32)
    assert lib.conv(x.ctypes.data, y.ctypes.data) == 0
    want = oracle.Model(param, bin_).run([x])[0]
    assert rel_l2(y, want) <= 1e-4
    y2 = np.empty_like(y)
    assert lib.conv(x.ctypes.data, y2.ctypes.data) == 0 and np.array_equal(y, y2)  # repeated calls agree
    assert lib.conv(None, y.ctypes.data) == 1 and lib.conv(x.ctypes.data, None) == 1  # NULL -> status 1
