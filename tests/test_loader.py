"""The runtime's .param/.bin loader against the reference's own loader.

tests/golden/loader_dumps/*.txt were produced by oracle/_ref/ref_dump, i.e. by the
reference's lib/Graph/graph.cpp + parser.cpp compiled from their sources.  The
runtime's ncnn_b200_describe must reproduce them byte for byte: layer order, blob
order, inputs/outputs, lexical typing of every parameter, weight shapes, storage
types, byte counts, FNV-1a hashes of the payloads and the error messages for
malformed files.  No GPU is needed.
"""
import glob
import os

import numpy as np
import pytest

from conftest import FIXTURES, GOLDEN

DUMPS = sorted(glob.glob(os.path.join(GOLDEN, "loader_dumps", "*.txt")))


def _files_for(name):
    if name.startswith("_malformed_"):
        base = os.path.join(FIXTURES, "_malformed", name[len("_malformed_"):])
        return base + ".param", base + ".bin"
    if name.endswith(".nobin"):
        return os.path.join(FIXTURES, name[:-6] + ".param"), None
    return os.path.join(FIXTURES, name + ".param"), os.path.join(FIXTURES, name + ".bin")


@pytest.mark.parametrize("dump", [d for d in DUMPS if not os.path.basename(d).startswith("zoo_")],
                         ids=lambda d: os.path.basename(d)[:-4])
def test_describe_matches_reference_loader(pkg, dump):
    name = os.path.basename(dump)[:-4]
    param, bin_ = _files_for(name)
    with open(dump) as f:
        want = f.read()
    assert pkg.describe(param, bin_) == want


def test_reference_dumps_cover_malformed_inputs():
    names = [os.path.basename(d) for d in DUMPS if "_malformed_" in d]
    assert len(names) >= 12
    for d in DUMPS:
        if "_malformed_" in d:
            assert open(d).read().startswith("ERROR: ")


ZOO = {
    "zoo_single_conv": lambda z, p: z.single_conv(p),
    "zoo_resnet18": lambda z, p: z.resnet18(p),
    "zoo_resnet18_int8": lambda z, p: z.resnet18(p, int8=True),
    "zoo_mobilenet_v2": lambda z, p: z.mobilenet_v2(p),
    "zoo_inner_product": lambda z, p: z.inner_product(p, 512, 1024),
    "zoo_inner_product_int8": lambda z, p: z.inner_product(p, 512, 1024, int8=True),
}


@pytest.mark.parametrize("name", sorted(ZOO))
def test_zoo_models_are_deterministic_and_load_like_the_reference(pkg, tmp_path, name):
    """The synthetic benchmark models are regenerated from their seeds and must hash to
    what the reference's loader saw when the golden dump was made."""
    param, bin_ = ZOO[name](pkg.zoo, str(tmp_path / name))
    with open(os.path.join(GOLDEN, "loader_dumps", name + ".txt")) as f:
        want = f.read()
    assert pkg.describe(param, bin_) == want


def test_oracle_reader_agrees_with_reference_loader(oracle):
    """The oracle has its own Python reader; its layer list and weight sizes must agree
    with the reference loader's dump for every fixture that carries weights."""
    import re
    for dump in DUMPS:
        name = os.path.basename(dump)[:-4]
        if name.startswith(("_malformed_", "zoo_")) or name.endswith(".nobin"):
            continue
        param, bin_ = _files_for(name)
        text = open(dump).read()
        layers = oracle.load_graph(param, bin_)
        rows = [ln for ln in text.splitlines() if re.match(r"\s+\[\s*\d+\] \S", ln) and " in=[" in ln]
        assert len(rows) == len(layers), name
        for row, layer in zip(rows, layers):
            assert row.split()[2] == layer.type and row.split()[3] == layer.name
            counts = [int(np.prod([int(d) for d in m.split(",")])) for m in re.findall(r"\[([\d,]+):\w+:\d+B\]", row)]
            assert counts == [int(w.size) for w in layer.weights], (name, row)
