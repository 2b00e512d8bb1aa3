"""GPU parity of the paths that the benchmark configurations exercise at full width: the contraction kernel
on CTA pairs (with and without tiles split between pairs), the whole InnerProduct/Gemm grid, Gemm on the
tensor cores with alpha and beta, Conv -> BatchNorm folding, and the batch-256 property checks.

Bars as everywhere: int8 bit exact against the oracle; fp32 relative L2 <= 1e-4 per layer (1e-3 is what the
benchmark contract allows), stated per test.
"""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _kernels(model, n):
    return [r["kernel"] for r in model.profile(n, 1)]


def _run(pkg, param, bin_, x, **kw):
    m = pkg.Model(param, bin_, **kw)
    got = m.run(x)[0].copy()
    kernels = _kernels(m, x.shape[0])
    m.close()
    return got, kernels


# ------------------------------------------------------------------ CTA pairs against the one-CTA kernel
def _force(monkeypatch, pairs, split):
    """pairs: every deep contraction goes to CTA pairs, whatever its width and tile count (by default only wide
    tiles that fill a wave do); split: tiles are split between workers wherever the workspace allows."""
    monkeypatch.setenv("NCNN_B200_CTA2", "1")
    monkeypatch.setenv("NCNN_B200_CTA2_ALWAYS", "1" if pairs else "0")
    monkeypatch.setenv("NCNN_B200_CTA2_MIN_BN", "32" if pairs else "192")
    monkeypatch.setenv("NCNN_B200_STREAMK", "1" if split else "0")


@pytest.mark.parametrize("h,c,cout,n", [(56, 64, 96, 8), (28, 128, 128, 8), (14, 256, 256, 16), (7, 512, 512, 24),
                                         (9, 192, 320, 5)])
def test_pair_kernel_equals_one_cta_kernel(pkg, oracle, tmp_path, monkeypatch, h, c, cout, n):
    """A tile of the pair kernel is 256 rows on two CTAs; every output still accumulates its K blocks in the
    same order as on one CTA, so the results are the same bits (whole tiles, nothing split)."""
    param, bin_ = pkg.zoo.residual_block(str(tmp_path / "rb"), h=h, w=h, c=c, cout=cout)
    x = np.random.default_rng(h + c).uniform(-1, 1, (n, c, h, h)).astype(np.float32)
    _force(monkeypatch, pairs=True, split=False)
    got, kernels = _run(pkg, param, bin_, x)
    assert any(k.startswith("tc_gemm2_kernel:pairs<") for k in kernels), kernels
    monkeypatch.setenv("NCNN_B200_CTA2", "0")
    base, kernels = _run(pkg, param, bin_, x)
    assert not any(k.startswith("tc_gemm2_kernel") for k in kernels), kernels
    assert np.array_equal(got, base)
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert rel_l2(got[:2], want) <= 1e-4


@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("h,c,cout,n", [(14, 256, 256, 16), (7, 512, 512, 24), (28, 128, 128, 8), (9, 192, 320, 24)])
def test_split_tiles_fp32(pkg, oracle, tmp_path, monkeypatch, pairs, h, c, cout, n):
    """Tiles split between workers (CTA pairs, or single CTAs): partial sums are added in a fixed order, so the
    result is reproducible; it differs from the unsplit sum by the rounding of the accumulator (tensor memory
    accumulates in fp32 with truncation, ~1e-5 relative L2 either way)."""
    param, bin_ = pkg.zoo.residual_block(str(tmp_path / "rb"), h=h, w=h, c=c, cout=cout)
    x = np.random.default_rng(h * c).uniform(-1, 1, (n, c, h, h)).astype(np.float32)
    _force(monkeypatch, pairs=pairs, split=True)
    got, kernels = _run(pkg, param, bin_, x)
    name = "tc_gemm2_kernel:pairs+split<" if pairs else "tc_gemm2_kernel:split<"
    assert any(k.startswith(name) for k in kernels), kernels
    again, _ = _run(pkg, param, bin_, x)
    assert np.array_equal(got, again)
    monkeypatch.setenv("NCNN_B200_CTA2", "0")
    base, _ = _run(pkg, param, bin_, x)
    assert rel_l2(got, base) <= 3e-5
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert rel_l2(got[:2], want) <= 1e-4


@pytest.mark.parametrize("pairs,split", [(True, False), (True, True), (False, True)])
def test_workers_int8_resnet18_bit_exact(pkg, oracle, tmp_path, monkeypatch, pairs, split):
    """Integer sums do not depend on their order: the int8 network on CTA pairs or on single CTAs, tiles split
    or not, is bit exact."""
    param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r18q"), int8=True)
    x = np.random.default_rng(401).uniform(-1, 1, (3, 3, 224, 224)).astype(np.float32)
    _force(monkeypatch, pairs=pairs, split=split)
    got, kernels = _run(pkg, param, bin_, x)
    assert any(k.startswith("tc_gemm2_kernel") for k in kernels), kernels
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert np.array_equal(got, want)


@pytest.mark.parametrize("pairs", [True, False])
def test_split_tiles_repeat_and_recover_flags(pkg, tmp_path, monkeypatch, pairs):
    """The flag words of the split workspace are back at zero after every launch: many runs in a row, with another
    batch size in between, give the same bits."""
    _force(monkeypatch, pairs=pairs, split=True)
    param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r18"), size=64, classes=100)
    rng = np.random.default_rng(9)
    x = rng.uniform(-1, 1, (64, 3, 64, 64)).astype(np.float32)
    m = pkg.Model(param, bin_)
    assert any("split<" in k for k in _kernels(m, 64))
    first = m.run(x)[0].copy()
    for _ in range(5):
        assert np.array_equal(m.run(x)[0], first)
    m.run(x[:5])
    assert np.array_equal(m.run(x)[0], first)
    m.check_status()  # raises when the device status word is set
    m.close()


# ------------------------------------------------------------------ config 4: the whole InnerProduct grid
GRID = [(m, k, n) for m in (1, 32, 256, 4096) for k in (512, 1024, 4096) for n in (512, 1024, 4096)]


def _oracle_rows(oracle, param, bin_, x, rows):
    model = oracle.Model(param, bin_)
    return np.stack([model.run([x[i]])[0] for i in rows])


@pytest.mark.parametrize("m,k,n", GRID)
def test_inner_product_grid(pkg, oracle, tmp_path, m, k, n):
    """Every (M, K, N) of the sweep, fp32 (rel-L2 <= 1e-4) and int8 (bit exact).  The oracle is a scalar loop, so
    at M = 4096 it checks 48 rows spread over the batch; the other rows are covered by the row-independence
    check (a row's result does not depend on which rows share its tile)."""
    x = np.random.default_rng(500 + m).uniform(-1, 1, (m, 1, 1, k)).astype(np.float32)
    rows = list(range(m)) if m <= 256 else sorted(set(np.random.default_rng(1).integers(0, m, 44).tolist() + [0, 127, 128, m - 1]))
    for int8 in (False, True):
        param, bin_ = pkg.zoo.inner_product(str(tmp_path / ("ipq" if int8 else "ip")), k, n, int8=int8)
        model = pkg.Model(param, bin_)
        got = model.run(x)[0].copy()
        if m > 256:
            # (a smaller batch may be planned with other tiles; fp32 sums then round differently)
            sub = model.run(x[rows])[0]
            assert np.array_equal(sub, got[rows]) if int8 else rel_l2(sub, got[rows]) <= 3e-5
        model.close()
        want = _oracle_rows(oracle, param, bin_, x, rows)
        if int8:
            assert np.array_equal(got[rows], want)
        else:
            assert rel_l2(got[rows], want) <= 1e-4


@pytest.mark.parametrize("m,k,n", [(3, 4104, 1031), (8, 2048, 4097), (5, 8192, 528), (1, 25088, 512)])
def test_few_rows_take_one_pass_over_the_weights(pkg, oracle, tmp_path, m, k, n):
    """InnerProduct with at most 8 rows and weights of 8 MB or more is a pass over the weights: the row kernel
    streams the packed bf16-pair (or int8) weights once, rows in shared memory, instead of filling 128-row tiles
    with one to eight live rows.  Ragged K steps, an odd column count, a K that needs most of shared memory."""
    x = np.random.default_rng(900 + m).uniform(-1, 1, (m, 1, 1, k)).astype(np.float32)
    for int8 in (False, True):
        param, bin_ = pkg.zoo.inner_product(str(tmp_path / ("ipq" if int8 else "ip")), k, n, int8=int8)
        got, kernels = _run(pkg, param, bin_, x)
        row_kernel = "k_ip_rows<i8>" if int8 else "k_ip_rows<bf16x2>"
        expected = k % (16 if int8 else 8) == 0 and k * n * (1 if int8 else 4) >= (8 << 20)
        assert (row_kernel in kernels) == expected, kernels
        want = _oracle_rows(oracle, param, bin_, x, range(m))
        if int8:
            assert np.array_equal(got, want)
        else:
            assert rel_l2(got, want) <= 2e-5
    # a small layer keeps the tensor-core path at every M: its results do not depend on the batch size
    param, bin_ = pkg.zoo.inner_product(str(tmp_path / "small"), 512, 1000)
    _, kernels = _run(pkg, param, bin_, x[:, :, :, :512].copy())
    assert not any(kn.startswith("k_ip_rows") for kn in kernels), kernels


@pytest.mark.parametrize("m,k,n,alpha,beta", [(256, 512, 1024, 0.5, -1.25), (32, 1024, 512, 1.75, 0.5),
                                              (200, 4096, 520, -0.25, 2.0), (1, 512, 512, 3.0, -1.0)])
def test_gemm_on_tensor_cores_alpha_beta(pkg, oracle, tmp_path, m, k, n, alpha, beta):
    """Gemm with static M at tensor-core shapes: y = (A * B^T + beta * C) * alpha, bias scaled by beta first, then
    the sum by alpha (NCNNToTosa.cpp:5079-5096).  The scaling runs in the contraction's epilogue."""
    param, bin_ = pkg.zoo.gemm(str(tmp_path / "g"), m, k, n, alpha, beta)
    x = np.random.default_rng(m + n).uniform(-1, 1, (2, m, 1, k)).astype(np.float32)
    model = pkg.Model(param, bin_)
    kernels = _kernels(model, 2)
    assert any(kn.startswith("tc_gemm") for kn in kernels), kernels
    assert "k_binary" not in kernels, kernels
    got = model.run(x)[0]
    model.close()
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert got.shape == want.shape == (2, m, n)
    assert rel_l2(got, want) <= 1e-4
    exact, _ = _run(pkg, param, bin_, x, accuracy_mode=2)
    assert rel_l2(exact, want) <= 2e-6


# ------------------------------------------------------------------ Conv -> BatchNorm
@pytest.mark.parametrize("kind,kw", [("conv", {}), ("conv", {"bias": False}), ("depthwise", {}),
                                     ("conv", {"eps": 0.0, "zero_var_channels": (0, 5, 63)}),
                                     ("depthwise", {"eps": 0.0, "zero_var_channels": (1, 2)})])
@pytest.mark.parametrize("mode", [0, 2])
def test_batchnorm_folds_into_fp32_convolution(pkg, oracle, tmp_path, kind, kw, mode):
    """FoldNCNNBatchNorm.cpp:55-178: the BatchNorm after a single-use fp32 convolution disappears into its weights
    and bias (var + eps == 0 takes the factor 10000, :99-160); one launch fewer, same values as the oracle's fold."""
    param, bin_ = pkg.zoo.conv_batchnorm(str(tmp_path / "cbn"), kind=kind, **kw)
    x = np.random.default_rng(77).uniform(-1, 1, (3, 64, 14, 14)).astype(np.float32)
    got, kernels = _run(pkg, param, bin_, x, accuracy_mode=mode)
    assert "k_unary" not in [k for k in kernels[1:-1]], kernels  # no stand-alone BatchNorm between the edges
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert np.isfinite(want).all()
    assert rel_l2(got, want) <= {0: 1e-4, 2: 2e-6}[mode]


def test_batchnorm_after_int8_convolution_is_not_folded(pkg, oracle, tmp_path):
    """A quantised convolution keeps its BatchNorm (FoldNCNNBatchNorm.cpp:63): integer weights cannot absorb the
    scale.  int8 sum, dequantise, then the explicit fp32 affine map: same bits as the oracle."""
    param, bin_ = pkg.zoo.conv_batchnorm(str(tmp_path / "cbnq"), int8=True)
    x = np.random.default_rng(78).uniform(-1, 1, (3, 64, 14, 14)).astype(np.float32)
    got, kernels = _run(pkg, param, bin_, x)
    assert "k_unary" in kernels[1:-1], kernels
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert np.array_equal(got, want)


# ------------------------------------------------------------------ batch 256 (configs 2 and 3)
@pytest.mark.parametrize("net", ["mobilenet_v2", "resnet18_int8"])
def test_batch_256_properties(pkg, oracle, tmp_path, net):
    """At the benchmark's batch 256 the oracle would need minutes, so: images are independent (a permuted batch
    gives permuted results, a repeated image repeated results, bit for bit), and the first and last two images
    match the oracle (int8: exactly)."""
    if net == "mobilenet_v2":
        param, bin_ = pkg.zoo.mobilenet_v2(str(tmp_path / "m"))
    else:
        param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r"), int8=True)
    rng = np.random.default_rng(256)
    x = rng.uniform(-1, 1, (256, 3, 224, 224)).astype(np.float32)
    x[100] = x[3]
    m = pkg.Model(param, bin_)
    y = m.run(x)[0].copy()
    assert np.array_equal(y[100], y[3])
    perm = rng.permutation(256)
    assert np.array_equal(m.run(x[perm])[0], y[perm])
    m.close()
    idx = [0, 1, 254, 255]
    om = oracle.Model(param, bin_)
    want = np.stack([om.run([x[i]])[0] for i in idx])
    if net.endswith("int8"):
        assert np.array_equal(y[idx], want)
    else:
        assert rel_l2(y[idx], want) <= 2e-4


# ------------------------------------------------------------------ a bounded wait that runs out
def test_bounded_wait_runs_out_as_status_7_and_the_handle_recovers(pkg, oracle, tmp_path, monkeypatch):
    """Every device-side wait of the contraction kernels has a limit and ends in a status word.  With
    NCNN_B200_TEST_STALL set, the one-CTA kernel leaves one pipeline stage unfilled (and shrinks the limit to 2 ms):
    the issuing warp's wait runs out, every role leaves through the abort path, tensor memory is released and the
    kernel returns.  Nothing faults or hangs.  The call reports status 7; the next call on the same handle is
    clean and correct."""
    param, bin_ = pkg.zoo.single_conv(str(tmp_path / "c"), h=8, w=8)
    x = np.random.default_rng(5).uniform(-1, 1, (2, 64, 8, 8)).astype(np.float32)
    m = pkg.Model(param, bin_)
    assert any(k.startswith("tc_gemm_kernel<") for k in _kernels(m, 2))
    good = m.run(x)[0].copy()
    monkeypatch.setenv("NCNN_B200_TEST_STALL", "1")
    with pytest.raises(pkg.NcnnB200Error) as err:
        m.run(x)
    assert err.value.status == 7 and "timed out" in str(err.value)
    monkeypatch.delenv("NCNN_B200_TEST_STALL")
    assert np.array_equal(m.run(x)[0], good)
    m.check_status()
    m.close()
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert rel_l2(good, want) <= 1e-4


# ------------------------------------------------------------------ several devices behind one handle
@pytest.mark.parametrize("n", [1, 5, 16])
def test_multi_device_handle_equals_single_handle(pkg, tmp_path, n):
    """ncnn_b200_multi_*: the batch is cut into contiguous shards, one replica (stream, graph, host thread) per
    listed device.  On a box with one GPU the same ordinal is listed twice (two replicas side by side); with more
    GPUs the first two.  Same bits as one handle: images are independent and every kernel is the same."""
    import torch
    devices = [0, 1] if torch.cuda.device_count() >= 2 else [0, 0]
    param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r"), size=64, classes=50)
    x = np.random.default_rng(n).uniform(-1, 1, (n, 3, 64, 64)).astype(np.float32)
    single = pkg.Model(param, bin_)
    want = single.run(x)[0].copy()
    single.close()
    multi = pkg.MultiModel(param, bin_, devices)
    for _ in range(2):
        got = multi.run(x)[0]
        assert np.array_equal(got, want)
    multi.close()


def test_handles_on_their_own_device_leave_the_callers_device_alone(pkg, tmp_path):
    """Every entry point makes the model's device current for the call and restores the caller's."""
    import torch
    param, bin_ = pkg.zoo.single_conv(str(tmp_path / "c"), h=8, w=8)
    last = torch.cuda.device_count() - 1
    torch.cuda.set_device(0)
    m = pkg.Model(param, bin_, device=last)
    assert torch.cuda.current_device() == 0
    x = np.random.default_rng(0).uniform(-1, 1, (2, 64, 8, 8)).astype(np.float32)
    y = m.run(x)[0]
    assert torch.cuda.current_device() == 0 and np.isfinite(y).all()
    m.close()
    assert torch.cuda.current_device() == 0


# ------------------------------------------------------------------ Quantize folded into the producer
def test_quantize_steps_fold_into_their_producers(pkg, oracle, tmp_path, monkeypatch):
    """The int8 network's Quantize steps (NCNNToTosa.cpp:4802-4824, one in front of every int8 contraction whose
    input is fp32) can be written by the layer that produces the fp32 tensor.  By default the pooling layers do
    (two launches fewer; three more where two steps read the same tensor and become one pass); with NCNN_B200_FUSE_QUANT=2 the residual convolutions emit the int8 copies for the next
    block as well (two where a strided block has a projection): twelve launches fewer.  Either way the same bits
    as the separate steps, and bit exact against the oracle."""
    param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r18q"), int8=True)
    x = np.random.default_rng(402).uniform(-1, 1, (4, 3, 224, 224)).astype(np.float32)
    results, counts = {}, {}
    for level in ("0", "1", "2"):
        monkeypatch.setenv("NCNN_B200_FUSE_QUANT", level)
        m = pkg.Model(param, bin_)
        kernels = _kernels(m, 4)
        counts[level] = (sum(k.startswith("k_quantize16") for k in kernels), len(kernels))
        results[level] = m.run(x)[0].copy()
        m.close()
    # (from level 1 on, the two steps that read the input of a strided block are one pass with two results)
    assert [counts[k][0] for k in ("0", "1", "2")] == [12, 7, 0], counts
    assert counts["0"][1] - counts["2"][1] == 12
    assert np.array_equal(results["1"], results["0"]) and np.array_equal(results["2"], results["0"])
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert np.array_equal(results["1"][:2], want)


# ------------------------------------------------------------------ patch-resident convolution on CTA pairs
@pytest.mark.parametrize("h,c,cout,n", [(56, 64, 96, 4), (28, 128, 128, 5), (14, 256, 256, 7), (40, 64, 64, 3)])
def test_patch_resident_pairs_match_the_im2col_kernel(pkg, oracle, tmp_path, monkeypatch, h, c, cout, n):
    """NCNN_B200_HALO=2: 3x3 stride-1 convolutions keep each tile's input patch in shared memory (loaded once per
    channel block, every tap reads it through a shifted descriptor) and run two pixel tiles per cluster of two
    CTAs that share each tap's weights.  Same products per output as the im2col kernel; sums may round
    differently (the channel blocks are the outer loop), so: rel-L2 <= 3e-5 against it, <= 1e-4 against the
    oracle, and the same bits from run to run.  Odd tile counts (a pair whose second tile does not exist) and
    images that the 8x16 tiles overhang are part of the cases."""
    param, bin_ = pkg.zoo.residual_block(str(tmp_path / "rb"), h=h, w=h, c=c, cout=cout)
    x = np.random.default_rng(h + n).uniform(-1, 1, (n, c, h, h)).astype(np.float32)
    monkeypatch.setenv("NCNN_B200_HALO", "2")
    got, kernels = _run(pkg, param, bin_, x)
    assert any(k.startswith("tc_conv_halo_kernel:pairs<") for k in kernels), kernels
    again, _ = _run(pkg, param, bin_, x)
    assert np.array_equal(got, again)
    monkeypatch.setenv("NCNN_B200_HALO", "0")
    base, kernels = _run(pkg, param, bin_, x)
    assert not any(k.startswith("tc_conv_halo_kernel") for k in kernels), kernels
    assert rel_l2(got, base) <= 3e-5
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert rel_l2(got[:2], want) <= 1e-4


# ------------------------------------------------------------------ depthwise fused into the projection
@pytest.mark.parametrize("n", [2, 5])
def test_depthwise_runs_inside_the_projection_kernel(pkg, oracle, tmp_path, monkeypatch, n):
    """The stride-1 3x3 depthwise layers of the inverted-residual blocks run inside the 1x1 convolution that
    follows them (their result goes from the CUDA cores into the MMA's shared-memory operand, never to HBM).
    Same values, same bf16 split, same order of products as the two separate layers: the same bits; and the
    network still matches the oracle.  (NCNN_B200_FUSE_EXPAND=0: the expand layers stay on the tensor cores.)"""
    param, bin_ = pkg.zoo.mobilenet_v2(str(tmp_path / "mbv2"))
    x = np.random.default_rng(300 + n).uniform(-1, 1, (n, 3, 224, 224)).astype(np.float32)
    monkeypatch.setenv("NCNN_B200_FUSE_EXPAND", "0")
    got, kernels = _run(pkg, param, bin_, x)
    fused = kernels.count("tc_dw_project_kernel<bf16x3>")
    assert fused >= 10, kernels
    monkeypatch.setenv("NCNN_B200_FUSE_DW", "0")
    base, plain = _run(pkg, param, bin_, x)
    assert not any(k.startswith("tc_dw_project_kernel") for k in plain) and len(plain) - len(kernels) == fused
    assert np.array_equal(got, base)
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert rel_l2(got[:2], want) <= 2e-4


@pytest.mark.parametrize("n", [3, 8])
def test_whole_inverted_residual_blocks_run_in_one_kernel(pkg, oracle, tmp_path, monkeypatch, n):
    """Blocks whose input has at most 32 channels run whole in the fused kernel: the expand layer on the CUDA cores
    in fp32 from the block's input patch, depthwise (stride 1 or 2) and projection as above.  The expanded tensor
    and the depthwise result never reach HBM.  fp32 instead of three bf16 products for the expand layer: not the
    bits of the separate layers, but as close to them as they are to the oracle."""
    param, bin_ = pkg.zoo.mobilenet_v2(str(tmp_path / "mbv2"))
    x = np.random.default_rng(400 + n).uniform(-1, 1, (n, 3, 224, 224)).astype(np.float32)
    monkeypatch.setenv("NCNN_B200_FUSE_EXPAND", "2")  # stride-1 blocks too (by default only stride-2 blocks: they gain)
    got, kernels = _run(pkg, param, bin_, x)
    whole = [k for k in kernels if k.startswith("tc_dw_project_kernel:expand")]
    assert len(whole) >= 5 and "tc_dw_project_kernel:expand+stride2<bf16x3>" in whole, kernels
    monkeypatch.setenv("NCNN_B200_FUSE_EXPAND", "1")
    _, default_kernels = _run(pkg, param, bin_, x)
    assert [k for k in default_kernels if k.startswith("tc_dw_project_kernel:expand")] == ["tc_dw_project_kernel:expand+stride2<bf16x3>"] * 3
    monkeypatch.setenv("NCNN_B200_FUSE_DW", "0")
    base, plain = _run(pkg, param, bin_, x)
    assert len(plain) > len(kernels) + 2 * len(whole) - 1
    assert rel_l2(got, base) <= 2e-5
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert rel_l2(got[:2], want) <= 2e-4


@pytest.mark.parametrize("h,w,cin,hidden,cout,stride,n", [
    (56, 56, 24, 144, 24, 1, 3),    # residual block, hidden channels end inside a 32-channel block
    (112, 112, 16, 96, 24, 2, 2),   # the widest tensors of MobileNetV2
    (56, 56, 24, 144, 32, 2, 3),
    (28, 28, 32, 192, 32, 1, 4),    # 32 input channels, residual
    (19, 13, 8, 40, 16, 1, 5),      # ragged tiles both ways, few channels
    (21, 17, 16, 64, 40, 2, 3),     # odd extent at stride 2: the last output pixel reads the zero padding
    (9, 9, 8, 72, 24, 1, 2),
    (40, 24, 16, 32, 16, 1, 3),     # a single channel block per tile: the two groups alternate tiles
    (33, 33, 8, 32, 128, 2, 2),     # the same at stride 2, and the widest projection the kernel takes
    (3, 3, 16, 48, 16, 1, 7),       # an image smaller than a tile
    (4, 4, 24, 64, 24, 2, 5),
])
def test_whole_block_shapes(pkg, oracle, tmp_path, monkeypatch, h, w, cin, hidden, cout, stride, n):
    param, bin_ = pkg.zoo.inverted_residual(str(tmp_path / "blk"), h, w, cin, hidden, cout, stride, seed=h * 31 + cin)
    x = np.random.default_rng(h * cin + stride).uniform(-2, 2, (n, cin, h, w)).astype(np.float32)
    monkeypatch.setenv("NCNN_B200_FUSE_DW", "2")  # also where the image fills its tiles badly
    monkeypatch.setenv("NCNN_B200_FUSE_EXPAND", "2")  # and stride-1 blocks
    got, kernels = _run(pkg, param, bin_, x)
    assert len(kernels) == 3 and kernels[1].startswith("tc_dw_project_kernel:expand"), kernels
    assert ("stride2" in kernels[1]) == (stride == 2)
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert rel_l2(got, want) <= 1e-4
    monkeypatch.setenv("NCNN_B200_FUSE_DW", "0")
    base, plain = _run(pkg, param, bin_, x)
    assert not any(k.startswith("tc_dw_project_kernel") for k in plain)
    assert rel_l2(got, base) <= 2e-5


@pytest.mark.parametrize("h,c,cout,n", [(14, 96, 24, 3), (30, 40, 64, 2), (7, 960, 320, 4), (9, 144, 16, 5)])
def test_depthwise_projection_block_shapes(pkg, oracle, tmp_path, monkeypatch, h, c, cout, n):
    """Single inverted-residual tails at awkward shapes: channel counts that end inside a 32-channel block, images
    that the 16 x 8 tiles overhang, a projection wider than one tile (320 = 2 x 160)."""
    net = pkg.zoo._Net(1000 + h)
    wr = net.w
    wr.layer("Input", "input", [], ["data"], f"0={h} 1={h} 2={c}")
    net.depthwise("dw", "data", "d", c, 3, 1, 1)
    wr.layer("Clip", "relu6", ["d"], ["d6"], "0=0.0 1=6.0")
    net.conv("project", "d6", "output", c, cout, 1, 1, 0, act=0, zero_bias=False)
    param, bin_ = wr.save(str(tmp_path / "blk"))
    x = np.random.default_rng(h * c).uniform(-3, 3, (n, c, h, h)).astype(np.float32)
    monkeypatch.setenv("NCNN_B200_FUSE_DW", "2")  # also where the image fills its tiles badly
    got, kernels = _run(pkg, param, bin_, x)
    assert "tc_dw_project_kernel<bf16x3>" in kernels, kernels
    monkeypatch.setenv("NCNN_B200_FUSE_DW", "0")
    base, _ = _run(pkg, param, bin_, x)
    assert np.array_equal(got, base)
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    assert rel_l2(got, want) <= 1e-4


# ------------------------------------------------------------------ device allocations that fail
def test_every_failed_device_allocation_is_reported_and_leaves_nothing_behind(pkg, oracle, tmp_path, monkeypatch):
    """NCNN_B200_TEST_FAIL_ALLOC=k makes the k-th device allocation of an engine return the driver's
    out-of-memory error (no GPU is filled up for this).  Whichever allocation it is - weights, the status word,
    the split workspace, the activation arena, the staging arrays of the host-pointer entry - the call that
    needed it fails with status 6 and an out-of-memory message, no kernel ever sees a null pointer, the same
    engine works once memory "is back", and the device has as much free memory afterwards as before."""
    import torch
    param, bin_ = pkg.zoo.conv_batchnorm(str(tmp_path / "blk"))
    x = np.random.default_rng(5).uniform(-1, 1, (3, 64, 14, 14)).astype(np.float32)
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    failures_at_load = failures_at_run = 0
    for k in range(1, 60):
        monkeypatch.setenv("NCNN_B200_TEST_FAIL_ALLOC", str(k))
        try:
            m = pkg.Model(param, bin_)
        except pkg.NcnnB200Error as e:
            assert e.status == 6 and "memory" in e.message, (k, e.message)
            failures_at_load += 1
            continue
        try:
            got = m.run(x)[0]
        except pkg.NcnnB200Error as e:
            assert e.status == 6 and "memory" in e.message, (k, e.message)
            failures_at_run += 1
            monkeypatch.delenv("NCNN_B200_TEST_FAIL_ALLOC")
            got = m.run(x)[0]  # the same engine, now that allocations succeed
            assert rel_l2(got, want) <= 1e-4
            m.close()
            continue
        assert rel_l2(got, want) <= 1e-4  # k is past the last allocation: nothing failed
        m.close()
        break
    else:
        raise AssertionError("allocations never ran out")
    assert failures_at_load >= 3 and failures_at_run >= 2, (failures_at_load, failures_at_run)
    monkeypatch.delenv("NCNN_B200_TEST_FAIL_ALLOC", raising=False)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before - (8 << 20)


# ------------------------------------------------------------------ the same bits, pass after pass
def test_mobilenet_v2_repeats_bit_for_bit(pkg, tmp_path):
    """150 passes at batch 256 through the host-pointer entry (uploads pipelined over the first layers, so the
    kernels run against DRAM latency that varies from pass to pass) and 150 at batch 64: every pass gives the bits of
    the first.  A patch ring of three slots once let a depthwise group, which then meets every second phase of a
    slot, take a phase for the one two before it when a load was late: one image in ~500 passes came out wrong."""
    param, bin_ = pkg.zoo.mobilenet_v2(str(tmp_path / "mbv2"))
    m = pkg.Model(param, bin_)
    for n in (256, 64):
        x = np.random.default_rng(n).uniform(-1, 1, (n, 3, 224, 224)).astype(np.float32)
        first = m.run(x)[0].copy()
        for i in range(150):
            assert np.array_equal(m.run(x)[0], first), (n, i)
    m.close()


def test_resnet18_repeats_bit_for_bit(pkg, tmp_path):
    """The stem + pooling kernel (two MMA-issuing warps on alternate rows, four row stages, four accumulators) and the
    int8 contractions with several K blocks per ring stage: 100 passes of each network through the host-pointer entry
    give the bits of the first pass."""
    for int8 in (False, True):
        param, bin_ = pkg.zoo.resnet18(str(tmp_path / ("r8" if int8 else "r")), int8=int8)
        m = pkg.Model(param, bin_)
        x = np.random.default_rng(5).uniform(-1, 1, (64, 3, 224, 224)).astype(np.float32)
        first = m.run(x)[0].copy()
        for i in range(100):
            assert np.array_equal(m.run(x)[0], first), (int8, i)
        m.close()


@pytest.mark.parametrize("size,n", [(224, 4), (64, 9)])
def test_int8_k_blocks_per_stage_change_no_bit(pkg, oracle, tmp_path, monkeypatch, size, n):
    """Int8 contractions that are not paired keep 2 to 4 K blocks in one ring stage (one barrier hand-shake for
    several small copies); the MMAs and their order are the same, so is every bit, and both equal the oracle."""
    param, bin_ = pkg.zoo.resnet18(str(tmp_path / "r8"), int8=True, size=size, classes=40)
    x = np.random.default_rng(size).uniform(-1, 1, (n, 3, size, size)).astype(np.float32)
    m = pkg.Model(param, bin_)
    got = m.run(x)[0]
    m.close()
    monkeypatch.setenv("NCNN_B200_SUB_BLOCKS", "0")
    m = pkg.Model(param, bin_)
    assert np.array_equal(m.run(x)[0], got)
    m.close()
    want = np.stack([oracle.Model(param, bin_).run([xi])[0] for xi in x[:2]])
    assert np.array_equal(got[:2], want)
