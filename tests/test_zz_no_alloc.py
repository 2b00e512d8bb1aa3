"""The allocation-free int8 InnerProduct entry point against the regular model path.

Hosts that may not allocate on the GPU (a real-time loop after start-up, a sandbox without
cudaMalloc, a process whose own pool owns the device) cannot use ncnn_b200_load/run, which
allocate an arena.  ncnn_b200_inner_product_int8_noalloc keeps its scratch in an array inside
the library instead.  This file is collected last on purpose: a failure here stops nothing
else.  The check: same weights through a loaded int8 InnerProduct model (existing entry
point) and through the new entry point, two calls in a row on different inputs (the second
call finds the first call's bytes in the shared scratch), bit-exact equality -- the bar the
other int8 tests use.
"""
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

INT8_TAG = 0x000D4B38


def write_int8_inner_product(prefix, wq, bias, weight_scales, input_scale, relu):
    n, k = wq.shape
    with open(prefix + ".param", "w") as f:
        f.write("7767517\n2 2\n")
        f.write(f"Input input 0 1 data 0={k} 1=1 2=1\n")
        f.write(f"InnerProduct ip 1 1 data output 0={n} 1=1 2={n * k} 8=1" + (" 9=1" if relu else "") + "\n")
    payload = wq.astype(np.int8).tobytes()
    with open(prefix + ".bin", "wb") as f:
        f.write(struct.pack("<I", INT8_TAG) + payload + bytes((-len(payload)) % 4))
        f.write(bias.astype(np.float32).tobytes())
        f.write(weight_scales.astype(np.float32).tobytes())
        f.write(np.array([input_scale], np.float32).tobytes())
    return prefix + ".param", prefix + ".bin"


@pytest.mark.parametrize("m,k,n,relu", [(37, 512, 1000, True), (5, 100, 7, False)])
def test_no_alloc_entry_matches_model_path_twice(pkg, tmp_path, m, k, n, relu):
    import torch
    rng = np.random.default_rng(77)
    wq = rng.integers(-127, 128, (n, k)).astype(np.int8)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    ws = rng.uniform(20, 200, n).astype(np.float32)
    ws[0] = 0.0  # a zero weight scale dequantises to 0, as the reference defines
    s_in = np.float32(17.25)
    param, bin_ = write_int8_inner_product(str(tmp_path / "ip"), wq, bias, ws, s_in, relu)
    model = pkg.Model(param, bin_)

    d_w = torch.from_numpy(wq).cuda()
    d_ws = torch.from_numpy(ws).cuda()
    d_b = torch.from_numpy(bias).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # the second call reuses the scratch the first one dirtied
        x = rng.uniform(-1.5, 1.5, (m, 1, 1, k)).astype(np.float32)
        want = model.run(x)[0]
        d_x = torch.from_numpy(x.reshape(m, k)).cuda()
        d_y = torch.full((m, n), float("nan"), device="cuda")
        status, message = pkg.inner_product_int8_noalloc(d_x.data_ptr(), d_w.data_ptr(), d_ws.data_ptr(), float(s_in),
                                                         d_b.data_ptr(), d_y.data_ptr(), m, k, n, relu, stream)
        assert status == 0, message
        torch.cuda.synchronize()
        got = d_y.cpu().numpy()
        assert np.array_equal(got, want), f"call {call}: max abs diff {np.abs(got - want).max()}"


def test_no_alloc_entry_takes_weights_at_any_byte_offset_and_matches_the_oracle(pkg, oracle, tmp_path):
    """A weight blob carved out of a larger buffer may start at an odd address: the entry point then reads it byte
    by byte instead of word by word.  Checked against the CPU oracle (the reference's int8 InnerProduct
    arithmetic), bit for bit, and against the aligned call."""
    import torch
    rng = np.random.default_rng(78)
    m, k, n = 9, 256, 33
    wq = rng.integers(-127, 128, (n, k)).astype(np.int8)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32)
    ws = rng.uniform(20, 200, n).astype(np.float32)
    s_in = np.float32(23.5)
    param, bin_ = write_int8_inner_product(str(tmp_path / "ip"), wq, bias, ws, s_in, True)
    x = rng.uniform(-1.5, 1.5, (m, 1, 1, k)).astype(np.float32)
    om = oracle.Model(param, bin_)
    want = np.stack([om.run([xi])[0] for xi in x])
    blob = torch.zeros(n * k + 16, dtype=torch.int8, device="cuda")
    d_ws, d_b = torch.from_numpy(ws).cuda(), torch.from_numpy(bias).cuda()
    d_x = torch.from_numpy(x.reshape(m, k)).cuda()
    for offset in (0, 1, 2, 3):
        blob[offset:offset + n * k] = torch.from_numpy(wq.reshape(-1)).cuda()
        d_y = torch.full((m, n), float("nan"), device="cuda")
        status, message = pkg.inner_product_int8_noalloc(d_x.data_ptr(), blob.data_ptr() + offset, d_ws.data_ptr(),
                                                         float(s_in), d_b.data_ptr(), d_y.data_ptr(), m, k, n, True, 0)
        assert status == 0, message
        torch.cuda.synchronize()
        assert np.array_equal(d_y.cpu().numpy(), want), f"weight offset {offset}"


def test_no_alloc_entry_refuses_oversized_requests(pkg):
    import torch
    t = torch.zeros(16, device="cuda")
    w = torch.zeros(16, dtype=torch.int8, device="cuda")
    status, message = pkg.inner_product_int8_noalloc(t.data_ptr(), w.data_ptr(), t.data_ptr(), 1.0, None, t.data_ptr(),
                                                     4097, 2048, 1, False, 0)  # 4097*2048 > 8 MiB
    assert status == 5 and "exceed the built-in scratch" in message
    status, _ = pkg.inner_product_int8_noalloc(None, w.data_ptr(), t.data_ptr(), 1.0, None, t.data_ptr(), 1, 16, 1)
    assert status == 1
    # a row count whose product with k wraps around 64 bits is refused like any other (nothing is launched)
    status, message = pkg.inner_product_int8_noalloc(t.data_ptr(), w.data_ptr(), t.data_ptr(), 1.0, None, t.data_ptr(),
                                                     2**61 + 1, 8, 1, False, 0)
    assert status == 5 and "exceed the built-in scratch" in message
