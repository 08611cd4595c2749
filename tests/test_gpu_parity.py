"""GPU parity: the CUDA path through the C ABI against the CPU oracle."""
import numpy as np
import pytest

import oracle
from litenn_b200 import capi, synth
from helpers import FORMATS, REL_TOL, assert_bit_exact, max_rel_err, random_payload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda(qmm_lib):
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    assert capi.device_count() >= 1
    torch.cuda.set_device(0)
    return torch


def gpu_dequant(torch, w):
    info = w.info()
    out = torch.empty((info.n, info.k), dtype=torch.float32, device="cuda")
    w.dequantize(out.data_ptr())
    torch.cuda.synchronize()
    return out.cpu().numpy()


def gpu_gemv(torch, w, x):
    info = w.info()
    m = x.shape[0]
    xd = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    y = torch.full((m, info.n), float("nan"), dtype=torch.float32, device="cuda")
    w.gemv_f32(xd.data_ptr(), y.data_ptr(), m)
    torch.cuda.synchronize()
    assert capi.kernel_status(0) == 0
    return y.cpu().numpy()


@pytest.mark.parametrize("fmt", FORMATS)
def test_dequant_golden_bit_exact(torch_cuda, golden, fmt):
    name = synth.FORMAT_NAMES[fmt]
    n, k = int(golden["rows"]), int(golden["k"])
    for variant in ("", "_syn"):
        payload = np.ascontiguousarray(golden[f"{name}{variant}_payload"])
        w = capi.Weight.from_host(fmt, payload, n, k)
        assert_bit_exact(gpu_dequant(torch_cuda, w), golden[f"{name}{variant}_values"], f"{name}{variant}")
        w.destroy()


def test_reference_q4_0_fixture_on_gpu(torch_cuda):
    payload = np.array([0x10, 0x00, 0x22, 0x44, 0x66, 0x88, 0xaa, 0xcc, 0xee, 0x11, 0x33, 0x55, 0x77, 0x99,
                        0xbb, 0xdd, 0xff, 0x7f], dtype=np.uint8)
    w = capi.Weight.from_host(capi.Q4_0, payload, 1, 32)
    assert_bit_exact(gpu_dequant(torch_cuda, w), oracle.dequant(capi.Q4_0, payload, 1, 32), "fixture")
    info = w.info()
    assert (info.fmt, info.n, info.k, info.payload_bytes) == (capi.Q4_0, 1, 32, 18)


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(16, 256), (40, 768), (7, 1024), (33, 2048), (1, 256), (300, 4096)])
def test_dequant_packed_and_raw_match_oracle(torch_cuda, fmt, shape):
    torch = torch_cuda
    n, k = shape
    payload = random_payload(fmt, n, k, seed=n * 7 + k + fmt)
    ref = oracle.dequant(fmt, payload, n, k)
    w = capi.Weight.from_host(fmt, payload, n, k)
    assert_bit_exact(gpu_dequant(torch, w), ref, "dequant(repacked)")
    raw = torch.from_numpy(payload).cuda()
    out = torch.empty((n, k), dtype=torch.float32, device="cuda")
    capi.dequantize_raw(fmt, raw.data_ptr(), n, k, out.data_ptr())
    torch.cuda.synchronize()
    assert_bit_exact(out.cpu().numpy(), ref, "dequant(raw)")
    # a payload that already lives on the device repacks to the same thing
    w2 = capi.Weight.from_device(fmt, raw.data_ptr(), payload.nbytes, n, k)
    assert_bit_exact(gpu_dequant(torch, w2), ref, "dequant(repacked from device payload)")


@pytest.mark.parametrize("fmt", [capi.Q4_0, capi.Q8_0])
def test_dequant_ragged_k(torch_cuda, fmt):
    for n, k in [(5, 96), (18, 1376), (16, 32)]:
        payload = random_payload(fmt, n, k, seed=k + fmt)
        w = capi.Weight.from_host(fmt, payload, n, k)
        assert_bit_exact(gpu_dequant(torch_cuda, w), oracle.dequant(fmt, payload, n, k), f"ragged {n}x{k}")


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8, 9, 15, 16])
def test_gemv_matches_oracle(torch_cuda, fmt, m):
    n, k = 200, 2048
    payload = synth.make_weight(fmt, n, k, seed=3, name=f"gemv-{fmt}")
    x = synth.make_activation(m, k, seed=3, name=f"x-{m}")
    ref = oracle.quantized_matmul(fmt, payload, n, k, x)
    w = capi.Weight.from_host(fmt, payload, n, k)
    got = gpu_gemv(torch_cuda, w, x)
    assert got.shape == ref.shape and np.isfinite(got).all()
    err = max_rel_err(got, ref)
    assert err <= REL_TOL, f"max relative error {err:.3e}"


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(1, 256), (17, 256), (16, 9984), (130, 512), (4096, 256)])
def test_gemv_shapes(torch_cuda, fmt, shape):
    """Single rows, row counts that are not a multiple of the 16-row tile, many and few K chunks."""
    n, k = shape
    payload = random_payload(fmt, n, k, seed=n + k + fmt)
    ref_w = oracle.dequant(fmt, payload, n, k)
    for m in (1, 5, 16):
        x = synth.make_activation(m, k, seed=n, name=f"shape-{m}")
        ref = oracle.matmul_nk(x, ref_w)
        w = capi.Weight.from_host(fmt, payload, n, k)
        got = gpu_gemv(torch_cuda, w, x)
        err = max_rel_err(got, ref)
        assert err <= REL_TOL, f"{n}x{k} m={m}: max relative error {err:.3e}"


@pytest.mark.parametrize("fmt", [capi.Q4_0, capi.Q8_0])
def test_gemv_ragged_k(torch_cuda, fmt):
    n, k = 64, 1376  # 43 blocks: 11008 / 8
    payload = random_payload(fmt, n, k, seed=17 + fmt)
    x = synth.make_activation(4, k, seed=17, name="ragged")
    ref = oracle.quantized_matmul(fmt, payload, n, k, x)
    w = capi.Weight.from_host(fmt, payload, n, k)
    assert max_rel_err(gpu_gemv(torch_cuda, w, x), ref) <= REL_TOL


def test_gemv_special_activations(torch_cuda):
    """All-zero activations, a single spike, and widely different magnitudes per chunk."""
    n, k = 64, 1024
    payload = synth.make_weight(capi.Q4_0, n, k, seed=11, name="special")
    w = capi.Weight.from_host(capi.Q4_0, payload, n, k)
    wf = oracle.dequant(capi.Q4_0, payload, n, k)
    x = np.zeros((3, k), dtype=np.float32)
    x[1, 517] = 3.25
    x[2] = synth.make_activation(1, k, seed=11, name="special-x")[0]
    x[2, :256] *= 1e-4
    x[2, 256:512] *= 1e4
    got = gpu_gemv(torch_cuda, w, x)
    ref = oracle.matmul_nk(x, wf)
    assert not got[0].any()
    assert np.allclose(got[1], ref[1], rtol=1e-4, atol=0)
    assert max_rel_err(got[2], ref[2]) <= REL_TOL


@pytest.mark.parametrize("fmt", FORMATS)
def test_shards_reassemble(torch_cuda, fmt):
    """N shards concatenate and K shards sum to the unsharded product (what the
    tensor-parallel linear relies on)."""
    n, k, tp = 128, 2048, 4
    payload = synth.make_weight(fmt, n, k, seed=5, name=f"shard-{fmt}")
    x = synth.make_activation(2, k, seed=5, name="shard-x")
    ref = oracle.quantized_matmul(fmt, payload, n, k, x)
    full_w = oracle.dequant(fmt, payload, n, k)
    parts = []
    ksum = np.zeros_like(ref)
    for rank in range(tp):
        wn = capi.Weight.from_host(fmt, payload, n, k, split=capi.SPLIT_N, tp_rank=rank, tp_size=tp)
        assert_bit_exact(gpu_dequant(torch_cuda, wn), full_w[rank * n // tp:(rank + 1) * n // tp], "N shard")
        parts.append(gpu_gemv(torch_cuda, wn, x))
        wk = capi.Weight.from_host(fmt, payload, n, k, split=capi.SPLIT_K, tp_rank=rank, tp_size=tp)
        cols = slice(rank * k // tp, (rank + 1) * k // tp)
        assert_bit_exact(gpu_dequant(torch_cuda, wk), full_w[:, cols], "K shard")
        ksum += gpu_gemv(torch_cuda, wk, np.ascontiguousarray(x[:, cols]))
    assert max_rel_err(np.concatenate(parts, axis=1), ref) <= REL_TOL
    assert max_rel_err(ksum, ref) <= REL_TOL


def test_host_buffer_entry_point(torch_cuda):
    n, k, m = 96, 1024, 4
    payload = synth.make_weight(capi.Q8_0, n, k, seed=2, name="host")
    x = synth.make_activation(m, k, seed=2, name="host-x")
    w = capi.Weight.from_host(capi.Q8_0, payload, n, k)
    y = np.empty((m, n), dtype=np.float32)
    w.gemv_f32_host(x, y, m)
    assert max_rel_err(y, oracle.quantized_matmul(capi.Q8_0, payload, n, k, x)) <= REL_TOL


def test_batch_limits(torch_cuda):
    payload = synth.make_weight(capi.Q4_0, 16, 256)
    w = capi.Weight.from_host(capi.Q4_0, payload, 16, 256)
    x = torch_cuda.zeros((17, 256), device="cuda")
    y = torch_cuda.zeros((17, 16), device="cuda")
    for m in (0, 17):
        with pytest.raises(capi.QmmError) as e:
            w.gemv_f32(x.data_ptr(), y.data_ptr(), m)
        assert e.value.code == capi.E_INVALID


# ---- BASELINE configurations at full size -------------------------------------------------

def test_config1_q8_0_matvec_full_size(torch_cuda):
    """Config 1: Q8_0 4096x4096, fp32 activation vector, seed 0 — compared element by element."""
    n = k = 4096
    payload = synth.make_weight(capi.Q8_0, n, k, seed=0, name="cfg1.w")
    x = synth.make_activation(1, k, seed=0, name="cfg1.x")
    ref = oracle.quantized_matmul(capi.Q8_0, payload, n, k, x)
    w = capi.Weight.from_host(capi.Q8_0, payload, n, k)
    assert max_rel_err(gpu_gemv(torch_cuda, w, x), ref) <= REL_TOL


@pytest.mark.parametrize("shape", [(11008, 4096), (4096, 11008)])
def test_config2_q4_0_ffn_shapes_full_size(torch_cuda, shape):
    """Config 2 at batch 1, 4, 8, 16; plus linearity in the activations (a property
    that does not need the oracle)."""
    torch = torch_cuda
    n, k = shape
    payload = synth.make_weight(capi.Q4_0, n, k, seed=0, name=f"cfg2.w.{n}x{k}")
    w = capi.Weight.from_host(capi.Q4_0, payload, n, k)
    wf = oracle.dequant(capi.Q4_0, payload, n, k)
    assert_bit_exact(gpu_dequant(torch, w), wf, "cfg2 dequant")
    for m in (1, 4, 8, 16):
        x = synth.make_activation(m, k, seed=0, name=f"cfg2.x.{m}")
        got = gpu_gemv(torch, w, x)
        err = max_rel_err(got, oracle.matmul_nk(x, wf))
        assert err <= REL_TOL, f"m={m}: {err:.3e}"
    a = synth.make_activation(1, k, seed=1, name="lin.a")
    b = synth.make_activation(1, k, seed=1, name="lin.b")
    ya, yb, yab = (gpu_gemv(torch, w, v) for v in (a, b, 2 * a - 3 * b))
    assert max_rel_err(yab, 2 * ya - 3 * yb) <= REL_TOL
