"""GPU parity of the prefill GEMM (tcgen05) through the C ABI against the CPU oracle.

The oracle rounds at the same two points as the kernel: activations are bf16, and the
dequantized fp32 weights are rounded to bf16 (nearest even) before the product; the
accumulation is fp32 (the tensor core) vs fp64 here, hence the 1e-3 bar.
"""
import numpy as np
import pytest

import oracle
from litenn_b200 import capi, synth
from helpers import FORMATS, REL_TOL, max_rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda(qmm_lib):
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch


def reference(fmt, payload, n, k, x_bf16_as_f32):
    w = oracle.fp32_to_bf16_round(oracle.dequant(fmt, payload, n, k))
    return oracle.matmul_nk_f64(x_bf16_as_f32, w)


def run_gemm(torch, w, x_f32, out_bf16=False):
    info = w.info()
    m = x_f32.shape[0]
    xb = torch.from_numpy(x_f32).cuda().to(torch.bfloat16).contiguous()
    y = torch.full((m, info.n), float("nan"), device="cuda", dtype=torch.bfloat16 if out_bf16 else torch.float32)
    w.gemm_bf16(xb.data_ptr(), y.data_ptr(), m, capi.OUT_BF16 if out_bf16 else capi.OUT_F32)
    torch.cuda.synchronize()
    assert capi.kernel_status(0) == 0
    return y.float().cpu().numpy(), xb.float().cpu().numpy()


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(128, 16, 256), (128, 256, 512), (1, 48, 256), (100, 200, 1024), (300, 528, 768),
                                   (512, 1000, 512),
                                   # more than 256 rows: CTA pairs share each dequantized tile; a second CTA with one
                                   # row, an odd number of 256-row groups (partner without rows), five groups
                                   (257, 272, 512), (600, 96, 512), (1100, 320, 768)])
def test_gemm_matches_oracle(torch_cuda, fmt, shape):
    m, n, k = shape
    payload = synth.make_weight(fmt, n, k, seed=8, name=f"gemm-{fmt}-{n}-{k}")
    x = synth.make_activation(m, k, seed=8, name=f"gemm-x-{m}")
    w = capi.Weight.from_host(fmt, payload, n, k)
    got, xb = run_gemm(torch_cuda, w, x)
    ref = reference(fmt, payload, n, k, xb)
    assert np.isfinite(got).all()
    err = max_rel_err(got, ref)
    assert err <= REL_TOL, f"max relative error {err:.3e}"


@pytest.mark.parametrize("m", [256, 512, 700])
def test_gemm_exact_on_small_integers(torch_cuda, m):
    """Integer-valued activations and Q8_0 weights with a power-of-two scale make every
    product and partial sum exact, so any layout or descriptor mistake shows as a mismatch
    (one CTA per row group at 256 rows, CTA pairs above)."""
    n, k = 64, 256
    rng = np.random.default_rng(0)
    blocks = np.zeros((n * k // 32, 34), dtype=np.uint8)
    blocks[:, 0:2] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    blocks[:, 2:] = rng.integers(-4, 5, size=(n * k // 32, 32), dtype=np.int8).view(np.uint8)
    payload = blocks.reshape(-1)
    x = rng.integers(-3, 4, size=(m, k)).astype(np.float32)
    w = capi.Weight.from_host(capi.Q8_0, payload, n, k)
    got, _ = run_gemm(torch_cuda, w, x)
    ref = x.astype(np.float64) @ oracle.dequant(capi.Q8_0, payload, n, k).astype(np.float64).T
    assert np.array_equal(got.astype(np.float64), ref)


@pytest.mark.parametrize("fmt", [capi.Q4_K, capi.Q6_K])
def test_gemm_bf16_output_and_ragged_k(torch_cuda, fmt):
    m, n, k = 130, 96, 1280
    payload = synth.make_weight(fmt, n, k, seed=9, name=f"gemm-bf16-{fmt}")
    x = synth.make_activation(m, k, seed=9, name="gemm-bf16-x")
    w = capi.Weight.from_host(fmt, payload, n, k)
    got, xb = run_gemm(torch_cuda, w, x, out_bf16=True)
    ref = reference(fmt, payload, n, k, xb)
    assert max_rel_err(got, ref) <= 5e-3  # bf16 output rounding (2^-9 relative) on top of the 1e-3 bar


def test_gemm_q4_0_ragged_k(torch_cuda):
    m, n, k = 64, 40, 1376  # 43 blocks of 32: not a multiple of the 256-wide tile
    payload = synth.make_weight(capi.Q4_0, n, k, seed=10, name="gemm-ragged")
    x = synth.make_activation(m, k, seed=10, name="gemm-ragged-x")
    w = capi.Weight.from_host(capi.Q4_0, payload, n, k)
    got, xb = run_gemm(torch_cuda, w, x)
    assert max_rel_err(got, reference(capi.Q4_0, payload, n, k, xb)) <= REL_TOL


@pytest.mark.parametrize("fmt", [capi.Q4_K, capi.Q6_K])
def test_config3_prefill_shape_full_size(torch_cuda, fmt):
    """Config 3: M=512, K=4096, N=14336.  A 1024-row sample of the outputs is checked against
    the oracle; the whole product is checked for linearity in the activations."""
    torch = torch_cuda
    m, k, n = 512, 4096, 14336
    payload = synth.make_weight(fmt, n, k, seed=0, name=f"cfg3.w.{fmt}")
    w = capi.Weight.from_host(fmt, payload, n, k)
    x = synth.make_activation(m, k, seed=0, name="cfg3.x")
    got, xb = run_gemm(torch, w, x)
    rows = np.random.default_rng(3).choice(n, size=1024, replace=False)
    rb = k // synth.BLOCK_ELEMS[fmt] * synth.BLOCK_BYTES[fmt]
    sub = np.concatenate([payload[r * rb:(r + 1) * rb] for r in rows])
    ref = reference(fmt, sub, len(rows), k, xb)
    assert max_rel_err(got[:, rows], ref) <= REL_TOL
    # linearity: W(2a - b) = 2 W a - W b for bf16-exact combinations
    a = np.round(synth.make_activation(m, k, seed=1, name="cfg3.a") * 8) / 8
    b = np.round(synth.make_activation(m, k, seed=1, name="cfg3.b") * 8) / 8
    ya, _ = run_gemm(torch, w, a.astype(np.float32))
    yb, _ = run_gemm(torch, w, b.astype(np.float32))
    yab, _ = run_gemm(torch, w, (2 * a - b).astype(np.float32))
    assert max_rel_err(yab, 2 * ya - yb) <= REL_TOL
