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


@pytest.mark.parametrize("name,fmt", [("q4_1", 2), ("q5_0", 3), ("q5_1", 4), ("q2_k", 7), ("q3_k", 8), ("q5_k", 10)])
def test_carried_formats_dequantize_bit_exactly_on_the_device(torch_cuda, name, fmt):
    """Formats without matmul kernels: raw dequantization on the GPU equals the committed ggml-py goldens and
    the oracle, bit for bit; creating a packed weight from them is refused."""
    import os
    torch = torch_cuda
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "dequant_carried_golden.npz"))
    n, k = int(g["rows"]), int(g["k"])
    payload = np.ascontiguousarray(g[name + "_payload"])
    raw = torch.from_numpy(payload).cuda()
    out = torch.empty((n, k), dtype=torch.float32, device="cuda")
    capi.dequantize_raw(fmt, raw.data_ptr(), n, k, out.data_ptr())
    torch.cuda.synchronize()
    assert_bit_exact(out.cpu().numpy(), g[name + "_values"], name + " vs golden")
    assert_bit_exact(out.cpu().numpy(), oracle.dequant(fmt, payload, n, k), name + " vs oracle")
    with pytest.raises(capi.QmmError) as e:
        capi.Weight.from_host(fmt, payload, n, k)
    assert e.value.code == capi.E_UNSUPPORTED


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


# ---- activation quantization: per-element bar, outliers ---------------------------------------

def per_element_violations(got, ref, rel=1e-3, abs_of_max=1e-4):
    """The reference's combined form |a - e| <= rel*|e| + abs (tests/GGUFImporterTest.cpp:69-97), judged
    per element, with the absolute term tied to the largest expected magnitude."""
    ref64 = ref.astype(np.float64)
    allowed = rel * np.abs(ref64) + abs_of_max * np.abs(ref64).max()
    return int((np.abs(got.astype(np.float64) - ref64) > allowed).sum()), float((np.abs(got - ref64) / allowed).max())


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("factor", [1e3, 1e4])
@pytest.mark.parametrize("m", [1, 4])
def test_gemv_with_an_outlier_inside_a_block(torch_cuda, fmt, factor, m):
    """One activation `factor` times larger than its neighbours.  Activations are quantized to 16
    bits against the largest magnitude of their own 32-wide block, so the outlier costs precision only
    to the 31 values that share its block.  Judged per element.  The absolute term is 1e-4 of the
    largest output: the fp32 reference loop itself (Device.h:645-658) differs from an exact sum by
    about 1e-6 of that magnitude on the rows where the terms cancel, so a tighter absolute term
    would test summation order, not the quantization."""
    n, k = 512, 4096
    payload = synth.make_weight(fmt, n, k, seed=9, name=f"outlier-{fmt}")
    x = synth.make_activation(m, k, seed=9, name="outlier-x")
    x[:, 1234] *= np.float32(factor)
    w = capi.Weight.from_host(fmt, payload, n, k)
    got = gpu_gemv(torch_cuda, w, x)
    ref = oracle.quantized_matmul(fmt, payload, n, k, x)
    bad, worst = per_element_violations(got, ref)
    assert bad == 0, f"{bad} elements outside the bar, worst at {worst:.2f} of the allowance"
    assert max_rel_err(got, ref) <= REL_TOL


def test_packed_activations_round_trip_error_bound(torch_cuda):
    """unpack(pack(x)) differs from x by at most half a quantization step of x's own 32-block."""
    torch = torch_cuda
    k = 4096 + 96
    x = synth.make_activation(1, k, seed=4, name="rt-x")
    x[0, 100] = 5e3
    x[0, 4100:4132] = 0.0
    xd = torch.from_numpy(x).cuda()
    packed = torch.zeros(capi.packed_activation_bytes(k, 1), dtype=torch.uint8, device="cuda")
    capi.pack_activations(xd.data_ptr(), 1, k, packed.data_ptr())
    back = torch.empty(k, dtype=torch.float32, device="cuda")
    capi.unpack_activations(packed.data_ptr(), k, back.data_ptr())
    torch.cuda.synchronize()
    got = back.cpu().numpy()
    amax = np.abs(x[0].reshape(-1, 32)).max(axis=1)
    step = np.repeat(amax / 32639.0, 32)
    assert (np.abs(got - x[0]) <= 0.51 * step + 1e-30).all()
    assert (got[4100:4132] == 0).all()


# ---- fused forms ----------------------------------------------------------------------------------

def _packed(torch, x_row):
    k = x_row.size
    xd = torch.from_numpy(np.ascontiguousarray(x_row.reshape(1, k))).cuda()
    packed = torch.zeros(capi.packed_activation_bytes(k, 1), dtype=torch.uint8, device="cuda")
    capi.pack_activations(xd.data_ptr(), 1, k, packed.data_ptr())
    return packed


def _unpacked(torch, packed, k):
    out = torch.empty(k, dtype=torch.float32, device="cuda")
    capi.unpack_activations(packed.data_ptr(), k, out.data_ptr())
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(512, 1024), (4096, 4096), (1024, 2560 + 256 * 17), (4096, 11008)])
def test_fused_residual_norm_chain(torch_cuda, fmt, shape):
    """h += W.x; the next matvec's input pack(h * w_norm) and sums of squares; then a matvec that applies
    1/rms — together RMSNorm(h + W.x) * w_norm followed by a linear (LLaMABuilder.cpp:502-557)."""
    from oracle import llama_ref as R
    torch = torch_cuda
    n, k = shape
    payload = synth.make_weight(fmt, n, k, seed=12, name=f"resid-{fmt}-{n}")
    x = synth.make_activation(1, k, seed=12, name="resid-x")
    h0 = synth.make_activation(1, n, seed=12, name="resid-h")[0]
    nw = synth.make_norm_weight(n, seed=12, name="resid-norm")
    w = capi.Weight.from_host(fmt, payload, n, k)
    h = torch.from_numpy(h0.copy()).cuda()
    nwd = torch.from_numpy(nw).cuda()
    packed_out = torch.zeros(capi.packed_activation_bytes(n, 1), dtype=torch.uint8, device="cuda")
    ss = torch.zeros(n // 32, dtype=torch.float64, device="cuda")
    w.gemv_packed_residual(_packed(torch, x).data_ptr(), h.data_ptr(), nwd.data_ptr(), packed_out.data_ptr(), ss.data_ptr())
    torch.cuda.synchronize()
    assert capi.kernel_status(0) == 0
    h_ref = (h0 + oracle.quantized_matmul(fmt, payload, n, k, x)[0]).astype(np.float32)
    h_got = h.cpu().numpy()
    assert max_rel_err(h_got, h_ref) <= REL_TOL
    # sums of squares and packed values are functions of the h the GPU holds
    want_ss = (h_got.astype(np.float64) ** 2).reshape(-1, 32).sum(axis=1)
    assert np.allclose(ss.cpu().numpy(), want_ss, rtol=1e-12, atol=0)
    scaled = h_got * nw
    step = np.repeat(np.abs(scaled.reshape(-1, 32)).max(axis=1) / 32639.0, 32)
    assert (np.abs(_unpacked(torch, packed_out, n) - scaled) <= 0.51 * step + 1e-30).all()
    # consumer: a second linear on RMSNorm(h) * w_norm
    n2 = 256
    payload2 = synth.make_weight(fmt, n2, n, seed=13, name=f"resid2-{fmt}-{n}")
    w2 = capi.Weight.from_host(fmt, payload2, n2, n)
    y2 = torch.full((n2,), float("nan"), dtype=torch.float32, device="cuda")
    w2.gemv_packed_rms(packed_out.data_ptr(), ss.data_ptr(), n // 32, n, 1e-6, y2.data_ptr())
    torch.cuda.synchronize()
    xn = R.rmsnorm(h_ref[None, :], nw, 1e-6)
    assert max_rel_err(y2.cpu().numpy(), oracle.quantized_matmul(fmt, payload2, n2, n, xn)[0]) <= REL_TOL


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(256, 512), (11008, 4096), (1376, 4096)])
def test_fused_swiglu(torch_cuda, fmt, shape):
    """silu(gate.x / rms) * (up.x / rms) from one interleaved gate|up weight (Layer/SwiGLU.h:54-64)."""
    from oracle import llama_ref as R
    torch = torch_cuda
    ffn, d = shape
    gate = synth.make_weight(fmt, ffn, d, seed=14, name=f"glu-gate-{fmt}-{ffn}")
    up = synth.make_weight(fmt, ffn, d, seed=14, name=f"glu-up-{fmt}-{ffn}")
    w = capi.Weight.from_host(fmt, capi.interleave_gate_up(fmt, gate, up, ffn, d), 2 * ffn, d)
    hrow = synth.make_activation(1, d, seed=14, name="glu-h")
    nw = synth.make_norm_weight(d, seed=14, name="glu-norm")
    ss = torch.from_numpy((hrow[0].astype(np.float64) ** 2).reshape(-1, 32).sum(axis=1)).cuda()
    packed_in = _packed(torch, hrow[0] * nw)
    act = torch.full((ffn,), float("nan"), dtype=torch.float32, device="cuda")
    w.gemv_packed_swiglu(packed_in.data_ptr(), ss.data_ptr(), d // 32, d, 1e-6, act.data_ptr())
    torch.cuda.synchronize()
    assert capi.kernel_status(0) == 0
    xn = R.rmsnorm(hrow, nw, 1e-6)
    g = oracle.quantized_matmul(fmt, gate, ffn, d, xn)[0]
    u = oracle.quantized_matmul(fmt, up, ffn, d, xn)[0]
    ref = (R.silu(g) * u).astype(np.float32)
    got = act.cpu().numpy()
    assert max_rel_err(got, ref) <= 2 * REL_TOL   # a product of two results, each within the bar


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(256, 512), (11008, 4096), (1376, 4096), (5504, 8192)])
def test_fused_swiglu_packed_output(torch_cuda, fmt, shape):
    """The same product written as the packed input of ffn_down: the fp32 copy equals the oracle's within the
    bar, and unpacking the packed record gives the fp32 copy within the 16-bit quantization step of its block."""
    from oracle import llama_ref as R
    torch = torch_cuda
    ffn, d = shape
    gate = synth.make_weight(fmt, ffn, d, seed=17, name=f"glup-gate-{fmt}-{ffn}")
    up = synth.make_weight(fmt, ffn, d, seed=17, name=f"glup-up-{fmt}-{ffn}")
    w = capi.Weight.from_host(fmt, capi.interleave_gate_up(fmt, gate, up, ffn, d), 2 * ffn, d)
    hrow = synth.make_activation(1, d, seed=17, name="glup-h")
    nw = synth.make_norm_weight(d, seed=17, name="glup-norm")
    ss = torch.from_numpy((hrow[0].astype(np.float64) ** 2).reshape(-1, 32).sum(axis=1)).cuda()
    packed_in = _packed(torch, hrow[0] * nw)
    act = torch.full((ffn,), float("nan"), dtype=torch.float32, device="cuda")
    packed_out = torch.zeros(capi.packed_activation_bytes(ffn, 1), dtype=torch.uint8, device="cuda")
    w.gemv_packed_swiglu_pack(packed_in.data_ptr(), ss.data_ptr(), d // 32, d, 1e-6, packed_out.data_ptr(), act.data_ptr())
    back = torch.empty(ffn, dtype=torch.float32, device="cuda")
    capi.unpack_activations(packed_out.data_ptr(), ffn, back.data_ptr())
    torch.cuda.synchronize()
    assert capi.kernel_status(0) == 0
    xn = R.rmsnorm(hrow, nw, 1e-6)
    g = oracle.quantized_matmul(fmt, gate, ffn, d, xn)[0]
    u = oracle.quantized_matmul(fmt, up, ffn, d, xn)[0]
    ref = (R.silu(g) * u).astype(np.float32)
    got = act.cpu().numpy()
    assert max_rel_err(got, ref) <= 2 * REL_TOL
    blocks = np.abs(got).reshape(-1, 32).max(axis=1, keepdims=True)
    step = blocks / 32639.0
    assert (np.abs(back.cpu().numpy().reshape(-1, 32) - got.reshape(-1, 32)) <= 0.51 * step + 1e-30).all()
    # without the fp32 copy the packed record is the same
    packed2 = torch.zeros_like(packed_out)
    w.gemv_packed_swiglu_pack(packed_in.data_ptr(), ss.data_ptr(), d // 32, d, 1e-6, packed2.data_ptr())
    torch.cuda.synchronize()
    assert torch.equal(packed2, packed_out)


def test_fused_swiglu_packed_rejects_rows_not_a_multiple_of_64(torch_cuda):
    torch = torch_cuda
    ffn, d = 48, 256
    gate = synth.make_weight(capi.Q4_0, ffn, d, seed=1, name="glup-bad")
    w = capi.Weight.from_host(capi.Q4_0, capi.interleave_gate_up(capi.Q4_0, gate, gate, ffn, d), 2 * ffn, d)
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.QmmError) as e:
        w.gemv_packed_swiglu_pack(buf.data_ptr(), 0, 0, 0, 0.0, buf.data_ptr())
    assert e.value.code == capi.E_INVALID


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(512, 1024 + 96), (4096, 11008)])
def test_fused_residual_from_fp32_activations(torch_cuda, fmt, shape):
    """h += W.x with x given as fp32 (the kernel packs it itself): the ffn_down step of a decoder block."""
    torch = torch_cuda
    n, k = shape
    if k % synth.BLOCK_ELEMS[fmt]:
        k = 1024 + 256
    payload = synth.make_weight(fmt, n, k, seed=15, name=f"f32resid-{fmt}-{n}")
    x = synth.make_activation(1, k, seed=15, name="f32resid-x")
    h0 = synth.make_activation(1, n, seed=15, name="f32resid-h")[0]
    nw = synth.make_norm_weight(n, seed=15, name="f32resid-norm")
    w = capi.Weight.from_host(fmt, payload, n, k)
    xd = torch.from_numpy(x).cuda()
    h = torch.from_numpy(h0.copy()).cuda()
    nwd = torch.from_numpy(nw).cuda()
    packed_out = torch.zeros(capi.packed_activation_bytes(n, 1), dtype=torch.uint8, device="cuda")
    ss = torch.zeros(n // 32, dtype=torch.float64, device="cuda")
    w.gemv_f32_residual(xd.data_ptr(), h.data_ptr(), nwd.data_ptr(), packed_out.data_ptr(), ss.data_ptr())
    torch.cuda.synchronize()
    assert capi.kernel_status(0) == 0
    h_got = h.cpu().numpy()
    assert max_rel_err(h_got, h0 + oracle.quantized_matmul(fmt, payload, n, k, x)[0]) <= REL_TOL
    assert np.allclose(ss.cpu().numpy(), (h_got.astype(np.float64) ** 2).reshape(-1, 32).sum(axis=1), rtol=1e-12, atol=0)
    scaled = h_got * nw
    step = np.repeat(np.abs(scaled.reshape(-1, 32)).max(axis=1) / 32639.0, 32)
    assert (np.abs(_unpacked(torch, packed_out, n) - scaled) <= 0.51 * step + 1e-30).all()
    # the plain batch-1 entry: same product without the residual
    y = torch.full((1, n), float("nan"), dtype=torch.float32, device="cuda")
    w.gemv_f32(xd.data_ptr(), y.data_ptr(), 1)
    torch.cuda.synchronize()
    assert max_rel_err(y.cpu().numpy(), oracle.quantized_matmul(fmt, payload, n, k, x)) <= REL_TOL


def test_fused_forms_reject_shapes_they_cannot_tile(torch_cuda):
    torch = torch_cuda
    payload = synth.make_weight(capi.Q4_0, 24, 256, seed=1, name="bad-fuse")
    w = capi.Weight.from_host(capi.Q4_0, payload, 24, 256)
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    f = torch.zeros(256, dtype=torch.float32, device="cuda")
    dd = torch.zeros(8, dtype=torch.float64, device="cuda")
    with pytest.raises(capi.QmmError) as e:
        w.gemv_packed_residual(buf.data_ptr(), f.data_ptr(), f.data_ptr(), buf.data_ptr(), dd.data_ptr())
    assert e.value.code == capi.E_INVALID
    with pytest.raises(capi.QmmError) as e:
        w.gemv_packed_swiglu(buf.data_ptr(), dd.data_ptr(), 8, 256, 1e-6, f.data_ptr())
    assert e.value.code == capi.E_INVALID
