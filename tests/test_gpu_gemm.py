"""GPU parity of the dense bf16 GEMM entry (qscb_gemm_bf16: router logits and the
shared-expert projections) against the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import bf16, f32, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm():
    from qs3_b200 import ops
    return ops.GemmContext()


def _ref(x, w):
    return f32(x).astype(np.float64) @ f32(w).astype(np.float64).T


def test_identity_known_answer(gemm):
    # one 128 x 128 x 64 tile: x = eye-like, weight rows = distinct small integers
    x = np.zeros((128, 64), np.float32)
    x[np.arange(128), np.arange(128) % 64] = 1.0
    w = (np.arange(128 * 64).reshape(128, 64) % 251 - 125).astype(np.float32)
    out = torch.zeros((128, 128), dtype=torch.float32, device="cuda")
    gemm.gemm_bf16(to_dev(bf16(x)), to_dev(bf16(w)), out)
    torch.cuda.synchronize()
    want = x.astype(np.float64) @ f32(bf16(w)).astype(np.float64).T
    assert np.array_equal(to_np(out), want.astype(np.float32))


@pytest.mark.parametrize("shape", [(2, 64, 128), (16, 256, 8), (130, 2048, 512), (64, 200, 96),
                                   (300, 72, 130), (8192 // 8, 2048, 512), (5, 12, 7), (128, 4096, 64)])
@pytest.mark.parametrize("out_dtype", ["f32", "bf16"])
def test_gemm_matches_oracle(gemm, oracle, shape, out_dtype):
    rows, k, n = shape
    rng = np.random.default_rng(rows * 7 + k + n)
    x = bf16(rng.standard_normal((rows, k), dtype=np.float32))
    w = bf16(rng.standard_normal((n, k), dtype=np.float32) * 0.05)
    ref64 = _ref(x, w)
    if out_dtype == "f32":
        out = torch.full((rows, n), 777.0, dtype=torch.float32, device="cuda")
        gemm.gemm_bf16(to_dev(x), to_dev(w), out)
        got = to_np(out).astype(np.float64)
        # tensor-core accumulation is a little below IEEE f32: ~2e-6 of the norm at k = 2048
        assert np.linalg.norm(got - ref64) <= 1e-5 * np.linalg.norm(ref64) + 1e-12
        o = oracle.gemm_bf16(x, w, "f32").astype(np.float64)
        assert np.linalg.norm(got - o) <= 1e-5 * np.linalg.norm(ref64) + 1e-12
    else:
        out = torch.full((rows, n), 777.0, dtype=torch.bfloat16, device="cuda")
        gemm.gemm_bf16(to_dev(x), to_dev(w), out)
        got = f32(to_np(out)).astype(np.float64)
        assert np.all(np.abs(got - ref64) <= np.abs(ref64) * 2.0 ** -8 + 1e-4)


def test_alpha_beta_and_padded_strides(gemm):
    # upstream tests_cuda_qscb_gemm.inc:719-921: f32 output with beta and padded row strides,
    # sentinel padding must survive
    rows, k, n = 37, 264, 48
    rng = np.random.default_rng(9)
    x_full = torch.full((rows, k + 8), 3.0, dtype=torch.bfloat16, device="cuda")
    w_full = torch.full((n, k + 16), -2.0, dtype=torch.bfloat16, device="cuda")
    o_full = torch.full((rows, n + 4), 5.0, dtype=torch.float32, device="cuda")
    x = bf16(rng.standard_normal((rows, k), dtype=np.float32))
    w = bf16(rng.standard_normal((n, k), dtype=np.float32) * 0.1)
    c = rng.standard_normal((rows, n), dtype=np.float32)
    x_full[:, :k] = to_dev(x)
    w_full[:, :k] = to_dev(w)
    o_full[:, :n] = to_dev(c)
    gemm.gemm_bf16(x_full[:, :k], w_full[:, :k], o_full[:, :n], alpha=0.5, beta=-1.5)
    got = to_np(o_full)
    want = 0.5 * _ref(x, w) - 1.5 * c
    assert np.allclose(got[:, :n], want, atol=2e-4, rtol=1e-5)
    assert np.all(got[:, n:] == 5.0)
    # bf16 output with beta
    ob = torch.full((rows, n), 0.0, dtype=torch.bfloat16, device="cuda")
    ob.copy_(to_dev(bf16(c)))
    gemm.gemm_bf16(x_full[:, :k], w_full[:, :k], ob, alpha=2.0, beta=1.0)
    want = 2.0 * _ref(x, w) + f32(bf16(c))
    assert np.all(np.abs(f32(to_np(ob)) - want) <= np.abs(want) * 2.0 ** -8 + 1e-5)


def test_validation_errors(gemm):
    from qs3_b200 import ops
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.Qs3Error) as e:
        gemm.gemm_bf16(x, w, torch.zeros((4, 9), dtype=torch.float32, device="cuda"))
    assert e.value.status == 1 and "shape mismatch" in e.value.message
    with pytest.raises(ops.Qs3Error) as e:
        gemm.gemm_bf16(x.float(), w, torch.zeros((4, 8), dtype=torch.float32, device="cuda"))
    assert e.value.status == 1


@pytest.mark.parametrize("kind", ["bf16", "fp8", "nvfp4"])
def test_tensor_peak_probe_runs(kind):
    # the probe is a measurement aid: it must finish, report a plausible positive rate
    # and leave the device error word clear (all its waits are bounded)
    from qs3_b200 import ops
    ctx = ops.Context()
    tf = ops.tensor_peak_probe(ctx, kind, n=128, iters=2000)
    assert 10.0 < tf < 40000.0
    assert ctx.read_device_error() == 0


@pytest.mark.parametrize("shape", [(65, 64, 128), (129, 64, 257), (257, 192, 300), (700, 1024, 2304), (128, 2048, 5000),
                                   (2100, 256, 2400), (2305, 128, 2048)])   # the last two: CTA-pair kernel
@pytest.mark.parametrize("out_dtype", ["f32", "bf16"])
def test_dense_kernel_edges_and_epilogue(gemm, shape, out_dtype):
    """More than 64 rows, k a multiple of 64, n >= 128: the persistent 128 x 256 kernel, or with at
    least 74 tiles of 256 x 256 its CTA-pair variant. Ragged rows and columns, alpha / beta, padded
    row strides (sentinel padding must survive)."""
    rows, k, n = shape
    rng = np.random.default_rng(rows + 3 * k + 5 * n)
    x = bf16(rng.standard_normal((rows, k), dtype=np.float32))
    w = bf16(rng.standard_normal((n, k), dtype=np.float32) * 0.05)
    c = bf16(rng.standard_normal((rows, n), dtype=np.float32))
    dt = torch.float32 if out_dtype == "f32" else torch.bfloat16
    x_full = torch.full((rows, k + 8), 3.0, dtype=torch.bfloat16, device="cuda")
    w_full = torch.full((n, k + 24), -2.0, dtype=torch.bfloat16, device="cuda")
    o_full = torch.full((rows, n + 8), 5.0, dtype=dt, device="cuda")
    x_full[:, :k] = to_dev(x)
    w_full[:, :k] = to_dev(w)
    o_full[:, :n] = to_dev(c).to(dt)
    gemm.gemm_bf16(x_full[:, :k], w_full[:, :k], o_full[:, :n], alpha=0.5, beta=-1.5)
    torch.cuda.synchronize()
    got = o_full.float().cpu().numpy().astype(np.float64)
    want = 0.5 * _ref(x, w) - 1.5 * f32(c).astype(np.float64)
    if out_dtype == "f32":
        assert np.linalg.norm(got[:, :n] - want) <= 1e-5 * np.linalg.norm(want) + 1e-9
    else:
        assert np.all(np.abs(got[:, :n] - want) <= np.abs(want) * 2.0 ** -7 + 2e-3)
    assert np.all(got[:, n:] == 5.0)
