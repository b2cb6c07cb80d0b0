"""NVFP4 operands pinned to a third party: cuBLASLt's block-scaled FP4 GEMM (through
``torch._scaled_mm``) is run on the codes and the TILED scale buffers this library's quantisers
write, and must give the product the CPU oracle computes by decoding the same bytes
(e2m1 code x e4m3 block scale, f64 dot product).

The reference has no NVFP4 arithmetic at all (qsfi_moe.cu:807-821), so the conventions are this
repository's: two codes per byte with the even element in the low nibble, one e4m3 scale per
16 elements, scales stored in 512-byte tiles of 128 rows x 4 blocks. If cuBLASLt reads those bytes
as the same numbers, the format, the scale tiling and the oracle's decoders are not private
inventions. What stays the repository's own: the f32 global scales (applied outside the GEMM on
both sides here), the interleaved gate / up tiling of gated weights, and where the chain
re-quantises."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(256, 384, 512), (128, 128, 2048), (200, 256, 1024)])
def test_cublaslt_reads_our_nvfp4_bytes_as_the_oracle_does(oracle, shape):
    from qs3_b200 import ops
    if not hasattr(torch, "float4_e2m1fn_x2"):
        pytest.skip("this torch build has no packed FP4 dtype")
    m, n, k = shape
    ctx = ops.Context()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(m + n + k)
    x = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=gen, device="cuda") * 0.05).to(torch.bfloat16)
    x_codes, x_scales = ops.nvfp4_quantize_act(ctx, x, 1.0)
    wq = ops.nvfp4_quantize_weight(ctx, w[None].contiguous(), gated=False)
    x_tiled = ops.nvfp4_tile_scales(ctx, x_scales[None].contiguous(), gated=False)
    torch.cuda.synchronize()
    fp4, e4m3 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    try:
        got = torch._scaled_mm(x_codes.view(fp4), wq.packed[0].view(fp4).t(), x_tiled.view(e4m3),
                               wq.scale_tiled.view(e4m3), out_dtype=torch.bfloat16)
        torch.cuda.synchronize()
    except (RuntimeError, NotImplementedError) as exc:
        pytest.skip(f"torch._scaled_mm has no NVFP4 path here: {str(exc)[:200]}")
    g = float(wq.global_scale[0].item())
    got = got.float().cpu().numpy().astype(np.float64) * g
    xd = oracle.nvfp4_dequantize(x_codes.cpu().numpy(), x_scales.cpu().numpy()).astype(np.float64)
    wd = oracle.nvfp4_dequantize(wq.packed[0].cpu().numpy(), wq.scale_linear[0].cpu().numpy()).astype(np.float64)
    ref = xd @ wd.T * g
    rel = np.linalg.norm(got - ref) / np.linalg.norm(ref)
    # cuBLASLt rounds its output to bf16 (2^-9 relative per element); a wrong nibble order, scale
    # position or decoder would show as an error of order one
    assert rel <= 4e-3, rel
    assert np.max(np.abs(got - ref)) <= 2.0 ** -6 * np.max(np.abs(ref))


def test_expert_chain_of_the_library_matches_a_chain_of_cublaslt_gemms():
    """One expert, every token routed to it with weight 1, through ``qsfi_moe_execute_nvfp4`` (this
    library's kernels: gather, grouped gate_up GEMM + SwiGLU + re-quantisation, grouped down GEMM,
    combine) against the same chain built from two cuBLASLt block-scaled FP4 GEMMs on the same operand
    bytes. The third-party chain rounds Y1 to bf16 and re-quantises the SwiGLU output from bf16 where
    the library keeps f32; re-quantisation to FP4 is discontinuous (a last-bit change of an input flips
    a code, a 17-33 % step of that element), so two correct chains differ by a few per cent (3.0e-2
    measured) where a wrong layout, nibble order or scale position gives an error of order one. The tight
    bound is the oracle's (tests/test_gpu_nvfp4.py); this one shows the kernels and cuBLASLt agree on
    what the bytes mean."""
    from qs3_b200 import ops
    if not hasattr(torch, "float4_e2m1fn_x2"):
        pytest.skip("this torch build has no packed FP4 dtype")
    t, h, i = 384, 512, 256
    ctx = ops.Context()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    rnd = lambda *s: torch.randn(s, generator=gen, device="cuda")
    x = rnd(t, h).to(torch.bfloat16)
    w_gu = (rnd(2 * i, h) * 0.16).to(torch.bfloat16)     # global scale 1: keep the block scales normal
    w_dn = (rnd(h, i) * 0.16).to(torch.bfloat16)
    xp, xs = ops.nvfp4_quantize_act(ctx, x, 1.0)
    gup, gus = ops.nvfp4_quantize_act(ctx, w_gu, 1.0)
    dnp, dns = ops.nvfp4_quantize_act(ctx, w_dn, 1.0)
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=1, top_k=1, backend=ops.capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros((t, 1), dtype=torch.int32, device="cuda")
    wts = torch.ones((t, 1), dtype=torch.float32, device="cuda")
    ops.moe_execute_nvfp4(plan, xp, xs, ids, wts, gup[None].contiguous(), gus[None].contiguous(),
                          dnp[None].contiguous(), dns[None].contiguous(), out, ws)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0

    fp4, e4m3 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
    tile = lambda s: ops.nvfp4_tile_scales(ctx, s[None].contiguous(), gated=False).view(e4m3)
    try:
        y1 = torch._scaled_mm(xp.view(fp4), gup.view(fp4).t(), tile(xs), tile(gus), out_dtype=torch.bfloat16)
    except (RuntimeError, NotImplementedError) as exc:
        pytest.skip(f"torch._scaled_mm has no NVFP4 path here: {str(exc)[:200]}")
    g, u = y1[:, :i].float(), y1[:, i:].float()
    act = (g * torch.sigmoid(g) * u).to(torch.bfloat16)
    ap, a_s = ops.nvfp4_quantize_act(ctx, act, 1.0)
    y2 = torch._scaled_mm(ap.view(fp4), dnp.view(fp4).t(), tile(a_s), tile(dns), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    want = y2.float().cpu().numpy().astype(np.float64)
    got = out.float().cpu().numpy().astype(np.float64)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 5e-2, rel
    assert np.max(np.abs(got - want)) <= 0.25 * np.max(np.abs(want))
