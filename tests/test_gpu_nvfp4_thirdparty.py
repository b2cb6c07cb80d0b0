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
