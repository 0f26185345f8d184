"""One mixture-of-experts FFN assembled from the kernels of this library, the way the reference's layer
chains its own (mslk/moe/layers.py:1104-1129): token gather + score scaling + FP8 row quantize, grouped
gate+up GEMM, fused SwiGLU + quantize, grouped down GEMM with the combine (scatter-add) in its epilogue.
Checked against the same layer in fp32 torch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _route(T, E, topk, gen):
    logits = torch.randn((T, E), generator=gen)
    scores = torch.softmax(logits, dim=1)
    top = torch.topk(scores, topk, dim=1).indices                     # [T, topk]
    token = torch.arange(T).repeat_interleave(topk)
    expert = top.reshape(-1)
    order = torch.sort(expert, stable=True).indices                   # rows stacked expert by expert
    return scores, token[order].to(torch.int32), expert[order], torch.bincount(expert, minlength=E)


@pytest.mark.parametrize("T,D,F,E,topk", [(512, 1024, 2048, 8, 2), (300, 512, 768, 16, 1), (64, 256, 512, 4, 4)])
def test_moe_ffn_matches_fp32_layer(T, D, F, E, topk):
    from mslk_b200 import compat
    compat.install()
    from mslk.gemm.triton.grouped_gemm import grouped_gemm_fp8_rowwise
    from mslk.moe.activation import silu_mul_quant
    from mslk.moe.gather_scatter import gather_scale_quant_dense_tokens
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    from mslk_b200._lib import device_status

    g = torch.Generator().manual_seed(T + E)
    x = torch.randn((T, D), generator=g).to(torch.bfloat16)
    w13 = (torch.randn((E, 2 * F, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn((E, D, F), generator=g) * F ** -0.5).to(torch.bfloat16)
    scores, tok, ex, counts = _route(T, E, topk, g)
    scores = scores.to(torch.bfloat16)

    xd, tokd, exd, sd = x.cuda(), tok.cuda(), ex.cuda(), scores.cuda()
    m_sizes = counts.to(torch.int64).cuda()
    w13q, w13s = quantize_fp8_row(w13.cuda())
    w2q, w2s = quantize_fp8_row(w2.cuda())

    xq, xs = gather_scale_quant_dense_tokens(xd, tokd, exd, sd)
    h = grouped_gemm_fp8_rowwise(xq, w13q.view(E * 2 * F, D), m_sizes, xs, w13s.view(-1))
    hq, hs = silu_mul_quant(h[:, :F], h[:, F:])
    out = torch.zeros((T, D), dtype=torch.bfloat16, device="cuda")
    grouped_gemm_fp8_rowwise(hq, w2q.view(E * D, F), m_sizes, hs, w2s.view(-1), _output_tensor=out,
                             _scatter_add_indices=tokd)
    assert device_status() == 0

    # fp32 layer
    ref = torch.zeros((T, D), dtype=torch.float32)
    xf, w13f, w2f = x.float(), w13.float(), w2.float()
    for i in range(tok.numel()):
        t, e = int(tok[i]), int(ex[i])
        a = (xf[t] * float(scores[t, e])) @ w13f[e].T
        y = torch.nn.functional.silu(a[:F]) * a[F:]
        ref[t] += y @ w2f[e].T
    err = (out.cpu().float() - ref).norm() / ref.norm()
    assert float(err) < 0.08, f"relative error {float(err)}"


@pytest.mark.parametrize("T,D,F,E,topk", [(384, 1024, 1024, 8, 2), (200, 512, 768, 4, 1)])
def test_moe_ffn_nvfp4_matches_fp32_layer(T, D, F, E, topk):
    """The same layer on the NVFP4 path: bf16 gather, per-expert global scales, stacked NVFP4 quantization, grouped
    NVFP4 GEMMs, unquantized SwiGLU, scatter-add of the expert outputs."""
    from mslk_b200 import compat
    compat.install()
    import mslk.gemm  # noqa: F401
    from mslk.moe.activation import silu_mul
    from mslk.moe.gather_scatter import gather_scale_dense_tokens, scatter_add_dense_tokens
    from mslk.quantize.triton.fp4_quantize import calculate_group_max, nvfp4_quantize_stacked
    from mslk_b200._lib import device_status

    g = torch.Generator().manual_seed(T + E)
    x = torch.randn((T, D), generator=g).to(torch.bfloat16)
    w13 = (torch.randn((E, 2 * F, D), generator=g) * D ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn((E, D, F), generator=g) * F ** -0.5).to(torch.bfloat16)
    scores, tok, ex, counts = _route(T, E, topk, g)
    scores = scores.to(torch.bfloat16)
    xd, tokd, exd, sd = x.cuda(), tok.cuda(), ex.cuda(), scores.cuda()
    m_sizes = counts.to(torch.int64).cuda()

    def quant_w(w, rows):      # [E, rows, K] -> stacked NVFP4 with one global scale per expert
        ms = torch.full((E,), rows, dtype=torch.int64, device="cuda")
        flat = w.cuda().reshape(E * rows, -1)
        gs, _ = calculate_group_max(flat, ms)
        q, s2 = nvfp4_quantize_stacked(ms, flat, gs)
        padded = (rows + 127) // 128 * 128
        return q.view(E, rows, -1), s2[: E * padded].view(E, padded, -1), gs

    w13q, w13s, w13g = quant_w(w13, 2 * F)
    w2q, w2s, w2g = quant_w(w2, D)

    xs_tok = gather_scale_dense_tokens(xd, tokd, exd, sd)                     # [a, D] bf16, rows stacked by expert
    gx, _ = calculate_group_max(xs_tok, m_sizes)
    xq, xsc = nvfp4_quantize_stacked(m_sizes, xs_tok, gx)
    h = torch.ops.mslk.f4f4bf16_grouped_stacked(xq, w13q, xsc, w13s, m_sizes, torch.reciprocal(gx * w13g), None, False)
    act = silu_mul(h[:, :F], h[:, F:])
    ga, _ = calculate_group_max(act, m_sizes)
    aq, asc = nvfp4_quantize_stacked(m_sizes, act, ga)
    y = torch.ops.mslk.f4f4bf16_grouped_stacked(aq, w2q, asc, w2s, m_sizes, torch.reciprocal(ga * w2g), None, False)
    out = torch.zeros((T, D), dtype=torch.float32, device="cuda")
    scatter_add_dense_tokens(out, y.float(), tokd)
    assert device_status() == 0

    ref = torch.zeros((T, D), dtype=torch.float32)
    xf, w13f, w2f = x.float(), w13.float(), w2.float()
    for i in range(tok.numel()):
        t, e = int(tok[i]), int(ex[i])
        a = (xf[t] * float(scores[t, e])) @ w13f[e].T
        ref[t] += (torch.nn.functional.silu(a[:F]) * a[F:]) @ w2f[e].T
    err = (out.cpu() - ref).norm() / ref.norm()
    # two 4-bit GEMMs in sequence: the CPU oracle of the same pipeline is 0.23 away from the fp32 layer
    assert float(err) < 0.3, f"relative error {float(err)}"
