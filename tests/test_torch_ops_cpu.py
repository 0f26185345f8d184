"""CPU tests of the operator layer: the extension loads, schemas match the reference's strings,
fake kernels infer shapes, the reference's module paths resolve, CPU tensors are rejected."""
import pytest
import torch


@pytest.fixture(scope="module")
def mslk():
    from mslk_b200 import build, compat
    build.build()
    compat.install()
    import mslk.gemm  # noqa: F401
    return torch.ops.mslk


def test_schemas_match_reference_strings(mslk):
    want = {
        "f8f8bf16_rowwise": "mslk::f8f8bf16_rowwise(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor? bias=None, bool use_fast_accum=True) -> Tensor",
        "f8f8bf16_rowwise_out": "mslk::f8f8bf16_rowwise_out(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor(a!) output, Tensor? bias=None, bool use_fast_accum=True) -> ()",
        "f8f8bf16_rowwise_batched": "mslk::f8f8bf16_rowwise_batched(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor? bias=None, bool use_fast_accum=True, Tensor(a!)? output=None) -> Tensor",
        "f8f8bf16_rowwise_grouped_stacked": "mslk::f8f8bf16_rowwise_grouped_stacked(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor M_sizes) -> Tensor",
        "f4f4bf16": "mslk::f4f4bf16(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor? output=None, Tensor? global_scale=None, int mxfp4_block_size=32) -> Tensor",
    }
    for name, schema in want.items():
        assert str(getattr(mslk, name).default._schema) == schema
    assert str(mslk.f4f4bf16_grouped_stacked.default._schema) == (
        "mslk::f4f4bf16_grouped_stacked(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor M_sizes, "
        "Tensor? global_scale=None, Tensor? starting_row_after_padding=None, bool use_mx=True) -> Tensor")
    assert str(mslk.f4f4bf16_grouped_mm.default._schema) == (
        "mslk::f4f4bf16_grouped_mm(Tensor XQ, Tensor WQ, Tensor x_scale, Tensor w_scale, Tensor offsets, "
        "Tensor(a!)? output=None, Tensor(a!)? global_scale=None) -> Tensor")
    import importlib
    importlib.import_module("mslk.moe.activation")   # mslk/moe/activation.py:137-176 defines these from Python
    assert str(mslk.silu_mul.default._schema) == "mslk::silu_mul(Tensor x0, Tensor x1, Tensor? valid_token_count=None) -> Tensor"
    assert str(mslk.silu_mul_quant.default._schema) == (
        "mslk::silu_mul_quant(Tensor x0, Tensor x1, Tensor? scale_ub=None, Tensor? valid_token_count=None) -> (Tensor, Tensor)")


def test_reference_module_paths_resolve(mslk):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row, quantize_fp8_row_meta, triton_quantize_fp8_row  # noqa: F401
    from mslk.quantize.triton.fp4_quantize import _to_blocked, triton_quantize_nvfp4  # noqa: F401
    from mslk.quantize.triton.fp4_utils import dequantize_nvfp4, global_scale_nvfp4  # noqa: F401
    assert str(torch.ops.triton.quantize_fp8_row.default._schema).startswith("triton::quantize_fp8_row(Tensor a")
    assert hasattr(mslk, "quantize_fp8_per_row")


def test_fake_kernels_infer_shapes(mslk):
    f8 = torch.float8_e4m3fn
    xq = torch.empty((3, 50, 256), dtype=f8, device="meta")
    wq = torch.empty((128, 256), dtype=f8, device="meta")
    xs = torch.empty((150,), device="meta")
    ws = torch.empty((128,), device="meta")
    y = mslk.f8f8bf16_rowwise(xq, wq, xs, ws)
    assert y.shape == (3, 50, 128) and y.dtype == torch.bfloat16
    wg = torch.empty((4, 128, 256), dtype=f8, device="meta")
    y = mslk.f8f8bf16_rowwise_grouped_stacked(xq.view(150, 256), wg, xs, torch.empty((512,), device="meta"),
                                              torch.empty((4,), dtype=torch.int64, device="meta"))
    assert y.shape == (150, 128)
    y = mslk.f8f8bf16_rowwise_batched(xq, torch.empty((3, 128, 256), dtype=f8, device="meta"),
                                      torch.empty((3, 50), device="meta"), torch.empty((3, 128), device="meta"))
    assert y.shape == (3, 50, 128) and y.dtype == torch.bfloat16
    y = mslk.f4f4bf16(torch.empty((5, 64), dtype=torch.uint8, device="meta"), torch.empty((32, 64), dtype=torch.uint8, device="meta"),
                      torch.empty((128, 8), dtype=f8, device="meta"), torch.empty((128, 8), dtype=f8, device="meta"),
                      None, torch.empty((1,), device="meta"))
    assert y.shape == (5, 32)
    q, s = torch.ops.triton.quantize_fp8_row(torch.empty((4, 2, 13), dtype=torch.bfloat16, device="meta"), None, None, True, None, 8)
    assert q.shape == (4, 2, 16) and q.dtype == f8 and s.shape == (4, 2) and s.dtype == torch.float32
    q, s = mslk.quantize_nvfp4(torch.empty((150, 64), dtype=torch.bfloat16, device="meta"))
    assert q.shape == (150, 32) and s.shape == (256, 4)


def test_cpu_tensors_are_rejected(mslk):
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row
    with pytest.raises(RuntimeError, match="CUDA"):
        quantize_fp8_row(torch.zeros((2, 16), dtype=torch.bfloat16))
    z = torch.zeros((2, 16)).to(torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="CUDA"):
        mslk.f8f8bf16_rowwise(z, z, torch.ones(2), torch.ones(2))


def test_nvfp4_layout_helpers_roundtrip():
    from mslk_b200.quantize.triton.fp4_utils import _from_blocked, _to_blocked
    x = torch.arange(150 * 9, dtype=torch.int32).reshape(150, 9).to(torch.uint8)
    b = _to_blocked(x)
    assert b.numel() == 256 * 12
    assert torch.equal(_from_blocked(b, (150, 9)), x)
    import oracle
    assert torch.equal(b, oracle.to_blocked(x))


def _fake_cuda(make):
    """Tensors that report device cuda:0 without a GPU (fake tensors): enough for the host-side argument
    checks of mslk_b200.ops, which inspect devices / dtypes / shapes before any kernel is launched."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode(allow_non_fake_inputs=True):
        return make()


def test_ops_reject_a_cpu_tensor_in_every_pointer_argument():
    """A CPU tensor in ANY slot whose raw pointer reaches a kernel must raise in Python, never launch."""
    from mslk_b200 import ops
    f8 = torch.float8_e4m3fn
    xq, wq, xs, ws, out, bias = _fake_cuda(lambda: (
        torch.empty((4, 64), dtype=f8, device="cuda"), torch.empty((128, 64), dtype=f8, device="cuda"),
        torch.empty((4,), device="cuda"), torch.empty((128,), device="cuda"),
        torch.empty((4, 128), dtype=torch.bfloat16, device="cuda"), torch.empty((128,), device="cuda")))
    cpu = {"xq": torch.empty((4, 64)).to(f8), "wq": torch.empty((128, 64)).to(f8), "xs": torch.empty(4),
           "ws": torch.empty(128), "out": torch.empty((4, 128), dtype=torch.bfloat16), "bias": torch.empty(128)}
    for slot in ("xq", "wq", "xs", "ws", "out", "bias"):
        args = {"xq": xq, "wq": wq, "xs": xs, "ws": ws, "out": out, "bias": bias}
        args[slot] = cpu[slot]
        with pytest.raises(RuntimeError, match="CUDA"):
            ops.f8f8bf16_rowwise_out(args["xq"], args["wq"], args["xs"], args["ws"], args["out"], args["bias"])
    # batched: user-provided output
    xq3, wq3, xs3, ws3 = _fake_cuda(lambda: (
        torch.empty((2, 4, 64), dtype=f8, device="cuda"), torch.empty((2, 128, 64), dtype=f8, device="cuda"),
        torch.empty((2, 4), device="cuda"), torch.empty((2, 128), device="cuda")))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.f8f8bf16_rowwise_batched(xq3, wq3, xs3, ws3, output=torch.empty((2, 4, 128), dtype=torch.bfloat16))
    # NVFP4: output and global_scale
    q, wq4, sx, sw, gs = _fake_cuda(lambda: (
        torch.empty((4, 32), dtype=torch.uint8, device="cuda"), torch.empty((128, 32), dtype=torch.uint8, device="cuda"),
        torch.empty((128, 4), dtype=f8, device="cuda"), torch.empty((128, 4), dtype=f8, device="cuda"),
        torch.empty((1,), device="cuda")))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.f4f4bf16(q, wq4, sx, sw, output=torch.empty((4, 128), dtype=torch.bfloat16), global_scale=gs)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.f4f4bf16(q, wq4, sx, sw, global_scale=torch.ones(1))


def test_ops_reject_scale_tensors_shorter_than_the_padded_swizzled_layout():
    """The NVFP4 kernels copy whole 512-byte scale atoms: an unpadded scale tensor would be read past its end."""
    from mslk_b200 import ops
    f8 = torch.float8_e4m3fn
    M, N, K = 4, 144, 64                      # padded layouts: x [128, 4], w [256, 4]
    q, wq, gs = _fake_cuda(lambda: (torch.empty((M, K // 2), dtype=torch.uint8, device="cuda"),
                                    torch.empty((N, K // 2), dtype=torch.uint8, device="cuda"),
                                    torch.empty((1,), device="cuda")))
    ok_x, ok_w, short_x, short_w = _fake_cuda(lambda: (
        torch.empty((128, 4), dtype=f8, device="cuda"), torch.empty((256, 4), dtype=f8, device="cuda"),
        torch.empty((M, 4), dtype=f8, device="cuda"), torch.empty((N, 4), dtype=f8, device="cuda")))
    with pytest.raises(RuntimeError, match="x_scale holds"):
        ops.f4f4bf16(q, wq, short_x, ok_w, global_scale=gs)
    with pytest.raises(RuntimeError, match="w_scale holds"):
        ops.f4f4bf16(q, wq, ok_x, short_w, global_scale=gs)
    # grouped: the weight scales of every group are padded separately
    wg, ms = _fake_cuda(lambda: (torch.empty((2, N, K // 2), dtype=torch.uint8, device="cuda"),
                                 torch.empty((2,), dtype=torch.int64, device="cuda")))
    gs2 = _fake_cuda(lambda: torch.empty((2,), device="cuda"))
    with pytest.raises(RuntimeError, match="w_scale holds"):
        ops.f4f4bf16_grouped_stacked(q, wg, ok_x, ok_w, ms, gs2, use_mx=False)


def test_mxfp4_and_k_grouped_argument_checks():
    """Host-side checks of the MXFP4 forms and of the 2D-2D grouped form: mode / global-scale mismatches, scale
    extents, offsets dtype, output shape -- all raised before any kernel could run."""
    from mslk_b200 import ops
    f8 = torch.float8_e4m3fn
    e8 = getattr(torch, "float8_e8m0fnu", torch.uint8)
    M, N, K, G = 128, 128, 256, 2
    q, wq, wq3, ms, offs, gs = _fake_cuda(lambda: (
        torch.empty((M, K // 2), dtype=torch.uint8, device="cuda"), torch.empty((N, K // 2), dtype=torch.uint8, device="cuda"),
        torch.empty((G, N, K // 2), dtype=torch.uint8, device="cuda"), torch.empty((G,), dtype=torch.int64, device="cuda"),
        torch.empty((G,), dtype=torch.int32, device="cuda"), torch.empty((G,), device="cuda")))
    sx_mx, sw_mx, sw3_mx, sx_nv, sw_nv, short = _fake_cuda(lambda: (
        torch.empty((128 * 8,), dtype=e8, device="cuda"), torch.empty((128 * 8,), dtype=e8, device="cuda"),
        torch.empty((G, 128 * 8), dtype=e8, device="cuda"), torch.empty((128, 16), dtype=f8, device="cuda"),
        torch.empty((128, 16), dtype=f8, device="cuda"), torch.empty((64,), dtype=e8, device="cuda")))
    with pytest.raises(RuntimeError, match="mxfp4_block_size"):
        ops.f4f4bf16(q, wq, sx_mx, sw_mx, mxfp4_block_size=8)
    with pytest.raises(RuntimeError, match="x_scale holds"):
        ops.f4f4bf16(q, wq, short, sw_mx)                      # MXFP4 needs [128, 8] scales for K = 256
    with pytest.raises(RuntimeError, match="use_mx=False"):
        ops.f4f4bf16_grouped_stacked(q, wq3, sx_mx, sw3_mx, ms, gs)          # a global scale with the MX default
    with pytest.raises(RuntimeError, match="needs global_scale"):
        ops.f4f4bf16_grouped_stacked(q, wq3, sx_mx, sw3_mx, ms, None, use_mx=False)
    # grouped_mm: the scale dtype names the format
    with pytest.raises(RuntimeError, match="needs global_scale"):
        ops.f4f4bf16_grouped_mm(q, wq3.transpose(-2, -1), sx_nv, sw_nv, offs)
    if e8 is not torch.uint8:
        with pytest.raises(RuntimeError, match="global_scale is for NVFP4"):
            ops.f4f4bf16_grouped_mm(q, wq3.transpose(-2, -1), sx_mx, sw3_mx, offs, None, gs)
        # 2D-2D: output must be [G, M, N]
        bad_out = _fake_cuda(lambda: torch.empty((M, N), dtype=torch.bfloat16, device="cuda"))
        with pytest.raises(RuntimeError, match=r"\(G, M, N\)"):
            ops.f4f4bf16_grouped_mm(q, wq.transpose(-2, -1), sx_mx, sw_mx, offs, bad_out)
        with pytest.raises(RuntimeError, match="x_scale holds"):
            ops.f4f4bf16_grouped_mm(q, wq.transpose(-2, -1), short, sw_mx, offs)
    with pytest.raises(RuntimeError, match="offsets must be int32"):
        ops.f4f4bf16_grouped_mm(q, wq.transpose(-2, -1), sx_mx, sw_mx, ms)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.quantize_mx4_stacked(torch.zeros(2, dtype=torch.int64), _fake_cuda(
            lambda: torch.empty((M, K), dtype=torch.bfloat16, device="cuda")))


def test_export_strict_traces_through_the_fake_kernels(mslk):
    """torch.export(strict=True) of a module that quantizes and multiplies, as the reference's
    ExportCompileTests.test_f8f8bf16_export does (test/gemm/gemm_test.py:236-289); meta tensors need no GPU."""
    from mslk.quantize.triton.fp8_quantize import quantize_fp8_row

    class Mod(torch.nn.Module):
        def forward(self, x, wq, ws, wg, wgs, m_sizes):
            xq, xs = quantize_fp8_row(x)
            y = torch.ops.mslk.f8f8bf16_rowwise(xq, wq, xs, ws)
            z = torch.ops.mslk.f8f8bf16_rowwise_grouped_stacked(xq, wg, xs, wgs, m_sizes)
            return y, z

    f8 = torch.float8_e4m3fn
    args = (torch.empty((64, 512), dtype=torch.bfloat16, device="meta"),
            torch.empty((256, 512), dtype=f8, device="meta"), torch.empty((256,), device="meta"),
            torch.empty((4, 128, 512), dtype=f8, device="meta"), torch.empty((512,), device="meta"),
            torch.empty((4,), dtype=torch.int64, device="meta"))
    ep = torch.export.export(Mod(), args, strict=True)
    targets = [str(n.target) for n in ep.graph.nodes if n.op == "call_function"]
    assert "triton.quantize_fp8_row.default" in targets
    assert "mslk.f8f8bf16_rowwise.default" in targets and "mslk.f8f8bf16_rowwise_grouped_stacked.default" in targets
    y, z = [n for n in ep.graph.nodes if n.op == "output"][0].args[0]
    assert tuple(y.meta["val"].shape) == (64, 256) and tuple(z.meta["val"].shape) == (64, 128)
