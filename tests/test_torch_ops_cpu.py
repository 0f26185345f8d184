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
