"""CPU tests of the drop-in boundary: the C-ABI library builds for sm_100a without a GPU, loads, exports every symbol
that include/es_b200.h declares, and rejects bad arguments before touching the device.  No compute is launched."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from expert_specialization_moe_b200 import _cabi
    return _cabi.load()


def test_library_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "es_b200.h").read_text()
    names = sorted(set(re.findall(r"\b(es_b200_[a-z0-9_]+)\s*\(", header)))
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/es_b200.h but not exported"


def test_version_and_error_strings(lib):
    assert b"sm_100a" in lib.es_b200_version()
    assert lib.es_b200_strerror(0) == b"ok"
    assert b"invalid" in lib.es_b200_strerror(1)


def test_argument_checks_happen_before_any_launch(lib):
    # k not a multiple of 128 / bad dtype / too many experts: rejected on the host (no CUDA call is needed for that)
    rc = lib.es_b200_mxfp8_grouped_quant(None, 0, None, None, None, None, None, 4, 16, 100, None)
    assert rc == 1 and b"k must align to 128" in lib.es_b200_last_error()
    rc = lib.es_b200_mxfp8_grouped_quant(None, 7, None, None, None, None, None, 4, 16, 128, None)
    assert rc == 1 and b"kFloat16 or kBFloat16" in lib.es_b200_last_error()
    rc = lib.es_b200_mxfp8_grouped_mm(None, None, None, None, None, 0, None, None, None, 2000, 16, 128, 128, 0, None, 0,
                                      None)
    assert rc == 1 and b"Number of experts cannot exceed 1024" in lib.es_b200_last_error()
    rc = lib.es_b200_fp8_blockwise_grouped_mm(None, None, None, None, None, 0, None, None, 4, 16, 100, 128, None, 0, None)
    assert rc == 1 and b"n should align 128" in lib.es_b200_last_error()
    assert lib.es_b200_grouped_mm_scratch_bytes(8, 512, 1024, 512) == 256      # the work counters
    assert lib.es_b200_set_tunable(b"no_such_tunable", 1) == 1 and b"unknown tunable" in lib.es_b200_last_error()
    # every name that include/es_b200.h documents is accepted (the values written are the built-in defaults)
    for name, value in ((b"mm_heavy_min_rows", 0), (b"mm_tiny_max_rows", 0), (b"mm_pair_first_clusters", 32),
                        (b"mm_split_min_rows", 256), (b"mm_stream_max_ctas", 0), (b"mm_pair_max_clusters", 0),
                        (b"mm_dynamic", 1), (b"mm_stream_lsu", 1), (b"mm_stream_mid_lead_ctas", -1),
                        (b"mm_item_k_steps", 16)):
        assert lib.es_b200_set_tunable(name, value) == 0, name
        assert name.decode() in (ROOT / "include" / "es_b200.h").read_text(), name


def test_ops_mirror_reference_signatures():
    import inspect
    from expert_specialization_moe_b200 import ops
    sig = lambda f: list(inspect.signature(f).parameters)
    assert sig(ops.es_sm100_mxfp8_blockscaled_grouped_quant) == [
        "input", "problem_sizes", "expert_offsets", "blockscale_offsets", "quant_output", "scale_factor"]
    assert sig(ops.es_sm100_mxfp8_blockscaled_grouped_mm) == [
        "output", "a", "b", "sfa", "sfb", "problem_sizes", "expert_offsets", "blockscale_offsets"]
    assert sig(ops.es_fp8_blockwise_scaled_grouped_mm) == [
        "output", "a", "b", "scales_a", "scales_b", "stride_a", "stride_b", "stride_d", "problem_sizes",
        "expert_offsets", "workspace"]


def test_ops_have_no_cpu_fallback():
    """As in the reference, only a CUDA kernel is registered: the dispatcher refuses CPU tensors."""
    from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_quant as quant
    x = torch.zeros((4, 128), dtype=torch.bfloat16)
    ps = torch.tensor([[4, 0, 128]], dtype=torch.int32)
    z = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CPU"):
        quant(x, ps, z, z, torch.zeros((4, 128), dtype=torch.uint8), torch.zeros((128, 4), dtype=torch.uint8))


# the operator schemas of the reference extension (expert_specialization/csrc/expert_specialization.cpp:57-66)
REFERENCE_SCHEMAS = {
    "es_fp8_blockwise_scaled_grouped_mm":
        "(Tensor output, Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor stride_a, Tensor stride_b, "
        "Tensor stride_d, Tensor problem_sizes, Tensor expert_offsets, Tensor workspace) -> ()",
    "es_sm100_mxfp8_blockscaled_grouped_mm":
        "(Tensor a, Tensor b, Tensor sfa, Tensor sfb, Tensor d, Tensor problem_sizes, Tensor expert_offsets, "
        "Tensor blockscale_offsets) -> ()",
    "es_sm100_mxfp8_blockscaled_grouped_quant":
        "(Tensor input, Tensor problem_sizes, Tensor expert_offsets, Tensor blockscale_offsets, Tensor quant_output, "
        "Tensor scale_factor) -> ()",
}


def test_torch_ops_are_registered_with_the_reference_schemas():
    from expert_specialization_moe_b200 import _cabi
    ops = _cabi.torch_ops()
    for name, want in REFERENCE_SCHEMAS.items():
        schema = str(getattr(ops, name).default._schema)
        assert schema == f"es_b200::{name}{want}", schema
        keys = torch._C._dispatch_dump(f"es_b200::{name}")
        assert "CUDA" in keys and "CPU:" not in keys, keys          # CUDA dispatch key only, as in the reference


def test_product_does_not_import_the_oracle():
    for f in (ROOT / "expert_specialization_moe_b200").rglob("*.py"):
        txt = f.read_text()
        assert "import oracle" not in txt and "from oracle" not in txt, f
