"""The public surface of the package, pinned (CPU): exported names of ``dense`` and ``moe``, the schemas of the four
custom ops and the C ABI's symbol list. Mirrors what tests/gemm/unit/test_public_surface.py of the reference pins
for the same two namespaces."""
import torch

import fish_scales_ops_b200 as fso

DENSE = {"FORMATS", "ACTIVATIONS", "DenseWeight", "prepare_weight", "linear", "linear_quantized",
         "quantize_activation", "activation_contract", "include_dir", "supported", "describe"}
MOE = {"FORMATS", "MoeExperts", "prepare_experts", "layer", "transient_bytes", "supported", "describe"}
SCHEMAS = {
    "dense_linear": "fish_scales_ops::dense_linear(Tensor x, Tensor weight, Tensor scale, str kind, "
                    "Tensor? bias=None, Tensor? x_scale=None, Tensor? residual=None, str? activation=None) -> Tensor",
    "dense_linear_quantized": "fish_scales_ops::dense_linear_quantized(Tensor x, Tensor weight, Tensor scale, "
                              "str kind, Tensor? bias=None, Tensor? x_scale=None, str? activation=None) "
                              "-> (Tensor, Tensor)",
    "dense_quantize_activation": "fish_scales_ops::dense_quantize_activation(Tensor x) -> (Tensor, Tensor)",
    "moe_layer": "fish_scales_ops::moe_layer(Tensor hidden, Tensor w13, Tensor sw13, Tensor w2, Tensor sw2, "
                 "Tensor topk_ids, Tensor topk_w, Tensor? bias, Tensor? bias_scale, str kind, "
                 "bool w13_interleaved) -> Tensor",
}


def test_exported_names():
    assert set(fso.dense.__all__) == DENSE
    assert set(fso.moe.__all__) == MOE
    for ns, names in ((fso.dense, DENSE), (fso.moe, MOE)):
        for n in names:
            assert hasattr(ns, n), n
    assert fso.dense.FORMATS == ("bsfp8", "mxfp8") and fso.moe.FORMATS == ("bsfp8", "mxfp8")
    assert fso.dense.ACTIVATIONS == ("gelu_erf",)


def test_custom_op_schemas():
    for name, want in SCHEMAS.items():
        op = getattr(torch.ops.fish_scales_ops, name).default
        assert str(op._schema) == want, name


def test_supported_and_describe_never_raise():
    for ns in (fso.dense, fso.moe):
        assert ns.supported("no-such-format") is False
        assert ns.supported(None) is False
        assert ns.supported("mxfp8", arch="sm_100") is True
        assert ns.supported("bsfp8", arch=103) is True
        assert ns.supported("mxfp8", arch="sm_90") is False
        assert isinstance(ns.describe(), str) and "sm_100" in ns.describe()


def test_include_dir_holds_the_headers():
    import os

    d = fso.dense.include_dir()
    for name in ("fso_b200.h", "fso_b200_activation_contract.h"):
        assert os.path.isfile(os.path.join(d, name)), name
