"""fish_scales_ops_b200: the MXFP8 block-scaled dense linear and MoE layer of fish-scales-ops, written from
scratch for NVIDIA B200 (sm_100a) and exposed through the reference's own Python surface::

    import fish_scales_ops_b200 as fso

    weight = fso.dense.prepare_weight(w, format="mxfp8");  y = fso.dense.linear(x, weight)
    experts = fso.moe.prepare_experts(w13, w2, format="mxfp8");  out = fso.moe.layer(h, experts, ids, wts)

The compute lives in ``libfso_b200.so`` (hand-written CUDA behind the C ABI of ``include/fso_b200.h``); Python only
validates arguments, allocates outputs and passes pointers. There is no other backend and no CPU path.
"""
from . import _build, _lib  # noqa: F401
from . import compat, dense, moe  # noqa: F401

__version__ = "0.1.0"


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile ``libfso_b200.so`` in-tree for sm_100a (nvcc); returns its path."""
    return _build.build(force=force, verbose=verbose)


def build_info() -> dict:
    import torch

    return {"version": __version__, "source_build": True, "torch": torch.__version__, "library": _lib.lib_path(),
            "arch": "sm_100a"}
