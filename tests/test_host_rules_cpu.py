"""Host-side rules that need no GPU: the decode-band rule of the MoE layer (a pure function of the call's shape and
the SM count) and the eager / traced dispatch of the public calls."""
import pytest
import torch


@pytest.fixture()
def moe_mod(monkeypatch):
    from fish_scales_ops_b200 import moe

    monkeypatch.setattr(moe, "_sm_count", lambda: 148)
    monkeypatch.delenv("FSO_B200_MOE_DECODE", raising=False)
    return moe


# (tokens, top-k, experts, I) -> (FC1 takes the band, FC2 takes the band)
BAND_CASES = [
    ((1, 2, 8, 14336), (True, True)),       # Mixtral, one token: two experts in use, 448 FC1 tiles
    ((4, 2, 8, 14336), (True, True)),
    ((16, 2, 8, 14336), (True, True)),      # 32 pairs: one 32-row token sub-tile per block
    ((24, 2, 8, 14336), (False, False)),    # six rows per expert: the prefill kernels keep the call
    ((64, 2, 8, 14336), (False, False)),
    ((64, 8, 256, 2048), (True, True)),     # DeepSeek-V3: two rows per expert in use
    ((1, 8, 256, 2048), (False, True)),     # eight experts x 32 FC1 panels do not fill the half-SM slots 1.5 times
    ((65, 8, 256, 2048), (False, False)),   # past the band's token limit
    ((0, 2, 8, 14336), (False, False)),
]


@pytest.mark.parametrize("shape,want", BAND_CASES)
def test_decode_band_rule(moe_mod, shape, want):
    assert moe_mod._decode_band(*shape) == want


def test_decode_band_switches(moe_mod, monkeypatch):
    monkeypatch.setenv("FSO_B200_MOE_DECODE", "0")
    assert moe_mod._decode_band(1, 2, 8, 14336) == (False, False)
    monkeypatch.setenv("FSO_B200_MOE_DECODE", "force")
    assert moe_mod._decode_band(64, 2, 8, 14336) == (True, True)
    assert moe_mod._decode_band(65, 2, 8, 14336) == (False, False)


def test_eager_calls_run_the_body_and_traced_calls_the_op():
    from fish_scales_ops_b200._lib import eager_or_op

    calls = []
    body = lambda *a: calls.append(("body", a)) or "body"      # noqa: E731
    op = lambda *a: calls.append(("op", a)) or "op"            # noqa: E731
    assert eager_or_op(body, op, 1, 2) == "body" and calls == [("body", (1, 2))]

    @torch.library.custom_op("fso_test::twice", mutates_args=())
    def twice(x: torch.Tensor) -> torch.Tensor:
        return x * 2

    @twice.register_fake
    def _(x):
        return torch.empty_like(x)

    seen = []

    def traced(x):
        seen.append(torch.compiler.is_compiling())
        return eager_or_op(lambda t: t * 2, torch.ops.fso_test.twice, x)

    x = torch.arange(4.0)
    assert torch.equal(traced(x), x * 2) and seen == [False]
    from torch._dynamo.testing import EagerAndRecordGraphs

    backend = EagerAndRecordGraphs()
    out = torch.compile(traced, backend=backend, fullgraph=True)(x)
    assert torch.equal(out, x * 2)
    nodes = [n for g in backend.graphs for n in g.graph.nodes if n.op == "call_function"]
    assert len(nodes) == 1 and "fso_test" in str(nodes[0].target)


# (M, N, K) on 148 SMs -> (weights on MMA-M, MMA-N tile, K slices, CTA-pair kernel)
DENSE_ROUTES = [
    ((8192, 28672, 4096), (False, 256, 1, True)),    # the headline cell: 3584 pair tiles on 74 pairs
    ((8192, 4096, 14336), (False, 256, 1, True)),
    ((8192, 3584, 4096), (False, 256, 1, True)),     # the headline cell's eighth (N-split over 8 GPUs)
    ((1024, 6144, 4096), (False, 128, 1, False)),    # 192 tiles of 256 would leave the second round a third full
    ((2048, 6144, 4096), (False, 256, 1, True)),     # 192 pair tiles: 3 rounds on 74 pairs against 3 on 148 CTAs
    ((1024, 4096, 4096), (False, 256, 1, False)),    # 128 tiles fit one round; the pair kernel would need two
    ((128, 28672, 4096), (False, 256, 1, False)),    # odd number of 128-row blocks: no pairs
    ((128, 4096, 4096), (True, 64, 3, False)),       # 65..128 rows: two 64-row token tiles per weight panel
    ((65, 4096, 4096), (True, 64, 3, False)),
    ((128, 6144, 4096), (True, 64, 2, False)),
    ((129, 4096, 4096), (False, 128, 2, False)),     # first M in the normal orientation on a small weight
    ((64, 4096, 4096), (True, 64, 4, False)),
    ((32, 6144, 4096), (True, 32, 4, False)),
    ((16, 28672, 4096), (True, 16, 1, False)),       # 224 weight panels: enough CTAs without slicing K
    ((16, 4096, 14336), (True, 16, 4, False)),
    ((1, 4096, 4096), (True, 16, 4, False)),
]


@pytest.mark.parametrize("shape,want", DENSE_ROUTES)
def test_dense_route_is_a_function_of_the_shape(shape, want, monkeypatch):
    from fish_scales_ops_b200 import _ops

    got = _ops.gemm_describe(*shape, 148)
    assert (got["swapped"], got["tile_n"], got["k_slices"], got["pair_kernel"]) == want
    m, n, k = shape
    assert got["k_slices"] * got["k_blocks_per_slice"] >= k // 128
    assert (got["k_slices"] - 1) * got["k_blocks_per_slice"] < k // 128          # no empty slice
    if not got["swapped"]:
        rows = 256 if got["pair_kernel"] else 128
        assert got["tiles"] == -(-m // rows) * -(-n // got["tile_n"])
    else:
        assert got["tiles"] == (n // 128) * -(-m // got["tile_n"])


def test_dense_route_refuses_bad_shapes():
    from fish_scales_ops_b200 import _ops

    with pytest.raises(Exception):
        _ops.gemm_describe(128, 100, 4096, 148)
    with pytest.raises(Exception):
        _ops.gemm_describe(128, 4096, 4096, -1)
    assert _ops.gemm_describe(0, 4096, 4096, 148)["tiles"] == 0


def test_host_buffers_are_pinned_next_to_the_gpu(tmp_path, monkeypatch):
    """bench.py narrows the process affinity to the GPU's local CPUs while it allocates the pinned buffers of the
    end-to-end leg, and puts the old affinity back."""
    import os
    import types

    import bench

    assert bench.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    props = types.SimpleNamespace(pci_domain_id=0, pci_bus_id=0x1B, pci_device_id=0)
    fake = types.SimpleNamespace(cuda=types.SimpleNamespace(get_device_properties=lambda i: props))
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    calls = []
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: {0, 1, 2, 3, 4, 5, 6, 7})
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: calls.append(set(cpus)))
    (dev / "local_cpulist").write_text("4-7,12-15\n")
    near = bench.NearGpu(fake, 0, sysfs=str(tmp_path))
    with near:
        assert calls == [{4, 5, 6, 7}]
    assert calls == [{4, 5, 6, 7}, {0, 1, 2, 3, 4, 5, 6, 7}] and "NUMA node" in near.note
    calls.clear()
    (dev / "local_cpulist").write_text("0-63\n")                  # one node: nothing to narrow
    with bench.NearGpu(fake, 0, sysfs=str(tmp_path)):
        pass
    assert calls == []
    with bench.NearGpu(fake, 0, sysfs=str(tmp_path / "missing")) as none:      # no sysfs entry: nothing changes
        pass
    assert calls == [] and "no NUMA information" in none.note
