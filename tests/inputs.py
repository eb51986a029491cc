"""Seeded synthetic inputs of the benchmark configurations (generated on the CPU so that the oracle and the GPU see
the same bits). They stand in for real checkpoints and traffic; no dataset is involved."""
import numpy as np
import torch


def gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def activation(m: int, k: int, seed: int) -> torch.Tensor:
    """bf16 [m, k] ~ N(0, 1)."""
    return torch.randn(m, k, generator=gen(seed), dtype=torch.float32).to(torch.bfloat16)


def weight(n: int, k: int, seed: int) -> torch.Tensor:
    """bf16 [n, k] ~ N(0, 0.02)."""
    return (0.02 * torch.randn(n, k, generator=gen(seed), dtype=torch.float32)).to(torch.bfloat16)


def edge_activation() -> torch.Tensor:
    """bf16 [130, 256] covering the quantizer's corner cases: all-zero blocks, values under the amax floor, the
    largest finite bf16, exact powers of two and the 1.75 * 2^e boundary of the scale-byte rule, negative zero,
    non-finite values (a NaN never becomes a block's amax, the reference's fmaxf chain passes over it; an Inf makes
    the amax infinite and the scale byte 254), and a ragged row count (130 is not a multiple of 128, so the padded
    rows' words are exercised)."""
    x = torch.randn(130, 256, generator=gen(1234), dtype=torch.float32)
    x[0] = 0.0
    x[1, :32] = 1e-12
    x[1, 32:64] = -0.0
    x[2, 0] = 3.0e38
    x[2, 40] = -3.3e38
    x[3, :32] = 448.0
    x[3, 32:64] = 449.0
    x[3, 64:96] = 447.0
    x[4, :32] = 2.0 ** -20
    x[4, 32:64] = 1.75 * 2.0 ** -3
    x[4, 64:96] = 1.7578125 * 2.0 ** -3
    x[4, 96:128] = 2.0 ** 10
    x[5] = x[5] * 1e-6
    x[6] = x[6] * 1e6
    x[7, ::2] = 0.0
    x[8, 128:] = 1e-10
    x[9, :] = 9.9e-11
    x[10, 3] = float("nan")                     # one NaN among ordinary values
    x[10, 32:64] = float("nan")                 # a block of NaNs only (amax falls to the floor)
    x[10, 70] = float("nan")
    x[10, 71] = 300.0
    x[11, 0] = float("inf")                     # an Inf among ordinary values
    x[11, 40] = float("-inf")
    x[11, 64:96] = float("inf")
    x[12, 5] = float("nan")                     # NaN and Inf in the same block
    x[12, 6] = float("-inf")
    x[12, 200] = float("nan")
    x[12, 255] = float("inf")
    return x.to(torch.bfloat16)


def block_fp8_checkpoint(n: int, k: int, seed: int):
    """(float8_e4m3fn [n, k], fp32 [n/128, k/128]): values N(0,1) clamped to +-448, scales log-uniform in
    [2^-8, 2^-4] (the block-FP8 checkpoint form of tests/gemm/unit/test_dense.py:108-117 of the reference)."""
    g = gen(seed)
    w = torch.randn(n, k, generator=g, dtype=torch.float32).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
    u = torch.rand(n // 128, k // 128, generator=g, dtype=torch.float32)
    s = torch.exp2(-8.0 + 4.0 * u)
    return w, s


def routing(tokens: int, num_experts: int, topk: int, seed: int, skew: float = 0.0, renorm: bool = True):
    """softmax top-k routing from N(0,1) logits; ``skew`` > 0 adds the log of a Zipf(skew) popularity over a seeded
    expert ranking. Returns (ids int32 [T, k], weights fp32 [T, k])."""
    g = gen(seed)
    logits = torch.randn(tokens, num_experts, generator=g, dtype=torch.float32)
    if skew > 0:
        rank = torch.randperm(num_experts, generator=g).to(torch.float32)
        logits = logits + torch.log((rank + 1.0) ** (-skew))
    p = torch.softmax(logits, dim=-1)
    w, ids = torch.topk(p, topk, dim=-1)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return ids.to(torch.int32), w.to(torch.float32)


def rel_frobenius(a: torch.Tensor, ref: torch.Tensor) -> float:
    a = a.double()
    ref = ref.double()
    return float((a - ref).norm() / ref.norm().clamp_min(1e-30))


def max_abs_over_refmax(a: torch.Tensor, ref: torch.Tensor) -> float:
    a = a.double()
    ref = ref.double()
    return float((a - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


# The tolerance of the bf16 outputs against the fp32 dequantize-then-matmul oracle.
REL_FRO_TOL = 1e-2
ELEM_TOL = 2e-2


def assert_close_to_oracle(out: torch.Tensor, ref_fp32: torch.Tensor, what: str = ""):
    rf = rel_frobenius(out.float().cpu(), ref_fp32)
    me = max_abs_over_refmax(out.float().cpu(), ref_fp32)
    assert rf <= REL_FRO_TOL and me <= ELEM_TOL, f"{what}: rel Frobenius {rf:.3e} (<= {REL_FRO_TOL}), " \
                                                 f"max |err| / max |ref| {me:.3e} (<= {ELEM_TOL})"
    return rf, me


def to_np_u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def to_np_u32(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().numpy().view(np.uint32)


GOLDEN = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)), "golden",
                                    "quantize_1x32.npz")
