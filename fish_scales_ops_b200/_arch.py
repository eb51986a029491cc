"""Architecture probe shared by the dense and MoE modules (python/fish_scales_ops/_arch.py and
python/fish_scales_ops/moe/__init__.py:79-97 of the reference): device 0 decides, resolved once."""
import re

import torch

_arch_cache = -1


def device_arch() -> int:
    """Compute capability of device 0 as ``major * 10 + minor`` (100 on a B200), 0 without a CUDA device."""
    global _arch_cache
    if _arch_cache < 0:
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability(0)
            _arch_cache = major * 10 + minor
        else:
            _arch_cache = 0
    return _arch_cache


def sm_major() -> int:
    return device_arch() // 10


def arch_label(arch: int) -> str:
    return f"sm_{arch}" if arch > 0 else "no CUDA device"


_ARCH_TEXT = re.compile(r"^(?:sm_?)?(\d+)(?:\.(\d+))?[af]?$")


def _major_of_number(n: int):
    """9, 10, 12 are majors as they stand; 90, 100, 103, 120, 121 carry the minor in the last digit."""
    if 0 < n < 20:
        return n
    if 20 <= n < 1000:
        return n // 10
    return None


def arch_major(arch) -> int:
    """Compute-capability major named by ``arch``. Accepted spellings, after the ``arch`` argument of
    python/fish_scales_ops/moe/__init__.py:129-156 of the reference: a major (10), ``major * 10 + minor`` (100, 103),
    a ``(major, minor)`` pair, and the text forms ``"sm_100"``, ``"sm100a"``, ``"100"``, ``"10.0"``. ValueError for
    anything else (booleans included)."""
    major = None
    if isinstance(arch, str):
        m = _ARCH_TEXT.match(arch.strip().lower())
        if m is not None:
            major = int(m.group(1)) if m.group(2) is not None else _major_of_number(int(m.group(1)))
    elif isinstance(arch, (tuple, list)):
        if len(arch) == 2 and all(isinstance(v, int) and not isinstance(v, bool) for v in arch):
            major = int(arch[0])
    elif isinstance(arch, int) and not isinstance(arch, bool):
        major = _major_of_number(arch)
    if major is None:
        raise ValueError(f"arch = {arch!r} is not a compute capability; write it like 'sm_100', 100, 10 or (10, 0)")
    return major


def env_flag(name: str, default: bool = False) -> bool:
    """A boolean ``FSO_*`` switch: unset or empty gives ``default``, a value starting with ``0`` is off, anything
    else is on (python/fish_scales_ops/_env.py:18-31 of the reference)."""
    import os

    value = os.environ.get(name)
    if not value:
        return default
    return value[0] != "0"


# This build serves one architecture family.
SERVED_MAJOR = 10
