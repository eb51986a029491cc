"""Architecture probe shared by the dense and MoE modules (python/fish_scales_ops/_arch.py and
python/fish_scales_ops/moe/__init__.py:79-97 of the reference): device 0 decides, resolved once."""
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


def arch_major(arch) -> int:
    """The compute-capability major of an ``arch`` argument: an int major (9, 10, 12), an int
    ``major * 10 + minor`` (90, 100, 103, 120, 121), a ``(major, minor)`` pair, or a string such as ``"sm_90"``,
    ``"sm_100a"``, ``"120"`` or ``"12.0"`` (the forms python/fish_scales_ops/moe/__init__.py:129-156 of the
    reference takes). Anything that names no compute capability raises ValueError."""
    if isinstance(arch, bool):
        raise ValueError(f"arch must name a compute capability, got {arch!r}")
    if isinstance(arch, (tuple, list)) and len(arch) == 2 and all(isinstance(v, int) for v in arch):
        return int(arch[0])
    if isinstance(arch, str):
        s = arch.strip().lower()
        if s.startswith("sm_"):
            s = s[3:]
        elif s.startswith("sm"):
            s = s[2:]
        if "." in s:
            head = s.split(".", 1)[0]
            if head.isdigit():
                return int(head)
        s = s.rstrip("af")
        if not s.isdigit():
            raise ValueError(f"arch {arch!r} does not name a compute capability (e.g. 'sm_90', 'sm_120')")
        arch = int(s)
    if isinstance(arch, int):
        if 0 < arch < 20:
            return arch
        if 20 <= arch < 1000:
            return arch // 10
    raise ValueError(f"arch {arch!r} does not name a compute capability (e.g. 'sm_90', 'sm_120')")


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
