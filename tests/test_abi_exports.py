"""The C-ABI library loads and exports every symbol include/msk.h declares (no GPU needed)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "msk.h")).read()
    return sorted(set(re.findall(r"^int\s+(msk_\w+)\s*\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol():
    from muse_spark_open_b200 import abi, build
    build.build()
    lib = abi.lib()
    names = _declared()
    assert "msk_proj_skinny" in names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/msk.h but not exported"
    assert sorted(abi.EXPORTS) == names
    assert lib.msk_version() >= 100


def test_no_cpu_fallback():
    import torch
    from muse_spark_open_b200 import abi, proj
    with pytest.raises(abi.MskError):
        proj.prepare({"w": torch.zeros(128, 64, dtype=torch.bfloat16)})
