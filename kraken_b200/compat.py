"""Drop-in aliasing: ``install_alias()`` registers this package under the name ``kraken`` so code
written against the reference (``import kraken``, ``kraken.comm.one_shot_all_reduce`` ...) runs
unchanged. Not done automatically, so that a real ``kraken`` install is never shadowed by surprise."""
from __future__ import annotations

import sys


def install_alias(name: str = "kraken") -> None:
    import kraken_b200

    if name in sys.modules and sys.modules[name] is not kraken_b200:
        raise RuntimeError(f"a different module named {name!r} is already imported")
    sys.modules[name] = kraken_b200
    for sub in ("comm", "fused", "_ptx_utils", "_logging"):
        sys.modules[f"{name}.{sub}"] = getattr(kraken_b200, sub)
