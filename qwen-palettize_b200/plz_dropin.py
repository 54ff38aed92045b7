"""Make the reference's own `qwen_model.PalettizedLinear` run on libplz.so, with qwen_model.py and train_qwen.py unchanged.

The reference module picks its kernels when it is CONSTRUCTED (scripts/qwen_model.py:104-130): it first tries
`from triton_soft_forward import ...` / `from triton_hard_forward import ...`, and only if those imports fail does it
`import fused_lut_linear_cuda` and bind `fused_lut_linear` / `fused_lut_linear_soft`.  qwen_model.py also pushes its own
directory to the front of sys.path (:27), so a PYTHONPATH entry cannot outrank the reference's files of those names.
`install()` therefore works on sys.modules, which every `import` consults before sys.path:

    import plz_dropin; plz_dropin.install()      # before the first PalettizedLinear is constructed
    import qwen_model                            # the reference's file, untouched

  * this package's fused_lut_linear_cuda is loaded from its file path and registered under that name;
  * the two Triton module names are mapped to None, which makes their import raise ImportError, so the module falls
    through to the `fused_lut_linear_cuda` branch (this library ships no Triton path and no CPU path).
`uninstall()` restores the previous entries.
"""
from __future__ import annotations

import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_NAMES = ("fused_lut_linear_cuda", "triton_soft_forward", "triton_hard_forward")
_saved: dict = {}
_MISSING = object()


def _load_ours():
    mod = sys.modules.get("fused_lut_linear_cuda")
    path = os.path.join(_HERE, "fused_lut_linear_cuda.py")
    if mod is not None and os.path.abspath(getattr(mod, "__file__", "") or "") == path:
        return mod
    if _HERE not in sys.path:
        sys.path.insert(0, _HERE)     # its own imports (plz_native, plz_ops) are found by name
    spec = importlib.util.spec_from_file_location("fused_lut_linear_cuda", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["fused_lut_linear_cuda"] = mod
    try:
        spec.loader.exec_module(mod)
    except Exception:
        sys.modules.pop("fused_lut_linear_cuda", None)
        raise
    return mod


def install():
    """Route `import fused_lut_linear_cuda` to this package and make the Triton modules unimportable.
    Returns the installed module.  Raises if libplz.so is missing (there is no other backend to fall back to)."""
    if not _saved:
        for n in _NAMES:
            _saved[n] = sys.modules.get(n, _MISSING)
        _saved["fused_lut_linear_cuda"] = sys.modules.pop("fused_lut_linear_cuda", _MISSING)
    mod = _load_ours()
    mod._get_module()                 # loads libplz.so now, so that a missing library fails here and not inside a forward
    sys.modules["fused_lut_linear_cuda"] = mod
    sys.modules["triton_soft_forward"] = None
    sys.modules["triton_hard_forward"] = None
    return mod


def uninstall():
    for n, v in _saved.items():
        if v is _MISSING:
            sys.modules.pop(n, None)
        else:
            sys.modules[n] = v
    _saved.clear()


def is_bound(module) -> bool:
    """True if a constructed reference PalettizedLinear dispatches to this library."""
    ours = sys.modules.get("fused_lut_linear_cuda")
    return (ours is not None and getattr(module, "_use_cuda", False) and not getattr(module, "_use_triton", False)
            and getattr(module, "_hard_kernel", None) is ours.fused_lut_linear
            and getattr(module, "_soft_kernel", None) is ours.fused_lut_linear_soft)
