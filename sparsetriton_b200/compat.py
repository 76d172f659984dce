"""Expose this package under the reference's import name.

    import sparsetriton_b200.compat as compat; compat.install()
    from sparsetriton import SparseTensor            # now this package
    from sparsetriton.nn.functional.conv.funcs import ConvHashOnTheFlyImplicitGEMM

Every already-imported `sparsetriton_b200[.x.y]` module is registered as `sparsetriton[.x.y]`
in sys.modules, so the reference's own test-suite can run unchanged against this code.
"""
import importlib
import pkgutil
import sys

_PREFIX = "sparsetriton_b200"
_ALIAS = "sparsetriton"


def install():
    if _ALIAS in sys.modules and not getattr(sys.modules[_ALIAS], "__name__", "").startswith(_PREFIX):
        raise RuntimeError("a different 'sparsetriton' package is already imported")
    root = importlib.import_module(_PREFIX)
    for info in pkgutil.walk_packages(root.__path__, prefix=_PREFIX + "."):
        if info.name.endswith(".build"):
            continue
        importlib.import_module(info.name)
    for name, module in list(sys.modules.items()):
        if name == _PREFIX or name.startswith(_PREFIX + "."):
            sys.modules[_ALIAS + name[len(_PREFIX):]] = module
    return sys.modules[_ALIAS]
