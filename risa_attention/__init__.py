"""Import-name alias: ``import risa_attention`` resolves to the B200-native package
``risaattention_b200`` (same public names as the reference project's package of this name, which
must not be installed beside this alias)."""
import importlib
import sys

import risaattention_b200 as _impl
from risaattention_b200 import *  # noqa: F401,F403

__all__ = list(_impl.__all__)
__version__ = _impl.__version__

for _name in ("attention", "dense", "sparse", "reference", "permutation", "_backend", "_execution",
              "_quantization", "_types", "_validation", "_key_mask"):
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"risaattention_b200.{_name}")
if _impl._backend._C is not None:
    sys.modules[f"{__name__}._C"] = _impl._backend._C
