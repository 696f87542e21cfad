"""deepgemm_b200 -- B200-native (sm_100a) W8A8 channelwise Mega MoE layer.

`deepgemm_b200.megamoe` mirrors the `megamoe` package of yuguo-Jack/DeepGEMM; the top-level `megamoe`
package of this repository re-exports it so existing callers keep their import line.
"""
from . import _lib  # noqa: F401

__all__ = ["megamoe"]
__version__ = "0.1"


def __getattr__(name):
    if name == "megamoe":
        import importlib
        return importlib.import_module(".megamoe", __name__)
    raise AttributeError(name)
