"""ComfyUI custom-node entry point: ComfyUI imports every directory under `custom_nodes/` and reads the two mappings.

The directory name is not an identifier, so ComfyUI loads this file under a synthetic module name; `fa_b200` is then
imported from beside this file, and a `fa_b200` that some other location already supplied is refused instead of being
mixed with this one (the reference's loader, __init__.py:1-27, has the same rule for its package).
"""
import os
import sys

_here = os.path.dirname(os.path.abspath(__file__))


def _load_mappings():
    already = sys.modules.get("fa_b200")
    if already is not None:
        origin = os.path.abspath(getattr(already, "__file__", "") or "")
        if os.path.commonpath([_here, origin or os.sep]) != _here:
            raise RuntimeError("A different fa_b200 package is already loaded; restart ComfyUI before loading this "
                               "custom node")
    sys.path.insert(0, _here)
    try:
        from fa_b200 import comfyui
    finally:
        sys.path.remove(_here)
    return comfyui.NODE_CLASS_MAPPINGS, comfyui.NODE_DISPLAY_NAME_MAPPINGS


NODE_CLASS_MAPPINGS, NODE_DISPLAY_NAME_MAPPINGS = _load_mappings()

__all__ = ["NODE_CLASS_MAPPINGS", "NODE_DISPLAY_NAME_MAPPINGS"]
