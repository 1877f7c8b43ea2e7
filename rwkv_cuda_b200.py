"""Import alias: the package lives in the directory ``rwkv-cuda_b200/`` (not a valid Python
identifier); this module turns itself into that package so it imports as ``rwkv_cuda_b200``."""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "rwkv-cuda_b200")]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__) as _f:
    exec(compile(_f.read(), __file__, "exec"))
