"""B200 (sm_100a) decode engine for Llama-family GGUF K-quant models: Python front end over the
C ABI in include/b200llama.h. The directory name contains a dot, so load the package with
importlib (see __graft_entry__.load_package) under the module name `tinyllama_cpp_b200`."""
from . import _build, api, gguf, synth  # noqa: F401
from .api import KV_F32, KV_I8, B200Error, Engine  # noqa: F401
