"""B200 (sm_100a) backend for the quantized indexed MoE path of the "laguna" engine.

``ops``  -- host mirror of the reference's ``src/ops`` dispatch functions;
``moe``  -- ``MoeBlock`` / ``FusedExperts`` / ``SharedExpert`` (src/moe.rs);
``gguf`` -- ``ExpertStack`` (src/gguf.rs:247-276).
Everything computes through ``liblmoe.so`` (hand-written CUDA behind the C ABI
of ``include/lmoe.h``); there is no CPU fallback.
"""
from . import build  # noqa: F401
from ._native import LmoeError, lib, lib_path  # noqa: F401
