"""pyraquant_b200: the INT8 deployment hot path of PyraQuant (deploy/int8_exec.py plus the routed
executor's token gather/scatter) as hand-written sm_100a CUDA behind the reference's Python API.

    from pyraquant_b200 import int8_exec      # drop-in for the reference's deploy/int8_exec.py
    from pyraquant_b200 import routing        # gather / scatter plans and operators

The CUDA library (libpq_b200.so, built by ``python -m pyraquant_b200.build``) is loaded on first use;
without it every operator raises -- there is no CPU fallback.
"""
from . import _lib, ops, int8_exec, routing  # noqa: F401

__all__ = ["int8_exec", "routing", "ops"]
__version__ = "0.1.0"
