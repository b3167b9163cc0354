"""B200 (sm_100a) provider for quantum-llm's MTP-4 speculative decode step.

The package is a thin Python mirror of the reference's provider interface over
the C-ABI library built from csrc/.  It has no CPU path: importing `lib` without
the compiled library, or calling it without a CUDA device, raises.
"""
from .lib import load, QllmError  # noqa: F401
from .provider import Nvfp4MtpProvider, RequestParameters, ExactDecodeResult  # noqa: F401
