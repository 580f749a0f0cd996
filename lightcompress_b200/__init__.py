"""B200-native kernels for LightCompress's calibration-time quantization hot path.

Host-side mirrors of the reference plugin interface (`IntegerQuantizer`, `FloatQuantizer`,
`GPTQ`, `RTN`) over a C-ABI library of hand-written sm_100a CUDA kernels.
"""
from . import _lib  # noqa: F401  (raises if the CUDA library is not built)
from .quant import FloatQuantizer, IntegerQuantizer, Weight48IntegerQuantizer  # noqa: F401
from .gptq import GPTQ  # noqa: F401
from .spqr import SpQR  # noqa: F401
from .rtn import RTN  # noqa: F401
from .awq import Awq  # noqa: F401
from .blockwise import GPTQBlockwise, FakeQuantLinear, llama_subsets  # noqa: F401
from .streaming import HostStagedGPTQ  # noqa: F401

__all__ = ['IntegerQuantizer', 'FloatQuantizer', 'Weight48IntegerQuantizer', 'GPTQ', 'SpQR', 'RTN', 'Awq', 'GPTQBlockwise', 'FakeQuantLinear', 'llama_subsets', 'HostStagedGPTQ']
