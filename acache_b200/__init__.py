"""B200-native affix-KV reuse for block-wise diffusion-LLM serving.

Host side: ``Sequence``, ``BlockManager``, ``Scheduler``, ``Config``,
``ModelRunner`` with the reference engine's interface.  Device side: hand-written
sm_100a CUDA kernels behind the C ABI declared in ``include/acache_b200.h``
(loaded by ``acache_b200._lib``); there is no CPU fallback.
"""
from .block_manager import BlockManager
from .config import Config
from .scheduler import Scheduler
from .sequence import Sequence, SequenceStatus
from .utils import Context, get_context, reset_context, set_context

__all__ = [
    "BlockManager",
    "Config",
    "Scheduler",
    "Sequence",
    "SequenceStatus",
    "Context",
    "get_context",
    "set_context",
    "reset_context",
]
