"""B200-native quantised decode path for aarambh-studio (host-side mirrors).

Every operator here calls the C ABI of ``libaarambh_b200.so``; importing the
package without the built library fails (no CPU or PyTorch fallback exists).
"""
from ._lib import Ab2Error, check, device_status, lib  # noqa: F401
from .qlinear import QuantLinear  # noqa: F401
from .kvcache import KVCache  # noqa: F401
from . import dispatch  # noqa: F401
from .model import AarambhModel, InferenceEngine, ModelConfig  # noqa: F401
from . import parallel  # noqa: F401
from .parallel import TensorParallel  # noqa: F401
from . import gguf  # noqa: F401
from . import sessions  # noqa: F401
