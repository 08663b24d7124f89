"""B200-native quantised decode path for aarambh-studio (host-side mirrors).

Every operator here calls the C ABI of ``libaarambh_b200.so``; importing the
package without the built library fails (no CPU or PyTorch fallback exists).
"""
from ._lib import Ab2Error, check, lib  # noqa: F401
from .qlinear import QuantLinear  # noqa: F401
