"""mplayers_b200: B200-native (sm_100a) TRWP / ISGMR min-sum message-passing layers behind the
operator API of zwxu064/MPLayers (`MPModule`, `TRWPFunction`, `ISGMRFunction`)."""
from .MP_module import ISGMRFunction, MPModule, TRWPFunction  # noqa: F401
from ._lib import kernel_launches  # noqa: F401

__all__ = ["MPModule", "TRWPFunction", "ISGMRFunction", "kernel_launches"]
