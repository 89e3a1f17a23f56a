"""recsdk_b200: B200-native (sm_100a) sparse-embedding hot path behind RecSDK's operator API.

Importing the package loads ``librecsdk_b200.so`` (the C ABI of include/recsdk_b200.h).
There is no CPU or pure-PyTorch fallback: a missing library is an ImportError.
"""
from . import _lib

_lib.load()

from . import ops  # noqa: E402
from .embcache import AdmitAndEvictConfig, EmbcacheManager, EmbConfig, SwapInfo  # noqa: E402
from .tables import FeatureFilter, IdsMapper, SwapManager  # noqa: E402

__all__ = ["ops", "IdsMapper", "SwapManager", "FeatureFilter", "EmbcacheManager", "EmbConfig", "AdmitAndEvictConfig",
           "SwapInfo"]
