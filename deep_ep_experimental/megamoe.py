"""``deep_ep_experimental.megamoe``: the fused-MoE API and its tooling under the reference's import name."""
from deepep_b200.models.mega_moe import *  # noqa: F401,F403
from deepep_b200.models.mega_moe import __all__ as _api
from deepep_b200.models.mega_tools import *  # noqa: F401,F403
from deepep_b200.models.mega_tools import __all__ as _tools

from deepep_b200.parallel.store import StoreGroup  # noqa: E402  (the reference exports it from here for store-only jobs)

__all__ = list(_api) + list(_tools) + ["StoreGroup"]
