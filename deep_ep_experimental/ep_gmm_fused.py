"""``deep_ep_experimental.ep_gmm_fused``: all-to-all-v + grouped matmul under the reference's import name."""
from deepep_b200.ops.ep_gmm_fused import *  # noqa: F401,F403
from deepep_b200.ops.ep_gmm_fused import __all__  # noqa: F401
