"""Drop-in import names of the reference's experimental packages.

``deep_ep_experimental.megamoe`` re-exports :mod:`deepep_b200.models.mega_moe` (fused MoE, plus its tooling) and
``deep_ep_experimental.ep_gmm_fused`` re-exports :mod:`deepep_b200.ops.ep_gmm_fused` (all-to-all-v + grouped matmul),
so code written against ``experiments/megamoe`` and ``experiments/ep_gmm_fused`` of the reference keeps its imports.
"""
