"""B200-native FlashMHF multi-head FFN operator (forward + backward) behind the reference's
``flash_mlp(Q, K, U, V, R)`` call.  CUDA only; importing works without a GPU, calling does not."""
import os
import sys

from .functional import FlashMHFFunction, backward_raw, check_device_status, flash_mhf, forward_raw  # noqa: F401

from .layer import expert_views, fused_prologue, mhffn_layer  # noqa: F401,E402

__all__ = ["flash_mhf", "FlashMHFFunction", "forward_raw", "backward_raw", "check_device_status", "install_reference_seam",
           "fused_prologue", "mhffn_layer", "expert_views"]


def install_reference_seam():
    """Make ``from ops.flash_mlp_moe import FlashMLPMoE`` and ``from flash_ffn_moe_torch import FlashFFNMoE``
    resolve to this package -- the two imports the reference layer tries when it is built with
    use_flash=True (models/flashmhf/modeling_mhffnmoe.py:303, 326)."""
    seam = os.path.join(os.path.dirname(os.path.abspath(__file__)), "seam")
    if seam not in sys.path:
        sys.path.insert(0, seam)
    return seam
