"""Drop-in for the reference's kernels/triton/flash_mlp_moe.py module surface: ``FlashMLPFunction``
(autograd Function, forward(ctx,Q,K,U,V,R)) and ``FlashMLPMoE`` (argument-less nn.Module)."""
import torch

from flashmhf_b200.functional import FlashMHFFunction as FlashMLPFunction  # noqa: F401


class FlashMLPMoE(torch.nn.Module):
    """forward(Q [B,H,S,d_h], K/U/V [H_kuv,E,d_e,d_h], R [B,H,S,E]) -> O [B,H,S,d_h]."""

    def forward(self, Q, K, U, V, R):
        return FlashMLPFunction.apply(Q, K, U, V, R)
