"""Drop-in for the reference's kernels/thunderkittens/flash_ffn_moe_torch.py module surface."""
import torch

from flashmhf_b200.functional import FlashMHFFunction as FlashFFNMoEFunction  # noqa: F401


class FlashFFNMoE(torch.nn.Module):
    def forward(self, Q, K, U, V, R):
        return FlashFFNMoEFunction.apply(Q, K, U, V, R)
