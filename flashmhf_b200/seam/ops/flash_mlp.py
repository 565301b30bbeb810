"""Drop-in for the reference's legacy module kernels/triton/flash_mlp.py (``FlashMLP``): one gated
FFN per head with no sub-networks and no routing weight, which is the operator with E = 1, R = 1."""
import torch

from flashmhf_b200.functional import flash_mhf


class FlashMLP(torch.nn.Module):
    """forward(Q [B,H,S,d_h], K/U/V [H_kuv,I,d_h], apply_dot_scaling, head_scaling, up_scaling, activation_fn)."""

    def forward(self, Q, K, U, V, apply_dot_scaling=False, head_scaling=1.0, up_scaling=1.0, activation_fn="silu"):
        if activation_fn != "silu":
            raise ValueError("FlashMLP currently supports only SiLU activation")
        # The reference's legacy module rejects dot scaling (kernels/triton/flash_mlp.py:1056-1057); its eager layer
        # applies it (models/flashmhf/modeling_mhffnmoe.py:420-422).  Here the operator takes the two constants, so the
        # legacy flash branch gives what the eager branch gives; final_scaling stays with the caller (modeling:403).
        if U is None:
            raise ValueError("FlashMLP SiLU variant requires up-projection tensor U (got None)")
        B, H, S, _ = Q.shape
        R = torch.ones(B, H, S, 1, dtype=torch.float32, device=Q.device)
        return flash_mhf(Q, K.unsqueeze(1), U.unsqueeze(1), V.unsqueeze(1), R, float(head_scaling), float(up_scaling), 1.0)
