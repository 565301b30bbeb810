"""Import seam: the reference layer does ``from ops.flash_mlp_moe import FlashMLPMoE``
(models/flashmhf/modeling_mhffnmoe.py:320-327) after appending a directory to sys.path."""
