"""CPU: the C-ABI library builds, loads, and exports every function include/flashmhf.h declares;
host-side argument checks raise before anything touches a device."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "flashmhf.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(flashmhf_[a-z0-9_]+)\s*\(", src)))


def test_header_functions_are_exported(lib):
    names = _declared_functions()
    assert "flashmhf_forward" in names and "flashmhf_backward" in names
    for n in names:
        assert hasattr(lib, n), n


def test_loader_lists_every_declared_function():
    from flashmhf_b200 import _lib
    assert sorted(_lib.EXPORTS) == _declared_functions()


def test_abi_version_and_strerror(lib):
    assert lib.flashmhf_abi_version() == 3
    assert lib.flashmhf_strerror(0) == b"ok"
    for code in range(-11, 0):
        assert len(lib.flashmhf_strerror(code)) > 3


def test_struct_layout_matches_header():
    """sizeof of the ctypes mirrors equals what the C compiler lays out (8 int32 + tensors of 4 x 8 bytes)."""
    from flashmhf_b200 import _lib
    assert C.sizeof(_lib.Dims) == 32 and C.sizeof(_lib.Tensor) == 32
    assert C.sizeof(_lib.Scaling) == 12
    assert C.sizeof(_lib.FwdParams) == 32 + 6 * 32 + 16 + 12 + 4     # three floats, padded to the struct's 8-byte alignment
    assert C.sizeof(_lib.BwdParams) == 32 + 11 * 32 + 16 + 12 + 4    # three floats and the 32-bit parts mask


def test_null_and_shape_errors_without_device(lib):
    from flashmhf_b200 import _lib
    assert lib.flashmhf_forward(None, None) == -1
    assert lib.flashmhf_backward(None, None) == -1
    one = _lib.Scaling(1.0, 1.0, 1.0)
    p = _lib.FwdParams(_lib.Dims(1, 2, 64, 80, 2, 1, 64, 0))   # d_h = 80 unsupported
    assert lib.flashmhf_forward(C.byref(p), None) == -2
    p = _lib.FwdParams(_lib.Dims(1, 2, 64, 64, 2, 1, 48, 0))   # d_e % 64 != 0
    assert lib.flashmhf_forward(C.byref(p), None) == -2
    p = _lib.FwdParams(_lib.Dims(1, 3, 64, 64, 2, 1, 64, 0))   # H % H_kuv != 0
    assert lib.flashmhf_forward(C.byref(p), None) == -2
    p = _lib.FwdParams(_lib.Dims(1, 2, 64, 64, 2, 1, 64, 7))   # dtype
    assert lib.flashmhf_forward(C.byref(p), None) == -3
    p = _lib.FwdParams(_lib.Dims(1, 2, 64, 64, 2, 1, 64, 0))   # scaling constants left at zero
    assert lib.flashmhf_forward(C.byref(p), None) == -2
    p = _lib.FwdParams(_lib.Dims(1, 2, 64, 64, 2, 1, 64, 0), scale=one)   # pointers NULL
    assert lib.flashmhf_forward(C.byref(p), None) == -1
    q = _lib.BwdParams(_lib.Dims(1, 2, 64, 64, 2, 1, 64, 0), scale=one, parts=4)   # unknown bit in the parts mask
    assert lib.flashmhf_backward(C.byref(q), None) == -2
    assert lib.flashmhf_selftest_bounded_wait(0, None) == -2   # limit out of range, checked before any device call


def test_workspace_bytes_is_pure_arithmetic(lib):
    from flashmhf_b200 import _lib
    d = _lib.Dims(16, 8, 2048, 128, 8, 11, 256, 0)
    n = lib.flashmhf_backward_workspace_bytes(C.byref(d))
    per_split = 3 * 8 * 11 * 256 * 128 * 4
    assert n % per_split == 0 and 1 <= n // per_split <= 16
    d.dtype = 1
    assert lib.flashmhf_backward_workspace_bytes(C.byref(d)) == 0


def test_forward_workspace_only_for_short_token_counts(lib):
    from flashmhf_b200 import _lib
    big = _lib.Dims(16, 8, 2048, 128, 8, 11, 256, 0)       # 2048 tiles: no split, no scratch
    assert lib.flashmhf_forward_workspace_bytes(C.byref(big)) == 0
    dec = _lib.Dims(1, 16, 64, 128, 16, 22, 256, 0)        # 1.3B decode: 16 tiles -> intermediate dimension split
    n = lib.flashmhf_forward_workspace_bytes(C.byref(dec))
    per_split = 1 * 16 * 64 * 128 * 4
    assert n % per_split == 0 and 2 <= n // per_split <= 88


def test_python_wrapper_rejects_bad_arguments_on_cpu():
    import flashmhf_b200 as fm
    Q = torch.zeros(1, 2, 64, 64, dtype=torch.bfloat16)
    K = torch.zeros(2, 1, 64, 64, dtype=torch.bfloat16)
    R = torch.ones(1, 2, 64, 1)
    with pytest.raises(ValueError):          # CPU tensors: there is no CPU path
        fm.forward_raw(Q, K, K, K, R)
    with pytest.raises(TypeError):
        fm.forward_raw(Q.half(), K, K, K, R)
    with pytest.raises(ValueError):
        fm.forward_raw(Q, K[:, :, :32], K[:, :, :32], K[:, :, :32], R)


def test_reference_seam_modules_import():
    import flashmhf_b200
    flashmhf_b200.install_reference_seam()
    from ops.flash_mlp_moe import FlashMLPFunction, FlashMLPMoE
    from ops.flash_mlp import FlashMLP
    from flash_ffn_moe_torch import FlashFFNMoE, FlashFFNMoEFunction
    assert issubclass(FlashMLPFunction, torch.autograd.Function) and FlashFFNMoEFunction is FlashMLPFunction
    for cls in (FlashMLPMoE, FlashMLP, FlashFFNMoE):
        assert isinstance(cls(), torch.nn.Module) and not list(cls().parameters())


def test_unmodified_reference_layer_picks_up_the_seam_module():
    """The reference layer's constructor does `from ops.flash_mlp_moe import FlashMLPMoE` after appending a directory to
    sys.path (models/flashmhf/modeling_mhffnmoe.py:318-329).  With this package's seam installed first, that import must
    resolve to this package's module.  Needs a checkout of the reference; skipped where there is none."""
    import flashmhf_b200
    from tests.golden.make_golden import load_reference
    from tests.golden_util import find_reference_checkout
    ref_root = find_reference_checkout()
    if ref_root is None:
        pytest.skip("no reference checkout on this machine")
    seam = flashmhf_b200.install_reference_seam()
    C_, M = load_reference(ref_root)
    cfg = C_.MHFFNMoEConfig(hidden_size=128, intermediate_size=128, num_attention_heads=2, mhffnmoe_num_heads=2,
                            mhffnmoe_num_kuv_heads=2, mhffnmoe_num_experts=2, mhffnmoe_use_flash=True,
                            mhffnmoe_custom_init=True, rms_norm_eps=1e-5)
    layer = M.MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=True)
    assert layer.flash is True
    mod = __import__("sys").modules[type(layer.flash_mlp).__module__]
    assert type(layer.flash_mlp).__module__ == "ops.flash_mlp_moe" and mod.__file__.startswith(seam)
    cfg.mhffnmoe_use_legacy_flash = True
    legacy = M.MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=True)
    assert type(legacy.flash_mlp).__module__ == "ops.flash_mlp" and legacy.flash is True
