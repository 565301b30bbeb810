"""Helpers shared by the tests: read the committed fixtures and rebuild seed-derived parameters."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REPO_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def find_reference_checkout():
    """A checkout of the reference project on this machine, or None: the FLASHMHF_REFERENCE environment variable, an
    install under baseline/_ref, or the `reference_path` the repository's BASELINE.json names."""
    import json
    cands = [os.environ.get("FLASHMHF_REFERENCE", ""), os.path.join(REPO_ROOT, "baseline", "_ref")]
    try:
        with open(os.path.join(REPO_ROOT, "BASELINE.json")) as f:
            cands.append(json.load(f).get("reference_path", ""))
    except (OSError, ValueError):
        pass
    for c in cands:
        if c and os.path.exists(os.path.join(c, "models", "flashmhf", "modeling_mhffnmoe.py")):
            return c
    return None


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: torch.from_numpy(z[k]) for k in z.files}
    hidden, inter, H, Hkuv, E, B, S, rms, seed, skip = (int(v) for v in d.pop("meta"))
    scaling = tuple(float(v) for v in d.pop("scaling")) if "scaling" in d else (1.0, 1.0, 1.0)
    d["cfg"] = dict(hidden=hidden, inter=inter, H=H, Hkuv=Hkuv, E=E, B=B, S=S, rmsnorm=bool(rms), seed=seed,
                    skip_linear=bool(skip), dh=hidden // H, scaling=scaling)
    if "x" not in d:   # full-size cases: the input and the loss weights are regenerated from the seed
        g = torch.Generator().manual_seed(seed + 1000)
        d["x"] = torch.randn(B, S, hidden, generator=g)
        d["wloss"] = torch.randn(B, S, hidden, generator=g)
    return d


def seeded_layer_params(cfg, std=0.02):
    """Same draw order as tests/golden/make_golden.py:seeded_params (parameter names sorted)."""
    hid, inter, H, Hkuv, E, dh = cfg["hidden"], cfg["inter"], cfg["H"], cfg["Hkuv"], cfg["E"], cfg["dh"]
    shapes = {"down_weight": (inter, Hkuv * dh), "gate_weight": (inter, Hkuv * dh), "q_norm.weight": (H, dh),
              "router": (H, dh, E), "up_weight": (inter, Hkuv * dh)}
    if not cfg["skip_linear"]:
        shapes.update({"w_self.weight": (hid, hid), "w_self_2.weight": (hid, hid)})
    g = torch.Generator().manual_seed(cfg["seed"])
    p = {}
    for name in sorted(shapes):
        if name == "q_norm.weight":
            p["q_norm"] = 1.0 + 0.1 * torch.randn(shapes[name], generator=g)
        else:
            p[name.replace(".weight", "")] = torch.randn(shapes[name], generator=g) * std
    return p


def layer_params(d):
    """Parameters of a fixture: stored ones if present, else regenerated from the seed."""
    cfg = d["cfg"]
    if "p_gate_weight" in d:
        p = {k[2:]: v.clone() for k, v in d.items() if k.startswith("p_")}
    else:
        p = seeded_layer_params(cfg)
    if cfg["skip_linear"]:
        eye = torch.eye(cfg["hidden"])
        p["w_self"], p["w_self_2"] = eye, eye.clone()
    return p
