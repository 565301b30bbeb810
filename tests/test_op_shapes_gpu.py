"""GPU: the bf16 operator on a seeded list of irregular shapes (token counts around tile and split boundaries, every
supported head dim, shared K/U/V heads, odd sub-network counts), forward and backward against the oracle."""
import random

import pytest
import torch

from oracle import mhffn_oracle as orc

pytestmark = pytest.mark.gpu


def _shapes(n=36, seed=2024):
    rng = random.Random(seed)
    edge_S = [1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, 383, 500, 640, 777]
    out = []
    for _ in range(n):
        dh = rng.choice([64, 96, 128])
        G = rng.choice([1, 1, 2, 3])
        Hk = rng.choice([1, 2, 3])
        out.append((rng.choice([1, 1, 2, 3]), Hk * G, Hk, rng.choice(edge_S), dh, rng.choice([1, 2, 3, 5]), rng.choice([64, 128, 192])))
    return out


@pytest.mark.parametrize("shape", _shapes())
def test_irregular_shape_forward_backward(shape):
    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=hash(shape) % 1000, dtype=torch.bfloat16)
    d = [t.cuda() for t in (Q, K, U, V, R, dO)]
    O = fm.forward_raw(*d[:5]).cpu().float()
    got = [g.cpu().float() for g in fm.backward_raw(*d)]
    _lib.device_status()
    f = [t.float() for t in (Q, K, U, V)]
    assert orc.rel_l2(O, orc.mhffn_forward(*f, R)) < 1e-2
    ref = orc.mhffn_backward(*(t.double() for t in f), R.double(), dO.double())
    for name, a, b in zip("dQ dK dU dV dR".split(), got, ref):
        assert orc.rel_l2(a, b) < 1e-2, (name, shape)
