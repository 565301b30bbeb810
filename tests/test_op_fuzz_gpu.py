"""GPU: the operator over seeded random shapes, forward and backward, against the oracle (bf16, rel-L2 <= 1e-2), plus the
shapes that steer the weight-gradient kernel's launch plans: a two-way token split with an uneven cut (blocks x 2 close
to a multiple of the SM count, 32 token tiles or more), an odd number of token tiles, and a one-way split."""
import random

import pytest
import torch

from oracle import mhffn_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _random_shapes(n, seed):
    rng = random.Random(seed)
    out = []
    while len(out) < n:
        dh = rng.choice([64, 96, 128])
        G = rng.choice([1, 1, 2, 3])
        Hk = rng.randint(1, 3)
        E = rng.randint(1, 5)
        de = rng.choice([64, 128, 192])
        B = rng.randint(1, 3)
        S = rng.choice([1, 2, 7, 64, 127, 128, 129, 200, 300, 385])
        out.append((B, Hk * G, Hk, S, dh, E, de))
    return out


PLAN_SHAPES = [
    (2, 5, 5, 2048, 128, 7, 128),    # 70 weight blocks: two-way token split, 32 token tiles -> uneven cut
    (1, 5, 5, 4224, 128, 7, 128),    # the same blocks, 33 token tiles (odd)
    (3, 10, 5, 1408, 64, 7, 128),    # shared K/U/V heads: 66 tiles per K/U/V head, d_h = 64
    (1, 4, 4, 1000, 96, 10, 256),    # 160 blocks: one-way split, more than one wave
]


def _check(shape, seed):
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=seed, dtype=torch.bfloat16)
    dev = [t.cuda() for t in (Q, K, U, V, R, dO)]
    O = fm.forward_raw(*dev[:5])
    grads = fm.backward_raw(*dev)
    again = fm.backward_raw(*dev)
    fm.check_device_status()
    f32 = [t.float() for t in (Q, K, U, V, R)]
    assert orc.rel_l2(O.cpu().float(), orc.mhffn_forward(*f32)) < TOL, ("O", shape)
    ref = orc.mhffn_backward(*f32, dO.float())
    for name, a, a2, b in zip("dQ dK dU dV dR".split(), grads, again, ref):
        assert orc.rel_l2(a.cpu().float(), b) < TOL, (name, shape)
        assert torch.equal(a, a2), (name, shape, "not reproducible")


@pytest.mark.parametrize("shape", _random_shapes(24, seed=2024))
def test_random_shapes_forward_backward(shape):
    _check(shape, seed=hash(shape) % 1000)


@pytest.mark.parametrize("shape", PLAN_SHAPES)
def test_shapes_that_steer_the_weight_gradient_plans(shape):
    _check(shape, seed=77)
