"""GPU parity: the CUDA operator (through the C ABI) against the CPU oracle on the same seeded inputs.

Tolerances (relative L2 error): fp32 check mode 1e-5; bf16 tensor-core path 1e-2 against the oracle
evaluated in fp32 on the same bf16-rounded inputs, and 1e-2 against the oracle's bf16 eager evaluation."""
import pytest
import torch

from oracle import mhffn_oracle as orc
from tests.golden_util import load_golden

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_BF16 = 1e-2

# (B, H, Hkuv, S, dh, E, de)
SHAPES_SMALL = [
    (1, 1, 1, 128, 128, 1, 64),
    (2, 2, 2, 200, 128, 2, 128),    # ragged tail (200 = 128 + 72)
    (1, 2, 2, 37, 64, 3, 64),       # shorter than one tile
    (2, 3, 3, 130, 96, 2, 64),      # the 128M model's head dim
    (1, 4, 2, 256, 128, 2, 64),     # shared K/U/V heads (G = 2)
    (1, 2, 1, 150, 96, 1, 192),     # G = 2, d_h = 96, single sub-network
]
SHAPES_MODEL = [
    (1, 8, 8, 512, 96, 8, 256),     # 128M layer dims
    (1, 8, 8, 384, 128, 11, 256),   # 370M layer dims
    (1, 2, 2, 300, 64, 8, 192),     # operator sweep d_h=64 point
    (1, 2, 2, 256, 128, 8, 320),    # operator sweep d_h=128 point
]


def _dev(ts):
    return [t.cuda() for t in ts]


def _oracle_grads(Q, K, U, V, R, dO):
    return orc.mhffn_backward(Q.double(), K.double(), U.double(), V.double(), R.double(), dO.double())


@pytest.fixture(autouse=True)
def _status_clean():
    from flashmhf_b200 import _lib
    yield
    _lib.device_status()  # raises if any kernel gave up on a bounded wait


@pytest.mark.parametrize("shape", SHAPES_SMALL)
def test_check_mode_forward_backward(shape):
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=11, dtype=torch.float32)
    O = fm.forward_raw(*_dev([Q, K, U, V, R])).cpu()
    assert orc.rel_l2(O, orc.mhffn_forward(Q.double(), K.double(), U.double(), V.double(), R.double())) < TOL_F32
    got = [g.cpu() for g in fm.backward_raw(*_dev([Q, K, U, V, R, dO]))]
    for name, a, b in zip("dQ dK dU dV dR".split(), got, _oracle_grads(Q, K, U, V, R, dO)):
        assert orc.rel_l2(a, b) < TOL_F32, name


@pytest.mark.parametrize("shape", SHAPES_SMALL + SHAPES_MODEL)
def test_bf16_forward(shape):
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=12, dtype=torch.bfloat16, with_dO=False)
    O = fm.forward_raw(*_dev([Q, K, U, V, R])).cpu().float()
    ref32 = orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), R)
    assert orc.rel_l2(O, ref32) < TOL_BF16
    assert orc.rel_l2(O, orc.mhffn_forward(Q, K, U, V, R).float()) < TOL_BF16  # the eager path in bf16


@pytest.mark.parametrize("shape", SHAPES_SMALL + SHAPES_MODEL)
def test_bf16_backward(shape):
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=13, dtype=torch.bfloat16)
    got = [g.cpu().float() for g in fm.backward_raw(*_dev([Q, K, U, V, R, dO]))]
    ref = _oracle_grads(Q.float(), K.float(), U.float(), V.float(), R, dO.float())
    for name, a, b in zip("dQ dK dU dV dR".split(), got, ref):
        assert orc.rel_l2(a, b) < TOL_BF16, name


@pytest.mark.parametrize("shape", [(64, 16, 16, 1, 128, 22, 256),   # 1.3B batched decode: 64 sequences, one new token each
                                   (1, 2, 2, 100, 128, 4, 128),     # one short tile, two heads
                                   (3, 1, 1, 1, 96, 3, 64),         # three single-token rows, d_h = 96
                                   (1, 4, 2, 64, 64, 5, 192)])      # shared K/U/V heads
def test_bf16_forward_short_token_counts_split_path(shape):
    """Fewer token tiles than SMs: the intermediate dimension is split over CTAs (fp32 partial outputs,
    fixed-order sum); decode-shaped [B,H,1,d_h] inputs are viewed as one sequence of B tokens."""
    import flashmhf_b200 as fm
    B, H, Hk, S, dh, E, de = shape
    Q, K, U, V, R = orc.make_op_inputs(B, H, S, dh, E, de, Hkuv=Hk, seed=22, dtype=torch.bfloat16, with_dO=False)
    out = torch.full(Q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    O = fm.forward_raw(*_dev([Q, K, U, V, R]), out=out).cpu().float()
    assert torch.isfinite(O).all()
    assert orc.rel_l2(O, orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), R)) < TOL_BF16
    again = fm.forward_raw(*_dev([Q, K, U, V, R])).cpu().float()
    assert torch.equal(O, again)


def test_autograd_function_matches_oracle_autograd():
    import flashmhf_b200 as fm
    Q, K, U, V, R, dO = orc.make_op_inputs(2, 2, 192, 128, 2, 64, seed=14, dtype=torch.bfloat16)
    ins = [t.cuda().requires_grad_(True) for t in (Q, K, U, V, R)]
    O = fm.flash_mhf(*ins)
    (O.float() * dO.cuda().float()).sum().backward()
    ref = _oracle_grads(Q.float(), K.float(), U.float(), V.float(), R, dO.float())
    for name, t, b in zip("dQ dK dU dV dR".split(), ins, ref):
        assert t.grad is not None and t.grad.dtype == t.dtype and t.grad.shape == t.shape
        assert orc.rel_l2(t.grad.cpu().float(), b) < TOL_BF16, name


def test_strided_views_are_read_in_place():
    """Q and dO as transposed views of [B,S,H,d_h] buffers, weights as views of [I, H*d_h] matrices."""
    import flashmhf_b200 as fm
    B, H, S, dh, E, de = 2, 2, 160, 128, 2, 64
    Q, K, U, V, R, dO = orc.make_op_inputs(B, H, S, dh, E, de, seed=15, dtype=torch.bfloat16)
    to_view = lambda t: t.cuda().transpose(1, 2).contiguous().transpose(1, 2)         # [B,H,S,dh] view, S-major memory
    w_view = lambda w: w.cuda().permute(1, 2, 0, 3).reshape(E * de, H * dh).contiguous().view(E, de, H, dh).permute(2, 0, 1, 3)
    Qv, dOv, Kv, Uv, Vv = to_view(Q), to_view(dO), w_view(K), w_view(U), w_view(V)
    assert not Qv.is_contiguous() and not Kv.is_contiguous()
    O = fm.forward_raw(Qv, Kv, Uv, Vv, R.cuda()).cpu().float()
    assert orc.rel_l2(O, orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), R)) < TOL_BF16
    got = [g.cpu().float() for g in fm.backward_raw(Qv, Kv, Uv, Vv, R.cuda(), dOv)]
    ref = _oracle_grads(Q.float(), K.float(), U.float(), V.float(), R, dO.float())
    for name, a, b in zip("dQ dK dU dV dR".split(), got, ref):
        assert orc.rel_l2(a, b) < TOL_BF16, name


@pytest.mark.parametrize("name", ["layer_tiny_dh64", "layer_tiny_gqa"])
def test_golden_operator_fixture(name):
    """The operands the reference hands to its flash back-end, and the O its eager path gives for them."""
    import flashmhf_b200 as fm
    d = load_golden(name)
    ops = [d["op_" + k] for k in "QKUVR"]
    O32 = fm.forward_raw(*_dev(ops)).cpu()
    assert orc.rel_l2(O32, d["op_O"]) < TOL_F32
    ops16 = [t.to(torch.bfloat16) for t in ops[:4]] + [ops[4]]
    O16 = fm.forward_raw(*_dev(ops16)).cpu().float()
    assert orc.rel_l2(O16, d["op_O"]) < TOL_BF16


def test_deterministic_bitwise():
    import flashmhf_b200 as fm
    ins = _dev(orc.make_op_inputs(2, 2, 300, 128, 3, 128, seed=16, dtype=torch.bfloat16))
    a = [fm.forward_raw(*ins[:5])] + list(fm.backward_raw(*ins))
    b = [fm.forward_raw(*ins[:5])] + list(fm.backward_raw(*ins))
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_outputs_fully_written_over_poison():
    """Every element of O is written even when the buffer starts as NaN (no pre-zeroing contract)."""
    import flashmhf_b200 as fm
    Q, K, U, V, R = _dev(orc.make_op_inputs(1, 2, 77, 64, 2, 64, seed=17, dtype=torch.bfloat16, with_dO=False))
    out = torch.full_like(Q, float("nan"))
    fm.forward_raw(Q, K, U, V, R, out=out)
    assert torch.isfinite(out.float()).all()


def test_argument_errors_are_python_exceptions():
    import flashmhf_b200 as fm
    Q, K, U, V, R = _dev(orc.make_op_inputs(1, 2, 64, 64, 2, 64, seed=18, dtype=torch.bfloat16, with_dO=False))
    with pytest.raises(TypeError):
        fm.forward_raw(Q.half(), K, U, V, R)
    with pytest.raises(ValueError):
        fm.forward_raw(Q, K[:, :, :32], U[:, :, :32], V[:, :, :32], R)
    with pytest.raises(ValueError):
        fm.forward_raw(Q[..., :32], K[..., :32], U[..., :32], V[..., :32], R)
    with pytest.raises(ValueError):
        fm.forward_raw(Q.cpu(), K.cpu(), U.cpu(), V.cpu(), R.cpu())


def test_large_shape_linearity_property():
    """At the 370M layer's full token count: O is linear in R, so O(R1) + O(R2) == O(R1 + R2) up to bf16 rounding,
    and a tile-aligned slice of a big batch equals the same rows computed alone (bitwise; the slice is large
    enough -- 128 token tiles -- not to take the split path for short token counts, which sums in another order)."""
    import flashmhf_b200 as fm
    B, H, S, dh, E, de = 4, 8, 2048, 128, 11, 256
    g = torch.Generator(device="cuda").manual_seed(19)
    Q = torch.randn(B, H, S, dh, device="cuda", generator=g).bfloat16()
    K, U, V = (torch.randn(H, E, de, dh, device="cuda", generator=g).mul(0.02).bfloat16() for _ in range(3))
    R1 = torch.rand(B, H, S, E, device="cuda", generator=g)
    R2 = torch.rand(B, H, S, E, device="cuda", generator=g)
    O1, O2, O12 = (fm.forward_raw(Q, K, U, V, r).float() for r in (R1, R2, R1 + R2))
    assert orc.rel_l2((O1 + O2).cpu(), O12.cpu()) < TOL_BF16
    sub = fm.forward_raw(Q[1:3, :, 256:1280].contiguous(), K, U, V, R1[1:3, :, 256:1280].contiguous())
    assert torch.equal(sub, fm.forward_raw(Q, K, U, V, R1)[1:3, :, 256:1280])


def test_forward_and_backward_replay_from_a_cuda_graph():
    """The calls only enqueue kernels on the given stream, so a stream capture records them; replaying the graph on
    new input values (same buffers) must give what the eager calls give.  Covers the split (short) and the plain path."""
    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib
    for shape in ((2, 2, 300, 128, 3, 128), (64, 4, 1, 128, 2, 128)):
        B, H, S, dh, E, de = shape
        Q, K, U, V, R, dO = (t.cuda() for t in orc.make_op_inputs(B, H, S, dh, E, de, seed=77, dtype=torch.bfloat16))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                fm.forward_raw(Q, K, U, V, R)
                fm.backward_raw(Q, K, U, V, R, dO)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            O = fm.forward_raw(Q, K, U, V, R)
            grads = fm.backward_raw(Q, K, U, V, R, dO)
        Q2, _, _, _, R2, dO2 = (t.cuda() for t in orc.make_op_inputs(B, H, S, dh, E, de, seed=78, dtype=torch.bfloat16))
        Q.copy_(Q2); R.copy_(R2); dO.copy_(dO2)
        graph.replay()
        torch.cuda.synchronize()
        got = [O.clone()] + [g.clone() for g in grads]
        want = [fm.forward_raw(Q, K, U, V, R)] + list(fm.backward_raw(Q, K, U, V, R, dO))
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        _lib.device_status()


def test_autograd_under_activation_checkpointing():
    """The function saves only its inputs and recomputes, so it must behave under torch.utils.checkpoint (re-entrant
    forward inside backward) exactly as without it."""
    import flashmhf_b200 as fm
    from torch.utils.checkpoint import checkpoint
    Q, K, U, V, R, dO = (t.cuda() for t in orc.make_op_inputs(2, 2, 150, 128, 2, 64, seed=91, dtype=torch.bfloat16))

    def run(use_ckpt):
        ins = [t.detach().clone().requires_grad_(True) for t in (Q, K, U, V, R)]
        O = checkpoint(fm.flash_mhf, *ins, use_reentrant=False) if use_ckpt else fm.flash_mhf(*ins)
        O.backward(dO)
        return [O.detach()] + [t.grad for t in ins]

    for a, b in zip(run(False), run(True)):
        assert torch.equal(a, b)


def test_two_host_threads_on_their_own_streams():
    """The library keeps no per-call state: two host threads, each on its own stream with its own inputs, get the
    results a single thread gets."""
    import threading
    import flashmhf_b200 as fm
    sets = [[t.cuda() for t in orc.make_op_inputs(1, 2, 260, 128, 2, 128, seed=s, dtype=torch.bfloat16)] for s in (5, 6)]
    want = [[fm.forward_raw(*d[:5])] + list(fm.backward_raw(*d)) for d in sets]
    torch.cuda.synchronize()
    got, errs = [None, None], []

    def work(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(20):
                    r = [fm.forward_raw(*sets[i][:5])] + list(fm.backward_raw(*sets[i]))
            st.synchronize()
            got[i] = r
        except Exception as e:  # surfaced in the main thread below
            errs.append(e)

    ths = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    assert not errs, errs
    for i in range(2):
        for a, b in zip(got[i], want[i]):
            assert torch.equal(a, b)


def test_decode_calls_with_weights_streamed_from_hbm():
    """Batched decode of the 1.3B layer with the weights of eight layers cycled (8 x 69 MB: far more than L2), so that
    every call's weight tiles arrive from HBM, late and out of step with the consumers -- the timing in which a barrier
    phase mistaken for an older one would show.  Every call must repeat bit for bit and match the oracle."""
    import flashmhf_b200 as fm
    B, H, dh, E, de = 64, 16, 128, 22, 256
    Q, K, U, V, R = orc.make_op_inputs(B, H, 1, dh, E, de, seed=23, dtype=torch.bfloat16, with_dO=False)
    Qd, Rd = Q.cuda(), R.cuda()
    g = torch.Generator(device="cuda").manual_seed(24)
    sets = [[K.cuda(), U.cuda(), V.cuda()]] + [
        [torch.randn(H, E, de, dh, device="cuda", generator=g).mul(0.02).bfloat16() for _ in range(3)] for _ in range(7)]
    first = [fm.forward_raw(Qd, *w, Rd) for w in sets]
    for _ in range(3):
        again = [fm.forward_raw(Qd, *w, Rd) for w in sets]
    torch.cuda.synchronize()
    for a, b in zip(first, again):
        assert torch.equal(a, b)
    ref = orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), R)
    assert orc.rel_l2(first[0].cpu().float(), ref) < TOL_BF16
    for w, o in zip(sets[1:3], first[1:3]):
        ref = orc.mhffn_forward(Q.float(), *(t.cpu().float() for t in w), R)
        assert orc.rel_l2(o.cpu().float(), ref) < TOL_BF16


@pytest.mark.parametrize("B,S,H,dh,E,de", [(64, 1, 16, 128, 22, 256), (8, 1, 16, 128, 22, 256), (3, 1, 4, 64, 2, 64),
                                           (5, 1, 6, 96, 3, 128), (2, 300, 4, 128, 4, 128)])
def test_chained_forward_equals_plain_forward(B, S, H, dh, E, de):
    """`flashmhf_forward_chained` (launch may overlap the end of the kernel before it; split partial sums added inside
    the kernel) gives the plain call's bits: single calls, a chain of eight layers whose O feeds the next Q, the chain
    replayed from a CUDA graph, and plain calls in between (the per-tile counters are back at zero after every call)."""
    import flashmhf_b200 as fm
    Q, K, U, V, R = orc.make_op_inputs(B, H, S, dh, E, de, seed=31, dtype=torch.bfloat16, with_dO=False)
    Qd, Rd = Q.cuda(), R.cuda()
    g = torch.Generator(device="cuda").manual_seed(32)
    sets = [[K.cuda(), U.cuda(), V.cuda()]] + [
        [torch.randn(H, E, de, dh, device="cuda", generator=g).mul(0.05).bfloat16() for _ in range(3)] for _ in range(7)]
    plain = fm.forward_raw(Qd, *sets[0], Rd)
    ref = orc.mhffn_forward(Q.float(), K.float(), U.float(), V.float(), R)
    assert orc.rel_l2(plain.cpu().float(), ref) < TOL_BF16
    for _ in range(3):
        assert torch.equal(fm.forward_raw(Qd, *sets[0], Rd, chained=True), plain)

    def chain(chained):
        q = Qd
        for w in sets:
            q = fm.forward_raw(q, *w, Rd, chained=chained) * 4.0   # a small kernel between the calls, as a model has
        return q

    want = chain(False)
    got = chain(True)
    assert torch.equal(got, want)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain(True)
    torch.cuda.current_stream().wait_stream(side)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        out = chain(True)
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert torch.equal(fm.forward_raw(Qd, *sets[0], Rd), plain)
    fm.check_device_status()
