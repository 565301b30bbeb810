"""Operator and LM measurements beyond the one line bench.py prints.

    python opbench.py --sweep      # operator forward+backward over a grid of shapes, next to a dense SwiGLU and the eager path on the GPU
    python opbench.py --lm         # forward tokens/s of the 128M and 1.3B LMs, training step of the 370M LM
    python opbench.py --decode     # decode-shaped forward calls (a few tokens, weights streamed from HBM)

Everything is timed with CUDA events after warm-up; inputs are seeded synthetic tensors (Q ~ N(0,1),
weights ~ N(0, 0.02), routing weights = normalised sigmoid of N(0,1) logits, dO ~ N(0,1)).
Algorithmic FLOPs of the operator: 18*T*H*I*d_h for forward+backward (recompute not counted); the dense
SwiGLU with the same parameter count (W_g, W_u, W_d of shape [I, H*d_h]) has the same count.
Prints markdown tables.
"""
import argparse
import time
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

NOMINAL_TFLOPS = 2250.0


def _measured_sustained():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except (OSError, KeyError, ValueError):
        return 1400.0


def _time(fn, target_s=0.25, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record(); torch.cuda.synchronize()
    n = max(3, min(200, int(target_s * 1e3 / max(e0.elapsed_time(e1), 1e-3))))
    e0.record()
    for _ in range(n):
        fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def sweep(args):
    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib
    sustained = _measured_sustained()
    dev = torch.device("cuda")
    print("| T | d_h | H | E | d_e | fwd ms | bwd ms | TFLOP/s | of nominal 2250 | of measured %.0f | peak MB | dense SwiGLU TFLOP/s | ratio | eager-on-GPU TFLOP/s |" % sustained)
    print("|---|---|---|---|---|---|---|---|---|---|---|---|---|---|")
    shapes = []
    for dh, des in ((128, (320, 256)), (64, (192,))):
        for de in des:
            for H in (8, 16):
                for E in (8, 16, 32):
                    for T in (4096, 16384, 65536, 262144):
                        shapes.append((T, dh, H, E, de))
    if args.quick:
        shapes = [s for s in shapes if s[0] in (4096, 65536) and s[3] != 16]
    for T, dh, H, E, de in shapes:
        B, S = T // 4096, 4096
        g = torch.Generator(device=dev).manual_seed(0)
        Q = torch.randn(B, H, S, dh, device=dev, generator=g).bfloat16()
        dO = torch.randn(B, H, S, dh, device=dev, generator=g).bfloat16()
        K, U, V = (torch.randn(H, E, de, dh, device=dev, generator=g).mul(0.02).bfloat16() for _ in range(3))
        R = torch.randn(B, H, S, E, device=dev, generator=g).sigmoid()
        R = R / R.sum(-1, keepdim=True)
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        tf = _time(lambda: fm.forward_raw(Q, K, U, V, R))
        tb = _time(lambda: fm.backward_raw(Q, K, U, V, R, dO))
        peak = (torch.cuda.max_memory_allocated() - base) / 2**20
        _lib.device_status()
        flops = 18.0 * T * H * E * de * dh
        tfl = flops / ((tf + tb) * 1e-3) / 1e12
        # dense SwiGLU of the same parameter count, torch matmul + autograd
        hid, I = H * dh, E * de
        X = Q.transpose(1, 2).reshape(T, hid).contiguous().requires_grad_(True)
        Wg, Wu, Wd = (torch.randn(I, hid, device=dev, generator=g).mul(0.02).bfloat16().requires_grad_(True) for _ in range(3))
        gO = dO.transpose(1, 2).reshape(T, hid).contiguous()

        def dense():
            y = (torch.nn.functional.silu(X @ Wg.t()) * (X @ Wu.t())) @ Wd
            y.backward(gO)
            X.grad = Wg.grad = Wu.grad = Wd.grad = None
        td = _time(dense)
        tfd = flops / (td * 1e-3) / 1e12
        # harness-side comparator: the reference's eager loop (the CPU oracle's restatement of it) run on the GPU in
        # bf16 with autograd -- what the reference layer does with use_flash=False; only where its [T, d_e]
        # intermediates fit comfortably
        tfe = None
        if T * H * de * 2 * 8 * E < 40e9:
            from oracle import mhffn_oracle as orc
            ins = [t.detach().clone().requires_grad_(True) for t in (Q, K, U, V, R)]

            def eager():
                orc.mhffn_forward(*ins).backward(dO)
                for t in ins:
                    t.grad = None
            tfe = flops / (_time(eager) * 1e-3) / 1e12
            del ins
        print(f"| {T} | {dh} | {H} | {E} | {de} | {tf:.3f} | {tb:.3f} | {tfl:.0f} | {tfl / NOMINAL_TFLOPS:.3f} | {tfl / sustained:.3f} | "
              f"{peak:.0f} | {tfd:.0f} | {tfl / tfd:.2f} | {'-' if tfe is None else format(tfe, '.0f')} |", flush=True)
        del Q, dO, K, U, V, R, X, Wg, Wu, Wd, gO
        torch.cuda.empty_cache()


def lm_runs(args):
    from flashmhf_b200 import _lib, lm
    dev = torch.device("cuda")
    print("| model | parameters | batch x seq | pass | ms | tokens/s | model TFLOP/s | FFN kernels' share |")
    print("|---|---|---|---|---|---|---|---|")
    for name, cfg, B, S in (("128M", lm.LMConfig.lm_128m(), 8, 2048), ("1.3B", lm.LMConfig.lm_1p3b(), 4, 8192)):
        model = lm.DecoderLM(cfg).init_weights(seed=0).to(dev).to(torch.bfloat16)
        ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(0)).to(dev)
        with torch.no_grad():
            ms = _time(lambda: model(ids), target_s=1.0)
            _lib.profile_begin(4096)
            model(ids)
            ours = sum(sum(v) for v in _lib.profile_end().values())
        fl = lm.train_flops_per_token(cfg, S) / 3 * B * S
        print(f"| {name} | {lm.param_count(model) / 1e6:.0f} M | {B} x {S} | forward | {ms:.2f} | {B * S / (ms * 1e-3):.0f} | "
              f"{fl / (ms * 1e-3) / 1e12:.0f} | {ours / ms:.2f} |", flush=True)
        del model
        torch.cuda.empty_cache()
    cfg, B, S = lm.LMConfig.lm_370m(), 16, 2048
    model = lm.DecoderLM(cfg).init_weights(seed=0).to(dev).to(torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(0)).to(dev)
    ms = _time(lambda: lm.train_step(model, opt, ids), target_s=2.0)
    _lib.profile_begin(4096)
    lm.train_step(model, opt, ids)
    ours = sum(sum(v) for v in _lib.profile_end().values())
    fl = lm.train_flops_per_token(cfg, S) * B * S
    print(f"| 370M | {lm.param_count(model) / 1e6:.0f} M | {B} x {S} | forward + backward + AdamW | {ms:.2f} | {B * S / (ms * 1e-3):.0f} | "
          f"{fl / (ms * 1e-3) / 1e12:.0f} | {ours / ms:.2f} |", flush=True)
    print(f"\npeak memory of the 370M training step: {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB")


def decode_runs(args):
    """Decode-shaped forward calls: B sequences, one new token each.  The weights of 8 layers are cycled so that every
    call streams its K, U, V from HBM (one layer's weights would stay in L2).  Reported per layer call: the time the
    interpreter needs to issue it, the time from Python (issue and execution overlapped), kernel-only time from CUDA
    events, the same calls replayed from a CUDA graph, and a chain of the eight layers (each call's O is the next
    call's Q) through the chained entry point, replayed from a graph; GB/s is the layer's weight bytes over that time
    (algorithmic bytes of the call: 6*H*E*d_e*d_h, Q/O/R are negligible)."""
    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib
    hbm = 6547.0
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm = float(json.load(f)["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        pass
    print(f"| shape | weights MB | host us per call | python call us | kernels us (fwd + reduce) | fwd kernel GB/s | of measured {hbm:.0f} | "
          f"graph replay us | graph GB/s | chained graph us | chained GB/s | of measured {hbm:.0f} |")
    print("|---|---|---|---|---|---|---|---|---|---|---|---|")
    for (B, H, E, de, dh, name) in [(64, 16, 22, 256, 128, "1.3B layer, 64 tokens"), (8, 16, 22, 256, 128, "1.3B layer, 8 tokens"),
                                    (64, 8, 11, 256, 128, "370M layer, 64 tokens")]:
        g = torch.Generator(device="cuda").manual_seed(0)
        Q = torch.randn(B, H, 1, dh, device="cuda", generator=g).bfloat16()
        Ws = [[torch.randn(H, E, de, dh, device="cuda", generator=g).mul(0.02).bfloat16() for _ in range(3)] for _ in range(8)]
        R = torch.rand(B, H, 1, E, device="cuda", generator=g)
        for i in range(8):
            fm.forward_raw(Q, *Ws[i], R)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        n = 80
        ev[0].record()
        t_host = time.perf_counter()
        for i in range(n):
            fm.forward_raw(Q, *Ws[i % 8], R)
        host_us = (time.perf_counter() - t_host) / n * 1e6   # time the interpreter needs to issue a call
        ev[1].record()
        torch.cuda.synchronize()
        call_us = ev[0].elapsed_time(ev[1]) / n * 1e3
        wbytes = 3 * H * E * de * dh * 2
        _lib.profile_begin(1024)
        for i in range(n):
            fm.forward_raw(Q, *Ws[i % 8], R)
        k = _lib.profile_end()
        _lib.device_status()
        fwd_us = sum(k["fwd_kernel"]) / len(k["fwd_kernel"]) * 1e3
        red_us = sum(k.get("o_reduce_kernel", [0.0])) / max(1, len(k.get("o_reduce_kernel", []))) * 1e3
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(8):
                fm.forward_raw(Q, *Ws[i], R)
        torch.cuda.current_stream().wait_stream(side)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            outs = [fm.forward_raw(Q, *Ws[i], R) for i in range(8)]
        gr.replay()
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(10):
            gr.replay()
        ev[1].record()
        torch.cuda.synchronize()
        graph_us = ev[0].elapsed_time(ev[1]) / 80 * 1e3
        # the same eight layers as a chain (each call's O is the next call's Q), with the chained entry point
        def chain(chained):
            q = Q
            for i in range(8):
                q = fm.forward_raw(q, *Ws[i], R, chained=chained)
            return q
        want = chain(False)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            got = chain(True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        same = torch.equal(want, got)
        gc = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gc):
            got = chain(True)
        gc.replay()
        torch.cuda.synchronize()
        same = same and torch.equal(want, got)
        ev[0].record()
        for _ in range(10):
            gc.replay()
        ev[1].record()
        torch.cuda.synchronize()
        _lib.device_status()
        chain_us = ev[0].elapsed_time(ev[1]) / 80 * 1e3
        print(f"| {name} | {wbytes / 1e6:.1f} | {host_us:.1f} | {call_us:.1f} | {fwd_us:.1f} + {red_us:.1f} | {wbytes / fwd_us / 1e3:.0f} | "
              f"{wbytes / fwd_us / 1e3 / hbm:.2f} | {graph_us:.1f} | {wbytes / graph_us / 1e3:.0f} | "
              f"{chain_us:.1f}{'' if same else ' (MISMATCH)'} | {wbytes / chain_us / 1e3:.0f} | {wbytes / chain_us / 1e3 / hbm:.2f} |",
              flush=True)
        del outs, gr, gc, Ws


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--lm", action="store_true")
    ap.add_argument("--decode", action="store_true")
    ap.add_argument("--quick", action="store_true", help="a quarter of the sweep grid")
    args = ap.parse_args()
    if not (args.sweep or args.lm or args.decode):
        ap.error("choose --sweep, --lm and/or --decode")
    if args.sweep:
        sweep(args)
    if args.lm:
        lm_runs(args)
    if args.decode:
        decode_runs(args)


if __name__ == "__main__":
    main()
