"""Benchmark of the FlashMHF operator, forward + backward, on the 370M model's FFN layer shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one forward and one backward pass of the operator over one batch of synthetic input
(per GPU: B=16 x S=2048 tokens, H=8 heads of d_h=128, E=11 sub-networks of d_e=256 -- the FFN of one
layer of the 370M configuration).  With N > 1 (one process per GPU, launched by torch.distributed.run)
every rank works on its own batch with replicated weights and the step holds one NCCL all-reduce of
dK, dU, dV (data-parallel training's only exchange), started as soon as the weight gradients exist and
running under the dQ/dR kernel; scaling is weak.

The metric is algorithmic TFLOP/s: 18*T*H*I*d_h FLOPs per step (3 forward + 6 gradient GEMMs; the
recomputation the backward needs is NOT counted) divided by the step time, summed over GPUs.
Next to it, in the same JSON line: the same through the public autograd API with host buffers (`e2e`),
the dominant kernel's roofline fraction, the CPU baseline, a full 370M training step (`train_370m`) and
three token-sharded inference runs (`infer_128m`, `prefill_1p3b`, `decode_1p3b`).  Prints ONE JSON line on rank 0.
"""
import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOAD = dict(name="flashmhf_370m_layer_op_fwd_bwd", B=16, S=2048, H=8, Hkuv=8, Dh=128, E=11, De=256)
NOMINAL_BF16_TFLOPS = 2250.0
KERNEL_SOURCES = ("tc_common.cuh", "tc_fwd.cu", "tc_bwd.cu")
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
CPU_CHUNK_ROWS = 4          # the CPU legs walk the batch in chunks of this many rows to bound host memory


def alg_flops(B, S, H, Dh, E, De, passes=18):
    return passes * B * S * H * E * De * Dh


def workload_config(w, world):
    """What both arms print as `config`: a description of the workload only (no measured values)."""
    return {"workload": w["name"], "B_per_gpu": w["B"], "S": w["S"], "H": w["H"], "Hkuv": w["Hkuv"], "Dh": w["Dh"],
            "E": w["E"], "De": w["De"], "flops_per_step": "18*T*H*E*De*Dh (recompute not counted)",
            "l2": "per-step working set (Q, dO, O, dQ, R, dR ~300 MB) exceeds the 126 MB L2",
            "parallelism": f"dp{world}" + (" + NCCL all-reduce of dK,dU,dV" if world > 1 else "")}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


def kernel_source_digest():
    """sha256 over the tensor-core kernel sources: ties a recorded ncu figure to the kernels it was taken from."""
    h = hashlib.sha256()
    for name in KERNEL_SOURCES:
        with open(os.path.join(ROOT, "flashmhf_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def recorded_traffic(kernel, w):
    """DRAM bytes (read + write) per launch of `kernel` from the recorded ncu capture, or None (with the reason) when
    the record was taken from other kernel sources or another workload than the ones running now."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f)
    except (OSError, ValueError):
        return None, "no recorded capture"
    if rec.get("kernel_source_sha256") != kernel_source_digest():
        return None, "recorded capture is of older kernel sources"
    if any(rec.get("workload", {}).get(k) != w[k] for k in ("B", "S", "H", "Hkuv", "Dh", "E", "De")):
        return None, "recorded capture is of another workload"
    v = rec.get("dram_bytes_per_launch", {}).get(kernel)
    return (float(v), rec.get("command", "")) if v is not None else (None, "kernel not in the recorded capture")


def choose_peak(peaks, timed_seconds):
    """Burst cuBLAS figure for a timed region shorter than a second (clocks have not settled under the power cap),
    the sustained one otherwise."""
    kind = "burst" if timed_seconds < 1.0 else "sustained"
    return kind, peaks[kind]


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            try:
                pw.append(float(f[2]))
            except ValueError:
                pass
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": statistics.median(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------- CPU legs
def find_reference():
    """A checkout of the reference project, if this machine has one (the GPU boxes normally do not)."""
    cands = [os.environ.get("FLASHMHF_REFERENCE", ""), os.path.join(ROOT, "baseline", "_ref")]
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            cands.append(json.load(f).get("reference_path", ""))
    except (OSError, ValueError):
        pass
    for c in cands:
        if c and os.path.exists(os.path.join(c, "models", "flashmhf", "modeling_mhffnmoe.py")):
            return c
    return None


def make_cpu_step(w, rows):
    """One CPU pass (fp32, all host threads) of forward + autograd backward over `rows` batch rows of the workload,
    walked in chunks of CPU_CHUNK_ROWS rows.  Uses the UNMODIFIED reference layer's eager branch when a checkout of the
    reference is on this machine (built with skip_linear so that the layer is the head split, the router and the
    eager loop, models/flashmhf/modeling_mhffnmoe.py:362-430), else the oracle's restatement of that loop.
    Returns (step function, kind)."""
    torch.set_num_threads(os.cpu_count() or 1)
    H, Hk, Dh, E, De, S = (w[k] for k in ("H", "Hkuv", "Dh", "E", "De", "S"))
    chunks = [min(CPU_CHUNK_ROWS, rows - i) for i in range(0, rows, CPU_CHUNK_ROWS)]
    ref = find_reference()
    if ref is not None:
        try:
            from tests.golden.make_golden import load_reference, seeded_params
            C_, M = load_reference(ref)
            cfg = C_.MHFFNMoEConfig(hidden_size=H * Dh, intermediate_size=E * De, num_attention_heads=H,
                                    mhffnmoe_num_heads=H, mhffnmoe_num_kuv_heads=Hk, mhffnmoe_num_experts=E,
                                    mhffnmoe_use_flash=False, mhffnmoe_custom_init=True, mhffnmoe_apply_rmsnorm=False,
                                    mhffnmoe_skip_linear=True, rms_norm_eps=1e-5)
            layer = M.MHFFNMoEMultiHeadFFNFlash(cfg, use_flash=False)
            seeded_params(layer, 0)
            g = torch.Generator().manual_seed(0)
            xs = [torch.randn(c, S, H * Dh, generator=g, requires_grad=True) for c in chunks]
            gs = [torch.randn(c, S, H * Dh, generator=g) for c in chunks]

            def step():
                layer.zero_grad(set_to_none=True)
                for x, gy in zip(xs, gs):
                    x.grad = None
                    layer(x).backward(gy)
            return step, "reference"
        except Exception as e:  # an unusable checkout is not an error of the benchmark
            print(f"bench: reference checkout at {ref} not usable ({type(e).__name__}: {e}); timing the oracle port",
                  file=sys.stderr)
    from oracle import mhffn_oracle as orc
    sets = []
    for i, c in enumerate(chunks):
        Q, K, U, V, R, dO = orc.make_op_inputs(c, H, S, Dh, E, De, Hkuv=Hk, seed=i)
        sets.append(([t.requires_grad_(True) for t in (Q, K, U, V, R)], dO))

    def step():
        for ins, dO in sets:
            for t in ins:
                t.grad = None
            orc.mhffn_forward(*ins).backward(dO)
    return step, "port"


def cpu_baseline(w, seconds=20.0):
    """The reference's CPU path for the operator, timed on this box's host cores on a bounded sample: whole passes over
    the full workload, as many as fit in about `seconds` (at least 2)."""
    step, kind = make_cpu_step(w, w["B"])
    step()
    t0 = time.perf_counter()
    step()
    first = time.perf_counter() - t0
    times = [first]
    while sum(times) < seconds - first and len(times) < 12:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    fl = alg_flops(w["B"], w["S"], w["H"], w["Dh"], w["E"], w["De"])
    what = ("the unmodified reference layer's eager branch" if kind == "reference" else
            "the oracle's restatement of the reference's eager loop")
    return {"value": fl / med / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{len(times)} passes (after 1 warm-up) over the full workload ({w['B']} x {w['S']} tokens, in chunks of "
                      f"{CPU_CHUNK_ROWS} rows), {what}, fp32 forward + autograd backward, median pass",
            "seconds_per_pass": med, "seconds_total": sum(times)}


def run_reference(args, rank, world):
    """`--impl reference`: the reference's CPU path for this operator on the box's host cores, all threads, on the GPU
    arm's workload: each step is one pass over the full per-GPU batch (B=16 x S=2048).  If a probe says warm-up + K
    steps would not end within about four minutes, a step covers fewer batch rows and the line says how many."""
    if rank != 0:
        return
    w = WORKLOAD
    probe, _ = make_cpu_step(w, 1)
    probe()
    t0 = time.perf_counter()
    probe()
    per_row = time.perf_counter() - t0
    rows = w["B"]
    budget = 240.0 / max(1, args.steps + args.warmup)
    if per_row * rows > budget:
        rows = max(1, int(budget / per_row))
    step, kind = make_cpu_step(w, rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = alg_flops(rows, w["S"], w["H"], w["Dh"], w["E"], w["De"]) / dt / 1e12
    what = ("the unmodified reference layer's eager branch (use_flash=False)" if kind == "reference" else
            "the reference's eager loop restated (the reference itself is Python source that is not on this box)")
    sample = (f"each step = {rows} of the workload's {w['B']} batch rows x {w['S']} tokens, fp32 PyTorch eager forward + "
              f"autograd backward, {what}")
    print(json.dumps({
        "impl": "reference", "metric": "flashmhf_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, world), "rows_per_step": rows,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def bind_to_gpu_numa_node(index):
    """Run this process on the CPUs next to its GPU, so that the pinned host buffers of the end-to-end leg are allocated
    on that NUMA node and their copies do not cross the socket interconnect.  Best effort: silently skipped without NVML."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


# --------------------------------------------------------------------------------------- LM legs
def lm_train_370m(args, rank, world, dev, sync_all):
    """The second half of the headline metric: full training steps (forward, backward, gradient all-reduce,
    AdamW) of the 370M decoder LM at batch 16 x 2048 per GPU, bf16, uniform random token ids, data-parallel.
    Token ids come from pinned host memory every step and the loss is read back to the host, inside the timed region."""
    from flashmhf_b200 import _lib, dp, lm
    cfg = lm.LMConfig.lm_370m()
    Bt, St = 16, 2048
    with torch.device(dev):                      # built and drawn on the GPU: same seed -> same weights on every rank
        model = lm.DecoderLM(cfg).to(torch.bfloat16).init_weights(seed=0)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    red = dp.GradReducer(buckets=dp.lm_buckets(model)) if world > 1 else None
    ids_host = torch.randint(0, cfg.vocab_size, (Bt, St), generator=torch.Generator().manual_seed(rank)).pin_memory()
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()

    def step():
        ids = ids_host.to(dev, non_blocking=True)
        loss = lm.train_step(model, opt, ids, red)
        loss_host.copy_(loss, non_blocking=True)

    for _ in range(3):
        step()
    sync_all()
    first_loss = float(loss_host)
    launches0 = _lib.launch_count()
    _lib.profile_begin(16 * cfg.num_hidden_layers * args.lm_steps + 16)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.lm_steps):
        step()
    e1.record()
    sync_all()
    kernel_ms = _lib.profile_end(capacity=16 * cfg.num_hidden_layers * args.lm_steps + 16)
    _lib.device_status()
    ms = dp.max_over_ranks(e0.elapsed_time(e1) / args.lm_steps, dev)
    ours_ms = sum(sum(v) for v in kernel_ms.values()) / args.lm_steps
    flops = lm.train_flops_per_token(cfg, St) * Bt * St
    return {"tokens_per_s": Bt * St * world / (ms * 1e-3), "ms_per_step": ms, "steps": args.lm_steps, "warmup": 3,
            "batch_per_gpu": Bt, "seq_len": St, "n_params": lm.param_count(model), "optimizer": "AdamW (torch fused), bf16 parameters",
            "model_tflops_per_gpu": flops / (ms * 1e-3) / 1e12,
            "ffn_kernels_ms_per_step": ours_ms, "ffn_kernels_share": ours_ms / ms,
            "library_kernel_launches_per_step": (_lib.launch_count() - launches0) / args.lm_steps,
            "loss_first_last": [first_loss, float(loss_host)],
            "outside_the_ffn": "attention = torch scaled_dot_product_attention, projections = cuBLAS, loss = torch cross_entropy",
            "parallelism": f"dp{world}" + (" + per-layer NCCL all-reduce overlapped with backward" if world > 1 else "")}


def lm_inference(name, cfg, rows, seq, what, args, rank, world, dev, sync_all):
    """Token-sharded inference: the batch rows of one request (`rows` x `seq` uniform random token ids, the same on every
    N) are split over the ranks with dp.shard_range; weights are replicated; no collective in the data path (attention
    stays inside a sequence, the FFN has no cross-token dependence).  A prefill on more ranks than sequences also cuts
    the sequences into consecutive parts (see below: the one case with an exchange, keys and values from part to part).  Each timed step copies this rank's ids from pinned
    host memory, runs the bf16 forward and reads the arg-max of the last position's logits back.  `what` = "logits"
    (full forward, logits at every position) or "prefill" (hidden states everywhere, logits of the last position).
    Reports whole-job tokens/s from the slowest rank's time."""
    from flashmhf_b200 import _lib, dp, lm
    a, b = dp.shard_range(rows, rank, world) if rank < min(world, rows) else (0, 0)
    parts, link, t_a, t_b, cuts = 1, None, 0, seq, [0, seq]
    if world > rows:
        if what == "prefill" and world % rows == 0 and seq % (world // rows) == 0:
            # More ranks than sequences: every sequence is cut into world/rows consecutive parts, one per rank.  The FFN,
            # the projections and the norms are position-wise; attention needs the earlier parts' keys and values, which
            # travel from part to part once per layer (NCCL send/recv between the ranks of one sequence).
            parts = world // rows
            row, part = rank // parts, rank % parts
            a, b = row, row + 1
            # Equal parts, except for two: the later part attends over the earlier one as well, so the earlier part is made
            # longer (9/16 of the sequence balances the two at this model's ratio of attention to position-wise work).
            cuts = [p_ * (seq // parts) for p_ in range(parts)] + [seq]
            if parts == 2 and seq % 2048 == 0:
                cuts[1] = seq * 9 // 16
            t_a, t_b = cuts[part], cuts[part + 1]
            link = lm.SequenceLink(first=t_a, recv_from=rank - 1 if part > 0 else None,
                                   send_to=rank + 1 if part + 1 < parts else None)
        else:                                          # the first `rows` ranks take one row each, the others have no work
            a, b = (rank, rank + 1) if rank < rows else (0, 0)
    with torch.device(dev):
        model = lm.DecoderLM(cfg).to(torch.bfloat16).init_weights(seed=0)
    ids_all = torch.randint(0, cfg.vocab_size, (rows, seq), generator=torch.Generator().manual_seed(0))
    ids_host = ids_all[a:b, t_a:t_b].contiguous().pin_memory() if b > a else None
    out_host = torch.zeros(max(1, b - a), dtype=torch.int64).pin_memory()

    ids_dev = ids_host.to(dev) if ids_host is not None else None   # static device buffer the captured graph reads

    @torch.no_grad()
    def forward():
        if what == "logits":
            last = model(ids_dev)[:, -1]
        else:
            last = model.lm_head(model.hidden(ids_dev, link=link)[:, -1])   # (the request's answer is the last part's)
        return last.float().argmax(-1)

    # The forward pass of a small model is hundreds of short kernels: replayed from a CUDA graph so that the step is
    # paced by the GPU and not by the Python interpreter (every kernel of this library only enqueues work and captures).
    graph, result, ffn_ms = None, None, 0.0
    if ids_host is not None:
        for _ in range(2):
            result = forward()
        torch.cuda.synchronize()
        _lib.profile_begin(16 * cfg.num_hidden_layers + 16)     # this library's kernels in one (eager) forward pass
        result = forward()
        ffn_ms = sum(sum(v) for v in _lib.profile_end(capacity=16 * cfg.num_hidden_layers + 16).values())
        try:
            if link is not None:
                raise RuntimeError("a split sequence exchanges keys and values between ranks: run eagerly")
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_):
                result = forward()
            graph = g_
        except Exception as e:   # capture is an optimisation of the harness, not a requirement
            if link is None:
                print(f"bench: {name} inference runs without a CUDA graph ({type(e).__name__}: {e})", file=sys.stderr)
            torch.cuda.synchronize()

    def step():
        nonlocal result
        if ids_host is None:
            return
        ids_dev.copy_(ids_host, non_blocking=True)
        if graph is not None:
            graph.replay()
        else:
            result = forward()
        out_host.copy_(result, non_blocking=True)

    for _ in range(2):
        step()
    sync_all()
    n = args.infer_steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    sync_all()
    _lib.device_status()
    mine = e0.elapsed_time(e1) / n
    ms = dp.max_over_ranks(mine, dev)
    share = dp.max_over_ranks(ffn_ms / mine if ids_host is not None and mine > 0 else 0.0, dev)
    del model
    torch.cuda.empty_cache()
    if parts == 1:
        split_note = f"batch rows over {min(world, rows)} of {world} ranks, no collective in the data path"
    else:
        sizes = " + ".join(str(cuts[i + 1] - cuts[i]) for i in range(parts))
        split_note = (f"{rows} sequences x {parts} consecutive parts ({sizes} tokens) over {world} ranks; keys and values pass "
                      "from part to part once per layer (NCCL send/recv), nothing else is exchanged")
    return {"model": name, "pass": "bf16 forward, " + ("logits at every position" if what == "logits" else
                                                        "prefill: hidden states of all tokens, logits of the last"),
            "rows": rows, "seq_len": seq, "tokens_per_s": rows * seq / (ms * 1e-3), "ms_per_step": ms, "steps": n, "warmup": 2,
            "split": split_note,
            "cuda_graph": graph is not None,
            "ranks_with_work": min(world, rows) * parts, "ffn_kernels_share": share,
            "h2d_bytes_per_step_per_rank": (b - a) * (t_b - t_a) * 8, "d2h_bytes_per_step_per_rank": (b - a) * 8}


def lm_decode(name, cfg, rows, context, args, rank, world, dev, sync_all):
    """Batched decode: `rows` sequences, each with `context` positions in the key/value cache (synthetic contents), one
    new token per sequence per step; the sequences are split over the ranks (weights replicated, no collective).  Each
    timed step copies this rank's token ids from pinned host memory, runs the bf16 step (replayed from a CUDA graph: a
    decode step is a few hundred short kernels) and reads the arg-max of the logits back.  The step is bound by HBM:
    it reads every weight matrix once and the cached keys and values of `context` positions; both byte counts and the
    achieved rate per GPU are reported, and the share of the step spent in this library's kernels."""
    from flashmhf_b200 import _lib, dp, lm
    a, b = dp.shard_range(rows, rank, world) if rank < min(world, rows) else (0, 0)
    if world > rows:
        a, b = (rank, rank + 1) if rank < rows else (0, 0)
    n_mine = b - a
    with torch.device(dev):
        model = lm.DecoderLM(cfg).to(torch.bfloat16).init_weights(seed=0)
    weight_bytes = sum(p.numel() * p.element_size() for k, p in model.named_parameters()
                       if cfg.tie_word_embeddings or not k.startswith("model.embed_tokens"))
    ids_all = torch.randint(0, cfg.vocab_size, (rows, 1), generator=torch.Generator().manual_seed(0))
    graph, result, ffn_ms, kv_bytes = None, None, 0.0, 0
    if n_mine:
        cache = lm.KVCache(cfg, n_mine, context + 8, dev)
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        cache.k.normal_(0.0, 1.0, generator=g)
        cache.v.normal_(0.0, 1.0, generator=g)
        kv_bytes = cache.nbytes(context + 1)
        ids_host = ids_all[a:b].contiguous().pin_memory()
        ids_dev = ids_host.to(dev)
        out_host = torch.zeros(n_mine, dtype=torch.int64).pin_memory()

        @torch.no_grad()
        def forward():
            return model.decode_step(ids_dev, cache, context).float().argmax(-1)

        for _ in range(2):
            result = forward()
        torch.cuda.synchronize()
        _lib.profile_begin(16 * cfg.num_hidden_layers + 16)
        result = forward()
        ffn_ms = sum(sum(v) for v in _lib.profile_end(capacity=16 * cfg.num_hidden_layers + 16).values())
        try:
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_):
                result = forward()
            graph = g_
        except Exception as e:   # capture is an optimisation of the harness, not a requirement
            print(f"bench: {name} decode runs without a CUDA graph ({type(e).__name__}: {e})", file=sys.stderr)
            torch.cuda.synchronize()

    def step():
        nonlocal result
        if not n_mine:
            return
        ids_dev.copy_(ids_host, non_blocking=True)
        if graph is not None:
            graph.replay()
        else:
            result = forward()
        out_host.copy_(result, non_blocking=True)

    for _ in range(3):
        step()
    sync_all()
    n = args.infer_steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    sync_all()
    _lib.device_status()
    mine = e0.elapsed_time(e1) / n
    ms = dp.max_over_ranks(mine, dev)
    share = dp.max_over_ranks(ffn_ms / mine if n_mine and mine > 0 else 0.0, dev)
    ffn_max = dp.max_over_ranks(ffn_ms, dev)
    kv_max = dp.max_over_ranks(float(kv_bytes), dev)
    if n_mine:
        del cache
    del model
    torch.cuda.empty_cache()
    return {"model": name, "pass": "bf16 decode step: one new token per sequence, attention over the cached context",
            "rows": rows, "context": context, "tokens_per_s": rows / (ms * 1e-3), "ms_per_step": ms, "steps": n, "warmup": 3,
            "split": f"sequences over {min(world, rows)} of {world} ranks, no collective in the data path",
            "cuda_graph": graph is not None, "ranks_with_work": min(world, rows),
            "weight_bytes_per_step_per_rank": weight_bytes, "kv_bytes_per_step_per_rank": kv_max,
            "hbm_gbs_per_rank": (weight_bytes + kv_max) / (ms * 1e-3) / 1e9,
            "ffn_kernels_ms": ffn_max, "ffn_kernels_share": share,
            "h2d_bytes_per_step_per_rank": n_mine * 8, "d2h_bytes_per_step_per_rank": n_mine * 8}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="B=2 instead of 16 (for profiler captures)")
    ap.add_argument("--no-lm", action="store_true", help="skip the LM measurements (370M training step, inference runs)")
    ap.add_argument("--lm-steps", type=int, default=8)
    ap.add_argument("--infer-steps", type=int, default=10)
    ap.add_argument("--prefill-rows", type=int, default=4, help="sequences of the 1.3B prefill request (4 in the headline configuration)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    if args.warmup < 3:
        args.warmup = 3 if not args.small else args.warmup

    import flashmhf_b200 as fm
    from flashmhf_b200 import _lib, dp
    _lib.load()  # fails loudly if the CUDA library is missing
    if world > 1:   # one rank per GPU shares the host: keep each rank's pinned buffers on its GPU's NUMA node
        bind_to_gpu_numa_node(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    w = dict(WORKLOAD)
    if args.small:
        w["B"] = 2
    B, S, H, Hk, Dh, E, De = (w[k] for k in ("B", "S", "H", "Hkuv", "Dh", "E", "De"))
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    gw = torch.Generator(device=dev).manual_seed(99)  # same weights on every rank
    Q = torch.randn(B, H, S, Dh, device=dev, generator=g).bfloat16()
    dO = torch.randn(B, H, S, Dh, device=dev, generator=g).bfloat16()
    R = torch.randn(B, H, S, E, device=dev, generator=g).sigmoid()
    R = R / R.sum(-1, keepdim=True)
    K, U, V = (torch.randn(Hk, E, De, Dh, device=dev, generator=gw).mul(0.02).bfloat16() for _ in range(3))
    bucket = dp.WeightGradBucket(K)   # dK, dU, dV as three views of one all-reduce buffer

    def device_step():
        O = fm.forward_raw(Q, K, U, V, R)
        # weight gradients first, straight into the bucket; their all-reduce (none on one GPU) runs under the dQ/dR kernel
        dQ, _, _, _, dR = dp.exchange_under_inputs(
            lambda views: fm.backward_raw(Q, K, U, V, R, dO, parts="weights", weight_grads=views),
            lambda: fm.backward_raw(Q, K, U, V, R, dO, parts="inputs"), bucket)
        return O, dQ, dR

    def sync_all():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        device_step()
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    _lib.profile_begin(8 * args.steps + 8)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    for _ in range(args.steps):
        device_step()
    ev1.record()
    sync_all()
    kernel_ms = _lib.profile_end()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = ev0.elapsed_time(ev1) / args.steps
    _lib.device_status()

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region.
    # Every step copies its own Q, dO, R from the host and copies O and all five gradients back.  The
    # three legs run on three streams with two sets of buffers, so that the copy-in of step n+1 and the
    # copy-out of step n-1 overlap the kernels of step n, as a training loop with a prefetching loader does.
    hQ, hdO, hR = (t.cpu().pin_memory() for t in (Q, dO, R))
    s_in, s_out, s_main = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.current_stream(dev)
    dev_in = [[torch.empty_like(t) for t in (Q, dO, R)] for _ in range(2)]
    outs_host = [None, None]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]
    for ev in in_free + out_done:
        ev.record(s_main)

    def e2e_step(n):
        b = n & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[b])                      # the kernels that read this buffer set are done
            for d, h in zip(dev_in[b], (hQ, hdO, hR)):
                d.copy_(h, non_blocking=True)
            in_ready[b].record(s_in)
        s_main.wait_event(in_ready[b])
        q = dev_in[b][0].detach().requires_grad_(True)
        r = dev_in[b][2].detach().requires_grad_(True)
        k, u, v = (t.detach().requires_grad_(True) for t in (K, U, V))
        o = fm.flash_mhf(q, k, u, v, r)
        o.backward(dev_in[b][1])
        dp.allreduce_weight_grads([k.grad, u.grad, v.grad])
        res = (o.detach(), q.grad, r.grad, k.grad, u.grad, v.grad)
        in_free[b].record(s_main)
        out_ready[b].record(s_main)
        if outs_host[b] is None:
            outs_host[b] = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in res]
        with torch.cuda.stream(s_out):
            s_out.wait_event(out_ready[b])
            for hst, t in zip(outs_host[b], res):
                hst.copy_(t, non_blocking=True)
            out_done[b].record(s_out)
        s_main.wait_event(out_done[b ^ 1])                   # results of step n-1 are on the host before their
        keep[b] = res                                        # device tensors (dropped here) can be reused
        return res

    e2e_steps = max(20, args.steps // 4) if not args.small else 4
    for n in range(2):
        e2e_step(n)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_main)
    res = None
    for n in range(e2e_steps):
        res = e2e_step(n)
    s_main.wait_event(out_done[0])
    s_main.wait_event(out_done[1])
    e1.record(s_main)
    sync_all()
    _lib.device_status()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in (hQ, hdO, hR))
    d2h = sum(t.numel() * t.element_size() for t in outs_host[0])

    ms, e2e_ms = dp.max_over_ranks(ms, dev), dp.max_over_ranks(e2e_ms, dev)
    fl = alg_flops(B, S, H, Dh, E, De) * world
    value = fl / (ms * 1e-3) / 1e12
    e2e_value = fl / (e2e_ms * 1e-3) / 1e12

    train = infer = prefill = decode = None
    if not args.no_lm and not args.small:
        from flashmhf_b200 import lm
        del res, outs_host, hQ, hdO, hR, keep, dev_in
        torch.cuda.empty_cache()
        train = lm_train_370m(args, rank, world, dev, sync_all)
        torch.cuda.empty_cache()
        infer = lm_inference("128M", lm.LMConfig.lm_128m(), 8, 2048, "logits", args, rank, world, dev, sync_all)
        prefill = lm_inference("1.3B", lm.LMConfig.lm_1p3b(), args.prefill_rows, 8192, "prefill", args, rank, world, dev, sync_all)
        decode = lm_decode("1.3B", lm.LMConfig.lm_1p3b(), 64, 4096, args, rank, world, dev, sync_all)

    if rank == 0:
        peaks = measured_peaks()
        per_kernel = {k: statistics.mean(v) for k, v in kernel_ms.items()}
        alg = {"fwd_kernel": 6, "bwd_dq_kernel": 6, "bwd_dw_kernel": 6}  # algorithmic FLOPs / (T*H*I*d_h): 3 GEMM passes each
        top = max((k for k in per_kernel if k in alg), key=lambda k: per_kernel[k])
        achieved = alg_flops(B, S, H, Dh, E, De, passes=alg[top]) / (per_kernel[top] * 1e-3) / 1e12
        peak_kind, peak = choose_peak(peaks, ms * 1e-3 * args.steps)
        traffic, traffic_note = recorded_traffic(top, w)
        roof = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak,
                "peak_source": f"{peaks['source']} cuBLAS bf16, {peak_kind} (timed region {ms * 1e-3 * args.steps:.2f} s)",
                "frac_of_burst": achieved / peaks["burst"], "frac_of_sustained": achieved / peaks["sustained"],
                "traffic": traffic, "traffic_note": traffic_note,
                "traffic_unit": "bytes of DRAM read+write per launch (one ncu capture of these kernel sources)",
                "kernel_ms": per_kernel,
                "kernel_frac_of_burst": {k: alg_flops(B, S, H, Dh, E, De, passes=alg[k]) / (per_kernel[k] * 1e-3) / 1e12 /
                                         peaks["burst"] for k in per_kernel if k in alg},
                "whole_step_frac_of_nominal_2250": value / world / NOMINAL_BF16_TFLOPS,
                "whole_step_frac_of_burst": value / world / peaks["burst"],
                "whole_step_frac_of_sustained": value / world / peaks["sustained"]}
        out = {
            "metric": "flashmhf_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, world),
            "tokens_per_s": B * S * world / (ms * 1e-3),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "pipeline": "copy-in, kernels and copy-out of consecutive steps overlap (3 streams, 2 buffer sets)"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roof,
        }
        if train is not None:
            train["mfu_of_measured_sustained"] = train["model_tflops_per_gpu"] / peaks["sustained"]
            out["train_370m"] = train
            out["infer_128m"] = infer
            out["prefill_1p3b"] = prefill
            out["decode_1p3b"] = decode
        if not args.no_cpu_baseline and world == 1:
            out["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(out))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
