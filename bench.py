"""Benchmark of the LaCT TTT-layer forward at the 760M-LLM shape on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" = one forward of the causal fused post-norm TTT op
(`postnorm_block_causal_lact_swiglu_fused_kernel_triton` signature) over ONE fixed problem:
batch 8 x 4 heads (32 merged (batch x head) units), 32768 tokens, head dim = fast-weight hidden =
384, chunk 2048, bf16 q/k/v/lr, fp32 fast weights, per-chunk momentum, 5-step Newton-Schulz, L2
renorm.  Synthetic seeded inputs (no dataset exists for this op).  With N GPUs the 32 units are
partitioned into contiguous blocks of 32 / N per rank (strong scaling, no collective on the data
path); `replicas` additionally reports N independent copies of the whole problem (weak scaling).

Prints ONE JSON line (rank 0).  `value` = tokens/s with inputs resident in HBM; `e2e` = the same
through the public Python API with pinned host buffers (H2D of all inputs and D2H of the output
inside the timed region); `roofline` = the dominant kernel class against the measured bf16 peak,
with per-class DRAM traffic from the ncu table in profiles/; `train` = forward + backward of the
same workload; `cpu_baseline` = the CPU oracle (a port of the reference arithmetic) on a bounded
sample.  `--impl reference` times that CPU port alone with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

BF16 = torch.bfloat16
CFG = dict(batch=8, heads=4, L=32768, D=384, H=384, chunk=2048, ns_steps=5)
METRIC = "ttt_layer_fwd_tokens_per_s_760M_shape"
TRAFFIC_TABLE = os.path.join(ROOT, "profiles", "dram_traffic_per_launch_small_case.md")
MIN_TRAFFIC_BYTES_FWD = 3.29e9  # q, k, v, o in bf16 + lr, momentum + fast weights in and out, whole problem


def dram_traffic_table():
    """Per kernel class: (units in the capture, DRAM bytes read, DRAM bytes written) per launch, from the
    ncu table committed under profiles/ (rows `| class | units | read | write |`)."""
    table = {}
    if not os.path.exists(TRAFFIC_TABLE):
        return table
    with open(TRAFFIC_TABLE) as fh:
        for line in fh:
            cells = [c.strip().strip("`") for c in line.strip().strip("|").split("|")]
            if len(cells) < 4:
                continue
            try:
                table[cells[0]] = (int(cells[1]), float(cells[2]), float(cells[3]))
            except ValueError:
                continue
    return table


# ------------------------------------------------------------------------------------------ helpers
def algorithmic_flops(B, L, D, H, C, ns_steps):
    """Algorithmic FLOPs of one forward (recomputation and elementwise work not counted):
    apply 6DH per token, update 12DH per updated token, Newton-Schulz steps*(4 m^2 n + 2 m^3) per
    matrix, on the concatenated [2H, D] gradient and on dw1, once per updated chunk."""
    n_upd = len(range(0, L - C, C))
    ns = lambda r, c: ns_steps * (4 * min(r, c) ** 2 * max(r, c) + 2 * min(r, c) ** 3)
    per_head = 6 * D * H * L + 12 * D * H * n_upd * C + n_upd * (ns(2 * H, D) + ns(D, H))
    return B * per_head


def class_flops(name, B, D, H, C, ns_steps):
    """Algorithmic FLOPs of ONE launch of a kernel class at the benchmark shape."""
    m1, n1 = min(D, H), max(D, H)
    m2, n2 = min(2 * H, D), max(2 * H, D)
    return {
        "gemm_swiglu_gate": 4 * D * H * C * B,
        "gemm_down_proj": 2 * D * H * C * B,
        "gemm_fwgrad_pointwise": 6 * D * H * C * B,
        "gemm_fwgrad_contract": 6 * D * H * C * B,
        "gemm_ns_gram": 2 * B * (m1 * m1 * n1 + m2 * m2 * n2),
        "gemm_ns_poly": 2 * B * (m1 ** 3 + m2 ** 3),
        "gemm_ns_update": 2 * B * (m1 * m1 * n1 + m2 * m2 * n2),
        "ns_fused": ns_steps * 2 * B * (2 * (m1 * m1 * n1 + m2 * m2 * n2) + m1 ** 3 + m2 ** 3),
    }.get(name)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return dict(bf16_burst=d.get("bf16_tflops"), bf16_sustained=d.get("bf16_tflops_sustained"),
                    hbm_gbs=d.get("hbm_gbs"), source="measured")
    return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark_load_start(self):
        """Samples taken before this call (idle GPU) are left out of the summary."""
        self.t_load = time.time()

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        t_load = getattr(self, "t_load", 0.0)
        for ts, ln in self.lines:
            if ts < t_load + 0.05:
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm_sorted = sorted(sm)
        return {"sm_mhz": sm_sorted[len(sm_sorted) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(device, seed, first_unit, n_units):
    """Seeded synthetic inputs of units [first_unit, first_unit + n_units) of the benchmark problem, generated on
    `device`.  Every (batch x head) unit has its own generator, so a unit's data does not depend on how the
    problem is partitioned."""
    L, D, H = CFG["L"], CFG["D"], CFG["H"]
    out = {n: torch.empty(n_units, L, D, dtype=BF16, device=device) for n in ("q", "k", "v")}
    out.update({n: torch.empty(n_units, H, D, device=device) for n in ("w0", "w2")})
    out["w1"] = torch.empty(n_units, D, H, device=device)
    out.update({n: torch.empty(n_units, L, 1, dtype=BF16, device=device) for n in ("lr0", "lr1", "lr2")})
    out["momentum"] = torch.empty(n_units, L, 1, device=device)
    for b in range(n_units):
        g = torch.Generator(device=device).manual_seed(seed * 100003 + first_unit + b)
        rn = lambda *s: torch.randn(*s, device=device, generator=g)
        for name in ("q", "k", "v"):
            x = rn(L, D)
            if name != "v":
                x = x / x.norm(dim=-1, keepdim=True)
            out[name][b] = x.to(BF16)
        out["w0"][b] = rn(H, D) / D ** 0.5
        out["w1"][b] = rn(D, H) / H ** 0.5
        out["w2"][b] = rn(H, D) / D ** 0.5
        for name in ("lr0", "lr1", "lr2"):
            out[name][b] = torch.nn.functional.softplus(rn(L, 1) - 2.0).to(BF16)
        out["momentum"][b] = torch.sigmoid(rn(L, 1))
    return out


ARG_ORDER = ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")


def run_step(lb, t):
    return lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        *[t[n] for n in ARG_ORDER], chunk_size=CFG["chunk"], use_muon=True, momentum=t["momentum"])


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_reference_sample(steps: int, warmup: int, threads: int):
    """Times the CPU port of the reference's fused arithmetic (oracle) on a bounded sample: one batch element
    (4 heads) x the full 32768 tokens (16 chunks, 15 updates) of the benchmark workload per step; the batch
    elements are independent, so the whole problem costs 8 such samples."""
    from oracle import lact_oracle as orc
    torch.set_num_threads(threads)
    Ls, heads = CFG["L"], CFG["heads"]
    i = orc.make_inputs(heads, Ls, CFG["D"], CFG["H"], seed=0, act_dtype=BF16, lr_dtype=BF16)
    fn = lambda: orc.block_causal_lact_swiglu_fused(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"],
                                                    i["lr1"], i["lr2"], chunk_size=CFG["chunk"], use_muon=True,
                                                    momentum=i["momentum"])
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    sample = (f"1 of {CFG['batch']} batch elements ({heads} heads) x {Ls} tokens ({Ls // CFG['chunk']} chunks) per step; "
              "tokens/s of the sample = tokens/s of the whole problem (independent batch elements)")
    return Ls / dt, dt, sample


def reference_arm(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 1))
    val, dt, sample = cpu_reference_sample(steps, warmup, threads)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU port (oracle) of the reference's fused-path arithmetic; the reference tree is Python and is "
                "not present on the GPU box",
    }
    print(json.dumps(line), flush=True)


def workload_config(n):
    units = CFG["batch"] * CFG["heads"]
    return {"workload": "causal LaCT TTT layer forward, 760M-LLM shape: batch 8 x seq 32768, 4 heads of dim 384, "
                        "fast-weight hidden 384, chunk 2048, apply-then-update, momentum + Muon(5) + L2 renorm, "
                        "bf16 q/k/v/lr, fp32 fast weights",
            "signature": "postnorm_block_causal_lact_swiglu_fused_kernel_triton",
            "global_batch": CFG["batch"], "seq_len": CFG["L"], "units": units,
            "units_per_gpu": [(units + n - 1 - r) // n for r in range(n)] if n > 1 else units,
            "parallelism": f"ONE problem, its {units} (batch x head) units partitioned over {n} rank(s), no collective",
            "l2": "inputs (3.2 GB per step over all ranks; 0.4 GB per rank at 8 ranks) exceed L2; no explicit flush"}


def other_config_timings(lb, dev, steps=5):
    """Forward time of the other BASELINE configurations on seeded synthetic inputs of their shapes
    (q, k L2-normalised N(0,1), v N(0,1), lr = softplus(N(-2,1)), momentum = sigmoid(N(0,1)))."""
    g = torch.Generator(device=dev).manual_seed(5)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)

    def inputs(B, L, D, H, dtype):
        q, k, v = rn(B, L, D), rn(B, L, D), rn(B, L, D)
        q, k = q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True)
        lr = [torch.nn.functional.softplus(rn(B, L, 1) - 2.0) for _ in range(3)]
        return dict(w0=rn(B, H, D) / D ** 0.5, w1=rn(B, D, H) / H ** 0.5, w2=rn(B, H, D) / D ** 0.5, q=q.to(dtype),
                    k=k.to(dtype), v=v.to(dtype), lr=lr, mom=torch.sigmoid(rn(B, L, 1)))

    def timed(fn, tokens):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3)}

    out = {}
    # config 1: bidirectional layer, fp32, batch 1 x 4 heads of 192, 4096 tokens, Muon on (accuracy mode: FFMA contractions)
    i = inputs(4, 4096, 192, 192, torch.float32)
    out["bidirectional_fp32_b1_l4096_4x192"] = timed(
        lambda: lb.bidirectional_lact_swiglu(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], *i["lr"], use_muon=True), 4096)
    ib = {k_: (v_.to(BF16) if k_ in ("q", "k", "v") else v_) for k_, v_ in i.items()}
    out["bidirectional_bf16_b1_l4096_4x192"] = timed(
        lambda: lb.bidirectional_lact_swiglu(ib["w0"], ib["w1"], ib["w2"], ib["q"], ib["k"], ib["v"], *ib["lr"], use_muon=True), 4096)
    # config 4: NVS block, batch 4 x 4 heads of 192, update on 49152 input tokens, apply to 4096 target tokens
    i = inputs(16, 53248, 192, 192, BF16)
    t_ = lambda w: w.transpose(1, 2).contiguous()
    nw = (t_(i["w0"]), t_(i["w1"]), t_(i["w2"]))
    order = [lb.TTTOperator(0, 49152, True, False), lb.TTTOperator(49152, 53248, False, True)]
    out["nvs_b4_48views_4x192"] = timed(
        lambda: lb.fast_weight_swish_glu_weight_norm_mini_batch_apply(*nw, i["q"], i["k"], i["v"], *i["lr"], order,
                                                                      muon_update_steps=5), 4 * 53248)
    del i, nw
    # config 5: AR video layer, batch 1 x 12 heads of 128, hidden 256, 21 frames of 1560 tokens
    i = inputs(12, 32760, 128, 256, BF16)
    out["ar_video_b1_12x128_h256_21x1560"] = timed(
        lambda: lb.ar_fast_weight_swish_glu_weight_norm_mini_batch_with_momentum(
            i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], *i["lr"], 1.0, mini_batch_size=1560, update_every=1560,
            use_moun=True, num_moun_iters=5, fw_momentum=i["mom"], use_momentum=True), 32760)
    lb.synchronize_and_check()
    # layer prologue at the benchmark shape: head split + SiLU + per-head l2 norm of q, k (SiLU of v) in one pass over
    # the three column blocks of a fused [b, s, 3 n_h d] projection; HBM-bound work: bytes = read + write
    from lact_b200 import layer_ops
    b_, s_, nh_, d_ = CFG["batch"], CFG["L"], CFG["heads"], CFG["D"]
    fused = rn(b_, s_, 3 * nh_ * d_).to(BF16)
    nd = nh_ * d_
    r = timed(lambda: layer_ops.qkv_prologue(fused[..., :nd], fused[..., nd:2 * nd], fused[..., 2 * nd:], nh_), b_ * s_)
    moved = 2 * 3 * b_ * s_ * nd * 2
    r["gb_per_s"] = moved / (r["ms_per_step"] * 1e-3) / 1e9
    r["frac_of_hbm_peak"] = r["gb_per_s"] / measured_peaks()["hbm_gbs"]
    out["qkv_prologue_760M_shape"] = r
    # output side: per-head RMSNorm * silu(gate projection), head merge, residual add, one pass
    fw_x = rn(b_ * nh_, s_, d_).to(BF16)
    gate, o_attn, wn = rn(b_, s_, nd).to(BF16), rn(b_, s_, nd).to(BF16), torch.ones(d_, device=dev)
    r = timed(lambda: layer_ops.out_epilogue(fw_x, wn, nh_, gate, o_attn), b_ * s_)
    moved = 4 * b_ * s_ * nd * 2
    r["gb_per_s"] = moved / (r["ms_per_step"] * 1e-3) / 1e9
    r["frac_of_hbm_peak"] = r["gb_per_s"] / measured_peaks()["hbm_gbs"]
    out["out_epilogue_760M_shape"] = r
    return out


def train_step_timing(lb, t, dev, B, L, D, H, C, global_tokens, world, barrier, peaks, steps=3):
    """Forward + backward of the same workload (the training configuration) on this rank's units: one step =
    forward, then backward from dO ~ N(0,1) bf16 to q, k, v, lr0/1/2, momentum and the initial W0/W1/W2."""
    import torch.distributed as dist
    leaves = {n: t[n].detach().clone().requires_grad_(True) for n in ARG_ORDER + ("momentum",)}
    dO = torch.randn(B, L, D, device=dev, generator=torch.Generator(device=dev).manual_seed(99)).to(BF16)

    def step():
        for v in leaves.values():
            v.grad = None
        o = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
            *[leaves[n] for n in ARG_ORDER], chunk_size=C, use_muon=True, momentum=leaves["momentum"])
        o.backward(dO)

    step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    lb.synchronize_and_check()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item()) / steps
    n_upd = len(range(0, L - C, C))
    ns = lambda r, c: CFG["ns_steps"] * (4 * min(r, c) ** 2 * max(r, c) + 2 * min(r, c) ** 3)
    fwd = algorithmic_flops(B, L, D, H, C, CFG["ns_steps"])
    bwd = B * (12 * D * H * L + 24 * D * H * n_upd * C + 2 * n_upd * (ns(2 * H, D) + ns(D, H)))
    tf = (fwd + bwd) / (ms_step * 1e-3) / 1e12
    return {"ms_per_step": ms_step, "tokens_per_s": global_tokens / (ms_step * 1e-3), "steps": steps,
            "algorithmic_flops_per_step_per_gpu": fwd + bwd, "tflops_per_gpu": tf,
            "frac_of_bf16_peak_burst": tf / peaks["bf16_burst"],
            "config": {"seq_len": L, "chunk": C, "units_per_gpu": B},
            "note": "forward on the fused kernels keeping the per-update state and every Newton-Schulz iterate; "
                    "backward = per-chunk reverse sweep driven from the host (pre-activations recomputed)"}


# ------------------------------------------------------------------------------------------ main arm
def engine_probe():
    """Steady-state cost of one output tile of the GEMM engine by tile width and contraction length, operands
    L2-resident: c = a b^T with M = 4096 / 8192 rows and N = 37 tile widths (8 / 16 rounds of 148 tiles); the
    difference of the two launches divided by 8 is the time of one tile with the launch overhead cancelled."""
    from lact_b200 import _lib as L
    dev = torch.device("cuda", 0)
    status = torch.zeros(64, dtype=torch.int32, device=dev)

    def run(M, N, K, iters=20):
        a = torch.randn(1, M, K, device=dev).to(BF16)
        b = torch.randn(1, N, K, device=dev).to(BF16)
        c = torch.empty(1, M, N, dtype=BF16, device=dev)

        def call():
            L.check(L.lib().lact_bmm_bf16(a.data_ptr(), 0, b.data_ptr(), 0, c.data_ptr(), L.dtype_code(c), 1, M, N, K,
                                          status.data_ptr(), L.stream_ptr()), "lact_bmm_bf16")
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        if int(status[0].item()) != 0:
            raise RuntimeError("device status %d" % int(status[0].item()))
        return e0.elapsed_time(e1) / iters * 1e3

    rows = []
    for bt in (64, 128, 192, 256):
        for K in (384, 768, 2048):
            t8, t16 = run(4096, 37 * bt, K), run(8192, 37 * bt, K)
            tile_us = (t16 - t8) / 8
            rows.append(dict(tile_n=bt, K=K, us_per_tile=round(tile_us, 3), us_per_kblock=round(tile_us / (K // 64), 3),
                             steady_tflops=round(2 * 128 * bt * K / tile_us * 148 / 1e6, 1),
                             launch_fixed_us=round(t8 - 8 * tile_us, 1)))
    print(json.dumps({"engine_probe": rows, "note": "128 x tile_n output tiles, bf16 in / bf16 out, fp32 accumulate, "
                      "148 tiles per round, launches back to back in one stream"}))


def swa_bench(lb, dev, warmup, steps, batch=None, seq_len=None):
    """Causal sliding-window attention at the benchmark model's layer shape: batch 8, 32768 tokens, 12 heads of 128,
    window 2048, bf16.  FLOPs counted over the band only (4 d per (query, visible key) pair)."""
    from lact_b200 import layer_ops
    b, l, h, d, w = batch or 8, seq_len or 32768, 12, 128, 2048
    g = torch.Generator(device=dev).manual_seed(0)
    q, k, v = (torch.randn(b, l, h, d, device=dev, generator=g).to(BF16) for _ in range(3))
    for _ in range(warmup):
        layer_ops.sliding_window_attention(q, k, v, w)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        layer_ops.sliding_window_attention(q, k, v, w)
    e1.record()
    torch.cuda.synchronize()
    lb.synchronize_and_check()
    ms = e0.elapsed_time(e1) / steps
    pairs = sum(min(i + 1, w) for i in range(l))
    flops = 4.0 * pairs * d * h * b
    peaks = measured_peaks()
    # forward + backward (dq, dk, dv): algorithmic FLOPs of the backward = 2.5 x the forward's (five products for two)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    dO = torch.randn(b, l, h, d, device=dev, generator=g).to(BF16)

    def train():
        for t in leaves:
            t.grad = None
        layer_ops.sliding_window_attention(*leaves, w).backward(dO)
    for _ in range(2):
        train()
    torch.cuda.synchronize()
    n_tr = max(2, steps // 2)
    e0.record()
    for _ in range(n_tr):
        train()
    e1.record()
    torch.cuda.synchronize()
    lb.synchronize_and_check()
    ms_tr = e0.elapsed_time(e1) / n_tr
    print(json.dumps({"metric": "swa_fwd_tokens_per_s", "value": b * l / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
                      "steps": steps, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                      "tflops": flops / (ms * 1e-3) / 1e12,
                      "frac_of_bf16_peak_burst": flops / (ms * 1e-3) / 1e12 / peaks["bf16_burst"],
                      "train": {"ms_per_step": ms_tr, "steps": n_tr, "tflops": 3.5 * flops / (ms_tr * 1e-3) / 1e12,
                                "frac_of_bf16_peak_burst": 3.5 * flops / (ms_tr * 1e-3) / 1e12 / peaks["bf16_burst"]},
                      "config": {"workload": "causal sliding-window attention forward", "batch": b, "seq_len": l,
                                 "heads": h, "head_dim": d, "window": w,
                                 "l2": "q, k, v, o (%.0f MB) exceed L2" % (4 * b * l * h * d * 2 / 1e6)}}))


def token_sharded_bench(lb, dev, rank, world, warmup, steps):
    """A shape whose (batch x head) axis cannot fill several GPUs but whose chunks can: 4 units, head dim 384,
    chunks of 32 768 tokens, 4 chunks (Muon and momentum on).  Every rank holds 1 / N of each chunk's tokens; the
    time is the device time of the whole recurrence, max over ranks."""
    import torch.distributed as dist
    from lact_b200 import token_sharded as ts
    B, D, H, C, n_chunks = 4, 384, 384, 32768, 4
    L = C * n_chunks
    g = torch.Generator().manual_seed(0)
    rn = lambda *sh: torch.randn(*sh, generator=g)
    w0, w1, w2 = rn(B, H, D) / D ** 0.5, rn(B, D, H) / H ** 0.5, rn(B, H, D) / D ** 0.5
    full = {}
    for n in ("q", "k", "v"):
        x = rn(B, L, D)
        full[n] = (x / x.norm(dim=-1, keepdim=True) if n != "v" else x).to(torch.bfloat16)
    for n in ("lr0", "lr1", "lr2"):
        full[n] = torch.nn.functional.softplus(rn(B, L, 1) - 2.0)
    full["momentum"] = torch.sigmoid(rn(B, L, 1))
    mine = {n: ts.shard_tokens(x, C, world, rank).to(dev) for n, x in full.items()}
    w = [t.to(dev) for t in (w0, w1, w2)]
    run = lambda: ts.token_sharded_block_causal_lact_swiglu(*w, mine["q"], mine["k"], mine["v"], mine["lr0"],
                                                            mine["lr1"], mine["lr2"], chunk_size=C, use_muon=True,
                                                            momentum=mine["momentum"])
    for _ in range(max(3, warmup)):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    lb.synchronize_and_check()
    if rank == 0:
        print(json.dumps({"metric": "ttt_token_sharded_tokens_per_s", "value": L / (ms.item() * 1e-3), "unit": "tokens/s",
                          "n_gpus": world, "steps": steps, "ms_per_step": ms.item(), "higher_is_better": True,
                          "scaling": "strong", "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": "token-sharded causal recurrence", "units": B, "head_dim": D,
                                     "hidden": H, "chunk": C, "seq_len": L, "use_muon": True, "momentum": True,
                                     "collective": "one NCCL all-reduce of B (3 D H + 1) fp32 per chunk",
                                     "l2": "inputs (%.0f MB per rank) exceed L2" % (3 * B * L * D * 2 / world / 1e6)}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-train", action="store_true", help="skip the forward + backward timing (\"train\")")
    ap.add_argument("--no-replicas", action="store_true",
                    help="N > 1: skip the weak-scaling run of N independent copies of the whole problem (\"replicas\")")
    ap.add_argument("--other-configs", action="store_true",
                    help="also time the other BASELINE configurations (bidirectional fp32, NVS block, AR video layer) "
                         "on one GPU; reported under \"other_configs\" (not the headline metric)")
    ap.add_argument("--engine-probe", action="store_true",
                    help="micro-benchmark of the GEMM engine alone (time per output tile by tile width and "
                         "contraction length); prints its own JSON line and exits")
    ap.add_argument("--token-sharded", action="store_true",
                    help="time the token-sharded recurrence (every chunk's tokens spread over the N ranks, one "
                         "all-reduce of the partial fast-weight gradients per chunk) on a few-unit, large-chunk shape; "
                         "prints its own JSON line and exits (not the headline metric)")
    ap.add_argument("--swa", action="store_true",
                    help="time the sliding-window attention kernel (the other half of a hybrid layer) at the layer "
                         "shape of the benchmark model; prints its own JSON line and exits (not the headline metric)")
    ap.add_argument("--slabs", type=int, default=None,
                    help="slabs of (batch x head) units the end-to-end arm streams through the device (default: 8 when "
                         "the units divide)")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the batch size (profiler captures on a small case; not a headline number)")
    ap.add_argument("--seq-len", type=int, default=None, help="override the sequence length (same caveat)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    reduced = args.batch is not None or args.seq_len is not None
    if args.batch is not None:
        CFG["batch"] = args.batch
    if args.seq_len is not None:
        CFG["L"] = args.seq_len
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.engine_probe:
        if rank == 0:
            engine_probe()
        return
    warmup = args.warmup if reduced else max(3, args.warmup)
    steps = max(1, args.steps)

    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # with NCCL_DEBUG set (VERSION, WARN, ...) NCCL prints its version banner and its messages on stdout, next to
        # the one JSON line this script owes: send them to a per-process log file instead
        # (NCCL honours the file only above the VERSION level)
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", os.path.join(tempfile.gettempdir(), "lact_b200_bench_nccl.%h.%p.log"))
        dist.init_process_group("nccl", device_id=dev)
    from lact_b200 import build
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    import lact_b200
    from lact_b200 import _lib as LL
    from lact_b200 import parallel

    if args.swa:
        if rank == 0:
            swa_bench(lact_b200, dev, max(3, warmup), steps, args.batch, args.seq_len)
        return
    if args.token_sharded:
        token_sharded_bench(lact_b200, dev, rank, world, warmup, steps)
        if world > 1:
            dist.destroy_process_group()
        return

    units, L, D, H, C = CFG["batch"] * CFG["heads"], CFG["L"], CFG["D"], CFG["H"], CFG["chunk"]
    global_tokens = CFG["batch"] * L
    first, last = parallel.partition(units, world, rank)
    B = last - first  # (batch x head) units of this rank
    if B < 1:
        raise SystemExit("more ranks than (batch x head) units")
    t = make_inputs(dev, 0, first, B)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_steps(tensors, n_steps, n_warm):
        """`n_steps` steps after `n_warm` untimed ones, bracketed by barrier + synchronize; max over ranks, ms."""
        for _ in range(n_warm):
            run_step(lact_b200, tensors)
        lact_b200.synchronize_and_check()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = LL.launch_count()
        e0.record()
        for _ in range(n_steps):
            run_step(lact_b200, tensors)
        e1.record()
        barrier()
        n_launch = LL.launch_count() - l0
        ms_ = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms_, op=dist.ReduceOp.MAX)
        return float(ms_.item()), n_launch

    with ClockSampler(local_rank) as clocks:
        # nvidia-smi needs a moment to start streaming: it is started before the warm-up and its
        # samples from the warm-up onwards (GPU under the same load) are summarised
        time.sleep(0.6)
        clocks.mark_load_start()
        total_ms, launches = timed_steps(t, steps, warmup)
        if total_ms < 400.0:  # keep the GPU under the same load until a few samples exist
            t_end = time.time() + 0.4
            while time.time() < t_end:
                run_step(lact_b200, t)
            torch.cuda.synchronize()
    lact_b200.synchronize_and_check()
    ms_per_step = total_ms / steps
    value = global_tokens / (ms_per_step * 1e-3)

    # per-kernel-class durations (CUDA events around every launch, on the launching stream), second pass
    peaks = measured_peaks()
    LL.profile_enable(True)
    prof_steps = min(steps, 3)
    for _ in range(prof_steps):
        run_step(lact_b200, t)
    torch.cuda.synchronize()
    prof = LL.profile_read()
    LL.profile_enable(False)
    total_prof = sum(v[0] for v in prof.values())
    top = max((k for k in prof if class_flops(k, B, D, H, C, CFG["ns_steps"])), key=lambda k: prof[k][0])
    top_ms = prof[top][0] / prof[top][1]
    achieved = class_flops(top, B, D, H, C, CFG["ns_steps"]) / (top_ms * 1e-3) / 1e12
    flops = algorithmic_flops(B, L, D, H, C, CFG["ns_steps"])
    step_tflops = flops / (ms_per_step * 1e-3) / 1e12
    # DRAM traffic per launch from the committed ncu table (captured on a smaller case; every class's traffic
    # grows in proportion to the units per launch), and the forward's total against its algorithmic minimum
    table = dram_traffic_table()
    traffic_of = lambda k: (table[k][1] + table[k][2]) * B / table[k][0] if k in table else None
    classes = {}
    fwd_traffic = 0.0
    for k, v in sorted(prof.items()):
        f = class_flops(k, B, D, H, C, CFG["ns_steps"])
        classes[k] = {"ms_per_launch": v[0] / v[1], "launches_per_step": v[1] / prof_steps, "share": v[0] / total_prof,
                      "tflops": f / (v[0] / v[1] * 1e-3) / 1e12 if f else None, "dram_bytes_per_launch": traffic_of(k)}
        if traffic_of(k) is not None:
            fwd_traffic += traffic_of(k) * v[1] / prof_steps
    roofline = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": peaks["bf16_sustained"],
                "unit": "TFLOP/s", "frac": achieved / peaks["bf16_sustained"],
                "traffic": traffic_of(top),
                "traffic_note": "DRAM read+write bytes per launch: ncu capture of a smaller case "
                                "(profiles/dram_traffic_per_launch_small_case.md) scaled by the units per launch",
                "peak_source": peaks["source"] + " (sustained cuBLAS bf16)",
                "kernel_share_of_step": prof[top][0] / total_prof,
                "step_dram_bytes": fwd_traffic if fwd_traffic > 0 else None,
                "step_dram_bytes_min": MIN_TRAFFIC_BYTES_FWD * B / units if not reduced else None,
                "classes": classes}

    # end to end through the public API with pinned host buffers
    e2e = None
    if not args.no_e2e:
        from lact_b200.host_io import HostPipeline
        host = {k: v.cpu().pin_memory() for k, v in t.items()}
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        out_host = torch.empty(B, L, D, dtype=BF16).pin_memory()
        d2h = out_host.numel() * out_host.element_size()
        n_e2e = max(2, min(steps, 4))
        # the public call, fed from pinned host memory in slabs of (batch x head) entries so that the
        # copies of one slab overlap the kernels of another (every entry is an independent recurrence)
        n_slabs = 8 if B % 8 == 0 and B >= 32 else (4 if B % 4 == 0 and B >= 16 else (2 if B % 2 == 0 and B >= 8 else 1))
        if args.slabs is not None and args.slabs >= 1 and B % args.slabs == 0:
            n_slabs = args.slabs
        pipe = HostPipeline(lambda **kw: run_step(lact_b200, kw), host, out_host, n_slabs=n_slabs, device=dev)
        e2e_step = pipe.run

        e2e_step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(n_e2e):
            e2e_step()
        ev1.record()
        barrier()
        ems = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
        hb = torch.tensor([float(h2d), float(d2h)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
            dist.all_reduce(hb, op=dist.ReduceOp.SUM)
        e2e = {"value": global_tokens / (float(ems.item()) / n_e2e * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(hb[0].item()), "d2h_bytes_per_step": int(hb[1].item()), "steps": n_e2e,
               "slabs": n_slabs}
        del host, pipe, out_host

    others = None
    if args.other_configs and rank == 0:
        others = other_config_timings(lact_b200, dev)
    train = None
    if not args.no_train:
        train = train_step_timing(lact_b200, t, dev, B, L, D, H, C, global_tokens, world, barrier, peaks)
        if world == 1 and not reduced:
            # the training configuration's second shape: 65536 tokens in chunks of 4096 (same units)
            del t
            torch.cuda.empty_cache()
            CFG["L"] = 2 * L
            try:
                t2 = make_inputs(dev, 0, first, B)
            finally:
                CFG["L"] = L
            train["seq65536_chunk4096"] = train_step_timing(lact_b200, t2, dev, B, 2 * L, D, H, 2 * C,
                                                            CFG["batch"] * 2 * L, world, barrier, peaks, steps=2)
            del t2
            torch.cuda.empty_cache()
            t = make_inputs(dev, 0, first, B)

    # weak scaling for comparison: every rank runs the WHOLE problem on its own data
    replicas = None
    if world > 1 and not args.no_replicas and not reduced:
        del t
        torch.cuda.empty_cache()
        t_full = make_inputs(dev, 1 + rank, 0, units)
        rms, _ = timed_steps(t_full, max(2, min(steps, 5)), 2)
        rms /= max(2, min(steps, 5))
        replicas = {"value": world * global_tokens / (rms * 1e-3), "unit": "tokens/s", "ms_per_step": rms,
                    "scaling": "weak", "units_per_gpu": units,
                    "note": "N independent copies of the whole problem, one per GPU"}
        del t_full

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        val, dt, sample = cpu_reference_sample(2, 1, threads)
        cpu = {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "step_tflops_per_gpu": step_tflops, "frac_of_bf16_peak_burst": step_tflops / peaks["bf16_burst"],
            "frac_of_bf16_peak_sustained": step_tflops / peaks["bf16_sustained"],
            "algorithmic_flops_per_step_per_gpu": flops,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks.summary(),
        }
        if train is not None:
            line["train"] = train
        if replicas is not None:
            line["replicas"] = replicas
        if others is not None:
            line["other_configs"] = others
        if reduced:
            line["reduced_case"] = "batch/seq overridden for a profiler capture: not the benchmark workload"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
