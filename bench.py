#!/usr/bin/env python
"""MoE-layer throughput benchmark (tokens/s, forward + backward) on N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c5] [--impl reference]

One step = one forward + backward pass of the MoE layer over one batch of seeded synthetic
tokens (N(0,1) activations, N(0,0.02^2) weights, N(0,1e-2^2) upstream gradient), through the
C ABI of include/tmt_moe.h. Default workload: config 5, the largest one (131072 tokens per
GPU, dim 2048, 64 experts, top-4, expert FFN 2048->2048->2048, fp32 router), the one the
1/2/4/8-GPU metric is quoted on; at N > 1 the experts are partitioned over the ranks (expert
parallel, weak scaling: tokens per GPU fixed). Rank 0 prints ONE JSON line.

`value` is timed with the inputs resident in HBM; `e2e` runs the same step through the
host-buffer entry point (pinned host X / dY in, Y / dX / statistics out, copies inside the
timed region). `roofline` is the grouped expert GEMM kernel against the measured bf16 peak;
`cpu_baseline` times the CPU oracle (a port of the reference's math; the reference itself has
no CPU path) on a bounded token sample of the same workload. `--impl reference` prints that
CPU timing as its own line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "test-model-thing-cuda_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

CONFIGS = {
    "c1": dict(T=2048, D=512, H=1024, E=4, K=2, router_f32=True, backward=False,
               desc="config 1: tokens=2048 dim=512 experts=4 topk=2 ffn 512-1024-512, forward only, fp32 router"),
    "c2": dict(T=16384, D=1024, H=4096, E=8, K=2, router_f32=False, backward=True,
               desc="config 2: tokens=16384 dim=1024 experts=8 topk=2 ffn 1024-4096-1024, fwd+bwd, aux 0.1 + z-loss"),
    "c3": dict(T=64, D=1024, H=2048, E=16, K=2, router_f32=False, backward=False, nvfp4=True, decode_steps=256,
               desc="config 3: NVFP4 decode, 64 streams x 1 position per decode step, 256 decode steps per step, "
                    "dim=1024 experts=16 topk=2 ffn 1024-2048-1024, forward only, bf16 router"),
    "c4": dict(T=65536, D=1024, H=4096, E=16, K=2, router_f32=False, backward=True, zipf=True,
               desc="config 4: tokens=65536 dim=1024 experts=16 topk=2 ffn 1024-4096-1024, Zipf(1.2) logit bias, fwd+bwd"),
    "c5": dict(T=131072, D=2048, H=2048, E=64, K=4, router_f32=True, backward=True,
               desc="config 5: tokens=131072 per GPU dim=2048 experts=64 topk=4 ffn 2048-2048-2048, fp32 router, fwd+bwd"),
}
AUX, ZCOEF = 0.1, 0.001
L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms. Samples are kept with their
    timestamps; stop(t0, t1) reports those taken inside the timed region [t0, t1] (wall clock)."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, t0, t1):
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": "timed region"}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 9 and parts[1].isdigit():
                    try:
                        ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    except ValueError:
                        ts = None
                    rows.append((ts, parts))
        os.unlink(self.path)
        inside = [p for ts, p in rows if ts is not None and t0 - 0.05 <= ts <= t1 + 0.05]
        if len(inside) >= 2:
            use = inside
        else:       # region shorter than two sampling periods: everything from one second before it to its end
            use = [p for ts, p in rows if ts is not None and t0 - 1.0 <= ts <= t1 + 0.05] or [p for _, p in rows[-3:]]
            out["window"] = "last second before and during the timed region (region shorter than two sampling periods)"
        if not use:
            return out
        out["samples"] = len(use)
        out["sm_mhz"] = statistics.median(int(r[1]) for r in use)
        out["sm_max_mhz"] = max(int(r[2]) for r in use)
        try:
            out["power_w_max"] = max(float(r[3]) for r in use)
        except ValueError:
            pass
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for i, n in enumerate(names):
            if any(r[5 + i].lower().startswith("active") for r in use):
                out["reasons"].append(n)
        return out


def cpu_sample_tokens(cfg):
    """Token sample whose forward+backward costs the oracle roughly 4e11 flops (10-30 s of host work)."""
    per_token = 12.0 * cfg["K"] * cfg["D"] * cfg["H"] if cfg["backward"] else 4.0 * cfg["K"] * cfg["D"] * cfg["H"]
    s = int(4e11 / per_token)
    s = max(256, min(cfg["T"], s // 256 * 256))
    return s


def run_cpu(cfg, host, sample, steps, warmup):
    """Times the CPU oracle on the first `sample` tokens. Returns (tokens/s, threads, seconds per step)."""
    from oracle import oracle as O
    O.build()
    threads = O.host_threads()
    X = host["X"][:sample]
    dY = host["dY"][:sample]
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        f = O.forward(X, host["Wr"], host["Wup"], host["Wdown"], cfg["K"], bias=host.get("bias"), threads=threads)
        if cfg["backward"]:
            O.backward(f, dY, AUX, ZCOEF, threads=threads)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return sample / sec, threads, sec


def make_device_data(cfg, T, local_experts, rank, torch):
    """Seeded synthetic tensors created on the GPU (bf16 as int16 views for the C ABI)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(1234 + rank)
    D, H, E = cfg["D"], cfg["H"], cfg["E"]

    def bf(shape, std):
        return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * std).to(torch.bfloat16)
    d = {}
    d["X"] = bf((T, D), 1.0)
    d["dY"] = bf((T, D), 1e-2)
    gw = torch.Generator(device="cuda")
    gw.manual_seed(99)                      # router identical on every rank (replicated parameter)
    wr = torch.randn((E, D), generator=gw, device="cuda", dtype=torch.float32) * 0.02
    d["Wr"] = wr if cfg["router_f32"] else wr.to(torch.bfloat16)
    # expert weights: one chunk per local expert, generated in slices to bound temporary memory
    d["Wup"] = torch.empty((local_experts, H, D), device="cuda", dtype=torch.bfloat16)
    d["Wdown"] = torch.empty((local_experts, D, H), device="cuda", dtype=torch.bfloat16)
    for e in range(local_experts):
        d["Wup"][e] = bf((H, D), 0.02)
        d["Wdown"][e] = bf((D, H), 0.02)
    d["dWr"] = torch.zeros((E, D), device="cuda", dtype=torch.float32)
    d["dWup"] = torch.zeros((local_experts, H, D), device="cuda", dtype=torch.float32)
    d["dWdown"] = torch.zeros((local_experts, D, H), device="cuda", dtype=torch.float32)
    d["Y"] = torch.zeros((T, D), device="cuda", dtype=torch.bfloat16)
    d["dX"] = torch.zeros((T, D), device="cuda", dtype=torch.bfloat16)
    if cfg.get("nvfp4"):
        import tmt_moe_b200 as M
        n = cfg["decode_steps"]
        d["Xsteps"] = bf((n, T, D), 1.0)                     # a fresh batch of 64 rows for every decode step
        d["q"] = {"up": [], "down": [], "keep": []}
        for e in range(local_experts):
            for name, W in (("up", d["Wup"][e]), ("down", d["Wdown"][e])):
                rows, cols = W.shape
                packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device="cuda")
                scales = torch.empty((rows, cols // 16), dtype=torch.uint8, device="cuda")
                ts = M.quantize_nvfp4(W, rows, cols, packed, scales)
                d["q"][name].append((packed, scales, ts, rows, cols))
                d["q"]["keep"] += [packed, scales]
    return d


def bench_adamw(args):
    """Multi-tensor AdamW (include/tmt_adamw.h) over config 5's parameters: 64 experts x (2048x2048 up + 2048x2048 down)
    and the 64x2048 router. One step = norm + clip + update + bf16 copies + gradient clearing. HBM-bound: 38 bytes per
    parameter (norm pass: read grad 4; update pass: read master, m, v, grad 16, write master, m, v 12, bf16 copy 2, cleared
    gradient 4)."""
    import numpy as np
    import torch
    import tmt_moe_b200 as M
    from oracle import oracle as O
    c5 = CONFIGS["c5"]
    sizes = [c5["H"] * c5["D"]] * c5["E"] + [c5["D"] * c5["H"]] * c5["E"] + [c5["E"] * c5["D"]]
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    mk = lambda n, std: torch.randn(n, generator=g, device="cuda", dtype=torch.float32) * std
    w = [mk(n, 0.02) for n in sizes]
    m = [mk(n, 1e-3) for n in sizes]
    v = [mk(n, 1e-3) ** 2 for n in sizes]
    gr = [mk(n, 1e-2) for n in sizes]
    work = [torch.zeros(n, dtype=torch.bfloat16, device="cuda") for n in sizes]
    opt = M.AdamW(sizes)
    hyp = dict(clip=1.0, lr=3e-4, b1=0.9, b2=0.999, eps=1e-8, wd=0.01, zero_grads=True)
    sampler = ClockSampler(0)
    sampler.start()
    for i in range(max(args.warmup, 3)):
        opt.step(w, m, v, gr, work, None, step=i + 1, **hyp)
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    wall0 = time.time()
    for i, (a, b) in enumerate(evs):
        a.record()
        opt.step(w, m, v, gr, work, None, step=10 + i, **hyp)
        b.record()
    torch.cuda.synchronize()
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1)
    ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    n = sum(sizes)
    pk, kind = peaks()
    gbs = 38.0 * n / (ms * 1e-3) / 1e9
    line = dict(metric="adamw_parameters_per_s", unit="parameters/s", n_gpus=1, steps=args.steps, warmup=max(args.warmup, 3),
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32 (bf16 working copies)", data="synthetic",
                value=n / (ms * 1e-3), ms_per_step=ms,
                config={"workload": "AdamW step over config 5's parameters: 128 expert matrices of 2048x2048 and the 64x2048 router "
                                    "(%d parameters), global-norm clipping on" % n,
                        "l2": "working set larger than L2 (no flush needed)"},
                clocks=clocks, gpu_launches=3 * args.steps,
                roofline={"bound": "hbm", "kernel": "adamw_kernel + sumsq_kernel", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": gbs / pk["hbm_gbs"], "traffic": None, "peak_kind": kind, "bytes_per_parameter": 38})
    if not args.no_cpu_baseline:
        sample = 1 << 22
        hw, hm, hv, hg = (x[0][:sample].cpu().numpy() for x in (w, m, v, gr))
        t0 = time.perf_counter()
        O.sumsq([hg])
        O.adamw(hw, hm, hv, hg, 1.0, 3e-4, 0.9, 0.999, 1e-8, 0.01, 5)
        sec = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": sample / sec, "unit": "parameters/s", "cores": 1, "kind": "port",
                                "sample": "first %d parameters of one expert matrix, norm + update, one thread (%.2f s)" % (sample, sec)}
    print(json.dumps(line), flush=True)


def bench_ln(args):
    """LayerNorm (include/tmt_norm.h) on config 5's activations (131072 x 2048 bf16), forward + backward per step.
    HBM-bound: forward reads X and writes Y (4 bytes per element), backward reads X and dY and writes dX (6 bytes)."""
    import numpy as np
    import torch
    import tmt_moe_b200 as M
    from oracle import oracle as O
    c5 = CONFIGS["c5"]
    rows, D = c5["T"], c5["D"]
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda")
    g.manual_seed(9)
    X = (torch.randn((rows, D), generator=g, device="cuda") * 1.5 + 0.3).to(torch.bfloat16)
    dY = (torch.randn((rows, D), generator=g, device="cuda") * 1e-2).to(torch.bfloat16)
    gamma = 1 + 0.1 * torch.randn(D, generator=g, device="cuda")
    beta = 0.1 * torch.randn(D, generator=g, device="cuda")
    Y, dX = torch.empty_like(X), torch.empty_like(X)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    dG, dB = torch.empty(D, device="cuda"), torch.empty(D, device="cuda")
    scratch = torch.empty(M.ln_backward_scratch_bytes(rows, D) // 4, device="cuda")

    def step():
        M.ln_forward(X, gamma, beta, Y, mean, rstd)
        M.ln_backward(X, dY, gamma, mean, rstd, dX, dG, dB, scratch)
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ef = [torch.cuda.Event(enable_timing=True) for _ in range(3 * args.steps)]
    wall0 = time.time()
    for i in range(args.steps):
        ef[3 * i].record()
        M.ln_forward(X, gamma, beta, Y, mean, rstd)
        ef[3 * i + 1].record()
        M.ln_backward(X, dY, gamma, mean, rstd, dX, dG, dB, scratch)
        ef[3 * i + 2].record()
    torch.cuda.synchronize()
    wall1 = time.time()
    clocks = sampler.stop(wall0, wall1)
    fwd = sum(ef[3 * i].elapsed_time(ef[3 * i + 1]) for i in range(args.steps)) / args.steps
    bwd = sum(ef[3 * i + 1].elapsed_time(ef[3 * i + 2]) for i in range(args.steps)) / args.steps
    pk, kind = peaks()
    n = rows * D
    gb_f, gb_b = 4.0 * n / (fwd * 1e-3) / 1e9, 6.0 * n / (bwd * 1e-3) / 1e9
    line = dict(metric="layernorm_rows_per_s_fwd_bwd", unit="rows/s", n_gpus=1, steps=args.steps, warmup=max(args.warmup, 3),
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16 (fp32 statistics)", data="synthetic",
                value=rows / ((fwd + bwd) * 1e-3), ms_per_step=fwd + bwd,
                config={"workload": "LayerNorm forward + backward on %d x %d bf16 activations (config 5's layer input)" % (rows, D),
                        "l2": "working set larger than L2 (no flush needed)"},
                clocks=clocks, gpu_launches=3 * args.steps,
                roofline={"bound": "hbm", "kernel": "ln_bwd_kernel (forward beside it)", "achieved": gb_b, "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": gb_b / pk["hbm_gbs"], "traffic": None, "peak_kind": kind,
                          "forward": {"ms": fwd, "achieved": gb_f, "frac": gb_f / pk["hbm_gbs"]}, "backward_ms": bwd})
    if not args.no_cpu_baseline:
        sample = 2048
        hx, hdy = X[:sample].cpu().view(torch.int16).numpy().view(np.uint16), dY[:sample].cpu().view(torch.int16).numpy().view(np.uint16)
        hg, hb = gamma.cpu().numpy(), beta.cpu().numpy()
        t0 = time.perf_counter()
        _, hm, hr = O.ln_forward(hx, hg, hb)
        O.ln_backward(hx, hdy, hg, hm, hr)
        sec = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": sample / sec, "unit": "rows/s", "cores": 1, "kind": "port",
                                "sample": "first %d rows, forward + backward, one thread (%.2f s)" % (sample, sec)}
    print(json.dumps(line), flush=True)


def bench_ref4(args):
    """The reference's own GPU implementation (tmt-cuda/src/moe.cu recompiled for sm_100a, cuBLAS per expert; oracle/_ref)
    beside this library on the same B200, same seeded inputs, same method: the reference's harness shape (profile.cu:
    dim 1280, top-2, 15 warm-ups, 60 iterations between two CUDA events) in reference mode (one dim x dim matrix per
    expert, SiLU in combine) with 4 experts, the most its fused router computes correctly (moe.cu:15-34), at 2048 and at
    16384 tokens. Forward alone and forward + backward."""
    import torch
    import tmt_moe_b200 as M
    from tmt_moe_b200 import synth
    from oracle import ref as R
    D, E, K = 1280, 4, 2
    warm, iters = 15, 60
    torch.cuda.set_device(0)
    want_ref = R.available()
    cases = []
    sampler = ClockSampler(0)
    sampler.start()
    wall0 = time.time()
    for N in (2048, 16384):
        host = synth.make(N, D, 0, E, K, False, seed=4242 + N, need_dy=True)
        case = {"tokens": N}
        if args.impl == "b200":
            dev = lambda a: torch.from_numpy(a.view("int16").copy()).cuda()
            X, dY, Wr, W = dev(host["X"]), dev(host["dY"]), dev(host["Wr"]), dev(host["Wup"])
            Wl = [W[e] for e in range(E)]
            Y, dX = torch.zeros_like(X), torch.zeros_like(X)
            dWr = torch.zeros((E, D), device="cuda")
            dW = torch.zeros((E, D, D), device="cuda")
            dWl = [dW[e] for e in range(E)]
            st = torch.cuda.Stream()
            torch.cuda.set_stream(st)
            moe = M.MoE(N, D, E, K, hidden=0, training=True, stream=st.cuda_stream)
            fwd = lambda: moe.forward(X, Wr, Wl, None, Y, 0.0)
            bwd = lambda: moe.backward(dY, Wr, Wl, None, dWr, dWl, None, dX, 0.01, 0.001)
            for _ in range(warm):
                fwd(); bwd()
            torch.cuda.synchronize()
            a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
            for _ in range(iters):
                fwd()
            b.record()
            for _ in range(iters):
                fwd(); bwd()
            c.record()
            torch.cuda.synchronize()
            if moe.device_status() != 0:
                raise SystemExit("device status %d" % moe.device_status())
            case["ms_fwd"], case["ms_fwd_bwd"] = a.elapsed_time(b) / iters, b.elapsed_time(c) / iters
            case["launches_per_fwd_bwd"] = None
            l0 = moe.launch_count
            fwd(); bwd()
            case["launches_per_fwd_bwd"] = moe.launch_count - l0
            torch.cuda.synchronize()
            moe.close()
            torch.cuda.set_stream(torch.cuda.default_stream())
        if want_ref:
            rf, rfb = R.time_moe(host["X"], host["Wr"], host["Wup"], K, host["dY"], 0.01, 0.001, warm, iters)
            case["reference_gpu"] = {"ms_fwd": rf, "ms_fwd_bwd": rfb, "kind": "reference recompiled sm_100a (cuBLAS per expert)"}
            if "ms_fwd" in case:
                case["speedup_fwd"], case["speedup_fwd_bwd"] = rf / case["ms_fwd"], rfb / case["ms_fwd_bwd"]
        cases.append(case)
    clocks = sampler.stop(wall0, time.time())
    big = cases[-1]
    work = ("reference mode (one dim x dim matrix per expert, SiLU in combine): dim=1280 experts=4 topk=2, tokens 2048 and 16384, "
            "fwd and fwd+bwd, %d warm-ups + %d iterations between CUDA events; value quoted at 16384 tokens" % (warm, iters))
    base = dict(metric="moe_layer_tokens_per_s_fwd_bwd", unit="tokens/s", n_gpus=1, steps=iters, warmup=warm, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                config={"workload": work, "l2": "working set of the 16384-token case larger than L2; 2048-token case not flushed "
                                                 "(the reference's own harness does not flush)"}, clocks=clocks)
    if args.impl == "reference":
        if not want_ref:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libtmt_ref.so is not built"}), flush=True)
            return
        ms = big["reference_gpu"]["ms_fwd_bwd"]
        print(json.dumps(dict(base, impl="reference", value=big["tokens"] / (ms * 1e-3), ms_per_step=ms, cases=cases,
                              gpu_launches=0)), flush=True)
        return
    ms = big["ms_fwd_bwd"]
    print(json.dumps(dict(base, value=big["tokens"] / (ms * 1e-3), ms_per_step=ms, cases=cases,
                          reference_gpu=big.get("reference_gpu"),
                          gpu_launches=(big["launches_per_fwd_bwd"] or 0) * iters)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="c5", choices=sorted(CONFIGS) + ["adamw5", "ln5", "ref4"],
                    help="c1..c5: the MoE layer workloads; adamw5: the optimizer step over config 5's expert and router parameters "
                         "(the component after the layer's backward pass); ln5: the LayerNorm in front of the layer on config 5's "
                         "activations, forward + backward. Both print their own metric, not the headline. ref4: the reference's own GPU "
                         "implementation (recompiled for sm_100a) timed beside this library in reference mode, 4 experts")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (not the headline workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="config c3: run the decode loop eagerly (per-phase times become available)")
    ap.add_argument("--gemm-cycles", action="store_true",
                    help="measurement only: print (stderr) where the TMA, MMA and epilogue threads of the last GEMM launches spent their cycles")
    ap.add_argument("--gemm", default="2cta", choices=["2cta", "1cta"],
                    help="grouped GEMM kernel: CTA pairs on 256x256 tiles (default) or one CTA per 128x256 tile")
    ap.add_argument("--ep-transport", default="peer", choices=["peer", "nccl", "dma"],
                    help="N > 1: rows move by peer loads/stores inside the gather/scatter kernels, by NCCL send/recv, or as "
                         "peer-to-peer copies of the copy engines in expert waves under the GEMMs")
    args = ap.parse_args()
    if args.config == "adamw5":
        return bench_adamw(args)
    if args.config == "ln5":
        return bench_ln(args)
    if args.config == "ref4":
        return bench_ref4(args)
    cfg = dict(CONFIGS[args.config])
    if args.tokens:
        cfg["T"] = args.tokens
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.gemm_cycles:
        os.environ["TMT_MOE_GEMM_CYCLES"] = "1"
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    T, D, H, E, K = cfg["T"], cfg["D"], cfg["H"], cfg["E"], cfg["K"]
    workload = cfg["desc"] + ("" if not args.tokens else " [tokens overridden to %d]" % args.tokens)
    base = {"metric": "moe_layer_tokens_per_s_fwd_bwd" if cfg["backward"] else "moe_layer_tokens_per_s_fwd",
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic"}

    if args.impl == "reference":
        # The reference ships only a GPU path; its math restated on the host (oracle/) is what this arm times.
        if rank != 0:
            return
        import numpy as np
        from tmt_moe_b200 import synth
        sample = 2048 if cfg.get("nvfp4") else min(cpu_sample_tokens(cfg), 1024 if args.steps + args.warmup > 4 else 1 << 30)
        host = synth.make(sample, D, H, E, K, cfg["router_f32"], seed=1234, need_dy=True)
        if cfg.get("zipf"):
            host["bias"] = synth.zipf_bias(E, 2.0)
        tps, threads, sec = run_cpu(cfg, host, sample, args.steps, args.warmup)
        line = dict(base, impl="reference", value=tps, ms_per_step=sec * 1e3,
                    config={"workload": workload, "sample_tokens_per_step": sample},
                    cpu_baseline={"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                                  "sample": "first %d tokens of the workload per step, all %d experts" % (sample, E)},
                    e2e={"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    gpu_launches=0)
        print(json.dumps(line), flush=True)
        return

    if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
        os.environ.pop("NCCL_DEBUG")               # keep NCCL's version banner out of the one-line output
    import torch
    import tmt_moe_b200 as M
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        import datetime
        # a rank that failed leaves the others in a collective: give up after five minutes, not after the default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()                        # nvidia-smi needs about a second before its first sample
    local_experts = E // world
    work_stream = torch.cuda.Stream()          # a real stream (not the legacy default), so the decode loop can be graph-captured
    torch.cuda.set_stream(work_stream)
    d = make_device_data(cfg, T, local_experts, rank, torch)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    moe = M.MoE(T, D, E, K, hidden=H, router_dtype=M.F32 if cfg["router_f32"] else M.BF16,
                training=cfg["backward"], device=local_rank, host_io=(not args.no_e2e and not cfg.get("nvfp4")),
                gemm_impl=M.GEMM_TCGEN05_2CTA if args.gemm == "2cta" else M.GEMM_TCGEN05,
                stream=stream, ep_world=world, ep_rank=rank,
                ep_transport={"peer": M.EP_PEER, "nccl": M.EP_NCCL, "dma": M.EP_DMA}[args.ep_transport])
    if cfg.get("zipf"):
        from tmt_moe_b200 import synth
        moe.set_router_bias(synth.zipf_bias(E, 2.0))
    if world > 1:
        moe.ep_init_torch(dist)
    Wup = [d["Wup"][e] for e in range(local_experts)]
    Wdown = [d["Wdown"][e] for e in range(local_experts)]
    dWup = [d["dWup"][e] for e in range(local_experts)]
    dWdown = [d["dWdown"][e] for e in range(local_experts)]

    graph_info = {}
    launches0_per_loop = 0
    if cfg.get("nvfp4"):
        xs = [d["Xsteps"][i] for i in range(cfg["decode_steps"])]

        def decode_loop():
            for x in xs:
                moe.forward_nvfp4(x, d["Wr"], d["q"]["up"], d["q"]["down"], d["Y"], 0.0)
        decode_loop()                        # expands the weights once, allocates the scratch
        torch.cuda.synchronize()
        lc = moe.launch_count
        decode_loop()
        launches0_per_loop = moe.launch_count - lc      # kernels one replay of the captured loop launches
        step = decode_loop
        try:                                 # the launch-bound loop as one CUDA graph on the handle's stream
            if args.no_graph:
                raise RuntimeError("eager loop requested (--no-graph)")
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=work_stream):
                decode_loop()
            g.replay()
            torch.cuda.synchronize()
            if moe.device_status() != 0:
                raise RuntimeError("device status after graph replay")
            step = g.replay
            graph_info = {"cuda_graph": True}
        except Exception as exc:             # noqa: BLE001  (capture is an optimisation, eager is the contract)
            graph_info = {"cuda_graph": False, "graph_error": str(exc)[:200]}
            torch.cuda.synchronize()
    else:
        def step():
            moe.forward(d["X"], d["Wr"], Wup, Wdown, d["Y"], 0.0)
            if cfg["backward"]:
                moe.backward(d["dY"], d["Wr"], Wup, Wdown, d["dWr"], dWup, dWdown, d["dX"], AUX, ZCOEF)

    working_set = d["X"].numel() * 2 * (2 + 2 * K)
    flush = working_set < 2 * L2_BYTES
    scrub = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda") if flush else None

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    if moe.device_status() != 0:
        raise SystemExit("device status %d after warm-up" % moe.device_status())
    launches0 = moe.launch_count
    moe.set_profile(not graph_info.get("cuda_graph", False))
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    wall0 = time.time()
    for a, b in evs:
        if scrub is not None:
            scrub.zero_()
        a.record()
        step()
        b.record()
    barrier()
    wall1 = time.time()
    phases = moe.profile(reset=True)
    moe.set_profile(False)
    if args.gemm_cycles and rank == 0:
        n, cyc = moe.gemm_cycles()
        per_step = max(1, n // (args.warmup + args.steps))
        names = ("mma_wait_full", "mma_issue", "mma_wait_acc", "tma_wait_empty", "tma_issue", "epi_wait_acc", "epi_work", "total")
        for j in range(per_step):
            c = cyc[(n - per_step + j) % cyc.shape[0]]
            c = c[c[:, 7] > 0]
            if len(c):
                print("gemm launch %d of a step (mean cycles over %d CTAs): " % (j, len(c)) +
                      ", ".join("%s %.0f" % (nm, v) for nm, v in zip(names, c.mean(axis=0))), file=sys.stderr)
    launches = moe.launch_count - launches0
    clocks = sampler.stop(wall0, wall1) if rank == 0 else None
    ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    status = moe.device_status()
    if status != 0:
        raise SystemExit("device status %d after the timed region" % status)
    tokens_per_step = T * cfg.get("decode_steps", 1)
    value = tokens_per_step * world / (ms * 1e-3)

    # ---- end to end through the host-buffer entry point (single GPU) ----
    e2e = None
    if world == 1 and not args.no_e2e and cfg.get("nvfp4"):
        # sampler loop: per decode step the 64 input rows come from pinned host memory and the 64 output rows go
        # back (the sampler needs them before it can choose the next byte), so every decode step synchronises
        n = cfg["decode_steps"]
        hXs = torch.empty((n, T, D), dtype=torch.bfloat16).pin_memory()
        hXs.copy_(d["Xsteps"])
        hY = torch.empty((T, D), dtype=torch.bfloat16).pin_memory()
        xin = torch.empty((T, D), dtype=torch.bfloat16, device="cuda")

        def host_loop():
            for i in range(n):
                xin.copy_(hXs[i], non_blocking=True)
                moe.forward_nvfp4(xin, d["Wr"], d["q"]["up"], d["q"]["down"], d["Y"], 0.0)
                hY.copy_(d["Y"], non_blocking=True)
                torch.cuda.current_stream().synchronize()
        host_loop()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            host_loop()
        e1.record()
        torch.cuda.synchronize()
        sync_ms = e0.elapsed_time(e1) / args.steps
        # the sampler session (include/tmt_sampler.h): the same rows travel every decode step, but the step is a replayed
        # graph over device-resident ring slots and the host waits once per ring round instead of once per decode step
        ring = 8
        ses = M.Sampler(T, D, H, E, K, router_dtype=M.F32 if cfg["router_f32"] else M.BF16, ring=ring, device=local_rank, seed=1)
        ses.set_weights(d["Wr"], d["q"]["up"], d["q"]["down"])
        hYs = [torch.empty((T, D), dtype=torch.bfloat16).pin_memory() for _ in range(ring)]

        def session_loop():
            for i in range(n):
                slot = i % ring
                ses.upload(slot, hXs[i])
                ses.step(slot, 0.0)
                ses.download(slot, hYs[slot])
                if slot == ring - 1:
                    ses.sync()
            ses.sync()
        session_loop()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            session_loop()
        e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        e2e = {"value": tokens_per_step / (e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": n * T * D * 2,
               "d2h_bytes_per_step": n * T * D * 2, "ms_per_step": e_ms,
               "timing": "host wall clock; sampler session, %d ring slots, every decode step uploads its %d rows from pinned host "
                         "memory and downloads its result rows, one wait per %d decode steps" % (ring, T, ring),
               "sync_every_decode_step": {"value": tokens_per_step / (sync_ms * 1e-3), "ms_per_step": sync_ms,
                                          "what": "tmt_moe_forward_nvfp4 per decode step with both copies and a synchronise"},
               "session_graphs": ses.graphs}
        ses.close()
    elif not args.no_e2e:
        # pinned host buffers first; every rank must have them before any rank enters the host steps (they contain
        # collectives under expert parallelism), so the outcome is agreed on before going on
        pinned_ok, pinned_err = 1, ""
        try:
            hX = torch.empty((T, D), dtype=torch.bfloat16).pin_memory()
            hX.copy_(d["X"])
            hdY = torch.empty((T, D), dtype=torch.bfloat16).pin_memory()
            hdY.copy_(d["dY"])
            hY = torch.empty((T, D), dtype=torch.bfloat16).pin_memory()
            hdX = torch.empty((T, D), dtype=torch.bfloat16).pin_memory()
            hstat = torch.empty(E + 1, dtype=torch.float32).pin_memory()
        except Exception as exc:             # noqa: BLE001
            pinned_ok, pinned_err = 0, str(exc)[:200]
        if dist is not None:
            flag = torch.tensor([pinned_ok], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            pinned_ok = int(flag.item())
        nbytes = T * D * 2
    if world >= 1 and not args.no_e2e and not cfg.get("nvfp4") and not pinned_ok:
        e2e = {"value": None, "unit": "tokens/s", "error": "pinned host buffers could not be allocated on every rank: " + pinned_err}
    elif not args.no_e2e and not cfg.get("nvfp4"):

        def host_step():
            # queued without waiting: the next step's uploads run under this step's GEMMs, downloads under the next compute
            moe.step_host(hX, hdY if cfg["backward"] else None, d["Wr"], Wup, Wdown, d["dWr"], dWup, dWdown,
                          hY, hdX if cfg["backward"] else None, hstat, 0.0, AUX, ZCOEF, wait=False)
        for _ in range(2):
            host_step()
        moe.host_wait()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            host_step()
        moe.host_wait()                     # every Y, dX and statistics vector of the timed steps is in host memory
        e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        if dist is not None:                # the slowest rank's time, as for the device-timed value
            t = torch.tensor([e_ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        nio = 2 if cfg["backward"] else 1
        e2e = {"value": T * world / (e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": nio * nbytes * world,
               "d2h_bytes_per_step": (nio * nbytes + (E + 1) * 4) * world, "ms_per_step": e_ms,
               "timing": "host wall clock (max over ranks) around %d queued tmt_moe_step_host_async calls and one "
                         "tmt_moe_host_wait per rank; bytes are the sum over the %d ranks" % (args.steps, world)}

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # the other ranks wait in their barrier for this report: reach ours whatever happens while the line is put together
    try:
        pk, pk_kind = peaks()
        A = T * K
        gemm_names = [n for n in phases if n.startswith("gemm_")]
        gemm_ms = sum(phases[n][0] for n in gemm_names) / args.steps
        gemm_launches = sum(phases[n][1] for n in gemm_names) // args.steps
        flops = (12.0 if cfg["backward"] else 4.0) * A * D * H          # all ranks' tokens processed by... this rank's share
        achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
        peak = pk.get("bf16_tflops_sustained", pk["bf16_tflops"])
        roofline = {"bound": "tensor", "kernel": "%s (%d launches per step)" % (
                        "gemm_tcgen05_2cta_kernel" if args.gemm == "2cta" else "gemm_tcgen05_kernel", gemm_launches),
                    "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    # dram read + write per launch, averaged over the six launches: ncu capture at 32768 tokens scaled to
                    # the full token count (activations x 4, weights fixed)
                    "traffic": 6.1e9 if (args.config == "c5" and not args.tokens and world == 1) else None,
                    "peak_kind": "%s, sustained (kernel timed inside a long step); burst %.1f" % (pk_kind, pk["bf16_tflops"]),
                    "flops_per_step": flops, "ms_per_step_in_kernel": gemm_ms}
        if cfg.get("nvfp4"):
            # weight-byte roofline: every expert hit in a decode step streams its packed weights once
            # (0.5 B per value + one scale byte per 16 values), 2*D*H values per expert; with 128 assignments over
            # 16 experts all experts are hit (P(miss) < 1e-3), plus the 64 input and output rows
            per_decode = E * 2.0 * D * H * (0.5 + 1.0 / 16) + 2 * T * D * 2
            gbs = per_decode * cfg["decode_steps"] / (ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": "decode step (router, fp4_rows_kernel up and down on the packed weights, combine)", "achieved": gbs,
                        "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "traffic": None,
                        "peak_kind": pk_kind + " copy bandwidth; algorithmic bytes are the packed weights of every expert hit, once per decode "
                                     "step (36 MB: they stay in the 126 MB L2 between decode steps, so this bounds the kernels' load path, not DRAM)",
                        "bytes_per_decode_step": per_decode}
        hbm = {}
        # dispatch also keeps X in token order for the router weight gradient when the handle trains (one more T*D*2 written)
        bytes_of = {"dispatch": (T * D * 2 + A * D * 2 + A * 12 + (T * D * 2 if cfg["backward"] else 0)), "combine": (A * D * 2 + T * D * 2),
                    "grad_dispatch": (T * D * 2 + A * D * 2), "scatter": (A * D * 2 + 2 * T * D * 2)}
        try:                                    # a label of the report only: never worth losing the line for
            waves = moe.ep_waves if world > 1 else 1
        except Exception:
            waves = int(os.environ.get("TMT_MOE_EP_WAVES", "1") or 1)
        for n, nb in bytes_of.items():
            if world > 1:
                break
            if n in phases and phases[n][0] > 0:
                gbs = nb / (phases[n][0] / phases[n][1] * 1e-3) / 1e9
                hbm[n] = {"achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                          "bytes_per_launch": nb}
        nvlink = {}
        if world > 1 and args.ep_transport == "peer":
            # Expert parallel: the row kernels move (world-1)/world of their grouped rows over NVLink and are bound by it, not
            # by HBM: rows leaving (dispatch, gradient dispatch) or entering (combine, scatter) this GPU per launch, against the
            # measured peer-copy bandwidth of this pool (770 GB/s per direction). Only kernels that run alone on the main stream
            # have a phase time: the scatter always runs on the second stream under the weight-gradient GEMMs, and with expert
            # waves so do the other three.
            out_bytes = A * D * 2 * (world - 1) / world
            for n in ("dispatch", "combine", "grad_dispatch"):
                if waves < 2 and n in phases and phases[n][0] > 0:
                    gbs = out_bytes / (phases[n][0] / phases[n][1] * 1e-3) / 1e9
                    nvlink[n] = {"achieved": gbs, "peak": 770.0, "unit": "GB/s", "frac": gbs / 770.0, "bytes_over_nvlink": out_bytes,
                                 "exposed_ms": phases[n][0] / phases[n][1]}
            nvlink["note"] = ("scatter runs on the second stream under the weight-gradient GEMMs" +
                              ("; with %d expert waves dispatch, combine and gradient dispatch run there too (no phase time)" % waves if waves > 1 else ""))
        if waves > 1:
            roofline["note"] = ("expert waves: the GEMM phases' events also bracket the main stream's waits for the waves' rows and the "
                                "row kernels running beside the CTAs, so this fraction is a lower bound of the kernels' own")
        line = dict(base, value=value, ms_per_step=ms,
                    config={"workload": workload, "tokens_per_gpu": T,
                            "parallelism": ("ep%d/%s%s" % (world, args.ep_transport, "/waves%d" % waves if waves > 1 else "")) if world > 1 else "single",
                            "l2": "L2 flushed between steps" if flush else "working set larger than L2 (no flush needed)"},
                    clocks=clocks, gpu_launches=launches if not graph_info.get("cuda_graph") else launches0_per_loop * args.steps,
                    roofline=roofline, hbm_kernels=hbm, **({"nvlink_kernels": nvlink} if nvlink else {}),
                    phases_ms_per_step={n: v[0] / args.steps for n, v in phases.items()})
        if clocks and clocks.get("sm_mhz"):
            # the step runs under the power cap, whose clock differs from box to box: ms x median SM MHz (= millions of SM
            # cycles per step) compares runs taken at different clocks
            line["mcycles_per_step"] = ms * clocks["sm_mhz"] * 1e-3
        line.update(graph_info)
        if cfg.get("nvfp4"):
            line["dtype"] = "nvfp4 weights, bf16 activations"
            line["config"]["decode_steps_per_step"] = cfg["decode_steps"]
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            from tmt_moe_b200 import synth
            sample = 2048 if cfg.get("nvfp4") else cpu_sample_tokens(cfg)
            host = synth.make(sample, D, H, E, K, cfg["router_f32"], seed=1234, need_dy=True)
            if cfg.get("zipf"):
                host["bias"] = synth.zipf_bias(E, 2.0)
            tps, threads, sec = run_cpu(cfg, host, sample, 1, 0)
            what = ("%d decode steps of %d rows as one batch, bf16 weights (same arithmetic as the dequantised ones)" % (sample // T, T)
                    if cfg.get("nvfp4") else "first %d tokens of the workload" % sample)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": "%s, all %d experts, one pass (%.1f s)" % (what, E, sec)}
        print(json.dumps(line), flush=True)
    finally:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
