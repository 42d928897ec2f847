"""Benchmark of the fused VQ-attention path: prefill TFLOP/s (+ decode tok/s) at 32K context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2_32k] [--impl ours|reference]

One step = one pass of the prefill hot path over one synthetic batch: key->code assignment,
per-block aggregates, fused attention (three kernels of libvqattn.so through the C ABI).
`value` is the algorithmic contraction TFLOP/s of the whole job (all ranks) with inputs resident in
HBM; `e2e` is the same metric through the host-buffer entry point with the host<->device copies
inside the timed region.  The CPU baseline is the PyTorch port of the reference's naive path
(oracle/torch_port.py) on a bounded sample of the same workload.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BLOCK = 128

WORKLOADS = {
    # the 32K-context headline point: config 2's Llama-7B shape at L = 32768
    "c2_32k": dict(B=1, Hq=32, Hkv=32, D=128, L=32768, W=1024, M=4, K=256, rerope=False, seed=1),
    "c2": dict(B=1, Hq=32, Hkv=32, D=128, L=8192, W=1024, M=4, K=256, rerope=False, seed=1),
    "c4": dict(B=2, Hq=32, Hkv=32, D=128, L=16384, W=512, M=4, K=512, rerope=True, seed=3),
    "c5_16k": dict(B=8, Hq=32, Hkv=8, D=128, L=16384, W=2048, M=8, K=256, rerope=False, seed=4),
}
DECODE = dict(B=16, Hq=32, Hkv=32, D=128, ctx=32768, W=1024, M=4, K=256, seed=2)  # config 3


def contraction_flops(B, Hq, L, D, W, M, K, **_):
    """4*D*B*Hq*[sum_i (i - boundary(i) + 1) + M*K*#{i: boundary(i) > 0}] (QK^T and PV per attended key)."""
    i = torch.arange(L, dtype=torch.int64)
    bd = ((i - W).clamp(min=0) // BLOCK) * BLOCK
    local = int((i - bd + 1).sum())
    far = int((bd > 0).sum()) * M * K
    return 4.0 * D * B * Hq * (local + far)


def decode_bytes(B, Hq, Hkv, D, W, M, K, cb_bytes=4, **_):
    """HBM bytes one decode step must move (bf16 window K/V, bf16 value sums, f32 counts, q/out, codebooks once per head)."""
    per_unit = 2 * W * D * 2 + M * K * D * 2 + M * K * 4 + (Hq // Hkv) * D * 2 * 2
    return B * Hkv * per_unit + Hkv * M * K * D * cb_bytes


def attention_bytes(w):
    """Algorithmic HBM bytes of one fused-attention launch: q, k, v, out once; value sums and counts of every far block."""
    B, Hq, Hkv, L, D, W, M, K = (w[k] for k in ("B", "Hq", "Hkv", "L", "D", "W", "M", "K"))
    nb = max(0, (L + BLOCK - 1) // BLOCK - W // BLOCK - 1)
    act = (2 * B * Hq * L * D + 2 * B * Hkv * L * D) * 2
    return act + B * Hkv * nb * M * K * (D * 2 + 4) + Hkv * M * K * D * 2


def stage_rooflines(w, stage_ms, peaks):
    """The two kernels in front of the attention, against the roofs that bound them (informational)."""
    B, Hkv, L, D, M, K, W = w["B"], w["Hkv"], w["L"], w["D"], w["M"], w["K"], w["W"]
    nb = max(0, (L + 127) // 128 - W // 128 - 1)                       # per-block snapshots the attention reads
    score_flops = 2.0 * B * Hkv * L * M * K * D                          # the fp32 chain that defines the codes
    agg_bytes = B * Hkv * (nb * M * K * (D * 2 + 4) + L * (D * 2 + M))   # snapshots written, values and codes read
    a_tf = score_flops / (stage_ms[0] * 1e-3) / 1e12
    g_gbs = agg_bytes / (stage_ms[1] * 1e-3) / 1e9
    return dict(
        assign_codes=dict(kernel="assign_tc_kernel", bound="tensor", achieved=a_tf, peak=peaks["tensor"], unit="TFLOP/s",
                          frac=a_tf / peaks["tensor"], note="algorithmic score FLOPs; the kernel is bound by the per-key "
                          "scan / exact re-score / residual chain between its MMAs, not by the tensor pipe"),
        build_aggregates=dict(kernel="build_aggregates_reg_kernel", bound="hbm", achieved=g_gbs, peak=peaks["hbm"], unit="GB/s",
                              frac=g_gbs / peaks["hbm"]),
    )


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops"], source="measured")
    return dict(hbm=6650.0, tensor=1590.0, source="fallback")


# ------------------------------------------------------------------------------------ inputs

def rope_tables(n, D, device):
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float64, device=device) / D))
    ang = torch.outer(torch.arange(n, dtype=torch.float64, device=device), inv)
    ang = torch.cat([ang, ang], -1)
    return ang.cos().float(), ang.sin().float()


def rotate(x, cos, sin):
    h = x.shape[-1] // 2
    xf = x.float()
    rot = torch.cat([-xf[..., h:], xf[..., :h]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


def make_inputs(w, device, seed_offset=0, dtype=torch.bfloat16):
    """q/k/v ~ N(0,1); RoPE (base 10000) applied to q/k; codebooks ~ N(0, D^-1/2). All seeded."""
    g = torch.Generator(device=device).manual_seed(w["seed"] * 1000003 + seed_offset)
    B, Hq, Hkv, L, D = w["B"], w["Hq"], w["Hkv"], w["L"], w["D"]
    q = torch.randn(B, Hq, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    k = torch.randn(B, Hkv, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    v = torch.randn(B, Hkv, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    cb = torch.randn(Hkv, w["M"], w["K"], D, generator=g, device=device, dtype=torch.float32) * D ** -0.25
    cos, sin = rope_tables(max(L, w["W"] + 2), D, device)
    q1 = rotate(q, cos[:L], sin[:L])
    k1 = rotate(k, cos[:L], sin[:L])
    if w["rerope"]:
        q2 = rotate(q, cos[w["W"] + 1], sin[w["W"] + 1])
        k3 = k
    else:
        q2, k3 = q1, k1
    return q1, q2, k1, k3, v, cb


# ------------------------------------------------------------------------------------ clocks

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, x in zip(names, r[5:9]) if x.lower().startswith("active")})
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=reasons,
                    samples=len(sm))


# ------------------------------------------------------------------------------------ CPU baseline

def cpu_baseline_run(w, seconds_budget=25.0):
    """The PyTorch CPU port of the reference's naive path on a bounded sample: heads of the workload, L capped."""
    from oracle import torch_port as tp
    torch.set_num_threads(os.cpu_count() or 1)
    Ls = min(w["L"], 8192)
    heads = 1
    ws = dict(w, B=1, Hq=heads * (w["Hq"] // w["Hkv"]), Hkv=heads, L=Ls)
    q1, q2, k1, k3, v, cb = make_inputs(ws, "cpu", dtype=torch.float32)
    flops = contraction_flops(**ws)
    t0 = time.perf_counter()
    reps = 0
    while True:
        tp.prefill(q1, q2, k1, k3, v, cb, w["W"])
        reps += 1
        el = time.perf_counter() - t0
        if el > seconds_budget * 0.4 or reps >= 32:
            break
    per = el / reps
    return dict(value=flops / per / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{heads} kv-head of {w['Hkv']}, L={Ls} of {w['L']}, fp32, {reps} reps, {per:.2f} s each "
                       f"(oracle/torch_port.py: quantize + dense-mask naive attention)",
                seconds=per, flops=flops)


# ------------------------------------------------------------------------------------ main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2_32k", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--attn-impl", default="auto", choices=["auto", "simt", "tensor"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--decode-codebook", default="bf16", choices=["bf16", "f32"],
                    help="dtype of the codebook the decode kernel scores with (bf16: the copy the prefill uses too)")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    w = WORKLOADS[args.workload]
    cfg = dict(workload=f"{args.workload}: B{w['B']} Hq{w['Hq']} Hkv{w['Hkv']} D{w['D']} L{w['L']} W{w['W']} M{w['M']}xK{w['K']} "
                        f"{'ReRoPE' if w['rerope'] else 'RoPE'} causal bf16 (per GPU)",
               sharding="(batch, kv-head) units, no collective on the hot path", l2="inputs larger than L2 (q,k,v 268 MB each)")

    if args.impl == "reference":
        if rank != 0:
            return
        vals = []
        for _ in range(max(0, args.warmup)):
            cpu_baseline_run(w, seconds_budget=5.0)
        base = None
        for _ in range(max(1, args.steps)):
            base = cpu_baseline_run(w, seconds_budget=5.0)
            vals.append(base["value"])
        v = statistics.median(vals)
        line = dict(metric="vq_attn_prefill_tflops_32k_ctx", value=v, unit="TFLOP/s", impl="reference", n_gpus=0,
                    steps=args.steps, warmup=args.warmup, ms_per_step=base["seconds"] * 1e3, higher_is_better=True,
                    scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", config=cfg,
                    cpu_baseline=dict(value=v, unit="TFLOP/s", cores=base["cores"], kind="port", sample=base["sample"]),
                    e2e=dict(value=v, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    from vqtree_b200 import api

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    q1, q2, k1, k3, v, cb = make_inputs(w, dev, seed_offset=rank)
    flops = contraction_flops(**w)
    Hkv, M, K, D, L, W = w["Hkv"], w["M"], w["K"], w["D"], w["L"], w["W"]
    nb = api.far_blocks(L, W)
    cb_act = cb.reshape(Hkv, M * K, D).to(torch.bfloat16)

    def step(events=None):
        rec = (lambda i: events[i].record()) if events else (lambda i: None)
        rec(0)
        codes = api.assign_codes(k3, cb)
        rec(1)
        cnt, vsum = api.build_aggregates(codes, v, K, nb)
        rec(2)
        out = api.prefill_from_aggregates(q1, q2, k1, k3, v, cb_act, cnt, vsum, W, impl=args.attn_impl)
        rec(3)
        return out

    for _ in range(args.warmup):
        out = step()
    torch.cuda.synchronize(dev)
    api.check_status(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(args.steps):
        out = step(evs[s])
    t_end.record()
    barrier()
    elapsed_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None
    api.check_status(dev)
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    stage_ms = [statistics.mean(e[i].elapsed_time(e[i + 1]) for e in evs) for i in range(3)]
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    peaks = load_peaks()
    attn_tflops = flops / (stage_ms[2] * 1e-3) / 1e12

    # ---- final output gather (outside the timed hot path, reported on its own) ----
    gather_ms = None
    if dist is not None:
        full = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        dist.all_gather_into_tensor(full, out)
        g1.record()
        torch.cuda.synchronize(dev)
        gather_ms = g0.elapsed_time(g1)
        del full

    # ---- end to end through the host-buffer entry point ----
    e2e = None
    if not args.no_e2e:
        host = [t.cpu().pin_memory() for t in (q1, k1, v)]
        hq1, hk1, hv = host
        hq2 = hq1 if q2 is q1 else q2.cpu().pin_memory()
        hk3 = hk1 if k3 is k1 else k3.cpu().pin_memory()
        hout = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
        h2d = sum(t.numel() * t.element_size() for t in {id(t): t for t in (hq1, hq2, hk1, hk3, hv)}.values())
        d2h = hout.numel() * hout.element_size()
        del q1, q2, k1, k3, v, out
        torch.cuda.empty_cache()
        n_e2e = max(2, min(args.steps, 5))
        for _ in range(2):
            api.vq_attention_prefill_host(hq1, hq2, hk1, hk3, hv, cb, W, device=dev, out=hout)
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            api.vq_attention_prefill_host(hq1, hq2, hk1, hk3, hv, cb, W, device=dev, out=hout)
        torch.cuda.synchronize(dev)
        el = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([el], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            el = float(t.item())
        e2e = dict(value=world * flops / (el / n_e2e) / 1e12, unit="TFLOP/s", h2d_bytes_per_step=h2d,
                   d2h_bytes_per_step=d2h, ms_per_step=el / n_e2e * 1e3, steps=n_e2e)
        del host, hq1, hq2, hk1, hk3, hv
    torch.cuda.empty_cache()

    # ---- decode (config 3): tok/s of the attention layer alone ----
    decode = None
    if not args.no_decode:
        d = DECODE
        g = torch.Generator(device=dev).manual_seed(d["seed"] * 1000003 + rank)
        MK = d["M"] * d["K"]
        nbuf = 4  # rotate among buffers whose total size exceeds L2 so the traffic is real HBM traffic
        rn = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32)
        bufs = []
        far_keys = d["ctx"] - d["W"]
        for _ in range(nbuf):
            codes = torch.randint(0, d["K"], (d["B"], d["Hkv"], far_keys, d["M"]), generator=g, device=dev).to(torch.uint8)
            cntd = torch.zeros(d["B"], d["Hkv"], MK, device=dev)
            for m in range(d["M"]):
                idx = codes[..., m].long() + m * d["K"]
                cntd.scatter_add_(2, idx, torch.ones_like(idx, dtype=torch.float32))
            vsumd = (rn(d["B"], d["Hkv"], MK, d["D"]) * cntd[..., None].sqrt()).bfloat16()
            bufs.append(dict(q=rn(d["B"], d["Hq"], d["D"]).bfloat16(), k=rn(d["B"], d["Hkv"], d["W"], d["D"]).bfloat16(),
                             v=rn(d["B"], d["Hkv"], d["W"], d["D"]).bfloat16(), cnt=cntd, vsum=vsumd))
            del codes
        cbd = rn(d["Hkv"], MK, d["D"]) * d["D"] ** -0.25
        if args.decode_codebook == "bf16":
            cbd = cbd.bfloat16()  # the activation-dtype copy the prefill scores with too
        ws = api.decode_workspace(d["B"], d["Hq"], d["Hkv"], d["D"], dev)
        outd = torch.empty(d["B"], d["Hq"], d["D"], dtype=torch.bfloat16, device=dev)
        run = lambda bf: api.vq_attention_decode(bf["q"], bf["q"], bf["k"], bf["k"], bf["v"], cbd, bf["cnt"], bf["vsum"],
                                                 workspace=ws, out=outd)
        for i in range(8):
            run(bufs[i % nbuf])
        nd = 200
        barrier()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for i in range(nd):
            run(bufs[i % nbuf])
        d1.record()
        torch.cuda.synchronize(dev)
        us = d0.elapsed_time(d1) / nd * 1e3
        if dist is not None:
            t = torch.tensor([us], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        by = decode_bytes(**d, cb_bytes=2 if args.decode_codebook == "bf16" else 4)
        decode = dict(tok_s=world * d["B"] / (us * 1e-6), us_per_step=us, bytes_per_step=by, achieved_gbs=by / (us * 1e-6) / 1e9,
                      frac_hbm=by / (us * 1e-6) / 1e9 / peaks["hbm"], peak_gbs=peaks["hbm"], peak_source=peaks["source"],
                      config=f"B{d['B']} H{d['Hq']} D{d['D']} ctx{d['ctx']} W{d['W']} M{d['M']}xK{d['K']} bf16, {args.decode_codebook} codebooks")
        del bufs

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_run(w)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}

    line = dict(
        metric="vq_attn_prefill_tflops_32k_ctx", value=value, unit="TFLOP/s", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None,
        dtype="bf16", data="synthetic", config=cfg,
        stages_ms=dict(assign_codes=stage_ms[0], build_aggregates=stage_ms[1], fused_attention=stage_ms[2]),
        roofline=dict(kernel="prefill_tc4_kernel (fused attention)", bound="tensor", achieved=attn_tflops, peak=peaks["tensor"],
                      unit="TFLOP/s", frac=attn_tflops / peaks["tensor"], peak_source=f"{peaks['source']} (burst bf16 matmul)",
                      traffic=attention_bytes(w) * 1.009, traffic_unit="bytes per launch",
                      traffic_note="algorithmic bytes x 1.009, the DRAM read+write / algorithmic ratio ncu measured on the c2 "
                                   "capture (profiles/); traffic grows in proportion to the units processed",
                      flops_per_launch=flops),
        stage_rooflines=stage_rooflines(w, stage_ms, peaks),
        cpu_baseline=cpu, e2e=e2e, gpu_launches=4 * args.steps, clocks=clocks, decode=decode, gather_ms=gather_ms,
    )
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
