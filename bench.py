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
                          frac=a_tf / peaks["tensor"], note="algorithmic score FLOPs (split_codebook + assign_tc + assign_repair "
                          "kernels); bound by the per-key scan / residual chain between its MMAs, not by the tensor pipe"),
        build_aggregates=dict(kernel="sort_block_codes_kernel + build_aggregates_sorted_kernel", bound="hbm", achieved=g_gbs,
                              peak=peaks["hbm"], unit="GB/s", frac=g_gbs / peaks["hbm"]),
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


# ------------------------------------------------------------------------------------ parity (checker, not timed)

def parity_check(api, w, tensors, cb, codes, out):
    """Sampled rows of the benchmarked launch against the naive CPU oracle, and the tensor-core codes against the
    exact kernel on every key.  Runs after the timed region; the oracle is only the checker here."""
    from oracle import sampled
    q1, q2, k1, k3, v = tensors
    B, Hkv, M, K, D, L, W = w["B"], w["Hkv"], w["M"], w["K"], w["D"], w["L"], w["W"]
    exact = api.assign_codes(k3, cb, impl="simt")
    codes_equal = bool(torch.equal(codes, exact))
    del exact
    units = [(0, 0), (B - 1, Hkv - 1)]
    codes_equal = codes_equal and sampled.codes_equal_on_ranges(codes, k3, cb, units, [(0, 256), (L - 256, L)])
    cb_seen = cb.reshape(Hkv, M * K, D).to(torch.bfloat16).float().reshape(Hkv, M, K, D)
    err, rows = sampled.prefill_rows_max_err(out, q1, q2, k1, k3, v, cb_seen, codes, W, units,
                                             sampled.row_ranges(L, W, seed=w["seed"]))
    return dict(max_abs=err, rows_checked=rows, codes_equal=codes_equal, tolerance=2e-2, ok=bool(err <= 2e-2 and codes_equal),
                oracle="oracle/vq_oracle.c naive per-query loop on sampled rows of 2 (batch, kv-head) units; codes: exact "
                       "kernel on all keys + oracle on sampled key ranges")


# ------------------------------------------------------------------------------------ the reference's own GPU kernels

REFGPU = dict(B=1, Hq=32, Hkv=32, D=128, L=32768, W=1024, M=1, K=1024)   # config 2's shape at 32K, ONE codebook of 1024


def reference_gpu_leg(dev, reps=5):
    """The reference's Triton kernels (JIT-compiled here by the installed Triton) and its PyTorch host preparation on
    the B200, and this library on the SAME tensors: the reference handles one codebook per head and no grouped-query
    heads, so the workload is config 2's shape at 32K with a single codebook of M*K = 1024 codewords (the same far
    work per query).  Returns times, the TFLOP/s of both, and the largest difference between the two outputs."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_gpu as rg
    ok, why = rg.available()
    if not ok:
        return dict(unavailable=why)
    from vqtree_b200 import api
    from vqtree_b200.fused_vq_attn import vq_attn_forward
    w = REFGPU
    try:
        ref = rg.run(w["B"], w["Hq"], w["L"], w["D"], w["K"], w["W"], reps=reps, device=dev)
    except Exception as e:  # e.g. the Triton JIT refusing the kernels on this architecture
        return dict(unavailable=f"{type(e).__name__}: {str(e)[:300]}")
    flops = contraction_flops(**w)

    def timed(fn, n):
        fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            r = fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / n, r

    args, kw = ref["kernel_args"], ref["kernel_kw"]
    # (1) the drop-in entry point on exactly the tensors the reference handed to its kernel
    compat_ms, ours = timed(lambda: vq_attn_forward(*args, **kw), reps)
    diff = float((ours.transpose(1, 2).flatten(2).float() - ref["out"].float()).abs().max())
    # (2) this library's own preparation + attention from the same raw q/k/v
    q1, q2, k1, k_vq, k_cnt, k3, v = args[0], args[1], args[2], args[3], args[4], args[5], args[6]
    cb32 = ref["inputs"]["codebook"].float()[:, None].contiguous()
    nb = api.far_blocks(w["L"], w["W"])

    def native():
        codes = api.assign_codes(k3, cb32)
        cnt, vsum = api.build_aggregates(codes, v, w["K"], nb)
        return api.prefill_from_aggregates(q1, q2, k1, k3, v, k_vq.contiguous(), cnt, vsum, w["W"])

    native_ms, ours2 = timed(native, reps)
    cnt, vsum = api.build_aggregates(api.assign_codes(k3, cb32), v, w["K"], nb)
    kern_ms, _ = timed(lambda: api.prefill_from_aggregates(q1, q2, k1, k3, v, k_vq.contiguous(), cnt, vsum, w["W"]), reps)
    diff2 = float((ours2.transpose(1, 2).flatten(2).float() - ref["out"].float()).abs().max())
    tf = lambda ms: flops / (ms * 1e-3) / 1e12
    return dict(workload=f"B{w['B']} H{w['Hq']} D{w['D']} L{w['L']} W{w['W']} one codebook of {w['K']} bf16 ReRoPE (the reference's limits: "
                         "single codebook, no grouped-query heads, L % 128 == 0)",
                reference=dict(kernels_ms=ref["kernel_ms"], host_prep_ms=ref["prep_ms"], total_ms=ref["total_ms"],
                               kernels_tflops=tf(ref["kernel_ms"]), total_tflops=tf(ref["total_ms"]),
                               what="ops/triton_fused_vq_attn.py vq_attn_forward (two Triton kernels + flashinfer merge), "
                                    "ops/attn_vq.py:352-417 host preparation (PyTorch)"),
                ours=dict(attention_ms=kern_ms, attention_tflops=tf(kern_ms), prep_plus_attention_ms=native_ms,
                          total_tflops=tf(native_ms), drop_in_call_ms=compat_ms,
                          what="attention_ms: vqattn_prefill alone; prep_plus_attention: assign (tensor-core kernel, K = 1024) + aggregates "
                               "+ attention; drop_in_call: fused_vq_attn.vq_attn_forward "
                               "on the reference's kernel arguments (format conversion included)"),
                speedup_kernels=ref["kernel_ms"] / kern_ms, speedup_total=ref["total_ms"] / native_ms,
                max_abs_diff_drop_in=diff, max_abs_diff_native=diff2, tolerance=2e-2)


# ------------------------------------------------------------------------------------ one fixed job split over the ranks

STRONG = dict(B=8, Hq=32, Hkv=8, D=128, L=131072, W=2048, M=8, K=256, decode_steps=256, seed=4)   # config 5


def strong_job(dist, dev, rank, world, barrier, L=None):
    """Config 5 as ONE job: its 64 (batch, kv-head) units are split over the ranks (64 / 32 / 16 / 8 per rank), each
    rank prefills its units through the attention module's own entry point (rotations, codes, aggregates, fused
    attention, cache state) and then generates 256 tokens from the cache.  No collective on the path; times are
    device times, maximum over ranks.  Inputs are seeded per unit, so every N computes the same job."""
    from vqtree_b200 import attn_vq, sharding
    w = dict(STRONG)
    if L:
        w["L"] = L
    B, Hq, Hkv, D, L, W, M, K = (w[k] for k in ("B", "Hq", "Hkv", "D", "L", "W", "M", "K"))
    G = Hq // Hkv
    lo, hi = sharding.unit_range(B * Hkv, world, rank)
    torch.manual_seed(0)
    cb_all = torch.empty(Hkv, M, K, D, device=dev)
    for h in range(Hkv):
        g = torch.Generator(device=dev).manual_seed(w["seed"] * 7919 + h)
        cb_all[h] = torch.randn(M, K, D, generator=g, device=dev) * D ** -0.25
    pieces = []
    for (b0, b1, h0, h1) in sharding.unit_pieces(B, Hkv, lo, hi):
        nb_, nh = b1 - b0, h1 - h0
        q = torch.empty(nb_, L, nh * G, D, dtype=torch.bfloat16, device=dev)
        k = torch.empty(nb_, L, nh, D, dtype=torch.bfloat16, device=dev)
        v = torch.empty(nb_, L, nh, D, dtype=torch.bfloat16, device=dev)
        for bi in range(nb_):
            for hi_ in range(nh):
                u = (b0 + bi) * Hkv + h0 + hi_
                g = torch.Generator(device=dev).manual_seed(w["seed"] * 1000003 + u)
                q[bi, :, hi_ * G:(hi_ + 1) * G] = torch.randn(L, G, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                k[bi, :, hi_] = torch.randn(L, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                v[bi, :, hi_] = torch.randn(L, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        steps = w["decode_steps"]
        qd = torch.randn(nb_, steps, nh * G, D, device=dev).to(torch.bfloat16)
        kd = torch.randn(nb_, steps, nh, D, device=dev).to(torch.bfloat16)
        vd = torch.randn(nb_, steps, nh, D, device=dev).to(torch.bfloat16)
        pieces.append(dict(q=q.transpose(1, 2), k=k.transpose(1, 2), v=v.transpose(1, 2), cb=cb_all[h0:h1].contiguous(),
                           qd=qd.transpose(1, 2), kd=kd.transpose(1, 2), vd=vd.transpose(1, 2)))

    def prefill():
        caches = []
        for p in pieces:
            c = attn_vq.VectorQuantizedReRoPECache(W, p["cb"])
            attn_vq.long_prefilling_sort_based_linear(p["q"], p["k"], p["v"], None, L, c)
            caches.append(c)
        return caches

    def timed(fn):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = fn()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, r

    prefill()                                   # warm-up (allocator, tensor maps, rope tables)
    torch.cuda.empty_cache()
    ms_prefill, caches = min((timed(prefill) for _ in range(2)), key=lambda x: x[0])

    def decode():
        for t in range(w["decode_steps"]):
            for p, c in zip(pieces, caches):
                attn_vq.decode_step(p["qd"][:, :, t:t + 1], p["kd"][:, :, t:t + 1], p["vd"][:, :, t:t + 1], None, c)

    ms_decode, _ = timed(decode)
    flops = contraction_flops(**w)
    from vqtree_b200 import api
    api.check_status(dev)
    return dict(workload=f"config 5 as one job: B{B} Hq{Hq} Hkv{Hkv} D{D} L{L} W{W} M{M}xK{K} bf16 ReRoPE, {B * Hkv} units split "
                         f"{hi - lo} per rank, then {w['decode_steps']} decode steps through the cache",
                units_per_rank=hi - lo, prefill_ms=ms_prefill, prefill_tflops=flops / (ms_prefill * 1e-3) / 1e12,
                decode_ms_per_step=ms_decode / w["decode_steps"], decode_tok_s=B / (ms_decode / w["decode_steps"] * 1e-3),
                decode_launches_per_token="2 per piece (rotate-and-append, attention) + 2 when a block leaves the window",
                timing="CUDA events around the whole phase, max over ranks; no collective inside")


# ------------------------------------------------------------------------------------ main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2_32k", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the timing of the reference's own GPU kernels")
    ap.add_argument("--attn-impl", default="auto", choices=["auto", "simt", "tensor"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--decode-codebook", default="bf16", choices=["bf16", "f32"],
                    help="dtype of the codebook the decode kernel scores with (bf16: the copy the prefill uses too)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the fixed config-5 job split over the ranks")
    ap.add_argument("--strong-len", type=int, default=0, help="context length of the split job (default: config 5's 131072)")
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

    if args.impl == "reference-gpu":
        if rank != 0:
            return
        torch.cuda.set_device(local)
        leg = reference_gpu_leg(torch.device("cuda", local), reps=max(3, args.steps))
        r = leg.get("reference", {})
        print(json.dumps(dict(metric="vq_attn_prefill_tflops_32k_ctx", value=r.get("total_tflops"), unit="TFLOP/s", impl="reference-gpu",
                              n_gpus=1, steps=args.steps, warmup=args.warmup, ms_per_step=r.get("total_ms"), higher_is_better=True,
                              scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
                              config=dict(workload=leg.get("workload")), reference_gpu=leg)))
        return

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

    last = {}

    def step(events=None):
        rec = (lambda i: events[i].record()) if events else (lambda i: None)
        rec(0)
        codes = api.assign_codes(k3, cb)
        rec(1)
        cnt, vsum = api.build_aggregates(codes, v, K, nb)
        rec(2)
        out = api.prefill_from_aggregates(q1, q2, k1, k3, v, cb_act, cnt, vsum, W, impl=args.attn_impl)
        rec(3)
        last["codes"] = codes
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

    # ---- parity of the benchmarked launch (rank 0, outside the timed region) ----
    parity = None
    if rank == 0 and not args.no_parity:
        parity = parity_check(api, w, (q1, q2, k1, k3, v), cb, last["codes"], out)
    last.clear()

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
                   d2h_bytes_per_step=d2h, ms_per_step=el / n_e2e * 1e3, steps=n_e2e,
                   h2d_gbs_per_rank=h2d / (el / n_e2e) / 1e9,
                   note="bounded by the host link: every rank streams its inputs from pinned host memory; ranks of one "
                        "node share the host's memory and PCIe fabric")
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
        # the true step at this context: the window holds 1152 keys (it starts at the 128-block boundary), the
        # first 127 of them scored with the constant-position query against the raw keys (a split tile)
        nwin, nbd = d["W"] + BLOCK, BLOCK - 1
        tb = [dict(q=rn(d["B"], d["Hq"], d["D"]).bfloat16(), q2=rn(d["B"], d["Hq"], d["D"]).bfloat16(),
                   k1=rn(d["B"], d["Hkv"], nwin, d["D"]).bfloat16(), k3=rn(d["B"], d["Hkv"], nwin, d["D"]).bfloat16(),
                   v=rn(d["B"], d["Hkv"], nwin, d["D"]).bfloat16()) for _ in range(nbuf)]
        run_true = lambda i: api.vq_attention_decode(tb[i]["q"], tb[i]["q2"], tb[i]["k1"], tb[i]["k3"], tb[i]["v"], cbd,
                                                     bufs[i]["cnt"], bufs[i]["vsum"], n_valid=nwin, n_bd=nbd, workspace=ws, out=outd)
        for i in range(8):
            run_true(i % nbuf)
        barrier()
        d0.record()
        for i in range(nd):
            run_true(i % nbuf)
        d1.record()
        torch.cuda.synchronize(dev)
        us_true = d0.elapsed_time(d1) / nd * 1e3
        if dist is not None:
            t = torch.tensor([us_true], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us_true = float(t.item())
        by_true = by + d["B"] * d["Hkv"] * 2 * BLOCK * d["D"] * 2
        del tb
        decode = dict(true_step=dict(us_per_step=us_true, tok_s=world * d["B"] / (us_true * 1e-6), bytes_per_step=by_true,
                                     frac_hbm=by_true / (us_true * 1e-6) / 1e9 / peaks["hbm"],
                                     config=f"window rows {nwin} of which the first {nbd} use the constant-position query (context {d['ctx']})"),
                      tok_s=world * d["B"] / (us * 1e-6), us_per_step=us, bytes_per_step=by, achieved_gbs=by / (us * 1e-6) / 1e9,
                      frac_hbm=by / (us * 1e-6) / 1e9 / peaks["hbm"], peak_gbs=peaks["hbm"], peak_source=peaks["source"],
                      config=f"B{d['B']} H{d['Hq']} D{d['D']} ctx{d['ctx']} W{d['W']} M{d['M']}xK{d['K']} bf16, {args.decode_codebook} codebooks")
        del bufs

    # ---- one fixed job (config 5) split over the ranks: strong scaling, prefill + decode through the cache ----
    strong = None
    if not args.no_strong:
        torch.cuda.empty_cache()
        strong = strong_job(dist, dev, rank, world, barrier, args.strong_len)
        torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    refgpu = None
    if world == 1 and not args.no_reference_gpu:
        torch.cuda.empty_cache()
        refgpu = reference_gpu_leg(dev, reps=5)
        torch.cuda.empty_cache()

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
                      traffic=attention_bytes(w) * 1.012, traffic_unit="bytes per launch",
                      traffic_note="algorithmic bytes x 1.012, the DRAM read+write / algorithmic ratio ncu measured on the c2 "
                                   "capture; traffic grows in proportion to the (query tile, work item) pairs processed",
                      flops_per_launch=flops),
        stage_rooflines=stage_rooflines(w, stage_ms, peaks),
        cpu_baseline=cpu, e2e=e2e, gpu_launches=6 * args.steps, clocks=clocks, decode=decode, gather_ms=gather_ms,
        parity=parity, strong=strong, reference_gpu=refgpu,
    )
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
