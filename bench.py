#!/usr/bin/env python
"""Benchmark of the NSA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): BASELINE.json configs[2], the configuration its metric is quoted on -- the full NSAAttention
module forward + backward in bf16, B=8, T=8192, Hq=64, Hkv=4, D=128, compression block 32 / stride 16,
selection block 64, top-16, window 512, q/k/v/dO ~ N(0,1), weights ~ N(0,0.02), seed 2.  With N > 1 the batch
is sharded over the ranks (one process per GPU, total work fixed: strong scaling) and the 1.05 M weight
gradients are all-reduced over NCCL inside the timed region.

One JSON line is printed by rank 0: whole-job tokens/s with inputs resident in HBM (`value`), the same through
the public API from pinned host buffers with the copies timed (`e2e`), the dominant kernel's roofline
(`roofline`, timed with CUDA events inside this run), a per-kernel breakdown with one roofline entry per kernel
(`kernel_rooflines`: tensor-pipe fraction on the keys actually visited; for the selected-attention kernels also the
L2 -> SM gather rate against a measured gather ceiling), the clocks sampled under load, the CPU baseline (the oracle
restatement of the reference's naive torch path on the host cores) and, under `secondary`, the other BASELINE.json
configurations measured in the same process: `selection_microbench` (configs[1], N=1 only), `context` (configs[3] at
the run's N) and `decode` (configs[4] at the run's N).

`--impl reference` times that CPU restatement alone (the reference itself is a Python/Triton source tree that is
not present where this runs; it has no compiled artefact that could travel).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(B=8, T=8192, Hq=64, Hkv=4, D=128, block=32, stride=16, sel_block=64, n_sel=16, window=512, seed=2)
WORKLOAD = "configs[2]: NSAAttention module fwd+bwd bf16, B=8 T=8192 Hq=64 Hkv=4 D=128, cmp 32/16, sel 64 top-16, window 512"
METRIC = "NSA fwd+bwd tokens/s"
# ncu DRAM traffic per launch, MB per 8192-token sequence (see run_gpu), and the build it was captured from
NCU_TRAFFIC_COMMIT = "2bd6f3b"
NCU_MB_PER_SEQ = {"sel_fwd": 238, "sel_dq": 376, "sel+swa_dkv(+reverse index)": 867, "cmp_attn_fwd+select": 227,
                  "swa_fwd": 243, "swa_dq": 394, "cmp_dq": 375, "cmp_dkv(+reduce)": 277,
                  # key-major forward 203 read + 1046 written, its merge 1109 + 88
                  "sel_fwd_keymajor(+reverse index,+merge)": 2446,
                  # key-major kernel with dQ partials 1278 read + 1077 written, their reduction 1210 + 81
                  "sel+swa_dkv+sel_dq(+reverse index,+reduce)": 3646}


# ---------------------------------------------------------------------------------------------------------
# algorithmic FLOPs (2 flops per MAC, causally useful work only)
# ---------------------------------------------------------------------------------------------------------
def flop_model(B, T, Hq, Hkv, D, block, stride, sel_block, n_sel, window, nsel_pairs=None):
    Tc = (T - block) // stride + 1
    nvis = sum(min(max((t - block) // stride + 1, 0), Tc) for t in range(T))
    nsel = sum(sel_block * min(n_sel, t // sel_block + 1) for t in range(T)) if nsel_pairs is None else nsel_pairs
    nswa = sum(min(t + 1, window) for t in range(T))
    f = {}
    f["cmp"] = 4.0 * D * B * Hq * nvis
    f["slc"] = 4.0 * D * B * Hq * nsel
    f["swa"] = 4.0 * D * B * Hq * nswa
    f["comp"] = 2.0 * (2 * block * D * D) * B * Hkv * Tc
    f["gate"] = 2.0 * D * 3 * B * T * Hq
    f["fwd"] = f["cmp"] + f["slc"] + f["swa"] + f["comp"] + f["gate"]
    f["bwd"] = 2.5 * (f["cmp"] + f["slc"] + f["swa"]) + 2 * (f["comp"] + f["gate"])
    f["total"] = f["fwd"] + f["bwd"]
    return f


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for ts, line in self.rows:
            if ts < t0 or ts > t1 + 0.3:
                continue
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------
# CPU arm: the oracle restatement of the reference's naive torch path
# ---------------------------------------------------------------------------------------------------------
def cpu_step(sample_T, steps, warmup):
    import torch
    from oracle import nsa_oracle as O
    c = CFG
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(c["seed"])
    q = torch.randn(1, sample_T, c["Hq"], c["D"], generator=gen).bfloat16().float().requires_grad_(True)
    k = torch.randn(1, sample_T, c["Hkv"], c["D"], generator=gen).bfloat16().float().requires_grad_(True)
    v = torch.randn(1, sample_T, c["Hkv"], c["D"], generator=gen).bfloat16().float().requires_grad_(True)
    do = torch.randn(1, sample_T, c["Hq"], c["D"], generator=gen)
    wk, wv = ((torch.randn(c["D"], c["D"], c["block"], generator=gen) * 0.02).requires_grad_(True) for _ in range(2))
    bk, bv = (torch.zeros(c["D"], requires_grad=True) for _ in range(2))
    wg, bg = (torch.randn(3, c["D"], generator=gen) * 0.02).requires_grad_(True), torch.zeros(3, requires_grad=True)
    times = []
    for i in range(warmup + steps):
        t0 = time.time()
        o = O.nsa_forward(q, k, v, wk, bk, wv, bv, wg, bg, stride=c["stride"], block=c["block"],
                          sel_block=c["sel_block"], n_sel=c["n_sel"], window=c["window"])
        o.backward(do)
        for t in (q, k, v, wk, wv, bk, bv, wg, bg):
            t.grad = None
        if i >= warmup:
            times.append(time.time() - t0)
    sec = sum(times) / len(times)
    return dict(value=sample_T / sec, unit="tokens/s", cores=torch.get_num_threads(), kind="port",
                sample="fwd+bwd of the fp32 oracle on 1 sequence x %d tokens of the workload (Hq=64, Hkv=4, D=128), "
                       "%d timed step(s), %.1f s each" % (sample_T, len(times), sec)), sec


def run_reference(args):
    """The CPU arm: every step is the oracle's fwd+bwd on a bounded 1024-token sample of one sequence of the workload.
    All requested steps are run unless they would take longer than about two minutes; the line reports the steps
    that were really timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _, sec1 = cpu_step(1024, 1, 0)                       # one untimed-for-the-record step sizes the run
    budget = 120.0
    steps = max(1, min(args.steps, int(budget / max(sec1, 1e-3))))
    warm = max(0, min(args.warmup, int(0.25 * budget / max(sec1, 1e-3))))
    cb, sec = cpu_step(1024, steps, warm)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warm, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "reference_arm": "CPU restatement (oracle) of the reference's naive "
                       "torch path; each step is a bounded 1024-token sample of one sequence of the workload.  Cost per "
                       "token grows with the sequence length (compressed and selected branches), so tokens/s at 1024 "
                       "tokens is an UPPER bound for the CPU at the workload's T=8192"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------
def per_kernel_breakdown(torch, nsa_b200, mod, q4, k4, v4, do4, reps=3):
    """Times every kernel family of the step separately with CUDA events on the current stream (each call is a
    C-ABI entry point restricted to one kernel).  Returns {name: ms} and the selection pair count."""
    from nsa_b200 import _lib
    L = _lib.lib()
    B, T, Hq, D = q4.shape
    Hkv = k4.shape[2]
    c = CFG
    scale = D ** -0.5
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=q4.device)
    k3, v3 = k4.view(B * T, Hkv, D), v4.view(B * T, Hkv, D)
    with torch.no_grad():
        ck, cv, _ = mod.compressor(k3, v3, cu, None)
    Tc = ck.shape[1]
    o_cmp, o_slc, o_swa = (torch.empty_like(q4) for _ in range(3))
    lse_cmp, lse_slc, lse_swa, delta = (torch.empty(B, T, Hq, dtype=torch.float32, device=q4.device) for _ in range(4))
    idx = torch.empty(B, T, Hkv, c["n_sel"], dtype=torch.int32, device=q4.device)
    dq, dk, dv = torch.empty_like(q4), torch.empty_like(k4), torch.empty_like(v4)
    dck, dcv = torch.empty_like(ck), torch.empty_like(cv)
    ws1 = torch.empty(max(_lib.sel_swa_bwd_workspace_bytes(B, T, T, Hq, Hkv, D, c["n_sel"], c["sel_block"]),
                          L.nsa_sel_swa_fwd_workspace_bytes(B, T, T, Hq, Hkv, D, c["n_sel"], c["sel_block"])),
                      dtype=torch.uint8, device=q4.device)
    ws2 = torch.empty(L.nsa_cmp_attn_bwd_workspace_bytes(B, T, Tc, Hkv, D), dtype=torch.uint8, device=q4.device)
    P, S = _lib.ptr, _lib.stream
    wk = mod.compressor.compressor_k.weight.detach().permute(2, 1, 0).reshape(c["block"] * D, D).contiguous()
    bk = mod.compressor.compressor_k.bias.detach()
    cin = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=q4.device)
    cout = torch.arange(0, (B + 1) * Tc, Tc, dtype=torch.int32, device=q4.device)
    dwk = torch.empty(c["block"] * D, D, dtype=torch.float32, device=q4.device)
    dbk = torch.empty(D, dtype=torch.float32, device=q4.device)
    ws3 = torch.empty(L.nsa_compress_bwd_workspace_bytes(B, Hkv, D, c["block"]), dtype=torch.uint8, device=q4.device)
    g1, g2, g3, dg1, dg2, dg3 = (torch.full((B, T, Hq), 0.5, dtype=torch.bfloat16, device=q4.device) for _ in range(6))
    delta2, delta3 = torch.empty_like(delta), torch.empty_like(delta)
    wg, bg = mod.gating.weight.detach(), mod.gating.bias.detach()
    dwg, dbg = torch.empty_like(wg), torch.empty_like(bg)
    ws4 = torch.empty(L.nsa_gate_bwd_workspace_bytes(B * T * Hq, D), dtype=torch.uint8, device=q4.device)

    calls = {
        "compress_fwd(one of k,v)": lambda: L.nsa_compress_fwd_uniform(P(k3), P(wk), P(bk), P(ck), B, T, Hkv, D, c["block"],
                                                                        c["stride"], S()),
        "cmp_attn_fwd+select": lambda: L.nsa_cmp_attn_fwd(P(q4), P(ck), P(cv), P(o_cmp), P(lse_cmp), P(idx), None, B, T,
                                                          Tc, Hq, Hkv, D, c["block"], c["stride"], 1, scale, c["n_sel"],
                                                          5, 4, 0, S()),
        "sel_fwd": lambda: L.nsa_sel_swa_fwd(P(q4), P(k4), P(v4), P(idx), 0, None, P(o_slc), P(lse_slc), None, None, None,
                                             None, None, None, None, B, T, Hq, Hkv, D, c["n_sel"], c["sel_block"], 0,
                                             scale, S()),
        # what a module step runs: the same forward key-major on the tensor cores (reverse index, one CTA per key block
        # over the queries that selected it, per-visit partial tiles, slot-order merge); "sel_fwd" above is the
        # query-major kernel that runs without a workspace
        "sel_fwd_keymajor(+reverse index,+merge)": lambda: L.nsa_sel_swa_fwd_ws(
            P(q4), P(k4), P(v4), P(idx), 0, None, P(o_slc), P(lse_slc), None, None, None, None, None, None, None, P(ws1),
            ws1.numel(), B, T, Hq, Hkv, D, c["n_sel"], c["sel_block"], 0, scale, T, 0, S()),
        "gather_probe": lambda: L.nsa_gather_probe(P(k4), P(v4), P(idx), 0, B, T, Hq, Hkv, D, c["n_sel"], c["sel_block"],
                                                   S()),
        "swa_fwd": lambda: L.nsa_sel_swa_fwd(P(q4), P(k4), P(v4), None, 0, None, None, None, P(o_swa), P(lse_swa), None,
                                             None, None, None, None, B, T, Hq, Hkv, D, c["n_sel"], c["sel_block"],
                                             c["window"], scale, S()),
        "combine": lambda: L.nsa_combine(P(o_slc), P(g1), P(o_swa), P(g1), P(o_cmp), P(g1), P(dq), B * T * Hq, D, S()),
        "gate_fwd": lambda: L.nsa_gate_fwd(P(q4), P(wg), P(bg), P(g1), P(g2), P(g3), B * T * Hq, D, S()),
        "rowdot3(delta,dgate)": lambda: L.nsa_rowdot3(P(o_slc), P(o_swa), P(o_cmp), P(do4), P(g1), P(g2), P(g3), P(delta),
                                                      P(delta2), P(delta3), P(dg1), P(dg2), P(dg3), B * T * Hq, D, S()),
        "sel_dq": lambda: L.nsa_sel_swa_bwd(P(q4), P(k4), P(v4), P(idx), 0, None, P(do4), P(lse_slc), P(delta), None, None,
                                            None, None, None, P(dq), 0, None, None, None, 0, B, T, Hq, Hkv, D, c["n_sel"],
                                            c["sel_block"], 0, scale, S()),
        "swa_dq": lambda: L.nsa_sel_swa_bwd(P(q4), P(k4), P(v4), None, 0, None, None, None, None, None, P(do4), P(lse_swa),
                                            P(delta), None, P(dq), 0, None, None, None, 0, B, T, Hq, Hkv, D, c["n_sel"],
                                            c["sel_block"], c["window"], scale, S()),
        "sel+swa_dkv(+reverse index)": lambda: L.nsa_sel_swa_bwd(
            P(q4), P(k4), P(v4), P(idx), 0, None, P(do4), P(lse_slc), P(delta), None, P(do4), P(lse_swa), P(delta), None,
            None, 0, P(dk), P(dv), P(ws1), ws1.numel(), B, T, Hq, Hkv, D, c["n_sel"], c["sel_block"], c["window"], scale,
            S()),
        # the call the module makes: window dQ, then the key-major kernel (dK, dV and the selected branch's dQ partials)
        # and the reduction of the partials (large workspace); the query-major "sel_dq" above is what runs instead when
        # a caller hands over only the small workspace
        "sel+swa_bwd(all)": lambda: L.nsa_sel_swa_bwd(
            P(q4), P(k4), P(v4), P(idx), 0, None, P(do4), P(lse_slc), P(delta), None, P(do4), P(lse_swa), P(delta), None,
            P(dq), 0, P(dk), P(dv), P(ws1), ws1.numel(), B, T, Hq, Hkv, D, c["n_sel"], c["sel_block"], c["window"], scale,
            S()),
        "cmp_dq": lambda: L.nsa_cmp_attn_bwd(P(q4), P(ck), P(cv), P(lse_cmp), P(do4), P(delta), None, P(dq), 0, None, None,
                                             None, 0, B, T, Tc, Hq, Hkv, D, c["block"], c["stride"], 1, scale, S()),
        "cmp_dkv(+reduce)": lambda: L.nsa_cmp_attn_bwd(P(q4), P(ck), P(cv), P(lse_cmp), P(do4), P(delta), None, None, 0,
                                                       P(dck), P(dcv), P(ws2), ws2.numel(), B, T, Tc, Hq, Hkv, D,
                                                       c["block"], c["stride"], 1, scale, S()),
        "gate_bwd": lambda: L.nsa_gate_bwd(P(q4), P(dg1), P(dg2), P(dg3), P(wg), P(dq), P(dwg), P(dbg), P(ws4), ws4.numel(),
                                           B * T * Hq, D, S()),
        "compress_bwd(one of k,v)": lambda: L.nsa_compress_bwd(P(k3), P(wk), P(dck), P(dk), P(dwk), P(dbk), P(ws3),
                                                                ws3.numel(), P(cin), P(cout), B, Hkv, D, c["block"],
                                                                c["stride"], T, B * Tc, S()),
    }
    out = {}
    for name, fn in calls.items():
        _lib.check(fn(), name)           # warm-up, and produces the tensors later calls read
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            _lib.check(fn(), name)
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / reps
    # derived: the composite call minus the window dQ kernel timed alone
    out["sel+swa_dkv+sel_dq(+reverse index,+reduce)"] = out["sel+swa_bwd(all)"] - out["swa_dq"]
    t = torch.arange(T, device=q4.device).view(1, T, 1, 1)
    valid = (idx >= 0) & (idx.long() * c["sel_block"] <= t)
    pairs = int(valid.sum().item())               # (token, kv head, block) visits
    keys_per_seq_head = pairs * c["sel_block"] / (B * Hkv)
    _lib.device_status()
    return out, keys_per_seq_head


def bind_to_gpu_numa_node(local):
    """Best effort: run this process (and so first-touch its pinned host buffers) on the CPU cores NVML reports as
    local to the GPU, so host<->device copies do not cross the socket interconnect.  Changes only this process's CPU
    affinity; skipped when NVML or the cores are not available.  Returns a short description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        allowed = os.sched_getaffinity(0)
        both = near & allowed
        if both and both != allowed:
            os.sched_setaffinity(0, both)
            return "bound to %d GPU-local cores of %d allowed" % (len(both), len(allowed))
        return "all %d allowed cores are %s" % (len(allowed), "GPU-local" if both else "remote from the GPU")
    except Exception as e:   # no NVML, no permission: leave the affinity alone
        return "unchanged (%s)" % type(e).__name__


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import nsa_b200
    from nsa_b200 import _lib
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    numa = bind_to_gpu_numa_node(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = CFG
    if c["B"] % world:
        raise SystemExit("batch %d does not divide over %d ranks" % (c["B"], world))
    Bl = c["B"] // world
    T, Hq, Hkv, D = c["T"], c["Hq"], c["Hkv"], c["D"]
    gen = torch.Generator().manual_seed(c["seed"] * 1000 + rank)
    host = {}
    for name, h in (("q", Hq), ("k", Hkv), ("v", Hkv), ("do", Hq)):
        host[name] = torch.randn(Bl * T, h, D, generator=gen).to(torch.bfloat16).pin_memory()
    wgen = torch.Generator().manual_seed(c["seed"])
    mod = nsa_b200.NSAAttention(D, True, None, 0.0, compression_stride=c["stride"], compression_block=c["block"],
                                selection_block=c["sel_block"], selected_block_count=c["n_sel"],
                                sliding_window=c["window"], device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn(p.shape, generator=wgen) * 0.02)
    params = list(mod.parameters())
    cu = torch.arange(0, (Bl + 1) * T, T, dtype=torch.int32, device=dev)
    q, k, v, do = (host[n].to(dev) for n in ("q", "k", "v", "do"))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out_h = {n: torch.empty_like(host[m]).pin_memory() for n, m in (("o", "q"), ("dq", "q"), ("dk", "k"), ("dv", "v"))}

    def step(qd, kd, vd, dod):
        for t in [qd, kd, vd] + params:
            t.grad = None
        o = mod(qd, kd, vd, cu, T)
        o.backward(dod)
        if world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            dist.all_reduce(flat)
        return o

    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    cu1 = torch.arange(0, 2 * T, T, dtype=torch.int32, device=dev)

    def step_e2e():
        """The same step from pinned host buffers through the module, one sequence at a time: the host-to-device
        copy of sequence i+1 and the device-to-host copy of sequence i-1's results overlap the compute of sequence i
        (three streams; sequences of a batch are independent, weight gradients accumulate in .grad)."""
        for p in params:
            p.grad = None
        main = torch.cuda.current_stream()
        keep = []
        for i in range(Bl):
            sl = slice(i * T, (i + 1) * T)
            with torch.cuda.stream(s_in):
                qd, kd, vd, dod = (host[n][sl].to(dev, non_blocking=True) for n in ("q", "k", "v", "do"))
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            main.wait_event(ev_in)
            for t_ in (qd, kd, vd, dod):
                t_.record_stream(main)
            qd.requires_grad_(True), kd.requires_grad_(True), vd.requires_grad_(True)
            o = mod(qd, kd, vd, cu1, T)
            o.backward(dod)
            ev_c = torch.cuda.Event()
            ev_c.record(main)
            s_out.wait_event(ev_c)
            for t_ in (o, qd.grad, kd.grad, vd.grad):
                t_.record_stream(s_out)
            with torch.cuda.stream(s_out):
                out_h["o"][sl].copy_(o.detach(), non_blocking=True)
                out_h["dq"][sl].copy_(qd.grad, non_blocking=True)
                out_h["dk"][sl].copy_(kd.grad, non_blocking=True)
                out_h["dv"][sl].copy_(vd.grad, non_blocking=True)
            keep.append((qd, kd, vd, dod, o))
        main.wait_stream(s_out)
        if world > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            dist.all_reduce(flat)
        return keep

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        w1 = time.time()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, w0, w1

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches = [0, 0]

    def counted_step():
        launches[0] = launches[0] or _lib.lib().nsa_kernel_launch_count()
        step(q, k, v, do)
        launches[1] = _lib.lib().nsa_kernel_launch_count()

    for _ in range(args.warmup):
        step(q, k, v, do)
    ms_step, w0, w1 = timed(counted_step, args.steps, 0)
    clocks = sampler.stop(w0, w1) if rank == 0 else None
    _lib.device_status()
    ms_e2e, _, _ = timed(step_e2e, max(1, min(args.steps, 5)), 1)
    _lib.device_status()
    h2d_bytes = sum(host[n].numel() * 2 for n in ("q", "k", "v", "do"))
    d2h_bytes = sum(t.numel() * 2 for t in out_h.values())

    tokens = c["B"] * T
    kern = keys_per = None
    if rank == 0:
        with torch.no_grad():
            kern, keys_per = per_kernel_breakdown(torch, nsa_b200, mod, q.detach().view(Bl, T, Hq, D),
                                                  k.detach().view(Bl, T, Hkv, D), v.detach().view(Bl, T, Hkv, D),
                                                  do.view(Bl, T, Hq, D))
    # the main workload's tensors are no longer needed: make room for the secondary workloads
    del q, k, v, do, host, out_h
    torch.cuda.empty_cache()
    secondary = {}
    sec_steps = max(2, min(args.steps, 5))
    if world == 1 and not args.no_secondary:
        secondary["selection_microbench"] = selection_microbench(torch, dev, read_peaks())
    if not args.no_secondary:
        secondary["context"] = measure_context(torch, dist, nsa_b200, rank, world, dev, sec_steps, 2, single_gpu_base=True)
        secondary["decode"] = measure_decode(torch, dist, nsa_b200, rank, world, dev, max(sec_steps, 5), 3)

    if rank == 0:
        peaks = read_peaks()
        fm_nom = flop_model(c["B"], T, Hq, Hkv, D, c["block"], c["stride"], c["sel_block"], c["n_sel"], c["window"])
        # the selection follows the reference's unmasked scoring, so about half of a token's 16 blocks lie in its future
        # and are skipped by every kernel: the FLOPs that count are those of the keys actually visited
        fm_vis = flop_model(c["B"], T, Hq, Hkv, D, c["block"], c["stride"], c["sel_block"], c["n_sel"], c["window"],
                            nsel_pairs=keys_per)
        fm_loc = flop_model(Bl, T, Hq, Hkv, D, c["block"], c["stride"], c["sel_block"], c["n_sel"], c["window"],
                            nsel_pairs=keys_per)
        # algorithmic flops per kernel launch (per rank): forward 4D per (row,key); the backward's 10D per (row,key)
        # is split 4D to the dQ kernel (dQ + half of the S/dP recompute) and 6D to the dK/dV kernel
        kflops = {
            "sel_fwd": fm_loc["slc"], "sel_fwd_keymajor(+reverse index,+merge)": fm_loc["slc"], "swa_fwd": fm_loc["swa"],
            "cmp_attn_fwd+select": fm_loc["cmp"],
            "sel_dq": fm_loc["slc"], "swa_dq": fm_loc["swa"], "cmp_dq": fm_loc["cmp"],
            "sel+swa_dkv(+reverse index)": 1.5 * (fm_loc["slc"] + fm_loc["swa"]), "cmp_dkv(+reduce)": 1.5 * fm_loc["cmp"],
            # the whole 10D of the selected branch (S, dP, dV, dK, dQ) and the window's 6D in one pass over the keys
            "sel+swa_dkv+sel_dq(+reverse index,+reduce)": 2.5 * fm_loc["slc"] + 1.5 * fm_loc["swa"],
            "compress_fwd(one of k,v)": fm_loc["comp"] / 2, "compress_bwd(one of k,v)": fm_loc["comp"],
        }
        # DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels that can dominate, from
        # one ncu capture of the B=1 slice of this workload (`--profile-case`), in MB per sequence; traffic grows in
        # proportion to the number of sequences (every sequence's K/V stays in L2, q/dO/o/dq are streamed once).
        # NCU_TRAFFIC_COMMIT names the build the capture was taken from: a kernel changed since then has a stale entry.
        # not part of the module's step with the workspaces: the query-major selected forward and dQ, the dK/dV-only call
        not_in_step = ("sel_fwd", "sel_dq", "sel+swa_dkv(+reverse index)")
        dom = max((n for n in kern if n in kflops and n not in not_in_step), key=lambda n: kern[n])
        # kernels timed alone (three launches back to back): the burst bf16 peak is their denominator
        peak = peaks["tf_burst"]
        kroof = {}
        for n in kflops:
            ach = kflops[n] / (kern[n] * 1e-3) / 1e12
            kroof[n] = {"ms": round(kern[n], 3), "tflops": round(ach, 1), "frac_of_burst_peak": round(ach / peak, 4)}
        # selected attention: the L2 -> SM gather of 32 KB (K and V block) per visited (token, kv head, block), used by
        # 16 query rows only, against the rate of the same gather with no arithmetic behind it (nsa_gather_probe)
        visits = keys_per * Bl * Hkv / c["sel_block"]
        gbytes = visits * 2 * c["sel_block"] * D * 2
        for n in ("sel_fwd", "sel_dq"):
            kroof[n].update({"pipe": "mma.sync (peak 574 TFLOP/s measured for m16n8k16 bf16)",
                             "frac_of_mma_sync_peak": round(kroof[n]["tflops"] / 574.0, 4),
                             "gather_bytes": gbytes, "gather_tbs": round(gbytes / (kern[n] * 1e-3) / 1e12, 2),
                             "gather_ceiling_tbs": round(gbytes / (kern["gather_probe"] * 1e-3) / 1e12, 2),
                             "frac_of_gather_ceiling": round(kern["gather_probe"] / kern[n], 4)})
        achieved = kflops[dom] / (kern[dom] * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": dom, "achieved": round(achieved, 2), "peak": peak, "unit": "TFLOP/s",
                "frac": round(achieved / peak, 4), "peak_source": peaks["source"] + " (burst bf16 GEMM: the kernel is timed alone)",
                "frac_of_sustained_peak": round(achieved / peaks["tf_sustained"], 4),
                "traffic": (NCU_MB_PER_SEQ[dom] * 1e6 * Bl) if dom in NCU_MB_PER_SEQ else None,
                "traffic_source": "ncu capture at B=1 (build %s) x sequences per rank" % NCU_TRAFFIC_COMMIT,
                "ms_per_launch": round(kern[dom], 3), "algorithmic_flops_per_launch": kflops[dom]}
        if dom in ("sel_fwd", "sel_dq"):
            roof.update({k_: v_ for k_, v_ in kroof[dom].items() if k_.startswith(("pipe", "frac_of_", "gather"))})
        cb = None
        if world == 1 and not args.no_cpu:
            cb, _ = cpu_step(1024, 1, 0)
        tf_vis = fm_vis["total"] / (ms_step * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": tokens / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": c["B"], "seq_len": T, "parallelism": "batch-sharded x%d" % world,
                       "l2": "inputs larger than L2 (q and dO are 1.07 GB each at N=1)",
                       "selection": "indices produced by the fused top-16 of the step itself (oracle-style scoring)"},
            # FLOPs of the keys actually visited (see above); the nominal figure (16 visited blocks per token) is kept
            # beside it under its own name
            "tflops_algorithmic": tf_vis,
            "tflops_frac_of_sustained_peak": tf_vis / world / peaks["tf_sustained"],
            "tflops_frac_of_burst_peak": tf_vis / world / peaks["tf_burst"],
            "tflops_nominal_selection": fm_nom["total"] / (ms_step * 1e-3) / 1e12,
            "flops_visited_per_step": fm_vis["total"], "flops_nominal_per_step": fm_nom["total"],
            "host_affinity": numa,
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes * world,
                    "d2h_bytes_per_step": d2h_bytes * world, "ms_per_step": ms_e2e,
                    "host_gbs_aggregate": round((h2d_bytes + d2h_bytes) * world / (ms_e2e * 1e-3) / 1e9, 1)},
            "gpu_launches": int(launches[1] - launches[0]),
            "roofline": roof, "kernels_ms": {n: round(v_, 3) for n, v_ in kern.items()}, "kernel_rooflines": kroof,
            "selected_keys_per_seq_kvhead": keys_per, "clocks": clocks, "cpu_baseline": cb, "secondary": secondary,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _event_time(torch, dist, fn, steps, warmup, world, dev):
    """CUDA-event time of `steps` calls after `warmup`, barrier + synchronize on both sides, max over ranks; ms per call."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()) / steps


def config1_indices(torch, B, T, H, S, BS, gen, device):
    """BASELINE.json configs[1]: per (b, t, kv head) min(S, t//BS+1) distinct blocks drawn uniformly from the causally
    valid ones, always with block 0 and the query's local block; unused slots are -1."""
    t = torch.arange(T, device=device)
    nblk = (t // BS + 1).view(1, T, 1, 1)
    NB = T // BS
    r = torch.rand(B, T, H, NB, generator=gen, device=device)
    blk = torch.arange(NB, device=device).view(1, 1, 1, NB)
    r = torch.where(blk < nblk, r, torch.full_like(r, -1.0))
    r = torch.where((blk == 0) | (blk == nblk - 1), torch.full_like(r, 2.0), r)
    top = torch.topk(r, S, dim=-1)
    return torch.where(top.values >= 0, top.indices, torch.full_like(top.indices, -1)).to(torch.int32)


def selection_microbench(torch, dev, peaks):
    """BASELINE.json configs[1]: the selected-attention forward alone, B=4 T=8192 Hq=64 Hkv=4 D=128 bf16, top-16 of
    64-key blocks, all 16 blocks causally valid (window 0), seed 1; once with a warm L2 and once with a 512 MB write
    between launches.  Also the gather ceiling (nsa_gather_probe) on the same indices."""
    from nsa_b200 import _lib
    L, P, S = _lib.lib(), _lib.ptr, _lib.stream
    B, T, Hq, Hkv, D, n, BS = 4, 8192, 64, 4, 128, 16, 64
    gen = torch.Generator(device=dev).manual_seed(1)
    q = torch.randn(B, T, Hq, D, generator=gen, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, generator=gen, device=dev, dtype=torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, generator=gen, device=dev, dtype=torch.bfloat16)
    idx = config1_indices(torch, B, T, Hkv, n, BS, gen, dev)
    o = torch.empty_like(q)
    lse = torch.empty(B, T, Hq, dtype=torch.float32, device=dev)
    scale = D ** -0.5
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def fwd():
        _lib.check(L.nsa_sel_swa_fwd(P(q), P(k), P(v), P(idx), 0, None, P(o), P(lse), None, None, None, None, None, None,
                                     None, B, T, Hq, Hkv, D, n, BS, 0, scale, S()), "nsa_sel_swa_fwd")

    nws = L.nsa_sel_swa_fwd_workspace_bytes(B, T, T, Hq, Hkv, D, n, BS)
    ws = torch.empty(nws, dtype=torch.uint8, device=dev)

    def fwd_kv():   # the same forward key-major on the tensor cores (what the Python layer calls)
        _lib.check(L.nsa_sel_swa_fwd_ws(P(q), P(k), P(v), P(idx), 0, None, P(o), P(lse), None, None, None, None, None, None,
                                        None, P(ws), nws, B, T, Hq, Hkv, D, n, BS, 0, scale, T, 0, S()), "nsa_sel_swa_fwd_ws")

    def probe():
        _lib.check(L.nsa_gather_probe(P(k), P(v), P(idx), 0, B, T, Hq, Hkv, D, n, BS, S()), "nsa_gather_probe")

    def timed(fn, reps, flushed):
        tot = 0.0
        for _ in range(reps):
            if flushed:
                flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / reps

    for _ in range(3):
        fwd()
        fwd_kv()
        probe()
    torch.cuda.synchronize()
    ms_kv, ms_kv_cold = timed(fwd_kv, 10, False), timed(fwd_kv, 5, True)
    ms_warm, ms_cold = timed(fwd, 10, False), timed(fwd, 5, True)
    ms_probe = timed(probe, 5, False)
    _lib.device_status()
    visits = int(((idx >= 0) & (idx.long() * BS <= torch.arange(T, device=dev).view(1, T, 1, 1))).sum().item())
    flops = 4.0 * D * (Hq // Hkv) * BS * visits
    gbytes = visits * 2.0 * BS * D * 2
    return {"workload": "configs[1]: selection_attn forward, B=4 T=8192 Hq=64 Hkv=4 D=128 bf16, top-16 of 64-key blocks, "
                        "indices uniform over causally valid blocks incl. block 0 and the local block, window 0, seed 1",
            "ms_warm_l2": round(ms_warm, 3), "ms_l2_flushed": round(ms_cold, 3),
            "tokens_per_s": B * T / (ms_warm * 1e-3),
            "kernel": "query-major mma.sync kernel (nsa_sel_swa_fwd); the key-major tcgen05 path is beside it",
            "key_major": {"entry": "nsa_sel_swa_fwd_ws (reverse index + tcgen05 key-major kernel + merge)",
                          "ms_warm_l2": round(ms_kv, 3), "ms_l2_flushed": round(ms_kv_cold, 3),
                          "tokens_per_s": B * T / (ms_kv * 1e-3), "tflops": round(flops / (ms_kv * 1e-3) / 1e12, 1),
                          "workspace_bytes": int(nws)},
            "visited_blocks_per_token_kvhead": visits / (B * T * Hkv),
            "tflops": round(flops / (ms_warm * 1e-3) / 1e12, 1),
            "frac_of_burst_peak": round(flops / (ms_warm * 1e-3) / 1e12 / peaks["tf_burst"], 4),
            "frac_of_mma_sync_peak": round(flops / (ms_warm * 1e-3) / 1e12 / 574.0, 4),
            "gather_bytes": gbytes, "gather_tbs": round(gbytes / (ms_warm * 1e-3) / 1e12, 2),
            "gather_ceiling_ms": round(ms_probe, 3), "gather_ceiling_tbs": round(gbytes / (ms_probe * 1e-3) / 1e12, 2),
            "frac_of_gather_ceiling": round(ms_probe / ms_warm, 4)}


def measure_context(torch, dist, nsa_b200, rank, world, dev, steps, warmup, single_gpu_base=False):
    """BASELINE configs[3]: one sequence of 65536 tokens, fwd+bwd, context-sharded over the ranks (zig-zag query chunks;
    see nsa_b200/context_parallel.py for what crosses NVLink).  With `single_gpu_base` and more than one rank, rank 0
    also times the unsharded step alone so the record carries its own scaling efficiency."""
    from nsa_b200 import _lib
    from nsa_b200.context_parallel import context_parallel_forward
    c = dict(CFG, B=1, T=65536, seed=3)
    T, Hq, Hkv, D = c["T"], c["Hq"], c["Hkv"], c["D"]
    Tl = T // world
    gen = torch.Generator(device=dev).manual_seed(c["seed"] * 1000 + rank)
    q, k, v, do = (torch.randn(1, Tl, h, D, generator=gen, device=dev, dtype=torch.bfloat16) for h in (Hq, Hkv, Hkv, Hq))
    wgen = torch.Generator().manual_seed(c["seed"])
    mod = nsa_b200.NSAAttention(D, True, None, 0.0, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn(p.shape, generator=wgen) * 0.02)
    params = list(mod.parameters())
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)

    def step_single(qq, kk, vv, dd):
        Tn = qq.shape[1]
        cu = torch.tensor([0, Tn], dtype=torch.int32, device=dev)
        for t in [qq, kk, vv] + params:
            t.grad = None
        o = mod(qq.view(Tn, Hq, D), kk.view(Tn, Hkv, D), vv.view(Tn, Hkv, D), cu, Tn)
        o.backward(dd.view(Tn, Hq, D))

    def step():
        if world == 1:
            step_single(q, k, v, do)
            return
        for t in [q, k, v] + params:
            t.grad = None
        o = context_parallel_forward(mod, q, k, v, None, zigzag=True)
        o.backward(do)
        flat = torch.cat([p.grad.reshape(-1) for p in params])
        dist.all_reduce(flat)

    ms_step = _event_time(torch, dist, step, steps, warmup, world, dev)
    _lib.device_status()
    out = {"workload": "configs[3]: NSAAttention fwd+bwd bf16, B=1 T=65536 Hq=64 Hkv=4 D=128, context-sharded "
                       "(zig-zag query chunks) x%d" % world,
           "n_gpus": world, "ms_per_step": ms_step, "tokens_per_s": T / (ms_step * 1e-3), "steps": steps}
    fm = flop_model(1, T, Hq, Hkv, D, c["block"], c["stride"], c["sel_block"], c["n_sel"], c["window"])
    out["tflops_nominal_selection"] = fm["total"] / (ms_step * 1e-3) / 1e12
    if world > 1 and single_gpu_base:
        base = torch.zeros(1, device=dev)
        del q, k, v, do
        torch.cuda.empty_cache()
        if rank == 0:
            g2 = torch.Generator(device=dev).manual_seed(c["seed"] * 1000)
            qf, kf, vf, df = (torch.randn(1, T, h, D, generator=g2, device=dev, dtype=torch.bfloat16)
                              for h in (Hq, Hkv, Hkv, Hq))
            qf.requires_grad_(True), kf.requires_grad_(True), vf.requires_grad_(True)
            base[0] = _event_time(torch, dist, lambda: step_single(qf, kf, vf, df), 2, 1, 1, dev)
            del qf, kf, vf, df
        dist.barrier()
        dist.broadcast(base, 0)
        out["single_gpu_ms_per_step_same_process"] = float(base.item())
        out["scaling_efficiency_vs_single_gpu"] = float(base.item()) / (ms_step * world)
    torch.cuda.empty_cache()
    return out


def decode_lengths():
    import torch
    return torch.randint(4096, 32769, (128,), generator=torch.Generator().manual_seed(4)).tolist()


def measure_decode(torch, dist, nsa_b200, rank, world, dev, steps, warmup):
    """BASELINE configs[4]: 128 sequences with KV lengths uniform in [4096, 32768] (seed 4), one new query token each;
    sequences are assigned to the ranks by longest-processing-time bin packing (work ~ L); no collective."""
    from nsa_b200 import _lib
    from nsa_b200.decode import compress_cache, nsa_decode
    c = CFG
    Hq, Hkv, D = c["Hq"], c["Hkv"], c["D"]
    lens = decode_lengths()
    bins = [[] for _ in range(world)]
    load = [0] * world
    for i in sorted(range(128), key=lambda i: -lens[i]):
        r = load.index(min(load))
        bins[r].append(i)
        load[r] += lens[i]
    mine = [lens[i] for i in bins[rank]]
    cu = [0]
    for n in mine:
        cu.append(cu[-1] + n)
    gen = torch.Generator(device=dev).manual_seed(4000 + rank)
    q = torch.randn(len(mine), Hq, D, generator=gen, device=dev, dtype=torch.bfloat16)
    k = torch.randn(cu[-1], Hkv, D, generator=gen, device=dev, dtype=torch.bfloat16)
    v = torch.randn(cu[-1], Hkv, D, generator=gen, device=dev, dtype=torch.bfloat16)
    mod = nsa_b200.NSAAttention(D, True, None, 0.0, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(4)) * 0.02)
        ms_stateless = _event_time(torch, dist, lambda: nsa_decode(mod, q, k, v, cu), steps, warmup, world, dev)
        cache = compress_cache(mod, k, v, cu)
        ms_cached = _event_time(torch, dist, lambda: nsa_decode(mod, q, k, v, cu, cache=cache), steps, warmup, world, dev)
    _lib.device_status()
    peaks = read_peaks()
    # bytes a step must read: stateless = all of K and V once (they are re-compressed); cached = the compressed cache,
    # the selected blocks and the window of every sequence
    kv_bytes = sum(lens) * Hkv * D * 2 * 2
    n_c = sum((L - c["block"]) // c["stride"] + 1 for L in lens)
    cached_bytes = (n_c + 128 * (c["n_sel"] * c["sel_block"] + c["window"])) * Hkv * D * 2 * 2
    out = {"workload": "configs[4]: varlen decode, 128 sequences, KV length U[4096,32768] seed 4, Hq=64 Hkv=4 D=128, "
                       "sequence-sharded x%d (LPT)" % world,
           "n_gpus": world, "sum_kv_len": sum(lens), "steps": steps,
           "stateless": {"ms_per_step": ms_stateless, "tokens_per_s": 128 / (ms_stateless * 1e-3),
                         "algorithmic_bytes": kv_bytes,
                         "hbm_gbs_per_gpu": round(kv_bytes / (ms_stateless * 1e-3) / 1e9 / world, 1),
                         "frac_of_hbm_peak": round(kv_bytes / (ms_stateless * 1e-3) / 1e9 / world / peaks["hbm_gbs"], 4)},
           "with_compressed_cache": {"ms_per_step": ms_cached, "tokens_per_s": 128 / (ms_cached * 1e-3),
                                     "algorithmic_bytes": cached_bytes,
                                     "hbm_gbs_per_gpu": round(cached_bytes / (ms_cached * 1e-3) / 1e9 / world, 1),
                                     "frac_of_hbm_peak": round(cached_bytes / (ms_cached * 1e-3) / 1e9 / world / peaks["hbm_gbs"], 4)}}
    del q, k, v, cache
    torch.cuda.empty_cache()
    return out


def _secondary_only(args, which):
    """`--workload context|decode`: the secondary workload alone, as its own JSON line."""
    import torch
    import torch.distributed as dist
    import nsa_b200
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if which == "context":
        r = measure_context(torch, dist, nsa_b200, rank, world, dev, args.steps, args.warmup, single_gpu_base=args.base)
        value, ms, metric = r["tokens_per_s"], r["ms_per_step"], METRIC
    else:
        r = measure_decode(torch, dist, nsa_b200, rank, world, dev, args.steps, args.warmup)
        value, ms = r["with_compressed_cache"]["tokens_per_s"], r["with_compressed_cache"]["ms_per_step"]
        metric = "NSA decode tokens/s (one new token per sequence, compressed cache kept)"
    if rank == 0:
        print(json.dumps({"metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": r["workload"]},
                          "detail": r}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_context(args):
    _secondary_only(args, "context")


def run_decode(args):
    _secondary_only(args, "decode")


def run_profile_case():
    """Small case for ncu: the B=1 slice of the workload (q, dO 134 MB each: larger than L2, well under 1 GB on the
    device), every kernel family of the step launched twice, then two batched decode steps over 16 cached sequences."""
    import torch
    import nsa_b200
    from nsa_b200.decode import compress_cache, nsa_decode
    c = CFG
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(c["seed"])
    T, Hq, Hkv, D = c["T"], c["Hq"], c["Hkv"], c["D"]
    q, k, v, do = (torch.randn(1, T, h, D, generator=gen).to(dev, torch.bfloat16) for h in (Hq, Hkv, Hkv, Hq))
    mod = nsa_b200.NSAAttention(D, True, None, 0.0, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
        kern, keys = per_kernel_breakdown(torch, nsa_b200, mod, q, k, v, do, reps=1)
        lens = decode_lengths()[:16]
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        g2 = torch.Generator(device=dev).manual_seed(4)
        qd = torch.randn(len(lens), Hq, D, generator=g2, device=dev, dtype=torch.bfloat16)
        kd = torch.randn(cu[-1], Hkv, D, generator=g2, device=dev, dtype=torch.bfloat16)
        vd = torch.randn(cu[-1], Hkv, D, generator=g2, device=dev, dtype=torch.bfloat16)
        cache = compress_cache(mod, kd, vd, cu)
        for _ in range(2):
            nsa_decode(mod, qd, kd, vd, cu, cache=cache)
        torch.cuda.synchronize()
    nsa_b200._lib.device_status()
    print(json.dumps({"profile_case": "B=1 T=8192 Hq=64 Hkv=4 D=128; decode: 16 sequences, %d cached tokens" % cu[-1],
                      "kernels_ms": kern, "selected_keys": keys}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads (configs[1], [3], [4])")
    ap.add_argument("--base", action="store_true", help="--workload context with N > 1: also time the unsharded step on rank 0")
    ap.add_argument("--workload", default="module", choices=["module", "context", "decode"],
                    help="module: configs[2], batch-sharded (default).  context: configs[3], B=1 T=65536 context-sharded")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for ncu: B=1 of the workload, every kernel family launched twice, no timing loop")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.profile_case:
        run_profile_case()
    elif args.workload == "context":
        run_context(args)
    elif args.workload == "decode":
        run_decode(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
