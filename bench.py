#!/usr/bin/env python3
"""Benchmark of the GEMM path: one "step" = the linear-layer GEMMs of a training
step (forward, dX, dW+dbias for every layer) on synthetic seeded inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c3c|c4|c5] [--impl reference]

Workloads (shapes of the reference's benchmark configurations):
  c2  GPT-2-small, M = 8192 tokens per GPU, C = 768: QKV 768->2304, attention
      out-proj 768->768, MLP fc 768->3072 (bias+GELU fused), MLP proj 3072->768;
      bf16 operands, fp32 accumulation, bf16 activations, fp32 dW/dbias.
  c5  GPT-2-XL MLP, C = 1600, 4C = 6400, M = 8192 tokens per GPU.
  c3  LM head 768->50257, fp32 logits, row pitch 50264; c3c the same with contiguous
      [tokens, 50257] logits and dLogits; c4 the six attention products.
The headline (`value`) is c2.  At N = 1 the default run also times the other workloads
(`workloads`), every GEMM of c2 on its own next to cuBLASLt called the way llmt calls it but
with bf16 operands (`comparators`), a two-second replay of the step (`sustained`) and the CPU
baselines.  With N > 1 every GPU runs the same per-GPU workload on its own token shard (weak
scaling) and the fp32 dW/dbias span is summed layer by layer on a side stream (--exchange:
the library's kernel through NVSwitch multicast or peer copies, or NCCL), overlapped with
the backward launches of the remaining layers; the sum is checked against NCCL's
(`exchange_check`) and config 5's literal form, M = 65536 split N ways, is timed too
(`config.c5_strong`).

Prints ONE JSON line. `value` is device-timed throughput with inputs resident in
HBM; `e2e` is the same step called with HOST (pinned) buffers, copies included.
`--impl reference` runs the unmodified llmt library (cuBLASLt, strict fp32 — the
only precision llmt's matmul accepts) on the same shapes.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = {
    "c2": dict(name="gpt2-small linear layers", C=768,
               layers=[("qkv", 768, 2304, False), ("attn_out", 768, 768, False),
                       ("mlp_fc", 768, 3072, True), ("mlp_proj", 3072, 768, False)]),
    "c5": dict(name="gpt2-xl MLP", C=1600,
               layers=[("mlp_fc", 1600, 6400, True), ("mlp_proj", 6400, 1600, False)]),
    # tied-embedding LM head: fp32 logits, no bias, vocabulary 50257 in a row pitch of 50264 ...
    "c3": dict(name="LM head, vocab 50257 (row pitch 50264), fp32 logits", C=768, bias=False, y_fp32=True,
               ld_out=50264, layers=[("lm_head", 768, 50257, False)]),
    # ... or contiguous (row pitch 50257: TMA cannot address it; logits leave through registers,
    # dLogits is first copied to an aligned pitch)
    "c3c": dict(name="LM head, vocab 50257 (contiguous), fp32 logits", C=768, bias=False, y_fp32=True,
                ld_out=50257, layers=[("lm_head", 768, 50257, False)]),
}
M_PER_GPU = 8192
L2_BYTES = 126 << 20


def step_flops(workload: str, m: int) -> float:
    return sum(3 * 2.0 * m * i * o for _, i, o, _ in LAYERS[workload]["layers"])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"tf": float(d["bf16_tflops"]), "tf_sustained": float(d.get("bf16_tflops_sustained", 1400.0)),
                "bw": float(d["hbm_gbs"]), "which": "measured"}
    return {"tf": 1590.0, "tf_sustained": 1400.0, "bw": 6650.0, "which": "fallback"}


def recorded_traffic(workload: str):
    """DRAM bytes per step from the ncu capture recorded under profiles/ (null when none is
    recorded for this workload)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        return json.load(open(path)).get(workload)
    except (OSError, ValueError):
        return None


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU while a timed region runs:
    NVML polled every 2 ms from a thread (read-only queries), nvidia-smi at 100 ms as fallback."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, pci_bus_id: str = None):
        self.index, self.pci = index, pci_bus_id
        self.rows = []          # nvidia-smi rows
        self.samples = []       # (sm_mhz, power_w, reasons_mask) from NVML
        self.proc = None
        self.nvml = None
        self.stop_flag = False
        self.max_mhz = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByPciBusId(self.pci.encode()) if self.pci else \
                pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.nvml = (pynvml, h)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _poll(self):
        pynvml, h = self.nvml
        reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons",
                          getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons", None))
        while not self.stop_flag:
            try:
                mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                watts = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                mask = int(reasons(h)) if reasons else 0
                self.samples.append((mhz, watts, mask))
            except Exception:
                pass
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
            pynvml, _ = self.nvml

            def bit(event_name, throttle_name, default):
                return getattr(pynvml, event_name, getattr(pynvml, throttle_name, default))
            bits = {"hw_slowdown": bit("nvmlClocksEventReasonHwSlowdown", "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                    "hw_thermal_slowdown": bit("nvmlClocksEventReasonHwThermalSlowdown",
                                               "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                    "sw_thermal_slowdown": bit("nvmlClocksEventReasonSwThermalSlowdown",
                                               "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                    "sw_power_cap": bit("nvmlClocksEventReasonSwPowerCap", "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
            sm = sorted(s[0] for s in self.samples)
            mask = 0
            for s in self.samples:
                mask |= s[2]
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                    "sm_max_mhz": self.max_mhz, "samples": len(sm),
                    "power_w_max": round(max((s[1] for s in self.samples), default=0.0), 1),
                    "reasons": sorted(n for n, b in bits.items() if mask & b), "source": "nvml, 2 ms period"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi, 100 ms period"}


def make_sampler(torch, dev):
    props = torch.cuda.get_device_properties(dev)
    try:
        pci = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except AttributeError:
        pci = None
    return ClockSampler(dev.index or 0, pci)


# --------------------------------------------------------------------- own arm ---

class LinearStep:
    """Device tensors and prebuilt C-ABI descriptors of one training step's GEMMs.

    Launch order (what a network's data dependencies allow): the forward of every layer, then,
    walking the layers backwards, one launch per layer that holds its dX and dW + dbias
    (llmt's Linear::backward, src/layers/linear.cpp:22-30, as one grouped launch).  With
    `defer` = {layer: later layer}, the dW + dbias of `layer` is not launched with its own dX
    but rides in the backward launch of `later layer`, which runs after it: dW depends on
    nothing but dy and x of its own layer, so it may run any time after them, and a short
    layer's few long dW tiles balance better inside a larger launch."""

    def __init__(self, workload, m, dev, seed, world=1, exchange="peer", comm_ctas=8, defer=None, ride_min_gflop=30.0):
        import torch
        import llmt_b200 as L
        from llmt_b200.dp import GradBucket, PeerExchange
        self.L, self.torch, self.m, self.workload = L, torch, m, workload
        g = torch.Generator(device=dev).manual_seed(seed)
        bf = torch.bfloat16
        cfg = LAYERS[workload]
        spec = cfg["layers"]
        has_bias = cfg.get("bias", True)
        self.has_bias = has_bias
        shapes = {k: v for n, i, o, _ in spec for k, v in ((n + ".dW", (o, i)), (n + ".dbias", (o,)))}
        # N > 1: the span lives in peer-mapped memory and is summed by the library's own kernel
        # over NVLink ("peer" / "nvls"), or stays private and goes through NCCL ("nccl")
        self.exchange = None
        self.ride = False   # slices ride along in later backward launches (llmt_b200_gemm_grouped_exchange)
        self.ride_min_flops = ride_min_gflop * 1e9  # a launch shorter than this carries nothing: the exchange would outlast it
        if world > 1 and exchange in ("peer", "nvls", "ride"):
            try:
                self.exchange = PeerExchange(GradBucket.layout_numel(shapes), dev, ctas=comm_ctas,
                                             multicast=(exchange in ("nvls", "ride")))
            except Exception as exc:  # no peer mapping on this machine: every rank falls back to NCCL
                print(f"[bench] peer-mapped span unavailable ({exc}); using NCCL", file=sys.stderr)
            ok = torch.tensor([1 if self.exchange is not None else 0], device=dev)
            torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
            if int(ok.item()) == 0:
                self.exchange = None
            elif exchange in ("nvls", "ride") and not self.exchange.multicast:
                # no multicast mapping offered: the peer-copy kernel needs SMs of its own
                self.exchange.ctas = 16
                L.set_sm_budget(torch.cuda.get_device_properties(dev).multi_processor_count - 16)
            elif exchange == "ride":
                self.ride = True
        self.bucket = GradBucket(shapes, dev, storage=self.exchange.attach if self.exchange else None)
        self.layers = []
        for n, i, o, gelu in spec:
            t = dict(name=n, gelu=gelu, i=i, o=o)
            ld = cfg.get("ld_out", o)  # row pitch of the [m, out] tensors (padded vocabulary)
            t["x"] = torch.randn(m, i, device=dev, generator=g).to(bf)
            t["w"] = (torch.randn(o, i, device=dev, generator=g) * 0.02).to(bf)
            t["b"] = torch.randn(o, device=dev, generator=g) * 0.02 if has_bias else None
            scale = 1e-4 if workload.startswith("c3") else 0.01
            t["dy"] = (torch.randn(m, ld, device=dev, generator=g) * scale).to(bf)[:, :o]
            t["y"] = torch.empty(m, ld, device=dev, dtype=torch.float32 if cfg.get("y_fp32") else bf)[:, :o]
            t["dx"] = torch.empty(m, i, device=dev, dtype=bf)
            t["dw"], t["db"] = self.bucket.view(n + ".dW"), self.bucket.view(n + ".dbias")
            self.layers.append(t)
        by_name = {t["name"]: t for t in self.layers}
        defer = {k: v for k, v in (defer or {}).items() if k in by_name and v in by_name}
        riders = {}
        for src, dst in defer.items():
            riders.setdefault(dst, []).append(by_name[src])
        self.ws = []
        for t in self.layers:
            t["d_fwd"] = L.make_desc(t["y"], t["x"], t["w"], False, True, bias=t["b"], gelu=t["gelu"])
            need = L.workspace_bytes(t["d_fwd"], t["x"], t["w"])
            buf = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
            t["d_fwd"].workspace, t["d_fwd"].workspace_bytes = buf.data_ptr(), buf.numel()
            self.ws.append(buf)

            def dw_problem(u):
                return (L.make_desc(u["dw"], u["dy"], u["x"], True, False, beta=1.0,
                                    dbias=u["db"] if has_bias else None, dbias_beta=1.0), u["dw"], u["dy"], u["x"])
            probs = [(L.make_desc(t["dx"], t["dy"], t["w"], False, False), t["dx"], t["dy"], t["w"])]
            t["carries"] = []
            if t["name"] not in defer:
                probs.append(dw_problem(t))
                t["carries"].append(t)
            for u in riders.get(t["name"], []):
                probs.append(dw_problem(u))
                t["carries"].append(u)
            t["bwd"] = L.Group(probs)
            bufs = [torch.empty(max(b, 256), dtype=torch.uint8, device=dev) for b in t["bwd"].workspace_bytes()]
            t["bwd"].set_workspaces(bufs)
            self.ws += bufs
            t["bwd_flops"] = 2.0 * m * t["i"] * t["o"] + sum(2.0 * m * u["i"] * u["o"] for u in t["carries"])
        self.comm_stream = torch.cuda.Stream(device=dev)
        self.flops = step_flops(workload, m)

    def launches(self):
        """(label, flops, callable, layers whose gradients are complete after it) in launch order."""
        out = []
        for t in self.layers:
            f = 2.0 * self.m * t["i"] * t["o"]
            out.append((t["name"] + ".fwd", f, (lambda t=t: self.L.gemm_desc(t["d_fwd"], t["y"], t["x"], t["w"])), [], None))
        for t in reversed(self.layers):
            label = t["name"] + ".bwd(dX" + "".join("+dW_" + u["name"] for u in t["carries"]) + ")"
            out.append((label, t["bwd_flops"], t["bwd"].run, t["carries"], t["bwd"]))
        return out

    def slice_runs(self, layers):
        """(offset, count) of the dW + dbias slices of `layers`: a layer's dW and dbias are adjacent
        in the flat span, and so are the slices of neighbouring layers, so every run of neighbours
        is one range."""
        order = [t["name"] for t in self.layers]
        idx = sorted(order.index(t["name"]) for t in layers)
        runs, start = [], None
        for j, i in enumerate(idx):
            if start is None:
                start = i
            if j + 1 == len(idx) or idx[j + 1] != i + 1:
                runs.append((start, i))
                start = None
        out = []
        for lo_i, hi_i in runs:
            names = [order[i] + sfx for i in range(lo_i, hi_i + 1) for sfx in (".dW", ".dbias")]
            out.append(self.bucket.span_of(names) + ([self.layers[i] for i in range(lo_i, hi_i + 1)],))
        return out

    def exchange_layers(self, layers, stream=None):
        """Sums the dW + dbias slices of `layers` over the ranks with one call per range, on the
        side stream (or on `stream`)."""
        torch = self.torch
        stream = stream if stream is not None else self.comm_stream
        for off, cnt, _ in self.slice_runs(layers):
            if self.exchange is not None:
                self.exchange.allreduce(off, cnt, stream=stream)
            else:
                with torch.cuda.stream(stream):
                    torch.distributed.all_reduce(self.bucket.flat[off:off + cnt])

    def run(self, world=1, events=None, exchange=True, zero=True):
        """Enqueues one step on the current stream.  With world > 1 the gradients are summed over
        the ranks.  "ride": the slice a backward launch completes travels inside the NEXT backward
        launch (its epilogue warps sum it through the switch while the tensor pipe runs that
        launch's tiles); only the last launch's slice needs a call of its own.  Otherwise every
        slice is all-reduced on a side stream as soon as the launch that completes it is enqueued."""
        torch = self.torch
        if zero:
            self.bucket.zero_()
        exchange = exchange and world > 1
        ride = exchange and self.ride
        if ride:
            self.L.exchange_begin_step(self.exchange.desc)
        pending, index = [], 0
        for label, lflops, fn, done, group in self.launches():
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e0.record()
            if ride and pending and group is not None and lflops >= self.ride_min_flops:
                off, cnt, covered = self.slice_runs(pending)[0]
                group.run_with_exchange(self.exchange.desc, off, cnt, index)
                index += 1
                pending = [t for t in pending if all(t is not u for u in covered)]
            else:
                fn()
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True); e1.record()
                events.append((label, e0, e1))
            if ride:
                pending += done
            elif exchange and done:
                ready = torch.cuda.Event(); ready.record()
                self.comm_stream.wait_event(ready)
                self.exchange_layers(done)
        if ride:
            # what no later launch could carry; its flag rounds also close the step for the slices
            # that rode along (every rank has finished every earlier launch)
            self.exchange_layers(pending, stream=torch.cuda.current_stream())
        elif exchange:
            torch.cuda.current_stream().wait_stream(self.comm_stream)


class AttentionStep:
    """Configuration 4: the six strided-batched attention products at B*H = 96, T = 1024, hd = 64
    (llmt src/kernels/attention.cpp:60-62 forward, docs/TODO.md:226-228 backward), bf16.
    P and dS are produced once by the softmax helpers outside the timed set. HBM-bound:
    every product moves one [96, T, T] matrix."""
    BH, T, HD = 96, 1024, 64

    def __init__(self, dev, seed, fused=False):
        import torch
        import llmt_b200 as L
        self.L, self.torch = L, torch
        g = torch.Generator(device=dev).manual_seed(seed)
        bf = torch.bfloat16
        BH, T, HD = self.BH, self.T, self.HD
        mk = lambda *shape, scale=1.0: (torch.randn(*shape, device=dev, generator=g) * scale).to(bf)
        self.q, self.k, self.v = mk(BH, T, HD), mk(BH, T, HD), mk(BH, T, HD)
        self.d_o = mk(BH, T, HD, scale=0.01)
        self.s = torch.empty(BH, T, T, device=dev, dtype=bf)
        self.p = torch.empty_like(self.s)
        self.dp = torch.empty_like(self.s)
        self.ds = torch.empty_like(self.s)
        self.o, self.dv, self.dq, self.dk = (torch.empty(BH, T, HD, device=dev, dtype=bf) for _ in range(4))
        a = 1.0 / 8.0
        L.gemm(self.s, self.q, self.k, False, True, alpha=a)
        L.softmax_fwd(self.p, self.s, causal=True)
        L.gemm(self.dp, self.d_o, self.v, False, True)
        L.softmax_bwd(self.ds, self.p, self.dp)
        md = L.make_desc
        self.calls = [
            ("S=aQK^T", md(self.s, self.q, self.k, False, True, alpha=a), self.s, self.q, self.k),
            ("O=PV", md(self.o, self.p, self.v, False, False), self.o, self.p, self.v),
            ("dV=P^TdO", md(self.dv, self.p, self.d_o, True, False), self.dv, self.p, self.d_o),
            ("dP=dOV^T", md(self.dp, self.d_o, self.v, False, True), self.dp, self.d_o, self.v),
            ("dQ=adSK", md(self.dq, self.ds, self.k, False, False, alpha=a), self.dq, self.ds, self.k),
            ("dK=adS^TQ", md(self.dk, self.ds, self.q, True, False, alpha=a), self.dk, self.ds, self.q),
        ]
        self.flops_each = 2.0 * BH * T * T * HD
        self.flops = 6 * self.flops_each
        # minimum bytes of one product: the [BH,T,T] matrix once plus three [BH,T,hd] tensors
        self.bytes_each = 2.0 * (BH * T * T + 3 * BH * T * HD)
        self.bytes_step = 6 * self.bytes_each
        self.fused = fused
        if fused:
            # Configuration 4 with the softmax inside the timed set, fused around the products
            # (llmt_b200_gemm_softmax_fwd / _bwd): S and dP are never stored.  The FLOP count stays
            # the six dense products' (the second pass over the score tiles is not counted);
            # bytes: P written once, read by O, dV and dS, dS written once, read by dQ and dK.
            self.lse = torch.empty(BH, T, device=dev)
            self.dvec = torch.empty(BH, T, device=dev)
            self.d_s = md(self.p, self.q, self.k, False, True, alpha=a)
            need = L.gemm_softmax_workspace_bytes(self.d_s, self.q, self.k)
            self.ws_s = torch.empty(need, dtype=torch.uint8, device=dev)
            self.d_s.workspace, self.d_s.workspace_bytes = self.ws_s.data_ptr(), need
            self.d_b = md(self.ds, self.d_o, self.v, False, True)
            self.ws_b = torch.empty(max(L.workspace_bytes(self.d_b, self.d_o, self.v), 256), dtype=torch.uint8, device=dev)
            self.d_b.workspace, self.d_b.workspace_bytes = self.ws_b.data_ptr(), self.ws_b.numel()
            L.gemm_desc(self.calls[1][1], self.o, self.p, self.v)
            self.bytes_step = 2.0 * (7 * BH * T * T + 16 * BH * T * HD)

    def launches(self):
        plain = [(lab, self.flops_each, (lambda d=d, c=c, a=a, b=b: self.L.gemm_desc(d, c, a, b)), [])
                 for lab, d, c, a, b in self.calls]
        if not self.fused:
            return plain
        L = self.L

        def fwd():
            L.gemm_softmax_fwd(self.d_s, self.p, self.q, self.k, True, self.lse)

        def bwd():
            L.rowdot(self.dvec, self.d_o, self.o)
            L.gemm_softmax_bwd(self.d_b, self.ds, self.d_o, self.v, self.p, self.dvec, True)

        return [("P=softmax(aQK^T)", self.flops_each, fwd, []), plain[1], plain[2],
                ("dS=P*(dOV^T-D)", self.flops_each, bwd, []), plain[4], plain[5]]

    def run(self, world=1, events=None):
        torch = self.torch
        for label, _, fn, _l in self.launches():
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e0.record()
            fn()
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True); e1.record()
                events.append((label, e0, e1))


def make_step(workload, m, dev, seed, world=1, args=None):
    if workload in ("c4", "c4f"):
        return AttentionStep(dev, seed, fused=workload == "c4f")
    defer = {"attn_out": "qkv"} if workload == "c2" and not (args and args.no_defer) else None
    return LinearStep(workload, m, dev, seed, world=world, exchange=args.exchange if args else "nccl",
                      comm_ctas=(args.comm_ctas if args and args.comm_ctas else 8), defer=defer,
                      ride_min_gflop=(args.ride_min_gflop if args else 30.0))


def timed_steps(torch, L, step, world, steps, warmup, use_graph, barrier):
    """W untimed steps, then exactly K steps between CUDA events.  One step (its GEMM launches
    and, for N > 1, the gradient exchanges on the side stream) is captured into a CUDA graph and
    replayed, so the host enqueues one graph per step instead of a dozen launches."""
    for _ in range(warmup):
        step.run(world)
    barrier()
    graph, per_step = None, None
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            n0 = L.launch_count()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                step.run(world)
            per_step = L.launch_count() - n0
            for _ in range(warmup):
                graph.replay()
        except Exception as exc:  # capture refused: fall back to direct launches and say so
            print(f"[bench] graph capture failed ({exc}); launching directly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    barrier()
    n0 = L.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps):
        if graph is not None:
            graph.replay()
        else:
            step.run(world)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    launches = per_step * steps if graph is not None else L.launch_count() - n0
    return ms, int(launches), graph


def sustained_replay(torch, graph, step, dev, seconds, flops, peaks):
    """The same step replayed for `seconds`: long enough for the power governor to settle."""
    sampler = make_sampler(torch, dev).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_end = time.perf_counter() + seconds
    n = 0
    e0.record()
    while time.perf_counter() < t_end:
        for _ in range(50):
            if graph is not None:
                graph.replay()
            else:
                step.run(1)
        n += 50
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    clocks = sampler.stop()
    tf = flops / ms / 1e9
    return {"tflops": round(tf, 1), "ms_per_step": round(ms, 4), "steps": n, "seconds": round(ms * n / 1e3, 2),
            "sm_mhz_median": clocks.get("sm_mhz"), "power_w_max": clocks.get("power_w_max"),
            "reasons": clocks.get("reasons"), "clock_samples": clocks.get("samples"),
            "frac_of_sustained_peak": round(tf / peaks["tf_sustained"], 4),
            "ms_x_ghz": round(ms * (clocks.get("sm_mhz") or 0) / 1e3, 4)}


class HostPipeline:
    """A step driven from HOST buffers, as an input pipeline would: every step its inputs travel
    from pinned host memory to the device and its result travels back, all inside the timed
    region.  The copy of step i+1's inputs (on a copy stream, into a staging set) overlaps step
    i's kernels; the compute stream moves the staged inputs into place with a device copy, runs
    the step, and a third stream carries the result to the host."""

    def __init__(self, torch, inputs, outputs, run_fn):
        """inputs / outputs: lists of (pinned host tensor, device tensor)."""
        self.torch, self.inputs, self.outputs, self.run_fn = torch, inputs, outputs, run_fn
        self.stage = [torch.empty_like(d) for _, d in inputs]
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.staged, self.stage_free, self.done, self.out_copied = (torch.cuda.Event() for _ in range(4))
        self.h2d_bytes = sum(h.numel() * h.element_size() for h, _ in inputs)
        self.d2h_bytes = sum(h.numel() * h.element_size() for h, _ in outputs)

    def run(self, steps):
        torch = self.torch
        main = torch.cuda.current_stream()
        self.stage_free.record(main)
        self.out_copied.record(main)
        for _ in range(steps):
            self.s_in.wait_event(self.stage_free)
            with torch.cuda.stream(self.s_in):
                for (h, _), s in zip(self.inputs, self.stage):
                    s.copy_(h, non_blocking=True)
                self.staged.record(self.s_in)
            main.wait_event(self.staged)
            for (_, d), s in zip(self.inputs, self.stage):
                d.copy_(s, non_blocking=True)
            self.stage_free.record(main)
            main.wait_event(self.out_copied)   # the previous result has left before it is overwritten
            self.run_fn()
            self.done.record(main)
            self.s_out.wait_event(self.done)
            with torch.cuda.stream(self.s_out):
                for h, d in self.outputs:
                    h.copy_(d, non_blocking=True)
                self.out_copied.record(self.s_out)
        main.wait_event(self.out_copied)


class HostStep(HostPipeline):
    """The own arm's step from host buffers: the layer inputs (x, dy) in, the reduced gradient span out."""

    def __init__(self, step: "LinearStep", world: int):
        torch = step.torch
        inputs = [(torch.empty_like(t[k], device="cpu").pin_memory().copy_(t[k]), t[k])
                  for t in step.layers for k in ("x", "dy")]
        outputs = [(torch.empty_like(step.bucket.flat, device="cpu").pin_memory(), step.bucket.flat)]
        super().__init__(torch, inputs, outputs, lambda: step.run(world))


# ------------------------------------------------------------- per-GEMM comparisons ---

def gemm_list(workload, m):
    """Every GEMM of the step: (label, kind, m, n, k, trans_a, trans_b, layer index)."""
    out = []
    for li, (n_, i, o, gelu) in enumerate(LAYERS[workload]["layers"]):
        out.append((n_ + ".fwd", "fwd", m, o, i, False, True, li))
        out.append((n_ + ".dX", "dx", m, i, o, False, False, li))
        out.append((n_ + ".dW", "dw", o, i, m, True, False, li))
    return out


def _loop_ms(torch, fns, iters=20, warm=3):
    """Mean time of one call when the calls in `fns` (the same GEMM on rotating buffer sets, so
    that no iteration finds its operands in L2) run back to back."""
    for w in range(warm):
        fns[w % len(fns)]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for it in range(iters):
        fns[it % len(fns)]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def lm_head_ce_comparison(torch, L, m, dev):
    """The LM-head forward of config 3 with its consumer, the cross-entropy (llmt
    src/kernels/cross_entropy.cu): the product stored as fp32 logits and read back by
    cross_entropy_fwd, against llmt_b200_lm_head_ce_fwd, whose epilogue keeps the row statistics so
    that the 1.65 GB of logits are never written.  Same loss (checked), times by CUDA events."""
    bf = torch.bfloat16
    V, C, LD = 50257, 768, 50264
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(m, C, device=dev, generator=g).to(bf)
    w = (torch.randn(V, C, device=dev, generator=g) * 0.02).to(bf)
    tg = torch.randint(0, V, (m,), device=dev, generator=g, dtype=torch.int32)
    mk = torch.ones(m, device=dev)
    logits = torch.empty(m, LD, device=dev)[:, :V]
    d1 = L.make_desc(logits, x, w, False, True)
    loss1, nll1 = torch.empty(1, device=dev), torch.empty(m, device=dev)

    def unfused():
        L.gemm_desc(d1, logits, x, w)
        L.cross_entropy_fwd(loss1, nll1, logits, tg, mk)

    d2 = L.GemmDesc()
    d2.m, d2.n, d2.k, d2.batch = m, V, C, 1
    d2.lda, d2.ldb, d2.ldc = C, C, V
    d2.trans_a, d2.trans_b = 0, 1
    d2.dtype_ab, d2.dtype_c = L.BF16, L.FP32
    d2.alpha = 1.0
    need = L.lm_head_ce_workspace_bytes(d2, x, w)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    d2.workspace, d2.workspace_bytes = ws.data_ptr(), need
    loss2, nll2 = torch.empty(1, device=dev), torch.empty(m, device=dev)

    def fused():
        L.lm_head_ce_fwd(d2, None, x, w, tg, mk, nll2, loss2)

    ms_u = _loop_ms(torch, [unfused], iters=10, warm=3)
    ms_f = _loop_ms(torch, [fused], iters=10, warm=3)
    L.device_status()
    # backward: dlogits in place of the stored logits (llmt's plan, docs/TODO.md:216-217) against the
    # product made again with the gradient as its epilogue (bf16 dlogits, no logits in memory)
    dl = torch.empty(m, LD, device=dev, dtype=bf)[:, :V]
    d3 = L.GemmDesc()
    d3.m, d3.n, d3.k, d3.batch = m, V, C, 1
    d3.lda, d3.ldb, d3.ldc = C, C, LD
    d3.trans_a, d3.trans_b = 0, 1
    d3.dtype_ab, d3.dtype_c = L.BF16, L.BF16
    d3.alpha = 1.0
    d3.workspace, d3.workspace_bytes = ws.data_ptr(), need

    def bwd_unfused():
        L.cross_entropy_bwd(logits, logits, tg, mk)

    def bwd_fused():
        L.lm_head_ce_bwd(d3, dl, x, w, tg, mk, 1.0, True)

    fused()  # leaves the statistics the fused backward reuses
    ms_bf = _loop_ms(torch, [bwd_fused], iters=10, warm=3)
    unfused()
    ref = torch.empty_like(logits)
    L.cross_entropy_bwd(ref, logits, tg, mk)
    bwd_err = float(((dl.float() - ref).norm() / ref.norm()).item())
    del ref
    ms_bu = _loop_ms(torch, [bwd_unfused], iters=10, warm=3)  # (in place: later iterations read gradients, same traffic)
    L.device_status()
    flops = 2.0 * m * V * C
    return {"shape": f"{m} x {V} x {C}, bf16 operands, fp32 logits (pitch {LD})",
            "gemm_then_cross_entropy_ms": round(ms_u, 4), "fused_ms": round(ms_f, 4),
            "gemm_then_cross_entropy_tflops": round(flops / ms_u / 1e9, 1), "fused_tflops": round(flops / ms_f / 1e9, 1),
            "loss_unfused": float(loss1.item()), "loss_fused": float(loss2.item()),
            "losses_agree": bool(abs(float(loss1.item()) - float(loss2.item())) <= 1e-4 * abs(float(loss1.item()))),
            "logit_bytes_not_written": int(m) * V * 4,
            "bwd_cross_entropy_bwd_in_place_ms": round(ms_bu, 4), "bwd_fused_ms": round(ms_bf, 4),
            "bwd_rel_fro_diff": bwd_err}


def attention_softmax_comparison(torch, L, dev):
    """Config 4's softmax, forward and backward (llmt src/kernels/attention.cpp:60-62,
    docs/TODO.md:226-228), at B*H = 96, T = 1024, hd = 64, bf16, causal: llmt's composition (scores
    GEMM, softmax kernel in place; dP GEMM, softmax-backward kernel) against the fused launches
    (llmt_b200_gemm_softmax_fwd: the scores are never stored; llmt_b200_gemm_softmax_bwd: dP is never
    stored).  Rotating buffer sets larger than L2, times by CUDA events, results compared."""
    bf = torch.bfloat16
    BH, T, HD = 96, 1024, 64
    g = torch.Generator(device=dev).manual_seed(11)
    sets = []
    for _ in range(2):  # 2 x (4 x 201 MB of T x T tensors) > L2
        q, k, v = (torch.randn(BH, T, HD, device=dev, generator=g).to(bf) for _ in range(3))
        do = (torch.randn(BH, T, HD, device=dev, generator=g) * 0.01).to(bf)
        s_u, p_f, ds_u, ds_f = (torch.empty(BH, T, T, device=dev, dtype=bf) for _ in range(4))
        o = torch.empty(BH, T, HD, device=dev, dtype=bf)
        dvec = torch.empty(BH, T, device=dev)
        d_s = L.make_desc(p_f, q, k, False, True, alpha=0.125)
        need = L.gemm_softmax_workspace_bytes(d_s, q, k)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        d_s.workspace, d_s.workspace_bytes = ws.data_ptr(), need
        d_b = L.make_desc(ds_f, do, v, False, True)
        wsb = torch.empty(max(L.workspace_bytes(d_b, do, v), 256), dtype=torch.uint8, device=dev)
        d_b.workspace, d_b.workspace_bytes = wsb.data_ptr(), wsb.numel()
        sets.append(dict(q=q, k=k, v=v, do=do, s_u=s_u, p_f=p_f, ds_u=ds_u, ds_f=ds_f, o=o, dvec=dvec,
                         d_s=d_s, d_b=d_b, ws=ws, wsb=wsb))

    def fwd_unfused(z):
        L.gemm(z["s_u"], z["q"], z["k"], False, True, alpha=0.125)
        L.softmax_fwd(z["s_u"], z["s_u"], causal=True)

    def fwd_fused(z):
        L.gemm_softmax_fwd(z["d_s"], z["p_f"], z["q"], z["k"], True)

    def bwd_unfused(z):
        L.gemm(z["ds_u"], z["do"], z["v"], False, True)
        L.softmax_bwd(z["ds_u"], z["p_f"], z["ds_u"])

    def bwd_fused(z):
        L.rowdot(z["dvec"], z["do"], z["o"])
        L.gemm_softmax_bwd(z["d_b"], z["ds_f"], z["do"], z["v"], z["p_f"], z["dvec"], True)

    out = {"shape": f"B*H = {BH}, T = {T}, hd = {HD}, bf16, causal; one T x T tensor is {BH * T * T * 2} bytes"}
    def best_of_two(fn):  # (the first loop after the allocations above has been seen to run long once)
        return min(_loop_ms(torch, [lambda z=z, fn=fn: fn(z) for z in sets], iters=10, warm=3) for _ in range(2))

    for name, fn in (("fwd_gemm_then_softmax_ms", fwd_unfused), ("fwd_fused_ms", fwd_fused)):
        out[name] = round(best_of_two(fn), 4)
    for z in sets:
        L.gemm(z["o"], z["p_f"], z["v"], False, False)
    for name, fn in (("bwd_gemm_then_softmax_bwd_ms", bwd_unfused), ("bwd_fused_ms", bwd_fused)):
        out[name] = round(best_of_two(fn), 4)
    L.device_status()
    z = sets[0]
    p_u, p_f = z["s_u"].float(), z["p_f"].float()
    out["fwd_max_abs_diff"] = float((p_u - p_f).abs().max().item())
    out["fwd_masked_exact_zero"] = bool((torch.triu(p_f[0], 1) == 0).all().item())
    ds_u, ds_f = z["ds_u"].float(), z["ds_f"].float()
    out["bwd_rel_fro_diff"] = float(((ds_u - ds_f).norm() / ds_u.norm()).item())
    out["t_x_t_bytes_not_moved"] = {"fwd": 2 * BH * T * T * 2, "bwd": 2 * BH * T * T * 2}
    return out


def mlp_gelu_comparison(torch, L, m, dev):
    """The GELU between the two MLP GEMMs of config 2 (C = 768, 4C = 3072) in training: forward keeping
    the pre-activation (llmt src/layers/mlp.cpp:14-18 runs matmul -> gelu kernel -> matmul) and the
    backward of the down projection with dX passing through the GELU (llmt docs/TODO.md:223 plans a
    gelu_bwd kernel).  Composition = this library's GEMMs plus torch's element-wise gelu /
    gelu_backward (tanh form); fused = EPI_SAVE_PRE / EPI_GELU_BWD.  Rotating sets, CUDA events."""
    bf = torch.bfloat16
    C, F = 768, 3072
    g = torch.Generator(device=dev).manual_seed(21)
    sets = []
    for _ in range(3):
        x = torch.randn(m, C, device=dev, generator=g).to(bf)
        w1 = (torch.randn(F, C, device=dev, generator=g) * 0.02).to(bf)
        b1 = torch.zeros(F, device=dev)
        w2 = (torch.randn(C, F, device=dev, generator=g) * 0.02).to(bf)
        dy = (torch.randn(m, C, device=dev, generator=g) * 0.01).to(bf)
        z = dict(x=x, w1=w1, b1=b1, w2=w2, dy=dy)
        for name in ("h", "pre", "h_u", "pre_u", "dpre", "dh_u"):
            z[name] = torch.empty(m, F, device=dev, dtype=bf)
        z["dw2"] = torch.zeros(C, F, device=dev)
        z["dw2_u"] = torch.zeros(C, F, device=dev)
        z["d_f"] = L.make_desc(z["h"], x, w1, False, True, bias=b1, gelu=True, save_pre=z["pre"])
        z["d_pre"] = L.make_desc(z["pre_u"], x, w1, False, True, bias=b1)
        L.gemm_desc(z["d_f"], z["h"], x, w1)
        gf = L.Group([(L.make_desc(z["dpre"], dy, w2, False, False, gelu_bwd_of=z["pre"]), z["dpre"], dy, w2),
                      (L.make_desc(z["dw2"], dy, z["h"], True, False, beta=1.0), z["dw2"], dy, z["h"])])
        gu = L.Group([(L.make_desc(z["dh_u"], dy, w2, False, False), z["dh_u"], dy, w2),
                      (L.make_desc(z["dw2_u"], dy, z["h"], True, False, beta=1.0), z["dw2_u"], dy, z["h"])])
        for grp in (gf, gu):
            bufs = [torch.empty(max(n, 256), dtype=torch.uint8, device=dev) for n in grp.workspace_bytes()]
            grp.set_workspaces(bufs)
        z["gf"], z["gu"] = gf, gu
        sets.append(z)

    def fwd_fused(z):
        L.gemm_desc(z["d_f"], z["h"], z["x"], z["w1"])

    def fwd_composed2(z):
        L.gemm_desc(z["d_pre"], z["pre_u"], z["x"], z["w1"])
        z["h_u"].copy_(torch.nn.functional.gelu(z["pre_u"], approximate="tanh"))

    def bwd_fused(z):
        z["gf"].run()

    def bwd_composed(z):
        z["gu"].run()
        z["dh_u"].copy_(torch.ops.aten.gelu_backward(z["dh_u"], z["pre"], approximate="tanh"))

    out = {"shape": f"M = {m}, C = {C}, 4C = {F}, bf16"}
    for name, fn in (("fwd_fused_two_results_ms", fwd_fused), ("fwd_gemm_then_gelu_ms", fwd_composed2),
                     ("bwd_fused_ms", bwd_fused), ("bwd_grouped_then_gelu_backward_ms", bwd_composed)):
        out[name] = round(_loop_ms(torch, [lambda z=z, fn=fn: fn(z) for z in sets], iters=12, warm=3), 4)
    L.device_status()
    z = sets[0]
    out["fwd_h_max_abs_diff"] = float((z["h"].float() - z["h_u"].float()).abs().max().item())
    out["bwd_rel_fro_diff"] = float(((z["dpre"].float() - z["dh_u"].float()).norm() / z["dh_u"].float().norm()).item())
    return out


def per_gemm_comparison(torch, L, workload, m, dev, want_cublaslt=True):
    """Each GEMM of the step timed on its own, back to back on rotating buffer sets (> 2 x L2
    in total), for this library and for cuBLASLt called the way llmt calls it (operand swap,
    32 MiB workspace, cached top-1 heuristic; llmt src/kernels/matmul.cpp:99-170) but with
    bf16 operands and fp32 accumulation.  Fused cases are timed for cuBLASLt both with its own
    epilogues (BIAS, GELU_BIAS, bias gradient) and as the unfused composition (plain GEMM, then
    torch element-wise kernels / a torch column sum)."""
    cfg = LAYERS[workload]
    has_bias = cfg.get("bias", True)
    lt = None
    notes = {}
    if want_cublaslt:
        try:
            from oracle import cublaslt_ref
            if cublaslt_ref.available():
                lt = cublaslt_ref.CublasLtBf16()
            else:
                notes["cublaslt_bf16"] = "comparator library not built (make -C oracle cmp)"
        except Exception as exc:
            notes["cublaslt_bf16"] = f"unavailable: {exc}"
    g = torch.Generator(device=dev).manual_seed(1234)
    bf = torch.bfloat16
    own, lib_fused, lib_unfused = {}, {}, {}
    for label, kind, gm, gn, gk, ta, tb, li in gemm_list(workload, m):
        _, i, o, gelu = cfg["layers"][li]
        cdt = torch.float32 if kind == "dw" or (kind == "fwd" and cfg.get("y_fp32")) else bf
        set_bytes = 2 * (gm * gk + gk * gn) + gm * gn * (4 if cdt == torch.float32 else 2)
        n_sets = max(2, min(8, -(-2 * L2_BYTES // set_bytes)))
        sets = []
        for _ in range(n_sets):
            a = torch.randn((gk, gm) if ta else (gm, gk), device=dev, generator=g).mul_(0.01 if kind != "fwd" else 1.0).to(bf)
            b = torch.randn((gn, gk) if tb else (gk, gn), device=dev, generator=g).mul_(0.02).to(bf)
            c = torch.zeros(gm, gn, device=dev, dtype=cdt)
            bias = (torch.randn(gn, device=dev, generator=g) * 0.02) if (kind == "fwd" and has_bias) else None
            db = torch.zeros(gm, device=dev) if (kind == "dw" and has_bias) else None
            sets.append((a, b, c, bias, db))
        flops = 2.0 * gm * gn * gk
        # this library
        fns, keep = [], []
        for a, b, c, bias, db in sets:
            d = L.make_desc(c, a, b, ta, tb, beta=1.0 if kind == "dw" else 0.0, bias=bias,
                            gelu=(kind == "fwd" and gelu), dbias=db, dbias_beta=1.0)
            need = L.workspace_bytes(d, a, b)
            ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
            d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
            keep.append((d, ws))
            fns.append(lambda d=d, c=c, a=a, b=b: L.gemm_desc(d, c, a, b))
        own[label] = round(flops / _loop_ms(torch, fns) / 1e9, 1)
        if lt is None:
            continue
        # cuBLASLt, fused epilogues (bias in C's type, as Lt requires)
        try:
            fns = []
            for a, b, c, bias, db in sets:
                lb = bias.to(c.dtype) if bias is not None else None
                fns.append(lambda a=a, b=b, c=c, lb=lb, db=db: lt.matmul(
                    c, a, b, ta, tb, beta=1.0 if kind == "dw" else 0.0, bias=lb,
                    gelu=(kind == "fwd" and gelu and lb is not None), dbias=db))
            lib_fused[label] = round(flops / _loop_ms(torch, fns) / 1e9, 1)
        except Exception as exc:
            lib_fused[label] = None
            notes["fused:" + label] = str(exc)
        # cuBLASLt, unfused composition
        try:
            fns = []
            for a, b, c, bias, db in sets:
                tmp = torch.empty(gm, device=dev) if db is not None else None
                c2 = torch.empty_like(c) if (kind == "fwd" and gelu) else None

                def unfused(a=a, b=b, c=c, bias=bias, db=db, tmp=tmp, c2=c2):
                    lt.matmul(c, a, b, ta, tb, beta=1.0 if kind == "dw" else 0.0)
                    if bias is not None:
                        c.add_(bias.to(c.dtype))
                    if c2 is not None:
                        torch.ops.aten.gelu.out(c, approximate="tanh", out=c2)
                    if db is not None:
                        torch.sum(a, dim=0, dtype=torch.float32, out=tmp)
                        db.add_(tmp)
                fns.append(unfused)
            lib_unfused[label] = round(flops / _loop_ms(torch, fns) / 1e9, 1)
        except Exception as exc:
            lib_unfused[label] = None
            notes["unfused:" + label] = str(exc)
        del sets, fns
    if lt is not None:
        lt.close()
    glist = gemm_list(workload, m)
    total = sum(2.0 * gm * gn * gk for _, _, gm, gn, gk, *_ in glist)

    def step_rate(table):
        if not table or any(table.get(lab) in (None, 0) for lab, *_ in glist):
            return None
        t = sum(2.0 * gm * gn * gk / (table[lab] * 1e9) for lab, _, gm, gn, gk, *_ in glist)
        return round(total / t / 1e9, 1)
    out = {"own_per_gemm_tflops": own, "own_step_tflops_sum_of_gemms": step_rate(own),
           "method": "each GEMM alone, 20 calls back to back after 3 warm-up calls, CUDA events, operands "
                     "rotating over buffer sets larger than twice L2"}
    if lt is not None or lib_fused:
        best = {lab: max(v for v in (lib_fused.get(lab), lib_unfused.get(lab)) if v) if
                (lib_fused.get(lab) or lib_unfused.get(lab)) else None for lab, *_ in glist}
        out["cublaslt_bf16"] = {
            "per_gemm_tflops_lt_epilogues": lib_fused, "per_gemm_tflops_unfused": lib_unfused,
            "step_tflops_lt_epilogues": step_rate(lib_fused), "step_tflops_unfused": step_rate(lib_unfused),
            "step_tflops": step_rate(best),
            "own_over_cublaslt": {lab: (round(own[lab] / best[lab], 3) if best.get(lab) else None) for lab, *_ in glist},
            "call_pattern": "llmt src/kernels/matmul.cpp:99-170 (operand swap, 32 MiB workspace, cached top-1 "
                            "heuristic) with CUDA_R_16BF operands and CUBLAS_COMPUTE_32F"}
    if notes:
        out["notes"] = notes
    return out


# -------------------------------------------------------------------- CPU baselines ---

def _best_median(fn, reps):
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter(); fn(); ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[0], ts[len(ts) // 2]


def cpu_baseline(workload):
    """Config 1 of the reference's benchmark set on this host's cores: the single fp32 linear
    forward Y = X W^T + b, X [256,768] ~ N(0,1), W [3072,768] ~ N(0,0.02), b ~ N(0,0.02), seed 0.
    Timed for the C port of the path (oracle/oracle.c, fp32, OpenMP) and for PyTorch on CPU,
    which is what llmt's own known-answer files were computed with (tools/gen_golden.py:94-98).
    `value` is the C port's best; a sample of the headline workload's shapes is timed beside it."""
    import numpy as np
    from oracle import oracle
    rng = np.random.default_rng(0)
    x = rng.standard_normal((256, 768)).astype(np.float32)
    w = (rng.standard_normal((3072, 768)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(3072) * 0.02).astype(np.float32)
    flops1 = 2.0 * 256 * 3072 * 768

    def port():
        y = oracle.gemm_f32(x, w, False, True)
        y += b
        return y
    port()
    best, med = _best_median(port, 25)
    out = {"value": round(flops1 / best / 1e12, 4), "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
           "sample": "config 1 itself: Y = X W^T + b, [256,768] x [3072,768]^T, fp32, seed 0 (1.208 GFLOP), "
                     "best of 25 runs of the OpenMP C port",
           "config1": {"port_best_ms": round(best * 1e3, 3), "port_median_ms": round(med * 1e3, 3),
                       "port_best_tflops": round(flops1 / best / 1e12, 4)}}
    try:
        import torch
        torch.manual_seed(0)
        tx, tw, tb = torch.randn(256, 768), torch.randn(3072, 768) * 0.02, torch.randn(3072) * 0.02
        fn = lambda: tx @ tw.T + tb
        fn()
        tbest, tmed = _best_median(fn, 25)
        out["config1"].update({"torch_cpu_best_ms": round(tbest * 1e3, 3), "torch_cpu_median_ms": round(tmed * 1e3, 3),
                               "torch_cpu_best_tflops": round(flops1 / tbest / 1e12, 4),
                               "torch_cpu_threads": torch.get_num_threads()})
    except Exception:
        pass
    # a bounded sample of the headline workload: the first 256 token rows of every GEMM of the step
    rows = 256
    spec = LAYERS[workload if workload in LAYERS else "c2"]["layers"]
    data = [(rng.standard_normal((rows, i)).astype(np.float32),
             (rng.standard_normal((o, i)) * 0.02).astype(np.float32),
             (rng.standard_normal((rows, o)) * 0.01).astype(np.float32)) for _, i, o, _g in spec]
    flops = sum(3 * 2.0 * rows * i * o for _, i, o, _ in spec)

    def one_pass():
        for xx, ww, dy in data:
            oracle.gemm_f32(xx, ww, False, True)
            oracle.gemm_f32(dy, ww, False, False)
            oracle.gemm_f32(dy, xx, True, False)
    one_pass()
    t_best, t_total, n = 1e30, 0.0, 0
    while t_total < 6.0 and n < 20:
        t0 = time.perf_counter(); one_pass(); dt = time.perf_counter() - t0
        t_best = min(t_best, dt); t_total += dt; n += 1
    out["step_sample"] = {"tflops": round(flops / t_best / 1e12, 4),
                          "sample": f"first {rows} token rows of every GEMM of the step ({flops / 1e9:.1f} GFLOP), "
                                    f"best of {n} passes of the C port"}
    return out


# --------------------------------------------------------------- reference arm ---

class ReferenceStep:
    """The same GEMMs through the unmodified llmt library: kernels::matmul (cuBLASLt, strict
    fp32), GELU as llmt's separate kernel (src/layers/mlp.cpp:14-18), no bias (llmt has none)."""

    def __init__(self, workload, m, dev, seed):
        import torch
        from oracle import llmt_ref
        self.torch = torch
        self.ref = llmt_ref.Llmt(dev.index or 0)
        g = torch.Generator(device=dev).manual_seed(seed)
        self.layers = []
        for n, i, o, gelu in LAYERS[workload]["layers"]:
            t = dict(name=n, gelu=gelu)
            t["x"] = torch.randn(m, i, device=dev, generator=g)
            t["w"] = torch.randn(o, i, device=dev, generator=g) * 0.02
            t["dy"] = torch.randn(m, o, device=dev, generator=g) * 0.01
            t["y"] = torch.empty(m, o, device=dev)
            t["dx"] = torch.empty(m, i, device=dev)
            t["dw"] = torch.zeros(o, i, device=dev)
            self.layers.append(t)

    def run(self):
        r = self.ref
        for t in self.layers:
            r.matmul(t["y"], t["x"], t["w"], False, True)
            if t["gelu"]:
                r.gelu(t["y"], t["y"])
        for t in reversed(self.layers):
            t["dw"].zero_()
            r.matmul(t["dw"], t["dy"], t["x"], True, False, 1.0, 1.0)
        for t in reversed(self.layers):
            r.matmul(t["dx"], t["dy"], t["w"], False, False)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import llmt_ref
    workload = args.workload if args.workload in LAYERS else "c2"
    flops = step_flops(workload, M_PER_GPU)
    base = {"impl": "reference", "metric": "GEMM TFLOP/s (fwd+dX+dW), whole job",
            "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": f"{workload}: {LAYERS[workload]['name']}, "
                                   f"M={M_PER_GPU} tokens, fwd+dX+dW per layer",
                       "l2": "working set larger than L2"}}
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if not (have_gpu and llmt_ref.available()):
        # llmt's matmul path is a GPU library call; without its build (or a GPU) the
        # C port on the host cores stands in.
        cb = cpu_baseline(workload)
        v = cb["step_sample"]["tflops"]
        cb["value"], cb["sample"] = v, cb["step_sample"]["sample"]
        base.update({"value": v, "dtype": "f32", "ms_per_step": None, "cpu_baseline": cb,
                     "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0},
                     "note": "llmt build or GPU unavailable: CPU port of the path timed instead"})
        print(json.dumps(base))
        return 0
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    step = ReferenceStep(workload, M_PER_GPU, dev, seed=0)
    for _ in range(max(args.warmup, 3)):
        step.run()
    torch.cuda.synchronize()
    sampler = ClockSampler(0).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step.run()
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # end to end: fp32 host inputs in, gradients out
    h_in = [(torch.empty_like(t[k], device="cpu").pin_memory().copy_(t[k]), t[k])
            for t in step.layers for k in ("x", "dy")]
    h_out = [(torch.empty_like(t["dw"], device="cpu").pin_memory(), t["dw"]) for t in step.layers]
    hp = HostPipeline(torch, h_in, h_out, step.run)   # the same pipeline as the own arm's
    hp.run(1); torch.cuda.synchronize()
    n_e2e = max(2, min(args.steps, 5))
    e0.record()
    hp.run(n_e2e)
    e1.record(); torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    clocks = sampler.stop()
    v = flops / ms / 1e9
    base.update({
        "value": round(v, 2), "ms_per_step": round(ms, 4), "dtype": "f32",
        "device": "gpu (llmt's matmul is cuBLASLt; llmt has no CPU implementation of this path)",
        "cpu_baseline": {"value": round(v, 2), "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                         "sample": "unmodified llmt library (oracle/_ref) on the GPU, full step"},
        "e2e": {"value": round(flops / ms_e2e / 1e9, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": hp.h2d_bytes, "d2h_bytes_per_step": hp.d2h_bytes},
        "clocks": clocks})
    print(json.dumps(base))
    return 0


# ------------------------------------------------------------------------ main ---

def workload_text(workload, m):
    if workload == "c4":
        return ("c4: strided-batched attention products, B*H=96, T=1024, hd=64: S, O, dV, dP, dQ, dK "
                "(dense FLOP count); P and dS from the softmax helpers outside the timed set")
    if workload == "c4f":
        return ("c4f: the same six products with the causal softmax and its backward INSIDE the timed set, fused "
                "around them (P = softmax(aQK^T) in two launches over the score tiles, dS in the dP launch); "
                "FLOP count of the six dense products")
    cfg = LAYERS[workload]
    return (f"{workload}: {cfg['name']}, M={m} tokens per GPU, fwd+dX+dW(+dbias) per layer"
            + (", bias+GELU fused in mlp_fc" if cfg.get("bias", True) else ""))


def roofline_of(step, workload, ms, peaks):
    """Roofline entry of a workload from the CUDA-event time of its timed loop (the loop is the
    GEMM kernel back to back)."""
    if workload in ("c4", "c4f"):
        gbs = step.bytes_step / ms / 1e6
        return {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["bw"], "unit": "GB/s",
                "frac": round(gbs / peaks["bw"], 4), "traffic": recorded_traffic(workload),
                "algorithmic_bytes": int(step.bytes_step), "peak_source": f"of {peaks['which']}",
                "tflops": round(step.flops / ms / 1e9, 1),
                "kernel": ("tc_grouped_pair_kernel (six batched launches; algorithmic bytes = one [96,T,T] "
                           "bf16 matrix + three [96,T,64] tensors per product)") if workload == "c4" else
                          ("tc_grouped_pair_kernel / tc_grouped_pair_lse_kernel (P written once and read three times, "
                           "dS written once and read twice: seven [96,T,T] bf16 matrices per step)")}
    tf = step.flops / ms / 1e9
    return {"bound": "tensor", "achieved": round(tf, 1), "peak": peaks["tf"], "unit": "TFLOP/s",
            "frac": round(tf / peaks["tf"], 4), "traffic": recorded_traffic(workload),
            "peak_source": f"of {peaks['which']}",
            "kernel": "tc_grouped_pair_kernel (all GEMM launches of the step; step FLOP / CUDA-event time "
                      "of the timed loop per step, per GPU)"}


def exchange_check(torch, step, world, rank, dev):
    """The timed step itself, started from random per-rank contents of the span, with and without
    its exchange.  Without: this rank's partial sums (the GEMMs are deterministic), which NCCL's
    all-reduce and a sum in rank order turn into the two references.  With: what the step leaves in
    the span.  Two ranks: bitwise equal to both references.  Peer-copy form: bitwise equal to the
    rank-order sum.  Sum formed inside the switch with more than two ranks: within 1e-6 of NCCL's
    (the order of the additions is the switch's).  In every case a rerun must reproduce its own
    bits and all ranks must hold the same bits."""
    import torch.distributed as dist
    flat = step.bucket.flat
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    start = torch.randn(flat.numel(), device=dev, generator=g)

    def run_from_start(exchange):
        flat.copy_(start)
        torch.cuda.synchronize(); dist.barrier()
        step.run(world, exchange=exchange, zero=False)
        torch.cuda.synchronize(); dist.barrier()
        return flat.clone()

    part = run_from_start(False)
    want_nccl = part.clone()
    dist.all_reduce(want_nccl)
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    want_order = parts[0].clone()
    for p_ in parts[1:]:
        want_order += p_
    del parts
    results = [run_from_start(True) for _ in range(2)]
    # only what the exchange covers (the padding between slices is covered too: it is inside the ranges)
    mask = torch.zeros(flat.numel(), dtype=torch.bool, device=dev)
    for layer in step.layers:
        off, cnt = step.bucket.span_of([layer["name"] + ".dW", layer["name"] + ".dbias"])
        mask[off:off + cnt] = True
    got, again = results[0][mask], results[1][mask]
    eq_nccl = bool(torch.equal(got, want_nccl[mask]))
    eq_order = bool(torch.equal(got, want_order[mask]))
    close_nccl = bool(torch.allclose(got, want_nccl[mask], rtol=1e-6, atol=1e-6))
    in_switch = step.exchange is not None and step.exchange.multicast
    if world == 2:
        ok_value = eq_nccl and eq_order
    elif step.exchange is not None and not in_switch:
        ok_value = eq_order
    else:
        ok_value = close_nccl
    ok_rerun = bool(torch.equal(got, again))
    same = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(same, got.contiguous())
    ok_ranks = all(torch.equal(same[0], t) for t in same)
    flag = torch.tensor([1 if (ok_value and ok_rerun and ok_ranks) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    detail = {"bitwise_equal_to_nccl": eq_nccl, "bitwise_equal_to_rank_order_sum": eq_order,
              "within_1e-6_of_nccl": close_nccl, "rerun_bitwise_equal": ok_rerun,
              "ranks_bitwise_equal": ok_ranks,
              "max_abs_err_vs_nccl": float((got - want_nccl[mask]).abs().max())}
    return ("ok" if int(flag.item()) == 1 else "FAILED"), detail


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=sorted(LAYERS) + ["c4", "c4f"], default="c2")
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="N = 1: skip the other workloads, the per-GEMM comparison and the sustained replay")
    ap.add_argument("--exchange", choices=["ride", "nvls", "peer", "nccl"], default="ride",
                    help="N > 1: how the gradient span is summed: ride = inside the next backward launch, by "
                         "its epilogue warps, through NVSwitch multicast (llmt_b200_gemm_grouped_exchange; the "
                         "last slice by the library's exchange kernel); nvls = that kernel per layer slice on a "
                         "side stream (both fall back to peer copies where no multicast mapping is offered); "
                         "peer = its peer-copy form; nccl = NCCL")
    ap.add_argument("--comm-ctas", type=int, default=None,
                    help="N > 1: CTAs of the exchange kernel (default 64 for nvls, 16 for peer; "
                         "with nccl: NCCL_MAX_CTAS, default unlimited)")
    ap.add_argument("--comm-sms", type=int, default=None,
                    help="N > 1: SMs kept free of GEMM CTAs for the exchange (default 0 for nvls, "
                         "--comm-ctas for peer, 0 for nccl)")
    ap.add_argument("--ride-min-gflop", type=float, default=30.0,
                    help="N > 1, --exchange ride: a backward launch with less work than this carries no slice "
                         "(the exchange would outlast it); its slice waits for the next launch")
    ap.add_argument("--no-defer", action="store_true",
                    help="c2: launch every layer's dW with its own dX (no deferred dW)")
    ap.add_argument("--no-graph", action="store_true",
                    help="enqueue every launch from the host instead of replaying one captured step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import llmt_b200 as L
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    L.lib()  # fail loudly if the CUDA library is missing
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist  # noqa: F401 (also binds torch.distributed)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if args.comm_ctas is None:
            args.comm_ctas = {"ride": 48, "nvls": 64, "peer": 16, "nccl": 0}[args.exchange]
        if args.exchange != "nccl":
            args.comm_ctas = max(1, min(args.comm_ctas, L.COMM_MAX_CTAS))
        elif args.comm_ctas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.comm_ctas))
        if args.comm_sms is None:
            # the multicast kernel's CTAs (no shared memory, 50 registers) fit beside a GEMM CTA
            args.comm_sms = {"ride": 0, "nvls": 0, "peer": args.comm_ctas, "nccl": 0}[args.exchange]
        if args.comm_sms > 0:
            # The GEMM kernels are persistent and fill every SM they are given; the gradient
            # exchange on the side stream only overlaps them if some SMs stay free for it.
            L.set_sm_budget(torch.cuda.get_device_properties(dev).multi_processor_count - args.comm_sms)
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    peaks = measured_peaks()
    attention = args.workload in ("c4", "c4f")
    step = make_step(args.workload, M_PER_GPU, dev, seed=rank, world=world, args=args)
    flops = step.flops
    sampler = make_sampler(torch, dev)
    if rank == 0:
        sampler.start()
    ms, launches, graph = timed_steps(torch, L, step, world, args.steps, args.warmup, not args.no_graph, barrier)
    clocks = sampler.stop() if rank == 0 else None
    L.device_status()

    # The same steps again with an event pair around every launch: per-launch device times
    # (kept out of the loop above, where events between kernels would defeat the overlap of
    # one kernel's prologue with the previous one's tail).
    events = []
    for _ in range(min(args.steps, 20)):
        step.run(world, events)
    barrier()
    per = {}
    for label, a, b in events:
        per.setdefault(label, []).append(a.elapsed_time(b))
    gemm_ms = sum(sum(v) / len(v) for v in per.values())
    gl = {lab: f for lab, f, *_ in step.launches()}
    per_launch = {lab: round(gl[lab] / (sum(v) / len(v)) / 1e9, 1) for lab, v in per.items()}

    # end to end from host buffers
    if attention:
        ms_e2e, h2d, d2h = float("nan"), 0, 0
    else:
        hs = HostStep(step, world)
        hs.run(1); barrier()
        n_e2e = max(2, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        hs.run(n_e2e)
        e1.record(); barrier()
        ms_e2e = e0.elapsed_time(e1) / n_e2e
        h2d, d2h = hs.h2d_bytes, hs.d2h_bytes
        del hs

    extras = {}
    xcheck, xdetail, c5_strong = None, None, None
    if world > 1 and not attention:
        xcheck, xdetail = exchange_check(torch, step, world, rank, dev)
    if world == 1 and not args.no_extras:
        extras["sustained"] = sustained_replay(torch, graph, step, dev, 2.0, flops, peaks)
        L.device_status()

    t = torch.tensor([ms, 0.0 if attention else ms_e2e, gemm_ms], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms, ms_e2e, gemm_ms = (float(x) for x in t.cpu())

    ar_bytes = step.bucket.nbytes() if (world > 1 and not attention) else 0
    exchange_name = (None if world == 1 or attention else "nccl" if step.exchange is None else
                     "llmt_b200_gemm_grouped_exchange (slices ride inside the next backward launch, NVSwitch multicast) + "
                     "llmt_b200_grad_allreduce for the last slice" if getattr(step, "ride", False) else
                     "llmt_b200_grad_allreduce, " + ("NVSwitch multicast" if step.exchange.multicast else "peer copies"))

    # release the headline step before the other workloads are built
    if graph is not None:
        graph.reset()
    graph = None
    main_roof = roofline_of(step, args.workload, ms, peaks)
    main_roof["achieved_per_launch_events"] = round(flops / gemm_ms / 1e9, 1)
    del step
    torch.cuda.empty_cache()

    if world > 1 and args.workload == "c2":
        # config 5 as it is written: M = 65536 tokens split over the N GPUs, gradients exchanged
        try:
            m5 = 65536 // world
            s5 = make_step("c5", m5, dev, seed=100 + rank, world=world, args=args)
            ms5, _, g5 = timed_steps(torch, L, s5, world, 10, 3, not args.no_graph, barrier)
            t5 = torch.tensor([ms5], device=dev, dtype=torch.float64)
            torch.distributed.all_reduce(t5, op=torch.distributed.ReduceOp.MAX)
            ms5 = float(t5.item())
            c5_strong = {"m_per_gpu": m5, "ms_per_step": round(ms5, 4),
                         "per_gpu_tflops": round(s5.flops / ms5 / 1e9, 1),
                         "whole_job_tflops": round(world * s5.flops / ms5 / 1e9, 1),
                         "allreduce_bytes": s5.bucket.nbytes(), "steps": 10}
            if g5 is not None:
                g5.reset()
            del s5, g5
            torch.cuda.empty_cache()
        except Exception as exc:  # never lose the headline line to the extra measurement
            c5_strong = {"error": str(exc)}

    if world == 1 and not args.no_extras:
        others = {}
        for wl in ("c3", "c3c", "c4", "c4f", "c5"):
            if wl == args.workload:
                continue
            try:
                s2 = make_step(wl, M_PER_GPU, dev, seed=7, world=1, args=args)
                smp = make_sampler(torch, dev).start()
                ms2, n2, g2 = timed_steps(torch, L, s2, 1, 20, 3, not args.no_graph, barrier)
                ck = smp.stop()
                L.device_status()
                roof = roofline_of(s2, wl, ms2, peaks)
                others[wl] = {"workload": workload_text(wl, M_PER_GPU), "ms_per_step": round(ms2, 4),
                              "tflops": round(s2.flops / ms2 / 1e9, 1), "steps": 20, "gpu_launches": n2,
                              "roofline": roof, "clocks": ck}
                if g2 is not None:
                    g2.reset()
                del s2, g2
            except Exception as exc:
                others[wl] = {"error": str(exc)}
            torch.cuda.empty_cache()
        extras["workloads"] = others
        if not attention:
            try:
                extras["comparators"] = per_gemm_comparison(torch, L, args.workload, M_PER_GPU, dev)
            except Exception as exc:
                extras["comparators"] = {"error": str(exc)}
            torch.cuda.empty_cache()
            try:
                extras["lm_head_ce"] = lm_head_ce_comparison(torch, L, M_PER_GPU, dev)
            except Exception as exc:
                extras["lm_head_ce"] = {"error": str(exc)}
            torch.cuda.empty_cache()
            try:
                extras["mlp_gelu"] = mlp_gelu_comparison(torch, L, M_PER_GPU, dev)
            except Exception as exc:
                extras["mlp_gelu"] = {"error": str(exc)}
            torch.cuda.empty_cache()
            try:
                extras["attention_softmax"] = attention_softmax_comparison(torch, L, dev)
            except Exception as exc:
                extras["attention_softmax"] = {"error": str(exc)}
            torch.cuda.empty_cache()
        h, mi = L.tensor_map_cache_stats()
        extras["tensor_map_cache"] = {"hits": h, "misses": mi}

    if rank == 0:
        nl = 0 if attention else len(LAYERS[args.workload]["layers"])
        launches_txt = ("6 batched GEMM launches" if attention else
                        f"{nl} forward GEMMs + {nl} grouped backward launches (dX of a layer with dW+dbias of that "
                        "layer or of one whose backward ran earlier) + split-K reductions + 1 zero-fill of the span")
        line = {
            "metric": "GEMM TFLOP/s (fwd+dX+dW), whole job", "value": round(world * flops / ms / 1e9, 2),
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_text(args.workload, M_PER_GPU), "launches_per_step": launches_txt,
                       "per_gpu_gflop_per_step": round(flops / 1e9, 1),
                       "allreduce_bytes_per_step": ar_bytes,
                       "exchange": exchange_name,
                       "comm_ctas": args.comm_ctas if world > 1 else 0,
                       "comm_sms": args.comm_sms if world > 1 else 0,
                       "l2": "working set of a step larger than L2 (operands stream from HBM)"},
            "per_gpu_tflops": round(flops / ms / 1e9, 2),
            "pct_of_bf16_peak": round(100.0 * flops / ms / 1e9 / peaks["tf"], 1),
            "roofline": main_roof,
            "per_launch_tflops": per_launch,
            "e2e": {"value": None if attention else round(world * flops / ms_e2e / 1e9, 2), "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "cuda_graph": not args.no_graph,
            "clocks": clocks,
        }
        if c5_strong is not None:
            line["config"]["c5_strong"] = c5_strong
        if xcheck is not None:
            line["exchange_check"] = xcheck
            line["exchange_check_detail"] = xdetail
        line.update(extras)
        if world == 1 and not args.no_cpu_baseline and not attention:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line))
    rc = 0
    if world > 1:
        if xcheck is not None and xcheck != "ok":
            rc = 3
        # Never let a stuck teardown outlive the measurement.
        sys.stdout.flush()
        guard = threading.Timer(60.0, os._exit, (rc,))
        guard.daemon = True
        guard.start()
        torch.cuda.synchronize()
        torch.distributed.destroy_process_group()
        guard.cancel()
    return rc


if __name__ == "__main__":
    sys.exit(main())
