#!/usr/bin/env python3
"""Benchmark of the GEMM path: one "step" = the linear-layer GEMMs of a training
step (forward, dX, dW+dbias for every layer) on synthetic seeded inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5] [--impl reference]

Workloads (shapes of the reference's benchmark configurations):
  c2  GPT-2-small, M = 8192 tokens per GPU, C = 768: QKV 768->2304, attention
      out-proj 768->768, MLP fc 768->3072 (bias+GELU fused), MLP proj 3072->768;
      bf16 operands, fp32 accumulation, bf16 activations, fp32 dW/dbias.
  c5  GPT-2-XL MLP, C = 1600, 4C = 6400, M = 8192 tokens per GPU.
  c3  LM head 768->50257 (row pitch 50264, fp32 logits); c4 the six attention products.
With N > 1 every GPU runs the same per-GPU workload on its own token shard
(weak scaling) and the fp32 dW/dbias span is summed layer by layer on a side stream
(--exchange: the library's kernel through NVSwitch multicast or peer copies, or NCCL),
overlapped with the backward launches of the remaining layers.

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
    # tied-embedding LM head: fp32 logits, no bias, vocabulary 50257 in a row pitch of 50264
    "c3": dict(name="LM head, vocab 50257 (row pitch 50264), fp32 logits", C=768, bias=False, y_fp32=True,
               ld_out=50264, layers=[("lm_head", 768, 50257, False)]),
}
M_PER_GPU = 8192


def step_flops(workload: str, m: int) -> float:
    return sum(3 * 2.0 * m * i * o for _, i, o, _ in LAYERS[workload]["layers"])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU while the timed region runs:
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
            return
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


# --------------------------------------------------------------------- own arm ---

class LinearStep:
    """Device tensors and prebuilt C-ABI descriptors of one training step's GEMMs."""

    def __init__(self, workload, m, dev, seed, world=1, exchange="peer", comm_ctas=8, split_last=False):
        import torch
        import llmt_b200 as L
        from llmt_b200.dp import GradBucket, PeerExchange
        self.L, self.torch, self.m = L, torch, m
        g = torch.Generator(device=dev).manual_seed(seed)
        bf = torch.bfloat16
        cfg = LAYERS[workload]
        spec = cfg["layers"]
        has_bias = cfg.get("bias", True)
        shapes = {k: v for n, i, o, _ in spec for k, v in ((n + ".dW", (o, i)), (n + ".dbias", (o,)))}
        # N > 1: the span lives in peer-mapped memory and is summed by the library's own kernel
        # over NVLink ("peer"), or stays private and goes through NCCL ("nccl")
        self.exchange = None
        if world > 1 and exchange in ("peer", "nvls"):
            try:
                self.exchange = PeerExchange(GradBucket.layout_numel(shapes), dev, ctas=comm_ctas,
                                             multicast=(exchange == "nvls"))
            except Exception as exc:  # no peer mapping on this machine: every rank falls back to NCCL
                print(f"[bench] peer-mapped span unavailable ({exc}); using NCCL", file=sys.stderr)
            ok = torch.tensor([1 if self.exchange is not None else 0], device=dev)
            torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
            if int(ok.item()) == 0:
                self.exchange = None
            elif exchange == "nvls" and not self.exchange.multicast:
                # no multicast mapping offered: the peer-copy kernel needs SMs of its own
                self.exchange.ctas = 16
                L.set_sm_budget(torch.cuda.get_device_properties(dev).multi_processor_count - 16)
        self.bucket = GradBucket(shapes, dev, storage=self.exchange.attach if self.exchange else None)
        self.layers, self.calls = [], []
        for n, i, o, gelu in spec:
            t = dict(name=n, gelu=gelu, i=i, o=o)
            ld = cfg.get("ld_out", o)  # row pitch of the [m, out] tensors (padded vocabulary)
            t["x"] = torch.randn(m, i, device=dev, generator=g).to(bf)
            t["w"] = (torch.randn(o, i, device=dev, generator=g) * 0.02).to(bf)
            t["b"] = torch.randn(o, device=dev, generator=g) * 0.02 if has_bias else None
            t["dy"] = (torch.randn(m, ld, device=dev, generator=g) * 0.01).to(bf)[:, :o]
            t["y"] = torch.empty(m, ld, device=dev, dtype=torch.float32 if cfg.get("y_fp32") else bf)[:, :o]
            t["dx"] = torch.empty(m, i, device=dev, dtype=bf)
            t["dw"], t["db"] = self.bucket.view(n + ".dW"), self.bucket.view(n + ".dbias")
            self.layers.append(t)
        for t in self.layers:
            t["d_fwd"] = L.make_desc(t["y"], t["x"], t["w"], False, True, bias=t["b"], gelu=t["gelu"])
            # Linear::backward as one launch: dx = dy W and dW += dy^T x (+ dbias) share a tile queue
            dx = L.make_desc(t["dx"], t["dy"], t["w"], False, False)
            dw = L.make_desc(t["dw"], t["dy"], t["x"], True, False, beta=1.0,
                             dbias=t["db"] if has_bias else None, dbias_beta=1.0)
            t["bwd"] = L.Group([(dx, t["dx"], t["dy"], t["w"]), (dw, t["dw"], t["dy"], t["x"])])
            # N > 1: the layer whose backward runs last launches dW on its own, ahead of dX, so that
            # the exchange of its gradients overlaps its dX instead of trailing the step
            if world > 1 and split_last and t is self.layers[0]:
                dx2 = L.make_desc(t["dx"], t["dy"], t["w"], False, False)
                dw2 = L.make_desc(t["dw"], t["dy"], t["x"], True, False, beta=1.0,
                                  dbias=t["db"] if has_bias else None, dbias_beta=1.0)
                t["bwd_dw"] = L.Group([(dw2, t["dw"], t["dy"], t["x"])])
                t["bwd_dx"] = L.Group([(dx2, t["dx"], t["dy"], t["w"])])
        # one scratch buffer per problem that needs one (split-K partial sums)
        self.ws = []
        for t in self.layers:
            need = L.workspace_bytes(t["d_fwd"])
            buf = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
            t["d_fwd"].workspace, t["d_fwd"].workspace_bytes = buf.data_ptr(), buf.numel()
            self.ws.append(buf)
            for key in ("bwd", "bwd_dw", "bwd_dx"):
                if key in t:
                    bufs = [torch.empty(max(b, 256), dtype=torch.uint8, device=dev) for b in t[key].workspace_bytes()]
                    t[key].set_workspaces(bufs)
                    self.ws += bufs
        self.comm_stream = torch.cuda.Stream(device=dev)

    def launches(self):
        """(label, flops, callable) in launch order: forwards, then the backward of every layer."""
        out = []
        for t in self.layers:
            f = 2.0 * self.m * t["i"] * t["o"]
            out.append((t["name"] + ".fwd", f, (lambda t=t: self.L.gemm_desc(t["d_fwd"], t["y"], t["x"], t["w"])), None))
        for t in reversed(self.layers):
            f = 4.0 * self.m * t["i"] * t["o"]
            if "bwd_dw" in t:
                out.append((t["name"] + ".bwd(dW)", f / 2, t["bwd_dw"].run, t))
                out.append((t["name"] + ".bwd(dX)", f / 2, t["bwd_dx"].run, None))
            else:
                out.append((t["name"] + ".bwd(dX+dW)", f, t["bwd"].run, t))
        return out

    def grad_slice(self, t):
        """The layer's dW and dbias are adjacent in the flat span: one view covers both."""
        lo = self.bucket.offsets[t["name"] + ".dW"][0]
        off, n, _ = self.bucket.offsets[t["name"] + ".dbias"]
        return self.bucket.flat[lo:off + n]

    def run(self, world, events=None):
        """Enqueues one step on the current stream. With world > 1 every layer's gradient
        slice is all-reduced on a side stream as soon as that layer's backward is enqueued,
        so the exchange overlaps the backward of the remaining layers."""
        torch = self.torch
        self.bucket.zero_()
        for label, _, fn, layer in self.launches():
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e0.record()
            fn()
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True); e1.record()
                events.append((label, e0, e1))
            if world > 1 and layer is not None:
                ready = torch.cuda.Event(); ready.record()
                self.comm_stream.wait_event(ready)
                if self.exchange is not None:
                    off, cnt = self.bucket.span_of([layer["name"] + ".dW", layer["name"] + ".dbias"])
                    self.exchange.allreduce(off, cnt, stream=self.comm_stream)
                else:
                    with torch.cuda.stream(self.comm_stream):
                        torch.distributed.all_reduce(self.grad_slice(layer))
        if world > 1:
            torch.cuda.current_stream().wait_stream(self.comm_stream)


class AttentionStep:
    """Configuration 4: the six strided-batched attention products at B*H = 96, T = 1024, hd = 64
    (llmt src/kernels/attention.cpp:60-62 forward, docs/TODO.md:226-228 backward), bf16.
    P and dS are produced once by the softmax helpers outside the timed set. HBM-bound:
    every product moves one [96, T, T] matrix."""
    BH, T, HD = 96, 1024, 64

    def __init__(self, dev, seed):
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
        # minimum bytes of one product: the [BH,T,T] matrix once plus three [BH,T,hd] tensors
        self.bytes_each = 2.0 * (BH * T * T + 3 * BH * T * HD)

    def launches(self):
        return [(lab, self.flops_each, (lambda d=d, c=c, a=a, b=b: self.L.gemm_desc(d, c, a, b)), None)
                for lab, d, c, a, b in self.calls]

    def run(self, world=1, events=None):
        torch = self.torch
        for label, _, fn, _l in self.launches():
            if events is not None:
                e0 = torch.cuda.Event(enable_timing=True); e0.record()
            fn()
            if events is not None:
                e1 = torch.cuda.Event(enable_timing=True); e1.record()
                events.append((label, e0, e1))


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


def cpu_baseline(workload, budget_s=12.0):
    """The C port of the path (oracle/oracle.c, fp32 arithmetic, OpenMP) timed on this
    host's cores on a bounded sample: the first 256 token rows of every GEMM of the step."""
    import numpy as np
    from oracle import oracle
    rows = 256
    rng = np.random.default_rng(0)
    spec = LAYERS[workload]["layers"]
    data = []
    for _, i, o, _g in spec:
        data.append((rng.standard_normal((rows, i)).astype(np.float32),
                     (rng.standard_normal((o, i)) * 0.02).astype(np.float32),
                     (rng.standard_normal((rows, o)) * 0.01).astype(np.float32)))
    flops = step_flops(workload, rows)

    def one_pass():
        for x, w, dy in data:
            oracle.gemm_f32(x, w, False, True)          # fwd
            oracle.gemm_f32(dy, w, False, False)        # dX
            oracle.gemm_f32(dy, x, True, False)         # dW
    one_pass()
    best, t_total, n = 1e30, 0.0, 0
    while t_total < budget_s and n < 50:
        t0 = time.perf_counter(); one_pass(); dt = time.perf_counter() - t0
        best = min(best, dt); t_total += dt; n += 1
    out = {"value": round(flops / best / 1e12, 4), "unit": "TFLOP/s", "cores": oracle.num_threads(),
           "kind": "port",
           "sample": f"first {rows} token rows of every GEMM of the step ({flops / 1e9:.1f} GFLOP), "
                     f"best of {n} passes, fp32 OpenMP C port"}
    try:  # PyTorch on CPU is the oracle llmt's own golden files were made with (tools/gen_golden.py)
        import torch
        tx = [(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(dy)) for x, w, dy in data]

        def torch_pass():
            for x, w, dy in tx:
                x @ w.T; dy @ w; dy.T @ x
        torch_pass()
        tb = 1e30
        for _ in range(10):
            t0 = time.perf_counter(); torch_pass(); tb = min(tb, time.perf_counter() - t0)
        out["torch_cpu_tflops"] = round(flops / tb / 1e12, 4)
        out["torch_cpu_threads"] = torch.get_num_threads()
    except Exception:
        pass
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
    flops = step_flops(args.workload, M_PER_GPU)
    base = {"impl": "reference", "metric": "GEMM TFLOP/s (fwd+dX+dW), whole job",
            "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": f"{args.workload}: {LAYERS[args.workload]['name']}, "
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
        cb = cpu_baseline(args.workload)
        base.update({"value": cb["value"], "dtype": "f32", "ms_per_step": None, "cpu_baseline": cb,
                     "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0},
                     "note": "llmt build or GPU unavailable: CPU port of the path timed instead"})
        print(json.dumps(base))
        return 0
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    step = ReferenceStep(args.workload, M_PER_GPU, dev, seed=0)
    for _ in range(max(args.warmup, 3)):
        step.run()
    torch.cuda.synchronize()
    sampler = ClockSampler(0); sampler.start()
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

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=sorted(LAYERS) + ["c4"], default="c2")
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", choices=["nvls", "peer", "nccl"], default="nvls",
                    help="N > 1: how the gradient span is summed: the library's kernel through NVSwitch "
                         "multicast (falls back to peer copies where no multicast mapping is offered), "
                         "its peer-copy kernel, or NCCL")
    ap.add_argument("--comm-ctas", type=int, default=None,
                    help="N > 1: CTAs of the exchange kernel (default 64 for nvls, 16 for peer; "
                         "with nccl: NCCL_MAX_CTAS, default unlimited)")
    ap.add_argument("--comm-sms", type=int, default=None,
                    help="N > 1: SMs kept free of GEMM CTAs for the exchange (default 0 for nvls, "
                         "--comm-ctas for peer, 0 for nccl)")
    ap.add_argument("--split-last", action="store_true",
                    help="N > 1: launch dW of the last backward on its own, ahead of dX")
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
            args.comm_ctas = {"nvls": 64, "peer": 16, "nccl": 0}[args.exchange]
        if args.exchange != "nccl":
            args.comm_ctas = max(1, min(args.comm_ctas, L.COMM_MAX_CTAS))
        elif args.comm_ctas > 0:
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.comm_ctas))
        if args.comm_sms is None:
            # the multicast kernel's CTAs (no shared memory, 50 registers) fit beside a GEMM CTA
            args.comm_sms = {"nvls": 0, "peer": args.comm_ctas, "nccl": 0}[args.exchange]
        if args.comm_sms > 0:
            # The GEMM kernels are persistent and fill every SM they are given; the gradient
            # exchange on the side stream only overlaps them if some SMs stay free for it.
            L.set_sm_budget(torch.cuda.get_device_properties(dev).multi_processor_count - args.comm_sms)
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    attention = args.workload == "c4"
    step = AttentionStep(dev, seed=rank) if attention else LinearStep(args.workload, M_PER_GPU, dev, seed=rank, world=world, exchange=args.exchange, comm_ctas=args.comm_ctas or 8, split_last=args.split_last)
    flops = 6 * step.flops_each if attention else step_flops(args.workload, M_PER_GPU)
    for _ in range(args.warmup):
        step.run(world)
    barrier()
    # One step (its GEMM launches and, for N > 1, the gradient all-reduces on the side stream)
    # captured into a CUDA graph: the timed loop replays it, so the host enqueues one graph
    # per step instead of a dozen launches.
    graph, per_step_launches = None, None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            n0 = L.launch_count()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                step.run(world)
            per_step_launches = L.launch_count() - n0
            for _ in range(args.warmup):
                graph.replay()
        except Exception as exc:  # capture refused: fall back to direct launches and say so
            print(f"[bench] graph capture failed ({exc}); launching directly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    barrier()
    props = torch.cuda.get_device_properties(dev)
    try:
        pci = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except AttributeError:
        pci = None
    sampler = ClockSampler(local, pci)
    if rank == 0:
        sampler.start()
    launches0 = L.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step.run(world)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = per_step_launches * args.steps if graph is not None else L.launch_count() - launches0
    # The same K steps again with an event pair around every launch: the per-launch device
    # times behind roofline.achieved (kept out of the loop above, where events between
    # kernels would defeat the overlap of one kernel's prologue with the previous one's tail).
    events = []
    for _ in range(args.steps):
        step.run(world, events)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    L.device_status()

    # per-launch device time
    per = {}
    for label, a, b in events:
        per.setdefault(label, []).append(a.elapsed_time(b))
    gemm_ms = sum(sum(v) / len(v) for v in per.values())
    gl = {lab: f for lab, f, *_ in step.launches()}
    per_gemm = {lab: round(gl[lab] / (sum(v) / len(v)) / 1e9, 1) for lab, v in per.items()}

    # end to end from host buffers
    if attention:
        ms_e2e, h2d, d2h = float("nan"), 0, 0
    else:
        hs = HostStep(step, world)
        hs.run(1); barrier()
        n_e2e = max(2, min(args.steps, 10))
        e0.record()
        hs.run(n_e2e)
        e1.record(); barrier()
        ms_e2e = e0.elapsed_time(e1) / n_e2e
        h2d, d2h = hs.h2d_bytes, hs.d2h_bytes

    t = torch.tensor([ms, 0.0 if attention else ms_e2e, gemm_ms], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms, ms_e2e, gemm_ms = (float(x) for x in t.cpu())
    if rank == 0:
        peak_tf, peak_bw, which = measured_peaks()
        achieved = flops / gemm_ms / 1e9
        if attention:
            wl = ("c4: strided-batched attention products, B*H=96, T=1024, hd=64: S, O, dV, dP, dQ, dK "
                  "(dense FLOP count); P and dS from the softmax helpers outside the timed set")
            launches_txt = "6 batched GEMM launches"
            gbs = 6 * step.bytes_each / gemm_ms / 1e6
            roof = {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak_bw, "unit": "GB/s",
                    "frac": round(gbs / peak_bw, 4), "traffic": None, "peak_source": f"of {which}",
                    "kernel": "tc_grouped_kernel (six batched launches; algorithmic bytes = one [96,T,T] "
                              "bf16 matrix + three [96,T,64] tensors per product)"}
            ar_bytes = 0
        else:
            cfg = LAYERS[args.workload]
            wl = (f"{args.workload}: {cfg['name']}, M={M_PER_GPU} tokens per GPU, fwd+dX+dW(+dbias) per layer"
                  + (", bias+GELU fused in mlp_fc" if cfg.get("bias", True) else ""))
            nl = len(cfg["layers"])
            launches_txt = (f"{nl} forward GEMMs + {nl} grouped backward launches (dX and dW+dbias of a layer "
                            "in one kernel) + split-K reductions")
            # DRAM bytes of one step's launches (dram__bytes_read.sum + dram__bytes_write.sum over the
            # 8 GEMM launches + 1 split-K reduction, one ncu capture of this workload at the default
            # settings; writes of a replayed launch partly stay in L2): 380.1 MB + 25.4 MB against
            # 343.6 MB of algorithmic operand reads.
            traffic = 405.5e6 if args.workload == "c2" and world == 1 else None
            # The timed loop is the GEMM kernel back to back (98.6 % of its kernel time, see profiles/):
            # its CUDA-event duration is the kernel's duration.  The per-launch sum of the second,
            # instrumented pass is reported beside it; it is longer because an event between two
            # launches keeps one launch's prologue from overlapping the previous launch's tail.
            in_loop = flops / ms / 1e9
            roof = {"bound": "tensor", "achieved": round(in_loop, 1), "peak": peak_tf,
                    "unit": "TFLOP/s", "frac": round(in_loop / peak_tf, 4), "traffic": traffic,
                    "peak_source": f"of {which}",
                    "achieved_per_launch_events": round(achieved, 1),
                    "kernel": "tc_grouped_kernel (all GEMM launches of the step; step FLOP / CUDA-event time "
                              "of the timed loop per step, per GPU)"}
            ar_bytes = step.bucket.nbytes() if world > 1 else 0
        line = {
            "metric": "GEMM TFLOP/s (fwd+dX+dW), whole job", "value": round(world * flops / ms / 1e9, 2),
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl, "launches_per_step": launches_txt,
                       "per_gpu_gflop_per_step": round(flops / 1e9, 1),
                       "allreduce_bytes_per_step": ar_bytes,
                       "exchange": (None if world == 1 else "nccl" if step.exchange is None else
                                    "llmt_b200_grad_allreduce, " + ("NVSwitch multicast" if step.exchange.multicast
                                                                    else "peer copies")),
                       "comm_ctas": args.comm_ctas if world > 1 else 0,
                       "comm_sms": args.comm_sms if world > 1 else 0,
                       "l2": "working set of a step larger than L2 (operands stream from HBM)"},
            "per_gpu_tflops": round(flops / ms / 1e9, 2),
            "pct_of_bf16_peak": round(100.0 * flops / ms / 1e9 / peak_tf, 1),
            "roofline": roof,
            "per_gemm_tflops": per_gemm,
            "e2e": {"value": None if attention else round(world * flops / ms_e2e / 1e9, 2), "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "cuda_graph": graph is not None,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline and not attention:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line))
    if world > 1:
        # The captured step holds NCCL work: release it before the communicator goes, and
        # never let a stuck teardown outlive the measurement.
        import threading
        sys.stdout.flush()
        guard = threading.Timer(60.0, os._exit, (0,))
        guard.daemon = True
        guard.start()
        if graph is not None:
            graph.reset()
            del graph
        torch.cuda.synchronize()
        torch.distributed.destroy_process_group()
        guard.cancel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
