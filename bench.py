"""Benchmark of the Selective Attention operator on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|decode|c5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward + backward of the operator over one batch of synthetic input (workload c2:
B=4, H=16, T=16384, D=64, bf16 q/k/v/dO ~ N(0,1), causal, <BOS> exempt, head 0 selects for all heads).

With N > 1 the SAME batch is sharded over the ranks (strong scaling): whole sequences per rank while N <= B,
and beyond that the heads of a sequence are split between N / B ranks, each of which holds a replica of the
selection head's q, k rows (``selector=``) and returns partial gradients for them; those partial gradients are
summed with one NCCL all-reduce per group of ranks sharing a sequence, inside the timed region and also
reported on its own.  No other data crosses GPUs.  ``--replicas`` instead gives every rank its own full batch
(weak scaling).  The reported value is the tokens of the whole job over the slowest rank's device time.

One JSON line is printed by rank 0:
  value        tokens/s with inputs resident in HBM (device time of the forward and backward calls)
  e2e          the same through the public Python API with host buffers: pinned host -> device copies of
               q, k, v, dO and device -> host copies of out and the gradients inside the timed region
  roofline     the backward kernel (the dominant launch): algorithmic FLOPs over its device time, measured
               with CUDA events around that launch, against the measured bf16 tensor peak
  cpu_baseline the reference's CPU listing timed on this host on a bounded sample (rank 0, N = 1 only)
--impl reference times the reference's own CPU implementation of the operator (its dense listing with
autograd, from the installed copy under baseline/_ref; the CPU oracle port when that copy is absent) on a
bounded sample of the same workload with all host threads, and, where the reference's Triton kernels run on
this GPU, also reports them at the full configuration under "reference_gpu".
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for sub in ("selective-attention-study_b200", "oracle"):
    sys.path.insert(0, os.path.join(ROOT, sub))

import torch

WORKLOADS = {
    # name: (batch, heads, seq, dim, per_head selection, backward?)
    "c2": dict(batch=4, heads=16, seq=16384, dim=64, per_head=False, backward=True),
    "c3": dict(batch=4, heads=16, seq=16384, dim=64, per_head=True, backward=True),
    # the counted FLOPs of c2 at head_dim 128 (eight heads)
    "c2d128": dict(batch=4, heads=8, seq=16384, dim=128, per_head=False, backward=True),
    "c4": dict(batch=1, heads=16, seq=131072, dim=64, per_head=False, backward=False),
    # one cached decode step against a 131,071-token cache (the serving continuation of c4)
    "decode": dict(batch=1, heads=16, seq=131072, dim=64, per_head=False, backward=False),
    # full decoder training step, data parallel (one sequence per GPU)
    "c5": dict(batch=1, heads=16, seq=16384, dim=64, per_head=False, backward=True, layers=24),
}
METRIC = "selective-attn fwd+bwd tokens/s/GPU @T=16K bf16; % of tcgen05 bf16 peak"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0      # B200 cuBLAS bf16 burst; used only when MEASURED_PEAKS.json is absent


def captured_traffic_per_head_tile(kernel: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of `kernel` divided by the head-tiles of the
    captured (smaller) case, from the record kept beside the ncu summaries; None when no capture is recorded."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as fh:
            rec = json.load(fh)[kernel]
        return float(rec["dram_bytes_per_launch"]) / float(rec["head_tiles"])
    except (OSError, KeyError, ValueError):
        return None


def pairs(seq: int) -> float:
    return seq * (seq + 1) / 2.0


def algorithmic_flops(w: dict) -> dict:
    """Counted once per selector, whatever a kernel recomputes.  P = causal pairs, N = batch * heads,
    Nsel = selectors.  Forward: attention 4 D P N, selection logits 2 D P Nsel, the column-sum pass
    2 D P Nsel, the triangular running-sum MMA 2 * 128 P Nsel.  Backward: attention 10 D P N, selection
    logits again 2 D P Nsel, head-0 gradient products 4 D P Nsel; its running sums are register
    recurrences, not MMAs, so no triangular term.  The per-head variant's selection logit is the head's
    own logit (no extra product)."""
    n = w["batch"] * w["heads"]
    nsel = n if w["per_head"] else w["batch"]
    p, d = pairs(w["seq"]), w["dim"]
    sel_logits = 0.0 if w["per_head"] else 2 * d * p * nsel
    fwd = 4 * d * p * n + sel_logits + 2 * d * p * nsel + 2 * 128 * p * nsel
    bwd = (10 * d * p * n + sel_logits + 4 * d * p * nsel) if w["backward"] else 0.0
    return dict(forward=fwd, backward=bwd, attention_only=(14 if w["backward"] else 4) * d * p * n)


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            data = json.load(fh)
        return float(data["bf16_tflops_sustained"]), "measured (cuBLAS bf16, sustained)"
    return FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs.  Read-only NVML queries from a thread
    (a sample every few milliseconds, so even a short timed region of one rank among eight is covered); the
    nvidia-smi polling route is the fall-back when NVML cannot be loaded."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40), ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None
        self.stop = threading.Event()
        self.nvml = None
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                props = torch.cuda.get_device_properties(index)
                bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
                self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _sample_nvml(self):
        n = self.nvml
        sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        try:
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        flags = {name: ("Active" if bits & bit else "Not Active") for name, bit in self.REASON_BITS}
        self.rows.append([str(sm), str(mx), flags["hw_slowdown"], flags["hw_thermal_slowdown"],
                          flags["sw_thermal_slowdown"], flags["sw_power_cap"]])

    def _poll_nvml(self):
        while not self.stop.is_set():
            try:
                self._sample_nvml()
            except Exception:
                return
            self.stop.wait(0.005)

    def _read_smi(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __enter__(self):
        if self.nvml is not None:
            try:
                self._sample_nvml()                            # one sample at the start of the region, always
            except Exception:
                self.nvml = None
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.nvml is not None:
            try:
                self._sample_nvml()                            # and one at its end (the work is still draining)
            except Exception:
                pass
            self.stop.set()
            if self.thread is not None:
                self.thread.join(timeout=2)
        elif self.proc is not None:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        clocks = sorted(int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit())
        reasons = set()
        for r in self.rows:
            if len(r) >= 6:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        mx = max((int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()), default=None)
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


def max_over_ranks(value_ms: float, world: int, device) -> float:
    """Slowest rank's time: the denominator of the whole-job throughput (device time, not wall clock)."""
    if world == 1:
        return float(value_ms)
    t = torch.tensor([float(value_ms)], dtype=torch.float64, device=device)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def whole_job_tokens_per_second(tokens_per_step: int, ms_per_step: float) -> float:
    """Tokens the whole job (all ranks together) processes per step over the slowest rank's device time."""
    return tokens_per_step / (ms_per_step * 1e-3)


def shard_plan(w: dict, rank: int, world: int, replicas: bool) -> dict:
    """Which part of the workload's batch this rank runs.

    replicas: every rank runs the whole batch (weak scaling, `tokens` grows with the ranks).
    otherwise (strong scaling, `tokens` is the workload's): whole sequences per rank while world <= batch;
    beyond that `world / batch` ranks share a sequence and split its heads evenly, each holding a replica of the
    selection head's rows.  The per-head variant has no shared selector: its (batch x heads) rows split evenly."""
    b, h = w["batch"], w["heads"]
    if replicas or world == 1:
        return dict(seqs=range(b), heads=range(h), selector=False, group=[rank], tokens=b * w["seq"] * world,
                    scaling="weak" if world > 1 else "strong", parallelism=f"{world} independent replicas" if world > 1 else "1 GPU")
    if w["per_head"]:
        rows = b * h
        if rows % world:
            raise ValueError(f"{rows} (batch x heads) rows do not split over {world} ranks")
        per = rows // world
        if per >= h:                      # whole sequences
            n = per // h
            return dict(seqs=range(rank * n, (rank + 1) * n), heads=range(h), selector=False, group=[rank],
                        tokens=b * w["seq"], scaling="strong", parallelism=f"batch split {world} ways")
        first = rank * per
        return dict(seqs=range(first // h, first // h + 1), heads=range(first % h, first % h + per), selector=False,
                    group=[rank], tokens=b * w["seq"], scaling="strong", parallelism=f"(batch x heads) rows split {world} ways")
    if world <= b:
        if b % world:
            raise ValueError(f"batch {b} does not split over {world} ranks")
        n = b // world
        return dict(seqs=range(rank * n, (rank + 1) * n), heads=range(h), selector=False, group=[rank],
                    tokens=b * w["seq"], scaling="strong", parallelism=f"batch split {world} ways")
    if world % b or h % (world // b):
        raise ValueError(f"{world} ranks do not split batch {b} x heads {h}")
    share = world // b                    # ranks per sequence
    per = h // share
    seq_index, part = rank // share, rank % share
    return dict(seqs=range(seq_index, seq_index + 1), heads=range(part * per, (part + 1) * per), selector=True,
                group=list(range(seq_index * share, (seq_index + 1) * share)), tokens=b * w["seq"], scaling="strong",
                parallelism=f"batch split {b} ways x heads split {share} ways (selector replicated, its gradient all-reduced)")


def bind_near_gpu(device_index: int) -> str:
    """Restricts this process to the CPU cores of its GPU's NUMA node, before any pinned buffer is allocated, so
    the host side of every copy stays on that node.  (The whole node, not a slice of it: on a shared host a
    fixed slice can coincide with cores another job keeps busy, which starves a rank's launch thread.)"""
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/local_cpulist") as fh:
            text = fh.read().strip()
        cores = []
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cores.extend(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cores) & set(os.sched_getaffinity(0)))
        if not allowed:
            return "unbound (no local core is allowed)"
        os.sched_setaffinity(0, allowed)
        return f"{len(allowed)} cores of the GPU's local list {text}"
    except (OSError, ValueError, AttributeError) as exc:
        return f"unbound ({type(exc).__name__})"


def make_inputs(w: dict, seed: int):
    """q, k, v, dO ~ N(0, 1) drawn in fp32 in that order from a CPU generator, rounded to bf16 once."""
    g = torch.Generator("cpu").manual_seed(seed)
    shape = (w["batch"], w["heads"], w["seq"], w["dim"])
    return tuple(torch.randn(shape, generator=g).bfloat16() for _ in range(4))


def run_ours(args, w, rank, world, device):
    from selective_attention_b200 import _lib, kernels

    if not kernels.HAS_KERNELS:
        raise RuntimeError("the CUDA library is missing; build it first (python __graft_entry__.py)")
    plan = shard_plan(w, rank, world, args.replicas)
    affinity = bind_near_gpu(device.index)
    # The full synthetic batch is generated from one seed and every rank slices its shard (replicas: own seed).
    full = make_inputs(w, seed=rank if plan["scaling"] == "weak" and world > 1 else 0)
    sl = (slice(plan["seqs"].start, plan["seqs"].stop), slice(plan["heads"].start, plan["heads"].stop))
    q_h, k_h, v_h, do_h = (t[sl[0], sl[1]].contiguous() for t in full)
    sel_h = tuple(t[sl[0], 0].contiguous() for t in full[:2]) if plan["selector"] else ()
    del full
    if w["per_head"]:                    # every head is its own one-head sequence
        q_h, k_h, v_h, do_h = (t.reshape(-1, 1, t.shape[2], t.shape[3]) for t in (q_h, k_h, v_h, do_h))
    tokens = plan["tokens"]
    flops = algorithmic_flops(w)
    group = None
    if plan["selector"]:
        for first in range(0, world, len(plan["group"])):          # every rank creates every group, in the same order
            ranks = list(range(first, first + len(plan["group"])))
            g = torch.distributed.new_group(ranks)
            if ranks == plan["group"]:
                group = g

    skip = bool(args.skip_dead_tiles)

    def operator(q, k, v, sel):
        return kernels.selective_attention(q, k, v, selector=sel or None, skip_dead_tiles=skip)

    def reduce_selector_grads(sel, record=None):
        """The ranks that share a sequence sum their partial gradients of the replicated selector rows."""
        flat = torch.cat([sel[0].grad.float().reshape(-1), sel[1].grad.float().reshape(-1)])
        if record is not None:
            record[0].record()
        torch.distributed.all_reduce(flat, group=group)
        if record is not None:
            record[1].record()
        return flat

    # ---- device-resident arm --------------------------------------------------------------------------
    q, k, v = (t.to(device).requires_grad_(w["backward"]) for t in (q_h, k_h, v_h))
    sel = tuple(t.to(device).requires_grad_(w["backward"]) for t in sel_h)
    d_out = do_h.to(device).float()            # the operator returns fp32, so its cotangent is fp32

    def step(record=None):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        if w["backward"]:
            out = operator(q, k, v, sel)
            ev[1].record()
            out.backward(d_out)
            ev[2].record()
            if sel:
                reduce_selector_grads(sel, (ev[2], ev[3]))
                sel[0].grad = sel[1].grad = None
            else:
                ev[3].record()
            q.grad = k.grad = v.grad = None
        else:
            with torch.no_grad():
                kernels.selective_attention_forward(q, k, v, return_aux=True, selector=sel or None, skip_dead_tiles=skip)
            ev[1].record(); ev[2].record(); ev[3].record()
        ev[4].record()
        if record is not None:
            record.append(ev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    if not w["backward"] and world > 1 and sel:                    # every shard must see the same per-key totals
        with torch.no_grad():
            _, aux = kernels.selective_attention_forward(q, k, v, return_aux=True, selector=sel)
        mine = aux["selected_total"].clone()
        theirs = mine.clone()
        torch.distributed.broadcast(theirs, src=plan["group"][0], group=group)
        if not torch.equal(mine, theirs):
            raise RuntimeError("selected_total differs between the ranks that share a sequence")
    for _ in range(args.warmup):
        step()
    dominant = "tc_backward" if w["backward"] else "tc_forward"
    _lib.profile_enable(dominant)
    events = []
    barrier()
    launches_before = _lib.launch_count()
    with ClockSampler(device.index) as sampler:
        for _ in range(args.steps):
            step(events)
        barrier()
    launches = _lib.launch_count() - launches_before
    kernel_ms = _lib.profile_collect()
    _lib.profile_enable("none")
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in events)
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in events)
    reduce_ms = sum(e[2].elapsed_time(e[3]) for e in events)
    own_ms = sum(e[0].elapsed_time(e[4]) for e in events)
    total_ms = max_over_ranks(own_ms, world, device)
    per_rank = None
    if world > 1:                        # every rank's own split of a step, for the record
        mine = torch.tensor([fwd_ms, bwd_ms, reduce_ms, own_ms], dtype=torch.float64, device=device) / args.steps
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        torch.distributed.all_gather(gathered, mine)
        per_rank = [[round(float(x), 3) for x in g] for g in gathered]
    status = _lib.device_status()
    if status:
        raise RuntimeError(f"a bounded device-side wait ran out (status {status:#x}); the timing is invalid")

    # ---- end-to-end arm: host buffers in, host buffers out ------------------------------------------------
    # Whole sequences with a shared selector go through the layer-facing call: one packed (B, T, 3, H, D) projection
    # output and one (B, T, H D) cotangent in, the merged output and the packed gradient out (the same bytes).
    packed = (w["backward"] and not w["per_head"] and not sel_h and w["dim"] in (64, 128) and args.e2e_call == "packed"
              and not skip)
    if packed:
        q_h, k_h, v_h, do_h = (t.transpose(1, 2) for t in (q_h, k_h, v_h, do_h))       # (B, T, H, D)
        qkv_h = torch.stack([q_h, k_h, v_h], dim=2).contiguous()                       # (B, T, 3, H, D)
        do_h = do_h.reshape(do_h.shape[0], do_h.shape[1], -1).contiguous()              # (B, T, H D)
        host_in = [qkv_h, do_h]
    else:
        host_in = [q_h, k_h, v_h] + ([do_h] if w["backward"] else []) + list(sel_h)
    pinned_in = [t.pin_memory() for t in host_in]
    n_main = 4 if w["backward"] else 3
    if packed:
        out_shapes = [do_h.shape, qkv_h.shape]
    else:
        out_shapes = [q_h.shape] * (4 if w["backward"] else 1) + ([sel_h[0].shape] * 2 if sel_h and w["backward"] else [])
    pinned_out = [torch.empty(shape, dtype=torch.bfloat16).pin_memory() for shape in out_shapes]
    h2d = sum(t.numel() * t.element_size() for t in pinned_in)
    d2h = sum(t.numel() * t.element_size() for t in pinned_out)

    # Every step copies its own inputs in and its own results out.  The copies run on their own streams and a step is
    # fed sequence by sequence: sequence k + 1 of a step (and then the next step's first) is uploaded while sequence k
    # is computed, and sequence k's results are downloaded under the next computation, as a training or serving loop
    # that feeds the operator from host memory would arrange it.  Only the first upload and the last download of the
    # timed region are not hidden.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    s_comp = torch.cuda.current_stream(device)
    dev_in = [[torch.empty_like(t, device=device) for t in pinned_in] for _ in range(2)]
    n_chunks = len(plan["seqs"])                               # this rank's sequences; every tensor has their rows on axis 0
    rows_per_chunk = pinned_in[0].shape[0] // n_chunks         #   (per-head form: the heads of a sequence are its rows)
    uploaded = [[torch.cuda.Event() for _ in range(n_chunks)] for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    downloaded = torch.cuda.Event()

    def e2e_compute(chunk):
        """One sequence (all of this rank's heads) through the public call; returns what goes back to the host."""
        if packed:
            xd = chunk[0].detach().requires_grad_(True)
            y = kernels.selective_attention_packed(xd)
            y.backward(chunk[1])
            return [y.detach(), xd.grad]
        qd, kd, vd = (t.detach() for t in chunk[:3])
        sd = tuple(t.detach() for t in chunk[n_main:])
        if w["backward"]:
            dd = chunk[3].float()
            for t in (qd, kd, vd) + sd:
                t.requires_grad_(True)
            out = operator(qd, kd, vd, sd)
            out.backward(dd)
            results = [out.detach().to(torch.bfloat16), qd.grad, kd.grad, vd.grad]
            if sd:
                flat = reduce_selector_grads(sd)
                half = flat.numel() // 2
                results += [flat[:half].to(torch.bfloat16).view(sd[0].shape), flat[half:].to(torch.bfloat16).view(sd[1].shape)]
            return results
        with torch.no_grad():
            return [kernels.selective_attention_forward(qd, kd, vd, selector=sd or None,
                                                        skip_dead_tiles=skip).to(torch.bfloat16)]

    def e2e_step(i: int):
        slot = i & 1
        for c in range(n_chunks):
            lo, hi = c * rows_per_chunk, (c + 1) * rows_per_chunk
            with torch.cuda.stream(s_in):
                if i >= 2 and c == 0:
                    s_in.wait_event(consumed[slot])        # the compute of step i - 2 has read this slot
                for dst, src in zip(dev_in[slot], pinned_in):
                    dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                uploaded[slot][c].record(s_in)
            s_comp.wait_event(uploaded[slot][c])
            results = e2e_compute([t[lo:hi] for t in dev_in[slot]])
            if c == n_chunks - 1:
                consumed[slot].record(s_comp)
            done = torch.cuda.Event()
            done.record(s_comp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(pinned_out, results):
                    src.record_stream(s_out)
                    dst[lo:hi].copy_(src, non_blocking=True)
                downloaded.record(s_out)

    for i in range(2):
        e2e_step(i)
    barrier()
    s0 = torch.cuda.Event(enable_timing=True); s1 = torch.cuda.Event(enable_timing=True)
    s0.record(s_in)
    for i in range(args.steps):
        e2e_step(i)
    s_comp.wait_event(downloaded)
    s1.record(s_comp)
    barrier()
    e2e_ms = max_over_ranks(s0.elapsed_time(s1) / args.steps, world, device)

    # the copies alone (no compute between them): the host-side ceiling of this rank's end-to-end step
    def copies_only():
        with torch.cuda.stream(s_in):
            for dst, src in zip(dev_in[0], pinned_in):
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(s_out):
            for dst in pinned_out:
                dst.copy_(dev_in[1][0].view(-1)[:dst.numel()].view(dst.shape), non_blocking=True)
    copies_only()
    barrier()
    c0 = torch.cuda.Event(enable_timing=True); c1 = torch.cuda.Event(enable_timing=True); c2 = torch.cuda.Event(enable_timing=True); c3 = torch.cuda.Event(enable_timing=True)
    c0.record(s_in); c2.record(s_out)
    for _ in range(3):
        copies_only()
    c1.record(s_in); c3.record(s_out)
    barrier()
    h2d_gbs = 3 * h2d / (c0.elapsed_time(c1) * 1e-3) / 1e9
    d2h_gbs = 3 * d2h / (c2.elapsed_time(c3) * 1e-3) / 1e9

    ms_per_step = total_ms / args.steps
    value = whole_job_tokens_per_second(tokens, ms_per_step)
    peak, peak_kind = measured_peaks()
    share = (len(plan["seqs"]) * len(plan["heads"])) / (w["batch"] * w["heads"])      # this rank's part of the batch
    live_fraction = None
    if skip:                                 # the share of the causal tiles that was computed (this rank's shard)
        with torch.no_grad():
            _, aux = kernels.selective_attention_forward(q, k, v, return_aux=True, selector=sel or None, skip_dead_tiles=True)
        live = aux.get("live_tiles")
        if live is not None:
            lower = torch.tril(torch.ones(live.shape[-1], live.shape[-1], dtype=torch.bool, device=live.device))
            live_fraction = float((live[:, lower] != 0).float().mean())
    kflops = (flops["backward"] if w["backward"] else flops["forward"]) * share * (live_fraction if live_fraction else 1.0)
    kernel_avg_ms = sum(kernel_ms) / max(len(kernel_ms), 1)
    achieved = kflops / (kernel_avg_ms * 1e-3) / 1e12 if kernel_ms else None
    ntile = math.ceil(w["seq"] / 128)
    head_tiles = len(plan["seqs"]) * len(plan["heads"]) * (ntile * (ntile + 1) // 2)
    per_tile = captured_traffic_per_head_tile(dominant if w["dim"] == 64 else f"{dominant}_d{w['dim']}")
    step_flops = (flops["forward"] + flops["backward"]) * (world if plan["scaling"] == "weak" else 1)
    dense_step_flops = step_flops
    if live_fraction:                        # rates below count the live tiles only
        step_flops *= live_fraction
        per_tile = None
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": plan["scaling"],
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: selective attention fwd{'+bwd' if w['backward'] else ''} B={w['batch']} "
                               f"H={w['heads']} T={w['seq']} D={w['dim']} bf16, "
                               f"{'per-head' if w['per_head'] else 'shared head-0'} selection, "
                               f"{'whole batch per GPU' if plan['scaling'] == 'weak' else 'one batch over all GPUs'}",
                   "parallelism": plan["parallelism"],
                   "rank0_shard": f"sequences {plan['seqs'].start}..{plan['seqs'].stop - 1}, heads {plan['heads'].start}..{plan['heads'].stop - 1}",
                   "tiles": ("every causal tile is computed" if not skip else
                             "NOT the dense workload: (query tile, key tile) pairs whose probabilities are all exactly zero "
                             f"are left out (results identical); live fraction {live_fraction}; the roofline's FLOPs are "
                             "the algorithmic count times that fraction"),
                   "l2": "inputs (q, k, v, dO) of every rank exceed the 126 MB L2; no explicit flush",
                   "engine": "tcgen05", "fwd_ms": fwd_ms / args.steps, "bwd_ms": bwd_ms / args.steps,
                   "selector_grad_allreduce_ms": reduce_ms / args.steps if (sel and w["backward"]) else None,
                   "selector_grad_allreduce_bytes": (2 * sel[0].numel() * 4) if (sel and w["backward"]) else 0,
                   "algorithmic_tflop_per_step": step_flops / 1e12,
                   "dense_workload_tflop_per_step": dense_step_flops / 1e12,
                   "attention_only_tflop_per_step": flops["attention_only"] * (world if plan["scaling"] == "weak" else 1) / 1e12,
                   "step_tflops_per_gpu": step_flops / world / (ms_per_step * 1e-3) / 1e12,
                   "frac_of_nominal_2250_per_gpu": step_flops / world / (ms_per_step * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS,
                   "per_rank_ms_fwd_bwd_allreduce_step": per_rank, "host_affinity": affinity},
        "e2e": {"value": whole_job_tokens_per_second(tokens, e2e_ms), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": args.steps,
                "copies_alone_gbs": {"h2d": h2d_gbs, "d2h": d2h_gbs}, "bytes_are": "per rank",
                "pipelining": f"{n_chunks} sequence(s) per step, one call each; uploads, computation and downloads on three streams",
                "call": "selective_attention_packed (fused QKV layout in, merged output and packed gradient out)" if packed
                        else "selective_attention / selective_attention_forward on (B, H, T, D) tensors"},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": (achieved / peak) if achieved else None, "peak_kind": peak_kind,
                     "launch_ms": kernel_avg_ms, "launches_timed": len(kernel_ms),
                     "traffic": (per_tile * head_tiles) if per_tile else None},
        "clocks": sampler.summary(),
    }
    return line


def run_decode(args, w, rank, world, device):
    """One cached decode step per 'step': K and V of the cache are streamed once (HBM-bound)."""
    from selective_attention_b200 import _lib, kernels

    b, h, t, d = w["batch"], w["heads"], w["seq"] - 1, w["dim"]
    g = torch.Generator("cpu").manual_seed(rank)
    cache = {"k": torch.randn(b, h, t + 1, d, generator=g).bfloat16().to(device),
             "v": torch.randn(b, h, t + 1, d, generator=g).bfloat16().to(device), "len": t,
             "selected": (3 * torch.rand(b, 1, t + 1, generator=g)).to(device)}
    live = bool(args.skip_dead_tiles)
    if live:
        # NOT the dense workload: the history vector of a real prefill of the N(0,1) prompt (strong selection), and
        # the key norms with which the step leaves out the part of the cache that no longer carries weight
        qp = torch.randn(b, h, t, d, generator=g).bfloat16().to(device)
        with torch.no_grad():
            _, aux = kernels.selective_attention_forward(qp, cache["k"][:, :, :t], cache["v"][:, :, :t], return_aux=True,
                                                         skip_dead_tiles=True)
        cache["selected"][:, 0, :t] = aux["selected_total"]
        cache["selected"][:, 0, t:] = 0
        cache["key_norms"] = kernels.key_norms(cache["k"]).contiguous()
        del qp, aux
    q1, k1, v1 = (torch.randn(b, h, 1, d, generator=g).bfloat16() for _ in range(3))
    qd, kd, vd = (x.to(device) for x in (q1, k1, v1))
    pinned = [x.pin_memory() for x in (q1, k1, v1)]
    y_host = torch.empty(b, h, 1, d).pin_memory()

    pristine = cache["selected"].clone() if live else None

    def step(host: bool):
        cache["len"] = t
        if live:                                   # every step starts from the same history (the step adds to it)
            cache["selected"].copy_(pristine)
        if host:
            a, c, e = (x.to(device, non_blocking=True) for x in pinned)
            y_host.copy_(kernels.decode_step(cache, a, c, e), non_blocking=True)
        else:
            kernels.decode_step(cache, qd, kd, vd)

    results = {}
    for host in (False, True):
        for _ in range(args.warmup):
            step(host)
        if not host:
            _lib.profile_enable("decode")
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        before = _lib.launch_count()
        with ClockSampler(device.index) as sampler:
            e0.record()
            for _ in range(args.steps):
                step(host)
            e1.record()
            torch.cuda.synchronize()
        results[host] = max_over_ranks(e0.elapsed_time(e1) / args.steps, world, device)
        if not host:
            step_kernels = _lib.profile_collect()
            _lib.profile_enable("none")
            clocks = sampler.summary()
            launches = _lib.launch_count() - before
    algorithmic_bytes = 2 * b * h * (t + 1) * d * 2 + b * (t + 1) * 8       # K and V once, `selected` read + written
    hbm_peak, hbm_kind = 6650.0, "fallback"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        hbm_peak, hbm_kind = float(json.load(open(path))["hbm_gbs"]), "measured (device copy)"
    achieved = algorithmic_bytes / (results[False] * 1e-3) / 1e9
    return {"metric": "selective-attn cached decode steps/s (batch tokens/s) @131K-token cache bf16", "value":
            world * b / (results[False] * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": results[False], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"decode: one token, B={b} H={h} D={d}, cache of {t} tokens, bf16 K/V, fp32 selected",
                       "keys": ("every cached key is read" if not live else
                                "NOT the dense workload: history from a real prefill of the N(0,1) prompt; keys whose weight is "
                                "below 2^-150 are not read (same outputs); each step also restores the 0.5 MB history vector"),
                       "step_kernels_ms": (sum(step_kernels) / len(step_kernels)) if step_kernels else None,
                       "l2": "the K and V cache (512 MiB) exceeds the 126 MB L2"},
            "e2e": {"value": world * b / (results[True] * 1e-3), "unit": "tokens/s", "ms_per_step": results[True],
                    "h2d_bytes_per_step": 3 * b * h * d * 2, "d2h_bytes_per_step": b * h * d * 4},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "kernel": "decode step (append, attend, combine, update)",
                         "achieved": None if live else achieved, "peak": hbm_peak, "peak_kind": hbm_kind, "unit": "GB/s",
                         "frac": None if live else achieved / hbm_peak, "traffic": None,
                         **({"note": "no byte count is claimed when dead keys are left out"} if live else {})},
            "clocks": clocks}


def run_decoder(args, w, rank, world, device):
    """Full decoder training step (24 layers, d_model 1024, 16 heads x 64, GELU MLP 4096, pre-LN, no position
    signal, vocab 50304, T = 16384, bf16 autocast, fused AdamW): forward, backward, optimizer step.  Data
    parallel: one sequence per GPU, gradients all-reduced by DistributedDataParallel (NCCL, bucketed and
    overlapped with the backward)."""
    from selective_attention_b200 import _lib
    from selective_attention_b200.decoder import SelectiveDecoder, synthetic_batch

    torch.manual_seed(0)
    model = SelectiveDecoder(vocab_size=50304, n_layers=w["layers"], d_model=w["heads"] * w["dim"],
                             n_heads=w["heads"]).to(device)
    params = sum(p.numel() for p in model.parameters())
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[device.index], gradient_as_bucket_view=True)
    opt = torch.optim.AdamW(model.parameters(), lr=6e-4, weight_decay=0.1, betas=(0.9, 0.95), fused=True)
    gen = torch.Generator("cpu").manual_seed(1000 + rank)
    idx_h, tgt_h = synthetic_batch(w["batch"], w["seq"], 50304, 50256, gen)
    idx_h, tgt_h = idx_h.pin_memory(), tgt_h.pin_memory()
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def step(host: bool, idx_d=None, tgt_d=None):
        if host:
            idx_d, tgt_d = idx_h.to(device, non_blocking=True), tgt_h.to(device, non_blocking=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(idx_d, tgt_d)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        if host:
            loss_host.copy_(loss.detach(), non_blocking=True)
        return loss

    idx_d, tgt_d = idx_h.to(device), tgt_h.to(device)
    times = {}
    for host in (False, True):
        for _ in range(args.warmup if not host else 1):
            step(host, idx_d, tgt_d)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        n_steps = args.steps if not host else max(1, min(args.steps, 3))
        before = _lib.launch_count()
        with ClockSampler(device.index) as sampler:
            e0.record()
            for _ in range(n_steps):
                loss = step(host, idx_d, tgt_d)
            e1.record()
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()
        times[host] = max_over_ranks(e0.elapsed_time(e1) / n_steps, world, device)
        if not host:
            clocks, last_loss = sampler.summary(), float(loss.detach())
            launches = _lib.launch_count() - before
    if not math.isfinite(last_loss):
        raise RuntimeError("the training loss is not finite")
    tokens = w["batch"] * w["seq"]
    return {"metric": "decoder training step tokens/s (24L d1024 16x64, T=16384, bf16, selective attention)",
            "value": whole_job_tokens_per_second(tokens * world, times[False]), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": times[False], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"c5: decoder training step, {w['layers']} layers, d_model {w['heads'] * w['dim']}, "
                                   f"{w['heads']} heads x {w['dim']}, GELU MLP x4, pre-LN, no position signal, vocab 50304, "
                                   f"T={w['seq']}, {w['batch']} sequence(s) per GPU, AdamW, grad clip 1.0",
                       "parameters": params, "parallelism": f"dp{world}", "loss": last_loss,
                       "l2": "activations and weights far exceed the 126 MB L2"},
            "e2e": {"value": whole_job_tokens_per_second(tokens * world, times[True]), "unit": "tokens/s",
                    "ms_per_step": times[True], "h2d_bytes_per_step": 2 * tokens * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "clocks": clocks}


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_listing():
    """The reference's own dense implementation of the operator (its ``selective_attention_reference``) from the
    installed copy under baseline/_ref, or None where that copy is absent (then the CPU oracle port stands in)."""
    if not os.path.isdir(os.path.join(REF_DIR, "selective_attention")):
        return None
    if REF_DIR not in sys.path:
        sys.path.append(REF_DIR)
    try:
        from selective_attention.kernels import selective_attention_reference
        return selective_attention_reference
    except Exception:
        return None


def _listing_fwd_bwd(listing, q, k, v, w):
    """One forward + backward on the CPU: autograd through the reference's listing, or the oracle port."""
    if listing is not None:
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        listing(qq, kk, vv).backward(w)
        return
    import selective_oracle as oracle
    if q.shape[2] > 4096:
        for b in range(q.shape[0]):
            oracle.sequence_fwd_bwd(q[b], k[b], v[b], w[b], head_chunk=1)
    else:
        oracle.attention_grads(q, k, v, w)


def cpu_baseline(seconds: float = 12.0) -> dict:
    """The reference's CPU implementation (or the oracle port of it) on the reference's own CPU-sized case:
    B=2, H=4, T=1024, D=64, fp32, seed 0."""
    listing = reference_listing()
    g = torch.Generator("cpu").manual_seed(0)
    q, k, v, w = (torch.randn(2, 4, 1024, 64, generator=g) for _ in range(4))
    _listing_fwd_bwd(listing, q, k, v, w)
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds:
        _listing_fwd_bwd(listing, q, k, v, w)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    kind = "reference" if listing is not None else "port"
    return {"value": 2 * 1024 / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{'reference listing + autograd' if listing else 'oracle'} fwd+bwd at B=2 H=4 T=1024 D=64 fp32 "
                      f"(the reference's CPU case), {reps} passes, {dt * 1e3:.1f} ms each"}


def reference_on_gpu(args, w, device) -> dict:
    """The reference's own Triton kernels (installed copy, unmodified) on this GPU at the workload's full
    configuration, timed like the product arm (CUDA events, same warm-up and steps)."""
    try:
        if REF_DIR not in sys.path:
            sys.path.append(REF_DIR)
        from selective_attention import kernels as ref
        if not ref.HAS_TRITON:
            return {"unavailable": "triton is not importable"}
        torch.cuda.set_device(device)
        q, k, v, d_out = (t.to(device) for t in make_inputs(w, seed=0))
        if w["per_head"]:
            q, k, v, d_out = (t.reshape(-1, 1, t.shape[2], t.shape[3]) for t in (q, k, v, d_out))
        d_out = d_out.float()
        for t in (q, k, v):
            t.requires_grad_(w["backward"])

        def step():
            if w["backward"]:
                ref.selective_attention(q, k, v).backward(d_out)
                q.grad = k.grad = v.grad = None
            else:
                with torch.no_grad():
                    ref.selective_attention_forward(q, k, v, return_aux=True)

        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        return {"value": w["batch"] * w["seq"] / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                "what": "the reference's Triton kernels through its selective_attention(), unmodified, on this GPU; "
                        "same shapes, dtype and inputs as the product arm, inputs resident in HBM"}
    except Exception as exc:                                     # a Triton build that cannot target this GPU, etc.
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


def run_reference(args, w):
    """The reference's CPU implementation of the operator on the host cores.  Each step is one sequence of the
    workload restricted to 2 of its heads (head 0, the selector, and one more) at a sample length T_s chosen so
    that the whole run stays within a few minutes; per-head work is equal and the work per head grows with the
    causal pairs T (T + 1) / 2, so the full workload's time is the sample's time x heads / 2 x pairs(T) / pairs(T_s)."""
    torch.set_num_threads(os.cpu_count() or 1)       # torchrun sets OMP_NUM_THREADS=1; this arm runs on rank 0 alone
    listing = reference_listing()
    heads_sample = min(2, w["heads"])
    g = torch.Generator("cpu").manual_seed(0)

    def sample(seq):
        return tuple(torch.randn(1, heads_sample, seq, w["dim"], generator=g).bfloat16().float() for _ in range(4))

    def one(q, k, v, d):
        if w["backward"]:
            _listing_fwd_bwd(listing, q, k, v, d)
        elif listing is not None:
            with torch.no_grad():
                listing(q, k, v)
        else:
            import selective_oracle as oracle
            oracle.tail_rows(q, k, v, tail=q.shape[2], chunk=4096)

    # calibrate on a short sequence, then take the longest sample length that keeps the run under ~3 minutes
    probe = sample(min(2048, w["seq"]))
    one(*probe)
    t0 = time.perf_counter()
    one(*probe)
    per_pair = (time.perf_counter() - t0) / pairs(probe[0].shape[2])
    seq_s = w["seq"]
    steps_total = args.steps + min(args.warmup, 1)
    avail = 0.45 * (os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES"))
    while seq_s > 2048 and (per_pair * pairs(seq_s) * steps_total > 180.0 or 14 * heads_sample * seq_s * seq_s * 4 > avail):
        seq_s //= 2
    q, k, v, d = sample(seq_s)
    for _ in range(min(args.warmup, 1)):
        one(q, k, v, d)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one(q, k, v, d)
    dt = (time.perf_counter() - t0) / args.steps
    scale = w["heads"] / heads_sample * pairs(w["seq"]) / pairs(seq_s)
    value = w["seq"] / (dt * scale)
    kind = "reference" if listing is not None else "port"
    what = ("the reference's selective_attention_reference with autograd (baseline/_ref)" if listing is not None
            else "CPU oracle port of the reference's listing")
    smp = (f"{what}: 1 sequence x {heads_sample} of {w['heads']} heads at T_s={seq_s} of T={w['seq']}, D={w['dim']}, "
           f"{'fwd+bwd' if w['backward'] else 'forward'}; {dt:.2f} s per step, scaled x{scale:g}")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: the reference's CPU implementation on a bounded sample"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                             "sample": smp},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if torch.cuda.is_available() and not args.no_reference_gpu and args.workload in ("c2", "c3", "c4"):
        line["reference_gpu"] = reference_on_gpu(args, w, torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    return line


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--seq", type=int, default=None, help="override T (profiling on a small case)")
    ap.add_argument("--batch", type=int, default=None, help="override B (profiling on a small case)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count of the c5 decoder")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-call", default="packed", choices=["packed", "plain"],
                    help="end-to-end arm: the layer-facing packed call (default where it applies) or the (B, H, T, D) call")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="--impl reference: skip timing the reference's Triton kernels on the GPU")
    ap.add_argument("--skip-dead-tiles", action="store_true",
                    help="a separate row, not the headline: leave out tiles whose probabilities are all exactly zero")
    ap.add_argument("--replicas", action="store_true",
                    help="N > 1: every rank runs its own full batch (weak scaling) instead of a shard of one batch")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    w = dict(WORKLOADS[args.workload])
    if args.seq:
        w["seq"] = args.seq
    if args.batch:
        w["batch"] = args.batch
    if args.layers and "layers" in w:
        w["layers"] = args.layers

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, w)), flush=True)
        return

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for the product)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    if args.warmup < 3:
        args.warmup = 3
    runner = {"decode": run_decode, "c5": run_decoder}.get(args.workload, run_ours)
    line = runner(args, w, rank, world, device)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and args.workload not in ("decode", "c5"):
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
