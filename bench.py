#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline metric: causal prefill attention throughput (TFLOP/s, algorithmic causal FLOPs) on the
long-context shape 16 heads x 128, bf16, T = 32768 (heads partitioned over N GPUs, head outputs
exchanged by the kernel's epilogue or a NCCL all-gather).  The same JSON line carries the decode
metric (tokens/s of the llama2-7B-shape KV-cache attention, batch 64, cache lengths uniform in
[512, 4096]) under "decode", and at N = 1 the other configurations under "train" (GPT-2-small
attention core, forward + backward, fp32 and bf16), "sweep" (prefill at other lengths and
batches), "backward", "decode_bf16" / "decode_b1" / "decode_b16" and "tft".  Inputs are seeded
synthetic tensors of those shapes, generated per head from fixed seeds so that every GPU count
computes the same global problem.  After the timed regions rank 0 compares a strided sample of
the timed prefill output (>= 512 query rows of every (batch, head)) and a few decode sequences
with the CPU oracle on the same inputs ("parity"); the run fails when a tolerance is exceeded.
The time the oracle takes for that sample is the CPU baseline.

``--impl reference`` times the reference's own CPU math for the same two workloads on the host
cores (bounded samples): the CPU restatement of attn.cu for prefill and the reference's
llama2_cpu.cpp, compiled from its source, for decode.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# workload (BASELINE config 5 / config 3)
PF_B, PF_H, PF_D, PF_T = 4, 16, 128, 32768
PREFILL_TRAFFIC_PER_ALGORITHMIC_BYTE = 2180408320 / 2147483648   # measured DRAM bytes / (Q+K+V+O bytes)
DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE = 2152038680 / 2148532224    # measured DRAM bytes / decode_bytes()
DEC_B, DEC_HEADS, DEC_HS, DEC_SEQ, DEC_LAYERS, DEC_BUFFERS = 64, 32, 128, 4096, 32, 4
DEC_LMIN, DEC_LMAX = 512, 4096


def causal_flops(B, H, T, D):
    """4*B*H*D*T*(T+1)/2: two products x 2 flop/MAC over the lower triangle incl. the diagonal."""
    return 4.0 * B * H * D * T * (T + 1) / 2.0


def decode_bytes(lengths, kv_dim, dim, elt):
    """Per layer-step: K and V rows 0..L-1 read once, the new k,v row written, q read and o written."""
    return float(sum(2 * L * kv_dim * elt + 2 * kv_dim * elt + 2 * dim * 4 for L in lengths))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle-reason samples during the timed region (read-only queries).  NVML through
    pynvml when it loads: a sample costs microseconds, so that a timed region of a few milliseconds still gets
    several; otherwise `nvidia-smi -lms 20`, whose first line arrives after about 100 ms."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []
        self.nvml, self.handle, self.samples, self.run = None, None, [], False
        try:
            import pynvml
            pynvml.nvmlInit()
            # CUDA_VISIBLE_DEVICES may renumber the devices: look the handle up by the CUDA device's PCI bus id
            import torch
            bus = torch.cuda.get_device_properties(gpu_index).pci_bus_id if hasattr(torch.cuda.get_device_properties(gpu_index), "pci_bus_id") else None
            self.handle = None
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    if int(pynvml.nvmlDeviceGetPciInfo(h).bus) == int(bus):
                        self.handle = h
                        break
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.nvml = pynvml
        except Exception:  # noqa: BLE001 - any NVML problem selects nvidia-smi
            self.nvml = None

    def _nvml_loop(self):
        n = self.nvml
        masks = [n.nvmlClocksEventReasonHwSlowdown, n.nvmlClocksEventReasonHwThermalSlowdown,
                 n.nvmlClocksEventReasonSwThermalSlowdown, n.nvmlClocksEventReasonSwPowerCap]
        while self.run:
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                smax = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
                bits = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.samples.append((float(sm), float(smax), [nm for nm, m in zip(self.NAMES, masks) if bits & m]))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def start(self):
        if self.nvml is not None:
            self.run = True
            self.t = threading.Thread(target=self._nvml_loop, daemon=True)
            self.t.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.run = False
            self.t.join(timeout=1)
            sm = [s_[0] for s_ in self.samples]
            reasons = sorted({r for s_ in self.samples for r in s_[2]})
            return {"sm_mhz": float(np.median(sm)) if sm else None,
                    "sm_max_mhz": max(s_[1] for s_ in self.samples) if self.samples else None,
                    "reasons": reasons, "samples": len(sm), "source": "nvml"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# --------------------------------------------------------------------------------------------- ours

class Ctx:
    """What every leg of the run needs: library, device, stream, rank layout, peaks."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from mycaffe_b200 import _lib
        self.args, self.torch, self.dist = args, torch, dist
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        # several ranks stage host tensors at once: keep each rank's (pinned) host memory on its GPU's NUMA node
        self.affinity = {"skipped": "single process"}
        if self.world > 1:
            from mycaffe_b200 import head_shard
            try:
                self.affinity = head_shard.bind_near_gpu(self.local)
            except Exception as e:       # never let the placement hint stop a run
                self.affinity = {"skipped": f"{type(e).__name__}: {e}"}
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.lib = _lib.load()
        self.peaks = measured_peaks()
        self.stream = torch.cuda.current_stream()
        self.sp = C.c_void_p(self.stream.cuda_stream)
        self.flush_buf = None

    def barrier(self):
        if self.world > 1 and self.dist.is_initialized():
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def flush_l2(self):
        """Write a buffer twice the size of the 126 MB L2 (for workloads smaller than L2)."""
        if self.flush_buf is None:
            self.flush_buf = self.torch.empty(256 << 20, dtype=self.torch.uint8, device=self.dev)
        self.flush_buf.zero_()

    def time_kernel(self, fn, iters, warm=2, flush=False):
        """Mean CUDA-event time (ms) of fn() on the current stream; with `flush` the L2 is overwritten before
        every timed call (outside the event pair)."""
        torch = self.torch
        for _ in range(warm):
            rc = fn()
            if rc:
                raise RuntimeError(f"launch failed with {rc}")
        torch.cuda.synchronize()
        total = 0.0
        if not flush:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(iters):
                fn()
            e1.record(self.stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters
        for _ in range(iters):
            self.flush_l2()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            fn()
            e1.record(self.stream)
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / iters


def prefill_head_inputs(torch, gen, B, T, D, h):
    """q, k, v (B,T,D) bf16 of global head h: the same values whichever rank generates them."""
    gen.manual_seed(1000 + h)
    return [(torch.randn(B, T, D, device=gen.device, generator=gen) / D ** 0.5).to(torch.bfloat16) for _ in range(3)]


def run_ours(args):
    from mycaffe_b200 import function_ids as ids, head_shard
    cx = Ctx(args)
    torch, dist, lib, dev, rank, world, local, sp, stream = cx.torch, cx.dist, cx.lib, cx.dev, cx.rank, cx.world, cx.local, cx.sp, cx.stream
    peaks = cx.peaks
    barrier = cx.barrier

    # ----------------------------------------------------------------- prefill (headline)
    B, H, D, T = args.batch, PF_H, PF_D, args.seq_len
    h_lo, h_hi = head_shard.head_range(rank, world, H)
    Hl = h_hi - h_lo
    gen = torch.Generator(device=dev)
    q = torch.empty(B, Hl, T, D, device=dev, dtype=torch.bfloat16)
    k, v = torch.empty_like(q), torch.empty_like(q)
    for hl in range(Hl):  # per-head seeds: the same global problem for every N
        qh, kh, vh = prefill_head_inputs(torch, gen, B, T, D, h_lo + hl)
        q[:, hl], k[:, hl], v[:, hl] = qh, kh, vh
    del qh, kh, vh
    y = torch.empty_like(q)
    y_all = torch.empty(world, B, Hl, T, D, device=dev, dtype=torch.bfloat16) if world > 1 else None
    status = torch.zeros(8, device=dev, dtype=torch.int32)
    # Exchange of the head outputs when world > 1: by default the kernel's epilogue stores its tiles straight
    # into every rank's (B,H,T,D) buffer over NVLink and a one-element all-reduce follows; if symmetric memory
    # cannot be set up on this box, a NCCL all-gather after the kernel.
    peer_out, exchange = None, "none"
    if world > 1:
        exchange = "nccl all-gather after the kernel"
        if not args.nccl_exchange:
            try:
                peer_out = head_shard.PeerOutput(B, H, T, D, dev)
                peer_dst, (ysb, ysh, yst) = peer_out.destinations(h_lo), peer_out.strides
                exchange = "kernel epilogue stores to every rank's buffer (peer memory over NVLink) + 1-element all-reduce"
            except Exception as exc:  # noqa: BLE001 - any failure to map peer memory selects the NCCL exchange
                peer_out = None
                exchange += f" (symmetric memory unavailable: {type(exc).__name__})"

    use_fused = [peer_out is not None]

    def launch_prefill():
        if use_fused[0]:
            return lib.mca_sdpa_forward_tc_scatter(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, Hl, T, D,
                                                   peer_dst, world, ysb, ysh, yst, None, status.data_ptr(), sp)
        return lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, Hl, T, D,
                                       y.data_ptr(), None, status.data_ptr(), sp)

    def exchange_outputs():
        if use_fused[0]:
            peer_out.wait()
        elif world > 1:
            head_shard.gather_heads(y, out=y_all, strided=True)

    def prefill_step():
        rc = launch_prefill()
        if rc:
            raise RuntimeError(f"prefill launch failed with {rc}")
        exchange_outputs()

    for _ in range(args.warmup):
        prefill_step()
    barrier()
    if int(status[0].item()) != 0:
        raise RuntimeError(f"prefill kernel reported status {status[:4].tolist()}")
    if peer_out is not None:
        # Both exchanges are checked against the oracle below; time two steps of each (max over ranks) and keep the
        # faster one for this size.
        trial = {}
        for name, flag in (("fused", True), ("nccl", False)):
            use_fused[0] = flag
            prefill_step()
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            prefill_step()
            prefill_step()
            t1.record(stream)
            barrier()
            trial[name] = cx.max_over_ranks([t0.elapsed_time(t1) / 2])[0]
        use_fused[0] = trial["fused"] <= trial["nccl"]
        if not use_fused[0]:
            exchange = "nccl all-gather after the kernel"
        exchange += " (chosen by a two-step trial: epilogue peer stores %.3f ms, kernel + NCCL all-gather %.3f ms per step)" % (
            trial["fused"], trial["nccl"])
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    kern_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    ev[0].record(stream)
    for i in range(args.steps):
        kern_ev[i][0].record(stream)
        rc = launch_prefill()
        kern_ev[i][1].record(stream)
        exchange_outputs()
        ev[i + 1].record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if rc or int(status[0].item()) != 0:
        raise RuntimeError(f"prefill launch {rc}, status {status[:4].tolist()}")
    total_ms = ev[0].elapsed_time(ev[-1])
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in kern_ev]))
    total_ms, kern_ms = cx.max_over_ranks([total_ms, kern_ms])
    ms_per_step = total_ms / args.steps
    flops_total = causal_flops(B, H, T, D)
    value = flops_total / (ms_per_step * 1e-3) / 1e12
    flops_launch = causal_flops(B, Hl, T, D)
    achieved = flops_launch / (kern_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "sdpa_fwd_tc_kernel<128>", "achieved": round(achieved, 2),
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4) if peaks.get("bf16_tflops_sustained") else None,
                "peak_source": peaks["source"], "kernel_ms": round(kern_ms, 4),
                # dram__bytes_read + dram__bytes_write of one launch of this workload (ncu, `--case prefill-full`):
                # 2.18 GB at B=4, T=32768 against 2.15 GB of Q, K, V, O; scaled by the bytes of other shapes
                "traffic": int(PREFILL_TRAFFIC_PER_ALGORITHMIC_BYTE * 4 * q.numel() * 2),
                "traffic_source": "ncu capture of one launch of `--case prefill-full` (sdpa_fwd_tc_kernel, B=4 T=32768)",
                "flops_per_launch": flops_launch, "flop_count": "causal 4*B*H*D*T*(T+1)/2"}
    if world > 1:
        # compute + exchange as one step: the target is the slower of this GPU's FLOPs at the measured GEMM peak and the
        # bytes it must send over NVLink (its (B, H/N, T, D) bf16 outputs to each of the N - 1 peers) at the measured
        # peer-copy rate of 770 GB/s per direction
        nvlink_bytes = (world - 1) * B * Hl * T * D * 2
        t_flops = flops_launch / (peaks["bf16_tflops"] * 1e12) * 1e3
        t_link = nvlink_bytes / 770e9 * 1e3
        roofline["with_exchange"] = {"nvlink_bytes_per_gpu": nvlink_bytes, "nvlink_GBps_reference": 770.0,
                                     "compute_ms_at_peak": round(t_flops, 4), "nvlink_ms_at_reference": round(t_link, 4),
                                     "target_ms": round(max(t_flops, t_link), 4), "achieved_ms": round(ms_per_step, 4),
                                     "frac": round(max(t_flops, t_link) / ms_per_step, 4),
                                     "fused": bool(use_fused[0])}

    # A strided sample of the timed output, every (batch, head), for the oracle comparison after the GPU legs.
    q_step = max(1, T // 512)
    q_begin = (q_step * 5) // 8
    rows = torch.arange(q_begin, T, q_step, device=dev)
    prefill_sample = None
    if rank == 0:
        def head_output(h):   # (B,T,D) of global head h as the exchange left it on this rank
            if world == 1:
                return y[:, h]
            if use_fused[0]:
                return peer_out.tensor[:, h]
            r, hl = divmod(h, Hl)
            return y_all[r, :, hl]
        prefill_sample = torch.stack([head_output(h).index_select(1, rows) for h in range(H)], 1).float().cpu().numpy()

    # ----------------------------------------------------------------- decode (secondary metric, rank-local heads)
    decode, decode_check = run_decode(cx, DEC_B, False, multi=True, steps=max(3, min(args.steps, 10)))

    # ----------------------------------------------------------------- end to end through the dispatch ABI (host buffers)
    e2e = run_e2e(args, torch, dev, local, rank, world, barrier, B, H, Hl, T, D, q, k, v)
    e2e["host_affinity"] = {k_: v_ for k_, v_ in cx.affinity.items() if k_ != "previous"}
    e2e["h2d_gbs_per_rank"] = round(e2e["h2d_bytes_per_step"] / (e2e["ms_per_step"] * 1e-3) / 1e9, 1)

    # ----------------------------------------------------------------- the other configurations (one GPU)
    extras, extra_checks = {}, {}
    del y_all
    if world == 1 and args.extras:
        del q, k, v, y
        torch.cuda.empty_cache()
        extras["sweep"] = run_sweep(cx)
        extras["backward"] = run_backward(cx)
        extras["fp32_prefill"] = run_fp32_prefill(cx)
        extras["train"] = run_train(cx)
        extras["train_function_ids"] = run_train_function_ids(cx)
        for key, (bt, bf) in {"decode_bf16": (DEC_B, True), "decode_b16": (16, False), "decode_b1": (1, False)}.items():
            extras[key], extra_checks[key] = run_decode(cx, bt, bf, multi=False, steps=3)
        extras["tft"] = run_tft(cx)
        extras["decode_projections"] = run_projections(cx)

    # ----------------------------------------------------------------- CPU legs: rank 0, after the process group is gone
    barrier()
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    if "previous" in cx.affinity:       # the CPU legs below use every core again
        try:
            os.sched_setaffinity(0, cx.affinity["previous"])
        except OSError:
            pass
    import oracle
    cores = oracle.set_num_threads()    # a launcher may have exported OMP_NUM_THREADS=1 for its workers
    parity, cpu_base = prefill_parity(torch, dev, B, H, T, D, q_begin, q_step, prefill_sample, cores)
    decode["parity"] = decode_parity(cx, decode_check)
    for key, chk in extra_checks.items():
        extras[key]["parity"] = decode_parity(cx, chk)
    line = {
        "metric": "attn_prefill_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"config5 causal prefill B={B} H={H} D={D} T={T} bf16, heads partitioned over {world} GPU(s)"
                               + (f"; exchange of head outputs: {exchange}" if world > 1 else ""),
                   "l2": "inputs (Q,K,V,O %.0f MB per rank) exceed the 126 MB L2" % (4 * B * Hl * T * D * 2 / 1e6),
                   "parallelism": f"heads/{world}"},
        "gpu_launches": args.steps, "clocks": clocks, "roofline": roofline, "parity": parity, "e2e": e2e, "decode": decode,
        "cpu_baseline": cpu_base,
    }
    line.update(extras)
    line["decode"]["cpu_baseline"] = cpu_baseline_decode()
    if world == 1 and args.cpu_baseline:
        try:
            line["decode"]["whole_model"] = whole_model_decode()
        except Exception as exc:   # an extra; never the reason the bench line is lost
            line["decode"]["whole_model"] = {"unavailable": repr(exc)}
    print(json.dumps(line), flush=True)
    bad = [n for n, pr in [("prefill", parity), ("decode", decode["parity"])] + [(k_, extras[k_]["parity"]) for k_ in extra_checks]
           if not pr["ok"]]
    if bad:
        raise SystemExit(f"parity against the CPU oracle failed for: {', '.join(bad)}")


def prefill_parity(torch, dev, B, H, T, D, q_begin, q_step, sample, cores):
    """The timed prefill output against the restated reference math on the same q, k, v: query rows
    q_begin::q_step of every (batch, head).  The same pass is the CPU baseline: its causal FLOPs over its time."""
    import oracle
    gen = torch.Generator(device=dev)
    worst, cpu_s, n_rows = 0.0, 0.0, 0
    for h in range(H):
        qh, kh, vh = (t_.float().cpu().numpy().reshape(B, 1, T, D) for t_ in prefill_head_inputs(torch, gen, B, T, D, h))
        t0 = time.perf_counter()
        ref = oracle.sdpa_forward_rows(qh, kh, vh, None, 3, q_begin, q_step)      # (B,1,rows,D)
        cpu_s += time.perf_counter() - t0
        got = sample[:, h:h + 1]
        worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
        n_rows = ref.shape[2]
    rows = np.arange(q_begin, T, q_step)
    flops = 4.0 * B * H * D * float(np.sum(rows + 1))
    tol = 2e-2
    parity = {"rows": int(n_rows) * B * H, "rows_per_batch_head": int(n_rows), "max_rel_err": worst, "tolerance": tol,
              "ok": bool(worst <= tol),
              "against": "oracle.sdpa_forward_rows (restated attn.cu:518-602, fp32) on the same bf16-rounded q, k, v; "
                         "error = max-abs difference over the max-abs of the reference, per (batch, head)"}
    cpu = {"value": round(flops / cpu_s / 1e12, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port",
           "sample": f"{n_rows} strided query rows of each of the {B * H} (batch, head) pairs of the T={T} causal problem "
                     f"({flops / 1e9:.1f} GFLOP causal, {cpu_s:.1f} s; the parity rows); full-problem time extrapolated from this rate"}
    return parity, cpu


def decode_head_tensors(torch, gen, batch, seq, hs, h, buf):
    """K and V cache columns (batch, seq, hs) of global head h in rotating buffer `buf`, fp32."""
    gen.manual_seed(5000 + 64 * buf + h)
    return (torch.randn(batch, seq, hs, device=gen.device, generator=gen),
            torch.randn(batch, seq, hs, device=gen.device, generator=gen))


def decode_head_token(torch, gen, batch, hs, h):
    """q, k_new, v_new (batch, hs) of global head h."""
    gen.manual_seed(9000 + h)
    return [torch.randn(batch, hs, device=gen.device, generator=gen) for _ in range(3)]


def run_decode(cx, batch, bf16, multi, steps):
    """llama2-7B-shape decode attention: one new token for `batch` sequences, one launch pair per layer.
    multi: heads partitioned over the ranks with an all-gather of the head outputs per layer-step.
    Returns the result and what the oracle comparison needs afterwards."""
    from mycaffe_b200 import head_shard
    torch, lib, dev, sp, stream, peaks = cx.torch, cx.lib, cx.dev, cx.sp, cx.stream, cx.peaks
    rank, world = (cx.rank, cx.world) if multi else (0, 1)
    lo, hi = head_shard.head_range(rank, world, DEC_HEADS)
    heads = hi - lo
    kv_dim = dim = heads * DEC_HS
    elt = 2 if bf16 else 4
    rng = np.random.default_rng(0)
    lengths = rng.integers(DEC_LMIN, DEC_LMAX + 1, max(batch, 2))[:batch]
    if batch == 1:
        lengths[:] = DEC_LMAX      # a single sequence: the full-length cache
    pos = torch.tensor(lengths - 1, dtype=torch.int32, device=dev)
    max_len = int(lengths.max())
    # distinct layer caches, rotated, so that together they are far larger than L2
    per_buffer = 2 * batch * DEC_SEQ * kv_dim * elt
    n_buf = max(DEC_BUFFERS, int(np.ceil(3 * 126e6 / per_buffer)))
    cdt = torch.bfloat16 if bf16 else torch.float32
    gen = torch.Generator(device=dev)
    caches = []
    for bi in range(n_buf):
        kc = torch.empty(batch, DEC_SEQ, kv_dim, device=dev, dtype=cdt)
        vc = torch.empty_like(kc)
        for hl in range(heads):
            kh, vh = decode_head_tensors(torch, gen, batch, DEC_SEQ, DEC_HS, lo + hl, bi)
            kc[:, :, hl * DEC_HS:(hl + 1) * DEC_HS], vc[:, :, hl * DEC_HS:(hl + 1) * DEC_HS] = kh, vh
        caches.append((kc, vc))
    qn, kn, vn = (torch.empty(batch, dim, device=dev) for _ in range(3))
    for hl in range(heads):
        for dst, src in zip((qn, kn, vn), decode_head_token(torch, gen, batch, DEC_HS, lo + hl)):
            dst[:, hl * DEC_HS:(hl + 1) * DEC_HS] = src
    out = torch.empty(batch, dim, device=dev)
    out_all = torch.empty(world, batch, dim, device=dev) if world > 1 else None
    # Exchange of the head outputs when world > 1: the library's exchange kernel (peer stores + flags, no collective
    # per layer-step) when symmetric memory can be set up, else a NCCL all-gather; a short trial picks the faster one.
    peer, exchange = None, "none"
    if world > 1:
        exchange = "nccl all-gather per layer-step"
        if not cx.args.nccl_exchange:
            try:
                peer = head_shard.PeerDecodeOutput(batch, world * dim, dev, lib)
                exchange = "exchange kernel per layer-step (peer stores over NVLink + flags)"
            except Exception as exc:  # noqa: BLE001 - any failure to map peer memory selects the NCCL exchange
                peer = None
                exchange += f" (symmetric memory unavailable: {type(exc).__name__})"
    use_peer = [peer is not None]
    last = [None]
    sl, ns, need = C.c_int(), C.c_int(), C.c_int64()
    lib.mca_decode_plan(batch, heads, heads, DEC_HS, max_len, C.byref(sl), C.byref(ns), C.byref(need))
    scratch = torch.empty(max(1, need.value), device=dev)
    fr = np.empty((DEC_SEQ, DEC_HS // 2), np.float32)
    fi = np.empty_like(fr)
    fp = C.POINTER(C.c_float)
    lib.mca_rope_tables_host(DEC_SEQ, DEC_HS, 10000.0, fr.ctypes.data_as(fp), fi.ctypes.data_as(fp))
    frd, fid = torch.from_numpy(fr).to(dev), torch.from_numpy(fi).to(dev)

    def layer(i):
        kc, vc = caches[i % n_buf]
        rc = lib.mca_decode_attention(qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), kc.data_ptr(), vc.data_ptr(), int(bf16),
                                      DEC_SEQ * kv_dim, pos.data_ptr(), batch, heads, heads, DEC_HS, DEC_SEQ, max_len,
                                      frd.data_ptr(), fid.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                      out.data_ptr(), sp)
        if rc:
            raise RuntimeError(f"mca_decode_attention failed with {rc}")
        if world > 1:  # the head outputs of every rank, as the Wo projection of the next step needs them
            if use_peer[0]:
                last[0] = peer.exchange(out, stream)
            else:
                head_shard.gather_decode_outputs(out, out=out_all)

    for i in range(3 * n_buf):
        layer(i)
    if multi:
        cx.barrier()
    else:
        torch.cuda.synchronize()
    if peer is not None:
        trial = {}
        for name, flag in (("peer", True), ("nccl", False)):
            use_peer[0] = flag
            for i in range(n_buf):
                layer(i)
            cx.barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for i in range(DEC_LAYERS):
                layer(i)
            t1.record(stream)
            cx.barrier()
            trial[name] = cx.max_over_ranks([t0.elapsed_time(t1)])[0]
        if peer.status()[0] != 0:
            raise RuntimeError(f"decode exchange gave up: {peer.status()}")
        use_peer[0] = trial["peer"] <= trial["nccl"]
        if not use_peer[0]:
            exchange = "nccl all-gather per layer-step"
        exchange += " (chosen by a trial of %d layer-steps: exchange kernel %.3f ms, NCCL all-gather %.3f ms)" % (DEC_LAYERS, trial["peer"], trial["nccl"])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for s in range(steps):
        for i in range(DEC_LAYERS):
            layer(i)
    e1.record(stream)
    if multi:
        cx.barrier()
    else:
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if multi:
        ms = cx.max_over_ranks([ms])[0]
    st = (C.c_int * 3)()
    lib.mca_decode_status(st)
    if st[0]:
        raise RuntimeError(f"decode kernel refused {st[0]} position(s)")
    ms_step = ms / steps
    layer_ms = ms_step / DEC_LAYERS
    bytes_layer = decode_bytes(lengths, kv_dim, dim, elt)
    gbs = bytes_layer / (layer_ms * 1e-3) / 1e9
    # what the oracle comparison needs: the gathered output of layer 0's buffer for a few sequences
    layer(0)
    torch.cuda.synchronize()
    seqs = sorted({int(np.argmin(lengths)), int(np.argmax(lengths)), batch // 2})
    if world > 1 and use_peer[0]:
        if peer.status()[0] != 0:
            raise RuntimeError(f"decode exchange gave up: {peer.status()}")
        got = last[0][seqs].cpu().numpy()
    elif world > 1:
        got = out_all.transpose(0, 1).reshape(batch, world * dim)[seqs].cpu().numpy()
    else:
        got = out[seqs].cpu().numpy()
    check = {"batch": batch, "bf16": bf16, "seqs": seqs, "lengths": lengths, "got": got, "heads_total": DEC_HEADS if multi else heads}
    res = {"metric": "decode_tokens_per_s", "value": round(batch / (ms_step * 1e-3), 1), "unit": "tok/s",
           "ms_per_step": round(ms_step, 4), "steps": steps, "dtype": "bf16" if bf16 else "f32",
           "config": {"exchange": exchange, "workload": f"config3 decode attention batch={batch} heads={DEC_HEADS} (x{DEC_HS}) over {world} GPU(s), "
                                  f"cache lengths U[{DEC_LMIN},{DEC_LMAX}] (mean {lengths.mean():.0f}), {'bf16' if bf16 else 'fp32'} cache, "
                                  f"{DEC_LAYERS} layer-steps per token rotating {n_buf} distinct layer caches "
                                  f"({n_buf * per_buffer / 1e6:.0f} MB in all, above the 126 MB L2)",
                      "split_len": sl.value, "nsplit": ns.value},
           "gpu_launches": steps * DEC_LAYERS * (2 if ns.value > 1 else 1),
           "roofline": {"bound": "hbm", "kernel": "decode_split_kernel<%s,128,1>" % ("bf16" if bf16 else "float"), "achieved": round(gbs, 1),
                        "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                        "peak_source": peaks["source"], "bytes_per_launch": bytes_layer, "kernel_ms": round(layer_ms, 5),
                        # ncu on the 16-sequence case reads 1.0016 x the algorithmic bytes; traffic grows with the keys read
                        "traffic": int(DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_layer),
                        "traffic_source": "ncu capture of `--case decode-small` (decode_split_kernel, 16 sequences of 4096 keys), scaled by bytes"}}
    del caches
    torch.cuda.empty_cache()
    return res, check


def decode_parity(cx, chk):
    """A few of the decode sequences against the restated reference step (llama2_cpu.cpp:290-342) on the same
    caches and token: all heads, whichever rank computed them."""
    import oracle
    torch, dev = cx.torch, cx.dev
    gen = torch.Generator(device=dev)
    batch, seqs, H, hs = chk["batch"], chk["seqs"], chk["heads_total"], DEC_HS
    n = len(seqs)
    kc = np.empty((n, DEC_SEQ, H * hs), np.float32)
    vc = np.empty_like(kc)
    q, kn, vn = (np.empty((n, H * hs), np.float32) for _ in range(3))
    idx = torch.tensor(seqs, device=dev)
    for h in range(H):
        kh, vh = decode_head_tensors(torch, gen, batch, DEC_SEQ, hs, h, 0)
        if chk["bf16"]:
            kh, vh = kh.bfloat16().float(), vh.bfloat16().float()
        kc[:, :, h * hs:(h + 1) * hs], vc[:, :, h * hs:(h + 1) * hs] = kh[idx].cpu().numpy(), vh[idx].cpu().numpy()
        for dst, src in zip((q, kn, vn), decode_head_token(torch, gen, batch, hs, h)):
            dst[:, h * hs:(h + 1) * hs] = src[idx].cpu().numpy()
    pos = (chk["lengths"][seqs] - 1).astype(np.int32)
    ref = oracle.llama_decode(q, kn, vn, kc, vc, pos, H, H)
    err = float(np.abs(chk["got"] - ref).max() / np.abs(ref).max())
    tol = 2e-2 if chk["bf16"] else 1e-4
    return {"sequences": [int(s_) for s_ in seqs], "lengths": [int(x) for x in chk["lengths"][seqs]], "heads": H, "max_rel_err": err,
            "tolerance": tol, "ok": bool(err <= tol), "against": "oracle.llama_decode (restated llama2_cpu.cpp:290-342) on the same caches"}


# --------------------------------------------------------------------------------------------- other configurations (N = 1)

def tensor_roofline(cx, tflops, kernel, kernel_ms, note=None):
    pk = cx.peaks
    r = {"bound": "tensor", "kernel": kernel, "achieved": round(tflops, 2), "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
         "frac": round(tflops / pk["bf16_tflops"], 4), "peak_source": pk["source"], "kernel_ms": round(kernel_ms, 4), "traffic": None}
    if note:
        r["note"] = note
    return r


def run_sweep(cx):
    """Config 5 forward at the other lengths and batches: CUDA-event time of the one launch per step."""
    from mycaffe_b200 import function_ids as ids
    torch, lib, dev, sp = cx.torch, cx.lib, cx.dev, cx.sp
    H, D = PF_H, PF_D
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    out = []
    for T in (2048, 4096, 8192, 32768):
        for B in (1, 4):
            if T == PF_T and B == PF_B:
                continue   # the headline
            q, k, v = (torch.randn(B, H, T, D, device=dev).div_(D ** 0.5).bfloat16() for _ in range(3))
            y = torch.empty_like(q)
            fn = lambda: lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D,
                                                 y.data_ptr(), None, st.data_ptr(), sp)
            nbytes = 4 * q.numel() * 2
            small = nbytes < 2 * 126e6
            ms = cx.time_kernel(fn, 10 if T <= 8192 else 4, warm=3, flush=small)
            tf = causal_flops(B, H, T, D) / (ms * 1e-3) / 1e12
            out.append({"B": B, "T": T, "ms": round(ms, 4), "tflops": round(tf, 1),
                        "roofline": tensor_roofline(cx, tf, "sdpa_fwd_tc_kernel<128>", ms),
                        "l2": "L2 flushed before every timed launch" if small else "inputs exceed L2"})
            del q, k, v, y
    # 64-wide heads (config 2's head size) at longer sequences: every length runs as CTAs of one query tile, two per SM
    out64 = []
    for B, H64, T in ((8, 12, 2048), (2, 12, 8192), (1, 12, 32768)):
        q, k, v = (torch.randn(B, H64, T, 64, device=dev).div_(8.0).bfloat16() for _ in range(3))
        y = torch.empty_like(q)
        fn = lambda: lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H64, T, 64,
                                             y.data_ptr(), None, st.data_ptr(), sp)
        ms = cx.time_kernel(fn, 10, warm=3, flush=True)
        tf = causal_flops(B, H64, T, 64) / (ms * 1e-3) / 1e12
        out64.append({"B": B, "H": H64, "T": T, "ms": round(ms, 4), "tflops": round(tf, 1),
                      "roofline": tensor_roofline(cx, tf, "sdpa_fwd_tc_kernel<64, one-tile shape>", ms,
                                                  "at this head size a key tile costs the softmax as much as at 128 and the tensor "
                                                  "pipe half: the exponential unit, not the tensor pipe, is the busiest resource"),
                      "l2": "L2 flushed before every timed launch"})
        del q, k, v, y
    if int(st[0].item()):
        raise RuntimeError(f"sweep: kernel status {st[:4].tolist()}")
    return {"workload": f"config5 causal prefill forward, H={H} D={D} bf16", "cases": out,
            "head_size_64": {"workload": "causal forward, 12 heads x 64, bf16", "cases": out64}}


def run_fp32_prefill(cx, B=1, T=PF_T):
    """The headline shape with fp32 tensors (what a default MyCaffe handle holds): the split-operand tensor-core
    forward for 128-wide heads next to the exact fp32 CUDA-core kernel, same inputs."""
    torch, lib, dev, sp = cx.torch, cx.lib, cx.dev, cx.sp
    H, D = PF_H, PF_D
    q, k, v = (torch.randn(B, H, T, D, device=dev).div_(D ** 0.5) for _ in range(3))
    y, y2 = torch.empty_like(q), torch.empty_like(q)
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    nbytes = lib.mca_sdpa_forward_f32_tc_workspace_bytes_d(B, H, T, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    rcs = []
    f_tc = lambda: rcs.append(lib.mca_sdpa_forward_f32_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), 1, B, H, T, D, y.data_ptr(), None, None,
                                                          None, None, ws.data_ptr(), nbytes, st.data_ptr(), 0, sp))
    f_cc = lambda: rcs.append(lib.mca_sdpa_forward_f32_layout(q.data_ptr(), k.data_ptr(), v.data_ptr(), None, 3, None, B, H, T, D,
                                                              y2.data_ptr(), None, None, None, 0, sp))
    ms_tc = cx.time_kernel(f_tc, 4, warm=3)
    ms_cc = cx.time_kernel(f_cc, 2, warm=1)
    if any(rcs) or int(st[0].item()):
        raise RuntimeError(f"fp32 prefill: rc {sorted(set(rcs))}, status {st[:4].tolist()}")
    diff = float((y - y2).abs().max().item())
    scale = float(y2.abs().max().item())
    if not diff <= 2e-5 * scale:
        raise RuntimeError(f"fp32 prefill: tensor-core and CUDA-core outputs differ by {diff} (scale {scale})")
    fl = causal_flops(B, H, T, D)
    tf = fl / (ms_tc * 1e-3) / 1e12
    return {"workload": f"config5 shape causal forward B={B} H={H} D={D} T={T}, fp32 tensors",
            "tensor_cores_ms": round(ms_tc, 3), "tflops": round(tf, 1), "cuda_cores_ms": round(ms_cc, 3),
            "cuda_cores_tflops": round(fl / (ms_cc * 1e-3) / 1e12, 1), "speedup": round(ms_cc / ms_tc, 2),
            "max_abs_diff_over_scale": diff / scale,
            "roofline": tensor_roofline(cx, tf, "split::amax_kernel + split::rows_kernel + sdpa_fwd_tc_kernel<128,split>", ms_tc,
                                        "useful flops of the fp32 problem over the whole call; the kernel executes three fp16 "
                                        "products per contraction, so 1/3 of the bf16 peak is its ceiling")}


def run_backward(cx, B=1, T=PF_T):
    """bf16 fused backward at the long-context shape (delta + dQ + dK/dV kernels per call)."""
    from mycaffe_b200 import function_ids as ids
    torch, lib, dev, sp = cx.torch, cx.lib, cx.dev, cx.sp
    H, D = PF_H, PF_D
    q, k, v, dy = (torch.randn(B, H, T, D, device=dev).div_(D ** 0.25).bfloat16() for _ in range(4))
    y, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse, delta = torch.empty(B, H, T, device=dev), torch.empty(B, H, T, device=dev)
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D, y.data_ptr(),
                                 lse.data_ptr(), st.data_ptr(), sp)
    fn = lambda: lib.mca_sdpa_backward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), dy.data_ptr(), lse.data_ptr(),
                                          delta.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D, dq.data_ptr(), dk.data_ptr(),
                                          dv.data_ptr(), st.data_ptr(), sp)
    ms = cx.time_kernel(fn, 4, warm=2)
    if rc or int(st[0].item()):
        raise RuntimeError(f"backward: rc {rc}, status {st[:4].tolist()}")
    useful = 2.5 * causal_flops(B, H, T, D)
    tf = useful / (ms * 1e-3) / 1e12
    return {"workload": f"config5 shape causal backward B={B} H={H} D={D} T={T} bf16", "ms": round(ms, 3), "tflops": round(tf, 1),
            "flop_count": "2.5 x causal forward (five products: S, dP, dV, dQ, dK)",
            "roofline": tensor_roofline(cx, tf, "bwd_delta_bf16_kernel + sdpa_bwd_dq_tc_kernel<128> + sdpa_bwd_dkdv_tc_kernel<128>", ms,
                                        "useful work over the time of the whole call; the kernels execute seven products for five")}


def run_train(cx, steps=4):
    """Config 2's attention core: 12 layers x (forward + backward), B=8, T=1024, 12 heads x 64, fp32 and bf16.
    A step runs the 12 forwards then the 12 backwards, layers on rotating tensor sets (together above L2)."""
    from mycaffe_b200 import function_ids as ids
    torch, lib, dev, sp, stream = cx.torch, cx.lib, cx.dev, cx.sp, cx.stream
    B, H, T, D, L = 8, 12, 1024, 64, 12
    fwd_flops, bwd_flops = L * causal_flops(B, H, T, D), 2.5 * L * causal_flops(B, H, T, D)
    res = {"workload": f"config2 attention core: {L} layers x (forward + backward), B={B} H={H} D={D} T={T}, causal",
           "flops_per_step": {"forward": fwd_flops, "backward": bwd_flops}}
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    ws_bytes = lib.mca_sdpa_forward_f32_tc_workspace_bytes(B, H, T)
    # fp32: what a default handle runs (forward and backward on the tensor cores with split fp16 operands);
    # fp32_cuda_cores: exact fp32 arithmetic on CUDA cores (MCA_FLAG_EXACT_FP32)
    # fp32_key_mask / fp32_key_mask_cuda_cores: the same shape without the causal mask but with a (B,T) key mask (what
    # MultiheadAttentionLayer passes, MultiheadAttentionLayer.cs:698-702; 30 % of the keys masked), on the tensor cores
    # (packed keep-bits) and on the exact CUDA-core kernels; twice the causal FLOPs
    keymask = (torch.rand(B, T, device=dev) > 0.3).float().contiguous()
    wpr = lib.mca_mask_bits_row_words(T)
    keybits = torch.zeros(B * wpr, dtype=torch.int32, device=dev)
    if lib.mca_mask_pack(keymask.data_ptr(), 2, B, T, keybits.data_ptr(), None, sp):
        raise RuntimeError("mask pack failed")
    for name in ("fp32", "fp32_cuda_cores", "bf16", "fp32_key_mask", "fp32_key_mask_cuda_cores"):
        bf = name == "bf16"
        split_fwd = name in ("fp32", "fp32_key_mask")
        masked = "key_mask" in name
        dt = torch.bfloat16 if bf else torch.float32
        n_sets = 4
        sets = []
        for _ in range(n_sets):
            q, k, v, dy = (torch.randn(B, H, T, D, device=dev).mul_(0.5).to(dt) for _ in range(4))
            sets.append(dict(q=q, k=k, v=v, dy=dy, y=torch.empty_like(q), dq=torch.empty_like(q), dk=torch.empty_like(q),
                             dv=torch.empty_like(q), a=torch.empty(B, H, T, device=dev), b=torch.empty(B, H, T, device=dev),
                             delta=torch.empty(B, H, T, device=dev), yc=torch.empty(B, H, T, D, device=dev) if not bf else None))
            if split_fwd:   # each layer keeps the fp16 halves of its q, k, v from forward to backward
                sets[-1]["ws_t"] = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
                sets[-1]["ws"] = sets[-1]["ws_t"].data_ptr()

        def fwd(s):
            if bf:
                return lib.mca_sdpa_forward_tc(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D,
                                               s["y"].data_ptr(), s["a"].data_ptr(), st.data_ptr(), sp)
            if split_fwd:
                return lib.mca_sdpa_forward_f32_tc_masked(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), 0 if masked else 1, B, H, T, D,
                                                          s["y"].data_ptr(), None, None, s["yc"].data_ptr(), s["a"].data_ptr(), s["ws"], ws_bytes,
                                                          st.data_ptr(), 0, keybits.data_ptr() if masked else None, 2 if masked else 0, sp)
            return lib.mca_sdpa_forward_f32(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), keymask.data_ptr() if masked else None,
                                            2 if masked else 3, None, B, H, T, D,
                                            s["y"].data_ptr(), s["a"].data_ptr(), s["b"].data_ptr(), s["yc"].data_ptr(), sp)

        def bwd(s):
            if bf:
                return lib.mca_sdpa_backward_tc(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), s["y"].data_ptr(), s["dy"].data_ptr(),
                                                s["a"].data_ptr(), s["delta"].data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D,
                                                s["dq"].data_ptr(), s["dk"].data_ptr(), s["dv"].data_ptr(), st.data_ptr(), sp)
            if split_fwd:
                return lib.mca_sdpa_backward_f32_tc_masked(s["dy"].data_ptr(), s["yc"].data_ptr(), s["a"].data_ptr(), s["delta"].data_ptr(),
                                                           0 if masked else 1, B, H, T, D, s["dq"].data_ptr(), s["dk"].data_ptr(),
                                                           s["dv"].data_ptr(), s["ws"], ws_bytes, st.data_ptr(), 0,
                                                           keybits.data_ptr() if masked else None, None, 2 if masked else 0, sp)
            return lib.mca_sdpa_backward_f32(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), s["dy"].data_ptr(), s["yc"].data_ptr(),
                                             keymask.data_ptr() if masked else None, 2 if masked else 3, None, s["a"].data_ptr(),
                                             s["b"].data_ptr(), s["delta"].data_ptr(), B, H, T, D,
                                             s["dq"].data_ptr(), s["dk"].data_ptr(), s["dv"].data_ptr(), sp)

        def step(evs=None):
            if evs:
                evs[0].record(stream)
            for l in range(L):
                rc = fwd(sets[l % n_sets])
                if rc:
                    raise RuntimeError(f"train {name}: forward failed with {rc}")
            if evs:
                evs[1].record(stream)
            for l in reversed(range(L)):
                rc = bwd(sets[l % n_sets])
                if rc:
                    raise RuntimeError(f"train {name}: backward failed with {rc}")
            if evs:
                evs[2].record(stream)

        step(); step()
        torch.cuda.synchronize()
        fms = bms = 0.0
        for _ in range(steps):
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            step(evs)
            torch.cuda.synchronize()
            fms += evs[0].elapsed_time(evs[1]); bms += evs[1].elapsed_time(evs[2])
        fms, bms = fms / steps, bms / steps
        ff, bfl = (2 * fwd_flops, 2 * bwd_flops) if masked else (fwd_flops, bwd_flops)   # no causal half without the causal mask
        tot = (ff + bfl) / ((fms + bms) * 1e-3) / 1e12
        entry = {"ms_per_step": round(fms + bms, 3), "forward_ms": round(fms, 3), "backward_ms": round(bms, 3), "tflops": round(tot, 1),
                 "forward_tflops": round(ff / (fms * 1e-3) / 1e12, 1), "backward_tflops": round(bfl / (bms * 1e-3) / 1e12, 1),
                 "gpu_launches": steps * L * (2 if bf else 2) }
        if bf:
            entry["roofline"] = tensor_roofline(cx, tot, "sdpa_fwd_tc_kernel<64> + backward kernels<64>", (fms + bms) / L,
                                                "useful FLOPs of forward + backward over their summed time, per layer")
        elif split_fwd:
            entry["roofline"] = tensor_roofline(cx, tot, "sdpa_fwd_tc_kernel<64,split> + sdpa_bwd_dkdv/dq_tc_kernel<64,split> (+ pre-passes)",
                                                (fms + bms) / L, "useful FLOPs over the summed time, per layer; every contraction is three "
                                                "fp16 products, so a third of the bf16 peak is this path's ceiling")
        else:
            peak = 148 * 128 * 2 * 1.965e9 / 1e12    # fp32 FMA lanes x 2 flop x max SM clock: no measured figure exists for this pipe
            entry["roofline"] = {"bound": "fp32 FMA issue (CUDA cores)", "kernel": "sdpa_fwd_f32_kernel<64> + sdpa_bwd_*_f32_kernel<64>",
                                 "achieved": round(tot, 2), "peak": round(peak, 1), "unit": "TFLOP/s", "frac": round(tot / peak, 4),
                                 "peak_source": "nominal (148 SMs x 128 lanes x 2 x 1965 MHz)", "kernel_ms": round((fms + bms) / L, 4),
                                 "traffic": None}
        res[name] = entry
        del sets
        torch.cuda.empty_cache()
    if int(st[0].item()):
        raise RuntimeError(f"train: kernel status {st[:4].tolist()}")
    return res


def run_projections(cx):
    """The weight-streaming projections of one llama2-7B decode layer (RMSNorm + q/k/v, Wo + residual, RMSNorm + W1/W3 +
    SwiGLU + W2 + residual) for 1, 16 and 64 sequences, fp32 weights: one sequence and up to eight share a streaming
    pass (`gemv_stream_kernel`); above that the tensor-core kernel (`proj_tc_kernel`) reads the weights once.  Every call
    takes the next of two weight sets (1.6 GB in all), so no weight byte is found in L2."""
    torch, lib, dev = cx.torch, cx.lib, cx.dev
    dim, hidden = DEC_HEADS * DEC_HS, 11008
    sets = 2
    mk = lambda r_, c_: [torch.randn(r_, c_, device=dev) * 0.02 for _ in range(sets)]
    wq, wk, wv, wo = mk(dim, dim), mk(dim, dim), mk(dim, dim), mk(dim, dim)
    w1, w3, w2 = mk(hidden, dim), mk(hidden, dim), mk(dim, hidden)
    rms = torch.ones(dim, device=dev)
    nbytes = (4 * dim * dim + 3 * hidden * dim) * 4
    pk = cx.peaks["hbm_gbs"]
    res = {"workload": f"decode projections of one layer, dim {dim}, hidden {hidden}, fp32 weights ({nbytes >> 20} MB per layer)", "batches": []}
    for Bn in (1, 16, 64):
        x = torch.randn(Bn, dim, device=dev)
        xb = torch.randn(Bn, dim, device=dev)
        qo, ko, vo = (torch.empty(Bn, dim, device=dev) for _ in range(3))
        hbuf = torch.empty(Bn, hidden, device=dev)

        def layer(i):
            rc = lib.mca_decode_qkv_rmsnorm(x.data_ptr(), rms.data_ptr(), 1e-5, wq[i].data_ptr(), wk[i].data_ptr(), wv[i].data_ptr(), 0, Bn, dim,
                                            dim, qo.data_ptr(), ko.data_ptr(), vo.data_ptr(), cx.sp)
            rc |= lib.mca_decode_out_proj(xb.data_ptr(), wo[i].data_ptr(), 0, Bn, dim, x.data_ptr(), cx.sp)
            rc |= lib.mca_decode_ffn(rms.data_ptr(), 1e-5, w1[i].data_ptr(), w2[i].data_ptr(), w3[i].data_ptr(), 0, Bn, dim, hidden,
                                     hbuf.data_ptr(), x.data_ptr(), cx.sp)
            return rc
        entry = {"sequences": Bn}
        for mode, on in (("tensor_core", 1), ("streaming", 0)) if Bn > 8 else (("streaming", 1),):
            lib.mca_proj_tc_enable(on)
            for i in range(3):
                x.normal_()
                if layer(i % sets):
                    raise RuntimeError("projection launch failed")
            iters = 8
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record(cx.stream)
            for i in range(iters):
                layer(i % sets)
            e1.record(cx.stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            entry[mode + "_ms"] = round(ms, 4)
            entry[mode + "_GBps"] = round(nbytes / ms / 1e6, 1)
        lib.mca_proj_tc_enable(1)
        best = "tensor_core" if Bn > 8 else "streaming"
        entry["roofline"] = {"bound": "hbm", "kernel": "proj_tc_kernel<float> + x_pieces_kernel" if Bn > 8 else "gemv_stream_kernel",
                             "achieved": entry[best + "_GBps"], "peak": pk, "unit": "GB/s", "frac": round(entry[best + "_GBps"] / pk, 4),
                             "peak_source": cx.peaks["source"], "kernel_ms": entry[best + "_ms"], "bytes_per_launch": nbytes,
                             "traffic": None, "note": "weight bytes of the layer over the time of its five launches"}
        res["batches"].append(entry)
    st = (C.c_int * 4)()
    lib.mca_proj_tc_status(st)
    res["status"] = list(st)
    if st[0] != 0:
        raise RuntimeError(f"projection kernel reported {list(st)}")
    return res


def run_train_function_ids(cx, steps=4):
    """Config 2's attention core the way the C# layers reach it: ATTN_FWD x 12 then ATTN_BWD x 12 through
    DLL_InvokeFloatEx2 with memory handles (CudaDnn.cs:5673-5701), host wall clock per step.  `as_the_reference_calls`:
    a (T,T) lower-triangular mask handle on every Forward and every call synchronised (attn.cu:601);
    `flag_and_async`: the analytic-mask flag on ATTN_SET and MCA_FN_SET_ASYNC."""
    import numpy as np
    from mycaffe_b200 import CudaDnn, function_ids as ids
    B, T, H, D, L = 8, 1024, 12, 64, 12
    cuda = CudaDnn(cx.local)
    rng = np.random.default_rng(0)
    mask = np.tril(np.ones((T, T), np.float32))
    out = {"workload": f"config2 attention core through function ids 163/164: {L} layers x (forward + backward), B={B} H={H} D={D} T={T}, "
                       "host wall clock", "legs": {}}
    try:
        for dname, dtype in (("fp32", None), ("bf16", ids.MCA_DTYPE_BF16)):
            alloc = cuda.AllocMemoryBf16 if dtype else cuda.AllocMemory
            for leg, flags, use_async in (("as_the_reference_calls", None, False), ("flag_and_async", ids.MCA_FLAG_CAUSAL_IMPLICIT, True)):
                layers, mem = [], []
                for _ in range(L):
                    hC, hA = cuda.CreateCuDNN(), cuda.CreateAttn()
                    cuda.SetAttn(hC, hA, 0, True, B, T, H, D, 0.0, 0, dtype, flags)
                    t = [alloc((0.5 * rng.standard_normal((B, H, T, D))).astype(np.float32)) for _ in range(4)]   # q, k, v, dy
                    o = [alloc(B * H * T * D) for _ in range(4)]                                                # y, dq, dk, dv
                    layers.append((hC, hA, t, o))
                    mem += t + o
                hM = cuda.AllocMemory(mask)
                cuda.SetAsync(use_async)

                def step():
                    for hC, hA, t, o in layers:
                        cuda.AttnScaledDotProductForward(hC, hA, T, t[0], t[1], t[2], hM, o[0], False)
                    for hC, hA, t, o in reversed(layers):
                        cuda.AttnScaledDotProductBackward(hC, hA, t[0], o[1], t[1], o[2], t[2], o[3], 0, o[0], t[3])
                    cuda.SynchronizeDevice()
                for _ in range(2):
                    step()
                t0 = time.perf_counter()
                for _ in range(steps):
                    step()
                ms = (time.perf_counter() - t0) / steps * 1e3
                cuda.SetAsync(False)
                out["legs"][f"{dname}_{leg}"] = {"ms_per_step": round(ms, 3)}
                for h in mem + [hM]:
                    cuda.FreeMemory(h)
                for hC, hA, _, _ in layers:
                    cuda.FreeAttn(hA)
                    cuda.FreeCuDNN(hC)
    finally:
        cuda.Dispose()
    return out


def run_tft(cx):
    """Config 4: TFT interpretable attention, batch 256, 4 heads, d 64, 192 keys; Nq = 24 (how the TFT net runs it)
    and Nq = 192 (explicit q, k, v mode); forward and backward, L2 flushed before every timed launch (75 MB problem)."""
    torch, lib, dev, sp = cx.torch, cx.lib, cx.dev, cx.sp
    B, H, Nk, d = 256, 4, 192, 64
    res = {"workload": f"config4 TFT attention B={B} H={H} Nk={Nk} d={d} fp32, causal-style mask", "modes": []}
    for Nq in (24, 192):
        q = torch.randn(B, H, Nq, d, device=dev)
        k = torch.randn(B, H, Nk, d, device=dev)
        v = torch.randn(B, Nk, d, device=dev)
        i = torch.arange(Nq, device=dev)[:, None]
        j = torch.arange(Nk, device=dev)[None, :]
        mask = ((j - (Nk - Nq)) > i).float().contiguous()
        out, attn = torch.empty(B, Nq, d, device=dev), torch.empty(B, Nq, Nk, device=dev)
        d_out, d_attn = torch.randn_like(out), torch.randn_like(attn)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        f = lambda: lib.mca_tft_attention_forward_f32(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), B, H, Nq, Nk, d,
                                                      out.data_ptr(), attn.data_ptr(), sp)
        b = lambda: lib.mca_tft_attention_backward_f32(q.data_ptr(), k.data_ptr(), v.data_ptr(), mask.data_ptr(), d_out.data_ptr(),
                                                       d_attn.data_ptr(), B, H, Nq, Nk, d, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), sp)
        fms = cx.time_kernel(f, 10, warm=3, flush=True)
        bms = cx.time_kernel(b, 10, warm=3, flush=True)
        fbytes = 4 * (q.numel() + k.numel() + v.numel() + out.numel() + attn.numel())
        bbytes = 4 * (2 * q.numel() + 2 * k.numel() + 2 * v.numel() + out.numel() + attn.numel())
        fflops = 2.0 * B * H * Nq * Nk * d + 2.0 * B * Nq * Nk * d
        # backward: S, dQ, dK per head; dP = dO V^T and dV = (mean P)^T dO are shared by the heads
        bflops = 2.0 * B * Nq * Nk * d * (3 * H + 2)
        pk = cx.peaks["hbm_gbs"]

        def roof(kernel, nbytes, ms):
            return {"bound": "hbm", "kernel": kernel, "achieved": round(nbytes / ms / 1e6, 1), "peak": pk, "unit": "GB/s",
                    "frac": round(nbytes / ms / 1e6 / pk, 4), "peak_source": cx.peaks["source"], "kernel_ms": round(ms, 5),
                    "bytes_per_launch": nbytes, "traffic": None}
        res["modes"].append({"Nq": Nq, "forward_us": round(fms * 1e3, 1), "backward_us": round(bms * 1e3, 1),
                             "forward_GBps": round(fbytes / fms / 1e6, 1), "backward_GBps": round(bbytes / bms / 1e6, 1),
                             "forward_gflops": round(fflops / fms / 1e6, 1), "backward_gflops": round(bflops / bms / 1e6, 1),
                             "roofline": roof("tft_fwd_tiled_kernel", fbytes, fms),
                             "roofline_backward": roof("tft_bwd_tiled_kernel", bbytes, bms)})
    return res


def run_e2e(args, torch, dev, local, rank, world, barrier, B, H, Hl, T, D, q, k, v):
    """The same prefill step from HOST tensors (pinned), copies inside the timed region, three ways:
    the chunked copy/compute pipeline on bf16 host tensors (id 2003; the headline), the same on fp32
    host tensors, and the reference's own call sequence SETMEM x3 -> ATTN_FWD -> GETMEM on handles."""
    from mycaffe_b200 import CudaDnn, function_ids as ids
    n = q.numel()
    steps = max(2, min(args.steps, 5))
    cuda = CudaDnn(local)

    def timed(step):
        step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        barrier()
        dt = (time.perf_counter() - t0) / steps
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt

    def entry(dt, h2d, d2h, path):
        return {"value": round(causal_flops(B, H, T, D) / dt / 1e12, 3), "unit": "TFLOP/s", "ms_per_step": round(dt * 1e3, 3),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps, "path": path}

    # ---- pipelined, bf16 host tensors
    hb = [t_.cpu().pin_memory() for t_ in (q, k, v)]
    yb = torch.empty_like(hb[0]).pin_memory()
    longs = [hb[0].data_ptr(), hb[1].data_ptr(), hb[2].data_ptr(), yb.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, Hl, T, D, 0]

    def step_bf16():
        cuda._invoke(ids.MCA_FN_ATTN_FWD_HOST, None, longs)
        return float(yb.view(-1)[0])

    res = entry(timed(step_bf16), 3 * n * 2, n * 2,
                "MCA_FN_ATTN_FWD_HOST: pinned bf16 host tensors, chunks of (batch, head) pairs, H2D / kernel / D2H "
                "overlapped on three streams, per-rank heads")
    # ---- pipelined, fp32 host tensors
    hf = [t_.float().cpu().pin_memory() for t_ in (q, k, v)]
    yf = torch.empty_like(hf[0]).pin_memory()
    longs_f = [hf[0].data_ptr(), hf[1].data_ptr(), hf[2].data_ptr(), yf.data_ptr(), ids.MCA_DTYPE_F32, 1, B, Hl, T, D, 0]

    def step_f32():
        cuda._invoke(ids.MCA_FN_ATTN_FWD_HOST, None, longs_f)
        return float(yf.view(-1)[0])

    res["host_f32_pipelined"] = entry(timed(step_f32), 3 * n * 4, n * 4,
                                      "MCA_FN_ATTN_FWD_HOST: pinned fp32 host tensors, converted to bf16 on the device")
    if not torch.equal(yf.view(-1)[:4096], yb.float().view(-1)[:4096]):
        raise RuntimeError("fp32-host and bf16-host pipelines disagree")
    # ---- the reference's call sequence on handles
    hA, hC = cuda.CreateAttn(), cuda.CreateCuDNN()
    cuda.SetAttn(hC, hA, local, False, B, T, Hl, D, 0.0, 0, ids.MCA_DTYPE_BF16, ids.MCA_FLAG_CAUSAL_IMPLICIT)
    hs = [cuda.AllocMemoryBf16(n) for _ in range(4)]
    packed = []  # host-side packed SETMEM arrays {handle, count, data...} (CudaDnn.cs SetMemory), pinned
    for h, src in zip(hs[:3], hf):
        buf = torch.empty(n + 2, dtype=torch.float32, pin_memory=True)
        buf[0], buf[1] = float(h), float(n)
        buf[2:] = src.flatten()
        packed.append(buf.numpy())
    out_host = yf.view(-1).numpy()

    def step_handles():
        for h, pk in zip(hs[:3], packed):
            cuda._invoke_raw(ids.CUDA_FN_SETMEM, pk, [h, n])
        cuda.AttnScaledDotProductForward(hC, hA, T, hs[0], hs[1], hs[2], 0, hs[3], False)
        cuda.GetMemoryInto(hs[3], out_host)
        return float(out_host[0])

    res["reference_call_sequence"] = entry(timed(step_handles), 3 * n * 4, n * 4,
                                           "SETMEM x3 (float host arrays, converted to bf16 on the device) -> ATTN_FWD "
                                           "-> GETMEM on handles, blocking copies as the reference issues them")
    for h in hs:
        cuda.FreeMemory(h)
    cuda.Dispose()
    return res


# --------------------------------------------------------------------------------------------- CPU legs

def whole_model_decode(tokens=24, start=200):
    """Token -> logits for a llama2.c-110M-shaped model (dim 768, 12 layers, 12 heads of 64, hidden 2048,
    vocabulary 8000, fp32), one sequence, on the SAME checkpoint file by both sides: TransformerGpu.forward
    (mca_llama_forward replayed from one CUDA graph + the logits copy to the host, as the reference's
    TransformerGpu::forward returns them) and the reference's own TransformerCpu::forward compiled from its source.  Both first
    fill positions 0..start-1, then `tokens` steps are timed; the logits of the last step are compared."""
    import oracle
    import tempfile
    from mycaffe_b200.llama2 import TransformerGpu
    if oracle.ref_lib() is None:
        return {"unavailable": "compiled reference twin not built"}
    dim, hidden, L, H, vocab, S = 768, 2048, 12, 12, 8000, 512
    rng = np.random.default_rng(0)
    g = lambda *sh: (0.04 * rng.standard_normal(sh)).astype(np.float32)
    w = {"rms_att_weight": np.ones((L, dim), np.float32), "rms_ffn_weight": np.ones((L, dim), np.float32),
         "rms_final_weight": np.ones(dim, np.float32), "token_embedding_table": rng.standard_normal((vocab, dim)).astype(np.float32),
         "wq": g(L, dim, dim), "wk": g(L, dim, dim), "wv": g(L, dim, dim), "wo": g(L, dim, dim),
         "w1": g(L, hidden, dim), "w2": g(L, dim, hidden), "w3": g(L, hidden, dim)}
    toks = rng.integers(0, vocab, start + tokens)
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "m110.bin")
        oracle.write_llama_checkpoint(path, dim, hidden, L, H, H, vocab, S, w)
        t = TransformerGpu(0, use_graph=True)
        t.build(path)
        for pos in range(start):
            t.forward(int(toks[pos]), pos)
        t0 = time.perf_counter()
        for pos in range(start, start + tokens):
            got = t.forward(int(toks[pos]), pos)
        gpu_dt = (time.perf_counter() - t0) / tokens
        ref = oracle.RefLlama(path)
        for pos in range(start):
            ref.forward(int(toks[pos]), pos)
        t0 = time.perf_counter()
        for pos in range(start, start + tokens):
            ref.forward(int(toks[pos]), pos)
        cpu_dt = (time.perf_counter() - t0) / tokens
        want = ref.state("logits").copy()
        ref.close()
    err = float(np.abs(got - want).max() / np.abs(want).max())
    params = L * (4 * dim * dim + 3 * dim * hidden) + vocab * dim
    return {"workload": f"llama2.c 110M geometry (dim {dim}, {L} layers, {H} heads, hidden {hidden}, vocab {vocab}), fp32, "
                        f"1 sequence, positions {start}..{start + tokens - 1}, host call to host logits",
            "value": round(1.0 / gpu_dt, 1), "unit": "tok/s", "ms_per_token": round(gpu_dt * 1e3, 4),
            "weight_GBps": round(params * 4 / gpu_dt / 1e9, 1),
            "reference_cpu": {"value": round(1.0 / cpu_dt, 2), "unit": "tok/s", "kind": "reference", "cores": oracle.num_threads(),
                              "sample": f"TransformerCpu::forward on the same checkpoint, {tokens} tokens"},
            "max_rel_err_vs_reference": err}


def cpu_baseline_decode(L=2304, dim=4096, n_heads=32):
    """The reference's own TransformerCpu::forward (llama2_cpu.cpp, compiled from its source) on a
    synthetic one-layer 7B-shape checkpoint at position L-1: rmsnorm, q/k/v/o GEMVs, RoPE, cache append
    and the attention loop (tiny FFN and vocabulary).  Falls back to the restated decode step."""
    import oracle
    import tempfile
    kind, dt, what = "port", None, ""
    if oracle.ref_lib() is not None:
        try:
            hidden, vocab = 8, 8
            rng = np.random.default_rng(0)
            w = {"rms_att_weight": np.ones((1, dim)), "rms_ffn_weight": np.ones((1, dim)), "rms_final_weight": np.ones(dim),
                 "token_embedding_table": rng.standard_normal((vocab, dim)),
                 "wq": 0.02 * rng.standard_normal((1, dim, dim)), "wk": 0.02 * rng.standard_normal((1, dim, dim)),
                 "wv": 0.02 * rng.standard_normal((1, dim, dim)), "wo": 0.02 * rng.standard_normal((1, dim, dim)),
                 "w1": np.zeros((1, hidden, dim)), "w2": np.zeros((1, dim, hidden)), "w3": np.zeros((1, hidden, dim))}
            with tempfile.TemporaryDirectory() as td:
                path = os.path.join(td, "l7b1.bin")
                oracle.write_llama_checkpoint(path, dim, hidden, 1, n_heads, n_heads, vocab, L, w)
                ref = oracle.RefLlama(path)
                ref.state("key_cache")[:] = rng.standard_normal(L * dim).astype(np.float32)
                ref.state("value_cache")[:] = rng.standard_normal(L * dim).astype(np.float32)
                ref.forward(1, L - 1)
                t0 = time.perf_counter()
                reps = 20
                for _ in range(reps):
                    ref.forward(1, L - 1)
                dt = (time.perf_counter() - t0) / reps
                ref.close()
            kind = "reference"
            what = (f"reference TransformerCpu::forward, 1 layer dim={dim} heads={n_heads} at pos={L - 1} "
                    f"(includes the four {dim}x{dim} GEMVs), {reps} reps")
        except Exception as exc:  # keep the bench alive; report the port instead
            what = f"reference twin failed ({exc}); "
    if dt is None:
        rng = np.random.default_rng(0)
        kc = rng.standard_normal((1, L, dim)).astype(np.float32)
        vc = rng.standard_normal((1, L, dim)).astype(np.float32)
        q, k, v = (rng.standard_normal((1, dim)).astype(np.float32) for _ in range(3))
        oracle.llama_decode(q, k, v, kc, vc, [L - 1], n_heads, n_heads)
        t0 = time.perf_counter()
        reps = 20
        for _ in range(reps):
            oracle.llama_decode(q, k, v, kc, vc, [L - 1], n_heads, n_heads)
        dt = (time.perf_counter() - t0) / reps
        what += f"restated decode step, 1 sequence L={L}, {reps} reps"
    return {"value": round(1.0 / (dt * DEC_LAYERS), 3), "unit": "tok/s", "cores": oracle.num_threads(), "kind": kind,
            "sample": what + f"; tok/s = 1 / ({DEC_LAYERS} layers x {dt * 1e3:.2f} ms), batch 1 as the reference runs it"}


def run_reference(args):
    """CPU reference arm: the reference's attention math on the host cores, rank 0 only.  Each step is a bounded
    sample of the headline workload (256 strided query rows of the 16 heads of one batch item, T = 32768), so
    that warm-up + steps end within a couple of minutes at any launcher setting."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    import oracle
    oracle.build()
    cores = oracle.set_num_threads()    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers
    T, D, H = args.seq_len, PF_D, PF_H
    rng = np.random.default_rng(0)
    q, k, v = ((rng.standard_normal((1, H, T, D), dtype=np.float32) / np.float32(np.sqrt(D))) for _ in range(3))
    q_step = max(1, T // 256)
    rows = np.arange(q_step // 2, T, q_step)
    flops = 4.0 * H * D * float(np.sum(rows + 1))

    def step():
        t0 = time.perf_counter()
        oracle.sdpa_forward_rows(q, k, v, None, 3, q_step // 2, q_step)
        return time.perf_counter() - t0

    for _ in range(min(args.warmup, 3)):
        step()
    budget_s, times = 100.0, []
    t_start = time.perf_counter()
    for _ in range(args.steps):
        times.append(step())
        if time.perf_counter() - t_start > budget_s:   # slow hosts: keep what was measured
            break
    dt = float(np.mean(times))
    val = flops / dt / 1e12
    base = {"value": round(val, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"per step {len(rows)} strided query rows x {H} heads of one batch item of the T={T} causal problem "
                      f"({flops / 1e9:.1f} GFLOP causal, {dt:.2f} s); {len(times)} of {args.steps} steps run; "
                      "full-problem time extrapolated from this rate"}
    dec = cpu_baseline_decode()
    world = int(os.environ.get("WORLD_SIZE", 1))
    line = {"impl": "reference", "metric": "attn_prefill_tflops", "value": round(val, 5), "unit": "TFLOP/s",
            "n_gpus": world, "steps": len(times), "warmup": min(args.warmup, 3), "ms_per_step": round(dt * 1e3, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"config5 causal prefill B={args.batch} H={PF_H} D={PF_D} T={args.seq_len}: reference math "
                                   f"(restated attn.cu:518-602) on {cores} host cores, each step a bounded sample of the query rows"},
            "cpu_baseline": base,
            "e2e": {"value": round(val, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "decode": {"metric": "decode_tokens_per_s", "value": dec["value"], "unit": "tok/s", "cpu_baseline": dec}}
    print(json.dumps(line), flush=True)


def run_profile_case(case):
    """Small stand-alone cases for `ncu` captures (a few launches, inputs above L2 where DRAM matters):
    `prefill-small` = config-5 shape at T = 8192, B = 1; `prefill-full` = the bench workload itself, two
    launches (single-pass metrics only); `bwd-small` = bf16 backward at the prefill-small shape;
    `decode-small` = config-3 shape, 16 sequences of 4096 keys; `gemv-small` = the decode projections at
    dim 4096 for 1 and 8 sequences plus the feed-forward half and the classifier for one (also prints their
    CUDA-event bandwidth); `proj-batch` = the same projections for 16 and 64 sequences, tensor-core kernel and
    streaming passes side by side; `norm-small` = the LayerNorm / RMSNorm layer kernels on a 268 MB tensor;
    `llama-step` = the whole decode step of an 8-layer llama2-7B-shaped model, eager and from a CUDA graph
    (a timing case, about 15 GB on the device: not for ncu); `tft`, `train`, `sweep`, `backward` = the N = 1 legs of
    the benchmark on their own."""
    import torch
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    if case in ("tft", "train", "sweep", "backward", "projections", "fp32-prefill", "train-ids"):
        # the N = 1 legs of the benchmark on their own (same code, same JSON fragment)
        cx = Ctx(argparse.Namespace())
        print(json.dumps({"case": case, case: {"tft": run_tft, "train": run_train, "sweep": run_sweep, "backward": run_backward, "projections": run_projections,
                                                "fp32-prefill": run_fp32_prefill, "train-ids": run_train_function_ids}[case](cx)}))
        return
    if case == "gemv-small":
        dim = DEC_HEADS * DEC_HS
        ws = [torch.randn(dim, dim, device=dev) * 0.02 for _ in range(4)]   # wq, wk, wv, wo: 67 MB each
        rms = torch.ones(dim, device=dev)
        res = {"case": case}
        for Bn in (1, 8):
            x = torch.randn(Bn, dim, device=dev)
            qo, ko, vo = (torch.empty(Bn, dim, device=dev) for _ in range(3))
            def qkv():
                return lib.mca_decode_qkv_rmsnorm(x.data_ptr(), rms.data_ptr(), 1e-5, ws[0].data_ptr(), ws[1].data_ptr(),
                                                  ws[2].data_ptr(), 0, Bn, dim, dim, qo.data_ptr(), ko.data_ptr(), vo.data_ptr(), None)
            def outp():
                return lib.mca_decode_out_proj(qo.data_ptr(), ws[3].data_ptr(), 0, Bn, dim, x.data_ptr(), None)
            for name, fn, nbytes in (("qkv", qkv, 3 * dim * dim * 4), ("out", outp, dim * dim * 4)):
                for _ in range(3):
                    rc = fn()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(20):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / 20
                res[f"{name}_B{Bn}"] = {"rc": rc, "ms": round(ms, 4), "weight_GBps": round(nbytes / ms / 1e6, 1)}
        # feed-forward half (RMSNorm + W1/W3 + SwiGLU, W2 + residual) and the classifier, one sequence
        hidden, vocab = 11008, 32000
        del ws
        w1, w3 = (torch.randn(hidden, dim, device=dev) * 0.02 for _ in range(2))
        w2 = torch.randn(dim, hidden, device=dev) * 0.02
        wc = torch.randn(vocab, dim, device=dev) * 0.02
        x = torch.randn(1, dim, device=dev)
        hbuf, logits = torch.empty(1, hidden, device=dev), torch.empty(1, vocab, device=dev)
        def ffn():
            return lib.mca_decode_ffn(rms.data_ptr(), 1e-5, w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), 0, 1, dim, hidden,
                                      hbuf.data_ptr(), x.data_ptr(), None)
        def cls():
            return lib.mca_decode_logits(x.data_ptr(), rms.data_ptr(), 1e-5, wc.data_ptr(), 0, 1, dim, vocab, logits.data_ptr(), None)
        for name, fn, nbytes in (("ffn", ffn, 3 * hidden * dim * 4), ("logits", cls, vocab * dim * 4)):
            for _ in range(3):
                rc = fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(20):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 20
            res[f"{name}_B1"] = {"rc": rc, "ms": round(ms, 4), "weight_GBps": round(nbytes / ms / 1e6, 1)}
        print(json.dumps(res))
        return
    if case == "proj-small":
        # ncu-sized: the q/k/v projection (three 67 MB fp32 matrices, above L2) and the gated feed-forward pair for 64
        # sequences, three launches each
        dim, hidden, Bn = DEC_HEADS * DEC_HS, 11008, 64
        rms = torch.ones(dim, device=dev)
        wq, wk, wv = (torch.randn(dim, dim, device=dev) * 0.02 for _ in range(3))
        w1, w3 = (torch.randn(hidden, dim, device=dev) * 0.02 for _ in range(2))
        w2 = torch.randn(dim, hidden, device=dev) * 0.02
        x = torch.randn(Bn, dim, device=dev)
        qo, ko, vo = (torch.empty(Bn, dim, device=dev) for _ in range(3))
        hbuf = torch.empty(Bn, hidden, device=dev)
        res = {"case": case}
        for name, fn, nbytes in (
                ("qkv", lambda: lib.mca_decode_qkv_rmsnorm(x.data_ptr(), rms.data_ptr(), 1e-5, wq.data_ptr(), wk.data_ptr(), wv.data_ptr(), 0, Bn,
                                                           dim, dim, qo.data_ptr(), ko.data_ptr(), vo.data_ptr(), None), 3 * dim * dim * 4),
                ("ffn", lambda: lib.mca_decode_ffn(rms.data_ptr(), 1e-5, w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), 0, Bn, dim, hidden,
                                                   hbuf.data_ptr(), x.data_ptr(), None), 3 * hidden * dim * 4)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            rc = fn()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(2):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 2
            res[name] = {"rc": rc, "ms": round(ms, 4), "weight_GBps": round(nbytes / ms / 1e6, 1)}
        print(json.dumps(res))
        return
    if case == "proj-batch":
        # decode projections of a 7B-shaped layer for 16 and 64 sequences: the tensor-core kernel against the streaming
        # passes it replaces; every call takes the next of several weight sets, so no weight byte is found in L2
        dim, hidden, vocab = DEC_HEADS * DEC_HS, 11008, 32000
        res = {"case": case, "peak_GBps": measured_peaks()["hbm_gbs"]}
        rms = torch.ones(dim, device=dev)
        for wname, wdt, esz in (("fp32", torch.float32, 4), ("bf16", torch.bfloat16, 2)):
            bf = int(wdt == torch.bfloat16)
            sets = 3
            mk = lambda r_, c_: [(torch.randn(r_, c_, device=dev) * 0.02).to(wdt) for _ in range(sets)]
            wq, wk, wv, wo = mk(dim, dim), mk(dim, dim), mk(dim, dim), mk(dim, dim)
            w1, w3, w2, wc = mk(hidden, dim), mk(hidden, dim), mk(dim, hidden), mk(vocab, dim)
            for Bn in (16, 64):
                x = torch.randn(Bn, dim, device=dev)
                qo, ko, vo = (torch.empty(Bn, dim, device=dev) for _ in range(3))
                hbuf, logits = torch.empty(Bn, hidden, device=dev), torch.empty(Bn, vocab, device=dev)
                calls = {
                    "qkv": (lambda i: lib.mca_decode_qkv_rmsnorm(x.data_ptr(), rms.data_ptr(), 1e-5, wq[i].data_ptr(), wk[i].data_ptr(),
                                                                 wv[i].data_ptr(), bf, Bn, dim, dim, qo.data_ptr(), ko.data_ptr(),
                                                                 vo.data_ptr(), None), 3 * dim * dim * esz),
                    "out": (lambda i: lib.mca_decode_out_proj(qo.data_ptr(), wo[i].data_ptr(), bf, Bn, dim, x.data_ptr(), None), dim * dim * esz),
                    "ffn": (lambda i: lib.mca_decode_ffn(rms.data_ptr(), 1e-5, w1[i].data_ptr(), w2[i].data_ptr(), w3[i].data_ptr(), bf, Bn, dim,
                                                         hidden, hbuf.data_ptr(), x.data_ptr(), None), 3 * hidden * dim * esz),
                    "logits": (lambda i: lib.mca_decode_logits(x.data_ptr(), rms.data_ptr(), 1e-5, wc[i].data_ptr(), bf, Bn, dim, vocab,
                                                               logits.data_ptr(), None), vocab * dim * esz),
                }
                for name, (fn, nbytes) in calls.items():
                    entry = {}
                    for mode, on in (("tensor_core", 1), ("streaming", 0)):
                        lib.mca_proj_tc_enable(on)
                        for i in range(3):
                            x.normal_()
                            rc = fn(i % sets)
                        iters = 9
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        torch.cuda.synchronize()
                        e0.record()
                        for i in range(iters):
                            fn(i % sets)
                        e1.record()
                        torch.cuda.synchronize()
                        ms = e0.elapsed_time(e1) / iters
                        entry[mode] = {"rc": rc, "ms": round(ms, 4), "weight_GBps": round(nbytes / ms / 1e6, 1)}
                    lib.mca_proj_tc_enable(1)
                    entry["frac_of_copy_bandwidth"] = round(entry["tensor_core"]["weight_GBps"] / res["peak_GBps"], 3)
                    res[f"{wname}_{name}_B{Bn}"] = entry
            del wq, wk, wv, wo, w1, w3, w2, wc
        import ctypes as C
        st = (C.c_int * 4)()
        lib.mca_proj_tc_status(st)
        res["status"] = list(st)
        print(json.dumps(res))
        return
    if case == "norm-small":
        # LayerNorm / RMSNorm layer kernels on a (16384, 4096) tensor (268 MB each way, above L2)
        rows, inner = 16384, 4096
        x, dy = torch.randn(rows, inner, device=dev), torch.randn(rows, inner, device=dev)
        y, dx = torch.empty_like(x), torch.empty_like(x)
        w, dw = torch.ones(inner, device=dev), torch.empty(inner, device=dev)
        stat = torch.empty(rows, device=dev)
        scratch = torch.empty(lib.mca_rmsnorm_backward_scratch_floats(inner), device=dev)
        calls = {
            "layernorm_fwd": (lambda: lib.mca_layernorm_forward_f32(x.data_ptr(), y.data_ptr(), stat.data_ptr(), rows, inner, 1e-5, None), 2),
            "layernorm_bwd": (lambda: lib.mca_layernorm_backward_f32(y.data_ptr(), dy.data_ptr(), stat.data_ptr(), dx.data_ptr(), rows, inner, 1e-5, None), 3),
            "rmsnorm_fwd": (lambda: lib.mca_rmsnorm_forward_f32(x.data_ptr(), w.data_ptr(), y.data_ptr(), stat.data_ptr(), rows, inner, 1e-5, None), 2),
            "rmsnorm_bwd": (lambda: lib.mca_rmsnorm_backward_f32(x.data_ptr(), w.data_ptr(), dy.data_ptr(), stat.data_ptr(), dx.data_ptr(),
                                                                 dw.data_ptr(), scratch.data_ptr(), scratch.numel(), rows, inner, None), 3),
        }
        res = {"case": case, "rows": rows, "inner": inner}
        for name, (fn, tensors) in calls.items():
            for _ in range(3):
                rc = fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 10
            res[name] = {"rc": rc, "ms": round(ms, 4), "GBps": round(tensors * rows * inner * 4 / ms / 1e6, 1)}
        print(json.dumps(res))
        return
    if case == "llama-step":
        # whole-transformer decode step, llama2-7B geometry cut to 8 layers, every sequence at position 2047;
        # 1, 16 and 64 sequences (above eight the projections run on the tensor cores)
        import ctypes as C
        from mycaffe_b200 import llama2 as M
        cfg = dict(dim=4096, hidden_dim=11008, n_layers=8, n_heads=32, n_kv_heads=32, vocab_size=32000, seq_len=2048)
        res = {"case": case, "config": cfg}
        for bf16 in (False, True):
            wdt = torch.bfloat16 if bf16 else torch.float32
            L, dim, hidden, vocab, S = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"], cfg["seq_len"]
            mk = lambda *sh, dt=torch.float32: (torch.randn(*sh, device=dev) * 0.02).to(dt)
            w = {"token_embedding_table": mk(vocab, dim), "rms_att_weight": torch.ones(L, dim, device=dev),
                 "rms_ffn_weight": torch.ones(L, dim, device=dev), "rms_final_weight": torch.ones(dim, device=dev),
                 "wq": mk(L, dim, dim, dt=wdt), "wk": mk(L, dim, dim, dt=wdt), "wv": mk(L, dim, dim, dt=wdt),
                 "wo": mk(L, dim, dim, dt=wdt), "w1": mk(L, hidden, dim, dt=wdt), "w2": mk(L, dim, hidden, dt=wdt),
                 "w3": mk(L, hidden, dim, dt=wdt), "wcls": mk(vocab, dim, dt=wdt)}
            fr, fi = np.empty((S, 64), np.float32), np.empty((S, 64), np.float32)
            fp = C.POINTER(C.c_float)
            lib.mca_rope_tables_host(S, 128, 10000.0, fr.ctypes.data_as(fp), fi.ctypes.data_as(fp))
            frd, fid = torch.from_numpy(fr).to(dev), torch.from_numpy(fi).to(dev)
            cfg_c = M.McaLlamaConfig(**cfg)
            names = ("token_embedding_table", "rms_att_weight", "rms_ffn_weight", "rms_final_weight", "wq", "wk", "wv", "wo",
                     "w1", "w2", "w3", "wcls")
            w_c = M.McaLlamaWeights(*[w[n].data_ptr() for n in names], int(bf16))
            sz = 2 if bf16 else 4
            for Bn in (1, 16, 64):
                kc, vc = (torch.empty(L, Bn, S, dim, device=dev, dtype=wdt).normal_() for _ in range(2))
                need = lib.mca_llama_workspace_floats(C.byref(cfg_c), Bn, S)
                ws_, logits = torch.empty(need, device=dev), torch.empty(Bn, vocab, device=dev)
                tok = torch.zeros(Bn, dtype=torch.int32, device=dev)
                pos = torch.full((Bn,), 2047, dtype=torch.int32, device=dev)
                s_c = M.McaLlamaState(kc.data_ptr(), vc.data_ptr(), int(bf16), frd.data_ptr(), fid.data_ptr(), ws_.data_ptr(), need)

                def step(stream=None):
                    st = stream if stream is not None else torch.cuda.current_stream()
                    return lib.mca_llama_forward(C.byref(cfg_c), C.byref(w_c), C.byref(s_c), tok.data_ptr(), pos.data_ptr(), Bn, 2048,
                                                 logits.data_ptr(), st.cuda_stream)
                for _ in range(3):
                    rc = step()
                side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    graph.capture_begin()
                    step(side)
                    graph.capture_end()
                torch.cuda.current_stream().wait_stream(side)
                out = {}
                for name, fn in (("eager", step), ("graph", graph.replay)):
                    fn()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    for _ in range(10):
                        fn()
                    e1.record()
                    torch.cuda.synchronize()
                    out[name + "_ms"] = round(e0.elapsed_time(e1) / 10, 4)
                nbytes = (L * (4 * dim * dim + 3 * dim * hidden) + vocab * dim) * sz + Bn * L * 2 * 2048 * dim * sz
                out.update({"rc": rc, "bytes": nbytes, "GBps_graph": round(nbytes / out["graph_ms"] / 1e6, 1),
                            "tokens_per_s_8_layers": round(Bn / out["graph_ms"] * 1e3, 1)})
                if Bn > 8:   # the same step with the streaming passes instead of the tensor-core projections
                    lib.mca_proj_tc_enable(0)
                    step()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    e0.record()
                    for _ in range(5):
                        step()
                    e1.record()
                    torch.cuda.synchronize()
                    lib.mca_proj_tc_enable(1)
                    out["eager_ms_streaming_projections"] = round(e0.elapsed_time(e1) / 5, 4)
                res[("bf16" if bf16 else "f32") + f"_B{Bn}"] = out
                del kc, vc, graph, ws_
                torch.cuda.empty_cache()
            del w
            torch.cuda.empty_cache()
        print(json.dumps(res))
        return
    if case in ("prefill-small", "prefill-full", "bwd-small"):
        B, H, T, D = (PF_B, PF_H, PF_T, PF_D) if case == "prefill-full" else (1, PF_H, 8192, PF_D)
        if case == "bwd-small":
            q, k, v, dy = (torch.randn(B, H, T, D, device=dev).div_(D ** 0.25).bfloat16() for _ in range(4))
            y, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
            lse, delta = torch.empty(B, H, T, device=dev), torch.empty(B, H, T, device=dev)
            st = torch.zeros(8, dtype=torch.int32, device=dev)
            lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D, y.data_ptr(),
                                    lse.data_ptr(), st.data_ptr(), None)
            for _ in range(2):
                rc = lib.mca_sdpa_backward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), y.data_ptr(), dy.data_ptr(),
                                              lse.data_ptr(), delta.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D,
                                              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), st.data_ptr(), None)
            torch.cuda.synchronize()
            print(json.dumps({"case": case, "rc": rc, "status": st[:4].tolist(),
                              "useful_flops": 2.5 * causal_flops(B, H, T, D)}))
            return
        q, k, v = (torch.randn(B, H, T, D, device=dev).div_(D ** 0.5).bfloat16() for _ in range(3))
        y = torch.empty_like(q)
        st = torch.zeros(8, dtype=torch.int32, device=dev)
        if case == "prefill-small":
            # the small case stands in for the headline launch: keep the two-tile CTA shape the headline runs in (at this
            # length the launcher would choose the one-tile shape, which `--case sweep` times)
            lib.mca_tc_narrow_len(0)
        for _ in range(2 if case == "prefill-full" else 3):
            rc = lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, H, T, D,
                                         y.data_ptr(), None, st.data_ptr(), None)
        torch.cuda.synchronize()
        print(json.dumps({"case": case, "rc": rc, "status": st[:4].tolist(), "causal_flops": causal_flops(B, H, T, D),
                          "algorithmic_bytes": 4 * q.numel() * 2}))
    else:
        Bd, nh, hs, S = 16, DEC_HEADS, DEC_HS, DEC_SEQ
        kv = nh * hs
        kc, vc = torch.randn(Bd, S, kv, device=dev), torch.randn(Bd, S, kv, device=dev)
        qn, kn, vn = (torch.randn(Bd, kv, device=dev) for _ in range(3))
        pos = torch.full((Bd,), S - 1, dtype=torch.int32, device=dev)
        out = torch.empty(Bd, kv, device=dev)
        sl, ns, need = C.c_int(), C.c_int(), C.c_int64()
        lib.mca_decode_plan(Bd, nh, nh, hs, S, C.byref(sl), C.byref(ns), C.byref(need))
        scratch = torch.empty(need.value, device=dev)
        fr, fi = torch.ones(S, hs // 2, device=dev), torch.zeros(S, hs // 2, device=dev)
        for _ in range(3):
            rc = lib.mca_decode_attention(qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), kc.data_ptr(), vc.data_ptr(), 0,
                                          S * kv, pos.data_ptr(), Bd, nh, nh, hs, S, S, fr.data_ptr(), fi.data_ptr(),
                                          scratch.data_ptr(), scratch.numel(), out.data_ptr(), None)
        torch.cuda.synchronize()
        print(json.dumps({"case": case, "rc": rc, "split_len": sl.value, "nsplit": ns.value,
                          "bytes_per_launch": decode_bytes([S] * Bd, kv, kv, 4)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=PF_B)
    ap.add_argument("--seq-len", type=int, default=PF_T)
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false",
                    help="skip the whole-model CPU comparison (the parity pass and its CPU baseline always run)")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="one GPU: skip the other configurations (train, sweep, backward, decode variants, tft)")
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="multi-GPU: exchange the head outputs with a NCCL all-gather instead of the kernel's peer stores")
    ap.add_argument("--case", default=None, choices=["prefill-small", "prefill-full", "bwd-small", "decode-small", "gemv-small", "proj-batch", "proj-small", "norm-small", "llama-step", "projections",
                                                     "tft", "train", "sweep", "backward", "fp32-prefill", "train-ids"],
                    help="run one small case a few times and exit (for ncu captures)")
    args = ap.parse_args()
    if args.case:
        return run_profile_case(args.case)
    args.warmup = max(args.warmup, 3)
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    run_ours(args)


if __name__ == "__main__":
    main()
