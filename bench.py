#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline metric: causal prefill attention throughput (TFLOP/s, algorithmic causal FLOPs) on the
long-context shape 16 heads x 128, bf16, T = 32768 (heads partitioned over N GPUs with an NCCL
all-gather of the head outputs).  The same JSON line carries the decode metric (tokens/s of the
llama2-7B-shape KV-cache attention, batch 64, cache lengths uniform in [512, 4096]) under
"decode".  Inputs are seeded synthetic tensors of those shapes.

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

def run_ours(args):
    import torch
    import torch.distributed as dist
    from mycaffe_b200 import CudaDnn, _lib, function_ids as ids, head_shard

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    peaks = measured_peaks()
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ----------------------------------------------------------------- prefill (headline)
    B, H, D, T = args.batch, PF_H, PF_D, args.seq_len
    h_lo, h_hi = head_shard.head_range(rank, world, H)
    Hl = h_hi - h_lo
    gen = torch.Generator(device=dev)
    q = torch.empty(B, Hl, T, D, device=dev, dtype=torch.bfloat16)
    k, v = torch.empty_like(q), torch.empty_like(q)
    for hl in range(Hl):  # per-head seeds: the same global problem for every N
        gen.manual_seed(1000 + h_lo + hl)
        for t_ in (q, k, v):
            t_[:, hl] = (torch.randn(B, T, D, device=dev, generator=gen) / D ** 0.5).to(torch.bfloat16)
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
        # the buffers every rank filled must equal what a NCCL all-gather of the same head outputs gives
        rc = lib.mca_sdpa_forward_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), ids.MCA_DTYPE_BF16, 1, B, Hl, T, D,
                                     y.data_ptr(), None, status.data_ptr(), sp)
        ref = head_shard.gather_heads(y, out=y_all)
        torch.cuda.synchronize()
        if rc or not torch.equal(ref, peer_out.tensor):
            raise RuntimeError("peer-store exchange disagrees with the NCCL all-gather")
        del ref
        # Both exchanges are correct; time two steps of each (max over ranks) and keep the faster one for this size.
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
            tt = torch.tensor([t0.elapsed_time(t1) / 2], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            trial[name] = float(tt.item())
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
    total_ms = ev[0].elapsed_time(ev[-1])
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in kern_ev]))
    if world > 1:
        tt = torch.tensor([total_ms, kern_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        total_ms, kern_ms = tt.tolist()
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
                "traffic_source": "ncu capture of the full-size launch (profiles/sdpa_fwd_tc_kernel_prefill.md)",
                "flops_per_launch": flops_launch, "flop_count": "causal 4*B*H*D*T*(T+1)/2"}

    # ----------------------------------------------------------------- decode (secondary metric, rank-local heads)
    decode = run_decode(args, lib, torch, dev, sp, stream, rank, world, barrier, peaks)

    # ----------------------------------------------------------------- end to end through the dispatch ABI (host buffers)
    e2e = run_e2e(args, torch, dev, local, rank, world, barrier, B, H, Hl, T, D, q, k, v)

    if rank == 0:
        line = {
            "metric": "attn_prefill_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"config5 causal prefill B={B} H={H} D={D} T={T} bf16, heads partitioned over {world} GPU(s)"
                                   + (f"; exchange of head outputs: {exchange}" if world > 1 else ""),
                       "l2": "inputs (Q,K,V,O %.0f MB per rank) exceed the 126 MB L2" % (4 * q.numel() * 2 / 1e6),
                       "parallelism": f"heads/{world}"},
            "gpu_launches": args.steps, "clocks": clocks, "roofline": roofline, "e2e": e2e, "decode": decode,
        }
        if args.cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_prefill(T, D, H)
            line["decode"]["cpu_baseline"] = cpu_baseline_decode()
            try:
                line["decode"]["whole_model"] = whole_model_decode()
            except Exception as exc:   # an extra; never the reason the bench line is lost
                line["decode"]["whole_model"] = {"unavailable": repr(exc)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decode(args, lib, torch, dev, sp, stream, rank, world, barrier, peaks):
    """llama2-7B-shape decode attention: one new token for 64 sequences, one launch pair per layer."""
    from mycaffe_b200 import head_shard
    lo, hi = head_shard.head_range(rank, world, DEC_HEADS)
    heads = hi - lo
    kv_dim = heads * DEC_HS
    dim = heads * DEC_HS
    rng = np.random.default_rng(0)
    lengths = rng.integers(DEC_LMIN, DEC_LMAX + 1, DEC_B)
    pos = torch.tensor(lengths - 1, dtype=torch.int32, device=dev)
    max_len = int(lengths.max())
    caches = []
    for _ in range(DEC_BUFFERS):  # distinct layer caches, each far larger than L2, rotated
        caches.append((torch.randn(DEC_B, DEC_SEQ, kv_dim, device=dev), torch.randn(DEC_B, DEC_SEQ, kv_dim, device=dev)))
    qn = torch.randn(DEC_B, dim, device=dev)
    kn = torch.randn(DEC_B, kv_dim, device=dev)
    vn = torch.randn(DEC_B, kv_dim, device=dev)
    out = torch.empty(DEC_B, dim, device=dev)
    out_all = torch.empty(world, DEC_B, dim, device=dev) if world > 1 else None
    sl, ns, need = C.c_int(), C.c_int(), C.c_int64()
    lib.mca_decode_plan(DEC_B, heads, heads, DEC_HS, max_len, C.byref(sl), C.byref(ns), C.byref(need))
    scratch = torch.empty(max(1, need.value), device=dev)
    fr = np.empty((DEC_SEQ, DEC_HS // 2), np.float32)
    fi = np.empty_like(fr)
    fp = C.POINTER(C.c_float)
    lib.mca_rope_tables_host(DEC_SEQ, DEC_HS, 10000.0, fr.ctypes.data_as(fp), fi.ctypes.data_as(fp))
    frd, fid = torch.from_numpy(fr).to(dev), torch.from_numpy(fi).to(dev)

    def layer(i):
        kc, vc = caches[i % DEC_BUFFERS]
        rc = lib.mca_decode_attention(qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), kc.data_ptr(), vc.data_ptr(), 0,
                                      DEC_SEQ * kv_dim, pos.data_ptr(), DEC_B, heads, heads, DEC_HS, DEC_SEQ, max_len,
                                      frd.data_ptr(), fid.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                      out.data_ptr(), sp)
        if rc:
            raise RuntimeError(f"mca_decode_attention failed with {rc}")
        if world > 1:  # the head outputs of every rank, as the Wo projection of the next step needs them
            head_shard.gather_decode_outputs(out, out=out_all)

    steps = max(3, min(args.steps, 10))
    for i in range(3 * DEC_BUFFERS):
        layer(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for s in range(steps):
        for i in range(DEC_LAYERS):
            layer(i)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / steps
    layer_ms = ms_step / DEC_LAYERS
    bytes_layer = decode_bytes(lengths, kv_dim, dim, 4)
    gbs = bytes_layer / (layer_ms * 1e-3) / 1e9
    return {"metric": "decode_tokens_per_s", "value": round(DEC_B / (ms_step * 1e-3), 1), "unit": "tok/s",
            "ms_per_step": round(ms_step, 4), "steps": steps, "dtype": "f32",
            "config": {"workload": f"config3 decode attention batch={DEC_B} heads={DEC_HEADS} (x{DEC_HS}) over {world} GPU(s), "
                                   f"cache lengths U[{DEC_LMIN},{DEC_LMAX}] (mean {lengths.mean():.0f}), fp32 cache, "
                                   f"{DEC_LAYERS} layer-steps per token rotating {DEC_BUFFERS} distinct layer caches (each > L2)",
                       "split_len": sl.value, "nsplit": ns.value},
            "gpu_launches": steps * DEC_LAYERS * (2 if ns.value > 1 else 1),
            "roofline": {"bound": "hbm", "kernel": "decode_split_kernel<float,128,1>", "achieved": round(gbs, 1),
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                         "peak_source": peaks["source"], "bytes_per_launch": bytes_layer,
                         # ncu on the 16-sequence case reads 1.0016 x the algorithmic bytes; traffic grows with the keys read
                         "traffic": int(DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_layer),
                         "traffic_source": "ncu capture of `--case decode-small`, scaled by bytes (profiles/decode_split_kernel.md)"}}


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

def cpu_baseline_prefill(T, D, H, q_step=4, heads=16):
    """Restated reference math (oracle port), OpenMP over all host cores, on a bounded sample:
    query rows q_step//2::q_step of `heads` heads; throughput is causal FLOPs of those rows / time."""
    import oracle
    rng = np.random.default_rng(0)
    q, k, v = ((rng.standard_normal((1, heads, T, D)) / np.sqrt(D)).astype(np.float32) for _ in range(3))
    rows = np.arange(q_step // 2, T, q_step)
    t0 = time.perf_counter()
    oracle.sdpa_forward_rows(q, k, v, None, 3, q_step // 2, q_step)
    dt = time.perf_counter() - t0
    flops = 4.0 * heads * D * float(np.sum(rows + 1))
    return {"value": round(flops / dt / 1e12, 5), "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{len(rows)} strided query rows x {heads} heads of the T={T} causal problem "
                      f"({flops / 1e9:.1f} GFLOP, {dt:.1f} s); full-problem time extrapolated from this rate"}


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
    """CPU reference arm: rank 0 only."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    import oracle
    oracle.build()
    vals = []
    for _ in range(args.warmup):
        cpu_baseline_prefill(args.seq_len, PF_D, PF_H, q_step=32, heads=16)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        vals.append(cpu_baseline_prefill(args.seq_len, PF_D, PF_H, q_step=32, heads=16))
    dt = time.perf_counter() - t0
    v = float(np.mean([x["value"] for x in vals]))
    base = dict(vals[-1])
    base["value"] = round(v, 5)
    dec = cpu_baseline_decode()
    world = int(os.environ.get("WORLD_SIZE", 1))
    line = {"impl": "reference", "metric": "attn_prefill_tflops", "value": round(v, 5), "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"config5 causal prefill B={args.batch} H={PF_H} D={PF_D} T={args.seq_len}: reference math "
                                   "on the host cores, each step a bounded sample of the query rows"},
            "cpu_baseline": base,
            "e2e": {"value": round(v, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "decode": {"metric": "decode_tokens_per_s", "value": dec["value"], "unit": "tok/s", "cpu_baseline": dec}}
    print(json.dumps(line), flush=True)


def run_profile_case(case):
    """Small stand-alone cases for `ncu` captures (a few launches, inputs above L2 where DRAM matters):
    `prefill-small` = config-5 shape at T = 8192, B = 1; `prefill-full` = the bench workload itself, two
    launches (single-pass metrics only); `bwd-small` = bf16 backward at the prefill-small shape;
    `decode-small` = config-3 shape, 16 sequences of 4096 keys; `gemv-small` = the decode projections at
    dim 4096 for 1 and 8 sequences plus the feed-forward half and the classifier for one (also prints their
    CUDA-event bandwidth); `norm-small` = the LayerNorm / RMSNorm layer kernels on a 268 MB tensor;
    `llama-step` = the whole decode step of an 8-layer llama2-7B-shaped model, eager and from a CUDA graph
    (a timing case, about 15 GB on the device: not for ncu)."""
    import torch
    from mycaffe_b200 import _lib, function_ids as ids
    lib = _lib.load()
    dev = torch.device("cuda", 0)
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
        # whole-transformer decode step, llama2-7B geometry cut to 8 layers, one sequence at position 2047
        import ctypes as C
        from mycaffe_b200 import llama2 as M
        cfg = dict(dim=4096, hidden_dim=11008, n_layers=8, n_heads=32, n_kv_heads=32, vocab_size=32000, seq_len=4096)
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
            kc, vc = (torch.randn(L, 1, S, dim, device=dev).to(wdt) for _ in range(2))
            fr, fi = np.empty((S, 64), np.float32), np.empty((S, 64), np.float32)
            fp = C.POINTER(C.c_float)
            lib.mca_rope_tables_host(S, 128, 10000.0, fr.ctypes.data_as(fp), fi.ctypes.data_as(fp))
            frd, fid = torch.from_numpy(fr).to(dev), torch.from_numpy(fi).to(dev)
            cfg_c = M.McaLlamaConfig(**cfg)
            need = lib.mca_llama_workspace_floats(C.byref(cfg_c), 1, S)
            ws_, logits = torch.empty(need, device=dev), torch.empty(1, vocab, device=dev)
            tok = torch.zeros(1, dtype=torch.int32, device=dev)
            pos = torch.full((1,), 2047, dtype=torch.int32, device=dev)
            names = ("token_embedding_table", "rms_att_weight", "rms_ffn_weight", "rms_final_weight", "wq", "wk", "wv", "wo",
                     "w1", "w2", "w3", "wcls")
            w_c = M.McaLlamaWeights(*[w[n].data_ptr() for n in names], int(bf16))
            s_c = M.McaLlamaState(kc.data_ptr(), vc.data_ptr(), int(bf16), frd.data_ptr(), fid.data_ptr(), ws_.data_ptr(), need)
            def step(stream=None):
                st = stream if stream is not None else torch.cuda.current_stream()
                return lib.mca_llama_forward(C.byref(cfg_c), C.byref(w_c), C.byref(s_c), tok.data_ptr(), pos.data_ptr(), 1, 2048,
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
            sz = 2 if bf16 else 4
            nbytes = (L * (4 * dim * dim + 3 * dim * hidden) + vocab * dim) * sz + L * 2 * 2048 * dim * sz
            out.update({"rc": rc, "bytes": nbytes, "GBps_graph": round(nbytes / out["graph_ms"] / 1e6, 1)})
            res["bf16" if bf16 else "f32"] = out
            del w, kc, vc, graph
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
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=PF_B)
    ap.add_argument("--seq-len", type=int, default=PF_T)
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="multi-GPU: exchange the head outputs with a NCCL all-gather instead of the kernel's peer stores")
    ap.add_argument("--case", default=None, choices=["prefill-small", "prefill-full", "bwd-small", "decode-small", "gemv-small", "norm-small", "llama-step"],
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
    args.cpu_baseline = args.cpu_baseline and world == 1
    run_ours(args)


if __name__ == "__main__":
    main()
