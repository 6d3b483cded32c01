"""Head-parallel execution of the attention path over the GPUs of one node.

Heads are independent in every variant of the path (per-(batch, head) scaled-dot-product attention;
the llama2 decode owns the KV-cache slice of its heads), so rank r of N computes heads
[r*H/N, (r+1)*H/N) and the only exchange is an all-gather of the head outputs.  The reference has no
counterpart: its only multi-GPU mode is data-parallel training (MyCaffe/common/Parallel.cs:351-508).

`torch.distributed` is the plumbing (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def _parse_cpulist(text: str) -> set[int]:
    """"0-15,64-79" -> {0..15, 64..79} (the format of sysfs cpulist files)."""
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_near_pci(bdf: str, sysfs_root: str = "/sys/bus/pci/devices") -> dict:
    """Restrict the calling thread to the CPUs local to PCI device `bdf` ("0000:1b:00.0"): its
    `local_cpulist` in sysfs, intersected with the CPUs the thread may already use.
    Returns {"cpus": n, "numa_node": k, "previous": set} or {"skipped": reason}; a missing sysfs entry
    (containers may hide it) is a skip, not an error.  Undo with os.sched_setaffinity(0, result["previous"])."""
    try:
        with open(os.path.join(sysfs_root, bdf, "local_cpulist")) as f:
            local = _parse_cpulist(f.read())
    except (OSError, ValueError) as e:
        return {"skipped": f"{type(e).__name__}: {e}"}
    node = -1
    try:
        with open(os.path.join(sysfs_root, bdf, "numa_node")) as f:
            node = int(f.read().strip())
    except (OSError, ValueError):
        pass
    previous = os.sched_getaffinity(0)
    cpus = local & previous
    if not cpus:
        return {"skipped": "no local CPU in the allowed set", "numa_node": node}
    try:
        os.sched_setaffinity(0, cpus)
    except OSError as e:                 # a sandbox may forbid it: run unbound rather than fail
        return {"skipped": f"{type(e).__name__}: {e}", "numa_node": node}
    return {"cpus": len(cpus), "numa_node": node, "previous": previous}


def bind_near_gpu(device_index: int) -> dict:
    """`bind_near_pci` for a CUDA device: host buffers the thread allocates and first touches afterwards, pinned
    ones included, then lie in the memory of the GPU's NUMA node.

    With one process per GPU and host tensors on both sides of every call, a rank whose staging memory sits on
    the other socket pays the inter-socket link on every copy, and eight ranks doing so at once share it."""
    try:
        pr = torch.cuda.get_device_properties(device_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
    except (AttributeError, RuntimeError, AssertionError, ValueError, TypeError) as e:
        return {"skipped": f"{type(e).__name__}: {e}"}
    return bind_near_pci(bdf)


def head_range(rank: int, world: int, n_heads: int, n_kv_heads: int | None = None) -> tuple[int, int]:
    """Heads owned by `rank`.  With grouped-query attention the split is by kv head, so that a rank
    owns whole groups of query heads together with their cache slice."""
    groups = n_kv_heads if n_kv_heads is not None else n_heads
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if groups % world != 0:
        raise ValueError(f"{groups} head groups do not divide over {world} ranks")
    per = (n_heads // groups) * (groups // world)
    return rank * per, (rank + 1) * per


def shard_heads(x: torch.Tensor, rank: int, world: int, head_dim: int = 1) -> torch.Tensor:
    """The slice of a (B, H, ...) tensor that `rank` owns (a contiguous copy)."""
    lo, hi = head_range(rank, world, x.shape[head_dim])
    return x.narrow(head_dim, lo, hi - lo).contiguous()


def gather_heads(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None,
                 strided: bool = False) -> torch.Tensor:
    """All-gather the (B, H/N, T, D) head outputs of every rank into (B, H, T, D).

    One collective per call: the ranks' slices land in a (N, B, H/N, T, D) buffer (`out`, reused when
    given).  By default they are copied back into head order; with `strided` the result is the
    (B, N, H/N, T, D) view of that buffer (head h = [h // (H/N), h % (H/N)]) and nothing is copied."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_local
    y_local = y_local.contiguous()
    if out is None:
        out = torch.empty((world,) + tuple(y_local.shape), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(out.view(-1), y_local.view(-1), group=group)
    B, Hl = y_local.shape[0], y_local.shape[1]
    if strided:
        return out.transpose(0, 1)
    # (N, B, Hl, ...) -> (B, N*Hl, ...)
    return out.transpose(0, 1).reshape((B, world * Hl) + tuple(y_local.shape[2:]))


def gather_decode_outputs(o_local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Decode step: (B, dim/N) per rank -> (B, dim), the input of the Wo projection."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return o_local
    o_local = o_local.contiguous()
    if out is None:
        out = torch.empty((world,) + tuple(o_local.shape), dtype=o_local.dtype, device=o_local.device)
    dist.all_gather_into_tensor(out.view(-1), o_local.view(-1), group=group)
    return out.transpose(0, 1).reshape(o_local.shape[0], world * o_local.shape[1])


class PeerOutput:
    """The full (B, H, T, D) bf16 attention output, held by every rank and filled by every rank's kernel.

    The buffers are symmetric memory (`torch.distributed._symmetric_memory`): each rank maps its peers'
    buffers, and the forward kernel stores every finished piece of its heads' output tiles into all of them
    (`mca_sdpa_forward_tc_scatter`), so the all-gather disappears into the kernel's epilogue.  `wait()` is the
    only synchronisation left: a one-element all-reduce on the current stream, after which every rank's
    stores have landed everywhere.

    Every rank writes into every buffer, so the buffer is also a write-after-read hazard: a rank that is still
    reading step n's result must not have step n+1's kernels of its peers writing into it.  `wait()` only orders
    "all kernels finished" before the local reads; a consumer therefore calls `release()` (a second collective)
    once it has finished reading and before anyone launches the next scatter -- or alternates between two
    `PeerOutput` buffers.  A caller with no consumer between steps (the benchmark) needs neither."""

    def __init__(self, B: int, H: int, T: int, D: int, device, group=None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem
        self.shape = (B, H, T, D)
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if not 1 <= self.world <= 8:
            raise ValueError("the scatter epilogue takes up to 8 destinations")
        self.tensor = symm_mem.empty((B, H, T, D), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != self.tensor.data_ptr() or any(p == 0 or p % 16 for p in ptrs):
            raise RuntimeError(f"unexpected symmetric-memory mapping {ptrs}")
        self._ptrs = ptrs
        self._flag = torch.zeros(1, device=device)
        self._ctypes = ctypes

    @property
    def strides(self) -> tuple[int, int, int]:
        B, H, T, D = self.shape
        return H * T * D, T * D, D

    def destinations(self, h_lo: int):
        """ctypes array of where head `h_lo` lies in every rank's buffer, this rank's own buffer first."""
        B, H, T, D = self.shape
        if not 0 <= h_lo < H:
            raise ValueError(f"head {h_lo} outside {H}")
        off = h_lo * T * D * 2
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        arr = (self._ctypes.c_void_p * self.world)(*[self._ptrs[r] + off for r in order])
        return arr

    def wait(self) -> None:
        """Every rank's kernel has finished (stream-ordered; the host does not block)."""
        dist.all_reduce(self._flag, group=self.group)

    def release(self) -> None:
        """Every rank has finished reading the buffer (stream-ordered): the next scatter may overwrite it."""
        dist.all_reduce(self._flag, group=self.group)


class PeerDecodeOutput:
    """The (B, dim) head outputs of a decode layer-step, held by every rank and completed by every rank's exchange
    kernel (`mca_decode_exchange`): each rank stores its (B, dim/N) slice into all N buffers over NVLink, raises its
    flag everywhere and waits for the others' flags, so no collective is launched per layer-step.

    Two buffers alternate by exchange (a rank may still be reading exchange g while its peers store g + 1); a buffer is
    reused by exchange g + 2, which no rank can reach before every rank has started exchange g + 1, i.e. has finished
    with the result of exchange g.  Buffers, flag arrays and the ticket are symmetric memory, zeroed at set-up."""

    def __init__(self, B: int, dim: int, device, lib, group=None, limit_ms: int = 2000):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if not 1 <= self.world <= 8 or dim % (4 * self.world):
            raise ValueError("up to 8 ranks, and dim / ranks must be a multiple of 4")
        self.B, self.dim, self.dim_local = B, dim, dim // self.world
        self.data = symm_mem.empty((2, B, dim), dtype=torch.float32, device=device)
        self.flags = symm_mem.empty((16,), dtype=torch.int32, device=device)   # [0..7] flags, [8] ticket, [12..15] status
        self.data.zero_()
        self.flags.zero_()
        hd = symm_mem.rendezvous(self.data, self.group)
        hf = symm_mem.rendezvous(self.flags, self.group)
        self._data_ptrs, self._flag_ptrs = [int(x) for x in hd.buffer_ptrs], [int(x) for x in hf.buffer_ptrs]
        if self._data_ptrs[self.rank] != self.data.data_ptr() or self._flag_ptrs[self.rank] != self.flags.data_ptr():
            raise RuntimeError("unexpected symmetric-memory mapping")
        self._handles = (hd, hf)
        self._lib, self._ctypes, self.limit_ms = lib, ctypes, int(limit_ms)
        self.generation = 0
        torch.cuda.synchronize(device)
        dist.barrier(self.group)         # every rank's buffers and flags are zero before anyone stores

    def exchange(self, out_local: torch.Tensor, stream=None) -> torch.Tensor:
        """Enqueue the exchange of `out_local` (B, dim/N) on the stream; returns the (B, dim) buffer that is complete
        when the enqueued kernel has finished."""
        C = self._ctypes
        self.generation += 1
        g = self.generation
        buf = g & 1
        off = buf * self.B * self.dim * 4
        dst = (C.c_void_p * self.world)(*[p_ + off for p_ in self._data_ptrs])
        fl = (C.c_void_p * self.world)(*self._flag_ptrs)
        st = stream if stream is not None else torch.cuda.current_stream()
        base = self.flags.data_ptr()
        rc = self._lib.mca_decode_exchange(out_local.data_ptr(), dst, fl, base, base + 8 * 4, base + 12 * 4, self.world, self.rank,
                                           self.B, self.dim_local, self.dim, self.rank * self.dim_local, g, self.limit_ms,
                                           st.cuda_stream)
        if rc:
            raise RuntimeError(f"mca_decode_exchange failed with {rc}")
        return self.data[buf]

    def status(self):
        """The exchange kernels' status words (blocking): [0] != 0 means a bounded wait gave up."""
        return self.flags[12:16].tolist()
