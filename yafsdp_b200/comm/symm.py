"""Peer-memory ("symmetric") collective backend: hand-written NVLink kernels instead of NCCL.

Every rank allocates its communication buffers from an arena of CUDA-IPC-exported memory and maps
every peer's arena, so a buffer at offset ``o`` of the local arena has a twin at offset ``o`` of each
peer's arena (all ranks allocate in the same order with the same sizes).  The kernels
(``csrc/comm.cu``) then *pull*:

* all-gather: each rank copies the peers' shards straight into its local layer buffer;
* reduce-scatter: each owner reads its chunk of every rank's fp32 gradient buffer, sums in rank
  order with fp32 accumulation, applies the averaging factor and accumulates into the sharded gradient
  in the same pass (reference: four separate steps, ``ya_fsdp/_collectives.py:93-218``).

With the ``mc`` transport the arena is bound to an NVSwitch multicast object (allocated through
``torch.distributed._symmetric_memory``) and the kernels use ``multimem`` instructions instead: the
reduce-scatter reads the switch-computed sum of all ranks' copies (``multimem.ld_reduce``), the all-gather
stores each shard once to the multicast address of the layer buffer (``multimem.st``).

Cross-GPU ordering uses signal pads (sequence-numbered flags in peer memory, raised with atomic max) with
bounded waits; a wait that runs out sets the library status word, which ``check()`` reads.

This is the structure the reference gets from its optional closed-source library (registered
buffers owned by the communication layer, in-place collectives, fp32 accumulation:
``ya_fsdp/_param_group.py:46-69``, ``ya_fsdp/_collectives.py:66-71,163-164``), written for one
NVSwitch-connected box.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native
from ..ops import kernels
from .backends import CommBackend

__all__ = ["SymmBackend", "SymmArena"]

_ALIGN = 1024


class _CudaBuffer:
    """Expose a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class SymmArena:
    """Bump allocator over chunks of IPC-shared device memory mapped by every rank of ``group``."""

    def __init__(self, device: torch.device, group: dist.ProcessGroup, chunk_bytes: int = 1 << 30, multicast: bool = False):
        self.device = device
        self.group = group
        self.rank = group.rank()
        self.world = group.size()
        self.chunk_bytes = chunk_bytes
        self.chunks: list[tuple[int, int, list[int], torch.Tensor]] = []  # (local base, nbytes, peer bases, tensor)
        self.offset = 0
        # multicast arena: chunks come from torch's symmetric-memory allocator, which also binds them to an NVSwitch
        # multicast object; `mc_bases[i]` is the multicast address of chunk i
        self.multicast = multicast
        self.mc_bases: list[int] = []
        self._mc_keep: list[object] = []

    def _new_chunk_multicast(self, nbytes: int) -> bool:
        """Allocate a chunk that every rank maps and that is bound to a multicast object.  Returns False (on every rank)
        when this system offers no multicast; the caller then falls back to CUDA IPC chunks."""
        import torch.distributed._symmetric_memory as symm_mem

        ok, err = 1, ""
        t = h = None
        try:
            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            h = symm_mem.rendezvous(t, self.group)
            if not int(h.multicast_ptr):
                ok, err = 0, "no multicast address"
        except Exception as e:  # noqa: BLE001 - any failure means: no multicast here
            ok, err = 0, f"{type(e).__name__}: {e}"
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self.multicast = False
            self.last_multicast_error = err
            return False
        assert t is not None and h is not None
        off = int(getattr(h, "offset", 0))
        bases = [int(p) + off for p in h.buffer_ptrs]
        if bases[self.rank] != t.data_ptr():
            raise RuntimeError("symmetric-memory allocation: the local buffer pointer does not match the tensor")
        t.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.chunks.append((t.data_ptr(), nbytes, bases, t))
        self.mc_bases.append(int(h.multicast_ptr) + off)
        self._mc_keep.append(h)
        self.offset = 0
        return True

    def mc_ptr(self, t: torch.Tensor) -> int:
        """Multicast address of a tensor of the arena (0 when the arena has none or the tensor is not part of it)."""
        if not self.mc_bases:
            return 0
        p = t.data_ptr()
        for (base, nbytes, _, _), mc in zip(self.chunks, self.mc_bases):
            if base <= p < base + nbytes:
                return mc + (p - base)
        return 0

    def _new_chunk(self, nbytes: int) -> None:
        if self.multicast and self._new_chunk_multicast(nbytes):
            return
        if self.mc_bases:
            raise RuntimeError("multicast allocation stopped working after the first chunk")
        lib = _native.lib()
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            rc = lib.yf_ipc_alloc(nbytes, ctypes.byref(ptr), handle)
        if rc != 0:
            raise RuntimeError(f"yf_ipc_alloc({nbytes}) failed with code {rc}")
        handles: list[bytes | None] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=self.group)
        bases: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                bases.append(int(ptr.value))  # type: ignore[arg-type]
                continue
            hb = (ctypes.c_ubyte * 64).from_buffer_copy(h)  # type: ignore[arg-type]
            peer = ctypes.c_void_p()
            with torch.cuda.device(self.device):
                rc = lib.yf_ipc_open(hb, ctypes.byref(peer))
            if rc != 0:
                raise RuntimeError(f"yf_ipc_open of rank {r}'s buffer failed with code {rc} (peer access over NVLink is required)")
            bases.append(int(peer.value))  # type: ignore[arg-type]
        tensor = torch.as_tensor(_CudaBuffer(int(ptr.value), nbytes), device=self.device)  # type: ignore[arg-type]
        self.chunks.append((int(ptr.value), nbytes, bases, tensor))  # type: ignore[arg-type]
        self.offset = 0

    def alloc(self, nbytes: int) -> torch.Tensor:
        nbytes = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        if not self.chunks or self.offset + nbytes > self.chunks[-1][1]:
            self._new_chunk(max(nbytes, self.chunk_bytes))
        base, _, _, tensor = self.chunks[-1]
        out = tensor[self.offset : self.offset + nbytes]
        self.offset += nbytes
        return out

    def contains(self, t: torch.Tensor) -> bool:
        p = t.data_ptr()
        return any(base <= p < base + nbytes for base, nbytes, _, _ in self.chunks)

    def peer_ptrs(self, t: torch.Tensor) -> list[int]:
        p = t.data_ptr()
        for base, nbytes, bases, _ in self.chunks:
            if base <= p < base + nbytes:
                return [b + (p - base) for b in bases]
        raise ValueError("tensor was not allocated from the symmetric arena")


def _ptr_array(ptrs: list[int]) -> ctypes.Array:
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class SymmBackend(CommBackend):
    """Peer-memory collectives.  ``ag_transport`` / ``rs_transport`` choose how the bytes move:

    * ``"ce"``: the copy engines (one ``cudaMemcpyAsync`` per peer, spread over a pool of copy streams per collective);
      the all-gather then takes no SM at all, the reduce-scatter only a local sum over staging slots;
    * ``"cp"`` (all-gather only): the copy engines again, but every rank WRITES its shard into the peers' gather outputs
      instead of reading theirs.  Copies that one GPU issues as reads of several peers run one after another on one engine
      (seen in the step trace: seven 50 MB copies back to back, each alone on the links while it runs); writes to different
      peers can use an engine each.  The gather outputs then live in the shared arena (``symmetric_gather_output=True`` or
      ``ag_transport="cp"`` at construction) and every gather is bracketed by two device-side barriers on its stream: all
      ranks are done with what the buffer held / all writes have landed;
    * ``"sm"``: the pull kernels load from peer memory themselves;
    * ``"mc"``: NVSwitch multicast (``multimem``): the switch sums the gradient copies and replicates the parameter
      shards, so each GPU receives 1/world of the gradient bytes and sends each shard once (needs ``multicast=True``).

    The defaults are per world size (``DEFAULT_TRANSPORTS``); the environment variables ``YAFSDP_AG_TRANSPORT``,
    ``YAFSDP_RS_TRANSPORT``, ``YAFSDP_SYMM_TRANSPORT`` (both), ``YAFSDP_AG_CTAS``, ``YAFSDP_RS_CTAS`` override the
    constructor arguments; :meth:`set_transports` switches between steps.

    Ordering between GPUs (all waits bounded, a wait that runs out sets the library status word):

    * all-gather: the gather inputs are final between the step barrier (after the optimizer) and the end of backward, so
      pulling needs no per-call synchronisation;
    * reduce-scatter ``s``: every rank signals "my gradients for ``s`` are complete" and waits for all such signals,
      reduces, then signals "I have read everyone's buffer for ``s``" WITHOUT waiting; the wait for those signals is
      deferred to :meth:`before_write`, which the owner of a reduce buffer calls right before the buffer is written
      again (one or two layers of backward later, when the signals have long arrived).
    """

    name = "symm"
    needs_registered_buffers = True

    N_SLOTS = 8
    SLOT_STEP, SLOT_RS_READY, SLOT_RS_DONE, SLOT_SYNC, SLOT_MC_PRE, SLOT_MC_POST = 0, 1, 2, 3, 4, 5
    #: measured on 2 and 8 x B200 (Llama-2-7B step, ``benchmarks/transport_sweep.py``): all-gather on the copy engines,
    #: reduce-scatter by the pull kernel, at every world size
    DEFAULT_TRANSPORTS = {"ag": lambda world: "ce", "rs": lambda world: "sm"}

    def __init__(self, device: torch.device, group: dist.ProcessGroup | None, *, ag_transport: str | None = None,
                 rs_transport: str | None = None, multicast: bool | None = None, ag_ctas: int = 0, rs_ctas: int = 0,
                 single_comm_stream: bool = False, timeout_ms: int | None = None, symmetric_gather_output: bool = False):
        if group is None or device.type != "cuda":
            raise ValueError("the symmetric backend needs a CUDA device and a process group")
        if group.size() > 16:
            raise ValueError("the symmetric backend supports at most 16 ranks (one NVSwitch domain)")
        self.device = device
        self.group = group
        self.rank = group.rank()
        self.world = group.size()
        env = os.environ.get
        both = env("YAFSDP_SYMM_TRANSPORT", "").lower() or None
        ag = (env("YAFSDP_AG_TRANSPORT", "").lower() or both or ag_transport or self.DEFAULT_TRANSPORTS["ag"](self.world)).lower()
        rs = (env("YAFSDP_RS_TRANSPORT", "").lower() or (both if both != "cp" else None) or rs_transport or self.DEFAULT_TRANSPORTS["rs"](self.world)).lower()
        if multicast is None:
            multicast = "mc" in (ag, rs) or env("YAFSDP_SYMM_MULTICAST", "0") == "1"
        self.arena = SymmArena(device, group, chunk_bytes=int(env("YAFSDP_SYMM_CHUNK_MB", "2048")) << 20, multicast=multicast)
        self.pads = self.arena.alloc(self.N_SLOTS * 16 * 8)
        self.has_multicast = bool(self.arena.mc_bases)
        # gather outputs that peers can write (the push all-gather): decided once, before the groups allocate their buffers
        self.symmetric_gather_output = symmetric_gather_output or ag == "cp" or env("YAFSDP_SYMM_GATHER_OUTPUT", "0") == "1"
        self._pad_ptrs = _ptr_array(self.arena.peer_ptrs(self.pads))
        self._seq = [0] * self.N_SLOTS
        self.timeout_ms = timeout_ms if timeout_ms is not None else int(env("YAFSDP_SYMM_TIMEOUT_MS", "30000"))
        self.ag_ctas = int(env("YAFSDP_AG_CTAS", str(ag_ctas)))
        self.rs_ctas = int(env("YAFSDP_RS_CTAS", str(rs_ctas)))
        self.prefers_single_comm_stream = single_comm_stream or env("YAFSDP_SINGLE_COMM_STREAM", "0") == "1"
        self._staging: torch.Tensor | None = None
        # copy-engine transfers from different peers go to several streams so that they run on different engines; each
        # collective has its own pool, so a prefetch all-gather never queues behind the previous layer's reduction copies
        n_ce = int(env("YAFSDP_CE_STREAMS", str(max(1, min(self.world - 1, 8)))))
        self._ag_ce_streams = [torch.cuda.Stream(device=device, priority=-1) for _ in range(n_ce)]
        self._rs_ce_streams = [torch.cuda.Stream(device=device, priority=-1) for _ in range(n_ce)]
        self._ptr_cache: dict[int, ctypes.Array] = {}
        self._int_ptr_cache: dict[int, list[int]] = {}
        # reduce buffers that peers may still be reading: data pointer -> sequence number of the reduce-scatter
        self._unread: dict[int, int] = {}
        # measurement aid: collectives move nothing between GPUs (gathers are skipped, reductions only read the own chunk),
        # so a step timed with it is the compute-only step at this world size; the numbers it trains on are meaningless
        self.dry_run = False
        self.ag_transport = self.rs_transport = "ce"
        self.set_transports(ag, rs, warn=True)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def set_transports(self, ag: str | None = None, rs: str | None = None, *, ag_ctas: int | None = None,
                       rs_ctas: int | None = None, warn: bool = False) -> None:
        """Switch transports (between steps, on every rank alike).  ``"mc"`` needs the multicast arena chosen at
        construction; without it the default transport is used instead."""
        for kind, want in (("ag", ag), ("rs", rs)):
            if want is None:
                continue
            want = want.lower()
            if want not in ("ce", "sm", "mc") and not (kind == "ag" and want == "cp"):
                raise ValueError(f"unknown transport {want!r} (expected 'ce', 'sm' or 'mc'; 'cp' for the all-gather)")
            if want == "cp" and not self.symmetric_gather_output:
                raise ValueError("the push all-gather needs gather outputs in the shared arena: construct the backend with "
                                 "ag_transport='cp' or symmetric_gather_output=True")
            if want == "mc" and not self.has_multicast:
                fallback = self.DEFAULT_TRANSPORTS[kind](self.world)
                if warn and self.rank == 0:
                    import warnings

                    warnings.warn(f"NVSwitch multicast is not available ({getattr(self.arena, 'last_multicast_error', 'arena built without it')}); "
                                  f"using the {fallback!r} transport", stacklevel=3)
                want = fallback
            setattr(self, f"{kind}_transport", want)
        if ag_ctas is not None:
            self.ag_ctas = ag_ctas
        if rs_ctas is not None:
            self.rs_ctas = rs_ctas

    # ------------------------------------------------------------------ memory
    def alloc(self, numel: int, dtype: torch.dtype, device: torch.device, kind: str) -> torch.Tensor:
        if kind == "gather_output" and not (self.has_multicast or self.symmetric_gather_output):
            return torch.empty(numel, dtype=dtype, device=device)  # only this rank reads or writes it
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self.arena.alloc(nbytes)[:nbytes].view(dtype)

    def _peers(self, t: torch.Tensor) -> ctypes.Array:
        key = t.data_ptr()
        arr = self._ptr_cache.get(key)
        if arr is None:
            arr = _ptr_array(self.arena.peer_ptrs(t))
            self._ptr_cache[key] = arr
        return arr

    def _peer_ints(self, t: torch.Tensor) -> list[int]:
        key = t.data_ptr()
        ptrs = self._int_ptr_cache.get(key)
        if ptrs is None:
            ptrs = self.arena.peer_ptrs(t)
            self._int_ptr_cache[key] = ptrs
        return ptrs

    # ------------------------------------------------------------------ ordering between GPUs
    def _pad(self, slot: int, seq: int, mode: int) -> None:
        rc = _native.lib().yf_signal_pad(self._pad_ptrs, self.rank, self.world, slot, seq, self.timeout_ms, mode,
                                         torch.cuda.current_stream().cuda_stream)
        kernels._check(rc, "yf_signal_pad")

    def barrier(self, slot: int = 0) -> None:
        """All ranks' current streams meet here (device-side, bounded wait)."""
        self._seq[slot] += 1
        self._pad(slot, self._seq[slot], 3)

    def step_barrier(self) -> None:
        if not self.dry_run:
            self.barrier(self.SLOT_STEP)

    def before_write(self, buf: torch.Tensor) -> None:
        """``buf`` (a reduce input of an earlier :meth:`reduce_scatter`) is about to be overwritten on the current stream:
        wait until every peer has signalled that it finished reading it."""
        seq = self._unread.pop(buf.data_ptr(), None)
        if seq is not None:
            self._pad(self.SLOT_RS_DONE, seq, 2)

    def _ce_copies(self, copies: list[tuple[int, int, int]], pool: list[torch.cuda.Stream]) -> None:
        """``(dst, src, nbytes)`` device copies, ordered after the work already queued on the current stream and joined
        back into it; spread over the copy streams of ``pool`` when there are several."""
        lib = _native.lib()
        cur = torch.cuda.current_stream()
        if len(pool) <= 1 or len(copies) <= 1:
            for d, s, n in copies:
                rc = lib.yf_memcpy_async(d, s, n, cur.cuda_stream)
                if rc != 0:
                    raise RuntimeError(f"peer copy failed with code {rc}")
        else:
            start = torch.cuda.Event()
            start.record(cur)
            used: list[torch.cuda.Stream] = []
            for i, (d, s, n) in enumerate(copies):
                st = pool[i % len(pool)]
                if st not in used:
                    st.wait_event(start)
                    used.append(st)
                rc = lib.yf_memcpy_async(d, s, n, st.cuda_stream)
                if rc != 0:
                    raise RuntimeError(f"peer copy failed with code {rc}")
            for st in used:
                done = torch.cuda.Event()
                done.record(st)
                cur.wait_event(done)
        kernels._launches += len(copies)

    # ------------------------------------------------------------------ collectives
    def _reduce_own_chunk(self, dst: torch.Tensor, inp: torch.Tensor, shard: int, scale: float, accumulate: bool,
                          sumsq: torch.Tensor | None) -> bool:
        own = _ptr_array([inp.data_ptr() + self.rank * shard * inp.element_size()])
        rc = _native.lib().yf_reduce_scatter_pull_sumsq(own, dst.data_ptr(), shard, 0, 1, float(scale), int(accumulate),
                                                        int(inp.dtype == torch.bfloat16), self.rs_ctas,
                                                        None if sumsq is None else sumsq.data_ptr(), torch.cuda.current_stream().cuda_stream)
        kernels._check(rc, "yf_reduce_scatter_pull")
        return sumsq is not None

    def _subgroup(self, group: dist.ProcessGroup | None) -> list[int] | None:
        """Arena indices of the ranks of ``group`` when it is a proper subgroup of the backend's group (hierarchical
        partitioning gathers inside the ranks of one node), else ``None``."""
        if group is None or group is self.group or group.size() == self.world:
            return None
        mine = dist.get_process_group_ranks(self.group)
        return [mine.index(r) for r in dist.get_process_group_ranks(group)]

    def subgroup_barrier(self) -> None:
        """All ranks meet (on their current streams) before a gather inside subgroups reads shards that peers wrote during
        the forward pass; the caller issues it once per backward pass."""
        if not self.dry_run:
            self.barrier(self.SLOT_SYNC)

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor, group: dist.ProcessGroup | None) -> None:
        if self.dry_run:
            return
        nbytes = inp.numel() * inp.element_size()
        sub = self._subgroup(group)
        if sub is not None:
            # inside a subgroup: copy engines or the pull kernel over the members' addresses (no multicast: the multicast
            # object spans the whole group)
            assert group is not None
            peers = self._peer_ints(inp)
            me, n = group.rank(), len(sub)
            with torch.autograd._unsafe_preserve_version_counter(out):
                if self.ag_transport == "sm":
                    rc = _native.lib().yf_allgather_pull(_ptr_array([peers[i] for i in sub]), out.data_ptr(), nbytes, me, n, self.ag_ctas,
                                                         torch.cuda.current_stream().cuda_stream)
                    kernels._check(rc, "yf_allgather_pull")
                else:
                    base = out.data_ptr()
                    self._ce_copies([(base + r * nbytes, peers[sub[r]], nbytes) for r in ((me + d) % n for d in range(n))], self._ag_ce_streams)
            return
        mc_out = self.arena.mc_ptr(out) if self.ag_transport == "mc" else 0
        if mc_out:
            stream = torch.cuda.current_stream().cuda_stream
            self.barrier(self.SLOT_MC_PRE)  # every rank is done with what its copy of `out` held before
            with torch.autograd._unsafe_preserve_version_counter(out):
                rc = _native.lib().yf_allgather_mc(inp.data_ptr(), mc_out, nbytes, self.rank, self.world, self.ag_ctas, stream)
            kernels._check(rc, "yf_allgather_mc")
            self.barrier(self.SLOT_MC_POST)  # every rank's stores have landed in every copy
            return
        if self.ag_transport == "cp" and self.arena.contains(out):
            outs = self._peer_ints(out)
            src, off = inp.data_ptr(), self.rank * nbytes
            self.barrier(self.SLOT_MC_PRE)  # every rank is done with what its copy of `out` held before
            with torch.autograd._unsafe_preserve_version_counter(out):
                self._ce_copies([(outs[r] + off, src, nbytes) for r in ((self.rank + d) % self.world for d in range(self.world))],
                                self._ag_ce_streams)
            self.barrier(self.SLOT_MC_POST)  # every rank's copies have landed in every output
            return
        if self.ag_transport in ("ce", "cp"):  # "cp" with an output outside the arena (allocated by the caller): read instead
            peers = self._peer_ints(inp)
            base = out.data_ptr()
            with torch.autograd._unsafe_preserve_version_counter(out):
                self._ce_copies([(base + r * nbytes, peers[r], nbytes) for r in ((self.rank + d) % self.world for d in range(self.world))],
                                self._ag_ce_streams)
            return
        with torch.autograd._unsafe_preserve_version_counter(out):
            rc = _native.lib().yf_allgather_pull(self._peers(inp), out.data_ptr(), nbytes, self.rank, self.world, self.ag_ctas,
                                                 torch.cuda.current_stream().cuda_stream)
        kernels._check(rc, "yf_allgather_pull")

    def gather_ranges(self, out: torch.Tensor, inp: torch.Tensor, ranges: list[tuple[int, int]]) -> None:
        """Copy the element ranges ``[lo, hi)`` of the gathered tensor ``out`` from the shards that hold them (``inp`` is
        this rank's shard; every rank's has the same size), on the current stream.  For the few small values that are
        needed before a kernel that gathers the rest itself (:func:`yafsdp_b200.ops.kernels.gemm_gathered`)."""
        if self.dry_run:
            return
        esz, shard = inp.element_size(), inp.numel()
        peers = self._peer_ints(inp)
        lib = _native.lib()
        stream = torch.cuda.current_stream().cuda_stream
        with torch.autograd._unsafe_preserve_version_counter(out):
            for lo, hi in ranges:
                while lo < hi:
                    r = lo // shard
                    end = min(hi, (r + 1) * shard)
                    rc = lib.yf_memcpy_async(out.data_ptr() + lo * esz, peers[r] + (lo - r * shard) * esz, (end - lo) * esz, stream)
                    if rc != 0:
                        raise RuntimeError(f"peer copy failed with code {rc}")
                    kernels._launches += 1
                    lo = end

    def reduce_scatter(self, dst: torch.Tensor, inp: torch.Tensor, group: dist.ProcessGroup | None, *, scale: float,
                       accumulate: bool, acc_fp32: bool = True, sumsq: torch.Tensor | None = None) -> bool:
        if dst.dtype != torch.float32 or inp.dtype not in (torch.float32, torch.bfloat16):
            raise NotImplementedError("the symmetric reduce-scatter produces fp32 from an fp32 or bf16 wire format")
        shard = inp.numel() // self.world
        if self.dry_run:
            return self._reduce_own_chunk(dst, inp, shard, scale, accumulate, sumsq)
        self.barrier(self.SLOT_RS_READY)  # every rank's gradients for this group are complete
        seq = self._seq[self.SLOT_RS_READY]
        stream = torch.cuda.current_stream().cuda_stream
        lib = _native.lib()
        bf16 = int(inp.dtype == torch.bfloat16)
        sq = None if sumsq is None else sumsq.data_ptr()
        if self.rs_transport == "ce":
            # copy engines bring every peer's chunk for this rank into local staging slots; a local kernel sums them
            esz = inp.element_size()
            need = self.world * shard * esz
            if self._staging is None or self._staging.numel() < need:
                self._staging = torch.empty(need, dtype=torch.uint8, device=self.device)
            peers = self._peer_ints(inp)
            sbase = self._staging.data_ptr()
            srcs = []
            copies = []
            for r in range(self.world):
                if r == self.rank:
                    srcs.append(inp.data_ptr())  # own chunk is read in place
                    continue
                copies.append((sbase + r * shard * esz, peers[r] + self.rank * shard * esz, shard * esz))
                srcs.append(sbase + r * shard * esz - self.rank * shard * esz)  # the kernel adds rank * shard
            self._ce_copies(copies, self._rs_ce_streams)
            self._pad(self.SLOT_RS_DONE, seq, 1)  # the peers' buffers have been read: the sum below is local
            rc = lib.yf_reduce_scatter_pull_sumsq(_ptr_array(srcs), dst.data_ptr(), shard, self.rank, self.world, float(scale),
                                                  int(accumulate), bf16, self.rs_ctas, sq, stream)
            kernels._check(rc, "yf_reduce_scatter_pull")
        else:
            if self.rs_transport == "mc" and self.arena.mc_ptr(inp):
                rc = lib.yf_reduce_scatter_mc(self.arena.mc_ptr(inp), dst.data_ptr(), shard, self.rank, self.world, float(scale),
                                              int(accumulate), bf16, self.rs_ctas, sq, stream)
            else:
                rc = lib.yf_reduce_scatter_pull_sumsq(self._peers(inp), dst.data_ptr(), shard, self.rank, self.world, float(scale),
                                                      int(accumulate), bf16, self.rs_ctas, sq, stream)
            kernels._check(rc, "yf_reduce_scatter_pull")
            self._pad(self.SLOT_RS_DONE, seq, 1)
        # this rank's buffer may be overwritten once every owner has read it: before_write() waits for that
        self._unread[inp.data_ptr()] = seq
        return sumsq is not None

    def peer_pointers(self, t: torch.Tensor) -> ctypes.Array:
        """Every rank's address of ``t`` (a tensor of the arena), as the native kernels take them."""
        return self._peers(t)

    def reduce_pushed(self, dst: torch.Tensor, slots: torch.Tensor, *, scale: float, accumulate: bool,
                      sumsq: torch.Tensor | None = None, valid_numel: int | None = None) -> bool:
        """Second half of the fused GEMM -> reduce-scatter: ``slots`` (this rank's reduce buffer, read as ``world`` slots of
        one shard each) holds what every rank pushed for this rank's shard; wait until all pushes have landed, then
        ``dst (+)= scale * sum of the slots`` in rank order (fp32, deterministic), optionally with the squared norm.
        Positions of the flat gradient at or beyond ``valid_numel`` (the layout's padding) are zeroed first."""
        if dst.dtype != torch.float32 or slots.dtype not in (torch.float32, torch.bfloat16):
            raise NotImplementedError("pushed gradients travel as fp32 or bf16 and are summed into fp32")
        esz = slots.element_size()
        shard = slots.numel() // self.world
        if self.dry_run:
            return self._reduce_own_chunk(dst, slots, shard, scale, accumulate, sumsq)
        self.barrier(self.SLOT_RS_READY)  # every rank's pushes for this group have completed
        seq = self._seq[self.SLOT_RS_READY]
        if valid_numel is not None:
            lo = max(0, min(shard, valid_numel - self.rank * shard))
            if lo < shard:
                slots.view(self.world, shard)[:, lo:].zero_()  # nobody pushes the padding
        base = slots.data_ptr()
        srcs = _ptr_array([base + (r - self.rank) * shard * esz for r in range(self.world)])  # the kernel adds rank * shard
        rc = _native.lib().yf_reduce_scatter_pull_sumsq(srcs, dst.data_ptr(), shard, self.rank, self.world, float(scale), int(accumulate),
                                                        int(esz == 2), self.rs_ctas, None if sumsq is None else sumsq.data_ptr(),
                                                        torch.cuda.current_stream().cuda_stream)
        kernels._check(rc, "yf_reduce_scatter_pull")
        self._pad(self.SLOT_RS_DONE, seq, 1)  # peers may push into these slots again (before_write() waits for this)
        self._unread[slots.data_ptr()] = seq
        return sumsq is not None

    def check(self) -> None:
        kernels.check_status()
