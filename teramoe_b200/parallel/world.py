"""Expert-parallel world: ranks, symmetric arenas and the host-side collectives around them.

Three ways to run the same per-rank pipeline (teramoe_b200/engine.py):

* ``EPWorld.from_group(group)``  one process per GPU; arenas are exchanged as CUDA IPC handles through
  ``torch.distributed`` (NCCL or gloo is only the bootstrap, like teramoe/buffer.py:74-101), or, with
  ``use_fabric=True`` / ``TERAMOE_ARENA=vmm``, allocated with the driver's virtual memory management and shared as POSIX
  file descriptors over Unix sockets (parallel/fdpass.py; reference: csrc/moe_extension.cpp:16-125).
  With CPU tensors the same class moves data with gloo collectives instead of peer stores.
* ``EPWorld.single(device)``      one rank, no peers.
* ``VirtualCluster(n, device)``   n ranks emulated in ONE process on ONE device (or on the CPU), stepped in
  lock-step phase by phase.  Cross-rank barriers are phase boundaries, so no kernel ever waits for
  another kernel on the same GPU.  Used by the tests to run the multi-rank index math and the real
  push kernels without several GPUs.

The pipeline is written as a generator that yields where it needs something from other ranks:
  ("barrier",)            all ranks reached this point and their peer stores are visible
  ("acquire",)            every rank has released the data arena after its previous call (see release_arena)
  ("allgather", tensor)   -> stacked tensor of all ranks (host path only)
  ("grow", nbytes)        the data arena must hold nbytes on every rank (all ranks ask together)
  ("push", {dst: [...]})  host path only: writes into peers' tables
"""
from __future__ import annotations

import os
from typing import Dict, Generator, List, Optional

import torch
import torch.distributed as dist

STATUS_RING = 64                 # status snapshots in flight before the oldest is waited for
STRICT_STATUS = os.environ.get("TERAMOE_STRICT_STATUS", "0") == "1"
CONTROL_ROW_INTS = 8192          # capacity of one metadata row (E + ranks + 2 ints must fit)
MAX_BLOCKS = 65536               # per-block arrival counters of the fused dispatch (8.4 M slot rows)
_ALIGN = 256
# "ipc": cudaMalloc + CUDA IPC handles.  "vmm": cuMemCreate + shareable descriptors (what `use_fabric=True` selects).
ARENA_KIND = os.environ.get("TERAMOE_ARENA", "ipc")


def _round_up(v: int, a: int = _ALIGN) -> int:
    return (v + a - 1) // a * a


class EPWorld:
    """One rank's view of the expert-parallel group."""

    def __init__(self, rank: int, size: int, device: torch.device, group=None, virtual_peers: Optional[list] = None,
                 use_fabric: bool = False):
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.group = group
        if ARENA_KIND not in ("ipc", "vmm"):
            raise ValueError(f"TERAMOE_ARENA must be 'ipc' or 'vmm', not {ARENA_KIND!r}")
        self.use_fabric = bool(use_fabric)
        self.arena_vmm = (self.use_fabric or ARENA_KIND == "vmm") and virtual_peers is None
        self.virtual_peers = virtual_peers          # list of EPWorld in a VirtualCluster
        self.is_cuda = self.device.type == "cuda"
        self.epoch = 0
        self.control = None
        self.data = None
        self.data_bytes = 0
        self._ptr_cache: Dict[str, torch.Tensor] = {}
        self.cpu_tables: Dict[str, torch.Tensor] = {}
        self.closed = False
        self.wait_limit_ms = 30_000          # what kernels use when the status block holds no limit (csrc/ptx.cuh)
        if self.is_cuda:
            from .._build import load_ext
            self.ext = load_ext()
            self.signal_offset = size * CONTROL_ROW_INTS * 4      # barrier / push-complete flags, one int per rank
            self.free_offset = self.signal_offset + 512           # arena-release flags, one int per rank
            self.blk_cnt_offset = self.signal_offset + 1024
            self.control_bytes = _round_up(self.blk_cnt_offset + MAX_BLOCKS * 4 + 4096)
            self.control = self._new_arena(self.control_bytes)
            # status block (csrc/ptx.cuh): words 0-3 error record, words 4-5 the limit (ns) of waits on other ranks
            self.status = torch.zeros(8, dtype=torch.int32, device=self.device)
            self.sizes_host = torch.zeros(12, dtype=torch.int32).pin_memory()
            self._status_ring = torch.zeros(STATUS_RING, 4, dtype=torch.int32).pin_memory()
            self._status_pending: list = []          # (ring row, event) of status snapshots not looked at yet
            self._status_next = 0
            ms = int(os.environ.get("TERAMOE_PEER_WAIT_LIMIT_MS", "0"))
            if ms > 0:
                self.set_wait_limit_ms(ms)
        self.strict_status = STRICT_STATUS
        self.arena_user = None               # who laid the data arena out last (the low-latency windows keep flags there)
        self._release_seq = 0            # calls whose arena reads this rank has released (same on all ranks at the same call)

    # ------------------------------------------------------------------ construction
    @classmethod
    def single(cls, device, use_fabric: bool = False) -> "EPWorld":
        w = cls(0, 1, device, use_fabric=use_fabric)
        if w.is_cuda:
            w.control.adopt_peer_pointers([w.control.local_ptr()])
        return w

    @classmethod
    def from_group(cls, group, device, use_fabric: bool = False) -> "EPWorld":
        rank, size = dist.get_rank(group), dist.get_world_size(group)
        w = cls(rank, size, device, group=group, use_fabric=use_fabric)
        if w.is_cuda:
            w._open_ipc(w.control)
        return w

    def _new_arena(self, nbytes: int):
        with torch.cuda.device(self.device):
            if self.arena_vmm:
                return self.ext.SymmetricArena(self.rank, self.size, nbytes, vmm=True, fabric=self.use_fabric)
            return self.ext.SymmetricArena(self.rank, self.size, nbytes)

    def _open_ipc(self, arena) -> None:
        """Map every peer's arena (collective)."""
        if self.size == 1:
            arena.adopt_peer_pointers([arena.local_ptr()])
            return
        if arena.is_vmm():
            from .fdpass import exchange_fds
            with torch.cuda.device(self.device):
                arena.open_peer_fds(exchange_fds(arena.export_fd(), self.rank, self.size, group=self.group))
            return
        handles: List[Optional[bytes]] = [None] * self.size
        dist.all_gather_object(handles, bytes(arena.export_handle()), group=self.group)
        if any(h is None or len(h) != 64 for h in handles):
            raise RuntimeError("teramoe_b200: malformed IPC handle received during bootstrap")
        arena.open_peers(handles)

    # ------------------------------------------------------------------ arenas
    def ptr_table(self, arena, offset: int, key: str) -> torch.Tensor:
        """Device int64 array with (peer base + offset) for every rank."""
        k = f"{key}:{arena.local_ptr()}:{offset}"
        t = self._ptr_cache.get(k)
        if t is None:
            t = torch.tensor([p + offset for p in arena.peer_ptrs()], dtype=torch.int64, device=self.device)
            self._ptr_cache[k] = t
        return t

    def blk_cnt_view(self) -> torch.Tensor:
        return self.control.view(self.blk_cnt_offset, [MAX_BLOCKS], torch.int32)

    def meta_view(self, C: int) -> torch.Tensor:
        return self.control.view(0, [self.size * C], torch.int32)

    def ensure_data(self, nbytes: int) -> None:
        """Real-mode growth of the data arena (collective over the group)."""
        if nbytes <= self.data_bytes:
            return
        assert self.virtual_peers is None, "virtual clusters grow through VirtualCluster.grow"
        new_bytes = _round_up(int(nbytes * 1.25))
        torch.cuda.synchronize(self.device)
        if self.group is not None and self.size > 1:
            dist.barrier(group=self.group)
        old = self.data
        self.data = self._new_arena(new_bytes)
        self._open_ipc(self.data)
        if old is not None:
            if self.group is not None and self.size > 1:
                dist.barrier(group=self.group)
            old.close()
        self.data_bytes = new_bytes
        self._ptr_cache = {k: v for k, v in self._ptr_cache.items() if k.startswith("control")}

    def side_stream(self):
        """High-priority stream for communication kernels that overlap compute."""
        if getattr(self, "_side_stream", None) is None:
            self._side_stream = torch.cuda.Stream(self.device, priority=-1)
        return self._side_stream

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # ------------------------------------------------------------------ drivers
    def set_wait_limit_ms(self, ms: int) -> None:
        """Limit of every device-side wait on ANOTHER rank (barriers, arrival counters), in milliseconds; 0 restores
        the built-in default (30 s; the reference budgets about 100 s, csrc/kernels/configs.cuh:20-26).  Waits inside
        one CTA pair keep their fixed 2 s."""
        self.wait_limit_ms = int(ms) if ms > 0 else 30_000
        if self.is_cuda:
            self.status[4:6].view(torch.int64).fill_(int(ms) * 1_000_000)

    def _raise_status(self, s) -> None:
        self.status[:4].zero_()
        self._status_pending.clear()
        names = {1: "mbarrier wait", 2: "flag wait", 3: "barrier", 4: "bad argument"}
        raise RuntimeError(f"teramoe_b200: a device-side wait ran out on rank {self.rank}: {names.get(s[0], s[0])} "
                           f"(site {s[1]}, block {s[2]}, detail {s[3]})")

    def check_status(self) -> None:
        """Blocking read of the status block; raises if a device-side wait of any earlier kernel ran out."""
        if not self.is_cuda:
            return
        s = self.status[:4].tolist()
        self._status_pending.clear()
        if s[0] != 0:
            self._raise_status(s)

    def note_status(self, strict: Optional[bool] = None) -> None:
        """End of a call: snapshot the status block into pinned memory behind the call's kernels (16 bytes, no host
        wait).  Snapshots are looked at by poll_status (every later call does that first) and by check_status; with
        `strict` (or TERAMOE_STRICT_STATUS=1) the host waits for this snapshot, so the call whose wait ran out is the one
        that raises, at the price of one stream wait per call."""
        if not self.is_cuda:
            return
        if len(self._status_pending) >= STATUS_RING:
            row, ev = self._status_pending.pop(0)
            ev.synchronize()
            if int(self._status_ring[row, 0]) != 0:
                self._raise_status(self._status_ring[row].tolist())
        row = self._status_next
        self._status_next = (row + 1) % STATUS_RING
        self._status_ring[row].copy_(self.status[:4], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._status_pending.append((row, ev))
        if self.strict_status if strict is None else strict:
            ev.synchronize()
        self.poll_status()

    def poll_status(self) -> None:
        """Look at the snapshots whose copies have completed; never waits."""
        if not self.is_cuda:
            return
        while self._status_pending and self._status_pending[0][1].query():
            row, _ = self._status_pending.pop(0)
            if int(self._status_ring[row, 0]) != 0:
                self._raise_status(self._status_ring[row].tolist())

    # ------------------------------------------------------------------ arena reuse between calls
    # Peers store into this rank's data arena and every call reuses it.  The rule that makes this safe: a rank
    # RELEASES its arena when it has enqueued the last read of a call (a signal-only kernel: one flag per peer, no
    # wait), and a call that lets peers write without having crossed a barrier first (backward dispatch, cached-handle
    # dispatch, un-fused combine) first ACQUIRES: it waits (a wait-only kernel on local flags, normally satisfied
    # long ago) until every rank has released as many calls as this rank has.  A forward needs no acquire: its count
    # exchange is a barrier that every rank signals after its previous call.  Combine pushes need none either: a peer
    # only pushes rows that this rank asked for in the same call.
    def release_arena(self) -> None:
        if not self.is_cuda or self.size == 1 or self.virtual_peers is not None:
            return
        self._release_seq += 1
        self.ext.ep_barrier(self.ptr_table(self.control, self.free_offset, "control_free"), self.rank, self.size, self._release_seq,
                            self.status, 540, 0, 1)

    def acquire_arena(self) -> None:
        if not self.is_cuda or self.size == 1 or self.virtual_peers is not None or self._release_seq == 0:
            return
        self.ext.ep_barrier(self.ptr_table(self.control, self.free_offset, "control_free"), self.rank, self.size, self._release_seq,
                            self.status, 560, 0, 2)

    def device_barrier(self, site: int = 500, limit_ms: int = 0, mask: Optional[torch.Tensor] = None) -> None:
        """Bounded all-rank barrier kernel on the current stream (limit_ms <= 0: the run-time limit for waits on other
        ranks).  `mask`: device int[ranks]; ranks marked there are neither signalled nor waited for."""
        if self.size == 1:
            return
        ep = self.next_epoch()
        self.ext.ep_barrier(self.ptr_table(self.control, self.signal_offset, "control_sig"), self.rank, self.size, ep,
                            self.status, site, limit_ms, 0, mask)

    def drive(self, gen: Generator):
        """Run a pipeline generator to completion in real (one process per rank) mode."""
        assert self.virtual_peers is None
        self.poll_status()
        try:
            req = next(gen)
            while True:
                kind = req[0]
                if kind == "barrier":
                    if self.is_cuda:
                        self.device_barrier()
                    else:
                        self._cpu_exchange_pushes()
                    req = gen.send(None)
                elif kind == "acquire":
                    self.acquire_arena()
                    req = gen.send(None)
                elif kind == "masked_barrier":
                    if self.is_cuda:
                        self.device_barrier(mask=req[1])
                    req = gen.send(None)
                elif kind == "allgather":
                    t = req[1]
                    if self.size == 1:
                        out = t.unsqueeze(0)
                    else:
                        lst = [torch.empty_like(t) for _ in range(self.size)]
                        dist.all_gather(lst, t, group=self.group)
                        out = torch.stack(lst)
                    req = gen.send(out)
                elif kind == "grow":
                    self.ensure_data(req[1])
                    req = gen.send(None)
                elif kind == "push":
                    self._pending_pushes = getattr(self, "_pending_pushes", [])
                    self._pending_pushes.append(req[1])
                    req = gen.send(None)
                else:
                    raise RuntimeError(f"unknown pipeline request {kind}")
        except StopIteration as stop:
            self.note_status()
            return stop.value

    def _cpu_exchange_pushes(self) -> None:
        pend = getattr(self, "_pending_pushes", [])
        self._pending_pushes = []
        merged: Dict[int, list] = {}
        for p in pend:
            for d, w in p.items():
                merged.setdefault(d, []).extend(w)
        gathered: List[Optional[dict]] = [None] * self.size
        if self.size == 1:
            gathered[0] = merged
        else:
            dist.all_gather_object(gathered, merged, group=self.group)
        for src in range(self.size):
            for (name, idx, val) in gathered[src].get(self.rank, []):
                apply_write(self.cpu_tables, name, idx, val)

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        if self.is_cuda:
            torch.cuda.synchronize(self.device)
            pending_error = None
            try:
                self.check_status()          # a wait that ran out in the last calls must not vanish with the buffer
            except RuntimeError as e:
                pending_error = e
            if self.group is not None and self.size > 1 and self.virtual_peers is None:
                try:
                    dist.barrier(group=self.group)
                except Exception:
                    pass
            if self.data is not None:
                self.data.close()
            self.control.close()
            self.data = None
            self._ptr_cache.clear()
            if pending_error is not None:
                raise pending_error


def apply_write(tables: Dict[str, torch.Tensor], name: str, idx: torch.Tensor, val: torch.Tensor) -> None:
    if idx.numel():
        tables[name][idx.long()] = val


class VirtualCluster:
    """n ranks in one process on one device, driven in lock step."""

    def __init__(self, n: int, device="cuda"):
        self.n = n
        self.device = torch.device(device)
        self.worlds: List[EPWorld] = []
        for r in range(n):
            self.worlds.append(EPWorld(r, n, self.device, virtual_peers=self.worlds))
        if self.device.type == "cuda":
            ptrs = [w.control.local_ptr() for w in self.worlds]
            for w in self.worlds:
                w.control.adopt_peer_pointers(ptrs)

    def grow(self, nbytes: int) -> None:
        if nbytes <= self.worlds[0].data_bytes:
            return
        new_bytes = _round_up(int(nbytes * 1.25))
        torch.cuda.synchronize(self.device)
        olds = [w.data for w in self.worlds]
        for w in self.worlds:
            with torch.cuda.device(self.device):
                w.data = w.ext.SymmetricArena(w.rank, self.n, new_bytes)
        ptrs = [w.data.local_ptr() for w in self.worlds]
        for w in self.worlds:
            w.data.adopt_peer_pointers(ptrs)
            w.data_bytes = new_bytes
            w._ptr_cache = {k: v for k, v in w._ptr_cache.items() if k.startswith("control")}
        for o in olds:
            if o is not None:
                o.close()

    def drive(self, gens: List[Generator]) -> list:
        """Step one generator per rank in lock step; returns their return values."""
        results = [None] * self.n
        reqs = [next(g) for g in gens]
        done = [False] * self.n
        while not all(done):
            kinds = {r[0] for r, d in zip(reqs, done) if not d}
            assert len(kinds) == 1 and not any(done), f"ranks diverged: {kinds}"
            kind = kinds.pop()
            if kind in ("barrier", "acquire"):      # ranks of a virtual cluster run one after the other on one stream
                sends = [None] * self.n
            elif kind == "allgather":
                stacked = torch.stack([r[1] for r in reqs])
                sends = [stacked] * self.n
            elif kind == "grow":
                self.grow(max(r[1] for r in reqs))
                sends = [None] * self.n
            elif kind == "push":
                for r in reqs:
                    for d, writes in r[1].items():
                        for (name, idx, val) in writes:
                            apply_write(self.worlds[d].cpu_tables, name, idx, val)
                sends = [None] * self.n
            else:
                raise RuntimeError(kind)
            for i, g in enumerate(gens):
                try:
                    reqs[i] = g.send(sends[i])
                except StopIteration as stop:
                    results[i] = stop.value
                    done[i] = True
        for w in self.worlds:
            w.check_status()
        return results

    def close(self) -> None:
        for w in self.worlds:
            w.close()
