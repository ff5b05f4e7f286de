"""`Buffer`: the public entry point, signature-compatible with the reference's `teramoe.Buffer`.

Reference counterparts: teramoe/buffer.py:32-147 (construction / destroy), :153-290 (knobs, configs),
:293-454 (layout, dispatch, combine), :537-708 (low-latency API), :710-818 (fused autograd entry
points).  Differences that matter to callers:

* `comm=` (an mpi4py communicator instead of a group) only carries the rendezvous of a process group, see `_group_from_mpi`.
* One NVSwitch node only (EP = 1, 2, 4, 8): `num_rdma_bytes`, `num_qps_per_rank`, `allow_mnnvl` are accepted and
  ignored; the documented constructor call works on <= 8 ranks (the reference rejects it there,
  csrc/moe_extension.cpp:161-162).
* `use_fabric=True` allocates the symmetric arenas with the driver's virtual memory management (cuMemCreate, shared as
  POSIX file descriptors; a fabric handle is requested too where the platform has one) instead of cudaMalloc + CUDA IPC.
* `num_nvl_bytes` is a starting size: the symmetric arena grows (collectively) when a call needs more.
* Slot assignment is deterministic, so results are bitwise reproducible run to run.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from .config import COMPUTE_BATCH_SIZES, Config, topk_idx_t
from .engine import EPEngine, LayerHandle
from .low_latency import LowLatencyMixin
from .parallel.world import EPWorld
from .utils.events import EventHandle, EventOverlap
from .utils.nvlink import check_nvlink_connections


def _rows_as_bf16(t: torch.Tensor) -> torch.Tensor:
    """[T, C] of any dtype -> the same bytes as bf16 rows, zero-padded to a multiple of 16 bytes per row."""
    t = t.contiguous()
    raw = t.view(torch.uint8).reshape(t.shape[0], t.shape[1] * t.element_size())
    pad = (-raw.shape[1]) % 16
    if pad:
        raw = torch.cat([raw, raw.new_zeros(raw.shape[0], pad)], dim=1)
    return raw.contiguous().view(torch.bfloat16)


def _rows_from_bf16(rows: torch.Tensor, dtype: torch.dtype, cols: int) -> torch.Tensor:
    raw = rows.contiguous().view(torch.uint8).reshape(rows.shape[0], rows.shape[1] * rows.element_size())
    nbytes = cols * torch.empty((), dtype=dtype).element_size()
    return raw[:, :nbytes].contiguous().view(dtype)


class _TeraMoEFunction(torch.autograd.Function):
    """Autograd wrapper of the layer: gradients for x, topk_weights, W_gateup and W_down."""

    @staticmethod
    def forward(ctx, buffer, x, topk_idx, topk_weights, W_gateup, W_down, num_experts, grad_topk_weights, opts):
        needs_bwd = any(t.requires_grad for t in (x, topk_weights, W_gateup, W_down))
        out, saved = buffer._drive(buffer._engine.forward_gen(x, topk_idx, topk_weights, W_gateup, W_down, num_experts,
                                                              keep_for_backward=needs_bwd, impl=opts))
        buffer._release()
        ctx.buffer = buffer
        ctx.saved = saved
        ctx.grad_topk_weights = grad_topk_weights
        ctx.opts = opts
        ctx.save_for_backward(W_gateup, W_down)          # x itself is not kept (teramoe/buffer.py:726-727)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_out):
        W_gateup, W_down = ctx.saved_tensors
        buffer = ctx.buffer
        dx, gtw, dWgu, dWd = buffer._drive(buffer._engine.backward_gen(ctx.saved, grad_out.contiguous(), W_gateup, W_down,
                                                                      impl=ctx.opts))
        buffer._release()
        ctx.saved = None
        if ctx.grad_topk_weights is not None:
            ctx.grad_topk_weights.copy_(gtw)
            gtw = ctx.grad_topk_weights
        return None, dx, None, gtw, dWgu, dWd, None, None, None


def _group_from_mpi(comm, want_cuda: bool):
    """A torch.distributed group over the ranks of an mpi4py-style communicator (`Get_rank`, `Get_size`, `bcast`,
    `allgather`), for callers that launch with MPI and have no process group yet (reference: teramoe/buffer.py:78-86, which
    all-gathers its handles through the communicator itself).  Here the communicator only carries the rendezvous: rank 0
    picks a free port on the loop-back interface (all ranks sit on one node), everybody joins a process group there, and
    the rest of the bootstrap is the usual one.  With a process group already initialised the communicator must span it."""
    rank, size = int(comm.Get_rank()), int(comm.Get_size())
    if size == 1:
        return None
    if size > 8:
        raise ValueError("teramoe_b200 runs on one NVSwitch node: at most 8 ranks")
    if dist.is_initialized():
        members = sorted(int(r) for r in comm.allgather(dist.get_rank()))
        if members != list(range(dist.get_world_size())):
            raise ValueError("the communicator covers only part of the initialised process group: pass `group=` instead")
        return dist.group.WORLD
    endpoint = None
    if rank == 0:
        import socket
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.bind(("127.0.0.1", 0))
            endpoint = ("127.0.0.1", s.getsockname()[1])
    addr, port = comm.bcast(endpoint, root=0)
    dist.init_process_group("nccl" if want_cuda else "gloo", init_method=f"tcp://{addr}:{port}", rank=rank, world_size=size)
    return dist.group.WORLD


class Buffer(LowLatencyMixin):
    """Expert-parallel communication + fused MoE layer on one NVSwitch node."""

    num_sms: int = 20

    def __init__(self, group: Optional[dist.ProcessGroup] = None, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0,
                 low_latency_mode: bool = False, num_qps_per_rank: int = 24, allow_nvlink_for_low_latency_mode: bool = True,
                 allow_mnnvl: bool = False, use_fabric: bool = False, explicitly_destroy: bool = False, enable_shrink: bool = False,
                 comm=None, device: Optional[Union[str, torch.device]] = None) -> None:
        if num_nvl_bytes % 128 != 0 or num_rdma_bytes % 128 != 0:
            raise ValueError("buffer sizes must be multiples of 128 bytes")
        if comm is not None and group is None:
            want_cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
            group = _group_from_mpi(comm, want_cuda)
        if group is None and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            group = dist.group.WORLD
        if device is None:
            use_cuda = torch.cuda.is_available() and (group is None or dist.get_backend(group) != "gloo")
            device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.group_size = dist.get_world_size(group) if group is not None else 1
        if self.group_size > 8:
            raise ValueError("teramoe_b200 runs on one NVSwitch node: at most 8 ranks")
        self.num_nvl_bytes, self.num_rdma_bytes = num_nvl_bytes, num_rdma_bytes
        self.low_latency_mode = low_latency_mode
        self.explicitly_destroy = explicitly_destroy
        self.enable_shrink = enable_shrink
        self._destroyed = False
        if group is not None and self.device.type == "cuda":
            check_nvlink_connections(group)
        self.use_fabric = bool(use_fabric)
        self._world = (EPWorld.from_group(group, self.device, use_fabric=self.use_fabric) if group is not None
                       else EPWorld.single(self.device, use_fabric=self.use_fabric))
        self._engine = EPEngine(self._world)
        self._comm_stream = torch.cuda.Stream(self.device, priority=-1) if self.device.type == "cuda" else None
        if self.device.type == "cuda" and num_nvl_bytes > 0:
            self._world.ensure_data(num_nvl_bytes)
        self._ll_masked = set()
        self._ll_next_buffer = 0

    # ------------------------------------------------------------------ lifecycle
    def destroy(self) -> None:
        """Release the symmetric arenas (collective).  Requires explicitly_destroy=True, like the reference."""
        if not self.explicitly_destroy:
            raise RuntimeError("`explicitly_destroy` flag must be set to call destroy()")
        self._destroy()

    def _destroy(self) -> None:
        if not self._destroyed:
            self._destroyed = True
            self._world.close()

    def __del__(self):
        try:
            if not self._destroyed and not self.explicitly_destroy:
                self._destroy()
        except Exception:
            pass

    def _drive(self, gen):
        if self._destroyed:
            raise RuntimeError("Buffer was destroyed")
        return self._world.drive(gen)

    def _release(self) -> None:
        """Every collective method ends with this, after its last read of the symmetric arena has been enqueued:
        peers may then overwrite the arena in their next call (EPWorld.release_arena)."""
        self._world.release_arena()

    def check_status(self) -> None:
        """Wait for the kernels enqueued so far and raise if a device-side wait of any of them ran out.  Every call
        on the buffer looks at the snapshots of the calls before it without waiting; this is the blocking form, for
        the end of a step or of a run."""
        self._world.check_status()

    def set_wait_limit_ms(self, ms: int) -> None:
        """Limit of the device-side waits on other ranks (default 30 s; 0 restores it)."""
        self._world.set_wait_limit_ms(ms)

    def trace(self, on: bool = True) -> None:
        """Start / stop recording per-phase device times of the fused layer calls (CUDA events)."""
        self._engine.enable_trace(on)

    def trace_report(self) -> dict:
        """Mean milliseconds per phase since tracing started (and restart the record)."""
        return self._engine.trace_report()

    def state(self) -> dict:
        """Sizes and configuration needed to rebuild an equivalent Buffer (nothing else persists between calls)."""
        return {"rank": self.rank, "group_size": self.group_size, "device": str(self.device), "num_nvl_bytes": self.num_nvl_bytes,
                "arena_bytes": self._world.data_bytes, "num_sms": Buffer.num_sms, "low_latency_mode": self.low_latency_mode,
                "last_paths": dict(getattr(self._engine, "last_paths", {}))}      # which fused kernels the last layer call used

    # ------------------------------------------------------------------ knobs
    @staticmethod
    def is_sm90_compiled() -> bool:
        return False

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        if new_num_sms % 2 != 0:
            raise ValueError("The SM count must be even")
        Buffer.num_sms = new_num_sms

    @staticmethod
    def capture() -> EventOverlap:
        return EventOverlap(EventHandle())

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int) -> int:
        """Bytes of symmetric memory used by the low-latency layout (two buffers of per-expert,
        per-source windows, bf16 payload + 16-byte header), cf. csrc/config.hpp:133-219."""
        per_msg = 16 + hidden * 2
        one = num_experts * num_max_dispatch_tokens_per_rank * per_msg
        return ((2 * 2 * one + num_experts * 8) + 127) // 128 * 128

    def get_comm_stream(self):
        return self._comm_stream

    def get_local_buffer_tensor(self, dtype: torch.dtype, size: Optional[torch.Size] = None, offset: int = 0,
                                use_rdma_buffer: bool = False) -> torch.Tensor:
        if self.device.type != "cuda" or self._world.data is None:
            raise RuntimeError("no symmetric arena allocated yet")
        elem = torch.empty((), dtype=dtype).element_size()
        n = (self._world.data_bytes - offset) // elem
        t = self._world.data.view(offset, [n], dtype)
        return t if size is None else t[: int(torch.Size(size).numel())].view(size)

    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        if num_ranks not in (1, 2, 4, 8):
            raise ValueError(f"unsupported number of EP ranks: {num_ranks}")
        return Config(Buffer.num_sms, 24 if num_ranks <= 2 else 6, 256, 6, 128)

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        if num_ranks not in (1, 2, 4, 8):
            raise ValueError(f"unsupported number of EP ranks: {num_ranks}")
        return Config(Buffer.num_sms, {1: 10, 2: 10, 4: 9, 8: 4}[num_ranks], 256, 6, 128)

    # ------------------------------------------------------------------ stream protocol helpers
    def _enter(self, previous_event, allocate_on_comm_stream):
        if self._comm_stream is None:
            return None
        cur = torch.cuda.current_stream(self.device)
        if previous_event is not None and previous_event.event is not None and previous_event.event.event is not None:
            self._comm_stream.wait_event(previous_event.event.event)
        else:
            self._comm_stream.wait_stream(cur)
        return cur

    def _leave(self, cur, async_finish, tensors) -> EventOverlap:
        if self._comm_stream is None:
            return EventOverlap(None)
        if async_finish:
            ev = EventHandle(self._comm_stream)
            for t in tensors:
                if isinstance(t, torch.Tensor) and t.is_cuda:
                    t.record_stream(self._comm_stream)
                    t.record_stream(cur)
            return EventOverlap(ev, tuple(t for t in tensors if isinstance(t, torch.Tensor)))
        cur.wait_stream(self._comm_stream)
        return EventOverlap(None)

    def _on_comm_stream(self, fn: Callable, previous_event, async_finish, allocate_on_comm_stream):
        if self._comm_stream is None:
            return fn(), EventOverlap(None)
        cur = self._enter(previous_event, allocate_on_comm_stream)
        with torch.cuda.stream(self._comm_stream):
            res = fn()
        flat = res if isinstance(res, (tuple, list)) else (res,)
        return res, self._leave(cur, async_finish, flat)

    # ------------------------------------------------------------------ layout / dispatch / combine
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventOverlap] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """-> (num_tokens_per_rank [ranks] i32, None, num_tokens_per_expert [E] i32, is_token_in_rank [T,ranks] bool, event)."""
        N = self.group_size

        def run():
            T, K = topk_idx.shape
            El = num_experts // N
            if topk_idx.is_cuda:
                # two kernels, nothing else: per-chunk histograms (which also write is_token_in_rank), then their column sums
                ext = self._world.ext
                C = num_experts + N + 2
                chunk = ext.route_chunk_tokens()
                chunks = max(1, (T + chunk - 1) // chunk)
                dev = topk_idx.device
                hist = torch.zeros(chunks * C, dtype=torch.int32, device=dev) if T == 0 else torch.empty(chunks * C, dtype=torch.int32, device=dev)
                in_rank = torch.empty(T, N, dtype=torch.bool, device=dev)
                if T > 0:
                    ext.route_hist(topk_idx.contiguous(), num_experts, N, hist, in_rank)
                tot = torch.empty(C, dtype=torch.int32, device=dev)
                ext.route_sum(hist, chunks, C, tot)
                per_expert, per_rank = tot[:num_experts], tot[num_experts:num_experts + N]
            else:
                from . import layout as L
                row = L.count_row(topk_idx, num_experts, N)
                per_expert, per_rank = row[:num_experts].contiguous(), row[num_experts:num_experts + N].contiguous()
                in_rank = L.token_rank_hits(topk_idx, num_experts, N)
            return per_rank, None, per_expert, in_rank

        res, ev = self._on_comm_stream(run, previous_event, async_finish, allocate_on_comm_stream)
        return (*res, ev)

    def deepep_dispatch(self, x, handle: Optional[LayerHandle] = None, num_tokens_per_rank=None, num_tokens_per_rdma_rank=None,
                        is_token_in_rank=None, num_tokens_per_expert=None, topk_idx: Optional[torch.Tensor] = None,
                        topk_weights: Optional[torch.Tensor] = None, expert_alignment: int = 1, num_worst_tokens: int = 0,
                        config: Optional[Config] = None, previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                        allocate_on_comm_stream: bool = False, num_experts: Optional[int] = None):
        """Un-fused dispatch.  -> (recv_x, recv_topk_idx, recv_topk_weights, num_recv_tokens_per_expert_list, handle, event).

        Rows arrive once per (token, rank), ordered by source rank then token.  `recv_topk_idx` holds
        LOCAL expert ids (-1 for experts of other ranks, weights zeroed there), like
        csrc/kernels/intranode.cu:369-378.  With `handle=` (cached mode) only the payload moves and
        no host synchronisation happens.  `num_worst_tokens > 0` gives fixed-shape outputs (padded rows are
        zero, expert id -1, empty per-expert list) without any host wait: the tables are sized for that many rows
        and the layout sizes stay on the device (`_dispatch_fixed_shape`)."""
        if isinstance(x, tuple):
            # FP8 payload (x_e4m3 [T,H], scales [T,H/128] fp32), teramoe/buffer.py:344-346: both parts travel as raw
            # bytes through the same kernels (the second with the cached handle) and come back as a tuple
            xq, xs = x
            res = self.deepep_dispatch(_rows_as_bf16(xq), handle, num_tokens_per_rank, num_tokens_per_rdma_rank, is_token_in_rank,
                                       num_tokens_per_expert, topk_idx, topk_weights, expert_alignment, num_worst_tokens, config,
                                       previous_event, False, allocate_on_comm_stream, num_experts)
            recv_q = _rows_from_bf16(res[0], xq.dtype, xq.shape[1])
            recv_s, *_rest = self.deepep_dispatch(_rows_as_bf16(xs), res[4])
            recv_s = _rows_from_bf16(recv_s, xs.dtype, xs.shape[1])
            if recv_q.shape[0] > recv_s.shape[0]:      # fixed-shape mode pads the payload rows only
                recv_s = torch.cat([recv_s, recv_s.new_zeros(recv_q.shape[0] - recv_s.shape[0], recv_s.shape[1])])
            return ((recv_q, recv_s), *res[1:])
        x = x.contiguous()

        def run():
            eng = self._engine
            if handle is not None:
                h = handle
                tabs, _ = self._drive(eng.dispatch_gen(h, x, None, with_meta=False))
                got = tabs["recv_x"][: h.rows].clone()
                self._release()
                return got, None, None, None, h
            if topk_idx is None or topk_weights is None:
                raise ValueError("topk_idx and topk_weights are required without a cached handle")
            E = num_experts if num_experts is not None else (int(num_tokens_per_expert.numel()) if num_tokens_per_expert is not None else None)
            if E is None:
                raise ValueError("pass num_tokens_per_expert (from get_dispatch_layout) or num_experts")
            if num_worst_tokens > 0 and x.is_cuda:
                return self._dispatch_fixed_shape(x, topk_idx.contiguous(), topk_weights.float().contiguous(), E, num_worst_tokens)
            h = self._drive(eng.layout_gen(topk_idx.contiguous(), E))
            h.topk_weights = topk_weights
            tabs, _ = self._drive(eng.dispatch_gen(h, x, topk_weights.float().contiguous(), with_meta=True))
            eng.snapshot_tables(h, tabs)
            R, K = h.rows, h.K
            # the sender's dispatch kernel wrote these next to the rows (csrc/comm.cu dispatch_push)
            recv_x = tabs["recv_x"][:R].clone()
            recv_idx = tabs["row_topk_idx"][:R].to(topk_idx.dtype, copy=True)
            recv_w = tabs["row_topk_w"][:R].clone()
            self._release()
            if num_worst_tokens > 0:
                # fixed-shape mode (csrc/deep_ep.cpp:377-386): outputs have `num_worst_tokens` rows, rows past the
                # received count are zero with expert id -1, and no per-expert list is produced
                if R > num_worst_tokens:
                    raise RuntimeError(f"received {R} rows, more than num_worst_tokens={num_worst_tokens}")
                pad = num_worst_tokens - R
                recv_x = torch.cat([recv_x, recv_x.new_zeros(pad, recv_x.shape[1])])
                recv_idx = torch.cat([recv_idx, recv_idx.new_full((pad, K), -1)])
                recv_w = torch.cat([recv_w, recv_w.new_zeros(pad, K)])
                return recv_x, recv_idx, recv_w, [], h
            counts = h.expert_total_local.tolist()
            counts = [(c + expert_alignment - 1) // expert_alignment * expert_alignment for c in counts]
            return recv_x, recv_idx, recv_w, counts, h

        res, ev = self._on_comm_stream(run, previous_event, async_finish, allocate_on_comm_stream)
        return (*res, ev)

    def _dispatch_fixed_shape(self, x, topk_idx, topk_weights, E, worst):
        """Dispatch with `num_worst_tokens` rows of output and NO host wait (csrc/kernels/intranode.cu:521-531 in the
        reference): the receive tables are sized for `worst` rows, the layout sizes stay on the device, rows past the
        received count are filled with "nothing" by a kernel that reads the count there, and the handle learns the sizes
        when a later call (deepep_combine) asks for them.  If more than `worst` rows would arrive anywhere, nothing is
        sent and that later call raises."""
        eng, K = self._engine, topk_idx.shape[1]
        El = E // self.group_size
        if x.shape[0] > worst:
            raise ValueError(f"{x.shape[0]} tokens exceed num_worst_tokens={worst}")
        slots_cap = (worst * min(K, El) + 127) // 128 * 128 + 128 * El
        h = self._drive(eng.layout_gen(topk_idx, E, caps=(worst, slots_cap, worst)))
        h.topk_weights = topk_weights
        tabs, _ = self._drive(eng.dispatch_gen(h, x, topk_weights, with_meta=True))
        eng.snapshot_tables(h, tabs)
        recv_x = tabs["recv_x"][:worst].clone()
        recv_idx = tabs["row_topk_idx"][:worst].clone()
        recv_w = tabs["row_topk_w"][:worst].clone()
        self._release()
        self._world.ext.tail_fill(recv_x, recv_idx, recv_w, h.recv_row_base[self.group_size:])
        if topk_idx.dtype != torch.int64:
            recv_idx = recv_idx.to(topk_idx.dtype)
        return recv_x, recv_idx, recv_w, [], h

    def deepep_combine(self, x: torch.Tensor, handle: LayerHandle, topk_weights: Optional[torch.Tensor] = None, bias=None,
                       config: Optional[Config] = None, previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                       allocate_on_comm_stream: bool = False):
        """Un-fused combine: un-weighted sum over ranks of the rows given for each token (+ up to two
        bias tensors).  -> (combined_x [T,H], combined_topk_weights [T,K] or None, event)."""
        h = handle

        def run():
            out, cw = self._drive(self._engine.combine_rows_gen(h, x, topk_weights))
            self._release()
            if bias is not None:
                for b in (bias if isinstance(bias, (tuple, list)) else (bias,)):
                    if b is not None:
                        out = (out.float() + b.float()).to(out.dtype)
            return out, cw

        res, ev = self._on_comm_stream(run, previous_event, async_finish, allocate_on_comm_stream)
        return (*res, ev)

    # reference aliases (teramoe/buffer.py:453-454)
    dispatch = deepep_dispatch
    combine = deepep_combine

    def internode_dispatch(self, *args, **kwargs):
        """There is no second (RDMA) tier on one NVSwitch node: same as deepep_dispatch."""
        return self.deepep_dispatch(*args, **kwargs)

    def internode_combine(self, *args, **kwargs):
        return self.deepep_combine(*args, **kwargs)

    # ------------------------------------------------------------------ fused layer
    def _check_layer_args(self, x, topk_idx, topk_weights, W_gateup, W_down, num_experts, num_dispatch_sms, num_combine_sms,
                          total_sms, stage, compute_batch_size, combine_start_head_percent):
        if x.is_cuda and x.dtype != torch.bfloat16:
            raise ValueError("teramoe_autograd only supports bf16 inputs on CUDA")
        if x.dim() != 2 or topk_idx.dim() != 2 or topk_weights.shape != topk_idx.shape or topk_idx.shape[0] != x.shape[0]:
            raise ValueError("expected x [T,H], topk_idx [T,K], topk_weights [T,K]")
        if topk_idx.dtype not in (torch.int64, torch.int32):
            raise ValueError("topk_idx must be int64 or int32")
        if topk_idx.shape[1] > 32:
            raise ValueError("top-k must be <= 32")
        if num_dispatch_sms % 2 or num_combine_sms % 2:
            raise ValueError("num_dispatch_sms and num_combine_sms must be even")
        if stage not in (1, 2):
            raise ValueError("stage must be 1 or 2")
        if compute_batch_size not in COMPUTE_BATCH_SIZES:
            raise ValueError("compute_batch_size must be one of 1024, 2048, 4096")
        if not 0 <= combine_start_head_percent <= 100:
            raise ValueError("combine_start_head_percent must be in [0, 100]")
        if num_dispatch_sms + num_combine_sms + 1 >= total_sms:
            raise ValueError("no SMs left for compute")
        if num_experts % self.group_size:
            raise ValueError("num_experts must be divisible by the number of ranks")
        if W_gateup.dim() != 3 or W_down.dim() != 3 or W_gateup.shape[1] % 2:
            raise ValueError("expected W_gateup [E_local, 2I, H] and W_down [E_local, H, I]")
        if x.is_cuda:
            H, I = x.shape[1], W_gateup.shape[1] // 2
            if H % 64 or I % 64:
                raise ValueError("the tcgen05 kernels need hidden and intermediate sizes that are multiples of 64")
            if not (W_gateup.is_contiguous() and W_down.is_contiguous()):
                raise ValueError("W_gateup and W_down must be contiguous")
            if W_gateup.dtype != torch.bfloat16 or W_down.dtype != torch.bfloat16:
                raise ValueError("weights must be bf16 on CUDA")

    def teramoe_autograd(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, W_gateup: torch.Tensor,
                         W_down: torch.Tensor, num_experts: int, num_dispatch_sms: int = 24, num_combine_sms: int = 24,
                         total_sms: int = 148, stage: int = 1, dispatch_config: Optional[Config] = None,
                         combine_config: Optional[Config] = None, grad_topk_weights: Optional[torch.Tensor] = None,
                         compute_batch_size: int = 2048, combine_start_head_percent: int = 70) -> torch.Tensor:
        """MoE layer forward with autograd: out[t] = sum_k W_down[e_k] (w_k * silu(g) * u).

        x [T,H] bf16; topk_idx [T,K] (global expert ids, -1 = none); topk_weights [T,K] fp32;
        W_gateup [E_local, 2I, H] with rows interleaved (g0,u0,g1,u1,...); W_down [E_local, H, I].
        Gradients flow to x, topk_weights, W_gateup, W_down.  `grad_topk_weights` may be a
        preallocated fp32 [T,K] tensor that receives d(topk_weights).

        What the schedule arguments do here (same names and accepted values as the reference, teramoe/buffer.py:764-790):
          num_dispatch_sms            SMs (two per CTA pair) that first stream this rank's rows to the other ranks and then
                                      join the GEMM work
          total_sms                   grid of the layer kernel / the GEMM kernels
          compute_batch_size          rows per batch of the work list (1024 / 2048 / 4096): a batch's second GEMM follows
                                      its first GEMM batch by batch, so it sets how much activation sits between them
          combine_start_head_percent  how far (percent of a batch) the first GEMM runs ahead before the batch's second
                                      GEMM, whose epilogue is the combine push, is scheduled
          stage                       how finely units are ordered by the arrival of their rows (1: four groups, 2: eight)
          num_combine_sms             the separate kernels only (small shapes): SMs of the combine push kernel; in the
                                      one-kernel path every worker's epilogue pushes, so there is nothing to set aside
          dispatch_config / combine_config   accepted for compatibility (chunk sizes of rings that do not exist here)
        `autotune_teramoe` sweeps compute_batch_size x combine_start_head_percent like the reference's tuner."""
        self._check_layer_args(x, topk_idx, topk_weights, W_gateup, W_down, num_experts, num_dispatch_sms, num_combine_sms, total_sms,
                               stage, compute_batch_size, combine_start_head_percent)
        opts = {"num_dispatch_sms": num_dispatch_sms, "num_combine_sms": num_combine_sms, "total_sms": total_sms, "stage": stage,
                "compute_batch_size": compute_batch_size, "combine_start_head_percent": combine_start_head_percent}
        tw = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        return _TeraMoEFunction.apply(self, x.contiguous(), topk_idx.contiguous(), tw.contiguous(), W_gateup, W_down, num_experts,
                                      grad_topk_weights, opts)

    def teramoe_forward(self, x, topk_idx, topk_weights, W_gateup, W_down, num_experts, num_dispatch_sms: int = 24,
                        num_combine_sms: int = 24, total_sms: int = 148, stage: int = 1, dispatch_config: Optional[Config] = None,
                        combine_config: Optional[Config] = None, compute_batch_size: int = 2048,
                        combine_start_head_percent: int = 70) -> torch.Tensor:
        """Inference-only forward (nothing is kept for backward)."""
        self._check_layer_args(x, topk_idx, topk_weights, W_gateup, W_down, num_experts, num_dispatch_sms, num_combine_sms, total_sms,
                               stage, compute_batch_size, combine_start_head_percent)
        opts = {"num_dispatch_sms": num_dispatch_sms, "num_combine_sms": num_combine_sms, "total_sms": total_sms, "stage": stage,
                "compute_batch_size": compute_batch_size, "combine_start_head_percent": combine_start_head_percent}
        with torch.no_grad():
            out, _ = self._drive(self._engine.forward_gen(x.contiguous(), topk_idx.contiguous(), topk_weights.float().contiguous(),
                                                          W_gateup, W_down, num_experts, keep_for_backward=False, impl=opts))
            self._release()
        return out
