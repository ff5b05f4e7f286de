"""Per-rank pipeline of the expert-parallel MoE layer (forward and backward) as phase generators.

Phase order, forward:   route counts -> [exchange] -> layout -> dispatch push -> [barrier] -> expand,
gate_up GEMM + SwiGLU, down GEMM, combine push -> [barrier] -> combine reduce.
Backward re-uses the forward layout (slots are deterministic): dispatch grad rows -> [barrier] ->
expand, grad_act GEMM + dSwiGLU, dX GEMM, two weight-gradient GEMMs, combine push (+ route-weight
gradients) -> [barrier] -> reduce.

For large shapes the default collapses these phases into fused kernels: "dispatch push -> barrier -> expand ->
first GEMM" becomes ONE cooperative kernel (csrc/fused.cu: dispatch CTA pairs feed compute CTA pairs through
per-block arrival counters, then join them), and "second GEMM -> combine push" becomes the GEMM with the
push epilogue (csrc/gemm2.cu, kEpiPush).  The switches and the measured rules are below.

Kept for backward, as in the reference (csrc/teramoe/teramoe_orchestrator.cu:3653-3678): the
dispatched X once per received token, the (gate, up) pre-activation per slot, and the slot tables.
`act` is recomputed from the pre-activation.

On CUDA tensors every step is a hand-written sm_100a kernel (csrc/); on CPU tensors the same steps
run as plain PyTorch index math (teramoe_b200/layout.py), which is what the CPU tests and the gloo
multi-process tests exercise.

Reference counterparts: csrc/moe_extension.cpp:1959-2408 (fused forward host path), :2461-2568
(backward host path), teramoe/buffer.py:710-762 (autograd function).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import layout as L
from .ops import gemm
from .config import UNIT_ROWS
from .parallel.world import EPWorld, _round_up

# Feed the GEMMs through TMA row gather (tile::gather4) instead of an expanded slot-space copy.
# Measured on B200 (H=7168, I=2048, 65,536 slot rows): gather4 sustains about one 4-row x 128-byte
# copy per ~70 cycles per SM, which caps the gate_up GEMM at 457 TFLOP/s against 1400 with a dense
# operand, while the expand pass costs 0.3 ms.  So the expanded copy is the default, and the gather kernels are only
# compiled when the extension is built with -DTMOE_WITH_GATHER4 (the switch raises otherwise).
USE_TMA_GATHER = os.environ.get("TERAMOE_TMA_GATHER", "0") == "1"
# CTA-pair (tcgen05 cta_group::2, 256x256 tiles) GEMM kernels: bitwise equal to the one-CTA 128x256
# kernels and 6-27 % faster (csrc/gemm2.cu).  "0" selects the one-CTA kernels.
USE_CTA_PAIRS = os.environ.get("TERAMOE_CTA_PAIRS", "1") == "1"
# Combine fused into the GEMM: the epilogues of the down GEMM (forward) and the dX GEMM (backward) store
# every output row straight into the landing table of the token's rank (coalesced peer stores over
# NVLink staged through shared memory, tile by tile, while the tensor cores work on the next tile).
# Measured at EP=4 (H=7168, I=2048, top-8): the down GEMM takes 1.40 ms with the pushed combine against
# 1.39 ms without, i.e. the all-to-all is hidden; the step drops from 17.3 to 16.8 ms.  (A first version
# that stored 64-byte fragments straight from the epilogue registers cost +4 ms.)  "0" = separate
# combine_push kernel (one row per (token, rank) on the wire instead of one per (token, k)).
# The push is only hidden when the GEMM lasts longer than its transfer.  Per byte pushed over NVLink the down GEMM
# does I FLOPs and the dX GEMM 2I (2*S*I*H resp. 2*S*2I*H FLOPs for S*H*2 bytes), and the machine balance is
# WIRE_BALANCE = sustained GEMM rate / per-direction link rate = 1.4e15 / 770e9 = 1818 FLOP per byte.  The epilogue
# push overlaps with the mainloop of the next tile, so the break-even sits a little below the balance: "auto" (the
# default) fuses when FLOPs per byte >= FUSE_MIN_BALANCE * WIRE_BALANCE, i.e. forward I >= 1455, backward I >= 728,
# and always on a single rank.  Checked against measurements: I=2048 wins fused at EP=2/4/8 (forward ratio 1.13),
# I=512 loses (ratio 0.28: the pushed down GEMM took 4.1 ms against 1.07 ms GEMM + 1.29 ms separate push at EP=4, the
# step 21.8 ms against 15.2 ms), I=14336 (ratio 7.9) wins.
_FUSED_MODE = os.environ.get("TERAMOE_FUSED_COMBINE", "auto")
FUSED_COMBINE = _FUSED_MODE != "0"
SUSTAINED_GEMM_FLOPS = 1.4e15            # cuBLAS bf16 under the power cap on this part
LINK_BYTES_PER_S = 770e9                 # measured peer copy, one direction
WIRE_BALANCE = SUSTAINED_GEMM_FLOPS / LINK_BYTES_PER_S
FUSE_MIN_BALANCE = float(os.environ.get("TERAMOE_FUSE_MIN_BALANCE", "0.8"))


def flops_per_wire_byte(I: int, backward: bool) -> float:
    """FLOPs of the GEMM whose epilogue pushes the combine rows, per byte it puts on the wire."""
    return float(2 * I if backward else I)


def use_fused_combine(I: int, num_ranks: int, backward: bool) -> bool:
    if _FUSED_MODE in ("0", "1"):
        return _FUSED_MODE == "1"
    return num_ranks == 1 or flops_per_wire_byte(I, backward) >= FUSE_MIN_BALANCE * WIRE_BALANCE
# Backward, more than one rank: the combine push of dX (+ barrier) can run on a side stream on a few SMs
# while the two weight-gradient GEMMs, which nothing downstream waits for, run on the remaining SMs.
# Measured at EP=2 (H=7168, I=2048): 18.0 ms per step with the overlap against 16.7 ms without (the
# step is compute bound, so the SMs taken from the GEMMs cost more than the hidden transfer saves).
# Off by default.
OVERLAP_BWD_COMBINE = os.environ.get("TERAMOE_OVERLAP_BWD_COMBINE", "0") == "1"
OVERLAP_COMM_SMS = int(os.environ.get("TERAMOE_OVERLAP_COMM_SMS", "8"))

TABLES = ("recv_x", "slot_row", "slot_w", "slot_tk", "row_tok", "row_land", "row_slots", "landing", "gtw", "row_topk_idx", "row_topk_w")
EXTRA_TABLES = ("slot_x", "row_first", "slot_src")   # fused dispatch: slot-space operand rows, first slot of every received row,
                                                     # slot that holds a slot's row (once-per-rank wire format)

# Dispatch fused into the GEMM that consumes it (csrc/fused.cu): one cooperative kernel, a few CTA pairs
# push rows to the peers while the others run the gate_up (forward) / grad_act (backward) GEMM on the
# rows that arrive; the dispatch pairs join the GEMM when their rows are out.  "auto": when the GEMM outlasts
# the transfer (same rule as the fused combine, which it requires) and the slot-space operand table, which
# then lives in the symmetric arena, stays under FUSED_DISPATCH_MAX_BYTES.
# Measured (H=7168, I=2048, top-8, 8192 tokens/rank, step ms fused / separate on the same box):
# EP=1 16.0 / 16.5 and 16.3 / 17.0 (two boxes' clocks), EP=2 17.0 / 17.4, EP=4 17.2 / 17.4, EP=8 19.0 / 19.1.
_FUSED_DISPATCH_MODE = os.environ.get("TERAMOE_FUSED_DISPATCH", "auto")
FUSED_DISPATCH_MAX_BYTES = int(float(os.environ.get("TERAMOE_FUSED_DISPATCH_MAX_BYTES", "8e9")))
# CTA pairs that dispatch before they join the GEMM: "n" or "forward,backward"
# Unset: the layer's `num_dispatch_sms` argument decides (two SMs per pair), like the reference's dispatch-SM knob.
_pairs_env = os.environ.get("TERAMOE_FUSED_DISPATCH_PAIRS")
_pairs = [int(v) for v in (_pairs_env or "16,16").split(",")]
FUSED_DISPATCH_CLUSTERS = (_pairs[0], _pairs[-1])


def dispatch_pairs(kind: int, num_dispatch_sms: int = 0) -> int:
    if _pairs_env is None and num_dispatch_sms > 0:
        return max(2, min(48, num_dispatch_sms // 2))
    return FUSED_DISPATCH_CLUSTERS[kind]
FUSED_DISPATCH_GROUPS = int(os.environ.get("TERAMOE_FUSED_DISPATCH_GROUPS", "4"))


# The whole layer direction as ONE cooperative kernel (csrc/layer.cu): dispatch, both GEMMs, the combine push, the
# weight gradients (backward) and the reduce run as items of one work list.  "auto": wherever the fused dispatch applies.
_LAYER_KERNEL_MODE = os.environ.get("TERAMOE_LAYER_KERNEL", "auto")
# NVTX marks at every phase boundary of the host path (TERAMOE_NVTX=1), for time lines taken with a system profiler.
NVTX_MARKS = os.environ.get("TERAMOE_NVTX", "0") == "1"
# Enqueue the whole forward before the host has read the layout sizes (see EPEngine.layout_gen); "0" waits for them first.
LAUNCH_AHEAD = os.environ.get("TERAMOE_LAUNCH_AHEAD", "1") == "1"
# Wire format of the dispatch inside the layer kernel.  "entry": one row per (token, k) entry, written by its sender straight
# into the entry's slot.  "rank": one row per (token, destination rank): it goes to the token's first slot on that rank and
# the receiver's gather warps copy it into the token's other slots there (top-8 over 8 ranks: 539 instead of 822 MB per rank
# and transfer on the headline shape).  Results are bit-identical.  Default "entry": the transfer is hidden behind the
# GEMMs at EP <= 8 on this shape (producers wait 0.35 ms per pair for arrivals at EP=8), and "rank" adds a local copy pass
# (measured at EP=1, where 7/8 of the rows become copies: 18.1 ms per step against 16.7-17.2 ms).
LAYER_WIRE = os.environ.get("TERAMOE_WIRE", "entry")
if LAYER_WIRE not in ("entry", "rank"):
    raise ValueError(f"TERAMOE_WIRE must be 'entry' or 'rank', not {LAYER_WIRE!r}")
LAYER_REDUCE_CHUNK = 64          # tokens per reduce item
LAYER_MIN_LAG_PER_PAIR = float(os.environ.get("TERAMOE_LAYER_MIN_LAG", "2"))


def use_layer_kernel() -> bool:
    return _LAYER_KERNEL_MODE != "0"


def use_fused_dispatch(I: int, num_ranks: int, table_bytes: int = 0) -> bool:
    if not USE_CTA_PAIRS or USE_TMA_GATHER:
        return False
    if _FUSED_DISPATCH_MODE in ("0", "1"):
        return _FUSED_DISPATCH_MODE == "1"
    # same balance rule as the forward combine (the kernel needs the pushed combine, and its GEMM does 2I FLOPs per byte received)
    return flops_per_wire_byte(I, False) >= FUSE_MIN_BALANCE * WIRE_BALANCE and table_bytes <= FUSED_DISPATCH_MAX_BYTES


@dataclass
class LayerHandle:
    """Everything that identifies where rows went; valid for one (topk_idx, num_experts) on one rank."""
    T: int
    K: int
    H: int
    E: int
    N: int
    rank: int
    rows: int            # token-once rows received by this rank
    slots: int           # padded slot rows of this rank
    land_rows: int       # landing rows of this rank (sum of distinct destination ranks of its tokens)
    maxima: tuple        # (rows, slots, land rows, tokens) maxima over ranks: arena geometry
    send_slot: torch.Tensor
    send_row: torch.Tensor
    land_off: torch.Tensor
    ndst: torch.Tensor
    recv_row_base: torch.Tensor
    seg_offsets: torch.Tensor
    mblock_expert: torch.Tensor
    num_mblocks: torch.Tensor
    expert_total_local: torch.Tensor
    send_order: Optional[torch.Tensor] = None    # fused dispatch: this rank's entries in sending order
    num_send: Optional[torch.Tensor] = None      # device scalar: number of entries in send_order
    unit_order: Optional[torch.Tensor] = None    # fused dispatch: units sorted by arrival group
    fused_dispatch: bool = False
    layer_kernel: bool = False                   # the whole direction runs as one kernel (csrc/layer.cu)
    pending: Optional[object] = None             # CUDA event behind the copy of the layout sizes, while the host has not read them
    geom_ok: Optional[torch.Tensor] = None       # device flag: the layout fits the capacities the tables were sized with
    opts: Optional[dict] = None                  # schedule knobs of the layer call (compute_batch_size, ...)
    num_dispatch_sms: int = 0                    # SMs that dispatch first in the fused dispatch + GEMM kernel (0: default)
    unit_blk: Optional[torch.Tensor] = None      # CTA-pair GEMMs: first block of every unit (+ sentinel)
    num_units: Optional[torch.Tensor] = None
    slot_row: Optional[torch.Tensor] = None
    slot_w: Optional[torch.Tensor] = None
    slot_tk: Optional[torch.Tensor] = None
    row_slots: Optional[torch.Tensor] = None
    row_land: Optional[torch.Tensor] = None
    row_tok: Optional[torch.Tensor] = None
    topk_idx: Optional[torch.Tensor] = None
    topk_weights: Optional[torch.Tensor] = None


@dataclass
class SavedForBackward:
    handle: LayerHandle
    saved_x: torch.Tensor        # [rows, H]
    preact: torch.Tensor         # [slots, 2I]
    stats: dict = field(default_factory=dict)


def _table_sizes(maxima, H: int, K: int):
    rmax, smax, lmax, tmax = [max(int(v), 1) for v in maxima]
    lmax = max(lmax, tmax * K)      # the fused combine lands one row per (token, k) entry
    smax = (smax + 127) // 128 * 128
    sizes = {
        "recv_x": rmax * H * 2, "slot_row": smax * 4, "slot_w": smax * 4, "slot_tk": smax * 4,
        "row_tok": rmax * 4, "row_land": rmax * 4, "row_slots": rmax * K * 4,
        "landing": lmax * H * 2, "gtw": tmax * K * 4, "row_topk_idx": rmax * K * 8, "row_topk_w": rmax * K * 4,
        "slot_x": smax * H * 2, "row_first": rmax * 4, "slot_src": smax * 4,
    }
    return sizes, (rmax, smax, lmax, tmax)


def _arena_geometry(maxima, H: int, K: int, fused_dispatch: bool = False):
    sizes, (rmax, smax, lmax, tmax) = _table_sizes(maxima, H, K)
    offs, off = {}, 0
    for name in TABLES + (EXTRA_TABLES if fused_dispatch else ()):
        offs[name] = off
        off += _round_up(sizes[name])
    return offs, off, (rmax, smax, lmax, tmax)


class EPEngine:
    def __init__(self, world: EPWorld):
        self.world = world
        self.is_cuda = world.is_cuda
        self.ext = world.ext if self.is_cuda else None
        self._trace = None          # list of (phase name, CUDA event) while tracing
        self._caps = {}             # (K, E, N) -> (rows, slots, tokens) capacities learnt from earlier calls (layout_gen)
        self.last_wait_ns = {}      # whole-layer kernel: {0: forward, 1: backward} -> int64[8] wait counters (csrc/layer.h LayerStat)
        self.last_paths = {}

    # ------------------------------------------------------------------ phase tracing
    def enable_trace(self, on: bool = True) -> None:
        """Record a CUDA event at every phase boundary of forward_gen / backward_gen (device time per
        phase, read with trace_report).  The reference has no in-kernel or per-phase timers
        (only a kineto helper in tests/utils.py:173-238)."""
        self._trace = [] if (on and self.is_cuda) else None

    def _mark(self, name: str) -> None:
        if NVTX_MARKS and self.is_cuda:
            torch.cuda.nvtx.mark("teramoe " + name.strip())      # phase boundaries on the host time line of a profiler
        if self._trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._trace.append((name, ev))

    def trace_report(self) -> dict:
        """Mean milliseconds per phase over the traced calls: time from the previous mark to this one."""
        if not self._trace:
            return {}
        torch.cuda.synchronize()
        acc, cnt = {}, {}
        prev = None
        cur_phase = "fwd"
        for name, ev in self._trace:
            if name.endswith(":start"):
                cur_phase = name.split(":")[0]
            if prev is not None and not name.endswith(":start"):
                name = name if not name.startswith("  ") else cur_phase + name

                acc[name] = acc.get(name, 0.0) + prev.elapsed_time(ev)
                cnt[name] = cnt.get(name, 0) + 1
            prev = ev
        self._trace = []
        return {k: acc[k] / cnt[k] for k in acc}

    # ------------------------------------------------------------------ arena reuse between calls
    def _acquire(self):
        """Before pushes that no barrier of the same call precedes: wait until every rank has released the arena after
        its previous call (EPWorld.release_arena / acquire_arena)."""
        if self.is_cuda and self.world.size > 1:
            yield ("acquire",)

    # ------------------------------------------------------------------ table access
    def _tables(self, offs, maxima, H, K, dtype):
        w = self.world
        w.arena_user = "tables"
        rmax, smax, lmax, tmax = maxima
        if self.is_cuda:
            v = w.data.view
            return {
                "recv_x": v(offs["recv_x"], [rmax, H], torch.bfloat16),
                "slot_row": v(offs["slot_row"], [smax], torch.int32),
                "slot_w": v(offs["slot_w"], [smax], torch.float32),
                "slot_tk": v(offs["slot_tk"], [smax], torch.int32),
                "row_tok": v(offs["row_tok"], [rmax], torch.int32),
                "row_land": v(offs["row_land"], [rmax], torch.int32),
                "row_slots": v(offs["row_slots"], [rmax, K], torch.int32),
                "landing": v(offs["landing"], [lmax, H], torch.bfloat16),
                "gtw": v(offs["gtw"], [tmax * K], torch.float32),
                "row_topk_idx": v(offs["row_topk_idx"], [rmax, K], torch.int64),
                "row_topk_w": v(offs["row_topk_w"], [rmax, K], torch.float32),
                **({"slot_x": v(offs["slot_x"], [smax, H], torch.bfloat16),
                    "row_first": v(offs["row_first"], [rmax], torch.int32),
                    "slot_src": v(offs["slot_src"], [smax], torch.int32)} if "slot_x" in offs else {}),
            }
        t = w.cpu_tables
        shapes = {"recv_x": ((rmax, H), dtype), "slot_row": ((smax,), torch.int32), "slot_w": ((smax,), torch.float32),
                  "slot_tk": ((smax,), torch.int32), "row_tok": ((rmax,), torch.int32), "row_land": ((rmax,), torch.int32),
                  "row_slots": ((rmax, K), torch.int32), "landing": ((lmax, H), dtype), "gtw": ((tmax * K,), torch.float32),
                  "row_topk_idx": ((rmax, K), torch.int64), "row_topk_w": ((rmax, K), torch.float32)}
        for name, (shape, dt) in shapes.items():
            cur = t.get(name)
            if cur is None or tuple(cur.shape) != shape or cur.dtype != dt:
                t[name] = torch.zeros(shape, dtype=dt)
        return t

    # ------------------------------------------------------------------ routing + dispatch
    def layout_gen(self, topk_idx: torch.Tensor, num_experts: int, caps=None):
        """Counts exchange and deterministic layout.  -> LayerHandle without receive tables.

        The sizes of the layout (rows, slots, maxima over ranks) are computed on the device.  Without `caps` the host
        waits for them here (one 48-byte read).  With `caps` = (rows, slots, tokens) capacities it does not: the handle
        comes back with `pending` set, its tables are sized by the capacities, the device flag `geom_ok` tells the
        kernels whether the layout fits them, and `resolve_sizes` reads the numbers later (behind kernels that are
        already enqueued, so the GPU never idles while the host catches up)."""
        w = self.world
        N, rank, E = w.size, w.rank, num_experts
        T, K = topk_idx.shape
        if E % N != 0:
            raise ValueError(f"num_experts ({E}) must be divisible by the number of ranks ({N})")
        if E + N + 2 > 8192:
            raise ValueError("too many experts for the metadata row")
        El = E // N
        dev = topk_idx.device
        if not self.is_cuda:
            row = L.count_row(topk_idx, E, N)
            meta = yield ("allgather", row)
            gl = L.global_layout(meta, E, N)
            sl = L.send_layout(topk_idx, E, N, rank, gl)
            seg_offsets, me = L.recv_tables(rank, E, N, gl)
            maxima = (int(gl.rows.max()), int(gl.slots_padded.max()), int(gl.land_rows.max()), int(meta[:, E + N + 1].max()))
            recv_row_base = torch.cat([gl.row_base[rank], gl.rows[rank:rank + 1]]).to(torch.int32)
            return LayerHandle(T, K, 0, E, N, rank, int(gl.rows[rank]), int(gl.slots_padded[rank]), int(gl.land_rows[rank]), maxima,
                               sl.send_slot, sl.send_row, sl.land_off, sl.ndst, recv_row_base, seg_offsets, me,
                               torch.tensor([me.numel()], dtype=torch.int32),
                               gl.expert_total.view(N, El)[rank].to(torch.int32).contiguous(), topk_idx=topk_idx)
        ext = self.ext
        C = E + N + 2
        chunk = ext.route_chunk_tokens()
        chunks = max(1, (T + chunk - 1) // chunk)
        chunk_hist = torch.zeros(chunks * C, dtype=torch.int32, device=dev)
        chunk_base = torch.empty(chunks * C, dtype=torch.int32, device=dev)
        if T > 0:
            ext.route_hist(topk_idx, E, N, chunk_hist)
        ext.route_scan(chunk_hist, chunk_base, chunks, E, rank, N, w.ptr_table(w.control, 0, "control_meta"),
                       w.ptr_table(w.control, w.signal_offset, "control_sig"), 0, w.status)
        yield ("barrier",)
        i32 = dict(dtype=torch.int32, device=dev)
        lay = [torch.empty(E, **i32), torch.empty(E, **i32), torch.empty(E, **i32), torch.empty(N, **i32),
               torch.empty(N + 1, **i32), torch.empty(El + 1, **i32), torch.empty(2, **i32), torch.empty(12, **i32),
               torch.empty(E, **i32)]
        ext.layout_finalize(w.meta_view(C), rank, N, E, lay, *(caps if caps is not None else (0, 0, 0)))
        w.sizes_host.copy_(lay[7], non_blocking=True)
        pending = None
        if caps is None:
            torch.cuda.current_stream(dev).synchronize()
            w.check_status()
            R, S, Lr, rmax, smax, lmax, nmb, tmax = w.sizes_host.tolist()[:8]
        else:
            pending = torch.cuda.Event()
            pending.record()
            rmax, smax, tmax = caps
            R, S, Lr, lmax, nmb = -1, -1, -1, 0, smax // 128
        send_slot = torch.empty(T, K, **i32)
        send_order = torch.empty(max(T * K, 1), **i32)
        send_row = torch.empty(T, N, **i32)
        land_off = torch.empty(T, **i32)
        ndst = torch.empty(T, **i32)
        if T > 0:
            ext.route_assign(topk_idx, E, N, chunk_base, lay, send_slot, send_row, land_off, ndst, send_order)
        mblock_expert = torch.empty(max(nmb, 1), **i32)
        unit_blk = torch.zeros((nmb + El) // 2 + 2, **i32)
        num_units = torch.zeros(1, **i32)
        h = LayerHandle(T, K, 0, E, N, rank, R, S, Lr, (rmax, smax, lmax, tmax), send_slot, send_row, land_off, ndst, lay[4], lay[5],
                        mblock_expert, lay[6], lay[0].view(N, El)[rank].contiguous(), topk_idx=topk_idx)
        h.unit_blk, h.num_units = unit_blk, num_units
        h.send_order, h.num_send = send_order, lay[6][1:2]
        h.num_mblocks = lay[6][0:1]
        h.pending, h.geom_ok = pending, lay[7][8:9]
        return h

    def resolve_sizes(self, h: LayerHandle) -> bool:
        """Read the layout sizes of a handle made with capacities (waits for the copy behind layout_finalize, not for
        the kernels enqueued after it).  False: the layout did not fit; the kernels of the call did nothing and the
        caller repeats the call with larger capacities (which this records)."""
        if h.pending is None:
            return True
        h.pending.synchronize()
        h.pending = None
        R, S, Lr, rmax, smax, lmax, nmb, tmax, ok = self.world.sizes_host.tolist()[:9]
        self._note_caps(h, (rmax, smax, tmax))
        if not ok:
            return False
        h.rows, h.slots, h.land_rows, h.maxima = R, S, Lr, (rmax, smax, lmax, tmax)
        for name, n in (("slot_row", S), ("slot_w", S), ("slot_tk", S), ("row_slots", R), ("row_land", R), ("row_tok", R)):
            t = getattr(h, name)
            if t is not None and t.shape[0] > n:     # copies taken with the capacity of the tables: cut to the real sizes
                setattr(h, name, t[:n])
        return True

    def _caps_key(self, h: LayerHandle):
        # only what every rank knows alike: the capacities decide the arena geometry, which must be the same on all ranks
        # (a rank's own token count is NOT part of the key; the maxima over ranks that feed the capacities are global)
        return (h.K, h.E, h.N)

    def _note_caps(self, h: LayerHandle, seen) -> None:
        """Capacities for the next call with the same shapes: what was seen plus a margin for the step-to-step change
        of the routing (slots in whole 128-row blocks); they only grow."""
        rmax, smax, tmax = seen
        want = (int(rmax * 1.06) + 64, (int(smax * 1.06) + 127) // 128 * 128 + 256, tmax)
        old = self._caps.get(self._caps_key(h), (0, 0, 0))
        self._caps[self._caps_key(h)] = tuple(max(a, b) for a, b in zip(old, want))

    def dispatch_gen(self, h: LayerHandle, x: torch.Tensor, topk_weights: Optional[torch.Tensor], with_meta: bool):
        """Push rows (and, with_meta, the slot / row tables) to their destination ranks.  After the
        barrier this returns the table views of this rank."""
        w = self.world
        T, H = x.shape
        K, N, E = h.K, h.N, h.E
        h.H = H
        offs, total, maxima = _arena_geometry(h.maxima, H, K)
        if self.is_cuda:
            yield ("grow", total)
        tabs = self._tables(offs, maxima, H, K, x.dtype)
        if not with_meta:      # cached handle / backward: no barrier of this call precedes the pushes
            yield from self._acquire()
        if self.is_cuda:
            ext = self.ext
            if with_meta:
                ext.slot_pad_fill(h.seg_offsets, h.expert_total_local, tabs["slot_row"], tabs["slot_w"], tabs["slot_tk"], h.mblock_expert,
                                  h.unit_blk, h.num_units, h.geom_ok if h.pending is not None else None)
            if T > 0:
                tw = topk_weights if topk_weights is not None else torch.empty(T, K, dtype=torch.float32, device=x.device)
                ext.dispatch_push(x, h.topk_idx, tw, E, N, h.send_slot, h.send_row, h.land_off,
                                  w.ptr_table(w.data, 0, "data"), [offs[n] for n in TABLES], with_meta, 0,
                                  h.geom_ok if h.pending is not None else None)
        else:
            if with_meta:
                tabs["slot_row"].fill_(-1)
                tabs["slot_w"].zero_()
                tabs["slot_tk"].fill_(-1)
                tabs["row_slots"].fill_(-1)
                tabs["row_topk_idx"].fill_(-1)
                tabs["row_topk_w"].zero_()
            yield ("push", _cpu_dispatch_writes(h, x, topk_weights, with_meta))
        self._mark("  dispatch push kernel")
        yield ("barrier",)
        self._mark("  dispatch barrier")
        return tabs, offs

    def snapshot_tables(self, h: LayerHandle, tabs) -> None:
        """Copy this rank's receive tables out of the (shared, reused) arena into the handle.  While the host has not
        read the layout sizes (fixed-shape dispatch) the copies have the capacity of the tables."""
        R, S = (h.maxima[0], h.maxima[1]) if h.pending is not None else (h.rows, h.slots)
        h.slot_row = tabs["slot_row"][:S].clone()
        h.slot_w = tabs["slot_w"][:S].clone()
        h.slot_tk = tabs["slot_tk"][:S].clone()
        h.row_slots = tabs["row_slots"][:R].clone()
        h.row_land = tabs["row_land"][:R].clone()
        h.row_tok = tabs["row_tok"][:R].clone()

    def expand(self, rows: torch.Tensor, h: LayerHandle) -> torch.Tensor:
        S, H = h.slots, rows.shape[1]
        out = torch.empty(S, H, dtype=rows.dtype, device=rows.device)
        if S == 0:
            return out
        if self.is_cuda:
            self.ext.expand_rows(rows, h.slot_row, out, S)
        else:
            sr = h.slot_row.long()
            out.copy_(torch.where((sr >= 0)[:, None], rows[sr.clamp(min=0)], torch.zeros((), dtype=rows.dtype)))
        return out

    def _combine_push(self, h: LayerHandle, y, offs, parts, with_payload=True, num_blocks=0):
        """Launch the push kernel (CUDA) or return the host writes (CPU)."""
        w = self.world
        if not self.is_cuda:
            return _cpu_combine_writes(h, y, parts, with_payload)
        if h.rows > 0:
            self.ext.combine_push(y, h.row_slots, h.row_land, h.recv_row_base, h.rows, h.N, w.ptr_table(w.data, 0, "data"),
                                  [offs[n] for n in TABLES], parts, h.slot_tk if parts is not None else None, with_payload, num_blocks)
        return None

    def _combine_reduce(self, h: LayerHandle, tabs, dtype, device, want_gtw: bool):
        T, K, H = h.T, h.K, h.H
        out = torch.empty(T, H, dtype=dtype, device=device)
        if T > 0:
            if self.is_cuda:
                self.ext.combine_reduce(tabs["landing"], h.land_off, h.ndst, out)
            else:
                land = tabs["landing"]
                lo, nd = h.land_off.long(), h.ndst.long()
                acc = torch.zeros(T, H, dtype=torch.float32)
                for j in range(int(nd.max())):
                    m = nd > j
                    acc[m] += land[(lo + j)[m]].float()
                out.copy_(acc.to(dtype))
        gtw = None
        if want_gtw:
            valid = (h.topk_idx >= 0) & (h.topk_idx < h.E)
            gtw = torch.where(valid, tabs["gtw"][:T * K].view(T, K), torch.zeros((), dtype=torch.float32, device=device))
        return out, gtw

    def combine_gen(self, h: LayerHandle, y: torch.Tensor, tabs, offs, droute_parts: Optional[torch.Tensor] = None, num_sms: int = 0):
        """Sum each received token's local expert outputs and push one row back to its source; after
        the barrier reduce the landed rows.  -> (out [T,H], gtw [T,K] or None).  num_sms > 0 limits the push kernel to
        eight blocks per SM on that many SMs (the layer call's num_combine_sms)."""
        writes = self._combine_push(h, y, offs, droute_parts, num_blocks=8 * num_sms)
        if writes is not None:
            yield ("push", writes)
        self._mark("  combine push kernel")
        yield ("barrier",)
        self._mark("  combine barrier")
        res = self._combine_reduce(h, tabs, y.dtype, y.device, droute_parts is not None)
        self._mark("  combine reduce kernel")
        return res

    def combine_rows_gen(self, h: LayerHandle, x: torch.Tensor, recv_topk_weights: Optional[torch.Tensor]):
        """Un-fused combine of one row per received token (x [rows,H]); optionally carries the
        received top-k weights back to their source entries.  -> (combined_x [T,H], weights [T,K] | None)."""
        import copy
        if not self.resolve_sizes(h):        # a handle of a fixed-shape dispatch: the sizes were copied long ago, this does not wait
            raise RuntimeError("the dispatch received more rows than num_worst_tokens allows; its outputs are not valid")
        R, K, dev = h.rows, h.K, x.device
        if x.shape[0] < R:
            raise ValueError(f"expected {R} rows (one per received token), got {x.shape[0]}")
        if x.shape[0] > R:      # fixed-shape dispatch outputs (num_worst_tokens): rows past the received count are padding
            x = x[:R]
            if recv_topk_weights is not None:
                recv_topk_weights = recv_topk_weights[:R]
        offs, total, maxima = _arena_geometry(h.maxima, x.shape[1], K)
        if self.is_cuda:
            yield ("grow", total)
        tabs = self._tables(offs, maxima, x.shape[1], K, x.dtype)
        hh = copy.copy(h)
        hh.H = x.shape[1]
        hh.row_slots = torch.full((R, K), -1, dtype=torch.int32, device=dev)
        if R:
            hh.row_slots[:, 0] = torch.arange(R, dtype=torch.int32, device=dev)
        yield from self._acquire()
        writes = [self._combine_push(hh, x.contiguous(), offs, None)]
        if recv_topk_weights is not None:
            # the side channel is indexed by slot: scatter the received weights into slot space
            rs = h.row_slots.long()
            valid = rs >= 0
            kpos = h.slot_tk.long()[rs.clamp(min=0)] % K
            rr = torch.arange(R, device=dev).view(R, 1).expand(R, K)
            parts = torch.zeros(max(h.slots, 1), 1, dtype=torch.float32, device=dev)
            parts[rs[valid], 0] = recv_topk_weights.float()[rr[valid], kpos[valid]]
            writes.append(self._combine_push(h, x.contiguous(), offs, parts, with_payload=False))
        for wri in writes:
            if wri is not None:
                yield ("push", wri)
        yield ("barrier",)
        return self._combine_reduce(hh, tabs, x.dtype, dev, recv_topk_weights is not None)

    def slots_combine_gen(self, h: LayerHandle, y: torch.Tensor, weights: Optional[torch.Tensor]):
        """One row per slot goes home to its (token,k) entry; the token's rank forms the (optionally
        weighted) sum over its valid entries.  y [slots,H] -> out [T,H]."""
        w = self.world
        T, K, N, E = h.T, h.K, h.N, h.E
        H = y.shape[1]
        offs, total, maxima = _arena_geometry(h.maxima, H, K)
        if self.is_cuda:
            yield ("grow", total)
        tabs = self._tables(offs, maxima, H, K, y.dtype)
        yield from self._acquire()
        if self.is_cuda:
            if h.slots > 0:
                self.ext.slot_rows_push(y.contiguous(), h.slot_tk, h.slot_row, h.recv_row_base, h.slots, w.ptr_table(w.data, 0, "data"),
                                        offs["landing"])
        else:
            valid = (h.slot_tk >= 0).nonzero(as_tuple=True)[0]
            rr = h.slot_row.long()[valid]
            src = torch.bucketize(rr, h.recv_row_base.long()[1:], right=True)
            writes = {}
            for s in range(N):
                m = src == s
                writes[s] = [("landing", h.slot_tk.long()[valid[m]], y[valid[m]])]
            yield ("push", writes)
        yield ("barrier",)
        out = torch.empty(T, H, dtype=y.dtype, device=y.device)
        if T == 0:
            return out
        if self.is_cuda:
            self.ext.combine_reduce_slots(tabs["landing"], h.topk_idx, E, out, weights)
        else:
            vmask = ((h.topk_idx >= 0) & (h.topk_idx < E)).float()
            ww = vmask if weights is None else vmask * weights.float()
            land = tabs["landing"][: T * K].float().view(T, K, H)
            land = torch.where(vmask.bool()[:, :, None], land, torch.zeros((), dtype=torch.float32))
            out.copy_((land * ww[:, :, None]).sum(1).to(y.dtype))
        return out

    # ------------------------------------------------------------------ layer forward / backward
    def forward_gen(self, x, topk_idx, topk_weights, W_gateup, W_down, num_experts, keep_for_backward=True, impl=None, num_sms=0):
        w = self.world
        T, H = x.shape
        El = num_experts // w.size
        if W_gateup.shape[0] != El or W_down.shape[0] != El:
            raise ValueError(f"expected {El} local experts, got W_gateup {tuple(W_gateup.shape)} W_down {tuple(W_down.shape)}")
        I = W_gateup.shape[1] // 2
        if W_gateup.shape[2] != H or tuple(W_down.shape[1:]) != (H, I):
            raise ValueError("weight shapes must be W_gateup [E_local, 2I, H] and W_down [E_local, H, I]")
        num_sms = num_sms or self._grid_sms(impl)
        self._mark("fwd:start")
        # Calls that will run as one kernel do not wait for the layout sizes: tables are sized by capacities learnt from
        # earlier calls with these shapes, and the sizes are read while the kernel runs (layout_gen, resolve_sizes).
        K0 = topk_idx.shape[1]
        caps = self._caps.get((K0, num_experts, w.size)) if (self.is_cuda and use_layer_kernel() and LAUNCH_AHEAD) else None
        h = yield from self.layout_gen(topk_idx, num_experts, caps=caps)
        self._mark("fwd:routing+layout")
        h.topk_weights = topk_weights
        st = w.status if self.is_cuda else None
        units = (h.unit_blk, h.num_units) if (self.is_cuda and USE_CTA_PAIRS and h.unit_blk is not None) else None
        # The fused dispatch kernel waits for rows that OTHER ranks' kernels send, so every rank must be running at the
        # same time: real ranks (one process per GPU) or a single rank; never the sequential launches of a virtual cluster.
        concurrent = w.size == 1 or w.virtual_peers is None
        h.fused_dispatch = bool(self.is_cuda and concurrent and use_fused_dispatch(I, w.size, h.maxima[1] * H * x.element_size())
                                and use_fused_combine(I, w.size, False)
                                and use_fused_combine(I, w.size, True))
        # which fused kernels this call uses (read by the benchmark and by Buffer.state())
        self.last_paths = {"fused_dispatch_gemm": h.fused_dispatch, "cta_pairs": bool(units is not None),
                           "fused_combine_fwd": bool(self.is_cuda and use_fused_combine(I, w.size, False)),
                           "fused_combine_bwd": bool(self.is_cuda and use_fused_combine(I, w.size, True))}
        h.layer_kernel = bool(h.fused_dispatch and use_layer_kernel())
        self.last_paths["layer_kernel"] = h.layer_kernel
        if h.layer_kernel:
            if caps is None and LAUNCH_AHEAD:
                self._note_caps(h, (h.maxima[0], h.maxima[1], h.maxima[3]))      # the next call with these shapes need not wait
            h.num_dispatch_sms = int((impl or {}).get("num_dispatch_sms", 0))
            h.opts = dict(impl or {})
            res = yield from self.layer_kernel_gen(h, 0, x, topk_weights, W_gateup, W_down, num_sms=num_sms)
            if res is None:
                # the layout outgrew the capacities: the kernels of this attempt did nothing (on every rank alike)
                return (yield from self.forward_gen(x, topk_idx, topk_weights, W_gateup, W_down, num_experts, keep_for_backward, impl, num_sms))
            out, preact, saved_x = res
            saved = SavedForBackward(h, saved_x, preact, stats=self._stats(h, H)) if keep_for_backward else None
            return out, saved
        if not self.resolve_sizes(h):        # other paths need the sizes on the host: read them, repeat if they did not fit
            return (yield from self.forward_gen(x, topk_idx, topk_weights, W_gateup, W_down, num_experts, keep_for_backward, impl, num_sms))
        if h.fused_dispatch:
            h.num_dispatch_sms = int((impl or {}).get("num_dispatch_sms", 0))
            tabs, offs, act, preact, _ = yield from self.fused_dispatch_gemm_gen(h, x, topk_weights, W_gateup, 0, num_sms=num_sms,
                                                                                 num_dispatch_sms=h.num_dispatch_sms)
            self._mark("fwd:dispatch + gate_up GEMM (one kernel)")
            R, S = h.rows, h.slots
            h.slot_row, h.slot_w, h.slot_tk = tabs["slot_row"][:S].clone(), tabs["slot_w"][:S].clone(), tabs["slot_tk"][:S].clone()
            saved_x = torch.empty(R, H, dtype=x.dtype, device=x.device)
            if R > 0:
                self.ext.expand_rows(tabs["slot_x"], tabs["row_first"], saved_x, R)     # one slot per received token
            self._mark("fwd:save tables and X")
        else:
            tabs, offs = yield from self.dispatch_gen(h, x, topk_weights, with_meta=True)
            self._mark("fwd:dispatch (rest)")
            self.snapshot_tables(h, tabs)
            saved_x = tabs["recv_x"][:h.rows].clone()
            self._mark("fwd:save tables and X")
        if h.fused_dispatch:
            pass
        elif USE_TMA_GATHER:
            act, preact = gemm.fwd_gateup(saved_x, W_gateup, h.slot_w, h.mblock_expert, h.num_mblocks, st, num_sms, gather_rows=h.slot_row)
        else:
            xperm = self.expand(saved_x, h)
            self._mark("fwd:expand")
            act, preact = gemm.fwd_gateup(xperm, W_gateup, h.slot_w, h.mblock_expert, h.num_mblocks, st, num_sms, units=units)
            del xperm
        self._mark("fwd:gate_up GEMM+SwiGLU")
        if self.is_cuda and use_fused_combine(I, w.size, False):
            gemm.fwd_down(act, W_down, h.mblock_expert, h.num_mblocks, st, num_sms, units=units, push=self._push_target(h, offs))
            del act
            self._mark("fwd:down GEMM + pushed combine")
            yield ("barrier",)
            self._mark("fwd:combine barrier")
            out = torch.empty(T, H, dtype=x.dtype, device=x.device)
            if T > 0:
                self.ext.combine_reduce_slots(tabs["landing"], h.topk_idx, h.E, out, None)
            self._mark("fwd:combine reduce (per-entry rows)")
        else:
            y = gemm.fwd_down(act, W_down, h.mblock_expert, h.num_mblocks, st, num_sms, units=units)
            del act
            self._mark("fwd:down GEMM")
            out, _ = yield from self.combine_gen(h, y, tabs, offs, num_sms=int((impl or {}).get("num_combine_sms", 0)))
            del y
        self._mark("fwd:combine (rest)")
        saved = SavedForBackward(h, saved_x, preact, stats=self._stats(h, H)) if keep_for_backward else None
        return out, saved

    def wait_report(self) -> dict:
        """Wait times of the last whole-layer kernels in ms per CTA pair (mean): how long the producers waited for
        rows of other ranks, for the first GEMM of a unit, for an expert's units (weight gradients), and how long the
        gather waited for every rank's pushes."""
        names = ("wait_arrival", "wait_first_gemm", "wait_wgrad", "wait_landed")
        rep = {}
        pairs = max(1, torch.cuda.get_device_properties(self.world.device).multi_processor_count // 2) if self.is_cuda else 1
        for kind, t in self.last_wait_ns.items():
            v = t.tolist()
            d = {n: round(v[i] / 1e6 / (pairs if i < 3 else pairs * 2), 4) for i, n in enumerate(names)}
            # when the epilogues took the first / finished the last item of every kind, relative to the first item at all
            firsts = {k: ~v[8 + k] & 0xFFFFFFFFFFFFFFFF for k in range(5) if v[8 + k] != 0}
            if firsts:
                t0 = min(firsts.values())
                kinds = ("gemm1", "gemm2", "wgrad_down", "wgrad_gateup", "reduce")
                d["spans_ms"] = {kinds[k]: (round((firsts[k] - t0) / 1e6, 3), round(((v[16 + k] & 0xFFFFFFFFFFFFFFFF) - t0) / 1e6, 3)) for k in firsts}
            rep["bwd" if kind else "fwd"] = d
        return rep

    def _stats(self, h: LayerHandle, H: int) -> dict:
        """Per-call numbers of the layer (tokens received, rows per expert, bytes that crossed NVLink)."""
        K, N = h.K, h.N
        fused = h.fused_dispatch
        return {"tokens": h.T, "rows_received": h.rows, "slots": h.slots, "per_expert_rows": h.expert_total_local,
                "paths": dict(self.last_paths),
                # bytes this rank RECEIVES per transfer: the fused paths move one row per (token, k) entry, the separate
                # kernels one row per (token, rank)
                "dispatch_bytes": (int(h.slots) if fused else int(h.rows)) * H * 2,
                "combine_bytes": (h.T * K if fused else int(h.land_rows)) * H * 2}

    def _grid_sms(self, impl) -> int:
        """`total_sms` of the layer call limits the grids of the GEMM kernels (0: all SMs of the device)."""
        total = int((impl or {}).get("total_sms", 0))
        if not self.is_cuda or total <= 0:
            return 0
        have = torch.cuda.get_device_properties(self.world.device).multi_processor_count
        return 0 if total >= have else max(4, total & ~1)

    def fused_dispatch_gemm_gen(self, h: LayerHandle, rows_in, topk_weights, weights, kind: int, preact=None, num_sms=0,
                                num_dispatch_sms=0):
        """Dispatch fused with the GEMM that consumes it (csrc/fused.cu).  kind 0: forward, rows_in = x, weights =
        W_gateup -> (act, preact); kind 1: backward, rows_in = grad_out, weights = W_down -> (act_w, dGU, route partials).
        Also returns the table views and offsets of this call."""
        w, ext = self.world, self.ext
        T, H = rows_in.shape
        K, N, E = h.K, h.N, h.E
        h.H = H
        I = weights.shape[1] // 2 if kind == 0 else weights.shape[2]
        offs, total, maxima = _arena_geometry(h.maxima, H, K, True)
        yield ("grow", total)
        tabs = self._tables(offs, maxima, H, K, rows_in.dtype)
        if kind == 1:
            yield from self._acquire()
        S = h.slots
        dev = rows_in.device
        if kind == 0:
            ext.slot_pad_fill(h.seg_offsets, h.expert_total_local, tabs["slot_row"], tabs["slot_w"], tabs["slot_tk"], h.mblock_expert,
                              h.unit_blk, h.num_units)
            h.unit_order = torch.zeros(h.unit_blk.numel(), dtype=torch.int32, device=dev)
            blk_group = torch.zeros(max(S // 128, 1), dtype=torch.int32, device=dev)
            ext.arrival_order(w.meta_view(E + N + 2), h.rank, N, E, max(1, min(FUSED_DISPATCH_GROUPS, N)), h.seg_offsets, h.unit_blk,
                              h.num_units, blk_group, h.unit_order)
        ext.zero_pad_rows(h.seg_offsets, h.expert_total_local, tabs["slot_x"])
        out0 = torch.empty(S, I, dtype=torch.bfloat16, device=dev)
        out1 = torch.empty(S, 2 * I, dtype=torch.bfloat16, device=dev)
        row_w = tabs["slot_w"] if kind == 0 else h.slot_w
        if kind == 0:
            gemm_t = [tabs["slot_x"], weights, row_w, out0, out1]
            parts = None
        else:
            parts = torch.empty(S, gemm.num_droute_parts(I), dtype=torch.float32, device=dev)
            gemm_t = [tabs["slot_x"], weights, row_w if S > 0 else torch.zeros(1, device=dev), out0, out1, preact, parts]
        send_t = [rows_in, h.topk_idx, h.send_order, h.num_send, h.send_slot.view(-1), h.send_row]
        if kind == 0:
            send_t.append(topk_weights)
        sym_t = [w.ptr_table(w.data, 0, "data"), w.ptr_table(w.control, 0, "control_base"), w.blk_cnt_view(), h.unit_order,
                 h.seg_offsets, h.expert_total_local, torch.zeros(1, dtype=torch.int32, device=dev)]
        offsets = [offs["slot_x"], offs["slot_w"], offs["slot_tk"], offs["slot_row"], offs["row_first"], w.blk_cnt_offset]
        ext.fused_dispatch_gemm(kind, gemm_t, [h.mblock_expert, h.num_mblocks, h.unit_blk, h.num_units], send_t, sym_t, offsets, E, N,
                                kind == 0, dispatch_pairs(kind, num_dispatch_sms), w.status, num_sms)
        # every row meant for this rank has arrived once the kernel is done: clear the arrival counters for the next use
        w.blk_cnt_view()[: max(S // 128, 1)].zero_()
        return tabs, offs, out0, out1, parts

    def layer_kernel_gen(self, h: LayerHandle, kind: int, rows_in, topk_weights, w1, w2, saved: Optional[SavedForBackward] = None,
                         num_sms=0):
        """One direction of the layer as ONE cooperative kernel (csrc/layer.cu) behind the routing preparation.
        kind 0: rows_in = x, w1 = W_gateup, w2 = W_down -> (out [T,H], preact, saved_x).
        kind 1: rows_in = grad_out, w1 = W_down, w2 = W_gateup -> (dx, d(topk_weights), dW_gateup, dW_down)."""
        w, ext = self.world, self.ext
        T, H = rows_in.shape
        K, N, E = h.K, h.N, h.E
        h.H = H
        bwd = kind == 1
        I = w1.shape[2] if bwd else w1.shape[1] // 2
        El = w1.shape[0]
        dev = rows_in.device
        opts = h.opts or {}
        offs, total, maxima = _arena_geometry(h.maxima, H, K, True)
        yield ("grow", total)
        tabs = self._tables(offs, maxima, H, K, rows_in.dtype)
        ahead = h.pending is not None                        # forward only: the host does not know the sizes yet
        S = h.maxima[1] if ahead else h.slots                # ... so its tensors get the capacity of the slot tables
        R = max(S, 128)                                      # rows of the tensors of this call (the kernel wants >= one block)
        ok = h.geom_ok if ahead else None
        i32 = dict(dtype=torch.int32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        if bwd:
            xperm = torch.empty(R, H, **bf)      # X back in slot space (operand of dW_gateup): filled inside the kernel
            yield from self._acquire()                       # no barrier of this call precedes the pushes
        else:
            ext.slot_pad_fill(h.seg_offsets, h.expert_total_local, tabs["slot_row"], tabs["slot_w"], tabs["slot_tk"], h.mblock_expert,
                              h.unit_blk, h.num_units, ok)
            h.unit_order = torch.zeros(h.unit_blk.numel(), **i32)
            blk_group = torch.zeros(max(S // 128, 1), **i32)
            # `stage` of the layer call: how finely units are ordered by the arrival time of their rows (stage 1: four
            # groups, stage 2: eight; the reference's stage splits every channel's tokens into that many sub-ranges)
            groups = FUSED_DISPATCH_GROUPS * max(1, int(opts.get("stage", 1)))
            ext.arrival_order(w.meta_view(E + N + 2), h.rank, N, E, max(1, min(groups, N)), h.seg_offsets, h.unit_blk,
                              h.num_units, blk_group, h.unit_order, ok)
        ext.zero_pad_rows(h.seg_offsets, h.expert_total_local, tabs["slot_x"], ok)
        out0 = torch.empty(R, I, **bf)
        out1 = torch.empty(R, 2 * I, **bf)
        out = torch.empty(T, H, **bf)
        max_units = h.unit_blk.numel() - 1
        max_work = ext.moe_layer_max_work(bwd, max_units, H, I, El, T, LAYER_REDUCE_CHUNK)
        work_t = [torch.empty(max_work * 4, **i32), torch.empty(1, **i32), torch.empty(2 * El, **i32), torch.zeros(8 + max_units, **i32)]
        layout = [h.mblock_expert, h.num_mblocks, h.unit_blk, h.num_units, h.seg_offsets, h.expert_total_local, h.unit_order]
        send_t = [rows_in, h.topk_idx, h.send_order, h.num_send, h.send_slot.view(-1), h.send_row]
        if bwd:
            parts = torch.empty(R, gemm.num_droute_parts(I), dtype=torch.float32, device=dev)
            dW_down = torch.empty(El, H, I, **bf)
            dW_gateup = torch.empty(El, 2 * I, H, **bf)
            gtw_out = torch.empty(T, K, dtype=torch.float32, device=dev)
            gemm_t = [tabs["slot_x"], w1, w2, out0, out1, h.slot_w if S > 0 else torch.zeros(R, device=dev), saved.preact, parts, xperm,
                      dW_down, dW_gateup]
            if saved.preact.shape[0] < R:
                gemm_t[6] = torch.zeros(R, 2 * I, **bf)
            push_t = [h.slot_tk, h.slot_row, h.recv_row_base] if S > 0 else [torch.full((R,), -1, **i32), torch.full((R,), -1, **i32),
                                                                             h.recv_row_base]
            red_t = [tabs["landing"], out, tabs["gtw"], gtw_out]
        else:
            send_t.append(topk_weights)
            gemm_t = [tabs["slot_x"], w1, w2, out0, out1, tabs["slot_w"]]
            push_t = [tabs["slot_tk"], tabs["slot_row"], h.recv_row_base]
            red_t = [tabs["landing"], out]
        sym_t = [w.ptr_table(w.data, 0, "data"), w.ptr_table(w.control, 0, "control_base"), w.blk_cnt_view(),
                 w.ptr_table(w.control, w.signal_offset, "control_sig"), w.control.view(w.signal_offset, [N], torch.int32)]
        offsets = [offs["slot_x"], offs["slot_w"], offs["slot_tk"], offs["slot_row"], offs["row_first"], w.blk_cnt_offset,
                   offs["landing"], offs["gtw"]]
        group_units = max(1, int(opts.get("compute_batch_size", 2048)) // UNIT_ROWS)
        lag = int(opts.get("combine_start_head_percent", 70))
        # a second-GEMM item should find its unit's first GEMM finished, not merely claimed: keep it about two items per
        # CTA pair behind (TERAMOE_LAYER_MIN_LAG: items per pair)
        sms = num_sms or torch.cuda.get_device_properties(dev).multi_processor_count
        min_lag = int(LAYER_MIN_LAG_PER_PAIR * (sms // 2))
        # per-role wait times of this launch (ns summed over waiting threads), kept on the device until somebody asks
        wait_ns = torch.zeros(24, dtype=torch.int64, device=dev)
        self.last_wait_ns[kind] = wait_ns
        wire_t = []
        if (opts.get("wire") or LAYER_WIRE) == "rank":
            wire_t = [tabs["slot_src"], torch.zeros(tabs["slot_x"].shape[0] // 128, **i32)]
            offsets.append(offs["slot_src"])
        epoch = w.next_epoch()
        if ahead and T > h.maxima[3]:
            # more tokens here than the tables were sized for: the device flag is 0 on EVERY rank (the maximum over ranks
            # exceeds the capacity), so their kernels return at once; nothing to launch, the call is repeated below
            pass
        else:
            ext.moe_layer(bwd, gemm_t, layout, send_t, sym_t, offsets, push_t, red_t, work_t, E, N, h.rank, epoch,
                          dispatch_pairs(kind, h.num_dispatch_sms), group_units, lag, min_lag, LAYER_REDUCE_CHUNK, w.status, num_sms, wait_ns,
                          saved.saved_x if (bwd and S > 0) else None, ok, wire_t)
        # every row meant for this rank has arrived once the kernel is done: clear the arrival counters for the next use
        w.blk_cnt_view()[: max(S // 128, 1)].zero_()
        if bwd:
            self._mark("bwd:layer kernel (dispatch, grad_act, dX + combine, weight gradients, reduce)")
            return out, gtw_out, dW_gateup, dW_down
        self._mark("fwd:layer kernel (dispatch, gate_up, down + combine, reduce)")
        if not self.resolve_sizes(h):
            return None
        S = h.slots
        R_rows = h.rows
        h.slot_row, h.slot_w, h.slot_tk = tabs["slot_row"][:S].clone(), tabs["slot_w"][:S].clone(), tabs["slot_tk"][:S].clone()
        saved_x = torch.empty(R_rows, H, **bf)
        if R_rows > 0:
            ext.expand_rows(tabs["slot_x"], tabs["row_first"], saved_x, R_rows)     # one slot per received token
        self._mark("fwd:save tables and X")
        return out, out1[:S] if S < R else out1, saved_x

    def _push_target(self, h: LayerHandle, offs):
        w = self.world
        return ([w.ptr_table(w.data, 0, "data"), h.slot_tk, h.slot_row, h.recv_row_base], offs["landing"])

    def backward_gen(self, saved: SavedForBackward, grad_out, W_gateup, W_down, impl=None, num_sms=0):
        w = self.world
        h = saved.handle
        El = W_gateup.shape[0]
        st = w.status if self.is_cuda else None
        num_sms = num_sms or self._grid_sms(impl)
        self._mark("bwd:start")
        if h.layer_kernel:
            return (yield from self.layer_kernel_gen(h, 1, grad_out, None, W_down, W_gateup, saved=saved, num_sms=num_sms))
        if h.fused_dispatch:
            tabs, offs, act_w, dgu, parts = yield from self.fused_dispatch_gemm_gen(h, grad_out, None, W_down, 1, preact=saved.preact,
                                                                                    num_sms=num_sms, num_dispatch_sms=h.num_dispatch_sms)
            self._mark("bwd:dispatch + grad_act GEMM (one kernel)")
            units = (h.unit_blk, h.num_units)
            dyperm = tabs["slot_x"][: h.slots]
            dxperm = None
            gemm.bwd_dx(dgu, W_gateup, h.mblock_expert, h.num_mblocks, st, num_sms, units=units, push=self._push_target(h, offs))
            if h.slots > 0:
                self.ext.droute_push(parts, h.slot_tk, h.slot_row, h.recv_row_base, h.slots, w.ptr_table(w.data, 0, "data"), offs["gtw"])
            self._mark("bwd:dX GEMM + pushed combine")
            dW_down = gemm.wgrad(dyperm, act_w, h.seg_offsets, El, st, num_sms, cta_pairs=True)
            self._mark("bwd:dW_down GEMM")
            xperm = self.expand(saved.saved_x, h)
            self._mark("bwd:expand X")
            dW_gateup = gemm.wgrad(dgu, xperm, h.seg_offsets, El, st, num_sms, cta_pairs=True)
            self._mark("bwd:dW_gateup GEMM")
            del xperm, dyperm
        else:
            tabs, offs = yield from self.dispatch_gen(h, grad_out, None, with_meta=False)
            self._mark("bwd:dispatch (rest)")
        if h.fused_dispatch:
            pass
        elif USE_TMA_GATHER:
            dy_rows = tabs["recv_x"]      # token-once rows of grad_out, read through h.slot_row by the GEMMs
            dgu, act_w, parts = gemm.bwd_gradact(dy_rows, W_down, saved.preact, h.slot_w, h.mblock_expert, h.num_mblocks, st, num_sms,
                                                 gather_rows=h.slot_row)
            dxperm = gemm.bwd_dx(dgu, W_gateup, h.mblock_expert, h.num_mblocks, st, num_sms)
            dW_down = gemm.wgrad(dy_rows, act_w, h.seg_offsets, El, st, num_sms, gather_rows=h.slot_row, gather_operand=1)
            dW_gateup = gemm.wgrad(dgu, saved.saved_x, h.seg_offsets, El, st, num_sms, gather_rows=h.slot_row, gather_operand=2)
        else:
            units = (h.unit_blk, h.num_units) if (self.is_cuda and USE_CTA_PAIRS and h.unit_blk is not None) else None
            pairs = units is not None
            dyperm = self.expand(tabs["recv_x"], h)
            self._mark("bwd:expand dY")
            dgu, act_w, parts = gemm.bwd_gradact(dyperm, W_down, saved.preact, h.slot_w, h.mblock_expert, h.num_mblocks, st, num_sms,
                                                 units=units)
            self._mark("bwd:grad_act GEMM+dSwiGLU")
            fused = self.is_cuda and use_fused_combine(W_down.shape[2], w.size, True)
            if fused:
                dxperm = None
                gemm.bwd_dx(dgu, W_gateup, h.mblock_expert, h.num_mblocks, st, num_sms, units=units, push=self._push_target(h, offs))
                if h.slots > 0:
                    self.ext.droute_push(parts, h.slot_tk, h.slot_row, h.recv_row_base, h.slots, w.ptr_table(w.data, 0, "data"), offs["gtw"])
                self._mark("bwd:dX GEMM + pushed combine")
            else:
                dxperm = gemm.bwd_dx(dgu, W_gateup, h.mblock_expert, h.num_mblocks, st, num_sms, units=units)
            self._mark("bwd:dX GEMM")
            overlap = self.is_cuda and not fused and w.size > 1 and OVERLAP_BWD_COMBINE
            if overlap:
                main, side = torch.cuda.current_stream(), w.side_stream()
                ev = torch.cuda.Event()
                ev.record(main)
                with torch.cuda.stream(side):
                    side.wait_event(ev)
                    self._combine_push(h, dxperm, offs, parts, num_blocks=OVERLAP_COMM_SMS * 8)   # 0 = full grid
                    yield ("barrier",)                       # the barrier kernel goes to the side stream too
                    pushed = torch.cuda.Event()
                    pushed.record(side)
                if OVERLAP_COMM_SMS > 0:
                    total = int((impl or {}).get("total_sms", 0)) or torch.cuda.get_device_properties(dyperm.device).multi_processor_count
                    num_sms = max(2, (total - OVERLAP_COMM_SMS) & ~1)
            dW_down = gemm.wgrad(dyperm, act_w, h.seg_offsets, El, st, num_sms, cta_pairs=pairs)
            del dyperm
            self._mark("bwd:dW_down GEMM")
            xperm = self.expand(saved.saved_x, h)
            self._mark("bwd:expand X")
            dW_gateup = gemm.wgrad(dgu, xperm, h.seg_offsets, El, st, num_sms, cta_pairs=pairs)
            self._mark("bwd:dW_gateup GEMM")
            del xperm
            if overlap:
                main.wait_event(pushed)
                del dgu, act_w
                dx, gtw = self._combine_reduce(h, tabs, grad_out.dtype, grad_out.device, True)
                dxperm.record_stream(side)
                self._mark("bwd:combine reduce (push overlapped)")
                return dx, gtw, dW_gateup, dW_down
        del dgu, act_w
        if dxperm is None and self.is_cuda and not USE_TMA_GATHER:
            # weight gradients were enqueued after the push so they overlap the other ranks' pushes
            yield ("barrier",)
            self._mark("bwd:combine barrier")
            T, K = h.T, h.K
            dx = torch.empty(T, h.H, dtype=grad_out.dtype, device=grad_out.device)
            if T > 0:
                self.ext.combine_reduce_slots(tabs["landing"], h.topk_idx, h.E, dx, None)
            valid = (h.topk_idx >= 0) & (h.topk_idx < h.E)
            gtw = torch.where(valid, tabs["gtw"][:T * K].view(T, K), torch.zeros((), dtype=torch.float32, device=dx.device))
            self._mark("bwd:combine reduce (per-entry rows)")
            return dx, gtw, dW_gateup, dW_down
        dx, gtw = yield from self.combine_gen(h, dxperm, tabs, offs, droute_parts=parts, num_sms=int((impl or {}).get("num_combine_sms", 0)))
        self._mark("bwd:combine (rest)")
        return dx, gtw, dW_gateup, dW_down


# ------------------------------------------------------------------------------------------------
# host (CPU tensor) restatements of the push kernels: produce the writes each peer receives
# ------------------------------------------------------------------------------------------------
def _cpu_dispatch_writes(h: LayerHandle, x, topk_weights, with_meta):
    T, K, N, E = h.T, h.K, h.N, h.E
    El = E // N
    idx = h.topk_idx.long()
    valid = (idx >= 0) & (idx < E)
    dst_k = torch.where(valid, idx // El, torch.full_like(idx, -1))
    hit = h.send_row >= 0
    dord = torch.cumsum(hit.long(), 1) - hit.long()
    writes = {}
    for d in range(N):
        tok = torch.nonzero(hit[:, d], as_tuple=True)[0]
        rows = h.send_row[tok, d].long()
        wl = [("recv_x", rows, x[tok])]
        if with_meta:
            m = dst_k == d
            tt, kk = torch.nonzero(m, as_tuple=True)
            slots = h.send_slot[tt, kk].long()
            wl.append(("slot_row", slots, h.send_row[tt, d]))
            wl.append(("slot_w", slots, topk_weights[tt, kk].float()))
            wl.append(("slot_tk", slots, (tt * K + kk).to(torch.int32)))
            wl.append(("row_tok", rows, tok.to(torch.int32)))
            wl.append(("row_land", rows, (h.land_off[tok].long() + dord[tok, d]).to(torch.int32)))
            pos = torch.cumsum(m.long(), 1) - m.long()
            rs = torch.full((T, K), -1, dtype=torch.int32)
            rs[tt, pos[tt, kk]] = h.send_slot[tt, kk]
            wl.append(("row_slots", rows, rs[tok]))
            here = (dst_k[tok] == d)
            wl.append(("row_topk_idx", rows, torch.where(here, idx[tok] - d * El, torch.full_like(idx[tok], -1))))
            wl.append(("row_topk_w", rows, torch.where(here, topk_weights[tok].float(), torch.zeros((), dtype=torch.float32))))
        writes[d] = wl
    return writes


def _cpu_combine_writes(h: LayerHandle, y, droute_parts, with_payload=True):
    N, K = h.N, h.K
    R = h.rows
    rs = h.row_slots.long()
    acc = torch.zeros(R, y.shape[1], dtype=torch.float32)
    if with_payload:
        for j in range(K):
            m = rs[:, j] >= 0
            acc[m] += y[rs[m, j]].float()
    acc = acc.to(y.dtype)
    base = h.recv_row_base.long()
    writes = {}
    for s in range(N):
        r0, r1 = int(base[s]), int(base[s + 1])
        wl = [("landing", h.row_land[r0:r1].long(), acc[r0:r1])] if with_payload else []
        if droute_parts is not None:
            sl = rs[r0:r1].reshape(-1)
            sl = sl[sl >= 0]
            wl.append(("gtw", h.slot_tk[sl].long(), droute_parts[sl].sum(1)))
        writes[s] = wl
    return writes
