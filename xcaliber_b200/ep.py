"""Expert-parallel execution of the fused MoE layer across the GPUs of one node.

Not in the reference (its plugin refuses TP/EP/DP != 1, vllm/xcaliber_int4_vllm/method.py:130-138).
One process per GPU. Rank g owns routed experts [g*E/G, (g+1)*E/G) (weights never move) and a
replica of the shared experts; tokens are data-parallel. Per layer call:

  1. route the local tokens over all E experts (router kernel);
  2. agree on the activation scale: local amax -> max all-reduce (4 bytes) -> XGS/XGSINV, so
     every rank quantises with the scale one GPU would have used on the whole batch;
  3. dispatch: each (token, slot) row travels to the owner rank with (local expert id, gate weight):
     by default as kernels that store straight into the owner's receive buffer over NVLink peer
     memory, positions agreed through a device-side count table (no host synchronisation,
     csrc/ep_p2p.cu); with transport="nccl" as one NCCL all-to-all grouped by destination rank
     (counts exchanged first, one host read);
  4. run the local pipeline (route pack -> NVFP4 quantise -> FF1 -> FF2) on the received rows;
  5. combine: one bf16 row per assignment returns to its home rank (peer transport: the FF2 epilogue
     stores it straight into the home rank's buffer; NCCL transport: the reverse all-to-all); the home
     rank sums its k rows (+ shared-expert rows) in slot order with the combine kernel.

The planning helpers are device-agnostic torch index arithmetic so that the exchange logic
can be tested on CPU ranks with the gloo backend and a stand-in for step 4.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist


@dataclasses.dataclass
class DispatchPlan:
    send_order: torch.Tensor    # i64 [N*k]: flat (token*k + slot) indices sorted by destination rank (stable)
    send_counts: torch.Tensor   # i32 [world] rows sent to each rank (device)
    slot_pos: torch.Tensor      # i32 [N, k]: position of (token, slot) in send order
    local_expert: torch.Tensor  # i32 [N*k] in send order: expert id relative to the owner rank


def plan_dispatch(topk_idx: torch.Tensor, experts_per_rank: int, world: int) -> DispatchPlan:
    """topk_idx [N, k] global expert ids -> grouping of the N*k assignments by owner rank.
    Stable counting sort over the (few) ranks with a one-hot running sum: no device sort."""
    n, k = topk_idx.shape
    flat = topk_idx.reshape(-1).to(torch.int64)
    dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
    onehot = (dest.unsqueeze(1) == torch.arange(world, device=flat.device).unsqueeze(0)).to(torch.int32)
    running = onehot.cumsum(0)                                   # [N*k, world], inclusive
    counts = running[-1] if n * k else torch.zeros(world, dtype=torch.int32, device=flat.device)
    starts = counts.cumsum(0) - counts
    pos = (starts[dest] + running.gather(1, dest.unsqueeze(1)).squeeze(1) - 1).to(torch.int32)
    order = torch.empty(n * k, dtype=torch.int64, device=flat.device)
    order[pos.long()] = torch.arange(n * k, dtype=torch.int64, device=flat.device)
    local = (flat - dest * experts_per_rank)[order].to(torch.int32)
    return DispatchPlan(order, counts, pos.reshape(n, k), local)


def exchange_counts(send_counts, group=None, device="cpu") -> tuple[list[int], list[int]]:
    """One collective and one host read: every rank learns the whole send-count matrix.
    Returns (send_counts, recv_counts) as host lists."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    s = torch.as_tensor(send_counts, dtype=torch.int64, device=device).reshape(world)
    parts = [torch.empty(world, dtype=torch.int64, device=device) for _ in range(world)]
    dist.all_gather(parts, s.contiguous(), group=group)
    host = torch.stack(parts).tolist()
    return host[rank], [host[r][rank] for r in range(world)]


def all_to_all_rows(rows: torch.Tensor, send_counts: list[int], recv_counts: list[int], group=None) -> torch.Tensor:
    out = torch.empty((sum(recv_counts),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts,
                           group=group)
    return out


def ep_forward(x, topk_idx, topk_w, experts_per_rank, local_experts_fn, combine_fn, shared_fn=None, group=None):
    """The exchange skeleton (steps 3-5). local_experts_fn(x_rows, local_expert_i32 [M,1], weight [M,1]) -> rows
    [M,H]; shared_fn(x) -> rows [N*n_shared, H] (token-major) or None; combine_fn(rows, topk_row) -> y [N,H]."""
    world = dist.get_world_size(group)
    n, k = topk_idx.shape
    plan = plan_dispatch(topk_idx, experts_per_rank, world)
    send_counts, recv_counts = exchange_counts(plan.send_counts, group, device=x.device)
    tok = torch.div(plan.send_order, k, rounding_mode="floor")
    x_send = x.index_select(0, tok)
    # (local expert id, gate weight) travel together: one int32 pair per row
    w_send = topk_w.reshape(-1)[plan.send_order]
    x_recv = all_to_all_rows(x_send, send_counts, recv_counts, group)
    if topk_w.element_size() == 2:
        meta = torch.stack([plan.local_expert, w_send.view(torch.int16).to(torch.int32)], dim=1)
        meta_recv = all_to_all_rows(meta, send_counts, recv_counts, group)
        e_recv = meta_recv[:, 0].contiguous()
        w_recv = meta_recv[:, 1].to(torch.int16).view(topk_w.dtype)
    else:
        e_recv = all_to_all_rows(plan.local_expert, send_counts, recv_counts, group)
        w_recv = all_to_all_rows(w_send, send_counts, recv_counts, group)
    y_recv = local_experts_fn(x_recv, e_recv.reshape(-1, 1), w_recv.reshape(-1, 1))
    n_sh_rows = 0
    y_sh = shared_fn(x) if shared_fn is not None else None
    if y_sh is not None:
        n_sh_rows = y_sh.shape[0]
    rows = torch.empty(n * k + n_sh_rows, x.shape[1], dtype=y_recv.dtype, device=x.device)
    dist.all_to_all_single(rows[: n * k], y_recv.contiguous(), output_split_sizes=send_counts,
                           input_split_sizes=recv_counts, group=group)
    topk_row = plan.slot_pos
    if y_sh is not None:
        rows[n * k:] = y_sh
        n_shared = n_sh_rows // n
        sh_pos = (n * k + torch.arange(n * n_shared, dtype=torch.int32, device=x.device)).reshape(n, n_shared)
        topk_row = torch.cat([topk_row, sh_pos], dim=1).contiguous()
    return combine_fn(rows, topk_row.contiguous())


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


class PeerExchange:
    """Exchange buffers of the peer-memory transport: one symmetric allocation per rank, mapped by
    every rank of the group (torch symmetric memory does the handle exchange; the library only sees
    plain device pointers), plus the per-call scratch, all sized once for `max_tokens`."""

    def __init__(self, shape, e_local: int, max_tokens: int, device, group=None):
        import ctypes as C

        import torch.distributed._symmetric_memory as symm

        from . import _lib

        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > _lib.EP_MAX_WORLD:
            raise RuntimeError(f"peer-memory exchange supports at most {_lib.EP_MAX_WORLD} ranks")
        k, h = shape.top_k, shape.hidden
        self.max_tokens = max_tokens
        self.cap_rows = _round_up(self.world * max_tokens * k, 128)
        self.ret_cap = max_tokens * (k + shape.num_shared_experts)
        sizes = dict(ctl=_lib.EP_CTL_BYTES, recv_x=self.cap_rows * h * 2, recv_meta=self.cap_rows * 16,
                     ret_rows=self.ret_cap * h * 2)
        offs, total = {}, 0
        for name, nbytes in sizes.items():
            offs[name] = total
            total += _round_up(nbytes, 1024)
        pg = group if group is not None else dist.group.WORLD
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buf, pg.group_name)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's control block is zero before anyone posts to it
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        b = _lib.XMoEEpBuffers()
        b.world, b.rank, b.hidden, b.experts_per_rank = self.world, self.rank, h, e_local
        b.cap_rows, b.ret_cap = self.cap_rows, self.ret_cap
        for r in range(self.world):
            b.ctl[r] = ptrs[r] + offs["ctl"]
            b.recv_x[r] = ptrs[r] + offs["recv_x"]
            b.recv_meta[r] = ptrs[r] + offs["recv_meta"]
            b.ret_rows[r] = ptrs[r] + offs["ret_rows"]
        self.c_buffers = b
        self.ref = C.byref(b)

        def local(name, dtype, *dims):
            return self.buf[offs[name]: offs[name] + sizes[name]].view(dtype).reshape(*dims)

        self.recv_x = local("recv_x", torch.bfloat16, self.cap_rows, h)
        self.ret_rows = local("ret_rows", torch.bfloat16, self.ret_cap, h)
        e = self.world * e_local
        i32 = dict(dtype=torch.int32, device=device)
        r_cap = max_tokens * k + 128 * e
        self.counts = torch.zeros(e, **i32)
        self.offsets = torch.zeros(e + 1, **i32)
        self.topk_off = torch.zeros(max_tokens, k, **i32)
        self.topk_row = torch.zeros(max_tokens, k, **i32)
        self.row_token = torch.zeros(r_cap, **i32)
        self.row_weight = torch.zeros(r_cap, dtype=torch.bfloat16, device=device)
        self.pack_scratch = torch.zeros(max(1, _lib.lib().xmoe_route_pack_scratch_bytes(max_tokens, e, 0)),
                                        dtype=torch.uint8, device=device)
        self.pack_status = torch.zeros(1, **i32)
        self.amax_global = torch.zeros(1, dtype=torch.float32, device=device)
        self.e_recv = torch.zeros(self.cap_rows, 1, **i32)
        self.w_recv = torch.zeros(self.cap_rows, 1, dtype=torch.bfloat16, device=device)
        self.n_recv = torch.zeros(1, **i32)
        self.home_slots = {}

    def slots(self, n: int, k_eff: int, device) -> torch.Tensor:
        """topk_row of the home-side combine: row (token * k + slot), shared-expert rows after n * k."""
        key = (n, k_eff)
        t = self.home_slots.get(key)
        if t is None:
            k = self.topk_off.shape[1]
            routed = torch.arange(n * k, dtype=torch.int32, device=device).reshape(n, k)
            if k_eff > k:
                ns = k_eff - k
                sh = (n * k + torch.arange(n * ns, dtype=torch.int32, device=device)).reshape(n, ns)
                routed = torch.cat([routed, sh], dim=1)
            t = self.home_slots[key] = routed.contiguous()
        return t

    def status(self) -> int:
        import ctypes as C

        from . import _lib
        from .ops import _stream

        bits = C.c_uint32(0)
        _lib.check(_lib.lib().xmoe_ep_status(self.ref, _stream(), C.byref(bits)), "xmoe_ep_status")
        return bits.value


def local_token_tile(rows: int, e_local: int) -> int:
    """Token tile of the local pipeline from the rows a rank expects under balanced routing (the
    library's own choice would see the receive buffer's capacity, world times larger): the library's rule,
    128 from about 24 rows per expert on average, else 32."""
    return 128 if rows / max(e_local, 1) >= 24.0 else 32


class ExpertParallelMoE:
    """The CUDA instantiation. transport="peer" (default): the exchange runs as kernels over peer
    memory with no host synchronisation; transport="nccl": NCCL all-to-all with host-side counts."""

    def __init__(self, shape, checkpoint, group=None, device="cuda", transport: str = "peer",
                 max_tokens: int = 4096, fused_return: bool = True, quantised_dispatch: bool = True):
        from . import ops
        from .synth import scaled_shape

        self.ops = ops
        self.shape = shape
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if shape.num_experts % self.world:
            raise RuntimeError("num_experts must divide evenly across the expert-parallel ranks")
        self.e_local = shape.num_experts // self.world
        e0, e1 = self.rank * self.e_local, (self.rank + 1) * self.e_local
        sl = slice(e0, e1)
        local_shape = scaled_shape(shape, num_experts=self.e_local, top_k=1, num_shared_experts=0, n_group=1,
                                   topk_group=1, router_bias=False, zipf_bias=0.0)
        pw = ops.PreparedWeights.from_checkpoint(local_shape, checkpoint.w13_packed[sl], checkpoint.w13_scale[sl],
                                                 checkpoint.w13_gs[sl], checkpoint.w2_qweight[sl],
                                                 checkpoint.w2_scales[sl], device=device)
        self.local = ops.FusedMoE(local_shape, pw)
        self._local_shape, self._local_pw, self._local_by_tile, self._local_ptrs = local_shape, pw, {}, {}
        if transport not in ("peer", "nccl"):
            raise ValueError("transport must be 'peer' or 'nccl'")
        self.transport = transport
        self.max_tokens = max_tokens
        import os

        # peer transport: FF2 writes its rows into the home ranks' buffers / tokens travel as NVFP4 packets
        # (XMOE_EP_FUSED_RETURN=0 / XMOE_EP_QUANTISED_DISPATCH=0 switch them off for comparisons)
        self.fused_return = fused_return and os.environ.get("XMOE_EP_FUSED_RETURN", "1") != "0"
        self.quantised_dispatch = quantised_dispatch and os.environ.get("XMOE_EP_QUANTISED_DISPATCH", "1") != "0"
        self._row_dst = {}
        self.peer = PeerExchange(shape, self.e_local, max_tokens, torch.device(device), group) \
            if transport == "peer" else None
        # router state lives with the full expert count
        self.router_weights = ops.PreparedWeights(
            pw.w13_packed, pw.w13_sf, pw.w13_gs, pw.w2_q, pw.w2_scale,
            None if checkpoint.router_bias is None else checkpoint.router_bias.to(device).float().contiguous(), None,
            ops.sigmoid_lut(device) if (checkpoint.router_bias is not None or shape.n_group > 1) else None)
        self.shared = None
        if shape.num_shared_experts:
            ns = shape.num_shared_experts
            sh = slice(shape.num_experts, shape.num_experts + ns)
            sh_shape = scaled_shape(shape, num_experts=ns, top_k=ns, num_shared_experts=0, n_group=1, topk_group=1,
                                    router_bias=False, zipf_bias=0.0)
            spw = ops.PreparedWeights.from_checkpoint(sh_shape, checkpoint.w13_packed[sh], checkpoint.w13_scale[sh],
                                                      checkpoint.w13_gs[sh], checkpoint.w2_qweight[sh],
                                                      checkpoint.w2_scales[sh], device=device)
            self.shared = ops.FusedMoE(sh_shape, spw)
        self._scale = None
        self._phase_events = None  # set by profile_phases(True): CUDA events between the phases of every call

    # -- optional per-phase timing (benchmarks) ---------------------------------------------------------
    PHASES = ("route", "dispatch", "shared", "wait_data", "local", "wait_ret", "combine")

    def profile_phases(self, on: bool) -> None:
        """Record a CUDA event at every phase boundary of the following peer-transport calls."""
        self._phase_events = [] if on else None

    def phase_ms(self) -> dict:
        """Mean milliseconds per phase over the recorded calls (synchronises); clears the record."""
        calls, self._phase_events = self._phase_events or [], []
        torch.cuda.synchronize()
        out = {name: 0.0 for name in self.PHASES}
        for marks in calls:
            for name, a, b in zip(self.PHASES, marks[:-1], marks[1:]):
                out[name] += a.elapsed_time(b)
        return {k: v / max(len(calls), 1) for k, v in out.items()}

    def _mark(self, marks):
        if marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append(ev)

    def _local_layer(self, home_tokens: int):
        """The local pipeline with the token tile fixed from this rank's own batch (both transports
        use the same rule, so they run the same kernels)."""
        tile = local_token_tile(home_tokens * self.shape.top_k, self.e_local)
        local = self._local_by_tile.get(tile)
        if local is None:
            local = self._local_by_tile[tile] = self.ops.FusedMoE(self._local_shape, self._local_pw, token_tile=tile)
        return tile, local

    def _local_experts(self, x_rows, e_local, w):
        return self._local_layer(self._home_tokens)[1].forward_routed(x_rows, e_local, w, act_scale=self._scale)

    def _shared_routing(self, n: int, device):
        """Every token to every shared expert with weight 1 (cached per batch size)."""
        key = ("shared_routing", n)
        cached = self._row_dst.get(key)
        if cached is None:
            ns = self.shape.num_shared_experts
            idx = torch.arange(ns, dtype=torch.int32, device=device).expand(n, ns).contiguous()
            cached = self._row_dst[key] = (idx, torch.ones(n, ns, dtype=torch.bfloat16, device=device))
        return cached

    def _shared(self, x):
        ns = self.shape.num_shared_experts
        n = x.shape[0]
        idx = torch.arange(ns, dtype=torch.int32, device=x.device).expand(n, ns).contiguous()
        w = torch.ones(n, ns, dtype=torch.bfloat16, device=x.device)
        self.shared.forward_routed(x, idx, w, act_scale=self._scale)
        # per-(token, shared expert) rows are the FF2 output rows in packed order; regather token-major
        v = self.shared.view(n)
        return v["out_rows"].index_select(0, v["topk_row"].reshape(-1).to(torch.int64))

    def _forward_peer(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """Steps 1-5 with the exchange as kernels over peer memory: nothing here waits on the host."""
        from . import _lib
        from .ops import _stream

        ops, px, lib = self.ops, self.peer, _lib.lib()
        n, k = x.shape[0], self.shape.top_k
        if n > px.max_tokens:
            raise RuntimeError(f"{n} tokens exceed the exchange buffers (max_tokens={px.max_tokens})")
        x = x.contiguous()
        marks = [] if self._phase_events is not None else None
        self._mark(marks)
        idx, w = ops.router_topk(router_logits, self.shape, self.router_weights)
        scale_local = ops.act_amax(x)
        st = _stream()
        e = self.shape.num_experts
        _lib.check(lib.xmoe_route_pack(idx.data_ptr(), w.data_ptr(), n, e, k, k, 0, px.pack_scratch.data_ptr(),
                                       px.counts.data_ptr(), px.offsets.data_ptr(), px.topk_off.data_ptr(),
                                       px.topk_row.data_ptr(), px.row_token.data_ptr(), px.row_weight.data_ptr(),
                                       px.pack_status.data_ptr(), st), "xmoe_route_pack")
        _lib.check(lib.xmoe_ep_post_counts(px.ref, px.counts.data_ptr(), scale_local[2:3].data_ptr(), st),
                   "xmoe_ep_post_counts")
        self._mark(marks)
        quantised = self.fused_return and self.quantised_dispatch
        dispatch = lib.xmoe_ep_dispatch_quantised if quantised else lib.xmoe_ep_dispatch
        _lib.check(dispatch(px.ref, x.data_ptr(), idx.data_ptr(), w.data_ptr(), px.topk_off.data_ptr(),
                            px.counts.data_ptr(), n, k, k, px.amax_global.data_ptr(), st), "xmoe_ep_dispatch")
        self._scale = ops.act_scale_from_amax(px.amax_global)
        self._mark(marks)
        k_eff = k
        if self.shared is not None:
            # the replicated shared experts run on the home tokens while the other ranks' rows are still arriving;
            # their FF2 epilogue writes each row where the final combine reads it (after the n * k routed slots)
            ns = self.shape.num_shared_experts
            sh_idx, sh_w = self._shared_routing(n, x.device)
            self.shared.forward_scatter(x, px.ret_rows[n * k:], topk_idx=sh_idx, topk_w=sh_w, act_scale=self._scale)
            k_eff = k + ns
        self._mark(marks)
        _lib.check(lib.xmoe_ep_wait_data(px.ref, px.e_recv.data_ptr(), px.w_recv.data_ptr(), px.n_recv.data_ptr(), st),
                   "xmoe_ep_wait_data")
        self._mark(marks)
        tile, local = self._local_layer(n)
        if self.fused_return:
            # the FF2 epilogue stores each row at its home rank; no separate return copy
            import ctypes as C

            ws = local.workspace(px.cap_rows)
            scratch = self._row_dst.get(tile)
            if scratch is None:
                rows = lib.xmoe_packed_rows(C.byref(local.cfg), px.cap_rows)
                scratch = self._row_dst[tile] = torch.zeros(rows, dtype=torch.int64, device=x.device)
            _lib.check(lib.xmoe_ep_forward_local(px.ref, C.byref(local.cfg), C.byref(local._wstruct),
                                                 px.e_recv.data_ptr(), px.w_recv.data_ptr(), self._scale.data_ptr(),
                                                 px.n_recv.data_ptr(), int(quantised), scratch.data_ptr(), ws.data_ptr(),
                                                 ws.numel(), st), "xmoe_ep_forward_local")
        else:
            local.forward_routed_rows(px.recv_x, px.e_recv, px.w_recv, act_scale=self._scale, n_valid=px.n_recv)
            ptrs = self._local_ptrs.get(tile)
            if ptrs is None:
                v = local.view(px.cap_rows)
                ptrs = self._local_ptrs[tile] = (v["out_rows"].data_ptr(), v["topk_row"].data_ptr())
            _lib.check(lib.xmoe_ep_return(px.ref, ptrs[0], ptrs[1], n * k, st), "xmoe_ep_return")
        self._mark(marks)
        _lib.check(lib.xmoe_ep_wait_ret(px.ref, st), "xmoe_ep_wait_ret")
        self._mark(marks)
        y = ops.combine(px.ret_rows, px.slots(n, k_eff, x.device))
        self._mark(marks)
        if marks is not None:
            self._phase_events.append(marks)
        return y

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        if self.peer is not None:
            return self._forward_peer(x, router_logits)
        ops = self.ops
        self._home_tokens = x.shape[0]
        idx, w = ops.router_topk(router_logits, self.shape, self.router_weights)
        scale = ops.act_amax(x)
        amax = scale[2:3].clone()
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        self._scale = ops.act_scale_from_amax(amax)
        return ep_forward(x, idx, w, self.e_local, self._local_experts, ops.combine,
                          self._shared if self.shared is not None else None, self.group)
