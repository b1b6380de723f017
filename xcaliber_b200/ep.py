"""Expert-parallel execution of the fused MoE layer across the GPUs of one node.

Not in the reference (its plugin refuses TP/EP/DP != 1, vllm/xcaliber_int4_vllm/method.py:130-138).
One process per GPU. Rank g owns routed experts [g*E/G, (g+1)*E/G) (weights never move) and a
replica of the shared experts; tokens are data-parallel. Per layer call:

  1. route the local tokens over all E experts (router kernel);
  2. agree on the activation scale: local amax -> max all-reduce (4 bytes) -> XGS/XGSINV, so
     every rank quantises with the scale one GPU would have used on the whole batch;
  3. dispatch: one NCCL all-to-all of (bf16 row, local expert id, gate weight) per assignment,
     grouped by destination rank (counts exchanged first);
  4. run the local pipeline (route pack -> NVFP4 quantise -> FF1 -> FF2) on the received rows;
  5. combine: the reverse all-to-all returns one bf16 row per assignment; the home rank sums
     its k rows (+ shared-expert rows) in slot order with the combine kernel.

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


class ExpertParallelMoE:
    """The CUDA instantiation: NCCL all-to-all + the library's kernels for every compute step."""

    def __init__(self, shape, checkpoint, group=None, device="cuda"):
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

    def _local_experts(self, x_rows, e_local, w):
        return self.local.forward_routed(x_rows, e_local, w, act_scale=self._scale)

    def _shared(self, x):
        ns = self.shape.num_shared_experts
        n = x.shape[0]
        idx = torch.arange(ns, dtype=torch.int32, device=x.device).expand(n, ns).contiguous()
        w = torch.ones(n, ns, dtype=torch.bfloat16, device=x.device)
        self.shared.forward_routed(x, idx, w, act_scale=self._scale)
        # per-(token, shared expert) rows are the FF2 output rows in packed order; regather token-major
        v = self.shared.view(n)
        return v["out_rows"].index_select(0, v["topk_row"].reshape(-1).to(torch.int64))

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        idx, w = ops.router_topk(router_logits, self.shape, self.router_weights)
        scale = ops.act_amax(x)
        amax = scale[2:3].clone()
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        self._scale = ops.act_scale_from_amax(amax)
        return ep_forward(x, idx, w, self.e_local, self._local_experts, ops.combine,
                          self._shared if self.shared is not None else None, self.group)
