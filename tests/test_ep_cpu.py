"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2): dispatch planning, the two
all-to-alls and the slot-ordered combine, with a stand-in for the per-rank expert compute."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from xcaliber_b200 import ep


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_fn_factory(rank, e_local, h):
    # "expert e" multiplies by (global_e + 1) and adds e: cheap, and different per expert
    def fn(x_rows, e_loc, w):
        ge = (e_loc.reshape(-1).float() + rank * e_local)
        return (x_rows.float() * (ge + 1)[:, None] + ge[:, None]) * w.float()
    return fn


def _combine(rows, topk_row):
    return rows[topk_row.long()].sum(dim=1)


def _worker(rank, world, port, n_shared, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        n, h, e, k = 13 + rank * 5, 8, 6, 3
        e_local = e // world
        x = torch.randn(n, h)
        idx = torch.stack([torch.randperm(e)[:k] for _ in range(n)]).to(torch.int32)
        w = torch.rand(n, k)
        shared = (lambda xx: torch.cat([xx.float() * 0.5 + s for s in range(n_shared)], dim=1).reshape(n * n_shared, h)) \
            if n_shared else None
        y = ep.ep_forward(x, idx, w, e_local, _expert_fn_factory(rank, e_local, h), _combine, shared)
        exp = torch.zeros(n, h)
        for s in range(k):
            ge = idx[:, s].float()
            exp += (x * (ge + 1)[:, None] + ge[:, None]) * w[:, s:s + 1]
        for s in range(n_shared):
            exp += x * 0.5 + s
        results[rank] = float((y - exp).abs().max())
        # planning invariants
        plan = ep.plan_dispatch(idx, e_local, world)
        assert int(plan.send_counts.sum()) == n * k
        dest = (idx.reshape(-1)[plan.send_order] // e_local)
        assert (dest[1:] >= dest[:-1]).all()
        assert (plan.send_order[plan.slot_pos.reshape(-1).long()] == torch.arange(n * k)).all()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_shared", [0, 1])
def test_ep_exchange_world2(n_shared):
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, n_shared, results), nprocs=world, join=True)
        assert len(results) == world
        assert max(results.values()) < 1e-5


def _failing_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            results[rank] = "left before the exchange"
            return  # this rank never joins the all-to-all
        try:
            ep.exchange_counts(torch.tensor([1, 1]), device="cpu")
            results[rank] = "no error"
        except Exception as exc:  # the survivor must see an error, not hang
            results[rank] = f"error: {type(exc).__name__}"
    finally:
        # no orderly teardown: with the peer gone, gloo's own shutdown may abort the process, which would
        # hide the result recorded above
        os._exit(0)


def test_ep_rank_leaving_is_detected():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        try:
            mp.spawn(_failing_worker, args=(world, port, results), nprocs=world, join=True)
        except Exception:  # a worker killed by the transport counts as detected, as long as nobody reported success
            pass
        assert results.get(0, "error: process ended").startswith("error")


def test_local_token_tile_rule():
    # the owner-side token tile follows the library's own rule applied to the rows a rank expects
    from xcaliber_b200.ep import local_token_tile

    assert local_token_tile(16 * 2, 4) == 32          # decode: 8 rows per expert
    assert local_token_tile(128 * 2, 8) == 128        # 32 rows per expert
    assert local_token_tile(4096 * 2, 4) == 128       # prefill
    assert local_token_tile(40, 2) == 32              # 20 rows per expert: below the 24-row mark
    assert local_token_tile(60, 1) == 128
