"""Worker for tests/test_gpu_ep.py: run under torch.distributed.run with 2+ ranks (NCCL).
Every rank runs the expert-parallel layer on its own tokens, once per transport (peer memory and
NCCL; they must agree bit for bit), and compares with the single-GPU layer holding all experts. Routing, activation scale and FF1 rows are the same bits on both paths;
FF2 adds its K stages in an order that depends on the token tile (small tiles accumulate in several
partial sums), so the outputs may differ by a rounding step of bf16: max relative difference 1e-2
(relative to max(|ref|, rms)), mean 1e-3."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from xcaliber_b200 import ops, synth  # noqa: E402
from xcaliber_b200.ep import ExpertParallelMoE  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    failures = []
    # toy; DeepSeek-V3-like routing (groups, bias, shared expert) without and with the activation top-k; a gpt-oss-like
    # shape (clamped SwiGLU, partial tiles); a shape whose FF2 runs on CTA pairs with rows stored at their home ranks
    cases = [("toy", dict(), 96),
             ("dsv3", dict(hidden=512, inter=256, num_experts=64, act_topk_keep=0), 80),
             ("dsv3", dict(hidden=512, inter=256, num_experts=64, act_topk_keep=64), 72),
             ("gptoss", dict(hidden=704, inter=352, num_experts=32), 100),
             ("toy", dict(hidden=512, inter=2048), 512)]
    for name, kw, n in cases:
        shape = synth.scaled_shape(synth.SHAPES[name], **kw)
        ck = synth.make_weights(shape, seed=0, device="cpu")
        xs, ls = [], []
        for r in range(world):
            x, lg = synth.make_inputs(shape, ck, n + 8 * r, seed=r)
            xs.append(x)
            ls.append(lg)
        ys = {}
        # peer: NVFP4 dispatch + FF2 stores rows at their home rank; peer-bf16: bf16 dispatch; peer-copy: also a
        # separate return kernel
        for transport in ("peer", "peer-bf16", "peer-copy", "nccl"):
            ep = ExpertParallelMoE(shape, ck, device=dev, transport=transport.split("-")[0], max_tokens=max(128, n + 8 * world),
                                   fused_return=transport != "peer-copy", quantised_dispatch=transport == "peer")
            for _ in range(3):  # repeated calls reuse the exchange buffers and their flags
                ys[transport] = ep.forward(xs[rank].to(dev), ls[rank].to(dev))
            torch.cuda.synchronize()
            if ep.peer is not None and ep.peer.status():
                failures.append(f"{name}: rank {rank} peer exchange status {ep.peer.status():#x}")
        if not all(torch.equal(ys[t], ys["nccl"]) for t in ("peer", "peer-bf16", "peer-copy")):
            failures.append(f"{name}: rank {rank} peer and nccl transports differ")
        y = ys["peer"]
        # single-GPU reference on the concatenation of all ranks' tokens (same global amax)
        pw = ops.PreparedWeights.from_checkpoint(shape, ck.w13_packed, ck.w13_scale, ck.w13_gs, ck.w2_qweight,
                                                 ck.w2_scales, router_bias=ck.router_bias, device=dev)
        full = ops.FusedMoE(shape, pw)
        y_all = full.forward(torch.cat(xs).to(dev), torch.cat(ls).to(dev))
        off = sum(t.shape[0] for t in xs[:rank])
        ref = y_all[off:off + xs[rank].shape[0]]
        yf, rf = y.float(), ref.float()
        rel = (yf - rf).abs() / torch.maximum(rf.abs(), rf.pow(2).mean().sqrt())
        if not (rel.max().item() <= 1e-2 and rel.mean().item() <= 1e-3):
            failures.append(f"{name}: rank {rank} rel diff max {rel.max().item():.3g} mean {rel.mean().item():.3g}")
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("EP_CHECK", "OK" if flag.item() == 0 else "FAIL", failures)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 0 else 1)


if __name__ == "__main__":
    main()
