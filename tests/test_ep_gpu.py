"""Fused expert-parallel MoE (peer-memory dispatch / combine) against the NCCL all-to-all form, 2 GPUs."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    from archlab_b200.models import moe
    from archlab_b200.ops import native
    from archlab_b200.parallel import ep

    dev = torch.device("cuda", rank)
    dim, inter, E, k, T = 256, 128, 8, 2, 96
    torch.manual_seed(0)
    ref = moe.ExpertParallelMoE(dim, inter, E, k, dist.group.WORLD, swiglu_limit=7.0, n_shared=1).to(dev)
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(std=0.05)
    ref = ref.bfloat16()
    ref.e_score_correction_bias = ref.e_score_correction_bias.float()
    buf = ep.EPBuffers(capacity=T * k * world, dim=dim, device=dev)
    fused = ep.FusedExpertParallelMoE(dim, inter, E, k, buf, swiglu_limit=7.0, n_shared=1, capacity_factor=2.0).to(dev).bfloat16()
    fused.e_score_correction_bias = fused.e_score_correction_bias.float()
    fused.load_state_dict(ref.state_dict())
    res = {}
    for it in range(2):
        g = torch.Generator(device=dev).manual_seed(10 * it + rank)
        x = torch.randn(T, dim, device=dev, generator=g).bfloat16()
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        ya, yb = ref(xa), fused(xb)
        res[f"out{it}"] = ((ya.float() - yb.float()).norm() / ya.float().norm()).item()
        go = torch.randn(T, dim, device=dev, generator=g).bfloat16()
        for m in (ref, fused):
            m.zero_grad()
        ya.backward(go)
        yb.backward(go)
        rel = lambda a, b: ((a.float() - b.float()).norm() / a.float().norm().clamp_min(1e-9)).item()
        res[f"dx{it}"] = rel(xa.grad, xb.grad)
        res[f"drouter{it}"] = rel(ref.router.grad, fused.router.grad)
        res[f"ddown{it}"] = rel(ref.experts.down.grad, fused.experts.down.grad)
        res[f"dgate_up{it}"] = rel(ref.experts.gate_up.grad, fused.experts.gate_up.grad)
    # the device-planned layer (fixed row bound, tile and reduction tables on the device) never waits for the GPU
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    fused.zero_grad()
    try:
        xs = x.clone().requires_grad_(True)
        ys = fused(xs)
        ys.backward(go)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    res["sync_free_out"] = ((ys.float() - yb.float()).abs().max()).item()          # same inputs as the last iteration
    res["ample_bound_drops_nothing"] = float(buf.check_overflow()["dropped_rows"])
    # the host-planned form (exact sizes read back) gives the same numbers
    exact = ep.FusedExpertParallelMoE(dim, inter, E, k, buf, swiglu_limit=7.0, n_shared=1, capacity_factor=None).to(dev).bfloat16()
    exact.e_score_correction_bias = exact.e_score_correction_bias.float()
    exact.load_state_dict(fused.state_dict())
    xe = x.clone().requires_grad_(True)
    ye = exact(xe)
    ye.backward(go)
    res["host_planned_out"] = ((ye.float() - yb.float()).abs().max()).item()
    res["host_planned_ddown"] = ((exact.experts.down.grad.float() - fused.experts.down.grad.float()).abs().max()).item()
    res["host_planned_dgate_up"] = ((exact.experts.gate_up.grad.float() - fused.experts.gate_up.grad.float()).abs().max()).item()
    # a bound that is too small is reported, not silently computed
    local = E // world
    shrink = -((local - 1) * 256) / (T * k)                              # leaves a bound of exactly one 256-row tile
    tight = ep.FusedExpertParallelMoE(dim, inter, E, k, buf, swiglu_limit=7.0, n_shared=1, capacity_factor=shrink).to(dev).bfloat16()
    tight.e_score_correction_bias = tight.e_score_correction_bias.float()
    tight.load_state_dict(fused.state_dict())
    with torch.no_grad():
        tight.router.zero_()
        tight.e_score_correction_bias[: k] += 10.0                       # every token to the first k experts: rank 0 overflows
        exact.load_state_dict(tight.state_dict())
        exact.e_score_correction_bias = tight.e_score_correction_bias.clone()
        y_tight, y_exact = tight(x), exact(x)
    info = buf.check_overflow()                                          # collective: the same verdict on every rank
    res["overflow_reported"] = 0.0 if info["dropped_rows"] > 0 else 1.0
    res["dropped_output_finite"] = 0.0 if bool(torch.isfinite(y_tight).all()) else 1.0
    kept_all = tight._last_keep.bool().all(1)
    res["some_tokens_dropped"] = 0.0 if (world == 1 or bool((~kept_all).any()) or rank != 0) else 1.0
    if bool(kept_all.any()):                                              # tokens that lost no slot are computed exactly
        res["kept_tokens_exact"] = (y_tight[kept_all].float() - y_exact[kept_all].float()).abs().max().item()
    lost = ~kept_all
    if bool(lost.any()):                                                  # the others lost (part of) their expert sum
        res["dropped_tokens_differ"] = 0.0 if (y_tight[lost].float() - y_exact[lost].float()).abs().max().item() > 1e-3 else 1.0
    torch.cuda.synchronize()
    native.check_status()
    torch.save(res, os.path.join(out_dir, f"ep_rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [pytest.param(w, marks=pytest.mark.skipif(torch.cuda.device_count() < w, reason=f"needs {w} GPUs"))
                                   for w in (2, 4, 8)])
def test_fused_ep_moe_matches_all_to_all(tmp_path, world):
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, world, 29641 + world, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    from conftest import join_ranks

    join_ranks(procs)
    for r in range(world):
        res = torch.load(tmp_path / f"ep_rank{r}.pt")
        for key, v in res.items():
            assert v < 3e-2, (r, key, v)
