"""Multi-GPU checks (skipped with fewer than two GPUs): the hidden-sharded RMSNorm over NCCL against the unsharded kernel, its
one-kernel form (partials by peer stores) against the two-kernel form bit for bit, and row sharding (no collective). One process per GPU, NVLS off (a test must leave the other ranks' GPUs sound whatever
happens to one rank)."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip('torch')
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _rank(rank, world, port, T, N, out):
    import torch.distributed as dist
    from caminus_b200 import dist as D, glue, synth
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    dev = torch.device(f'cuda:{rank}'); torch.cuda.set_device(dev)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    try:
        x0, r0, w = synth.add_rms_inputs(T, N, seed=7, dtype=np.float16)
        a, b = D.col_shard(N, rank, world)
        xs = torch.from_numpy(np.ascontiguousarray(x0[:, a:b])).to(dev); rs = torch.from_numpy(np.ascontiguousarray(r0[:, a:b])).to(dev)
        norm = D.TPRmsNorm(torch.from_numpy(w[a:b].copy()).to(dev), N, 1e-6)
        x_in = xs.clone()
        h = norm(xs, rs)
        # the one-kernel form: partials exchanged by peer stores. Reference: this rank's apply kernel on the partials of all ranks
        # added in rank order (the fused kernel's order), so the comparison is bit for bit; two calls (the tag's parity alternates)
        fused = D.TPRmsNormFused(norm.nw, N, T, 1e-6)
        fused_ok = True
        for rep in range(2):
            xa = x_in.clone() if rep == 0 else (x_in * 0.5).clone()
            xb = xa.clone()
            parts = [torch.empty(T, device=dev) for _ in range(world)]
            dist.all_gather(parts, norm.partial(xa, rs).clone())
            tot = torch.zeros(T, device=dev)
            for p_ in parts: tot = tot + p_
            h_ref = norm.apply(xa, tot, d=rs)
            h_f = fused(xb, rs); fused.check()
            fused_ok = fused_ok and torch.equal(h_f, h_ref) and torch.equal(xa, xb)
        dist.barrier()
        fused.close()
        dist.barrier()
        # one exchange per rank serving two norms (a model's layers): one exported buffer, one tag sequence, calls alternating
        ex = D.TPExchange(T, device=dev)
        na, nb = D.TPRmsNormFused(norm.nw, N, exchange=ex), D.TPRmsNormFused((norm.nw * 0.5).contiguous(), N, exchange=ex)
        norm_b = D.TPRmsNorm(nb.nw, N, 1e-6)
        for rep in range(4):
            fn, two = (na, norm) if rep % 2 == 0 else (nb, norm_b)
            xa = x_in.clone(); xb = xa.clone()
            parts = [torch.empty(T, device=dev) for _ in range(world)]
            dist.all_gather(parts, two.partial(xa, rs).clone())
            tot = torch.zeros(T, device=dev)
            for p_ in parts: tot = tot + p_
            h_ref = two.apply(xa, tot, d=rs)
            h_f = fn(xb, rs); fn.check()
            fused_ok = fused_ok and torch.equal(h_f, h_ref) and torch.equal(xa, xb) and ex.tag == rep + 1
        dist.barrier()
        ex.close()
        dist.barrier()
        # the unsharded kernel on this rank's rows of the full-width batch (row sharding: no collective)
        ra, rb = D.row_shard(T, rank, world)
        xr = torch.from_numpy(x0[ra:rb].copy()).to(dev)
        hr = glue.add_rms_f16(xr, torch.from_numpy(w).to(dev), 1e-6, d=torch.from_numpy(r0[ra:rb].copy()).to(dev))
        torch.cuda.synchronize()
        gath = [None] * world
        dist.all_gather_object(gath, (a, b, xs.cpu().numpy(), h.cpu().numpy(), ra, rb, xr.cpu().numpy(), hr.cpu().numpy(), fused_ok))
        if rank == 0:
            X = np.zeros((T, N), np.float16); H = np.zeros((T, N), np.float16); XR = np.zeros((T, N), np.float16); HR = np.zeros((T, N), np.float16)
            for a_, b_, xs_, h_, ra_, rb_, xr_, hr_, _ in gath:
                X[:, a_:b_] = xs_; H[:, a_:b_] = h_; XR[ra_:rb_] = xr_; HR[ra_:rb_] = hr_
            ref = HR.astype(np.float64); ulp = np.abs(np.spacing(np.abs(HR))).astype(np.float64)
            ok = np.array_equal(X.view(np.uint16), XR.view(np.uint16)) and \
                bool((np.abs(H.astype(np.float64) - ref) <= ulp + 1e-5 * np.abs(ref).max()).all())
            out.put(ok and all(g_[-1] for g_ in gath))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_tp_rmsnorm_over_nccl_matches_the_unsharded_rows():
    import torch.multiprocessing as mp
    world = 2 if torch.cuda.device_count() < 4 else 4
    ctx = mp.get_context('spawn')
    out = ctx.Queue()
    port = _free_port()
    for N in (5120, 640 * world):                                      # shards the staged kernel takes (two ranks) and the lean one
        port = _free_port()
        procs = [ctx.Process(target=_rank, args=(r, world, port, 512, N, out)) for r in range(world)]
        for p in procs: p.start()
        for p in procs: p.join(300)
        assert all(p.exitcode == 0 for p in procs)
        assert out.get(timeout=10)
