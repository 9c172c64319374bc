"""The multi-rank host logic on CPU: two gloo ranks run the hidden-sharded RMSNorm's sequence (partial -> all-reduce ->
apply) with the kernels replaced by the CPU oracle's restatements of them, and two ranks split token rows with no
communication at all. Only the rank plumbing of caminus_b200.dist is under test here; the kernels have their GPU tests."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip('torch')
import torch.distributed as dist   # noqa: E402
import torch.multiprocessing as mp   # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _rank(rank, world, port, T, N, out):
    import oracle
    from caminus_b200 import dist as D, synth
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        x0, r0, w = synth.add_rms_inputs(T, N, seed=3, dtype=np.float16)
        a, b = D.col_shard(N, rank, world)

        class OnCpu(D.TPRmsNorm):     # the two launches, restated by the oracle on host tensors
            def partial(self, x, d=None):
                self._ss = torch.from_numpy(oracle.rms_partial_f16(x.numpy(), None if d is None else d.numpy(), threads=1))
                return self._ss

            def apply(self, x, tot, h16=None, d=None):
                xo, ho = oracle.rms_apply_f16(x.numpy(), tot.numpy(), self.nw.numpy(), self.eps, self.Nfull, None if d is None else d.numpy(), threads=1)
                x.copy_(torch.from_numpy(xo))
                return torch.from_numpy(ho.copy())

        norm = OnCpu(torch.from_numpy(w[a:b].copy()), N, 1e-6)
        xs = torch.from_numpy(np.ascontiguousarray(x0[:, a:b])); rs = torch.from_numpy(np.ascontiguousarray(r0[:, a:b]))
        h = norm(xs, rs)
        # rows sharded, no collective: each rank norms its own rows of the full-width batch
        ra, rb = D.row_shard(T, rank, world)
        xr, hr = oracle.add_rms_f16(x0[ra:rb], w, 1e-6, r0[ra:rb], threads=1)
        gath = [None] * world
        dist.all_gather_object(gath, (a, b, xs.numpy(), h.numpy(), ra, rb, xr, hr))
        if rank == 0:
            full_x, full_h = oracle.add_rms_f16(x0, w, 1e-6, r0, threads=1)
            X = np.zeros_like(full_x); H = np.zeros_like(full_h); XR = np.zeros_like(full_x); HR = np.zeros_like(full_h)
            for a_, b_, xs_, h_, ra_, rb_, xr_, hr_ in gath:
                X[:, a_:b_] = xs_; H[:, a_:b_] = h_; XR[ra_:rb_] = xr_; HR[ra_:rb_] = hr_
            ulp = np.abs(np.spacing(np.abs(full_h))).astype(np.float64)
            ok_tp = np.array_equal(X.view(np.uint16), full_x.view(np.uint16)) and \
                bool((np.abs(H.astype(np.float64) - full_h.astype(np.float64)) <= ulp + 1e-5 * np.abs(full_h.astype(np.float64)).max()).all())
            ok_rows = np.array_equal(XR.view(np.uint16), full_x.view(np.uint16)) and np.array_equal(HR.view(np.uint16), full_h.view(np.uint16))
            out.put((ok_tp, ok_rows))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_tp_norm_and_row_shards():
    ctx = mp.get_context('spawn')
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, 48, 2048, out)) for r in range(2)]
    for p in procs: p.start()
    for p in procs: p.join(120)
    assert all(p.exitcode == 0 for p in procs)
    ok_tp, ok_rows = out.get(timeout=10)
    assert ok_tp and ok_rows


def test_tp_norm_refuses_bad_shards():
    from caminus_b200 import dist as D
    norm = D.TPRmsNorm(torch.ones(640), 5120, all_reduce=lambda t: None)
    with pytest.raises(ValueError): norm(torch.zeros(4, 644, dtype=torch.float16))          # not a multiple of 8 columns
    with pytest.raises(ValueError): norm(torch.zeros(4, 640, dtype=torch.float32))
    with pytest.raises(ValueError): norm(torch.zeros(4, 640, dtype=torch.float16), d=torch.zeros(4, 320, dtype=torch.float16))
    with pytest.raises(ValueError): D.TPRmsNorm(torch.ones(320), 5120, all_reduce=lambda t: None)(torch.zeros(4, 640, dtype=torch.float16))
