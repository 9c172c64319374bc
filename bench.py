"""Benchmark of the per-layer glue path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--ops]

A step is one pass of the per-layer glue over one batch of token rows (Qwen3-32B shape, fp16 storage): residual add +
RMSNorm (hidden 5120) -> q/k RMSNorm + NeoX RoPE (64 q + 8 kv heads of 128) -> SwiGLU + Q8_1 (intermediate 25600), three
launches. Every rank (one process per GPU; torchrun for N > 1) processes T = 65536 rows of its own: rows are independent,
so there is no data-path collective and the scaling is weak. `value` = rows of all ranks / the slowest rank's device time
with inputs resident in HBM; `e2e` = the same through the host-buffer call (pinned host inputs copied in, outputs copied
back, inside the timed region). `roofline` is for the dominant kernel (SwiGLU + Q8_1) from CUDA events recorded around it in
the timed steps. `cpu_baseline` is the CPU oracle on a bounded sample of rows on this box's host cores. `ops` holds the four
single-op workloads (add + RMSNorm fp32 at hidden 2048 for T = 1 and T = 65536, q/k norm + RoPE at T = 4096, SwiGLU + Q8_1 at
T = 8192, Q4_K rows 16384 x 2048) with their GB/s; --ops adds one entry per further op of the library.
--impl reference times the CPU implementations alone: the C restatement of the kernels on all host threads (the line's value) and
the NumPy restatement of the reference's host path, op by op, on one core (`cpu_baseline_numpy`).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path: sys.path.insert(0, ROOT)

import numpy as np   # noqa: E402

T_PER_GPU, HIDDEN, NH, NKV, INTER = 65536, 5120, 64, 8, 25600
BYTES_PER_TOKEN = {'add_rms_f16': 4 * HIDDEN * 2, 'qk_rope_f16': (NH + NKV) * 128 * 2 * 2, 'swiglu_q8_1_f16': 2 * INTER * 2 + INTER // 32 * 36}
# DRAM bytes per token row of the dominant kernel, from one ncu capture of swiglu_q8_fast_kernel at T = 8192, I = 25600
# (dram__bytes_read.sum + dram__bytes_write.sum = 838.90 + 215.24 MB); the traffic grows in proportion to the rows, so a launch
# of T rows is scaled from it
SWIGLU_DRAM_BYTES_PER_TOKEN = (838_904_320 + 215_235_072) / 8192
METRIC = 'per-layer glue throughput (residual add + RMSNorm -> q/k norm + RoPE -> SwiGLU + Q8_1), tokens/s'


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.isfile(p):
        try: return float(json.load(open(p))['hbm_gbs']), 'measured'
        except Exception: pass
    return 6650.0, 'fallback'


class Clocks:
    """samples the SM clock and the throttle reasons of one GPU during the timed region: NVML polled every 2 ms from a
    thread (reads only), or `nvidia-smi -lms 20` when the NVML binding is missing"""
    Q = 'index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,' \
        'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'
    BITS = {'hw_slowdown': 0x8, 'hw_thermal_slowdown': 0x40, 'sw_thermal_slowdown': 0x20, 'sw_power_cap': 0x4}

    def __init__(self, index):
        self.index, self.proc, self.path, self.thread, self.stop_flag = index, None, None, None, False
        self.sm, self.reasons, self.max_mhz = [], set(), None

    def _poll(self, nv, h):
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h)) if hasattr(nv, 'nvmlDeviceGetCurrentClocksEventReasons') \
                    else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                for name, bit in self.BITS.items():
                    if r & bit: self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            vis = os.environ.get('CUDA_VISIBLE_DEVICES')
            idx = int(vis.split(',')[self.index]) if vis and all(v.strip().isdigit() for v in vis.split(',')) else self.index
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, args=(nv, h), daemon=True); self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            f = tempfile.NamedTemporaryFile('w', suffix='.csv', delete=False); self.path = f.name
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={self.index}', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', '20'],
                                         stdout=f, stderr=subprocess.DEVNULL)
            time.sleep(0.5)     # (the tool needs a moment before its first sample)
        except Exception:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag = True; self.thread.join(1.0)
            if not self.sm: return {'sm_mhz': None, 'sm_max_mhz': self.max_mhz, 'reasons': ['no samples']}
            return {'sm_mhz': float(np.median(self.sm)), 'sm_max_mhz': self.max_mhz, 'reasons': sorted(self.reasons), 'samples': len(self.sm), 'via': 'nvml'}
        if self.proc is None: return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.05)
        self.proc.terminate()
        try: self.proc.wait(timeout=5)
        except Exception: self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            c = [v.strip() for v in line.split(',')]
            if len(c) < 9: continue
            try: sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError: continue
            for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), c[5:9]):
                if v.lower().startswith('active'): reasons.add(name)
        try: os.unlink(self.path)
        except OSError: pass
        if not sm: return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['no samples']}
        return {'sm_mhz': float(np.median(sm)), 'sm_max_mhz': float(max(mx)), 'reasons': sorted(reasons), 'samples': len(sm), 'via': 'nvidia-smi'}


def host_mem_available():
    """bytes of host memory the kernel counts as available (/proc/meminfo MemAvailable), capped by the cgroup's limit when one is set; 0 if unknown"""
    avail = 0
    try:
        for ln in open('/proc/meminfo'):
            if ln.startswith('MemAvailable:'): avail = int(ln.split()[1]) * 1024
    except OSError:
        return 0
    for pth, used in (('/sys/fs/cgroup/memory.max', '/sys/fs/cgroup/memory.current'),
                      ('/sys/fs/cgroup/memory/memory.limit_in_bytes', '/sys/fs/cgroup/memory/memory.usage_in_bytes')):
        try:
            lim = open(pth).read().strip()
            if lim.isdigit() and int(lim) < 1 << 60:
                left = int(lim) - int(open(used).read().strip())
                avail = min(avail, left) if avail else left
        except (OSError, ValueError):
            pass
    return max(avail, 0)


def cpu_layer_glue(sample, threads):
    """the CPU oracle over `sample` rows of the same workload: seconds for one pass"""
    import oracle
    from caminus_b200 import synth
    x0, r0, w = synth.add_rms_inputs(sample, HIDDEN, dtype=np.float16)
    q0, k0 = synth.qk_inputs(sample, NH, NKV); g0, u0 = synth.swiglu_inputs(sample, INTER); par = synth.rope_par()
    oracle.add_rms_f16(x0[:8], w, 1e-6, r0[:8], threads=1)     # (library load, page-in)
    t0 = time.perf_counter()
    oracle.add_rms_f16(x0, w, 1e-6, r0, threads=threads)
    oracle.qk_rope_f16(q0, k0, par, 0, threads=threads)
    oracle.swiglu_q8_1(g0.reshape(-1), u0.reshape(-1), sum_order=1, threads=threads)
    return time.perf_counter() - t0


def numpy_path_times(rows=64, reps=3):
    """the NumPy restatement of the reference's host path (oracle/numpy_path.py), op by op on one core: tokens/s (rows/s) of each op
    on `rows` token rows of the benchmarked shapes, best of `reps`"""
    from oracle import numpy_path as NP
    from caminus_b200 import synth
    def best(fn):
        fn(); ts = []
        for _ in range(reps): t0 = time.perf_counter(); fn(); ts.append(time.perf_counter() - t0)
        return min(ts)
    x0, r0, w = synth.add_rms_inputs(rows, HIDDEN, dtype=np.float16); q0, k0 = synth.qk_inputs(rows, NH, NKV); g0, u0 = synth.swiglu_inputs(rows, INTER)
    par = synth.rope_par(); pos = np.arange(rows)
    t_add = best(lambda: NP.add_rms_f32(x0, r0, w)); t_swi = best(lambda: NP.swiglu_q8_1(g0.reshape(-1), u0.reshape(-1)))
    t_qk = best(lambda: (NP.qk_norm_rope_f64(q0, par[:128], pos), NP.qk_norm_rope_f64(k0, par[128:256], pos)))
    g = np.random.default_rng(0); vocab, nrow = 4096, 1024
    W = g.integers(0, 256, (vocab, 8, 144), dtype=np.uint8); W[:, :, 0:4] = np.abs(g.standard_normal((vocab, 8, 2)) * 1e-3).astype(np.float16).view(np.uint8).reshape(vocab, 8, 4)
    ids = g.integers(0, vocab, nrow).astype(np.int32)
    t_q4k = best(lambda: NP.q4k_rows(W, ids))
    x1 = g.standard_normal((1, 2048)).astype(np.float32); d1 = g.standard_normal((1, 2048)).astype(np.float32); w1 = (1 + 0.05 * g.standard_normal(2048)).astype(np.float32)
    t_one = best(lambda: NP.add_rms_f32(x1, d1, w1))
    return {'value': rows / (t_add + t_qk + t_swi), 'unit': 'tokens/s', 'cores': 1, 'kind': 'reference host path restated in NumPy (float32 norm, float64 rotation, Q8_1 and Q4_K as its decoders define them)',
            'sample': f'{rows} token rows per op ({nrow} rows for the Q4_K gather), best of {reps}',
            'per_op': {'add_rms_f16_h5120_tokens_per_s': rows / t_add, 'qk_rope_72heads_tokens_per_s': rows / t_qk, 'swiglu_q8_1_I25600_tokens_per_s': rows / t_swi,
                       'q4k_get_rows_2048_rows_per_s': nrow / t_q4k, 'add_rms_f32_h2048_T1_us': t_one * 1e6}}


def run_reference(args, rank):
    """the reference arm: the path's CPU implementations on this box's host cores, a bounded sample of the workload per step. The
    line's value is the C restatement of the reference's kernels (its HIP sources do not compile for a CPU) on all host threads;
    `cpu_baseline_numpy` is the NumPy restatement of the reference's own host path on one core"""
    if rank != 0: return
    import oracle
    oracle.build()
    threads = oracle.default_threads()
    sample = 256
    for _ in range(args.warmup): cpu_layer_glue(sample, threads)
    ts = [cpu_layer_glue(sample, threads) for _ in range(args.steps)]
    sec = float(np.mean(ts)); val = sample / sec
    try: npy = numpy_path_times()
    except Exception as e: npy = {'unavailable': f'{type(e).__name__}: {e}'[:200]}
    print(json.dumps({
        'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': 'tokens/s', 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': sec * 1e3, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': f'per-layer glue, Qwen3-32B shape: hidden {HIDDEN}, {NH} q + {NKV} kv heads x 128, '
                               f'intermediate {INTER}, fp16 storage', 'rows_per_step': sample},
        'cpu_baseline': {'value': val, 'unit': 'tokens/s', 'cores': threads, 'kind': 'port',
                         'sample': f'{sample} token rows per step through all three ops (the C oracle, rows split over {threads} host threads)'},
        'cpu_baseline_numpy': npy,
        'e2e': {'value': val, 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0}), flush=True)


HEADLINE_OPS = ('add_rms16_f32_h2048_T1', 'add_rms16_f32_h2048_T65536', 'qk_rope_f16_T4096', 'swiglu_q8_1_f16_T8192', 'q4k_get_rows_16384x2048')


def single_op_lines(torch, dev, peak, only=(), headline=False):
    """device-resident GB/s of the single-op workloads (median over batches of event-timed launches; buffers rotated where a
    workload's data would fit in L2). headline: only the four workloads the metric is quoted on (HEADLINE_OPS)"""
    from caminus_b200 import glue, synth
    from caminus_b200.engine import gguf
    from caminus_b200.prefill import q3m_ops
    O = q3m_ops.Ops(dev)
    out = {}

    def timed(fn, reps=9, rot=1, inner=10):
        """per-launch seconds: `inner` launches back to back between two events (the queue never runs dry, as inside a model's
        layer loop), median and minimum over `reps` such batches"""
        def run():
            for i in range(3): fn(i % rot)
            torch.cuda.synchronize(dev)
            ts = []
            for r in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for i in range(inner): fn((r * inner + i) % rot)
                b.record(); b.synchronize(); ts.append(a.elapsed_time(b) * 1e-3 / inner)
            return float(np.median(ts)), float(np.min(ts))
        return run              # (run by line() if the op is selected)

    def graphed(fn, launches=200):
        """per-launch seconds of `launches` launches captured in one CUDA graph (no host launch cost between them)"""
        try:
            st = torch.cuda.Stream(dev)
            with torch.cuda.stream(st):
                fn(0); st.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    for i in range(launches): fn(i)
                gr.replay(); st.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(st); gr.replay(); b.record(st); b.synchronize()
            return a.elapsed_time(b) * 1e-3 / launches
        except Exception as e:     # (capture refused: report why, keep the bench alive)
            return f'{type(e).__name__}: {e}'[:160]

    def line(name, nbytes, sec, units, unit, copy_ref=False, graph_fn=None):
        if headline and name not in HEADLINE_OPS: return
        if only and not any(o in name for o in only): return
        med, mn = sec()
        out[name] = {'bytes': nbytes, 'us_median': med * 1e6, 'us_min': mn * 1e6, 'gbs': nbytes / med / 1e9, 'frac_of_peak': nbytes / med / 1e9 / peak,
                     'frac_of_8tbs': nbytes / med / 8e12, unit: units / med}
        if graph_fn is not None:      # a launch this short can be bounded by the host's launch rate: the same launches replayed from a CUDA graph
            gs = graphed(graph_fn, 40)
            out[name]['us_in_cuda_graph'] = gs * 1e6 if isinstance(gs, float) else gs
            if isinstance(gs, float): out[name]['frac_of_peak_in_cuda_graph'] = nbytes / gs / 1e9 / peak
        if copy_ref:      # a launch this short does not reach the bandwidth of a long copy: a plain device copy moving the same bytes, timed the same way
            half = nbytes // 2 // 16 * 16
            srcs = [torch.empty(half, dtype=torch.uint8, device=dev) for _ in range(4)]; dsts = [torch.empty(half, dtype=torch.uint8, device=dev) for _ in range(4)]
            cmed, _ = timed(lambda i: dsts[i].copy_(srcs[i]), rot=4)()
            out[name]['us_plain_copy_same_bytes'] = cmed * 1e6; out[name]['frac_of_plain_copy_same_bytes'] = cmed / med

    g = torch.Generator(device=dev); g.manual_seed(0)
    # config 1: add + RMSNorm fp32, hidden 2048: T = 1 (latency) and a T sweep
    for T in ((1, 65536) if headline else (1, 64, 4096, 65536)):
        rot = 8 if T <= 4096 else 1
        xs = [torch.randn(T, 2048, device=dev, generator=g) for _ in range(rot)]; d = torch.randn(T, 2048, device=dev, generator=g)
        nw = 1 + 0.05 * torch.randn(2048, device=dev, generator=g); h = torch.empty(T, 2048, device=dev); h16 = torch.empty(T, 2048, dtype=torch.float16, device=dev)
        sec = timed(lambda i: O.add_rms16(xs[i], nw, 1e-6, h16, T, 2048, d=d, S=1, h=h), rot=rot, inner=100 if T == 1 else 10)
        line(f'add_rms16_f32_h2048_T{T}', T * (4 * 8192 + 4096) + 8192, sec, T, 'tokens_per_s',
             graph_fn=(lambda i: O.add_rms16(xs[i % rot], nw, 1e-6, h16, T, 2048, d=d, S=1, h=h)) if 1 < T <= 4096 else None)
        if T == 1 and f'add_rms16_f32_h2048_T{T}' in out:
            gs = graphed(lambda i: O.add_rms16(xs[i % rot], nw, 1e-6, h16, T, 2048, d=d, S=1, h=h))
            out[f'add_rms16_f32_h2048_T{T}']['us_in_cuda_graph'] = gs * 1e6 if isinstance(gs, float) else gs
            torch.cuda.synchronize(dev); t0 = time.perf_counter()            # the host's cost of one call through the loader interface
            for i in range(2000): O.add_rms16(xs[i % rot], nw, 1e-6, h16, T, 2048, d=d, S=1, h=h)
            host_s = (time.perf_counter() - t0) / 2000; torch.cuda.synchronize(dev)
            out[f'add_rms16_f32_h2048_T{T}']['us_per_call_host'] = host_s * 1e6
        del xs, d, h, h16
    # config 2: q/k norm + RoPE fp16, T = 4096, 32 + 4 heads (75 MB: 4 rotating copies)
    T = 4096
    qs = [torch.randn(T, 32, 128, device=dev, generator=g).half() for _ in range(4)]; ks = [torch.randn(T, 4, 128, device=dev, generator=g).half() for _ in range(4)]
    par = torch.from_numpy(synth.rope_par()).to(dev)
    line('qk_rope_f16_T4096', T * 36 * 128 * 4 + 1032, timed(lambda i: glue.qk_rope_f16(qs[i], ks[i], par, 0), rot=4), T, 'tokens_per_s', copy_ref=True,
         graph_fn=lambda i: glue.qk_rope_f16(qs[i % 4], ks[i % 4], par, 0))
    del qs, ks
    # config 3: SwiGLU + Q8_1, T = 8192, I = 25600
    T = 8192
    gt = (torch.randn(T * INTER, device=dev, generator=g) * 1.5).half(); up = (torch.randn(T * INTER, device=dev, generator=g) * 1.5).half()
    yq = torch.empty(T * INTER // 32 * 36, dtype=torch.uint8, device=dev)
    line('swiglu_q8_1_f16_T8192', T * BYTES_PER_TOKEN['swiglu_q8_1_f16'], timed(lambda i: gguf.swiglu_q8_1(gt, up, yq)), T, 'tokens_per_s')
    line('swiglu_q8_1_f16_sums_T8192', T * BYTES_PER_TOKEN['swiglu_q8_1_f16'], timed(lambda i: gguf.swiglu_q8_1(gt, up, yq, sums=True)), T, 'tokens_per_s')
    line('swiglu_q8_1_f16_strict_T8192', T * BYTES_PER_TOKEN['swiglu_q8_1_f16'], timed(lambda i: gguf.swiglu_q8_1(gt, up, yq, strict=True)), T, 'tokens_per_s')
    del gt, up, yq
    # config 4: Q4_K rows, vocab 151936 x 2048, 16384 ids (output 134 MB: 2 rotating outputs)
    vocab, N, n = 151936, 2048, 16384
    W = torch.randint(0, 256, (vocab, 8, 144), device=dev, dtype=torch.uint8, generator=g)
    W[:, :, 0:4] = (torch.randn(vocab, 8, 2, device=dev, generator=g) * 1e-3).abs().half().view(torch.uint8).view(vocab, 8, 4)
    toks = torch.randint(0, vocab, (n,), device=dev, dtype=torch.int32, generator=g)
    xo = [torch.empty(n, N, device=dev) for _ in range(2)]
    line('q4k_get_rows_16384x2048', n * (4 + 1152 + 8192), timed(lambda i: O.emb(W.view(-1), 1152, vocab, toks, xo[i], n, N), rot=2), n, 'rows_per_s', copy_ref=True,
         graph_fn=lambda i: O.emb(W.view(-1), 1152, vocab, toks, xo[i % 2], n, N))
    del W, toks, xo
    if headline: return out
    # ---- the later rows of the path (hyper-connection glue, MMQ layout, Q8_0 KV form, the training line's quantiser) ----
    import ctypes
    from caminus_b200.prefill import glue as PG
    from caminus_b200.train import actq as A
    rnd = lambda *s_, scale=1.0: torch.randn(*s_, device=dev, generator=g) * scale
    gl = PG.Glue(dev); D = gl.D; T, HC = 8192, 4; R = T * HC
    x = rnd(R, D, scale=3.0); w = 0.5 + torch.rand(HC, D, device=dev, generator=g); y = torch.empty_like(x); ybf = torch.empty(R, D, dtype=torch.bfloat16, device=dev)
    scl = torch.empty(R, device=dev)
    line('pf_rms_mul_R32768_K2560_bf16_scale', R * D * (4 + 2) + R * 4, timed(lambda i: gl.rms_mul(x, w, None, R, 1e-6, ybf=ybf, scale=scl)), R, 'rows_per_s')
    line('pf_rms_mul_R32768_K2560_f32', R * D * 8, timed(lambda i: gl.rms_mul(x, w, y, R, 1e-6)), R, 'rows_per_s')
    b = rnd(T, D); inj = rnd(T, HC, scale=3.0)
    line('pf_hc_post_rms_T8192_HC4_bf16_scale', R * D * (8 + 2) + T * D * 4, timed(lambda i: gl.hc_post_rms(b, inj, x, w, T, HC, 1e-6, xnbf=ybf, scale=scl)), T, 'tokens_per_s')
    line('pf_hc_post_T8192_HC4', T * D * 4 + R * D * 8, timed(lambda i: gl.hc_post(b, inj, x, T, HC)), T, 'tokens_per_s')
    gate = rnd(R, D); outm = torch.empty(T, D, device=dev)
    line('pf_hc_mean_T8192_HC4', R * D * 8 + T * D * 4, timed(lambda i: gl.hc_mean(x, gate, outm, T, HC, scale=scl, w=w)), T, 'tokens_per_s')
    del x, y, ybf, gate, outm, b
    rows, K = 8192, 25600
    gh = (rnd(rows, K, scale=1.5)).half(); uh = (rnd(rows, K, scale=1.5)).half(); ym = torch.empty(K // 128, rows, 144, dtype=torch.uint8, device=dev)
    line('swiglu_mmq_q8_1_f16_T8192_K25600_D4', rows * K * 4 + rows * K // 128 * 144, timed(lambda i: gguf.quantize_mmq_q8_1(gh, 'D4', u=uh, y=ym)), rows, 'tokens_per_s')
    line('swiglu_mmq_q8_1_f16_T8192_K25600_DS4', rows * K * 4 + rows * K // 128 * 144, timed(lambda i: gguf.quantize_mmq_q8_1(gh, 'DS4', u=uh, y=ym)), rows, 'tokens_per_s')
    del gh, uh, ym
    T, nh, nkv = 4096, 32, 4; M = nkv * 128; ldq = nh * 128 + 2 * M; rowb = 2 * (M // 32) * 34
    Q8 = q3m_ops.Ops(dev, q8=True)
    qkv = [rnd(T * ldq, scale=3.0) for _ in range(2)]; q16 = torch.empty(T, nh, 128, dtype=torch.float16, device=dev)
    cache = torch.zeros(T * rowb, dtype=torch.uint8, device=dev); err = torch.zeros(1, dtype=torch.int32, device=dev)
    line('qk_rope_q8_f32_T4096', T * (ldq * 4 + nh * 256 + rowb), timed(lambda i: Q8.qk_rope(qkv[i], ldq, nh, nkv, par, 0, q16, cache, T, err=err), rot=2), T, 'tokens_per_s',
         graph_fn=lambda i: Q8.qk_rope(qkv[i % 2], ldq, nh, nkv, par, 0, q16, cache, T, err=err))
    F16 = q3m_ops.Ops(dev); c16 = torch.zeros(T * 2 * M, dtype=torch.float16, device=dev)
    line('qk_rope_f32_cache_T4096', T * (ldq * 4 + nh * 256 + 2 * M * 2), timed(lambda i: F16.qk_rope(qkv[i], ldq, nh, nkv, par, 0, q16, c16, T), rot=2), T, 'tokens_per_s',
         graph_fn=lambda i: F16.qk_rope(qkv[i % 2], ldq, nh, nkv, par, 0, q16, c16, T))
    del qkv, cache, c16
    T2 = 32768                                               # the same two forms on a batch that fills the device for longer
    qkv2 = rnd(T2 * ldq, scale=3.0); q16b = torch.empty(T2, nh, 128, dtype=torch.float16, device=dev)
    cache2 = torch.zeros(T2 * rowb, dtype=torch.uint8, device=dev); c16b = torch.zeros(T2 * 2 * M, dtype=torch.float16, device=dev)
    line('qk_rope_q8_f32_T32768', T2 * (ldq * 4 + nh * 256 + rowb), timed(lambda i: Q8.qk_rope(qkv2, ldq, nh, nkv, par, 0, q16b, cache2, T2, err=err)), T2, 'tokens_per_s')
    line('qk_rope_f32_cache_T32768', T2 * (ldq * 4 + nh * 256 + 2 * M * 2), timed(lambda i: F16.qk_rope(qkv2, ldq, nh, nkv, par, 0, q16b, c16b, T2)), T2, 'tokens_per_s')
    del qkv2, cache2, c16b, q16b
    Mr, Kq = 32768, 1024
    xa = rnd(Mr, Kq, scale=2.0).bfloat16()
    line('actq_codes_bf16_M32768_K1024', Mr * Kq * (2 + 2 + 0.5) + Mr * 4, timed(lambda i: A.actq_codes(xa, 4, 1.0)), Mr, 'rows_per_s')
    for Kq2, Mr2 in ((2048, 16384), (4096, 8192)):
        xa2 = rnd(Mr2, Kq2, scale=2.0).bfloat16()
        line(f'actq_codes_bf16_M{Mr2}_K{Kq2}', Mr2 * Kq2 * (2 + 2 + 0.5) + Mr2 * 4, timed(lambda i: A.actq_codes(xa2, 4, 1.0)), Mr2, 'rows_per_s')
        del xa2
    gu = rnd(8192, 2 * 4096, scale=2.0).bfloat16()
    line('silu_mul_actq_M8192_F4096', 8192 * 4096 * (4 + 2 + 0.5) + 8192 * 4, timed(lambda i: A.silu_mul_actq(gu, 4, 1.0)), 8192, 'rows_per_s')
    xe = rnd(Mr, 896, scale=2.0); nwe = 0.5 + torch.rand(896, device=dev, generator=g); wab = rnd(8, 896, scale=0.05).bfloat16()
    line('block_entry_M32768_d896_nab8', Mr * 896 * (4 + 2 + 0.5) + Mr * (8 + 16), timed(lambda i: A.block_entry(xe, nwe, wab, 1e-6, 4, 1.0)), Mr, 'rows_per_s')
    # ---- router glue (Qwen3-30B-A3B shapes: hidden 2048, 128 experts, top 8), IQ4 row gathers, the norm with a Q8_1 copy ----
    n, E, K, k = 8192, 128, 2048, 8
    hh = rnd(n, K); Wr = rnd(E, K, scale=0.05); lg = torch.empty(n, E, device=dev)
    line('q3p_router_T8192_E128_K2048', n * K * 4 + E * K * 4 + n * E * 4, timed(lambda i: O.router(hh, Wr, E, K, lg, n)), n, 'tokens_per_s')
    if 'q3p_router_T8192_E128_K2048' in out: out['q3p_router_T8192_E128_K2048']['gflops'] = 2.0 * n * E * K / out['q3p_router_T8192_E128_K2048']['us_median'] / 1e3
    ids = torch.zeros(n * k, dtype=torch.int32, device=dev); wts = torch.zeros(n * k, device=dev); er = torch.zeros(1, dtype=torch.int32, device=dev)
    line('q3p_topk_T8192_E128_k8', n * E * 4 + n * k * 8, timed(lambda i: O.topk(lg, E, k, 6.103515625e-5, ids, wts, er, n)), n, 'tokens_per_s',
         graph_fn=lambda i: O.topk(lg, E, k, 6.103515625e-5, ids, wts, er, n))
    xs_, yd_ = (torch.zeros(n * k, dtype=torch.int32, device=dev) for _ in range(2))
    items = torch.zeros(q3m_ops.items_bound(n * k, E), 4, dtype=torch.int32, device=dev); nit = torch.zeros(1, dtype=torch.int32, device=dev)
    line('q3p_group_65536_pairs_E128', n * k * 12, timed(lambda i: O.group(ids, n * k, k, E, xs_, yd_, items, nit, er)), n, 'tokens_per_s',
         graph_fn=lambda i: O.group(ids, n * k, k, E, xs_, yd_, items, nit, er))
    lg256 = rnd(2048, 256, scale=3.0); ids10 = torch.zeros(2048 * 10, dtype=torch.int32, device=dev); wts10 = torch.zeros(2048 * 10, device=dev)
    line('pf_router_T2048_E256_k10', 2048 * 256 * 4 + 2048 * 10 * 8, timed(lambda i: gl.router(lg256, 2048, 256, 10, ids10, wts10, er)), 2048, 'tokens_per_s',
         graph_fn=lambda i: gl.router(lg256, 2048, 256, 10, ids10, wts10, er))
    del hh, Wr, lg
    from caminus_b200.device import cuda as CU
    feed = CU.Module('prefill_feed'); I = ctypes.c_int
    vocab, nblk, nt = 151936, 8, 16384
    tab = torch.randint(0, 256, (vocab, nblk, 136), device=dev, dtype=torch.uint8, generator=g)
    tab[:, :, 0:2] = (torch.randn(vocab, nblk, 1, device=dev, generator=g) * 1e-3).abs().half().view(torch.uint8).view(vocab, nblk, 2)
    tk = torch.randint(0, vocab, (nt,), device=dev, dtype=torch.int32, generator=g); xo = [torch.empty(nt, nblk * 256, device=dev) for _ in range(2)]
    line('embd_rows_iq4xs_16384x2048', nt * (4 + nblk * 136 + nblk * 1024), timed(lambda i: feed.embd_rows_iq4xs((1,), (256,), tab.view(-1), tk, I(vocab), I(nt), I(nblk), xo[i], er), rot=2), nt, 'rows_per_s',
         graph_fn=lambda i: feed.embd_rows_iq4xs((1,), (256,), tab.view(-1), tk, I(vocab), I(nt), I(nblk), xo[i % 2], er))
    bpr = 64; raw = torch.randint(0, 256, (vocab, bpr, 18), device=dev, dtype=torch.uint8, generator=g)
    raw[:, :, 0:2] = (torch.randn(vocab, bpr, 1, device=dev, generator=g) * 1e-3).abs().half().view(torch.uint8).view(vocab, bpr, 2)
    line('ple_rows_iq4nl_16384x2048', nt * (4 + bpr * 18 + bpr * 128), timed(lambda i: feed.ple_rows_iq4nl((1,), (256,), raw.view(-1), tk, I(vocab), I(nt), I(bpr), xo[i], er), rot=2), nt, 'rows_per_s',
         graph_fn=lambda i: feed.ple_rows_iq4nl((1,), (256,), raw.view(-1), tk, I(vocab), I(nt), I(bpr), xo[i % 2], er))
    tq6 = torch.randint(0, 256, (vocab, nblk, 210), device=dev, dtype=torch.uint8, generator=g)
    tq6[:, :, 208:210] = (torch.randn(vocab, nblk, 1, device=dev, generator=g) * 1e-3).half().view(torch.uint8).view(vocab, nblk, 2)
    line('emb_rows_q6k_16384x2048', nt * (4 + nblk * 210 + nblk * 1024), timed(lambda i: O.emb_q6k(tq6.view(-1), nblk * 210, vocab, tk, xo[i], nt, nblk * 256), rot=2), nt, 'rows_per_s',
         graph_fn=lambda i: O.emb_q6k(tq6.view(-1), nblk * 210, vocab, tk, xo[i % 2], nt, nblk * 256))
    ti2 = torch.randint(0, 256, (vocab, nblk, 82), device=dev, dtype=torch.uint8, generator=g)
    ti2[:, :, 0:2] = (torch.randn(vocab, nblk, 1, device=dev, generator=g) * 1e-2).half().view(torch.uint8).view(vocab, nblk, 2)
    CU.set_iq2s_grid(np.array([8, 25, 43], np.uint8)[np.random.default_rng(5).integers(0, 3, (1024, 8))])     # a stand-in grid: the timing does not depend on its entries
    from caminus_b200.prefill import q35own
    OT = q35own.Ops(dev, module=q35own.MODULE_TCAP)
    line('emb_rows_iq2s_16384x2048', nt * (4 + nblk * 82 + nblk * 1024), timed(lambda i: OT.emb_iq2s(ti2.view(-1), nblk * 82, vocab, tk, xo[i], nt, nblk * 256), rot=2), nt, 'rows_per_s',
         graph_fn=lambda i: OT.emb_iq2s(ti2.view(-1), nblk * 82, vocab, tk, xo[i % 2], nt, nblk * 256))
    del tab, raw, xo, tq6, ti2
    from caminus_b200 import lib as LB
    Rq, Kq8 = 32768, 2560
    xq = rnd(Rq, Kq8, scale=3.0); wq8 = 0.5 + torch.rand(1, Kq8, device=dev, generator=g); yq8 = torch.empty(Rq, Kq8, device=dev)
    q8o = torch.empty(Rq * Kq8 // 32 * 36, dtype=torch.uint8, device=dev); Lc = LB.load(); cs = torch.cuda.current_stream(dev).cuda_stream
    line('rms_mul_q8_1_R32768_K2560', Rq * Kq8 * 8 + Rq * Kq8 // 32 * 36,
         timed(lambda i: LB.check(Lc.cam_rms_mul_q8_1(xq.data_ptr(), wq8.data_ptr(), yq8.data_ptr(), q8o.data_ptr(), Rq, 1, 1e-6, Kq8, cs), 'cam_rms_mul_q8_1')), Rq, 'rows_per_s')
    del xq, yq8, q8o
    xq1 = rnd(8192 * 5120, scale=2.0)
    line('gg_quantize_q8_1_f32_41943040', 8192 * 5120 * 4 + 8192 * 5120 // 32 * 36, timed(lambda i: gguf.quantize_q8_1(xq1)), 8192, 'rows_per_s')
    uq1 = rnd(8192 * 5120, scale=2.0); hq1 = torch.empty_like(xq1)
    line('gg_silu_mul_f32_41943040', 8192 * 5120 * 12, timed(lambda i: gguf.silu_mul(xq1, uq1)), 8192, 'rows_per_s')
    del xq1, uq1, hq1
    # ---- the remaining small ops of the path (per-head norm + partial rotation, the training line's elementwise forwards) ----
    L_ = ctypes.c_long; Fc = ctypes.c_float
    rows_h, heads_h, Dh = 8192, 16, 256                          # pf_qk_nr: 8192 tokens x 16 heads of 256, 64 rotated dims
    xh = rnd(rows_h * heads_h, Dh, scale=1.5); wh = 0.5 + torch.rand(Dh, device=dev, generator=g); oh = torch.empty_like(xh)
    attn = CU.Module('prefill_attn'); ts_h = float(np.float32(np.float32(1e7) ** np.float32(-2.0 / 64)))
    line('pf_qk_nr_T8192_16heads_D256', rows_h * heads_h * Dh * 8, timed(lambda i: attn.pf_qk_nr((rows_h * heads_h,), (256,), xh, I(Dh), I(heads_h), wh, I(Dh), I(64), Fc(ts_h), Fc(1e-6), I(0), oh)), rows_h, 'tokens_per_s')
    del xh, oh
    core, fuse = CU.Module('core'), CU.Module('fuse'); ne, de = 65536, 896; nel = ne * de
    xe_ = rnd(ne, de); we_ = 0.5 + torch.rand(de, device=dev, generator=g); oe_ = torch.empty_like(xe_)
    line('rmsnorm_f32_65536x896', nel * 8, timed(lambda i: core.rmsnorm_f32((ne,), (256,), xe_, we_, oe_, I(de), Fc(1e-5))), ne, 'rows_per_s')
    mb = rnd(ne, de).bfloat16(); lb = rnd(ne, de).bfloat16()
    line('residual3_65536x896', nel * 12, timed(lambda i: core.residual3(((nel + 255) // 256,), (256,), xe_, mb, lb, oe_, ctypes.c_int64(nel))), ne, 'rows_per_s')
    line('residual_slices_fwd_65536x896', nel * 12, timed(lambda i: fuse.residual_slices_fwd(((nel // 4 + 255) // 256,), (256,), xe_, mb, lb, ctypes.c_void_p(None), ctypes.c_void_p(None), oe_, I(de), L_(nel // 4))), ne, 'rows_per_s')
    cb_ = torch.empty(ne, de, dtype=torch.bfloat16, device=dev)
    line('cast_bf16_65536x896', nel * 6, timed(lambda i: core.cast_bf16(((nel + 255) // 256,), (256,), xe_, cb_, ctypes.c_int64(nel))), ne, 'rows_per_s')
    gub = rnd(ne, 2 * de, scale=2.0).bfloat16(); ab_ = torch.empty(ne, de, dtype=torch.bfloat16, device=dev)
    line('silu_mul_bf16_65536x896', nel * 6, timed(lambda i: core.silu_mul_bf16(((nel + 255) // 256,), (256,), gub, ab_, I(de), ctypes.c_int64(nel))), ne, 'rows_per_s')
    ya_ = rnd(ne, de)
    line('pf_add_sum_65536x896', nel * 16, timed(lambda i: gl.add_sum(xe_, oe_, ya_, nel)), ne, 'rows_per_s')
    yb_ = torch.empty(PG.tpad(ne), de, dtype=torch.bfloat16, device=dev)
    line('pf_silu_bf16_65536x896', nel * 6, timed(lambda i: gl.silu_bf16(xe_, yb_, ne, de, 0.5)), ne, 'rows_per_s')
    line('pf_to_bf16_65536x896', nel * 6, timed(lambda i: gl.to_bf16(xe_, yb_, ne, de)), ne, 'rows_per_s')
    tp_ = CU.Module('prefill_tp')
    line('pf_swiglu_f32_65536x896', nel * 12, timed(lambda i: tp_.pf_swiglu(((nel + 255) // 256,), (256,), xe_, oe_, ya_, L_(nel))), ne, 'rows_per_s')
    toks_e = torch.randint(0, ne, (ne,), device=dev, dtype=torch.int32, generator=g)
    line('embedding_f32_65536x896', nel * 8, timed(lambda i: core.embedding_f32((ne,), (256,), toks_e, xe_, oe_, I(de))), ne, 'rows_per_s')
    del xe_, oe_, mb, lb, cb_, gub, ab_, ya_, yb_
    # the one-kernel tensor-parallel norm run by a single rank (its own partial is the only word it waits for): the kernel's HBM side
    from caminus_b200 import dist as DD
    for Ns_ in (640, 2560):
        xt = rnd(65536, Ns_).half(); dt_ = rnd(65536, Ns_).half(); ht = torch.empty_like(xt)
        ft = DD.TPRmsNormFused(torch.ones(Ns_, device=dev), Ns_, 65536, 1e-6, device=dev)
        line(f'tp_rms_fused_one_rank_T65536_Ns{Ns_}', 65536 * Ns_ * 8, timed(lambda i: ft(xt, dt_, ht)), 65536, 'rows_per_s')
        ft.check(); del xt, dt_, ht
    xm = rnd(8192, 5120, scale=2.0); ym2 = torch.empty(5120 // 128, 8192, 144, dtype=torch.uint8, device=dev)
    line('quantize_mmq_q8_1_f32_8192x5120_D4', 8192 * 5120 * 4 + 8192 * 40 * 144, timed(lambda i: gguf.quantize_mmq_q8_1(xm, 'D4', y=ym2)), 8192, 'rows_per_s')
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1); ap.add_argument('--steps', type=int, default=20); ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--rows', type=int, default=T_PER_GPU, help='token rows per GPU (the configured workload is 65536)')
    ap.add_argument('--e2e-chunk', type=int, default=1024, help='rows per chunk of the host-buffer pass (two chunks in flight)')
    ap.add_argument('--ops', action='store_true', help='time every op of the library on rank 0, not only the four headline workloads')
    ap.add_argument('--only', default='', help='with --ops: comma-separated substrings of the op names to time (default: all)')
    ap.add_argument('--cpu-sample', type=int, default=512)
    ap.add_argument('--skip-e2e', action='store_true', help='leave out the host-buffer leg (profiling runs)')
    ap.add_argument('--skip-cpu', action='store_true', help='leave out the CPU baseline leg (profiling runs)')
    ap.add_argument('--e2e-rows', type=int, default=0, help='token rows per GPU of the host-buffer leg (0: the whole batch if the host can pin it, 229 KB per row and rank)')
    args = ap.parse_args()
    rank, world, local = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1)), int(os.environ.get('LOCAL_RANK', 0))
    if args.impl == 'reference': return run_reference(args, rank)
    args.warmup = max(args.warmup, 3)

    import torch
    from caminus_b200 import glue, lib
    lib.load()
    dev = torch.device(f'cuda:{local}'); torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=dev)
    T = args.rows
    gen = torch.Generator(device=dev); gen.manual_seed(1000 + rank)
    rn = lambda *s, scale=1.0: (torch.randn(*s, device=dev, generator=gen) * scale).half()
    x = rn(T, HIDDEN); resid = rn(T, HIDDEN); q = rn(T, NH, 128); k = rn(T, NKV, 128)
    gate = torch.empty(T, INTER, dtype=torch.float16, device=dev); up = torch.empty(T, INTER, dtype=torch.float16, device=dev)
    for a in range(0, T, 8192): gate[a:a + 8192] = rn(min(8192, T - a), INTER, scale=1.5); up[a:a + 8192] = rn(min(8192, T - a), INTER, scale=1.5)
    from caminus_b200 import synth
    nw = (1 + 0.05 * torch.randn(HIDDEN, device=dev, generator=gen)).float(); par = torch.from_numpy(synth.rope_par()).to(dev)
    h16 = torch.empty_like(x); yq = torch.empty(T * INTER // 32 * 36, dtype=torch.uint8, device=dev)

    def step(ev=None):      # x, q, k are updated in place, as the path does: the next step runs on this step's rows (still finite)
        if ev: ev[0].record()
        glue.add_rms_f16(x, nw, 1e-6, h16=h16, d=resid)
        if ev: ev[1].record()
        glue.qk_rope_f16(q, k, par, 0)
        if ev: ev[2].record()
        glue.swiglu_q8_1(gate.view(-1), up.view(-1), yq)
        if ev: ev[3].record()

    def barrier():
        if world > 1: torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup): step()
    barrier()
    clocks = Clocks(local); clocks.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    barrier()
    for i in range(args.steps): step(evs[i])
    barrier()
    clk = clocks.stop()
    # device time of exactly K steps: first step's first event to the last step's last; per-kernel times from the events between
    per = np.array([[e[j].elapsed_time(e[j + 1]) for j in range(3)] for e in evs]) * 1e-3     # [steps, 3] seconds
    total = evs[0][0].elapsed_time(evs[-1][3]) * 1e-3
    if world > 1:
        t = torch.tensor([total], device=dev, dtype=torch.float64); torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX); total = float(t.item())
    ms_per_step = total / args.steps * 1e3
    value = T * world / (total / args.steps)

    # the hidden-sharded RMSNorm (N > 1 only): this rank's hidden / N columns of all T rows, partial -> NCCL all-reduce of [T] fp32 -> apply
    tp = None
    if world > 1 and HIDDEN % (8 * world) == 0:
        from caminus_b200 import dist as D
        Ns = HIDDEN // world
        xs0 = rn(T, Ns); ds = rn(T, Ns); hs = torch.empty_like(xs0); xs = xs0.clone()
        norm = D.TPRmsNorm(nw[rank * Ns:(rank + 1) * Ns].contiguous(), HIDDEN, 1e-6)

        def all_true(flag):
            t = torch.tensor([1 if flag else 0], device=dev, dtype=torch.int32); torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
            return bool(t.item())

        def timed_norm(fn):
            for _ in range(3): fn()
            barrier()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            for _ in range(args.steps): fn()
            ev[1].record(); barrier()
            t = torch.tensor([ev[0].elapsed_time(ev[1]) * 1e-3 / args.steps], device=dev, dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            return float(t.item())

        # the value check's reference: this rank's apply kernel on all ranks' partials added in rank order from 0.0f
        xa = xs0.clone()
        parts = [torch.empty(T, device=dev) for _ in range(world)]
        torch.distributed.all_gather(parts, norm.partial(xa, ds).clone())
        tot = torch.zeros(T, device=dev)
        for p_ in parts: tot = tot + p_
        h_ref = norm.apply(xa, tot, d=ds).clone()                     # (xa is now fp16(x + d))
        xb = xs0.clone(); h_nccl = norm(xb, ds).clone()
        rel = float(((h_nccl.float() - h_ref.float()).abs().max() / h_ref.float().abs().max()).item())
        nccl_ok = all_true(torch.equal(xb, xa) and rel <= 1e-3)      # (fp16 outputs: one rounding step of 2^-11; the sums differ only in order)
        tps = timed_norm(lambda: norm(xs, ds, hs))
        tp = {'us_per_step': tps * 1e6, 'tokens_per_s': T / tps, 'hbm_gbs_per_gpu': T * 4 * Ns * 2 / tps / 1e9, 'frac_of_peak': T * 4 * Ns * 2 / tps / 1e9 / peaks()[0],
              'nvlink_bytes_per_rank': T * 4, 'vs_rank_ordered_sum': {'x_bitwise': nccl_ok, 'h16_max_rel': rel},
              'note': f'hidden {HIDDEN} in {world} shards of {Ns}; every rank holds all {T} rows'}
        # the same norm as one kernel per rank (partials by peer stores over NVLink, no collective call)
        try:
            fused = D.TPRmsNormFused(norm.nw, HIDDEN, T, 1e-6)

            def checked():                                            # a wait that ran out on one rank ends the leg on every rank (the ranks' collectives stay matched)
                err = None
                try: fused.check()
                except RuntimeError as e_: err = e_
                if not all_true(err is None): raise RuntimeError(str(err) if err else 'a wait for another rank ran out on another rank')
            xc = xs0.clone(); h_f = fused(xc, ds); checked()
            bitwise = all_true(torch.equal(h_f, h_ref) and torch.equal(xc, xa))
            xc.copy_(xs0); h_f2 = fused(xc, ds); checked()               # the next call (the other half of the exchange buffer)
            bitwise = all_true(torch.equal(h_f2, h_ref) and torch.equal(xc, xa)) and bitwise
            rel_f = float(((h_f.float() - h_nccl.float()).abs().max() / h_nccl.float().abs().max()).item())
            tf = timed_norm(lambda: fused(xs, ds, hs))
            checked()
            tp['fused'] = {'us_per_step': tf * 1e6, 'tokens_per_s': T / tf, 'hbm_gbs_per_gpu': T * 4 * Ns * 2 / tf / 1e9, 'frac_of_peak': T * 4 * Ns * 2 / tf / 1e9 / peaks()[0],
                           'nvlink_bytes_per_rank': T * 8 * (world - 1), 'parity': 'bitwise' if bitwise else 'MISMATCH',
                           'vs_nccl_form_max_rel': rel_f, 'note': 'one launch per rank: per-row partials stored into every peer, rows normalised as they complete; '
                           'parity = h16 and x equal, on every rank and on two consecutive calls, to the apply kernel on the rank-ordered sum of the all-gathered partials'}
            barrier(); fused.close(); barrier()              # (every rank has unmapped before any buffer can go)
        except Exception as e:      # (peer mapping refused on this box: keep the collective form's number)
            tp['fused'] = {'unavailable': f'{type(e).__name__}: {e}'[:200]}
        # the fused kernel run by this rank alone on the same shard (world = 1: it waits for its own partial only): the kernel's HBM side
        try:
            one = D.TPRmsNormFused(norm.nw, Ns, T, 1e-6, group=D.SOLO)
            for _ in range(3): one(xs, ds, hs)
            torch.cuda.synchronize(dev)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            for _ in range(args.steps): one(xs, ds, hs)
            ev[1].record(); ev[1].synchronize(); one.check()
            t1 = ev[0].elapsed_time(ev[1]) * 1e-3 / args.steps
            tp['fused_one_rank'] = {'us_per_step': t1 * 1e6, 'frac_of_peak': T * 4 * Ns * 2 / t1 / 1e9 / peaks()[0]}
        except Exception as e:
            tp['fused_one_rank'] = {'unavailable': f'{type(e).__name__}: {e}'[:200]}
        barrier()
        del xs, xs0, ds, hs, xa, xb, h_ref, h_nccl, parts, tot

    from caminus_b200 import host
    # rows of the host-buffer leg: the whole workload when the host can pin it for every rank (209 KB per row and rank, twice: the
    # batch and the plain-copy check below share the buffers), else as many as a third of the available host memory holds
    row_bytes = sum(BYTES_PER_TOKEN.values()) + HIDDEN * 2           # (the residual comes in too)
    avail = host_mem_available()
    fit = int(avail / 3 / world / row_bytes) // 1024 * 1024 if avail else 16384
    Te = min(T, args.e2e_rows if args.e2e_rows > 0 else max(1024, fit))
    rows_note = 'the whole batch' if Te == T else (f'--e2e-rows {args.e2e_rows}' if args.e2e_rows > 0 else
                                                   f'{Te} rows: a third of the {avail / 2**30:.0f} GiB of available host memory over {world} ranks at {row_bytes} pinned bytes per row')
    e2e = None
    if not args.skip_e2e:
        Hrun = host.HostLayerGlue(Te, HIDDEN, NH, NKV, INTER, nw, par, dev, chunk=args.e2e_chunk)
        Hrun.fill_from(x, resid, q, k, gate, up)
        del gate, up, yq, h16, x, q, k, resid
        torch.cuda.empty_cache()
        for _ in range(3 if Te <= 16384 else 2): Hrun.run()
        barrier()
        e2e_steps = max(2, min(args.steps, 5 if Te <= 16384 else 3))
        t0 = time.perf_counter()
        for _ in range(e2e_steps): Hrun.run()
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        # the host link alone: the same pinned buffers, the same bytes, plain copies in both directions at once (no kernel), every rank
        # at the same time: what the copies of one step cost on this box at this N
        link_s = Hrun.copies_only()
        barrier()
        t0 = time.perf_counter()
        for _ in range(2): Hrun.copies_only()
        barrier()
        link_s = (time.perf_counter() - t0) / 2
        if world > 1:
            t = torch.tensor([e2e_s, link_s], device=dev, dtype=torch.float64); torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            e2e_s, link_s = float(t[0].item()), float(t[1].item())
        e2e = {'value': Te * world / e2e_s, 'unit': 'tokens/s', 'rows_per_gpu': Te, 'rows_note': rows_note, 'h2d_bytes_per_step': Hrun.h2d_bytes,
               'd2h_bytes_per_step': Hrun.d2h_bytes, 'ms_per_step': e2e_s * 1e3,
               'host_link': {'ms_copies_only': link_s * 1e3, 'h2d_gbs_per_gpu': Hrun.h2d_bytes / link_s / 1e9, 'd2h_gbs_per_gpu': Hrun.d2h_bytes / link_s / 1e9,
                             'gbs_all_gpus_both_ways': (Hrun.h2d_bytes + Hrun.d2h_bytes) * world / link_s / 1e9,
                             'tokens_per_s_if_only_copies': Te * world / link_s, 'frac_of_copies_only': link_s / e2e_s,
                             'note': 'the same pinned buffers and bytes as a step, copied in and out concurrently with no kernel between, all ranks at once'}}

    if rank == 0:
        peak, which = peaks()
        names = ['add_rms_f16', 'qk_rope_f16', 'swiglu_q8_1_f16']
        med = np.median(per, 0)
        kern = {n: {'us': float(med[i] * 1e6), 'gbs': T * BYTES_PER_TOKEN[n] / float(med[i]) / 1e9,
                    'frac': T * BYTES_PER_TOKEN[n] / float(med[i]) / 1e9 / peak} for i, n in enumerate(names)}
        dom = 'swiglu_q8_1_f16'
        ach = T * BYTES_PER_TOKEN[dom] / float(per[:, 2].mean()) / 1e9
        cpu = None
        if not args.skip_cpu:
            import oracle
            threads = oracle.default_threads()
            cs = cpu_layer_glue(args.cpu_sample, threads)
            cpu = {'value': args.cpu_sample / cs, 'unit': 'tokens/s', 'cores': threads, 'kind': 'port',
                   'sample': f'{args.cpu_sample} token rows through all three ops (the C oracle, rows split over {threads} host threads)'}
        line = {
            'metric': METRIC, 'value': value, 'unit': 'tokens/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32',
            'data': 'synthetic',
            'config': {'workload': f'per-layer glue, Qwen3-32B shape: T = {T} token rows per GPU, hidden {HIDDEN}, {NH} q + {NKV} kv '
                                   f'heads x 128, intermediate {INTER}, fp16 storage, fp32 arithmetic', 'rows_per_gpu': T,
                       'parallelism': f'token rows x {world} (no collective)', 'l2': 'inputs (13.7 GB per step) larger than L2',
                       'bytes_per_token': sum(BYTES_PER_TOKEN.values())},
            'clocks': clk,
            'e2e': e2e,
            'gpu_launches': 3 * args.steps, 'gpu_launches_note': 'the three glue kernels per timed step (the e2e, ops and tensor-parallel legs launch more, outside the timed region)',
            'roofline': {'bound': 'hbm', 'kernel': 'swiglu_q8_fast_kernel<fp16> (SwiGLU + Q8_1)', 'achieved': ach, 'peak': peak, 'unit': 'GB/s',
                         'frac': ach / peak, 'peak_source': which, 'frac_of_8tbs': ach / 8000.0, 'traffic': SWIGLU_DRAM_BYTES_PER_TOKEN * T,
                         'traffic_note': 'bytes per launch, scaled by rows from an ncu capture at T = 8192', 'algorithmic_bytes': T * BYTES_PER_TOKEN[dom]},
            'kernels': kern,
            'hbm_gbs_all_three': T * sum(BYTES_PER_TOKEN.values()) / (total / args.steps) / 1e9,
            'cpu_baseline': cpu,
            'tp_rmsnorm': tp,
        }
        line['ops'] = single_op_lines(torch, dev, peak, tuple(o for o in args.only.split(',') if o), headline=not args.ops)
        print(json.dumps(line), flush=True)
    if world > 1: torch.distributed.destroy_process_group()


if __name__ == '__main__':
    main()
