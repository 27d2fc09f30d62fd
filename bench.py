"""Benchmark of the block-sparse operator path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras | --extras LIST]

One step = one pass of the hot path over one batch of seeded synthetic input.  The headline workload
is SparseLinear fp16, x[4096 tokens, 4096] . W[4096, 4096]^T + b with a 32x32-block weight mask at 75 %
block sparsity (dsd, weight held as BCSR values); metric = TFLOP/s on the FLOPs of the kept blocks.
With N > 1 every rank runs that workload on its own shard of 4096 token rows (weak scaling, no
collective on the data path).  Rank 0 prints ONE JSON line.

At every N the line also carries ``ranks`` (minimum / median / maximum over the ranks of the headline step
and of the end-to-end step, and each rank's host <-> device copy rate) and ``extras.attention_c5_sharded``:
the large attention configuration (bf16, 64 x 32 heads, S 8192, D 128) with its batch x head dimension
sharded over the N ranks, forward time per rank, and the optional all-gather of the outputs over NVLink
(NCCL) timed separately.

Extras (rank 0, N = 1): the other sparsities and the dds form, a dense fp16 GEMM of the same shape beside the
headline, the fused sparse attention forward (B4 H16 S4096 D64, ms), the GPU mask -> BCSR conversion of 32
masks of 2048 x 2048 (us, GB/s), that conversion plus the dds matmul (dynamic sparsity), the fp32 README
workload, and -- when the reference's own kernels have been compiled (``oracle/_ref``) -- those kernels on
the README and notebook workloads of the reference (``ref_gpu``).  ``--extras refgrid`` (not in the default
set) runs the grid of the reference's own benchmark scripts: M 3072, K 768, N 4096, mask granularity
1 / 8 / 32, twelve sparsities.

``--impl reference`` times the reference's own way of computing the same thing on the host cores:
masked-dense torch (the computation its unit tests compare against), via the oracle.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOKENS, IN_F, OUT_F, BLOCK = 4096, 4096, 4096, 32
SPARSITY = 0.75
# dram__bytes_read.sum + dram__bytes_write.sum of one bsmm_dsd_tc_kernel launch on this workload
# (profiles/bsmm_dsd_tc_linear4096_sp75.md); algorithmic bytes are 75.5 MB
DSD75_TRAFFIC_BYTES = 46.17e6
E2E_CHUNK = 1024  # token rows per chunk of the end-to-end pipeline (measured with graph replay: 512 rows 1.00 ms, 1024 rows 0.945 ms, 2048 rows 1.02 ms per step)


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return {'hbm_gbs': p['hbm_gbs'], 'tflops': p['bf16_tflops'],
                'tflops_sustained': p.get('bf16_tflops_sustained', p['bf16_tflops']), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'tflops': 1590.0, 'tflops_sustained': 1400.0, 'source': 'fallback'}


# ------------------------------------------------------------------------------------------------
# synthetic inputs (seeded on the CPU so that every rank and the CPU baseline see the same bits)
# ------------------------------------------------------------------------------------------------

def linear_inputs(sparsity, seed=2023, tokens=TOKENS):
    from oracle import oracle  # input generator shared with the checker; not on the timed path
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, IN_F), generator=g).half()
    w = (torch.randn((OUT_F, IN_F), generator=g) * 0.02).half()
    b = torch.randn((OUT_F,), generator=g).half()
    mask = oracle.block_mask((OUT_F, IN_F), (BLOCK, BLOCK), sparsity, generator=g)
    return x, w * mask, b, mask


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, device_index):
        self.index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.QUERY}', '--format=csv,noheader,nounits', '-lms', '100',
                 '-i', str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [s.strip() for s in line.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'], f[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        sm.sort()
        return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': sorted(reasons), 'samples': len(sm)}


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so that the next step starts cold."""

    def __init__(self, device, nbytes=256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.fill_(1)


def time_steps(fn, steps, warmup, flush, barrier=None):
    """Per-step CUDA-event timing on the current stream, L2 flushed (untimed) before every step.
    Returns the summed milliseconds of the ``steps`` timed steps."""
    for _ in range(warmup):
        flush()
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush()
        starts[i].record()
        fn()
        stops[i].record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return sum(s.elapsed_time(e) for s, e in zip(starts, stops))


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------

def token_tile():
    """Token rows per CTA tile of the dsd kernel: 128 for the tcgen05 kernel, 64 for the FMA kernel."""
    from sparta_b200 import _lib
    first = _lib.tile_table(_lib.OP_DSD, _lib.F16)[0]
    return first.block_m if first.impl == _lib.IMPL_TCGEN05 else 64


def build_linear(device, sparsity, mode='dsd', tokens=TOKENS, like=None):
    """``like``: an earlier result whose weight, bias and mask are reused (with its first ``tokens`` rows of x)."""
    import sparta_b200 as sparta
    if like is None:
        x, w, b, mask = linear_inputs(sparsity, tokens=tokens)
    else:
        x, w, b, mask = like['x'][:tokens], like['w'], like['b'], like['mask']
    dense = torch.nn.Linear(IN_F, OUT_F, device=device, dtype=torch.float16)
    dense.load_state_dict({'weight': w.to(device), 'bias': b.to(device)})
    if mode == 'dsd':
        op = sparta.nn.SparseLinear(dense, weight_mask=mask.to(device))
        cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': token_tile(), 'BLOCK_SIZE_K_VALUE': BLOCK,
               'BLOCK_SIZE_N_VALUE': BLOCK}
    else:
        # dds: dense operands, output restricted to the same block pattern over [tokens, out]
        op = sparta.nn.SparseBatchMatMul(C_mask=mask[:tokens].to(device), transpose_B=True, compressed=True)
        cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': BLOCK, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': BLOCK}
    xd = x.to(device)
    if mode == 'dsd':
        op.build({'forward:C': cfg}, sample_inputs=[xd])
        nnz = op.get_sparse_indexes('B').block_nnz
        fn = lambda: op(xd)
    else:
        wd = w.to(device).unsqueeze(0)
        xd3 = xd.unsqueeze(0)
        op.build({'forward:C': cfg}, sample_inputs=[xd3, wd])
        nnz = op.get_sparse_indexes('C').block_nnz
        fn = lambda: op(xd3, wd)
    flops = 2.0 * (tokens * BLOCK * BLOCK * nnz if mode == 'dsd' else BLOCK * BLOCK * IN_F * nnz)
    if mode == 'dsd':
        bytes_ = 2.0 * (tokens * IN_F + tokens * OUT_F + nnz * BLOCK * BLOCK + OUT_F)
    else:
        bytes_ = 2.0 * (tokens * IN_F + OUT_F * IN_F + nnz * BLOCK * BLOCK)
    return dict(op=op, fn=fn, x=x, w=w, b=b, mask=mask, xd=xd, nnz=nnz, flops=flops, bytes=bytes_)



def _sparse_linear_fp(device, x, w, b, mask, tile, dtype):
    """SparseLinear (weight mask) built for ``tile`` = (BM, BK, BN) on ``dtype`` copies of the inputs."""
    import sparta_b200 as sparta
    dense = torch.nn.Linear(w.shape[1], w.shape[0], device=device, dtype=dtype)
    dense.load_state_dict({'weight': (w * mask).to(device=device, dtype=dtype), 'bias': b.to(device=device, dtype=dtype)})
    op = sparta.nn.SparseLinear(dense, weight_mask=mask.to(device))
    xd = x.to(device=device, dtype=dtype)
    op.build({'forward:C': {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': tile[0], 'BLOCK_SIZE_K_VALUE': tile[1],
                            'BLOCK_SIZE_N_VALUE': tile[2]}}, sample_inputs=[xd])
    return op, xd


def ref_gpu_extras(device, timed):
    """The reference's dsd kernels (32 x 32 x 32 ``sparta`` tile with 4 x 4 x 4 thread tiles, and the fixed
    32 x 64 x 32 ``openai`` kernel; fp32, the only type they have) on two workloads of the reference itself:
    the README example (1024^3, 8 x 8-block mask, 90 %) and the notebook examples/sparse_linear.ipynb
    (4096 x 3072 -> 768, 32 x 32 blocks, 80 %).  ``kernel_us`` times the kernel alone on a pre-zeroed
    output; ``call_us`` adds the torch.zeros the reference allocates per call
    (sparta/specializer/kernels/matmul.py:171).  This library runs beside it in fp32 (FMA kernel) and fp16
    (tcgen05 kernel) through the public operator."""
    from oracle import oracle, ref_kernels
    ref = ref_kernels.ReferenceKernels()
    out = {}
    for name, (M, K, N, gran, sp) in {'readme_1024_8x8_90': (1024, 1024, 1024, 8, 0.9),
                                      'notebook_4096x3072x768_32x32_80': (4096, 3072, 768, 32, 0.8)}.items():
        g = torch.Generator().manual_seed(2022)
        x = torch.rand((M, K), generator=g)
        w = torch.rand((N, K), generator=g)
        b = torch.rand((N,), generator=g)
        mask = oracle.block_mask((N, K), (gran, gran), sp, generator=g)
        xd, wd, bd, md = x.to(device), (w * mask).to(device), b.to(device), mask.to(device)
        want = torch.nn.functional.linear(xd, wd, bd)
        rec = {}
        for impl, tile in (('sparta', (32, 32, 32)), ('openai', (32, 64, 32))):
            ix = ref.build_indexes(md, tile[2], tile[1], True, False)  # dsd, B stored [N, K]: BN x BK blocks, BCSR
            wc = ref.convert(wd.unsqueeze(0), ix)
            c = torch.zeros((1, M, N), device=device)
            got = ref.matmul(impl, 'dsd', xd.unsqueeze(0), wc, bd.unsqueeze(0), ix, M, K, N, False, True, True)
            err = float((got[0] - want).abs().max())
            kernel_ms = timed(lambda: ref.matmul(impl, 'dsd', xd.unsqueeze(0), wc, bd.unsqueeze(0), ix, M, K, N,
                                                 False, True, True, out=c), steps=10)
            call_ms = timed(lambda: ref.matmul(impl, 'dsd', xd.unsqueeze(0), wc, bd.unsqueeze(0), ix, M, K, N,
                                               False, True, True), steps=10)
            rec[f'reference_{impl}_fp32'] = {'kernel_us': round(kernel_ms * 1e3, 2), 'call_us': round(call_ms * 1e3, 2),
                                             'covering_blocks': ix['nnz'], 'max_abs_err_vs_dense': err}
        small = gran < 32
        op, xs = _sparse_linear_fp(device, x, w, b, mask, (64, gran, gran) if small else (64, 32, 32), torch.float32)
        rec['this_library_fp32'] = {'call_us': round(timed(lambda: op(xs), steps=10) * 1e3, 2),
                                    'max_abs_err_vs_dense': float((op(xs) - want).abs().max())}
        if not small:
            op16, x16 = _sparse_linear_fp(device, x, w, b, mask, (token_tile(), 32, 32), torch.float16)
            rec['this_library_fp16'] = {'call_us': round(timed(lambda: op16(x16), steps=10) * 1e3, 2)}
        rec['dense_torch_fp32_us'] = round(timed(lambda: torch.nn.functional.linear(xd, wd, bd), steps=10) * 1e3, 2)
        out[name] = rec
    return out


def refgrid_extras(device, timed):
    """Forward latency over the grid of the reference's benchmark scripts
    (test/bench/matmul/matmul.py:18-23: M 3072, K 768, N 4096, mask granularity 1 / 8 / 32, twelve
    sparsities; B sparse, stored [N, K], compressed), in microseconds: torch dense fp32 and fp16, this
    library fp32 (FMA kernel, 32 x 32 blocks over the finer mask like the reference's tuned configurations)
    and fp16 (tcgen05), and the reference's 32 x 64 x 32 kernel when compiled."""
    from oracle import oracle, ref_kernels
    M, K, N = 3072, 768, 4096
    ref = ref_kernels.ReferenceKernels() if ref_kernels.available() else None
    rows = []
    for gran in (1, 8, 32):
        for sp in (0, 0.2, 0.4, 0.6, 0.8, 0.9, 0.95, 0.99, 0.995, 0.999, 0.9995, 0.9999):
            g = torch.Generator().manual_seed(2022)
            x = torch.rand((M, K), generator=g)
            w = torch.rand((N, K), generator=g)
            b = torch.zeros((N,))
            mask = oracle.block_mask((N, K), (gran, gran), sp, generator=g)
            if int(mask.sum()) == 0:
                continue
            xd, wd = x.to(device), (w * mask).to(device)
            row = {'granularity': gran, 'sparsity': sp,
                   'dense_fp32_us': round(timed(lambda: torch.matmul(xd, wd.T), steps=5) * 1e3, 1)}
            xh, wh = xd.half(), wd.half()
            row['dense_fp16_us'] = round(timed(lambda: torch.matmul(xh, wh.T), steps=5) * 1e3, 1)
            op, xs = _sparse_linear_fp(device, x, w, b, mask, (64, 32, 32), torch.float32)
            row['ours_fp32_us'] = round(timed(lambda: op(xs), steps=5) * 1e3, 1)
            row['covering_blocks_32x32'] = op.get_sparse_indexes('B').block_nnz
            op16, x16 = _sparse_linear_fp(device, x, w, b, mask, (token_tile(), 32, 32), torch.float16)
            row['ours_fp16_us'] = round(timed(lambda: op16(x16), steps=5) * 1e3, 1)
            if ref is not None:
                md = mask.to(device)
                ix = ref.build_indexes(md, 32, 64, True, False)
                wc = ref.convert(wd.unsqueeze(0), ix)
                c = torch.zeros((1, M, N), device=device)
                row['reference_openai_fp32_us'] = round(timed(
                    lambda: ref.matmul('openai', 'dsd', xd.unsqueeze(0), wc, None, ix, M, K, N, False, True, True, out=c),
                    steps=5) * 1e3, 1)
            rows.append(row)
            del op, op16
    return rows


def refgrid_attention_extras(device, timed):
    """Forward and backward latency over the grid of the reference's attention benchmark
    (test/bench/attention/attention.py:18-23: one head, Ns 4096, Nt 3072, E 768, uniform [0, 1) inputs, mask
    granularity 1 / 8 / 32; five of its twelve sparsities), in microseconds: the masked dense softmax attention in
    torch (fp32), this library's three-operator SparseAttention in fp32 (FMA kernels, 32 x 32 tiles) and in fp16 with
    every matmul on a tcgen05 tile.  E = 768 is outside the fused kernel (64 / 128), as in the reference."""
    import sparta_b200 as sparta
    from oracle import oracle
    Ns, Nt, E = 4096, 3072, 768
    mm = lambda m, k, n, fam: {'_impl': 'sparta', '_family': fam, 'BLOCK_SIZE_M_VALUE': m, 'BLOCK_SIZE_K_VALUE': k,
                               'BLOCK_SIZE_N_VALUE': n}
    sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 32, 'BLOCK_SIZE_W_VALUE': 32, 'ROW_TILE_VALUE': 4}
    slots = ['qk/forward:C', 'qk/backward:A', 'qk/backward:B', 'out/forward:C', 'out/backward:A', 'out/backward:B']
    fma_cfg = {**{n: mm(32, 32, 32, 'simt') for n in slots}, 'sm/forward:y': sm, 'sm/backward:x': sm}
    dds, sdd = mm(32, 64, 32, 'tcgen05'), mm(32, 32, 128, 'tcgen05')
    tc_cfg = {'qk/forward:C': dds, 'qk/backward:A': sdd, 'qk/backward:B': sdd, 'out/forward:C': sdd,
              'out/backward:A': dds, 'out/backward:B': sdd, 'sm/forward:y': sm, 'sm/backward:x': sm}
    rows = []
    for gran in (1, 8, 32):
        for sp in (0, 0.6, 0.9, 0.99, 0.999):
            g = torch.Generator().manual_seed(2022)
            q = torch.rand((1, Nt, E), generator=g)
            k, v = torch.rand((1, Ns, E), generator=g), torch.rand((1, Ns, E), generator=g)
            go = torch.rand((1, Nt, E), generator=g)
            mask = oracle.block_mask((Nt, Ns), (gran, gran), sp, generator=g)
            if int(mask.sum()) == 0:
                continue
            md = mask.to(device)
            row = {'granularity': gran, 'sparsity': sp}

            def fwd_bwd(fn, q_, k_, v_, go_):
                q_.grad = k_.grad = v_.grad = None
                fn(q_, k_, v_).backward(go_)

            def dense(q_, k_, v_):
                s_ = torch.matmul(q_, k_.transpose(1, 2)) / (E ** 0.5)
                s_ = s_.masked_fill(md == 0, float('-inf'))
                p_ = torch.nan_to_num(torch.softmax(s_, dim=-1))
                return torch.matmul(p_, v_)
            legs = [('dense_fp32', dense, torch.float32, None), ('ours_fp32', None, torch.float32, fma_cfg),
                    ('ours_fp16_tcgen05', None, torch.float16, tc_cfg)]
            for name, fn, dtype, cfg in legs:
                qd, kd, vd = (t.to(device=device, dtype=dtype).requires_grad_() for t in (q, k, v))
                gd = go.to(device=device, dtype=dtype)
                if fn is None:
                    op = sparta.nn.SparseAttention(mask=md, fused=False)
                    op.build(cfg, sample_inputs=[qd, kd, vd])
                    fn = op
                with torch.no_grad():
                    row[name + '_fwd_us'] = round(timed(lambda: fn(qd, kd, vd), steps=5) * 1e3, 1)
                row[name + '_fwd_bwd_us'] = round(timed(lambda: fwd_bwd(fn, qd, kd, vd, gd), steps=5) * 1e3, 1)
            rows.append(row)
    return rows


def run_extras(device, peaks, flush, only=None):
    """Secondary measurements (each: 3 warm-ups, 10 timed steps, L2 flushed between steps)."""
    import sparta_b200 as sparta
    from oracle import oracle
    extras = {}

    def timed(fn, steps=10, do_flush=True):
        return time_steps(fn, steps, 3, flush if do_flush else (lambda: None)) / steps

    want = lambda name: only is None or name in only
    for mode in (('dsd', 'dds') if want('linear') else ()):
        for sp in (0.75, 0.9, 0.95):
            if mode == 'dsd' and sp == SPARSITY:
                continue
            try:
                wl = build_linear(device, sp, mode)
                ms = timed(wl['fn'])
                tf = wl['flops'] / ms / 1e9
                extras[f'linear_{mode}_{int(sp * 100)}'] = {
                    'ms': round(ms, 4), 'nnz_blocks': wl['nnz'], 'tflops': round(tf, 2),
                    'frac_tensor_peak': round(tf / peaks['tflops'], 4),
                    'gbs': round(wl['bytes'] / ms / 1e6, 1), 'frac_hbm_peak': round(wl['bytes'] / ms / 1e6 / peaks['hbm_gbs'], 4)}
                del wl
            except Exception as e:  # an extra must not take the headline number down
                extras[f'linear_{mode}_{int(sp * 100)}'] = {'error': repr(e)[:200]}

    # SparseLinear training step at 75 % (forward, input gradient = dsd with the BCSC weight, weight gradient = dds
    # with A stored [K, M]), all three on tcgen05 tiles, beside the same step on the FMA tiles
    try:
        if not want('linear_train'):
            raise KeyError('skipped')
        x, w, b, mask = linear_inputs(SPARSITY)
        gy = torch.randn((TOKENS, OUT_F), generator=torch.Generator().manual_seed(5)).half().to(device)
        rec = {}
        for fam, tiles in (('tcgen05', ((128, 32, 32), (128, 32, 32), (32, 64, 32))),
                           ('simt', ((64, 32, 32), (64, 32, 32), (32, 64, 32)))):
            dense = torch.nn.Linear(IN_F, OUT_F, device=device, dtype=torch.float16)
            dense.load_state_dict({'weight': w.to(device), 'bias': b.to(device)})
            op = sparta.nn.SparseLinear(dense, weight_mask=mask.to(device))
            xd = x.to(device).requires_grad_(True)
            op.build({name: {'_impl': 'sparta', '_family': fam, 'BLOCK_SIZE_M_VALUE': t[0], 'BLOCK_SIZE_K_VALUE': t[1],
                             'BLOCK_SIZE_N_VALUE': t[2]}
                      for name, t in zip(('forward:C', 'backward:A', 'backward:B'), tiles)}, sample_inputs=[xd.detach()])
            nnz = op.get_sparse_indexes('B').block_nnz

            def step():
                xd.grad = None
                op.weight.grad = None
                op(xd).backward(gy)
            ms = timed(step)
            ctx = op._sparse_ctx
            wv = op.weight.detach().unsqueeze(0)
            parts = {'fwd_ms': timed(lambda: ctx.forward_C(xd.detach().unsqueeze(0), wv, op.bias.detach().unsqueeze(0))),
                     'dgrad_ms': timed(lambda: ctx.backward_A(gy.unsqueeze(0), wv)),
                     'wgrad_ms': timed(lambda: ctx.backward_B(gy.unsqueeze(0), xd.detach().unsqueeze(0)))}
            tf = 3 * 2.0 * TOKENS * BLOCK * BLOCK * nnz / ms / 1e9
            rec[fam] = {'step_ms': round(ms, 4), **{k: round(v, 4) for k, v in parts.items()}, 'tflops': round(tf, 2),
                        'frac_tensor_peak': round(tf / peaks['tflops'], 4)}
            del op, dense
        rec['nnz_blocks'] = nnz
        extras['linear_train_75'] = rec
    except KeyError:
        pass
    except Exception as e:
        extras['linear_train_75'] = {'error': repr(e)[:200]}

    # fused sparse attention forward: B4 H16 S4096 D64 fp16, band + global + 5 % random 64x64 blocks
    try:
        if not want('attention'):
            raise KeyError('skipped')
        heads, S, D = 64, 4096, 64
        g = torch.Generator().manual_seed(2024)
        q, k, v = (torch.randn((heads, S, D), generator=g).half().to(device) for _ in range(3))
        amask = oracle.band_global_random_mask(S, S, 64, 8, 0.05, seed=0).to(device)
        attn = sparta.nn.SparseAttention(mask=amask)
        mm = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 64}
        sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 64, 'BLOCK_SIZE_W_VALUE': 64, 'ROW_TILE_VALUE': 4}
        attn.build({'qk/forward:C': mm, 'sm/forward:y': sm, 'out/forward:C': mm}, sample_inputs=[q, k, v])
        nnz = attn.get_sparse_indexes().block_nnz
        ms = timed(lambda: attn(q, k, v), steps=5)
        flops = 4.0 * heads * nnz * 64 * 64 * D
        extras['attention_b4h16s4096d64'] = {
            'fwd_ms': round(ms, 4), 'nnz_blocks': nnz, 'fused': bool(attn._use_fused),
            'tflops': round(flops / ms / 1e9, 2), 'frac_tensor_peak': round(flops / ms / 1e9 / peaks['tflops'], 4)}
        del q, k, v, attn
    except Exception as e:
        extras['attention_b4h16s4096d64'] = {'error': repr(e)[:200]}

    # one rank's share of the large attention configuration at 1/32 of its head count: bf16, 64 heads, S 8192,
    # D 128 (403 MB of q, k, v, o): the case the kernel with two Q tiles per CTA is profiled on
    try:
        if not want('attention_d128'):
            raise KeyError('skipped')
        heads, S, D = 64, 8192, 128
        dg = torch.Generator(device=device).manual_seed(2026)
        q, k, v = (torch.randn((heads, S, D), generator=dg, device=device, dtype=torch.bfloat16) for _ in range(3))
        amask = oracle.band_global_random_mask(S, S, 64, 8, 0.05, seed=0).to(device)
        attn = sparta.nn.SparseAttention(mask=amask)
        mm = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 64}
        sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 64, 'BLOCK_SIZE_W_VALUE': 64, 'ROW_TILE_VALUE': 4}
        attn.build({'qk/forward:C': mm, 'sm/forward:y': sm, 'out/forward:C': mm}, sample_inputs=[q, k, v])
        nnz = attn.get_sparse_indexes().block_nnz
        with torch.no_grad():
            ms = timed(lambda: attn(q, k, v), steps=5)
        flops = 4.0 * heads * nnz * 64 * 64 * D
        extras['attention_h64s8192d128_bf16'] = {
            'fwd_ms': round(ms, 4), 'nnz_blocks': nnz, 'fused': bool(attn._use_fused),
            'tflops': round(flops / ms / 1e9, 2), 'frac_tensor_peak': round(flops / ms / 1e9 / peaks['tflops'], 4)}
        del q, k, v, attn
    except Exception as e:
        extras['attention_h64s8192d128_bf16'] = {'error': repr(e)[:200]}

    # stand-alone SparseSoftmax forward on compressed scores of the same attention mask (the fused kernel
    # above never materialises them; this is the operator the unfused composition and the API expose)
    try:
        if not want('softmax'):
            raise KeyError('skipped')
        heads, S = 64, 4096
        amask = oracle.band_global_random_mask(S, S, 64, 8, 0.05, seed=0).to(device)
        sop = sparta.nn.SparseSoftmax(amask, 8.0, compressed=True)
        dg = torch.Generator(device=device).manual_seed(7)
        xd = torch.randn((heads, S, S), generator=dg, device=device, dtype=torch.float16)
        tile = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 64, 'BLOCK_SIZE_W_VALUE': 64, 'ROW_TILE_VALUE': 4}
        sop.build({'forward:y': tile, 'backward:x': tile}, sample_inputs=[xd])
        six = sop.get_sparse_indexes('y')
        xc = six.convert(xd)
        del xd
        nnz = six.block_nnz
        nbytes = 2.0 * heads * nnz * 64 * 64 * 2  # read x + write y, kept blocks only (1.35 GB: larger than L2)
        with torch.no_grad():
            ms = time_steps(lambda: sop(xc), 5, 3, lambda: None) / 5
            yc = sop(xc)
            gc = torch.randn(xc.shape, generator=dg, device=device, dtype=torch.float16)
            bwd_ms = time_steps(lambda: sop._sparse_ctx.backward(gc, yc), 5, 3, lambda: None) / 5
        extras['softmax_b4h16s4096_compressed'] = {
            'fwd_ms': round(ms, 4), 'nnz_blocks': nnz, 'gbs': round(nbytes / ms / 1e6, 1),
            'frac_hbm_peak': round(nbytes / ms / 1e6 / peaks['hbm_gbs'], 4), 'l2': 'operands (1.35 GB) larger than L2, no flush',
            'bwd_ms': round(bwd_ms, 4), 'bwd_gbs': round(1.5 * nbytes / bwd_ms / 1e6, 1),  # reads dy and y, writes dx
            'bwd_frac_hbm_peak': round(1.5 * nbytes / bwd_ms / 1e6 / peaks['hbm_gbs'], 4)}
        del xc, yc, gc, sop
    except Exception as e:
        extras['softmax_b4h16s4096_compressed'] = {'error': repr(e)[:200]}

    # mask -> BCSR on the GPU: 32 masks of 2048 x 2048, 32x32 blocks, 90 % sparse
    try:
        if not want('convert'):
            raise KeyError('skipped')
        gdev = torch.Generator(device=device).manual_seed(7)
        coarse = (torch.rand((32, 64, 64), device=device, generator=gdev) > 0.9).to(torch.uint8)
        masks = coarse.repeat_interleave(32, 1).repeat_interleave(32, 2).contiguous()
        fnc = sparta.tesa.get_bcs_function(32, 32, True, False)
        # the 134 MB input is larger than the 126 MB L2, so no flush is interposed here (a flush leaves
        # 126 MB of dirty lines whose write-back would be charged to this read-only kernel)
        ms_api = timed(lambda: fnc.build_indexes(masks), steps=20, do_flush=False)
        # the same conversion through the C ABI with caller-owned outputs (no per-call allocation)
        from sparta_b200 import _lib
        L = _lib.lib()
        i32 = dict(dtype=torch.int32, device=device)
        row_ptr, idxb, cnt = torch.empty((32, 65), **i32), torch.empty((32, 4096), **i32), torch.empty((2, 32), **i32)
        nb = L.sparta_bcs_build_workspace_bytes(32, 2048, 2048, 32, 32)
        ws = torch.zeros(nb, dtype=torch.uint8, device=device)
        ptrs = (masks.data_ptr(), row_ptr.data_ptr(), idxb.data_ptr(), cnt[0].data_ptr(), cnt[1].data_ptr(), ws.data_ptr())
        stream = _lib.stream_ptr(device)

        def convert_cabi():
            _lib.check(L.sparta_bcs_build(ptrs[0], 32, 2048, 2048, 32, 32, 1, 0, ptrs[1], ptrs[2], None, None, 4096,
                                          ptrs[3], ptrs[4], None, ptrs[5], nb, stream), 'sparta_bcs_build')
        ms = timed(convert_cabi, steps=20, do_flush=False)
        gbs = masks.numel() / ms / 1e6
        extras['bcsr_convert_32x2048x2048'] = {'us': round(ms * 1e3, 2), 'gbs': round(gbs, 1),
                                               'frac_hbm_peak': round(gbs / peaks['hbm_gbs'], 4),
                                               'us_python_api': round(ms_api * 1e3, 2),
                                               'l2': 'input (134 MB) larger than L2, no flush',
                                               'note': 'us: sparta_bcs_build through the C ABI with caller-owned '
                                                       'outputs; us_python_api: build_indexes() incl. allocations'}
        # dynamic sparsity: conversion + dds matmul, A[32,2048,128] . B[32,128,2048]
        g = torch.Generator().manual_seed(8)
        A = torch.randn((32, 2048, 128), generator=g).half().to(device)
        B = torch.randn((32, 128, 2048), generator=g).half().to(device)
        op = sparta.nn.SparseBatchMatMul(C_mask=masks, compressed=True, capacity=1024)
        cfg = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 32, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 32}
        op.build({'forward:C': cfg}, sample_inputs=[A, B])
        op.set_dynamic(True)
        ms = timed(lambda: op(A, B), steps=10)
        nnz_total = int(op.get_sparse_indexes('C').nnz_dev.sum())
        flops = 2.0 * 128 * 32 * 32 * nnz_total
        extras['dynamic_dds_b32_2048x2048_k128'] = {
            'us': round(ms * 1e3, 2), 'nnz_blocks_total': nnz_total, 'tflops': round(flops / ms / 1e9, 3),
            'gbs': round((masks.numel() + 2 * (A.numel() + B.numel()) + 2 * nnz_total * 1024) / ms / 1e6, 1)}
        del A, B, masks, op
    except Exception as e:
        extras['bcsr_convert_32x2048x2048'] = extras.get('bcsr_convert_32x2048x2048', {'error': repr(e)[:200]})
        extras['dynamic_dds_b32_2048x2048_k128'] = {'error': repr(e)[:200]}

    # README workload: fp32, 1024^3, 8x8-block weight mask at 90 %
    try:
        if not want('readme'):
            raise KeyError('skipped')
        g = torch.Generator().manual_seed(2022)
        x = torch.rand((1024, 1024), generator=g).to(device)
        w = torch.rand((1024, 1024), generator=g)
        b = torch.rand((1024,), generator=g)
        mask = oracle.block_mask((1024, 1024), (8, 8), 0.9, generator=g)
        dense = torch.nn.Linear(1024, 1024, device=device)
        dense.load_state_dict({'weight': (w * mask).to(device), 'bias': b.to(device)})
        op = sparta.nn.SparseLinear(dense, weight_mask=mask.to(device))
        op.build({'forward:C': {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 8,
                                'BLOCK_SIZE_N_VALUE': 8}}, sample_inputs=[x])
        ms = timed(lambda: op(x), steps=20)
        nnz = op.get_sparse_indexes('B').block_nnz
        extras['linear_fp32_1024_8x8_90'] = {'us': round(ms * 1e3, 2), 'nnz_blocks': nnz,
                                             'gflops': round(2.0 * 1024 * 64 * nnz / ms / 1e6, 1)}
    except Exception as e:
        extras['linear_fp32_1024_8x8_90'] = {'error': repr(e)[:200]}

    # a dense fp16 GEMM of the headline's shape through torch (cuBLAS), same events and flush: the
    # comparison the reference's own benchmark makes (test/bench/matmul/matmul.py:143-156,192)
    try:
        if not want('dense'):
            raise KeyError('skipped')
        x, w, b, mask = linear_inputs(SPARSITY)
        xd, wd, bd = x.to(device), w.to(device), b.to(device)
        ms = timed(lambda: torch.nn.functional.linear(xd, wd, bd), steps=20)
        kept = int((mask.reshape(OUT_F // BLOCK, BLOCK, IN_F // BLOCK, BLOCK).amax((1, 3)) > 0).sum())
        extras['dense_fp16_4096'] = {
            'ms': round(ms, 4), 'dense_tflops': round(2.0 * TOKENS * IN_F * OUT_F / ms / 1e9, 1),
            'nnz_block_tflops_equiv_75': round(2.0 * TOKENS * BLOCK * BLOCK * kept / ms / 1e9, 1),
            'note': 'torch.nn.functional.linear on the masked-dense fp16 weight (zeros multiplied), library GEMM'}
        del xd, wd, bd
    except Exception as e:
        extras['dense_fp16_4096'] = {'error': repr(e)[:200]}

    # the reference's own kernels (rendered from its templates, compiled for sm_100a) beside this library
    try:
        if not want('ref_gpu'):
            raise KeyError('skipped')
        from oracle import ref_kernels
        if not ref_kernels.available():
            raise RuntimeError('oracle/_ref not built (no checkout of the reference at build time)')
        extras['ref_gpu'] = ref_gpu_extras(device, timed)
    except Exception as e:
        extras['ref_gpu'] = {'error': repr(e)[:200]}

    try:
        if only is None or 'refgrid' not in only:
            raise KeyError('skipped')
        extras['refgrid'] = refgrid_extras(device, timed)
    except Exception as e:
        extras['refgrid'] = {'error': repr(e)[:200]}
    try:
        if only is None or 'refgrid_attention' not in only:
            raise KeyError('skipped')
        extras['refgrid_attention'] = refgrid_attention_extras(device, timed)
    except Exception as e:
        extras['refgrid_attention'] = {'error': repr(e)[:200]}
    return {k: v for k, v in extras.items() if not (isinstance(v, dict) and 'skipped' in str(v.get('error', '')))}



def rank_summary(local, world, device):
    """min / median / max over the ranks of each value of ``local`` (a dict of floats); every rank calls."""
    names = sorted(local)
    mine = torch.tensor([float(local[n]) for n in names], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist
        rows = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(rows, mine)
        table = torch.stack(rows)
    else:
        table = mine.unsqueeze(0)
    out = {}
    for i, n in enumerate(names):
        col = table[:, i].sort().values
        out[n] = {'min': round(float(col[0]), 5), 'median': round(float(col[len(col) // 2]), 5),
                  'max': round(float(col[-1]), 5)}
    return out


def attention_c5_sharded(device, world, rank, peaks, barrier):
    """The large attention configuration -- bf16, 64 x 32 = 2048 heads, S 8192, D 128, the band + global +
    random mask on a 128 x 128 grid of 64 x 64 blocks -- with the batch x head dimension sharded over the
    ranks (``parallel.shard_bounds``); masks and indexes are replicated, there is no exchange on the data
    path.  The optional all-gather of the outputs (NCCL, every rank ends up with all 2048 heads) is timed on
    its own.  Every rank calls; returns the same dictionary on every rank."""
    import sparta_b200 as sparta
    from sparta_b200 import parallel
    from oracle import oracle  # mask generator shared with the checker
    heads_total, S, D = 2048, 8192, 128
    lo, hi = parallel.shard_bounds(heads_total, world, rank)
    heads = hi - lo
    dg = torch.Generator(device=device).manual_seed(2025 + rank)
    q, k, v = (torch.randn((heads, S, D), generator=dg, device=device, dtype=torch.bfloat16) for _ in range(3))
    amask = oracle.band_global_random_mask(S, S, 64, 8, 0.05, seed=0).to(device)
    attn = sparta.nn.SparseAttention(mask=amask)
    mm = {'_impl': 'sparta', 'BLOCK_SIZE_M_VALUE': 64, 'BLOCK_SIZE_K_VALUE': 64, 'BLOCK_SIZE_N_VALUE': 64}
    sm = {'_impl': 'sparta', 'BLOCK_SIZE_H_VALUE': 64, 'BLOCK_SIZE_W_VALUE': 64, 'ROW_TILE_VALUE': 4}
    attn.build({'qk/forward:C': mm, 'sm/forward:y': sm, 'out/forward:C': mm}, sample_inputs=[q, k, v])
    nnz = attn.get_sparse_indexes().block_nnz
    no_flush = lambda: None  # the operands of a rank (17 GB / world) are far larger than L2
    with torch.no_grad():
        fwd_ms = time_steps(lambda: attn(q, k, v), 3, 3, no_flush, barrier) / 3
        o = attn(q, k, v)
    local = {'fwd_ms': fwd_ms}
    gather = {}
    if world > 1:
        import torch.distributed as dist
        full = torch.empty((heads_total, S, D), dtype=o.dtype, device=device)
        ag_ms = time_steps(lambda: parallel.all_gather_outputs(o, out=full), 3, 2, no_flush, barrier) / 3
        local['allgather_ms'] = ag_ms
        received = (heads_total - heads) * S * D * 2
        local['allgather_in_gbs'] = received / ag_ms / 1e6
        ok = bool(torch.equal(full[lo:hi], o))
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather = {'allgather_bytes_received_per_rank': received, 'allgather_own_shard_intact': bool(flag.item()),
                  'collective': 'NCCL all_gather_into_tensor over NVLink / NVSwitch'}
        # the same exchange folded into the attention kernel: every output tile is also stored, from shared memory
        # with bulk tensor stores over NVLink, into this rank's slice of every peer's gathered output (symmetric
        # memory), so the transfer overlaps the remaining tiles' compute and O is not read again
        try:
            gathered = parallel.GatheredHeads(heads, S, D, o.dtype, device)
            with torch.no_grad():
                step = lambda: attn.forward_gathered(q, k, v, gathered.local, gathered.peer_addresses)
                local['fused_gather_ms'] = time_steps(step, 3, 2, no_flush, barrier) / 3
            same = bool(torch.equal(gathered.wait(), full))
            flag = torch.tensor([1 if same else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            gather['fused_gather'] = {'how': 'attention kernel stores each tile to O and to the peers\' buffers (peer memory, '
                                             'cp.async.bulk.tensor stores over NVLink); no separate collective',
                                      'equals_nccl_allgather_bitwise': bool(flag.item())}
            del gathered
        except Exception as e:
            gather['fused_gather'] = {'error': repr(e)[:200]}
            local['fused_gather_ms'] = -1.0  # every rank reports the same keys
        del full
    stats = rank_summary(local, world, device)
    flops = 4.0 * heads_total * nnz * 64 * 64 * D
    worst = stats['fwd_ms']['max']
    out = {'heads_per_rank': heads, 'nnz_blocks': nnz, 'fused': bool(attn._use_fused), 'dtype': 'bf16',
           'fwd_ms': stats['fwd_ms'], 'aggregate_tflops': round(flops / worst / 1e9, 1),
           'frac_tensor_peak_per_gpu': round(flops / world / worst / 1e9 / peaks['tflops'], 4), **gather}
    for name in ('allgather_ms', 'allgather_in_gbs'):
        if name in stats:
            out[name] = stats[name]
    if 'fused_gather_ms' in stats and stats['fused_gather_ms']['min'] >= 0 and 'error' not in out['fused_gather']:
        out['fused_gather']['ms'] = stats['fused_gather_ms']
        out['fused_gather']['separate_passes_ms'] = round(stats['fwd_ms']['max'] + stats['allgather_ms']['max'], 4)
    del q, k, v, o, attn
    torch.cuda.empty_cache()
    return out


def cpu_baseline_linear(x, w, b, repeats=3):
    """Masked-dense torch on the host cores: the computation the reference's tests compare with
    (inputs upcast to fp32; w is already multiplied by its mask)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    xf, wf, bf = x.float(), w.float(), b.float()
    torch.nn.functional.linear(xf[:256], wf, bf)  # warm-up
    best = float('inf')
    for _ in range(repeats):
        t0 = time.perf_counter()
        torch.nn.functional.linear(xf, wf, bf)
        best = min(best, time.perf_counter() - t0)
    return best, cores


def config_dict(n_gpus):
    return {'workload': f'SparseLinear fp16 dsd: x[{TOKENS},{IN_F}] . W[{OUT_F},{IN_F}]^T + b, 32x32-block '
                        f'weight mask, {int(SPARSITY * 100)}% block sparsity',
            'tokens_per_gpu': TOKENS, 'in_features': IN_F, 'out_features': OUT_F, 'block': [BLOCK, BLOCK],
            'sparsity': SPARSITY, 'parallelism': f'token-row shards x{n_gpus}, no collective',
            'l2': 'flushed (256 MB write) before every timed step'}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--no-extras', action='store_true')
    ap.add_argument('--extras', default=None,
                    help='comma list of extra measurements to run: linear,linear_train,dense,attention,attention_d128,attention_c5,softmax,convert,readme,ref_gpu (default: all of these), refgrid and refgrid_attention (only when named)')
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    peaks = load_peaks()
    metric = 'nnz_block_tflops'

    if args.impl == 'reference':
        if rank != 0:
            return
        x, w, b, mask = linear_inputs(SPARSITY)
        nnz = int((mask.reshape(OUT_F // BLOCK, BLOCK, IN_F // BLOCK, BLOCK).amax((1, 3)) > 0).sum())
        flops = 2.0 * TOKENS * BLOCK * BLOCK * nnz
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        xf, wf, bf = x.float(), w.float(), b.float()
        for _ in range(max(args.warmup, 1)):
            torch.nn.functional.linear(xf, wf, bf)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            torch.nn.functional.linear(xf, wf, bf)
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
        value = flops / ms / 1e9
        print(json.dumps({
            'impl': 'reference', 'metric': metric, 'value': value, 'unit': 'TFLOP/s', 'n_gpus': args.gpus,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32 (fp16 inputs upcast)', 'data': 'synthetic',
            'config': config_dict(args.gpus),
            'cpu_baseline': {'value': value, 'unit': 'TFLOP/s', 'cores': cores, 'kind': 'port',
                             'sample': 'whole workload per step: F.linear(x, W*mask, b) in fp32, masked-dense'},
            'e2e': {'value': value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        }))
        return

    assert torch.cuda.is_available(), 'bench.py needs a CUDA device (there is no CPU fallback)'
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    barrier = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=device)
        barrier = lambda: dist.barrier(device_ids=[local_rank])

    wl = build_linear(device, SPARSITY, 'dsd')
    flush = L2Flusher(device)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # device-resident timing (the kernel, plus the output allocation of the operator)
    total_ms = time_steps(wl['fn'], args.steps, args.warmup, flush, barrier)

    # end-to-end through the public operator with host buffers: token rows are independent, so the
    # operator is built for E2E_CHUNK rows and HostStreamedRows overlaps copy-in, kernel and copy-out
    import sparta_b200 as sparta
    x_host = wl['x'].pin_memory()
    y_host = torch.empty((TOKENS, OUT_F), dtype=torch.float16).pin_memory()
    chunk = build_linear(device, SPARSITY, 'dsd', tokens=E2E_CHUNK, like=wl)
    streamed = sparta.nn.HostStreamedRows(chunk['op'], E2E_CHUNK, graph=True)

    def e2e_step():
        streamed(x_host, y_host)

    e2e_how = 'the sequence replayed from a CUDA graph'
    try:
        e2e_step()
        e2e_step()  # the first call ran plainly once, captured and replayed; this one replays
    except Exception:  # capture refused on this box: plain launches
        torch.cuda.synchronize()
        streamed = sparta.nn.HostStreamedRows(chunk['op'], E2E_CHUNK)
        e2e_how = 'plain launches (graph capture failed)'
        e2e_step()
    torch.cuda.synchronize()
    if not torch.allclose(y_host.float(), wl['fn']().float().cpu(), rtol=2e-2, atol=2e-2):
        raise RuntimeError('end-to-end result differs from the device-resident result')
    e2e_ms = time_steps(e2e_step, args.steps, args.warmup, flush, barrier)
    clocks = sampler.stop() if rank == 0 else None

    # per-rank view first (who is slow?), then the maximum over the ranks, which is what the line reports
    h2d_bytes, d2h_bytes = x_host.numel() * 2, y_host.numel() * 2
    ranks = rank_summary({'step_ms': total_ms / args.steps, 'e2e_ms': e2e_ms / args.steps,
                          'e2e_host_link_gbs': (h2d_bytes + d2h_bytes) / (e2e_ms / args.steps) / 1e6}, world, device)
    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = times.tolist()
    ms_per_step = total_ms / args.steps
    value = world * wl['flops'] / ms_per_step / 1e9
    e2e_value = world * wl['flops'] / (e2e_ms / args.steps) / 1e9

    # full-size parity of the headline against the oracle (masked-dense fp32 on the host), outside any timed region
    parity = None
    if rank == 0:
        want = torch.nn.functional.linear(wl['x'][:512].float(), wl['w'].float(), wl['b'].float())
        with torch.no_grad():
            got = wl['fn']()[:512].float().cpu()
        parity = {'max_abs_err': float((got - want).abs().max()), 'tolerance': 2e-2,
                  'checked': 'first 512 token rows of the device-resident headline output against F.linear in fp32 on the host; '
                             'the end-to-end output was checked against the device-resident one'}
        if not torch.allclose(got, want, rtol=2e-2, atol=2e-2):
            raise RuntimeError(f'headline result differs from the oracle: {parity}')

    # the sharded attention configuration runs on every rank, at every N (not for --no-extras)
    c5 = None
    if not args.no_extras and (args.extras is None or 'attention_c5' in args.extras.split(',')):
        del chunk, streamed
        try:
            c5 = attention_c5_sharded(device, world, rank, peaks, barrier)
        except Exception as e:  # an extra must not take the headline number down
            c5 = {'error': repr(e)[:200]}

    if rank == 0:
        kernel_tflops = wl['flops'] / ms_per_step / 1e9
        out = {
            'metric': metric, 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': ms_per_step, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'f16 (fp32 accumulate)', 'data': 'synthetic',
            'config': config_dict(world), 'nnz_blocks': wl['nnz'],
            'roofline': {'bound': 'tensor', 'achieved': kernel_tflops, 'peak': peaks['tflops'], 'unit': 'TFLOP/s',
                         'frac': kernel_tflops / peaks['tflops'], 'traffic': DSD75_TRAFFIC_BYTES,
                         'traffic_note': 'dram read+write per launch from the ncu capture in profiles/ (output stays in L2)',
                         'peak_source': f"{peaks['source']} bf16 burst", 'hbm_gbs': wl['bytes'] / ms_per_step / 1e6,
                         'hbm_frac': wl['bytes'] / ms_per_step / 1e6 / peaks['hbm_gbs']},
            'e2e': {'value': e2e_value, 'unit': 'TFLOP/s', 'ms_per_step': e2e_ms / args.steps,
                    'h2d_bytes_per_step': h2d_bytes, 'd2h_bytes_per_step': d2h_bytes,
                    'how': f'SparseLinear built for {E2E_CHUNK} rows, called through sparta.nn.HostStreamedRows: '
                           f'{TOKENS // E2E_CHUNK} chunks, copy-in / kernel / copy-out overlapped on three streams, ' + e2e_how},
            'gpu_launches': args.steps,
            'clocks': clocks,
            'ranks': ranks,
            'parity': parity,
        }
        if world == 1:
            secs, cores = cpu_baseline_linear(wl['x'], wl['w'], wl['b'])
            out['cpu_baseline'] = {'value': wl['flops'] / secs / 1e12, 'unit': 'TFLOP/s', 'cores': cores,
                                   'kind': 'port', 'sample': 'whole workload, best of 3: F.linear(x, W*mask, b) fp32'}
            if not args.no_extras:
                only = set(args.extras.split(',')) if args.extras else None
                out['extras'] = run_extras(device, peaks, flush, only)
        if c5 is not None:
            out.setdefault('extras', {})['attention_c5_sharded'] = c5
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
