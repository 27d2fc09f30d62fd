"""Generate the golden vectors of ``tests/golden`` from the reference's own CPU-capable code.

Run once in a container that holds the reference checkout (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/SparTA

``import sparta`` fails without pycuda and the compiled extensions, so the three modules that only
need torch / numpy are loaded by file path: ``sparta/testing/math.py``, ``sparta/testing/mask.py``
and, from ``test/unit/test_tesa.py``, the ``reduce_mask_ref`` helper (extracted with ``ast`` because
the test module itself imports ``sparta``).  ``SparseMatMulKernel.reference`` -- the dense computation
the reference's matmul kernels are checked against (sparta/specializer/kernels/matmul.py:211-227) -- is
extracted from its class the same way and run on a stand-in for ``self``.  Outputs are small ``.npz``
files.  ``--only NAME`` regenerates one file (masks, tesa, softmax_attention, matmul).
"""
import ast
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_function(path, func_name):
    tree = ast.parse(open(path).read())
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == func_name)
    ns = {'torch': torch}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, 'exec'), ns)
    return ns[func_name]


def load_method(path, class_name, method_name):
    """A method of a class, compiled on its own (the class body needs modules that do not import here)."""
    tree = ast.parse(open(path).read())
    cls = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == class_name)
    node = next(n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == method_name)
    ns = {'torch': torch}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, 'exec'), ns)
    return ns[method_name]


def matmul_vectors(ref_root, mask_ref, reduce_mask_ref):
    """Inputs and outputs of SparseMatMulKernel.reference for every mode / transposition / bias, before
    ``compile`` (``ready`` false: dds output times the element mask) and after (``ready`` true: dds output
    times the block coverage, which the reference takes from ``indexes.get_mask()`` = the block mask of
    ``reduce_mask_ref`` repeated over the block, sparta/tesa/block_compressed.py:47-50)."""
    from types import SimpleNamespace as NS
    reference = load_method(os.path.join(ref_root, 'sparta/specializer/kernels/matmul.py'),
                            'SparseMatMulKernel', 'reference')
    batch, M, K, N, BM, BN = 2, 16, 24, 32, 8, 16
    out = {'shape': np.array([batch, M, K, N, BM, BN])}
    torch.manual_seed(2024)
    for mode in ('sdd', 'dsd', 'dds'):
        for tA in (False, True):
            for tB in (False, True):
                shapes = {'A': (K, M) if tA else (M, K), 'B': (N, K) if tB else (K, N), 'C': (M, N)}
                port = {'sdd': 'A', 'dsd': 'B', 'dds': 'C'}[mode]
                A = torch.rand((batch,) + shapes['A'])
                B = torch.rand((batch,) + shapes['B'])
                bias = torch.rand((batch, N))
                mask = mask_ref.block_mask(shapes[port], block=(4, 4), sparsity=0.7, device='cpu')
                cover = None
                if mode == 'dds':
                    cover = reduce_mask_ref(mask, BM, BN).to(torch.uint8)
                    cover = cover.repeat_interleave(BM, 0).repeat_interleave(BN, 1)
                key = f'{mode}_{int(tA)}{int(tB)}'
                out[f'{key}_A'], out[f'{key}_B'] = A.numpy(), B.numpy()
                out[f'{key}_bias'], out[f'{key}_mask'] = bias.numpy(), mask.numpy()
                for biased in (False, True):
                    for ready in (False, True):
                        me = NS(_mode=mode, _transpose_A=tA, _transpose_B=tB, _biased=biased, ready=ready,
                                ports={port: NS(mask=mask, indexes=NS(get_mask=lambda c=cover: c))})
                        args = (A, B, bias) if biased else (A, B)
                        out[f'{key}_C_b{int(biased)}_r{int(ready)}'] = reference(me, *args).numpy()
    np.savez_compressed(os.path.join(HERE, 'matmul.npz'), **out)


def main(ref_root, only=None):
    math_ref = load_by_path('ref_math', os.path.join(ref_root, 'sparta/testing/math.py'))
    mask_ref = load_by_path('ref_mask', os.path.join(ref_root, 'sparta/testing/mask.py'))
    reduce_mask_ref = load_function(os.path.join(ref_root, 'test/unit/test_tesa.py'), 'reduce_mask_ref')

    if only in (None, 'matmul'):
        matmul_vectors(ref_root, mask_ref, reduce_mask_ref)
    if only == 'matmul':
        return
    assert only is None, 'partial regeneration is offered for matmul.npz only (the others share one RNG stream each)'

    # ---- masks: the reference generator on the CPU, seeded through the global RNG ----
    out = {}
    for i, (shape, block, sparsity, seed) in enumerate([
        ((256, 192), (1, 1), 0.99, 2023),
        ((128, 256), (8, 8), 0.9, 2022),
        ((64, 64), (32, 32), 0.5, 7),
    ]):
        torch.manual_seed(seed)
        m = mask_ref.block_mask(shape, block=block, sparsity=sparsity, device='cpu')
        out[f'mask{i}'] = m.numpy()
        out[f'mask{i}_args'] = np.array([*shape, *block, int(sparsity * 10000), seed])
    np.savez_compressed(os.path.join(HERE, 'masks.npz'), **out)

    # ---- block occupancy (reduce_mask_ref) for the test_tesa.py block-size grid ----
    torch.manual_seed(2023)
    mask = mask_ref.block_mask((256, 384), sparsity=0.995, device='cpu')
    out = {'mask': mask.numpy()}
    for BH in [4, 8, 16, 32, 64, 128]:
        for BW in [4, 8, 16, 32, 64, 128]:
            out[f'occ_{BH}_{BW}'] = reduce_mask_ref(mask, BH, BW).numpy()
    np.savez_compressed(os.path.join(HERE, 'tesa.npz'), **out)

    # ---- softmax forward / backward and attention ----
    torch.manual_seed(2022)
    H, W = 64, 128
    x = torch.rand((2, H, W))
    grad = torch.rand((2, H, W))
    mask = mask_ref.block_mask((H, W), block=(8, 8), sparsity=0.9, device='cpu')
    mask[5 * 8:6 * 8] = 0  # make some rows fully masked
    T = float(np.sqrt(W))
    y = math_ref.sparse_softmax_forward_reference(x, mask, T)
    dx = math_ref.sparse_softmax_backward_reference(grad, y, mask, T)
    q = torch.rand((2, 64, 32))
    k = torch.rand((2, 96, 32))
    v = torch.rand((2, 96, 32))
    amask = mask_ref.block_mask((64, 96), block=(8, 8), sparsity=0.8, device='cpu')
    o = math_ref.sparse_multi_head_attention_reference(q, k, v, amask)
    np.savez_compressed(
        os.path.join(HERE, 'softmax_attention.npz'),
        x=x.numpy(), grad=grad.numpy(), mask=mask.numpy(), T=np.float64(T), y=y.numpy(), dx=dx.numpy(),
        q=q.numpy(), k=k.numpy(), v=v.numpy(), amask=amask.numpy(), o=o.numpy(),
    )
    print('golden vectors written to', HERE)


if __name__ == '__main__':
    if len(sys.argv) not in (2, 4) or (len(sys.argv) == 4 and sys.argv[2] != '--only'):
        sys.exit('usage: python make_golden.py <path of a SparTA checkout> [--only matmul]')
    main(sys.argv[1], sys.argv[3] if len(sys.argv) == 4 else None)
