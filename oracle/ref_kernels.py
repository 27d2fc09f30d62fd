"""TEST INFRASTRUCTURE -- the reference's own CUDA kernels as a second oracle and GPU-side baseline.

The reference (microsoft/SparTA) keeps its kernels as jinja2 templates that it renders with the kernel
object's parameter dictionary and compiles at run time through pycuda
(sparta/specializer/kernels/kernel_base.py:179-190, sparta/specializer/kernels/matmul.py:190-193,
sparta/tesa/block_compressed.py:213-219).  pycuda is not available, so this module does the same two
steps with jinja2 and nvcc:

* ``build_ref(reference_root)`` renders the templates *where they lie in a checkout of the reference*
  for a fixed list of configurations (the shapes of the reference's unit tests and of its notebook /
  README workloads), wraps each source in ``extern "C"`` exactly as pycuda's SourceModule does, and
  compiles it to a cubin for sm_100a under ``oracle/_ref/`` (git-ignored; no reference source is copied
  into the repository).  A manifest records entry names and parameters.
* ``ReferenceKernels`` loads those cubins through the CUDA driver API (ctypes on libcuda) and launches
  them on torch tensors with the reference's own grid / block formulas and argument order.

Only ``tests/``, ``bench.py``'s baseline legs and ``__graft_entry__`` may import this module; the product
(``sparta_b200``) never does.
"""
import concurrent.futures
import ctypes
import json
import os
import shutil
import subprocess
import sys
from typing import Any, Dict, List, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, '_ref')
MANIFEST = os.path.join(REF_DIR, 'manifest.json')

MATMUL_TEMPLATES = 'sparta/specializer/kernels/templates'
TESA_TEMPLATE = 'sparta/tesa/templates/block_compressed.cu.j2'


# ------------------------------------------------------------------------------------------------
# configuration list
# ------------------------------------------------------------------------------------------------
def _bcs_flags(mode: str, trans_a: bool, trans_b: bool) -> Tuple[bool, bool]:
    """Index form a stand-alone kernel uses (sparta/specializer/kernels/matmul.py:60-87,111-120)."""
    if mode == 'sdd':
        return (not trans_a, trans_a)
    if mode == 'dsd':
        return (trans_b, not trans_b)
    return (True, False)


def matmul_name(impl: str, mode: str, biased: bool, trans_a: bool, trans_b: bool, compressed: bool,
                tile: Tuple[int, int, int] = (32, 32, 32), thread: Tuple[int, int, int] = (4, 4, 4)) -> str:
    if impl == 'openai':
        tile, thread = (32, 64, 32), (0, 0, 0)
    return (f'matmul_{impl}_{mode}_b{int(biased)}_ta{int(trans_a)}_tb{int(trans_b)}_c{int(compressed)}'
            f'_{tile[0]}x{tile[1]}x{tile[2]}_t{thread[0]}x{thread[1]}x{thread[2]}')


def tesa_name(BH: int, BW: int, bcsr: bool, bcsc: bool) -> str:
    return f'tesa_{BH}x{BW}_r{int(bcsr)}_c{int(bcsc)}'


def softmax_name(direction: str, H: int, W: int, BH: int, BW: int, RT: int, compressed: bool) -> str:
    return f'softmax_{direction}_{H}x{W}_{BH}x{BW}_rt{RT}_c{int(compressed)}'


def variants() -> List[Dict[str, Any]]:
    """Every (template, parameter dict) pair that is rendered.  Matmul kernels take M, K, N at run time,
    so one cubin per layout serves every shape; softmax kernels bake H and W in."""
    out: List[Dict[str, Any]] = []
    for impl in ('sparta', 'openai'):
        for mode in ('sdd', 'dsd', 'dds'):
            for biased in (False, True):
                for ta in (False, True):
                    for tb in (False, True):
                        for comp in (False, True):
                            tiles = [((32, 32, 32), (4, 4, 4))] if impl == 'sparta' else [((32, 64, 32), (0, 0, 0))]
                            # the tile the reference's look-up table assigns to 64 x 64 x 64 blocks is not used:
                            # one tuned point per layout is enough for a baseline
                            for tile, thread in tiles:
                                bcsr, bcsc = _bcs_flags(mode, ta, tb)
                                params = {
                                    'BATCH_SIZE': 1, 'GLOBAL_M_VALUE': 0, 'GLOBAL_K_VALUE': 0, 'GLOBAL_N_VALUE': 0,
                                    'BIASED': biased, 'TRANSPOSE_A': ta, 'TRANSPOSE_B': tb, 'COMPRESSED': comp,
                                    'BCSR': bcsr, 'BCSC': bcsc,
                                    'BLOCK_SIZE_M_VALUE': tile[0], 'BLOCK_SIZE_K_VALUE': tile[1],
                                    'BLOCK_SIZE_N_VALUE': tile[2],
                                    'THREAD_SIZE_M_VALUE': thread[0], 'THREAD_SIZE_K_VALUE': thread[1],
                                    'THREAD_SIZE_N_VALUE': thread[2],
                                }
                                out.append({
                                    'name': matmul_name(impl, mode, biased, ta, tb, comp, tile, thread),
                                    'template': f'{MATMUL_TEMPLATES}/{impl}_sparse_matmul_{mode}.cuh.j2',
                                    'params': params,
                                })
    for BH, BW in ((8, 8), (16, 16), (32, 32), (32, 64), (64, 32), (64, 64)):
        for bcsr, bcsc in ((True, False), (False, True), (True, True)):
            out.append({'name': tesa_name(BH, BW, bcsr, bcsc), 'template': TESA_TEMPLATE,
                        'params': {'BH': BH, 'BW': BW, 'BCSR': bcsr, 'BCSC': bcsc}})
    for H, W, BH, BW, RT in ((128, 256, 32, 32, 4), (256, 256, 16, 16, 4), (1024, 1024, 32, 32, 4),
                             (4096, 4096, 64, 64, 4)):
        for comp in (False, True):
            for direction in ('forward', 'backward'):
                out.append({
                    'name': softmax_name(direction, H, W, BH, BW, RT, comp),
                    'template': f'{MATMUL_TEMPLATES}/sparta_sparse_softmax_{direction}.cuh.j2',
                    'params': {'GLOBAL_H_VALUE': H, 'GLOBAL_W_VALUE': W, 'BLOCK_SIZE_H_VALUE': BH,
                               'BLOCK_SIZE_W_VALUE': BW, 'ROW_TILE_VALUE': RT, 'COMPRESSED': comp,
                               'BATCH_SIZE': 1},
                })
    return out


# ------------------------------------------------------------------------------------------------
# render + compile
# ------------------------------------------------------------------------------------------------
def _entries(code: str) -> List[str]:
    """Names of the ``__global__`` functions, found the way the reference finds its entry point
    (sparta/specializer/kernels/kernel_base.py:183-184)."""
    names, pos = [], 0
    while True:
        pos = code.find('__global__ void', pos)
        if pos < 0:
            return names
        rest = code[pos + 15:]
        names.append(rest[:rest.find('(')].strip())
        pos += 15


def _compile_one(reference_root: str, variant: Dict[str, Any], force: bool) -> Dict[str, Any]:
    import jinja2
    name = variant['name']
    template_path = os.path.join(reference_root, variant['template'])
    src_path = os.path.join(REF_DIR, name + '.cu')
    cubin_path = os.path.join(REF_DIR, name + '.cubin')
    with open(template_path) as f:
        code = jinja2.Template(f.read()).render(variant['params'])
    record = {'name': name, 'cubin': name + '.cubin', 'entries': _entries(code), 'params': variant['params'],
              'template': variant['template']}
    if not force and os.path.exists(cubin_path) and os.path.getmtime(cubin_path) >= os.path.getmtime(template_path):
        return record
    with open(src_path, 'w') as f:
        f.write('extern "C" {\n' + code + '\n}\n')  # what pycuda's SourceModule does unless no_extern_c is set
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    cmd = [nvcc, '-cubin', '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-w', '-o', cubin_path, src_path]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f'nvcc failed on the rendered reference template {variant["template"]} ({name}):\n'
                           + res.stderr[-2000:])
    os.remove(src_path)  # rendered reference source is an intermediate: only the cubin is kept
    return record


def build_ref(reference_root: str, force: bool = False, workers: int = 8) -> str:
    """Render and compile every variant; returns the manifest path."""
    if not os.path.isdir(os.path.join(reference_root, 'sparta')):
        raise FileNotFoundError(f'{reference_root} is not a checkout of the reference')
    os.makedirs(REF_DIR, exist_ok=True)
    todo = variants()
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        records = list(pool.map(lambda v: _compile_one(reference_root, v, force), todo))
    with open(MANIFEST, 'w') as f:
        json.dump({r['name']: r for r in records}, f, indent=1, sort_keys=True)
    return MANIFEST


def available() -> bool:
    return os.path.exists(MANIFEST)


# ------------------------------------------------------------------------------------------------
# driver-API loader
# ------------------------------------------------------------------------------------------------
class _Driver:
    """The four driver calls needed to run a cubin, through ctypes on libcuda."""

    def __init__(self):
        self.lib = ctypes.CDLL('libcuda.so.1')
        self.lib.cuInit(0)
        self.lib.cuModuleLoadData.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
        self.lib.cuModuleGetFunction.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_char_p]
        self.lib.cuLaunchKernel.argtypes = [ctypes.c_void_p] + [ctypes.c_uint] * 6 + [
            ctypes.c_uint, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p)]

    def check(self, code: int, what: str):
        if code != 0:
            raise RuntimeError(f'{what} failed with CUresult {code}')

    def load(self, image: bytes) -> ctypes.c_void_p:
        mod = ctypes.c_void_p()
        self.check(self.lib.cuModuleLoadData(ctypes.byref(mod), image), 'cuModuleLoadData')
        return mod

    def function(self, mod: ctypes.c_void_p, name: str) -> ctypes.c_void_p:
        fn = ctypes.c_void_p()
        self.check(self.lib.cuModuleGetFunction(ctypes.byref(fn), mod, name.encode()), f'cuModuleGetFunction({name})')
        return fn

    def launch(self, fn, grid, block, stream: int, args: List[Any]):
        holders = []
        for a in args:
            if isinstance(a, (ctypes.c_int32, ctypes.c_float, ctypes.c_void_p)):
                holders.append(a)
            elif isinstance(a, float):
                holders.append(ctypes.c_float(a))
            elif isinstance(a, int):
                holders.append(ctypes.c_int32(a))
            else:  # a torch tensor
                holders.append(ctypes.c_void_p(a.data_ptr()))
        ptrs = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
        self.check(self.lib.cuLaunchKernel(fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], 0,
                                           ctypes.c_void_p(stream), ptrs, None), 'cuLaunchKernel')


class ReferenceKernels:
    """Runs the compiled reference kernels on torch CUDA tensors.  Methods mirror the reference's host
    code (cited per method) down to the grid / block formulas, the zero-filled fp32 outputs and the
    host synchronisation of the index build."""

    def __init__(self):
        import torch
        if not available():
            raise RuntimeError('oracle/_ref/manifest.json is missing: run `python -m oracle.ref_kernels <reference>`')
        with open(MANIFEST) as f:
            self.manifest = json.load(f)
        torch.cuda.init()
        torch.zeros(1, device='cuda')  # makes the primary context current on this thread
        self.torch = torch
        self.drv = _Driver()
        self._functions: Dict[Tuple[str, str], ctypes.c_void_p] = {}
        self._modules: Dict[str, ctypes.c_void_p] = {}

    def _fn(self, name: str, entry: Optional[str] = None):
        rec = self.manifest[name]
        entry = entry or rec['entries'][0]
        key = (name, entry)
        if key not in self._functions:
            if name not in self._modules:
                with open(os.path.join(REF_DIR, rec['cubin']), 'rb') as f:
                    self._modules[name] = self.drv.load(f.read())
            self._functions[key] = self.drv.function(self._modules[name], entry)
        return self._functions[key]

    def _stream(self) -> int:
        return self.torch.cuda.current_stream().cuda_stream

    # ---- TeSA (sparta/tesa/block_compressed.py:231-309) ----
    def build_indexes(self, mask, BH: int, BW: int, bcsr: bool, bcsc: bool) -> Dict[str, Any]:
        torch = self.torch
        name = tesa_name(BH, BW, bcsr, bcsc)
        H, W = mask.shape
        R, C = H // BH, W // BW
        extra = torch.zeros((R + C + 3 * R * C,), dtype=torch.int32, device=mask.device)
        row_ptr = torch.zeros((R + 1,), dtype=torch.int32, device=mask.device)
        col_ptr = torch.zeros((C + 1,), dtype=torch.int32, device=mask.device)
        block = ((BH * BW) // min(BW, 16), 1, 1)
        ptrs = ([row_ptr] if bcsr else []) + ([col_ptr] if bcsc else [])
        self.drv.launch(self._fn(name, 'bcs_index_1'), (C, R, 1), block, self._stream(), [mask, *ptrs, extra, H, W])
        if bcsr:
            row_ptr = torch.cumsum(row_ptr, dim=0, dtype=torch.int32)
        if bcsc:
            col_ptr = torch.cumsum(col_ptr, dim=0, dtype=torch.int32)
        nnz = int((row_ptr if bcsr else col_ptr)[-1].item())
        out: Dict[str, Any] = {'nnz': nnz, 'BH': BH, 'BW': BW, 'H': H, 'W': W, 'name': name, 'bcsr': bcsr, 'bcsc': bcsc}
        idx_args = []
        if bcsr:
            out['row_ptr'] = row_ptr
            out['BCSR_idx'] = torch.empty((nnz,), dtype=torch.int32, device=mask.device)
        if bcsc:
            out['col_ptr'] = col_ptr
            out['BCSC_idx'] = torch.empty((nnz,), dtype=torch.int64 if bcsr else torch.int32, device=mask.device)
        idx_args = ([row_ptr] if bcsr else []) + ([col_ptr] if bcsc else []) + \
                   ([out['BCSR_idx']] if bcsr else []) + ([out['BCSC_idx']] if bcsc else [])
        self.drv.launch(self._fn(name, 'bcs_index_2'), (C, R, 1), (1, 1, 1), self._stream(), [*idx_args, extra])
        return out

    def _order_index(self, ix: Dict[str, Any]):
        return ix['BCSR_idx'] if ix['bcsr'] else ix['BCSC_idx']

    def convert(self, dense, ix: Dict[str, Any]):
        """dense [batch, H, W] fp32 -> [batch, nnz * BH * BW] (block_compressed.py:311-333)."""
        torch = self.torch
        batch = dense.shape[0]
        bs = ix['BH'] * ix['BW']
        sparse = torch.empty((batch, ix['nnz'] * bs), dtype=torch.float32, device=dense.device)
        if ix['nnz'] == 0:
            return sparse
        self.drv.launch(self._fn(ix['name'], 'dense_to_bcs_val'), (ix['nnz'], batch, 1), (min(bs // 4, 256), 1, 1),
                        self._stream(), [dense.contiguous(), sparse, self._order_index(ix), ix['nnz'], ix['H'], ix['W']])
        return sparse

    def inverse(self, sparse, ix: Dict[str, Any]):
        """[batch, nnz * BH * BW] -> dense [batch, H, W] (block_compressed.py:335-358)."""
        torch = self.torch
        batch = sparse.shape[0]
        bs = ix['BH'] * ix['BW']
        dense = torch.zeros((batch, ix['H'], ix['W']), dtype=torch.float32, device=sparse.device)
        if ix['nnz'] == 0:
            return dense
        self.drv.launch(self._fn(ix['name'], 'bcs_val_to_dense'), (ix['nnz'], batch, 1), (min(bs // 4, 256), 1, 1),
                        self._stream(), [sparse.contiguous(), dense, self._order_index(ix), ix['nnz'], ix['H'], ix['W']])
        return dense

    # ---- matmul (sparta/specializer/kernels/matmul.py:143-188,272-275,322-323) ----
    def matmul(self, impl: str, mode: str, A, B, bias, ix: Dict[str, Any], M: int, K: int, N: int,
               trans_a: bool, trans_b: bool, compressed: bool, out=None):
        """fp32 tensors with a leading batch dimension; the sparse operand is compressed when
        ``compressed``.  ``ix`` must come from ``build_indexes`` with the block shape and index form of
        this layout.  Returns a zero-initialised fp32 output like the reference; pass ``out`` (zeroed by
        the caller) to time the kernel alone."""
        torch = self.torch
        tile, thread = ((32, 32, 32), (4, 4, 4)) if impl == 'sparta' else ((32, 64, 32), (0, 0, 0))
        name = matmul_name(impl, mode, bias is not None, trans_a, trans_b, compressed, tile, thread)
        BM, BK, BN = tile
        batch = A.shape[0]
        if out is None:
            shape = (batch, ix['nnz'] * BM * BN) if (mode == 'dds' and compressed) else (batch, M, N)
            out = torch.zeros(shape, dtype=torch.float32, device=A.device)
        by_row = _bcs_flags(mode, trans_a, trans_b)[0]
        ptr, idx = (ix['row_ptr'], ix['BCSR_idx']) if by_row else (ix['col_ptr'], ix['BCSC_idx'])
        tesa = [idx, ix['nnz']] if mode == 'dds' else [ptr, idx, ix['nnz']]
        block = (BN // thread[2], BM // thread[0], 1) if impl == 'sparta' else (256, 1, 1)
        grid = (ix['nnz'], batch, 1) if mode == 'dds' else (N // BN, M // BM, batch)
        if grid[0] == 0:
            return out
        args = [A, B] + ([bias] if bias is not None else []) + [out, *tesa, M, K, N]
        self.drv.launch(self._fn(name), grid, block, self._stream(), args)
        return out

    # ---- softmax (sparta/specializer/kernels/softmax.py:64-89,115-141,182-189) ----
    def softmax_forward(self, x, ix: Dict[str, Any], mask_u8, inv_temperature: float, H: int, W: int, RT: int,
                        compressed: bool, out=None):
        torch = self.torch
        name = softmax_name('forward', H, W, ix['BH'], ix['BW'], RT, compressed)
        batch = x.shape[0]
        if out is None:
            out = torch.zeros_like(x, dtype=torch.float32)
        self.drv.launch(self._fn(name), (H // RT, batch, 1), (RT * 32, 1, 1), self._stream(),
                        [x, ix['row_ptr'], ix['BCSR_idx'], mask_u8, float(inv_temperature), out])
        return out

    def softmax_backward(self, grad_y, y, ix: Dict[str, Any], mask_u8, inv_temperature: float, H: int, W: int,
                         RT: int, compressed: bool):
        torch = self.torch
        name = softmax_name('backward', H, W, ix['BH'], ix['BW'], RT, compressed)
        batch = y.shape[0]
        out = torch.zeros_like(y, dtype=torch.float32)
        self.drv.launch(self._fn(name), (H // RT, batch, 1), (RT * 32, 1, 1), self._stream(),
                        [grad_y, ix['row_ptr'], ix['BCSR_idx'], y, mask_u8, float(inv_temperature), out])
        return out


if __name__ == '__main__':
    if len(sys.argv) < 2:
        sys.exit('usage: python -m oracle.ref_kernels <path of a SparTA checkout> [--force]')
    print(build_ref(sys.argv[1], force='--force' in sys.argv[2:]))
