"""The C-ABI library builds, loads and exports exactly what include/hgq_b200.h declares (no GPU needed)."""

import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope='module')
def built_lib():
    from hgq2_b200 import build

    build.build()
    from hgq2_b200 import _lib

    return _lib.lib()


def declared_symbols() -> set[str]:
    text = (ROOT / 'include' / 'hgq_b200.h').read_text()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return set(re.findall(r'\b(hgq_[a-z0-9_]+)\s*\(', text))


def test_header_and_binding_agree(built_lib):
    from hgq2_b200 import _lib

    decl = declared_symbols()
    assert decl, 'no declarations found'
    assert decl == set(_lib.SIGNATURES), (decl ^ set(_lib.SIGNATURES))
    for name in decl:
        assert hasattr(built_lib, name), f'{name} is declared but not exported'


def test_status_strings(built_lib):
    assert built_lib.hgq_status_string(0) == b'ok'
    for code in range(-7, 0):
        assert built_lib.hgq_status_string(code) not in (b'', b'unknown status')
    assert built_lib.hgq_abi_version() >= 1


def test_argument_errors_need_no_gpu(built_lib):
    # argument validation happens before any CUDA call
    L = built_lib
    assert L.hgq_quantize_fwd(None, None, None, None, None, None, 16, 0, 1, 2, 0, None) == -1
    assert L.hgq_quantize_fwd(None, None, None, None, None, None, -1, 0, 1, 2, 0, None) == -2
    assert L.hgq_quantize_fwd(None, None, None, None, None, None, 16, 5, 1, 2, 0, None) == -2
    assert L.hgq_quantize_fwd(None, None, None, None, None, None, 16, 0, 7, 2, 0, None) == -3
    assert L.hgq_quantize_fwd(None, None, None, None, None, None, 0, 0, 1, 2, 0, None) == 0
    assert L.hgq_quantize_bwd_workspace(1 << 20, 1 << 20) == 0
    assert L.hgq_quantize_bwd_workspace(1 << 20, 64) > 0


def test_dense_stack_limits_need_no_gpu(built_lib):
    """hgq_dense_chain_supported / _workspace are host arithmetic: layer count, widths, shared-memory budget."""
    from hgq2_b200._lib import ChainLayer

    def stack(widths):
        arr = (ChainLayer * (len(widths) - 1))()
        for a, k, n in zip(arr, widths[:-1], widths[1:]):
            a.K, a.N = k, n
        return len(arr), arr

    L = built_lib
    assert L.hgq_dense_chain_supported(*stack((16, 64, 32, 32, 5))) == 1
    assert L.hgq_dense_chain_supported(*stack((16, 65))) == 0          # a layer wider than 64
    assert L.hgq_dense_chain_supported(*stack((16, 64, 32, 5)[:1] + (64, 31, 5))) == 1
    assert L.hgq_dense_chain_supported(*stack((8,) * 10)) == 0         # nine layers
    assert L.hgq_dense_chain_supported(*stack((64,) * 9)) == 0         # eight 64 x 64 layers: weights and records exceed shared memory
    n, arr = stack((16, 64, 32, 32, 5))
    assert L.hgq_dense_chain_workspace(16384, n, arr) >= 128 * (16 * 64 + 64 + 16) * 4
    assert L.hgq_dense_chain_workspace(0, n, arr) == 0
    assert L.hgq_dense_chain_fwd(None, 16, n, arr, None) == -1         # null input: refused before any CUDA call
    arr[1].K = 63                                                       # widths that do not chain
    assert L.hgq_dense_chain_supported(n, arr) == 0


def test_product_path_has_no_cpu_fallback():
    import torch

    from hgq2_b200 import kernels

    x = torch.zeros(8)
    with pytest.raises(RuntimeError, match='CUDA tensors only'):
        kernels.quantize_fwd(x, torch.zeros(8, dtype=torch.uint8), x, x, 'RND', 'SAT')


def test_package_never_imports_the_oracle():
    for path in (ROOT / 'hgq2_b200').rglob('*.py'):
        text = path.read_text()
        assert not re.search(r'^\s*(from|import)\s+oracle\b', text, flags=re.M), path


def test_descriptor_structs_match_the_header(tmp_path):
    """hgq_slot_desc / hgq_weight_desc / hgq_chain_layer as the C compiler lays them out equal their ctypes mirrors field by field."""
    import ctypes
    import shutil
    import subprocess

    from hgq2_b200._lib import ChainLayer, EbopsDenseDesc, SlotDesc, WeightDesc

    gcc = shutil.which('gcc')
    if gcc is None:
        pytest.skip('no C compiler')
    fields = [('hgq_slot_desc', SlotDesc), ('hgq_weight_desc', WeightDesc), ('hgq_chain_layer', ChainLayer),
              ('hgq_ebops_dense_desc', EbopsDenseDesc)]
    body = ''.join(f'printf("%zu\\n", sizeof({c}));' + ''.join(f'printf("%zu\\n", offsetof({c}, {name}));' for name, _ in s._fields_)
                   for c, s in fields)
    src = tmp_path / 'layout.c'
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "hgq_b200.h"\nint main(void){' + body + 'return 0;}\n')
    exe = tmp_path / 'layout'
    subprocess.run([gcc, '-I', str(ROOT / 'include'), str(src), '-o', str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = []
    for _, s in fields:
        want.append(ctypes.sizeof(s))
        want += [getattr(s, name).offset for name, _ in s._fields_]
    assert got == want
