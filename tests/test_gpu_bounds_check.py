"""-m gpu: the ragged and odd-shaped cases once more through the CHECKED build of the library
(``libw4a16_b200_checked.so``: the streaming kernel compiled with ``-DW4A16_BOUNDS_CHECK``, every shared- and
global-memory index compared with the extent it must stay inside, violations counted in a device word and the access
skipped).  compute-sanitizer is not available on this pool; this is the stand-in.  The checked library is loaded in a
child interpreter so that the ordinary one stays the library every other test runs."""
from __future__ import annotations

import pathlib
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parent.parent

CHILD = r"""
import ctypes, os, sys
os.environ["W4A16_CHECKED_LIB"] = "1"
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import torch
from nibble_b200 import _native
from nibble_b200.quantization import pack_int4, quantize_groupwise
from capi_helpers import capi_linear, check_against_oracle, new_workspace

lib = _native.core()
assert "checked" in lib._name
site, count = ctypes.c_uint32(9), ctypes.c_uint32(9)
assert lib.w4a16_bounds_check_status(ctypes.byref(site), ctypes.byref(count)) == 0 and count.value == 0

def case(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    codes, scales = quantize_groupwise((torch.randn((n, k), generator=g)).half(), 128)
    return torch.randn((m, k), generator=g).half().cuda(), pack_int4(codes).cuda(), scales.cuda()

launches = 0
for m in (1, 2, 3, 8, 9, 16, 17, 33, 64):
    for k, n in ((128, 1), (256, 7), (384, 13), (5632, 33), (1024, 17), (2048, 250), (2048, 2048)):
        x, packed, scales = case(m, k, n, k + n + m)
        ws = new_workspace(m, n, k)
        check_against_oracle(capi_linear(x, packed, scales, workspace=ws), x, packed, scales)
        launches += 1
        for config in ((1, 8, 2, 2, 0), (1, 1, 1, 1, 3), (2, 2, 1, 2, 4), (1, 4, 4, 2, 3)):
            if m > 16 and config[0] == 2:
                continue
            y = torch.empty((m, n), dtype=torch.float16, device="cuda")
            cfg = _native.LinearConfig(*config)
            status = lib.w4a16_linear_f16_config(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), y.data_ptr(), m, n, k, 128,
                                                 ws.data_ptr(), ws.numel(), 0, ctypes.byref(cfg),
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            if status == 0:
                check_against_oracle(y, x, packed, scales)
                launches += 1
torch.cuda.synchronize()
assert lib.w4a16_bounds_check_status(ctypes.byref(site), ctypes.byref(count)) == 0
print("launches", launches, "violations", count.value, "site", site.value)
assert count.value == 0, (site.value, count.value)
"""


def test_ragged_cases_through_the_bounds_checking_build():
    from nibble_b200 import _native

    if not _native.CHECKED_LIB.exists():
        pytest.skip("the checked library is not built (python nibble_b200/_build.py --bounds-check)")
    proc = subprocess.run([sys.executable, "-c", CHILD, str(ROOT)], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    assert "violations 0" in proc.stdout


def test_the_ordinary_build_has_no_checks():
    import ctypes

    from nibble_b200 import _native

    site, count = ctypes.c_uint32(0), ctypes.c_uint32(0)
    assert _native.core().w4a16_bounds_check_status(ctypes.byref(site), ctypes.byref(count)) == -6
