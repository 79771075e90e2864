"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports every
symbol include/dflash_cuda.h declares, validates arguments before touching the device, and
its host-only helpers work."""
import ctypes as C
import os
import re

import pytest

from swiftlm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dflash_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dflash_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 10
    handle = C.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(handle, name), name
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_counters():
    L = _lib.lib()
    assert b"sm_100a" in L.dflash_version()
    assert L.dflash_launch_count() >= 0


def test_argument_validation_needs_no_device():
    L = _lib.lib()
    # null pointers
    assert L.dflash_gated_delta_tape(*([None] * 11), 1, 16, 1, 2, 128, 128, 0, 0, 0, None) == _lib.ERR_INVALID_ARG
    assert b"null" in L.dflash_last_error_string()
    fake = 0x1000  # never dereferenced: validation fails first
    # Dk not a multiple of 32 -> unsupported (the reference falls back to its ops path there)
    st = L.dflash_gated_delta_tape(*([fake] * 6), None, None, fake, fake, None, 1, 16, 1, 2, 48, 128, 0, 0, 0, None)
    assert st == _lib.ERR_UNSUPPORTED
    st = L.dflash_tape_replay(fake, fake, fake, fake, None, None, fake, 1, 16, 3, 4, 128, 128, 0, 0, 0, None)
    assert st == _lib.ERR_UNSUPPORTED and b"Hv" in L.dflash_last_error_string()
    # SDPA eligibility mirrors the reference's nil-return guards
    def sdpa(T=16, D=256, Hq=16, Hkv=2, dtype=_lib.BF16, N=64):
        return L.dflash_verify_sdpa(fake, fake, fake, None, None, None, fake, None, 0, 1, Hq, Hkv, T, D, N,
                                    0, 0, 0, 0.0625, dtype, 0, None)
    assert sdpa(T=8) == _lib.ERR_UNSUPPORTED
    assert sdpa(D=64) == _lib.ERR_UNSUPPORTED
    assert sdpa(Hq=15) == _lib.ERR_UNSUPPORTED
    assert sdpa(dtype=_lib.F32) == _lib.ERR_UNSUPPORTED
    assert sdpa(N=8) == _lib.ERR_UNSUPPORTED
    # misaligned base pointer
    assert L.dflash_verify_sdpa(fake + 2, fake, fake, None, None, None, fake, None, 0, 1, 16, 2, 16, 256, 64,
                                0, 0, 0, 0.0625, _lib.BF16, 0, None) == _lib.ERR_INVALID_ARG


@pytest.mark.parametrize("units,gpus", [(64, 8), (16, 8), (10, 4), (3, 8), (0, 2), (73, 1)])
def test_partition_plan(units, gpus):
    L = _lib.lib()
    arr = (C.c_int32 * (2 * gpus))()
    assert L.dflash_partition_plan(units, gpus, arr) == 0
    spans = [(arr[2 * i], arr[2 * i + 1]) for i in range(gpus)]
    assert spans[0][0] == 0 and spans[-1][1] == units
    sizes = [e - b for b, e in spans]
    assert all(spans[i][1] == spans[i + 1][0] for i in range(gpus - 1))
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert L.dflash_partition_plan(4, 0, arr) == _lib.ERR_INVALID_ARG


def test_verify_step_descriptor_layout_matches_the_header(tmp_path):
    """The ctypes mirror of dflash_verify_step_desc against the C compiler's layout of the header's struct."""
    import ctypes as C
    import subprocess

    from swiftlm_b200 import _lib
    fields = [name for name, _ in _lib.VerifyStepDesc._fields_]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{os.path.join(ROOT, "include", "dflash_cuda.h")}"',
             'int main(void) {', '  printf("%zu\\n", sizeof(dflash_verify_step_desc));']
    lines += [f'  printf("%zu\\n", offsetof(dflash_verify_step_desc, {name}));' for name in fields]
    lines += ['  printf("%zu %zu\\n", sizeof(dflash_turbo_kv), offsetof(dflash_turbo_kv, n_cold));', '  return 0;', '}']
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    assert int(out[0]) == C.sizeof(_lib.VerifyStepDesc)
    for name, line in zip(fields, out[1:]):
        assert int(line) == getattr(_lib.VerifyStepDesc, name).offset, name
    size, off = map(int, out[1 + len(fields)].split())
    assert size == C.sizeof(_lib.TurboKV) and off == _lib.TurboKV.n_cold.offset
