"""CPU-side checks of the boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "fss_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fss_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fast_sequential_scan_b200 import _lib
    L = _lib.lib()
    names = declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(L, name), f"{name} declared in include/fss_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    assert L.fss_abi_version() == 1


def test_struct_layouts_match_the_header():
    from fast_sequential_scan_b200 import _lib
    assert ctypes.sizeof(_lib.View) == 24
    assert ctypes.sizeof(_lib.ScanCtx) == 48
    assert ctypes.sizeof(_lib.ForwardState) == 40 and ctypes.sizeof(_lib.BackwardState) == 40


def test_carry_source_and_flag_constants_match_the_header():
    """Field order of fss_carry_source and the values of the FSS_FLAG_* / FSS_ALGO_* constants, read from the header text."""
    from fast_sequential_scan_b200 import _lib
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    body = re.search(r"typedef struct fss_carry_source \{(.*?)\} fss_carry_source;", text, flags=re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if decl:
            fields += [re.sub(r"[^A-Za-z0-9_]", "", part.split()[-1]) for part in decl.split(",")]
    assert fields == [name for name, _ in _lib.CarrySource._fields_]
    assert ctypes.sizeof(_lib.CarrySource) == 72
    defines = dict(re.findall(r"#define (FSS_(?:FLAG|ALGO)_[A-Z_]+) (0x[0-9a-fA-F]+|\d+)", text))
    assert len(defines) >= 7
    for name, value in defines.items():
        assert getattr(_lib, name[4:]) == int(value, 0), f"{name}: header {value}, ctypes {getattr(_lib, name[4:])}"


def test_error_strings_and_argument_checks_need_no_device():
    from fast_sequential_scan_b200 import _lib
    L = _lib.lib()
    assert L.fss_strerror(0) == b"ok"
    for code in range(-12, 0):
        assert L.fss_strerror(code) != b"unknown error code"
    v = _lib.View(0, 0, 0)
    ctx = _lib.ScanCtx(ctypes.sizeof(_lib.ScanCtx), -1, None, None, 0, None, 0, 0)
    call = lambda c, B, T, D, *views: L.fss_scan_forward_half(ctypes.byref(c), B, T, D, *[ctypes.byref(x) for x in views])
    assert call(ctx, 2, 4, 8, v, v, v) == -1                       # NULL tensor
    assert call(ctx, -1, 4, 8, v, v, v) == -2                      # negative extent
    assert call(ctx, 0, 4, 8, v, v, v) == 0                        # empty problem: nothing to do
    bad = _lib.ScanCtx(8, -1, None, None, 0, None, 0, 0)
    assert call(bad, 2, 4, 8, v, v, v) == -10                      # struct size skew
    ctx.algo = 9
    assert call(ctx, 2, 4, 8, v, v, v) == -7
    ctx.algo = 0
    buf = (ctypes.c_uint16 * 64)()
    p = _lib.View(ctypes.addressof(buf), 32, 4)                    # row stride 4 < D = 8
    assert call(ctx, 2, 4, 8, p, p, p) == -2
    ok = [_lib.View(ctypes.addressof(buf) + 128 * k, 32, 8) for k in range(3)]
    assert call(ctx, 2, 4, 8, *ok) == -4                           # no workspace
    assert call(ctx, 2, 4, 8, ok[0], ok[1], ok[0]) == -12          # h starts where alpha starts
    assert call(ctx, 2, 4, 8, ok[0], ok[1], ok[1]) == -12          # ... or where beta starts
    # the chunked kernels run on a linear grid of (channel blocks x chunks x batch) CTAs; a problem
    # whose grid would not fit 31 bits is refused instead of being launched with a truncated grid
    T, D = 1 << 34, 1 << 14
    huge = [_lib.View(ctypes.addressof(buf) + 128 * k, T * D, D) for k in range(3)]
    ctx.algo = _lib.ALGO_CHUNKED
    assert call(ctx, 64, T, D, *huge) == -2
    ctx.algo = 0
    wide = _lib.View(ctypes.addressof(buf), 1 << 62, 8)            # batch stride whose extent overflows
    assert call(ctx, 16, 4, 8, wide, ok[1], ok[2]) == -2
    assert L.fss_workspace_bytes(8, 2048, 1024, 0) > 256
    assert L.fss_workspace_bytes(0, 0, 0, 0) >= 256
    assert L.fss_block_rows(0, 1, 65536, 4096, 1) >= 1


def test_package_has_no_fallback_when_library_is_missing(monkeypatch, tmp_path):
    from fast_sequential_scan_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("FSS_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.lib()
    monkeypatch.delenv("FSS_B200_LIB")
    monkeypatch.setattr(_lib, "_lib", None)
    _lib.lib()


def test_product_never_imports_the_oracle():
    pkg = ROOT / "fast_sequential_scan_b200"
    for path in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu*")):
        text = path.read_text()
        assert "oracle" not in text.replace("# oracle", ""), f"{path} mentions the oracle"


def test_python_surface_mirrors_the_reference_names():
    import fast_sequential_scan_b200 as pkg
    from fast_sequential_scan_b200 import scan_cuda, sequential_scan_cuda as native
    assert callable(pkg.scan_cu) and callable(pkg.scan_cu_single)
    for name in ("SequentialScan", "SequentialScanSingle", "scan", "scan_single"):
        assert hasattr(scan_cuda, name)
    for name in ("scan_forward", "scan_backward", "scan_forward_half", "scan_backward_half"):
        assert callable(getattr(native, name))


def test_backward_mode_switch_validates_its_argument():
    from fast_sequential_scan_b200 import scan_cuda
    assert scan_cuda.BACKWARD_MODES == ("saved", "inplace", "recompute")
    previous = scan_cuda.set_backward_mode("recompute")
    try:
        assert previous == "saved" and scan_cuda._resolve(None) == "recompute"
        assert scan_cuda._resolve("inplace") == "inplace"
        with pytest.raises(ValueError):
            scan_cuda.set_backward_mode("in-place")
        with pytest.raises(ValueError):
            scan_cuda._resolve("keep")
    finally:
        scan_cuda.set_backward_mode(previous)


def test_reference_arm_of_the_bench_prints_the_contract_line():
    """`bench.py --impl reference` runs on host cores only; one JSON line with the agreed keys."""
    import json
    import subprocess
    import sys
    root = Path(__file__).resolve().parent.parent
    out = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["higher_is_better"] is True and line["value"] > 0
    for key in ("metric", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "config", "cpu_baseline", "e2e"):
        assert key in line
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
