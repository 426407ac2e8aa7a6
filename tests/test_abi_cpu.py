"""Host-side checks of the C ABI that need no GPU: every declared symbol is exported, the message and
status constants agree between the C headers and the Python mirror, messages are validated with the
reference's status codes before any CUDA call, and the nnz-balanced row sharding."""
import ctypes
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import fusedmm_b200
from fusedmm_b200 import api, messages as M

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from fusedmm_b200.build import build
    build()
    return api.lib()


def declared_symbols():
    text = (ROOT / "include" / "fusedmm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(fusedmm_b200_\w+)\s*\(", text))
    names |= set(re.findall(r"FUSEDMM_B200_DECL_(?:CSR|CSR_UDEF|G|G_UDEF)\((\w+),", text))
    names |= set(re.findall(r"\bint\s+([sd]fusedMM_csr_\w+)\s*\(", text))
    names.discard("NAME")
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 31 and "fusedMM_csr" in names and "sfusedMM_csr_p64i32" in names and "dgfusedMM_csr_i32_udef" in names
    for name in names:
        assert hasattr(lib, name), name


def test_headers_compile_as_c_and_cxx_and_agree_with_python(tmp_path):
    src = tmp_path / "t.c"
    names = [n for n in dir(M) if n.isupper() and n.split("_")[0] in ("VOP", "ROP", "SOP", "VSC", "AOP")
             and n not in ("SOP_IDENTITY", "SOP_SIGMOID", "SOP_SIGMOID_TABLE_C", "SOP_FR", "SOP_TDIST",
                           "SOP_TDIST_CLAMPED", "SOP_LL", "SOP_FA", "SOP_AFFINE_RECIP")]
    body = "".join(f'  printf("{n} %d\\n", (int){n});\n' for n in names)
    src.write_text('#include <stdio.h>\n#include <stdint.h>\n#define VALUETYPE double\n#define INDEXTYPE int32_t\n'
                   '#include "fusedMM.h"\nint SOP_UDEF_FUNC(double v, double *o) { *o = v; return 0; }\n'
                   'int main(void) {\n' + body +
                   '  int32_t m = 0; SET_VOP_FLAG(m, VOP_SUBR); SET_ROP_FLAG(m, ROP_NORMR); SET_SOP_FLAG(m, SOP_UDEF);\n'
                   '  SET_VSC_FLAG(m, VSC_MUL); SET_AOP_FLAG(m, AOP_ADD); printf("MSG %d\\n", (int)m);\n'
                   '  printf("GET %d %d\\n", (int)GET_ROP_FLAG(m), (int)GET_AOP_FLAG(m));\n'
                   '  /* an invalid message must come back with the reference status, no GPU involved */\n'
                   '  printf("ST %d\\n", fusedMM_csr(0x11F18, 0, 0, 0, 0.0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0.0, 0, 0));\n'
                   '  return 0; }\n')
    exe = tmp_path / "t"
    libdir = api.LIB_PATH.parent
    for cc in ("gcc", "g++"):
        subprocess.run([cc, "-x", "c" if cc == "gcc" else "c++", str(src), f"-I{ROOT / 'include'}",
                        f"-L{libdir}", "-lfusedmm_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)], check=True)
        out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
        got = dict(line.split(" ", 1) for line in out if line)
        for n in names:
            assert int(got[n]) == getattr(M, n), n
        assert int(got["MSG"]) == M.MSG_TDIST == 0x11F55
        assert got["GET"] == f"{M.ROP_NORMR} {M.AOP_ADD}"
        assert int(got["ST"]) == M.ERR_VOP


def test_kernels_header_compiles_as_c_and_cxx_for_both_index_types(tmp_path):
    """include/kernels.h maps the reference's {s,d}gfusedMM_csr and trusted_ names (kernels/include/kernels.h:17-43)
    onto the typed symbols from the caller's INDEXTYPE; with and without VALUETYPE / fusedMM.h in the same program.
    An unknown kernel letter prints the reference's message and touches no GPU."""
    libdir = api.LIB_PATH.parent
    for it in ("int32_t", "int64_t"):
        for with_fusedmm in (False, True):
            src = tmp_path / "k.c"
            src.write_text('#include <stdio.h>\n#include <stdint.h>\n#define INDEXTYPE ' + it + '\n' +
                           ('#define VALUETYPE float\n#include "fusedMM.h"\n' if with_fusedmm else '') +
                           '#include "kernels.h"\n' +
                           ('int SOP_UDEF_FUNC(float v, float *o) { *o = v; return 0; }\n' if with_fusedmm else '') +
                           'int main(void) {\n'
                           '  sgfusedMM_csr(\'x\', 0, 0, 0, 0.0f, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0.0f, 0, 0);\n'
                           '  dgfusedMM_csr(\'x\', 0, 0, 0, 0.0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0.0, 0, 0);\n'
                           '  trusted_sgfusedMM_csr(\'x\', 0, 0, 0, 0.0f, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0.0f, 0, 0);\n'
                           '  trusted_dgfusedMM_csr(\'g\', 0, 0, 0, 0.0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0.0, 0, 0);\n'
                           '  puts("done"); return 0; }\n')
            for cc in ("gcc", "g++"):
                exe = tmp_path / "k"
                subprocess.run([cc, "-Wall", "-Werror", "-x", "c" if cc == "gcc" else "c++", str(src), f"-I{ROOT / 'include'}",
                                f"-L{libdir}", "-lfusedmm_b200", f"-Wl,-rpath,{libdir}", "-o", str(exe)], check=True)
                run = subprocess.run([str(exe)], check=True, capture_output=True, text=True)
                assert "done" in run.stdout and run.stderr.count("Kernel not implemented yet!!!") == 3


def test_kernels_for_other_messages_can_be_built_ahead_of_time_without_a_gpu(lib, tmp_path, monkeypatch):
    """fusedmm_b200_jit_prepare compiles the kernel specialised for a message with NVRTC and files the cubin; a
    second request is answered from the process, a new process from the file."""
    monkeypatch.setenv("FUSEDMM_B200_JIT_CACHE", str(tmp_path))
    msg = M.VOP_MIN | M.ROP_ADD_RHS | M.SOP_COPY | M.VSC_ADD | M.AOP_MIN
    before = api.jit_stats()
    assert api.jit_prepare(msg, 96, np.float32) == 0
    assert api.jit_prepare(msg, 96, np.float32) == 0
    assert api.jit_prepare(msg, 24, np.float64) == 0
    after = api.jit_stats()
    assert after["nvrtc_found"] == 1 and after["compiled"] - before["compiled"] == 2 and after["failures"] == before["failures"]
    files = sorted(tmp_path.glob("sm100a_*.cubin"))
    assert len(files) == 2 and all(f.stat().st_size > 10_000 for f in files)
    assert b"fused_vec_kernel" in files[0].read_bytes()[:400]    # first line: the kernel's mangled name
    # nothing to build: a built-in pattern, K not a multiple of 16 bytes; an invalid message keeps its status
    assert api.jit_prepare(M.MSG_TDIST, 128) == 0 and api.jit_prepare(msg, 7) == 0
    assert api.jit_prepare(0x11F18, 128) == M.ERR_VOP
    assert api.jit_stats()["compiled"] == after["compiled"]
    code = ("import sys; sys.path.insert(0, %r); import numpy as np; from fusedmm_b200 import api; "
            "assert api.jit_prepare(%d, 96, np.float32) == 0; s = api.jit_stats(); "
            "assert s['disk_hits'] == 1 and s['compiled'] == 0, s" % (str(ROOT), msg))
    subprocess.run([sys.executable, "-c", code], check=True)


def test_named_messages():
    assert (M.MSG_SIGMOID, M.MSG_TDIST, M.MSG_SPMM, M.MSG_GCN) == (0x11F12, 0x11F55, 0x11102, 0x10002)


def _call(msg, sop=None):
    a = np.zeros(4, np.float32)
    i = np.zeros(4, np.int32)
    return api.fusedMM_csr(msg, 0, 0, 0, 1.0, 0, 0, 0, a, i, i, i, a, 4, a, 4, 0.0, a, 4, sop=sop)


def test_status_codes_of_invalid_messages(lib):
    # order and values of fusedMM.c:610-628; VOP_NOOP is rejected (fusedMM.c:346-350)
    assert _call(0x11F10) == M.ERR_VOP
    assert _call(0x11F18) == M.ERR_VOP
    assert _call(0x11F62) == M.ERR_ROP
    assert _call(0x11212) == M.ERR_SOP
    assert _call(0x13F12) == M.ERR_VSC
    assert _call(0x41F12) == M.ERR_AOP
    assert _call(0x41F68) == M.ERR_VOP  # first failing stage wins
    # user-defined stages other than SOP: the default stubs' status (fusedMM_internal.h:50-84)
    for msg in (0x11F1F, 0x11FF2, 0x1FF12, 0xF1F12):
        assert _call(msg) == M.ERR_UDEF
    assert _call(M.MSG_SIGMOID, sop=99) == M.ERR_UDEF
    assert _call(M.MSG_SIGMOID) == M.OK  # m == 0: nothing to do


def test_options_and_sop_registry(lib):
    assert api.get_option("hub_chunk") == 256
    assert api.set_option("hub_chunk", 64) == 0 and api.get_option("hub_chunk") == 64
    assert api.set_option("hub_chunk", 256) == 0
    assert api.set_option("hub_chunk", 3) == M.ERR_ARG
    assert api.set_option("no_such_option", 1) == M.ERR_ARG
    assert api.set_option("accept_vop_noop", 1) == 0
    assert _call(0x11F10) == M.OK
    assert api.set_option("accept_vop_noop", 0) == 0
    assert api.set_sop(M.SOP_FR) == 0
    spec = api.SopSpec()
    lib.fusedmm_b200_get_sop(ctypes.byref(spec))
    assert spec.kind == M.SOP_FR
    assert api.set_sop(42) == M.ERR_ARG
    assert api.set_sop(M.SOP_SIGMOID) == 0
    assert b"VOP" in lib.fusedmm_b200_status_string(2)


@pytest.mark.parametrize("dt", [np.int32, np.int64])
def test_shard_rows_balances_edges(lib, dt):
    rng = np.random.default_rng(0)
    deg = rng.poisson(6, size=5000)
    deg[100] = 4000  # a hub row is never split between shards
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(dt)
    for g in (1, 2, 3, 8):
        b = api.shard_rows(rowptr[:-1], rowptr[1:], g)
        assert b[0] == 0 and b[-1] == 5000 and (np.diff(b) >= 0).all()
        per = [int(rowptr[b[i + 1]] - rowptr[b[i]]) for i in range(g)]
        assert sum(per) == int(rowptr[-1])
        assert max(per) <= rowptr[-1] / g + 4000 + 1
    b = api.shard_rows(np.zeros(0, dt), np.zeros(0, dt), 4)
    assert (b == 0).all()
    b = api.shard_rows(np.zeros(10, dt), np.zeros(10, dt), 4)  # no edges at all
    assert b[0] == 0 and b[-1] == 10 and (np.diff(b) >= 0).all()


def test_shard_rows_with_a_row_weight_balances_rows_plus_edges(lib):
    rng = np.random.default_rng(1)
    deg = rng.poisson(3, size=6000)
    deg[:50] = 2000  # the heavy rows come first, as in an R-MAT graph
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    plain = api.shard_rows(rowptr[:-1], rowptr[1:], 2)
    assert (plain == api.shard_rows(rowptr[:-1], rowptr[1:], 2, row_weight=0)).all()
    w = 40
    b = api.shard_rows(rowptr[:-1], rowptr[1:], 2, row_weight=w)
    cost = [int(rowptr[b[i + 1]] - rowptr[b[i]]) + w * int(b[i + 1] - b[i]) for i in range(2)]
    assert abs(cost[0] - cost[1]) <= 2000 + w and b[1] > plain[1]  # the first shard takes more of the light rows
    with pytest.raises(api.FusedMMError):
        api.shard_rows(rowptr[:-1], rowptr[1:], 2, row_weight=-1)
    # no edges at all: rows alone are balanced
    b = api.shard_rows(np.zeros(10, np.int32), np.zeros(10, np.int32), 5, row_weight=1)
    assert list(b) == [0, 2, 4, 6, 8, 10]


def test_every_option_is_documented_in_the_header():
    """Every option name the library accepts (fusedmm_b200_set_option / FUSEDMM_B200_OPTIONS) has its paragraph in
    include/fusedmm_b200.h."""
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    src = (root / "fusedmm_b200" / "csrc" / "fusedmm_capi.cu").read_text()
    hdr = (root / "include" / "fusedmm_b200.h").read_text()
    names = re.findall(r'!strcmp\(name, "([a-z_0-9]+)"\)', src)
    assert len(names) >= 25
    assert [n for n in names if f'"{n}"' not in hdr] == []
