"""Generates tests/golden/reference_general_kernel.npz by RUNNING THE REFERENCE.

Needs oracle/_ref (built by oracle/build_ref.sh from the HipGraph/FusedMM sources).  Every case is a small
seeded input; the stored output is what the reference's own fusedMM_csr (general kernel,
fusedMM.c:487-744) wrote into a zero-initialised Z.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from cases import MESSAGES, dense, random_csr  # noqa: E402
from fusedmm_b200 import messages as M  # noqa: E402
from oracle.cpu import Reference  # noqa: E402

SOP_FOR = {"sigmoid": M.SOP_SIGMOID, "tdist": M.SOP_TDIST_CLAMPED, "subl_norml_udef_mul_max": M.SOP_TDIST,
           "copyrhs_dot_udef_mul_add_fr": M.SOP_SIGMOID_TABLE_C}


def main():
    ref = Reference()
    ref.threads(1)
    out = {}
    case = 0
    for name, msg in MESSAGES.items():
        for vt in (np.float32, np.float64):
            for it in (np.int32, np.int64):
                rng = np.random.default_rng(1000 + case)
                m, n, k = 37, 29, (24 if case % 2 == 0 else 13)
                ld = k + (case % 3)
                pntrb, pntre, indx, val = random_csr(rng, m, n, 5, it, it, hub=70, gaps=(case % 2 == 1))
                val = val.astype(vt)
                generic = msg not in (M.MSG_SIGMOID, M.MSG_TDIST, M.MSG_SPMM, M.MSG_GCN)
                lo, hi = (0.1, 1.0) if generic else (-0.5, 0.5)  # no cancelling reductions feeding a product
                x = dense(rng, m, k, ld, vt, lo, hi)
                y = dense(rng, n, k, ld, vt, lo, hi)
                z = np.zeros((m, ld), dtype=vt)
                sop = SOP_FOR.get(name, M.SOP_IDENTITY)
                st = ref.csr(msg, m, n, k, val, indx, pntrb, pntre, np.nan_to_num(x), ld, np.nan_to_num(y), ld,
                             0.0, z, ld, sop_kind=sop)
                assert st == 0, (name, st)
                key = f"{case:03d}"
                out[key + "_meta"] = np.array([msg, m, n, k, ld, sop], dtype=np.int64)
                out[key + "_name"] = np.array(name)
                for nm, arr in (("pntrb", pntrb), ("pntre", pntre), ("indx", indx), ("val", val),
                                ("x", np.nan_to_num(x)), ("y", np.nan_to_num(y)), ("z", z)):
                    out[f"{key}_{nm}"] = arr
                case += 1
    np.savez_compressed(Path(__file__).with_name("reference_general_kernel.npz"), **out)
    print(f"wrote {case} cases")


if __name__ == "__main__":
    main()
