"""Runs the reference packages' own smoke suites with this library's operators in place of theirs.

    python baseline/run_reference_smoke.py [varlen] [absorb]

Needs a B200, the built library and the installed reference (bash baseline/install_ref.sh <reference checkout>).  The suites are the
unmodified files of the installed packages:

  triton_fa_varlen_v2/test_smoke.py       smoke_test(): tiny / cross-block / stage-1 / stage-2 / aligned cases,
                                          no-grad, partial-grad, 4-D layout, head dim 128, five seeds,
                                          bit repeatability, the 2 M-key business batch and its variants
  triton_target_attn_absorb/test_smoke.py the nine fp32 and seven bf16 correctness cases of its __main__ block
                                          (production widths d_q = 968, d_kv = 216, all five gradients)

Only the operator each suite imports is replaced (the name it binds from the package's interface module); its
inputs, its torch oracle, its tolerances and its PASS / FAIL lines are its own.  Exit code 0 = every suite that
ran ended without a FAIL line or an exception.
"""
import contextlib
import io
import os
import runpy
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(HERE, "_ref"))


class _Tee(io.TextIOBase):
    def __init__(self, *sinks):
        self.sinks = sinks

    def write(self, s):
        for k in self.sinks:
            k.write(s)
        return len(s)

    def flush(self):
        for k in self.sinks:
            k.flush()


def run_varlen(vb) -> bool:
    import triton_fa_varlen_v2.test_smoke as T
    T.packed_varlen_attn = vb.packed_varlen_attn
    buf = io.StringIO()
    with contextlib.redirect_stdout(_Tee(sys.stdout, buf)):
        T.smoke_test()
    return "smoke test PASS" in buf.getvalue()


def run_absorb(vb) -> bool:
    import triton_target_attn_absorb.interface as I
    I.packed_target_attn = vb.packed_target_attn
    I.target_attn_inner = vb.target_attn_inner
    I.prepare_target_attn_indices = vb.prepare_target_attn_indices
    sys.modules.pop("triton_target_attn_absorb.test_smoke", None)
    buf = io.StringIO()
    argv = sys.argv
    sys.argv = ["triton_target_attn_absorb.test_smoke"]
    try:
        with contextlib.redirect_stdout(_Tee(sys.stdout, buf)):
            runpy.run_module("triton_target_attn_absorb.test_smoke", run_name="__main__")
    except SystemExit as e:
        if e.code not in (0, None):
            print(f"the suite exited with {e.code}")
            return False
    finally:
        sys.argv = argv
    out = buf.getvalue()
    n_pass, n_fail = out.count("[PASS]"), out.count("[FAIL]")
    print(f"absorb suite: {n_pass} PASS lines, {n_fail} FAIL lines")
    return n_pass > 0 and n_fail == 0


def main() -> int:
    if not os.path.isdir(os.path.join(HERE, "_ref", "triton_fa_varlen_v2")):
        print("baseline/_ref is absent: bash baseline/install_ref.sh <reference checkout>")
        return 2
    import varlenabsorbflashattn_b200 as vb
    which = [a for a in sys.argv[1:] if a in ("varlen", "absorb")] or ["varlen", "absorb"]
    ok = True
    for w in which:
        print(f"===== {w}: the reference's own smoke suite on this library =====", flush=True)
        good = run_varlen(vb) if w == "varlen" else run_absorb(vb)
        print(f"===== {w}: {'PASS' if good else 'FAIL'} =====", flush=True)
        ok = ok and good
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
