"""Run one of the reference's own gate scripts, unmodified, on the CUDA kernels of this package.

    python tests/run_reference_gate.py test_kernel.py          # one gate
    python tests/run_reference_gate.py all                     # the four, as VERIFY_KERNELS=1 does

The scripts (copied to oracle/_ref by oracle/make_ref.py) import the kernel-path callables by
name from nsa_selection_kernel / nsa_selection_backward / nsa_fused_kernel; the drop-in rebinds
those names before the script's own imports run, so the script compares this package's kernels
with the reference's pure-torch functions and exits 0 / 1 exactly as it does for the Triton
kernels (train.py:184-197).  Test infrastructure: nothing in the product imports this.
"""
import importlib
import os
import runpy
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import make_ref  # noqa: E402


def run(script):
    ref_dir = make_ref.import_path()
    done = importlib.import_module("openbox-llm_b200.dropin").install(allow_synthetic=False)
    assert set(done.values()) == {"patched"}, done
    path = os.path.join(ref_dir, script)
    sys.argv = [path]
    runpy.run_path(path, run_name="__main__")     # the script ends with sys.exit(0 / 1)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what == "all":
        for g in make_ref.GATES:
            print(f"\n----- {g} -----", flush=True)
            r = subprocess.run([sys.executable, os.path.abspath(__file__), g])
            if r.returncode != 0:
                print(f"GATE FAILED: {g} (exit {r.returncode})")
                sys.exit(r.returncode)
        print("\n=== ALL KERNEL GATES GREEN on this GPU ===")
        sys.exit(0)
    run(what)
