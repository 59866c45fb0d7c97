"""Bring the reference's own pure-Python modules next to the oracle (test infrastructure).

The reference is plain Python, so there is nothing to compile: "building" it means placing an
unmodified copy of the modules of the attention path, and of the four gate scripts that define
its parity, into oracle/_ref/ (ignored by git, so no reference source enters the history; the
folder still travels to the GPU machine with the working tree).  What it is used for:

  * tests: the drop-in rebinding is exercised on the real modules, the unmodified
    NSATransformer(attn_impl="fused") runs on the CUDA kernels, and the four gate scripts
    (test_kernel.py, test_kernel_backward.py, test_kernel_fused.py, test_integration.py; the
    set train.py:184-197 runs under VERIFY_KERNELS=1) run as they are through the shim;
  * bench.py: the CPU arm times the reference's own functions (kind "reference").

The checkout is looked for in $OPENBOX_LLM_REFERENCE, then in a `reference` folder beside the
repository.  Nothing outside oracle/_ref/ is written, and the product package never imports it.

    python oracle/make_ref.py            # copy if a checkout is reachable, else say so
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

MODULES = ["nsa_model.py", "nsa_selection_kernel.py", "nsa_selection_backward.py",
           "nsa_fused_kernel.py", "nsa_fsa.py"]
GATES = ["test_kernel.py", "test_kernel_backward.py", "test_kernel_fused.py", "test_integration.py"]


def find_checkout():
    cands = [os.environ.get("OPENBOX_LLM_REFERENCE"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and all(os.path.isfile(os.path.join(c, m)) for m in MODULES):
            return c
    return None


def available():
    """True when oracle/_ref holds every module of the attention path."""
    return all(os.path.isfile(os.path.join(REF_DIR, m)) for m in MODULES)


def make_ref(verbose=False):
    """Copy the modules and gate scripts when a checkout is reachable.  Returns the folder, or
    None when there is neither a checkout nor an earlier copy."""
    src = find_checkout()
    if src is None:
        return REF_DIR if available() else None
    os.makedirs(REF_DIR, exist_ok=True)
    for name in MODULES + GATES:
        s = os.path.join(src, name)
        if os.path.isfile(s):
            shutil.copyfile(s, os.path.join(REF_DIR, name))
            if verbose:
                print("copied", name)
    return REF_DIR


def import_path():
    """Put oracle/_ref on sys.path (once) so that `import nsa_model` finds the reference."""
    if not available():
        raise ImportError("oracle/_ref is empty: run `python oracle/make_ref.py` where a reference "
                          "checkout is reachable")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return REF_DIR


if __name__ == "__main__":
    out = make_ref(verbose=True)
    print(out if out else "no reference checkout reachable; oracle/_ref left as it is")
