"""The drop-in rebinding (openbox-llm_b200/dropin.py) and, on a GPU, the reference's own gate
scripts run unmodified through it."""
import os
import subprocess
import sys

import pytest

from oracle import make_ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HAVE_REF = make_ref.available()

_PATCH_CHECK = r"""
import importlib, sys
sys.path.insert(0, {root!r})
if {with_ref}:
    from oracle import make_ref
    make_ref.import_path()
dropin = importlib.import_module("openbox-llm_b200.dropin")
ops = importlib.import_module("openbox-llm_b200.ops")
done = dropin.install()
want = "patched" if {with_ref} else "synthetic"
assert set(done) == {{"nsa_selection_kernel", "nsa_selection_backward", "nsa_fsa", "nsa_fused_kernel"}}, done
assert set(done.values()) == {{want}}, done
import nsa_fused_kernel, nsa_selection_backward, nsa_selection_kernel, nsa_fsa
# the names nsa_model.py:316-317 imports at call time, and the wrappers the gates and benches use
assert nsa_fused_kernel.compression_attn_triton is ops.compression_attn_triton
assert nsa_fused_kernel.window_attn_triton is ops.window_attn_triton
assert nsa_selection_backward.selection_attn_triton is ops.selection_attn_triton
assert nsa_selection_backward.SelectionAttnTriton is ops.SelectionAttnTriton
assert nsa_selection_backward.selection_backward_triton is ops.selection_backward_triton
assert nsa_selection_kernel.selection_forward_triton is ops.selection_forward_triton
assert nsa_fused_kernel.nsa_fused_forward is ops.nsa_fused_forward
assert nsa_fused_kernel._RangeAttn is ops._RangeAttn
assert nsa_fsa.build_block_to_query_csr is ops.build_block_to_query_csr
if {with_ref}:
    # the pure-torch side of the reference stays the reference's own
    assert nsa_selection_kernel.selection_forward_reference.__module__ == "nsa_selection_kernel"
    assert nsa_fused_kernel.nsa_fused_reference.__module__ == "nsa_fused_kernel"
    import nsa_model
    m = nsa_model.NSAAttention(64, 4, 2, block_size=16, n_selected_blocks=2, window=8, attn_impl="fused")
    assert m.attn_impl == "fused"
else:
    assert sys.modules["nsa_fused_kernel"].__doc__.startswith("kernel-path names")
    try:
        dropin.install(allow_synthetic=False)
    except ImportError:
        pass
    else:
        raise AssertionError("allow_synthetic=False must raise without a checkout")
print("ok")
"""


def _run(code):
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    env.pop("PYTHONPATH", None)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd="/")


@pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref is empty (no reference checkout was reachable at build time)")
def test_install_patches_the_reference_modules():
    r = _run(_PATCH_CHECK.format(root=ROOT, with_ref=True))
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


def test_install_registers_synthetic_modules_without_a_checkout():
    r = _run(_PATCH_CHECK.format(root=ROOT, with_ref=False))
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref is empty (no reference checkout was reachable at build time)")
@pytest.mark.parametrize("gate", make_ref.GATES)
def test_reference_gate_script_is_green_through_the_shim(gate):
    """test_kernel.py:25-36,70-76 (forward, 7 configs), test_kernel_backward.py:28,41-74 (dQ/dK/dV,
    fp32 + bf16), test_kernel_fused.py:25-70 (three branches + 8 gradients), test_integration.py:24-88
    (NSATransformer ref vs fused: 8-step loss parity and per-parameter gradient parity): the
    unmodified scripts, their own tolerances, exit code 0."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "run_reference_gate.py"), gate],
                       capture_output=True, text=True, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "GREEN" in r.stdout, tail
