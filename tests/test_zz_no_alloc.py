"""The CSR entry point that brings its own scratch (for callers that may not allocate device
memory) against the workspace-taking one, through the C ABI.  Collected last on purpose."""
import importlib

import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


def _csr(fn_name, idx, block_size, with_workspace):
    L = importlib.import_module("openbox-llm_b200._lib")
    lib = L.lib()
    B, Hkv, T, S = idx.shape
    n_blk = T // block_size
    cap = max(B * Hkv * T * S, 1)
    qob = torch.full((cap,), -7, dtype=torch.int32, device="cuda")
    pbh = torch.full((cap,), -7, dtype=torch.int32, device="cuda")
    off = torch.zeros(B, Hkv, n_blk + 1, dtype=torch.int32, device="cuda")
    if with_workspace:
        nws = lib.nsa_csr_workspace_bytes(B, Hkv, T, S, block_size)
        ws = L.workspace(nws, idx.device)
        rc = lib.nsa_build_block_to_query_csr(L.ptr(idx), B, Hkv, T, S, block_size, L.ptr(qob),
                                              L.ptr(off), L.ptr(pbh), L.ptr(ws), nws, L.stream())
    else:
        rc = lib.nsa_build_block_to_query_csr_noalloc(L.ptr(idx), B, Hkv, T, S, block_size,
                                                      L.ptr(qob), L.ptr(off), L.ptr(pbh), L.stream())
    torch.cuda.synchronize()
    return rc, qob, off, pbh


def test_noalloc_csr_matches_workspace_csr_twice_in_a_row():
    """Two calls in a row on different block lists: the second must not see the first one's
    bitmap (the shared scratch is cleared per call).  Integer output: bit-exact."""
    lists = [O.make_block_idx(2, 2, 512, 32, 6, seed=11).cuda(),
             O.make_block_idx_recent(2, 2, 512, 32, 6).cuda()]
    for idx in lists:
        rc_a, qob_a, off_a, pbh_a = _csr("noalloc", idx, 32, with_workspace=False)
        rc_b, qob_b, off_b, pbh_b = _csr("workspace", idx, 32, with_workspace=True)
        assert rc_a == 0 and rc_b == 0
        P = int(off_b.view(-1)[-1])
        assert P > 0
        assert torch.equal(off_a, off_b)
        assert torch.equal(qob_a[:P], qob_b[:P])
        assert torch.equal(pbh_a[:P], pbh_b[:P])
        r_qob, r_off, r_pbh = O.build_block_to_query_csr(idx.cpu(), 32)
        assert (qob_a[:P].cpu().numpy() == r_qob).all() and (off_a.cpu().numpy() == r_off).all()
        assert (pbh_a[:P].cpu().numpy() == r_pbh).all()


def test_noalloc_csr_refuses_shapes_beyond_its_scratch():
    L = importlib.import_module("openbox-llm_b200._lib")
    lib = L.lib()
    B, Hkv, T, S, bs = 8, 2, 32768, 16, 64
    assert lib.nsa_csr_workspace_bytes(B, Hkv, T, S, bs) > lib.nsa_csr_builtin_scratch_bytes()
    rc = lib.nsa_build_block_to_query_csr_noalloc(None, B, Hkv, T, S, bs, None, None, None, None)
    assert rc == -4
    assert b"built-in scratch" in lib.nsa_last_error()
