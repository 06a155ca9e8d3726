"""The C-ABI library loads without a GPU and exports every symbol that include/tdb_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "tdb_b200.h")).read()
    return sorted(set(re.findall(r"TDB_API\s+[\w\s\*]+?\b(tdb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from turbodeberta_b200 import _cabi, build
    build.build()
    names = _declared()
    assert len(names) >= 9
    assert sorted(names) == sorted(_cabi.EXPORTS)
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), n


def test_version_and_error_strings():
    from turbodeberta_b200 import _cabi
    assert _cabi.lib.tdb_version() == 100
    assert b"timed out" in _cabi.lib.tdb_strerror(_cabi.ERR_TIMEOUT)
    assert b"unknown" in _cabi.lib.tdb_strerror(-99)
    assert _cabi.lib.tdb_attn_workspace_bytes(4, 1000) >= 16 + 8 * (8 + 4)


def test_host_side_validation_needs_no_gpu():
    """Bad arguments are rejected before anything touches a device."""
    from turbodeberta_b200 import _cabi
    lib = _cabi.lib
    assert lib.tdb_bucket_table(256, 512, 100, None, None) == _cabi.ERR_ARG
    assert lib.tdb_bucket_table(256, 100, 100, 16, None) == _cabi.ERR_ARG       # max_pos <= buckets/2
    assert lib.tdb_relpos_project(None, None, None, 1, 1, 1, 1, 0, None, None, None) == _cabi.ERR_ARG
    a = 4096  # fake, aligned, never dereferenced: validation fails first
    rc = lib.tdb_attn_fwd_fixed(a, a, a, a, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, None, None, 0, None, 0, None, None, 0, 0,
                                None, 1, 16, 2, 32, 0.1, 0, 0, 0, None, a, None)
    assert rc == _cabi.ERR_SHAPE                                                 # head_dim 32
    rc = lib.tdb_attn_fwd_fixed(a + 2, a, a, a, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, None, None, 0, None, 0, None, None, 0, 0,
                                None, 1, 16, 2, 64, 0.1, 0, 1, 0, None, a, None)
    assert rc == _cabi.ERR_ALIGN
    rc = lib.tdb_attn_fwd_fixed(a, a, a, a, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, None, None, 0, None, 0, None, None, 0, 0,
                                None, 1, 16, 2, 64, 0.1, 3, 1, 0, None, a, None)
    assert rc == _cabi.ERR_SHAPE or rc == _cabi.ERR_ARG                          # position terms without tables
    rc = lib.tdb_attn_fwd_varlen(a, a, a, a, 128, 64, 128, 64, 128, 64, 128, 64, None, None, 0, None, 0, None, None, 0, 0,
                                 a, 2, 100, 50, 2, 64, 0.1, 0, 1, 2, None, 0, None, a, None)
    assert rc == _cabi.ERR_WORKSPACE
    assert b"workspace" in lib.tdb_last_error()


def test_ops_refuse_cpu_tensors():
    import torch
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    q = torch.zeros(1, 2, 16, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_attention_with_disentangled(q, q, q, None, None)
