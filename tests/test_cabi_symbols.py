"""The C-ABI library loads and exports every symbol include/shflbw.h declares; op entry
points fail with a status (never abort, never compute on the CPU) when no GPU is present."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import shflbw_sparse_nn_b200 as sb
from shflbw_sparse_nn_b200 import _cabi

HEADER = Path(__file__).resolve().parent.parent / "include" / "shflbw.h"


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(shflbw_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    declared = _declared_functions()
    assert len(declared) >= 35
    lib = C.CDLL(str(_cabi.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in shflbw.h but not exported"
    assert declared == _cabi.exported_symbols(), "ctypes prototypes out of sync with the header"
    assert _cabi.lib().shflbw_abi_version() == 1


def test_state_structs_match_the_header_field_order():
    text = HEADER.read_text()
    for struct, cls in (("shflbw_spmm_state", _cabi.SpmmState), ("shflbw_spconv_state", _cabi.SpconvState)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s_t;" % (struct, struct), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                names.append(re.sub(r"[\*\s]", " ", re.sub(r"\[.*?\]", "", part)).split()[-1])   # arrays: name without [n]
        assert names == [f[0] for f in cls._fields_], struct


def test_strerror_covers_all_codes():
    l = _cabi.lib()
    texts = {l.shflbw_strerror(i).decode() for i in range(8)}
    assert len(texts) == 8 and "unknown status" not in texts
    assert l.shflbw_strerror(99).decode() == "unknown status"


def _no_gpu() -> bool:
    import torch
    return not torch.cuda.is_available()


@pytest.mark.skipif(not _no_gpu(), reason="checks the no-GPU error path")
def test_ops_report_cuda_error_without_a_gpu():
    m = sb.BlockwiseSpMatrix().init_random(64, 64, 32, 1, 0.2, True, 1, values="uniform")
    with pytest.raises(sb.ShflbwError) as e:
        m.transform_and_sync_device()
    assert e.value.status == _cabi.ERR_CUDA
    st = _cabi.SpmmState()
    rc = _cabi.lib().shflbw_spmm_init(m._h, 64, 16, 1.0, None, 0.0, 32, 0, C.byref(st))
    assert rc == _cabi.ERR_NOT_ON_DEVICE and st.init_success == 0
    B = np.zeros((64, 64), np.float16)
    with pytest.raises(sb.ShflbwError):
        sb.spmm_host(m, 64, B, np.zeros((64, 64), np.float16))   # no CPU fallback


def test_init_argument_checks():
    l = _cabi.lib()
    st = _cabi.SpmmState()
    m = sb.BlockwiseSpMatrix().init_random(64, 64, 32, 1, 0.2, False, 1, values="uniform")
    assert l.shflbw_spmm_init(None, 64, 16, 1.0, None, 0.0, 32, 0, C.byref(st)) == _cabi.ERR_INVALID_ARG
    assert l.shflbw_spmm_init(m._h, 64, None, 1.0, None, 0.0, 32, 0, C.byref(st)) == _cabi.ERR_INVALID_ARG
    assert l.shflbw_spmm_init(m._h, 64, 16, 1.0, None, 1.0, 32, 0, C.byref(st)) == _cabi.ERR_INVALID_ARG  # beta w/o C
    assert l.shflbw_spmm_init(m._h, 64, 16, 1.0, None, 0.0, 32, 9, C.byref(st)) == _cabi.ERR_INVALID_ARG  # bad kernel id
    assert l.shflbw_spmm_exec(C.byref(st), None) == _cabi.ERR_INVALID_ARG                                   # not initialised
    cst = _cabi.SpconvState()
    assert l.shflbw_spconv_init(m._h, 8, 6, 6, 1, 16, 32, 1.0, 0, C.byref(cst)) == _cabi.ERR_INVALID_ARG   # not a filter
