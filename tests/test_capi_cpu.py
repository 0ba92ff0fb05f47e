"""CPU checks of the C-ABI boundary: the library builds, loads and exports what include/slime_ca.h declares."""
import ctypes
import os
import re

import pytest

from slime_b200 import build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "slime_ca.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(slime_ca_[a-z_]+|launch_multi_head_ca)\s*\(", text)))


def test_header_and_binding_list_agree():
    assert declared_symbols() == sorted(capi.SYMBOLS)


def test_library_builds_loads_and_exports_every_symbol():
    path = build.build()
    assert os.path.exists(path)
    L = ctypes.CDLL(path)
    for name in declared_symbols():
        assert hasattr(L, name), f"{name} is declared in include/slime_ca.h but not exported"
    capi.lib()


def test_no_silent_fallback_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(capi.SlimeCAError) as e:
        capi.Handle(1, 8, 8)
    assert e.value.status == 2          # SLIME_CA_ECUDA: the product path fails loudly, nothing runs on the CPU


def test_bad_arguments_are_rejected_before_any_cuda_call():
    cfg = capi.Config(0, 8, 8, 1, 0, 0.1, 0, 0, 0)
    h = ctypes.c_void_p()
    assert capi.lib().slime_ca_create(ctypes.byref(cfg), ctypes.byref(h)) == 1
    assert capi.lib().slime_ca_create(None, ctypes.byref(h)) == 1
    assert capi.lib().slime_ca_step(None, 1, None) == 1
    assert capi.lib().slime_ca_destroy(None) == 1
    assert capi.lib().slime_ca_last_error(None) == b"null handle"


def test_config_struct_layout():
    assert ctypes.sizeof(capi.Config) == 9 * 4
