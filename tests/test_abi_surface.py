"""The C-ABI library loads without a GPU and exports every entry point the header declares."""
import ctypes as C

from bonsai_vk_b200 import lib as L


def test_library_exports_every_declared_symbol():
    lib = L.load_library()
    names = L.declared_symbols()
    assert "bn_init" in names and "bn_gemv_q81" in names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/bonsai_cuda.h but not exported: {missing}"
    unbound = [n for n in names if n not in lib._bn_signatures]
    assert not unbound, f"declared but not bound in bonsai_vk_b200/lib.py: {unbound}"


def test_pack_size_contract():
    lib = L.load_library()
    assert lib.bn_act_pack_bytes(128) == (36 + 512) * 4
    assert lib.bn_act_pack_bytes(4096) == 32 * (36 + 512) * 4
    assert lib.bn_act_pack_bytes(100) == 0


def test_init_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        return
    lib = L.load_library()
    h = C.c_void_p()
    rc = lib.bn_init(0, C.byref(h))
    assert rc != 0
    assert b"no CUDA device" in lib.bn_last_error()
