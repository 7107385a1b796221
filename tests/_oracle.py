"""ctypes access to the CPU oracle (oracle/_build/liboracle.so) and to the reference shim
(oracle/_ref/libref.so). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "liboracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libref.so")

_o = None
_r = None


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def load_oracle():
    global _o
    if _o is None:
        if not os.path.exists(ORACLE_SO):
            subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
        _o = Oracle(C.CDLL(ORACLE_SO))
    return _o


def load_ref():
    global _r
    if _r is None:
        if not os.path.exists(REF_SO):
            return None
        _r = C.CDLL(REF_SO)
    return _r


class Oracle:
    def __init__(self, lib):
        self.lib = lib

    def f16_to_f32(self, bits):
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.size, dtype=np.float32)
        self.lib.bo_f16_to_f32(_p(bits), bits.size, _p(out))
        return out

    def f32_to_f16(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.size, dtype=np.uint16)
        self.lib.bo_f32_to_f16(_p(x), x.size, _p(out))
        return out

    def ptq_dequant(self, blocks):
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 28)
        out = np.empty((b.shape[0], 128), dtype=np.float32)
        self.lib.bo_ptq_dequant(_p(b), C.c_long(b.shape[0]), _p(out))
        return out

    def ptq_trits(self, blocks):
        b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 28)
        out = np.empty((b.shape[0], 128), dtype=np.int8)
        self.lib.bo_ptq_trits(_p(b), C.c_long(b.shape[0]), _p(out))
        return out

    def ptq_encode(self, sym, scale_bits):
        s = np.ascontiguousarray(sym, dtype=np.int8).reshape(-1, 128)
        sb = np.ascontiguousarray(scale_bits, dtype=np.uint16).reshape(-1)
        out = np.empty((s.shape[0], 28), dtype=np.uint8)
        self.lib.bo_ptq_encode(_p(s), _p(sb), C.c_long(s.shape[0]), _p(out))
        return out

    def quantize_q8_1(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.size // 128 * 36, dtype=np.uint32)
        self.lib.bo_quantize_q8_1(_p(x), x.size, _p(out))
        return out

    def quantize_q8_0(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        codes = np.empty(x.size, dtype=np.int8)
        scales = np.empty(x.size // 32, dtype=np.uint16)
        self.lib.bo_quantize_q8_0(_p(x), x.size, _p(codes), _p(scales))
        return codes, scales

    def block_dots(self, block, xq_block, shader=False, fast=False):
        b = np.ascontiguousarray(block, dtype=np.uint8)
        xq = np.ascontiguousarray(xq_block, dtype=np.uint32)
        out = np.empty(4, dtype=np.int32)
        fn = self.lib.bo_block_dots_fast if fast else (self.lib.bo_block_dots_shader if shader else self.lib.bo_block_dots_def)
        fn(_p(b), _p(xq), _p(out))
        return out

    def gemv_q81(self, W, M, K, xq, want_dots=False, threads=8):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        xq = np.ascontiguousarray(xq, dtype=np.uint32)
        out = np.empty(M, dtype=np.float32)
        exact = np.empty(M, dtype=np.float64)
        dots = np.empty((M, K // 128, 4), dtype=np.int32) if want_dots else None
        self.lib.bo_gemv_q81(_p(W), M, K, _p(xq), _p(out), _p(exact), _p(dots), threads)
        return out, exact, dots

    def gemv_f32act(self, W, M, K, x, n_splits=1, threads=8):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(M, dtype=np.float32)
        exact = np.empty(M, dtype=np.float64)
        self.lib.bo_gemv_f32act(_p(W), M, K, _p(x), n_splits, _p(out), _p(exact), threads)
        return out, exact

    def gemv_dequant_f64(self, W, M, K, x, threads=1):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(M, dtype=np.float64)
        self.lib.bo_gemv_dequant_f64(_p(W), M, K, _p(x), _p(out), threads)
        return out

    def fwht(self, x, block):
        s = np.array(x, dtype=np.float32, copy=True)
        self.lib.bo_fwht(_p(s), s.size, block)
        return s

    def rotate_fwd(self, x, signs, block):
        x = np.ascontiguousarray(x, dtype=np.float32)
        sg = np.ascontiguousarray(signs, dtype=np.int32)
        y = np.empty_like(x)
        self.lib.bo_rotate_fwd(_p(x), _p(sg), x.size, block, _p(y))
        return y

    def rotate_inv(self, x, signs, block):
        x = np.ascontiguousarray(x, dtype=np.float32)
        sg = np.ascontiguousarray(signs, dtype=np.int32)
        y = np.empty_like(x)
        self.lib.bo_rotate_inv(_p(x), _p(sg), x.size, block, _p(y))
        return y

    def rms_norm(self, x, w, eps):
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.bo_rms_norm(_p(x), _p(w), x.size, C.c_float(eps), _p(y))
        return y

    def l2_norm(self, x, eps):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.bo_l2_norm(_p(x), x.size, C.c_float(eps), _p(y))
        return y

    def _unary(self, fn, x, *extra):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        fn(_p(x), x.size, *extra, _p(y))
        return y

    def silu(self, x):
        return self._unary(self.lib.bo_silu, x)

    def sigmoid(self, x):
        return self._unary(self.lib.bo_sigmoid, x)

    def softplus(self, x, thr=20.0):
        return self._unary(self.lib.bo_softplus, x, C.c_float(thr))

    def swiglu(self, a, b):
        a = np.ascontiguousarray(a, dtype=np.float32)
        b = np.ascontiguousarray(b, dtype=np.float32)
        y = np.empty_like(a)
        self.lib.bo_swiglu(_p(a), _p(b), a.size, _p(y))
        return y


class OracleModel:
    """Whole-token CPU oracle over the same tensors (borrowed numpy arrays kept alive here)."""

    def __init__(self, hp, tensors: dict, signs, threads: int = 8, attn_order: int = 1):
        self.o = load_oracle()
        lib = self.o.lib
        lib.bo_model_new.restype = C.c_void_p
        ip = np.array([hp.n_layer, hp.hidden, hp.ffn, hp.vocab, hp.n_head, hp.n_kv, hp.head_dim, hp.n_rot,
                       hp.attn_interval, hp.gdn_heads, hp.gdn_qk_heads, hp.gdn_dim, hp.hat_block, hp.act_mode,
                       hp.k_mode, hp.v_mode], dtype=np.int32)
        fp = np.array([hp.rms_eps, hp.rope_base], dtype=np.float32)
        self.hp = hp
        self.m = C.c_void_p(lib.bo_model_new(_p(ip), _p(fp)))
        lib.bo_model_set_cap(self.m, hp.cap, threads)
        # attn_order 1 = sums grouped as the CUDA kernels group them (pv split rule of bn_model_finalize)
        self.pv_splits = 256 if hp.cap >= 16384 else (64 if hp.cap >= 4096 else (8 if hp.cap >= 512 else 1))
        lib.bo_model_set_attn_order(self.m, attn_order, self.pv_splits)
        mask = int(getattr(hp, "attn_mask", 0))
        lib.bo_model_set_attn_mask(self.m, C.c_uint32(mask & 0xFFFFFFFF), C.c_uint32(mask >> 32))
        self.keep = {n: np.ascontiguousarray(t) for n, t in tensors.items()}
        for n, t in self.keep.items():
            lib.bo_model_set_tensor(self.m, n.encode(), _p(t))
        self.signs = np.ascontiguousarray(signs, dtype=np.int32)
        lib.bo_model_set_signs(self.m, _p(self.signs))
        lib.bo_model_reset(self.m)
        for f in ("bo_model_gdn_state", "bo_model_conv_hist", "bo_model_kq", "bo_model_ks", "bo_model_vq",
                  "bo_model_vs", "bo_model_k16", "bo_model_v16"):
            getattr(lib, f).restype = C.c_void_p

    def set_attn_order(self, order, pv_splits=None):
        self.o.lib.bo_model_set_attn_order(self.m, order, self.pv_splits if pv_splits is None else pv_splits)

    def reset(self):
        self.o.lib.bo_model_reset(self.m)

    def token(self, tok, pos, stop_after=-1):
        """Returns (logits or None, residual)."""
        hp = self.hp
        logits = np.empty(hp.vocab, dtype=np.float32) if stop_after < 0 else None
        res = np.empty(hp.hidden, dtype=np.float32)
        self.o.lib.bo_model_token(self.m, tok, pos, _p(logits), _p(res), stop_after)
        return logits, res

    def argmax(self, logits):
        return int(self.o.lib.bo_argmax(_p(logits), logits.size))

    def _view(self, fn, index, dtype, count):
        ptr = fn(self.m, index)
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(np.ctypeslib.as_ctypes_type(dtype))), shape=(count,)).copy()

    def gdn_state(self, gi):
        hp = self.hp
        return self._view(self.o.lib.bo_model_gdn_state, gi, np.float32, hp.gdn_heads * hp.gdn_dim * hp.gdn_dim)

    def conv_hist(self, gi):
        return self._view(self.o.lib.bo_model_conv_hist, gi, np.float32, self.hp.qkv_dim * 3)

    def kv(self, li):
        hp = self.hp
        n = hp.cap * hp.n_kv * hp.head_dim
        L = self.o.lib
        k = (self._view(L.bo_model_kq, li, np.int8, n), self._view(L.bo_model_ks, li, np.uint16, n // 32)) if hp.k_mode == 0 \
            else (self._view(L.bo_model_k16, li, np.uint16, n), None)
        v = (self._view(L.bo_model_vq, li, np.int8, n), self._view(L.bo_model_vs, li, np.uint16, n // 32)) if hp.v_mode == 0 \
            else (self._view(L.bo_model_v16, li, np.uint16, n), None)
        return k, v

    def close(self):
        self.o.lib.bo_model_free(self.m)
