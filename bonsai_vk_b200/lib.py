"""ctypes binding of libbonsai_cuda.so (C ABI: include/bonsai_cuda.h)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BONSAI_CUDA_LIB") or os.path.join(HERE, "libbonsai_cuda.so")     # override: a differently built copy (experiments)

_lib = None


class BonsaiError(RuntimeError):
    pass


class HParamsC(C.Structure):
    """Mirror of bn_hparams (include/bonsai_cuda.h)."""
    _fields_ = [(n, C.c_int32) for n in (
        "n_layer", "hidden", "ffn", "vocab", "n_head", "n_kv", "head_dim", "n_rot", "attn_interval",
        "gdn_heads", "gdn_qk_heads", "gdn_dim", "hat_block", "act_mode", "k_mode", "v_mode", "cap")] + [
        ("rms_eps", C.c_float), ("rope_base", C.c_float)] + [(n, C.c_int32) for n in ("n_streams", "block_begin", "block_end", "batch_cols")] + [
        ("attn_mask_lo", C.c_uint32), ("attn_mask_hi", C.c_uint32)]


class AttnDimsC(C.Structure):
    """Mirror of bn_attn_dims."""
    _fields_ = [(n, C.c_int32) for n in ("n_head", "n_kv", "head_dim", "n_rot", "cap", "k_mode", "v_mode")] + [
        ("rms_eps", C.c_float), ("rope_base", C.c_float)]


READ_LOGITS, READ_RESIDUAL, READ_GDN_STATE, READ_CONV_HIST, READ_K_DATA, READ_K_SCALE, READ_V_DATA, READ_V_SCALE = range(8)


def load_library() -> C.CDLL:
    """Load the CUDA library. Raises if it has not been built (python bonsai_vk_b200/build.py)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BonsaiError(f"{LIB_PATH} is missing: build it with `python bonsai_vk_b200/build.py` "
                          "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    sig = {
        "bn_last_error": (C.c_char_p, []),
        "bn_init": (i32, [i32, C.POINTER(vp)]),
        "bn_destroy": (None, [vp]),
        "bn_device_info": (i32, [vp, C.POINTER(i32), C.POINTER(sz), C.POINTER(sz)]),
        "bn_alloc": (i32, [vp, sz, C.POINTER(vp)]),
        "bn_free": (i32, [vp, vp]),
        "bn_buf_size": (sz, [vp]),
        "bn_upload": (i32, [vp, vp, sz, vp, sz]),
        "bn_upload_async": (i32, [vp, vp, sz, vp, sz]),
        "bn_download": (i32, [vp, vp, sz, vp, sz]),
        "bn_memset": (i32, [vp, vp, sz, i32, sz]),
        "bn_sync": (i32, [vp]),
        "bn_selftest_wait": (i32, [vp, i32]),
        "bn_host_alloc": (i32, [sz, C.POINTER(vp)]),
        "bn_host_free": (i32, [vp]),
        "bn_event_create": (i32, [vp, C.POINTER(vp)]),
        "bn_event_record": (i32, [vp, vp]),
        "bn_event_elapsed_ms": (i32, [vp, vp, vp, C.POINTER(C.c_float)]),
        "bn_event_destroy": (i32, [vp, vp]),
        "bn_launch_count": (C.c_uint64, [vp]),
        "bn_act_pack_bytes": (sz, [i32]),
        "bn_act_quant_q81": (i32, [vp, vp, sz, i32, vp, sz]),
        "bn_gemv_q81": (i32, [vp, vp, sz, i32, i32, vp, sz, vp, sz, vp, sz]),
        "bn_gemv_q81_static": (i32, [vp, vp, sz, i32, i32, vp, sz, vp, sz]),
        "bn_gemv_f32act_splits": (i32, [i32, i32]),
        "bn_gemv_f32act": (i32, [vp, vp, sz, i32, i32, vp, sz, i32, vp, sz]),
        "bn_gemm_image_bytes": (sz, [i32, i32]),
        "bn_gemm_act_quant": (i32, [vp, vp, sz, sz, i32, i32, vp, sz, i32, vp, sz]),
        "bn_gemm_q81": (i32, [vp, vp, sz, i32, i32, i32, vp, sz, i32, vp, sz, sz]),
        "bn_gemm_tiled_bytes": (sz, [i32, i32]),
        "bn_gemm_repack": (i32, [vp, vp, sz, i32, i32, vp, sz]),
        "bn_attn_kv_bytes": (sz, [C.POINTER(AttnDimsC)]),
        "bn_attn_scratch_bytes": (sz, [C.POINTER(AttnDimsC)]),
        "bn_attn_insert": (i32, [vp, C.POINTER(AttnDimsC), vp, sz, vp, sz, vp, sz, i32, i32, vp, sz, vp, sz, vp, sz, vp, sz]),
        "bn_attn_attend": (i32, [vp, C.POINTER(AttnDimsC), vp, sz, i32, vp, sz, vp, sz, vp, sz]),
        "bn_model_create": (i32, [vp, C.POINTER(HParamsC), C.POINTER(vp)]),
        "bn_model_set_tensor": (i32, [vp, C.c_char_p, vp, sz, sz]),
        "bn_model_set_signs": (i32, [vp, vp, sz, i32]),
        "bn_model_finalize": (i32, [vp]),
        "bn_model_reset": (i32, [vp]),
        "bn_model_destroy": (None, [vp]),
        "bn_model_token": (i32, [vp, i32, i32, i32, C.POINTER(i32)]),
        "bn_model_read": (i32, [vp, i32, i32, vp, sz]),
        "bn_model_decode": (i32, [vp, i32, i32, i32, C.POINTER(i32)]),
        "bn_model_stage_prepare": (i32, [vp, i32, i32]),
        "bn_model_stage": (i32, [vp, i32, i32, i32, vp, sz, vp, sz]),
        "bn_model_stage_batch": (i32, [vp, i32, i32, vp, vp, vp, sz, vp, sz]),
        "bn_model_reset_stream": (i32, [vp, i32]),
        "bn_model_prefill": (i32, [vp, vp, i32, i32, C.POINTER(i32)]),
        "bn_model_set_head_rows": (i32, [vp, i32, i32]),
        "bn_model_head_batch": (i32, [vp, i32, vp, sz, vp, sz]),
        "bn_model_pick_batch": (i32, [vp, i32, i32, vp, sz, vp, sz]),
        "bn_model_fill_kv": (i32, [vp, i32, i32]),
        "bn_wrap": (i32, [vp, vp, sz, C.POINTER(vp)]),
        "bn_use_stream": (i32, [vp, vp]),
        "bn_model_gemv_sweep": (i32, [vp, i32, C.POINTER(C.c_float)]),
        "bn_model_mixer_sweep": (i32, [vp, i32, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
        "bn_model_profile_token": (i32, [vp, i32, i32, vp, i32, C.POINTER(i32)]),
    }
    for name, (res, args) in sig.items():
        f = getattr(lib, name)
        f.restype = res
        f.argtypes = args
    lib._bn_signatures = sig
    _lib = lib
    return lib


def declared_symbols() -> list[str]:
    """Entry points declared in include/bonsai_cuda.h (parsed from the header text)."""
    import re
    hdr = os.path.join(os.path.dirname(HERE), "include", "bonsai_cuda.h")
    text = open(hdr).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bn_[a-z0-9_]+)\s*\(", text)))


def _check(rc: int, what: str):
    if rc != 0:
        msg = load_library().bn_last_error().decode()
        raise BonsaiError(f"{what} failed ({rc}): {msg}")


class Buffer:
    """Device buffer owned by the library; named by handle + byte offset in every op."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx = ctx
        self.nbytes = int(nbytes)
        h = C.c_void_p()
        _check(ctx.lib.bn_alloc(ctx.h, self.nbytes, C.byref(h)), "bn_alloc")
        self.h = h

    def upload(self, arr: np.ndarray, off: int = 0):
        a = np.ascontiguousarray(arr)
        _check(self.ctx.lib.bn_upload(self.ctx.h, self.h, off, a.ctypes.data_as(C.c_void_p), a.nbytes), "bn_upload")
        return self

    def download(self, dtype, count: int, off: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        _check(self.ctx.lib.bn_download(self.ctx.h, self.h, off, out.ctypes.data_as(C.c_void_p), out.nbytes),
               "bn_download")
        return out

    def memset(self, byte: int = 0, off: int = 0, n: int | None = None):
        _check(self.ctx.lib.bn_memset(self.ctx.h, self.h, off, byte, self.nbytes - off if n is None else n), "bn_memset")

    def free(self):
        if self.h is not None:
            self.ctx.lib.bn_free(self.ctx.h, self.h)
            self.h = None


class Context:
    """One context per GPU (reference: the single Vulkan device + queue of vk_ctx_init)."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = C.c_void_p()
        _check(self.lib.bn_init(device, C.byref(h)), "bn_init")
        self.h = h
        self.device = device

    def close(self):
        if self.h is not None:
            self.lib.bn_destroy(self.h)
            self.h = None

    def alloc(self, nbytes: int) -> Buffer:
        return Buffer(self, nbytes)

    def from_numpy(self, arr: np.ndarray) -> Buffer:
        a = np.ascontiguousarray(arr)
        return Buffer(self, max(a.nbytes, 16)).upload(a)

    def sync(self):
        _check(self.lib.bn_sync(self.h), "bn_sync")

    def selftest_wait(self, which: int):
        """Queue a kernel whose bounded wait must give up (0: copy-ring wait, 1: tensor-core pipeline wait); the next
        sync() then raises BonsaiError with code BN_ERR_TIMEOUT and the context stays usable."""
        _check(self.lib.bn_selftest_wait(self.h, which), "bn_selftest_wait")

    def use_stream(self, cuda_stream: int):
        """Run this context's kernels on a stream owned by the caller (e.g. torch's current stream)."""
        _check(self.lib.bn_use_stream(self.h, C.c_void_p(cuda_stream)), "bn_use_stream")

    def wrap(self, device_ptr: int, nbytes: int) -> "Buffer":
        """A Buffer over device memory the caller owns (e.g. a torch tensor used for NCCL send/recv)."""
        b = Buffer.__new__(Buffer)
        b.ctx, b.nbytes = self, int(nbytes)
        h = C.c_void_p()
        _check(self.lib.bn_wrap(self.h, C.c_void_p(device_ptr), int(nbytes), C.byref(h)), "bn_wrap")
        b.h = h
        return b

    def info(self):
        sm, fr, tot = C.c_int(), C.c_size_t(), C.c_size_t()
        _check(self.lib.bn_device_info(self.h, C.byref(sm), C.byref(fr), C.byref(tot)), "bn_device_info")
        return {"sm_count": sm.value, "free_bytes": fr.value, "total_bytes": tot.value}

    @property
    def launches(self) -> int:
        return int(self.lib.bn_launch_count(self.h))

    # events
    def event(self):
        h = C.c_void_p()
        _check(self.lib.bn_event_create(self.h, C.byref(h)), "bn_event_create")
        return h

    def record(self, ev):
        _check(self.lib.bn_event_record(self.h, ev), "bn_event_record")

    def elapsed_ms(self, a, b) -> float:
        ms = C.c_float()
        _check(self.lib.bn_event_elapsed_ms(self.h, a, b, C.byref(ms)), "bn_event_elapsed_ms")
        return float(ms.value)

    # ops
    def act_pack_bytes(self, K: int) -> int:
        return int(self.lib.bn_act_pack_bytes(K))

    def act_quant_q81(self, x: Buffer, K: int, pack: Buffer, x_off: int = 0, pack_off: int = 0):
        _check(self.lib.bn_act_quant_q81(self.h, x.h, x_off, K, pack.h, pack_off), "bn_act_quant_q81")

    def gemv_q81(self, w: Buffer, M: int, K: int, pack: Buffer, out: Buffer, w_off: int = 0, pack_off: int = 0,
                 out_off: int = 0, dots: Buffer | None = None, dots_off: int = 0):
        _check(self.lib.bn_gemv_q81(self.h, w.h, w_off, M, K, pack.h, pack_off, out.h, out_off,
                                    dots.h if dots is not None else None, dots_off), "bn_gemv_q81")

    def attn_sizes(self, dims: "AttnDimsC"):
        return int(self.lib.bn_attn_kv_bytes(C.byref(dims))), int(self.lib.bn_attn_scratch_bytes(C.byref(dims)))

    def attn_insert(self, dims, kv: Buffer, k_rows: Buffer, v_rows: Buffer, n: int, pos0: int, qg: Buffer, q_norm: Buffer,
                    k_norm: Buffer, scratch: Buffer, k_off: int = 0, v_off: int = 0):
        _check(self.lib.bn_attn_insert(self.h, C.byref(dims), kv.h, 0, k_rows.h, k_off, v_rows.h, v_off, n, pos0, qg.h, 0,
                                       q_norm.h, 0, k_norm.h, 0, scratch.h, 0), "bn_attn_insert")

    def attn_attend(self, dims, kv: Buffer, pos: int, scratch: Buffer, pregate: "Buffer | None", gated: Buffer):
        _check(self.lib.bn_attn_attend(self.h, C.byref(dims), kv.h, 0, pos, scratch.h, 0,
                                       pregate.h if pregate is not None else None, 0, gated.h, 0), "bn_attn_attend")

    def gemv_q81_static(self, w: Buffer, M: int, K: int, pack: Buffer, out: Buffer, w_off: int = 0, pack_off: int = 0,
                        out_off: int = 0):
        """The projection with its scratch in the library's built-in array: no device allocation."""
        _check(self.lib.bn_gemv_q81_static(self.h, w.h, w_off, M, K, pack.h, pack_off, out.h, out_off), "bn_gemv_q81_static")


def _gemm_methods():
    def gemm_image_bytes(self, K: int, ncol: int) -> int:
        return int(self.lib.bn_gemm_image_bytes(K, ncol))

    def gemm_act_quant(self, x: Buffer, K: int, ncol: int, image: Buffer, signs: "Buffer | None" = None, hat_block: int = 0,
                       x_stride: int = 0, x_off: int = 0, signs_off: int = 0):
        """ncol fp32 vectors -> the activation image of the multi-column projection (optional rotation first)."""
        _check(self.lib.bn_gemm_act_quant(self.h, x.h, x_off, x_stride or K, K, ncol, signs.h if signs is not None else None,
                                          signs_off, hat_block, image.h, 0), "bn_gemm_act_quant")

    def gemm_q81(self, w: Buffer, M: int, K: int, image: Buffer, ncol: int, out: Buffer, out_stride: int = 0, w_off: int = 0,
                 tiled: bool = False):
        _check(self.lib.bn_gemm_q81(self.h, w.h, w_off, 1 if tiled else 0, M, K, image.h, 0, ncol, out.h, 0, out_stride or M),
               "bn_gemm_q81")

    def gemm_repack(self, w: Buffer, M: int, K: int, w_off: int = 0) -> Buffer:
        """The tile-major copy of a weight matrix for gemm_q81(tiled=True)."""
        out = self.alloc(int(self.lib.bn_gemm_tiled_bytes(M, K)))
        _check(self.lib.bn_gemm_repack(self.h, w.h, w_off, M, K, out.h, 0), "bn_gemm_repack")
        return out

    def gemv_f32act(self, w: Buffer, M: int, K: int, x: Buffer, out: Buffer, n_splits: int = 0):
        """The reference engine's fp32-activation projection (n_splits 0 = the reference's split rule)."""
        _check(self.lib.bn_gemv_f32act(self.h, w.h, 0, M, K, x.h, 0, n_splits, out.h, 0), "bn_gemv_f32act")

    Context.gemv_f32act = gemv_f32act
    Context.gemm_image_bytes, Context.gemm_act_quant, Context.gemm_q81 = gemm_image_bytes, gemm_act_quant, gemm_q81
    Context.gemm_repack = gemm_repack


_gemm_methods()


class Model:
    """Device-resident model: tensors registered by GGUF name (reference: engine_init + fwd_init)."""

    def __init__(self, ctx: Context, hp, tensors: dict, signs: np.ndarray, head_rows=None):
        """head_rows = (row_begin, row_end): this model holds that slice of the output head for the multi-sequence pass
        (bn_model_set_head_rows); its last stage then returns hidden states and head_batch / pick_batch make the pick."""
        self.ctx, self.hp = ctx, hp
        self.head_rows = head_rows
        lib = ctx.lib
        fields = {f[0] for f in HParamsC._fields_}
        hc = HParamsC(**{k: (float(v) if k in ("rms_eps", "rope_base") else int(v)) for k, v in hp.asdict().items() if k in fields})
        mask = int(getattr(hp, "attn_mask", 0))
        hc.attn_mask_lo, hc.attn_mask_hi = mask & 0xFFFFFFFF, mask >> 32
        h = C.c_void_p()
        _check(lib.bn_model_create(ctx.h, C.byref(hc), C.byref(h)), "bn_model_create")
        self.h = h
        al = lambda n: (n + 255) & ~255
        total = sum(al(np.asarray(t).nbytes) for t in tensors.values()) + al(signs.nbytes)
        self.weights = ctx.alloc(total)
        off = 0
        b0, b1 = getattr(hp, "block_begin", 0), (getattr(hp, "block_end", 0) or hp.n_layer)

        def local(name: str) -> bool:
            if name.startswith("blk."):
                return b0 <= int(name.split(".")[1]) < b1
            if name == "token_embd.weight":
                return b0 == 0
            return b1 == hp.n_layer or head_rows is not None     # output.weight, output_norm.weight

        tensors = {n: t for n, t in tensors.items() if local(n)}
        total = sum(al(np.asarray(t).nbytes) for t in tensors.values()) + al(signs.nbytes)
        self.weights.free()
        self.weights = ctx.alloc(total)
        for name, t in tensors.items():
            a = np.ascontiguousarray(t)
            self.weights.upload(a, off)
            _check(lib.bn_model_set_tensor(self.h, name.encode(), self.weights.h, off, a.nbytes), f"set_tensor {name}")
            off += al(a.nbytes)
        sg = np.ascontiguousarray(signs, dtype=np.int32)
        self.weights.upload(sg, off)
        _check(lib.bn_model_set_signs(self.h, self.weights.h, off, sg.size), "bn_model_set_signs")
        if head_rows is not None:
            _check(lib.bn_model_set_head_rows(self.h, int(head_rows[0]), int(head_rows[1])), "bn_model_set_head_rows")
        _check(lib.bn_model_finalize(self.h), "bn_model_finalize")

    def reset(self):
        _check(self.ctx.lib.bn_model_reset(self.h), "bn_model_reset")

    def reset_stream(self, stream: int):
        _check(self.ctx.lib.bn_model_reset_stream(self.h, stream), "bn_model_reset_stream")

    def token(self, tok: int, pos: int, stop_after: int = -1, want_next: bool = True):
        nxt = C.c_int32(-1)
        _check(self.ctx.lib.bn_model_token(self.h, tok, pos, stop_after, C.byref(nxt) if want_next else None),
               "bn_model_token")
        return int(nxt.value)

    def stage(self, stream: int, tok: int, pos: int, inp: "Buffer | None", out: "Buffer", in_off: int = 0, out_off: int = 0):
        """One pipeline stage for one token of one stream (enqueue only)."""
        _check(self.ctx.lib.bn_model_stage(self.h, stream, tok, pos, inp.h if inp is not None else None, in_off, out.h, out_off),
               "bn_model_stage")

    def stage_prepare(self, stream0: int, ncol: int = 0):
        """Build the replayable schedule of stage() (ncol = 0) or of stage_batch() over ncol sequences from stream0. May
        synchronise the device: call it before any NCCL traffic. Unprepared calls of stage / stage_batch are refused."""
        _check(self.ctx.lib.bn_model_stage_prepare(self.h, stream0, ncol), "bn_model_stage_prepare")

    def stage_batch(self, stream0: int, toks, pos, inp: "Buffer | None", out: "Buffer", in_off: int = 0, out_off: int = 0):
        """One pipeline stage for len(pos) consecutive sequences at once (enqueue only). toks: token ids (first stage)
        or None (ids or hidden states are read from inp)."""
        n = len(pos)
        pa = (C.c_int32 * n)(*[int(p) for p in pos])
        ta = (C.c_int32 * n)(*[int(t) for t in toks]) if toks is not None else None
        _check(self.ctx.lib.bn_model_stage_batch(self.h, stream0, n, ta, pa, inp.h if inp is not None else None, in_off, out.h, out_off),
               "bn_model_stage_batch")

    def prefill(self, toks, pos0: int, want_next: bool = True):
        """len(toks) consecutive positions of the sequence in one pass (batched prefill); returns the pick after the last."""
        n = len(toks)
        ta = (C.c_int32 * n)(*[int(t) for t in toks])
        nxt = C.c_int32(-1)
        _check(self.ctx.lib.bn_model_prefill(self.h, ta, n, pos0, C.byref(nxt) if want_next else None), "bn_model_prefill")
        return int(nxt.value)

    def head_batch(self, ncol: int, inp: "Buffer", out: "Buffer", in_off: int = 0, out_off: int = 0):
        """This model's shard of the output head for ncol sequences: final hidden states in, (value, row) candidates out."""
        _check(self.ctx.lib.bn_model_head_batch(self.h, ncol, inp.h, in_off, out.h, out_off), "bn_model_head_batch")

    def pick_batch(self, ncol: int, n_shards: int, cands: "Buffer", out: "Buffer", cands_off: int = 0, out_off: int = 0):
        """First maximum over the shards' candidates (shards in ascending row order): ncol token ids."""
        _check(self.ctx.lib.bn_model_pick_batch(self.h, ncol, n_shards, cands.h, cands_off, out.h, out_off), "bn_model_pick_batch")

    def fill_kv(self, stream: int, n_positions: int):
        _check(self.ctx.lib.bn_model_fill_kv(self.h, stream, n_positions), "bn_model_fill_kv")

    def decode(self, first_tok: int, pos0: int, n_steps: int, fetch: bool = True):
        """n_steps greedy tokens chained on the device; returns the picks (or None when fetch=False)."""
        out = (C.c_int32 * n_steps)() if fetch else None
        _check(self.ctx.lib.bn_model_decode(self.h, first_tok, pos0, n_steps, out), "bn_model_decode")
        return list(out) if fetch else None

    def profile_token(self, tok: int, pos: int, max_phases: int = 256) -> np.ndarray:
        """[n_phases, 8] device time stamps (ns) of the fused projection kernels of one token."""
        out = np.zeros((max_phases, 8), dtype=np.uint64)
        n = C.c_int32()
        _check(self.ctx.lib.bn_model_profile_token(self.h, tok, pos, out.ctypes.data_as(C.c_void_p), max_phases, C.byref(n)),
               "bn_model_profile_token")
        return out[: n.value]

    def mixer_sweep_us(self, reps: int = 3):
        """(us per gated-delta-net core, us per attention chain) at the current position, device-timed."""
        a, b = C.c_float(0), C.c_float(0)
        _check(self.ctx.lib.bn_model_mixer_sweep(self.h, reps, C.byref(a), C.byref(b)), "bn_model_mixer_sweep")
        return float(a.value), float(b.value)

    def gemv_sweep_ms(self, reps: int = 3) -> float:
        ms = C.c_float()
        _check(self.ctx.lib.bn_model_gemv_sweep(self.h, reps, C.byref(ms)), "bn_model_gemv_sweep")
        return float(ms.value)

    def read(self, what: int, dtype, count: int, index: int = 0) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        _check(self.ctx.lib.bn_model_read(self.h, what, index, out.ctypes.data_as(C.c_void_p), out.nbytes), "bn_model_read")
        return out

    def logits(self, col: int = 0):
        """Logits of the last token; col = the column of a multi-sequence pass."""
        return self.read(READ_LOGITS, np.float32, self.hp.vocab, index=col)

    def residual(self):
        return self.read(READ_RESIDUAL, np.float32, self.hp.hidden)

    def close(self):
        if self.h is not None:
            self.ctx.lib.bn_model_destroy(self.h)
            self.h = None
            self.weights.free()
