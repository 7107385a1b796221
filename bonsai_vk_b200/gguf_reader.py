"""GGUF v3 reader for the Python side (the server): header, metadata and tensor table, tensors as read-only memory
maps. Same file conventions as gguf_writer (reference: runtime_vk/bonsai_gguf.h:72-155, hyper-parameter keys
bonsai_model.h:642-760, prism.hadamard.* :773-912). The C++ host (host/bonsai_host.h) carries the full contract with its
exit codes; this reader takes the layer typing from the interval key or from the tensor table and refuses a file
without the version-1 rotation contract."""
from __future__ import annotations

import struct

import numpy as np

from . import synth

_FIXED = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


def read_header(path: str):
    """-> (kv dict, [(name, dims, dtype, offset)], data_start)."""
    with open(path, "rb") as f:
        buf = f.read()
    if buf[:4] != b"GGUF":
        raise ValueError(f"{path} is not a GGUF file")
    at = 4
    def take(fmt):
        nonlocal at
        v = struct.unpack_from(fmt, buf, at)
        at += struct.calcsize(fmt)
        return v if len(v) > 1 else v[0]
    def text():
        nonlocal at
        n = take("<Q")
        if n > len(buf) - at:
            raise ValueError("truncated GGUF string")
        s = buf[at:at + n].decode("utf-8", "replace")
        at += n
        return s
    def value(ty):
        if ty == 8:
            return text()
        if ty not in _FIXED:
            raise ValueError(f"bad GGUF value type {ty}")
        return take(_FIXED[ty])
    _version, n_tensors, n_kv = take("<IQQ")
    kv = {}
    for _ in range(n_kv):
        key, ty = text(), take("<I")
        if ty == 9:
            et, n = take("<IQ")
            if n > len(buf) - at:
                raise ValueError(f"array {key} is longer than the file")
            if et in _FIXED and et != 8:
                a = np.frombuffer(buf, dtype=np.dtype(_FIXED[et]), count=n, offset=at)
                at += a.nbytes
                kv[key] = a
            else:
                kv[key] = [value(et) for _ in range(n)]
        else:
            kv[key] = value(ty)
    tensors = []
    for _ in range(n_tensors):
        name, nd = text(), take("<I")
        dims = [take("<Q") for _ in range(nd)]
        dtype, off = take("<IQ")
        tensors.append((name, dims, dtype, off))
    align = int(kv.get("general.alignment", 32))
    return kv, tensors, (at + align - 1) // align * align


def load(path: str, cap: int = 4096):
    """-> (HParams, {name: array}, signs). PTQ1_0 tensors come as uint8 [rows, K/128*28], f32 tensors in their shape."""
    kv, table, start = read_header(path)
    A = kv["general.architecture"] + "."
    if int(kv.get("prism.hadamard.version", 0)) != 1:
        raise ValueError("refusing: prism.hadamard.version 1 is required (the weights are stored rotated)")
    names = {t[0] for t in table}
    n_layer = int(kv[A + "block_count"])
    attn = [f"blk.{b}.attn_q.weight" in names for b in range(n_layer)]
    interval = int(kv.get(A + "full_attention_interval", 0))
    if interval and attn != [b % interval == interval - 1 for b in range(n_layer)]:
        raise ValueError("full_attention_interval disagrees with the tensor table")
    hp = synth.HParams(
        n_layer=n_layer, hidden=int(kv[A + "embedding_length"]), ffn=int(kv[A + "feed_forward_length"]),
        vocab=len(kv["tokenizer.ggml.tokens"]), n_head=int(kv[A + "attention.head_count"]), n_kv=int(kv[A + "attention.head_count_kv"]),
        head_dim=int(kv[A + "attention.key_length"]), n_rot=int(kv[A + "rope.dimension_count"]), attn_interval=interval,
        attn_mask=0 if interval else sum(1 << b for b in range(n_layer) if attn[b]),
        gdn_heads=int(kv[A + "ssm.time_step_rank"]), gdn_qk_heads=int(kv[A + "ssm.group_count"]), gdn_dim=int(kv[A + "ssm.state_size"]),
        hat_block=int(kv["prism.hadamard.block_size"]), cap=cap, rms_eps=float(kv[A + "attention.layer_norm_rms_epsilon"]),
        rope_base=float(kv[A + "rope.freq_base"]))
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    tensors = {}
    for name, dims, dtype, off in table:
        n = int(np.prod(dims))
        if dtype == 143:
            nb = n // 128 * 28
            rows = dims[1] if len(dims) > 1 else 1
            tensors[name] = mm[start + off:start + off + nb].reshape(rows, -1)
        elif dtype == 0:
            tensors[name] = mm[start + off:start + off + 4 * n].view(np.float32).reshape(tuple(reversed(dims)))
        else:
            raise ValueError(f"tensor {name}: dtype {dtype} is neither PTQ1_0 (143) nor f32 (0)")
        if start + off + tensors[name].nbytes > mm.size:
            raise ValueError(f"tensor {name} lies outside the file")
    signs = np.asarray(kv["prism.hadamard.sign_values"], dtype=np.int32)
    if signs.size != hp.hidden + hp.ffn:
        raise ValueError(f"prism.hadamard.sign_values holds {signs.size} values, need {hp.hidden + hp.ffn}")
    return hp, tensors, signs
