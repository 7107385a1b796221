"""GGUF v3 writer for synthetic models of the qwen35/PTQ1_0 shape, so that the C++ host can be driven end to
end without a checkpoint. The keys and conventions are the ones the reference loader reads
(runtime_vk/bonsai_gguf.h:72-155 header and tensor table; runtime_vk/bonsai_model.h:642-760 hyper-parameter keys,
:773-912 prism.hadamard.* keys): d0 is the reduction length, PTQ1_0 is dtype 143, f32 is dtype 0, tensor data
starts at the next multiple of general.alignment and every tensor offset is aligned to it.
"""
from __future__ import annotations

import struct

import numpy as np

from . import synth

T_U32, T_I32, T_F32, T_STR, T_ARR, T_U64 = 4, 5, 6, 8, 9, 10
DTYPE_F32, DTYPE_PTQ1_0 = 0, 143
ARCH = "qwen35"


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, ty: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", ty) + payload


def kv_u32(k, v): return _kv(k, T_U32, struct.pack("<I", v))
def kv_f32(k, v): return _kv(k, T_F32, struct.pack("<f", v))
def kv_str(k, v): return _kv(k, T_STR, _s(v))
def kv_arr_i32(k, a): return _kv(k, T_ARR, struct.pack("<IQ", T_I32, len(a)) + np.asarray(a, dtype="<i4").tobytes())
def kv_arr_str(k, a): return _kv(k, T_ARR, struct.pack("<IQ", T_STR, len(a)) + b"".join(_s(x) for x in a))


def layer_type_kv(hp: synth.HParams, spelling: str) -> list[bytes]:
    """The layer-typing keys in one of the spellings the loader accepts (reference contract: bonsai_model.h:432-468):
    "interval" (full_attention_interval), "list" (string array, one token per block), "string" (one comma-separated
    string), "numeric" (array of 0/1), "both" (interval and list), "none" (no key: the tensor table alone decides)."""
    A = ARCH + "."
    tokens = ["full_attention" if hp.is_attn(b) else "linear_attention" for b in range(hp.n_layer)]
    out = []
    if spelling in ("interval", "both"):
        out.append(kv_u32(A + "full_attention_interval", hp.attn_interval))
    if spelling in ("list", "both"):
        out.append(kv_arr_str(A + "attention.layer_types", tokens))
    if spelling == "string":
        out.append(kv_str(A + "layer_types", ", ".join(tokens)))
    if spelling == "numeric":
        out.append(kv_arr_i32(A + "layers.types", [1 if hp.is_attn(b) else 0 for b in range(hp.n_layer)]))
    if spelling not in ("interval", "both", "list", "string", "numeric", "none"):
        raise ValueError(f"unknown layer spelling {spelling}")
    return out


def byte_image() -> list[str]:
    """The printable stand-in of every byte that byte-level BPE vocabularies use (the GPT-2 table): bytes 33..126,
    161..172 and 174..255 stand for themselves, the others are moved to code points 256, 257, ... in byte order."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    out, extra = {}, 0
    for b in range(256):
        if b in keep:
            out[b] = chr(b)
        else:
            out[b] = chr(256 + extra)
            extra += 1
    return [out[b] for b in range(256)]


def toy_tokenizer(vocab: int, words=("hello", "world", "the")) -> tuple[list[str], list[str]]:
    """A small byte-level BPE vocabulary for tests: ids 0..255 are the single bytes (so any text can be encoded),
    then the merge products that build each of `words` left to right, then fillers. Returns (tokens, merges)."""
    img = byte_image()
    tokens = list(img)
    merges = []
    for w in words:
        cur = img[ord(w[0])]
        for ch in w[1:]:
            nxt = img[ord(ch)]
            if f"{cur} {nxt}" not in merges:
                merges.append(f"{cur} {nxt}")
            cur = cur + nxt
            if cur not in tokens:
                tokens.append(cur)
    assert len(tokens) <= vocab
    tokens += [f"<filler{i}>" for i in range(len(tokens), vocab)]
    return tokens, merges


def metadata(hp: synth.HParams, signs: np.ndarray, hat_version: int = 1, names: list[str] | None = None,
             layer_spelling: str | None = None, extra_kv: list[bytes] | None = None, tokenizer=None) -> list[bytes]:
    A = ARCH + "."
    if layer_spelling is None:
        layer_spelling = "interval" if hp.attn_interval > 0 else "list"
    kv = [
        kv_str("general.architecture", ARCH),
        kv_u32("general.alignment", 32),
        kv_u32(A + "block_count", hp.n_layer),
        kv_u32(A + "embedding_length", hp.hidden),
        kv_u32(A + "feed_forward_length", hp.ffn),
        kv_u32(A + "attention.head_count", hp.n_head),
        kv_u32(A + "attention.head_count_kv", hp.n_kv),
        kv_u32(A + "attention.key_length", hp.head_dim),
        kv_u32(A + "attention.value_length", hp.head_dim),
        kv_u32(A + "rope.dimension_count", hp.n_rot),
        *layer_type_kv(hp, layer_spelling),
        *(extra_kv or []),
        kv_u32(A + "ssm.conv_kernel", 4),
        kv_u32(A + "ssm.state_size", hp.gdn_dim),
        kv_u32(A + "ssm.group_count", hp.gdn_qk_heads),
        kv_u32(A + "ssm.time_step_rank", hp.gdn_heads),
        kv_u32(A + "ssm.inner_size", hp.gdn_heads * hp.gdn_dim),
        kv_f32(A + "attention.layer_norm_rms_epsilon", hp.rms_eps),
        kv_f32(A + "rope.freq_base", hp.rope_base),
        kv_arr_str("tokenizer.ggml.tokens", tokenizer[0] if tokenizer else [f"<{i}>" for i in range(hp.vocab)]),
    ]
    if tokenizer:
        kv += [kv_str("tokenizer.ggml.model", "gpt2"), kv_arr_str("tokenizer.ggml.merges", tokenizer[1])]
    if hat_version is not None:
        kv.append(kv_u32("prism.hadamard.version", hat_version))
        kv += [
            kv_str("prism.hadamard.transform", "normalized-sylvester-walsh-hadamard"),
            kv_u32("prism.hadamard.block_size", hp.hat_block),
            kv_str("prism.hadamard.sign_mode", "explicit"),
            kv_arr_i32("prism.hadamard.sign_widths", [hp.hidden, hp.ffn]),
            kv_arr_i32("prism.hadamard.sign_values", signs),
        ]
    return kv


def write(path: str, hp: synth.HParams, seed: int = 0, hat_version: int | None = 1, shuffle: bool = False,
          override_dtype: dict[str, int] | None = None, layer_spelling: str | None = None,
          extra_kv: list[bytes] | None = None, tokenizer=None, repeat: bool = False) -> dict:
    """Write a synthetic model. Tensors are generated one at a time (the 9B shape never sits in memory whole).
    shuffle=True stores the tensors in name-sorted order (as real checkpoints do) instead of layer order.
    repeat=True reuses one generated tensor per kind of tensor for every block and one 16 384-row chunk for the two
    vocabulary-sized tensors (synth.make_model_repeated's rule): a file of the full 9B size in seconds, for timing
    the loader; the values repeat, the bytes and shapes are the real ones.
    Returns {"tensors": n, "bytes": file size}."""
    shapes = synth.tensor_shapes(hp)
    names = sorted(shapes) if shuffle else list(shapes)
    signs = synth.make_signs(hp, seed)
    kv = metadata(hp, signs, hat_version, layer_spelling=layer_spelling, extra_kv=extra_kv, tokenizer=tokenizer)
    recs, off = [], 0
    for n in names:
        spec = shapes[n]
        if spec[0] == "ptq":
            dims, dtype, nbytes = (spec[2], spec[1]), DTYPE_PTQ1_0, spec[1] * spec[2] // 128 * 28
        else:
            dims, dtype, nbytes = tuple(reversed(spec[1])), DTYPE_F32, int(np.prod(spec[1])) * 4
        if override_dtype and n in override_dtype:
            dtype = override_dtype[n]
        recs.append((n, dims, dtype, off, nbytes))
        off = (off + nbytes + 31) // 32 * 32
    head = b"GGUF" + struct.pack("<IQQ", 3, len(recs), len(kv)) + b"".join(kv)
    for n, dims, dtype, o, _ in recs:
        head += _s(n) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", dtype, o)
    pad = (-len(head)) % 32
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        base = f.tell()
        cache = {}
        for n, dims, dtype, o, nbytes in recs:
            f.seek(base + o)
            if repeat:
                key = n.split(".", 2)[-1] if n.startswith("blk.") else ("vocab" if shapes[n][0] == "ptq" else n)
                if key not in cache:
                    if key == "vocab":
                        from . import ptq
                        chunk = ptq.synth_matrix(np.random.default_rng(seed + 1), min(16384, hp.vocab), hp.hidden)
                        cache[key] = np.concatenate([chunk] * ((hp.vocab + len(chunk) - 1) // len(chunk)), axis=0)[:hp.vocab]
                    else:
                        cache[key] = synth.make_tensor(hp, seed, n, shapes[n])
                a = np.ascontiguousarray(cache[key])
            else:
                a = np.ascontiguousarray(synth.make_tensor(hp, seed, n, shapes[n]))
            assert a.nbytes == nbytes, (n, a.nbytes, nbytes)
            f.write(a.tobytes())
        size = f.tell()
    return {"tensors": len(recs), "bytes": size}


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="write a seeded synthetic qwen35/PTQ1_0 GGUF")
    ap.add_argument("path")
    ap.add_argument("--shape", choices=["tiny", "9b"], default="tiny")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--repeat", action="store_true", help="reuse one tensor per kind for every block (a full-size file in seconds)")
    a = ap.parse_args()
    print(write(a.path, synth.tiny() if a.shape == "tiny" else synth.HParams(), a.seed, repeat=a.repeat))
