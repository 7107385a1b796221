"""Seeded synthetic models of the qwen35/PTQ1_0 shape (random-init weights; no checkpoint is
available offline). Tensor names and shapes follow the real checkpoint's tensor table
(reference: gguf_meta.txt:238-260); value distributions follow the benchmark configs: trits i.i.d.
P(-1)=P(+1)=0.3, P(0)=0.4, one fp16 scale per 128 weights drawn from |N(0, 0.02)|.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, asdict

import numpy as np

from . import ptq


@dataclass
class HParams:
    n_layer: int = 32
    hidden: int = 4096
    ffn: int = 12288
    vocab: int = 248320
    n_head: int = 16
    n_kv: int = 4
    head_dim: int = 256
    n_rot: int = 64
    attn_interval: int = 4
    gdn_heads: int = 32
    gdn_qk_heads: int = 16
    gdn_dim: int = 128
    hat_block: int = 4096
    act_mode: int = 0
    k_mode: int = 0
    v_mode: int = 0
    cap: int = 256
    rms_eps: float = 1e-6
    rope_base: float = 1e7
    n_streams: int = 1          # independent sequences resident on the device
    block_begin: int = 0        # pipeline stage: this device holds blocks [block_begin, block_end)
    block_end: int = 0          # 0 = n_layer
    batch_cols: int = 0         # > 0: the multi-sequence pass (stage_batch) may take up to this many sequences per call
    attn_mask: int = 0          # attn_interval == 0: explicit layer typing, bit b set = block b is an attention block

    def is_attn(self, b: int) -> bool:
        if self.attn_interval == 0:
            return bool((self.attn_mask >> b) & 1)
        return b % self.attn_interval == self.attn_interval - 1

    @property
    def qkv_dim(self) -> int:
        return 2 * self.gdn_qk_heads * self.gdn_dim + self.gdn_heads * self.gdn_dim

    def asdict(self):
        return asdict(self)


def tiny(**kw) -> HParams:
    """A small model with every structural feature of the 9B (GDN + attention blocks, GQA 4:1,
    rope on a prefix of the head, 3 Hadamard blocks in the FFN)."""
    base = dict(n_layer=4, hidden=1024, ffn=3072, vocab=2048, n_head=4, n_kv=1, gdn_heads=8, gdn_qk_heads=4,
                hat_block=1024, cap=64)
    base.update(kw)
    return HParams(**base)


def _rng(seed: int, name: str) -> np.random.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return np.random.default_rng(int.from_bytes(h[:8], "little"))


def tensor_shapes(hp: HParams) -> dict[str, tuple]:
    """name -> ("ptq", M, K) | ("f32", shape)."""
    out: dict[str, tuple] = {}
    H, D = hp.hidden, hp.gdn_dim
    QD, KD = hp.n_head * hp.head_dim, hp.n_kv * hp.head_dim
    IN = hp.gdn_heads * D
    out["token_embd.weight"] = ("ptq", hp.vocab, H)
    out["output.weight"] = ("ptq", hp.vocab, H)
    out["output_norm.weight"] = ("f32", (H,))
    for b in range(hp.n_layer):
        B = f"blk.{b}."
        out[B + "attn_norm.weight"] = ("f32", (H,))
        out[B + "post_attention_norm.weight"] = ("f32", (H,))
        out[B + "ffn_gate.weight"] = ("ptq", hp.ffn, H)
        out[B + "ffn_up.weight"] = ("ptq", hp.ffn, H)
        out[B + "ffn_down.weight"] = ("ptq", H, hp.ffn)
        if hp.is_attn(b):
            out[B + "attn_q.weight"] = ("ptq", 2 * QD, H)
            out[B + "attn_k.weight"] = ("ptq", KD, H)
            out[B + "attn_v.weight"] = ("ptq", KD, H)
            out[B + "attn_output.weight"] = ("ptq", H, QD)
            out[B + "attn_q_norm.weight"] = ("f32", (hp.head_dim,))
            out[B + "attn_k_norm.weight"] = ("f32", (hp.head_dim,))
        else:
            out[B + "attn_qkv.weight"] = ("ptq", hp.qkv_dim, H)
            out[B + "attn_gate.weight"] = ("ptq", IN, H)
            out[B + "ssm_out.weight"] = ("ptq", H, IN)
            out[B + "ssm_alpha.weight"] = ("f32", (hp.gdn_heads, H))
            out[B + "ssm_beta.weight"] = ("f32", (hp.gdn_heads, H))
            out[B + "ssm_dt.bias"] = ("f32", (hp.gdn_heads,))
            out[B + "ssm_a"] = ("f32", (hp.gdn_heads,))
            out[B + "ssm_conv1d.weight"] = ("f32", (hp.qkv_dim, 4))      # GGUF dims {4, channels}
            out[B + "ssm_norm.weight"] = ("f32", (D,))
    return out


def make_tensor(hp: HParams, seed: int, name: str, spec: tuple) -> np.ndarray:
    rng = _rng(seed, name)
    if spec[0] == "ptq":
        _, M, K = spec
        return ptq.synth_matrix(rng, M, K)
    shape = spec[1]
    if name.endswith("norm.weight"):
        return (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32)
    if name.endswith("ssm_alpha.weight") or name.endswith("ssm_beta.weight"):
        return (0.02 * rng.standard_normal(shape)).astype(np.float32)
    if name.endswith("ssm_dt.bias"):
        return rng.standard_normal(shape).astype(np.float32)
    if name.endswith("ssm_a"):
        return (-np.exp(0.5 * rng.standard_normal(shape)) * 0.5).astype(np.float32)   # negative: log decay
    if name.endswith("ssm_conv1d.weight"):
        return (0.5 * rng.standard_normal(shape)).astype(np.float32)
    raise KeyError(name)


def make_signs(hp: HParams, seed: int) -> np.ndarray:
    """prism.hadamard.sign_values: +-1 int32, [hidden values | ffn values]."""
    rng = _rng(seed, "prism.hadamard.sign_values")
    return (rng.integers(0, 2, size=hp.hidden + hp.ffn, dtype=np.int32) * 2 - 1).astype(np.int32)


def make_model(hp: HParams, seed: int = 0):
    """Returns (tensors: name -> ndarray, signs). Fine for small models; the 9B goes through the
    streaming GGUF writer instead."""
    tensors = {n: make_tensor(hp, seed, n, s) for n, s in tensor_shapes(hp).items()}
    return tensors, make_signs(hp, seed)


def make_model_repeated(hp: HParams, seed: int = 0, head_everywhere: bool = False):
    """Seeded synthetic tensors of a large shape, quickly: generating 8.9e9 trits in numpy takes minutes, so one
    GDN block, one attention block and one FFN set are generated and reused for every block, and the two
    vocab-sized tensors tile a 16384-row chunk. Timing depends on shapes and bytes, not on values. Only the
    tensors of the local blocks [block_begin, block_end) are produced (head_everywhere: the output head and its norm
    too, whatever the block range - every stage holds a slice of a sharded head)."""
    cache, tensors = {}, {}
    b0, b1 = hp.block_begin, (hp.block_end or hp.n_layer)
    for name, spec in tensor_shapes(hp).items():
        if name.startswith("blk."):
            if not (b0 <= int(name.split(".")[1]) < b1):
                continue
            key = name.split(".", 2)[-1]
        else:
            key = name
            if (name == "token_embd.weight" and b0 != 0) or (name != "token_embd.weight" and b1 != hp.n_layer and not head_everywhere):
                continue
        if key in ("token_embd.weight", "output.weight"):
            if "vocab" not in cache:
                chunk = ptq.synth_matrix(np.random.default_rng(seed + 1), 16384, hp.hidden)
                cache["vocab"] = np.concatenate([chunk] * ((hp.vocab + 16383) // 16384), axis=0)[:hp.vocab]
            tensors[name] = cache["vocab"]
            continue
        if key not in cache:
            cache[key] = make_tensor(hp, seed, name, spec)
        tensors[name] = cache[key]
    return tensors, make_signs(hp, seed)
