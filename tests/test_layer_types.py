"""Layer typing of the C++ host (reference contract: runtime_vk/bonsai_model.h:432-472): explicit per-layer lists in
their three payload forms, the interval key, counts as cross-checks, the tensor table, and the agreement rule - every
spelling that answers must give the same mask, anything else is refused with exit code 2 before any GPU work."""
import dataclasses
import os
import subprocess

import pytest

from bonsai_vk_b200 import build, gguf_writer, synth
from bonsai_vk_b200.gguf_writer import ARCH, kv_arr_str, kv_str, kv_u32


@pytest.fixture(scope="module")
def exe():
    build.build_lib()
    return build.build_host()


def info(exe, path):
    return subprocess.run([exe, path, "info"], capture_output=True, text=True, env=dict(os.environ), timeout=300)


IRREGULAR = synth.tiny(n_layer=6, attn_interval=0, attn_mask=0b110010)        # R A R R A A


@pytest.mark.parametrize("spelling", ["list", "string", "numeric", "none"])
def test_explicit_spellings_give_the_same_layers(exe, tmp_path, spelling):
    p = str(tmp_path / f"{spelling}.gguf")
    gguf_writer.write(p, IRREGULAR, seed=2, layer_spelling=spelling)
    r = info(exe, p)
    assert r.returncode == 0, r.stderr
    assert "layer types RARRAA " in r.stdout
    assert "interval 0 " in r.stdout


def test_interval_and_list_that_agree_are_accepted(exe, tmp_path):
    hp = synth.tiny()                                                     # interval 4: R R R A
    p = str(tmp_path / "both.gguf")
    gguf_writer.write(p, hp, seed=2, layer_spelling="both")
    r = info(exe, p)
    assert r.returncode == 0, r.stderr
    assert "layer types RRRA " in r.stdout
    p2 = str(tmp_path / "interval.gguf")
    gguf_writer.write(p2, hp, seed=2)
    r2 = info(exe, p2)
    assert r2.returncode == 0 and "layer types RRRA " in r2.stdout and "interval 4 " in r2.stdout


def test_disagreement_and_malformed_lists_are_refused(exe, tmp_path):
    A = ARCH + "."
    hp = synth.tiny()
    cases = {
        # the list says block 0 is attention, the interval and the tensor table say block 3
        "conflict": dict(hp=hp, layer_spelling="interval",
                         extra_kv=[kv_arr_str(A + "attention.layer_types", ["attn", "ssm", "ssm", "ssm"])], want="disagrees"),
        "short": dict(hp=hp, layer_spelling="interval", extra_kv=[kv_arr_str(A + "layer_types", ["ssm", "ssm", "attn"])], want="entries"),
        "window": dict(hp=hp, layer_spelling="interval",
                       extra_kv=[kv_str(A + "layer_types", "ssm, ssm, ssm, sliding_window")], want="no kernels"),
        "word": dict(hp=hp, layer_spelling="interval", extra_kv=[kv_str(A + "layer_types", "ssm ssm ssm banana")], want="unknown layer type"),
        "zero": dict(hp=dataclasses.replace(hp, attn_interval=0, attn_mask=0b1000), layer_spelling="list",
                     extra_kv=[kv_u32(A + "full_attention_interval", 0)], want="must be >= 1"),
        "count": dict(hp=hp, layer_spelling="interval", extra_kv=[kv_u32(A + "ssm_layer_count", 2)], want="ssm_layer_count"),
        "count_alone": dict(hp=dataclasses.replace(hp, attn_interval=0, attn_mask=0b1000), layer_spelling="none",
                            extra_kv=[kv_u32(A + "attn_layer_count", 1)], want="cannot say where"),
        # the tensor table is always computed: a list that contradicts the tensors each block carries is refused
        "table": dict(hp=dataclasses.replace(hp, attn_interval=0, attn_mask=0b1000), layer_spelling="none",
                      extra_kv=[kv_arr_str("prism.layer_types", ["ssm", "attn", "ssm", "attn"])], want="disagrees"),
    }
    for tag, c in cases.items():
        p = str(tmp_path / f"{tag}.gguf")
        gguf_writer.write(p, c["hp"], seed=2, layer_spelling=c["layer_spelling"], extra_kv=c["extra_kv"])
        r = info(exe, p)
        assert r.returncode == 2, (tag, r.stdout, r.stderr)
        assert c["want"] in r.stderr, (tag, r.stderr)


def test_counts_that_agree_pass(exe, tmp_path):
    A = ARCH + "."
    p = str(tmp_path / "counts.gguf")
    gguf_writer.write(p, synth.tiny(), seed=2, extra_kv=[kv_u32(A + "ssm_layer_count", 3), kv_u32(A + "full_attention_layer_count", 1)])
    assert info(exe, p).returncode == 0
