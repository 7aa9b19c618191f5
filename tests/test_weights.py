import json
import struct

import pytest
import torch

from conftest import TINY
from lumenllm_b200.config import config_from_dict
from lumenllm_b200.engine.model import expected_tensors
from lumenllm_b200.weights import (WeightError, load_weights, open_checkpoint, random_weights,
                                   read_header, write_file, write_random_model)


def _expected(name):
    """(shapes of the tensors the model must find, kinds of all it reads)."""
    spec = config_from_dict(TINY[name]).model_spec()
    kinds = expected_tensors(spec)
    return {n: s for n, (s, k) in kinds.items() if k != "optional"}, kinds


def test_random_model_reads_back_by_name(tiny_models):
    for name, folder in tiny_models.items():
        exp, kinds = _expected(name)
        w = load_weights(folder, exp, "cpu")
        assert set(w) == set(exp)
        assert all(t.dtype == torch.bfloat16 for t in w.values())
        again = random_weights(kinds, 11 + list(TINY).index(name), 0.05, 0.1, torch.bfloat16)
        for n in exp:
            assert torch.equal(w[n], again[n]), n
        cfg = json.loads((folder / "config.json").read_text())
        assert cfg["hidden_size"] == TINY[name]["hidden_size"]


def test_tied_head_has_no_tensor_of_its_own():
    expA, kindsA = _expected("A")
    expB, _ = _expected("B")
    assert "lm_head.weight" not in expA and "lm_head.weight" in expB
    assert kindsA["lm_head.weight"][1] == "optional"
    assert "lm_head.weight" not in random_weights(kindsA, 1, 0.05, 0.1, torch.float32)


def test_the_head_is_chosen_by_what_the_file_stores(tmp_path):
    """As the reference does (executor/full.rs:171-181): a stored lm_head.weight is the head,
    whatever config.json says about tying; without one the embedding is."""
    from lumenllm_b200.engine.model import tensor_fallbacks
    from lumenllm_b200.parts import build_part
    from lumenllm_b200.parts.base import Runtime
    rt = Runtime(torch.device("cpu"), torch.float32)
    # tied by config.json, and the file stores a head all the same
    spec = config_from_dict(TINY["A"]).model_spec()
    kinds = expected_tensors(spec)
    t = random_weights(kinds, 3, 0.05, 0.1, torch.bfloat16)
    t["lm_head.weight"] = torch.randn(kinds["lm_head.weight"][0]).to(torch.bfloat16)
    write_file(tmp_path / "model.safetensors", t)
    shapes = {n: s for n, (s, _) in kinds.items()}
    w = load_weights(tmp_path, shapes, "cpu", optional=["lm_head.weight"], fallbacks=tensor_fallbacks(spec))
    assert torch.equal(build_part("head", spec.head, w, rt).proj.weight, t["lm_head.weight"])
    del t["lm_head.weight"]
    write_file(tmp_path / "model.safetensors", t)
    w = load_weights(tmp_path, shapes, "cpu", optional=["lm_head.weight"], fallbacks=tensor_fallbacks(spec))
    assert "lm_head.weight" not in w and not w.stood_in
    assert torch.equal(build_part("head", spec.head, w, rt).proj.weight, t["model.embed_tokens.weight"])
    # untied by config.json, and the file stores no head
    spec = config_from_dict(TINY["B"]).model_spec()
    kinds = expected_tensors(spec)
    shapes = {n: s for n, (s, _) in kinds.items()}
    t = random_weights(kinds, 3, 0.05, 0.1, torch.bfloat16)
    del t["lm_head.weight"]
    write_file(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightError, match="missing tensors"):
        load_weights(tmp_path, shapes, "cpu")
    w = load_weights(tmp_path, shapes, "cpu", fallbacks=tensor_fallbacks(spec))
    assert w.stood_in == {"lm_head.weight": "model.embed_tokens.weight"}
    assert torch.equal(build_part("head", spec.head, w, rt).proj.weight, t["model.embed_tokens.weight"])


def test_harmless_extras_and_the_strict_switch(tmp_path):
    exp, kinds = _expected("B")
    t = random_weights(kinds, 3, 0.05, 0.1, torch.bfloat16)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.randn(16)
    write_file(tmp_path / "model.safetensors", t)
    assert load_weights(tmp_path, exp, "cpu").unexpected == []      # a table nobody reads
    t["model.layers.0.extra.weight"] = torch.randn(2)
    write_file(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightError, match="unexpected tensors") as ei:
        load_weights(tmp_path, exp, "cpu")
    assert ei.value.unexpected == ["model.layers.0.extra.weight"]
    w = load_weights(tmp_path, exp, "cpu", strict=False)
    assert w.unexpected == ["model.layers.0.extra.weight"] and set(w) == set(exp)
    del t["model.norm.weight"]                 # a missing tensor stays fatal without strict
    write_file(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightError, match="missing tensors"):
        load_weights(tmp_path, exp, "cpu", strict=False)


def test_values_do_not_depend_on_order():
    _, kinds = _expected("A")
    a = random_weights(kinds, 5, 0.05, 0.1, torch.float32)
    b = random_weights(dict(reversed(list(kinds.items()))), 5, 0.05, 0.1, torch.float32)
    assert all(torch.equal(a[n], b[n]) for n in a) and set(a) == set(b)
    c = random_weights(kinds, 6, 0.05, 0.1, torch.float32)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert float((a["model.norm.weight"] - 1).abs().max()) <= 0.1


def test_kept_dtypes(tmp_path):
    t = {"a": torch.randn(3, 4).to(torch.bfloat16), "b": torch.randn(3), "c": torch.randn(2).half(),
         "d": torch.tensor([1, 2, 3], dtype=torch.int64)}
    write_file(tmp_path / "model.safetensors", t)
    w = load_weights(tmp_path, {"a": (3, 4), "b": (3,), "c": (2,), "d": (3,)}, "cpu")
    assert w["a"].dtype == torch.bfloat16 and torch.equal(w["a"], t["a"])
    assert w["b"].dtype == torch.float32 and torch.equal(w["b"], t["b"])
    assert w["c"].dtype == torch.float32 and torch.equal(w["c"], t["c"].float())
    assert w["d"].dtype == torch.int32 and w["d"].tolist() == [1, 2, 3]


def test_one_error_lists_everything(tmp_path, tiny_models):
    exp, _ = _expected("B")
    import plain_qwen3 as P
    tensors = P.read_safetensors(tiny_models["B"] / "model.safetensors")
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(7, 96, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    write_file(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as ei:
        load_weights(tmp_path, exp, "cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (256, 96), (7, 96))]
    text = str(e)
    for s in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)",
              "expected [256, 96], got [7, 96]"):
        assert s in text


def test_file_errors(tmp_path):
    with pytest.raises(WeightError, match="missing file"):
        open_checkpoint(tmp_path)
    p = tmp_path / "model.safetensors"
    write_file(p, {"a": torch.zeros(4, 4)})
    raw = p.read_bytes()
    p.write_bytes(raw[:-8])
    with pytest.raises(WeightError, match="truncated"):
        open_checkpoint(tmp_path)
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hlen])
    hdr["a"]["dtype"] = "F8_E4M3"
    hj = json.dumps(hdr).encode()
    p.write_bytes(struct.pack("<Q", len(hj)) + hj + raw[8 + hlen:])
    with pytest.raises(WeightError, match="unsupported dtype"):
        open_checkpoint(tmp_path)
    hdr["a"]["dtype"] = "F32"
    hdr["a"]["shape"] = [4, 5]
    hj = json.dumps(hdr).encode()
    p.write_bytes(struct.pack("<Q", len(hj)) + hj + raw[8 + hlen:])
    with pytest.raises(WeightError, match="needs 80"):
        open_checkpoint(tmp_path)
    p.write_bytes(b"version https://git-lfs.github.com/spec/v1\noid sha256:0\nsize 1\n")
    with pytest.raises(WeightError, match="git-lfs"):
        open_checkpoint(tmp_path)


def test_sharded_index(tmp_path):
    write_file(tmp_path / "s1.safetensors", {"a": torch.ones(2)})
    write_file(tmp_path / "s2.safetensors", {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    w = load_weights(tmp_path, {"a": (2,), "b": (3,)}, "cpu")
    assert w["a"].tolist() == [1, 1] and w["b"].shape == (3,)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s1.safetensors"}}))
    with pytest.raises(WeightError, match="does not hold"):
        open_checkpoint(tmp_path)


def test_header_reader():
    import tempfile, os
    d = tempfile.mkdtemp()
    write_file(os.path.join(d, "x.safetensors"), {"t": torch.arange(6, dtype=torch.float32).view(2, 3)})
    h = read_header(os.path.join(d, "x.safetensors"))
    assert h["t"].shape == (2, 3) and h["t"].dtype == "F32" and h["t"].end - h["t"].begin == 24
