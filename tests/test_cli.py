"""The command line (`bin/lumenllm`, `python -m lumenllm_b200`): what runs without a GPU
(parsing, the random-model command, loud failure on a machine without one) and, marked gpu,
`generate` and `bench-generate` as programs against the plain implementation and against the
Python entry point, flags over the parameters file, and the errors a user sees."""
import json
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P
from conftest import ROOT, TINY
from lumenllm_b200 import cli

BIN = str(ROOT / "bin" / "lumenllm")


def run(*args):
    return subprocess.run([sys.executable, BIN, *map(str, args)], capture_output=True, text=True, timeout=600)


def test_token_lists_parse():
    assert cli._ids("1,2, 3  4") == [1, 2, 3, 4]
    assert cli._ids("  ") == []
    with pytest.raises(ValueError):
        cli._ids("1,x")


def test_random_model_command_writes_a_folder_the_plain_loader_reads(tmp_path):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY["B"]))
    out = tmp_path / "model"
    assert cli.main(["random-model", "--config-json", str(cfg), "--out", str(out), "--seed", "5",
                     "--std", "0.05", "--norm-jitter", "0.1"]) == 0
    assert (out / "config.json").exists() and (out / "model.safetensors").exists()
    got, w = P.load_model(out)
    assert got["hidden_size"] == TINY["B"]["hidden_size"]
    assert w["model.embed_tokens.weight"].shape == (TINY["B"]["vocab_size"], TINY["B"]["hidden_size"])
    from lumenllm_b200.weights.safetensors_io import read_header
    assert read_header(out / "model.safetensors")["model.embed_tokens.weight"].dtype == "BF16"
    # the same seed gives the same weights, another seed others
    again = tmp_path / "again"
    cli.main(["random-model", "--config-json", str(cfg), "--out", str(again), "--seed", "5",
              "--std", "0.05", "--norm-jitter", "0.1"])
    assert torch.equal(P.load_model(again)[1]["lm_head.weight"], w["lm_head.weight"])
    other = tmp_path / "other"
    cli.main(["random-model", "--config-json", str(cfg), "--out", str(other), "--seed", "6",
              "--std", "0.05", "--norm-jitter", "0.1"])
    assert not torch.equal(P.load_model(other)[1]["lm_head.weight"], w["lm_head.weight"])


def test_a_command_is_required_and_unknown_flags_are_refused(capsys):
    with pytest.raises(SystemExit):
        cli.main([])
    with pytest.raises(SystemExit):
        cli.main(["generate", "--no-such-flag"])
    capsys.readouterr()


@pytest.mark.skipif(torch.cuda.is_available(), reason="this is what a machine without a GPU sees")
def test_without_a_gpu_generate_says_so(tiny_models):
    r = run("generate", "--model", tiny_models["A"], "--prompt-tokens", "1,2,3")
    assert r.returncode != 0
    assert "no CPU path" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_as_a_program(dtype, tiny_models):
    cfg, w = P.load_model(tiny_models["B"])
    prompts = [[5, 17, 3, 200, 9], [7], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]]
    args = ["generate", "--model", tiny_models["B"], "--dtype", dtype, "--ctx-size", 128, "--max-tokens", 6]
    for p in prompts:
        args += ["--prompt-tokens", ",".join(map(str, p))]
    r = run(*args)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert len(lines) == len(prompts)
    for p, line in zip(prompts, lines):
        toks = [int(x) for x in line.split(",")]
        assert len(toks) == 6
        if dtype == "float32":
            assert toks == P.generate_greedy(cfg, w, p, 6)[0]
        else:       # each token is the plain implementation's best, or within rounding of it
            lg = P.forward_logits(cfg, w, p + toks)
            for k, t in enumerate(toks):
                row = lg[len(p) - 1 + k]
                assert float(row.max() - row[t]) <= 0.06 * max(1.0, float(row.abs().max()))
    status = [l for l in r.stderr.splitlines() if l.startswith("finish=")]
    assert status == [f"finish=length prompt_tokens={len(p)} completion_tokens=6" for p in prompts]


@pytest.mark.gpu
def test_generate_json_stop_eos_and_the_python_entry_agree(tiny_models, tmp_path):
    from lumenllm_b200 import EngineConfig, GenerateRequest, build
    folder = tiny_models["D"]
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [2, 7, 1, 8]]
    pf = tmp_path / "prompts.json"
    pf.write_text(json.dumps(prompts))
    built = build(EngineConfig(model_path=str(folder), dtype="float32", context_size=128))
    free = built.generate([GenerateRequest(p, 8) for p in prompts], eos_token_ids=[])
    r = run("generate", "--model", folder, "--dtype", "float32", "--ctx-size", 128, "--prompt-file", pf,
            "--max-tokens", 8, "--format", "json", "--eos", "")
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout)
    assert [g["tokens"] for g in got] == [o.tokens for o in free]
    assert all(g["finish_reason"] == "length" and g["completion_tokens"] == 8 for g in got)
    # the third token of the first request as a stop token: kept, and the request ends there;
    # as an end-of-sequence token: not kept
    third = free[0].tokens[2]
    first_at = free[0].tokens.index(third)
    r = run("generate", "--model", folder, "--dtype", "float32", "--ctx-size", 128, "--prompt-tokens",
            ",".join(map(str, prompts[0])), "--max-tokens", 8, "--format", "json", "--stop", third, "--eos", "")
    g = json.loads(r.stdout)[0]
    assert g["tokens"] == free[0].tokens[:first_at + 1] and g["finish_reason"] == "stop"
    r = run("generate", "--model", folder, "--dtype", "float32", "--ctx-size", 128, "--prompt-tokens",
            ",".join(map(str, prompts[0])), "--max-tokens", 8, "--format", "json", "--eos", third)
    g = json.loads(r.stdout)[0]
    assert g["tokens"] == free[0].tokens[:first_at] and g["finish_reason"] == "eos_token"


@pytest.mark.gpu
def test_flags_override_the_parameters_file_and_seeded_sampling_repeats(tiny_models, tmp_path):
    params = tmp_path / "parameters.json"
    params.write_text(json.dumps({"model": {
        "path": str(tiny_models["A"]), "dtype": "bfloat16",
        "hidden-layers": {"kv-cache": {"context-size": 128}},
        "other-parameters": {"temperature": 0.9, "top-k": 20, "top-p": 0.9, "seed": 4}}}))
    base = ["generate", "--config", params, "--prompt-tokens", "9,8,7,6", "--max-tokens", 12]
    a, b = run(*base), run(*base)
    assert a.returncode == 0, a.stderr
    assert a.stdout == b.stdout                         # the file's seed: the same draw twice
    c = run(*base, "--seed", 5)
    d = run(*base, "--temp", 0)                         # the flag turns sampling off
    e = run("generate", "--model", tiny_models["A"], "--ctx-size", 128, "--prompt-tokens", "9,8,7,6",
            "--max-tokens", 12)                         # no file: greedy by default
    assert c.returncode == 0 and d.returncode == 0 and e.returncode == 0
    assert d.stdout == e.stdout
    assert c.stdout != a.stdout or a.stdout != d.stdout   # some option changed some draw
    # an unknown key in the file is refused by name
    params.write_text(json.dumps({"model": {"path": str(tiny_models["A"]), "no-such-key": 1}}))
    r = run(*base)
    assert r.returncode == 2 and "no-such-key" in r.stderr


@pytest.mark.gpu
def test_bench_generate_and_the_errors_a_user_sees(tiny_models, tmp_path):
    r = run("bench-generate", "--model", tiny_models["A"], "--ctx-size", 128, "--prompt-tokens", "1,2,3,4",
            "--prompt-tokens", "5,6", "--max-tokens", 5, "--warmup", 1, "--runs", 2, "--format", "json")
    assert r.returncode == 0, r.stderr
    rec = json.loads(r.stdout)
    assert rec["runs"] == 2 and rec["prompt_tokens"] == 6 and rec["completion_tokens"] == 10
    assert rec["prefill_s"] > 0 and rec["decode_tok_s"] > 0
    # a token outside the vocabulary, a prompt longer than the context, a folder without weights
    r = run("generate", "--model", tiny_models["A"], "--ctx-size", 128, "--prompt-tokens", "1,99999")
    assert r.returncode == 2 and "error:" in r.stderr
    r = run("generate", "--model", tiny_models["A"], "--ctx-size", 64, "--prompt-tokens",
            ",".join(["1"] * 80), "--max-tokens", 4)
    assert r.returncode == 2 and "error:" in r.stderr
    empty = tmp_path / "empty"
    empty.mkdir()
    (empty / "config.json").write_text(json.dumps(TINY["A"]))
    r = run("generate", "--model", empty, "--prompt-tokens", "1")
    assert r.returncode == 2 and "model.safetensors" in r.stderr
