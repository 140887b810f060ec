"""The command line: parsing on the CPU, a generation on the GPU."""
import json
import os
import subprocess
import sys

import pytest

from herbert_rs_b200.cli import build_parser, main, parse_ids

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_defaults_are_the_references():
    a = build_parser().parse_args(["--model", "m", "--prompt-ids", "1,2"])
    assert (a.backend, a.max_tokens, a.temperature, a.top_k, a.top_p) == ("auto", 2048, 0.4, 40, 0.9)
    assert not a.ignore_eos and not a.no_repeat_check and not a.verbose


def test_prompt_ids_parsing():
    assert parse_ids("1, 2,3") == [1, 2, 3] and parse_ids("7 8") == [7, 8]
    with pytest.raises(ValueError):
        parse_ids("1,a")
    with pytest.raises(ValueError):
        parse_ids(" ")


def test_backend_help_and_errors(capsys):
    assert main(["--backend", "help"]) == 0
    assert "cuda-bf16" in capsys.readouterr().out
    assert main(["--prompt", "hello"]) == 1
    assert "tokenizer" in capsys.readouterr().err
    assert main(["--model", "x"]) == 1
    assert "no prompt" in capsys.readouterr().err


@pytest.mark.gpu
def test_cli_generates_what_the_library_call_generates(model_dirs, tmp_path):
    import herbert_rs_b200 as hb
    cmd = [sys.executable, os.path.join(ROOT, "bin", "herbert-cli"), "--model", model_dirs["B"], "--backend", "cuda-fp32",
           "--prompt-ids", "5,17,3", "--prompt-ids", "9", "--max-tokens", "6", "--temperature", "0", "--ignore-eos",
           "--verbose", "--logits-out", str(tmp_path / "l.f32")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.strip().splitlines()]
    eng = hb.Engine.from_folder(model_dirs["B"], dtype="float32", max_tokens=256)
    want = hb.generate(eng, [[5, 17, 3], [9]], hb.GenerationOptions(max_tokens=6, ignore_eos=True),
                       hb.SamplingParams(temperature=0.0)).tokens
    assert lines == want
    stats = json.loads(p.stderr.strip().splitlines()[-1])
    assert stats["generated_tokens"] == 12 and stats["backend"] == "cuda-fp32"
    assert os.path.getsize(tmp_path / "l.f32") == 2 * 384 * 4
    p = subprocess.run(cmd[:4] + ["--backend", "tpu", "--prompt-ids", "1"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 1 and "unknown backend" in p.stderr


def test_microbench_says_what_it_needs_without_a_gpu():
    import torch
    from herbert_rs_b200.ops import microbench
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(SystemExit, match="CUDA device"):
        microbench.main(["decode-gemm", "--rows", "8"])
    with pytest.raises(SystemExit):
        microbench.main(["no-such-kernel"])
