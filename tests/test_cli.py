"""The command line: option names, defaults and exit codes of the reference's `hos`
(src/main.rs:3459-3577); generation through it on the GPU."""
import os
import subprocess

import pytest

from hos_b200.engine import cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOS = os.path.join(ROOT, "bin", "hos")


def test_defaults_are_the_references():
    a = cli.parse_args([])
    assert (a.n_predict, a.temp, a.top_k, a.top_p, a.rep_penalty, a.repeat_last_n, a.seed) == (64, 0.0, 40, 0.95, 1.1, 64, 42)
    assert a.prompts == [] and not a.no_echo and not a.bench and a.model is None


def test_options_parse():
    a = cli.parse_args(["-m", "dir", "-p", "1,2, 3", "--prompt", "7", "-n", "5", "--temp", "0.7", "--top-k", "3",
                        "--top-p", "0.5", "--repeat-penalty", "1.3", "--repeat-last-n", "9", "--seed", "11",
                        "--no-echo", "--bench", "--fp32", "--gpu", "--batch", "4", "--prompt-len", "100", "--ctx", "512"])
    assert a.model == "dir" and a.prompts == [[1, 2, 3], [7]]
    assert (a.batch, a.prompt_len, a.ctx) == (4, 100, 512)
    assert cli.bench_prompt(50, 7, 0) != cli.bench_prompt(50, 7, 1) and len(cli.bench_prompt(50, 7, 1)) == 7
    assert (a.n_predict, a.temp, a.top_k, a.top_p, a.rep_penalty, a.repeat_last_n, a.seed) == (5, 0.7, 3, 0.5, 1.3, 9, 11)
    assert a.no_echo and a.bench and a.fp32


@pytest.mark.parametrize("argv,code,text", [(["--help"], 0, "usage: hos"), (["--frobnicate"], 2, "unknown argument"),
                                            (["-p", "1,x"], 2, "token ids"), (["-p", "1,2"], 1, "no model")])
def test_exit_codes(argv, code, text):
    env = dict(os.environ)
    env.pop("HOS_MODEL", None)
    p = subprocess.run([HOS] + argv, stdout=subprocess.PIPE, stderr=subprocess.PIPE, env=env)
    assert p.returncode == code and text in p.stderr.decode() and p.stdout == b""


def test_a_broken_model_folder_is_an_error_not_a_crash(tmp_path):
    (tmp_path / "config.json").write_text('{"architectures": ["NopeForCausalLM"]}')
    p = subprocess.run([HOS, "-m", str(tmp_path), "-p", "1"], stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    assert p.returncode == 1 and "unsupported architecture" in p.stderr.decode()


@pytest.mark.gpu
def test_generation_and_bench_through_the_command_line(tmp_path):
    from plain import gemma2_plain as P
    from helpers import make_folder, plain_model
    folder = make_folder(tmp_path, "A")
    w, cfg = plain_model(folder)
    prompt = [9, 200, 31, 4]
    want = P.greedy_generate(w, cfg, prompt, 6)
    base = [HOS, "-m", folder, "--fp32", "--repeat-penalty", "1.0", "-n", "6"]
    p = subprocess.run(base + ["-p", ",".join(map(str, prompt))], stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    assert p.returncode == 0, p.stderr.decode()
    assert p.stdout.decode().strip() == ",".join(map(str, prompt + want))        # the prompt is echoed
    assert "[hos] generated 6 tokens" in p.stderr.decode()
    p = subprocess.run(base + ["--no-echo", "-p", ",".join(map(str, prompt)), "-p", "5"], stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, env=dict(os.environ, HOS_MODEL="/nonexistent"))
    lines = p.stdout.decode().strip().splitlines()
    assert p.returncode == 0 and lines[0] == ",".join(map(str, want)) and len(lines) == 2
    p = subprocess.run([HOS, "--bench", "-n", "4"], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                       env=dict(os.environ, HOS_MODEL=folder))
    out = p.stdout.decode()
    assert p.returncode == 0 and "=== HOS benchmark ===" in out and "prefill    : 16 tok" in out and "decode     : " in out
    p = subprocess.run([HOS, "--bench", "-n", "4", "--batch", "3", "--prompt-len", "10", "--ctx", "64"],
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, env=dict(os.environ, HOS_MODEL=folder))
    out = p.stdout.decode()
    assert p.returncode == 0, p.stderr.decode()
    assert "prefill    : 30 tok" in out and "decode     : " in out
