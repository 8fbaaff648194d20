"""The scripts under ``examples/`` run end to end on CPU (small sizes; the multi-rank ones as two gloo processes
started by ``torch.distributed.run``) and do what their docstrings say."""
import importlib.util
import os
import socket
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torchrun(script, *args, nproc=2):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "examples", script), *args]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout


def test_llama_from_hf_example():
    pytest.importorskip("transformers")
    err, losses, back = _load("llama_from_hf").main(["--steps", "3", "--seq", "32", "--new-tokens", "4"])
    assert err < 1e-4 and back < 1e-4 and losses[-1] < losses[0]


@pytest.mark.parametrize("family,paged", [("gemma", 1), ("gpt", 0), ("mixtral", 0)])
def test_generation_example(family, paged):
    out = _load("generation").main(["--family", family, "--paged", str(paged), "--batch", "3", "--prompt", "6",
                                    "--new-tokens", "5", "--temperature", "0.8", "--top-k", "20"])
    assert out.shape == (3, 11)


def test_seq2seq_example_learns():
    losses = _load("seq2seq_t5").main(["--steps", "60", "--batch", "16", "--length", "6", "--vocab", "16"])
    assert sum(losses[-5:]) / 5 < 0.8 * losses[0]


def test_quantized_model_init_example():
    losses, same = _load("quantized_model_init").main(["--recipe", "current", "--steps", "6", "--hidden", "128"])
    assert same and losses[-1] < losses[0]


def test_moe_example_single_process():
    losses = _load("moe_expert_parallel").main(["--steps", "4", "--seq", "32"])
    assert losses[-1] < losses[0]


def test_moe_example_expert_parallel():
    out = _torchrun("moe_expert_parallel.py", "--steps", "3", "--seq", "32")
    assert "2 rank(s), 2 of 4 experts each" in out


@pytest.mark.parametrize("init", ["none", "mxfp8"])
def test_fsdp_example(init):
    pytest.importorskip("torch.distributed.fsdp")
    out = _torchrun("fsdp.py", "--quantized-init", init, "--steps", "4", "--hidden", "256", "--seq", "64")
    assert ("MXFP8Tensor" if init == "mxfp8" else "Tensor") in out
    first, last = (float(x) for x in out.strip().splitlines()[-1].split("loss ")[1].split(" -> "))
    assert last < first
