"""GPU, end to end: the stage drivers on seeded synthetic layers.

Two sets of executables run the same files: bin/zkllm-driver (this repository's
driver source) and bin/ref-drivers/* (the reference's six driver sources compiled
UNMODIFIED against host/ and linked with the two libraries - the drop-in check;
present when the build ran where the reference sources are).  Every stage proves
what it computes and exits non-zero if a verifier equation fails.  Integer outputs
are checked against exact numpy int64 arithmetic.
"""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "zkllm-ccs2024_b200" / "bin"
SETS = [("own", BIN)] + ([("reference-source", BIN / "ref-drivers")] if (BIN / "ref-drivers" / "ffn").exists() else [])


def run(bindir: Path, stage: str, args, cwd: Path, seed: int = 1234) -> str:
    env = dict(os.environ, ZKLLM_CHALLENGE_SEED=str(seed))
    res = subprocess.run([str(bindir / stage), *[str(a) for a in args]], cwd=cwd, env=env, capture_output=True, text=True, timeout=1200)
    assert res.returncode == 0, f"{stage} failed:\n{res.stdout[-2000:]}\n{res.stderr[-2000:]}"
    return res.stdout


def rescale(x: np.ndarray, sf: int) -> np.ndarray:
    """rescaling.cu:8-21 on int64: remainder centred in [-sf/2, sf/2)"""
    h = sf >> 1
    rem = np.mod(x + h, sf) - h
    return (x - rem) // sf


def save_int(path: Path, a: np.ndarray):
    a.astype(np.int32).tofile(path)


def make_param(bindir, workdir: Path, prefix: str, name: str, w_int: np.ndarray, in_dim: int, out_dim: int, gen_size: int):
    pp = workdir / f"{name}-pp.bin"
    if not pp.exists():
        run(bindir, "ppgen", [gen_size, pp], workdir)
    save_int(workdir / f"{prefix}-{name}-int.bin", w_int)
    out = run(bindir, "commit-param", [pp, workdir / f"{prefix}-{name}-int.bin", workdir / f"{prefix}-{name}-commitment.bin", in_dim, out_dim], workdir)
    assert "Commitment size:" in out


@pytest.mark.parametrize("label,bindir", SETS)
def test_skip_connection_and_rmsnorm(label, bindir, tmp_path):
    rng = np.random.Generator(np.random.PCG64(11))
    seq, embed = 256, 256
    x = np.rint(rng.standard_normal((seq, embed)) * 65536).astype(np.int64)
    y = np.rint(rng.standard_normal((seq, embed)) * 65536).astype(np.int64)
    save_int(tmp_path / "x.bin", x)
    save_int(tmp_path / "y.bin", y)
    run(bindir, "skip-connection", ["x.bin", "y.bin", "z.bin"], tmp_path)
    assert np.array_equal(np.fromfile(tmp_path / "z.bin", dtype=np.int32).astype(np.int64), (x + y).reshape(-1))

    w = np.rint((1.0 + 0.1 * rng.standard_normal(embed)) * 65536).astype(np.int64)
    make_param(bindir, tmp_path, "layer-0", "input_layernorm.weight", w, 1, embed, embed)
    xf = x / 65536.0
    rms_inv = np.rint(65536.0 / np.sqrt((xf ** 2).mean(axis=1) + 1e-5)).astype(np.int64)     # llama-rmsnorm.py:38-39
    save_int(tmp_path / "rms_inv_temp.bin", rms_inv)
    out = run(bindir, "rmsnorm", ["input", "x.bin", seq, embed, tmp_path, "layer-0", "out.bin"], tmp_path)
    assert out.count("Rescaling proof complete.") == 2 and "Opening complete" in out
    g = rescale(np.outer(rms_inv, w), 1 << 16)
    exp = rescale(g * x, 1 << 16)
    assert np.array_equal(np.fromfile(tmp_path / "out.bin", dtype=np.int32).astype(np.int64), exp.reshape(-1))


@pytest.mark.parametrize("label,bindir", SETS)
def test_ffn(label, bindir, tmp_path):
    rng = np.random.Generator(np.random.PCG64(12))
    seq, embed, hidden = 1024, 64, 4096            # seq * hidden = 2^22, the size of the SwiGLU table
    w = {nm: np.rint(rng.standard_normal(shape) * 0.02 * 65536).astype(np.int64)
         for nm, shape in (("up", (embed, hidden)), ("gate", (embed, hidden)), ("down", (hidden, embed)))}
    make_param(bindir, tmp_path, "layer-0", "mlp.up_proj.weight", w["up"], embed, hidden, hidden)
    make_param(bindir, tmp_path, "layer-0", "mlp.gate_proj.weight", w["gate"], embed, hidden, hidden)
    make_param(bindir, tmp_path, "layer-0", "mlp.down_proj.weight", w["down"], hidden, embed, embed)
    xs = np.arange(-(1 << 21), 1 << 21, dtype=np.float64) / 4096.0            # llama-ffn.py:16-19
    table = np.rint(xs / (1.0 + np.exp(-xs)) * 16).astype(np.int64)
    save_int(tmp_path / "swiglu-table.bin", table)
    x = np.rint(rng.standard_normal((seq, embed)) * 65536).astype(np.int64)
    save_int(tmp_path / "in.bin", x)
    out = run(bindir, "ffn", ["in.bin", seq, embed, hidden, tmp_path, "layer-0", "out.bin"], tmp_path)
    assert out.count("Rescaling proof complete.") == 4 and out.count("Opening complete") == 3 and "SwiGLU proof complete." in out
    up_ = rescale(x @ w["up"], 1 << 16)
    gate_ = rescale(x @ w["gate"], 1 << 20)
    assert gate_.min() >= -(1 << 21) and gate_.max() < (1 << 21)
    act = table[gate_ + (1 << 21)]
    down_in_ = rescale(act * up_, 1 << 16)
    exp = down_in_ @ w["down"]                       # the driver saves the value before the last rescaling
    assert np.array_equal(np.fromfile(tmp_path / "out.bin", dtype=np.int32).astype(np.int64), exp.reshape(-1))


def test_self_attention_both_driver_sets_agree(tmp_path):
    rng = np.random.Generator(np.random.PCG64(13))
    seq, embed = 1024, 1024                          # seq * seq = 2^20, the size of the softmax tables
    ws = {nm: np.rint(rng.standard_normal((embed, embed)) * 0.02 * 65536).astype(np.int64) for nm in "qkv"}
    x = np.rint(rng.standard_normal((seq, embed)) * 65536).astype(np.int64)
    results = {}
    for label, bindir in SETS:
        d = tmp_path / label
        d.mkdir()
        for nm in "qkv":
            make_param(bindir, d, "layer-0", f"self_attn.{nm}_proj.weight", ws[nm], embed, embed, embed)
        save_int(d / "in.bin", x)
        out = run(bindir, "self-attn", ["linear", "in.bin", seq, embed, d, "layer-0", "unused.bin"], d)
        assert "QKV linear proof successfully verified!" in out and out.count("Opening complete") == 3
        for nm in "qkv":
            got = np.fromfile(d / f"temp_{nm.upper()}.bin", dtype=np.int32).astype(np.int64)
            assert np.array_equal(got, rescale(x @ ws[nm], 1 << 16).reshape(-1))
        out = run(bindir, "self-attn", ["attn", "in.bin", seq, embed, d, "layer-0", "unused.bin"], d)
        assert "Self attention proof successfully verified!" in out
        results[label] = ((d / "temp_head_Y.bin").read_bytes(), (d / "temp_head_out.bin").read_bytes())
        y = np.frombuffer(results[label][0], dtype=np.int64).reshape(seq, seq)
        # softmax rows at output scale 2^40 (theta 2^18 * 2^22) sum to about one
        sums = y.sum(axis=1) / float(1 << 40)
        assert np.all(np.abs(sums - 1.0) < 0.05)
    if len(results) == 2:
        assert results["own"] == results["reference-source"]


def test_batch_mode_runs_stages_in_one_process(tmp_path):
    """`zkllm-driver batch -`: the same stage command lines, one per line, in one resident process; a line is answered
    by "[batch] <stage> <seconds> s" on stderr and gives the same files as separate processes; a bad line ends the batch."""
    rng = np.random.Generator(np.random.PCG64(12))
    seq, embed = 128, 256
    x = np.rint(rng.standard_normal((seq, embed)) * 65536).astype(np.int64)
    y = np.rint(rng.standard_normal((seq, embed)) * 65536).astype(np.int64)
    save_int(tmp_path / "x.bin", x)
    save_int(tmp_path / "y.bin", y)
    script = tmp_path / "stages.txt"
    script.write_text("# two stages\nskip-connection x.bin y.bin z.bin\n\nskip-connection z.bin y.bin w.bin\n")
    env = dict(os.environ, ZKLLM_CHALLENGE_SEED="1234")
    res = subprocess.run([str(BIN / "zkllm-driver"), "batch", str(script)], cwd=tmp_path, env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stderr.count("[batch] skip-connection") == 2
    assert np.array_equal(np.fromfile(tmp_path / "w.bin", dtype=np.int32).astype(np.int64), (x + 2 * y).reshape(-1))
    # the output files come from a writer thread by default; written in place they are the same
    first = (tmp_path / "z.bin").read_bytes(), (tmp_path / "w.bin").read_bytes()
    res = subprocess.run([str(BIN / "zkllm-driver"), "batch", str(script)], cwd=tmp_path, env=dict(env, ZKLLM_DEFERRED_SAVES="0"),
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert ((tmp_path / "z.bin").read_bytes(), (tmp_path / "w.bin").read_bytes()) == first
    # from standard input, and an unknown stage fails loudly
    res = subprocess.run([str(BIN / "zkllm-driver"), "batch", "-"], cwd=tmp_path, env=env, capture_output=True, text=True,
                         input="skip-connection x.bin y.bin z2.bin\nno-such-stage a b\n", timeout=600)
    assert res.returncode != 0
    assert np.array_equal(np.fromfile(tmp_path / "z2.bin", dtype=np.int32), np.fromfile(tmp_path / "z.bin", dtype=np.int32))
