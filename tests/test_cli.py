"""The `skywalker` command-line driver: reference flag surface and stdout rows."""
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "skywalker_b200", "skywalker")


def _run(*args, check=True):
    p = subprocess.run([CLI] + list(args), capture_output=True, text=True, timeout=600)
    if check:
        assert p.returncode == 0, p.stderr
    return p


def test_cli_rejects_unknown_flags_and_missing_input():
    assert os.path.exists(CLI), "build the CLI with python -m skywalker_b200.build"
    p = _run("--bogus", check=False)
    assert p.returncode == 1 and "unknown command line flag" in p.stderr
    p = _run("--deepwalk", check=False)
    assert p.returncode == 1 and "--input" in p.stderr
    p = _run("--n", check=False)
    assert p.returncode == 1 and "missing its argument" in p.stderr


def _paths_from_printresult(out):
    rows = []
    for m in re.finditer(r"(\d+)rd path len (\d+) \n([^\n]*)\n", out):
        rows.append((int(m.group(2)), [int(x) for x in m.group(3).split()]))
    return rows


@pytest.fixture(scope="module")
def gr_file(tmp_path_factory, rmat12):
    from skywalker_b200.gr import write_gr
    p = str(tmp_path_factory.mktemp("gr") / "rmat12.w.gr")
    write_gr(p, rmat12.xadj, rmat12.adjncy, np.floor(rmat12.adjwgt).astype(np.uint32))
    return p


@pytest.mark.gpu
def test_cli_offline_deepwalk_matches_oracle(oracle, rmat12, gr_file):
    g = rmat12
    w = np.floor(g.adjwgt).astype(np.float32)
    out = _run("--deepwalk", "--d", "10", "--bias=1", "--ol=0", "-n", "64", "--input", gr_file, "--printresult").stdout
    lines = out.strip().split("\n")
    assert lines[0] == "rmat12.w.gr"                          # graph name first (include/graph.cuh:186-192)
    nums = re.findall(r"^([\d.]+)\t$", out, re.M)
    assert len(nums) == 3                                     # table ms, time ms, MSEPS (src/main.cu:408-419)
    table = oracle.alias_build(g.xadj, w)
    starts = np.arange(64, dtype=np.uint32)                   # walker g starts at vertex g (sampler.cuh:494-503)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, w, table, starts, 11, seed=42)
    shown = _paths_from_printresult(out)
    assert len(shown) == 3
    for j, (length, row) in enumerate(shown):
        assert length == olens[j]
        assert row == list(opaths[j, :length + 1])
    # online mode walks the same paths; --csv prints one line
    out2 = _run("--deepwalk", "--d", "10", "--bias=1", "--ol=1", "-n", "64", "--input", gr_file, "--printresult").stdout
    assert _paths_from_printresult(out2) == shown
    csv = _run("--deepwalk", "--d", "10", "--bias=1", "--ol=0", "-n", "64", "--input", gr_file, "--csv").stdout
    assert re.fullmatch(r"rmat12\.w\.gr,[\d.]+,\t[\d.]+,\t[\d.]+,\n", csv)


@pytest.mark.gpu
def test_cli_presets_and_modes(gr_file):
    # --ppr sets tp = 0.15 and d = 100; --sage samples 25,10; --node2vec runs the rejection walk
    for args in (["--ppr"], ["--sage"], ["--sage", "--ol=1"], ["--node2vec", "--d", "8"], ["--ppr", "--records"],
                 ["--k", "3", "--d", "2"]):
        out = _run(*args, "--bias=1", "-n", "256", "--input", gr_file).stdout
        mseps = float(out.strip().split("\n")[-1])
        assert mseps > 0
    p = _run("--deepwalk", "--input", gr_file + ".missing", check=False)
    assert p.returncode == 2 and "cannot open" in p.stderr


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.gpu
def test_cli_two_gpus_same_total_as_one(gr_file):
    """--ngpu 2 shards the walkers (interleaved ids) and gathers the lengths on GPU 0 over NCCL; the
    walks, hence the sampled-edge total, do not depend on the GPU count."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    args = ["--ppr", "--bias=1", "--ol=0", "-n", "20000", "--input", gr_file, "-v"]
    one = _run(*args, "--ngpu", "1").stdout
    two = _run(*args, "--ngpu", "2").stdout
    e1 = int(re.search(r"sampled_edges (\d+)", one).group(1))
    e2 = int(re.search(r"sampled_edges (\d+)", two).group(1))
    m = re.search(r"gathered (\d+) walk lengths on GPU 0 over NCCL, sum (\d+)", two)
    assert m and int(m.group(1)) == 20000
    assert e1 == e2 == int(m.group(2)) and e1 > 0


@pytest.mark.gpu
def test_cli_start_vertex_conventions(oracle, rmat12, gr_file):
    """--itl (default) and --itl=0 give walker g the start vertex g either way on one GPU; --full walks
    from every vertex; --randstart draws the starts from the seeded stream."""
    g = rmat12
    w = np.floor(g.adjwgt).astype(np.float32)
    table = oracle.alias_build(g.xadj, w)
    base = ["--deepwalk", "--d", "6", "--bias=1", "--ol=0", "--input", gr_file, "--printresult"]
    a = _paths_from_printresult(_run(*base, "-n", "32").stdout)
    b = _paths_from_printresult(_run(*base, "-n", "32", "--itl=0").stdout)
    assert a == b and [r[1][0] for r in a] == [0, 1, 2]
    full = _run(*base, "--full", "-v").stdout
    _, olens = oracle.walk(g.xadj, g.adjncy, w, table, np.arange(g.V, dtype=np.uint32), 7, seed=42)
    assert int(re.search(r"sampled_edges (\d+)", full).group(1)) == int(olens.sum())
    r = _paths_from_printresult(_run(*base, "-n", "32", "--randstart", "--seed", "9").stdout)
    starts = oracle.gen_starts(32, g.V, 9)
    assert [row[1][0] for row in r] == [int(x) for x in starts[:3]]
    op, ol = oracle.walk(g.xadj, g.adjncy, w, table, starts, 7, seed=9)
    assert [row[1] for row in r] == [list(op[j, :ol[j] + 1]) for j in range(3)]


@pytest.mark.gpu
def test_cli_unbiased_modes(oracle, rmat12, gr_file):
    # --bias=0: uniform neighbour choice, no table row (src/main.cu:408-419 prints it only with --bias)
    g = rmat12
    out = _run("--deepwalk", "--d", "10", "--bias=0", "-n", "64", "--input", gr_file, "--printresult").stdout
    assert len(re.findall(r"^([\d.]+)\t$", out, re.M)) == 2
    starts = np.arange(64, dtype=np.uint32)
    opaths, olens = oracle.walk(g.xadj, g.adjncy, None, None, starts, 11, seed=42, unbiased=True)
    shown = _paths_from_printresult(out)
    assert len(shown) == 3
    for j, (length, row) in enumerate(shown):
        assert length == olens[j] and row == list(opaths[j, :length + 1])
    for args in (["--ppr"], ["--sage"], ["--node2vec", "--d", "8"]):
        out = _run(*args, "--bias=0", "-n", "256", "--input", gr_file).stdout
        assert float(out.strip().split("\n")[-1]) > 0
