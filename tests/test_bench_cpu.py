"""bench.py on a machine without a GPU: the reference arm says it is unavailable and exits 0, the
product arm refuses loudly (there is no CPU path to fall back to)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _no_gpu():
    try:
        import torch
        return not torch.cuda.is_available()
    except Exception:
        return True


@pytest.mark.skipif(not _no_gpu(), reason="meant for machines without a GPU")
def test_bench_without_gpu():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1"],
                       capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, p.stderr
    line = json.loads(p.stdout.strip().split("\n")[-1])
    assert line["impl"] == "reference" and "unavailable" in line
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1"],
                       capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode != 0
    assert "no CPU path" in p.stdout
