"""GPU: the reference project's own benchmark scripts, unmodified, against this library under the package name
`flashomni` (the drop-in proof). Each script is run as a child process from the reference's benchmark/ directory
with this repository on PYTHONPATH, and the checks it prints are read back: the attention script's
`scaled_dot_masked vs flashomni, all close: True` line (its `--check` mode, benchmark/test_flashomni_attention.py:297)
and the `True` that the GEMM-Q / GEMM-O scripts print from `torch.allclose` (test_flashomni_gemm_q.py:89,
test_flashomni_gemm_o.py:84). Skipped where no checkout of the reference is present (FLASHOMNI_REFERENCE_DIR)."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_dir():
    ref = os.environ.get("FLASHOMNI_REFERENCE_DIR", "")
    d = os.path.join(ref, "benchmark") if ref else ""
    if not d or not os.path.isfile(os.path.join(d, "test_flashomni_gemm_q.py")):
        pytest.skip("no checkout of the reference (set FLASHOMNI_REFERENCE_DIR)")
    return d


def _run(script, *args):
    d = _bench_dir()
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, script, *args], cwd=d, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


def test_reference_gemm_q_script(cuda_device):
    out = _run("test_flashomni_gemm_q.py")
    lines = [ln.strip() for ln in out.splitlines()]
    assert "True" in lines and "False" not in lines, out[-1500:]


def test_reference_gemm_o_script(cuda_device):
    out = _run("test_flashomni_gemm_o.py")
    lines = [ln.strip() for ln in out.splitlines()]
    assert "True" in lines and "False" not in lines, out[-1500:]


def test_reference_attention_script_check_mode(cuda_device):
    pytest.importorskip("flashinfer")
    pytest.importorskip("flash_attn")
    out = _run("test_flashomni_attention.py", "--check", "--warmup", "1", "--iters", "2")
    hit = [ln for ln in out.splitlines() if "scaled_dot_masked vs flashomni" in ln]
    assert hit and "all close: True" in hit[0], out[-2500:]
