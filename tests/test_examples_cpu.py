"""The FSDP2 example script runs end to end on CPU ranks (gloo), with and without on-demand communication."""
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("env", [{"ODC": "1"}, {"ODC": "1", "HPZ": "1"}, {"ODC": "0"}])
def test_fsdp2_example_cpu(env, tmp_path):
    e = dict(os.environ, **env, ODC_SYMMETRIC_SIZE="256M")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + len(env) + (1 if env.get("ODC") == "0" else 0)),
           os.path.join(REPO, "examples/FSDP2/example.py"), "--cpu", "--checkpoint-dir", str(tmp_path)]
    r = subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "step 9 loss" in r.stdout
