"""World-size-2 gloo run on CPU of the host-side logic of the N > 1 path."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_host_logic_over_gloo(tmp_path, oracle):
    out = tmp_path / "gloo.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "mp_worker.py"), "gloo", str(out)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    got = json.loads(out.read_text())
    assert got["ok"] and got["world"] == 2
    # the scale moved in all three ways: x1.02, x0.5 (inf on steps 5, 10), x0.9 (step 7)
    s = got["scales"]
    assert s[0] == 256.0 * 1.02 or abs(s[0] - 261.12) < 1e-3
    assert s[4] < s[3] * 0.6 and s[6] < s[5] and s[6] > s[5] * 0.85
