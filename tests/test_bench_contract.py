"""The parts of bench.py's contract that need no GPU: the flags the driver passes, the default of one GPU and a
short run, and the line the reference arm prints when the reference installation is not there."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_flags_and_defaults():
    sys.path.insert(0, str(ROOT))
    try:
        import bench
    finally:
        sys.path.pop(0)
    old = sys.argv
    try:
        sys.argv = ["bench.py"]
        a = bench.parse()
        assert a.gpus == 1 and a.warmup >= 3 and a.steps >= 1 and a.impl == "ours"
        sys.argv = ["bench.py", "--impl", "reference", "--gpus", "8", "--steps", "7", "--warmup", "4"]
        a = bench.parse()
        assert (a.impl, a.gpus, a.steps, a.warmup) == ("reference", 8, 7, 4)
    finally:
        sys.argv = old


def test_reference_arm_says_unavailable_without_the_installation(tmp_path):
    """With the installation prefix pointed at an empty folder the arm prints its one JSON line and exits 0
    before anything touches a GPU."""
    code = (
        "import sys, pathlib; sys.path.insert(0, %r)\n"
        "from baseline import reference_arm\n"
        "reference_arm.PREFIX = pathlib.Path(%r)\n"
        "import bench\n"
        "sys.argv = ['bench.py', '--impl', 'reference']\n"
        "sys.exit(bench.main())\n" % (str(ROOT), str(tmp_path))
    )
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "missing" in line["unavailable"]
