"""The reference arm of bench.py: the unmodified reference code, the same counts and configuration as the main arm,
an end-to-end figure, and nothing of this library in its process."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

PROBE = r"""
import io, json, runpy, sys, contextlib
sys.argv = ["bench.py", "--impl", "reference", "--gpus", "2", "--bytes", str(8 << 20), "--steps", "4", "--warmup", "3"]
buf = io.StringIO()
with contextlib.redirect_stdout(buf):
    try:
        runpy.run_path("bench.py", run_name="__main__")
    except SystemExit:
        pass
maps = open("/proc/self/maps").read()
print(json.dumps({"line": buf.getvalue().strip().splitlines()[-1],
                  "package_imported": any(m.startswith("configurable_hierarchical") for m in sys.modules),
                  "torch_imported": "torch" in sys.modules, "libchb_mapped": "libchb" in maps}))
"""


def test_reference_arm_is_self_contained_and_matches_the_main_arms_shape():
    if not (ROOT / "baseline" / "_ref" / "ref_driver").exists() and not Path("/root/reference").exists():
        pytest.skip("the reference sources are not available here")
    r = subprocess.run([sys.executable, "-c", PROBE], cwd=ROOT, capture_output=True, text=True, timeout=600,
                       env={"PATH": "/usr/bin:/bin", "WORLD_SIZE": "2", "RANK": "0"})
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert not rec["package_imported"] and not rec["libchb_mapped"], rec
    d = json.loads(rec["line"])
    if "unavailable" in d:
        pytest.skip(d["unavailable"])
    assert d["impl"] == "reference" and d["steps"] == 4 and d["warmup"] == 3 and d["n_gpus"] == 2
    assert d["is_correct"] is True and d["value"] > 0
    # the same configuration record as the main arm prints
    sys.path.insert(0, str(ROOT))
    import bench
    assert d["config"] == bench.headline_config(2, 8 << 20) and d["metric"] == bench.METRIC
    # host buffer in, host buffer out: the timed call is the end-to-end figure, with nothing over PCIe
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == "GB/s" and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0
    assert e["steps"] == 4 and e["ms_per_step"] == d["ms_per_step"]
