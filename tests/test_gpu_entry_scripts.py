"""The reference's own entry scripts, unchanged, on this backend: `python -m lingbot_map_b200.run <script> ...`
(lingbot_map_b200/run.py rebinds the global block, the cache manager, the frame attention and the camera-head
attention, then runs the script as __main__).

* demo.py (random-init model, generated PNG frames, streaming mode with keyframe interval 2): model build, the
  aggregator cast to bf16 under autocast (demo.py:458-460,545-552), inference_streaming and post-processing run to
  the end (the viewer package is not installed, demo.py:598-600 prints the prediction keys instead).
* gct_profile.py --dtype both: its bf16 run (torch.compile of the hot modules, streaming through this backend) and
  its fp32 run, which sets kv_cache_force_fp32 (gct_profile.py:293-296): the reference's own fp32 gather + SDPA
  manager is handed back for that mode (select._manager_selector) and the script must finish and report finite
  frame rates for both.

Needs the reference package under baseline/_ref (skipped otherwise)."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "demo.py")),
                                 reason="reference package and scripts not installed under baseline/_ref")]


def _run(script, *args, timeout=900):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, REF, env.get("PYTHONPATH", "")])
    return subprocess.run([sys.executable, "-m", "lingbot_map_b200.run", os.path.join(REF, script), *args],
                          env=env, capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def test_demo_script_runs_on_this_backend(tmp_path):
    from PIL import Image
    rs = np.random.RandomState(0)
    for i in range(10):
        Image.fromarray(rs.randint(0, 255, (378, 518, 3), dtype=np.uint8)).save(tmp_path / f"frame_{i:03d}.png")
    r = _run("demo.py", "--model_path", "", "--image_folder", str(tmp_path), "--num_scale_frames", "4",
             "--keyframe_interval", "2", "--camera_num_iterations", "2")
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    assert "Inference done" in r.stdout and "Casting aggregator to torch.bfloat16" in r.stdout
    assert "Predictions contain keys" in r.stdout or "3D viewer" in r.stdout


def test_profile_script_runs_bf16_and_the_fp32_comparison_mode():
    out = "/tmp/profile_results_126x182_20f_both.json"
    if os.path.exists(out):
        os.remove(out)
    r = _run("gct_profile.py", "--backend", "flashinfer", "--dtype", "both", "--img_h", "126", "--img_w", "182",
             "--num_frames", "20", "--camera_num_iterations", "1", timeout=1500)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    with open(out) as f:
        res = json.load(f)
    assert set(res) == {"flashinfer_bf16", "flashinfer_fp32"}
    for key, d in res.items():
        vals = [v for v in d.values() if isinstance(v, (int, float))]
        assert vals and all(math.isfinite(v) for v in vals), (key, d)
