"""bench.py without a GPU: the reference arm (the CPU path timed on the host cores) prints one JSON line with the
keys the contract names, and the workload table points at network builders that exist."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "resnet50_train_images_per_s" and d["unit"] == "img/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "resnet50_imagenet_train"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_workload_table_names_existing_builders():
    sys.path.insert(0, ROOT)
    import bench
    from pydtnn_b200 import nets
    assert set(bench.WORKLOADS) == {"resnet50", "vgg16bn", "alexnet"}
    for name, wl in bench.WORKLOADS.items():
        assert callable(getattr(nets, wl["build"])), name
        assert wl["layout"] in ("NHWC", "NCHW") and wl["batch"] > 0
    assert bench.WORKLOADS["resnet50"]["metric"] == bench.METRIC


def test_sweep_points_cover_the_shape_sweep():
    import bench
    pts = bench.sweep_points()
    assert len(pts) == 640 and len(set(pts)) == 640
    for n, h, w, ci, co, k, s, p in pts:
        assert n == 32 and h == w and h in (7, 14, 28, 56, 112) and k in (1, 3, 5, 7) and s in (1, 2)
        assert ci in (64, 128, 256, 512) and co in (64, 128, 256, 512) and p == (k - 1) // 2
        assert (h + 2 * p - k) // s + 1 == (h + s - 1) // s          # 'same' padding: ceil(h / stride) outputs
