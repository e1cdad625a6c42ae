"""CPU check of bench.py's output contract on the arm that needs no GPU (--impl reference): exactly one JSON
line on stdout with the agreed keys.  The small 1024^3 workload keeps it to a few seconds."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg1",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOPS" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["n_gpus"] == 1 and d["steps"] == 1 and d["gpu_launches"] == 0
    assert d["config"]["workload"] == "cfg1"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_other_ranks_of_the_reference_arm_stay_silent():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--workload", "cfg1", "--steps", "1", "--warmup", "0"], capture_output=True, text=True,
                       timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_kernel_variant_names():
    """decxb200_last_kernel_variant() codes -> template names, as bench.py prints them in `roofline.kernel`."""
    sys.path.insert(0, ROOT)
    import bench
    assert bench.variant_name(0) is None
    assert bench.variant_name(22) == "gemm_tcgen05_kernel<0,2,2,0>"
    assert bench.variant_name(1022) == "gemm_tcgen05_kernel<0,2,2,2>"
    assert bench.variant_name(121) == "gemm_tcgen05_kernel<1,2,1,0>"
    assert bench.variant_name(5111) == "gemm_tcgen05_kernel<1,1,1,0,64>"
    assert bench.variant_name(26111) == "gemm_tcgen05_kernel<1,1,1,0,128> (implicit conv)"
    assert bench.variant_name(20111) == "gemm_tcgen05_kernel<1,1,1,0> (implicit conv)"
